"""Built-in architectures.  Importing this package registers them."""
from . import darolix, dibulix, kikerax, kotutar, qwen2  # noqa: F401
