"""Built-in architectures.  Importing this package registers them."""
from . import darolix, dibulix, kotutar, qwen2  # noqa: F401
