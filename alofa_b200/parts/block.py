"""How one layer arranges its parts.

``sandwich_residual``: a norm before and a norm after each sublayer,
``h += norm_b(mixer(norm_a(h))); h += norm_d(feed_forward(norm_c(h)))``; the
feed-forward may be absent.  ``embedding_mix_in``: no sublayers at all, ``h =
W [h; e]`` with ``e`` the embedding output of the step's tokens.

``parallel_residual``: one norm whose output both sublayers read,
``x = norm(h); h += mixer(x) + feed_forward(x)`` (the feed-forward may be
absent).  ``embedding_add``: no sublayers, ``h += e``.

``hyper_residual``: several copies of the stream side by side; a sublayer reads
a weighted sum of them and its output is written back into all of them while
they are mixed among themselves (see :class:`HyperResidual`).

``postnorm_residual``: a norm on each sublayer's output only, ``h +=
norm_a(mixer(h)); h += norm_b(feed_forward(h))``; the sublayers read the
stream itself (the feed-forward may be absent).

``prenorm_residual``: ``h += mixer(norm_a(h)); h += feed_forward(norm_b(h))``
(src/alofa/model/arch/qwen.mojo:1367-1372, 1418-1510).  The residual stream
``h`` is fp32; the parts add into it."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..errors import AlofaError
from .base import Part, TensorSpec, as_float32_vector, build_part, register_part
from .linear import STORE, Linear


class PrenormResidual(Part):
    family = "block"

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.mixer = build_part("mixer", self.param("mixer"), rt)
        self.feed_forward = build_part("feed_forward", self.param("feed_forward"), rt)
        self.mixer_norm = build_part("norm", self.param("mixer_norm"), rt)
        self.feed_forward_norm = build_part("norm", self.param("feed_forward_norm"), rt)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def tensors(self):
        out = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, state):
        for part in self.parts():
            part.load(state)

    @property
    def graph_safe(self):
        return all(part.graph_safe for part in self.parts())

    def cache_spec(self):
        return self.mixer.cache_spec()

    def scratch_row_bytes(self) -> int:
        return sum(getattr(part, "scratch_row_bytes", lambda: 0)() for part in self.parts())

    absorbs_pending = True  # its norms add partial sums owed to h; other readers get them flushed first

    def _norm(self, norm, ctx, h, reader):
        if not getattr(norm, "absorbs_pending", False):
            ctx.flush_pending()
            return norm.forward(ctx, h)
        # a reader that says so may get rows still to be made (the norm folded into its own product)
        if getattr(reader, "takes_normed_rows", False) and getattr(norm, "gives_normed_rows", False):
            return norm.forward(ctx, h, lazy=True)
        return norm.forward(ctx, h)

    def forward(self, ctx, h, cache, writes=True):
        x = self._norm(self.mixer_norm, ctx, h, self.mixer)
        self.mixer.forward(ctx, x, h, cache, writes)
        x = self._norm(self.feed_forward_norm, ctx, h, self.feed_forward)
        self.feed_forward.forward(ctx, x, h)


class SandwichResidual(Part):
    """Norms on both sides of each sublayer.  The sublayer's output goes to an
    fp32 buffer of its own (parts that say ``stores_output`` write it, any
    other part adds into a zeroed one); one kernel then normalises it, adds it
    to the stream and, for the mixer, also yields the normed input of the
    feed-forward."""

    family = "block"

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.mixer = build_part("mixer", self.param("mixer"), rt)
        self.mixer_norm = build_part("norm", self.param("mixer_norm"), rt)
        self.mixer_post = build_part("norm", self.param("mixer_post_norm"), rt)
        ff = self.params.get("feed_forward")
        self.feed_forward = build_part("feed_forward", ff, rt) if ff is not None else None
        self.feed_forward_norm = build_part("norm", self.param("feed_forward_norm"), rt) if ff is not None else None
        self.feed_forward_post = build_part("norm", self.param("feed_forward_post_norm"), rt) if ff is not None else None

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.mixer_post, self.feed_forward_norm, self.feed_forward, self.feed_forward_post) if p is not None)

    def tensors(self):
        out = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, state):
        for part in self.parts():
            part.load(state)

    @property
    def graph_safe(self):
        return all(part.graph_safe for part in self.parts())

    def cache_spec(self):
        return self.mixer.cache_spec()

    def scratch_row_bytes(self) -> int:
        return 12 * self.mixer_norm.size + sum(getattr(part, "scratch_row_bytes", lambda: 0)() for part in self.parts())

    def _sublayer(self, ctx, part, x, h, *args):
        """The part's output for the rows ``x``, fp32, in a buffer of its own."""
        y = ctx.buf(tuple(h.shape), h.dtype)
        if getattr(part, "stores_output", False):
            part.forward(ctx, x, y, *args, store=True)
        else:
            y.zero_()
            part.forward(ctx, x, y, *args)
            ctx.flush_pending()
        return y

    def forward(self, ctx, h, cache, writes=True):
        x = self.mixer_norm.forward(ctx, h)
        y = self._sublayer(ctx, self.mixer, x, h, cache, writes)
        if self.feed_forward is None:
            ops.sandwich_norm(h, y, self.mixer_post.weight, self.mixer_post.eps)
            return
        x = ctx.buf(tuple(h.shape), self.rt.dtype)
        ops.sandwich_norm(h, y, self.mixer_post.weight, self.mixer_post.eps, x, self.feed_forward_norm.weight, self.feed_forward_norm.eps)
        y = self._sublayer(ctx, self.feed_forward, x, h)
        ops.sandwich_norm(h, y, self.feed_forward_post.weight, self.feed_forward_post.eps)


class PostnormResidual(Part):
    """A norm on the output of each sublayer, none on its input: the sublayer
    reads the stream's rows themselves, rounded to the compute dtype.  The
    sublayer's output goes to an fp32 buffer of its own; one kernel normalises
    it, adds it to the stream and, for the mixer, also yields the rows the
    feed-forward reads."""

    family = "block"

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.mixer = build_part("mixer", self.param("mixer"), rt)
        self.mixer_post = build_part("norm", self.param("mixer_post_norm"), rt)
        ff = self.params.get("feed_forward")
        self.feed_forward = build_part("feed_forward", ff, rt) if ff is not None else None
        self.feed_forward_post = build_part("norm", self.param("feed_forward_post_norm"), rt) if ff is not None else None
        for part in (self.mixer, self.feed_forward):
            if part is not None and not getattr(part, "stores_output", False):
                raise AlofaError("unsupported", "a sublayer whose output is normed must be able to store it", f"kind={part.spec.kind}")

    def parts(self):
        return tuple(p for p in (self.mixer, self.mixer_post, self.feed_forward, self.feed_forward_post) if p is not None)

    def tensors(self):
        out = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, state):
        for part in self.parts():
            part.load(state)

    @property
    def graph_safe(self):
        return all(part.graph_safe for part in self.parts())

    def cache_spec(self):
        return self.mixer.cache_spec()

    def scratch_row_bytes(self) -> int:
        return 12 * self.mixer_post.size + sum(getattr(part, "scratch_row_bytes", lambda: 0)() for part in self.parts())

    @staticmethod
    def _output(ctx, part, h, x, *args):
        """The sublayer's output for the rows ``x``: an fp32 buffer, or the split sums its last product left for the norm's kernel to add."""
        y = ctx.buf(tuple(h.shape), torch.float32)
        if getattr(part, "defers_output", False) and x.shape[0] > 64:  # in steps of a few tokens the kernel that settles the sums first measured faster
            owed = part.forward(ctx, x, y, *args, store=True, defer=True)
            return y if owed is None else owed
        part.forward(ctx, x, y, *args, store=True)
        return y

    def forward(self, ctx, h, cache, writes=True):
        ctx.flush_pending()
        wide = self.rt.dtype == torch.float32
        x = h  # the 32-bit path reads the stream in place: a sublayer is done with it before the norm's kernel adds to it
        if not wide:
            left, ctx.stream_rows = ctx.stream_rows, None
            if left is not None and left[0] is h and left[2] == ctx.layer_no - 1:
                x = left[1]  # the layer before this one left the rows with its last norm
            else:
                x = ctx.buf(tuple(h.shape), self.rt.dtype)
                ops.cast_rows(x, h)
        y = self._output(ctx, self.mixer, h, x, cache, writes)
        if self.feed_forward is not None:
            x = None if wide else ctx.buf(tuple(h.shape), self.rt.dtype)
            ops.sandwich_norm(h, y, self.mixer_post.weight, self.mixer_post.eps, x)
            y = self._output(ctx, self.feed_forward, h, h if wide else x)
        last = self.feed_forward_post if self.feed_forward is not None else self.mixer_post
        # the layer's last norm also leaves the rows that the next layer's mixer reads (a scratch buffer of a layer lives until the layer after next begins)
        x = None if wide else ctx.buf(tuple(h.shape), self.rt.dtype)
        ops.sandwich_norm(h, y, last.weight, last.eps, x)
        if x is not None:
            ctx.stream_rows = (h, x, ctx.layer_no)


class EmbeddingMixIn(Part):
    """``h = W [h; e]``: the stream and the embedding output ``e`` of the same
    tokens, side by side, through one matrix [hidden, 2 * hidden] (the stream's
    columns first).  It keeps no cache; the model keeps ``e`` for the step."""

    family = "block"
    graph_safe = True
    needs_embedding_output = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(self.param("hidden_size"))
        self.name = self.prefix + str(self.params.get("weight_name", "weight"))
        self.linear = None

    def tensors(self):
        return {self.name: TensorSpec((self.hidden, 2 * self.hidden))}

    def load(self, state):
        self.linear = Linear(state[self.name], None, STORE)

    def cache_spec(self):
        return None

    def scratch_row_bytes(self) -> int:
        return 8 * self.hidden

    def forward(self, ctx, h, cache, writes=True):
        both = ctx.buf((h.shape[0], 2 * self.hidden), self.rt.dtype)
        ops.concat_rows(both, h, ctx.embedding_output)
        self.linear(h, both, buf=ctx.buf)


class ParallelResidual(Part):
    """One norm, and the mixer and the feed-forward side by side on its
    output; each adds what it makes into the fp32 stream."""

    family = "block"
    absorbs_pending = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.norm = build_part("norm", self.param("norm"), rt)
        self.mixer = build_part("mixer", self.param("mixer"), rt)
        ff = self.params.get("feed_forward")
        self.feed_forward = build_part("feed_forward", ff, rt) if ff is not None else None

    def parts(self):
        return tuple(p for p in (self.norm, self.mixer, self.feed_forward) if p is not None)

    def tensors(self):
        out = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, state):
        for part in self.parts():
            part.load(state)

    @property
    def graph_safe(self):
        return all(part.graph_safe for part in self.parts())

    def cache_spec(self):
        return self.mixer.cache_spec()

    def scratch_row_bytes(self) -> int:
        return sum(getattr(part, "scratch_row_bytes", lambda: 0)() for part in self.parts())

    def forward(self, ctx, h, cache, writes=True):
        if not getattr(self.norm, "absorbs_pending", False):
            ctx.flush_pending()
        x = self.norm.forward(ctx, h)
        # the feed-forward first: it adds into h itself, while the mixer's last product may leave sums for the next reader to add
        if self.feed_forward is not None:
            ctx.flush_pending()
            self.feed_forward.forward(ctx, x, h)
        self.mixer.forward(ctx, x, h, cache, writes)


class EmbeddingAdd(Part):
    """``h += e`` with ``e`` the embedding output of the step's tokens: what a
    stretch of layers that runs several times gets before each further pass."""

    family = "block"
    graph_safe = True
    needs_embedding_output = True

    def cache_spec(self):
        return None

    def forward(self, ctx, h, cache, writes=True):
        ctx.flush_pending()
        ops.add_rows(h, ctx.embedding_output)


class HyperResidual(Part):
    """Pre-norm sublayers over ``streams`` copies x_1 .. x_S of the residual
    stream (all equal to the embedding output at the start; the model's output
    is their sum).  Sublayer q (1: the mixer, 2: the feed-forward, which may be
    absent) reads ``u = sum_s in[s] x_s``, computes ``y = f(norm(u))``, and
    then every stream moves at once from the old ones: ``x_t <- sum_s mix[s,
    t] x_s + out[t] y``.  Tensors ``<prefix>hc<q>.in`` [S], ``.out`` [S],
    ``.mix`` [S, S] (from, to).  With ``connections`` False there are no such
    tensors and one stream: the plain ``x += f(norm(x))``.

    The streams live in ``ctx.streams`` [S, T, W] fp32 (the model makes them:
    ``stream_copies`` says how many).  A sublayer's write is left owed
    (``ctx.streams_owed``) and done by the kernel that reads the streams next:
    the next sublayer's read and norm, or the sum at the model's end."""

    family = "block"

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.width = int(self.param("hidden_size"))
        self.connections = bool(self.params.get("connections", True))
        self.stream_copies = int(self.param("streams")) if self.connections else 1
        if not 1 <= self.stream_copies <= ops.HYPER_MAX_STREAMS:
            raise AlofaError("unsupported", "the number of residual streams must lie in [1, 8]", f"streams={self.stream_copies}")
        self.mixer = build_part("mixer", self.param("mixer"), rt)
        self.mixer_norm = build_part("norm", self.param("mixer_norm"), rt)
        ff = self.params.get("feed_forward")
        self.feed_forward = build_part("feed_forward", ff, rt) if ff is not None else None
        self.feed_forward_norm = build_part("norm", self.param("feed_forward_norm"), rt) if ff is not None else None
        for part in (self.mixer, self.feed_forward):
            if part is not None and not getattr(part, "stores_output", False):
                raise AlofaError("unsupported", "a sublayer over several streams must be able to store its output", f"kind={part.spec.kind}")
        self.weights = {}

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None)

    def _numbers(self):
        return (1, 2) if self.feed_forward is not None else (1,)

    def tensors(self):
        out = {}
        for part in self.parts():
            out.update(part.tensors())
        if self.connections:
            S = self.stream_copies
            for q in self._numbers():
                pre = f"{self.prefix}hc{q}."
                out[pre + "in"] = TensorSpec((S,), "ones")
                out[pre + "out"] = TensorSpec((S,), "ones")
                out[pre + "mix"] = TensorSpec((S, S), "identity")
        return out

    def load(self, state):
        for part in self.parts():
            part.load(state)
        dev = self.mixer_norm.weight.device
        for q in self._numbers():
            if self.connections:
                pre = f"{self.prefix}hc{q}."
                self.weights[q] = tuple(as_float32_vector(state[pre + n]) for n in ("in", "out", "mix"))
            else:
                self.weights[q] = (torch.ones(1, device=dev), torch.ones(1, device=dev), torch.ones((1, 1), device=dev))

    @property
    def graph_safe(self):
        return all(part.graph_safe for part in self.parts())

    def cache_spec(self):
        return self.mixer.cache_spec()

    def scratch_row_bytes(self) -> int:
        return 12 * self.width + sum(getattr(part, "scratch_row_bytes", lambda: 0)() for part in self.parts())

    def _sublayer(self, ctx, q, norm, part, *args):
        w_in, w_out, w_mix = self.weights[q]
        hs = ctx.streams
        n = hs.shape[1]
        x = ctx.buf((n, self.width), self.rt.dtype)
        owed = ctx.streams_owed
        ctx.streams_owed = None
        # the write the sublayer before left owed, this one's read and its norm: one pass over the streams
        ops.hyper_connect(hs, owed[0] if owed else None, owed[2] if owed else None, owed[1] if owed else None, w_in, norm.weight, norm.eps, x_out=x)
        y = ctx.buf((n, self.width), torch.float32)
        part.forward(ctx, x, y, *args, store=True)
        ctx.streams_owed = (y, w_out, w_mix)

    def forward(self, ctx, h, cache, writes=True):
        if ctx.streams is None or ctx.streams.shape[0] != self.stream_copies:
            raise AlofaError("state", "the step has no residual streams of this block's number", f"streams={self.stream_copies}")
        self._sublayer(ctx, 1, self.mixer_norm, self.mixer, cache, writes)
        if self.feed_forward is not None:
            self._sublayer(ctx, 2, self.feed_forward_norm, self.feed_forward)


register_part("block", "hyper_residual", HyperResidual)
register_part("block", "prenorm_residual", PrenormResidual)
register_part("block", "postnorm_residual", PostnormResidual)
register_part("block", "parallel_residual", ParallelResidual)
register_part("block", "embedding_add", EmbeddingAdd)
register_part("block", "sandwich_residual", SandwichResidual)
register_part("block", "embedding_mix_in", EmbeddingMixIn)
