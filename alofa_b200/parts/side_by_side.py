"""Several mixers side by side on the same input: each makes its output in a
buffer of its own, each output is RMS-normed over the model width with a plain
weight of its own (``<prefix><name>.out``), and their mean is added into the
residual stream (two branches: half the sum).  With ``combine`` "weighted"
there are no norms and no such weights: the result is ``sum_i scales[i] *
branch_i``, added into the stream or (``store``) written.  The branches keep
their own caches (pages, state slots), so this mixer's cache is the tuple of
theirs."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..errors import AlofaError
from .base import Part, TensorSpec, as_float32_vector, build_part, register_part


class SideBySide(Part):
    family = "mixer"

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(self.param("hidden_size"))
        self.eps = float(self.param("eps"))
        self.names = [str(n) for n in self.param("names")]
        self.branches = [build_part("mixer", s, rt) for s in self.param("branches")]
        if len(self.names) != len(self.branches) or not self.branches:
            raise AlofaError("invalid_argument", "side_by_side needs a name for every branch", f"names={self.names}")
        self.combine = str(self.params.get("combine", "normed_mean"))
        if self.combine not in ("normed_mean", "weighted"):
            raise AlofaError("invalid_argument", "side_by_side combines by 'normed_mean' or 'weighted'", f"combine={self.combine}")
        self.scales = [float(v) for v in self.params.get("scales", [])]
        if self.combine == "weighted" and len(self.scales) != len(self.branches):
            raise AlofaError("invalid_argument", "a weighted side_by_side needs a factor for every branch", f"scales={self.scales}")
        self.stores_output = self.combine == "weighted"  # forward(..., store=True) writes the result instead of adding it
        self.weights = None

    @property
    def graph_safe(self):
        return all(b.graph_safe for b in self.branches)

    def cache_spec(self):
        return tuple(b.cache_spec() for b in self.branches)

    def scratch_row_bytes(self) -> int:
        return 4 * self.hidden * len(self.branches) + sum(getattr(b, "scratch_row_bytes", lambda: 0)() for b in self.branches)

    def tensors(self):
        t = {}
        for name, b in zip(self.names, self.branches):
            t.update(b.tensors())
            if self.combine == "normed_mean":
                t[self.prefix + name + ".out"] = TensorSpec((self.hidden,), "ones")
        return t

    def load(self, state):
        for b in self.branches:
            b.load(state)
        if self.combine == "normed_mean":
            self.weights = [as_float32_vector(state[self.prefix + name + ".out"]) for name in self.names]

    def forward(self, ctx, x, h, cache, writes=True, store=False):
        outs = []
        for b, c in zip(self.branches, cache):
            y = ctx.buf(tuple(h.shape), torch.float32)
            if getattr(b, "stores_output", False):
                b.forward(ctx, x, y, c, writes, store=True)
            else:
                ctx.flush_pending()
                y.zero_()
                b.forward(ctx, x, y, c, writes)
                ctx.flush_pending()
            outs.append(y)
        ctx.flush_pending()  # the sums below go into h itself
        if self.combine == "weighted":
            for i in range(0, len(outs), 2):
                pair, sc = outs[i : i + 2], self.scales[i : i + 2]
                ops.scaled_sum(h, pair[0], sc[0], pair[1] if len(pair) > 1 else None, sc[1] if len(pair) > 1 else 0.0, accumulate=not store or i > 0)
            return
        scale = 1.0 / len(outs)
        for i in range(0, len(outs), 2):
            pair = outs[i : i + 2]
            ops.branch_norm_add(h, pair[0], self.weights[i], pair[1] if len(pair) > 1 else None, self.weights[i + 1] if len(pair) > 1 else None, self.eps, scale)


register_part("mixer", "side_by_side", SideBySide)
