"""Dense gated feed-forward: ``h += (act(x Wg^T) * (x Wu^T)) Wd^T`` with
``silu(z) = z / (1 + exp(-z))``, no biases
(src/alofa/model/arch/qwen.mojo:1481-1510; src/alofa/kernels/cpu/scalar.mojo:208-231).
The gate and up weights are stacked at load so that one product with a fused
epilogue writes ``silu(gate) * up`` directly."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..errors import AlofaError
from .base import Part, TensorSpec, as_float32_vector, register_part
from .linear import GATED, RESIDUAL, STORE, Linear, add_into_stream


class GatedMLP(Part):
    family = "feed_forward"
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(self.param("hidden_size"))
        self.inter = int(self.param("intermediate_size"))
        act = self.param("activation", "silu")
        if act != "silu":
            raise AlofaError("unsupported", "gated_mlp supports the silu activation only", f"activation={act}")
        self.gate_up = self.down = None

    def tensors(self):
        pre = self.prefix
        return {
            pre + "gate_proj.weight": TensorSpec((self.inter, self.hidden)),
            pre + "up_proj.weight": TensorSpec((self.inter, self.hidden)),
            pre + "down_proj.weight": TensorSpec((self.hidden, self.inter)),
        }

    def load(self, state):
        pre = self.prefix
        self.gate_up = Linear(torch.cat([state[pre + "gate_proj.weight"], state[pre + "up_proj.weight"]], dim=0), None, GATED)
        self.down = Linear(state[pre + "down_proj.weight"], None, RESIDUAL)

    def scratch_row_bytes(self) -> int:
        return 4 * self.inter + 2 * 4 * self.hidden  # the activation, and the down product's depth split in two

    takes_normed_rows = True  # ``x`` may be rows still to be made: the gate/up product folds the norm in

    def forward(self, ctx, x, h):
        act = ctx.buf((x.shape[0], self.inter), self.rt.dtype)
        self.gate_up(act, x, buf=ctx.buf)
        add_into_stream(ctx, self.down, h, act)


class DenseMLP(Part):
    """``Wdown act(Wup x (+ bup)) (+ bdown)`` with tensors ``<prefix>up``,
    ``<prefix>down`` (``.b`` for the biases); ``activation``: gelu_erf (the
    exact one), gelu_tanh, silu, relu.  The activation is taken on the fp32
    sums, before they are rounded to the compute dtype.  ``gated``: ``Wdown
    (silu(Wgate x) * (Wup x))`` with a third tensor ``<prefix>gate``, no
    biases (gate and up are one product whose epilogue multiplies them)."""

    family = "feed_forward"
    graph_safe = True
    stores_output = True  # forward(..., store=True) writes its output instead of adding it
    defers_output = True  # forward(..., store=True, defer=True) may hand back the down product's split sums instead of the finished output

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(self.param("hidden_size"))
        self.inter = int(self.param("intermediate_size"))
        self.act = str(self.param("activation", "gelu_erf"))
        self.bias = bool(self.params.get("bias", False))
        self.gated = bool(self.params.get("gated", False))
        if self.act not in ops.ACTIVATIONS:
            raise AlofaError("unsupported", "unknown activation", f"activation={self.act} known={sorted(ops.ACTIVATIONS)}")
        if self.gated and (self.act != "silu" or self.bias):
            raise AlofaError("unsupported", "a gated feed-forward takes the silu activation and no biases", f"activation={self.act} bias={self.bias}")
        self.up = self.down = None

    def tensors(self):
        pre = self.prefix
        t = {pre + "up": TensorSpec((self.inter, self.hidden)), pre + "down": TensorSpec((self.hidden, self.inter))}
        if self.gated:
            t[pre + "gate"] = TensorSpec((self.inter, self.hidden))
        if self.bias:
            t[pre + "up.b"] = TensorSpec((self.inter,))
            t[pre + "down.b"] = TensorSpec((self.hidden,))
        return t

    def load(self, state):
        pre = self.prefix
        if self.gated:  # gate rows first, then up rows
            self.up = Linear(torch.cat([state[pre + "gate"], state[pre + "up"]], dim=0), None, GATED)
        else:
            self.up = Linear(state[pre + "up"], as_float32_vector(state[pre + "up.b"]) if self.bias else None, STORE, act=self.act)
        self.down = Linear(state[pre + "down"], as_float32_vector(state[pre + "down.b"]) if self.bias else None, STORE)

    def scratch_row_bytes(self) -> int:
        return 4 * self.inter + 4 * self.hidden

    def forward(self, ctx, x, h, store=False, defer=False):
        n = x.shape[0]
        mid = ctx.buf((n, self.inter), self.rt.dtype)
        self.up(mid, x, buf=ctx.buf)  # bias and activation on the fp32 sums, in the product's epilogue
        if store:
            return self.down(h, mid, defer=defer, buf=ctx.buf)  # None, or the split sums a caller that asked for them adds up itself
        else:
            y = ctx.buf((n, self.hidden), torch.float32)
            self.down(y, mid, buf=ctx.buf)
            h.add_(y)


register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("feed_forward", "mlp", DenseMLP)
