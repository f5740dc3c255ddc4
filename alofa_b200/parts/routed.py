"""Routed feed-forward (mixture of experts).

``experts`` small feed-forwards ``Wdown act(Wup .)`` without biases, of which
every token uses ``top``.  Router logits ``z = x Wr^T`` and the scores made from
them are fp32 (``score``: "sigmoid" per expert, or "softmax" over the experts);
the ``top`` largest scores choose the experts and are their weights
(``renormalize``: divided by their sum).  The weight multiplies the expert's
input (``weight_on_input``) or its output.  Options: ``gated`` experts
``Wdown (act(Wgate .) * (Wup .))`` (tensors ``e<i>.gate``); ``correction``, a
stored vector added to the scores for the choice only (the weights stay the
scores); ``identity``: the last so many of the router's outputs are experts
without tensors whose output is their input; ``renorm_eps`` added to the sum
that ``renormalize`` divides by; ``groups`` / ``keep``: the experts form
``groups`` equal groups of neighbours, a group's score is the sum of its two
largest choice scores (score + correction), and only experts of the ``keep``
best groups can be chosen; ``route_scale``: a factor on the weights.  A shared
expert of the same form
(``shared_ff`` > 0) runs for every token and is added, times ``sigmoid(x
wsg^T)`` when ``shared_gate`` is set.

Nothing here asks the host: the tokens' choices stay on the device.  The
(token, choice) pairs are sorted by expert into a matrix in which every expert's
rows are padded to whole tiles, so one launch per projection multiplies each
tile by its expert's weights (in bfloat16 the tcgen05 product with the tokens on
the M side: a tile's expert is an offset into the stacked weight's rows); the
outputs are gathered back and added in the order of the choices."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..errors import AlofaError
from .base import Part, TensorSpec, register_part
from .feed_forward import DenseMLP
from .linear import STORE, Linear


class RoutedExperts(Part):
    family = "feed_forward"
    graph_safe = True
    stores_output = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.param
        self.hidden = int(p("hidden_size"))
        self.experts = int(p("experts"))
        self.top = int(p("top"))
        self.ff = int(p("expert_ff"))
        self.shared_ff = int(self.params.get("shared_ff") or 0)
        self.act = str(p("activation", "gelu_erf"))
        self.score = str(p("score", "sigmoid"))
        self.renormalize = bool(self.params.get("renormalize", False))
        self.weight_on_input = bool(self.params.get("weight_on_input", False))
        self.shared_gate = bool(self.params.get("shared_gate", False)) and self.shared_ff > 0
        self.gated = bool(self.params.get("gated", False))
        self.identity = int(self.params.get("identity") or 0)
        self.correction_name = self.prefix + "correction" if self.params.get("correction") else None
        self.renorm_eps = float(self.params.get("renorm_eps") or 0.0)
        self.groups = int(self.params.get("groups") or 1)
        self.keep = int(self.params.get("keep") or self.groups)
        self.route_scale = float(self.params.get("route_scale", 1.0))
        if self.groups > 1 and (self.identity or self.experts % self.groups or not 0 < self.keep <= self.groups or self.keep * (self.experts // self.groups) < self.top):
            raise AlofaError("invalid_argument", "groups must divide the experts, and the groups kept must hold at least top experts",
                             f"experts={self.experts} groups={self.groups} keep={self.keep} top={self.top}")
        self.routed = self.experts + self.identity  # outputs of the router
        if self.gated and self.act != "silu":
            raise AlofaError("unsupported", "gated experts take the silu activation only", f"activation={self.act}")
        if self.identity and self.weight_on_input:
            raise AlofaError("unsupported", "identity experts need the weight on the expert's output")
        if self.act not in ops.ACTIVATIONS or self.score not in ("sigmoid", "softmax"):
            raise AlofaError("unsupported", "unknown activation or score of a routed feed-forward", f"activation={self.act} score={self.score}")
        if not 0 < self.top <= min(self.experts + int(self.params.get("identity") or 0), 32) or self.experts <= 0:
            raise AlofaError("invalid_argument", "top must lie in [1, min(experts, 32)]", f"top={self.top} experts={self.experts}")
        self.shared = None
        if self.shared_ff:
            from ..config.spec import PartSpec

            self.shared = DenseMLP(PartSpec("mlp", {"hidden_size": self.hidden, "intermediate_size": self.shared_ff, "activation": self.act, "bias": False, "gated": self.gated},
                                            prefix=self.prefix + "shared."), rt)

    def tensors(self):
        pre = self.prefix
        t = {pre + "router": TensorSpec((self.routed, self.hidden))}
        if self.correction_name:
            t[self.correction_name] = TensorSpec((self.routed,))
        for e in range(self.experts):
            if self.gated:
                t[pre + f"e{e}.gate"] = TensorSpec((self.ff, self.hidden))
            t[pre + f"e{e}.up"] = TensorSpec((self.ff, self.hidden))
            t[pre + f"e{e}.down"] = TensorSpec((self.hidden, self.ff))
        if self.shared is not None:
            t.update(self.shared.tensors())
            if self.shared_gate:
                t[pre + "shared.sg"] = TensorSpec((1, self.hidden))
        return t

    def load(self, state):
        pre = self.prefix
        rows = [state[pre + "router"]] + ([state[pre + "shared.sg"]] if self.shared_gate else [])
        self.router = torch.cat(rows, dim=0).to(torch.float32).contiguous()  # the router is fp32 whatever the compute dtype
        if self.gated:  # gate rows first, then up rows: one product yields both
            self.up = torch.stack([torch.cat([state[pre + f"e{e}.gate"], state[pre + f"e{e}.up"]], dim=0) for e in range(self.experts)]).contiguous()
        else:
            self.up = torch.stack([state[pre + f"e{e}.up"] for e in range(self.experts)]).contiguous()  # [E, ff, hidden]
        self.correction = state[self.correction_name].to(torch.float32).contiguous() if self.correction_name else None
        self.down = torch.stack([state[pre + f"e{e}.down"] for e in range(self.experts)]).contiguous()  # [E, hidden, ff]
        if self.shared is not None:
            self.shared.load(state)

    def scratch_row_bytes(self) -> int:
        return 2 * self.top * (4 * self.hidden + (12 if self.gated else 4) * self.ff + 4 * self.hidden) + 8 * self.hidden + 4 * self.shared_ff + 4 * (self.experts + 1)

    def forward(self, ctx, x, h, store=False):
        n, dt, top = x.shape[0], self.rt.dtype, self.top
        # tiles of 128 rows where the tcgen05 product takes them (bfloat16, depths that are multiples of 8), else of 64
        tile = ops.MOE_TILE_TC if dt == torch.bfloat16 and self.hidden % 8 == 0 and self.ff % 8 == 0 else ops.MOE_TILE
        i32, f32 = torch.int32, torch.float32
        choice, weight = ctx.buf((n, top), i32), ctx.buf((n, top), f32)
        gate = ctx.buf((n,), f32) if self.shared_gate else None
        ops.moe_router(choice, weight, gate, x, self.router, self.routed, top, self.score == "softmax", self.renormalize, self.correction, self.renorm_eps,
                       self.groups, self.keep, self.route_scale)
        pairs = n * top
        tiles = -(-pairs // tile) + self.experts  # every expert may end on a tile that is not full
        dest, tile_expert = ctx.buf((n, top), i32), ctx.buf((tiles,), i32)
        ops.moe_sort(dest, tile_expert, choice, self.experts, tile)
        rows = tiles * tile
        xs = ctx.buf((rows, self.hidden), dt)
        ops.moe_scatter(xs, x, weight if self.weight_on_input else None, dest, top)
        mid = ctx.buf((rows, self.ff), dt)
        if self.gated:
            # gate and up in one product whose epilogue multiplies them (the tcgen05 kernel), else the sums of both and a kernel that gates
            if not ops.gemm_by_tile_gated(mid, xs, self.up, tile_expert, tile):
                both = ctx.buf((rows, 2 * self.ff), f32)
                ops.gemm_by_tile(both, xs, self.up, tile_expert, tile)
                ops.gate_up(mid, both)
        else:
            ops.gemm_by_tile(mid, xs, self.up, tile_expert, tile, act=self.act)
        ys = ctx.buf((rows, self.hidden), f32)
        ops.gemm_by_tile(ys, mid, self.down, tile_expert, tile)
        shared = None
        if self.shared is not None:
            shared = ctx.buf((n, self.hidden), f32)
            self.shared.forward(ctx, x, shared, store=True)
        # written when the caller wants the output alone, else added into the stream in the same kernel
        ops.moe_combine(h, ys, dest, None if self.weight_on_input else weight, shared, gate, top, x if self.identity else None, add=not store)


register_part("feed_forward", "routed_experts", RoutedExperts)
