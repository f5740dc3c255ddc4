"""Latent attention over a paged cache of one row per token.

Queries and keys/values both go through a low-rank latent: ``c_q = rmsnorm(x
Wdq^T)``, ``q = c_q Wuq^T`` laid out head by head as [dim unrotated | rot
rotated]; ``x Wdkv^T`` gives kv_rank numbers whose RMSNorm is the latent ``c``
and rot numbers that, turned by the position, are ONE rotated key part shared
by all heads.  Per head the unrotated key is ``Wuk_h c`` and the value ``Wuv_h
c``; the score is ``(q_h . k_h + qr_h . kr) * scale``; the softmax denominator
may hold one more term ``exp(sink_h)`` that belongs to no key; the output
projection takes the concatenated heads.

Only ``[c | kr]`` is cached (:class:`~alofa_b200.parts.base.PagedRows`).  The
unrotated query is carried into the latent space once (``Wuk_h^T q_h``, a
product per head) so that every head attends to the same cached rows, whose
first kv_rank numbers also serve as the value; ``Wuv_h`` is applied to the
attention output of the head.  Both per-head products are one batched launch.
The stacked ``[Wdq; Wdkv]`` makes both down-projections one product.

Options: ``q_rank`` 0 or absent: no query latent, ``q = x Wq^T`` (tensor
``q``) and the down-projection is ``Wdkv`` alone; ``gate``: head h's output is
multiplied by ``sigmoid(x Wg^T)_h`` (tensor ``g`` [heads, hidden], stacked
under the down-projection); the position part may pair halves and carry a
magnitude (:class:`~alofa_b200.parts.position.RotaryInterleaved`)."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..errors import AlofaError
from . import fast_linear
from .base import PagedRows, Part, TensorSpec, as_float32_vector, build_part, register_part
from .linear import STORE, Linear


class LatentAttention(Part):
    family = "mixer"
    stores_output = True  # forward(..., store=True) writes its output instead of adding it

    @property
    def graph_safe(self):
        return self.position.graph_safe

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.param
        self.hidden = int(p("hidden_size"))
        self.heads = int(p("heads"))
        self.dim = int(p("dim", 0) or 0)
        self.rot = int(p("rot_dim", 0) or 0)
        self.vdim = int(p("vdim"))
        self.kv_rank = int(p("kv_rank"))
        self.q_rank = int(self.params.get("q_rank") or 0)  # 0: queries come straight from x
        self.gate = bool(self.params.get("gate", False))
        self.scale = float(p("scale"))
        self.eps = float(p("eps"))
        self.has_sink = bool(p("sink", False))
        self.window = self.params.get("window")
        if self.dim + self.rot <= 0 or self.kv_rank > 1024:
            raise AlofaError("unsupported", "latent attention wants a head of at least one dimension and a latent of at most 1024", f"dim={self.dim} rot={self.rot} kv_rank={self.kv_rank}")
        self.position = build_part("position", p("position"), rt)
        self.rot_dims = int(getattr(self.position, "dims", 0))
        self.halves = bool(getattr(self.position, "halves", False))
        self.magnitude = float(getattr(self.position, "magnitude", 1.0))
        if self.rot_dims > self.rot:
            raise AlofaError("invalid_argument", "more rotated dimensions than the rotated part has", f"dims={self.rot_dims} rot_dim={self.rot}")
        self.width = self.kv_rank + self.rot  # a cache row
        self.down = self.up_q = self.out = self.uk_t = self.uv = self.sink = None

    def cache_spec(self):
        return PagedRows(self.width, self.window)

    def scratch_row_bytes(self) -> int:
        h = self.heads
        return 4 * (self.q_rank + self.width + h) + 4 * self.q_rank + 4 * h * (self.dim + self.rot) + 4 * h * self.width + 4 * h * self.kv_rank + 4 * h * self.vdim + 4 * self.hidden

    def tensors(self):
        pre, h = self.prefix, self.heads
        t = {
            pre + "dkv": TensorSpec((self.width, self.hidden)),
            pre + "dkv.norm": TensorSpec((self.kv_rank,), "ones"),
            pre + "uk": TensorSpec((h * self.dim, self.kv_rank)),
            pre + "uv": TensorSpec((h * self.vdim, self.kv_rank)),
            pre + "o": TensorSpec((self.hidden, h * self.vdim)),
        }
        if self.q_rank:
            t.update({pre + "dq": TensorSpec((self.q_rank, self.hidden)), pre + "dq.norm": TensorSpec((self.q_rank,), "ones"),
                      pre + "uq": TensorSpec((h * (self.dim + self.rot), self.q_rank))})
        else:
            t[pre + "q"] = TensorSpec((h * (self.dim + self.rot), self.hidden))
        if self.gate:
            t[pre + "g"] = TensorSpec((h, self.hidden))
        if self.has_sink:
            t[pre + "sink"] = TensorSpec((h,))
        t.update(self.position.tensors())
        return t

    def load(self, state):
        pre, h = self.prefix, self.heads
        # one product for everything that leaves fp32 sums: [Wdq; Wdkv; Wg]
        stacked = ([state[pre + "dq"]] if self.q_rank else []) + [state[pre + "dkv"]] + ([state[pre + "g"]] if self.gate else [])
        self.down = Linear(torch.cat(stacked, dim=0), None, STORE)
        self.q_norm = as_float32_vector(state[pre + "dq.norm"]) if self.q_rank else None
        self.kv_norm = as_float32_vector(state[pre + "dkv.norm"])
        self.up_q = Linear(state[pre + "uq"] if self.q_rank else state[pre + "q"], None, STORE)
        # [heads, kv_rank, dim]: row c of head h holds column c of Wuk_h, so the per-head product q_h -> Wuk_h^T q_h reads rows
        self.uk_t = state[pre + "uk"].view(h, self.dim, self.kv_rank).transpose(1, 2).contiguous() if self.dim else None
        self.uv = state[pre + "uv"].contiguous()
        self.out = Linear(state[pre + "o"], None, STORE)
        self.sink = as_float32_vector(state[pre + "sink"]) if self.has_sink else None
        self.position.load(state)

    def forward(self, ctx, x, h, cache, writes=True, store=False):
        """``h`` += (or, with ``store``, =) the mixer's output for the rows ``x``;
        ``h`` is fp32 [tokens, hidden]."""
        n, dt, heads = x.shape[0], self.rt.dtype, self.heads
        group = ctx.groups[cache.group]
        freq = self.position.frequencies()
        gate_at = self.q_rank + self.width
        lat = ctx.buf((n, gate_at + (heads if self.gate else 0)), torch.float32)
        self.down(lat, x, buf=ctx.buf)
        cq = ctx.buf((n, self.q_rank), dt) if self.q_rank else None
        ops.latent_prepare(cq, cache.k if writes else None, lat, self.q_norm, self.kv_norm, freq, ctx.positions, group.slot_map,
                           self.q_rank, self.kv_rank, self.rot, self.rot_dims, self.eps, self.halves, self.magnitude)
        q = ctx.buf((n, heads * (self.dim + self.rot)), dt)
        self.up_q(q, cq if self.q_rank else x, buf=ctx.buf)
        qa = ctx.buf((n, heads * self.width), dt)
        ops.latent_query_turn(qa, q, freq, ctx.positions, heads, self.dim, self.rot, self.rot_dims, self.kv_rank, self.halves, self.magnitude)
        if self.dim:
            # per head: qa[:, h, :kv_rank] = q[:, h, :dim] Wuk_h
            ops.gemm_batched(qa, q, self.uk_t, heads, n, self.kv_rank, self.dim, heads * (self.dim + self.rot), self.dim + self.rot,
                             self.dim, self.kv_rank * self.dim, heads * self.width, self.width)
        else:
            qa.view(n, heads, self.width)[:, :, : self.kv_rank].zero_()
        o_lat = ctx.buf((n, heads * self.kv_rank), dt)
        self.attend(ctx, o_lat, qa, cache, group)
        o = ctx.buf((n, heads * self.vdim), dt)
        # per head: o[:, h] = o_lat[:, h] Wuv_h^T
        ops.gemm_batched(o, o_lat, self.uv, heads, n, self.vdim, self.kv_rank, heads * self.kv_rank, self.kv_rank, self.kv_rank, self.vdim * self.kv_rank,
                         heads * self.vdim, self.vdim)
        if self.gate:
            ops.head_gate(o, lat, gate_at, heads, self.vdim)
        if store:
            self.out(h, o, buf=ctx.buf)
        else:
            y = ctx.buf(tuple(h.shape), torch.float32)
            self.out(y, o, buf=ctx.buf)
            h.add_(y)

    def attend(self, ctx, o_lat, qa, cache, group):
        """Attention of the step's rows over the cached latent rows: on tensor
        cores for bfloat16 and sizes that kernel is built for, else the kernel
        that takes every size."""
        if qa.dtype == torch.bfloat16 and ops.latent_attention_bf16_supported(self.kv_rank, self.rot):
            splits, per_split, part_o, part_ml = 1, 0, None, None
            if ctx.decode_only:
                # a request alone is one CTA per 64 (token, head) rows: its key blocks are dealt to as many CTAs as are
                # resident together (two per SM up to a latent of 256, else one; a second wave doubled the time),
                # no split shorter than 256 keys; a recorded step is sized for its bucket of contexts
                longest = ctx.max_context if ctx.capturing else ctx.max_kv_len
                blocks = -(-max(1, longest) // ops.LATENT_KEY_BLOCK)
                narrow = self.heads <= 16  # the kernel's narrow shape: 16-row tiles, two CTAs to an SM whatever the latent
                ctas = ctx.n_seqs * -(-self.heads // (16 if narrow else 64))
                splits = max(1, min((2 if narrow or self.kv_rank <= 256 else 1) * fast_linear.SMS // ctas, blocks // 8))
                per_split = -(-blocks // splits)
                splits = -(-blocks // per_split)
                if splits > 1:
                    part_o = ctx.buf((splits, ctx.n_tokens * self.heads, self.kv_rank), torch.float32)
                    part_ml = ctx.buf((splits, ctx.n_tokens * self.heads, 2), torch.float32)
            ops.latent_attention_bf16(o_lat, qa, cache.k, self.sink, ctx.q_start, ctx.kv_len, group.block_table, group.page_size, ctx.n_seqs, ctx.max_q_len,
                                      self.heads, self.kv_rank, self.rot, self.window, self.scale, splits, per_split, part_o, part_ml)
            return
        ops.latent_attention(o_lat, qa, cache.k, self.sink, ctx.positions, ctx.seq_of_token, group.block_table, group.page_size,
                             self.heads, self.kv_rank, self.rot, self.window, self.scale)


register_part("mixer", "latent_attention", LatentAttention)
