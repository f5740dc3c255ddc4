"""Mixers that carry a state of fixed size per request instead of a growing
cache: a state-space mixer with one scalar decay per head, and gated linear
attention with one decay per key channel.  Both are the recurrence

    S_t = diag(a_t) S_(t-1) + k_t v_t^T,    y_t = S_t^T q_t

over a matrix state per head (key channels x value channels), run by one kernel
(``ops.linear_scan``) that walks a request's tokens in order, in prompts and in
decoding alike.  The state is fp32 and lives in the request's slot
(:class:`~alofa_b200.parts.base.SlotState`); it is zero when a request starts.
Decays, step sizes, softplus and exponentials, the norms and the gates are
fp32 in both compute dtypes; bfloat16 only rounds the rows handed to the
projections.

``state_space``: ``[z | x | B | C | dt] = W_in h``; x, B and C pass a causal
convolution per channel (``conv`` taps, bias, silu; the last ``conv - 1`` inputs
are part of the state); ``dt = softplus(dt + dt_bias)``; per head, with the
keys and queries of its group, ``a_t = exp(-exp(A_log) dt_t)``, ``k_t = dt_t
B_t``, ``q_t = C_t``, ``y_t += D x_t``; then ``y * silu(z)``, an RMS norm in
``norm_groups`` equal parts times a weight, and the output projection.

``gated_linear_attention``: ``q = W_q h / sqrt(dim)``, ``k = W_k h``, ``v = W_v
h``; ``a_t = sigmoid(W_a2 (W_a1 h) + b)^(1/tau)`` per key channel; each head's
output is RMS-normed over its value channels with one weight shared by the
heads, the heads are concatenated, multiplied by ``silu(W_g h)`` and projected.

``min_gru``: a recurrence element by element whose gates read the current
token only: ``z = sigmoid(W_z h + b_z)``, ``x = W_x h + b_x``, the candidate ``x
+ 1/2`` where ``x >= 0`` and ``sigmoid(x)`` below, ``S_t = (1 - z) S_(t-1) + z
* candidate``; the output is ``W_o (S_t * silu(W_g h))``.

``gated_delta``: the gated delta rule over a matrix state per head with one
decay per head and key channel, ``S <- diag(g_t) S; u = beta_t (v_t - S^T
k_t); S <- S + k_t u^T; o_t = S^T q_t``; q, k and v each pass a short causal
convolution per channel (no bias) and silu, q and k are made unit vectors per
head (q also times ``dim^(-1/2)``), ``beta = sigmoid(W_b h)``, ``g =
exp(-exp(A_log) * softplus(W_a2 (W_a1 h) + dt_bias))``; every head's output is
RMS-normed over its value channels with one weight shared by the heads and
multiplied by ``sigmoid(W_g2 (W_g1 h))``, then projected.

``gated_lru``: the recurrent block with a real-gated linear recurrent unit.
Two branches of ``width`` channels: ``y = act(W_y h + b_y)`` and ``u =
conv(W_x h + b_x)``, a causal convolution per channel with a bias and no
activation.  The channels form ``blocks`` equal parts, and in each part b ``r =
sigmoid(A_b u_b + a_b)``, ``i = sigmoid(I_b u_b + i_b)`` with square matrices;
``log a = -decay_scale * r * softplus(lam)``, ``S_t = a S_(t-1) + sqrt(1 - a^2)
* i * u`` from ``S = 0`` (the first token is no special case); the output is
``W_o (S_t * y)``."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..errors import AlofaError
from .base import Part, SlotState, TensorSpec, as_float32_vector, register_part
from .linear import RESIDUAL, STORE, Linear, add_into_stream

# blocks a scan launch should have before its value channels stop being dealt to more of them (about one per SM)
SCAN_SPREAD = 128


def _project_out(ctx, linear_add: Linear, linear_store: Linear, h, x, store: bool) -> None:
    if store:
        linear_store(h, x, buf=ctx.buf)
    else:
        add_into_stream(ctx, linear_add, h, x)


class StateSpaceMixer(Part):
    family = "mixer"
    graph_safe = True
    stores_output = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.param
        self.hidden = int(p("hidden_size"))
        self.heads, self.vdim, self.state, self.groups = int(p("heads")), int(p("vdim")), int(p("state")), int(p("groups"))
        self.taps, self.norm_groups, self.eps = int(p("conv")), int(p("norm_groups")), float(p("eps"))
        if min(self.heads, self.vdim, self.state, self.groups, self.taps, self.norm_groups) <= 0 or self.heads % self.groups:
            raise AlofaError("invalid_argument", "state-space sizes must be positive and groups must divide heads", f"params={self.params}")
        if self.state > 1024:
            raise AlofaError("unsupported", "the recurrence kernel holds at most 1,024 key channels a head", f"state={self.state}")
        self.inner = self.heads * self.vdim
        if self.inner % self.norm_groups:
            raise AlofaError("invalid_argument", "norm_groups must divide heads * vdim", f"inner={self.inner} norm_groups={self.norm_groups}")
        self.bc = self.groups * self.state
        self.channels = self.inner + 2 * self.bc  # what passes the convolution: x, B, C
        self.in_rows = 2 * self.inner + 2 * self.bc + self.heads
        self.conv_words = (self.taps - 1) * self.channels
        self.scan_words = self.heads * self.vdim * self.state

    def cache_spec(self):
        # one fp32 vector per request: the recurrence's state [head][value][key], then the convolution's last inputs
        return SlotState((self.scan_words + self.conv_words,), torch.float32)

    def scratch_row_bytes(self) -> int:
        return 4 * (self.in_rows + self.channels + 2 * self.inner + 2 * self.heads) + 8 * self.hidden

    def tensors(self):
        pre = self.prefix
        return {
            pre + "in": TensorSpec((self.in_rows, self.hidden)),
            pre + "conv": TensorSpec((self.channels, self.taps)),
            pre + "conv.b": TensorSpec((self.channels,)),
            pre + "dt_bias": TensorSpec((self.heads,)),
            pre + "A_log": TensorSpec((self.heads,)),
            pre + "D": TensorSpec((self.heads,), "ones"),
            pre + "norm": TensorSpec((self.inner,), "ones"),
            pre + "o": TensorSpec((self.hidden, self.inner)),
        }

    def load(self, state):
        pre = self.prefix
        self.w_in = Linear(state[pre + "in"], None, STORE)
        self.conv_w = state[pre + "conv"].to(torch.float32).contiguous()
        self.conv_b = as_float32_vector(state[pre + "conv.b"])
        self.dt_bias = as_float32_vector(state[pre + "dt_bias"])
        self.a_log = as_float32_vector(state[pre + "A_log"])
        self.d_skip = as_float32_vector(state[pre + "D"])
        self.norm_w = as_float32_vector(state[pre + "norm"])
        self.out_add = Linear(state[pre + "o"], None, RESIDUAL)
        self.out_store = Linear(state[pre + "o"], None, STORE)

    def forward(self, ctx, x, h, cache, writes=True, store=False):
        n, f32 = x.shape[0], torch.float32
        inner, bc = self.inner, self.bc
        u = ctx.buf((n, self.in_rows), f32)  # [z | x | B | C | dt], the projection's fp32 sums
        self.w_in(u, x, buf=ctx.buf)
        st = cache.state
        xbc = ctx.buf((n, self.channels), f32)
        ops.causal_conv(xbc, u, inner, self.conv_w, self.conv_b, st[:, self.scan_words:], ctx.q_start, ctx.state_slots, ctx.seq_of_token, ctx.n_seqs)
        y = ctx.buf((n, inner), f32)
        work = ctx.buf((ops.linear_scan_work(n, self.heads, self.state, 0),), f32)
        ops.linear_scan(y, xbc, 0, xbc, inner, xbc, inner + bc, u, 2 * inner + 2 * bc, st, ctx.q_start, ctx.state_slots, ctx.n_seqs, self.heads, self.groups,
                        self.state, self.vdim, 0, dt_bias=self.dt_bias, a_log=self.a_log, d_skip=self.d_skip, spread=SCAN_SPREAD, work=work)
        normed = ctx.buf((n, inner), self.rt.dtype)
        ops.gated_group_norm(normed, y, u, 0, self.norm_w, self.norm_groups, self.eps, gate_first=True)
        _project_out(ctx, self.out_add, self.out_store, h, normed, store)


class GatedLinearAttention(Part):
    family = "mixer"
    graph_safe = True
    stores_output = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.param
        self.hidden = int(p("hidden_size"))
        self.heads, self.dim, self.vdim = int(p("heads")), int(p("dim")), int(p("vdim"))
        self.tau, self.eps = float(p("tau")), float(p("eps"))
        if min(self.heads, self.dim, self.vdim) <= 0 or self.tau <= 0:
            raise AlofaError("invalid_argument", "gated linear attention sizes and tau must be positive", f"params={self.params}")
        if self.dim > 1024:
            raise AlofaError("unsupported", "the recurrence kernel holds at most 1,024 key channels a head", f"dim={self.dim}")
        self.qk, self.v = self.heads * self.dim, self.heads * self.vdim
        self.rows = 2 * self.qk + 2 * self.v  # [q | k | v | g]
        self.rank = None  # the decay's inner size, from the tensor's shape

    def cache_spec(self):
        return SlotState((self.heads * self.vdim * self.dim,), torch.float32)

    def scratch_row_bytes(self) -> int:
        return 4 * (self.rows + 2 * self.qk + 2 * self.v) + 8 * self.hidden + 64

    def tensors(self):
        pre = self.prefix
        rank = -int(self.params.get("decay_rank") or 16)  # the decay's inner size is the tensors' own; this many for random weights
        return {
            pre + "q": TensorSpec((self.qk, self.hidden)), pre + "k": TensorSpec((self.qk, self.hidden)), pre + "v": TensorSpec((self.v, self.hidden)),
            pre + "g": TensorSpec((self.v, self.hidden)), pre + "o": TensorSpec((self.hidden, self.v)), pre + "norm": TensorSpec((self.vdim,), "ones"),
            pre + "a1": TensorSpec((rank, self.hidden)), pre + "a2": TensorSpec((self.qk, rank)), pre + "a2.b": TensorSpec((self.qk,)),
        }

    def load(self, state):
        pre = self.prefix
        self.w_in = Linear(torch.cat([state[pre + n] for n in ("q", "k", "v", "g")], dim=0), None, STORE)
        self.a1 = Linear(state[pre + "a1"], None, STORE)
        self.a2 = Linear(state[pre + "a2"], as_float32_vector(state[pre + "a2.b"]), STORE)
        self.rank = state[pre + "a1"].shape[0]
        if state[pre + "a2"].shape[1] != self.rank:
            raise AlofaError("invalid_argument", "the two decay projections disagree about their inner size", f"a1={tuple(state[pre + 'a1'].shape)} a2={tuple(state[pre + 'a2'].shape)}")
        self.norm_w = as_float32_vector(state[pre + "norm"])
        self.out_add = Linear(state[pre + "o"], None, RESIDUAL)
        self.out_store = Linear(state[pre + "o"], None, STORE)

    def forward(self, ctx, x, h, cache, writes=True, store=False):
        n, f32 = x.shape[0], torch.float32
        u = ctx.buf((n, self.rows), f32)  # [q | k | v | g]
        self.w_in(u, x, buf=ctx.buf)
        low = ctx.buf((n, self.rank), self.rt.dtype)
        self.a1(low, x, buf=ctx.buf)
        z = ctx.buf((n, self.qk), f32)  # the decays' logits, one per key channel
        self.a2(z, low, buf=ctx.buf)
        y = ctx.buf((n, self.v), f32)
        work = ctx.buf((ops.linear_scan_work(n, self.heads, self.dim, 1),), f32)
        ops.linear_scan(y, u, 2 * self.qk, u, self.qk, u, 0, z, 0, cache.state, ctx.q_start, ctx.state_slots, ctx.n_seqs, self.heads, self.heads, self.dim,
                        self.vdim, 1, tau=self.tau, q_scale=self.dim ** -0.5, spread=SCAN_SPREAD, work=work)
        normed = ctx.buf((n, self.v), self.rt.dtype)
        ops.gated_group_norm(normed, y, u, 2 * self.qk + self.v, self.norm_w, self.heads, self.eps, gate_first=False)
        _project_out(ctx, self.out_add, self.out_store, h, normed, store)


class MinGRU(Part):
    family = "mixer"
    graph_safe = True
    stores_output = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden, self.width = int(self.param("hidden_size")), int(self.param("width"))
        if self.width <= 0:
            raise AlofaError("invalid_argument", "the recurrence's width must be positive", f"params={self.params}")

    def cache_spec(self):
        return SlotState((self.width,), torch.float32)

    def scratch_row_bytes(self) -> int:
        return 4 * 3 * self.width + 4 * self.width + 8 * self.hidden

    def tensors(self):
        pre = self.prefix
        return {pre + "z": TensorSpec((self.width, self.hidden)), pre + "z.b": TensorSpec((self.width,)), pre + "x": TensorSpec((self.width, self.hidden)),
                pre + "x.b": TensorSpec((self.width,)), pre + "g": TensorSpec((self.width, self.hidden)), pre + "o": TensorSpec((self.hidden, self.width))}

    def load(self, state):
        pre = self.prefix
        bias = torch.cat([as_float32_vector(state[pre + "z.b"]), as_float32_vector(state[pre + "x.b"]), torch.zeros(self.width, dtype=torch.float32, device=state[pre + "g"].device)])
        self.w_in = Linear(torch.cat([state[pre + n] for n in ("z", "x", "g")], dim=0), bias, STORE)  # [z | x | g]
        self.out_add = Linear(state[pre + "o"], None, RESIDUAL)
        self.out_store = Linear(state[pre + "o"], None, STORE)

    def forward(self, ctx, x, h, cache, writes=True, store=False):
        n, w = x.shape[0], self.width
        u = ctx.buf((n, 3 * w), torch.float32)  # the projections' fp32 sums, biases added
        self.w_in(u, x, buf=ctx.buf)
        y = ctx.buf((n, w), self.rt.dtype)
        ops.min_gru(y, u, 0, w, 2 * w, cache.state, ctx.q_start, ctx.state_slots, ctx.n_seqs)
        _project_out(ctx, self.out_add, self.out_store, h, y, store)


class GatedDelta(Part):
    family = "mixer"
    graph_safe = True
    stores_output = True

    UNIT_EPS = 1e-6  # inside the root of the unit norms of q and k

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.param
        self.hidden = int(p("hidden_size"))
        self.heads, self.kv_heads, self.dim, self.vdim = int(p("heads")), int(p("kv_heads")), int(p("dim")), int(p("vdim"))
        self.taps, self.eps = int(p("conv")), float(p("eps"))
        if min(self.heads, self.kv_heads, self.dim, self.vdim, self.taps) <= 0 or self.heads % self.kv_heads:
            raise AlofaError("invalid_argument", "delta-rule sizes must be positive and kv_heads must divide heads", f"params={self.params}")
        if self.dim > 1024:
            raise AlofaError("unsupported", "the recurrence kernel holds at most 1,024 key channels a head", f"dim={self.dim}")
        self.qk, self.v = self.kv_heads * self.dim, self.heads * self.vdim
        self.decays = self.heads * self.dim
        self.channels = 2 * self.qk + self.v  # what passes the convolution: q, k, v
        self.in_rows = self.channels + self.heads  # [q | k | v | beta]
        self.scan_words = self.heads * self.vdim * self.dim
        self.conv_words = (self.taps - 1) * self.channels
        self.rank_a = self.rank_g = None  # the inner sizes of the decays' and the gate's projections, from the tensors

    def cache_spec(self):
        # one fp32 vector per request: the state [head][value][key], then the convolution's last inputs
        return SlotState((self.scan_words + self.conv_words,), torch.float32)

    def scratch_row_bytes(self) -> int:
        return 4 * (self.in_rows + self.channels + 2 * (self.decays + self.v) + 2 * self.qk + 2 * self.heads + self.kv_heads + 2 * self.v) + 8 * self.hidden + 512

    def tensors(self):
        pre = self.prefix
        ra, rg = -int(self.params.get("decay_rank") or 16), -int(self.params.get("gate_rank") or 16)  # the files' own; these for random weights
        return {
            pre + "q": TensorSpec((self.qk, self.hidden)), pre + "q.conv": TensorSpec((self.qk, self.taps)),
            pre + "k": TensorSpec((self.qk, self.hidden)), pre + "k.conv": TensorSpec((self.qk, self.taps)),
            pre + "v": TensorSpec((self.v, self.hidden)), pre + "v.conv": TensorSpec((self.v, self.taps)),
            pre + "b": TensorSpec((self.heads, self.hidden)), pre + "A_log": TensorSpec((self.heads,)), pre + "norm": TensorSpec((self.vdim,), "ones"),
            pre + "a1": TensorSpec((ra, self.hidden)), pre + "a2": TensorSpec((self.decays, ra)), pre + "dt_bias": TensorSpec((self.decays,)),
            pre + "g1": TensorSpec((rg, self.hidden)), pre + "g2": TensorSpec((self.v, rg)), pre + "o": TensorSpec((self.hidden, self.v)),
        }

    def load(self, state):
        pre = self.prefix
        self.w_in = Linear(torch.cat([state[pre + n] for n in ("q", "k", "v", "b")], dim=0), None, STORE)
        self.conv_w = torch.cat([state[pre + n + ".conv"] for n in ("q", "k", "v")], dim=0).to(torch.float32).contiguous()
        a1, a2, g1, g2 = (state[pre + n] for n in ("a1", "a2", "g1", "g2"))
        self.rank_a, self.rank_g = a1.shape[0], g1.shape[0]
        if a2.shape[1] != self.rank_a or g2.shape[1] != self.rank_g:
            raise AlofaError("invalid_argument", "the two halves of a low-rank projection disagree about their inner size",
                             f"a1={tuple(a1.shape)} a2={tuple(a2.shape)} g1={tuple(g1.shape)} g2={tuple(g2.shape)}")
        # both low-rank maps as two products: [a1; g1], then the second halves on the diagonal of one matrix (its zero blocks add exact zeros)
        self.low = Linear(torch.cat([a1, g1], dim=0), None, STORE)
        second = torch.zeros((self.decays + self.v, self.rank_a + self.rank_g), dtype=a2.dtype, device=a2.device)
        second[: self.decays, : self.rank_a] = a2
        second[self.decays :, self.rank_a :] = g2
        self.high = Linear(second, None, STORE)
        self.dt_bias = as_float32_vector(state[pre + "dt_bias"])
        self.a_log = as_float32_vector(state[pre + "A_log"])
        self.norm_w = as_float32_vector(state[pre + "norm"])
        self.out_add = Linear(state[pre + "o"], None, RESIDUAL)
        self.out_store = Linear(state[pre + "o"], None, STORE)

    def forward(self, ctx, x, h, cache, writes=True, store=False):
        n, f32 = x.shape[0], torch.float32
        H, G, N, P = self.heads, self.kv_heads, self.dim, self.vdim
        u = ctx.buf((n, self.in_rows), f32)  # [q | k | v | beta], the projection's fp32 sums
        self.w_in(u, x, buf=ctx.buf)
        low = ctx.buf((n, self.rank_a + self.rank_g), self.rt.dtype)
        self.low(low, x, buf=ctx.buf)
        z = ctx.buf((n, self.decays + self.v), f32)  # the decays' logits, then the output gate's
        self.high(z, low, buf=ctx.buf)
        st = cache.state
        xc = ctx.buf((n, self.channels), f32)
        ops.causal_conv(xc, u, 0, self.conv_w, None, st[:, self.scan_words:], ctx.q_start, ctx.state_slots, ctx.seq_of_token, ctx.n_seqs)
        qn, kn = ctx.buf((n, self.qk), f32), ctx.buf((n, self.qk), f32)
        kq, g, beta = ctx.buf((n, G), f32), ctx.buf((n, self.decays), f32), ctx.buf((n, H), f32)
        ops.delta_prepare(qn, kn, kq, g, beta, xc, z, u, self.channels, self.dt_bias, self.a_log, H, G, N, self.UNIT_EPS, N ** -0.5)
        y = ctx.buf((n, self.v), f32)
        ops.delta_scan(y, xc, 2 * self.qk, kn, qn, kq, g, beta, st, ctx.q_start, ctx.state_slots, ctx.n_seqs, H, G, N, P, spread=SCAN_SPREAD)
        normed = ctx.buf((n, self.v), self.rt.dtype)
        ops.gated_group_norm(normed, y, z, self.decays, self.norm_w, H, self.eps, gate_first=False, sigmoid=True)
        _project_out(ctx, self.out_add, self.out_store, h, normed, store)


class GatedLRU(Part):
    family = "mixer"
    graph_safe = True
    stores_output = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.param
        self.hidden, self.width, self.blocks, self.taps = int(p("hidden_size")), int(p("width")), int(p("blocks")), int(p("conv"))
        self.decay_scale = float(p("decay_scale"))
        self.act = str(p("activation", "gelu_tanh"))
        if min(self.width, self.blocks, self.taps) <= 0 or self.width % self.blocks or self.decay_scale <= 0:
            raise AlofaError("invalid_argument", "the recurrent unit's sizes must be positive and blocks must divide its width", f"params={self.params}")
        if self.act not in ops.ACTIVATIONS:
            raise AlofaError("unsupported", "unknown activation", f"activation={self.act} known={sorted(ops.ACTIVATIONS)}")
        self.block_size = self.width // self.blocks
        if self.block_size > 4096:
            raise AlofaError("unsupported", "the gates' kernel holds at most 4,096 channels a block", f"width={self.width} blocks={self.blocks}")

    def cache_spec(self):
        # one fp32 vector per request: the recurrence's state, then the convolution's last inputs
        return SlotState((self.width * self.taps,), torch.float32)

    def scratch_row_bytes(self) -> int:
        return 4 * 6 * self.width + 8 * self.hidden

    def tensors(self):
        pre, w, bs = self.prefix, self.width, self.block_size
        return {pre + "y": TensorSpec((w, self.hidden)), pre + "y.b": TensorSpec((w,)), pre + "x": TensorSpec((w, self.hidden)), pre + "x.b": TensorSpec((w,)),
                pre + "conv": TensorSpec((w, self.taps)), pre + "conv.b": TensorSpec((w,)),
                pre + "ra": TensorSpec((self.blocks, bs, bs)), pre + "ra.b": TensorSpec((self.blocks, bs)),
                pre + "ri": TensorSpec((self.blocks, bs, bs)), pre + "ri.b": TensorSpec((self.blocks, bs)),
                pre + "lam": TensorSpec((w,)), pre + "o": TensorSpec((self.hidden, w))}

    def load(self, state):
        pre, f32 = self.prefix, torch.float32
        bias = torch.cat([as_float32_vector(state[pre + "y.b"]), as_float32_vector(state[pre + "x.b"])])
        self.w_in = Linear(torch.cat([state[pre + "y"], state[pre + "x"]], dim=0), bias, STORE)  # [y | x]
        self.conv_w = state[pre + "conv"].to(f32).contiguous()
        self.conv_b = as_float32_vector(state[pre + "conv.b"])
        # the gates are part of the recurrence: fp32 whatever the compute dtype, [block][in][out] for the kernel
        self.wa_rows, self.wi_rows = state[pre + "ra"].to(f32).contiguous(), state[pre + "ri"].to(f32).contiguous()  # as stored, for steps of a few tokens
        self.wa_t, self.wi_t = self.wa_rows.transpose(1, 2).contiguous(), self.wi_rows.transpose(1, 2).contiguous()
        self.ba = as_float32_vector(state[pre + "ra.b"].reshape(-1))
        self.bi = as_float32_vector(state[pre + "ri.b"].reshape(-1))
        self.lam = as_float32_vector(state[pre + "lam"])
        self.out_add = Linear(state[pre + "o"], None, RESIDUAL)
        self.out_store = Linear(state[pre + "o"], None, STORE)

    def forward(self, ctx, x, h, cache, writes=True, store=False):
        n, w, f32 = x.shape[0], self.width, torch.float32
        u = ctx.buf((n, 2 * w), f32)  # the projections' fp32 sums, biases added
        self.w_in(u, x, buf=ctx.buf)
        st = cache.state
        xc = ctx.buf((n, w), f32)
        ops.causal_conv(xc, u, w, self.conv_w, self.conv_b, st[:, w:], ctx.q_start, ctx.state_slots, ctx.seq_of_token, ctx.n_seqs, act=False)
        a, b = ctx.buf((n, w), f32), ctx.buf((n, w), f32)
        ops.lru_gates(a, b, xc, self.wa_t, self.wi_t, self.ba, self.bi, self.lam, self.decay_scale, self.blocks, self.wa_rows, self.wi_rows)
        y = ctx.buf((n, w), self.rt.dtype)
        ops.lru_scan(y, a, b, u, 0, self.act, st, ctx.q_start, ctx.state_slots, ctx.n_seqs)
        _project_out(ctx, self.out_add, self.out_store, h, y, store)


register_part("mixer", "gated_lru", GatedLRU)
register_part("mixer", "min_gru", MinGRU)
register_part("mixer", "gated_delta", GatedDelta)
register_part("mixer", "state_space", StateSpaceMixer)
register_part("mixer", "gated_linear_attention", GatedLinearAttention)
