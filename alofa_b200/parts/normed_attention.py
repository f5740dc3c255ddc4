"""Softmax attention without rotation over a paged key/value cache, with the
options of designs that take positions in by other means:

* ``qk_norm``: q and k are divided by their root mean square over the head's
  channels (eps inside the root, no weight);
* ``q_temp_coef`` / ``q_temp_every``: the query at position p is multiplied by
  ``1 + coef * ln(floor((p + 1) / every) + 1)``;
* ``scale``: scores are ``(q . k) * scale``;
* ``softcap``: then ``softcap * tanh(score / softcap)``;
* ``bias``: q, k and v have biases (``<tensor>.b``), added in the projection;
* ``position``: a position part whose rotation (neighbouring pairs, angles in
  fp32 in the kernel) turns the first dimensions of every q and k head;
* ``sink``: the softmax's denominator holds one more term ``exp(sink)`` that
  belongs to no key and has no value (0.0: "one added to the denominator");
* keys of ``dim`` channels per head, values of ``vdim`` (the two caches have
  their own widths); query head h reads key/value head ``h // (heads /
  kv_heads)``; causal, all keys or the last ``window``.

q, k and v come from one stacked projection whose fp32 sums a kernel norms,
scales and writes to the query buffer and the tokens' cache slots.  Scores and
softmax are fp32 in both compute dtypes."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..errors import AlofaError
from .attention import PagedAttend
from .base import PagedKV, Part, TensorSpec, as_float32_vector, build_part, register_part
from .linear import RESIDUAL, STORE, Linear, add_into_stream


class NormedAttention(PagedAttend, Part):
    family = "mixer"
    graph_safe = True
    stores_output = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.param
        self.hidden = int(p("hidden_size"))
        self.heads, self.kv_heads, self.dim, self.vdim = int(p("heads")), int(p("kv_heads")), int(p("dim")), int(p("vdim"))
        self.scale = float(p("scale"))
        self.softcap = float(self.params.get("softcap") or 0.0)
        self.qk_norm = bool(self.params.get("qk_norm", False))
        self.eps = float(self.params.get("eps") or 0.0)
        self.coef = float(self.params.get("q_temp_coef") or 0.0)
        self.every = int(self.params.get("q_temp_every") or 1)
        self.window = self.params.get("window")
        self.bias = bool(self.params.get("bias", False))
        self.sink_score = self.params.get("sink")  # None: no sink
        self.sink = None
        self.position = build_part("position", self.params["position"], rt) if self.params.get("position") is not None else None
        self.rot_dims = int(getattr(self.position, "dims", 0)) if self.position is not None else 0
        if self.position is not None and (not hasattr(self.position, "frequencies") or self.rot_dims > self.dim):
            raise AlofaError("unsupported", "this attention rotates neighbouring pairs only, at most the head's dimensions", f"position={self.params['position']}")
        if min(self.heads, self.kv_heads, self.dim, self.vdim) <= 0 or self.heads % self.kv_heads:
            raise AlofaError("invalid_argument", "kv heads must divide heads, sizes must be positive", f"params={self.params}")
        if self.vdim > 256:
            raise AlofaError("unsupported", "value heads of more than 256 channels", f"vdim={self.vdim}")
        if self.every <= 0 or self.softcap < 0:
            raise AlofaError("invalid_argument", "q_temp_every must be positive and softcap not negative", f"params={self.params}")
        self.q_dim, self.k_dim, self.v_dim = self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim
        self.nh, self.nkv, self.hd = self.heads, self.kv_heads, self.dim  # what the shared choice of kernels goes by (keys and values alike only)

    def cache_spec(self):
        return PagedKV(self.kv_heads, self.dim, self.window, self.vdim)

    def scratch_row_bytes(self) -> int:
        return 4 * (self.q_dim + self.k_dim + self.v_dim) + 4 * self.q_dim + 4 * self.heads * self.vdim + 8 * self.hidden

    def tensors(self):
        pre = self.prefix
        t = {pre + "q": TensorSpec((self.q_dim, self.hidden)), pre + "k": TensorSpec((self.k_dim, self.hidden)), pre + "v": TensorSpec((self.v_dim, self.hidden)),
             pre + "o": TensorSpec((self.hidden, self.heads * self.vdim))}
        if self.bias:
            t.update({pre + "q.b": TensorSpec((self.q_dim,)), pre + "k.b": TensorSpec((self.k_dim,)), pre + "v.b": TensorSpec((self.v_dim,))})
        return t

    def load(self, state):
        pre = self.prefix
        b = as_float32_vector(torch.cat([state[pre + n + ".b"] for n in "qkv"], dim=0)) if self.bias else None
        self.qkv = Linear(torch.cat([state[pre + n] for n in "qkv"], dim=0), b, STORE)
        if self.position is not None:
            self.position.load(state)
        if self.sink_score is not None:
            self.sink = torch.full((self.heads,), float(self.sink_score), dtype=torch.float32, device=state[pre + "o"].device)
        self.out_add = Linear(state[pre + "o"], None, RESIDUAL)
        self.out_store = Linear(state[pre + "o"], None, STORE)

    def forward(self, ctx, x, h, cache, writes=True, store=False):
        if not writes:
            raise AlofaError("unsupported", "this attention does not read another run's cache")
        n, dt = x.shape[0], self.rt.dtype
        group = ctx.groups[cache.group]
        sums = ctx.buf((n, self.q_dim + self.k_dim + self.v_dim), torch.float32)
        self.qkv(sums, x, buf=ctx.buf)
        q = ctx.buf((n, self.q_dim), dt)
        ops.qkv_prepare(q, cache.k, cache.v, sums, ctx.positions, group.slot_map, self.heads, self.kv_heads, self.dim, self.vdim, self.qk_norm, self.eps, self.coef, self.every,
                        self.position.frequencies() if self.rot_dims else None, self.rot_dims)
        if self.dim == self.vdim:
            out = self.attend(ctx, q, cache, group)  # the tensor-core kernels in bfloat16 for the head sizes they are built for, else the every-size kernel
        else:
            out = ctx.buf((n, self.heads * self.vdim), dt)
            ops.paged_attention_generic(out, q, cache.k, cache.v, ctx.positions, ctx.seq_of_token, group.block_table, group.page_size, self.heads, self.kv_heads,
                                        self.dim, self.window, self.scale, self.softcap, self.vdim, self.sink)
        if store:
            self.out_store(h, out, buf=ctx.buf)
        else:
            add_into_stream(ctx, self.out_add, h, out)


register_part("mixer", "normed_attention", NormedAttention)
