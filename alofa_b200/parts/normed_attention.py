"""Softmax attention without rotation over a paged key/value cache, with the
options of designs that take positions in by other means:

* ``qk_norm``: q and k are divided by their root mean square over the head's
  channels (eps inside the root); with ``norm_weight`` then multiplied by a
  plain weight of ``dim`` numbers, one for the queries and one for the keys
  (``q.norm``, ``k.norm``), shared by all heads;
* ``q_temp_coef`` / ``q_temp_every``: the query at position p is multiplied by
  ``1 + coef * ln(floor((p + 1) / every) + 1)``;
* ``scale``: scores are ``(q . k) * scale``;
* ``softcap``: then ``softcap * tanh(score / softcap)``;
* ``bias``: q, k and v have biases (``<tensor>.b``), added in the projection;
* ``position``: a position part whose rotation (neighbouring pairs, angles in
  fp32 in the kernel) turns the first dimensions of every q and k head;
* ``sink``: the softmax's denominator holds one more term ``exp(sink)`` that
  belongs to no key and has no value (0.0: "one added to the denominator");
* ``values`` "keys": there is no value projection, the values are the keys
  as projected, before their norm;
* ``gate``: head h's output is multiplied by ``sigmoid(W_g x)_h`` (``g``
  [heads, hidden]) before the output projection; ``out_bias``: that
  projection has a bias (``o.b``);
* ``chunk``: a query at position p sees only the keys from ``p - p % chunk`` on
  (chunks counted from the sequence's position 0);
* ``maps`` 2 with ``diff``: differential attention.  Every head has two
  queries and every key head two keys (rows laid out head by head as [map 1,
  map 2]), each pair a softmax attention of its own over the same values; with
  ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff`` (tensors of ``dim``
  numbers) the head's output is ``o = a_1 - lambda a_2``, then ``o /
  sqrt(mean(o^2) + eps) * (1 - diff)``;
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


DEFER_ABOVE = 64  # tokens in a step above which a product's split sums are left for its reader to add


class NormedAttention(PagedAttend, Part):
    family = "mixer"
    graph_safe = True
    stores_output = True
    defers_output = True  # forward(..., store=True, defer=True) may hand back its last product's split sums instead of the finished output

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
        self.norm_weight = bool(self.params.get("norm_weight", False))
        self.values_from_keys = str(self.params.get("values", "projected")) == "keys"
        self.gate = bool(self.params.get("gate", False))
        self.out_bias = bool(self.params.get("out_bias", False))
        self.chunk = int(self.params.get("chunk") or 0)
        self.maps = int(self.params.get("maps") or 1)
        self.diff = float(self.params.get("diff") or 0.0)
        self.difference = 0.0  # lambda, made at load
        self.q_weight = self.k_weight = None
        self.position = build_part("position", self.params["position"], rt) if self.params.get("position") is not None else None
        self.rot_dims = int(getattr(self.position, "dims", 0)) if self.position is not None else 0
        if self.position is not None and (not hasattr(self.position, "frequencies") or self.rot_dims > self.dim):
            raise AlofaError("unsupported", "this attention rotates neighbouring pairs only, at most the head's dimensions", f"position={self.params['position']}")
        if min(self.heads, self.kv_heads, self.dim, self.vdim) <= 0 or self.heads % self.kv_heads:
            raise AlofaError("invalid_argument", "kv heads must divide heads, sizes must be positive", f"params={self.params}")
        if self.vdim > 256:
            raise AlofaError("unsupported", "value heads of more than 256 channels", f"vdim={self.vdim}")
        if self.maps not in (1, 2) or (self.maps == 2 and (self.sink_score is not None or self.values_from_keys)):
            raise AlofaError("unsupported", "one or two softmax maps a head; two take neither a sink nor the keys as values", f"params={self.params}")
        if self.values_from_keys and self.dim != self.vdim:
            raise AlofaError("invalid_argument", "keys that are also the values have the values' size", f"dim={self.dim} vdim={self.vdim}")
        if self.chunk < 0 or (self.chunk and self.window):
            raise AlofaError("invalid_argument", "a chunked mask takes a positive size and no window beside it", f"chunk={self.chunk} window={self.window}")
        if self.norm_weight and not self.qk_norm:
            raise AlofaError("invalid_argument", "a norm's weight needs the norm", f"params={self.params}")
        if self.every <= 0 or self.softcap < 0:
            raise AlofaError("invalid_argument", "q_temp_every must be positive and softcap not negative", f"params={self.params}")
        self.q_dim, self.k_dim = self.heads * self.maps * self.dim, self.kv_heads * self.maps * self.dim
        self.v_dim = 0 if self.values_from_keys else self.kv_heads * self.vdim  # columns of the stacked projection
        self.rows = self.q_dim + self.k_dim + self.v_dim + (self.heads if self.gate else 0)  # [q | k | v | gate]
        # the bfloat16 tensor-core kernels take keys and values of one size and as many value heads as key heads: with several maps a
        # head the values are then kept once per map (the every-size kernel reads one value head for all of a key head's maps)
        self.tensor_cores = rt.dtype == torch.bfloat16 and self.dim == self.vdim and ops.attention_bf16_supported(self.dim)
        self.v_copies = self.maps if self.tensor_cores else 1
        self.nh, self.nkv, self.hd = self.heads * self.maps, self.kv_heads * self.maps, self.dim  # what the shared choice of kernels goes by (keys and values alike only)

    def cache_spec(self):
        # a chunk never reaches further back than its own size: the pages behind it are given back like a window's
        value_heads = self.kv_heads * self.v_copies
        return PagedKV(self.kv_heads * self.maps, self.dim, self.chunk or self.window, self.vdim, None if value_heads == self.kv_heads * self.maps else value_heads)

    def scratch_row_bytes(self) -> int:
        return 4 * self.rows + 4 * self.q_dim + 4 * (self.maps + 1) * self.heads * self.vdim + 8 * self.hidden

    def tensors(self):
        pre = self.prefix
        t = {pre + "q": TensorSpec((self.q_dim, self.hidden)), pre + "k": TensorSpec((self.k_dim, self.hidden)), pre + "o": TensorSpec((self.hidden, self.heads * self.vdim))}
        if not self.values_from_keys:
            t[pre + "v"] = TensorSpec((self.v_dim, self.hidden))
        if self.bias:
            t.update({pre + n + ".b": TensorSpec((t[pre + n].shape[0],)) for n in self._stacked()})
        if self.norm_weight:
            t.update({pre + "q.norm": TensorSpec((self.dim,), "ones"), pre + "k.norm": TensorSpec((self.dim,), "ones")})
        if self.gate:
            t[pre + "g"] = TensorSpec((self.heads, self.hidden))
        if self.out_bias:
            t[pre + "o.b"] = TensorSpec((self.hidden,))
        if self.maps == 2:
            t.update({pre + n: TensorSpec((self.dim,)) for n in ("lq1", "lk1", "lq2", "lk2")})
        return t

    def _stacked(self):
        return ("q", "k") if self.values_from_keys else ("q", "k", "v")

    def load(self, state):
        pre = self.prefix
        names = self._stacked()
        weights = [state[pre + n] for n in names] + ([state[pre + "g"]] if self.gate else [])
        b = None
        if self.bias:  # the gate has none
            b = as_float32_vector(torch.cat([state[pre + n + ".b"] for n in names] + ([torch.zeros_like(state[pre + "q.b"][: self.heads])] if self.gate else []), dim=0))
        self.qkv = Linear(torch.cat(weights, dim=0), b, STORE)
        if self.position is not None:
            self.position.load(state)
        dev = state[pre + "o"].device
        if self.sink_score is not None:
            self.sink = torch.full((self.heads,), float(self.sink_score), dtype=torch.float32, device=dev)
        if self.norm_weight:
            self.q_weight, self.k_weight = as_float32_vector(state[pre + "q.norm"]), as_float32_vector(state[pre + "k.norm"])
        if self.maps == 2:  # one number for the layer, in fp32
            lq1, lk1, lq2, lk2 = (state[pre + n].to(torch.float32) for n in ("lq1", "lk1", "lq2", "lk2"))
            self.difference = float((torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum())).item()) + self.diff
        ob = as_float32_vector(state[pre + "o.b"]) if self.out_bias else None
        self.out_add = Linear(state[pre + "o"], ob, RESIDUAL)
        self.out_store = Linear(state[pre + "o"], ob, STORE)

    def forward(self, ctx, x, h, cache, writes=True, store=False, defer=False):
        if not writes:
            raise AlofaError("unsupported", "this attention does not read another run's cache")
        n, dt = x.shape[0], self.rt.dtype
        group = ctx.groups[cache.group]
        sums = ctx.buf((n, self.rows), torch.float32)
        # over prompt portions the kernel below adds the product's split sums up as it reads (1.388 -> 1.368 ms for a 2,048-token prompt of the
        # 1k bench size); in steps of a few tokens the kernel that settles them first measured faster (0.373 against 0.381 ms a step at batch 8)
        owed = self.qkv(sums, x, defer=n > DEFER_ABOVE, buf=ctx.buf)
        q = ctx.buf((n, self.q_dim), dt)
        rotated = self.rot_dims > 0
        g_off = self.q_dim + self.k_dim + self.v_dim  # the gates' column in the stacked projection's sums
        gates, gates_at = (sums, g_off) if self.gate else (None, 0)
        if owed is not None and self.gate:
            gates, gates_at = ctx.buf((n, self.heads), torch.float32), 0  # the gates' logits, finished, for the kernel after the attention
        ops.qkv_prepare(q, cache.k, cache.v, sums if owed is None else owed, ctx.positions, group.slot_map, self.heads, self.kv_heads, self.dim, self.vdim, self.qk_norm,
                        self.eps, self.coef, self.every, self.position.frequencies() if rotated else None, self.rot_dims, self.maps, self.q_weight, self.k_weight,
                        float(getattr(self.position, "magnitude", 1.0)) if rotated else 1.0, self.values_from_keys, self.v_copies,
                        gates if owed is not None and self.gate else None, g_off)
        if self.tensor_cores or (self.dim == self.vdim and self.maps == 1 and not self.chunk):
            out = self.attend(ctx, q, cache, group)  # the tensor-core kernels in bfloat16 for the head sizes they are built for, else the every-size kernel
            if (self.gate or self.maps > 1) and not isinstance(out, torch.Tensor):
                out = out.rows()
            if self.maps > 1:
                a, out = out, ctx.buf((n, self.heads * self.vdim), dt)
                ops.heads_finish(out, a, self.heads, self.kv_heads, self.vdim, self.maps, self.difference, self.eps, 1.0 - self.diff, gates, gates_at)
            elif self.gate:
                ops.head_gate(out, gates, gates_at, self.heads, self.vdim)
        else:
            # the every-size kernel; what is still to be combined or gated stays fp32 until it has been
            plain = self.maps == 1 and not self.gate
            a = ctx.buf((n, self.heads * self.maps * self.vdim), dt if plain else torch.float32)
            ops.paged_attention_generic(a, q, cache.k, cache.v, ctx.positions, ctx.seq_of_token, group.block_table, group.page_size, self.heads * self.maps,
                                        self.kv_heads * self.maps, self.dim, self.window, self.scale, self.softcap, self.vdim, self.sink, self.chunk, self.maps)
            out = a
            if not plain:
                out = ctx.buf((n, self.heads * self.vdim), dt)
                ops.heads_finish(out, a, self.heads, self.kv_heads, self.vdim, self.maps, self.difference, self.eps, 1.0 - self.diff if self.maps == 2 else 1.0,
                                 gates, gates_at)
        if store:
            return self.out_store(h, out, defer=defer, buf=ctx.buf)  # None, or the split sums a caller that asked for them adds up itself
        add_into_stream(ctx, self.out_add, h, out)


register_part("mixer", "normed_attention", NormedAttention)
