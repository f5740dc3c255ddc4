"""Python face of the CUDA kernels.

Each function checks what the kernel cannot check for itself (device, dtype,
contiguity, matching sizes), then launches on the current CUDA stream through
the library's C entry point.  There is no fallback of any kind: tensors that
are not on a CUDA device are refused, and a library that cannot be built or
loaded raises when it is first needed."""
from __future__ import annotations

import ctypes
import os

import torch

from ..errors import AlofaError
from .build import load_library

EPI_STORE, EPI_RESIDUAL, EPI_GATED = 0, 1, 2

_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_libs: dict = {}
_launches = 0  # kernels launched through this module (graph replays add their kernels)


def launch_count() -> int:
    """How many of this package's kernels have been launched so far."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def _generic():
    lib = _libs.get("generic")
    if lib is None:
        lib = load_library("alofa_generic", ["kernels/generic.cu"])
        sigs = {
            "alofa_embed_gather": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P],
            "alofa_rmsnorm": [_P, _P, _P, _P, _I, _I, _F, _I, _P],
            "alofa_gemm_generic": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
            "alofa_rope_store": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
            "alofa_paged_attention_generic": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _F, _P, _I, _I, _I, _I, _P],
        }
        for name, args in sigs.items():
            fn = getattr(lib, name)
            fn.restype = _I
            fn.argtypes = args
        _libs["generic"] = lib
    return lib


def _sampling():
    lib = _libs.get("sampling")
    if lib is None:
        lib = load_library("alofa_sampling", ["kernels/sampling.cu"])
        sigs = {
            "alofa_sample": [_P, _P, _P, _P, _I, _I, _P, _I, _P],
            "alofa_sample_chain": [_P, _P, _P, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P],
        }
        for name, args in sigs.items():
            fn = getattr(lib, name)
            fn.restype = _I
            fn.argtypes = args
        _libs["sampling"] = lib
    return lib


def _gemm_tc():
    lib = _libs.get("gemm_tc")
    if lib is None:
        lib = load_library("alofa_gemm_tc", ["kernels/gemm_tc.cu"])
        lib.alofa_gemm_tc.restype = _I
        lib.alofa_gemm_tc.argtypes = [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _F, _P, _P, _P, _I, _P]
        lib.alofa_splitk_reduce.restype = _I
        lib.alofa_splitk_reduce.argtypes = [_P, _P, _P, _I, _I, _I, _I, _I, _P]
        lib.alofa_gemm_tc_reduces_in_cluster.restype = _I
        lib.alofa_gemm_tc_reduces_in_cluster.argtypes = [_I, _I, _I]
        lib.alofa_gemm_tc_rope.restype = _I
        lib.alofa_gemm_tc_rope.argtypes = [_P, _P, _P, _I, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _F, _P, _P, _P]
        lib.alofa_gemm_tc_rope_resident_clusters.restype = _I
        lib.alofa_gemm_tc_rope_resident_clusters.argtypes = [_I, _I]
        lib.alofa_gemm_tc_splits.restype = _I
        lib.alofa_gemm_tc_splits.argtypes = [_I, _I]
        _libs["gemm_tc"] = lib
    return lib


def _attention(head_dim: int, capped: bool = False):
    """The attention library of one head size; ``capped``: the build whose scores are bounded by softcap * tanh(. / softcap)."""
    key = f"attention_hd{head_dim}" + ("_cap" if capped else "")
    lib = _libs.get(key)
    if lib is None:
        defines = {"HEAD_DIM": head_dim}
        if capped:
            defines["SOFTCAP"] = 1
        lib = load_library(f"alofa_{key}", ["kernels/attention_bf16.cu"], defines=defines)
        lib.alofa_attention_bf16.restype = _I
        lib.alofa_attention_bf16.argtypes = [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P, _I, ctypes.c_longlong, _P, _I, _F, _P, _P]
        lib.alofa_attention_combine.restype = _I
        lib.alofa_attention_combine.argtypes = [_P, _P, _P, _P, _I, _I, _I, _I, _P, _P]
        lib.alofa_attention_decode_wide_warps.restype = _I
        lib.alofa_attention_decode_wide_warps.argtypes = []
        lib.alofa_attention_decode_slots.restype = _I
        lib.alofa_attention_decode_slots.argtypes = [_I, _I]
        _libs[key] = lib
    return lib


_decode_slots = {}


def attention_decode_wide_warps(head_dim: int, capped: bool = False) -> int:
    """Warps of the decode attention kernel's wide form at this head size (one
    CTA per SM; its splits are multiples of 64 keys a warp), 0 when it has none."""
    return _attention(head_dim, capped).alofa_attention_decode_wide_warps()


def attention_decode_slots(head_dim: int, page_size: int, warps: int = 4, capped: bool = False) -> int:
    """How many CTAs of the decode attention kernel with ``warps`` warps (4, or
    the wide form's) the device holds at a time, 0 when that kernel is not
    built for this head size and kind of page (asked once each)."""
    key = (head_dim, page_size % 64 == 0, warps, capped)
    if key not in _decode_slots:
        _decode_slots[key] = max(0, _attention(head_dim, capped).alofa_attention_decode_slots(page_size, warps))
    return _decode_slots[key]


def attention_bf16_supported(head_dim: int) -> bool:
    """Head sizes the bfloat16 attention kernel is built for."""
    return head_dim % 16 == 0 and 16 <= head_dim <= 128


def _elementwise():
    lib = _libs.get("elementwise")
    if lib is None:
        lib = load_library("alofa_elementwise_bf16", ["kernels/elementwise_bf16.cu"])
        lib.alofa_norm_fused.restype = _I
        lib.alofa_norm_fused.argtypes = [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P, _P, _P, _P]
        lib.alofa_stream_settle.restype = _I
        lib.alofa_stream_settle.argtypes = [_P, _P, _P, _P, _I, _P]
        lib.alofa_rope_store_fused.restype = _I
        lib.alofa_rope_store_fused.argtypes = [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]
        _libs["elementwise"] = lib
    return lib


_bound_stream = None  # the stream handle of the step in progress, looked up once per step


def _stream() -> int:
    return _bound_stream if _bound_stream is not None else torch.cuda.current_stream().cuda_stream


class bound_stream:
    """Within the block, every launch of this module goes to the stream that is
    current on entry, without asking torch for it at each launch (the lookup
    costs as much as a launch).  The caller must not switch streams inside."""

    def __enter__(self):
        global _bound_stream
        self._before = _bound_stream
        _bound_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _bound_stream
        _bound_stream = self._before
        return False


def _dev(t: torch.Tensor, name: str, dtype=None) -> int:
    if not t.is_cuda:
        raise AlofaError("unsupported", "kernels run on CUDA tensors only", f"{name} is on {t.device}")
    if not t.is_contiguous():
        raise AlofaError("invalid_argument", "kernel operand must be contiguous", name)
    if dtype is not None and t.dtype != dtype:
        raise AlofaError("invalid_argument", "kernel operand has the wrong dtype", f"{name} is {t.dtype}, want {dtype}")
    return t.data_ptr()


def _is_bf16(t: torch.Tensor, name: str) -> int:
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise AlofaError("unsupported", "kernel operand must be float32 or bfloat16", f"{name} is {t.dtype}")


def _done(rc: int, what: str, detail: str = "") -> None:
    global _launches
    if rc == 0:
        _launches += 1
        return
    if rc == 1:
        raise AlofaError("unsupported", f"{what}: the kernel does not take these sizes", detail)
    raise AlofaError("state", f"{what}: the CUDA runtime refused the launch", detail + " " + str(torch.cuda.get_device_name()))


def embed_gather(out, table, ids, status=None, src=None, fed=None) -> None:
    """out[t] = table[ids[t]] widened to fp32; out [T, H] fp32.  With ``src``
    and ``fed`` (int32 on the device) token t is ``fed[src[t]]`` where
    ``src[t] >= 0``: a token the step before sampled, never seen by the host."""
    n, hidden = out.shape
    _done(
        _generic().alofa_embed_gather(
            _dev(out, "out", torch.float32), _dev(table, "table"), _dev(ids, "ids", torch.int32),
            _dev(src, "src", torch.int32) if src is not None else None, _dev(fed, "fed", torch.int32) if src is not None else None,
            n, hidden, table.shape[0],
            _is_bf16(table, "table"), _dev(status, "status", torch.int32) if status is not None else None, _stream(),
        ),
        "embed_gather",
    )


def rmsnorm(out, x, weight, eps: float, rows=None) -> None:
    """out[r] = rmsnorm(x[rows[r] or r]) * weight; x fp32, weight fp32."""
    n, hidden = out.shape
    if x.shape[-1] != hidden or weight.shape[0] != hidden:
        raise AlofaError("invalid_argument", "rmsnorm sizes disagree", f"out={tuple(out.shape)} x={tuple(x.shape)} w={tuple(weight.shape)}")
    _done(
        _generic().alofa_rmsnorm(
            _dev(out, "out"), _dev(x, "x", torch.float32), _dev(weight, "weight", torch.float32),
            _dev(rows, "rows", torch.int32) if rows is not None else None, n, hidden, float(eps), _is_bf16(out, "out"), _stream(),
        ),
        "rmsnorm",
    )


def gemm_generic(out, x, w, bias, epi: int, act: int = 0) -> None:
    """out = x @ w.T (+bias) with the epilogue ``epi``; any sizes.  ``act``
    (EPI_STORE only): a code of ``ACTIVATIONS`` applied to the fp32 sums."""
    m, k = x.shape
    n = out.shape[1]
    rows_w = 2 * n if epi == EPI_GATED else n
    if w.shape != (rows_w, k) or out.shape[0] != m or (bias is not None and bias.shape[0] != rows_w):
        raise AlofaError("invalid_argument", "gemm sizes disagree", f"out={tuple(out.shape)} x={tuple(x.shape)} w={tuple(w.shape)} epi={epi}")
    _done(
        _generic().alofa_gemm_generic(
            _dev(out, "out"), _dev(x, "x"), _dev(w, "w"), _dev(bias, "bias", torch.float32) if bias is not None else None,
            m, n, k, epi | (act << 4), _is_bf16(x, "x"), _is_bf16(w, "w"), _is_bf16(out, "out"), _stream(),
        ),
        "gemm_generic", f"M={m} N={n} K={k} epi={epi}",
    )


def rope_store(q_out, k_cache, v_cache, qkv, cos_sin, positions, slot_map, nh, nkv, hd, rot, write_cache=True) -> None:
    """Rotate q and k, write k and v into the cache slots of ``slot_map``."""
    n = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd or q_out.shape != (n, nh * hd):
        raise AlofaError("invalid_argument", "rope_store sizes disagree", f"qkv={tuple(qkv.shape)} q_out={tuple(q_out.shape)}")
    if rot and cos_sin.shape[1] * 2 != rot:
        raise AlofaError("invalid_argument", "rotary table does not match rotary_dim", f"table={tuple(cos_sin.shape)} rot={rot}")
    dt = qkv.dtype
    _done(
        _generic().alofa_rope_store(
            _dev(q_out, "q_out", dt), _dev(k_cache, "k_cache", dt) if write_cache else None,
            _dev(v_cache, "v_cache", dt) if write_cache else None, _dev(qkv, "qkv"),
            _dev(cos_sin, "cos_sin", torch.float32) if rot else None, _dev(positions, "positions", torch.int32),
            _dev(slot_map, "slot_map", torch.int32) if write_cache else None, n, nh, nkv, hd, rot, 1 if write_cache else 0,
            _is_bf16(qkv, "qkv"), _stream(),
        ),
        "rope_store", f"hd={hd} rot={rot}",
    )


def paged_attention_generic(out, q, k_cache, v_cache, positions, seq_of_token, block_table, page_size, nh, nkv, hd, window, scale, softcap: float = 0.0, vd=None, sink=None,
                            chunk: int = 0, v_share: int = 1) -> None:
    """Causal grouped-query attention over the paged cache for every size and
    both dtypes; fp32 scores and softmax.  ``softcap`` > 0 bounds the scaled
    scores by ``softcap * tanh(score / softcap)``; ``vd`` is the values' head
    size when it differs from the keys' ``hd``; ``sink`` (fp32, one score per
    head) adds ``exp(sink[h])`` to the softmax's denominator, a term that
    belongs to no key and has no value.  ``chunk`` > 0: a query at position p
    sees only the keys from ``p - p % chunk`` on.  ``v_share``: so many
    neighbouring key heads read one value head (the value cache has ``nkv /
    v_share`` heads).  ``out`` may be fp32 while q and the caches are
    bfloat16."""
    n = q.shape[0]
    vd = hd if vd is None else vd
    dt = q.dtype
    if (tuple(k_cache.shape[1:]) != (nkv, hd) or nkv % v_share or tuple(v_cache.shape[1:]) != (nkv // v_share, vd) or tuple(q.shape) != (n, nh * hd)
            or tuple(out.shape) != (n, nh * vd) or out.dtype not in (dt, torch.float32)):
        raise AlofaError("invalid_argument", "attention sizes disagree", f"q={tuple(q.shape)} out={tuple(out.shape)} k={tuple(k_cache.shape)} v={tuple(v_cache.shape)}")
    _done(
        _generic().alofa_paged_attention_generic(
            _dev(out, "out"), _dev(q, "q"), _dev(k_cache, "k_cache", dt), _dev(v_cache, "v_cache", dt),
            _dev(positions, "positions", torch.int32), _dev(seq_of_token, "seq_of_token", torch.int32), _dev(block_table, "block_table", torch.int32),
            block_table.shape[1], page_size, n, nh, nkv, hd, vd, int(window or 0), float(scale), float(softcap or 0.0),
            _dev(sink, "sink", torch.float32) if sink is not None else None, _is_bf16(q, "q"), int(chunk or 0), int(v_share), 1 if out.dtype == torch.float32 else 0, _stream(),
        ),
        "paged_attention_generic", f"heads={nh} kv_heads={nkv} head_dim={hd} v_head_dim={vd}",
    )


ARGMAX_PARTS = 32


def sample(tokens, logits, temperature, uniform, scratch=None, any_hot: bool = True) -> None:
    """tokens[r] = argmax (temperature 0) or inverse-CDF draw of softmax(x/T).
    With ``scratch`` (fp32, 2 * rows * ARGMAX_PARTS words) greedy rows are found
    in two stages over many blocks; ``any_hot`` False promises that no row has a
    positive temperature, so the draw kernel is not launched at all."""
    n, vocab = logits.shape
    if scratch is not None and scratch.numel() < 2 * n * ARGMAX_PARTS:
        raise AlofaError("invalid_argument", "sample scratch is too small", f"have={scratch.numel()} need={2 * n * ARGMAX_PARTS}")
    _done(
        _sampling().alofa_sample(
            _dev(tokens, "tokens", torch.int32), _dev(logits, "logits", torch.float32),
            _dev(temperature, "temperature", torch.float32) if temperature is not None else None,
            _dev(uniform, "uniform", torch.float32) if uniform is not None else None, n, vocab,
            _dev(scratch, "scratch", torch.float32) if scratch is not None else None, 1 if any_hot else 0, _stream(),
        ),
        "sample",
    )
    if scratch is not None:
        count_launches(2 if any_hot else 1)


def sample_chain(tokens, logits, work, fparams, iparams, bias_start, bias_index, bias_value, hist_start, hist_token, hist_count) -> None:
    """The whole sampling chain per row (bias, penalties, temperature, top-k,
    top-p, min-p, draw); ``work`` is fp32 scratch of the logits' shape."""
    n, vocab = logits.shape
    if work.shape != logits.shape or fparams.shape != (n, 8) or iparams.shape != (n, 4):
        raise AlofaError("invalid_argument", "sample_chain sizes disagree", f"logits={tuple(logits.shape)} work={tuple(work.shape)}")
    f32, i32 = torch.float32, torch.int32
    _done(
        _sampling().alofa_sample_chain(
            _dev(tokens, "tokens", i32), _dev(logits, "logits", f32), _dev(work, "work", f32), n, vocab,
            _dev(fparams, "fparams", f32), _dev(iparams, "iparams", i32), _dev(bias_start, "bias_start", i32),
            _dev(bias_index, "bias_index", i32), _dev(bias_value, "bias_value", f32), _dev(hist_start, "hist_start", i32),
            _dev(hist_token, "hist_token", i32), _dev(hist_count, "hist_count", i32), _stream(),
        ),
        "sample_chain", f"vocab={vocab}",
    )


_rope_clusters = {}


def gemm_tc_rope_splits(m_tiles: int, normed: bool, most: int = 8) -> int:
    """The largest depth split (a cluster of that many CTAs per 128-row tile)
    of the q/k/v kernel for which all ``m_tiles`` clusters are resident
    together: a GPC holds whole clusters only, so the answer comes from the
    runtime's occupancy of clusters, asked once per size."""
    for splits in range(most, 1, -1):
        key = (splits, bool(normed))
        if key not in _rope_clusters:
            _rope_clusters[key] = _gemm_tc().alofa_gemm_tc_rope_resident_clusters(splits, 1 if normed else 0)
        if _rope_clusters[key] >= m_tiles:
            return splits
    return 1


def gemm_tc_splits(k: int, splits: int) -> int:
    """The number of k-splits gemm_tc really uses for depth ``k``."""
    return _gemm_tc().alofa_gemm_tc_splits(k, splits)


B_ROWS, B_MERGED_SPLITS, B_NORMED = 0, 1, 2


def gemm_tc(out, x, w, bias, epi: int, bn: int, splits: int = 1, partial=None, status=None, reduce: bool = True, computed=None, acc=None, act: int = 0,
            tile_batch=None, batches: int = 1) -> bool:
    """Tensor-core product ``out = x @ w.T`` (bf16 operands, fp32 sums) with
    the epilogue fused.  Returns False, having launched nothing, when the
    kernel does not take these sizes (depth not a multiple of 8, unaligned).

    ``computed`` (residual products with ``bn`` = 16 only) replaces ``x`` by
    rows the kernel makes as it goes: ``(B_MERGED_SPLITS, partial_o,
    partial_ml, positions, heads, head_dim, window, split_keys)``, the
    attention output of decode tokens whose key splits are not merged yet; or,
    for gated products, ``(B_NORMED, base, acc or None, gamma, eps, new_base,
    zero or None)``: the RMSNorm of the residual stream ``base + acc``, which
    is also written to ``new_base`` while ``zero`` is cleared.

    ``acc`` (residual products, weights on M): the sums are added into this
    int64 accumulator ``[tokens, features]`` (units of 2^-32) with atomic adds
    instead of into ``out``; nothing else is written.

    ``act`` (EPI_STORE only): a code of ``ACTIVATIONS`` applied to the fp32
    sums plus bias before they are stored.

    ``tile_batch`` (int32 on the device; tokens on M, EPI_STORE or EPI_GATED,
    no bias): ``w`` is [batches * N, K] (gated: [batches * 2N, K], a batch's
    gate rows before its up rows) and the i-th tile of 128 token rows multiplies
    by the rows of batch ``tile_batch[i]``; a negative entry skips the tile."""
    n = out.shape[1]
    rows_w = (2 * n if epi == EPI_GATED else n) * (batches if tile_batch is not None else 1)
    k = w.shape[1]
    m = out.shape[0]
    if w.shape[0] != rows_w or (x is not None and tuple(x.shape) != (m, k)) or (bias is not None and bias.shape[0] != rows_w):
        raise AlofaError("invalid_argument", "gemm sizes disagree", f"out={tuple(out.shape)} w={tuple(w.shape)} epi={epi}")
    f32, i64 = torch.float32, torch.int64
    b_kind, b_src, b_ml, b_pos, heads, hd, window, split_keys = B_ROWS, None, None, None, 0, 0, 0, 0
    n_acc = n_gamma = n_out = n_zero = None
    n_eps = 0.0
    if computed is not None and computed[0] == B_NORMED:
        b_kind, base, acc_in, gamma, n_eps, new_base, zero = computed
        if tuple(base.shape) != (m, k) or tuple(new_base.shape) != (m, k) or gamma.shape[0] != k:
            raise AlofaError("invalid_argument", "normed operand sizes disagree", f"base={tuple(base.shape)} gamma={tuple(gamma.shape)} k={k}")
        b_src, n_gamma, n_out = _dev(base, "base", f32), _dev(gamma, "gamma", f32), _dev(new_base, "new_base", f32)
        n_acc = _dev(acc_in, "acc", i64) if acc_in is not None else None
        n_zero = _dev(zero, "zero", i64) if zero is not None else None
    elif computed is not None:
        b_kind, po, pml, positions, heads, hd, window, split_keys = computed
        b_src, b_ml, b_pos, window = _dev(po, "partial_o", f32), _dev(pml, "partial_ml", f32), _dev(positions, "positions", torch.int32), int(window or 0)
    elif x is None:
        raise AlofaError("invalid_argument", "gemm without a token operand")
    rc = _gemm_tc().alofa_gemm_tc(
        _dev(out, "out"), _dev(x, "x", torch.bfloat16) if x is not None else None, _dev(w, "w", torch.bfloat16),
        _dev(bias, "bias", f32) if bias is not None else None,
        _dev(partial, "partial", f32) if partial is not None else None,
        m, n, k, epi | (act << 4), _is_bf16(out, "out"), bn, splits, 1 if reduce else 0,
        _dev(status, "status", torch.int32) if status is not None else None,
        b_kind, b_src, b_ml, b_pos, heads, hd, window, split_keys,
        _dev(acc, "acc", i64) if acc is not None else None, n_acc, n_gamma, float(n_eps), n_out, n_zero,
        _dev(tile_batch, "tile_batch", torch.int32) if tile_batch is not None else None, batches, _stream(),
    )
    if rc == 1:
        return False
    _done(rc, "gemm_tc", f"M={m} N={n} K={k} epi={epi} bn={bn} splits={splits}")
    if splits > 1 and reduce and acc is None and b_kind != B_NORMED and not _gemm_tc().alofa_gemm_tc_reduces_in_cluster(epi, bn, splits):
        count_launches(1)  # the kernel that adds the split sums up
    return True


def gemm_tc_rope(x, w, bias, q_out, k_cache, v_cache, slot_map, positions, cos_sin, nh: int, nkv: int, hd: int, splits: int, status=None, normed=None) -> bool:
    """q/k/v of up to 16 tokens in one kernel: ``x @ w.T + bias`` for the
    stacked weight [q; k; v] (``nkv`` = 0: q only), q and k rotated, q to
    ``q_out``, k and v to their cache slots.  With ``normed`` = ``(base, acc or
    None, gamma, eps, new_base, zero or None)`` the operand is not ``x`` (None
    then) but the RMSNorm of the residual stream ``base + acc``, made in the
    kernel; the stream is also written to ``new_base`` and ``zero`` cleared.
    False, having launched nothing, when the kernel does not take these sizes."""
    bf, f32, i64 = torch.bfloat16, torch.float32, torch.int64
    t, k = (x.shape if normed is None else normed[0].shape)
    if t > 16 or 128 % hd or w.shape != ((nh + 2 * nkv) * hd, k):
        return False
    n_base = n_acc = n_gamma = n_out = n_zero = None
    n_eps = 0.0
    if normed is not None:
        base, acc_in, gamma, n_eps, new_base, zero = normed
        if tuple(new_base.shape) != (t, k) or gamma.shape[0] != k:
            raise AlofaError("invalid_argument", "normed operand sizes disagree", f"base={tuple(base.shape)} gamma={tuple(gamma.shape)}")
        n_base, n_gamma, n_out = _dev(base, "base", f32), _dev(gamma, "gamma", f32), _dev(new_base, "new_base", f32)
        n_acc = _dev(acc_in, "acc", i64) if acc_in is not None else None
        n_zero = _dev(zero, "zero", i64) if zero is not None else None
    rc = _gemm_tc().alofa_gemm_tc_rope(
        _dev(x, "x", bf) if x is not None else None, _dev(w, "w", bf), _dev(bias, "bias", f32) if bias is not None else None, t, k, _dev(q_out, "q_out", bf),
        _dev(k_cache, "k_cache", bf) if nkv else None, _dev(v_cache, "v_cache", bf) if nkv else None,
        _dev(slot_map, "slot_map", torch.int32) if nkv else None, _dev(positions, "positions", torch.int32), _dev(cos_sin, "cos_sin", f32),
        nh, nkv, hd, splits, _dev(status, "status", torch.int32) if status is not None else None,
        n_base, n_acc, n_gamma, float(n_eps), n_out, n_zero, _stream(),
    )
    if rc == 1:
        return False
    _done(rc, "gemm_tc_rope", f"T={t} K={k} heads={nh}+2x{nkv} hd={hd}")
    return True


def attention_bf16(out, q, k_cache, v_cache, q_start, kv_len, positions, block_table, page_size, n_seqs, max_q_len, nh, nkv, hd, window, scale,
                   n_splits: int = 0, split_keys: int = 0, partial_o=None, partial_ml=None, max_kv_len: int = 0, status=None, combine: bool = True, softcap: float = 0.0, sink=None) -> None:
    """Causal GQA over the paged bf16 cache for a step's requests; with
    ``n_splits`` > 0 the keys of each request (decode tokens) or of each query
    tile (prompt portions) are split over several CTAs and merged - unless
    ``combine`` is False (decode tokens only): then ``partial_o`` / ``partial_ml``
    keep the splits for :func:`attention_combine` or a product that merges them.
    ``softcap`` > 0 (the library built for it): scaled scores are bounded by
    ``softcap * tanh(score / softcap)``.  ``sink`` [nh] fp32: one more term
    ``exp(sink[h])`` of every row's denominator (merged splits only)."""
    n = q.shape[0]
    bf = torch.bfloat16
    g = nh // nkv
    tiles = -(-(max_q_len * g) // 64)
    rc = _attention(hd, softcap > 0).alofa_attention_bf16(
        _dev(out, "out", bf), _dev(q, "q", bf), _dev(k_cache, "k_cache", bf), _dev(v_cache, "v_cache", bf),
        _dev(q_start, "q_start", torch.int32), _dev(kv_len, "kv_len", torch.int32), _dev(positions, "positions", torch.int32),
        _dev(block_table, "block_table", torch.int32),
        block_table.shape[1], page_size, n_seqs, n, tiles, nh, nkv, int(window or 0), float(scale), n_splits, split_keys,
        _dev(partial_o, "partial_o", torch.float32) if partial_o is not None else None,
        _dev(partial_ml, "partial_ml", torch.float32) if partial_ml is not None else None,
        int(max_kv_len) if max_kv_len else block_table.shape[1] * page_size, k_cache.shape[0],
        _dev(status, "status", torch.int32) if status is not None else None, 1 if combine else 0, float(softcap or 0.0),
        _dev(sink, "sink", torch.float32) if sink is not None else None, _stream(),
    )
    _done(rc, "attention_bf16", f"hd={hd} nh={nh} nkv={nkv} splits={n_splits}")
    if n_splits > 1 and combine:
        count_launches(1)


def attention_combine(out, partial_o, partial_ml, positions, nh: int, hd: int, window, split_keys: int, sink=None, capped: bool = False) -> None:
    """Merge the key splits of decode tokens: out [T, nh * hd] bf16.  ``capped``:
    take the kernel from the library built for capped scores (the one the
    splits came from), so that no second library is built for it."""
    rc = _attention(hd, capped).alofa_attention_combine(
        _dev(out, "out", torch.bfloat16), _dev(partial_o, "partial_o", torch.float32), _dev(partial_ml, "partial_ml", torch.float32),
        _dev(positions, "positions", torch.int32), out.shape[0], nh, int(window or 0), split_keys,
        _dev(sink, "sink", torch.float32) if sink is not None else None, _stream(),
    )
    _done(rc, "attention_combine")


def norm_fused(out, h, weight, eps: float, rows=None, partial=None, splits: int = 0, bias=None, base=None, acc=None, other=None) -> bool:
    """RMSNorm of rows of the fp32 stream ``h`` (vectorised; hidden % 4 == 0).
    With ``partial`` [splits, T, hidden] the pending partial sums (and bias)
    are first added into ``h``.  With ``base`` the stream's values are read
    from there (``h`` is written, complete), with ``acc`` (int64, units of
    2^-32; every row, ``rows`` None) that accumulator is added on top and left
    zero, as is ``other``.  Returns False when the size is not taken."""
    n, hidden = out.shape
    if hidden % 4:
        return False
    f32, i64 = torch.float32, torch.int64
    rc = _elementwise().alofa_norm_fused(
        _dev(out, "out"), _dev(h, "h", f32), _dev(weight, "weight", f32), _dev(partial, "partial", f32) if partial is not None else None,
        _dev(bias, "bias", f32) if bias is not None else None, _dev(rows, "rows", torch.int32) if rows is not None else None,
        n, h.shape[0], hidden, splits, float(eps), _is_bf16(out, "out"),
        _dev(base, "base", f32) if base is not None else None, _dev(acc, "acc", i64) if acc is not None else None,
        _dev(other, "other", i64) if other is not None else None, _stream(),
    )
    if rc == 1:
        return False
    _done(rc, "norm_fused")
    return True


def stream_settle(h, base, acc, other=None) -> None:
    """``h = base + acc`` (the residual stream of a small decode step brought
    back to one fp32 tensor); ``acc`` and ``other`` (int64, units of 2^-32) are
    left zero."""
    f32, i64 = torch.float32, torch.int64
    _done(
        _elementwise().alofa_stream_settle(_dev(h, "h", f32), _dev(base, "base", f32), _dev(acc, "acc", i64),
                                           _dev(other, "other", i64) if other is not None else None, h.numel(), _stream()),
        "stream_settle",
    )


def rope_store_fused(q_out, k_cache, v_cache, qkv, partial, splits, bias, cos_sin, positions, slot_map, nh, nkv, hd, write_cache=True) -> None:
    """bf16 rotate-and-store with full rotary (rot == hd, hd % 16 == 0); the
    source is ``qkv`` (bf16) or split-K ``partial`` sums [splits, T, C] + bias."""
    n = q_out.shape[0]
    bf, f32 = torch.bfloat16, torch.float32
    _done(
        _elementwise().alofa_rope_store_fused(
            _dev(q_out, "q_out", bf), _dev(k_cache, "k_cache", bf) if write_cache else None, _dev(v_cache, "v_cache", bf) if write_cache else None,
            _dev(qkv, "qkv", bf) if qkv is not None else None, _dev(partial, "partial", f32) if partial is not None else None,
            _dev(bias, "bias", f32) if bias is not None else None, _dev(cos_sin, "cos_sin", f32), _dev(positions, "positions", torch.int32),
            _dev(slot_map, "slot_map", torch.int32) if write_cache else None, n, nh, nkv, hd, splits, 1 if write_cache else 0, _stream(),
        ),
        "rope_store_fused", f"hd={hd}",
    )


def splitk_reduce(out, partial, bias, splits: int, epi: int) -> None:
    """out (op)= bias + sum of ``partial`` [splits, T, N] in split order."""
    t, n = out.shape
    _done(
        _gemm_tc().alofa_splitk_reduce(
            _dev(out, "out"), _dev(partial, "partial", torch.float32), _dev(bias, "bias", torch.float32) if bias is not None else None,
            t, n, splits, epi, _is_bf16(out, "out"), _stream(),
        ),
        "splitk_reduce",
    )


# -- latent attention, sandwich norms, routed feed-forwards -------------------------------------------
ACTIVATIONS = {"none": 0, "gelu_erf": 1, "gelu_tanh": 2, "silu": 3, "relu": 4, "relu_squared": 5}
_L = ctypes.c_longlong


def _latent():
    lib = _libs.get("latent")
    if lib is None:
        lib = load_library("alofa_latent", ["kernels/latent.cu", "kernels/gemm_batched_bf16.cu"])
        sigs = {
            "alofa_latent_prepare": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _F, _I, _P],
            "alofa_latent_query_turn": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P],
            "alofa_rotary_interleaved": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
            "alofa_gemm_batched": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _L, _L, _L, _L, _I, _I, _I, _I, _I, _P],
            "alofa_gemm_batched_bf16": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _L, _L, _L, _L, _I, _I, _I, _P],
            "alofa_activate": [_P, _P, _P, _L, _I, _I, _I, _P],
            "alofa_latent_attention": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P],
            "alofa_sandwich_norm": [_P, _P, _P, _F, _P, _P, _F, _I, _I, _I, _I, _L, _P, _P],
            "alofa_concat_rows": [_P, _P, _P, _I, _I, _I, _P],
            "alofa_moe_route": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
            "alofa_moe_router": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _F, _I, _I, _F, _P],
            "alofa_cast_rows": [_P, _P, _L, _I, _P],
            "alofa_moe_sort": [_P, _P, _P, _I, _I, _I, _I, _P],
            "alofa_moe_scatter": [_P, _P, _P, _P, _I, _I, _I, _I, _P],
            "alofa_moe_combine": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _I, _I, _P],
            "alofa_gate_up": [_P, _P, _L, _I, _I, _P],
        }
        for name, args in sigs.items():
            fn = getattr(lib, name)
            fn.restype = _I
            fn.argtypes = args
        _libs["latent"] = lib
    return lib


def latent_prepare(cq, cache_rows, lat, wq, wkv, freq, positions, slot_map, q_rank: int, kv_rank: int, rot: int, rot_dims: int, eps: float,
                   halves: bool = False, mag: float = 1.0) -> None:
    """From the stacked down-projection ``lat`` [T, >= q_rank + kv_rank + rot]
    (fp32; further columns are not read): ``cq`` = RMSNorm of the first part
    (``q_rank`` 0: there is none, ``cq`` and ``wq`` are None); the cache row of
    each token = [RMSNorm of the second part | the third part, its first
    ``rot_dims`` numbers turned by the token's position: neighbouring pairs, or
    with ``halves`` number i with number i + rot_dims / 2; cosine and sine
    times ``mag``].  ``cache_rows`` None: no write."""
    f32 = torch.float32
    n = lat.shape[0]
    if lat.shape[1] < q_rank + kv_rank + rot or (q_rank and tuple(cq.shape) != (n, q_rank)) or (cache_rows is not None and cache_rows.shape[1] != kv_rank + rot):
        raise AlofaError("invalid_argument", "latent_prepare sizes disagree", f"lat={tuple(lat.shape)} q_rank={q_rank} kv_rank={kv_rank} rot={rot}")
    if q_rank == 0 and cache_rows is None:
        return
    dt = cq.dtype if q_rank else cache_rows.dtype
    _done(
        _latent().alofa_latent_prepare(
            _dev(cq, "cq") if q_rank else None, _dev(cache_rows, "cache", dt) if cache_rows is not None else None, _dev(lat, "lat", f32),
            _dev(wq, "wq", f32) if q_rank else None,
            _dev(wkv, "wkv", f32), _dev(freq, "freq", f32) if rot_dims else None, _dev(positions, "positions", torch.int32),
            _dev(slot_map, "slot_map", torch.int32) if cache_rows is not None else None, n, q_rank, kv_rank, rot, rot_dims, float(eps), lat.shape[1],
            1 if halves else 0, float(mag), 1 if dt == torch.bfloat16 else 0, _stream(),
        ),
        "latent_prepare",
    )


def latent_query_turn(qa, q, freq, positions, heads: int, dim: int, rot: int, rot_dims: int, kv_rank: int, halves: bool = False, mag: float = 1.0) -> None:
    """The rotated part of q [T, heads * (dim + rot)] turned by position into
    columns ``kv_rank``.. of qa [T, heads * (kv_rank + rot)]; ``halves`` and
    ``mag`` as in :func:`latent_prepare`."""
    n = q.shape[0]
    if q.shape[1] != heads * (dim + rot) or tuple(qa.shape) != (n, heads * (kv_rank + rot)):
        raise AlofaError("invalid_argument", "latent_query_turn sizes disagree", f"q={tuple(q.shape)} qa={tuple(qa.shape)}")
    if rot == 0:
        return
    _done(
        _latent().alofa_latent_query_turn(_dev(qa, "qa", q.dtype), _dev(q, "q"), _dev(freq, "freq", torch.float32) if rot_dims else None,
                                          _dev(positions, "positions", torch.int32), n, heads, dim, rot, rot_dims, kv_rank, 1 if halves else 0, float(mag),
                                          _is_bf16(q, "q"), _stream()),
        "latent_query_turn",
    )


def rotary_interleaved(x, freq, positions, heads: int, hd: int, rot_dims: int) -> None:
    """Turn the pairs (2i, 2i+1), i < rot_dims / 2, of every head of the view
    ``x`` [T, heads, hd] (unit stride inside a row) in place."""
    if x.shape[0] == 0 or heads == 0 or rot_dims == 0:
        return
    if not x.is_cuda or x.stride(2) != 1 or x.stride(1) != hd:
        raise AlofaError("invalid_argument", "rotary_interleaved wants heads packed in rows", f"strides={x.stride()}")
    _done(
        _latent().alofa_rotary_interleaved(x.data_ptr(), _dev(freq, "freq", torch.float32), _dev(positions, "positions", torch.int32), x.shape[0], heads, hd,
                                           x.stride(0), rot_dims, _is_bf16(x, "x"), _stream()),
        "rotary_interleaved",
    )


def gemm_batched(out, x, w, batches: int, m: int, n: int, k: int, ldx: int, x_batch: int, ldw: int, w_batch: int, ldo: int, out_batch: int,
                 bias=None, bias_batch: int = 0, act: str = "none", tile_batch=None, tile_rows: int = 64) -> None:
    """``out_b[m, n] = act(x_b[m, :] . w_b[n, :] + bias_b[n])`` for every batch
    b, operands addressed by row and batch strides (in elements) from the
    tensors' first elements.  With ``tile_batch`` (int32, one entry per tile of
    ``tile_rows`` rows, a multiple of 64) there is one x and one out and tile i
    uses the weight of batch ``tile_batch[i]``; negative entries are skipped.  bfloat16 operands whose
    depth and strides are multiples of 8 go to the tensor-core kernel, all
    others to the one that takes every size."""
    for t, name in ((out, "out"), (x, "x"), (w, "w")):
        if not t.is_cuda:
            raise AlofaError("unsupported", "kernels run on CUDA tensors only", f"{name} is on {t.device}")
    bf = torch.bfloat16
    if (x.dtype == bf and w.dtype == bf and not (k % 8 or ldx % 8 or ldw % 8 or x_batch % 8 or w_batch % 8 or x.data_ptr() % 16 or w.data_ptr() % 16)
            and os.environ.get("ALOFA_BATCHED_TC", "1") != "0"):
        _done(
            _latent().alofa_gemm_batched_bf16(
                out.data_ptr(), x.data_ptr(), w.data_ptr(), _dev(bias, "bias", torch.float32) if bias is not None else None,
                _dev(tile_batch, "tile_batch", torch.int32) if tile_batch is not None else None, batches, m, n, k, ldx, x_batch, ldw, w_batch, ldo, out_batch,
                bias_batch, ACTIVATIONS[act], tile_rows, _is_bf16(out, "out"), _stream(),
            ),
            "gemm_batched_bf16", f"batches={batches} M={m} N={n} K={k}",
        )
        return
    _done(
        _latent().alofa_gemm_batched(
            out.data_ptr(), x.data_ptr(), w.data_ptr(), _dev(bias, "bias", torch.float32) if bias is not None else None,
            _dev(tile_batch, "tile_batch", torch.int32) if tile_batch is not None else None, batches, m, n, k, ldx, x_batch, ldw, w_batch, ldo, out_batch,
            bias_batch, ACTIVATIONS[act], tile_rows, _is_bf16(x, "x"), _is_bf16(w, "w"), _is_bf16(out, "out"), _stream(),
        ),
        "gemm_batched", f"batches={batches} M={m} N={n} K={k}",
    )


def activate(out, x, bias, act: str) -> None:
    """out = act(x + bias): x fp32 [rows, n], out in its own dtype."""
    rows, n = x.shape
    _done(_latent().alofa_activate(_dev(out, "out"), _dev(x, "x", torch.float32), _dev(bias, "bias", torch.float32) if bias is not None else None,
                                   rows, n, ACTIVATIONS[act], _is_bf16(out, "out"), _stream()), "activate")


def latent_attention(out, qa, cache_rows, sink, positions, seq_of_token, block_table, page_size: int, heads: int, kv_rank: int, rot: int, window, scale: float) -> None:
    """Causal attention of absorbed queries qa [T, heads * (kv_rank + rot)]
    over the paged rows [c | kr]; out [T, heads * kv_rank] = sum_j p_j c_j,
    softmax in fp32 with ``exp(sink[h])`` (fp32 [heads], or None) as one more
    term of the denominator."""
    n = qa.shape[0]
    if qa.shape[1] != heads * (kv_rank + rot) or tuple(out.shape) != (n, heads * kv_rank) or cache_rows.shape[1] != kv_rank + rot:
        raise AlofaError("invalid_argument", "latent_attention sizes disagree", f"qa={tuple(qa.shape)} out={tuple(out.shape)} cache={tuple(cache_rows.shape)}")
    dt = qa.dtype
    _done(
        _latent().alofa_latent_attention(
            _dev(out, "out", dt), _dev(qa, "qa"), _dev(cache_rows, "cache", dt), _dev(sink, "sink", torch.float32) if sink is not None else None,
            _dev(positions, "positions", torch.int32), _dev(seq_of_token, "seq_of_token", torch.int32), _dev(block_table, "block_table", torch.int32),
            block_table.shape[1], page_size, n, heads, kv_rank, rot, int(window or 0), float(scale), _is_bf16(qa, "qa"), _stream(),
        ),
        "latent_attention", f"heads={heads} kv_rank={kv_rank} rot={rot}",
    )


def sandwich_norm(h, y, w_post, eps_post: float, x=None, w_next=None, eps_next: float = 0.0) -> None:
    """``h += rmsnorm(y) * w_post`` (fp32 stream); with ``x`` also ``x =
    rmsnorm(h) * w_next`` of the updated rows (without ``w_next``: the updated
    rows themselves), in x's dtype.  ``y`` is the sublayer's output [rows,
    hidden] fp32, or the partial sums a product left owed (``.sums`` [splits,
    rows, hidden], ``.splits``, ``.bias``): they are added here, in split
    order, as the kernel that settles them would have."""
    rows, hidden = h.shape
    f32 = torch.float32
    splits, plane, bias = 0, 0, None
    if not isinstance(y, torch.Tensor):
        splits, bias, y = int(y.splits), y.bias, y.sums
        if tuple(y.shape) != (splits, rows, hidden):
            raise AlofaError("invalid_argument", "sandwich_norm: owed sums disagree with the stream", f"h={tuple(h.shape)} sums={tuple(y.shape)}")
        plane = rows * hidden
    elif tuple(y.shape) != (rows, hidden):
        raise AlofaError("invalid_argument", "sandwich_norm sizes disagree", f"h={tuple(h.shape)} y={tuple(y.shape)}")
    if x is not None and tuple(x.shape) != (rows, hidden):
        raise AlofaError("invalid_argument", "sandwich_norm sizes disagree", f"h={tuple(h.shape)} x={tuple(x.shape)}")
    _done(
        _latent().alofa_sandwich_norm(_dev(h, "h", f32), _dev(y, "y", f32), _dev(w_post, "w_post", f32), float(eps_post), _dev(x, "x") if x is not None else None,
                                      _dev(w_next, "w_next", f32) if x is not None and w_next is not None else None, float(eps_next), rows, hidden,
                                      _is_bf16(x, "x") if x is not None else 0, splits, plane, _dev(bias, "bias", f32) if bias is not None else None, _stream()),
        "sandwich_norm",
    )


def cast_rows(out, a) -> None:
    """out = a (fp32) in out's dtype, same shape."""
    if out.shape != a.shape:
        raise AlofaError("invalid_argument", "cast_rows sizes disagree", f"out={tuple(out.shape)} a={tuple(a.shape)}")
    _done(_latent().alofa_cast_rows(_dev(out, "out"), _dev(a, "a", torch.float32), out.numel(), _is_bf16(out, "out"), _stream()), "cast_rows")


def concat_rows(out, a, b) -> None:
    """out [T, 2 * hidden] = [a | b] from two fp32 matrices, in out's dtype."""
    rows, hidden = a.shape
    if tuple(b.shape) != (rows, hidden) or tuple(out.shape) != (rows, 2 * hidden):
        raise AlofaError("invalid_argument", "concat_rows sizes disagree", f"a={tuple(a.shape)} b={tuple(b.shape)} out={tuple(out.shape)}")
    _done(_latent().alofa_concat_rows(_dev(out, "out"), _dev(a, "a", torch.float32), _dev(b, "b", torch.float32), rows, hidden, _is_bf16(out, "out"), _stream()), "concat_rows")


MOE_TILE = 64  # rows per tile of the sorted matrix: every expert's rows are padded to whole tiles
MOE_TILE_TC = 128  # the same where the tcgen05 product takes the tiles (its token tile)


def gemm_by_tile(out, x, w, tile_batch, tile_rows: int, act: str = "none") -> None:
    """``out[rows of tile i] = act(x[rows of tile i] @ w[tile_batch[i]].T)``: x
    [rows, K], w [batches, N, K], out [rows, N], tiles of ``tile_rows`` rows.
    bfloat16 operands in tiles of 128 rows go to the tcgen05 product with the
    tokens on the M side (the tile's batch is an offset into the stacked
    weight's rows), all else to :func:`gemm_batched`."""
    batches, n, k = w.shape
    rows = x.shape[0]
    if (tile_rows == MOE_TILE_TC and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k % 8 == 0 and rows % 128 == 0
            and os.environ.get("ALOFA_BY_TILE_TC", "1") != "0"):
        wide = -256 if n > 128 else -128
        if gemm_tc(out, x, w.view(batches * n, k), None, EPI_STORE, wide, act=ACTIVATIONS[act], tile_batch=tile_batch, batches=batches):
            return
    gemm_batched(out, x, w, 1, rows, n, k, k, 0, k, n * k, n, 0, act=act, tile_batch=tile_batch, tile_rows=tile_rows)


def gemm_by_tile_gated(out, x, w, tile_batch, tile_rows: int) -> bool:
    """``out[rows of tile i] = silu(x_i @ Wg^T) * (x_i @ Wu^T)`` with ``w``
    [batches, 2N, K] holding each batch's gate rows before its up rows: the
    tcgen05 product with the gated epilogue.  False, having launched nothing,
    for operands it does not take (the caller then multiplies and gates in
    two steps)."""
    batches, n2, k = w.shape
    rows = x.shape[0]
    if (tile_rows != MOE_TILE_TC or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or k % 8 or rows % 128 or n2 % 2
            or os.environ.get("ALOFA_BY_TILE_TC", "1") == "0"):
        return False
    return gemm_tc(out, x, w.view(batches * n2, k), None, EPI_GATED, -256, tile_batch=tile_batch, batches=batches)


def moe_route(choice, weight, gate, z, experts: int, top: int, softmax: bool = False, renormalize: bool = False) -> None:
    """From router logits z [T, experts (+1)] fp32: the ``top`` experts of each
    token by score (sigmoid, or softmax over the experts), their scores as
    weights, and ``gate`` = sigmoid of the last column when given."""
    i32, f32 = torch.int32, torch.float32
    _done(
        _latent().alofa_moe_route(_dev(choice, "choice", i32), _dev(weight, "weight", f32), _dev(gate, "gate", f32) if gate is not None else None, _dev(z, "z", f32),
                                  z.shape[0], experts, top, z.shape[1], 1 if softmax else 0, 1 if renormalize else 0, _stream()),
        "moe_route", f"experts={experts} top={top}",
    )


def moe_router(choice, weight, gate, x, wr, experts: int, top: int, softmax: bool = False, renormalize: bool = False, correction=None,
               renorm_eps: float = 0.0, groups: int = 1, keep: int = 1, route_scale: float = 1.0) -> None:
    """:func:`moe_route` with the router's product in the same kernel: ``x``
    [T, hidden] in the compute dtype, ``wr`` fp32 [experts (+1 with ``gate``),
    hidden]; logits and scores are fp32.  ``correction`` (fp32 [experts]) is
    added to the scores for the choice only, the weights stay the scores;
    ``renorm_eps`` is added to the sum that ``renormalize`` divides by.
    ``groups`` > 1: the experts form that many equal groups of neighbours; a
    group's score is the sum of its two largest choice scores (score +
    correction), and only experts of the ``keep`` best groups can be chosen.
    ``route_scale``: a factor on the weights."""
    i32, f32 = torch.int32, torch.float32
    if wr.shape != (experts + (1 if gate is not None else 0), x.shape[1]) or (correction is not None and correction.shape[0] != experts):
        raise AlofaError("invalid_argument", "router sizes disagree", f"wr={tuple(wr.shape)} x={tuple(x.shape)} experts={experts}")
    _done(
        _latent().alofa_moe_router(_dev(choice, "choice", i32), _dev(weight, "weight", f32), _dev(gate, "gate", f32) if gate is not None else None, _dev(x, "x"),
                                   _dev(wr, "wr", f32), x.shape[0], experts, top, x.shape[1], 1 if softmax else 0, 1 if renormalize else 0, _is_bf16(x, "x"),
                                   _dev(correction, "correction", f32) if correction is not None else None, float(renorm_eps), int(groups), int(keep), float(route_scale),
                                   _stream()),
        "moe_router", f"experts={experts} top={top} groups={groups} keep={keep}",
    )


def moe_sort(dest, tile_expert, choice, experts: int, tile: int = MOE_TILE) -> None:
    """Rows of the (token, choice) pairs in a matrix sorted by expert, every
    expert padded to whole tiles: ``dest`` [pairs], ``tile_expert`` [tiles]."""
    i32 = torch.int32
    _done(_latent().alofa_moe_sort(_dev(dest, "dest", i32), _dev(tile_expert, "tile_expert", i32), _dev(choice, "choice", i32), choice.numel(), experts, tile,
                                   tile_expert.numel(), _stream()), "moe_sort")


def moe_scatter(xs, x, weight, dest, top: int) -> None:
    """xs[dest[t, k]] = x[t] (times weight[t, k] when given)."""
    _done(_latent().alofa_moe_scatter(_dev(xs, "xs", x.dtype), _dev(x, "x"), _dev(weight, "weight", torch.float32) if weight is not None else None,
                                      _dev(dest, "dest", torch.int32), dest.numel(), top, x.shape[1], _is_bf16(x, "x"), _stream()), "moe_scatter")


def moe_combine(y, ys, dest, weight, shared, gate, top: int, x=None, add: bool = False) -> None:
    """y[t] = sum_k (weight[t, k] *) ys[dest[t, k]] + (gate[t] *) shared[t], fp32;
    a pair whose ``dest`` is negative (an expert that is the identity) takes
    the token's own input ``x[t]`` instead of a row; ``add``: y += the sum."""
    f32 = torch.float32
    _done(
        _latent().alofa_moe_combine(_dev(y, "y", f32), _dev(ys, "ys", f32), _dev(dest, "dest", torch.int32), _dev(weight, "weight", f32) if weight is not None else None,
                                    _dev(shared, "shared", f32) if shared is not None else None, _dev(gate, "gate", f32) if gate is not None else None,
                                    y.shape[0], top, y.shape[1], _dev(x, "x") if x is not None else None, _is_bf16(x, "x") if x is not None else 0,
                                    1 if add else 0, _stream()),
        "moe_combine",
    )


def gate_up(mid, gu) -> None:
    """mid[r, c] = silu(gu[r, c]) * gu[r, ff + c] for rows of fp32 sums that
    hold gate and up side by side; ``mid`` in its own dtype."""
    rows, ff = mid.shape
    if tuple(gu.shape) != (rows, 2 * ff):
        raise AlofaError("invalid_argument", "gate_up sizes disagree", f"mid={tuple(mid.shape)} gu={tuple(gu.shape)}")
    _done(_latent().alofa_gate_up(_dev(mid, "mid"), _dev(gu, "gu", torch.float32), rows, ff, _is_bf16(mid, "mid"), _stream()), "gate_up")


def latent_attention_bf16_supported(kv_rank: int, rot: int) -> bool:
    """Latent sizes the tensor-core kernel is built for (one library per size,
    compiled at first use): whole 16-column MMA tiles for each half of the
    value columns and for the row width, accumulators that fit the registers,
    tiles that fit shared memory."""
    width = kv_rank + rot
    return kv_rank % 32 == 0 and width % 16 == 0 and 32 <= kv_rank <= 512 and (64 + 3 * 32) * (width + 8) * 2 + 4 * 1280 <= 220 * 1024


def _latent_attention_lib(kv_rank: int, rot: int):
    key = f"latent_attention_kv{kv_rank}_r{rot}"
    lib = _libs.get(key)
    if lib is None:
        lib = load_library(f"alofa_{key}", ["kernels/latent_attention_bf16.cu"], defines={"KV_RANK": kv_rank, "ROT": rot})
        lib.alofa_latent_attention_bf16.restype = _I
        lib.alofa_latent_attention_bf16.argtypes = [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P, _P, _I, _I, _I, _P]
        _libs[key] = lib
    return lib


LATENT_KEY_BLOCK = 32  # rows of the cache per key block of the tensor-core kernel


def latent_attention_bf16(out, qa, cache_rows, sink, q_start, kv_len, block_table, page_size: int, n_seqs: int, max_q_len: int, heads: int, kv_rank: int, rot: int,
                          window, scale: float, splits: int = 1, blocks_per_split: int = 0, part_o=None, part_ml=None) -> None:
    """The same attention as :func:`latent_attention` on tensor cores, for
    bfloat16 and sizes :func:`latent_attention_bf16_supported` names: the rows
    of request r are ``q_start[r] .. q_start[r + 1]``, the last of them at
    position ``kv_len[r] - 1``.  With ``splits`` > 1 every request's key
    blocks (of ``LATENT_KEY_BLOCK`` rows) are dealt to that many CTAs,
    ``blocks_per_split`` each, which leave their shares in ``part_o`` [splits,
    T * heads, kv_rank] and ``part_ml`` [splits, T * heads, 2] (fp32) for a
    second kernel to merge."""
    bf = torch.bfloat16
    n = qa.shape[0]
    if qa.shape[1] != heads * (kv_rank + rot) or tuple(out.shape) != (n, heads * kv_rank) or cache_rows.shape[1] != kv_rank + rot:
        raise AlofaError("invalid_argument", "latent_attention sizes disagree", f"qa={tuple(qa.shape)} out={tuple(out.shape)} cache={tuple(cache_rows.shape)}")
    _done(
        _latent_attention_lib(kv_rank, rot).alofa_latent_attention_bf16(
            _dev(out, "out", bf), _dev(qa, "qa", bf), _dev(cache_rows, "cache", bf), _dev(sink, "sink", torch.float32) if sink is not None else None,
            _dev(q_start, "q_start", torch.int32), _dev(kv_len, "kv_len", torch.int32), _dev(block_table, "block_table", torch.int32), block_table.shape[1],
            page_size, n_seqs, max_q_len, heads, int(window or 0), float(scale),
            _dev(part_o, "part_o", torch.float32) if splits > 1 else None, _dev(part_ml, "part_ml", torch.float32) if splits > 1 else None,
            splits, blocks_per_split, n * heads, _stream(),
        ),
        "latent_attention_bf16", f"heads={heads} kv_rank={kv_rank} rot={rot} splits={splits}",
    )
    if splits > 1:
        count_launches(1)


# -- mixers with a state of fixed size, and what stands around them --------------------------------
def _recurrent():
    lib = _libs.get("recurrent")
    if lib is None:
        lib = load_library("alofa_recurrent", ["kernels/recurrent.cu"])
        sigs = {
            "alofa_embed_scaled": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _F, _I, _P, _P],
            "alofa_add_rows": [_P, _P, _L, _P],
            "alofa_causal_conv": [_P, _P, _I, _I, _P, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _P],
            "alofa_linear_scan": [_P, _P, _I, _I, _P, _I, _I, _P, _I, _I, _P, _I, _I, _P, _P, _P, _F, _F, _P, _L, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
            "alofa_gated_group_norm": [_P, _P, _P, _I, _I, _P, _I, _I, _I, _I, _F, _I, _I, _P],
            "alofa_branch_norm_add": [_P, _P, _P, _P, _P, _I, _I, _F, _F, _P],
            "alofa_qkv_prepare": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _F, _F, _I, _P, _I, _F, _I, _I, _I, _I, _L, _P, _P, _I, _I, _P],
            "alofa_heads_finish": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _F, _F, _I, _I, _P],
        }
        for name, args in sigs.items():
            fn = getattr(lib, name)
            fn.restype = _I
            fn.argtypes = args
        _libs["recurrent"] = lib
    return lib


def embed_scaled(out, table, ids, positions, scale: float, freq=None, status=None, src=None, fed=None) -> None:
    """out[t] = table[ids[t]] * scale (+ the sinusoidal position vector of
    ``positions[t]``: entry 2i sin(p freq[i]), entry 2i + 1 cos(p freq[i]));
    out fp32 [T, H], freq fp32 [ceil(H / 2)] or None.  ``src`` / ``fed`` as in
    :func:`embed_gather`."""
    n, hidden = out.shape
    if freq is not None and freq.shape[0] != (hidden + 1) // 2:
        raise AlofaError("invalid_argument", "embed_scaled sizes disagree", f"out={tuple(out.shape)} freq={tuple(freq.shape)}")
    i32 = torch.int32
    _done(
        _recurrent().alofa_embed_scaled(
            _dev(out, "out", torch.float32), _dev(table, "table"), _dev(ids, "ids", i32), _dev(src, "src", i32) if src is not None else None,
            _dev(fed, "fed", i32) if src is not None else None, _dev(positions, "positions", i32), _dev(freq, "freq", torch.float32) if freq is not None else None,
            n, hidden, table.shape[0], float(scale), _is_bf16(table, "table"), _dev(status, "status", i32) if status is not None else None, _stream(),
        ),
        "embed_scaled",
    )


def add_rows(out, x) -> None:
    """out += x (fp32, same shape)."""
    if out.shape != x.shape:
        raise AlofaError("invalid_argument", "add_rows sizes disagree", f"out={tuple(out.shape)} x={tuple(x.shape)}")
    _done(_recurrent().alofa_add_rows(_dev(out, "out", torch.float32), _dev(x, "x", torch.float32), out.numel(), _stream()), "add_rows")


def causal_conv(out, u, offset: int, w, bias, state, q_start, state_slots, seq_of_token, n_seqs: int, act: bool = True) -> None:
    """out [T, C] = silu(bias + causal convolution per channel) (``act`` False: no silu) of the columns
    ``offset .. offset + C`` of u [T, ld] (fp32), w [C, taps] fp32 with the
    token's own tap last; ``state`` [slots, >= (taps - 1) * C] fp32 holds each
    request's last taps - 1 inputs and is brought up to date."""
    n, channels = out.shape
    taps = w.shape[1]
    f32, i32 = torch.float32, torch.int32
    if w.shape[0] != channels or u.shape[0] != n or offset + channels > u.shape[1] or state.stride(0) < (taps - 1) * channels:
        raise AlofaError("invalid_argument", "causal_conv sizes disagree", f"out={tuple(out.shape)} u={tuple(u.shape)} w={tuple(w.shape)}")
    if state.dtype != f32 or not state.is_cuda or state.stride(-1) != 1:
        raise AlofaError("invalid_argument", "causal_conv needs an fp32 state on the device")
    _done(
        _recurrent().alofa_causal_conv(
            _dev(out, "out", f32), _dev(u, "u", f32), u.shape[1], offset, _dev(w, "w", f32), _dev(bias, "bias", f32) if bias is not None else None,
            state.data_ptr(), state.stride(0), _dev(q_start, "q_start", i32), _dev(state_slots, "state_slots", i32), _dev(seq_of_token, "seq_of_token", i32),
            n, n_seqs, channels, taps, 1 if act else 0, _stream(),
        ),
        "causal_conv", f"channels={channels} taps={taps}",
    )
    if taps > 1:
        count_launches(1)  # the kernel that moves the state on


def linear_scan(y, v, v_off: int, b, b_off: int, c, c_off: int, dec, d_off: int, state, q_start, state_slots, n_seqs: int, heads: int, groups: int, n: int, p: int,
                mode: int, dt_bias=None, a_log=None, d_skip=None, tau: float = 1.0, q_scale: float = 1.0, spread: int = 0, work=None) -> None:
    """The recurrence ``S_t = diag(a_t) S_(t-1) + k_t v_t^T, y_t = S_t^T q_t``
    per head over each request's tokens of the step in order, all fp32; the
    state [slots, >= heads * p * n] (per head [p][n]) is read and left up to
    date.  ``v``, ``b`` (keys), ``c`` (queries), ``dec`` are fp32 matrices of
    one row per token, read at the given column offsets.  ``mode`` 0: one
    decay per head, ``dt = softplus(dec[t, h] + dt_bias[h])``, ``a =
    exp(-exp(a_log[h]) dt)``, keys times dt, ``y += d_skip[h] v``, keys and
    queries shared by the heads of a group.  ``mode`` 1: one decay per key
    channel, ``a = sigmoid(dec[t, h, :]) ** (1 / tau)``, queries times
    ``q_scale``.  ``work``: fp32 scratch for the decays, :func:`linear_scan_work`
    numbers (allocated when absent: callers inside a step pass step scratch)."""
    f32, i32 = torch.float32, torch.int32
    rows = y.shape[0]
    if tuple(y.shape) != (rows, heads * p) or state.stride(0) < heads * p * n or state.dtype != f32 or not state.is_cuda:
        raise AlofaError("invalid_argument", "linear_scan sizes disagree", f"y={tuple(y.shape)} state={tuple(state.shape)} heads={heads} n={n} p={p}")
    for t_, name in ((v, "v"), (b, "b"), (c, "c"), (dec, "dec")):
        if t_.shape[0] != rows or t_.dtype != f32 or t_.dim() != 2:
            raise AlofaError("invalid_argument", "linear_scan operand must be fp32 with one row per token", name)
    opt = lambda t_, name: _dev(t_, name, f32) if t_ is not None else None
    need = linear_scan_work(rows, heads, n, mode)
    if work is None:
        work = torch.empty((need,), dtype=f32, device=y.device)
    if work.numel() < need:
        raise AlofaError("invalid_argument", "linear_scan scratch is too small", f"have={work.numel()} need={need}")
    count_launches(1)  # the kernel that makes the decays
    _done(
        _recurrent().alofa_linear_scan(
            _dev(y, "y", f32), _dev(v, "v"), v.shape[1], v_off, _dev(b, "b"), b.shape[1], b_off, _dev(c, "c"), c.shape[1], c_off, _dev(dec, "dec"), dec.shape[1], d_off,
            opt(dt_bias, "dt_bias"), opt(a_log, "a_log"), opt(d_skip, "d_skip"), 1.0 / float(tau), float(q_scale), state.data_ptr(), state.stride(0),
            _dev(q_start, "q_start", i32), _dev(state_slots, "state_slots", i32), rows, n_seqs, heads, groups, n, p, mode, spread, _dev(work, "work", f32), _stream(),
        ),
        "linear_scan", f"heads={heads} groups={groups} n={n} p={p} mode={mode}",
    )


def linear_scan_work(rows: int, heads: int, n: int, mode: int) -> int:
    """How many fp32 numbers of scratch :func:`linear_scan` needs."""
    return rows * (heads * n if mode else 2 * heads)


def gated_group_norm(out, y, gate, g_off: int, w, groups: int, eps: float, gate_first: bool, sigmoid: bool = False) -> None:
    """out = rows of y [T, width] normed in ``groups`` equal parts (each by
    its own root mean square), times ``w[c % len(w)]``, with the gate
    ``silu(gate[t, g_off + c])`` multiplied in before the norm
    (``gate_first``) or after it (``sigmoid``: the gate is ``sigmoid(.)``
    instead); fp32 in, out in its own dtype."""
    n, width = y.shape
    f32 = torch.float32
    if tuple(out.shape) != (n, width) or (gate is not None and (gate.shape[0] != n or g_off + width > gate.shape[1])):
        raise AlofaError("invalid_argument", "gated_group_norm sizes disagree", f"y={tuple(y.shape)} out={tuple(out.shape)}")
    _done(
        _recurrent().alofa_gated_group_norm(_dev(out, "out"), _dev(y, "y", f32), _dev(gate, "gate", f32) if gate is not None else None,
                                            gate.shape[1] if gate is not None else 0, g_off, _dev(w, "w", f32), w.shape[0], n, width, groups, float(eps),
                                            (1 if gate_first else 0) | (2 if sigmoid else 0), _is_bf16(out, "out"), _stream()),
        "gated_group_norm", f"width={width} groups={groups}",
    )


def branch_norm_add(h, ya, wa, yb, wb, eps: float, scale: float) -> None:
    """h += scale * (rmsnorm(ya) * wa + rmsnorm(yb) * wb), all fp32 [T, hidden]; ``yb`` may be None."""
    f32 = torch.float32
    rows, hidden = h.shape
    if tuple(ya.shape) != (rows, hidden) or (yb is not None and tuple(yb.shape) != (rows, hidden)):
        raise AlofaError("invalid_argument", "branch_norm_add sizes disagree", f"h={tuple(h.shape)} ya={tuple(ya.shape)}")
    _done(
        _recurrent().alofa_branch_norm_add(_dev(h, "h", f32), _dev(ya, "ya", f32), _dev(wa, "wa", f32), _dev(yb, "yb", f32) if yb is not None else None,
                                           _dev(wb, "wb", f32) if yb is not None else None, rows, hidden, float(eps), float(scale), _stream()),
        "branch_norm_add",
    )


def qkv_prepare(q_out, k_cache, v_cache, qkv, positions, slot_map, heads: int, kv_heads: int, d: int, dv: int, qk_norm: bool, eps: float, coef: float, every: int,
                freq=None, rot_dims: int = 0, maps: int = 1, q_weight=None, k_weight=None, magnitude: float = 1.0, values_from_keys: bool = False, v_copies: int = 1, extra_out=None, extra_at: int = 0) -> None:
    """From the fp32 sums of a stacked projection whose rows start [q | k | v]
    (more columns may follow): q and k divided by their root mean square per
    head (``qk_norm``) and multiplied by ``q_weight`` / ``k_weight`` (fp32
    [d], may be None), q times ``1 + coef * ln(floor((p + 1) / every) + 1)`` at
    position p, the first ``rot_dims`` numbers of every q and k head turned by
    the position (neighbouring pairs, pair i by the angle ``p * freq[i]``,
    cosine and sine times ``magnitude``), q to ``q_out``, k and v to the
    tokens' cache slots; out tensors in the compute dtype.  ``maps`` > 1: every
    head has that many queries and every key head that many keys, side by side
    per head; the queries are written as ``[key head][map][head of the
    group]``, so that a kernel which gives query unit ``i`` the key unit ``i //
    (heads / kv_heads)`` pairs map with map.  ``values_from_keys``: there are
    no v columns, the values are the keys as projected (before their norm).
    ``v_copies`` > 1: every value head is written that many times side by side
    (the value cache then has ``kv_heads * v_copies`` heads), for kernels that
    want a value head for each key head.  ``qkv`` may be the partial sums a
    product left owed (``.sums`` [splits, T, ld], ``.splits``, ``.bias``): they
    are added here, in split order.  ``extra_out`` (fp32 [T, m]): the m columns
    from ``extra_at`` on (what follows q, k and v in the row) are written there,
    finished."""
    f32 = torch.float32
    splits, plane, bias = 0, 0, None
    if not isinstance(qkv, torch.Tensor):
        splits, bias, sums = int(qkv.splits), qkv.bias, qkv.sums
        qkv = sums[0]
        plane = sums.shape[1] * sums.shape[2]
        if sums.shape[0] != splits or not sums.is_contiguous():
            raise AlofaError("invalid_argument", "qkv_prepare: owed sums disagree with their count", f"sums={tuple(sums.shape)} splits={splits}")
    n = qkv.shape[0]
    dt = q_out.dtype
    if extra_out is not None and (extra_out.shape[0] != n or extra_at + extra_out.shape[1] > qkv.shape[1]):
        raise AlofaError("invalid_argument", "qkv_prepare: the extra columns lie outside the row", f"qkv={tuple(qkv.shape)} extra={tuple(extra_out.shape)} at={extra_at}")
    need = (heads + kv_heads) * maps * d + (0 if values_from_keys else kv_heads * dv)
    if (qkv.shape[1] < need or tuple(q_out.shape) != (n, heads * maps * d) or tuple(k_cache.shape[1:]) != (kv_heads * maps, d) or tuple(v_cache.shape[1:]) != (kv_heads * v_copies, dv)
            or (q_weight is not None and q_weight.shape[0] != d) or (k_weight is not None and k_weight.shape[0] != d)):
        raise AlofaError("invalid_argument", "qkv_prepare sizes disagree", f"qkv={tuple(qkv.shape)} q={tuple(q_out.shape)} k={tuple(k_cache.shape)} v={tuple(v_cache.shape)}")
    _done(
        _recurrent().alofa_qkv_prepare(_dev(q_out, "q_out"), _dev(k_cache, "k_cache", dt), _dev(v_cache, "v_cache", dt), _dev(qkv, "qkv", f32), qkv.shape[1],
                                       _dev(positions, "positions", torch.int32), _dev(slot_map, "slot_map", torch.int32), n, heads, kv_heads, d, dv, int(maps),
                                       1 if qk_norm else 0, _dev(q_weight, "q_weight", f32) if q_weight is not None else None,
                                       _dev(k_weight, "k_weight", f32) if k_weight is not None else None, float(eps), float(coef), int(every),
                                       _dev(freq, "freq", f32) if rot_dims else None, int(rot_dims), float(magnitude), 1 if values_from_keys else 0, int(v_copies),
                                       _is_bf16(q_out, "q_out"), splits, plane, _dev(bias, "bias", f32) if bias is not None else None,
                                       _dev(extra_out, "extra_out", f32) if extra_out is not None else None, int(extra_at),
                                       extra_out.shape[1] if extra_out is not None else 0, _stream()),
        "qkv_prepare", f"heads={heads} kv_heads={kv_heads} d={d} dv={dv} maps={maps}",
    )


def heads_finish(out, a, heads: int, kv_heads: int, dv: int, maps: int = 1, difference: float = 0.0, eps: float = 0.0, post: float = 1.0, gate=None, g_off: int = 0) -> None:
    """What stands between some attentions and their output projection, fp32:
    ``a`` [T, heads * maps * dv] (fp32, or bfloat16 like ``out``) holds the attention outputs in the order
    :func:`qkv_prepare` gave the queries.  ``maps`` 2: ``o = a_1 - difference *
    a_2``, then ``o / sqrt(mean(o^2) + eps) * post`` per head; ``gate`` (fp32
    [T, ld], sums of a projection): ``o *= sigmoid(gate[t, g_off + h])``.  out
    [T, heads * dv] in the compute dtype, heads in their own order."""
    n = a.shape[0]
    if tuple(a.shape) != (n, heads * maps * dv) or tuple(out.shape) != (n, heads * dv) or (gate is not None and (gate.shape[0] != n or g_off + heads > gate.shape[1])):
        raise AlofaError("invalid_argument", "heads_finish sizes disagree", f"a={tuple(a.shape)} out={tuple(out.shape)}")
    _done(_recurrent().alofa_heads_finish(_dev(out, "out"), _dev(a, "a"), _dev(gate, "gate", torch.float32) if gate is not None else None,
                                          gate.shape[1] if gate is not None else 0, g_off, n, heads, kv_heads, dv, maps, float(difference), float(eps), float(post),
                                          _is_bf16(out, "out"), _is_bf16(a, "a"), _stream()), "heads_finish", f"heads={heads} dv={dv} maps={maps}")


def _hyper():
    lib = _libs.get("hyper")
    if lib is None:
        lib = load_library("alofa_hyper", ["kernels/hyper.cu"])
        sigs = {
            "alofa_hyper_connect": [_P, _L, _P, _P, _P, _P, _P, _F, _P, _P, _I, _I, _I, _I, _P],
            "alofa_streams_fill": [_P, _L, _P, _L, _I, _P],
            "alofa_scaled_sum": [_P, _P, _F, _P, _F, _L, _I, _P],
            "alofa_scale_rows": [_P, _F, _L, _P],
            "alofa_softcap_rows": [_P, _F, _L, _P],
            "alofa_head_gate": [_P, _P, _I, _I, _I, _I, _I, _I, _P],
        }
        for name, args in sigs.items():
            fn = getattr(lib, name)
            fn.restype = _I
            fn.argtypes = args
        _libs["hyper"] = lib
    return lib


HYPER_MAX_STREAMS = 8


def hyper_connect(streams, y=None, mix=None, out_w=None, in_w=None, norm_w=None, eps: float = 0.0, x_out=None, sum_out=None) -> None:
    """One pass over several residual streams ``streams`` [S, T, W] (fp32), any
    subset of: with ``y`` [T, W] (a sublayer's output) every stream moves at
    once, ``x_t <- sum_s mix[s, t] x_s + out_w[t] y``; with ``x_out`` the next
    sublayer's input ``rmsnorm(sum_s in_w[s] x_s) * norm_w`` is written in
    ``x_out``'s dtype; with ``sum_out`` (fp32 [T, W]) the streams' sum."""
    f32 = torch.float32
    S, n, width = streams.shape
    if streams.dtype != f32 or not streams.is_cuda or streams.stride(2) != 1 or streams.stride(1) != width:
        raise AlofaError("invalid_argument", "hyper_connect wants fp32 streams [S, T, W] with packed rows")
    for t_, name in ((y, "y"), (x_out, "x_out"), (sum_out, "sum_out")):
        if t_ is not None and tuple(t_.shape) != (n, width):
            raise AlofaError("invalid_argument", "hyper_connect sizes disagree", f"{name}={tuple(t_.shape)} streams={tuple(streams.shape)}")
    if (y is not None and (tuple(mix.shape) != (S, S) or out_w.shape[0] != S)) or (x_out is not None and (in_w.shape[0] != S or norm_w.shape[0] != width)):
        raise AlofaError("invalid_argument", "hyper_connect weights disagree with the streams", f"S={S} width={width}")
    _done(
        _hyper().alofa_hyper_connect(
            streams.data_ptr(), streams.stride(0), _dev(y, "y", f32) if y is not None else None, _dev(mix, "mix", f32) if y is not None else None,
            _dev(out_w, "out_w", f32) if y is not None else None, _dev(in_w, "in_w", f32) if x_out is not None else None,
            _dev(norm_w, "norm_w", f32) if x_out is not None else None, float(eps), _dev(x_out, "x_out") if x_out is not None else None,
            _dev(sum_out, "sum_out", f32) if sum_out is not None else None, n, S, width, _is_bf16(x_out, "x_out") if x_out is not None else 0, _stream(),
        ),
        "hyper_connect", f"S={S} width={width}",
    )


def streams_fill(streams, h) -> None:
    """streams[s] = h for every s: streams [S, T, W] fp32, h [T, W] fp32."""
    if tuple(streams.shape[1:]) != tuple(h.shape) or streams.dtype != torch.float32 or streams.stride(1) != h.shape[1] or streams.stride(2) != 1:
        raise AlofaError("invalid_argument", "streams_fill sizes disagree", f"streams={tuple(streams.shape)} h={tuple(h.shape)}")
    _done(_hyper().alofa_streams_fill(streams.data_ptr(), streams.stride(0), _dev(h, "h", torch.float32), h.numel(), streams.shape[0], _stream()), "streams_fill")


def scaled_sum(out, ya, sa: float, yb=None, sb: float = 0.0, accumulate: bool = False) -> None:
    """out (+)= sa * ya + sb * yb, fp32, same shapes (``yb`` may be None)."""
    f32 = torch.float32
    if out.shape != ya.shape or (yb is not None and yb.shape != ya.shape):
        raise AlofaError("invalid_argument", "scaled_sum sizes disagree", f"out={tuple(out.shape)} ya={tuple(ya.shape)}")
    _done(_hyper().alofa_scaled_sum(_dev(out, "out", f32), _dev(ya, "ya", f32), float(sa), _dev(yb, "yb", f32) if yb is not None else None, float(sb), out.numel(),
                                    1 if accumulate else 0, _stream()), "scaled_sum")


def scale_rows(x, scale: float) -> None:
    """x *= scale (fp32, in place)."""
    _done(_hyper().alofa_scale_rows(_dev(x, "x", torch.float32), float(scale), x.numel(), _stream()), "scale_rows")


def softcap_rows(x, cap: float) -> None:
    """x = cap * tanh(x / cap) (fp32, in place)."""
    _done(_hyper().alofa_softcap_rows(_dev(x, "x", torch.float32), float(cap), x.numel(), _stream()), "softcap_rows")


def head_gate(o, gate, g_off: int, heads: int, vdim: int) -> None:
    """o[t, h, :] *= sigmoid(gate[t, g_off + h]) in place: o [T, heads * vdim]
    in its own dtype, gate fp32 [T, ld] (sums of a projection)."""
    n = o.shape[0]
    if o.shape[1] != heads * vdim or gate.shape[0] != n or g_off + heads > gate.shape[1]:
        raise AlofaError("invalid_argument", "head_gate sizes disagree", f"o={tuple(o.shape)} gate={tuple(gate.shape)}")
    _done(_hyper().alofa_head_gate(_dev(o, "o"), _dev(gate, "gate", torch.float32), gate.shape[1], g_off, n, heads, vdim, _is_bf16(o, "o"), _stream()), "head_gate")


def _delta():
    lib = _libs.get("delta")
    if lib is None:
        lib = load_library("alofa_delta", ["kernels/delta.cu"])
        sigs = {
            "alofa_min_gru": [_P, _P, _I, _I, _I, _I, _P, _L, _P, _P, _I, _I, _I, _I, _P],
            "alofa_delta_prepare": [_P, _P, _P, _P, _P, _P, _I, _P, _I, _P, _I, _I, _P, _P, _I, _I, _I, _I, _F, _F, _P],
            "alofa_delta_scan": [_P, _P, _I, _I, _P, _P, _P, _P, _P, _P, _L, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
        }
        for name, args in sigs.items():
            fn = getattr(lib, name)
            fn.restype = _I
            fn.argtypes = args
        _libs["delta"] = lib
    return lib


def _slot_state(state, words: int, what: str) -> None:
    if state.dtype != torch.float32 or not state.is_cuda or state.stride(-1) != 1 or state.stride(0) < words:
        raise AlofaError("invalid_argument", f"{what} needs an fp32 state on the device with room for every slot", f"state={tuple(state.shape)} words={words}")


def min_gru(out, u, z_off: int, x_off: int, g_off: int, state, q_start, state_slots, n_seqs: int) -> None:
    """Element by element over each request's tokens of the step in order:
    ``z = sigmoid(u[t, z_off + c])``, ``x = u[t, x_off + c]``, the candidate
    ``x + 1/2`` where ``x >= 0`` and ``sigmoid(x)`` below, ``S = (1 - z) S + z
    * candidate``, ``out[t, c] = S * silu(u[t, g_off + c])``.  u fp32 [T, ld];
    out [T, width] in its own dtype; state [slots, >= width] fp32, read and
    left up to date."""
    n, width = out.shape
    i32 = torch.int32
    if u.shape[0] != n or max(z_off, x_off, g_off) + width > u.shape[1]:
        raise AlofaError("invalid_argument", "min_gru sizes disagree", f"out={tuple(out.shape)} u={tuple(u.shape)}")
    _slot_state(state, width, "min_gru")
    _done(_delta().alofa_min_gru(_dev(out, "out"), _dev(u, "u", torch.float32), u.shape[1], z_off, x_off, g_off, state.data_ptr(), state.stride(0),
                                 _dev(q_start, "q_start", i32), _dev(state_slots, "state_slots", i32), n_seqs, n, width, _is_bf16(out, "out"), _stream()), "min_gru")


def delta_prepare(qn, kn, kq, g, beta, conv, dz, u, b_off: int, dt_bias, a_log, heads: int, groups: int, n: int, unit_eps: float, q_scale: float) -> None:
    """What :func:`delta_scan` reads, all fp32: from conv [T, ld] = [q: groups *
    n | k: groups * n | v ...] the unit vectors ``qn = q / sqrt(sum q^2 +
    unit_eps) * q_scale`` and ``kn`` (no scale) per group, ``kq = kn . qn``;
    from the first heads * n columns of dz [T, ld''] the decays ``g = exp(-exp(a_log[h]) * softplus(dz +
    dt_bias))``; from u [T, ld'] ``beta = sigmoid(u[t, b_off + h])``."""
    f32 = torch.float32
    rows = conv.shape[0]
    if (tuple(qn.shape) != (rows, groups * n) or tuple(kn.shape) != (rows, groups * n) or tuple(kq.shape) != (rows, groups) or tuple(g.shape) != (rows, heads * n)
            or tuple(beta.shape) != (rows, heads) or dz.shape[0] != rows or dz.shape[1] < heads * n or conv.shape[1] < 2 * groups * n or u.shape[0] != rows
            or b_off + heads > u.shape[1] or dt_bias.shape[0] != heads * n or a_log.shape[0] != heads):
        raise AlofaError("invalid_argument", "delta_prepare sizes disagree", f"conv={tuple(conv.shape)} dz={tuple(dz.shape)} heads={heads} groups={groups} n={n}")
    _done(_delta().alofa_delta_prepare(_dev(qn, "qn", f32), _dev(kn, "kn", f32), _dev(kq, "kq", f32), _dev(g, "g", f32), _dev(beta, "beta", f32), _dev(conv, "conv", f32),
                                       conv.shape[1], _dev(dz, "dz", f32), dz.shape[1], _dev(u, "u", f32), u.shape[1], b_off, _dev(dt_bias, "dt_bias", f32), _dev(a_log, "a_log", f32),
                                       rows, heads, groups, n, float(unit_eps), float(q_scale), _stream()), "delta_prepare")


def delta_scan(y, v, v_off: int, kn, qn, kq, g, beta, state, q_start, state_slots, n_seqs: int, heads: int, groups: int, n: int, p: int, spread: int = 0) -> None:
    """The gated delta rule per head over each request's tokens of the step in
    order, all fp32: ``S <- diag(g_t) S; u = beta_t (v_t - S^T k_t); S <- S +
    k_t u^T; y_t = S^T q_t``.  The state [slots, >= heads * p * n] (per head
    [p][n]) is read and left up to date; v fp32 [T, ld] at column offset
    ``v_off`` (heads * p columns); head h reads the keys and queries of group
    ``h // (heads / groups)``."""
    f32, i32 = torch.float32, torch.int32
    rows = y.shape[0]
    if (tuple(y.shape) != (rows, heads * p) or v.shape[0] != rows or v_off + heads * p > v.shape[1] or tuple(kn.shape) != (rows, groups * n)
            or tuple(qn.shape) != (rows, groups * n) or tuple(kq.shape) != (rows, groups) or tuple(g.shape) != (rows, heads * n) or tuple(beta.shape) != (rows, heads)):
        raise AlofaError("invalid_argument", "delta_scan sizes disagree", f"y={tuple(y.shape)} v={tuple(v.shape)} heads={heads} groups={groups} n={n} p={p}")
    _slot_state(state, heads * p * n, "delta_scan")
    _done(_delta().alofa_delta_scan(_dev(y, "y", f32), _dev(v, "v", f32), v.shape[1], v_off, _dev(kn, "kn", f32), _dev(qn, "qn", f32), _dev(kq, "kq", f32), _dev(g, "g", f32),
                                    _dev(beta, "beta", f32), state.data_ptr(), state.stride(0), _dev(q_start, "q_start", i32), _dev(state_slots, "state_slots", i32),
                                    rows, n_seqs, heads, groups, n, p, spread, _stream()), "delta_scan", f"heads={heads} groups={groups} n={n} p={p}")


# -- the real-gated linear recurrent unit ------------------------------------------------------------
def _gated_lru():
    lib = _libs.get("gated_lru")
    if lib is None:
        lib = load_library("alofa_gated_lru", ["kernels/gated_lru.cu"])
        sigs = {
            "alofa_lru_gates": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _F, _I, _I, _I, _P],
            "alofa_lru_scan": [_P, _P, _P, _P, _I, _I, _I, _P, _L, _P, _P, _I, _I, _I, _I, _P],
        }
        for name, args in sigs.items():
            fn = getattr(lib, name)
            fn.restype = _I
            fn.argtypes = args
        _libs["gated_lru"] = lib
    return lib


def lru_gates(a, b, u, wa_t, wi_t, ba, bi, lam, decay_scale: float, blocks: int, wa_rows=None, wi_rows=None) -> None:
    """Decays and driven inputs of the gated linear recurrent unit, all fp32:
    per block of ``W / blocks`` channels ``r = sigmoid(A u_b + ba)``, ``i =
    sigmoid(I u_b + bi)``; ``a = exp(-decay_scale * r * softplus(lam))`` (``lam``
    [W]) and ``b = sqrt(1 - a^2) * i * u``.  u, a, b [T, W]; ``wa_t``, ``wi_t``
    [blocks, in, out]: the blocks' matrices transposed; ``wa_rows``, ``wi_rows``
    (optional): the same as [blocks, out, in], which steps of a few tokens read
    with a warp per output channel."""
    f32 = torch.float32
    n, width = u.shape
    if width % blocks:
        raise AlofaError("invalid_argument", "the blocks must divide the recurrence's width", f"width={width} blocks={blocks}")
    bs = width // blocks
    if (tuple(a.shape) != (n, width) or tuple(b.shape) != (n, width) or tuple(wa_t.shape) != (blocks, bs, bs) or tuple(wi_t.shape) != (blocks, bs, bs)
            or ba.shape[0] != width or bi.shape[0] != width or lam.shape[0] != width):
        raise AlofaError("invalid_argument", "lru_gates sizes disagree", f"u={tuple(u.shape)} wa={tuple(wa_t.shape)} blocks={blocks}")
    rows = wa_rows is not None and wi_rows is not None
    if rows and (tuple(wa_rows.shape) != (blocks, bs, bs) or tuple(wi_rows.shape) != (blocks, bs, bs)):
        raise AlofaError("invalid_argument", "lru_gates sizes disagree", f"wa_rows={tuple(wa_rows.shape)} blocks={blocks}")
    _done(_gated_lru().alofa_lru_gates(_dev(a, "a", f32), _dev(b, "b", f32), _dev(u, "u", f32), _dev(wa_t, "wa", f32), _dev(wi_t, "wi", f32),
                                       _dev(wa_rows, "wa_rows", f32) if rows else None, _dev(wi_rows, "wi_rows", f32) if rows else None, _dev(ba, "ba", f32),
                                       _dev(bi, "bi", f32), _dev(lam, "lam", f32), float(decay_scale), n, width, blocks, _stream()), "lru_gates", f"width={width} blocks={blocks}")


def lru_scan(out, a, b, y, y_off: int, act: str, state, q_start, state_slots, n_seqs: int) -> None:
    """``S = a_t * S + b_t`` element by element over each request's tokens of
    the step in order; ``out[t] = S_t * act(y[t, y_off + c])``.  a, b fp32 [T,
    W]; y fp32 [T, ld]; out [T, W] in its own dtype; state [slots, >= W] fp32,
    read and left up to date."""
    n, width = out.shape
    f32, i32 = torch.float32, torch.int32
    if tuple(a.shape) != (n, width) or tuple(b.shape) != (n, width) or y.shape[0] != n or y_off + width > y.shape[1]:
        raise AlofaError("invalid_argument", "lru_scan sizes disagree", f"out={tuple(out.shape)} a={tuple(a.shape)} y={tuple(y.shape)}")
    _slot_state(state, width, "lru_scan")
    _done(_gated_lru().alofa_lru_scan(_dev(out, "out"), _dev(a, "a", f32), _dev(b, "b", f32), _dev(y, "y", f32), y.shape[1], y_off, ACTIVATIONS[act], state.data_ptr(),
                                      state.stride(0), _dev(q_start, "q_start", i32), _dev(state_slots, "state_slots", i32), n_seqs, n, width, _is_bf16(out, "out"),
                                      _stream()), "lru_scan")
