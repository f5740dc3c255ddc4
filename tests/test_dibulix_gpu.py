"""Dibulix on the GPU against the plain implementation (tests/plain_dibulix.py).

Mechanisms alone (kernel against the plain function of the same mechanism):
the connections between several residual streams (the owed write, the read and
its norm, the sum), the minGRU recurrence and the gated delta rule over
portions and reused slots (a far token whose trace must survive), the windowed
attention with a sink, biases and a rotated part of each head (keys just
inside and just outside the window, at page borders, far keys), the latent
attention with halves paired, scaled frequencies, a window and a gate per
head, the squared relu.  Then whole models of four configurations, in 32-bit
and bfloat16: whole prompts, prefill against token-by-token decoding, portions
down to two tokens, batches of unequal requests in a pool so small that pages
and slots are used again, long decoding from the first token, the stream after
every layer, and greedy generation through the engine and the programs."""
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_dibulix as plain
import replay
import tiny_dibulix as tiny
from gpu_util import assert_close, dev, rounded

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16
# Largest |engine - plain| on logits, times max(1, max|plain|): fp32 sums against float64; bfloat16 rounds
# activations and cache rows to 8 bits of mantissa.
TOL = {"float32": 3e-5, "bfloat16": 9e-2}
KERNEL_TOL = {F32: 1e-5, BF16: 2e-2}


def meta(counts, slots):
    q_start = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    seq = np.concatenate([np.full(c, s, dtype=np.int32) for s, c in enumerate(counts)])
    return dev(q_start), dev(np.asarray(slots, dtype=np.int32)), dev(seq)


def in_portions(lengths, cuts, slots_of, run):
    """Walk requests of ``lengths`` tokens through steps: request r brings ``cuts[(step + r) % len(cuts)]`` tokens and
    sits out every third step.  ``run(live, spans, q_start, slots, seq)`` -> rows [tokens of the step, ...] (numpy);
    returns per request the rows of all its tokens in order."""
    got = [[] for _ in lengths]
    at = [0] * len(lengths)
    step = 0
    while any(at[r] < lengths[r] for r in range(len(lengths))):
        live = [r for r in range(len(lengths)) if at[r] < lengths[r] and (step + r) % 3 != 2]
        step += 1
        if not live:
            continue
        counts = [min(cuts[(step + r) % len(cuts)], lengths[r] - at[r]) for r in live]
        spans = [(at[r], at[r] + c) for r, c in zip(live, counts)]
        q_start, slots, seq = meta(counts, [slots_of[r] for r in live])
        rows = run(live, spans, q_start, slots, seq)
        k = 0
        for r, c in zip(live, counts):
            got[r].append(rows[k : k + c])
            k += c
            at[r] += c
    return [np.concatenate(g) for g in got]


# ---------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("S,width", [(1, 96), (2, 100), (3, 64), (4, 1030), (8, 33)])
def test_streams_are_moved_read_normed_and_summed(dtype, S, width):
    """One pass does the owed write, the next read with its norm, or the sum; every stream from the OLD ones."""
    from alofa_b200.csrc import ops

    rng = np.random.default_rng(1)
    n, eps = 7, 2e-5
    xs = rounded(rng.standard_normal((S, n, width)) * 3, F32)
    y = rounded(rng.standard_normal((n, width)), F32)
    mix, out_w, in_w = (rounded(rng.standard_normal(s), F32) for s in ((S, S), (S,), (S,)))
    norm_w = rounded(1 + 0.2 * rng.standard_normal(width), F32)
    moved = plain.connect(list(xs), y, mix, out_w)
    # filled from one row block
    streams = torch.empty((S, n, width), dtype=F32, device="cuda")
    ops.streams_fill(streams, dev(xs[0], F32))
    assert all(torch.equal(streams[s], streams[0]) for s in range(S)) and np.array_equal(streams[0].cpu().numpy(), xs[0].astype(np.float32))
    # read and norm alone
    streams = dev(xs, F32)
    x_out = torch.empty((n, width), dtype=dtype, device="cuda")
    ops.hyper_connect(streams, in_w=dev(in_w, F32), norm_w=dev(norm_w, F32), eps=eps, x_out=x_out)
    assert_close(x_out.float().cpu(), plain.rms_norm(sum(in_w[s] * xs[s] for s in range(S)), norm_w, eps), KERNEL_TOL[dtype], "read")
    assert np.array_equal(streams.cpu().numpy(), xs.astype(np.float32)), "a read moved the streams"
    # the owed write, then the read of the moved streams
    ops.hyper_connect(streams, dev(y, F32), dev(mix, F32), dev(out_w, F32), dev(in_w, F32), dev(norm_w, F32), eps, x_out=x_out)
    assert_close(streams.cpu(), np.stack(moved), 1e-6, "moved streams")
    assert_close(x_out.float().cpu(), plain.rms_norm(sum(in_w[s] * moved[s] for s in range(S)), norm_w, eps), KERNEL_TOL[dtype], "read after the write")
    # the owed write and the sum
    streams = dev(xs, F32)
    total = torch.empty((n, width), dtype=F32, device="cuda")
    ops.hyper_connect(streams, dev(y, F32), dev(mix, F32), dev(out_w, F32), sum_out=total)
    assert_close(total.cpu(), sum(moved), 1e-6, "sum")


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("width", [7, 64, 300])
def test_min_gru_carries_its_state(dtype, width):
    """Three requests in portions of 1, 2 and many tokens; gates that mostly keep the state, so that it must be carried."""
    from alofa_b200.csrc import ops

    rng = np.random.default_rng(2)
    lengths, ld, off = [61, 30, 1], 3 * width + 5, (2, 2 + width, 2 + 2 * width)
    data = [rounded(rng.standard_normal((n, ld)) * 2, F32) for n in lengths]
    for u in data:
        u[:, off[0] : off[0] + width] -= 3.0
    want = [plain.min_gru_recurrence(u[:, off[0] : off[0] + width], u[:, off[1] : off[1] + width], u[:, off[2] : off[2] + width]) for u in data]
    state = torch.zeros((5, width + 3), dtype=F32, device="cuda")

    def run(live, spans, q_start, slots, seq):
        rows = dev(np.concatenate([data[r][a:b] for r, (a, b) in zip(live, spans)]), F32)
        out = torch.empty((rows.shape[0], width), dtype=dtype, device="cuda")
        ops.min_gru(out, rows, off[0], off[1], off[2], state, q_start, slots, len(live))
        return out.float().cpu().numpy()

    got = in_portions(lengths, [1, 2, 17, 1, 40], [4, 0, 2], run)
    for r in range(3):
        assert_close(got[r], want[r], KERNEL_TOL[dtype], f"request {r}")
    assert (state[[1, 3]] == 0).all() and (state[:, width:] == 0).all(), "state of another slot, or words after the state, were written"
    # the state itself is the recurrence's last value, in 32-bit whatever the output's type
    last = plain.min_gru_recurrence(data[0][:, off[0] : off[0] + width], data[0][:, off[1] : off[1] + width], np.full((61, width), 50.0))[-1] / 50.0
    assert_close(state[4, :width].cpu(), last, 1e-5, "state")


@pytest.mark.parametrize("lengths,portions", [([700], [300, 1, 33, 366]), ([530, 40, 259], [64, 200, 1, 265]), ([33, 2000], [16, 1000, 984])])
def test_min_gru_over_long_portions(lengths, portions):
    """Portions long enough that several warps share a request's tokens, beside short ones and single tokens: the
    stretches' ends fall anywhere, and the state a later portion starts from is the one the last stretch left."""
    from alofa_b200.csrc import ops

    rng = np.random.default_rng(21)
    width = 45
    data = [rounded(rng.standard_normal((n, 3 * width)) * 2, F32) for n in lengths]
    for u in data:
        u[:, :width] -= 3.0
    want = [plain.min_gru_recurrence(u[:, :width], u[:, width : 2 * width], u[:, 2 * width :]) for u in data]
    state = torch.zeros((len(lengths) + 1, width), dtype=F32, device="cuda")

    def run(live, spans, q_start, slots, seq):
        rows = dev(np.concatenate([data[r][a:b] for r, (a, b) in zip(live, spans)]), F32)
        out = torch.empty((rows.shape[0], width), dtype=F32, device="cuda")
        ops.min_gru(out, rows, 0, width, 2 * width, state, q_start, slots, len(live))
        return out.cpu().numpy()

    got = in_portions(lengths, portions, list(range(1, len(lengths) + 1)), run)
    for r in range(len(lengths)):
        assert_close(got[r], want[r], KERNEL_TOL[F32], f"request {r}")


def delta_case(rng, n, H, G, N, P, boost=None):
    """Rows as the mixer's kernels get them: conv = [q | k | v] after convolution and silu, the decays' logits, beta's logits."""
    f = lambda *s: rounded(rng.standard_normal(s), F32)
    conv, dz, u = f(n, 2 * G * N + H * P), f(n, H * N + 3) - 1.0, f(n, H + 2)
    if boost is not None and n > boost[1]:  # one early value written large; much later one query alone reads along its key
        conv[boost[0], 2 * G * N :] *= 30.0
        conv[boost[1], : G * N] = conv[boost[0], G * N : 2 * G * N] * 4.0
        dz[:, : H * N] -= 6.0  # slow decays, and later tokens that write (and so erase) little: the trace survives hundreds of tokens
        u[:, 1 : 1 + H] -= 6.0
        u[boost[0], 1 : 1 + H] = 4.0
    return conv, dz, u


def plain_delta(conv, dz, u, dt_bias, a_log, H, G, N, P):
    n = conv.shape[0]
    of = np.arange(H) // (H // G)
    q = (plain.unit_vectors(conv[:, : G * N].reshape(n, G, N)) * N ** -0.5)[:, of]
    k = plain.unit_vectors(conv[:, G * N : 2 * G * N].reshape(n, G, N))[:, of]
    g = plain.channel_decays(dz[:, : H * N].reshape(n, H, N), dt_bias, a_log)
    return plain.delta_rule(q, k, conv[:, 2 * G * N :].reshape(n, H, P), plain.sigmoid(u[:, 1 : 1 + H]), g).reshape(n, H * P)


def run_delta(lengths, cuts, H, G, N, P, seed=3, boost=None, state=None, slots_of=(4, 0, 2)):
    from alofa_b200.csrc import ops

    rng = np.random.default_rng(seed)
    dt_bias, a_log = rounded(rng.uniform(-3, 0.5, H * N), F32), rounded(np.log(rng.uniform(0.1, 2.0, H)), F32)
    data = [delta_case(rng, n, H, G, N, P, boost) for n in lengths]
    want = [plain_delta(*d, dt_bias, a_log, H, G, N, P) for d in data]
    if state is None:
        state = torch.zeros((5, H * P * N + 2), dtype=F32, device="cuda")

    def run(live, spans, q_start, slots, seq):
        cat = lambda i: dev(np.concatenate([data[r][i][a:b] for r, (a, b) in zip(live, spans)]), F32)
        conv, dz, u = cat(0), cat(1), cat(2)
        rows = conv.shape[0]
        e = lambda w: torch.empty((rows, w), dtype=F32, device="cuda")
        qn, kn, kq, g, beta, y = e(G * N), e(G * N), e(G), e(H * N), e(H), e(H * P)
        ops.delta_prepare(qn, kn, kq, g, beta, conv, dz, u, 1, dev(dt_bias, F32), dev(a_log, F32), H, G, N, 1e-6, N ** -0.5)
        ops.delta_scan(y, conv, 2 * G * N, kn, qn, kq, g, beta, state, q_start, slots, len(live), H, G, N, P)
        return y.cpu().numpy()

    got = in_portions(lengths, cuts, list(slots_of), run)
    for r in range(len(lengths)):
        assert_close(got[r], want[r], 2e-5, f"request {r} of {lengths[r]} tokens")
    return state, want


@pytest.mark.parametrize("H,G,N,P", [(4, 2, 24, 16), (2, 1, 8, 40), (3, 3, 20, 12), (2, 2, 64, 64), (2, 1, 70, 12), (1, 1, 130, 8), (1, 1, 1, 1), (6, 2, 128, 128)])
def test_gated_delta_rule_over_portions(H, G, N, P):
    """Portions of 1, 2, 17 and 40 tokens of three requests, requests sitting steps out, slots in another order."""
    state, _ = run_delta([70, 33, 1], [1, 2, 17, 1, 40], H, G, N, P)
    assert (state[[1, 3]] == 0).all() and (state[:, H * P * N :] == 0).all()


def test_delta_rule_keeps_a_far_token_and_a_freed_slot_starts_anew():
    """Token 1's value is written large; 300 tokens later, all decoded one by one, a query reads along its key: the
    output there is mostly that value.  Then the slot is zeroed and used by another request."""
    state, want = run_delta([402], [2] + [1] * 7, 2, 1, 16, 8, seed=5, boost=(1, 300), slots_of=(4,))
    assert np.abs(want[0][300]).max() > 5 * np.median(np.abs(want[0][250:299]).max(axis=1)), "the test's far token does not stand out"
    # the output 300 tokens later points along what token 1 wrote
    assert abs(np.corrcoef(want[0][300][:8], want[0][1][:8])[0, 1]) > 0.95
    assert float(state[4].abs().max()) > 0
    state[4].zero_()
    run_delta([3], [3], 2, 1, 16, 8, seed=6, state=state, slots_of=(4,))


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_squared_relu_in_the_products_epilogue(dtype):
    from alofa_b200.parts.linear import STORE, Linear

    rng = np.random.default_rng(4)
    for tokens, depth, width in ((5, 96, 72), (200, 128, 320), (130, 100, 70)):
        x = rounded(rng.standard_normal((tokens, depth)), dtype)
        w = rounded(rng.standard_normal((width, depth)) / np.sqrt(depth), dtype)
        out = torch.empty((tokens, width), dtype=dtype, device="cuda")
        Linear(dev(w, dtype), None, STORE, act="relu_squared")(out, dev(x, dtype))
        assert_close(out.float().cpu(), np.maximum(x @ w.T, 0.0) ** 2, KERNEL_TOL[dtype], f"tokens={tokens}")


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_group_norm_with_a_sigmoid_gate_and_one_weight_for_all_heads(dtype):
    from alofa_b200.csrc import ops

    rng = np.random.default_rng(5)
    n, H, P, eps, g_off = 6, 3, 40, 1e-4, 9
    y, gate, w = rounded(3 * rng.standard_normal((n, H * P)), F32), rounded(rng.standard_normal((n, H * P + 20)), F32), rounded(1 + 0.2 * rng.standard_normal(P), F32)
    out = torch.empty((n, H * P), dtype=dtype, device="cuda")
    ops.gated_group_norm(out, dev(y, F32), dev(gate, F32), g_off, dev(w, F32), H, eps, gate_first=False, sigmoid=True)
    o = y.reshape(n, H, P)
    want = (o / np.sqrt((o * o).mean(-1, keepdims=True) + eps) * w).reshape(n, H * P) * plain.sigmoid(gate[:, g_off : g_off + H * P])
    assert_close(out.float().cpu(), want, KERNEL_TOL[dtype], "gated norm")


def windowed_case(rng, lengths, H, G, d, dv, dims, base, dtype, page, standout=None):
    """Raw projections per request (biases already in) -> rotated queries and paged caches written by the kernel
    itself through scattered pages; plain q, k, v as the kernel holds them.  ``standout`` = (key, query): that key
    and that query of the longest request point the same way and are long, so that one score stands out."""
    from alofa_b200.csrc import ops

    blocks = [-(-n // page) for n in lengths]
    total = sum(blocks) + 3
    order = rng.permutation(total)
    table = np.full((len(lengths), max(blocks) + 1), -1, dtype=np.int32)
    k_cache = torch.full((total * page, G, d), 7.0, dtype=dtype, device="cuda")
    v_cache = torch.full((total * page, G, dv), -7.0, dtype=dtype, device="cuda")
    freq = plain.rotary_frequencies(dims, base)[0].astype(np.float32) if dims else None
    plains, queries, at = [], [], 0
    for r, n in enumerate(lengths):
        table[r, : blocks[r]] = order[at : at + blocks[r]]
        at += blocks[r]
        raw = rounded(rng.standard_normal((n, H * d + G * d + G * dv)), F32)
        if standout is not None and n == max(lengths):
            direction = rng.standard_normal(d - dims)  # in the part that is not turned: the score does not depend on the distance
            raw[standout[0], H * d + dims : H * d + d] = 5.0 * direction
            raw[standout[1], dims:d] = 5.0 * direction
        slot_map = np.array([table[r, j // page] * page + j % page for j in range(n)], dtype=np.int32)
        q = torch.empty((n, H * d), dtype=dtype, device="cuda")
        pos = np.arange(n, dtype=np.int32)
        ops.qkv_prepare(q, k_cache, v_cache, dev(raw, F32), dev(pos), dev(slot_map), H, G, d, dv, False, 0.0, 0.0, 1, dev(freq) if dims else None, dims)
        queries.append(q)
        pq = plain.rotate(raw[:, : H * d].reshape(n, H, d), pos, dims, base, "pairs")
        pk = plain.rotate(raw[:, H * d : (H + G) * d].reshape(n, G, d), pos, dims, base, "pairs")
        plains.append((rounded(pq, dtype), rounded(pk, dtype), rounded(raw[:, (H + G) * d :].reshape(n, G, dv), dtype)))
    return plains, queries, k_cache, v_cache, dev(table)


def run_windowed(queries, picks, k_cache, v_cache, table, page, H, G, d, dv, window, scale, dtype, sink=True):
    from alofa_b200.csrc import ops

    q = torch.cat([queries[r][picks[r]] for r in range(len(picks))]).contiguous()
    positions = dev(np.concatenate([np.array(p, dtype=np.int32) for p in picks]))
    seq = dev(np.concatenate([np.full(len(p), r, dtype=np.int32) for r, p in enumerate(picks)]))
    out = torch.empty((q.shape[0], H * dv), dtype=dtype, device="cuda")
    ops.paged_attention_generic(out, q, k_cache, v_cache, positions, seq, table, page, H, G, d, window, scale, 0.0, dv,
                                torch.zeros(H, dtype=F32, device="cuda") if sink else None)
    return out.float().cpu().numpy()


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("H,G,d,dv,dims,window", [(6, 3, 16, 8, 6, 21), (5, 5, 12, 12, 12, 16), (2, 1, 10, 30, 2, 40), (4, 2, 64, 64, 32, 4096), (2, 2, 24, 16, 8, 100), (3, 1, 40, 8, 0, 2)])
def test_windowed_attention_with_a_sink_over_paged_keys(dtype, H, G, d, dv, dims, window):
    """Prompts and decoding at lengths around page borders (16), the kernel's chunk borders (128) and the window's
    edge; a part of each head turned by the position; one added to the softmax's denominator."""
    rng = np.random.default_rng(9)
    lengths = sorted({1, 2, 15, 16, 17, 127, 128, 129, 300, window - 1, window, window + 1, 2 * window} - {0} - set(range(301, 10000)))
    page, scale, base = 16, 0.3, 500.0
    plains, queries, k_cache, v_cache, table = windowed_case(rng, lengths, H, G, d, dv, dims, base, dtype, page)
    want = [plain.attend(q, k, v, scale, window, sink=True).reshape(len(q), H * dv) for q, k, v in plains]
    for last_only in (False, True):
        picks = [[n - 1] if last_only else list(range(n)) for n in lengths]
        got, at = run_windowed(queries, picks, k_cache, v_cache, table, page, H, G, d, dv, window, scale, dtype), 0
        for r, p in enumerate(picks):
            assert_close(got[at : at + len(p)], want[r][p], KERNEL_TOL[dtype], f"request {r} ({lengths[r]} keys), decoding={last_only}")
            at += len(p)
    # without the sink the weights sum to one: the kernel's other form, on the same caches
    q, k, v = plains[-1]
    n = lengths[-1]
    got = run_windowed(queries, [[]] * (len(lengths) - 1) + [list(range(n))], k_cache, v_cache, table, page, H, G, d, dv, window, scale, dtype, sink=False)
    assert_close(got, plain.attend(q, k, v, scale, window, sink=False).reshape(n, H * dv), KERNEL_TOL[dtype], "no sink")


@pytest.mark.parametrize("H,G,d,dims,window,page", [(4, 2, 64, 32, 100, 64), (4, 1, 128, 64, 300, 64), (8, 2, 128, 128, 4096, 64), (3, 3, 32, 8, 70, 16), (6, 2, 64, 64, 257, 16),
                                                   (6, 2, 96, 40, 75, 64), (2, 2, 80, 80, 300, 16)])
def test_tensor_core_attention_with_a_sink(H, G, d, dims, window, page):
    """The bfloat16 kernels for keys and values of one size (whole prompts, prompt portions, single tokens with their
    keys in one split and in several that a second kernel merges): one added to the denominator against plain, other
    sink scores against the every-size kernel."""
    from alofa_b200.csrc import ops

    rng = np.random.default_rng(12)
    lengths = [1, 2, 63, 64, 65, 300, 700, window + 1 if window < 1000 else 129]
    scale = d ** -0.5
    plains, queries, k_cache, v_cache, table = windowed_case(rng, lengths, H, G, d, d, dims, 1e4, BF16, page)
    want = [plain.attend(q, k, v, scale, window, sink=True).reshape(len(q), H * d) for q, k, v in plains]
    kv_len = dev(np.array(lengths, dtype=np.int32))

    def run(picks, sink, split_keys=0):
        q = torch.cat([queries[r][picks[r]] for r in range(len(picks))]).contiguous()
        counts = [len(p) for p in picks]
        positions = dev(np.concatenate([np.array(p, dtype=np.int32) for p in picks]))
        q_start = dev(np.concatenate([[0], np.cumsum(counts)]).astype(np.int32))
        out = torch.empty_like(q)
        splits, po, pml = 0, None, None
        if split_keys:
            splits = -(-max(lengths) // split_keys)
            po = torch.empty(splits, q.shape[0] * H, d, device="cuda")
            pml = torch.empty(splits, q.shape[0] * H, 2, device="cuda")
        ops.attention_bf16(out, q, k_cache, v_cache, q_start, kv_len, positions, table, page, len(picks), max(counts), H, G, d, window, scale, splits, split_keys, po, pml,
                           max(lengths), sink=sink)
        return out.float().cpu().numpy()

    zero = torch.zeros(H, dtype=F32, device="cuda")
    other = dev(np.linspace(-3.0, 4.0, H).astype(np.float32))
    shapes = {"whole": ([list(range(n)) for n in lengths], 0), "portion": ([list(range(n // 2, n)) for n in lengths], 0), "last": ([[n - 1] for n in lengths], 0),
              "last in splits": ([[n - 1] for n in lengths], 256)}
    for what, (picks, split_keys) in shapes.items():
        got, at = run(picks, zero, split_keys), 0
        for r, p in enumerate(picks):
            assert_close(got[at : at + len(p)], want[r][p], KERNEL_TOL[BF16], f"{what}: request {r} ({lengths[r]} keys)")
            at += len(p)
        q = torch.cat([queries[r][picks[r]] for r in range(len(picks))]).contiguous()
        positions = dev(np.concatenate([np.array(p, dtype=np.int32) for p in picks]))
        seq = dev(np.concatenate([np.full(len(p), r, dtype=np.int32) for r, p in enumerate(picks)]))
        ref = torch.empty_like(q)
        ops.paged_attention_generic(ref, q, k_cache, v_cache, positions, seq, table, page, H, G, d, window, scale, 0.0, d, other)
        assert_close(run(picks, other, split_keys), ref.float().cpu().numpy(), KERNEL_TOL[BF16], f"{what}: other sink scores")
        assert np.abs(run(picks, other, split_keys) - got).max() > 0.02, "the sink's score does not show"


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("window", [3, 16, 17, 130, 600])
def test_a_key_just_inside_and_just_outside_the_window(dtype, window):
    """One key and one query of 700 point the same way.  The query sits ``window - 1`` tokens after the key (the last
    position that sees it) or ``window`` tokens after (the first that does not), in a prompt and decoded alone: seen,
    the output is nearly that key's value; not seen, it is not."""
    H, G, d, dv, dims, page, scale, n = 2, 1, 32, 16, 8, 16, 1.0, 700
    for key in (0, 5, 31, 64):
        for gap, seen in ((window - 1, True), (window, False)):
            query = key + gap
            rng = np.random.default_rng(10)
            plains, queries, k_cache, v_cache, table = windowed_case(rng, [n], H, G, d, dv, dims, 100.0, dtype, page, standout=(key, query))
            q, k, v = plains[0]
            want = plain.attend(q, k, v, scale, window, sink=True).reshape(n, H * dv)
            near = np.abs(want[query, :dv] - v[key, 0]).max() < 0.05 * np.abs(v[key, 0]).max()
            assert near == seen, f"the test's key {key} does not show at query {query} as it should (window {window})"
            whole = run_windowed(queries, [list(range(n))], k_cache, v_cache, table, page, H, G, d, dv, window, scale, dtype)
            assert_close(whole[query], want[query], KERNEL_TOL[dtype], f"prompt: key {key}, query {query}, window {window}")
            alone = run_windowed(queries, [[query]], k_cache, v_cache, table, page, H, G, d, dv, window, scale, dtype)
            assert_close(alone[0], want[query], KERNEL_TOL[dtype], f"decoded: key {key}, query {query}, window {window}")


def test_the_sink_takes_weight_from_a_first_token():
    """The first token sees itself alone: its output is v e^s / (1 + e^s), not v."""
    rng = np.random.default_rng(11)
    H, G, d, dv = 2, 2, 8, 4
    plains, queries, k_cache, v_cache, table = windowed_case(rng, [1], H, G, d, dv, 4, 10.0, F32, 16)
    q, k, v = plains[0]
    got = run_windowed(queries, [[0]], k_cache, v_cache, table, 16, H, G, d, dv, 5, 0.5, F32).reshape(H, dv)
    for h in range(H):
        e = np.exp(0.5 * float(q[0, h] @ k[0, h]))
        assert_close(got[h], v[0, h] * e / (1 + e), 1e-5, f"head {h}")
    assert np.abs(got - v[0]).max() > 0.05


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("H,dim,rot,dims,P,rank,window,scaling", [(3, 16, 8, 8, 24, 40, 9, (4.0, 64, 8.0, 1.0)), (1, 12, 4, 4, 20, 16, 2, (2.0, 16, 4.0, 0.5)),
                                                                   (4, 32, 32, 32, 32, 64, 70, (8.0, 128, 32.0, 1.0)), (2, 8, 16, 16, 16, 32, 130, (16.0, 256, 16.0, 2.0)),
                                                                   (2, 24, 16, 8, 8, 48, 33, None)])
def test_latent_attention_with_halves_paired_scaled_frequencies_and_a_head_gate(dtype, H, dim, rot, dims, P, rank, window, scaling):
    """The mixer's kernels in its order: latent rows normed, their shared key part turned and stored; queries turned and
    carried into the latent space; attention over the rows inside the window; values out of the latent; a gate per head."""
    from alofa_b200.csrc import ops

    rng = np.random.default_rng(12)
    lengths, page, eps, base, scale = sorted({1, 2, 17, window, window + 1, 2 * window + 3, 150}), 16, 1e-5, 300.0, 0.2
    sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    freq, mag = plain.rotary_frequencies(dims, base, sc)
    uk = rounded(rng.standard_normal((H * dim, rank)) / np.sqrt(rank), dtype)
    uv = rounded(rng.standard_normal((H * P, rank)) / np.sqrt(rank), dtype)
    norm_w = rounded(1 + 0.2 * rng.standard_normal(rank), F32)
    uk_t = dev(uk.reshape(H, dim, rank).transpose(0, 2, 1), dtype)
    blocks = [-(-n // page) for n in lengths]
    order = rng.permutation(sum(blocks) + 2)
    table = np.full((len(lengths), max(blocks) + 1), -1, dtype=np.int32)
    cache = torch.full(((sum(blocks) + 2) * page, rank + rot), 5.0, dtype=dtype, device="cuda")
    at = 0
    for r, n in enumerate(lengths):
        table[r, : blocks[r]] = order[at : at + blocks[r]]
        at += blocks[r]
        pos = np.arange(n, dtype=np.int32)
        lat = rounded(rng.standard_normal((n, rank + rot + H)) * 2, F32)  # [latent | shared key part | the gate's logits]
        q = rounded(rng.standard_normal((n, H, dim + rot)), dtype)
        slot_map = np.array([table[r, j // page] * page + j % page for j in range(n)], dtype=np.int32)
        ops.latent_prepare(None, cache, dev(lat, F32), None, dev(norm_w, F32), dev(freq.astype(np.float32)), dev(pos), dev(slot_map), 0, rank, rot, dims, eps, True, mag)
        c = rounded(plain.rms_norm(lat[:, :rank], norm_w, eps), dtype)
        kr = rounded(plain.rotate(lat[:, rank : rank + rot].reshape(n, 1, rot), pos, dims, base, "halves", sc), dtype)
        got_rows = cache.float().cpu().numpy()[slot_map]
        # angles are fp32 in the kernel: at position p the angle carries an error of about p * 6e-8
        assert_close(got_rows, np.concatenate([c, kr[:, 0]], axis=-1), KERNEL_TOL[dtype], f"rows of request {r}")
        qd = dev(q.reshape(n, -1), dtype)
        qa = torch.zeros((n, H * (rank + rot)), dtype=dtype, device="cuda")
        ops.latent_query_turn(qa, qd, dev(freq.astype(np.float32)), dev(pos), H, dim, rot, dims, rank, True, mag)
        ops.gemm_batched(qa, qd, uk_t, H, n, rank, dim, H * (dim + rot), dim + rot, dim, rank * dim, H * (rank + rot), rank + rot)
        o_lat = torch.empty((n, H * rank), dtype=dtype, device="cuda")
        ops.latent_attention(o_lat, qa, cache, None, dev(pos), dev(np.zeros(n, dtype=np.int32)), dev(table[r : r + 1]), page, H, rank, rot, window, scale)
        o = torch.empty((n, H * P), dtype=dtype, device="cuda")
        ops.gemm_batched(o, o_lat, dev(uv, dtype), H, n, P, rank, H * rank, rank, rank, P * rank, H * P, P)
        ops.head_gate(o, dev(lat, F32), rank + rot, H, P)
        qr = plain.rotate(q[:, :, dim:], pos, dims, base, "halves", sc)
        qq = np.concatenate([q[:, :, :dim], qr], axis=-1)
        kk = np.concatenate([(c @ uk.T).reshape(n, H, dim), np.repeat(kr, H, axis=1)], axis=-1)
        want = plain.attend(qq, kk, (c @ uv.T).reshape(n, H, P), scale, window, sink=False) * plain.sigmoid(lat[:, rank + rot :])[:, :, None]
        assert_close(o.float().cpu().numpy().reshape(n, H, P), want, KERNEL_TOL[dtype] * (3 if dtype == BF16 else 1), f"request {r} of {n} tokens")


# ---------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------
LENGTHS = {"A": [1, 2, 23, 64, 65, 129, 200], "B": [3, 16, 17, 33, 80, 131], "C": [5, 64, 190, 257], "D": [2, 63, 150, 300], "E": [4, 76, 140, 330]}
DECODED = 12


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("dibulix_gpu")
    return {name: tiny.write(base / name, name, seed=10 + i) for i, name in enumerate(tiny.CONFIGS)}


def make_requests(name):
    reqs, prompts = {}, {}
    for i, n in enumerate(LENGTHS[name]):
        reqs[f"r{i}"] = tiny.tokens(name, n + DECODED, seed=i)
        prompts[f"r{i}"] = n
    return reqs, prompts


@pytest.fixture(scope="module")
def plain_logits(folders):
    out = {}
    for name, folder in folders.items():
        w, cfg = plain.load(folder)
        out[name] = {rid: plain.forward(w, cfg, toks) for rid, toks in make_requests(name)[0].items()}
    return out


def runner_for(folder, dtype, block, pages, max_requests=8, graphs=True):
    from alofa_b200.engine.loading import load_model
    from alofa_b200.engine.step import StepRunner

    model, *_ = load_model(folder, dtype)
    return StepRunner(model, block_size=block, num_pages=pages, max_requests=max_requests, max_tokens=pages * block, max_step_tokens=512, cuda_graphs=graphs)


def compare(steps, outputs, want, vocab, tol, what):
    got = replay.collect(steps, outputs, vocab)
    for rid, rows in got.items():
        ref = want[rid][: len(rows)]
        assert rows.shape == ref.shape, f"{what} {rid}: {rows.shape} vs {ref.shape}"
        err = np.abs(rows - ref).max(axis=-1) / max(1.0, float(np.abs(ref).max()))
        # rounding to bfloat16 now and then moves one position several times as far as most (a gate or a softmax near a
        # tie); a key, a state or a window that is wrong moves many positions by order one
        assert np.quantile(err, 0.9) <= tol / 3 and err.max() <= (tol if tol < 1e-3 else 3 * tol), (
            f"{what} {rid}: position {int(err.argmax())} differs by {err.max():.3e}, nine in ten by at most {np.quantile(err, 0.9):.3e} (limit {tol:.1e})")
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_whole_decoded_portions_and_mixed_batches(folders, plain_logits, name, dtype):
    """The same requests whole, with the last tokens decoded one by one, in portions down to two tokens, and mixed
    (portions beside single tokens, four live at most) in a pool that holds two of the longest: pages and slots are
    given back and used again.  Every position against plain."""
    reqs, prompts = make_requests(name)
    vocab = tiny.CONFIGS[name]["vocab"]
    block = 16 if name in ("B", "D") else 64
    per_request = -(-max(len(t) for t in reqs.values()) // block)
    schedules = {
        "whole": (replay.whole(reqs), per_request),
        "decoded": (replay.tail_decoded(reqs, tail=DECODED + 20), per_request),
        "portions": (replay.portions(reqs), per_request),
        "mixed": (replay.mixed(reqs, prompts, 2 * per_request * block + block, block, seed=3), 2 * per_request + 1),
    }
    for what, (steps, pages) in schedules.items():
        runner = runner_for(folders[name], dtype, block, pages, max_requests=4)
        out = replay.run_inprocess(runner, steps)
        compare(steps, out, plain_logits[name], vocab, TOL[dtype], f"{name}/{dtype}/{what}")
        assert set(runner.manager.free_pages()) == {pages} and runner.manager.live_requests() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_long_decoding_from_the_first_token(folders, name, dtype):
    """One prompt token, then 170 tokens one by one (past page borders and past every window of the configuration),
    two requests side by side that started 40 steps apart; decode steps are replayed as graphs."""
    from alofa_b200.engine.step import StepEntry

    w, cfg = plain.load(folders[name])
    a, b = tiny.tokens(name, 171, seed=50), tiny.tokens(name, 131, seed=51)
    want_a, want_b = plain.forward(w, cfg, a), plain.forward(w, cfg, b)
    runner = runner_for(folders[name], dtype, 16, 22, max_requests=2)
    sa, sb = runner.admit(0), None
    for i in range(171):
        entries = [StepEntry(sa, [a[i]], [0])]
        if i >= 40:
            if sb is None:
                sb = runner.admit(1)
            entries.append(StepEntry(sb, [b[i - 40]], [0]))
        rows = runner.forward(entries).float().cpu().numpy()
        assert_close(rows[0], want_a[i], TOL[dtype], f"first request, token {i}")
        if i >= 40:
            assert_close(rows[1], want_b[i - 40], TOL[dtype], f"second request, token {i - 40}")
    runner.check_status()
    assert runner.manager.defects() == 0


def test_batches_and_cuts_do_not_change_a_request(folders):
    """float32: a request's logits in portions and in a mixed batch equal, to rounding of the sums' order, those it gets alone and whole."""
    name = "D"
    reqs, prompts = make_requests(name)
    vocab = tiny.CONFIGS[name]["vocab"]
    alone = replay.collect(replay.whole(reqs), replay.run_inprocess(runner_for(folders[name], "float32", 16, 20), replay.whole(reqs)), vocab)
    for what, steps, pages in (("portions", replay.portions(reqs), 20), ("mixed", replay.mixed(reqs, prompts, 700, 16, seed=9), 44)):
        other = replay.collect(steps, replay.run_inprocess(runner_for(folders[name], "float32", 16, pages, max_requests=4), steps), vocab)
        for rid in reqs:
            assert np.abs(alone[rid] - other[rid]).max() <= 5e-6 * max(1.0, np.abs(alone[rid]).max()), f"{what} {rid}"


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_the_stream_after_every_layer(folders, name):
    """float32: the streams' sum after each layer (the write a layer's last sublayer leaves owed is done here, on a copy)."""
    import alofa_b200.parts.block as block
    from alofa_b200.engine.step import StepEntry

    w, cfg = plain.load(folders[name])
    ids = tiny.tokens(name, 30, seed=77)
    want = []
    plain.forward(w, cfg, ids, layer_outputs=want)
    seen, original = [], block.HyperResidual.forward

    def recording(self, ctx, h, cache, writes=True):
        original(self, ctx, h, cache, writes)
        xs = ctx.streams.double().cpu().numpy()
        if ctx.streams_owed is not None:
            y, w_out, w_mix = (t.double().cpu().numpy() for t in ctx.streams_owed)
            xs = np.stack(plain.connect(list(xs), y, w_mix.reshape(len(xs), len(xs)), w_out))
        seen.append(xs.sum(axis=0))

    block.HyperResidual.forward = recording
    try:
        runner = runner_for(folders[name], "float32", 64, 1, graphs=False)
        runner.forward([StepEntry(runner.admit(0), ids, [0])])
    finally:
        block.HyperResidual.forward = original
    assert len(seen) == len(want) == len(cfg["layers"])
    for k, (got, ref) in enumerate(zip(seen, want)):
        assert_close(got, ref, TOL["float32"], f"after layer {k}")  # the logits' own limit: a layer's stream carries the same rounding


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_greedy_generation_through_the_engine(folders, name):
    """Engine.generate (scheduler, chunked prefill, decode graphs): float32 tokens equal plain greedy; bfloat16 tokens
    are each within rounding of the plain maximum."""
    from alofa_b200.engine.engine import Engine

    w, cfg = plain.load(folders[name])
    prompts = [tiny.tokens(name, n, seed=200 + i) for i, n in enumerate([1, 7, 40, 90, 18])]
    want = [plain.greedy(w, cfg, p, 6) for p in prompts]
    eng = Engine(str(folders[name]), dtype="float32", block_size=16, max_batch=3, token_budget=48, max_chunk=32, max_tokens=128)
    assert eng.generate(prompts, max_new_tokens=6) == want
    assert eng.stats()["defects"] == 0
    eng16 = Engine(str(folders[name]), dtype="bfloat16", block_size=16, max_batch=3, token_budget=48, max_chunk=32, max_tokens=128)
    for p, out in zip(prompts, eng16.generate(prompts, max_new_tokens=6)):
        seq = list(p)
        for tok in out:
            row = plain.forward(w, cfg, seq)[-1]
            assert row.max() - row[tok] <= 8e-2 * max(1.0, float(np.abs(row).max())), "a bfloat16 token is not near the plain maximum"
            seq.append(tok)
    eng16.runner.check_status()


def test_the_programs_take_the_architecture(folders, tmp_path):
    """bin/trace_run replays a schedule and bin/generate generates, both choosing the model by config.json."""
    name = "C"
    reqs, _ = make_requests(name)
    reqs = {k: reqs[k] for k in ("r0", "r2")}
    w, cfg = plain.load(folders[name])
    want = {rid: plain.forward(w, cfg, t) for rid, t in reqs.items()}
    steps = replay.portions(reqs, sizes=(40, 2, 3, 64, 1))
    out = replay.run_trace_program(folders[name], "float32", steps, tmp_path / "out", 512)
    compare(steps, out, want, cfg["vocab"], TOL["float32"], "trace_run")
    prompt = tiny.tokens(name, 12, seed=5)
    done = subprocess.run([sys.executable, str(replay.ROOT / "bin" / "generate"), "--model", str(folders[name]), "--dtype", "float32", "--prompt-ids",
                           ",".join(map(str, prompt)), "--max-new-tokens", "5", "--max-tokens", "64", "--json"], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert json.loads(done.stdout.strip().splitlines()[-1])["out_ids"] == [plain.greedy(w, cfg, prompt, 5)]
