#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--shape 0.5b|1.5b|7b] [--no-extra]
    python bench.py --design kotutar [--size 1k|2k]     (another line: that design beside Qwen2 at equal layer sizes)
    python bench.py --design darolix [--size 1k|2k]     (another line: that design beside Kotutar at equal layer sizes)
    python bench.py --design dibulix [--size 1k|2k]     (another line: that design beside Darolix at equal layer sizes)
    python bench.py --design kikerax [--size 1k|2k]     (another line: that design beside Darolix at equal layer sizes)

The default run has the layer sizes of the Qwen2.5-0.5B shape with random
weights, a batch of 8 requests with 2,048-token prompts inside a 4,096-token
context, and times K decode steps on the device after W warm-up steps.  One
JSON line is printed:

* ``value``: decoded tokens per second at the default batch (device time of K
  steps of the engine's own step function, CUDA events);
* ``e2e``: the same through ``Engine.generate`` (host token ids in, host token
  ids out, every step copying its inputs to the device and its tokens back);
* ``prefill``: one 2,048-token prompt in one step;
* ``roofline``: bytes a decode step has to read (every weight once, the cache
  of the live requests) over its time, against the measured copy bandwidth;
* ``points``: decode at batch 1 and 64, and, unless ``--no-extra``, the other
  measurements: decode at batch 8 and 64 with prompts that fill the 4,096-token
  context; the Qwen2.5-1.5B shape serving 64 requests with prompt lengths
  uniform in [128, 2048] and 256 new tokens each through ``Engine.generate``
  (scheduler included); the Qwen2.5-7B shape at batch 1, 8 and 64 and its
  2,048-token prefill.  ``points_detail`` gives each point's time per step
  (median, min, max over the steps, each step timed by its own event pair), its
  fraction of the roofline from the same formula, and the scheduler's counts.

Method, after the reference's own benchmark (src/alofa/cli.mojo:62-82,
819-850): warm-up first, then every repetition timed on its own and the median
reported with the span; ``value`` itself is the time of K steps
between one pair of events.

Peaks come from MEASURED_PEAKS.json beside this file when present, else from
the fallback figures 6.65 TB/s and 1.59 PFLOP/s.  Every decode step reads more
than a gigabyte of weights and cache, far more than the 126 MB L2, so no L2
flush is needed between steps (``config.l2``)."""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "decode tok/s @ batch 8 (Qwen2.5-0.5B shape, 2,048-token prompts, context 4096)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}

# the shapes the measurements are quoted on (their published config.json values)
SHAPES = {
    "0.5b": ("Qwen2.5-0.5B shape", dict(num_hidden_layers=24, hidden_size=896, num_attention_heads=14, num_key_value_heads=2, head_dim=64,
                                        intermediate_size=4864, vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True,
                                        max_position_embeddings=32768)),
    "1.5b": ("Qwen2.5-1.5B shape", dict(num_hidden_layers=28, hidden_size=1536, num_attention_heads=12, num_key_value_heads=2, head_dim=128,
                                        intermediate_size=8960, vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True,
                                        max_position_embeddings=32768)),
    "7b": ("Qwen2.5-7B shape", dict(num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
                                    intermediate_size=18944, vocab_size=152064, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False,
                                    max_position_embeddings=32768)),
}
SHAPE = SHAPES["0.5b"][1]
PROMPT_LEN = 2048
CONTEXT = 4096


def _find_number(raw, key):
    """The number under ``key`` anywhere in a nested JSON value (a figure may be
    a bare number or an object with a ``value``); None when absent."""
    if isinstance(raw, dict):
        if key in raw:
            v = raw[key]
            if isinstance(v, dict):
                v = v.get("value")
            try:
                return float(v)
            except (TypeError, ValueError):
                return None
        for v in raw.values():
            found = _find_number(v, key)
            if found is not None:
                return found
    elif isinstance(raw, list):
        for v in raw:
            found = _find_number(v, key)
            if found is not None:
                return found
    return None


def peaks() -> tuple:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            raw = json.loads(path.read_text())
        except ValueError:
            raw = None
        hbm = _find_number(raw, "hbm_gbs")
        # the prefill is timed over a few milliseconds: the burst figure is its denominator
        flops = _find_number(raw, "bf16_tflops") or _find_number(raw, "bf16_tflops_sustained")
        if hbm and flops:
            return {"hbm_gbs": hbm, "bf16_tflops": flops}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while timing."""

    QUERY = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self):
        self.samples = []
        self.proc = None
        self.begin = 0.0

    def start(self):
        """Start sampling; nvidia-smi takes a moment to give its first line, so
        this goes before the warm-up and :meth:`mark` before the timed steps."""
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append((time.perf_counter(), parts))

    def mark(self):
        """The timed region starts now: only samples from here on count."""
        self.begin = time.perf_counter()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, reasons, max_mhz = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for at, s in self.samples:
            if at < self.begin:
                continue
            try:
                clocks.append(int(s[0]))
                max_mhz = int(s[1])
            except ValueError:
                continue
            for name, flag in zip(names, s[2:]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(clocks)) if clocks else None, "sm_max_mhz": max_mhz, "reasons": sorted(reasons), "samples": len(clocks)}


def model_numbers(cfg, layers: int) -> dict:
    """Bytes a decode step reads and flops a prefill does, from the sizes."""
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    per_layer_params = H * (q + 2 * kv) + (q + 2 * kv) + q * H + 3 * H * I + 2 * H
    weight_bytes = 2 * (layers * per_layer_params + V * H + H)  # bf16; the head (tied table) is read once
    kv_bytes_per_token = layers * 2 * kv * 2
    return {"weight_bytes": weight_bytes, "kv_bytes_per_token": kv_bytes_per_token, "per_layer_matmul_params": H * (q + 2 * kv) + q * H + 3 * H * I, "q": q}


def prefill_flops(cfg, layers: int, tokens: int, numbers: dict) -> float:
    gemm = 2.0 * tokens * layers * numbers["per_layer_matmul_params"]
    attn = layers * 4.0 * numbers["q"] * tokens * (tokens + 1) / 2
    head = 2.0 * cfg.hidden_size * cfg.vocab_size
    return gemm + attn + head


class Bench:
    """One engine of one shape and the measurements made on it."""

    def __init__(self, shape: str, layers: int, max_batch: int, context: int = CONTEXT):
        import numpy as np

        from alofa_b200.engine.engine import Engine
        from alofa_b200.models.qwen2 import NAME, Qwen2Config

        self.label, values = SHAPES[shape]
        values = dict(values)
        self.full_layers = values["num_hidden_layers"]
        values["num_hidden_layers"] = layers or self.full_layers
        self.cfg = Qwen2Config(**values)
        self.layers = self.cfg.num_hidden_layers
        self.engine = Engine.from_random(NAME, self.cfg, seed=0, dtype="bfloat16", generate_on_device=True, block_size=64, max_batch=max_batch,
                                         max_tokens=context, token_budget=PROMPT_LEN + max_batch, max_chunk=PROMPT_LEN)
        self.runner = self.engine.runner
        self.numbers = model_numbers(self.cfg, self.layers)
        self.peaks, self.peaks_kind = peaks()
        self.rng = np.random.default_rng(0)

    def prompt(self, n: int) -> list:
        return [int(t) for t in self.rng.integers(0, self.cfg.vocab_size, size=n)]

    @staticmethod
    def timed_each(fn, reps: int) -> tuple:
        """(mean ms over one pair of events around all repetitions, [ms of each
        repetition by its own pair of events])."""
        import torch

        marks = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
        torch.cuda.synchronize()
        marks[0].record()
        for i in range(reps):
            fn()
            marks[i + 1].record()
        torch.cuda.synchronize()
        each = [marks[i].elapsed_time(marks[i + 1]) for i in range(reps)]
        return marks[0].elapsed_time(marks[reps]) / reps, each

    @staticmethod
    def spread(each: list) -> dict:
        return {"median": round(statistics.median(each), 4), "min": round(min(each), 4), "max": round(max(each), 4), "n": len(each)}

    def prefill(self, warmup: int, reps: int = 10) -> dict:
        """One 2,048-token prompt in one step, `reps` times; the median."""
        from alofa_b200.engine.step import StepEntry

        tokens = self.prompt(PROMPT_LEN)

        def one():
            slot = self.runner.admit(10_000)
            self.runner.forward_logits([StepEntry(slot, tokens, (PROMPT_LEN - 1,))])
            self.runner.release(slot)

        for _ in range(max(3, warmup)):  # a shape met a third time is recorded as a graph: time what serving replays
            one()
        _, each = self.timed_each(one, reps)
        ms = statistics.median(each)
        flops = prefill_flops(self.cfg, self.layers, PROMPT_LEN, self.numbers)
        return {"value": round(PROMPT_LEN / ms * 1e3, 1), "tokens": PROMPT_LEN, "ms": round(ms, 4),
                "frac": round(flops / (ms * 1e-3) / (self.peaks["bf16_tflops"] * 1e12), 4), "reps": self.spread(each)}

    def decode(self, batch: int, steps: int, warmup: int, prompt_len: int = PROMPT_LEN, clocks=None) -> dict:
        """`steps` decode steps of `batch` requests whose prompts of `prompt_len`
        tokens were run first, one request per step."""
        import torch

        from alofa_b200.csrc import ops
        from alofa_b200.engine.step import StepEntry

        runner = self.runner
        slots = [runner.admit(20_000 + i) for i in range(batch)]
        for s in slots:
            toks = self.prompt(prompt_len)
            for lo in range(0, prompt_len, PROMPT_LEN):
                runner.forward_logits([StepEntry(s, toks[lo : lo + PROMPT_LEN], ())])
        feed = self.rng.integers(0, self.runner.model.spec.vocab_size, size=(steps + warmup, batch))
        state = {"i": 0}

        def one_step():
            toks = feed[state["i"]]
            state["i"] += 1
            runner.forward_sampled([StepEntry(s, (int(t),), (0,)) for s, t in zip(slots, toks)])

        if clocks:
            clocks.start()
        for _ in range(warmup):
            one_step()
        if clocks:
            torch.cuda.synchronize()
            time.sleep(0.3)  # the sampler's first lines
            clocks.mark()
        launches0 = ops.launch_count()
        ms, each = self.timed_each(one_step, steps)
        clock_report = clocks.stop() if clocks else None
        launches = ops.launch_count() - launches0
        mean_kv = prompt_len + warmup + steps / 2
        for s in slots:
            runner.release(s)
        step_bytes = self.numbers["weight_bytes"] + self.numbers["kv_bytes_per_token"] * mean_kv * batch + self.numbers.get("state_bytes_per_request", 0) * batch
        achieved = step_bytes / (ms * 1e-3) / 1e9
        return {"ms": ms, "tok_s": batch / ms * 1e3, "bytes": step_bytes, "launches": launches, "clocks": clock_report, "step_ms": self.spread(each),
                "gbs": achieved, "frac": achieved / self.peaks["hbm_gbs"]}

    def detail(self, point: dict) -> dict:
        return {"tok_s": round(point["tok_s"], 1), "ms_per_step": round(point["ms"], 4), "step_ms": point["step_ms"],
                "hbm_gbs": round(point["gbs"], 1), "hbm_frac": round(point["frac"], 4)}

    def serve(self, n_requests: int, new_tokens: int, lo: int, hi: int) -> dict:
        """`n_requests` with prompt lengths uniform in [lo, hi] and `new_tokens`
        new tokens each through Engine.generate, scheduler included; run once
        untimed (records the graphs), then timed by the wall clock."""
        engine = self.engine
        prompts = [self.prompt(int(n)) for n in self.rng.integers(lo, hi + 1, size=n_requests)]
        engine.generate(prompts, max_new_tokens=new_tokens)
        engine.marks.clear()
        before = dict(engine.counters)
        for key in engine.timings:
            engine.timings[key].clear()
        t0 = time.perf_counter()
        outs = engine.generate(prompts, max_new_tokens=new_tokens)
        wall = time.perf_counter() - t0
        made = sum(len(o) for o in outs)
        by_rows = {}
        for _, kind, rows in engine.marks:
            bucket = kind + ":" + ("1-16" if rows <= 16 else "17-64" if rows <= 64 else "65-512" if rows <= 512 else "513+")
            by_rows[bucket] = by_rows.get(bucket, 0) + 1
        stats = engine.stats()
        return {"tok_s": round(made / wall, 1), "wall_s": round(wall, 3), "requests": n_requests, "new_tokens": made,
                "prompt_tokens": sum(len(p) for p in prompts), "ticks": stats["ticks"] - before["ticks"],
                "preemptions": stats["preempt_total"], "steps_by_rows": by_rows,
                "decode_step_ms_median": round(statistics.median(engine.timings["decode_ms"]), 4) if engine.timings["decode_ms"] else None}

    def close(self) -> None:
        import gc

        import torch

        self.engine.close()
        self.engine = self.runner = None
        gc.collect()
        torch.cuda.empty_cache()


def extra_points(args, first: Bench) -> tuple:
    """The measurements beside the headline; each guarded, so that a failure of
    one is reported under its own name and costs nothing else."""
    points, detail = {}, {}

    def guarded(name, fn):
        try:
            fn()
        except Exception as err:  # noqa: BLE001 - reported in the line, never fatal to the headline
            detail[name] = {"error": f"{type(err).__name__}: {err}"[:300]}

    steps = max(64, args.steps // 2)

    def long_context():
        fill = CONTEXT - steps - args.warmup - 8  # prompts that leave room for the timed steps only
        for batch in (8, 64):
            point = first.decode(batch, steps, args.warmup, prompt_len=fill)
            points[f"decode_b{batch}_ctx4096"] = round(point["tok_s"], 1)
            detail[f"decode_b{batch}_ctx4096"] = dict(first.detail(point), prompt_len=fill)

    guarded("decode_ctx4096", long_context)
    first.close()

    def shape_15b():
        bench = Bench("1.5b", 0, 64)
        try:
            served = bench.serve(64, 256, 128, 2048)
            points["qwen2.5-1.5b_serve64_tok_s"] = served["tok_s"]
            detail["qwen2.5-1.5b_serve64"] = served
            point = bench.decode(8, steps, args.warmup)
            points["qwen2.5-1.5b_decode_b8"] = round(point["tok_s"], 1)
            detail["qwen2.5-1.5b_decode_b8"] = bench.detail(point)
        finally:
            bench.close()

    def shape_7b():
        bench = Bench("7b", 0, 64)
        try:
            for batch in (1, 8, 64):
                point = bench.decode(batch, steps, args.warmup)
                points[f"qwen2.5-7b_decode_b{batch}"] = round(point["tok_s"], 1)
                detail[f"qwen2.5-7b_decode_b{batch}"] = bench.detail(point)
            pre = bench.prefill(args.warmup)
            points["qwen2.5-7b_prefill_tok_s"] = pre["value"]
            detail["qwen2.5-7b_prefill"] = pre
        finally:
            bench.close()

    guarded("qwen2.5-1.5b", shape_15b)
    guarded("qwen2.5-7b", shape_7b)
    return points, detail


def run(args) -> dict:
    from alofa_b200.engine.context import Layout

    bench = Bench(args.shape, args.layers, max(64, args.batch))
    cfg, layers, engine, runner = bench.cfg, bench.layers, bench.engine, bench.runner

    if args.phase == "decode":
        prefill = None
    else:
        prefill = bench.prefill(args.warmup)
    if args.phase == "prefill":
        print(json.dumps({"phase": "prefill", "ms": prefill["ms"], "tok_s": prefill["value"], "reps": prefill["reps"]}))
        raise SystemExit(0)

    main = bench.decode(args.batch, args.steps, args.warmup, clocks=ClockSampler())
    if args.phase == "decode":
        print(json.dumps({"phase": "decode", "batch": args.batch, "ms_per_step": main["ms"], "tok_s": main["tok_s"], "launches": main["launches"], "step_ms": main["step_ms"]}))
        raise SystemExit(0)
    b1 = bench.decode(1, max(8, args.steps // 2), args.warmup)
    b64 = bench.decode(64, max(8, args.steps // 2), args.warmup)

    # -- end to end: Engine.generate, host tokens in and out --------------------
    # as many new tokens as timed steps: the requests start and end a tick apart each, so a short
    # run is mostly steps with fewer rows than the batch
    e2e_new = max(8, min(256, args.steps))
    prompts = [bench.prompt(PROMPT_LEN) for _ in range(args.batch)]
    engine.generate(prompts, max_new_tokens=e2e_new)  # the same run once untimed: records the CUDA graphs it uses
    engine.marks.clear()
    rows_before = engine.counters["decode_rows"]
    t0 = time.perf_counter()
    outs = engine.generate(prompts, max_new_tokens=e2e_new)
    wall = time.perf_counter() - t0
    # wall clock of the decoding part: from the arrival of the last step that held a prompt portion
    # to the arrival of the last tokens, scheduler and bookkeeping included
    last_prefill = max((t for t, kind, _ in engine.marks if kind == "prefill"), default=t0)
    decode_wall = max((t for t, kind, _ in engine.marks if kind == "decode"), default=last_prefill) - last_prefill
    decode_rows = sum(rows for t, kind, rows in engine.marks if kind == "decode" and t > last_prefill)
    assert decode_rows <= engine.counters["decode_rows"] - rows_before
    e2e_value = decode_rows / decode_wall if decode_wall > 0 else None

    h2d = Layout.make(args.batch, args.batch, args.batch, runner._group_shapes).total * 4
    points = {"decode_b1": round(b1["tok_s"], 1), "decode_b64": round(b64["tok_s"], 1)}
    detail = {"decode_b1": bench.detail(b1), f"decode_b{args.batch}": bench.detail(main), "decode_b64": bench.detail(b64)}
    if args.extra and args.shape == "0.5b" and not args.layers:
        more_points, more_detail = extra_points(args, bench)
        points.update(more_points)
        detail.update(more_detail)
    metric = METRIC if args.shape == "0.5b" else METRIC.replace("Qwen2.5-0.5B shape", bench.label)
    result = {
        "metric": metric, "value": round(main["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights, uniform random token ids", "impl": "alofa_b200",
        "config": {
            "model": bench.label, "layers": layers, "layers_full": bench.full_layers, "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "global_batch": args.batch, "prompt_len": PROMPT_LEN, "seq_len": CONTEXT, "block_size": 64, "parallelism": "single GPU",
            "l2": "inputs>L2 (each step reads >1 GB)", "peaks": bench.peaks_kind,
        },
        "e2e": {"value": round(e2e_value, 1) if e2e_value else None, "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch + 4,
                "new_tokens": e2e_new, "wall_s_with_prefill": round(wall, 3), "outputs": len(outs)},
        "gpu_launches": main["launches"],
        "prefill": {k: v for k, v in prefill.items() if k != "reps"},
        "roofline": {"bound": "hbm", "achieved": round(main["gbs"], 1), "peak": bench.peaks["hbm_gbs"], "unit": "GB/s", "frac": round(main["frac"], 4)},
        "points": points,
        "step_ms": main["step_ms"],
        "prefill_reps": prefill["reps"],
        "points_detail": detail,
        "clocks": main["clocks"],
    }
    return result


# ---------------------------------------------------------------------------------------------------
# --design kotutar: the latent-attention design beside the Qwen2 design at equal layer sizes
# ---------------------------------------------------------------------------------------------------
# Layer sizes after published latent-attention models with routed feed-forwards (random weights):
# width, heads, unrotated / rotated / value size per head, latent ranks, dense and expert widths.
DESIGN_SIZES = {
    "1k": dict(width=1024, heads=8, dim=64, rot=32, vdim=64, kv_rank=256, q_rank=512, ff=4096, experts=16, top=2, expert_ff=512, shared_ff=1024, vocab=32000, layers=4),
    "2k": dict(width=2048, heads=16, dim=128, rot=64, vdim=128, kv_rank=512, q_rank=1536, ff=8192, experts=64, top=6, expert_ff=1408, shared_ff=2816, vocab=32000, layers=4),
}


# --design darolix: state-space / attention + linear-attention layers with routed experts, beside the Kotutar design at the
# same width, layers, heads, experts and expert width.  Inner sizes after published models of the kind: the state-space
# inner size twice the width in heads of 64 with a state of 128, attention heads of 128, linear attention with keys half and
# values as wide as the model.
DAROLIX_SIZES = {
    "1k": dict(ssm_heads=32, ssm_vdim=64, state=128, groups=1, conv=4, norm_groups=1, kv_heads=2, att_dim=128, gla_heads=4, gla_dim=128, gla_vdim=256, identity=2),
    "2k": dict(ssm_heads=64, ssm_vdim=64, state=128, groups=1, conv=4, norm_groups=1, kv_heads=4, att_dim=128, gla_heads=8, gla_dim=128, gla_vdim=256, identity=4),
}


def darolix_config(z: dict, d: dict):
    """State-space and side-by-side layers in turn, every layer with routed experts, no loop."""
    from alofa_b200.models.darolix import DarolixConfig, DarolixLayer, LeftConfig, MoeConfig, RightConfig, StateSpaceConfig

    ssm = StateSpaceConfig(d["ssm_heads"], d["ssm_vdim"], d["state"], d["groups"], d["conv"], d["norm_groups"])
    pair = (LeftConfig(z["heads"], d["kv_heads"], d["att_dim"], d["att_dim"], d["att_dim"] ** -0.5, 50.0, 0.3, 128), RightConfig(d["gla_heads"], d["gla_dim"], d["gla_vdim"], 16.0))
    moe = MoeConfig(z["experts"], z["top"], z["expert_ff"], d["identity"])
    layers = [DarolixLayer("mamba2", ssm, moe) if i % 2 == 0 else DarolixLayer("parallel", pair, moe) for i in range(z["layers"])]
    return DarolixConfig(z["vocab"], z["width"], 1e-6, float(z["width"]) ** 0.5, layers)


def kotutar_config_routed(z: dict):
    """The closest existing design at equal size: latent attention and routed experts (no shared one) in every layer."""
    from alofa_b200.models.kotutar import KotutarConfig, KotutarLayer, LatentMixerConfig, MlpConfig

    mixer = LatentMixerConfig(z["heads"], z["dim"], z["rot"], z["vdim"], z["kv_rank"], z["q_rank"], (z["dim"] + z["rot"]) ** -0.5, 1e4, z["rot"])
    return KotutarConfig(z["vocab"], z["width"], 1e-6, [KotutarLayer("latent_attention", mixer, MlpConfig("moe", z["expert_ff"], z["experts"], z["top"], 0)) for _ in range(z["layers"])])


def kotutar_config(z: dict):
    """Half of the layers dense, half routed, no loop: what a step costs per layer is what is measured."""
    from alofa_b200.models.kotutar import KotutarConfig, KotutarLayer, LatentMixerConfig, MlpConfig

    mixer = LatentMixerConfig(z["heads"], z["dim"], z["rot"], z["vdim"], z["kv_rank"], z["q_rank"], (z["dim"] + z["rot"]) ** -0.5, 1e4, z["rot"])
    layers = [KotutarLayer("latent_attention", mixer, MlpConfig("dense", z["ff"]) if i % 2 == 0 else MlpConfig("moe", z["expert_ff"], z["experts"], z["top"], z["shared_ff"]))
              for i in range(z["layers"])]
    return KotutarConfig(z["vocab"], z["width"], 1e-6, layers)


def qwen2_config_like(z: dict):
    """The closest existing design at equal size: same width, layers, heads, head size, vocabulary and feed-forward width; 2 KV heads."""
    from alofa_b200.models.qwen2 import Qwen2Config

    return Qwen2Config(num_hidden_layers=z["layers"], hidden_size=z["width"], num_attention_heads=z["heads"], num_key_value_heads=2, head_dim=z["width"] // z["heads"],
                       intermediate_size=z["ff"], vocab_size=z["vocab"], rms_norm_eps=1e-6, rope_theta=1e4, tie_word_embeddings=False, max_position_embeddings=32768)


# --design dibulix: gated-delta-rule, latent-attention and attention + minGRU layers over four residual streams, every layer
# with a dense feed-forward (squared relu), beside the Darolix design at the same width, layers, heads and vocabulary.  Inner
# sizes after published models of the kind: the delta rule with keys half and values as wide as the model in heads of 128 x
# 256 and low-rank maps of 16 for decays and gate; the latent attention of DESIGN_SIZES with a window of 1,024 and stretched
# frequencies; attention heads of 128 (half of each turned) with a window of 1,024 beside a minGRU twice the model's width.
DIBULIX_SIZES = {
    "1k": dict(delta_heads=4, delta_kv_heads=2, delta_dim=128, delta_vdim=256, conv=4, low_rank=16, kv_heads=2, att_dim=128, att_rot=64, window=1024, gru_width=2048, streams=4),
    "2k": dict(delta_heads=8, delta_kv_heads=4, delta_dim=128, delta_vdim=256, conv=4, low_rank=16, kv_heads=4, att_dim=128, att_rot=64, window=1024, gru_width=4096, streams=4),
}


def dibulix_config(z: dict, b: dict):
    """Delta-rule, latent-attention, side-by-side and delta-rule layers in turn, every layer with a dense feed-forward."""
    from alofa_b200.models.dibulix import DeltaConfig, DibulixConfig, DibulixLayer, LatentConfig, ParallelConfig, Rotary, WindowedAttentionConfig

    delta = DeltaConfig(b["delta_heads"], b["delta_kv_heads"], b["delta_dim"], b["delta_vdim"], b["conv"])
    latent = LatentConfig(z["heads"], z["dim"], z["rot"], z["vdim"], z["kv_rank"], (z["dim"] + z["rot"]) ** -0.5,
                          Rotary(1e4, z["rot"], {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0}), b["window"])
    pair = ParallelConfig(WindowedAttentionConfig(z["heads"], b["kv_heads"], b["att_dim"], b["att_dim"], b["att_dim"] ** -0.5, Rotary(1e6, b["att_rot"]), b["window"]),
                          b["gru_width"], 1.0, 1.0)
    kinds = (("channel_delta", delta), ("latent_attention", latent), ("parallel", pair), ("channel_delta", delta))
    layers = [DibulixLayer(*kinds[i % 4], z["ff"]) for i in range(z["layers"])]
    return DibulixConfig(z["vocab"], z["width"], 1e-6, 1.0, b["streams"], layers)


def dibulix_numbers(z: dict, b: dict) -> dict:
    """Bytes a decode step reads and flops a token costs for the Dibulix sizes (bf16 weights and caches, fp32 states).  Both
    windows are shorter than the bench's prompts, so a decode step reads a window's worth of cache rows per request,
    whatever the context: that is counted as state, and nothing grows with the context."""
    w, h = z["width"], z["heads"]
    qk, v, dec, r = b["delta_kv_heads"] * b["delta_dim"], b["delta_heads"] * b["delta_vdim"], b["delta_heads"] * b["delta_dim"], b["low_rank"]
    delta = w * (2 * qk + v + b["delta_heads"]) + r * (2 * w + dec + v) + v * w
    d_row = z["kv_rank"] + z["rot"]
    latent = w * h * (z["dim"] + z["rot"]) + w * d_row + h * z["dim"] * z["kv_rank"] + h * z["vdim"] * z["kv_rank"] + h * w + h * z["vdim"] * w
    att = w * (h + 2 * b["kv_heads"]) * b["att_dim"] + h * b["att_dim"] * w
    gru = 4 * w * b["gru_width"]
    kinds = [("delta", delta), ("latent", latent), ("pair", att + gru), ("delta", delta)]
    used = [kinds[i % 4] for i in range(z["layers"])]
    n = {k: sum(1 for name, _ in used if name == k) for k in ("delta", "latent", "pair")}
    params = sum(p for _, p in used) + z["layers"] * 2 * w * z["ff"]
    state_bytes = 4 * (n["delta"] * (dec * b["delta_vdim"] + (b["conv"] - 1) * (2 * qk + v)) + n["pair"] * b["gru_width"])
    window_bytes = 2 * b["window"] * (n["latent"] * d_row + n["pair"] * 2 * b["kv_heads"] * b["att_dim"])
    return {"weight_bytes": 2 * (params + z["vocab"] * w), "kv_bytes_per_token": 0, "flops_per_token": 2.0 * params,
            "attn_flops_per_pair": n["latent"] * 2.0 * h * (d_row + z["kv_rank"]) + n["pair"] * 4.0 * h * b["att_dim"], "head_flops": 2.0 * w * z["vocab"],
            "state_bytes_per_request": 2 * state_bytes + window_bytes}


# --design kikerax: differential attention in chunks and attention + gated linear recurrent unit layers in turn, dense and
# routed feed-forwards in turn, beside the Darolix design at the same width, layers, heads, experts and vocabulary.  Inner
# sizes after published models of the kind: two maps a head with keys and values of 128 over chunks of 1,024 tokens, a quarter
# of each map turned; attention heads of 128 beside a recurrent unit 4/3 as wide as the model in blocks of 256 channels with
# four taps; four groups of experts of which two are kept.
KIKERAX_SIZES = {
    "1k": dict(kv_heads=2, att_dim=128, att_rot=32, chunk=1024, lru_width=1280, lru_block=256, conv=4, groups=4, keep=2),
    "2k": dict(kv_heads=4, att_dim=128, att_rot=32, chunk=1024, lru_width=2560, lru_block=256, conv=4, groups=8, keep=4),
}


def kikerax_config(z: dict, b: dict):
    """Differential attention with a dense feed-forward and attention beside the recurrent unit with routed experts, in turn."""
    from alofa_b200.models.kikerax import DifferentialConfig, FeedForwardConfig, KeyedAttentionConfig, KikeraxConfig, KikeraxLayer, ParallelConfig, RecurrentConfig

    d = b["att_dim"]
    attention = DifferentialConfig(z["heads"], b["kv_heads"], d, d, d ** -0.5, 0.6, {"base": 1e4, "dims": b["att_rot"], "scaling": {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0}},
                                   b["chunk"])
    pair = ParallelConfig(KeyedAttentionConfig(z["heads"], b["kv_heads"], d, d, d ** -0.5, 50.0, {"coef": 0.3, "every": 128}),
                          RecurrentConfig(b["lru_width"], b["lru_width"] // b["lru_block"], b["conv"]), 0.6, 0.9)
    dense = FeedForwardConfig("dense", z["ff"])
    routed = FeedForwardConfig("moe", z["expert_ff"], z["experts"], z["top"], 2.0, {"count": b["groups"], "keep": b["keep"]}, z["shared_ff"])
    layers = [KikeraxLayer("attention", attention, dense) if i % 2 == 0 else KikeraxLayer("parallel", pair, routed) for i in range(z["layers"])]
    return KikeraxConfig(z["vocab"], z["width"], 1e-6, 30.0, layers)


def kikerax_numbers(z: dict, b: dict) -> dict:
    """Bytes a decode step reads and flops a token costs for the Kikerax sizes (bf16 weights and caches, fp32 states and gates).
    The chunked layers' keys never reach further back than a chunk, so their share of a decode step is counted as state."""
    w, h, d, g = z["width"], z["heads"], b["att_dim"], b["kv_heads"]
    diff = w * (2 * h * d + 2 * g * d + g * d + h) + h * d * w
    keyed = w * (h * d + g * d + h) + h * d * w
    W, bs = b["lru_width"], b["lru_block"]
    lru = 3 * w * W + W * b["conv"]
    gates = 2 * W * bs  # fp32
    n_att, n_pair = (z["layers"] + 1) // 2, z["layers"] // 2
    expert = 3 * w * z["expert_ff"]
    routed_all, routed_tok = z["experts"] * expert + 3 * w * z["shared_ff"] + z["experts"] * w, z["top"] * expert + 3 * w * z["shared_ff"] + z["experts"] * w
    params_all = n_att * (diff + 2 * w * z["ff"]) + n_pair * (keyed + lru + routed_all)
    per_token = n_att * (diff + 2 * w * z["ff"]) + n_pair * (keyed + lru + gates + routed_tok)
    state_bytes = 4 * n_pair * W * b["conv"]
    chunk_bytes = 2 * n_att * (b["chunk"] // 2) * (2 * g * d + g * d)  # half a chunk on average
    return {"weight_bytes": 2 * (params_all + z["vocab"] * w) + 4 * n_pair * gates, "kv_bytes_per_token": n_pair * 2 * g * d * 2, "flops_per_token": 2.0 * per_token,
            "attn_flops_per_pair": n_pair * 4.0 * h * d, "head_flops": 2.0 * w * z["vocab"], "state_bytes_per_request": 2 * state_bytes + chunk_bytes}


class KernelClock:
    """Times every kernel call of the package's ops module with its own pair of CUDA events during one
    step (run outright, no graph), and sets each beside the time its own operands allow: the larger of
    flops over the measured matrix rate and bytes over the measured copy bandwidth."""

    PRODUCTS = ("gemm_tc", "gemm_generic", "gemm_batched", "gemm_tc_rope")
    ATTENTION = ("attention_bf16", "latent_attention_bf16", "latent_attention", "paged_attention_generic")
    STATE = ("linear_scan", "causal_conv", "delta_scan", "min_gru", "lru_scan")  # read and leave a state per request

    def __init__(self, peaks: dict):
        self.peaks = peaks
        self.calls = []

    @staticmethod
    def _bytes(args, kwargs) -> int:
        import torch

        total = 0
        for a in list(args) + list(kwargs.values()):
            if isinstance(a, torch.Tensor):
                total += a.numel() * a.element_size()
            elif isinstance(getattr(a, "sums", None), torch.Tensor):  # a product's split sums, which the kernel adds up as it reads
                total += a.sums.numel() * a.sums.element_size()
        return total

    def ideal_us(self, name, args, kwargs, kv_rows: int) -> tuple:
        import torch

        byts, flops = self._bytes(args, kwargs), 0.0
        if name in ("gemm_tc", "gemm_generic"):
            out, x, w = args[0], args[1], args[2]
            flops = 2.0 * out.shape[0] * (out.shape[1] if kwargs.get("tile_batch") is not None else w.shape[0]) * w.shape[1]  # by tile: one batch's rows per token row
        elif name == "gemm_batched":
            out, x, w, batches, m, n, k = args[:7]
            by_tile = kwargs.get("tile_batch") is not None
            flops = 2.0 * m * n * k * (1 if by_tile else batches)
            byts = (out.element_size() * m * n + x.element_size() * m * k) * (1 if by_tile else batches) + w.numel() * w.element_size()
        elif name == "linear_scan":
            # y, v, ., b, ., c, ., dec, ., state, q_start, slots, n_seqs, heads, groups, n, p: the rows once, the live requests' states read and written
            y, n_seqs, heads, groups, n, p = args[0], args[12], args[13], args[14], args[15], args[16]
            rows = y.shape[0]
            byts = 4 * rows * (2 * heads * p + 2 * groups * n + (heads * n if args[17] else heads)) + 8 * n_seqs * heads * n * p
            # the recurrence is 32-bit by the design: a multiply and two multiply-adds per state element and token on the fp32 pipe
            # (no tensor-core mode is 32-bit), against the nominal fp32 rate: 128 lanes x 2 x 1.965 GHz per SM
            import torch as _t

            fp32_rate = _t.cuda.get_device_properties(0).multi_processor_count * 128 * 2 * 1.965e9
            ideal = max(5.0 * rows * heads * n * p / fp32_rate, byts / (self.peaks["hbm_gbs"] * 1e9)) * 1e6
            return ideal, 5.0 * rows * heads * n * p, byts
        elif name == "delta_scan":
            # y, v, ., kn, qn, kq, g, beta, state, q_start, slots, n_seqs, heads, groups, n, p: the rows once, the live requests' states read and written
            y, n_seqs, heads, groups, n, p = args[0], args[11], args[12], args[13], args[14], args[15]
            rows = y.shape[0]
            byts = 4 * rows * (2 * heads * p + 2 * groups * n + heads * n + heads + groups) + 8 * n_seqs * heads * n * p
            # 32-bit by the design: the decay's multiply, the two dot products with key and query and the write's multiply-add per
            # state element and token on the fp32 pipe, against the nominal fp32 rate: 128 lanes x 2 x 1.965 GHz per SM
            import torch as _t

            fp32_rate = _t.cuda.get_device_properties(0).multi_processor_count * 128 * 2 * 1.965e9
            ideal = max(7.0 * rows * heads * n * p / fp32_rate, byts / (self.peaks["hbm_gbs"] * 1e9)) * 1e6
            return ideal, 7.0 * rows * heads * n * p, byts
        elif name == "min_gru":
            out, n_seqs = args[0], args[8]
            byts = out.numel() * (12 + out.element_size()) + 8 * n_seqs * out.shape[1]
        elif name == "lru_scan":
            # out, a, b, y, ., ., state, q_start, slots, n_seqs: decays, driven inputs and the other branch once, the outputs once, the live requests' states read and written
            out, n_seqs = args[0], args[9]
            byts = out.numel() * (12 + out.element_size()) + 8 * n_seqs * out.shape[1]
        elif name == "lru_gates":
            # a, b, u, wa, wi, ...: 32-bit by the design: two block-diagonal products on the fp32 pipe, against the nominal fp32 rate
            a, wa = args[0], args[3]
            import torch as _t

            fp32_rate = _t.cuda.get_device_properties(0).multi_processor_count * 128 * 2 * 1.965e9
            flops = 4.0 * a.shape[0] * a.shape[1] * wa.shape[1]
            byts = 12 * a.numel() + 8 * wa.numel()
            return max(flops / fp32_rate, byts / (self.peaks["hbm_gbs"] * 1e9)) * 1e6, flops, byts
        elif name == "hyper_connect":
            # the streams read once, and written once when a sublayer's output is owed; that output, the next input and the sum once each
            streams = args[0]
            given = lambda i, key: (args[i] if len(args) > i else kwargs.get(key))
            y, x_out, sum_out = given(1, "y"), given(7, "x_out"), given(8, "sum_out")
            byts = streams.numel() * 4 * (2 if y is not None else 1) + sum(t.numel() * t.element_size() for t in (y, x_out, sum_out) if t is not None)
        elif name == "causal_conv":
            out = args[0]
            byts = 8 * out.numel() + 8 * args[9] * (args[3].shape[1] - 1) * out.shape[1]
        elif name in self.ATTENTION:
            # out, q, cache(s): every visible row of the cache is read once per request (bytes) and multiplied by every query row (flops)
            out, q = args[0], args[1]
            caches = [a for a in args[2:4] if isinstance(a, torch.Tensor) and a.dim() >= 2 and a.dtype == q.dtype]
            row_bytes = sum(c[0].numel() * c.element_size() for c in caches)
            byts = out.numel() * out.element_size() + q.numel() * q.element_size() + kv_rows * row_bytes
            flops = 2.0 * self.pairs * (q.shape[1] + out.shape[1])  # per (query token, key) pair: heads * (score width + value width) multiply-adds
        ideal = max(flops / (self.peaks["bf16_tflops"] * 1e12), byts / (self.peaks["hbm_gbs"] * 1e9)) * 1e6
        return ideal, flops, byts

    def run(self, step, kv_rows: int, pairs: float) -> list:
        """``step()`` runs one step; ``kv_rows``: cache rows the step's requests hold; ``pairs``: (query token, visible key) pairs."""
        import torch

        from alofa_b200.csrc import ops

        self.pairs = pairs
        names = [n for n in dir(ops) if not n.startswith("_") and callable(getattr(ops, n)) and getattr(getattr(ops, n), "__module__", "") == ops.__name__
                 and n not in ("launch_count", "count_launches", "bound_stream", "attention_decode_wide_warps", "attention_decode_slots", "attention_bf16_supported",
                               "gemm_tc_rope_splits", "gemm_tc_splits", "latent_attention_bf16_supported", "load_library", "gemm_by_tile")]  # gemm_by_tile only chooses: its product is timed
        originals = {n: getattr(ops, n) for n in names}
        records = []

        def wrap(name, fn):
            def timed(*args, **kwargs):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                result = fn(*args, **kwargs)
                b.record()
                records.append((name, a, b, self.ideal_us(name, args, kwargs, kv_rows)))
                return result
            return timed

        for n, fn in originals.items():
            setattr(ops, n, wrap(n, fn))
        try:
            step()
            torch.cuda.synchronize()
        finally:
            for n, fn in originals.items():
                setattr(ops, n, fn)
        table = {}
        for name, a, b, (ideal, flops, byts) in records:
            us = a.elapsed_time(b) * 1e3
            row = table.setdefault(name, {"kernel": name, "calls": 0, "us": 0.0, "ideal_us": 0.0})
            row["calls"] += 1
            row["us"] += us
            row["ideal_us"] += ideal
        out = sorted(table.values(), key=lambda r: -r["us"])
        for r in out:
            r["of_roofline"] = round(r["ideal_us"] / r["us"], 4) if r["us"] > 0 else None
            r["us"], r["ideal_us"] = round(r["us"], 1), round(r["ideal_us"], 1)
        return out


class DesignBench(Bench):
    """One engine of one design at one size, measured like the headline bench's."""

    def __init__(self, architecture: str, cfg, label: str, vocab: int, weight_bytes: int, kv_bytes_per_token: int, flops_per_token: float, attn_flops_per_pair: float, max_batch: int,
                 state_bytes_per_request: int = 0, window: int = 0):
        import numpy as np

        from alofa_b200.engine.engine import Engine

        self.label, self.cfg = label, cfg
        self.vocab = vocab
        self.engine = Engine.from_random(architecture, cfg, seed=0, dtype="bfloat16", generate_on_device=True, block_size=64, max_batch=max_batch,
                                         max_tokens=CONTEXT, token_budget=PROMPT_LEN + max_batch, max_chunk=PROMPT_LEN)
        self.runner = self.engine.runner
        self.numbers = {"weight_bytes": weight_bytes, "kv_bytes_per_token": kv_bytes_per_token, "state_bytes_per_request": state_bytes_per_request}
        self.flops_per_token, self.attn_flops_per_pair = flops_per_token, attn_flops_per_pair
        self.window = window  # every attention of the design sees this many keys at most (0: all)
        self.peaks, self.peaks_kind = peaks()
        self.rng = np.random.default_rng(0)

    def prompt(self, n: int) -> list:
        return [int(t) for t in self.rng.integers(0, self.vocab, size=n)]

    def pairs(self, tokens: int) -> float:
        """(query, visible key) pairs of one prompt of ``tokens`` tokens."""
        if not self.window or self.window >= tokens:
            return tokens * (tokens + 1) / 2
        return self.window * (self.window + 1) / 2 + (tokens - self.window) * self.window

    def prefill(self, warmup: int, reps: int = 10) -> dict:
        from alofa_b200.engine.step import StepEntry

        tokens = self.prompt(PROMPT_LEN)

        def one():
            slot = self.runner.admit(10_000)
            self.runner.forward_logits([StepEntry(slot, tokens, (PROMPT_LEN - 1,))])
            self.runner.release(slot)

        for _ in range(max(3, warmup)):
            one()
        _, each = self.timed_each(one, reps)
        ms = statistics.median(each)
        flops = self.flops_per_token * PROMPT_LEN + self.attn_flops_per_pair * self.pairs(PROMPT_LEN)
        return {"tok_s": round(PROMPT_LEN / ms * 1e3, 1), "ms": round(ms, 4), "flops_frac": round(flops / (ms * 1e-3) / (self.peaks["bf16_tflops"] * 1e12), 4)}

    def kernels(self, batch: int) -> dict:
        """Per-kernel times of one prefill step and one decode step of ``batch`` requests, run outright."""
        from alofa_b200.engine.step import StepEntry

        clock = KernelClock(self.peaks)
        runner = self.runner
        graphs, runner.cuda_graphs, runner.prompt_graphs = (runner.cuda_graphs, runner.prompt_graphs), False, False
        try:
            tokens = self.prompt(PROMPT_LEN)
            slot = runner.admit(30_000)
            runner.forward_logits([StepEntry(slot, tokens, (PROMPT_LEN - 1,))])  # loads every kernel
            runner.release(slot)
            slot = runner.admit(30_001)
            prefill = clock.run(lambda: runner.forward_logits([StepEntry(slot, tokens, (PROMPT_LEN - 1,))]), PROMPT_LEN, self.pairs(PROMPT_LEN))
            runner.release(slot)
            slots = [runner.admit(31_000 + i) for i in range(batch)]
            for s_ in slots:
                runner.forward_logits([StepEntry(s_, self.prompt(PROMPT_LEN), ())])
            one = lambda: runner.forward_logits([StepEntry(s_, (1,), (0,)) for s_ in slots])
            one()
            seen = min(PROMPT_LEN + 2, self.window or PROMPT_LEN + 2)
            decode = clock.run(one, batch * seen, batch * seen)
            for s_ in slots:
                runner.release(s_)
        finally:
            runner.cuda_graphs, runner.prompt_graphs = graphs
        return {"prefill_2048": prefill[:8], f"decode_b{batch}": decode[:8]}


def design_numbers(design: str, z: dict, routed_only: bool = False) -> dict:
    """Bytes a decode step reads and flops a token costs, from the sizes (bf16)."""
    w, h = z["width"], z["heads"]
    if design == "kotutar":
        d_row = z["kv_rank"] + z["rot"]
        mixer = w * (z["q_rank"] + d_row) + z["q_rank"] * h * (z["dim"] + z["rot"]) + h * z["dim"] * z["kv_rank"] + h * z["vdim"] * z["kv_rank"] + h * z["vdim"] * w
        dense = 2 * w * z["ff"]
        expert = 2 * w * z["expert_ff"]
        shared = 2 * w * z["shared_ff"]
        n_dense, n_moe = (z["layers"] + 1) // 2, z["layers"] // 2
        if routed_only:  # every layer routed, no shared expert
            n_dense, n_moe, shared = 0, z["layers"], 0
        params_all = z["layers"] * mixer + n_dense * dense + n_moe * (z["experts"] * expert + shared + (z["experts"] + 1) * w)
        per_token = z["layers"] * mixer + n_dense * dense + n_moe * (z["top"] * expert + shared + (z["experts"] + 1) * w)
        return {"weight_bytes": 2 * (params_all + z["vocab"] * w), "kv_bytes_per_token": z["layers"] * d_row * 2, "flops_per_token": 2.0 * per_token,
                "attn_flops_per_pair": z["layers"] * 2.0 * h * (d_row + z["kv_rank"]), "head_flops": 2.0 * w * z["vocab"]}
    hd, kv = w // h, 2 * (w // h)
    per_layer = w * (h * hd + 2 * kv) + h * hd * w + 3 * w * z["ff"]
    return {"weight_bytes": 2 * (z["layers"] * per_layer + 2 * z["vocab"] * w), "kv_bytes_per_token": z["layers"] * 2 * kv * 2, "flops_per_token": 2.0 * z["layers"] * per_layer,
            "attn_flops_per_pair": z["layers"] * 4.0 * h * hd, "head_flops": 2.0 * w * z["vocab"]}


def darolix_numbers(z: dict, d: dict) -> dict:
    """Bytes a decode step reads and flops a token costs for the Darolix sizes (bf16 weights, fp32 states)."""
    w = z["width"]
    inner, bc = d["ssm_heads"] * d["ssm_vdim"], d["groups"] * d["state"]
    ssm = w * (2 * inner + 2 * bc + d["ssm_heads"]) + inner * w
    att = w * (z["heads"] + 2 * d["kv_heads"]) * d["att_dim"] + z["heads"] * d["att_dim"] * w
    qk, v = d["gla_heads"] * d["gla_dim"], d["gla_heads"] * d["gla_vdim"]
    gla = w * (2 * qk + 2 * v) + v * w + 16 * (w + qk)
    expert = 3 * w * z["expert_ff"]
    router = (z["experts"] + d["identity"]) * w
    n_ssm, n_pair = (z["layers"] + 1) // 2, z["layers"] // 2
    params_all = n_ssm * ssm + n_pair * (att + gla) + z["layers"] * (z["experts"] * expert + router)
    per_token = n_ssm * ssm + n_pair * (att + gla) + z["layers"] * (z["top"] * expert + router)
    state_bytes = 4 * (n_ssm * (inner * d["state"] + (d["conv"] - 1) * (inner + 2 * bc)) + n_pair * qk * d["gla_vdim"])
    return {"weight_bytes": 2 * (params_all + 2 * z["vocab"] * w), "kv_bytes_per_token": n_pair * 2 * d["kv_heads"] * d["att_dim"] * 2, "flops_per_token": 2.0 * per_token,
            "attn_flops_per_pair": n_pair * 4.0 * z["heads"] * d["att_dim"], "head_flops": 2.0 * w * z["vocab"], "state_bytes_per_request": 2 * state_bytes}


def run_designs(args) -> dict:
    """Prefill and decode of a design beside its closest existing design at equal layer sizes (Kotutar
    beside Qwen2, Darolix beside Kotutar, Dibulix beside Darolix), and the kernels of one step of each
    against their own rooflines."""
    from alofa_b200.models import darolix, dibulix, kikerax, kotutar, qwen2

    pair = {"kikerax": "Kikerax design beside Darolix", "dibulix": "Dibulix design beside Darolix", "darolix": "Darolix design beside Kotutar", "kotutar": "Kotutar design beside Qwen2"}[args.design]
    out = {"metric": f"prefill and decode of the {pair} at equal layer sizes", "dtype": "bf16", "data": "synthetic", "n_gpus": 1,
           "prompt_tokens": PROMPT_LEN, "context": CONTEXT, "steps": args.steps, "warmup": args.warmup, "sizes": {}}
    for size in ([args.size] if args.size else sorted(DESIGN_SIZES)):
        z = DESIGN_SIZES[size]
        row = {"sizes": z}
        if args.design == "kikerax":
            row["kikerax_sizes"], row["darolix_sizes"] = KIKERAX_SIZES[size], DAROLIX_SIZES[size]
            arms = (("kikerax", kikerax.NAME, kikerax_config(z, KIKERAX_SIZES[size])), ("darolix", darolix.NAME, darolix_config(z, DAROLIX_SIZES[size])))
        elif args.design == "dibulix":
            row["dibulix_sizes"], row["darolix_sizes"] = DIBULIX_SIZES[size], DAROLIX_SIZES[size]
            arms = (("dibulix", dibulix.NAME, dibulix_config(z, DIBULIX_SIZES[size])), ("darolix", darolix.NAME, darolix_config(z, DAROLIX_SIZES[size])))
        elif args.design == "darolix":
            row["darolix_sizes"] = DAROLIX_SIZES[size]
            arms = (("darolix", darolix.NAME, darolix_config(z, DAROLIX_SIZES[size])), ("kotutar", kotutar.NAME, kotutar_config_routed(z)))
        else:
            arms = (("kotutar", kotutar.NAME, kotutar_config(z)), ("qwen2", qwen2.NAME, qwen2_config_like(z)))
        for design, name, cfg in arms:
            if design == "kikerax":
                n = kikerax_numbers(z, KIKERAX_SIZES[size])
            elif design == "dibulix":
                n = dibulix_numbers(z, DIBULIX_SIZES[size])
            elif design == "darolix":
                n = darolix_numbers(z, DAROLIX_SIZES[size])
            else:
                n = design_numbers(design, z, routed_only=args.design == "darolix")
            window = DIBULIX_SIZES[size]["window"] if design == "dibulix" else 0
            bench = DesignBench(name, cfg, f"{design} {size}", z["vocab"], n["weight_bytes"], n["kv_bytes_per_token"], n["flops_per_token"], n["attn_flops_per_pair"], 64,
                                n.get("state_bytes_per_request", 0), window=window)
            res = {"prefill_2048": bench.prefill(args.warmup)}
            for batch in (8, 64):
                point = bench.decode(batch, min(args.steps, 64), args.warmup)
                res[f"decode_b{batch}"] = {"tok_s": round(point["tok_s"], 1), "ms_per_step": round(point["ms"], 4), "hbm_frac": round(point["frac"], 4), "launches_per_step": point["launches"] // max(1, min(args.steps, 64))}
            res["kernels"] = bench.kernels(64)
            res["peaks"] = bench.peaks_kind
            row[design] = res
            bench.close()
        out["sizes"][size] = row
    return out


def reference_arm() -> dict:
    """The reference is a Mojo project: it has no Python package to install and
    neither `mojo` nor `pixi` exists in this image, so it cannot run here."""
    return {"impl": "reference", "unavailable": "mojothon/alofa is pure Mojo (no setup.py/pyproject; pip finds nothing to install) and no Mojo toolchain is in the image; CPU-only in any case"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="alofa_b200")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the full shape (named in config)")
    ap.add_argument("--phase", choices=["all", "decode", "prefill"], default="all", help="profiling aid: run only one part; the JSON line then lacks the others")
    ap.add_argument("--shape", choices=sorted(SHAPES), default="0.5b", help="whose layer sizes the headline run has")
    ap.add_argument("--no-extra", dest="extra", action="store_false", help="leave out the measurements beside the headline (long contexts, the 1.5B and 7B shapes)")
    ap.add_argument("--design", choices=["kotutar", "darolix", "dibulix", "kikerax"], help="instead of the headline run: this design beside its closest existing one (Qwen2 for kotutar, Kotutar for darolix, Darolix for dibulix and kikerax) at equal layer sizes (prefill, decode, kernels against their rooflines)")
    ap.add_argument("--size", choices=sorted(DESIGN_SIZES), help="with --design: one of the sizes only")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps(reference_arm()))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.design:
        print(json.dumps(run_designs(args)))
        return 0
    print(json.dumps(run(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
