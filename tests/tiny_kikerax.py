"""The tests' own small Kikerax configurations and weights.

Sizes differ between the configurations and from layer to layer: either mixer
first, last and in the middle; layers without a feed-forward, with a dense one
and with a routed one after either mixer; fewer key heads than heads and as
many; values wider and narrower than keys and as wide; rotation of a part of a
map, of all of it and none, with and without stretched frequencies; chunks of
two tokens, of less than a page, of exactly a page, of several pages, and no
chunks at all; with and without query temperature, score cap and logit cap;
one block and several in the recurrent unit, one tap to four; routers with and
without groups (groups of one, two and three experts; all groups kept and
one), with and without a shared expert; widths that are no multiple of 8.
Weights are drawn here: matrices N(0, gain / sqrt(inputs)), decays near one so
that the state is carried, corrections large enough to change choices."""
import json
from pathlib import Path

import numpy as np
import torch


def rot(base, dims, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def attention(heads, kv_heads, dim, vdim, scale, diff, rot_=None, chunk=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if rot_ is not None:
        out["rot"] = rot_
    if chunk is not None:
        out["mask"] = {"size": chunk}
    return out


def parallel(heads, kv_heads, dim, scale, width, blocks, conv, left_scale, right_scale, softcap=None, q_temp=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if softcap is not None:
        left["softcap"] = softcap
    if q_temp is not None:
        left["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"left": left, "right": {"width": width, "blocks": blocks, "conv": conv}, "left_scale": left_scale, "right_scale": right_scale}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, scale, groups=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


CONFIGS = {
    # differential attention first; chunks shorter than a page (9) and a page and a half (21); values wider than keys and narrower; groups of two experts, two of three kept
    "A": {"architecture": "Kikerax", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "logit_softcap": 12.0,
          "layers": [layer("attention", attention(4, 2, 16, 24, 0.6, 0.3, rot(300.0, 8, (4.0, 64, 8.0, 1.0)), 9), dense(72)),
                     layer("parallel", parallel(6, 3, 16, 0.7, 48, 3, 3, 1.3, 0.4, softcap=5.0, q_temp=(0.4, 7)), moe(6, 2, 24, 1.5, (3, 2), 40)),
                     layer("attention", attention(3, 3, 12, 8, 0.8, 0.55, rot(100.0, 12), 21), None),
                     layer("parallel", parallel(2, 1, 24, 0.5, 40, 1, 2, 0.7, 1.1, q_temp=(1.0, 16)), dense(40))]},
    # a width that is no multiple of 8; the recurrent block first, one tap, no cap, no temperature; a router without groups or shared expert; attention
    # without rotation and without chunks (every key), then chunks of exactly a page of 16 and of two tokens; no logit cap
    "B": {"architecture": "Kikerax", "vocab": 157, "width": 100, "norm": {"eps": 3e-6},
          "layers": [layer("parallel", parallel(5, 5, 12, 0.8, 70, 1, 1, 0.5, 2.0), moe(5, 2, 28, 1.0)),
                     layer("attention", attention(2, 1, 10, 30, 0.9, 0.8), None),
                     layer("attention", attention(2, 2, 20, 20, 0.6, 0.2, rot(50.0, 6), 16), dense(24)),
                     layer("attention", attention(1, 1, 8, 12, 1.0, 0.5, rot(7.0, 8, (2.0, 16, 4.0, 0.5)), 2), moe(4, 1, 16, 2.5, (4, 2)))]},
    # sizes in multiples of 64 that the tensor-core kernels take (left heads of 64; keys and values of 64 in the differential attention); chunks of a
    # page of 64; four taps; groups of two experts, half of them kept
    "C": {"architecture": "Kikerax", "vocab": 320, "width": 128, "norm": {"eps": 2e-6}, "logit_softcap": 25.0,
          "layers": [layer("parallel", parallel(4, 2, 64, 0.35, 128, 2, 4, 0.6, 0.9, softcap=20.0, q_temp=(0.6, 32)), moe(8, 2, 64, 1.75, (4, 2), 64)),
                     layer("attention", attention(2, 1, 64, 64, 0.3, 0.65, rot(10000.0, 32, (8.0, 128, 32.0, 1.0)), 64), dense(128)),
                     layer("parallel", parallel(2, 2, 64, 0.3, 64, 4, 2, 1.0, 1.0), None),
                     layer("attention", attention(2, 2, 32, 128, 0.45, 0.1, rot(500.0, 32), 128), moe(6, 3, 32, 0.5, None, 32))]},
    # chunks over several pages (100, 130) for long prompts; a temperature that steps every 50 tokens; groups of three experts of which one is kept
    "D": {"architecture": "Kikerax", "vocab": 190, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 8.0,
          "layers": [layer("attention", attention(2, 2, 24, 16, 0.5, 0.7, rot(500000.0, 8), 100), None),
                     layer("parallel", parallel(4, 1, 8, 1.0, 96, 2, 4, 0.9, 0.8, softcap=50.0, q_temp=(0.7, 50)), moe(9, 3, 16, 1.0, (3, 1), 24)),
                     layer("attention", attention(2, 1, 16, 16, 0.6, 0.45, rot(1000.0, 16, (16.0, 256, 16.0, 2.0)), 130), dense(32))]},
}


def tensor_shapes(cfg):
    w = cfg["width"]
    shapes = {"embed": (cfg["vocab"], w), "final.norm": (w,)}
    for i, spec in enumerate(cfg["layers"]):
        p, m = f"l{i}.", spec["mixer"]
        shapes[p + "norm1"] = (w,)
        if spec["type"] == "parallel":
            a, r = m["left"], m["right"]
            W, B = r["width"], r["blocks"]
            q = p + "mix.left."
            shapes.update({q + "q": (a["heads"] * a["dim"], w), q + "k": (a["kv_heads"] * a["dim"], w), q + "q.norm": (a["dim"],), q + "k.norm": (a["dim"],),
                           q + "g": (a["heads"], w), q + "o": (w, a["heads"] * a["vdim"])})
            q = p + "mix.right."
            shapes.update({q + "y": (W, w), q + "y.b": (W,), q + "x": (W, w), q + "x.b": (W,), q + "conv": (W, r["conv"]), q + "conv.b": (W,),
                           q + "ra": (B, W // B, W // B), q + "ra.b": (B, W // B), q + "ri": (B, W // B, W // B), q + "ri.b": (B, W // B), q + "lam": (W,), q + "o": (w, W)})
        else:
            q = p + "mix."
            for n, rows in (("q", m["heads"] * 2 * m["dim"]), ("k", m["kv_heads"] * 2 * m["dim"]), ("v", m["kv_heads"] * m["vdim"])):
                shapes[q + n] = (rows, w)
                shapes[q + n + ".b"] = (rows,)
            shapes.update({q + "q.norm": (m["dim"],), q + "k.norm": (m["dim"],), q + "lq1": (m["dim"],), q + "lk1": (m["dim"],), q + "lq2": (m["dim"],), q + "lk2": (m["dim"],),
                           q + "g": (m["heads"], w), q + "o": (w, m["heads"] * m["vdim"]), q + "o.b": (w,)})
        mlp = spec["mlp"]
        if mlp is None:
            continue
        shapes[p + "norm2"] = (w,)
        q = p + "mlp."
        if mlp["kind"] == "dense":
            shapes.update({q + "up": (mlp["ff"], w), q + "down": (w, mlp["ff"])})
        else:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            shapes.update({q + "router": (E, w), q + "correction": (E,)})
            for e in range(E):
                shapes.update({q + f"e{e}.gate": (ff, w), q + f"e{e}.up": (ff, w), q + f"e{e}.down": (w, ff)})
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                shapes.update({q + "shared.gate": (sf, w), q + "shared.up": (sf, w), q + "shared.down": (w, sf)})
    return shapes


def weights(cfg, seed):
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        parts = name.split(".")
        last = parts[-1]
        if last in ("norm", "norm1", "norm2"):
            v = 1.0 + 0.1 * rng.standard_normal(shape)
        elif last == "lam":
            v = rng.uniform(-6.0, -2.0, size=shape)  # decays near one: the state is carried over hundreds of tokens
        elif last == "correction":
            v = 0.3 * rng.standard_normal(shape)  # large enough to change choices
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            v = rng.standard_normal(shape) / np.sqrt(np.sqrt(shape[0]))
        elif last == "b":
            v = 0.5 * rng.standard_normal(shape)
        elif last == "conv":
            v = rng.standard_normal(shape) / np.sqrt(shape[-1]) + (np.arange(shape[-1]) == shape[-1] - 1)
        elif name == "embed":
            v = rng.standard_normal(shape)
        else:
            gain = 2.0 if last in ("router", "g", "ra", "ri") else 1.0
            v = gain * rng.standard_normal(shape) / np.sqrt(shape[-1])
        out[name] = torch.from_numpy(np.asarray(v)).to(torch.bfloat16)
    return out


def write(folder, name, seed=0, cfg=None, tensors=None):
    from alofa_b200.weights.safetensors_io import write_safetensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    cfg = cfg or CONFIGS[name]
    (folder / "config.json").write_text(json.dumps(cfg, indent=1) + "\n")
    write_safetensors(folder / "model.safetensors", tensors if tensors is not None else weights(cfg, seed), {"format": "pt"})
    return folder


def tokens(name, n, seed=0):
    rng = np.random.default_rng(7000 + seed)
    return [int(t) for t in rng.integers(0, CONFIGS[name]["vocab"], size=n)]
