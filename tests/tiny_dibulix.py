"""The tests' own small Dibulix configurations and weights.

Sizes differ between the configurations and from layer to layer: one, two,
three and four residual streams; every mixer first, last and in the middle;
layers with and without a feed-forward after every kind of mixer; key and
value sizes that differ and that agree; as many key/value heads as heads and
fewer, in the attention and in the delta rule; rotation of a part of the head
and of all of it; windows of two tokens, of less than a page, of exactly a
page, of several pages and longer than any prompt; one to four taps; a latent
of 16 to 64 numbers with rotated parts smaller than, equal to and larger than
the unrotated part; widths that are no multiple of 8.  Weights are drawn here:
matrices N(0, gain / sqrt(inputs)), decays and gates of order one, connection
weights near "read the mean, keep every stream, write into all"."""
import json
from pathlib import Path

import numpy as np
import torch


def rot(base, dims, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def parallel(heads, kv_heads, dim, vdim, scale, rot_, window, width, left_scale, right_scale):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot_, "mask": {"size": window}}
    return {"left": left, "right": {"width": width}, "left_scale": left_scale, "right_scale": right_scale}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, rot_, window):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot_, "mask": {"size": window}}


def layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CONFIGS = {
    # two streams; a latent layer first; fewer key/value heads than heads everywhere; windows shorter than a page (9) and a page and a half (21)
    "A": {"architecture": "Dibulix", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "logit_scale": 0.7, "streams": 2,
          "layers": [layer("latent_attention", latent(3, 16, 8, 24, 40, 0.21, rot(300.0, 8, (4.0, 64, 8.0, 1.0)), 9), 72),
                     layer("channel_delta", delta(4, 2, 24, 16, 3), 40),
                     layer("parallel", parallel(6, 3, 16, 8, 0.3, rot(100.0, 6), 21, 50, 1.3, 0.4), None),
                     layer("channel_delta", delta(2, 1, 8, 40, 2), None)]},
    # one stream; a width that is no multiple of 8; the attention first, all of its head rotated, its window a page of 16; one tap; a window of 2; one latent head
    "B": {"architecture": "Dibulix", "vocab": 157, "width": 100, "norm": {"eps": 3e-6}, "logit_scale": 1.0, "streams": 1,
          "layers": [layer("parallel", parallel(5, 5, 12, 12, 0.25, rot(50.0, 12), 16, 7, 0.5, 2.0), 24),
                     layer("channel_delta", delta(3, 3, 20, 12, 1), None),
                     layer("latent_attention", latent(1, 12, 4, 20, 16, 0.4, rot(20.0, 4, (2.0, 16, 4.0, 0.5)), 2), None),
                     layer("parallel", parallel(2, 1, 10, 30, 0.35, rot(7.0, 2), 40, 33, 1.0, 1.0), 16)]},
    # four streams; sizes in multiples of 64 that the tensor-core kernels take; a window longer than any prompt; 70 key channels (no multiple of four)
    "C": {"architecture": "Dibulix", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 0.25, "streams": 4,
          "layers": [layer("channel_delta", delta(2, 2, 64, 64, 4), 64),
                     layer("latent_attention", latent(4, 32, 32, 32, 64, 0.125, rot(10000.0, 32, (8.0, 128, 32.0, 1.0)), 70), 64),
                     layer("parallel", parallel(4, 2, 64, 64, 0.125, rot(10000.0, 32), 4096, 128, 0.6, 0.9), 128),
                     layer("channel_delta", delta(2, 1, 70, 12, 4), None)]},
    # three streams; windows over several pages (100, 130) for long prompts; a rotated part larger than the unrotated one; 130 key channels in the delta rule
    "D": {"architecture": "Dibulix", "vocab": 190, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 2.0, "streams": 3,
          "layers": [layer("parallel", parallel(2, 2, 24, 16, 0.2, rot(500000.0, 8), 100, 64, 0.9, 0.8), None),
                     layer("latent_attention", latent(2, 8, 16, 16, 32, 0.2, rot(1000.0, 16, (16.0, 256, 16.0, 2.0)), 130), None),
                     layer("channel_delta", delta(1, 1, 130, 8, 2), 32),
                     layer("latent_attention", latent(2, 16, 16, 8, 48, 0.18, rot(1000.0, 16, (3.0, 32, 6.0, 1.0)), 33), 32)]},
    # five streams; head sizes 96 and 80 with keys and values alike, which the bfloat16 attention kernels are built for at first use (neither
    # 64 nor 128: no bulk copies), part of a head turned and all of it; a latent of 96 with three heads; windows of 50, 75 and 300; three taps
    "E": {"architecture": "Dibulix", "vocab": 400, "width": 192, "norm": {"eps": 2e-6}, "logit_scale": 0.4, "streams": 5,
          "layers": [layer("latent_attention", latent(3, 48, 16, 40, 96, 0.13, rot(40000.0, 16, (4.0, 128, 16.0, 2.0)), 50), None),
                     layer("parallel", parallel(6, 2, 96, 96, 0.1, rot(20000.0, 40), 75, 200, 0.8, 1.1), 256),
                     layer("channel_delta", delta(6, 2, 48, 80, 3), None),
                     layer("parallel", parallel(2, 2, 80, 80, 0.11, rot(3000.0, 80), 300, 96, 1.2, 0.7), 128)]},
}


def tensor_shapes(cfg, low_rank=6):
    w, S = cfg["width"], cfg["streams"]
    shapes = {"embed": (cfg["vocab"], w), "final.norm": (w,)}
    for i, spec in enumerate(cfg["layers"]):
        p, m = f"l{i}.", spec["mixer"]
        shapes[p + "norm1"] = (w,)
        numbers = [1]
        if spec["type"] == "parallel":
            a, r = m["left"], m["right"]["width"]
            for n, rows in (("q", a["heads"] * a["dim"]), ("k", a["kv_heads"] * a["dim"]), ("v", a["kv_heads"] * a["vdim"])):
                shapes[p + f"mix.left.{n}"] = (rows, w)
                shapes[p + f"mix.left.{n}.b"] = (rows,)
            shapes[p + "mix.left.o"] = (w, a["heads"] * a["vdim"])
            shapes.update({p + "mix.right.z": (r, w), p + "mix.right.z.b": (r,), p + "mix.right.x": (r, w), p + "mix.right.x.b": (r,), p + "mix.right.g": (r, w),
                           p + "mix.right.o": (w, r)})
        elif spec["type"] == "channel_delta":
            qk, v, dec = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"], m["heads"] * m["dim"]
            ra, rg = low_rank + i, low_rank + 2 + i  # the two low-rank maps have inner sizes of their own
            for n, rows in (("q", qk), ("k", qk), ("v", v)):
                shapes[p + f"mix.{n}"] = (rows, w)
                shapes[p + f"mix.{n}.conv"] = (rows, m["conv"])
            shapes.update({p + "mix.b": (m["heads"], w), p + "mix.A_log": (m["heads"],), p + "mix.norm": (m["vdim"],), p + "mix.a1": (ra, w), p + "mix.a2": (dec, ra),
                           p + "mix.dt_bias": (dec,), p + "mix.g1": (rg, w), p + "mix.g2": (v, rg), p + "mix.o": (w, v)})
        else:
            h = m["heads"]
            shapes.update({p + "mix.q": (h * (m["dim"] + m["rot_dim"]), w), p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], w), p + "mix.dkv.norm": (m["kv_rank"],),
                           p + "mix.uk": (h * m["dim"], m["kv_rank"]), p + "mix.uv": (h * m["vdim"], m["kv_rank"]), p + "mix.g": (h, w), p + "mix.o": (w, h * m["vdim"])})
        if spec["mlp"] is not None:
            numbers.append(2)
            shapes.update({p + "norm2": (w,), p + "mlp.up": (spec["mlp"]["ff"], w), p + "mlp.down": (w, spec["mlp"]["ff"])})
        for q in numbers:
            shapes.update({p + f"hc{q}.in": (S,), p + f"hc{q}.out": (S,), p + f"hc{q}.mix": (S, S)})
    return shapes


def weights(cfg, seed):
    rng = np.random.default_rng(seed)
    S = cfg["streams"]
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        parts = name.split(".")
        last = parts[-1]
        if len(parts) > 1 and parts[1].startswith("hc"):
            if last == "in":
                v = 1.0 / S + 0.2 * rng.standard_normal(shape)
            elif last == "out":
                v = 1.0 + 0.2 * rng.standard_normal(shape)
            else:
                v = 0.8 * np.eye(S) + 0.25 * rng.standard_normal(shape)
        elif last in ("norm", "norm1", "norm2"):
            v = 1.0 + 0.1 * rng.standard_normal(shape)
        elif last == "A_log":
            v = np.log(rng.uniform(0.05, 2.0, size=shape))
        elif last == "dt_bias":
            v = rng.uniform(-3.5, 0.0, size=shape)
        elif last == "b" and len(shape) == 1:
            v = (-2.0 if parts[-2] == "z" else 0.0) + 0.5 * rng.standard_normal(shape)  # the update gate mostly keeps the state: it must be carried
        elif last == "conv":
            v = rng.standard_normal(shape) / np.sqrt(shape[-1]) + (np.arange(shape[-1]) == shape[-1] - 1)
        elif name == "embed":
            v = rng.standard_normal(shape)
        else:
            gain = 2.0 if last in ("a2", "g2", "g", "z") else 1.0
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
