"""Kikerax, plain and slow: NumPy float64, one whole sequence at a time, no
cache (every attention position looks at its whole prefix) and the recurrence
walked token by token from a zero state, one function per mechanism.  It
shares nothing with the package: it reads config.json as a dict and
model.safetensors with its own few lines."""
import json
import math
import struct
from pathlib import Path

import numpy as np


def load(folder):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    meta = json.loads(raw[8 : 8 + n])
    data = raw[8 + n :]
    w = {}
    for name, m in meta.items():
        if name == "__metadata__":
            continue
        lo, hi = m["data_offsets"]
        if m["dtype"] == "BF16":
            arr = (np.frombuffer(data[lo:hi], dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif m["dtype"] == "F32":
            arr = np.frombuffer(data[lo:hi], dtype="<f4").astype(np.float64)
        else:
            raise ValueError(m["dtype"])
        w[name] = arr.reshape(m["shape"])
    return w, cfg


def sigmoid(z):
    return 0.5 * (1.0 + np.tanh(0.5 * np.asarray(z, dtype=np.float64)))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_norm(x, weight, eps):
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * weight


def softmax_rows(s):
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


# ---- rotary positions ----------------------------------------------------------------------------------------
def rotary_frequencies(dims, base, scaling=None):
    """(f_i for i < dims / 2, the factor on cosine and sine)."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, dims, base, scaling=None):
    """x [T, units, d]: the first ``dims`` numbers of every unit, 2i with 2i + 1, turned by the position."""
    if not dims:
        return x
    f, mag = rotary_frequencies(dims, base, scaling)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(ang) * mag)[:, None, :], (np.sin(ang) * mag)[:, None, :]
    out = x.copy()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ---- masks ---------------------------------------------------------------------------------------------------
def causal_mask(T):
    i = np.arange(T)
    return i[None, :] <= i[:, None]


def chunk_mask(T, size):
    i = np.arange(T)
    return (i[None, :] <= i[:, None]) & ((i[None, :] // size) == (i[:, None] // size))


def masked_softmax(scores, mask):
    return softmax_rows(np.where(mask, scores, -np.inf))


# ---- attention beside the recurrence ---------------------------------------------------------------------------
def keyed_attention(w, p, m, h, eps):
    """Softmax attention whose values are the keys as projected (before their
    norm): weighted RMS norm of q and k per head, queries growing with the
    logarithm of the position, capped scores, a sigmoid gate per head."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T).reshape(T, H, d)
    k = (h @ w[p + "k"].T).reshape(T, G, d)
    v = k
    qn, kn = rms_norm(q, w[p + "q.norm"], eps), rms_norm(k, w[p + "k.norm"], eps)
    if m.get("q_temp"):
        pos = np.arange(T)
        qn = qn * (1.0 + m["q_temp"]["coef"] * np.log(np.floor((pos + 1) / m["q_temp"]["every"]) + 1.0))[:, None, None]
    mask = causal_mask(T)
    gate = sigmoid(h @ w[p + "g"].T)
    out = np.zeros((T, H, v.shape[-1]))
    for a in range(H):
        g = a // (H // G)
        s = (qn[:, a] @ kn[:, g].T) * m["scale"]
        if m.get("softcap"):
            s = m["softcap"] * np.tanh(s / m["softcap"])
        out[:, a] = masked_softmax(s, mask) @ v[:, g]
    out = out * gate[:, :, None]
    return out.reshape(T, -1) @ w[p + "o"].T


def causal_conv(x, taps, bias):
    """x [T, C], taps [C, K] (last column: the current token), zeros before the start."""
    T, K = x.shape[0], taps.shape[1]
    out = np.zeros_like(x)
    for j in range(K):
        back = K - 1 - j
        out[back:] += x[: T - back] * taps[:, j] if back else x * taps[:, j]
    return out + bias


def gated_recurrent_unit(w, p, m, h):
    """y = gelu(W_y h + b); u = conv(W_x h + b); per block r, i = sigmoid(A_b u_b + b); a = exp(-8 r softplus(lam));
    S_t = a S_(t-1) + sqrt(1 - a^2) i u; out = W_o (S * y)."""
    T, width, B = h.shape[0], m["width"], m["blocks"]
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    ub = u.reshape(T, B, width // B)
    r = sigmoid(np.einsum("tbi,boi->tbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(T, width)
    i = sigmoid(np.einsum("tbi,boi->tbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(T, width)
    a = np.exp(-8.0 * r * softplus(w[p + "lam"]))
    drive = np.sqrt(1.0 - a * a) * i * u
    S = np.zeros(width)
    states = np.zeros((T, width))
    for t in range(T):
        S = a[t] * S + drive[t]
        states[t] = S
    return (states * y) @ w[p + "o"].T


def parallel_mixer(w, p, m, h, eps):
    return m["left_scale"] * keyed_attention(w, p + "left.", m["left"], h, eps) + m["right_scale"] * gated_recurrent_unit(w, p + "right.", m["right"], h)


# ---- differential attention ------------------------------------------------------------------------------------
def difference_weight(w, p, diff):
    return math.exp(float((w[p + "lq1"] * w[p + "lk1"]).sum())) - math.exp(float((w[p + "lq2"] * w[p + "lk2"]).sum())) + diff


def differential_attention(w, p, m, h, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H * 2, d)  # head by head, [map 1, map 2]
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G * 2, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    q, k = rms_norm(q, w[p + "q.norm"], eps), rms_norm(k, w[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot:
        pos = np.arange(T)
        q = rotate_pairs(q, pos, rot["dims"], rot["base"], rot.get("scaling"))
        k = rotate_pairs(k, pos, rot["dims"], rot["base"], rot.get("scaling"))
    mask = chunk_mask(T, m["mask"]["size"]) if m.get("mask") else causal_mask(T)
    lam = difference_weight(w, p, m["diff"])
    gate = sigmoid(h @ w[p + "g"].T)
    out = np.zeros((T, H, dv))
    for a in range(H):
        g = a // (H // G)
        maps = [masked_softmax((q[:, 2 * a + j] @ k[:, 2 * g + j].T) * m["scale"], mask) @ v[:, g] for j in range(2)]
        o = maps[0] - lam * maps[1]
        out[:, a] = o / np.sqrt((o * o).mean(axis=-1, keepdims=True) + eps) * (1.0 - m["diff"])
    out = out * gate[:, :, None]
    return out.reshape(T, -1) @ w[p + "o"].T + w[p + "o.b"]


# ---- feed-forwards -----------------------------------------------------------------------------------------------
def dense_ff(w, p, h):
    return gelu_tanh(h @ w[p + "up"].T) @ w[p + "down"].T


def gated_expert(w, p, h):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(w, p, r, h):
    """(chosen experts [T, top], their weights [T, top], margin [T]) for every token; ``margin`` is the smallest gap
    between what was taken and what was not (choice scores of experts, scores of groups), so that tests know a
    close call."""
    E, top = r["experts"], r["top"]
    s = sigmoid(h @ w[p + "router"].T)
    c = s + w[p + "correction"]
    groups = r.get("groups")
    group_margin = np.full(len(c), np.inf)
    if groups:
        per = E // groups["count"]
        cg = c.reshape(-1, groups["count"], per)
        gscore = np.sort(cg, axis=-1)[..., -2:].sum(axis=-1) if per >= 2 else cg.sum(axis=-1)
        order = np.argsort(-gscore, axis=-1, kind="stable")
        allowed = np.zeros_like(gscore, dtype=bool)
        np.put_along_axis(allowed, order[:, : groups["keep"]], True, axis=-1)
        if groups["keep"] < groups["count"]:
            ranked_groups = -np.sort(-gscore, axis=-1)
            group_margin = ranked_groups[:, groups["keep"] - 1] - ranked_groups[:, groups["keep"]]
        c = np.where(np.repeat(allowed, per, axis=-1), c, -np.inf)
    chosen = np.argsort(-c, axis=-1, kind="stable")[:, :top]
    picked = np.take_along_axis(s, chosen, axis=-1)
    weights = picked / (picked.sum(axis=-1, keepdims=True) + 1e-20) * r["scale"]
    ranked = -np.sort(-c, axis=-1)
    margin = ranked[:, top - 1] - ranked[:, top] if E > top else np.full(len(c), np.inf)
    return chosen, weights, np.minimum(margin, group_margin)


def routed_ff(w, p, mlp, h):
    chosen, weights, _ = route(w, p, mlp["router"], h)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t], weights[t]):
            out[t] += g * gated_expert(w, f"{p}e{e}.", h[t : t + 1])[0]
    if mlp.get("shared"):
        out += gated_expert(w, p + "shared.", h)
    return out


# ---- the model ----------------------------------------------------------------------------------------------------
def layer_forward(w, cfg, i, x):
    spec, eps, p = cfg["layers"][i], cfg["norm"]["eps"], f"l{i}."
    if spec["type"] == "parallel":
        y = parallel_mixer(w, p + "mix.", spec["mixer"], x, eps)
    elif spec["type"] == "attention":
        y = differential_attention(w, p + "mix.", spec["mixer"], x, eps)
    else:
        raise ValueError(spec["type"])
    x = x + rms_norm(y, w[p + "norm1"], eps)
    mlp = spec.get("mlp")
    if mlp:
        y = dense_ff(w, p + "mlp.", x) if mlp["kind"] == "dense" else routed_ff(w, p + "mlp.", mlp, x)
        x = x + rms_norm(y, w[p + "norm2"], eps)
    return x


def forward(w, cfg, tokens, streams=False):
    """Logits [T, vocab] of one whole sequence; with ``streams`` also the residual stream after every layer."""
    x = w["embed"][np.asarray(tokens)]
    after = []
    for i in range(len(cfg["layers"])):
        x = layer_forward(w, cfg, i, x)
        after.append(x.copy())
    logits = rms_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["embed"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * np.tanh(logits / cap)
    return (logits, np.stack(after)) if streams else logits


def router_margins(w, cfg, tokens):
    """The smallest router margin at every position over all routed layers (inf without one)."""
    x = w["embed"][np.asarray(tokens)]
    worst = np.full(len(tokens), np.inf)
    for i, spec in enumerate(cfg["layers"]):
        p, eps = f"l{i}.", cfg["norm"]["eps"]
        y = parallel_mixer(w, p + "mix.", spec["mixer"], x, eps) if spec["type"] == "parallel" else differential_attention(w, p + "mix.", spec["mixer"], x, eps)
        x = x + rms_norm(y, w[p + "norm1"], eps)
        mlp = spec.get("mlp")
        if mlp:
            if mlp["kind"] == "moe":
                worst = np.minimum(worst, route(w, p + "mlp.", mlp["router"], x)[2])
                y = routed_ff(w, p + "mlp.", mlp, x)
            else:
                y = dense_ff(w, p + "mlp.", x)
            x = x + rms_norm(y, w[p + "norm2"], eps)
    return worst


def sure_prefix(margins, least=0.02):
    """How many leading positions come before the first close call of any router (a margin below ``least``)."""
    close = np.asarray(margins) < least
    return int(np.argmax(close)) if close.any() else len(close)


def greedy(w, cfg, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(np.argmax(forward(w, cfg, seq)[-1])))
    return seq[len(prompt):]
