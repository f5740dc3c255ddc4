"""Dibulix, plain and slow: NumPy float64, one whole sequence at a time, no
cache (every attention position looks at the whole prefix) and recurrences
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
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_norm(x, weight, eps):
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * weight


# ---- rotary positions ----------------------------------------------------------------------------------------
def rotary_frequencies(dims, base, scaling=None):
    """(f_i for i < dims / 2, the factor on cosine and sine).  ``scaling``
    (factor, original, fast, slow) blends each frequency between itself and
    itself / factor along a ramp over the pair index."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turns_to_index(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turns_to_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turns_to_index(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, dims, base, layout, scaling=None):
    """x [T, heads, hd]: the first ``dims`` numbers of every head turned by the
    position; ``layout`` "pairs" joins 2i with 2i + 1, "halves" i with i + dims / 2."""
    if not dims:
        return x
    f, mag = rotary_frequencies(dims, base, scaling)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(ang) * mag)[:, None, :], (np.sin(ang) * mag)[:, None, :]
    out = x.copy()
    if layout == "pairs":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        half = dims // 2
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


# ---- softmax attention ---------------------------------------------------------------------------------------
def attend(q, k, v, scale, window, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  Position i sees j
    with 0 <= i - j < window (None: every j <= i); ``sink`` adds one to the
    softmax's denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = 0 if not window else max(0, i - window + 1)
            s = (k[lo : i + 1, g] @ q[i, h]) * scale
            m = max(s.max(), 0.0) if sink else s.max()
            e = np.exp(s - m)
            den = e.sum() + (math.exp(-m) if sink else 0.0)
            out[i, h] = (e / den) @ v[lo : i + 1, g]
    return out


def windowed_attention(h, w, p, m):
    """The left branch of the 'parallel' mixer."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]

    def proj(name):
        y = h @ w[p + name].T
        return y + w[p + name + ".b"] if p + name + ".b" in w else y

    q, k, v = proj("q").reshape(T, H, d), proj("k").reshape(T, G, d), proj("v").reshape(T, G, dv)
    rot = m.get("rot")
    if rot:
        pos = np.arange(T)
        q = rotate(q, pos, rot["dims"], rot["base"], "pairs")
        k = rotate(k, pos, rot["dims"], rot["base"], "pairs")
    window = (m.get("mask") or {}).get("size")
    o = attend(q, k, v, m["scale"], window, sink=True)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def min_gru_recurrence(z_logit, u, gate_logit):
    """All [T, width]: the state after every token, times silu(gate)."""
    z = sigmoid(z_logit)
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    S = np.zeros(z.shape[1])
    out = np.zeros_like(z)
    for t in range(z.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        out[t] = S * silu(gate_logit[t])
    return out


def min_gru(h, w, p):
    """The right branch of the 'parallel' mixer."""
    return min_gru_recurrence(h @ w[p + "z"].T + w[p + "z.b"], h @ w[p + "x"].T + w[p + "x.b"], h @ w[p + "g"].T) @ w[p + "o"].T


def parallel_mixer(h, w, p, m):
    return m["left_scale"] * windowed_attention(h, w, p + "left.", m["left"]) + m["right_scale"] * min_gru(h, w, p + "right.")


def short_convolution(u, taps_w):
    """u [T, C]; taps_w [C, taps], the last column multiplies the token itself; zeros before the start; then silu."""
    T, taps = u.shape[0], taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, u.shape[1])), u], axis=0)
    out = np.zeros_like(u)
    for l in range(taps):
        out += padded[l : l + T] * taps_w[:, l][None, :]
    return silu(out)


def delta_rule(q, k, v, beta, g):
    """q, k [T, H, d] (already per value head), v [T, H, dv], beta [T, H], g [T, H, d] -> [T, H, dv]."""
    T, H, d = q.shape
    dv = v.shape[2]
    out = np.zeros((T, H, dv))
    for h in range(H):
        S = np.zeros((d, dv))
        for t in range(T):
            S = g[t, h][:, None] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, h])
            S = S + np.outer(k[t, h], u)
            out[t, h] = S.T @ q[t, h]
    return out


def unit_vectors(x):
    return x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)


def channel_decays(logits, dt_bias, a_log):
    """logits [T, H, d] -> g = exp(-exp(A_log_h) * softplus(logits + dt_bias))."""
    T, H, d = logits.shape
    return np.exp(-np.exp(a_log)[None, :, None] * softplus(logits + dt_bias.reshape(1, H, d)))


def channel_delta_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_convolution(h @ w[p + "q"].T, w[p + "q.conv"]).reshape(T, G, d)
    k = short_convolution(h @ w[p + "k"].T, w[p + "k.conv"]).reshape(T, G, d)
    v = short_convolution(h @ w[p + "v"].T, w[p + "v.conv"]).reshape(T, H, dv)
    q = unit_vectors(q) * d ** -0.5
    k = unit_vectors(k)
    heads_of = np.arange(H) // (H // G)
    q, k = q[:, heads_of], k[:, heads_of]
    beta = sigmoid(h @ w[p + "b"].T)
    g = channel_decays(((h @ w[p + "a1"].T) @ w[p + "a2"].T).reshape(T, H, d), w[p + "dt_bias"], w[p + "A_log"])
    o = delta_rule(q, k, v, beta, g)
    o = o / np.sqrt((o * o).mean(-1, keepdims=True) + eps) * w[p + "norm"][None, None, :]
    o = o * sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).reshape(T, H, dv)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def latent_attention_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[p + "q"].T).reshape(T, H, d + r)
    low = h @ w[p + "dkv"].T
    c = rms_norm(low[:, :rank], w[p + "dkv.norm"], eps)
    kr = low[:, rank:].reshape(T, 1, r)
    rot = m.get("rot") or {}
    pos = np.arange(T)
    if r:
        qr = rotate(q[:, :, d:], pos, rot.get("dims", 0), rot.get("base", 1.0), "halves", rot.get("scaling"))
        kr = rotate(kr, pos, rot.get("dims", 0), rot.get("base", 1.0), "halves", rot.get("scaling"))
    else:
        qr = q[:, :, d:]
    ku = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    qq = np.concatenate([q[:, :, :d], qr], axis=-1)
    kk = np.concatenate([ku, np.repeat(kr, H, axis=1)], axis=-1)
    window = (m.get("mask") or {}).get("size")
    o = attend(qq, kk, v, m["scale"], window, sink=False)
    o = o * sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T


def dense_feed_forward(h, w, p):
    a = np.maximum(h @ w[p + "up"].T, 0.0)
    return (a * a) @ w[p + "down"].T


def mixer(kind, h, w, p, m, eps):
    if kind == "parallel":
        return parallel_mixer(h, w, p, m)
    if kind == "channel_delta":
        return channel_delta_mixer(h, w, p, m, eps)
    if kind == "latent_attention":
        return latent_attention_mixer(h, w, p, m, eps)
    raise ValueError(kind)


def connect(xs, y, w_mix, w_out):
    """Every stream at once from the old ones: x_t <- sum_s mix[s, t] x_s + out[t] y."""
    S = len(xs)
    return [sum(w_mix[s, t] * xs[s] for s in range(S)) + w_out[t] * y for t in range(S)]


def greedy(w, cfg, prompt, n_new):
    """The next ``n_new`` tokens by the largest logit, the whole sequence recomputed for each."""
    seq, out = list(prompt), []
    for _ in range(n_new):
        tok = int(np.argmax(forward(w, cfg, seq)[-1]))
        out.append(tok)
        seq.append(tok)
    return out


def forward(w, cfg, ids, layer_outputs=None):
    """Logits [T, vocab] of one whole sequence.  ``layer_outputs`` (a list)
    collects the residual stream after every layer (the streams' sum)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(ids)]
    streams = cfg.get("streams")
    xs = [x.copy() for _ in range(streams)] if streams else None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        subs = [(1, lambda u: mixer(layer["type"], u, w, p + "mix.", layer["mixer"], eps))]
        if layer.get("mlp") is not None:
            subs.append((2, lambda u: dense_feed_forward(u, w, p + "mlp.")))
        for number, f in subs:
            if xs is None:
                x = x + f(rms_norm(x, w[p + f"norm{number}"], eps))
                continue
            hc = p + f"hc{number}."
            u = sum(w[hc + "in"][s] * xs[s] for s in range(streams))
            y = f(rms_norm(u, w[p + f"norm{number}"], eps))
            xs = connect(xs, y, w[hc + "mix"], w[hc + "out"])
        if layer_outputs is not None:
            layer_outputs.append(sum(xs) if xs is not None else x.copy())
    if xs is not None:
        x = sum(xs)
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T * cfg["logit_scale"]
