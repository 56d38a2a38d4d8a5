"""Plain restatement of the Toredra decoder, for tests only.

Whole sequences, no cache, no batching, numpy float64 throughout, one function per mechanism.
Nothing here is imported by the engine and nothing of the engine is imported here: the file has
its own reader of config.json and of safetensors.

Notation.  T tokens at positions 0..T-1, width D, e the embedded tokens.  A layer is

    y = mixer(norm1(x));  x <- x + norm1b(y * sigmoid(rg1 norm1(x) + b1))
    z = ff(norm2(x));     x <- x + norm2b(z * sigmoid(rg2 norm2(x) + b2))

(a sublayer's result is gated by its own input, normed again, and only then added).  Layers
start..stop-1 of the list run `times` times with the same weights and a fresh memory each pass;
from the second pass on e is added to x in front of the pass.  Two mixers: `parallel` (softmax
attention with rotated heads and a learned extra term in the denominator, beside a gated linear
recurrence; the mean of the two, each normed) and `general_delta` (a recurrence whose state decays
per key channel and loses what it holds along the current unit key before it is written).
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np

F = np.float64


def read_safetensors(path: str) -> dict:
    with open(path, "rb") as f:
        blob = f.read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen].decode("utf-8"))
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = blob[base + b: base + e]
        dt = info["dtype"]
        if dt == "BF16":
            arr = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(F)
        elif dt == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(F)
        elif dt == "I32":
            arr = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name}")
        out[name] = arr.reshape(tuple(info["shape"])).copy()
    return out


def read_model(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ---- small functions -------------------------------------------------------------------------

def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


def linear(x, w, b=None):
    """Rows of x times w^T, w stored [out, in]."""
    y = x @ w.T
    return y if b is None else y + b


def relu_squared(z):
    r = np.maximum(z, 0.0)
    return r * r


# ---- rotation --------------------------------------------------------------------------------

def rotary_frequencies(rot: dict) -> np.ndarray:
    """One frequency per pair of the first rot['dims'] dimensions, base^(-2i/dims), stretched for
    long wavelengths: wavelengths under original/high keep their frequency, those over original/low
    get frequency/factor, the ones between are blended linearly in original/wavelength."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = []
        for fi in f:
            wave = 2.0 * math.pi / fi
            if wave < orig / high:
                out.append(fi)
            elif wave > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wave - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = np.array(out, dtype=F)
    return f


def rotate_interleaved(x: np.ndarray, positions: np.ndarray, freq: np.ndarray) -> np.ndarray:
    """x [T, heads, d]: dimensions 2i and 2i+1 (i < len(freq)) turn by positions * freq[i]; the rest
    of a head passes unchanged."""
    out = x.copy()
    n = freq.shape[0]
    ang = positions[:, None].astype(F) * freq[None, :]          # [T, n]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out[..., 0:2 * n:2] = u * c - v * s
    out[..., 1:2 * n:2] = v * c + u * s
    return out


# ---- mixers ----------------------------------------------------------------------------------

def sink_attention(q, k, v, scale, sink):
    """Causal softmax attention, q [T, H, d], k [T, G, d], v [T, G, dv], query head h on key head
    h // (H / G); the denominator of head h also holds exp(sink[h]), which carries no value."""
    T, H, _ = q.shape
    G, dv = k.shape[1], v.shape[2]
    out = np.zeros((T, H, dv), dtype=F)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            s = (k[:i + 1, g] @ q[i, h]) * scale
            m = max(float(s.max()), float(sink[h]))
            p = np.exp(s - m)
            out[i, h] = (p @ v[:i + 1, g]) / (p.sum() + math.exp(float(sink[h]) - m))
    return out


def rotary_sink_mixer(h, W, p, m, eps):
    """The attention side of a parallel mixer: biased projections, rotated q and k, sink softmax."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = linear(h, W[p + "q"], W[p + "q.b"]).reshape(T, H, d)
    k = linear(h, W[p + "k"], W[p + "k.b"]).reshape(T, G, d)
    v = linear(h, W[p + "v"], W[p + "v.b"]).reshape(T, G, dv)
    freq = rotary_frequencies(m["rot"])
    pos = np.arange(T)
    q, k = rotate_interleaved(q, pos, freq), rotate_interleaved(k, pos, freq)
    o = sink_attention(q, k, v, float(m["scale"]), W[p + "sink"])
    return linear(o.reshape(T, H * dv), W[p + "o"])


def gated_linear_recurrence(q, f, v):
    """Per head S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T, o_t = S_t^T q_t; q, f [T, H, d], v [T, H, dv]."""
    T, H, d = q.shape
    dv = v.shape[2]
    out = np.zeros((T, H, dv), dtype=F)
    S = np.zeros((H, d, dv), dtype=F)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = np.einsum("hdv,hd->hv", S, q[t])
    return out


def forget_gate_mixer(h, W, p, m, eps):
    """The recurrent side of a parallel mixer: the forget gate, bounded below, also sets what is written."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(linear(h, W[p + "q"])).reshape(T, H, d)
    v = linear(h, W[p + "v"]).reshape(T, H, dv)
    low = W[p + "lower"]
    f = (low + (1.0 - low) * sigmoid(linear(h, W[p + "f"], W[p + "f.b"]))).reshape(T, H, d)
    o = gated_linear_recurrence(q, f, v)
    o = rms_norm(o, W[p + "norm"], eps)
    return linear(o.reshape(T, H * dv), W[p + "o"])


def parallel_mixer(h, W, p, m, eps):
    left = rotary_sink_mixer(h, W, p + "left.", m["left"], eps)
    right = forget_gate_mixer(h, W, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, W[p + "left.out"], eps) + rms_norm(right, W[p + "right.out"], eps))


DECAY_RATE = math.exp(-0.5)


def removal_recurrence(r, k, v, w, a):
    """Per head, with u = k / sqrt(sum k^2 + 1e-6):
    S_t = diag(w_t) S_{t-1} - (a_t * u_t) (u_t^T S_{t-1}) + k_t v_t^T, o_t = S_t^T r_t.  All [T, H, d]."""
    T, H, d = r.shape
    out = np.zeros((T, H, d), dtype=F)
    S = np.zeros((H, d, d), dtype=F)
    for t in range(T):
        u = k[t] / np.sqrt(np.sum(k[t] * k[t], axis=-1, keepdims=True) + 1e-6)
        held = np.einsum("hd,hdv->hv", u, S)
        S = w[t][:, :, None] * S - (a[t] * u)[:, :, None] * held[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        out[t] = np.einsum("hdv,hd->hv", S, r[t])
    return out


def general_delta_mixer(h, W, p, m, eps):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    r = linear(h, W[p + "r"]).reshape(T, H, d)
    k = linear(h, W[p + "k"]).reshape(T, H, d)
    v = linear(h, W[p + "v"]).reshape(T, H, d)
    w = np.exp(-DECAY_RATE * sigmoid(linear(np.tanh(linear(h, W[p + "w1"])), W[p + "w2"]) + W[p + "w0"])).reshape(T, H, d)
    a = sigmoid(linear(h, W[p + "a"], W[p + "a.b"])).reshape(T, H, d)
    o = removal_recurrence(r, k, v, w, a)
    o = unit_rms(o, eps).reshape(T, H * d) * W[p + "norm"] * sigmoid(linear(h, W[p + "g"]))
    return linear(o, W[p + "o"])


def dense_ff(h, W, p):
    return linear(relu_squared(linear(h, W[p + "up"])), W[p + "down"])


# ---- the model -------------------------------------------------------------------------------

def layer_order(cfg: dict):
    """(layer index, pass number, first of its pass) for every layer run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, 0, False) for i in range(start)]
    for rep in range(times if stop > start else 0):
        runs += [(i, rep, i == start) for i in range(start, stop)]
    runs += [(i, 0, False) for i in range(max(stop, start), n)]
    return runs


def layer_forward(x, W, cfg, i):
    L, p, eps = cfg["layers"][i], f"l{i}.", float(cfg["norm"]["eps"])
    h = rms_norm(x, W[p + "norm1"], eps)
    if L["type"] == "parallel":
        y = parallel_mixer(h, W, p + "mix.", L["mixer"], eps)
    elif L["type"] == "general_delta":
        y = general_delta_mixer(h, W, p + "mix.", L["mixer"], eps)
    else:
        raise ValueError(f"plain: layer type {L['type']}")
    y = y * sigmoid(linear(h, W[p + "rg1"], W[p + "rg1.b"]))
    x = x + rms_norm(y, W[p + "norm1b"], eps)
    if L.get("mlp") is not None:
        h = rms_norm(x, W[p + "norm2"], eps)
        z = dense_ff(h, W, p + "mlp.") * sigmoid(linear(h, W[p + "rg2"], W[p + "rg2.b"]))
        x = x + rms_norm(z, W[p + "norm2b"], eps)
    return x


def forward(cfg: dict, W: dict, tokens, layers_out=None) -> np.ndarray:
    """Logits [T, vocab] of one sequence; ``layers_out``, a list, receives x after every layer run."""
    eps = float(cfg["norm"]["eps"])
    e = W["embed"][np.asarray(tokens)]
    x = e.copy()
    for i, rep, first in layer_order(cfg):
        if first and rep > 0:
            x = x + e
        x = layer_forward(x, W, cfg, i)
        if layers_out is not None:
            layers_out.append(x.copy())
    n = rms_norm(x, W["final.norm"], eps)
    logits = (n @ W["embed"].T) * float(cfg.get("logit_scale", 1.0))
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * np.tanh(logits / cap) if cap > 0 else logits
