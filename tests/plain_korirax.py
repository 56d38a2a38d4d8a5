"""A plain statement of the Korirax decoder in numpy float64: one function per mechanism, whole
sequences at once, no cache.  It shares nothing with the engine: it reads the checkpoint itself
and takes the configuration as the dictionary that config.json holds.

Notation: x is the residual stream [T, width] of ONE request, positions are 0 .. T-1, weights are
[out, in] and applied as x @ W.T.
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np


def read_checkpoint(path):
    """name -> float64 array (integer tables stay integers) of a safetensors file."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, rec in head.items():
        if name == "__metadata__":
            continue
        a, b = rec["data_offsets"]
        raw = data[a:b]
        if rec["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(np.float32).astype(np.float64)
        elif rec["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif rec["dtype"] == "I32":
            arr = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(rec["dtype"])
        out[name] = arr.reshape(rec["shape"])
    return out


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    erf = np.vectorize(math.erf)
    return 0.5 * z * (1.0 + erf(z / math.sqrt(2.0)))


def softplus(z):
    return np.logaddexp(0.0, z)


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


def softmax_rows(s):
    s = s - s.max(axis=-1, keepdims=True)
    e = np.exp(s)
    return e / e.sum(axis=-1, keepdims=True)


# ---------------------------------------------------------------- positions

def yarn_frequencies(dims, base, scaling):
    """Frequencies of the dims/2 rotated pairs and the factor on cos and sin."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def where(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(scaling["fast"])), 0)
    hi = min(math.ceil(where(scaling["slow"])), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(v, pos, freq, mult):
    """v [T, ..., dims] with pairs (2i, 2i+1) turned by pos * freq[i]; cos and sin times mult."""
    T = v.shape[0]
    ang = pos.astype(np.float64)[:, None] * freq[None, :]
    shape = (T,) + (1,) * (v.ndim - 2) + (freq.shape[0],)
    c, s = (np.cos(ang) * mult).reshape(shape), (np.sin(ang) * mult).reshape(shape)
    a, b = v[..., 0::2], v[..., 1::2]
    out = np.empty_like(v)
    out[..., 0::2] = a * c - b * s
    out[..., 1::2] = b * c + a * s
    return out


def distance_bucket(n, rows, far):
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


# ---------------------------------------------------------------- mixers

def mix_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    pos = np.arange(T)
    qt = m.get("q_temp")
    if qt:
        temp = 1.0 + qt["coef"] * np.log(np.floor((pos + 1) / qt["every"]) + 1.0)
        q = q * temp[:, None, None]
    rel = w[p + "rel"]
    rows = rel.shape[0]
    buckets = np.array([distance_bucket(n, rows, m["bias_max"]) for n in range(T)], dtype=np.int64)
    dist = pos[:, None] - pos[None, :]
    seen = dist >= 0
    bias = rel[buckets[np.where(seen, dist, 0)]]            # [T, T, H]
    out = np.empty((T, H, dv))
    for n in range(H):
        g = n // (H // G)
        s = q[:, n] @ k[:, g].T * m["scale"] + bias[:, :, n]
        s = np.where(seen, s, -np.inf)
        out[:, n] = softmax_rows(s) @ v[:, g]
    out = out.reshape(T, H * dv) * sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def mix_latent(h, w, p, m, eps):
    T = h.shape[0]
    H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, d + dr)
    kv = h @ w[p + "dkv"].T
    c = rms_norm(kv[:, :R], w[p + "dkv.norm"], eps)
    k_rot = kv[:, R:]
    pos = np.arange(T)
    rot = m["rot"]
    freq, mult = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    rd = rot["dims"]
    q_rot = q[:, :, d:].copy()
    q_rot[:, :, :rd] = rotate_interleaved(q_rot[:, :, :rd], pos, freq, mult)
    k_rot = k_rot.copy()
    k_rot[:, :rd] = rotate_interleaved(k_rot[:, :rd], pos, freq, mult)
    k = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    seen = pos[:, None] >= pos[None, :]
    out = np.empty((T, H, dv))
    for n in range(H):
        s = (q[:, n, :d] @ k[:, n].T + q_rot[:, n] @ k_rot.T) * m["scale"]
        out[:, n] = softmax_rows(np.where(seen, s, -np.inf)) @ v[:, n]
    out = out.reshape(T, H * dv) * sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def causal_conv(x, taps_w, bias):
    """x [T, C]; taps_w [C, taps], last column the current token's; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C)), x], axis=0)
    out = np.zeros((T, C))
    for j in range(taps):
        out += padded[j:j + T] * taps_w[:, j]
    return out + bias


def mix_rglru(h, w, p, m, eps):
    T = h.shape[0]
    width, blocks = m["width"], m["blocks"]
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    ub = u.reshape(T, blocks, width // blocks)
    r = sigmoid(np.einsum("tbi,boi->tbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(T, width)
    i = sigmoid(np.einsum("tbi,boi->tbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(T, width)
    log_a = -8.0 * r * softplus(w[p + "lam"])
    a = np.exp(log_a)
    drive = np.sqrt(1.0 - a * a) * i * u
    S = np.zeros(width)
    states = np.empty((T, width))
    for t in range(T):
        S = a[t] * S + drive[t]
        states[t] = S
    return (states * y) @ w[p + "o"].T


# ---------------------------------------------------------------- feed-forward

def ff_dense(h, w, p):
    g = h @ w[p + "gate"].T
    return (g * sigmoid(g) * (h @ w[p + "up"].T)) @ w[p + "down"].T


MARGINS = None      # a list, while a caller wants to know how close the routers' calls were: (token, margin) of every call


def _margin(sorted_desc, kept):
    """Per row: the gap between the last value that is kept and the best that is not (inf where all are kept)."""
    if kept >= sorted_desc.shape[-1]:
        return np.full(sorted_desc.shape[0], np.inf)
    gap = sorted_desc[:, kept - 1] - sorted_desc[:, kept]
    return np.where(np.isnan(gap), np.inf, gap)        # -inf minus -inf: closed experts on both sides


def route(h, w, p, r):
    """Chosen experts [T, top] and their weights."""
    E, top = r["experts"], r["top"]
    s = sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"]
    groups = r.get("groups")
    margin = np.full(h.shape[0], np.inf)
    if groups and groups["count"] > 1:
        per = E // groups["count"]
        byg = choice.reshape(-1, groups["count"], per)
        gs = np.sort(byg, axis=-1)[..., -2:].sum(axis=-1) if per > 1 else byg[..., 0]
        keep = np.argsort(-gs, axis=-1, kind="stable")[:, :groups["keep"]]
        margin = np.minimum(margin, _margin(-np.sort(-gs, axis=-1), groups["keep"]))
        allowed = np.zeros(gs.shape, dtype=bool)
        np.put_along_axis(allowed, keep, True, axis=-1)
        choice = np.where(np.repeat(allowed, per, axis=-1), choice, -np.inf)
    ids = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    if MARGINS is not None:
        with np.errstate(invalid="ignore"):
            margin = np.minimum(margin, _margin(-np.sort(-choice, axis=-1), top))
        MARGINS.extend(enumerate(margin))
    ws = np.take_along_axis(s, ids, axis=-1)
    ws = ws / (ws.sum(axis=-1, keepdims=True) + 1e-20) * r.get("scale", 1.0)
    return ids, ws


def expert(h, up, down):
    return gelu_erf(h @ up.T) @ down.T


def ff_moe(h, w, p, f):
    ids, ws = route(h, w, p, f["router"])
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, g in zip(ids[t], ws[t]):
            out[t] += g * expert(h[t:t + 1], w[p + f"e{e}.up"], w[p + f"e{e}.down"])[0]
    if f.get("shared"):
        out += expert(h, w[p + "shared.up"], w[p + "shared.down"])
    return out


# ---------------------------------------------------------------- the model

def token_side(x, tokens, w, i, dim, eps):
    p = f"l{i}.side."
    e = w["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    g = gelu_tanh(x @ w[p + "gate"].T) * e
    y = g @ w[p + "proj"].T
    return x + unit_rms(y, eps) * w[p + "norm"]


def layer(x, tokens, w, cfg, i):
    L = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    h = rms_norm(x, w[f"l{i}.norm1"], eps)
    mixers = {"attention": mix_attention, "latent_attention": mix_latent, "rglru": mix_rglru}
    add = mixers[L["type"]](h, w, f"l{i}.mix.", L["mixer"], eps)
    f = L.get("mlp")
    if f:
        add = add + (ff_dense(h, w, f"l{i}.mlp.") if f["kind"] == "dense" else ff_moe(h, w, f"l{i}.mlp.", f))
    x = x + add
    side = cfg.get("token_side")
    if side and side.get("dim"):
        x = token_side(x, tokens, w, i, side["dim"], eps)
    return x


def layer_runs(cfg):
    """(layer, pass number or None, first of its pass) in the order of execution."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop.get("times", 1) < 1:
        return [(i, None, False) for i in range(n)]
    runs = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None, False) for i in range(loop["stop"], n)]


def forward(tokens, w, cfg, streams=None):
    """Logits [T, vocab] of one request given whole; ``streams`` collects x after every layer run."""
    tokens = np.asarray(tokens, dtype=np.int64)
    x = w["embed"][tokens] * cfg.get("embedding", {}).get("scale", 1.0)
    for i, t, first in layer_runs(cfg):
        if first:
            x = x + w["loop.step"][t]
        x = layer(x, tokens, w, cfg, i)
        if streams is not None:
            streams.append(x.copy())
    return rms_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T
