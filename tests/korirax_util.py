"""Helpers of the Korirax tests: small configurations of their own, a writer of random weights whose scale lets every
mechanism matter, and the comparison of the engine with the plain implementation (`plain_korirax`).  The writer names
every tensor itself, so a weight slot that the engine forgets or misnames shows as a loading error."""
from __future__ import annotations

import functools
import json
import os
from typing import Dict, List, Tuple

import numpy as np

import plain_korirax as P
from zidivik_util import PartHarness, bf16_round, load_part, write_model  # noqa: F401  (helpers that know no architecture)


def attn(heads, kv_heads, dim, vdim, scale, bias_max, rows, q_temp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": bias_max, "bias_rows": rows}
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": "attention", "mixer": m}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, dims, base, scaling=None):
    rot = {"dims": dims, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank,
                                                  "kv_rank": kv_rank, "scale": scale, "rot": rot}}


def rglru(width, blocks, conv):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups, keep, scale, shared):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}},
            "shared": {"ff": shared} if shared else None}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


# K1: the looped stretch opens the model and runs three times; grouped heads with values narrower than keys; a query
# temperature that changes every 16 positions and a table of distance terms that is exhausted at distance 40; a rotated
# part with pairs in all three bands of the ramp; four blocks and four taps; three groups of experts of which two stay;
# a layer without feed-forward; a token input.
K1 = {"architecture": "Korirax", "vocab": 211, "width": 80, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0}, "token_side": {"dim": 12},
      "loop": {"start": 0, "stop": 2, "times": 3}, "layers": [
    layer(attn(6, 2, 24, 16, 0.2, 40, 10, (0.7, 16)), dense(96)),
    layer(latent(3, 16, 8, 24, 40, 48, 0.22, 8, 100.0, (8.0, 32, 4.0, 1.0)), moe(12, 3, 40, 3, 2, 1.7, 56)),
    layer(rglru(64, 4, 4), None),
    layer(latent(2, 24, 16, 8, 32, 40, 0.18, 16, 10000.0, (4.0, 64, 8.0, 2.0)), dense(72)),
]}
# K2: sizes that are no multiples of 8 (the plain kernels in bfloat16 too); no loop, no token input, no factor on the
# embedding, no query temperature, no stretching; fewer rotated dimensions than the rotated part has; five heads on one
# kv head; groups of one expert; experts without a shared one; two taps; an odd number of table rows.
K2 = {"architecture": "Korirax", "vocab": 97, "width": 70, "norm": {"eps": 1e-6}, "layers": [
    layer(rglru(42, 3, 2), dense(30)),
    layer(attn(5, 1, 12, 20, 0.3, 25, 7), moe(6, 2, 22, 6, 3, 1.0, 0)),
    layer(latent(5, 10, 6, 14, 26, 36, 0.25, 4, 50.0), dense(44)),
]}
# K3: heads of 128 and a cache row of 256 (the tensor-core kernels' largest), the loop in the middle, one block, one tap,
# a single expert chosen, every group kept.
K3 = {"architecture": "Korirax", "vocab": 131, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5}, "token_side": {"dim": 8},
      "loop": {"start": 1, "stop": 2, "times": 2}, "layers": [
    layer(attn(4, 2, 128, 128, 0.09, 300, 24, (0.3, 64)), moe(16, 1, 48, 4, 4, 2.0, 32)),
    layer(latent(2, 64, 64, 128, 48, 192, 0.1, 64, 100000.0, (16.0, 128, 16.0, 2.0)), dense(72)),
    layer(rglru(256, 1, 1), dense(48)),
]}
# K4: no routed experts (a run in bfloat16 cannot route otherwise than the plain one): long requests in reduced precision
K4 = {"architecture": "Korirax", "vocab": 151, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0}, "token_side": {"dim": 16},
      "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [
    layer(attn(4, 2, 32, 48, 0.15, 90, 12, (0.4, 50)), dense(128)),
    layer(rglru(128, 4, 3), dense(64)),
    layer(latent(4, 32, 16, 32, 64, 80, 0.15, 16, 1000.0, (4.0, 96, 8.0, 1.0)), None),
]}
CONFIGS = {"K1": (K1, 3), "K2": (K2, 8), "K3": (K3, 5), "K4": (K4, 13)}


def tensors_of(cfg: dict, seed: int) -> Dict[str, np.ndarray]:
    """Random float32 tensors for ``cfg``, by name.  Matrices N(0, g / sqrt(in)) so that activations keep their size through the
    layers; norm weights around 1; biases of order 1; distance terms of order 1; corrections that spread the experts' chances."""
    rng = np.random.default_rng(seed)
    D, V = cfg["width"], cfg["vocab"]
    W: Dict[str, np.ndarray] = {}

    def mat(name, out, inn, gain=1.0):
        W[name] = (rng.standard_normal((out, inn)) * gain / np.sqrt(inn)).astype(np.float32)

    def vec(name, shape, mean=0.0, std=1.0):
        W[name] = (mean + std * rng.standard_normal(shape)).astype(np.float32)

    W["embed"] = (rng.standard_normal((V, D)) / cfg.get("embedding", {}).get("scale", 1.0)).astype(np.float32)
    side = (cfg.get("token_side") or {}).get("dim", 0)
    if side:
        W["side.embed"] = rng.standard_normal((V, side * len(cfg["layers"]))).astype(np.float32)
    loop = cfg.get("loop")
    if loop:
        vec("loop.step", (loop["times"], D), 0.0, 0.5)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        vec(p + "norm1", D, 1.0, 0.1)
        if L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                mat(p + "mix." + n, rows, D, 1.5)
                vec(p + f"mix.{n}.b", rows, 0.0, 0.3)
            vec(p + "mix.q.norm", d, 1.0, 0.3)
            vec(p + "mix.k.norm", d, 1.0, 0.3)
            vec(p + "mix.rel", (m["bias_rows"], H), 0.0, 1.0)
            mat(p + "mix.g", H * dv, D, 2.0)
            mat(p + "mix.o", D, H * dv)
        elif L["type"] == "latent_attention":
            H, d, dr, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            mat(p + "mix.dq", Q, D)
            vec(p + "mix.dq.norm", Q, 1.0, 0.2)
            mat(p + "mix.uq", H * (d + dr), Q, 2.0)
            mat(p + "mix.dkv", R + dr, D, 1.5)
            vec(p + "mix.dkv.norm", R, 1.0, 0.2)
            mat(p + "mix.uk", H * d, R, 2.0)
            mat(p + "mix.uv", H * dv, R)
            mat(p + "mix.g", H * dv, D, 2.0)
            mat(p + "mix.o", D, H * dv)
        else:
            C, B = m["width"], m["blocks"]
            bw = C // B
            for n in ("y", "x"):
                mat(p + "mix." + n, C, D, 1.5)
                vec(p + f"mix.{n}.b", C, 0.0, 0.3)
            vec(p + "mix.conv", (C, m["conv"]), 0.3, 0.5)
            vec(p + "mix.conv.b", C, 0.0, 0.2)
            for n in ("ra", "ri"):
                W[p + "mix." + n] = (rng.standard_normal((B, bw, bw)) * 1.5 / np.sqrt(bw)).astype(np.float32)
                vec(p + f"mix.{n}.b", (B, bw), 0.0, 0.5)
            vec(p + "mix.lam", C, -2.0, 1.5)          # softplus(lam) from 0.02 to 1: decays from slow to fast
            mat(p + "mix.o", D, C)
        f = L.get("mlp")
        if f is not None and f["kind"] == "dense":
            mat(p + "mlp.gate", f["ff"], D, 1.5)
            mat(p + "mlp.up", f["ff"], D)
            mat(p + "mlp.down", D, f["ff"])
        elif f is not None:
            r = f["router"]
            mat(p + "mlp.router", r["experts"], D, 2.0)
            vec(p + "mlp.correction", r["experts"], 0.0, 0.3)
            for e in range(r["experts"]):
                mat(p + f"mlp.e{e}.up", f["expert"]["ff"], D, 1.5)
                mat(p + f"mlp.e{e}.down", D, f["expert"]["ff"])
            if f.get("shared"):
                mat(p + "mlp.shared.up", f["shared"]["ff"], D, 1.5)
                mat(p + "mlp.shared.down", D, f["shared"]["ff"])
        if side:
            mat(p + "side.gate", side, D, 1.5)
            mat(p + "side.proj", D, side)
            vec(p + "side.norm", D, 0.5, 0.1)
    vec("final.norm", D, 1.0, 0.1)
    mat("head", V, D)
    return W


@functools.lru_cache(maxsize=None)
def _model(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, P.read_checkpoint(os.path.join(model_dir, "model.safetensors"))


@functools.lru_cache(maxsize=None)
def _plain(model_dir: str, tokens: Tuple[int, ...]):
    cfg, W = _model(model_dir)
    P.MARGINS = []
    try:
        logits = P.forward(list(tokens), W, cfg)
        close = [t for t, m in P.MARGINS if m < CLOSE_CALL]
    finally:
        P.MARGINS = None
    return logits, (min(close) if close else len(tokens))


def plain_logits(model_dir: str, tokens) -> np.ndarray:
    return _plain(model_dir, tuple(int(t) for t in tokens))[0]


def first_close_call(model_dir: str, tokens) -> int:
    """First position at which some router separates what it keeps (a group, an expert) from the best it leaves out by
    less than `CLOSE_CALL`: from there on a run in reduced precision may route otherwise (len(tokens) if none)."""
    return _plain(model_dir, tuple(int(t) for t in tokens))[1]


CLOSE_CALL = 0.03
# |engine - plain| as a fraction of the largest |plain logit| of the request.  float32: sums in another order.  bfloat16:
# operands, activations between products and the cache are rounded to 8 bits of mantissa.  A fault of the cache, a state, a
# mask or a table moves the positions it touches by tenths; the float32 comparison on the same traces allows 2e-5.
TOL = {"float32": 2e-5, "bfloat16": 5e-2}


def compare_with_plain(model_dir_f32: str, reqs: Dict[str, List[int]], got, dtype: str, label: str = "") -> float:
    """Every logits row of a trace against the plain implementation.  In bfloat16, positions from a request's first close
    router call on are left out (the float32 run covers them).  Names the first wrong (request, position)."""
    worst, n = 0.0, 0
    for name, toks in reqs.items():
        ref = plain_logits(model_dir_f32, toks)
        scale = float(np.abs(ref).max())
        upto = len(toks) if dtype == "float32" else first_close_call(model_dir_f32, toks)
        assert set(got[name]) == set(range(len(toks))), f"{label}: {name} misses positions"
        for p in range(upto):
            row = got[name][p]
            assert np.isfinite(row).all(), f"{label}: {name} position {p}: logits are not finite"
            err = float(np.abs(row - ref[p]).max()) / scale
            worst, n = max(worst, err), n + 1
            assert err <= TOL[dtype], (f"{label}: first wrong place: request {name} position {p} of {len(toks)}: "
                                       f"error {err:.3e} of the largest logit, allowed {TOL[dtype]:.1e}")
    print(f"[korirax] {label}: {n} positions, worst {worst:.3e}")
    return worst


def requests(name: str, lengths, seed: int) -> Dict[str, List[int]]:
    rng = np.random.default_rng(seed)
    vocab = CONFIGS[name][0]["vocab"]
    return {f"r{i}": rng.integers(0, vocab, size=n).tolist() for i, n in enumerate(lengths)}
