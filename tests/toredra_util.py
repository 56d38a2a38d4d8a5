"""Helpers of the Toredra tests: small configurations of their own, a writer of random weights whose scale lets
every mechanism matter, and the comparison of the engine with the plain implementation (`plain_toredra`).  The
writer names every tensor itself, so a weight slot that the engine forgets or misnames shows as a loading error."""
from __future__ import annotations

import functools
from typing import Dict, List, Tuple

import numpy as np

import plain_toredra as P
from zidivik_util import PartHarness, bf16_round, load_part, write_model  # noqa: F401  (helpers that know no architecture)


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def parallel(heads, kv_heads, dim, vdim, scale, rotary, r_heads, r_dim, r_vdim):
    return {"type": "parallel", "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rotary},
                                          "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim}}}


def delta(heads, dim, rank):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}}


def layer(mixer, ff=None):
    return dict(mixer, mlp={"kind": "dense", "ff": ff} if ff else None)


# R1: a delta layer first; the looped stretch in the middle, three passes; values wider and narrower than keys; part of a
# head rotated, with wavelengths in all three bands of the stretching; as many kv heads as heads; a layer without
# feed-forward; logits scaled so that the cap bends the large ones without flattening them.
R1 = {"architecture": "Toredra", "vocab": 173, "width": 72, "norm": {"eps": 1e-5}, "logit_scale": 0.25, "logit_softcap": 9.0,
      "loop": {"start": 1, "stop": 3, "times": 3}, "layers": [
    layer(delta(3, 24, 12), 96),
    layer(parallel(6, 2, 16, 24, 0.3, rot(8, 100.0, (4.0, 1.0, 4.0, 64)), 2, 24, 40), None),
    layer(delta(2, 40, 7), 40),
    layer(parallel(4, 4, 32, 8, 0.25, rot(32, 10000.0), 3, 8, 16), 56),
]}
# R2: a width and head sizes that are no multiples of 8 (the plain kernels in bfloat16 too); no loop, no cap, no scale;
# five heads on one kv head; one recurrent head; a key size that is no multiple of 4.
R2 = {"architecture": "Toredra", "vocab": 97, "width": 70, "norm": {"eps": 1e-6}, "layers": [
    layer(parallel(5, 1, 12, 20, 0.4, rot(6, 50.0, (8.0, 1.0, 4.0, 32)), 1, 14, 10), 30),
    layer(delta(5, 14, 5), None),
    layer(parallel(2, 2, 10, 10, 0.5, rot(10, 1000.0), 2, 36, 12), 44),
    layer(delta(1, 18, 9), 62),
]}
# R3: heads of 128 (prompt portions on the tcgen05 attention kernel), a recurrence of 128 key channels, the whole model
# looped twice.
R3 = {"architecture": "Toredra", "vocab": 131, "width": 64, "norm": {"eps": 1e-6}, "logit_scale": 0.5, "logit_softcap": 30.0,
      "loop": {"start": 0, "stop": 2, "times": 2}, "layers": [
    layer(parallel(4, 2, 128, 128, 0.09, rot(64, 10000.0, (8.0, 1.0, 4.0, 128)), 2, 64, 128), 72),
    layer(delta(1, 128, 16), 48),
]}
CONFIGS = {"R1": (R1, 3), "R2": (R2, 8), "R3": (R3, 5)}


def tensors_of(cfg: dict, seed: int) -> Dict[str, np.ndarray]:
    """Random float32 tensors for ``cfg``, by name.  Matrices N(0, g / sqrt(in)) so that activations keep their size
    through the layers; norm weights around 1; biases, sinks and gate offsets of order 1; lower bounds inside (0, 1)."""
    rng = np.random.default_rng(seed)
    D, V = cfg["width"], cfg["vocab"]
    W: Dict[str, np.ndarray] = {}

    def mat(name, out, inn, gain=1.0):
        W[name] = (rng.standard_normal((out, inn)) * gain / np.sqrt(inn)).astype(np.float32)

    def vec(name, n, mean=0.0, std=1.0):
        W[name] = (mean + std * rng.standard_normal(n)).astype(np.float32)

    W["embed"] = rng.standard_normal((V, D)).astype(np.float32)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for n in ("norm1", "norm1b"):
            vec(p + n, D, 1.0, 0.1)
        mat(p + "rg1", D, D, 1.5)
        vec(p + "rg1.b", D, 0.5, 0.5)
        if L["type"] == "parallel":
            a, b = m["left"], m["right"]
            H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                mat(p + "mix.left." + n, rows, D, 2.0 if n != "v" else 1.0)
                vec(p + f"mix.left.{n}.b", rows, 0.0, 0.3)
            vec(p + "mix.left.sink", H, 0.5, 1.5)
            mat(p + "mix.left.o", D, H * dv)
            vec(p + "mix.left.out", D, 1.0, 0.2)
            H, d, dv = b["heads"], b["dim"], b["vdim"]
            mat(p + "mix.right.q", H * d, D, 1.5)
            mat(p + "mix.right.f", H * d, D, 2.0)
            vec(p + "mix.right.f.b", H * d, 1.0, 1.0)
            W[p + "mix.right.lower"] = rng.uniform(0.0, 0.9, H * d).astype(np.float32)
            mat(p + "mix.right.v", H * dv, D)
            vec(p + "mix.right.norm", dv, 1.0, 0.2)
            mat(p + "mix.right.o", D, H * dv)
            vec(p + "mix.right.out", D, 1.0, 0.2)
        else:
            H, d, r = m["heads"], m["dim"], m["decay_rank"]
            for n in ("r", "k", "v", "g"):
                mat(p + "mix." + n, H * d, D, 1.5)
            mat(p + "mix.a", H * d, D, 2.0)
            vec(p + "mix.a.b", H * d, 0.0, 1.0)
            mat(p + "mix.w1", r, D, 1.5)
            mat(p + "mix.w2", H * d, r, 3.0)
            vec(p + "mix.w0", H * d, -0.5, 1.5)
            vec(p + "mix.norm", H * d, 1.0, 0.2)
            mat(p + "mix.o", D, H * d)
        f = L.get("mlp")
        if f is not None:
            for n in ("norm2", "norm2b"):
                vec(p + n, D, 1.0, 0.1)
            mat(p + "rg2", D, D, 1.5)
            vec(p + "rg2.b", D, 0.5, 0.5)
            mat(p + "mlp.up", f["ff"], D, 1.5)
            mat(p + "mlp.down", D, f["ff"])
    vec("final.norm", D, 1.0, 0.1)
    return W


@functools.lru_cache(maxsize=None)
def _model(model_dir: str):
    return P.read_model(model_dir)


@functools.lru_cache(maxsize=None)
def plain_logits(model_dir: str, tokens: Tuple[int, ...]) -> np.ndarray:
    cfg, W = _model(model_dir)
    return P.forward(cfg, W, list(tokens))


# |engine - plain| as a fraction of the largest |plain logit| of the request: the most at any one position, and the most
# for the mean over a trace's positions.  Every sublayer's result is normed to unit size before it is added, so a small
# result's rounding enters the stream at full weight, through every run of a looped layer: in bfloat16 single positions
# reach a few hundredths while the mean stays near one hundredth.  A fault of the cache, a state or a mask moves the
# positions it touches by tenths and more, and the float32 comparison on the same traces allows 2e-5.
TOL = {"float32": 2e-5, "bfloat16": 8e-2}
TOL_MEAN = {"float32": 2e-5, "bfloat16": 1e-2}


def compare_with_plain(model_dir_f32: str, reqs: Dict[str, List[int]], got, dtype: str, label: str = "") -> float:
    """Every logits row of a trace against the plain implementation; names the first wrong (request, position)."""
    worst, errs = 0.0, []
    for name, toks in reqs.items():
        ref = plain_logits(model_dir_f32, tuple(toks))
        scale = float(np.abs(ref).max())
        assert set(got[name]) == set(range(len(toks))), f"{label}: {name} misses positions"
        for p in range(len(toks)):
            row = got[name][p]
            assert np.isfinite(row).all(), f"{label}: {name} position {p}: logits are not finite"
            err = float(np.abs(row - ref[p]).max()) / scale
            worst = max(worst, err)
            errs.append(err)
            assert err <= TOL[dtype], (f"{label}: first wrong place: request {name} position {p} of {len(toks)}: "
                                       f"error {err:.3e} of the largest logit, allowed {TOL[dtype]:.1e}")
    mean = float(np.mean(errs))
    print(f"[toredra] {label}: {len(errs)} positions, worst {worst:.3e}, mean {mean:.3e}")
    assert mean <= TOL_MEAN[dtype], f"{label}: mean error {mean:.3e} over {len(errs)} positions, allowed {TOL_MEAN[dtype]:.1e}"
    return worst


def steady_first_tokens(cfg: dict, W: Dict[str, np.ndarray], floor: float = 0.02) -> List[int]:
    """Tokens that may open a request in a comparison at reduced precision.  At a request's first token the delta rule's
    state is k v^T, its read-out (r . k) v, and the norm over the head keeps of r . k only the sign: where r . k is tiny
    beside |r| |k|, rounding decides the sign, in any implementation.  This lists the tokens for which every head of every
    run of a delta layer has |r . k| >= floor |r| |k| at position 0."""
    eps = float(cfg["norm"]["eps"])
    Wd = {n: a.astype(np.float64) for n, a in W.items()}
    good = []
    for tok in range(int(cfg["vocab"])):
        e = Wd["embed"][[tok]]
        x, ok = e.copy(), True
        for i, rep, first in P.layer_order(cfg):
            if first and rep > 0:
                x = x + e
            L = cfg["layers"][i]
            if L["type"] == "general_delta":
                m, p = L["mixer"], f"l{i}.mix."
                h = P.rms_norm(x, Wd[f"l{i}.norm1"], eps)
                r = P.linear(h, Wd[p + "r"]).reshape(m["heads"], m["dim"])
                k = P.linear(h, Wd[p + "k"]).reshape(m["heads"], m["dim"])
                ok = ok and bool((np.abs((r * k).sum(-1)) >= floor * np.linalg.norm(r, axis=-1) * np.linalg.norm(k, axis=-1)).all())
            x = P.layer_forward(x, Wd, cfg, i)
        if ok:
            good.append(tok)
    return good


@functools.lru_cache(maxsize=None)
def _steady_of(name: str) -> Tuple[int, ...]:
    import torch
    cfg, seed = CONFIGS[name]
    W = {n: torch.from_numpy(a).to(torch.bfloat16).to(torch.float64).numpy() for n, a in tensors_of(cfg, seed).items()}
    return tuple(steady_first_tokens(cfg, W))


def requests(name: str, lengths, seed: int) -> Dict[str, List[int]]:
    """Random requests r0, r1, ... for the configuration ``name``, each opened by a token of `steady_first_tokens`."""
    cfg = CONFIGS[name][0]
    rng = np.random.default_rng(seed)
    good = _steady_of(name)
    assert len(good) >= 8, f"{name}: only {len(good)} tokens can open a request"
    out = {}
    for i, n in enumerate(lengths):
        toks = rng.integers(0, cfg["vocab"], size=n).tolist()
        toks[0] = int(good[int(rng.integers(0, len(good)))])
        out[f"r{i}"] = toks
    return out
