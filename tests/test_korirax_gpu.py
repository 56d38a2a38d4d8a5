"""The Korirax decoder in the engine against its plain statement (`plain_korirax`): every mechanism alone, then whole
models under every way of cutting and batching the work, then generation through the scheduler (GPU)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import korirax_util as K
import plain_korirax as P
import replay_util as R

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")
PART_TOL = {"float32": 3e-5, "bfloat16": 4e-2}      # of the largest entry of the plain result
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RAMP = (8.0, 32, 4.0, 1.0)                          # a stretching whose ramp rises inside the pairs used below


@pytest.fixture(scope="module")
def kdirs(tmp_path_factory):
    return {name: K.write_model(cfg, K.tensors_of(cfg, seed), tmp_path_factory.mktemp("korirax_" + name)) for name, (cfg, seed) in K.CONFIGS.items()}


def _close(got, want, dtype, what, scale=None, tol=None):
    scale = float(np.abs(want).max()) if scale is None else scale
    assert np.isfinite(got).all(), f"{what}: not finite"
    err = float(np.abs(got - want).max()) / scale
    allowed = PART_TOL[dtype] if tol is None else tol
    assert err <= allowed, f"{what}: error {err:.3e} of the largest entry, allowed {allowed:.1e}"
    return err


def _torch_dtype(dtype):
    import torch
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]


def _exact(h):
    """Rows that both number formats hold exactly, so that the parts' inputs are the same."""
    import torch
    return torch.from_numpy(np.asarray(h, dtype=np.float32)).to(torch.bfloat16).to(torch.float64).numpy()


def _model_of(layers, width, dtype, eps=1e-6, seed=0, vocab=11, **top):
    from kestrel_llm_b200.config import resolve_architecture
    cfg = dict({"architecture": "Korirax", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}, **top)
    W = K.tensors_of(cfg, seed)
    arch = resolve_architecture("Korirax")
    model = arch.build(arch.config_class.from_dict(cfg), _torch_dtype(dtype), "cuda:0")
    return model, W, cfg


PLAIN_MIXER = {"attention": P.mix_attention, "latent_attention": P.mix_latent, "rglru": P.mix_rglru}


def _mixer_case(layer, dtype, page, n_tokens, cuts, seed=0, width=48, prepare=None, eps=1e-6):
    """One mixer alone; ``cuts`` are the portion sizes the tokens arrive in.  ``prepare(W, h)`` may shape weights and inputs
    and return other inputs whose plain result is handed back as well.  Returns (engine, plain, plain of the other inputs
    or the harness)."""
    rng = np.random.default_rng(seed)
    model, W, _ = _model_of([K.layer(layer, None)], width, dtype, eps=eps, seed=seed)
    mixer = model.blocks[0].mixer
    h = _exact(rng.standard_normal((n_tokens, width)))
    other = None
    if prepare is not None:
        other = prepare(W, h)
        h = _exact(h)
    assert K.load_part(mixer, W) == {k for k in W if k.startswith("l0.mix.")}
    Wr = K.bf16_round(W)
    plain = PLAIN_MIXER[layer["type"]]
    want = plain(h, Wr, "l0.mix.", layer["mixer"], eps)
    hs = K.PartHarness(mixer, dtype, max_tokens=((n_tokens + 63) // 64) * 64 + 64, page_size=page)
    got, at = [], 0
    for n in cuts:
        got.append(hs.step([(7, h[at:at + n])])[0])
        at += n
    assert at == n_tokens
    if other is not None:
        return np.concatenate(got), want, plain(_exact(other), Wr, "l0.mix.", layer["mixer"], eps)
    return np.concatenate(got), want, hs


# one entry per mechanism and shape of sizes
MIXERS = [
    ("attention 4/2 x 16/24, temperature every 16, 10 rows to 40", K.attn(4, 2, 16, 24, 0.3, 40, 10, (0.7, 16))),
    ("attention 3/1 x 40/8, no temperature, 7 rows to 25", K.attn(3, 1, 40, 8, 0.2, 25, 7)),
    ("attention 2/2 x 64/64, 16 rows to 300", K.attn(2, 2, 64, 64, 0.15, 300, 16, (0.2, 30))),
    ("attention 5/1 x 12/20 (no multiples of 8), 2 rows to 3", K.attn(5, 1, 12, 20, 0.3, 3, 2, (1.0, 1))),
    ("attention 2/1 x 128/128", K.attn(2, 1, 128, 128, 0.09, 60, 12, (0.5, 64))),
    ("latent 3 x 16+8/24, ranks 40/48, stretched", K.latent(3, 16, 8, 24, 40, 48, 0.22, 8, 100.0, RAMP)),
    ("latent 5 x 10+6/14, ranks 26/36, four of six turned", K.latent(5, 10, 6, 14, 26, 36, 0.25, 4, 50.0)),
    ("latent 2 x 64+64/128, ranks 48/192", K.latent(2, 64, 64, 128, 48, 192, 0.1, 64, 100000.0, (16.0, 128, 16.0, 2.0))),
    ("latent 4 x 32+16/32, ranks 64/80", K.latent(4, 32, 16, 32, 64, 80, 0.15, 16, 1000.0, (4.0, 96, 8.0, 1.0))),
    ("latent 1 x 8+2/8, ranks 8/8", K.latent(1, 8, 2, 8, 8, 8, 0.4, 2, 10.0)),
    ("latent 2 x 16+16/16, ranks 24/272 (a cache row beyond the tensor-core kernels' sizes)", K.latent(2, 16, 16, 16, 24, 272, 0.2, 16, 100.0, RAMP)),
    ("recurrence 64 in 4 blocks, 4 taps", K.rglru(64, 4, 4)),
    ("recurrence 42 in 3 blocks, 2 taps", K.rglru(42, 3, 2)),
    ("recurrence 256 in 1 block, 1 tap", K.rglru(256, 1, 1)),
    ("recurrence 144 in 2 blocks, 9 taps", K.rglru(144, 2, 9)),
]


# ---- each mechanism alone --------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("label,layer", MIXERS, ids=[m[0] for m in MIXERS])
def test_mixer_alone_whole_and_cut(dtype, label, layer):
    n = 90
    whole, want, _ = _mixer_case(layer, dtype, 16, n, [n], seed=len(label))
    _close(whole, want, dtype, f"{label}, whole")
    cut, want, _ = _mixer_case(layer, dtype, 8, n, [33, 2, 17, 2, 7, 8, 9, 6] + [1] * 6, seed=len(label))
    _close(cut, want, dtype, f"{label}, portions and single tokens")
    single, want, _ = _mixer_case(layer, dtype, 16, 21, [1] * 21, seed=len(label))
    _close(single, want, dtype, f"{label}, token by token from the first")


def _spike(kind, i, j):
    """Weights and inputs so that token i asks for token j above all others (beside itself).  Attention: keys are made from
    the first half of a token's input and values from the second, queries by the keys' own weights, and token i gets the first
    half of token j's input - so q_i . k_j is a squared length while the two tokens' values differ.  Recurrence: the decays
    are held near 1 and token j's input is made large.  Returns inputs in which another token stands in j's place."""
    def prepare(W, h):
        p, half = "l0.mix.", h.shape[1] // 2
        fresh = np.random.default_rng(5).standard_normal(h.shape[1])
        if kind == "rglru":
            other = h.copy()
            W[p + "lam"][:] = -9.0            # softplus 1e-4: what token j writes is still there hundreds of tokens later
            h[j] *= 40.0
            return other
        m = SPIKE_LAYERS[kind]["mixer"]
        if kind == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            W[p + "k"][:, half:] = 0.0
            W[p + "v"][:, :half] = 0.0
            for n in range(H):
                g = n // (H // G)
                W[p + "q"][n * d:(n + 1) * d] = W[p + "k"][g * d:(g + 1) * d]
                W[p + "q.b"][n * d:(n + 1) * d] = W[p + "k.b"][g * d:(g + 1) * d]
            W[p + "q.norm"][:] = W[p + "k.norm"]
        else:
            H, d, dr, R = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
            assert m["q_rank"] == R
            W[p + "dkv"][:R // 2, half:] = 0.0           # the latent's first half from the input's first half: what keys are made of
            W[p + "dkv"][R // 2:R, :half] = 0.0          # its second half from the input's second half: what values are made of
            W[p + "uk"][:, R // 2:] = 0.0
            W[p + "uv"][:, :R // 2] = 0.0
            W[p + "dq"][:] = W[p + "dkv"][:R]
            W[p + "dq.norm"][:] = W[p + "dkv.norm"]
            for n in range(H):
                W[p + "uq"][n * (d + dr):n * (d + dr) + d] = W[p + "uk"][n * d:(n + 1) * d]
                W[p + "uq"][n * (d + dr) + d:(n + 1) * (d + dr)] *= 0.1
        h[i, :half] = h[j, :half]
        other = h.copy()
        other[j] = fresh
        return other
    return prepare


SPIKE_LAYERS = {"attention": K.attn(4, 2, 16, 24, 0.5, 40, 10, (0.7, 16)),
                "latent": K.latent(2, 64, 8, 24, 128, 128, 0.3, 8, 100.0, RAMP),
                "rglru": K.rglru(64, 4, 3)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("where", ["far", "page_end", "page_start", "first_token", "previous_token"])
@pytest.mark.parametrize("kind", ["attention", "latent", "rglru"])
def test_mixer_reads_what_lies_far_back(kind, dtype, decode, where):
    """One token stands out and one later token asks for it: hundreds of tokens back, on either side of a page border, at
    the request's first position, and right before.  The plain result with an ordinary token in its place differs widely:
    the engine must match the true one, in a prompt's portions and decoded token by token."""
    page, n, i = 16, 300, 297
    j = {"far": 3, "page_end": 255, "page_start": 256, "first_token": 0, "previous_token": i - 1}[where]
    cuts = [290] + [1] * 10 if decode else [140, 160]
    got, want, other = _mixer_case(SPIKE_LAYERS[kind], dtype, page, n, cuts, prepare=_spike(kind, i, j), width=160)
    scale, told = float(np.abs(want).max()), float(np.abs(want[i] - other[i]).max())
    assert told > 0.1 * np.abs(want[i]).max(), f"{kind}, {where}: the case does not tell whether token {j} was read"
    err = float(np.abs(got - want).max()) / scale
    assert np.isfinite(got).all() and err <= {"float32": 1e-4, "bfloat16": 4e-2}[dtype], f"{kind}, {where}: error {err:.3e}"
    assert np.abs(got[i] - want[i]).max() < 0.2 * told


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
def test_distance_terms_by_bucket_and_beyond_the_last(dtype, decode):
    """The table of distance terms decides alone: queries and keys are switched off (scale 0), so a token's weights are
    the softmax of its row of terms.  One bucket at a time gets a large term; the plain result then reads the tokens
    of that bucket's distances and nothing else - at the buckets' edges, at the distance where the last bucket begins,
    and far beyond it."""
    rows, far, n = 10, 40, 120
    layer = K.attn(2, 1, 16, 16, 0.0, far, rows)
    for bucket in (0, 4, 5, 7, rows - 1):
        def prepare(W, h, b=bucket):
            W["l0.mix.rel"][:] = 0.0
            W["l0.mix.rel"][b, :] = 9.0
            return h.copy()
        got, want, _ = _mixer_case(layer, dtype, 16, n, [100] + [1] * 20 if decode else [50, 70], prepare=prepare, seed=bucket)
        _close(got, want, dtype, f"bucket {bucket}")
    # the buckets themselves: every distance up to the last row's and the next ones, against the formula's own words
    half = rows // 2
    edges = [n_ for n_ in range(1, 200) if P.distance_bucket(n_, rows, far) != P.distance_bucket(n_ - 1, rows, far)]
    assert edges[:half] == list(range(1, half + 1)) and P.distance_bucket(far, rows, far) == rows - 1 == P.distance_bucket(10 * far, rows, far)


@pytest.mark.parametrize("cuts", [[700], [300, 400], [520, 2, 178], [900, 400]])
def test_distance_terms_in_portions_of_head_size_128(cuts):
    """bfloat16 portions of head size 128 take the tcgen05 kernel: key tiles near the diagonal look every score's term up,
    tiles that lie wholly beyond the table's last distance take one term; later portions cut their keys into slices."""
    layer = K.attn(4, 2, 128, 128, 0.09, 60, 12, (0.5, 64))

    def prepare(W, h):
        W["l0.mix.rel"][:] *= 3.0
        W["l0.mix.rel"][-1, :] = np.array([4.0, -4.0, 2.0, 0.0])
        return h.copy()
    got, want, _ = _mixer_case(layer, "bfloat16", 16, sum(cuts), cuts, prepare=prepare)
    _close(got, want, "bfloat16", f"portions {cuts}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_query_temperature_steps_with_the_position(dtype):
    """A temperature that changes every 7 positions with a large coefficient: switched off in the plain statement, the
    result differs from the first change on and not before."""
    layer = K.attn(3, 3, 16, 16, 0.4, 30, 8, (2.0, 7))
    got, want, _ = _mixer_case(layer, dtype, 16, 40, [23, 2] + [1] * 15)
    _close(got, want, dtype, "with temperature")
    rng = np.random.default_rng(0)
    W = K.bf16_round(K.tensors_of({"architecture": "Korirax", "width": 48, "vocab": 11, "norm": {"eps": 1e-6}, "layers": [K.layer(layer, None)]}, 0))
    h = _exact(rng.standard_normal((40, 48)))
    cold = P.mix_attention(h, W, "l0.mix.", dict(layer["mixer"], q_temp=None), 1e-6)
    assert np.abs(cold[:6] - want[:6]).max() < 1e-9 and np.abs(cold[6:] - want[6:]).max() > 0.02 * np.abs(want).max()


@pytest.mark.parametrize("dtype", DTYPES)
def test_rotated_key_part_and_its_scale(dtype):
    """The rotated part alone decides: the unrotated expansion of the keys is zero, so every score is the shared key part's.
    Frequencies in all bands of the ramp, positions up to 400; the factor on cos and sin enters squared."""
    layer = K.latent(2, 8, 16, 8, 24, 16, 0.6, 16, 200.0, (16.0, 64, 8.0, 1.0))

    def prepare(W, h):
        W["l0.mix.uk"][:] = 0.0
        return h.copy()
    got, want, _ = _mixer_case(layer, dtype, 16, 400, [250, 130] + [1] * 20, prepare=prepare)
    _close(got, want, dtype, "rotated part alone", tol={"float32": 1e-4, "bfloat16": 4e-2}[dtype])
    f, mult = P.yarn_frequencies(16, 200.0, dict(zip(("factor", "original", "fast", "slow"), (16.0, 64, 8.0, 1.0))))
    f0 = 200.0 ** (-2.0 * np.arange(8) / 16)
    assert f[0] == f0[0] and np.isclose(f[-1], f0[-1] / 16.0) and 0 < ((f < f0 * 0.99) & (f > f0 / 15.9)).sum() and mult > 1.2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("layer", [K.rglru(64, 4, 4), K.rglru(42, 3, 2), K.rglru(264, 2, 3)], ids=["64", "42", "264"])
def test_recurrence_in_chunks_and_token_by_token(dtype, layer):
    """Portions of 128 tokens and more run the recurrence in chunks (a chunk's action on the state, then the chunks in
    order); shorter ones and single tokens run it token by token.  Both against the plain statement over 700 tokens with
    slow decays, the state handed from one form to the other and back; and the two forms against each other."""
    from kestrel_llm_b200.csrc import ops

    def prepare(W, h):
        W["l0.mix.lam"][:] = np.linspace(-7.0, 1.0, W["l0.mix.lam"].shape[0])
        return h.copy()
    cuts = [3, 297, 1, 1, 130, 268]
    got, want, _ = _mixer_case(layer, dtype, 16, 700, cuts, prepare=prepare)
    _close(got, want, dtype, "chunks and single tokens")
    ops.rglru_chunked = False
    try:
        seq, _, _ = _mixer_case(layer, dtype, 16, 700, cuts, prepare=prepare)
    finally:
        ops.rglru_chunked = True
    _close(got, seq, dtype, "chunked against sequential", scale=float(np.abs(want).max()), tol={"float32": 1e-5, "bfloat16": 2e-2}[dtype])


def test_recurrence_in_chunks_of_unequal_requests():
    """Three requests in one step, 400, 129 and 2 tokens: the grid is sized by the longest, the others' chunks end early."""
    layer = K.rglru(64, 4, 4)
    rng = np.random.default_rng(3)
    model, W, _ = _model_of([K.layer(layer, None)], 48, "float32", seed=3)
    mixer = model.blocks[0].mixer
    K.load_part(mixer, W)
    Wr = K.bf16_round(W)
    hs_ = [_exact(rng.standard_normal((n, 48))) for n in (430, 140, 5)]
    want = [P.mix_rglru(h, Wr, "l0.mix.", layer["mixer"], 1e-6) for h in hs_]
    hs = K.PartHarness(mixer, "float32", max_tokens=640, page_size=16, slots=3)
    o1 = hs.step([(1, hs_[0][:400]), (2, hs_[1][:129]), (3, hs_[2][:2])])
    o2 = hs.step([(3, hs_[2][2:5]), (1, hs_[0][400:430]), (2, hs_[1][129:140])])
    for r, (a, b) in enumerate(((o1[0], o2[1]), (o1[1], o2[2]), (o1[2], o2[0]))):
        _close(np.concatenate([a, b]), want[r], "float32", f"request {r}")


def _ffn_case(mlp, dtype, n, seed=0, width=48, prepare=None):
    import torch
    model, W, _ = _model_of([K.layer(K.rglru(8, 1, 1), mlp)], width, dtype, seed=seed)
    ffn = model.blocks[0].ffn
    if prepare is not None:
        prepare(W)
    K.load_part(ffn, W)
    Wr = K.bf16_round(W)
    rng = np.random.default_rng(seed)
    h = _exact(rng.standard_normal((n, width)))
    x = torch.from_numpy(h.astype(np.float32)).to("cuda:0").to(_torch_dtype(dtype))
    out = ffn.forward(x, None)
    outs = out if isinstance(out, tuple) else (out,)
    got = sum(o.reduce(torch.float32).cpu().numpy().astype(np.float64) for o in outs)
    return got, h, Wr, ffn


MOES = [("12 experts in 3 groups, 2 kept, 3 chosen, shared", K.moe(12, 3, 40, 3, 2, 1.7, 56)),
        ("6 groups of one, 3 kept, 2 chosen", K.moe(6, 2, 22, 6, 3, 1.0, 0)),
        ("16 experts in 4 groups, all kept, 1 chosen", K.moe(16, 1, 48, 4, 4, 2.0, 32)),
        ("one group of 40, 8 chosen", K.moe(40, 8, 16, 1, 1, 0.5, 0)),
        ("8 experts in 4 groups, 1 kept, 2 chosen (a whole group)", K.moe(8, 2, 24, 4, 1, 3.0, 8))]


@pytest.mark.parametrize("n", [5, 700])
@pytest.mark.parametrize("label,mlp", MOES, ids=[m[0] for m in MOES])
def test_routed_experts_alone(label, mlp, n):
    """float32, so that the engine's router and the plain one make the same calls: groups, the correction that chooses but
    does not weigh, normalised weights, the shared expert; few tokens and enough for the grouped products' many tiles."""
    got, h, Wr, _ = _ffn_case(mlp, "float32", n, seed=len(label))
    want = P.ff_moe(h, Wr, "l0.mlp.", mlp)
    _close(got, want, "float32", label)


@pytest.mark.parametrize("n", [9, 1500])
def test_routed_experts_in_bfloat16_where_no_call_is_close(n):
    """bfloat16 on the tensor cores (few pairs: mma.sync; many: tcgen05).  Corrections far apart decide the groups and the
    experts whatever the rounding; the scores still weigh."""
    mlp = K.moe(12, 3, 40, 3, 2, 1.7, 56)

    def prepare(W):
        W["l0.mlp.correction"][:] = np.array([5, 1, 3, 0, 2, 9, 4, 8, 6, 7, 11, 10], dtype=np.float32) * 3.0
    got, h, Wr, _ = _ffn_case(mlp, "bfloat16", n, prepare=prepare)
    want = P.ff_moe(h, Wr, "l0.mlp.", mlp)
    ids, _ = P.route(h, Wr, "l0.mlp.", mlp["router"])
    assert set(np.unique(ids)) == {5, 10, 11}          # the groups of experts 4 .. 7 and 8 .. 11 stay; the three largest of them
    _close(got, want, "bfloat16", "experts in bfloat16")


def test_correction_chooses_but_does_not_weigh():
    """The correction moves the choice; the weights are the scores without it.  A closed group's experts are never chosen,
    although their choice scores are the largest negative ones' betters."""
    mlp = K.moe(8, 2, 24, 4, 1, 3.0, 0)

    def prepare(W):
        W["l0.mlp.correction"][:] = np.array([-6, -7, -9, -9.5, -8, -8.2, -20, -30], dtype=np.float32)
    got, h, Wr, _ = _ffn_case(mlp, "float32", 64, prepare=prepare)
    ids, ws = P.route(h, Wr, "l0.mlp.", mlp["router"])
    assert set(np.unique(ids)) == {0, 1} and np.allclose(ws.sum(-1), 3.0)       # negative choice scores, group 0 the best
    _close(got, P.ff_moe(h, Wr, "l0.mlp.", mlp), "float32", "negative choice scores")


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_adds_both_sublayers_then_the_token_input(dtype):
    """One layer as the model runs it: a norm that mixer and feed-forward both read, their sum, then the token input made
    from the new stream and this layer's part of the table row - a part that is not the first."""
    import torch
    from kestrel_llm_b200.engine import Entry
    from kestrel_llm_b200.engine.batch import StepBatch
    layers = [K.layer(K.rglru(16, 2, 2), K.dense(40)), K.layer(K.attn(2, 1, 16, 8, 0.3, 20, 6), K.moe(6, 2, 16, 3, 2, 1.5, 24))]
    model, W, cfg = _model_of(layers, 48, dtype, vocab=37, token_side={"dim": 10}, embedding={"scale": 4.0})
    for s in model.weight_slots():
        with torch.no_grad():
            s.dest.copy_(torch.from_numpy(W[s.name]).to(torch.bfloat16).to(s.dest.dtype))
    Wr = K.bf16_round(W)
    toks = np.random.default_rng(2).integers(0, 37, size=40).tolist()
    want = []
    P.forward(toks, Wr, cfg, want)
    from kestrel_llm_b200.cache import CacheManager
    cache = CacheManager(model.cache_specs(), model.dtype, "cuda:0", 16, 8, 2, 1 << 12)
    cache.admit(0)
    cache.reserve(0, len(toks))
    cache.clear_admitted()
    batch = StepBatch([Entry(0, toks, [])], cache, "cuda:0")
    x, pending = model.forward_embed(batch)
    assert np.abs(x.cpu().numpy() - Wr["embed"][toks] * 4.0).max() == 0
    for i in range(2):
        x, pending = model.forward_calls(x, pending, batch, cache, i, i + 1)
        assert pending is None
        if dtype == "float32" or i == 0:         # bfloat16 may route a token otherwise than the plain statement
            _close(x.cpu().numpy(), want[i], dtype, f"stream after layer {i}")


# ---- requests beside each other, memory used again --------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", [0, 5, 8, 10, 13])
def test_requests_beside_each_other_and_memory_used_again(dtype, which):
    """Three requests of unequal length in one step, portions beside single tokens, against each alone; then two are given
    back and a new request runs on their pages and slot."""
    label, layer = MIXERS[which]
    rng = np.random.default_rng(which)
    model, W, _ = _model_of([K.layer(layer, None)], 48, dtype, seed=which)
    mixer = model.blocks[0].mixer
    K.load_part(mixer, W)
    Wr = K.bf16_round(W)
    plain = PLAIN_MIXER[layer["type"]]
    ha, hb, hc, hd = (_exact(rng.standard_normal((n, 48))) for n in (70, 33, 5, 64))
    wa, wb, wc, wd = (plain(h, Wr, "l0.mix.", layer["mixer"], 1e-6) for h in (ha, hb, hc, hd))
    hs = K.PartHarness(mixer, dtype, max_tokens=192, page_size=8, slots=3)
    o1 = hs.step([(1, ha[:40]), (2, hb[:2]), (3, hc[:1])])
    o2 = hs.step([(2, hb[2:30]), (1, ha[40:41]), (3, hc[1:5])])
    o3 = hs.step([(1, ha[41:70]), (2, hb[30:33])])
    _close(np.concatenate([o1[0], o2[1], o3[0]]), wa, dtype, f"{label}, request a beside others")
    _close(np.concatenate([o1[1], o2[0], o3[1]]), wb, dtype, f"{label}, request b beside others")
    _close(np.concatenate([o1[2], o2[2]]), wc, dtype, f"{label}, request c beside others")
    hs.cache.release(2)
    hs.cache.release(3)
    _close(np.concatenate([hs.step([(4, hd[:50])])[0]] + [hs.step([(4, hd[t:t + 1])])[0] for t in range(50, 64)]), wd, dtype,
           f"{label}, a new request on pages and a slot that were given back")


# ---- whole models ----------------------------------------------------------------------------------

LENGTHS = {"K1": (1, 2, 37, 70, 129, 64), "K2": (3, 50, 97, 130, 17), "K3": (2, 150, 33), "K4": (1, 2, 45, 140, 64)}
LENGTHS_MIXED = {"K1": (5, 33, 70, 129, 47, 90, 16, 65, 31), "K2": (3, 50, 97, 130, 64, 81, 17, 49), "K4": (7, 120, 33, 260, 64, 81, 2, 49)}


def _run(kdirs, name, dtype, family, lengths=None, page_size=16, batch_max=4, graphs=False, **kw):
    reqs = K.requests(name, lengths or LENGTHS[name], seed=11 + len(name))
    steps, max_tokens = family(reqs, **kw)
    engine = R.make_engine(kdirs[name][dtype], dtype, max_tokens, page_size=page_size, batch_max=batch_max, graphs=graphs)
    got = R.run_trace(engine, steps)
    assert engine.cache.live_requests() == 0
    engine.cache.check()
    K.compare_with_plain(kdirs[name]["float32"], reqs, got, dtype, f"{name}/{dtype}/{family.__name__}")
    return got


def test_residual_stream_after_every_layer_run(kdirs):
    """float32: the stream after each run of a layer against the plain implementation's - layers that run several times,
    each pass's own vector in front of it - so that a fault names its place."""
    from kestrel_llm_b200.engine import Entry
    from kestrel_llm_b200.engine.batch import StepBatch
    for name in K.CONFIGS:
        cfg = K.CONFIGS[name][0]
        toks = K.requests(name, (75,), seed=4)["r0"]
        _, W = K._model(kdirs[name]["float32"])
        want = []
        P.forward(toks, W, cfg, want)
        engine = R.make_engine(kdirs[name]["float32"], "float32", 128)
        engine.cache.admit(0)
        engine.cache.reserve(0, len(toks))
        engine.cache.clear_admitted()
        batch = StepBatch([Entry(0, toks, [])], engine.cache, "cuda:0")
        model = engine.model
        assert len(model.order) == len(want) == len(P.layer_runs(cfg))
        x, pending = model.forward_embed(batch)
        for i in range(len(model.order)):
            x, pending = model.forward_calls(x, pending, batch, engine.cache, i, i + 1)
            err = np.abs(x.cpu().numpy() - want[i]).max() / np.abs(want[i]).max()
            assert pending is None and err < 2e-5, f"{name}: layer run {i} (layer {model.order[i].block}): error {err:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["K1", "K2", "K3", "K4"])
@pytest.mark.parametrize("family", [R.trace_whole, R.trace_tail_decode, R.trace_portions])
def test_model_alone_whole_decoded_and_in_portions(kdirs, name, dtype, family):
    _run(kdirs, name, dtype, family)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", [("K1", 16), ("K2", 16), ("K4", 8), ("K4", 64)])
def test_model_mixed_batches_pages_and_slots_used_again(kdirs, name, dtype, page):
    """Up to four live requests, portions beside single tokens; eight or nine requests through four slots and a pool that
    holds four of them, so that pages and slots are used again."""
    _run(kdirs, name, dtype, R.trace_mixed, lengths=LENGTHS_MIXED[name], page_size=page, live_max=4)


def test_model_with_heads_of_128_mixed_batches(kdirs):
    _run(kdirs, "K3", "float32", R.trace_mixed, lengths=(150, 33, 129, 90, 300), live_max=4, sizes=(70, 2, 140, 3, 66, 2, 210, 5))
    _run(kdirs, "K3", "bfloat16", R.trace_mixed, lengths=(150, 33, 129, 90, 300), live_max=4, sizes=(70, 2, 140, 3, 66, 2, 210, 5))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["K1", "K4"])
def test_long_decoding_through_captured_steps(kdirs, name, dtype):
    """Five prompt tokens, then 215 tokens one by one through captured decode steps: past every bucket of distances, over
    several changes of the query temperature, through pages that fill one by one."""
    _run(kdirs, name, dtype, R.trace_tail_decode, lengths=(220,), graphs=True, tail=215)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_prompt_then_decoding(kdirs, dtype):
    """600 tokens: a prompt in three portions, then 40 tokens one by one; distances far beyond the table's last row."""
    _run(kdirs, "K4", dtype, R.trace_portions, lengths=(600,), sizes=(250, 200, 110) + (1,) * 40)


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_scheduler(kdirs, dtype):
    """`LLM.generate`: six requests through three slots, prompts in portions of at most 24 tokens."""
    from kestrel_llm_b200 import LLM, SamplingParams
    name = "K4"
    cfg = K.CONFIGS[name][0]
    prompts = list(K.requests(name, (1, 40, 70, 9, 33, 55), seed=4).values())
    llm = LLM(kdirs[name][dtype], dtype=dtype, page_size=16, batch_max=3, max_tokens=512, prefill_batch=24, max_step_tokens=64)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    _, W = K._model(kdirs[name]["float32"])
    for prompt, o in zip(prompts, outs):
        toks = list(prompt)
        assert len(o.token_ids) == 8
        for got in o.token_ids:
            logits = P.forward(toks, W, cfg)[-1]
            want = int(np.argmax(logits))
            if got != want:          # a tie within rounding is not a fault; anything else is
                gap = float(logits[want] - logits[got])
                assert gap <= (2e-5 if dtype == "float32" else 4e-2) * float(np.abs(logits).max()), f"{dtype}: token {got} instead of {want}"
            toks.append(got)


# ---- the programs a user runs ------------------------------------------------------------------------

@pytest.mark.parametrize("dtype,graphs", [("float32", 1), ("bfloat16", 1), ("bfloat16", 0)])
def test_trace_replay_program(kdirs, dtype, graphs, tmp_path):
    """bin/trace_run in a process of its own on a mixed trace: four slots for seven requests, decode steps replayed from
    captured graphs (the default) and launched kernel by kernel."""
    name = "K2" if dtype == "float32" else "K4"
    reqs = K.requests(name, (5, 33, 70, 47, 90, 16, 65), seed=21)
    steps, max_tokens = R.trace_mixed(reqs, live_max=4, seed=5)
    lines = "".join(json.dumps(dict(step=i, **s)) + "\n" for i, s in enumerate(steps))
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", kdirs[name][dtype], "--dtype", dtype, "--out", str(out),
                        "--max-tokens", str(max_tokens), "--cuda-graphs", str(graphs)], input=lines, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    V = K.CONFIGS[name][0]["vocab"]
    pos = {n: 0 for n in reqs}
    got = {n: {} for n in reqs}
    for i, s in enumerate(steps):
        arr = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)
        r = 0
        for e in s["entries"]:
            for w in e["want"]:
                got[e["id"]][pos[e["id"]] + w] = arr[r]
                r += 1
            pos[e["id"]] += len(e["tokens"])
        assert r == arr.shape[0]
    K.compare_with_plain(kdirs[name]["float32"], reqs, got, dtype, f"trace_run/{dtype}")


def test_command_line_writes_random_weights_and_generates(tmp_path):
    """bin/kestrel: `--random-weights` writes a Korirax folder from a config.json with the design's own keys, and the
    streaming harness prints the plain implementation's greedy tokens."""
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(K.K4))
    model_dir = tmp_path / "written"
    prompt = R.random_requests(K.K4["vocab"], (23,), seed=2)["r0"]
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kestrel"), "--model", str(model_dir), "--config", str(cfg_file),
                        "--random-weights", "5", "--dtype", "float32", "--stream-test", "--stream-n", "8", "--prompt-ids",
                        ",".join(str(t) for t in prompt), "--ignore-eos", "--max-tokens", "256", "--batch-max", "2"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    line = [l for l in p.stdout.splitlines() if l.startswith("[STREAM] TOKIDS:")]
    assert len(line) == 1
    with open(model_dir / "config.json") as f:
        pcfg = json.load(f)
    W = P.read_checkpoint(str(model_dir / "model.safetensors"))
    assert W["l0.mix.rel"].shape == (12, 4) and W["loop.step"].shape == (2, K.K4["width"]) and "l2.mlp.up" not in W
    toks, want = list(prompt), []
    for _ in range(8):
        want.append(int(np.argmax(P.forward(toks, W, pcfg)[-1])))
        toks.append(want[-1])
    assert [int(t) for t in line[0].split(":")[1].split()] == want
