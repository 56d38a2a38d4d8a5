"""The Toredra decoder in the engine against its plain statement (`plain_toredra`): every mechanism alone, then whole
models under every way of cutting and batching the work, then generation through the scheduler (GPU)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_toredra as P
import replay_util as R
import toredra_util as T

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")
PART_TOL = {"float32": 3e-5, "bfloat16": 4e-2}      # of the largest entry of the plain result
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SC = (8.0, 1.0, 4.0, 64)                            # a stretching whose three bands all occur below


@pytest.fixture(scope="module")
def tdirs(tmp_path_factory):
    return {name: T.write_model(cfg, T.tensors_of(cfg, seed), tmp_path_factory.mktemp("toredra_" + name)) for name, (cfg, seed) in T.CONFIGS.items()}


def _close(got, want, dtype, what, scale=None):
    scale = float(np.abs(want).max()) if scale is None else scale
    assert np.isfinite(got).all(), f"{what}: not finite"
    err = float(np.abs(got - want).max()) / scale
    assert err <= PART_TOL[dtype], f"{what}: error {err:.3e} of the largest entry, allowed {PART_TOL[dtype]:.1e}"
    return err


def _torch_dtype(dtype):
    import torch
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]


def _rows(rng, n, width):
    """Input rows that both number formats hold exactly, so that the parts' inputs are the same."""
    import torch
    x = rng.standard_normal((n, width)).astype(np.float32)
    return torch.from_numpy(x).to(torch.bfloat16).to(torch.float64).numpy()


def _exact(h):
    import torch
    return torch.from_numpy(np.asarray(h, dtype=np.float32)).to(torch.bfloat16).to(torch.float64).numpy()


def _left(H, G, d, dv, scale=0.4, dims=None, base=100.0, scaling=None):
    """A parallel layer whose attention side is what the case is about (a small recurrence beside it)."""
    return T.parallel(H, G, d, dv, scale, T.rot(d if dims is None else dims, base, scaling), 1, 8, 8)


def _right(H, d, dv):
    return T.parallel(1, 1, 8, 8, 0.3, T.rot(8, 100.0), H, d, dv)


def _model_of(layers, width, dtype, eps=1e-6, seed=0, vocab=11, **top):
    from kestrel_llm_b200.config import ToredraConfig, resolve_architecture
    cfg = dict({"architecture": "Toredra", "width": width, "vocab": vocab, "norm": {"eps": eps},
                "layers": [dict(L, mlp=L.get("mlp")) for L in layers]}, **top)
    W = T.tensors_of(cfg, seed)
    model = resolve_architecture("Toredra").build(ToredraConfig.from_dict(cfg), _torch_dtype(dtype), "cuda:0")
    return model, W, cfg


def _pick(mixer, side):
    return mixer if side is None else getattr(mixer, side)


def _plain_mixer(layer, side, Wr, h, eps):
    m, p = layer["mixer"], "l0.mix."
    if layer["type"] == "general_delta":
        return P.general_delta_mixer(h, Wr, p, m, eps)
    if side == "left":
        return P.rotary_sink_mixer(h, Wr, p + "left.", m["left"], eps)
    if side == "right":
        return P.forget_gate_mixer(h, Wr, p + "right.", m["right"], eps)
    return P.parallel_mixer(h, Wr, p, m, eps)


def _mixer_case(layer, side, dtype, page, n_tokens, cuts, seed=0, width=48, prepare=None, eps=1e-6):
    """One mixer alone (``side``: "left" / "right" of a parallel mixer, None for the whole); ``cuts`` are the portion
    sizes the tokens arrive in.  ``prepare(W, h)`` may shape weights and inputs and return other inputs whose plain
    result is handed back as well.  Returns (engine, plain, plain of the other inputs or the harness)."""
    rng = np.random.default_rng(seed)
    model, W, _ = _model_of([layer], width, dtype, eps=eps, seed=seed)
    whole = model.blocks[0].mixer
    h = _rows(rng, n_tokens, width)
    other = None
    if prepare is not None:
        other = prepare(W, h)
        h = _exact(h)
    assert T.load_part(whole, W) == {k for k in W if k.startswith("l0.mix.")}
    Wr = T.bf16_round(W)
    want = _plain_mixer(layer, side, Wr, h, eps)
    hs = T.PartHarness(_pick(whole, side), dtype, max_tokens=((n_tokens + 63) // 64) * 64 + 64, page_size=page)
    got, at = [], 0
    for n in cuts:
        got.append(hs.step([(7, h[at:at + n])])[0])
        at += n
    assert at == n_tokens
    if other is not None:
        return np.concatenate(got), want, _plain_mixer(layer, side, Wr, _exact(other), eps)
    return np.concatenate(got), want, hs


# one entry per mechanism and shape of sizes: (label, layer, side)
MIXERS = [
    ("attention 4/2 x 16/24, half of a head rotated, stretched", _left(4, 2, 16, 24, dims=8, scaling=SC), "left"),
    ("attention 3/1 x 40/8, whole head rotated", _left(3, 1, 40, 8, base=10000.0), "left"),
    ("attention 2/2 x 64/64", _left(2, 2, 64, 64, dims=32, scaling=SC), "left"),
    ("attention 5/1 x 12/20 (no multiples of 8)", _left(5, 1, 12, 20, dims=6, base=50.0, scaling=SC), "left"),
    ("attention 4/2 x 80/48, two rotated dimensions", _left(4, 2, 80, 48, dims=2), "left"),
    ("forget gate 2 x 24/40", _right(2, 24, 40), "right"),
    ("forget gate 3 x 8/16", _right(3, 8, 16), "right"),
    ("forget gate 1 x 14/10", _right(1, 14, 10), "right"),
    ("forget gate 2 x 72/136", _right(2, 72, 136), "right"),
    ("forget gate 1 x 256/24", _right(1, 256, 24), "right"),
    ("delta 3 x 24, rank 12", T.delta(3, 24, 12), None),
    ("delta 5 x 14, rank 5", T.delta(5, 14, 5), None),
    ("delta 1 x 128, rank 16", T.delta(1, 128, 16), None),
    ("delta 2 x 200, rank 1", T.delta(2, 200, 1), None),
    ("both sides, 6/2 x 16/24 beside 2 x 24/40", T.parallel(6, 2, 16, 24, 0.3, T.rot(8, 100.0, SC), 2, 24, 40), None),
    ("both sides, 2/2 x 10/10 beside 2 x 36/12", T.parallel(2, 2, 10, 10, 0.5, T.rot(10, 1000.0), 2, 36, 12), None),
]


# ---- each mechanism alone --------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("label,layer,side", MIXERS, ids=[m[0] for m in MIXERS])
def test_mixer_alone_whole_and_cut(dtype, label, layer, side):
    n = 90
    whole, want, _ = _mixer_case(layer, side, dtype, 16, n, [n], seed=len(label))
    _close(whole, want, dtype, f"{label}, whole")
    cut, want, _ = _mixer_case(layer, side, dtype, 8, n, [33, 2, 17, 2, 7, 8, 9, 6] + [1] * 6, seed=len(label))
    _close(cut, want, dtype, f"{label}, portions and single tokens")
    single, want, _ = _mixer_case(layer, side, dtype, 16, 21, [1] * 21, seed=len(label))
    _close(single, want, dtype, f"{label}, token by token from the first")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", [0, 5, 10, 14])
def test_first_tokens_and_shortest_requests(dtype, which):
    """Requests of one and two tokens; the first positions, where the memory is empty; portions that end on and around
    the eight tokens the scan stages at a time."""
    label, layer, side = MIXERS[which]
    for n, cuts in ((1, [1]), (2, [2]), (2, [1, 1]), (9, [7, 1, 1]), (17, [8, 8, 1]), (40, [3, 2, 30] + [1] * 5)):
        got, want, _ = _mixer_case(layer, side, dtype, 16, n, cuts, seed=n)
        _close(got, want, dtype, f"{label}, {n} tokens as {cuts[:3]}")


def _spike(kind, i, j):
    """Weights and inputs such that what token j wrote decides the output at token i, however far back j lies: the
    other inputs (returned) are the same with token j's value taken away."""
    def prepare(W, h):
        p = "l0.mix."
        h *= 0.05
        h[:, :3] = 0.0
        h[i, 0] = 6.0                          # i asks along channel 0
        h[j, 1] = 6.0                          # j's value stands out along channel 1
        if kind == "left":
            h[j, 2] = 6.0                      # j answers as a key, along channel 2: i's own key does not answer
            p += "left."
            W[p + "q"][:, 0] = W[p + "k"][:, 2] = 1.0       # every dimension of q_i and k_j is 6: the dimensions that
            W[p + "v"][:, 1] = 1.0                           # are not rotated alone lift the score far above the rest
            W[p + "k"][:, 0] = W[p + "v"][:, 0] = W[p + "v"][:, 2] = 0.0
            for n in ("q.b", "k.b", "v.b"):
                W[p + n] *= 0.05
        elif kind == "right":
            h[j, 2] = 6.0                      # j's forget gate closes: the state becomes j's value
            p += "right."
            W[p + "q"][:, 0] = 1.0
            W[p + "v"][:, 1] = 1.0
            W[p + "v"][:, :1] = 0.0
            W[p + "f"][:] = 0.0
            W[p + "f"][:, 2] = -5.0
            W[p + "f.b"][:] = 9.0              # every other token keeps 0.9999 of the state
            W[p + "lower"][:] = 0.0
        else:
            h[j, 2] = 6.0
            W[p + "r"][:, 0] = W[p + "k"][:, 2] = 1.0
            W[p + "v"][:, 1] = 1.0
            W[p + "k"][:, 0] = W[p + "v"][:, 0] = W[p + "v"][:, 2] = 0.0
            W[p + "w2"][:] = 0.0
            W[p + "w0"][:] = -12.0             # no decay to speak of
            W[p + "a"][:] = 0.0
            W[p + "a.b"][:] = -12.0            # and nothing removed
        other = h.copy()
        other[j, 1] = 0.0
        return other
    return prepare


SPIKE_LAYERS = {"left": (_left(2, 1, 16, 8, scale=0.5, dims=8, scaling=SC), "left"), "right": (_right(2, 16, 24), "right"),
                "delta": (T.delta(2, 16, 4), None)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("where", ["far", "page_end", "page_start", "first_token", "previous_token"])
@pytest.mark.parametrize("kind", ["left", "right", "delta"])
def test_mixer_reads_what_lies_far_back(kind, dtype, decode, where):
    """One token's value stands out and one later token asks for it: hundreds of tokens back, on either side of a page
    border, at the request's first position, and right before.  The plain result without that value differs widely
    from the true one: the engine must match the true one, in a prompt's portions and decoded token by token."""
    page, n, i = 16, 300, 297
    j = {"far": 3, "page_end": 255, "page_start": 256, "first_token": 0, "previous_token": i - 1}[where]
    cuts = [290] + [1] * 10 if decode else [140, 160]
    layer, side = SPIKE_LAYERS[kind]
    got, want, other = _mixer_case(layer, side, dtype, page, n, cuts, prepare=_spike(kind, i, j))
    scale = float(np.abs(want).max())
    assert np.abs(want[i] - other[i]).max() > 0.25 * scale, f"{kind}, {where}: the case does not tell whether token {j} was read"
    # float32: up to 300 multiplications by a decay that is itself rounded to float32, on entries hundreds of times the
    # ordinary ones, before a norm: rounding alone reaches 1e-4 of the largest entry here
    err = float(np.abs(got - want).max()) / scale
    assert np.isfinite(got).all() and err <= {"float32": 3e-4, "bfloat16": 4e-2}[dtype], f"{kind}, {where}: error {err:.3e}"
    assert np.abs(got[i] - want[i]).max() < 0.1 * np.abs(want[i] - other[i]).max()


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_softmax_extra_term_is_each_heads_own(dtype):
    """A head whose learned term is huge puts out nothing, one whose term is tiny is an ordinary softmax, the others lie
    between - and all differ from the result with every term at exp(0)."""
    layer = _left(4, 2, 16, 24, dims=8)
    seen = {}

    def prepare(W, h):
        W["l0.mix.left.sink"][:] = [30.0, -30.0, 2.0, -1.0]
        W["l0.mix.left.o"][:] = 0.0
        for c in range(4 * 24):
            W["l0.mix.left.o"][c % 48, c] = 1.0               # the heads' outputs come out side by side, two heads a column
        seen["W"] = W
        return h.copy()
    got, want, _ = _mixer_case(layer, "left", dtype, 16, 70, [50, 2] + [1] * 18, prepare=prepare)
    _close(got, want, dtype, "learned terms 30, -30, 2, -1")
    Wz = T.bf16_round(seen["W"])
    Wz["l0.mix.left.sink"] = np.zeros(4)
    zero = P.rotary_sink_mixer(_exact(_rows(np.random.default_rng(0), 70, 48)), Wz, "l0.mix.left.", layer["mixer"]["left"], 1e-6)
    assert np.abs(zero - want).max() > 0.2 * np.abs(want).max()


@pytest.mark.parametrize("dtype", DTYPES)
def test_rotation_pairs_bands_and_positions(dtype):
    """Positions into the thousands (a request that starts with a long portion), a rotation over part of the head with
    all three bands of stretching: the plain result with unstretched frequencies, and the one with the pairs (j, j + half),
    differ widely from the true one."""
    import torch
    from kestrel_llm_b200.csrc import ops  # noqa: F401
    layer = _left(2, 1, 32, 16, scale=0.3, dims=24, base=200.0, scaling=(8.0, 1.0, 4.0, 64))
    n = 2100
    got, want, _ = _mixer_case(layer, "left", dtype, 32, n, [2048, 40, 2] + [1] * 10, seed=3, width=32)
    tail = slice(2040, n)
    # a float32 angle at position p is off by up to p 2^-24 radians, 1.3e-4 here, and the scores move by as much
    err = float(np.abs(got[tail] - want[tail]).max()) / float(np.abs(want).max())
    assert err <= {"float32": 2e-4, "bfloat16": 4e-2}[dtype], f"rotation at positions beyond 2,040: error {err:.3e}"
    _, W, _ = _model_of([layer], 32, "float32", seed=3)
    Wr = T.bf16_round(W)
    h = _rows(np.random.default_rng(3), n, 32)
    m = dict(layer["mixer"]["left"])
    m["rot"] = T.rot(24, 200.0)
    plain_freq = P.rotary_sink_mixer(h, Wr, "l0.mix.left.", m, 1e-6)
    assert np.abs(plain_freq[tail] - want[tail]).max() > 0.1 * np.abs(want).max()


def test_block_gates_norms_and_feed_forward():
    """One layer's block alone, float32: norm, mixer, gate by the sublayer's own input, second norm, add; then the same
    around the feed-forward (square of relu).  Also a block without feed-forward."""
    import torch
    from kestrel_llm_b200.engine.batch import Entry, StepBatch
    from kestrel_llm_b200.cache import CacheManager
    for layer in (T.layer(T.delta(2, 12, 3), 40), T.layer(T.delta(2, 12, 3), None), T.layer(T.parallel(2, 1, 8, 12, 0.4, T.rot(4, 30.0), 1, 6, 10), 52)):
        model, W, cfg = _model_of([layer], 36, "float32", eps=1e-5, seed=4)
        block = model.blocks[0]
        T.load_part(block, W)
        Wr = T.bf16_round(W)
        x = _rows(np.random.default_rng(1), 23, 36) * 3.0
        want = P.layer_forward(x.copy(), Wr, cfg, 0)
        cache = CacheManager([block.mixer.cache_spec()], torch.float32, "cuda:0", 16, 8, 2, 1 << 12)
        cache.admit(1)
        cache.reserve(1, 23)
        cache.clear_admitted()
        batch = StepBatch([Entry(1, [0] * 23, [])], cache, "cuda:0")
        res, pending = block.forward(torch.from_numpy(x.astype(np.float32)).to("cuda:0"), None, batch, cache.layer(0, True))
        assert pending is None
        _close(res.cpu().numpy().astype(np.float64), want, "float32", f"block, {layer['type']}, mlp {layer['mlp']}")
        gated_off = dict(Wr)
        gated_off["l0.rg1.b"] = Wr["l0.rg1.b"] + 50.0          # a gate that is always open is another layer
        gated_off["l0.rg1"] = Wr["l0.rg1"] * 0.0
        assert np.abs(P.layer_forward(x.copy(), gated_off, cfg, 0) - want).max() > 0.05 * np.abs(want).max()


@pytest.mark.parametrize("act", ["relu2", "tanh", "silu"])
@pytest.mark.parametrize("T_,N,K", [(129, 264, 72), (700, 1024, 256), (2048, 520, 136), (64, 256, 64), (300, 100, 70)])
def test_activation_in_the_products_epilogue(act, T_, N, K):
    """bfloat16: act(x w^T) with the activation as the epilogue of the tcgen05 product on CTA pairs (many tokens, sizes
    the product takes uncut) against the product's slices summed and activated by the elementwise kernel - the same
    bits - and against numpy; few tokens and sizes that are no multiples of 8 take the second way by themselves."""
    import torch
    from kestrel_llm_b200.csrc import ops
    rng = np.random.default_rng(T_ + N)
    x = torch.from_numpy(rng.standard_normal((T_, K)).astype(np.float32)).to(torch.bfloat16)
    w = torch.from_numpy((rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)).to(torch.bfloat16)
    xd, wd = x.to("cuda:0"), w.to("cuda:0")
    fused = ops.linear_act(xd, wd, act)
    ops.raise_on_kernel_error()
    ops.linear_act_fused = False
    try:
        slices = ops.linear_act(xd, wd, act)
    finally:
        ops.linear_act_fused = True
    z = x.to(torch.float64).numpy() @ w.to(torch.float64).numpy().T
    want = {"relu2": np.maximum(z, 0.0) ** 2, "tanh": np.tanh(z), "silu": z / (1.0 + np.exp(-z))}[act]
    assert fused.dtype == torch.bfloat16 and tuple(fused.shape) == (T_, N)
    _close(fused.float().cpu().numpy(), want, "bfloat16", f"{act} in the epilogue", scale=max(1.0, float(np.abs(want).max())))
    if ops.library().kestrel_gemm_tc_plan(xd.data_ptr(), wd.data_ptr(), T_, N, K, xd.stride(0), wd.stride(0)) == 1:
        assert torch.equal(fused, slices)
    else:
        _close(slices.float().cpu().numpy(), want, "bfloat16", f"{act} on slices", scale=max(1.0, float(np.abs(want).max())))


@pytest.mark.parametrize("d", [520, 1024, 2056])
def test_wide_rows_have_the_same_bits_in_steps_of_few_and_of_many_tokens(d):
    """The kernels that take a row a block pick their thread count by the step's size, and the gates of the delta rule a
    form of their own for few tokens; a row's bits must not move with either.  600 rows at once against the first 3 alone,
    at widths that fold 2 and 4 virtual threads into one, products of 1, 3 and 9 slices; also against numpy."""
    import torch
    from kestrel_llm_b200.csrc import ops
    rng = np.random.default_rng(d)
    T_, few = 600, 3

    def product(S, width, rows=T_):
        return torch.from_numpy(rng.standard_normal((S, rows, width)).astype(np.float32)).to("cuda:0")

    def vec(width, mean=0.0):
        return torch.from_numpy((mean + rng.standard_normal(width)).astype(np.float32)).to("cuda:0")
    y, g, a, b = product(9, d), product(3, d), product(1, d), product(9, d)
    w, wn, wa, wb, yb, gb = vec(d, 1.0), vec(d, 1.0), vec(d, 1.0), vec(d, 1.0), vec(d), vec(d)
    x0 = torch.from_numpy(rng.standard_normal((T_, d)).astype(np.float32)).to("cuda:0")
    outs = {}
    for rows in (T_, few):
        x = x0[:rows].clone()
        nxt = torch.empty((rows, d), dtype=torch.float32, device="cuda:0")
        ops.add_gated_normed(x, ops.Partials(y[:, :rows].contiguous(), yb), ops.Partials(g[:, :rows].contiguous(), gb), w, 1e-6, wn, 1e-5, nxt)
        c = ops.combine_normed(ops.Partials(a[:, :rows].contiguous()), wa, ops.Partials(b[:, :rows].contiguous()), wb, 1e-6, 0.5)
        ops.raise_on_kernel_error()
        outs[rows] = (x, nxt, c.data[0])
    for many, alone in zip(outs[T_], outs[few]):
        assert torch.equal(many[:few], alone)
    ys = y.double().sum(0).cpu().numpy() + yb.double().cpu().numpy()
    gs = g.double().sum(0).cpu().numpy() + gb.double().cpu().numpy()
    z = ys / (1.0 + np.exp(-gs))
    want = x0.double().cpu().numpy() + z / np.sqrt((z ** 2).mean(-1, keepdims=True) + 1e-6) * w.double().cpu().numpy()
    _close(outs[T_][0].cpu().numpy(), want, "float32", "gated, normed, added")
    _close(outs[T_][1].cpu().numpy(), want / np.sqrt((want ** 2).mean(-1, keepdims=True) + 1e-5) * wn.double().cpu().numpy(), "float32", "the next norm")
    # the delta rule's gates: a head size for each form of the few-token kernel
    for H, dh in ((3, 40), (2, 128), (2, 200)):
        n = H * dh
        fused, wz = product(3, 4 * n + 8), product(2, n)
        ab, wb0 = vec(n), vec(n)
        many = ops.removal_gates(ops.Partials(fused), 0, n, 2 * n, 3 * n, ab, ops.Partials(wz), wb0, 0.6, H, dh)
        alone = ops.removal_gates(ops.Partials(fused[:, :few].contiguous()), 0, n, 2 * n, 3 * n, ab, ops.Partials(wz[:, :few].contiguous()), wb0, 0.6, H, dh)
        ops.raise_on_kernel_error()
        for m, o in zip(many, alone):
            assert torch.equal(m[:few], o)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("scale,cap", [(1.0, 0.0), (2.5, 0.0), (1.0, 7.0), (0.3, 4.0)])
def test_output_head_scales_then_caps(dtype, scale, cap):
    import torch
    model, W, cfg = _model_of([T.layer(T.delta(1, 8, 2), None)], 40, dtype, seed=2, vocab=77, logit_scale=scale, **({"logit_softcap": cap} if cap else {}))
    for part in (model.embedding, model.final_norm):
        T.load_part(part, W)
    Wr = T.bf16_round(W)
    x = _rows(np.random.default_rng(5), 9, 40) * 2.0
    n = _exact(P.rms_norm(x, Wr["final.norm"], 1e-6)) if dtype == "bfloat16" else P.rms_norm(x, Wr["final.norm"], 1e-6)
    want = (n @ Wr["embed"].T) * scale
    want = cap * np.tanh(want / cap) if cap else want
    normed = model.final_norm.add_forward(torch.from_numpy(x.astype(np.float32)).to("cuda:0"), None, _torch_dtype(dtype))
    got = model.lm_head.forward(normed).cpu().numpy().astype(np.float64)
    _close(got, want, dtype, f"logits, scale {scale}, cap {cap}", scale=max(1.0, float(np.abs(want).max())))
    if cap:
        assert np.abs(got).max() < cap and np.abs(want).max() > 0.6 * cap         # the cap bends these logits


@pytest.mark.parametrize("sizes,page,n,cuts", [((8, 2, 128, 128), 16, 700, [300, 400]), ((2, 2, 128, 128), 32, 200, [200]),
                                               ((4, 1, 128, 128), 16, 300, [129, 2, 140] + [1] * 29), ((6, 6, 128, 128), 8, 520, [260, 100, 160]),
                                               ((16, 1, 128, 128), 64, 90, [50, 40])])
def test_portions_of_head_size_128_on_tcgen05(sizes, page, n, cuts):
    """bfloat16: prompt portions of head size 128 take the tcgen05 kernel, with each head's learned term closing its rows:
    against the plain statement and against the same mixer kept on the mma.sync kernel."""
    from kestrel_llm_b200.csrc import ops
    from kestrel_llm_b200.parts import GatedWindowAttention
    layer = _left(*sizes, scale=0.09, dims=64, base=10000.0, scaling=(8.0, 1.0, 4.0, 128))
    calls = {"n": 0}
    real = ops.attention_tc

    def counted(*a, **kw):
        calls["n"] += 1
        return real(*a, **kw)
    ops.attention_tc = counted
    try:
        fast, want, _ = _mixer_case(layer, "left", "bfloat16", page, n, cuts, seed=5, width=64)
    finally:
        ops.attention_tc = real
    ops.raise_on_kernel_error()
    assert calls["n"] == sum(1 for c in cuts if c * (sizes[0] // sizes[1]) > GatedWindowAttention.TC_MIN_ROWS)
    _close(fast, want, "bfloat16", "attention on tcgen05")
    GatedWindowAttention.tcgen05 = False
    try:
        slow, _, _ = _mixer_case(layer, "left", "bfloat16", page, n, cuts, seed=5, width=64)
    finally:
        GatedWindowAttention.tcgen05 = True
    assert np.abs(fast - slow).max() <= 2e-2 * np.abs(want).max()


@pytest.mark.parametrize("sizes,page,n,cuts,slice_len", [((8, 2, 128, 128), 16, 700, [300, 400], 128), ((4, 4, 128, 128), 32, 530, [530], 128),
                                                         ((2, 1, 128, 128), 16, 900, [70, 500, 330], 256), ((4, 2, 128, 128), 16, 1500, [1500], 512)])
def test_long_prompts_cut_their_keys_into_slices(sizes, page, n, cuts, slice_len):
    """bfloat16: without a window the key range of few tiles far into a request is cut into slices on the tcgen05 kernel and
    merged, each head's learned term entering once, in the merge (here forced for every portion): against the plain statement
    and against the same portions in one slice."""
    from kestrel_llm_b200.csrc import ops
    from kestrel_llm_b200.parts import GatedWindowAttention
    layer = _left(*sizes, scale=0.09, dims=64, base=10000.0, scaling=(8.0, 1.0, 4.0, 128))
    seen = []
    real, real_len, real_fill = ops.attention_tc, GatedWindowAttention.TC_SLICE, GatedWindowAttention.TC_SLICE_FILL

    def noted(*a, **kw):
        seen.append(kw.get("slices", 1))
        return real(*a, **kw)
    ops.attention_tc, GatedWindowAttention.TC_SLICE, GatedWindowAttention.TC_SLICE_FILL = noted, slice_len, 1 << 20
    try:
        cut, want, _ = _mixer_case(layer, "left", "bfloat16", page, n, cuts, seed=7, width=64)
        ops.raise_on_kernel_error()
        GatedWindowAttention.TC_SLICE = 1 << 20
        whole, _, _ = _mixer_case(layer, "left", "bfloat16", page, n, cuts, seed=7, width=64)
    finally:
        ops.attention_tc, GatedWindowAttention.TC_SLICE, GatedWindowAttention.TC_SLICE_FILL = real, real_len, real_fill
    ops.raise_on_kernel_error()
    assert max(seen[:len(cuts)]) == -(-n // slice_len) and max(seen[len(cuts):]) == 1
    _close(cut, want, "bfloat16", "attention in slices of keys")
    assert np.abs(cut - whole).max() <= 1e-2 * np.abs(want).max()


@pytest.mark.parametrize("sizes,n", [((4, 2, 64, 64), 420), ((8, 2, 32, 48), 500), ((3, 3, 128, 128), 200), ((24, 1, 32, 32), 300), ((6, 3, 96, 64), 700)])
def test_single_token_steps_share_their_keys_out_over_ctas(sizes, n):
    """bfloat16: a step of single tokens cuts its keys into shares, a CTA each, merged by a second kernel that also adds
    each head's learned term once - against the plain statement, against the same steps with one CTA a request and key
    head, and against the mixer on the plain kernels."""
    from kestrel_llm_b200.csrc import ops
    from kestrel_llm_b200.parts import GatedWindowAttention
    layer = _left(*sizes, scale=0.3, dims=16, scaling=SC)
    cuts = [n - 12, 2] + [1] * 10
    shared, want, _ = _mixer_case(layer, "left", "bfloat16", 16, n, cuts, seed=9, width=64)
    _close(shared, want, "bfloat16", "keys over several CTAs")
    ops.attention_window_set_splits(False)
    try:
        one, _, _ = _mixer_case(layer, "left", "bfloat16", 16, n, cuts, seed=9, width=64)
    finally:
        ops.attention_window_set_splits(True)
    assert np.abs(shared - one).max() <= 2e-2 * np.abs(want).max()
    GatedWindowAttention.force_plain = True
    try:
        slow, _, _ = _mixer_case(layer, "left", "bfloat16", 16, n, cuts, seed=9, width=64)
    finally:
        GatedWindowAttention.force_plain = False
    assert np.abs(shared - slow).max() <= 2e-2 * np.abs(want).max()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", [14, 10, 8, 12])
def test_requests_beside_each_other_and_memory_used_again(dtype, which):
    """Two requests of unequal portions in one batch against each request alone; a third request then runs on the pages
    AND the state slot the first two gave back: what they left there must not reach it."""
    label, layer, side = MIXERS[which]
    rng = np.random.default_rng(3)
    model, W, _ = _model_of([layer], 48, dtype, seed=2)
    T.load_part(model.blocks[0].mixer, W)
    mixer = _pick(model.blocks[0].mixer, side)
    Wr = T.bf16_round(W)
    ha, hb, hc = _rows(rng, 60, 48), _rows(rng, 37, 48), _rows(rng, 64, 48)
    wa, wb, wc = (_plain_mixer(layer, side, Wr, h, 1e-6) for h in (ha, hb, hc))
    hs = T.PartHarness(mixer, dtype, max_tokens=128, page_size=16, slots=2)
    got_a, got_b, at_a, at_b = [], [], 0, 0
    for ka, kb in [(7, 2), (2, 13), (30, 2), (2, 5), (3, 1), (1, 1), (15, 13)]:
        out = hs.step([(2, ha[at_a:at_a + ka]), (3, hb[at_b:at_b + kb])])
        got_a.append(out[0])
        got_b.append(out[1])
        at_a, at_b = at_a + ka, at_b + kb
    assert (at_a, at_b) == (60, 37)
    _close(np.concatenate(got_a), wa, dtype, f"{label}, request a in portions beside b")
    _close(np.concatenate(got_b), wb, dtype, f"{label}, request b in portions beside a")
    hs.cache.release(2)
    hs.cache.release(3)
    _close(np.concatenate([hs.step([(4, hc[:50])])[0]] + [hs.step([(4, hc[t:t + 1])])[0] for t in range(50, 64)]), wc, dtype,
           f"{label}, a new request on pages and a slot that were given back")


# ---- whole models ----------------------------------------------------------------------------------

LENGTHS = {"R1": (1, 2, 37, 70, 129, 64), "R2": (3, 50, 97, 130, 17), "R3": (2, 150, 33)}
LENGTHS_MIXED = {"R1": (5, 33, 70, 129, 47, 90, 16, 65, 31), "R2": (3, 50, 97, 130, 64, 81, 17, 49)}


def _run(tdirs, name, dtype, family, lengths=None, page_size=16, batch_max=4, graphs=False, **kw):
    cfg = T.CONFIGS[name][0]
    reqs = T.requests(name, lengths or LENGTHS[name], seed=11 + len(name))
    steps, max_tokens = family(reqs, **kw)
    engine = R.make_engine(tdirs[name][dtype], dtype, max_tokens, page_size=page_size, batch_max=batch_max, graphs=graphs)
    got = R.run_trace(engine, steps)
    assert engine.cache.live_requests() == 0
    engine.cache.check()
    worst = T.compare_with_plain(tdirs[name]["float32"], reqs, got, dtype, f"{name}/{dtype}/{family.__name__}")
    print(f"[toredra] {name} {dtype} {family.__name__}: worst {worst:.3e}")
    return got


def test_residual_stream_after_every_layer_run(tdirs):
    """float32: the stream after each run of a layer against the plain implementation's - layers that run several
    times, the embedded tokens fed in again in front of every further pass - so that a fault names its place."""
    import torch
    from kestrel_llm_b200.engine import Entry
    from kestrel_llm_b200.engine.batch import StepBatch
    for name in ("R1", "R2", "R3"):
        cfg = T.CONFIGS[name][0]
        toks = T.requests(name, (75,), seed=4)["r0"]
        pcfg, W = P.read_model(tdirs[name]["float32"])
        want = []
        P.forward(pcfg, W, toks, want)
        engine = R.make_engine(tdirs[name]["float32"], "float32", 128)
        engine.cache.admit(0)
        engine.cache.reserve(0, len(toks))
        engine.cache.clear_admitted()
        batch = StepBatch([Entry(0, toks, [])], engine.cache, "cuda:0")
        model = engine.model
        assert len(model.order) == len(want) == len(P.layer_order(cfg))
        x, pending = model.forward_embed(batch)
        for i in range(len(model.order)):
            x, pending = model.forward_calls(x, pending, batch, engine.cache, i, i + 1)
            now = x.clone() if pending is None else x + pending.reduce(torch.float32)
            err = np.abs(now.cpu().numpy() - want[i]).max() / np.abs(want[i]).max()
            assert err < 2e-5, f"{name}: layer run {i} (layer {model.order[i].block}): error {err:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["R1", "R2", "R3"])
@pytest.mark.parametrize("family", [R.trace_whole, R.trace_tail_decode, R.trace_portions])
def test_model_alone_whole_decoded_and_in_portions(tdirs, name, dtype, family):
    _run(tdirs, name, dtype, family)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", [("R1", 16), ("R2", 16), ("R1", 8), ("R2", 64)])
def test_model_mixed_batches_pages_and_slots_used_again(tdirs, name, dtype, page):
    """Up to four live requests, portions beside single tokens; nine requests through four slots and a pool that holds
    four of them, so that pages and slots are used again."""
    _run(tdirs, name, dtype, R.trace_mixed, lengths=LENGTHS_MIXED[name], page_size=page, live_max=4)


def test_model_with_heads_of_128_mixed_batches(tdirs):
    """bfloat16: portions of several requests in one step through the tcgen05 kernel beside single tokens on the mma.sync
    kernel, pages and slots used again."""
    _run(tdirs, "R3", "bfloat16", R.trace_mixed, lengths=(150, 33, 400, 129, 260, 90, 16), live_max=4, sizes=(70, 2, 140, 3, 66, 2, 210, 5))
    _run(tdirs, "R3", "bfloat16", R.trace_portions, lengths=(300, 131), sizes=(70, 2, 130, 2, 50, 3, 170, 2, 31, 4))
    _run(tdirs, "R3", "float32", R.trace_mixed, lengths=(150, 33, 129, 90), live_max=4, sizes=(70, 2, 140, 3, 66, 2, 210, 5))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["R1", "R2"])
def test_long_decoding_through_captured_steps(tdirs, name, dtype):
    """Five prompt tokens, then 215 tokens one by one through captured decode steps."""
    _run(tdirs, name, dtype, R.trace_tail_decode, lengths=(220,), graphs=True, tail=215)


@pytest.mark.parametrize("name", ["R1", "R2"])
def test_cuttings_agree_in_float32(tdirs, name):
    """The float32 logits of a position do not depend on how the work was cut or batched: every sum's order is fixed per
    output element."""
    a = _run(tdirs, name, "float32", R.trace_whole, lengths=LENGTHS_MIXED[name])
    b = _run(tdirs, name, "float32", R.trace_mixed, lengths=LENGTHS_MIXED[name], live_max=4)
    c = _run(tdirs, name, "float32", R.trace_portions, lengths=LENGTHS_MIXED[name])
    for r in a:
        for p in a[r]:
            assert np.array_equal(a[r][p], b[r][p]) and np.array_equal(a[r][p], c[r][p]), f"{name}: request {r} position {p}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_scheduler(tdirs, dtype):
    """`LLM.generate`: six requests through three slots, prompts in portions of at most 24 tokens."""
    from kestrel_llm_b200 import LLM, SamplingParams
    name = "R1"
    cfg = T.CONFIGS[name][0]
    prompts = list(T.requests(name, (1, 40, 70, 9, 33, 55), seed=4).values())
    llm = LLM(tdirs[name][dtype], dtype=dtype, page_size=16, batch_max=3, max_tokens=512, prefill_batch=24, max_step_tokens=64)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    pcfg, W = P.read_model(tdirs[name]["float32"])
    for prompt, o in zip(prompts, outs):
        toks = list(prompt)
        assert len(o.token_ids) == 8
        for got in o.token_ids:
            logits = P.forward(pcfg, W, toks)[-1]
            want = int(np.argmax(logits))
            if got != want:          # a tie within rounding is not a fault; anything else is
                gap = float(logits[want] - logits[got])
                assert gap <= (2e-5 if dtype == "float32" else 4e-2) * float(np.abs(logits).max()), f"{dtype}: token {got} instead of {want}"
            toks.append(got)


# ---- the programs a user runs ------------------------------------------------------------------------

@pytest.mark.parametrize("dtype,graphs", [("float32", 1), ("bfloat16", 1), ("bfloat16", 0)])
def test_trace_replay_program(tdirs, dtype, graphs, tmp_path):
    """bin/trace_run in a process of its own on a mixed trace: four slots for seven requests, decode steps replayed from
    captured graphs (the default) and launched kernel by kernel."""
    name = "R2"
    reqs = T.requests(name, (5, 33, 70, 47, 90, 16, 65), seed=21)
    steps, max_tokens = R.trace_mixed(reqs, live_max=4, seed=5)
    lines = "".join(json.dumps(dict(step=i, **s)) + "\n" for i, s in enumerate(steps))
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", tdirs[name][dtype], "--dtype", dtype, "--out", str(out),
                        "--max-tokens", str(max_tokens), "--cuda-graphs", str(graphs)], input=lines, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    V = T.CONFIGS[name][0]["vocab"]
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
    T.compare_with_plain(tdirs[name]["float32"], reqs, got, dtype, f"trace_run/{dtype}")


def test_command_line_writes_random_weights_and_generates(tmp_path):
    """bin/kestrel: `--random-weights` writes a Toredra folder from a config.json with the design's own keys, and the
    streaming harness prints the plain implementation's greedy tokens."""
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(T.R1))
    model_dir = tmp_path / "written"
    prompt = R.random_requests(T.R1["vocab"], (23,), seed=2)["r0"]
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kestrel"), "--model", str(model_dir), "--config", str(cfg_file),
                        "--random-weights", "5", "--dtype", "float32", "--stream-test", "--stream-n", "8", "--prompt-ids",
                        ",".join(str(t) for t in prompt), "--ignore-eos", "--max-tokens", "256", "--batch-max", "2"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    line = [l for l in p.stdout.splitlines() if l.startswith("[STREAM] TOKIDS:")]
    assert len(line) == 1
    pcfg, W = P.read_model(str(model_dir))
    assert ((W["l1.mix.right.lower"] >= 0) & (W["l1.mix.right.lower"] < 1)).all() and "l1.norm2" not in W and "l0.norm2" in W
    assert W["l0.mix.w1"].shape == (12, T.R1["width"])
    toks, want = list(prompt), []
    for _ in range(8):
        want.append(int(np.argmax(P.forward(pcfg, W, toks)[-1])))
        toks.append(want[-1])
    assert [int(t) for t in line[0].split(":")[1].split()] == want
