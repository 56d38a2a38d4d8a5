"""Toredra without a GPU: its configuration class, the registry, the weight slots against the tensors a checkpoint
holds, the order of layer runs and what they ask of the cache, the stretched rotary frequencies, and the plain
implementation against itself (prefixes, passes, the extra term of the softmax, the recurrences in closed form)."""
import json
import math
import os

import numpy as np
import pytest

import plain_toredra as P
import toredra_util as T


def test_config_round_trip_and_registry(tmp_path):
    from kestrel_llm_b200.config import ConfigError, ToredraConfig, load_config
    for name, (raw, _) in T.CONFIGS.items():
        d = tmp_path / name
        os.makedirs(d)
        with open(d / "config.json", "w") as f:
            json.dump(raw, f)
        cfg = load_config(str(d))
        assert isinstance(cfg, ToredraConfig) and cfg.num_hidden_layers == len(raw["layers"])
        assert ToredraConfig.from_dict(cfg.to_json_dict()) == cfg
    c = ToredraConfig.from_dict(T.R1)
    left = c.layers[1].mixer.left
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.rot.dims, left.rot.scaling) == (6, 2, 16, 24, 8, (4.0, 1.0, 4.0, 64.0))
    assert c.layers[3].mixer.left.rot.scaling is None and c.layers[1].mlp is None and c.layers[0].mixer.decay_rank == 12
    assert (c.loop.start, c.loop.stop, c.loop.times, c.logit_scale, c.logit_softcap) == (1, 3, 3, 0.25, 9.0)
    c2 = ToredraConfig.from_dict(T.R2)
    assert c2.loop is None and c2.logit_scale == 1.0 and c2.logit_softcap == 0.0
    for breaker in (lambda r: r["layers"][1]["mixer"]["left"].update(kv_heads=4),         # 6 heads on 4 kv heads
                    lambda r: r["layers"][1]["mixer"].pop("right"),
                    lambda r: r["layers"][1]["mixer"]["left"]["rot"].update(dims=18),      # more than the head
                    lambda r: r["layers"][1]["mixer"]["left"]["rot"].update(dims=7),
                    lambda r: r["layers"][0]["mlp"].update(kind="moe"),
                    lambda r: r["layers"][0].update(type="delta"),
                    lambda r: r["loop"].update(stop=5),
                    lambda r: r.update(logit_softcap=-1.0),
                    lambda r: r.pop("norm")):
        bad = json.loads(json.dumps(T.R1))
        breaker(bad)
        with pytest.raises(ConfigError):
            ToredraConfig.from_dict(bad)


def test_the_rank_of_the_decay_comes_from_the_checkpoint():
    from kestrel_llm_b200.config import ConfigError, ToredraConfig
    raw = json.loads(json.dumps(T.R1))
    for L in raw["layers"]:
        L["mixer"].pop("decay_rank", None)
    c = ToredraConfig.from_dict(raw)
    assert c.layers[0].mixer.decay_rank == 0
    shapes = {n: a.shape for n, a in T.tensors_of(T.R1, 1).items()}
    assert ToredraConfig.from_dict(raw).with_tensor_shapes(shapes) == ToredraConfig.from_dict(T.R1)
    with pytest.raises(ConfigError):
        c.with_tensor_shapes({})


def test_weight_slots_layer_runs_and_cache_layers():
    import torch
    from kestrel_llm_b200.config import ToredraConfig, resolve_architecture
    from kestrel_llm_b200.parts import CombinedSpec, FixedStateSpec, PagedKVSpec
    for name, (raw, seed) in T.CONFIGS.items():
        W = T.tensors_of(raw, seed)
        cfg = ToredraConfig.from_dict(raw)
        model = resolve_architecture("Toredra").build(cfg, torch.bfloat16, "meta")
        slots = {s.name: tuple(s.dest.shape) for s in model.weight_slots()}
        assert slots == {n: a.shape for n, a in W.items()}
        assert model.graph_safe and model.step_program(None) is None     # decode steps are captured; other steps walk the parts
        runs = [(i, again) for i, _rep, again in cfg.layer_runs()]
        assert runs == [(i, first and rep > 0) for i, rep, first in P.layer_order(raw)]
        assert [(c.block, c.cache, c.add_embedding) for c in model.order] == [(i, n, again) for n, (i, again) in enumerate(runs)]
        for (i, _), spec in zip(runs, model.cache_specs()):           # every run of a layer has a memory of its own
            m = raw["layers"][i]["mixer"]
            if raw["layers"][i]["type"] == "parallel":
                a, b = m["left"], m["right"]
                assert spec == CombinedSpec(PagedKVSpec(a["kv_heads"], a["dim"], 0, 0, a["vdim"]), FixedStateSpec((b["heads"] * b["dim"] * b["vdim"],)))
            else:
                assert spec == FixedStateSpec((m["heads"] * m["dim"] * m["dim"],))
    assert [i for i, _, _ in ToredraConfig.from_dict(T.R1).layer_runs()] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [a for _, _, a in ToredraConfig.from_dict(T.R1).layer_runs()] == [False, False, False, True, False, True, False, False]
    assert [i for i, _, _ in ToredraConfig.from_dict(T.R3).layer_runs()] == [0, 1, 0, 1]


def test_cache_layer_with_pages_and_a_state_slot():
    import torch
    from kestrel_llm_b200.cache import CacheManager
    from kestrel_llm_b200.parts import CombinedSpec, FixedStateSpec, PagedKVSpec
    cm = CacheManager([CombinedSpec(PagedKVSpec(2, 8, 0, 0, 12), FixedStateSpec((30,))), FixedStateSpec((7,)), PagedKVSpec(1, 4, 0, 0, 4)],
                      torch.float32, "cpu", 8, 6, 2, 256)
    assert tuple(cm.k[0].shape) == (7, 2, 8, 8) and tuple(cm.v[0].shape) == (7, 2, 8, 12) and tuple(cm.state[0].shape) == (3, 30)
    assert cm.k[1] is None and tuple(cm.state[1].shape) == (3, 7) and cm.state[2] is None
    assert cm.layer_group == [0, -1, 0] and cm.bytes_per_token() == 4 * (2 * (8 + 12) + 2 * 4)
    lc = cm.layer(0)
    assert lc.k is cm.k[0] and lc.state is cm.state[0]
    slot = cm.admit(5)
    cm.state[0][slot].fill_(3.0)
    cm.release(5)
    assert cm.admit(6) == slot and float(cm.state[0][slot].abs().sum()) == 0.0     # a slot that is used again starts from zero


def test_stretched_frequencies():
    from kestrel_llm_b200.parts import FrequencyScaling, RotaryInterleaved
    r = T.R1["layers"][1]["mixer"]["left"]["rot"]
    want = P.rotary_frequencies(r)
    plain = np.array([r["base"] ** (-2.0 * i / r["dims"]) for i in range(r["dims"] // 2)])
    ratio = want / plain
    assert ratio[0] == 1.0 and ratio[-1] == 0.25 and 0.25 < ratio[1] < 1.0 and 0.25 < ratio[2] < 1.0       # all three bands
    sc = r["scaling"]
    got = RotaryInterleaved(16, r["base"], "cpu", rotary_dim=r["dims"], scaling=FrequencyScaling(sc["factor"], sc["low"], sc["high"], sc["original"]))
    assert np.allclose(got.inv_freq.numpy(), want, rtol=1e-7) and got.rotary().pairing == "interleaved" and got.rotary().dim == 8
    none = RotaryInterleaved(16, r["base"], "cpu", rotary_dim=r["dims"])
    assert np.allclose(none.inv_freq.numpy(), plain, rtol=2e-7)
    # a wavelength exactly on a band's edge belongs to the middle band, whose blend meets both sides there
    edge = FrequencyScaling(4.0, 1.0, 4.0, 64.0).apply(np.array([2 * math.pi / 16, 2 * math.pi / 64]))
    assert np.allclose(edge, [2 * math.pi / 16, 2 * math.pi / 64 / 4.0])


def test_plain_prefixes_passes_and_sink():
    for name, (cfg, seed) in T.CONFIGS.items():
        W = {n: a.astype(np.float64) for n, a in T.tensors_of(cfg, seed).items()}
        toks = np.random.default_rng(1).integers(0, cfg["vocab"], 45).tolist()
        full = P.forward(cfg, W, toks)
        assert np.allclose(P.forward(cfg, W, toks[:20]), full[:20], atol=1e-9)          # a position sees only what is before it
        cap = cfg.get("logit_softcap")
        if cap:
            assert np.abs(full).max() < cap
    # one pass of the loop is no loop; further passes change the result
    cfg = json.loads(json.dumps(T.R1))
    W = {n: a.astype(np.float64) for n, a in T.tensors_of(cfg, 3).items()}
    toks = list(range(30))
    three = P.forward(cfg, W, toks)
    cfg["loop"]["times"] = 1
    once = P.forward(cfg, W, toks)
    cfg.pop("loop")
    assert np.array_equal(P.forward(cfg, W, toks), once) and np.abs(three - once).max() > 1e-2
    # the softmax's extra term: a very low one is no term; a high one takes nearly all the weight
    rng = np.random.default_rng(0)
    q, k, v = rng.standard_normal((9, 2, 4)), rng.standard_normal((9, 1, 4)), rng.standard_normal((9, 1, 3))
    none = P.sink_attention(q, k, v, 0.5, np.array([-1e4, -1e4]))
    assert np.allclose(none[0, 0], v[0, 0]) and np.abs(P.sink_attention(q, k, v, 0.5, np.array([30.0, -1e4]))[:, 0]).max() < 1e-6
    assert np.allclose(P.sink_attention(q, k, v, 0.5, np.array([30.0, -1e4]))[:, 1], none[:, 1])


def test_plain_recurrences_in_closed_form():
    rng = np.random.default_rng(2)
    T_, H, d, dv = 7, 2, 3, 4
    q, v = rng.standard_normal((T_, H, d)), rng.standard_normal((T_, H, dv))
    f = rng.uniform(0.1, 0.9, (T_, H, d))
    got = P.gated_linear_recurrence(q, f, v)
    for t in range(T_):                       # o_t = sum_s (q_t * prod_{s<u<=t} f_u * (1 - f_s)) . 1  v_s
        want = np.zeros((H, dv))
        for s in range(t + 1):
            wgt = (1.0 - f[s]) * np.prod(f[s + 1:t + 1], axis=0)
            want += np.einsum("hd,hd->h", q[t], wgt)[:, None] * v[s]
        assert np.allclose(got[t], want)
    # the delta rule with a = 1, w = 1 and a key repeated: the second write replaces what the first left along that key
    k = np.zeros((2, 1, 3))
    k[:, 0, 0] = 2.0
    v2 = rng.standard_normal((2, 1, 3))
    out = P.removal_recurrence(k.copy(), k, v2, np.ones((2, 1, 3)), np.ones((2, 1, 3)))
    assert np.allclose(out[1, 0], 4.0 * v2[1, 0], atol=1e-5)           # u^T S removed the first value: only the second is read
    out = P.removal_recurrence(k.copy(), k, v2, np.ones((2, 1, 3)), np.zeros((2, 1, 3)))
    assert np.allclose(out[1, 0], 4.0 * (v2[0, 0] + v2[1, 0]))         # nothing removed: both are
