"""Korirax without a GPU: the configuration, the model's weight slots against the tests' own list of tensor names, the
layer order with its loop, and the plain statement against itself."""
import copy

import numpy as np
import pytest

import korirax_util as K
import plain_korirax as P


def _config(cfg):
    from kestrel_llm_b200.config import resolve_architecture
    arch = resolve_architecture("Korirax")
    return arch, arch.config_class.from_dict(cfg)


@pytest.mark.parametrize("name", list(K.CONFIGS))
def test_configuration_round_trip_and_weight_slots(name):
    import torch
    cfg, seed = K.CONFIGS[name]
    arch, c = _config(cfg)
    assert arch.config_class.from_dict(c.to_json_dict()) == c
    model = arch.build(c, torch.bfloat16, "meta")
    slots = {s.name: tuple(s.dest.shape) for s in model.weight_slots()}
    W = K.tensors_of(cfg, seed)
    assert slots == {n: a.shape for n, a in W.items()}
    assert [(call.block, call.add_row) for call in model.order] == [(i, -1 if not first else t) for i, t, first in P.layer_runs(cfg)]
    assert len({call.cache for call in model.order}) == len(model.order)          # every run of a layer has its own memory


def test_sizes_of_a_table_come_from_the_checkpoint():
    cfg = copy.deepcopy(K.K2)
    del cfg["layers"][1]["mixer"]["bias_rows"]
    arch, c = _config(cfg)
    import torch
    with pytest.raises(ValueError):
        arch.build(c, torch.bfloat16, "meta")
    c = c.with_tensor_shapes({"l1.mix.rel": (7, 5)})
    assert c.layers[1].mixer.bias_rows == 7
    arch.build(c, torch.bfloat16, "meta")


@pytest.mark.parametrize("bad", [("layers", 0, "type", "window"), ("layers", 1, "mlp", {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 6, "top": 4, "groups": {"count": 3, "keep": 1}}}),
                                 ("layers", 0, "mixer", {"width": 42, "blocks": 4, "conv": 2}), ("loop", None, None, {"start": 2, "stop": 9, "times": 2})])
def test_configuration_refuses(bad):
    from kestrel_llm_b200.config.model_config import ConfigError
    cfg = copy.deepcopy(K.K2)
    key, i, sub, value = bad
    if i is None:
        cfg[key] = value
    else:
        cfg[key][i][sub] = value
    with pytest.raises(ConfigError):
        _config(cfg)


def test_plain_statement_is_causal_and_its_loop_runs_in_order():
    cfg, seed = K.CONFIGS["K1"]
    W = K.bf16_round(K.tensors_of(cfg, seed))
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], size=50).tolist()
    whole = P.forward(toks, W, cfg)
    assert np.abs(whole[:31] - P.forward(toks[:31], W, cfg)).max() < 1e-9
    runs = P.layer_runs(cfg)
    assert [i for i, _, _ in runs] == [0, 1, 0, 1, 0, 1, 2, 3] and [t for _, t, first in runs if first] == [0, 1, 2]


def test_distance_buckets():
    rows, far = 16, 120
    b = [P.distance_bucket(n, rows, far) for n in range(400)]
    assert b[:8] == list(range(8)) and b[8] == 8 and b[far] == rows - 1 and b[399] == rows - 1
    assert all(y - x in (0, 1) for x, y in zip(b, b[1:]))
    rows, far = 7, 25          # an odd number of rows: the linear part is rows // 2 long
    b = [P.distance_bucket(n, rows, far) for n in range(60)]
    assert b[:4] == [0, 1, 2, 3] and max(b) == 6 and b[25] == 6
