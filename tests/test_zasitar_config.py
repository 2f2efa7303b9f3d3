"""Zasitar's configuration: keys, errors, layout, which layer reads whose keys, what the layers keep in the cache.
No GPU."""
import copy
import math

import pytest
import torch

from zasitar_helpers import CONFIGS, MIXED, RAGGED, SMALL, WIDE


def cfg_of(raw):
    from llmplayer_b200.config import config_from_dict
    return config_from_dict(raw)


def test_round_trip_and_registry():
    from llmplayer_b200.config import known_architectures
    from llmplayer_b200.config.zasitar import ZasitarConfig
    assert "Zasitar" in known_architectures()
    for raw, _, _ in CONFIGS.values():
        cfg = cfg_of(raw)
        assert isinstance(cfg, ZasitarConfig)
        assert cfg_of(cfg.to_dict()) == cfg
        assert cfg.max_positions() >= 65536
        assert "Zasitar" in cfg.describe()


@pytest.mark.parametrize("path,value", [
    (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "rot", "dims"), 26), (("layers", 0, "mixer", "rot", "dims"), 7),
    (("layers", 0, "mixer", "mask", "size"), 0), (("layers", 0, "mixer", "scale"), None), (("layers", 1, "type"), "lstm"),
    (("layers", 1, "mixer", "heads"), 0), (("layers", 2, "mixer", "kv_from"), 2), (("layers", 2, "mixer", "kv_from"), 1),
    (("layers", 2, "mixer", "kv_from"), 4), (("layers", 2, "mixer", "vdim"), 24), (("layers", 2, "mixer", "kv_heads"), 4),
    (("layers", 0, "mlp", "router", "top"), 7), (("layers", 0, "mlp", "expert", "limit"), 0.0),
    (("layers", 0, "mlp", "shared", "limit"), -1.0), (("layers", 1, "mlp", "kind"), "sparse"), (("layers", 1, "mlp", "ff"), None),
    (("layers", 4, "mixer", "rot", "scaling", "high"), 2.0), (("layers", 4, "mixer", "rot", "scaling", "factor"), 0.0),
    (("norm", "eps"), 0.0), (("width",), 0), (("vocab",), -3),
])
def test_bad_values_are_refused(path, value):
    from llmplayer_b200.errors import ConfigError
    raw = copy.deepcopy(SMALL)
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError):
        cfg_of(raw)


def test_a_layer_cannot_read_keys_of_a_layer_that_reads_others():
    from llmplayer_b200.errors import ConfigError
    raw = copy.deepcopy(WIDE)
    raw["layers"].append(copy.deepcopy(raw["layers"][3]))
    raw["layers"][4]["mixer"]["kv_from"] = 3
    with pytest.raises(ConfigError):
        cfg_of(raw)


def test_order_of_runs_and_whose_cache_they_read():
    runs = cfg_of(SMALL).layout().run_order()
    assert [r.layer for r in runs] == [0, 1, 2, 3, 4]
    assert [r.reads_cache_of for r in runs] == [None, None, 0, None, None]
    runs = cfg_of(WIDE).layout().run_order()
    assert [r.reads_cache_of for r in runs] == [None, None, None, 1]
    assert not any(r.reads_cache_of for r in cfg_of(RAGGED).layout().run_order())
    assert [r.reads_cache_of for r in cfg_of(MIXED).layout().run_order()] == [None, None, 1, 1, None, None, None]


def test_tensors_and_cache_requests():
    from llmplayer_b200.cache.sequence_cache import KVRequest, StateRequest
    from llmplayer_b200.engine.model import Model
    model = Model(cfg_of(SMALL).layout())
    specs = model.tensor_specs()
    assert specs["embed"].shape == (211, 72) and specs["head"].shape == (211, 72) and specs["final.norm"].shape == (72,)
    assert specs["l0.mix.q"].shape == (96, 72) and specs["l0.mix.k"].shape == (48, 72) and specs["l0.mix.v"].shape == (80, 72)
    assert specs["l0.mix.o"].shape == (72, 160) and specs["l0.mix.o.b"].shape == (72,) and specs["l0.mix.v.b"].shape == (80,)
    assert specs["l0.mix.q.norm"].shape == (24,) and specs["l0.mix.k.norm"].shape == (24,)
    assert specs["l0.norm1"].shape == specs["l0.ls1"].shape == specs["l0.ls2"].shape == (72,)
    # the layer that reads layer 0's keys has queries and an output only; without a feed-forward, no second norm
    assert specs["l2.mix.q"].shape == (96, 72) and specs["l2.mix.q.norm"].shape == (24,)
    assert not any(n.startswith(("l2.mix.k", "l2.mix.v", "l2.mlp.", "l2.norm2", "l2.ls2")) for n in specs)
    assert specs["l1.mix.r"].shape == (60, 72) and specs["l1.mix.o"].shape == (72, 60) and specs["l1.mix.u"].shape == (3, 20)
    assert specs["l1.mix.mu.w"].shape == (72,) and specs["l1.mix.w0"].shape == (60,) and specs["l1.mix.norm"].shape == (60,)
    assert specs["l1.mix.w1"].shape[1] == 72 and specs["l1.mix.w2"].shape[0] == 60
    assert specs["l1.mlp.gate.b"].shape == (104,) and specs["l1.mlp.down.b"].shape == (72,)
    assert specs["l0.mlp.e5.down"].shape == (72, 24) and specs["l0.mlp.shared.gate"].shape == (40, 72)
    assert specs["l0.mlp.shared.sg"].shape == (1, 72) and specs["l0.mlp.router.b"].shape == (6,)
    assert "l3.mlp.shared.up" not in specs and "l3.mlp.shared.sg" not in specs and "l0.mlp.e6.gate" not in specs
    reqs = model.cache_requests()
    assert len(reqs) == 5
    # layer 0's own window is 9 tokens, but layer 2 looks 17 tokens back over the same keys: the cache keeps 17.
    # Keys of 24 and values of 40 are stored in heads of 48.
    assert reqs[0] == KVRequest(2, 48, 17) and reqs[2] is None
    assert reqs[1] == (StateRequest((3, 20, 20), torch.float32), StateRequest((72,), torch.float32))
    assert reqs[3][0].shape == (1, 36, 36) and reqs[4] == KVRequest(3, 16, 1000)
    wide = Model(cfg_of(WIDE).layout()).cache_requests()
    assert wide[1] == KVRequest(1, 64, 70) and wide[3] is None and wide[2] == KVRequest(2, 128, 128)
    mixed = Model(cfg_of(MIXED).layout()).cache_requests()
    assert mixed[1] == KVRequest(2, 32, 300) and mixed[2] is None and mixed[3] is None and mixed[5] == KVRequest(1, 80, 64)


def test_stretched_frequencies():
    """The frequencies the library hands its rotation kernel against the rule in its plainest form: kept below the
    short wavelength, divided by the factor above the long one, blended linearly in original / wavelength between."""
    from llmplayer_b200.parts.position import inverse_frequencies
    import plain_zasitar
    for raw in (SMALL, WIDE, RAGGED):
        layout = cfg_of(raw).layout()
        for layer, entry in zip(layout.layers, raw["layers"]):
            if entry["type"] != "attention":
                continue
            got = inverse_frequencies(layer.mixer.position).double()
            ref = torch.tensor(plain_zasitar.rotary_frequencies(entry["mixer"]["rot"]), dtype=torch.float64)
            assert got.shape == ref.shape and float(((got - ref).abs() / ref).max()) < 1e-6
    # the three regimes all occur in WIDE's stretched layers: untouched, blended, divided
    rot = WIDE["layers"][1]["mixer"]["rot"]
    plain = [rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)]
    ratio = [s / p for s, p in zip(plain_zasitar.rotary_frequencies(rot), plain)]
    assert any(math.isclose(r, 1.0) for r in ratio) and any(math.isclose(r, 1 / 8.0) for r in ratio)
    assert any(1 / 8.0 + 1e-3 < r < 1.0 - 1e-3 for r in ratio)


def test_cache_gives_back_a_clean_state():
    from llmplayer_b200.cache.sequence_cache import SequenceCache
    from llmplayer_b200.engine.model import Model
    model = Model(cfg_of(SMALL).layout())
    cache = SequenceCache(model.cache_requests(), max_tokens=256, max_slots=3, kv_dtype=torch.float32, device="cpu")
    a = cache.acquire()
    cache.view(1).blocks[0][a].fill_(3.0)
    cache.view(1).blocks[1][a].fill_(-2.0)
    cache.release(a)
    b = cache.acquire()
    assert b == a and float(cache.view(1).blocks[0][b].abs().max()) == 0.0 and float(cache.view(1).blocks[1][b].abs().max()) == 0.0
    # the layer that reads layer 0's keys sees layer 0's pages
    assert cache.view(2) is None or cache.view(2).pages.data_ptr() == cache.view(0).pages.data_ptr()
