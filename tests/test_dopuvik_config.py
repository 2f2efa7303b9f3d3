"""Dopuvik's configuration: keys, errors, layout, tensors, what the layers keep in the cache (pages with kept first
tokens beside recurrent states in one layer), stretched frequencies. No GPU."""
import copy
import math

import pytest
import torch

from dopuvik_helpers import ATTENTIVE, CONFIGS, RAGGED, RECURRENT, SMALL, WIDE


def cfg_of(raw):
    from llmplayer_b200.config import config_from_dict
    return config_from_dict(raw)


def test_round_trip_and_registry():
    from llmplayer_b200.config import known_architectures
    from llmplayer_b200.config.dopuvik import DopuvikConfig
    assert "Dopuvik" in known_architectures()
    for raw, _, _ in CONFIGS.values():
        cfg = cfg_of(raw)
        assert isinstance(cfg, DopuvikConfig)
        assert cfg_of(cfg.to_dict()) == cfg
        assert cfg.max_positions() >= 65536
        assert "Dopuvik" in cfg.describe()
    cfg = cfg_of(SMALL)
    assert cfg.embedding_scale == 1.5 and cfg.logit_scale == 0.6 and cfg.norm_eps == 2e-6
    layout = cfg.layout()
    assert layout.embedding.scale == 1.5 and layout.head.logit_scale == 0.6 and layout.head.norm.kind == "layernorm"
    # constants that a model may leave out take their neutral values
    bare = copy.deepcopy(SMALL)
    del bare["embedding"], bare["logit_scale"]
    assert cfg_of(bare).embedding_scale == 1.0 and cfg_of(bare).logit_scale == 1.0


@pytest.mark.parametrize("path,value", [
    (("layers", 0, "mixer", "left", "kv_heads"), 3), (("layers", 0, "mixer", "left", "rot", "dims"), 26),
    (("layers", 0, "mixer", "left", "rot", "dims"), 7), (("layers", 0, "mixer", "left", "mask", "size"), 0),
    (("layers", 0, "mixer", "left", "mask", "keep_first"), -1), (("layers", 0, "mixer", "left", "scale"), None),
    (("layers", 0, "mixer", "right", "kv_heads"), 3), (("layers", 0, "mixer", "right", "conv"), 0),
    (("layers", 0, "mixer", "right", "conv"), 9), (("layers", 0, "mixer", "left_scale"), None),
    (("layers", 1, "type"), "lstm"), (("layers", 1, "mixer", "heads"), 0), (("layers", 1, "mixer", "groups"), 4),
    (("layers", 1, "mixer", "norm_groups"), 5), (("layers", 1, "mixer", "state"), None),
    (("layers", 2, "mixer", "kv_rank"), 0), (("layers", 2, "mixer", "q_rank"), None), (("layers", 2, "mixer", "rot", "dims"), 10),
    (("layers", 2, "mixer", "rot", "scaling", "factor"), 0.0), (("layers", 2, "mixer", "rot", "scaling", "fast"), -1.0),
    (("layers", 2, "mixer", "mask", "size"), -4),
    (("layers", 0, "mlp", "router", "top"), 5), (("layers", 0, "mlp", "router", "groups", "count"), 4),
    (("layers", 0, "mlp", "router", "groups", "keep"), 4), (("layers", 0, "mlp", "router", "identity"), -1),
    (("layers", 0, "mlp", "kind"), "dense"), (("layers", 0, "mlp", "expert", "ff"), 0),
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


def test_kept_tokens_need_a_window():
    from llmplayer_b200.errors import ConfigError
    raw = copy.deepcopy(SMALL)
    raw["layers"][0]["mixer"]["left"]["mask"] = {"keep_first": 3}
    with pytest.raises(ConfigError):
        cfg_of(raw)


def test_tensors_and_cache_requests():
    from llmplayer_b200.cache.sequence_cache import BundleRequest, KVRequest, RowsRequest, StateRequest
    from llmplayer_b200.engine.model import Model
    model = Model(cfg_of(SMALL).layout())
    specs = model.tensor_specs()
    assert specs["embed"].shape == (211, 72) and specs["head"].shape == (211, 72) and specs["final.norm"].shape == (72,)
    # the pair: attention with additive vectors, values wider than keys; a delta rule whose keys have fewer heads
    assert specs["l0.mix.left.q"].shape == (96, 72) and specs["l0.mix.left.k"].shape == (48, 72) and specs["l0.mix.left.v"].shape == (80, 72)
    assert specs["l0.mix.left.o"].shape == (72, 160) and specs["l0.mix.left.o.b"].shape == (72,) and specs["l0.mix.left.v.b"].shape == (80,)
    assert specs["l0.mix.right.q"].shape == (40, 72) and specs["l0.mix.right.k.conv"].shape == (40, 4) and specs["l0.mix.right.v"].shape == (48, 72)
    assert specs["l0.mix.right.v.conv"].shape == (48, 4) and specs["l0.mix.right.b"].shape == (4, 72) and specs["l0.mix.right.a"].shape == (4, 72)
    assert specs["l0.mix.right.A_log"].shape == (4,) and specs["l0.mix.right.dt_bias"].shape == (4,) and specs["l0.mix.right.norm"].shape == (12,)
    assert specs["l0.mix.right.g"].shape == (48, 72) and specs["l0.mix.right.o"].shape == (72, 48)
    assert "l0.mix.right.q.b" not in specs and "l0.mix.right.conv.b" not in specs
    # the state space: [z | x | B | C | dt] rows, convolution over x, B and C
    assert specs["l1.mix.in"].shape == (2 * 48 + 2 * 40 + 6, 72) and specs["l1.mix.conv"].shape == (128, 4) and specs["l1.mix.conv.b"].shape == (128,)
    assert specs["l1.mix.D"].shape == (6,) and specs["l1.mix.norm"].shape == (48,) and specs["l1.mix.o"].shape == (72, 48)
    assert not any(n.startswith(("l1.mlp.", "l1.norm2")) for n in specs)
    # latent attention: queries through a latent of 28, keys and values from one of 40 plus 8 shared rotated values
    assert specs["l2.mix.dq"].shape == (28, 72) and specs["l2.mix.dq.norm"].shape == (28,) and specs["l2.mix.uq"].shape == (96, 28)
    assert specs["l2.mix.dkv"].shape == (48, 72) and specs["l2.mix.dkv.norm"].shape == (40,) and specs["l2.mix.uk"].shape == (72, 40)
    assert specs["l2.mix.uv"].shape == (60, 40) and specs["l2.mix.o"].shape == (72, 60)
    # experts: router outputs and corrections count the identity experts, which have no tensors
    assert specs["l0.mlp.router"].shape == (6, 72) and specs["l0.mlp.correction"].shape == (6,)
    assert specs["l0.mlp.e4.down"].shape == (72, 24) and "l0.mlp.e5.gate" not in specs
    assert specs["l3.mlp.router"].shape == (8, 72) and "l3.mlp.e6.up" not in specs and specs["l2.mlp.router"].shape == (4, 72)
    reqs = model.cache_requests()
    assert len(reqs) == 5
    # keys of 24 and values of 40 are stored in heads of 48; the window's pages and the kept first tokens' pages
    assert reqs[0] == BundleRequest((KVRequest(2, 48, 9, 3),
                                     (StateRequest((4, 12, 20), torch.float32), StateRequest((3, 128), torch.float32))))
    assert reqs[1] == (StateRequest((6, 8, 20), torch.float32), StateRequest((3, 128), torch.float32))
    assert reqs[2] == RowsRequest(48, 17)
    assert reqs[3] == (StateRequest((2, 16, 8), torch.float32), StateRequest((1, 48), torch.float32))
    # one tap: nothing of the convolution is carried
    assert reqs[4] == BundleRequest((KVRequest(3, 16, 1000, 0),
                                     (StateRequest((2, 24, 16), torch.float32), StateRequest((0, 80), torch.float32))))
    wide = Model(cfg_of(WIDE).layout()).cache_requests()
    assert wide[0] == RowsRequest(96, 70) and wide[1].members[0] == KVRequest(1, 64, 64, 70) and wide[4] == RowsRequest(192, None)
    assert all(isinstance(r, tuple) for r in Model(cfg_of(RECURRENT).layout()).cache_requests())
    assert all(isinstance(r, RowsRequest) for r in Model(cfg_of(ATTENTIVE).layout()).cache_requests())


def test_a_mixture_counts_identities_in_its_groups():
    layout = cfg_of(SMALL).layout()
    routing = layout.layers[0].ffn.routing
    assert (routing.num_experts, routing.identity_experts, routing.groups, routing.keep_groups, routing.top) == (5, 1, 3, 2, 2)
    assert routing.scoring == "softmax_groups" and routing.weight_scale == 1.5 and routing.correction == "l0.mlp.correction"
    assert layout.layers[1].ffn is None and layout.layers[1].ffn_norm is None
    assert layout.layers[0].mixer.left_scale == 0.7 and layout.layers[0].mixer.right_scale == 1.3
    assert layout.layers[0].mixer.left.keep_first == 3 and layout.layers[4].mixer.left.keep_first is None


def test_stretched_frequencies_and_their_factor():
    """The frequencies the library hands its rotation kernels against the rule in its plainest form: a ramp over the
    pair index between the pairs that make ``fast`` and ``slow`` turns over the original context."""
    from llmplayer_b200.parts.position import inverse_frequencies, rotation_magnitude
    import plain_dopuvik
    seen = 0
    for raw in (SMALL, WIDE, ATTENTIVE):
        layout = cfg_of(raw).layout()
        for layer, entry in zip(layout.layers, raw["layers"]):
            if entry["type"] != "latent_attention":
                continue
            rot = entry["mixer"]["rot"]
            got = inverse_frequencies(layer.mixer.position).double()
            if rot.get("scaling"):
                ref, magnitude = plain_dopuvik.yarn_frequencies(rot["base"], rot["dims"], rot["scaling"])
                seen += 1
            else:
                ref, magnitude = plain_dopuvik.plain_frequencies(rot["base"], rot["dims"]), 1.0
            ref = torch.tensor(ref, dtype=torch.float64)
            assert got.shape == ref.shape and float(((got - ref).abs() / ref).max()) < 1e-6
            assert math.isclose(rotation_magnitude(layer.mixer.position), magnitude)
            assert layer.mixer.position.pairing == "interleaved"
    assert seen == 3
    # untouched, blended and divided frequencies all occur in WIDE's first layer
    rot = WIDE["layers"][0]["mixer"]["rot"]
    plain = plain_dopuvik.plain_frequencies(rot["base"], rot["dims"])
    ratio = [s / p for s, p in zip(plain_dopuvik.yarn_frequencies(rot["base"], rot["dims"], rot["scaling"])[0], plain)]
    assert any(math.isclose(r, 1.0) for r in ratio) and any(math.isclose(r, 1 / 8.0) for r in ratio)
    assert any(1 / 8.0 + 1e-3 < r < 1.0 - 1e-3 for r in ratio)
    assert math.isclose(plain_dopuvik.yarn_frequencies(rot["base"], rot["dims"], rot["scaling"])[1], 0.1 * math.log(8.0) + 1.0)


def test_pages_behind_a_window_go_back_but_not_the_kept_ones():
    from llmplayer_b200.cache.pages import PageMap
    pages = PageMap(16, window=64, keep_first=70)          # two pages hold the kept tokens
    pages.open(0)
    pages.extend(0, 64 * 6)
    pages.trim(0, 64 * 6)
    table = pages.table(0)
    assert table[0] >= 0 and table[1] >= 0 and table[2] == -1 and table[3] == -1 and table[4] == -1 and table[5] >= 0
    plain = PageMap(16, window=64)
    plain.open(0)
    plain.extend(0, 64 * 6)
    plain.trim(0, 64 * 6)
    assert plain.table(0)[:5] == [-1] * 5 and plain.table(0)[5] >= 0
    one = PageMap(16, window=10, keep_first=1)
    one.open(3)
    one.extend(3, 200)
    one.trim(3, 200)
    assert one.table(3)[0] >= 0 and one.table(3)[1] == -1 and one.table(3)[2] >= 0 and one.pool.num_free == 16 - 3


def test_cache_gives_back_clean_states_and_serves_both_members_of_a_pair():
    from llmplayer_b200.cache.sequence_cache import BundleView, KVView, SequenceCache, StateView
    from llmplayer_b200.engine.model import Model
    model = Model(cfg_of(SMALL).layout())
    cache = SequenceCache(model.cache_requests(), max_tokens=256, max_slots=3, kv_dtype=torch.float32, device="cpu")
    pair = cache.view(0)
    assert isinstance(pair, BundleView) and isinstance(pair.members[0], KVView) and isinstance(pair.members[1], StateView)
    assert pair.members[0].pages.shape[1:] == (2, 2, 64, 48) and pair.members[1].blocks[1].shape[1:] == (3, 128)
    # the two pairs' pages live in groups of their own (their windows differ); the latent rows in a third
    assert len({pair.members[0].group_index, cache.view(4).members[0].group_index, cache.view(2).group_index}) == 3
    a = cache.acquire()
    for view in (pair.members[1], cache.view(1), cache.view(3), cache.view(4).members[1]):
        for block in view.blocks:
            block[a].fill_(3.0)
    cache.release(a)
    b = cache.acquire()
    assert b == a
    for view in (pair.members[1], cache.view(1), cache.view(3), cache.view(4).members[1]):
        for block in view.blocks:
            assert block[b].numel() == 0 or float(block[b].abs().max()) == 0.0
    # a step that outgrows the window gives pages back, except the one with the kept first tokens
    cache.reserve([b], [200])
    cache.commit([b], [200])
    table = cache.groups[pair.members[0].group_index].pages.table(b)
    assert table[0] >= 0 and table[1] == -1 and table[2] == -1 and table[3] >= 0
