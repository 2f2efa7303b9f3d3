"""Small Dopuvik configurations with sizes of their own, and seeded model folders for them."""
import json
import os

import torch


def _moe(ff, experts, identity, top, count=1, keep=1, scale=1.0):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "identity": identity, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}


# Odd sizes: values wider than keys and narrower, a rotation over part of a head and none at all, kept first tokens
# with a short window, a window wider than every prompt without kept tokens, a delta rule whose values have more heads
# than its keys, convolutions of 4, 2 and ONE tap, a state space with two groups and a norm in three parts, layers
# without a feed-forward, experts without identities and without groups, groups of two router outputs of which one is an
# identity.
SMALL = {
    "architecture": "Dopuvik", "vocab": 211, "width": 72, "norm": {"eps": 2e-6}, "embedding": {"scale": 1.5}, "logit_scale": 0.6,
    "layers": [
        {"type": "parallel",
         "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 40, "scale": 0.3, "mask": {"size": 9, "keep_first": 3},
                            "rot": {"base": 10000.0, "dims": 16}},
                   "right": {"heads": 4, "kv_heads": 2, "dim": 20, "vdim": 12, "conv": 4},
                   "left_scale": 0.7, "right_scale": 1.3},
         "mlp": _moe(24, 5, 1, 2, count=3, keep=2, scale=1.5)},
        {"type": "mamba2", "mixer": {"heads": 6, "vdim": 8, "state": 20, "groups": 2, "conv": 4, "norm_groups": 3}, "mlp": None},
        {"type": "latent_attention",
         "mixer": {"heads": 3, "dim": 24, "rot_dim": 8, "vdim": 20, "kv_rank": 40, "q_rank": 28, "scale": 0.2, "mask": {"size": 17},
                   "rot": {"base": 5000.0, "dims": 8, "scaling": {"factor": 3.0, "original": 32, "fast": 8.0, "slow": 1.0}}},
         "mlp": _moe(16, 4, 0, 1)},
        {"type": "mamba2", "mixer": {"heads": 2, "vdim": 16, "state": 8, "groups": 1, "conv": 2, "norm_groups": 1},
         "mlp": _moe(8, 6, 2, 4, count=4, keep=3, scale=0.8)},
        {"type": "parallel",
         "mixer": {"left": {"heads": 3, "kv_heads": 3, "dim": 16, "vdim": 16, "scale": 0.25, "mask": {"size": 1000, "keep_first": 0}},
                   "right": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 24, "conv": 1},
                   "left_scale": 1.0, "right_scale": 0.5},
         "mlp": None},
    ],
}
# Sizes the tensor-core kernels take: a latent window of 70 (its edge crosses a page's border of 64 while decoding),
# MORE kept first tokens than a page holds beside a window of exactly one page, eight query heads on one key head,
# rotation over half of a head, heads of 128, a latent layer without window and without stretching whose heads (64 +
# 64, values of 128) fill the prompt kernel's size, a state space with heads of 64 in two groups.
WIDE = {
    "architecture": "Dopuvik", "vocab": 384, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0}, "logit_scale": 1.0,
    "layers": [
        {"type": "latent_attention",
         "mixer": {"heads": 4, "dim": 32, "rot_dim": 32, "vdim": 64, "kv_rank": 64, "q_rank": 48, "scale": 0.15, "mask": {"size": 70},
                   "rot": {"base": 1000000.0, "dims": 32, "scaling": {"factor": 8.0, "original": 64, "fast": 4.0, "slow": 1.0}}},
         "mlp": _moe(64, 8, 4, 3, count=4, keep=2, scale=2.0)},
        {"type": "parallel",
         "mixer": {"left": {"heads": 8, "kv_heads": 1, "dim": 64, "vdim": 64, "scale": 0.2, "mask": {"size": 64, "keep_first": 70},
                            "rot": {"base": 10000.0, "dims": 32}},
                   "right": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 32, "conv": 4},
                   "left_scale": 1.0, "right_scale": 0.5},
         "mlp": _moe(32, 6, 0, 2, count=2, keep=1)},
        {"type": "mamba2", "mixer": {"heads": 4, "vdim": 64, "state": 64, "groups": 2, "conv": 4, "norm_groups": 2},
         "mlp": _moe(64, 8, 4, 3, count=4, keep=2, scale=2.0)},
        {"type": "parallel",
         "mixer": {"left": {"heads": 2, "kv_heads": 2, "dim": 128, "vdim": 64, "scale": 0.09, "mask": {"size": 128, "keep_first": 1},
                            "rot": {"base": 50000.0, "dims": 128}},
                   "right": {"heads": 2, "kv_heads": 2, "dim": 128, "vdim": 128, "conv": 3},
                   "left_scale": 0.8, "right_scale": 1.2},
         "mlp": None},
        {"type": "latent_attention",
         "mixer": {"heads": 2, "dim": 64, "rot_dim": 64, "vdim": 128, "kv_rank": 128, "q_rank": 64, "scale": 0.1,
                   "rot": {"base": 10000.0, "dims": 64}},
         "mlp": _moe(48, 4, 2, 2, count=3, keep=2, scale=1.25)},
    ],
}
# A width that is no multiple of 8 (every product leaves the tensor cores, also in bfloat16), a latent window of ONE
# token, a window of two with five kept first tokens (more kept than seen), one head, one group, every router output
# chosen (top = experts + identities), groups of one expert of which one is kept.
RAGGED = {
    "architecture": "Dopuvik", "vocab": 131, "width": 52, "norm": {"eps": 3e-5}, "embedding": {"scale": 1.0}, "logit_scale": 2.0,
    "layers": [
        {"type": "mamba2", "mixer": {"heads": 1, "vdim": 12, "state": 6, "groups": 1, "conv": 3, "norm_groups": 2},
         "mlp": _moe(12, 2, 1, 3)},
        {"type": "latent_attention",
         "mixer": {"heads": 5, "dim": 10, "rot_dim": 2, "vdim": 12, "kv_rank": 10, "q_rank": 6, "scale": 0.4, "mask": {"size": 1},
                   "rot": {"base": 100.0, "dims": 2}},
         "mlp": _moe(8, 3, 0, 1, count=3, keep=1)},
        {"type": "parallel",
         "mixer": {"left": {"heads": 5, "kv_heads": 1, "dim": 10, "vdim": 12, "scale": 0.4, "mask": {"size": 2, "keep_first": 5},
                            "rot": {"base": 100.0, "dims": 2}},
                   "right": {"heads": 1, "kv_heads": 1, "dim": 6, "vdim": 10, "conv": 2},
                   "left_scale": 1.1, "right_scale": 0.9},
         "mlp": _moe(20, 3, 3, 2, count=2, keep=2, scale=0.5)},
    ],
}
# Models of one kind of layer only: no pages at all, and no recurrent state at all.
RECURRENT = {
    "architecture": "Dopuvik", "vocab": 150, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0}, "logit_scale": 1.0,
    "layers": [
        {"type": "mamba2", "mixer": {"heads": 4, "vdim": 16, "state": 16, "groups": 4, "conv": 4, "norm_groups": 4}, "mlp": _moe(16, 4, 2, 2, count=2, keep=2)},
        {"type": "mamba2", "mixer": {"heads": 8, "vdim": 8, "state": 32, "groups": 1, "conv": 3, "norm_groups": 1}, "mlp": None},
    ],
}
ATTENTIVE = {
    "architecture": "Dopuvik", "vocab": 170, "width": 80, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0}, "logit_scale": 1.0,
    "layers": [
        {"type": "latent_attention",
         "mixer": {"heads": 5, "dim": 16, "rot_dim": 16, "vdim": 16, "kv_rank": 32, "q_rank": 24, "scale": 0.18, "mask": {"size": 12},
                   "rot": {"base": 800.0, "dims": 16}},
         "mlp": _moe(24, 5, 3, 3, count=4, keep=2)},
        {"type": "latent_attention",
         "mixer": {"heads": 2, "dim": 8, "rot_dim": 32, "vdim": 40, "kv_rank": 16, "q_rank": 16, "scale": 0.2, "mask": {"size": 100},
                   "rot": {"base": 800.0, "dims": 32, "scaling": {"factor": 2.0, "original": 40, "fast": 16.0, "slow": 2.0}}},
         "mlp": None},
    ],
}
CONFIGS = {"small": (SMALL, 41, 0.09), "wide": (WIDE, 42, 0.06), "ragged": (RAGGED, 43, 0.1), "recurrent": (RECURRENT, 44, 0.1),
           "attentive": (ATTENTIVE, 45, 0.1)}

# bfloat16: at most four times the worst error that the comparisons of each configuration achieved on a B200 at all but
# one position in fifty (4.5e-3, 3.9e-3, 2.5e-3, 5.1e-3, 2.5e-3; see test_dopuvik_model.close)
BFLOAT16_BOUND = {"small": 1.8e-2, "wide": 1.6e-2, "ragged": 1e-2, "recurrent": 2e-2, "attentive": 1e-2}
ROUTER_FACTOR = 0.6
ROUTE_CHANNELS = 12         # channels of the stream that carry each token's routing code (see make_model)


def bound(dtype, name):
    return 2e-5 if dtype == "float32" else BFLOAT16_BOUND[name]


def _mixer_prefixes(p, layer):
    if layer["type"] == "parallel":
        return [p + "mix.left.", p + "mix.right."]
    return [p + "mix."]


def make_model(tmp_path, name, dtype="bfloat16"):
    """A model folder for configuration ``name``: the library's seeded writer, then

    * the tensors whose random draw would switch a mechanism off are drawn again: the additive vectors of the
      projections, the convolutions' taps and bias (of order one, so that the silu behind them bends), the step sizes'
      bias (decays from nearly 1 to nearly 0), the choice's correction;
    * the routing is made robust against rounding: the first ROUTE_CHANNELS channels of the stream carry a code per
      token (a permutation of distinct levels with wide gaps, in the embedding), no sublayer writes to these channels
      (the rows of every output map are zero there; identity experts scale the code, which keeps its order), and every
      router reads only them, one channel per router output. Corrections are -2, 0 or 2: where two differ they decide, where they agree the scores do. No choice of experts
      then rests on a close call, and bfloat16 runs choose as float64 does;
    * a delta rule's output is divided by its own root mean square, so early in a sequence, where the state holds one
      write, its SIGN is that of q . k: with unrelated maps that product is near zero every so often and the output then
      rests on rounding. The query maps and taps are therefore the key maps and taps plus a third of a random draw;
      a state space's C rows likewise follow its B rows.
    """
    from llmplayer_b200.config import config_from_dict
    from llmplayer_b200.weights import write_random_model
    from llmplayer_b200.weights.safetensors_io import write_safetensors
    from plain_llama import read_safetensors
    raw, seed, std = CONFIGS[name]
    out = os.path.join(str(tmp_path), f"dopuvik_{name}_{dtype}")
    write_random_model(config_from_dict(raw), seed, out, dtype=dtype, std=std)
    path = os.path.join(out, "model.safetensors")
    tensors = read_safetensors(path)
    gen = torch.Generator().manual_seed(seed + 100)
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    d, C = raw["width"], ROUTE_CHANNELS

    def draw(*shape, scale=1.0, shift=0.0):
        return (shift + scale * torch.randn(*shape, generator=gen)).to(store)

    def mixed(name_a, name_b):
        return (tensors[name_b].to(torch.float32) + 0.3 * tensors[name_a].to(torch.float32)).to(store)

    levels = torch.linspace(-2.2, 2.2, C)
    embed = tensors["embed"].to(torch.float32)
    for t in range(raw["vocab"]):
        embed[t, :C] = levels[torch.randperm(C, generator=gen)]
    tensors["embed"] = embed.to(store)
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "mamba2":
            q = p + "mix."
            inner, GN = m["heads"] * m["vdim"], m["groups"] * m["state"]
            taps = draw(inner + 2 * GN, m["conv"], scale=0.6).to(torch.float32)
            taps[inner + GN:] = taps[inner:inner + GN] + 0.3 * taps[inner + GN:]
            tensors[q + "conv"] = taps.to(store)
            tensors[q + "conv.b"] = draw(inner + 2 * GN, scale=0.3)
            tensors[q + "dt_bias"] = draw(m["heads"], scale=1.5)
            tensors[q + "A_log"] = draw(m["heads"], scale=0.7)
            w_in = tensors[q + "in"].to(torch.float32)
            w_in[2 * inner + GN:2 * inner + 2 * GN] = w_in[2 * inner:2 * inner + GN] + 0.3 * w_in[2 * inner + GN:2 * inner + 2 * GN]
            tensors[q + "in"] = w_in.to(store)
        elif layer["type"] == "parallel":
            l, r = p + "mix.left.", p + "mix.right."
            ml, mr = m["left"], m["right"]
            tensors[l + "q.b"] = draw(ml["heads"] * ml["dim"], scale=0.3)
            tensors[l + "k.b"] = draw(ml["kv_heads"] * ml["dim"], scale=0.3)
            tensors[l + "v.b"] = draw(ml["kv_heads"] * ml["vdim"], scale=0.3)
            tensors[l + "o.b"] = draw(d, scale=0.3)
            for n, rows in (("q", mr["kv_heads"] * mr["dim"]), ("k", mr["kv_heads"] * mr["dim"]), ("v", mr["heads"] * mr["vdim"])):
                tensors[r + n + ".conv"] = draw(rows, mr["conv"], scale=0.6)
            tensors[r + "q"] = mixed(r + "q", r + "k")
            tensors[r + "q.conv"] = mixed(r + "q.conv", r + "k.conv")
            tensors[r + "dt_bias"] = draw(mr["heads"], scale=1.5)
            tensors[r + "A_log"] = draw(mr["heads"], scale=0.7)
        for q in _mixer_prefixes(p, layer):
            o = tensors[q + "o"].clone()
            o[:C] = 0
            tensors[q + "o"] = o
            if q + "o.b" in tensors:
                b = tensors[q + "o.b"].clone()
                b[:C] = 0
                tensors[q + "o.b"] = b
        mlp = layer["mlp"]
        if mlp is not None:
            r = mlp["router"]
            outputs = r["experts"] + r["identity"]
            assert outputs <= C
            router = torch.zeros(outputs, d)
            router[torch.arange(outputs), torch.arange(outputs)] = ROUTER_FACTOR
            tensors[p + "mlp.router"] = router.to(store)
            tensors[p + "mlp.correction"] = (2.0 * torch.randint(-1, 2, (outputs,), generator=gen).float()).to(store)
            for e in range(r["experts"]):
                down = tensors[f"{p}mlp.e{e}.down"].clone()
                down[:C] = 0
                tensors[f"{p}mlp.e{e}.down"] = down
            gain = tensors[p + "norm2"].to(torch.float32)
            gain[:C] = 1.0
            tensors[p + "norm2"] = gain.to(store)
    write_safetensors(path, tensors, metadata={"format": "pt"})
    with open(os.path.join(out, "config.json"), "w") as fh:
        json.dump(raw, fh, indent=1)
    return out


def plain_logits(model_dir, tokens, rows=None, gaps=None, streams=None):
    import plain_dopuvik
    cfg, w = plain_dopuvik.read_model(model_dir)
    return plain_dopuvik.forward(cfg, w, tokens, dtype=torch.float64, rows=rows, gaps=gaps, streams=streams)
