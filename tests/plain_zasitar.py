"""Plain implementation of the Zasitar decoder for the tests: whole sequences, no cache, float64 by default,
one function per mechanism, written from the design's equations. It shares no code with the library's parts.

Notation: x is the stream [T, d]; positions count from 0; matrices are stored [out, in] and applied as h @ W.T.
A layer reads the stream itself (no norm in front of a sublayer) and adds the sublayer's result after an RMS norm
with a gain and a second per-feature factor (the layer scale):

    x <- x + ls1 * rms_norm(mixer(x), norm1);   x <- x + ls2 * rms_norm(ffn(x), norm2)
"""
import json
import math
import os

import torch

from plain_llama import read_safetensors


def read_model(model_dir):
    with open(os.path.join(model_dir, "config.json")) as fh:
        cfg = json.load(fh)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# --------------------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    """x divided by the root of (its mean square + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, gain, eps):
    return unit_rms(x, eps) * gain


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_frequencies(rot):
    """f_i = base^(-2i / dims), stretched by wavelength: kept where 2 pi / f < original / high, divided by ``factor``
    where 2 pi / f > original / low, blended linearly in original / wavelength in between."""
    dims, s = rot["dims"], rot.get("scaling")
    out = []
    for i in range(dims // 2):
        f = rot["base"] ** (-2.0 * i / dims)
        if s:
            wavelength = 2.0 * math.pi / f
            if wavelength > s["original"] / s["low"]:
                f = f / s["factor"]
            elif not wavelength < s["original"] / s["high"]:
                t = (s["original"] / wavelength - s["low"]) / (s["high"] - s["low"])
                f = (1.0 - t) * f / s["factor"] + t * f
        out.append(f)
    return out


def rotate_split_halves(v, positions, rot):
    """Rotate the first ``dims`` features of the last axis: feature i pairs with i + dims / 2, by the angle
    position * f_i; (u, w) -> (u cos - w sin, w cos + u sin). The rest pass unchanged. ``v``: [T, heads, n]."""
    dims = rot["dims"]
    if dims == 0:
        return v
    out = v.clone()
    half = dims // 2
    for i, f in enumerate(rotary_frequencies(rot)):
        angle = positions.to(v.dtype) * f
        cos, sin = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        u, w = v[..., i], v[..., i + half]
        out[..., i] = u * cos - w * sin
        out[..., i + half] = w * cos + u * sin
    return out


def softmax_plus_one(scores):
    """Row-wise exp(s_j) / (1 + sum_j exp(s_j)): a softmax with one more term of score 0 that carries no value."""
    big = torch.clamp(scores.max(-1, keepdim=True).values, min=0.0)
    e = torch.exp(scores - big)
    return e / (e.sum(-1, keepdim=True) + torch.exp(-big))


def window_mask(positions, size):
    """seen[i, j]: 0 <= position_i - position_j < size."""
    gap = positions[:, None] - positions[None, :]
    return (gap >= 0) & (gap < size)


# --------------------------------------------------------------------------- mixers
def attention_keys_values(h, w, p, m, eps, positions):
    """The keys (normed per head with a gain shared by the heads, then rotated) and values of a layer that has its own."""
    T = h.shape[0]
    G, dk, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, dk)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    k = rotate_split_halves(rms_norm(k, w[p + "k.norm"], eps), positions, m["rot"])
    return k, v


def windowed_attention(h, w, p, m, eps, kv=None, positions=None):
    """Grouped-query attention over a sliding window with the plus-one softmax. ``kv``: the keys and values of
    another layer to attend over (this layer then has none of its own). Returns the output and the (k, v) used."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T) if positions is None else positions
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, dk)
    q = rotate_split_halves(rms_norm(q, w[p + "q.norm"], eps), positions, m["rot"])
    k, v = attention_keys_values(h, w, p, m, eps, positions) if kv is None else kv
    seen = window_mask(positions, m["mask"]["size"])
    heads = []
    for head in range(H):
        g = head // (H // G)
        s = ((q[:, head] @ k[:, g].T) * m["scale"]).masked_fill(~seen, -math.inf)
        heads.append(softmax_plus_one(s) @ v[:, g])
    return torch.cat(heads, dim=-1) @ w[p + "o"].T + w[p + "o.b"], (k, v)


def wkv(h, w, p, m, eps, state=None):
    """Time mixing with a matrix state per head. With h' the previous token's input (zeros before the first):
    every one of r, k, v, g, w reads h + (h' - h) * mu of its own; decay = exp(-exp(W2 tanh(W1 mix_w) + w0)) per key
    channel; o_t = (S + diag(u) k_t v_t^T)^T r_t from the state BEFORE the token, then S <- diag(decay_t) S + k_t v_t^T.
    ``state``: (previous input [d], S [H, dk, dk]) to go on from. Returns the output and the state it leaves."""
    T, d = h.shape
    H, n = m["heads"], m["dim"]
    if state is None:
        last, S = torch.zeros(d, dtype=h.dtype), torch.zeros(H, n, n, dtype=h.dtype)
    else:
        last, S = state
    before = torch.cat([last[None], h[:-1]], dim=0)

    def mix(which):
        return h + (before - h) * w[p + "mu." + which]

    r = (mix("r") @ w[p + "r"].T).view(T, H, n)
    k = (mix("k") @ w[p + "k"].T).view(T, H, n)
    v = (mix("v") @ w[p + "v"].T).view(T, H, n)
    g = mix("g") @ w[p + "g"].T
    gate = g * torch.sigmoid(g)
    decay = torch.exp(-torch.exp(torch.tanh(mix("w") @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, n)
    u = w[p + "u"]
    out = []
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[t]))
        S = decay[t][:, :, None] * S + kv
    o = unit_rms(torch.stack(out), eps).reshape(T, H * n) * w[p + "norm"] * gate
    return o @ w[p + "o"].T, (h[-1].clone(), S)


# --------------------------------------------------------------------------- feed-forwards
def dense_ffn(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T + w[p + "gate.b"]) * (h @ w[p + "up"].T + w[p + "up.b"])) @ w[p + "down"].T + w[p + "down.b"]


def clamped_expert(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(logits, top):
    """logits [T, E] -> (chosen experts [T, top], their weights = softmax over the chosen logits alone, the smallest
    gap between the last chosen and the first refused logit)."""
    ranked = logits.sort(dim=-1, descending=True)
    gap = float((ranked.values[:, top - 1] - ranked.values[:, top]).min()) if top < logits.shape[1] else math.inf
    return ranked.indices[:, :top], torch.softmax(ranked.values[:, :top], dim=-1), gap


def mixture_ffn(h, w, p, mlp, gaps=None):
    r = mlp["router"]
    chosen, weights, gap = route(h @ w[p + "router"].T + w[p + "router.b"], r["top"])
    if gaps is not None:
        gaps.append(gap)
    out = torch.zeros_like(h)
    for e in range(r["experts"]):
        for slot in range(r["top"]):
            rows = (chosen[:, slot] == e).nonzero().flatten()
            if rows.numel():
                out[rows] += weights[rows, slot][:, None] * clamped_expert(h[rows], w, f"{p}e{e}.", mlp["expert"]["limit"])
    if mlp.get("shared"):
        share = torch.sigmoid(h @ w[p + "shared.sg"].T)                  # one number per token
        out = out + share * clamped_expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


# --------------------------------------------------------------------------- the model
def forward(cfg, w, tokens, dtype=torch.float64, rows=None, streams=None, gaps=None):
    """Logits [T (or len(rows)), vocab] of a whole sequence. ``streams``: a list that receives the stream after
    every layer; ``gaps``: a list that receives the smallest deciding gap of every routing."""
    w = {k: v.to(dtype) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)].clone()
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            source = m.get("kv_from")
            y, kept[i] = windowed_attention(x, w, p + "mix.", m, eps, kv=None if source is None else kept[source])
        else:
            y, _ = wkv(x, w, p + "mix.", m, eps)
        x = x + rms_norm(y, w[p + "norm1"], eps) * w[p + "ls1"]
        if layer["mlp"] is not None:
            if layer["mlp"]["kind"] == "dense":
                y = dense_ffn(x, w, p + "mlp.")
            else:
                y = mixture_ffn(x, w, p + "mlp.", layer["mlp"], gaps)
            x = x + rms_norm(y, w[p + "norm2"], eps) * w[p + "ls2"]
        if streams is not None:
            streams.append(x.clone())
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long)]
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
