"""Plain implementation of the Dopuvik decoder for the tests: whole sequences, no cache, float64 by default,
one function per mechanism, written from the design's equations. It shares no code with the library's parts.

Notation: x is the stream [T, d]; positions count from 0; matrices are stored [out, in] and applied as h @ W.T.
A layer is pre-norm with layer norms (a gain, no bias):

    x <- x + mixer(layer_norm(x, norm1));   x <- x + ffn(layer_norm(x, norm2))

Mixers: ``mamba2`` (a selective state space per head behind a short convolution), ``latent_attention`` (queries
through a normed latent, keys and values from one cached latent plus one shared rotated key part, a sliding window)
and ``parallel`` (softmax attention over a window that also keeps a sequence's first tokens, beside a gated delta
rule, their results summed with two constants). The feed-forward is a mixture of gated experts, some of which are
identities.
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
def layer_norm(x, gain, eps):
    mean = x.mean(-1, keepdim=True)
    dev = x - mean
    return dev / torch.sqrt((dev * dev).mean(-1, keepdim=True) + eps) * gain


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def short_convolution(u, taps, bias=None):
    """u [T, C], taps [C, K]: out[t, c] = sum_j taps[c, j] * u[t - (K - 1) + j, c] with zeros before the start
    (the last column multiplies the current token)."""
    T, C = u.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u], dim=0)
    out = torch.zeros_like(u)
    for j in range(K):
        out = out + padded[j:j + T] * taps[:, j]
    if bias is not None:
        out = out + bias
    return out


# --------------------------------------------------------------------------- rotations
def plain_frequencies(base, dims):
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def yarn_frequencies(base, dims, sc):
    """Frequencies stretched by YaRN and the factor that multiplies cos and sin."""
    def turn(t):
        return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(turn(sc["fast"])), 0)
    hi = min(math.ceil(turn(sc["slow"])), dims - 1)
    out = []
    for i, f in enumerate(plain_frequencies(base, dims)):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / sc["factor"] * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate(v, positions, freqs, dims, interleaved, magnitude=1.0):
    """v [T, heads, n]: rotate the first ``dims`` features by position * f_i. interleaved: feature 2i pairs with
    2i + 1; otherwise i pairs with i + dims / 2. (u, w) -> (u cos - w sin, w cos + u sin), cos and sin times
    ``magnitude``."""
    f = torch.tensor(freqs, dtype=v.dtype)
    angle = positions.to(v.dtype)[:, None] * f[None, :]                      # [T, dims / 2]
    cos, sin = (torch.cos(angle) * magnitude)[:, None, :], (torch.sin(angle) * magnitude)[:, None, :]
    out = v.clone()
    if interleaved:
        a, b = v[..., 0:dims:2], v[..., 1:dims:2]
        out[..., 0:dims:2] = a * cos - b * sin
        out[..., 1:dims:2] = b * cos + a * sin
    else:
        half = dims // 2
        a, b = v[..., :half], v[..., half:dims]
        out[..., :half] = a * cos - b * sin
        out[..., half:dims] = b * cos + a * sin
    return out


def masked_softmax_attention(q, k, v, scale, visible):
    """q [T, H, dk], k [T, H, dk], v [T, H, dv], visible [T, T] bool (query row, key column) -> [T, H, dv]."""
    scores = torch.einsum("thd,shd->hts", q, k) * scale
    scores = scores.masked_fill(~visible[None], -math.inf)
    return torch.einsum("hts,shd->thd", torch.softmax(scores, dim=-1), v)


# --------------------------------------------------------------------------- mixers
def mamba2(h, w, p, m, eps):
    """The state-space mixer. Returns [T, d]."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_convolution(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])                                     # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)                       # [T, H]
    group_of = [hh // (H // G) for hh in range(H)]
    S = torch.zeros(H, N, P, dtype=h.dtype)
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for t in range(T):
        for hh in range(H):
            g = group_of[hh]
            S[hh] = decay[t, hh] * S[hh] + dt[t, hh] * torch.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ C[t, g] + w[p + "D"][hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def latent_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(T)
    cq = unit_rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, dn + dr)
    down = h @ w[p + "dkv"].T
    c = unit_rms(down[:, :rank], eps) * w[p + "dkv.norm"]
    shared = down[:, rank:].reshape(T, 1, dr)
    rot = m["rot"]
    if rot.get("scaling"):
        freqs, magnitude = yarn_frequencies(rot["base"], rot["dims"], rot["scaling"])
    else:
        freqs, magnitude = plain_frequencies(rot["base"], rot["dims"]), 1.0
    q_rot = rotate(q[..., dn:], positions, freqs, rot["dims"], True, magnitude)
    k_rot = rotate(shared, positions, freqs, rot["dims"], True, magnitude).expand(T, H, dr)
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    gap = positions[:, None] - positions[None, :]
    visible = gap >= 0
    if m.get("mask") and m["mask"].get("size") is not None:
        visible = visible & (gap < m["mask"]["size"])
    o = masked_softmax_attention(torch.cat([q[..., :dn], q_rot], -1), torch.cat([k_plain, k_rot], -1), v, m["scale"], visible)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def kept_window_attention(h, w, p, m):
    """The left half of a parallel mixer: grouped softmax attention with biases, rotate-half rotation, a window that
    also keeps the first ``keep_first`` tokens."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T)
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, dk)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, dk)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    rot = m.get("rot")
    if rot and rot["dims"] > 0:
        freqs = plain_frequencies(rot["base"], rot["dims"])
        q = rotate(q, positions, freqs, rot["dims"], False)
        k = rotate(k, positions, freqs, rot["dims"], False)
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    gap = positions[:, None] - positions[None, :]
    visible = gap >= 0
    mask = m.get("mask")
    if mask and mask.get("size") is not None:
        visible = visible & ((gap < mask["size"]) | (positions[None, :] < mask.get("keep_first", 0)))
    o = masked_softmax_attention(q, k, v, m["scale"], visible)
    return o.reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"]


def gated_delta_rule(h, w, p, m, eps):
    """The right half of a parallel mixer."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, dk)
    k = silu(short_convolution(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, dk)
    v = silu(short_convolution(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                              # [T, H]
    g = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))   # [T, H]
    S = torch.zeros(H, dk, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        for hh in range(H):
            kk, qq = k[t, hh // (H // G)], q[t, hh // (H // G)]
            S[hh] = g[t, hh] * S[hh]
            u = beta[t, hh] * (v[t, hh] - S[hh].T @ kk)
            S[hh] = S[hh] + torch.outer(kk, u)
            o[t, hh] = S[hh].T @ qq
    o = unit_rms(o, eps) * w[p + "norm"] * silu(h @ w[p + "g"].T).reshape(T, H, dv)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    return (m["left_scale"] * kept_window_attention(h, w, p + "left.", m["left"])
            + m["right_scale"] * gated_delta_rule(h, w, p + "right.", m["right"], eps))


# --------------------------------------------------------------------------- feed-forward
def route(scores, correction, r):
    """scores [T, E] (softmax over all router outputs) -> (chosen [T, top], weights [T, top], smallest deciding gap).
    The choice is made on scores + correction, inside the best ``keep`` of ``count`` groups of neighbours (a group's
    score is its largest choice score); the weights are the chosen scores themselves times ``scale``."""
    T, E = scores.shape
    choice = scores + correction
    gap = math.inf
    groups = r.get("groups")
    if groups and groups["count"] > 1:
        per = E // groups["count"]
        best = choice.reshape(T, groups["count"], per).max(-1).values
        ranked = best.sort(dim=-1, descending=True)
        if groups["keep"] < groups["count"]:
            gap = min(gap, float((ranked.values[:, groups["keep"] - 1] - ranked.values[:, groups["keep"]]).min()))
        allowed = torch.zeros(T, groups["count"], dtype=torch.bool)
        allowed.scatter_(1, ranked.indices[:, :groups["keep"]], True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    ranked = choice.sort(dim=-1, descending=True)
    top = r["top"]
    if top < E:
        rest = ranked.values[:, top]
        finite = torch.isfinite(rest)
        if finite.any():
            gap = min(gap, float((ranked.values[:, top - 1] - rest)[finite].min()))
    chosen = ranked.indices[:, :top]
    return chosen, scores.gather(1, chosen) * r["scale"], gap


def mixture_ffn(h, w, p, mlp, gaps=None):
    r = mlp["router"]
    real, ident = r["experts"], r.get("identity", 0)
    scores = torch.softmax(h @ w[p + "router"].T, dim=-1)
    chosen, weights, gap = route(scores, w[p + "correction"], r)
    if gaps is not None:
        gaps.append(gap)
    out = torch.zeros_like(h)
    for e in range(real + ident):
        for slot in range(r["top"]):
            rows = (chosen[:, slot] == e).nonzero().flatten()
            if not rows.numel():
                continue
            hr = h[rows]
            if e < real:
                q = f"{p}e{e}."
                hr = (silu(hr @ w[q + "gate"].T) * (hr @ w[q + "up"].T)) @ w[q + "down"].T
            out[rows] += weights[rows, slot][:, None] * hr
    return out


# --------------------------------------------------------------------------- the model
def forward(cfg, w, tokens, dtype=torch.float64, rows=None, streams=None, gaps=None):
    """Logits [T (or len(rows)), vocab] of a whole sequence. ``streams``: a list that receives the stream after
    every layer; ``gaps``: a list that receives the smallest deciding gap of every routing."""
    w = {k: v.to(dtype) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg.get("embedding", {}).get("scale", 1.0)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = layer_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "mamba2":
            y = mamba2(h, w, p + "mix.", m, eps)
        elif layer["type"] == "latent_attention":
            y = latent_attention(h, w, p + "mix.", m, eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + y
        if layer["mlp"] is not None:
            x = x + mixture_ffn(layer_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"], gaps)
        if streams is not None:
            streams.append(x.clone())
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long)]
    return layer_norm(x, w["final.norm"], eps) @ w["head"].T * cfg.get("logit_scale", 1.0)
