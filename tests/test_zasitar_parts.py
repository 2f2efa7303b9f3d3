"""Each mechanism of the Zasitar decoder alone, its kernels against the plain implementation's function:
the norm behind a sublayer with an additive vector and a layer scale, the gated tanh-GELU with additive vectors, the
clamped experts' activation, routing by the largest logits with a softmax over the chosen, queries and keys normed
per head with a shared gain and rotated in split halves over part of a head, sliding-window attention with one more
term in the softmax's denominator (prompts and decoding; a key that stands out just inside and just outside the
window, at page borders, far back), and time mixing (blends with the previous token across steps and slots, the
double-exponential decay, the recurrence with a bonus over steps, slots and chunks, the per-head unit norm)."""
import math

import pytest
import torch

import plain_zasitar as P
from helpers import check_error

pytestmark = pytest.mark.gpu
PAGE = 64


def rel(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all()
    return float((got - ref).abs().max() / ref.abs().max())


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


def scratch(name, shape, dtype):
    return torch.empty(shape, dtype=dtype, device="cuda")


# --------------------------------------------------------------------------- small kernels
@pytest.mark.parametrize("rows,d", [(1, 8), (5, 72), (3, 1000), (2, 4100)])
def test_norm_behind_a_sublayer_with_vector_and_layer_scale(rows, d):
    """x += ls * rms_norm(y + b, w): the additive vector must enter the mean square, the layer scale must not."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(d)
    y, x = (torch.randn(rows, d) * 3).cuda(), torch.randn(rows, d).cuda()
    w, ls, b = (1 + 0.3 * torch.randn(d)).cuda(), (0.2 + torch.rand(d)).cuda(), (2.0 * torch.randn(d)).cuda()
    ref = x.double().cpu() + P.rms_norm(y.double().cpu() + b.double().cpu(), w.double().cpu(), 1e-5) * ls.double().cpu()
    got = x.clone()
    ops.post_norm_add(y, w, 1e-5, got, y_bias=b, scale=ls)
    check_error("post norm + vector + layer scale, float32", f"{rows}x{d}", rel(got, ref), 2e-6)
    for dtype, lim in ((torch.float32, 0.0), (torch.bfloat16, 4e-3)):
        again, copy = x.clone(), torch.empty(rows, d, device="cuda", dtype=dtype)
        ops.post_norm_add(y, w, 1e-5, again, y_bias=b, scale=ls, next_out=copy)     # the new stream once more, as it is
        assert torch.equal(again, got) and rel(copy, got) <= lim
    wrong = x.clone()
    ops.post_norm_add(y + b, w * ls, 1e-5, wrong)            # the same thing by other means
    assert rel(wrong, ref) < 3e-6
    plain = x.clone()
    ops.post_norm_add(y, w, 1e-5, plain, scale=ls)           # without the vector the result differs visibly
    assert rel(plain, ref) > 1e-2


@pytest.mark.parametrize("T,F", [(1, 8), (7, 104), (33, 257)])
def test_gated_tanh_gelu(T, F):
    from llmplayer_b200.kernels import ops
    torch.manual_seed(F)
    wide = (2.5 * torch.randn(T, 2 * F + 16)).cuda()
    z = wide[:, 8:8 + 2 * F]                                  # a column slice of a wider buffer
    bias = torch.randn(2 * F).cuda()
    full = z.double().cpu() + bias.double().cpu()
    ref = P.gelu_tanh(full[:, :F]) * full[:, F:]
    for dtype, lim in ((torch.float32, 2e-6), (torch.bfloat16, 5e-3)):
        out = torch.empty(T, F, device="cuda", dtype=dtype)
        ops.gated_act(z, bias, out, "gelu_tanh")
        check_error(f"gated tanh-GELU, {dtype}", f"{T}x{F}", rel(out, ref), lim)
    none = torch.empty(T, F, device="cuda")
    ops.gated_act(z, None, none, "gelu_tanh")
    assert rel(none, P.gelu_tanh(z.double().cpu()[:, :F]) * z.double().cpu()[:, F:]) < 2e-6
    # the erf form of GELU is another function: the kernel must be told apart from it
    erf = torch.nn.functional.gelu(full[:, :F]) * full[:, F:]
    exact = torch.empty(T, F, device="cuda")
    ops.gated_act(z, bias, exact, "gelu_tanh")
    assert float((erf - ref).abs().max()) > 20 * float((exact.double().cpu() - ref).abs().max())


@pytest.mark.parametrize("E,ff,rest,limit,limit_rest", [(6, 24, 40, 1.5, 0.75), (4, 16, 0, 3.0, 0.0), (3, 12, 20, 0.5, 1.25), (1, 8, 8, 1.0, 2.0),
                                                        (2, 6, 10, 2.5, 1.0)])
def test_clamped_expert_activation(E, ff, rest, limit, limit_rest):
    """Sums well beyond the limits: min on the gate only from above, the up sum from both sides, (u + 1), and the
    constant 1.702; the last columns belong to an expert with a limit and a weight column of its own."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(E * ff)
    T, total = 11, E * ff + rest
    z = (3.0 * torch.randn(T, 2 * total)).cuda()
    weights = (torch.rand(T, E + (1 if rest else 0)) * (torch.rand(T, E + (1 if rest else 0)) > 0.4)).cuda()
    zd, wd = z.double().cpu(), weights.double().cpu()
    g, u = zd[:, :total], zd[:, total:]
    lim = torch.cat([torch.full((E * ff,), limit), torch.full((rest,), limit_rest)]).double()
    gc, uc = torch.minimum(g, lim), torch.maximum(torch.minimum(u, lim), -lim)
    per_column = torch.cat([wd[:, :E].repeat_interleave(ff, dim=1)] + ([wd[:, E:].expand(T, rest)] if rest else []), dim=1)
    ref = gc * torch.sigmoid(1.702 * gc) * (uc + 1.0) * per_column
    for dtype, bound in ((torch.float32, 2e-6), (torch.bfloat16, 5e-3)):
        hidden = torch.empty(T, total, device="cuda", dtype=dtype)
        ops.expert_act(z, weights, hidden, num_experts=E, expert_size=ff, limit=limit, limit_rest=limit_rest)
        check_error(f"clamped experts, {dtype}", f"{E} x {ff} + {rest}", rel(hidden, ref), bound)
    assert float(g.min()) < -limit and float(g.max()) > limit and float(u.min()) < -limit      # the clamps were at work
    # against the plain expert as a whole, one expert and no weights
    h = torch.randn(T, 10, dtype=torch.float64)
    w = {"gate": torch.randn(ff, 10, dtype=torch.float64), "up": torch.randn(ff, 10, dtype=torch.float64),
         "down": torch.randn(10, ff, dtype=torch.float64)}
    sums = torch.cat([h @ w["gate"].T, h @ w["up"].T], dim=1).float().cuda()
    hidden = torch.empty(T, ff, device="cuda")
    ops.expert_act(sums, None, hidden, num_experts=1, expert_size=ff, limit=limit)
    assert rel(hidden.double().cpu() @ w["down"].T, P.clamped_expert(h, w, "", limit)) < 3e-6


@pytest.mark.parametrize("E,top,extra", [(6, 2, 1), (4, 1, 0), (8, 3, 1), (3, 3, 1), (16, 4, 1), (64, 6, 0), (2, 1, 2)])
def test_routing_by_the_largest_logits(E, top, extra):
    """The ``top`` largest of logits + vector, weights = softmax over the chosen alone; further columns are gates of
    experts that every token uses (a sigmoid each). The vector decides: without it other experts would win."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(E + top)
    T = 300
    wide = (2.0 * torch.randn(T, E + extra + 5)).cuda()
    logits = wide[:, 3:3 + E + extra]
    bias = (1.5 * torch.randn(E)).cuda()
    weights = torch.full((T, E + extra), 9.0, device="cuda")
    ops.route_top(logits, bias, weights, num_experts=E, top=top)
    full = logits.double().cpu()[:, :E] + bias.double().cpu()
    chosen, w, _ = P.route(full, top)
    ref = torch.zeros(T, E, dtype=torch.float64).scatter_(1, chosen, w)
    clear = torch.tensor([P.route(full[t:t + 1], top)[2] > 1e-5 for t in range(T)])
    assert int(clear.sum()) > T - 5
    assert rel(weights[:, :E][clear.cuda()], ref[clear]) < 2e-6
    assert int((weights[:, :E] > 0).sum(-1).min()) == int((weights[:, :E] > 0).sum(-1).max()) == top
    assert float((weights[:, :E].sum(-1) - 1).abs().max()) < 1e-5
    if extra:
        assert rel(weights[:, E:], torch.sigmoid(logits.double().cpu()[:, E:])) < 2e-6
    if top < E:
        without, _, _ = P.route(logits.double().cpu()[:, :E], top)
        assert int((without.sort(-1).values != chosen.sort(-1).values).any(-1).sum()) > T // 10


# --------------------------------------------------------------------------- queries, keys, values
@pytest.mark.parametrize("H,G,dk,dv,rd,scaling", [
    (4, 2, 24, 40, 16, None), (8, 1, 64, 64, 32, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}),
    (5, 1, 10, 12, 2, None), (2, 2, 128, 64, 128, None), (3, 3, 16, 16, 16, {"factor": 3.0, "low": 2.0, "high": 6.0, "original": 96}),
    (2, 2, 12, 6, 0, None)])
def test_queries_and_keys_normed_then_rotated(H, G, dk, dv, rd, scaling):
    """Additive vectors, then the RMS norm of every head with ONE gain shared by the heads, then the rotation in split
    halves over the first ``rd`` features with stretched frequencies; values get their vector only. Positions on both
    sides of page borders and far out; heads padded with zeros to the stored size. Then queries alone (a layer that
    attends over another layer's keys): the pages stay as they were."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(H * dk + rd)
    eps = 1e-5
    hdp = -(-max(dk, dv) // 16) * 16
    positions = [0, 1, 63, 64, 65, 130, 1000]
    T = len(positions)
    F = (H + G) * dk + G * dv
    qkv, bias = torch.randn(T, F).cuda(), (0.5 * torch.randn(F)).cuda()
    q_gain, k_gain = (1 + 0.4 * torch.randn(dk)).cuda(), (1 + 0.4 * torch.randn(dk)).cuda()
    rot = {"base": 10000.0, "dims": rd, "scaling": scaling}
    freq = torch.tensor(P.rotary_frequencies(rot), dtype=torch.float64).float().cuda() if rd else None
    rotation = ops.Rotation(freq, rd, False) if rd else ops.NO_ROTATION
    pages = torch.full((20, 2, G, PAGE, hdp), 7.0, device="cuda")
    table = i32([[3, 9, 1] + [0] * 13])                   # positions 0..191 in pages 3, 9, 1; position 1000 in page 0
    q_out = torch.full((T, H * hdp), 7.0, device="cuda")
    ops.qkv_prepare(qkv, bias, rotation, i32(positions), i32([0] * T), table, q_out, pages, num_heads=H, num_kv_heads=G,
                    key_dim=dk, value_dim=dv, unit_norm_eps=None, q_gain=q_gain, k_gain=k_gain, gain_eps=eps)
    full = qkv.double().cpu() + bias.double().cpu()
    pos = torch.tensor(positions)
    q = P.rotate_split_halves(P.rms_norm(full[:, :H * dk].view(T, H, dk), q_gain.double().cpu(), eps), pos, rot)
    k = P.rotate_split_halves(P.rms_norm(full[:, H * dk:(H + G) * dk].view(T, G, dk), k_gain.double().cpu(), eps), pos, rot)
    v = full[:, (H + G) * dk:].view(T, G, dv)
    got_q = q_out.view(T, H, hdp)
    # the angle position * frequency is a float32 product: at position 1000 its rounding alone is worth 1e-5
    check_error("normed and rotated queries", f"{H}x{dk}, rotation over {rd}", rel(got_q[:, :, :dk], q), 3e-5)
    assert hdp == dk or float(got_q[:, :, dk:].abs().max()) == 0.0
    for t, p in enumerate(positions):
        page = [3, 9, 1][p // PAGE] if p < 192 else 0
        got_k, got_v = pages[page, 0, :, p % PAGE], pages[page, 1, :, p % PAGE]
        assert rel(got_k[:, :dk], k[t]) < 3e-5 and rel(got_v[:, :dv], v[t]) < 1e-6
        assert float(got_k[:, dk:].abs().sum()) == 0.0 and float(got_v[:, dv:].abs().sum()) == 0.0
    assert float((pages[2] - 7.0).abs().max()) == 0.0     # a page of nobody's stays untouched
    if rd and rd < dk:                                     # features beyond the rotation pass unchanged by position
        unrotated = P.rms_norm(full[:, :H * dk].view(T, H, dk), q_gain.double().cpu(), eps)
        assert rel(got_q[:, :, rd:dk], unrotated[:, :, rd:]) < 2e-6 and rel(got_q[-1:, :, :rd], unrotated[-1:, :, :rd]) > 1e-2
    # queries alone
    before = pages.clone()
    alone = torch.full((T, H * hdp), 7.0, device="cuda")
    ops.qkv_prepare(qkv[:, :H * dk].contiguous(), bias[:H * dk].contiguous(), rotation, i32(positions), i32([0] * T), table, alone,
                    pages, num_heads=H, num_kv_heads=G, key_dim=dk, value_dim=dv, unit_norm_eps=None, q_gain=q_gain,
                    gain_eps=eps, write_kv=False)
    assert torch.equal(alone, q_out) and torch.equal(pages, before)


# --------------------------------------------------------------------------- windowed attention with one more term
def fill_pages(k, v, table_rows, num_pages, dtype):
    """k, v: [T, G, hd] of ONE sequence -> pages [num_pages, 2, G, 64, hd] laid out through ``table_rows``."""
    T, G, hd = k.shape
    pages = torch.zeros(num_pages, 2, G, PAGE, hd, dtype=dtype, device="cuda")
    for t in range(T):
        page = table_rows[t // PAGE]
        pages[page, 0, :, t % PAGE] = k[t].to(dtype)
        pages[page, 1, :, t % PAGE] = v[t].to(dtype)
    return pages


def plain_window_attention(q, k, v, scale, window, first_query):
    """q [Tq, H, hd] at positions first_query.., k / v [Tk, G, hd] at positions 0..: the plain sliding window with the
    softmax whose denominator holds one more term."""
    Tq, H, hd = q.shape
    G = k.shape[1]
    out = torch.zeros(Tq, H, v.shape[2], dtype=torch.float64)
    gap = torch.arange(first_query, first_query + Tq)[:, None] - torch.arange(k.shape[0])[None, :]
    seen = (gap >= 0) & (gap < window)
    for h in range(H):
        g = h // (H // G)
        s = ((q[:, h] @ k[:, g].T) * scale).masked_fill(~seen, -math.inf)
        out[:, h] = P.softmax_plus_one(s) @ v[:, g]
    return out


def run_attention(kind, dtype, qd, pages, table, length, new, window, H, G, hd, scale, sink=True, exact=True):
    from llmplayer_b200.kernels import ops
    out = torch.empty_like(qd)
    sinks = torch.zeros(H, device="cuda") if sink else None
    if kind == "plain":
        ops.attention_plain(qd, out, pages, table, i32([0] * new), i32(list(range(length - new, length))), num_heads=H,
                            num_kv_heads=G, head_dim=hd, scale=scale, window=window, sinks=sinks)
    elif kind == "prompt":
        ops.attention_prefill(qd, out, pages, table, i32([0, new]), i32([length]), new, num_heads=H, num_kv_heads=G,
                              head_dim=hd, scale=scale, window=window, sinks=sinks, exact_weights=exact)
    else:
        ops.attention_decode(qd, out, pages, table, i32([length]), scratch, num_heads=H, num_kv_heads=G, head_dim=hd,
                             scale=scale, window=window, sinks=sinks, exact_weights=exact)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,length,new,window", [(4, 2, 48, 200, 200, 9), (8, 1, 64, 321, 321, 70), (2, 2, 128, 150, 57, 128),
                                                      (6, 2, 96, 700, 700, 33), (3, 3, 16, 65, 2, 1000), (5, 1, 16, 130, 130, 1),
                                                      (2, 1, 64, 400, 300, 64), (2, 2, 64, 260, 260, 65)])
def test_prompt_attention_in_a_window(dtype, H, G, hd, length, new, window):
    """The last ``new`` tokens of a sequence of ``length`` attend over their windows (pages in a scrambled order):
    the plain kernel in float32, the tensor-core prompt kernel in bfloat16. Small scores, so that the one more term
    in the denominator holds a good part of the weight; without it, and with the window one token wider or
    narrower, the result differs visibly."""
    torch.manual_seed(length + hd)
    scale = 0.3
    q = torch.randn(new, H, hd).to(dtype)
    k, v = torch.randn(length, G, hd).to(dtype), torch.randn(length, G, hd).to(dtype)
    rows = list(torch.randperm(16).tolist())[:-(-length // PAGE)]
    pages = fill_pages(k, v, rows, 16, dtype)
    ref = plain_window_attention(q.double(), k.double(), v.double(), scale, window, length - new)
    qd = q.reshape(new, H * hd).cuda()
    table = i32([rows + [0] * (16 - len(rows))])
    kind, lim = ("plain", 3e-6) if dtype == torch.float32 else ("prompt", 6e-3)
    out = run_attention(kind, dtype, qd, pages, table, length, new, window, H, G, hd, scale)
    check_error(f"windowed attention over a prompt, {dtype}", f"{H}/{G} x {hd}, {new} of {length}, window {window}",
                rel(out.view(new, H, hd), ref), lim)
    if dtype == torch.bfloat16:
        rough = run_attention(kind, dtype, qd, pages, table, length, new, window, H, G, hd, scale, exact=False)
        check_error("windowed attention over a prompt, bfloat16 weights", f"{H}/{G} x {hd}, window {window}",
                    rel(rough.view(new, H, hd), ref), 1.5e-2)
    no_sink = run_attention(kind, dtype, qd, pages, table, length, new, window, H, G, hd, scale, sink=False)
    if dtype == torch.float32:
        assert rel(no_sink, out) > 5e-5
    if window > 40:            # among many keys one term more or one key more changes little: the narrow windows show it
        return
    assert rel(no_sink.view(new, H, hd), ref) > 2e-2
    for other in (window - 1, window + 1):
        if 0 < other and min(window, other) < length:
            off = run_attention(kind, dtype, qd, pages, table, length, new, other, H, G, hd, scale)
            assert rel(off.view(new, H, hd), ref) > 2e-2, other


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("step", ["prompt", "decode"])
@pytest.mark.parametrize("length,window", [(700, 70), (700, 64), (700, 65), (700, 128), (700, 129), (300, 33), (200, 9), (130, 2),
                                           (130, 1), (700, 637), (700, 700), (700, 5000)])
def test_a_key_at_the_window_s_edge(dtype, step, length, window):
    """Head 1's query is made to fit ONE key far better than all others. Placed on the last position inside the
    window (gap = window - 1) its value must come through nearly alone; placed one further back (gap = window) it must
    not be seen at all. The last query is checked, in a prompt step of 40 tokens and in a one-token step; the edge
    falls before, on and behind page borders."""
    torch.manual_seed(window)
    H, G, hd, scale = 4, 2, 64, 0.5
    new = 40 if step == "prompt" else 1
    direction = torch.randn(hd)
    direction /= direction.norm()
    last = length - 1
    for gap in (window - 1, window):
        at = last - gap
        k, v = 0.3 * torch.randn(length, G, hd), torch.randn(length, G, hd)
        q = 0.3 * torch.randn(new, H, hd)
        q[-1, 1] = 8.0 * direction
        if at >= 0:
            k[at, 0] = 8.0 * direction                     # score 64 * 0.5 = 32 against scores near 0
        k, v, q = k.to(dtype), v.to(dtype), q.to(dtype)
        rows = torch.randperm(16).tolist()[:-(-length // PAGE)]
        pages = fill_pages(k, v, rows, 16, dtype)
        table = i32([rows + [0] * (16 - len(rows))])
        qd = q.reshape(new, H * hd).cuda()
        kind = "plain" if dtype == torch.float32 else step
        out = run_attention(kind, dtype, qd, pages, table, length, new, window, H, G, hd, scale).view(new, H, hd)
        ref = plain_window_attention(q.double(), k.double(), v.double(), scale, window, length - new)
        check_error(f"windowed attention, a key at gap {'window - 1' if gap < window else 'window'}, {step}, {dtype}",
                    f"length {length}, window {window}", rel(out, ref), 3e-6 if dtype == torch.float32 else 6e-3)
        got = out[-1, 1].double().cpu()
        if at < 0:
            continue
        if gap < window:
            assert float((got - v[at, 0].double()).abs().max()) < 1e-3 + (0.02 if dtype == torch.bfloat16 else 0.0)
        else:
            assert float((got - v[at, 0].double()).abs().max()) > 0.5


@pytest.mark.parametrize("shares", [(1, 16), (4, 4), (8, 2)])
def test_decode_attention_in_shares_counts_the_extra_term_once(shares):
    """The same decode step cut into 1, 4 and 8 shares of pages, with and without a window: the one more term of the
    denominator is counted once, whatever the cut; two sequences of unequal lengths in the batch."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(5)
    H, G, hd = 6, 2, 96
    num, per = shares
    lengths = [1000, 37]
    k = [torch.randn(n, G, hd).bfloat16() for n in lengths]
    v = [torch.randn(n, G, hd).bfloat16() for n in lengths]
    q = torch.randn(2, H, hd).bfloat16()
    perm = torch.randperm(20).tolist()
    rows = [perm[:16], perm[16:17] + [0] * 15]
    pages = fill_pages(k[0], v[0], rows[0], 20, torch.bfloat16) + fill_pages(k[1], v[1], rows[1], 20, torch.bfloat16)
    qd = q.reshape(2, H * hd).cuda()
    for window in (None, 300, 50):
        out = torch.empty_like(qd)
        ops.attention_decode(qd, out, pages, i32(rows), i32(lengths), scratch, num_heads=H, num_kv_heads=G, head_dim=hd,
                             scale=0.1, window=window, sinks=torch.zeros(H, device="cuda"), pages_per_split=per,
                             num_splits=num, exact_weights=True)
        for b, n in enumerate(lengths):
            ref = plain_window_attention(q[b:b + 1].double(), k[b].double(), v[b].double(), 0.1, window or 10 ** 6, n - 1)
            check_error("windowed decode attention, bfloat16", f"{num} shares, window {window}, sequence {b}",
                        rel(out.view(2, H, hd)[b:b + 1], ref), 6e-3)


# --------------------------------------------------------------------------- time mixing
def time_mix_weights(H, n, d, rank, seed):
    g = torch.Generator().manual_seed(seed)
    C = H * n
    w = {name: 0.3 * torch.randn(C, d, generator=g, dtype=torch.float64) for name in ("r", "k", "v", "g")}
    w.update({"mu." + b: torch.rand(d, generator=g, dtype=torch.float64) for b in "rkvgw"})
    w["w1"] = 0.3 * torch.randn(rank, d, generator=g, dtype=torch.float64)
    w["w2"] = 0.5 * torch.randn(C, rank, generator=g, dtype=torch.float64)
    w["w0"] = -2.0 + 1.5 * torch.randn(C, generator=g, dtype=torch.float64)      # decays from nearly 1 to nearly 0
    w["u"] = 0.5 + torch.rand(H, n, generator=g, dtype=torch.float64)
    w["norm"] = 1 + 0.2 * torch.randn(C, generator=g, dtype=torch.float64)
    w["o"] = 0.3 * torch.randn(d, C, generator=g, dtype=torch.float64)
    return w


def run_time_mix_kernels(x, w, H, n, eps, state, last, slots, q_start, max_new):
    """The mixer's kernels on the step's float32 inputs ``x`` [T, d]: the blends, then (projections formed here in
    float64 from the kernel's blends, so that only the mixer's own kernels are under test) the decay, the recurrence
    and the per-head norm with the gate; returns the heads [T, H * n] before the output projection."""
    from llmplayer_b200.kernels import ops
    T, d = x.shape
    C = H * n
    seq_ids = [b for b in range(len(slots)) for _ in range(q_start[b + 1] - q_start[b])]
    mu = torch.stack([w["mu." + b] for b in "rkvgw"]).float().cuda()
    blends = torch.empty(5, T, d, device="cuda")
    ops.token_shift(x.float().cuda(), last, mu, i32(slots), i32(q_start), i32(seq_ids), blends)
    b = blends.double().cpu()
    rank = w["w1"].shape[0]
    proj = torch.cat([b[0] @ w["r"].T, b[1] @ w["k"].T, b[2] @ w["v"].T, b[3] @ w["g"].T, b[4] @ w["w1"].T], dim=1).float().cuda()
    decay = torch.empty(T, C, device="cuda")
    ops.gla_decay(proj[:, 4 * C:4 * C + rank], w["w2"].float().cuda(), w["w0"].float().cuda(), decay, double_exp=True)
    raw = torch.empty(T, C, device="cuda")
    ops.gla_scan(proj, 0, C, 2 * C, decay, state, i32(slots), i32(q_start), raw, num_heads=H, key_dim=n, value_dim=n,
                 q_scale=1.0, max_new=max_new, scratch=scratch, bonus=w["u"].float().cuda())
    out = torch.empty(T, C, device="cuda")
    ops.gla_finish(raw, w["norm"].float().cuda(), eps, proj[:, 3 * C:4 * C], out, num_heads=H, value_dim=n, gain_per_head=True)
    return out, blends, decay


@pytest.mark.parametrize("d", [52, 50, 1028, 2048])
def test_blends_with_the_previous_token(d):
    """Two sequences in slots 3 and 1 of five over three steps: before a sequence's first token stands a row of
    zeros, before the first token of a later step the last token of the step before; the other slots stay untouched.
    Rows of a multiple of four values (four features per thread) and others; a buffer cleared on the side."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(11)
    seqs = [torch.randn(9, d), torch.randn(5, d)]
    mu = torch.rand(5, d)
    last = torch.zeros(5, d, device="cuda")
    last[[0, 2, 4]] = 7.0
    at = [0, 0]
    for a, b in [(4, 1), (1, 1), (4, 3)]:
        x = torch.cat([seqs[0][at[0]:at[0] + a], seqs[1][at[1]:at[1] + b]])
        out = torch.empty(5, a + b, d, device="cuda")
        side = torch.full((1000,), 3.0, device="cuda")
        ops.token_shift(x.cuda(), last, mu.cuda(), i32([3, 1]), i32([0, a, a + b]), i32([0] * a + [1] * b), out, clear=side[:777])
        assert float(side[:777].abs().max()) == 0.0 and float((side[777:] - 3.0).abs().max()) == 0.0
        for s, (seq, lo, cnt, off) in enumerate(((seqs[0], at[0], a, 0), (seqs[1], at[1], b, a))):
            full = torch.cat([torch.zeros(1, d), seq]).double()
            cur, prev = full[1 + lo:1 + lo + cnt], full[lo:lo + cnt]
            ref = cur[None] + (prev - cur)[None] * mu.double()[:, None, :]
            assert rel(out[:, off:off + cnt], ref) < 1e-6, (s, lo)
        at = [at[0] + a, at[1] + b]
        assert torch.equal(last[3].cpu(), seqs[0][at[0] - 1]) and torch.equal(last[1].cpu(), seqs[1][at[1] - 1])
    assert float((last[[0, 2, 4]] - 7.0).abs().max()) == 0.0
    half = torch.empty(5, 4, d, device="cuda", dtype=torch.bfloat16)
    ops.token_shift(seqs[0][:4].cuda(), torch.zeros(5, d, device="cuda"), mu.cuda(), i32([0]), i32([0, 4]), i32([0] * 4), half)
    full = torch.cat([torch.zeros(1, d), seqs[0][:4]]).double()
    assert rel(half, full[1:][None] + (full[:-1] - full[1:])[None] * mu.double()[:, None, :]) < 5e-3


def test_double_exponential_decay():
    from llmplayer_b200.kernels import ops
    torch.manual_seed(4)
    T, C, R = 17, 60, 13
    wide = (1.5 * torch.randn(T, R + 11)).cuda()
    low = wide[:, 8:8 + R]
    up, bias = (0.8 * torch.randn(C, R)).cuda(), (-1.0 + 2.0 * torch.randn(C)).cuda()
    out = torch.empty(T, C, device="cuda")
    ops.gla_decay(low, up, bias, out, double_exp=True)
    ref = torch.exp(-torch.exp(torch.tanh(low.double().cpu()) @ up.double().cpu().T + bias.double().cpu()))
    assert float((out.double().cpu() - ref).abs().max()) < 2e-6
    assert float(ref.min()) < 0.05 and float(ref.max()) > 0.95 and float(out.min()) >= 0.0 and float(out.max()) <= 1.0


@pytest.mark.parametrize("H,n,rank", [(3, 20, 7), (1, 36, 16), (2, 64, 32), (2, 6, 3), (5, 16, 8)])
def test_time_mixing_over_steps_and_slots(H, n, rank):
    """Two sequences in slots 2 and 0 of four: a prompt each (one of 300 tokens: chunks side by side), then portions
    and single tokens; every output against the plain recurrence over the whole sequence; the untouched slots stay
    zero; state and previous input end as the plain ones do."""
    d, eps = 40, 1e-5
    w = time_mix_weights(H, n, d, rank, seed=H * n)
    m = {"heads": H, "dim": n}
    wp = {"mix." + name: t for name, t in w.items()}
    torch.manual_seed(n)
    # inputs as the library's stream holds them: float32 values
    seq = [torch.randn(420, d).double(), torch.randn(60, d).double()]
    full = [P.wkv(s, wp, "mix.", m, eps) for s in seq]
    state, last = torch.zeros(4, H, n, n, device="cuda"), torch.zeros(4, d, device="cuda")
    slots = [2, 0]
    cuts = [(300, 7), (2, 1), (117, 51), (1, 1)]           # new tokens of the two sequences, step by step
    at = [0, 0]
    got = [[], []]
    for a, b in cuts:
        x = torch.cat([seq[0][at[0]:at[0] + a], seq[1][at[1]:at[1] + b]])
        out, _, _ = run_time_mix_kernels(x, w, H, n, eps, state, last, slots, [0, a, a + b], max(a, b))
        got[0].append(out[:a])
        got[1].append(out[a:])
        at = [at[0] + a, at[1] + b]
    for s in range(2):
        heads = torch.cat(got[s]).double().cpu() @ w["o"].T
        check_error("time mixing, float32", f"{H} x {n}, sequence {s}", rel(heads, full[s][0]), 3e-5)
    assert float(state[[1, 3]].abs().max()) == 0.0 and float(last[[1, 3]].abs().max()) == 0.0
    prev, S = full[0][1]
    assert rel(state[2].transpose(1, 2), S) < 2e-5 and rel(last[2], prev) < 1e-7      # stored [head, value column, key channel]


def test_the_bonus_counts_for_the_current_token_only():
    """A sequence's first token sees an empty state: its output is (u * k) . r times v alone, so with u = 0 it would
    be zero; and a token's own k v^T enters later outputs without u."""
    H, n, d, eps = 2, 8, 12, 1e-6
    w = time_mix_weights(H, n, d, 4, seed=3)
    torch.manual_seed(6)
    x = torch.randn(3, d).double()
    state, last = torch.zeros(1, H, n, n, device="cuda"), torch.zeros(1, d, device="cuda")
    from llmplayer_b200.kernels import ops
    out, blends, decay = run_time_mix_kernels(x, w, H, n, eps, state, last, [0], [0, 3], 3)
    b = blends.double().cpu()
    r, k, v = (b[0] @ w["r"].T).view(3, H, n), (b[1] @ w["k"].T).view(3, H, n), (b[2] @ w["v"].T).view(3, H, n)
    g = b[3] @ w["g"].T
    first = ((w["u"] * k[0] * r[0]).sum(-1, keepdim=True) * v[0])                           # [H, n]
    ref0 = (P.unit_rms(first, eps).reshape(-1) * w["norm"] * g[0] * torch.sigmoid(g[0]))
    assert rel(out[0], ref0) < 1e-5
    second = ((w["u"] * k[1] * r[1]).sum(-1, keepdim=True) * v[1]) + ((k[0] * r[1]).sum(-1, keepdim=True) * v[0])
    ref1 = (P.unit_rms(second, eps).reshape(-1) * w["norm"] * g[1] * torch.sigmoid(g[1]))
    assert rel(out[1], ref1) < 1e-5
    S1 = torch.einsum("hk,hv->hkv", k[0], v[0])
    S2 = decay[1].double().cpu().view(H, n)[:, :, None] * S1 + torch.einsum("hk,hv->hkv", k[1], v[1])
    S3 = decay[2].double().cpu().view(H, n)[:, :, None] * S2 + torch.einsum("hk,hv->hkv", k[2], v[2])
    assert rel(state[0].transpose(1, 2), S3) < 1e-5       # the first token's decay touches an empty state only


def test_time_mixing_remembers_an_early_token():
    """Decays held at nearly 1 (a very negative bias) and one early token whose key is large: a query that fits it
    must still find its value 400 tokens later, through the chunks of a long prompt and then token by token."""
    H, n, d, eps = 1, 16, 12, 1e-6
    w = time_mix_weights(H, n, d, 4, seed=9)
    w["w2"] = torch.zeros_like(w["w2"])
    w["w0"] = torch.full_like(w["w0"], -9.0)               # decay = exp(-exp(-9)) = 0.99988 per step
    for b in "rkvgw":
        w["mu." + b] = torch.zeros_like(w["mu." + b])      # every map reads the token itself
    torch.manual_seed(1)
    x = 0.1 * torch.randn(420, d).double()
    x[2] = 20.0 * x[2] / x[2].norm()
    x[-1] = x[2]
    w["r"] = w["k"].clone()                                # the last token's r is token 2's k
    ref, _ = P.wkv(x, {"mix." + name: t for name, t in w.items()}, "mix.", {"heads": H, "dim": n}, eps)
    state, last = torch.zeros(1, H, n, n, device="cuda"), torch.zeros(1, d, device="cuda")
    first, _, _ = run_time_mix_kernels(x[:400], w, H, n, eps, state, last, [0], [0, 400], 400)
    rest = [run_time_mix_kernels(x[t:t + 1], w, H, n, eps, state, last, [0], [0, 1], 1)[0] for t in range(400, 420)]
    got = torch.cat([first] + rest).double().cpu() @ w["o"].T
    check_error("time mixing, float32", "an early token through 400 steps", rel(got, ref), 5e-5)
    # the direction of the last output is that of token 2's value (the norm takes the size away)
    v2 = (x[2] @ w["v"].T)
    raw_dir = P.unit_rms(v2.view(H, n), eps).reshape(-1) * w["norm"]
    g = x[-1] @ w["g"].T
    expected = (raw_dir * g * torch.sigmoid(g)) @ w["o"].T
    cos = float(torch.nn.functional.cosine_similarity(got[-1], expected, dim=0))
    assert cos > 0.98, cos
