"""Each mechanism of the Dopuvik decoder alone, its kernels against the plain implementation's function: the choice of
experts in groups with a correction and identity experts, the short convolution carried over steps and slots, step
sizes / decays / write strengths, unit heads, the gate in front of a norm in parts, the state-space recurrence with
shared keys (whole and in chunks side by side), the gated delta rule over steps and slots, rotation of neighbouring
pairs with a factor on cosine and sine, latent attention in a window, attention with kept first tokens (a key that
stands out just inside and just outside the window and the kept tokens, at page borders, far back), the two-member
sum, the layer norm that clears a buffer on the side."""
import math

import pytest
import torch

import plain_dopuvik as P
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


# --------------------------------------------------------------------------- experts
@pytest.mark.parametrize("E,groups,keep,top,scale", [(6, 3, 2, 2, 1.5), (12, 3, 2, 3, 2.5), (4, 1, 1, 1, 1.0), (8, 4, 3, 4, 0.8),
                                                     (3, 1, 1, 3, 1.0), (3, 3, 1, 1, 1.0), (64, 8, 4, 6, 1.0), (6, 2, 2, 2, 0.5)])
def test_choice_in_groups_with_a_correction(E, groups, keep, top, scale):
    """Scores over ALL outputs, choice on score + correction inside the best groups (a group's score its largest choice
    score; corrections are negative too, so a refused group must count as minus infinity, not zero), weights the
    chosen scores times a constant, not renormalised. The correction decides: without it other experts would win."""
    from llmplayer_b200.kernels import ops
    T = 300
    r = {"top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}
    for seed in range(50):            # a draw in which no choice rests on a close call (float32 against float64)
        torch.manual_seed(E + top + 100 * seed)
        wide = (1.5 * torch.randn(T, E + 5)).cuda()
        z = wide[:, 3:3 + E]
        corr = (torch.randint(-3, 3, (E,)).float() / 4.0 - 0.6).cuda()          # all of them may be negative
        scores = torch.softmax(z.double().cpu(), dim=-1)
        chosen, weights, gap = P.route(scores, corr.double().cpu(), r)
        if gap > 2e-5:
            break
    assert gap > 2e-5
    ref = torch.zeros(T, E, dtype=torch.float64).scatter_(1, chosen, weights)
    got = torch.empty(T, E, device="cuda")
    ops.route_softmax(z, corr, got, groups=groups, keep=keep, top=top, scale=scale)
    assert torch.equal(got.cpu() != 0, ref != 0)
    check_error("choice of experts in groups, float32", f"{E} in {groups}, {keep} kept, top {top}", rel(got, ref), 2e-6)
    assert float((got.sum(-1).cpu() - scale).abs().min()) > 1e-3 or top == E      # not renormalised
    if top < E:
        plain = torch.empty(T, E, device="cuda")
        ops.route_softmax(z, None, plain, groups=groups, keep=keep, top=top, scale=scale)
        assert not torch.equal(plain.cpu() != 0, ref != 0)


def test_identity_experts_pass_their_input_on():
    from llmplayer_b200.kernels import ops
    torch.manual_seed(5)
    T, d, E = 37, 52, 7
    x, h = torch.randn(T, d).cuda(), torch.randn(T, d)
    w = (torch.rand(T, E) * (torch.rand(T, E) > 0.5)).cuda()
    ref = x.double().cpu() + h.double() * w[:, 4:].double().cpu().sum(-1, keepdim=True)
    for dtype, lim in ((torch.float32, 2e-6), (torch.bfloat16, 4e-3)):
        got = x.clone()
        ops.identity_experts(got, h.to(dtype).cuda(), w, 4, 3)
        check_error(f"identity experts, {dtype}", f"{T}x{d}", rel(got, ref), lim)
    # the hidden activations of the real experts only are scaled by the first columns of the weights
    hidden = torch.randn(T, 4 * 8).cuda()
    ref = hidden.double().cpu() * w[:, :4].double().cpu().repeat_interleave(8, dim=1)
    ops.expert_scale(hidden, w, 8, num_experts=4)
    assert rel(hidden, ref) < 2e-6
    # both in one launch: the identities' share rides with the scaling (generic kernel and the eight-column one)
    for dtype, ff, lim in ((torch.float32, 5, 2e-6), (torch.bfloat16, 8, 4e-3)):
        hidden = torch.randn(T, 4 * ff).to(dtype).cuda()
        want_hidden = hidden.double().cpu() * w[:, :4].double().cpu().repeat_interleave(ff, dim=1)
        got = x.clone()
        ops.expert_scale(hidden, w, ff, num_experts=4, identity=(got, h.to(dtype).cuda(), 4, 3))
        want_x = x.double().cpu() + h.to(dtype).double() * w[:, 4:].double().cpu().sum(-1, keepdim=True)
        assert rel(hidden, want_hidden) < (2e-6 if dtype == torch.float32 else 4e-3) and rel(got, want_x) < 2e-6


# --------------------------------------------------------------------------- short convolution
@pytest.mark.parametrize("C,K,bias", [(88, 4, True), (130, 2, False), (48, 1, True), (512, 8, True), (7, 3, False)])
def test_short_convolution_over_steps_and_slots(C, K, bias):
    """Two sequences in slots 2 and 0 (slot 1 stays untouched), cut into steps of unequal numbers of tokens (among them
    fewer than taps - 1, and more than a chunk of the kernel): every cut must give the whole sequence's result, from a
    tail that starts at zero."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(C + K)
    lengths = [150, 41]
    xs = [torch.randn(n, C + 6) for n in lengths]
    taps, b = torch.randn(C, K), (torch.randn(C) if bias else None)
    refs = [P.silu(P.short_convolution(x[:, 3:3 + C].double(), taps.double(), None if b is None else b.double())) for x in xs]
    tail = torch.zeros(3, max(K - 1, 0), C, device="cuda")
    tail[1] = 7.0
    done = [0, 0]
    got = [[], []]
    for step in ([1, 1], [2, 1], [1, 3], [70, 0], [5, 30], [71, 6]):
        seqs = [i for i in (0, 1) if step[i] > 0]
        x = torch.cat([xs[i][done[i]:done[i] + step[i]] for i in seqs]).cuda()
        starts = [0]
        for i in seqs:
            starts.append(starts[-1] + step[i])
        out = torch.full((x.shape[0], C + 2), 9.0, device="cuda")
        ops.short_conv(x[:, 3:3 + C], taps.cuda(), None if b is None else b.cuda(), tail, i32([[2, 0][i] for i in seqs]), i32(starts),
                       out[:, 1:1 + C], max_new=max(step))
        assert float((out[:, 0] - 9.0).abs().max()) == 0.0 and float((out[:, -1] - 9.0).abs().max()) == 0.0
        for j, i in enumerate(seqs):
            got[i].append(out[starts[j]:starts[j + 1], 1:1 + C].cpu())
            done[i] += step[i]
    assert done == lengths
    for i in (0, 1):
        check_error("short convolution over steps, float32", f"{C} channels, {K} taps, sequence {i}", rel(torch.cat(got[i]), refs[i]), 3e-6)
    assert tail[1].numel() == 0 or float((tail[1] - 7.0).abs().max()) == 0.0
    if K > 1:        # the tail holds the last inputs, oldest first
        assert torch.equal(tail[2].cpu(), xs[0][-(K - 1):, 3:3 + C])


def test_decays_step_sizes_and_write_strengths():
    from llmplayer_b200.kernels import ops
    torch.manual_seed(3)
    T, H = 50, 6
    proj = (3.0 * torch.randn(T, 40)).cuda()
    proj[0, 5] = 30.0                                         # beyond where exp would overflow a naive softplus' float32
    dt_bias, a_log = torch.randn(H).cuda(), torch.randn(H).cuda()
    decay, dt, strength = (torch.empty(T, H, device="cuda") for _ in range(3))
    ops.decay_gates(proj, 5, dt_bias, a_log, decay, dt=dt, strength=strength, b_off=20)
    p = proj.double().cpu()
    ref_dt = P.softplus(p[:, 5:5 + H] + dt_bias.double().cpu())
    assert rel(dt, ref_dt) < 2e-6 and rel(decay, torch.exp(-torch.exp(a_log.double().cpu()) * ref_dt)) < 2e-6
    assert rel(strength, torch.sigmoid(p[:, 20:20 + H])) < 2e-6
    assert float(dt[0, 0]) > 25.0                              # no clamp on the step size


def test_unit_heads():
    from llmplayer_b200.kernels import ops
    torch.manual_seed(4)
    T, G, dk = 9, 3, 20
    x = torch.randn(T, 2 * G * dk + 11).cuda()
    x[0, :dk] = 0.0                                            # a zero head stays zero (the constant inside the root)
    ref = x.double().cpu().clone()
    heads = ref[:, :2 * G * dk].reshape(T, 2 * G, dk)
    heads = heads / torch.sqrt((heads * heads).sum(-1, keepdim=True) + 1e-6)
    heads[:, :G] *= dk ** -0.5
    ref[:, :2 * G * dk] = heads.reshape(T, -1)
    ops.head_unit_norm(x, 0, 2 * G, dk, 1e-6, dk ** -0.5, scaled_heads=G)
    assert rel(x, ref) < 2e-6 and float(x[0, :dk].abs().max()) == 0.0


@pytest.mark.parametrize("H,Pd,parts", [(6, 8, 3), (2, 16, 1), (4, 64, 2), (1, 12, 2), (8, 8, 8)])
def test_gate_then_norm_in_parts(H, Pd, parts):
    """(y + D x) * silu(z), then every part by its own root mean square. Norm first and gate second is another function."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(H * Pd)
    T, W = 13, H * Pd
    raw, wide = torch.randn(T, W).cuda(), torch.randn(T, 2 * W + 4).cuda()
    z, x = wide[:, :W], wide[:, W + 4:]
    skip, gain = torch.randn(H).cuda(), (1 + 0.3 * torch.randn(W)).cuda()
    y = (raw.double().cpu() + skip.double().cpu().repeat_interleave(Pd) * x.double().cpu()) * P.silu(z.double().cpu())
    ref = P.unit_rms(y.reshape(T, parts, W // parts), 1e-5).reshape(T, W) * gain.double().cpu()
    for dtype, lim in ((torch.float32, 3e-6), (torch.bfloat16, 5e-3)):
        out = torch.empty(T, W, device="cuda", dtype=dtype)
        ops.gated_part_norm(raw, z, gain, 1e-5, out, num_heads=H, head_dim=Pd, parts=parts, values=x, skip=skip)
        check_error(f"gate, then norm in parts, {dtype}", f"{H} x {Pd} in {parts}", rel(out, ref), lim)
    other = P.unit_rms((raw.double().cpu() + skip.double().cpu().repeat_interleave(Pd) * x.double().cpu()).reshape(T, parts, -1), 1e-5)
    assert rel(other.reshape(T, W) * gain.double().cpu() * P.silu(z.double().cpu()), ref) > 1e-2


# --------------------------------------------------------------------------- state space
def plain_state_space(x, B, C, dt, decay, S):
    """x [T, H, P], B / C [T, G, N], dt / decay [T, H], S [H, N, P] (changed in place) -> y [T, H, P]."""
    T, H, _ = x.shape
    G = B.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for h in range(H):
            g = h // (H // G)
            S[h] = decay[t, h] * S[h] + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S[h].T @ C[t, g]
    return y


@pytest.mark.parametrize("H,G,N,Pd", [(6, 2, 20, 8), (2, 1, 8, 16), (4, 4, 64, 64), (8, 1, 128, 16)])
def test_state_space_recurrence_over_steps_and_slots(H, G, N, Pd):
    """Keys and queries shared by the heads of a group, one decay per head, the step size as the keys' gain; two
    sequences in slots 3 and 1, the second step long enough for chunks side by side from a state that is not zero."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(H + N)
    lengths = [300, 9]
    inner = H * Pd
    state = torch.zeros(4, H, Pd, N, device="cuda")
    state[2] = 5.0
    data = []
    for n in lengths:
        x, B, C = torch.randn(n, H, Pd), torch.randn(n, G, N) / math.sqrt(N), torch.randn(n, G, N)
        dt, decay = torch.rand(n, H) + 0.1, torch.rand(n, H) * 0.6 + 0.4
        S = torch.zeros(H, N, Pd, dtype=torch.float64)
        ref = plain_state_space(x.double(), B.double(), C.double(), dt.double(), decay.double(), S)
        data.append((x, B, C, dt, decay, ref, S))
    done, got = [0, 0], [[], []]
    for step in ([4, 1], [296, 8]):
        parts = [torch.cat([d[0][done[i]:done[i] + step[i]].reshape(step[i], -1), d[1][done[i]:done[i] + step[i]].reshape(step[i], -1),
                            d[2][done[i]:done[i] + step[i]].reshape(step[i], -1)], dim=1) for i, d in enumerate(data)]
        mixed = torch.cat(parts).cuda()
        decay = torch.cat([d[4][done[i]:done[i] + step[i]] for i, d in enumerate(data)]).cuda()
        dt = torch.cat([d[3][done[i]:done[i] + step[i]] for i, d in enumerate(data)]).cuda()
        out = torch.empty(sum(step), inner, device="cuda")
        ops.gla_scan(mixed, inner + G * N, inner, 0, decay, state, i32([3, 1]), i32([0, step[0], sum(step)]), out, num_heads=H,
                     key_dim=N, value_dim=Pd, q_scale=1.0, max_new=max(step), scratch=scratch, decay_per_head=True, key_gain=dt,
                     qk_heads=G)
        got[0].append(out[:step[0]].cpu())
        got[1].append(out[step[0]:].cpu())
        done = [done[i] + step[i] for i in (0, 1)]
    for i in (0, 1):
        check_error("state-space recurrence, float32", f"{H} heads in {G} groups, {N} x {Pd}, sequence {i}",
                    rel(torch.cat(got[i]).view(lengths[i], H, Pd), data[i][5]), 2e-5)
        assert rel(state[[3, 1][i]].transpose(1, 2), data[i][6]) < 2e-5
    assert float((state[2] - 5.0).abs().max()) == 0.0 and float(state[0].abs().max()) == 0.0


# --------------------------------------------------------------------------- gated delta rule
def plain_delta_rule(q, k, v, beta, g, S):
    """q / k [T, G, dk], v [T, H, dv], beta / g [T, H], S [H, dk, dv] (changed in place) -> o [T, H, dv]."""
    T, H, _ = v.shape
    G = k.shape[1]
    o = torch.zeros_like(v)
    for t in range(T):
        for h in range(H):
            kk, qq = k[t, h // (H // G)], q[t, h // (H // G)]
            S[h] = g[t, h] * S[h]
            u = beta[t, h] * (v[t, h] - S[h].T @ kk)
            S[h] = S[h] + torch.outer(kk, u)
            o[t, h] = S[h].T @ qq
    return o


@pytest.mark.parametrize("H,G,dk,dv", [(4, 2, 20, 12), (2, 1, 16, 24), (2, 2, 128, 128), (4, 2, 64, 32), (1, 1, 6, 10), (3, 3, 256, 40)])
def test_delta_rule_over_steps_and_slots(H, G, dk, dv):
    """Steps of 1, 2, 30, 117 and 300 tokens (the last in chunks side by side, each chunk with its transition matrix)
    for two sequences in slots 2 and 3; slots 0 and 1 stay as they were."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(dk + dv)
    lengths = [420, 333]             # the last step is long enough for chunks side by side, from a state that is not zero
    state = torch.zeros(4, H, dv, dk, device="cuda")
    state[0] = -4.0
    data = []
    for n in lengths:
        q, k = torch.randn(n, G, dk), torch.randn(n, G, dk)
        q, k = q / q.norm(dim=-1, keepdim=True) * dk ** -0.5, k / k.norm(dim=-1, keepdim=True)
        v, beta, g = torch.randn(n, H, dv), torch.rand(n, H), torch.rand(n, H) * 0.5 + 0.5
        S = torch.zeros(H, dk, dv, dtype=torch.float64)
        ref = plain_delta_rule(q.double(), k.double(), v.double(), beta.double(), g.double(), S)
        data.append((q, k, v, beta, g, ref, S))
    done, got = [0, 0], [[], []]
    for step in ([1, 1], [2, 30], [117, 2], [300, 300]):
        cat = lambda j: torch.cat([d[j][done[i]:done[i] + step[i]].reshape(step[i], -1) for i, d in enumerate(data)])
        mixed = torch.cat([cat(0), cat(1), cat(2)], dim=1).cuda()
        out = torch.empty(sum(step), H * dv, device="cuda")
        ops.gla_scan(mixed, 0, G * dk, 2 * G * dk, cat(4).cuda(), state, i32([2, 3]), i32([0, step[0], sum(step)]), out, num_heads=H,
                     key_dim=dk, value_dim=dv, q_scale=1.0, max_new=max(step), scratch=scratch, decay_per_head=True, qk_heads=G,
                     delta_strength=cat(3).cuda())
        got[0].append(out[:step[0]].cpu())
        got[1].append(out[step[0]:].cpu())
        done = [done[i] + step[i] for i in (0, 1)]
    for i in (0, 1):
        check_error("gated delta rule, float32", f"{H} heads on {G}, {dk} x {dv}, sequence {i}",
                    rel(torch.cat(got[i]).view(lengths[i], H, dv), data[i][5]), 2e-5)
        assert rel(state[[2, 3][i]].transpose(1, 2), data[i][6]) < 2e-5
    assert float((state[0] + 4.0).abs().max()) == 0.0 and float(state[1].abs().max()) == 0.0


def test_delta_rule_replaces_what_a_key_held():
    """Full strength, no decay: writing a second value under the same unit key must REPLACE the first (a plain sum
    would hold both), and the read-out must see the token's own write."""
    from llmplayer_b200.kernels import ops
    dk, dv = 32, 16
    key = torch.zeros(dk)
    key[3] = 1.0
    v1, v2 = torch.randn(dv), torch.randn(dv)
    mixed = torch.zeros(2, 2 * dk + dv)
    mixed[:, :dk] = key
    mixed[:, dk:2 * dk] = key
    mixed[0, 2 * dk:], mixed[1, 2 * dk:] = v1, v2
    state = torch.zeros(1, 1, dv, dk, device="cuda")
    out = torch.empty(2, dv, device="cuda")
    ones = torch.ones(2, 1, device="cuda")
    ops.gla_scan(mixed.cuda(), 0, dk, 2 * dk, ones, state, i32([0]), i32([0, 2]), out, num_heads=1, key_dim=dk, value_dim=dv,
                 q_scale=1.0, max_new=2, decay_per_head=True, delta_strength=ones)
    assert float((out[0].cpu() - v1).abs().max()) < 1e-6 and float((out[1].cpu() - v2).abs().max()) < 1e-6
    assert float((state[0, 0, :, 3].cpu() - v2).abs().max()) < 1e-6


# --------------------------------------------------------------------------- latent attention
def latent_reference(q, rows, dn, rank, uk, uv, scale, window, first_query):
    """q [Tq, H, dn + dr] (rotated), rows [Tk, rank + dr] (normed latent | rotated shared key part)."""
    Tq, H, _ = q.shape
    c, kr = rows[:, :rank], rows[:, rank:]
    gap = torch.arange(first_query, first_query + Tq)[:, None] - torch.arange(rows.shape[0])[None, :]
    seen = (gap >= 0) & ((gap < window) if window else True)
    dv = uv.shape[0] // H
    out = torch.zeros(Tq, H, dv, dtype=torch.float64)
    for h in range(H):
        k = torch.cat([c @ uk[h * dn:(h + 1) * dn].T, kr], dim=1)
        s = ((q[:, h] @ k.T) * scale).masked_fill(~seen, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ (c @ uv[h * dv:(h + 1) * dv].T)
    return out


@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dn,dr,dv,rank,length,new,window", [(3, 24, 8, 20, 40, 200, 200, 17), (4, 32, 32, 64, 64, 321, 321, 70),
                                                               (5, 10, 2, 12, 10, 130, 130, 1), (2, 64, 64, 128, 128, 300, 57, None),
                                                               (2, 16, 16, 16, 32, 700, 1, 64), (2, 16, 16, 16, 32, 700, 1, 65),
                                                               (4, 8, 8, 8, 16, 400, 300, 129)])
def test_latent_attention_in_a_window(kv_dtype, H, dn, dr, dv, rank, length, new, window):
    """Rotation of neighbouring pairs with a factor on cosine and sine, rows through scrambled pages, the absorbed
    form in 1, 3 and 8 shares, the window by position difference; one token wider or narrower differs visibly."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(length + rank)
    scale, eps, magnitude = 0.3, 1e-5, 1.2
    freqs = P.plain_frequencies(500.0, dr)
    positions = torch.arange(length)
    down = torch.randn(length, rank + dr)
    gain = 1 + 0.3 * torch.randn(rank)
    q_raw = torch.randn(length, H * (dn + dr))
    uk, uv = torch.randn(H * dn, rank) / math.sqrt(rank), torch.randn(H * dv, rank) / math.sqrt(rank)
    c = P.unit_rms(down[:, :rank].double(), eps) * gain.double()
    kr = P.rotate(down[:, rank:].double().reshape(length, 1, dr), positions, freqs, dr, True, magnitude).reshape(length, dr)
    qh = q_raw.double().reshape(length, H, dn + dr)
    qrot = torch.cat([qh[..., :dn], P.rotate(qh[..., dn:], positions, freqs, dr, True, magnitude)], dim=-1)
    rows_exact = torch.cat([c, kr], dim=1)
    order = torch.randperm(16).tolist()[:-(-length // PAGE)]
    table = i32([order + [0] * (16 - len(order))])
    pages = torch.zeros(16, PAGE, rank + dr, dtype=kv_dtype, device="cuda")
    rotation = ops.Rotation(torch.tensor(freqs, dtype=torch.float32).cuda(), dr, True, magnitude)
    # the whole sequence's rows are prepared (as earlier steps would have), then the last `new` tokens attend
    proj = torch.cat([torch.zeros(length, 5), down], dim=1).cuda()
    q_all = torch.empty(length, H, dn + dr, device="cuda")
    ops.latent_prepare(proj, 0, 5, gain.cuda(), eps, rotation, i32(list(range(length))), i32([0] * length), table, q_all, pages,
                       num_heads=H, nope_dim=dn, rope_dim=dr, kv_rank=rank, q_from=q_raw.cuda())
    assert rel(q_all, qrot) < 4e-5            # the angle position x frequency is a float32 product: its rounding grows with the position
    stored = torch.stack([pages[order[t // PAGE], t % PAGE] for t in range(length)])
    assert rel(stored, rows_exact) < (4e-5 if kv_dtype == torch.float32 else 8e-3)
    # the attention itself is held against the rows as the cache holds them
    ref = latent_reference(qrot[length - new:], stored.double().cpu(), dn, rank, uk.double(), uv.double(), scale, window, length - new)
    q_new = q_all[length - new:].contiguous()
    q_abs = torch.empty(new, H, rank + dr, device="cuda")
    ops.latent_absorb(q_new, uk.cuda(), q_abs, nope_dim=dn, rope_dim=dr)
    results = []
    for shares in (1, 3, 8):
        partials = torch.empty(new, H, shares, rank + 2, device="cuda")
        ops.latent_attend(q_abs, pages, table, i32([0, new]), i32([length]), partials, max_new=new, kv_rank=rank, scale=scale,
                          window=window)
        out = torch.empty(new, H * dv, device="cuda")
        ops.latent_expand(partials, uv.cuda(), None, out, value_dim=dv)
        check_error(f"latent attention in a window, cache {kv_dtype}", f"{H} x ({dn}+{dr}), rank {rank}, {new} of {length}, window {window}, "
                    f"{shares} shares", rel(out.view(new, H, dv), ref), 2e-5)
        results.append(out)
    if window and window <= 70 and window < length:
        for other in (window - 1, window + 1):
            if other > 0:
                partials = torch.empty(new, H, 1, rank + 2, device="cuda")
                ops.latent_attend(q_abs, pages, table, i32([0, new]), i32([length]), partials, max_new=new, kv_rank=rank, scale=scale,
                                  window=other)
                off = torch.empty(new, H * dv, device="cuda")
                ops.latent_expand(partials, uv.cuda(), None, off, value_dim=dv)
                assert rel(off.view(new, H, dv), ref) > 1e-3, other


def test_queries_through_their_own_latent():
    from llmplayer_b200.kernels import ops
    torch.manual_seed(8)
    T, rank = 21, 28
    proj = torch.randn(T, rank + 9).cuda()
    gain = (1 + 0.3 * torch.randn(rank)).cuda()
    ref = P.unit_rms(proj[:, 4:4 + rank].double().cpu(), 2e-6) * gain.double().cpu()
    for dtype, lim in ((torch.float32, 2e-6), (torch.bfloat16, 4e-3)):
        out = torch.empty(T, rank, device="cuda", dtype=dtype)
        ops.latent_query_norm(proj, 4, gain, 2e-6, out)
        assert rel(out, ref) < lim


# --------------------------------------------------------------------------- attention with kept first tokens
def fill_pages(k, v, table_rows, num_pages, dtype):
    T, G, hd = k.shape
    pages = torch.zeros(num_pages, 2, G, PAGE, hd, dtype=dtype, device="cuda")
    for t in range(T):
        page = table_rows[t // PAGE]
        pages[page, 0, :, t % PAGE] = k[t].to(dtype)
        pages[page, 1, :, t % PAGE] = v[t].to(dtype)
    return pages


def plain_kept_attention(q, k, v, scale, window, keep, first_query):
    Tq, H, hd = q.shape
    G = k.shape[1]
    keys = torch.arange(k.shape[0])
    gap = torch.arange(first_query, first_query + Tq)[:, None] - keys[None, :]
    seen = (gap >= 0) & ((gap < window) | (keys[None, :] < keep))
    out = torch.zeros(Tq, H, v.shape[2], dtype=torch.float64)
    for h in range(H):
        g = h // (H // G)
        s = ((q[:, h] @ k[:, g].T) * scale).masked_fill(~seen, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def run_kept(kind, qd, pages, table, length, new, window, keep, H, G, hd, scale):
    from llmplayer_b200.kernels import ops
    out = torch.empty_like(qd)
    if kind == "plain":
        ops.attention_plain(qd, out, pages, table, i32([0] * new), i32(list(range(length - new, length))), num_heads=H,
                            num_kv_heads=G, head_dim=hd, scale=scale, window=window, keep_first=keep)
    elif kind == "prompt":
        ops.attention_prefill(qd, out, pages, table, i32([0, new]), i32([length]), new, num_heads=H, num_kv_heads=G,
                              head_dim=hd, scale=scale, window=window, exact_weights=True, keep_first=keep)
    else:
        ops.attention_decode(qd, out, pages, table, i32([length]), scratch, num_heads=H, num_kv_heads=G, head_dim=hd,
                             scale=scale, window=window, exact_weights=True, keep_first=keep)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,length,new,window,keep", [(4, 2, 48, 200, 200, 9, 3), (8, 1, 64, 321, 321, 64, 70), (2, 2, 128, 400, 57, 128, 1),
                                                           (6, 2, 96, 700, 700, 33, 130), (5, 1, 16, 130, 130, 2, 5), (2, 1, 64, 400, 300, 44, 18),
                                                           (3, 3, 16, 300, 1, 10, 64), (2, 2, 64, 260, 2, 65, 0), (2, 1, 64, 500, 500, 1, 1),
                                                           (8, 1, 64, 900, 1, 64, 70), (6, 2, 128, 1000, 1, 200, 130), (4, 4, 32, 1000, 1, 40, 0),
                                                           (2, 2, 192, 300, 300, 100, 10), (2, 1, 192, 200, 1, 70, 65)])
def test_attention_with_kept_first_tokens(dtype, H, G, hd, length, new, window, keep):
    """The last ``new`` tokens of a sequence of ``length`` see their window AND the sequence's first ``keep`` tokens
    (pages in a scrambled order; the pages between the kept ones and the window are not in the table at all): the
    plain kernel in float32 and bfloat16, the tensor-core prompt and decode kernels in bfloat16. One kept token more or fewer differs."""
    torch.manual_seed(length + hd + keep)
    scale = 0.3
    q = torch.randn(new, H, hd).to(dtype)
    k, v = torch.randn(length, G, hd).to(dtype), torch.randn(length, G, hd).to(dtype)
    rows = torch.randperm(16).tolist()[:-(-length // PAGE)]
    pages = fill_pages(k, v, rows, 16, dtype)
    # what the cache would have given back by now: pages wholly between the kept tokens and the first query's window
    first_needed = (length - new) - window + 1
    listed = [r if (b < -(-keep // PAGE) or b >= max(0, first_needed) // PAGE) else -1 for b, r in enumerate(rows)]
    table = i32([listed + [0] * (16 - len(listed))])
    ref = plain_kept_attention(q.double(), k.double(), v.double(), scale, window, keep, length - new)
    qd = q.reshape(new, H * hd).cuda()
    kinds = [("plain", 3e-6)] if dtype == torch.float32 else [("plain", 6e-3), ("prompt", 6e-3) if new > 1 else ("decode", 6e-3)]
    for kind, lim in kinds:
        out = run_kept(kind, qd, pages, table, length, new, window, keep, H, G, hd, scale)
        check_error(f"attention with kept first tokens, {kind} kernel, {dtype}", f"{H}/{G} x {hd}, {new} of {length}, window {window}, "
                    f"keep {keep}", rel(out.view(new, H, hd), ref), lim)
        full = i32([rows + [0] * (16 - len(rows))])
        for other in (keep - 1, keep + 1):
            if other >= 0 and window + max(keep, other) < length and window <= 40:
                off = run_kept(kind, qd, pages, full, length, new, window, other, H, G, hd, scale)
                assert rel(off.view(new, H, hd), ref) > 1e-3, (kind, other)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("step", ["prompt", "decode"])
@pytest.mark.parametrize("length,window,keep", [(700, 70, 20), (700, 64, 64), (700, 65, 65), (700, 128, 1), (300, 33, 130), (200, 9, 3),
                                                (130, 2, 5), (130, 1, 1), (700, 40, 128), (700, 40, 129)])
def test_a_key_at_the_edges_of_window_and_kept_tokens(dtype, step, length, window, keep):
    """Head 1's last query is made to fit ONE key far better than all others. On the last position inside the window
    or on the last kept position its value must come through nearly alone; one further back, or on the first position
    that is not kept, it must not be seen at all. A prompt step of 40 tokens and a one-token step; the edges fall before,
    on and behind page borders."""
    torch.manual_seed(window + keep)
    H, G, hd, scale = 4, 2, 64, 0.5
    new = 40 if step == "prompt" else 1
    direction = torch.randn(hd)
    direction /= direction.norm()
    last = length - 1
    for at, seen in ((last - (window - 1), True), (last - window, False), (keep - 1, True), (keep, False), (0, keep > 0)):
        if at < 0 or (not seen and (last - at < window or at < keep)):
            continue
        k, v = 0.3 * torch.randn(length, G, hd), torch.randn(length, G, hd)
        q = 0.3 * torch.randn(new, H, hd)
        q[-1, 1] = 8.0 * direction
        k[at, 0] = 8.0 * direction                         # score 64 * 0.5 = 32 against scores near 0
        k, v, q = k.to(dtype), v.to(dtype), q.to(dtype)
        rows = torch.randperm(16).tolist()[:-(-length // PAGE)]
        pages = fill_pages(k, v, rows, 16, dtype)
        table = i32([rows + [0] * (16 - len(rows))])
        qd = q.reshape(new, H * hd).cuda()
        kind = "plain" if dtype == torch.float32 else step
        out = run_kept(kind, qd, pages, table, length, new, window, keep, H, G, hd, scale).view(new, H, hd)
        ref = plain_kept_attention(q.double(), k.double(), v.double(), scale, window, keep, length - new)
        check_error(f"kept first tokens, a key that stands out, {step}, {dtype}", f"length {length}, window {window}, keep {keep}, key at {at}",
                    rel(out, ref), 3e-6 if dtype == torch.float32 else 6e-3)
        got = out[-1, 1].double().cpu()
        if seen:
            assert float((got - v[at, 0].double()).abs().max()) < 1e-3 + (0.02 if dtype == torch.bfloat16 else 0.0), at
        else:
            assert float((got - v[at, 0].double()).abs().max()) > 0.5, at


# --------------------------------------------------------------------------- small kernels
def test_two_results_summed_with_constants():
    from llmplayer_b200.kernels import ops
    torch.manual_seed(6)
    T, d = 19, 52
    x, a, b = torch.randn(T, d).cuda(), torch.randn(T, d).cuda(), torch.randn(T, d).cuda()
    va = torch.randn(d).cuda()
    ref = x.double().cpu() + 1.2 * (a.double().cpu() + va.double().cpu()) + 0.7 * b.double().cpu()
    got = x.clone()
    ops.scaled_sum(got, a, 1.2, b, 0.7, a_vector=va)
    assert rel(got, ref) < 2e-6
    alone = x.clone()
    ops.scaled_sum(alone, a, -0.5)
    assert rel(alone, x.double().cpu() - 0.5 * a.double().cpu()) < 2e-6


def test_layer_norm_clears_on_the_side():
    from llmplayer_b200.kernels import ops
    torch.manual_seed(7)
    x, w = (3 + 2 * torch.randn(9, 72)).cuda(), (1 + 0.3 * torch.randn(72)).cuda()
    junk = torch.full((1000,), 3.0, device="cuda")
    out = torch.empty(9, 72, device="cuda")
    ops.layernorm(x, w, 2e-6, out, clear=junk)
    assert rel(out, P.layer_norm(x.double().cpu(), w.double().cpu(), 2e-6)) < 3e-6 and float(junk.abs().max()) == 0.0
