"""The Dopuvik decoder through the engine's step function, cache and generation loop, against the plain
implementation: whole prompts, the stream after every layer, prompts against token-by-token decoding, portions down
to two tokens, unequal batches, slots and pages that are used again, long decoding past every window and past the kept
first tokens, the first tokens, greedy generation, the command line, trace replay."""
import json
import os
import subprocess
import sys

import pytest
import torch

from helpers import check_error, random_tokens, relative_error
from dopuvik_helpers import CONFIGS, bound, make_model, plain_logits

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NAMES = ["small", "wide", "ragged", "recurrent", "attentive"]


def close(got, ref, dtype, name, what):
    """float32: every position within the bound. bfloat16: a delta rule's head is divided by its own root mean square,
    and where the terms of that output nearly cancel (a position here and there) rounding is amplified; so at most
    one position in fifty (or one) may exceed the bound, and none four times the bound."""
    if dtype == "float32":
        return check_error(f"Dopuvik logits, {dtype}", f"{name} {what}", relative_error(got, ref), bound(dtype, name))
    got, ref = torch.as_tensor(got, dtype=torch.float64).cpu(), torch.as_tensor(ref, dtype=torch.float64).cpu()
    assert got.shape == ref.shape and torch.isfinite(got).all()
    rows = (got - ref).abs().reshape(-1, ref.shape[-1]).max(-1).values / ref.abs().max()
    allowed = max(1, rows.numel() // 50)
    usual = float(rows.sort().values[-(allowed + 1)]) if rows.numel() > allowed else 0.0
    check_error(f"Dopuvik logits, {dtype}, {name}, all but one position in fifty", f"{what}", usual, bound(dtype, name))
    return check_error(f"Dopuvik logits, {dtype}, {name}, worst position", f"{what}", float(rows.max()), 4 * bound(dtype, name))


def vocab(name):
    return CONFIGS[name][0]["vocab"]


def reference(model_dir, tokens):
    """Plain logits; every routing must have been decided by a clear gap, or a bfloat16 comparison would test the
    rounding of a tie and not the mechanism."""
    gaps = []
    ref = plain_logits(model_dir, tokens, gaps=gaps)
    assert not gaps or min(gaps) > 5e-4, min(gaps)
    return ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,length", [("small", 1), ("small", 2), ("small", 97), ("small", 300), ("wide", 33), ("wide", 71),
                                         ("wide", 200), ("wide", 321), ("ragged", 3), ("ragged", 270), ("recurrent", 280),
                                         ("attentive", 150)])
def test_whole_sequence(tmp_path, name, length, dtype):
    from llmplayer_b200 import Engine
    model_dir = make_model(tmp_path, name, dtype)
    tokens = random_tokens(length, vocab(name), seed=length)
    eng = Engine.load(model_dir, dtype=dtype, max_tokens=512)
    slot = eng.acquire()
    logits = eng.step([(slot, tokens)], [list(range(length))]).cpu()
    eng.release(slot)
    eng.check()
    close(logits, reference(model_dir, tokens), dtype, name, f"whole {length}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["small", "wide"])
def test_the_stream_after_every_layer(tmp_path, name, dtype):
    import plain_dopuvik
    from llmplayer_b200 import Engine
    model_dir = make_model(tmp_path, name, dtype)
    tokens = random_tokens(90, vocab(name), seed=17)
    cfg, w = plain_dopuvik.read_model(model_dir)
    streams = []
    plain_dopuvik.forward(cfg, w, tokens, streams=streams)
    eng = Engine.load(model_dir, dtype=dtype, max_tokens=128)
    seen = []
    for block in eng.model.blocks:
        def wrapped(ctx, cache, residual, _inner=block.forward, **kw):
            out = _inner(ctx, cache, residual, **kw)
            seen.append(residual.detach().float().cpu().clone())
            return out
        block.forward = wrapped
    slot = eng.acquire()
    eng.step([(slot, tokens)], [[0]])
    assert len(seen) == len(streams) == len(cfg["layers"])
    for j, (got, ref) in enumerate(zip(seen, streams)):
        check_error(f"Dopuvik stream, {dtype}", f"{name} after layer {j}", relative_error(got, ref), 1e-5 if dtype == "float32" else 3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_token_by_token(tmp_path, name, dtype):
    """Most of a sequence in one step, the rest one token at a time: the decoded tokens cross a page's border
    (position 128) and, in ``wide``, the windows of 70, 64 and 128 tokens pass from prompt keys onto decoded keys while
    the 70 kept first tokens (more than a page) stay in sight."""
    from llmplayer_b200 import Engine
    model_dir = make_model(tmp_path, name, dtype)
    tokens = random_tokens(236, vocab(name), seed=4)
    ref = reference(model_dir, tokens)
    eng = Engine.load(model_dir, dtype=dtype, max_tokens=256)
    slot = eng.acquire()
    first = eng.step([(slot, tokens[:93])], [[0, 1, 63, 64, 92]]).cpu().clone()
    close(first, ref[[0, 1, 63, 64, 92]], dtype, name, "prompt part")
    rows = [eng.step([(slot, [t])], [[0]]).cpu().clone() for t in tokens[93:]]
    eng.release(slot)
    eng.check()
    close(torch.cat(rows), ref[93:], dtype, name, "decoded part")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_a_prompt(tmp_path, name, dtype):
    """A prompt cut into portions of 2, 3, 7, 64, 65, 1, 31 and 260 tokens (the last long enough for the recurrence's
    chunks that run side by side, from a state that is not zero): the states, the convolutions' last inputs, the
    windows and the kept first tokens carry over, whatever the cut."""
    from llmplayer_b200 import Engine
    model_dir = make_model(tmp_path, name, dtype)
    cuts = [2, 3, 7, 64, 65, 1, 31, 260]
    tokens = random_tokens(sum(cuts), vocab(name), seed=8)
    ref = reference(model_dir, tokens)
    eng = Engine.load(model_dir, dtype=dtype, max_tokens=512)
    slot = eng.acquire()
    rows, at = [], 0
    for n in cuts:
        rows.append(eng.step([(slot, tokens[at:at + n])], [list(range(n))]).cpu().clone())
        at += n
    eng.release(slot)
    close(torch.cat(rows), ref, dtype, name, "portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_and_reuse(tmp_path, name, dtype):
    """Requests of unequal lengths in one batch, decoded together while the shorter ones end; then new requests
    in the slots and pages that were given back (their states and convolution tails must start at zero); each against
    itself alone."""
    from llmplayer_b200 import Engine
    model_dir = make_model(tmp_path, name, dtype)
    eng = Engine.load(model_dir, dtype=dtype, max_tokens=640, max_slots=4)
    V = vocab(name)

    def run_batch(lengths, decode, seed):
        seqs = [random_tokens(n + d, V, seed=seed + i) for i, (n, d) in enumerate(zip(lengths, decode))]
        refs = [reference(model_dir, s) for s in seqs]
        slots = [eng.acquire() for _ in seqs]
        got = [[] for _ in seqs]
        out = eng.step([(s, q[:n]) for s, q, n in zip(slots, seqs, lengths)], [[n - 1] for n in lengths]).cpu().clone()
        for i in range(len(seqs)):
            got[i].append(out[i:i + 1])
        live = list(range(len(seqs)))
        step = 0
        while live:
            live = [i for i in live if step < decode[i]]
            if not live:
                break
            out = eng.step([(slots[i], [seqs[i][lengths[i] + step]]) for i in live], [[0]] * len(live)).cpu().clone()
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
            step += 1
            for i in list(live):
                if step >= decode[i]:
                    eng.release(slots[i])
        for i in range(len(seqs)):
            if decode[i] == 0:
                eng.release(slots[i])
            close(torch.cat(got[i]), refs[i][lengths[i] - 1:], dtype, name, f"batch request {i}")
        return slots

    first = run_batch([70, 5, 131, 1], [20, 3, 9, 0], seed=30)
    second = run_batch([3, 66, 64], [6, 6, 70], seed=60)
    assert set(second) <= set(first)                       # the slots were handed out again
    eng.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["small", "wide"])
def test_long_decoding_and_first_tokens(tmp_path, name, dtype):
    """One token, then 300 more one by one (four page borders; every window but the widest fills up and moves on
    over decoded keys alone): the first positions and all others."""
    from llmplayer_b200 import Engine
    model_dir = make_model(tmp_path, name, dtype)
    tokens = random_tokens(301, vocab(name), seed=2)
    ref = reference(model_dir, tokens)
    eng = Engine.load(model_dir, dtype=dtype, max_tokens=320)
    slot = eng.acquire()
    rows = [eng.step([(slot, [t])], [[0]]).cpu().clone() for t in tokens]
    eng.release(slot)
    eng.check()
    got = torch.cat(rows)
    close(got[:4], ref[:4], dtype, name, "first tokens")
    close(got, ref, dtype, name, "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["small", "wide"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype):
    """``Engine.generate`` (the scheduler, captured steps and the native host loop in bfloat16): a batch of
    unequal prompts over three slots; tokens against the plain implementation's argmax wherever its margin
    exceeds what rounding can flip."""
    import plain_dopuvik
    from llmplayer_b200 import Engine
    from llmplayer_b200.sampling import SamplerConfig
    model_dir = make_model(tmp_path, name, dtype)
    cfg, w = plain_dopuvik.read_model(model_dir)
    eng = Engine.load(model_dir, dtype=dtype, max_tokens=512, max_slots=3)
    prompts = [random_tokens(n, vocab(name), seed=70 + n) for n in (9, 70, 2, 31, 64)]
    out = eng.generate(prompts, SamplerConfig.greedy(), max_tokens=12, stop_token_ids=())
    slack = 1e-4 if dtype == "float32" else 2 * bound(dtype, name)
    compared = 0
    for prompt, response in zip(prompts, out):
        assert response.token_count == 12
        logits = plain_dopuvik.forward(cfg, w, list(prompt) + response.token_ids)
        for i, tok in enumerate(response.token_ids):
            row = logits[len(prompt) - 1 + i]
            assert float(row[tok]) >= float(row.max()) - slack * float(row.abs().max()), (name, dtype, i)
            compared += 1
    assert compared == 60


def test_sampled_generation_steps_the_state_once(tmp_path):
    """A seeded sampler: the captured steps of the native host loop must draw the same tokens as plain stepping,
    which they only do if no step ever ran twice over the recurrent states or the convolutions' tails."""
    from llmplayer_b200 import Engine
    from llmplayer_b200.sampling import SamplerConfig
    model_dir = make_model(tmp_path, "wide", "bfloat16")
    prompts = [random_tokens(n, vocab("wide"), seed=90 + n) for n in (12, 40, 3)]
    fast = Engine.load(model_dir, dtype="bfloat16", max_tokens=512, max_slots=3)
    slow = Engine.load(model_dir, dtype="bfloat16", max_tokens=512, max_slots=3, host_loop=False, graphs=False)
    for again in range(2):                                 # the second time re-uses slots, pages and captured graphs
        a = fast.generate(prompts, SamplerConfig(seed=5 + again), max_tokens=24, stop_token_ids=())
        b = slow.generate(prompts, SamplerConfig(seed=5 + again), max_tokens=24, stop_token_ids=())
        assert [r.token_ids for r in a] == [r.token_ids for r in b]


def test_command_line_generates(tmp_path):
    model_dir = make_model(tmp_path, "small", "bfloat16")
    proc = subprocess.run([sys.executable, "-m", "llmplayer_b200", "--model", model_dir, "--prompt", "5 17 3 99", "-n", "8",
                           "--temperature", "0", "--context-length", "128"], capture_output=True, text=True, timeout=600,
                          cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "8 generated" in proc.stdout, proc.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay(tmp_path, dtype):
    """``bin/trace_run`` on a Dopuvik folder: two requests together, then decoded together, one ending early."""
    model_dir = make_model(tmp_path, "small", dtype)
    a, b = random_tokens(40, vocab("small"), seed=5), random_tokens(71, vocab("small"), seed=6)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:37], "want": [0, 36]},
                                     {"id": "b", "tokens": b[:68], "want": [67]}], "end": []}]
    for k in range(3):
        steps.append({"step": k + 1, "entries": [{"id": "a", "tokens": [a[37 + k]], "want": [0]},
                                                 {"id": "b", "tokens": [b[68 + k]], "want": [] if k == 1 else [0]}],
                      "end": ["a", "b"] if k == 2 else []})
    out_dir = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", "192"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb = reference(model_dir, a), reference(model_dir, b)
    V = vocab("small")

    def read(i):
        return torch.frombuffer(bytearray(open(out_dir / f"{i}.f32", "rb").read()), dtype=torch.float32).reshape(-1, V)
    close(read(0), torch.stack([ra[0], ra[36], rb[67]]), dtype, "small", "trace step 0")
    close(read(1), torch.stack([ra[37], rb[68]]), dtype, "small", "trace step 1")
    close(read(2), torch.stack([ra[38]]), dtype, "small", "trace step 2")
    close(read(3), torch.stack([ra[39], rb[70]]), dtype, "small", "trace step 3")
