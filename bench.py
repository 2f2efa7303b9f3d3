#!/usr/bin/env python3
"""Benchmark: decode tokens per second of a Llama shape with random bf16 weights, through ``Engine.generate``.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--shape 1b|3b|8b]
    python bench.py --design ramupel [--size s|m|l] [--layers N]      (the hybrid design beside Llama at equal size)
    python bench.py --design botuvik [--size s|m|l] [--layers N]      (the same for the Botuvik design, beside both)
    python bench.py --design zasitar [--size s|m|l] [--layers N]      (the Zasitar design beside Botuvik and Llama)
    python bench.py --design dopuvik [--size s|m|l] [--layers N]      (the Dopuvik design beside Zasitar and Llama)

One "step" is one decode step of the whole batch. The default run has the Llama-3.2-1B shape, a batch of 8
sequences with 512-token prompts in a cache sized for a context of 4096. Every figure comes from the library's
own generation loop (host token ids in, host token ids out): one generation call per measured point, whose first W
decode steps are warm-up and whose following decode steps are timed in laps of exactly K steps; the median over
the laps is reported. It prints ONE JSON line:

* ``value``: decoded tokens per second of a lap of K steps on the device's clock (CUDA events at the lap's
  boundaries), ``e2e``: the same laps on the host's clock;
* ``prefill``: one 2,048-token prompt; ``roofline``: the bytes a decode step must read over its time against
  the HBM peak; ``points``: decode at batch 1 and 64, and at contexts of about 1,024 / 2,048 / 3,584 for
  batches of 1, 8 and 64, with ``points_detail`` giving ms per step, bytes and the HBM fraction of each.

``--shape 3b`` / ``8b`` run the other two shapes the baseline names (batch 16 with prompts of 64 to 1,024 tokens
and 256 steps; batch 32 with 2,048-token prompts and 512 steps) unless ``--steps`` says otherwise.
``--profile`` adds the device time per section of the model walk (a separate, short run in profile mode).

``--design ramupel`` measures something else and leaves the default workload alone: prefill (one 2,048-token prompt)
and decode (batch 8 from 512-token prompts) throughput of the Ramupel design at a few layer sizes, beside a Llama of
the same width, depth, head count and feed-forward parameters, both with random weights, plus the device time per
section of the model walk of each and what the mixers' core kernels reach of their rooflines.
``--design botuvik`` does the same for the Botuvik design (matrix-memory layers, capped attention with sinks, dense
and routed feed-forwards) beside Ramupel, the closest existing design (a recurrence among attention layers), and Llama.
``--design dopuvik`` does the same for the Dopuvik design (state-space layers, latent attention in a window, attention
with kept first tokens beside a gated delta rule, experts chosen in groups with identity experts) beside Zasitar, the
closest existing design (a recurrence among windowed attention layers, routed experts), and Llama.
``--design zasitar`` does the same for the Zasitar design (time-mixing layers, sliding-window attention with normed
heads and keys shared between layers, results normed behind the sublayers) beside Botuvik, the closest existing design
(a matrix recurrence among attention layers with sinks, dense and routed feed-forwards), and Llama.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def llama_shape(layers, hidden, heads, kv_heads, head_dim, ffn, factor, tied):
    return {
        "architectures": ["LlamaForCausalLM"], "num_hidden_layers": layers, "hidden_size": hidden,
        "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim,
        "intermediate_size": ffn, "vocab_size": 128256, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 8192},
        "rms_norm_eps": 1e-5, "tie_word_embeddings": tied, "max_position_embeddings": 131072,
        "torch_dtype": "bfloat16",
    }


# name -> (config.json keys, seed, batch, prompt lengths (lo, hi), decode steps, context the cache is sized for)
SHAPES = {
    "1b": ("Llama-3.2-1B shape", llama_shape(16, 2048, 32, 8, 64, 8192, 32.0, True), 2, 8, (512, 512), 256, 4096),
    "3b": ("Llama-3.2-3B shape", llama_shape(28, 3072, 24, 8, 128, 8192, 32.0, True), 3, 16, (64, 1024), 256, 1280),
    "8b": ("Llama-3.1-8B shape", llama_shape(32, 4096, 32, 8, 128, 14336, 8.0, False), 4, 32, (2048, 2048), 512, 2560),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
REPEATS = 5


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            raw = json.load(fh)
        return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])),
                "source": "measured"}
    except (OSError, ValueError, KeyError):
        return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi for the whole run; a window of the samples
    (by wall-clock time) is summarised for each measured point."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def window(self, begin, end):
        sm, mx, reasons = [], [], set()
        for stamp, row in list(self.rows):
            if not begin - 0.05 <= stamp <= end + 0.15 or len(row) < 6:
                continue
            try:
                sm.append(float(row[0]))
                mx.append(float(row[1]))
            except ValueError:
                continue
            for name, cell in zip(self.NAMES, row[2:6]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def layer_weights(cfg):
    d, F = cfg["hidden_size"], cfg["intermediate_size"]
    H, G, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    return H * hd * d + 2 * G * hd * d + d * H * hd + 3 * d * F


def decode_bytes(cfg, layers, cached_tokens):
    """Bytes one decode step has to read: every weight it uses once (the layers and the head; of the embedding
    only the gathered rows, which are not counted) and the keys and values of the live requests."""
    G, hd = cfg["num_key_value_heads"], cfg["head_dim"]
    weights = (layers * layer_weights(cfg) + cfg["vocab_size"] * cfg["hidden_size"]) * 2
    return weights + cached_tokens * layers * 2 * G * hd * 2


def prefill_flops(cfg, layers, lengths):
    H, hd = cfg["num_attention_heads"], cfg["head_dim"]
    tokens = sum(lengths)
    attention = layers * sum(2 * H * hd * n * n for n in lengths)          # causal: half of 4 H hd n^2
    return 2.0 * layers * layer_weights(cfg) * tokens + attention + 2.0 * cfg["vocab_size"] * cfg["hidden_size"] * len(lengths)


# ------------------------------------------------------------------ the hybrid design beside Llama
# name -> (width, heads, latent (dim, rot_dim, vdim, kv_rank), gla (heads, dim, vdim), feed-forward width)
HYBRID_SIZES = {
    "s": (1024, 8, (64, 32, 64, 256), (4, 64, 256), 4096),
    "m": (2048, 16, (128, 64, 128, 512), (8, 128, 256), 8192),
    "l": (4096, 32, (128, 64, 128, 512), (16, 128, 256), 14336),
}


def hybrid_configs(size, layers):
    width, heads, (dn, dr, dv, rank), (gh, gk, gv), ff = HYBRID_SIZES[size]
    latent = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": ff},
              "mixer": {"heads": heads, "dim": dn, "rot_dim": dr, "vdim": dv, "kv_rank": rank, "scale": (dn + dr) ** -0.5,
                        "rot": {"base": 10000.0, "dims": dr}}}
    gla = {"type": "gla", "mlp": {"kind": "dense", "ff": ff}, "mixer": {"heads": gh, "dim": gk, "vdim": gv, "tau": 16.0}}
    ramupel = {"architecture": "Ramupel", "vocab": 32000, "width": width, "embedding": {"scale": float(width) ** 0.5},
               "norm": {"eps": 1e-5}, "layers": [gla if i % 4 == 0 else latent for i in range(layers)]}
    # the same feed-forward parameters in three matrices instead of two
    llama = llama_shape(layers, width, heads, max(1, heads // 4), width // heads, (2 * ff // 3 + 127) // 128 * 128, 8.0, True)
    llama["vocab_size"] = 32000
    return ramupel, llama


def botuvik_config(size, layers):
    """Every fourth layer a matrix memory, the others capped attention with a sink (grouped as in the Llama beside
    it); dense and routed feed-forwards alternate (8 experts of a quarter of the dense width in 4 groups, 2 of 2 groups
    chosen, plus a shared expert of that size)."""
    width, heads, _, (gh, gk, gv), ff = HYBRID_SIZES[size]
    hd = width // heads
    attention = {"type": "attention", "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": hd, "vdim": hd,
                                                "scale": hd ** -0.5 * 4.0, "softcap": 30.0, "rot": {"base": 10000.0, "dims": hd}}}
    memory = {"type": "mlstm", "mixer": {"heads": gh, "dim": gk, "vdim": gv, "gate_cap": 15.0}}
    dense = {"kind": "dense", "ff": ff}
    routed = {"kind": "moe", "expert": {"ff": ff // 4}, "shared": {"ff": ff // 4},
              "router": {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 2}}}
    return {"architecture": "Botuvik", "vocab": 32000, "width": width, "norm": {"eps": 1e-5},
            "layers": [dict(memory if i % 4 == 0 else attention, mlp=routed if i % 2 else dense) for i in range(layers)]}


ZASITAR_WINDOW = 1024          # half of the measured prompt: the window's edge passes through the prompt kernels' tiles


def zasitar_config(size, layers):
    """Every fourth layer time mixing (heads of 64 channels over the whole width), the others attention over a window
    of ZASITAR_WINDOW tokens (grouped as in the Llama beside it, rotation over half of each head); of every four
    layers the third attends over the second's keys and values; dense and routed feed-forwards alternate as in the
    Botuvik beside it (8 experts of a quarter of the dense width, 2 chosen, plus a gated shared expert of that size)."""
    width, heads, _, _, ff = HYBRID_SIZES[size]
    hd = width // heads
    mixer = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": hd, "vdim": hd, "scale": hd ** -0.5,
             "mask": {"size": ZASITAR_WINDOW},
             "rot": {"base": 500000.0, "dims": hd // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    time_mix = {"type": "wkv", "mixer": {"heads": width // 64, "dim": 64}}
    dense = {"kind": "dense", "ff": ff}
    routed = {"kind": "moe", "expert": {"ff": ff // 4, "limit": 7.0}, "shared": {"ff": ff // 4, "limit": 7.0},
              "router": {"experts": 8, "top": 2}}
    out = []
    for i in range(layers):
        if i % 4 == 0:
            layer = dict(time_mix)
        else:
            layer = {"type": "attention", "mixer": dict(mixer, kv_from=i - 1) if i % 4 == 2 else dict(mixer)}
        out.append(dict(layer, mlp=routed if i % 2 else dense))
    return {"architecture": "Zasitar", "vocab": 32000, "width": width, "norm": {"eps": 1e-5}, "layers": out}


DOPUVIK_WINDOW, DOPUVIK_KEEP = 1024, 4


def dopuvik_config(size, layers):
    """Of every four layers the first is a state space (heads of 64 values over twice the width, states of 128, a
    convolution of 4 taps), the second and fourth latent attention (the sizes of the Ramupel design's latent layers,
    queries through a latent of 1.5 x the key / value rank, a window of DOPUVIK_WINDOW tokens, stretched rotation), the
    third attention (grouped as in the Llama beside it, the same window plus DOPUVIK_KEEP kept first tokens) beside a
    gated delta rule (as many heads of dim x dim as the Ramupel design's linear attention has, convolutions of 4 taps).
    Every feed-forward is routed: 8 experts of a quarter of the dense width and 2 identities in 5 groups of which 3 are
    kept, 2 chosen (the Zasitar beside it routes every second layer's and has a shared expert instead)."""
    width, heads, (dn, dr, dv, rank), (gh, gk, _), ff = HYBRID_SIZES[size]
    hd = width // heads
    space = {"type": "mamba2", "mixer": {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 1, "conv": 4, "norm_groups": 1}}
    latent = {"type": "latent_attention",
              "mixer": {"heads": heads, "dim": dn, "rot_dim": dr, "vdim": dv, "kv_rank": rank, "q_rank": 3 * rank // 2,
                        "scale": (dn + dr) ** -0.5, "mask": {"size": DOPUVIK_WINDOW},
                        "rot": {"base": 10000.0, "dims": dr, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    pair = {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": hd, "vdim": hd, "scale": hd ** -0.5,
                               "mask": {"size": DOPUVIK_WINDOW, "keep_first": DOPUVIK_KEEP}, "rot": {"base": 10000.0, "dims": hd}},
                      "right": {"heads": gh, "kv_heads": gh, "dim": gk, "vdim": gk, "conv": 4},
                      "left_scale": 1.0, "right_scale": 1.0}}
    routed = {"kind": "moe", "expert": {"ff": ff // 4},
              "router": {"experts": 8, "identity": 2, "top": 2, "scale": 1.0, "groups": {"count": 5, "keep": 3}}}
    order = (space, latent, pair, latent)
    return {"architecture": "Dopuvik", "vocab": 32000, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "logit_scale": 1.0, "layers": [dict(order[i % 4], mlp=routed) for i in range(layers)]}


def compare_designs(args, peaks) -> int:
    import torch
    from llmplayer_b200 import Engine
    from llmplayer_b200.config import config_from_dict
    from llmplayer_b200.sampling import SamplerConfig
    from llmplayer_b200.weights import write_random_model
    layers = args.layers or 4
    repeats = max(1, args.repeats)
    steps = args.steps or 64
    warmup = max(3, args.warmup)
    prompt, batch, prefill_len = args.prompt_len or 512, args.batch or 8, 2048
    context = max(prefill_len, prompt + warmup + repeats * steps + 2)
    gen = torch.Generator().manual_seed(5)
    clocks = ClockSampler()
    clocks.start()
    botuvik, zasitar, dopuvik = args.design == "botuvik", args.design == "zasitar", args.design == "dopuvik"
    title = {"botuvik": "Botuvik design beside Ramupel and ", "zasitar": "Zasitar design beside Botuvik and ",
             "ramupel": "Ramupel design beside ", "dopuvik": "Dopuvik design beside Zasitar and "}[args.design]
    out = {"metric": f"prefill and decode tok/s of the {title}Llama at equal size (bf16)", "impl": "ours",
           "layers": layers, "batch": batch, "prompt_len": prompt, "prefill_len": prefill_len, "peaks": peaks, "sizes": {}}
    try:
        for size in ([args.size] if args.size else sorted(HYBRID_SIZES, key="sml".index)):
            row = {}
            designs = list(zip(("ramupel", "llama"), hybrid_configs(size, layers)))
            if botuvik:
                designs.insert(0, ("botuvik", botuvik_config(size, layers)))
            if zasitar:
                designs = [("zasitar", zasitar_config(size, layers)), ("botuvik", botuvik_config(size, layers)), designs[1]]
            if dopuvik:
                designs = [("dopuvik", dopuvik_config(size, layers)), ("zasitar", zasitar_config(size, layers)), designs[1]]
            for name, raw in designs:
                vocab = raw.get("vocab", raw.get("vocab_size"))
                tmp = tempfile.mkdtemp(prefix="llmplayer_b200_bench_")
                try:
                    write_random_model(config_from_dict(raw), 7, tmp, dtype="bfloat16")
                    engine = Engine.load(tmp, dtype="bfloat16", context_length=context, max_batch=batch)
                    profiled = Engine.load(tmp, dtype="bfloat16", context_length=context, max_batch=batch, profile=True)
                finally:
                    shutil.rmtree(tmp, ignore_errors=True)

                def tokens(n):
                    return torch.randint(0, vocab, (n,), generator=gen).tolist()
                begin = time.time()
                times = []
                long_prompt = tokens(prefill_len)
                for i in range(2 + repeats):
                    slot = engine.acquire()
                    torch.cuda.synchronize()
                    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    start.record()
                    engine.step([(slot, long_prompt)], [[prefill_len - 1]])
                    stop.record()
                    torch.cuda.synchronize()
                    engine.release(slot)
                    if i >= 2:
                        times.append(start.elapsed_time(stop))
                prefill_ms = statistics.median(times)
                ps = [tokens(prompt) for _ in range(batch)]
                engine.generate(ps, SamplerConfig.greedy(), max_tokens=warmup + repeats * steps + 1, stop_token_ids=(),
                                laps=(warmup, steps))
                laps = engine.last_generation_stats.laps
                decode_ms = statistics.median(lap["device_ms"] / lap["steps"] for lap in laps)
                engine.check()
                end = time.time()
                # sections: one prompt alone, then decode steps alone (profile mode: no graphs, no overlap)
                slot = profiled.acquire()
                profiled.step([(slot, long_prompt)], [[prefill_len - 1]])
                profiled.release(slot)
                profiled.profile_report(reset=True)
                slot = profiled.acquire()
                profiled.step([(slot, long_prompt)], [[prefill_len - 1]])
                profiled.release(slot)
                pre = profiled.profile_report(reset=True)
                slots = [profiled.acquire() for _ in ps]
                profiled.step(list(zip(slots, ps)), [[prompt - 1]] * batch)
                for _ in range(4):
                    profiled.step([(s, [1]) for s in slots], [[0]] * batch)
                profiled.profile_report(reset=True)
                for _ in range(16):
                    profiled.step([(s, [1]) for s in slots], [[0]] * batch)
                dec = profiled.profile_report(reset=True)
                row[name] = {
                    "prefill_tok_s": prefill_len / (prefill_ms / 1e3), "prefill_ms": prefill_ms,
                    "decode_tok_s": batch / (decode_ms / 1e3), "decode_ms_per_step": decode_ms,
                    "clocks": clocks.window(begin, end),
                    "prefill_sections_ms": {k: round(v["ms_per_step"], 4) for k, v in pre["sections"].items()},
                    "decode_sections_ms": {k: round(v["ms_per_step"], 4) for k, v in dec["sections"].items()},
                }
                del engine, profiled
                torch.cuda.empty_cache()
            row["rooflines"] = {} if zasitar or dopuvik else hybrid_rooflines(size, layers, row, peaks, batch, prompt + 10, prefill_len)
            if dopuvik:
                row["rooflines"].update(dopuvik_rooflines(size, layers, row, peaks, batch, prompt + 10, prefill_len))
            if botuvik or zasitar:
                row["rooflines"].update(botuvik_rooflines(size, layers, row, peaks, batch, prompt + 10, prefill_len))
            if zasitar:
                row["rooflines"].update(zasitar_rooflines(size, layers, row, peaks, batch, prompt + 10, prefill_len))
            out["sizes"][size] = row
        print(json.dumps(out))
        return 0
    finally:
        clocks.stop()


def hybrid_rooflines(size, layers, row, peaks, batch, context, n):
    """What the mixers' core kernels reach of their rooflines, per layer that has them: prompt kernels against the
    bf16 tensor peak (algorithmic FLOPs / time), decode kernels against the copy bandwidth (bytes they must read)."""
    width, heads, (dn, dr, dv, rank), (gh, gk, gv), ff = HYBRID_SIZES[size]
    n_gla = sum(1 for i in range(layers) if i % 4 == 0)
    n_lat = layers - n_gla
    flops, gbs = peaks["bf16_tflops"] * 1e12, peaks["hbm_gbs"] * 1e9
    r, l = row["ramupel"], row["llama"]
    hd, G = width // heads, max(1, heads // 4)
    out = {}

    def frac(work, ms, count, peak):
        return None if not ms or not count else work / (ms / count / 1e3) / peak
    # prompt attention: causal scores and weighted sums (the latent layers in the form they run in for prompts:
    # per head, keys of dim + rot_dim and values of vdim)
    out["prefill latent attention (of tensor peak)"] = frac(
        heads * n * (n + 1) * ((dn + dr) + dv), r["prefill_sections_ms"].get("attention.scores"), n_lat, flops)
    out["prefill llama attention (of tensor peak)"] = frac(
        heads * n * (n + 1) * 2 * hd, l["prefill_sections_ms"].get("attention.scores"), layers, flops)
    out["prefill gla recurrence (of tensor peak)"] = frac(
        6.0 * gh * gk * gv * n, r["prefill_sections_ms"].get("recurrence.scan"), n_gla, flops)
    # decode: the cached rows / keys and values / states that must be read (and states written)
    out["decode latent attention (of copy bandwidth)"] = frac(
        batch * context * (rank + dr) * 2, r["decode_sections_ms"].get("attention.scores"), n_lat, gbs)
    out["decode llama attention (of copy bandwidth)"] = frac(
        batch * context * 2 * G * hd * 2, l["decode_sections_ms"].get("attention.scores"), layers, gbs)
    out["decode gla recurrence (of copy bandwidth)"] = frac(
        batch * gh * gk * gv * 4 * 2, r["decode_sections_ms"].get("recurrence.scan"), n_gla, gbs)
    return out


def botuvik_rooflines(size, layers, row, peaks, batch, context, n):
    """The Botuvik kernels that have no twin in the products (which are the same kernels for every design): prompt
    kernels against the bf16 tensor peak, decode kernels against the copy bandwidth."""
    width, heads, _, (gh, gk, gv), ff = HYBRID_SIZES[size]
    n_mem = sum(1 for i in range(layers) if i % 4 == 0)
    n_att = layers - n_mem
    n_routed = sum(1 for i in range(layers) if i % 2)
    flops, gbs = peaks["bf16_tflops"] * 1e12, peaks["hbm_gbs"] * 1e9
    b = row["botuvik"]
    hd, G = width // heads, max(1, heads // 4)

    def frac(work, ms, count, peak):
        return None if not ms or not count else work / (ms / count / 1e3) / peak
    routed_rows = 8 * (ff // 4) + ff // 4
    return {
        "prefill botuvik attention (of tensor peak)": frac(
            heads * n * (n + 1) * 2 * hd, b["prefill_sections_ms"].get("attention.scores"), n_att, flops),
        "prefill botuvik recurrence (of tensor peak)": frac(
            6.0 * gh * gk * (gv + 1) * n, b["prefill_sections_ms"].get("recurrence.scan"), n_mem, flops),
        "prefill botuvik routed gate/up product, all experts (of tensor peak)": frac(
            2.0 * n * width * 2 * routed_rows, b["prefill_sections_ms"].get("ffn.gate_up"), n_routed, flops),
        "decode botuvik attention (of copy bandwidth)": frac(
            batch * context * 2 * G * hd * 2, b["decode_sections_ms"].get("attention.scores"), n_att, gbs),
        "decode botuvik recurrence (of copy bandwidth)": frac(
            batch * gh * gk * (gv + 1) * 4 * 2, b["decode_sections_ms"].get("recurrence.scan"), n_mem, gbs),
    }


def zasitar_rooflines(size, layers, row, peaks, batch, context, n):
    """The Zasitar kernels beside their Botuvik twins (``botuvik_rooflines``): prompt kernels against the bf16 tensor
    peak, decode and elementwise kernels against the copy bandwidth. A windowed layer's work counts the keys inside
    the window only."""
    width, heads, _, _, ff = HYBRID_SIZES[size]
    n_mix = sum(1 for i in range(layers) if i % 4 == 0)
    n_att = layers - n_mix
    n_routed = sum(1 for i in range(layers) if i % 2)
    flops, gbs = peaks["bf16_tflops"] * 1e12, peaks["hbm_gbs"] * 1e9
    z = row["zasitar"]
    hd, G, W = width // heads, max(1, heads // 4), ZASITAR_WINDOW
    th, tn = width // 64, 64

    def frac(work, ms, count, peak):
        return None if not ms or not count else work / (ms / count / 1e3) / peak
    seen = sum(min(i + 1, W) for i in range(n))                  # (query, key) pairs inside the window
    routed_rows = 8 * (ff // 4) + ff // 4
    pre, dec = z["prefill_sections_ms"], z["decode_sections_ms"]
    out = {
        "prefill zasitar attention, keys in the window (of tensor peak)": frac(heads * seen * 4 * hd, pre.get("attention.scores"), n_att, flops),
        "prefill zasitar recurrence (of tensor peak)": frac(6.0 * th * tn * tn * n, pre.get("recurrence.scan"), n_mix, flops),
        "prefill zasitar routed gate/up product, all experts (of tensor peak)": frac(
            2.0 * n * width * 2 * routed_rows, pre.get("ffn.gate_up"), n_routed, flops),
        "decode zasitar attention (of copy bandwidth)": frac(
            batch * min(context, W) * 2 * G * hd * 2, dec.get("attention.scores"), n_att, gbs),
        "decode zasitar recurrence (of copy bandwidth)": frac(batch * th * tn * tn * 4 * 2, dec.get("recurrence.scan"), n_mix, gbs),
        # the kernel behind every sublayer: reads the sublayer's float32 result and the float32 stream, writes the
        # stream and its bfloat16 copy (two per layer that has a feed-forward)
        "prefill zasitar norm behind a sublayer (of copy bandwidth)": frac(n * width * (4 + 4 + 4 + 2), pre.get("norm"), 2 * layers, gbs),
        # blends of neighbouring tokens: reads the stream, writes five bfloat16 blends
        "prefill zasitar token blends (of copy bandwidth)": frac(n * width * (4 + 5 * 2), pre.get("recurrence.shift"), n_mix, gbs),
    }
    b, l = row.get("botuvik"), row.get("llama")
    if b is not None:
        out["prefill botuvik norm behind a sublayer (of copy bandwidth)"] = frac(
            n * width * (4 + 4 + 4 + 2), b["prefill_sections_ms"].get("norm"), 2 * layers, gbs)
    if l is not None:
        out["prefill llama attention (of tensor peak)"] = frac(
            heads * n * (n + 1) * 2 * hd, l["prefill_sections_ms"].get("attention.scores"), layers, flops)
        out["decode llama attention (of copy bandwidth)"] = frac(
            batch * context * 2 * G * hd * 2, l["decode_sections_ms"].get("attention.scores"), layers, gbs)
    return out


def dopuvik_rooflines(size, layers, row, peaks, batch, context, n):
    """The Dopuvik kernels beside their Zasitar (and Llama) twins: prompt kernels against the bf16 tensor peak, decode
    and elementwise kernels against the copy bandwidth. A windowed layer's work counts the keys inside the window (and
    the kept first tokens) only."""
    width, heads, (dn, dr, dv, rank), (gh, gk, _), ff = HYBRID_SIZES[size]
    kinds = [i % 4 for i in range(layers)]
    n_space, n_lat, n_pair = kinds.count(0), kinds.count(1) + kinds.count(3), kinds.count(2)
    flops, gbs = peaks["bf16_tflops"] * 1e12, peaks["hbm_gbs"] * 1e9
    d, z, l = row["dopuvik"], row.get("zasitar"), row.get("llama")
    hd, G, W, K = width // heads, max(1, heads // 4), DOPUVIK_WINDOW, DOPUVIK_KEEP
    sh, sp, sn = 2 * width // 64, 64, 128

    def frac(work, ms, count, peak):
        return None if not ms or not count else work / (ms / count / 1e3) / peak
    seen = sum(min(i + 1, W) for i in range(n))                                   # (query, key) pairs inside the window
    seen_kept = seen + sum(min(K, max(0, i + 1 - W)) for i in range(n))           # and the kept first tokens behind it
    routed_rows = 8 * (ff // 4)
    pre, dec = d["prefill_sections_ms"], d["decode_sections_ms"]
    out = {
        "prefill dopuvik latent attention, keys in the window (of tensor peak)": frac(
            heads * seen * 2 * ((dn + dr) + dv), pre.get("attention.scores"), n_lat, flops),
        "prefill dopuvik attention with kept tokens, keys seen (of tensor peak)": frac(
            heads * seen_kept * 4 * hd, pre.get("left.attention.scores"), n_pair, flops),
        "prefill dopuvik state-space recurrence (of tensor peak)": frac(6.0 * sh * sn * sp * n, pre.get("recurrence.scan"), n_space, flops),
        "prefill dopuvik delta-rule recurrence (of tensor peak)": frac(8.0 * gh * gk * gk * n, pre.get("right.recurrence.scan"), n_pair, flops),
        "prefill dopuvik routed gate/up product, all experts (of tensor peak)": frac(
            2.0 * n * width * 2 * routed_rows, pre.get("ffn.gate_up"), layers, flops),
        "prefill dopuvik short convolutions (of copy bandwidth)": frac(
            n * (2 * width + 2 * sn) * 8, pre.get("recurrence.conv"), n_space, gbs),
        "decode dopuvik latent attention (of copy bandwidth)": frac(
            batch * min(context, W) * (rank + dr) * 2, dec.get("attention.scores"), n_lat, gbs),
        "decode dopuvik attention with kept tokens (of copy bandwidth)": frac(
            batch * min(context, W + K) * 2 * G * hd * 2, dec.get("left.attention.scores"), n_pair, gbs),
        "decode dopuvik state-space recurrence (of copy bandwidth)": frac(batch * sh * sn * sp * 4 * 2, dec.get("recurrence.scan"), n_space, gbs),
        "decode dopuvik delta-rule recurrence (of copy bandwidth)": frac(batch * gh * gk * gk * 4 * 2, dec.get("right.recurrence.scan"), n_pair, gbs),
    }
    if z is not None:
        zh, zn = width // 64, 64
        zpre, zdec = z["prefill_sections_ms"], z["decode_sections_ms"]
        z_att = sum(1 for i in range(layers) if i % 4)
        z_mix = layers - z_att
        out["prefill zasitar attention, keys in the window (of tensor peak)"] = frac(heads * seen * 4 * hd, zpre.get("attention.scores"), z_att, flops)
        out["prefill zasitar recurrence (of tensor peak)"] = frac(6.0 * zh * zn * zn * n, zpre.get("recurrence.scan"), z_mix, flops)
        out["prefill zasitar routed gate/up product, all experts (of tensor peak)"] = frac(
            2.0 * n * width * 2 * (8 * (ff // 4) + ff // 4), zpre.get("ffn.gate_up"), sum(1 for i in range(layers) if i % 2), flops)
        out["decode zasitar attention (of copy bandwidth)"] = frac(
            batch * min(context, ZASITAR_WINDOW) * 2 * G * hd * 2, zdec.get("attention.scores"), z_att, gbs)
        out["decode zasitar recurrence (of copy bandwidth)"] = frac(batch * zh * zn * zn * 4 * 2, zdec.get("recurrence.scan"), z_mix, gbs)
    if l is not None:
        out["prefill llama attention (of tensor peak)"] = frac(
            heads * n * (n + 1) * 2 * hd, l["prefill_sections_ms"].get("attention.scores"), layers, flops)
        out["decode llama attention (of copy bandwidth)"] = frac(
            batch * context * 2 * G * hd * 2, l["decode_sections_ms"].get("attention.scores"), layers, gbs)
    return out


def spread(values):
    return {"median": statistics.median(values), "min": min(values), "max": max(values), "repeats": len(values)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--shape", default="1b", choices=sorted(SHAPES))
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--context", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (both are reported)")
    ap.add_argument("--repeats", type=int, default=REPEATS)
    ap.add_argument("--no-points", action="store_true", help="skip the other batches and contexts and the prefill")
    ap.add_argument("--prefill-only", action="store_true",
                    help="measure only the 2,048-token prefill (small runs for profiling)")
    ap.add_argument("--profile", action="store_true", help="add the device time per section of the model walk")
    ap.add_argument("--design", default="llama", choices=("llama", "ramupel", "botuvik", "zasitar", "dopuvik"),
                    help="ramupel / botuvik / zasitar / dopuvik: that design beside the closest others at equal size (another workload; see "
                         "the module text)")
    ap.add_argument("--size", default=None, choices=sorted(HYBRID_SIZES), help="with --design ramupel / botuvik / zasitar: one size only")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "DenzoSOFTHub/LLMPlayer is a Java/Maven project: pip finds neither setup.py nor "
                          "pyproject.toml, and this image has no JVM to run it"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported by this single-GPU library")
        return 2
    if args.design in ("ramupel", "botuvik", "zasitar", "dopuvik"):
        return compare_designs(args, load_peaks())
    args.warmup = max(3, args.warmup)
    repeats = max(1, args.repeats)

    import torch
    from llmplayer_b200 import Engine
    from llmplayer_b200.config import config_from_dict
    from llmplayer_b200.sampling import SamplerConfig
    from llmplayer_b200.weights import write_random_model

    peaks = load_peaks()
    title, base, seed, batch0, (len_lo, len_hi), steps0, context0 = SHAPES[args.shape]
    cfg = dict(base)
    model_layers = cfg["num_hidden_layers"]
    layers = args.layers or model_layers
    cfg["num_hidden_layers"] = layers
    batch = args.batch or batch0
    steps = args.steps or steps0
    if args.prompt_len:
        len_lo = len_hi = args.prompt_len
    context = args.context or max(context0, len_hi + args.warmup + repeats * steps + 2)
    main_shape = args.shape == "1b"
    with_points = main_shape and not args.no_points and not args.prefill_only
    tmp = tempfile.mkdtemp(prefix="llmplayer_b200_bench_")
    try:
        write_random_model(config_from_dict(cfg), seed, tmp, dtype="bfloat16")
        max_batch = 1 if args.prefill_only else max(batch, 64 if with_points else 1)
        engine = Engine.load(tmp, dtype="bfloat16", context_length=context, max_batch=max_batch)
        profiled = Engine.load(tmp, dtype="bfloat16", context_length=context, max_batch=batch, profile=True) \
            if args.profile else None
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    gen = torch.Generator().manual_seed(seed)
    clocks = ClockSampler()
    clocks.start()

    def prompts(count, lo, hi):
        lengths = [lo] * count if lo == hi else torch.randint(lo, hi + 1, (count,), generator=gen).tolist()
        return [torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist() for n in lengths]

    greedy = SamplerConfig.greedy()

    def timed_decode(count, lo, hi, k, warmup, sampler=greedy):
        """One generation call through Engine.generate: the prompts, `warmup` untimed decode steps, then
        `repeats` laps of exactly k decode steps each, timed on the device (CUDA events at the lap boundaries) and
        on the host; the medians over the laps are reported."""
        ps = prompts(count, lo, hi)
        begin = time.time()
        engine.generate(ps, sampler, max_tokens=warmup + repeats * k + 1, stop_token_ids=(), laps=(warmup, k))
        end = time.time()
        laps = engine.last_generation_stats.laps
        assert len(laps) == repeats and all(lap["steps"] == k and lap["tokens"] == count * k for lap in laps), laps
        device = [lap["tokens"] / (lap["device_ms"] / 1e3) for lap in laps]
        host = [lap["tokens"] / (lap["host_ms"] / 1e3) for lap in laps]
        tok_s = statistics.median(device)
        ms = count / tok_s * 1e3
        cached = sum(len(p) for p in ps) + count * (warmup + repeats * k // 2)      # the live requests' cache, mid-run
        nbytes = decode_bytes(cfg, layers, cached)
        return {"tok_s": tok_s, "ms_per_step": ms, "e2e_tok_s": statistics.median(host),
                "launches": int(statistics.median(lap.get("launches", 0) for lap in laps)),
                "context_mid": cached // count, "gb_per_step": nbytes / 1e9,
                "hbm_frac": nbytes / (ms / 1e3) / 1e9 / peaks["hbm_gbs"],
                "spread_tok_s": spread(device), "clocks": clocks.window(begin, end),
                "h2d": engine.last_step_h2d_bytes, "d2h": engine.last_step_d2h_bytes}

    def timed_prefill(lengths):
        ps = [torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist() for n in lengths]
        times = []
        for i in range(2 + repeats):                  # two warm-up passes
            slots = [engine.acquire() for _ in ps]
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.step(list(zip(slots, ps)), [[len(p) - 1] for p in ps])
            stop.record()
            torch.cuda.synchronize()
            for s in slots:
                engine.release(s)
            if i >= 2:
                times.append(start.elapsed_time(stop))
        ms = statistics.median(times)
        tokens = sum(lengths)
        return {"value": tokens / (ms / 1e3), "tokens": tokens, "ms": ms,
                "frac": prefill_flops(cfg, layers, lengths) / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12),
                "of": peaks["source"], "spread_ms": spread(times)}

    try:
        if args.prefill_only:
            print(json.dumps({"metric": f"prefill tok/s ({title}, bf16)", "impl": "ours", "layers": layers,
                              "model_layers": model_layers, "prefill": timed_prefill([2048])}))
            return 0

        run = timed_decode(batch, len_lo, len_hi, steps, args.warmup)
        result = {
            "metric": "decode tok/s (%s, bf16, batch %d)" % (title, batch),
            "value": run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
            "ms_per_step": run["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic: seeded random weights N(0, 0.02) and uniform random token ids",
            "impl": "ours",
            "config": {
                "model": title, "layers": layers, "model_layers": model_layers, "hidden_size": cfg["hidden_size"],
                "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                "head_dim": cfg["head_dim"], "intermediate_size": cfg["intermediate_size"],
                "vocab_size": cfg["vocab_size"], "global_batch": batch, "seq_len": context,
                "prompt_len": len_lo if len_lo == len_hi else f"{len_lo}-{len_hi}",
                "decode_context_mid": run["context_mid"], "parallelism": "single GPU",
                "l2": "inputs larger than L2 (a step reads %.2f GB)" % run["gb_per_step"],
                "peaks": peaks["source"], "repeats": repeats, "timed": "median over laps of K decode steps inside one "
                "Engine.generate call, CUDA events",
            },
            "clocks": run["clocks"],
            "e2e": {"value": run["e2e_tok_s"], "unit": "tokens/s", "h2d_bytes_per_step": run["h2d"],
                    "d2h_bytes_per_step": run["d2h"]},
            "gpu_launches": int(run["launches"]),
            "roofline": {"bound": "hbm", "achieved": run["hbm_frac"] * peaks["hbm_gbs"], "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": run["hbm_frac"], "of": peaks["source"]},
            "spread": run["spread_tok_s"],
        }
        if not main_shape and not args.no_points:
            # the other shapes: the prompts of the run itself, processed in one step
            lengths = [len(p) for p in prompts(batch, len_lo, len_hi)]
            result["prefill"] = timed_prefill(lengths)
        if with_points:
            result["prefill"] = timed_prefill([2048])
            points, detail = {}, {}

            def point(name, count, length, k, sampler=greedy):
                r = timed_decode(count, length, length, k, max(3, args.warmup // 2), sampler)
                points[name] = r["tok_s"]
                detail[name] = {key: r[key] for key in ("ms_per_step", "gb_per_step", "hbm_frac", "context_mid",
                                                        "e2e_tok_s", "spread_tok_s", "clocks")}
            k = max(16, steps // 2)
            for b in (1, 64):
                point(f"decode_b{b}", b, len_lo, k)
            warm = max(3, args.warmup // 2)
            for length in (1024, 2048, 3584):
                for b in (1, 8, 64):
                    # prompts such that the middle of the timed steps lies at this context, within the cache's 4096
                    kk = max(1, min(k, (2 * (context - 1 - length) - warm) // repeats))
                    point(f"decode_b{b}_ctx{length}", b, length - (warm + repeats * kk) // 2, kk)
            # the same entry point with the reference's default sampler (temperature 0.7, top-k 40, top-p 0.9,
            # repetition penalty 1.1) instead of the greedy choice: every step goes through the interpreter
            r = timed_decode(batch, len_lo, len_hi, k, max(3, args.warmup // 2), SamplerConfig(seed=1))
            points["e2e_reference_sampler"] = r["e2e_tok_s"]
            result["points"] = points
            result["points_detail"] = detail
        if profiled is not None:
            ps = prompts(batch, len_lo, len_hi)
            profiled.generate(ps, greedy, max_tokens=4, stop_token_ids=())
            profiled.profile_report(reset=True)
            profiled.generate(ps, greedy, max_tokens=1, stop_token_ids=())
            prefill_sections = profiled.profile_report(reset=True)
            profiled.generate(ps, greedy, max_tokens=min(steps, 32) + 1, stop_token_ids=())
            report = profiled.profile_report()
            result["profile"] = {"decode_and_prompt": report, "prompt_only": prefill_sections,
                                 "note": "sections timed with CUDA events in profile mode (no graphs, no overlap "
                                         "between kernels); the second entry is one call that stops after the prompt"}
        print(json.dumps(result))
        return 0
    finally:
        clocks.stop()


if __name__ == "__main__":
    sys.exit(main())
