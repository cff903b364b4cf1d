#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of the Qwen2.5-0.5B configuration (24
layers, hidden 896, 14 query heads, 2 KV heads, head size 64, intermediate
4864, vocabulary 151936, tied head) with random bfloat16 weights, a batch of 8
requests and contexts that end at 4096 tokens.  A "step" is one decode step of
the whole batch.  One JSON line is printed:

  value      decoded tokens per second: K calls of the engine's step(), the call a user
             makes, timed on the device with CUDA events on the engine's stream
             (median of three runs of K)
  e2e        the same K calls by the wall clock until the last tokens are on the host:
             every step the packed batch metadata goes up from pinned host memory and
             the sampled token ids come back to the host
  prefill    one prompt of 2,048 tokens in one step
  roofline   bytes the decode step has to read (every weight once, the cache of
             the live requests) / its time, against the measured copy bandwidth
  points     decode at batch 1 and 64 (points_roofline: their fractions of the HBM
             roofline), and the main batch with the engine's default options
  fp32       the 32-bit path's decode step at the same batch, for information

Inputs of a step (about 1.3 GB of weights and cache) are larger than the L2, so
no flush is needed between steps.

For profiling and for further sizes (one short line each, never the JSON line above):

    python bench.py --only decode|prefill|timeline|gemm|attention|serve [--batch B] [--layers L] [--context C] [--sizes 0.5b|1.5b|7b]

`serve` runs 64 concurrent requests (prompts of 128..4096 tokens in portions of 512 beside
decoding requests, 512 new tokens each) through the engine and reports wall-clock tokens a second.
The engine is the native one (csrc/engine); `timeline` and `gemm` use the kernels' Python face.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CONFIG_05B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 24, "hidden_size": 896, "num_attention_heads": 14, "num_key_value_heads": 2,
    "intermediate_size": 4864, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 32768, "bos_token_id": -1, "eos_token_id": -1,
    "use_sliding_window": False,
}
# Layer sizes of the larger models of the family, for `--only` runs at further sizes (the default
# run and its JSON line are always the 0.5B sizes above).
SIZES = {
    "0.5b": {},
    "1.5b": {"num_hidden_layers": 28, "hidden_size": 1536, "num_attention_heads": 12, "num_key_value_heads": 2,
             "intermediate_size": 8960},
    "7b": {"num_hidden_layers": 28, "hidden_size": 3584, "num_attention_heads": 28, "num_key_value_heads": 4,
           "intermediate_size": 18944, "vocab_size": 152064, "tie_word_embeddings": False},
}
CONTEXT = 4096
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi in the background during the timed region (read-only queries)."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        sm = sorted(int(r[0]) for r in self.rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": int(self.rows[0][1]), "reasons": reasons,
                "samples": len(self.rows)}


def model_folder(config, seed=0):
    import hashlib

    from easy_gpt.cpp_b200.weights.random_init import write_random_model

    tag = hashlib.sha256(json.dumps(config, sort_keys=True).encode()).hexdigest()[:12]
    folder = Path(tempfile.gettempdir()) / f"easy_gpt_bench_{os.getuid()}_{tag}_{seed}"
    if not (folder / "model.safetensors").is_file() or not (folder / "done").is_file():
        t0 = time.time()
        write_random_model(folder, config, seed, std=0.02, store_dtype="bfloat16")
        (folder / "done").write_text("ok")
        print(f"[bench] wrote random weights to {folder} in {time.time() - t0:.1f}s", file=sys.stderr, flush=True)
    return folder


def prompts_for(batch, length, vocab, seed):
    import numpy as np

    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=length).tolist() for _ in range(batch)]


def time_steps(engine, ids, steps):
    """K decode steps through the engine's step(), the product's own loop (scheduler, captured step, sampling kernel,
    tokens back on the host every step).  Returns (seconds on the device by CUDA events on the engine's stream around
    the K steps, wall-clock seconds until the last step's tokens are on the host, kernels launched, bytes a step has
    to read on average)."""
    kv_per_token = engine.kv_bytes_per_token()
    weights = engine.stats()["weight_bytes_per_step"]
    # step s (from 0) reads the weights once and the keys and values of every request: what it held before, plus s + 1
    held = sum(engine.cached_length(r) for r in ids)
    step_bytes = steps * weights + kv_per_token * (steps * held + len(ids) * steps * (steps + 1) // 2)
    replays0 = engine.stats()["graph_replays"]
    device, wall = engine.time_steps(steps)
    replays = engine.stats()["graph_replays"] - replays0
    assert replays == steps, "the timed steps did not go through the captured decode step"
    launches = replays * (engine.last_step_launches() + 1)             # the captured step's kernels and the sampling kernel
    return device, wall, launches, step_bytes / steps


def median(values):
    values = sorted(values)
    return values[len(values) // 2]


REPEATS = 3


def measure_decode(folder, config, batch, steps, warmup, want_e2e, dtype="bfloat16", default_options=False):
    """Decode steps that end at CONTEXT tokens: W warm-up steps, then REPEATS runs of K steps; the median of their device
    times is `value`, the median of their wall-clock times `e2e`.  ``default_options``: the engine's own defaults for
    page size and request length instead of pages of 64 tokens and requests sized for this run."""
    from easy_gpt.cpp_b200.native import NativeEngine
    from easy_gpt.cpp_b200.sampling import GREEDY

    total_steps = warmup + REPEATS * steps + 4
    start_context = CONTEXT - total_steps
    # the prompts are prefilled in large steps, so that the requests admitted first decode only a few tokens
    # while the others' prompts are still on their way (those tokens get room of their own)
    prefill_budget = 32768
    room = CONTEXT + 64 + -(-batch * start_context // prefill_budget) + 1
    options = dict(cache_tokens=batch * (room + 63), max_active=batch, prefill_batch=batch, max_batch_tokens=prefill_budget,
                   chunk_size=4096)
    if not default_options:
        options.update(page_size=64, max_tokens_per_request=room)
    engine = NativeEngine(folder, dtype=dtype, **options)
    ids = [engine.add_request(p, GREEDY, max_new_tokens=total_steps + 64)
           for p in prompts_for(batch, start_context, config["vocab_size"], seed=batch)]
    while any(engine.request(r)["computed"] < start_context for r in ids):       # until every request is decoding
        engine.step()
    engine.time_steps(warmup)
    with ClockSampler() as clocks:
        timed = [time_steps(engine, ids, steps) for _ in range(REPEATS)]
    out = {"clocks": clocks.summary()}
    seconds = median([t[0] for t in timed])
    out["seconds"], out["launches"], out["step_bytes"] = seconds, timed[0][2], median([t[3] for t in timed])
    out["tok_s"] = batch * steps / seconds
    out["repeats_ms"] = [round(1e3 * t[0] / steps, 4) for t in timed]
    if want_e2e:
        out["e2e_tok_s"] = batch * steps / median([max(t[0], t[1]) for t in timed])
        # per step: the packed metadata of the batch goes up, the sampled tokens come back
        out["h2d"] = engine.last_step_h2d_bytes()
        out["d2h"] = batch * 4
    out["context_end"] = max(engine.cached_length(r) for r in ids)
    out["page_size"] = options.get("page_size", 16)
    del engine
    return out


def prefill_flops(config, tokens):
    H, I, V = config["hidden_size"], config["intermediate_size"], config["vocab_size"]
    NH, NKV = config["num_attention_heads"], config["num_key_value_heads"]
    HD = config.get("head_dim") or H // NH
    L = config["num_hidden_layers"]
    per_token = 2 * (H * (NH + 2 * NKV) * HD + NH * HD * H + 3 * H * I)
    gemm = L * per_token * tokens + 2 * H * V                      # logits at the last position only
    attention = L * 4 * NH * HD * (tokens * (tokens + 1) // 2)      # QK^T and PV over the causal half
    return gemm + attention


def measure_prefill(folder, config, repeats=5):
    """One prompt of PREFILL_TOKENS tokens in one step through the step function (logits at its last token); the
    median of the step's time on the device."""
    from easy_gpt.cpp_b200.native import NativeStepRunner

    runner = NativeStepRunner(folder, "bfloat16", page_size=64, num_pages=2 * PREFILL_TOKENS // 64, max_slots=2)
    prompt = prompts_for(1, PREFILL_TOKENS, config["vocab_size"], seed=99)[0]
    times = []
    for i in range(repeats + 2):
        runner.run([("p", prompt, [PREFILL_TOKENS - 1])])
        runner.end("p")
        if i >= 2:
            times.append(runner.last_step_device_seconds)
    del runner
    return median(times)


def print_timeline(folder, config, batch):
    """Device-side timeline of one captured decode step: for every kind of kernel its launches, the
    mean time from its first CTA's start to its last CTA's end (this includes waiting for the kernel
    in front, since kernels are launched ahead of their dependencies), and how long before the end of
    the kernel in front it started.  Uses the kernels' optional %globaltimer trace."""
    import collections

    import torch

    from easy_gpt.cpp_b200 import kernels
    from easy_gpt.cpp_b200.engine import GptEngine

    kernels.Timeline.start()
    start_context = CONTEXT - 40
    prefill_budget = 32768
    room = CONTEXT + 64 + -(-batch * start_context // prefill_budget) + 1
    engine = GptEngine(folder, dtype="bfloat16", page_size=64, cache_tokens=batch * (room + 63), max_active=batch,
                       prefill_batch=batch, max_batch_tokens=prefill_budget, chunk_size=4096, max_tokens_per_request=room)
    kernels.Timeline.names = []
    from easy_gpt.cpp_b200.sampling import GREEDY

    reqs = [engine.add_request(p, GREEDY, max_new_tokens=100) for p in prompts_for(batch, start_context, config["vocab_size"], 1)]
    while any(r.known - r.computed != 1 or r.state != "running" for r in reqs):
        engine.step()
    engine.sync()
    for _ in range(5):
        engine.step()
    torch.cuda.synchronize()
    kernels.Timeline.reset()
    engine.step()
    torch.cuda.synchronize()
    rows = sorted((r for r in kernels.Timeline.read() if r[2] > 0), key=lambda r: r[1])
    t0, t1 = rows[0][1], max(r[2] for r in rows)
    print(f"decode step, batch {batch}, context {CONTEXT}: {len(rows)} traced kernels, {(t1 - t0) / 1e3:.1f} us from first start to last end")
    agg = collections.OrderedDict()
    prev_end = t0
    for name, start, end, marks in rows:
        a = agg.setdefault(name, [0, 0.0, 0.0, [0.0] * 6, 0.0, [0.0] * 6])
        a[0] += 1
        a[1] += (end - start) / 1e3
        a[2] += (prev_end - start) / 1e3
        for i in range(6):                           # the kernel's phase stamps (latest over its CTAs), counted from the end of the kernel in front
            a[3][i] += (marks[i] - prev_end) / 1e3 if marks[i] else 0.0
            earliest = ~marks[7 + i] & ((1 << 64) - 1) if marks[7 + i] else 0      # stored as its complement
            a[5][i] += (earliest - prev_end) / 1e3 if earliest else 0.0
        a[4] += (end - prev_end) / 1e3
        prev_end = end
    print(f"{'kernel':58s} {'n':>4s} {'first start..last end us':>25s} {'started before previous end us':>31s}")
    for name, (n, dur, early, _, _, _) in agg.items():
        print(f"{name:58s} {n:4d} {dur / n:25.2f} {early / n:31.2f}")
    print("\nphases, microseconds after the end of the kernel in front (mean): before the dependency wait, after it, input rows ready, "
          "product done, summed inside the CTA, summed across CTAs, end of the kernel")
    for name, (n, _, _, marks, total, _) in agg.items():
        print(f"{name:58s} " + " ".join(f"{m / n:7.2f}" for m in marks) + f" {total / n:7.2f}")
    print("\nthe same for the CTA (at 'product done': the warp) that gets there first")
    for name, (n, _, _, _, _, firsts) in agg.items():
        print(f"{name:58s} " + " ".join(f"{m / n:7.2f}" for m in firsts))
    return 0


def print_fused_timeline(folder, config, batch):
    """The decode step as ONE persistent kernel (csrc/decode_fused.cu, an option of the step function): per kind of
    operation the mean time from the last CTA's leaving the operation in front to the last CTA's entering this one (the
    barrier across the grid), and inside the operation until the input rows are staged, until the products are done, and
    in all.  From %globaltimer stamps that the kernel's CTAs leave; no profiler attached."""
    import collections

    os.environ["EASY_GPT_FUSED_DECODE"] = "1"
    os.environ["EASY_GPT_FUSED_TRACE"] = "1"
    from easy_gpt.cpp_b200.native import NativeEngine
    from easy_gpt.cpp_b200.sampling.params import SamplingParams

    start_context = CONTEXT - 40
    room = CONTEXT + 64
    engine = NativeEngine(str(folder), dtype="bfloat16", page_size=64, cache_tokens=batch * (room + 63), max_active=batch, prefill_batch=batch,
                          max_batch_tokens=32768, chunk_size=4096, max_tokens_per_request=room)
    for p in prompts_for(batch, start_context, config["vocab_size"], 1):
        engine.add_request(p, SamplingParams(greedy=True), max_new_tokens=100)
    for _ in range(12):
        engine.step()
    engine.sync()
    engine.fused_trace()
    engine.step()
    engine.sync()
    rows = [[int(v) for v in r] for r in engine.fused_trace()]
    if not rows:
        print("the step did not run as one fused kernel (sizes it does not take, or more than 8 tokens)")
        return 1
    names = {11: "norm -> head (float32 logits)", 12: "norm -> gate/up + SwiGLU", 13: "norm -> QKV + rotation + cache", 23: "embedding + norm -> QKV + ...",
             100: "attention"}
    agg = collections.OrderedDict()
    previous_left, nth_rows = None, 0
    for entered, staged, done, left, kind in rows:
        label = names.get(kind)
        if label is None:                               # rows -> residual: the output projection, then the down projection
            label = "rows -> residual (O)" if nth_rows % 2 == 0 else "rows -> residual (down)"
            nth_rows += 1
        a = agg.setdefault(label, [0, 0.0, 0.0, 0.0, 0.0])
        a[0] += 1
        a[1] += (entered - (previous_left if previous_left is not None else entered)) / 1e3
        a[2] += ((staged or entered) - entered) / 1e3
        a[3] += ((done or left) - (staged or entered)) / 1e3
        a[4] += (left - entered) / 1e3
        previous_left = left
    print(f"fused decode step, batch {batch}, context {CONTEXT}: {len(rows)} operations, {(rows[-1][3] - rows[0][0]) / 1e3:.1f} us from the first entered to the last left")
    print(f"{'operation':34s} {'n':>3s} {'barrier us':>11s} {'staging us':>11s} {'products us':>12s} {'whole us':>9s}")
    for label, (n, barrier, staging, products, whole) in agg.items():
        print(f"{label:34s} {n:3d} {barrier / n:11.2f} {staging / n:11.2f} {products / n:12.2f} {whole / n:9.2f}")
    return 0


def print_gemm_comparison(config, tokens=PREFILL_TOKENS):
    """The package's tcgen05/TMA product against the library product at the prefill shapes: each
    timed as a CUDA graph of eight launches on distinct weights with the L2 flushed before."""
    import torch

    from easy_gpt.cpp_b200 import kernels

    dev = "cuda"
    flush = torch.empty(256 << 20, dtype=torch.int8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    H, I = config["hidden_size"], config["intermediate_size"]
    qkv = (config["num_attention_heads"] + 2 * config["num_key_value_heads"]) * (H // config["num_attention_heads"])

    def graph_us(fns):
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for f in fns:
                f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for f in fns:
                f()
        times = []
        for i in range(12):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            if i >= 2:
                times.append(a.elapsed_time(b) * 1e3 / len(fns))
        return sorted(times)[len(times) // 2]

    print(f"{tokens} tokens; microseconds per product and TFLOP/s")
    for name, N, K in (("qkv", qkv, H), ("o", H, H), ("gate_up", 2 * I, H), ("down", H, I)):
        x = torch.randn(tokens, K, device=dev).bfloat16()
        ws = [(torch.randn(N, K, device=dev) * 0.05).bfloat16() for _ in range(8)]
        out = torch.empty(tokens, N, device=dev, dtype=torch.bfloat16)
        ours = graph_us([(lambda w=w: kernels.gemm_tcgen05(x, w, None, out, status)) for w in ws])
        lib = graph_us([(lambda w=w: torch.nn.functional.linear(x, w)) for w in ws])
        flops = 2 * tokens * N * K
        us = graph_us([(lambda w=w: kernels.gemm_tcgen05(x, w, None, out, status, pair=True)) for w in ws])
        pair = f"   CTA pairs {us:7.2f} us {flops / us / 1e6:7.1f}"
        print(f"  {name:8s} [{N} x {K}]  tcgen05 {ours:7.2f} us {flops / ours / 1e6:7.1f}   library {lib:7.2f} us {flops / lib / 1e6:7.1f}{pair}")
    assert status.item() == 0
    return 0


def print_attention_timings():
    """The two prompt-attention kernels alone (warp-level `mma.sync` and tcgen05), one request, pages of 64: each timed
    as a CUDA graph of eight launches, the tcgen05 kernel with the parts the engine's policy gives it."""
    import math

    import torch

    from easy_gpt.cpp_b200 import kernels

    dev = "cuda"
    page = 64
    print("tokens, context before them, heads x head size: microseconds and TFLOP/s, mma.sync | tcgen05 (parts)")
    for T, ctx0, NH, NKV, HD in ((2048, 0, 14, 2, 64), (8192, 0, 14, 2, 64), (2048, 0, 28, 4, 128), (512, 3584, 14, 2, 64),
                                 (512, 7680, 28, 4, 128), (64, 4000, 14, 2, 64), (256, 1024, 14, 2, 64)):
        pages = (ctx0 + T + page - 1) // page
        kv = torch.randn(pages + 1, 2, NKV, page, HD, device=dev).bfloat16()
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, -1)
        q = torch.randn(T, (NH + 2 * NKV) * HD, device=dev).bfloat16()
        positions = torch.arange(ctx0, ctx0 + T, dtype=torch.int32, device=dev)
        tiles = torch.tensor([(0, o, min(128, T - o)) for o in range(0, T, 128)], dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        parts, part_tiles = kernels.attention_prefill_parts(len(tiles), NH, HD)
        flops = 4 * HD * NH * (T * (T + 1) / 2 + T * ctx0)
        line, outs = f"  T={T:5d} ctx {ctx0:5d}  {NH:2d} x {HD:3d}", []
        for fn, extra in ((kernels.attention_prefill, {}), (kernels.attention_prefill_tcgen05, {"parts": parts, "part_tiles": part_tiles})):
            out = torch.zeros(T, NH * HD, device=dev, dtype=torch.bfloat16)

            def launch():
                fn(q, kv[:, 0], kv[:, 1], table, positions, tiles, out, NH, NKV, HD, None, 1 / math.sqrt(HD), status, **extra)

            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                launch()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(8):
                    launch()
            times = []
            for _ in range(10):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                g.replay()
                b.record()
                torch.cuda.synchronize()
                times.append(a.elapsed_time(b) * 1e3 / 8)
            us = sorted(times)[len(times) // 2]
            line += f"   {us:8.2f} us {flops / us / 1e6:6.1f}"
            outs.append(out.float())
        print(f"{line}  ({parts} parts)   largest difference between the kernels {float((outs[0] - outs[1]).abs().max()):.4f}")
        assert status.item() == 0
    return 0


def measure_serving(folder, config, requests=64, new_tokens=512, chunk=512, budget=2048, seed=0, repeats=2):
    """Continuous batching through the engine: `requests` concurrent requests with prompt lengths uniform in
    [128, 4096] and `new_tokens` generated tokens each, prompts cut into portions of `chunk` tokens that share
    steps with the decoding requests.  Wall clock from the first add_request to the last token on the host;
    the first repeat warms up (the decode steps' graphs are captured), the last one is reported."""
    import numpy as np

    from easy_gpt.cpp_b200.native import NativeEngine
    from easy_gpt.cpp_b200.sampling import GREEDY

    rng = np.random.default_rng(seed)
    lengths = rng.integers(128, 4097, size=requests)
    prompts = [rng.integers(0, config["vocab_size"], size=int(n)).tolist() for n in lengths]
    engine = NativeEngine(folder, dtype="bfloat16", page_size=64, cache_tokens=requests * (4096 + new_tokens + 64),
                          max_active=requests, prefill_batch=4, max_batch_tokens=budget, chunk_size=chunk,
                          max_tokens_per_request=4096 + new_tokens + 64)
    out = {}
    for _ in range(repeats):
        before = engine.stats()
        engine.sync()
        t0 = time.perf_counter()
        ids = [engine.add_request(p, GREEDY, max_new_tokens=new_tokens) for p in prompts]
        engine.run_to_completion()
        engine.sync()
        seconds = time.perf_counter() - t0
        for r in ids:
            assert len(engine.output(r)) == new_tokens and not engine.request(r)["error"]
            engine.forget(r)
        stats = engine.stats()
        steps = stats["steps"] - before["steps"]
        out = {"requests": requests, "prompt_tokens": int(lengths.sum()), "generated_tokens": requests * new_tokens,
               "seconds": round(seconds, 3), "steps": steps, "preemptions": stats["preemptions"] - before["preemptions"],
               "generated_tok_s": round(requests * new_tokens / seconds, 1),
               "all_tok_s": round((int(lengths.sum()) + requests * new_tokens) / seconds, 1),
               "ms_per_step": round(1e3 * seconds / max(1, steps), 3), "graph_replays": stats["graph_replays"] - before["graph_replays"]}
    return out


def run_ours(args):
    config = dict(CONFIG_05B, **SIZES[args.sizes])
    if args.sizes != "0.5b" and not args.only:
        print("bench.py: --sizes other than 0.5b goes with --only (the JSON line is defined for the 0.5B sizes)")
        return 2
    if args.only == "attention":                                   # kernels alone: no model folder
        return print_attention_timings()
    layers_full = config["num_hidden_layers"]
    if args.layers:
        config["num_hidden_layers"] = args.layers
    pk = peaks()
    folder = model_folder(config)
    if args.fused:
        os.environ["EASY_GPT_FUSED_DECODE"] = "1"
    if args.only == "decode":
        r = measure_decode(folder, config, args.batch, args.steps, args.warmup, want_e2e=False, dtype=args.dtype,
                           default_options=args.default_options)
        gb_s = r["step_bytes"] / (r["seconds"] / args.steps) / 1e9
        print(json.dumps({"only": "decode", "sizes": args.sizes, "dtype": args.dtype, "batch": args.batch,
                          "layers": config["num_hidden_layers"], "context": CONTEXT, "page_size": r["page_size"],
                          "tok_s": round(r["tok_s"], 1), "ms_per_step": round(1e3 * r["seconds"] / args.steps, 4),
                          "repeats_ms_per_step": r["repeats_ms"], "gb_s": round(gb_s, 1),
                          "roofline_frac": round(gb_s / pk["hbm_gbs"], 4), "peaks": pk["source"], "clocks": r["clocks"]}))
        return 0
    if args.only == "serve":
        print(json.dumps({"only": "serve", "sizes": args.sizes, "layers": config["num_hidden_layers"],
                          **measure_serving(folder, config, requests=args.batch if args.batch != 8 else 64)}))
        return 0
    if args.only == "timeline":
        return print_fused_timeline(folder, config, args.batch) if args.fused else print_timeline(folder, config, args.batch)
    if args.only == "gemm":
        return print_gemm_comparison(config)
    if args.only == "prefill":
        sec = measure_prefill(folder, config)
        flops = prefill_flops(config, PREFILL_TOKENS)
        print(json.dumps({"only": "prefill", "sizes": args.sizes, "tokens": PREFILL_TOKENS, "layers": config["num_hidden_layers"],
                          "ms": round(sec * 1e3, 3), "tok_s": round(PREFILL_TOKENS / sec, 1), "tflops": round(flops / sec / 1e12, 1),
                          "frac": round(flops / sec / (pk["bf16_tflops"] * 1e12), 4), "peaks": pk["source"]}))
        return 0
    main = measure_decode(folder, config, args.batch, args.steps, args.warmup, want_e2e=True)
    points, points_roofline = {}, {}
    for b in (1, 64):
        r = measure_decode(folder, config, b, args.steps, args.warmup, want_e2e=False)
        points[f"decode_b{b}"] = round(r["tok_s"], 1)
        points_roofline[f"decode_b{b}"] = round(r["step_bytes"] / (r["seconds"] / args.steps) / 1e9 / pk["hbm_gbs"], 4)
    # the same batch with the engine's own defaults for page size and request length (what a user gets unasked)
    r = measure_decode(folder, config, args.batch, args.steps, args.warmup, want_e2e=False, default_options=True)
    points[f"decode_b{args.batch}_default_options"] = round(r["tok_s"], 1)
    # the 32-bit path, for information (its own FFMA products: no tensor cores)
    fp32_steps = min(args.steps, 16)
    r32 = measure_decode(folder, config, args.batch, fp32_steps, 3, want_e2e=False, dtype="float32")
    prefill_s = measure_prefill(folder, config)
    flops = prefill_flops(config, PREFILL_TOKENS)
    achieved = main["step_bytes"] / (main["seconds"] / args.steps) / 1e9
    line = {
        "metric": "decode tok/s", "value": round(main["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 * main["seconds"] / args.steps, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {
            "model": "qwen2.5-0.5b-sizes-random-weights", "global_batch": args.batch, "seq_len": CONTEXT,
            "parallelism": "single-gpu", "layers": config["num_hidden_layers"], "layers_full": layers_full,
            "hidden": config["hidden_size"], "heads": config["num_attention_heads"],
            "kv_heads": config["num_key_value_heads"], "head_dim": config["hidden_size"] // config["num_attention_heads"],
            "intermediate": config["intermediate_size"], "vocab": config["vocab_size"], "tied_head": True,
            "context_end": main["context_end"], "page_size": main["page_size"], "prefill_tokens": PREFILL_TOKENS,
            "l2": "inputs of a step exceed L2", "sampling": "greedy", "repeats": f"median of {REPEATS}",
        },
        "clocks": main["clocks"],
        "repeats_ms_per_step": main["repeats_ms"],
        "e2e": {"value": round(main["e2e_tok_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": main["h2d"],
                "d2h_bytes_per_step": main["d2h"]},
        "gpu_launches": main["launches"],
        "prefill": {"value": round(PREFILL_TOKENS / prefill_s, 1), "tokens": PREFILL_TOKENS, "ms": round(prefill_s * 1e3, 3),
                    "frac": round(flops / prefill_s / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]},
        "points": points,
        "points_roofline": points_roofline,
        "fp32": {"ms_per_step": round(1e3 * r32["seconds"] / fp32_steps, 3), "value": round(r32["tok_s"], 1), "unit": "tokens/s",
                 "steps": fp32_steps, "note": "the 32-bit path at the same batch and context, for information"},
    }
    print(json.dumps(line))
    return 0


def run_reference(args):
    """The unmodified reference through its own command line (baseline/reference_arm.py): the same model
    sizes, batch, context and K last decode steps; the line has the shape of the other arm's."""
    from baseline import reference_arm

    config = dict(CONFIG_05B)
    try:
        folder = model_folder(config)
        with ClockSampler() as clocks:
            r = reference_arm.run(folder, config, args.batch, CONTEXT, args.steps, prompt_tokens=args.ref_prompt)
    except reference_arm.Unavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e)}))
        return 0
    print(json.dumps({
        "metric": "decode tok/s", "value": round(r["tok_s"], 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": r["decode_steps"] - args.steps, "ms_per_step": round(r["ms_per_step"], 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": {"model": "qwen2.5-0.5b-sizes-random-weights", "global_batch": args.batch, "seq_len": CONTEXT,
                   "parallelism": "single-gpu", "layers": config["num_hidden_layers"], "layers_full": config["num_hidden_layers"],
                   "hidden": config["hidden_size"], "heads": config["num_attention_heads"], "kv_heads": config["num_key_value_heads"],
                   "head_dim": config["hidden_size"] // config["num_attention_heads"], "intermediate": config["intermediate_size"],
                   "vocab": config["vocab_size"], "tied_head": True, "context_end": CONTEXT, "prompt_tokens": r["prompt_tokens"],
                   "sampling": "greedy", "build": "cmake RelWithDebInfo, CUDA backend, sm_100",
                   "timing": "host clock of the reference's own log lines around the last K decode steps"},
        "clocks": clocks.summary(),
        "e2e": {"value": round(r["tok_s"], 2), "unit": "tokens/s", "note": "its loop takes and returns host token ids every step"},
        "whole_run": {"decode_steps": r["decode_steps"], "avg_ms_per_step": r["avg_ms_per_step_whole_run"],
                      "wall_s": round(r["wall_s"], 1)},
    }))
    return 0


def main():
    global CONTEXT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--context", type=int, default=CONTEXT, help="context length the decode steps end at (default 4096)")
    ap.add_argument("--sizes", choices=list(SIZES), default="0.5b", help="layer sizes for --only runs")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16", help="precision of --only decode")
    ap.add_argument("--default-options", action="store_true",
                    help="--only decode with the engine's default page size and request length")
    ap.add_argument("--ref-prompt", type=int, default=0,
                    help="prompt length of the reference arm (0: 1536, or the longest its int-indexed logits allow)")
    ap.add_argument("--fused", action="store_true", help="with --only timeline or decode: the decode step as one persistent kernel (EASY_GPT_FUSED_DECODE=1)")
    ap.add_argument("--only", choices=["decode", "prefill", "timeline", "gemm", "attention", "serve"], default=None,
                    help="measure one part only and print a short line (for profiling runs)")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    CONTEXT = args.context
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
