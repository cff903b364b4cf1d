"""Decode steps of up to eight tokens as ONE persistent kernel (csrc/decode_fused.cu; an option of the step function,
EASY_GPT_FUSED_DECODE=1), against the plain implementation and against the same steps run kernel by kernel (GPU): tokens
decoded one by one after a prompt, up to eight requests decoding together, decoding across page edges and a window's
edge, pages that are used again, and generation through the entry point."""
import os

import numpy as np
import pytest

import engine_harness as H
import plain_model
import tiny_configs
from test_native_engine_gpu import run_native

pytestmark = pytest.mark.gpu

BF16_REL = 2.5e-2


@pytest.fixture(scope="module", params=["F", "G"])
def model(request, tmp_path_factory):
    name = request.param
    folder = tiny_configs.write_tiny(name, tmp_path_factory.mktemp(f"fused_{name}"))
    cfg = tiny_configs.CONFIGS[name][0]
    lengths = [150, 77, 260, 64, 41, 97, 130, 55]
    requests = {f"r{i}": tiny_configs.random_tokens(cfg["vocab_size"], n, 500 + i) for i, n in enumerate(lengths)}
    c, w = plain_model.read_model_dir(folder, round_to_bf16=True)
    refs = {rid: plain_model.forward_logits(c, w, toks).numpy() for rid, toks in requests.items()}
    return dict(name=name, folder=folder, cfg=cfg, requests=requests, refs=refs)


def decode_together(requests, prompt_tokens, live):
    """Prompts of `prompt_tokens` tokens whole, then the rest of `live` requests one token a step, all together."""
    names = list(requests)[:live]
    steps = [{"step": 0, "entries": [{"id": n, "tokens": requests[n][:prompt_tokens], "want": [prompt_tokens - 1]} for n in names], "end": []}]
    at = {n: prompt_tokens for n in names}
    while any(at[n] < len(requests[n]) for n in names):
        entries, end = [], []
        for n in names:
            if at[n] < len(requests[n]):
                entries.append({"id": n, "tokens": [requests[n][at[n]]], "want": [0]})
                at[n] += 1
                if at[n] == len(requests[n]):
                    end.append(n)
        steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


@pytest.mark.parametrize("live, page_size", [(1, 16), (3, 16), (4, 64), (8, 16)])
def test_fused_decode_matches_plain(model, live, page_size, monkeypatch):
    from easy_gpt.cpp_b200.native import NativeStepRunner

    monkeypatch.setenv("EASY_GPT_FUSED_DECODE", "1")
    steps = decode_together(model["requests"], 33, live)
    pool_tokens = H.max_live_tokens(steps, round_to=page_size)
    runner = NativeStepRunner(model["folder"], "bfloat16", page_size, pool_tokens // page_size, 8, pool_tokens)
    got = run_native(runner, steps)
    tol = BF16_REL * max(float(np.abs(r).max()) for r in model["refs"].values())
    worst = H.compare(got, model["refs"], tol, f"fused {model['name']} live {live}")
    print(f"fused {model['name']} live {live} pages of {page_size}: max |error| {worst:.3e}")
    assert runner.info("fused_steps") >= 20, "the decode steps did not run as one kernel"


def test_fused_and_kernel_by_kernel_agree(model, monkeypatch):
    """The same trace with the fused kernel and with the chain of kernels: the logits agree to rounding."""
    from easy_gpt.cpp_b200.native import NativeStepRunner

    steps = H.trace_mixed({k: v for k, v in list(model["requests"].items())[:5]})
    pool_tokens = H.max_live_tokens(steps, round_to=16)
    outs = []
    for fused in ("1", "0"):
        monkeypatch.setenv("EASY_GPT_FUSED_DECODE", fused)
        runner = NativeStepRunner(model["folder"], "bfloat16", 16, pool_tokens // 16, 4, pool_tokens)
        outs.append(run_native(runner, steps))
        assert (runner.info("fused_steps") > 0) == (fused == "1")
    scale = max(float(np.abs(r).max()) for r in model["refs"].values())
    for key, row in outs[0].items():
        assert float(np.abs(row - outs[1][key]).max()) <= BF16_REL * scale, key
    H.compare(outs[0], model["refs"], BF16_REL * scale, f"fused mixed {model['name']}")


def test_fused_generation_follows_the_plain_rule(model, monkeypatch):
    from easy_gpt.cpp_b200.native import NativeEngine
    from test_native_engine_gpu import check_greedy

    monkeypatch.setenv("EASY_GPT_FUSED_DECODE", "1")
    prompts = [model["requests"][f"r{i}"][:20 + 7 * i] for i in range(5)]
    engine = NativeEngine(model["folder"], dtype="bfloat16", page_size=16, cache_tokens=4096, max_active=8)
    outputs = engine.generate(prompts, max_new_tokens=40, greedy=True)
    assert engine.fused_steps() >= 30
    check_greedy(model["folder"], prompts, outputs, "bfloat16", 0.08)
