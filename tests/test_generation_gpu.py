"""Generation through the Python entry point and the command line (GPU)."""
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_model
import tiny_configs

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def model_a(tmp_path_factory):
    return tiny_configs.write_tiny("A", tmp_path_factory.mktemp("gen_A"))


@pytest.fixture(scope="module")
def model_b(tmp_path_factory):
    return tiny_configs.write_tiny("B", tmp_path_factory.mktemp("gen_B"))


def check_greedy(folder, prompts, outputs, dtype, tol):
    """Every generated token is the plain implementation's best token for the
    same prefix, up to `tol` in the logit (ties and bfloat16 rounding)."""
    cfg, w = plain_model.read_model_dir(folder, round_to_bf16=(dtype == "bfloat16"))
    for prompt, out in zip(prompts, outputs):
        logits = plain_model.forward_logits(cfg, w, list(prompt) + list(out))
        for i, tok in enumerate(out):
            row = logits[len(prompt) + i - 1]
            assert float(row.max() - row[tok]) <= tol, (dtype, i, tok, int(row.argmax()))


@pytest.mark.parametrize("dtype, tol", [("float32", 1e-4), ("bfloat16", 0.08)])
def test_greedy_generation_matches_plain(model_a, dtype, tol):
    from easy_gpt.cpp_b200.engine import GptEngine

    prompts = [tiny_configs.random_tokens(256, n, s) for n, s in ((5, 1), (17, 2), (31, 3))]
    engine = GptEngine(model_a, dtype=dtype, page_size=4, cache_tokens=1024, max_active=4, chunk_size=16, max_batch_tokens=24)
    outputs = engine.generate(prompts, max_new_tokens=16, greedy=True)
    assert [len(o) for o in outputs] == [16, 16, 16]
    check_greedy(model_a, prompts, outputs, dtype, tol)
    if dtype == "float32":
        cfg, w = plain_model.read_model_dir(model_a)
        assert outputs[0] == plain_model.greedy_generate(cfg, w, prompts[0], 16)
    assert not engine.runner.cache.live_requests()


def test_long_decoding_and_eos(model_b):
    """300 tokens decoded one by one through windowed and full layers (float32);
    config B ends a request at token 7."""
    from easy_gpt.cpp_b200.engine import GptEngine

    engine = GptEngine(model_b, dtype="float32", page_size=16, cache_tokens=2048, max_active=4)
    prompts = [tiny_configs.random_tokens(391, 3, 11), tiny_configs.random_tokens(391, 50, 12)]
    outputs = engine.generate(prompts, max_new_tokens=300, greedy=True)
    check_greedy(model_b, prompts, outputs, "float32", 1e-4)
    for out in outputs:
        assert len(out) == 300 or out[-1] == 7
        assert 7 not in out[:-1]
    assert max(len(o) for o in outputs) > 100


def test_preemption_does_not_change_outputs(model_a):
    from easy_gpt.cpp_b200.engine import GptEngine

    prompts = [tiny_configs.random_tokens(256, 9 + 3 * i, 20 + i) for i in range(4)]
    results = {}
    for name, cache_tokens in (("roomy", 1024), ("tight", 96)):
        engine = GptEngine(model_a, dtype="float32", page_size=4, cache_tokens=cache_tokens, max_active=4,
                           chunk_size=16, max_batch_tokens=64)
        results[name] = engine.generate(prompts, max_new_tokens=30, temperature=0.9, top_k=0, top_p=1.0, seed=5)
        results[name + "_preemptions"] = engine.scheduler.stats.preemptions
    assert results["roomy_preemptions"] == 0 and results["tight_preemptions"] > 0
    assert results["roomy"] == results["tight"]


def test_max_steps_and_step_by_step_api(model_a):
    from easy_gpt.cpp_b200.engine import GptEngine
    from easy_gpt.cpp_b200.sampling import GREEDY

    engine = GptEngine(model_a, dtype="bfloat16", page_size=16, cache_tokens=512, max_active=2)
    r = engine.add_request([1, 2, 3, 4, 5], GREEDY, max_steps=10)           # 10 - 5 + 1 = 6 new tokens
    with pytest.raises(ValueError, match="outside the vocabulary"):
        engine.add_request([1, 999], GREEDY, max_steps=10)
    finished = []
    while engine.scheduler.has_work():
        finished += engine.step()
    assert finished == [r] and len(r.output) == 6 and r.finish_reason == "length"


def test_command_line(model_a, tmp_path):
    prompts = tmp_path / "prompts.txt"
    prompts.write_text("5 17 3\n\n9,8,7,6\n")
    cmd = [sys.executable, str(ROOT / "bin" / "easy_llm"), "--model", str(model_a), "--token-ids", "--greedy",
           "--max-steps", "12", "--dtype", "float32", "-f", str(prompts)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    lines = (tmp_path / "prompts_output.txt").read_text().splitlines()
    assert len(lines) == 2
    outs = [[int(t) for t in line.split()] for line in lines]
    assert len(outs[0]) == 10 and len(outs[1]) == 9                       # max(1, max_steps - prompt + 1)
    check_greedy(model_a, [[5, 17, 3], [9, 8, 7, 6]], outs, "float32", 1e-4)
    assert r.stdout.splitlines()[-2:] == lines
