"""The benchmark's model checked, not only timed: the whole Qwen2.5-0.5B-sized model (24 layers,
width 896, 14 query heads on 2 KV heads of 64, feed-forward 4864, vocabulary 151,936, tied head,
pages of 64 tokens) with random weights against the plain implementation, in 32-bit (1e-4, the same
greedy tokens) and in bfloat16: requests whole, the last 32 tokens one by one, and a mixed trace.
(The formulas: src/models/gpt_model.cpp:310-333.)"""
import numpy as np
import pytest
import torch

import engine_harness as H
import plain_model

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 24, "hidden_size": 896, "num_attention_heads": 14, "num_key_value_heads": 2,
    "intermediate_size": 4864, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 32768, "bos_token_id": -1, "eos_token_id": -1,
    "use_sliding_window": False,
}
LENGTHS = {"long": 300, "short": 64, "middle": 150}
F32_ATOL = 1e-4
# bfloat16: the largest error seen on B200 is 0.037 where the largest logit is 3.26, that is 1.1% (whole 1.0%, tail
# 0.9%, mixed 1.1%); the bound is 2.7 times that
BF16_REL = 3e-2


@pytest.fixture(scope="module")
def full_size(tmp_path_factory):
    from easy_gpt.cpp_b200.weights.random_init import write_random_model

    folder = write_random_model(tmp_path_factory.mktemp("qwen25_05b_sizes"), CONFIG, seed=0, std=0.02, store_dtype="bfloat16")
    rng = np.random.default_rng(11)
    requests = {name: rng.integers(0, CONFIG["vocab_size"], size=n).tolist() for name, n in LENGTHS.items()}
    # the weights are stored in bfloat16, so the plain implementation holds the very same numbers in both modes
    cfg, w = plain_model.read_model_dir(folder)
    with torch.no_grad():
        refs = {rid: plain_model.forward_logits(cfg, w, toks).numpy() for rid, toks in requests.items()}
    del w
    return dict(folder=folder, requests=requests, refs=refs)


def traces(requests):
    whole = []
    for rid, toks in requests.items():
        n = len(toks)
        whole.append({"step": len(whole), "entries": [{"id": rid, "tokens": toks, "want": [0, 1, n // 2, n - 2, n - 1]}], "end": [rid]})
    tail = []
    toks = requests["long"]
    head = len(toks) - 32
    tail.append({"step": 0, "entries": [{"id": "long", "tokens": toks[:head], "want": [head - 1]}], "end": []})
    for i in range(head, len(toks)):
        tail.append({"step": len(tail), "entries": [{"id": "long", "tokens": [toks[i]], "want": [0]}],
                     "end": ["long"] if i == len(toks) - 1 else []})
    mixed = H.trace_mixed(requests, portion=40, max_live=3, seed=2)
    return {"whole": whole, "tail_one_by_one": tail, "mixed": mixed}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_size_model_matches_plain(full_size, dtype):
    from easy_gpt.cpp_b200.engine import Model, StepRunner

    model = Model.from_dir(full_size["folder"], device="cuda:0",
                           dtype={"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype])
    refs = full_size["refs"]
    largest = max(float(np.abs(r).max()) for r in refs.values())
    tol = F32_ATOL if dtype == "float32" else BF16_REL * largest
    for mode, steps in traces(full_size["requests"]).items():
        runner = StepRunner(model, page_size=64, num_pages=H.max_live_tokens(steps, 64) // 64 + 1, max_slots=4)
        got = H.run_in_process(runner, steps)
        worst = H.compare(got, refs, tol, f"0.5B sizes {dtype} {mode}")
        print(f"0.5B sizes {dtype} {mode}: max |error| {worst:.3e} (largest logit {largest:.2f})")
        # the same greedy token wherever the plain implementation's best token leads by more than the error allows
        for (rid, pos), row in got.items():
            ref = refs[rid][pos]
            top2 = np.partition(ref, -2)[-2:]
            if top2[1] - top2[0] > 2 * tol:
                assert int(row.argmax()) == int(ref.argmax()), (mode, rid, pos)
        assert not runner.cache.live_requests()
        del runner
    del model
    torch.cuda.empty_cache()


def test_full_size_greedy_generation(full_size):
    """Eight new tokens through the entry point in 32-bit: the plain implementation's tokens."""
    from easy_gpt.cpp_b200.engine import GptEngine

    prompt = full_size["requests"]["short"]
    engine = GptEngine(full_size["folder"], dtype="float32", page_size=64, cache_tokens=1024, max_active=2)
    out = engine.generate([prompt], max_new_tokens=8, greedy=True)[0]
    cfg, w = plain_model.read_model_dir(full_size["folder"])
    with torch.no_grad():
        logits = plain_model.forward_logits(cfg, w, prompt + out)
    for i, tok in enumerate(out):
        row = logits[len(prompt) + i - 1]
        assert float(row.max() - row[tok]) <= 2e-4, (i, tok, int(row.argmax()))
    del engine
    torch.cuda.empty_cache()
