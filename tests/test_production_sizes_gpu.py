"""One decoder layer at the layer sizes of larger models (head size 128, widths of 1536 and 3584,
feed-forward widths of 8960 and 18944) against the plain implementation: the kernels choose tiles,
splits and shared-memory layouts by size, and the tiny configurations reach only the small ends of
those choices.  The vocabulary is kept small so that the folders stay small."""
import numpy as np
import pytest
import torch

import engine_harness as H
import plain_model
import tiny_configs

pytestmark = pytest.mark.gpu

SIZES = {
    # hidden 1536 = 12 heads of 128 in 2 groups, tied head
    "1.5b-layer": dict(hidden_size=1536, num_attention_heads=12, num_key_value_heads=2, intermediate_size=8960,
                       tie_word_embeddings=True, rms_norm_eps=1e-6),
    # hidden 3584 = 28 heads of 128 in 4 groups, untied head
    "7b-layer": dict(hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944,
                     tie_word_embeddings=False, rms_norm_eps=1e-6),
}


@pytest.fixture(scope="module", params=list(SIZES))
def layer_model(request, tmp_path_factory):
    from easy_gpt.cpp_b200.weights.random_init import write_random_model

    cfg = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 1, "vocab_size": 1000,
           "rope_theta": 1000000.0, "max_position_embeddings": 4096, "bos_token_id": -1, "eos_token_id": -1,
           "use_sliding_window": False, **SIZES[request.param]}
    folder = write_random_model(tmp_path_factory.mktemp(request.param), cfg, seed=21, std=0.02, bias_std=0.3, gain_std=0.1)
    requests = {"long": tiny_configs.random_tokens(1000, 300, 7), "short": tiny_configs.random_tokens(1000, 90, 8),
                "third": tiny_configs.random_tokens(1000, 45, 9)}
    refs = {}
    for dtype, rounded in (("float32", False), ("bfloat16", True)):
        c, w = plain_model.read_model_dir(folder, round_to_bf16=rounded)
        refs[dtype] = {rid: plain_model.forward_logits(c, w, toks).numpy() for rid, toks in requests.items()}
    return dict(folder=folder, requests=requests, refs=refs)


def runner_for(folder, dtype, steps, page_size=16):
    from easy_gpt.cpp_b200.engine import Model, StepRunner

    model = Model.from_dir(folder, device="cuda:0", dtype={"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype])
    pool_tokens = H.max_live_tokens(steps, round_to=page_size)
    return StepRunner(model, page_size=page_size, num_pages=pool_tokens // page_size, max_slots=4,
                      max_tokens_per_request=pool_tokens)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "tail_one_by_one", "mixed"])
def test_one_layer_of_a_larger_model(layer_model, dtype, mode):
    reqs = layer_model["requests"]
    steps = {"whole": H.trace_whole, "tail_one_by_one": lambda r: H.trace_tail_one_by_one({"long": r["long"], "short": r["short"]}),
             "mixed": H.trace_mixed}[mode](reqs)
    if dtype == "float32":
        tol = 1e-4
    else:
        tol = 3e-2 * max(float(np.abs(r).max()) for r in layer_model["refs"][dtype].values())
    runner = runner_for(layer_model["folder"], dtype, steps)
    got = H.run_in_process(runner, steps)
    assert len(got) == sum(len(e["want"]) for s in steps for e in s["entries"])
    H.compare(got, layer_model["refs"][dtype], tol, what=f"{mode} {dtype}")
    assert not runner.cache.live_requests()
