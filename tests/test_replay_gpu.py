"""Trace replay on the GPU against the plain implementation: whole requests, a
tail decoded one by one, portions of changing size, and mixed batches with page
reuse — in 32-bit and in bfloat16, for the tiny configurations."""
import numpy as np
import pytest
import torch

import engine_harness as H
import plain_model
import tiny_configs

pytestmark = pytest.mark.gpu

F32_ATOL = 1e-4
# bfloat16: 8 bits of mantissa on every activation the kernels round; the bound is relative to the largest
# logit of the model (about 3 for these configurations).  Seen on B200, the same in every replay mode: 0.6% (A),
# 1.2% (B), 0.9% (C), 0.9% (D), 1.2% (E) of it; the bound is twice the worst of these.
BF16_REL = 2.5e-2


@pytest.fixture(scope="module", params=["A", "B", "C", "D", "E"])
def tiny(request, tmp_path_factory):
    name = request.param
    folder = tiny_configs.write_tiny(name, tmp_path_factory.mktemp(f"tiny_{name}"))
    cfg = tiny_configs.CONFIGS[name][0]
    lengths = {"A": [5, 70, 131, 97, 33, 120], "B": [40, 77, 130, 64, 201, 18], "C": [90, 150, 33, 260, 75],
               "D": [61, 140, 35, 99], "E": [50, 133, 41]}[name]
    requests = {f"r{i}": tiny_configs.random_tokens(cfg["vocab_size"], n, 100 + i) for i, n in enumerate(lengths)}
    refs = {}
    for mode, rounded in (("float32", False), ("bfloat16", True)):
        c, w = plain_model.read_model_dir(folder, round_to_bf16=rounded)
        refs[mode] = {rid: plain_model.forward_logits(c, w, toks).numpy() for rid, toks in requests.items()}
    return dict(name=name, folder=folder, cfg=cfg, requests=requests, refs=refs)


def make_runner(folder, dtype, steps, page_size):
    from easy_gpt.cpp_b200.engine import Model, StepRunner

    model = Model.from_dir(folder, device="cuda:0", dtype={"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype])
    # exactly as many pages as the trace's worst moment needs: nothing spare
    pool_tokens = H.max_live_tokens(steps, round_to=page_size)
    return StepRunner(model, page_size=page_size, num_pages=pool_tokens // page_size, max_slots=4,
                      max_tokens_per_request=pool_tokens)


def tolerance(tiny, dtype):
    if dtype == "float32":
        return F32_ATOL
    return BF16_REL * max(float(np.abs(r).max()) for r in tiny["refs"][dtype].values())


TRACES = {
    "whole": lambda reqs: H.trace_whole(reqs),
    "tail_one_by_one": lambda reqs: H.trace_tail_one_by_one({k: v for k, v in reqs.items() if len(v) > 40}),
    "portions": lambda reqs: H.trace_portions(reqs),
    "mixed": lambda reqs: H.trace_mixed(reqs),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", list(TRACES))
@pytest.mark.parametrize("page_size", [4, 16])
def test_replay_matches_plain(tiny, dtype, mode, page_size):
    steps = TRACES[mode](tiny["requests"])
    runner = make_runner(tiny["folder"], dtype, steps, page_size)
    got = H.run_in_process(runner, steps)
    assert got
    worst = H.compare(got, tiny["refs"][dtype], tolerance(tiny, dtype), f"{tiny['name']} {dtype} {mode} page {page_size}")
    print(f"{tiny['name']} {dtype} {mode} page={page_size}: max |error| {worst:.3e}")
    assert not runner.cache.live_requests()
    assert all(g.pool.free_count == g.pool.num_pages for g in runner.cache.groups)
    if mode == "mixed":
        # the pool is so small that pages were handed out again
        assert all(g.pool.total_allocated > g.pool.num_pages for g in runner.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tiny, dtype, tmp_path):
    steps = H.trace_mixed(tiny["requests"])
    got = H.run_program(tiny["folder"], dtype, steps, tmp_path / "out")
    H.compare(got, tiny["refs"][dtype], tolerance(tiny, dtype), f"trace_run {tiny['name']} {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(tiny, dtype):
    """Requests of one, two and three tokens: whole, and token by token from an empty cache
    (position 0 has one key, itself; nothing earlier may leak in from a page used before)."""
    vocab = tiny["cfg"]["vocab_size"]
    requests = {f"s{n}": tiny_configs.random_tokens(vocab, n, 50 + n) for n in (1, 2, 3)}
    c, w = plain_model.read_model_dir(tiny["folder"], round_to_bf16=(dtype == "bfloat16"))
    refs = {rid: plain_model.forward_logits(c, w, toks).numpy() for rid, toks in requests.items()}
    tol = 1e-4 if dtype == "float32" else tolerance(tiny, dtype)
    # first fill the only pages with another request, so that the short ones get used pages
    warm = {"warm": tiny_configs.random_tokens(vocab, 48, 7)}
    one_by_one = []
    for rid, toks in requests.items():
        for i, t in enumerate(toks):
            one_by_one.append({"step": len(one_by_one), "entries": [{"id": rid, "tokens": [t], "want": [0]}],
                               "end": [rid] if i == len(toks) - 1 else []})
    for steps in (H.trace_whole(requests), one_by_one):
        runner = make_runner(tiny["folder"], dtype, H.trace_whole(warm), 16)
        H.run_in_process(runner, H.trace_whole(warm))
        got = H.run_in_process(runner, steps)
        H.compare(got, refs, tol, f"first tokens {tiny['name']} {dtype}")
