"""The native engine (csrc/engine: C++ over the kernel library, no PyTorch on its path) against the plain
implementation (GPU): trace replay in its four modes for the tiny configurations in both precisions, many live
requests, generation (greedy and sampled) with and without preemption, the easy_llm program, and the same
tokens as the Python engine."""
import subprocess

import numpy as np
import pytest

import engine_harness as H
import plain_model
import tiny_configs

pytestmark = pytest.mark.gpu

F32_ATOL = 1e-4
BF16_REL = 2.5e-2


def run_native(runner, steps):
    """-> {(request, position): logits row}; checks the cache's books after every step."""
    rows = H.rows_of(steps)
    got = {}
    for s in steps:
        logits = runner.run([(e["id"], e["tokens"], e["want"]) for e in s["entries"]])
        if logits is not None:
            assert logits.shape[0] == len(rows[s["step"]])
            for key, row in zip(rows[s["step"]], logits):
                got[key] = row.copy()
        for rid in s["end"]:
            runner.end(rid)
        assert runner.info("books_in_order") == 1
    return got


@pytest.fixture(scope="module", params=["A", "B", "C", "D", "E", "TINY_B"])
def tiny(request, tmp_path_factory):
    name = request.param
    folder = tiny_configs.write_tiny(name, tmp_path_factory.mktemp(f"native_{name}"))
    cfg = tiny_configs.CONFIGS[name][0]
    lengths = {"A": [5, 70, 131, 97, 33], "B": [40, 77, 130, 64, 201], "C": [90, 150, 33, 260], "D": [61, 140, 35], "E": [50, 133, 41],
               "TINY_B": [1, 40, 77, 130]}[name]
    requests = {f"r{i}": tiny_configs.random_tokens(cfg["vocab_size"], n, 100 + i) for i, n in enumerate(lengths)}
    refs = {}
    for mode, rounded in (("float32", False), ("bfloat16", True)):
        c, w = plain_model.read_model_dir(folder, round_to_bf16=rounded)
        refs[mode] = {rid: plain_model.forward_logits(c, w, toks).numpy() for rid, toks in requests.items()}
    return dict(name=name, folder=folder, cfg=cfg, requests=requests, refs=refs)


def tolerance(tiny, dtype):
    return F32_ATOL if dtype == "float32" else BF16_REL * max(float(np.abs(r).max()) for r in tiny["refs"][dtype].values())


TRACES = {
    "whole": lambda reqs: H.trace_whole(reqs),
    "tail_one_by_one": lambda reqs: H.trace_tail_one_by_one({k: v for k, v in reqs.items() if len(v) > 40}),
    "portions": lambda reqs: H.trace_portions(reqs),
    "mixed": lambda reqs: H.trace_mixed(reqs),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", list(TRACES))
def test_native_replay_matches_plain(tiny, dtype, mode):
    from easy_gpt.cpp_b200.native import NativeStepRunner

    steps = TRACES[mode](tiny["requests"])
    page_size = 16
    pool_tokens = H.max_live_tokens(steps, round_to=page_size)
    runner = NativeStepRunner(tiny["folder"], dtype, page_size, pool_tokens // page_size, 4, pool_tokens)
    got = run_native(runner, steps)
    assert got
    worst = H.compare(got, tiny["refs"][dtype], tolerance(tiny, dtype), f"native {tiny['name']} {dtype} {mode}")
    print(f"native {tiny['name']} {dtype} {mode}: max |error| {worst:.3e}")
    assert runner.info("live_requests") == 0
    for g in range(runner.info("groups")):
        assert runner.info("free_pages", g) == runner.info("pages", g)
        if mode == "mixed":
            assert runner.info("pages_handed_out", g) > runner.info("pages", g)       # pages were handed out again
    if mode == "tail_one_by_one":
        assert runner.info("graph_replays") >= 32                                     # the single tokens went through captured steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("live, config", [(24, "C"), (64, "TINY_B")])
def test_native_many_live_requests(live, config, dtype, tmp_path):
    from easy_gpt.cpp_b200.native import NativeStepRunner
    from test_schedules_gpu import trace_many_live

    folder = tiny_configs.write_tiny(config, tmp_path / "m")
    vocab = tiny_configs.CONFIGS[config][0]["vocab_size"]
    rng = np.random.default_rng(live)
    requests = {f"q{i}": tiny_configs.random_tokens(vocab, int(rng.integers(20, 70)), 300 + i) for i in range(live)}
    cfg, w = plain_model.read_model_dir(folder, round_to_bf16=(dtype == "bfloat16"))
    refs = {rid: plain_model.forward_logits(cfg, w, toks).numpy() for rid, toks in requests.items()}
    steps = trace_many_live(requests, decode_tokens=10, per_step=12, portion=16)
    runner = NativeStepRunner(folder, dtype, 16, H.max_live_tokens(steps, 16) // 16, live)
    got = run_native(runner, steps)
    tol = F32_ATOL if dtype == "float32" else 1.5e-2 * max(float(np.abs(r).max()) for r in refs.values())
    H.compare(got, refs, tol, f"native {live} live {config} {dtype}")
    assert runner.info("graph_replays") >= 9


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_native_captures_a_step_shape_of_several_entries(dtype, tmp_path):
    """Two decoding requests beside a portion of six tokens of a third, 24 steps in a row: the shape is captured when
    it has come often enough and replayed afterwards; every step, eager or replayed, agrees with the plain implementation."""
    from easy_gpt.cpp_b200.native import NativeStepRunner

    folder = tiny_configs.write_tiny("TINY_B", tmp_path / "m")
    requests = {"d0": tiny_configs.random_tokens(384, 54, 1), "d1": tiny_configs.random_tokens(384, 47, 2),
                "p": tiny_configs.random_tokens(384, 144, 3)}
    cfg, w = plain_model.read_model_dir(folder, round_to_bf16=(dtype == "bfloat16"))
    refs = {rid: plain_model.forward_logits(cfg, w, toks).numpy() for rid, toks in requests.items()}
    steps = [{"step": 0, "entries": [{"id": "d0", "tokens": requests["d0"][:30], "want": [29]},
                                     {"id": "d1", "tokens": requests["d1"][:23], "want": [22]}], "end": []}]
    for i in range(24):
        steps.append({"step": len(steps), "end": [], "entries": [
            {"id": "d0", "tokens": [requests["d0"][30 + i]], "want": [0]},
            {"id": "d1", "tokens": [requests["d1"][23 + i]], "want": [0]},
            {"id": "p", "tokens": requests["p"][6 * i:6 * i + 6], "want": [0, 5]}]})
    steps[-1]["end"] = ["d0", "d1", "p"]
    runner = NativeStepRunner(folder, dtype, 16, H.max_live_tokens(steps, 16) // 16, 4)
    got = run_native(runner, steps)
    tol = F32_ATOL if dtype == "float32" else 1.5e-2 * max(float(np.abs(r).max()) for r in refs.values())
    H.compare(got, refs, tol, f"native captured mixed step {dtype}")
    assert runner.info("captured_shapes") == 1 and runner.info("graph_replays") >= 8


def check_greedy(folder, prompts, outputs, dtype, tol):
    cfg, w = plain_model.read_model_dir(folder, round_to_bf16=(dtype == "bfloat16"))
    for prompt, out in zip(prompts, outputs):
        logits = plain_model.forward_logits(cfg, w, list(prompt) + list(out))
        for i, tok in enumerate(out):
            row = logits[len(prompt) + i - 1]
            assert float(row.max() - row[tok]) <= tol, (dtype, i, tok, int(row.argmax()))


@pytest.mark.parametrize("dtype, tol", [("float32", 1e-4), ("bfloat16", 0.08)])
def test_native_greedy_generation_and_the_python_engines_tokens(dtype, tol, tmp_path):
    from easy_gpt.cpp_b200.engine import GptEngine
    from easy_gpt.cpp_b200.native import NativeEngine

    folder = tiny_configs.write_tiny("A", tmp_path / "m")
    prompts = [tiny_configs.random_tokens(256, n, s) for n, s in ((5, 1), (17, 2), (31, 3))]
    options = dict(dtype=dtype, page_size=4, cache_tokens=1024, max_active=4, chunk_size=16, max_batch_tokens=24)
    engine = NativeEngine(folder, **options)
    outputs = engine.generate(prompts, max_new_tokens=16, greedy=True)
    assert [len(o) for o in outputs] == [16, 16, 16]
    check_greedy(folder, prompts, outputs, dtype, tol)
    assert engine.stats()["live_requests"] == 0 and engine.stats()["graph_replays"] > 0
    if dtype == "float32":
        cfg, w = plain_model.read_model_dir(folder)
        assert outputs[0] == plain_model.greedy_generate(cfg, w, prompts[0], 16)
        assert outputs == GptEngine(folder, **options).generate(prompts, max_new_tokens=16, greedy=True)
    with pytest.raises(ValueError, match="outside the vocabulary"):
        engine.add_request([1, 999])


def test_native_sampled_generation_follows_the_plain_rule_and_survives_preemption(tmp_path):
    from easy_gpt.cpp_b200.native import NativeEngine
    from easy_gpt.cpp_b200.sampling import SamplingParams
    from test_schedules_gpu import check_sampled

    folder = tiny_configs.write_tiny("TINY_A", tmp_path / "m")
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, 256, size=n).tolist() for n in (5, 17, 31, 12)]
    params = SamplingParams(temperature=0.8, top_p=0.95, top_k=20, seed=2)
    results = {}
    for name, cache_tokens in (("roomy", 1024), ("tight", 96)):
        engine = NativeEngine(folder, dtype="float32", page_size=4, cache_tokens=cache_tokens, max_active=4, chunk_size=16, max_batch_tokens=64)
        ids = [engine.add_request(p, params, max_new_tokens=24) for p in prompts]
        engine.run_to_completion()
        results[name] = [engine.output(i) for i in ids]
        results[name + "_preemptions"] = engine.stats()["preemptions"]
        if name == "roomy":
            for rid, prompt, out in zip(ids, prompts, results[name]):
                assert len(out) == 24 and engine.request(rid)["finish_reason"] == "length"
                check_sampled(folder, prompt, out, rid, 0.8, 20, 0.95, 2)
    assert results["roomy_preemptions"] == 0 and results["tight_preemptions"] > 0
    assert results["roomy"] == results["tight"]


def test_native_program(tmp_path):
    """easy_llm, the C++ program: a model folder and prompts go in, token ids come out; no interpreter in that process."""
    from easy_gpt.cpp_b200.csrc.build import engine_paths

    _, exe = engine_paths()
    folder = tiny_configs.write_tiny("A", tmp_path / "m")
    prompts = tmp_path / "prompts.txt"
    prompts.write_text("5 17 3\n\n9,8,7,6\n")
    r = subprocess.run([str(exe), "--model", str(folder), "--token-ids", "--greedy", "--max-steps", "12", "--dtype", "float32", "-f", str(prompts)],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    lines = (tmp_path / "prompts_output.txt").read_text().splitlines()
    assert len(lines) == 2 and r.stdout.splitlines()[-2:] == lines
    outs = [[int(t) for t in line.split()] for line in lines]
    assert len(outs[0]) == 10 and len(outs[1]) == 9                       # max(1, max_steps - prompt + 1)
    check_greedy(folder, [[5, 17, 3], [9, 8, 7, 6]], outs, "float32", 1e-4)
    # a model folder written by the program itself, a prompt on the command line, sampling with the reference's defaults
    own = tmp_path / "own"
    cfg = tmp_path / "config.json"
    cfg.write_text((folder / "config.json").read_text())
    r = subprocess.run([str(exe), "--model", str(own), "--random-weights", "7", "--config", str(cfg), "--token-ids", "--max-steps", "20", "1 2 3 4"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert len(r.stdout.split()) == 17 and (own / "model.safetensors").is_file()
    r = subprocess.run([str(exe), "--model", str(tmp_path / "nowhere"), "--token-ids", "1 2"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 1 and "no config.json" in r.stderr
