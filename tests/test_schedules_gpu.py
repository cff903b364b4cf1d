"""The schedules a benchmark runs, against the plain implementation (GPU): many live requests
(decode buckets with padding rows, the decode attention's split policy for more than 16 tokens, the
products of 17 to 64 tokens), captured steps of several entries, the two tiny configurations of the
benchmark description with their workloads through the entry point (greedy and sampled), and
preemption of requests whose mixer keeps state of its own."""
import numpy as np
import pytest
import torch

import engine_harness as H
import plain_model
import tiny_configs

pytestmark = pytest.mark.gpu
TORCH_DTYPE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def plain_refs(folder, requests, dtype):
    cfg, w = plain_model.read_model_dir(folder, round_to_bf16=(dtype == "bfloat16"))
    return {rid: plain_model.forward_logits(cfg, w, toks).numpy() for rid, toks in requests.items()}


def tolerance(refs, dtype):
    return 1e-4 if dtype == "float32" else 1.5e-2 * max(float(np.abs(r).max()) for r in refs.values())


def trace_many_live(requests: dict, decode_tokens: int, per_step: int, portion: int):
    """All requests become live: their prompts go in `per_step` at a time in portions of `portion`
    tokens; then all of them decode together, one token each per step, for `decode_tokens` steps
    (every second step one request sits out, so that the batch size moves inside a bucket)."""
    steps = []
    rids = list(requests)
    for lo in range(0, len(rids), per_step):
        group = rids[lo:lo + per_step]
        pos = {r: 0 for r in group}
        while any(pos[r] < len(requests[r]) - decode_tokens for r in group):
            entries = []
            for r in group:
                head = len(requests[r]) - decode_tokens
                if pos[r] < head:
                    n = min(portion, head - pos[r])
                    entries.append({"id": r, "tokens": list(requests[r][pos[r]:pos[r] + n]), "want": [n - 1]})
                    pos[r] += n
            steps.append({"step": len(steps), "entries": entries, "end": []})
    pos = {r: len(requests[r]) - decode_tokens for r in rids}
    turn = 0
    while pos:
        sits_out = list(pos)[turn % len(pos)] if (turn % 2 == 1 and len(pos) > 1) else None
        entries, ended = [], []
        for r in list(pos):
            if r == sits_out:
                continue
            entries.append({"id": r, "tokens": [requests[r][pos[r]]], "want": [0]})
            pos[r] += 1
            if pos[r] == len(requests[r]):
                ended.append(r)
                del pos[r]
        steps.append({"step": len(steps), "entries": entries, "end": ended})
        turn += 1
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("live, config", [(8, "TINY_B"), (24, "C"), (64, "TINY_B"), (24, "D")])
def test_many_live_requests_match_plain(live, config, dtype, tmp_path):
    from easy_gpt.cpp_b200.engine import Model, StepRunner

    folder = tiny_configs.write_tiny(config, tmp_path / "m")
    vocab = tiny_configs.CONFIGS[config][0]["vocab_size"]
    rng = np.random.default_rng(live)
    requests = {f"q{i}": tiny_configs.random_tokens(vocab, int(rng.integers(20, 70)), 300 + i) for i in range(live)}
    refs = plain_refs(folder, requests, dtype)
    steps = trace_many_live(requests, decode_tokens=10, per_step=min(live, 12), portion=16)
    model = Model.from_dir(folder, device="cuda:0", dtype=TORCH_DTYPE[dtype])
    runner = StepRunner(model, page_size=16, num_pages=H.max_live_tokens(steps, 16) // 16, max_slots=live)
    got = H.run_in_process(runner, steps)
    worst = H.compare(got, refs, tolerance(refs, dtype), f"{live} live, {config}, {dtype}")
    print(f"{live} live {config} {dtype}: max |error| {worst:.3e}")
    assert runner.graph_replays >= 9                      # the decode steps went through a captured bucket
    assert not runner.cache.live_requests()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_shape_of_several_entries_is_captured_and_replayed(dtype, tmp_path):
    """Two decoding requests beside a portion of six tokens of a third, eight steps in a row: the shape
    is captured when it has come often enough and replayed afterwards; every step, eager or
    replayed, agrees with the plain implementation."""
    from easy_gpt.cpp_b200.engine import Model, StepRunner

    folder = tiny_configs.write_tiny("TINY_B", tmp_path / "m")
    requests = {"d0": tiny_configs.random_tokens(384, 40, 1), "d1": tiny_configs.random_tokens(384, 33, 2),
                "p": tiny_configs.random_tokens(384, 60, 3)}
    refs = plain_refs(folder, requests, dtype)
    steps = [{"step": 0, "entries": [{"id": "d0", "tokens": requests["d0"][:30], "want": [29]},
                                     {"id": "d1", "tokens": requests["d1"][:23], "want": [22]}], "end": []}]
    for i in range(10):
        steps.append({"step": len(steps), "end": [], "entries": [
            {"id": "d0", "tokens": [requests["d0"][30 + i]], "want": [0]},
            {"id": "d1", "tokens": [requests["d1"][23 + i]], "want": [0]},
            {"id": "p", "tokens": requests["p"][6 * i:6 * i + 6], "want": [0, 5]}]})
    steps[-1]["end"] = ["d0", "d1", "p"]
    model = Model.from_dir(folder, device="cuda:0", dtype=TORCH_DTYPE[dtype])
    runner = StepRunner(model, page_size=16, num_pages=H.max_live_tokens(steps, 16) // 16, max_slots=4)
    got = H.run_in_process(runner, steps)
    H.compare(got, refs, tolerance(refs, dtype), f"captured mixed step {dtype}")
    signature = ((1, 1, 6), ((0,), (0,), (0, 5)))
    assert any(key[:2] == signature for key in runner._signature_graphs)     # (the key's third part is the context bucket)
    assert runner.graph_replays >= 10 - runner.CAPTURE_MIXED_AFTER


# ---------------------------------------------------------------------------
# the benchmark description's two tiny configurations, with their workloads
# ---------------------------------------------------------------------------

def check_sampled(folder, prompt, out, request_id, temperature, top_k, top_p, seed, dtype="float32"):
    """Every sampled token is the plain rule's token for the plain logits of the same prefix and the
    uniform number keyed by (seed, request, index) (src/sampler.cpp:39-106).  Where the engine's
    logits (1e-4 from the plain ones) move a boundary of the CDF across the uniform number, the
    neighbouring token is accepted."""
    cfg, w = plain_model.read_model_dir(folder, round_to_bf16=(dtype == "bfloat16"))
    logits = plain_model.forward_logits(cfg, w, list(prompt) + list(out))
    exact = 0
    for i, tok in enumerate(out):
        row = logits[len(prompt) + i - 1]
        u = plain_model.uniform_from_counter(seed, request_id, i)
        want = plain_model.sample_token(row, temperature, top_k, top_p, u)
        if tok == want:
            exact += 1
            continue
        p = plain_model.sampling_distribution(row, temperature, top_k, top_p)
        cdf = np.cumsum(p)
        lo, hi = (cdf[tok - 1] if tok else 0.0), cdf[tok]
        assert p[tok] > 0 and lo - 5e-4 <= u <= hi + 5e-4, (i, tok, want, lo, u, hi)
    return exact


def test_tiny_a_workload_greedy_and_sampled(tmp_path):
    """Tiny A: 3 prompts of 5, 17 and 31 ids from seed 1, 16 new tokens each, pages of 4 tokens; once
    greedy and once at temperature 0.8 with sampling seed 2."""
    from easy_gpt.cpp_b200.engine import GptEngine
    from easy_gpt.cpp_b200.sampling import SamplingParams

    folder = tiny_configs.write_tiny("TINY_A", tmp_path / "m")
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, 256, size=n).tolist() for n in (5, 17, 31)]
    cfg, w = plain_model.read_model_dir(folder)
    engine = GptEngine(folder, dtype="float32", page_size=4, cache_tokens=256, max_active=4, chunk_size=16, max_batch_tokens=32)
    outs = engine.generate(prompts, max_new_tokens=16, greedy=True)
    for prompt, out in zip(prompts, outs):
        assert out == plain_model.greedy_generate(cfg, w, prompt, 16)
    params = SamplingParams(temperature=0.8, top_p=1.0, top_k=0, seed=2)
    requests = [engine.add_request(p, params, max_new_tokens=16) for p in prompts]
    engine.run_to_completion()
    exact = 0
    for r in requests:
        assert len(r.output) == 16 and not r.error
        exact += check_sampled(folder, r.prompt, r.output, r.id, 0.8, 0, 1.0, 2)
    assert exact >= 46                                    # of 48: a boundary case is rare
    assert len({tuple(r.output) for r in requests}) == 3
    # the reference's own defaults (top-k 20, top-p 0.95) through the same path
    params = SamplingParams(temperature=0.8, top_p=0.95, top_k=20, seed=2)
    requests = [engine.add_request(p, params, max_new_tokens=16) for p in prompts]
    engine.run_to_completion()
    for r in requests:
        check_sampled(folder, r.prompt, r.output, r.id, 0.8, 20, 0.95, 2)
    assert not engine.runner.cache.live_requests()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tiny_b_workload_chunked_prefill_beside_decoding(dtype, tmp_path):
    """Tiny B: 4 prompts of 1, 40, 77 and 130 ids from seed 4, prefilled in portions of 32 beside the
    requests that already decode, 24 new tokens each, pages of 16 tokens, through the scheduler."""
    from easy_gpt.cpp_b200.engine import GptEngine

    folder = tiny_configs.write_tiny("TINY_B", tmp_path / "m")
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, 384, size=n).tolist() for n in (1, 40, 77, 130)]
    engine = GptEngine(folder, dtype=dtype, page_size=16, cache_tokens=4 * 160, max_active=4, prefill_batch=2,
                       chunk_size=32, max_batch_tokens=36)
    outs = engine.generate(prompts, max_new_tokens=24, greedy=True)
    assert [len(o) for o in outs] == [24] * 4
    stats = engine.scheduler.stats
    assert stats.steps > 24 + 4                           # the prompts did not go in whole
    cfg, w = plain_model.read_model_dir(folder, round_to_bf16=(dtype == "bfloat16"))
    for prompt, out in zip(prompts, outs):
        logits = plain_model.forward_logits(cfg, w, list(prompt) + list(out))
        for i, tok in enumerate(out):
            row = logits[len(prompt) + i - 1]
            assert float(row.max() - row[tok]) <= (1e-4 if dtype == "float32" else 0.05), (dtype, i, tok, int(row.argmax()))
    if dtype == "float32":
        assert outs[1] == plain_model.greedy_generate(cfg, w, prompts[1], 24)


# ---------------------------------------------------------------------------
# preemption and slot reuse with a mixer that keeps state of its own
# ---------------------------------------------------------------------------

def test_state_slots_are_cleared_on_reuse_and_after_preemption(tmp_path):
    """A toy mixer with a running sum per request beside an attention layer, through the entry point
    with fewer slots than requests (slots are taken again by later requests) and with a cache so
    tight that running requests are preempted and computed again: every request's output is what
    it is when it runs alone."""
    from easy_gpt.cpp_b200 import register_part
    from easy_gpt.cpp_b200.config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
    from easy_gpt.cpp_b200.engine import GptEngine, Model
    from easy_gpt.cpp_b200.parts.base import Mixer, StateNeed
    from easy_gpt.cpp_b200.weights.loader import TensorRequest
    from easy_gpt.cpp_b200.weights.safetensors_io import write_safetensors
    import easy_gpt.cpp_b200.registry as registry

    class RunningSum(Mixer):
        """s <- 0.8 s + x W, out = s; s lives in the request's state slot."""

        def tensor_requests(self):
            n = self.params["hidden_size"]
            return [TensorRequest.matrix(self.prefix + ".w", n, n)]

        def load(self, tensors, device, dtype):
            self.w = tensors[self.prefix + ".w"].to(device=device, dtype=torch.float32)

        def cache_need(self):
            return StateNeed((self.params["hidden_size"],))

        def forward(self, x, ctx, cache):
            out = torch.empty_like(x)
            y = x.float() @ self.w.t()
            for i in range(ctx.num_seqs):
                lo, hi, slot = ctx.host_seq_starts[i], ctx.host_seq_starts[i + 1], ctx.host_seq_slots[i]
                s = cache.state[slot]
                for t in range(lo, hi):
                    s = 0.8 * s + y[t]
                    out[t] = s.to(x.dtype)
                cache.state[slot] = s
            return out

    register_part("mixer", "test_running_sum", RunningSum)
    hidden, vocab = 32, 64
    norm = lambda prefix: PartSpec("rmsnorm", dict(size=hidden, eps=1e-5), prefix)

    def build_spec(cfg):
        ff = lambda p: PartSpec("swiglu", dict(hidden_size=hidden, intermediate_size=48, bias=False), p)
        return ModelSpec(
            architecture="test_stateful", vocab_size=vocab, hidden_size=hidden, max_positions=512,
            layers=(LayerSpec(mixer=PartSpec("test_running_sum", dict(hidden_size=hidden), "l0.mix"), feed_forward=ff("l0.mlp"),
                              mixer_norm=norm("l0.n1"), feed_forward_norm=norm("l0.n2")),
                    LayerSpec(mixer=PartSpec("attention", dict(hidden_size=hidden, num_heads=2, num_kv_heads=1, head_dim=16,
                                                               qkv_bias=False, out_bias=False, window=None), "l1.att"),
                              feed_forward=ff("l1.mlp"), mixer_norm=norm("l1.n1"), feed_forward_norm=norm("l1.n2"),
                              position=PartSpec("rope", dict(head_dim=16, rotary_dim=16, theta=10000.0)))),
            run_order=(RunEntry(0, 0), RunEntry(1, 1)),
            embedding=PartSpec("embedding", dict(vocab_size=vocab, hidden_size=hidden), "emb"), final_norm=norm("norm"),
            lm_head=PartSpec("lm_head", dict(vocab_size=vocab, hidden_size=hidden, tied_to="emb"), "head"))

    registry.register_architecture("test_stateful", lambda d: d, build_spec)
    folder = tmp_path / "m"
    folder.mkdir()
    (folder / "config.json").write_text('{"architectures": ["test_stateful"], "model_type": "test_stateful"}')
    model = Model(build_spec({}), "cpu", torch.float32)
    g = torch.Generator().manual_seed(3)
    write_safetensors(folder / "model.safetensors", [
        (r.name, torch.ones(r.shapes[0]) if len(r.shapes[0]) == 1 else torch.randn(r.shapes[0], generator=g) * 0.3)
        for r in model.tensor_requests()])
    prompts = [tiny_configs.random_tokens(vocab, 6 + 5 * i, 40 + i) for i in range(6)]

    def generate(prompts, **options):
        engine = GptEngine(folder, dtype="float32", page_size=4, chunk_size=8, max_batch_tokens=24, **options)
        assert not engine.runner.use_graphs               # the toy mixer plans on the host: every step runs eagerly
        outs = engine.generate(prompts, max_new_tokens=20, greedy=True)
        return outs, engine.scheduler.stats.preemptions

    alone = [generate([p], cache_tokens=256, max_active=1)[0][0] for p in prompts]
    reused, _ = generate(prompts, cache_tokens=1024, max_active=2)          # six requests through two slots
    assert reused == alone
    tight, preemptions = generate(prompts, cache_tokens=112, max_active=4)
    assert preemptions > 0
    assert tight == alone
