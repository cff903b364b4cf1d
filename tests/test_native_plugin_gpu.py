"""A plugin of the native engine, defined by the tests (tests/native/toy_plugin.cu): a mixer with state of its own, a routed
feed-forward, learned positions at the embedding, and an architecture that puts them beside the engine's own attention and
SwiGLU in a post-norm layer.  It is built, loaded, and its model stepped, generated from and preempted without a change to
the engine's files (GPU)."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import engine_harness as H
import plain_model

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
HIDDEN, VOCAB, EXPERTS, DECAY, EPS, POSITIONS = 32, 50, 3, 0.9, 1e-5, 256


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    from easy_gpt.cpp_b200 import native
    from easy_gpt.cpp_b200.csrc.build import build_plugin
    from easy_gpt.cpp_b200.weights.safetensors_io import write_safetensors

    folder = tmp_path_factory.mktemp("toy_native")
    native.load_plugin(build_plugin(ROOT / "tests" / "native" / "toy_plugin.cu", folder / "libtoy_plugin.so"))
    (folder / "config.json").write_text(json.dumps({"architectures": ["ToyModel"], "model_type": "toy_native", "width": HIDDEN, "vocabulary": VOCAB,
                                                    "experts": EXPERTS, "positions": POSITIONS, "eps": EPS, "decay": DECAY}))
    g = torch.Generator().manual_seed(7)
    mat = lambda *shape: torch.randn(*shape, generator=g) * 0.2
    gain = lambda: torch.ones(HIDDEN) + 0.1 * torch.randn(HIDDEN, generator=g)
    w = {"emb.weight": mat(VOCAB, HIDDEN), "pos.table": mat(POSITIONS, HIDDEN), "l0.mix.w": mat(HIDDEN, HIDDEN), "l0.ff.router": mat(EXPERTS, HIDDEN),
         "l0.n1.weight": gain(), "l0.n2.weight": gain(), "l1.n1.weight": gain(), "l1.n2.weight": gain(), "norm.weight": gain(),
         "l1.att.q_proj.weight": mat(32, HIDDEN), "l1.att.k_proj.weight": mat(16, HIDDEN), "l1.att.v_proj.weight": mat(16, HIDDEN),
         "l1.att.o_proj.weight": mat(HIDDEN, 32), "l1.mlp.gate_proj.weight": mat(48, HIDDEN), "l1.mlp.up_proj.weight": mat(48, HIDDEN),
         "l1.mlp.down_proj.weight": mat(HIDDEN, 48)}
    for e in range(EXPERTS):
        w[f"l0.ff.expert{e}"] = mat(HIDDEN, HIDDEN)
    write_safetensors(folder / "model.safetensors", w.items())
    return dict(folder=folder, weights=w)


def reference(w, ids):
    pos = torch.arange(len(ids))
    norm = lambda name, t: plain_model.rms_norm(t, w[name + ".weight"], EPS)
    x = w["emb.weight"][torch.tensor(ids)] + w["pos.table"][pos]
    y = norm("l0.n1", x) @ w["l0.mix.w"].t()
    s, outs = torch.zeros(HIDDEN), []
    for t in range(len(ids)):
        s = DECAY * s + y[t]
        outs.append(s)
    x = x + torch.stack(outs)
    h = norm("l0.n2", x)
    prob, choice = torch.softmax(h @ w["l0.ff.router"].t(), -1).max(-1)
    ex = torch.stack([w[f"l0.ff.expert{i}"] for i in range(EXPERTS)])
    x = x + torch.relu(torch.einsum("th,thk->tk", h, ex[choice].transpose(1, 2))) * prob[:, None]
    sz = dict(NH=2, NKV=1, HD=16, theta=10000.0)
    att = plain_model.attention(x, {"L.self_attn." + k.split(".", 2)[2]: v for k, v in w.items() if k.startswith("l1.att.")}, "L.", sz, pos, None)
    x = norm("l1.n1", x + att)
    x = norm("l1.n2", x + plain_model.swiglu_mlp(x, {"L.mlp." + k.split(".", 2)[2]: v for k, v in w.items() if k.startswith("l1.mlp.")}, "L."))
    return norm("norm", x) @ w["emb.weight"].t()


def test_plugin_model_steps_like_its_reference(toy):
    from easy_gpt.cpp_b200.native import NativeStepRunner
    from test_native_engine_gpu import run_native

    requests = {f"r{i}": np.random.default_rng(i).integers(0, VOCAB, n).tolist() for i, n in enumerate([40, 23, 64, 31, 12])}
    refs = {rid: reference(toy["weights"], ids).numpy() for rid, ids in requests.items()}
    steps = H.trace_mixed(requests, portion=7, max_live=3)
    runner = NativeStepRunner(toy["folder"], "float32", 16, H.max_live_tokens(steps, 16) // 16, 3)
    got = run_native(runner, steps)
    assert len(got) == sum(len(v) for v in requests.values())
    H.compare(got, refs, 2e-4, "plugin parts")
    assert runner.info("graph_replays") > 0            # the toy parts are capturable: single tokens went through captured steps


def test_plugin_state_is_cleared_for_every_new_owner_of_a_slot(toy):
    """Generation through the native entry point with fewer slots than requests, and with a cache so tight that running
    requests are preempted and computed again: every request's tokens are what they are when it runs alone."""
    from easy_gpt.cpp_b200.native import NativeEngine

    prompts = [np.random.default_rng(40 + i).integers(0, VOCAB, 6 + 5 * i).tolist() for i in range(6)]

    def generate(prompts, **options):
        engine = NativeEngine(toy["folder"], dtype="float32", page_size=4, chunk_size=8, max_batch_tokens=24, **options)
        return engine.generate(prompts, max_new_tokens=20, greedy=True), engine.stats()["preemptions"]

    alone = [generate([p], cache_tokens=256, max_active=1)[0][0] for p in prompts]
    logits = reference(toy["weights"], prompts[2] + alone[2])
    for i, tok in enumerate(alone[2]):
        row = logits[len(prompts[2]) + i - 1]
        assert float(row.max() - row[tok]) <= 2e-4
    reused, _ = generate(prompts, cache_tokens=1024, max_active=2)          # six requests through two slots
    assert reused == alone
    tight, preemptions = generate(prompts, cache_tokens=112, max_active=4)
    assert preemptions > 0 and tight == alone


def test_unknown_architecture_and_missing_plugin(tmp_path):
    from easy_gpt.cpp_b200 import native

    with pytest.raises(native.NativeError, match="cannot load the plugin"):
        native.load_plugin(tmp_path / "nothing.so")
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["SomethingElse"], "model_type": "else"}))
    with pytest.raises(native.NativeError, match="Unsupported model architecture/model_type: architecture='SomethingElse', model_type='else'"):
        native.NativeStepRunner(tmp_path, "float32", 16, 4, 2)
