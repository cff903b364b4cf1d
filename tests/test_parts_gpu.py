"""Each part alone against the plain implementation, a model whose run order names
a layer twice and lets a layer read another layer's cache, and toy parts defined
here (a mixer with state of its own, a routed feed-forward, another position
encoding) that are registered, built and stepped without touching the package (GPU)."""
import json
import math

import numpy as np
import pytest
import torch

import engine_harness as H
import plain_model
import tiny_configs

pytestmark = pytest.mark.gpu
DEV = "cuda"


def make_ctx(dtype, seqs, page_size=16, kv=None):
    """A StepContext and CacheManager for sequences given as (context, query) lengths."""
    from easy_gpt.cpp_b200.cache import CacheManager
    from easy_gpt.cpp_b200.parts.base import GroupTables, StepContext

    needs = {0: kv} if kv is not None else {}
    total = sum(c + q for c, q in seqs)
    cache = CacheManager(needs, page_size, -(-total // page_size) + len(seqs) + 2, len(seqs), 4096, device=DEV, dtype=dtype)
    starts, context, slots, token_seq, positions = [0], [], [], [], []
    for i, (c, q) in enumerate(seqs):
        slots.append(cache.begin_request(i))
        if c:
            cache.reserve(i, c)
            cache.commit(i, c)
        cache.reserve(i, q)
        context.append(c)
        starts.append(starts[-1] + q)
        token_seq += [i] * q
        positions += list(range(c, c + q))
    T = starts[-1]
    t32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    groups = {}
    for g in cache.groups:
        width = max(-(-(c + q) // page_size) for c, q in seqs)
        table = t32(cache.table_rows(g.index, list(range(len(seqs))), width).tolist())
        slot_map = t32(np.concatenate([cache.slot_positions(g.index, i, c, q) for i, (c, q) in enumerate(seqs)]).tolist())
        groups[g.index] = GroupTables(page_size, table, slot_map)
    tiles = [(i, starts[i] + o, min(64, q - o)) for i, (c, q) in enumerate(seqs) for o in range(0, q, 64)]
    ctx = StepContext(dtype=dtype, device=torch.device(DEV), num_tokens=T, num_seqs=len(seqs),
                      token_ids=torch.zeros(T, dtype=torch.int32, device=DEV), positions=t32(positions),
                      token_seq=t32(token_seq), seq_starts=t32(starts), seq_context=t32(context), seq_slots=t32(slots),
                      status=torch.zeros(1, dtype=torch.int32, device=DEV), groups=groups, host_seq_starts=starts,
                      host_seq_context=context, host_seq_slots=slots, max_query_len=max(q for _, q in seqs),
                      max_context_len=max(c + q for c, q in seqs), all_decode=all(q == 1 for _, q in seqs),
                      query_tiles=t32(tiles))
    return ctx, cache


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_rope_feed_forward_and_head_alone(dtype, tmp_path):
    from easy_gpt.cpp_b200.parts.embedding import LMHead, TokenEmbedding
    from easy_gpt.cpp_b200.parts.mlp import SwiGLU
    from easy_gpt.cpp_b200.parts.norm import RMSNorm

    tol = 2e-5 if dtype == torch.float32 else 3e-2
    g = torch.Generator().manual_seed(0)
    H_, I_, V_, T = 96, 208, 391, 21
    ctx, _ = make_ctx(dtype, [(0, T)])
    lowp = (lambda t: t) if dtype == torch.float32 else (lambda t: t.bfloat16().float())

    # norm (its own eps), on all rows and on a few
    norm = RMSNorm(dict(size=H_, eps=3e-4), "n")
    gain = 1 + 0.2 * torch.randn(H_, generator=g)
    norm.load({"n.weight": gain}, DEV, dtype)
    resid, delta = torch.randn(T, H_, generator=g), lowp(torch.randn(T, H_, generator=g))
    r = resid.to(DEV)
    out = norm.forward(r, delta.to(DEV).to(dtype), torch.empty(T, H_, dtype=dtype, device=DEV))
    want = plain_model.rms_norm(resid + delta, gain, 3e-4)
    assert float((out.float().cpu() - want).abs().max()) <= tol * float(want.abs().max())
    assert torch.equal(r.cpu(), resid + delta)

    # feed-forward (interleaved gate/up inside, plain names outside)
    ff = SwiGLU(dict(hidden_size=H_, intermediate_size=I_, bias=True), "mlp")
    w = {f"mlp.{n}_proj.weight": lowp(torch.randn(*s, generator=g) * 0.1) for n, s in
         (("gate", (I_, H_)), ("up", (I_, H_)), ("down", (H_, I_)))}
    w.update({f"mlp.{n}_proj.bias": torch.randn(s, generator=g) * 0.1 for n, s in (("gate", I_), ("up", I_), ("down", H_))})
    ff.load(w, DEV, dtype)
    x = lowp(torch.randn(T, H_, generator=g))
    got = ff.forward(x.to(DEV).to(dtype), ctx)
    want = plain_model.swiglu_mlp(x, {"L." + k: v for k, v in w.items()}, "L.")
    assert float((got.float().cpu() - want).abs().max()) <= tol * float(want.abs().max())

    # embedding and heads, tied and not
    emb = TokenEmbedding(dict(vocab_size=V_, hidden_size=H_), "emb")
    table = lowp(torch.randn(V_, H_, generator=g))
    emb.load({"emb.weight": table}, DEV, dtype)
    ids = torch.randint(0, V_, (T,), generator=g, dtype=torch.int32)
    r = torch.empty(T, H_, device=DEV)
    ctx.token_ids = ids.to(DEV)
    emb.forward(ctx, r)
    assert torch.equal(r.cpu(), table[ids.long()])
    for tied in (True, False):
        head = LMHead(dict(vocab_size=V_, hidden_size=H_, tied_to="emb" if tied else None), "head")
        hw = lowp(torch.randn(V_, H_, generator=g) * 0.1)
        head.load({"head.weight": hw}, DEV, dtype, tied_table=emb.table)
        assert (head.linear.weight.data_ptr() == emb.table.data_ptr()) == tied       # tied: the table itself, no copy
        logits = head.forward(x.to(DEV).to(dtype))
        want = x @ (table if tied else hw).t()
        assert logits.dtype == torch.float32
        assert float((logits.cpu() - want).abs().max()) <= tol * float(want.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 19])
def test_attention_part_alone(dtype, window):
    """Portions, continuations and single tokens in one batch, with and without a window."""
    from easy_gpt.cpp_b200.parts.attention import Attention
    from easy_gpt.cpp_b200.parts.base import PagedKVNeed
    from easy_gpt.cpp_b200.parts.rope import RotaryEncoding

    g = torch.Generator().manual_seed(1)
    H_, NH, NKV, HD = 112, 6, 2, 32
    lowp = (lambda t: t) if dtype == torch.float32 else (lambda t: t.bfloat16().float())
    rope = RotaryEncoding(dict(head_dim=HD, rotary_dim=HD, theta=50000.0))
    att = Attention(dict(hidden_size=H_, num_heads=NH, num_kv_heads=NKV, head_dim=HD, qkv_bias=True, out_bias=True,
                         window=window), "a", rope)
    assert att.cache_need() == PagedKVNeed(NKV, HD, window)
    w = {"a.q_proj.weight": (NH * HD, H_), "a.k_proj.weight": (NKV * HD, H_), "a.v_proj.weight": (NKV * HD, H_),
         "a.o_proj.weight": (H_, NH * HD)}
    w = {k: lowp(torch.randn(*s, generator=g) * 0.15) for k, s in w.items()}
    w.update({"a.q_proj.bias": torch.randn(NH * HD, generator=g) * 0.2, "a.k_proj.bias": torch.randn(NKV * HD, generator=g) * 0.2,
              "a.v_proj.bias": torch.randn(NKV * HD, generator=g) * 0.2, "a.o_proj.bias": torch.randn(H_, generator=g) * 0.2})
    assert sorted(r.name for r in att.tensor_requests()) == sorted(w)
    att.load(w, DEV, dtype)
    lengths = [70, 33, 50]
    xs = [lowp(torch.randn(n, H_, generator=g)) for n in lengths]
    sizes = dict(NH=NH, NKV=NKV, HD=HD, theta=50000.0)
    want = [plain_model.attention(x, {"L.self_attn." + k[2:]: v for k, v in w.items()}, "L.", sizes,
                                  torch.arange(len(x)), window) for x in xs]
    # step 1: first parts of all three; step 2: a portion, a single token, a two-token portion
    cuts = [[(0, 41), (41, 29)], [(0, 32), (32, 1)], [(0, 48), (48, 2)]]
    from easy_gpt.cpp_b200.cache import CacheManager
    ctx, cache = make_ctx(dtype, [(0, c[0][1]) for c in cuts], kv=att.cache_need())
    tol = (3e-5 if dtype == torch.float32 else 3e-2) * max(float(x.abs().max()) for x in want)
    view = cache.view(0)
    out = att.forward(torch.cat([x[:c[0][1]] for x, c in zip(xs, cuts)]).to(DEV).to(dtype), ctx, view)
    got = out.float().cpu().split([c[0][1] for c in cuts])
    for i in range(3):
        assert float((got[i] - want[i][:cuts[i][0][1]]).abs().max()) <= tol
        cache.commit(i, cuts[i][0][1])
    # second step on the same cache
    from easy_gpt.cpp_b200.parts.base import GroupTables
    seqs = [(c[1][0], c[1][1]) for c in cuts]
    for i, (c, q) in enumerate(seqs):
        cache.reserve(i, q)
    t32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    starts = [0]
    for _, q in seqs:
        starts.append(starts[-1] + q)
    width = max(-(-(c + q) // 16) for c, q in seqs)
    ctx2, _ = make_ctx(dtype, seqs)            # metadata only; tables come from the live cache
    ctx2.groups = {0: GroupTables(16, t32(cache.table_rows(0, [0, 1, 2], width).tolist()),
                                  t32(np.concatenate([cache.slot_positions(0, i, c, q) for i, (c, q) in enumerate(seqs)]).tolist()))}
    out = att.forward(torch.cat([x[c:c + q] for x, (c, q) in zip(xs, seqs)]).to(DEV).to(dtype), ctx2, view)
    got = out.float().cpu().split([q for _, q in seqs])
    for i, (c, q) in enumerate(seqs):
        assert float((got[i] - want[i][c:c + q]).abs().max()) <= tol, (i, window)
    assert ctx.status.item() == 0 and ctx2.status.item() == 0


# ---------------------------------------------------------------------------
# a run order that names a layer twice and lets a layer read another layer's cache
# ---------------------------------------------------------------------------

def plain_with_run_order(cfg, w, ids, order):
    """order: (layer, cache, writes).  A reading entry attends the keys and values that the
    writing entry of its cache computed (from that entry's input), with its own queries."""
    sz = plain_model.sizes(cfg)
    pos = torch.arange(len(ids))
    x = plain_model.embed(w["model.embed_tokens.weight"], ids)
    kv = {}
    for layer, cache, writes in order:
        p = f"model.layers.{layer}."
        h = plain_model.rms_norm(x, w[p + "input_layernorm.weight"], sz["eps"])
        T = len(ids)
        q = plain_model.linear(h, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"]).reshape(T, sz["NH"], sz["HD"])
        q = plain_model.rope(q, pos, sz["theta"])
        if writes:
            k = plain_model.linear(h, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"]).reshape(T, sz["NKV"], sz["HD"])
            v = plain_model.linear(h, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"]).reshape(T, sz["NKV"], sz["HD"])
            kv[cache] = (plain_model.rope(k, pos, sz["theta"]), v)
        k, v = kv[cache]
        a = plain_model.linear(plain_model.attention_core(q, k, v, pos, sz["window"][layer]), w[p + "self_attn.o_proj.weight"])
        x = x + a
        x = x + plain_model.swiglu_mlp(plain_model.rms_norm(x, w[p + "post_attention_layernorm.weight"], sz["eps"]), w, p)
    return plain_model.lm_head(x, w, sz)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_run_order_with_a_repeated_layer_and_a_shared_cache(dtype, tmp_path):
    import dataclasses

    from easy_gpt.cpp_b200.config.spec import RunEntry
    from easy_gpt.cpp_b200.engine import Model, StepRunner
    from easy_gpt.cpp_b200.registry import model_spec_from_config

    folder = tiny_configs.write_tiny("A", tmp_path / "m")
    # layer 0, layer 1, layer 0 again (own cache), layer 1 reading the cache that its first run wrote
    order = [(0, 0, True), (1, 1, True), (0, 2, True), (1, 1, False)]
    spec = dataclasses.replace(model_spec_from_config(tiny_configs.CONFIG_A),
                               run_order=tuple(RunEntry(l, c, wr) for l, c, wr in order))
    tdtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    model = Model(spec, DEV, tdtype)
    model.load_weights(folder / "model.safetensors")
    assert sorted(model.cache_needs()) == [0, 1, 2]
    cfg, w = plain_model.read_model_dir(folder, round_to_bf16=(dtype == "bfloat16"))
    requests = {"a": tiny_configs.random_tokens(256, 75, 1), "b": tiny_configs.random_tokens(256, 40, 2)}
    refs = {rid: plain_with_run_order(cfg, w, ids, order).numpy() for rid, ids in requests.items()}
    steps = H.trace_mixed(requests, portion=9)
    runner = StepRunner(model, page_size=16, num_pages=H.max_live_tokens(steps) // 16, max_slots=4)
    got = H.run_in_process(runner, steps)
    tol = 1e-4 if dtype == "float32" else 3e-2 * max(float(np.abs(r).max()) for r in refs.values())
    H.compare(got, refs, tol, f"run order {dtype}")


# ---------------------------------------------------------------------------
# toy parts, defined and registered here
# ---------------------------------------------------------------------------

def register_toys():
    from easy_gpt.cpp_b200 import register_part
    from easy_gpt.cpp_b200.parts.base import FeedForward, Mixer, PositionEncoding, StateNeed
    from easy_gpt.cpp_b200.weights.loader import TensorRequest

    class DecayingSum(Mixer):
        """A mixer with state of fixed size per request: s <- decay * s + x W; out = s.
        (Toy: plain torch ops, one request after another.)"""

        def tensor_requests(self):
            n = self.params["hidden_size"]
            return [TensorRequest.matrix(self.prefix + ".w", n, n)]

        def load(self, tensors, device, dtype):
            self.w = tensors[self.prefix + ".w"].to(device=device, dtype=torch.float32)
            self.decay = float(self.params["decay"])

        def cache_need(self):
            return StateNeed((self.params["hidden_size"],))

        def forward(self, x, ctx, cache):
            out = torch.empty_like(x)
            y = x.float() @ self.w.t()
            for i in range(ctx.num_seqs):
                lo, hi, slot = ctx.host_seq_starts[i], ctx.host_seq_starts[i + 1], ctx.host_seq_slots[i]
                s = cache.state[slot]
                for t in range(lo, hi):
                    s = self.decay * s + y[t]
                    out[t] = s.to(x.dtype)
                cache.state[slot] = s
            return out

    class TopOneExperts(FeedForward):
        """A routed feed-forward: each token goes to the expert with the largest router logit
        (computed in float32) and gets relu(x W_e) scaled by the softmax weight of that expert."""

        def tensor_requests(self):
            n, e = self.params["hidden_size"], self.params["experts"]
            return [TensorRequest.matrix(self.prefix + ".router", e, n)] + \
                   [TensorRequest.matrix(f"{self.prefix}.expert{i}", n, n) for i in range(e)]

        def load(self, tensors, device, dtype):
            e = self.params["experts"]
            self.router = tensors[self.prefix + ".router"].to(device=device, dtype=torch.float32)
            self.experts = torch.stack([tensors[f"{self.prefix}.expert{i}"] for i in range(e)]).to(device=device, dtype=torch.float32)

        def forward(self, x, ctx):
            logits = x.float() @ self.router.t()
            prob, choice = torch.softmax(logits, dim=-1).max(dim=-1)
            y = torch.relu(torch.einsum("th,thk->tk", x.float(), self.experts[choice].transpose(1, 2)))
            return (y * prob[:, None]).to(x.dtype)

    class LearnedOffsets(PositionEncoding):
        """Another position encoding: a learned vector per position, added to the residual stream at the embedding."""

        def tensor_requests(self):
            return [TensorRequest.matrix(self.prefix + ".table", self.params["max_positions"], self.params["hidden_size"])]

        def load(self, tensors, device, dtype):
            self.table = tensors[self.prefix + ".table"].to(device=device, dtype=torch.float32)

        def add_to_embedding(self, residual, ctx):
            residual += self.table[ctx.positions.long()]

    class SignFlip(PositionEncoding):
        """A position encoding that is no half rotation: queries and keys at odd positions change sign
        (so scores between positions of different parity are negated)."""

        def apply_to_query_key(self, q, k, ctx):
            sign = (1 - 2 * (ctx.positions % 2)).to(q.dtype)[:, None, None]
            q.mul_(sign)
            k.mul_(sign)

    register_part("mixer", "toy_decaying_sum", DecayingSum)
    register_part("feed_forward", "toy_top_one_experts", TopOneExperts)
    register_part("position", "toy_learned_offsets", LearnedOffsets)
    register_part("position", "toy_sign_flip", SignFlip)


def toy_attention(h, w, p, pos, flip=False, rotate=True):
    """The framework's attention restated with the toy model's options: no rotation at all, or the
    sign flip of the toy position encoding in place of it."""
    T = h.shape[0]
    q = (h @ w[p + ".att.q_proj.weight"].t()).reshape(T, 2, 16)
    k = (h @ w[p + ".att.k_proj.weight"].t()).reshape(T, 1, 16)
    v = (h @ w[p + ".att.v_proj.weight"].t()).reshape(T, 1, 16)
    if rotate:
        q, k = plain_model.rope(q, pos, 10000.0), plain_model.rope(k, pos, 10000.0)
    if flip:
        sign = (1 - 2 * (pos % 2)).float()[:, None, None]
        q, k = q * sign, k * sign
    return plain_model.attention_core(q, k, v, pos) @ w[p + ".att.o_proj.weight"].t()


def toy_reference(w, ids, hidden, experts, decay, eps):
    pos = torch.arange(len(ids))
    x = w["emb.weight"][torch.tensor(ids)] + w["pos.table"][pos]          # learned positions at the embedding
    norm = lambda name, t: plain_model.rms_norm(t, w[name + ".weight"], eps)
    # layer 0 (pre-norm): the toy mixer with state of its own, then routed experts
    y = norm("l0.n1", x) @ w["l0.mix.w"].t()
    s, outs = torch.zeros(hidden), []
    for t in range(len(ids)):
        s = decay * s + y[t]
        outs.append(s)
    x = x + torch.stack(outs)
    h = norm("l0.n2", x)
    prob, choice = torch.softmax(h @ w["l0.ff.router"].t(), -1).max(-1)
    ex = torch.stack([w[f"l0.ff.expert{i}"] for i in range(experts)])
    x = x + torch.relu(torch.einsum("th,thk->tk", h, ex[choice].transpose(1, 2))) * prob[:, None]
    # layer 1 (post-norm): x = norm(x + attention(x)); x = norm(x + swiglu(x))
    x = norm("l1.n1", x + toy_attention(x, w, "l1", pos))
    x = norm("l1.n2", x + plain_model.swiglu_mlp(x, {"L.mlp." + k.split(".", 2)[2]: v for k, v in w.items() if k.startswith("l1.mlp.")}, "L."))
    # layer 2: attention with the sign-flip encoding between two norms (a sandwich), and no feed-forward
    x = x + norm("l2.n_out", toy_attention(norm("l2.n_in", x), w, "l2", pos, flip=True, rotate=False))
    # layer 3: attention with no position encoding and no norm at all
    x = x + toy_attention(x, w, "l3", pos, rotate=False)
    return norm("norm", x) @ w["emb.weight"].t()


def test_toy_parts_register_build_and_step(tmp_path):
    """A model of a toy layer (mixer with state, routed experts) behind learned positions at the
    embedding, a post-norm layer, a layer with norms on both sides of its mixer, another position
    encoding and no feed-forward, and a layer with no norm and no position encoding: built from a
    spec alone, loaded by name, stepped in portions and single tokens with requests coming and
    going; the state slots are zeroed and kept per request."""
    from easy_gpt.cpp_b200.config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
    from easy_gpt.cpp_b200.engine import Model, StepRunner
    from easy_gpt.cpp_b200.weights.safetensors_io import write_safetensors

    register_toys()
    hidden, vocab, experts, decay, eps = 32, 50, 3, 0.9, 1e-5
    norm = lambda prefix: PartSpec("rmsnorm", dict(size=hidden, eps=eps), prefix)
    from easy_gpt.cpp_b200.config.spec import SubLayerSpec

    attention = lambda prefix: PartSpec("attention", dict(hidden_size=hidden, num_heads=2, num_kv_heads=1, head_dim=16,
                                                            qkv_bias=False, out_bias=False, window=None), prefix)
    spec = ModelSpec(
        architecture="toy", vocab_size=vocab, hidden_size=hidden, max_positions=256,
        layers=(
            # pre-norm, written with the four fields
            LayerSpec(mixer=PartSpec("toy_decaying_sum", dict(hidden_size=hidden, decay=decay), "l0.mix"),
                      feed_forward=PartSpec("toy_top_one_experts", dict(hidden_size=hidden, experts=experts), "l0.ff"),
                      mixer_norm=norm("l0.n1"), feed_forward_norm=norm("l0.n2")),
            # post-norm, by spec alone
            LayerSpec(sublayers=(SubLayerSpec("mixer", attention("l1.att"), norm("l1.n1"), "post"),
                                 SubLayerSpec("feed_forward", PartSpec("swiglu", dict(hidden_size=hidden, intermediate_size=48, bias=False), "l1.mlp"),
                                              norm("l1.n2"), "post")),
                      position=PartSpec("rope", dict(head_dim=16, rotary_dim=16, theta=10000.0))),
            # a norm before and a norm after the mixer, another position encoding, no feed-forward
            LayerSpec(sublayers=(SubLayerSpec("mixer", attention("l2.att"), norm("l2.n_in"), "pre", output_norm=norm("l2.n_out")),),
                      position=PartSpec("toy_sign_flip")),
            # no norm and no position encoding at all
            LayerSpec(sublayers=(SubLayerSpec("mixer", attention("l3.att")),)),
        ),
        run_order=(RunEntry(0, 0), RunEntry(1, 1), RunEntry(2, 2), RunEntry(3, 3)),
        embedding=PartSpec("embedding", dict(vocab_size=vocab, hidden_size=hidden), "emb"),
        embedding_position=PartSpec("toy_learned_offsets", dict(hidden_size=hidden, max_positions=256), "pos"),
        final_norm=norm("norm"), lm_head=PartSpec("lm_head", dict(vocab_size=vocab, hidden_size=hidden, tied_to="emb"), "head"))
    model = Model(spec, DEV, torch.float32)
    g = torch.Generator().manual_seed(7)
    w = {}
    for r in model.tensor_requests():
        shape = r.shapes[0]
        w[r.name] = torch.ones(shape) + 0.1 * torch.randn(shape, generator=g) if len(shape) == 1 else torch.randn(shape, generator=g) * 0.2
    write_safetensors(tmp_path / "toy.safetensors", w.items())
    model.load_weights(tmp_path / "toy.safetensors")
    from easy_gpt.cpp_b200.parts.base import PagedKVNeed, StateNeed
    kv = PagedKVNeed(1, 16, None)
    assert model.cache_needs() == {0: StateNeed((hidden,)), 1: kv, 2: kv, 3: kv}

    requests = {f"r{i}": np.random.default_rng(i).integers(0, vocab, n).tolist() for i, n in enumerate([40, 23, 64, 31, 12])}
    refs = {rid: toy_reference(w, ids, hidden, experts, decay, eps).numpy() for rid, ids in requests.items()}
    steps = H.trace_mixed(requests, portion=7, max_live=3)
    runner = StepRunner(model, page_size=16, num_pages=H.max_live_tokens(steps) // 16, max_slots=3)
    got = H.run_in_process(runner, steps)
    assert len(got) == sum(len(v) for v in requests.values())
    H.compare(got, refs, 2e-4, "toy parts")
