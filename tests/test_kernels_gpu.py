"""Each kernel alone against its plain float32 reference, at sizes other than the
engine's tiny models (GPU)."""
import math

import numpy as np
import pytest
import torch

import plain_model

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gen(seed):
    return torch.Generator().manual_seed(seed)


# -- embedding ---------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_gather_and_bad_ids(dtype):
    from easy_gpt.cpp_b200 import kernels

    table = torch.randn(301, 70, generator=gen(0)).to(dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32)
    out = torch.full((5, 70), 7.0, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.embedding_gather(ids.to(DEV), table.to(DEV), out, status)
    assert torch.equal(out.cpu(), plain_model.embed(table.float(), ids.tolist()))
    assert status.item() == 0
    bad = torch.tensor([3, 301, -1], dtype=torch.int32, device=DEV)
    kernels.embedding_gather(bad, table.to(DEV), out[:3], status)
    assert status.item() == 1 and float(out[1].abs().sum()) == 0.0 and float(out[2].abs().sum()) == 0.0
    with pytest.raises(kernels.KernelError, match="no CPU path"):
        kernels.embedding_gather(ids, table, out.cpu(), status)


# -- norm ----------------------------------------------------------------------

@pytest.mark.parametrize("hidden, eps, rows", [(70, 1e-6, 9), (896, 1e-5, 9), (3584, 1e-6, 9), (5000, 3e-4, 9),
                                               (896, 1e-6, 203), (200, 1e-5, 64), (2048, 1e-6, 77), (1540, 1e-5, 130)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(hidden, eps, rows, dtype):
    from easy_gpt.cpp_b200 import kernels

    resid = torch.randn(rows, hidden, generator=gen(1)) * 3
    delta = (torch.randn(rows, hidden, generator=gen(2))).to(dtype)
    gain = 1 + 0.2 * torch.randn(hidden, generator=gen(3))
    want_resid = resid + delta.float()
    want = plain_model.rms_norm(want_resid, gain, eps)
    r = resid.to(DEV)
    out = torch.empty(rows, hidden, dtype=dtype, device=DEV)
    kernels.add_rmsnorm(r, delta.to(DEV), gain.to(DEV), out, eps)
    assert torch.equal(r.cpu(), want_resid)                        # the float32 sum is exact to the bit
    tol = 2e-6 * float(want.abs().max()) if dtype == torch.float32 else 8e-3 * float(want.abs().max())
    assert float((out.float().cpu() - want).abs().max()) <= tol
    # without delta; and only some rows (the final norm), residual untouched
    out2 = torch.empty(3, hidden, dtype=dtype, device=DEV)
    rows_idx = torch.tensor([7, 0, 4], dtype=torch.int32, device=DEV)
    before = r.clone()
    kernels.add_rmsnorm(r, delta.to(DEV), gain.to(DEV), out2, eps, rows=rows_idx)
    assert torch.equal(r, before)
    want2 = plain_model.rms_norm(want_resid[[7, 0, 4]] + delta.float()[[7, 0, 4]], gain, eps)
    assert float((out2.float().cpu() - want2).abs().max()) <= tol * 2
    kernels.add_rmsnorm(r, None, gain.to(DEV), out, eps)
    assert float((out.float().cpu() - want).abs().max()) <= tol


# -- float32 matrix product ---------------------------------------------------------

@pytest.mark.parametrize("M, N, K", [(1, 70, 33), (5, 1152, 896), (67, 129, 250), (130, 64, 17)])
def test_gemm_f32_is_true_32_bit_and_batch_invariant(M, N, K):
    from easy_gpt.cpp_b200 import kernels

    a = torch.randn(M, K, generator=gen(4))
    w = torch.randn(N, K, generator=gen(5))
    b = torch.randn(N, generator=gen(6))
    out = torch.empty(M, N, device=DEV)
    kernels.gemm_f32_nt(a.to(DEV), w.to(DEV), b.to(DEV), out)
    want = (a.double() @ w.double().t() + b.double())
    # float32 accumulation error of a K-term sum, far below TF32's 1e-3
    assert float((out.cpu().double() - want).abs().max()) <= 2e-6 * math.sqrt(K) * float(want.abs().max())
    # a row's result does not depend on the other rows of the batch
    one = torch.empty(1, N, device=DEV)
    kernels.gemm_f32_nt(a[M // 2:M // 2 + 1].to(DEV), w.to(DEV), b.to(DEV), one)
    assert torch.equal(one[0], out[M // 2])
    # strided input (a slice of a wider buffer)
    wide = torch.randn(M, K + 40, generator=gen(7)).to(DEV)
    kernels.gemm_f32_nt(wide[:, 8:8 + K], w.to(DEV), None, out)
    want = wide[:, 8:8 + K].cpu().double() @ w.double().t()
    assert float((out.cpu().double() - want).abs().max()) <= 2e-6 * math.sqrt(K) * float(want.abs().max())


# -- rotary encoding + cache write -----------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("NH, NKV, HD, rot, theta", [(4, 2, 16, 16, 1e4), (14, 2, 64, 64, 1e6), (3, 1, 48, 32, 5e4)])
def test_rope_cache(dtype, NH, NKV, HD, rot, theta):
    from easy_gpt.cpp_b200 import kernels
    from easy_gpt.cpp_b200.parts.rope import RotaryEncoding

    T, ps, pages = 11, 8, 6
    width = (NH + 2 * NKV) * HD
    qkv = torch.randn(T, width, generator=gen(8)).to(dtype)
    bias = torch.randn(width, generator=gen(9)) * 0.5
    positions = torch.tensor([0, 1, 2, 3, 4000, 4001, 7, 131071, 9, 10, 11], dtype=torch.int32)
    slots = torch.tensor([0, 1, 2, 3, 40, 41, 15, 16, 47, 8, 9], dtype=torch.int32)
    kc = torch.zeros(pages, NKV, ps, HD, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    inv = RotaryEncoding.inverse_frequencies(rot, theta)
    assert torch.equal(inv, plain_model.rope_inverse_frequencies(rot, theta))
    x = qkv.to(DEV).clone()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.rope_cache(x, bias.to(DEV), positions.to(DEV), slots.to(DEV), kc, vc, inv.to(DEV), NH, NKV, HD, rot, ps, status)
    assert status.item() == 0
    full = qkv.float() + bias
    q = full[:, :NH * HD].reshape(T, NH, HD)
    k = full[:, NH * HD:(NH + NKV) * HD].reshape(T, NKV, HD)
    v = full[:, (NH + NKV) * HD:].reshape(T, NKV, HD)

    def rotate(t):
        return torch.cat([plain_model.rope(t[..., :rot], positions.long(), theta), t[..., rot:]], dim=-1)

    tol = 3e-6 * float(full.abs().max()) if dtype == torch.float32 else 8e-3 * float(full.abs().max())
    assert float((x[:, :NH * HD].float().cpu().reshape(T, NH, HD) - rotate(q)).abs().max()) <= tol
    kr = rotate(k)
    for t in range(T):
        page, off = int(slots[t]) // ps, int(slots[t]) % ps
        assert float((kc[page, :, off].float().cpu() - kr[t]).abs().max()) <= tol
        assert float((vc[page, :, off].float().cpu() - v[t]).abs().max()) <= tol
    used = {(int(s) // ps, int(s) % ps) for s in slots}
    for page in range(pages):
        for off in range(ps):
            if (page, off) not in used:
                assert float(kc[page, :, off].abs().sum()) == 0.0       # nothing else was touched
    # a layer that reads another's cache: q rotated, nothing stored; and a bad slot is flagged
    kc.zero_()
    y = qkv.to(DEV).clone()
    kernels.rope_cache(y, bias.to(DEV), positions.to(DEV), None, None, None, inv.to(DEV), NH, NKV, HD, rot, ps, status)
    assert torch.equal(y[:, :NH * HD], x[:, :NH * HD]) and float(kc.abs().sum()) == 0.0
    kernels.rope_cache(y, None, positions.to(DEV), torch.full((T,), pages * ps, dtype=torch.int32, device=DEV), kc, vc,
                       inv.to(DEV), NH, NKV, HD, rot, ps, status)
    assert status.item() == 4


# -- attention over the paged cache ----------------------------------------------------------

def paged_case(seed, NH, NKV, HD, ps, contexts, queries, dtype, window=None, spike=None, point=None, point_strength=40.0,
               keep_keys=False):
    """Builds a cache holding `contexts[i] + queries[i]` keys for each sequence in
    shuffled pages, and the query tokens (the last queries[i] positions of each).
    ``point(sequence, position)`` names the key that the query at that position is aimed at (all of
    its heads): the query becomes point_strength times that key's direction, so the key's score
    stands out by far.  ``keep_keys``: the keys and values per sequence are returned too."""
    g = gen(seed)
    nseq = len(contexts)
    totals = [c + q for c, q in zip(contexts, queries)]
    pages_per = [-(-t // ps) for t in totals]
    num_pages = sum(pages_per) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    width = max(pages_per)
    table = torch.full((nseq, width), -1, dtype=torch.int32)
    kc = torch.randn(num_pages, NKV, ps, HD, generator=g)          # unused slots hold garbage on purpose
    vc = torch.randn(num_pages, NKV, ps, HD, generator=g)
    K, V = [], []
    it = iter(perm)
    for s in range(nseq):
        k = torch.randn(totals[s], NKV, HD, generator=g)
        v = torch.randn(totals[s], NKV, HD, generator=g)
        if spike is not None and totals[s] > spike[0]:
            k[spike[0]] *= spike[1]                                   # one far key that must not be missed
        for lp in range(pages_per[s]):
            page = next(it)
            table[s, lp] = page
            n = min(ps, totals[s] - lp * ps)
            kc[page, :, :n] = k[lp * ps:lp * ps + n].transpose(0, 1)
            vc[page, :, :n] = v[lp * ps:lp * ps + n].transpose(0, 1)
        K.append(k)
        V.append(v)
    T = sum(queries)
    q = torch.randn(T, NH, HD, generator=g)
    if point is not None:
        # every query head looks straight at one key of its KV head: that key's score beats all others by far
        row = 0
        for s in range(nseq):
            for i in range(queries[s]):
                j = point(s, contexts[s] + i)
                if j is not None and 0 <= j < totals[s]:
                    for h in range(NH):
                        kj = K[s][j, h // (NH // NKV)]
                        q[row + i, h] = point_strength * kj / kj.norm()
            row += queries[s]
    token_seq = torch.tensor([s for s in range(nseq) for _ in range(queries[s])], dtype=torch.int32)
    positions = torch.tensor([contexts[s] + i for s in range(nseq) for i in range(queries[s])], dtype=torch.int32)
    if dtype == torch.bfloat16:
        q, kc, vc = q.bfloat16(), kc.bfloat16(), vc.bfloat16()
        K = [k.bfloat16().float() for k in K]
        V = [v.bfloat16().float() for v in V]
    # plain reference: whole-sequence attention, rows of the query tokens picked out
    want = torch.empty(T, NH * HD)
    row = 0
    for s in range(nseq):
        n = totals[s]
        qs = torch.zeros(n, NH, HD)
        qs[contexts[s]:] = q[row:row + queries[s]].float()
        full = plain_model.attention_core(qs, K[s], V[s], torch.arange(n), window)
        want[row:row + queries[s]] = full[contexts[s]:]
        row += queries[s]
    out = dict(q=q.reshape(T, NH * HD), kc=kc, vc=vc, table=table, token_seq=token_seq, positions=positions, want=want)
    if keep_keys:
        out.update(keys=K, values=V)
    return out


ATTENTION_CASES = [
    # NH, NKV, HD, page, contexts, queries, window
    (4, 2, 16, 4, [0, 9, 30], [5, 1, 7], None),
    (6, 2, 32, 16, [100, 0, 63, 64], [1, 33, 1, 2], None),
    (14, 2, 64, 16, [700, 15, 16, 17], [1, 1, 1, 1], None),
    (14, 2, 64, 64, [300, 0], [40, 130], None),
    (12, 2, 128, 32, [257, 1000], [3, 1], None),
    (3, 1, 64, 16, [200, 90], [1, 20], 40),
    (8, 8, 32, 16, [77], [5], 17),
    (40, 2, 32, 16, [50], [2], None),            # 20 query heads per KV head: two row blocks
    (2, 1, 80, 16, [45], [4], None),             # a head size only the generic kernel takes
    (4, 2, 256, 16, [130], [2], None),
    (14, 2, 64, 16, [0, 100, 5], [200, 77, 64], None),        # prompt portions over several query tiles
    (6, 3, 128, 32, [31], [150], 50),
    (4, 1, 32, 16, [0], [129], 33),
    (14, 2, 64, 16, [1000, 0], [130, 515], None),             # many key tiles: every buffer of the pipeline comes round
    (4, 2, 64, 16, [300], [260], 100),                        # a window shorter than the portion
    (4, 4, 128, 16, [129], [300], None),
]


@pytest.mark.parametrize("case", ATTENTION_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_kernels(case, dtype):
    from easy_gpt.cpp_b200 import kernels

    NH, NKV, HD, ps, contexts, queries, window = case
    c = paged_case(11, NH, NKV, HD, ps, contexts, queries, dtype, window)
    scale = 1.0 / math.sqrt(HD)
    T = c["q"].shape[0]
    args = [c[k].to(DEV) for k in ("q", "kc", "vc", "table", "token_seq", "positions")]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    tol = 2e-5 if dtype == torch.float32 else 2.5e-2
    out = torch.zeros(T, NH * HD, dtype=dtype, device=DEV)
    kernels.attention_generic(*args, out, NH, NKV, HD, window, scale, status)
    assert status.item() == 0
    err = float((out.float().cpu() - c["want"]).abs().max())
    assert err <= tol, f"generic: {err}"
    if kernels.attention_paged_takes(dtype, HD, ps):
        for splits in (1, 2, 5, 64):
            out = torch.zeros(T, NH * HD, dtype=dtype, device=DEV)
            kernels.attention_paged(*args, out, NH, NKV, HD, window, scale, splits, status)
            assert status.item() == 0
            err = float((out.float().cpu() - c["want"]).abs().max())
            assert err <= tol, f"paged splits={splits}: {err}"
        # told how many keys were cached before the step, it fetches those ahead of its dependency wait
        out = torch.zeros(T, NH * HD, dtype=dtype, device=DEV)
        kernels.attention_paged(*args, out, NH, NKV, HD, window, scale, 3, status,
                                seq_context=torch.tensor(contexts, dtype=torch.int32, device=DEV))
        err = float((out.float().cpu() - c["want"]).abs().max())
        assert err <= tol and status.item() == 0, f"paged with seq_context: {err}"
        # only some tokens of the step (decoded tokens beside prompt portions): the others' rows stay as they were
        some = torch.arange(T - 1, -1, -2, dtype=torch.int32, device=DEV)
        out = torch.full((T, NH * HD), 5.0, dtype=dtype, device=DEV)
        kernels.attention_paged(*args, out, NH, NKV, HD, window, scale, 2, status, token_list=some)
        picked = some.long().cpu()
        err = float((out.float().cpu()[picked] - c["want"][picked]).abs().max())
        assert err <= tol and status.item() == 0, f"paged with a token list: {err}"
        rest = torch.ones(T, dtype=torch.bool)
        rest[picked] = False
        assert bool((out.float().cpu()[rest] == 5.0).all())
    else:
        assert dtype == torch.float32 or HD == 80 or ps % 16
        if dtype == torch.bfloat16:
            with pytest.raises(kernels.KernelError, match="attention_paged takes"):
                kernels.attention_paged(*args, out, NH, NKV, HD, window, scale, 1, status)
    if kernels.attention_prefill_takes(dtype, HD, ps):
        tiles, t0 = [], 0
        for s_idx, n in enumerate(queries):
            tiles += [(s_idx, t0 + o, min(64, n - o)) for o in range(0, n, 64)]
            t0 += n
        out = torch.zeros(T, NH * HD, dtype=dtype, device=DEV)
        kernels.attention_prefill(args[0], args[1], args[2], args[3], args[5], torch.tensor(tiles, dtype=torch.int32, device=DEV),
                                  out, NH, NKV, HD, window, scale, status)
        assert status.item() == 0
        err = float((out.float().cpu() - c["want"]).abs().max())
        assert err <= tol, f"prefill: {err}"
        # listed tiles may hold up to 128 tokens
        tiles, t0 = [], 0
        for s_idx, n in enumerate(queries):
            tiles += [(s_idx, t0 + o, min(128, n - o)) for o in range(0, n, 128)]
            t0 += n
        tiles = torch.tensor(tiles, dtype=torch.int32, device=DEV)
        out = torch.zeros(T, NH * HD, dtype=dtype, device=DEV)
        kernels.attention_prefill(args[0], args[1], args[2], args[3], args[5], tiles, out, NH, NKV, HD, window, scale, status)
        err = float((out.float().cpu() - c["want"]).abs().max())
        assert err <= tol and status.item() == 0, f"prefill, tiles of 128: {err}"
        if kernels.attention_prefill_tcgen05_takes(dtype, HD, ps):
            out = torch.zeros(T, NH * HD, dtype=dtype, device=DEV)
            kernels.attention_prefill_tcgen05(args[0], args[1], args[2], args[3], args[5], tiles, out, NH, NKV, HD, window,
                                              scale, status)
            assert status.item() == 0
            err = float((out.float().cpu() - c["want"]).abs().max())
            assert err <= tol, f"prefill tcgen05: {err}"
            # the keys of a query tile shared by several CTAs, merged by the last to finish; twice: the tickets return to zero
            for parts, part_tiles in ((2, 4), (5, 1), (5, 1), (16, 2)):
                out = torch.zeros(T, NH * HD, dtype=dtype, device=DEV)
                kernels.attention_prefill_tcgen05(args[0], args[1], args[2], args[3], args[5], tiles, out, NH, NKV, HD, window,
                                                  scale, status, parts=parts, part_tiles=part_tiles)
                err = float((out.float().cpu() - c["want"]).abs().max())
                assert err <= tol and status.item() == 0, f"prefill tcgen05, {parts} parts of {part_tiles} tiles: {err}"


def pointed_weight(c, NH, NKV, HD, s_keys, q_row, head, key, pos, window):
    """Softmax weight that query row `q_row`, head `head` gives key `key` under the causal / window mask (float64)."""
    k = s_keys[:pos + 1, head // (NH // NKV)].double()
    scores = (k @ c["q"].float().reshape(-1, NH, HD)[q_row, head].double()) / math.sqrt(HD)
    if window is not None:
        scores[:max(0, pos - window + 1)] = -math.inf
    w = torch.softmax(scores, 0)
    return float(w[key]) if key <= pos else 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_one_far_key_and_a_windows_edge(dtype):
    """Every query head points at one key among hundreds, so that this key carries nearly all the weight
    when it is visible: at position 0, at a page's edge, at a tile's edge, far away, and just inside /
    just outside a window's edge.  A kernel that misses the key, or sees one it must not, is off by
    the size of a value."""
    from easy_gpt.cpp_b200 import kernels

    NH, NKV, HD, ps = 4, 2, 64, 16
    scale = 1.0 / math.sqrt(HD)
    for far, window in ((0, None), (63, None), (64, None), (511, None), (600 - 100 + 1, 100), (600 - 100, 100)):
        c = paged_case(far + 1, NH, NKV, HD, ps, [600], [1], dtype, window, point=lambda s, pos: far, keep_keys=True)
        visible = window is None or far > 600 - window
        weight = pointed_weight(c, NH, NKV, HD, c["keys"][0], 0, 1, far, 600, window)
        v_far = c["values"][0][far].repeat_interleave(NH // NKV, dim=0).reshape(-1)
        if visible:
            assert weight > 0.9, (far, window, weight)
            assert float((c["want"][0] - v_far).abs().max()) < 0.5
        else:
            assert weight == 0.0 and float((c["want"][0] - v_far).abs().max()) > 1.0
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        dev = [c[k].to(DEV) for k in ("q", "kc", "vc", "table", "token_seq", "positions")]
        tol = 3e-5 if dtype == torch.float32 else 3e-2
        runs = [("generic", lambda out: kernels.attention_generic(*dev, out, NH, NKV, HD, window, scale, status))]
        if dtype == torch.bfloat16:
            runs += [(f"paged splits={n}", lambda out, n=n: kernels.attention_paged(*dev, out, NH, NKV, HD, window, scale, n, status))
                     for n in (1, 3, 8)]
        for name, run in runs:
            out = torch.zeros(1, NH * HD, dtype=dtype, device=DEV)
            run(out)
            err = float((out.float().cpu() - c["want"]).abs().max())
            assert err <= tol and status.item() == 0, (name, far, window, err)


POINTED_PREFILL_CASES = [
    # NH, NKV, HD, contexts, queries, window, which key the query at position p points at
    (4, 2, 64, [300], [260], 100, lambda s, p: p - 99 if p % 2 == 0 else p - 100),       # just inside / just outside the window
    (4, 2, 64, [129], [300], None, lambda s, p: (p, p + 1, p - 1)[p % 3]),                 # the diagonal, one beyond it, one before
    (4, 2, 128, [200], [200], None, lambda s, p: (63, 64, 127, 128, 0, 191, 192)[p % 7]),  # edges of the tiles of 64 and 128 keys
    (14, 2, 64, [0, 70], [333, 190], 150, lambda s, p: (p - 149, p - 150, p, p + 1)[p % 4] if p >= 150 else (0, p)[p % 2]),
    (6, 2, 32, [40], [150], 33, lambda s, p: (p - 32, p - 33, p)[p % 3] if p >= 33 else p),
]


@pytest.mark.parametrize("case", POINTED_PREFILL_CASES)
def test_prompt_attention_at_the_windows_edge_the_diagonal_and_tile_edges(case):
    """The prompt-portion kernels (warp-level and tcgen05, keys cut into parts and not) on queries that each
    point at one key: the first key inside the window or the last one outside it, the token itself or
    the one after it, keys on both sides of a tile's edge."""
    from easy_gpt.cpp_b200 import kernels

    NH, NKV, HD, contexts, queries, window, point = case
    ps = 16
    c = paged_case(5, NH, NKV, HD, ps, contexts, queries, torch.bfloat16, window, point=point, keep_keys=True)
    scale = 1.0 / math.sqrt(HD)
    # the oracle's own sanity: the pointed key dominates where it is visible and has no weight where it is not
    row, seen, hidden = 0, 0, 0
    for s, (ctx, n) in enumerate(zip(contexts, queries)):
        for i in range(0, n, 7):
            pos = ctx + i
            key = point(s, pos)
            w = pointed_weight(c, NH, NKV, HD, c["keys"][s], row + i, NH - 1, key, pos, window) if 0 <= key < ctx + n else None
            if w is None:
                continue
            visible = key <= pos and (window is None or key > pos - window)
            assert (w > 0.9) if visible else (w == 0.0), (s, pos, key, w)
            seen, hidden = seen + visible, hidden + (not visible)
        row += n
    assert seen > 5 and (hidden > 5 or case is POINTED_PREFILL_CASES[2])      # (the tile-edge case points at visible keys only)
    T = c["q"].shape[0]
    args = [c[k].to(DEV) for k in ("q", "kc", "vc", "table", "token_seq", "positions")]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    tol = 3e-2
    for tile in (64, 128):
        tiles, t0 = [], 0
        for s_idx, n in enumerate(queries):
            tiles += [(s_idx, t0 + o, min(tile, n - o)) for o in range(0, n, tile)]
            t0 += n
        tiles = torch.tensor(tiles, dtype=torch.int32, device=DEV)
        out = torch.zeros(T, NH * HD, dtype=torch.bfloat16, device=DEV)
        kernels.attention_prefill(args[0], args[1], args[2], args[3], args[5], tiles, out, NH, NKV, HD, window, scale, status)
        err = float((out.float().cpu() - c["want"]).abs().max())
        assert err <= tol and status.item() == 0, f"warp-level, tiles of {tile}: {err}"
    if kernels.attention_prefill_tcgen05_takes(torch.bfloat16, HD, ps):
        for parts, part_tiles in ((1, 0), (3, 1), (8, 1), (2, 2)):
            out = torch.zeros(T, NH * HD, dtype=torch.bfloat16, device=DEV)
            kernels.attention_prefill_tcgen05(args[0], args[1], args[2], args[3], args[5], tiles, out, NH, NKV, HD, window, scale,
                                              status, parts=parts, part_tiles=part_tiles)
            err = float((out.float().cpu() - c["want"]).abs().max())
            assert err <= tol and status.item() == 0, f"tcgen05, {parts} parts of {part_tiles} tiles: {err}"
    # the decode kernel takes the same tokens one by one
    for splits in (1, 4):
        out = torch.zeros(T, NH * HD, dtype=torch.bfloat16, device=DEV)
        kernels.attention_paged(*args, out, NH, NKV, HD, window, scale, splits, status)
        err = float((out.float().cpu() - c["want"]).abs().max())
        assert err <= tol and status.item() == 0, f"paged, {splits} splits: {err}"


def test_attention_flags_a_missing_page():
    from easy_gpt.cpp_b200 import kernels

    c = paged_case(3, 4, 2, 64, 16, [40], [1], torch.bfloat16)
    c["table"][0, 1] = -1
    dev = [c[k].to(DEV) for k in ("q", "kc", "vc", "table", "token_seq", "positions")]
    for fn, extra in ((kernels.attention_generic, ()), (kernels.attention_paged, (2,))):
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        out = torch.zeros(1, 4 * 64, dtype=torch.bfloat16, device=DEV)
        fn(*dev, out, 4, 2, 64, None, 0.125, *extra, status)
        assert status.item() == 2
        assert torch.isfinite(out.float()).all()


# -- SwiGLU ---------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T, I", [(1, 208), (7, 4864), (300, 37)])
def test_swiglu(dtype, T, I):
    from easy_gpt.cpp_b200 import kernels

    gu = (torch.randn(T, 2 * I, generator=gen(12)) * 3).to(dtype)
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    kernels.swiglu(gu.to(DEV), out)
    g, u = gu.float()[:, 0::2], gu.float()[:, 1::2]                 # interleaved rows: gate_0, up_0, gate_1, ...
    want = u * (g * (1.0 / (1.0 + torch.exp(-g))))
    tol = 1e-6 * float(want.abs().max()) if dtype == torch.float32 else 8e-3 * float(want.abs().max())
    assert float((out.float().cpu() - want).abs().max()) <= tol


# -- the decode-step product with its prologues and epilogues -------------------------------

def bf(t):
    return t.to(torch.bfloat16)


@pytest.mark.parametrize("M", [1, 3, 8, 13, 32, 64])
@pytest.mark.parametrize("N, K, plan", [(48, 48, (1, 1, 1)), (1152, 896, (4, 2, 1)), (200, 4864, (1, 8, 3)), (391, 80, (8, 2, 1)),
                                        (896, 896, (2, 4, 2)), (896, 4864, None), (4000, 208, None)])
def test_gemm_skinny_plain(M, N, K, plan):
    from easy_gpt.cpp_b200 import kernels

    x = bf(torch.randn(M, K, generator=gen(20)))
    w = bf(torch.randn(N, K, generator=gen(21)) * 0.1)
    b = torch.randn(N, generator=gen(22))
    want = x.float() @ w.float().t() + b
    scale = float(want.abs().max())
    out32 = torch.empty(M, N, device=DEV)
    kernels.gemm_skinny(w.to(DEV), b.to(DEV), out32, kernels.EPI_F32, x=x.to(DEV), plan=plan)
    assert float((out32.cpu() - want).abs().max()) <= 1e-5 * scale * math.sqrt(K)          # float32 accumulation
    out16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_skinny(w.to(DEV), None, out16, kernels.EPI_STORE, x=x.to(DEV))
    assert float((out16.float().cpu() - (want - b)).abs().max()) <= 8e-3 * scale
    # a token's result does not depend on the other tokens of the step
    one = torch.empty(1, N, device=DEV)
    kernels.gemm_skinny(w.to(DEV), b.to(DEV), one, kernels.EPI_F32, x=x[M - 1:M].to(DEV).clone(), plan=plan)
    assert float((one[0] - out32[M - 1]).abs().max()) <= 1e-6 * scale


@pytest.mark.parametrize("M", [2, 8, 40])
def test_gemm_skinny_norm_prologue_and_swiglu(M):
    from easy_gpt.cpp_b200 import kernels

    K, I = 896, 304
    resid = torch.randn(M, K, generator=gen(23)) * 2
    delta = bf(torch.randn(M, K, generator=gen(24)))
    gain = 1 + 0.1 * torch.randn(K, generator=gen(25))
    gate, up = torch.randn(I, K, generator=gen(26)) * 0.05, torch.randn(I, K, generator=gen(27)) * 0.05
    w = bf(torch.stack([gate, up], dim=1).reshape(2 * I, K))
    eps = 1e-5
    summed = resid + delta.float()
    xn = bf(plain_model.rms_norm(summed, gain, eps)).float()                     # the kernel rounds x to bfloat16 too
    g = xn @ bf(gate).float().t()
    u = xn @ bf(up).float().t()
    want = u * (g / (1 + torch.exp(-g)))
    out = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    r_in, r_out = resid.to(DEV), torch.zeros(M, K, device=DEV)
    kernels.gemm_skinny(w.to(DEV), None, out, kernels.EPI_SWIGLU, resid_in=r_in, resid_out=r_out, delta=delta.to(DEV),
                        gain=gain.to(DEV), eps=eps)
    assert torch.equal(r_out.cpu(), summed) and torch.equal(r_in.cpu(), resid)
    assert float((out.float().cpu() - want).abs().max()) <= 1e-2 * float(want.abs().max())
    # without delta: nothing is written to a residual
    out2 = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_skinny(w.to(DEV), None, out2, kernels.EPI_SWIGLU, resid_in=r_out, gain=gain.to(DEV), eps=eps)
    assert float((out2.float() - out.float()).abs().max()) <= 1e-2 * float(want.abs().max())


@pytest.mark.parametrize("M, H, I, plan", [(1, 896, 4864, None), (8, 896, 4864, None), (5, 208, 304, (1, 4, 1)),
                                          (13, 80, 176, (2, 2, 3)), (16, 1536, 2048, None)])
def test_gemm_skinny_residual_norm_epilogue_feeds_prenormed_prologue(M, H, I, plan):
    """A product that adds its result to the residual and prepares the next norm (down or O product), and a
    second product that starts from those rows and partial sums (gate/up): against add, RMSNorm and the
    products one by one."""
    from easy_gpt.cpp_b200 import kernels

    act = bf(torch.randn(M, I, generator=gen(61)))
    w_down = bf(torch.randn(H, I, generator=gen(62)) * 0.05)
    bias = torch.randn(H, generator=gen(63)) * 0.1
    resid = torch.randn(M, H, generator=gen(64)) * 2
    gain = 1 + 0.1 * torch.randn(H, generator=gen(65))
    gate, up = torch.randn(72, H, generator=gen(66)) * 0.05, torch.randn(72, H, generator=gen(67)) * 0.05
    w_next = bf(torch.stack([gate, up], dim=1).reshape(144, H))
    eps = 1e-5
    delta = bf(act.float() @ w_down.float().t() + bias).float()
    summed = resid + delta
    xn = bf(plain_model.rms_norm(summed, gain, eps)).float()
    g, u = xn @ bf(gate).float().t(), xn @ bf(up).float().t()
    want = u * (g / (1 + torch.exp(-g)))

    r = resid.to(DEV)
    rows, ss_parts = kernels.gemm_skinny(w_down.to(DEV), bias.to(DEV), None, kernels.EPI_RESID_NORM, x=act.to(DEV), plan=plan,
                                         follow=dict(residual=r, gain=gain.to(DEV)))
    # the sum differs from the reference's by the rounding of the product only (the delta is rounded to bfloat16)
    assert float((r.cpu() - summed).abs().max()) <= 2 ** -7 * float(delta.abs().max()) + 1e-6
    assert ss_parts.shape[1] == kernels.skinny_padded_tokens(M)
    v = r.cpu()
    assert torch.allclose(ss_parts.sum(0).cpu()[:M], (v * v).sum(1), rtol=1e-5)
    assert torch.equal(rows.cpu(), bf(gain * v))
    out = torch.empty(M, 72, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.gemm_skinny(w_next.to(DEV), None, out, kernels.EPI_SWIGLU, prenormed=(rows, ss_parts), eps=eps, status=status)
    assert int(status.item()) == 0
    assert float((out.float().cpu() - want).abs().max()) <= 1e-2 * float(want.abs().max())


@pytest.mark.parametrize("NH, NKV, HD", [(14, 2, 64), (6, 2, 32), (3, 1, 128), (4, 4, 16)])
def test_gemm_skinny_qkv_rope_cache(NH, NKV, HD):
    """The fused kernel against the unfused chain: norm, product, rope_cache."""
    from easy_gpt.cpp_b200 import kernels
    from easy_gpt.cpp_b200.parts.rope import RotaryEncoding

    M, K, ps, pages = 5, 80 if HD == 16 else 896, 16, 9      # K = 80: a width that is no multiple of 64
    N = (NH + 2 * NKV) * HD
    resid = torch.randn(M, K, generator=gen(30))
    delta = bf(torch.randn(M, K, generator=gen(31)) * 0.5)
    gain = 1 + 0.1 * torch.randn(K, generator=gen(32))
    w = bf(torch.randn(N, K, generator=gen(33)) * 0.05)
    bias = torch.randn(N, generator=gen(34)) * 0.3
    positions = torch.tensor([0, 5, 77, 4000, 130], dtype=torch.int32)
    slots = torch.tensor([3, 20, 143, 64, 17], dtype=torch.int32)
    inv = RotaryEncoding.inverse_frequencies(HD, 1e6)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kc = torch.zeros(pages, NKV, ps, HD, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    q = torch.empty(M, NH * HD, dtype=torch.bfloat16, device=DEV)
    r_out = torch.empty(M, K, device=DEV)
    kernels.gemm_skinny(w.to(DEV), bias.to(DEV), q, kernels.EPI_QKV_ROPE, resid_in=resid.to(DEV), resid_out=r_out,
                        delta=delta.to(DEV), gain=gain.to(DEV), eps=1e-6,
                        rope=dict(num_heads=NH, num_kv_heads=NKV, head_dim=HD, positions=positions.to(DEV),
                                  slot_map=slots.to(DEV), k_cache=kc, v_cache=vc, inv_freq=inv.to(DEV), status=status))
    assert status.item() == 0
    # plain chain in float32 on the same bfloat16-rounded inputs
    xn = bf(plain_model.rms_norm(resid + delta.float(), gain, 1e-6)).float()
    full = xn @ w.float().t() + bias
    qw = plain_model.rope(full[:, :NH * HD].reshape(M, NH, HD), positions.long(), 1e6).reshape(M, -1)
    kw = plain_model.rope(full[:, NH * HD:(NH + NKV) * HD].reshape(M, NKV, HD), positions.long(), 1e6)
    vw = full[:, (NH + NKV) * HD:].reshape(M, NKV, HD)
    tol = 1e-2 * float(full.abs().max())
    assert float((q.float().cpu() - qw).abs().max()) <= tol
    for m in range(M):
        page, off = int(slots[m]) // ps, int(slots[m]) % ps
        assert float((kc[page, :, off].float().cpu() - kw[m]).abs().max()) <= tol
        assert float((vc[page, :, off].float().cpu() - vw[m]).abs().max()) <= tol
    assert int((kc.float().abs().sum(dim=(1, 3)) > 0).sum()) == M                  # only the five slots were written


def test_gemm_skinny_refuses_what_it_does_not_take():
    from easy_gpt.cpp_b200 import kernels

    w = bf(torch.randn(32, 48)).to(DEV)
    with pytest.raises(kernels.KernelError, match="takes 1..64 tokens"):
        kernels.gemm_skinny(w, None, torch.empty(65, 32, dtype=torch.bfloat16, device=DEV), kernels.EPI_STORE,
                            x=bf(torch.randn(65, 48)).to(DEV))
    w2 = bf(torch.randn(32, 40)).to(DEV)
    with pytest.raises(kernels.KernelError):
        kernels.gemm_skinny(w2, None, torch.empty(2, 32, dtype=torch.bfloat16, device=DEV), kernels.EPI_STORE,
                            x=bf(torch.randn(2, 40)).to(DEV))


@pytest.mark.parametrize("dtype, T, NH, NKV, HD, ps, pages", [
    (torch.float32, 37, 5, 1, 24, 8, 7), (torch.bfloat16, 37, 5, 1, 48, 8, 7),       # half a head: three 16-byte pieces
    (torch.float32, 300, 6, 3, 32, 16, 20), (torch.bfloat16, 300, 6, 3, 64, 16, 20)])
def test_rope_cache_with_table_equals_rope_cache(dtype, T, NH, NKV, HD, ps, pages):
    from easy_gpt.cpp_b200 import kernels
    from easy_gpt.cpp_b200.parts.rope import RotaryEncoding

    width = (NH + 2 * NKV) * HD
    qkv = torch.randn(T, width, generator=gen(40)).to(dtype).to(DEV)
    positions = torch.randint(0, 70000, (T,), generator=gen(41), dtype=torch.int32).to(DEV)
    slots = torch.randperm(pages * ps, generator=gen(42))[:T].to(torch.int32).to(DEV)
    inv = RotaryEncoding.inverse_frequencies(HD, 1e6).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    a, b = qkv.clone(), qkv.clone()
    ka, va = (torch.zeros(pages, NKV, ps, HD, dtype=dtype, device=DEV) for _ in range(2))
    kb, vb = torch.zeros_like(ka), torch.zeros_like(va)
    kernels.rope_cache(a, None, positions, slots, ka, va, inv, NH, NKV, HD, HD, ps, status)
    table = kernels.rope_table(positions, inv)
    ang = positions.float()[:, None] * inv[None, :]
    assert torch.equal(table[..., 0], torch.cos(ang)) or float((table[..., 0] - torch.cos(ang)).abs().max()) <= 2e-7
    kernels.rope_cache_table(b, table, slots, kb, vb, NH, NKV, HD, ps, status)
    # the same cos/sin and the same formula; in float32 the compiler may fuse the multiply-adds of the two
    # kernels differently, which is worth one rounding of the result
    ulp = 0.0 if dtype == torch.bfloat16 else 2.5e-7 * float(a.float().abs().max())
    for x, y in ((a, b), (ka, kb), (va, vb)):
        assert float((x.float() - y.float()).abs().max()) <= ulp
    assert status.item() == 0


def test_kernels_are_right_without_clusters_too():
    """Where CTAs share a result (the decode attention's splits, the K parts of a decode product) they meet in a
    cluster's shared memory if the launch allows it, else through scratch memory and a ticket.  The tests above take
    whichever path the launcher chooses; here the same tests run once more in a process that has the clusters
    switched off, so that the ticket paths stay covered."""
    import os
    import subprocess
    import sys

    env = dict(os.environ, EASY_GPT_CLUSTER_MERGE="0", EASY_GPT_CLUSTER_REDUCE="0")
    out = subprocess.run([sys.executable, "-m", "pytest", __file__, "-q", "-x", "-m", "gpu", "-k", "(paged or skinny or attention) and not without_clusters and not softmax_groups"],
                         env=env, capture_output=True, text=True, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-2000:]
    assert " passed" in out.stdout


@pytest.mark.parametrize("groups", [1, 2])
def test_prompt_attention_with_either_number_of_softmax_groups(groups):
    """The tcgen05 prompt attention has two forms: CTAs with one softmax group, two to an SM, and CTAs with two groups
    that share a unit's key tiles, one to an SM; the launcher picks by head size.  Here the attention tests run once
    more with either form forced for every head size."""
    import os
    import subprocess
    import sys

    env = dict(os.environ, EASY_GPT_PREFILL_GROUPS=str(groups))
    out = subprocess.run([sys.executable, "-m", "pytest", __file__, "-q", "-x", "-m", "gpu", "-k", "(attention or prefill) and not without_clusters and not softmax_groups"],
                         env=env, capture_output=True, text=True, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-2000:]
    assert " passed" in out.stdout
