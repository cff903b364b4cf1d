"""The host runtime's packing of a step's metadata (no GPU): against a restatement in numpy, for
random batches over a cache whose pages have been used before."""
import numpy as np
from hypothesis import given, settings, strategies as st

from easy_gpt.cpp_b200 import host
from easy_gpt.cpp_b200.cache import CacheManager
from easy_gpt.cpp_b200.parts.base import PagedKVNeed

QUERY_TILE, SMALL = 128, 4


def manager(page_size, num_pages=64, slots=6):
    return CacheManager({0: PagedKVNeed(2, 16, None), 1: PagedKVNeed(2, 16, 3 * page_size)}, page_size, num_pages, slots, 4096)


def pack(m, rids, token_lists, want_lists):
    n = len(rids)
    handles = np.array([m.handle(r, create=True) for r in rids], dtype=np.int64)
    counts = np.array([len(t) for t in token_lists], dtype=np.int64)
    info = np.zeros(3, dtype=np.int32)
    rc = m._lib.egh_step_reserve(m.core, n, handles.ctypes.data, counts.ctypes.data, info.ctypes.data)
    if rc != 0:
        return rc, None
    tokens = np.concatenate([np.asarray(t, dtype=np.int64) for t in token_lists])
    want_offsets = np.zeros(n + 1, dtype=np.int64)
    want_offsets[1:] = np.cumsum([len(w) for w in want_lists])
    wants = np.array([w for ws in want_lists for w in ws], dtype=np.int64)
    G = len(m.groups)
    bound = m._lib.egh_step_bound(m.core, n, int(counts.sum()), len(wants), QUERY_TILE)
    buf = np.full(bound, -7, dtype=np.int32)
    layout = np.zeros(2 * (9 + 2 * G), dtype=np.int64)
    widths = np.zeros(G, dtype=np.int32)
    scalars = np.zeros(8, dtype=np.int64)
    rc = m._lib.egh_step_pack(m.core, n, handles.ctypes.data, counts.ctypes.data, tokens.ctypes.data, want_offsets.ctypes.data,
                              wants.ctypes.data, QUERY_TILE, SMALL, buf.ctypes.data, bound, layout.ctypes.data,
                              widths.ctypes.data, scalars.ctypes.data)
    assert rc == 0 and scalars[0] <= bound
    names = ["token_ids", "positions", "token_seq", "seq_starts", "seq_context", "seq_slots", "logit_rows", "query_tiles",
             "small_tokens"] + [f"{k}{g}" for g in range(G) for k in ("slot_map", "table")]
    out = {name: buf[layout[2 * i]:layout[2 * i] + layout[2 * i + 1]].copy() for i, name in enumerate(names)}
    for i in range(len(names) - 1):                      # sections do not overlap and start on 16 bytes
        assert layout[2 * i] % 4 == 0 and layout[2 * i] + layout[2 * i + 1] <= layout[2 * (i + 1)]
    return 0, dict(out, widths=widths.tolist(), scalars=scalars.tolist())


def expected(m, rids, token_lists, want_lists, lengths_before):
    """The same arrays from numpy and the manager's slower queries."""
    n = len(rids)
    counts = np.array([len(t) for t in token_lists])
    starts = np.zeros(n + 1, dtype=np.int64)
    starts[1:] = np.cumsum(counts)
    context = np.array(lengths_before)
    T = int(counts.sum())
    want = {"token_ids": np.concatenate([np.asarray(t) for t in token_lists]),
            "positions": np.arange(T) - np.repeat(starts[:-1], counts) + np.repeat(context, counts),
            "token_seq": np.repeat(np.arange(n), counts), "seq_starts": starts, "seq_context": context,
            "seq_slots": np.array([m.slot_of(r) for r in rids]),
            "logit_rows": np.array([starts[i] + w for i, ws in enumerate(want_lists) for w in ws], dtype=np.int64)}
    tiles, small = [], []
    for i, c in enumerate(counts):
        if c > SMALL:
            tiles += [(i, starts[i] + o, min(QUERY_TILE, c - o)) for o in range(0, c, QUERY_TILE)]
        else:
            small += list(range(starts[i], starts[i] + c))
    want["query_tiles"] = np.array(tiles, dtype=np.int64).reshape(-1)
    want["small_tokens"] = np.array(small, dtype=np.int64)
    width = -(-int((context + counts).max()) // m.page_size)
    for g in m.groups:
        want[f"slot_map{g.index}"] = np.concatenate([m.slot_positions(g.index, r, int(context[i]), int(counts[i]))
                                                     for i, r in enumerate(rids)])
        want[f"table{g.index}"] = m.table_rows(g.index, rids, width).reshape(-1)
    return want, width


@settings(max_examples=40, deadline=None)
@given(st.lists(st.lists(st.tuples(st.integers(0, 5), st.integers(1, 300)), min_size=1, max_size=4, unique_by=lambda t: t[0]),
                min_size=1, max_size=12), st.sampled_from([4, 16]), st.randoms(use_true_random=False))
def test_packed_steps_equal_the_numpy_restatement(steps, page_size, rnd):
    m = manager(page_size)
    lengths = {}
    for step in steps:
        rids = [r for r, _ in step]
        token_lists = [[rnd.randrange(1000) for _ in range(c)] for _, c in step]
        want_lists = [sorted(rnd.sample(range(c), min(c, rnd.randrange(0, 3)))) for _, c in step]
        before = [lengths.get(r, 0) for r in rids]
        free = [g.pool.free_count for g in m.groups]
        live = set(m.live_requests())
        rc, got = pack(m, rids, token_lists, want_lists)
        if rc != 0:
            # nothing changed: no request begun, no page taken
            assert rc in (host.OUT_OF_PAGES, host.TOO_LONG)
            assert [g.pool.free_count for g in m.groups] == free and set(m.live_requests()) == live
            m.check()
            victim = max(lengths, key=lengths.get, default=None)
            if victim is not None:
                m.end_request(victim)
                del lengths[victim]
            continue
        want, width = expected(m, rids, token_lists, want_lists, before)
        for name, arr in want.items():
            assert got[name].tolist() == arr.tolist(), name
        assert got["widths"] == [width] * len(m.groups)
        T = sum(c for _, c in step)
        assert got["scalars"][1:6] == [T, sum(len(w) for w in want_lists), max(c for _, c in step),
                                       max(b + c for b, (_, c) in zip(before, step)), int(all(c == 1 for _, c in step))]
        for (r, c) in step:
            m.commit(r, c)
            lengths[r] = lengths.get(r, 0) + c
        m.check()
        if rnd.random() < 0.3:
            r = rnd.choice(list(lengths))
            m.end_request(r)
            del lengths[r]


def test_replay_pack_writes_the_live_rows_only():
    m = manager(4)
    for rid, n in ((3, 9), (8, 5)):
        m.begin_request(rid)
        m.reserve(rid, n)
        m.commit(rid, n)
        m.reserve(rid, 2)
    counts = np.array([2, 2, 2], dtype=np.int32)             # a signature of three entries, two of them live
    handles = np.array([3, 8], dtype=np.int64)
    W = m.max_pages_per_request
    off = {"positions": 0, "context": 8, "slots": 12, "slot_map": [16, 24], "table": [32, 32 + 3 * W]}
    buf = np.full(32 + 6 * W, -7, dtype=np.int32)
    off_slot_map, off_table = np.array(off["slot_map"], dtype=np.int64), np.array(off["table"], dtype=np.int64)
    rc = m._lib.egh_replay_pack(m.core, 2, handles.ctypes.data, counts.ctypes.data, buf.ctypes.data, off["positions"], off["context"],
                                off["slots"], off_slot_map.ctypes.data, off_table.ctypes.data, W)
    assert rc == 0
    assert buf[0:6].tolist() == [9, 10, 5, 6, -7, -7]
    assert buf[8:11].tolist() == [9, 5, -7] and buf[12:15].tolist() == [m.slot_of(3), m.slot_of(8), -7]
    for g in m.groups:
        sm = np.concatenate([m.slot_positions(g.index, 3, 9, 2), m.slot_positions(g.index, 8, 5, 2)])
        assert buf[off["slot_map"][g.index]:off["slot_map"][g.index] + 4].tolist() == sm.tolist()
        rows = buf[off["table"][g.index]:off["table"][g.index] + 3 * W].reshape(3, W)
        assert rows[:2].tolist() == m.table_rows(g.index, [3, 8], W).tolist() and (rows[2] == -7).all()
    missing = np.array([3, 99], dtype=np.int64)
    assert m._lib.egh_replay_pack(m.core, 2, missing.ctypes.data, counts.ctypes.data, buf.ctypes.data, 0, 8, 12,
                                  off_slot_map.ctypes.data, off_table.ctypes.data, W) == host.UNKNOWN_REQUEST
