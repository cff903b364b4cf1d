"""Traces in the format of bin/trace_run, and ways to run them: in process
through StepRunner, or through the bin/trace_run program."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent


# ---------------------------------------------------------------------------
# traces: lists of {"step", "entries": [{"id", "tokens", "want"}], "end"}
# ---------------------------------------------------------------------------

def trace_whole(requests: dict):
    """Each request alone and whole, logits everywhere."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def trace_tail_one_by_one(requests: dict, tail=32):
    """Most of a request in one step, its last `tail` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = len(toks) - tail
        assert head >= 1
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(toks[:head]), "want": list(range(head))}],
                      "end": []})
        for i in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
    return steps


PORTIONS = [7, 2, 13, 3, 2, 31, 5, 2, 17, 4, 64, 2, 9]


def trace_portions(requests: dict, sizes=PORTIONS):
    """Portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in requests.items():
        pos, k = 0, 0
        while pos < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - pos)
            if len(toks) - pos - n == 1:         # never leave a single token: keep portions >= 2
                n += 1
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(toks[pos:pos + n]), "want": list(range(n))}],
                          "end": [rid] if pos + n == len(toks) else []})
            pos += n
    return steps


def trace_mixed(requests: dict, prefill_part=0.6, portion=11, max_live=4, seed=0):
    """Up to `max_live` live requests; each is fed its first part in portions
    (of changing size) and the rest token by token, so that steps hold portions
    of some requests beside single tokens of others; requests start as others
    end.  Now and then a live request sits a step out."""
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    live = {}                       # rid -> position
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = 0
            if rng.random() < 0.5:
                break               # stagger the starts
        entries, ended = [], []
        for rid in list(live):
            toks = requests[rid]
            pos = live[rid]
            if len(live) > 1 and rng.random() < 0.15:
                continue            # left out of this step, goes on later
            if pos < int(len(toks) * prefill_part):
                n = int(min(max(2, portion + rng.integers(-6, 7)), len(toks) - pos))
                if len(toks) - pos - n == 1:
                    n += 1
            else:
                n = 1
            entries.append({"id": rid, "tokens": list(toks[pos:pos + n]), "want": list(range(n))})
            live[rid] = pos + n
            if live[rid] == len(toks):
                ended.append(rid)
                del live[rid]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def max_live_tokens(steps, round_to=64):
    """The --max-tokens a trace needs: the most tokens live requests hold at any
    time, each request rounded up to a multiple of `round_to`."""
    held, worst = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return worst


# ---------------------------------------------------------------------------
# running a trace
# ---------------------------------------------------------------------------

def rows_of(steps):
    """(request, position) of every wanted row, per step."""
    pos = {}
    out = {}
    for s in steps:
        rows = []
        for e in s["entries"]:
            start = pos.get(e["id"], 0)
            rows += [(e["id"], start + w) for w in e["want"]]
            pos[e["id"]] = start + len(e["tokens"])
        for rid in s["end"]:
            pos.pop(rid, None)
        out[s["step"]] = rows
    return out


def run_in_process(runner, steps):
    """-> {(request, position): logits row (numpy float32)}"""
    from easy_gpt.cpp_b200.engine import StepEntry

    rows = rows_of(steps)
    got = {}
    for s in steps:
        logits = runner.run([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]])
        if logits is not None:
            arr = logits.float().cpu().numpy()
            assert arr.shape[0] == len(rows[s["step"]])
            for key, row in zip(rows[s["step"]], arr):
                got[key] = row
        for rid in s["end"]:
            runner.end(rid)
        runner.cache.check()
    return got


def run_program(model_dir, dtype, steps, out_dir, max_tokens=None, extra_args=(), env=None):
    """Runs bin/trace_run as a child process, one step at a time (the next step is
    sent only after `done <step>` came back)."""
    max_tokens = max_tokens or max_live_tokens(steps)
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens), *extra_args]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {s['step']}", f"expected 'done {s['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    rows = rows_of(steps)
    got = {}
    for s in steps:
        if not rows[s["step"]]:
            continue
        arr = np.fromfile(Path(out_dir) / f"{s['step']}.f32", dtype="<f4")
        arr = arr.reshape(len(rows[s["step"]]), -1)
        for key, row in zip(rows[s["step"]], arr):
            got[key] = row
    return got


def compare(got, reference, atol, what=""):
    """reference: {request: [S, V] array}.  Returns the largest error; on failure
    names the first wrong row (lowest position of the first failing request)."""
    worst, first_bad = 0.0, None
    for (rid, pos), row in sorted(got.items(), key=lambda kv: (str(kv[0][0]), kv[0][1])):
        ref = reference[rid][pos]
        err = float(np.abs(row - ref).max())
        worst = max(worst, err)
        if err > atol and first_bad is None:
            first_bad = (rid, pos, err)
    assert first_bad is None, f"{what}: first wrong row: request {first_bad[0]!r} position {first_bad[1]} " \
                              f"(error {first_bad[2]:.3e} > {atol:.1e}); worst {worst:.3e}"
    return worst
