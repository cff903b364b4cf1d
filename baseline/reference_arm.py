"""The reference arm of ``bench.py``: the unmodified reference program, built out
of tree and run through its own command line, timed from its own log.

What runs is the reference's stock one-shot path (``easy_llm -f prompts.txt
--greedy -m <total length>``, src/main.cpp:24-125 -> ``GptEngine::run``,
src/gpt_engine.cpp:33-43 -> ``GptModel::forward``, src/models/gpt_model.cpp:155-190)
built with its CUDA backend switched on.  None of this repository's kernels,
engine or model code is on that path; this module only writes the input files
the program reads from ``data/model/`` (config.json, model.safetensors with
random weights, a tokenizer whose one word maps to one token id) and parses the
program's log.

How the numbers are taken.  The program logs ``----------Step N : ...`` at the
start of every decode step (src/models/gpt_model.cpp:269) with a millisecond
time stamp, and ``Decode finished: steps=…, avg_ms_per_step=…`` at the end
(:283-288).  ``value`` is batch x K divided by the time between the stamp of
step (context - K) and the stamp of the finish line: the same K steps, ending
at the same context length, that the other arm times.  The loop inside takes
token ids from the host and hands sampled ids back to the host on every step,
so the same figure is the end-to-end one.

What the program cannot hold.  Its prefill computes logits at every position
as one host tensor indexed by ``int`` (include/tensor.hpp:23-40,
src/ops.cpp:460-488): batch x prompt length x vocabulary must stay below 2^31,
which at a vocabulary of 151,936 and batch 8 allows prompts of at most 1,766
tokens.  So the prompts here are shorter than the other arm's and the program
decodes its way up to the context length (more decode steps, the same last K).
"""
from __future__ import annotations

import json
import os
import re
import shutil
import subprocess
import sys
import tempfile
import time
from datetime import datetime
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
SOURCE_COPY = REF_DIR / "src_copy"
BUILD_DIR = REF_DIR / "build"
WORD = "z"                      # a letter the chat template does not contain (src/cli_options.cpp:49-55)
WORD_ID = 7
STEP_RE = re.compile(r"^\[(\d{4}-\d\d-\d\d \d\d:\d\d:\d\d\.\d{3})\] \[info\] -+Step (\d+) : remaining batch size (\d+)-+")
DONE_RE = re.compile(r"^\[(\d{4}-\d\d-\d\d \d\d:\d\d:\d\d\.\d{3})\] \[info\] Decode finished: steps=(\d+), avg_ms_per_step=([0-9.]+), total_ms=([0-9.]+)")


class Unavailable(RuntimeError):
    pass


def _stamp(text: str) -> float:
    return datetime.strptime(text, "%Y-%m-%d %H:%M:%S.%f").timestamp()


def reference_source() -> Path:
    """The reference's tree: the copy kept beside the build (it travels with the repository's
    working folder), made from the mounted checkout when that is there."""
    if (SOURCE_COPY / "CMakeLists.txt").is_file():
        return SOURCE_COPY
    mounted = Path(os.environ.get("EASY_GPT_REFERENCE_SRC", "/root/reference"))
    if not (mounted / "CMakeLists.txt").is_file():
        raise Unavailable(f"no reference checkout at {mounted} and no copy under {SOURCE_COPY}")
    REF_DIR.mkdir(parents=True, exist_ok=True)
    shutil.copytree(mounted, SOURCE_COPY, ignore=shutil.ignore_patterns(".git", "build"))
    return SOURCE_COPY


def binary(log=sys.stderr) -> Path:
    """Path of the reference's ``easy_llm`` with the CUDA backend, building it if need be.
    RelWithDebInfo is the configuration of the reference's own build.sh:10 (Release would add
    -march=native and tie the binary to the machine that built it); the architecture is 100
    where build.sh names 120 (CMakeLists.txt:9-15 takes it from the command line)."""
    exe = BUILD_DIR / "easy_llm"
    if exe.is_file():
        try:
            if subprocess.run([str(exe), "--help"], capture_output=True, timeout=60).returncode == 0:
                return exe
        except (OSError, subprocess.TimeoutExpired):
            pass
    src = reference_source()
    cmake = shutil.which("cmake")
    if cmake is None:
        raise Unavailable("cmake is not installed, the reference cannot be built")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    print("[reference] building the reference with its CUDA backend (about half a minute)", file=log, flush=True)
    if BUILD_DIR.exists():
        shutil.rmtree(BUILD_DIR)
    BUILD_DIR.mkdir(parents=True)
    with open(REF_DIR / "build.log", "w") as out:
        for cmd in ([cmake, "-S", str(src), "-B", str(BUILD_DIR), "-DCMAKE_BUILD_TYPE=RelWithDebInfo", "-DEASY_LLM_ENABLE_CUDA=ON",
                     "-DCMAKE_CUDA_ARCHITECTURES=100", f"-DCMAKE_CUDA_COMPILER={nvcc}"],
                    [cmake, "--build", str(BUILD_DIR), "--target", "easy_llm", "-j", str(min(16, os.cpu_count() or 4))]):
            rc = subprocess.run(cmd, stdout=out, stderr=subprocess.STDOUT).returncode
            if rc != 0:
                raise Unavailable(f"building the reference failed ({' '.join(cmd[:3])} ... exit {rc}, see baseline/_ref/build.log)")
    if not exe.is_file():
        raise Unavailable("the reference's build produced no easy_llm")
    return exe


def write_inputs(folder: Path, model_folder: Path, config: dict, batch: int, prompt_tokens: int) -> Path:
    """``folder/data/model`` as the program expects it (include/config.hpp:32-35) and a prompt file.
    The tokenizer has one merge, so that every word ``z`` of a prompt becomes the one token ``Ġz``;
    every other piece of the chat template is not in the vocabulary and is dropped
    (src/tokenizer.cpp:135-142): a prompt of n words is n tokens."""
    model = folder / "data" / "model"
    model.mkdir(parents=True)
    os.symlink(model_folder / "model.safetensors", model / "model.safetensors")
    (model / "config.json").write_text(json.dumps(config))
    vocab = {f"t{i}": i for i in range(config["vocab_size"])}       # every id has a name (src/data_manager.cpp:106-108)
    del vocab[f"t{WORD_ID}"]
    vocab["\u0120" + WORD] = WORD_ID
    (model / "tokenizer.json").write_text(json.dumps({"model": {"vocab": vocab, "merges": ["\u0120 " + WORD]}}))
    (model / "tokenizer_config.json").write_text(json.dumps({"added_tokens_decoder": {}, "pad_token": "t0"}))
    prompts = folder / "prompts.txt"
    prompts.write_text("\n".join(" ".join([WORD] * prompt_tokens) for _ in range(batch)) + "\n")
    return prompts


def longest_prompt(batch: int, vocab: int) -> int:
    """The longest prompt whose [batch, prompt, vocabulary] logits the program can index with an int."""
    return (2 ** 31 - 1) // (batch * vocab)


def run(model_folder: Path, config: dict, batch: int, context: int, steps: int, prompt_tokens: int = 0,
        timeout_s: float = 1500.0, log=sys.stderr, allow_cpu: bool = False) -> dict:
    """Runs the reference until the requests hold ``context`` tokens and returns the timing of its last
    ``steps`` decode steps: {tok_s, ms_per_step, avg_ms_per_step_whole_run, decode_steps, prompt_tokens, wall_s}."""
    exe = binary(log)
    limit = longest_prompt(batch, config["vocab_size"])
    if not prompt_tokens:
        prompt_tokens = min(1536, limit)
    if prompt_tokens > limit:
        raise Unavailable(f"batch {batch} x prompt {prompt_tokens} x vocabulary {config['vocab_size']} overflows the int index of "
                          "the reference's logits tensor (include/tensor.hpp:36-40)")
    if context - prompt_tokens < steps:
        raise Unavailable("the context leaves fewer decode steps than are to be timed")
    work = Path(tempfile.mkdtemp(prefix="easy_gpt_reference_"))
    try:
        prompts = write_inputs(work, model_folder, config, batch, prompt_tokens)
        out_path = work / "run.log"
        print(f"[reference] batch {batch}, prompts of {prompt_tokens} tokens, decoding to context {context} "
              f"({context - prompt_tokens} steps)", file=log, flush=True)
        t0 = time.time()
        with open(out_path, "w") as out:
            proc = subprocess.Popen([str(exe), "-f", str(prompts), "--greedy", "-m", str(context)], cwd=work,
                                    stdout=out, stderr=subprocess.STDOUT)
            try:
                while True:
                    try:
                        rc = proc.wait(timeout=30)
                        break
                    except subprocess.TimeoutExpired:
                        if time.time() - t0 > timeout_s:
                            proc.kill()
                            proc.wait()
                            raise Unavailable(f"the reference did not finish within {timeout_s:.0f} s") from None
                        print(f"[reference] running, {time.time() - t0:.0f} s", file=log, flush=True)
            finally:
                if proc.poll() is None:
                    proc.kill()
        wall = time.time() - t0
        keep = os.environ.get("EASY_GPT_REFERENCE_LOG")
        if keep:                                     # a short copy of the program's log, for the record
            with open(out_path, errors="replace") as f:
                lines = [l[:300].rstrip("\n") for l in f]
            Path(keep).write_text("\n".join(lines[:150] + ["..."] + lines[-60:]) + "\n")
        stamps, done = {}, None
        cuda_seen = False
        tail = []
        with open(out_path, errors="replace") as f:
            for line in f:
                m = STEP_RE.match(line)
                if m:
                    stamps[int(m.group(2))] = (_stamp(m.group(1)), int(m.group(3)))
                    continue
                m = DONE_RE.match(line)
                if m:
                    done = (_stamp(m.group(1)), int(m.group(2)), float(m.group(3)), float(m.group(4)))
                if "CUDA unavailable" in line and not allow_cpu:
                    raise Unavailable("the reference found no CUDA device: " + line.strip()[-160:])
                if "cuda" in line.lower():
                    cuda_seen = True
                tail = (tail + [line.rstrip()])[-5:]
        if rc != 0 or done is None:
            raise Unavailable(f"the reference exited with {rc}; its log ends: " + " | ".join(t[-200:] for t in tail))
        first = context - steps
        if first not in stamps or stamps[first][1] != batch:
            raise Unavailable(f"the reference's log has no step {first} at batch {batch}")
        seconds = done[0] - stamps[first][0]
        return {"tok_s": batch * steps / seconds, "ms_per_step": 1e3 * seconds / steps,
                "avg_ms_per_step_whole_run": done[2], "decode_steps": done[1], "prompt_tokens": prompt_tokens,
                "wall_s": wall, "cuda_lines_in_log": cuda_seen}
    finally:
        shutil.rmtree(work, ignore_errors=True)
