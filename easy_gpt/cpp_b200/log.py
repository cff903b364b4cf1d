"""A levelled logger to stderr and optional NVTX ranges.

``EASYGPT_LOG`` sets the level: ``error``, ``warn`` (the default), ``info``, ``debug`` or ``trace``
(the reference forces its spdlog level to debug in main, src/main.cpp:25, logs a completion line per
request at info, src/continuous_batch_server.cpp:249-256, and the top-5 tokens of a step at trace,
src/models/gpt_model.cpp:76-110).  ``EASY_GPT_NVTX=1`` puts NVTX ranges around steps, forward passes
and parts, for a profiler's timeline; without it ``nvtx_range`` costs one comparison.
"""
from __future__ import annotations

import contextlib
import os
import sys
import time

LEVELS = {"error": 0, "warn": 1, "info": 2, "debug": 3, "trace": 4}


def _level_from_env() -> int:
    name = os.environ.get("EASYGPT_LOG", "warn").strip().lower()
    if name not in LEVELS:
        print(f"[easy_gpt] EASYGPT_LOG={name!r} is no level ({', '.join(LEVELS)}); using warn", file=sys.stderr)
        return LEVELS["warn"]
    return LEVELS[name]


level = _level_from_env()
NVTX = os.environ.get("EASY_GPT_NVTX", "0") not in ("", "0")
_start = time.time()


def set_level(name: str) -> None:
    global level
    level = LEVELS[name]


def enabled(name: str) -> bool:
    return level >= LEVELS[name]


def log(name: str, message: str) -> None:
    if level >= LEVELS[name]:
        print(f"[easy_gpt {time.time() - _start:9.3f}s] [{name}] {message}", file=sys.stderr, flush=True)


def error(message: str) -> None:
    log("error", message)


def warn(message: str) -> None:
    log("warn", message)


def info(message: str) -> None:
    log("info", message)


def debug(message: str) -> None:
    log("debug", message)


def trace(message: str) -> None:
    log("trace", message)


@contextlib.contextmanager
def _nvtx(name: str):
    import torch

    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


_NO_RANGE = contextlib.nullcontext()


def nvtx_range(name: str):
    """``with nvtx_range("step"):`` — an NVTX range when EASY_GPT_NVTX is set, nothing otherwise."""
    return _nvtx(name) if NVTX else _NO_RANGE
