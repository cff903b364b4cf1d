"""Python face of the native engine (``csrc/engine``: configuration, weights, parts, step function, scheduler and
sampling in C++ over the kernel library, cuBLAS and the CUDA runtime; no PyTorch on its path).

``NativeEngine`` is ``GptEngine`` of ``csrc/engine/engine.hpp`` behind its C interface: token ids in, token ids out.
``NativeStepRunner`` is the bare step function for trace replay and tests: any mix of prompt portions and single
tokens in, float32 logits at the wanted places out.  The same library is what the ``easy_llm`` program of
``csrc/engine/main.cpp`` is made of.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int, c_longlong, c_void_p
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np

from .csrc.build import engine_paths
from .sampling.params import SamplingParams


class NativeError(RuntimeError):
    pass


_lib = None
_I64 = POINTER(c_longlong)


def library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path, _ = engine_paths()
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise NativeError(f"cannot load the native engine {path}: {e}") from None
        sig = {
            "ege_engine_create": (c_void_p, [c_char_p, c_char_p, c_void_p, c_char_p, c_int]),
            "ege_engine_destroy": (None, [c_void_p]),
            "ege_engine_add_request": (c_longlong, [c_void_p, c_void_p, c_longlong, c_float, c_float, c_int, c_longlong, c_int, c_longlong, c_char_p, c_int]),
            "ege_engine_step": (c_longlong, [c_void_p, c_void_p, c_int, c_char_p, c_int]),
            "ege_engine_has_work": (c_int, [c_void_p]),
            "ege_engine_run_to_completion": (c_longlong, [c_void_p, c_char_p, c_int]),
            "ege_engine_output": (c_longlong, [c_void_p, c_longlong, c_void_p, c_longlong]),
            "ege_engine_request": (c_int, [c_void_p, c_longlong, c_void_p, c_char_p, c_int]),
            "ege_engine_forget": (None, [c_void_p, c_longlong]),
            "ege_engine_stats": (None, [c_void_p, c_void_p]),
            "ege_engine_figure": (c_longlong, [c_void_p, c_int, c_longlong]),
            "ege_engine_sync": (None, [c_void_p]),
            "ege_engine_fused_trace": (c_longlong, [c_void_p, c_void_p, c_longlong]),
            "ege_engine_time_steps": (c_longlong, [c_void_p, c_int, c_void_p, c_char_p, c_int]),
            "ege_load_plugin": (c_longlong, [c_char_p, c_char_p, c_int]),
            "ege_runner_create": (c_void_p, [c_char_p, c_char_p, c_int, c_int, c_int, c_longlong, c_int, c_char_p, c_int]),
            "ege_runner_destroy": (None, [c_void_p]),
            "ege_runner_step": (c_longlong, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_char_p, c_int]),
            "ege_runner_end": (None, [c_void_p, c_longlong]),
            "ege_runner_info": (c_longlong, [c_void_p, c_int, c_int]),
            "ege_plan": (None, [c_int, c_void_p, c_void_p]),
        }
        for name, (restype, argtypes) in sig.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
        _lib = lib
    return _lib


_ERR = 2048


def plan(what: int, *numbers: int):
    """A launch plan as the native engine computes it (``ege_plan`` in ``csrc/engine/engine_api.cpp`` lists what
    ``what`` may be): four numbers, of which the plan uses the first ones."""
    args = (ctypes.c_longlong * 8)(*numbers)
    out = (ctypes.c_longlong * 4)()
    library().ege_plan(int(what), args, out)
    return tuple(int(v) for v in out)


def load_plugin(path) -> None:
    """Loads a shared library that registers further parts and architectures with the native engine (built with
    ``csrc.build.build_plugin`` from a source that includes ``csrc/engine/plugin.hpp``)."""
    err = ctypes.create_string_buffer(_ERR)
    if library().ege_load_plugin(str(path).encode(), err, _ERR) < 0:
        raise NativeError(err.value.decode(errors="replace"))


_STATES = ("waiting", "running", "finished")
_REASONS = (None, "empty", "eos", "length", "max_positions", "error")


class NativeEngine:
    def __init__(self, model_dir, dtype: str = "bfloat16", page_size: int = 16, cache_tokens: Optional[int] = None,
                 max_active: int = 16, prefill_batch: int = 4, max_batch_tokens: int = 2048, chunk_size: int = 512,
                 max_tokens_per_request: Optional[int] = None, use_graphs: bool = True):
        self._lib = library()
        self._err = ctypes.create_string_buffer(_ERR)
        options = np.asarray([page_size, cache_tokens or 0, max_active, prefill_batch, max_batch_tokens, chunk_size,
                              max_tokens_per_request or 0, int(use_graphs)], dtype=np.int64)
        self._h = self._lib.ege_engine_create(str(model_dir).encode(), str(dtype).encode(), options.ctypes.data, self._err, _ERR)
        if not self._h:
            raise NativeError(self._err.value.decode(errors="replace"))
        self.max_active = max_active
        self._finished = np.zeros(max_active + 1, dtype=np.int64)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.ege_engine_destroy(h)

    def _fail(self):
        raise NativeError(self._err.value.decode(errors="replace"))

    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None, max_new_tokens: Optional[int] = None,
                    max_steps: Optional[int] = None) -> int:
        params = params or SamplingParams()
        if max_new_tokens is None:
            max_new_tokens = max(1, (max_steps if max_steps is not None else 100) - len(prompt) + 1)
        arr = np.asarray(list(prompt), dtype=np.int64)
        rid = self._lib.ege_engine_add_request(self._h, arr.ctypes.data, len(arr), params.temperature, params.top_p, params.top_k, params.seed,
                                               int(params.greedy), int(max_new_tokens), self._err, _ERR)
        if rid < 0:
            msg = self._err.value.decode(errors="replace")
            raise ValueError(msg) if "vocabulary" in msg or "must be" in msg else NativeError(msg)
        return int(rid)

    def step(self) -> List[int]:
        """One scheduler round and one model step; the ids of the requests that finished."""
        n = self._lib.ege_engine_step(self._h, self._finished.ctypes.data, len(self._finished), self._err, _ERR)
        if n < 0:
            self._fail()
        return self._finished[:n].tolist()

    def has_work(self) -> bool:
        return bool(self._lib.ege_engine_has_work(self._h))

    def run_to_completion(self) -> None:
        if self._lib.ege_engine_run_to_completion(self._h, self._err, _ERR) < 0:
            self._fail()

    def output(self, rid: int) -> List[int]:
        n = self._lib.ege_engine_output(self._h, rid, None, 0)
        if n < 0:
            raise KeyError(rid)
        buf = np.zeros(max(n, 1), dtype=np.int64)
        self._lib.ege_engine_output(self._h, rid, buf.ctypes.data, n)
        return buf[:n].tolist()

    def request(self, rid: int) -> Dict[str, object]:
        out = np.zeros(10, dtype=np.int64)
        text = ctypes.create_string_buffer(512)
        if self._lib.ege_engine_request(self._h, rid, out.ctypes.data, text, 512) != 0:
            raise KeyError(rid)
        v = out.tolist()
        return dict(prompt_len=v[0], output_len=v[1], max_new_tokens=v[2], computed=v[3], state=_STATES[v[4]], finish_reason=_REASONS[v[5]],
                    error=text.value.decode() or None, pending=v[7], preemptions=v[8])

    def forget(self, rid: int) -> None:
        self._lib.ege_engine_forget(self._h, rid)

    def stats(self) -> Dict[str, int]:
        out = np.zeros(12, dtype=np.int64)
        self._lib.ege_engine_stats(self._h, out.ctypes.data)
        names = ("steps", "prompt_tokens", "decode_tokens", "preemptions", "finished", "failed", "graph_replays", "steps_run", "live_requests",
                 "free_pages", "vocab_size", "weight_bytes_per_step")
        return dict(zip(names, out.tolist()))

    def kv_bytes_per_token(self) -> int:
        return int(self._lib.ege_engine_figure(self._h, 0, 0))

    def last_step_h2d_bytes(self) -> int:
        return int(self._lib.ege_engine_figure(self._h, 1, 0))

    def last_step_launches(self) -> int:
        """Kernels that one replay of the last captured step launches."""
        return int(self._lib.ege_engine_figure(self._h, 3, 0))

    def cached_length(self, rid: int) -> int:
        return int(self._lib.ege_engine_figure(self._h, 2, rid))

    def fused_trace(self):
        """Rows (entered, input ready, products done, left, kind) of GPU nanosecond stamps, one per operation of the
        fused decode kernel's last run; empty unless EASY_GPT_FUSED_TRACE=1 was set when the engine was made."""
        import numpy as np

        out = np.zeros((4096, 5), dtype=np.uint64)
        n = int(self._lib.ege_engine_fused_trace(self._h, out.ctypes.data_as(ctypes.c_void_p), 4096))
        return out[:n]

    def fused_steps(self) -> int:
        """Steps so far that ran as one persistent kernel (csrc/decode_fused.cu)."""
        return int(self._lib.ege_engine_figure(self._h, 4, 0))

    def sync(self) -> None:
        self._lib.ege_engine_sync(self._h)

    def time_steps(self, steps: int):
        """Runs ``steps`` steps and returns (seconds on the device by CUDA events on the engine's stream around them,
        wall-clock seconds until the last step's tokens are on the host)."""
        out = np.zeros(2, dtype=np.float64)
        if self._lib.ege_engine_time_steps(self._h, int(steps), out.ctypes.data, self._err, _ERR) < 0:
            self._fail()
        return float(out[0]) / 1e3, float(out[1]) / 1e3

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: Optional[int] = None, max_steps: Optional[int] = None,
                 temperature: float = 0.8, top_p: float = 0.95, top_k: int = 20, seed: int = 42, greedy: bool = False) -> List[List[int]]:
        """Generates for every prompt (lists of token ids) and returns the new tokens of each."""
        params = SamplingParams(temperature=temperature, top_p=top_p, top_k=top_k, seed=seed, greedy=greedy)
        ids = [self.add_request(p, params, max_new_tokens, max_steps) for p in prompts]
        self.run_to_completion()
        outputs, errors = [], []
        for rid in ids:
            outputs.append(self.output(rid))
            info = self.request(rid)
            if info["error"]:
                errors.append((rid, info["error"]))
            self.forget(rid)
        if errors:
            raise RuntimeError(f"request {errors[0][0]}: {errors[0][1]}")
        return outputs


class NativeStepRunner:
    """The step function alone: ``run`` takes entries (request, tokens, want) and returns float32 logits [wanted, vocab]
    as a numpy array (None if nothing is wanted)."""

    def __init__(self, model_dir, dtype: str, page_size: int, num_pages: int, max_slots: int, max_tokens_per_request: Optional[int] = None,
                 use_graphs: bool = True):
        self._lib = library()
        self._err = ctypes.create_string_buffer(_ERR)
        self._h = self._lib.ege_runner_create(str(model_dir).encode(), str(dtype).encode(), page_size, num_pages, max_slots,
                                              max_tokens_per_request or 0, int(use_graphs), self._err, _ERR)
        if not self._h:
            raise NativeError(self._err.value.decode(errors="replace"))
        self.vocab = int(self._lib.ege_runner_info(self._h, 0, 0))
        self._device_ms = np.zeros(1, dtype=np.float64)
        self._handles: Dict[Hashable, int] = {}
        self._next = 1 << 40

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.ege_runner_destroy(h)

    def _handle(self, rid) -> int:
        if isinstance(rid, (int, np.integer)) and not isinstance(rid, bool) and 0 <= int(rid) < (1 << 40):
            return int(rid)
        if rid not in self._handles:
            self._handles[rid] = self._next
            self._next += 1
        return self._handles[rid]

    def run(self, entries) -> Optional[np.ndarray]:
        """entries: (request, tokens, want) triples or objects with those attributes."""
        triples = [(e.request, e.tokens, e.want) if hasattr(e, "request") else e for e in entries]
        n = len(triples)
        rids = np.asarray([self._handle(r) for r, _, _ in triples], dtype=np.int64)
        counts = np.asarray([len(t) for _, t, _ in triples], dtype=np.int64)
        tokens = np.asarray([x for _, t, _ in triples for x in t], dtype=np.int64)
        want_offsets = np.zeros(n + 1, dtype=np.int64)
        want_offsets[1:] = np.cumsum([len(w) for _, _, w in triples])
        wants = np.asarray([x for _, _, w in triples for x in w] or [0], dtype=np.int64)
        rows = int(want_offsets[n])
        logits = np.empty((max(rows, 1), self.vocab), dtype=np.float32)
        got = self._lib.ege_runner_step(self._h, n, rids.ctypes.data, counts.ctypes.data, tokens.ctypes.data, want_offsets.ctypes.data,
                                        wants.ctypes.data, logits.ctypes.data, logits.size, self._device_ms.ctypes.data, self._err, _ERR)
        if got < 0:
            raise NativeError(self._err.value.decode(errors="replace"))
        return logits[:rows] if rows else None

    @property
    def last_step_device_seconds(self) -> float:
        """The last step's time on the device (CUDA events on the runner's stream around its launches)."""
        return float(self._device_ms[0]) / 1e3

    def end(self, rid) -> None:
        self._lib.ege_runner_end(self._h, self._handle(rid))
        self._handles.pop(rid, None)

    def info(self, what: str, group: int = 0) -> int:
        index = {"vocab": 0, "live_requests": 1, "graph_replays": 2, "free_pages": 3, "pages": 4, "pages_handed_out": 5, "groups": 6,
                 "books_in_order": 7, "captured_shapes": 8, "fused_steps": 9}[what]
        return int(self._lib.ege_runner_info(self._h, index, group))
