"""Python face of the hand-written CUDA kernels (``csrc/*.cu``).

The kernels are plain ``extern "C"`` launchers in one shared library built by
``csrc/build.py``; they are called through ctypes with raw device pointers and
the current torch stream, so they are captured by CUDA graphs like any other
launch.  There is no other implementation behind these functions: if the
library cannot be built or loaded, importing it raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .csrc.build import library_path

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

STATUS_BITS = {1: "a token id lies outside the vocabulary",
               2: "a block table entry needed by attention is not a valid page",
               4: "a cache write position lies outside the pool",
               8: "a bounded wait inside a kernel gave up"}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


_lib = None
launch_count = 0     # number of kernel launches issued through this module (for the bench's gpu_launches)


def library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = library_path()
        try:
            _lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelError(f"cannot load the CUDA kernel library {path}: {e}") from None
        for name in dir(_Signatures):
            if name.startswith("eg_"):
                fn = getattr(_lib, name)
                fn.argtypes = getattr(_Signatures, name)
                fn.restype = c_int
    return _lib


class _Signatures:
    eg_embedding_gather = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    eg_add_rmsnorm = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float]
    eg_gemm_f32_nt = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int]
    eg_rope_cache = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                     c_int, c_int, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p]
    eg_rope_table = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int]
    eg_rope_cache_vec = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                         c_longlong, c_longlong, c_longlong, c_void_p]
    eg_attention_generic = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                            c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int, c_int,
                            c_float, c_void_p]
    eg_attention_paged = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                          c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int, c_int, c_float,
                          c_int, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p]
    eg_attention_prefill = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p,
                            c_int, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int, c_int, c_float, c_void_p]
    eg_attention_prefill_tcgen05 = [c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                    c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int, c_int,
                                    c_float, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p]
    eg_attention_prefill_groups = [c_int]
    eg_gemm_skinny = [c_void_p, c_int, c_int, c_int, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p, c_longlong,
                      c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p,
                      c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_longlong,
                      c_longlong, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                      c_void_p, c_void_p]
    eg_gemm_tcgen05 = [c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int, c_int,
                       c_int, c_void_p]
    eg_gemm_tcgen05_pair = [c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int, c_int,
                            c_int, c_int, c_void_p, c_void_p]
    eg_gemm_tcgen05_few = [c_void_p, c_int, c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong,
                           c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]
    eg_swiglu = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int]
    eg_argmax = [c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p]
    eg_wait_probe = [c_void_p, ctypes.c_uint, c_int, c_void_p, c_void_p]
    eg_sample = [c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]


class Timeline:
    """Optional device-side timeline of the decode kernels: every launch while ``active`` gets a
    slot where its CTAs record their earliest start and latest end (GPU nanosecond clock).  Inside
    a CUDA graph the slots are rewritten by every replay.  For profiling; costs nothing when off."""
    active = False
    buffer: Optional[torch.Tensor] = None
    names: list = []

    @classmethod
    def start(cls, device="cuda", capacity=4096):
        cls.buffer = torch.zeros((capacity, 16), dtype=torch.int64, device=device)
        cls.names = []
        cls.active = True
        cls.reset()

    @classmethod
    def reset(cls):
        cls.buffer[:, 0] = (1 << 62)
        cls.buffer[:, 1:] = 0

    @classmethod
    def slot(cls, name: str):
        if not cls.active or len(cls.names) >= cls.buffer.shape[0]:
            return None
        cls.names.append(name)
        return cls.buffer.data_ptr() + 128 * (len(cls.names) - 1)

    @classmethod
    def read(cls):
        rows = cls.buffer[:len(cls.names)].cpu().tolist()
        return [(n, r[0], r[1], r[2:]) for n, r in zip(cls.names, rows)]


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream of the current device as a raw handle (the short way: building a Stream
    object costs about 15 microseconds, and every kernel call asks)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _check(code: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code}" + (" (a size this kernel does not take)" if code == 1 else ""))


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only; there is no CPU path")


def embedding_gather(ids: torch.Tensor, table: torch.Tensor, residual: torch.Tensor, status: torch.Tensor) -> None:
    """residual[t] = float32(table[ids[t]]); a bad id sets a status bit."""
    _cuda(ids, table, residual, status)
    _need(ids.dtype == torch.int32 and residual.dtype == torch.float32, "ids int32, residual float32")
    _need(table.is_contiguous() and residual.is_contiguous(), "contiguous table and residual")
    T, (V, H) = ids.numel(), table.shape
    _need(residual.shape[-1] == H and residual.numel() >= T * H, "residual too small")
    _check(library().eg_embedding_gather(_stream(), dtype_code(table.dtype), _ptr(ids), _ptr(table), _ptr(residual),
                                         T, H, V, _ptr(status)), "embedding_gather")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor, out: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """residual += delta (if given, and rows is None); out = rmsnorm(residual) * gain.
    With rows: out[r] is computed from row rows[r] and the residual is not written."""
    _cuda(residual, delta, gain, out, rows)
    H = residual.shape[-1]
    _need(residual.dtype == torch.float32 and gain.dtype == torch.float32, "residual and gain are float32")
    _need(residual.is_contiguous() and out.is_contiguous() and (delta is None or delta.is_contiguous()), "contiguous rows")
    _need(gain.numel() == H and out.shape[-1] == H and (delta is None or delta.shape[-1] == H), "width mismatch")
    n = rows.numel() if rows is not None else residual.numel() // H
    _need(out.numel() >= n * H, "out too small")
    if rows is not None:
        _need(rows.dtype == torch.int32, "rows int32")
    dd = dtype_code(delta.dtype) if delta is not None else dtype_code(out.dtype)
    _check(library().eg_add_rmsnorm(_stream(), dd, dtype_code(out.dtype), _ptr(residual), _ptr(delta), _ptr(rows),
                                    _ptr(gain), _ptr(out), n, H, float(eps)), "add_rmsnorm")


def gemm_f32_nt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T + bias, all float32, true 32-bit arithmetic."""
    _cuda(a, w, bias, out)
    _need(a.dtype == w.dtype == out.dtype == torch.float32, "float32 only")
    _need(a.dim() == 2 and w.dim() == 2 and out.dim() == 2, "matrices")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape[0] == M and out.shape[1] == N, "shape mismatch")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "unit inner strides")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == N, "bias float32 [N]")
    _check(library().eg_gemm_f32_nt(_stream(), _ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out),
                                    out.stride(0), M, N, K), "gemm_f32_nt")


def rope_cache(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
               slot_map: Optional[torch.Tensor], k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
               inv_freq: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int,
               page_size: int, status: torch.Tensor) -> None:
    """Rotates q and k of qkv [T, (NH+2NKV)*HD] (q in place) and stores k, v at
    slot_map[t] of caches shaped [pages, NKV, page_size, HD] (slices of one pool).
    rotary_dim 0: no rotation, only the store (inv_freq may be None)."""
    _cuda(qkv, bias, positions, slot_map, k_cache, v_cache, inv_freq, status)
    T = qkv.shape[0]
    _need(qkv.stride(1) == 1 and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim, "qkv row layout")
    _need(positions.dtype == torch.int32, "positions int32")
    if rotary_dim:
        _need(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == rotary_dim,
              "inv_freq: float32 with rotary_dim/2 entries")
    else:
        inv_freq = None                                  # nothing is rotated: q and k pass through, k and v are stored
    page_stride = head_stride = pool_slots = 0
    if slot_map is not None:
        _need(k_cache is not None and v_cache is not None and slot_map.dtype == torch.int32, "cache and int32 slot map")
        _need(k_cache.dtype == qkv.dtype == v_cache.dtype, "cache dtype equals activation dtype")
        _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim) and k_cache.shape == v_cache.shape,
              "cache shape [pages, NKV, page_size, HD]")
        _need(k_cache.stride(3) == 1 and k_cache.stride(2) == head_dim and k_cache.stride() == v_cache.stride(),
              "cache strides")
        page_stride, head_stride = k_cache.stride(0), k_cache.stride(1)
        pool_slots = k_cache.shape[0] * page_size
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == qkv.shape[1], "bias float32 over the whole row")
    _check(library().eg_rope_cache(_stream(), dtype_code(qkv.dtype), _ptr(qkv), qkv.stride(0), _ptr(bias), _ptr(positions),
                                   _ptr(slot_map), _ptr(k_cache), _ptr(v_cache), _ptr(inv_freq), T, num_heads,
                                   num_kv_heads, head_dim, rotary_dim, page_size, page_stride, head_stride, pool_slots,
                                   _ptr(status)), "rope_cache")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """float32 [T, rotary_dim/2, 2]: (cos, sin) of float32(position) * inv_freq, by the accurate cosf/sinf."""
    _cuda(positions, inv_freq)
    _need(positions.dtype == torch.int32 and inv_freq.dtype == torch.float32, "positions int32, inv_freq float32")
    T, half = positions.numel(), inv_freq.numel()
    table = torch.empty((T, half, 2), dtype=torch.float32, device=positions.device)
    _check(library().eg_rope_table(_stream(), _ptr(positions), _ptr(inv_freq), _ptr(table), T, half), "rope_table")
    return table


def rope_cache_table(qkv: torch.Tensor, table: torch.Tensor, slot_map: Optional[torch.Tensor],
                     k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int,
                     head_dim: int, page_size: int, status: torch.Tensor) -> None:
    """``rope_cache`` for the whole head rotated, with cos/sin from ``rope_table`` (shared by the
    layers of a step) and 16-byte accesses: half a head must be a multiple of 16 bytes (head_dim
    % 16 == 0 in bfloat16, % 8 in float32)."""
    _cuda(qkv, table, slot_map, k_cache, v_cache, status)
    T = qkv.shape[0]
    _need(qkv.stride(1) == 1 and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim and head_dim % (32 // qkv.element_size()) == 0, "qkv row layout")
    _need(table.dtype == torch.float32 and table.is_contiguous() and tuple(table.shape) == (T, head_dim // 2, 2), "table [T, HD/2, 2]")
    page_stride = head_stride = pool_slots = 0
    if slot_map is not None:
        _need(k_cache is not None and v_cache is not None and slot_map.dtype == torch.int32, "cache and int32 slot map")
        _need(k_cache.dtype == qkv.dtype == v_cache.dtype, "cache dtype equals activation dtype")
        _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim) and k_cache.shape == v_cache.shape
              and k_cache.stride(3) == 1 and k_cache.stride(2) == head_dim and k_cache.stride() == v_cache.stride(), "cache layout")
        page_stride, head_stride = k_cache.stride(0), k_cache.stride(1)
        pool_slots = k_cache.shape[0] * page_size
    _check(library().eg_rope_cache_vec(_stream(), dtype_code(qkv.dtype), _ptr(qkv), qkv.stride(0), _ptr(table), _ptr(slot_map),
                                       _ptr(k_cache), _ptr(v_cache), T, num_heads, num_kv_heads, head_dim, page_size,
                                       page_stride, head_stride, pool_slots, _ptr(status)), "rope_cache_table")


def attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                      token_seq: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, num_heads: int,
                      num_kv_heads: int, head_dim: int, window: Optional[int], scale: float,
                      status: torch.Tensor) -> None:
    """q: [T, >=NH*HD] rows (a view into the qkv buffer is fine); out [T, NH*HD]."""
    _cuda(q, k_cache, v_cache, block_table, token_seq, positions, out, status)
    T = q.shape[0]
    _need(head_dim <= 256, f"attention_generic takes head sizes up to 256, not {head_dim}")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_cache.dtype, "q/out/cache layout")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.stride(1) == 1, "block table")
    _need(token_seq.dtype == torch.int32 and positions.dtype == torch.int32, "int32 metadata")
    page_size = k_cache.shape[2]
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim) and k_cache.stride() == v_cache.stride()
          and k_cache.stride(3) == 1 and k_cache.stride(2) == head_dim, "cache shape [pages, NKV, page_size, HD]")
    _check(library().eg_attention_generic(
        _stream(), dtype_code(q.dtype), _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
        block_table.stride(0), _ptr(token_seq), _ptr(positions), _ptr(out), out.stride(0), T, num_heads, num_kv_heads,
        head_dim, page_size, k_cache.stride(0), k_cache.stride(1), k_cache.shape[0], int(window or 0), float(scale),
        _ptr(status)), "attention_generic")


PAGED_ATTENTION_HEAD_DIMS = (32, 64, 128, 256)
_sm_count = None


def sm_count() -> int:
    """Streaming multiprocessors of the current device (launch plans hang off it).  EASY_GPT_SM_COUNT
    sets it by hand; without a device (plans are also computed on machines that have none) it is the
    B200's 148."""
    global _sm_count
    if _sm_count is None:
        forced = os.environ.get("EASY_GPT_SM_COUNT")
        if forced:
            _sm_count = int(forced)
        elif torch.cuda.is_available():
            _sm_count = int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
        else:
            _sm_count = 148
    return _sm_count


def attention_paged_takes(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    """Sizes the tensor-core kernel takes; the rest goes to ``attention_generic``."""
    return dtype == torch.bfloat16 and head_dim in PAGED_ATTENTION_HEAD_DIMS and page_size % 16 == 0


def attention_paged_splits(tokens: int, num_heads: int, num_kv_heads: int, max_context: int, head_dim: int = 64) -> int:
    """How many CTAs share one (token, KV head).  Measured on B200 (context 4096): up to 16 tokens the kernel
    is fastest with one wave of 128 to 256 CTAs (two per SM, five key tiles of 64 in flight each) that walk
    about eight tiles; more, smaller CTAs pay in partial results and in the merge.  With more tokens it is
    fastest with about 400 to 600 CTAs, four per SM with three tiles in flight each (the kernel picks that
    pipeline when there are more CTAs than two per SM); heads of more than 64 leave room for two CTAs per SM
    only, and are fastest with up to that many.  A power of two, at least four tiles per CTA."""
    forced = os.environ.get("EASY_GPT_ATTENTION_SPLITS")
    base = tokens * num_kv_heads * (-(-(num_heads // num_kv_heads) // 16))
    tiles = max(1, -(-max_context // 64))
    if forced:
        return max(1, min(int(forced), tiles, 128))
    most = 256 if tokens <= SKINNY_MAX_TOKENS else (2 if head_dim > 64 else 4) * sm_count()
    splits = 1
    while splits * 2 * base <= most and tiles // (splits * 2) >= 4 and splits < 128:
        splits *= 2
    return splits


_attention_tickets = {}


def _attention_counters(device, n: int) -> torch.Tensor:
    """Zeroed ticket counters for the split merge (the kernel leaves them zero)."""
    key = str(device)
    have = _attention_tickets.get(key)
    if have is None or have.numel() < n:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("attention counters must exist before a CUDA graph is captured (run the step once eagerly first)")
        have = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
        _attention_tickets[key] = have
    return have


def attention_paged(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                    token_seq: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, num_heads: int,
                    num_kv_heads: int, head_dim: int, window: Optional[int], scale: float, splits: int,
                    status: torch.Tensor, prefetch: Optional[torch.Tensor] = None,
                    seq_context: Optional[torch.Tensor] = None, token_list: Optional[torch.Tensor] = None) -> None:
    """bfloat16 attention over the paged cache on the tensor cores; same contract as
    ``attention_generic``.  With splits > 1 it uses scratch memory for the partial results.
    ``seq_context`` (int32 per block-table row): keys cached before this step; given it, the kernel
    fetches those while the kernel in front of it (which writes the new keys) is still running.
    ``token_list`` (int32): only these tokens (the decoded tokens of a step that also holds prompt portions)."""
    _cuda(q, k_cache, v_cache, block_table, token_seq, positions, out, status, token_list)
    _need(token_list is None or (token_list.dtype == torch.int32 and token_list.dim() == 1 and token_list.is_contiguous()), "int32 token list")
    T = q.shape[0]
    page_size = k_cache.shape[2]
    _need(attention_paged_takes(q.dtype, head_dim, page_size),
          f"attention_paged takes bfloat16, head sizes {PAGED_ATTENTION_HEAD_DIMS} and pages of a multiple of 16 tokens")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and out.dtype == k_cache.dtype == torch.bfloat16, "q/out/cache layout")
    _need(q.data_ptr() % 4 == 0 and q.stride(0) % 2 == 0, "q rows must be 4-byte aligned")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.stride(1) == 1, "block table")
    _need(token_seq.dtype == torch.int32 and positions.dtype == torch.int32, "int32 metadata")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim) and k_cache.stride() == v_cache.stride()
          and k_cache.stride(3) == 1 and k_cache.stride(2) == head_dim and k_cache.data_ptr() % 16 == 0
          and k_cache.stride(0) % 8 == 0 and k_cache.stride(1) % 8 == 0, "cache shape [pages, NKV, page_size, HD], 16-byte rows")
    acc = ml = counters = None
    if splits > 1:
        acc = torch.empty(T * num_heads * splits * head_dim, dtype=torch.float32, device=q.device)
        ml = torch.empty(T * num_heads * splits * 2, dtype=torch.float32, device=q.device)
        counters = _attention_counters(q.device, T * num_kv_heads * (-(-(num_heads // num_kv_heads) // 16)))
    _check(library().eg_attention_paged(
        _stream(), _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.stride(0),
        _ptr(token_seq), _ptr(positions), _ptr(seq_context), _ptr(out), out.stride(0), _ptr(acc), _ptr(ml),
        T if token_list is None else token_list.numel(), num_heads, num_kv_heads,
        head_dim, page_size, k_cache.stride(0), k_cache.stride(1), k_cache.shape[0], int(window or 0), float(scale),
        int(splits), _ptr(status), _ptr(prefetch) if PREFETCH_WEIGHTS else None,
        prefetch.numel() * prefetch.element_size() if (prefetch is not None and PREFETCH_WEIGHTS) else 0,
        _ptr(counters), USE_PDL, Timeline.slot(f"attention s={splits}"), _ptr(token_list)), "attention_paged")


MAX_HEAD_DIM = 256             # the generic attention kernel keeps up to eight dimensions of a head per lane
PREFILL_ATTENTION_HEAD_DIMS = (32, 64, 128)
QUERY_TILE = 128               # tokens per listed tile of a prompt portion
SMALL_ENTRY_TOKENS = 4         # entries of up to this many tokens go through the decode attention kernel, token by token


def query_tiles_of(starts, counts):
    """(tiles, small_tokens) of a step: tiles [(entry, first token, count <= QUERY_TILE)] of the entries that
    bring more than SMALL_ENTRY_TOKENS tokens, and the token indices of all other entries."""
    tiles, small = [], []
    for i, c in enumerate(counts):
        c, s0 = int(c), int(starts[i])
        if c > SMALL_ENTRY_TOKENS:
            tiles += [(i, s0 + o, min(QUERY_TILE, c - o)) for o in range(0, c, QUERY_TILE)]
        else:
            small += list(range(s0, s0 + c))
    return tiles, small
TCGEN05_ATTENTION = os.environ.get("EASY_GPT_TCGEN05_ATTENTION", "1") != "0"
TCGEN05_ATTENTION_MIN_QUERY = 33   # shorter portions leave most of the 128-row tile empty: the warp-level kernel takes them


def attention_prefill_takes(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in PREFILL_ATTENTION_HEAD_DIMS and page_size % 16 == 0


def attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                      positions: torch.Tensor, tiles: torch.Tensor, out: torch.Tensor, num_heads: int,
                      num_kv_heads: int, head_dim: int, window: Optional[int], scale: float,
                      status: torch.Tensor) -> None:
    """bfloat16 attention for prompt portions: ``tiles`` [n, 3] int32 lists (block table row,
    first token, count <= 128) for runs of consecutive tokens of one request (warp-level kernel)."""
    _cuda(q, k_cache, v_cache, block_table, positions, tiles, out, status)
    page_size = k_cache.shape[2]
    _need(attention_prefill_takes(q.dtype, head_dim, page_size),
          f"attention_prefill takes bfloat16, head sizes {PREFILL_ATTENTION_HEAD_DIMS} and pages of a multiple of 16 tokens")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and out.dtype == k_cache.dtype == torch.bfloat16, "q/out/cache layout")
    _need(q.data_ptr() % 4 == 0 and q.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0 and out.stride(0) % 2 == 0, "4-byte aligned rows")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.stride(1) == 1, "block table")
    _need(positions.dtype == torch.int32 and tiles.dtype == torch.int32 and tiles.dim() == 2 and tiles.shape[1] == 3
          and tiles.is_contiguous(), "int32 positions and tiles [n, 3]")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim) and k_cache.stride() == v_cache.stride()
          and k_cache.stride(3) == 1 and k_cache.stride(2) == head_dim and k_cache.data_ptr() % 16 == 0
          and k_cache.stride(0) % 8 == 0 and k_cache.stride(1) % 8 == 0, "cache shape [pages, NKV, page_size, HD], 16-byte rows")
    _check(library().eg_attention_prefill(
        _stream(), _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.stride(0),
        _ptr(positions), _ptr(tiles), tiles.shape[0], _ptr(out), out.stride(0), num_heads, num_kv_heads, head_dim,
        page_size, k_cache.stride(0), k_cache.stride(1), k_cache.shape[0], int(window or 0), float(scale),
        _ptr(status)), "attention_prefill")


PREFILL_PARTS_SCRATCH_BYTES = 256 << 20
PREFILL_PART_TILES = int(os.environ.get("EASY_GPT_PREFILL_PART_TILES", "4"))      # fewest key tiles (of 64) per part
_parts_scratch = {}


def _prefill_parts_scratch(device, slots: int, parts: int, head_dim: int):
    """Scratch of the prompt attention: partial results when key ranges are cut (grown, never
    shrunk), tickets and the work queue, which stay zero between launches."""
    key = (device, head_dim)
    need = slots * parts * 128 if parts > 1 else 0
    have = _parts_scratch.get(key)
    if have is None or have[0].numel() < need * head_dim or have[2].numel() < slots:
        have = (torch.empty(max(need * head_dim, 1), dtype=torch.float32, device=device),
                torch.empty(max(need * 2, 1), dtype=torch.float32, device=device),
                torch.zeros(max(slots, 1024), dtype=torch.int32, device=device),
                have[3] if have is not None else torch.zeros(2, dtype=torch.int32, device=device))
        _parts_scratch[key] = have
    return have


def attention_prefill_parts(num_tiles: int, num_heads: int, head_dim: int = 64):
    """(parts, part_tiles): the most parts a query tile's keys are cut into, and the fewest key tiles
    (of 64) of a part; the kernel cuts a tile's keys into min(parts, key tiles / part_tiles) parts, so
    the cut follows the contexts of the step at hand (a captured step is replayed with others).
    A part costs its CTA a start-up of some microseconds and a pass of the merge kernel, which pays
    only while there are fewer (tile, head) pairs than CTAs (one per SM for heads of 64, whose CTAs
    share a unit's keys between two softmax groups already; two per SM else): the kernel is bound by
    what an SM gets through (about 0.64 key tiles a microsecond), not by its longest unit.  Measured on
    B200 (14 heads of 64, pages of 64): a portion of 512 tokens on a context of 3,584 (56 pairs) takes
    68 us uncut with one softmax group a CTA and 34 us in 4 parts; a prompt of 2,048 tokens (224 pairs)
    41 us uncut and 40 to 62 us however it is cut, with two groups a CTA 30 us.  (The native engine's
    rule, ``plans::attention_prefill_parts``, also cuts key ranges of 48 tiles and more into parts of 24
    when the units are many, which pays in serving runs with portions deep in long contexts; this face
    keeps the plain rule.)"""
    ctas = sm_count() * (1 if library().eg_attention_prefill_groups(head_dim) == 2 else 2)
    wanted = min(ctas // max(1, num_tiles * num_heads), 8)
    return (wanted, PREFILL_PART_TILES) if wanted >= 2 else (1, 1 << 20)


def attention_prefill_tcgen05_takes(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in (64, 128) and page_size % 16 == 0


def attention_prefill_tcgen05(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                              positions: torch.Tensor, tiles: torch.Tensor, out: torch.Tensor, num_heads: int,
                              num_kv_heads: int, head_dim: int, window: Optional[int], scale: float,
                              status: torch.Tensor, trace: Optional[torch.Tensor] = None, parts: int = 1,
                              part_tiles: int = 0) -> None:
    """The same as ``attention_prefill`` on the tcgen05 tensor cores (TMA-fed, accumulators in
    TMEM): persistent CTAs, two per SM, deal out units of (128 query rows, head, part of the key
    range).  ``parts``: the most parts a query tile's keys are cut into, of about ``part_tiles``
    tiles of 64 keys.  The cache's last page must hold finite numbers."""
    _cuda(q, k_cache, v_cache, block_table, positions, tiles, out, status)
    page_size = k_cache.shape[2]
    _need(attention_prefill_tcgen05_takes(q.dtype, head_dim, page_size),
          "attention_prefill_tcgen05 takes bfloat16, head sizes 64 and 128 and pages of a multiple of 16 tokens")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16, "q/out/cache layout")
    _need(q.data_ptr() % 16 == 0 and q.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0 and out.stride(0) % 8 == 0
          and q.shape[1] >= num_heads * head_dim, "16-byte aligned rows")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.stride(1) == 1, "block table")
    _need(positions.dtype == torch.int32 and tiles.dtype == torch.int32 and tiles.dim() == 2 and tiles.shape[1] == 3
          and tiles.is_contiguous(), "int32 positions and tiles [n, 3]")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim) and k_cache.stride() == v_cache.stride()
          and k_cache.shape == v_cache.shape and k_cache.stride(3) == 1 and k_cache.stride(2) == head_dim
          and k_cache.data_ptr() % 16 == 0 and v_cache.data_ptr() % 16 == 0
          and k_cache.stride(0) % head_dim == 0 and k_cache.stride(1) % head_dim == 0,
          "cache shape [pages, NKV, page_size, HD], strides in whole rows")
    parts = max(1, min(int(parts), 8))
    slots = tiles.shape[0] * num_heads
    while parts > 1 and slots * parts * 128 * (head_dim + 2) * 4 > PREFILL_PARTS_SCRATCH_BYTES:
        parts -= 1
    partial_o, partial_ml, tickets, queue = _prefill_parts_scratch(q.device, slots, parts, head_dim)
    _check(library().eg_attention_prefill_tcgen05(
        _stream(), _ptr(q), q.stride(0), q.shape[0], _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.stride(0),
        _ptr(positions), _ptr(tiles), tiles.shape[0], _ptr(out), out.stride(0), num_heads, num_kv_heads, head_dim,
        page_size, k_cache.stride(0), k_cache.stride(1), k_cache.shape[0], int(window or 0), float(scale),
        _ptr(status), _ptr(trace) if trace is not None else None, parts, int(part_tiles or PREFILL_PART_TILES),
        _ptr(partial_o), _ptr(partial_ml), _ptr(queue)), "attention_prefill_tcgen05")


SKINNY_KERNEL_TOKENS = 64      # what the kernel takes
# up to where it beats the library product (the policy of ``gemm_skinny_takes``); EASY_GPT_SKINNY_MAX_TOKENS moves it
SKINNY_MAX_TOKENS = int(os.environ.get("EASY_GPT_SKINNY_MAX_TOKENS", "16"))
PREFETCH_WEIGHTS = os.environ.get("EASY_GPT_PREFETCH", "0") != "0"
# every CTA repeats the norm prologue: worth it only for a few tokens (EASY_GPT_FUSED_NORM_MAX_TOKENS moves it)
FUSED_NORM_MAX_TOKENS = int(os.environ.get("EASY_GPT_FUSED_NORM_MAX_TOKENS", "16"))
EPI_STORE, EPI_F32, EPI_SWIGLU, EPI_QKV_ROPE, EPI_RESID_NORM = 0, 1, 2, 3, 4
# Programmatic dependent launch between the decode kernels (EASY_GPT_PDL).  2: a kernel lets the next one start when it has
# passed its own wait (the next one then streams its first weights while this one works); 1: at its very start, so
# that several kernels' CTAs sit waiting on the SMs (measured 5% slower per decode step); 0: no overlap.
USE_PDL = int(os.environ.get("EASY_GPT_PDL", "2"))


def fused_norm_max_tokens(width: int) -> int:
    """Up to how many tokens a step's add + RMSNorm over rows of ``width`` can ride in the decode product's
    prologue: the policy's limit, lowered where the rows of a token tile (8 or 16 tokens, bfloat16, padded),
    the gain and the partial sums of squares of a product in front (one per 16 output rows at most) would not
    fit the kernel's 200 KB of shared memory.  0: the norm runs as a kernel of its own (also for widths that
    are no multiple of 16, which the decode product does not take)."""
    if width % 16:
        return 0
    for tile in (16, 8):
        row = -(-2 * width // 128) * 128 + 64
        need = tile * row + tile * 4 + width * 4 + tile * 32 + -(-width // 16) * tile * 4
        if need <= 200 * 1024:
            return min(tile, FUSED_NORM_MAX_TOKENS)
    return 0


def skinny_plan(n_rows: int, in_features: int, head_dim: int = 0):
    """(row_blocks, k_slices, k_split): how the warps of a CTA and the CTAs of the grid share a
    [n_rows, in_features] weight matrix.  Every warp should have about four 64-wide chunks of K to
    stream (all in flight at once); big matrices put two 16-row blocks in a CTA, small ones cut K
    across CTAs so that most SMs take part."""
    chunks = -(-in_features // 64)
    if head_dim:                                   # fused QKV: one CTA per head
        rb = head_dim // 16
        ks = 1
        while ks * 2 * rb <= 16 and chunks > 4 * ks:
            ks *= 2
        # a head of a larger model is more than one SM should stream alone: its K range is cut across up to
        # 8 CTAs (a cluster) of about 128 KB each, at least four chunks a warp
        split = max(1, min(8, (head_dim * in_features * 2 + (64 << 10)) // (128 << 10)))
        heads = max(1, n_rows // head_dim)
        split = max(1, min(split, sm_count() // heads))      # no more CTAs than SMs
        if heads * 8 > sm_count():                            # only where the heads leave most SMs idle
            split = 1
        while split > 1 and chunks < 4 * ks * split:
            split -= 1
        return rb, ks, split
    if n_rows >= 64 * sm_count():                    # wide matrices (gate/up, the head): 64 rows per CTA
        return 4, 2, 1                             # (sixteen warps per CTA measured slower: one CTA per SM)
    rb, ks = 1, 8
    split = max(1, min(8, round(chunks / (ks * 2.5))))
    groups = -(-n_rows // 16)
    if groups >= sm_count():                         # the row groups alone fill the SMs
        split = 1
    while split > 1 and groups * split > 2 * sm_count():      # no more CTAs than are on the GPU at once, two an SM
        split -= 1
    return rb, ks, split


def gemm_skinny_takes(dtype: torch.dtype, tokens: int, in_features: int) -> bool:
    return dtype == torch.bfloat16 and 0 < tokens <= SKINNY_MAX_TOKENS and in_features % 16 == 0


_skinny_scratch = {}


def _scratch_for(device, floats: int, row_groups: int):
    """Per-device scratch for products whose K range is cut across CTAs: partial sums and
    ticket counters (zero between launches).  Allocated once, outside any graph capture."""
    key = str(device)
    have = _skinny_scratch.get(key)
    if have is None or have[0].numel() < floats or have[1].numel() < row_groups:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the decode scratch must be allocated before a CUDA graph is captured "
                              "(run the step once eagerly first)")
        have = (torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device),
                torch.zeros(max(row_groups, 1 << 14), dtype=torch.int32, device=device))
        _skinny_scratch[key] = have
    return have


def skinny_padded_tokens(tokens: int) -> int:
    """The token tile of ``gemm_skinny`` for this many tokens (8, 16, 32 or 64)."""
    return 8 if tokens <= 8 else 16 if tokens <= 16 else 32 if tokens <= 32 else 64


def gemm_skinny(weight: torch.Tensor, bias: Optional[torch.Tensor], out: Optional[torch.Tensor], epilogue: int, *,
                x: Optional[torch.Tensor] = None, resid_in: Optional[torch.Tensor] = None,
                resid_out: Optional[torch.Tensor] = None, delta: Optional[torch.Tensor] = None,
                gain: Optional[torch.Tensor] = None, eps: float = 0.0, tokens: Optional[int] = None,
                plan=None, rope: Optional[dict] = None, prefetch: Optional[torch.Tensor] = None,
                status: Optional[torch.Tensor] = None, prenormed: Optional[tuple] = None,
                follow: Optional[dict] = None, norm=None):
    """Decode-step product out = f(x W^T + bias) for up to 64 tokens, bfloat16 weights
    streamed once.  The input is ``x`` (bfloat16 [M, K]), or the norm prologue (``resid_in``,
    optional ``delta`` and ``resid_out``, ``gain``, ``eps``), or ``prenormed`` = (xn, ss_parts)
    with ``eps``: what an EPI_RESID_NORM product in front has left.  Epilogues:
    EPI_STORE (bfloat16), EPI_F32, EPI_SWIGLU (interleaved gate/up rows), EPI_QKV_ROPE
    (``rope``: num_heads, num_kv_heads, head_dim, positions, slot_map, k_cache, v_cache,
    inv_freq, status), EPI_RESID_NORM (``follow``: residual float32 [M, N], updated in place,
    and gain float32 [N] of the norm that follows; ``out`` is None and the call returns
    (xn, ss_parts) for the next product's ``prenormed``).  ``plan``: (row_blocks, k_slices,
    k_split), by default ``skinny_plan``.  ``prefetch``: a contiguous tensor (weights of a
    kernel that runs soon) that this kernel asks the L2 to fetch while it works.  ``norm``: the
    same input given as one object with the fields eps, gain, residual, delta, residual_out,
    prepared_rows, prepared_sums (``parts.base.NormInFront``).  ``status``:
    the step's status word, where the bounded wait for the prologue's staged input reports
    if it gives up."""
    if norm is not None:
        eps = norm.eps
        if norm.prepared_rows is not None:
            prenormed = (norm.prepared_rows, norm.prepared_sums)
        else:
            resid_in, resid_out, delta, gain = norm.residual, norm.residual_out, norm.delta, norm.gain
    _cuda(weight, bias, out, x, resid_in, resid_out, delta, gain, prefetch, status)
    N, K = weight.shape
    ss_in, ss_parts = None, 0
    if prenormed is not None:
        xn, ss_in = prenormed
        _cuda(xn, ss_in)
        M = tokens if tokens is not None else xn.shape[0]
        _need(xn.dtype == torch.bfloat16 and xn.is_contiguous() and xn.shape[-1] == K, "prenormed rows: bfloat16 [M, K]")
        _need(ss_in.dtype == torch.float32 and ss_in.is_contiguous() and ss_in.dim() == 2
              and ss_in.shape[1] == skinny_padded_tokens(M), "partial sums: float32 [parts, padded tokens]")
        norm_mode, delta, ss_parts = 2, xn, ss_in.shape[0]
    elif x is None:
        norm_mode = 1
        _need(resid_in is not None and gain is not None and resid_in.dtype == gain.dtype == torch.float32
              and resid_in.is_contiguous() and resid_in.shape[-1] == K, "norm prologue: float32 residual [M, K] and gain")
        _need(delta is None or (delta.dtype == torch.bfloat16 and delta.is_contiguous() and delta.shape[-1] == K), "delta bfloat16 [M, K]")
        _need(resid_out is None or (resid_out.dtype == torch.float32 and resid_out.is_contiguous()
                                    and resid_out.data_ptr() != resid_in.data_ptr()), "resid_out: another float32 buffer")
        M = tokens if tokens is not None else resid_in.shape[0]
    else:
        norm_mode = 0
        _need(x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] == K and x.stride(1) == 1
              and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0, "x: bfloat16 [M, K], 16-byte aligned rows")
        M = x.shape[0]
    _need(weight.dtype == torch.bfloat16 and weight.stride(1) == 1 and weight.stride(0) % 16 == 0
          and weight.data_ptr() % 32 == 0, "weight: bfloat16 [N, K], 32-byte aligned rows")
    _need(0 < M <= SKINNY_KERNEL_TOKENS and K % 16 == 0, f"gemm_skinny takes 1..{SKINNY_KERNEL_TOKENS} tokens and K % 16 == 0")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == N), "bias float32 [N]")
    r = rope or {}
    result = None
    follow_args = (None, None, None, None)
    if epilogue == EPI_QKV_ROPE:
        kc, vc = r["k_cache"], r["v_cache"]
        _need(out.dtype == torch.bfloat16 and out.stride(1) == 1 and out.shape[1] == r["num_heads"] * r["head_dim"], "q out")
        _need(r["inv_freq"].numel() * 2 == r["head_dim"], "the fused rotation covers the whole head")
        _need(kc.dtype == torch.bfloat16 and kc.stride(3) == 1 and kc.stride(2) == r["head_dim"] and kc.stride() == vc.stride(), "cache layout")
        rb, ks, split = plan or skinny_plan(N, K, r["head_dim"])
        extra = (r["num_heads"], r["num_kv_heads"], r["head_dim"], _ptr(r["positions"]), _ptr(r["slot_map"]), _ptr(kc),
                 _ptr(vc), _ptr(r["inv_freq"]), kc.shape[2], kc.stride(0), kc.stride(1), kc.shape[0] * kc.shape[2],
                 _ptr(r["status"]))
    else:
        rb, ks, split = plan or skinny_plan(N, K)
        if epilogue == EPI_RESID_NORM:
            residual, gain_out = follow["residual"], follow["gain"]
            _cuda(residual, gain_out)
            _need(residual.dtype == gain_out.dtype == torch.float32 and residual.is_contiguous() and residual.dim() == 2
                  and residual.shape[0] >= M and residual.shape[1] == N and gain_out.numel() == N,
                  "follow: float32 residual [M, N] and gain [N]")
            xn_out = torch.empty((M, N), device=weight.device, dtype=torch.bfloat16)
            ss_out = torch.empty((-(-N // (rb * 16)), skinny_padded_tokens(M)), device=weight.device, dtype=torch.float32)
            follow_args = (_ptr(residual), _ptr(gain_out), _ptr(xn_out), _ptr(ss_out))
            result = (xn_out, ss_out)
        else:
            want = torch.float32 if epilogue == EPI_F32 else torch.bfloat16
            cols = N // 2 if epilogue == EPI_SWIGLU else N
            _need(out.dtype == want and out.dim() == 2 and out.stride(1) == 1 and out.shape[0] >= M and out.shape[1] == cols, "out shape")
        extra = (0, 0, 0, None, None, None, None, None, 0, 0, 0, 0, _ptr(status))
    scratch = counters = None
    if split > 1:
        groups = -(-N // (rb * 16))
        scratch, counters = _scratch_for(weight.device, split * groups * rb * 16 * skinny_padded_tokens(M), groups)
    _check(library().eg_gemm_skinny(
        _stream(), epilogue, norm_mode, USE_PDL, _ptr(weight), weight.stride(0), _ptr(bias), M, N, K,
        _ptr(x), 0 if norm_mode else x.stride(0), _ptr(resid_in), _ptr(resid_out), _ptr(delta), _ptr(gain), float(eps),
        _ptr(out), out.stride(0) if out is not None else 0, rb, ks, split, _ptr(scratch), _ptr(counters), *extra,
        _ptr(prefetch) if PREFETCH_WEIGHTS else None,
        prefetch.numel() * prefetch.element_size() if (prefetch is not None and PREFETCH_WEIGHTS) else 0,
        Timeline.slot(f"skinny e={epilogue} n={norm_mode} {N}x{K} plan={rb},{ks},{split}"),
        _ptr(ss_in), ss_parts, *follow_args), "gemm_skinny")
    return result


# The package's own tcgen05/TMA product reaches 0.85 PFLOP/s on the widest prefill product against the library's
# 1.22 (profiles/), but with SwiGLU in its epilogue it saves the separate activation kernel and the round trip of the
# [tokens, 2 x intermediate] product through memory: a 2,048-token prefill takes 3.00 ms with it and 3.26 ms with the
# library product plus the SwiGLU kernel.  So gate/up + SwiGLU goes through ours where the wide kernel takes the
# shape; the other products of a prompt stay with the library.  EASY_GPT_TCGEN05=0 switches it off.
USE_TCGEN05 = os.environ.get("EASY_GPT_TCGEN05", "1") != "0"
# the wide products on CTA pairs (tcgen05.mma.cta_group::2, 256 x 256 tiles, TMA-store epilogue); 0: one CTA per 128 x 256 tile
USE_TCGEN05_PAIR = os.environ.get("EASY_GPT_TCGEN05_PAIR", "1") != "0"


def gemm_tcgen05_takes(dtype: torch.dtype, tokens: int, out_features: int, in_features: int) -> bool:
    """Shapes the tcgen05/TMA product takes: bfloat16, N a multiple of 128, K a multiple of 64."""
    return (dtype == torch.bfloat16 and tokens > SKINNY_MAX_TOKENS and out_features % 128 == 0
            and in_features % 64 == 0)


def gemm_tcgen05_wide_takes(dtype: torch.dtype, tokens: int, out_features: int, in_features: int) -> bool:
    """Products wide and tall enough for the persistent 128 x 256 tile kernel (one tile per SM at least)."""
    return (USE_TCGEN05 and gemm_tcgen05_takes(dtype, tokens, out_features, in_features) and out_features % 256 == 0
            and -(-tokens // 128) * (out_features // 256) >= sm_count())


def gemm_tcgen05(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                 status: torch.Tensor, swiglu_epilogue: bool = False, pair: bool = False,
                 trace: Optional[torch.Tensor] = None) -> None:
    """out = x @ weight^T + bias on the tcgen05 tensor cores (TMA-fed, accumulator in TMEM).  With
    ``swiglu_epilogue`` the weight's rows are interleaved gate/up and out is [M, N/2]."""
    _cuda(x, weight, bias, out, status)
    M, K = x.shape
    N = weight.shape[0]
    _need(x.dtype == weight.dtype == out.dtype == torch.bfloat16, "bfloat16 only")
    _need(weight.shape[1] == K and N % 128 == 0 and K % 64 == 0, "gemm_tcgen05 takes N % 128 == 0 and K % 64 == 0")
    _need(x.stride(1) == 1 and weight.stride(1) == 1 and out.stride(1) == 1, "unit inner strides")
    _need(x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and out.stride(0) % 8 == 0
          and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0, "16-byte aligned rows")
    _need(tuple(out.shape) == (M, N // 2 if swiglu_epilogue else N), "out shape")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == N), "bias float32 [N]")
    if pair:
        tile_n = 256 if (N % 256 == 0 and (swiglu_epilogue or -(-M // 256) * (N // 256) >= sm_count() // 2)) else 128
        _need(N % tile_n == 0, "SwiGLU on CTA pairs takes N % 256 == 0")
        _check(library().eg_gemm_tcgen05_pair(_stream(), EPI_SWIGLU if swiglu_epilogue else EPI_STORE, _ptr(x), x.stride(0),
                                              _ptr(weight), weight.stride(0), _ptr(bias), _ptr(out), out.stride(0), M, N, K,
                                              tile_n, _ptr(status), _ptr(trace)), "gemm_tcgen05_pair")
        return
    _check(library().eg_gemm_tcgen05(_stream(), EPI_SWIGLU if swiglu_epilogue else EPI_STORE, _ptr(x), x.stride(0),
                                     _ptr(weight), weight.stride(0), _ptr(bias), _ptr(out), out.stride(0), M, N, K,
                                     _ptr(status)), "gemm_tcgen05")


FEW_ROWS_MAX = 128             # rows of the tcgen05 product for the larger decode batches and short prompt portions
# Measured at 64 rows against the library product (microseconds, L2 flushed): qkv 7.2 / 4.6, gate+up 9.5 / 7.7,
# down 14.3 / 9.7, head 80 / 57; a decode step at batch 64 takes 2.54 ms with it and 1.81 ms without.  A tile's
# start-up (TMEM, barriers, the first TMA round trip) is too long for products this small, so it is off by default.
USE_TCGEN05_FEW = os.environ.get("EASY_GPT_TCGEN05_FEW", "0") != "0"
_few_scratch = {}


def gemm_tcgen05_few_plan(out_features: int, in_features: int):
    """(tile_n, slices): output columns per CTA and slices of K, so that about two CTAs per SM
    stream the weights; None if the kernel does not take the shape."""
    if in_features % 64 or out_features % 32:
        return None
    tile_n = 32
    for t in (128, 64):
        if out_features % t == 0 and out_features // t >= 2 * sm_count():
            tile_n = t
            break
    tiles = out_features // tile_n
    slices = max(1, min(round(2 * sm_count() / tiles), in_features // 64, 8))
    return tile_n, slices


def gemm_tcgen05_few_takes(dtype: torch.dtype, tokens: int, out_features: int, in_features: int) -> bool:
    return (USE_TCGEN05_FEW and dtype == torch.bfloat16 and SKINNY_MAX_TOKENS < tokens <= FEW_ROWS_MAX
            and gemm_tcgen05_few_plan(out_features, in_features) is not None)


def gemm_tcgen05_few(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                     status: torch.Tensor, epilogue: int = 0, plan=None) -> None:
    """out = f(x @ weight^T + bias) for at most 128 rows on the tcgen05 tensor cores: narrow
    column tiles and slices of K so that every SM streams a share of the weights once; slices
    are added up by the CTA that finishes last.  Epilogues: EPI_STORE (bfloat16), EPI_F32,
    EPI_SWIGLU (interleaved gate/up rows, out [M, N/2])."""
    _cuda(x, weight, bias, out, status)
    M, K = x.shape
    N = weight.shape[0]
    plan = plan or gemm_tcgen05_few_plan(N, K)
    _need(plan is not None and 0 < M <= FEW_ROWS_MAX, "gemm_tcgen05_few takes at most 128 rows, N % 32 == 0 and K % 64 == 0")
    tile_n, slices = plan
    _need(x.dtype == weight.dtype == torch.bfloat16 and weight.shape[1] == K, "bfloat16 x and weight")
    _need(epilogue in (EPI_STORE, EPI_F32, EPI_SWIGLU), "epilogue")
    _need(out.dtype == (torch.float32 if epilogue == EPI_F32 else torch.bfloat16)
          and tuple(out.shape) == (M, N // 2 if epilogue == EPI_SWIGLU else N), "out dtype and shape")
    _need(x.stride(1) == 1 and weight.stride(1) == 1 and out.stride(1) == 1, "unit inner strides")
    _need(x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and out.stride(0) % 8 == 0
          and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0, "16-byte aligned rows")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == N), "bias float32 [N]")
    partial = tickets = None
    if slices > 1:
        tiles = N // tile_n
        floats = tiles * slices * 128 * tile_n
        key = str(x.device)
        have = _few_scratch.get(key)
        if have is None or have[0].numel() < floats or have[1].numel() < tiles:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("the product's scratch must be allocated before a CUDA graph is captured "
                                  "(run the step once eagerly first)")
            have = (torch.empty(max(floats, 1 << 22), dtype=torch.float32, device=x.device),
                    torch.zeros(max(tiles, 1 << 12), dtype=torch.int32, device=x.device))
            _few_scratch[key] = have
        partial, tickets = have
    _check(library().eg_gemm_tcgen05_few(_stream(), epilogue, int(USE_PDL), _ptr(x), x.stride(0), _ptr(weight), weight.stride(0),
                                         _ptr(bias), _ptr(out), out.stride(0), M, N, K, tile_n, slices, _ptr(partial),
                                         _ptr(tickets), _ptr(status)), "gemm_tcgen05_few")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = up * silu(gate) for rows laid out [gate_0, up_0, gate_1, up_1, ...]."""
    _cuda(gate_up, out)
    T, two_i = gate_up.shape
    inter = two_i // 2
    _need(two_i == 2 * inter and out.shape == (T, inter) and gate_up.dtype == out.dtype, "swiglu shapes")
    _need(gate_up.stride(1) == 1 and out.stride(1) == 1, "unit inner strides")
    _check(library().eg_swiglu(_stream(), dtype_code(out.dtype), _ptr(gate_up), gate_up.stride(0), _ptr(out),
                               out.stride(0), T, inter), "swiglu")


_argmax_scratch = {}
ARGMAX_BLOCKS = 32


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = lowest index of the maximum of logits[r, :] (float32 rows)."""
    _cuda(logits, out)
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "float32 rows")
    _need(out.dtype == torch.int32 and out.numel() >= logits.shape[0], "int32 out")
    rows, vocab = logits.shape
    blocks = max(1, min(ARGMAX_BLOCKS, vocab // 4096))
    vals = idxs = counters = None
    if blocks > 1:
        key = str(logits.device)
        have = _argmax_scratch.get(key)
        if have is None or have[2].numel() < rows:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("argmax scratch must exist before a CUDA graph is captured")
            cap = max(rows, 1024)
            have = (torch.empty(cap * ARGMAX_BLOCKS, dtype=torch.float32, device=logits.device),
                    torch.empty(cap * ARGMAX_BLOCKS, dtype=torch.int32, device=logits.device),
                    torch.zeros(cap, dtype=torch.int32, device=logits.device))
            _argmax_scratch[key] = have
        vals, idxs, counters = have
    _check(library().eg_argmax(_stream(), _ptr(logits), logits.stride(0), rows, vocab, _ptr(out), blocks, _ptr(vals),
                               _ptr(idxs), _ptr(counters)), "argmax")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           uniform: torch.Tensor, out: torch.Tensor) -> None:
    """Per row: temperature <= 0 -> greedy; else softmax(logits / T) cut by top_k
    (0 = off) and top_p (1 = off), drawn by inverse CDF in index order with uniform[r]."""
    _cuda(logits, temperature, top_k, top_p, uniform, out)
    rows = logits.shape[0]
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "float32 rows")
    _need(temperature.dtype == top_p.dtype == uniform.dtype == torch.float32 and top_k.dtype == torch.int32
          and out.dtype == torch.int32, "float32 temperature/top_p/uniform, int32 top_k/out")
    _need(min(temperature.numel(), top_k.numel(), top_p.numel(), uniform.numel(), out.numel()) >= rows, "one value per row")
    _check(library().eg_sample(_stream(), _ptr(logits), logits.stride(0), rows, logits.shape[1], _ptr(temperature),
                               _ptr(top_k), _ptr(top_p), _ptr(uniform), _ptr(out)), "sample")


def wait_probe(limit: int, threads: int, status: torch.Tensor) -> int:
    """Launches one CTA of ``threads`` threads that all wait, through the kernels' bounded wait with a limit of
    ``limit`` polls, on a barrier that nothing completes.  The wait runs out, EG_STATUS_WAIT_TIMEOUT is
    set in ``status`` and the kernel returns.  Returns how many threads gave up (all of them).  For
    tests: it shows on a healthy GPU what the host sees when a wait inside a kernel runs out."""
    _cuda(status)
    _need(status.dtype == torch.int32, "status int32")
    gave_up = torch.zeros(1, dtype=torch.int32, device=status.device)
    _check(library().eg_wait_probe(_stream(), int(limit), int(threads), _ptr(status), _ptr(gave_up)), "wait_probe")
    return int(gave_up.item())


def describe_status(word: int) -> str:
    return "; ".join(text for bit, text in STATUS_BITS.items() if word & bit) or "ok"
