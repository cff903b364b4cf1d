"""eg_argmax_noalloc, the entry point that allocates nothing, called through its exported C
symbol and compared with the existing entry point (kernels.argmax), twice in a row.

It is for callers that cannot allocate while they run: code inside or replaying a CUDA graph
capture, a decode loop whose memory was handed out at start-up, or a user of the shared
library's C symbols without torch's allocator behind them.  Its scratch memory is a fixed
device array inside the library (csrc/argmax_noalloc.h).  This file sorts last on purpose,
so that a run that stops at the first failure has run every other test before it; it passes
alone in a fresh process as well."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def load():
    from easy_gpt.cpp_b200.csrc.build import library_path

    lib = ctypes.CDLL(str(library_path()))
    fn = lib.eg_argmax_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    lib.eg_argmax_noalloc_message.argtypes = [ctypes.c_int]
    lib.eg_argmax_noalloc_message.restype = ctypes.c_char_p
    return lib


def lowest_index_of_the_maximum(logits: torch.Tensor) -> np.ndarray:
    """The rule on the CPU, by numpy: NaN never wins; a row without any number that can win gives 0."""
    a = logits.detach().float().cpu().numpy()
    a = np.where(np.isnan(a), -np.inf, a)
    return np.argmax(a, axis=1).astype(np.int32)


def call(lib, logits, out):
    stream = torch.cuda.current_stream().cuda_stream
    return lib.eg_argmax_noalloc(stream, logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1], out.data_ptr())


@pytest.mark.parametrize("rows, vocab", [(8, 151936), (64, 4097), (256, 391), (3, 20000)])
def test_matches_the_existing_entry_point_twice_in_a_row(rows, vocab):
    from easy_gpt.cpp_b200 import kernels

    lib = load()
    g = torch.Generator().manual_seed(rows * 1000 + vocab)
    for attempt in range(2):                                  # the second call finds the first call's scratch
        logits = torch.randn(rows, vocab, generator=g).cuda()
        logits[0, vocab - 1] = logits[0, 3] = 40.0            # a tie: the lower index
        if rows > 2:
            logits[2, 5] = float("nan")
        want = torch.empty(rows, dtype=torch.int32, device="cuda")
        kernels.argmax(logits, want)
        got = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
        # number of allocations torch's allocator has served so far (frees by a garbage collection
        # that happens to run meanwhile do not change it)
        before = torch.cuda.memory_stats().get("allocation.all.allocated", 0)
        code = call(lib, logits, got)
        assert code == 0, lib.eg_argmax_noalloc_message(code).decode()
        assert torch.cuda.memory_stats().get("allocation.all.allocated", 0) == before     # nothing came from torch's allocator either
        torch.cuda.synchronize()
        assert torch.equal(got, want), (attempt, got[:8].tolist(), want[:8].tolist())     # token ids: exact
        assert got[0].item() == 3
        assert np.array_equal(got.cpu().numpy(), lowest_index_of_the_maximum(logits))     # and the rule itself, by numpy


def test_rows_without_a_winner_a_row_stride_and_stale_scratch():
    """Against numpy alone: a row of NaN only and a row of -inf only (both give token 0, like the CPU
    rule over NaN-masked logits), rows that are a column slice of a wider tensor (row stride larger
    than the vocabulary), and a small call right after the largest one, whose partial results are
    still in the array."""
    lib = load()
    g = torch.Generator().manual_seed(5)
    big = torch.randn(256, 151936, generator=g).cuda()
    out = torch.full((256,), -7, dtype=torch.int32, device="cuda")
    assert call(lib, big, out) == 0
    small = torch.randn(3, 20000, generator=g).cuda()                        # fewer blocks a row, fewer rows: stale partials all around
    small[1, 19999] = 9.0
    got = torch.full((3,), -7, dtype=torch.int32, device="cuda")
    assert call(lib, small, got) == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), lowest_index_of_the_maximum(big))
    assert np.array_equal(got.cpu().numpy(), lowest_index_of_the_maximum(small)) and got[1].item() == 19999
    odd = torch.randn(6, 9000, generator=g)
    odd[0] = float("nan")
    odd[1] = float("-inf")
    odd[2, :4500] = float("nan")
    odd[3, 17] = float("inf")
    odd[4, 8999] = odd[4].max() + 1
    odd = odd.cuda()
    got = torch.full((6,), -7, dtype=torch.int32, device="cuda")
    assert call(lib, odd, got) == 0
    want = lowest_index_of_the_maximum(odd)
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), want) and want[0] == 0 and want[1] == 0 and want[3] == 17
    wide = torch.randn(5, 12000, generator=g).cuda()
    part = wide[:, 1000:9001]                                                # 8001 columns, row stride 12000
    assert part.stride(0) == 12000 and not part.is_contiguous()
    got = torch.full((5,), -7, dtype=torch.int32, device="cuda")
    assert call(lib, part, got) == 0
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), lowest_index_of_the_maximum(part))


def test_refuses_more_rows_than_its_scratch_holds():
    lib = load()
    logits = torch.zeros(257, 16, device="cuda")
    out = torch.full((257,), -7, dtype=torch.int32, device="cuda")
    code = call(lib, logits, out)
    assert code == -1
    assert b"at most 256 rows" in lib.eg_argmax_noalloc_message(code)
    torch.cuda.synchronize()
    assert (out == -7).all()                                  # nothing ran
    assert lib.eg_argmax_noalloc(0, None, 16, 1, 16, out.data_ptr()) == -2
    assert call(lib, logits[:0], out) == 0                    # no rows: nothing to do
