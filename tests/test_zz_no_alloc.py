"""eg_argmax_noalloc, the entry point that allocates nothing, called through its exported C
symbol and compared with the existing entry point (kernels.argmax), twice in a row.

It is for callers that cannot allocate while they run: code inside or replaying a CUDA graph
capture, a decode loop whose memory was handed out at start-up, or a user of the shared
library's C symbols without torch's allocator behind them.  Its scratch memory is a fixed
device array inside the library (csrc/argmax_noalloc.h).  This file sorts last on purpose,
so that a run that stops at the first failure has run every other test before it; it passes
alone in a fresh process as well."""
import ctypes

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
