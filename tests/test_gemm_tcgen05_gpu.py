"""The tcgen05/TMA matrix product against a float32 reference (GPU)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def bf(t):
    return t.to(torch.bfloat16)


@pytest.mark.parametrize("M, N, K", [(128, 128, 64), (128, 128, 256), (200, 256, 128), (17, 128, 64), (2048, 1152, 896),
                                      (333, 896, 4864), (1000, 9728, 896), (1300, 4096, 128), (2500, 2048, 64),
                                      (4096, 512, 320)])
def test_store_epilogue(M, N, K):
    from easy_gpt.cpp_b200 import kernels

    g = torch.Generator().manual_seed(M + N + K)
    x = bf(torch.randn(M, K, generator=g)).to(DEV)
    w = bf(torch.randn(N, K, generator=g) * 0.1).to(DEV)
    b = torch.randn(N, generator=g).to(DEV)
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.gemm_tcgen05(x, w, b, out, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    want = x.float() @ w.float().t() + b
    err = float((out.float() - want).abs().max())
    assert err <= 8e-3 * float(want.abs().max()), err
    # no bias, strided input (a slice of a wider buffer)
    wide = bf(torch.randn(M, K + 64, generator=g)).to(DEV)
    kernels.gemm_tcgen05(wide[:, 8:8 + K], w, None, out, status)
    want = wide[:, 8:8 + K].float() @ w.float().t()
    assert float((out.float() - want).abs().max()) <= 8e-3 * float(want.abs().max())
    assert status.item() == 0


@pytest.mark.parametrize("M, I, K", [(130, 64, 64), (2048, 4864, 896)])
def test_swiglu_epilogue(M, I, K):
    from easy_gpt.cpp_b200 import kernels

    g = torch.Generator().manual_seed(M + I)
    x = bf(torch.randn(M, K, generator=g)).to(DEV)
    gate, up = bf(torch.randn(I, K, generator=g) * 0.05), bf(torch.randn(I, K, generator=g) * 0.05)
    w = torch.stack([gate, up], dim=1).reshape(2 * I, K).to(DEV)
    out = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.gemm_tcgen05(x, w, None, out, status, swiglu_epilogue=True)
    gv, uv = x.float() @ gate.float().to(DEV).t(), x.float() @ up.float().to(DEV).t()
    want = uv * (gv / (1 + torch.exp(-gv)))
    assert status.item() == 0
    assert float((out.float() - want).abs().max()) <= 1e-2 * float(want.abs().max())


def test_refuses_other_shapes():
    from easy_gpt.cpp_b200 import kernels

    x = bf(torch.randn(64, 80)).to(DEV)
    w = bf(torch.randn(100, 80)).to(DEV)
    with pytest.raises(kernels.KernelError, match="N % 128"):
        kernels.gemm_tcgen05(x, w, None, torch.empty(64, 100, dtype=torch.bfloat16, device=DEV),
                             torch.zeros(1, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("M, N, K", [(17, 32, 64), (64, 1152, 896), (128, 896, 4864), (33, 9728, 896), (100, 96, 640),
                                      (64, 151936 // 4, 896)])
def test_few_rows_product(M, N, K):
    """At most 128 rows: every tile width and several slices of K, each epilogue, twice (the tickets return to zero)."""
    from easy_gpt.cpp_b200 import kernels

    g = torch.Generator().manual_seed(M * 7 + N + K)
    x = bf(torch.randn(M, K, generator=g)).to(DEV)
    w = bf(torch.randn(N, K, generator=g) * 0.1).to(DEV)
    b = torch.randn(N, generator=g).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    want = x.float() @ w.float().t() + b
    scale = float(want.abs().max())
    plans = [None] + [(t, s) for t in (32, 64, 128) if N % t == 0 for s in sorted({1, min(3, K // 64), min(K // 64, 8)})]
    for plan in plans + plans[:2]:
        out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
        kernels.gemm_tcgen05_few(x, w, b, out, status, plan=plan)
        assert status.item() == 0
        assert float((out.float() - want).abs().max()) <= 8e-3 * scale, plan
        out32 = torch.empty((M, N), dtype=torch.float32, device=DEV)
        kernels.gemm_tcgen05_few(x, w, None, out32, status, epilogue=kernels.EPI_F32, plan=plan)
        assert float((out32 - (want - b)).abs().max()) <= 1e-4 * scale, plan
    # SwiGLU on interleaved gate / up rows
    gv, uv = want[:, 0::2] - b[0::2], want[:, 1::2] - b[1::2]
    act = torch.empty((M, N // 2), dtype=torch.bfloat16, device=DEV)
    for plan in plans:
        kernels.gemm_tcgen05_few(x, w, None, act, status, epilogue=kernels.EPI_SWIGLU, plan=plan)
        ref = uv * (gv / (1 + torch.exp(-gv)))
        assert float((act.float() - ref).abs().max()) <= 1e-2 * float(ref.abs().max()) + 1e-6, plan
    assert status.item() == 0
    # a strided input (a slice of a wider buffer)
    wide = bf(torch.randn(M, K + 64, generator=g)).to(DEV)
    out = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tcgen05_few(wide[:, 8:8 + K], w, None, out, status)
    ref = wide[:, 8:8 + K].float() @ w.float().t()
    assert float((out.float() - ref).abs().max()) <= 8e-3 * float(ref.abs().max())


def test_few_rows_refuses():
    from easy_gpt.cpp_b200 import kernels

    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    x = torch.zeros(129, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(64, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(kernels.KernelError):
        kernels.gemm_tcgen05_few(x, w, None, torch.empty(129, 64, dtype=torch.bfloat16, device=DEV), status)
    with pytest.raises(kernels.KernelError):
        kernels.gemm_tcgen05_few(x[:8, :48], w[:, :48], None, torch.empty(8, 64, dtype=torch.bfloat16, device=DEV), status)


@pytest.mark.parametrize("M, N, K", [(256, 256, 64), (256, 128, 64), (300, 896, 192), (2048, 1152, 896), (333, 640, 320),
                                      (1000, 9728, 896), (130, 2304, 4864)])
def test_cta_pair_product(M, N, K):
    """Two CTAs per 256-row tile (tcgen05.mma.cta_group::2), both tile widths, rows and a last K step that end inside a
    tile, TMA-store epilogue; twice in a row."""
    from easy_gpt.cpp_b200 import kernels

    g = torch.Generator().manual_seed(M + N + K)
    x = bf(torch.randn(M, K, generator=g)).to(DEV)
    w = bf(torch.randn(N, K, generator=g) * 0.1).to(DEV)
    b = torch.randn(N, generator=g).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    want = x.float() @ w.float().t() + b
    for _ in range(2):
        out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
        kernels.gemm_tcgen05(x, w, b, out, status, pair=True)
        assert status.item() == 0
        assert float((out.float() - want).abs().max()) <= 8e-3 * float(want.abs().max())
    # a strided input and a strided output (slices of wider buffers)
    wide = bf(torch.randn(M, K + 64, generator=g)).to(DEV)
    out_wide = torch.full((M, N + 64), 3.0, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tcgen05(wide[:, 8:8 + K], w, None, out_wide[:, 32:32 + N], status, pair=True)
    ref = wide[:, 8:8 + K].float() @ w.float().t()
    assert float((out_wide[:, 32:32 + N].float() - ref).abs().max()) <= 8e-3 * float(ref.abs().max())
    assert bool((out_wide[:, :32] == 3.0).all()) and bool((out_wide[:, 32 + N:] == 3.0).all()) and status.item() == 0


@pytest.mark.parametrize("M, I, K", [(256, 128, 64), (300, 384, 192), (2048, 4864, 896)])
def test_cta_pair_swiglu(M, I, K):
    from easy_gpt.cpp_b200 import kernels

    g = torch.Generator().manual_seed(M + I)
    x = bf(torch.randn(M, K, generator=g)).to(DEV)
    gate, up = bf(torch.randn(I, K, generator=g) * 0.05), bf(torch.randn(I, K, generator=g) * 0.05)
    w = torch.stack([gate, up], dim=1).reshape(2 * I, K).to(DEV)
    out = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.gemm_tcgen05(x, w, None, out, status, swiglu_epilogue=True, pair=True)
    gv, uv = x.float() @ gate.float().to(DEV).t(), x.float() @ up.float().to(DEV).t()
    want = uv * (gv / (1 + torch.exp(-gv)))
    assert status.item() == 0
    assert float((out.float() - want).abs().max()) <= 1e-2 * float(want.abs().max())
