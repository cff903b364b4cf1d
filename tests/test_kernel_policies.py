"""Host-side choices of the kernel bindings (no GPU needed): which sizes go to which kernel."""
import torch

from easy_gpt.cpp_b200 import kernels


def test_fused_norm_limit_follows_the_width():
    assert kernels.fused_norm_max_tokens(896) == kernels.FUSED_NORM_MAX_TOKENS
    assert kernels.fused_norm_max_tokens(3584) == kernels.FUSED_NORM_MAX_TOKENS
    # 16 rows of 8192 bfloat16 values do not fit 200 KB of shared memory, 8 rows do
    assert kernels.fused_norm_max_tokens(8192) == min(8, kernels.FUSED_NORM_MAX_TOKENS)
    assert kernels.fused_norm_max_tokens(20000) == 0
    assert kernels.fused_norm_max_tokens(120) == 0            # rows of 240 bytes: the decode product wants multiples of 32


def test_decode_product_policy():
    assert kernels.gemm_skinny_takes(torch.bfloat16, 1, 896)
    assert kernels.gemm_skinny_takes(torch.bfloat16, kernels.SKINNY_MAX_TOKENS, 4864)
    assert not kernels.gemm_skinny_takes(torch.bfloat16, kernels.SKINNY_MAX_TOKENS + 1, 896)
    assert not kernels.gemm_skinny_takes(torch.bfloat16, 4, 900)            # K % 16
    assert not kernels.gemm_skinny_takes(torch.float32, 4, 896)
    assert [kernels.skinny_padded_tokens(m) for m in (1, 8, 9, 16, 17, 33, 64)] == [8, 8, 16, 16, 32, 64, 64]


def test_decode_product_plans_cover_the_matrix():
    for rows, width, head in ((1152, 896, 64), (896, 896, 0), (9728, 896, 0), (896, 4864, 0), (151936, 896, 0),
                              (4608, 3584, 128), (3584, 18944, 0), (48, 48, 0), (391, 80, 0)):
        rb, ks, split = kernels.skinny_plan(rows, width, head)
        assert rb >= 1 and ks >= 1 and split >= 1
        assert rb * ks <= 32                                        # warps of a CTA
        if head:
            assert rb * 16 == head and 1 <= split <= 8
            # only heads that are much for one SM are cut, and only where the heads leave most SMs idle
            assert (split == 1) == (head * width * 2 < (192 << 10) or (rows // head) * 8 > kernels.sm_count())
