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


def test_the_native_engine_plans_like_the_pytorch_face():
    """The launch rules exist twice, in ``csrc/engine/plans.hpp`` for the native engine and in ``kernels.py`` for the
    PyTorch face: over the sizes of the family's models and some odd ones they must give the same plans."""
    from easy_gpt.cpp_b200 import native

    assert native.plan(4)[0] == kernels.sm_count()
    shapes = [(1152, 896, 64), (896, 896, 0), (9728, 896, 0), (896, 4864, 0), (151936, 896, 0), (2048, 1536, 128),
              (1536, 1536, 0), (17920, 1536, 0), (1536, 8960, 0), (151936, 1536, 0), (4608, 3584, 128), (3584, 3584, 0),
              (37888, 3584, 0), (3584, 18944, 0), (152064, 3584, 0), (48, 48, 0), (391, 80, 0), (160, 112, 16), (96, 2048, 32),
              (256, 4096, 0), (640, 640, 0), (5120, 5120, 128), (8192, 8192, 0), (1024, 28672, 0)]
    for rows, width, head in shapes:
        assert native.plan(0, rows, width, head)[:3] == tuple(kernels.skinny_plan(rows, width, head)), (rows, width, head)
    for tokens in (1, 2, 4, 8, 9, 16, 17, 24, 32, 48, 64, 128):
        for heads, kv, head in ((14, 2, 64), (12, 2, 128), (28, 4, 128), (4, 4, 32), (16, 1, 256), (3, 1, 64)):
            for context in (1, 63, 64, 500, 4096, 8192, 32768, 131072):
                assert native.plan(1, tokens, heads, kv, context, head)[0] == \
                    kernels.attention_paged_splits(tokens, heads, kv, context, head), (tokens, heads, kv, context, head)
    for width in (48, 120, 896, 1536, 3584, 5000, 8192, 20000):
        assert native.plan(2, width)[0] == kernels.fused_norm_max_tokens(width), width
    # the prompt attention's rule, for contexts short enough that the native engine's extra rule for long ranges is silent
    for tiles in (1, 2, 3, 4, 8, 16, 40, 200):
        for heads, head in ((14, 64), (12, 128), (28, 128), (4, 64)):
            assert native.plan(3, tiles, heads, head, 2048)[:2] == tuple(kernels.attention_prefill_parts(tiles, heads, head)), (tiles, heads, head)
