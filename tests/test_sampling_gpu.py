"""The sampling kernels against the plain rule (GPU)."""
import numpy as np
import pytest
import torch

import plain_model
from easy_gpt.cpp_b200.sampling.rng import uniform

pytestmark = pytest.mark.gpu


def test_uniform_numbers_match_the_plain_twin():
    for args in ((0, 0, 0), (42, 7, 123), (2**40 + 5, 3, 2**33)):
        u = uniform(*args)
        assert 0.0 <= u < 1.0 and u == plain_model.uniform_from_counter(*args)
    us = [uniform(1, r, i) for r in range(40) for i in range(50)]
    assert abs(np.mean(us) - 0.5) < 0.02 and len(set(us)) > 1990


@pytest.mark.parametrize("vocab", [203, 1000, 151936])
def test_argmax_lowest_index_wins(vocab):
    from easy_gpt.cpp_b200 import kernels

    g = torch.Generator().manual_seed(vocab)
    logits = torch.randn(5, vocab, generator=g)
    logits[1, vocab - 1] = logits[1, 17] = 50.0           # a tie: the lower index
    logits[2, 0] = 60.0
    logits[3, vocab - 1] = 60.0
    logits[4, 5] = float("nan")
    out = torch.empty(5, dtype=torch.int32, device="cuda")
    kernels.argmax(logits.cuda(), out)
    want = [int(np.argmax(np.nan_to_num(logits[r].numpy(), nan=-np.inf))) for r in range(5)]
    assert out.tolist() == want and want[1] == 17


CASES = [(0.8, 0, 1.0), (1.0, 0, 1.0), (0.3, 20, 0.95), (1.5, 5, 1.0), (0.8, 0, 0.9), (2.0, 1, 1.0), (1.0, 50, 0.5),
         (0.7, 1000000, 0.3)]


@pytest.mark.parametrize("vocab", [203, 4097, 151936])
def test_sampling_follows_the_rule(vocab):
    """For many rows and settings the kernel's token lies in the kept set of the
    plain rule and the uniform number falls into that token's slice of the CDF."""
    from easy_gpt.cpp_b200 import kernels

    rng = np.random.default_rng(vocab)
    rows = len(CASES) * 6
    logits = torch.from_numpy(rng.normal(0, 2.5, size=(rows, vocab)).astype(np.float32))
    logits[3, 10:14] = logits[3].max() + 1.0               # ties at the top across a top-k edge
    temps = torch.tensor([CASES[r % len(CASES)][0] for r in range(rows)], dtype=torch.float32)
    topk = torch.tensor([min(CASES[r % len(CASES)][1], 2**31 - 1) for r in range(rows)], dtype=torch.int32)
    topp = torch.tensor([CASES[r % len(CASES)][2] for r in range(rows)], dtype=torch.float32)
    us = torch.tensor([uniform(9, r, 0) for r in range(rows)], dtype=torch.float32)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    kernels.sample(logits.cuda(), temps.cuda(), topk.cuda(), topp.cuda(), us.cuda(), out)
    got = out.tolist()
    exact = 0
    for r in range(rows):
        p = plain_model.sampling_distribution(logits[r], float(temps[r]), int(topk[r]), float(topp[r]))
        tok = got[r]
        cdf = np.cumsum(p)
        lo, hi = (cdf[tok - 1] if tok else 0.0), cdf[tok]
        u = float(us[r])
        slack = 2e-5
        kept = np.nonzero(p)[0]
        if p[tok] == 0.0:
            # only a token at the very edge of the top-p cut may differ (float32 against float64 mass)
            edge = plain_model.sampling_distribution(logits[r], float(temps[r]), int(topk[r]), min(1.0, float(topp[r]) + 1e-4))
            assert edge[tok] > 0.0, (r, tok, "token outside the kept set")
        else:
            assert lo - slack <= u <= hi + slack, (r, tok, lo, u, hi)
        exact += tok == plain_model.sample_token(logits[r], float(temps[r]), int(topk[r]), float(topp[r]), u)
        if int(topk[r]) == 1:
            assert tok == int(np.argmax(logits[r].numpy()))
        assert len(kept) <= (int(topk[r]) if 0 < int(topk[r]) < vocab else vocab)
    assert exact >= rows - 2


def test_greedy_rows_inside_a_sampled_batch():
    from easy_gpt.cpp_b200 import kernels

    logits = torch.randn(4, 500, generator=torch.Generator().manual_seed(1))
    temps = torch.tensor([0.0, 1.0, 0.0, 0.5])
    out = torch.empty(4, dtype=torch.int32, device="cuda")
    kernels.sample(logits.cuda(), temps.cuda(), torch.zeros(4, dtype=torch.int32).cuda(), torch.ones(4).cuda(),
                   torch.full((4,), 0.5).cuda(), out)
    assert out[0].item() == int(logits[0].argmax()) and out[2].item() == int(logits[2].argmax())


def test_distribution_over_many_draws():
    from easy_gpt.cpp_b200 import kernels

    vocab, n = 12, 4000
    row = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, 3.0, 2.5, -3.0, 0.2, 0.1, 1.7, -0.4])
    logits = row.repeat(n, 1).cuda()
    us = torch.tensor([uniform(3, 0, i) for i in range(n)], dtype=torch.float32).cuda()
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    kernels.sample(logits, torch.full((n,), 0.7).cuda(), torch.full((n,), 6, dtype=torch.int32).cuda(),
                   torch.full((n,), 0.9).cuda(), us, out)
    freq = np.bincount(out.cpu().numpy(), minlength=vocab) / n
    p = plain_model.sampling_distribution(row, 0.7, 6, 0.9)
    assert np.abs(freq - p).max() < 0.03 and (freq[p == 0] == 0).all()


@pytest.mark.parametrize("top_k,top_p", [(0, 1.0), (5, 1.0), (0, 0.8), (600, 0.9)])
def test_a_nan_logit_is_never_drawn(top_k, top_p):
    """A NaN in a row is left out at every temperature, as the greedy path leaves it out: the drawn
    token follows the plain rule over the other logits."""
    from easy_gpt.cpp_b200 import kernels

    vocab, rows = 500, 16
    rng = np.random.default_rng(top_k + 7)
    logits = torch.from_numpy(rng.normal(0, 2.0, size=(rows, vocab)).astype(np.float32))
    nan_at = [int(logits[r].argmax()) if r % 2 else 3 * r for r in range(rows)]       # the would-be winner, or any place
    for r in range(rows):
        logits[r, nan_at[r]] = float("nan")
        logits[r, (nan_at[r] + 250) % vocab] = float("nan")
    us = torch.tensor([uniform(5, r, 1) for r in range(rows)], dtype=torch.float32)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    kernels.sample(logits.cuda(), torch.full((rows,), 0.9).cuda(), torch.full((rows,), top_k, dtype=torch.int32).cuda(),
                   torch.full((rows,), top_p).cuda(), us.cuda(), out)
    exact = 0
    for r, tok in enumerate(out.tolist()):
        assert not np.isnan(float(logits[r, tok])), (r, tok)
        clean = torch.nan_to_num(logits[r], nan=-1e30)
        p = plain_model.sampling_distribution(clean, 0.9, top_k, top_p)
        assert p[nan_at[r]] == 0.0
        edge = plain_model.sampling_distribution(clean, 0.9, top_k, min(1.0, top_p + 1e-4))
        assert edge[tok] > 0.0, (r, tok)
        exact += tok == plain_model.sample_token(clean, 0.9, top_k, top_p, float(us[r]))
    assert exact >= rows - 1
