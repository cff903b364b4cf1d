"""The plain implementation against logits that the reference's own CPU model
code produced in true 32-bit (tests/golden/make_golden.py)."""
import tempfile
from pathlib import Path

import numpy as np
import torch

import plain_model
from golden import golden_model


def test_plain_matches_reference_logits():
    ref = np.load(Path(__file__).parent / "golden" / "ref_logits.npy")
    with tempfile.TemporaryDirectory() as tmp:
        golden_model.write_model_dir(tmp)
        cfg, w = plain_model.read_model_dir(tmp)
    # The reference rounds the scaled scores through bfloat16 even in its 32-bit
    # build (src/tensor.cpp:95-99).  With that one quirk restated the two agree
    # to float32 rounding; without it the gap is the size of that rounding.
    for quirk, bound in ((True, 3e-6), (False, 5e-4)):
        whole = {rid: plain_model.forward_logits(cfg, w, ids, round_scores_like_reference=quirk).numpy()
                 for rid, ids in golden_model.REQUESTS.items()}
        mine = np.stack([whole[rid][pos] for rid, pos in golden_model.wanted_rows()])
        assert mine.shape == ref.shape
        assert np.abs(mine - ref).max() < bound, (quirk, np.abs(mine - ref).max())
        assert (mine.argmax(-1) == ref.argmax(-1)).all()


def test_plain_matches_reference_logits_at_positions_in_the_thousands():
    """RoPE base 1e6 over 2,100 positions (angles of thousands of radians), with a portion of 50 tokens
    and two single tokens on top of a cache of 2,048: the reference's own 32-bit CPU logits at the rows
    of golden_model.KEPT_LONG."""
    ref = np.load(Path(__file__).parent / "golden" / "ref_logits_long.npy")
    with tempfile.TemporaryDirectory() as tmp:
        golden_model.write_model_dir(tmp, golden_model.CONFIG_LONG)
        cfg, w = plain_model.read_model_dir(tmp)
    assert cfg["rope_theta"] == 1e6
    ids = golden_model.long_request()
    with torch.no_grad():
        mine = plain_model.forward_logits(cfg, w, ids, round_scores_like_reference=True).numpy()[golden_model.KEPT_LONG]
    assert mine.shape == ref.shape
    err = np.abs(mine - ref).max()
    assert err < 2e-5, err
    assert (mine.argmax(-1) == ref.argmax(-1)).all()


def test_plain_float64_agrees_with_float32():
    with tempfile.TemporaryDirectory() as tmp:
        golden_model.write_model_dir(tmp)
        cfg, w32 = plain_model.read_model_dir(tmp)
        _, w64 = plain_model.read_model_dir(tmp, dtype=torch.float64)
    ids = golden_model.REQUESTS[0]
    a = plain_model.forward_logits(cfg, w32, ids)
    b = plain_model.forward_logits(cfg, w64, ids)
    assert (a.double() - b).abs().max() < 1e-5
