"""Pins the CPU oracle to outputs of the reference project's own PyTorch code (tests/golden/)."""

import json
import os

import numpy as np
import pytest
import torch

from tests.conftest import GOLDEN
from oracle import sigattn_oracle as orc
from tests.golden.make_golden import SMALL_CASES


@pytest.fixture(scope="module")
def golden():
    return np.load(os.path.join(GOLDEN, "small_cases.npz"))


def _case(golden, name):
    c = SMALL_CASES[name]
    t = lambda k: torch.from_numpy(golden[f"{name}/{k}"].astype(np.float32))
    lq = torch.tensor(c["lens_q"], dtype=torch.int32) if "lens_q" in c else None
    lk = torch.tensor(c["lens_k"], dtype=torch.int32) if "lens_k" in c else None
    sm = t("score_mod") if c.get("score_mod") else None
    kw = dict(seq_lens_k=lk, seq_lens_q=lq, is_causal=c.get("causal", False), scale=c.get("scale"),
              sigmoid_bias=c.get("sigmoid_bias"), score_mod=sm)
    return t, kw


@pytest.mark.parametrize("name", sorted(SMALL_CASES))
def test_oracle_matches_reference_outputs(golden, name):
    t, kw = _case(golden, name)
    o = orc.sigattn_forward(t("q"), t("k"), t("v"), **kw)
    dq, dk, dv = orc.sigattn_backward(t("q"), t("k"), t("v"), t("do"), **kw)
    # fp32 on both sides; the reference adds 1e-6 inside its log for the padded bias
    for got, key in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        ref = t(key)
        assert got.shape == ref.shape
        assert torch.isfinite(got).all()
        assert (got - ref).abs().max().item() <= 2e-5, (name, key)


@pytest.mark.parametrize("name", sorted(SMALL_CASES))
def test_oracle_fp64_agrees_with_fp32(golden, name):
    t, kw = _case(golden, name)
    o32 = orc.sigattn_forward(t("q"), t("k"), t("v"), **kw)
    o64 = orc.sigattn_forward(t("q"), t("k"), t("v"), work=torch.float64, **kw)
    assert (o32.double() - o64).abs().max().item() <= 2e-5


def test_oracle_config1_sums():
    """B=2, N=256, H=4, D=64, seed 0 - the CPU-runnable benchmark configuration."""
    with open(os.path.join(GOLDEN, "config1_sums.json")) as f:
        sums = json.load(f)
    torch.manual_seed(0)
    q, k, v, do = [torch.randn(2, 256, 4, 64) for _ in range(4)]
    got_in = float(sum(t.double().abs().sum() for t in (q, k, v, do)))
    if abs(got_in - sums["input_abs_sum"]) > 1e-6 * sums["input_abs_sum"]:
        pytest.skip("torch CPU RNG stream differs from the one the fixture was made with")
    lens = torch.tensor(sums["lens"], dtype=torch.int32)
    for name, (l, causal) in {"dense": (None, False), "causal": (None, True),
                              "padded": (lens, False), "padded_causal": (lens, True)}.items():
        o = orc.sigattn_forward(q, k, v, seq_lens_k=l, seq_lens_q=l, is_causal=causal, work=torch.float64)
        dq, dk, dv = orc.sigattn_backward(q, k, v, do, seq_lens_k=l, seq_lens_q=l, is_causal=causal,
                                          work=torch.float64)
        ref = sums[name]
        assert float(o.sum()) == pytest.approx(ref["sum_o"], rel=1e-4, abs=1e-2)
        assert float(o.abs().sum()) == pytest.approx(ref["abs_o"], rel=1e-4)
        assert float(dq.abs().sum()) == pytest.approx(ref["abs_dq"], rel=1e-4)
        assert float(dk.abs().sum()) == pytest.approx(ref["abs_dk"], rel=1e-4)
        assert float(dv.abs().sum()) == pytest.approx(ref["abs_dv"], rel=1e-4)


def test_padded_rows_are_zero(golden):
    t, kw = _case(golden, "padded")
    o = orc.sigattn_forward(t("q"), t("k"), t("v"), **kw)
    dq, dk, dv = orc.sigattn_backward(t("q"), t("k"), t("v"), t("do"), **kw)
    assert o[0, 77:].abs().max() == 0 and o[1, 31:].abs().max() == 0
    assert dq[1, 31:].abs().max() == 0 and dk[1, 31:].abs().max() == 0 and dv[1, 31:].abs().max() == 0


def test_zero_length_keys_give_zeros():
    q, k, v, do = [torch.randn(2, 32, 2, 16) for _ in range(4)]
    lk = torch.tensor([0, 20], dtype=torch.int32)
    o = orc.sigattn_forward(q, k, v, seq_lens_k=lk)
    grads = orc.sigattn_backward(q, k, v, do, seq_lens_k=lk)
    for x in (o, *grads):
        assert torch.isfinite(x).all()
    assert o[0].abs().max() == 0
