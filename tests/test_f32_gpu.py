"""float32 tensors: the exact single-precision kernels against the float64 oracle.

The reference accepts float32 and holds it to 1e-5 (tests/conftest.py:27-34 and
tests/test_sigmoid_dense.py:38-135 of the reference); the same inputs (std 0.5) and gate are
used here, with the oracle evaluated in float64 so that the gate measures the kernels only.
"""

import json
import math
import os

import pytest
import torch

import triton_sigmoid_b200 as m
from oracle import sigattn_oracle as orc
from tests.gpu_util import make_inputs, rel_l2

pytestmark = pytest.mark.gpu

O_TOL_F32 = 1e-5       # max-abs on O while |O| <= 1, relative to max|O| beyond
GRAD_REL_L2_F32 = 1e-5
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _check(q, k, v, do, lens_q=None, lens_k=None, **kw):
    B, Tq, H, D = q.shape
    Tk = k.shape[1]
    if lens_q is not None or lens_k is not None:
        out = m.sigmoid_attention_padded(q, k, v, seq_lens_k=lens_k, seq_lens_q=lens_q, **kw)
    else:
        out = m.sigmoid_attention(q, k, v, **kw)
    assert out.dtype == torch.float32 and out.shape == q.shape
    okw = dict(seq_lens_k=lens_k, seq_lens_q=lens_q, is_causal=kw.get("is_causal", False), scale=kw.get("scale"),
               sigmoid_bias=kw.get("sigmoid_bias"), score_mod=kw.get("score_mod"), work=torch.float64)
    ref = orc.sigattn_forward(q, k, v, **okw)
    got = out.detach().double().cpu()
    assert torch.isfinite(got).all()
    gate = O_TOL_F32 * max(1.0, ref.abs().max().item())
    assert (got - ref).abs().max().item() <= gate
    mq, mk = orc.valid_row_masks(B, Tq, Tk, lens_q, lens_k)
    if (~mq).any():
        assert got[~mq].abs().max().item() == 0
    out.backward(do)
    rdq, rdk, rdv = orc.sigattn_backward(q, k, v, do, **okw)
    for name, g, r, mask in (("dq", q.grad, rdq, mq), ("dk", k.grad, rdk, mk), ("dv", v.grad, rdv, mk)):
        g = g.double().cpu()
        assert torch.isfinite(g).all(), name
        assert rel_l2(g, r) <= GRAD_REL_L2_F32, name
        if (~mask).any():
            assert g[~mask].abs().max().item() == 0, f"{name}: padded rows must be zero"


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,H,T,D", [(1, 2, 128, 64), (2, 4, 256, 64), (1, 2, 512, 128), (1, 1, 1024, 64)])
def test_dense(B, H, T, D, causal):
    q, k, v, do = make_inputs(B, T, T, H, D, torch.float32, std=0.5, seed=T + D, requires_grad=True)
    _check(q, k, v, do, is_causal=causal)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("T", [1, 7, 63, 65, 129, 300])
def test_ragged_lengths(T, causal):
    q, k, v, do = make_inputs(2, T, T, 2, 64, torch.float32, std=0.5, seed=T, requires_grad=True)
    _check(q, k, v, do, is_causal=causal)


def test_cross_lengths():
    B, Tq, Tk, H, D = 2, 100, 333, 2, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    q = (torch.randn(B, Tq, H, D, device="cuda", generator=g) * 0.5).requires_grad_()
    k = (torch.randn(B, Tk, H, D, device="cuda", generator=g) * 0.5).requires_grad_()
    v = (torch.randn(B, Tk, H, D, device="cuda", generator=g) * 0.5).requires_grad_()
    do = torch.randn(B, Tq, H, D, device="cuda", generator=g) * 0.5
    # different query and key lengths exist in the padded entry point only (as in the reference)
    _check(q, k, v, do, lens_k=torch.tensor([333, 200], dtype=torch.int32, device="cuda"))


@pytest.mark.parametrize("D", [16, 32, 96])
def test_small_head_dims(D):
    q, k, v, do = make_inputs(2, 200, 200, 2, D, torch.float32, std=0.5, seed=D, requires_grad=True)
    _check(q, k, v, do, is_causal=True)


def _fill_padding(tensors, lens, value):
    with torch.no_grad():
        for b in range(len(lens)):
            for t in tensors:
                t[b, int(lens[b]):] = value


@pytest.mark.parametrize("causal", [False, True])
def test_padded(causal):
    B, T, H, D = 4, 256, 2, 64
    q, k, v, do = make_inputs(B, T, T, H, D, torch.float32, std=0.5, seed=9, requires_grad=True)
    lens = torch.tensor([256, 77, 0, 130], dtype=torch.int32, device="cuda")
    _fill_padding((q, k, v, do), lens, 1.0e3)  # finite garbage (the oracle multiplies masked zeros with it)
    _check(q, k, v, do, lens_q=lens, lens_k=lens, is_causal=causal)


def test_padding_content_never_reaches_a_result():
    """Non-finite padding must give bit-identical results to zero padding."""
    B, T, H, D = 3, 200, 2, 64
    lens = torch.tensor([200, 33, 129], dtype=torch.int32, device="cuda")
    results = []
    for fill in (0.0, float("nan")):
        q, k, v, do = make_inputs(B, T, T, H, D, torch.float32, std=0.5, seed=14, requires_grad=True)
        _fill_padding((q, k, v, do), lens, fill)
        out = m.sigmoid_attention_padded(q, k, v, seq_lens_k=lens, seq_lens_q=lens, is_causal=True)
        out.backward(do)
        results.append((out.detach(), q.grad, k.grad, v.grad))
    for a, b in zip(*results):
        assert torch.isfinite(b).all()
        assert torch.equal(a, b)


def test_padded_keys_only_and_queries_only():
    B, T, H, D = 2, 192, 2, 64
    lens = torch.tensor([100, 192], dtype=torch.int32, device="cuda")
    q, k, v, do = make_inputs(B, T, T, H, D, torch.float32, std=0.5, seed=10, requires_grad=True)
    _check(q, k, v, do, lens_k=lens)
    q, k, v, do = make_inputs(B, T, T, H, D, torch.float32, std=0.5, seed=11, requires_grad=True)
    _check(q, k, v, do, lens_q=lens)


def test_scale_bias_and_score_mod():
    B, T, H, D = 2, 160, 2, 64
    q, k, v, do = make_inputs(B, T, T, H, D, torch.float32, std=0.5, seed=12, requires_grad=True)
    mod = torch.randn(B, T, device="cuda") * 0.5
    _check(q, k, v, do, scale=0.2, sigmoid_bias=-1.5, score_mod=mod, is_causal=True)


def test_benchmark_config_1_against_reference_sums():
    """B=2, N=256, H=4, D=64 float32, seed 0 (the reference's CPU-runnable configuration): the
    sums the reference's torch formula produced for these inputs."""
    with open(os.path.join(GOLDEN, "config1_sums.json")) as f:
        sums = json.load(f)
    torch.manual_seed(0)
    q, k, v, do = [torch.randn(2, 256, 4, 64) for _ in range(4)]
    got_in = float(sum(t.double().abs().sum() for t in (q, k, v, do)))
    if abs(got_in - sums["input_abs_sum"]) > 1e-6 * sums["input_abs_sum"]:
        pytest.skip("torch CPU RNG stream differs from the one the fixture was made with")
    lens = torch.tensor(sums["lens"], dtype=torch.int32, device="cuda")
    for name, (l, causal) in {"dense": (None, False), "causal": (None, True),
                              "padded": (lens, False), "padded_causal": (lens, True)}.items():
        qc, kc, vc = [t.cuda().requires_grad_() for t in (q, k, v)]
        if l is None:
            out = m.sigmoid_attention(qc, kc, vc, is_causal=causal)
        else:
            out = m.sigmoid_attention_padded(qc, kc, vc, seq_lens_k=l, seq_lens_q=l, is_causal=causal)
        out.backward(do.cuda())
        out = out.detach()
        ref = sums[name]
        assert float(out.double().sum()) == pytest.approx(ref["sum_o"], rel=1e-4, abs=1e-2)
        assert float(out.double().abs().sum()) == pytest.approx(ref["abs_o"], rel=1e-4)
        assert float(qc.grad.double().abs().sum()) == pytest.approx(ref["abs_dq"], rel=1e-4)
        assert float(kc.grad.double().abs().sum()) == pytest.approx(ref["abs_dk"], rel=1e-4)
        assert float(vc.grad.double().abs().sum()) == pytest.approx(ref["abs_dv"], rel=1e-4)


def test_deterministic_forward_and_backward():
    q, k, v, do = make_inputs(2, 300, 300, 2, 64, torch.float32, std=0.5, seed=21, requires_grad=True)
    outs = []
    for _ in range(2):
        for t in (q, k, v):
            t.grad = None
        o = m.sigmoid_attention(q, k, v, is_causal=True)
        o.backward(do)
        outs.append((o.detach().clone(), q.grad.clone(), k.grad.clone(), v.grad.clone()))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_compiled_call():
    q, k, v, do = make_inputs(1, 128, 128, 2, 64, torch.float32, std=0.5, seed=22, requires_grad=True)
    fn = torch.compile(m.sigmoid_attention, backend="aot_eager")
    out = fn(q, k, v, is_causal=True)
    ref = orc.sigattn_forward(q, k, v, is_causal=True, work=torch.float64)
    assert (out.detach().double().cpu() - ref).abs().max().item() <= O_TOL_F32
    out.backward(do)
    assert q.grad is not None and math.isfinite(q.grad.abs().sum().item())
