"""GPU parity of sigmoid_attention (dense) with the CPU oracle, through the public API and
therefore through the C ABI.  Shapes, seeds and tolerances follow the reference's
tests/test_sigmoid_dense.py, plus the benchmark configurations."""

import math

import pytest
import torch

import triton_sigmoid_b200 as m
from tests.conftest import tolerance
from tests.gpu_util import O_TOL, check_against_oracle, make_inputs, rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,H,T,D", [(1, 2, 128, 64), (4, 2, 256, 64), (1, 8, 512, 128), (2, 2, 1024, 64),
                                     (1, 2, 2048, 128)])
def test_parity_sweep(B, H, T, D, causal, dtype):
    # inputs ~ N(0, 0.5) as in the reference's sweep; reference-level tolerance on O
    q, k, v, do = make_inputs(B, T, T, H, D, dtype, std=0.5, seed=T + D, requires_grad=True)
    check_against_oracle(m.sigmoid_attention, q, k, v, do, dtype, is_causal=causal, o_tol=tolerance(dtype))


@pytest.mark.parametrize("causal", [False, True])
def test_benchmark_config_small_fp32_case(causal):
    """B=2, N=256, H=4, D=64, N(0,1) inputs (the CPU-runnable configuration), in fp16."""
    q, k, v, do = make_inputs(2, 256, 256, 4, 64, torch.float16, seed=0, requires_grad=True)
    check_against_oracle(m.sigmoid_attention, q, k, v, do, torch.float16, is_causal=causal)


@pytest.mark.parametrize("T", [1, 7, 15, 33, 127, 129, 255, 257, 300])
@pytest.mark.parametrize("causal", [False, True])
def test_ragged_lengths(T, causal):
    q, k, v, do = make_inputs(2, T, T, 2, 64, torch.float16, std=0.5, seed=T, requires_grad=True)
    check_against_oracle(m.sigmoid_attention, q, k, v, do, torch.float16, is_causal=causal)


@pytest.mark.parametrize("D", [16, 32, 96])
def test_small_head_dims_are_zero_extended(D):
    q, k, v, do = make_inputs(2, 200, 200, 3, D, torch.bfloat16, std=0.5, seed=D, requires_grad=True)
    check_against_oracle(m.sigmoid_attention, q, k, v, do, torch.bfloat16, is_causal=True)


def test_explicit_scale_and_bias():
    q, k, v, do = make_inputs(2, 384, 384, 2, 64, torch.float16, seed=5, requires_grad=True)
    check_against_oracle(m.sigmoid_attention, q, k, v, do, torch.float16, scale=0.2, sigmoid_bias=-2.0)
    q.grad = k.grad = v.grad = None
    check_against_oracle(m.sigmoid_attention, q, k, v, do, torch.float16, sigmoid_bias=0.0)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_score_mod(dtype):
    q, k, v, do = make_inputs(2, 320, 320, 2, 64, dtype, std=0.5, seed=9, requires_grad=True)
    sm = torch.randn(2, 320, device="cuda", dtype=dtype)
    check_against_oracle(m.sigmoid_attention, q, k, v, do, dtype, score_mod=sm, is_causal=True)
    zeros = torch.zeros(2, 320, device="cuda")
    a = m.sigmoid_attention(q, k, v, score_mod=zeros)
    b = m.sigmoid_attention(q, k, v)
    assert (a.float() - b.float()).abs().max().item() <= 1e-5


def test_causality():
    q, k, v, _ = make_inputs(1, 512, 512, 2, 64, torch.float16, seed=11)
    o1 = m.sigmoid_attention(q, k, v, is_causal=True)
    k2, v2 = k.clone(), v.clone()
    k2[:, 300:] += 1.0
    v2[:, 300:] -= 2.0
    o2 = m.sigmoid_attention(q, k2, v2, is_causal=True)
    assert torch.equal(o1[:, :300], o2[:, :300])
    assert not torch.equal(o1[:, 300:], o2[:, 300:])
    assert not torch.equal(o1, m.sigmoid_attention(q, k, v, is_causal=False))


def test_linearity_in_v_at_benchmark_size():
    """Size-independent property at B=4, N=4096, H=16, D=64 (fp16): O is linear in V."""
    q, k, v1, _ = make_inputs(4, 4096, 4096, 16, 64, torch.float16, seed=1)
    v2 = torch.randn_like(v1)
    o1 = m.sigmoid_attention(q, k, v1).float()
    o2 = m.sigmoid_attention(q, k, v2).float()
    o12 = m.sigmoid_attention(q, k, (v1.float() * 0.5 + v2.float() * 0.25).half()).float()
    assert (o12 - (0.5 * o1 + 0.25 * o2)).abs().max().item() <= 4e-3


@pytest.mark.parametrize("causal", [False, True])
def test_benchmark_size_against_gpu_fp32_math(causal):
    """B=4, N=4096, H=16, D=64 fp16 (benchmark configuration) against fp32 torch math on the GPU,
    one batch element at a time to bound memory."""
    B, T, H, D = 4, 4096, 16, 64
    q, k, v, do = make_inputs(B, T, T, H, D, torch.float16, seed=1, requires_grad=True)
    out = m.sigmoid_attention(q, k, v, is_causal=causal)
    out.backward(do)
    for b in range(B):
        qb, kb, vb = [t[b:b + 1].detach().float().requires_grad_() for t in (q, k, v)]
        # the library's default bias is -log(T), the torch formula adds 1e-6 inside the log
        ref = m.sigmoid_attention_ref(qb, kb, vb, causal=causal, sigmoid_bias=-math.log(T))
        ref.backward(do[b:b + 1].float())
        assert (out[b:b + 1].float() - ref).abs().max().item() <= O_TOL[torch.float16]
        for g, r in ((q.grad, qb.grad), (k.grad, kb.grad), (v.grad, vb.grad)):
            assert rel_l2(g[b:b + 1], r) <= 1e-2


def test_long_sequence_d128_against_gpu_fp32_math():
    """bf16 causal, N=8192, D=128 (the shape family of the multi-GPU configuration), two heads."""
    B, T, H, D = 1, 8192, 2, 128
    q, k, v, do = make_inputs(B, T, T, H, D, torch.bfloat16, std=0.5, seed=3, requires_grad=True)
    out = m.sigmoid_attention(q, k, v, is_causal=True)
    out.backward(do)
    qb, kb, vb = [t.detach().float().requires_grad_() for t in (q, k, v)]
    ref = m.sigmoid_attention_ref(qb, kb, vb, causal=True, sigmoid_bias=-math.log(T))
    ref.backward(do.float())
    assert (out.float() - ref).abs().max().item() <= O_TOL[torch.bfloat16]
    for g, r in ((q.grad, qb.grad), (k.grad, kb.grad), (v.grad, vb.grad)):
        assert rel_l2(g, r) <= 1e-2


def test_forward_is_deterministic():
    q, k, v, _ = make_inputs(2, 1024, 1024, 4, 64, torch.bfloat16, seed=13)
    assert torch.equal(m.sigmoid_attention(q, k, v, is_causal=True), m.sigmoid_attention(q, k, v, is_causal=True))


def test_large_inputs_stay_finite():
    q, k, v, do = make_inputs(1, 256, 256, 2, 64, torch.float16, std=10.0, seed=17, requires_grad=True)
    out = m.sigmoid_attention(q, k, v)
    out.backward(do)
    for t in (out, q.grad, k.grad, v.grad):
        assert torch.isfinite(t).all()
        assert t.abs().max().item() < 1e6


def test_zeros_and_ones():
    z = torch.zeros(1, 128, 2, 64, device="cuda", dtype=torch.float16)
    o = m.sigmoid_attention(z, z, torch.ones_like(z), sigmoid_bias=0.0)
    assert (o.float() - 64.0).abs().max().item() <= 0.1  # 128 keys x sigmoid(0) = 64


def test_autograd_semantics():
    q, k, v, do = make_inputs(1, 128, 128, 2, 64, torch.float16, seed=19)
    assert not m.sigmoid_attention(q, k, v).requires_grad
    q.requires_grad_()
    out = m.sigmoid_attention(q, k, v)
    assert out.requires_grad
    out.backward(do)
    assert q.grad is not None and k.grad is None and v.grad is None


def test_non_contiguous_inputs():
    base = torch.randn(2, 2, 256, 64, device="cuda", dtype=torch.float16) * 0.5  # (B,H,T,D)
    q = k = v = base.transpose(1, 2)  # (B,T,H,D) view, not contiguous
    a = m.sigmoid_attention(q, k, v)
    b = m.sigmoid_attention(q.contiguous(), k.contiguous(), v.contiguous())
    assert torch.equal(a, b)


def test_many_heads_and_batches():
    for B, H in ((16, 1), (32, 4), (1, 32)):
        q, k, v, _ = make_inputs(B, 128, 128, H, 64, torch.float16, seed=B + H)
        o = m.sigmoid_attention(q, k, v)
        assert o.shape == q.shape and torch.isfinite(o).all()


def test_empty_batch_and_empty_sequence():
    e = torch.empty(0, 128, 2, 64, device="cuda", dtype=torch.float16)
    assert m.sigmoid_attention(e, e, e).shape == e.shape
    e = torch.empty(2, 0, 2, 64, device="cuda", dtype=torch.float16)
    assert m.sigmoid_attention(e, e, e).shape == e.shape
