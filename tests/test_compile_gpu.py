"""torch.compile over the public functions: compiled == eager, backward included, and a second
call with other (B, T) works (the reference's tests/test_torch_compile.py checks the same).
Inductor's CPU C++ codegen may be unusable in some images; the ops themselves are opaque custom
ops, so the aot_eager backend exercises exactly the same tracing and fake-kernel machinery."""

import pytest
import torch

import triton_sigmoid_b200 as m
from tests.gpu_util import make_inputs

pytestmark = pytest.mark.gpu


def _compile(fn):
    torch._dynamo.reset()
    return torch.compile(fn, backend="aot_eager")


@pytest.mark.parametrize("causal", [False, True])
def test_dense_compiled_matches_eager(causal):
    fn = _compile(lambda q, k, v: m.sigmoid_attention(q, k, v, is_causal=causal))
    for B, T in ((2, 256), (3, 384)):  # second shape: recompilation / dynamic shapes must work
        q, k, v, do = make_inputs(B, T, T, 2, 64, torch.float16, std=0.5, seed=T, requires_grad=True)
        out = fn(q, k, v)
        out.backward(do)
        g = [t.grad.clone() for t in (q, k, v)]
        q.grad = k.grad = v.grad = None
        ref = m.sigmoid_attention(q, k, v, is_causal=causal)
        ref.backward(do)
        assert torch.equal(out, ref)
        # dQ is accumulated with floating-point atomics: equal up to summation order
        assert torch.allclose(g[0].float(), q.grad.float(), atol=1e-3, rtol=1e-2)
        assert torch.equal(g[1], k.grad) and torch.equal(g[2], v.grad)


def test_padded_compiled_matches_eager_with_score_mod():
    fn = _compile(lambda q, k, v, lk, lq, sm: m.sigmoid_attention_padded(q, k, v, seq_lens_k=lk, seq_lens_q=lq,
                                                                         is_causal=True, score_mod=sm))
    q, k, v, do = make_inputs(2, 192, 320, 2, 128, torch.bfloat16, std=0.5, seed=3, requires_grad=True)
    lq = torch.tensor([192, 100], dtype=torch.int32, device="cuda")
    lk = torch.tensor([300, 320], dtype=torch.int32, device="cuda")
    sm = torch.randn(2, 320, device="cuda")
    out = fn(q, k, v, lk, lq, sm)
    out.backward(do)
    gk = k.grad.clone()
    q.grad = k.grad = v.grad = None
    ref = m.sigmoid_attention_padded(q, k, v, seq_lens_k=lk, seq_lens_q=lq, is_causal=True, score_mod=sm)
    ref.backward(do)
    assert torch.equal(out, ref) and torch.equal(gk, k.grad)


def test_opcheck():
    from triton_sigmoid_b200 import ops

    q, k, v, _ = make_inputs(1, 128, 128, 2, 64, torch.float16, seed=5, requires_grad=True)
    bias = torch.zeros(1, device="cuda")
    torch.library.opcheck(ops.sigmoid_attention_fwd_op, (q, k, v, bias, None, 0.125, True),
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))


def test_varlen_compiled_matches_eager():
    lens = [100, 260, 31]
    cu = torch.tensor([0, 100, 360, 391], dtype=torch.int32, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(7)
    q, k, v, do = [(torch.randn(391, 2, 64, device="cuda", generator=g) * 0.5).half() for _ in range(4)]
    for t in (q, k, v):
        t.requires_grad_()
    fn = _compile(lambda q, k, v, cu: m.sigmoid_attention_varlen(q, k, v, cu, cu, max(lens), max(lens), is_causal=True))
    out = fn(q, k, v, cu)
    out.backward(do)
    gk = k.grad.clone()
    q.grad = k.grad = v.grad = None
    ref = m.sigmoid_attention_varlen(q, k, v, cu, cu, max(lens), max(lens), is_causal=True)
    ref.backward(do)
    assert torch.equal(out, ref) and torch.equal(gk, k.grad)
