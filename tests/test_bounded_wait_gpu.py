"""The kernels' waits are bounded: a wait whose signal never comes gives up after its limit, records
where in the device's health word and returns, the context stays usable, calls made while the word
is set are refused with an error (RuntimeError from the Python functions), and reading the word
clears it.  The expiry is provoked on a barrier that nothing arrives on (a few milliseconds), never
by a fault or an endless loop."""

import ctypes
import math

import pytest
import torch

import triton_sigmoid_b200 as m
from oracle import sigattn_oracle as orc
from triton_sigmoid_b200 import _cabi

pytestmark = pytest.mark.gpu


def _fwd_params(q, k, v, o):
    B, T, H, D = q.shape
    p = _cabi.SigAttnParams()
    p.struct_bytes = ctypes.sizeof(p)
    p.dtype, p.B, p.H, p.D, p.Tq, p.Tk = _cabi.SIGATTN_FP16, B, H, D, T, T
    p.scale = 1.0 / math.sqrt(D)
    p.bias_scalar = -math.log(T)
    p.device = 0
    p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    s3 = (ctypes.c_int64 * 3)(*q.stride()[:3])
    p.q_strides = p.k_strides = p.v_strides = p.o_strides = s3
    p.stream = torch.cuda.current_stream().cuda_stream
    return p


def test_expired_wait_is_reported_and_the_library_recovers():
    lib = _cabi.load()
    torch.cuda.synchronize()
    assert lib.sigattn_device_status(0) == 0
    assert lib.sigattn_query(99) == -1  # (unknown query: the library answers, nothing is pending)

    assert lib.sigattn_selftest_bounded_wait(0, 20) == 1, lib.sigattn_last_error()

    # the health word is set now: calls are refused, nothing is launched, outputs stay untouched
    torch.manual_seed(0)
    q, k, v = [torch.randn(1, 256, 2, 64, device="cuda", dtype=torch.float16) * 0.5 for _ in range(3)]
    o = torch.full_like(q, 7.0)
    p = _fwd_params(q, k, v, o)
    assert lib.sigattn_fwd(ctypes.byref(p)) == -5
    assert b"gave up on a bounded wait" in lib.sigattn_last_error() and b"0x30001" in lib.sigattn_last_error()
    torch.cuda.synchronize()
    assert (o == 7.0).all()
    # the Python functions turn that into an exception, forward and backward
    with pytest.raises(RuntimeError, match="gave up on a bounded wait"):
        m.sigmoid_attention(q, k, v)
    lens = torch.tensor([200], dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="gave up on a bounded wait"):
        m.sigmoid_attention_padded(q, k, v, seq_lens_k=lens)

    code = lib.sigattn_device_status(0)
    assert code == 0x30001  # the self-test's wait site
    assert lib.sigattn_device_status(0) == 0  # reading it cleared it

    # and the same call now computes
    assert lib.sigattn_fwd(ctypes.byref(p)) == 0, lib.sigattn_last_error()
    torch.cuda.synchronize()
    ref = orc.sigattn_forward(q, k, v)
    assert (o.float().cpu() - ref).abs().max().item() <= 2e-3
    out = m.sigmoid_attention(q, k, v)
    assert torch.equal(out, o)
    assert lib.sigattn_device_status(0) == 0


def test_python_status_helper_and_debug_mode(monkeypatch):
    """`device_status()` reads and clears the word; with SIGATTN_B200_DEBUG=1 every call synchronises and
    checks (outputs are poison-filled first, and a healthy call overwrites all of it)."""
    lib = _cabi.load()
    assert m.device_status() == 0
    assert lib.sigattn_selftest_bounded_wait(0, 10) == 1, lib.sigattn_last_error()
    torch.manual_seed(1)
    q, k, v, do = [torch.randn(2, 300, 2, 64, device="cuda", dtype=torch.bfloat16) * 0.5 for _ in range(4)]
    monkeypatch.setenv("SIGATTN_B200_DEBUG", "1")
    with pytest.raises(RuntimeError, match="gave up on a bounded wait"):
        m.sigmoid_attention(q, k, v)
    assert m.device_status() == 0x30001
    assert m.device_status() == 0
    for t in (q, k, v):
        t.requires_grad_()
    out = m.sigmoid_attention(q, k, v, is_causal=True)
    out.backward(do)
    for t in (out, q.grad, k.grad, v.grad):
        assert torch.isfinite(t).all()
    monkeypatch.delenv("SIGATTN_B200_DEBUG")
    ref = m.sigmoid_attention(q.detach(), k.detach(), v.detach(), is_causal=True)
    assert torch.equal(out.detach(), ref)


def test_selftest_rejects_unbounded_limits():
    lib = _cabi.load()
    assert lib.sigattn_selftest_bounded_wait(0, 0) < 0
    assert lib.sigattn_selftest_bounded_wait(0, 100000) < 0
    assert b"limit_ms" in lib.sigattn_last_error()
