"""The backward entry point that needs no workspace from the caller (`sigattn_bwd_static_scratch`).

Hosts that may not allocate device memory when they call the library - a plugin inside a server
whose memory pool is fixed at start-up, code that runs during a stream capture, a latency-critical
loop that must stay out of the driver's allocator - use it instead of `sigattn_bwd`: the fp32 dQ
accumulator then lives in an array built into the library.  This file calls it through the C ABI
with raw pointers, twice in a row on differently sized problems (the second call must not see what
the first one left in the shared array), and compares with `sigattn_bwd`: given an ordinary
caller-owned workspace (same kernel: dK / dV bitwise equal), and in its workspace-free split mode
(tolerance of the parity tests).  Collected last on purpose (file name), so a `-x` run has
already run everything else.
"""

import ctypes
import math

import pytest
import torch

from triton_sigmoid_b200 import _cabi

pytestmark = pytest.mark.gpu


def _s3(t):
    return (ctypes.c_int64 * 3)(*t.stride()[:3])


def _params(q, k, v, do, dq, dk, dv, causal, lens=None):
    B, T, H, D = q.shape
    p = _cabi.SigAttnParams()
    p.struct_bytes = ctypes.sizeof(p)
    p.dtype = _cabi.SIGATTN_BF16 if q.dtype == torch.bfloat16 else _cabi.SIGATTN_FP16
    p.B, p.H, p.D, p.Tq, p.Tk = B, H, D, T, T
    p.flags = _cabi.SIGATTN_CAUSAL if causal else 0
    p.scale = 1.0 / math.sqrt(D)
    p.bias_scalar = -math.log(T)
    p.device = q.device.index or 0
    p.q, p.k, p.v, p.dout = q.data_ptr(), k.data_ptr(), v.data_ptr(), do.data_ptr()
    p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    for name in ("q", "k", "v", "do", "dq", "dk", "dv"):
        setattr(p, name + "_strides", _s3(q))
    if lens is not None:
        p.seq_lens_q = p.seq_lens_k = lens.data_ptr()
    p.stream = torch.cuda.current_stream().cuda_stream
    return p


def _run_both(B, T, H, D, dtype, causal, seed, lens=None):
    lib = _cabi.load()
    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k, v, do = [(torch.randn(B, T, H, D, device="cuda", generator=g) * 0.5).to(dtype) for _ in range(4)]
    # reference: the ordinary entry point (same kernel) with a caller-owned workspace
    ref = [torch.full_like(q, float("nan")) for _ in range(3)]
    ws = torch.empty(lib.sigattn_bwd_workspace_bytes(B, T, H, D) // 4, dtype=torch.float32, device="cuda")
    p = _params(q, k, v, do, *ref, causal, lens)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel() * 4
    assert lib.sigattn_bwd(ctypes.byref(p)) == 0, lib.sigattn_last_error()
    # second reference: the library's other backward (streaming kernels, no workspace at all)
    dflt = [torch.full_like(q, float("nan")) for _ in range(3)]
    p0 = _params(q, k, v, do, *dflt, causal, lens)
    p0.flags |= _cabi.SIGATTN_BWD_SPLIT
    assert lib.sigattn_bwd(ctypes.byref(p0)) == 0, lib.sigattn_last_error()
    # under test: no workspace given at all
    got = [torch.full_like(q, float("nan")) for _ in range(3)]
    p2 = _params(q, k, v, do, *got, causal, lens)
    assert lib.sigattn_bwd_static_scratch(ctypes.byref(p2)) == 0, lib.sigattn_last_error()
    torch.cuda.synchronize()
    assert lib.sigattn_device_status(0) == 0
    for name, a, b in zip(("dq", "dk", "dv"), got, ref):
        assert torch.isfinite(a).all(), name
        rel = ((a.float() - b.float()).norm() / (b.float().norm() + 1e-30)).item()
        # same kernels, same inputs: dK/dV are bitwise equal, dQ differs only by the order of the
        # floating-point reductions; the gate is the one the parity tests use for gradients
        assert rel <= 1e-2, f"{name}: relative L2 difference {rel:.3e}"
    assert torch.equal(got[1], ref[1]) and torch.equal(got[2], ref[2])
    for name, a, b in zip(("dq", "dk", "dv"), got, dflt):
        rel = ((a.float() - b.float()).norm() / (b.float().norm() + 1e-30)).item()
        assert rel <= 1e-2, f"{name} against the split backward: relative L2 difference {rel:.3e}"


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    # first a larger problem, then a smaller one whose accumulator overlaps what the first left behind
    _run_both(2, 1024, 4, 64, torch.float16, causal=False, seed=1)
    lens = torch.tensor([300, 77, 512], dtype=torch.int32, device="cuda")
    _run_both(3, 512, 2, 128, torch.bfloat16, causal=True, seed=2, lens=lens)


def test_float32_and_packed_layouts_through_the_same_entry_point():
    """float32 tensors use no accumulator at all, so the size limit does not apply to them; packed
    (cu_seqlens) batches go through the built-in accumulator like padded ones."""
    lib = _cabi.load()
    g = torch.Generator(device="cuda").manual_seed(5)
    # float32, larger than the limit would allow for 16-bit tensors
    B, T, H, D = 1, 2304, 64, 64
    assert B * T * H * D > _cabi.SIGATTN_STATIC_SCRATCH_ELEMS
    q, k, v, do = [torch.randn(B, T, H, D, device="cuda", generator=g) * 0.5 for _ in range(4)]
    got = [torch.full_like(q, float("nan")) for _ in range(3)]
    ref = [torch.full_like(q, float("nan")) for _ in range(3)]
    for outs, fn in ((got, lib.sigattn_bwd_static_scratch), (ref, lib.sigattn_bwd)):
        p = _params(q, k, v, do, *outs, True)
        p.dtype = _cabi.SIGATTN_FP32
        assert fn(ctypes.byref(p)) == 0, lib.sigattn_last_error()
    torch.cuda.synchronize()
    for a, b in zip(got, ref):
        assert torch.equal(a, b)
    # packed: three sequences of 100, 37 and 163 tokens in (300, H, D) tensors
    total, H, D = 300, 2, 64
    cu = torch.tensor([0, 100, 137, 300], dtype=torch.int32, device="cuda")
    q, k, v, do = [(torch.randn(total, H, D, device="cuda", generator=g) * 0.5).half() for _ in range(4)]
    outs = {}
    for key, fn in (("static", lib.sigattn_bwd_static_scratch), ("default", lib.sigattn_bwd)):
        ws = torch.empty(lib.sigattn_bwd_workspace_bytes(1, total, H, D) // 4, dtype=torch.float32, device="cuda")
        o = [torch.zeros_like(q) for _ in range(3)]
        p = _cabi.SigAttnParams()
        p.struct_bytes = ctypes.sizeof(p)
        p.dtype, p.B, p.H, p.D, p.Tq, p.Tk = _cabi.SIGATTN_FP16, 3, H, D, 163, 163
        p.scale, p.bias_scalar, p.device = 1.0 / math.sqrt(D), -4.0, 0
        p.q, p.k, p.v, p.dout = q.data_ptr(), k.data_ptr(), v.data_ptr(), do.data_ptr()
        p.dq, p.dk, p.dv = [t.data_ptr() for t in o]
        s3 = (ctypes.c_int64 * 3)(0, q.stride(0), q.stride(1))
        for name in ("q", "k", "v", "do", "dq", "dk", "dv"):
            setattr(p, name + "_strides", s3)
        p.cu_seqlens_q = p.cu_seqlens_k = cu.data_ptr()
        p.total_q = p.total_k = total
        p.stream = torch.cuda.current_stream().cuda_stream
        if key == "default":
            p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel() * 4
        assert fn(ctypes.byref(p)) == 0, lib.sigattn_last_error()
        outs[key] = o
    torch.cuda.synchronize()
    assert lib.sigattn_device_status(0) == 0
    for a, b in zip(outs["static"], outs["default"]):
        rel = ((a.float() - b.float()).norm() / (b.float().norm() + 1e-30)).item()
        assert torch.isfinite(a).all() and rel <= 1e-2


def test_oversized_problem_is_rejected_with_a_clear_error():
    lib = _cabi.load()
    x = torch.zeros(1, 128, 1, 64, device="cuda", dtype=torch.float16)
    p = _params(x, x, x, x, x, x, x, False)
    p.B, p.Tq, p.Tk, p.H = 8, 8192, 8192, 32  # 8*8192*32*64 elements > the built-in limit; nothing is launched
    rc = lib.sigattn_bwd_static_scratch(ctypes.byref(p))
    assert rc < 0
    msg = lib.sigattn_last_error()
    assert b"too large for the built-in scratch" in msg and str(_cabi.SIGATTN_STATIC_SCRATCH_ELEMS).encode() in msg
