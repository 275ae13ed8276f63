"""Calls the C ABI directly with raw device pointers (no torch ops in between) and checks the
results, the error reporting on a GPU box, and the event hooks."""

import ctypes
import math

import pytest
import torch

from oracle import sigattn_oracle as orc
from triton_sigmoid_b200 import _cabi
from triton_sigmoid_b200.profiling import time_main_kernel

pytestmark = pytest.mark.gpu


def _s3(t):
    return (ctypes.c_int64 * 3)(*t.stride()[:3])


def test_raw_forward_and_backward_calls():
    lib = _cabi.load()
    torch.manual_seed(1)
    B, T, H, D = 2, 200, 3, 128
    q, k, v, do = [torch.randn(B, T, H, D, device="cuda", dtype=torch.float16) * 0.5 for _ in range(4)]
    o, dq, dk, dv = [torch.full_like(q, float("nan")) for _ in range(4)]
    ws = torch.empty(lib.sigattn_bwd_workspace_bytes(B, T, H, D) // 4, dtype=torch.float32, device="cuda")
    p = _cabi.SigAttnParams()
    p.struct_bytes = ctypes.sizeof(p)
    p.dtype, p.B, p.H, p.D, p.Tq, p.Tk = _cabi.SIGATTN_FP16, B, H, D, T, T
    p.flags = _cabi.SIGATTN_CAUSAL
    p.scale = 1.0 / math.sqrt(D)
    p.bias_scalar = -math.log(T)  # bias pointer left NULL: scalar bias for every batch
    p.device = 0
    p.q, p.k, p.v, p.o, p.dout = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr()
    p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    for name in ("q", "k", "v", "o", "do", "dq", "dk", "dv"):
        setattr(p, name + "_strides", _s3(q))
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel() * 4
    p.stream = torch.cuda.current_stream().cuda_stream
    assert lib.sigattn_fwd(ctypes.byref(p)) == 0, lib.sigattn_last_error()
    assert lib.sigattn_bwd(ctypes.byref(p)) == 0, lib.sigattn_last_error()
    assert lib.sigattn_device_status(0) == 0
    ref_o = orc.sigattn_forward(q, k, v, is_causal=True)
    ref = orc.sigattn_backward(q, k, v, do, is_causal=True)
    assert (o.float().cpu() - ref_o).abs().max().item() <= 2e-3
    for g, r in zip((dq, dk, dv), ref):
        assert ((g.float().cpu() - r).norm() / r.norm()).item() <= 1e-2
    # the split backward (streaming kernels): no workspace, against the oracle, and run-to-run deterministic
    p.workspace, p.workspace_bytes = None, 0
    p.flags |= _cabi.SIGATTN_BWD_SPLIT
    runs = []
    for _ in range(2):
        outs = [torch.full_like(q, float("nan")) for _ in range(3)]
        p.dq, p.dk, p.dv = [t.data_ptr() for t in outs]
        assert lib.sigattn_bwd(ctypes.byref(p)) == 0, lib.sigattn_last_error()
        runs.append(outs)
    assert lib.sigattn_device_status(0) == 0
    for g, r in zip(runs[0], ref):
        assert ((g.float().cpu() - r).norm() / r.norm()).item() <= 1e-2
    for a, b in zip(*runs):
        assert torch.equal(a, b)


def test_workspace_too_small_is_reported():
    lib = _cabi.load()
    q = torch.zeros(1, 128, 1, 64, device="cuda", dtype=torch.float16)
    p = _cabi.SigAttnParams()
    p.struct_bytes = ctypes.sizeof(p)
    p.dtype, p.B, p.H, p.D, p.Tq, p.Tk = 0, 1, 1, 64, 128, 128
    p.scale = 0.125
    p.q = p.k = p.v = p.dout = p.dq = p.dk = p.dv = q.data_ptr()
    for name in ("q", "k", "v", "do", "dq", "dk", "dv"):
        setattr(p, name + "_strides", _s3(q))
    p.workspace, p.workspace_bytes = q.data_ptr(), 64
    assert lib.sigattn_bwd(ctypes.byref(p)) < 0
    assert b"workspace too small" in lib.sigattn_last_error()


def test_misaligned_pointer_is_reported():
    lib = _cabi.load()
    q = torch.zeros(1, 128, 1, 64 + 8, device="cuda", dtype=torch.float16)
    p = _cabi.SigAttnParams()
    p.struct_bytes = ctypes.sizeof(p)
    p.dtype, p.B, p.H, p.D, p.Tq, p.Tk = 0, 1, 1, 64, 128, 128
    p.q = q.data_ptr() + 2
    p.k = p.v = p.o = q.data_ptr()
    for name in ("q", "k", "v", "o"):
        setattr(p, name + "_strides", _s3(q))
    assert lib.sigattn_fwd(ctypes.byref(p)) < 0
    assert b"16-byte aligned" in lib.sigattn_last_error()


def test_event_hooks_time_the_main_kernel():
    q, k, v, do = [torch.randn(2, 1024, 4, 64, device="cuda", dtype=torch.bfloat16) for _ in range(4)]
    for direction in ("fwd", "bwd"):
        ms = time_main_kernel(direction, q, k, v, do, iters=3)
        assert len(ms) == 3 and all(0 < x < 100 for x in ms)


def test_forward_launch_replays_from_a_cuda_graph():
    """A forward call recorded into a stream capture (after a first, ordinary call on the device) replays
    with the same result; launches made under capture draw their work-item counters from a pool of their own."""
    lib = _cabi.load()
    torch.manual_seed(3)
    B, T, H, D = 2, 384, 2, 64
    q, k, v = [torch.randn(B, T, H, D, device="cuda", dtype=torch.bfloat16) * 0.5 for _ in range(3)]
    eager = torch.empty_like(q)
    replayed = torch.full_like(q, float("nan"))

    def params(o, stream):
        p = _cabi.SigAttnParams()
        p.struct_bytes = ctypes.sizeof(p)
        p.dtype, p.B, p.H, p.D, p.Tq, p.Tk = _cabi.SIGATTN_BF16, B, H, D, T, T
        p.flags = _cabi.SIGATTN_CAUSAL
        p.scale, p.bias_scalar, p.device = 1.0 / math.sqrt(D), -math.log(T), 0
        p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
        for name in ("q", "k", "v", "o"):
            setattr(p, name + "_strides", _s3(q))
        p.stream = stream
        return p

    p0 = params(eager, torch.cuda.current_stream().cuda_stream)
    assert lib.sigattn_fwd(ctypes.byref(p0)) == 0, lib.sigattn_last_error()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.graph(graph, stream=side):
        p1 = params(replayed, torch.cuda.current_stream().cuda_stream)
        assert lib.sigattn_fwd(ctypes.byref(p1)) == 0, lib.sigattn_last_error()
    for _ in range(3):
        replayed.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(replayed, eager)
    assert lib.sigattn_device_status(0) == 0
