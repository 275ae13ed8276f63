"""Times the main attention kernel of a forward or backward call alone, using the optional
event pair of the C ABI (``ev_main_start`` / ``ev_main_stop`` in ``include/sigattn_b200.h``)."""

from __future__ import annotations

import ctypes
import math
from typing import List, Optional

import torch

from . import _cabi
from .ops import _base_params, _check_kernel_inputs, _prep_aux, _strides3


def _event() -> torch.cuda.Event:
    e = torch.cuda.Event(enable_timing=True)
    e.record()  # creates the underlying cudaEvent_t
    return e


def time_main_kernel(direction: str, q, k, v, dout=None, seq_lens_q=None, seq_lens_k=None, bias=None, scale=None,
                     is_causal=False, iters: int = 10, flush: Optional[torch.Tensor] = None, split_bwd: bool = False) -> List[float]:
    """Milliseconds of the main kernel(s) of `iters` calls of sigattn_fwd ("fwd") or sigattn_bwd
    ("bwd": the fused kernel alone, or the two streaming kernels when `split_bwd`).  If `flush` is given it
    is zero-filled between calls (L2 flush)."""
    _check_kernel_inputs(q, k, v)
    B, Tq, H, D = q.shape
    Tk = k.shape[1]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if bias is None:
        bias = torch.full((B,), -math.log(float(Tk)), dtype=torch.float32, device=q.device)
    bias, _, seq_lens_q, seq_lens_k = _prep_aux(q, bias, None, seq_lens_q, seq_lens_k)
    lib = _cabi.load()
    p = _base_params(q, k, v, bias, None, seq_lens_q, seq_lens_k, scale, is_causal)
    keep = []
    if direction == "fwd":
        out = torch.empty_like(q)
        p.o, p.o_strides = out.data_ptr(), _strides3(out)
        call = lib.sigattn_fwd
        keep.append(out)
    elif direction == "bwd":
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        p.dout, p.do_strides = dout.data_ptr(), _strides3(dout)
        p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
        p.dq_strides, p.dk_strides, p.dv_strides = _strides3(dq), _strides3(dk), _strides3(dv)
        keep += [dq, dk, dv]
        if split_bwd:
            p.flags |= _cabi.SIGATTN_BWD_SPLIT
        else:
            ws = torch.empty(max(lib.sigattn_bwd_workspace_bytes(B, Tq, H, D), 16) // 4, dtype=torch.float32,
                             device=q.device)
            p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel() * 4
            keep.append(ws)
        call = lib.sigattn_bwd
    else:
        raise ValueError("direction must be 'fwd' or 'bwd'")
    pairs = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = _event(), _event()
        p.ev_main_start, p.ev_main_stop = e0.cuda_event, e1.cuda_event
        _cabi.check(call(ctypes.byref(p)), f"sigattn_{direction}")
        pairs.append((e0, e1))
    torch.cuda.synchronize(q.device)
    return [a.elapsed_time(b) for a, b in pairs]


def _main() -> None:
    """``python -m triton_sigmoid_b200.profiling B N H D fp16|bf16|fp32 [causal]``: one forward and one
    backward of that shape through the public API (seed 0), for a profiler to capture."""
    import sys

    from .ops import sigmoid_attention

    B, N, H, D = (int(x) for x in sys.argv[1:5])
    dtype = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}[sys.argv[5] if len(sys.argv) > 5 else "fp16"]
    causal = len(sys.argv) > 6 and sys.argv[6] == "causal"
    torch.manual_seed(0)
    q, k, v, do = (torch.randn(B, N, H, D, device="cuda", dtype=dtype) for _ in range(4))
    for t in (q, k, v):
        t.requires_grad_()
    out = sigmoid_attention(q, k, v, is_causal=causal)
    out.backward(do)
    torch.cuda.synchronize()
    print("ok", float(out.detach().float().abs().mean()), float(q.grad.float().abs().mean()))


if __name__ == "__main__":
    _main()
