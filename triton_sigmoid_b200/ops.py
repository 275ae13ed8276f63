"""torch.library custom ops around the C ABI, and the public functions.

Mirrors the reference's operator layer: four ops (dense / padded, forward / backward) with
``register_fake`` and ``register_autograd`` so eager autograd and ``torch.compile`` both work
(reference: ``src/triton_sigmoid/sigmoid_triton_dense.py:475-753`` and
``src/triton_sigmoid/sigmoid_triton_padded.py:517-846``), and the two public wrappers with
the reference's signatures, defaults, validation and error texts
(``sigmoid_triton_dense.py:761-853``, ``sigmoid_triton_padded.py:853-1010``).

All arithmetic happens in the CUDA library; nothing here computes attention.
"""

from __future__ import annotations

import contextlib
import ctypes
import math
import os
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _cabi

_NS = "sigattn_b200"
_SUPPORTED_DTYPES = (torch.float16, torch.bfloat16, torch.float32)
_DTYPE_CODE = {torch.float16: _cabi.SIGATTN_FP16, torch.bfloat16: _cabi.SIGATTN_BF16, torch.float32: _cabi.SIGATTN_FP32}
_DEVICE_OK: dict = {}


def _require_b200(dev: torch.device) -> None:
    """The kernels are built for sm_100a only (code that is not forward compatible, not even with
    other 10.x parts); anything else is an error, never a fallback."""
    if dev.type != "cuda":
        raise RuntimeError(f"triton_sigmoid_b200 runs on CUDA tensors only, got device '{dev}'")
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    ok = _DEVICE_OK.get(idx)
    if ok is None:
        major, minor = torch.cuda.get_device_capability(idx)
        ok = _DEVICE_OK[idx] = (major, minor) == (10, 0)
    if not ok:
        major, minor = torch.cuda.get_device_capability(idx)
        raise RuntimeError(f"triton_sigmoid_b200 requires an sm_100 GPU (B200), found sm_{major}{minor}")


# ----------------------------------------------------------------------------- run-time switches
_TRUE = ("1", "true", "yes", "on")
_accurate_override: Optional[bool] = None


def _accurate() -> bool:
    """Accurate-sigmoid mode: the reference's ``TRITON_SIGMOID_ACCURATE`` environment switch (same
    accepted values, ``src/triton_sigmoid/kernel_utils.py:190-193``), read when an op runs rather than at
    import, unless :func:`accurate_sigmoid` overrides it."""
    if _accurate_override is not None:
        return _accurate_override
    return os.environ.get("TRITON_SIGMOID_ACCURATE", "").lower() in _TRUE


@contextlib.contextmanager
def accurate_sigmoid(enabled: Optional[bool] = True):
    """Within the block, run the tensor-core kernels with the accurate sigmoid (``True``), the default fast
    one (``False``), or whatever the environment says (``None``)."""
    global _accurate_override
    prev, _accurate_override = _accurate_override, enabled
    try:
        yield
    finally:
        _accurate_override = prev


def _debug_sync() -> bool:
    """``SIGATTN_B200_DEBUG=1``: synchronise after every launch and raise at once if a kernel gave up on a
    bounded wait (outputs are poison-filled beforehand so that unwritten rows show)."""
    return os.environ.get("SIGATTN_B200_DEBUG", "").lower() in _TRUE


def device_status(device=None) -> int:
    """Synchronise `device` and return its health word: 0, or the code of the bounded wait a kernel of this
    library gave up on since the last call (reading a failure clears it, after which the library is usable
    again; results of launches made in between are undefined)."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    rc = _cabi.load().sigattn_device_status(idx if idx is not None else torch.cuda.current_device())
    if rc < 0:
        raise RuntimeError(f"sigattn_device_status failed (code {rc}): {_cabi.last_error()}")
    return rc


def _bwd_split() -> bool:
    """``SIGATTN_B200_BWD_SPLIT=1`` selects the pair of streaming backward kernels (7 GEMMs per tile pair, no
    workspace, no atomics, run-to-run deterministic gradients) instead of the default fused kernel (5 GEMMs,
    dQ accumulated with fp32 reductions into a workspace), which was measured faster."""
    return os.environ.get("SIGATTN_B200_BWD_SPLIT", "").lower() in _TRUE


def _flags(is_causal: bool) -> int:
    return (_cabi.SIGATTN_CAUSAL if is_causal else 0) | (_cabi.SIGATTN_ACCURATE if _accurate() else 0)


def _bwd_workspace(p, lib, B, Tq, H, D, device):
    """The fused backward's fp32 dQ accumulator; the split backward needs none (and gets its flag here)."""
    if _bwd_split():
        p.flags |= _cabi.SIGATTN_BWD_SPLIT
        return None
    ws_bytes = lib.sigattn_bwd_workspace_bytes(B, Tq, H, D)
    ws = torch.empty(max(ws_bytes, 16) // 4, dtype=torch.float32, device=device)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel() * 4
    return ws


def _launch(fn, p, what: str, outputs) -> None:
    """One C-ABI call.  A kernel that gave up on a wait earlier makes the call itself fail (the library
    keeps a host-visible copy of the health word), which surfaces here as RuntimeError; in debug mode the
    device is synchronised and checked after the launch as well."""
    debug = _debug_sync()
    if debug:
        for t in outputs:
            t.fill_(float("nan"))
    _cabi.check(fn(ctypes.byref(p)), what)
    if debug:
        code = device_status(torch.device("cuda", p.device))
        if code != 0:
            raise RuntimeError(f"{what}: a kernel gave up on a bounded wait (site 0x{code:x}); its outputs are "
                               "undefined.  The health word has been cleared, the library is usable again.")


def _strides3(t: torch.Tensor):
    sb, st, sh, sd = t.stride()
    assert sd == 1
    return (ctypes.c_int64 * 3)(sb, st, sh)


def _base_params(q, k, v, bias, score_mod, seq_lens_q, seq_lens_k, scale, is_causal) -> _cabi.SigAttnParams:
    B, Tq, H, D = q.shape
    p = _cabi.SigAttnParams()
    p.struct_bytes = ctypes.sizeof(_cabi.SigAttnParams)
    p.dtype = _DTYPE_CODE[q.dtype]
    p.B, p.H, p.D, p.Tq, p.Tk = B, H, D, Tq, k.shape[1]
    p.flags = _flags(is_causal)
    p.scale = float(scale)
    p.device = q.device.index if q.device.index is not None else torch.cuda.current_device()
    p.q, p.k, p.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    p.q_strides, p.k_strides, p.v_strides = _strides3(q), _strides3(k), _strides3(v)
    p.seq_lens_q = seq_lens_q.data_ptr() if seq_lens_q is not None else None
    p.seq_lens_k = seq_lens_k.data_ptr() if seq_lens_k is not None else None
    if isinstance(bias, torch.Tensor):  # one value per batch element
        p.bias, p.bias_scalar = bias.data_ptr(), 0.0
    elif bias is None:                  # the padded default, -log(valid keys), computed by the kernels
        p.bias, p.bias_scalar = None, 0.0
        p.flags |= _cabi.SIGATTN_BIAS_NEG_LOG_LK
    else:                               # one value for the whole call: no device tensor needed
        p.bias, p.bias_scalar = None, float(bias)
    p.score_mod = score_mod.data_ptr() if score_mod is not None else None
    p.stream = torch.cuda.current_stream(q.device).cuda_stream
    return p


def _prep_aux(q, bias, score_mod, seq_lens_q, seq_lens_k):
    if isinstance(bias, torch.Tensor):
        bias = bias.to(device=q.device, dtype=torch.float32).contiguous()
    if score_mod is not None:
        score_mod = score_mod.to(device=q.device, dtype=torch.float32).contiguous()
    if seq_lens_q is not None:
        seq_lens_q = seq_lens_q.to(device=q.device, dtype=torch.int32).contiguous()
    if seq_lens_k is not None:
        seq_lens_k = seq_lens_k.to(device=q.device, dtype=torch.int32).contiguous()
    return bias, score_mod, seq_lens_q, seq_lens_k


def _check_kernel_inputs(q, k, v):
    _require_b200(q.device)
    if q.dtype not in _SUPPORTED_DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise NotImplementedError(
            f"triton_sigmoid_b200 kernels take float16, bfloat16 or float32 q/k/v of one dtype, got "
            f"{q.dtype}, {k.dtype}, {v.dtype}"
        )
    if q.shape[-1] not in (64, 128):
        raise NotImplementedError(f"kernel head dimension must be 64 or 128, got {q.shape[-1]}")


def _run_fwd(q, k, v, bias, score_mod, seq_lens_q, seq_lens_k, scale, is_causal) -> torch.Tensor:
    _check_kernel_inputs(q, k, v)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    out = torch.empty_like(q)
    if out.numel() == 0:
        return out
    bias, score_mod, seq_lens_q, seq_lens_k = _prep_aux(q, bias, score_mod, seq_lens_q, seq_lens_k)
    p = _base_params(q, k, v, bias, score_mod, seq_lens_q, seq_lens_k, scale, is_causal)
    p.o = out.data_ptr()
    p.o_strides = _strides3(out)
    _launch(_cabi.load().sigattn_fwd, p, "sigattn_fwd", (out,))
    return out


def _run_bwd(q, k, v, do, bias, score_mod, seq_lens_q, seq_lens_k, scale, is_causal):
    _check_kernel_inputs(q, k, v)
    q, k, v, do = q.contiguous(), k.contiguous(), v.contiguous(), do.contiguous()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    if q.numel() == 0 and k.numel() == 0:
        return dq, dk, dv
    bias, score_mod, seq_lens_q, seq_lens_k = _prep_aux(q, bias, score_mod, seq_lens_q, seq_lens_k)
    lib = _cabi.load()
    B, Tq, H, D = q.shape
    p = _base_params(q, k, v, bias, score_mod, seq_lens_q, seq_lens_k, scale, is_causal)
    p.dout = do.data_ptr()
    p.do_strides = _strides3(do)
    p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    p.dq_strides, p.dk_strides, p.dv_strides = _strides3(dq), _strides3(dk), _strides3(dv)
    ws = _bwd_workspace(p, lib, B, Tq, H, D, q.device)  # noqa: F841  (kept alive until the launch is queued)
    _launch(lib.sigattn_bwd, p, "sigattn_bwd", (dq, dk, dv))
    return dq, dk, dv


# ----------------------------------------------------------------------------- dense ops
@torch.library.custom_op(f"{_NS}::sigmoid_attention_fwd", mutates_args=())
def sigmoid_attention_fwd_op(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, bias: torch.Tensor,
                             score_mod: Optional[torch.Tensor], sm_scale: float, is_causal: bool) -> torch.Tensor:
    return _run_fwd(Q, K, V, bias, score_mod, None, None, sm_scale, is_causal)


@sigmoid_attention_fwd_op.register_fake
def _(Q, K, V, bias, score_mod, sm_scale, is_causal):
    return torch.empty_like(Q, memory_format=torch.contiguous_format)


@torch.library.custom_op(f"{_NS}::sigmoid_attention_bwd", mutates_args=())
def sigmoid_attention_bwd_op(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, dO: torch.Tensor,
                             bias: torch.Tensor, score_mod: Optional[torch.Tensor], sm_scale: float,
                             is_causal: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return _run_bwd(Q, K, V, dO, bias, score_mod, None, None, sm_scale, is_causal)


@sigmoid_attention_bwd_op.register_fake
def _(Q, K, V, dO, bias, score_mod, sm_scale, is_causal):
    c = torch.contiguous_format
    return (torch.empty_like(Q, memory_format=c), torch.empty_like(K, memory_format=c),
            torch.empty_like(V, memory_format=c))


def _dense_setup_context(ctx, inputs, output):
    Q, K, V, bias, score_mod, sm_scale, is_causal = inputs
    ctx.save_for_backward(Q, K, V, bias, score_mod)
    ctx.sm_scale = sm_scale
    ctx.is_causal = is_causal


def _dense_backward(ctx, dO):
    Q, K, V, bias, score_mod = ctx.saved_tensors
    dQ, dK, dV = sigmoid_attention_bwd_op(Q, K, V, dO, bias, score_mod, ctx.sm_scale, ctx.is_causal)
    return dQ, dK, dV, None, None, None, None


sigmoid_attention_fwd_op.register_autograd(_dense_backward, setup_context=_dense_setup_context)


# ----------------------------------------------------------------------------- padded ops
@torch.library.custom_op(f"{_NS}::sigmoid_attn_padded_fwd", mutates_args=())
def sigmoid_attn_padded_fwd_op(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, seq_lens_k: torch.Tensor,
                               seq_lens_q: torch.Tensor, bias: torch.Tensor, score_mod: Optional[torch.Tensor],
                               sm_scale: float, is_causal: bool) -> torch.Tensor:
    return _run_fwd(Q, K, V, bias, score_mod, seq_lens_q, seq_lens_k, sm_scale, is_causal)


@sigmoid_attn_padded_fwd_op.register_fake
def _(Q, K, V, seq_lens_k, seq_lens_q, bias, score_mod, sm_scale, is_causal):
    return torch.empty_like(Q, memory_format=torch.contiguous_format)


@torch.library.custom_op(f"{_NS}::sigmoid_attn_padded_bwd", mutates_args=())
def sigmoid_attn_padded_bwd_op(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, dO: torch.Tensor,
                               seq_lens_k: torch.Tensor, seq_lens_q: torch.Tensor, bias: torch.Tensor,
                               score_mod: Optional[torch.Tensor], sm_scale: float,
                               is_causal: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return _run_bwd(Q, K, V, dO, bias, score_mod, seq_lens_q, seq_lens_k, sm_scale, is_causal)


@sigmoid_attn_padded_bwd_op.register_fake
def _(Q, K, V, dO, seq_lens_k, seq_lens_q, bias, score_mod, sm_scale, is_causal):
    c = torch.contiguous_format
    return (torch.empty_like(Q, memory_format=c), torch.empty_like(K, memory_format=c),
            torch.empty_like(V, memory_format=c))


def _padded_setup_context(ctx, inputs, output):
    Q, K, V, seq_lens_k, seq_lens_q, bias, score_mod, sm_scale, is_causal = inputs
    ctx.save_for_backward(Q, K, V, seq_lens_k, seq_lens_q, bias, score_mod)
    ctx.sm_scale = sm_scale
    ctx.is_causal = is_causal


def _padded_backward(ctx, dO):
    Q, K, V, seq_lens_k, seq_lens_q, bias, score_mod = ctx.saved_tensors
    dQ, dK, dV = sigmoid_attn_padded_bwd_op(Q, K, V, dO, seq_lens_k, seq_lens_q, bias, score_mod, ctx.sm_scale,
                                            ctx.is_causal)
    return dQ, dK, dV, None, None, None, None, None, None


sigmoid_attn_padded_fwd_op.register_autograd(_padded_backward, setup_context=_padded_setup_context)


# ----------------------------------------------------------------------------- eager shortcut
class _EagerSigmoidAttention(torch.autograd.Function):
    """What the dense and padded ops do, minus the dispatcher: in eager mode the public functions call the
    library through this plain autograd function, because a `torch.library.custom_op` round trip with its
    generated autograd wrapper costs about 100 us of host time per forward + backward pair, which is more
    than the kernels of a short-sequence call take.  Under `torch.compile` the public functions use the
    registered ops (fake kernels, autograd registration) instead.  `bias` is a [B] tensor, a Python float
    (one value for the whole call, passed by value) or None (minus the logarithm of each batch element's
    number of valid keys, computed by the kernels)."""

    @staticmethod
    def forward(ctx, q, k, v, bias, score_mod, seq_lens_q, seq_lens_k, scale, is_causal):
        bias_t = bias if isinstance(bias, torch.Tensor) else None
        ctx.save_for_backward(q, k, v, bias_t, score_mod, seq_lens_q, seq_lens_k)
        ctx.bias_value = None if bias_t is not None else bias
        ctx.scale, ctx.is_causal = scale, is_causal
        return _run_fwd(q, k, v, bias, score_mod, seq_lens_q, seq_lens_k, scale, is_causal)

    @staticmethod
    def backward(ctx, dO):
        q, k, v, bias_t, score_mod, seq_lens_q, seq_lens_k = ctx.saved_tensors
        bias = bias_t if bias_t is not None else ctx.bias_value
        dq, dk, dv = _run_bwd(q, k, v, dO, bias, score_mod, seq_lens_q, seq_lens_k, ctx.scale, ctx.is_causal)
        return dq, dk, dv, None, None, None, None, None, None


def _eager_attention(q, k, v, bias, score_mod, seq_lens_q, seq_lens_k, scale, is_causal):
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        return _EagerSigmoidAttention.apply(q, k, v, bias, score_mod, seq_lens_q, seq_lens_k, scale, is_causal)
    return _run_fwd(q, k, v, bias, score_mod, seq_lens_q, seq_lens_k, scale, is_causal)


# ----------------------------------------------------------------------------- packed (variable-length) ops
def _varlen_params(q, k, v, cu_q, cu_k, max_q, max_k, bias, score_mod, scale, is_causal) -> _cabi.SigAttnParams:
    """Parameters of a call on packed (total, H, D) tensors: B = number of sequences, Tq / Tk = the
    longest sequence, lengths and row offsets from the cumulative-length arrays."""
    total_q, H, D = q.shape
    p = _cabi.SigAttnParams()
    p.struct_bytes = ctypes.sizeof(_cabi.SigAttnParams)
    p.dtype = _DTYPE_CODE[q.dtype]
    p.B, p.H, p.D, p.Tq, p.Tk = cu_q.numel() - 1, H, D, int(max_q), int(max_k)
    p.flags = _flags(is_causal)
    p.scale = float(scale)
    p.bias_scalar = 0.0
    p.device = q.device.index if q.device.index is not None else torch.cuda.current_device()
    p.q, p.k, p.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    s3 = lambda t: (ctypes.c_int64 * 3)(0, t.stride(0), t.stride(1))
    p.q_strides, p.k_strides, p.v_strides = s3(q), s3(k), s3(v)
    p.cu_seqlens_q, p.cu_seqlens_k = cu_q.data_ptr(), cu_k.data_ptr()
    p.total_q, p.total_k = total_q, k.shape[0]
    if isinstance(bias, torch.Tensor):
        p.bias = bias.data_ptr()
    elif bias is None:  # -log(number of keys of the sequence), computed by the kernels
        p.bias = None
        p.flags |= _cabi.SIGATTN_BIAS_NEG_LOG_LK
    else:
        p.bias, p.bias_scalar = None, float(bias)
    p.score_mod = score_mod.data_ptr() if score_mod is not None else None
    p.stream = torch.cuda.current_stream(q.device).cuda_stream
    return p


def _check_varlen_kernel_inputs(q, k, v):
    _require_b200(q.device)
    if q.dtype not in _SUPPORTED_DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise NotImplementedError(f"packed sequences take float16, bfloat16 or float32 q/k/v of one dtype, got "
                                  f"{q.dtype}, {k.dtype}, {v.dtype}")
    if q.shape[-1] not in (64, 128):
        raise NotImplementedError(f"kernel head dimension must be 64 or 128, got {q.shape[-1]}")


@torch.library.custom_op(f"{_NS}::sigmoid_attn_varlen_fwd", mutates_args=())
def sigmoid_attn_varlen_fwd_op(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, cu_seqlens_q: torch.Tensor,
                               cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int, bias: torch.Tensor,
                               score_mod: Optional[torch.Tensor], sm_scale: float, is_causal: bool) -> torch.Tensor:
    return _run_varlen_fwd(Q, K, V, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, bias, score_mod, sm_scale,
                           is_causal)


def _run_varlen_fwd(Q, K, V, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, bias, score_mod, sm_scale, is_causal):
    _check_varlen_kernel_inputs(Q, K, V)
    Q, K, V = Q.contiguous(), K.contiguous(), V.contiguous()
    # only rows of the sequences are written: rows between or behind them, and rows of a sequence beyond
    # max_seqlen_q, stay zero (as in the backward)
    out = torch.zeros_like(Q)
    if out.numel() == 0:
        return out
    bias, score_mod, _, _ = _prep_aux(Q, bias, score_mod, None, None)
    p = _varlen_params(Q, K, V, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, bias, score_mod, sm_scale,
                       is_causal)
    p.o = out.data_ptr()
    p.o_strides = (ctypes.c_int64 * 3)(0, out.stride(0), out.stride(1))
    _cabi.check(_cabi.load().sigattn_fwd(ctypes.byref(p)), "sigattn_fwd")
    if _debug_sync() and device_status(Q.device) != 0:
        raise RuntimeError("sigattn_fwd: a kernel gave up on a bounded wait; its outputs are undefined")
    return out


@sigmoid_attn_varlen_fwd_op.register_fake
def _(Q, K, V, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, bias, score_mod, sm_scale, is_causal):
    return torch.empty_like(Q, memory_format=torch.contiguous_format)


@torch.library.custom_op(f"{_NS}::sigmoid_attn_varlen_bwd", mutates_args=())
def sigmoid_attn_varlen_bwd_op(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, dO: torch.Tensor,
                               cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor, max_seqlen_q: int,
                               max_seqlen_k: int, bias: torch.Tensor, score_mod: Optional[torch.Tensor],
                               sm_scale: float, is_causal: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return _run_varlen_bwd(Q, K, V, dO, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, bias, score_mod, sm_scale,
                           is_causal)


def _run_varlen_bwd(Q, K, V, dO, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, bias, score_mod, sm_scale,
                    is_causal):
    _check_varlen_kernel_inputs(Q, K, V)
    Q, K, V, dO = Q.contiguous(), K.contiguous(), V.contiguous(), dO.contiguous()
    # rows between or behind the sequences (there are none when cu_seqlens covers the tensors) stay zero
    dq, dk, dv = torch.zeros_like(Q), torch.zeros_like(K), torch.zeros_like(V)
    if Q.numel() == 0 or K.numel() == 0:
        return dq, dk, dv
    bias, score_mod, _, _ = _prep_aux(Q, bias, score_mod, None, None)
    lib = _cabi.load()
    total_q, H, D = Q.shape
    p = _varlen_params(Q, K, V, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, bias, score_mod, sm_scale,
                       is_causal)
    s3 = lambda t: (ctypes.c_int64 * 3)(0, t.stride(0), t.stride(1))
    p.dout, p.do_strides = dO.data_ptr(), s3(dO)
    p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    p.dq_strides, p.dk_strides, p.dv_strides = s3(dq), s3(dk), s3(dv)
    ws = _bwd_workspace(p, lib, 1, total_q, H, D, Q.device)  # noqa: F841
    _cabi.check(lib.sigattn_bwd(ctypes.byref(p)), "sigattn_bwd")
    if _debug_sync() and device_status(Q.device) != 0:
        raise RuntimeError("sigattn_bwd: a kernel gave up on a bounded wait; its outputs are undefined")
    return dq, dk, dv


@sigmoid_attn_varlen_bwd_op.register_fake
def _(Q, K, V, dO, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, bias, score_mod, sm_scale, is_causal):
    c = torch.contiguous_format
    return (torch.empty_like(Q, memory_format=c), torch.empty_like(K, memory_format=c),
            torch.empty_like(V, memory_format=c))


def _varlen_setup_context(ctx, inputs, output):
    Q, K, V, cu_q, cu_k, max_q, max_k, bias, score_mod, sm_scale, is_causal = inputs
    ctx.save_for_backward(Q, K, V, cu_q, cu_k, bias, score_mod)
    ctx.max_q, ctx.max_k = max_q, max_k
    ctx.sm_scale = sm_scale
    ctx.is_causal = is_causal


def _varlen_backward(ctx, dO):
    Q, K, V, cu_q, cu_k, bias, score_mod = ctx.saved_tensors
    dQ, dK, dV = sigmoid_attn_varlen_bwd_op(Q, K, V, dO, cu_q, cu_k, ctx.max_q, ctx.max_k, bias, score_mod,
                                            ctx.sm_scale, ctx.is_causal)
    return dQ, dK, dV, None, None, None, None, None, None, None, None


sigmoid_attn_varlen_fwd_op.register_autograd(_varlen_backward, setup_context=_varlen_setup_context)


class _EagerSigmoidAttentionVarlen(torch.autograd.Function):
    """The packed entry point's counterpart of :class:`_EagerSigmoidAttention` (same reasons, same `bias` forms)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, max_q, max_k, bias, score_mod, scale, is_causal):
        bias_t = bias if isinstance(bias, torch.Tensor) else None
        ctx.save_for_backward(q, k, v, cu_q, cu_k, bias_t, score_mod)
        ctx.bias_value = None if bias_t is not None else bias
        ctx.max_q, ctx.max_k, ctx.scale, ctx.is_causal = max_q, max_k, scale, is_causal
        return _run_varlen_fwd(q, k, v, cu_q, cu_k, max_q, max_k, bias, score_mod, scale, is_causal)

    @staticmethod
    def backward(ctx, dO):
        q, k, v, cu_q, cu_k, bias_t, score_mod = ctx.saved_tensors
        bias = bias_t if bias_t is not None else ctx.bias_value
        dq, dk, dv = _run_varlen_bwd(q, k, v, dO, cu_q, cu_k, ctx.max_q, ctx.max_k, bias, score_mod, ctx.scale,
                                     ctx.is_causal)
        return dq, dk, dv, None, None, None, None, None, None, None, None


# ----------------------------------------------------------------------------- public API
def _validate_qkv(query, key, value):
    if query.dim() != 4 or key.dim() != 4 or value.dim() != 4:
        raise ValueError("Expected query, key, and value to be 4D tensors")
    B, T_q, H, D = query.shape
    B_k, T_k, H_k, D_k = key.shape
    B_v, T_v, H_v, D_v = value.shape
    if B != B_k or B != B_v:
        raise ValueError(f"Batch size mismatch: Q={B}, K={B_k}, V={B_v}")
    if H != H_k or H != H_v:
        raise ValueError(f"Number of heads mismatch: Q={H}, K={H_k}, V={H_v}")
    if D != D_k or D != D_v:
        raise ValueError(f"Head dimension mismatch: Q={D}, K={D_k}, V={D_v}")
    return B, T_q, T_k, T_v, H, D


def _kernel_head_dim(D: int) -> int:
    if D <= 64:
        return 64
    if D <= 128:
        return 128
    raise NotImplementedError(f"head dimension {D} is larger than the 128 the kernels support")


def _pad_head_dim(x: torch.Tensor, D_kernel: int) -> torch.Tensor:
    """Zero-extend the head dimension (zeros add nothing to Q.K and only yield extra output
    columns, which the caller slices away again)."""
    D = x.shape[-1]
    return x if D == D_kernel else F.pad(x, (0, D_kernel - D))


def _check_dtype(query, key, value):
    """float16 / bfloat16 run on the tensor cores; float32 runs the exact single-precision
    kernels (slower by design: the reference holds float32 to 1e-5, which tf32 cannot meet)."""
    if query.dtype not in _SUPPORTED_DTYPES:
        raise NotImplementedError(f"unsupported dtype {query.dtype}: use float16, bfloat16 or float32")
    if key.dtype != query.dtype or value.dtype != query.dtype:
        raise ValueError(f"query, key and value must share one dtype, got {query.dtype}, {key.dtype}, {value.dtype}")


def sigmoid_attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    is_causal: bool = False,
    scale: Optional[float] = None,
    sigmoid_bias: Optional[float] = None,
    score_mod: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Sigmoid attention for dense (same-length) sequences, differentiable in q, k, v.

    ``output = sigmoid(Q @ K^T * scale + sigmoid_bias + score_mod[key]) @ V`` on
    ``[B, T, H, D]`` tensors.  ``scale`` defaults to ``1/sqrt(D)``, ``sigmoid_bias`` to
    ``-log(T)``; ``score_mod`` is an optional ``[B, T]`` additive per-key bias without
    gradient.  Same contract as the reference's ``sigmoid_attention``
    (``sigmoid_triton_dense.py:761-853``).
    """
    B, T_q, T_k, T_v, H, D = _validate_qkv(query, key, value)
    if T_q != T_k or T_q != T_v:
        raise ValueError(f"Dense attention requires same sequence length for Q, K, V, got {T_q}, {T_k}, {T_v}")
    if score_mod is not None:
        if score_mod.shape != (B, T_k):
            raise ValueError(f"score_mod must have shape ({B}, {T_k}), got {score_mod.shape}")
        score_mod = score_mod.contiguous()
    _check_dtype(query, key, value)

    if scale is None:
        scale = 1.0 / math.sqrt(D)
    Dk = _kernel_head_dim(D)
    query, key, value = (_pad_head_dim(t, Dk).contiguous() for t in (query, key, value))

    bias_value = float(sigmoid_bias) if sigmoid_bias is not None else (-math.log(float(T_q)) if T_q > 0 else 0.0)
    if torch.compiler.is_compiling():
        for x in (query, key, value):
            torch._dynamo.mark_static(x, -2)  # heads
            torch._dynamo.mark_static(x, -1)  # head dimension
        bias = torch.full((B,), bias_value, dtype=torch.float32, device=query.device)
        out = sigmoid_attention_fwd_op(query, key, value, bias, score_mod, float(scale), bool(is_causal))
    else:
        out = _eager_attention(query, key, value, bias_value, score_mod, None, None, float(scale), bool(is_causal))
    return out if Dk == D else out[..., :D]


def sigmoid_attention_padded(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    seq_lens_k: Optional[torch.Tensor] = None,
    seq_lens_q: Optional[torch.Tensor] = None,
    is_causal: bool = False,
    scale: Optional[float] = None,
    sigmoid_bias: Optional[float] = None,
    score_mod: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Sigmoid attention for sequences with trailing padding, differentiable in q, k, v.

    ``query`` is ``[B, T_q, H, D]``, ``key`` / ``value`` are ``[B, T_k, H, D]``;
    ``seq_lens_k`` / ``seq_lens_q`` (``[B]``, integer) give the number of valid tokens per
    batch element (``None`` = all).  Output rows at or beyond ``seq_lens_q[b]`` are zero, and
    so are the matching gradient rows.  ``sigmoid_bias`` defaults to ``-log(seq_lens_k[b])``.
    Same contract as the reference's ``sigmoid_attention_padded``
    (``sigmoid_triton_padded.py:853-1010``); lengths outside ``[0, T]`` are clamped.
    """
    B, T_q, T_k, T_v, H, D = _validate_qkv(query, key, value)
    if T_k != T_v:
        raise ValueError(f"Key and value sequence lengths must match, got K={T_k}, V={T_v}")

    compiling = torch.compiler.is_compiling()
    full_k = seq_lens_k is None
    if seq_lens_k is None:
        if compiling:  # the op's schema wants tensors; the eager path passes "all valid" as a null pointer
            seq_lens_k = torch.full((B,), T_k, dtype=torch.int32, device=query.device)
    else:
        if seq_lens_k.shape != (B,):
            raise ValueError(f"seq_lens_k must have shape ({B},), got {seq_lens_k.shape}")
        if seq_lens_k.dtype != torch.int32:
            seq_lens_k = seq_lens_k.to(torch.int32)
        seq_lens_k = seq_lens_k.to(query.device).contiguous()
    if seq_lens_q is None:
        if compiling:
            seq_lens_q = torch.full((B,), T_q, dtype=torch.int32, device=query.device)
    else:
        if seq_lens_q.shape != (B,):
            raise ValueError(f"seq_lens_q must have shape ({B},), got {seq_lens_q.shape}")
        if seq_lens_q.dtype != torch.int32:
            seq_lens_q = seq_lens_q.to(torch.int32)
        seq_lens_q = seq_lens_q.to(query.device).contiguous()

    if score_mod is not None:
        if score_mod.shape != (B, T_k):
            raise ValueError(f"score_mod must have shape ({B}, {T_k}), got {score_mod.shape}")
        score_mod = score_mod.contiguous()
    _check_dtype(query, key, value)

    if scale is None:
        scale = 1.0 / math.sqrt(D)
    Dk = _kernel_head_dim(D)
    query, key, value = (_pad_head_dim(t, Dk).contiguous() for t in (query, key, value))

    if sigmoid_bias is not None:
        bias = float(sigmoid_bias)
    elif full_k:
        bias = -math.log(float(T_k)) if T_k > 0 else float("inf")
    elif compiling:
        # -log(0) = +inf for an empty key set; every probability is masked there anyway
        bias = -torch.log(seq_lens_k.clamp(min=0, max=T_k).float())
    else:
        bias = None  # the same value, computed by the kernels from the lengths they clamp anyway

    if compiling:
        for x in (query, key, value):
            torch._dynamo.mark_static(x, -2)  # heads
            torch._dynamo.mark_static(x, -1)  # head dimension
        if not isinstance(bias, torch.Tensor):
            bias = torch.full((B,), bias, dtype=torch.float32, device=query.device)
        out = sigmoid_attn_padded_fwd_op(query, key, value, seq_lens_k, seq_lens_q, bias, score_mod, float(scale),
                                         bool(is_causal))
    else:
        out = _eager_attention(query, key, value, bias, score_mod, seq_lens_q, seq_lens_k, float(scale), bool(is_causal))
    return out if Dk == D else out[..., :D]


def sigmoid_attention_varlen(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    is_causal: bool = False,
    scale: Optional[float] = None,
    sigmoid_bias: Optional[float] = None,
    score_mod: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Sigmoid attention on packed variable-length sequences, differentiable in q, k, v.

    ``query`` is ``[total_q, H, D]``, ``key`` / ``value`` are ``[total_k, H, D]``; sequence ``b`` owns rows
    ``cu_seqlens_q[b] : cu_seqlens_q[b+1]`` of the query-side tensors and ``cu_seqlens_k[b] :
    cu_seqlens_k[b+1]`` of the key-side ones (``[B+1]`` integer tensors starting at 0, as flash-attention's
    varlen functions take them); ``max_seqlen_*`` are upper bounds of the lengths.  Each sequence is
    computed exactly as one batch element of :func:`sigmoid_attention_padded` with those lengths
    (default bias ``-log(length of the key sequence)``, causal mask aligned top-left, ``score_mod`` of
    shape ``[total_k]``), but no padded tile is loaded or stored.  The reference has no such entry
    point; its benchmark feeds this layout to the flash-attention provider it compares with.
    """
    if query.dim() != 3 or key.dim() != 3 or value.dim() != 3:
        raise ValueError("Expected query, key, and value to be 3D tensors [total_tokens, H, D]")
    total_q, H, D = query.shape
    total_k, H_k, D_k = key.shape
    if value.shape != key.shape:
        raise ValueError(f"Key and value shapes must match, got K={tuple(key.shape)}, V={tuple(value.shape)}")
    if H != H_k:
        raise ValueError(f"Number of heads mismatch: Q={H}, K={H_k}")
    if D != D_k:
        raise ValueError(f"Head dimension mismatch: Q={D}, K={D_k}")
    if cu_seqlens_q.dim() != 1 or cu_seqlens_k.shape != cu_seqlens_q.shape or cu_seqlens_q.numel() < 1:
        raise ValueError(f"cu_seqlens_q and cu_seqlens_k must be 1D of equal length B+1, got "
                         f"{tuple(cu_seqlens_q.shape)} and {tuple(cu_seqlens_k.shape)}")
    B = cu_seqlens_q.numel() - 1
    if score_mod is not None:
        if score_mod.shape != (total_k,):
            raise ValueError(f"score_mod must have shape ({total_k},), got {score_mod.shape}")
        score_mod = score_mod.contiguous()
    _check_dtype(query, key, value)
    cu_seqlens_q = cu_seqlens_q.to(device=query.device, dtype=torch.int32).contiguous()
    cu_seqlens_k = cu_seqlens_k.to(device=query.device, dtype=torch.int32).contiguous()

    if scale is None:
        scale = 1.0 / math.sqrt(D)
    Dk = _kernel_head_dim(D)
    query, key, value = (_pad_head_dim(t, Dk).contiguous() for t in (query, key, value))

    if torch.compiler.is_compiling():
        if sigmoid_bias is None:
            lens_k = (cu_seqlens_k[1:] - cu_seqlens_k[:-1]).clamp(min=0, max=int(max_seqlen_k))
            bias = -torch.log(lens_k.float())  # +inf for an empty key set; every probability is masked there anyway
        else:
            bias = torch.full((B,), float(sigmoid_bias), dtype=torch.float32, device=query.device)
        out = sigmoid_attn_varlen_fwd_op(query, key, value, cu_seqlens_q, cu_seqlens_k, int(max_seqlen_q),
                                         int(max_seqlen_k), bias, score_mod, float(scale), bool(is_causal))
    else:
        # eager: no dispatcher round trip, the default bias computed by the kernels, an explicit one passed by value
        bias = None if sigmoid_bias is None else float(sigmoid_bias)
        args = (query, key, value, cu_seqlens_q, cu_seqlens_k, int(max_seqlen_q), int(max_seqlen_k), bias, score_mod,
                float(scale), bool(is_causal))
        if torch.is_grad_enabled() and (query.requires_grad or key.requires_grad or value.requires_grad):
            out = _EagerSigmoidAttentionVarlen.apply(*args)
        else:
            out = _run_varlen_fwd(*args)
    return out if Dk == D else out[..., :D]
