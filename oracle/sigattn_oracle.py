"""CPU oracle for the sigmoid-attention hot path.  TEST INFRASTRUCTURE ONLY.

This file is the checker, never the product: only the test-suite, the smoke
check and the benchmark's CPU-baseline leg may import it.  The shipped library
computes on the GPU and raises when its CUDA extension is missing.

It restates, in plain fp32/fp64 torch math on the CPU, the algorithm of the
reference project (paths relative to the reference repository):

* forward formula, masking order (bias -> score_mod -> causal -inf -> sigmoid
  -> key padding zero -> P.V -> query padding zero):
  ``src/triton_sigmoid/sigmoid_reference.py:50-152`` and the kernels
  ``src/triton_sigmoid/sigmoid_triton_dense.py:109-154``,
  ``src/triton_sigmoid/sigmoid_triton_padded.py:124-171``;
* bias conventions: dense ``-log(T)``
  (``sigmoid_triton_dense.py:840-843``), padded ``-log(seq_lens_k[b])``
  (``sigmoid_triton_padded.py:995-998``);
* backward formulas dV = P^T dO, dP = dO V^T, dS = P (1-P) dP, dQ = s dS K,
  dK = s dS^T Q with gradients re-masked to zero
  (``sigmoid_triton_dense.py:251-302`` and ``:405-459``);
* zero rows for padded queries / keys
  (``sigmoid_triton_padded.py:93,169-171,337-339,504-509``).

Parity pin: ``tests/golden/`` holds outputs of the reference's own
``sigmoid_attention_ref`` (run on the CPU from the reference checkout by
``tests/golden/make_golden.py``); ``tests/test_oracle.py`` checks this file
against them, and against the reference's autograd gradients stored there.

The ``emulate_dtype`` switch additionally rounds P and dS to the 16-bit input
type before the second GEMM of each chain, which is what the reference kernels
(and the CUDA kernels of this repository) do
(``sigmoid_triton_dense.py:149,299,443,456``).
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def default_bias(B: int, Tk: int, seq_lens_k: Optional[torch.Tensor], sigmoid_bias: Optional[float]) -> torch.Tensor:
    """Per-batch fp32 bias exactly as the reference's public wrappers build it.

    dense: ``sigmoid_triton_dense.py:840-843``; padded: ``sigmoid_triton_padded.py:995-998``.
    """
    if sigmoid_bias is not None:
        return torch.full((B,), float(sigmoid_bias), dtype=torch.float32)
    if seq_lens_k is None:
        return torch.full((B,), -math.log(float(Tk)), dtype=torch.float32)
    return -torch.log(seq_lens_k.detach().cpu().float())


def _valid_mask(B, Tq, Tk, lens_q, lens_k, causal) -> torch.Tensor:
    """[B,1,Tq,Tk] boolean mask: i < Lq[b], j < Lk[b], and i >= j when causal
    (top-left aligned also when Tq != Tk; ``sigmoid_triton_padded.py:152-159``)."""
    i = torch.arange(Tq).view(1, Tq, 1)
    j = torch.arange(Tk).view(1, 1, Tk)
    m = torch.ones(B, Tq, Tk, dtype=torch.bool)
    if lens_q is not None:
        m &= i < lens_q.detach().cpu().long().clamp(min=0, max=Tq).view(B, 1, 1)
    if lens_k is not None:
        m &= j < lens_k.detach().cpu().long().clamp(min=0, max=Tk).view(B, 1, 1)
    if causal:
        m &= i >= j
    return m.view(B, 1, Tq, Tk)


def _scores(q, k, bias, score_mod, scale, work):
    B, Tq, H, D = q.shape
    Tk = k.shape[1]
    qh = q.detach().cpu().to(work).permute(0, 2, 1, 3)
    kh = k.detach().cpu().to(work).permute(0, 2, 1, 3)
    s = torch.matmul(qh, kh.transpose(-1, -2)) * scale + bias.to(work).view(B, 1, 1, 1)
    if score_mod is not None:
        s = s + score_mod.detach().cpu().to(work).view(B, 1, 1, Tk)
    return s


def sigattn_forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    seq_lens_k: Optional[torch.Tensor] = None,
    seq_lens_q: Optional[torch.Tensor] = None,
    is_causal: bool = False,
    scale: Optional[float] = None,
    sigmoid_bias: Optional[float] = None,
    score_mod: Optional[torch.Tensor] = None,
    work: torch.dtype = torch.float32,
    emulate_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """O[b,i,h,:] = sum_j P[i,j] V[b,j,h,:], P = valid ? sigmoid(s q.k + bias + mod) : 0.

    Inputs are (B, T, H, D); the result is returned in ``work`` precision (callers
    round to the input dtype when they need to).
    """
    B, Tq, H, D = q.shape
    Tk = k.shape[1]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    bias = default_bias(B, Tk, seq_lens_k, sigmoid_bias)
    s = _scores(q, k, bias, score_mod, scale, work)
    valid = _valid_mask(B, Tq, Tk, seq_lens_q, seq_lens_k, is_causal)
    p = torch.where(valid, torch.sigmoid(s), torch.zeros((), dtype=work))
    if emulate_dtype is not None:
        p = p.to(emulate_dtype).to(work)
    vh = v.detach().cpu().to(work).permute(0, 2, 1, 3)
    o = torch.matmul(p, vh)  # [B,H,Tq,D]
    return o.permute(0, 2, 1, 3).contiguous()


def sigattn_backward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    do: torch.Tensor,
    seq_lens_k: Optional[torch.Tensor] = None,
    seq_lens_q: Optional[torch.Tensor] = None,
    is_causal: bool = False,
    scale: Optional[float] = None,
    sigmoid_bias: Optional[float] = None,
    score_mod: Optional[torch.Tensor] = None,
    work: torch.dtype = torch.float32,
    emulate_dtype: Optional[torch.dtype] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Manual recomputation backward (no autograd): returns (dQ, dK, dV) in ``work`` precision."""
    B, Tq, H, D = q.shape
    Tk = k.shape[1]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    bias = default_bias(B, Tk, seq_lens_k, sigmoid_bias)
    s = _scores(q, k, bias, score_mod, scale, work)
    valid = _valid_mask(B, Tq, Tk, seq_lens_q, seq_lens_k, is_causal)
    zero = torch.zeros((), dtype=work)
    p = torch.where(valid, torch.sigmoid(s), zero)
    qh = q.detach().cpu().to(work).permute(0, 2, 1, 3)
    kh = k.detach().cpu().to(work).permute(0, 2, 1, 3)
    vh = v.detach().cpu().to(work).permute(0, 2, 1, 3)
    doh = do.detach().cpu().to(work).permute(0, 2, 1, 3)
    dp = torch.matmul(doh, vh.transpose(-1, -2))
    ds = torch.where(valid, p * (1.0 - p) * dp, zero)
    if emulate_dtype is not None:
        p = p.to(emulate_dtype).to(work)
        ds = ds.to(emulate_dtype).to(work)
    dv = torch.matmul(p.transpose(-1, -2), doh)
    dq = torch.matmul(ds, kh) * scale
    dk = torch.matmul(ds.transpose(-1, -2), qh) * scale
    back = lambda t: t.permute(0, 2, 1, 3).contiguous()
    return back(dq), back(dk), back(dv)


def valid_row_masks(B, Tq, Tk, seq_lens_q, seq_lens_k):
    """Boolean [B,Tq] / [B,Tk] masks of the rows the reference's tests compare
    (``tests/test_sigmoid_padded.py:123-124``)."""
    mq = torch.ones(B, Tq, dtype=torch.bool)
    mk = torch.ones(B, Tk, dtype=torch.bool)
    if seq_lens_q is not None:
        mq = torch.arange(Tq).view(1, Tq) < seq_lens_q.detach().cpu().long().view(B, 1)
    if seq_lens_k is not None:
        mk = torch.arange(Tk).view(1, Tk) < seq_lens_k.detach().cpu().long().view(B, 1)
    return mq, mk
