"""Plain PyTorch statement of sigmoid attention (autograd-differentiable, any device).

Exported as ``sigmoid_attention_ref`` with the keyword arguments of the reference package's
function of that name (``src/triton_sigmoid/sigmoid_reference.py:16-28``) so that user code
that imports it keeps working.  The CUDA ops never call it.
"""

from __future__ import annotations

import math
from typing import Optional

import torch


def sigmoid_attention_ref(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    seq_lens_k: Optional[torch.Tensor] = None,
    seq_lens_q: Optional[torch.Tensor] = None,
    scale: Optional[float] = None,
    sigmoid_bias: Optional[float] = None,
    upcast: bool = True,
    reorder_ops: bool = False,
    causal: bool = False,
    score_mod: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``sigmoid(q k^T scale + bias + score_mod) v`` on ``[B, T, H, D]`` tensors.

    ``upcast=True`` computes in float32; ``upcast=False`` keeps both matrix products in the
    input dtype (scores are promoted to float32 only for the bias and the sigmoid).
    ``reorder_ops`` folds ``scale`` into the keys instead of the queries.  The default bias is
    ``-log(number of valid keys + 1e-6)``.
    """
    B, Tq, H, D = q.shape
    Tk = k.shape[1]
    out_dtype = q.dtype
    dev = q.device
    if scale is None:
        scale = 1.0 / math.sqrt(D)

    if sigmoid_bias is not None:
        bias = torch.full((B, 1, 1, 1), float(sigmoid_bias), dtype=torch.float32, device=dev)
    elif seq_lens_k is not None:
        bias = -(seq_lens_k.to(dev).float() + 1e-6).log().view(B, 1, 1, 1)
    else:
        bias = torch.full((B, 1, 1, 1), -math.log(float(Tk) + 1e-6), dtype=torch.float32, device=dev)

    if upcast:
        q, k, v = q.float(), k.float(), v.float()
    qh, kh, vh = (t.transpose(1, 2) for t in (q, k, v))  # [B,H,T,D]
    if reorder_ops:
        scores = qh @ (kh * scale).transpose(-1, -2)
    else:
        scores = (qh * scale) @ kh.transpose(-1, -2)
    scores = scores.float() + bias
    if score_mod is not None:
        scores = scores + score_mod.to(dev).float().view(B, 1, 1, Tk)

    keep = torch.ones(B, 1, Tq, Tk, dtype=torch.bool, device=dev)
    if causal:
        rows = torch.arange(Tq, device=dev).view(1, 1, Tq, 1)
        cols = torch.arange(Tk, device=dev).view(1, 1, 1, Tk)
        keep = keep & (cols <= rows)
    if seq_lens_k is not None:
        cols = torch.arange(Tk, device=dev).view(1, 1, 1, Tk)
        keep = keep & (cols < seq_lens_k.to(dev).view(B, 1, 1, 1))
    probs = torch.sigmoid(scores.masked_fill(~keep, float("-inf")))
    probs = probs.masked_fill(~keep, 0.0)
    if not upcast:
        probs = probs.to(out_dtype)
    out = (probs @ vh).transpose(1, 2)
    if seq_lens_q is not None:
        rows = torch.arange(Tq, device=dev).view(1, Tq, 1, 1)
        out = out.masked_fill(rows >= seq_lens_q.to(dev).view(B, 1, 1, 1), 0.0)
    return out.to(out_dtype)
