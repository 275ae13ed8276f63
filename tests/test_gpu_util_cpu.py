"""The fp32 torch math the large-size GPU tests compare with (`blockwise_fp32_reference`) is itself tied to
the CPU oracle here, on the CPU, on a small cross-attention case with lengths and a causal mask."""

import torch

from oracle import sigattn_oracle as orc
from tests.gpu_util import blockwise_fp32_reference, valid_masks_gpu


def test_blockwise_reference_matches_the_oracle():
    torch.manual_seed(0)
    B, Tq, Tk, H, D = 2, 200, 260, 3, 32
    q, k, v, do = [torch.randn(B, T, H, D) for T in (Tq, Tk, Tk, Tq)]
    lq, lk = torch.tensor([200, 77]), torch.tensor([260, 130])
    for causal in (False, True):
        got = blockwise_fp32_reference(q, k, v, do, lens_q=lq, lens_k=lk, causal=causal, block_q=64)
        ref = (orc.sigattn_forward(q, k, v, seq_lens_k=lk, seq_lens_q=lq, is_causal=causal),
               *orc.sigattn_backward(q, k, v, do, seq_lens_k=lk, seq_lens_q=lq, is_causal=causal))
        for a, b in zip(got, ref):
            assert (a - b).abs().max().item() <= 2e-6
    # explicit bias, no lengths, forward only
    bias = torch.tensor([-1.0, 0.5])
    o, dq, dk, dv = blockwise_fp32_reference(q, k, v, None, bias=bias, scale=0.2)
    assert dq is None and dk is None and dv is None
    for b in range(B):
        ref = orc.sigattn_forward(q[b:b + 1], k[b:b + 1], v[b:b + 1], scale=0.2, sigmoid_bias=float(bias[b]))
        assert (o[b:b + 1] - ref).abs().max().item() <= 2e-6


def test_valid_masks():
    mq, mk = valid_masks_gpu(2, 4, 5, torch.tensor([4, 1]), None, torch.device("cpu"))
    assert mq.tolist() == [[True] * 4, [True, False, False, False]] and mk.all()
