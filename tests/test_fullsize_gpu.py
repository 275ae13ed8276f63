"""Parity at the sizes the benchmark tables quote, against fp32 torch math on the GPU computed in blocks of
query rows (`blockwise_fp32_reference`, which tests/test_gpu_util_cpu.py ties to the CPU oracle):

* the padded bf16 configuration with all 16 of its sequences (N_max = 2048, H = 8, D = 64, lengths uniform in
  [256, 2048], N(0,1) values in the padding too), both masks;
* the long end of the sequence-length sweep: one batch element and two heads of N = 16384 and N = 32768 at
  D = 64 and D = 128, and one padded sweep point (lengths uniform in [N/4, N]);
* a (batch, head) slab of the dense bf16 causal B=8, N=8192, H=32, D=128 configuration.

Gates: O max-abs <= 2e-3 (fp16) / 1e-2 (bf16), gradients relative L2 <= 1e-2, rows beyond the valid lengths
exactly zero.  Forward and both backward modes (fused default, split).
"""

import pytest
import torch

import triton_sigmoid_b200 as m
from tests.gpu_util import O_TOL, blockwise_fp32_reference, make_inputs, rel_l2, valid_masks_gpu

pytestmark = pytest.mark.gpu


def _check(q, k, v, do, dtype, lens=None, causal=False, block_q=2048):
    B, T = q.shape[0], q.shape[1]
    for t in (q, k, v):
        t.requires_grad_()
    if lens is not None:
        out = m.sigmoid_attention_padded(q, k, v, seq_lens_k=lens, seq_lens_q=lens, is_causal=causal)
    else:
        out = m.sigmoid_attention(q, k, v, is_causal=causal)
    out.backward(do)
    o32, dq32, dk32, dv32 = blockwise_fp32_reference(q, k, v, do, lens_q=lens, lens_k=lens, causal=causal, block_q=block_q)
    mq, mk = valid_masks_gpu(B, T, T, lens, lens, q.device)
    assert torch.isfinite(out).all()
    assert (out.detach().float() - o32)[mq].abs().max().item() <= O_TOL[dtype]
    for name, g, r, mask in (("dq", q.grad, dq32, mq), ("dk", k.grad, dk32, mk), ("dv", v.grad, dv32, mk)):
        assert torch.isfinite(g).all(), name
        assert rel_l2(g[mask], r[mask]) <= 1e-2, name
        if (~mask).any():
            assert g[~mask].abs().max().item() == 0, name
    if (~mq).any():
        assert out[~mq].abs().max().item() == 0


@pytest.mark.parametrize("split", [False, True])
@pytest.mark.parametrize("causal", [False, True])
def test_padded_benchmark_config_all_sequences(monkeypatch, causal, split):
    if split:
        monkeypatch.setenv("SIGATTN_B200_BWD_SPLIT", "1")
    B, T, H, D = 16, 2048, 8, 64
    q, k, v, do = make_inputs(B, T, T, H, D, torch.bfloat16, seed=2)
    lens = torch.randint(256, 2049, (B,), generator=torch.Generator().manual_seed(2), dtype=torch.int32).cuda()
    _check(q, k, v, do, torch.bfloat16, lens=lens, causal=causal)


@pytest.mark.parametrize("N,D,dtype,causal", [(16384, 64, torch.float16, False), (16384, 128, torch.bfloat16, True),
                                              (32768, 64, torch.bfloat16, False), (32768, 64, torch.float16, True),
                                              (32768, 128, torch.bfloat16, False)])
def test_long_sequences(N, D, dtype, causal):
    q, k, v, do = make_inputs(1, N, N, 2, D, dtype, seed=5)
    _check(q, k, v, do, dtype, causal=causal, block_q=2048)


def test_long_sequences_split_backward(monkeypatch):
    monkeypatch.setenv("SIGATTN_B200_BWD_SPLIT", "1")
    q, k, v, do = make_inputs(1, 16384, 16384, 2, 64, torch.bfloat16, seed=5)
    _check(q, k, v, do, torch.bfloat16, causal=True, block_q=2048)


@pytest.mark.parametrize("causal", [False, True])
def test_padded_sweep_point(causal):
    """2^18 tokens per batch at N = 8192: 32 sequences in the sweep, 4 of them here, lengths uniform in [N/4, N]."""
    B, N, H, D = 4, 8192, 2, 64
    q, k, v, do = make_inputs(B, N, N, H, D, torch.float16, seed=5)
    lens = torch.randint(N // 4, N + 1, (32,), generator=torch.Generator().manual_seed(5), dtype=torch.int32)[:B].cuda()
    _check(q, k, v, do, torch.float16, lens=lens, causal=causal)


def test_long_causal_d128_slab():
    """One batch element and four heads of dense bf16 causal B=8, N=8192, H=32, D=128 (inputs 0.5 N(0,1), seed 3)."""
    q, k, v, do = make_inputs(1, 8192, 8192, 4, 128, torch.bfloat16, std=0.5, seed=3)
    _check(q, k, v, do, torch.bfloat16, causal=True)
