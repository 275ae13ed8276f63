"""GPU parity of sigmoid_attention_padded with the CPU oracle (public API -> C ABI).
Follows the reference's tests/test_sigmoid_padded.py: cross-attention shapes, lengths in
[0.8 T, T], padded rows exactly zero, edge lengths."""

import pytest
import torch

import triton_sigmoid_b200 as m
from tests.gpu_util import check_against_oracle, make_inputs, rel_l2

pytestmark = pytest.mark.gpu


def _lens(B, T, lo_frac, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(int(lo_frac * T), T + 1, (B,), generator=g, dtype=torch.int32).cuda()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("Tq,Tk", [(128, 128), (256, 512), (512, 256), (1024, 1024)])
@pytest.mark.parametrize("D", [64, 128])
def test_parity_sweep(Tq, Tk, D, causal, dtype):
    if causal and Tq > Tk:
        pytest.skip("the reference skips causal with more queries than keys")
    B, H = 3, 2
    q, k, v, do = make_inputs(B, Tq, Tk, H, D, dtype, std=0.5, seed=Tq + Tk + D, requires_grad=True)
    lq, lk = _lens(B, Tq, 0.8, 1), _lens(B, Tk, 0.8, 2)
    check_against_oracle(m.sigmoid_attention_padded, q, k, v, do, dtype, lens_q=lq, lens_k=lk, is_causal=causal)


@pytest.mark.parametrize("causal", [False, True])
def test_benchmark_varlen_config_reduced(causal):
    """bf16, N_max=2048, H=8, D=64, lengths uniform in [256, 2048] with N(0,1) garbage in the
    padding (benchmark configuration 3, with 4 of its 16 sequences to keep the oracle quick)."""
    B, T, H, D = 4, 2048, 8, 64
    q, k, v, do = make_inputs(B, T, T, H, D, torch.bfloat16, seed=2, requires_grad=True)
    lens = torch.randint(256, 2049, (16,), generator=torch.Generator().manual_seed(2), dtype=torch.int32)[:B].cuda()
    check_against_oracle(m.sigmoid_attention_padded, q, k, v, do, torch.bfloat16, lens_q=lens, lens_k=lens,
                         is_causal=causal)


@pytest.mark.parametrize("lens", [[16, 64], [128, 256], [1, 255], [129, 0]])
def test_edge_lengths(lens):
    q, k, v, do = make_inputs(2, 256, 256, 2, 64, torch.float16, std=0.5, seed=sum(lens), requires_grad=True)
    l = torch.tensor(lens, dtype=torch.int32, device="cuda")
    check_against_oracle(m.sigmoid_attention_padded, q, k, v, do, torch.float16, lens_q=l, lens_k=l)


def test_zero_length_keys_give_zeros_without_nan():
    q, k, v, do = make_inputs(2, 128, 128, 2, 64, torch.float16, seed=3, requires_grad=True)
    lk = torch.tensor([0, 100], dtype=torch.int32, device="cuda")
    out = m.sigmoid_attention_padded(q, k, v, seq_lens_k=lk)
    out.backward(do)
    for t in (out, q.grad, k.grad, v.grad):
        assert torch.isfinite(t).all()
    assert out[0].abs().max().item() == 0 and q.grad[0].abs().max().item() == 0


def test_none_lengths_mean_no_padding_and_match_dense():
    q, k, v, _ = make_inputs(2, 384, 384, 2, 64, torch.float16, std=0.5, seed=4)
    a = m.sigmoid_attention_padded(q, k, v)
    full = torch.full((2,), 384, dtype=torch.int32, device="cuda")
    b = m.sigmoid_attention_padded(q, k, v, seq_lens_k=full, seq_lens_q=full)
    c = m.sigmoid_attention(q, k, v)
    assert torch.equal(a, b)
    assert (a.float() - c.float()).abs().max().item() <= 2e-3


def test_int64_lengths_are_cast():
    q, k, v, _ = make_inputs(2, 128, 128, 2, 64, torch.float16, seed=5)
    l32 = torch.tensor([100, 60], dtype=torch.int32, device="cuda")
    assert torch.equal(m.sigmoid_attention_padded(q, k, v, seq_lens_k=l32, seq_lens_q=l32),
                       m.sigmoid_attention_padded(q, k, v, seq_lens_k=l32.long(), seq_lens_q=l32.long()))


def test_out_of_range_lengths_are_clamped():
    q, k, v, _ = make_inputs(2, 128, 128, 2, 64, torch.float16, seed=6)
    big = torch.tensor([500, -3], dtype=torch.int32, device="cuda")
    out = m.sigmoid_attention_padded(q, k, v, seq_lens_k=big, seq_lens_q=big, sigmoid_bias=-1.0)
    assert out.shape == q.shape and torch.isfinite(out).all()
    assert out[1].abs().max().item() == 0


def test_score_mod_cross_attention():
    q, k, v, do = make_inputs(2, 192, 320, 2, 64, torch.bfloat16, std=0.5, seed=7, requires_grad=True)
    sm = torch.randn(2, 320, device="cuda")
    lq = torch.tensor([192, 50], dtype=torch.int32, device="cuda")
    lk = torch.tensor([300, 320], dtype=torch.int32, device="cuda")
    check_against_oracle(m.sigmoid_attention_padded, q, k, v, do, torch.bfloat16, lens_q=lq, lens_k=lk, score_mod=sm)


def test_causality_with_padding():
    q, k, v, _ = make_inputs(2, 512, 512, 2, 64, torch.float16, seed=8)
    l = torch.tensor([512, 400], dtype=torch.int32, device="cuda")
    o1 = m.sigmoid_attention_padded(q, k, v, seq_lens_k=l, seq_lens_q=l, is_causal=True)
    k2 = k.clone()
    k2[:, 260:] += 3.0
    o2 = m.sigmoid_attention_padded(q, k2, v, seq_lens_k=l, seq_lens_q=l, is_causal=True)
    assert torch.equal(o1[:, :260], o2[:, :260])


def test_nan_in_padding_does_not_leak():
    """Padded key/value/query rows may hold anything, NaN included."""
    q, k, v, do = make_inputs(2, 256, 256, 2, 64, torch.float16, std=0.5, seed=9, requires_grad=True)
    l = torch.tensor([200, 77], dtype=torch.int32, device="cuda")
    with torch.no_grad():
        for t in (q, k, v, do):
            t[0, 200:] = float("nan")
            t[1, 77:] = float("nan")
    out = m.sigmoid_attention_padded(q, k, v, seq_lens_k=l, seq_lens_q=l)
    out.backward(do)
    for t in (out, q.grad, k.grad, v.grad):
        assert torch.isfinite(t).all()


def test_forward_is_deterministic():
    q, k, v, _ = make_inputs(3, 640, 640, 2, 128, torch.bfloat16, seed=10)
    l = _lens(3, 640, 0.3, 3)
    a = m.sigmoid_attention_padded(q, k, v, seq_lens_k=l, seq_lens_q=l, is_causal=True)
    assert torch.equal(a, m.sigmoid_attention_padded(q, k, v, seq_lens_k=l, seq_lens_q=l, is_causal=True))


@pytest.mark.parametrize("D,dtype", [(64, torch.float16), (128, torch.bfloat16)])
@pytest.mark.parametrize("causal", [False, True])
def test_many_items_with_mixed_lengths_against_gpu_fp32_math(D, dtype, causal):
    """Several times more (batch, head, block) items than SMs, with empty, ragged and full ones mixed:
    every CTA of the persistent kernels walks through all kinds of items, in an order that depends
    on timing.  Compared with fp32 torch math on the GPU; padded rows must be exactly zero."""
    B, T, H = 24, 640, 8
    lens = torch.tensor([640, 0, 1, 127, 128, 129, 255, 256, 257, 300, 383, 384, 385, 511, 512, 513, 600, 639, 17, 64,
                         200, 450, 77, 640], dtype=torch.int32, device="cuda")
    q, k, v, do = make_inputs(B, T, T, H, D, dtype, std=0.5, seed=D + int(causal), requires_grad=True)
    out = m.sigmoid_attention_padded(q, k, v, seq_lens_k=lens, seq_lens_q=lens, is_causal=causal)
    out.backward(do)
    qf, kf, vf = [t.detach().float().requires_grad_() for t in (q, k, v)]
    ref = m.sigmoid_attention_ref(qf, kf, vf, seq_lens_k=lens, seq_lens_q=lens, causal=causal)
    valid = torch.arange(T, device="cuda")[None, :] < lens[:, None]  # [B, T]
    ref = ref * valid[:, :, None, None]
    ref.backward(do.float() * valid[:, :, None, None])
    tol = {torch.float16: 2e-3, torch.bfloat16: 1e-2}[dtype]
    assert (out.float() - ref).abs().max().item() <= tol
    assert out[~valid].abs().max().item() == 0
    for g, r in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
        assert torch.isfinite(g).all()
        assert g[~valid].abs().max().item() == 0
        assert rel_l2(g[valid], r[valid]) <= 1e-2


@pytest.mark.parametrize("D,dtype", [(64, torch.float16), (128, torch.bfloat16)])
def test_query_tile_without_work_for_many_items(D, dtype):
    """Cross-attention with 256 query slots of which most batch elements use only the first 128 (so the second
    query tile of their work items has no keys at all) against 640 keys, a few full ones in between: in the
    forward kernel the warps of the second query tile then sit out whole items while the first tile's run
    through five jobs each, and must still be in step with the score buffers when their next job comes.
    Repeated, since the order of items per SM depends on timing."""
    B, Tq, Tk, H = 48, 256, 640, 8
    lq = torch.full((B,), 128, dtype=torch.int32)
    lq[5::7] = 256
    lq[11] = 129
    lq = lq.cuda()
    lk = torch.full((B,), Tk, dtype=torch.int32, device="cuda")
    q, k, v, _ = make_inputs(B, Tq, Tk, H, D, dtype, std=0.5, seed=D)
    qf, kf, vf = q.float(), k.float(), v.float()
    ref = m.sigmoid_attention_ref(qf, kf, vf, seq_lens_k=lk, seq_lens_q=lq)
    valid = torch.arange(Tq, device="cuda")[None, :] < lq[:, None]
    ref = ref * valid[:, :, None, None]
    tol = {torch.float16: 2e-3, torch.bfloat16: 1e-2}[dtype]
    for _ in range(20):
        out = m.sigmoid_attention_padded(q, k, v, seq_lens_k=lk, seq_lens_q=lq)
        assert m.device_status() == 0
        assert (out.float() - ref).abs().max().item() <= tol
        assert out[~valid].abs().max().item() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_default_bias_computed_on_the_device_matches_the_bias_tensor(dtype):
    """The eager padded call lets the kernels compute the default bias -log(valid keys) (C-ABI flag
    SIGATTN_BIAS_NEG_LOG_LK); the registered op gets it as a [B] tensor computed by torch, as the reference
    does (sigmoid_triton_padded.py:995-998).  Same results up to the last bit of the logarithm, also for an
    element without keys, lengths beyond the tensor and the split backward's kernels."""
    from triton_sigmoid_b200 import ops

    B, T, H, D = 5, 300, 2, 64
    q, k, v, do = make_inputs(B, T, T, H, D, dtype, std=0.5, seed=9, requires_grad=True)
    lens = torch.tensor([300, 0, 17, 129, 400], dtype=torch.int32, device="cuda")
    scale = 1.0 / D ** 0.5
    out = m.sigmoid_attention_padded(q, k, v, seq_lens_k=lens, seq_lens_q=lens, is_causal=True)
    out.backward(do)
    bias = -torch.log(lens.clamp(min=0, max=T).float())
    ref_o = ops.sigmoid_attn_padded_fwd_op(q.detach(), k.detach(), v.detach(), lens, lens, bias, None, scale, True)
    ref_g = ops.sigmoid_attn_padded_bwd_op(q.detach(), k.detach(), v.detach(), do, lens, lens, bias, None, scale, True)
    tol = 1e-6 if dtype == torch.float32 else 2e-3
    assert torch.isfinite(out).all()
    assert (out.detach().float() - ref_o.float()).abs().max().item() <= tol
    for g, r in zip((q.grad, k.grad, v.grad), ref_g):
        assert torch.isfinite(g).all()
        assert (g.float() - r.float()).abs().max().item() <= tol * max(1.0, r.float().abs().max().item())


@pytest.mark.parametrize("D,T", [(64, 2048), (128, 1024)])
def test_backward_repeatable_with_short_and_long_items_mixed(D, T):
    """Cross-attention lengths drawn independently for queries and keys (B=16, H=8; T=2048 at D=64): key tiles
    with a handful of query tiles and with sixteen follow each other on every SM.  In the backward kernel the
    epilogue of the short ones belongs to the drain warps and that of the long ones to the compute warps, which
    run ahead of each other; dK and dV are accumulated in a fixed order, so any mix-up in handing the
    accumulators back shows as a run-to-run difference.  Also compared with fp32 torch math."""
    B, H = 16, 8
    g = torch.Generator().manual_seed(7)
    q, k, v, do = make_inputs(B, T, T, H, D, torch.bfloat16, std=0.5, seed=3, requires_grad=True)
    for trial in range(3):
        lq = torch.randint(0, T + 1, (B,), generator=g, dtype=torch.int32)
        lk = torch.randint(0, T + 1, (B,), generator=g, dtype=torch.int32)
        lq[trial], lq[trial + 3], lq[trial + 6] = 58, 128, 303
        lq, lk = lq.cuda(), lk.cuda()
        first = None
        for rep in range(10):
            q.grad = k.grad = v.grad = None
            out = m.sigmoid_attention_padded(q, k, v, seq_lens_k=lk, seq_lens_q=lq)
            out.backward(do)
            cur = (out.detach().clone(), k.grad.clone(), v.grad.clone(), q.grad.clone())
            assert m.device_status() == 0
            if first is None:
                first = cur
            else:
                for name, a, b in zip(("o", "dk", "dv"), cur, first):
                    assert torch.equal(a, b), f"{name} differs between runs (trial {trial}, repetition {rep})"
                assert rel_l2(cur[3], first[3]) <= 1e-4
        qf, kf, vf = [t.detach().float().requires_grad_() for t in (q, k, v)]
        vq = torch.arange(T, device="cuda")[None, :] < lq[:, None]
        vk = torch.arange(T, device="cuda")[None, :] < lk[:, None]
        ref = m.sigmoid_attention_ref(qf, kf, vf, seq_lens_k=lk, seq_lens_q=lq) * vq[:, :, None, None]
        ref.backward(do.float() * vq[:, :, None, None])
        assert (first[0].float() - ref).abs().max().item() <= 1e-2
        for gr, r, mask in ((first[3], qf.grad, vq), (first[1], kf.grad, vk), (first[2], vf.grad, vk)):
            assert torch.isfinite(gr).all()
            assert gr[~mask].abs().max().item() == 0
            if mask.any() and r[mask].abs().max() > 0:
                assert rel_l2(gr[mask], r[mask]) <= 1e-2
