"""Packed variable-length sequences (sigmoid_attention_varlen): each sequence must equal one batch
element of the padded / dense computation with the same lengths, checked against the CPU oracle
per sequence and against the padded entry point of this library."""

import pytest
import torch

import triton_sigmoid_b200 as m
from oracle import sigattn_oracle as orc
from tests.gpu_util import GRAD_REL_L2, O_TOL, rel_l2

pytestmark = pytest.mark.gpu


def _packed(lens_q, lens_k, H, D, dtype, seed, std=0.5):
    g = torch.Generator(device="cuda").manual_seed(seed)
    tq, tk = int(sum(lens_q)), int(sum(lens_k))
    mk = lambda n: (torch.randn(n, H, D, device="cuda", generator=g) * std).to(dtype)
    q, k, v, do = mk(tq), mk(tk), mk(tk), mk(tq)
    cu = lambda ls: torch.tensor([0] + list(torch.tensor(ls).cumsum(0)), dtype=torch.int32, device="cuda")
    return q, k, v, do, cu(lens_q), cu(lens_k)


def _check_against_oracle(lens_q, lens_k, H, D, dtype, causal, seed, score_mod=False, **kw):
    q, k, v, do, cu_q, cu_k = _packed(lens_q, lens_k, H, D, dtype, seed)
    for t in (q, k, v):
        t.requires_grad_()
    mod = torch.randn(k.shape[0], device="cuda") * 0.5 if score_mod else None
    out = m.sigmoid_attention_varlen(q, k, v, cu_q, cu_k, max(lens_q), max(lens_k), is_causal=causal, score_mod=mod, **kw)
    assert out.shape == q.shape and out.dtype == dtype
    out.backward(do)
    oq = ok = 0
    for lq, lk in zip(lens_q, lens_k):
        sq, sk = slice(oq, oq + lq), slice(ok, ok + lk)
        oq, ok = oq + lq, ok + lk
        if lq == 0:
            continue
        if lk == 0:
            assert out[sq].abs().max().item() == 0 and q.grad[sq].abs().max().item() == 0
            continue
        okw = dict(is_causal=causal, scale=kw.get("scale"), sigmoid_bias=kw.get("sigmoid_bias"),
                   score_mod=None if mod is None else mod[sk][None])
        args = [t[s][None] for t, s in ((q, sq), (k, sk), (v, sk))]
        ref = orc.sigattn_forward(*args, **okw)[0]
        got = out[sq].detach().float().cpu()
        assert torch.isfinite(got).all()
        assert (got - ref).abs().max().item() <= O_TOL[dtype] * max(1.0, ref.abs().max().item())
        rdq, rdk, rdv = orc.sigattn_backward(*args, do[sq][None], **okw)
        for name, g, r in (("dq", q.grad[sq], rdq[0]), ("dk", k.grad[sk], rdk[0]), ("dv", v.grad[sk], rdv[0])):
            g = g.float().cpu()
            assert torch.isfinite(g).all(), name
            assert rel_l2(g, r) <= GRAD_REL_L2, f"{name} of a sequence with lengths {lq}, {lk}"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D", [64, 128])
def test_self_attention_lengths(D, causal, dtype):
    lens = [128, 1, 300, 255, 256, 257, 77, 512]
    _check_against_oracle(lens, lens, 2, D, dtype, causal, seed=D + int(causal))


@pytest.mark.parametrize("causal", [False, True])
def test_cross_attention_lengths(causal):
    lens_q = [100, 260, 5, 129]
    lens_k = [333, 260, 700, 64] if not causal else [333, 260, 700, 129]
    _check_against_oracle(lens_q, lens_k, 2, 64, torch.float16, causal, seed=3)


def test_empty_sequences_and_score_mod():
    _check_against_oracle([64, 0, 130, 40], [64, 50, 0, 200], 2, 64, torch.bfloat16, False, seed=4, score_mod=True)


def test_explicit_scale_bias_and_small_head_dim():
    _check_against_oracle([200, 90], [200, 90], 2, 32, torch.float16, True, seed=5, scale=0.3, sigmoid_bias=-2.0)


@pytest.mark.parametrize("causal", [False, True])
def test_matches_the_padded_entry_point_bitwise_in_forward(causal):
    """Same tiles, same arithmetic: the packed forward must reproduce the padded one exactly on the
    valid rows (neighbouring sequences' rows in a tile must not leak in)."""
    B, T, H, D = 6, 384, 4, 64
    lens = [384, 200, 129, 1, 383, 256]
    g = torch.Generator(device="cuda").manual_seed(11)
    qp, kp, vp = [(torch.randn(B, T, H, D, device="cuda", generator=g)).half() for _ in range(3)]
    lt = torch.tensor(lens, dtype=torch.int32, device="cuda")
    ref = m.sigmoid_attention_padded(qp, kp, vp, seq_lens_k=lt, seq_lens_q=lt, is_causal=causal)
    pack = lambda x: torch.cat([x[b, :lens[b]] for b in range(B)])
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    out = m.sigmoid_attention_varlen(pack(qp), pack(kp), pack(vp), cu, cu, T, T, is_causal=causal)
    assert torch.equal(out, pack(ref))


def test_many_sequences_many_items():
    """More items than SMs, mixed lengths, compared with the padded entry point (forward and backward)."""
    torch.manual_seed(0)
    B, H, D, T = 40, 8, 64, 512
    lens = [int(x) for x in torch.randint(0, T + 1, (B,))]
    lens[3], lens[7] = 0, T
    g = torch.Generator(device="cuda").manual_seed(12)
    qp, kp, vp, dop = [(torch.randn(B, T, H, D, device="cuda", generator=g) * 0.5).bfloat16() for _ in range(4)]
    for t in (qp, kp, vp):
        t.requires_grad_()
    lt = torch.tensor(lens, dtype=torch.int32, device="cuda")
    ref = m.sigmoid_attention_padded(qp, kp, vp, seq_lens_k=lt, seq_lens_q=lt, is_causal=True)
    ref.backward(dop)
    pack = lambda x: torch.cat([x[b, :lens[b]] for b in range(B)])
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    q, k, v = [pack(t.detach()).requires_grad_() for t in (qp, kp, vp)]
    out = m.sigmoid_attention_varlen(q, k, v, cu, cu, T, T, is_causal=True)
    out.backward(pack(dop))
    assert torch.equal(out, pack(ref.detach()))
    assert torch.equal(k.grad, pack(kp.grad)) and torch.equal(v.grad, pack(vp.grad))
    assert rel_l2(q.grad, pack(qp.grad)) <= 1e-3  # dQ: same terms, reduction order differs


def test_float32_sequences():
    """float32 takes the exact kernels: same gate as the dense float32 tests (1e-5 against the float64 oracle)."""
    lens_q, lens_k = [70, 0, 129, 33], [70, 20, 200, 64]
    q, k, v, do, cu_q, cu_k = _packed(lens_q, lens_k, 2, 64, torch.float32, seed=8)
    for t in (q, k, v):
        t.requires_grad_()
    out = m.sigmoid_attention_varlen(q, k, v, cu_q, cu_k, max(lens_q), max(lens_k))
    out.backward(do)
    oq = ok = 0
    for lq, lk in zip(lens_q, lens_k):
        sq, sk = slice(oq, oq + lq), slice(ok, ok + lk)
        oq, ok = oq + lq, ok + lk
        if lq == 0:
            assert k.grad[sk].abs().max().item() == 0
            continue
        args = [t[s][None] for t, s in ((q, sq), (k, sk), (v, sk))]
        ref = orc.sigattn_forward(*args, work=torch.float64)[0]
        assert (out[sq].detach().double().cpu() - ref).abs().max().item() <= 1e-5
        rd = orc.sigattn_backward(*args, do[sq][None], work=torch.float64)
        for g, r in ((q.grad[sq], rd[0][0]), (k.grad[sk], rd[1][0]), (v.grad[sk], rd[2][0])):
            assert rel_l2(g.double().cpu(), r) <= 1e-5


def test_rows_outside_the_sequences_stay_zero():
    """Packed buffers larger than the sequences (rows behind the last one), gaps between sequences and an
    understated max_seqlen_q: the rows no sequence covers come back as zeros in the output and in dQ."""
    H, D = 2, 64
    # sequences at rows [0, 100), [128, 190) (a gap of 28 rows), 10 spare rows at the end
    cu_q = torch.tensor([0, 100, 190], dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0, 100, 190], dtype=torch.int32, device="cuda")
    total = 200
    g = torch.Generator(device="cuda").manual_seed(4)
    q, k, v, do = [(torch.randn(total, H, D, device="cuda", generator=g) * 0.5).half() for _ in range(4)]
    for t in (q, k, v):
        t.requires_grad_()
    out = m.sigmoid_attention_varlen(q, k, v, cu_q, cu_k, 64, 100)  # second sequence has 90 queries: cut at 64
    out.backward(do)
    assert torch.isfinite(out).all() and torch.isfinite(q.grad).all()
    assert out[190:].abs().max().item() == 0 and q.grad[190:].abs().max().item() == 0       # behind the sequences
    assert out[164:190].abs().max().item() == 0 and q.grad[164:190].abs().max().item() == 0  # beyond max_seqlen_q
    assert out[:64].abs().max().item() > 0 and out[100:164].abs().max().item() > 0
