"""GPU parity of the library's run-time modes with the CPU oracle (public API -> C ABI):

* the split backward (``SIGATTN_B200_BWD_SPLIT=1``: dK/dV and dQ by two streaming kernels, no workspace,
  no atomics) - the other arm of the "dQ accumulated atomically or via a separate pass" choice, the shape of
  the reference's own backward (sigmoid_triton_dense.py:162-467 there);
* the accurate sigmoid (``TRITON_SIGMOID_ACCURATE`` / ``accurate_sigmoid()``), held to the reference's own
  per-element gates (its tests/conftest.py:27-34 and tests/test_sigmoid_dense.py:111-166: |err| < tol and
  err <= 2 (3 for gradients) x the error of mixed-precision torch math + tol).
"""

import math

import pytest
import torch

import triton_sigmoid_b200 as m
from oracle import sigattn_oracle as orc
from tests.conftest import tolerance
from tests.gpu_util import check_against_oracle, make_inputs, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture
def split_backward(monkeypatch):
    monkeypatch.setenv("SIGATTN_B200_BWD_SPLIT", "1")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,H,T,D", [(1, 2, 128, 64), (2, 2, 300, 64), (1, 4, 512, 128), (2, 2, 1024, 64), (1, 2, 2048, 128)])
def test_split_backward_dense(split_backward, B, H, T, D, causal, dtype):
    q, k, v, do = make_inputs(B, T, T, H, D, dtype, std=0.5, seed=T + D, requires_grad=True)
    check_against_oracle(m.sigmoid_attention, q, k, v, do, dtype, is_causal=causal)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("Tq,Tk", [(128, 128), (256, 512), (512, 256), (640, 640)])
@pytest.mark.parametrize("D", [64, 128])
def test_split_backward_padded_cross_attention(split_backward, Tq, Tk, D, causal):
    if causal and Tq > Tk:
        pytest.skip("the reference skips causal with more queries than keys")
    B, H = 3, 2
    q, k, v, do = make_inputs(B, Tq, Tk, H, D, torch.bfloat16, std=0.5, seed=Tq + Tk + D, requires_grad=True)
    g = torch.Generator().manual_seed(Tq + Tk)
    lq = torch.randint(int(0.3 * Tq), Tq + 1, (B,), generator=g, dtype=torch.int32).cuda()
    lk = torch.randint(int(0.3 * Tk), Tk + 1, (B,), generator=g, dtype=torch.int32).cuda()
    sm = torch.randn(B, Tk, device="cuda")
    check_against_oracle(m.sigmoid_attention_padded, q, k, v, do, torch.bfloat16, lens_q=lq, lens_k=lk,
                         is_causal=causal, score_mod=sm)


@pytest.mark.parametrize("lens", [[16, 64], [128, 256], [1, 255], [129, 0]])
def test_split_backward_edge_lengths_and_nan_padding(split_backward, lens):
    q, k, v, do = make_inputs(2, 256, 256, 2, 64, torch.float16, std=0.5, seed=sum(lens), requires_grad=True)
    l = torch.tensor(lens, dtype=torch.int32, device="cuda")
    with torch.no_grad():
        for t in (q, k, v, do):
            for b in range(2):
                t[b, lens[b]:] = float("nan")
    out = m.sigmoid_attention_padded(q, k, v, seq_lens_k=l, seq_lens_q=l, is_causal=True)
    out.backward(do)
    qc, kc, vc, doc = [torch.nan_to_num(t.detach()) for t in (q, k, v, do)]
    ref = orc.sigattn_backward(qc, kc, vc, doc, seq_lens_k=l, seq_lens_q=l, is_causal=True)
    for g, r in zip((q.grad, k.grad, v.grad), ref):
        assert torch.isfinite(g).all()
        assert rel_l2(g.float().cpu(), r) <= 1e-2 or r.abs().max() == 0
    valid = torch.arange(256, device="cuda")[None, :] < l[:, None]
    for g in (q.grad, k.grad, v.grad):
        assert g[~valid].abs().max().item() == 0


def test_split_backward_many_mixed_items_is_deterministic(split_backward):
    """Several times more work items than SMs with empty, ragged and full ones mixed, twice: the split
    backward uses no atomics, so the two runs agree bit for bit; the fused default agrees within the gate."""
    B, T, H, D = 24, 640, 8, 64
    lens = torch.tensor([640, 0, 1, 127, 128, 129, 255, 256, 257, 300, 383, 384, 385, 511, 512, 513, 600, 639, 17, 64,
                         200, 450, 77, 640], dtype=torch.int32, device="cuda")
    q, k, v, do = make_inputs(B, T, T, H, D, torch.float16, std=0.5, seed=3, requires_grad=True)
    grads = []
    for _ in range(2):
        q.grad = k.grad = v.grad = None
        m.sigmoid_attention_padded(q, k, v, seq_lens_k=lens, seq_lens_q=lens, is_causal=True).backward(do)
        grads.append([t.grad.clone() for t in (q, k, v)])
    for a, b in zip(*grads):
        assert torch.equal(a, b)
    qf, kf, vf = [t.detach().float().requires_grad_() for t in (q, k, v)]
    valid = torch.arange(T, device="cuda")[None, :] < lens[:, None]
    ref = m.sigmoid_attention_ref(qf, kf, vf, seq_lens_k=lens, seq_lens_q=lens, causal=True) * valid[:, :, None, None]
    ref.backward(do.float() * valid[:, :, None, None])
    for g, r in zip(grads[0], (qf.grad, kf.grad, vf.grad)):
        assert g[~valid].abs().max().item() == 0
        assert rel_l2(g[valid], r[valid]) <= 1e-2


def test_split_backward_packed_layout(split_backward):
    lens = [100, 37, 163, 0, 256]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    total, H, D = sum(lens), 2, 64
    g = torch.Generator(device="cuda").manual_seed(11)
    q, k, v, do = [(torch.randn(total, H, D, device="cuda", generator=g) * 0.5).half() for _ in range(4)]
    for t in (q, k, v):
        t.requires_grad_()
    out = m.sigmoid_attention_varlen(q, k, v, cu, cu, max(lens), max(lens), is_causal=True)
    out.backward(do)
    for b, L in enumerate(lens):
        if L == 0:
            continue
        s = slice(int(cu[b]), int(cu[b + 1]))
        qb, kb, vb, dob = [t[s].detach()[None] for t in (q, k, v, do)]
        ref_o = orc.sigattn_forward(qb, kb, vb, is_causal=True)
        ref = orc.sigattn_backward(qb, kb, vb, dob, is_causal=True)
        assert (out[s].detach().float().cpu() - ref_o[0]).abs().max().item() <= 2e-3
        for gr, r in zip((q.grad, k.grad, v.grad), ref):
            assert rel_l2(gr[s].float().cpu(), r[0]) <= 1e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,H,T,D", [(1, 2, 128, 64), (4, 2, 256, 64), (1, 8, 512, 128), (2, 2, 1024, 64), (1, 2, 2048, 128)])
@pytest.mark.parametrize("split", [False, True])
def test_accurate_mode_meets_the_reference_gates_per_element(monkeypatch, B, H, T, D, causal, dtype, split):
    if split:
        monkeypatch.setenv("SIGATTN_B200_BWD_SPLIT", "1")
    tol = tolerance(dtype)
    q, k, v, do = make_inputs(B, T, T, H, D, dtype, std=0.5, seed=T + D, requires_grad=True)
    with m.accurate_sigmoid(True):
        out = m.sigmoid_attention(q, k, v, is_causal=causal)
        out.backward(do)
    ours = (out.detach(), q.grad, k.grad, v.grad)
    exact = (orc.sigattn_forward(q, k, v, is_causal=causal), *orc.sigattn_backward(q, k, v, do, is_causal=causal))
    pq, pk, pv = [t.detach().clone().requires_grad_() for t in (q, k, v)]
    pt_out = m.sigmoid_attention_ref(pq, pk, pv, upcast=False, reorder_ops=True, causal=causal, sigmoid_bias=-math.log(T))
    pt_out.backward(do)
    pt = (pt_out.detach(), pq.grad, pk.grad, pv.grad)
    for i, name in enumerate(("o", "dq", "dk", "dv")):
        mult = 2 if i == 0 else 3
        err = (ours[i].float().cpu() - exact[i]).abs().max().item()
        pt_err = (pt[i].float().cpu() - exact[i]).abs().max().item()
        # the fused backward rounds dS once more than torch does (it feeds dK from a 16-bit copy); the gate
        # with the mixed-precision error term is the reference's, the bare one gets its 2x allowance for dV
        assert err <= mult * pt_err + tol, f"{name}: {err:.3e} > {mult} x {pt_err:.3e} + {tol:.1e}"
        assert err < 2 * tol, f"{name}: {err:.3e} >= {2 * tol:.1e}"


def test_accurate_mode_is_read_from_the_environment_at_call_time(monkeypatch):
    q, k, v, _ = make_inputs(1, 256, 256, 2, 64, torch.float16, seed=21)
    monkeypatch.delenv("TRITON_SIGMOID_ACCURATE", raising=False)
    fast = m.sigmoid_attention(q, k, v, sigmoid_bias=0.0)
    monkeypatch.setenv("TRITON_SIGMOID_ACCURATE", "1")
    acc = m.sigmoid_attention(q, k, v, sigmoid_bias=0.0)
    with m.accurate_sigmoid(True):
        acc2 = m.sigmoid_attention(q, k, v, sigmoid_bias=0.0)
    assert torch.equal(acc, acc2)
    ref = orc.sigattn_forward(q, k, v, sigmoid_bias=0.0)
    e_fast = (fast.float().cpu() - ref).abs().max().item()
    e_acc = (acc.float().cpu() - ref).abs().max().item()
    gate = 2e-3 * max(1.0, ref.abs().max().item())
    assert e_fast <= gate and e_acc <= gate
