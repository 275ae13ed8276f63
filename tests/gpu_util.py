"""Helpers shared by the GPU parity tests (not collected by pytest)."""

import torch

from oracle import sigattn_oracle as orc

# gates from the benchmark specification: max-abs on O, relative L2 on gradients
O_TOL = {torch.float16: 2e-3, torch.bfloat16: 1e-2}
GRAD_REL_L2 = 1e-2


def rel_l2(got: torch.Tensor, ref: torch.Tensor) -> float:
    return ((got.double() - ref.double()).norm() / (ref.double().norm() + 1e-30)).item()


def make_inputs(B, Tq, Tk, H, D, dtype, std=1.0, seed=0, requires_grad=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda T: (torch.randn(B, T, H, D, device="cuda", generator=g) * std).to(dtype)
    q, k, v, do = mk(Tq), mk(Tk), mk(Tk), mk(Tq)
    if requires_grad:
        q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    return q, k, v, do


def check_against_oracle(fn, q, k, v, do, dtype, lens_q=None, lens_k=None, backward=True, o_tol=None, **kw):
    """Run `fn` (public API) forward (+backward) and compare with the CPU oracle on valid rows;
    padded rows must be exactly zero."""
    B, Tq, H, D = q.shape
    Tk = k.shape[1]
    padded = lens_q is not None or lens_k is not None
    if padded:
        out = fn(q, k, v, seq_lens_k=lens_k, seq_lens_q=lens_q, **kw)
    else:
        out = fn(q, k, v, **kw)
    okw = dict(seq_lens_k=lens_k, seq_lens_q=lens_q, is_causal=kw.get("is_causal", False), scale=kw.get("scale"),
               sigmoid_bias=kw.get("sigmoid_bias"), score_mod=kw.get("score_mod"))
    ref = orc.sigattn_forward(q, k, v, **okw)
    got = out.detach().float().cpu()
    assert torch.isfinite(got).all(), "non-finite values in O"
    err = (got - ref).abs().max().item()
    # absolute gate while |O| <= 1 (the default-bias regime), relative to max|O| beyond that
    gate = (o_tol or O_TOL[dtype]) * max(1.0, ref.abs().max().item())
    assert err <= gate, f"O max-abs error {err:.3e} (gate {gate:.3e})"
    mq, mk = orc.valid_row_masks(B, Tq, Tk, lens_q, lens_k)
    assert got[~mq].abs().max().item() == 0 if (~mq).any() else True
    res = {"o_err": err}
    if backward:
        out.backward(do)
        rdq, rdk, rdv = orc.sigattn_backward(q, k, v, do, **okw)
        for name, g, r, mask in (("dq", q.grad, rdq, mq), ("dk", k.grad, rdk, mk), ("dv", v.grad, rdv, mk)):
            g = g.float().cpu()
            assert torch.isfinite(g).all(), f"non-finite values in {name}"
            rl = rel_l2(g, r)
            assert rl <= GRAD_REL_L2, f"{name} relative L2 error {rl:.3e}"
            if (~mask).any():
                assert g[~mask].abs().max().item() == 0, f"{name}: padded rows must be zero"
            res[name] = rl
    return res


def blockwise_fp32_reference(q, k, v, do=None, lens_q=None, lens_k=None, causal=False, scale=None, bias=None,
                             block_q=2048):
    """fp32 torch math of forward (and backward when `do` is given) on the GPU, in blocks of query rows so
    that sequences of 16k-32k tokens fit; same formulas as the CPU oracle (which tests/test_api_cpu.py ties
    to this kind of torch math).  `bias`: [B] tensor or None = -log(valid keys).  Returns fp32
    (O, dQ, dK, dV); rows beyond the valid lengths are zero."""
    import math

    B, Tq, H, D = q.shape
    Tk = k.shape[1]
    dev = q.device
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    lq = torch.full((B,), Tq, device=dev, dtype=torch.int64) if lens_q is None else lens_q.to(dev).long().clamp(0, Tq)
    lk = torch.full((B,), Tk, device=dev, dtype=torch.int64) if lens_k is None else lens_k.to(dev).long().clamp(0, Tk)
    if bias is None:
        bias = -torch.log(lk.float())
    qf, kf, vf = (t.detach().float().transpose(1, 2) for t in (q, k, v))  # [B,H,T,D]
    dof = do.detach().float().transpose(1, 2) if do is not None else None
    o = torch.zeros_like(qf)
    dq = torch.zeros_like(qf) if do is not None else None
    dk = torch.zeros_like(kf) if do is not None else None
    dv = torch.zeros_like(vf) if do is not None else None
    cols = torch.arange(Tk, device=dev).view(1, 1, 1, Tk)
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        for r0 in range(0, Tq, block_q):
            r1 = min(Tq, r0 + block_q)
            rows = torch.arange(r0, r1, device=dev).view(1, 1, r1 - r0, 1)
            keep = (cols < lk.view(B, 1, 1, 1)) & (rows < lq.view(B, 1, 1, 1))
            if causal:
                keep = keep & (cols <= rows)
            s = (qf[:, :, r0:r1] @ kf.transpose(-1, -2)) * scale + bias.view(B, 1, 1, 1)
            p = torch.sigmoid(s).masked_fill(~keep, 0.0)
            del s
            o[:, :, r0:r1] = p @ vf
            if do is not None:
                dob = dof[:, :, r0:r1]
                dv += p.transpose(-1, -2) @ dob
                ds = p * (1.0 - p) * (dob @ vf.transpose(-1, -2))
                dq[:, :, r0:r1] = (ds @ kf) * scale
                dk += (ds.transpose(-1, -2) @ qf[:, :, r0:r1]) * scale
                del ds
            del p, keep
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    back = lambda t: None if t is None else t.transpose(1, 2).contiguous()
    return back(o), back(dq), back(dk), back(dv)


def valid_masks_gpu(B, Tq, Tk, lens_q, lens_k, device):
    """[B, Tq] and [B, Tk] boolean masks of the valid rows."""
    mq = torch.ones(B, Tq, dtype=torch.bool, device=device)
    mk = torch.ones(B, Tk, dtype=torch.bool, device=device)
    if lens_q is not None:
        mq = torch.arange(Tq, device=device)[None, :] < lens_q.to(device)[:, None]
    if lens_k is not None:
        mk = torch.arange(Tk, device=device)[None, :] < lens_k.to(device)[:, None]
    return mq, mk
