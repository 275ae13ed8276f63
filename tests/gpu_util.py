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
