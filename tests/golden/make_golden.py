"""Regenerate the golden fixtures from the reference project's own CPU code.

Run from a machine that has the reference checkout (it is NOT needed to run the tests):

    python tests/golden/make_golden.py /path/to/triton-sigmoid

The reference package refuses to import without a CUDA GPU
(``src/triton_sigmoid/__init__.py:56-60``), but its PyTorch reference
``src/triton_sigmoid/sigmoid_reference.py`` depends only on ``math`` and ``torch``,
so it is loaded by file path and run in fp32 (``upcast=True``) on the CPU.
Gradients come from autograd through that function.

Outputs (next to this script):
  * ``small_cases.npz``   - full input and output tensors of a handful of tiny cases
                            (inputs stored as float16, exactly representable);
  * ``config1_sums.json`` - sum statistics of O, dQ, dK, dV for the B=2, N=256, H=4,
                            D=64, seed-0 configuration (dense, causal, padded, padded+causal).
"""

from __future__ import annotations

import importlib.util
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name -> dict(B, Tq, Tk, H, D, causal, lens_q, lens_k, score_mod, scale, sigmoid_bias)
SMALL_CASES = {
    "dense": dict(B=2, Tq=80, Tk=80, H=2, D=16),
    "dense_causal": dict(B=2, Tq=80, Tk=80, H=2, D=16, causal=True),
    "padded": dict(B=2, Tq=80, Tk=80, H=2, D=16, lens_q=[77, 31], lens_k=[77, 31]),
    "padded_causal": dict(B=2, Tq=80, Tk=80, H=2, D=16, lens_q=[80, 45], lens_k=[80, 45], causal=True),
    "padded_cross": dict(B=2, Tq=48, Tk=80, H=2, D=16, lens_q=[48, 20], lens_k=[64, 80]),
    "score_mod": dict(B=2, Tq=80, Tk=80, H=2, D=16, score_mod=True),
    "explicit_bias_scale": dict(B=1, Tq=40, Tk=40, H=3, D=32, sigmoid_bias=-1.5, scale=0.3, causal=True),
    "klen_only": dict(B=2, Tq=64, Tk=64, H=1, D=16, lens_k=[1, 50]),
}


def load_reference(ref_root: str):
    path = os.path.join(ref_root, "src", "triton_sigmoid", "sigmoid_reference.py")
    spec = importlib.util.spec_from_file_location("_ref_sigmoid_reference", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.sigmoid_attention_ref


def case_inputs(name: str, c: dict):
    """Seeded inputs, rounded to float16 so they can be stored exactly."""
    g = torch.Generator().manual_seed(1000 + sorted(SMALL_CASES).index(name))
    B, Tq, Tk, H, D = c["B"], c["Tq"], c["Tk"], c["H"], c["D"]
    mk = lambda *s: torch.randn(*s, generator=g).half().float()
    q, k, v, do = mk(B, Tq, H, D), mk(B, Tk, H, D), mk(B, Tk, H, D), mk(B, Tq, H, D)
    sm = mk(B, Tk) if c.get("score_mod") else None
    return q, k, v, do, sm


def run_ref(ref, q, k, v, do, lens_q, lens_k, causal, scale, bias, sm):
    q, k, v = [t.clone().requires_grad_() for t in (q, k, v)]
    o = ref(q, k, v, seq_lens_k=lens_k, seq_lens_q=lens_q, scale=scale, sigmoid_bias=bias,
            upcast=True, causal=causal, score_mod=sm)
    o.backward(do)
    return o.detach(), q.grad, k.grad, v.grad


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of MSDLLCpapers/triton-sigmoid>")
    ref_root = sys.argv[1]
    ref = load_reference(ref_root)
    torch.set_num_threads(1)

    out = {}
    for name, c in SMALL_CASES.items():
        q, k, v, do, sm = case_inputs(name, c)
        lq = torch.tensor(c["lens_q"], dtype=torch.int32) if "lens_q" in c else None
        lk = torch.tensor(c["lens_k"], dtype=torch.int32) if "lens_k" in c else None
        o, dq, dk, dv = run_ref(ref, q, k, v, do, lq, lk, c.get("causal", False), c.get("scale"),
                                c.get("sigmoid_bias"), sm)
        for key, t in (("q", q), ("k", k), ("v", v), ("do", do)):
            out[f"{name}/{key}"] = t.numpy().astype(np.float16)
        if sm is not None:
            out[f"{name}/score_mod"] = sm.numpy().astype(np.float16)
        for key, t in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
            out[f"{name}/{key}"] = t.numpy().astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "small_cases.npz"), **out)

    # Configuration 1 of the benchmark plan: sums only (the tensors are 0.5 MB each).
    torch.manual_seed(0)
    q, k, v, do = [torch.randn(2, 256, 4, 64) for _ in range(4)]
    lens = torch.randint(64, 257, (2,), generator=torch.Generator().manual_seed(2), dtype=torch.int32)
    sums = {"lens": lens.tolist(), "input_abs_sum": float(sum(t.double().abs().sum() for t in (q, k, v, do)))}
    for name, (l, causal) in {"dense": (None, False), "causal": (None, True),
                              "padded": (lens, False), "padded_causal": (lens, True)}.items():
        o, dq, dk, dv = run_ref(ref, q, k, v, do, l, l, causal, None, None, None)
        sums[name] = {"sum_o": float(o.double().sum()), "abs_o": float(o.double().abs().sum()),
                      "abs_dq": float(dq.double().abs().sum()), "abs_dk": float(dk.double().abs().sum()),
                      "abs_dv": float(dv.double().abs().sum())}
    with open(os.path.join(HERE, "config1_sums.json"), "w") as f:
        json.dump(sums, f, indent=1)
    print("wrote", os.path.join(HERE, "small_cases.npz"), "and config1_sums.json")


if __name__ == "__main__":
    main()
