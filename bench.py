#!/usr/bin/env python
"""Benchmark of the sigmoid-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference-cpu]
                    [--workload NAME]

One "step" is a forward + backward pass of the workload through the public API
(`sigmoid_attention` / `sigmoid_attention_padded` + `.backward`).  The default workload is the
configuration the headline metric is quoted on: dense fp16, B=4, N=4096, H=16, D=64, q,k,v,dO ~
N(0,1) (seed 1), non-causal; with --gpus N every rank (one process per GPU, no collective on the
data path) runs that workload on its own data, i.e. weak scaling with a global batch of 4 N.

FLOP accounting (the reference's benchmark): forward 4 B H N^2 D, halved when causal, padded
4 H D sum_b Lq_b Lk_b; backward 2.5x forward; forward+backward 3.5x.

Rank 0 prints ONE JSON line.  `value` is forward+backward TFLOP/s with inputs resident in HBM;
`e2e` is the same metric with pinned HOST inputs and outputs, the copies inside the timed region (one
batch element at a time over three streams, so that the upload of element b+1 and the download of
element b-1 run under the computation of element b);
`roofline` is the backward kernel (the dominant one) timed alone through the C ABI's event hooks;
`extra.workloads` holds device-timed forward and forward+backward figures of the other configurations
(causal variant, padded, the dense causal D=128 configuration - sharded over the ranks under torchrun -
and two sequence-length sweep points), a few steps each;
`cpu_baseline` is the reference's own PyTorch CPU code timed on the host cores (rank 0, N=1).

--impl reference runs the unmodified reference package (its Triton kernels, installed under
baseline/_ref) on the same workload, same timing; --impl reference-cpu runs the reference's CPU
PyTorch code on a bounded sample of the workload.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: B, N, H, D, dtype, causal, padded, std, seed
    # cfg1 is the reference's CPU-runnable case (float32: the exact FMA-pipe kernels, not the tensor-core ones)
    "cfg1": dict(B=2, N=256, H=4, D=64, dtype="fp32", causal=False, padded=False, std=1.0, seed=0),
    "cfg2": dict(B=4, N=4096, H=16, D=64, dtype="fp16", causal=False, padded=False, std=1.0, seed=1),
    "cfg2-causal": dict(B=4, N=4096, H=16, D=64, dtype="fp16", causal=True, padded=False, std=1.0, seed=1),
    "cfg3": dict(B=16, N=2048, H=8, D=64, dtype="bf16", causal=False, padded=True, lo=256, std=1.0, seed=2),
    "cfg3-causal": dict(B=16, N=2048, H=8, D=64, dtype="bf16", causal=True, padded=True, lo=256, std=1.0, seed=2),
    "cfg4": dict(B=8, N=8192, H=32, D=128, dtype="bf16", causal=True, padded=False, std=0.5, seed=3, strong=True),
}
DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}


def parse_workload(name: str) -> dict:
    """Named configurations, or sweep points 'sweep:N:D:dtype:dense|padded:causal|full'
    (2^18 tokens per batch of sequences, H=16)."""
    if name in WORKLOADS:
        return dict(WORKLOADS[name], name=name)
    if name.startswith("sweep:"):
        _, n, d, dt, pad, cz = name.split(":")
        n, d = int(n), int(d)
        return dict(name=name, B=(1 << 18) // n, N=n, H=16, D=d, dtype=dt, causal=(cz == "causal"),
                    padded=(pad == "padded"), lo=n // 4, std=1.0, seed=5)
    raise SystemExit(f"unknown workload {name}")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            pk = json.load(f)
        return dict(burst=float(pk["bf16_tflops"]), sustained=float(pk.get("bf16_tflops_sustained", pk["bf16_tflops"])),
                    hbm_gbs=float(pk.get("hbm_gbs", 6650.0)), source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = []
        with open(self.path) as f:
            for line in f:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) >= 7 and parts[0].isdigit():
                    rows.append(parts)
        os.unlink(self.path)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = [int(r[0]) for r in rows]
        busy = [x for x in sm if x > 0.5 * max(sm)] or sm
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        power = [float(r[2]) for r in rows if r[2].replace(".", "", 1).isdigit()]
        return {"sm_mhz": int(statistics.median(busy)), "sm_max_mhz": int(rows[0][1]), "reasons": reasons,
                "samples": len(rows), "power_w_max": max(power) if power else None}


# ----------------------------------------------------------------------------- workload
def make_data(w: dict, device, rank: int):
    """Seeded synthetic tensors of the workload's shapes (a different stream per rank)."""
    dt = DTYPES[w["dtype"]]
    g = torch.Generator(device=device).manual_seed(w["seed"] + 1000 * rank)
    B, N, H, D = w["B"], w["N"], w["H"], w["D"]
    mk = lambda: (torch.randn(B, N, H, D, device=device, generator=g) * w["std"]).to(dt)
    q, k, v, do = mk(), mk(), mk(), mk()
    lens = None
    if w["padded"]:
        lens = torch.randint(w["lo"], N + 1, (B,), generator=torch.Generator().manual_seed(w["seed"]),
                             dtype=torch.int32).to(device)
    return q, k, v, do, lens


def fwd_flops(w: dict, lens) -> float:
    if w["padded"]:
        l = lens.double().cpu()
        f = 4.0 * w["H"] * w["D"] * float((l * l).sum())
    else:
        f = 4.0 * w["B"] * w["H"] * float(w["N"]) ** 2 * w["D"]
    return f / 2 if w["causal"] else f


def get_impl(impl: str):
    """Returns (dense_fn, padded_fn, label)."""
    if impl == "ours":
        import triton_sigmoid_b200 as m

        return m.sigmoid_attention, m.sigmoid_attention_padded, "triton_sigmoid_b200"
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "triton_sigmoid")):
        raise RuntimeError("baseline/_ref/triton_sigmoid is missing (reference not installed)")
    sys.path.insert(0, ref_dir)
    import triton_sigmoid as ref  # the unmodified reference package: Triton kernels

    return ref.sigmoid_attention, ref.sigmoid_attention_padded, f"triton_sigmoid {getattr(ref, '__version__', '?')}"


def make_step(w, fns, q, k, v, do, lens):
    dense, padded, _ = fns
    causal = w["causal"]

    def fwd_only():
        with torch.no_grad():
            if w["padded"]:
                return padded(q, k, v, seq_lens_k=lens, seq_lens_q=lens, is_causal=causal)
            return dense(q, k, v, is_causal=causal)

    def fwd_bwd():
        q.grad = k.grad = v.grad = None
        if w["padded"]:
            o = padded(q, k, v, seq_lens_k=lens, seq_lens_q=lens, is_causal=causal)
        else:
            o = dense(q, k, v, is_causal=causal)
        o.backward(do)
        return o

    return fwd_only, fwd_bwd


def timed(fn, steps: int, warmup: int, flush, barrier) -> float:
    """Total device milliseconds of `steps` calls (CUDA events around each, L2 flushed between)."""
    for _ in range(warmup):
        flush.zero_()
        fn()
    torch.cuda.synchronize()
    barrier()
    pairs = []
    for _ in range(steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        pairs.append((e0, e1))
    torch.cuda.synchronize()
    barrier()
    return sum(a.elapsed_time(b) for a, b in pairs)


def e2e_step_factory(w, fns, q, k, v, do, lens):
    """Step with pinned host inputs/outputs, what a caller whose tensors live on the host would do: per batch
    element, H2D of q,k,v and then dO on a copy stream, forward and backward on the compute stream (the forward
    starts when q,k,v have arrived), D2H of O (during the backward) and of dQ,dK,dV on a third stream, chained
    by events, so uploads, computation and downloads of neighbouring elements overlap.
    Returns (step, bytes in, bytes out); `step` leaves the current stream waiting for every download."""
    host_in = [t.detach().cpu().pin_memory() for t in (q, k, v, do)]
    host_out = [torch.empty_like(t).pin_memory() for t in host_in]
    dense, padded, _ = fns
    dev = q.device
    B = q.shape[0]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def step():
        main = torch.cuda.current_stream(dev)
        start = torch.cuda.Event()
        start.record(main)
        s_in.wait_event(start)
        s_out.wait_event(start)
        staged = []
        for b in range(B):
            with torch.cuda.stream(s_in):
                xs = [t[b:b + 1].to(dev, non_blocking=True) for t in host_in[:3]]
                ev_qkv = torch.cuda.Event()
                ev_qkv.record(s_in)  # the forward needs q, k, v only
                dob = host_in[3][b:b + 1].to(dev, non_blocking=True)
                ev_do = torch.cuda.Event()
                ev_do.record(s_in)
            staged.append((xs, dob, ev_qkv, ev_do))
        for b, (xs, dob, ev_qkv, ev_do) in enumerate(staged):
            main.wait_event(ev_qkv)
            qb, kb, vb = xs
            for t in xs:
                t.record_stream(main)
            qb.requires_grad_(), kb.requires_grad_(), vb.requires_grad_()
            if w["padded"]:
                lb = lens[b:b + 1]
                o = padded(qb, kb, vb, seq_lens_k=lb, seq_lens_q=lb, is_causal=w["causal"])
            else:
                o = dense(qb, kb, vb, is_causal=w["causal"])
            fwd_done = torch.cuda.Event()
            fwd_done.record(main)
            with torch.cuda.stream(s_out):  # O goes home while the backward runs
                s_out.wait_event(fwd_done)
                od = o.detach()
                od.record_stream(s_out)
                host_out[0][b:b + 1].copy_(od, non_blocking=True)
            main.wait_event(ev_do)
            dob.record_stream(main)
            o.backward(dob)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for dst, src in zip(host_out[1:], (qb.grad, kb.grad, vb.grad)):
                    src.record_stream(s_out)
                    dst[b:b + 1].copy_(src, non_blocking=True)
        main.wait_stream(s_out)

    nbytes = sum(t.numel() * t.element_size() for t in host_in)
    return step, nbytes, nbytes


def host_link_probe(device, nbytes: int = 64 << 20) -> dict:
    """What this box's host link gives: 64 MiB pinned copies host-to-device, device-to-host and both at once
    (CUDA events, best of three).  The end-to-end step streams in both directions at the same time, so a box on
    which the two directions do not overlap (both-at-once close to the sum of the two) shows in `e2e` directly."""
    h_in = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d_in = torch.empty(nbytes, dtype=torch.uint8, device=device)
    d_out = torch.empty(nbytes, dtype=torch.uint8, device=device)
    s1, s2 = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def run(up: bool, down: bool) -> float:
        best = float("inf")
        for _ in range(4):
            torch.cuda.synchronize(device)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            main = torch.cuda.current_stream(device)
            a.record(main)
            s1.wait_event(a)
            s2.wait_event(a)
            if up:
                with torch.cuda.stream(s1):
                    d_in.copy_(h_in, non_blocking=True)
            if down:
                with torch.cuda.stream(s2):
                    h_out.copy_(d_out, non_blocking=True)
            main.wait_stream(s1)
            main.wait_stream(s2)
            b.record(main)
            torch.cuda.synchronize(device)
            best = min(best, a.elapsed_time(b))
        return best

    up, down, both = run(True, False), run(False, True), run(True, True)
    return {"h2d_gbs": nbytes / up / 1e6, "d2h_gbs": nbytes / down / 1e6, "both_at_once_ms": both,
            "one_direction_ms": max(up, down), "mib": nbytes >> 20}


# ----------------------------------------------------------------------------- CPU baseline
def cpu_baseline(w: dict, budget_s: float = 20.0) -> dict:
    """Reference's own PyTorch CPU code (fp32, autograd) on a bounded sample of the workload:
    one batch element and as many heads as fit a ~1 GiB score matrix, repeated within the budget."""
    ref_path = os.path.join(ROOT, "baseline", "_ref", "triton_sigmoid", "sigmoid_reference.py")
    kind = "reference"
    if os.path.exists(ref_path):
        import importlib.util

        spec = importlib.util.spec_from_file_location("_ref_cpu_sigmoid_reference", ref_path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)

        def run(q, k, v, do, lens, causal):
            q, k, v = [t.clone().requires_grad_() for t in (q, k, v)]
            o = mod.sigmoid_attention_ref(q, k, v, seq_lens_k=lens, seq_lens_q=lens, upcast=True, causal=causal)
            o.backward(do)
    else:
        kind = "port"
        from oracle import sigattn_oracle as orc

        def run(q, k, v, do, lens, causal):
            orc.sigattn_forward(q, k, v, seq_lens_k=lens, seq_lens_q=lens, is_causal=causal)
            orc.sigattn_backward(q, k, v, do, seq_lens_k=lens, seq_lens_q=lens, is_causal=causal)

    N, D = w["N"], w["D"]
    Hs = max(1, min(w["H"], (1 << 28) // (N * N)))  # heads per pass: score matrix <= 2^28 elements
    g = torch.Generator().manual_seed(w["seed"])
    q, k, v, do = [torch.randn(1, N, Hs, D, generator=g) * w["std"] for _ in range(4)]
    lens = None
    f = 4.0 * Hs * float(N) ** 2 * D
    if w["padded"]:
        lens = torch.tensor([(w["lo"] + N) // 2], dtype=torch.int32)
        f = 4.0 * Hs * D * float(lens[0]) ** 2
    if w["causal"]:
        f /= 2
    run(q, k, v, do, lens, w["causal"])  # warm-up
    t0 = time.perf_counter()
    passes = 0
    while True:
        run(q, k, v, do, lens, w["causal"])
        passes += 1
        el = time.perf_counter() - t0
        if el > budget_s or passes >= 50:
            break
    return {"value": 3.5 * f * passes / el / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
            "sample": f"fp32 torch CPU forward+backward of 1 batch x {Hs} heads of the workload (N={N}, D={D}), "
                      f"{passes} passes in {el:.1f} s; nproc={os.cpu_count()}"}


# ----------------------------------------------------------------------------- main
# Other configurations recorded (device-timed, a few steps each) in `extra.workloads` of the JSON line.
EXTRA_WORKLOADS = ["cfg2-causal", "cfg3", "cfg3-causal", "cfg4", "sweep:512:64:bf16:dense:full",
                   "sweep:32768:64:bf16:dense:full", "sweep:8192:128:bf16:dense:full"]

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of the named kernel on the default
# workload (dense fp16, B=4, N=4096, H=16, D=64), from an `ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum
# --clock-control none -k regex:<kernel> -c 1` capture of this very launch; None = not captured for the
# current kernels.  Only reported for that workload on one GPU.
NCU_DRAM_BYTES_DEFAULT_WORKLOAD = {"sigattn_bwd_kernel": 201936384 + 93511424, "sigattn_fwd_kernel": 100867072 + 14927360}


class Dist:
    """torch.distributed when launched under torchrun, no-ops otherwise."""

    def __init__(self, device):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.device = device
        self.pg = None
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=device)
            self.pg = dist

    def barrier(self):
        if self.pg is not None:
            self.pg.barrier()

    def _reduce(self, x: float, op) -> float:
        if self.pg is None:
            return x
        t = torch.tensor([x], device=self.device, dtype=torch.float64)
        self.pg.all_reduce(t, op=op)
        return float(t.item())

    def max(self, x: float) -> float:
        return self._reduce(x, self.pg.ReduceOp.MAX if self.pg else None)

    def sum(self, x: float) -> float:
        return self._reduce(x, self.pg.ReduceOp.SUM if self.pg else None)

    def close(self):
        if self.pg is not None:
            self.pg.destroy_process_group()


def setup_workload(w, device, d: Dist):
    """Tensors of this rank: its own data (weak scaling) or its shard of the one problem (strong scaling)."""
    strong = bool(w.get("strong")) and d.world > 1
    if strong:
        from triton_sigmoid_b200.launcher import plan_shard, take_shard

        sh = plan_shard(w["B"], w["H"], d.world, d.rank)
        q, k, v, do, lens = make_data(w, device, 0)
        q, k, v, do = [take_shard(t, sh).contiguous() for t in (q, k, v, do)]
        if lens is not None:
            lens = take_shard(lens, sh, None).contiguous()
        wl = dict(w, B=sh.b1 - sh.b0, H=sh.h1 - sh.h0)
    else:
        q, k, v, do, lens = make_data(w, device, d.rank)
        wl = w
    for t in (q, k, v):
        t.requires_grad_()
    return wl, strong, q, k, v, do, lens


def measure_extra(name, fns, device, d: Dist, flush, pk) -> dict:
    """Forward and forward+backward of one more configuration, 3 warm-up + 3 timed steps each, device-timed,
    max over ranks, whole-job FLOPs."""
    w = parse_workload(name)
    wl, strong, q, k, v, do, lens = setup_workload(w, device, d)
    F_total = d.sum(fwd_flops(wl, lens))
    fwd_only, fwd_bwd = make_step(wl, fns, q, k, v, do, lens)
    ms_fb = d.max(timed(fwd_bwd, 3, 3, flush, d.barrier)) / 3
    ms_f = d.max(timed(fwd_only, 3, 3, flush, d.barrier)) / 3
    q.grad = k.grad = v.grad = None
    res = {"B_per_gpu": wl["B"], "N": w["N"], "H_per_gpu": wl["H"], "D": w["D"], "dtype": w["dtype"], "causal": w["causal"],
           "padded": w["padded"], "scaling": "strong" if strong else "weak",
           "fwd_tflops": F_total / (ms_f * 1e-3) / 1e12, "fwd_bwd_tflops": 3.5 * F_total / (ms_fb * 1e-3) / 1e12,
           "fwd_ms": ms_f, "fwd_bwd_ms": ms_fb}
    res["fwd_frac_of_peak"] = res["fwd_tflops"] / (pk["burst"] * d.world)
    res["fwd_bwd_frac_of_peak"] = res["fwd_bwd_tflops"] / (pk["burst"] * d.world)
    del q, k, v, do, lens, fwd_only, fwd_bwd
    torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-cpu"])
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-breakdown", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the extra.workloads record")
    ap.add_argument("--extra-workloads", default=None,
                    help="comma-separated workload names for the extra.workloads record instead of the default list "
                         "(e.g. a sequence-length sweep: sweep:512:64:bf16:dense:full,sweep:2048:64:bf16:dense:full)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    w = parse_workload(args.workload)
    pk = peaks()

    if args.impl == "reference-cpu":
        if rank != 0:
            return
        cb = cpu_baseline(w, budget_s=30.0)
        line = {"impl": "reference", "metric": "forward+backward TFLOP/s", "value": cb["value"], "unit": "TFLOP/s",
                "n_gpus": 0, "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": w["name"], "l2": "n/a (CPU)"}, "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU (there is no CPU path in this library)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    d = Dist(device)
    world = d.world

    try:
        fns = get_impl(args.impl)
    except Exception as e:  # reference arm only: the package could not be imported
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:300]}))
        d.close()
        return

    # strong-scaling workloads shard their (batch, head) units; the default workload is weak
    wl, strong, q, k, v, do, lens = setup_workload(w, device, d)
    F = fwd_flops(wl, lens)
    fwd_only, fwd_bwd = make_step(wl, fns, q, k, v, do, lens)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)  # > 126 MB L2
    F_total = d.sum(F)

    # ---- headline: forward+backward, device-resident
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_total = d.max(timed(fwd_bwd, args.steps, args.warmup, flush, d.barrier))
    clocks = sampler.stop() if rank == 0 else None
    ms_step = ms_total / args.steps
    value = 3.5 * F_total / (ms_step * 1e-3) / 1e12

    # ---- end to end with host buffers
    e2e_fn, bi, bo = e2e_step_factory(wl, fns, q, k, v, do, lens)
    e2e_steps = max(3, min(args.steps, 10))
    ms_e2e = d.max(timed(e2e_fn, e2e_steps, 3, flush, d.barrier)) / e2e_steps
    e2e = {"value": 3.5 * F_total / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": bi,
           "d2h_bytes_per_step": bo, "ms_per_step": ms_e2e,
           "how": "pinned host tensors; per batch element H2D (q,k,v, then dO), forward, backward, D2H (O during the backward, then the gradients) on three streams",
           # what the host link alone allows: both directions at once, nothing else in the step
           "pcie_bound_ms_at_50GBs": max(bi, bo) / 50e9 * 1e3}
    if rank == 0:
        e2e["host_link_probe"] = host_link_probe(device)

    breakdown = {}
    if not args.no_breakdown:
        ms_f = d.max(timed(fwd_only, args.steps, 3, flush, d.barrier)) / args.steps
        breakdown["fwd_tflops"] = F_total / (ms_f * 1e-3) / 1e12
        breakdown["fwd_ms"] = ms_f
        breakdown["fwd_bwd_tflops"] = value
        breakdown["bwd_only_tflops_est"] = 2.5 * F_total / (max(ms_step - ms_f, 1e-6) * 1e-3) / 1e12
        breakdown["fwd_frac_of_peak"] = breakdown["fwd_tflops"] / (pk["burst"] * world)
        breakdown["fwd_bwd_frac_of_peak"] = value / (pk["burst"] * world)

    line = {
        "metric": "forward+backward TFLOP/s (4BHN^2D fwd, x3.5 fwd+bwd)", "value": value, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
        "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": w["name"], "B_per_gpu": wl["B"], "N": w["N"], "H": wl["H"], "D": w["D"],
                   "causal": w["causal"], "padded": w["padded"], "global_batch": w["B"] if strong else w["B"] * world,
                   "parallelism": f"independent (batch, head) shards x{world}, no collective",
                   "l2": "256 MiB buffer zero-filled between timed steps (L2 flush)"},
        "library": fns[2],
        "clocks": clocks, "e2e": e2e, "breakdown": breakdown,
        "peak_tflops": {"value": pk["burst"], "source": pk["source"]},
    }

    if args.impl == "ours":
        from triton_sigmoid_b200.profiling import time_main_kernel

        kw = dict(seq_lens_q=lens, seq_lens_k=lens, is_causal=w["causal"], iters=max(5, min(args.steps, 20)), flush=flush)
        qd, kd, vd = q.detach(), k.detach(), v.detach()
        time_main_kernel("bwd", qd, kd, vd, do, **dict(kw, iters=3))
        kb = statistics.mean(time_main_kernel("bwd", qd, kd, vd, do, **kw))
        kf = statistics.mean(time_main_kernel("fwd", qd, kd, vd, **kw))
        elems = float(wl["B"]) * w["N"] * wl["H"] * w["D"]
        default_launch = w["name"] == "cfg2" and world == 1
        traffic_bwd = NCU_DRAM_BYTES_DEFAULT_WORKLOAD["sigattn_bwd_kernel"] if default_launch else None
        traffic_fwd = NCU_DRAM_BYTES_DEFAULT_WORKLOAD["sigattn_fwd_kernel"] if default_launch else None
        ach = 2.5 * F / (kb * 1e-3) / 1e12
        line["roofline"] = {"bound": "tensor", "kernel": "sigattn_bwd_kernel", "achieved": ach, "peak": pk["burst"],
                            "unit": "TFLOP/s", "frac": ach / pk["burst"], "traffic": traffic_bwd,
                            "algorithmic_bytes": 14.0 * elems,
                            "peak_source": f"{pk['source']} bf16 cuBLAS burst", "ms_per_launch": kb,
                            "fwd_kernel": {"traffic": traffic_fwd, "algorithmic_bytes": 8.0 * elems, "achieved": F / (kf * 1e-3) / 1e12, "frac": F / (kf * 1e-3) / 1e12 / pk["burst"],
                                           "ms_per_launch": kf},
                            # the same launches against the HBM roof (short sequences come near it: the
                            # arithmetic intensity of the forward is N/2 FLOP per byte)
                            "hbm": {"bwd_gbs": 14.0 * elems / (kb * 1e-3) / 1e9, "fwd_gbs": 8.0 * elems / (kf * 1e-3) / 1e9,
                                    "peak_gbs": pk["hbm_gbs"], "bwd_frac": 14.0 * elems / (kb * 1e-3) / 1e9 / pk["hbm_gbs"],
                                    "fwd_frac": 8.0 * elems / (kf * 1e-3) / 1e9 / pk["hbm_gbs"]}}
        # the other arm of the backward (two streaming kernels, no atomics), same launch, for the record
        ks = statistics.mean(time_main_kernel("bwd", qd, kd, vd, do, **dict(kw, split_bwd=True)))
        line["roofline"]["bwd_split_kernels"] = {"ms_per_launch_pair": ks, "achieved": 2.5 * F / (ks * 1e-3) / 1e12,
                                                 "frac": 2.5 * F / (ks * 1e-3) / 1e12 / pk["burst"]}
        # kernels of this library per timed step: forward, backward, dQ convert
        line["gpu_launches"] = 3 * args.steps
    else:
        line["impl"] = "reference"

    del q, k, v, do, fwd_only, fwd_bwd, e2e_fn
    torch.cuda.empty_cache()
    if not args.no_extra:
        extra = {}
        for name in (args.extra_workloads.split(",") if args.extra_workloads else EXTRA_WORKLOADS):
            if name == w["name"]:
                continue
            try:
                extra[name] = measure_extra(name, fns, device, d, flush, pk)
            except Exception as e:  # a configuration that does not fit or fails is recorded, not fatal
                extra[name] = {"error": f"{type(e).__name__}: {e}"[:200]}
                torch.cuda.empty_cache()
        line["extra"] = {"workloads": extra, "how": "3 warm-up + 3 timed steps each, CUDA events, L2 flushed between steps, max over ranks"}

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(w)

    if rank == 0:
        print(json.dumps(line))
    d.close()


if __name__ == "__main__":
    main()
