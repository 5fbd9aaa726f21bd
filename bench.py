#!/usr/bin/env python
"""Benchmark of the GLA forward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c5|k32]

Headline (the JSON line's `value`): one forward of the operator over one batch of seeded synthetic inputs with the
benchmark's shapes and value distributions (no dataset or checkpoint is involved): workload c3 = B4 H12 T6400
(80x80 patch grid), K=V=64, fp16, scan direction alternating per call.  A timed step is `inner` such forwards back to
back (`timing.forwards_per_step`, chosen so that the timed region lasts about a second and the driver's clock can
see it); `ms_per_step` is per step, `roofline.kernel_us` per forward.  `value` is tokens/s (sequence positions, all
heads) with inputs resident in HBM; `e2e` is the same metric through the public Python call with host buffers:
pinned host -> device copies of q,k,v,g and the device -> host read of the output are inside the timed region.
With N > 1 (torchrun, one rank per GPU) every rank runs the same per-GPU workload on its own batch (weak scaling, no
collective on the data path); the time is the max over ranks and `ranks` names each rank's own time and clock.

`extra` (single-GPU runs): the other configurations (c2, c5, K = 32 heads), the call the backbone makes (fused
RMSNorm * w * silu(gate) epilogue, raw gate logits, strided views of one packed projection), two more CPU baselines
and, where Triton runs, flash-linear-attention's own chunk_gla on the same GPU as a comparator.

`--impl reference` times the reference's CPU path for this operator (its pure-PyTorch token recurrence, restated in
oracle/gla_ref.py) on the host cores, on the same workload.  `cpu_baseline` (the same recurrence, timed beside the
GPU run) is reported by single-GPU runs only.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from gtr_b200 import workloads  # noqa: E402

FALLBACK_HBM_GBS = 6650.0

WORKLOADS = {
    "c2": "configs[1]: B8 H6 T1600 K=V=64 fp16, four scan orders",
    "c3": "configs[2]: B4 H12 T6400 K=V=64 fp16, scan direction alternating per call",
    "c5": "configs[4]: B2 H8 T8192 K=V=64 fp16 stress gates",
    "k32": "configs[2]'s shape with the released models' key heads: B4 H12 T6400 K=32 V=64 fp16",
}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def ncu_traffic_bytes(workload):
    """DRAM bytes per launch of the operator kernel from the committed ncu figures (None if absent)."""
    try:
        with open(os.path.join(ROOT, "profiles", "gla_fwd_kernel.json")) as f:
            return float(json.load(f)[workload]["dram_bytes_per_launch"])
    except Exception:
        return None


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            p = [x.strip() for x in line.split(",")]
            if len(p) < 7:
                continue
            try:
                sm.append(float(p[0]))
                mx.append(float(p[1]))
            except ValueError:
                continue
            for n, v in zip(names, p[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def percentiles(xs):
    xs = sorted(xs)
    pick = lambda f: xs[min(len(xs) - 1, int(f * len(xs)))]
    return {"min": xs[0], "median": statistics.median(xs), "p95": pick(0.95), "mean": statistics.mean(xs)}


def workload_config(name, B, H, T, K):
    """Names the workload; identical for both arms of the benchmark."""
    return {"workload": WORKLOADS[name], "B": B, "H": H, "T": T, "K": K, "V": 64,
            "grid": list(workloads.CONFIGS[name]["grid"]), "seed": 0,
            "per_gpu": "every rank runs this workload on its own seeded batch"}


# ------------------------------------------------------------------------------------------------- CPU baselines
def time_cpu(fn, budget_s, min_runs=3, max_runs=20):
    fn()                                                        # warm-up
    times, t_start = [], time.perf_counter()
    while len(times) < min_runs or (time.perf_counter() - t_start < budget_s and len(times) < max_runs):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    return statistics.median(times), len(times)


def cpu_port_tokens_per_s(cfg, budget_s=12.0, max_tokens=None):
    """The reference's CPU path (pure-PyTorch fp32 token recurrence) on a bounded sample."""
    from oracle import gla_ref
    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v, g = workloads.config_inputs(cfg, seed=0, dtype=torch.float32)
    if max_tokens is not None:
        q, k, v, g = (x[:, :max_tokens] for x in (q, k, v, g))
    B, T = q.shape[:2]
    med, n = time_cpu(lambda: gla_ref.recurrent_gla(q, k, v, g), budget_s)
    return B * T / med, med, n, torch.get_num_threads(), (B, T)


def more_cpu_baselines(budget_s=4.0):
    """configs[0] (B1 H6 T1600, fp32, CPU) through two more pure-PyTorch paths: flash-linear-attention's own
    naive_recurrent_gla (the third-party recurrence the reference's tests lean on) and the chunkwise fp32
    formulation of the oracle."""
    from oracle import gla_ref
    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v, g = workloads.config_inputs("c1", seed=0, dtype=torch.float32)
    B, T = q.shape[:2]
    out = {"shape": "configs[0]: B1 H6 T1600 K=V=64 fp32", "cores": torch.get_num_threads(), "unit": "tokens/s"}
    med, n = time_cpu(lambda: gla_ref.chunk_gla(q, k, v, g), budget_s)
    out["chunkwise_fp32"] = {"value": B * T / med, "runs": n, "s_per_run": med}
    try:
        from fla.ops.gla.naive import naive_recurrent_gla
        med, n = time_cpu(lambda: naive_recurrent_gla(q, k, v, g), budget_s)
        out["fla_naive_recurrent_gla"] = {"value": B * T / med, "runs": n, "s_per_run": med}
    except Exception as e:
        out["fla_naive_recurrent_gla"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    return out


def fla_triton_comparator(timeout_s=150, backward=False):
    """flash-linear-attention's Triton chunk_gla (what the reference falls back to at K = 64) on this GPU, c3 shape.
    Run in a child process with a time limit (a Triton build can take a while); context only, never the target."""
    code = r"""
import json, sys, torch
sys.path.insert(0, %r)
from gtr_b200 import workloads
from fla.ops.gla import chunk_gla
q, k, v, g = (x.cuda() for x in workloads.config_inputs('c3'))
for _ in range(3): chunk_gla(q, k, v, g)
torch.cuda.synchronize()
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
e0.record()
for _ in range(20): o, _ = chunk_gla(q, k, v, g)
e1.record(); torch.cuda.synchronize()
us = e0.elapsed_time(e1) * 1000 / 20
res = {'us_per_forward': us, 'tokens_per_s': q.shape[0] * q.shape[1] / (us * 1e-6), 'finite': bool(torch.isfinite(o).all())}
print(json.dumps(res), flush=True)
if not %r: sys.exit(0)
leaves = [x.clone().requires_grad_(True) for x in (q, k, v, g)]
do = torch.randn_like(v)
def both():
    o, _ = chunk_gla(*leaves)
    o.backward(do)
for _ in range(3): both()
torch.cuda.synchronize()
e0.record()
for _ in range(10): both()
e1.record(); torch.cuda.synchronize()
res['us_forward_and_backward'] = e0.elapsed_time(e1) * 1000 / 10
print(json.dumps(res), flush=True)
""" % (ROOT, bool(backward))
    try:
        run = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=timeout_s)
        lines = [l for l in run.stdout.strip().splitlines() if l.startswith("{")]
        if not lines:
            return {"unavailable": (run.stderr.strip().splitlines() or ["failed"])[-1][:200]}
        res = json.loads(lines[-1])          # the forward figure stands even if the backward leg fails to build
        res["what"] = "fla.ops.gla.chunk_gla (Triton), c3 shape, 20 forwards back to back, inputs L2-resident between calls"
        if backward:
            res["what"] += "; then 10 forward + backward pairs through its autograd"
        return res
    except subprocess.TimeoutExpired:
        return {"unavailable": f"no result within {timeout_s} s"}
    except Exception as e:
        return {"unavailable": f"{type(e).__name__}: {e}"[:200]}


def run_reference(args, rank, world):
    if rank != 0:
        return
    from oracle import gla_ref
    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v, g = workloads.config_inputs(args.workload, seed=0, dtype=torch.float32)
    B, T, H, K = q.shape
    # one step = one forward over a bounded sample of the workload: the first `tok` tokens of every sequence, sized
    # so that the K steps together stay near a minute on the host cores (the recurrence's tokens/s does not depend
    # on the length)
    steps = args.steps
    tok = max(64, min(T, 1600, int(2.5e6 / (steps * B)) // 64 * 64))
    q, k, v, g = (x[:, :tok].contiguous() for x in (q, k, v, g))
    for _ in range(max(args.warmup, 1)):
        gla_ref.recurrent_gla(q[:, :128], k[:, :128], v[:, :128], g[:, :128])
    t0 = time.perf_counter()
    for _ in range(steps):
        gla_ref.recurrent_gla(q, k, v, g)
    dt = (time.perf_counter() - t0) / steps
    value = B * tok / dt
    threads = torch.get_num_threads()
    sample = f"first {tok} of {T} tokens of every sequence (B{B} H{H}), fp32 PyTorch token recurrence"
    line = {
        "impl": "reference", "metric": "gla_fwd_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, B, H, T, K),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------- backbone
def backbone_flops_per_image(dim=768, depth=12, heads=12, tokens=8192, inter=3072, low_rank=16):
    """Dense FLOPs of one image through the blocks (GEMMs, depthwise conv, GLA recurrence count)."""
    gemm = 2 * (dim * (4 * dim + low_rank) + low_rank * dim + dim * dim + 3 * dim * inter)
    gla = heads * (4 * 64 * 64 + 4 * 64 * 64)        # recurrence 4KV per token-head + chunk-local scores/products
    conv = 2 * 9 * inter
    return depth * tokens * (gemm + gla + conv)


def run_backbone(args, rank, local_rank, world, dist):
    """configs[3]: 12 blocks, dim 768, 12 heads of 64, Spatial SwiGLU hidden 3072, 1024x2048 images
    (64x128 = 8192 tokens), batch 32 in total sharded across the ranks (strong scaling), random-init
    weights, pixels ~ U(0,1).  One CUDA graph per rank; no collective on the data path."""
    from gtr_b200.backbone import GTRBackbone, GraphedBackbone
    dev = torch.device("cuda", local_rank)
    total_batch = args.backbone_batch
    if total_batch % world:
        return {"unavailable": f"batch {total_batch} does not divide over {world} ranks"}
    b = total_batch // world
    torch.manual_seed(0)
    model = GTRBackbone().half().to(dev).eval().convert_to_deploy()
    runner = GraphedBackbone(model)
    img = torch.rand(b, 3, 1024, 2048, generator=torch.Generator().manual_seed(rank)).half().to(dev)
    steps = args.backbone_steps
    for _ in range(3):
        out = runner(img)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = runner(img)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    finite = bool(torch.isfinite(out[-1]).all())
    sec = ms.item() * 1e-3
    img_s = total_batch * steps / sec
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak_tf, kind = float(json.load(f)["bf16_tflops_sustained"]), "of measured"
    except Exception:
        peak_tf, kind = 1400.0, "of fallback"
    tf_per_gpu = backbone_flops_per_image() * img_s / world / 1e12
    return {"metric": "backbone_img_per_s", "value": img_s, "unit": "img/s", "n_gpus": world, "scaling": "strong",
            "batch_total": total_batch, "batch_per_gpu": b, "steps": steps, "ms_per_step": ms.item() / steps,
            "image": [1024, 2048], "tokens": 8192, "finite": finite, "gla_launches_per_step": 12,
            "scan_cycle": "row, row_rev, col, col_rev per block (vit_adapter.py:896-898)", "seed": 0,
            "roofline": {"bound": "tensor", "achieved": tf_per_gpu, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": tf_per_gpu / peak_tf, "peak_kind": kind}}


# ------------------------------------------------------------------------------------------------- operator timing
def time_forwards(fn, steps, inner, warmup_steps, sync):
    """`steps` timed steps of `inner` forwards each; CUDA events around every step on the launching stream.
    Returns (total ms over the timed region, per-forward microseconds of every step)."""
    i = 0
    for _ in range(warmup_steps * inner):
        fn(i)
        i += 1
    sync()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    t0.record()
    for s in range(steps):
        evs[s][0].record()
        for _ in range(inner):
            fn(i)
            i += 1
        evs[s][1].record()
    t1.record()
    sync()
    return t0.elapsed_time(t1), [a.elapsed_time(b) * 1e3 / inner for a, b in evs]


def device_sets(name, dev, seed0, min_bytes=160e6):
    """Enough distinct input sets of a workload that one pass over them exceeds the L2."""
    first = workloads.config_inputs(name, seed=seed0)
    in_bytes = sum(x.numel() * 2 for x in first)
    n_sets = max(2, int(-(-2.2 * 126 * 1024 * 1024 // in_bytes))) if in_bytes < min_bytes else 3
    host = [first] + [workloads.config_inputs(name, seed=seed0 + i) for i in range(1, n_sets)]
    return host, [tuple(x.to(dev) for x in s) for s in host], in_bytes


def extra_workload(gtr_b200, name, dev, peak):
    """Short device-resident run of another configuration: tokens/s and fraction of the HBM roofline."""
    c = workloads.CONFIGS[name]
    host, sets, in_bytes = device_sets(name, dev, seed0=50)
    B, T, H, K = host[0][0].shape
    ws = gtr_b200.make_workspace(B, T, H, dev)
    o = torch.empty(B, T, H, 64, dtype=torch.float16, device=dev)
    scale = K ** -0.5
    fn = lambda i: gtr_b200.chunk_gla_run(*sets[i % len(sets)], scale, ws, o, direction=i % 4, grid_hw=c["grid"])
    total_ms, per = time_forwards(fn, steps=40, inner=5, warmup_steps=3, sync=torch.cuda.synchronize)
    gtr_b200.check_status(ws)
    us = statistics.mean(per)
    algo = B * T * H * workloads.algorithmic_bytes_per_token_head(K)
    return {"workload": WORKLOADS[name], "tokens_per_s": B * T * 200 / (total_ms * 1e-3), "kernel_us": percentiles(per),
            "algorithmic_bytes_per_launch": algo, "roofline_frac": algo / (us * 1e-6) / 1e9 / peak,
            "input_sets": len(sets), "finite": bool(torch.isfinite(o).all())}


def extra_gradient(gtr_b200, name, dev):
    """The operator's gradient (gla_b200_backward: dq, dk, dv, dg) on a configuration's shape: time per call and one
    sequence of it checked against the float64 oracle."""
    from oracle import gla_bwd_ref
    q, k, v, g = (x.to(dev) for x in workloads.config_inputs(name, seed=77))
    B, T, H, K = q.shape
    do = (torch.randn(B, T, H, 64, generator=torch.Generator().manual_seed(78)) / 8).half().to(dev)
    fn = lambda i: gtr_b200.chunk_gla_backward(q, k, v, g, do)
    total_ms, per = time_forwards(fn, steps=10, inner=2, warmup_steps=3, sync=torch.cuda.synchronize)
    n = min(T, 512)
    got = gtr_b200.chunk_gla_backward(q[:1, :n], k[:1, :n], v[:1, :n], g[:1, :n], do[:1, :n])
    want = gla_bwd_ref.recurrent_gla_backward(q[:1, :n].cpu(), k[:1, :n].cpu(), v[:1, :n].cpu(), g[:1, :n].cpu(), do[:1, :n].cpu())
    rel = [float((a.double().cpu() - b).norm() / b.norm()) for a, b in zip(got[:4], want[:4])]
    return {"workload": WORKLOADS[name], "us_per_call": percentiles(per), "tokens_per_s": B * T / (statistics.mean(per) * 1e-6),
            "kernels_per_call": 4 if T >= 512 and 3 * B * H < 600 else 2,
            "rel_l2_vs_oracle": dict(zip(("dq", "dk", "dv", "dg"), rel)), "checked": f"first {n} tokens of sequence 0"}


def extra_gated(gtr_b200, dev, peak, B, T, H, grid, label):
    """The call a backbone block makes: q, k, v, output gate and raw gate logits are strided views of one packed
    projection buffer, logsigmoid(x)/16 is applied in the kernel, RMSNorm * w * silu(gate) is fused."""
    D = H * 64
    gen = torch.Generator(device=dev).manual_seed(7)
    n_sets = 2 if B * T * 5 * D * 2 > 200e6 else 3
    packs = []
    for _ in range(n_sets):
        p = torch.randn(B, T, 5 * D, generator=gen, device=dev, dtype=torch.float16)
        p[..., :2 * D] *= 0.125
        packs.append(p)
    w = (torch.rand(64, generator=gen, device=dev) + 0.5).half()
    ws = gtr_b200.make_workspace(B, T, H, dev)
    y = torch.empty(B, T, H, 64, dtype=torch.float16, device=dev)
    view = lambda p, i: p[..., i * D:(i + 1) * D].unflatten(-1, (H, 64))

    def fn(i):
        p = packs[i % n_sets]
        gtr_b200.chunk_gla_run_gated(view(p, 0), view(p, 1), view(p, 2), view(p, 4), view(p, 3), w, 0.125, 1e-5, ws, y,
                                     16.0, direction=i % 4, grid_hw=grid)
    total_ms, per = time_forwards(fn, steps=20, inner=4, warmup_steps=2, sync=torch.cuda.synchronize)
    gtr_b200.check_status(ws)
    us = statistics.mean(per)
    algo = B * T * H * workloads.algorithmic_bytes_per_token_head(64, gated=True)
    return {"call": label, "B": B, "T": T, "H": H, "tokens_per_s": B * T * 80 / (total_ms * 1e-3),
            "kernel_us": percentiles(per), "algorithmic_bytes_per_launch": algo,
            "roofline_frac": algo / (us * 1e-6) / 1e9 / peak, "finite": bool(torch.isfinite(y).all())}


def run_ours(args, rank, local_rank, world):
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the operator)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # stdout carries the one JSON line.  NCCL prints its version banner straight to stdout when it first comes up
        # (NCCL_DEBUG=VERSION is set on some boxes), so the descriptor points at stderr while it does.
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
    import gtr_b200
    from oracle import gla_ref

    if args.profile_backbone:
        # a short run for a profiler: the backbone leg alone (three warm-up passes, graph capture, `--backbone-steps` replays)
        out = run_backbone(args, rank, local_rank, world, dist)
        if rank == 0:
            print(json.dumps({"profile_backbone": out}))
        return

    name = args.workload
    grid = workloads.CONFIGS[name]["grid"]
    host_sets, dev_sets, in_bytes = device_sets(name, dev, seed0=1000 * rank)
    n_sets = len(dev_sets)
    B, T, H, K = host_sets[0][0].shape
    scale = K ** -0.5
    pinned = [tuple(x.pin_memory() for x in s) for s in host_sets]
    ws = gtr_b200.make_workspace(B, T, H, dev)
    o = torch.empty(B, T, H, 64, dtype=torch.float16, device=dev)
    o_host = torch.empty(B, T, H, 64, dtype=torch.float16).pin_memory()
    stage = tuple(torch.empty_like(x, device=dev) for x in host_sets[0])
    out_bytes = o.numel() * 2
    algo_bytes = B * T * H * workloads.algorithmic_bytes_per_token_head(K)

    def step(i, tensors=None):
        q, k, v, g = tensors if tensors is not None else dev_sets[i % n_sets]
        gtr_b200.chunk_gla_run(q, k, v, g, scale, ws, o, direction=i % 4, grid_hw=grid)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.profile_backward > 0:
        # a short run for a profiler: the gradient call on the workload's shape
        q, k, v, g = dev_sets[0]
        do = torch.randn(B, T, H, 64, device=dev).half()
        for _ in range(args.warmup + args.profile_backward):
            gtr_b200.chunk_gla_backward(q, k, v, g, do)
        torch.cuda.synchronize()
        if rank == 0:
            print(json.dumps({"profile_backward": args.profile_backward, "warmup_calls": args.warmup,
                              "config": workload_config(args.workload, B, H, T, K)}))
        return

    if args.profile_forwards > 0:
        # a short run for a profiler: the same forwards on the same inputs, no one-second warm-up, nothing else
        for i in range(args.warmup + args.profile_forwards):
            step(i)
        torch.cuda.synchronize()
        gtr_b200.check_status(ws)
        if rank == 0:
            print(json.dumps({"profile_forwards": args.profile_forwards, "warmup_forwards": args.warmup,
                              "config": workload_config(args.workload, B, H, T, K)}))
        return

    # ---- device-resident timing.  Warm-up: at least `warmup` steps and one second under load (clocks ramp);
    # the clock sampler then runs across the timed region only.
    t_w = time.perf_counter()
    i = 0
    while i < max(args.warmup, 3) or time.perf_counter() - t_w < 1.0:
        step(i)
        i += 1
        if i % 64 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for j in range(20):
        step(j)
    e1.record()
    torch.cuda.synchronize()
    est_us = max(e0.elapsed_time(e1) * 1e3 / 20, 1.0)
    # forwards per step so that the K timed steps last about a second (at least half a second)
    inner = max(1, min(2048, int(-(-1.0e6 // (est_us * args.steps)))))
    if world > 1:                                   # the ranks must agree
        t = torch.tensor([inner], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        inner = int(t.item())
    sampler = ClockSampler(local_rank)
    total_ms, per_fwd_us = time_forwards(step, args.steps, inner, 0, barrier)
    clocks = sampler.stop()
    gtr_b200.check_status(ws)

    # ---- end to end: pinned host inputs -> device, forward, output -> host, every step.  The three legs of a
    # step run on three streams over two sets of staging buffers, so that step i+1's inputs come in and step
    # i-1's outputs go out (PCIe is full duplex) while step i computes; every step still moves all of its bytes.
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    stages = (stage, tuple(torch.empty_like(x) for x in stage))
    outs = (o, torch.empty_like(o))
    o_hosts = (o_host, torch.empty_like(o_host).pin_memory())
    computed = [None, None]       # event: the kernel that read stages[j] / wrote outs[j] has finished
    drained = [None, None]        # event: outs[j] has been copied to the host

    def e2e_step(i):
        j = i & 1
        src = pinned[i % n_sets]
        with torch.cuda.stream(s_in):
            if computed[j] is not None:
                s_in.wait_event(computed[j])
            for d, s_ in zip(stages[j], src):
                d.copy_(s_, non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record(s_in)
        main.wait_event(arrived)
        if drained[j] is not None:
            main.wait_event(drained[j])
        q, k, v, g = stages[j]
        gtr_b200.chunk_gla_run(q, k, v, g, scale, ws, outs[j], direction=i % 4, grid_hw=grid)
        computed[j] = torch.cuda.Event()
        computed[j].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(computed[j])
            o_hosts[j].copy_(outs[j], non_blocking=True)
            drained[j] = torch.cuda.Event()
            drained[j].record(s_out)

    def e2e_join():
        main.wait_stream(s_in)
        main.wait_stream(s_out)

    for i in range(2):
        e2e_step(i)
    e2e_join()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(10, min(args.steps, 40))
    s_in.wait_stream(main)
    s_out.wait_stream(main)
    e0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    e2e_join()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    gtr_b200.check_status(ws)
    # the last step's host-side output is the operator's output for that step's inputs
    last = e2e_steps - 1
    step(last, dev_sets[last % n_sets])
    torch.cuda.synchronize()
    e2e_ok = bool(torch.allclose(o_hosts[last & 1].float(), o.float().cpu(), rtol=0.0, atol=2e-3))

    # ---- max over ranks, and every rank's own figures
    mine = torch.tensor([total_ms, e2e_ms, statistics.mean(per_fwd_us), clocks.get("sm_mhz") or 0.0],
                        dtype=torch.float64, device=dev)
    if world > 1:
        gathered = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        allr = torch.stack(gathered)
    else:
        allr = mine[None]
    total_ms, e2e_ms, kern_us = allr[:, 0].max().item(), allr[:, 1].max().item(), allr[:, 2].max().item()
    ranks = [{"rank": r, "kernel_us": allr[r, 2].item(), "timed_region_ms": allr[r, 0].item(),
              "sm_mhz_median": allr[r, 3].item() or None} for r in range(world)]

    backbone = None
    if args.backbone_steps > 0:
        try:
            backbone = run_backbone(args, rank, local_rank, world, dist)
        except Exception as e:   # reported, never hidden: the operator line below stays valid
            backbone = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    loader = None
    if rank == 0 and not args.no_extras:
        # what the kernel's loading scheme alone streams on this GPU (reads only, nothing computed): the ceiling the
        # ring of five 32 KB stages per SM puts under any kernel built on it
        try:
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            p4 = gtr_b200.stream_probe(ctas=min(144, sms), tiles=4, chunks=33, device=dev)
            p3 = gtr_b200.stream_probe(ctas=min(96, sms), tiles=3, chunks=34, device=dev)
            loader = {"what": "TMA ring of 5 stages x 64-row x 128-byte tiles per CTA, one head per CTA, cold L2, nothing computed; "
                              "GB/s over the whole launch (start-up and tail included)",
                      "output_pass_like": {"ctas": p4["ctas"], "tiles_per_chunk": 4, "GBs": p4["GBs"], "us": p4["us"]},
                      "pre_pass_like": {"ctas": p3["ctas"], "tiles_per_chunk": 3, "GBs": p3["GBs"], "us": p3["us"]}}
        except Exception as e:      # reported, never hidden
            loader = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    if rank == 0:
        # ---- sanity: the timed output equals the oracle on a slice (cheap, outside the timed region)
        from oracle import c_oracle
        i = args.steps - 1
        hs = host_sets[i % n_sets]
        ref, _ = c_oracle.forward(hs[0][:1], hs[1][:1], hs[2][:1], hs[3][:1], direction=i % 4, grid_hw=grid)
        step(i, dev_sets[i % n_sets])
        torch.cuda.synchronize()
        m = gla_ref.error_metrics(ref, o[:1].float().cpu())
        parity = {"rel_l2": m["rel_l2"], "max_abs": m["max_abs"], "finite": m["finite"]}
        peak, peak_kind = measured_peak()
        # the CPU baselines and the extras are single-GPU-run figures: under a multi-rank launch the host cores and the
        # box are shared with the other ranks' processes
        cpu, extra = None, None
        if world == 1:
            cpu = cpu_port_tokens_per_s(name, max_tokens=1600)
            extra = {}
            if not args.no_extras:
                for wname in ("c2", "c5", "k32", "c3"):
                    if wname == name:
                        continue
                    try:
                        extra[wname] = extra_workload(gtr_b200, wname, dev, peak)
                    except Exception as e:
                        extra[wname] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
                try:
                    extra["gated"] = [
                        extra_gated(gtr_b200, dev, peak, 4, 6400, 12, (80, 80), "c3 shape, fused epilogue + raw gate logits"),
                        extra_gated(gtr_b200, dev, peak, 32, 8192, 12, (64, 128),
                                    "configs[3]'s per-block call at 1 GPU (B32 T8192 H12), fused epilogue + raw gate logits")]
                except Exception as e:
                    extra["gated"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
                try:
                    extra["gradient"] = [extra_gradient(gtr_b200, w, dev) for w in ("c3", "c2")]
                except Exception as e:
                    extra["gradient"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
                extra["cpu_baselines"] = more_cpu_baselines()
                extra["fla_triton_chunk_gla"] = (fla_triton_comparator(400, backward=True) if args.fla_backward
                                                 else fla_triton_comparator())
        tokens_per_step = B * T * inner
        value = world * tokens_per_step * args.steps / (total_ms * 1e-3)
        achieved = algo_bytes / (kern_us * 1e-6) / 1e9
        line = {
            "metric": "gla_fwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 in/out, f32 accumulate",
            "data": "synthetic",
            "config": workload_config(name, B, H, T, K),
            "timing": {"forwards_per_step": inner, "events": "CUDA events around every step on the launching stream",
                       "l2": f"inputs rotate over {n_sets} sets of {in_bytes / 1e6:.0f} MB each (L2 is 126 MB)"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "algorithmic_bytes_per_launch": algo_bytes,
                         "kernel_us": kern_us, "kernel_us_stats": percentiles(per_fwd_us),
                         "traffic": ncu_traffic_bytes(name), "loader_ceiling": loader},
            "cpu_baseline": None if cpu is None else {
                "value": cpu[0], "unit": "tokens/s", "cores": cpu[3], "kind": "port",
                "sample": f"first {cpu[4][1]} of {T} tokens of every sequence (B{cpu[4][0]} H{H}), fp32 PyTorch token "
                          f"recurrence, median of {cpu[2]} runs ({cpu[1]:.2f} s each)"},
            "e2e": {"value": world * B * T * e2e_steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes, "steps": e2e_steps,
                    "pipelined": "3 streams, 2 staging sets", "output_checked": e2e_ok},
            "gpu_launches": args.steps * inner, "clocks": clocks, "timed_region_s": total_ms * 1e-3, "ranks": ranks,
            "gpu": torch.cuda.get_device_name(dev), "host_cores": os.cpu_count(),
            "parity_check": parity, "backbone": backbone, "extra": extra,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--backbone-steps", type=int, default=5,
                    help="timed steps of the full synthetic backbone (reported under 'backbone'); 0 skips it")
    ap.add_argument("--backbone-batch", type=int, default=32,
                    help="images per backbone step over all ranks (32 = the named configuration; smaller for profiling)")
    ap.add_argument("--no-extras", action="store_true", help="skip the other workloads, CPU baselines and comparator")
    ap.add_argument("--profile-backbone", action="store_true",
                    help="run only the backbone leg (--backbone-batch, --backbone-steps) and exit (for ncu)")
    ap.add_argument("--profile-forwards", type=int, default=0,
                    help="run only warmup + N forwards of the workload (for ncu) and exit")
    ap.add_argument("--fla-backward", action="store_true",
                    help="also time the Triton comparator's forward + backward (its kernels take minutes to build)")
    ap.add_argument("--profile-backward", type=int, default=0,
                    help="run this many gradient calls (gla_b200_backward) on the workload after --warmup calls, then exit")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    args = ap.parse_args()
    rank, local_rank, world = dist_env()
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
