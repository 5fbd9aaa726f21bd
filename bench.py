#!/usr/bin/env python
"""Benchmark of the GLA forward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c5]

A step is one forward of the operator over one batch of seeded synthetic inputs with the
benchmark's shapes and value distributions (no dataset or checkpoint is involved):
workload c3 = B4 H12 T6400 (80x80 patch grid), K=V=64, fp16, scan direction alternating per
call.  `value` is tokens/s (sequence positions, all heads) with inputs resident in HBM;
`e2e` is the same metric through the public Python call with host buffers: pinned host ->
device copies of q,k,v,g and the device -> host read of the output are inside the timed
region.  With N > 1 (torchrun, one rank per GPU) every rank runs the same per-GPU workload
on its own batch (weak scaling, no collective on the data path); the time is the max over
ranks.  `--impl reference` times the reference's CPU path for this operator (its pure-PyTorch
token recurrence, restated in oracle/gla_ref.py) on the host cores, on the same workload.
`cpu_baseline` (the same recurrence, timed beside the GPU run) is reported by single-GPU runs only.
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

ALGO_BYTES_PER_TOKEN_HEAD = 640          # fp16 q,k,g (3*64*2) + v (64*2) read, o (64*2) written
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126 * 1024 * 1024

WORKLOADS = {
    "c2": dict(cfg="c2", grid=(40, 40), desc="configs[1]: B8 H6 T1600 K=V=64 fp16, four scan orders"),
    "c3": dict(cfg="c3", grid=(80, 80), desc="configs[2]: B4 H12 T6400 K=V=64 fp16, scan direction alternating per call"),
    "c5": dict(cfg="c5", grid=(64, 128), desc="configs[4]: B2 H8 T8192 K=V=64 fp16 stress gates"),
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
    """DRAM bytes per launch from the committed ncu summary of this workload (None if absent)."""
    path = os.path.join(ROOT, "profiles", f"gla_fwd_kernel_{workload}.md")
    try:
        for line in open(path):
            if line.startswith("dram_bytes_per_launch:"):
                return float(line.split(":")[1].split()[0])
    except Exception:
        pass
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


def make_sets(cfg, n_sets, seed0):
    from oracle import gla_ref
    return [gla_ref.config_inputs(cfg, seed=seed0 + i) for i in range(n_sets)]


def workload_config(w, B, H, T, n_sets=None, in_bytes=None):
    c = {"workload": w["desc"], "B": B, "H": H, "T": T, "K": 64, "V": 64, "grid": list(w["grid"]),
         "per_gpu": "every rank runs this workload on its own seeded batch"}
    if n_sets is not None:
        c["l2"] = f"inputs rotate over {n_sets} sets of {in_bytes / 1e6:.0f} MB each (L2 is 126 MB)"
    return c


def cpu_port_tokens_per_s(cfg, budget_s=12.0, max_tokens=None):
    """The reference's CPU path (pure-PyTorch fp32 token recurrence) on a bounded sample."""
    from oracle import gla_ref
    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v, g = gla_ref.config_inputs(cfg, seed=0, dtype=torch.float32)
    if max_tokens is not None:
        q, k, v, g = (x[:, :max_tokens] for x in (q, k, v, g))
    B, T = q.shape[:2]
    gla_ref.recurrent_gla(q[:, :64], k[:, :64], v[:, :64], g[:, :64])        # warm-up
    times = []
    t_start = time.perf_counter()
    while len(times) < 3 or (time.perf_counter() - t_start < budget_s and len(times) < 20):
        t0 = time.perf_counter()
        gla_ref.recurrent_gla(q, k, v, g)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return B * T / med, med, len(times), torch.get_num_threads(), (B, T)


def run_reference(args, rank, world):
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    from oracle import gla_ref
    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v, g = gla_ref.config_inputs(w["cfg"], seed=0, dtype=torch.float32)
    B, T, H, _ = q.shape
    # one step = one forward over a bounded sample of the workload: the first `tok` tokens of every sequence
    tok = min(T, 1600)
    q, k, v, g = (x[:, :tok].contiguous() for x in (q, k, v, g))
    for _ in range(max(args.warmup, 1)):
        gla_ref.recurrent_gla(q[:, :128], k[:, :128], v[:, :128], g[:, :128])
    t0 = time.perf_counter()
    for _ in range(args.steps):
        gla_ref.recurrent_gla(q, k, v, g)
    dt = (time.perf_counter() - t0) / args.steps
    value = B * tok / dt
    threads = torch.get_num_threads()
    sample = f"first {tok} of {T} tokens of every sequence (B{B} H{H}), fp32 PyTorch token recurrence"
    line = {
        "impl": "reference", "metric": "gla_fwd_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, B, H, T),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


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
            "roofline": {"bound": "tensor", "achieved": tf_per_gpu, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": tf_per_gpu / peak_tf, "peak_kind": kind}}


def run_ours(args, rank, local_rank, world):
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the operator)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    import gtr_b200
    from oracle import gla_ref

    w = WORKLOADS[args.workload]
    grid = w["grid"]
    n_sets = 3
    host_sets = make_sets(w["cfg"], n_sets, seed0=1000 * rank)
    B, T, H, _ = host_sets[0][0].shape
    scale = 64 ** -0.5
    dev_sets = [tuple(x.to(dev) for x in s) for s in host_sets]
    pinned = [tuple(x.pin_memory() for x in s) for s in host_sets]
    ws = gtr_b200.make_workspace(B, T, H, dev)
    o = torch.empty(B, T, H, 64, dtype=torch.float16, device=dev)
    o_host = torch.empty(B, T, H, 64, dtype=torch.float16).pin_memory()
    stage = tuple(torch.empty_like(x, device=dev) for x in host_sets[0])
    in_bytes = sum(x.numel() * 2 for x in host_sets[0])
    out_bytes = o.numel() * 2
    algo_bytes = B * T * H * ALGO_BYTES_PER_TOKEN_HEAD

    def step(i, tensors):
        q, k, v, g = tensors
        gtr_b200.chunk_gla_run(q, k, v, g, scale, ws, o, direction=i % 4, grid_hw=grid)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: CUDA events around every launch on the launching stream.
    # The clock sampler runs from the warm-up on (at least `warmup` steps and one second under
    # load, so that clocks have ramped) through the timed region.
    sampler = ClockSampler(local_rank) if rank == 0 else None
    t_w = time.perf_counter()
    i = 0
    while i < max(args.warmup, 3) or time.perf_counter() - t_w < 1.0:
        step(i, dev_sets[i % n_sets])
        i += 1
        if i % 64 == 0:
            torch.cuda.synchronize()
    barrier()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    t_all0, t_all1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_all0.record()
    for i in range(args.steps):
        evs[i][0].record()
        step(i, dev_sets[i % n_sets])
        evs[i][1].record()
    t_all1.record()
    barrier()
    total_ms = t_all0.elapsed_time(t_all1)
    kernel_ms = [a.elapsed_time(b) for a, b in evs]
    clocks = sampler.stop() if sampler else None
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
    e2e_steps = min(args.steps, 10)
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

    # ---- max over ranks
    times = torch.tensor([total_ms, e2e_ms, statistics.mean(kernel_ms)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, kern_ms = times.tolist()

    # ---- sanity: the timed output equals the oracle on a slice (cheap, outside the timed region)
    backbone = None
    if args.backbone_steps > 0:
        try:
            backbone = run_backbone(args, rank, local_rank, world, dist)
        except Exception as e:   # reported, never hidden: the operator line below stays valid
            backbone = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    if rank == 0:
        from oracle import c_oracle
        i = args.steps - 1
        hs = host_sets[i % n_sets]
        ref, _ = c_oracle.forward(hs[0][:1], hs[1][:1], hs[2][:1], hs[3][:1], direction=i % 4, grid_hw=grid)
        step(i, dev_sets[i % n_sets])
        torch.cuda.synchronize()
        m = gla_ref.error_metrics(ref, o[:1].float().cpu())
        parity = {"rel_l2": m["rel_l2"], "max_abs": m["max_abs"], "finite": m["finite"]}
        # the CPU baseline is a single-GPU-run figure: under a multi-rank launch the host cores are shared with the
        # other ranks' processes and the number means nothing
        cpu = cpu_port_tokens_per_s(w["cfg"], max_tokens=1600) if world == 1 else None
        peak, peak_kind = measured_peak()
        tokens_per_step = B * T
        value = world * tokens_per_step * args.steps / (total_ms * 1e-3)
        achieved = algo_bytes / (kern_ms * 1e-3) / 1e9
        line = {
            "metric": "gla_fwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 in/out, f32 accumulate",
            "data": "synthetic",
            "config": workload_config(w, B, H, T, n_sets, in_bytes),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "algorithmic_bytes_per_launch": algo_bytes,
                         "kernel_us": kern_ms * 1e3, "traffic": ncu_traffic_bytes(args.workload)},
            "cpu_baseline": None if cpu is None else {
                "value": cpu[0], "unit": "tokens/s", "cores": cpu[3], "kind": "port",
                "sample": f"first {cpu[4][1]} of {T} tokens of every sequence (B{cpu[4][0]} H{H}), fp32 PyTorch token "
                          f"recurrence, median of {cpu[2]} runs ({cpu[1]:.2f} s each)"},
            "e2e": {"value": world * tokens_per_step * e2e_steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes, "steps": e2e_steps,
                    "pipelined": "3 streams, 2 staging sets", "output_checked": e2e_ok},
            "gpu_launches": args.steps, "clocks": clocks, "parity_check": parity, "backbone": backbone,
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
