#!/usr/bin/env python
"""Benchmark of the headline metric: Mrays/s of one training step
(volume_render forward + MSE + backward into data.grad) on the sparse-shell
SH-degree-2 scene with 2^20 rays per step ("config 4"), on 1..8 B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Under torchrun (N > 1) every rank holds the whole tree and renders its own
2^20 rays per step (weak scaling: the global batch grows with N); the step
ends with one NCCL all-reduce of data.grad.  Rank 0 prints ONE JSON line whose
value is the rays of all ranks per second.  ``--impl reference`` times the CPU oracle (the
C restatement of the reference's algorithm) on the host cores instead.

Inputs are seeded synthetic data (svox_b200/workloads.py): no real scene is
available offline.  The tree's data tensor (1.18 GB) is far larger than L2
(126 MB), so no explicit L2 flush is needed between steps.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "Mrays/s volume_render fwd+bwd (SH deg 2, 2^20 rays)"
UNIT = "Mrays/s"
# DRAM bytes (read + write) of one launch on the default workload, from the ncu capture
# summarised in profiles/training_step_config4_ncu_full.md
NCU_TRAFFIC_FWD = 18.7e9
NCU_TRAFFIC_BWD = 5.7e9 + 4.1e9


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="b200", choices=["b200", "reference"])
    p.add_argument("--rays", type=int, default=1 << 20, help="rays per step and GPU")
    p.add_argument("--init-refine", type=int, default=5)
    p.add_argument("--extra-levels", type=int, default=3)
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--overlap-parts", type=int, default=-1,
                   help="N > 1: leaf ranges whose all-reduce overlaps the backward (0 = one "
                        "all-reduce of the whole gradient after the backward; 1 = one all-reduce "
                        "of the leaf ranges that hold samples; -1 = 8 up to 4 GPUs, else 4)")
    p.add_argument("--overlap-reserve", type=int, default=-1,
                   help="SMs the backward scatter leaves to the collective (-1 = 16 up to 4 "
                        "GPUs, else 32)")
    return p.parse_args()


def workload_name(a):
    fine = 2 ** (a.init_refine + 1 + a.extra_levels)
    return (f"config4: shell tree {2 ** (a.init_refine + 1)}^3 -> {fine}^3, SH9 (K=28), "
            f"{a.rays} rays/step/GPU, MSE, backward into data.grad")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "50", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.t.join(timeout=2)
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names)
                   if any(len(r) >= 9 and r[5 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


# ---------------------------------------------------------------------------
def oracle_step_fn(tree, rays, targets):
    """One CPU step (forward, MSE gradient, backward incl. zero-fill) on a ray sample."""
    from oracle import oracle as orc
    ot = orc.Tree.from_n3tree(tree)
    opt = orc.options(basis_dim=9)
    n = int(np.prod(ot.data.shape))
    grad = np.zeros(n, np.float64)
    C = orc.C

    def step(o, d, v, tg):
        out = orc.volume_render(ot, o, d, v, opt)
        g = (2.0 / out.size) * (out - tg)
        grad[:] = 0.0
        orc.lib().orc_volume_render_backward(
            C.byref(ot.c), orc._ptr(orc._f32(o)), orc._ptr(orc._f32(d)), orc._ptr(orc._f32(v)),
            C.c_int64(o.shape[0]), C.byref(opt), orc._ptr(orc._f32(g)), orc._ptr(grad), None, None)
        return float(((out - tg) ** 2).mean())

    return step, orc.num_threads()


def cpu_reference(a, tree, rays, targets, budget_s):
    """Times the oracle on a bounded ray sample; returns (Mrays/s, ms/step, info)."""
    from oracle import oracle as orc
    # torchrun sets OMP_NUM_THREADS=1; the CPU arm uses every core this process may run on
    orc.set_num_threads(len(os.sched_getaffinity(0)))
    step, threads = oracle_step_fn(tree, rays, targets)
    o, d, v = [t.numpy() for t in rays]
    tg = targets.numpy()
    probe = min(2048, o.shape[0])
    t0 = time.perf_counter()
    step(o[:probe], d[:probe], v[:probe], tg[:probe])
    per_ray = (time.perf_counter() - t0) / probe
    n_steps = a.steps + a.warmup
    sample = int(min(o.shape[0], max(1024, (budget_s / max(n_steps, 1)) / per_ray)))
    sample = max(1024, (sample // 1024) * 1024)
    for _ in range(a.warmup):
        step(o[:sample], d[:sample], v[:sample], tg[:sample])
    t0 = time.perf_counter()
    for _ in range(a.steps):
        step(o[:sample], d[:sample], v[:sample], tg[:sample])
    dt = (time.perf_counter() - t0) / a.steps
    info = {"cores": threads, "kind": "port",
            "sample": f"first {sample} rays of the step's {o.shape[0]} (same tree), per step"}
    return sample / dt / 1e6, dt * 1e3, info


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from svox_b200 import workloads as W
    tree, rays, targets = W.config4(Q=min(a.rays, 1 << 17), init_refine=a.init_refine,
                                    extra_levels=a.extra_levels)
    val, ms, info = cpu_reference(a, tree, rays, targets, budget_s=150.0)
    info["value"] = val
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT,
            "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": workload_name(a),
                                            "l2": "inputs larger than L2"},
            "cpu_baseline": info,
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
def run_b200(a):
    import torch.distributed as dist
    import svox_b200
    from svox_b200 import csrc, distributed as D, workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py --impl b200 needs a GPU"
    assert csrc.is_built(), "native library missing (no fallback)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        if a.overlap_parts < 0:
            a.overlap_parts = 8 if world <= 4 else 4
        if a.overlap_reserve < 0:
            # SMs left to the collective: NCCL needs more of them on 8 GPUs (timeline of one
            # backward + all-reduce at N = 8: 6.0 ms plain, 6.0 ms with 16, 5.2 ms with 32)
            a.overlap_reserve = 16 if world <= 4 else 32
        D.overlap_grad_allreduce(a.overlap_parts, reserve_sms=a.overlap_reserve)

    tree_cpu, rays_cpu, targets_cpu = W.config4(Q=a.rays, init_refine=a.init_refine,
                                                extra_levels=a.extra_levels)
    Q = a.rays
    if rank > 0:   # every rank draws its own rays and targets for the same scene
        gen = torch.Generator().manual_seed(3 + 1000 * rank)
        rays_cpu = W.sphere_rays(Q, gen, 4.0, 0.2, 0.8)
        targets_cpu = torch.rand(Q, 3, generator=gen)
    tree = tree_cpu.to(dev)
    rays_h = [t.contiguous().pin_memory() for t in rays_cpu]
    tg_h = targets_cpu.contiguous().pin_memory()
    rays = svox_b200.Rays(*[t.to(dev) for t in rays_h])
    targets = tg_h.to(dev)
    renderer = svox_b200.VolumeRenderer(tree)
    denom = float(Q * world * 3)

    def step(r=rays, tg=targets):
        tree.zero_grad(set_to_none=True)
        out = renderer(r)
        loss = ((out - tg) ** 2).sum() / denom      # this rank's share of the global MSE
        loss.backward()
        D.allreduce_grad(tree)
        return loss

    # End to end: every step copies its inputs from pinned host memory and reads the loss back.
    # Like a training loop's data loader, the copy of step k+1 is issued on a copy stream right
    # after step k's kernels have been launched, into the other of two device buffer sets (the
    # loss read-back at the end of step k-1 guarantees nobody still reads that set).
    copy_stream = torch.cuda.Stream(device=dev)
    dev_sets = [([torch.empty_like(t, device=dev) for t in rays_h],
                 torch.empty_like(tg_h, device=dev)) for _ in range(2)]
    ready = [None, None]
    e2e_state = {"k": 0}

    def upload(slot):
        with torch.cuda.stream(copy_stream):
            for d, h in zip(dev_sets[slot][0], rays_h):
                d.copy_(h, non_blocking=True)
            dev_sets[slot][1].copy_(tg_h, non_blocking=True)
            ready[slot] = torch.cuda.Event()
            ready[slot].record(copy_stream)

    def e2e_step():
        slot = e2e_state["k"] & 1
        e2e_state["k"] += 1
        if ready[slot] is None:
            upload(slot)                     # very first step: nothing was prefetched
        torch.cuda.current_stream().wait_event(ready[slot])
        ready[slot] = None
        loss = step(svox_b200.Rays(*dev_sets[slot][0]), dev_sets[slot][1])
        upload(slot ^ 1)                     # the next step's inputs travel meanwhile
        return loss.item()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        a0, b0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(steps):
            fn()
        b0.record()
        barrier()
        ms = torch.tensor([a0.elapsed_time(b0)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / steps

    # byte model: exact per-ray visit / contribution counts of this rank's rays
    vis, cf, cb = csrc.march_stats(tree._spec(), svox_b200.render._rays_spec_from_rays(rays),
                                   renderer._get_options())
    n_local = Q
    K = tree.data_dim
    sums = torch.stack([vis.sum(), cf.sum(), cb.sum()]).double()
    fwd_bytes = n_local * 48 + 8 * sums[0].item() + 4 * (K - 1) * sums[1].item()
    bwd_bytes = n_local * 48 + 8 * sums[0].item() + 8 * K * sums[2].item()

    for _ in range(max(a.warmup, 3)):
        step()
    records = []
    csrc.set_timing(records)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_step = timed(step, a.steps)
    clocks = sampler.stop() if rank == 0 else None
    csrc.set_timing(None)
    torch.cuda.synchronize()
    per_call = {}
    for name, ea, eb in records:
        per_call.setdefault(name, []).append(ea.elapsed_time(eb))
    ms_fwd = float(np.mean(per_call["volume_render"]))
    ms_bwd = float(np.mean(per_call["volume_render_backward"]))

    e2e = None
    if not a.no_e2e:
        for _ in range(2):
            e2e_step()
        ms_e2e = timed(e2e_step, a.steps)
        e2e = {"value": Q / ms_e2e / 1e3, "unit": UNIT,
               "h2d_bytes_per_step": int(sum(t.numel() * 4 for t in rays_h) + tg_h.numel() * 4),
               "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e,
               "h2d": "pinned host buffers, copied on a copy stream while the previous step "
                      "computes (double-buffered)"}

    peak, peak_src = peaks()
    total = Q * world
    if e2e is not None:
        e2e["value"] = total / e2e["ms_per_step"] / 1e3
    line = {
        "metric": METRIC, "value": total / ms_step / 1e3, "unit": UNIT, "n_gpus": world,
        "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload_name(a), "rays_per_gpu": n_local,
                   "rays_per_step": total,
                   "parallelism": f"rays sharded x{world}, tree replicated, "
                                  + ((f"NCCL all-reduce of the leaf ranges of data.grad that hold "
                                      f"samples, in {a.overlap_parts} part(s) overlapped with the "
                                      "backward scatter" if a.overlap_parts
                                      else "one NCCL all-reduce of data.grad")
                                     if world > 1 else "no collective"),
                   "l2": "inputs larger than L2 (1.18 GB tree data vs 126 MB)",
                   "visits_per_ray": sums[0].item() / n_local,
                   "contrib_per_ray": sums[2].item() / n_local},
        # dominant kernel: the logged forward march (render_queue_kernel).  `traffic` is the
        # DRAM read + write of one launch from the committed ncu capture of this workload.
        "roofline": {"bound": "hbm", "kernel": "render_queue_kernel, logged forward (volume_render)",
                     "achieved": fwd_bytes / ms_fwd / 1e6, "peak": peak, "unit": "GB/s",
                     "frac": fwd_bytes / ms_fwd / 1e6 / peak,
                     "traffic": NCU_TRAFFIC_FWD if Q == 1 << 20 else None,
                     "peak_source": peak_src, "ms_per_launch": ms_fwd,
                     "algorithmic_bytes_per_launch": fwd_bytes},
        "roofline_backward": {"bound": "hbm",
                              "kernel": "replay_bin_kernel + replay_scatter_kernel "
                                        "(volume_render_backward)",
                              "achieved": bwd_bytes / ms_bwd / 1e6, "peak": peak, "unit": "GB/s",
                              "frac": bwd_bytes / ms_bwd / 1e6 / peak,
                              "traffic": NCU_TRAFFIC_BWD if Q == 1 << 20 else None,
                              "ms_per_launch": ms_bwd,
                              "algorithmic_bytes_per_launch": bwd_bytes},
        "roofline_step": {"algorithmic_bytes": fwd_bytes + bwd_bytes,
                          "achieved": (fwd_bytes + bwd_bytes) / ms_step / 1e6,
                          "frac": (fwd_bytes + bwd_bytes) / ms_step / 1e6 / peak},
        "e2e": e2e,
        # per step: forward = annotate, leaf table, brick assign, brick fill, march;
        # backward = prefix, ray pack, bin, scatter
        "gpu_launches": 9 * a.steps,
        "clocks": clocks,
    }
    if rank == 0 and world == 1 and not a.no_cpu_baseline:
        val, ms, info = cpu_reference(
            argparse.Namespace(steps=2, warmup=1),
            tree_cpu, svox_b200.Rays(*[t[:1 << 16] for t in rays_cpu]), targets_cpu[:1 << 16],
            budget_s=25.0)
        info.update(value=val, unit=UNIT, ms_per_step=ms)
        line["cpu_baseline"] = info
    csrc.check_device_status()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)
