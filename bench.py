#!/usr/bin/env python
"""Benchmarks of the svox hot path on 1..8 B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload train|query|image3|image5]

``--workload train`` (default, the headline metric): Mrays/s of one training step
-- volume_render forward + MSE + backward into data.grad -- on the sparse-shell
SH-degree-2 scene with 2^20 rays per step.  Under torchrun (N > 1) every rank
holds the whole tree and renders a contiguous slice of the SAME 2^20 rays
(strong scaling); the step ends with the all-reduce of data.grad.  Four
ways of doing that all-reduce are timed and labelled in the JSON line:

  allreduce_after_backward   one all-reduce of the whole gradient after the backward
  allreduce_inside_backward  the backward hands finished leaf ranges to NCCL while it
                             still computes the next ones
  allreduce_multicast        the gradient lies in symmetric memory and the NVSwitch sums it
                             (multimem.ld_reduce / multimem.st, svoxb_allreduce_multimem)
  allreduce_under_next_step  the all-reduce of step i runs beside the forward and backward
                             of step i+1 (two gradient buffers; legitimate here because
                             nothing consumes the gradient between steps)

``value`` is the best of the first three (the gradient of a step is complete
when the step ends); the last is reported beside it.  At N > 1 the reduced
gradient is also compared, outside the timed region, with the single-GPU
gradient of the same 2^20 rays, and every rank's colours with the single-GPU
render.  The other workloads are the point query (2^24 points, 256^3 leaves,
SH degree 3) and the two forward image renders; they print the same kind of
line with their own metric.

``--impl reference`` times the CPU oracle (the C restatement of the reference's
algorithm) on the host cores instead.  Inputs are seeded synthetic data
(svox_b200/workloads.py): no real scene is available offline.  Every tree's
data tensor is far larger than L2 (126 MB), so no L2 flush is needed between steps.
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

UNIT = "Mrays/s"
METRICS = {
    "train": "Mrays/s volume_render fwd+bwd (SH deg 2, 2^20 rays)",
    "query": "Mpoints/s query_vertical fwd+bwd (SH deg 3, 256^3 leaves, 2^24 points)",
    "image3": "Mrays/s render_persp forward (SH deg 3, 512^3 shell, 800x800 views)",
    "image5": "Mrays/s render_persp forward (SH deg 3, three shells at 1024^3, 1920x1080 views)",
}
# DRAM bytes (read + write) of one launch of the dominant kernel of the training step (the
# logged forward march), from an ncu capture of a 2^17-ray launch (1.450 GB read + 0.353 GB
# written) scaled by 8 to the 2^20-ray launch: its traffic grows with the rays.  The backward's
# does not (the gradient is read and written once whatever the number of rays), so its figure
# comes from a one-pass capture (DRAM bytes and duration only) of the two replay kernels at
# full size: bin pass 3.583 GB read + 2.227 GB written, scatter 3.167 GB + 0.900 GB.
# Printed only together with `traffic_source`, which names the capture.
NCU_TRAFFIC = {"forward": 8 * (1.449616e9 + 0.352721e9),
               "backward": 3.583350e9 + 2.226789e9 + 3.167486e9 + 0.900214e9}
NCU_TRAFFIC_SOURCE = ("ncu --set full of render_queue_kernel<9,640,ForwardLogged> at 2^17 rays "
                      "x 8 (profiles/training_step_rays131072_ncu_full.md); valid for the "
                      "kernel as of library version " + "0.3.0")


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="b200", choices=["b200", "reference"])
    p.add_argument("--workload", default="train", choices=list(METRICS))
    p.add_argument("--rays", type=int, default=1 << 20, help="train: rays per step (all GPUs)")
    p.add_argument("--points", type=int, default=1 << 24, help="query: points per step")
    p.add_argument("--views", type=int, default=0, help="image3/5: views per step (0 = 8 / 4)")
    p.add_argument("--init-refine", type=int, default=-1)
    p.add_argument("--extra-levels", type=int, default=3)
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-other-workloads", action="store_true",
                   help="train, N = 1: leave out the query / image workloads' digest")
    p.add_argument("--multicast", action="store_true",
                   help="train, N > 1: also time the variant that sums the gradient in the "
                        "switch (needs multicast memory on every GPU)")
    p.add_argument("--no-ref-cuda", action="store_true")
    p.add_argument("--no-weak", action="store_true")
    p.add_argument("--overlap-parts", type=int, default=-1,
                   help="N > 1: leaf ranges of the all-reduce inside the backward "
                        "(-1 = 8 up to 4 GPUs, else 4)")
    p.add_argument("--overlap-reserve", type=int, default=-1,
                   help="SMs the backward scatter leaves to the collective (-1 = 16 up to 4 "
                        "GPUs, else 32)")
    a = p.parse_args()
    if a.init_refine < 0:
        a.init_refine = {"train": 5, "query": 7, "image3": 5, "image5": 6}[a.workload]
    if a.views <= 0:
        a.views = 8 if a.workload == "image3" else 4
    return a


def workload_name(a):
    fine = 2 ** (a.init_refine + 1 + a.extra_levels)
    if a.workload == "train":
        return (f"config4: shell tree {2 ** (a.init_refine + 1)}^3 -> {fine}^3, SH9 (K=28), "
                f"{a.rays} rays/step, MSE, backward into data.grad")
    if a.workload == "query":
        return (f"config2: uniform tree {2 ** (a.init_refine + 1)}^3 leaves, SH16 (K=49), "
                f"{a.points} points/step, values + ids, backward of a N(0,1) upstream gradient")
    if a.workload == "image3":
        return (f"config3: shell tree {2 ** (a.init_refine + 1)}^3 -> {fine}^3, SH16 (K=49), "
                f"{a.views} views of 800x800, fx=fy=1111, stop_thresh 1e-2, forward only")
    return (f"config5: three shells {2 ** (a.init_refine + 1)}^3 -> {fine}^3, SH16 (K=49), "
            f"{a.views} of the 64 views of 1920x1080, fx=fy=1600, step 5e-4, fast=True, "
            "forward only")


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

    def ensure(self, step, n=2, limit_s=3.0):
        """Short timed regions can end before nvidia-smi delivers its first sample: keep the
        GPU under the same load (extra, untimed steps) until ``n`` samples have arrived."""
        t0 = time.perf_counter()
        while self.proc is not None and len(self.rows) < n and \
                time.perf_counter() - t0 < limit_s:
            step()
            torch.cuda.synchronize()

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
# CPU arm: the oracle (port of the reference's algorithm) on the host cores

def _oracle_threads():
    from oracle import oracle as orc
    # torchrun sets OMP_NUM_THREADS=1; the CPU arm uses every core this process may run on
    orc.set_num_threads(len(os.sched_getaffinity(0)))
    return orc.num_threads()


def oracle_train_step(tree):
    """One CPU training step (forward, MSE gradient, backward incl. zero-fill) on a ray sample."""
    from oracle import oracle as orc
    ot = orc.Tree.from_n3tree(tree)
    opt = orc.options(basis_dim=9)
    grad = np.zeros(int(np.prod(ot.data.shape)), np.float64)
    C = orc.C

    def step(o, d, v, tg):
        out = orc.volume_render(ot, o, d, v, opt)
        g = (2.0 / out.size) * (out - tg)
        grad[:] = 0.0
        orc.lib().orc_volume_render_backward(
            C.byref(ot.c), orc._ptr(orc._f32(o)), orc._ptr(orc._f32(d)), orc._ptr(orc._f32(v)),
            C.c_int64(o.shape[0]), C.byref(opt), orc._ptr(orc._f32(g)), orc._ptr(grad), None, None)
    return step


def cpu_sampled(step, arrays, n_items, steps, warmup, budget_s, what):
    """Times ``step`` on a leading sample of ``arrays`` (items drawn like the workload's) sized
    to ``budget_s`` seconds in all; returns (M items/s, ms/step, info)."""
    threads = _oracle_threads()
    probe = min(2048, n_items)
    t0 = time.perf_counter()
    step(*[x[:probe] for x in arrays])
    per_item = (time.perf_counter() - t0) / probe
    n_steps = steps + warmup
    sample = int(min(n_items, max(1024, (budget_s / max(n_steps, 1)) / per_item)))
    sample = min(n_items, max(1024, (sample // 1024) * 1024))
    for _ in range(warmup):
        step(*[x[:sample] for x in arrays])
    t0 = time.perf_counter()
    for _ in range(steps):
        step(*[x[:sample] for x in arrays])
    dt = (time.perf_counter() - t0) / steps
    info = {"cores": threads, "kind": "port",
            "sample": f"{sample} {what} per step, drawn like the workload's (same tree)"}
    return sample / dt / 1e6, dt * 1e3, info


def cpu_arm(a, steps, warmup, budget_s):
    """(value, ms, info) of the CPU oracle on a bounded sample of the workload."""
    from oracle import oracle as orc
    from svox_b200 import workloads as W
    if a.workload == "train":
        tree, rays, targets = W.config4(Q=min(a.rays, 1 << 17), init_refine=a.init_refine,
                                        extra_levels=a.extra_levels)
        arrays = [t.numpy() for t in rays] + [targets.numpy()]
        return cpu_sampled(oracle_train_step(tree), arrays, arrays[0].shape[0], steps, warmup,
                           budget_s, "rays")
    if a.workload == "query":
        tree, pts = W.config2(Q=min(a.points, 1 << 20), init_refine=a.init_refine)
        ot = orc.Tree.from_n3tree(tree)
        gen = torch.Generator().manual_seed(11)
        gout = torch.randn(pts.shape[0], tree.data_dim, generator=gen).numpy()

        def step(p, g):
            orc.query_vertical(ot, p)
            orc.query_vertical_backward(ot, p, g)
        return cpu_sampled(step, [pts.numpy(), gout], pts.shape[0], steps, warmup, budget_s,
                           "points")
    tree, cams = (W.config3 if a.workload == "image3" else W.config5)(
        n_views=1, init_refine=a.init_refine, extra_levels=a.extra_levels)
    w, h, f = (800, 800, 1111.0) if a.workload == "image3" else (1920, 1080, 1600.0)
    ot = orc.Tree.from_n3tree(tree)
    if a.workload == "image3":
        opt = orc.options(basis_dim=16, stop_thresh=1e-2)
    else:
        opt = orc.options(basis_dim=16, step_size=5e-4, sigma_thresh=1e-2, stop_thresh=1e-2)
    o, d = orc.pixel_rays(cams[0].numpy(), f, f, w, h)
    # a strided sample of the view's pixels: a leading block would be background only
    stride = 16
    o, d = o[::stride], d[::stride]

    def step(oo, dd):
        orc.volume_render(ot, oo, dd, dd, opt)
    val, ms, info = cpu_sampled(step, [o, d], o.shape[0], steps, warmup, budget_s, "pixels")
    info["sample"] = "every 16th pixel of one view: " + info["sample"]
    return val, ms, info


def run_reference(a):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    val, ms, info = cpu_arm(a, a.steps, a.warmup, budget_s=150.0)
    info["value"] = val
    line = {"impl": "reference", "metric": METRICS[a.workload], "value": val, "unit": UNIT_OF(a),
            "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": workload_name(a), "l2": "inputs larger than L2"},
            "cpu_baseline": info,
            "reference_python_path": "not measured here: the reference's own CPU tensor path is "
                                     "Python and its checkout is not on the GPU box; this arm "
                                     "times the C restatement of its algorithm",
            "e2e": {"value": val, "unit": UNIT_OF(a), "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def UNIT_OF(a):
    return "Mpoints/s" if a.workload == "query" else UNIT


# ---------------------------------------------------------------------------
class Harness:
    """Process group, device and the timing loop shared by the workloads."""

    def __init__(self, a):
        import torch.distributed as dist
        from svox_b200 import csrc
        self.a, self.dist = a, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        assert torch.cuda.is_available(), "bench.py --impl b200 needs a GPU"
        assert csrc.is_built(), "native library missing (no fallback)"
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.sampler = ClockSampler(self.local)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def timed(self, fn, steps, finish=None):
        """ms per step of ``steps`` calls, device time, maximum over the ranks."""
        self.barrier()
        a0, b0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for i in range(steps):
            fn(i)
        if finish is not None:
            finish()
        b0.record()
        self.barrier()
        ms = torch.tensor([a0.elapsed_time(b0)], device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(ms, op=self.dist.ReduceOp.MAX)
        return ms.item() / steps

    def done(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def ref_cuda_train(tree, rays, targets, steps=5):
    """fwd / bwd / step ms of the UNMODIFIED reference extension (oracle/_ref, built from the
    reference's own sources) on the same tree and rays -- the GPU implementation the reference
    ships, as a baseline leg only."""
    try:
        from oracle.build_ref import load_module
        ref = load_module()
    except Exception as e:                       # the parity target is optional
        return {"unavailable": f"{type(e).__name__}: {e}"}
    if ref is None:
        return {"unavailable": "oracle/_ref holds no built reference extension"}
    dev = tree.data.device
    spec = ref.TreeSpec()
    spec.data, spec.child, spec.parent_depth = tree.data.data, tree.child, tree.parent_depth
    spec.extra_data = torch.empty((0, 0), device=dev)
    spec.offset, spec.scaling = tree.offset, tree.invradius
    spec._weight_accum = torch.empty(0, device=dev)
    spec._weight_accum_max = False
    opt = ref.RenderOptions()
    opt.step_size, opt.background_brightness, opt.format, opt.basis_dim = 1e-3, 1.0, 1, 9
    opt.ndc_width, opt.ndc_height, opt.ndc_focal = -1, -1, 0.0
    opt.min_comp, opt.max_comp, opt.sigma_thresh, opt.stop_thresh = 0, 8, 0.0, 0.0
    opt.density_softplus, opt.rgb_padding = False, 0.0
    rs = ref.RaysSpec()
    rs.origins, rs.dirs, rs.vdirs = rays.origins, rays.dirs, rays.viewdirs
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    fwd, bwd = [], []
    for i in range(steps + 1):
        ev[0].record()
        out = ref.volume_render(spec, rs, opt)
        g = (2.0 / out.numel()) * (out - targets)
        ev[1].record()
        ref.volume_render_backward(spec, rs, opt, g.contiguous())
        ev[2].record()
        torch.cuda.synchronize()
        if i:
            fwd.append(ev[0].elapsed_time(ev[1]))
            bwd.append(ev[1].elapsed_time(ev[2]))
    step = float(np.mean(fwd) + np.mean(bwd))
    n = rays.origins.shape[0]
    return {"what": "unmodified reference CUDA extension (sm_100 build of svox/csrc) on the "
                    "same tree and rays, one GPU; forward incl. the MSE gradient",
            "ms_fwd": float(np.mean(fwd)), "ms_bwd": float(np.mean(bwd)), "ms_per_step": step,
            "value": n / step / 1e3, "unit": UNIT, "rays": n}


# ---------------------------------------------------------------------------
def run_train(a):
    import svox_b200
    from svox_b200 import csrc, distributed as D, workloads as W
    H = Harness(a)
    dist, dev, world, rank = H.dist, H.dev, H.world, H.rank
    if a.overlap_parts < 0:
        a.overlap_parts = 8 if world <= 4 else 4
    if a.overlap_reserve < 0:
        # SMs left to the collective: NCCL needs more of them on 8 GPUs
        a.overlap_reserve = 16 if world <= 4 else 32

    tree_cpu, rays_cpu, targets_cpu = W.config4(Q=a.rays, init_refine=a.init_refine,
                                                extra_levels=a.extra_levels)
    Q = a.rays
    lo, hi = D.shard_bounds(Q, rank, world)
    n_local = hi - lo
    tree = tree_cpu.to(dev)
    rays_h = [t[lo:hi].contiguous().pin_memory() for t in rays_cpu]
    tg_h = targets_cpu[lo:hi].contiguous().pin_memory()
    rays = svox_b200.Rays(*[t.to(dev) for t in rays_h])
    targets = tg_h.to(dev)
    renderer = svox_b200.VolumeRenderer(tree)
    state = {"denom": float(Q * 3), "rays": rays, "targets": targets, "keep": [None, None],
             "works": [None, None]}

    def fwd_bwd(r, tg):
        tree.zero_grad(set_to_none=True)
        out = renderer(r)
        loss = ((out - tg) ** 2).sum() / state["denom"]   # this rank's share of the global MSE
        loss.backward()
        return loss

    def step(i=0, r=None, tg=None):
        loss = fwd_bwd(r or state["rays"], tg if tg is not None else state["targets"])
        D.allreduce_grad(tree)
        return loss

    def step_pipelined(i):
        # the all-reduce of this step's gradient is left running while the next step computes;
        # the buffer of the step before last must be done before it is dropped
        k = i & 1
        if state["works"][k] is not None:
            state["works"][k].wait()
        fwd_bwd(state["rays"], state["targets"])
        g = tree.data.grad
        state["keep"][k] = g
        state["works"][k] = dist.all_reduce(g, op=dist.ReduceOp.SUM, async_op=True)

    def drain():
        for k in (0, 1):
            if state["works"][k] is not None:
                state["works"][k].wait()
                state["works"][k] = None

    # the gradient in symmetric memory, summed by the switch (on request: it moves fewer bytes
    # than the ring from 4 GPUs on, but measured no faster there).  Every rank has to succeed,
    # or none uses it.
    multicast = None
    if world >= 2 and a.multicast:
        try:
            multicast = D.MulticastGradient(tree)
        except Exception as e:                      # no multicast memory on this box
            multicast = None
            if rank == 0:
                print(f"[bench] no multicast gradient: {e!r}"[:300], file=sys.stderr)
        have = torch.tensor([int(multicast is not None)], device=dev)
        dist.all_reduce(have, op=dist.ReduceOp.MIN)
        if not have.item():
            multicast = None

    def set_variant(name):
        D.overlap_grad_allreduce(a.overlap_parts if name == "allreduce_inside_backward" else 0,
                                 reserve_sms=a.overlap_reserve)
        if name == "allreduce_multicast":
            multicast.enable()
        else:
            D.MulticastGradient.disable()

    # byte model: exact per-ray visit / contribution counts of this rank's rays
    vis, cf, cb = csrc.march_stats(tree._spec(), svox_b200.render._rays_spec_from_rays(rays),
                                   renderer._get_options())
    K = tree.data_dim
    sums = torch.stack([vis.sum(), cf.sum(), cb.sum()]).double()
    if world > 1:
        dist.all_reduce(sums)
    fwd_bytes = Q * 48 + 8 * sums[0].item() + 4 * (K - 1) * sums[1].item()
    bwd_bytes = Q * 48 + 8 * sums[0].item() + 8 * K * sums[2].item()
    # what THIS design's backward moves instead (it never re-reads records): per contributing
    # sample the log entry (44 B) in, a 32-byte packet out and in again; per touched gradient
    # element one read and one write; 96 B per ray of packed inputs
    n_leaf_slots = int((tree.child[:tree.n_internal] == 0).sum().item())
    replay_bytes = sums[2].item() * (44 + 32 + 32) + 2 * 4 * K * n_leaf_slots + Q * 96

    warm = max(a.warmup, 3)
    variants = {}
    names = ["allreduce_after_backward"] if world == 1 else \
        ["allreduce_after_backward", "allreduce_inside_backward"]
    if multicast is not None:
        names.insert(0, "allreduce_multicast")
    records = []
    clocks = None
    if rank == 0:
        H.sampler.start()        # sampled through the warm-up and timed steps of every variant
    for name in names:
        set_variant(name)
        for _ in range(warm):
            step()
        last = name == names[-1]
        if last:
            csrc.set_timing(records)
        ms = H.timed(step, a.steps)
        if last:
            csrc.set_timing(None)
        variants[name] = {"ms_per_step": ms, "value": Q / ms / 1e3}
    if world == 1:
        H.sampler.ensure(step)   # (single process only: extra steps on one rank of several
    clocks = H.sampler.stop() if rank == 0 else None     #  would leave its collectives alone)
    torch.cuda.synchronize()
    per_call = {}
    for name, ea, eb in records:
        per_call.setdefault(name, []).append(ea.elapsed_time(eb))
    ms_fwd = float(np.mean(per_call["volume_render"]))
    ms_bwd = float(np.mean(per_call["volume_render_backward"]))
    best = min(variants, key=lambda n: variants[n]["ms_per_step"])
    ms_step = variants[best]["ms_per_step"]

    if world > 1:
        set_variant("allreduce_after_backward")
        csrc.reserve_sms(a.overlap_reserve)      # the collective runs beside every kernel now
        for i in range(warm):
            step_pipelined(i)
        drain()
        ms = H.timed(step_pipelined, a.steps, finish=drain)
        csrc.reserve_sms(0)
        variants["allreduce_under_next_step"] = {"ms_per_step": ms, "value": Q / ms / 1e3,
                                                 "reserved_sms": a.overlap_reserve}

    # ---- correctness of the multi-GPU step (outside the timed region) ----------------------
    check = None
    if world > 1:
        full_rays = svox_b200.Rays(*[t.to(dev) for t in rays_cpu])
        full_tg = targets_cpu.to(dev)
        D.overlap_grad_allreduce(0)
        tree.zero_grad(set_to_none=True)
        out_full = renderer(full_rays)
        (((out_full - full_tg) ** 2).sum() / state["denom"]).backward()
        single = tree.data.grad.clone()
        top = single.abs().max().item()
        check = {"what": "reduced data.grad of the sharded step against the gradient of the same "
                         f"{Q} rays computed on one GPU (max |diff| / max |grad|); colours of "
                         "every rank's slice against the one-GPU render (bit-equal)"}
        with torch.no_grad():
            mine = renderer(rays)
        same = torch.tensor([int(torch.equal(mine, out_full[lo:hi].detach()))], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        check["rgb_shards_bit_equal"] = bool(same.item())
        for name in names:
            set_variant(name)
            step()
            err = torch.tensor([(tree.data.grad - single).abs().max().item() / top], device=dev)
            dist.all_reduce(err, op=dist.ReduceOp.MAX)
            check[name] = err.item()
        check["ok"] = check["rgb_shards_bit_equal"] and all(check[n] <= 1e-4 for n in names)
        del single, out_full, full_rays, full_tg
        set_variant(best)

    # ---- weak scaling (2^20 rays on every GPU), same step --------------------------------
    weak = None
    if world > 1 and not a.no_weak:
        gen = torch.Generator().manual_seed(3 + 1000 * rank)
        wr = W.sphere_rays(Q, gen, 4.0, 0.2, 0.8) if rank else svox_b200.Rays(*rays_cpu)
        wt = torch.rand(Q, 3, generator=gen) if rank else targets_cpu
        state["rays"] = svox_b200.Rays(*[t.to(dev) for t in wr])
        state["targets"] = wt.to(dev)
        state["denom"] = float(Q * world * 3)
        for _ in range(warm):
            step()
        ms = H.timed(step, a.steps)
        weak = {"rays_per_gpu": Q, "ms_per_step": ms, "value": Q * world / ms / 1e3,
                "variant": best}
        state["rays"], state["targets"], state["denom"] = rays, targets, float(Q * 3)

    # ---- end to end: every step copies its inputs from pinned host memory and reads the loss
    # back.  Like a training loop's data loader, the copy of step k+1 is issued on a copy stream
    # right after step k's kernels have been launched, into the other of two device buffer sets
    # (the loss read-back at the end of step k-1 guarantees nobody still reads that set).
    e2e = None
    if not a.no_e2e:
        copy_stream = torch.cuda.Stream(device=dev)
        dev_sets = [([torch.empty_like(t, device=dev) for t in rays_h],
                     torch.empty_like(tg_h, device=dev)) for _ in range(2)]
        ready = [None, None]

        def upload(slot):
            with torch.cuda.stream(copy_stream):
                for d, h in zip(dev_sets[slot][0], rays_h):
                    d.copy_(h, non_blocking=True)
                dev_sets[slot][1].copy_(tg_h, non_blocking=True)
                ready[slot] = torch.cuda.Event()
                ready[slot].record(copy_stream)

        def e2e_step(k):
            slot = k & 1
            if ready[slot] is None:
                upload(slot)                     # very first step: nothing was prefetched
            torch.cuda.current_stream().wait_event(ready[slot])
            ready[slot] = None
            loss = step(0, svox_b200.Rays(*dev_sets[slot][0]), dev_sets[slot][1])
            upload(slot ^ 1)                     # the next step's inputs travel meanwhile
            return loss.item()

        for k in range(2):
            e2e_step(k)
        ms_e2e = H.timed(e2e_step, a.steps)
        e2e = {"value": Q / ms_e2e / 1e3, "unit": UNIT,
               "h2d_bytes_per_step": int(sum(t.numel() * 4 for t in rays_h) + tg_h.numel() * 4),
               "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e,
               "h2d": "pinned host buffers (this rank's slice), copied on a copy stream while "
                      "the previous step computes (double-buffered)"}

    peak, peak_src = peaks()
    # the captured traffic describes this workload on one GPU with the kernels of one version
    traffic_ok = Q == 1 << 20 and world == 1 and csrc.version() in NCU_TRAFFIC_SOURCE
    line = {
        "metric": METRICS["train"], "value": Q / ms_step / 1e3, "unit": UNIT, "n_gpus": world,
        "steps": a.steps, "warmup": warm, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload_name(a), "rays_per_gpu": n_local, "rays_per_step": Q,
                   "parallelism": f"the same {Q} rays cut into {world} contiguous slices, tree "
                                  "replicated, " + (f"NCCL all-reduce of data.grad: {best}"
                                                    if world > 1 else "no collective"),
                   "l2": "inputs larger than L2 (1.18 GB tree data vs 126 MB)",
                   "visits_per_ray": sums[0].item() / Q, "contrib_per_ray": sums[2].item() / Q},
        "variants": variants,
        # dominant kernel: the logged forward march (render_queue_kernel); ms_per_launch is the
        # library call's device time on this rank's slice (index build + march)
        "roofline": {"bound": "hbm", "kernel": "render_queue_kernel, logged forward (volume_render)",
                     "achieved": fwd_bytes / world / ms_fwd / 1e6, "peak": peak, "unit": "GB/s",
                     "frac": fwd_bytes / world / ms_fwd / 1e6 / peak,
                     "traffic": NCU_TRAFFIC["forward"] if traffic_ok else None,
                     "traffic_source": NCU_TRAFFIC_SOURCE if traffic_ok else None,
                     "peak_source": peak_src, "ms_per_launch": ms_fwd,
                     "algorithmic_bytes_per_launch": fwd_bytes / world},
        # The backward replays the forward's item log.  `model_frac` divides the bytes of the
        # REFERENCE's backward (march again, re-read every record, accumulate the gradient once)
        # by this design's time: how much faster than that algorithm's roofline it runs.  The
        # design's own traffic model (log in, packets out and in, touched gradient in and out)
        # gives `achieved`, the bandwidth it really sustains.
        "roofline_backward": {"bound": "hbm",
                              "kernel": "replay_bin_kernel + replay_scatter_kernel "
                                        "(volume_render_backward)",
                              "achieved": replay_bytes / world / ms_bwd / 1e6, "peak": peak,
                              "unit": "GB/s", "frac": replay_bytes / world / ms_bwd / 1e6 / peak,
                              "bytes_of_this_design_per_launch": replay_bytes / world,
                              "model_frac": bwd_bytes / world / ms_bwd / 1e6 / peak,
                              "algorithmic_bytes_per_launch": bwd_bytes / world,
                              "traffic": NCU_TRAFFIC["backward"] if traffic_ok else None,
                              "ms_per_launch": ms_bwd},
        "roofline_step": {"algorithmic_bytes": fwd_bytes + bwd_bytes,
                          "achieved": (fwd_bytes + bwd_bytes) / ms_step / 1e6,
                          "frac": (fwd_bytes + bwd_bytes) / ms_step / 1e6 / (peak * world)},
        "e2e": e2e,
        # per step: forward = annotate, leaf table, brick assign, brick fill, march; backward =
        # prefix, ray pack, bin, scatter (one launch per part), and the five launches of the
        # marching fallback, which return at once unless the log overflowed
        "gpu_launches": (5 + 3 + (a.overlap_parts if best == "allreduce_inside_backward" else 1)
                         + 5 + (1 if best == "allreduce_multicast" else 0)) * a.steps,
        "clocks": clocks,
    }
    if check is not None:
        line["multi_gpu_check"] = check
    if weak is not None:
        line["weak_scaling"] = weak
    if world > 1:
        line["note"] = ("strong scaling of a 7.5 ms step against an all-reduce of the dense "
                        "1.18 GB gradient (about 2-3 ms over NVLink at any N): 7x at 8 GPUs "
                        "would need the whole step, collective included, in 1.1 ms")
    if rank == 0 and world == 1:
        if not a.no_ref_cuda:
            line["ref_cuda"] = ref_cuda_train(tree, rays, targets)
        if not a.no_cpu_baseline:
            val, ms, info = cpu_arm(a, 2, 1, budget_s=25.0)
            info.update(value=val, unit=UNIT, ms_per_step=ms)
            line["cpu_baseline"] = info
    csrc.check_device_status()
    if check is not None and not check["ok"]:
        line["error"] = "multi-GPU gradient check failed"
    if rank == 0 and world == 1 and not a.no_other_workloads:
        # the other configurations of the benchmark, each in a process of its own on this GPU
        del tree, rays, targets, renderer, state
        torch.cuda.empty_cache()
        line["other_workloads"] = other_workloads(a)
    if rank == 0:
        print(json.dumps(line), flush=True)
    H.done()
    if check is not None and not check["ok"]:
        sys.exit(1)


def other_workloads(a):
    """Point query and the two forward image renders at their full sizes, run as
    ``bench.py --workload ...`` child processes; -> a digest of each one's JSON line."""
    out = {}
    for w in ("query", "image3", "image5"):
        cmd = [sys.executable, os.path.abspath(__file__), "--workload", w, "--steps", "5",
               "--warmup", "3", "--no-cpu-baseline"]
        try:
            res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
            rows = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
            d = json.loads(rows[-1])
            keep = {k: d[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "warmup")}
            keep["workload"] = d["config"]["workload"]
            keep["roofline"] = {k: d["roofline"].get(k) for k in
                                ("kernel", "achieved", "peak", "unit", "frac", "ms_per_launch")}
            for extra in ("roofline_backward", "variants", "e2e"):
                if extra in d:
                    keep[extra] = d[extra]
            out[w] = keep
        except Exception as e:          # reported, and the headline line still goes out
            out[w] = {"error": repr(e)[:300]}
    return out


# ---------------------------------------------------------------------------
def run_query(a):
    import svox_b200
    from svox_b200 import csrc, distributed as D, workloads as W
    H = Harness(a)
    dev, world, rank = H.dev, H.world, H.rank
    tree_cpu, pts_cpu = W.config2(Q=a.points, init_refine=a.init_refine)
    Q = a.points
    lo, hi = D.shard_bounds(Q, rank, world)
    tree = tree_cpu.to(dev)
    del tree_cpu
    K = tree.data_dim
    pts_h = pts_cpu[lo:hi].contiguous().pin_memory()
    pts = pts_h.to(dev)
    gen = torch.Generator(device=dev).manual_seed(11 + rank)
    gout = torch.randn(hi - lo, K, device=dev, generator=gen)
    rec = []

    def step(i=0, p=None):
        tree.zero_grad(set_to_none=True)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ev[0].record()
        vals, ids = tree(p if p is not None else pts, want_node_ids=True)
        ev[1].record()
        vals.backward(gout)
        ev[2].record()
        rec.append(ev)
        return vals

    warm = max(a.warmup, 3)
    if rank == 0:
        H.sampler.start()        # sampled through the warm-up and the timed steps
    for _ in range(warm):
        step()
    del rec[:]
    ms_step = H.timed(step, a.steps)
    n_timed = len(rec)
    if rank == 0:
        H.sampler.ensure(step)
    clocks = H.sampler.stop() if rank == 0 else None
    del rec[n_timed:]
    torch.cuda.synchronize()
    ms_fwd = float(np.mean([e[0].elapsed_time(e[1]) for e in rec]))
    ms_bwd = float(np.mean([e[1].elapsed_time(e[2]) for e in rec]))
    n = hi - lo
    fwd_bytes = n * (12 + 4 + 4 * K + 4 * K + 8)
    bwd_bytes = n * (12 + 4 + 4 * K + 4 * K)
    fill_bytes = tree.data.numel() * 4

    e2e = None
    if not a.no_e2e:
        buf = torch.empty_like(pts)

        def e2e_step(k):
            buf.copy_(pts_h, non_blocking=True)
            return float(step(0, buf).sum().item())     # a checksum of the values comes back
        e2e_step(0)
        ms_e2e = H.timed(e2e_step, a.steps)
        e2e = {"value": Q / ms_e2e / 1e3, "unit": "Mpoints/s",
               "h2d_bytes_per_step": int(pts_h.numel() * 4), "d2h_bytes_per_step": 4,
               "ms_per_step": ms_e2e, "h2d": "pinned host points (this rank's slice)"}
    peak, peak_src = peaks()
    line = {
        "metric": METRICS["query"], "value": Q / ms_step / 1e3, "unit": "Mpoints/s",
        "n_gpus": world, "steps": a.steps, "warmup": warm, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload_name(a), "points_per_gpu": n,
                   "parallelism": f"points cut into {world} slices, tree replicated, no collective",
                   "l2": "inputs larger than L2 (3.76 GB tree data, 3.3 GB of values)"},
        "roofline": {"bound": "hbm", "kernel": "query_kernel<0> (query_vertical)",
                     "achieved": fwd_bytes / ms_fwd / 1e6, "peak": peak, "unit": "GB/s",
                     "frac": fwd_bytes / ms_fwd / 1e6 / peak, "traffic": None,
                     "peak_source": peak_src, "ms_per_launch": ms_fwd,
                     "algorithmic_bytes_per_launch": fwd_bytes},
        "roofline_backward": {"bound": "hbm", "kernel": "zero-fill + query_kernel<1> "
                                                        "(query_vertical_backward)",
                              "achieved": (bwd_bytes + fill_bytes) / ms_bwd / 1e6, "peak": peak,
                              "unit": "GB/s",
                              "frac": (bwd_bytes + fill_bytes) / ms_bwd / 1e6 / peak,
                              "ms_per_launch": ms_bwd,
                              "algorithmic_bytes_per_launch": bwd_bytes,
                              "zero_fill_bytes": fill_bytes, "traffic": None},
        "e2e": e2e, "gpu_launches": 4 * a.steps, "clocks": clocks,
    }
    if rank == 0 and world == 1 and not a.no_cpu_baseline:
        val, ms, info = cpu_arm(a, 2, 1, budget_s=20.0)
        info.update(value=val, unit="Mpoints/s", ms_per_step=ms)
        line["cpu_baseline"] = info
    csrc.check_device_status()
    if rank == 0:
        print(json.dumps(line), flush=True)
    H.done()


# ---------------------------------------------------------------------------
def run_image(a):
    import svox_b200
    from svox_b200 import csrc, distributed as D, workloads as W
    H = Harness(a)
    dev, world, rank = H.dev, H.world, H.rank
    five = a.workload == "image5"
    tree_cpu, cams = (W.config5 if five else W.config3)(
        n_views=a.views, init_refine=a.init_refine, extra_levels=a.extra_levels)
    w, h, f = (1920, 1080, 1600.0) if five else (800, 800, 1111.0)
    tree = tree_cpu.to(dev)
    del tree_cpu
    tree.requires_grad_(False)
    if five:
        renderer = svox_b200.VolumeRenderer(tree, step_size=5e-4)
        fast = True
    else:
        renderer = svox_b200.VolumeRenderer(tree)
        renderer.stop_thresh = 1e-2
        fast = False
    lo, hi = D.shard_bounds(a.views, rank, world)          # whole views per rank
    cams_h = cams[lo:hi].contiguous().pin_memory()
    cams_d = cams_h.to(dev)
    n_px = a.views * w * h
    K = tree.data_dim

    def step(i=0, c=None):
        c = cams_d if c is None else c
        imgs = None
        for v in range(c.shape[0]):
            imgs = renderer.render_persp(c[v], width=w, height=h, fx=f, fast=fast)
        return imgs

    def step_frozen(i=0):
        with renderer.frozen_tree():
            return step()

    warm = max(a.warmup, 3)
    # byte model from one view's sample counts (the ray form of the view's pixels)
    pr = renderer.persp_rays(cams_d[0] if hi > lo else cams[0].to(dev), w, h, f)
    pr = svox_b200.Rays(*[t.contiguous() for t in pr])
    vis, cf, _ = csrc.march_stats(tree._spec(), svox_b200.render._rays_spec_from_rays(pr),
                                  renderer._get_options(fast))
    per_view = w * h * 12 + 8 * vis.sum().item() + 4 * (K - 1) * cf.sum().item()
    del pr
    out = {}
    if rank == 0:
        H.sampler.start()        # sampled through the warm-up and timed steps of both variants
    for name, fn in (("plain", step), ("frozen_tree", step_frozen)):
        for _ in range(warm):
            fn()
        ms = H.timed(fn, a.steps)
        out[name] = {"ms_per_step": ms, "value": n_px / ms / 1e3,
                     "ms_per_view": ms / max(hi - lo, 1)}
    if rank == 0:
        H.sampler.ensure(step)
    clocks = H.sampler.stop() if rank == 0 else None
    ms_step = out["plain"]["ms_per_step"]
    e2e = None
    if not a.no_e2e:
        host_img = torch.empty((h, w, 3), dtype=torch.float32).pin_memory()
        buf = torch.empty_like(cams_d)

        def e2e_step(k):
            buf.copy_(cams_h, non_blocking=True)
            img = step(0, buf)
            if img is not None:
                host_img.copy_(img, non_blocking=True)       # the last view travels back
            torch.cuda.current_stream().synchronize()
        e2e_step(0)
        ms_e2e = H.timed(e2e_step, a.steps)
        e2e = {"value": n_px / ms_e2e / 1e3, "unit": UNIT,
               "h2d_bytes_per_step": int(cams_h.numel() * 4),
               "d2h_bytes_per_step": int(host_img.numel() * 4), "ms_per_step": ms_e2e,
               "h2d": "camera matrices from pinned host memory; the last rendered view is "
                      "copied back to pinned host memory"}
    peak, peak_src = peaks()
    ms_view = out["frozen_tree"]["ms_per_view"]
    line = {
        "metric": METRICS[a.workload], "value": n_px / ms_step / 1e3, "unit": UNIT,
        "n_gpus": world, "steps": a.steps, "warmup": warm, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload_name(a), "views_per_gpu": hi - lo,
                   "parallelism": f"whole views dealt to {world} GPU(s), tree replicated, no "
                                  "collective",
                   "l2": f"inputs larger than L2 ({tree.data.numel() * 4 / 1e9:.2f} GB tree data)",
                   "visits_per_ray": vis.sum().item() / (w * h),
                   "contrib_per_ray": cf.sum().item() / (w * h)},
        "variants": out,
        # the march alone (index kept by renderer.frozen_tree()) against the byte model of a view
        "roofline": {"bound": "hbm", "kernel": "render_queue_kernel, forward, pixel rays "
                                               "(volume_render_image)",
                     "achieved": per_view / ms_view / 1e6, "peak": peak, "unit": "GB/s",
                     "frac": per_view / ms_view / 1e6 / peak, "traffic": None,
                     "peak_source": peak_src, "ms_per_launch": ms_view,
                     "algorithmic_bytes_per_launch": per_view},
        "e2e": e2e, "gpu_launches": 5 * (hi - lo) * a.steps, "clocks": clocks,
    }
    if rank == 0 and world == 1 and not a.no_cpu_baseline:
        val, ms, info = cpu_arm(a, 2, 1, budget_s=20.0)
        info.update(value=val, unit=UNIT, ms_per_step=ms)
        line["cpu_baseline"] = info
    csrc.check_device_status()
    if rank == 0:
        print(json.dumps(line), flush=True)
    H.done()


if __name__ == "__main__":
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "train":
        run_train(args)
    elif args.workload == "query":
        run_query(args)
    else:
        run_image(args)
