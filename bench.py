#!/usr/bin/env python3
"""Benchmark of the plane-sweep cost-volume hot path: forward + backward, voxel*views per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one forward (CostVolume) plus one backward (CostVolumeGrad) over one batch of synthetic
input.  A unit of work is one (b,h,w,d) voxel x one source view; units per step = B*H*W*D*N.
At N GPUs every rank processes its own batch item of the workload (batch sharding, no collective
in the data path): weak scaling.  `--shard depth` instead splits ONE item's depth range over the
ranks and all-reduces the partial gradients (strong scaling; exercises the NCCL exchange).

The line printed by rank 0 carries
  value        device-timed throughput with inputs resident in HBM (CUDA events, max over ranks)
  e2e          the same work through the public op functions from pinned HOST buffers, with every
               host<->device copy inside the timed region
  roofline     the dominant kernel against the measured HBM copy bandwidth
  cpu_baseline the reference's kernel source compiled for the host cores (a bounded sample)
`--impl reference` times only that CPU implementation (all host threads) and prints the same line.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

TRAFFIC_FILE = os.path.join(ROOT, "profiles", "dram_traffic.json")
KERNEL_SOURCES = ("cv_packed.cuh", "cv_tuned.cuh", "cv_project.cuh", "chop_common.cuh", "cv_launch.cuh")
CONV_SOURCES = ("sc_umma.cu", "sc_common.cuh", "sc_abi.cu")


def cost_volume_config(workload, shard, B, N, C, H, W, D):
    """`config` of a CostVolume line; the CUDA arm and the reference arm print the same dictionary."""
    return {"workload": "%s: CostVolume fwd+bwd fp32, B=%d per GPU, V=%d, C=%d, %dx%d, D=%d, MEAN" %
                        (workload, B, N + 1, C, H, W, D),
            "shard": shard,
            "l2": "inputs_exceed_l2 (cost and cost_grad are %d MB each, L2 is 126 MB)" % (B * H * W * D * C * 4 // 2**20)}


def kernel_source_digest(names=KERNEL_SOURCES):
    """sha1 over the kernel sources a workload compiles from: ties a recorded ncu figure to the code it was taken on."""
    import hashlib
    h = hashlib.sha1()
    for name in names:
        with open(os.path.join(ROOT, "custom_helper_op_b200", "csrc", name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def recorded_counters(workload, which, names=KERNEL_SOURCES):
    """The ncu figures of one kernel of a workload, as written into profiles/dram_traffic.json when the capture was
    summarised (dram_bytes = dram__bytes_read.sum + dram__bytes_write.sum per launch; tensor_pipe_util where it
    applies).  None if there is no record, or if the kernel sources have changed since (a stale figure is worse
    than none)."""
    try:
        rec = json.load(open(TRAFFIC_FILE))[workload]
        if rec.get("source_sha1") != kernel_source_digest(names):
            return None
        return rec[which]
    except Exception:
        return None


def recorded_traffic(workload, which):
    rec = recorded_counters(workload, which)
    return None if rec is None else float(rec["dram_bytes"])

LAUNCHES_PER_STEP = 3
METRIC = "cost_volume_fwd_bwd_voxel_views_per_s"
UNIT = "voxel*views/s"


# ------------------------------------------------------------------------------------------------
# workload description and algorithmic traffic
# ------------------------------------------------------------------------------------------------
def workload_dims(name):
    from custom_helper_op_b200 import synth
    c = dict(synth.CONFIGS[name])
    return dict(kind=c["kind"], B=c["B"], N=c["V"] - 1, C=c["C"], H=c["H"], W=c["W"], D=c["D"],
                G=c.get("groups", 1))


def algorithmic_bytes(w, feat_bytes=4):
    """Compulsory HBM traffic of one forward and one backward call: every tensor touched once,
    gathers and atomics assumed to be served by L2."""
    B, N, C, H, W, D = w["B"], w["N"], w["C"], w["H"], w["W"], w["D"]
    Vx = B * H * W * D
    Co = C if w["kind"] == 1 else w["G"]
    F = (1 + N) * B * H * W * C * feat_bytes
    P = 4 * (B * H * W + B * D) if w["kind"] == 1 else 4 * Vx
    fwd = F + P + 4 * Vx * Co + 4 * Vx
    bwd = 4 * Vx * Co + 4 * Vx + F + P + 4 * (1 + N) * B * H * W * C + (4 * B * H * W if w["kind"] == 1 else 4 * Vx)
    return fwd, bwd


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.samples = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self, t0, t1):
        rows = []
        for ts, line in self.samples:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                rows.append((ts, float(parts[0]), float(parts[1]), parts[3:7]))
            except ValueError:
                continue
        inside = [r for r in rows if t0 <= r[0] <= t1]
        window = "timed_region"
        if len(inside) < 3:
            inside, window = rows, "timed_region_plus_probe_loop"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "window": "unavailable"}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in inside for n, v in zip(names, r[3]) if v.lower().startswith("active")})
        return {"sm_mhz": float(np.median([r[1] for r in inside])), "sm_max_mhz": inside[0][2], "reasons": reasons,
                "samples": len(inside), "window": window}


# ------------------------------------------------------------------------------------------------
# CPU reference (the reference's kernel bodies compiled for the host, or the C restatement)
# ------------------------------------------------------------------------------------------------
def cpu_reference_run(workload, budget_s, steps=1, warmup=0):
    """Time forward+backward on the host cores over a band of image rows sized to `budget_s` per
    step.  Returns (units_per_s, info)."""
    import oracle
    from custom_helper_op_b200 import synth
    impl, kind = ("ref", "reference") if oracle.have_ref() else ("port", "port")
    w = synth.make(workload, with_grad=False)
    dims = workload_dims(workload)
    cores = oracle.max_threads()
    H, W, D, N, B = dims["H"], dims["W"], dims["D"], dims["N"], dims["B"]

    def run(rows, reps):
        ref = np.ascontiguousarray(w["ref"][:1, :rows])
        base = np.ascontiguousarray(w["base_plane"][:1, :rows])
        src, offs, Rs, Ts = w["src"][:1], w["offsets"][:1], w["Rs"][:1], w["Ts"][:1]
        cg = np.random.default_rng(1).standard_normal((1, rows, W, D, dims["C"])).astype(np.float32)
        best = []
        for _ in range(reps):
            t0 = time.perf_counter()
            cost, mask = oracle.cost_fwd(1, ref, src, base, offs, Rs, Ts, impl=impl, nthreads=cores)
            oracle.cost_bwd(1, ref, src, base, offs, Rs, Ts, cg, mask, impl=impl, nthreads=cores)
            best.append(time.perf_counter() - t0)
        return best

    # calibrate on a thin band, then size the sample
    probe_rows = max(2, H // 32)
    t_probe = min(run(probe_rows, 2))
    rows = int(min(H, max(probe_rows, probe_rows * budget_s / max(t_probe, 1e-6))))
    for _ in range(warmup):
        run(rows, 1)
    times = run(rows, max(1, steps))
    units = rows * W * D * N  # one batch item
    t = float(np.median(times))
    info = {"kind": kind, "cores": cores,
            "sample": "rows 0..%d of %d of one batch item (all %d depth planes, %d source views), median of %d" %
                      (rows, H, D, N, len(times)),
            "ms_per_step": t * 1e3, "units_per_step": units}
    return units / t, info


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def gpu_main(args):
    import torch
    import torch.distributed as dist

    from custom_helper_op_b200 import synth
    from custom_helper_op_b200.python.ops import custom_helper_ops as ops

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus != world and world > 1:
        raise SystemExit("--gpus %d does not match WORLD_SIZE %d" % (args.gpus, world))
    if args.gpus > 1 and world == 1:
        raise SystemExit("launch N>1 with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    dims = workload_dims(args.workload)
    if dims["kind"] != 1:
        raise SystemExit("bench.py times the CostVolume (v1) workloads; %s is a parity-test case" % args.workload)
    B, N, C, H, W, D = dims["B"], dims["N"], dims["C"], dims["H"], dims["W"], dims["D"]

    # synthetic inputs: rank r takes batch item r of a global batch of `world` items
    wl = synth.make(args.workload, with_grad=False)
    rng = np.random.default_rng(synth.CONFIG_SEEDS[args.workload] + 1000 * rank)
    if world > 1:
        wl["ref"] = rng.standard_normal(wl["ref"].shape).astype(np.float32)
        wl["src"] = rng.standard_normal(wl["src"].shape).astype(np.float32)
    host = {k: torch.from_numpy(np.ascontiguousarray(v)).pin_memory() for k, v in wl.items()}
    t = {k: v.to(dev, non_blocking=True) for k, v in host.items()}
    d_lo, d_hi = 0, D
    if args.shard == "depth" and world > 1:
        from custom_helper_op_b200 import shard
        mine = shard.partition(B, D, world)[rank][0]   # B = 1: every rank gets one depth range of the item
        d_lo, d_hi = mine.d_begin, mine.d_end
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    cost_grad = torch.randn((B, H, W, D, C), device=dev, generator=gen)
    cost = torch.empty((B, H, W, D, C), device=dev)
    mask = torch.empty((B, H, W, D, 1), dtype=torch.int32, device=dev)
    grads = (torch.empty((B, H, W, C), device=dev), torch.empty((B, N, H, W, C), device=dev),
             torch.empty((B, H, W, 1), device=dev))
    packed = None
    if args.shard == "depth" and world > 1:
        n_el = sum(g.numel() for g in grads)
        packed = torch.empty(n_el, device=dev)
        views, o = [], 0
        for g in grads:
            views.append(packed[o:o + g.numel()].view(g.shape))
            o += g.numel()
        grads = tuple(views)
    drange = None if (d_lo, d_hi) == (0, D) else (d_lo, d_hi)

    def fwd():
        ops.cost_forward(1, t["ref"], t["src"], t["base_plane"], t["offsets"], t["Rs"], t["Ts"], d_range=drange,
                         out=(cost, mask))

    if drange is None:
        # full-range call: the library zero-fills the gradient outputs itself
        def bwd():
            return ops.cost_backward(1, t["ref"], t["src"], t["base_plane"], t["offsets"], t["Rs"], t["Ts"],
                                     cost_grad, mask)
    else:
        # depth shard: partial gradients into one packed buffer, summed over the ranks by NCCL
        def bwd():
            packed.zero_()
            ops.cost_backward(1, t["ref"], t["src"], t["base_plane"], t["offsets"], t["Rs"], t["Ts"], cost_grad, mask,
                              d_range=drange, accumulate_into=grads)
            dist.all_reduce(packed)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        fwd()
        bwd()
    barrier()

    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    t_wall0 = time.time()
    for i in range(K):
        ev[i][0].record()
        fwd()
        ev[i][1].record()
        bwd()
        ev[i][2].record()
    barrier()
    t_wall1 = time.time()
    total_ms = ev[0][0].elapsed_time(ev[K - 1][2])
    fwd_ms = float(np.mean([e[0].elapsed_time(e[1]) for e in ev]))
    bwd_ms = float(np.mean([e[1].elapsed_time(e[2]) for e in ev]))
    if world > 1:
        tt = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        total_ms = float(tt.item())
    ms_per_step = total_ms / K
    units_rank = B * H * W * (d_hi - d_lo) * N
    units_total = units_rank * world if args.shard == "batch" else B * H * W * D * N
    value = units_total / (ms_per_step * 1e-3)

    # A short probe loop after the timed region so the clock sampler sees load even for small K.  Every
    # rank runs the same number of steps (derived from the reduced step time, identical on all ranks):
    # with depth sharding a step contains a collective, so the ranks must stay in lockstep.
    if ms_per_step * K < 1000.0 and not args.profile:
        n_probe = int(min(20000, max(1, 1000.0 / max(ms_per_step, 1e-3))))
        for _ in range(n_probe):
            fwd()
            bwd()
        barrier()
    if rank == 0:
        sampler.stop()

    # ---- end to end through the public op functions with host buffers (rank-local, N-way total) ----
    e2e = None
    if args.shard == "batch" and not args.profile:
        from custom_helper_op_b200.host import HostPipeline
        h_cg = torch.empty(cost_grad.shape, dtype=torch.float32).pin_memory()
        h_cg.copy_(cost_grad)
        h_out = dict(cost=torch.empty(cost.shape).pin_memory(), mask=torch.empty(mask.shape, dtype=torch.int32).pin_memory(),
                     ref_grad=torch.empty(grads[0].shape).pin_memory(), src_grad=torch.empty(grads[1].shape).pin_memory(),
                     base_plane_grad=torch.empty(grads[2].shape).pin_memory())
        # the public host-buffer entry: chunked over depth, copies in both directions overlap the kernels
        pipe = HostPipeline(B, N, H, W, C, D, dev, nchunks=args.e2e_chunks)
        h2d, d2h = pipe.h2d_bytes, pipe.d2h_bytes

        def e2e_step():
            pipe.run(host, h_cg, h_out)

        ke = max(3, min(K, 20))
        for _ in range(2):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(ke):
            e2e_step()
        barrier()
        dt = (time.perf_counter() - t0) / ke
        if world > 1:
            tt = torch.tensor([dt], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            dt = float(tt.item())
        e2e = {"value": units_rank * world / dt, "unit": UNIT, "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(d2h), "ms_per_step": dt * 1e3, "steps": ke}
        # copy-only probe: the step's host->device and device->host bytes from the same pinned buffers, both directions
        # at once, no kernel, all ranks together - the floor the host side sets for ms_per_step at this N
        s_a, s_b = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

        def copy_only():
            with torch.cuda.stream(s_a):
                for k in t:
                    t[k].copy_(host[k], non_blocking=True)
                cost_grad.copy_(h_cg, non_blocking=True)
            with torch.cuda.stream(s_b):
                h_out["cost"].copy_(cost, non_blocking=True)
                h_out["mask"].copy_(mask, non_blocking=True)
                for name, g_ in zip(("ref_grad", "src_grad", "base_plane_grad"), grads):
                    h_out[name].copy_(g_, non_blocking=True)
            s_a.synchronize()
            s_b.synchronize()

        copy_only()
        barrier()
        t0 = time.perf_counter()
        for _ in range(ke):
            copy_only()
        barrier()
        dtc = (time.perf_counter() - t0) / ke
        if world > 1:
            tt = torch.tensor([dtc], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            dtc = float(tt.item())
        e2e["copy_only_ms"] = dtc * 1e3
        e2e["copy_only_gbs_per_rank"] = (h2d + d2h) / dtc / 1e9
        e2e["copy_only_gbs_aggregate"] = (h2d + d2h) * world / dtc / 1e9
        del pipe, h_cg, h_out

    # ---- the legs that exercise the sharding module: one item split by depth, and the large batch dealt out ----
    depth_leg = c3_leg = None
    if args.shard == "batch" and not args.profile and not args.no_extra_legs:
        del cost, mask, cost_grad
        torch.cuda.empty_cache()
        if world > 1:
            depth_leg = depth_shard_leg(args, rank, world, dev, ms_per_step)
        c3_leg = c3_batch_leg(args, rank, world, dev)

    if rank == 0:
        fwd_b, bwd_b = algorithmic_bytes(dict(dims, D=(d_hi - d_lo)))
        peak, peak_kind = measured_peak()
        dom = ("CostVolumeGrad kernel (+ the zero fill of the gradient outputs)", bwd_b, bwd_ms, "bwd") if bwd_ms >= fwd_ms else \
              ("CostVolume kernel", fwd_b, fwd_ms, "fwd")
        ach = dom[1] / (dom[2] * 1e-3) / 1e9
        # DRAM bytes per launch of the dominant kernel from the recorded ncu capture of this workload; null when the
        # kernel sources are newer than the record
        traffic = recorded_traffic(args.workload, dom[3]) if (args.shard == "batch" and d_lo == 0 and d_hi == D) else None
        roof = {"bound": "hbm", "kernel": dom[0], "achieved": ach, "peak": peak, "peak_source": peak_kind,
                "unit": "GB/s", "frac": ach / peak, "traffic": traffic,
                "fwd": {"ms": fwd_ms, "algorithmic_bytes": fwd_b, "gbs": fwd_b / (fwd_ms * 1e-3) / 1e9},
                "bwd": {"ms": bwd_ms, "algorithmic_bytes": bwd_b, "gbs": bwd_b / (bwd_ms * 1e-3) / 1e9,
                        "note": "includes the zero-fill kernel of the three gradient outputs"},
                "fwd_plus_bwd_frac": (fwd_b + bwd_b) / (ms_per_step * 1e-3) / 1e9 / peak}
        cpu = None
        if world == 1 and not args.no_cpu_baseline and not args.profile:
            v, info = cpu_reference_run(args.workload, budget_s=6.0, steps=3)
            cpu = {"value": v, "unit": UNIT, "cores": info["cores"], "kind": info["kind"], "sample": info["sample"]}
            # the reference's CPU-sized configuration (BASELINE configs[0]) in full, beside the sample of this workload
            v0, info0 = cpu_reference_run("c0_cpu", budget_s=1e9, steps=5, warmup=1)
            cpu["c0_cpu"] = {"value": v0, "unit": UNIT, "cores": info0["cores"], "kind": info0["kind"],
                             "sample": info0["sample"], "ms_per_step": info0["ms_per_step"]}
        out = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K,
               "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
               "scaling": "weak" if args.shard == "batch" else "strong", "vs_baseline": None, "dtype": "f32",
               "data": "synthetic",
               "config": cost_volume_config(args.workload, args.shard, B, N, C, H, W, D),
               "clocks": sampler.summary(t_wall0, t_wall1), "e2e": e2e,
               # per step: the forward kernel, one zero-fill kernel over the three gradient outputs, the gradient kernel
               "gpu_launches": LAUNCHES_PER_STEP * K,
               "roofline": roof, "cpu_baseline": cpu}
        if depth_leg is not None:
            out["depth_shard"] = depth_leg
        if c3_leg is not None:
            out["c3"] = c3_leg
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def depth_shard_leg(args, rank, world, dev, n1_ms):
    """ONE item of the workload split over all ranks by depth range (shard.partition(1, D, world)): every rank runs
    forward + backward on its planes and the partial [ref_grad | src_grad | base_plane_grad] are summed by one NCCL
    all-reduce on a packed buffer, inside the timed region.  Consecutive steps alternate between two packed buffers,
    so a step's all-reduce overlaps the next step's forward (shard.PipelinedReducer).  `check` compares the reduced
    gradients with this rank's own full-range backward on the same inputs, outside the timed region."""
    import torch
    import torch.distributed as dist

    from custom_helper_op_b200 import shard, synth
    from custom_helper_op_b200.python.ops import custom_helper_ops as ops

    dims = workload_dims(args.workload)
    B, N, C, H, W, D = 1, dims["N"], dims["C"], dims["H"], dims["W"], dims["D"]
    wl = synth.make(args.workload, with_grad=False)          # the same item on every rank
    t = {k: torch.from_numpy(np.ascontiguousarray(v[:1])).to(dev) for k, v in wl.items()}
    a = (t["ref"], t["src"], t["base_plane"], t["offsets"], t["Rs"], t["Ts"])
    gen = torch.Generator(device=dev)
    gen.manual_seed(4321)                                     # the same upstream gradient on every rank
    cost_grad = torch.randn((B, H, W, D, C), device=dev, generator=gen)
    cost = torch.empty((B, H, W, D, C), device=dev)
    mask = torch.empty((B, H, W, D, 1), dtype=torch.int32, device=dev)
    mine = shard.partition(1, D, world)[rank][0]
    d0, d1 = mine.d_begin, mine.d_end
    shapes = [(B, H, W, C), (B, N, H, W, C), (B, H, W, 1)]
    pipe = shard.PipelinedReducer(shapes, torch.float32, dev, dist.group.WORLD)

    def step():
        if d1 > d0:
            ops.cost_forward(1, *a, d_range=(d0, d1), out=(cost, mask))
        views = pipe.next_views()                             # joins the all-reduce issued two steps ago
        if d1 > d0:
            ops.cost_backward(1, *a, cost_grad, mask, d_range=(d0, d1), zero_into=tuple(views))
        else:
            pipe.slots[pipe.k % 2].zero_()
        return pipe.reduce_async()

    def sync():
        dist.barrier()
        torch.cuda.synchronize()

    for _ in range(5):
        step()
    pipe.finish()
    sync()
    K = max(20, min(args.steps, 200))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        last = step()
    pipe.finish()
    e1.record()
    sync()
    ms = e0.elapsed_time(e1) / K
    # the collective alone (no overlap), and a serial step for comparison
    red = shard.GradReducer(shapes, torch.float32, dev, dist.group.WORLD, zero=True)
    for _ in range(3):
        red.all_reduce()
    sync()
    e0.record()
    for _ in range(20):
        red.all_reduce()
    e1.record()
    sync()
    ar_ms = e0.elapsed_time(e1) / 20
    e0.record()
    for _ in range(20):
        if d1 > d0:
            ops.cost_forward(1, *a, d_range=(d0, d1), out=(cost, mask))
            ops.cost_backward(1, *a, cost_grad, mask, d_range=(d0, d1), zero_into=tuple(red.views))
        red.all_reduce()
    e1.record()
    sync()
    serial_ms = e0.elapsed_time(e1) / 20
    stats = torch.tensor([ms, ar_ms, serial_ms], device=dev, dtype=torch.float64)
    dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    ms, ar_ms, serial_ms = (float(x) for x in stats.tolist())
    # result check, outside the timed region: the reduced gradients of the last step against this rank's own
    # full-range gradient (the full mask comes from a full-range forward)
    got = [g.clone() for g in pipe.result(last)]
    ops.cost_forward(1, *a, out=(cost, mask))
    want = ops.cost_backward(1, *a, cost_grad, mask)
    scale_err, elem_err = 0.0, 0.0
    for g, w_ in zip(got, want):
        diff = (g - w_).abs()
        top = float(w_.abs().max())
        scale_err = max(scale_err, float(diff.max()) / max(top, 1e-30))
        elem_err = max(elem_err, float((diff / (1e-4 * w_.abs() + 1e-5 * top)).max()))
    chk = torch.tensor([scale_err, elem_err], device=dev, dtype=torch.float64)
    dist.all_reduce(chk, op=dist.ReduceOp.MAX)
    units = H * W * D * N
    return {"what": "one %s item split by depth over %d ranks, packed all-reduce of %.1f MB per step in the timed region, "
                    "overlapped with the next step's forward" % (args.workload, world, sum(int(np.prod(s_)) for s_ in shapes) * 4 / 1e6),
            "ms_per_step": ms, "value": units / (ms * 1e-3), "unit": UNIT, "steps": K, "planes_per_rank": d1 - d0,
            "speedup_vs_n1": n1_ms / ms, "allreduce_ms": ar_ms, "serial_ms_per_step": serial_ms,
            "check": {"max_scale_relative_error": float(chk[0]), "elementwise_excess_rtol1e-4_atol1e-5max": float(chk[1]),
                      "pass": bool(float(chk[0]) <= 1e-4 and float(chk[1]) <= 1.0)}}


def c3_batch_leg(args, rank, world, dev):
    """BASELINE configs[3]: B=8, V=7, C=32, 296x400, D=256 (inverse-depth planes), bf16 features, dealt out by
    shard.partition(8, 256, world) and run through shard.sharded_forward_backward: with world <= 8 every rank owns
    whole items (8/world each) and nothing is exchanged; with more ranks than items the depth ranges of an item are
    all-reduced.  Features are drawn on the device (N(0,1) rounded to bf16), cameras and depths as in synth."""
    import torch
    import torch.distributed as dist

    from custom_helper_op_b200 import shard, synth

    cfg = synth.CONFIGS["c3_large"]
    Bt, N, C, H, W, D = cfg["B"], cfg["V"] - 1, cfg["C"], cfg["H"], cfg["W"], cfg["D"]
    plan = shard.partition(Bt, D, world)
    groups = shard.make_groups(plan) if world > 1 else {}
    inputs = {}
    lo, hi = cfg["depth_range"]
    offs = torch.tensor(1.0 / np.linspace(1.0 / lo, 1.0 / hi, D), dtype=torch.float32, device=dev)[None]
    for sh in plan[rank]:
        b = sh.item
        gen = torch.Generator(device=dev)
        gen.manual_seed(20245 * 100 + b)
        Rs, Ts = synth.random_cameras(np.random.default_rng(20245 * 100 + b), 1, N, H, W)
        inputs[b] = dict(ref=torch.randn((1, H, W, C), device=dev, generator=gen).bfloat16(),
                         src=torch.randn((1, N, H, W, C), device=dev, generator=gen).bfloat16(),
                         base_plane=torch.zeros((1, H, W, 1), device=dev), offsets=offs,
                         Rs=torch.from_numpy(Rs.astype(np.float32)).to(dev), Ts=torch.from_numpy(Ts.astype(np.float32)).to(dev))
    cost = torch.empty((1, H, W, D, C), device=dev)
    mask = torch.empty((1, H, W, D, 1), dtype=torch.int32, device=dev)
    cost_grad = torch.randn((1, H, W, D, C), device=dev)
    fwd, bwd = shard.cuda_compute_fns(buffers=(cost, mask))

    def step():
        return shard.sharded_forward_backward(rank, plan, groups, inputs, lambda b, c_: cost_grad, fwd, bwd, dev)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    step()
    sync()
    K = 3
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        res = step()
    e1.record()
    sync()
    ms = e0.elapsed_time(e1) / K
    seen = float(sum((r[1] > 0).float().mean().item() for r in res.values() if r[1] is not None) / max(1, len(res)))
    if world > 1:
        tt = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
    units = Bt * H * W * D * N
    fwd_b, bwd_b = algorithmic_bytes(dict(kind=1, B=Bt, N=N, C=C, H=H, W=W, D=D, G=1), feat_bytes=2)
    peak, _ = measured_peak()
    return {"what": "c3_large: CostVolume fwd+bwd, bf16 features / fp32 accumulate, B=%d, V=%d, C=%d, %dx%d, D=%d; "
                    "%d item(s) per rank" % (Bt, N + 1, C, H, W, D, len(plan[rank])),
            "ms_per_step": ms, "value": units / (ms * 1e-3), "unit": UNIT, "steps": K, "items_per_rank": len(plan[rank]),
            "algorithmic_bytes": fwd_b + bwd_b, "hbm_frac_per_gpu": (fwd_b + bwd_b) / world / (ms * 1e-3) / 1e9 / peak,
            "voxels_seen_fraction": seen}


def sparse_conv_main(args):
    """Secondary workload (not the headline line): manifold 3-D convolution forward + backward, c4:
    B=1, 256x320, 9-plane band, 3x3x3, 16->16 channels, bf16 storage / fp32 accumulate.  Single GPU."""
    import torch

    from custom_helper_op_b200 import _lib, synth
    from custom_helper_op_b200.python.ops import custom_helper_ops as ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    w = synth.manifold_conv(20246)
    img = torch.from_numpy(w["images"]).to(dev).to(torch.bfloat16)
    flt = torch.from_numpy(w["filters"]).to(dev).to(torch.bfloat16)
    og = torch.from_numpy(w["out_grad"]).to(dev).to(torch.bfloat16)
    bp = torch.from_numpy(w["base_plane"]).to(dev)
    defv = torch.zeros((), dtype=torch.bfloat16, device=dev)
    B, H, W, D, Cin = img.shape
    Cout = flt.shape[4]
    nvox = B * H * W * D
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > L2: the tensors (24 MB each) would stay resident

    def step():
        ops.sparse_conv3d_forward(img, flt, defv, bp)
        ops.sparse_conv3d_backward(img, flt, defv, bp, og)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    for i in range(K):
        if not args.profile:
            flush.zero_()
        ev[i][0].record()
        ops.sparse_conv3d_forward(img, flt, defv, bp)
        ev[i][1].record()
        ops.sparse_conv3d_backward(img, flt, defv, bp, og)
        ev[i][2].record()
    torch.cuda.synchronize()
    fwd_ms = float(np.mean([e[0].elapsed_time(e[1]) for e in ev]))
    bwd_ms = float(np.mean([e[1].elapsed_time(e[2]) for e in ev]))
    # algorithmic bytes: every activation tensor once (bf16), weights, base_plane
    act = nvox * Cin * 2
    fwd_b = act + nvox * Cout * 2 + 27 * Cin * Cout * 2 + B * H * W * 4
    bwd_b = 2 * (act + nvox * Cout * 2) + act + 27 * Cin * Cout * 6 + 2 * B * H * W * 4   # wgrad reads img+og, dgrad reads og writes img_grad
    flops_fwd = 2.0 * nvox * 27 * Cin * Cout
    peak, peak_kind = measured_peak()
    tpeak = 1643.8
    try:
        tpeak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
    except Exception:
        pass
    ms = fwd_ms + bwd_ms
    rec_f = recorded_counters("c4_sparse_conv", "fwd", CONV_SOURCES)
    rec_w = recorded_counters("c4_sparse_conv", "wgrad", CONV_SOURCES)
    out = {"metric": "sparse_conv3d_fwd_bwd_voxels_per_s", "value": nvox / (ms * 1e-3), "unit": "voxels/s", "n_gpus": 1,
           "steps": K, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
           "config": {"workload": "c4_sparse_conv: SparseConv3DFast fwd+bwd, B=%d, %dx%d, band of %d planes, 3x3x3, %d->%d, bf16/fp32-acc"
                                  % (B, H, W, D, Cin, Cout), "l2": "flushed between steps (256 MB write)"},
           "gpu_launches": 4 * K, "umma_timeouts": _lib.lib().chop_umma_timeouts(),
           "roofline": {"bound": "hbm", "kernel": "sc_umma_rows_kernel (forward)", "achieved": fwd_b / (fwd_ms * 1e-3) / 1e9, "peak": peak,
                        "peak_source": peak_kind, "unit": "GB/s", "frac": fwd_b / (fwd_ms * 1e-3) / 1e9 / peak,
                        "traffic": (rec_f or {}).get("dram_bytes"),
                        # sm__pipe_tensor_cycles_active of the recorded ncu captures (null once sc_umma.cu has changed)
                        "tensor_pipe_util": None if rec_f is None else {"fwd": rec_f.get("tensor_pipe_util"),
                                                                        "wgrad": (rec_w or {}).get("tensor_pipe_util")},
                        "fwd": {"ms": fwd_ms, "algorithmic_bytes": fwd_b, "tflops": flops_fwd / (fwd_ms * 1e-3) / 1e12,
                                "tensor_frac_of_measured": flops_fwd / (fwd_ms * 1e-3) / 1e12 / tpeak},
                        "bwd": {"ms": bwd_ms, "algorithmic_bytes": bwd_b, "tflops": 2 * flops_fwd / (bwd_ms * 1e-3) / 1e12,
                                "tensor_frac_of_measured": 2 * flops_fwd / (bwd_ms * 1e-3) / 1e12 / tpeak}},
           "cpu_baseline": None, "e2e": None}
    print(json.dumps(out), flush=True)


def secondary_main(args):
    """Secondary workloads, one JSON line each (not the headline): device-timed ops that sit either side of the
    hot path.  c4_updown: the strided manifold convolution (2,2,2) that halves the c4 band, the transposed
    convolution that brings it back and SparsePad, bf16, forward + gradient each.  c1_v3: CostVolumeV3 (8 groups,
    MEAN) forward + gradient on the c1 shapes, fp32.  c1_fa: FeatureAggregate forward + gradient on the c1 shapes
    (the forward allocates its 1 GB output every step, as the op does).  c1_min: CostVolume and CostAggregate with the MIN
    reduction, forward + gradient each, c1 shapes, fp32.  c2_min: CostVolumeV2 MIN on the first cascade stage; c2_cascade: CostVolumeV2 MEAN on all three.  c3_item: one batch item of the large configuration.  Single GPU, L2 flushed between steps."""
    import torch

    from custom_helper_op_b200 import synth
    from custom_helper_op_b200.python.ops import custom_helper_ops as ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    K, Wm = args.steps, max(args.warmup, 3)
    peak, peak_kind = measured_peak()

    def timed(fns):
        """Mean milliseconds of every callable in fns, K steps, L2 flushed before each step."""
        for _ in range(Wm):
            for f in fns:
                f()
        torch.cuda.synchronize()
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(fns) + 1)] for _ in range(K)]
        for i in range(K):
            flush.zero_()
            ev[i][0].record()
            for j, f in enumerate(fns):
                f()
                ev[i][j + 1].record()
        torch.cuda.synchronize()
        return [float(np.mean([e[j].elapsed_time(e[j + 1]) for e in ev])) for j in range(len(fns))]

    if args.workload == "c4_updown":
        w = synth.manifold_conv(20246)
        bf = torch.bfloat16
        fine = torch.from_numpy(w["images"]).to(dev).to(bf)
        flt = torch.from_numpy(w["filters"]).to(dev).to(bf)
        bp = torch.from_numpy(w["base_plane"]).to(dev)
        B, H, W_, D, C = fine.shape
        st = (2, 2, 2)
        coarse = ops.sparse_conv3d_forward(fine, flt, 0.0, bp, st)
        og_c, og_f = torch.randn_like(coarse), torch.randn_like(fine)
        size = (H, W_, D)
        padded_bp = bp[:, :coarse.shape[1] * 2, :coarse.shape[2] * 2].contiguous()
        padded = ops.sparse_pad_forward(coarse, padded_bp, st)
        og_p = torch.randn_like(padded)
        names = ["down_fwd", "down_bwd", "up_fwd", "up_bwd", "pad_fwd", "pad_bwd"]
        ms = timed([lambda: ops.sparse_conv3d_forward(fine, flt, 0.0, bp, st),
                    lambda: ops.sparse_conv3d_backward(fine, flt, 0.0, bp, og_c, st),
                    lambda: ops.sparse_conv3d_transpose_forward(coarse, flt, 0.0, bp, size, st),
                    lambda: ops.sparse_conv3d_transpose_backward(coarse, flt, 0.0, bp, size, og_f, st),
                    lambda: ops.sparse_pad_forward(coarse, padded_bp, st),
                    lambda: ops.sparse_pad_backward(coarse, padded_bp, og_p, st)])
        nf, nc, npad = fine.numel() * 2, coarse.numel() * 2, padded.numel() * 2
        wb, bpb = flt.numel() * 2, bp.numel() * 4
        alg = [nf + nc + wb + bpb, 2 * (nf + nc) + nf + 3 * wb + 2 * bpb, nc + nf + wb + bpb,
               2 * (nf + nc) + nc + 3 * wb + 2 * bpb, nc + npad + bpb, npad // 8 + nc + bpb]
        units, unit = fine.numel() // C, "fine voxels/s"
        desc = "c4_updown: SparseConv3DFast strides (2,2,2) + SparseConv3DTransposeFast + SparsePad, fine band %dx%dx%d, " \
               "3x3x3, %d->%d, bf16/fp32-acc" % (H, W_, D, C, C)
        launches = 10
    elif args.workload == "c1_min":
        # the MIN reduction (the reference layers' default): CostVolume and CostAggregate, forward + gradient
        wl = synth.make("c1_mvsnet", with_grad=False)
        t = {k: torch.from_numpy(v).to(dev) for k, v in wl.items()}
        B, H, W_, C = t["ref"].shape
        D, N = t["offsets"].shape[1], t["src"].shape[1]
        a = (t["ref"], t["src"], t["base_plane"], t["offsets"], t["Rs"], t["Ts"])
        cost1, mask1 = ops.cost_forward(1, *a, "MIN")
        cg1 = torch.randn_like(cost1)
        cost3, mask3 = ops.cost_forward(3, *a, "MIN")
        cg3 = torch.randn_like(cost3)
        names = ["cost_volume_min_fwd", "cost_volume_min_bwd", "cost_aggregate_min_fwd", "cost_aggregate_min_bwd"]
        ms = timed([lambda: ops.cost_forward(1, *a, "MIN", out=(cost1, mask1)),
                    lambda: ops.cost_backward(1, *a, cg1, mask1, "MIN"),
                    lambda: ops.cost_forward(3, *a, "MIN", out=(cost3, mask3)),
                    lambda: ops.cost_backward(3, *a, cg3, mask3, "MIN")])
        feats = (1 + N) * B * H * W_ * C * 4
        vox = B * H * W_ * D
        small = 4 * B * H * W_
        # cost and arg indices are both [.., C] for CostVolume MIN, one value per voxel for CostAggregate
        alg = [feats + 8 * vox * C + small, 2 * feats + 8 * vox * C + 2 * small,
               feats + 8 * vox + small, 2 * feats + 8 * vox + 2 * small]
        units, unit = 2 * vox * N, UNIT
        desc = "c1_min: CostVolume and CostAggregate, MIN, fwd+bwd fp32, B=%d, V=%d, C=%d, %dx%d, D=%d" % (B, N + 1, C, H, W_, D)
        launches = 10
    elif args.workload == "c2_cascade":
        # CostVolumeV2 MEAN on the three cascade stages (bf16 features, 8 groups), forward + gradient each
        names, ms, alg, units = [], [], [], 0
        parts = []
        for st_name in ("c2_stage1", "c2_stage2", "c2_stage3"):
            wl = synth.make(st_name, with_grad=False)
            t = {k: (torch.from_numpy(v).to(dev) if isinstance(v, np.ndarray) else v) for k, v in wl.items()}
            B, H, W_, C = t["ref"].shape
            D, N, G = t["depth_grid"].shape[3], t["src"].shape[1], 8
            a = (t["ref"].bfloat16(), t["src"].bfloat16(), t["depth_grid"], None, t["Rs"], t["Ts"])
            cost, mask = ops.cost_forward(2, *a, "MEAN", G)
            cg = torch.randn_like(cost)
            m2 = timed([lambda: ops.cost_forward(2, *a, "MEAN", G, out=(cost, mask)),
                        lambda: ops.cost_backward(2, *a, cg, mask, "MEAN", G)])
            feats = (1 + N) * B * H * W_ * C * 2
            vox = B * H * W_ * D
            names += [st_name + "_fwd", st_name + "_bwd"]
            ms += m2
            alg += [feats + 4 * vox + 4 * vox * G + 4 * vox, feats + 4 * vox + 4 * vox * G + 4 * vox + 4 * (1 + N) * B * H * W_ * C + 4 * vox]
            units += vox * N
            parts.append("%s %.1f G units/s" % (st_name, vox * N / (sum(m2) * 1e-3) / 1e9))
            del t, a, cost, mask, cg
            torch.cuda.empty_cache()
        unit = UNIT
        desc = "c2_cascade: CostVolumeV2 MEAN fwd+bwd on the three cascade stages, bf16 features, V=5, groups=8 (" + "; ".join(parts) + ")"
        launches = 12
    elif args.workload == "c3_item":
        # one batch item of the large configuration (what one GPU holds at 8-way batch sharding), bf16 features
        # --rows H: fewer image rows (same width, planes and views, so the footprints move as in the full item) for
        # profiler captures of this workload
        wl = synth.make("c3_large", with_grad=False, B=1, **({"H": args.rows} if args.rows else {}))
        t = {k: torch.from_numpy(v).to(dev) for k, v in wl.items()}
        B, H, W_, C = t["ref"].shape
        D, N = t["offsets"].shape[1], t["src"].shape[1]
        a = (t["ref"].bfloat16(), t["src"].bfloat16(), t["base_plane"], t["offsets"], t["Rs"], t["Ts"])
        cost, mask = ops.cost_forward(1, *a)
        cg = torch.randn_like(cost)
        names = ["c3_fwd", "c3_bwd"]
        ms = timed([lambda: ops.cost_forward(1, *a, out=(cost, mask)), lambda: ops.cost_backward(1, *a, cg, mask)])
        feats = (1 + N) * B * H * W_ * C * 2
        vox = B * H * W_ * D
        small = 4 * B * H * W_ + 4 * B * D
        alg = [feats + small + 4 * vox * C + 4 * vox, 4 * vox * C + 4 * vox + feats + small + 4 * (1 + N) * B * H * W_ * C + 4 * B * H * W_]
        units, unit = vox * N, UNIT
        desc = "c3_item: CostVolume MEAN fwd+bwd, bf16 features, B=%d, V=%d, C=%d, %dx%d, D=%d" % (B, N + 1, C, H, W_, D)
        launches = 5
    elif args.workload == "c2_min":
        # CostVolumeV2 with the MIN reduction on the first cascade stage (bf16 features, 8 groups)
        wl = synth.make("c2_stage1", with_grad=False)
        t = {k: (torch.from_numpy(v).to(dev) if isinstance(v, np.ndarray) else v) for k, v in wl.items()}
        B, H, W_, C = t["ref"].shape
        D, N, G = t["depth_grid"].shape[3], t["src"].shape[1], 8
        a = (t["ref"].bfloat16(), t["src"].bfloat16(), t["depth_grid"], None, t["Rs"], t["Ts"])
        cost, mask = ops.cost_forward(2, *a, "MIN", G)
        cg = torch.randn_like(cost)
        names = ["v2_min_fwd", "v2_min_bwd"]
        ms = timed([lambda: ops.cost_forward(2, *a, "MIN", G, out=(cost, mask)),
                    lambda: ops.cost_backward(2, *a, cg, mask, "MIN", G)])
        feats = (1 + N) * B * H * W_ * C * 2
        vox = B * H * W_ * D
        alg = [feats + 4 * vox + 8 * vox * G, feats + 8 * vox + 8 * vox * G + 4 * (1 + N) * B * H * W_ * C]
        units, unit = vox * N, UNIT
        desc = "c2_min: CostVolumeV2 MIN fwd+bwd, bf16 features, B=%d, V=%d, C=%d, groups=%d, %dx%d, D=%d" % (B, N + 1, C, G, H, W_, D)
        launches = 4
    elif args.workload == "c1_fa":
        wl = synth.make("c1_mvsnet", with_grad=False)
        t = {k: torch.from_numpy(v).to(dev) for k, v in wl.items()}
        B, H, W_, C = t["ref"].shape
        D, N = t["offsets"].shape[1], t["src"].shape[1]
        a = (t["src"], t["base_plane"], t["offsets"], t["Rs"], t["Ts"])
        mapped, mask = ops.feature_aggregate_forward(*a)
        mg = torch.randn_like(mapped)
        names = ["fa_fwd", "fa_bwd"]
        ms = timed([lambda: ops.feature_aggregate_forward(*a), lambda: ops.feature_aggregate_backward(*a, mg, mask)])
        feats = N * B * H * W_ * C * 4
        vox = B * H * W_ * D
        alg = [feats + vox * N * (C * 4 + 4) + 4 * B * H * W_, 2 * feats + vox * N * (C * 4 + 4) + 8 * B * H * W_]
        units, unit = vox * N, UNIT
        desc = "c1_fa: FeatureAggregate fwd+bwd fp32, B=%d, N=%d, C=%d, %dx%d, D=%d" % (B, N, C, H, W_, D)
        launches = 4
    else:
        wl = synth.make("c1_mvsnet", with_grad=False)
        t = {k: torch.from_numpy(v).to(dev) for k, v in wl.items()}
        B, H, W_, C = t["ref"].shape
        D, N, G = t["offsets"].shape[1], t["src"].shape[1], 8
        a = (t["ref"], t["src"], t["base_plane"], t["offsets"], t["Rs"], t["Ts"])
        cost, mask = ops.cost_forward(4, *a, "MEAN", G)
        cg = torch.randn_like(cost)
        names = ["v3_fwd", "v3_bwd"]
        ms = timed([lambda: ops.cost_forward(4, *a, "MEAN", G, out=(cost, mask)),
                    lambda: ops.cost_backward(4, *a, cg, mask, "MEAN", G)])
        feats = (1 + N) * B * H * W_ * C * 4
        vox = B * H * W_ * D
        alg = [feats + 8 * vox + 4 * B * H * W_, 2 * feats + 8 * vox + 8 * B * H * W_]
        units, unit = vox * N, UNIT
        desc = "c1_v3: CostVolumeV3 fwd+bwd fp32, B=%d, V=%d, C=%d, groups=%d, %dx%d, D=%d, MEAN" % (B, N + 1, C, G, H, W_, D)
        launches = 5
    total = float(sum(ms))
    out = {"metric": args.workload + "_fwd_bwd", "value": units / (total * 1e-3), "unit": unit, "n_gpus": 1, "steps": K,
           "warmup": Wm, "ms_per_step": total, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "bf16" if args.workload == "c4_updown" else "f32", "data": "synthetic",
           "config": {"workload": desc, "l2": "flushed between steps (256 MB write)"}, "gpu_launches": launches * K,
           "roofline": {"bound": "hbm", "peak": peak, "peak_source": peak_kind, "unit": "GB/s", "traffic": None,
                        "ops": {n: {"ms": m, "algorithmic_bytes": b, "achieved": b / (m * 1e-3) / 1e9,
                                    "frac": b / (m * 1e-3) / 1e9 / peak} for n, m, b in zip(names, ms, alg)}},
           "cpu_baseline": None, "e2e": None}
    print(json.dumps(out), flush=True)


def reference_main(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dims = workload_dims(args.workload)
    K = args.steps
    budget = max(0.02, min(10.0, 150.0 / max(1, K + args.warmup)))
    v, info = cpu_reference_run(args.workload, budget_s=budget, steps=K, warmup=args.warmup)
    out = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": world, "steps": K,
           "warmup": args.warmup, "ms_per_step": info["ms_per_step"], "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           # the same dictionary as the CUDA arm prints for this workload: both arms describe one configuration
           "config": cost_volume_config(args.workload, args.shard, dims.get("B", 1), dims["N"], dims["C"], dims["H"],
                                        dims["W"], dims["D"]),
           "note": "the reference registers GPU kernels only; this is its kernel source compiled for the host and "
                   "swept over all host threads",
           "cpu_baseline": {"value": v, "unit": UNIT, "cores": info["cores"], "kind": info["kind"],
                            "sample": info["sample"]},
           "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c1_mvsnet")
    ap.add_argument("--shard", default="batch", choices=["batch", "depth"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-chunks", type=int, default=2, help="depth chunks of the host-buffer pipeline")
    ap.add_argument("--rows", type=int, default=0, help="c3_item only: image rows (default: the configuration's 296)")
    ap.add_argument("--no-extra-legs", action="store_true",
                    help="skip the depth-shard leg (N > 1) and the c3 batch leg that follow the headline measurement")
    ap.add_argument("--profile", action="store_true",
                    help="device-timed loop only (no clock probe loop, e2e leg or CPU baseline): the command to run under ncu")
    args = ap.parse_args()
    if args.workload in ("c4_updown", "c1_v3", "c1_fa", "c1_min", "c2_min", "c2_cascade", "c3_item"):
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "secondary workload: timed on the GPU only"}))
        else:
            secondary_main(args)
    elif args.workload == "c4_sparse_conv":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference has no CPU kernel for SparseConv3DFast and its "
                                                                  "GPU kernels are warp-cooperative (not compilable for the host)"}))
        else:
            sparse_conv_main(args)
    elif args.impl == "reference":
        reference_main(args)
    else:
        gpu_main(args)


if __name__ == "__main__":
    main()
