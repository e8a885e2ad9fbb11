"""Headline benchmark: forward + backward surfel tracing throughput (Mrays/s) and hierarchy build time.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 3]

One "step" is one forward + backward trace of every ray of the workload against a resident
hierarchy (upstream gradient of ones on rgb), as a training iteration does. The N = 1 workload is
the configuration the metric is quoted on: 3,000,000 surfels, one 1920x1080 camera, SH degree 3,
one reflection bounce (seeded synthetic scene, see diff-surfel-tracing_b200/workloads.py).
With N > 1 rank r traces the 1920x1080 camera number r of a ring of eight around the replicated
scene (rank 0: the N = 1 camera), so the ranks' costs differ as they would in training, and the
per-surfel gradients are summed with one NCCL all-reduce per step ("weak" scaling: per-GPU work
fixed, the exchange step added). The same line carries, as `scale_out`, the strong-scaling protocol
(6,000,000 surfels, eight cameras split over the ranks, two bounces, hierarchy rebuilt every step)
and, with N > 1, a check that sharded rays + all-reduce reproduce the single-GPU gradients.

`--impl reference` times the CPU stand-in for the reference (its own shader sources compiled for the
host where that build exists, else the CPU restatement) on a bounded sample of the same
workload; the reference's OptiX path itself cannot run on this hardware/software stack.
"""
import argparse
import json
import math
import os
import re
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "diff-surfel-tracing_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC = "fwd+bwd Mrays/s (3M surfels, 1080p, 1 bounce)"


def log(*a):
    print(*a, file=sys.stderr, flush=True)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.idx, self.rows, self.proc = device_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def algorithmic_bytes(counters, R, sh_degree, has_aux, training, backward):
    """Implementation-independent bytes of one launch (per-ray I/O + per-hit gathers / scatters).

    counters: [segments, enumerations, nodes, quads, slots evaluated, contributions] of the launch.
    Per evaluated slot: quad 48 B + mean 12 + scale 8 + rotation 16 + opacity 4 = 88 B.
    Per contribution: colour row (12 * (D+1)^2 B with SH, else 12), +8 B with auxiliaries,
    +4 B (forward, training: weight) or the gradient addends (backward):
    4 * (3 mean + 3 grads3D + 2 scale + 4 rotation + 1 opacity + 3 colour [+2 aux] [+3 (D+1)^2 SH]) B.
    Per ray: origin+direction 24 B, outputs 52 B, 64 B per traced segment of the per-bounce record,
    and for the backward 48 B of upstream gradients + 24 B of ray gradients.
    """
    segs, evals, cons = int(counters[0]), int(counters[4]), int(counters[5])
    ncoef = (sh_degree + 1) ** 2 if sh_degree is not None else 0
    colour = 12 * ncoef if sh_degree is not None else 12
    aux = 8 if has_aux else 0
    per_ray = 24 + 52
    if backward:
        grad = 4 * (3 + 3 + 2 + 4 + 1 + 3 + (2 if has_aux else 0) + (3 * ncoef if sh_degree is not None else 0))
        return R * (per_ray + 48 + 24) + segs * 64 + evals * 88 + cons * (colour + aux + grad)
    return R * per_ray + segs * 64 + evals * 88 + cons * (colour + aux + (4 if training else 0))


def measured_peak_hbm():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s)"


def committed_dram_traffic():
    """DRAM bytes per ray and per surfel of the forward and backward sequences, from the committed launch-list summary
    (lines `traffic.<key>: <number>`); None where the summary does not carry them."""
    path = os.path.join(ROOT, "profiles", "launch_list_config3_step.md")
    try:
        txt = open(path).read()
    except OSError:
        return None
    out = {}
    for k, v in re.findall(r"^\s*traffic\.([a-z_]+):\s*([0-9.eE+-]+)\s*$", txt, flags=re.M):
        out[k] = float(v)
    need = ("forward_bytes_per_ray", "forward_bytes_per_surfel", "backward_bytes_per_ray", "backward_bytes_per_surfel")
    return out if all(k in out for k in need) else None


def ring_camera(index, count=8, radius=4.0):
    ang = 2 * math.pi * index / count
    return (radius * math.sin(ang), -radius * math.cos(ang), 0.0)


def config_block(w, P, rays_per_gpu, world, scale_out=False):
    return {"workload": w["name"], "surfels": P, "rays_per_gpu": rays_per_gpu, "sh_degree": w["sh_degree"],
            "max_trace_depth": w["max_trace_depth"], "specular_threshold": w["specular_threshold"],
            "parallelism": (f"rows of 8 cameras dealt over {world} GPUs, hierarchy replicated and rebuilt every step, 1 all-reduce/step" if scale_out
                            else f"one camera of a ring of 8 per GPU x{world}, 4-row blocks of every camera dealt over the GPUs, hierarchy replicated, 1 all-reduce/step" if world > 1 else "1 GPU"),
            "l2": "inputs larger than L2 (hierarchy + surfel records + SH rows > 126 MB), no flush"}


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def run_cpu(w, steps, warmup, stride):
    """Times the CPU stand-in on every `stride`-th pixel in both directions of the same workload, on all host threads
    (set explicitly: launchers such as torch.distributed.run export OMP_NUM_THREADS=1)."""
    from oracle import oracle as orc
    impl = "reference" if orc.reference_built() else "restatement"
    ws = dict(w, ray_o=w["ray_o"][::stride, ::stride].contiguous(), ray_d=w["ray_d"][::stride, ::stride].contiguous())
    t0 = time.perf_counter()
    sc = orc.Scene(w["v"])
    t_bvh = time.perf_counter() - t0
    nt = host_threads()
    o = orc.Oracle(sc, impl=impl, portable_exp=False, nthreads=nt)
    R = ws["ray_o"].shape[0] * ws["ray_o"].shape[1]
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        f = o.forward(ws, training=True)
        o.backward(ws, f, dict(rgb=np.ones_like(f["rgb"])))
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    ms = 1e3 * float(np.median(times))
    return dict(value=R / (ms * 1e-3) / 1e6, unit="Mrays/s", cores=nt, kind="reference" if impl == "reference" else "port",
                sample=f"every {stride}th ray in both directions of the {w['ray_o'].shape[0]}x{w['ray_o'].shape[1]} ray grid ({R} rays) against the full "
                       f"{w['means3D'].shape[0]}-surfel scene, fwd+bwd, median of {steps} steps after {warmup} warm-up, host hierarchy built in {t_bvh:.1f} s (not timed)"), ms, R


def reference_arm(args, rank):
    """The reference's own shader sources on the host cores (rank 0 only; the other ranks have nothing to do)."""
    if rank != 0:
        return
    import workloads
    w = workloads.make_workload(args.config, P=args.surfels, H=args.height, W=args.width)
    H, W = w["ray_o"].shape[:2]
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    # a step of the 3,600-ray sample takes under a second on 16 cores; the sample shrinks when the requested step count is large
    stride = 24 if H * W >= 1_000_000 else 4
    while (H // stride) * (W // stride) * (steps + warmup) > 3600 * 60 and stride < 96:
        stride *= 2
    cb, ms, R = run_cpu(w, steps, warmup, stride)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "Mrays/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_block(w, w["means3D"].shape[0], H * W, max(1, args.gpus)),
            "note": "CPU stand-in for the reference (its OptiX path cannot run here) on a bounded ray sample of the workload `config` names",
            "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": "Mrays/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def timed(fn, n=5):
    for _ in range(2):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(n):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / n


class Stepper:
    """Forward + backward of one workload through the extension-level functions, tensors resident on the device."""

    def __init__(self, tracer, w, wc, world):
        from diff_surfel_tracing import _C
        import shard
        self._C, self.shard, self.tracer, self.st, self.w, self.wc, self.world = _C, shard, tracer, tracer.optix_context, w, wc, world
        dev = wc["means3D"].device
        H, W = wc["ray_o"].shape[:2]
        self.e = torch.empty((0,), device=dev)
        self.shs = wc["shs"] if wc["shs"] is not None else self.e
        self.cols = wc["colors_precomp"] if wc["colors_precomp"] is not None else self.e
        self.oth = wc["others_precomp"] if wc["others_precomp"] is not None else self.e
        self.ones = torch.ones((H, W, 3), device=dev)
        self.z1, self.z2, self.z3 = torch.zeros((H, W, 1), device=dev), torch.zeros((H, W, 2), device=dev), torch.zeros((H, W, 3), device=dev)
        self.ar_events = []

    def fwd(self, diag=None):
        w, wc, e = self.w, self.wc, self.e
        return self._C.trace_surfels(self.st, True, w["start_from_first"], wc["ray_o"], wc["ray_d"], wc["v"], wc["bg"], wc["means3D"], self.shs,
                                     w["sh_degree"], self.cols, self.oth, wc["opacities"], wc["scales"], 1.0, wc["rotations"], e, e, e, e,
                                     False, False, w["max_trace_depth"], w["specular_threshold"], _diag=diag)

    def bwd(self, f, diag=None):
        w, wc, e = self.w, self.wc, self.e
        return self._C.trace_surfels_backward(self.st, w["start_from_first"], wc["ray_o"], wc["ray_d"], wc["v"], wc["bg"], wc["means3D"], self.shs,
                                              w["sh_degree"], self.cols, self.oth, wc["opacities"], wc["scales"], 1.0, wc["rotations"], e, e, e, e,
                                              False, False, w["max_trace_depth"], w["specular_threshold"],
                                              f[0], f[1], f[2], f[3], f[4], f[5], f[6], self.ones, self.z1, self.z1, self.z3, self.z1, self.z2,
                                              _diag=diag, _forward_serial=self.st.last_forward_serial)

    def step(self, rebuild=False, time_allreduce=False):
        if rebuild:
            self.tracer.build_acceleration_structure(self.wc["v"], self.wc["f"], rebuild=True)
        f = self.fwd()
        g = self.bwd(f)
        if self.world > 1:
            if time_allreduce:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                self.shard.allreduce_surfel_gradients(self.st)
                b.record()
                self.ar_events.append((a, b))
            else:
                self.shard.allreduce_surfel_gradients(self.st)
        return f, g

    def allreduce_ms(self):
        ms = [a.elapsed_time(b) for a, b in self.ar_events]
        self.ar_events = []
        return float(np.mean(ms)) if ms else None


def rank_spread(value, world, dev):
    """[min, max] of a per-rank number over the ranks."""
    import torch.distributed as dist
    if world == 1:
        return [value, value]
    t = torch.tensor([value], device=dev, dtype=torch.float64)
    lo, hi = t.clone(), t.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    return [float(lo.item()), float(hi.item())]


def multi_gpu_grad_check(dev, rank, world):
    """Sharded rays + CUDA backward + all-reduce on every rank against rank 0 tracing all rays alone, on a reduced
    two-bounce scene (outside any timed region). Returns the largest relative L2 difference over the gradient tensors."""
    import torch.distributed as dist
    import workloads
    import shard
    from diff_surfel_tracing import SurfelTracer
    w = workloads.make_workload(5, P=90_000, H=8, W=54 * 96)
    wc = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in w.items()}
    tracer = SurfelTracer().to(dev)
    tracer.optix_context.set_image_width(96)
    tracer.build_acceleration_structure(wc["v"], wc["f"], rebuild=True)
    names = ("rot", "means", "g3d", "shs", "colors", "others", "opac", "scales")
    idx = dict(rot=10, means=2, g3d=3, shs=5, colors=6, others=7, opac=8, scales=9)

    def run(ro, rd):
        s = Stepper(tracer, w, dict(wc, ray_o=ro.contiguous(), ray_d=rd.contiguous()), 1)
        f = s.fwd()
        g = s.bwd(f)
        return {n: g[idx[n]].clone() for n in names}

    ro, rd = shard.shard_rays(wc["ray_o"], wc["ray_d"], world, rank)
    mine = run(ro, rd)
    flat = torch.cat([mine[n].reshape(-1) for n in names])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM)
    worst = 0.0
    if rank == 0:
        full = run(wc["ray_o"], wc["ray_d"])
        off = 0
        for n in names:
            cnt = full[n].numel()
            got, want = flat[off:off + cnt].double(), full[n].reshape(-1).double()
            off += cnt
            m = torch.isfinite(want) & torch.isfinite(got)
            den = float(want[m].norm())
            err = float((got[m] - want[m]).norm()) / den if den > 0 else float((got[m] - want[m]).norm())
            worst = max(worst, err)
    t = torch.tensor([worst], device=dev, dtype=torch.float64)
    dist.broadcast(t, 0)
    return float(t.item())


def scale_out_record(dev, rank, world, steps=3, warmup=1):
    """The strong-scaling protocol: 6,000,000 surfels, eight 1920x1080 cameras split over the ranks, two bounces,
    every step = hierarchy rebuild + forward + backward (+ all-reduce). Device-timed, max over ranks."""
    import torch.distributed as dist
    import workloads
    import shard
    from diff_surfel_tracing import SurfelTracer
    w = workloads.make_workload(5)
    total_rays = w["ray_o"].shape[0] * w["ray_o"].shape[1]
    if world > 1:
        # every rank takes 4-row blocks of every camera round-robin: equal shares of every camera and every part of the frame
        ro, rd = shard.shard_image_rows(w["ray_o"], w["ray_d"], world, rank, 1080, 1920)
        w = dict(w, ray_o=ro, ray_d=rd)
    wc = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in w.items()}
    tracer = SurfelTracer().to(dev)
    st = tracer.optix_context
    st.set_image_width(1920)
    st.profile(1)
    s = Stepper(tracer, w, wc, world)
    for _ in range(warmup):
        s.step(rebuild=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    st.profile_read()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        s.step(rebuild=True, time_allreduce=True)
    b.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / steps
    pr = st.profile_read()
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    log_info = st.chunk_log()
    rec = {"workload": w["name"], "surfels": w["means3D"].shape[0], "total_rays": total_rays, "rays_per_gpu": w["ray_o"].shape[0] * w["ray_o"].shape[1],
           "split": "4-row blocks of every camera dealt round-robin over the ranks" if world > 1 else "none",
           "steps": steps, "warmup": warmup, "scaling": "strong", "value": total_rays / (ms * 1e-3) / 1e6, "unit": "Mrays/s", "ms_per_step": ms,
           "build_ms": rank_spread(pr["build"][0] / max(pr["build"][1], 1), world, dev),
           "forward_ms": rank_spread(pr["forward"][0] / max(pr["forward"][1], 1), world, dev),
           "backward_ms": rank_spread(pr["backward"][0] / max(pr["backward"][1], 1), world, dev),
           "allreduce_ms": s.allreduce_ms(), "allreduce_bytes": int(st.grad_bucket.numel() * 4) if st.grad_bucket is not None else None,
           "chunk_log_gb": log_info["records_held"] * log_info["bytes_per_record"] / 1e9,
           "chunk_log_records_wanted": log_info["records_wanted"], "chunk_log_records_held": log_info["records_held"],
           "rays_retraced_by_backward": (st.round_counts() or [0])[0], "device_status": st.status()}
    del s, tracer, wc
    torch.cuda.empty_cache()
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=3)
    ap.add_argument("--surfels", type=int, default=None, help="override the surfel count (profiling on a smaller case)")
    ap.add_argument("--height", type=int, default=None)
    ap.add_argument("--width", type=int, default=None)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-scale-out", action="store_true", help="skip the strong-scaling sub-record")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        reference_arm(args, rank)
        return
    args.warmup = max(args.warmup, 3)

    import workloads
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from diff_surfel_tracing import SurfelTracer, SurfelTracingSettings, _C

    t0 = time.perf_counter()
    w = workloads.make_workload(args.config, P=args.surfels, H=args.height, W=args.width)
    # Configuration 5 on its own (--config 5) is the strong-scaling protocol as the main line. All other configurations:
    # with N > 1 rank r traces camera r of the ring (weak scaling; the exchange step is what is added).
    scale_out = args.config == 5
    total_rays = w["ray_o"].shape[0] * w["ray_o"].shape[1]
    dealt_width = None
    if scale_out and world > 1:
        import shard
        ro, rd = shard.shard_image_rows(w["ray_o"], w["ray_d"], world, rank, 1080, 1920)
        w = dict(w, ray_o=ro, ray_d=rd)
    elif args.config == 3 and world > 1:
        # weak scaling: the job is one camera of the ring per GPU (camera 0 is the N = 1 workload). The cameras' costs
        # differ by up to a third, so a rank does not trace "its" camera: 4-row blocks of every camera are dealt round-robin
        # over the ranks and every rank traces 1/N of each of the N images, one image's worth of rays in all.
        import shard
        ih, iw = w["ray_o"].shape[:2]
        cams = [workloads.pinhole_rays(ih, iw, 50.0, ring_camera(c)) for c in range(world)]
        ro = torch.stack([c[0].reshape(-1, 3) for c in cams]); rd = torch.stack([c[1].reshape(-1, 3) for c in cams])
        total_rays = world * ih * iw
        ro, rd = shard.shard_image_rows(ro, rd, world, rank, ih, iw)
        w = dict(w, ray_o=ro, ray_d=rd)
        dealt_width = iw
    H, W = w["ray_o"].shape[:2]
    log(f"[rank {rank}] workload '{w['name']}' generated in {time.perf_counter() - t0:.1f} s")
    wc = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in w.items()}
    R, P = H * W, w["means3D"].shape[0]

    tracer = SurfelTracer().to(dev)
    st = tracer.optix_context
    st.profile(1)
    if scale_out:
        st.set_image_width(1920)          # what SurfelTracingSettings.image_width tells the module API: 1080x1920 images
    elif dealt_width:
        st.set_image_width(dealt_width)
    # hierarchy: build (timed 3x) and refit (timed 3x)
    for _ in range(3):
        tracer.build_acceleration_structure(wc["v"], wc["f"], rebuild=True)
    torch.cuda.synchronize()
    st.profile_read()
    for _ in range(3):
        tracer.build_acceleration_structure(wc["v"], wc["f"], rebuild=True)
    build_ms = st.profile_read()["build"]
    for _ in range(3):
        tracer.build_acceleration_structure(wc["v"], wc["f"], rebuild=False)
    refit_ms = st.profile_read()["build"]
    build_ms, refit_ms = build_ms[0] / max(build_ms[1], 1), refit_ms[0] / max(refit_ms[1], 1)

    # the steps on either side of the tracer in the reference's pipeline, on a handle of their own: quad
    # expansion (get_triangles), expansion fused with the refit, the same with torch tensor ops, ray generation
    neighbours = None
    peak, peak_src = measured_peak_hbm()
    if rank == 0:
        t2 = SurfelTracer().to(dev)
        m_, s_, r_ = wc["means3D"], wc["scales"], wc["rotations"]
        vbuf = t2.build_from_surfels(m_, s_, r_, rebuild=True)
        quads_ms = timed(lambda: _C.surfel_quads(t2.optix_context, m_, s_, r_, True))
        torch_ms = timed(lambda: workloads.get_triangles(m_, s_, r_))
        st2 = t2.optix_context
        st2.profile(1)
        timed(lambda: t2.build_from_surfels(m_, s_, r_, rebuild=False, vertices=vbuf))
        two = st2.profile_read()["build"]            # the library's own events around its kernels, as for bvh_refit_ms
        two_ms = two[0] / max(two[1], 1)
        st2.set_single_kernel_refit(True)
        timed(lambda: t2.build_from_surfels(m_, s_, r_, rebuild=False, vertices=vbuf))
        fused = st2.profile_read()["build"]
        fused_ms = fused[0] / max(fused[1], 1)
        st2.set_single_kernel_refit(False)
        timed(lambda: t2.build_from_surfels(m_, s_, r_, rebuild=True, vertices=vbuf))
        fused_b = st2.profile_read()["build"]
        fused_build_ms = fused_b[0] / max(fused_b[1], 1)
        Kc, Rc, Tc = workloads.pinhole_camera(1080, 1920, 50.0, (4.0, 0.0, 0.0))
        rays_ms = timed(lambda: t2.get_rays(1080, 1920, Kc, Rc, Tc))
        qb, rb = (36 + 48 + 24) * P, 24 * 1080 * 1920
        neighbours = {"quad_expansion": {"ms": quads_ms, "algorithmic_bytes": qb, "achieved_gbs": qb / quads_ms / 1e6,
                                         "frac_of_hbm_peak": qb / quads_ms / 1e6 / peak, "torch_ops_ms": torch_ms},
                      "refit_from_surfels_ms": two_ms, "refit_from_surfels_single_kernel_ms": fused_ms,
                      "build_from_surfels_ms": fused_build_ms,
                      "torch_expansion_then_refit_ms": torch_ms + refit_ms,
                      "ray_generation_1080p": {"ms": rays_ms, "algorithmic_bytes": rb, "achieved_gbs": rb / rays_ms / 1e6,
                                               "frac_of_hbm_peak": rb / rays_ms / 1e6 / peak}}
        del t2, vbuf

    s = Stepper(tracer, w, wc, world)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # counters of one forward and one backward launch (diagnostic variant of the kernels, outside the timed region)
    dfw, dbw = {}, {}
    f = s.fwd(dfw)
    s.bwd(f, dbw)
    torch.cuda.synchronize()
    cf, cb_ = dfw["counters"].cpu().numpy(), dbw["counters"].cpu().numpy()
    status = st.status()
    del f

    for _ in range(args.warmup):
        s.step(rebuild=scale_out)
    barrier()
    st.profile_read()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = st.kernel_launches()
    ev0.record()
    for _ in range(args.steps):
        s.step(rebuild=scale_out, time_allreduce=True)
    ev1.record()
    launches = st.kernel_launches() - launches0
    barrier()
    clocks = sampler.stop()
    ms_total = ev0.elapsed_time(ev1)
    prof = st.profile_read()
    allreduce_ms = s.allreduce_ms()
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    job_rays = total_rays if (scale_out or dealt_width) else world * R
    value = job_rays / (ms_step * 1e-3) / 1e6
    fwd_ms = prof["forward"][0] / max(prof["forward"][1], 1)
    bwd_ms = prof["backward"][0] / max(prof["backward"][1], 1)
    per_rank = {"forward_ms": rank_spread(fwd_ms, world, dev), "backward_ms": rank_spread(bwd_ms, world, dev)}
    log_info = st.chunk_log()
    retraced = (st.round_counts() or [0])[0]          # rays the logged backward had to queue for re-tracing (its round 0)

    # the gather kernel alone: a measuring pass of its own with an event pair around every launch
    st.profile(2)
    for _ in range(2):
        s.step(rebuild=scale_out)
    torch.cuda.synchronize()
    gather = st.profile_launches("gather")
    pass_prof = st.profile_read()
    st.profile(1)
    gather_ms_step = sum(gather) / 2 if gather else 0.0
    pass_fwd_ms = pass_prof["forward"][0] / max(pass_prof["forward"][1], 1)

    # end to end through the public module API: pinned host rays in, loss out, every step
    e2e = None
    if not args.no_e2e:
        ro_h, rd_h = w["ray_o"].pin_memory(), w["ray_d"].pin_memory()
        leaves = {k: wc[k].clone().requires_grad_(True) for k in ("means3D", "opacities", "scales", "rotations")}
        shs_l = wc["shs"].clone().requires_grad_(True) if wc["shs"] is not None else None
        col_l = wc["colors_precomp"].clone().requires_grad_(True) if wc["colors_precomp"] is not None else None
        oth_l = wc["others_precomp"].clone().requires_grad_(True) if wc["others_precomp"] is not None else None
        g3d = torch.zeros_like(wc["means3D"], requires_grad=True)
        z = torch.zeros(1, device=dev)
        # image size as the module API hears it: this rank's rows of every image when the rays were dealt out
        ih, iw = (W // 1920, 1920) if scale_out else (W // dealt_width, dealt_width) if dealt_width else (H, W)
        settings = SurfelTracingSettings(ih, iw, 1.0, 1.0, wc["bg"], 1.0, z, z, w["sh_degree"], z, False, False,
                                         w["max_trace_depth"], w["specular_threshold"])
        tracer.train()
        tracer.set_gradient_group(world > 1)          # the gradient sum happens inside the autograd backward

        def e2e_step():
            ro, rd = ro_h.to(dev, non_blocking=True), rd_h.to(dev, non_blocking=True)
            if scale_out:
                tracer.build_acceleration_structure(wc["v"], wc["f"], rebuild=True)
            out = tracer(ro, rd, wc["v"], leaves["means3D"], g3d, shs=shs_l, colors_precomp=col_l, others_precomp=oth_l,
                         opacities=leaves["opacities"], scales=leaves["scales"], rotations=leaves["rotations"],
                         tracer_settings=settings, start_from_first=w["start_from_first"])
            loss = out[0].sum()
            loss.backward()
            for t_ in list(leaves.values()) + [shs_l, col_l, oth_l, g3d]:
                if t_ is not None:
                    t_.grad = None
            return float(loss.item())

        for _ in range(2):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        barrier()
        e2e_ms = 1e3 * (time.perf_counter() - t0) / args.steps
        if world > 1:
            t = torch.tensor([e2e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        e2e = {"value": job_rays / (e2e_ms * 1e-3) / 1e6, "unit": "Mrays/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": int(ro_h.numel() * 4 + rd_h.numel() * 4), "d2h_bytes_per_step": 4}
        tracer.set_gradient_group(False)
        del leaves, shs_l, col_l, oth_l, g3d

    # roofline of the dominant sequence (the longer of the two trace sequences), and of the gather kernel inside it
    sh_deg = w["sh_degree"] if w["shs"] is not None else None
    has_aux = w["others_precomp"] is not None
    bytes_f = algorithmic_bytes(cf, R, sh_deg, has_aux, True, False)
    bytes_b = algorithmic_bytes(cb_, R, sh_deg, has_aux, True, True)
    dom = "backward" if bwd_ms >= fwd_ms else "forward"
    dom_bytes, dom_ms = (bytes_b, bwd_ms) if dom == "backward" else (bytes_f, fwd_ms)
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9 if dom_ms > 0 else 0.0
    traffic = None
    tr = committed_dram_traffic()
    if tr is not None and args.config == 3:
        traffic = int(tr[f"{dom}_bytes_per_ray"] * R + tr[f"{dom}_bytes_per_surfel"] * P)
    # bytes the hierarchy walk fetches (implementation-dependent: 64 B per node visited, 48 B + 4 B per quad tested, 64 B per
    # evaluated slot), served by the L2 cache; against the measured L2 streaming bandwidth
    try:
        l2_peak = st.read_bandwidth(64 << 20, 50)
    except Exception as ex:
        l2_peak = None
        log(f"L2 bandwidth probe failed: {ex}")
    fetched = int(cf[2]) * 64 + int(cf[3]) * 52 + int(cf[4]) * 64
    l2 = {"peak_gbs": l2_peak, "peak_how": "64 MB buffer read 50 times with 16-byte L1-bypassing loads, CUDA events",
          "bytes_fetched_per_ray_forward": fetched / R, "achieved_gbs": fetched / (fwd_ms * 1e-3) / 1e9 if fwd_ms > 0 else None}
    l2["frac"] = l2["achieved_gbs"] / l2_peak if (l2_peak and l2["achieved_gbs"]) else None
    roofline = {"bound": "hbm", "kernel": f"{dom} trace sequence (gather rounds + composite kernels + tail)" if dom == "forward" else "backward trace sequence (logged re-composite + gradient reductions)",
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "traffic_source": "profiles/launch_list_config3_step.md (ncu, quarter resolution, scaled by rays and surfels)" if traffic else None,
                "peak_source": peak_src, "algorithmic_bytes_per_launch": int(dom_bytes),
                "kernel_ms": {"forward": fwd_ms, "backward": bwd_ms},
                "other_kernel": {"algorithmic_bytes_per_launch": int(bytes_f if dom == "backward" else bytes_b),
                                 "achieved": (bytes_f if dom == "backward" else bytes_b) / ((fwd_ms if dom == "backward" else bwd_ms) * 1e-3) / 1e9},
                "gather_kernel": {"name": "k_enum", "launches_per_step": len(gather) // 2, "ms_per_step": gather_ms_step,
                                  "forward_ms_of_that_pass": pass_fwd_ms,
                                  "share_of_that_forward": gather_ms_step / pass_fwd_ms if pass_fwd_ms > 0 else None,
                                  "how": "a pass of its own with an event pair around every launch; per-launch timing runs the rounds of the whole "
                                         "frame one after another (the timed steps run them as four slices on four streams, whose kernels overlap), "
                                         "so this is the kernel's serial time",
                                  "achieved_vs_forward_algorithmic_bytes": bytes_f / (gather_ms_step * 1e-3) / 1e9 / peak if gather_ms_step > 0 else None},
                "l2": l2}

    if rank == 0 and world == 1 and not args.no_cpu and neighbours is not None:
        # the CPU restatement of the two neighbouring steps on the host cores (whole workload, a few repetitions)
        try:
            from oracle import oracle as orc
            Kc, Rc, Tc = workloads.pinhole_camera(1080, 1920, 50.0, (4.0, 0.0, 0.0))
            orc.surfel_quads(w["means3D"], w["scales"], w["rotations"])
            t0 = time.perf_counter()
            for _ in range(3):
                orc.surfel_quads(w["means3D"], w["scales"], w["rotations"])
            neighbours["quad_expansion"]["cpu_ms"] = 1e3 * (time.perf_counter() - t0) / 3
            orc.pinhole_rays(1080, 1920, Kc.numpy(), Rc.numpy(), Tc.numpy())
            t0 = time.perf_counter()
            for _ in range(3):
                orc.pinhole_rays(1080, 1920, Kc.numpy(), Rc.numpy(), Tc.numpy())
            neighbours["ray_generation_1080p"]["cpu_ms"] = 1e3 * (time.perf_counter() - t0) / 3
            neighbours["cpu_cores"] = host_threads()
        except Exception as ex:
            neighbours["cpu_error"] = str(ex)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        try:
            cpu_baseline, _, _ = run_cpu(w, 3, 1, stride=24 if R >= 1_000_000 else 4)
        except Exception as ex:  # the baseline is a report, never a reason to lose the GPU numbers
            cpu_baseline = {"value": None, "unit": "Mrays/s", "cores": host_threads(), "kind": "port", "sample": f"failed: {ex}"}

    bucket_bytes = int(st.grad_bucket.numel() * 4) if st.grad_bucket is not None else None
    # free the main workload before the sub-records allocate theirs
    del s, wc, tracer
    torch.cuda.empty_cache()
    grad_check = None
    if world > 1:
        grad_check = {"rel_l2_max": multi_gpu_grad_check(dev, rank, world), "tolerance": 1e-3,
                      "what": "reduced two-bounce scene: rays sharded over the ranks, CUDA backward, all-reduce, against rank 0 tracing all rays"}
    so = None
    if not args.no_scale_out and args.config == 3 and args.surfels is None and args.height is None:
        try:
            so = scale_out_record(dev, rank, world)
        except Exception as ex:
            so = {"error": str(ex)}

    if rank == 0:
        per_ray = lambda c: {"segments": c[0] / R, "enumerations": c[1] / R, "nodes_visited": c[2] / R, "quads_tested": c[3] / R,
                             "slots_evaluated": c[4] / R, "contributions": c[5] / R}
        line = {"metric": METRIC, "value": value, "unit": "Mrays/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if scale_out else "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": config_block(w, P, R, world, scale_out),
                "bvh_build_ms": build_ms, "bvh_refit_ms": refit_ms, "device_status": status, "neighbours": neighbours,
                "per_ray": {"forward": per_ray(cf), "backward": per_ray(cb_)}, "per_rank": per_rank,
                "allreduce_ms": allreduce_ms, "allreduce_bytes": bucket_bytes if world > 1 else None,
                "chunk_log": {"gb_held": log_info["records_held"] * log_info["bytes_per_record"] / 1e9, "records_wanted": log_info["records_wanted"],
                              "records_held": log_info["records_held"], "rays_retraced_by_backward": retraced},
                "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "multi_gpu_grad_check": grad_check, "scale_out": so,
                "gpu_launches": launches, "clocks": clocks}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if grad_check is not None and not (grad_check["rel_l2_max"] <= 1e-3):
        sys.exit(f"multi-GPU gradient check failed: relative L2 {grad_check['rel_l2_max']}")


if __name__ == "__main__":
    main()
