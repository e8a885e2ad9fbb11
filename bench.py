"""Headline benchmark: forward + backward surfel tracing throughput (Mrays/s) and hierarchy build time.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 3]

One "step" is one forward + backward trace of every ray of the workload against a resident
hierarchy (upstream gradient of ones on rgb), as a training iteration does. The N = 1 workload is
the configuration the metric is quoted on: 3,000,000 surfels, one 1920x1080 camera, SH degree 3,
one reflection bounce (seeded synthetic scene, see diff-surfel-tracing_b200/workloads.py).
With N > 1 every rank traces one 1920x1080 camera batch (the same synthetic batch on every rank)
of the replicated scene and the per-surfel gradients are summed with one NCCL all-reduce per
step ("weak" scaling: per-GPU work fixed, the exchange step added).

`--impl reference` times the CPU stand-in for the reference (its own shader sources compiled for
the host where that build exists, else the CPU restatement) on a bounded sample of the same
workload; the reference's OptiX path itself cannot run on this hardware/software stack.
"""
import argparse
import json
import os
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


def algorithmic_bytes(counters, R, depth_stride_floats, sh_degree, has_aux, training, backward):
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
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def cpu_sample(w, step):
    return dict(w, ray_o=w["ray_o"][::step, ::step].contiguous(), ray_d=w["ray_d"][::step, ::step].contiguous())


def run_cpu(w, kind, steps, warmup, stride=24):
    """Times the CPU stand-in on every `stride`-th pixel in both directions of the same workload."""
    from oracle import oracle as orc
    impl = "reference" if (kind == "reference" and orc.reference_built()) else "restatement"
    ws = cpu_sample(w, stride)
    t0 = time.perf_counter()
    sc = orc.Scene(w["v"])
    t_bvh = time.perf_counter() - t0
    o = orc.Oracle(sc, impl=impl, portable_exp=False)
    R = ws["ray_o"].shape[0] * ws["ray_o"].shape[1]
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        f = o.forward(ws, training=True)
        o.backward(ws, f, dict(rgb=np.ones_like(f["rgb"])))
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    ms = 1e3 * float(np.mean(times))
    return dict(value=R / (ms * 1e-3) / 1e6, unit="Mrays/s", cores=os.cpu_count(), kind="reference" if impl == "reference" else "port",
                sample=f"every {stride}th ray in both directions of the {w['ray_o'].shape[0]}x{w['ray_o'].shape[1]} ray grid ({R} rays) against the full {w['means3D'].shape[0]}-surfel scene, "
                       f"fwd+bwd, host hierarchy built in {t_bvh:.1f} s (not timed)"), ms, R


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
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    import workloads
    if args.impl == "reference":
        if rank != 0:
            return
        w = workloads.make_workload(args.config, P=args.surfels, H=args.height, W=args.width)
        cb, ms, R = run_cpu(w, "reference", max(1, min(args.steps, 5)), min(args.warmup, 1))
        line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "Mrays/s", "n_gpus": args.gpus,
                "steps": max(1, min(args.steps, 5)), "warmup": min(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": w["name"], "note": "CPU stand-in for the reference (its OptiX path cannot run here); bounded ray sample"},
                "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": "Mrays/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return

    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from diff_surfel_tracing import SurfelTracer, SurfelTracingSettings, _C
    import shard

    t0 = time.perf_counter()
    w = workloads.make_workload(args.config, P=args.surfels, H=args.height, W=args.width)
    # Configuration 5 is the scale-out protocol: 8 cameras split over the ranks (strong scaling), and every step
    # rebuilds the hierarchy before tracing. All other configurations: with N > 1 every rank traces one synthetic
    # camera batch of identical cost (weak scaling): per-GPU work is fixed, what is added is the gradient exchange.
    scale_out = args.config == 5
    total_rays = w["ray_o"].shape[0] * w["ray_o"].shape[1]
    if scale_out and world > 1:
        ro, rd = shard.shard_rays(w["ray_o"], w["ray_d"], world, rank)
        w = dict(w, ray_o=ro.contiguous(), ray_d=rd.contiguous())
    H, W = w["ray_o"].shape[:2]
    log(f"[rank {rank}] workload '{w['name']}' generated in {time.perf_counter() - t0:.1f} s")
    wc = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in w.items()}
    R, P = H * W, w["means3D"].shape[0]

    tracer = SurfelTracer().to(dev)
    st = tracer.optix_context
    st.profile(True)
    if scale_out:
        st.set_image_width(1920)          # what SurfelTracingSettings.image_width tells the module API: 1080x1920 images
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
    if rank == 0:
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
        t2 = SurfelTracer().to(dev)
        m_, s_, r_ = wc["means3D"], wc["scales"], wc["rotations"]
        vbuf = t2.build_from_surfels(m_, s_, r_, rebuild=True)
        quads_ms = timed(lambda: _C.surfel_quads(t2.optix_context, m_, s_, r_, True))
        torch_ms = timed(lambda: workloads.get_triangles(m_, s_, r_))
        st2 = t2.optix_context
        st2.profile(True)
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
        peak_n, _ = measured_peak_hbm()
        qb, rb = (36 + 48 + 24) * P, 24 * 1080 * 1920
        neighbours = {"quad_expansion": {"ms": quads_ms, "algorithmic_bytes": qb, "achieved_gbs": qb / quads_ms / 1e6,
                                         "frac_of_hbm_peak": qb / quads_ms / 1e6 / peak_n, "torch_ops_ms": torch_ms},
                      "refit_from_surfels_ms": two_ms, "refit_from_surfels_single_kernel_ms": fused_ms,
                      "build_from_surfels_ms": fused_build_ms,
                      "torch_expansion_then_refit_ms": torch_ms + refit_ms,
                      "ray_generation_1080p": {"ms": rays_ms, "algorithmic_bytes": rb, "achieved_gbs": rb / rays_ms / 1e6,
                                               "frac_of_hbm_peak": rb / rays_ms / 1e6 / peak_n}}
        del t2, vbuf

    e = torch.empty((0,), device=dev)
    shs = wc["shs"] if wc["shs"] is not None else e
    cols = wc["colors_precomp"] if wc["colors_precomp"] is not None else e
    oth = wc["others_precomp"] if wc["others_precomp"] is not None else e
    ones = torch.ones((H, W, 3), device=dev)
    z1, z2, z3 = torch.zeros((H, W, 1), device=dev), torch.zeros((H, W, 2), device=dev), torch.zeros((H, W, 3), device=dev)

    def fwd(diag=None):
        return _C.trace_surfels(st, True, w["start_from_first"], wc["ray_o"], wc["ray_d"], wc["v"], wc["bg"], wc["means3D"], shs,
                                w["sh_degree"], cols, oth, wc["opacities"], wc["scales"], 1.0, wc["rotations"], e, e, e, e,
                                False, False, w["max_trace_depth"], w["specular_threshold"], _diag=diag)

    def bwd(f, diag=None):
        return _C.trace_surfels_backward(st, w["start_from_first"], wc["ray_o"], wc["ray_d"], wc["v"], wc["bg"], wc["means3D"], shs,
                                         w["sh_degree"], cols, oth, wc["opacities"], wc["scales"], 1.0, wc["rotations"], e, e, e, e,
                                         False, False, w["max_trace_depth"], w["specular_threshold"],
                                         f[0], f[1], f[2], f[3], f[4], f[5], f[6], ones, z1, z1, z3, z1, z2, _diag=diag,
                                         _forward_serial=st.last_forward_serial)

    def step():
        if scale_out:
            tracer.build_acceleration_structure(wc["v"], wc["f"], rebuild=True)
        f = fwd()
        g = bwd(f)
        if world > 1:
            shard.allreduce_surfel_gradients(st)
        return f, g

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # counters of one forward and one backward launch (diagnostic variant of the kernels, outside the timed region)
    dfw, dbw = {}, {}
    f = fwd(dfw)
    bwd(f, dbw)
    torch.cuda.synchronize()
    cf, cb_ = dfw["counters"].cpu().numpy(), dbw["counters"].cpu().numpy()
    status = st.status()
    del f

    for _ in range(args.warmup):
        step()
    barrier()
    st.profile_read()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = st.kernel_launches()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    launches = st.kernel_launches() - launches0
    barrier()
    clocks = sampler.stop()
    ms_total = ev0.elapsed_time(ev1)
    prof = st.profile_read()
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    job_rays = total_rays if scale_out else world * R
    value = job_rays / (ms_step * 1e-3) / 1e6

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
        ih, iw = (1080, 1920) if scale_out else (H, W)
        settings = SurfelTracingSettings(ih, iw, 1.0, 1.0, wc["bg"], 1.0, z, z, w["sh_degree"], z, False, False,
                                         w["max_trace_depth"], w["specular_threshold"])
        tracer.train()

        def e2e_step():
            ro, rd = ro_h.to(dev, non_blocking=True), rd_h.to(dev, non_blocking=True)
            if scale_out:
                tracer.build_acceleration_structure(wc["v"], wc["f"], rebuild=True)
            out = tracer(ro, rd, wc["v"], leaves["means3D"], g3d, shs=shs_l, colors_precomp=col_l, others_precomp=oth_l,
                         opacities=leaves["opacities"], scales=leaves["scales"], rotations=leaves["rotations"],
                         tracer_settings=settings, start_from_first=w["start_from_first"])
            loss = out[0].sum()
            loss.backward()
            if world > 1:
                shard.allreduce_surfel_gradients(st)
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

    # roofline of the dominant kernel (the longer of the two trace kernels)
    fwd_ms = prof["forward"][0] / max(prof["forward"][1], 1)
    bwd_ms = prof["backward"][0] / max(prof["backward"][1], 1)
    peak, peak_src = measured_peak_hbm()
    sh_deg = w["sh_degree"] if w["shs"] is not None else None
    has_aux = w["others_precomp"] is not None
    bytes_f = algorithmic_bytes(cf, R, 0, sh_deg, has_aux, True, False)
    bytes_b = algorithmic_bytes(cb_, R, 0, sh_deg, has_aux, True, True)
    dom = "backward" if bwd_ms >= fwd_ms else "forward"
    dom_bytes, dom_ms = (bytes_b, bwd_ms) if dom == "backward" else (bytes_f, fwd_ms)
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9 if dom_ms > 0 else 0.0
    # DRAM bytes of one trace sequence from the ncu launch list (profiles/launch_list_config3_step.md: measured at a quarter
    # of the rays; the per-ray part is scaled to the ray count, the per-surfel part kept); only quoted for the workload it
    # was measured on
    traffic = None
    if args.config == 3 and P == 3_000_000:
        per_ray_q, per_surfel = (2.72e9 - 0.255e9, 0.255e9) if dom == "forward" else (1.41e9 - 0.705e9, 0.705e9)
        traffic = int(per_ray_q * R / 518400 + per_surfel)
    roofline = {"bound": "hbm", "kernel": f"{dom} trace sequence (k_enum gather rounds + k_{'bwd' if dom == 'backward' else 'fwd'}_shade + tail)",
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "peak_source": peak_src, "algorithmic_bytes_per_launch": int(dom_bytes),
                "kernel_ms": {"forward": fwd_ms, "backward": bwd_ms},
                "other_kernel": {"algorithmic_bytes_per_launch": int(bytes_f if dom == "backward" else bytes_b),
                                 "achieved": (bytes_f if dom == "backward" else bytes_b) / ((fwd_ms if dom == "backward" else bwd_ms) * 1e-3) / 1e9}}

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
            neighbours["cpu_cores"] = os.cpu_count()
        except Exception as ex:
            neighbours["cpu_error"] = str(ex)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        try:
            cpu_baseline, _, _ = run_cpu(w, "reference", 1, 0, stride=24 if R >= 1_000_000 else 4)
        except Exception as ex:  # the baseline is a report, never a reason to lose the GPU numbers
            cpu_baseline = {"value": None, "unit": "Mrays/s", "cores": os.cpu_count(), "kind": "port", "sample": f"failed: {ex}"}

    if rank == 0:
        per_ray = lambda c: {"segments": c[0] / R, "enumerations": c[1] / R, "nodes_visited": c[2] / R, "quads_tested": c[3] / R,
                             "slots_evaluated": c[4] / R, "contributions": c[5] / R}
        line = {"metric": METRIC, "value": value, "unit": "Mrays/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if scale_out else "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic",
                "config": {"workload": w["name"], "surfels": P, "rays_per_gpu": R, "sh_degree": w["sh_degree"],
                           "max_trace_depth": w["max_trace_depth"], "specular_threshold": w["specular_threshold"],
                           "parallelism": (f"8 cameras split over {world} GPUs, hierarchy replicated and rebuilt every step, 1 all-reduce/step" if scale_out
                                           else f"one camera batch per GPU x{world}, hierarchy replicated, 1 all-reduce/step" if world > 1 else "1 GPU"),
                           "l2": "inputs larger than L2 (hierarchy + surfel records + SH rows > 126 MB), no flush"},
                "bvh_build_ms": build_ms, "bvh_refit_ms": refit_ms, "device_status": status, "neighbours": neighbours,
                "per_ray": {"forward": per_ray(cf), "backward": per_ray(cb_)},
                "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
                "gpu_launches": launches, "clocks": clocks}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
