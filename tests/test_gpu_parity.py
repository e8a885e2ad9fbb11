"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle on the same seeded inputs.

Bars (from the task statement): per-ray contributing hit sequences equal, forward outputs within
1e-4 absolute, every gradient within 1e-3 relative L2. The forward path is specified as an exact
sequence of IEEE operations, so the forward checks are in fact made bit for bit.
"""
import numpy as np
import pytest
import torch

import helpers as hp

pytestmark = pytest.mark.gpu

FWD_ATOL = 1e-4
GRAD_RTOL = 1e-3


@pytest.fixture(scope="module")
def C():
    from diff_surfel_tracing import _C
    assert torch.cuda.is_available()
    _C.lib()
    return _C


def _build(C, wc, wave=False):
    st = C.OptiXStateWrapper("")
    if wave:
        st.set_wavefront_min_rays(0)      # run the wavefront rounds even on these small ray counts
    C.build_acceleration_structure(st, wc["v"], wc["f"], 1)
    return st


def test_quad_frames_bit_exact(C, oracle_mod):
    w = hp.reduced_workload(3)
    wc = hp.to_cuda(w)
    st = _build(C, wc)
    got = C.debug_quad_frames(st).cpu().numpy()
    want = oracle_mod.Scene(w["v"], brute=True).quad_records()
    assert got.shape == want.shape
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert st.status() == 0


@pytest.mark.parametrize("config", [1, 3, 4])
def test_knearest_walk_equals_exhaustive(C, oracle_mod, config):
    """Hierarchy walk == exhaustive testing on the GPU == the oracle's enumerator, bit for bit."""
    w = hp.reduced_workload(config)
    if config != 1:
        w = hp.workloads.make_workload(config, P=8000, H=hp.REDUCED[config]["H"], W=hp.REDUCED[config]["W"])
    wc = hp.to_cuda(w)
    st = _build(C, wc)
    ro, rd = wc["ray_o"].reshape(-1, 3)[::7].contiguous(), wc["ray_d"].reshape(-1, 3)[::7].contiguous()
    k_walk, c_walk = C.debug_knearest(st, ro, rd, brute=False)
    k_all, c_all = C.debug_knearest(st, ro, rd, brute=True)
    assert torch.equal(c_walk, c_all)
    assert torch.equal(k_walk, k_all)
    assert st.status() == 0
    sc = oracle_mod.Scene(w["v"], brute=True)
    ron, rdn = ro.cpu().numpy(), rd.cpu().numpy()
    kw = k_walk.cpu().numpy().view(np.uint64)
    cw = c_walk.cpu().numpy()
    for r in range(0, ron.shape[0], 13):
        keys = sc.knearest(ron[r], rdn[r])
        assert len(keys) == cw[r]
        assert np.array_equal(keys, kw[r, :len(keys)])
    assert int(cw.max()) > 0


def _forward_pair(C, oracle_mod, config, hit_cap=320, wave=False):
    w = hp.reduced_workload(config)
    wc = hp.to_cuda(w)
    st = _build(C, wc, wave)
    diag = dict(hit_cap=hit_cap)
    got = hp.cuda_forward(C, st, wc, training=True, diag=diag)
    torch.cuda.synchronize()
    assert st.status() == 0
    sc = oracle_mod.Scene(w["v"], brute=False)
    orc = oracle_mod.Oracle(sc, impl="restatement", hit_cap=hit_cap, portable_exp=True)
    want = orc.forward(w, training=True)
    return w, wc, st, got, want, diag, orc


@pytest.mark.parametrize("wave", [False, True], ids=["per-ray", "wavefront"])
@pytest.mark.parametrize("config", [1, 2, 3, 4, 5])
def test_forward_parity(C, oracle_mod, config, wave):
    w, wc, st, got, want, diag, _ = _forward_pair(C, oracle_mod, config, wave=wave)
    H, W = w["ray_o"].shape[:2]
    # contributing hit sequences: exact, on every ray, over all bounces
    cnt = diag["hit_cnt"].cpu().numpy()
    assert np.array_equal(cnt, want["hit_cnt"])
    assert np.array_equal(diag["hit_log"].cpu().numpy(), want["hit_log"])
    assert cnt.max() > 0
    for k in ("rgb", "dpt", "acc", "norm", "aux", "mid"):
        g = got[k].cpu().numpy().reshape(want[k].shape)
        err = np.abs(g - want[k]).max()
        assert err <= FWD_ATOL, f"{k}: max abs err {err}"
        # the forward path is specified operation by operation: expect identical bits
        assert np.array_equal(g.view(np.uint32), want[k].view(np.uint32)), f"{k} not bit-identical"
    assert float(got["dist"].abs().max()) == 0.0
    assert got["dist"].shape == (H, W, 3)
    wet = got["wet"].cpu().numpy()
    assert np.abs(wet - want["wet"]).max() <= FWD_ATOL * max(1.0, float(np.abs(want["wet"]).max()))
    c = diag["counters"].cpu().numpy()
    assert c[5] == want["stats"][3] and c[4] == want["stats"][2] and c[1] == want["stats"][0]


@pytest.mark.parametrize("mode", ["per-ray", "wavefront", "chunk-log"])
@pytest.mark.parametrize("config", [1, 2, 3, 4, 5])
def test_backward_parity(C, oracle_mod, config, mode):
    """Three routes to the same gradients: re-trace one thread per ray, re-trace in wavefront rounds,
    and re-compositing the chunks the forward call logged (no hierarchy walk)."""
    w, wc, st, got, want, diag, orc = _forward_pair(C, oracle_mod, config, hit_cap=0, wave=(mode == "wavefront"))
    serial = st.last_forward_serial if mode == "chunk-log" else 0
    assert st.last_forward_serial != 0
    gen = torch.Generator().manual_seed(100 + config)
    H, W = w["ray_o"].shape[:2]
    # unit upstream gradients on the outputs the configuration names, plus a seeded random run on all of them
    for upstream in ("unit", "random"):
        if upstream == "unit":
            up = {k: torch.ones((H, W, 3 if k in ("rgb", "norm") else 2 if k == "aux" else 1)) for k in w["upstream"]}
        else:
            up = {k: torch.randn((H, W, c), generator=gen) for k, c in (("rgb", 3), ("dpt", 1), ("acc", 1), ("norm", 3), ("aux", 2))}
        dg = {}
        gb = hp.cuda_backward(C, st, wc, got, {k: v.cuda() for k, v in up.items()}, diag=dg, serial=serial)
        torch.cuda.synchronize()
        assert st.status() == 0
        cb = dg["counters"].cpu().numpy()
        assert (cb[2] == 0) == (mode == "chunk-log")        # nodes visited: none when the log is used
        ob = orc.backward(w, want, {k: v.numpy() for k, v in up.items()})
        for k in hp.GRAD_KEYS:
            g = gb[k].cpu().numpy().reshape(ob[k].shape)
            if not np.isfinite(ob[k]).all():
                # the reference divides by the accumulated specular weight (backward.cu:771); where that is 0 both sides are non-finite
                assert np.array_equal(np.isfinite(g), np.isfinite(ob[k])), k
                m = np.isfinite(ob[k])
                g, o = g[m], ob[k][m]
            else:
                o = ob[k]
            e = hp.rel_l2(g, o)
            assert e <= GRAD_RTOL, f"config {config} {mode} {upstream} grad {k}: rel L2 {e}"
        assert float(gb["grads3D_abs"].abs().max()) == 0.0 and float(gb["trans"].abs().max()) == 0.0


def test_stale_chunk_log_is_not_used(C, oracle_mod):
    """A backward whose forward is no longer the one the handle's log belongs to must re-trace."""
    w = hp.reduced_workload(1)
    wc = hp.to_cuda(w)
    st = _build(C, wc)
    f1 = hp.cuda_forward(C, st, wc)
    s1 = st.last_forward_serial
    H, W = w["ray_o"].shape[:2]
    up = {"rgb": torch.ones((H, W, 3), device="cuda")}
    ref = hp.cuda_backward(C, st, wc, f1, up, serial=0)
    # a second forward over other rays replaces the log
    wc2 = dict(wc, ray_o=wc["ray_o"].flip(0).contiguous(), ray_d=wc["ray_d"].flip(0).contiguous())
    hp.cuda_forward(C, st, wc2)
    assert st.last_forward_serial != s1
    dg = {}
    g = hp.cuda_backward(C, st, wc, f1, up, diag=dg, serial=s1)
    assert int(dg["counters"][2]) > 0                       # it walked the hierarchy
    for k in ("means3D", "opacities", "scales", "rotations", "shs"):
        assert hp.rel_l2(g[k].cpu().numpy(), ref[k].cpu().numpy()) < 1e-5, k
    # a rebuild invalidates the log as well
    f3 = hp.cuda_forward(C, st, wc)
    s3 = st.last_forward_serial
    C.build_acceleration_structure(st, wc["v"], wc["f"], 1)
    dg = {}
    hp.cuda_backward(C, st, wc, f3, up, diag=dg, serial=s3)
    assert int(dg["counters"][2]) > 0


def test_full_chunk_log_falls_back_to_retrace(C, oracle_mod):
    """A log too small for the call: rays that did not fit are re-traced, gradients unchanged."""
    w = hp.reduced_workload(3)
    wc = hp.to_cuda(w)
    H, W = w["ray_o"].shape[:2]
    up = {"rgb": torch.ones((H, W, 3), device="cuda"), "dpt": torch.ones((H, W, 1), device="cuda")}
    ref_state = _build(C, wc)
    f = hp.cuda_forward(C, ref_state, wc)
    ref = hp.cuda_backward(C, ref_state, wc, f, up, serial=0)
    for wave in (False, True):
        st = _build(C, wc, wave)
        st.set_chunk_log_max_records(2000)          # the call needs about 50,000 records
        f2 = hp.cuda_forward(C, st, wc)
        dg = {}
        g = hp.cuda_backward(C, st, wc, f2, up, diag=dg, serial=st.last_forward_serial)
        torch.cuda.synchronize()
        assert st.status() == 0
        c = dg["counters"].cpu().numpy()
        assert c[2] > 0 and c[5] == int(f2["wet"].numel() * 0 + c[5])      # some rays walked the hierarchy
        for k in hp.GRAD_KEYS:
            a, b = g[k].cpu().numpy(), ref[k].cpu().numpy()
            m = np.isfinite(b)
            assert hp.rel_l2(a[m], b[m]) < 1e-4, (wave, k)


@pytest.mark.parametrize("config", [3, 5])
def test_list_order_does_not_change_results(C, config):
    """Scheduling option of the wavefront rounds (live lists kept in tile order, or appended warp by warp): same bits."""
    wc = hp.to_cuda(hp.reduced_workload(config))
    outs = []
    for mode in (0, 1):
        st = _build(C, wc, wave=True)
        st.set_stable_lists(mode)
        f = hp.cuda_forward(C, st, wc)
        g = hp.cuda_backward(C, st, wc, f, dict(rgb=torch.ones_like(f["rgb"])), serial=0)       # re-tracing backward: its rounds use the lists too
        torch.cuda.synchronize()
        assert st.status() == 0
        outs.append((f, g))
    for k in ("rgb", "dpt", "acc", "norm", "aux", "mid"):
        assert torch.equal(outs[0][0][k], outs[1][0][k]), k
    for k in ("ray_o", "ray_d"):
        assert torch.equal(outs[0][1][k], outs[1][1][k]), k
    for k in ("means3D", "shs", "opacities", "scales", "rotations"):
        assert hp.rel_l2(outs[0][1][k].cpu().numpy(), outs[1][1][k].cpu().numpy()) < 1e-4, k


def test_forward_slices_do_not_change_results(C):
    """A large forward call runs as up to four slices of the ray grid on streams of their own (scheduling only): the
    outputs equal those of the unsliced call bit for bit, call after call, and the backward over the chunk log the
    slices wrote together gives the same gradients."""
    import workloads
    wc = hp.to_cuda(workloads.make_workload(3, P=150000, H=1080, W=1024))
    up = dict(rgb=torch.ones((1080, 1024, 3), device="cuda"))
    ref_f = ref_g = None
    for slices in (1, 4, 2, 4):
        st = _build(C, wc)
        st.set_forward_slices(slices)
        for rep in range(3):
            f = hp.cuda_forward(C, st, wc)
            g = hp.cuda_backward(C, st, wc, f, up, serial=st.last_forward_serial)
            torch.cuda.synchronize()
            assert st.status() == 0
            if ref_f is None:
                ref_f, ref_g = f, g
                continue
            for k in ("rgb", "dpt", "acc", "norm", "aux", "mid"):
                assert torch.equal(f[k], ref_f[k]), (slices, rep, k)
            for k in ("ray_o", "ray_d"):
                assert torch.equal(g[k], ref_g[k]), (slices, rep, k)
            for k in ("means3D", "shs", "opacities", "scales", "rotations"):
                assert hp.rel_l2(g[k].cpu().numpy(), ref_g[k].cpu().numpy()) < 1e-4, (slices, rep, k)


def test_image_width_hint_does_not_change_results(C):
    """(B, h*w, 3) ray batches walked in pixel tiles (image width known) or in the order given: same bits."""
    wc = hp.to_cuda(hp.reduced_workload(5))               # 2 cameras of 54 x 96 pixels as a (2, 5184, 3) batch
    outs = []
    for width in (0, 96):
        st = _build(C, wc, wave=True)
        st.set_image_width(width)
        f = hp.cuda_forward(C, st, wc)
        g = hp.cuda_backward(C, st, wc, f, dict(rgb=torch.ones_like(f["rgb"])), serial=st.last_forward_serial)
        torch.cuda.synchronize()
        assert st.status() == 0
        outs.append((f, g))
    for k in ("rgb", "dpt", "acc", "norm", "aux", "mid"):
        assert torch.equal(outs[0][0][k], outs[1][0][k]), k
    for k in ("ray_o", "ray_d"):
        assert torch.equal(outs[0][1][k], outs[1][1][k]), k
    for k in ("means3D", "shs", "opacities", "scales", "rotations"):
        assert hp.rel_l2(outs[0][1][k].cpu().numpy(), outs[1][1][k].cpu().numpy()) < 1e-4, k


def test_adaptive_round_count_keeps_results(C):
    """Later calls of one shape enqueue fewer wavefront rounds (history of the earlier ones); rays that then need more
    rounds are finished by the tail kernel. Results do not depend on it."""
    w = hp.reduced_workload(3)
    wc = hp.to_cuda(w)
    st = _build(C, wc, wave=True)
    n0 = st.kernel_launches()
    first = hp.cuda_forward(C, st, wc)
    torch.cuda.synchronize()
    n1 = st.kernel_launches()
    hp.cuda_forward(C, st, wc)              # reads the history of the first call, leaves its own
    torch.cuda.synchronize()
    n2 = st.kernel_launches()
    again = hp.cuda_forward(C, st, wc)
    torch.cuda.synchronize()
    n3 = st.kernel_launches()
    assert n3 - n2 < n1 - n0                # fewer rounds enqueued than the 48 of a call without history
    for k in ("rgb", "dpt", "acc", "norm", "aux", "mid"):
        assert torch.equal(first[k], again[k]), k
    # same shape, harder rays (camera inside the scene, more chunks and bounces per ray): the short round list is
    # not enough, the tail kernel finishes the rest, and the result is that of a state without history
    o2, d2 = hp.workloads.pinhole_rays(wc["ray_o"].shape[0], wc["ray_o"].shape[1], 90.0, (0.9, 0.1, 0.05))
    wc2 = dict(wc, ray_o=o2.cuda(), ray_d=d2.cuda())
    got = hp.cuda_forward(C, st, wc2)
    ref = hp.cuda_forward(C, _build(C, wc, wave=True), wc2)
    torch.cuda.synchronize()
    for k in ("rgb", "dpt", "acc", "norm", "aux", "mid"):
        assert torch.equal(got[k], ref[k]), k
    assert st.status() == 0


def test_refit_matches_rebuild(C, oracle_mod):
    """rebuild=0 keeps the topology and refits boxes and frames: results equal a fresh build on the moved vertices."""
    w = hp.reduced_workload(2)
    wc = hp.to_cuda(w)
    st = _build(C, wc)
    gen = torch.Generator().manual_seed(7)
    means2 = w["means3D"] + 0.01 * torch.randn(w["means3D"].shape, generator=gen)
    v2, f2 = hp.workloads.get_triangles(means2, w["scales"], w["rotations"])
    w2 = dict(w, means3D=means2, v=v2, f=f2)
    wc2 = hp.to_cuda(w2)
    C.build_acceleration_structure(st, wc2["v"], wc2["f"], 0)
    got_refit = hp.cuda_forward(C, st, wc2)
    st2 = _build(C, wc2)
    got_build = hp.cuda_forward(C, st2, wc2)
    torch.cuda.synchronize()
    assert st.status() == 0 and st2.status() == 0
    for k in ("rgb", "dpt", "acc", "norm", "mid"):
        assert torch.equal(got_refit[k], got_build[k]), k
    want = oracle_mod.Oracle(oracle_mod.Scene(v2), impl="restatement").forward(w2)
    assert np.array_equal(got_refit["rgb"].cpu().numpy().view(np.uint32), want["rgb"].view(np.uint32))


def test_errors_and_edge_cases(C):
    w = hp.workloads.make_workload(1, P=64, H=4, W=8)
    wc = hp.to_cuda(w)
    st = C.OptiXStateWrapper("")
    with pytest.raises(RuntimeError, match="before"):
        hp.cuda_forward(C, st, wc)                                   # trace before build
    with pytest.raises(RuntimeError, match="before"):
        C.build_acceleration_structure(st, wc["v"], wc["f"], 0)      # refit before build
    with pytest.raises(RuntimeError, match="dimensions"):
        C.build_acceleration_structure(st, wc["v"].reshape(-1), wc["f"], 1)
    with pytest.raises(RuntimeError, match="4 vertices"):
        C.build_acceleration_structure(st, wc["v"][:6], None, 1)
    C.build_acceleration_structure(st, wc["v"], wc["f"], 1)
    with pytest.raises(RuntimeError, match="surfel count"):
        C.build_acceleration_structure(st, wc["v"][:8], None, 0)     # refit with another surfel count
    bad = dict(wc, means3D=wc["means3D"][:10])
    with pytest.raises(RuntimeError, match="surfels"):
        hp.cuda_forward(C, st, bad)
    out = hp.cuda_forward(C, st, wc)
    assert out["mid"].shape == (4, 8, 32) and out["wet"].shape == (64, 1)
    # a single surfel, rays that all miss, zero-length directions
    one = hp.workloads.make_workload(1, P=1, H=2, W=2)
    oc = hp.to_cuda(one)
    st1 = _build(C, oc)
    oc["ray_d"] = torch.zeros_like(oc["ray_d"])
    o1 = hp.cuda_forward(C, st1, oc)
    torch.cuda.synchronize()
    assert float(o1["acc"].abs().max()) == 0.0 and st1.status() == 0


def test_module_api_and_autograd(C):
    """The nn.Module front end: same call as the reference's example, gradients reach the leaves."""
    from diff_surfel_tracing import SurfelTracer, SurfelTracingSettings
    w = hp.reduced_workload(1)
    wc = hp.to_cuda(w)
    tracer = SurfelTracer()
    tracer.build_acceleration_structure(wc["v"], wc["f"], rebuild=True)
    leaves = {k: wc[k].clone().requires_grad_(True) for k in ("means3D", "shs", "opacities", "scales", "rotations")}
    grads3D = torch.zeros_like(wc["means3D"], requires_grad=True) + 0
    grads3D.retain_grad()
    e = torch.zeros(1, device="cuda")
    settings = SurfelTracingSettings(image_height=128, image_width=128, tanfovx=1.0, tanfovy=1.0, bg=wc["bg"], scale_modifier=1.0,
                                     viewmatrix=e, projmatrix=e, sh_degree=0, campos=e, prefiltered=False, debug=False)
    with pytest.raises(Exception, match="excatly one"):
        tracer(wc["ray_o"], wc["ray_d"], wc["v"], leaves["means3D"], grads3D, opacities=leaves["opacities"],
               scales=leaves["scales"], rotations=leaves["rotations"], tracer_settings=settings)
    rgb, dpt, acc, norm, dist, aux, mid, wet = tracer(wc["ray_o"], wc["ray_d"], wc["v"], leaves["means3D"], grads3D,
                                                       shs=leaves["shs"], opacities=leaves["opacities"], scales=leaves["scales"],
                                                       rotations=leaves["rotations"], tracer_settings=settings)
    assert rgb.shape == (128, 128, 3) and dist.shape == (128, 128, 1) and mid.shape == (128, 128, 32) and wet.shape == (10000, 1)
    (rgb.sum() + dpt.sum()).backward()
    for k, t in leaves.items():
        assert t.grad is not None and torch.isfinite(t.grad).all() and float(t.grad.abs().sum()) > 0, k
    assert grads3D.grad is not None and float(grads3D.grad.abs().sum()) > 0
    tracer.eval()
    out = tracer(wc["ray_o"], wc["ray_d"], wc["v"], wc["means3D"], grads3D, shs=wc["shs"], opacities=wc["opacities"],
                 scales=wc["scales"], rotations=wc["rotations"], tracer_settings=settings)
    assert out[7].shape == (10000,) and float(out[7].abs().max()) == 0.0
    assert torch.equal(out[0], rgb.detach())


def test_ray_scratch_grows_once_per_larger_call(C):
    """The handle's per-ray scratch is grow-only: a call larger than any before replaces it once (keeping the larger
    of the old and new record size), repeated and smaller calls allocate nothing."""
    w = hp.workloads.make_workload(1, P=3000, H=96, W=96)
    wc = hp.to_cuda(w)
    st = _build(C, wc)
    st.set_chunk_log(False)               # the chunk log sizes itself from the previous call; this test watches the ray scratch

    def sub(n):
        return dict(wc, ray_o=wc["ray_o"][:n, :n].contiguous(), ray_d=wc["ray_d"][:n, :n].contiguous())

    def pair(n):
        s = sub(n)
        f = hp.cuda_forward(C, st, s)
        b_f = st.info()["device_bytes"]
        hp.cuda_backward(C, st, s, f, dict(rgb=torch.ones((n, n, 3), device="cuda")))
        return b_f, st.info()["device_bytes"]

    pair(32)                              # first use: the forward sizes the records, the backward enlarges them
    base = st.info()["device_bytes"]
    assert pair(32) == (base, base) and pair(16) == (base, base)
    f64, b64 = pair(64)
    assert f64 > base and b64 == f64      # one growth, at the forward; the backward finds its record size already there
    assert pair(64) == (f64, f64) and pair(32) == (f64, f64)
    f96, b96 = pair(96)
    assert f96 > f64 and b96 == f96
    torch.cuda.synchronize()
    assert st.status() == 0
