"""GPU parity tests of the options the five benchmark configurations leave at their defaults, and a direct
comparison with the reference's own shader sources.

* the CUDA path against optix_tracer/forward.cu and backward.cu compiled for the host (oracle/_ref, built
  where the reference tree was present): one link instead of CUDA -> restatement -> reference;
* a non-zero background (the reference's demo renders on white, example/render.py:84; the backward counts the
  background twice, optix_tracer/backward.cu:545-548);
* start_from_first=False (near plane 0 instead of 0.2 on the primary segment, optix_tracer/forward.cu:353);
* SH degrees 1 and 2, and a degree below what the coefficient tensor holds (optix_tracer/forward.cu:30-56);
* training=False (no per-surfel weights; same per-ray outputs).

Bars as in test_gpu_parity.py: contributing hit sequences equal, forward outputs identical bit for bit (the
forward is specified operation by operation), every gradient within 1e-3 relative L2.
"""
import numpy as np
import pytest
import torch

import helpers as hp

pytestmark = pytest.mark.gpu

GRAD_RTOL = 1e-3


@pytest.fixture(scope="module")
def C():
    from diff_surfel_tracing import _C
    assert torch.cuda.is_available()
    _C.lib()
    return _C


def _state(C, wc, wave):
    st = C.OptiXStateWrapper("")
    if wave:
        st.set_wavefront_min_rays(0)
    C.build_acceleration_structure(st, wc["v"], wc["f"], 1)
    return st


def _compare(C, orc, w, wave, hit_ids_are_surfels=False, training=True):
    """Forward + backward of workload `w` on the CUDA path and on oracle `orc`; asserts the bars."""
    wc = hp.to_cuda(w)
    st = _state(C, wc, wave)
    diag = dict(hit_cap=320)
    got = hp.cuda_forward(C, st, wc, training=training, diag=diag)
    torch.cuda.synchronize()
    assert st.status() == 0
    want = orc.forward(w, training=training)
    cnt = diag["hit_cnt"].cpu().numpy()
    assert np.array_equal(cnt, want["hit_cnt"]) and cnt.max() > 0
    log = diag["hit_log"].cpu().numpy()
    if hit_ids_are_surfels:        # the reference logs surfel ids (primitive id / 2), the CUDA path primitive ids
        log = np.where(log >= 0, log >> 1, -1)
    assert np.array_equal(log, want["hit_log"])
    for k in ("rgb", "dpt", "acc", "norm", "aux"):
        g = got[k].cpu().numpy().reshape(want[k].shape)
        assert np.array_equal(g.view(np.uint32), want[k].view(np.uint32)), f"{k} not bit-identical"
    # per-bounce records: wherever the bounce was traced (the reference leaves the others uninitialised, the CUDA path zeroes them)
    gm = got["mid"].cpu().numpy().reshape(-1, got["mid"].shape[-1] // 16, 16)
    wm = want["mid"].reshape(gm.shape)
    traced = np.abs(gm[..., 3:6]).sum(-1) > 0
    assert np.array_equal(gm[traced].view(np.uint32), wm[traced].view(np.uint32))
    assert float(np.abs(gm[~traced]).max(initial=0.0)) == 0.0
    if training:
        wet = got["wet"].cpu().numpy()
        assert np.abs(wet - want["wet"]).max() <= 1e-4 * max(1.0, float(np.abs(want["wet"]).max()))
    else:
        assert got["wet"] is None
    H, W = w["ray_o"].shape[:2]
    gen = torch.Generator().manual_seed(11)
    up = {k: torch.randn((H, W, c), generator=gen) for k, c in (("rgb", 3), ("dpt", 1), ("acc", 1), ("norm", 3), ("aux", 2))}
    gb = hp.cuda_backward(C, st, wc, got, {k: v.cuda() for k, v in up.items()}, serial=st.last_forward_serial)
    torch.cuda.synchronize()
    assert st.status() == 0
    # both backward implementations start from the same saved forward state: the CUDA path's outputs (identical to the
    # oracle's on every traced bounce, asserted above, and zero where the reference leaves its per-bounce record
    # uninitialised, optix_tracer/forward.cu:446, which its backward nevertheless reads, backward.cu:690-703)
    saved = {k: got[k].cpu().numpy().reshape(want[k].shape) for k in ("rgb", "dpt", "acc", "norm", "dist", "aux", "mid")}
    ob = orc.backward(w, saved, {k: v.numpy() for k, v in up.items()})
    for k in hp.GRAD_KEYS:
        g, o = gb[k].cpu().numpy().reshape(ob[k].shape), ob[k]
        if not np.isfinite(o).all():
            # the reference divides by the accumulated specular weight (backward.cu:771); where that is 0 both sides are non-finite
            assert np.array_equal(np.isfinite(g), np.isfinite(o)), k
            m = np.isfinite(o)
            g, o = g[m], o[m]
        e = hp.rel_l2(g, o)
        assert e <= GRAD_RTOL, f"grad {k}: rel L2 {e}"
    return got, want


@pytest.mark.parametrize("config", [1, 3, 5])
def test_cuda_path_against_the_host_compiled_reference(C, oracle_mod, config):
    """The reference's forward.cu / backward.cu compiled for the host, run on the same inputs with the same
    enumerator and the fixed-sequence exp: identical forward bits, gradients within 1e-3."""
    if not oracle_mod.reference_built():
        pytest.skip("oracle/_ref is not built (the reference tree was absent at build time)")
    w = hp.reduced_workload(config)
    orc = oracle_mod.Oracle(oracle_mod.Scene(w["v"]), impl="reference", hit_cap=320, portable_exp=True)
    _compare(C, orc, w, wave=(config != 1), hit_ids_are_surfels=True)


@pytest.mark.parametrize("wave", [False, True], ids=["per-ray", "wavefront"])
@pytest.mark.parametrize("config", [1, 3])
def test_white_background(C, oracle_mod, config, wave):
    w = dict(hp.reduced_workload(config), bg=torch.tensor([1.0, 1.0, 1.0]))
    orc = oracle_mod.Oracle(oracle_mod.Scene(w["v"]), impl="restatement", hit_cap=320, portable_exp=True)
    got, want = _compare(C, orc, w, wave)
    # rays that hit nothing show the background
    miss = want["acc"].reshape(-1) == 0
    assert miss.any() or config != 1
    assert np.all(got["rgb"].cpu().numpy().reshape(-1, 3)[miss] == 1.0)


@pytest.mark.parametrize("config", [1, 4])
def test_start_from_first_false(C, oracle_mod, config):
    w = dict(hp.reduced_workload(config), start_from_first=False)
    if config == 1:
        # a camera inside the cloud: surfels nearer than 0.2 exist, which start_from_first=True would skip
        o, d = hp.workloads.pinhole_rays(64, 64, 70.0, (0.3, 0.1, 0.05), target=(-1.0, 0.2, 0.0))
        w = dict(w, ray_o=o, ray_d=d)
    orc = oracle_mod.Oracle(oracle_mod.Scene(w["v"]), impl="restatement", hit_cap=320, portable_exp=True)
    got, _ = _compare(C, orc, w, wave=False)
    if config == 1:
        other = hp.cuda_forward(C, _state(C, hp.to_cuda(w), False), hp.to_cuda(dict(w, start_from_first=True)))
        assert not torch.equal(other["rgb"], got["rgb"])          # the option changes what these rays see


@pytest.mark.parametrize("degree,coeffs", [(1, 4), (2, 9), (1, 16), (0, 16)])
def test_sh_degrees(C, oracle_mod, degree, coeffs):
    """Degree 1 and 2 rows (4 and 9 coefficients: 12- and 27-float rows, the latter not 16-byte aligned), and a
    degree below what the tensor holds."""
    w = hp.reduced_workload(2)
    w = dict(w, shs=w["shs"][:, :coeffs].contiguous(), sh_degree=degree)
    orc = oracle_mod.Oracle(oracle_mod.Scene(w["v"]), impl="restatement", hit_cap=320, portable_exp=True)
    _compare(C, orc, w, wave=(degree == 2))


def test_inference_mode(C, oracle_mod):
    """training=False: no per-surfel weights, the same per-ray outputs; the module returns zeros of shape (P,)."""
    w = hp.reduced_workload(3)
    orc = oracle_mod.Oracle(oracle_mod.Scene(w["v"]), impl="restatement", hit_cap=320, portable_exp=True)
    got, want = _compare(C, orc, w, wave=True, training=False)
    assert float(np.abs(want["wet"]).max()) == 0.0


@pytest.mark.parametrize("config,wave", [(1, False), (3, True), (4, False)])
def test_distortion_extension(C, oracle_mod, config, wave):
    """The depth-distortion output (an extension: zeros in the reference) against the CPU restatement of the same
    formula: forward within 1e-5, gradients of an upstream on dist (alone, and mixed with the others) within 1e-3
    relative L2; every other output keeps its bits; off by default."""
    w = hp.reduced_workload(config)
    wc = hp.to_cuda(w)
    st = _state(C, wc, wave)
    off = hp.cuda_forward(C, st, wc)
    assert float(off["dist"].abs().max()) == 0.0
    st.set_distortion(True)
    got = hp.cuda_forward(C, st, wc)
    orc = oracle_mod.Oracle(oracle_mod.Scene(w["v"]), impl="restatement", portable_exp=True, distortion=True)
    want = orc.forward(w)
    for k in ("rgb", "dpt", "acc", "norm", "aux", "mid"):
        assert torch.equal(got[k], off[k]), k
    gd = got["dist"].cpu().numpy().reshape(want["dist"].shape)
    assert float(np.abs(want["dist"][..., 0]).max()) > 0
    assert np.abs(gd - want["dist"]).max() <= 1e-4 * float(np.abs(want["dist"]).max())          # free-form arithmetic on both sides
    H, W = w["ray_o"].shape[:2]
    gen = torch.Generator().manual_seed(3)
    ups = [dict(dist=torch.ones((H, W, 1))),
           {k: torch.randn((H, W, c), generator=gen) for k, c in (("rgb", 3), ("dpt", 1), ("acc", 1), ("norm", 3), ("aux", 2), ("dist", 1))}]
    for serial in (st.last_forward_serial, 0):
        for up in ups:
            gb = hp.cuda_backward(C, st, wc, got, {k: v.cuda() for k, v in up.items()}, serial=serial)
            torch.cuda.synchronize()
            assert st.status() == 0
            saved = {k: got[k].cpu().numpy().reshape(want[k].shape) for k in ("rgb", "dpt", "acc", "norm", "dist", "aux", "mid")}
            ob = orc.backward(w, saved, {k: v.numpy() for k, v in up.items()})
            for k in hp.GRAD_KEYS:
                g, o = gb[k].cpu().numpy().reshape(ob[k].shape), ob[k]
                m = np.isfinite(o)
                assert np.array_equal(np.isfinite(g), m), k
                if k in ("means3D", "opacities", "scales", "rotations"):
                    assert float(np.abs(o[m]).max()) > 0, k
                assert hp.rel_l2(g[m], o[m]) <= GRAD_RTOL, f"config {config} grad {k}: {hp.rel_l2(g[m], o[m])}"


def test_distortion_through_the_module(C):
    from diff_surfel_tracing import SurfelTracer, SurfelTracingSettings
    w = hp.reduced_workload(1)
    wc = hp.to_cuda(w)
    tracer = SurfelTracer()
    tracer.enable_distortion(True)
    tracer.build_acceleration_structure(wc["v"], wc["f"], rebuild=True)
    leaves = {k: wc[k].clone().requires_grad_(True) for k in ("means3D", "shs", "opacities", "scales", "rotations")}
    g3d = torch.zeros_like(wc["means3D"], requires_grad=True)
    e = torch.zeros(1, device="cuda")
    settings = SurfelTracingSettings(128, 128, 1.0, 1.0, wc["bg"], 1.0, e, e, 0, e, False, False)
    out = tracer(wc["ray_o"], wc["ray_d"], wc["v"], leaves["means3D"], g3d, shs=leaves["shs"], opacities=leaves["opacities"],
                 scales=leaves["scales"], rotations=leaves["rotations"], tracer_settings=settings)
    dist = out[4]
    assert dist.shape == (128, 128, 1) and float(dist.max()) > 0 and float(dist.min()) >= -1e-7
    dist.sum().backward()
    for k in ("means3D", "opacities", "scales", "rotations"):
        assert leaves[k].grad is not None and torch.isfinite(leaves[k].grad).all() and float(leaves[k].grad.abs().sum()) > 0, k
    assert float(leaves["shs"].grad.abs().sum()) == 0.0          # the distortion does not depend on colour
