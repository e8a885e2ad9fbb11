"""GPU parity tests of the two steps next to the tracer: quad expansion (+ fused refit) and ray generation.

Bars: the CUDA kernels follow the CPU oracle's operation order, so they are compared bit for bit with
it; against the golden vectors produced by the reference's own Python functions the quad vertices are
bit-identical and normalised ray directions agree to 2e-7 relative (the reference's `norm` reduction
order is not specified).
"""
import math

import numpy as np
import pytest
import torch

import helpers as hp
import make_golden_prep as mg

pytestmark = pytest.mark.gpu

RAY_RTOL = 2e-7


@pytest.fixture(scope="module")
def C():
    from diff_surfel_tracing import _C
    assert torch.cuda.is_available()
    _C.lib()
    return _C


@pytest.fixture(scope="module")
def golden():
    import os
    return np.load(os.path.join(os.path.dirname(mg.__file__), "prep.npz"))


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def _look_at(eye, H, W, fov_deg):
    eye = np.asarray(eye, dtype=np.float64)
    fwd = -eye / np.linalg.norm(eye)
    right = np.cross(fwd, [0.0, 0.0, 1.0]); right /= np.linalg.norm(right)
    down = np.cross(fwd, right)
    R = np.stack([right, down, fwd], 0)
    T = -R @ eye
    fl = 0.5 * W / math.tan(math.radians(0.5 * fov_deg))
    K = np.array([[fl, 0, 0.5 * W], [0, fl, 0.5 * H], [0, 0, 1.0]])
    return K.astype(np.float32), R.astype(np.float32), T.astype(np.float32)


def test_surfel_quads_match_reference_golden_and_oracle(C, oracle_mod, golden):
    means, _, _, _ = mg.prep_inputs()
    st = C.OptiXStateWrapper("")
    m, s, r = (torch.from_numpy(np.ascontiguousarray(x)).cuda() for x in (means, golden["scales"], golden["rotations"]))
    v, f = C.surfel_quads(st, m, s, r)
    assert v.shape == (4 * mg.P_GOLDEN, 3) and f.shape == (2 * mg.P_GOLDEN, 3) and f.dtype == torch.int32
    assert np.array_equal(_bits(v.cpu().numpy()), _bits(golden["v"]))          # the reference's own output
    assert np.array_equal(f.cpu().numpy(), golden["f"])
    # a larger seeded case with un-normalised quaternions against the oracle, bit for bit
    g = torch.Generator().manual_seed(11)
    P = 200_003
    m = torch.randn((P, 3), generator=g) * 5
    s = torch.exp(torch.randn((P, 2), generator=g) - 4)
    r = torch.randn((P, 4), generator=g) * 3
    v, f = C.surfel_quads(st, m.cuda(), s.cuda(), r.cuda(), with_triangles=False)
    want, _ = oracle_mod.surfel_quads(m, s, r, with_triangles=False)
    assert f is None
    assert np.array_equal(_bits(v.cpu().numpy()), _bits(want))


@pytest.mark.parametrize("single_kernel", [False, True], ids=["expand-then-refit", "single-kernel-refit"])
def test_build_from_surfels_equals_expand_then_build(C, oracle_mod, single_kernel):
    """One call from the parameters == get_triangles + build_acceleration_structure, for build and for refit."""
    w = hp.reduced_workload(3)
    wc = hp.to_cuda(w)
    v_ref, _ = oracle_mod.surfel_quads(w["means3D"], w["scales"], w["rotations"], with_triangles=False)
    st = C.OptiXStateWrapper("")
    st.set_single_kernel_refit(single_kernel)
    v = C.build_from_surfels(st, wc["means3D"], wc["scales"], wc["rotations"], 1)
    assert np.array_equal(_bits(v.cpu().numpy()), _bits(v_ref))
    st_b = C.OptiXStateWrapper("")
    C.build_acceleration_structure(st_b, torch.from_numpy(v_ref).cuda(), None, 1)
    assert torch.equal(C.debug_quad_frames(st), C.debug_quad_frames(st_b))
    out_a = hp.cuda_forward(C, st, dict(wc, v=v))
    out_b = hp.cuda_forward(C, st_b, dict(wc, v=v))
    for k in ("rgb", "dpt", "acc", "norm", "aux", "mid"):
        assert torch.equal(out_a[k], out_b[k]), k
    assert torch.allclose(out_a["wet"], out_b["wet"], rtol=1e-4, atol=1e-6)      # float atomics: the order differs run to run
    # refit: the surfels move; the new vertices are written into the same tensor
    gen = torch.Generator().manual_seed(5)
    means2 = w["means3D"] + 0.01 * torch.randn(w["means3D"].shape, generator=gen)
    rot2 = w["rotations"] + 0.02 * torch.randn(w["rotations"].shape, generator=gen)
    v2_ref, _ = oracle_mod.surfel_quads(means2, w["scales"], rot2, with_triangles=False)
    v_again = C.build_from_surfels(st, means2.cuda(), wc["scales"], rot2.cuda(), 0, vertices=v)
    assert v_again.data_ptr() == v.data_ptr()
    assert np.array_equal(_bits(v.cpu().numpy()), _bits(v2_ref))
    C.build_acceleration_structure(st_b, torch.from_numpy(v2_ref).cuda(), None, 0)
    assert torch.equal(C.debug_quad_frames(st), C.debug_quad_frames(st_b))
    wc2 = dict(wc, means3D=means2.cuda(), rotations=rot2.cuda(), v=v)
    out_a = hp.cuda_forward(C, st, wc2)
    out_b = hp.cuda_forward(C, st_b, wc2)
    torch.cuda.synchronize()
    for k in ("rgb", "dpt", "acc", "norm", "aux", "mid"):
        assert torch.equal(out_a[k], out_b[k]), k
    assert st.status() == 0 and st_b.status() == 0
    # and the result is the oracle's on those vertices
    want = oracle_mod.Oracle(oracle_mod.Scene(v2_ref), impl="restatement").forward(dict(w, means3D=means2, rotations=rot2, v=torch.from_numpy(v2_ref)))
    assert np.array_equal(_bits(out_a["rgb"].cpu().numpy()), _bits(want["rgb"]))


def test_build_from_surfels_errors_and_single_surfel(C, oracle_mod):
    st = C.OptiXStateWrapper("")
    m = torch.zeros((1, 3), device="cuda"); s = torch.full((1, 2), 0.5, device="cuda"); r = torch.tensor([[2.0, 0, 0, 0]], device="cuda")
    with pytest.raises(RuntimeError, match="before"):
        C.build_from_surfels(st, m, s, r, 0)                      # refit before any build
    v = C.build_from_surfels(st, m, s, r, 1)
    want = np.array([[-1.5, 1.5, 0], [-1.5, -1.5, 0], [1.5, 1.5, 0], [1.5, -1.5, 0]], dtype=np.float32)
    assert np.array_equal(v.cpu().numpy(), want)
    with pytest.raises(RuntimeError, match="dimensions"):
        C.build_from_surfels(st, m, s[:, :1], r, 1)
    with pytest.raises(RuntimeError, match="surfel count"):
        C.build_from_surfels(st, m.repeat(2, 1), s.repeat(2, 1), r.repeat(2, 1), 0)
    with pytest.raises(RuntimeError, match="shape"):
        C.build_from_surfels(st, m, s, r, 1, vertices=torch.empty((3, 3), device="cuda"))


def test_pinhole_rays_match_reference_golden_and_oracle(C, oracle_mod, golden):
    _, _, _, cams = mg.prep_inputs()
    st = C.OptiXStateWrapper("")
    H, W = mg.H_GOLDEN, mg.W_GOLDEN
    for c, (K, R, T) in enumerate(cams):
        for z in (0, 1):
            o, d = C.pinhole_rays(st, H, W, K, R, T, True, bool(z))
            o, d = o.cpu().numpy(), d.cpu().numpy()
            wo, wd = oracle_mod.pinhole_rays(H, W, K, R, T, True, bool(z))
            assert np.array_equal(_bits(o), _bits(wo)) and np.array_equal(_bits(d), _bits(wd))
            go, gd = golden[f"ray_o_{c}_{z}"], golden[f"ray_d_{c}_{z}"]
            assert np.array_equal(_bits(o), _bits(go))
            assert np.abs(d - gd).max() <= RAY_RTOL * np.abs(gd).max()
    # a batch of cameras in one call, full-HD, and without the half-pixel shift
    Ks, Rs, Ts = (np.stack([c[i] for c in cams]) for i in range(3))
    o, d = C.pinhole_rays(st, 1080, 1920, Ks, Rs, Ts, False, False)
    assert o.shape == (3, 1080, 1920, 3)
    for b in (0, 2):
        wo, wd = oracle_mod.pinhole_rays(1080, 1920, Ks[b], Rs[b], Ts[b], False, False)
        assert np.array_equal(_bits(d[b].cpu().numpy()), _bits(wd)) and np.array_equal(_bits(o[b].cpu().numpy()), _bits(wo))
    with pytest.raises(RuntimeError, match="at most"):
        C.pinhole_rays(st, 2, 2, np.tile(Ks[:1], (65, 1, 1)), np.tile(Rs[:1], (65, 1, 1)), np.tile(Ts[:1], (65, 1, 1)))


def test_forward_camera_equals_forward_on_generated_rays(C):
    """The trace call that generates its rays gives the outputs and gradients of get_rays followed by the plain call."""
    from diff_surfel_tracing import SurfelTracer, SurfelTracingSettings
    w = hp.reduced_workload(3)
    wc = hp.to_cuda(w)
    H, W = 72, 128
    K, R, T = _look_at([4.0, 0.5, 0.3], H, W, 50.0)
    tracer = SurfelTracer()
    v = tracer.build_from_surfels(wc["means3D"], wc["scales"], wc["rotations"], rebuild=True)
    ray_o, ray_d = tracer.get_rays(H, W, K, R, T)
    e = torch.zeros(1, device="cuda")
    settings = SurfelTracingSettings(image_height=H, image_width=W, tanfovx=1.0, tanfovy=1.0, bg=wc["bg"], scale_modifier=1.0,
                                     viewmatrix=e, projmatrix=e, sh_degree=3, campos=e, prefiltered=False, debug=False,
                                     max_trace_depth=1, specular_threshold=0.5)

    def run(camera):
        leaves = {k: wc[k].clone().requires_grad_(True) for k in ("means3D", "shs", "opacities", "scales", "rotations", "others_precomp")}
        g3 = torch.zeros_like(wc["means3D"], requires_grad=True) + 0
        kw = dict(shs=leaves["shs"], others_precomp=leaves["others_precomp"], opacities=leaves["opacities"], scales=leaves["scales"],
                  rotations=leaves["rotations"], tracer_settings=settings)
        if camera:
            out = tracer.forward_camera(H, W, K, R, T, v, leaves["means3D"], g3, **kw)
        else:
            out = tracer(ray_o, ray_d, v, leaves["means3D"], g3, **kw)
        out[0].sum().backward()
        return out, leaves

    out_a, la = run(True)
    out_b, lb = run(False)
    assert torch.equal(tracer.last_rays[0], ray_o) and torch.equal(tracer.last_rays[1], ray_d)
    for a, b in zip(out_a[:7], out_b[:7]):
        assert torch.equal(a, b)
    assert torch.allclose(out_a[7], out_b[7], rtol=1e-4, atol=1e-6)
    assert float(out_a[2].detach().sum()) > 0
    for k in la:
        assert hp.rel_l2(la[k].grad.cpu().numpy(), lb[k].grad.cpu().numpy()) < 1e-3, k      # fp32 atomics: order differs run to run
    assert tracer.optix_context.status() == 0


def test_example_render_script(tmp_path):
    """The counterpart of the reference's example/render.py runs end to end on a synthetic scene and writes its images."""
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "diff-surfel-tracing_b200", "example", "render.py")
    spec = importlib.util.spec_from_file_location("example_render", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = str(tmp_path / "render")
    status = mod.main(["--result_dir", out, "--surfels", "30000", "--height", "54", "--width", "96", "--frames", "2",
                       "--max_trace_depth", "1", "--specular_threshold", "0.5"])
    assert status == 0
    for sub in ("RENDER", "DEPTH", "NORMAL"):
        files = sorted(os.listdir(os.path.join(out, sub)))
        assert len(files) == 2 and all(os.path.getsize(os.path.join(out, sub, f)) > 100 for f in files), sub
    from PIL import Image
    img = np.asarray(Image.open(os.path.join(out, "RENDER", "0000.png")))
    assert img.shape == (54, 96, 3) and img.max() > 0
