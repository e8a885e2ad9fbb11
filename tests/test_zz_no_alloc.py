"""The allocation-free forward entry point (dst_forward_static) against the regular one (dst_forward).

Collected last on purpose (file name): a run that stops at the first failure has then already
run every other test. Some callers of the library cannot allocate device memory at the point of
the call (a host application whose memory pool owns the device, a plug-in that only gets lent
buffers, a loop that cannot take an allocation's synchronisation); for them the library offers a forward trace whose scratch is a fixed array inside the
library image. This test calls it through the C ABI twice in a row and requires the results of
the regular entry point: identical bits for the per-ray outputs (same kernels, same arithmetic),
the usual 1e-4 for the atomically accumulated per-surfel weights.
"""
import pytest
import torch

import helpers as hp

pytestmark = pytest.mark.gpu


def _call_static(C, st, wc):
    e = hp.empty(wc["means3D"].device)
    return C.trace_surfels_static(st, True, wc["start_from_first"], wc["ray_o"], wc["ray_d"], wc["v"], wc["bg"], wc["means3D"],
                                  wc["shs"] if wc["shs"] is not None else e, wc["sh_degree"],
                                  wc["colors_precomp"] if wc["colors_precomp"] is not None else e,
                                  wc["others_precomp"] if wc["others_precomp"] is not None else e,
                                  wc["opacities"], wc["scales"], 1.0, wc["rotations"],
                                  wc["max_trace_depth"], wc["specular_threshold"])


def test_static_forward_matches_regular_forward_twice():
    from diff_surfel_tracing import _C as C
    assert torch.cuda.is_available()
    # different workloads back to back: the shared scratch keeps the previous call's contents during the next. The
    # third has 51,200 rays: above 32,768 the entry point runs one thread per ray instead of one warp per ray.
    for config, kw in ((3, dict(P=30_000, H=48, W=64)), (1, dict(P=10_000, H=128, W=128)), (1, dict(P=20_000, H=200, W=256))):
        w = hp.workloads.make_workload(config, **kw)
        wc = hp.to_cuda(w)
        st = C.OptiXStateWrapper("")
        C.build_acceleration_structure(st, wc["v"], wc["f"], 1)
        want = hp.cuda_forward(C, st, wc, training=True)
        for call in range(2):
            got = _call_static(C, st, wc)
            torch.cuda.synchronize()
            assert st.status() == 0
            for name, g in zip(hp.FWD_KEYS[:7], got[:7]):
                assert torch.equal(g, want[name]), f"config {config} call {call}: {name} differs"
            tol = 1e-4 * max(1.0, float(want["wet"].abs().max()))
            assert float((got[7] - want["wet"]).abs().max()) <= tol
        assert float(want["acc"].max()) > 0.5


def test_static_forward_on_a_narrow_grid_and_backward_after_it(oracle_mod):
    """A tall one-column grid (its 8x4 pixel tiling would not fit the fixed ray list, so the rays are walked in the
    order given) equals the regular forward; and a backward of the static call's outputs re-traces: it must not
    re-composite the chunk log an earlier regular forward left in the handle (the static call keeps none)."""
    from diff_surfel_tracing import _C as C
    w = hp.workloads.make_workload(1, P=4_000, H=64, W=64)
    wc = hp.to_cuda(w)
    st = C.OptiXStateWrapper("")
    C.build_acceleration_structure(st, wc["v"], wc["f"], 1)
    tall = dict(wc, ray_o=wc["ray_o"].reshape(4096, 1, 3).repeat(8, 1, 1).contiguous(), ray_d=wc["ray_d"].reshape(4096, 1, 3).repeat(8, 1, 1).contiguous())
    want = hp.cuda_forward(C, st, tall, training=True)
    got = _call_static(C, st, tall)
    torch.cuda.synchronize()
    assert st.status() == 0
    for name, g in zip(hp.FWD_KEYS[:7], got[:7]):
        assert torch.equal(g, want[name]), name
    # regular training forward on inputs A (leaves a chunk log), static forward on inputs B, then the backward of B
    wa = wc
    wb = dict(wc, ray_o=wc["ray_o"].flip(1).contiguous(), ray_d=wc["ray_d"].flip(1).contiguous())
    hp.cuda_forward(C, st, wa, training=True)
    assert st.last_forward_serial != 0
    fb = dict(zip(hp.FWD_KEYS, _call_static(C, st, wb)))
    assert st.last_forward_serial == 0
    up = {"rgb": torch.ones((64, 64, 3), device="cuda")}
    gb = hp.cuda_backward(C, st, wb, fb, up, serial=st.last_forward_serial)
    torch.cuda.synchronize()
    assert st.status() == 0
    import numpy as np
    wbh = dict(w, ray_o=w["ray_o"].flip(1).contiguous(), ray_d=w["ray_d"].flip(1).contiguous())
    o = oracle_mod.Oracle(oracle_mod.Scene(w["v"]), impl="restatement", portable_exp=True)
    fo = o.forward(wbh, training=True)
    assert np.array_equal(fb["rgb"].cpu().numpy().view(np.uint32), fo["rgb"].view(np.uint32))
    bo = o.backward(wbh, fo, dict(rgb=np.ones_like(fo["rgb"])))
    for k in ("means3D", "opacities", "scales", "rotations", "shs", "ray_o"):
        assert hp.rel_l2(gb[k].cpu().numpy().reshape(bo[k].shape), bo[k]) <= 1e-3, k


def test_static_forward_rejects_oversized_calls():
    from diff_surfel_tracing import _C as C
    w = hp.workloads.make_workload(1, P=2_000, H=320, W=320)       # 102,400 rays > 65,536
    wc = hp.to_cuda(w)
    st = C.OptiXStateWrapper("")
    C.build_acceleration_structure(st, wc["v"], wc["f"], 1)
    with pytest.raises(RuntimeError, match="at most 65536 rays"):
        _call_static(C, st, wc)
    big = hp.workloads.make_workload(1, P=70_000, H=8, W=8)         # 70,000 surfels > 65,536
    bc = hp.to_cuda(big)
    st2 = C.OptiXStateWrapper("")
    C.build_acceleration_structure(st2, bc["v"], bc["f"], 1)
    with pytest.raises(RuntimeError, match="at most 65536 surfels"):
        _call_static(C, st2, bc)
