"""The reference's own Python front end running on this repository's extension module.

The adoption route for a user of the reference: keep its `diff_surfel_tracing/__init__.py` (the autograd function,
the settings tuple, the nn.Module) and replace only the compiled `_C` module with this repository's binding. The
test loads that file, unmodified, from the reference tree named by $DST_REFERENCE_DIR (skipped where no reference
tree is present), installs this repository's `_C` as its `_C`, and runs a forward + backward through the
reference's `SurfelTracer` against the CPU oracle. It also checks that the backward of that route re-composites
the chunks the forward logged (the reference passes no serial number; the call is recognised by its saved
`mid_val` tensor) instead of walking the hierarchy again.
"""
import importlib.util
import os
import sys

import numpy as np
import pytest
import torch

import helpers as hp

pytestmark = pytest.mark.gpu


def _reference_frontend():
    root = os.environ.get("DST_REFERENCE_DIR", "")
    path = os.path.join(root, "diff_surfel_tracing", "__init__.py")
    if not root or not os.path.exists(path):
        pytest.skip("no reference tree ($DST_REFERENCE_DIR) on this machine")
    from diff_surfel_tracing import _C
    name = "dst_reference_frontend"
    spec = importlib.util.spec_from_file_location(name, path, submodule_search_locations=[])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    sys.modules[name + "._C"] = _C          # what `from . import _C` inside the reference's file resolves to
    spec.loader.exec_module(mod)
    return mod, _C


def test_reference_frontend_on_this_extension(oracle_mod):
    ref, C = _reference_frontend()
    w = hp.reduced_workload(1)
    wc = hp.to_cuda(w)
    tracer = ref.SurfelTracer()
    tracer.build_acceleration_structure(wc["v"], wc["f"], rebuild=True)
    leaves = {k: wc[k].clone().requires_grad_(True) for k in ("means3D", "shs", "opacities", "scales", "rotations")}
    grads3D = torch.zeros_like(wc["means3D"], requires_grad=True) + 0
    grads3D.retain_grad()
    e = torch.zeros(1, device="cuda")
    settings = ref.SurfelTracingSettings(image_height=128, image_width=128, tanfovx=1.0, tanfovy=1.0, bg=wc["bg"], scale_modifier=1.0,
                                         viewmatrix=e, projmatrix=e, sh_degree=0, campos=e, prefiltered=False, debug=False)
    rgb, dpt, acc, norm, dist, aux, mid, wet = tracer(wc["ray_o"], wc["ray_d"], wc["v"], leaves["means3D"], grads3D, shs=leaves["shs"],
                                                       opacities=leaves["opacities"], scales=leaves["scales"], rotations=leaves["rotations"],
                                                       tracer_settings=settings)
    assert rgb.shape == (128, 128, 3) and dist.shape == (128, 128, 1) and mid.shape == (128, 128, 32) and wet.shape == (10000, 1)
    (rgb.sum() + dpt.sum()).backward()
    torch.cuda.synchronize()
    st = tracer.optix_context
    assert st.status() == 0
    assert st.round_counts() == []          # the logged backward queued no ray for re-tracing and ran no ray-init kernel

    o = oracle_mod.Oracle(oracle_mod.Scene(w["v"]), impl="restatement", portable_exp=True)
    f = o.forward(w, training=True)
    for k, got in (("rgb", rgb), ("dpt", dpt), ("acc", acc), ("norm", norm)):
        assert np.array_equal(got.detach().cpu().numpy().view(np.uint32), f[k].view(np.uint32)), k
    b = o.backward(w, f, dict(rgb=np.ones_like(f["rgb"]), dpt=np.ones_like(f["dpt"])))
    for name, got in (("means3D", leaves["means3D"].grad), ("opacities", leaves["opacities"].grad), ("shs", leaves["shs"].grad),
                      ("scales", leaves["scales"].grad), ("rotations", leaves["rotations"].grad), ("grads3D", grads3D.grad)):
        assert hp.rel_l2(got.cpu().numpy().reshape(b[name].shape), b[name]) <= 1e-3, name
    # inference mode of the reference's module: zeros of shape (P,) as the weights
    tracer.eval()
    out = tracer(wc["ray_o"], wc["ray_d"], wc["v"], wc["means3D"], grads3D, shs=wc["shs"], opacities=wc["opacities"],
                 scales=wc["scales"], rotations=wc["rotations"], tracer_settings=settings)
    assert out[7].shape == (10000,) and torch.equal(out[0], rgb.detach())
