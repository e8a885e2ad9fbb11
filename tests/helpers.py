"""Shared helpers of the parity tests: reduced workloads, running the CUDA path and the oracle."""
import numpy as np
import torch

import workloads

# reduced versions of the five configurations: same distributions, sizes the CPU oracle finishes in seconds
REDUCED = {
    1: dict(),                                   # 10k surfels, 128x128: the full tiny configuration
    2: dict(P=60_000, H=96, W=96),
    3: dict(P=90_000, H=72, W=128),
    4: dict(P=60_000, H=4, W=16 * 256),
    5: dict(P=90_000, H=2, W=54 * 96),
}

FWD_KEYS = ("rgb", "dpt", "acc", "norm", "dist", "aux", "mid", "wet")
GRAD_KEYS = ("ray_o", "ray_d", "means3D", "grads3D", "shs", "colors", "others", "opacities", "scales", "rotations")


def reduced_workload(config):
    return workloads.make_workload(config, **REDUCED[config])


def to_cuda(w):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in w.items()}


def empty(dev):
    return torch.empty((0,), dtype=torch.float32, device=dev)


def cuda_forward(_C, state, wc, training=True, diag=None):
    """Calls the binding's trace_surfels with the reference's positional arguments."""
    dev = wc["means3D"].device
    e = empty(dev)
    out = _C.trace_surfels(state, training, wc["start_from_first"], wc["ray_o"], wc["ray_d"], wc["v"], wc["bg"], wc["means3D"],
                           wc["shs"] if wc["shs"] is not None else e, wc["sh_degree"],
                           wc["colors_precomp"] if wc["colors_precomp"] is not None else e,
                           wc["others_precomp"] if wc["others_precomp"] is not None else e,
                           wc["opacities"], wc["scales"], 1.0, wc["rotations"], e, e, e, e, False, False,
                           wc["max_trace_depth"], wc["specular_threshold"], _diag=diag)
    return dict(zip(FWD_KEYS, out))


def cuda_backward(_C, state, wc, fwd, grads, diag=None, serial=0):
    dev = wc["means3D"].device
    e = empty(dev)
    H, W = wc["ray_o"].shape[:2]
    g = lambda k, c: grads[k] if k in grads else torch.zeros((H, W, c), device=dev)
    out = _C.trace_surfels_backward(state, wc["start_from_first"], wc["ray_o"], wc["ray_d"], wc["v"], wc["bg"], wc["means3D"],
                                    wc["shs"] if wc["shs"] is not None else e, wc["sh_degree"],
                                    wc["colors_precomp"] if wc["colors_precomp"] is not None else e,
                                    wc["others_precomp"] if wc["others_precomp"] is not None else e,
                                    wc["opacities"], wc["scales"], 1.0, wc["rotations"], e, e, e, e, False, False,
                                    wc["max_trace_depth"], wc["specular_threshold"],
                                    fwd["rgb"], fwd["dpt"], fwd["acc"], fwd["norm"], fwd["dist"], fwd["aux"], fwd["mid"],
                                    g("rgb", 3), g("dpt", 1), g("acc", 1), g("norm", 3), g("dist", 1), g("aux", 2), _diag=diag,
                                    _forward_serial=serial)
    names = ("ray_o", "ray_d", "means3D", "grads3D", "grads3D_abs", "shs", "colors", "others", "opacities", "scales", "rotations", "trans")
    return dict(zip(names, out))


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    n = np.linalg.norm(b)
    d = np.linalg.norm(a - b)
    return d / n if n > 0 else d
