"""Generates tests/golden/prep.npz by running the reference's own Python functions on CPU.

  GaussianModel.get_triangles     example/utils/gaussian_utils.py:176-210
  get_rays                        example/utils/ray_utils.py:80-136

Run in a container that has the reference tree: `python tests/golden/make_golden_prep.py`.
The reference modules are imported in place ($DST_REFERENCE_DIR, or the location used when this
repository was developed); `plyfile`, which only the model loader needs, is replaced by an empty
stand-in module. Inputs are regenerated from the seed by prep_inputs(); the file stores the
reference's outputs only.
"""
import math
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("DST_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")

P_GOLDEN = 517
CAMERAS = 3
H_GOLDEN, W_GOLDEN = 13, 29


def prep_inputs():
    """Seeded surfel parameters and cameras: the value distributions of the benchmark workloads
    (unit-ball core + large shell surfels, un-normalised quaternions) at a size that is cheap to store."""
    g = np.random.default_rng(20240611)
    P = P_GOLDEN
    means = g.normal(size=(P, 3)).astype(np.float32)
    means[P // 2:] *= np.float32(20.0)
    log_scales = g.normal(-4.0, 1.0, size=(P, 2)).astype(np.float32)
    log_scales[P // 2:] += np.float32(3.0)
    rot = g.normal(size=(P, 4)).astype(np.float32) * g.uniform(0.2, 5.0, size=(P, 1)).astype(np.float32)
    cams = []
    for c in range(CAMERAS):
        ang = 2.0 * math.pi * c / CAMERAS + 0.3
        eye = np.array([4.0 * math.cos(ang), 4.0 * math.sin(ang), 0.7 * c - 0.5])
        fwd = -eye / np.linalg.norm(eye)
        right = np.cross(fwd, np.array([0.0, 0.0, 1.0])); right /= np.linalg.norm(right)
        down = np.cross(fwd, right)
        R = np.stack([right, down, fwd], 0)                 # world -> camera rows
        T = -R @ eye
        fl = 0.5 * W_GOLDEN / math.tan(math.radians(25.0 + 10.0 * c))
        K = np.array([[fl, 0.0, 0.5 * W_GOLDEN + 0.25 * c], [0.0, fl * (1.0 + 0.05 * c), 0.5 * H_GOLDEN], [0.0, 0.0, 1.0]])
        cams.append((K.astype(np.float32), R.astype(np.float32), T.astype(np.float32).reshape(3, 1)))
    return means, log_scales, rot, cams


def main():
    import torch
    sys.modules.setdefault("plyfile", types.SimpleNamespace(PlyData=None))
    sys.path.insert(0, os.path.join(REF, "example"))
    from utils.gaussian_utils import GaussianModel
    from utils.ray_utils import get_rays

    means, log_scales, rot, cams = prep_inputs()
    torch.set_num_threads(1)
    pcd = GaussianModel(3)
    pcd._xyz = torch.from_numpy(means)
    pcd._scaling = torch.from_numpy(log_scales)
    pcd._rotation = torch.from_numpy(rot)
    with torch.no_grad():
        v, f = pcd.get_triangles()
        scales = pcd.get_scaling.numpy().copy()           # what the tracer receives (exp of the stored value)
        rotations = pcd.get_rotation.numpy().copy()       # normalised quaternions, as render.py passes them
    out = {"v": v.numpy(), "f": f.numpy(), "scales": scales, "rotations": rotations}
    for c, (K, R, T) in enumerate(cams):
        for z in (0, 1):
            o, d = get_rays(H_GOLDEN, W_GOLDEN, torch.from_numpy(K), torch.from_numpy(R), torch.from_numpy(T), z_depth=bool(z))
            out[f"ray_o_{c}_{z}"] = o.numpy()
            out[f"ray_d_{c}_{z}"] = d.numpy()
    path = os.path.join(HERE, "prep.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
