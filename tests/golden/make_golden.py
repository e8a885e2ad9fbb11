"""Generates the golden vectors under tests/golden/ from the reference's own shader sources.

Run in a container that has the reference tree (oracle/build.py compiles its forward.cu /
backward.cu for the host into oracle/_ref/): `python tests/golden/make_golden.py`.
Each file holds, for one small seeded workload, the forward outputs, the per-ray contributing
surfel sequences and the gradients (unit upstream gradient on the outputs the configuration
names) produced by that build with libm's expf, single-threaded. The inputs are regenerated from the seed by
golden_workload(); only outputs are stored.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (ROOT, os.path.join(ROOT, "diff-surfel-tracing_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

SIZES = {1: dict(P=10000, H=32, W=32), 3: dict(P=40000, H=20, W=32), 4: dict(P=20000, H=2, W=512)}
HIT_CAP = 160


def golden_workload(config):
    import workloads
    return workloads.make_workload(config, **SIZES[config])


def main():
    from oracle import build as obuild
    from oracle import oracle as orc
    obuild.build_restatement()
    assert obuild.build_reference(), "the reference tree is needed to generate golden vectors"
    for config in SIZES:
        w = golden_workload(config)
        o = orc.Oracle(orc.Scene(w["v"]), impl="reference", clean=True, hit_cap=HIT_CAP, portable_exp=False, nthreads=1)
        f = o.forward(w)
        assert f["hit_cnt"].max() <= HIT_CAP
        b = o.backward(w, f, {k: np.ones_like(f[k]) for k in w["upstream"]})
        out = {"hit_cap": np.int32(HIT_CAP), "hit_cnt": f["hit_cnt"], "hit_log": f["hit_log"].astype(np.int32)}
        for k in ("rgb", "dpt", "acc", "norm", "aux"):
            out["fwd_" + k] = f[k]
        for k in ("ray_o", "ray_d", "means3D", "grads3D", "shs", "colors", "others", "opacities", "scales", "rotations"):
            out["grad_" + k] = b[k].astype(np.float32)
        path = os.path.join(HERE, f"config{config}.npz")
        np.savez_compressed(path, **out)
        print(path, os.path.getsize(path), "bytes; contributions/ray", float(f["hit_cnt"].mean()))


if __name__ == "__main__":
    main()
