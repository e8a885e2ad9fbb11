"""Two GPUs: rays sharded over the ranks, surfels replicated, the per-surfel gradients summed by one NCCL
all-reduce INSIDE the autograd backward (SurfelTracer.set_gradient_group). The leaf parameters sit behind
activations (exp / sigmoid / normalisation), as in a training loop, so that a sum applied after
`loss.backward()` would come too late; their gradients must equal those of one GPU tracing all rays.
Skipped on machines with fewer than two GPUs.
"""
import os
import re
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_WORKER = r'''
import os, sys, torch, torch.distributed as dist
root = sys.argv[1]
sys.path.insert(0, root); sys.path.insert(0, os.path.join(root, "diff-surfel-tracing_b200")); sys.path.insert(0, os.path.join(root, "tests"))
import shard, helpers as hp
from diff_surfel_tracing import SurfelTracer, SurfelTracingSettings
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
w = hp.reduced_workload(3)
wc = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in w.items()}

def run(ro, rd, reduce):
    tracer = SurfelTracer().to(dev)
    tracer.set_gradient_group(reduce)
    tracer.build_acceleration_structure(wc["v"], wc["f"], rebuild=True)
    # raw parameters behind the activations a Gaussian model applies
    raw = dict(means=wc["means3D"].clone(), log_scales=wc["scales"].log(), logit_opac=torch.logit(wc["opacities"].clamp(1e-6, 1 - 1e-6)),
               quat=wc["rotations"] * 1.7, shs=wc["shs"].clone(), others=torch.logit(wc["others_precomp"].clamp(1e-6, 1 - 1e-6)))
    raw = {k: v.detach().requires_grad_(True) for k, v in raw.items()}
    g3d = torch.zeros_like(wc["means3D"], requires_grad=True)
    z = torch.zeros(1, device=dev)
    st = SurfelTracingSettings(ro.shape[0], ro.shape[1], 1.0, 1.0, wc["bg"], 1.0, z, z, w["sh_degree"], z, False, False,
                               w["max_trace_depth"], w["specular_threshold"])
    out = tracer(ro, rd, wc["v"], raw["means"], g3d, shs=raw["shs"], others_precomp=torch.sigmoid(raw["others"]),
                 opacities=torch.sigmoid(raw["logit_opac"]), scales=torch.exp(raw["log_scales"]),
                 rotations=torch.nn.functional.normalize(raw["quat"], dim=-1), tracer_settings=st)
    (out[0].sum() + 0.1 * out[1].sum()).backward()
    torch.cuda.synchronize()
    assert tracer.optix_context.status() == 0
    grads = {k: v.grad.clone() for k, v in raw.items()}
    grads["g3d"] = g3d.grad.clone()
    return grads

ro, rd = shard.shard_rays(wc["ray_o"], wc["ray_d"], world, rank)
mine = run(ro.contiguous(), rd.contiguous(), True)
worst = 0.0
if rank == 0:
    full = run(wc["ray_o"], wc["ray_d"], False)
    for k in full:
        a, b = mine[k].double(), full[k].double()
        m = torch.isfinite(a) & torch.isfinite(b)
        err = float((a[m] - b[m]).norm() / b[m].norm().clamp_min(1e-30))
        worst = max(worst, err)
        print("GRAD", k, err)
    print("WORST", worst)
dist.barrier()
dist.destroy_process_group()
'''


def test_two_gpu_gradients_equal_single_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29671", str(script), ROOT]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    m = re.search(r"WORST ([0-9.eE+-]+)", r.stdout)
    assert m and float(m.group(1)) <= 1e-3, r.stdout[-2000:]
