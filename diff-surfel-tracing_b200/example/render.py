"""Renders a camera path around a synthetic surfel scene: the counterpart of the reference's
example/render.py for a machine without its trained model, camera file, OpenCV or ffmpeg.

Same flow as the reference script (example/render.py:48-142): surfel parameters -> quads ->
acceleration structure -> for every camera: rays -> tracer -> colour / depth / normal images. The
quads, the rays and the trace all run in this package's CUDA kernels; images are written as PNG
(Pillow) or, without Pillow, binary PPM.

    python diff-surfel-tracing_b200/example/render.py --result_dir /tmp/render --frames 8
"""
import argparse
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import workloads  # noqa: E402
from diff_surfel_tracing import SurfelTracer, SurfelTracingSettings  # noqa: E402


def parse_args(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--result_dir", type=str, default="data/result/synthetic")
    p.add_argument("--scene", type=int, default=3, choices=[1, 2, 3], help="synthetic scene (one of the pinhole benchmark configurations)")
    p.add_argument("--surfels", type=int, default=200_000)
    p.add_argument("--height", type=int, default=270)
    p.add_argument("--width", type=int, default=480)
    p.add_argument("--frames", type=int, default=8)
    p.add_argument("--fov", type=float, default=50.0)
    p.add_argument("--radius", type=float, default=4.0)
    p.add_argument("--white_bg", action="store_true", help="Use white background")
    p.add_argument("--max_trace_depth", type=int, default=0, help="0 means one trace, no bounce")
    p.add_argument("--specular_threshold", type=float, default=0.0)
    p.add_argument("--vis_ext", type=str, default=".png")
    return p.parse_args(argv)


def save_image(path, img):
    """img: (H, W, 3) or (H, W, 1) tensor in [0, 1]."""
    os.makedirs(os.path.dirname(path), exist_ok=True)
    a = img.detach().clamp(0, 1).mul(255).round().to(torch.uint8).cpu().numpy()
    if a.shape[-1] == 1:
        a = np.repeat(a, 3, axis=-1)
    try:
        from PIL import Image
        Image.fromarray(a).save(path)
    except ImportError:
        with open(os.path.splitext(path)[0] + ".ppm", "wb") as f:
            f.write(b"P6 %d %d 255\n" % (a.shape[1], a.shape[0]))
            f.write(a.tobytes())


def normalize_depth(depth, p=0.01):       # example/utils/data_utils.py:52-58
    n = max(int(depth.numel() * p), 1)
    near = depth.ravel().topk(n, largest=False)[0].max()
    far = depth.ravel().topk(n, largest=True)[0].min()
    return (1 - (depth - near) / (far - near + 1e-12)).clip(0, 1)


def visualize_normal(n, R, eps=1e-8):     # example/utils/data_utils.py:61-69
    n = n / (torch.norm(n, dim=-1, keepdim=True) + eps)
    n = n @ R.mT
    n[..., [1, 2]] *= -1
    return n * 0.5 + 0.5


def main(argv=None):
    args = parse_args(argv)
    dev = torch.device("cuda")
    w = workloads.make_workload(args.scene, P=args.surfels, H=8, W=8)
    means3D, scales, rotations, opacities = (w[k].to(dev) for k in ("means3D", "scales", "rotations", "opacities"))
    shs = w["shs"].to(dev) if w["shs"] is not None else None
    colors = w["colors_precomp"].to(dev) if w["colors_precomp"] is not None else None
    others = w["others_precomp"].to(dev) if w["others_precomp"] is not None else None
    print(f"[INFO] Synthetic scene '{w['name']}': {means3D.shape[0]} surfels.")

    tracer = SurfelTracer().eval()
    v = tracer.build_from_surfels(means3D, scales, rotations, rebuild=True)      # get_triangles + build in one call
    print(f"[INFO] Acceleration structure built over {v.shape[0] // 2} triangles.")

    bg = torch.full((3,), 1.0 if args.white_bg else 0.0, device=dev)
    grads3D = torch.zeros_like(means3D)
    z = torch.zeros(1, device=dev)
    H, W = args.height, args.width
    settings = SurfelTracingSettings(image_height=H, image_width=W, tanfovx=math.tan(math.radians(args.fov) / 2),
                                     tanfovy=math.tan(math.radians(args.fov) / 2) * H / W, bg=bg, scale_modifier=1.0,
                                     viewmatrix=z, projmatrix=z, sh_degree=w["sh_degree"], campos=z, prefiltered=False, debug=False,
                                     max_trace_depth=args.max_trace_depth, specular_threshold=args.specular_threshold)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total_ms = 0.0
    for i in range(args.frames):
        ang = 2.0 * math.pi * i / max(args.frames, 1)
        eye = (args.radius * math.cos(ang), args.radius * math.sin(ang), 0.4 * args.radius * math.sin(0.5 * ang))
        K, R, T = workloads.pinhole_camera(H, W, args.fov, eye)
        ev0.record()
        with torch.no_grad():
            rgb, dpt, acc, norm, dist, aux, mid, wet = tracer.forward_camera(
                H, W, K, R, T, v, means3D, grads3D, shs=shs, colors_precomp=colors, others_precomp=others, opacities=opacities,
                scales=scales, rotations=rotations, tracer_settings=settings, start_from_first=w["start_from_first"])
        ev1.record()
        torch.cuda.synchronize()
        total_ms += ev0.elapsed_time(ev1)
        save_image(os.path.join(args.result_dir, "RENDER", f"{i:04d}{args.vis_ext}"), rgb)
        save_image(os.path.join(args.result_dir, "DEPTH", f"{i:04d}{args.vis_ext}"), normalize_depth(dpt))
        save_image(os.path.join(args.result_dir, "NORMAL", f"{i:04d}{args.vis_ext}"), visualize_normal(norm, R.to(dev)))
    status = tracer.optix_context.status()
    print(f"[INFO] Rendering finished: {args.frames} frames of {W}x{H}, {total_ms / max(args.frames, 1):.2f} ms per frame on the GPU, "
          f"device status {status}.")
    return status


if __name__ == "__main__":
    sys.exit(1 if main() else 0)
