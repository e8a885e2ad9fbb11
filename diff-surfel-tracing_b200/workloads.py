"""Seeded synthetic workloads for the five benchmark configurations.

The reference ships no data; its demo needs a downloaded trained scene. These generators
stand in for such scenes with the shapes, sizes and value distributions of the five
configurations (tiny plumbing scene, object-scale sphere, unbounded reflective scene,
LiDAR street layout, scale-out), built on the CPU from a seeded ``torch.Generator`` so that
every consumer (CUDA path, CPU oracle, bench) sees identical bits.

Geometry follows the reference's surfel -> quad expansion
(example/utils/gaussian_utils.py:176-210): surfel g owns vertices
``mu + 3 * (cu * sx * R[:, 0] + cv * sy * R[:, 1])`` for (cu, cv) = (-1, 1), (-1, -1), (1, 1),
(1, -1) and faces (4g, 4g+1, 4g+2), (4g+1, 4g+2, 4g+3). Rays follow the pinhole convention of
example/utils/ray_utils.py:80-136 (pixel centres at +0.5, unit directions).
"""
import math
from typing import Optional

import torch


def build_rotation(q: torch.Tensor) -> torch.Tensor:
    """Rotation matrices of quaternions stored as (w, x, y, z); columns 0/1 are the tangents."""
    q = q / q.norm(dim=-1, keepdim=True)
    r, x, y, z = q[:, 0], q[:, 1], q[:, 2], q[:, 3]
    R = torch.empty((q.shape[0], 3, 3), dtype=q.dtype, device=q.device)
    R[:, 0, 0] = 1 - 2 * (y * y + z * z)
    R[:, 0, 1] = 2 * (x * y - r * z)
    R[:, 0, 2] = 2 * (x * z + r * y)
    R[:, 1, 0] = 2 * (x * y + r * z)
    R[:, 1, 1] = 1 - 2 * (x * x + z * z)
    R[:, 1, 2] = 2 * (y * z - r * x)
    R[:, 2, 0] = 2 * (x * z - r * y)
    R[:, 2, 1] = 2 * (y * z + r * x)
    R[:, 2, 2] = 1 - 2 * (x * x + y * y)
    return R


def get_triangles(means3D: torch.Tensor, scales: torch.Tensor, rotations: torch.Tensor):
    """(P,3), (P,2), (P,4) -> v (4P,3) float32, f (2P,3) int32."""
    R = build_rotation(rotations)
    a = R[:, :, 0] * scales[:, 0:1]
    b = R[:, :, 1] * scales[:, 1:2]
    corners = torch.tensor([[-1.0, 1.0], [-1.0, -1.0], [1.0, 1.0], [1.0, -1.0]], dtype=means3D.dtype, device=means3D.device) * 3
    v = means3D[:, None, :] + corners[None, :, 0:1] * a[:, None, :] + corners[None, :, 1:2] * b[:, None, :]
    v = v.reshape(-1, 3).contiguous()
    idx = torch.arange(v.shape[0], device=v.device).reshape(-1, 4)
    f = torch.stack([idx[:, :3], idx[:, 1:]], dim=1).reshape(-1, 3).int().contiguous()
    return v, f


def _look_at(cam_pos: torch.Tensor, target: torch.Tensor, up=(0.0, 0.0, 1.0)):
    fwd = target - cam_pos
    fwd = fwd / fwd.norm()
    upv = torch.tensor(up, dtype=cam_pos.dtype)
    if abs(float((fwd * upv).sum())) > 0.999:
        upv = torch.tensor((0.0, 1.0, 0.0), dtype=cam_pos.dtype)
    right = torch.linalg.cross(fwd, upv)
    right = right / right.norm()
    down = torch.linalg.cross(fwd, right)
    return right, down, fwd


def pinhole_rays(H: int, W: int, fovx_deg: float, cam_pos, target=(0.0, 0.0, 0.0), fovy_deg: Optional[float] = None):
    """Unit-direction pinhole rays through pixel centres, shape (H, W, 3) each."""
    cam_pos = torch.as_tensor(cam_pos, dtype=torch.float32)
    target = torch.as_tensor(target, dtype=torch.float32)
    right, down, fwd = _look_at(cam_pos, target)
    fx = 0.5 * W / math.tan(0.5 * math.radians(fovx_deg))
    fy = fx if fovy_deg is None else 0.5 * H / math.tan(0.5 * math.radians(fovy_deg))
    i, j = torch.meshgrid(torch.arange(H, dtype=torch.float32), torch.arange(W, dtype=torch.float32), indexing="ij")
    x = (j + 0.5 - 0.5 * W) / fx
    y = (i + 0.5 - 0.5 * H) / fy
    d = x[..., None] * right + y[..., None] * down + fwd
    d = d / d.norm(dim=-1, keepdim=True)
    o = cam_pos.expand(H, W, 3).contiguous()
    return o, d.contiguous()


def pinhole_camera(H: int, W: int, fovx_deg: float, cam_pos, target=(0.0, 0.0, 0.0)):
    """K (3,3), R (3,3), T (3,) of the camera pinhole_rays() describes, in the reference's convention
    (world-to-camera R, T; example/utils/ray_utils.py:80-136), as float32 tensors."""
    cam_pos = torch.as_tensor(cam_pos, dtype=torch.float32)
    right, down, fwd = _look_at(cam_pos, torch.as_tensor(target, dtype=torch.float32))
    R = torch.stack([right, down, fwd], dim=0)
    T = -(R @ cam_pos)
    fx = 0.5 * W / math.tan(0.5 * math.radians(fovx_deg))
    K = torch.tensor([[fx, 0.0, 0.5 * W], [0.0, fx, 0.5 * H], [0.0, 0.0, 1.0]], dtype=torch.float32)
    return K, R, T


def _rand_quat(n, g):
    q = torch.randn((n, 4), generator=g)
    return q / q.norm(dim=-1, keepdim=True)


def _quat_from_normal(nrm: torch.Tensor, g, jitter: float = 0.0):
    """Quaternions (w,x,y,z) whose third rotation column is `nrm`, with optional small random rotation."""
    n = nrm / nrm.norm(dim=-1, keepdim=True)
    z = torch.tensor([0.0, 0.0, 1.0]).expand_as(n)
    w = 1.0 + (z * n).sum(-1, keepdim=True)
    xyz = torch.linalg.cross(z, n)
    flip = w[:, 0] < 1e-6
    q = torch.cat([w, xyz], dim=-1)
    q[flip] = torch.tensor([0.0, 1.0, 0.0, 0.0])
    q = q / q.norm(dim=-1, keepdim=True)
    if jitter > 0:
        ax = torch.randn((n.shape[0], 3), generator=g) * jitter
        ang = ax.norm(dim=-1, keepdim=True)
        axn = ax / ang.clamp_min(1e-12)
        dq = torch.cat([torch.cos(0.5 * ang), axn * torch.sin(0.5 * ang)], dim=-1)
        # q <- dq * q
        w1, x1, y1, z1 = dq.unbind(-1)
        w2, x2, y2, z2 = q.unbind(-1)
        q = torch.stack([w1 * w2 - x1 * x2 - y1 * y2 - z1 * z2, w1 * x2 + x1 * w2 + y1 * z2 - z1 * y2,
                         w1 * y2 - x1 * z2 + y1 * w2 + z1 * x2, w1 * z2 + x1 * y2 - y1 * x2 + z1 * w2], dim=-1)
    return q.contiguous()


def _sh(n, deg, g):
    M = (deg + 1) ** 2
    shs = torch.randn((n, M, 3), generator=g) * 0.05
    shs[:, 0, :] = 0.5 + 0.2 * torch.randn((n, 3), generator=g)
    return shs.contiguous()


def _unit_dirs(n, g):
    d = torch.randn((n, 3), generator=g)
    return d / d.norm(dim=-1, keepdim=True)


def _unbounded(P, g):
    """2/3 of the surfels in the unit ball, 1/3 in a shell with log-uniform radius in [2, 50]."""
    n_in = (2 * P) // 3
    n_out = P - n_in
    r_in = torch.rand((n_in, 1), generator=g) ** (1.0 / 3.0)
    means_in = _unit_dirs(n_in, g) * r_in
    scales_in = torch.exp(-5.5 + 0.5 * torch.randn((n_in, 2), generator=g))
    r_out = torch.exp(math.log(2.0) + (math.log(50.0) - math.log(2.0)) * torch.rand((n_out, 1), generator=g))
    means_out = _unit_dirs(n_out, g) * r_out
    scales_out = r_out * torch.exp(-4.0 + 0.5 * torch.randn((n_out, 2), generator=g))
    means = torch.cat([means_in, means_out]).contiguous()
    scales = torch.cat([scales_in, scales_out]).contiguous()
    return means, scales


def _street(P, g):
    """Ground plane z=0 over 100x100 m plus faces of 200 random axis-aligned boxes."""
    n_ground = P // 2
    n_box = P - n_ground
    ground = torch.cat([(torch.rand((n_ground, 2), generator=g) - 0.5) * 100.0, torch.zeros((n_ground, 1))], dim=-1)
    ground_n = torch.tensor([0.0, 0.0, 1.0]).expand(n_ground, 3)
    nb = 200
    centre = torch.cat([(torch.rand((nb, 2), generator=g) - 0.5) * 90.0, torch.zeros((nb, 1))], dim=-1)
    size = 1.0 + 9.0 * torch.rand((nb, 3), generator=g)
    centre[:, 2] = 0.5 * size[:, 2]
    bi = torch.randint(0, nb, (n_box,), generator=g)
    face = torch.randint(0, 6, (n_box,), generator=g)
    uvw = torch.rand((n_box, 3), generator=g) - 0.5
    axis = face // 2
    sign = (face % 2).float() * 2 - 1
    uvw[torch.arange(n_box), axis] = 0.5 * sign
    pts = centre[bi] + uvw * size[bi]
    nrm = torch.zeros((n_box, 3))
    nrm[torch.arange(n_box), axis] = sign
    means = torch.cat([ground, pts]).contiguous()
    normals = torch.cat([ground_n, nrm]).contiguous()
    return means, normals


def lidar_rays(B=4, beams=64, azimuths=2048, g=None):
    """(B, beams*azimuths, 3) spinning-scan rays from B poses 1.8 m above the ground."""
    el = torch.deg2rad(torch.linspace(-25.0, 3.0, beams))
    az = torch.arange(azimuths, dtype=torch.float32) * (2 * math.pi / azimuths)
    ce, se = torch.cos(el)[:, None], torch.sin(el)[:, None]
    d = torch.stack([ce * torch.cos(az)[None, :], ce * torch.sin(az)[None, :], se.expand(beams, azimuths)], dim=-1)
    d = d.reshape(1, beams * azimuths, 3).expand(B, -1, -1).contiguous()
    pos = torch.cat([(torch.rand((B, 2), generator=g) - 0.5) * 60.0, torch.full((B, 1), 1.8)], dim=-1)
    o = pos[:, None, :].expand(B, beams * azimuths, 3).contiguous()
    return o, d


CONFIG_DEFAULTS = {
    1: dict(P=10_000, H=128, W=128),
    2: dict(P=500_000, H=800, W=800),
    3: dict(P=3_000_000, H=1080, W=1920),
    4: dict(P=1_000_000, H=4, W=64 * 2048),
    5: dict(P=6_000_000, H=8, W=1080 * 1920),
}


def make_workload(config: int, P: Optional[int] = None, H: Optional[int] = None, W: Optional[int] = None,
                  seed: Optional[int] = None, cameras: Optional[int] = None):
    """Builds one configuration (optionally at reduced surfel / ray counts) as CPU float32 tensors.

    Returns a dict with: means3D, scales, rotations, opacities, shs | colors_precomp,
    others_precomp | None, v, f, ray_o, ray_d (H, W, 3), bg, sh_degree, max_trace_depth,
    specular_threshold, start_from_first, upstream (names of the outputs that get a unit
    upstream gradient), name.
    """
    d = CONFIG_DEFAULTS[config]
    P = d["P"] if P is None else P
    H = d["H"] if H is None else H
    W = d["W"] if W is None else W
    g = torch.Generator().manual_seed(0 if config == 1 else config if seed is None else seed)
    out = dict(config=config, bg=torch.zeros(3), others_precomp=None, shs=None, colors_precomp=None,
               max_trace_depth=0, specular_threshold=0.0, start_from_first=True, sh_degree=0, upstream=("rgb",))
    if config == 1:
        r = torch.rand((P, 1), generator=g) ** (1.0 / 3.0)
        means = _unit_dirs(P, g) * r
        scales = torch.exp(-4.0 + 0.5 * torch.randn((P, 2), generator=g))
        rots = _rand_quat(P, g)
        opac = torch.sigmoid(1.5 * torch.randn((P, 1), generator=g))
        out["shs"] = _sh(P, 0, g)
        ray_o, ray_d = pinhole_rays(H, W, 60.0, (0.0, -3.0, 0.0), fovy_deg=60.0)
        out["name"] = f"tiny {P} surfels / {H}x{W} rays / SH0"
    elif config == 2:
        dirs = _unit_dirs(P, g)
        means = dirs * (1.0 + 0.02 * torch.randn((P, 1), generator=g))
        scales = torch.exp(-5.0 + 0.4 * torch.randn((P, 2), generator=g))
        rots = _quat_from_normal(dirs, g, jitter=0.1)
        opac = torch.sigmoid(1.0 + torch.randn((P, 1), generator=g))
        out["shs"] = _sh(P, 3, g)
        out["sh_degree"] = 3
        ray_o, ray_d = pinhole_rays(H, W, 40.0, (0.0, -4.0, 0.0))
        out["name"] = f"object {P} surfels / {H}x{W} rays / SH3"
    elif config in (3, 5):
        means, scales = _unbounded(P, g)
        rots = _rand_quat(P, g)
        opac = torch.sigmoid(0.5 + 1.5 * torch.randn((P, 1), generator=g))
        out["shs"] = _sh(P, 3, g)
        out["sh_degree"] = 3
        out["others_precomp"] = torch.rand((P, 2), generator=g).contiguous()
        if config == 3:
            out["max_trace_depth"], out["specular_threshold"] = 1, 0.5
            ray_o, ray_d = pinhole_rays(H, W, 50.0, (0.0, -4.0, 0.0))
            out["name"] = f"unbounded reflective {P} surfels / {H}x{W} rays / SH3 / 1 bounce"
        else:
            out["max_trace_depth"], out["specular_threshold"] = 2, 0.3
            ncam = H if cameras is None else cameras
            per = W
            hh = 1080 if per == 1080 * 1920 else max(1, int(round(math.sqrt(per * 9 / 16))))
            ww = per // hh
            os_, ds_ = [], []
            for c in range(ncam):
                ang = 2 * math.pi * c / ncam
                o, dd = pinhole_rays(hh, ww, 50.0, (4.0 * math.sin(ang), -4.0 * math.cos(ang), 0.0))
                os_.append(o.reshape(-1, 3))
                ds_.append(dd.reshape(-1, 3))
            ray_o, ray_d = torch.stack(os_).contiguous(), torch.stack(ds_).contiguous()
            out["name"] = f"scale-out {P} surfels / {ncam}x{hh}x{ww} rays / SH3 / 2 bounces"
    elif config == 4:
        means, normals = _street(P, g)
        scales = torch.exp(-3.0 + 0.4 * torch.randn((P, 2), generator=g))
        rots = _quat_from_normal(normals, g)
        opac = torch.sigmoid(2.0 + torch.randn((P, 1), generator=g))
        out["colors_precomp"] = torch.rand((P, 3), generator=g).contiguous()
        beams = 64 if (W % 64 == 0 and W >= 64 * 64) else 16 if W % 16 == 0 else 1
        az = W // beams
        ray_o, ray_d = lidar_rays(H, beams, az, g)
        out["upstream"] = ("rgb", "dpt")
        out["name"] = f"lidar {P} surfels / {H}x{beams}x{az} rays / precomputed colours"
    else:
        raise ValueError(f"unknown config {config}")
    v, f = get_triangles(means, scales, rots)
    out.update(means3D=means.contiguous(), scales=scales.contiguous(), rotations=rots.contiguous(),
               opacities=opac.contiguous(), v=v, f=f, ray_o=ray_o.contiguous(), ray_d=ray_d.contiguous())
    return out
