"""Drop-in Python API of the B200-native differentiable surfel tracer.

Same names, argument order, return tuple and error behaviour as the reference package
(diff_surfel_tracing/__init__.py:14-48, 51-201, 204-218, 221-290 of xbillowy/diff-surfel-tracing):

    tracer = SurfelTracer()
    tracer.build_acceleration_structure(v, f, rebuild=True)
    rgb, dpt, acc, norm, dist, aux, mid, wet = tracer(ray_o, ray_d, v, means3D, grads3D, shs=..., ...)

The work is done by hand-written CUDA kernels for sm_100a behind a C ABI (include/dst.h); there
is no OptiX, no CPU path and no eager fallback.
"""
from typing import NamedTuple

import torch
import torch.nn as nn

from . import _C


def cpu_deep_copy_tuple(input_tuple):
    copied_tensors = [item.cpu().clone() if isinstance(item, torch.Tensor) else item for item in input_tuple]
    return tuple(copied_tensors)


def trace_surfels(optix_context, training, start_from_first, ray_o, ray_d, vertices, means3D, grads3D, shs,
                  colors_precomp, others_precomp, opacities, scales, rotations, cov3Ds_precomp, tracer_settings):
    return _TraceSurfels.apply(optix_context, training, start_from_first, ray_o, ray_d, vertices, means3D, grads3D, shs,
                               colors_precomp, others_precomp, opacities, scales, rotations, cov3Ds_precomp, tracer_settings)


class _TraceSurfels(torch.autograd.Function):
    @staticmethod
    def forward(ctx, optix_context, training, start_from_first, ray_o, ray_d, vertices, means3D, grads3D, shs,
                colors_precomp, others_precomp, opacities, scales, rotations, cov3Ds_precomp, tracer_settings):
        s = tracer_settings
        # image_width / image_height are unused by the reference's tracer; here they tell the kernels that a
        # (B, h*w, 3) ray batch consists of whole images, so that they can be walked in pixel tiles (scheduling only)
        iw, ih = int(s.image_width or 0), int(s.image_height or 0)
        optix_context.set_image_width(iw if (iw > 0 and ih > 0 and ray_o.dim() == 3 and ray_o.shape[1] == iw * ih) else 0)
        args = (optix_context, training, start_from_first, ray_o, ray_d, vertices, s.bg, means3D, shs, s.sh_degree,
                colors_precomp, others_precomp, opacities, scales, s.scale_modifier, rotations, cov3Ds_precomp,
                s.viewmatrix, s.projmatrix, s.campos, s.prefiltered, s.debug, s.max_trace_depth, s.specular_threshold)
        if s.debug:
            cpu_args = cpu_deep_copy_tuple(args[1:])
            try:
                out = _C.trace_surfels(*args)
            except Exception as ex:
                torch.save(cpu_args, "snapshot_fw.dump")
                print("\nAn error occured in forward. Please forward snapshot_fw.dump for debugging.")
                raise ex
        else:
            out = _C.trace_surfels(*args)
        out_rgb, out_dpt, out_acc, out_norm, out_dist, out_aux, mid_val, a_weights = out

        ctx.tracer_settings = tracer_settings
        ctx.optix_context = optix_context
        ctx.start_from_first = start_from_first
        ctx.forward_serial = getattr(optix_context, "last_forward_serial", 0)
        ctx.save_for_backward(ray_o, ray_d, vertices, means3D, shs, colors_precomp, others_precomp, opacities, scales,
                              rotations, cov3Ds_precomp, out_rgb, out_dpt, out_acc, out_norm, out_dist, out_aux, mid_val)
        acc_wet = a_weights if a_weights is not None else torch.zeros_like(means3D[:, 0])
        return out_rgb, out_dpt, out_acc, out_norm, out_dist[..., :1].clone(), out_aux, mid_val, acc_wet

    @staticmethod
    def backward(ctx, grad_out_rgb, grad_out_dpt, grad_out_acc, grad_out_norm, grad_out_dist, grad_out_aux, grad_mid_val,
                 grad_acc_wet):
        s = ctx.tracer_settings
        (ray_o, ray_d, vertices, means3D, shs, colors_precomp, others_precomp, opacities, scales, rotations, cov3Ds_precomp,
         out_rgb, out_dpt, out_acc, out_norm, out_dist, out_aux, mid_val) = ctx.saved_tensors
        args = (ctx.optix_context, ctx.start_from_first, ray_o, ray_d, vertices, s.bg, means3D, shs, s.sh_degree,
                colors_precomp, others_precomp, opacities, scales, s.scale_modifier, rotations, cov3Ds_precomp,
                s.viewmatrix, s.projmatrix, s.campos, s.prefiltered, s.debug, s.max_trace_depth, s.specular_threshold,
                out_rgb, out_dpt, out_acc, out_norm, out_dist, out_aux, mid_val,
                grad_out_rgb, grad_out_dpt, grad_out_acc, grad_out_norm, grad_out_dist, grad_out_aux)
        if s.debug:
            cpu_args = cpu_deep_copy_tuple(args[1:])
            try:
                grads = _C.trace_surfels_backward(*args, _forward_serial=ctx.forward_serial)
            except Exception as ex:
                torch.save(cpu_args, "snapshot_bw.dump")
                print("\nAn error occured in backward. Writing snapshot_bw.dump for debugging.\n")
                raise ex
        else:
            grads = _C.trace_surfels_backward(*args, _forward_serial=ctx.forward_serial)
        (grad_ray_o, grad_ray_d, grad_means3D, grad_grads3D, grad_grads3D_abs, grad_shs, grad_colors_precomp,
         grad_others_precomp, grad_opacities, grad_scales, grad_rotations, grad_cov3Ds_precomp) = grads

        def fit(g, t):      # placeholders (empty tensors standing in for absent inputs) take no gradient
            return g if t.numel() != 0 else None

        return (None, None, None, grad_ray_o, grad_ray_d, None, grad_means3D, grad_grads3D, fit(grad_shs, shs),
                fit(grad_colors_precomp, colors_precomp), fit(grad_others_precomp, others_precomp), grad_opacities,
                grad_scales, grad_rotations, fit(grad_cov3Ds_precomp, cov3Ds_precomp), None)


class SurfelTracingSettings(NamedTuple):
    image_height: int  # unused by the tracer, kept for compatibility
    image_width: int  # unused
    tanfovx: float  # unused
    tanfovy: float  # unused
    bg: torch.Tensor
    scale_modifier: float
    viewmatrix: torch.Tensor
    projmatrix: torch.Tensor
    sh_degree: int
    campos: torch.Tensor
    prefiltered: bool
    debug: bool
    max_trace_depth: int = 0
    specular_threshold: float = 0.0


class SurfelTracer(nn.Module):
    def __init__(self) -> None:
        super().__init__()
        self.pkg_dir = _C._PKG
        # name kept from the reference; the object owns the hierarchy and scratch memory of this GPU
        self.optix_context = _C.OptiXStateWrapper(self.pkg_dir)

    def build_acceleration_structure(self, vertices: torch.Tensor, triangles: torch.Tensor, rebuild: bool = 1):
        return _C.build_acceleration_structure(self.optix_context, vertices, triangles, rebuild)

    def enable_distortion(self, enabled: bool = True):
        """Extension: `dist` becomes the depth-distortion map of 2D Gaussian splatting over the primary segment's
        contributions (mapped depth with near 0.2, far 100), differentiable. Off by default: the reference returns zeros."""
        self.optix_context.set_distortion(enabled)

    def set_gradient_group(self, enabled: bool = True, group=None):
        """Multi-GPU training with sharded rays and replicated surfels (the reference is single-GPU): when enabled,
        every backward call sums the per-surfel gradients over the ranks of `group` (None: the default process
        group) with one all-reduce of one flat buffer before autograd receives them. Ray gradients stay local."""
        self.optix_context.reduce_gradients = bool(enabled)
        self.optix_context.process_group = group

    def forward(self, ray_o: torch.Tensor, ray_d: torch.Tensor, vertices: torch.Tensor, means3D: torch.Tensor,
                grads3D: torch.Tensor, shs: torch.Tensor = None, colors_precomp: torch.Tensor = None,
                others_precomp: torch.Tensor = None, opacities: torch.Tensor = None, scales: torch.Tensor = None,
                rotations: torch.Tensor = None, cov3D_precomp: torch.Tensor = None,
                tracer_settings: SurfelTracingSettings = None, start_from_first: bool = True):
        if (shs is None and colors_precomp is None) or (shs is not None and colors_precomp is not None):
            raise Exception('Please provide excatly one of either SHs or precomputed colors!')
        if ((scales is None or rotations is None) and cov3D_precomp is None) or \
                ((scales is not None or rotations is not None) and cov3D_precomp is not None):
            raise Exception('Please provide exactly one of either scale/rotation pair or precomputed 3D covariance!')

        dev = means3D.device
        empty = lambda: torch.empty((0,), dtype=torch.float32, device=dev)
        if shs is None: shs = empty()
        if colors_precomp is None: colors_precomp = empty()
        if others_precomp is None: others_precomp = empty()
        if scales is None: scales = empty()
        if rotations is None: rotations = empty()
        if cov3D_precomp is None: cov3D_precomp = empty()
        if vertices is None: vertices = empty()

        return trace_surfels(self.optix_context, self.training, start_from_first, ray_o, ray_d, vertices, means3D, grads3D,
                             shs, colors_precomp, others_precomp, opacities, scales, rotations, cov3D_precomp, tracer_settings)

    # ---- the two steps that sit next to the tracer in the reference's example pipeline ----

    def get_triangles(self, means3D: torch.Tensor, scales: torch.Tensor, rotations: torch.Tensor):
        """GaussianModel.get_triangles (example/utils/gaussian_utils.py:176-210): (v (4P,3), f (2P,3) int32)."""
        return _C.surfel_quads(self.optix_context, means3D, scales, rotations, True)

    def build_from_surfels(self, means3D: torch.Tensor, scales: torch.Tensor, rotations: torch.Tensor,
                           rebuild: bool = 1, vertices: torch.Tensor = None):
        """get_triangles followed by build_acceleration_structure as one call; returns `v` for the tracer."""
        return _C.build_from_surfels(self.optix_context, means3D, scales, rotations, rebuild, vertices)

    def get_rays(self, H: int, W: int, K, R, T, correct_pix: bool = True, z_depth: bool = False):
        """get_rays (example/utils/ray_utils.py:80-136): (ray_o, ray_d), each (H,W,3) (or (B,H,W,3) for batched K, R, T)."""
        return _C.pinhole_rays(self.optix_context, H, W, K, R, T, correct_pix, z_depth)

    def forward_camera(self, H: int, W: int, K, R, T, vertices: torch.Tensor, means3D: torch.Tensor, grads3D: torch.Tensor,
                       shs: torch.Tensor = None, colors_precomp: torch.Tensor = None, others_precomp: torch.Tensor = None,
                       opacities: torch.Tensor = None, scales: torch.Tensor = None, rotations: torch.Tensor = None,
                       cov3D_precomp: torch.Tensor = None, tracer_settings: SurfelTracingSettings = None,
                       start_from_first: bool = True):
        """forward() for the rays of one pinhole camera, generated inside the trace call instead of by a
        separate get_rays step. Returns forward()'s tuple; the generated rays are kept in `self.last_rays`."""
        dev = means3D.device
        ray_o = torch.empty((H, W, 3), dtype=torch.float32, device=dev)
        ray_d = torch.empty((H, W, 3), dtype=torch.float32, device=dev)
        self.optix_context.next_camera = _C.make_camera(K, R, T, True, False)
        try:
            out = self.forward(ray_o, ray_d, vertices, means3D, grads3D, shs, colors_precomp, others_precomp, opacities,
                               scales, rotations, cov3D_precomp, tracer_settings, start_from_first)
        finally:
            self.optix_context.next_camera = None
        self.last_rays = (ray_o, ray_d)
        return out
