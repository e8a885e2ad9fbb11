"""Binding of libdst_b200.so with the call surface of the reference's extension module.

Mirrors ext.cpp:7-12 of the reference: a state object plus build_acceleration_structure,
trace_surfels and trace_surfels_backward with the same argument order and return tuples
(trace_surfels.h:10-83). Tensors are allocated here with torch and handed to the C ABI
(include/dst.h) as raw device pointers; all work is enqueued on torch's current CUDA stream.
There is no CPU path: loading fails loudly when the library is missing and every call fails when
no CUDA device is present.
"""
import ctypes as C
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(os.path.dirname(_PKG), "libdst_b200.so")

NUM_CHANNELS = 3
AUX_CHANNELS = 2
MID_CHANNELS = 16


class _TraceInputs(C.Structure):
    _fields_ = ([(n, C.c_int32) for n in ("H", "W", "P", "sh_degree", "sh_coeffs", "max_trace_depth", "mid_stride", "start_from_first")]
                + [("specular_threshold", C.c_float), ("scale_modifier", C.c_float)]
                + [(n, C.c_void_p) for n in ("ray_o", "ray_d", "vertices", "background", "means3D", "shs", "colors_precomp",
                                             "others_precomp", "opacities", "scales", "rotations")])


class _FwdArgs(C.Structure):
    _fields_ = ([("inp", _TraceInputs), ("training", C.c_int32), ("hit_cap", C.c_int32)]
                + [(n, C.c_void_p) for n in ("out_rgb", "out_dpt", "out_acc", "out_norm", "out_dist", "out_aux", "mid_val", "a_weights",
                                             "hit_log", "hit_cnt", "counters")])


class _BwdArgs(C.Structure):
    _fields_ = ([("inp", _TraceInputs)]
                + [(n, C.c_void_p) for n in ("out_rgb", "out_dpt", "out_acc", "out_norm", "out_dist", "out_aux", "mid_val",
                                             "dL_drgb", "dL_ddpt", "dL_dacc", "dL_dnorm", "dL_ddist", "dL_daux",
                                             "dL_dray_o", "dL_dray_d", "dL_dmeans3D", "dL_dgrads3D", "dL_dshs", "dL_dcolors",
                                             "dL_dothers", "dL_dopacities", "dL_dscales", "dL_drotations", "counters")]
                + [("forward_serial", C.c_uint64)])


_lib = None


class _Camera(C.Structure):
    _fields_ = [("K", C.c_float * 9), ("R", C.c_float * 9), ("T", C.c_float * 3), ("correct_pix", C.c_int32), ("z_depth", C.c_int32)]


MAX_CAMERAS = 64


def lib():
    """Loads the CUDA library on first use; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise ImportError(f"{_LIB_PATH} not found: build it with `python diff-surfel-tracing_b200/build.py` "
                              "(this package has no CPU or eager fallback)")
        l = C.CDLL(_LIB_PATH)
        l.dst_create.argtypes = [C.c_int, C.POINTER(C.c_void_p)]
        l.dst_destroy.argtypes = [C.c_void_p]
        l.dst_last_error.argtypes = [C.c_void_p]
        l.dst_last_error.restype = C.c_char_p
        l.dst_build.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int, C.c_void_p]
        l.dst_forward.argtypes = [C.c_void_p, C.POINTER(_FwdArgs), C.c_void_p]
        l.dst_backward.argtypes = [C.c_void_p, C.POINTER(_BwdArgs), C.c_void_p]
        l.dst_forward_static.argtypes = [C.c_void_p, C.POINTER(_FwdArgs), C.c_void_p]
        l.dst_surfel_quads.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]
        l.dst_build_from_surfels.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_void_p]
        l.dst_pinhole_rays.argtypes = [C.c_void_p, C.POINTER(_Camera), C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        l.dst_forward_camera.argtypes = [C.c_void_p, C.POINTER(_FwdArgs), C.POINTER(_Camera), C.c_void_p]
        l.dst_status.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), C.c_void_p]
        l.dst_bvh_info.argtypes = [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
        l.dst_debug_knearest.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        l.dst_forward_serial.argtypes = [C.c_void_p, C.POINTER(C.c_uint64)]
        l.dst_set_option.argtypes = [C.c_void_p, C.c_int, C.c_int64]
        l.dst_kernel_launches.argtypes = [C.c_void_p, C.POINTER(C.c_int64)]
        l.dst_profile_enable.argtypes = [C.c_void_p, C.c_int]
        l.dst_profile_read.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_int32)]
        l.dst_profile_launches.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_float), C.c_int32, C.POINTER(C.c_int32)]
        l.dst_debug_round_counts.argtypes = [C.c_void_p, C.POINTER(C.c_int32), C.c_int32, C.c_void_p]
        l.dst_debug_read_bandwidth.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.POINTER(C.c_float), C.c_void_p]
        l.dst_debug_chunk_log.argtypes = [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
        l.dst_debug_quad_frames.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        _lib = l
    return _lib


def _stream(state=None):
    """torch's current stream on the state's GPU (the device the library switches to for the call)."""
    return C.c_void_p(torch.cuda.current_stream(None if state is None else state.device).cuda_stream)


def _check(state, rc):
    if rc != 0:
        msg = lib().dst_last_error(state.handle if state is not None else None)
        raise RuntimeError((msg or b"unknown error").decode())


def _on_device(state, t, name):
    """Every tensor of a call must live on the GPU the state was created on: the library runs its kernels
    there, and a pointer into another GPU's memory would fault inside a kernel instead of raising here."""
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")          # CHECK_INPUT, trace_surfels.cpp:23-24
    if state is not None and t.device.index != state.device:
        raise RuntimeError(f"{name} is on cuda:{t.device.index} but this tracer state was created on cuda:{state.device}")


def _cuda_f32(t, name, state=None):
    """Contiguous float32 CUDA storage of `t`, 16-byte aligned (the kernels use vector loads)."""
    _on_device(state, t, name)
    if t.dtype != torch.float32:
        raise RuntimeError(f"{name} must be float32")
    t = t.contiguous()
    if t.data_ptr() % 16 != 0:
        t = t.clone()
    return t


def _ptr(t):
    return None if t is None or t.numel() == 0 else t.data_ptr()


class OptiXStateWrapper:
    """Tracer state for the current CUDA device (name kept from the reference, ext.cpp:8).

    The constructor argument (the reference's package directory holding its PTX files,
    optix_wrapper.cpp:166-204) is accepted and ignored: nothing is compiled at run time.
    """

    def __init__(self, pkg_dir: str = ""):
        if not torch.cuda.is_available():
            raise RuntimeError("diff_surfel_tracing needs a CUDA device; there is no CPU path")
        self.device = torch.cuda.current_device()
        h = C.c_void_p()
        rc = lib().dst_create(self.device, C.byref(h))
        if rc != 0:
            raise RuntimeError(lib().dst_last_error(None).decode())
        self.handle = h
        self._keep = None
        self.last_forward_serial = 0
        self._logged_mid = None
        self.reduce_gradients = False   # sum the per-surfel gradients over `process_group` inside every backward call
        self.process_group = None
        self.grad_bucket = None     # flat buffer holding the per-surfel gradients of the last backward call

    def __del__(self):
        try:
            if getattr(self, "handle", None):
                lib().dst_destroy(self.handle)
                self.handle = None
        except Exception:
            pass

    def status(self):
        """Synchronises and returns (then clears) the device status bits (DST_STATUS_* of dst.h)."""
        f = C.c_uint32(0)
        _check(self, lib().dst_status(self.handle, C.byref(f), _stream(self)))
        return f.value

    def set_wavefront_min_rays(self, n):
        """Trace calls with at least `n` rays run as rounds of gather / composite kernels over the
        live rays; smaller calls use one thread per ray for the whole path (same results)."""
        _check(self, lib().dst_set_option(self.handle, 1, int(n)))

    def set_chunk_log_max_records(self, n):
        """Upper limit on the chunk-log size in records of 136 bytes (0: built-in limit only)."""
        _check(self, lib().dst_set_option(self.handle, 3, int(n)))

    def set_image_width(self, width):
        """Hint for (B, h*w, 3) ray batches of whole images: the image width (0: unknown). Scheduling only."""
        _check(self, lib().dst_set_option(self.handle, 6, int(width)))

    def set_single_kernel_refit(self, on):
        """build_from_surfels(rebuild=0): expand the quads inside the refit kernel (one launch) instead of before it."""
        _check(self, lib().dst_set_option(self.handle, 4, int(bool(on))))

    def set_chunk_log(self, on):
        """Keep (default) or drop the per-ray chunk log training forwards leave for the backward (about 1.6 KB per ray)."""
        _check(self, lib().dst_set_option(self.handle, 2, int(bool(on))))

    def kernel_launches(self):
        """Kernels this state has enqueued since it was created."""
        n = C.c_int64(0)
        _check(self, lib().dst_kernel_launches(self.handle, C.byref(n)))
        return n.value

    def set_distortion(self, on):
        """Extension: compute the depth-distortion output (channel 0 of out_dist) and its gradient. Off by default: the
        reference leaves the output at zero."""
        _check(self, lib().dst_set_option(self.handle, 8, int(bool(on))))

    def set_stable_lists(self, on):
        """Wavefront rounds keep the live-ray list in its original (pixel tile) order (default) or append survivors
        warp by warp as they finish. Scheduling only."""
        _check(self, lib().dst_set_option(self.handle, 7, int(bool(on))))

    def set_forward_slices(self, n):
        """Large forward calls run as `n` independent slices of the ray grid on streams of their own (0: chosen from the
        ray count, 1: no slicing). Scheduling only."""
        _check(self, lib().dst_set_option(self.handle, 9, int(n)))

    def profile(self, on=True):
        """Records CUDA events around the build, forward and backward kernels of later calls; on=2 also around
        every launch of the gather kernel."""
        _check(self, lib().dst_profile_enable(self.handle, int(on)))

    def profile_launches(self, kind="gather", cap=1024):
        """Milliseconds of every recorded launch of `kind` since the last read (waits for the events)."""
        which = ("build", "forward", "backward", "gather").index(kind)
        buf, n = (C.c_float * cap)(), C.c_int32(0)
        _check(self, lib().dst_profile_launches(self.handle, which, buf, cap, C.byref(n)))
        return [buf[i] for i in range(min(n.value, cap))]

    def profile_read(self):
        """{kind: (summed ms, launches)} since the last read; waits for the recorded events."""
        out = {}
        for i, k in enumerate(("build", "forward", "backward")):
            ms, n = C.c_float(0), C.c_int32(0)
            _check(self, lib().dst_profile_read(self.handle, i, C.byref(ms), C.byref(n)))
            out[k] = (ms.value, n.value)
        return out

    def round_counts(self):
        """Live-list length of every wavefront round of the last trace call (synchronises)."""
        buf = (C.c_int32 * 50)()
        _check(self, lib().dst_debug_round_counts(self.handle, buf, 50, _stream(self)))
        out = list(buf)
        while out and out[-1] == 0:
            out.pop()
        return out

    def read_bandwidth(self, nbytes=64 << 20, reps=50):
        """GB/s of repeated streaming reads of an `nbytes` buffer (64 MB fits the L2 cache: the L2 read bandwidth)."""
        v = C.c_float(0)
        _check(self, lib().dst_debug_read_bandwidth(self.handle, int(nbytes), int(reps), C.byref(v), _stream(self)))
        return v.value

    def chunk_log(self):
        """dict(records_wanted, records_held, bytes_per_record) of the chunk log (records_wanted -1: not known yet)."""
        a, b, c = C.c_int64(), C.c_int64(), C.c_int64()
        _check(self, lib().dst_debug_chunk_log(self.handle, C.byref(a), C.byref(b), C.byref(c)))
        return dict(records_wanted=a.value, records_held=b.value, bytes_per_record=c.value)

    def info(self):
        a, b, c = C.c_int64(), C.c_int64(), C.c_int64()
        _check(self, lib().dst_bvh_info(self.handle, C.byref(a), C.byref(b), C.byref(c)))
        return dict(surfels=a.value, nodes=b.value, device_bytes=c.value)


def build_acceleration_structure(state, vertices, triangles, rebuild):
    """trace_surfels.cpp:36-159: (Nv, 3) float vertices, (Nt, 3) int32 triangles, rebuild > 0 builds, 0 refits."""
    if vertices.dim() != 2 or vertices.size(1) != 3:
        raise RuntimeError("vertices must have dimensions (num_vertices, 3)")
    if triangles is not None and (triangles.dim() != 2 or triangles.size(1) != 3):
        raise RuntimeError("triangles must have dimensions (num_triangles, 3)")
    v = _cuda_f32(vertices, "vertices", state)
    if triangles is not None:
        _on_device(state, triangles, "triangles")
        if triangles.dtype != torch.int32:
            raise RuntimeError("triangles must be int32")
        triangles = triangles.contiguous()
    nt = 0 if triangles is None else triangles.size(0)
    rc = lib().dst_build(state.handle, v.data_ptr(), v.size(0), _ptr(triangles), nt, int(rebuild), _stream(state))
    _check(state, rc)
    state._keep = (v, triangles)      # the build kernels read them asynchronously on the current stream


def _check_element_counts(P, t):
    """Element counts the kernels rely on (a wrong-sized tensor would be read out of bounds on the device).
    t: name -> tensor; empty tensors stand for absent optional inputs."""
    want = dict(vertices=12 * P, background=3, opacities=P, scales=2 * P, rotations=4 * P)
    if t["colors_precomp"].numel() != 0:
        want["colors_precomp"] = 3 * P
    if t["others_precomp"].numel() != 0:
        want["others_precomp"] = 2 * P
    for n, cnt in want.items():
        if t[n].numel() != cnt:
            raise RuntimeError(f"{n} has {t[n].numel()} elements, expected {cnt} for {P} surfels")
    if t["shs"].numel() != 0 and (t["shs"].dim() != 3 or t["shs"].size(0) != P or t["shs"].size(2) != 3):
        raise RuntimeError(f"shs must have dimensions ({P}, coefficients, 3)")


def _inputs(state, start_from_first, ray_o, ray_d, vertices, background, means3D, shs, degree, colors_precomp,
            others_precomp, opacities, scales, scale_modifier, rotations, max_trace_depth, specular_threshold):
    if means3D.dim() != 2 or means3D.size(1) != 3:
        raise RuntimeError("means3D must have dimensions (num_points, 3)")
    if ray_o.dim() != 3 or ray_o.size(2) != 3 or ray_o.shape != ray_d.shape:
        raise RuntimeError("ray_o and ray_d must have dimensions (H, W, 3)")
    keep = {n: _cuda_f32(t, n, state) for n, t in (
        ("ray_o", ray_o), ("ray_d", ray_d), ("vertices", vertices), ("background", background), ("means3D", means3D), ("shs", shs),
        ("colors_precomp", colors_precomp), ("others_precomp", others_precomp), ("opacities", opacities), ("scales", scales),
        ("rotations", rotations))}
    if keep["scales"].numel() == 0 or keep["rotations"].numel() == 0:
        raise RuntimeError("scales and rotations are required (a precomputed covariance is never read by the tracer)")
    _check_element_counts(means3D.size(0), keep)
    i = _TraceInputs()
    i.H, i.W, i.P = ray_o.size(0), ray_o.size(1), means3D.size(0)
    i.sh_degree = int(degree)
    i.sh_coeffs = keep["shs"].size(1) if keep["shs"].numel() != 0 else 0
    i.max_trace_depth = int(max_trace_depth)
    i.mid_stride = MID_CHANNELS * max(2, int(max_trace_depth) + 1)
    i.start_from_first = int(bool(start_from_first))
    i.specular_threshold = float(specular_threshold)
    i.scale_modifier = float(scale_modifier)
    for n in ("ray_o", "ray_d", "vertices", "background", "means3D", "shs", "colors_precomp", "others_precomp",
              "opacities", "scales", "rotations"):
        setattr(i, n, _ptr(keep[n]))
    return i, keep


def trace_surfels(state, training, start_from_first, ray_o, ray_d, vertices, background, means3D, shs, degree,
                  colors_precomp, others_precomp, opacities, scales, scale_modifier, rotations, transMat_precomp,
                  viewmatrix, projmatrix, campos, prefiltered, debug, max_trace_depth, specular_threshold,
                  _diag=None):
    """trace_surfels.cpp:162-304. Returns out_rgb, out_dpt, out_acc, out_norm, out_dist, out_aux, mid_val, a_weights.

    `mid_val` has 16 * max(2, max_trace_depth + 1) channels (the reference is compiled for one bounce
    and always returns 32). `_diag`, if a dict, receives per-ray hit logs and traversal counters.
    """
    i, keep = _inputs(state, start_from_first, ray_o, ray_d, vertices, background, means3D, shs, degree, colors_precomp,
                      others_precomp, opacities, scales, scale_modifier, rotations, max_trace_depth, specular_threshold)
    H, W, P = i.H, i.W, i.P
    dev = means3D.device
    f32 = dict(dtype=torch.float32, device=dev)
    out_rgb = torch.empty((H, W, NUM_CHANNELS), **f32)
    out_dpt = torch.empty((H, W, 1), **f32)
    out_acc = torch.empty((H, W, 1), **f32)
    out_norm = torch.empty((H, W, 3), **f32)
    out_dist = torch.empty((H, W, 3), **f32)
    out_aux = torch.empty((H, W, AUX_CHANNELS), **f32)
    mid_val = torch.empty((H, W, i.mid_stride), **f32)
    a_weights = torch.empty((P, 1), **f32) if training else None
    a = _FwdArgs()
    a.inp = i
    a.training = int(bool(training))
    a.out_rgb, a.out_dpt, a.out_acc, a.out_norm = out_rgb.data_ptr(), out_dpt.data_ptr(), out_acc.data_ptr(), out_norm.data_ptr()
    a.out_dist, a.out_aux, a.mid_val = out_dist.data_ptr(), out_aux.data_ptr(), mid_val.data_ptr()
    a.a_weights = _ptr(a_weights)
    if _diag is not None:
        cap = int(_diag.get("hit_cap", 0))
        if cap:
            _diag["hit_log"] = torch.full((H * W, cap), -1, dtype=torch.int32, device=dev)
            _diag["hit_cnt"] = torch.zeros((H * W,), dtype=torch.int32, device=dev)
            a.hit_cap, a.hit_log, a.hit_cnt = cap, _diag["hit_log"].data_ptr(), _diag["hit_cnt"].data_ptr()
        _diag["counters"] = torch.zeros((8,), dtype=torch.int64, device=dev)
        a.counters = _diag["counters"].data_ptr()
    cam = getattr(state, "next_camera", None)
    state.next_camera = None
    if cam is not None:       # the rays are generated by the first kernel of the call, into ray_o / ray_d
        if keep["ray_o"].data_ptr() != ray_o.data_ptr() or keep["ray_d"].data_ptr() != ray_d.data_ptr():
            raise RuntimeError("with a camera, ray_o and ray_d must be contiguous 16-byte aligned buffers")
        _check(state, lib().dst_forward_camera(state.handle, C.byref(a), C.byref(cam), _stream(state)))
    else:
        _check(state, lib().dst_forward(state.handle, C.byref(a), _stream(state)))
    ser = C.c_uint64(0)
    _check(state, lib().dst_forward_serial(state.handle, C.byref(ser)))
    state.last_forward_serial = ser.value       # names the chunk log this call left in the handle (0: none)
    # the saved tensor that identifies this call to a backward that is not told the serial (a caller written against
    # the reference's extension module passes exactly the reference's arguments)
    state._logged_mid = (mid_val.data_ptr(), tuple(mid_val.shape)) if ser.value else None
    return out_rgb, out_dpt, out_acc, out_norm, out_dist, out_aux, mid_val, a_weights


def trace_surfels_backward(state, start_from_first, ray_o, ray_d, vertices, background, means3D, shs, degree, colors_precomp,
                           others_precomp, opacities, scales, scale_modifier, rotations, transMat_precomp, viewmatrix,
                           projmatrix, campos, prefiltered, debug, max_trace_depth, specular_threshold,
                           out_rgb, out_dpt, out_acc, out_norm, out_dist, out_aux, mid_val,
                           dL_drgb, dL_ddpt, dL_dacc, dL_dnorm, dL_ddist, dL_daux, _diag=None, _forward_serial=None):
    """trace_surfels.cpp:307-464. Returns the 12 gradients in the reference's order:
    ray_o, ray_d, means3D, grads3D, grads3D_abs (zeros), shs, colors_precomp, others_precomp,
    opacities, scales, rotations, transMat_precomp (zeros).

    `_forward_serial`: `state.last_forward_serial` as it was right after the forward call these saved
    tensors come from; when it still names the handle's chunk log the backward re-composites the logged
    chunks instead of walking the hierarchy again (same result). When it is not given (None), the call is
    recognised by its `mid_val` tensor: if that is the one the state's last training forward returned, its
    serial is used. Pass 0 to force a re-trace."""
    if _forward_serial is None:
        key = (mid_val.data_ptr(), tuple(mid_val.shape))
        _forward_serial = state.last_forward_serial if getattr(state, "_logged_mid", None) == key else 0
    i, keep = _inputs(state, start_from_first, ray_o, ray_d, vertices, background, means3D, shs, degree, colors_precomp,
                      others_precomp, opacities, scales, scale_modifier, rotations, max_trace_depth, specular_threshold)
    H, W, P, M = i.H, i.W, i.P, i.sh_coeffs
    if mid_val.size(-1) != i.mid_stride:
        raise RuntimeError(f"mid_val must have {i.mid_stride} channels for max_trace_depth={max_trace_depth}")
    dev = means3D.device
    f32 = dict(dtype=torch.float32, device=dev)
    sv = [_cuda_f32(t, n, state) for t, n in ((out_rgb, "out_rgb"), (out_dpt, "out_dpt"), (out_acc, "out_acc"), (out_norm, "out_norm"),
                                         (out_dist, "out_dist"), (out_aux, "out_aux"), (mid_val, "mid_val"))]

    def up(g, shape, name):
        if g is None:
            return torch.zeros(shape, **f32)
        return _cuda_f32(g.expand(shape) if g.shape != torch.Size(shape) else g, name, state)

    ug = [up(dL_drgb, (H, W, 3), "dL_drgb"), up(dL_ddpt, (H, W, 1), "dL_ddpt"), up(dL_dacc, (H, W, 1), "dL_dacc"),
          up(dL_dnorm, (H, W, 3), "dL_dnorm"), up(dL_ddist, (H, W, 1), "dL_ddist"), up(dL_daux, (H, W, 2), "dL_daux")]
    g_ray_o = torch.empty((H, W, 3), **f32)
    g_ray_d = torch.empty((H, W, 3), **f32)
    # The per-surfel gradients a caller can use live in ONE flat buffer (16-byte aligned views), so that a multi-GPU
    # run sums them with a single all-reduce. Gradients nobody receives (of the colour or auxiliary tensor that was
    # not given) are computed as the reference computes them, but kept out of that buffer.
    has_colors, has_others = keep["colors_precomp"].numel() != 0, keep["others_precomp"].numel() != 0
    sizes = [("rot", P * 4, True), ("means", P * 3, True), ("g3d", P * 3, True), ("shs", P * M * 3, True),
             ("colors", P * NUM_CHANNELS, has_colors), ("others", P * AUX_CHANNELS, has_others), ("opac", P, True), ("scales", P * 2, True)]
    offs, total, side_total = {}, 0, 0
    for name, n, shared in sizes:
        if shared:
            offs[name] = (True, total)
            total += (n + 3) // 4 * 4
        else:
            offs[name] = (False, side_total)
            side_total += (n + 3) // 4 * 4
    bucket = torch.empty((total,), **f32)
    side = torch.empty((side_total,), **f32)

    def view(name, n, shape):
        shared, off = offs[name]
        return (bucket if shared else side)[off:off + n].view(shape)

    g_rot = view("rot", P * 4, (P, 4))
    g_means = view("means", P * 3, (P, 3))
    g_g3d = view("g3d", P * 3, (P, 3))
    g_shs = view("shs", P * M * 3, (P, M, 3))
    g_colors = view("colors", P * NUM_CHANNELS, (P, NUM_CHANNELS))
    g_others = view("others", P * AUX_CHANNELS, (P, AUX_CHANNELS))
    g_opac = view("opac", P, (P, 1))
    g_scales = view("scales", P * 2, (P, 2))
    g_g3d_abs = torch.zeros((P, 3), **f32)
    state.grad_bucket = bucket
    g_trans = torch.zeros((P, 9), **f32)
    a = _BwdArgs()
    a.inp = i
    (a.out_rgb, a.out_dpt, a.out_acc, a.out_norm, a.out_dist, a.out_aux, a.mid_val) = [t.data_ptr() for t in sv]
    (a.dL_drgb, a.dL_ddpt, a.dL_dacc, a.dL_dnorm, a.dL_ddist, a.dL_daux) = [t.data_ptr() for t in ug]
    a.dL_dray_o, a.dL_dray_d, a.dL_dmeans3D, a.dL_dgrads3D = g_ray_o.data_ptr(), g_ray_d.data_ptr(), g_means.data_ptr(), g_g3d.data_ptr()
    a.dL_dshs = _ptr(g_shs)
    a.dL_dcolors, a.dL_dothers, a.dL_dopacities = g_colors.data_ptr(), g_others.data_ptr(), g_opac.data_ptr()
    a.dL_dscales, a.dL_drotations = g_scales.data_ptr(), g_rot.data_ptr()
    a.forward_serial = int(_forward_serial or 0)
    if _diag is not None:
        _diag["counters"] = torch.zeros((8,), dtype=torch.int64, device=dev)
        a.counters = _diag["counters"].data_ptr()
    _check(state, lib().dst_backward(state.handle, C.byref(a), _stream(state)))
    if getattr(state, "reduce_gradients", False):
        # multi-GPU: rays are sharded, surfels replicated; the sum over the ranks happens here, before autograd hands
        # the views on, so that leaf gradients behind any chain of activations are the global ones
        import torch.distributed as dist
        torch.cuda.nvtx.range_push("dst_gradient_allreduce")
        dist.all_reduce(bucket, op=dist.ReduceOp.SUM, group=state.process_group)
        torch.cuda.nvtx.range_pop()
    return g_ray_o, g_ray_d, g_means, g_g3d, g_g3d_abs, g_shs, g_colors, g_others, g_opac, g_scales, g_rot, g_trans


def debug_knearest(state, ray_o, ray_d, brute=False, t_cut=None, counters=None):
    """The 16 nearest hits of each ray (one enumeration): (keys (n,16) int64 bit patterns, counts (n,)).
    t_cut: optional (n,) float bound per ray; counters: optional int64 tensor of 8 (nodes -> [2], quads -> [3])."""
    ro, rd = _cuda_f32(ray_o.reshape(-1, 3), "ray_o", state), _cuda_f32(ray_d.reshape(-1, 3), "ray_d", state)
    n = ro.size(0)
    keys = torch.zeros((n, 16), dtype=torch.int64, device=ro.device)
    counts = torch.zeros((n,), dtype=torch.int32, device=ro.device)
    _check(state, lib().dst_debug_knearest(state.handle, ro.data_ptr(), rd.data_ptr(), n, keys.data_ptr(), counts.data_ptr(),
                                           int(brute), _ptr(t_cut), _ptr(counters), _stream(state)))
    return keys, counts


def debug_quad_frames(state):
    """Per-quad plane frames (P, 12) in surfel order, as the build kernels computed them."""
    info = state.info()
    out = torch.zeros((info["surfels"], 12), dtype=torch.float32, device=f"cuda:{state.device}")
    _check(state, lib().dst_debug_quad_frames(state.handle, out.data_ptr(), _stream(state)))
    return out


STATIC_MAX_SURFELS = 65536
STATIC_MAX_RAYS = 65536


def trace_surfels_static(state, training, start_from_first, ray_o, ray_d, vertices, background, means3D, shs, degree,
                         colors_precomp, others_precomp, opacities, scales, scale_modifier, rotations,
                         max_trace_depth, specular_threshold):
    """Forward trace through dst_forward_static: same outputs as trace_surfels, but the library call
    allocates nothing (its scratch is a fixed array inside the library, at most STATIC_MAX_SURFELS
    surfels and STATIC_MAX_RAYS rays per call). For callers that may not allocate device memory at
    the point of the call, e.g. under a memory pool that owns the whole device or inside a loop
    that cannot take an allocation's synchronisation; the output tensors here are still allocated
    by torch before the call.
    Concurrent calls on one device share the array and must be serialised."""
    i, keep = _inputs(state, start_from_first, ray_o, ray_d, vertices, background, means3D, shs, degree, colors_precomp,
                      others_precomp, opacities, scales, scale_modifier, rotations, max_trace_depth, specular_threshold)
    H, W, P = i.H, i.W, i.P
    f32 = dict(dtype=torch.float32, device=means3D.device)
    outs = [torch.empty((H, W, c), **f32) for c in (NUM_CHANNELS, 1, 1, 3, 3, AUX_CHANNELS, i.mid_stride)]
    a_weights = torch.empty((P, 1), **f32) if training else None
    a = _FwdArgs()
    a.inp = i
    a.training = int(bool(training))
    (a.out_rgb, a.out_dpt, a.out_acc, a.out_norm, a.out_dist, a.out_aux, a.mid_val) = [t.data_ptr() for t in outs]
    a.a_weights = _ptr(a_weights)
    _check(state, lib().dst_forward_static(state.handle, C.byref(a), _stream(state)))
    # this entry point keeps no chunk log: a backward of these outputs must re-trace, never reuse the log of an earlier call
    state.last_forward_serial = 0
    state._logged_mid = None
    return (*outs, a_weights)


def _surfel_params(state, means3D, scales, rotations):
    if means3D.dim() != 2 or means3D.size(1) != 3:
        raise RuntimeError("means3D must have dimensions (num_points, 3)")
    P = means3D.size(0)
    if tuple(scales.shape) != (P, 2) or tuple(rotations.shape) != (P, 4):
        raise RuntimeError("scales must have dimensions (num_points, 2) and rotations (num_points, 4)")
    return (_cuda_f32(means3D.detach(), "means3D", state), _cuda_f32(scales.detach(), "scales", state),
            _cuda_f32(rotations.detach(), "rotations", state))


def surfel_quads(state, means3D, scales, rotations, with_triangles=True):
    """GaussianModel.get_triangles (example/utils/gaussian_utils.py:176-210) as one kernel:
    v (4P,3) float32 and f (2P,3) int32 (None unless with_triangles) from the activated surfel
    parameters the tracer also receives. No gradient flows to the parameters (the reference detaches
    the vertices before use, example/render.py:62)."""
    m, s, r = _surfel_params(state, means3D, scales, rotations)
    P = m.size(0)
    v = torch.empty((4 * P, 3), dtype=torch.float32, device=m.device)
    f = torch.empty((2 * P, 3), dtype=torch.int32, device=m.device) if with_triangles else None
    _check(state, lib().dst_surfel_quads(state.handle, m.data_ptr(), s.data_ptr(), r.data_ptr(), P, v.data_ptr(), _ptr(f), _stream(state)))
    return v, f


def build_from_surfels(state, means3D, scales, rotations, rebuild, vertices=None):
    """get_triangles + build_acceleration_structure in one call; returns the vertex tensor (4P,3) to pass
    to the tracer.
    `vertices`, if given, is the (4P,3) buffer to fill (so a training loop can reuse one tensor)."""
    m, s, r = _surfel_params(state, means3D, scales, rotations)
    P = m.size(0)
    if vertices is None:
        vertices = torch.empty((4 * P, 3), dtype=torch.float32, device=m.device)
    elif tuple(vertices.shape) != (4 * P, 3) or vertices.dtype != torch.float32 or not vertices.is_cuda or \
            vertices.device.index != state.device or not vertices.is_contiguous() or vertices.data_ptr() % 16:
        raise RuntimeError("vertices must be a contiguous 16-byte aligned float32 CUDA tensor of shape (4 * num_points, 3)")
    _check(state, lib().dst_build_from_surfels(state.handle, m.data_ptr(), s.data_ptr(), r.data_ptr(), P, vertices.data_ptr(),
                                               int(rebuild), _stream(state)))
    state._keep = (m, s, r, vertices)
    return vertices


def make_camera(K, R, T, correct_pix=True, z_depth=False):
    """dst_camera from 3x3 K, 3x3 R and 3 (or 3x1) T given as tensors, arrays or nested lists."""
    def flat(x, n):
        if isinstance(x, torch.Tensor):
            x = x.detach().cpu()
        t = torch.as_tensor(x, dtype=torch.float32).reshape(-1)
        if t.numel() != n:
            raise RuntimeError(f"camera matrix has {t.numel()} elements, expected {n}")
        return t.tolist()
    c = _Camera()
    c.K[:] = flat(K, 9)
    c.R[:] = flat(R, 9)
    c.T[:] = flat(T, 3)
    c.correct_pix, c.z_depth = int(bool(correct_pix)), int(bool(z_depth))
    return c


def pinhole_rays(state, H, W, K, R, T, correct_pix=True, z_depth=False, device=None):
    """get_rays (example/utils/ray_utils.py:80-136): ray_o, ray_d of shape (H,W,3), or (B,H,W,3) when
    K, R, T carry a leading batch dimension."""
    Kt = torch.as_tensor(K, dtype=torch.float32) if not isinstance(K, torch.Tensor) else K.detach().float().cpu()
    batched = Kt.dim() == 3
    B = Kt.size(0) if batched else 1
    if B > MAX_CAMERAS:
        raise RuntimeError(f"at most {MAX_CAMERAS} cameras per call")
    Rt = torch.as_tensor(R, dtype=torch.float32).reshape(B, 9) if not isinstance(R, torch.Tensor) else R.detach().float().cpu().reshape(B, 9)
    Tt = torch.as_tensor(T, dtype=torch.float32).reshape(B, 3) if not isinstance(T, torch.Tensor) else T.detach().float().cpu().reshape(B, 3)
    Kt = Kt.reshape(B, 9)
    cams = (_Camera * B)()
    for b in range(B):
        cams[b] = make_camera(Kt[b], Rt[b], Tt[b], correct_pix, z_depth)
    dev = torch.device("cuda", state.device) if device is None else torch.device(device)
    if dev.type != "cuda" or (dev.index is not None and dev.index != state.device):
        raise RuntimeError(f"rays can only be generated on cuda:{state.device}, the GPU of this tracer state")
    dev = torch.device("cuda", state.device)
    shape = (B, H, W, 3) if batched else (H, W, 3)
    ray_o = torch.empty(shape, dtype=torch.float32, device=dev)
    ray_d = torch.empty(shape, dtype=torch.float32, device=dev)
    _check(state, lib().dst_pinhole_rays(state.handle, cams, B, int(H), int(W), ray_o.data_ptr(), ray_d.data_ptr(), _stream(state)))
    return ray_o, ray_d
