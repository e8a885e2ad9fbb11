"""TEST INFRASTRUCTURE ONLY: ctypes front end of the CPU oracle.

Two back ends with one interface:
  impl="restatement"  liboracle.so   (oracle/surfel_oracle.cpp, always available after build)
  impl="reference"    _ref/libref_*.so (the reference's own shader sources compiled for the host,
                                       present only where oracle/build.py found the reference tree)
Only tests, the smoke entry point and bench.py's CPU baseline may import this module.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_f = C.POINTER(C.c_float)


class OrcArgs(C.Structure):
    _fields_ = (
        [(n, C.c_int32) for n in ("P", "H", "W", "D", "M", "max_trace_depth", "training", "start_from_first",
                                  "clean", "nthreads", "mid_stride", "hit_cap", "portable_exp", "distortion")]
        + [("specular_threshold", C.c_float), ("scale_modifier", C.c_float)]
        + [(n, C.c_void_p) for n in (
            "ray_o", "ray_d", "vertices", "background", "means3D", "shs", "colors_precomp", "others_precomp",
            "opacities", "scales", "rotations",
            "out_rgb", "out_dpt", "out_acc", "out_norm", "out_dist", "out_aux", "mid_val", "a_weights",
            "dL_drgb", "dL_ddpt", "dL_dacc", "dL_ddist", "dL_dnorm", "dL_daux",
            "dL_dray_o", "dL_dray_d", "dL_dmeans3D", "dL_dgrads3D", "dL_dshs", "dL_dcolors", "dL_dothers",
            "dL_dopacities", "dL_dscales", "dL_drotations",
            "hit_log", "hit_cnt", "fragile", "stats")]
    )


_libs = {}


def _lib(name):
    if name not in _libs:
        path = os.path.join(HERE, name)
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} is missing: run `python oracle/build.py`")
        lib = C.CDLL(path)
        _libs[name] = lib
    return _libs[name]


def restatement_lib():
    lib = _lib("liboracle.so")
    lib.orc_scene_create.restype = C.c_void_p
    lib.orc_scene_create.argtypes = [C.c_void_p, C.c_int, C.c_int]
    lib.orc_scene_destroy.argtypes = [C.c_void_p]
    lib.orc_forward.argtypes = [C.c_void_p, C.POINTER(OrcArgs)]
    lib.orc_backward.argtypes = [C.c_void_p, C.POINTER(OrcArgs)]
    lib.orc_knearest.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.orc_all_hits.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
    lib.orc_quad_records.argtypes = [C.c_void_p, C.c_void_p]
    if not lib.orc_cpu_has_fma():
        raise RuntimeError("the oracle is built with -mfma and this CPU has no FMA unit")
    return lib


def reference_built():
    return all(os.path.exists(os.path.join(HERE, "_ref", f"libref_{w}{m}.so")) for w in ("fwd", "bwd") for m in (1, 2))


def _np(x, dtype=np.float32):
    if x is None:
        return None
    if hasattr(x, "detach"):
        x = x.detach().cpu().numpy()
    return np.ascontiguousarray(x, dtype=dtype)


def _ptr(a):
    return None if a is None else a.ctypes.data


class Scene:
    """Quad frames + host hierarchy of one vertex buffer (4 vertices per surfel)."""

    def __init__(self, vertices, brute=False):
        self.lib = restatement_lib()
        self.v = _np(vertices).reshape(-1, 3)
        assert self.v.shape[0] % 4 == 0
        self.P = self.v.shape[0] // 4
        self.handle = self.lib.orc_scene_create(self.v.ctypes.data, self.P, int(brute))

    def __del__(self):
        try:
            self.lib.orc_scene_destroy(self.handle)
        except Exception:
            pass

    def knearest(self, o, d):
        o, d = _np(o), _np(d)
        keys = np.zeros(16, dtype=np.uint64)
        n = self.lib.orc_knearest(self.handle, o.ctypes.data, d.ctypes.data, keys.ctypes.data)
        return keys[:n]

    def all_hits(self, o, d, cap=65536):
        o, d = _np(o), _np(d)
        keys = np.zeros(cap, dtype=np.uint64)
        n = self.lib.orc_all_hits(self.handle, o.ctypes.data, d.ctypes.data, keys.ctypes.data, cap)
        return keys[:min(n, cap)]

    def quad_records(self):
        out = np.zeros((self.P, 12), dtype=np.float32)
        self.lib.orc_quad_records(self.handle, out.ctypes.data)
        return out


def key_t(keys):
    return (np.asarray(keys, dtype=np.uint64) >> np.uint64(32)).astype(np.uint32).view(np.float32)


def key_pidx(keys):
    return (np.asarray(keys, dtype=np.uint64) & np.uint64(0xFFFFFFFF)).astype(np.int64)


class Oracle:
    """forward()/backward() with the reference's argument meanings (trace_surfels.h:20-83)."""

    def __init__(self, scene: Scene, impl="restatement", clean=True, nthreads=0, hit_cap=0, portable_exp=True, distortion=False):
        self.scene, self.impl, self.clean, self.nthreads, self.hit_cap = scene, impl, clean, nthreads, hit_cap
        self.portable_exp = portable_exp
        self.distortion = distortion       # restatement only: the reference has no distortion code to compare with
        if impl == "reference" and not reference_built():
            raise FileNotFoundError("oracle/_ref is not built (the reference tree was absent at build time)")

    def _mid_stride(self, depth):
        return 16 * max(2, depth + 1)

    def _run(self, backward, a, depth):
        if self.impl == "restatement":
            lib = self.scene.lib
            (lib.orc_backward if backward else lib.orc_forward)(self.scene.handle, C.byref(a))
        else:
            mtd = 1 if depth <= 1 else 2
            lib = _lib(os.path.join("_ref", f"libref_{'bwd' if backward else 'fwd'}{mtd}.so"))
            lib.ref_run.argtypes = [C.c_void_p, C.POINTER(OrcArgs)]
            assert lib.ref_mid_stride() == a.mid_stride
            lib.ref_run(self.scene.handle, C.byref(a))

    def _common(self, w, training):
        """w: dict of array-likes as produced by workloads.make_workload."""
        keep = {}
        a = OrcArgs()
        ray_o = _np(w["ray_o"])
        a.H, a.W = ray_o.shape[0], ray_o.shape[1]
        a.P = self.scene.P
        shs = _np(w.get("shs"))
        a.D = int(w.get("sh_degree", 0))
        a.M = 0 if shs is None else shs.shape[1]
        a.max_trace_depth = int(w.get("max_trace_depth", 0))
        a.training = int(training)
        a.start_from_first = int(w.get("start_from_first", True))
        a.clean = int(self.clean)
        a.nthreads = self.nthreads
        a.portable_exp = int(self.portable_exp)
        a.distortion = int(self.distortion)
        a.mid_stride = self._mid_stride(a.max_trace_depth)
        a.specular_threshold = float(w.get("specular_threshold", 0.0))
        a.scale_modifier = 1.0
        for name, key in (("ray_o", "ray_o"), ("ray_d", "ray_d"), ("background", "bg"), ("means3D", "means3D"),
                          ("shs", "shs"), ("colors_precomp", "colors_precomp"), ("others_precomp", "others_precomp"),
                          ("opacities", "opacities"), ("scales", "scales"), ("rotations", "rotations")):
            arr = _np(w.get(key))
            keep[name] = arr
            setattr(a, name, _ptr(arr))
        a.vertices = self.scene.v.ctypes.data
        return a, keep

    def forward(self, w, training=True):
        a, keep = self._common(w, training)
        R, P = a.H * a.W, a.P
        out = dict(rgb=np.zeros((a.H, a.W, 3), np.float32), dpt=np.zeros((a.H, a.W, 1), np.float32),
                   acc=np.zeros((a.H, a.W, 1), np.float32), norm=np.zeros((a.H, a.W, 3), np.float32),
                   dist=np.zeros((a.H, a.W, 3), np.float32), aux=np.zeros((a.H, a.W, 2), np.float32),
                   mid=np.zeros((a.H, a.W, a.mid_stride), np.float32), wet=np.zeros((P, 1), np.float32),
                   stats=np.zeros(6, np.int64), fragile=np.zeros(R, np.uint8))
        a.out_rgb, a.out_dpt, a.out_acc = _ptr(out["rgb"]), _ptr(out["dpt"]), _ptr(out["acc"])
        a.out_norm, a.out_dist, a.out_aux = _ptr(out["norm"]), _ptr(out["dist"]), _ptr(out["aux"])
        a.mid_val, a.a_weights = _ptr(out["mid"]), _ptr(out["wet"])
        a.stats, a.fragile = _ptr(out["stats"]), _ptr(out["fragile"])
        if self.hit_cap:
            out["hit_log"] = np.full((R, self.hit_cap), -1, np.int32)
            out["hit_cnt"] = np.zeros(R, np.int32)
            a.hit_cap, a.hit_log, a.hit_cnt = self.hit_cap, _ptr(out["hit_log"]), _ptr(out["hit_cnt"])
        self._run(False, a, a.max_trace_depth)
        return out

    def backward(self, w, fwd, grads):
        """fwd: dict returned by forward(); grads: dict with any of rgb, dpt, acc, norm, aux (zeros otherwise)."""
        a, keep = self._common(w, False)
        H, Wd, P = a.H, a.W, a.P
        M = max(a.M, 0)
        for k in ("rgb", "dpt", "acc", "norm", "dist", "aux", "mid"):
            keep["o_" + k] = _np(fwd[k])
        a.out_rgb, a.out_dpt, a.out_acc = _ptr(keep["o_rgb"]), _ptr(keep["o_dpt"]), _ptr(keep["o_acc"])
        a.out_norm, a.out_dist, a.out_aux, a.mid_val = _ptr(keep["o_norm"]), _ptr(keep["o_dist"]), _ptr(keep["o_aux"]), _ptr(keep["o_mid"])
        shapes = dict(rgb=(H, Wd, 3), dpt=(H, Wd, 1), acc=(H, Wd, 1), dist=(H, Wd, 1), norm=(H, Wd, 3), aux=(H, Wd, 2))
        for k, shp in shapes.items():
            g = grads.get(k)
            keep["g_" + k] = np.zeros(shp, np.float32) if g is None else _np(g).reshape(shp)
        a.dL_drgb, a.dL_ddpt, a.dL_dacc = _ptr(keep["g_rgb"]), _ptr(keep["g_dpt"]), _ptr(keep["g_acc"])
        a.dL_ddist, a.dL_dnorm, a.dL_daux = _ptr(keep["g_dist"]), _ptr(keep["g_norm"]), _ptr(keep["g_aux"])
        out = dict(ray_o=np.zeros((H, Wd, 3), np.float32), ray_d=np.zeros((H, Wd, 3), np.float32),
                   means3D=np.zeros((P, 3), np.float32), grads3D=np.zeros((P, 3), np.float32),
                   shs=np.zeros((P, M, 3), np.float32), colors=np.zeros((P, 3), np.float32),
                   others=np.zeros((P, 2), np.float32), opacities=np.zeros((P, 1), np.float32),
                   scales=np.zeros((P, 2), np.float32), rotations=np.zeros((P, 4), np.float32),
                   stats=np.zeros(6, np.int64))
        a.dL_dray_o, a.dL_dray_d = _ptr(out["ray_o"]), _ptr(out["ray_d"])
        a.dL_dmeans3D, a.dL_dgrads3D, a.dL_dshs = _ptr(out["means3D"]), _ptr(out["grads3D"]), _ptr(out["shs"])
        a.dL_dcolors, a.dL_dothers, a.dL_dopacities = _ptr(out["colors"]), _ptr(out["others"]), _ptr(out["opacities"])
        a.dL_dscales, a.dL_drotations = _ptr(out["scales"]), _ptr(out["rotations"])
        a.stats = _ptr(out["stats"])
        self._run(True, a, a.max_trace_depth)
        return out


def surfel_quads(means3D, scales, rotations, with_triangles=True):
    """get_triangles (example/utils/gaussian_utils.py:176-210): (v (4P,3) f32, f (2P,3) i32 or None)."""
    lib = restatement_lib()
    m, s, r = _np(means3D), _np(scales), _np(rotations)
    P = m.shape[0]
    v = np.empty((4 * P, 3), np.float32)
    f = np.empty((2 * P, 3), np.int32) if with_triangles else None
    lib.orc_surfel_quads.argtypes = [C.c_int64] + [C.c_void_p] * 5
    lib.orc_surfel_quads(P, _ptr(m), _ptr(s), _ptr(r), _ptr(v), _ptr(f))
    return v, f


def pinhole_rays(H, W, K, R, T, correct_pix=True, z_depth=False):
    """get_rays (example/utils/ray_utils.py:80-136) for one camera: (ray_o, ray_d), each (H,W,3) f32."""
    lib = restatement_lib()
    K, R, T = _np(K).reshape(9), _np(R).reshape(9), _np(T).reshape(3)
    o = np.empty((H, W, 3), np.float32)
    d = np.empty((H, W, 3), np.float32)
    lib.orc_pinhole_rays.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    lib.orc_pinhole_rays(H, W, _ptr(K), _ptr(R), _ptr(T), int(correct_pix), int(z_depth), _ptr(o), _ptr(d))
    return o, d
