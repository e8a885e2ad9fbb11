/*
 * dst.h - C ABI of the B200-native differentiable surfel tracer.
 *
 * One shared library (libdst_b200.so) replaces the reference's host glue and OptiX programs:
 *   ext.cpp:7-12                         (pybind surface)         -> the functions below
 *   trace_surfels.cpp:36-159             BuildAccelerationStructure -> dst_build
 *   trace_surfels.cpp:162-304            TraceSurfelsCUDA           -> dst_forward
 *   trace_surfels.cpp:307-464            TraceSurfelsBackwardCUDA   -> dst_backward
 *   optix_tracer/optix_wrapper.cpp:166-222  OptiXStateWrapper ctor/dtor -> dst_create / dst_destroy
 *   optix_tracer/common.h:38-60          OPTIX_CHECK / CUDA_CHECK   -> int status + dst_last_error
 *
 * Conventions: every pointer inside an argument block is a DEVICE pointer on the handle's GPU;
 * a null pointer means "absent" exactly where the reference treats an empty tensor as absent
 * (data_ptr() == nullptr, optix_tracer/forward.cu:265, 278). All arrays are contiguous float32
 * unless stated. `stream` is a cudaStream_t passed as void*; all work is enqueued on it and the
 * calls do not synchronise. Functions return 0 on success, a negative DST_E_* code otherwise; no
 * C++ exception crosses this boundary.
 */
#ifndef DST_H_INCLUDED
#define DST_H_INCLUDED

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DST_OK            0
#define DST_E_ARG        -1   /* bad argument (shape, null pointer, size mismatch)            */
#define DST_E_CUDA       -2   /* a CUDA runtime call failed; see dst_last_error               */
#define DST_E_STATE      -3   /* call order (trace or refit before a build)                   */
#define DST_E_NOMEM      -4   /* device allocation failed                                     */

/* bits of the device status word returned by dst_status */
#define DST_STATUS_STACK_OVERFLOW  1u   /* traversal stack exhausted: some hits may be missing */
#define DST_STATUS_CHUNK_LIMIT     2u   /* a ray hit the bound on 16-hit enumerations          */
#define DST_STATUS_LOG_MISMATCH    8u   /* the chunk log ended before the backward of a ray did */

#define DST_MID_CHANNELS 16             /* per-bounce record, optix_tracer/config.h:7-15       */
#ifndef DST_CHUNK
#define DST_CHUNK 16                    /* hits gathered per enumeration, config.h:20          */
#endif

typedef struct dst_handle dst_handle;

/* Creates the tracer state for one GPU (replaces OptiXStateWrapper's constructor,
 * optix_tracer/optix_wrapper.cpp:166-204; no program compilation happens here). */
int dst_create(int device, dst_handle** out);
int dst_destroy(dst_handle* h);
/* Message of the last failure on this handle (h may be NULL for dst_create failures). */
const char* dst_last_error(const dst_handle* h);

/* Build (rebuild != 0) or refit (rebuild == 0) the hierarchy over the surfel quads
 * (trace_surfels.cpp:36-159). vertices: (n_vertices, 3) with n_vertices = 4 * surfels, laid out
 * as example/utils/gaussian_utils.py:176-210 produces them; triangles: (n_triangles, 3) int32,
 * n_triangles = 2 * surfels, accepted for signature compatibility (the device code of the
 * reference hard-codes the 4-vertex/2-triangle layout, optix_tracer/backward.cu:583-602) and may
 * be NULL. A refit keeps the topology of the last build and needs the same surfel count. */
int dst_build(dst_handle* h, const float* vertices, int64_t n_vertices,
              const int32_t* triangles, int64_t n_triangles, int rebuild, void* stream);

typedef struct dst_trace_inputs {
    int32_t H, W;                 /* ray grid: ray index = row * W + col (trace_surfels.cpp:198-200) */
    int32_t P;                    /* surfels                                                      */
    int32_t sh_degree, sh_coeffs; /* D and M of optix_tracer/params.h:33 (M = 0 without SH)       */
    int32_t max_trace_depth;      /* bounces after the primary segment                            */
    int32_t mid_stride;           /* floats of mid_val per ray, >= 16 * (max_trace_depth + 1)     */
    int32_t start_from_first;
    float specular_threshold, scale_modifier;
    const float *ray_o, *ray_d;   /* (H, W, 3)                                                    */
    const float *vertices;        /* (4P, 3), the buffer the hierarchy was built/refitted from    */
    const float *background;      /* (3)                                                          */
    const float *means3D;         /* (P, 3)                                                       */
    const float *shs;             /* (P, M, 3) or NULL                                            */
    const float *colors_precomp;  /* (P, 3) or NULL; exactly one of shs / colors_precomp          */
    const float *others_precomp;  /* (P, 2) specular, roughness; or NULL                          */
    const float *opacities;       /* (P, 1)                                                       */
    const float *scales;          /* (P, 2)                                                       */
    const float *rotations;       /* (P, 4) as (w, x, y, z)                                       */
} dst_trace_inputs;

typedef struct dst_fwd_args {
    dst_trace_inputs in;
    int32_t training;             /* accumulate per-surfel weights into a_weights                 */
    int32_t hit_cap;              /* slots per ray of hit_log                                     */
    /* outputs, all written for every ray (no pre-zeroing needed)                                 */
    float *out_rgb;               /* (H, W, 3)  */
    float *out_dpt;               /* (H, W, 1)  */
    float *out_acc;               /* (H, W, 1)  */
    float *out_norm;              /* (H, W, 3)  */
    float *out_dist;              /* (H, W, 3), zeros as upstream unless DST_OPT_DISTORTION is set  */
    float *out_aux;               /* (H, W, 2)  */
    float *mid_val;               /* (H, W, mid_stride); untraced bounces are zero                */
    float *a_weights;             /* (P, 1), zeroed then accumulated here when training; or NULL  */
    /* optional diagnostics (NULL to disable)                                                     */
    int32_t *hit_log;             /* (H*W, hit_cap) contributing primitive ids in compositing order */
    int32_t *hit_cnt;             /* (H*W) number of contributions over all bounces               */
    unsigned long long *counters; /* [0] ray segments [1] enumerations [2] nodes visited [3] quads tested
                                     [4] slots evaluated [5] contributions; accumulated, not zeroed */
} dst_fwd_args;

typedef struct dst_bwd_args {
    dst_trace_inputs in;
    /* state saved by the forward call */
    const float *out_rgb, *out_dpt, *out_acc, *out_norm, *out_dist, *out_aux, *mid_val;
    /* upstream gradients, shapes of the forward outputs; dL_ddist is (H, W, 1), read only with DST_OPT_DISTORTION */
    const float *dL_drgb, *dL_ddpt, *dL_dacc, *dL_dnorm, *dL_ddist, *dL_daux;
    /* gradient outputs, fully written by the call (no pre-zeroing needed)                        */
    float *dL_dray_o, *dL_dray_d; /* (H, W, 3)                                                    */
    float *dL_dmeans3D;           /* (P, 3)                                                       */
    float *dL_dgrads3D;           /* (P, 3) = sum of dL_dmeans3D * 0.5 * depth                    */
    float *dL_dshs;               /* (P, M, 3) or NULL                                            */
    float *dL_dcolors;            /* (P, 3), accumulated in SH mode too (backward.cu:543)         */
    float *dL_dothers;            /* (P, 2)                                                       */
    float *dL_dopacities;         /* (P, 1)                                                       */
    float *dL_dscales;            /* (P, 2)                                                       */
    float *dL_drotations;         /* (P, 4)                                                       */
    unsigned long long *counters; /* as in dst_fwd_args, or NULL                                  */
    unsigned long long forward_serial; /* value of dst_forward_serial right after the forward call whose saved state
                                     this is, or 0. When it still names the chunk log the handle holds, the backward
                                     re-composites the logged chunks instead of walking the hierarchy again
                                     (same result); otherwise it re-traces.                        */
} dst_bwd_args;

/* Forward trace (trace_surfels.cpp:162-304 + optix_tracer/forward.cu). */
int dst_forward(dst_handle* h, const dst_fwd_args* args, void* stream);
/* Backward trace (trace_surfels.cpp:307-464 + optix_tracer/backward.cu). */
int dst_backward(dst_handle* h, const dst_bwd_args* args, void* stream);

/* Serial number of the last dst_forward call with training != 0 on this handle (0 if none, or if a
 * later dst_build invalidated it). Such a call keeps, in handle-owned memory, the 16-hit chunks
 * every ray composited; dst_backward uses them when dst_bwd_args.forward_serial matches. */
int dst_forward_serial(const dst_handle* h, unsigned long long* serial);

/* Forward trace that allocates nothing. It has no counterpart in the reference.
 *
 * dst_forward grows handle-owned scratch buffers with cudaMalloc whenever a call is larger than
 * any before it. Some callers must not do that: a host application that has given all device
 * memory to its own pool and forbids driver allocations, a plug-in that only ever receives
 * buffers lent by its host, a latency-bound render or control loop that cannot afford the
 * device-wide synchronisation a driver allocation implies.
 * For them this variant keeps its scratch (per-surfel shading records, per-ray state, the ray
 * list) in a fixed array that is part of the loaded library image: about 15 MB of device memory
 * per GPU that loads the library, held until the process exits. Limits: at most
 * DST_STATIC_MAX_SURFELS surfels and DST_STATIC_MAX_RAYS rays per call (a larger call is
 * rejected with DST_E_ARG and an explanatory message; nothing runs). The hierarchy must have been
 * built before with dst_build on the same handle (that call does allocate). Results are those
 * of dst_forward on the same arguments.
 *
 * The first call on each device looks up the array's device address (a one-time set-up that
 * should happen before any stream capture begins); later calls only enqueue kernels and
 * memsets on `stream`. All calls on one device share the one array and it keeps the last call's
 * contents, so two calls whose GPU work overlaps (different streams, or different handles, on the
 * same device) race: serialise them. */
#define DST_STATIC_MAX_SURFELS 65536
#define DST_STATIC_MAX_RAYS    65536
int dst_forward_static(dst_handle* h, const dst_fwd_args* args, void* stream);

/* ---- The two steps next to the tracer in the reference's example pipeline ------------------------ */

/* Quad expansion: GaussianModel.get_triangles (example/utils/gaussian_utils.py:176-210). For each
 * surfel the 4 corners mean +- 3 s_x R[:,0] +- 3 s_y R[:,1] in the order (-,+), (-,-), (+,+), (+,-),
 * with R = build_rotation(rotations) (quaternion (w,x,y,z), normalised inside; :214-249).
 * means3D (P,3), scales (P,2) (already activated, as the tracer receives them), rotations (P,4);
 * vertices (4P,3) out; triangles (2P,3) int32 out or NULL: (4g,4g+1,4g+2), (4g+1,4g+2,4g+3).
 * vertices and rotations 16-byte aligned, scales and triangles 8-byte aligned. */
int dst_surfel_quads(dst_handle* h, const float* means3D, const float* scales, const float* rotations, int64_t n_surfels,
                     float* vertices, int32_t* triangles, void* stream);

/* get_triangles followed by build_acceleration_structure (the pair the reference's training loop
 * runs every iteration, example/render.py:58-63) as one call. `vertices` (4P,3) is an output the
 * caller keeps and later hands to dst_forward / dst_backward. The quads are expanded by one
 * coalesced kernel (36 bytes of parameters in, 48 bytes of vertices out per surfel) and the
 * hierarchy is then built or refitted as dst_build does; with DST_OPT_SINGLE_KERNEL_REFIT the refit
 * expands the quads itself and never reads the vertices back. */
int dst_build_from_surfels(dst_handle* h, const float* means3D, const float* scales, const float* rotations, int64_t n_surfels,
                           float* vertices, int rebuild, void* stream);

/* One pinhole camera as get_rays takes it (example/utils/ray_utils.py:80-136): intrinsics K (3x3),
 * world-to-camera rotation R (3x3), translation T (3), row-major; correct_pix adds 0.5 to the pixel
 * indices (the reference's default); z_depth leaves the directions un-normalised. */
typedef struct dst_camera {
    float K[9];
    float R[9];
    float T[3];
    int32_t correct_pix;
    int32_t z_depth;
} dst_camera;
#define DST_MAX_CAMERAS 64

/* Ray generation: get_rays for n_cameras cameras (host array) of H x W pixels. ray_o, ray_d
 * (n_cameras, H, W, 3) out, device memory. */
int dst_pinhole_rays(dst_handle* h, const dst_camera* cameras, int n_cameras, int H, int W, float* ray_o, float* ray_d, void* stream);

/* dst_forward with the rays of one camera generated in its first kernel instead of loaded:
 * args->in.ray_o / ray_d must point to (H,W,3) buffers, which the call FILLS (the backward and the
 * caller read them afterwards); everything else as dst_forward. Same rays as dst_pinhole_rays. */
int dst_forward_camera(dst_handle* h, const dst_fwd_args* args, const dst_camera* camera, void* stream);

/* Synchronises `stream`, returns and clears the device status word (DST_STATUS_* bits). */
int dst_status(dst_handle* h, uint32_t* flags, void* stream);

/* Number of kernels this handle has enqueued since it was created (build, trace, unpack and neighbouring
 * steps; memsets and copies are not counted). The number of wavefront rounds a trace call enqueues adapts to
 * what earlier calls of the same shape used, so the count per call is not a constant. */
int dst_kernel_launches(const dst_handle* h, int64_t* launches);

/* Hierarchy facts for tests and reports: surfels, internal nodes, bytes held on the device. */
int dst_bvh_info(const dst_handle* h, int64_t* surfels, int64_t* nodes, int64_t* device_bytes);

/* Tunables. DST_OPT_WAVEFRONT_MIN_RAYS: trace calls with at least this many rays run as rounds of
 * separate gather / composite kernels over the live rays (default 32768); smaller calls run one
 * kernel that takes every ray through its whole path (one warp per ray in the forward, one thread per
 * ray in the backward). Results do not depend on the setting. */
#define DST_OPT_WAVEFRONT_MIN_RAYS 1
/* DST_OPT_CHUNK_LOG: 1 (default) keeps the chunk log of training forwards for the backward, 0 disables it. */
#define DST_OPT_CHUNK_LOG 2
/* DST_OPT_CHUNK_LOG_MAX_RECORDS: upper limit on the records (136 bytes each) the chunk log may hold; 0 = only the
 * built-in limit. Rays whose chunks did not fit are re-traced by the backward, with the same result. */
#define DST_OPT_CHUNK_LOG_MAX_RECORDS 3
/* Hint for rays given as (B, h*w, 3) batches of whole images (the reference's "(B, P, 3)" form, __init__.py:246):
 * the image width w. The kernels then walk the rays in 8x4 pixel tiles, as they do for (H, W, 3) rays, so that a
 * warp holds neighbouring pixels. 0 (default): unknown, batched rays are walked in the order given. Results are
 * not affected. */
#define DST_OPT_IMAGE_WIDTH 6
/* dst_build_from_surfels with rebuild == 0: non-zero expands the quads inside the refit kernel (one
 * launch, no re-read of the vertices); zero (default) runs the expansion kernel and then the refit,
 * which is faster on large scenes because the expansion's writes are coalesced. Same results. */
#define DST_OPT_SINGLE_KERNEL_REFIT 4
/* Order of the live-ray lists of the wavefront rounds (results are not affected): 1 (default) keeps every
 * list in the order of the first one (8x4 pixel tiles, tile after tile; within a round, rays on their primary
 * segment before rays on a reflected one), so that the 32 rays a warp of the gather kernel takes keep
 * starting close to each other; 0 appends the survivors warp by warp in the order the warps happen to finish. */
#define DST_OPT_STABLE_LISTS 7
/* Depth distortion, an EXTENSION: the reference declares a distortion output and leaves it at zero with a TODO
 * (optix_tracer/forward.cu:286, backward.cu:526, 570). 0 (default): zeros, as the reference. 1: out_dist[..., 0] is the
 * depth-distortion sum of 2D Gaussian splatting over the contributions of the primary segment,
 * sum_i sum_{j<i} w_i w_j (m_i - m_j)^2 with the mapped depth m = far / (far - near) * (1 - near / depth), near = 0.2 and
 * far = 100 (the constants optix_tracer/auxiliary.h:20-21 defines and never uses); out_dist[..., 1] and [..., 2] hold the
 * moments sum w m and sum w m^2 the backward needs; dst_backward then adds the gradient of dL_ddist to every input
 * gradient. There is nothing upstream to compare this with: it is tested against a CPU restatement of the same formula
 * and against finite differences. */
#define DST_OPT_DISTORTION 8
/* Slices of a large forward call (results are not affected): the ray slots are cut into this many contiguous ranges
 * whose wavefront rounds run on streams of their own, ordered after what the caller's stream held at the call and
 * joined into it before the call returns, so that the slow last batches of one slice's round overlap with the other
 * slices' work. 0 (default): 4 for calls of a million rays and more, fewer for smaller ones; 1: no slicing; at most 8. */
#define DST_OPT_FORWARD_SLICES 9
int dst_set_option(dst_handle* h, int option, int64_t value);

/* Timing of the main kernels with CUDA events on the launching stream. While enabled, every
 * dst_build / dst_forward / dst_backward call records an event pair around its dominant kernel
 * (which = 0: the whole build or refit sequence, 1: the forward trace kernel, 2: the backward trace
 * kernel). dst_profile_read waits for the recorded events, returns the summed milliseconds and the
 * number of launches since the last read, and resets the counters. At most 1024 launches per kind
 * are kept between reads. */
/* on = 2 additionally records a pair around every launch of the gather kernel (which = 3), the kernel that
 * dominates a trace call; meant for a separate measuring pass, since two event records per wavefront round
 * are not free. dst_profile_launches is dst_profile_read with the milliseconds of every launch (the first
 * `cap` of them) instead of their sum. */
int dst_profile_enable(dst_handle* h, int on);
int dst_profile_read(dst_handle* h, int which, float* ms_sum, int32_t* launches);
int dst_profile_launches(dst_handle* h, int which, float* ms, int32_t cap, int32_t* launches);

/* Diagnostics: the DST_CHUNK nearest hits of each ray (one enumeration from the given origins),
 * keys = (bits of t) << 32 | primitive id, ascending; counts = hits found (<= DST_CHUNK).
 * brute != 0 tests every quad instead of walking the hierarchy. t_cut (n_rays floats, or NULL):
 * hits beyond t_cut[r] are ignored for ray r. counters (or NULL): [2] += nodes visited, [3] += quads tested. */
int dst_debug_knearest(dst_handle* h, const float* ray_o, const float* ray_d, int64_t n_rays,
                       unsigned long long* keys, int32_t* counts, int brute, const float* t_cut,
                       unsigned long long* counters, void* stream);
/* Diagnostics: synchronises `stream` and copies the live-list length of every wavefront round of the last trace
 * call (host array of `cap` ints; round r of the call saw counts[r] rays, 0 from the first unused round on; for a
 * forward that ran as slices, the sum over the slices' rounds r). */
int dst_debug_round_counts(dst_handle* h, int32_t* counts, int32_t cap, void* stream);
/* Diagnostics: bandwidth of repeated streaming reads (16-byte loads that bypass L1) of a zeroed scratch buffer of
 * `bytes` bytes, `reps` passes, timed with CUDA events on `stream` after a warming pass; allocates and frees
 * the buffer. With a buffer that fits the L2 cache this is the L2 read bandwidth quoted beside the HBM figure. */
int dst_debug_read_bandwidth(dst_handle* h, int64_t bytes, int reps, float* gb_per_s, void* stream);
/* Diagnostics: the chunk log of the last training forward whose read-back has completed: records it wanted
 * (-1: not known yet), records the log can hold, bytes per record. Rays whose records did not fit are re-traced
 * by the backward. */
int dst_debug_chunk_log(const dst_handle* h, int64_t* records_wanted, int64_t* records_held, int64_t* bytes_per_record);
/* Diagnostics: copies the per-quad plane frames (12 floats each, surfel order) to `out`. */
int dst_debug_quad_frames(dst_handle* h, float* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif
