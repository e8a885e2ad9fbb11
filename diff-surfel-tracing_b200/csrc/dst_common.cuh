// Shared declarations of the B200-native surfel tracer: handle, device-side views, exact-arithmetic helpers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/dst.h"

// ---------------------------------------------------------------------------------------------
// Hierarchy layout in HBM
//   nodes      (P-1) x 64 B : boxes of both children + child links (Aila-Laine style,
//                             one 64-byte fetch = four 16-byte vector loads per visited node)
//   quads      P x 48 B     : plane frame of each quad in LEAF ORDER (three 16-byte loads per test)
//   leaf_gid   P x 4 B      : leaf position -> surfel id
// A child link c >= 0 is an internal node, c < 0 is leaf position ~c.
// ---------------------------------------------------------------------------------------------
struct __align__(16) BvhNode {
    float box[12];      // [0..2] lo of child 0, [3..5] hi of child 0, [6..8] lo of child 1, [9..11] hi of child 1
    int c0, c1;         // topology of the Karras tree: child >= 0 internal node, < 0 leaf position ~c
    int t0, t1;         // links the walk follows: >= 0 internal node, < 0 a run of leaves (DST_LEAF_* below);
                        // a subtree whose boxes overlap so much that testing all its quads is cheaper is one run
};
#define DST_LEAF_FLAG 0x80000000u
#define DST_LEAF_POS_BITS 26
#ifndef DST_LEAF_MAX
#define DST_LEAF_MAX 32               // most quads in one run (five count bits; the gather kernel tests a run with one quad per lane)
#endif
#define DST_HULL_MIN 2                 // runs of at most this many quads are tested exactly by every lane, longer ones go through the hull test first
#define DST_LEAF_LINK(first, count) ((int)(DST_LEAF_FLAG | ((unsigned int)((count) - 1) << DST_LEAF_POS_BITS) | (unsigned int)(first)))
#define DST_LEAF_FIRST(link) ((int)((unsigned int)(link) & ((1u << DST_LEAF_POS_BITS) - 1u)))
#define DST_LEAF_COUNT(link) ((int)(((unsigned int)(link) >> DST_LEAF_POS_BITS) & 31u) + 1)
static_assert(sizeof(BvhNode) == 64, "node must be one 64-byte record");

// header floats: [0..2] scene lo, [3..5] scene hi, [6] largest |coordinate|
#define DST_HDR_FLOATS 8

struct BvhView {
    const float4* nodes;
    const float4* quads;
    const int* leaf_gid;
    const float* header;
    int P;          // surfels = leaves
};

// Per-surfel shading record rebuilt at the start of every trace call (parameters change each
// training step): rows of the tangent frame, the frame origin, opacity and scales, 64 B so that
// one evaluated hit costs two 32-byte sectors instead of four scattered gathers.
//   f4[0] = (R0.xyz, T.x)  f4[1] = (R1.xyz, T.y)  f4[2] = (R2.xyz, opacity)  f4[3] = (sx, sy, 0, 0)
struct SurfelCacheView { const float4* rec; };

// packed per-surfel gradient rows (16-byte aligned so that 4-float vector reductions apply):
//   [0..3] rotation  [4..6] mean  [7] opacity  [8..10] grads3D  [11] -  [12..13] scale  [14..15] others  [16..18] colour  [19] -
#define DST_ARENA_FLOATS 20
#define DST_LOG_MAX_RECORDS (320ll << 20)     // 136 B each: at most 43.5 GB of chunk log

#define DST_MAX_SLICES 8
struct dst_handle {
    int device;
    char err[512];
    bool built;
    int64_t P;            // surfels of the current hierarchy
    int64_t cap;          // surfels the build buffers can hold
    BvhNode* nodes;
    float4* quads;
    int* leaf_gid;
    int* leaf_parent;
    int* node_parent;             // -1 for the root
    int* node_first;              // first leaf position under each node
    int* node_count;              // leaves under each node
    float* child_cost;            // 2 per node: expected walk cost of each child subtree (bottom-up pass)
    unsigned int* arrive;         // per-node arrival counters of the bottom-up pass
    unsigned long long *keys, *keys_alt;
    unsigned int *vals, *vals_alt;
    unsigned int* block_hist;     // 256 x sort blocks
    int64_t hist_cap;
    float* header;                // DST_HDR_FLOATS floats + 8 uint bounds words
    unsigned int* status;         // device status word
    float4* cache; int64_t cache_cap;
    float* arena;  int64_t arena_cap;
    void* cam_dev;      // camera constants of the last ray-generation call
    long long image_width;     // hint: rays given as (B, h*w, 3) are whole images of this width (0: unknown)
    int single_kernel_refit;   // dst_build_from_surfels(rebuild = 0): expand the quads inside the refit kernel
    int sm_count;
    // ray scratch of the wavefront trace (grow-only): state records, enumeration requests, hit buffers, live lists
    void* wf_state; size_t wf_state_bytes; void* wf_req; unsigned long long* wf_kbuf; int* wf_kcnt; int* wf_list[2]; int* wf_counts;
    int* wf_tmp; int* wf_wcnt; int* wf_bcnt;      // order-preserving list hand-over (LiveLists in dst_trace.cuh); wf_bcnt holds both counter sets
    long long wf_cap;
    int distortion;               // 1: the depth-distortion output and its gradient are computed (default 0: zeros, as the reference)
    int stable_lists;             // 1 (default): live lists keep their order from round to round; 0: survivors are appended per warp
    long long wf_min_rays;        // launches with fewer rays skip the wavefront rounds
    // Slices of the forward wavefront: the ray slots of a large call are cut into up to DST_MAX_SLICES contiguous ranges
    // whose rounds run on streams of their own (slice 0 on the caller's), so that the stragglers of one slice's round
    // overlap with the other slices' work. fwd_slices: 0 = chosen from the ray count, n = at most n.
    int fwd_slices, slices_used;
    cudaStream_t slice_stream[DST_MAX_SLICES - 1];
    cudaEvent_t slice_fork, slice_join[DST_MAX_SLICES - 1];
    bool slice_streams_ready;
    // Predicted search bounds of the forward gather (forward_common): device counters {bounded searches, of them failed} of
    // the current call, their pinned read-back, and how many coming calls leave the prediction off after a call in which it
    // failed too often.
    int* bound_stats; int* bound_host; cudaEvent_t bound_event; bool bound_pending; int bound_off_calls;
    // chunk log: the 16-hit chunks every ray composited in the last training forward, chained per ray and segment,
    // so that the backward re-composites them without walking the hierarchy again
    unsigned long long* log_keys; int2* log_hdr; int* log_count; int* log_seg_head; unsigned char* log_ray_ok;
    long long log_cap;            // records
    long long log_rays_cap; int log_seg_stride_cap;
    unsigned long long log_serial;      // serial of the forward call the log belongs to (0 = none)
    unsigned long long serial_counter;
    int log_H, log_W, log_depth;
    int log_enabled;
    long long log_max_records;    // user limit on the log size (0: only the built-in limit)
    int* log_needed_host; cudaEvent_t log_needed_event;     // pinned read-back of the record count of the last forward
    long long log_known_sig, log_known_needed;              // last completed read-back: call shape and records wanted (0: none yet)
    long long log_pending_sig;                              // call shape of the forward whose read-back is in flight
    // pinned read-back of the per-round list lengths of the last wavefront forward, for the round count of the next one
    long long launches;        // kernels enqueued by this handle so far (dst_kernel_launches)
    int* rounds_host; cudaEvent_t rounds_event;
    long long rounds_pending_sig, rounds_known_sig; int rounds_pending_min, rounds_known;
    // optional event timing (dst_profile_enable)
    int profiling;
    cudaEvent_t* ev[4];           // per kind: 2 * DST_PROF_SLOTS events (start, stop pairs); kind 3 = every gather launch (profiling >= 2)
    int ev_n[4];
};
#define DST_PROF_SLOTS 1024
// records the start (which_end = 0) or stop (1) event of the current launch of `kind`; no-op unless profiling
void dst_prof_mark(dst_handle* h, int kind, int which_end, cudaStream_t st);

#define DST_CUDA_TRY(h, expr)                                                                    \
    do {                                                                                         \
        cudaError_t e_ = (expr);                                                                 \
        if (e_ != cudaSuccess) {                                                                 \
            snprintf((h)->err, sizeof((h)->err), "%s failed: %s (%s:%d)", #expr,                 \
                     cudaGetErrorString(e_), __FILE__, __LINE__);                                \
            return DST_E_CUDA;                                                                   \
        }                                                                                        \
    } while (0)

int dst_set_error(dst_handle* h, int code, const char* fmt, ...);
void dst_global_error(const char* msg);

// host entry points implemented in the kernel translation units
int dst_bvh_build_impl(dst_handle* h, const float* v, int64_t P, int rebuild, cudaStream_t st,
                       const float* means = nullptr, const float* scales = nullptr, const float* rotations = nullptr);
int dst_surfel_quads_impl(dst_handle* h, const float* means, const float* scales, const float* rotations, int64_t P,
                          float* vertices, int32_t* triangles, cudaStream_t st);
int dst_pinhole_rays_impl(dst_handle* h, const dst_camera* cams, int n_cameras, int H, int W, float* ray_o, float* ray_d, cudaStream_t st);
int dst_forward_camera_impl(dst_handle* h, const dst_fwd_args* args, const dst_camera* cam, cudaStream_t st);
int dst_forward_impl(dst_handle* h, const dst_fwd_args* a, cudaStream_t st);
int dst_backward_impl(dst_handle* h, const dst_bwd_args* a, cudaStream_t st);
int dst_knearest_impl(dst_handle* h, const float* ro, const float* rd, int64_t n, unsigned long long* keys,
                      int32_t* counts, int brute, const float* t_cut, unsigned long long* counters, cudaStream_t st);
int dst_prepare_cache(dst_handle* h, const dst_trace_inputs* in, cudaStream_t st);
int dst_export_frames_impl(dst_handle* h, float* out, cudaStream_t st);
int dst_ensure_wavefront(dst_handle* h, long long slots, size_t state_bytes);
int dst_ensure_chunk_log(dst_handle* h, long long rays, int segs);
int dst_wavefront_grid(const dst_handle* h, long long slots, int threads, int per_sm);

#ifdef __CUDACC__
// ---------------------------------------------------------------------------------------------
// Exactly rounded binary32 operations. Everything that decides WHICH hits a ray sees (quad frames,
// the ray/quad predicate, depth bookkeeping, the tangent-plane coordinates) is written with these
// so that it is reproducible bit for bit on a CPU: one IEEE round-to-nearest per operation, fused
// multiply-add only where xfma is written.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float xmul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float xadd(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float xsub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float xdiv(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ float xfma(float a, float b, float c) { return __fmaf_rn(a, b, c); }
__device__ __forceinline__ float xsqrt(float a) { return __fsqrt_rn(a); }
__device__ __forceinline__ float xdop(float a, float b, float c, float d) { return xfma(a, b, -xmul(c, d)); }
__device__ __forceinline__ float xdot3(float ax, float ay, float az, float bx, float by, float bz) {
    return xfma(az, bz, xfma(ay, by, xmul(ax, bx)));
}
// the reference's dot(): ((ax*bx + ay*by) + az*bz), each operation rounded
__device__ __forceinline__ float rdot3(float ax, float ay, float az, float bx, float by, float bz) {
    return xadd(xadd(xmul(ax, bx), xmul(ay, by)), xmul(az, bz));
}

struct QuadFrame { float p0x, p0y, p0z, nx, ny, nz, wux, wuy, wuz, wvx, wvy, wvz; };

// Plane frame of the quad (v0, v1, v2, v3): corner p0 = v1, edges eu = v3 - v1, ev = v0 - v1,
// n = eu x ev, wu = (ev x n)/(n.n), wv = (n x eu)/(n.n).
__device__ __forceinline__ QuadFrame make_quad_frame(const float* v) {
    QuadFrame q;
    q.p0x = v[3]; q.p0y = v[4]; q.p0z = v[5];
    const float eux = xsub(v[9], v[3]), euy = xsub(v[10], v[4]), euz = xsub(v[11], v[5]);
    const float evx = xsub(v[0], v[3]), evy = xsub(v[1], v[4]), evz = xsub(v[2], v[5]);
    q.nx = xdop(euy, evz, euz, evy); q.ny = xdop(euz, evx, eux, evz); q.nz = xdop(eux, evy, euy, evx);
    const float nn = xdot3(q.nx, q.ny, q.nz, q.nx, q.ny, q.nz);
    const float cux = xdop(evy, q.nz, evz, q.ny), cuy = xdop(evz, q.nx, evx, q.nz), cuz = xdop(evx, q.ny, evy, q.nx);
    const float cvx = xdop(q.ny, euz, q.nz, euy), cvy = xdop(q.nz, eux, q.nx, euz), cvz = xdop(q.nx, euy, q.ny, eux);
    q.wux = xdiv(cux, nn); q.wuy = xdiv(cuy, nn); q.wuz = xdiv(cuz, nn);
    q.wvx = xdiv(cvx, nn); q.wvy = xdiv(cvy, nn); q.wvz = xdiv(cvz, nn);
    return q;
}

#define DST_T_MAX 1e16f
// mapped depth of the distortion term, m = DST_DIST_K (1 - DST_DIST_NEAR / depth): far / (far - near) with the near = 0.2 and
// far = 100 the reference defines for it (optix_tracer/auxiliary.h:20-21)
#define DST_DIST_NEAR 0.2f
#define DST_DIST_K (100.0f / (100.0f - 0.2f))

// Ray/quad predicate. Returns true with t in [0, 1e16) and tri = 0/1 (which triangle of the quad,
// by the side of the shared diagonal). `tcut`: hits with t > tcut are of no interest to the caller
// (they cannot enter a full k-buffer) and are rejected before the in-quad test.
__device__ __forceinline__ bool ray_quad(const float4 qa, const float4 qb, const float4 qc,
                                         float ox, float oy, float oz, float dx, float dy, float dz,
                                         float tcut, float& t, int& tri) {
    const float rx = xsub(qa.x, ox), ry = xsub(qa.y, oy), rz = xsub(qa.z, oz);
    const float nx = qa.w, ny = qb.x, nz = qb.y;
    const float b = xdot3(nx, ny, nz, dx, dy, dz);
    if (!(b != 0.0f)) return false;
    const float a = xdot3(nx, ny, nz, rx, ry, rz);
    float tt = xdiv(a, b);
    if (!(tt >= 0.0f && tt < DST_T_MAX)) return false;
    if (tt > tcut) return false;
    tt = xadd(tt, 0.0f);
    const float hx = xfma(tt, dx, -rx), hy = xfma(tt, dy, -ry), hz = xfma(tt, dz, -rz);
    const float u = xdot3(qb.z, qb.w, qc.x, hx, hy, hz);
    const float w = xdot3(qc.y, qc.z, qc.w, hx, hy, hz);
    if (!(u >= 0.0f && u <= 1.0f && w >= 0.0f && w <= 1.0f)) return false;
    t = tt; tri = (u > w) ? 1 : 0;
    return true;
}
#endif  // __CUDACC__
