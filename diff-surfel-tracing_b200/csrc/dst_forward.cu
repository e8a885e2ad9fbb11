// Forward trace: replaces the OptiX ray-generation / any-hit programs of optix_tracer/forward.cu
// (__raygen__ot 428-477, tracePath 318-424, traceRay 136-315, __anyhit__ot 481-525) and their
// host launcher TraceSurfelsCUDA (trace_surfels.cpp:162-304).
//
// The per-ray loop of the reference (bounces { enumerations { gather 16 hits; composite } }) is
// flattened into a state machine: a ray's state is {segment, running sums, depth bookkeeping}, and
// one step is "gather the 16 nearest hits from the moved origin" followed by "composite them and
// decide": continue the segment, start the reflected segment, or finish. Large launches run the
// steps as a wavefront (k_enum / k_fwd_shade / k_compact rounds over the list of live rays, state in
// scratch memory); the stragglers and small launches run in k_fwd_tail_warp, one warp per ray to
// completion (k_fwd_tail, one thread per ray, above 32,768 rays).
#include "dst_trace.cuh"
#ifndef DST_ENUM_GRID_PER_SM
#define DST_ENUM_GRID_PER_SM 12       // blocks per SM of the forward gather and composite kernels (persistent: more blocks than fit just start later)
#endif
#ifndef DST_TAIL_DIV
#define DST_TAIL_DIV 64              // the wavefront hands over to the tail kernel when fewer than rays / DST_TAIL_DIV
#define DST_TAIL_MIN 8192            // (but at least DST_TAIL_MIN, at most DST_WARP_TAIL_MAX_RAYS) rays are left
#endif
#ifndef DST_WARP_TAIL_MAX_RAYS
#define DST_WARP_TAIL_MAX_RAYS 32768   // up to this many rays the tail kernel runs one warp per ray
#endif
#ifndef DST_FWD_SLICES
#define DST_FWD_SLICES 4               // slices of a large forward call (see forward_common)
#endif
#ifndef DST_SLICE_MIN_SLOTS
#define DST_SLICE_MIN_SLOTS 262144     // a slice is at least this many ray slots
#endif
#ifndef DST_BOUND_FACTOR
#define DST_BOUND_FACTOR 3.0f         // search bound of a continuing segment in units of the previous chunk's span (0: none)
#endif
#define DST_BOUND_OFF_CALLS 64        // calls without predicted bounds after a call in which they failed too often
#ifndef DST_SHADE_GRID_PER_SM
#define DST_SHADE_GRID_PER_SM 4        // what fits an SM at once at 128 registers (measured: 8 is 2.5 % slower on the headline workload)
#endif
#include <string.h>

namespace {

#ifndef DST_SHADE_THREADS
#define DST_SHADE_THREADS 128
#endif
#ifndef DST_TAIL_THREADS
#define DST_TAIL_THREADS 128
#endif
constexpr int SHADE_THREADS = DST_SHADE_THREADS;
constexpr int TAIL_THREADS = DST_TAIL_THREADS;

// One pinhole camera, reduced on the host to what a pixel needs: inverse intrinsics, rotation,
// translation and centre (example/utils/ray_utils.py:19-60, 107).
struct CamConst { float invK[9], R[9], T[3], c[3]; int correct_pix, z_depth; };

struct FwdParams {
    dst_fwd_args a;
    CamConst cam;       // used when cam_on: rays are generated, not loaded
    int cam_on;
    int dist_on;        // depth-distortion extension (dst.h, DST_OPT_DISTORTION)
    BvhView bvh;
    const float4* cache;
    unsigned int* status;
    int tiled, grid_h, grid_w;      // ray order: 8x4 tiles over a grid_h x grid_w pixel grid, or linear
    long long slot0;                // first ray slot of the slice these lists belong to (see forward_common)
    int* bound_stats;               // {bounded searches issued, of them failed} in this call, or null: no predicted bounds
    float bound_factor;
    // wavefront scratch
    void* state;
    EnumReq* req;
    unsigned long long* kbuf;
    int* kcnt;
    int* list[2];
    int* counts;
    int min_count;
    int rounds;
    LiveLists lv;
    // chunk log (null log_keys: disabled)
    unsigned long long* log_keys; int2* log_hdr; int* log_count; int* log_seg_head; unsigned char* log_ray_ok;
    int log_cap, log_seg_stride;
};

struct __align__(16) FwdState {
    float sox, soy, soz, sdx;
    float sdy, sdz, offset, dpt;
    float T_prev, C0, C1, C2;
    float D, Nx, Ny, Nz;
    float O0, O1, s_prod, rgb0;
    float rgb1, rgb2; int last_gidx, contributor;
    int bounce, chunk, hit_count; float m0;      // m0: mapped depth of the first contribution (distortion extension)
    int log_prev;       // last chunk-log record of the current segment, -1 at a segment start
    float dist, m1, m2; // depth distortion of the primary segment and the two moments of the mapped depth (extension)
};
static_assert(sizeof(FwdState) == 128, "ray state is one 128-byte record");

// Per-surfel shading record: tangent-frame rows from the quaternion exactly as
// quat_to_rotmat_transpose does on an IEEE host (optix_tracer/auxiliary.h:403-429, with rsqrtf
// taken as 1/sqrt), the frame origin T = R p (forward.cu:76), opacity and scales.
__global__ void __launch_bounds__(256) k_prepare_cache(int P, const float* __restrict__ means, const float* __restrict__ scales,
                                                       const float* __restrict__ rots, const float* __restrict__ opac,
                                                       float4* __restrict__ cache) {
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= P) return;
    const float q0 = rots[4 * (size_t)g], q1 = rots[4 * (size_t)g + 1], q2 = rots[4 * (size_t)g + 2], q3 = rots[4 * (size_t)g + 3];
    const float s = xdiv(1.0f, xsqrt(xadd(xadd(xadd(xmul(q3, q3), xmul(q0, q0)), xmul(q1, q1)), xmul(q2, q2))));
    const float w = xmul(q0, s), x = xmul(q1, s), y = xmul(q2, s), z = xmul(q3, s);
    const float r0x = xsub(1.f, xmul(2.f, xadd(xmul(y, y), xmul(z, z))));
    const float r0y = xmul(2.f, xadd(xmul(x, y), xmul(w, z)));
    const float r0z = xmul(2.f, xsub(xmul(x, z), xmul(w, y)));
    const float r1x = xmul(2.f, xsub(xmul(x, y), xmul(w, z)));
    const float r1y = xsub(1.f, xmul(2.f, xadd(xmul(x, x), xmul(z, z))));
    const float r1z = xmul(2.f, xadd(xmul(y, z), xmul(w, x)));
    const float r2x = xmul(2.f, xadd(xmul(x, z), xmul(w, y)));
    const float r2y = xmul(2.f, xsub(xmul(y, z), xmul(w, x)));
    const float r2z = xsub(1.f, xmul(2.f, xadd(xmul(x, x), xmul(y, y))));
    const float px = means[3 * (size_t)g], py = means[3 * (size_t)g + 1], pz = means[3 * (size_t)g + 2];
    const float tx = rdot3(r0x, r0y, r0z, px, py, pz), ty = rdot3(r1x, r1y, r1z, px, py, pz);
    float4* o = cache + 4 * (size_t)g;
    o[0] = make_float4(r0x, r0y, r0z, tx);
    o[1] = make_float4(r1x, r1y, r1z, ty);
    o[2] = make_float4(r2x, r2y, r2z, opac[g]);
    o[3] = make_float4(scales[2 * (size_t)g], scales[2 * (size_t)g + 1], 0.f, 0.f);
}

// a_weights[gidx] += w (optix_tracer/forward.cu:295), aggregated over the lanes of the warp that are here together.
// The lanes of a warp are neighbouring pixels walking their chunks in step, and they composite the same surfels at the
// same time: the lanes that hold the same surfel add their weights up with shuffles and one of them issues the atomic.
// As one atomic per contribution this was 7 of the 16 ms the composite kernel takes on the 3M-surfel 1080p workload
// (the L2 serialises additions to one address, and surfels near the camera are hit by thousands of rays).
__device__ __forceinline__ void add_weight(float* __restrict__ a_weights, int gidx, float w) {
    const unsigned int act = __activemask();
    unsigned int peers = __match_any_sync(act, gidx);
    const int lane = threadIdx.x & 31;
    const int first = __ffs(peers) - 1;
    int rel_pos = __popc(peers << (32 - lane)) * (lane != 0);        // my rank among the peers (a shift by 32 is undefined: lane 0 has rank 0)
    peers &= (0xfffffffeu << lane);                                  // peers above me
    while (__any_sync(act, peers != 0u)) {
        const int next = __ffs(peers);
        const float t = __shfl_sync(act, w, next ? next - 1 : lane);
        if (next) w += t;
        const bool done = rel_pos & 1;                               // my value was taken in this step
        peers &= __ballot_sync(act, !done);
        rel_pos >>= 1;
    }
    if (lane == first) atomicAdd(a_weights + gidx, w);
}

__device__ __forceinline__ void fwd_begin_segment(FwdState& s) {
    s.offset = 0.f; s.dpt = 0.f; s.T_prev = 1.f;
    s.C0 = s.C1 = s.C2 = 0.f; s.D = 0.f; s.Nx = s.Ny = s.Nz = 0.f; s.O0 = s.O1 = 0.f;
    s.last_gidx = -1; s.contributor = 0; s.chunk = 0; s.log_prev = -1;
}

// Ray of pixel (i, j) as get_rays_from_ij computes it (example/utils/ray_utils.py:121-133): camera point
// invK (j+.5, i+.5, 1), world point R^T (camera point - T), direction = world point - centre, divided
// by (norm + 1e-8) unless z_depth. One rounding per operation, sums left to right.
__device__ __forceinline__ void pinhole_ray(const CamConst& c, int i, int j, float* d) {
    const float x = c.correct_pix ? xadd((float)j, 0.5f) : (float)j, y = c.correct_pix ? xadd((float)i, 0.5f) : (float)i;
    float pc[3];
#pragma unroll
    for (int a = 0; a < 3; a++) pc[a] = xsub(xadd(xadd(xmul(c.invK[3 * a], x), xmul(c.invK[3 * a + 1], y)), c.invK[3 * a + 2]), c.T[a]);
#pragma unroll
    for (int a = 0; a < 3; a++) d[a] = xsub(xadd(xadd(xmul(c.R[a], pc[0]), xmul(c.R[3 + a], pc[1])), xmul(c.R[6 + a], pc[2])), c.c[a]);
    if (!c.z_depth) {
        const float n = xadd(xsqrt(xadd(xadd(xmul(d[0], d[0]), xmul(d[1], d[1])), xmul(d[2], d[2]))), 1e-8f);
        d[0] = xdiv(d[0], n); d[1] = xdiv(d[1], n); d[2] = xdiv(d[2], n);
    }
}

// get_rays for a batch of cameras: ray_o, ray_d (B, H, W, 3)
__global__ void __launch_bounds__(256) k_pinhole_rays(const CamConst* __restrict__ cams, int H, int W, long long total,
                                                      float* __restrict__ ray_o, float* __restrict__ ray_d) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long per = (long long)H * W;
    const int b = (int)(idx / per);
    const int pix = (int)(idx - b * per);
    const CamConst& c = cams[b];
    float d[3];
    pinhole_ray(c, pix / W, pix % W, d);
    ray_o[3 * idx] = c.c[0]; ray_o[3 * idx + 1] = c.c[1]; ray_o[3 * idx + 2] = c.c[2];
    ray_d[3 * idx] = d[0]; ray_d[3 * idx + 1] = d[1]; ray_d[3 * idx + 2] = d[2];
}

__device__ __forceinline__ void fwd_init_state(const FwdParams& p, int ray, FwdState& s) {
    const dst_trace_inputs& in = p.a.in;
    if (p.cam_on) {
        // generated here and written to the caller's ray buffers, which the backward reads
        float d[3];
        pinhole_ray(p.cam, ray / in.W, ray % in.W, d);
        s.sox = p.cam.c[0]; s.soy = p.cam.c[1]; s.soz = p.cam.c[2]; s.sdx = d[0]; s.sdy = d[1]; s.sdz = d[2];
        float* o = const_cast<float*>(in.ray_o) + 3 * (size_t)ray;
        float* dd = const_cast<float*>(in.ray_d) + 3 * (size_t)ray;
        o[0] = s.sox; o[1] = s.soy; o[2] = s.soz; dd[0] = s.sdx; dd[1] = s.sdy; dd[2] = s.sdz;
    } else {
        s.sox = __ldg(in.ray_o + 3 * (size_t)ray); s.soy = __ldg(in.ray_o + 3 * (size_t)ray + 1); s.soz = __ldg(in.ray_o + 3 * (size_t)ray + 2);
        s.sdx = __ldg(in.ray_d + 3 * (size_t)ray); s.sdy = __ldg(in.ray_d + 3 * (size_t)ray + 1); s.sdz = __ldg(in.ray_d + 3 * (size_t)ray + 2);
    }
    s.s_prod = 1.f; s.rgb0 = s.rgb1 = s.rgb2 = 0.f; s.bounce = 0; s.hit_count = 0;
    s.dist = s.m1 = s.m2 = 0.f; s.m0 = -1.f;
    fwd_begin_segment(s);
}

// origin of the next enumeration: the segment origin, moved along the ray past the last evaluated hit (forward.cu:303-306)
__device__ __forceinline__ void fwd_request(const FwdState& s, EnumReq& q) {
    if (s.chunk == 0) { q.ox = s.sox; q.oy = s.soy; q.oz = s.soz; }
    else { q.ox = xadd(s.sox, xmul(s.offset, s.sdx)); q.oy = xadd(s.soy, xmul(s.offset, s.sdy)); q.oz = xadd(s.soz, xmul(s.offset, s.sdz)); }
    q.dx = s.sdx; q.dy = s.sdy; q.dz = s.sdz; q.kmax0 = DST_T_MAX; q.pad = s.bounce > 0 ? 1.f : 0.f;       // pad: the ray is on a reflected segment
}

// Composites one gathered chunk (forward.cu:197-306) and, when the segment ends, finishes it
// (forward.cu:309-314, tracePath 378-422). Returns true while the ray needs another enumeration.
// kb: the chunk's keys with stride KS; cnt: how many.
template <bool DIAG, int KS>
__device__ __forceinline__ bool fwd_shade(const FwdParams& p, int ray, FwdState& s, const unsigned long long* kb, int cnt, TraceCounters& tc) {
    const dst_trace_inputs& in = p.a.in;
    const bool use_sh = in.colors_precomp == nullptr;
    const bool has_aux = in.others_precomp != nullptr;
    const int ncoef = (in.sh_degree + 1) * (in.sh_degree + 1);
    const bool sh_aligned = ((in.sh_coeffs * 3) & 3) == 0 && ((reinterpret_cast<uintptr_t>(in.shs) & 15) == 0);
    const float min_depth = s.bounce == 0 ? (in.start_from_first ? 0.2f : 0.0f) : 0.06f;       // forward.cu:353
    const float T_threshold = 0.0001f;
    float sb[16];
    if (use_sh) sh_basis(in.sh_degree, s.sdx, s.sdy, s.sdz, sb);
    if (DIAG) { if (s.chunk == 0) tc.segs++; }
    if (p.log_keys) {
        // keep this chunk for the backward: one record per chunk, chained per segment
        const int idx = atomicAdd(p.log_count, 1);
        if (idx >= 0 && idx < p.log_cap) {
            ulonglong2* dst = reinterpret_cast<ulonglong2*>(p.log_keys + (size_t)idx * DST_CHUNK);
#pragma unroll
            for (int k = 0; k < DST_CHUNK / 2; k++) if (2 * k < cnt) dst[k] = make_ulonglong2(kb[(2 * k) * KS], kb[(2 * k + 1) * KS]);
            p.log_hdr[idx] = make_int2(-1, cnt);
            if (s.log_prev < 0) p.log_seg_head[(size_t)ray * p.log_seg_stride + s.bounce] = idx;
            else p.log_hdr[s.log_prev].x = idx;
            s.log_prev = idx;
        } else p.log_ray_ok[ray] = 0;       // log full: this ray's backward walks the hierarchy again
    }

    float T_next = 1.0f;
    bool stop = false;
    for (int i = 0; i < cnt; i++) {
        const unsigned long long key = kb[i * KS];
        const int pidx = (int)(unsigned int)key;
        const int gidx = pidx >> 1;
        if (gidx == s.last_gidx) continue;                                // forward.cu:207
        if (DIAG) tc.evals++;
        SlotEval e;
        const bool ok = eval_slot(key, s.offset, s.sox, s.soy, s.soz, s.sdx, s.sdy, s.sdz, min_depth, p.cache, gidx, e);
        s.dpt = e.dpt;                                                    // :211 (kept even when the slot is skipped)
        if (!ok) continue;
        const float alpha = e.alpha, nsign = e.nsign;
        const float4 r2 = e.r2;
        T_next = xmul(s.T_prev, xsub(1.0f, alpha));
        if (T_next < T_threshold) { stop = true; break; }
        s.contributor++;
        if (s.contributor > DST_MAX_INTERSECTION) { stop = true; break; }
        s.last_gidx = gidx;
        const float w = xmul(alpha, s.T_prev);
        if (use_sh) {
            float c[48];
            load_sh_row(in.shs + 3 * (size_t)gidx * in.sh_coeffs, 3 * ncoef, sh_aligned, c);
            s.C0 = xadd(s.C0, xmul(w, fmaxf(sh_channel(ncoef, sb, c, 0), 0.f)));
            s.C1 = xadd(s.C1, xmul(w, fmaxf(sh_channel(ncoef, sb, c, 1), 0.f)));
            s.C2 = xadd(s.C2, xmul(w, fmaxf(sh_channel(ncoef, sb, c, 2), 0.f)));
        } else {
            const float* cp = in.colors_precomp + 3 * (size_t)gidx;
            s.C0 = xadd(s.C0, xmul(w, __ldg(cp))); s.C1 = xadd(s.C1, xmul(w, __ldg(cp + 1))); s.C2 = xadd(s.C2, xmul(w, __ldg(cp + 2)));
        }
        if (has_aux) {
            const float2 ax = __ldg(reinterpret_cast<const float2*>(in.others_precomp) + gidx);
            s.O0 = xadd(s.O0, xmul(w, ax.x)); s.O1 = xadd(s.O1, xmul(w, ax.y));
        }
        if (p.dist_on && s.bounce == 0) {
            // Depth distortion of 2D Gaussian splatting over the contributions of the primary segment (an extension: the
            // reference leaves the output at zero, forward.cu:286): sum_i sum_{j<i} w_i w_j (m_i - m_j)^2, accumulated front to
            // back, with the mapped depth m taken relative to the first contribution's (only differences enter).
            const float m_abs = DST_DIST_K * (1.0f - DST_DIST_NEAR / s.dpt);
            if (s.contributor == 1) s.m0 = m_abs;
            const float m = m_abs - s.m0;
            s.dist += w * (m * m * (1.0f - s.T_prev) + s.m2 - 2.0f * m * s.m1);
            s.m1 += m * w; s.m2 += m * m * w;
        }
        s.D = xadd(s.D, xmul(w, s.dpt));
        s.Nx = xadd(s.Nx, xmul(w, nsign * r2.x)); s.Ny = xadd(s.Ny, xmul(w, nsign * r2.y)); s.Nz = xadd(s.Nz, xmul(w, nsign * r2.z));
        s.T_prev = T_next;
        if (p.a.training && p.a.a_weights) add_weight(p.a.a_weights, gidx, w);          // forward.cu:295
        if (DIAG) {
            tc.contribs++;
            if (p.a.hit_log && s.hit_count < p.a.hit_cap) p.a.hit_log[(size_t)ray * p.a.hit_cap + s.hit_count] = pidx;
            s.hit_count++;
        }
    }
    s.chunk++;
    bool seg_done = stop || T_next < T_threshold || cnt < DST_CHUNK || s.contributor > DST_MAX_INTERSECTION;   // :299
    if (!seg_done && s.chunk >= DST_MAX_CHUNKS) { atomicOr(p.status, DST_STATUS_CHUNK_LIMIT); seg_done = true; }
    if (!seg_done) {
        s.offset = (float)((double)s.dpt + 0.00001);                                     // :303
        return true;
    }
    // ---- end of the segment (forward.cu:309-314) ----
    const float bg0 = __ldg(in.background), bg1 = __ldg(in.background + 1), bg2 = __ldg(in.background + 2);
    const float C0 = xadd(s.C0, xmul(s.T_prev, bg0)), C1 = xadd(s.C1, xmul(s.T_prev, bg1)), C2 = xadd(s.C2, xmul(s.T_prev, bg2));
    const float A = xsub(1.0f, s.T_prev);
    // tracePath, forward.cu:378-412
    if (s.bounce == 0) {
        p.a.out_dpt[ray] = s.D; p.a.out_acc[ray] = A;
        p.a.out_norm[3 * (size_t)ray] = s.Nx; p.a.out_norm[3 * (size_t)ray + 1] = s.Ny; p.a.out_norm[3 * (size_t)ray + 2] = s.Nz;
        p.a.out_aux[2 * (size_t)ray] = s.O0; p.a.out_aux[2 * (size_t)ray + 1] = s.O1;
        // zeros as the reference, or (extension) the distortion and the two moments its gradient needs
        p.a.out_dist[3 * (size_t)ray] = s.dist; p.a.out_dist[3 * (size_t)ray + 1] = s.m1; p.a.out_dist[3 * (size_t)ray + 2] = s.m2;
    }
    const float f_this = (s.bounce == in.max_trace_depth) ? 1.0f : xsub(1.0f, s.O0);
    s.rgb0 = xadd(s.rgb0, xmul(xmul(C0, f_this), s.s_prod));
    s.rgb1 = xadd(s.rgb1, xmul(xmul(C1, f_this), s.s_prod));
    s.rgb2 = xadd(s.rgb2, xmul(xmul(C2, f_this), s.s_prod));
    s.s_prod = xmul(s.s_prod, s.O0);
    float* mid = p.a.mid_val + (size_t)ray * in.mid_stride;
    float4* m4 = reinterpret_cast<float4*>(mid + s.bounce * DST_MID_CHANNELS);
    m4[0] = make_float4(s.sox, s.soy, s.soz, s.sdx);
    m4[1] = make_float4(s.sdy, s.sdz, s.D, A);
    m4[2] = make_float4(s.Nx, s.Ny, s.Nz, s.O0);
    m4[3] = make_float4(s.O1, C0, C1, C2);
    const float nlen = xsqrt(rdot3(s.Nx, s.Ny, s.Nz, s.Nx, s.Ny, s.Nz));
    if (nlen == 0.0f || s.O0 <= in.specular_threshold || s.bounce == in.max_trace_depth) {        // :416
        // the ray is finished; bounces that were never traced read as zeros (the reference leaves them uninitialised, forward.cu:446)
        for (int k = (s.bounce + 1) * DST_MID_CHANNELS; k < in.mid_stride; k += 4)
            *reinterpret_cast<float4*>(mid + k) = make_float4(0.f, 0.f, 0.f, 0.f);
        p.a.out_rgb[3 * (size_t)ray] = s.rgb0; p.a.out_rgb[3 * (size_t)ray + 1] = s.rgb1; p.a.out_rgb[3 * (size_t)ray + 2] = s.rgb2;
        if (DIAG && p.a.hit_cnt) p.a.hit_cnt[ray] = s.hit_count;
        return false;
    }
    // reflect about the accumulated normal, restart 0.06 along the new direction (:420-422);
    // exactly rounded, because the bounce ray decides which quads the next segment sees
    const float nx = xdiv(s.Nx, nlen), ny = xdiv(s.Ny, nlen), nz = xdiv(s.Nz, nlen);
    const float k = xmul(2.0f, rdot3(nx, ny, nz, s.sdx, s.sdy, s.sdz));
    const float Ex = xadd(s.sox, xmul(s.D, s.sdx)), Ey = xadd(s.soy, xmul(s.D, s.sdy)), Ez = xadd(s.soz, xmul(s.D, s.sdz));
    s.sdx = xsub(s.sdx, xmul(k, nx)); s.sdy = xsub(s.sdy, xmul(k, ny)); s.sdz = xsub(s.sdz, xmul(k, nz));
    s.sox = xadd(Ex, xmul(0.06f, s.sdx)); s.soy = xadd(Ey, xmul(0.06f, s.sdy)); s.soz = xadd(Ez, xmul(0.06f, s.sdz));
    s.bounce++;
    fwd_begin_segment(s);
    return true;
}

__device__ __forceinline__ void load_state(const void* base, int ray, FwdState& s) {
    const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const FwdState*>(base) + ray);
    float4* dst = reinterpret_cast<float4*>(&s);
#pragma unroll
    for (int i = 0; i < 8; i++) dst[i] = src[i];
}
__device__ __forceinline__ void store_state(void* base, int ray, const FwdState& s) {
    float4* dst = reinterpret_cast<float4*>(reinterpret_cast<FwdState*>(base) + ray);
    const float4* src = reinterpret_cast<const float4*>(&s);
#pragma unroll
    for (int i = 0; i < 8; i++) dst[i] = src[i];
}

__device__ __forceinline__ void flush_counters(unsigned long long* counters, const TraceCounters& tc) {
    if (!counters) return;
    if (tc.segs) atomicAdd(counters + 0, tc.segs);
    if (tc.enums) atomicAdd(counters + 1, tc.enums);
    if (tc.nodes) atomicAdd(counters + 2, tc.nodes);
    if (tc.quads) atomicAdd(counters + 3, tc.quads);
    if (tc.evals) atomicAdd(counters + 4, tc.evals);
    if (tc.contribs) atomicAdd(counters + 5, tc.contribs);
}

// round 0: list of all rays in tile order, initial state and first enumeration request
__global__ void __launch_bounds__(256) k_fwd_init(const __grid_constant__ FwdParams p, long long slots) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= slots) return;
    if (i == 0) p.counts[0] = (int)slots;
    const int ray = ray_of_slot(p.slot0 + i, p.grid_h, p.grid_w, p.tiled != 0);
    p.list[0][i] = ray;
    if (ray < 0) return;
    FwdState s;
    fwd_init_state(p, ray, s);
    if (p.log_keys) {
        p.log_ray_ok[ray] = 1;
        for (int k = 0; k < p.log_seg_stride; k++) p.log_seg_head[(size_t)ray * p.log_seg_stride + k] = -1;
    }
    store_state(p.state, ray, s);
    EnumReq q;
    fwd_request(s, q);
    p.req[ray] = q;
}

template <bool DIAG>
__global__ void __launch_bounds__(SHADE_THREADS) k_fwd_shade(const __grid_constant__ FwdParams p, int round) {
    const int n = p.counts[round];
    if (n < p.min_count) return;
    const int* list = p.list[round & 1];
    int* next_list = p.list[(round + 1) & 1];
    TraceCounters tc = { 0, 0, 0, 0, 0, 0 };
    const int n_pad = (n + 31) & ~31;
    // Predicted bounds stay on while they hold: where rays run out of hits (a sparse scene, the rim of an object) a bounded
    // search that comes back short has to be repeated, and past one failure in twelve the repeats cost more than the bounds save.
    bool bound_on = false;
    if (p.bound_stats && p.bound_factor > 0.0f) {
        const int issued = __ldcg(p.bound_stats), fails = __ldcg(p.bound_stats + 1);
        bound_on = issued < 4096 || fails * 12 < issued;
    }
    for (int i = blockIdx.x * SHADE_THREADS + threadIdx.x; i < n_pad; i += gridDim.x * SHADE_THREADS) {
        const int ray = i < n ? list[i] : -1;
        bool alive = false, bounded = false, failed = false;
        int cls = 0;
        if (ray >= 0) {
            FwdState s;
            load_state(p.state, ray, s);
            const unsigned long long* kb = p.kbuf + (size_t)ray * DST_CHUNK;
            const int cnt = p.kcnt[ray];
            if (cnt < DST_CHUNK && p.req[ray].kmax0 < DST_T_MAX) {
                // The gather searched within a predicted distance (below) and found fewer than 16 hits there: that says nothing
                // about what lies beyond. Nothing is composited; the same request goes out again without a bound.
                p.req[ray].kmax0 = DST_T_MAX;
                alive = true;
                cls = s.bounce > 0;
                failed = true;
                if (DIAG && p.a.counters) atomicAdd(p.a.counters + 1, ~0ull);        // (the counter reports completed enumerations)
            } else {
                alive = fwd_shade<DIAG, 1>(p, ray, s, kb, cnt, tc);
                if (alive) {
                    store_state(p.state, ray, s);
                    EnumReq q;
                    fwd_request(s, q);
                    // A segment that goes on: its next 16 hits are searched within bound_factor times the distance the last 16
                    // spanned (first to last). A walk that knows its bound from the start opens a fifth fewer nodes than one that
                    // learns it from its 16th hit; the spans of consecutive chunks differ by less than that factor for all but
                    // a per cent of the rays of a dense scene, and those search again.
                    if (bound_on && s.chunk > 0 && cnt == DST_CHUNK) {
                        q.kmax0 = fmaxf(p.bound_factor * (hitkey_t(kb[DST_CHUNK - 1]) - hitkey_t(kb[0])), 1e-4f);
                        bounded = true;
                    }
                    p.req[ray] = q;
                    cls = s.bounce > 0;
                }
            }
        }
        if (p.bound_stats) {
            const unsigned int mb = __ballot_sync(0xffffffffu, bounded), mf = __ballot_sync(0xffffffffu, failed);
            if ((threadIdx.x & 31) == 0) { if (mb) atomicAdd(p.bound_stats, __popc(mb)); if (mf) atomicAdd(p.bound_stats + 1, __popc(mf)); }
        }
        if (p.lv.stable) live_out(p.lv, round, i, alive, ray, cls);
        else append_alive(alive, ray, next_list, p.counts + round + 1);
    }
    if (DIAG) flush_counters(p.a.counters, tc);
}

// runs every ray of the first list the wavefront left alone to completion, one thread per ray
template <bool BRUTE, bool DIAG>
__global__ void __launch_bounds__(TAIL_THREADS) k_fwd_tail(const __grid_constant__ FwdParams p) {
    __shared__ unsigned long long kshared[DST_CHUNK * TAIL_THREADS];
    const int round = first_skipped_round(p.counts, p.rounds, p.min_count);
    const int n = p.counts[round];
    const int* list = p.list[round & 1];
    unsigned long long* kb = kshared + threadIdx.x;
    TraceCounters tc = { 0, 0, 0, 0, 0, 0 };
    for (int i = blockIdx.x * TAIL_THREADS + threadIdx.x; i < n; i += gridDim.x * TAIL_THREADS) {
        const int ray = list[i];
        if (ray < 0) continue;
        FwdState s;
        load_state(p.state, ray, s);
        bool alive = true;
        while (alive) {
            EnumReq q;
            fwd_request(s, q);
            const int cnt = knearest<BRUTE, DIAG, TAIL_THREADS>(p.bvh, q.ox, q.oy, q.oz, q.dx, q.dy, q.dz, kb, p.status, tc, q.kmax0);
            if (DIAG) tc.enums++;
            alive = fwd_shade<DIAG, TAIL_THREADS>(p, ray, s, kb, cnt, tc);
        }
    }
    if (DIAG) flush_counters(p.a.counters, tc);
}

// The same for few rays (what the wavefront leaves over, or a small call): one WARP per ray. The warp gathers
// the chunk together (knearest_warp), lane 0 composites it. The longest ray, whose serial work is what this
// kernel takes, gets through its walks several times faster than a thread on its own.
constexpr int WTAIL_THREADS = 128;
template <bool DIAG>
__global__ void __launch_bounds__(WTAIL_THREADS) k_fwd_tail_warp(const __grid_constant__ FwdParams p) {
    __shared__ unsigned long long wstack[WTAIL_THREADS / 32][DST_WARP_STACK];
    __shared__ unsigned long long wkeys[WTAIL_THREADS / 32][DST_CHUNK];
    constexpr unsigned int FULL = 0xffffffffu;
    const int round = first_skipped_round(p.counts, p.rounds, p.min_count);
    const int n = p.counts[round];
    const int* list = p.list[round & 1];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int warps = gridDim.x * (WTAIL_THREADS / 32);
    TraceCounters tc = { 0, 0, 0, 0, 0, 0 };
    for (int i = blockIdx.x * (WTAIL_THREADS / 32) + w; i < n; i += warps) {
        const int ray = list[i];
        if (ray < 0) continue;
        FwdState s;
        if (lane == 0) load_state(p.state, ray, s);
        bool alive = true;
        while (alive) {
            EnumReq q;
            if (lane == 0) fwd_request(s, q);
            const float ox = __shfl_sync(FULL, q.ox, 0), oy = __shfl_sync(FULL, q.oy, 0), oz = __shfl_sync(FULL, q.oz, 0);
            const float dx = __shfl_sync(FULL, q.dx, 0), dy = __shfl_sync(FULL, q.dy, 0), dz = __shfl_sync(FULL, q.dz, 0);
            const float k0 = __shfl_sync(FULL, q.kmax0, 0);
            unsigned long long key;
            const int cnt = knearest_warp<DIAG>(p.bvh, ox, oy, oz, dx, dy, dz, k0, wstack[w], key, p.status, tc);
            if (lane < DST_CHUNK) wkeys[w][lane] = key;
            __syncwarp();
            bool go = false;
            if (lane == 0) {
                if (DIAG) tc.enums++;
                go = fwd_shade<DIAG, 1>(p, ray, s, wkeys[w], cnt, tc);
            }
            alive = __shfl_sync(FULL, go, 0);
        }
    }
    if (DIAG) flush_counters(p.a.counters, tc);
}

// one enumeration per ray, for tests of the hierarchy walk against exhaustive testing
template <bool BRUTE>
__global__ void __launch_bounds__(TAIL_THREADS) k_knearest(BvhView bvh, const float* __restrict__ ro, const float* __restrict__ rd,
                                                           long long n, unsigned long long* keys, int* counts, unsigned int* status,
                                                           const float* __restrict__ t_cut, unsigned long long* counters) {
    __shared__ unsigned long long kbuf[DST_CHUNK * TAIL_THREADS];
    const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n) return;
    unsigned long long* kb = kbuf + threadIdx.x;
    TraceCounters tc = { 0, 0, 0, 0, 0, 0 };
    const int c = knearest<BRUTE, true, TAIL_THREADS>(bvh, ro[3 * r], ro[3 * r + 1], ro[3 * r + 2], rd[3 * r], rd[3 * r + 1], rd[3 * r + 2],
                                                     kb, status, tc, t_cut ? t_cut[r] : DST_T_MAX);
    if (counters) { atomicAdd(counters + 2, tc.nodes); atomicAdd(counters + 3, tc.quads); }
    counts[r] = c;
    for (int i = 0; i < DST_CHUNK; i++) keys[r * DST_CHUNK + i] = i < c ? kb[i * TAIL_THREADS] : 0ull;
}

}  // namespace

BvhView dst_bvh_view(const dst_handle* h) {
    BvhView b;
    b.nodes = reinterpret_cast<const float4*>(h->nodes);
    b.quads = h->quads; b.leaf_gid = h->leaf_gid; b.header = h->header; b.P = (int)h->P;
    return b;
}

int dst_check_inputs(dst_handle* h, const dst_trace_inputs* in) {
    if (!h->built) return dst_set_error(h, DST_E_STATE, "trace requested before build_acceleration_structure");
    if (in->P != h->P) return dst_set_error(h, DST_E_ARG, "means3D has %d surfels but the hierarchy was built over %lld", in->P, (long long)h->P);
    if (in->H <= 0 || in->W <= 0) return dst_set_error(h, DST_E_ARG, "ray grid must be non-empty, got %d x %d", in->H, in->W);
    if ((long long)in->H * in->W > 0x3fffffffll) return dst_set_error(h, DST_E_ARG, "too many rays");
    if (!in->ray_o || !in->ray_d || !in->means3D || !in->opacities || !in->scales || !in->rotations || !in->background || !in->vertices)
        return dst_set_error(h, DST_E_ARG, "a required input pointer is null");
    if ((in->shs == nullptr) == (in->colors_precomp == nullptr))
        return dst_set_error(h, DST_E_ARG, "exactly one of shs / colors_precomp must be given");
    if (in->shs && (in->sh_degree < 0 || in->sh_degree > 3 || (in->sh_degree + 1) * (in->sh_degree + 1) > in->sh_coeffs))
        return dst_set_error(h, DST_E_ARG, "sh_degree %d needs at most 16 and at least (degree+1)^2 coefficients, got %d", in->sh_degree, in->sh_coeffs);
    if (in->max_trace_depth < 0 || in->max_trace_depth > 15) return dst_set_error(h, DST_E_ARG, "max_trace_depth must be in [0, 15]");
    if (in->mid_stride < DST_MID_CHANNELS * (in->max_trace_depth + 1) || (in->mid_stride & 3))
        return dst_set_error(h, DST_E_ARG, "mid_stride must be a multiple of 4 and at least 16 * (max_trace_depth + 1)");
    return DST_OK;
}

int dst_prepare_cache(dst_handle* h, const dst_trace_inputs* in, cudaStream_t st) {
    if (in->P > h->cache_cap) {
        cudaFree(h->cache); h->cache = nullptr; h->cache_cap = 0;
        const int64_t cap = in->P + in->P / 8 + 1024;
        if (cudaMalloc(&h->cache, 64 * cap) != cudaSuccess) { cudaGetLastError(); return dst_set_error(h, DST_E_NOMEM, "surfel cache allocation failed"); }
        h->cache_cap = cap;
    }
    k_prepare_cache<<<(in->P + 255) / 256, 256, 0, st>>>(in->P, in->means3D, in->scales, in->rotations, in->opacities, h->cache);
    h->launches += 1;
    DST_CUDA_TRY(h, cudaGetLastError());
    return DST_OK;
}

// scratch for `slots` list entries / rays of `state_bytes` each (grow-only: a call that needs more slots or a larger
// state record replaces the buffers with ones that hold the larger of the old and the new value of each)
int dst_ensure_wavefront(dst_handle* h, long long slots, size_t state_bytes) {
    if (slots <= h->wf_cap && state_bytes <= h->wf_state_bytes) return DST_OK;
    const long long cap = slots > h->wf_cap ? slots + slots / 16 + 1024 : h->wf_cap;
    const size_t sb = state_bytes > h->wf_state_bytes ? state_bytes : h->wf_state_bytes;
    cudaFree(h->wf_state); cudaFree(h->wf_req); cudaFree(h->wf_kbuf); cudaFree(h->wf_kcnt); cudaFree(h->wf_list[0]); cudaFree(h->wf_list[1]);
    cudaFree(h->wf_counts); cudaFree(h->wf_tmp); cudaFree(h->wf_wcnt); cudaFree(h->wf_bcnt);
    h->wf_state = nullptr; h->wf_req = nullptr; h->wf_kbuf = nullptr; h->wf_kcnt = nullptr; h->wf_list[0] = h->wf_list[1] = nullptr; h->wf_counts = nullptr;
    h->wf_tmp = nullptr; h->wf_wcnt = nullptr; h->wf_bcnt = nullptr;
    h->wf_cap = 0; h->wf_state_bytes = 0;
    cudaError_t e = cudaMalloc(&h->wf_state, sb * (size_t)cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->wf_req, 32 * (size_t)cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->wf_kbuf, 8 * DST_CHUNK * (size_t)cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->wf_kcnt, 4 * (size_t)cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->wf_list[0], 4 * (size_t)cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->wf_list[1], 4 * (size_t)cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->wf_counts, 4 * (size_t)DST_COUNTS_STRIDE * DST_MAX_SLICES);
    if (e == cudaSuccess) e = cudaMalloc(&h->wf_tmp, 4 * (size_t)(cap + 32));
    if (e == cudaSuccess) e = cudaMalloc(&h->wf_wcnt, 4 * (size_t)(cap / 32 + 2));
    if (e == cudaSuccess) e = cudaMalloc(&h->wf_bcnt, 4 * 2 * (size_t)dst_live_blocks(cap));
    if (e != cudaSuccess) { cudaGetLastError(); return dst_set_error(h, DST_E_NOMEM, "ray scratch allocation for %lld rays failed: %s", slots, cudaGetErrorString(e)); }
    h->wf_cap = cap; h->wf_state_bytes = sb;
    return DST_OK;
}

// the list hand-over buffers of the handle as the kernels see them; clears both sets of block counters
int dst_live_lists(dst_handle* h, long long slots, LiveLists* lv, cudaStream_t st) {
    lv->tmp = h->wf_tmp; lv->wcnt = h->wf_wcnt;
    lv->bcnt[0] = h->wf_bcnt; lv->bcnt[1] = h->wf_bcnt + dst_live_blocks(h->wf_cap);
    lv->stable = h->stable_lists;
    if (lv->stable) DST_CUDA_TRY(h, cudaMemsetAsync(h->wf_bcnt, 0, 4 * 2 * (size_t)dst_live_blocks(h->wf_cap), st));
    (void)slots;
    return DST_OK;
}

// Pixel grid the rays are walked over in 8x4 tiles. Rays given as (B, h*w, 3) batches of whole images are
// contiguous image rows, so with the image width known they form one (B*h) x w grid; otherwise the (H, W) of the call.
void dst_slot_grid(const dst_handle* h, const dst_trace_inputs* in, int* gh, int* gw) {
    *gh = in->H; *gw = in->W;
    const long long iw = h->image_width;
    if (iw >= 8 && in->W > iw && in->W % iw == 0 && (long long)in->H * (in->W / iw) < 0x7fffffffll) { *gh = (int)(in->H * (in->W / iw)); *gw = (int)iw; }
}

// one number for "the same kind of call": ray grid, surfel count, bounce limit
long long dst_call_signature(const dst_trace_inputs* in) {
    return ((long long)in->H * 1000003ll + in->W) * 1000033ll + (long long)in->P * 131ll + in->max_trace_depth + 1;
}

// chunk-log buffers for `rays` rays of up to `segs` segments (grow-only)
int dst_ensure_chunk_log(dst_handle* h, long long rays, int segs) {
    // first guess 12 chunks per ray; afterwards what the previous training forward actually needed (read back
    // asynchronously, see dst_forward_impl), within DST_LOG_MAX_RECORDS. Rays beyond the log re-trace in the backward.
    long long want = rays * 12 + 4096;
    if (h->log_needed_host && h->log_needed_event && cudaEventQuery(h->log_needed_event) == cudaSuccess) {
        const long long seen = *h->log_needed_host;
        if (seen > 0 && seen + seen / 8 > want) want = seen + seen / 8;
        if (seen > 0) { h->log_known_needed = seen; h->log_known_sig = h->log_pending_sig; }
    } else cudaGetLastError();
    if (want > DST_LOG_MAX_RECORDS) want = DST_LOG_MAX_RECORDS;
    if (h->log_max_records > 0 && want > h->log_max_records) want = h->log_max_records;
    if (want > h->log_cap || (h->log_max_records > 0 && h->log_cap > h->log_max_records)) {
        cudaFree(h->log_keys); cudaFree(h->log_hdr); h->log_keys = nullptr; h->log_hdr = nullptr; h->log_cap = 0;
        cudaError_t e = cudaMalloc(&h->log_keys, 8 * DST_CHUNK * (size_t)want);
        if (e == cudaSuccess) e = cudaMalloc(&h->log_hdr, sizeof(int2) * (size_t)want);
        if (e != cudaSuccess) { cudaGetLastError(); return dst_set_error(h, DST_E_NOMEM, "chunk log allocation failed: %s", cudaGetErrorString(e)); }
        h->log_cap = want;
    }
    if (!h->log_count && cudaMalloc(&h->log_count, 4) != cudaSuccess) { cudaGetLastError(); return dst_set_error(h, DST_E_NOMEM, "chunk log allocation failed"); }
    if (rays > h->log_rays_cap || segs > h->log_seg_stride_cap) {
        cudaFree(h->log_seg_head); cudaFree(h->log_ray_ok); h->log_seg_head = nullptr; h->log_ray_ok = nullptr;
        const long long rc = rays > h->log_rays_cap ? rays + rays / 16 + 1024 : h->log_rays_cap;
        const int sc = segs > h->log_seg_stride_cap ? segs : h->log_seg_stride_cap;
        cudaError_t e = cudaMalloc(&h->log_seg_head, 4 * (size_t)rc * sc);
        if (e == cudaSuccess) e = cudaMalloc(&h->log_ray_ok, (size_t)rc);
        if (e != cudaSuccess) { cudaGetLastError(); h->log_rays_cap = 0; h->log_seg_stride_cap = 0; return dst_set_error(h, DST_E_NOMEM, "chunk log allocation failed: %s", cudaGetErrorString(e)); }
        h->log_rays_cap = rc; h->log_seg_stride_cap = sc;
    }
    return DST_OK;
}

int dst_wavefront_grid(const dst_handle* h, long long slots, int threads, int per_sm) {
    const long long want = (slots + threads - 1) / threads;
    const long long cap = (long long)h->sm_count * per_sm;
    return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

// Host part of get_rays: torch_inverse_3x3 of K (example/utils/ray_utils.py:19-60; float epsilon
// added to the determinant) and the centre -R^T T (:107), in binary32 with the reference's order.
static void camera_constants(const dst_camera* cam, CamConst* out) {
    const float* K = cam->K; const float* R = cam->R; const float* T = cam->T;
    const float r00 = K[0], r01 = K[1], r02 = K[2], r10 = K[3], r11 = K[4], r12 = K[5], r20 = K[6], r21 = K[7], r22 = K[8];
    volatile float M[9];      // volatile: every product and sum is rounded to binary32 as written
    M[0] = r11 * r22 - r21 * r12;
    M[3] = -r10 * r22 + r20 * r12;
    M[6] = r10 * r21 - r20 * r11;
    M[1] = -r01 * r22 + r21 * r02;
    M[4] = r00 * r22 - r20 * r02;
    M[7] = -r00 * r21 + r20 * r01;
    M[2] = r01 * r12 - r11 * r02;
    M[5] = -r00 * r12 + r10 * r02;
    M[8] = r00 * r11 - r10 * r01;
    volatile float D = r00 * M[0] + r01 * M[3];
    D = D + r02 * M[6];
    const float den = D + 1.1920928955078125e-07f;
    for (int i = 0; i < 9; i++) { out->invK[i] = M[i] / den; out->R[i] = R[i]; }
    for (int a = 0; a < 3; a++) {
        volatile float acc = R[a] * T[0] + R[3 + a] * T[1];
        acc = acc + R[6 + a] * T[2];
        out->c[a] = -acc; out->T[a] = T[a];
    }
    out->correct_pix = cam->correct_pix != 0; out->z_depth = cam->z_depth != 0;
}

int dst_pinhole_rays_impl(dst_handle* h, const dst_camera* cams, int n_cameras, int H, int W, float* ray_o, float* ray_d, cudaStream_t st) {
    if (n_cameras <= 0 || n_cameras > DST_MAX_CAMERAS) return dst_set_error(h, DST_E_ARG, "camera count must be in [1, %d], got %d", DST_MAX_CAMERAS, n_cameras);
    if (H <= 0 || W <= 0) return dst_set_error(h, DST_E_ARG, "ray grid must be non-empty, got %d x %d", H, W);
    const long long total = (long long)n_cameras * H * W;
    if (total > 0x3fffffffll) return dst_set_error(h, DST_E_ARG, "too many rays");
    if (!h->cam_dev) {
        if (cudaMalloc(&h->cam_dev, sizeof(CamConst) * DST_MAX_CAMERAS) != cudaSuccess) { cudaGetLastError(); h->cam_dev = nullptr; return dst_set_error(h, DST_E_NOMEM, "camera buffer allocation failed"); }
    }
    // a copy from pageable host memory has left the source buffer when the call returns, so a local array will do
    CamConst stage[DST_MAX_CAMERAS];
    for (int b = 0; b < n_cameras; b++) camera_constants(cams + b, stage + b);
    DST_CUDA_TRY(h, cudaMemcpyAsync(h->cam_dev, stage, sizeof(CamConst) * n_cameras, cudaMemcpyHostToDevice, st));
    k_pinhole_rays<<<(unsigned int)((total + 255) / 256), 256, 0, st>>>(static_cast<const CamConst*>(h->cam_dev), H, W, total, ray_o, ray_d);
    h->launches += 1;
    DST_CUDA_TRY(h, cudaGetLastError());
    return DST_OK;
}

static int forward_common(dst_handle* h, const dst_fwd_args* a, const dst_camera* cam, cudaStream_t st);
int dst_forward_impl(dst_handle* h, const dst_fwd_args* a, cudaStream_t st) { return forward_common(h, a, nullptr, st); }
int dst_forward_camera_impl(dst_handle* h, const dst_fwd_args* a, const dst_camera* cam, cudaStream_t st) { return forward_common(h, a, cam, st); }

static int forward_common(dst_handle* h, const dst_fwd_args* a, const dst_camera* cam, cudaStream_t st) {
    int rc = dst_check_inputs(h, &a->in);
    if (rc != DST_OK) return rc;
    if (!a->out_rgb || !a->out_dpt || !a->out_acc || !a->out_norm || !a->out_dist || !a->out_aux || !a->mid_val)
        return dst_set_error(h, DST_E_ARG, "a forward output pointer is null");
    if ((reinterpret_cast<uintptr_t>(a->mid_val) & 15) != 0) return dst_set_error(h, DST_E_ARG, "mid_val must be 16-byte aligned");
    FwdParams p;
    p.a = *a; p.bvh = dst_bvh_view(h); p.cache = h->cache; p.status = h->status;
    p.cam_on = cam != nullptr;
    p.slot0 = 0;
    p.dist_on = h->distortion;
    if (cam) camera_constants(cam, &p.cam); else memset(&p.cam, 0, sizeof(p.cam));
    dst_slot_grid(h, &a->in, &p.grid_h, &p.grid_w);
    p.tiled = p.grid_h >= 16;
    const long long slots = slots_of_grid(p.grid_h, p.grid_w, p.tiled != 0);
    rc = dst_ensure_wavefront(h, slots, sizeof(FwdState));
    if (rc != DST_OK) return rc;
    rc = dst_prepare_cache(h, &a->in, st);
    if (rc != DST_OK) return rc;
    p.cache = h->cache;
    if (a->training && a->a_weights) DST_CUDA_TRY(h, cudaMemsetAsync(a->a_weights, 0, 4 * (size_t)a->in.P, st));
    p.state = h->wf_state; p.req = static_cast<EnumReq*>(h->wf_req); p.kbuf = h->wf_kbuf; p.kcnt = h->wf_kcnt;
    p.list[0] = h->wf_list[0]; p.list[1] = h->wf_list[1]; p.counts = h->wf_counts;
    // chunk log for the backward (training calls only)
    p.log_keys = nullptr; p.log_hdr = nullptr; p.log_count = nullptr; p.log_seg_head = nullptr; p.log_ray_ok = nullptr;
    p.log_cap = 0; p.log_seg_stride = a->in.max_trace_depth + 1;
    h->log_serial = 0;
    if (a->training && h->log_enabled) {
        rc = dst_ensure_chunk_log(h, (long long)a->in.H * a->in.W, a->in.max_trace_depth + 1);
        if (rc != DST_OK) return rc;
        p.log_keys = h->log_keys; p.log_hdr = h->log_hdr; p.log_count = h->log_count; p.log_seg_head = h->log_seg_head;
        p.log_ray_ok = h->log_ray_ok; p.log_cap = (int)h->log_cap;
        DST_CUDA_TRY(h, cudaMemsetAsync(h->log_count, 0, 4, st));
        h->log_serial = ++h->serial_counter;
        h->log_H = a->in.H; h->log_W = a->in.W; h->log_depth = a->in.max_trace_depth;
    }
    // small launches go straight to the per-ray kernel; large ones run wavefront rounds until few rays are left
    const bool wave = slots >= h->wf_min_rays;
    p.rounds = wave ? DST_WF_ROUNDS : 0;
    // Slices. A round ends when its slowest batch of 32 rays does, and on scenes with reflections a few batches take ten
    // times the mean: measured on the 3M-surfel 1080p workload the gather kernels kept the SMs 30-80 % busy, the later
    // rounds least. So a large call is cut into contiguous ranges of ray slots whose rounds are independent (own lists,
    // counters and cursors; ray-indexed scratch is shared) and run on streams of their own: while one slice waits for its
    // stragglers the blocks of the next slice's kernel take the free SMs. Per-launch timing (profile level 2) keeps one slice.
    int nsl = 1;
    if (wave && h->profiling < 2) {
        nsl = h->fwd_slices > 0 ? h->fwd_slices : (p.tiled ? DST_FWD_SLICES : 1);       // linear ray lists (a few short rounds) gain nothing
        if (nsl > DST_MAX_SLICES) nsl = DST_MAX_SLICES;
        while (nsl > 1 && slots / nsl < DST_SLICE_MIN_SLOTS) nsl--;
    }
    if (nsl > 1 && !h->slice_streams_ready) {
        bool ok = cudaEventCreateWithFlags(&h->slice_fork, cudaEventDisableTiming) == cudaSuccess;
        for (int g = 0; g < DST_MAX_SLICES - 1 && ok; g++) {
            ok = cudaStreamCreateWithFlags(&h->slice_stream[g], cudaStreamNonBlocking) == cudaSuccess &&
                 cudaEventCreateWithFlags(&h->slice_join[g], cudaEventDisableTiming) == cudaSuccess;
        }
        if (!ok) { cudaGetLastError(); return dst_set_error(h, DST_E_CUDA, "creating the streams of the forward slices failed"); }
        h->slice_streams_ready = true;
    }
    h->slices_used = nsl;
    long long hand_over = slots / DST_TAIL_DIV > DST_TAIL_MIN ? slots / DST_TAIL_DIV : DST_TAIL_MIN;
    if (hand_over > DST_WARP_TAIL_MAX_RAYS) hand_over = DST_WARP_TAIL_MAX_RAYS;       // what the warp-per-ray tail takes
    if (nsl > 1) { hand_over /= nsl; if (hand_over < 1024) hand_over = 1024; }
    p.min_count = wave ? (int)hand_over : 1;
    // Rounds are enqueued without knowing how many the rays will need; a round on an exhausted list costs a few
    // microseconds per kernel. The list lengths of the previous forward of the same shape (read back without
    // synchronising) say how many were used: enqueue that many plus a margin. Scheduling only: rays that need more
    // are finished by the tail kernel, and the next call sees the longer history.
    const long long sig = dst_call_signature(&a->in) * 16 + nsl;
    if (wave) {
        if (h->rounds_host && h->rounds_event && cudaEventQuery(h->rounds_event) == cudaSuccess) {
            int used = 0;
            for (int g = 0; g < DST_MAX_SLICES; g++) {
                int u = 0;
                while (u < DST_WF_ROUNDS && h->rounds_host[g * DST_COUNTS_STRIDE + u] >= h->rounds_pending_min) u++;
                if (u > used) used = u;
            }
            h->rounds_known = used; h->rounds_known_sig = h->rounds_pending_sig;
        } else cudaGetLastError();
        if (h->rounds_known > 0 && h->rounds_known_sig == sig) {
            const int want = h->rounds_known + (h->rounds_known / 2 > 4 ? h->rounds_known / 2 : 4);
            p.rounds = want < DST_WF_ROUNDS ? want : DST_WF_ROUNDS;
        }
    }
    const bool diag = a->hit_log || a->hit_cnt || a->counters;
    // predicted search bounds: on unless the last call that used them saw them fail too often (read back without synchronising)
    p.bound_stats = nullptr; p.bound_factor = 0.0f;
    if (wave && DST_BOUND_FACTOR > 0.0f) {
        if (!h->bound_stats) {
            if (cudaMalloc(&h->bound_stats, 8) != cudaSuccess) { cudaGetLastError(); h->bound_stats = nullptr; }
            if (h->bound_stats && cudaMallocHost(&h->bound_host, 8) != cudaSuccess) { cudaGetLastError(); h->bound_host = nullptr; }
            if (h->bound_host && cudaEventCreateWithFlags(&h->bound_event, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); h->bound_event = nullptr; }
        }
        if (h->bound_pending && h->bound_event && cudaEventQuery(h->bound_event) == cudaSuccess) {
            h->bound_pending = false;
            if (h->bound_host[0] >= 4096 && (long long)h->bound_host[1] * 12 >= h->bound_host[0]) h->bound_off_calls = DST_BOUND_OFF_CALLS;
        } else cudaGetLastError();
        if (h->bound_off_calls > 0) h->bound_off_calls--;
        else if (h->bound_stats) { p.bound_stats = h->bound_stats; p.bound_factor = DST_BOUND_FACTOR; DST_CUDA_TRY(h, cudaMemsetAsync(h->bound_stats, 0, 8, st)); }
    }
    DST_CUDA_TRY(h, cudaMemsetAsync(h->wf_counts, 0, 4 * (size_t)DST_COUNTS_STRIDE * DST_MAX_SLICES, st));
    rc = dst_live_lists(h, slots, &p.lv, st);
    if (rc != DST_OK) return rc;
    dst_prof_mark(h, 1, 0, st);
    // the slices: ranges of whole list blocks, each with its own view of the lists and counters
    FwdParams ps[DST_MAX_SLICES];
    cudaStream_t sst[DST_MAX_SLICES];
    long long sslots[DST_MAX_SLICES];
    {
        const long long blocks_total = (slots + DST_LIVE_BLOCK - 1) / DST_LIVE_BLOCK;
        for (int g = 0; g < nsl; g++) {
            const long long b0 = blocks_total * g / nsl, b1 = blocks_total * (g + 1) / nsl;
            const long long s0 = b0 * DST_LIVE_BLOCK, s1 = g == nsl - 1 ? slots : b1 * DST_LIVE_BLOCK;
            FwdParams& q = ps[g];
            q = p;
            q.slot0 = s0;
            q.list[0] = p.list[0] + s0; q.list[1] = p.list[1] + s0;
            q.counts = p.counts + (size_t)g * DST_COUNTS_STRIDE;
            q.lv.tmp = p.lv.tmp + s0; q.lv.wcnt = p.lv.wcnt + s0 / 32;
            q.lv.bcnt[0] = p.lv.bcnt[0] + b0; q.lv.bcnt[1] = p.lv.bcnt[1] + b0;
            sslots[g] = s1 - s0;
            sst[g] = g == 0 ? st : h->slice_stream[g - 1];
        }
    }
    if (nsl > 1) {
        DST_CUDA_TRY(h, cudaEventRecord(h->slice_fork, st));
        for (int g = 1; g < nsl; g++) DST_CUDA_TRY(h, cudaStreamWaitEvent(sst[g], h->slice_fork, 0));
    }
    for (int g = 0; g < nsl; g++) k_fwd_init<<<(unsigned int)((sslots[g] + 255) / 256), 256, 0, sst[g]>>>(ps[g], sslots[g]);
    for (int r = 0; r < p.rounds; r++) {
        for (int g = 0; g < nsl; g++) {
            const FwdParams& q = ps[g];
            const int g_enum = dst_wavefront_grid(h, sslots[g], ENUM_THREADS, DST_ENUM_GRID_PER_SM), g_shade = dst_wavefront_grid(h, sslots[g], SHADE_THREADS, DST_SHADE_GRID_PER_SM);
            const int g_compact = (int)((sslots[g] + DST_LIVE_BLOCK - 1) / DST_LIVE_BLOCK);
            dst_prof_mark(h, 3, 0, sst[g]);
            launch_gather(diag, g_enum, sst[g], q.bvh, q.req, q.list[r & 1], q.counts + r, q.counts + DST_WF_ROUNDS + 2 + r, q.min_count, q.kbuf, q.kcnt,
                          q.status, a->counters, r + 1, q.tiled != 0);
            dst_prof_mark(h, 3, 1, sst[g]);
            if (diag) k_fwd_shade<true><<<g_shade, SHADE_THREADS, 0, sst[g]>>>(q, r);
            else k_fwd_shade<false><<<g_shade, SHADE_THREADS, 0, sst[g]>>>(q, r);
            if (q.lv.stable) k_compact<<<g_compact, 256, 0, sst[g]>>>(q.lv, q.counts + r, q.counts + r + 1, q.min_count, q.list[(r + 1) & 1], r);
        }
    }
    // few rays left (or a small call): one warp per ray; many: one thread per ray
    for (int g = 0; g < nsl; g++) {
        const FwdParams& q = ps[g];
        const long long tail_rays = wave ? q.min_count : sslots[g];
        if (tail_rays <= DST_WARP_TAIL_MAX_RAYS) {
            const int g_wtail = dst_wavefront_grid(h, tail_rays * 32, WTAIL_THREADS, 16);
            if (diag) k_fwd_tail_warp<true><<<g_wtail, WTAIL_THREADS, 0, sst[g]>>>(q);
            else k_fwd_tail_warp<false><<<g_wtail, WTAIL_THREADS, 0, sst[g]>>>(q);
        } else {
            const int g_tail = dst_wavefront_grid(h, tail_rays, TAIL_THREADS, 8);
            if (diag) k_fwd_tail<false, true><<<g_tail, TAIL_THREADS, 0, sst[g]>>>(q);
            else k_fwd_tail<false, false><<<g_tail, TAIL_THREADS, 0, sst[g]>>>(q);
        }
    }
    for (int g = 1; g < nsl; g++) {
        DST_CUDA_TRY(h, cudaEventRecord(h->slice_join[g - 1], sst[g]));
        DST_CUDA_TRY(h, cudaStreamWaitEvent(st, h->slice_join[g - 1], 0));
    }
    dst_prof_mark(h, 1, 1, st);
    DST_CUDA_TRY(h, cudaGetLastError());
    h->launches += (long long)nsl * (2 + (p.lv.stable ? 3 : 2) * p.rounds);       // per slice: ray init, the rounds, tail
    if (wave) {
        if (!h->rounds_host) {
            if (cudaMallocHost(&h->rounds_host, 4 * (size_t)DST_COUNTS_STRIDE * DST_MAX_SLICES) != cudaSuccess) { cudaGetLastError(); h->rounds_host = nullptr; }
            if (h->rounds_host && cudaEventCreateWithFlags(&h->rounds_event, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); h->rounds_event = nullptr; }
        }
        if (h->rounds_host && h->rounds_event && cudaEventQuery(h->rounds_event) != cudaErrorNotReady) {
            // (a copy still in flight keeps the buffer: its event decides when the buffer may be read)
            cudaGetLastError();
            cudaMemcpyAsync(h->rounds_host, h->wf_counts, 4 * (size_t)DST_COUNTS_STRIDE * DST_MAX_SLICES, cudaMemcpyDeviceToHost, st);
            cudaEventRecord(h->rounds_event, st);
            h->rounds_pending_sig = sig; h->rounds_pending_min = p.min_count;
        }
    }
    if (p.bound_stats && h->bound_host && h->bound_event && !h->bound_pending) {
        cudaMemcpyAsync(h->bound_host, h->bound_stats, 8, cudaMemcpyDeviceToHost, st);
        cudaEventRecord(h->bound_event, st);
        h->bound_pending = true;
    }
    if (p.log_keys) {
        // how many records this call wanted, for sizing the log of the next one (no synchronisation here)
        if (!h->log_needed_host) {
            if (cudaMallocHost(&h->log_needed_host, sizeof(int)) != cudaSuccess) { cudaGetLastError(); h->log_needed_host = nullptr; }
            else *h->log_needed_host = 0;
            if (h->log_needed_host && cudaEventCreateWithFlags(&h->log_needed_event, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); h->log_needed_event = nullptr; }
        }
        if (h->log_needed_host && h->log_needed_event) {
            cudaMemcpyAsync(h->log_needed_host, h->log_count, sizeof(int), cudaMemcpyDeviceToHost, st);
            cudaEventRecord(h->log_needed_event, st);
            h->log_pending_sig = dst_call_signature(&a->in);      // (the backward compares with the plain shape: slices are the forward's business)
        }
    }
    return DST_OK;
}

int dst_knearest_impl(dst_handle* h, const float* ro, const float* rd, int64_t n, unsigned long long* keys, int32_t* counts,
                      int brute, const float* t_cut, unsigned long long* counters, cudaStream_t st) {
    if (!h->built) return dst_set_error(h, DST_E_STATE, "no hierarchy has been built");
    if (n <= 0) return DST_OK;
    const unsigned int blocks = (unsigned int)((n + TAIL_THREADS - 1) / TAIL_THREADS);
    if (brute) k_knearest<true><<<blocks, TAIL_THREADS, 0, st>>>(dst_bvh_view(h), ro, rd, n, keys, counts, h->status, t_cut, counters);
    else k_knearest<false><<<blocks, TAIL_THREADS, 0, st>>>(dst_bvh_view(h), ro, rd, n, keys, counts, h->status, t_cut, counters);
    DST_CUDA_TRY(h, cudaGetLastError());
    return DST_OK;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free forward trace (dst_forward_static, include/dst.h): the per-call scratch lives in
// a file-scope device array instead of handle-owned cudaMalloc buffers.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr long long ST_SLOTS = 98304;                        // list entries: rays rounded up to whole 8x4 tiles
constexpr size_t ST_OFF_CACHE = 0;                                                        // 64 B per surfel
constexpr size_t ST_OFF_STATE = ST_OFF_CACHE + 64ull * DST_STATIC_MAX_SURFELS;            // 128 B per ray
constexpr size_t ST_OFF_REQ = ST_OFF_STATE + sizeof(FwdState) * (size_t)DST_STATIC_MAX_RAYS;  // 32 B per ray
constexpr size_t ST_OFF_LIST = ST_OFF_REQ + sizeof(EnumReq) * (size_t)DST_STATIC_MAX_RAYS;    // 4 B per slot
constexpr size_t ST_OFF_COUNTS = ST_OFF_LIST + 4ull * ST_SLOTS;                               // round counters
constexpr size_t ST_BYTES = ST_OFF_COUNTS + 4ull * 2 * (DST_WF_ROUNDS + 2) + 256;
}
// In host code this name is only a handle for cudaGetSymbolAddress; kernels get the looked-up device pointer.
static __device__ __align__(256) unsigned char g_static_scratch[ST_BYTES];
static unsigned char* g_static_ptr[64] = { nullptr };        // per device, filled on the first call there

extern "C" int dst_forward_static(dst_handle* h, const dst_fwd_args* a, void* stream) {
    if (!h) return DST_E_ARG;
    if (!a) return dst_set_error(h, DST_E_ARG, "args is null");
    cudaStream_t st = (cudaStream_t)stream;
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess) return dst_set_error(h, DST_E_CUDA, "cudaGetDevice failed");
    if (prev != h->device && cudaSetDevice(h->device) != cudaSuccess) return dst_set_error(h, DST_E_CUDA, "cudaSetDevice(%d) failed", h->device);
    struct Restore { int prev, cur; ~Restore() { if (prev >= 0 && prev != cur) cudaSetDevice(prev); } } restore{ prev, h->device };

    int rc = dst_check_inputs(h, &a->in);
    if (rc != DST_OK) return rc;
    if (!a->out_rgb || !a->out_dpt || !a->out_acc || !a->out_norm || !a->out_dist || !a->out_aux || !a->mid_val)
        return dst_set_error(h, DST_E_ARG, "a forward output pointer is null");
    if ((reinterpret_cast<uintptr_t>(a->mid_val) & 15) != 0) return dst_set_error(h, DST_E_ARG, "mid_val must be 16-byte aligned");
    const long long R = (long long)a->in.H * a->in.W;
    if (a->in.P > DST_STATIC_MAX_SURFELS)
        return dst_set_error(h, DST_E_ARG, "dst_forward_static handles at most %d surfels per call, got %d (use dst_forward)", DST_STATIC_MAX_SURFELS, a->in.P);
    if (R > DST_STATIC_MAX_RAYS)
        return dst_set_error(h, DST_E_ARG, "dst_forward_static handles at most %d rays per call, got %lld (use dst_forward)", DST_STATIC_MAX_RAYS, R);
    // 8x4 pixel tiles round the grid up; a narrow grid whose tiled form would not fit the list is walked in ray order instead
    const bool tiled = a->in.H >= 16 && slots_of_grid(a->in.H, a->in.W, true) <= ST_SLOTS;
    const long long slots = slots_of_grid(a->in.H, a->in.W, tiled);
    if (h->device < 0 || h->device >= 64) return dst_set_error(h, DST_E_ARG, "device index %d out of range", h->device);
    // one-time set-up per device, with that device current: the device address of the scratch array
    if (!g_static_ptr[h->device]) {
        unsigned char* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr) {
            cudaGetLastError();
            return dst_set_error(h, DST_E_CUDA, "cudaGetSymbolAddress for the static scratch failed: %s", cudaGetErrorString(e));
        }
        g_static_ptr[h->device] = ptr;
    }
    unsigned char* base = g_static_ptr[h->device];

    FwdParams p;
    p.a = *a; p.bvh = dst_bvh_view(h); p.status = h->status; p.tiled = tiled; p.grid_h = a->in.H; p.grid_w = a->in.W;
    p.cam_on = 0; memset(&p.cam, 0, sizeof(p.cam));
    p.slot0 = 0; p.bound_stats = nullptr; p.bound_factor = 0.0f;
    p.dist_on = h->distortion;
    p.cache = reinterpret_cast<const float4*>(base + ST_OFF_CACHE);
    p.state = base + ST_OFF_STATE;
    p.req = reinterpret_cast<EnumReq*>(base + ST_OFF_REQ);
    p.kbuf = nullptr; p.kcnt = nullptr;                          // only the per-ray kernel runs: no round buffers
    p.list[0] = reinterpret_cast<int*>(base + ST_OFF_LIST); p.list[1] = p.list[0];
    p.counts = reinterpret_cast<int*>(base + ST_OFF_COUNTS);
    p.rounds = 0; p.min_count = 1;
    memset(&p.lv, 0, sizeof(p.lv));                              // no rounds, no list hand-over
    p.log_keys = nullptr; p.log_hdr = nullptr; p.log_count = nullptr; p.log_seg_head = nullptr; p.log_ray_ok = nullptr;
    p.log_cap = 0; p.log_seg_stride = 0;
    // the array keeps the previous call's contents: the round counters must start at zero, everything else is rewritten
    DST_CUDA_TRY(h, cudaMemsetAsync(p.counts, 0, 4 * 2 * (DST_WF_ROUNDS + 2), st));
    if (a->training && a->a_weights) DST_CUDA_TRY(h, cudaMemsetAsync(a->a_weights, 0, 4 * (size_t)a->in.P, st));
    k_prepare_cache<<<(a->in.P + 255) / 256, 256, 0, st>>>(a->in.P, a->in.means3D, a->in.scales, a->in.rotations, a->in.opacities,
                                                             reinterpret_cast<float4*>(base + ST_OFF_CACHE));
    k_fwd_init<<<(unsigned int)((slots + 255) / 256), 256, 0, st>>>(p, slots);
    const bool diag = a->hit_log || a->hit_cnt || a->counters;
    if (slots <= DST_WARP_TAIL_MAX_RAYS) {
        const int g_wtail = dst_wavefront_grid(h, slots * 32, WTAIL_THREADS, 16);
        if (diag) k_fwd_tail_warp<true><<<g_wtail, WTAIL_THREADS, 0, st>>>(p);
        else k_fwd_tail_warp<false><<<g_wtail, WTAIL_THREADS, 0, st>>>(p);
    } else {
        const int g_tail = dst_wavefront_grid(h, slots, TAIL_THREADS, 8);
        if (diag) k_fwd_tail<false, true><<<g_tail, TAIL_THREADS, 0, st>>>(p);
        else k_fwd_tail<false, false><<<g_tail, TAIL_THREADS, 0, st>>>(p);
    }
    DST_CUDA_TRY(h, cudaGetLastError());
    h->launches += 3;
    return DST_OK;
}

#ifdef DST_ROUND_STATS
// build-time diagnostic (see dst_trace.cuh): copies and clears the per-round gather statistics of this translation unit
extern "C" int dst_debug_round_stats(unsigned long long* out) {
    if (cudaMemcpyFromSymbol(out, g_round_stats, sizeof(unsigned long long) * 64 * 8) != cudaSuccess) return DST_E_CUDA;
    static unsigned long long zero[64 * 8];
    return cudaMemcpyToSymbol(g_round_stats, zero, sizeof(zero)) == cudaSuccess ? DST_OK : DST_E_CUDA;
}
#endif
