// Backward trace: replaces optix_tracer/backward.cu (__raygen__ot 857-928, tracePath 658-853,
// traceRay 332-655 and its helpers) and the host launcher TraceSurfelsBackwardCUDA
// (trace_surfels.cpp:307-464).
//
// Bounces are visited last to first; each segment is re-traced front to back with the forward
// kernel's exact decision code (eval_slot), and every contributing hit adds its gradients. As in
// the forward trace the per-ray loop is a state machine run as wavefront rounds (k_enum gathers,
// k_bwd_shade composites and differentiates) with a one-thread-per-ray tail. Per-surfel gradients go to a packed arena of 16-byte aligned rows with 4-float
// vector reductions (5 per contribution instead of 18 scalar atomics; SH rows 12 instead of 48),
// and are unpacked into the caller's tensors by a streaming kernel afterwards.
#include "dst_trace.cuh"

namespace {

#ifndef DST_BWD_THREADS
#define DST_BWD_THREADS 128
#endif
constexpr int BWD_THREADS = DST_BWD_THREADS;
#ifndef DST_BWD_LOGGED_BLOCKS
#define DST_BWD_LOGGED_BLOCKS 1      // resident blocks per SM the logged backward is compiled for
#endif

struct BwdParams {
    dst_bwd_args a;
    BvhView bvh;
    const float4* cache;
    float* arena;
    unsigned int* status;
    int tiled, grid_h, grid_w;      // ray order, as in the forward
    int dist_on;                    // depth-distortion extension
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
    // chunk log of the matching forward call (null: not available)
    const unsigned long long* log_keys; const int2* log_hdr; const int* log_seg_head; const unsigned char* log_ray_ok;
    int log_seg_stride;
};

struct __align__(16) BwdState {
    float sox, soy, soz, sdx;
    float sdy, sdz, offset, dpt;
    float T_prev, C0, C1, C2;
    float D, Nx, Ny, Nz;
    float O0, O1, s_prod, Cp0;
    float Cp1, Cp2, cp0, cp1;
    float cp2, t_rgb0, t_rgb1, t_rgb2;
    float t_dpt, t_acc, t_aux0, t_aux1;
    float t_nx, t_ny, t_nz, dir_g0;
    float dir_g1, dir_g2, dro_x, dro_y;
    float dro_z, drd_x, drd_y, drd_z;
    int last_gidx, contributor, chunk, seg;
    int dir_gidx;
    float dm0, dvs, dws;        // distortion term on the primary segment: mapped depth of the first contribution, running sums of w c^2 and w
};
static_assert(sizeof(BwdState) == 208, "ray state is thirteen 16-byte words");

__device__ __forceinline__ void red4(float* addr, float a, float b, float c, float d) {
    atomicAdd(reinterpret_cast<float4*>(addr), make_float4(a, b, c, d));
}

// ---------------------------------------------------------------------------------------------
// Gradient rows leave the SM as bulk reductions. A contribution adds an 80-byte row to the packed arena and (with
// SH colours) a 48- or 192-byte row of coefficient gradients. As vector reductions that is 5 + 12 red.global.add.v4.f32
// per contribution and lane, and the L2's reduction path is what the kernel then waits for (without the reductions the
// logged backward of the headline workload takes 13 ms instead of 42). Instead every thread stages its rows in shared
// memory and hands each to the bulk copy engine as ONE cp.reduce.async.bulk (shared -> global, add.f32): a 192-byte row
// is one request instead of twelve. Two staging buffers per thread: a row is rewritten only after the engine has read
// the one staged two contributions earlier (cp.async.bulk.wait_group.read 1). Bulk operations want 16-byte aligned
// addresses and sizes that are multiples of 16 bytes: arena rows always qualify, SH rows when the gradient tensor is
// 16-byte aligned and 12 * (degree + 1)^2 is a multiple of 16 (degrees 1 and 3); other rows keep the vector reductions.
// ---------------------------------------------------------------------------------------------
#ifndef DST_BWD_BULK
#define DST_BWD_BULK 1
#endif
constexpr int STAGE_FLOATS = DST_ARENA_FLOATS + 48;                       // arena row + the longest SH row
constexpr size_t BWD_STAGE_BYTES = 2ull * BWD_THREADS * STAGE_FLOATS * 4;  // dynamic shared memory of every backward kernel

struct BulkStage {
    float* base;        // this thread's two staging rows (shared memory), STAGE_FLOATS each
    unsigned int n;     // rows handed over so far
};
__device__ __forceinline__ BulkStage bulk_stage_init(unsigned char* dyn_smem) {
    BulkStage b;
    b.base = reinterpret_cast<float*>(dyn_smem) + (size_t)threadIdx.x * STAGE_FLOATS;
    b.n = 0;
    return b;
}
// the row to fill next (waits until the engine has read what it held)
__device__ __forceinline__ float* bulk_stage_row(BulkStage& b) {
    asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
    return b.base + (size_t)(b.n & 1u) * BWD_THREADS * STAGE_FLOATS;
}
// adds `bytes` bytes of floats at shared-memory `src` to global `dst` (both 16-byte aligned, bytes a multiple of 16)
__device__ __forceinline__ void bulk_add(float* dst, const float* src, int bytes) {
    const unsigned int s = (unsigned int)__cvta_generic_to_shared(src);
    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" :: "l"(dst), "r"(s), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_stage_commit(BulkStage& b) {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    b.n++;
}
// Rows of the same surfel staged by several lanes of a warp are summed in shared memory before they leave, and only
// the lowest lane of each group hands its (summed) row to the engine. The lanes of a warp are neighbouring pixels that
// walk their chunk logs in step, so at one point of the loop most of them hold one of a handful of surfels; without the
// summing every lane's row is an addition of its own at the L2, which serialises additions to one address (the
// reductions were 11 of the backward's 26 ms on the 3M-surfel 1080p workload). The lanes that are here together split the
// 17 float4 columns of a row between them and each sums its columns over the rows of a group, in lane order.
// gidx < 0: this lane has no row. Returns true for the lanes that send their row.
#ifndef DST_BWD_AGGREGATE
#define DST_BWD_AGGREGATE 1
#endif
__device__ __forceinline__ bool bulk_stage_aggregate(const BulkStage& b, int gidx) {
#if DST_BWD_AGGREGATE
    const unsigned int act = __activemask();
    const int lane = threadIdx.x & 31;
    const unsigned int staged = __ballot_sync(act, gidx >= 0);           // lanes without a row pass -1 and form a group that is skipped
    // Worth it only where neighbouring pixels do hold the same surfels: when fewer than three quarters of the rows have the
    // surfel of the lane next door, every lane sends its own row (grouping costs more than it saves on scenes whose
    // surfels are small against the pixel spacing).
    const int next_door = __shfl_xor_sync(act, gidx, 1);
    const unsigned int paired = __ballot_sync(act, gidx >= 0 && ((act >> (lane ^ 1)) & 1u) != 0u && next_door == gidx);
    if (4 * __popc(paired) < 3 * __popc(staged)) return gidx >= 0;
    const unsigned int peers = __match_any_sync(act, gidx);
    const int first = __ffs(peers) - 1;
    const unsigned int leaders = __ballot_sync(act, lane == first) & staged;
    const unsigned int parity = __ballot_sync(act, (b.n & 1u) != 0u);
    __syncwarp(act);                                                     // every lane's row is staged
    if (leaders != staged) {                                              // some surfel is held by more than one lane
        float* warp_rows = b.base - (size_t)lane * STAGE_FLOATS;         // buffer 0 of lane 0
        const int rank = __popc(act & ((1u << lane) - 1u)), nact = __popc(act);
        for (unsigned int todo = leaders; todo; todo &= todo - 1u) {
            const int lead = __ffs(todo) - 1;
            const unsigned int grp = __shfl_sync(act, peers, lead);
            if ((grp & (grp - 1u)) == 0u) continue;                      // a lane alone with its surfel
            for (int col = rank; col < STAGE_FLOATS / 4; col += nact) {
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
                for (unsigned int q = grp; q;) {                         // four rows per pass, so that their loads are in flight together
                    const int r0 = __ffs(q) - 1; q &= q - 1u;
                    const int r1 = __ffs(q) - 1; q &= q - 1u;
                    const int r2 = __ffs(q) - 1; q &= q - 1u;
                    const int r3 = __ffs(q) - 1; q &= q - 1u;
#define DST_STAGED(r) reinterpret_cast<const float4*>(warp_rows + ((r) + (int)((parity >> (r)) & 1u) * BWD_THREADS) * STAGE_FLOATS)[col]
                    const float4 x0 = DST_STAGED(r0);
                    const float4 x1 = r1 >= 0 ? DST_STAGED(r1) : zero;
                    const float4 x2 = r2 >= 0 ? DST_STAGED(r2) : zero;
                    const float4 x3 = r3 >= 0 ? DST_STAGED(r3) : zero;
#undef DST_STAGED
                    acc.x += (x0.x + x1.x) + (x2.x + x3.x); acc.y += (x0.y + x1.y) + (x2.y + x3.y);
                    acc.z += (x0.z + x1.z) + (x2.z + x3.z); acc.w += (x0.w + x1.w) + (x2.w + x3.w);
                }
                reinterpret_cast<float4*>(warp_rows + (lead + (int)((parity >> lead) & 1u) * BWD_THREADS) * STAGE_FLOATS)[col] = acc;
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp(act);                                                 // the sums are in place
    }
    return lane == first && gidx >= 0;
#else
    return true;
#endif
}
// before the kernel ends: every row has been read from shared memory and added
__device__ __forceinline__ void bulk_stage_drain() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// The colour of a contribution as the backward needs it: a factor of gradients, not an input of a decision, so the sum
// may be fused (the forward's sh_channel() rounds every product and sum as the reference does: twice the instructions).
__device__ __forceinline__ float sh_channel_fused(int ncoef, const float* b, const float* c, int ch) {
    float r = b[0] * c[ch];
#pragma unroll
    for (int j = 1; j < 16; j++) if (j < ncoef) r = fmaf(b[j], c[3 * j + ch], r);
    return r + 0.5f;
}

struct V3 { float x, y, z; };
__device__ __forceinline__ V3 v3(float x, float y, float z) { V3 r; r.x = x; r.y = y; r.z = z; return r; }
__device__ __forceinline__ V3 operator+(V3 a, V3 b) { return v3(a.x + b.x, a.y + b.y, a.z + b.z); }
__device__ __forceinline__ V3 operator-(V3 a, V3 b) { return v3(a.x - b.x, a.y - b.y, a.z - b.z); }
__device__ __forceinline__ V3 operator*(float s, V3 a) { return v3(s * a.x, s * a.y, s * a.z); }
__device__ __forceinline__ float dot(V3 a, V3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
__device__ __forceinline__ V3 cross(V3 a, V3 b) { return v3(a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x); }

// optix_tracer/auxiliary.h:111-121
__device__ __forceinline__ V3 dnormvdv(V3 v, V3 dv) {
    const float sum2 = v.x * v.x + v.y * v.y + v.z * v.z;
    const float inv = 1.0f / sqrtf(sum2 * sum2 * sum2);
    return v3(((sum2 - v.x * v.x) * dv.x - v.y * v.x * dv.y - v.z * v.x * dv.z) * inv,
              (-v.x * v.y * dv.x + (sum2 - v.y * v.y) * dv.y - v.z * v.y * dv.z) * inv,
              (-v.x * v.z * dv.x - v.y * v.z * dv.y + (sum2 - v.z * v.z) * dv.z) * inv);
}
// optix_tracer/auxiliary.h:234-243
__device__ __forceinline__ V3 ddotndndn(V3 n, V3 d, V3 g) {
    const float nd = dot(n, d);
    return v3(g.x * (nd + d.x * n.x) + g.y * d.x * n.y + g.z * d.x * n.z,
              g.x * d.y * n.x + g.y * (nd + d.y * n.y) + g.z * d.y * n.z,
              g.x * d.z * n.x + g.y * d.z * n.y + g.z * (nd + d.z * n.z));
}
// optix_tracer/auxiliary.h:245-252
__device__ __forceinline__ V3 ddotndndd(V3 n, V3 g) {
    const float s = g.x * n.x + g.y * n.y + g.z * n.z;
    return v3(s * n.x, s * n.y, s * n.z);
}

// direction gradient of the SH colour (optix_tracer/backward.cu:96-165), s[j] = sh[j] . dL_dRGB
__device__ __forceinline__ V3 sh_dir_grad(int deg, const float* s, float x, float y, float z) {
    float gx = 0.f, gy = 0.f, gz = 0.f;
    if (deg > 0) {
        gx = -SHC1 * s[3]; gy = -SHC1 * s[1]; gz = SHC1 * s[2];
        if (deg > 1) {
            const float xx = x * x, yy = y * y, zz = z * z, xy = x * y, yz = y * z, xz = x * z;
            gx += SHC2_0 * y * s[4] + SHC2_2 * 2.f * -x * s[6] + SHC2_3 * z * s[7] + SHC2_4 * 2.f * x * s[8];
            gy += SHC2_0 * x * s[4] + SHC2_1 * z * s[5] + SHC2_2 * 2.f * -y * s[6] + SHC2_4 * 2.f * -y * s[8];
            gz += SHC2_1 * y * s[5] + SHC2_2 * 4.f * z * s[6] + SHC2_3 * x * s[7];
            if (deg > 2) {
                gx += SHC3_0 * s[9] * 6.f * xy + SHC3_1 * s[10] * yz + SHC3_2 * s[11] * -2.f * xy + SHC3_3 * s[12] * -6.f * xz +
                      SHC3_4 * s[13] * (-3.f * xx + 4.f * zz - yy) + SHC3_5 * s[14] * 2.f * xz + SHC3_6 * s[15] * 3.f * (xx - yy);
                gy += SHC3_0 * s[9] * 3.f * (xx - yy) + SHC3_1 * s[10] * xz + SHC3_2 * s[11] * (-3.f * yy + 4.f * zz - xx) +
                      SHC3_3 * s[12] * -6.f * yz + SHC3_4 * s[13] * -2.f * xy + SHC3_5 * s[14] * -2.f * yz + SHC3_6 * s[15] * -6.f * xy;
                gz += SHC3_1 * s[10] * xy + SHC3_2 * s[11] * 8.f * yz + SHC3_3 * s[12] * 3.f * (2.f * zz - xx - yy) +
                      SHC3_4 * s[13] * 8.f * xz + SHC3_5 * s[14] * (xx - yy);
            }
        }
    }
    return v3(gx, gy, gz);
}


__device__ __forceinline__ void bwd_load_state(const void* base, int ray, BwdState& s) {
    const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const BwdState*>(base) + ray);
    float4* dst = reinterpret_cast<float4*>(&s);
#pragma unroll
    for (int i = 0; i < 13; i++) dst[i] = src[i];
}
__device__ __forceinline__ void bwd_store_state(void* base, int ray, const BwdState& s) {
    float4* dst = reinterpret_cast<float4*>(reinterpret_cast<BwdState*>(base) + ray);
    const float4* src = reinterpret_cast<const float4*>(&s);
#pragma unroll
    for (int i = 0; i < 13; i++) dst[i] = src[i];
}

__device__ __forceinline__ void bwd_request(const BwdState& s, EnumReq& q) {
    if (s.chunk == 0) { q.ox = s.sox; q.oy = s.soy; q.oz = s.soz; }
    else { q.ox = xadd(s.sox, xmul(s.offset, s.sdx)); q.oy = xadd(s.soy, xmul(s.offset, s.sdy)); q.oz = xadd(s.soz, xmul(s.offset, s.sdz)); }
    q.dx = s.sdx; q.dy = s.sdy; q.dz = s.sdz; q.kmax0 = DST_T_MAX; q.pad = s.seg > 0 ? 1.f : 0.f;       // pad: the ray is on a reflected segment
}

// Finds the next segment to differentiate, from segment `start` downwards (backward.cu:706-802):
// skips the ones the reference skips, derives the segment's upstream gradients and the reflection
// chain, and resets the running sums. Writes the ray gradients and returns false when none is left.
__device__ __forceinline__ bool bwd_next_segment(const BwdParams& p, int ray, BwdState& s, int start) {
    const dst_trace_inputs& in = p.a.in;
    const int depth = in.max_trace_depth;
    const float* mid = p.a.mid_val + (size_t)ray * in.mid_stride;
    for (int i = start; i >= 0; i--) {
        const float4* mp = reinterpret_cast<const float4*>(mid + i * DST_MID_CHANNELS);
        const float4 m0 = __ldg(mp), m1 = __ldg(mp + 1), m2 = __ldg(mp + 2), m3 = __ldg(mp + 3);
        const float sdx = m0.w, sdy = m1.x, sdz = m1.y;
        const float tot_dpt = m1.z;
        const V3 tot_n = v3(m2.x, m2.y, m2.z);
        const float tot_o0 = m2.w, tot_c0 = m3.y, tot_c1 = m3.z, tot_c2 = m3.w;
        const float s_prev = i > 0 ? __ldg(mid + (i - 1) * DST_MID_CHANNELS + 11) : 1.0f;
        if (sqrtf(sdx * sdx + sdy * sdy + sdz * sdz) == 0.0f || s_prev <= in.specular_threshold) continue;    // :724

        const float g_rgb0 = __ldg(p.a.dL_drgb + 3 * (size_t)ray), g_rgb1 = __ldg(p.a.dL_drgb + 3 * (size_t)ray + 1), g_rgb2 = __ldg(p.a.dL_drgb + 3 * (size_t)ray + 2);
        const float f_this = (i == depth) ? 1.0f : 1.0f - tot_o0;
        s.t_rgb0 = g_rgb0 * f_this * s.s_prod; s.t_rgb1 = g_rgb1 * f_this * s.s_prod; s.t_rgb2 = g_rgb2 * f_this * s.s_prod;   // :760
        s.s_prod /= s_prev;                                                                                   // :762
        s.t_dpt = 0.f; s.t_acc = 0.f; s.t_aux0 = 0.f; s.t_aux1 = 0.f;
        V3 t_norm = v3(0.f, 0.f, 0.f);
        V3 dro = v3(s.dro_x, s.dro_y, s.dro_z), drd = v3(s.drd_x, s.drd_y, s.drd_z);
        if (i != depth) {
            // :769-774
            s.t_aux0 += g_rgb0 * (s.Cp0 / tot_o0) + g_rgb1 * (s.Cp1 / tot_o0) + g_rgb2 * (s.Cp2 / tot_o0);
            if (i > 0) {
                const float4 pm3 = __ldg(reinterpret_cast<const float4*>(mid + (i - 1) * DST_MID_CHANNELS) + 3);
                s.cp0 = pm3.y; s.cp1 = pm3.z; s.cp2 = pm3.w;
            } else { s.cp0 = s.cp1 = s.cp2 = 0.f; }
            s.Cp0 -= s.s_prod * (s.cp0 - tot_c0); s.Cp1 -= s.s_prod * (s.cp1 - tot_c1); s.Cp2 -= s.s_prod * (s.cp2 - tot_c2);
            const float nl = sqrtf(dot(tot_n, tot_n));
            if (nl != 0.0f) {                                                                                 // :778-790
                const V3 d = v3(sdx, sdy, sdz);
                drd = drd + 0.00001f * dro;
                const V3 n = (1.0f / nl) * tot_n;
                s.t_dpt += dro.x * sdx + dro.y * sdy + dro.z * sdz;
                const V3 gm2 = -2.0f * drd;
                t_norm = t_norm + dnormvdv(tot_n, ddotndndn(n, d, gm2));
                drd = tot_dpt * dro + drd + ddotndndd(n, gm2);
            }
        }
        if (i == 0) {                                                                                         // :793-802
            s.t_dpt += __ldg(p.a.dL_ddpt + ray); s.t_acc += __ldg(p.a.dL_dacc + ray);
            t_norm = t_norm + v3(__ldg(p.a.dL_dnorm + 3 * (size_t)ray), __ldg(p.a.dL_dnorm + 3 * (size_t)ray + 1), __ldg(p.a.dL_dnorm + 3 * (size_t)ray + 2));
            s.t_aux0 += __ldg(p.a.dL_daux + 2 * (size_t)ray); s.t_aux1 += __ldg(p.a.dL_daux + 2 * (size_t)ray + 1);
        }
        s.t_nx = t_norm.x; s.t_ny = t_norm.y; s.t_nz = t_norm.z;
        s.drd_x = drd.x; s.drd_y = drd.y; s.drd_z = drd.z;
        s.sox = m0.x; s.soy = m0.y; s.soz = m0.z; s.sdx = sdx; s.sdy = sdy; s.sdz = sdz;
        s.offset = 0.f; s.dpt = 0.f; s.T_prev = 1.f;
        s.C0 = s.C1 = s.C2 = 0.f; s.D = 0.f; s.Nx = s.Ny = s.Nz = 0.f; s.O0 = s.O1 = 0.f;
        s.last_gidx = -1; s.contributor = 0; s.chunk = 0; s.seg = i; s.dir_gidx = -1;
        s.dm0 = s.dvs = s.dws = 0.f;
        return true;
    }
    p.a.dL_dray_o[3 * (size_t)ray] = s.dro_x; p.a.dL_dray_o[3 * (size_t)ray + 1] = s.dro_y; p.a.dL_dray_o[3 * (size_t)ray + 2] = s.dro_z;
    p.a.dL_dray_d[3 * (size_t)ray] = s.drd_x; p.a.dL_dray_d[3 * (size_t)ray + 1] = s.drd_y; p.a.dL_dray_d[3 * (size_t)ray + 2] = s.drd_z;
    return false;
}

// backward.cu:683-703 (specular product over all bounces and the colour "behind" each one), then the first segment
__device__ __forceinline__ bool bwd_init_state(const BwdParams& p, int ray, BwdState& s) {
    const dst_trace_inputs& in = p.a.in;
    const float* mid = p.a.mid_val + (size_t)ray * in.mid_stride;
    s.Cp0 = __ldg(p.a.out_rgb + 3 * (size_t)ray); s.Cp1 = __ldg(p.a.out_rgb + 3 * (size_t)ray + 1); s.Cp2 = __ldg(p.a.out_rgb + 3 * (size_t)ray + 2);
    s.cp0 = s.cp1 = s.cp2 = 0.f;
    s.s_prod = 1.0f;
    for (int i = 0; i < in.max_trace_depth; i++) {
        const float4 m3 = __ldg(reinterpret_cast<const float4*>(mid + i * DST_MID_CHANNELS) + 3);
        const float4 m2 = __ldg(reinterpret_cast<const float4*>(mid + i * DST_MID_CHANNELS) + 2);
        s.Cp0 += s.s_prod * (s.cp0 - m3.y); s.Cp1 += s.s_prod * (s.cp1 - m3.z); s.Cp2 += s.s_prod * (s.cp2 - m3.w);
        s.cp0 = m3.y; s.cp1 = m3.z; s.cp2 = m3.w;
        s.s_prod *= m2.w;
    }
    s.dro_x = s.dro_y = s.dro_z = 0.f; s.drd_x = s.drd_y = s.drd_z = 0.f;
    s.dir_g0 = s.dir_g1 = s.dir_g2 = 0.f; s.dm0 = s.dvs = s.dws = 0.f;
    return bwd_next_segment(p, ray, s, in.max_trace_depth);
}

// b[j] for a run-time j without indexing the array (which would move it from registers to local memory)
__device__ __forceinline__ float basis_at(const float* b, int j) {
    float r = b[0];
#pragma unroll
    for (int k = 1; k < 16; k++) r = (j == k) ? b[k] : r;
    return r;
}

// Re-composites one gathered chunk of segment s.seg and accumulates the gradients of every
// contributing hit (backward.cu:429-655). Returns true while the ray needs another enumeration.
template <bool DIAG, int KS, bool DIST>
__device__ __forceinline__ bool bwd_shade(const BwdParams& p, int ray, BwdState& s, const unsigned long long* kb, int cnt, TraceCounters& tc, BulkStage& stage) {
    const dst_trace_inputs& in = p.a.in;
    const bool use_sh = in.colors_precomp == nullptr;
    const bool has_aux = in.others_precomp != nullptr;
    const int ncoef = (in.sh_degree + 1) * (in.sh_degree + 1);
    const bool sh_aligned = ((in.sh_coeffs * 3) & 3) == 0 && ((reinterpret_cast<uintptr_t>(in.shs) & 15) == 0);
    const bool dsh_aligned = ((in.sh_coeffs * 3) & 3) == 0 && ((reinterpret_cast<uintptr_t>(p.a.dL_dshs) & 15) == 0);
    const float bg0 = __ldg(in.background), bg1 = __ldg(in.background + 1), bg2 = __ldg(in.background + 2);
    const float4* mp = reinterpret_cast<const float4*>(p.a.mid_val + (size_t)ray * in.mid_stride + s.seg * DST_MID_CHANNELS);
    const float4 m1 = __ldg(mp + 1), m2 = __ldg(mp + 2), m3 = __ldg(mp + 3);
    const float tot_dpt = m1.z, tot_acc = m1.w;
    const V3 tot_n = v3(m2.x, m2.y, m2.z);
    const float tot_o0 = m2.w, tot_o1 = m3.x, tot_c0 = m3.y, tot_c1 = m3.z, tot_c2 = m3.w;
    const float sox = s.sox, soy = s.soy, soz = s.soz, sdx = s.sdx, sdy = s.sdy, sdz = s.sdz;
    const float t_rgb0 = s.t_rgb0, t_rgb1 = s.t_rgb1, t_rgb2 = s.t_rgb2, t_dpt = s.t_dpt, t_acc = s.t_acc, t_aux0 = s.t_aux0, t_aux1 = s.t_aux1;
    const V3 t_norm = v3(s.t_nx, s.t_ny, s.t_nz);
    const float min_depth = s.seg == 0 ? (in.start_from_first ? 0.2f : 0.0f) : 0.06f;
    const float T_threshold = 0.0001f;
    const float T_final = 1.0f - tot_acc;
    float C0 = s.C0, C1 = s.C1, C2 = s.C2, D = s.D, O0 = s.O0, O1 = s.O1;
    V3 N = v3(s.Nx, s.Ny, s.Nz);
    float T_prev = s.T_prev, T_next = 1.0f, dpt = s.dpt;
    const float offset = s.offset;
    int last_gidx = s.last_gidx, contributor = s.contributor;
    V3 dL_dray_o = v3(s.dro_x, s.dro_y, s.dro_z), dL_dray_d = v3(s.drd_x, s.drd_y, s.drd_z);
    int dir_gidx = s.dir_gidx; float dir_g0 = s.dir_g0, dir_g1 = s.dir_g1, dir_g2 = s.dir_g2;
    float sb[16];
    if (use_sh) sh_basis(in.sh_degree, sdx, sdy, sdz, sb);
    if (DIAG) { if (s.chunk == 0) tc.segs++; }
    // Distortion extension (primary segment only; see fwd_shade): upstream gradient, the totals the forward saved, the
    // running sums. With W = sum w (the accumulated opacity), mu = M1 / W, c_k = m_k - mu, V = M2 - M1^2 / W = sum w c^2:
    // d dist / d m_k = 2 w_k W c_k, d dist / d w_k = W c_k^2 + V, and what lies behind hit k enters through the
    // transmittance: sum_{i>k} (d dist / d w_i) w_i = W (V - V_k) + V (W - W_k) with the running sums through k.
    const bool dist_on = DIST && s.seg == 0 && p.a.dL_ddist && p.a.out_dist && tot_acc > 0.0f;
    const float t_dist = dist_on ? __ldg(p.a.dL_ddist + ray) : 0.f;
    const float dist_mu = dist_on ? __ldg(p.a.out_dist + 3 * (size_t)ray + 1) / tot_acc : 0.f;
    const float dist_V = dist_on ? __ldg(p.a.out_dist + 3 * (size_t)ray + 2) - __ldg(p.a.out_dist + 3 * (size_t)ray + 1) * dist_mu : 0.f;
    float dm0 = s.dm0, dvs = s.dvs, dws = s.dws;

    bool stop = false;
    for (int sl = 0; sl < cnt; sl++) {
        // One pass of the body per hit; a hit that does not contribute leaves it early. The lanes of the warp meet again
        // behind it, where the rows of the lanes that did contribute are summed per surfel and sent.
        bool staged = false;
        int gsent = -1;
        float4* st = nullptr;
        do {
        const unsigned long long key = kb[sl * KS];
        const int pidx = (int)(unsigned int)key;
        const int gidx = pidx >> 1;
        if (gidx == last_gidx) break;
        if (DIAG) tc.evals++;
        SlotEval e;
        const bool ok = eval_slot(key, offset, sox, soy, soz, sdx, sdy, sdz, min_depth, p.cache, gidx, e);
        dpt = e.dpt;
        if (!ok) break;
        const float alpha = e.alpha;
        T_next = xmul(T_prev, xsub(1.0f, alpha));
        if (T_next < T_threshold) { stop = true; break; }
        contributor++;
        if (contributor > DST_MAX_INTERSECTION) { stop = true; break; }
        last_gidx = gidx;
        if (DIAG) tc.contribs++;
        const float w = xmul(alpha, T_prev);
        const V3 normal = v3(e.nsign * e.r2.x, e.nsign * e.r2.y, e.nsign * e.r2.z);
        float c0, c1, c2, k0 = 1.f, k1 = 1.f, k2 = 1.f;       // colour and its clamp mask
        float csh[48];
        float pc0 = 0.f, pc1 = 0.f, pc2 = 0.f;
        if (use_sh) load_sh_row(in.shs + 3 * (size_t)gidx * in.sh_coeffs, 3 * ncoef, sh_aligned, csh);
        else { const float* cp = in.colors_precomp + 3 * (size_t)gidx; pc0 = __ldg(cp); pc1 = __ldg(cp + 1); pc2 = __ldg(cp + 2); }
        float2 ax = make_float2(0.f, 0.f);
        if (has_aux) ax = __ldg(reinterpret_cast<const float2*>(in.others_precomp) + gidx);
        const float4* vq = reinterpret_cast<const float4*>(in.vertices + 12 * (size_t)gidx);
        const float4 va = __ldg(vq), vb = __ldg(vq + 1), vc = __ldg(vq + 2);
        const V3 pm = v3(__ldg(in.means3D + 3 * (size_t)gidx), __ldg(in.means3D + 3 * (size_t)gidx + 1), __ldg(in.means3D + 3 * (size_t)gidx + 2));
        const float4 q = __ldg(reinterpret_cast<const float4*>(in.rotations) + gidx);
        if (use_sh) {
            c0 = sh_channel_fused(ncoef, sb, csh, 0); c1 = sh_channel_fused(ncoef, sb, csh, 1); c2 = sh_channel_fused(ncoef, sb, csh, 2);
            k0 = c0 < 0.f ? 0.f : 1.f; k1 = c1 < 0.f ? 0.f : 1.f; k2 = c2 < 0.f ? 0.f : 1.f;
            c0 = fmaxf(c0, 0.f); c1 = fmaxf(c1, 0.f); c2 = fmaxf(c2, 0.f);
        } else { c0 = pc0; c1 = pc1; c2 = pc2; }
        C0 = xadd(C0, xmul(w, c0)); C1 = xadd(C1, xmul(w, c1)); C2 = xadd(C2, xmul(w, c2));
        float ox0 = 0.f, ox1 = 0.f;
        if (has_aux) {
            ox0 = ax.x; ox1 = ax.y;
            O0 = xadd(O0, xmul(w, ox0)); O1 = xadd(O1, xmul(w, ox1));
        }
        D = xadd(D, xmul(w, dpt));
        N.x = xadd(N.x, xmul(w, normal.x)); N.y = xadd(N.y, xmul(w, normal.y)); N.z = xadd(N.z, xmul(w, normal.z));

        // gradient w.r.t. alpha from every composited quantity (backward.cu:529-568)
        const float inv = 1.0f / (1.0f - alpha);
        float dL_dalpha = t_rgb0 * (T_prev * c0 - (tot_c0 - C0) * inv) + t_rgb1 * (T_prev * c1 - (tot_c1 - C1) * inv) +
                          t_rgb2 * (T_prev * c2 - (tot_c2 - C2) * inv);
        dL_dalpha += (t_rgb0 * bg0 + t_rgb1 * bg1 + t_rgb2 * bg2) * (-T_final * inv);   // background counted a second time, as the reference does
        if (has_aux) dL_dalpha += t_aux0 * (T_prev * ox0 - (tot_o0 - O0) * inv) + t_aux1 * (T_prev * ox1 - (tot_o1 - O1) * inv);
        dL_dalpha += t_dpt * (T_prev * dpt - (tot_dpt - D) * inv);
        dL_dalpha += t_norm.x * (T_prev * normal.x - (tot_n.x - N.x) * inv) + t_norm.y * (T_prev * normal.y - (tot_n.y - N.y) * inv) +
                     t_norm.z * (T_prev * normal.z - (tot_n.z - N.z) * inv);
        dL_dalpha += t_acc * (T_prev - tot_acc * inv);      // the reference's running weight sum stays 0 (backward.cu:359, 568)
        float dist_dd = 0.f;       // gradient of the distortion with respect to this hit's depth
        if (DIST && dist_on) {
            const float m_abs = DST_DIST_K * (1.0f - DST_DIST_NEAR / dpt);
            if (contributor == 1) dm0 = m_abs;
            const float cm = (m_abs - dm0) - dist_mu;
            dws += w; dvs += w * cm * cm;
            const float d_dw = tot_acc * cm * cm + dist_V;
            const float behind = tot_acc * (dist_V - dvs) + dist_V * (tot_acc - dws);
            dL_dalpha += t_dist * (d_dw * T_prev - behind * inv);
            dist_dd = t_dist * 2.0f * w * tot_acc * cm * DST_DIST_K * DST_DIST_NEAR / (dpt * dpt);
        }

        const float opac = e.r2.w, G = e.G;
        const float dL_dG = dL_dalpha * opac;
        const float pc = (opac * G) > 0.99f ? 0.0f : 1.0f;
        const float dL_dopac = dL_dalpha * G * pc;

        // geometry (backward.cu:201-287, 581-607)
        const float sx = e.r3.x, sy = e.r3.y, u = e.u, v = e.v;
        const V3 R0 = v3(e.r0.x, e.r0.y, e.r0.z), R1 = v3(e.r1.x, e.r1.y, e.r1.z);
        const V3 rel = v3(e.X - pm.x, e.Y - pm.y, e.Z - pm.z);
        const float kk = dL_dG * pc;
        const float dL_du = kk * -G * u, dL_dv = kk * -G * v;
        V3 dR0 = (dL_du / sx) * rel, dR1 = (dL_dv / sy) * rel;
        const V3 dR2 = v3(t_norm.x * w * e.nsign, t_norm.y * w * e.nsign, t_norm.z * w * e.nsign);
        float dsx = kk * (G * u * u / sx), dsy = kk * (G * v * v / sy);
        V3 dmean = (kk * G) * ((u / sx) * R0 + (v / sy) * R1);
        const V3 dxyz = (dL_du / sx) * R0 + (dL_dv / sy) * R1;
        const V3 rd = v3(sdx, sdy, sdz), ro = v3(sox, soy, soz);
        const float dL_dd = t_dpt * w + dist_dd + dot(dxyz, rd);
        V3 p1, p2, p3; float h1x, h1y, h2x, h2y, h3x, h3y;
        {
            if ((pidx & 1) == 0) {
                p1 = v3(va.x, va.y, va.z); p2 = v3(va.w, vb.x, vb.y); p3 = v3(vb.z, vb.w, vc.x);
                h1x = -3.f; h1y = 3.f; h2x = -3.f; h2y = -3.f; h3x = 3.f; h3y = 3.f;
            } else {
                p1 = v3(va.w, vb.x, vb.y); p2 = v3(vb.z, vb.w, vc.x); p3 = v3(vc.y, vc.z, vc.w);
                h1x = -3.f; h1y = -3.f; h2x = 3.f; h2y = 3.f; h3x = 3.f; h3y = -3.f;
            }
        }
        const V3 n = cross(p2 - p1, p3 - p1);
        const V3 cvec = p1 - ro;
        const float pp = dot(n, cvec), qq = dot(n, rd);
        const float iq = 1.0f / qq;
        const V3 dn = iq * (cvec - (pp * iq) * rd);
        const V3 dv1 = dL_dd * cross(p2 - p3, dn) + (dL_dd * iq) * n;
        const V3 dv2 = dL_dd * cross(p3 - p1, dn);
        const V3 dv3 = dL_dd * cross(p1 - p2, dn);
        dL_dray_o = dL_dray_o + dxyz - (dL_dd * iq) * n;
        if (!use_sh) dL_dray_d = dL_dray_d + dpt * dxyz - (dL_dd * pp * iq * iq) * n;   // with SH the value is replaced below
        const V3 shx = h1x * dv1 + h2x * dv2 + h3x * dv3, shy = h1y * dv1 + h2y * dv2 + h3y * dv3;
        dR0 = dR0 + sx * shx; dR1 = dR1 + sy * shy;
        dsx += dot(R0, shx); dsy += dot(R1, shy);
        dmean = dmean + dv1 + dv2 + dv3;
        // quaternion (auxiliary.h:433-477; no gradient through the normalisation)
        const float qs = rsqrtf(q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z);
        const float qw = q.x * qs, qx = q.y * qs, qy = q.z * qs, qz = q.w * qs;
        const float dq0 = 2.f * (qx * (dR1.z - dR2.y) + qy * (dR2.x - dR0.z) + qz * (dR0.y - dR1.x));
        const float dq1 = 2.f * (-2.f * qx * (dR1.y + dR2.z) + qy * (dR0.y + dR1.x) + qz * (dR0.z + dR2.x) + qw * (dR1.z - dR2.y));
        const float dq2 = 2.f * (qx * (dR0.y + dR1.x) - 2.f * qy * (dR0.x + dR2.z) + qz * (dR1.z + dR2.y) + qw * (dR2.x - dR0.z));
        const float dq3 = 2.f * (qx * (dR0.z + dR2.x) + qy * (dR1.z + dR2.y) - 2.f * qz * (dR0.x + dR1.y) + qw * (dR0.y - dR1.x));

        // per-surfel accumulation (backward.cu:543, 557, 578, 610-626)
#if !DST_BWD_BULK
        float* row = p.arena + (size_t)gidx * DST_ARENA_FLOATS;
#endif
        const float hd = 0.5f * dpt;
        const float dc0 = t_rgb0 * w, dc1 = t_rgb1 * w, dc2 = t_rgb2 * w;
        const float m0c = dc0 * k0, m1c = dc1 * k1, m2c = dc2 * k2;
        const int nf = 3 * ncoef, nv = nf >> 2;
        float* dsh = use_sh ? p.a.dL_dshs + 3 * (size_t)gidx * in.sh_coeffs : nullptr;
#if DST_BWD_BULK
        {
            st = reinterpret_cast<float4*>(bulk_stage_row(stage));
            st[0] = make_float4(dq0, dq1, dq2, dq3);
            st[1] = make_float4(dmean.x, dmean.y, dmean.z, dL_dopac);
            st[2] = make_float4(dmean.x * hd, dmean.y * hd, dmean.z * hd, 0.f);
            st[3] = make_float4(dsx, dsy, has_aux ? t_aux0 * w : 0.f, has_aux ? t_aux1 * w : 0.f);
            st[4] = make_float4(dc0, dc1, dc2, 0.f);
            const bool sh_bulk = use_sh && dsh_aligned && (nf & 3) == 0;
            if (sh_bulk) {
#pragma unroll
                for (int q4 = 0; q4 < 12; q4++) {
                    if (q4 < nv) {
                        float o4[4];
#pragma unroll
                        for (int l = 0; l < 4; l++) { const int f = 4 * q4 + l; const int j = f / 3, ch = f - 3 * j; o4[l] = sb[j] * (ch == 0 ? m0c : ch == 1 ? m1c : m2c); }
                        st[DST_ARENA_FLOATS / 4 + q4] = make_float4(o4[0], o4[1], o4[2], o4[3]);
                    }
                }
            }
            staged = true; gsent = gidx;
            if (use_sh && !sh_bulk) {
                if (dsh_aligned) {
#pragma unroll
                    for (int q4 = 0; q4 < 12; q4++) {
                        if (q4 < nv) {
                            float o4[4];
#pragma unroll
                            for (int l = 0; l < 4; l++) { const int f = 4 * q4 + l; const int j = f / 3, ch = f - 3 * j; o4[l] = sb[j] * (ch == 0 ? m0c : ch == 1 ? m1c : m2c); }
                            red4(dsh + 4 * q4, o4[0], o4[1], o4[2], o4[3]);
                        }
                    }
                    for (int f = nv << 2; f < nf; f++) { const int j = f / 3, ch = f - 3 * j; atomicAdd(dsh + f, basis_at(sb, j) * (ch == 0 ? m0c : ch == 1 ? m1c : m2c)); }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        if (j < ncoef) { atomicAdd(dsh + 3 * j, sb[j] * m0c); atomicAdd(dsh + 3 * j + 1, sb[j] * m1c); atomicAdd(dsh + 3 * j + 2, sb[j] * m2c); }
                    }
                }
            }
        }
#else
        red4(row, dq0, dq1, dq2, dq3);
        red4(row + 4, dmean.x, dmean.y, dmean.z, dL_dopac);
        red4(row + 8, dmean.x * hd, dmean.y * hd, dmean.z * hd, 0.f);
        red4(row + 12, dsx, dsy, has_aux ? t_aux0 * w : 0.f, has_aux ? t_aux1 * w : 0.f);
        red4(row + 16, dc0, dc1, dc2, 0.f);
        if (use_sh) {
            if (dsh_aligned) {
                // 3*ncoef floats as 4-float reductions (ncoef = 4, 16 -> 3, 12 vectors; 1, 9 leave a scalar tail)
#pragma unroll
                for (int q4 = 0; q4 < 12; q4++) {
                    if (q4 < nv) {
                        float o4[4];
#pragma unroll
                        for (int l = 0; l < 4; l++) { const int f = 4 * q4 + l; const int j = f / 3, ch = f - 3 * j; o4[l] = sb[j] * (ch == 0 ? m0c : ch == 1 ? m1c : m2c); }
                        red4(dsh + 4 * q4, o4[0], o4[1], o4[2], o4[3]);
                    }
                }
                for (int f = nv << 2; f < nf; f++) { const int j = f / 3, ch = f - 3 * j; atomicAdd(dsh + f, basis_at(sb, j) * (ch == 0 ? m0c : ch == 1 ? m1c : m2c)); }
            } else {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    if (j < ncoef) { atomicAdd(dsh + 3 * j, sb[j] * m0c); atomicAdd(dsh + 3 * j + 1, sb[j] * m1c); atomicAdd(dsh + 3 * j + 2, sb[j] * m2c); }
                }
            }
        }
#endif
        if (use_sh) {
            dir_gidx = gidx; dir_g0 = m0c; dir_g1 = m1c; dir_g2 = m2c;
        }
        T_prev = T_next;
        } while (false);
#if DST_BWD_BULK
        if ((p.tiled ? bulk_stage_aggregate(stage, gsent) : true) && staged) {       // linear ray lists: neighbours in the list are not neighbours on a surface
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the staged values become visible to the bulk copy engine
            bulk_add(p.arena + (size_t)gsent * DST_ARENA_FLOATS, reinterpret_cast<const float*>(st), DST_ARENA_FLOATS * 4);
            if (use_sh && dsh_aligned && ((3 * ncoef) & 3) == 0)
                bulk_add(p.a.dL_dshs + 3 * (size_t)gsent * in.sh_coeffs, reinterpret_cast<const float*>(st + DST_ARENA_FLOATS / 4), 3 * ncoef * 4);
            bulk_stage_commit(stage);
        }
#endif
        if (stop) break;
    }
    s.C0 = C0; s.C1 = C1; s.C2 = C2; s.D = D; s.O0 = O0; s.O1 = O1; s.Nx = N.x; s.Ny = N.y; s.Nz = N.z;
    s.T_prev = T_prev; s.dpt = dpt; s.last_gidx = last_gidx; s.contributor = contributor;
    s.dro_x = dL_dray_o.x; s.dro_y = dL_dray_o.y; s.dro_z = dL_dray_o.z;
    s.drd_x = dL_dray_d.x; s.drd_y = dL_dray_d.y; s.drd_z = dL_dray_d.z;
    s.dir_gidx = dir_gidx; s.dir_g0 = dir_g0; s.dir_g1 = dir_g1; s.dir_g2 = dir_g2;
    s.dm0 = dm0; s.dvs = dvs; s.dws = dws;
    s.chunk++;
    bool seg_done = stop || T_next < T_threshold || cnt < DST_CHUNK || contributor > DST_MAX_INTERSECTION;
    if (!seg_done && s.chunk >= DST_MAX_CHUNKS) { atomicOr(p.status, DST_STATUS_CHUNK_LIMIT); seg_done = true; }
    if (!seg_done) {
        s.offset = (float)((double)dpt + 0.00001);
        return true;
    }
    // With SH colours the reference ASSIGNS the SH direction gradient to the ray-direction
    // accumulator at every contribution (backward.cu:165, 631-632), so what survives a segment
    // is the value of its last contribution.
    if (use_sh && dir_gidx >= 0) {
        float csh[48], sj[16];
        load_sh_row(in.shs + 3 * (size_t)dir_gidx * in.sh_coeffs, 3 * ncoef, sh_aligned, csh);
#pragma unroll
        for (int j = 0; j < 16; j++) sj[j] = j < ncoef ? csh[3 * j] * dir_g0 + csh[3 * j + 1] * dir_g1 + csh[3 * j + 2] * dir_g2 : 0.f;
        const V3 g = sh_dir_grad(in.sh_degree, sj, sdx, sdy, sdz);
        s.drd_x = g.x; s.drd_y = g.y; s.drd_z = g.z;
    }
    return bwd_next_segment(p, ray, s, s.seg - 1);
}

__global__ void __launch_bounds__(256) k_bwd_init(const __grid_constant__ BwdParams p, long long slots) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= slots) return;
    if (i == 0) p.counts[0] = (int)slots;
    int ray = ray_of_slot(i, p.grid_h, p.grid_w, p.tiled != 0);
    if (ray >= 0) {
        BwdState s;
        if (bwd_init_state(p, ray, s)) {
            bwd_store_state(p.state, ray, s);
            EnumReq q;
            bwd_request(s, q);
            p.req[ray] = q;
        } else ray = -1;       // no segment to differentiate: the (zero) ray gradients are already written
    }
    p.list[0][i] = ray;
}

template <bool DIAG, bool DIST>
__global__ void __launch_bounds__(BWD_THREADS) k_bwd_shade(const __grid_constant__ BwdParams p, int round) {
    const int n = p.counts[round];
    if (n < p.min_count) return;
    const int* list = p.list[round & 1];
    int* next_list = p.list[(round + 1) & 1];
    TraceCounters tc = { 0, 0, 0, 0, 0, 0 };
    extern __shared__ __align__(128) unsigned char dyn_smem[];
    BulkStage stage = bulk_stage_init(dyn_smem);
    const int n_pad = (n + 31) & ~31;
    for (int i = blockIdx.x * BWD_THREADS + threadIdx.x; i < n_pad; i += gridDim.x * BWD_THREADS) {
        const int ray = i < n ? list[i] : -1;
        bool alive = false;
        int cls = 0;
        if (ray >= 0) {
            BwdState s;
            bwd_load_state(p.state, ray, s);
            alive = bwd_shade<DIAG, 1, DIST>(p, ray, s, p.kbuf + (size_t)ray * DST_CHUNK, p.kcnt[ray], tc, stage);
            if (alive) {
                bwd_store_state(p.state, ray, s);
                EnumReq q;
                bwd_request(s, q);
                p.req[ray] = q;
                cls = s.seg > 0;
            }
        }
        if (p.lv.stable) live_out(p.lv, round, i, alive, ray, cls);
        else append_alive(alive, ray, next_list, p.counts + round + 1);
    }
    bulk_stage_drain();
    if (DIAG && p.a.counters) {
        atomicAdd(p.a.counters + 0, tc.segs); atomicAdd(p.a.counters + 4, tc.evals); atomicAdd(p.a.counters + 5, tc.contribs);
    }
}

template <bool DIAG, bool DIST>
__global__ void __launch_bounds__(BWD_THREADS) k_bwd_tail(const __grid_constant__ BwdParams p) {
    __shared__ unsigned long long kshared[DST_CHUNK * BWD_THREADS];
    const int round = first_skipped_round(p.counts, p.rounds, p.min_count);
    const int n = p.counts[round];
    const int* list = p.list[round & 1];
    unsigned long long* kb = kshared + threadIdx.x;
    TraceCounters tc = { 0, 0, 0, 0, 0, 0 };
    extern __shared__ __align__(128) unsigned char dyn_smem[];
    BulkStage stage = bulk_stage_init(dyn_smem);
    for (int i = blockIdx.x * BWD_THREADS + threadIdx.x; i < n; i += gridDim.x * BWD_THREADS) {
        const int ray = list[i];
        if (ray < 0) continue;
        BwdState s;
        bwd_load_state(p.state, ray, s);
        bool alive = true;
        while (alive) {
            EnumReq q;
            bwd_request(s, q);
            const int cnt = knearest<false, DIAG, BWD_THREADS>(p.bvh, q.ox, q.oy, q.oz, q.dx, q.dy, q.dz, kb, p.status, tc, q.kmax0);
            if (DIAG) tc.enums++;
            alive = bwd_shade<DIAG, BWD_THREADS, DIST>(p, ray, s, kb, cnt, tc, stage);
        }
    }
    bulk_stage_drain();
    if (DIAG && p.a.counters) {
        atomicAdd(p.a.counters + 0, tc.segs); atomicAdd(p.a.counters + 1, tc.enums); atomicAdd(p.a.counters + 2, tc.nodes);
        atomicAdd(p.a.counters + 3, tc.quads); atomicAdd(p.a.counters + 4, tc.evals); atomicAdd(p.a.counters + 5, tc.contribs);
    }
}

__device__ __forceinline__ void bwd_flush_counters(unsigned long long* counters, const TraceCounters& tc) {
    if (!counters) return;
    if (tc.segs) atomicAdd(counters + 0, tc.segs);
    if (tc.enums) atomicAdd(counters + 1, tc.enums);
    if (tc.nodes) atomicAdd(counters + 2, tc.nodes);
    if (tc.quads) atomicAdd(counters + 3, tc.quads);
    if (tc.evals) atomicAdd(counters + 4, tc.evals);
    if (tc.contribs) atomicAdd(counters + 5, tc.contribs);
}

// Backward over the chunk log of the matching forward call: every ray re-composites the chunks the
// forward composited (chained per segment), so no hierarchy walk is needed; one thread per ray, all
// segments. Rays whose log is incomplete (log full during the forward) are initialised and queued
// for k_bwd_tail, which re-traces them.
template <bool DIAG, bool DIST>
__global__ void __launch_bounds__(BWD_THREADS, DST_BWD_LOGGED_BLOCKS) k_bwd_logged(const __grid_constant__ BwdParams p, long long slots) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int ray = i < slots ? ray_of_slot(i, p.grid_h, p.grid_w, p.tiled != 0) : -1;
    TraceCounters tc = { 0, 0, 0, 0, 0, 0 };
    extern __shared__ __align__(128) unsigned char dyn_smem[];
    BulkStage stage = bulk_stage_init(dyn_smem);
    bool requeue = false, active = false;
    BwdState s;
    s.seg = -1;
    const int* heads = nullptr;
    int idx = -1;
    if (ray >= 0 && bwd_init_state(p, ray, s)) {
        if (!p.log_ray_ok[ray]) {
            bwd_store_state(p.state, ray, s);
            EnumReq q;
            bwd_request(s, q);
            p.req[ray] = q;
            requeue = true;
        } else {
            heads = p.log_seg_head + (size_t)ray * p.log_seg_stride;
            idx = heads[s.seg];
            active = true;
        }
    }
    // The warp walks its rays' chunk chains in step: one chunk per pass, and only the lanes whose ray is in the
    // latest segment still open in the warp (the backward visits a ray's segments last to first). Neighbouring pixels then
    // composite the same surfels in the same pass of the hit loop, which is what bulk_stage_aggregate() feeds on, and
    // the lanes run one instruction stream instead of drifting apart chunk by chunk.
    for (;;) {
        const int cur = __reduce_max_sync(0xffffffffu, active ? s.seg : -1);
        if (cur < 0) break;
        if (active && s.seg == cur) {
            if (idx < 0) { atomicOr(p.status, DST_STATUS_LOG_MISMATCH); active = false; }
            else {
                const int2 hdr = __ldg(p.log_hdr + idx);
                if (DIAG) tc.enums++;
                if (!bwd_shade<DIAG, 1, DIST>(p, ray, s, p.log_keys + (size_t)idx * DST_CHUNK, hdr.y, tc, stage)) active = false;
                else idx = (s.chunk == 0) ? heads[s.seg] : hdr.x;      // chunk == 0: an earlier segment has begun
            }
        }
    }
    bulk_stage_drain();
    append_alive(requeue, ray, p.list[0], p.counts);
    if (DIAG) bwd_flush_counters(p.a.counters, tc);
}

// arena rows -> the caller's gradient tensors
__global__ void __launch_bounds__(256) k_unpack(int P, const float* __restrict__ arena, float* __restrict__ d_rot, float* __restrict__ d_mean,
                                                float* __restrict__ d_opac, float* __restrict__ d_g3d, float* __restrict__ d_scale,
                                                float* __restrict__ d_others, float* __restrict__ d_color) {
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= P) return;
    const float4* r = reinterpret_cast<const float4*>(arena + (size_t)g * DST_ARENA_FLOATS);
    const float4 a = r[0], b = r[1], c = r[2], d = r[3], e = r[4];
    reinterpret_cast<float4*>(d_rot)[g] = a;
    d_mean[3 * (size_t)g] = b.x; d_mean[3 * (size_t)g + 1] = b.y; d_mean[3 * (size_t)g + 2] = b.z;
    d_opac[g] = b.w;
    d_g3d[3 * (size_t)g] = c.x; d_g3d[3 * (size_t)g + 1] = c.y; d_g3d[3 * (size_t)g + 2] = c.z;
    d_scale[2 * (size_t)g] = d.x; d_scale[2 * (size_t)g + 1] = d.y;
    d_others[2 * (size_t)g] = d.z; d_others[2 * (size_t)g + 1] = d.w;
    d_color[3 * (size_t)g] = e.x; d_color[3 * (size_t)g + 1] = e.y; d_color[3 * (size_t)g + 2] = e.z;
}

}  // namespace

BvhView dst_bvh_view(const dst_handle* h);
int dst_check_inputs(dst_handle* h, const dst_trace_inputs* in);
long long dst_call_signature(const dst_trace_inputs* in);
void dst_slot_grid(const dst_handle* h, const dst_trace_inputs* in, int* gh, int* gw);

// the staging rows need more dynamic shared memory than a kernel gets by default: raise the limit of every instantiation once per device
template <typename K>
static cudaError_t allow_stage_smem(K kernel) { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BWD_STAGE_BYTES); }
static int backward_kernel_setup(dst_handle* h) {
    static bool done[64] = { false };
    if (h->device >= 0 && h->device < 64 && done[h->device]) return DST_OK;
    cudaError_t e = cudaSuccess;
#define DST_SETUP(K) if (e == cudaSuccess) e = allow_stage_smem(K<false, false>); if (e == cudaSuccess) e = allow_stage_smem(K<false, true>); \
                     if (e == cudaSuccess) e = allow_stage_smem(K<true, false>); if (e == cudaSuccess) e = allow_stage_smem(K<true, true>);
    DST_SETUP(k_bwd_shade) DST_SETUP(k_bwd_tail) DST_SETUP(k_bwd_logged)
#undef DST_SETUP
    if (e != cudaSuccess) { cudaGetLastError(); return dst_set_error(h, DST_E_CUDA, "raising the shared-memory limit of the backward kernels failed: %s", cudaGetErrorString(e)); }
    if (h->device >= 0 && h->device < 64) done[h->device] = true;
    return DST_OK;
}

int dst_backward_impl(dst_handle* h, const dst_bwd_args* a, cudaStream_t st) {
    int rc = dst_check_inputs(h, &a->in);
    if (rc != DST_OK) return rc;
    rc = backward_kernel_setup(h);
    if (rc != DST_OK) return rc;
    if (!a->out_rgb || !a->mid_val || !a->dL_drgb || !a->dL_ddpt || !a->dL_dacc || !a->dL_dnorm || !a->dL_daux)
        return dst_set_error(h, DST_E_ARG, "a saved forward output or upstream gradient pointer is null");
    if (!a->dL_dray_o || !a->dL_dray_d || !a->dL_dmeans3D || !a->dL_dgrads3D || !a->dL_dcolors || !a->dL_dothers ||
        !a->dL_dopacities || !a->dL_dscales || !a->dL_drotations || (a->in.shs && !a->dL_dshs))
        return dst_set_error(h, DST_E_ARG, "a gradient output pointer is null");
    if ((reinterpret_cast<uintptr_t>(a->mid_val) & 15) || (reinterpret_cast<uintptr_t>(a->in.vertices) & 15) ||
        (reinterpret_cast<uintptr_t>(a->in.rotations) & 15) || (reinterpret_cast<uintptr_t>(a->dL_drotations) & 15) ||
        (a->in.others_precomp && (reinterpret_cast<uintptr_t>(a->in.others_precomp) & 7)))
        return dst_set_error(h, DST_E_ARG, "mid_val, vertices, rotations and dL_drotations must be 16-byte aligned");
    const int64_t P = a->in.P;
    if (P > h->arena_cap) {
        cudaFree(h->arena); h->arena = nullptr; h->arena_cap = 0;
        const int64_t cap = P + P / 8 + 1024;
        if (cudaMalloc(&h->arena, 4 * DST_ARENA_FLOATS * cap) != cudaSuccess) { cudaGetLastError(); return dst_set_error(h, DST_E_NOMEM, "gradient arena allocation failed"); }
        h->arena_cap = cap;
    }
    rc = dst_prepare_cache(h, &a->in, st);
    if (rc != DST_OK) return rc;
    DST_CUDA_TRY(h, cudaMemsetAsync(h->arena, 0, 4 * DST_ARENA_FLOATS * (size_t)P, st));
    if (a->dL_dshs) DST_CUDA_TRY(h, cudaMemsetAsync(a->dL_dshs, 0, 12 * (size_t)P * a->in.sh_coeffs, st));
    BwdParams p;
    p.a = *a; p.bvh = dst_bvh_view(h); p.cache = h->cache; p.arena = h->arena; p.status = h->status;
    p.dist_on = h->distortion;
    dst_slot_grid(h, &a->in, &p.grid_h, &p.grid_w);
    p.tiled = p.grid_h >= 16;
    const long long slots = slots_of_grid(p.grid_h, p.grid_w, p.tiled != 0);
    rc = dst_ensure_wavefront(h, slots, sizeof(BwdState));
    if (rc != DST_OK) return rc;
    p.state = h->wf_state; p.req = static_cast<EnumReq*>(h->wf_req); p.kbuf = h->wf_kbuf; p.kcnt = h->wf_kcnt;
    p.list[0] = h->wf_list[0]; p.list[1] = h->wf_list[1]; p.counts = h->wf_counts;
    const bool diag = a->counters != nullptr;
    const bool dist = h->distortion != 0 && a->dL_ddist != nullptr && a->out_dist != nullptr;
    const bool use_log = a->forward_serial != 0 && a->forward_serial == h->log_serial && h->log_H == a->in.H && h->log_W == a->in.W &&
                         h->log_depth == a->in.max_trace_depth;
    p.log_keys = h->log_keys; p.log_hdr = h->log_hdr; p.log_seg_head = h->log_seg_head; p.log_ray_ok = h->log_ray_ok;
    p.log_seg_stride = a->in.max_trace_depth + 1;
    DST_CUDA_TRY(h, cudaMemsetAsync(h->wf_counts, 0, 4 * 2 * (DST_WF_ROUNDS + 2), st));
    h->slices_used = 1;
    const bool wave = slots >= h->wf_min_rays;
    rc = dst_live_lists(h, slots, &p.lv, st);
    if (rc != DST_OK) return rc;
    const int g_compact = (int)((slots + DST_LIVE_BLOCK - 1) / DST_LIVE_BLOCK);
    p.rounds = wave ? DST_WF_ROUNDS : 0;
    p.min_count = wave ? (int)(slots / 512 > 2048 ? slots / 512 : 2048) : 1;
    // With the chunk log the rounds only serve rays the log could not hold. When the last completed read-back of a
    // forward of this shape shows that everything fitted, a dozen rounds are enqueued instead of all of them
    // (scheduling only: whatever is left after them is finished by the tail kernel).
    if (wave && use_log && h->log_known_needed > 0 && h->log_known_sig == dst_call_signature(&a->in) && h->log_known_needed <= h->log_cap)
        p.rounds = 12;
    dst_prof_mark(h, 2, 0, st);
    if (use_log) {
        // the forward kept its chunks: re-composite them; rays the log could not hold are queued as round 0 of the
        // re-trace below (normally none: the rounds then find an empty list and return at once)
        const unsigned int blocks = (unsigned int)((slots + BWD_THREADS - 1) / BWD_THREADS);
        if (dist) { if (diag) k_bwd_logged<true, true><<<blocks, BWD_THREADS, BWD_STAGE_BYTES, st>>>(p, slots); else k_bwd_logged<false, true><<<blocks, BWD_THREADS, BWD_STAGE_BYTES, st>>>(p, slots); }
        else { if (diag) k_bwd_logged<true, false><<<blocks, BWD_THREADS, BWD_STAGE_BYTES, st>>>(p, slots); else k_bwd_logged<false, false><<<blocks, BWD_THREADS, BWD_STAGE_BYTES, st>>>(p, slots); }
    } else {
        k_bwd_init<<<(unsigned int)((slots + 255) / 256), 256, 0, st>>>(p, slots);
    }
    const int g_enum = dst_wavefront_grid(h, slots, ENUM_THREADS, 10), g_shade = dst_wavefront_grid(h, slots, BWD_THREADS, 4);
    for (int r = 0; r < p.rounds; r++) {
        dst_prof_mark(h, 3, 0, st);
        launch_gather(diag, g_enum, st, p.bvh, p.req, p.list[r & 1], p.counts + r, p.counts + DST_WF_ROUNDS + 2 + r, p.min_count, p.kbuf, p.kcnt,
                      p.status, a->counters, r + 1, p.tiled != 0);
        dst_prof_mark(h, 3, 1, st);
        if (dist) { if (diag) k_bwd_shade<true, true><<<g_shade, BWD_THREADS, BWD_STAGE_BYTES, st>>>(p, r); else k_bwd_shade<false, true><<<g_shade, BWD_THREADS, BWD_STAGE_BYTES, st>>>(p, r); }
        else { if (diag) k_bwd_shade<true, false><<<g_shade, BWD_THREADS, BWD_STAGE_BYTES, st>>>(p, r); else k_bwd_shade<false, false><<<g_shade, BWD_THREADS, BWD_STAGE_BYTES, st>>>(p, r); }
        if (p.lv.stable) k_compact<<<g_compact, 256, 0, st>>>(p.lv, p.counts + r, p.counts + r + 1, p.min_count, p.list[(r + 1) & 1], r);
    }
    const int g_tail = dst_wavefront_grid(h, wave ? p.min_count : slots, BWD_THREADS, 4);
    if (dist) { if (diag) k_bwd_tail<true, true><<<g_tail, BWD_THREADS, BWD_STAGE_BYTES, st>>>(p); else k_bwd_tail<false, true><<<g_tail, BWD_THREADS, BWD_STAGE_BYTES, st>>>(p); }
    else { if (diag) k_bwd_tail<true, false><<<g_tail, BWD_THREADS, BWD_STAGE_BYTES, st>>>(p); else k_bwd_tail<false, false><<<g_tail, BWD_THREADS, BWD_STAGE_BYTES, st>>>(p); }
    dst_prof_mark(h, 2, 1, st);
    DST_CUDA_TRY(h, cudaGetLastError());
    k_unpack<<<(unsigned int)((P + 255) / 256), 256, 0, st>>>((int)P, h->arena, a->dL_drotations, a->dL_dmeans3D, a->dL_dopacities,
                                                              a->dL_dgrads3D, a->dL_dscales, a->dL_dothers, a->dL_dcolors);
    DST_CUDA_TRY(h, cudaGetLastError());
    h->launches += 3 + (p.lv.stable ? 3 : 2) * p.rounds;       // logged re-composite or ray init, the rounds, tail, unpack
    return DST_OK;
}
