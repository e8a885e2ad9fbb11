// Device code shared by the forward and backward trace kernels: the k-nearest hierarchy walk that
// replaces optixTrace + __anyhit__ot (optix_tracer/forward.cu:117-132, 481-525), the ray/ray-grid
// mapping, and spherical-harmonics colour.
#pragma once
#include "dst_common.cuh"

#define DST_STACK 96                 // >= depth bound of a Karras tree over 63-bit keys + 32-bit index tie-breaks
#define DST_MAX_CHUNKS 4096          // bound on enumerations per ray segment (the reference loops without one)
#define DST_MAX_INTERSECTION 256     // optix_tracer/config.h:23
#define DST_NODE_VOTE 10                // lanes with node work needed to stay in the node phase of k_enum
// The warp gives up walking together when fewer than this % of the lane tests are wanted. Pixel tiles: never. Measured on
// tiled image grids (forward, 0 / 10 / 25 %): 3M-surfel reflective scene 61.6 / 62.7 / 67.1 ms, object-scale scene 9.0 / 10.7 /
// 13.8 ms: even batches of reflected rays, whose directions have little in common, start from one small patch and find their
// 16 nearest hits close to it. Linear ray lists (LiDAR sweeps: one origin, directions fanning out over metres of a sparse
// scene) are the opposite case: 4.4 / 3.95 / 3.3 ms.
#ifndef DST_SHARE_MIN_PCT_TILED
#define DST_SHARE_MIN_PCT_TILED 0
#endif
#ifndef DST_SHARE_MIN_PCT_LINEAR
#define DST_SHARE_MIN_PCT_LINEAR 25
#endif
#ifndef DST_SHARE_VOTE
#define DST_SHARE_VOTE 1                // lanes that must want a subtree for the warp to walk it together (k_enum)
#endif
#define DST_PAD_FACTOR 4e-6f         // box padding per unit of coordinate magnitude, see knearest()

struct TraceCounters { unsigned long long segs, enums, nodes, quads, evals, contribs; };

__device__ __forceinline__ unsigned long long make_key(float t, unsigned int pidx) {
    return ((unsigned long long)__float_as_uint(t) << 32) | pidx;
}
__device__ __forceinline__ float hitkey_t(unsigned long long k) { return __uint_as_float((unsigned int)(k >> 32)); }

// The DST_CHUNK smallest (t, primitive id) hits with 0 <= t < 1e16 from origin o, ascending, in
// kb[0], kb[KS], kb[2 KS], ... (a column of a shared-memory array). Returns min(#hits, DST_CHUNK).
//
// Differences from the reference's scheme (every hit on the whole ray goes through an any-hit
// program that insertion-sorts into a 16-slot buffer): nodes and quads whose nearest possible t
// lies beyond the current 16th hit are culled, so the cost is that of a k-nearest query instead
// of growing with the number of hits behind the chunk.
//
// Conservativeness: a hit accepted by ray_quad() lies on the ray within ~20 ulp(M) of the quad,
// M = |o|_inf + largest |coordinate| of the scene. Child boxes are therefore padded by
// DST_PAD_FACTOR * M through the per-ray plane offsets (no extra work per node), which also
// covers the rounding of the slab arithmetic itself.
template <bool BRUTE, bool COUNT, int KS>
__device__ __forceinline__ int knearest(const BvhView& bvh, float ox, float oy, float oz, float dx, float dy, float dz,
                                        unsigned long long* kb, unsigned int* status, TraceCounters& tc,
                                        float kmax0 = DST_T_MAX) {
    int n = 0;
    float kmax = kmax0;          // hits beyond kmax0 are of no interest to the caller
    if (bvh.P <= 0) return 0;

    auto offer = [&](int pos) {
        const float4* qp = bvh.quads + 3 * (size_t)pos;
        const float4 qa = __ldg(qp), qb = __ldg(qp + 1), qc = __ldg(qp + 2);
        if (COUNT) tc.quads++;
        float t; int tri;
        if (!ray_quad(qa, qb, qc, ox, oy, oz, dx, dy, dz, kmax, t, tri)) return;
        const unsigned int gid = (unsigned int)__ldg(bvh.leaf_gid + pos);
        const unsigned long long key = make_key(t, 2u * gid + (unsigned int)tri);
        if (n == DST_CHUNK && key >= kb[(DST_CHUNK - 1) * KS]) return;
        int j = n;
        while (j > 0 && kb[(j - 1) * KS] > key) j--;
        if (n == DST_CHUNK) n = DST_CHUNK - 1;
        for (int i = n; i > j; i--) kb[i * KS] = kb[(i - 1) * KS];
        kb[j * KS] = key;
        n++;
        if (n == DST_CHUNK) kmax = hitkey_t(kb[(DST_CHUNK - 1) * KS]);
    };

    if (BRUTE) {
        for (int pos = 0; pos < bvh.P; pos++) offer(pos);
        return n;
    }

    const float omax = fmaxf(fabsf(ox), fmaxf(fabsf(oy), fabsf(oz)));
    if (!(omax < INFINITY)) return 0;
    const float pad = DST_PAD_FACTOR * (omax + __ldg(bvh.header + 6)) + 1e-30f;
    const float sdx = fabsf(dx) < 1e-20f ? copysignf(1e-20f, dx) : dx;
    const float sdy = fabsf(dy) < 1e-20f ? copysignf(1e-20f, dy) : dy;
    const float sdz = fabsf(dz) < 1e-20f ? copysignf(1e-20f, dz) : dz;
    const float ix = 1.0f / sdx, iy = 1.0f / sdy, iz = 1.0f / sdz;
    const bool px = !(sdx < 0.0f), py = !(sdy < 0.0f), pz = !(sdz < 0.0f);
    // entry plane t = near * i - on, exit plane t = far * i - of, with the padding folded in
    const float onx = fmaf(ox, ix, pad * fabsf(ix)), ofx = fmaf(ox, ix, -pad * fabsf(ix));
    const float ony = fmaf(oy, iy, pad * fabsf(iy)), ofy = fmaf(oy, iy, -pad * fabsf(iy));
    const float onz = fmaf(oz, iz, pad * fabsf(iz)), ofz = fmaf(oz, iz, -pad * fabsf(iz));

    unsigned long long stack[DST_STACK];
    int sp = 0;
    constexpr int DONE = 0x7fffffff;
    // pops the next subtree that can still hold a hit nearer than the 16th
    auto pop = [&]() -> int {
        while (sp > 0) {
            const unsigned long long e = stack[--sp];
            if (__uint_as_float((unsigned int)(e >> 32)) <= kmax) return (int)(unsigned int)e;
        }
        return DONE;
    };
    int cur = 0;
    for (;;) {
        // "while-while": lanes walk internal nodes until each holds a leaf (or is done), then test leaves together
        while ((unsigned int)cur < (unsigned int)DONE) {
            const float4* np = bvh.nodes + 4 * (size_t)cur;
            const float4 a = __ldg(np), b = __ldg(np + 1), c = __ldg(np + 2);
            const int4 lk = __ldg(reinterpret_cast<const int4*>(np + 3));
            if (COUNT) tc.nodes++;
            // child 0: lo (a.x a.y a.z) hi (a.w b.x b.y); child 1: lo (b.z b.w c.x) hi (c.y c.z c.w)
            const float n0x = px ? a.x : a.w, f0x = px ? a.w : a.x;
            const float n0y = py ? a.y : b.x, f0y = py ? b.x : a.y;
            const float n0z = pz ? a.z : b.y, f0z = pz ? b.y : a.z;
            const float n1x = px ? b.z : c.y, f1x = px ? c.y : b.z;
            const float n1y = py ? b.w : c.z, f1y = py ? c.z : b.w;
            const float n1z = pz ? c.x : c.w, f1z = pz ? c.w : c.x;
            const float tn0 = fmaxf(fmaxf(fmaf(n0x, ix, -onx), fmaf(n0y, iy, -ony)), fmaxf(fmaf(n0z, iz, -onz), 0.0f));
            const float tf0 = fminf(fminf(fmaf(f0x, ix, -ofx), fmaf(f0y, iy, -ofy)), fmaf(f0z, iz, -ofz));
            const float tn1 = fmaxf(fmaxf(fmaf(n1x, ix, -onx), fmaf(n1y, iy, -ony)), fmaxf(fmaf(n1z, iz, -onz), 0.0f));
            const float tf1 = fminf(fminf(fmaf(f1x, ix, -ofx), fmaf(f1y, iy, -ofy)), fmaf(f1z, iz, -ofz));
            const bool h0 = (tn0 <= tf0) && (tn0 <= kmax);
            const bool h1 = (tn1 <= tf1) && (tn1 <= kmax);
            if (h0 && h1) {
                const bool swap = tn1 < tn0 || (tn1 == tn0 && tf1 < tf0);      // entered first; on a tie (inside both boxes) left first
                const int cf = swap ? lk.z : lk.w;
                const float tfar = swap ? tn0 : tn1;
                if (sp < DST_STACK) stack[sp++] = ((unsigned long long)__float_as_uint(tfar) << 32) | (unsigned int)cf;
                else atomicOr(status, DST_STATUS_STACK_OVERFLOW);
                cur = swap ? lk.w : lk.z;
            } else if (h0) cur = lk.z;
            else if (h1) cur = lk.w;
            else cur = pop();
        }
        if (cur == DONE) break;
        {   // a run of leaves: test every quad of it
            const int first = DST_LEAF_FIRST(cur), count = DST_LEAF_COUNT(cur);
            for (int q = 0; q < count; q++) offer(first + q);
        }
        cur = pop();
    }
    return n;
}

// SH constants, optix_tracer/auxiliary.h:26-43
#define SHC0 0.28209479177387814f
#define SHC1 0.4886025119029199f
#define SHC2_0 1.0925484305920792f
#define SHC2_1 -1.0925484305920792f
#define SHC2_2 0.31539156525252005f
#define SHC2_3 -1.0925484305920792f
#define SHC2_4 0.5462742152960396f
#define SHC3_0 -0.5900435899266435f
#define SHC3_1 2.890611442640554f
#define SHC3_2 -0.4570457994644658f
#define SHC3_3 0.3731763325901154f
#define SHC3_4 -0.4570457994644658f
#define SHC3_5 1.445305721320277f
#define SHC3_6 -0.5900435899266435f

// loads the first 3*ncoef floats of a row of SH coefficients; vectorised when the row is 16-byte aligned
__device__ __forceinline__ void load_sh_row(const float* __restrict__ row, int nfloat, bool aligned, float* c) {
    if (aligned) {
        const float4* r4 = reinterpret_cast<const float4*>(row);
        const int nv = nfloat >> 2;
#pragma unroll
        for (int i = 0; i < 12; i++) {
            if (i < nv) { const float4 q = __ldg(r4 + i); c[4 * i] = q.x; c[4 * i + 1] = q.y; c[4 * i + 2] = q.z; c[4 * i + 3] = q.w; }
        }
#pragma unroll
        for (int i = 0; i < 48; i++) if (i >= (nv << 2) && i < nfloat) c[i] = __ldg(row + i);
    } else {
#pragma unroll
        for (int i = 0; i < 48; i++) if (i < nfloat) c[i] = __ldg(row + i);
    }
}

// Signed basis factors b[j] such that the reference's expression tree for the SH colour
// (optix_tracer/forward.cu:18-58) is r = b0*sh0; r = r + b[j]*sh[j] (j = 1..); r + 0.5; max(r, 0),
// one rounding per operation, in that order.
__device__ __forceinline__ void sh_basis(int deg, float x, float y, float z, float* b) {
    b[0] = SHC0;
    if (deg > 0) {
        b[1] = -xmul(SHC1, y); b[2] = xmul(SHC1, z); b[3] = -xmul(SHC1, x);
        if (deg > 1) {
            const float xx = xmul(x, x), yy = xmul(y, y), zz = xmul(z, z), xy = xmul(x, y), yz = xmul(y, z), xz = xmul(x, z);
            b[4] = xmul(SHC2_0, xy); b[5] = xmul(SHC2_1, yz);
            b[6] = xmul(SHC2_2, xsub(xsub(xmul(2.0f, zz), xx), yy));
            b[7] = xmul(SHC2_3, xz); b[8] = xmul(SHC2_4, xsub(xx, yy));
            if (deg > 2) {
                b[9] = xmul(xmul(SHC3_0, y), xsub(xmul(3.0f, xx), yy));
                b[10] = xmul(xmul(SHC3_1, xy), z);
                b[11] = xmul(xmul(SHC3_2, y), xsub(xsub(xmul(4.0f, zz), xx), yy));
                b[12] = xmul(xmul(SHC3_3, z), xsub(xsub(xmul(2.0f, zz), xmul(3.0f, xx)), xmul(3.0f, yy)));
                b[13] = xmul(xmul(SHC3_4, x), xsub(xsub(xmul(4.0f, zz), xx), yy));
                b[14] = xmul(xmul(SHC3_5, z), xsub(xx, yy));
                b[15] = xmul(xmul(SHC3_6, x), xsub(xx, xmul(3.0f, yy)));
            }
        }
    }
}

// unclamped colour channel ch (0..2) from the loaded coefficient row
__device__ __forceinline__ float sh_channel(int ncoef, const float* b, const float* c, int ch) {
    float r = xmul(b[0], c[ch]);
#pragma unroll
    for (int j = 1; j < 16; j++) if (j < ncoef) r = xadd(r, xmul(b[j], c[3 * j + ch]));
    return xadd(r, 0.5f);
}

// exp for x <= 0 as a fixed sequence of rounded operations (Cody-Waite reduction, degree-7 Taylor
// polynomial, exact power-of-two scaling): reproducible bit for bit on a CPU, about 1 ulp from a
// correctly rounded exp. The falloff G = exp(-rho/2) decides which hits contribute
// (optix_tracer/forward.cu:247-252), so it belongs to the exactly specified part.
__device__ __forceinline__ float pexp(float x) {
    if (!(x >= -87.0f)) return (x != x) ? x : 0.0f;
    if (x > 88.0f) x = 88.0f;
    const float kf = xsub(xadd(xmul(x, 1.44269504088896341f), 12582912.0f), 12582912.0f);
    float r = xfma(kf, -0.693145751953125f, x);
    r = xfma(kf, -1.42860682030941723212e-6f, r);
    float p = 0.0001984126984126984f;
    p = xfma(p, r, 0.001388888888888889f);
    p = xfma(p, r, 0.008333333333333333f);
    p = xfma(p, r, 0.041666666666666664f);
    p = xfma(p, r, 0.16666666666666666f);
    p = xfma(p, r, 0.5f);
    p = xfma(p, r, 1.0f);
    p = xfma(p, r, 1.0f);
    return xmul(p, __int_as_float(((int)kf + 127) << 23));
}

// Everything the compositing loop needs to know about one gathered hit.
struct SlotEval {
    float dpt, X, Y, Z;       // depth along the segment and world position
    float u, v;               // tangent-plane coordinates in units of the scales
    float nsign;              // +1 / -1: the normal is flipped toward the ray (DUAL_VISIABLE)
    float G, alpha;
    float4 r0, r1, r2, r3;    // the surfel's shading record
};

// Steps of optix_tracer/forward.cu:211-249 for one k-buffer entry, in the reference's operation
// order with one rounding per operation: depth, position, compute_transmat_uv (63-90), the
// visibility / near-depth / support tests and alpha. Returns false where the reference `continue`s.
// Shared by the forward and backward kernels so that the retrace takes identical decisions.
__device__ __forceinline__ bool eval_slot(unsigned long long key, float offset, float sox, float soy, float soz,
                                          float sdx, float sdy, float sdz, float min_depth, const float4* __restrict__ cache,
                                          int gidx, SlotEval& e) {
    e.dpt = xadd(hitkey_t(key), offset);
    e.X = xadd(sox, xmul(e.dpt, sdx)); e.Y = xadd(soy, xmul(e.dpt, sdy)); e.Z = xadd(soz, xmul(e.dpt, sdz));
    const float4* rec = cache + 4 * (size_t)gidx;
    e.r0 = __ldg(rec); e.r1 = __ldg(rec + 1); e.r2 = __ldg(rec + 2); e.r3 = __ldg(rec + 3);
    const float u1 = xadd(rdot3(e.r0.x, e.r0.y, e.r0.z, e.X, e.Y, e.Z), -e.r0.w);
    const float v1 = xadd(rdot3(e.r1.x, e.r1.y, e.r1.z, e.X, e.Y, e.Z), -e.r1.w);
    e.u = xdiv(u1, e.r3.x); e.v = xdiv(v1, e.r3.y);
    const float rho3d = xadd(xmul(e.u, e.u), xmul(e.v, e.v));
    const float cosv = -rdot3(sdx, sdy, sdz, e.r2.x, e.r2.y, e.r2.z);
    if (cosv == 0.0f) return false;
    e.nsign = cosv > 0.0f ? 1.0f : -1.0f;
    if (e.dpt < min_depth) return false;
    const float power = -0.5f * rho3d;
    if (power > 0.0f) return false;
    e.G = pexp(power);
    e.alpha = fminf(0.99f, xmul(e.r2.w, e.G));
    if (e.alpha < 1.0f / 255.0f) return false;
    return true;
}

// ---------------------------------------------------------------------------------------------
// Wavefront plumbing. A trace call runs as rounds of two kernels over the list of rays that are
// still alive: k_enum gathers the 16 nearest hits of each ray's current enumeration (small
// register footprint, every lane busy), a shade kernel composites them and decides what the ray
// does next. Ray state, hit buffers and the lists live in scratch memory owned by the handle.
// counts[r] is the length of list[r & 1] in round r; a round whose list is shorter than
// `min_count` is skipped by both kernels and left to the tail kernel, which runs the remaining
// rays to completion one thread per ray.
// ---------------------------------------------------------------------------------------------
struct __align__(16) EnumReq { float ox, oy, oz, dx, dy, dz, kmax0, pad; };

constexpr int ENUM_THREADS = 128;
#ifndef DST_ENUM_MIN_BLOCKS
#define DST_ENUM_MIN_BLOCKS 6         // resident blocks per SM the gather kernel is compiled for
#endif
#define DST_WF_ROUNDS 48
#define DST_COUNTS_STRIDE (2 * (DST_WF_ROUNDS + 2))      // ints per set of round counters: list lengths, then batch cursors

// Slab constants of one ray for the padded child-box test (see knearest()).
struct RaySlab {
    float ix, iy, iz, onx, ony, onz, ofx, ofy, ofz;
    bool px, py, pz, valid;
};
__device__ __forceinline__ RaySlab make_slab(float ox, float oy, float oz, float dx, float dy, float dz, float absmax) {
    RaySlab r;
    const float omax = fmaxf(fabsf(ox), fmaxf(fabsf(oy), fabsf(oz)));
    r.valid = omax < INFINITY;
    const float pad = DST_PAD_FACTOR * (omax + absmax) + 1e-30f;
    const float sdx = fabsf(dx) < 1e-20f ? copysignf(1e-20f, dx) : dx;
    const float sdy = fabsf(dy) < 1e-20f ? copysignf(1e-20f, dy) : dy;
    const float sdz = fabsf(dz) < 1e-20f ? copysignf(1e-20f, dz) : dz;
    r.ix = 1.0f / sdx; r.iy = 1.0f / sdy; r.iz = 1.0f / sdz;
    r.px = !(sdx < 0.0f); r.py = !(sdy < 0.0f); r.pz = !(sdz < 0.0f);
    r.onx = fmaf(ox, r.ix, pad * fabsf(r.ix)); r.ofx = fmaf(ox, r.ix, -pad * fabsf(r.ix));
    r.ony = fmaf(oy, r.iy, pad * fabsf(r.iy)); r.ofy = fmaf(oy, r.iy, -pad * fabsf(r.iy));
    r.onz = fmaf(oz, r.iz, pad * fabsf(r.iz)); r.ofz = fmaf(oz, r.iz, -pad * fabsf(r.iz));
    return r;
}

// Gather kernel: per live ray, the 16 nearest hits from the requested origin (same result as knearest()).
//
// A warp takes 32 consecutive entries of the live list: neighbouring pixels in the same stage (the lists keep their
// tile order, see k_compact), whose rays start close to each other. Large overlapping quads put hundreds of boxes
// around any origin, and every one of the 32 rays has to open them, so the walk is split in two:
//   shared phase   the warp walks the hierarchy TOGETHER from the root with one stack; a node is fetched once (one
//                  broadcast load instead of 32 scattered ones) and every lane tests its own ray against both
//                  child boxes. A child wanted by at least DST_SHARE_VOTE lanes (1: any lane, measured best) stays
//                  in the shared walk; a child wanted by fewer goes onto the private stacks of those lanes.
//                  A leaf run reached here is NOT tested quad by quad by every lane: lane q fetches quad q and
//                  decides, against the hull of the batch's rays (hull_quad), whether any ray of the batch can hit
//                  it; only the survivors (a few of 32 for neighbouring rays) are handed round and tested exactly
//                  by every lane. For linear ray lists only: when most lanes sit out most tests (after 64 nodes, under
//                  share_min_pct % of the lane x test slots wanted) the warp gives the shared walk up and every lane
//                  takes the pending subtrees onto its own stack (see DST_SHARE_MIN_PCT_TILED above).
//   private phase  every lane drains its own stack as in knearest(), lanes alternating between a node phase (kept
//                  while at least DST_NODE_VOTE lanes have node work) and a leaf phase.
// Pruning uses each lane's own 16th-nearest distance throughout (before a lane has 16 hits: the bound its request carries,
// see k_fwd_shade, or none) and the hull test is conservative, so the hit set is exactly that of an independent walk per
// ray within that bound. Blocks are persistent and take batches from a shared cursor.
#define DST_SHARED_STACK 64
#define DST_ENUM_STACK 160       // private stack of k_enum: subtrees deferred by the shared walk + one depth-first descent
#define DST_ENUM_DEFER 64        // the shared walk pauses to drain the private stacks when a lane holds this many entries
// Hull of the rays of one batch (origins and directions, component by component), kept in shared memory per warp.
struct BeamQ { float omin[3], omax[3], dmin[3], dmax[3], dabs[3], dsum; };      // dabs: largest |d| per axis, dsum: their sum

__device__ __forceinline__ unsigned int f2ord_q(float f) {
    const unsigned int u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ord2f_q(unsigned int u) { return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u); }
__device__ __forceinline__ float wmin_f(float v) { return ord2f_q(__reduce_min_sync(0xffffffffu, f2ord_q(v))); }
__device__ __forceinline__ float wmax_f(float v) { return ord2f_q(__reduce_max_sync(0xffffffffu, f2ord_q(v))); }

// [rl, rh] += c * [lo, hi]
__device__ __forceinline__ void ivmul(float c, float lo, float hi, float& rl, float& rh) {
    const bool pos = c >= 0.f;
    rl = fmaf(c, pos ? lo : hi, rl); rh = fmaf(c, pos ? hi : lo, rh);
}
// Conservative test of one quad against the hull of a batch of rays, in interval arithmetic over the hull's origins
// and directions: can ANY ray of the batch pass ray_quad() with a hit no farther than kmaxb? The steps are those of
// ray_quad(): t = n.(p0 - o) / n.d, h = t d - (p0 - o), u = wu.h, v = wv.h, accepted iff 0 <= t <= kmax and u, v in
// [0, 1]. Every interval is widened by margins orders of magnitude above the rounding of either computation, so a
// quad some ray hits is never rejected. For neighbouring rays (close origins, directions a degree apart) the
// intervals are narrow: nearly every quad that no ray hits is rejected here by ONE lane, and the lanes of a warp
// do that for 32 quads at a time, instead of every lane testing every quad against its own ray.
__device__ __forceinline__ bool hull_quad(const BeamQ& bm, const float4 qa, const float4 qb, const float4 qc, float kmaxb) {
    const float p0[3] = { qa.x, qa.y, qa.z }, nn[3] = { qa.w, qb.x, qb.y }, wu[3] = { qb.z, qb.w, qc.x }, wv[3] = { qc.y, qc.z, qc.w };
    float rl[3], rh[3];
    float bl = 0.f, bh = 0.f, al = 0.f, ah = 0.f, scale = 0.f;
#pragma unroll
    for (int a = 0; a < 3; a++) {
        rl[a] = p0[a] - bm.omax[a]; rh[a] = p0[a] - bm.omin[a];
        ivmul(nn[a], bm.dmin[a], bm.dmax[a], bl, bh);
        ivmul(nn[a], rl[a], rh[a], al, ah);
        scale = fmaxf(scale, fmaxf(fabsf(rl[a]), fabsf(rh[a])));
    }
    const float nmag = fabsf(nn[0]) + fabsf(nn[1]) + fabsf(nn[2]);
    const float eb = 4e-6f * nmag * bm.dsum, ea = 12e-6f * nmag * scale;
    bl -= eb; bh += eb; al -= ea; ah += ea;
    if (!(bl > 1e-30f || bh < -1e-30f)) return true;        // some direction of the hull is (all but) parallel to the plane: no bound
    // quotients by approximate reciprocals (two units in the last place; the interval is widened by 1e-5 relative below)
    const float ibl = __fdividef(1.0f, bl), ibh = __fdividef(1.0f, bh);
    const float t1 = al * ibl, t2 = al * ibh, t3 = ah * ibl, t4 = ah * ibh;
    float tl = fminf(fminf(t1, t2), fminf(t3, t4)), th = fmaxf(fmaxf(t1, t2), fmaxf(t3, t4));
    tl -= 1e-5f * fabsf(tl) + 1e-30f; th += 1e-5f * fabsf(th) + 1e-30f;
    if (th < 0.f || tl > kmaxb) return false;
    tl = fmaxf(tl, 0.f); th = fminf(th, kmaxb);
    float ul = 0.f, uh = 0.f, vl = 0.f, vh = 0.f, hmag = 0.f;
#pragma unroll
    for (int a = 0; a < 3; a++) {
        // t in [tl, th] with 0 <= tl <= th, d in [dmin, dmax]: the smallest t d is at (tl, dmin) or (th, dmin), the largest at (th, dmax) or (tl, dmax)
        const float hl = bm.dmin[a] * (bm.dmin[a] >= 0.f ? tl : th) - rh[a], hh = bm.dmax[a] * (bm.dmax[a] >= 0.f ? th : tl) - rl[a];
        ivmul(wu[a], hl, hh, ul, uh);
        ivmul(wv[a], hl, hh, vl, vh);
        hmag = fmaxf(hmag, fmaxf(fabsf(hl), fabsf(hh)) + scale + th * bm.dabs[a]);
    }
    // u and v are of order 1; their rounding error is that of h (cancellation of t d against p0 - o) times |w|
    const float eu = 1e-5f + 8e-6f * hmag * (fabsf(wu[0]) + fabsf(wu[1]) + fabsf(wu[2]));
    const float ev = 1e-5f + 8e-6f * hmag * (fabsf(wv[0]) + fabsf(wv[1]) + fabsf(wv[2]));
    return !(uh < -eu || ul > 1.f + eu || vh < -ev || vl > 1.f + ev);
}

#ifdef DST_ROUND_STATS
// build-time diagnostic: per wavefront round [0] batches, [1] shared node steps, [2] shared quad steps, [3] private
// node-phase warp steps, [4] private leaf-phase warp steps (quads), [5] batches that gave the shared walk up,
// [6] lane tests wanted in the shared phase, [7] lanes active at batch start
static __device__ unsigned long long g_round_stats[64][8];
#define RSTAT(i, v) do { const unsigned long long v_ = (v); if (lane == 0) rs[i] += v_; } while (0)      // v may hold a warp vote: every lane evaluates it
#else
#define RSTAT(i, v) do { } while (0)
#endif
template <bool COUNT>
__global__ void __launch_bounds__(ENUM_THREADS, DST_ENUM_MIN_BLOCKS) k_enum(BvhView bvh, const EnumReq* __restrict__ req, const int* __restrict__ list,
                                                       const int* __restrict__ count_ptr, int* cursor, int min_count,
                                                       unsigned long long* __restrict__ kbuf, int* __restrict__ kcnt,
                                                       unsigned int* status, unsigned long long* counters, int tag, int share_min_pct) {
    __shared__ unsigned long long kshared[DST_CHUNK * ENUM_THREADS];
    __shared__ int sstack[ENUM_THREADS / 32][DST_SHARED_STACK];
    __shared__ BeamQ sbeam[ENUM_THREADS / 32];
    const int total = *count_ptr;
    if (total < min_count || bvh.P <= 0) return;
    constexpr int KS = ENUM_THREADS;
    constexpr int DONE = 0x7fffffff;
    constexpr unsigned int FULL = 0xffffffffu;
    unsigned long long* kb = kshared + threadIdx.x;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const float absmax = __ldg(bvh.header + 6);
    TraceCounters tc = { 0, 0, 0, 0, 0, 0 };
#ifdef DST_ROUND_STATS
    unsigned long long rs[8] = { 0, 0, 0, 0, 0, 0, 0, 0 };
#endif
    unsigned long long stack[DST_ENUM_STACK];
    int sp = 0, n = 0;
    float kmax = -1.0f;
    float ox = 0.f, oy = 0.f, oz = 0.f, dx = 0.f, dy = 0.f, dz = 0.f;
    RaySlab sl = make_slab(0.f, 0.f, 0.f, 1.f, 1.f, 1.f, 0.f);

    auto pop = [&]() -> int {
        while (sp > 0) {
            const unsigned long long e = stack[--sp];
            if (__uint_as_float((unsigned int)(e >> 32)) <= kmax) return (int)(unsigned int)e;
        }
        return DONE;
    };
    auto push = [&](int link, float tn) {
        if (sp < DST_ENUM_STACK) stack[sp++] = ((unsigned long long)__float_as_uint(tn) << 32) | (unsigned int)link;
        else atomicOr(status, DST_STATUS_STACK_OVERFLOW);
    };
    // both child boxes of one node against this lane's ray
    auto test_node = [&](int node, float& tn0, float& tn1, bool& h0, bool& h1, int& l0, int& l1, bool& near1) {
        const float4* np = bvh.nodes + 4 * (size_t)node;
        const float4 a = __ldg(np), b = __ldg(np + 1), c = __ldg(np + 2);
        const int4 lk = __ldg(reinterpret_cast<const int4*>(np + 3));
        const float n0x = sl.px ? a.x : a.w, f0x = sl.px ? a.w : a.x;
        const float n0y = sl.py ? a.y : b.x, f0y = sl.py ? b.x : a.y;
        const float n0z = sl.pz ? a.z : b.y, f0z = sl.pz ? b.y : a.z;
        const float n1x = sl.px ? b.z : c.y, f1x = sl.px ? c.y : b.z;
        const float n1y = sl.py ? b.w : c.z, f1y = sl.py ? c.z : b.w;
        const float n1z = sl.pz ? c.x : c.w, f1z = sl.pz ? c.w : c.x;
        tn0 = fmaxf(fmaxf(fmaf(n0x, sl.ix, -sl.onx), fmaf(n0y, sl.iy, -sl.ony)), fmaxf(fmaf(n0z, sl.iz, -sl.onz), 0.0f));
        const float tf0 = fminf(fminf(fmaf(f0x, sl.ix, -sl.ofx), fmaf(f0y, sl.iy, -sl.ofy)), fmaf(f0z, sl.iz, -sl.ofz));
        tn1 = fmaxf(fmaxf(fmaf(n1x, sl.ix, -sl.onx), fmaf(n1y, sl.iy, -sl.ony)), fmaxf(fmaf(n1z, sl.iz, -sl.onz), 0.0f));
        const float tf1 = fminf(fminf(fmaf(f1x, sl.ix, -sl.ofx), fmaf(f1y, sl.iy, -sl.ofy)), fmaf(f1z, sl.iz, -sl.ofz));
        h0 = tn0 <= fminf(tf0, kmax);
        h1 = tn1 <= fminf(tf1, kmax);
        l0 = lk.z; l1 = lk.w;
        // which child first when both are wanted: the one entered first; when the ray starts inside both boxes (entry 0 for
        // both, the usual case among large overlapping quads) the one it leaves first, whose hits lie nearer on average.
        // Without the second rule child 0 (the lower coordinates) always went first on a tie, which is the far child for
        // every ray that travels towards lower coordinates: views along -x cost 50 % more than views along +x.
        near1 = tn1 < tn0 || (tn1 == tn0 && tf1 < tf0);
    };
    // exact test of one quad and insertion into this lane's k-buffer
    auto offer_quad = [&](const float4 qa, const float4 qb, const float4 qc, unsigned int gid) {
        float t; int tri;
        if (!ray_quad(qa, qb, qc, ox, oy, oz, dx, dy, dz, kmax, t, tri)) return;
        const unsigned long long key = make_key(t, 2u * gid + (unsigned int)tri);
        if (n == DST_CHUNK && key >= kb[(DST_CHUNK - 1) * KS]) return;
        int j = n;
        while (j > 0 && kb[(j - 1) * KS] > key) j--;
        if (n == DST_CHUNK) n = DST_CHUNK - 1;
        for (int i = n; i > j; i--) kb[i * KS] = kb[(i - 1) * KS];
        kb[j * KS] = key;
        n++;
        if (n == DST_CHUNK) kmax = hitkey_t(kb[(DST_CHUNK - 1) * KS]);
    };
    auto offer = [&](int pos) {
        const float4* qp = bvh.quads + 3 * (size_t)pos;
        offer_quad(__ldg(qp), __ldg(qp + 1), __ldg(qp + 2), (unsigned int)__ldg(bvh.leaf_gid + pos));
    };

    for (;;) {
        // ---- next batch of 32 list entries for this warp ----
        int base = 0;
        if (lane == 0) base = atomicAdd(cursor, 32);
        base = __shfl_sync(FULL, base, 0);
        if (base >= total) break;
        // The list is taken from its end: rays on a reflected segment come last in it (k_compact) and their batches are
        // the slow ones, so they start first and the cheap batches of primary rays fill the end of the round.
        const int idx = (((total + 31) >> 5) - 1 - (base >> 5)) * 32 + lane;
        int ray = idx < total ? list[idx] : -1;
        bool active = false;
        // takes up `ray`: request, slab constants, empty k-buffer and stack
        auto begin_ray = [&]() {
            n = 0; sp = 0; kmax = -1.0f;
            active = false;
            if (ray >= 0) {
                const float4 r0 = __ldg(reinterpret_cast<const float4*>(req + ray)), r1 = __ldg(reinterpret_cast<const float4*>(req + ray) + 1);
                ox = r0.x; oy = r0.y; oz = r0.z; dx = r0.w; dy = r1.x; dz = r1.y;
                sl = make_slab(ox, oy, oz, dx, dy, dz, absmax);
                active = sl.valid;
                if (active) kmax = r1.z;
                if (COUNT) tc.enums++;
            }
        };
        // writes the chunk of `ray` and lets go of it
        auto publish = [&]() {
            if (ray >= 0) {
                kcnt[ray] = n;
                ulonglong2* out = reinterpret_cast<ulonglong2*>(kbuf + (size_t)ray * DST_CHUNK);
#pragma unroll
                for (int k = 0; k < DST_CHUNK / 2; k++) {
                    if (2 * k < n) out[k] = make_ulonglong2(kb[(2 * k) * KS], kb[(2 * k + 1) * KS]);
                }
            }
            ray = -1;
        };
        begin_ray();
        RSTAT(0, 1); RSTAT(7, __popc(__ballot_sync(FULL, active)));
        {   // hull of the batch's rays, for culling the quads of leaf runs the warp reaches together
            const float o3[3] = { ox, oy, oz }, d3[3] = { dx, dy, dz };
#pragma unroll
            for (int a = 0; a < 3; a++) {
                const float lo = wmin_f(active ? o3[a] : INFINITY), hi = wmax_f(active ? o3[a] : -INFINITY);
                const float dl = wmin_f(active ? d3[a] : INFINITY), dh = wmax_f(active ? d3[a] : -INFINITY);
                if (lane == 0) { sbeam[wid].omin[a] = lo; sbeam[wid].omax[a] = hi; sbeam[wid].dmin[a] = dl; sbeam[wid].dmax[a] = dh; sbeam[wid].dabs[a] = fmaxf(fabsf(dl), fabsf(dh)); }
            }
            __syncwarp();
            if (lane == 0) sbeam[wid].dsum = sbeam[wid].dabs[0] + sbeam[wid].dabs[1] + sbeam[wid].dabs[2];
            __syncwarp();
        }
        int ssp = 0, scur = __any_sync(FULL, active) ? 0 : DONE;     // shared walk: stack pointer and current link (uniform)
        int s_tests = 0, s_wanted = 0;                                // child tests made together / of them wanted by their lane
        bool drain = false;                                           // (uniform) a private stack is about to fill up
        for (;;) {
        // ---- shared phase (left early when a private stack is about to fill up: deferred subtrees pile up there) ----
        if (scur != DONE) {
            for (;;) {
                if (drain) { drain = false; break; }                  // drain the private stacks first, then come back to scur
                if (share_min_pct > 0 && s_tests >= 64 * 32 && s_wanted * 100 < s_tests * share_min_pct && ssp + 1 <= DST_ENUM_STACK - DST_ENUM_DEFER - 40) {
                    // these rays do not travel together (most lanes sit out most tests): every lane takes the
                    // pending subtrees onto its own stack and the batch continues lane by lane
                    if (active) {
                        push(scur, 0.0f);
                        for (int e = 0; e < ssp; e++) push(sstack[wid][e], 0.0f);
                    }
                    ssp = 0; scur = DONE;
                    RSTAT(5, 1);
                    break;
                }
                if (scur >= 0) {
                    float tn0, tn1; bool h0, h1, near1; int l0, l1;
                    test_node(scur, tn0, tn1, h0, h1, l0, l1, near1);
                    if (COUNT && lane == 0) tc.nodes++;
                    const bool w0 = h0, w1 = h1;           // (a lane without a ray has kmax = -1 and every tn is >= 0: it never wants a child)
                    const unsigned int m0 = __ballot_sync(FULL, w0), m1 = __ballot_sync(FULL, w1);
                    if (share_min_pct > 0) { s_tests += 64; s_wanted += __popc(m0) + __popc(m1); }
                    RSTAT(1, 1); RSTAT(6, __popc(m0) + __popc(m1));
                    const bool s0 = DST_SHARE_VOTE <= 1 ? m0 != 0u : __popc(m0) >= DST_SHARE_VOTE, s1 = DST_SHARE_VOTE <= 1 ? m1 != 0u : __popc(m1) >= DST_SHARE_VOTE;
                    int next = DONE;
                    if (s0 && s1) {
                        // the majority of the lanes that want both decides which child comes first
                        const unsigned int pref1 = __ballot_sync(FULL, w0 && w1 && near1);
                        const bool first1 = 2 * __popc(pref1) > __popc(m0 & m1);
                        const int other = first1 ? l0 : l1;
                        if (ssp < DST_SHARED_STACK) { if (lane == 0) sstack[wid][ssp] = other; ssp++; }
                        else {                                                            // shared stack full: defer privately
                            if (first1 ? w0 : w1) push(other, first1 ? tn0 : tn1);
                            drain = __any_sync(FULL, sp >= DST_ENUM_DEFER);
                        }
                        next = first1 ? l1 : l0;
                    } else {
                        if (DST_SHARE_VOTE > 1) {
                            // children wanted by too few lanes go onto those lanes' own stacks (farther one first)
                            const bool d0 = w0 && !s0, d1 = w1 && !s1;
                            if (d0 && d1) { if (tn1 < tn0) { push(l0, tn0); push(l1, tn1); } else { push(l1, tn1); push(l0, tn0); } }
                            else if (d0) push(l0, tn0);
                            else if (d1) push(l1, tn1);
                            drain = __any_sync(FULL, sp >= DST_ENUM_DEFER);
                        }
                        if (s0) next = l0; else if (s1) next = l1;
                    }
                    if (next != DONE) { scur = next; continue; }
                } else {
                    // A run of leaves reached together. Lane q fetches quad q of the run and decides for the whole batch whether
                    // any of its rays can hit it (hull_quad); the few quads that pass are handed round and tested exactly
                    // by every lane against its own ray.
                    const int first = DST_LEAF_FIRST(scur), count = DST_LEAF_COUNT(scur);
                    if (count <= DST_HULL_MIN) {
                        for (int lq = 0; lq < count; lq++) {
                            if (COUNT && lane == 0) tc.quads++;
                            RSTAT(2, 1);
                            if (active) offer(first + lq);
                        }
                    } else {
                    const bool mine = lane < count;
                    float4 qa = make_float4(0.f, 0.f, 0.f, 0.f), qb = qa, qc = qa;
                    unsigned int qgid = 0u;
                    if (mine) {
                        const float4* qp = bvh.quads + 3 * (size_t)(first + lane);
                        qa = __ldg(qp); qb = __ldg(qp + 1); qc = __ldg(qp + 2);
                        qgid = (unsigned int)__ldg(bvh.leaf_gid + first + lane);
                    }
                    const float krun = wmax_f(kmax);        // (-1 on lanes without a ray)
                    unsigned int maybe = __ballot_sync(FULL, mine && hull_quad(sbeam[wid], qa, qb, qc, krun));
                    RSTAT(4, count);
                    while (maybe) {
                        const int src = __ffs(maybe) - 1;
                        maybe &= maybe - 1u;
                        const float4 sa = make_float4(__shfl_sync(FULL, qa.x, src), __shfl_sync(FULL, qa.y, src), __shfl_sync(FULL, qa.z, src), __shfl_sync(FULL, qa.w, src));
                        const float4 sb = make_float4(__shfl_sync(FULL, qb.x, src), __shfl_sync(FULL, qb.y, src), __shfl_sync(FULL, qb.z, src), __shfl_sync(FULL, qb.w, src));
                        const float4 sc = make_float4(__shfl_sync(FULL, qc.x, src), __shfl_sync(FULL, qc.y, src), __shfl_sync(FULL, qc.z, src), __shfl_sync(FULL, qc.w, src));
                        const unsigned int sg = __shfl_sync(FULL, qgid, src);
                        if (COUNT && lane == 0) tc.quads++;
                        RSTAT(2, 1);
                        if (active) offer_quad(sa, sb, sc, sg);
                    }
                    }
                }
                if (ssp == 0) { scur = DONE; break; }
                __syncwarp();
                scur = sstack[wid][--ssp];
                __syncwarp();
            }
        }
        // ---- private phase ----
        int cur = active ? pop() : DONE;
        for (;;) {
            const unsigned int busy = __ballot_sync(FULL, cur != DONE);
            if (busy == 0u) break;
            // node phase: kept while at least DST_NODE_VOTE lanes have node work or nobody holds a leaf
            for (;;) {
                const bool is_node = (unsigned int)cur < (unsigned int)DONE;
                const unsigned int m = __ballot_sync(FULL, is_node);
                if (m == 0u) break;
                if (__popc(m) < DST_NODE_VOTE && __any_sync(FULL, cur < 0)) break;
                RSTAT(3, 1);
                if (!is_node) continue;
                float tn0, tn1; bool h0, h1, near1; int l0, l1;
                test_node(cur, tn0, tn1, h0, h1, l0, l1, near1);
                if (COUNT) tc.nodes++;
                if (h0 && h1) {
                    const bool swap = near1;
                    push(swap ? l0 : l1, swap ? tn0 : tn1);
                    cur = swap ? l1 : l0;
                } else if (h0) cur = l0;
                else if (h1) cur = l1;
                else cur = pop();
            }
            // leaf phase
            if (cur < 0) {
                const int first = DST_LEAF_FIRST(cur), count = DST_LEAF_COUNT(cur);
                for (int lq = 0; lq < count; lq++) { if (COUNT) tc.quads++; offer(first + lq); }
                cur = pop();
            }
        }
        if (scur == DONE) break;
        }
        // ---- publish the chunks of this batch ----
        publish();
    }
    if (COUNT && counters) { atomicAdd(counters + 1, tc.enums); atomicAdd(counters + 2, tc.nodes); atomicAdd(counters + 3, tc.quads); }
#ifdef DST_ROUND_STATS
    if (lane == 0) for (int k = 0; k < 8; k++) if (rs[k]) atomicAdd(&g_round_stats[tag & 63][k], rs[k]);
#endif
}

// one gather launch of a wavefront round (diag: with traversal counters)
static inline void launch_gather(bool diag, int grid, cudaStream_t st, const BvhView& bvh, const EnumReq* req, const int* list,
                                 const int* count_ptr, int* cursor, int min_count, unsigned long long* kbuf, int* kcnt, unsigned int* status,
                                 unsigned long long* counters, int tag, bool tiled) {
    const int share_min_pct = tiled ? DST_SHARE_MIN_PCT_TILED : DST_SHARE_MIN_PCT_LINEAR;
    if (diag) k_enum<true><<<grid, ENUM_THREADS, 0, st>>>(bvh, req, list, count_ptr, cursor, min_count, kbuf, kcnt, status, counters, tag, share_min_pct);
    else k_enum<false><<<grid, ENUM_THREADS, 0, st>>>(bvh, req, list, count_ptr, cursor, min_count, kbuf, kcnt, status, nullptr, tag, share_min_pct);
}

// The 16 nearest hits of ONE ray, found by a whole warp (same result as knearest()). For the few rays the
// wavefront leaves to the tail kernel, and for small calls, what counts is the latency of a single walk:
// a thread on its own pays one dependent memory round trip per box and per quad. Here every step takes up
// to 16 entries from the top of a stack in shared memory (nearest first); leaf runs among them are tested
// 16 quads at a time, one quad per lane, and the nodes among them 32 child boxes at a time, one box per
// lane. The k-buffer lives in registers, one key per lane (lanes 0..15, ascending); an insertion is a
// ballot and a shuffle. All arguments are warp-uniform. `stack` holds DST_WARP_STACK entries.
#define DST_WARP_STACK 512
#define DST_WARP_STEP_LIMIT (1 << 20)      // bound on the steps of one walk (status flag instead of a hang)
template <bool COUNT>
__device__ __forceinline__ int knearest_warp(const BvhView& bvh, float ox, float oy, float oz, float dx, float dy, float dz,
                                             float kmax0, unsigned long long* stack, unsigned long long& mykey,
                                             unsigned int* status, TraceCounters& tc) {
    constexpr unsigned int FULL = 0xffffffffu;
    constexpr unsigned long long EMPTY = ~0ull;
    const int lane = threadIdx.x & 31;
    mykey = EMPTY;
    int n = 0;
    float kmax = kmax0;
    if (bvh.P <= 0) return 0;
    const RaySlab sl = make_slab(ox, oy, oz, dx, dy, dz, __ldg(bvh.header + 6));
    if (!sl.valid) return 0;
    // inserts a hit (uniform key) into the sorted keys held by lanes 0..15
    auto insert = [&](unsigned long long key) {
        const unsigned long long last = __shfl_sync(FULL, mykey, DST_CHUNK - 1);
        if (key >= last) return;                                            // not among the 16 nearest (or the buffer is full of nearer ones)
        const int pos = __popc(__ballot_sync(FULL, lane < DST_CHUNK && mykey < key));
        const unsigned long long up = __shfl_up_sync(FULL, mykey, 1);
        if (lane < DST_CHUNK) mykey = lane < pos ? mykey : (lane == pos ? key : up);
        if (n < DST_CHUNK) n++;
        if (n == DST_CHUNK) kmax = hitkey_t(__shfl_sync(FULL, mykey, DST_CHUNK - 1));
    };
    int sp = 0;
    if (lane == 0) stack[0] = 0ull;            // the root: nearest possible t 0, link 0
    sp = 1;
    __syncwarp();
    for (int step = 0; sp > 0; step++) {
        if (step >= DST_WARP_STEP_LIMIT) { if (lane == 0) atomicOr(status, DST_STATUS_STACK_OVERFLOW); break; }
        // lanes 30/31 take the top entry, lanes 28/29 the next, ...: lane order is then the order in which
        // surviving children go back onto the stack (farthest first)
        const int take = sp < 16 ? sp : 16;
        const int slot = 15 - (lane >> 1);                                  // 0 = top of the stack
        unsigned long long e = 0ull;
        bool valid = slot < take;
        if (valid) e = stack[sp - 1 - slot];
        sp -= take;
        __syncwarp();
        const int link = (int)(unsigned int)e;
        valid = valid && __uint_as_float((unsigned int)(e >> 32)) <= kmax;
        // ---- leaf runs among the entries, nearest first ----
        unsigned int leaves = __ballot_sync(FULL, valid && link < 0 && (lane & 1) == 1);
        while (leaves) {
            const int src = 31 - __clz(leaves);                             // highest lane = nearest entry
            leaves &= ~(1u << src);
            const int lnk = __shfl_sync(FULL, link, src);
            const float etn = __uint_as_float((unsigned int)(__shfl_sync(FULL, e, src) >> 32));
            if (etn > kmax) continue;                                       // the bound has shrunk meanwhile
            const int first = DST_LEAF_FIRST(lnk), count = DST_LEAF_COUNT(lnk);
            for (int base = 0; base < count; base += 32) {
                bool hit = false;
                unsigned long long key = 0ull;
                if (base + lane < count) {
                    const int pos = first + base + lane;
                    const float4* qp = bvh.quads + 3 * (size_t)pos;
                    const float4 qa = __ldg(qp), qb = __ldg(qp + 1), qc = __ldg(qp + 2);
                    float t; int tri;
                    if (ray_quad(qa, qb, qc, ox, oy, oz, dx, dy, dz, kmax, t, tri)) {
                        const unsigned int gid = (unsigned int)__ldg(bvh.leaf_gid + pos);
                        key = make_key(t, 2u * gid + (unsigned int)tri);
                        hit = true;
                    }
                }
                if (COUNT && lane == 0) tc.quads += (unsigned long long)(count - base < 32 ? count - base : 32);
                unsigned int hits = __ballot_sync(FULL, hit);
                while (hits) {
                    const int hl = __ffs(hits) - 1;
                    hits &= hits - 1u;
                    insert(__shfl_sync(FULL, key, hl));
                }
            }
        }
        // ---- nodes among the entries: one child box per lane ----
        bool h = false;
        float tn = 0.0f, tf = 0.0f;
        int clink = 0;
        if (valid && link >= 0 && __uint_as_float((unsigned int)(e >> 32)) <= kmax) {
            const float4* np = bvh.nodes + 4 * (size_t)link;
            const float4 a = __ldg(np), b = __ldg(np + 1), c = __ldg(np + 2);
            const int4 lk = __ldg(reinterpret_cast<const int4*>(np + 3));
            float lox, loy, loz, hix, hiy, hiz;
            if ((lane & 1) == 0) { lox = a.x; loy = a.y; loz = a.z; hix = a.w; hiy = b.x; hiz = b.y; clink = lk.z; }
            else { lox = b.z; loy = b.w; loz = c.x; hix = c.y; hiy = c.z; hiz = c.w; clink = lk.w; }
            const float nx = sl.px ? lox : hix, fx = sl.px ? hix : lox;
            const float ny = sl.py ? loy : hiy, fy = sl.py ? hiy : loy;
            const float nz = sl.pz ? loz : hiz, fz = sl.pz ? hiz : loz;
            tn = fmaxf(fmaxf(fmaf(nx, sl.ix, -sl.onx), fmaf(ny, sl.iy, -sl.ony)), fmaxf(fmaf(nz, sl.iz, -sl.onz), 0.0f));
            tf = fminf(fminf(fmaf(fx, sl.ix, -sl.ofx), fmaf(fy, sl.iy, -sl.ofy)), fmaf(fz, sl.iz, -sl.ofz));
            h = (tn <= tf) && (tn <= kmax);
            if (COUNT && (lane & 1) == 0) tc.nodes++;
        }
        // within a pair the farther child goes first (even lane), the nearer second (odd lane)
        {
            const float ptn = __shfl_xor_sync(FULL, tn, 1), ptf = __shfl_xor_sync(FULL, tf, 1);
            const int plink = __shfl_xor_sync(FULL, clink, 1);
            const bool ph = __shfl_xor_sync(FULL, h, 1);
            const bool even = (lane & 1) == 0;
            // nearer = entered first, on a tie (the ray starts inside both boxes) left first
            const bool mine_nearer = tn < ptn || (tn == ptn && (tf < ptf || (tf == ptf && even)));
            if (h && ph && (even ? mine_nearer : !mine_nearer)) { tn = ptn; clink = plink; }
        }
        const unsigned int pushes = __ballot_sync(FULL, h);
        const int npush = __popc(pushes);
        if (sp + npush > DST_WARP_STACK) {
            if (lane == 0) atomicOr(status, DST_STATUS_STACK_OVERFLOW);
            break;
        }
        if (h) stack[sp + __popc(pushes & ((1u << lane) - 1u))] = ((unsigned long long)__float_as_uint(tn) << 32) | (unsigned int)clink;
        sp += npush;
        __syncwarp();
    }
    return n;
}

// List entry i of round 0 -> ray index (or -1). Image-like grids are walked in 8x4 pixel tiles (one tile = the 32
// rays a warp of the gather kernel takes), and the tiles in Z order inside blocks of 8x8 tiles (64x32 pixels): any
// aligned run of 2 or 4 consecutive tiles is a compact 16x4 or 16x8 pixel patch. That matters once rays have
// dropped out: the lists keep this order, so a warp of a later round holds the survivors of a few consecutive
// tiles, and the tighter the patch they come from, the tighter the hull of their rays. Batched ray lists (few rows)
// are walked linearly.
#ifndef DST_TILE_BLOCK
#define DST_TILE_BLOCK 8              // tiles per side of a Z-ordered block (1: row-major tile order)
#endif
__device__ __forceinline__ int ray_of_slot(long long i, int H, int W, bool tiled) {
    if (!tiled) return i < (long long)H * W ? (int)i : -1;
    const int tiles_x = (W + 7) >> 3;
    long long tile = i >> 5;
    const int lane = (int)(i & 31);
    int tx, ty;
    if (DST_TILE_BLOCK > 1) {
        constexpr int BB = DST_TILE_BLOCK * DST_TILE_BLOCK;
        const int blocks_x = (tiles_x + DST_TILE_BLOCK - 1) / DST_TILE_BLOCK;
        const long long blk = tile / BB;
        const unsigned int in = (unsigned int)(tile - blk * BB);
        // Z order inside the block: even bits -> x, odd bits -> y
        const unsigned int zx = (in & 1u) | ((in >> 1) & 2u) | ((in >> 2) & 4u), zy = ((in >> 1) & 1u) | ((in >> 2) & 2u) | ((in >> 3) & 4u);
        tx = (int)(blk % blocks_x) * DST_TILE_BLOCK + (int)zx;
        ty = (int)(blk / blocks_x) * DST_TILE_BLOCK + (int)zy;
    } else { tx = (int)(tile % tiles_x); ty = (int)(tile / tiles_x); }
    const int x = tx * 8 + (lane & 7);
    const int y = ty * 4 + (lane >> 3);
    if (x >= W || y >= H) return -1;
    return y * W + x;
}
__host__ __device__ __forceinline__ long long slots_of_grid(int H, int W, bool tiled) {
    if (!tiled) return (long long)H * W;
    const long long tiles_x = (W + 7) >> 3, tiles_y = (H + 3) >> 2;
    if (DST_TILE_BLOCK > 1) {
        const long long bx = (tiles_x + DST_TILE_BLOCK - 1) / DST_TILE_BLOCK, by = (tiles_y + DST_TILE_BLOCK - 1) / DST_TILE_BLOCK;
        return bx * by * DST_TILE_BLOCK * DST_TILE_BLOCK * 32;
    }
    return tiles_x * tiles_y * 32;
}

// appends `ray` to the next round's list when `alive`; one atomic per warp, order kept within a warp
__device__ __forceinline__ void append_alive(bool alive, int ray, int* __restrict__ next_list, int* next_count) {
    __syncwarp();
    const unsigned int m = __ballot_sync(__activemask(), alive);
    if (!alive) return;
    const int lane = threadIdx.x & 31;
    const int leader = __ffs(m) - 1;
    int base = 0;
    if (lane == leader) base = atomicAdd(next_count, __popc(m));
    base = __shfl_sync(m, base, leader);
    next_list[base + __popc(m & ((1u << lane) - 1u))] = ray;
}

// ---------------------------------------------------------------------------------------------
// Order-preserving hand-over of the live list from one round to the next.
//
// append_alive() above packs the survivors of every warp behind one atomic counter: cheap, but the
// warps arrive in whatever order the scheduler ran them, so after a few rounds neighbouring list
// entries are unrelated rays and the gather kernel's shared walk (one hierarchy walk for 32
// neighbouring rays) falls apart. The stable form keeps the list in its original order (8x4 pixel
// tiles, tile after tile) and, within that, puts rays on their primary segment before rays on a
// reflected one, so that a warp of the next round again holds rays that start close together and
// are in the same stage:
//   shade kernel   live_out(): survivor (or -1) of list position i into tmp[i]; survivors per warp
//                  and class into wcnt[i / 32]; the same added to the counter of the 4096-entry
//                  block the position lies in (bcnt, two classes packed 16 + 16 bits).
//   k_compact      one block per 4096 positions: sums the block counters before its own (and all of
//                  them, for the start of the second class), scans its 128 warp counts and copies
//                  every survivor to its final position. Block 0 publishes the new list length.
// The block counters come in two sets used by alternate rounds; k_compact of round r clears the set
// round r + 1 accumulates into (nothing waits on anything: all of this is ordinary stream order).
// ---------------------------------------------------------------------------------------------
#define DST_LIVE_BLOCK 4096
#define DST_LIVE_CLASS_BIT 30            // ray indices stay below 2^30 (checked on the host)
struct LiveLists {
    int* tmp;            // per list position of the current round: ray | class << 30, or -1
    int* wcnt;           // per 32 positions: survivors of class 0 | survivors of class 1 << 16
    int* bcnt[2];        // per DST_LIVE_BLOCK positions, same packing; set (round & 1) belongs to the current round
    int stable;          // 0: append_alive() order (atomic per warp)
};
static inline long long dst_live_blocks(long long slots) { return slots / DST_LIVE_BLOCK + 2; }
int dst_live_lists(dst_handle* h, long long slots, LiveLists* lv, cudaStream_t st);

// called by all 32 lanes of a warp for 32 consecutive list positions (i of lane 0 is a multiple of 32)
__device__ __forceinline__ void live_out(const LiveLists& lv, int round, int i, bool alive, int ray, int cls) {
    __syncwarp();
    const unsigned int m0 = __ballot_sync(0xffffffffu, alive && cls == 0), m1 = __ballot_sync(0xffffffffu, alive && cls != 0);
    lv.tmp[i] = alive ? (ray | (cls != 0 ? (1 << DST_LIVE_CLASS_BIT) : 0)) : -1;
    if ((threadIdx.x & 31) == 0) {
        const int packed = __popc(m0) | (__popc(m1) << 16);
        lv.wcnt[i >> 5] = packed;
        if (packed) atomicAdd(lv.bcnt[round & 1] + i / DST_LIVE_BLOCK, packed);
    }
}

static __global__ void __launch_bounds__(256) k_compact(LiveLists lv, const int* __restrict__ count_ptr, int* next_count, int min_count,
                                                        int* __restrict__ next_list, int round) {
    __shared__ int red[4][8];
    __shared__ int woff[DST_LIVE_BLOCK / 32];
    const int n = *count_ptr;
    if (n < min_count) return;
    const int nb = (n + DST_LIVE_BLOCK - 1) / DST_LIVE_BLOCK;
    const int b = blockIdx.x;
    if (b >= nb) return;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int* bc = lv.bcnt[round & 1];
    // survivors per class in the blocks before this one, and in all blocks
    int before0 = 0, before1 = 0, all0 = 0, all1 = 0;
    for (int j = threadIdx.x; j < nb; j += 256) {
        const int c = bc[j], c0 = c & 0xffff, c1 = c >> 16;
        all0 += c0; all1 += c1;
        if (j < b) { before0 += c0; before1 += c1; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        before0 += __shfl_xor_sync(0xffffffffu, before0, o); before1 += __shfl_xor_sync(0xffffffffu, before1, o);
        all0 += __shfl_xor_sync(0xffffffffu, all0, o); all1 += __shfl_xor_sync(0xffffffffu, all1, o);
    }
    if (lane == 0) { red[0][w] = before0; red[1][w] = before1; red[2][w] = all0; red[3][w] = all1; }
    // exclusive scan of this block's 128 warp counts (both classes in one packed add: sums stay below 2^16)
    const int wpos = b * (DST_LIVE_BLOCK / 32) + threadIdx.x;
    int x = 0;
    if (threadIdx.x < DST_LIVE_BLOCK / 32 && wpos * 32 < n) x = lv.wcnt[wpos];
    int incl = x;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += y; }
    __shared__ int wsum[8];
    if (lane == 31) wsum[w] = incl;
    __syncthreads();
    before0 = before1 = all0 = all1 = 0;
#pragma unroll
    for (int k = 0; k < 8; k++) { before0 += red[0][k]; before1 += red[1][k]; all0 += red[2][k]; all1 += red[3][k]; }
    if (threadIdx.x < DST_LIVE_BLOCK / 32) {
        int carry = 0;
        for (int k = 0; k < w; k++) carry += wsum[k];
        woff[threadIdx.x] = carry + incl - x;
    }
    __syncthreads();
    if (b == 0 && threadIdx.x == 0) *next_count = all0 + all1;
    if (threadIdx.x == 0) lv.bcnt[(round + 1) & 1][b] = 0;          // the set the next round accumulates into
    // every warp copies 16 groups of 32 positions
    for (int g = w; g < DST_LIVE_BLOCK / 32; g += 8) {
        const int i = (b * (DST_LIVE_BLOCK / 32) + g) * 32 + lane;
        const int v = i < n ? lv.tmp[i] : -1;          // positions up to the next multiple of 32 were written, the rest is dead
        const bool alive = v >= 0;
        const bool second = alive && ((v >> DST_LIVE_CLASS_BIT) & 1);
        const unsigned int m0 = __ballot_sync(0xffffffffu, alive && !second), m1 = __ballot_sync(0xffffffffu, second);
        if (!alive) continue;
        const int off = woff[g], below = (1u << lane) - 1u;
        const int pos = second ? all0 + before1 + (off >> 16) + __popc(m1 & below) : before0 + (off & 0xffff) + __popc(m0 & below);
        next_list[pos] = v & ((1 << DST_LIVE_CLASS_BIT) - 1);
    }
}

// first round the wavefront kernels left alone (list shorter than min_count)
__device__ __forceinline__ int first_skipped_round(const int* __restrict__ counts, int rounds, int min_count) {
    for (int r = 0; r < rounds; r++) if (counts[r] < min_count) return r;
    return rounds;
}
