// Hierarchy build / refit over surfel quads: replaces optixAccelBuild as called from
// trace_surfels.cpp:36-159 (OPERATION_BUILD when rebuild > 0, OPERATION_UPDATE otherwise).
//
// Build:  centroid bounds -> 63-bit Morton keys -> LSD radix sort (8 x 8-bit passes, 64-bit key /
//         32-bit value) -> Karras hierarchy -> bottom-up box pass (also writes the per-quad plane
//         frames in leaf order).
// Refit:  the bottom-up pass alone, on the topology and leaf order of the last build.
// All kernels are plain HBM-bound streaming / scatter kernels; nothing waits on another block
// (the bottom-up pass uses arrival counters: the first thread to reach a node leaves, the second
// continues), so there is no device-side spin anywhere.
#include "dst_common.cuh"
#include <math.h>

namespace {

constexpr int SORT_THREADS = 256;
constexpr int SORT_ITEMS = 16;
constexpr int SORT_TILE = SORT_THREADS * SORT_ITEMS;   // 4096 keys per block
constexpr int SORT_WARPS = SORT_THREADS / 32;

__device__ __forceinline__ unsigned int f2ord(float f) {
    unsigned int u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ord2f(unsigned int u) {
    return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

// words 0..2: min of quad-box centres, 3..5: max (ordered-uint encoding)
__global__ void k_init_bounds(unsigned int* bw) {
    if (threadIdx.x < 3) bw[threadIdx.x] = 0xffffffffu;
    else if (threadIdx.x < 6) bw[threadIdx.x] = 0u;
}

__device__ __forceinline__ void quad_box(const float* __restrict__ v, float* lo, float* hi) {
#pragma unroll
    for (int a = 0; a < 3; a++) {
        lo[a] = fminf(fminf(v[a], v[3 + a]), fminf(v[6 + a], v[9 + a]));
        hi[a] = fmaxf(fmaxf(v[a], v[3 + a]), fmaxf(v[6 + a], v[9 + a]));
    }
}

__global__ void __launch_bounds__(256) k_centre_bounds(const float* __restrict__ verts, int P, unsigned int* bw) {
    float lo[3] = { INFINITY, INFINITY, INFINITY }, hi[3] = { -INFINITY, -INFINITY, -INFINITY };
    for (int g = blockIdx.x * blockDim.x + threadIdx.x; g < P; g += gridDim.x * blockDim.x) {
        float v[12];
        const float4* p = reinterpret_cast<const float4*>(verts + 12 * (size_t)g);
        float4 a = __ldg(p), b = __ldg(p + 1), c = __ldg(p + 2);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        v[8] = c.x; v[9] = c.y; v[10] = c.z; v[11] = c.w;
        float l[3], h[3];
        quad_box(v, l, h);
#pragma unroll
        for (int a2 = 0; a2 < 3; a2++) {
            float cc = 0.5f * (l[a2] + h[a2]);
            if (isfinite(cc)) { lo[a2] = fminf(lo[a2], cc); hi[a2] = fmaxf(hi[a2], cc); }
        }
    }
#pragma unroll
    for (int a = 0; a < 3; a++) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            lo[a] = fminf(lo[a], __shfl_xor_sync(0xffffffffu, lo[a], o));
            hi[a] = fmaxf(hi[a], __shfl_xor_sync(0xffffffffu, hi[a], o));
        }
    }
    if ((threadIdx.x & 31) == 0) {
#pragma unroll
        for (int a = 0; a < 3; a++) {
            if (lo[a] <= hi[a]) { atomicMin(&bw[a], f2ord(lo[a])); atomicMax(&bw[3 + a], f2ord(hi[a])); }
        }
    }
}

__device__ __forceinline__ unsigned long long spread21(unsigned long long x) {
    x &= 0x1fffffull;
    x = (x | x << 32) & 0x1f00000000ffffull;
    x = (x | x << 16) & 0x1f0000ff0000ffull;
    x = (x | x << 8) & 0x100f00f00f00f00full;
    x = (x | x << 4) & 0x10c30c30c30c30c3ull;
    x = (x | x << 2) & 0x1249249249249249ull;
    return x;
}

__global__ void __launch_bounds__(256) k_morton(const float* __restrict__ verts, int P, const unsigned int* __restrict__ bw,
                                                unsigned long long* __restrict__ keys, unsigned int* __restrict__ vals) {
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= P) return;
    float v[12];
    const float4* p = reinterpret_cast<const float4*>(verts + 12 * (size_t)g);
    float4 a = __ldg(p), b = __ldg(p + 1), c = __ldg(p + 2);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    v[8] = c.x; v[9] = c.y; v[10] = c.z; v[11] = c.w;
    float l[3], h[3];
    quad_box(v, l, h);
    unsigned long long key = 0;
#pragma unroll
    for (int ax = 0; ax < 3; ax++) {
        const float lo = ord2f(bw[ax]), hi = ord2f(bw[3 + ax]);
        const float ext = hi - lo;
        float cc = 0.5f * (l[ax] + h[ax]);
        float q = (ext > 0.0f && isfinite(cc)) ? (cc - lo) / ext * 2097152.0f : 0.0f;
        q = fminf(fmaxf(q, 0.0f), 2097151.0f);
        key |= spread21((unsigned long long)(unsigned int)q) << (2 - ax);
    }
    keys[g] = key;
    vals[g] = (unsigned int)g;
}

// ---- LSD radix sort, one 8-bit digit per pass --------------------------------------------------
__global__ void __launch_bounds__(SORT_THREADS) k_sort_hist(const unsigned long long* __restrict__ keys, int n, int shift,
                                                            unsigned int* __restrict__ block_hist, int nblocks) {
    __shared__ unsigned int sh[256];
    sh[threadIdx.x] = 0;
    __syncthreads();
    const int base = blockIdx.x * SORT_TILE;
#pragma unroll
    for (int i = 0; i < SORT_ITEMS; i++) {
        const int idx = base + i * SORT_THREADS + threadIdx.x;
        if (idx < n) atomicAdd(&sh[(unsigned int)(keys[idx] >> shift) & 255u], 1u);
    }
    __syncthreads();
    block_hist[threadIdx.x * nblocks + blockIdx.x] = sh[threadIdx.x];
}

// Exclusive scan of the per-block counts of ONE digit (block d of the grid takes digit d): block_hist[d][0..nblocks)
// becomes the number of keys with digit d in the blocks before, and digit_total[d] their number in all blocks. The
// scatter kernel adds the keys with smaller digits itself (a 256-entry scan every block repeats), so no block of any
// kernel waits for another and no single block walks all 256 x nblocks counters.
__global__ void __launch_bounds__(256) k_sort_scan(unsigned int* __restrict__ block_hist, int nblocks, unsigned int* __restrict__ digit_total) {
    __shared__ unsigned int warp_sum[8];
    __shared__ unsigned int carry_s;
    unsigned int* data = block_hist + (size_t)blockIdx.x * nblocks;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    for (int base = 0; base < nblocks; base += 256) {
        const int idx = base + threadIdx.x;
        unsigned int x = idx < nblocks ? data[idx] : 0u, incl = x;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { unsigned int y = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += y; }
        if (lane == 31) warp_sum[wid] = incl;
        __syncthreads();
        unsigned int before = 0;
#pragma unroll
        for (int k = 0; k < 8; k++) if (k < wid) before += warp_sum[k];
        const unsigned int carry = carry_s;
        if (idx < nblocks) data[idx] = carry + before + incl - x;
        __syncthreads();
        if (threadIdx.x == 255) carry_s = carry + before + incl;
        __syncthreads();
    }
    if (threadIdx.x == 0) digit_total[blockIdx.x] = carry_s;
}

// stable scatter: warp w of a block owns 512 consecutive keys and ranks them 32 at a time
__global__ void __launch_bounds__(SORT_THREADS) k_sort_scatter(const unsigned long long* __restrict__ keys_in,
                                                               const unsigned int* __restrict__ vals_in,
                                                               unsigned long long* __restrict__ keys_out,
                                                               unsigned int* __restrict__ vals_out, int n, int shift,
                                                               const unsigned int* __restrict__ block_offs, int nblocks,
                                                               const unsigned int* __restrict__ digit_total) {
    __shared__ unsigned int wc[SORT_WARPS][257];
    __shared__ unsigned int digit_base[256];
    __shared__ unsigned int dsum[SORT_WARPS];
    {   // keys with a smaller digit, in all blocks: exclusive scan of the 256 digit totals
        const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
        const unsigned int x = digit_total[threadIdx.x];
        unsigned int incl = x;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { unsigned int y = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += y; }
        if (lane == 31) dsum[w] = incl;
        __syncthreads();
        unsigned int before = 0;
#pragma unroll
        for (int k = 0; k < SORT_WARPS; k++) if (k < w) before += dsum[k];
        digit_base[threadIdx.x] = before + incl - x;
    }
    for (int i = threadIdx.x; i < SORT_WARPS * 257; i += SORT_THREADS) (&wc[0][0])[i] = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int base = blockIdx.x * SORT_TILE + w * (SORT_ITEMS * 32);
    unsigned long long key[SORT_ITEMS];
    unsigned int val[SORT_ITEMS];
    unsigned short rank[SORT_ITEMS];
#pragma unroll
    for (int s = 0; s < SORT_ITEMS; s++) {
        const int idx = base + s * 32 + lane;
        const bool valid = idx < n;
        key[s] = valid ? keys_in[idx] : ~0ull;
        val[s] = valid ? vals_in[idx] : 0u;
        const unsigned int d = valid ? ((unsigned int)(key[s] >> shift) & 255u) : 256u;
        const unsigned int mask = __match_any_sync(0xffffffffu, d);
        const int leader = __ffs(mask) - 1;
        unsigned int old = 0;
        if (lane == leader) { old = wc[w][d]; wc[w][d] = old + __popc(mask); }
        old = __shfl_sync(0xffffffffu, old, leader);
        rank[s] = (unsigned short)(old + __popc(mask & ((1u << lane) - 1u)));
    }
    __syncthreads();
    {
        const int d = threadIdx.x;     // SORT_THREADS == 256 digits
        unsigned int sum = digit_base[d] + block_offs[d * nblocks + blockIdx.x];
#pragma unroll
        for (int ww = 0; ww < SORT_WARPS; ww++) { unsigned int c = wc[ww][d]; wc[ww][d] = sum; sum += c; }
    }
    __syncthreads();
#pragma unroll
    for (int s = 0; s < SORT_ITEMS; s++) {
        const int idx = base + s * 32 + lane;
        if (idx < n) {
            const unsigned int d = (unsigned int)(key[s] >> shift) & 255u;
            const unsigned int pos = wc[w][d] + rank[s];
            keys_out[pos] = key[s];
            vals_out[pos] = val[s];
        }
    }
}

// ---- Karras 2012 hierarchy over the sorted keys -----------------------------------------------
__device__ __forceinline__ int key_delta(const unsigned long long* __restrict__ keys, int n, int i, unsigned long long ki, int j) {
    if (j < 0 || j >= n) return -1;
    const unsigned long long x = ki ^ keys[j];
    return x ? __clzll((long long)x) : 64 + __clz(i ^ j);
}

__global__ void __launch_bounds__(256) k_karras(const unsigned long long* __restrict__ keys, int n, BvhNode* __restrict__ nodes,
                                                int* __restrict__ leaf_parent, int* __restrict__ node_parent,
                                                int* __restrict__ node_first, int* __restrict__ node_count) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n - 1) return;
    const unsigned long long ki = keys[i];
    const int d = (key_delta(keys, n, i, ki, i + 1) - key_delta(keys, n, i, ki, i - 1)) >= 0 ? 1 : -1;
    const int dmin = key_delta(keys, n, i, ki, i - d);
    int lmax = 2;
    while (key_delta(keys, n, i, ki, i + lmax * d) > dmin) lmax <<= 1;
    int l = 0;
    for (int t = lmax >> 1; t >= 1; t >>= 1)
        if (key_delta(keys, n, i, ki, i + (l + t) * d) > dmin) l += t;
    const int j = i + l * d;
    const int dnode = key_delta(keys, n, i, ki, j);
    int s = 0, t = l;
    do {
        t = (t + 1) >> 1;
        if (key_delta(keys, n, i, ki, i + (s + t) * d) > dnode) s += t;
    } while (t > 1);
    const int gamma = i + s * d + min(d, 0);
    const int lo = min(i, j), hi = max(i, j);
    int c0, c1;
    if (lo == gamma) { c0 = ~gamma; leaf_parent[gamma] = i; } else { c0 = gamma; node_parent[gamma] = i; }
    if (hi == gamma + 1) { c1 = ~(gamma + 1); leaf_parent[gamma + 1] = i; } else { c1 = gamma + 1; node_parent[gamma + 1] = i; }
    nodes[i].c0 = c0; nodes[i].c1 = c1;
    node_first[i] = lo; node_count[i] = hi - lo + 1;
    if (i == 0) node_parent[0] = -1;
}

// single-surfel scene: one node whose second child is an empty box
__global__ void k_single_leaf(BvhNode* nodes, int* leaf_parent, int* node_parent, int* node_first, int* node_count, unsigned int* arrive) {
    nodes[0].c0 = ~0; nodes[0].c1 = ~0; node_parent[0] = -1; node_first[0] = 0; node_count[0] = 1;
    nodes[0].t0 = DST_LEAF_LINK(0, 1); nodes[0].t1 = DST_LEAF_LINK(0, 1);
    for (int a = 0; a < 3; a++) { nodes[0].box[6 + a] = INFINITY; nodes[0].box[9 + a] = -INFINITY; }
    leaf_parent[0] = 0;
    arrive[0] = 1;      // the lone leaf acts as the second arrival
}

// ---- bottom-up pass: quad frames + leaf boxes, then boxes of all ancestors ----------------------
// On the way up every node also gets the expected cost of walking its subtree (surface-area
// heuristic) and decides whether the walk should treat it as ONE run of leaves: where boxes overlap
// almost completely (large quads crossing each other) descending costs more than testing every quad.
#ifndef DST_COST_NODE
#define DST_COST_NODE 1.2f
#endif
// Cost of testing a leaf run of `count` quads, in units of one child-box test. The gather kernel tests a run of more
// than DST_HULL_MIN quads with one quad per lane against the hull of its batch of rays (a fixed cost of a few node
// steps for up to 32 quads) and hands only the survivors to all lanes for the exact test; shorter runs are tested
// exactly right away. Where boxes overlap heavily (quads crossing each other in all directions) descending costs
// far more than that and subtrees collapse into runs of up to DST_LEAF_MAX quads; where the children of a node
// share little space (quads tiling a surface) the tree is kept down to single quads.
#ifndef DST_RUN_FIXED
#define DST_RUN_FIXED 3.5f
#endif
#ifndef DST_RUN_PER_QUAD
#define DST_RUN_PER_QUAD 0.25f
#endif
#define DST_COST_QUAD 1.0f
__device__ __forceinline__ float run_cost(int count) {
    return count <= DST_HULL_MIN ? DST_COST_QUAD * (float)count : DST_RUN_FIXED + DST_RUN_PER_QUAD * (float)count;
}
__device__ __forceinline__ float box_area(const float* lo, const float* hi) {
    const float dx = hi[0] - lo[0], dy = hi[1] - lo[1], dz = hi[2] - lo[2];
    const float a = dx * dy + dy * dz + dz * dx;
    return (a > 0.0f && a < INFINITY) ? a : 0.0f;
}

// The 4 corners of surfel g from its parameters, in the reference's expression order
// (example/utils/gaussian_utils.py:176-210 with build_cov :286-296, build_scaling_rotation :273-282,
// build_rotation :214-249): q = r / |r| in (w,x,y,z) order, tangent columns of R scaled by s_x and
// s_y, corner k = (3 cu_k) L0 + (3 cv_k) L1 + mean, (cu,cv) = (-1,+1), (-1,-1), (+1,+1), (+1,-1).
// One rounding per operation; bit-identical to the reference's CPU tensor ops on the test vectors.
struct SurfelSource { const float* means; const float* scales; const float* rotations; float* v_out; };

__device__ __forceinline__ void surfel_corners(const SurfelSource& src, int g, float* v) {
    const float4 r = __ldg(reinterpret_cast<const float4*>(src.rotations) + g);
    const float2 sc = __ldg(reinterpret_cast<const float2*>(src.scales) + g);
    const float m[3] = { __ldg(src.means + 3 * (size_t)g), __ldg(src.means + 3 * (size_t)g + 1), __ldg(src.means + 3 * (size_t)g + 2) };
    const float n = xsqrt(xadd(xadd(xadd(xmul(r.x, r.x), xmul(r.y, r.y)), xmul(r.z, r.z)), xmul(r.w, r.w)));
    const float w = xdiv(r.x, n), x = xdiv(r.y, n), y = xdiv(r.z, n), z = xdiv(r.w, n);
    float c0[3], c1[3];
    c0[0] = xsub(1.0f, xmul(2.0f, xadd(xmul(y, y), xmul(z, z))));
    c0[1] = xmul(2.0f, xadd(xmul(x, y), xmul(w, z)));
    c0[2] = xmul(2.0f, xsub(xmul(x, z), xmul(w, y)));
    c1[0] = xmul(2.0f, xsub(xmul(x, y), xmul(w, z)));
    c1[1] = xsub(1.0f, xmul(2.0f, xadd(xmul(x, x), xmul(z, z))));
    c1[2] = xmul(2.0f, xadd(xmul(y, z), xmul(w, x)));
#pragma unroll
    for (int a = 0; a < 3; a++) {
        const float lu = xmul(c0[a], sc.x), lv = xmul(c1[a], sc.y);
        const float u3 = xmul(lu, 3.0f), v3 = xmul(lv, 3.0f);
        v[0 + a] = xadd(xadd(-u3, v3), m[a]);
        v[3 + a] = xadd(xadd(-u3, -v3), m[a]);
        v[6 + a] = xadd(xadd(u3, v3), m[a]);
        v[9 + a] = xadd(xadd(u3, -v3), m[a]);
    }
}

// get_triangles as one kernel: 36 B of parameters in, 48 B of vertices (+ 24 B of indices) out per surfel
__global__ void __launch_bounds__(256) k_surfel_quads(SurfelSource src, int P, int32_t* __restrict__ tri) {
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= P) return;
    float v[12];
    surfel_corners(src, g, v);
    float4* o = reinterpret_cast<float4*>(src.v_out + 12 * (size_t)g);
    o[0] = make_float4(v[0], v[1], v[2], v[3]); o[1] = make_float4(v[4], v[5], v[6], v[7]); o[2] = make_float4(v[8], v[9], v[10], v[11]);
    if (tri) {
        const int b = 4 * g;
        int2* t = reinterpret_cast<int2*>(tri + 6 * (size_t)g);
        t[0] = make_int2(b, b + 1); t[1] = make_int2(b + 2, b + 1); t[2] = make_int2(b + 2, b + 3);
    }
}

// Bottom-up pass over the hierarchy: leaf level from the quads, then boxes, costs and walk links of
// every ancestor. FROM_SURFELS: the quad corners are computed from the surfel parameters here and
// written to the caller's vertex buffer on the way (the refit then never reads the vertices).
template <bool FROM_SURFELS>
__global__ void __launch_bounds__(256) k_refit(const float* __restrict__ verts, SurfelSource src, int P, const unsigned int* __restrict__ vals,
                                               BvhNode* nodes, const int* __restrict__ leaf_parent, const int* __restrict__ node_parent,
                                               const int* __restrict__ node_first, const int* __restrict__ node_count,
                                               float* child_cost, unsigned int* arrive,
                                               float4* __restrict__ quads, int* __restrict__ leaf_gid, float* header) {
    const int pos = blockIdx.x * blockDim.x + threadIdx.x;
    if (pos >= P) return;
    const int gid = (int)vals[pos];
    float v[12];
    if (FROM_SURFELS) {
        surfel_corners(src, gid, v);
        float4* o = reinterpret_cast<float4*>(src.v_out + 12 * (size_t)gid);
        o[0] = make_float4(v[0], v[1], v[2], v[3]); o[1] = make_float4(v[4], v[5], v[6], v[7]); o[2] = make_float4(v[8], v[9], v[10], v[11]);
    } else {
        const float4* p = reinterpret_cast<const float4*>(verts + 12 * (size_t)gid);
        float4 a = __ldg(p), b = __ldg(p + 1), c = __ldg(p + 2);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        v[8] = c.x; v[9] = c.y; v[10] = c.z; v[11] = c.w;
    }
    const QuadFrame q = make_quad_frame(v);
    quads[3 * (size_t)pos + 0] = make_float4(q.p0x, q.p0y, q.p0z, q.nx);
    quads[3 * (size_t)pos + 1] = make_float4(q.ny, q.nz, q.wux, q.wuy);
    quads[3 * (size_t)pos + 2] = make_float4(q.wuz, q.wvx, q.wvy, q.wvz);
    leaf_gid[pos] = gid;
    float lo[3], hi[3];
    quad_box(v, lo, hi);
    int child = ~pos;                           // topology id of the subtree being carried up
    int link = DST_LEAF_LINK(pos, 1);           // how the walk reaches it
    float cost = DST_COST_QUAD;
    int parent = leaf_parent[pos];
    // the depth of a Karras tree over 64-bit keys with index tie-breaks is below 128
    for (int guard = 0; guard < 128; guard++) {
        BvhNode* nd = nodes + parent;
        const int slot = (nd->c0 == child) ? 0 : 1;
        float2* dst = reinterpret_cast<float2*>(nd->box + 6 * slot);
        dst[0] = make_float2(lo[0], lo[1]); dst[1] = make_float2(lo[2], hi[0]); dst[2] = make_float2(hi[1], hi[2]);
        (&nd->t0)[slot] = link;
        child_cost[2 * (size_t)parent + slot] = cost;
        __threadfence();
        if (atomicAdd(&arrive[parent], 1u) == 0u) return;      // the sibling subtree is not done yet
        const float2* src = reinterpret_cast<const float2*>(nd->box + 6 * (1 - slot));
        const float2 s0 = __ldcg(src), s1 = __ldcg(src + 1), s2 = __ldcg(src + 2);
        const float sib_cost = __ldcg(child_cost + 2 * (size_t)parent + (1 - slot));
        float slo[3] = { s0.x, s0.y, s1.x }, shi[3] = { s1.y, s2.x, s2.y };
        const float a_me = box_area(lo, hi), a_sib = box_area(slo, shi);
        lo[0] = fminf(lo[0], s0.x); lo[1] = fminf(lo[1], s0.y); lo[2] = fminf(lo[2], s1.x);
        hi[0] = fmaxf(hi[0], s1.y); hi[1] = fmaxf(hi[1], s2.x); hi[2] = fmaxf(hi[2], s2.y);
        if (parent == 0) {
            float am = 0.0f;
#pragma unroll
            for (int a = 0; a < 3; a++) {
                header[a] = lo[a]; header[3 + a] = hi[a];
                if (isfinite(lo[a])) am = fmaxf(am, fabsf(lo[a]));
                if (isfinite(hi[a])) am = fmaxf(am, fabsf(hi[a]));
            }
            header[6] = am;
            return;
        }
        const float a_all = box_area(lo, hi);
        const float p_me = a_all > 0.0f ? fminf(a_me / a_all, 1.0f) : 1.0f, p_sib = a_all > 0.0f ? fminf(a_sib / a_all, 1.0f) : 1.0f;
        const float cost_split = DST_COST_NODE + p_me * cost + p_sib * sib_cost;
        const int count = node_count[parent];
        const float cost_run = run_cost(count);
        if (count <= DST_LEAF_MAX && cost_run <= cost_split) { link = DST_LEAF_LINK(node_first[parent], count); cost = cost_run; }
        else { link = parent; cost = cost_split; }
        child = parent;
        parent = node_parent[parent];
    }
}

// plane frames back in surfel order, for tests
__global__ void __launch_bounds__(256) k_export_frames(int P, const float4* __restrict__ quads, const int* __restrict__ leaf_gid,
                                                       float* __restrict__ out) {
    const int pos = blockIdx.x * blockDim.x + threadIdx.x;
    if (pos >= P) return;
    const float4 a = quads[3 * (size_t)pos], b = quads[3 * (size_t)pos + 1], c = quads[3 * (size_t)pos + 2];
    float* o = out + 12 * (size_t)leaf_gid[pos];
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
    o[8] = c.x; o[9] = c.y; o[10] = c.z; o[11] = c.w;
}

int ensure_capacity(dst_handle* h, int64_t P) {
    if (P <= h->cap) return DST_OK;
    // grow-only arena; the old buffers are released first (a rebuild does not need them)
    cudaFree(h->nodes); cudaFree(h->quads); cudaFree(h->leaf_gid); cudaFree(h->leaf_parent); cudaFree(h->arrive);
    cudaFree(h->node_parent); cudaFree(h->node_first); cudaFree(h->node_count); cudaFree(h->child_cost);
    h->node_parent = h->node_first = h->node_count = nullptr; h->child_cost = nullptr;
    cudaFree(h->keys); cudaFree(h->keys_alt); cudaFree(h->vals); cudaFree(h->vals_alt); cudaFree(h->block_hist);
    h->nodes = nullptr; h->quads = nullptr; h->leaf_gid = nullptr; h->leaf_parent = nullptr; h->arrive = nullptr;
    h->keys = h->keys_alt = nullptr; h->vals = h->vals_alt = nullptr; h->block_hist = nullptr;
    h->cap = 0; h->built = false;
    const int64_t cap = P + P / 8 + 1024;
    const int64_t nblocks = (cap + SORT_TILE - 1) / SORT_TILE;
    cudaError_t e = cudaSuccess;
    if (e == cudaSuccess) e = cudaMalloc(&h->nodes, sizeof(BvhNode) * cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->quads, 48 * cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->leaf_gid, 4 * cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->leaf_parent, 4 * cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->arrive, 4 * cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->node_parent, 4 * cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->node_first, 4 * cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->node_count, 4 * cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->child_cost, 8 * cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->keys, 8 * cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->keys_alt, 8 * cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->vals, 4 * cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->vals_alt, 4 * cap);
    if (e == cudaSuccess) e = cudaMalloc(&h->block_hist, 4 * 256 * (nblocks + 1));       // + the 256 digit totals
    if (e != cudaSuccess) {
        cudaGetLastError();
        return dst_set_error(h, DST_E_NOMEM, "device allocation for %lld surfels failed: %s", (long long)P, cudaGetErrorString(e));
    }
    h->cap = cap; h->hist_cap = nblocks;
    return DST_OK;
}

}  // namespace

int dst_surfel_quads_impl(dst_handle* h, const float* means, const float* scales, const float* rotations, int64_t P,
                          float* vertices, int32_t* triangles, cudaStream_t st) {
    if (P <= 0 || P > (1ll << DST_LEAF_POS_BITS)) return dst_set_error(h, DST_E_ARG, "surfel count must be in [1, 2^26], got %lld", (long long)P);
    if ((reinterpret_cast<uintptr_t>(vertices) & 15) || (reinterpret_cast<uintptr_t>(rotations) & 15) || (reinterpret_cast<uintptr_t>(scales) & 7) ||
        (reinterpret_cast<uintptr_t>(triangles) & 7))
        return dst_set_error(h, DST_E_ARG, "vertices and rotations must be 16-byte aligned, scales and triangles 8-byte aligned");
    const SurfelSource src = { means, scales, rotations, vertices };
    k_surfel_quads<<<(unsigned int)((P + 255) / 256), 256, 0, st>>>(src, (int)P, triangles);
    DST_CUDA_TRY(h, cudaGetLastError());
    h->launches += 1;
    return DST_OK;
}

// v: the vertex buffer. With means/scales/rotations non-null it is an OUTPUT: the quads are expanded
// from the surfel parameters (rebuild: by k_surfel_quads before the sort; refit: inside k_refit).
int dst_bvh_build_impl(dst_handle* h, const float* v, int64_t P, int rebuild, cudaStream_t st,
                       const float* means, const float* scales, const float* rotations) {
    const bool from_surfels = means != nullptr;
    const SurfelSource src = { means, scales, rotations, const_cast<float*>(v) };
    if (from_surfels && ((reinterpret_cast<uintptr_t>(rotations) & 15) || (reinterpret_cast<uintptr_t>(scales) & 7)))
        return dst_set_error(h, DST_E_ARG, "rotations must be 16-byte aligned and scales 8-byte aligned");
    if (P <= 0) return dst_set_error(h, DST_E_ARG, "vertices must hold at least one surfel (4 vertices)");
    if (P > (1ll << DST_LEAF_POS_BITS)) return dst_set_error(h, DST_E_ARG, "at most 2^26 surfels are supported");
    if ((reinterpret_cast<uintptr_t>(v) & 15) != 0) return dst_set_error(h, DST_E_ARG, "vertices must be 16-byte aligned");
    if (!rebuild) {
        if (!h->built) return dst_set_error(h, DST_E_STATE, "refit (rebuild=0) requested before any build");
        if (P != h->P) return dst_set_error(h, DST_E_ARG, "refit needs the surfel count of the last build (%lld), got %lld",
                                            (long long)h->P, (long long)P);
    }
    const int n = (int)P;
    const int tpb = 256, grid = (n + tpb - 1) / tpb;
    unsigned int* bw = reinterpret_cast<unsigned int*>(h->header + DST_HDR_FLOATS);
    if (rebuild) {
        int rc = ensure_capacity(h, P);
        if (rc != DST_OK) return rc;
    }
    dst_prof_mark(h, 0, 0, st);
    if (rebuild) {
        h->built = false;
        if (from_surfels) k_surfel_quads<<<grid, tpb, 0, st>>>(src, n, nullptr);
        k_init_bounds<<<1, 32, 0, st>>>(bw);
        const int rgrid = min(grid, h->sm_count * 8);
        k_centre_bounds<<<rgrid, tpb, 0, st>>>(v, n, bw);
        k_morton<<<grid, tpb, 0, st>>>(v, n, bw, h->keys, h->vals);
        const int nblocks = (n + SORT_TILE - 1) / SORT_TILE;
        unsigned long long *kin = h->keys, *kout = h->keys_alt;
        unsigned int *vin = h->vals, *vout = h->vals_alt;
        for (int pass = 0; pass < 8; pass++) {
            const int shift = 8 * pass;
            k_sort_hist<<<nblocks, SORT_THREADS, 0, st>>>(kin, n, shift, h->block_hist, nblocks);
            k_sort_scan<<<256, 256, 0, st>>>(h->block_hist, nblocks, h->block_hist + 256 * (size_t)nblocks);
            k_sort_scatter<<<nblocks, SORT_THREADS, 0, st>>>(kin, vin, kout, vout, n, shift, h->block_hist, nblocks, h->block_hist + 256 * (size_t)nblocks);
            unsigned long long* tk = kin; kin = kout; kout = tk;
            unsigned int* tv = vin; vin = vout; vout = tv;
        }
        // 8 passes: the sorted data is back in keys / vals
        if (n > 1) k_karras<<<(n - 1 + tpb - 1) / tpb, tpb, 0, st>>>(h->keys, n, h->nodes, h->leaf_parent, h->node_parent, h->node_first, h->node_count);
        h->P = P;
    } else if (from_surfels && !h->single_kernel_refit) {
        // measured at 3M surfels: the coalesced expansion pass (0.07 ms) plus the refit's gathered re-read of the
        // vertices is faster than one kernel that scatters 48-byte vertex writes in Morton order (0.57 vs 0.64 ms)
        k_surfel_quads<<<grid, tpb, 0, st>>>(src, n, nullptr);
    }
    DST_CUDA_TRY(h, cudaMemsetAsync(h->arrive, 0, 4 * (size_t)(n > 1 ? n - 1 : 1), st));
    if (n == 1) k_single_leaf<<<1, 1, 0, st>>>(h->nodes, h->leaf_parent, h->node_parent, h->node_first, h->node_count, h->arrive);
    if (from_surfels && !rebuild && h->single_kernel_refit)
        k_refit<true><<<grid, tpb, 0, st>>>(v, src, n, h->vals, h->nodes, h->leaf_parent, h->node_parent, h->node_first, h->node_count, h->child_cost,
                                            h->arrive, h->quads, h->leaf_gid, h->header);
    else
        k_refit<false><<<grid, tpb, 0, st>>>(v, src, n, h->vals, h->nodes, h->leaf_parent, h->node_parent, h->node_first, h->node_count, h->child_cost,
                                             h->arrive, h->quads, h->leaf_gid, h->header);
    dst_prof_mark(h, 0, 1, st);
    DST_CUDA_TRY(h, cudaGetLastError());
    h->launches += (rebuild ? 27 + (n > 1 ? 1 : 0) : 0) + (from_surfels && (rebuild || !h->single_kernel_refit) ? 1 : 0) + (n == 1 ? 1 : 0) + 1;
    h->built = true;
    return DST_OK;
}

int dst_export_frames_impl(dst_handle* h, float* out, cudaStream_t st) {
    if (!h->built) return dst_set_error(h, DST_E_STATE, "no hierarchy has been built");
    k_export_frames<<<(unsigned int)((h->P + 255) / 256), 256, 0, st>>>((int)h->P, h->quads, h->leaf_gid, out);
    DST_CUDA_TRY(h, cudaGetLastError());
    return DST_OK;
}
