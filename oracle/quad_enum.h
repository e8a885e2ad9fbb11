// TEST INFRASTRUCTURE ONLY (CPU oracle). Nothing on the product path may include this file.
//
// Ray / surfel-quad hit enumerator used by both oracle builds (the restatement in
// surfel_oracle.cpp and the reference shaders compiled by ref_driver.cpp).
//
// The reference delegates this step to the closed OptiX runtime (optixAccelBuild at
// trace_surfels.cpp:84-108, optixTrace at optix_tracer/forward.cu:117-132 and
// optix_tracer/backward.cu:314-329); no source, test or golden vector of the reference pins
// its rounding ("parity unpinned" for this step). The enumerator below therefore DEFINES the
// hit predicate. It is written as an exact sequence of IEEE-754 binary32 operations (round to
// nearest, fused multiply-add only where fmaf is spelled out; build with -ffp-contract=off) so
// that a second implementation can reproduce it bit for bit.
//
// Geometry contract (example/utils/gaussian_utils.py:176-210, optix_tracer/backward.cu:583-602):
// surfel g owns vertices v[4g..4g+3] = mu + 3*(cu*sx*Ru + cv*sy*Rv) for (cu,cv) =
// (-1,+1), (-1,-1), (+1,+1), (+1,-1) and triangles 2g = (v0,v1,v2), 2g+1 = (v1,v2,v3).
// One hit per quad per enumeration is reported; the primitive id is 2g + (u > v), i.e. the
// triangle on whose side of the shared diagonal v1-v2 the hit lies (the lower id on the diagonal).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>

namespace orc {

static const int   KCHUNK   = 16;        // CHUNK_SIZE, optix_tracer/config.h:20
static const float T_MAX    = 1e16f;     // DEPTH_INFINTY / optixTrace tmax, config.h:21, forward.cu:124

struct QuadRec { float p0[3], n[3], wu[3], wv[3]; };

static inline float dop(float a, float b, float c, float d) { float w = c * d; return fmaf(a, b, -w); }
static inline float dot3(const float* a, const float* b) { return fmaf(a[2], b[2], fmaf(a[1], b[1], a[0] * b[0])); }
static inline void cross3(const float* a, const float* b, float* r) {
    r[0] = dop(a[1], b[2], a[2], b[1]);
    r[1] = dop(a[2], b[0], a[0], b[2]);
    r[2] = dop(a[0], b[1], a[1], b[0]);
}

// Plane frame of one quad: corner p0 = v1, edges eu = v3 - v1, ev = v0 - v1, n = eu x ev,
// reciprocal edges wu = (ev x n)/(n.n), wv = (n x eu)/(n.n), so that for a point p0 + h in the
// plane u = wu.h and v = wv.h are its edge coordinates in [0,1]^2.
static inline void make_quad(const float* v, QuadRec& q) {
    float eu[3], ev[3], cu[3], cv[3];
    for (int a = 0; a < 3; a++) { q.p0[a] = v[3 + a]; eu[a] = v[9 + a] - v[3 + a]; ev[a] = v[a] - v[3 + a]; }
    cross3(eu, ev, q.n);
    float nn = dot3(q.n, q.n);
    cross3(ev, q.n, cu);
    cross3(q.n, eu, cv);
    for (int a = 0; a < 3; a++) { q.wu[a] = cu[a] / nn; q.wv[a] = cv[a] / nn; }
}

// Returns true and (t, tri) when the ray o + t d, 0 <= t < 1e16, meets the quad.
static inline bool ray_quad(const QuadRec& q, const float* o, const float* d, float& t, int& tri) {
    float r[3] = { q.p0[0] - o[0], q.p0[1] - o[1], q.p0[2] - o[2] };
    float b = dot3(q.n, d);
    if (!(b != 0.0f)) return false;
    float a = dot3(q.n, r);
    float tt = a / b;
    if (!(tt >= 0.0f && tt < T_MAX)) return false;
    tt = tt + 0.0f;                                   // -0 -> +0 so that the bit pattern orders like the value
    float h[3] = { fmaf(tt, d[0], -r[0]), fmaf(tt, d[1], -r[1]), fmaf(tt, d[2], -r[2]) };
    float u = dot3(q.wu, h), w = dot3(q.wv, h);
    if (!(u >= 0.0f && u <= 1.0f && w >= 0.0f && w <= 1.0f)) return false;
    t = tt; tri = (u > w) ? 1 : 0;
    return true;
}

// Portable exp for x <= 0 (used for the Gaussian falloff, optix_tracer/forward.cu:247): Cody-Waite
// reduction x = k ln2 + r, degree-7 Taylor polynomial in r, exact scaling by 2^k. Every step is one
// rounded binary32 operation (or one fused multiply-add where written), so the CUDA kernels
// reproduce it bit for bit; it agrees with a correctly rounded exp to about 1 ulp.
static inline float pexp(float x) {
    if (!(x >= -87.0f)) return (x != x) ? x : 0.0f;
    if (x > 88.0f) x = 88.0f;
    float kf = (x * 1.44269504088896341f + 12582912.0f) - 12582912.0f;
    float r = fmaf(kf, -0.693145751953125f, x);
    r = fmaf(kf, -1.42860682030941723212e-6f, r);
    float p = 0.0001984126984126984f;
    p = fmaf(p, r, 0.001388888888888889f);
    p = fmaf(p, r, 0.008333333333333333f);
    p = fmaf(p, r, 0.041666666666666664f);
    p = fmaf(p, r, 0.16666666666666666f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    int32_t bits = ((int32_t)kf + 127) << 23;
    float sc; memcpy(&sc, &bits, 4);
    return p * sc;
}

// 64-bit sort key: (bits of t) << 32 | primitive id. t >= +0 so the bit pattern is monotone.
static inline uint64_t hit_key(float t, uint32_t pidx) { uint32_t b; memcpy(&b, &t, 4); return ((uint64_t)b << 32) | pidx; }
static inline float    key_t(uint64_t k) { uint32_t b = (uint32_t)(k >> 32); float t; memcpy(&t, &b, 4); return t; }
static inline uint32_t key_pidx(uint64_t k) { return (uint32_t)k; }

struct Scene {
    int P = 0;
    bool brute = false;
    std::vector<QuadRec> quads;
    // median-split BVH over quad boxes (host only; any conservative hierarchy gives the same hit sets)
    struct Node { float lo[3], hi[3]; int left, right, first, count; };
    std::vector<Node> nodes;
    std::vector<int> order;
    std::vector<float> blo, bhi;   // per-quad boxes
    float absmax = 0.f;

    void init(const float* v, int P_, bool brute_) {
        P = P_; brute = brute_;
        quads.resize(P); blo.resize(3 * (size_t)P); bhi.resize(3 * (size_t)P); order.resize(P);
        absmax = 0.f;
        for (int g = 0; g < P; g++) {
            make_quad(v + 12 * (size_t)g, quads[g]);
            for (int a = 0; a < 3; a++) {
                float lo = INFINITY, hi = -INFINITY;
                for (int k = 0; k < 4; k++) { float x = v[12 * (size_t)g + 3 * k + a]; lo = std::min(lo, x); hi = std::max(hi, x); }
                blo[3 * (size_t)g + a] = lo; bhi[3 * (size_t)g + a] = hi;
                if (std::isfinite(lo)) absmax = std::max(absmax, std::fabs(lo));
                if (std::isfinite(hi)) absmax = std::max(absmax, std::fabs(hi));
            }
            order[g] = g;
        }
        nodes.clear();
        if (!brute && P > 0) { nodes.reserve(2 * (size_t)P / 2 + 16); build(0, P); }
    }

    int build(int first, int last) {
        int id = (int)nodes.size(); nodes.push_back(Node());
        float lo[3] = { INFINITY, INFINITY, INFINITY }, hi[3] = { -INFINITY, -INFINITY, -INFINITY };
        float clo[3] = { INFINITY, INFINITY, INFINITY }, chi[3] = { -INFINITY, -INFINITY, -INFINITY };
        for (int i = first; i < last; i++) {
            int g = order[i];
            for (int a = 0; a < 3; a++) {
                lo[a] = std::min(lo[a], blo[3 * (size_t)g + a]); hi[a] = std::max(hi[a], bhi[3 * (size_t)g + a]);
                float c = 0.5f * (blo[3 * (size_t)g + a] + bhi[3 * (size_t)g + a]);
                clo[a] = std::min(clo[a], c); chi[a] = std::max(chi[a], c);
            }
        }
        Node nd; for (int a = 0; a < 3; a++) { nd.lo[a] = lo[a]; nd.hi[a] = hi[a]; }
        nd.first = first; nd.count = last - first; nd.left = nd.right = -1;
        if (last - first > 4) {
            int ax = 0; float ext = chi[0] - clo[0];
            for (int a = 1; a < 3; a++) if (chi[a] - clo[a] > ext) { ext = chi[a] - clo[a]; ax = a; }
            int mid = (first + last) / 2;
            std::nth_element(order.begin() + first, order.begin() + mid, order.begin() + last, [&](int x, int y) {
                float cx = blo[3 * (size_t)x + ax] + bhi[3 * (size_t)x + ax], cy = blo[3 * (size_t)y + ax] + bhi[3 * (size_t)y + ax];
                return cx < cy || (cx == cy && x < y); });
            nd.count = 0;
            nodes[id] = nd;
            int l = build(first, mid); int r = build(mid, last);
            nodes[id].left = l; nodes[id].right = r;
        } else nodes[id] = nd;
        return id;
    }

    // Visits every leaf quad whose padded box the ray may touch. `limit()` returns the current
    // pruning distance (hits at or beyond it are of no interest), `offer(g)` tests quad g.
    template <class Limit, class Offer>
    void walk(const float* o, const float* d, Limit limit, Offer offer) const {
        if (brute) { for (int g = 0; g < P; g++) offer(g); return; }
        if (P == 0) return;
        // generous, ray-dependent padding keeps the box test conservative against rounding
        float omax = std::max(std::fabs(o[0]), std::max(std::fabs(o[1]), std::fabs(o[2])));
        if (!std::isfinite(omax)) return;
        float pad = 1e-5f * (omax + absmax) + 1e-30f;
        double inv[3]; for (int a = 0; a < 3; a++) inv[a] = 1.0 / (double)d[a];
        int stack[256]; int sp = 0; stack[sp++] = 0;
        while (sp) {
            const Node& nd = nodes[stack[--sp]];
            double tn = 0.0, tf = (double)T_MAX; bool miss = false;
            for (int a = 0; a < 3; a++) {
                double lo = (double)nd.lo[a] - pad - (double)o[a], hi = (double)nd.hi[a] + pad - (double)o[a];
                if (d[a] == 0.0f) { if (lo > 0.0 || hi < 0.0) { miss = true; break; } continue; }
                double t0 = lo * inv[a], t1 = hi * inv[a]; if (t0 > t1) std::swap(t0, t1);
                tn = std::max(tn, t0); tf = std::min(tf, t1);
            }
            if (miss || !(tn <= tf * (1.0 + 1e-6) + 1e-30)) continue;
            if (tn * (1.0 - 1e-6) > (double)limit() * (1.0 + 1e-6)) continue;
            if (nd.left < 0) { for (int i = 0; i < nd.count; i++) offer(order[nd.first + i]); }
            else if (sp + 2 <= 256) { stack[sp++] = nd.left; stack[sp++] = nd.right; }
        }
    }

    // The KCHUNK smallest (t, pidx) hits with t >= 0 from origin o; returns min(total hits, KCHUNK).
    // `tested` (optional) counts exact quad tests.
    int knearest(const float* o, const float* d, uint64_t* buf, long* tested = nullptr) const {
        int n = 0;
        walk(o, d,
             [&]() { return n == KCHUNK ? key_t(buf[KCHUNK - 1]) : T_MAX; },
             [&](int g) {
                 float t; int tri;
                 if (tested) (*tested)++;
                 if (!ray_quad(quads[g], o, d, t, tri)) return;
                 uint64_t key = hit_key(t, 2u * (uint32_t)g + (uint32_t)tri);
                 if (n == KCHUNK) { if (key >= buf[KCHUNK - 1]) return; n--; }
                 int j = n; while (j > 0 && buf[j - 1] > key) { buf[j] = buf[j - 1]; j--; }
                 buf[j] = key; n++;
             });
        return n;
    }

    // every hit on the ray, sorted by key (through the hierarchy unless the scene is brute force)
    void all_hits(const float* o, const float* d, std::vector<uint64_t>& out) const {
        out.clear();
        walk(o, d, [&]() { return T_MAX; },
             [&](int g) { float t; int tri; if (ray_quad(quads[g], o, d, t, tri)) out.push_back(hit_key(t, 2u * (uint32_t)g + (uint32_t)tri)); });
        std::sort(out.begin(), out.end());
    }
    // every hit on the ray by exhaustive testing
    void all_hits_brute(const float* o, const float* d, std::vector<uint64_t>& out) const {
        out.clear();
        for (int g = 0; g < P; g++) { float t; int tri; if (ray_quad(quads[g], o, d, t, tri)) out.push_back(hit_key(t, 2u * (uint32_t)g + (uint32_t)tri)); }
        std::sort(out.begin(), out.end());
    }
};

} // namespace orc
