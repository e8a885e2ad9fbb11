// Backward trace: replaces optix_tracer/backward.cu (__raygen__ot 857-928, tracePath 658-853,
// traceRay 332-655 and its helpers) and the host launcher TraceSurfelsBackwardCUDA
// (trace_surfels.cpp:307-464).
//
// One thread per ray. Bounces are visited last to first; each segment is re-traced front to back
// with the forward kernel's exact decision code (eval_slot), and every contributing hit adds its
// gradients. Per-surfel gradients go to a packed arena of 16-byte aligned rows with 4-float
// vector reductions (5 per contribution instead of 18 scalar atomics; SH rows 12 instead of 48),
// and are unpacked into the caller's tensors by a streaming kernel afterwards.
#include "dst_trace.cuh"

namespace {

constexpr int BWD_THREADS = 128;

struct BwdParams {
    dst_bwd_args a;
    BvhView bvh;
    const float4* cache;
    float* arena;
    unsigned int* status;
    int tiled;
};

__device__ __forceinline__ void red4(float* addr, float a, float b, float c, float d) {
    atomicAdd(reinterpret_cast<float4*>(addr), make_float4(a, b, c, d));
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

template <bool DIAG>
__global__ void __launch_bounds__(BWD_THREADS) k_backward(const __grid_constant__ BwdParams p) {
    __shared__ unsigned long long kbuf[DST_CHUNK * BWD_THREADS];
    const dst_trace_inputs& in = p.a.in;
    const long long ray = ray_of_thread(in.H, in.W, p.tiled != 0);
    if (ray < 0) return;
    unsigned long long* kb = kbuf + threadIdx.x;
    TraceCounters tc = { 0, 0, 0, 0, 0, 0 };

    const int depth = in.max_trace_depth;
    const bool use_sh = in.colors_precomp == nullptr;
    const bool has_aux = in.others_precomp != nullptr;
    const int ncoef = (in.sh_degree + 1) * (in.sh_degree + 1);
    const bool sh_aligned = ((in.sh_coeffs * 3) & 3) == 0 && ((reinterpret_cast<uintptr_t>(in.shs) & 15) == 0);
    const bool dsh_aligned = ((in.sh_coeffs * 3) & 3) == 0 && ((reinterpret_cast<uintptr_t>(p.a.dL_dshs) & 15) == 0);
    const float bg0 = __ldg(in.background), bg1 = __ldg(in.background + 1), bg2 = __ldg(in.background + 2);
    const float* mid = p.a.mid_val + (size_t)ray * in.mid_stride;

    const float g_rgb0 = __ldg(p.a.dL_drgb + 3 * ray), g_rgb1 = __ldg(p.a.dL_drgb + 3 * ray + 1), g_rgb2 = __ldg(p.a.dL_drgb + 3 * ray + 2);
    const float g_dpt = __ldg(p.a.dL_ddpt + ray), g_acc = __ldg(p.a.dL_dacc + ray);
    const V3 g_norm = v3(__ldg(p.a.dL_dnorm + 3 * ray), __ldg(p.a.dL_dnorm + 3 * ray + 1), __ldg(p.a.dL_dnorm + 3 * ray + 2));
    const float g_aux0 = __ldg(p.a.dL_daux + 2 * ray), g_aux1 = __ldg(p.a.dL_daux + 2 * ray + 1);

    V3 dL_dray_o = v3(0.f, 0.f, 0.f), dL_dray_d = v3(0.f, 0.f, 0.f);

    // backward.cu:683-703: specular product over all bounces and the colour "behind" each one
    float Cp0 = __ldg(p.a.out_rgb + 3 * ray), Cp1 = __ldg(p.a.out_rgb + 3 * ray + 1), Cp2 = __ldg(p.a.out_rgb + 3 * ray + 2);
    float cp0 = 0.f, cp1 = 0.f, cp2 = 0.f;
    float s_prod = 1.0f;
    for (int i = 0; i < depth; i++) {
        const float4 m3 = __ldg(reinterpret_cast<const float4*>(mid + i * DST_MID_CHANNELS) + 3);
        const float4 m2 = __ldg(reinterpret_cast<const float4*>(mid + i * DST_MID_CHANNELS) + 2);
        Cp0 += s_prod * (cp0 - m3.y); Cp1 += s_prod * (cp1 - m3.z); Cp2 += s_prod * (cp2 - m3.w);
        cp0 = m3.y; cp1 = m3.z; cp2 = m3.w;
        s_prod *= m2.w;
    }

    for (int i = depth; i >= 0; i--) {
        const float4* mp = reinterpret_cast<const float4*>(mid + i * DST_MID_CHANNELS);
        const float4 m0 = __ldg(mp), m1 = __ldg(mp + 1), m2 = __ldg(mp + 2), m3 = __ldg(mp + 3);
        const float sox = m0.x, soy = m0.y, soz = m0.z, sdx = m0.w, sdy = m1.x, sdz = m1.y;
        const float tot_dpt = m1.z, tot_acc = m1.w;
        const V3 tot_n = v3(m2.x, m2.y, m2.z);
        const float tot_o0 = m2.w, tot_o1 = m3.x, tot_c0 = m3.y, tot_c1 = m3.z, tot_c2 = m3.w;
        const float s_prev = i > 0 ? __ldg(mid + (i - 1) * DST_MID_CHANNELS + 11) : 1.0f;
        if (sqrtf(sdx * sdx + sdy * sdy + sdz * sdz) == 0.0f || s_prev <= in.specular_threshold) continue;    // :724

        const float f_this = (i == depth) ? 1.0f : 1.0f - tot_o0;
        const float t_rgb0 = g_rgb0 * f_this * s_prod, t_rgb1 = g_rgb1 * f_this * s_prod, t_rgb2 = g_rgb2 * f_this * s_prod;   // :760
        s_prod /= s_prev;                                                                                     // :762
        float t_dpt = 0.f, t_acc = 0.f, t_aux0 = 0.f, t_aux1 = 0.f;
        V3 t_norm = v3(0.f, 0.f, 0.f);
        if (i != depth) {
            // :769-774
            t_aux0 += g_rgb0 * (Cp0 / tot_o0) + g_rgb1 * (Cp1 / tot_o0) + g_rgb2 * (Cp2 / tot_o0);
            if (i > 0) {
                const float4 pm3 = __ldg(reinterpret_cast<const float4*>(mid + (i - 1) * DST_MID_CHANNELS) + 3);
                cp0 = pm3.y; cp1 = pm3.z; cp2 = pm3.w;
            } else { cp0 = cp1 = cp2 = 0.f; }
            Cp0 -= s_prod * (cp0 - tot_c0); Cp1 -= s_prod * (cp1 - tot_c1); Cp2 -= s_prod * (cp2 - tot_c2);
            const float nl = sqrtf(dot(tot_n, tot_n));
            if (nl != 0.0f) {                                                                                 // :778-790
                const V3 d = v3(sdx, sdy, sdz);
                dL_dray_d = dL_dray_d + 0.00001f * dL_dray_o;
                const V3 n = (1.0f / nl) * tot_n;
                t_dpt += dL_dray_o.x * sdx + dL_dray_o.y * sdy + dL_dray_o.z * sdz;
                const V3 gm2 = -2.0f * dL_dray_d;
                t_norm = t_norm + dnormvdv(tot_n, ddotndndn(n, d, gm2));
                dL_dray_d = tot_dpt * dL_dray_o + dL_dray_d + ddotndndd(n, gm2);
            }
        }
        if (i == 0) { t_dpt += g_dpt; t_acc += g_acc; t_norm = t_norm + g_norm; t_aux0 += g_aux0; t_aux1 += g_aux1; }   // :793-802

        // ---- re-trace of segment i with gradients (backward.cu:332-655) ----
        const float min_depth = i == 0 ? (in.start_from_first ? 0.2f : 0.0f) : 0.06f;
        const float T_threshold = 0.0001f;
        const float T_final = 1.0f - tot_acc;
        float C0 = 0.f, C1 = 0.f, C2 = 0.f, D = 0.f, O0 = 0.f, O1 = 0.f;
        V3 N = v3(0.f, 0.f, 0.f);
        float T_prev = 1.0f, T_next = 1.0f, dpt = 0.0f, offset = 0.0f;
        int last_gidx = -1, contributor = 0;
        float tox = sox, toy = soy, toz = soz;
        float sb[16];
        if (use_sh) sh_basis(in.sh_degree, sdx, sdy, sdz, sb);
        int dir_gidx = -1; float dir_g0 = 0.f, dir_g1 = 0.f, dir_g2 = 0.f;     // last SH contribution, for the direction gradient
        if (DIAG) tc.segs++;

        for (int chunk = 0;; chunk++) {
            if (chunk >= DST_MAX_CHUNKS) { atomicOr(p.status, DST_STATUS_CHUNK_LIMIT); break; }
            const int cnt = knearest<false, DIAG, BWD_THREADS>(p.bvh, tox, toy, toz, sdx, sdy, sdz, kb, p.status, tc);
            if (DIAG) tc.enums++;
            bool stop = false;
            for (int s = 0; s < cnt; s++) {
                const unsigned long long key = kb[s * BWD_THREADS];
                const int pidx = (int)(unsigned int)key;
                const int gidx = pidx >> 1;
                if (gidx == last_gidx) continue;
                if (DIAG) tc.evals++;
                SlotEval e;
                const bool ok = eval_slot(key, offset, sox, soy, soz, sdx, sdy, sdz, min_depth, p.cache, gidx, e);
                dpt = e.dpt;
                if (!ok) continue;
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
                if (use_sh) {
                    load_sh_row(in.shs + 3 * (size_t)gidx * in.sh_coeffs, 3 * ncoef, sh_aligned, csh);
                    c0 = sh_channel(ncoef, sb, csh, 0); c1 = sh_channel(ncoef, sb, csh, 1); c2 = sh_channel(ncoef, sb, csh, 2);
                    k0 = c0 < 0.f ? 0.f : 1.f; k1 = c1 < 0.f ? 0.f : 1.f; k2 = c2 < 0.f ? 0.f : 1.f;
                    c0 = fmaxf(c0, 0.f); c1 = fmaxf(c1, 0.f); c2 = fmaxf(c2, 0.f);
                } else {
                    const float* cp = in.colors_precomp + 3 * (size_t)gidx;
                    c0 = __ldg(cp); c1 = __ldg(cp + 1); c2 = __ldg(cp + 2);
                }
                C0 = xadd(C0, xmul(w, c0)); C1 = xadd(C1, xmul(w, c1)); C2 = xadd(C2, xmul(w, c2));
                float ox0 = 0.f, ox1 = 0.f;
                if (has_aux) {
                    const float2 ax = __ldg(reinterpret_cast<const float2*>(in.others_precomp) + gidx);
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

                const float opac = e.r2.w, G = e.G;
                const float dL_dG = dL_dalpha * opac;
                const float pc = (opac * G) > 0.99f ? 0.0f : 1.0f;
                const float dL_dopac = dL_dalpha * G * pc;

                // geometry (backward.cu:201-287, 581-607)
                const float sx = e.r3.x, sy = e.r3.y, u = e.u, v = e.v;
                const V3 R0 = v3(e.r0.x, e.r0.y, e.r0.z), R1 = v3(e.r1.x, e.r1.y, e.r1.z);
                const V3 pm = v3(__ldg(in.means3D + 3 * (size_t)gidx), __ldg(in.means3D + 3 * (size_t)gidx + 1), __ldg(in.means3D + 3 * (size_t)gidx + 2));
                const V3 rel = v3(e.X - pm.x, e.Y - pm.y, e.Z - pm.z);
                const float kk = dL_dG * pc;
                const float dL_du = kk * -G * u, dL_dv = kk * -G * v;
                V3 dR0 = (dL_du / sx) * rel, dR1 = (dL_dv / sy) * rel;
                const V3 dR2 = v3(t_norm.x * w * e.nsign, t_norm.y * w * e.nsign, t_norm.z * w * e.nsign);
                float dsx = kk * (G * u * u / sx), dsy = kk * (G * v * v / sy);
                V3 dmean = (kk * G) * ((u / sx) * R0 + (v / sy) * R1);
                const V3 dxyz = (dL_du / sx) * R0 + (dL_dv / sy) * R1;
                const V3 rd = v3(sdx, sdy, sdz), ro = v3(sox, soy, soz);
                const float dL_dd = t_dpt * w + dot(dxyz, rd);
                V3 p1, p2, p3; float h1x, h1y, h2x, h2y, h3x, h3y;
                {
                    const float4* vq = reinterpret_cast<const float4*>(in.vertices + 12 * (size_t)gidx);
                    const float4 va = __ldg(vq), vb = __ldg(vq + 1), vc = __ldg(vq + 2);
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
                const float4 q = __ldg(reinterpret_cast<const float4*>(in.rotations) + gidx);
                const float qs = rsqrtf(q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z);
                const float qw = q.x * qs, qx = q.y * qs, qy = q.z * qs, qz = q.w * qs;
                const float dq0 = 2.f * (qx * (dR1.z - dR2.y) + qy * (dR2.x - dR0.z) + qz * (dR0.y - dR1.x));
                const float dq1 = 2.f * (-2.f * qx * (dR1.y + dR2.z) + qy * (dR0.y + dR1.x) + qz * (dR0.z + dR2.x) + qw * (dR1.z - dR2.y));
                const float dq2 = 2.f * (qx * (dR0.y + dR1.x) - 2.f * qy * (dR0.x + dR2.z) + qz * (dR1.z + dR2.y) + qw * (dR2.x - dR0.z));
                const float dq3 = 2.f * (qx * (dR0.z + dR2.x) + qy * (dR1.z + dR2.y) - 2.f * qz * (dR0.x + dR1.y) + qw * (dR0.y - dR1.x));

                // per-surfel accumulation (backward.cu:543, 557, 578, 610-626)
                float* row = p.arena + (size_t)gidx * DST_ARENA_FLOATS;
                red4(row, dq0, dq1, dq2, dq3);
                red4(row + 4, dmean.x, dmean.y, dmean.z, dL_dopac);
                const float hd = 0.5f * dpt;
                red4(row + 8, dmean.x * hd, dmean.y * hd, dmean.z * hd, 0.f);
                red4(row + 12, dsx, dsy, has_aux ? t_aux0 * w : 0.f, has_aux ? t_aux1 * w : 0.f);
                const float dc0 = t_rgb0 * w, dc1 = t_rgb1 * w, dc2 = t_rgb2 * w;
                red4(row + 16, dc0, dc1, dc2, 0.f);
                if (use_sh) {
                    const float m0c = dc0 * k0, m1c = dc1 * k1, m2c = dc2 * k2;
                    float* dsh = p.a.dL_dshs + 3 * (size_t)gidx * in.sh_coeffs;
                    if (dsh_aligned) {
                        // 3*ncoef floats as 4-float reductions (ncoef = 4, 16 -> 3, 12 vectors; 1, 9 leave a scalar tail)
                        const int nf = 3 * ncoef, nv = nf >> 2;
#pragma unroll
                        for (int q4 = 0; q4 < 12; q4++) {
                            if (q4 < nv) {
                                float o4[4];
#pragma unroll
                                for (int l = 0; l < 4; l++) { const int f = 4 * q4 + l; const int j = f / 3, ch = f - 3 * j; o4[l] = sb[j] * (ch == 0 ? m0c : ch == 1 ? m1c : m2c); }
                                red4(dsh + 4 * q4, o4[0], o4[1], o4[2], o4[3]);
                            }
                        }
                        for (int f = nv << 2; f < nf; f++) { const int j = f / 3, ch = f - 3 * j; atomicAdd(dsh + f, sb[j] * (ch == 0 ? m0c : ch == 1 ? m1c : m2c)); }
                    } else {
                        for (int j = 0; j < ncoef; j++) { atomicAdd(dsh + 3 * j, sb[j] * m0c); atomicAdd(dsh + 3 * j + 1, sb[j] * m1c); atomicAdd(dsh + 3 * j + 2, sb[j] * m2c); }
                    }
                    dir_gidx = gidx; dir_g0 = m0c; dir_g1 = m1c; dir_g2 = m2c;
                }
                T_prev = T_next;
            }
            if (stop || T_next < T_threshold || cnt < DST_CHUNK || contributor > DST_MAX_INTERSECTION) break;
            offset = (float)((double)dpt + 0.00001);
            tox = xadd(sox, xmul(offset, sdx)); toy = xadd(soy, xmul(offset, sdy)); toz = xadd(soz, xmul(offset, sdz));
        }
        // With SH colours the reference ASSIGNS the SH direction gradient to the ray-direction
        // accumulator at every contribution (backward.cu:165, 631-632), so what survives a segment
        // is the value of its last contribution.
        if (use_sh && dir_gidx >= 0) {
            float csh[48], sj[16];
            load_sh_row(in.shs + 3 * (size_t)dir_gidx * in.sh_coeffs, 3 * ncoef, sh_aligned, csh);
#pragma unroll
            for (int j = 0; j < 16; j++) sj[j] = j < ncoef ? csh[3 * j] * dir_g0 + csh[3 * j + 1] * dir_g1 + csh[3 * j + 2] * dir_g2 : 0.f;
            dL_dray_d = sh_dir_grad(in.sh_degree, sj, sdx, sdy, sdz);
        }
    }
    p.a.dL_dray_o[3 * ray] = dL_dray_o.x; p.a.dL_dray_o[3 * ray + 1] = dL_dray_o.y; p.a.dL_dray_o[3 * ray + 2] = dL_dray_o.z;
    p.a.dL_dray_d[3 * ray] = dL_dray_d.x; p.a.dL_dray_d[3 * ray + 1] = dL_dray_d.y; p.a.dL_dray_d[3 * ray + 2] = dL_dray_d.z;
    if (DIAG && p.a.counters) {
        atomicAdd(p.a.counters + 0, tc.segs); atomicAdd(p.a.counters + 1, tc.enums); atomicAdd(p.a.counters + 2, tc.nodes);
        atomicAdd(p.a.counters + 3, tc.quads); atomicAdd(p.a.counters + 4, tc.evals); atomicAdd(p.a.counters + 5, tc.contribs);
    }
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

int dst_backward_impl(dst_handle* h, const dst_bwd_args* a, cudaStream_t st) {
    int rc = dst_check_inputs(h, &a->in);
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
    p.tiled = a->in.H >= 16;
    const long long R = (long long)a->in.H * a->in.W;
    const long long blocks = p.tiled ? (long long)((a->in.W + 15) / 16) * ((a->in.H + 7) / 8) : (R + BWD_THREADS - 1) / BWD_THREADS;
    dst_prof_mark(h, 2, 0, st);
    if (a->counters) k_backward<true><<<(unsigned int)blocks, BWD_THREADS, 0, st>>>(p);
    else k_backward<false><<<(unsigned int)blocks, BWD_THREADS, 0, st>>>(p);
    dst_prof_mark(h, 2, 1, st);
    DST_CUDA_TRY(h, cudaGetLastError());
    k_unpack<<<(unsigned int)((P + 255) / 256), 256, 0, st>>>((int)P, h->arena, a->dL_drotations, a->dL_dmeans3D, a->dL_dopacities,
                                                              a->dL_dgrads3D, a->dL_dscales, a->dL_dothers, a->dL_dcolors);
    DST_CUDA_TRY(h, cudaGetLastError());
    return DST_OK;
}
