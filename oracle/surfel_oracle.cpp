// TEST INFRASTRUCTURE ONLY. CPU restatement of the reference's surfel-tracing hot path.
//
// Nothing on the product path links, imports or executes this file; it exists to check the CUDA
// kernels (tests, the smoke entry point) and to give bench.py a CPU baseline.
//
// What is restated (reference file:line in each function's comment):
//   forward   optix_tracer/forward.cu  : computeColorFromSH 18-58, compute_transmat_uv 63-90,
//             traceRay 136-315, tracePath 318-424, __raygen__ot 428-477, __anyhit__ot 481-525
//   backward  optix_tracer/backward.cu : computeColorFromSHBackward 68-166,
//             compute_transmat_uv_backward 201-287, traceRay 332-655, tracePath 658-853,
//             __raygen__ot 857-928
//   helpers   optix_tracer/auxiliary.h : quat_to_rotmat_transpose 403-429, quat_to_rotmat_vjp 433-477,
//             dnormvdv 111-121, ddotndndn 234-243, ddotndndd 245-252; constants config.h:5-29
// The closed OptiX step (hit enumeration) is supplied by quad_enum.h.
//
// Pinning: the reference ships no tests, golden vectors or fixtures for this path. This file is
// pinned against the reference's own shader sources compiled for the host (ref_driver.cpp ->
// oracle/_ref/*.so, same enumerator) by tests/test_cpu_host.py, and against vectors generated
// from that build and committed under tests/golden/. The enumeration step itself stays unpinned.
//
// Semantics are the "clean" ones: every enumeration starts from an empty 16-slot buffer. The
// verbatim reference leaves a slot that was skipped by the repeated-surfel test un-reset
// (forward.cu:207-216), which makes its result depend on OptiX's hit arrival order.
//
// Arithmetic: binary32, one rounding per written operation, no contraction
// (build with -ffp-contract=off), so expression shapes below are significant.
#include "quad_enum.h"
#include "orc_args.h"
#include <omp.h>
#include <cstdio>

namespace {

struct F2 { float x, y; };
struct F3 { float x, y, z; };
struct F4 { float x, y, z, w; };
static inline F3 mk3(float x, float y, float z) { F3 r = { x, y, z }; return r; }
static inline F2 mk2(float x, float y) { F2 r = { x, y }; return r; }
static inline F3 operator+(F3 a, F3 b) { return mk3(a.x + b.x, a.y + b.y, a.z + b.z); }
static inline F3 operator-(F3 a, F3 b) { return mk3(a.x - b.x, a.y - b.y, a.z - b.z); }
static inline F3 operator*(F3 a, F3 b) { return mk3(a.x * b.x, a.y * b.y, a.z * b.z); }
static inline F3 operator*(F3 a, float b) { return mk3(a.x * b, a.y * b, a.z * b); }
static inline F3 operator*(float a, F3 b) { return mk3(a * b.x, a * b.y, a * b.z); }
static inline F3 operator/(F3 a, float b) { return mk3(a.x / b, a.y / b, a.z / b); }
static inline F3 operator-(F3 a) { return mk3(-a.x, -a.y, -a.z); }
static inline F3& operator+=(F3& a, F3 b) { a.x += b.x; a.y += b.y; a.z += b.z; return a; }
static inline F2 operator*(F2 a, F2 b) { return mk2(a.x * b.x, a.y * b.y); }
static inline F2 operator*(float a, F2 b) { return mk2(a * b.x, a * b.y); }
static inline F2 operator/(F2 a, F2 b) { return mk2(a.x / b.x, a.y / b.y); }
static inline float dot(F3 a, F3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
static inline float dot(F2 a, F2 b) { return a.x * b.x + a.y * b.y; }
static inline float sumf3(F3 a) { return a.x + a.y + a.z; }
static inline float length(F3 a) { return sqrtf(dot(a, a)); }
static inline F3 normalize(F3 a) { return a / sqrtf(dot(a, a)); }
static inline F3 cross(F3 a, F3 b) { return mk3(a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x); }
static inline F3 max0(F3 a) { return mk3(a.x > 0.0f ? a.x : 0.0f, a.y > 0.0f ? a.y : 0.0f, a.z > 0.0f ? a.z : 0.0f); }
static inline F3 ld3(const float* p) { return mk3(p[0], p[1], p[2]); }

// optix_tracer/config.h:5-29, auxiliary.h:20
static const int NUM_CHANNELS = 3, AUX_CHANNELS = 2, MID_CHANNELS = 16;
static const int RAYO_MID = 0, RAYD_MID = 3, DPT_MID = 6, ACC_MID = 7, NORM_MID = 8, AUX_MID = 11, RGB_MID = 13;
static const int SPECULAR = 0;
static const int MAX_INTERSECTION = 256;
static const double STEP_EPSILON = 0.00001;
static const double START_OFFSET = 0.06;
static const float NEAR_N = 0.2;
static const int MAX_CHUNKS = 4096;      // loop bound the reference lacks; never reached by a terminating ray

// auxiliary.h:26-43
static const float SH_C0 = 0.28209479177387814f;
static const float SH_C1 = 0.4886025119029199f;
static const float SH_C2[] = { 1.0925484305920792f, -1.0925484305920792f, 0.31539156525252005f, -1.0925484305920792f, 0.5462742152960396f };
static const float SH_C3[] = { -0.5900435899266435f, 2.890611442640554f, -0.4570457994644658f, 0.3731763325901154f,
                               -0.4570457994644658f, 1.445305721320277f, -0.5900435899266435f };

// auxiliary.h:403-429. The stored quaternion is (w,x,y,z); rows of the result are tangent u, tangent v, normal.
static void quat_rows(const float* q, F3* R) {
    float s = 1.0f / sqrtf(q[3] * q[3] + q[0] * q[0] + q[1] * q[1] + q[2] * q[2]);
    float w = q[0] * s, x = q[1] * s, y = q[2] * s, z = q[3] * s;
    R[0] = mk3(1.f - 2.f * (y * y + z * z), 2.f * (x * y + w * z), 2.f * (x * z - w * y));
    R[1] = mk3(2.f * (x * y - w * z), 1.f - 2.f * (x * x + z * z), 2.f * (y * z + w * x));
    R[2] = mk3(2.f * (x * z + w * y), 2.f * (y * z - w * x), 1.f - 2.f * (x * x + y * y));
}

// auxiliary.h:433-477 (no gradient through the normalisation)
static void quat_rows_vjp(const float* q, const F3* vR, float* out) {
    float s = 1.0f / sqrtf(q[3] * q[3] + q[0] * q[0] + q[1] * q[1] + q[2] * q[2]);
    float w = q[0] * s, x = q[1] * s, y = q[2] * s, z = q[3] * s;
    out[0] = 2.f * (x * (vR[1].z - vR[2].y) + y * (vR[2].x - vR[0].z) + z * (vR[0].y - vR[1].x));
    out[1] = 2.f * (-2.f * x * (vR[1].y + vR[2].z) + y * (vR[0].y + vR[1].x) + z * (vR[0].z + vR[2].x) + w * (vR[1].z - vR[2].y));
    out[2] = 2.f * (x * (vR[0].y + vR[1].x) - 2.f * y * (vR[0].x + vR[2].z) + z * (vR[1].z + vR[2].y) + w * (vR[2].x - vR[0].z));
    out[3] = 2.f * (x * (vR[0].z + vR[2].x) + y * (vR[1].z + vR[2].y) - 2.f * z * (vR[0].x + vR[1].y) + w * (vR[0].y - vR[1].x));
}

// auxiliary.h:111-121
static F3 dnormvdv(F3 v, F3 dv) {
    float sum2 = v.x * v.x + v.y * v.y + v.z * v.z;
    float invsum32 = 1.0f / sqrtf(sum2 * sum2 * sum2);
    F3 r;
    r.x = ((+sum2 - v.x * v.x) * dv.x - v.y * v.x * dv.y - v.z * v.x * dv.z) * invsum32;
    r.y = (-v.x * v.y * dv.x + (sum2 - v.y * v.y) * dv.y - v.z * v.y * dv.z) * invsum32;
    r.z = (-v.x * v.z * dv.x - v.y * v.z * dv.y + (sum2 - v.z * v.z) * dv.z) * invsum32;
    return r;
}
// auxiliary.h:234-243
static F3 ddotndndn(F3 n, F3 d, F3 g) {
    float dotnd = dot(n, d);
    F3 r;
    r.x = g.x * (dotnd + d.x * n.x) + g.y * d.x * n.y + g.z * d.x * n.z;
    r.y = g.x * d.y * n.x + g.y * (dotnd + d.y * n.y) + g.z * d.y * n.z;
    r.z = g.x * d.z * n.x + g.y * d.z * n.y + g.z * (dotnd + d.z * n.z);
    return r;
}
// auxiliary.h:245-252
static F3 ddotndndd(F3 n, F3, F3 g) {
    F3 r;
    r.x = g.x * n.x * n.x + g.y * n.x * n.y + g.z * n.x * n.z;
    r.y = g.x * n.y * n.x + g.y * n.y * n.y + g.z * n.y * n.z;
    r.z = g.x * n.z * n.x + g.y * n.z * n.y + g.z * n.z * n.z;
    return r;
}

// forward.cu:18-58 / backward.cu:18-63: SH colour in the ray direction, +0.5, clamped at 0
static F3 sh_color(int deg, const float* shrow, F3 dir, float* clamped) {
    const F3* sh = (const F3*)shrow;
    F3 result = SH_C0 * sh[0];
    if (deg > 0) {
        float x = dir.x, y = dir.y, z = dir.z;
        result = result - SH_C1 * y * sh[1] + SH_C1 * z * sh[2] - SH_C1 * x * sh[3];
        if (deg > 1) {
            float xx = x * x, yy = y * y, zz = z * z, xy = x * y, yz = y * z, xz = x * z;
            result = result + SH_C2[0] * xy * sh[4] + SH_C2[1] * yz * sh[5] + SH_C2[2] * (2.0f * zz - xx - yy) * sh[6] +
                     SH_C2[3] * xz * sh[7] + SH_C2[4] * (xx - yy) * sh[8];
            if (deg > 2) {
                result = result + SH_C3[0] * y * (3.0f * xx - yy) * sh[9] + SH_C3[1] * xy * z * sh[10] +
                         SH_C3[2] * y * (4.0f * zz - xx - yy) * sh[11] + SH_C3[3] * z * (2.0f * zz - 3.0f * xx - 3.0f * yy) * sh[12] +
                         SH_C3[4] * x * (4.0f * zz - xx - yy) * sh[13] + SH_C3[5] * z * (xx - yy) * sh[14] +
                         SH_C3[6] * x * (xx - 3.0f * yy) * sh[15];
            }
        }
    }
    result = result + mk3(0.5f, 0.5f, 0.5f);
    if (clamped) { clamped[0] = (result.x < 0); clamped[1] = (result.y < 0); clamped[2] = (result.z < 0); }
    return max0(result);
}

// backward.cu:68-166: gradient to the SH coefficients; the direction gradient REPLACES the caller's accumulator (:165)
static void sh_color_vjp(int deg, const float* shrow, F3 dir, const float* clamped, const float* dL_dcolor, F3* dL_dsh, F3& dL_ddir) {
    const F3* sh = (const F3*)shrow;
    F3 g = mk3(dL_dcolor[0], dL_dcolor[1], dL_dcolor[2]);
    g.x *= clamped[0] ? 0 : 1; g.y *= clamped[1] ? 0 : 1; g.z *= clamped[2] ? 0 : 1;
    F3 dx = mk3(0, 0, 0), dy = mk3(0, 0, 0), dz = mk3(0, 0, 0);
    float x = dir.x, y = dir.y, z = dir.z;
    dL_dsh[0] = SH_C0 * g;
    if (deg > 0) {
        dL_dsh[1] = (-SH_C1 * y) * g; dL_dsh[2] = (SH_C1 * z) * g; dL_dsh[3] = (-SH_C1 * x) * g;
        dx = -SH_C1 * sh[3]; dy = -SH_C1 * sh[1]; dz = SH_C1 * sh[2];
        if (deg > 1) {
            float xx = x * x, yy = y * y, zz = z * z, xy = x * y, yz = y * z, xz = x * z;
            dL_dsh[4] = (SH_C2[0] * xy) * g; dL_dsh[5] = (SH_C2[1] * yz) * g; dL_dsh[6] = (SH_C2[2] * (2.f * zz - xx - yy)) * g;
            dL_dsh[7] = (SH_C2[3] * xz) * g; dL_dsh[8] = (SH_C2[4] * (xx - yy)) * g;
            dx += SH_C2[0] * y * sh[4] + SH_C2[2] * 2.f * -x * sh[6] + SH_C2[3] * z * sh[7] + SH_C2[4] * 2.f * x * sh[8];
            dy += SH_C2[0] * x * sh[4] + SH_C2[1] * z * sh[5] + SH_C2[2] * 2.f * -y * sh[6] + SH_C2[4] * 2.f * -y * sh[8];
            dz += SH_C2[1] * y * sh[5] + SH_C2[2] * 2.f * 2.f * z * sh[6] + SH_C2[3] * x * sh[7];
            if (deg > 2) {
                dL_dsh[9] = (SH_C3[0] * y * (3.f * xx - yy)) * g; dL_dsh[10] = (SH_C3[1] * xy * z) * g;
                dL_dsh[11] = (SH_C3[2] * y * (4.f * zz - xx - yy)) * g; dL_dsh[12] = (SH_C3[3] * z * (2.f * zz - 3.f * xx - 3.f * yy)) * g;
                dL_dsh[13] = (SH_C3[4] * x * (4.f * zz - xx - yy)) * g; dL_dsh[14] = (SH_C3[5] * z * (xx - yy)) * g;
                dL_dsh[15] = (SH_C3[6] * x * (xx - 3.f * yy)) * g;
                dx += (SH_C3[0] * sh[9] * 3.f * 2.f * xy + SH_C3[1] * sh[10] * yz + SH_C3[2] * sh[11] * -2.f * xy +
                       SH_C3[3] * sh[12] * -3.f * 2.f * xz + SH_C3[4] * sh[13] * (-3.f * xx + 4.f * zz - yy) +
                       SH_C3[5] * sh[14] * 2.f * xz + SH_C3[6] * sh[15] * 3.f * (xx - yy));
                dy += (SH_C3[0] * sh[9] * 3.f * (xx - yy) + SH_C3[1] * sh[10] * xz + SH_C3[2] * sh[11] * (-3.f * yy + 4.f * zz - xx) +
                       SH_C3[3] * sh[12] * -3.f * 2.f * yz + SH_C3[4] * sh[13] * -2.f * xy + SH_C3[5] * sh[14] * -2.f * yz +
                       SH_C3[6] * sh[15] * -3.f * 2.f * xy);
                dz += (SH_C3[1] * sh[10] * xy + SH_C3[2] * sh[11] * 4.f * 2.f * yz + SH_C3[3] * sh[12] * 3.f * (2.f * zz - xx - yy) +
                       SH_C3[4] * sh[13] * 4.f * 2.f * xz + SH_C3[5] * sh[14] * (xx - yy));
            }
        }
    }
    dL_ddir = mk3(dot(dx, g), dot(dy, g), dot(dz, g));
}

struct Ctx { const OrcArgs* a; const orc::Scene* sc; };

struct TraceOut { float C[3]; float D, A; F3 N; float O[2]; float T; F3 E; float Dist, M1, M2, m0; };
struct TraceBwd {   // per-trace totals and upstream gradients, backward.cu:342-354, and the register accumulators :366-367
    float out_rgb[3]; float out_dpt, out_acc; F3 out_norm; float out_aux[2];
    float dL_drgb[3]; float dL_ddpt, dL_dacc; F3 dL_dnorm; float dL_daux[2];
    F3* dL_dray_o; F3* dL_dray_d;
    float dL_ddist, out_m1, out_m2;      // distortion extension: upstream gradient and the two moments the forward saved
};
struct Tally { long enums, tests, evals, contribs, anyhits, segs; };

static inline void atomic_add(float* p, float v) {
#pragma omp atomic
    *p += v;
}

// forward.cu:136-315 and backward.cu:332-655: chunked nearest-16 gather, front-to-back compositing,
// and (bw != nullptr) the per-contribution gradients.
//
// Distortion (dist_on; NOT in the reference, which leaves the output at zero with a TODO, forward.cu:286 and
// backward.cu:526, 570): the depth-distortion sum of 2D Gaussian splatting over the contributions of the primary
// segment, dist = sum_i sum_{j<i} w_i w_j (m_i - m_j)^2 with the mapped depth m = far / (far - near) * (1 - near / dpt),
// near = 0.2 and far = 100 being the two constants the reference defines for it (auxiliary.h:20-21) and never uses.
// Only differences of m enter, so m is taken relative to the first contribution's value m0 (mapped depths of one ray
// sit close together just below 1; their squares would cancel). Accumulated front to back as
// dist += w (m^2 A + M2 - 2 m M1), M1 += m w, M2 += m^2 w, A = 1 - T_prev. Gradient, with the totals W = sum w (the
// accumulated opacity), M1, M2 of the whole segment, mu = M1 / W, c_k = m_k - mu, V = M2 - M1^2 / W = sum w c^2:
// d dist / d m_k = 2 w_k W c_k, d dist / d w_k = W c_k^2 + V, and through w_i = alpha_i T_{i-1}:
// d dist / d alpha_k = (d dist / d w_k) T_{k-1} - [W (V - V_k) + V (W - W_k)] / (1 - alpha_k), the bracket being
// sum_{i>k} (d dist / d w_i) w_i written with the running sums V_k = sum_{j<=k} w_j c_j^2 and W_k through k.
static const float DIST_K = 100.0f / (100.0f - 0.2f);
static void trace_ray(const Ctx& cx, int ray, F3 ray_o, F3 ray_d, float min_depth, float T_threshold,
                      TraceOut& out, TraceBwd* bw, Tally& tl, bool dist_on = false)
{
    const OrcArgs& A = *cx.a;
    uint64_t buf[orc::KCHUNK];
    int last_gidx = -1, contributor = 0;
    float T_prev = 1.0f, T_next = 1.0f, dpt = 0.0f;
    float offset = 0.0f;                      // payload.dpt
    F3 ray_ot = ray_o;
    float c[3] = { 0, 0, 0 }, clamped[3] = { 0, 0, 0 };
    float W = 0.0f;                           // never updated by the reference (backward.cu:359, 568)
    float Wsum = 0.0f, Vsum = 0.0f;           // running sums of w and w c^2, for the distortion gradient
    bool dist_first = true;
    const float T_final = bw ? 1.0f - bw->out_acc : 0.f;
    tl.segs++;

    for (int chunk = 0; chunk < MAX_CHUNKS; chunk++) {
        float o3[3] = { ray_ot.x, ray_ot.y, ray_ot.z }, d3[3] = { ray_d.x, ray_d.y, ray_d.z };
        int cnt = cx.sc->knearest(o3, d3, buf, &tl.tests);       // forward.cu:194 (+ __anyhit__ot 481-525)
        tl.enums++;
        bool stop = false;
        for (int i = 0; i < cnt; i++) {
            int pidx = (int)orc::key_pidx(buf[i]);
            int gidx = pidx / 2;
            if (gidx == last_gidx) continue;                       // forward.cu:207-208
            tl.evals++;
            dpt = orc::key_t(buf[i]) + offset;                     // :211
            F3 xyz = ray_o + dpt * ray_d;                          // :212
            // compute_transmat_uv, forward.cu:63-90
            F3 p_orig = ld3(A.means3D + 3 * (size_t)gidx);
            F2 scale = mk2(A.scales[2 * (size_t)gidx], A.scales[2 * (size_t)gidx + 1]);
            const float* rot = A.rotations + 4 * (size_t)gidx;
            F3 R[3]; quat_rows(rot, R);
            F3 Tt = mk3(dot(R[0], p_orig), dot(R[1], p_orig), dot(R[2], p_orig));
            F3 normal = R[2];
            float uvx = R[0].x * xyz.x + R[0].y * xyz.y + R[0].z * xyz.z + (-Tt.x) * 1.0f;
            float uvy = R[1].x * xyz.x + R[1].y * xyz.y + R[1].z * xyz.z + (-Tt.y) * 1.0f;
            F2 uv = mk2(uvx / scale.x, uvy / scale.y);
            float rho3d = dot(uv, uv);
            // DUAL_VISIABLE, forward.cu:226-232
            float cosv = -sumf3(ray_d * normal);
            if (cosv == 0) continue;
            float normal_sign = cosv > 0 ? 1.0f : -1.0f;
            normal = normal_sign * normal;
            if (dpt < min_depth) continue;                         // :235
            float power = -0.5f * rho3d;
            if (power > 0.0f) continue;                            // :240
            const float opac = A.opacities[gidx];
            const float G = A.portable_exp ? orc::pexp(power) : expf(power);
            float alpha = std::min(0.99f, opac * G);               // :247
            if (A.fragile && fabsf(alpha - 1.0f / 255.0f) < 3e-8f) A.fragile[ray] = 1;
            if (alpha < 1.0f / 255.0f) continue;
            T_next = T_prev * (1 - alpha);                         // :250
            if (A.fragile && fabsf(T_next - T_threshold) < 2e-8f) A.fragile[ray] = 1;
            if (T_next < T_threshold) { stop = true; break; }
            contributor++;
            if (contributor > MAX_INTERSECTION) { stop = true; break; }   // :254-257
            last_gidx = gidx;
            tl.contribs++;
            if (A.hit_log) { int k = A.hit_cnt[ray]; if (k < A.hit_cap) A.hit_log[(size_t)ray * A.hit_cap + k] = pidx; A.hit_cnt[ray] = k + 1; }
            float w = alpha * T_prev;
            if (A.colors_precomp == nullptr) {                     // :265-276
                F3 result = sh_color(A.D, A.shs + 3 * (size_t)gidx * A.M, ray_d, clamped);
                out.C[0] += w * result.x; out.C[1] += w * result.y; out.C[2] += w * result.z;
                c[0] = result.x; c[1] = result.y; c[2] = result.z;
            } else {
                for (int ch = 0; ch < 3; ch++) { c[ch] = A.colors_precomp[ch + 3 * (size_t)gidx]; out.C[ch] += w * c[ch]; }
            }
            if (A.others_precomp != nullptr)
                for (int ch = 0; ch < AUX_CHANNELS; ch++) out.O[ch] += w * A.others_precomp[ch + AUX_CHANNELS * (size_t)gidx];
            out.D += w * dpt;
            out.N += w * normal;
            float dist_m = 0.0f;
            if (dist_on) {
                const float m_abs = DIST_K * (1.0f - 0.2f / dpt);
                if (dist_first) { out.m0 = m_abs; dist_first = false; }
                dist_m = m_abs - out.m0;
                out.Dist += w * (dist_m * dist_m * (1.0f - T_prev) + out.M2 - 2.0f * dist_m * out.M1);
                out.M1 += dist_m * w; out.M2 += dist_m * dist_m * w;
            }

            if (!bw) {
                if (A.training && A.a_weights) atomic_add(A.a_weights + gidx, w);   // forward.cu:291-296
            } else {
                // backward.cu:529-568
                float dL_dalpha = 0.0f;
                float numerator = 1.0f - alpha;
                float dL_dcolor[3];
                for (int ch = 0; ch < 3; ch++) {
                    const float channel = c[ch], dL_dchannel = bw->dL_drgb[ch];
                    dL_dcolor[ch] = dL_dchannel * w;
                    atomic_add(A.dL_dcolors + ch + 3 * (size_t)gidx, dL_dchannel * w);      // also in SH mode
                    dL_dalpha += dL_dchannel * (T_prev * channel - (bw->out_rgb[ch] - out.C[ch]) / numerator);
                    dL_dalpha += dL_dchannel * A.background[ch] * (-T_final / numerator);   // background counted twice, as the reference does
                }
                if (A.others_precomp != nullptr) {
                    for (int ch = 0; ch < AUX_CHANNELS; ch++) {
                        const float channel = A.others_precomp[ch + AUX_CHANNELS * (size_t)gidx], dL_dchannel = bw->dL_daux[ch];
                        atomic_add(A.dL_dothers + ch + AUX_CHANNELS * (size_t)gidx, dL_dchannel * w);
                        dL_dalpha += dL_dchannel * (T_prev * channel - (bw->out_aux[ch] - out.O[ch]) / numerator);
                    }
                }
                float dL_dD = bw->dL_ddpt * w;
                dL_dalpha += bw->dL_ddpt * (T_prev * dpt - (bw->out_dpt - out.D) / numerator);
                F3 dL_dN = bw->dL_dnorm * w;
                dL_dalpha += sumf3(bw->dL_dnorm * (T_prev * normal - (bw->out_norm - out.N) / numerator));
                dL_dalpha += bw->dL_dacc * (T_prev * 1.f - (bw->out_acc - W) / numerator);
                if (dist_on) {
                    const float Wt = bw->out_acc, mu = bw->out_m1 / Wt, V = bw->out_m2 - bw->out_m1 * mu;
                    const float cm = dist_m - mu;
                    Wsum += w; Vsum += w * cm * cm;
                    const float d_dw = Wt * cm * cm + V;
                    const float behind = Wt * (V - Vsum) + V * (Wt - Wsum);
                    dL_dalpha += bw->dL_ddist * (d_dw * T_prev - behind / numerator);
                    dL_dD += bw->dL_ddist * 2.0f * w * Wt * cm * DIST_K * 0.2f / (dpt * dpt);
                }
                // :573-578
                const float dL_dG = dL_dalpha * opac;
                float power_clamped = (opac * G) > 0.99f ? 0.0f : 1.0f;
                atomic_add(A.dL_dopacities + gidx, dL_dalpha * G * power_clamped);
                // :581-602 triangle of the hit and its corner coordinates
                const float cutoff = 3.0f;
                const float* vb = A.vertices + 12 * (size_t)gidx;
                F3 v1, v2, v3, h1, h2, h3;
                if (pidx % 2 == 0) {
                    v1 = ld3(vb); v2 = ld3(vb + 3); v3 = ld3(vb + 6);
                    h1 = mk3(-1.0f, 1.0f, 1.0f) * cutoff; h2 = mk3(-1.0f, -1.0f, 1.0f) * cutoff; h3 = mk3(1.0f, 1.0f, 1.0f) * cutoff;
                } else {
                    v1 = ld3(vb + 3); v2 = ld3(vb + 6); v3 = ld3(vb + 9);
                    h1 = mk3(-1.0f, -1.0f, 1.0f) * cutoff; h2 = mk3(1.0f, 1.0f, 1.0f) * cutoff; h3 = mk3(1.0f, -1.0f, 1.0f) * cutoff;
                }
                // compute_transmat_uv_backward, backward.cu:201-287
                F2 dL_duv = dL_dG * power_clamped * -G * uv;
                F3 dL_dR[3];
                dL_dR[0] = dL_duv.x * (xyz - p_orig) / scale.x;
                dL_dR[1] = dL_duv.y * (xyz - p_orig) / scale.y;
                dL_dR[2] = dL_dN * normal_sign;
                F2 dL_dscale = dL_dG * power_clamped * (G * uv * uv / scale);
                F3 dG_dmean3D = G * (R[0] * uv.x / scale.x + R[1] * uv.y / scale.y);
                F3 dL_dmean3D = dL_dG * power_clamped * dG_dmean3D;
                F3 dL_dxyz = mk3(dL_duv.x / scale.x * R[0].x + dL_duv.y / scale.y * R[1].x,
                                 dL_duv.x / scale.x * R[0].y + dL_duv.y / scale.y * R[1].y,
                                 dL_duv.x / scale.x * R[0].z + dL_duv.y / scale.y * R[1].z);
                float dL_dd = dL_dD + dot(dL_dxyz, ray_d);
                F3 n = cross(v2 - v1, v3 - v1);
                F3 cc = v1 - ray_o;
                float p = dot(n, cc), q = dot(n, ray_d);
                F3 dL_dn = (cc - p / q * ray_d) / q;
                F3 dL_dv1 = dL_dd * cross(v2 - v3, dL_dn) + dL_dd * n / q;
                F3 dL_dv2 = dL_dd * cross(v3 - v1, dL_dn);
                F3 dL_dv3 = dL_dd * cross(v1 - v2, dL_dn);
                *bw->dL_dray_o += dL_dxyz + dL_dd * -n / q;
                *bw->dL_dray_d += dL_dxyz * dpt + dL_dd * -p / (q * q) * n;
                dL_dR[0].x += scale.x * (h1.x * dL_dv1.x + h2.x * dL_dv2.x + h3.x * dL_dv3.x);
                dL_dR[0].y += scale.x * (h1.x * dL_dv1.y + h2.x * dL_dv2.y + h3.x * dL_dv3.y);
                dL_dR[0].z += scale.x * (h1.x * dL_dv1.z + h2.x * dL_dv2.z + h3.x * dL_dv3.z);
                dL_dR[1].x += scale.y * (h1.y * dL_dv1.x + h2.y * dL_dv2.x + h3.y * dL_dv3.x);
                dL_dR[1].y += scale.y * (h1.y * dL_dv1.y + h2.y * dL_dv2.y + h3.y * dL_dv3.y);
                dL_dR[1].z += scale.y * (h1.y * dL_dv1.z + h2.y * dL_dv2.z + h3.y * dL_dv3.z);
                float dL_drot[4]; quat_rows_vjp(rot, dL_dR, dL_drot);
                dL_dscale.x += dot(R[0], h1.x * dL_dv1 + h2.x * dL_dv2 + h3.x * dL_dv3);
                dL_dscale.y += dot(R[1], h1.y * dL_dv1 + h2.y * dL_dv2 + h3.y * dL_dv3);
                dL_dmean3D += dL_dv1 + dL_dv2 + dL_dv3;
                // :609-626
                atomic_add(A.dL_dscales + 2 * (size_t)gidx, dL_dscale.x);
                atomic_add(A.dL_dscales + 2 * (size_t)gidx + 1, dL_dscale.y);
                for (int k = 0; k < 4; k++) atomic_add(A.dL_drotations + 4 * (size_t)gidx + k, dL_drot[k]);
                atomic_add(A.dL_dmeans3D + 3 * (size_t)gidx, dL_dmean3D.x);
                atomic_add(A.dL_dmeans3D + 3 * (size_t)gidx + 1, dL_dmean3D.y);
                atomic_add(A.dL_dmeans3D + 3 * (size_t)gidx + 2, dL_dmean3D.z);
                atomic_add(A.dL_dgrads3D + 3 * (size_t)gidx, dL_dmean3D.x * 0.5f * dpt);
                atomic_add(A.dL_dgrads3D + 3 * (size_t)gidx + 1, dL_dmean3D.y * 0.5f * dpt);
                atomic_add(A.dL_dgrads3D + 3 * (size_t)gidx + 2, dL_dmean3D.z * 0.5f * dpt);
                // :629-640
                if (A.colors_precomp == nullptr) {
                    F3 dL_dsh[16];
                    sh_color_vjp(A.D, A.shs + 3 * (size_t)gidx * A.M, ray_d, clamped, dL_dcolor, dL_dsh, *bw->dL_dray_d);
                    for (int j = 0; j < (A.D + 1) * (A.D + 1); j++) {
                        float* dst = A.dL_dshs + 3 * ((size_t)j + (size_t)A.M * gidx);
                        atomic_add(dst, dL_dsh[j].x); atomic_add(dst + 1, dL_dsh[j].y); atomic_add(dst + 2, dL_dsh[j].z);
                    }
                }
            }
            T_prev = T_next;
        }
        // forward.cu:299-306
        if (stop || T_next < T_threshold || cnt < orc::KCHUNK || contributor > MAX_INTERSECTION) break;
        offset = (float)((double)dpt + STEP_EPSILON);
        ray_ot = ray_o + offset * ray_d;
    }
    // forward.cu:309-314
    if (!bw) for (int ch = 0; ch < 3; ch++) out.C[ch] += T_prev * A.background[ch];
    out.A = 1 - T_prev;
    out.T = T_prev;
    out.E = ray_o + out.D * ray_d;
}

static float min_depth_of(const OrcArgs& A, int i) {     // forward.cu:353
    return (i == 0 && A.start_from_first) ? NEAR_N : (float)((i == 0 && !A.start_from_first) ? 0.0f : START_OFFSET);
}

// forward.cu:318-424 + 428-477
static void forward_ray(const Ctx& cx, int ray, Tally& tl) {
    const OrcArgs& A = *cx.a;
    F3 ray_o = ld3(A.ray_o + 3 * (size_t)ray), ray_d = ld3(A.ray_d + 3 * (size_t)ray);
    float out_rgb[3] = { 0, 0, 0 }, out_dpt = 0, out_acc = 0, out_aux[2] = { 0, 0 }, out_dist[3] = { 0, 0, 0 };
    F3 out_norm = mk3(0, 0, 0);
    float* mid = A.mid_val + (size_t)ray * A.mid_stride;
    for (int k = 0; k < A.mid_stride; k++) mid[k] = 0.0f;     // the reference leaves untraced bounces uninitialised (forward.cu:446)
    F3 ray_ot = ray_o, ray_dt = ray_d;
    float s_prod = 1.0f;
    for (int i = 0; i < A.max_trace_depth + 1; i++) {
        TraceOut t; memset(&t, 0, sizeof(t)); t.T = 1.0f;
        trace_ray(cx, ray, ray_ot, ray_dt, min_depth_of(A, i), 0.0001f, t, nullptr, tl, i == 0 && A.distortion);
        if (i == 0) { out_dist[0] = t.Dist; out_dist[1] = t.M1; out_dist[2] = t.M2; }
        if (i == 0) { out_dpt = t.D; out_acc = t.A; out_norm = t.N; out_aux[0] = t.O[0]; out_aux[1] = t.O[1]; }
        float f_this = (i == A.max_trace_depth) ? 1.0f : 1 - t.O[SPECULAR];
        for (int ch = 0; ch < 3; ch++) out_rgb[ch] += t.C[ch] * f_this * s_prod;
        s_prod *= t.O[SPECULAR];
        float* m = mid + i * MID_CHANNELS;
        m[RAYO_MID] = ray_ot.x; m[RAYO_MID + 1] = ray_ot.y; m[RAYO_MID + 2] = ray_ot.z;
        m[RAYD_MID] = ray_dt.x; m[RAYD_MID + 1] = ray_dt.y; m[RAYD_MID + 2] = ray_dt.z;
        for (int ch = 0; ch < 3; ch++) m[RGB_MID + ch] = t.C[ch];
        m[DPT_MID] = t.D; m[ACC_MID] = t.A;
        m[NORM_MID] = t.N.x; m[NORM_MID + 1] = t.N.y; m[NORM_MID + 2] = t.N.z;
        m[AUX_MID] = t.O[0]; m[AUX_MID + 1] = t.O[1];
        if (A.fragile && i < A.max_trace_depth && length(t.N) != 0.0f && fabsf(t.O[SPECULAR] - A.specular_threshold) < 1e-5f) A.fragile[ray] = 1;
        if (length(t.N) == 0.0f || t.O[SPECULAR] <= A.specular_threshold) break;    // :416
        F3 n = normalize(t.N);
        ray_dt = ray_dt - 2 * dot(n, ray_dt) * n;                                     // :421
        ray_ot = t.E + (float)START_OFFSET * ray_dt;                                  // :422
    }
    for (int ch = 0; ch < 3; ch++) A.out_rgb[3 * (size_t)ray + ch] = out_rgb[ch];
    A.out_dpt[ray] = out_dpt; A.out_acc[ray] = out_acc;
    A.out_norm[3 * (size_t)ray] = out_norm.x; A.out_norm[3 * (size_t)ray + 1] = out_norm.y; A.out_norm[3 * (size_t)ray + 2] = out_norm.z;
    // zeros as upstream (forward.cu:286) unless the distortion extension is on: then the sum and the two moments its gradient needs
    for (int k = 0; k < 3; k++) A.out_dist[3 * (size_t)ray + k] = out_dist[k];
    A.out_aux[2 * (size_t)ray] = out_aux[0]; A.out_aux[2 * (size_t)ray + 1] = out_aux[1];
}

// backward.cu:658-853 + 857-928
static void backward_ray(const Ctx& cx, int ray, Tally& tl) {
    const OrcArgs& A = *cx.a;
    const int depth = A.max_trace_depth;
    const float* mid = A.mid_val + (size_t)ray * A.mid_stride;
    float out_rgb[3]; for (int ch = 0; ch < 3; ch++) out_rgb[ch] = A.out_rgb[3 * (size_t)ray + ch];
    float g_rgb[3]; for (int ch = 0; ch < 3; ch++) g_rgb[ch] = A.dL_drgb[3 * (size_t)ray + ch];
    const float g_dpt = A.dL_ddpt[ray], g_acc = A.dL_dacc[ray];
    const F3 g_norm = ld3(A.dL_dnorm + 3 * (size_t)ray);
    const float g_aux[2] = { A.dL_daux[2 * (size_t)ray], A.dL_daux[2 * (size_t)ray + 1] };
    F3 dL_dray_o = mk3(0, 0, 0), dL_dray_d = mk3(0, 0, 0);

    // :683-703 rebuild the specular product and the colour seen "behind" each bounce
    float C_prev[3] = { out_rgb[0], out_rgb[1], out_rgb[2] }, c_prev[3] = { 0, 0, 0 };
    float s_prod = 1.0f;
    for (int i = 0; i < depth; i++) {
        for (int ch = 0; ch < 3; ch++) {
            float c_curr = mid[ch + RGB_MID + i * MID_CHANNELS];
            C_prev[ch] = C_prev[ch] + s_prod * (c_prev[ch] - c_curr);
            c_prev[ch] = c_curr;
        }
        s_prod *= mid[SPECULAR + AUX_MID + i * MID_CHANNELS];
    }
    for (int i = depth; i >= 0; i--) {
        const float* m = mid + i * MID_CHANNELS;
        F3 ray_ot = ld3(m + RAYO_MID), ray_dt = ld3(m + RAYD_MID);
        float s_prev = (i > 0) ? mid[SPECULAR + AUX_MID + (i - 1) * MID_CHANNELS] : 1.0f;
        if (length(ray_dt) == 0.0f || s_prev <= A.specular_threshold) continue;       // :724 (skips the s_prod update below)
        TraceBwd b;
        for (int ch = 0; ch < 3; ch++) b.out_rgb[ch] = m[RGB_MID + ch];
        b.out_dpt = m[DPT_MID]; b.out_acc = m[ACC_MID]; b.out_norm = ld3(m + NORM_MID);
        b.out_aux[0] = m[AUX_MID]; b.out_aux[1] = m[AUX_MID + 1];
        b.dL_ddpt = 0; b.dL_dacc = 0; b.dL_dnorm = mk3(0, 0, 0); b.dL_daux[0] = b.dL_daux[1] = 0;
        float f_this = (i == depth) ? 1.0f : 1 - b.out_aux[SPECULAR];
        for (int ch = 0; ch < 3; ch++) b.dL_drgb[ch] = g_rgb[ch] * f_this * s_prod;   // :760
        s_prod /= s_prev;                                                              // :762
        if (i != depth) {
            for (int ch = 0; ch < 3; ch++) {                                           // :769-774
                b.dL_daux[SPECULAR] += g_rgb[ch] * (C_prev[ch] / b.out_aux[SPECULAR]);
                c_prev[ch] = (i > 0) ? mid[ch + RGB_MID + (i - 1) * MID_CHANNELS] : 0.0f;
                C_prev[ch] = C_prev[ch] - s_prod * (c_prev[ch] - b.out_rgb[ch]);
            }
            if (length(b.out_norm) != 0) {                                             // :778-790
                dL_dray_d = dL_dray_d + dL_dray_o * (float)STEP_EPSILON;
                F3 n = normalize(b.out_norm);
                b.dL_ddpt += sumf3(dL_dray_o * ray_dt);
                b.dL_dnorm += dnormvdv(b.out_norm, ddotndndn(n, ray_dt, dL_dray_d * -2.0f));
                dL_dray_d = dL_dray_o * b.out_dpt + dL_dray_d + ddotndndd(n, ray_dt, dL_dray_d * -2.0f);
            }
        }
        if (i == 0) {                                                                  // :793-802
            b.dL_ddpt += g_dpt; b.dL_dacc += g_acc; b.dL_dnorm += g_norm;
            b.dL_daux[0] += g_aux[0]; b.dL_daux[1] += g_aux[1];
        }
        b.dL_dray_o = &dL_dray_o; b.dL_dray_d = &dL_dray_d;
        const bool dist_on = i == 0 && A.distortion && A.dL_ddist && A.out_dist;
        b.dL_ddist = dist_on ? A.dL_ddist[ray] : 0.0f;
        b.out_m1 = dist_on ? A.out_dist[3 * (size_t)ray + 1] : 0.0f; b.out_m2 = dist_on ? A.out_dist[3 * (size_t)ray + 2] : 0.0f;
        TraceOut t; memset(&t, 0, sizeof(t)); t.T = 1.0f;
        trace_ray(cx, ray, ray_ot, ray_dt, min_depth_of(A, i), 0.0001f, t, &b, tl, dist_on);
    }
    A.dL_dray_o[3 * (size_t)ray] = dL_dray_o.x; A.dL_dray_o[3 * (size_t)ray + 1] = dL_dray_o.y; A.dL_dray_o[3 * (size_t)ray + 2] = dL_dray_o.z;
    A.dL_dray_d[3 * (size_t)ray] = dL_dray_d.x; A.dL_dray_d[3 * (size_t)ray + 1] = dL_dray_d.y; A.dL_dray_d[3 * (size_t)ray + 2] = dL_dray_d.z;
}

template <bool BWD>
static void run(const orc::Scene* sc, const OrcArgs* a) {
    Ctx cx = { a, sc };
    const int R = a->H * a->W;
    long e = 0, t = 0, ev = 0, c = 0, s = 0;
    const int nt = a->nthreads > 0 ? a->nthreads : omp_get_max_threads();
#pragma omp parallel for schedule(dynamic, 64) num_threads(nt) reduction(+ : e, t, ev, c, s)
    for (int r = 0; r < R; r++) {
        Tally tl = { 0, 0, 0, 0, 0, 0 };
        if (BWD) backward_ray(cx, r, tl); else forward_ray(cx, r, tl);
        e += tl.enums; t += tl.tests; ev += tl.evals; c += tl.contribs; s += tl.segs;
    }
    if (a->stats) { a->stats[0] = e; a->stats[1] = t; a->stats[2] = ev; a->stats[3] = c; a->stats[4] = 0; a->stats[5] = s; }
}

} // namespace

extern "C" {

void* orc_scene_create(const float* vertices, int P, int brute) {
    orc::Scene* s = new orc::Scene();
    s->init(vertices, P, brute != 0);
    return s;
}
void orc_scene_destroy(void* s) { delete (orc::Scene*)s; }

// Output buffers must be zero-filled by the caller where they are accumulated into
// (a_weights, hit_cnt, fragile, every dL_d* per-surfel array), as torch::zeros does in
// trace_surfels.cpp:224-231, 376-387.
void orc_forward(void* scene, const OrcArgs* a) { run<false>((orc::Scene*)scene, a); }
void orc_backward(void* scene, const OrcArgs* a) { run<true>((orc::Scene*)scene, a); }

// enumerator access for tests: the 16 nearest hits of one ray -> keys; returns the count
int orc_knearest(void* scene, const float* o, const float* d, uint64_t* keys) { return ((orc::Scene*)scene)->knearest(o, d, keys); }
// every hit of one ray (brute force), up to cap keys; returns the total
int orc_all_hits(void* scene, const float* o, const float* d, uint64_t* keys, int cap) {
    std::vector<uint64_t> v; ((orc::Scene*)scene)->all_hits_brute(o, d, v);
    for (int i = 0; i < (int)v.size() && i < cap; i++) keys[i] = v[i];
    return (int)v.size();
}
// plane frames of all quads, 12 floats each (p0, n, wu, wv)
void orc_quad_records(void* scene, float* out) {
    orc::Scene* s = (orc::Scene*)scene;
    memcpy(out, s->quads.data(), sizeof(orc::QuadRec) * (size_t)s->P);
}
int orc_cpu_has_fma() { return __builtin_cpu_supports("fma") ? 1 : 0; }
}
