// TEST INFRASTRUCTURE ONLY -- CPU restatement of the two steps that feed the tracer in the reference's
// example pipeline. Nothing in the shipped library or package may call this file; the tests, the
// smoke check and the benchmark's CPU leg use it as the checker.
//
//   orc_surfel_quads   GaussianModel.get_triangles  (example/utils/gaussian_utils.py:176-210) with
//                      build_cov / build_scaling_rotation / build_rotation (:214-249, :273-296)
//   orc_pinhole_rays   get_rays -> get_rays_from_ij  (example/utils/ray_utils.py:80-136) with
//                      torch_inverse_3x3 (:19-60) and normalize (:12-15)
//
// The reference evaluates both with torch tensor ops whose summation order inside `@` and `norm`
// is not specified; this file fixes one order (every operation one IEEE binary32 rounding, compiled
// with -ffp-contract=off) and the CUDA kernels follow it bit for bit. Parity with the reference
// itself is pinned by golden vectors produced by running the reference's Python functions
// (tests/golden/make_golden_prep.py); they agree to a few units in the last place.
#include <cmath>
#include <cstdint>

namespace {

// build_rotation (gaussian_utils.py:214-249): q = r / ||r||, (w, x, y, z) order; columns 0 and 1
// of R are the two tangent directions of the surfel.
inline void tangent_columns(const float* r, float* c0, float* c1) {
    const float n = std::sqrt(((r[0] * r[0] + r[1] * r[1]) + r[2] * r[2]) + r[3] * r[3]);
    const float w = r[0] / n, x = r[1] / n, y = r[2] / n, z = r[3] / n;
    c0[0] = 1.0f - 2.0f * (y * y + z * z);
    c0[1] = 2.0f * (x * y + w * z);
    c0[2] = 2.0f * (x * z - w * y);
    c1[0] = 2.0f * (x * y - w * z);
    c1[1] = 1.0f - 2.0f * (x * x + z * z);
    c1[2] = 2.0f * (y * z + w * x);
}

}  // namespace

extern "C" {

// v (4P,3): corner k of surfel g is mean + (3 cu_k) (s_x R[:,0]) + (3 cv_k) (s_y R[:,1]) with
// (cu, cv) = (-1,+1), (-1,-1), (+1,+1), (+1,-1) (gaussian_utils.py:186-198; the third column of the
// splat-to-world matrix is zeroed at :180, the fourth is the mean). f (2P,3), nullable:
// (4g, 4g+1, 4g+2), (4g+1, 4g+2, 4g+3) (:201-205).
void orc_surfel_quads(int64_t P, const float* means, const float* scales, const float* rotations, float* v, int32_t* f) {
    static const float CU[4] = { -3.0f, -3.0f, 3.0f, 3.0f }, CV[4] = { 3.0f, -3.0f, 3.0f, -3.0f };
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < P; g++) {
        float c0[3], c1[3];
        tangent_columns(rotations + 4 * g, c0, c1);
        const float sx = scales[2 * g], sy = scales[2 * g + 1];
        for (int k = 0; k < 4; k++)
            for (int a = 0; a < 3; a++) {
                const float lu = c0[a] * sx, lv = c1[a] * sy;       // L = R diag(s_x, s_y, 1)  (:273-282)
                v[12 * g + 3 * k + a] = (lu * CU[k] + lv * CV[k]) + means[3 * g + a];
            }
        if (f) {
            const int32_t b = (int32_t)(4 * g);
            int32_t* o = f + 6 * g;
            o[0] = b; o[1] = b + 1; o[2] = b + 2; o[3] = b + 1; o[4] = b + 2; o[5] = b + 3;
        }
    }
}

// Constants of one camera: inverse intrinsics (torch_inverse_3x3, ray_utils.py:19-60, eps = float
// machine epsilon added to the determinant) and the centre -R^T T (:107). out: invK[9], centre[3].
void orc_camera_constants(const float* K, const float* R, const float* T, float* invK, float* centre) {
    const float r00 = K[0], r01 = K[1], r02 = K[2], r10 = K[3], r11 = K[4], r12 = K[5], r20 = K[6], r21 = K[7], r22 = K[8];
    float M[9];
    M[0] = r11 * r22 - r21 * r12;
    M[3] = -r10 * r22 + r20 * r12;
    M[6] = r10 * r21 - r20 * r11;
    M[1] = -r01 * r22 + r21 * r02;
    M[4] = r00 * r22 - r20 * r02;
    M[7] = -r00 * r21 + r20 * r01;
    M[2] = r01 * r12 - r11 * r02;
    M[5] = -r00 * r12 + r10 * r02;
    M[8] = r00 * r11 - r10 * r01;
    const float D = (r00 * M[0] + r01 * M[3]) + r02 * M[6];
    const float den = D + 1.1920928955078125e-07f;
    for (int i = 0; i < 9; i++) invK[i] = M[i] / den;
    for (int a = 0; a < 3; a++) centre[a] = -((R[0 + a] * T[0] + R[3 + a] * T[1]) + R[6 + a] * T[2]);
}

// ray_o, ray_d (H,W,3): pixel (i, j) -> xy1 = (j + 0.5, i + 0.5, 1) (:121-126), camera point
// invK xy1, world point R^T (camera point - T) (:127-128), direction = world point - centre,
// divided by (its norm + 1e-8) unless z_depth (:131-133).
void orc_pinhole_rays(int H, int W, const float* K, const float* R, const float* T, int correct_pix, int z_depth,
                      float* ray_o, float* ray_d) {
    float invK[9], c[3];
    orc_camera_constants(K, R, T, invK, c);
#pragma omp parallel for schedule(static)
    for (int i = 0; i < H; i++)
        for (int j = 0; j < W; j++) {
            const float x = correct_pix ? (float)j + 0.5f : (float)j, y = correct_pix ? (float)i + 0.5f : (float)i;
            float pc[3], d[3];
            for (int a = 0; a < 3; a++) pc[a] = ((invK[3 * a] * x + invK[3 * a + 1] * y) + invK[3 * a + 2]) - T[a];
            for (int a = 0; a < 3; a++) d[a] = ((R[a] * pc[0] + R[3 + a] * pc[1]) + R[6 + a] * pc[2]) - c[a];
            if (!z_depth) {
                const float n = std::sqrt((d[0] * d[0] + d[1] * d[1]) + d[2] * d[2]) + 1e-8f;
                for (int a = 0; a < 3; a++) d[a] = d[a] / n;
            }
            float* o = ray_o + 3 * ((size_t)i * W + j);
            float* dd = ray_d + 3 * ((size_t)i * W + j);
            for (int a = 0; a < 3; a++) { o[a] = c[a]; dd[a] = d[a]; }
        }
}

}  // extern "C"
