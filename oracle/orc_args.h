// TEST INFRASTRUCTURE ONLY (CPU oracle). Argument block shared by the two oracle builds and
// mirrored field for field by the ctypes structure in oracle/oracle.py.
// Field meanings follow the launch-parameter struct of the reference, optix_tracer/params.h:21-84.
#pragma once
#include <cstdint>

extern "C" {
struct OrcArgs {
    int32_t P, H, W, D, M;
    int32_t max_trace_depth, training, start_from_first;
    int32_t clean;          // 1: every enumeration starts from an empty 16-slot buffer; 0: verbatim reference behaviour
    int32_t nthreads;       // OpenMP threads (0 = default)
    int32_t mid_stride;     // floats of mid_val per ray
    int32_t hit_cap;        // slots of hit_log per ray
    int32_t portable_exp;   // 1: the Gaussian falloff uses orc::pexp (reproducible on the GPU); 0: libm expf
    int32_t distortion;     // 1: the depth-distortion output and its gradient (an extension: the reference leaves them at zero)
    float specular_threshold, scale_modifier;
    const float *ray_o, *ray_d, *vertices, *background, *means3D, *shs, *colors_precomp, *others_precomp,
                *opacities, *scales, *rotations;
    float *out_rgb, *out_dpt, *out_acc, *out_norm, *out_dist, *out_aux, *mid_val, *a_weights;
    const float *dL_drgb, *dL_ddpt, *dL_dacc, *dL_ddist, *dL_dnorm, *dL_daux;
    float *dL_dray_o, *dL_dray_d, *dL_dmeans3D, *dL_dgrads3D, *dL_dshs, *dL_dcolors, *dL_dothers,
          *dL_dopacities, *dL_dscales, *dL_drotations;
    int32_t *hit_log;       // (R, hit_cap) contributing ids in compositing order (restatement: primitive id; reference build: surfel id)
    int32_t *hit_cnt;       // (R,) number of contributions over all bounces
    uint8_t *fragile;       // (R,) 1 where a threshold decision sat within rounding distance (restatement only)
    int64_t *stats;         // [0] enumerations, [1] exact quad tests, [2] slots evaluated, [3] contributions, [4] any-hit invocations, [5] ray segments
};
}
