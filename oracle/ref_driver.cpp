// TEST INFRASTRUCTURE ONLY. Compiles the reference's own shader source for the host.
//
// The reference's forward.cu / backward.cu are #included from where they lie (the build passes
// -I<reference>/optix_tracer); nothing of the reference is copied. Built four times by build.py:
// forward or backward (-DREF_BACKWARD), bounce capacity 1 or 2 (-DREF_MTD). Outputs go to
// oracle/_ref/ only. The OptiX entry points the shaders call are defined here on top of the
// enumerator in quad_enum.h, which stands in for the closed OptiX traversal.
//
// Two source-level problems of the reference are worked around with the preprocessor instead of
// editing it: quat_to_rotmat_transpose is declared to return float3 but never returns
// (optix_tracer/auxiliary.h:403-429), which is undefined behaviour on the host; and
// MAX_TRACE_DEPTH is a compile-time 1 (optix_tracer/config.h:27) while one workload needs 2.
#include "optix.h"
#include "quad_enum.h"
#include "orc_args.h"
#include <omp.h>

#ifndef REF_MTD
#define REF_MTD 1
#endif

#include "config.h"
#undef MAX_TRACE_DEPTH
#define MAX_TRACE_DEPTH REF_MTD

// turn `inline float3 quat_to_rotmat_transpose(A, B) {...}` into a void function of another name
#define quat_to_rotmat_transpose(A, B) orc_never_defined(); inline void orc_quat_rows(A, B)
#include "auxiliary.h"
#undef quat_to_rotmat_transpose
#define quat_to_rotmat_transpose orc_quat_rows

static thread_local uint3 g_idx, g_dim;
static thread_local unsigned g_p0, g_p1, g_prim;
static thread_local float g_t;
static thread_local long g_anyhit, g_enums, g_contrib;
int g_orc_portable_exp = 0;
float orc_portable_exp(float x) { return orc::pexp(x); }
static const orc::Scene* g_scene;
static const OrcArgs* g_args;

uint3 optixGetLaunchIndex() { return g_idx; }
uint3 optixGetLaunchDimensions() { return g_dim; }
unsigned optixGetPayload_0() { return g_p0; }
unsigned optixGetPayload_1() { return g_p1; }
float optixGetRayTmax() { return g_t; }
unsigned optixGetPrimitiveIndex() { return g_prim; }
void optixIgnoreIntersection() {}

#ifdef REF_BACKWARD
#include "backward.cu"
#else
#include "forward.cu"
#endif

// a_weights is the only per-surfel array the forward shader adds to (forward.cu:295): use it to log contributions
float atomicAdd(float* p, float v) {
    const OrcArgs* a = g_args;
    if (a->hit_log && a->a_weights && p >= a->a_weights && p < a->a_weights + a->P) {
        int ray = (int)(g_idx.x * g_dim.y + g_idx.y);
        int k = a->hit_cnt[ray];
        if (k < a->hit_cap) a->hit_log[(size_t)ray * a->hit_cap + k] = (int)(p - a->a_weights);
        a->hit_cnt[ray] = k + 1;
        g_contrib++;
    }
#pragma omp atomic
    *p += v;
    return 0.f;
}

// Stand-in for OptiX traversal: every quad hit with 0 <= t < 1e16 is handed to the reference's
// any-hit program in ascending (t, primitive id) order.
void optixTrace(OptixTraversableHandle, float3 o, float3 d, float, float, float, OptixVisibilityMask, int, int, int, int,
                unsigned& p0, unsigned& p1) {
    g_p0 = p0; g_p1 = p1; g_enums++;
    if (g_args->clean) {
        RayPayload* pl = (RayPayload*)(((uint64_t)p0 << 32) | p1);      // forward.cu:94-113
        for (int i = 0; i < CHUNK_SIZE; i++) { pl->buffer[i].tmx = DEPTH_INFINTY; pl->buffer[i].idx = 0; }
    }
    static thread_local std::vector<uint64_t> hits;
    float o3[3] = { o.x, o.y, o.z }, d3[3] = { d.x, d.y, d.z };
    g_scene->all_hits(o3, d3, hits);
    for (uint64_t k : hits) { g_t = orc::key_t(k); g_prim = orc::key_pidx(k); g_anyhit++; __anyhit__ot(); }
}

extern "C" {

int ref_mid_stride() { return MID_CHANNELS * (MAX_TRACE_DEPTH + 1); }

// Fills the reference's launch-parameter block (trace_surfels.cpp:235-285, 390-446) and runs
// its ray-generation program once per ray (optixLaunch(H, W, 1), trace_surfels.cpp:295, 456).
void ref_run(void* scene, const OrcArgs* a) {
    g_scene = (const orc::Scene*)scene; g_args = a; g_orc_portable_exp = a->portable_exp;
    params = Params();
    params.P = a->P; params.H = a->H; params.W = a->W; params.D = a->D; params.M = a->M;
    params.max_trace_depth = a->max_trace_depth; params.specular_threshold = a->specular_threshold;
    params.training = a->training != 0; params.start_from_first = a->start_from_first != 0;
    params.scale_modifier = a->scale_modifier;
    params.ray_o = (float3*)a->ray_o; params.ray_d = (float3*)a->ray_d; params.vertices = (float3*)a->vertices;
    params.background = (float*)a->background; params.means3D = (float3*)a->means3D; params.shs = (float3*)a->shs;
    params.colors_precomp = (float*)a->colors_precomp; params.others_precomp = (float*)a->others_precomp;
    params.opacities = (float*)a->opacities; params.scales = (float2*)a->scales; params.rotations = (float4*)a->rotations;
    params.out_rgb = a->out_rgb; params.out_dpt = a->out_dpt; params.out_acc = a->out_acc;
    params.out_norm = (float3*)a->out_norm; params.out_dist = (float3*)a->out_dist; params.out_aux = a->out_aux;
    params.mid_val = a->mid_val; params.a_weights = a->a_weights;
    params.dL_drgb = (float*)a->dL_drgb; params.dL_ddpt = (float*)a->dL_ddpt; params.dL_dacc = (float*)a->dL_dacc;
    params.dL_ddist = (float*)a->dL_ddist; params.dL_dnorm = (float3*)a->dL_dnorm; params.dL_daux = (float*)a->dL_daux;
    params.dL_dray_o = (float3*)a->dL_dray_o; params.dL_dray_d = (float3*)a->dL_dray_d;
    params.dL_dmeans3D = (float3*)a->dL_dmeans3D; params.dL_dgrads3D = (float3*)a->dL_dgrads3D;
    params.dL_dshs = (float3*)a->dL_dshs; params.dL_dcolors = a->dL_dcolors; params.dL_dothers = a->dL_dothers;
    params.dL_dopacities = a->dL_dopacities; params.dL_dscales = (float2*)a->dL_dscales; params.dL_drotations = (float4*)a->dL_drotations;
    const int R = a->H * a->W;
    long ah = 0, en = 0, co = 0;
    const int nt = a->nthreads > 0 ? a->nthreads : omp_get_max_threads();
#pragma omp parallel for schedule(dynamic, 64) num_threads(nt) reduction(+ : ah, en, co)
    for (int r = 0; r < R; r++) {
        g_idx = make_uint3(r / a->W, r % a->W, 0); g_dim = make_uint3(a->H, a->W, 1);
        g_anyhit = 0; g_enums = 0; g_contrib = 0;
        __raygen__ot();
        ah += g_anyhit; en += g_enums; co += g_contrib;
    }
    if (a->stats) { a->stats[0] = en; a->stats[1] = 0; a->stats[2] = 0; a->stats[3] = co; a->stats[4] = ah; a->stats[5] = 0; }
}
}
