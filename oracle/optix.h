// TEST INFRASTRUCTURE ONLY. Host stand-in for the OptiX device API, placed first on the include
// path when the reference's shader sources (optix_tracer/forward.cu, backward.cu) are compiled
// for the CPU by ref_driver.cpp. It declares only what those two files use
// (optix_tracer/forward.cu:3, 119-131, 158-159, 110-111, 488-489, 524); ref_driver.cpp defines it.
#pragma once
#include <cuda_runtime.h>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <algorithm>

typedef unsigned long long OptixTraversableHandle;
typedef unsigned int OptixVisibilityMask;
enum { OPTIX_RAY_FLAG_NONE = 0 };

// CUDA's mixed-type min/max overloads and float math the shaders rely on
#define ORC_MINMAX(T, U, R) \
    static inline R min(T a, U b) { return (R)a < (R)b ? (R)a : (R)b; } \
    static inline R max(T a, U b) { return (R)a > (R)b ? (R)a : (R)b; }
ORC_MINMAX(int, int, int) ORC_MINMAX(unsigned, unsigned, unsigned) ORC_MINMAX(unsigned, int, unsigned) ORC_MINMAX(int, unsigned, unsigned)
ORC_MINMAX(float, float, float) ORC_MINMAX(double, double, double) ORC_MINMAX(float, double, double) ORC_MINMAX(double, float, double)
extern int g_orc_portable_exp;                                 // set per run by ref_driver.cpp
float orc_portable_exp(float x);
// device code resolves exp(float) to the float overload
static inline float exp(float x) { return g_orc_portable_exp ? orc_portable_exp(x) : expf(x); }
static inline float rsqrtf(float x) { return 1.0f / sqrtf(x); }
static inline void __trap() { abort(); }
float atomicAdd(float* p, float v);

uint3 optixGetLaunchIndex();
uint3 optixGetLaunchDimensions();
unsigned optixGetPayload_0();
unsigned optixGetPayload_1();
float optixGetRayTmax();
unsigned optixGetPrimitiveIndex();
void optixIgnoreIntersection();
void optixTrace(OptixTraversableHandle, float3, float3, float, float, float, OptixVisibilityMask, int, int, int, int,
                unsigned&, unsigned&);
