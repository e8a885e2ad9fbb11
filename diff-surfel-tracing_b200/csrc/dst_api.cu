// C ABI of the surfel tracer (include/dst.h): handle life cycle, argument checks, error strings.
#include "dst_common.cuh"
#include <stdarg.h>
#include <string.h>
#include <new>
#include <nvtx3/nvToolsExt.h>       // header-only: ranges cost nothing unless a profiler is attached

static char g_global_err[512] = "";

int dst_set_error(dst_handle* h, int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(h ? h->err : g_global_err, 512, fmt, ap);
    va_end(ap);
    return code;
}
void dst_global_error(const char* msg) { snprintf(g_global_err, sizeof(g_global_err), "%s", msg); }

void dst_prof_mark(dst_handle* h, int kind, int which_end, cudaStream_t st) {
    if (!h->profiling || (kind == 3 && h->profiling < 2)) return;
    if (!h->ev[kind]) {
        h->ev[kind] = new (std::nothrow) cudaEvent_t[2 * DST_PROF_SLOTS];
        if (!h->ev[kind]) return;
        for (int i = 0; i < 2 * DST_PROF_SLOTS; i++) cudaEventCreate(&h->ev[kind][i]);
        h->ev_n[kind] = 0;
    }
    if (which_end == 0) {
        if (h->ev_n[kind] >= DST_PROF_SLOTS) return;
        cudaEventRecord(h->ev[kind][2 * h->ev_n[kind]], st);
    } else {
        if (h->ev_n[kind] >= DST_PROF_SLOTS) return;
        cudaEventRecord(h->ev[kind][2 * h->ev_n[kind] + 1], st);
        h->ev_n[kind]++;
    }
}

namespace {
// NVTX range around the host side of one entry point (the kernels it enqueues are attributed to it by profilers)
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
};

// streaming read of a buffer that fits the L2 cache, for the L2 bandwidth figure reports quote beside the HBM one
__global__ void __launch_bounds__(256) k_stream_read(const float4* __restrict__ buf, long long n_vec, int reps, float* sink) {
    float acc = 0.0f;
    for (int r = 0; r < reps; r++) {
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (long long)gridDim.x * blockDim.x) {
            float4 v;
            asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(buf + i));      // L2 only: every repetition really goes to the L2
            acc += v.x + v.y + v.z + v.w;
        }
    }
    if (acc == 123456.789f) *sink = acc;     // never true for a zeroed buffer; keeps the loads alive
}

struct DeviceGuard {
    int prev = -1; bool ok = true;
    explicit DeviceGuard(int dev) { if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; } if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false; }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};
}

extern "C" {

int dst_create(int device, dst_handle** out) {
    if (!out) { dst_global_error("dst_create: out is null"); return DST_E_ARG; }
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        dst_global_error("dst_create: no CUDA device is available (this library has no CPU path)");
        return DST_E_CUDA;
    }
    if (device < 0 || device >= count) { dst_global_error("dst_create: device index out of range"); return DST_E_ARG; }
    DeviceGuard g(device);
    if (!g.ok) { dst_global_error("dst_create: cudaSetDevice failed"); return DST_E_CUDA; }
    dst_handle* h = new (std::nothrow) dst_handle();
    if (!h) { dst_global_error("dst_create: out of host memory"); return DST_E_NOMEM; }
    memset(h, 0, sizeof(*h));
    h->device = device;
    h->wf_min_rays = 1 << 15;
    h->log_enabled = 1;
    h->stable_lists = 1;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { delete h; dst_global_error("dst_create: cudaGetDeviceProperties failed"); return DST_E_CUDA; }
    h->sm_count = prop.multiProcessorCount;
    if (cudaMalloc(&h->header, 4 * (DST_HDR_FLOATS + 8)) != cudaSuccess || cudaMalloc(&h->status, 4) != cudaSuccess ||
        cudaMemset(h->header, 0, 4 * (DST_HDR_FLOATS + 8)) != cudaSuccess || cudaMemset(h->status, 0, 4) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(h->header); cudaFree(h->status); delete h;
        dst_global_error("dst_create: device allocation failed");
        return DST_E_NOMEM;
    }
    *out = h;
    return DST_OK;
}

int dst_destroy(dst_handle* h) {
    if (!h) return DST_OK;
    DeviceGuard g(h->device);
    cudaFree(h->nodes); cudaFree(h->quads); cudaFree(h->leaf_gid); cudaFree(h->leaf_parent); cudaFree(h->arrive);
    cudaFree(h->node_parent); cudaFree(h->node_first); cudaFree(h->node_count); cudaFree(h->child_cost);
    cudaFree(h->keys); cudaFree(h->keys_alt); cudaFree(h->vals); cudaFree(h->vals_alt); cudaFree(h->block_hist);
    cudaFree(h->header); cudaFree(h->status); cudaFree(h->cache); cudaFree(h->arena); cudaFree(h->cam_dev);
    if (h->log_needed_host) cudaFreeHost(h->log_needed_host);
    if (h->log_needed_event) cudaEventDestroy(h->log_needed_event);
    if (h->rounds_host) cudaFreeHost(h->rounds_host);
    if (h->rounds_event) cudaEventDestroy(h->rounds_event);
    cudaFree(h->log_keys); cudaFree(h->log_hdr); cudaFree(h->log_count); cudaFree(h->log_seg_head); cudaFree(h->log_ray_ok);
    cudaFree(h->wf_state); cudaFree(h->wf_req); cudaFree(h->wf_kbuf); cudaFree(h->wf_kcnt); cudaFree(h->wf_list[0]); cudaFree(h->wf_list[1]); cudaFree(h->wf_counts);
    cudaFree(h->wf_tmp); cudaFree(h->wf_wcnt); cudaFree(h->wf_bcnt);
    cudaFree(h->bound_stats);
    if (h->bound_host) cudaFreeHost(h->bound_host);
    if (h->bound_event) cudaEventDestroy(h->bound_event);
    if (h->slice_streams_ready) {
        cudaEventDestroy(h->slice_fork);
        for (int g = 0; g < DST_MAX_SLICES - 1; g++) { cudaStreamDestroy(h->slice_stream[g]); cudaEventDestroy(h->slice_join[g]); }
    }
    for (int k = 0; k < 4; k++) {
        if (h->ev[k]) { for (int i = 0; i < 2 * DST_PROF_SLOTS; i++) cudaEventDestroy(h->ev[k][i]); delete[] h->ev[k]; }
    }
    delete h;
    return DST_OK;
}

const char* dst_last_error(const dst_handle* h) { return h ? h->err : g_global_err; }

int dst_build(dst_handle* h, const float* vertices, int64_t n_vertices, const int32_t* triangles, int64_t n_triangles,
              int rebuild, void* stream) {
    NvtxRange range("dst_build");
    if (!h) return DST_E_ARG;
    if (!vertices) return dst_set_error(h, DST_E_ARG, "vertices is null");
    if (n_vertices <= 0 || (n_vertices & 3)) return dst_set_error(h, DST_E_ARG, "vertices must hold 4 vertices per surfel, got %lld", (long long)n_vertices);
    if (triangles && n_triangles * 2 != n_vertices)
        return dst_set_error(h, DST_E_ARG, "triangles must hold 2 per surfel: %lld triangles for %lld vertices", (long long)n_triangles, (long long)n_vertices);
    DeviceGuard g(h->device);
    if (!g.ok) return dst_set_error(h, DST_E_CUDA, "cudaSetDevice(%d) failed", h->device);
    h->log_serial = 0;      // the logged chunks refer to the hierarchy that is about to change
    return dst_bvh_build_impl(h, vertices, n_vertices / 4, rebuild, (cudaStream_t)stream);
}

int dst_surfel_quads(dst_handle* h, const float* means3D, const float* scales, const float* rotations, int64_t n_surfels,
                     float* vertices, int32_t* triangles, void* stream) {
    if (!h) return DST_E_ARG;
    if (!means3D || !scales || !rotations || !vertices) return dst_set_error(h, DST_E_ARG, "a required pointer is null");
    DeviceGuard g(h->device);
    if (!g.ok) return dst_set_error(h, DST_E_CUDA, "cudaSetDevice(%d) failed", h->device);
    return dst_surfel_quads_impl(h, means3D, scales, rotations, n_surfels, vertices, triangles, (cudaStream_t)stream);
}

int dst_build_from_surfels(dst_handle* h, const float* means3D, const float* scales, const float* rotations, int64_t n_surfels,
                           float* vertices, int rebuild, void* stream) {
    NvtxRange range("dst_build_from_surfels");
    if (!h) return DST_E_ARG;
    if (!means3D || !scales || !rotations || !vertices) return dst_set_error(h, DST_E_ARG, "a required pointer is null");
    DeviceGuard g(h->device);
    if (!g.ok) return dst_set_error(h, DST_E_CUDA, "cudaSetDevice(%d) failed", h->device);
    h->log_serial = 0;
    return dst_bvh_build_impl(h, vertices, n_surfels, rebuild, (cudaStream_t)stream, means3D, scales, rotations);
}

int dst_pinhole_rays(dst_handle* h, const dst_camera* cameras, int n_cameras, int H, int W, float* ray_o, float* ray_d, void* stream) {
    if (!h) return DST_E_ARG;
    if (!cameras || !ray_o || !ray_d) return dst_set_error(h, DST_E_ARG, "a required pointer is null");
    DeviceGuard g(h->device);
    if (!g.ok) return dst_set_error(h, DST_E_CUDA, "cudaSetDevice(%d) failed", h->device);
    return dst_pinhole_rays_impl(h, cameras, n_cameras, H, W, ray_o, ray_d, (cudaStream_t)stream);
}

int dst_forward_camera(dst_handle* h, const dst_fwd_args* args, const dst_camera* camera, void* stream) {
    NvtxRange range("dst_forward_camera");
    if (!h) return DST_E_ARG;
    if (!args || !camera) return dst_set_error(h, DST_E_ARG, "args or camera is null");
    DeviceGuard g(h->device);
    if (!g.ok) return dst_set_error(h, DST_E_CUDA, "cudaSetDevice(%d) failed", h->device);
    return dst_forward_camera_impl(h, args, camera, (cudaStream_t)stream);
}

int dst_forward(dst_handle* h, const dst_fwd_args* args, void* stream) {
    NvtxRange range("dst_forward");
    if (!h) return DST_E_ARG;
    if (!args) return dst_set_error(h, DST_E_ARG, "args is null");
    DeviceGuard g(h->device);
    if (!g.ok) return dst_set_error(h, DST_E_CUDA, "cudaSetDevice(%d) failed", h->device);
    return dst_forward_impl(h, args, (cudaStream_t)stream);
}

int dst_backward(dst_handle* h, const dst_bwd_args* args, void* stream) {
    NvtxRange range("dst_backward");
    if (!h) return DST_E_ARG;
    if (!args) return dst_set_error(h, DST_E_ARG, "args is null");
    DeviceGuard g(h->device);
    if (!g.ok) return dst_set_error(h, DST_E_CUDA, "cudaSetDevice(%d) failed", h->device);
    return dst_backward_impl(h, args, (cudaStream_t)stream);
}

int dst_status(dst_handle* h, uint32_t* flags, void* stream) {
    if (!h || !flags) return DST_E_ARG;
    DeviceGuard g(h->device);
    cudaStream_t st = (cudaStream_t)stream;
    DST_CUDA_TRY(h, cudaMemcpyAsync(flags, h->status, 4, cudaMemcpyDeviceToHost, st));
    DST_CUDA_TRY(h, cudaMemsetAsync(h->status, 0, 4, st));
    DST_CUDA_TRY(h, cudaStreamSynchronize(st));
    return DST_OK;
}

int dst_bvh_info(const dst_handle* h, int64_t* surfels, int64_t* nodes, int64_t* device_bytes) {
    if (!h) return DST_E_ARG;
    if (surfels) *surfels = h->built ? h->P : 0;
    if (nodes) *nodes = h->built ? (h->P > 1 ? h->P - 1 : 1) : 0;
    if (device_bytes) *device_bytes = h->cap * (64 + 48 + 4 + 4 + 4 + 16 + 8 + 20) + h->hist_cap * 1024 + h->cache_cap * 64 + h->arena_cap * 4 * DST_ARENA_FLOATS +
                                      h->wf_cap * (long long)(h->wf_state_bytes + 32 + 8 * DST_CHUNK + 4 + 8 + 4 + 4);
    return DST_OK;
}

int dst_debug_knearest(dst_handle* h, const float* ray_o, const float* ray_d, int64_t n_rays, unsigned long long* keys,
                       int32_t* counts, int brute, const float* t_cut, unsigned long long* counters, void* stream) {
    if (!h) return DST_E_ARG;
    if (!ray_o || !ray_d || !keys || !counts) return dst_set_error(h, DST_E_ARG, "null pointer");
    DeviceGuard g(h->device);
    return dst_knearest_impl(h, ray_o, ray_d, n_rays, keys, counts, brute, t_cut, counters, (cudaStream_t)stream);
}

int dst_set_option(dst_handle* h, int option, int64_t value) {
    if (!h) return DST_E_ARG;
    switch (option) {
        case DST_OPT_WAVEFRONT_MIN_RAYS: h->wf_min_rays = value < 0 ? 0 : value; return DST_OK;
        case DST_OPT_CHUNK_LOG_MAX_RECORDS: h->log_max_records = value < 0 ? 0 : value; h->log_serial = 0; return DST_OK;
        case DST_OPT_IMAGE_WIDTH: h->image_width = value < 0 ? 0 : value; h->log_serial = 0; return DST_OK;
        case DST_OPT_SINGLE_KERNEL_REFIT: h->single_kernel_refit = value != 0; return DST_OK;
        case DST_OPT_DISTORTION: h->distortion = value != 0; return DST_OK;
        case DST_OPT_STABLE_LISTS: h->stable_lists = value != 0; return DST_OK;
        case DST_OPT_FORWARD_SLICES: h->fwd_slices = value < 0 ? 0 : (value > DST_MAX_SLICES ? DST_MAX_SLICES : (int)value); return DST_OK;
        case DST_OPT_CHUNK_LOG: h->log_enabled = value != 0; if (!h->log_enabled) h->log_serial = 0; return DST_OK;
        default: return dst_set_error(h, DST_E_ARG, "unknown option %d", option);
    }
}

int dst_forward_serial(const dst_handle* h, unsigned long long* serial) {
    if (!h || !serial) return DST_E_ARG;
    *serial = h->log_serial;
    return DST_OK;
}

int dst_kernel_launches(const dst_handle* h, int64_t* launches) {
    if (!h || !launches) return DST_E_ARG;
    *launches = h->launches;
    return DST_OK;
}

int dst_profile_enable(dst_handle* h, int on) {
    if (!h) return DST_E_ARG;
    h->profiling = on < 0 ? 0 : (on > 2 ? 2 : on);
    return DST_OK;
}

int dst_profile_launches(dst_handle* h, int which, float* ms, int32_t cap, int32_t* launches) {
    if (!h || which < 0 || which > 3 || !ms || !launches || cap < 0) return DST_E_ARG;
    DeviceGuard g(h->device);
    const int n = h->ev[which] ? h->ev_n[which] : 0;
    for (int i = 0; i < n; i++) {
        float one = 0.f;
        DST_CUDA_TRY(h, cudaEventSynchronize(h->ev[which][2 * i + 1]));
        DST_CUDA_TRY(h, cudaEventElapsedTime(&one, h->ev[which][2 * i], h->ev[which][2 * i + 1]));
        if (i < cap) ms[i] = one;
    }
    *launches = n;
    h->ev_n[which] = 0;
    return DST_OK;
}

int dst_profile_read(dst_handle* h, int which, float* ms_sum, int32_t* launches) {
    if (!h || which < 0 || which > 3 || !ms_sum || !launches) return DST_E_ARG;
    DeviceGuard g(h->device);
    float sum = 0.f;
    const int n = h->ev[which] ? h->ev_n[which] : 0;
    for (int i = 0; i < n; i++) {
        float ms = 0.f;
        DST_CUDA_TRY(h, cudaEventSynchronize(h->ev[which][2 * i + 1]));
        DST_CUDA_TRY(h, cudaEventElapsedTime(&ms, h->ev[which][2 * i], h->ev[which][2 * i + 1]));
        sum += ms;
    }
    *ms_sum = sum; *launches = n;
    h->ev_n[which] = 0;
    return DST_OK;
}

int dst_debug_round_counts(dst_handle* h, int32_t* counts, int32_t cap, void* stream) {
    if (!h || !counts || cap < 0) return DST_E_ARG;
    if (!h->wf_counts) return dst_set_error(h, DST_E_STATE, "no trace call has run on this handle");
    DeviceGuard g(h->device);
    const int n = cap < 50 ? cap : 50;      // DST_WF_ROUNDS + 2 list lengths
    // one set of counters per slice of the last forward call (one set for every other call): the lengths add up
    int32_t all[DST_MAX_SLICES * 100];
    const int sets = h->slices_used > 1 ? h->slices_used : 1;
    DST_CUDA_TRY(h, cudaMemcpyAsync(all, h->wf_counts, sizeof(int32_t) * 100 * (size_t)sets, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    DST_CUDA_TRY(h, cudaStreamSynchronize((cudaStream_t)stream));
    for (int i = 0; i < cap; i++) counts[i] = 0;
    for (int g = 0; g < sets; g++) for (int i = 0; i < n; i++) counts[i] += all[g * 100 + i];
    return DST_OK;
}

int dst_debug_read_bandwidth(dst_handle* h, int64_t bytes, int reps, float* gb_per_s, void* stream) {
    if (!h || !gb_per_s || bytes < (1 << 20) || reps < 1) return DST_E_ARG;
    DeviceGuard g(h->device);
    cudaStream_t st = (cudaStream_t)stream;
    float4* buf = nullptr; float* sink = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    const long long n_vec = bytes / 16;
    int rc = DST_OK;
    if (cudaMalloc(&buf, (size_t)n_vec * 16) != cudaSuccess || cudaMalloc(&sink, 4) != cudaSuccess) { cudaGetLastError(); rc = dst_set_error(h, DST_E_NOMEM, "bandwidth probe allocation failed"); }
    if (rc == DST_OK && (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess)) rc = dst_set_error(h, DST_E_CUDA, "event creation failed");
    if (rc == DST_OK) {
        cudaMemsetAsync(buf, 0, (size_t)n_vec * 16, st);
        const int grid = h->sm_count * 8;
        k_stream_read<<<grid, 256, 0, st>>>(buf, n_vec, 2, sink);          // warm the cache
        cudaEventRecord(e0, st);
        k_stream_read<<<grid, 256, 0, st>>>(buf, n_vec, reps, sink);
        cudaEventRecord(e1, st);
        float ms = 0.f;
        if (cudaEventSynchronize(e1) != cudaSuccess || cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess || !(ms > 0.f)) rc = dst_set_error(h, DST_E_CUDA, "bandwidth probe failed: %s", cudaGetErrorString(cudaGetLastError()));
        else *gb_per_s = (float)((double)n_vec * 16.0 * reps / (ms * 1e-3) / 1e9);
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(buf); cudaFree(sink);
    return rc;
}

int dst_debug_chunk_log(const dst_handle* h, int64_t* records_wanted, int64_t* records_held, int64_t* bytes_per_record) {
    if (!h) return DST_E_ARG;
    if (records_wanted) *records_wanted = (h->log_needed_host && h->log_needed_event && cudaEventQuery(h->log_needed_event) == cudaSuccess) ? *h->log_needed_host : -1;
    if (records_held) *records_held = h->log_cap;
    if (bytes_per_record) *bytes_per_record = 8 * DST_CHUNK + (int64_t)sizeof(int2);
    return DST_OK;
}

int dst_debug_quad_frames(dst_handle* h, float* out, void* stream) {
    if (!h) return DST_E_ARG;
    if (!out) return dst_set_error(h, DST_E_ARG, "null pointer");
    DeviceGuard g(h->device);
    return dst_export_frames_impl(h, out, (cudaStream_t)stream);
}

}  // extern "C"
