// Forward trace: replaces the OptiX ray-generation / any-hit programs of optix_tracer/forward.cu
// (__raygen__ot 428-477, tracePath 318-424, traceRay 136-315, __anyhit__ot 481-525) and their
// host launcher TraceSurfelsCUDA (trace_surfels.cpp:162-304).
//
// One thread per ray. Per ray segment: repeat { gather the 16 nearest quad hits with a pruned
// hierarchy walk into a shared-memory k-buffer; composite them front to back } until the
// transmittance threshold, the contribution cap or the end of the ray. Bounces re-enter the same
// loop from the reflected ray.
#include "dst_trace.cuh"

namespace {

constexpr int FWD_THREADS = 128;

struct FwdParams {
    dst_fwd_args a;
    BvhView bvh;
    const float4* cache;
    unsigned int* status;
    int tiled;
};

// Per-surfel shading record: tangent-frame rows from the quaternion exactly as
// quat_to_rotmat_transpose does on an IEEE host (optix_tracer/auxiliary.h:403-429, with rsqrtf
// taken as 1/sqrt), the frame origin T = R p (forward.cu:76), opacity and scales.
__global__ void __launch_bounds__(256) k_prepare_cache(int P, const float* __restrict__ means, const float* __restrict__ scales,
                                                       const float* __restrict__ rots, const float* __restrict__ opac,
                                                       float4* __restrict__ cache) {
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= P) return;
    const float q0 = rots[4 * (size_t)g], q1 = rots[4 * (size_t)g + 1], q2 = rots[4 * (size_t)g + 2], q3 = rots[4 * (size_t)g + 3];
    const float s = xdiv(1.0f, xsqrt(xadd(xadd(xadd(xmul(q3, q3), xmul(q0, q0)), xmul(q1, q1)), xmul(q2, q2))));
    const float w = xmul(q0, s), x = xmul(q1, s), y = xmul(q2, s), z = xmul(q3, s);
    const float r0x = xsub(1.f, xmul(2.f, xadd(xmul(y, y), xmul(z, z))));
    const float r0y = xmul(2.f, xadd(xmul(x, y), xmul(w, z)));
    const float r0z = xmul(2.f, xsub(xmul(x, z), xmul(w, y)));
    const float r1x = xmul(2.f, xsub(xmul(x, y), xmul(w, z)));
    const float r1y = xsub(1.f, xmul(2.f, xadd(xmul(x, x), xmul(z, z))));
    const float r1z = xmul(2.f, xadd(xmul(y, z), xmul(w, x)));
    const float r2x = xmul(2.f, xadd(xmul(x, z), xmul(w, y)));
    const float r2y = xmul(2.f, xsub(xmul(y, z), xmul(w, x)));
    const float r2z = xsub(1.f, xmul(2.f, xadd(xmul(x, x), xmul(y, y))));
    const float px = means[3 * (size_t)g], py = means[3 * (size_t)g + 1], pz = means[3 * (size_t)g + 2];
    const float tx = rdot3(r0x, r0y, r0z, px, py, pz), ty = rdot3(r1x, r1y, r1z, px, py, pz);
    float4* o = cache + 4 * (size_t)g;
    o[0] = make_float4(r0x, r0y, r0z, tx);
    o[1] = make_float4(r1x, r1y, r1z, ty);
    o[2] = make_float4(r2x, r2y, r2z, opac[g]);
    o[3] = make_float4(scales[2 * (size_t)g], scales[2 * (size_t)g + 1], 0.f, 0.f);
}

template <bool BRUTE, bool DIAG>
__global__ void __launch_bounds__(FWD_THREADS) k_forward(const __grid_constant__ FwdParams p) {
    __shared__ unsigned long long kbuf[DST_CHUNK * FWD_THREADS];
    const dst_trace_inputs& in = p.a.in;
    const long long ray = ray_of_thread(in.H, in.W, p.tiled != 0);
    if (ray < 0) return;
    unsigned long long* kb = kbuf + threadIdx.x;
    TraceCounters tc = { 0, 0, 0, 0, 0, 0 };

    const float rox = __ldg(in.ray_o + 3 * ray), roy = __ldg(in.ray_o + 3 * ray + 1), roz = __ldg(in.ray_o + 3 * ray + 2);
    const float rdx = __ldg(in.ray_d + 3 * ray), rdy = __ldg(in.ray_d + 3 * ray + 1), rdz = __ldg(in.ray_d + 3 * ray + 2);
    const float bg0 = __ldg(in.background), bg1 = __ldg(in.background + 1), bg2 = __ldg(in.background + 2);
    const bool use_sh = in.colors_precomp == nullptr;
    const bool has_aux = in.others_precomp != nullptr;
    const int ncoef = (in.sh_degree + 1) * (in.sh_degree + 1);
    const bool sh_aligned = ((in.sh_coeffs * 3) & 3) == 0 && ((reinterpret_cast<uintptr_t>(in.shs) & 15) == 0);

    float out_rgb0 = 0.f, out_rgb1 = 0.f, out_rgb2 = 0.f, out_dpt = 0.f, out_acc = 0.f;
    float out_nx = 0.f, out_ny = 0.f, out_nz = 0.f, out_aux0 = 0.f, out_aux1 = 0.f;
    float* mid = p.a.mid_val + (size_t)ray * in.mid_stride;
    int hit_count = 0;

    float sox = rox, soy = roy, soz = roz, sdx = rdx, sdy = rdy, sdz = rdz;    // segment origin / direction
    float s_prod = 1.0f;
    int bounce = 0;
    for (; bounce <= in.max_trace_depth; bounce++) {
        // forward.cu:353
        const float min_depth = bounce == 0 ? (in.start_from_first ? 0.2f : 0.0f) : 0.06f;
        const float T_threshold = 0.0001f;
        float C0 = 0.f, C1 = 0.f, C2 = 0.f, D = 0.f, Nx = 0.f, Ny = 0.f, Nz = 0.f, O0 = 0.f, O1 = 0.f;
        float T_prev = 1.0f, T_next = 1.0f, dpt = 0.0f, offset = 0.0f;
        int last_gidx = -1, contributor = 0;
        float tox = sox, toy = soy, toz = soz;                                 // moved origin of the current enumeration
        float sb[16];
        if (use_sh) sh_basis(in.sh_degree, sdx, sdy, sdz, sb);
        if (DIAG) tc.segs++;

        for (int chunk = 0;; chunk++) {
            if (chunk >= DST_MAX_CHUNKS) { atomicOr(p.status, DST_STATUS_CHUNK_LIMIT); break; }
            const int cnt = knearest<BRUTE, DIAG, FWD_THREADS>(p.bvh, tox, toy, toz, sdx, sdy, sdz, kb, p.status, tc);
            if (DIAG) tc.enums++;
            bool stop = false;
            for (int i = 0; i < cnt; i++) {
                const unsigned long long key = kb[i * FWD_THREADS];
                const int pidx = (int)(unsigned int)key;
                const int gidx = pidx >> 1;
                if (gidx == last_gidx) continue;                                // forward.cu:207
                if (DIAG) tc.evals++;
                SlotEval e;
                const bool ok = eval_slot(key, offset, sox, soy, soz, sdx, sdy, sdz, min_depth, p.cache, gidx, e);
                dpt = e.dpt;                                                    // :211 (kept even when the slot is skipped)
                if (!ok) continue;
                const float alpha = e.alpha, nsign = e.nsign;
                const float4 r2 = e.r2;
                T_next = xmul(T_prev, xsub(1.0f, alpha));
                if (T_next < T_threshold) { stop = true; break; }
                contributor++;
                if (contributor > DST_MAX_INTERSECTION) { stop = true; break; }
                last_gidx = gidx;
                const float w = xmul(alpha, T_prev);
                if (use_sh) {
                    float c[48];
                    load_sh_row(in.shs + 3 * (size_t)gidx * in.sh_coeffs, 3 * ncoef, sh_aligned, c);
                    C0 = xadd(C0, xmul(w, fmaxf(sh_channel(ncoef, sb, c, 0), 0.f)));
                    C1 = xadd(C1, xmul(w, fmaxf(sh_channel(ncoef, sb, c, 1), 0.f)));
                    C2 = xadd(C2, xmul(w, fmaxf(sh_channel(ncoef, sb, c, 2), 0.f)));
                } else {
                    const float* cp = in.colors_precomp + 3 * (size_t)gidx;
                    C0 = xadd(C0, xmul(w, __ldg(cp))); C1 = xadd(C1, xmul(w, __ldg(cp + 1))); C2 = xadd(C2, xmul(w, __ldg(cp + 2)));
                }
                if (has_aux) {
                    const float2 ax = __ldg(reinterpret_cast<const float2*>(in.others_precomp) + gidx);
                    O0 = xadd(O0, xmul(w, ax.x)); O1 = xadd(O1, xmul(w, ax.y));
                }
                D = xadd(D, xmul(w, dpt));
                Nx = xadd(Nx, xmul(w, nsign * r2.x)); Ny = xadd(Ny, xmul(w, nsign * r2.y)); Nz = xadd(Nz, xmul(w, nsign * r2.z));
                T_prev = T_next;
                if (p.a.training && p.a.a_weights) atomicAdd(p.a.a_weights + gidx, w);          // forward.cu:295
                if (DIAG) {
                    tc.contribs++;
                    if (p.a.hit_log && hit_count < p.a.hit_cap) p.a.hit_log[(size_t)ray * p.a.hit_cap + hit_count] = pidx;
                    hit_count++;
                }
            }
            if (stop || T_next < T_threshold || cnt < DST_CHUNK || contributor > DST_MAX_INTERSECTION) break;   // :299
            offset = (float)((double)dpt + 0.00001);                                               // :303
            tox = xadd(sox, xmul(offset, sdx)); toy = xadd(soy, xmul(offset, sdy)); toz = xadd(soz, xmul(offset, sdz));
        }
        // forward.cu:309-314
        C0 = xadd(C0, xmul(T_prev, bg0)); C1 = xadd(C1, xmul(T_prev, bg1)); C2 = xadd(C2, xmul(T_prev, bg2));
        const float A = xsub(1.0f, T_prev);
        // tracePath, forward.cu:378-412
        if (bounce == 0) { out_dpt = D; out_acc = A; out_nx = Nx; out_ny = Ny; out_nz = Nz; out_aux0 = O0; out_aux1 = O1; }
        const float f_this = (bounce == in.max_trace_depth) ? 1.0f : xsub(1.0f, O0);
        out_rgb0 = xadd(out_rgb0, xmul(xmul(C0, f_this), s_prod));
        out_rgb1 = xadd(out_rgb1, xmul(xmul(C1, f_this), s_prod));
        out_rgb2 = xadd(out_rgb2, xmul(xmul(C2, f_this), s_prod));
        s_prod = xmul(s_prod, O0);
        float4* m4 = reinterpret_cast<float4*>(mid + bounce * DST_MID_CHANNELS);
        m4[0] = make_float4(sox, soy, soz, sdx);
        m4[1] = make_float4(sdy, sdz, D, A);
        m4[2] = make_float4(Nx, Ny, Nz, O0);
        m4[3] = make_float4(O1, C0, C1, C2);
        const float nlen = xsqrt(rdot3(Nx, Ny, Nz, Nx, Ny, Nz));
        if (nlen == 0.0f || O0 <= in.specular_threshold) { bounce++; break; }                      // :416
        if (bounce == in.max_trace_depth) { bounce++; break; }
        // reflect about the accumulated normal, restart 0.06 along the new direction (:420-422);
        // exactly rounded, because the bounce ray decides which quads the next segment sees
        const float nx = xdiv(Nx, nlen), ny = xdiv(Ny, nlen), nz = xdiv(Nz, nlen);
        const float k = xmul(2.0f, rdot3(nx, ny, nz, sdx, sdy, sdz));
        const float Ex = xadd(sox, xmul(D, sdx)), Ey = xadd(soy, xmul(D, sdy)), Ez = xadd(soz, xmul(D, sdz));
        sdx = xsub(sdx, xmul(k, nx)); sdy = xsub(sdy, xmul(k, ny)); sdz = xsub(sdz, xmul(k, nz));
        sox = xadd(Ex, xmul(0.06f, sdx)); soy = xadd(Ey, xmul(0.06f, sdy)); soz = xadd(Ez, xmul(0.06f, sdz));
    }
    // bounces that were never traced read as zeros (the reference leaves them uninitialised, forward.cu:446)
    for (int k = bounce * DST_MID_CHANNELS; k < in.mid_stride; k += 4)
        *reinterpret_cast<float4*>(mid + k) = make_float4(0.f, 0.f, 0.f, 0.f);

    p.a.out_rgb[3 * ray] = out_rgb0; p.a.out_rgb[3 * ray + 1] = out_rgb1; p.a.out_rgb[3 * ray + 2] = out_rgb2;
    p.a.out_dpt[ray] = out_dpt; p.a.out_acc[ray] = out_acc;
    p.a.out_norm[3 * ray] = out_nx; p.a.out_norm[3 * ray + 1] = out_ny; p.a.out_norm[3 * ray + 2] = out_nz;
    p.a.out_dist[3 * ray] = 0.f; p.a.out_dist[3 * ray + 1] = 0.f; p.a.out_dist[3 * ray + 2] = 0.f;
    p.a.out_aux[2 * ray] = out_aux0; p.a.out_aux[2 * ray + 1] = out_aux1;
    if (DIAG) {
        if (p.a.hit_cnt) p.a.hit_cnt[ray] = hit_count;
        if (p.a.counters) {
            atomicAdd(p.a.counters + 0, tc.segs); atomicAdd(p.a.counters + 1, tc.enums); atomicAdd(p.a.counters + 2, tc.nodes);
            atomicAdd(p.a.counters + 3, tc.quads); atomicAdd(p.a.counters + 4, tc.evals); atomicAdd(p.a.counters + 5, tc.contribs);
        }
    }
}

// one enumeration per ray, for tests of the hierarchy walk against exhaustive testing
template <bool BRUTE>
__global__ void __launch_bounds__(FWD_THREADS) k_knearest(BvhView bvh, const float* __restrict__ ro, const float* __restrict__ rd,
                                                          long long n, unsigned long long* keys, int* counts, unsigned int* status,
                                                          const float* __restrict__ t_cut, unsigned long long* counters) {
    __shared__ unsigned long long kbuf[DST_CHUNK * FWD_THREADS];
    const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n) return;
    unsigned long long* kb = kbuf + threadIdx.x;
    TraceCounters tc = { 0, 0, 0, 0, 0, 0 };
    const int c = knearest<BRUTE, true, FWD_THREADS>(bvh, ro[3 * r], ro[3 * r + 1], ro[3 * r + 2], rd[3 * r], rd[3 * r + 1], rd[3 * r + 2],
                                                    kb, status, tc, t_cut ? t_cut[r] : DST_T_MAX);
    if (counters) { atomicAdd(counters + 2, tc.nodes); atomicAdd(counters + 3, tc.quads); }
    counts[r] = c;
    for (int i = 0; i < DST_CHUNK; i++) keys[r * DST_CHUNK + i] = i < c ? kb[i * FWD_THREADS] : 0ull;
}

}  // namespace

BvhView dst_bvh_view(const dst_handle* h) {
    BvhView b;
    b.nodes = reinterpret_cast<const float4*>(h->nodes);
    b.quads = h->quads; b.leaf_gid = h->leaf_gid; b.header = h->header; b.P = (int)h->P;
    return b;
}

int dst_check_inputs(dst_handle* h, const dst_trace_inputs* in) {
    if (!h->built) return dst_set_error(h, DST_E_STATE, "trace requested before build_acceleration_structure");
    if (in->P != h->P) return dst_set_error(h, DST_E_ARG, "means3D has %d surfels but the hierarchy was built over %lld", in->P, (long long)h->P);
    if (in->H <= 0 || in->W <= 0) return dst_set_error(h, DST_E_ARG, "ray grid must be non-empty, got %d x %d", in->H, in->W);
    if ((long long)in->H * in->W > 0x7fffffffll) return dst_set_error(h, DST_E_ARG, "too many rays");
    if (!in->ray_o || !in->ray_d || !in->means3D || !in->opacities || !in->scales || !in->rotations || !in->background || !in->vertices)
        return dst_set_error(h, DST_E_ARG, "a required input pointer is null");
    if ((in->shs == nullptr) == (in->colors_precomp == nullptr))
        return dst_set_error(h, DST_E_ARG, "exactly one of shs / colors_precomp must be given");
    if (in->shs && (in->sh_degree < 0 || in->sh_degree > 3 || (in->sh_degree + 1) * (in->sh_degree + 1) > in->sh_coeffs))
        return dst_set_error(h, DST_E_ARG, "sh_degree %d needs at most 16 and at least (degree+1)^2 coefficients, got %d", in->sh_degree, in->sh_coeffs);
    if (in->max_trace_depth < 0 || in->max_trace_depth > 15) return dst_set_error(h, DST_E_ARG, "max_trace_depth must be in [0, 15]");
    if (in->mid_stride < DST_MID_CHANNELS * (in->max_trace_depth + 1) || (in->mid_stride & 3))
        return dst_set_error(h, DST_E_ARG, "mid_stride must be a multiple of 4 and at least 16 * (max_trace_depth + 1)");
    return DST_OK;
}

int dst_prepare_cache(dst_handle* h, const dst_trace_inputs* in, cudaStream_t st) {
    if (in->P > h->cache_cap) {
        cudaFree(h->cache); h->cache = nullptr; h->cache_cap = 0;
        const int64_t cap = in->P + in->P / 8 + 1024;
        if (cudaMalloc(&h->cache, 64 * cap) != cudaSuccess) { cudaGetLastError(); return dst_set_error(h, DST_E_NOMEM, "surfel cache allocation failed"); }
        h->cache_cap = cap;
    }
    k_prepare_cache<<<(in->P + 255) / 256, 256, 0, st>>>(in->P, in->means3D, in->scales, in->rotations, in->opacities, h->cache);
    DST_CUDA_TRY(h, cudaGetLastError());
    return DST_OK;
}

int dst_forward_impl(dst_handle* h, const dst_fwd_args* a, cudaStream_t st) {
    int rc = dst_check_inputs(h, &a->in);
    if (rc != DST_OK) return rc;
    if (!a->out_rgb || !a->out_dpt || !a->out_acc || !a->out_norm || !a->out_dist || !a->out_aux || !a->mid_val)
        return dst_set_error(h, DST_E_ARG, "a forward output pointer is null");
    if ((reinterpret_cast<uintptr_t>(a->mid_val) & 15) != 0) return dst_set_error(h, DST_E_ARG, "mid_val must be 16-byte aligned");
    rc = dst_prepare_cache(h, &a->in, st);
    if (rc != DST_OK) return rc;
    if (a->training && a->a_weights) DST_CUDA_TRY(h, cudaMemsetAsync(a->a_weights, 0, 4 * (size_t)a->in.P, st));
    FwdParams p;
    p.a = *a; p.bvh = dst_bvh_view(h); p.cache = h->cache; p.status = h->status;
    p.tiled = a->in.H >= 16;
    const long long R = (long long)a->in.H * a->in.W;
    long long blocks = p.tiled ? (long long)((a->in.W + 15) / 16) * ((a->in.H + 7) / 8) : (R + FWD_THREADS - 1) / FWD_THREADS;
    const bool diag = a->hit_log || a->hit_cnt || a->counters;
    dst_prof_mark(h, 1, 0, st);
    if (diag) k_forward<false, true><<<(unsigned int)blocks, FWD_THREADS, 0, st>>>(p);
    else k_forward<false, false><<<(unsigned int)blocks, FWD_THREADS, 0, st>>>(p);
    dst_prof_mark(h, 1, 1, st);
    DST_CUDA_TRY(h, cudaGetLastError());
    return DST_OK;
}

int dst_knearest_impl(dst_handle* h, const float* ro, const float* rd, int64_t n, unsigned long long* keys, int32_t* counts,
                      int brute, const float* t_cut, unsigned long long* counters, cudaStream_t st) {
    if (!h->built) return dst_set_error(h, DST_E_STATE, "no hierarchy has been built");
    if (n <= 0) return DST_OK;
    const unsigned int blocks = (unsigned int)((n + FWD_THREADS - 1) / FWD_THREADS);
    if (brute) k_knearest<true><<<blocks, FWD_THREADS, 0, st>>>(dst_bvh_view(h), ro, rd, n, keys, counts, h->status, t_cut, counters);
    else k_knearest<false><<<blocks, FWD_THREADS, 0, st>>>(dst_bvh_view(h), ro, rd, n, keys, counts, h->status, t_cut, counters);
    DST_CUDA_TRY(h, cudaGetLastError());
    return DST_OK;
}
