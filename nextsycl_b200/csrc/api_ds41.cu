// api_ds41.cu: the deepseek41 engine's attention symbols (kernels/llm/deepseek41/silo/ds41.h:28-36) on CUDA.
//
// MQA with heads of 512 where a key is also its value: a row at position p reads its last `window` raw keys from a ring
// (slot pos % R) and the compressed cells it sees - the first (p+1)/ratio of them, or the K its indexer picked when it
// sees more than K - with a per-head sink that joins the softmax denominator only (silo/attn.cpp:83-94,246-256,266-285).
// Here a row's cells are gathered to a dense fp16 matrix (blocks of rows at a time, so the staging stays bounded) and the
// tensor-core latent-attention kernel of mla_decode.cu runs on it with the sink folded into its normalisation.
#include "kernels.cuh"

#include <algorithm>

namespace {

constexpr int D512 = 512;
constexpr float LOG2E = 1.4426950408889634f;

// the cells of row t (silo/attn.cpp:83-94): n_raw = min(window, p+1) ring slots, then compressed cells
__device__ __forceinline__ void row_cells(int64_t p, int64_t window, bool has_comp, int64_t ratio, bool has_sel, int64_t K, int64_t& n_raw,
                                          int64_t& n_comp, bool& pick) {
    n_raw = min(window, p + 1);
    const int64_t vis = has_comp ? (p + 1) / ratio : 0;
    pick = has_sel && vis > K;
    n_comp = pick ? K : vis;
}

// rows [t0, t0+rows) gathered to stage [rows][NC][512] (zeros past a row's count), counts[r] = its cells. A warp a cell.
__global__ void __launch_bounds__(256) ds41_gather_kernel(const __half* __restrict__ raw, int64_t R, const __half* __restrict__ comp, int64_t ratio,
                                                          const int32_t* __restrict__ sel, int64_t K, int64_t pos0, int64_t t0, int64_t window,
                                                          int64_t NC, __half* __restrict__ stage, int* __restrict__ counts) {
    const int64_t r = blockIdx.y, t = t0 + r, p = pos0 + t;
    int64_t n_raw, n_comp;
    bool pick;
    row_cells(p, window, comp != nullptr, ratio, sel != nullptr, K, n_raw, n_comp, pick);
    const int64_t n = min(n_raw + n_comp, NC);
    if (blockIdx.x == 0 && threadIdx.x == 0) counts[r] = (int) n;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t i = (int64_t) blockIdx.x * 8 + warp;
    if (i >= NC) return;
    uint4* dst = reinterpret_cast<uint4*>(stage + (r * NC + i) * D512);
    if (i >= n) {
        dst[lane] = make_uint4(0, 0, 0, 0);
        dst[lane + 32] = make_uint4(0, 0, 0, 0);
        return;
    }
    const __half* src;
    if (i < n_raw) {
        src = raw + ((p - n_raw + 1 + i) % R) * D512;
    } else {
        const int64_t k = i - n_raw;
        int64_t c = pick ? (int64_t) sel[t * K + k] : k;
        const int64_t vis = (p + 1) / ratio;
        c = c < 0 ? 0 : (c >= vis ? vis - 1 : c);   // an index outside what the row sees cannot leave the buffer
        src = comp + c * D512;
    }
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    dst[lane] = s4[lane];
    dst[lane + 32] = s4[lane + 32];
}

// kernels/llm/deepseek41/silo/ds41.cpp:116-133
__global__ void ds41_ring_put_kernel(const float* __restrict__ kv, __half* __restrict__ ring, int64_t T, int64_t pos0, int64_t R, int64_t D) {
    const int64_t n = T * D;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t t = i / D, c = i % D;
        ring[((pos0 + t) % R) * D + c] = __float2half_rn(kv[i]);
    }
}
__global__ void ds41_rows_f16_kernel(const float* __restrict__ x, __half* __restrict__ cache, int64_t n, int64_t j0, int64_t D) {
    const int64_t m = n * D;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < m; i += (int64_t) gridDim.x * blockDim.x) cache[j0 * D + i] = __float2half_rn(x[i]);
}

int attend(ns_gpu* g, const char* name, const float* q, const uint16_t* raw, int64_t R, const uint16_t* comp, int64_t ratio, const int32_t* sel,
           int64_t K, const float* sinks, float* out, int64_t T, int64_t H, int64_t pos0, int64_t window, float scale) {
    if (ns_enter(g, name)) return -1;
    if (T <= 0) return 0;
    if (!q || !raw || !sinks || !out) return ns_fail(std::string(name) + ": a null buffer");
    if (H < 1 || H > 1024 || R < 1 || window < 1 || window > R) return ns_fail(std::string(name) + ": 1..1024 heads, a window within the ring");
    if (comp && ratio < 1) return ns_fail(std::string(name) + ": a compression ratio of at least 1");
    if (sel && K < 1) return ns_fail(std::string(name) + ": a selection without its width");
    if (pos0 < 0 || pos0 + T >= ((int64_t) 1 << 31)) return ns_fail(std::string(name) + ": positions below 2^31");
    // the most cells a row of this pass reads
    const int64_t last = pos0 + T - 1;
    int64_t vis = comp ? (last + 1) / ratio : 0;
    if (sel && vis > K) vis = K;
    int64_t NC = std::min<int64_t>(window, last + 1) + vis;
    NC = (NC + 63) / 64 * 64;
    // rows in blocks whose gathered cells stay under 256 MiB
    int64_t rows_blk = std::max<int64_t>(1, std::min<int64_t>(T, ((int64_t) 256 << 20) / (NC * D512 * 2)));
    const int64_t q_bytes = (rows_blk * H * D512 * 2 + 255) / 256 * 256, st_bytes = (rows_blk * NC * D512 * 2 + 255) / 256 * 256;
    const int64_t cnt_bytes = (rows_blk * 4 + 255) / 256 * 256;
    const int64_t part = ns_mla_partial_floats(NC, rows_blk, H, g->sms);
    void* kept = nullptr;
    if (ns_kept(g, (size_t) (q_bytes + st_bytes + cnt_bytes + part * 4), &kept)) return -1;
    __half* q16 = (__half*) kept;
    __half* stage = (__half*) ((uint8_t*) kept + q_bytes);
    int* counts = (int*) ((uint8_t*) kept + q_bytes + st_bytes);
    float* pbuf = part ? (float*) ((uint8_t*) kept + q_bytes + st_bytes + cnt_bytes) : nullptr;
    for (int64_t t0 = 0; t0 < T; t0 += rows_blk) {
        const int64_t rows = std::min(rows_blk, T - t0);
        // the queries scaled by scale log2(e) and rounded to fp16 as the reference stages them (silo/attn.cpp:262)
        if (ns_launch_scale_to_f16(g, q + t0 * H * D512, H * D512, q16, H * D512, rows, H * D512, scale * LOG2E)) return -1;
        dim3 grid((unsigned) ((NC + 7) / 8), (unsigned) rows);
        ds41_gather_kernel<<<grid, 256, 0, g->compute>>>((const __half*) raw, R, (const __half*) comp, ratio, sel, K, pos0, t0, window, NC, stage, counts);
        if (ns_launched(name)) return -1;
        // the kernel multiplies scores by scale x log2(e); the queries carry both already
        MlaDecodeArgs a{q16, stage, out + t0 * H * D512, pbuf, rows, H, pos0 + t0, 1.0f / LOG2E, 0, NC, counts, NC * D512, sinks};
        if (ns_launch_mla_decode(g, a, name)) return -1;
    }
    return 0;
}

}  // namespace

extern "C" {

int ns_ds41_attend_xmx_supported(int64_t H, int64_t D) { return D == 512 && H >= 1; }

int ns_ds41_attend_xmx(ns_gpu* g, const float* q, const uint16_t* raw, int64_t R, const uint16_t* comp, int64_t ratio, const int32_t* sel, int64_t K,
                       const float* sinks, float* out, int64_t T, int64_t H, int64_t pos0, int64_t window, float scale) {
    NS_TRY
    return attend(g, "ns_ds41_attend_xmx", q, raw, R, comp, ratio, sel, K, sinks, out, T, H, pos0, window, scale);
    NS_CATCH("ns_ds41_attend_xmx")
}

int ns_ds41_attend(ns_gpu* g, const float* q, const uint16_t* raw, int64_t R, const uint16_t* comp, int64_t ratio, const int32_t* sel, int64_t K,
                   const float* sinks, float* out, int64_t T, int64_t H, int64_t pos0, int64_t window, float scale) {
    NS_TRY
    return attend(g, "ns_ds41_attend", q, raw, R, comp, ratio, sel, K, sinks, out, T, H, pos0, window, scale);
    NS_CATCH("ns_ds41_attend")
}

int ns_ds41_ring_put(ns_gpu* g, const float* kv, uint16_t* ring, int64_t T, int64_t pos0, int64_t R, int64_t D) {
    NS_TRY
    if (ns_enter(g, "ns_ds41_ring_put")) return -1;
    if (T <= 0) return 0;
    if (R < 1 || D < 1 || pos0 < 0) return ns_fail("ns_ds41_ring_put: a ring of at least one slot");
    ds41_ring_put_kernel<<<(unsigned) std::min<int64_t>(4096, (T * D + 255) / 256), 256, 0, g->compute>>>(kv, (__half*) ring, T, pos0, R, D);
    return ns_launched("ns_ds41_ring_put");
    NS_CATCH("ns_ds41_ring_put")
}

int ns_ds41_rows_f16(ns_gpu* g, const float* x, uint16_t* cache, int64_t n, int64_t j0, int64_t D) {
    NS_TRY
    if (ns_enter(g, "ns_ds41_rows_f16")) return -1;
    if (n <= 0) return 0;
    ds41_rows_f16_kernel<<<(unsigned) std::min<int64_t>(4096, (n * D + 255) / 256), 256, 0, g->compute>>>(x, (__half*) cache, n, j0, D);
    return ns_launched("ns_ds41_rows_f16");
    NS_CATCH("ns_ds41_rows_f16")
}

}  // extern "C"
