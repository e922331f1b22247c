// api_glm.cu: the glm5next engine's MLA attention symbols (kernels/llm/glm5next/glm.h:47,58-66,76-80) on CUDA.
//
// The reference has three vector-unit kernels for the absorbed 512-wide latent attention (dense fp32 ns_mla_attend,
// decode-width mla_dec<512> over a selection of cells in fp16 or q8, prompt-width mla_sel) and a GEMM form built from
// helper kernels plus oneMKL. Here every selection-based call - any number of rows - gathers the rows' cells to fp16
// (what the reference's prompt path does with ns_mla_cells + ns_gather_h / ns_gather_q8_h) and runs the tensor-core
// latent-attention kernel of mla_decode.cu on them; the helper kernels are exported under their own names as well.
#include "kernels.cuh"

#include <algorithm>

namespace {

constexpr int L512 = 512;
constexpr int Q8ROW = 544;   // 16 fp16 scales then 512 int8 (glm.cpp:1074-1077)

// a row's i-th cell and its cell count (glm.cpp:1094-1102; ns_mla_cells glm.cpp:1023-1039)
__device__ __forceinline__ int64_t cell_count(int64_t p, int32_t ns) {
    const int64_t tail0 = 4 * ((p + 1) / 4);
    return ns < 0 ? p + 1 : 4 * (int64_t) ns + (p + 1 - tail0);
}
__device__ __forceinline__ int64_t cell_of(int64_t i, int64_t p, int32_t ns, const int32_t* sel_row) {
    if (ns < 0) return i;
    if (i < 4 * (int64_t) ns) return 4 * (int64_t) sel_row[i / 4] + i % 4;
    return 4 * ((p + 1) / 4) + (i - 4 * (int64_t) ns);
}

// ns_mla_attend (glm.cpp:782-812): dense causal, fp32 latents, exact two-pass softmax with natural exp. A block a (t, h).
__global__ void __launch_bounds__(256) mla_attend_f32_kernel(const float* __restrict__ qa, const float* __restrict__ c, float* __restrict__ u, int64_t H,
                                                             int64_t Lw, int64_t pos0, float scale) {
    extern __shared__ float sm[];   // [Lw] the query, [32] reduction scratch
    float* qs = sm;
    float* red = sm + Lw;
    const int64_t th = blockIdx.x, t = th / H, n = pos0 + t + 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int64_t r = tid; r < Lw; r += 256) qs[r] = qa[th * Lw + r];
    __syncthreads();
    // pass 1: the maximum score (a warp a cell)
    float mx = -INFINITY;
    for (int64_t s = warp; s < n; s += 8) {
        float d = 0.f;
        for (int64_t r = lane; r < Lw; r += 32) d += qs[r] * c[s * Lw + r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        mx = fmaxf(mx, d * scale);
    }
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
    // pass 2: the weights, their sum, the weighted latents; each warp its cells, then the warps added
    float sum = 0.f;
    float acc[16];   // Lw <= 512: 16 features a lane
#pragma unroll
    for (int k = 0; k < 16; ++k) acc[k] = 0.f;
    for (int64_t s = warp; s < n; s += 8) {
        float d = 0.f;
        for (int64_t r = lane; r < Lw; r += 32) d += qs[r] * c[s * Lw + r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        const float p = expf(d * scale - mx);
        sum += p;
#pragma unroll
        for (int k = 0; k < 16; ++k)
            if (lane + 32 * k < Lw) acc[k] += p * c[s * Lw + lane + 32 * k];
    }
    __shared__ float part[8][512];
    __shared__ float sums[8];
#pragma unroll
    for (int k = 0; k < 16; ++k)
        if (lane + 32 * k < Lw) part[warp][lane + 32 * k] = acc[k];
    if (lane == 0) sums[warp] = sum;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < 8; ++w) tot += sums[w];
    for (int64_t r = tid; r < Lw; r += 256) {
        float v = 0.f;
        for (int w = 0; w < 8; ++w) v += part[w][r];
        u[th * Lw + r] = v / tot;
    }
}

// the rows' cells gathered to fp16 [T][NC][512] (zeros past a row's count) and counts[t] = min(count, NC); cells fp16
// rows (Q8 = false) or q8 rows (true). A warp a cell: 16-byte stores.
template <bool Q8>
__global__ void __launch_bounds__(256) mla_gather_kernel(const void* __restrict__ cv, const int32_t* __restrict__ sel, const int32_t* __restrict__ sel_cnt,
                                                         int64_t K, int64_t pos0, int64_t NC, __half* __restrict__ out, int* __restrict__ counts) {
    const int64_t t = blockIdx.y, p = pos0 + t;
    const int32_t ns = sel_cnt ? sel_cnt[t] : -1;
    const int64_t cnt = min(cell_count(p, ns), NC);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t i = (int64_t) blockIdx.x * 8 + warp;
    if (blockIdx.x == 0 && threadIdx.x == 0) counts[t] = (int) cnt;
    if (i >= NC) return;
    uint4* dst = reinterpret_cast<uint4*>(out + (t * NC + i) * L512);   // 64 x 16 bytes a row: 2 a lane
    if (i >= cnt) {
        dst[lane] = make_uint4(0, 0, 0, 0);
        dst[lane + 32] = make_uint4(0, 0, 0, 0);
        return;
    }
    const int64_t cell = cell_of(i, p, ns, sel ? sel + t * K : nullptr);
    if (!Q8) {
        const uint4* src = reinterpret_cast<const uint4*>((const __half*) cv + cell * L512);
        dst[lane] = src[lane];
        dst[lane + 32] = src[lane + 32];
    } else {
        const uint8_t* row = (const uint8_t*) cv + cell * Q8ROW;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int v0 = (lane + 32 * k) * 8;   // 8 values
            const float d = __half2float(reinterpret_cast<const __half*>(row)[v0 / 32]);
            const int2 q = *reinterpret_cast<const int2*>(row + 32 + v0);
            const int8_t* qb = reinterpret_cast<const int8_t*>(&q);
            __half2 h[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(d * (float) qb[2 * e], d * (float) qb[2 * e + 1]);
            dst[lane + 32 * k] = *reinterpret_cast<uint4*>(h);
        }
    }
}

__global__ void to_f16_kernel(const float* __restrict__ x, __half* __restrict__ y, int64_t n) {
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) y[i] = __float2half_rn(x[i]);
}

// glm.cpp:1023-1039
__global__ void mla_cells_kernel(const int32_t* sel, const int32_t* sel_cnt, int64_t T, int64_t K, int64_t pos0, int32_t* idx, int32_t* n, int64_t NC) {
    const int64_t t = blockIdx.y, i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= NC) return;
    const int64_t p = pos0 + t;
    const int32_t ns = sel_cnt ? sel_cnt[t] : -1;
    const int64_t cnt = cell_count(p, ns);
    idx[t * NC + i] = i < cnt ? (int32_t) cell_of(i, p, ns, sel ? sel + t * K : nullptr) : 0;
    if (i == 0) n[t] = (int32_t) min(cnt, NC);
}

// glm.cpp:1042-1060: rows of NC scores, row r's heads valid over its first n[r] cells
__global__ void __launch_bounds__(256) softmax_masked_kernel(float* S, int64_t H, int64_t NC, const int32_t* n, float scale) {
    __shared__ float red[8];
    const int64_t rh = blockIdx.x, r = rh / H;
    float* row = S + rh * NC;
    const int64_t m = n[r];
    const int tid = threadIdx.x;
    float mx = -INFINITY;
    for (int64_t i = tid; i < m; i += 256) mx = fmaxf(mx, row[i] * scale);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
    float sum = 0.f;
    for (int64_t i = tid; i < m; i += 256) sum += expf(row[i] * scale - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((tid & 31) == 0) red[tid >> 5] = sum;
    __syncthreads();
    sum = 0.f;
    for (int w = 0; w < 8; ++w) sum += red[w];
    for (int64_t i = tid; i < NC; i += 256) row[i] = i < m ? expf(row[i] * scale - mx) / sum : 0.f;
}

// glm.cpp:1282-1299: a warp a row, a lane half a block of 32 (the block's two lanes share the maximum)
__global__ void __launch_bounds__(256) to_q8row_kernel(const float* __restrict__ x, uint8_t* __restrict__ y, int64_t n) {
    const int64_t r = (int64_t) blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= n) return;
    const int lane = threadIdx.x & 31;
    const float* xr = x + r * 512 + lane * 16;
    float v[16], amax = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        v[e] = xr[e];
        amax = fmaxf(amax, fabsf(v[e]));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const __half dh = __float2half_rn(amax / 127.f);
    const float d = __half2float(dh), inv = d > 0.f ? 1.f / d : 0.f;
    uint8_t* row = y + r * Q8ROW;
    if ((lane & 1) == 0) reinterpret_cast<__half*>(row)[lane >> 1] = dh;
    int8_t q[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) q[e] = (int8_t) fminf(127.f, fmaxf(-127.f, roundf(v[e] * inv)));
    *reinterpret_cast<uint4*>(row + 32 + lane * 16) = *reinterpret_cast<uint4*>(q);
}

// rows idx[i] of src gathered: fp16 rows of C values, or q8 rows dequantised (glm.cpp:1301-1325)
template <bool Q8>
__global__ void __launch_bounds__(256) gather_rows_kernel(const void* __restrict__ src, const int32_t* __restrict__ idx, __half* __restrict__ out, int64_t n,
                                                          int64_t Cw) {
    const int64_t i = (int64_t) blockIdx.x * 8 + (threadIdx.x >> 5);
    if (i >= n) return;
    const int lane = threadIdx.x & 31;
    const int64_t row = idx[i];
    uint4* dst = reinterpret_cast<uint4*>(out + i * Cw);
    if (!Q8) {
        const uint4* s = reinterpret_cast<const uint4*>((const __half*) src + row * Cw);
        for (int64_t k = lane; k < Cw / 8; k += 32) dst[k] = s[k];
    } else {
        const uint8_t* r8 = (const uint8_t*) src + row * Q8ROW;
        for (int k = lane; k < 64; k += 32) {
            const float d = __half2float(reinterpret_cast<const __half*>(r8)[k / 4]);
            const int2 q = *reinterpret_cast<const int2*>(r8 + 32 + k * 8);
            const int8_t* qb = reinterpret_cast<const int8_t*>(&q);
            __half2 h[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(d * (float) qb[2 * e], d * (float) qb[2 * e + 1]);
            dst[k] = *reinterpret_cast<uint4*>(h);
        }
    }
}

int attend_sel(ns_gpu* g, const char* name, const float* qa, const void* c, bool q8, float* u, int64_t T, int64_t H, int64_t Lw, int64_t pos0,
               float scale, const int32_t* sel, const int32_t* sel_cnt, int64_t K) {
    if (ns_enter(g, name)) return -1;
    if (T <= 0) return 0;
    if (Lw != 512) return ns_fail(std::string(name) + ": latent width 512");
    if (T > 4096 || H < 1 || H > 1024) return ns_fail(std::string(name) + ": up to 4096 rows, 1024 heads");
    if (pos0 < 0 || pos0 + T >= ((int64_t) 1 << 31)) return ns_fail(std::string(name) + ": positions below 2^31");
    if (!qa || !c || !u) return ns_fail(std::string(name) + ": a null buffer");
    if (sel_cnt && (!sel || K < 1)) return ns_fail(std::string(name) + ": a selection without its indices");
    if (!sel_cnt && q8) return ns_fail(std::string(name) + ": dense rows over a q8 cache go through the selection form");
    const int64_t q_bytes = (T * H * Lw * 2 + 255) / 256 * 256;
    if (!sel_cnt) {
        // dense causal over the fp16 cache as it lies: no gather
        const int64_t part = ns_mla_partial_floats(pos0 + T, T, H, g->sms);
        void* kept = nullptr;
        if (ns_kept(g, (size_t) (q_bytes + part * 4), &kept)) return -1;
        to_f16_kernel<<<1024, 256, 0, g->compute>>>(qa, (__half*) kept, T * H * Lw);
        MlaDecodeArgs a{kept, c, u, part ? (float*) ((uint8_t*) kept + q_bytes) : nullptr, T, H, pos0, scale, 0, pos0 + T, nullptr, 0, nullptr};
        return ns_launch_mla_decode(g, a, name);
    }
    // a row reads its selected pools' cells and its incomplete pool, or (count < 0) every earlier token up to 2,560
    int64_t NC = 4 * K + 3;
    const int64_t dense_cap = pos0 + T < 2560 ? pos0 + T : 2560;
    if (NC < dense_cap) NC = dense_cap;
    NC = (NC + 63) / 64 * 64;
    const int64_t st_bytes = (T * NC * Lw * 2 + 255) / 256 * 256, cnt_bytes = (T * 4 + 255) / 256 * 256;
    const int64_t part = ns_mla_partial_floats(NC, T, H, g->sms);
    void* kept = nullptr;
    if (ns_kept(g, (size_t) (q_bytes + st_bytes + cnt_bytes + part * 4), &kept)) return -1;
    __half* q16 = (__half*) kept;
    __half* stage = (__half*) ((uint8_t*) kept + q_bytes);
    int* counts = (int*) ((uint8_t*) kept + q_bytes + st_bytes);
    float* pbuf = part ? (float*) ((uint8_t*) kept + q_bytes + st_bytes + cnt_bytes) : nullptr;
    to_f16_kernel<<<1024, 256, 0, g->compute>>>(qa, q16, T * H * Lw);
    dim3 grid((unsigned) ((NC + 7) / 8), (unsigned) T);
    if (q8) mla_gather_kernel<true><<<grid, 256, 0, g->compute>>>(c, sel, sel_cnt, K, pos0, NC, stage, counts);
    else mla_gather_kernel<false><<<grid, 256, 0, g->compute>>>(c, sel, sel_cnt, K, pos0, NC, stage, counts);
    if (ns_launched(name)) return -1;
    MlaDecodeArgs a{q16, stage, u, pbuf, T, H, pos0, scale, 0, NC, counts, NC * Lw, nullptr};
    return ns_launch_mla_decode(g, a, name);
}

}  // namespace

extern "C" {

int ns_mla_attend(ns_gpu* g, const float* qa, const float* c, float* u, int64_t T, int64_t H, int64_t Lw, int64_t pos0, float scale) {
    NS_TRY
    if (ns_enter(g, "ns_mla_attend")) return -1;
    if (T <= 0) return 0;
    if (Lw < 1 || Lw > 512) return ns_fail("ns_mla_attend: latent width up to 512");
    if (!qa || !c || !u) return ns_fail("ns_mla_attend: a null buffer");
    mla_attend_f32_kernel<<<(unsigned) (T * H), 256, (size_t) (Lw + 32) * 4, g->compute>>>(qa, c, u, H, Lw, pos0, scale);
    return ns_launched("ns_mla_attend");
    NS_CATCH("ns_mla_attend")
}

int ns_mla_attend_sel(ns_gpu* g, const float* qa, const uint16_t* c16, float* u, int64_t T, int64_t H, int64_t Lw, int64_t pos0, float scale,
                      const int32_t* sel, const int32_t* sel_cnt, int64_t K) {
    NS_TRY
    return attend_sel(g, "ns_mla_attend_sel", qa, c16, false, u, T, H, Lw, pos0, scale, sel, sel_cnt, K);
    NS_CATCH("ns_mla_attend_sel")
}

int ns_mla_attend_sel_q8(ns_gpu* g, const float* qa, const void* c, float* u, int64_t T, int64_t H, int64_t Lw, int64_t pos0, float scale,
                         const int32_t* sel, const int32_t* sel_cnt, int64_t K) {
    NS_TRY
    return attend_sel(g, "ns_mla_attend_sel_q8", qa, c, true, u, T, H, Lw, pos0, scale, sel, sel_cnt, K);
    NS_CATCH("ns_mla_attend_sel_q8")
}

int ns_mla_cells(ns_gpu* g, const int32_t* sel, const int32_t* sel_cnt, int64_t T, int64_t K, int64_t pos0, int32_t* idx, int32_t* n, int64_t NC) {
    NS_TRY
    if (ns_enter(g, "ns_mla_cells")) return -1;
    if (T <= 0 || NC <= 0) return 0;
    dim3 grid((unsigned) ((NC + 255) / 256), (unsigned) T);
    mla_cells_kernel<<<grid, 256, 0, g->compute>>>(sel, sel_cnt, T, K, pos0, idx, n, NC);
    return ns_launched("ns_mla_cells");
    NS_CATCH("ns_mla_cells")
}

int ns_softmax_masked(ns_gpu* g, float* S, int64_t R, int64_t H, int64_t NC, const int32_t* n, float scale) {
    NS_TRY
    if (ns_enter(g, "ns_softmax_masked")) return -1;
    if (R * H <= 0) return 0;
    softmax_masked_kernel<<<(unsigned) (R * H), 256, 0, g->compute>>>(S, H, NC, n, scale);
    return ns_launched("ns_softmax_masked");
    NS_CATCH("ns_softmax_masked")
}

int ns_to_f16(ns_gpu* g, const float* x, uint16_t* y, int64_t n) {
    NS_TRY
    if (ns_enter(g, "ns_to_f16")) return -1;
    if (n <= 0) return 0;
    to_f16_kernel<<<(unsigned) std::min<int64_t>(4096, (n + 255) / 256), 256, 0, g->compute>>>(x, (__half*) y, n);
    return ns_launched("ns_to_f16");
    NS_CATCH("ns_to_f16")
}

int ns_to_q8row(ns_gpu* g, const float* x, void* y, int64_t n, int64_t Lw) {
    NS_TRY
    if (ns_enter(g, "ns_to_q8row")) return -1;
    if (Lw != 512) return ns_fail("ns_to_q8row: latent width 512");
    if (n <= 0) return 0;
    to_q8row_kernel<<<(unsigned) ((n + 7) / 8), 256, 0, g->compute>>>(x, (uint8_t*) y, n);
    return ns_launched("ns_to_q8row");
    NS_CATCH("ns_to_q8row")
}

int ns_gather_q8_h(ns_gpu* g, const void* src, const int32_t* idx, uint16_t* out, int64_t n, int64_t Lw) {
    NS_TRY
    if (ns_enter(g, "ns_gather_q8_h")) return -1;
    if (Lw != 512) return ns_fail("ns_gather_q8_h: latent width 512");
    if (n <= 0) return 0;
    gather_rows_kernel<true><<<(unsigned) ((n + 7) / 8), 256, 0, g->compute>>>(src, idx, (__half*) out, n, Lw);
    return ns_launched("ns_gather_q8_h");
    NS_CATCH("ns_gather_q8_h")
}

int ns_gather_h(ns_gpu* g, const uint16_t* src, const int32_t* idx, uint16_t* out, int64_t n, int64_t Cw) {
    NS_TRY
    if (ns_enter(g, "ns_gather_h")) return -1;
    if (Cw % 8 != 0) return ns_fail("ns_gather_h: a row width that is a multiple of 8");
    if (n <= 0) return 0;
    gather_rows_kernel<false><<<(unsigned) ((n + 7) / 8), 256, 0, g->compute>>>(src, idx, (__half*) out, n, Cw);
    return ns_launched("ns_gather_h");
    NS_CATCH("ns_gather_h")
}

}  // extern "C"
