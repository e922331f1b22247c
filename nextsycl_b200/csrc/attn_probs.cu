// attn_probs.cu: ns_q35_attn_probs (kernels/llm/qwen35/q35.cpp:464-506) - the softmax weights of one query row over the
// first n keys of a cache (fp16, q8_0 or q4_0 rows; heads of 256), reduced over the heads per key (their mean or their
// largest) and added to out [n]. The reference walks the cache three times (maximum, sum, weights); here the scores are
// computed once into a kept buffer [Hq][n] and the two reductions read that.
#include "kernels.cuh"

#include <algorithm>

namespace {

constexpr int D = 256;

// 8 consecutive values of a cache row as floats: fp16 as they are; quantised float(q) * float(d) (q35.cpp:19-25)
__device__ __forceinline__ void row_values8(const uint8_t* row, int kt, int c, float (&f)[8]) {
    if (kt == 0) {
        const uint4 w = *reinterpret_cast<const uint4*>(row + 16 * c);
        const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 x = __half22float2(h[e]);
            f[2 * e] = x.x, f[2 * e + 1] = x.y;
        }
    } else if (kt == 1) {
        const uint2 w = *reinterpret_cast<const uint2*>(row + 8 * c);
        const float d = __half2float(reinterpret_cast<const __half*>(row + 256)[c >> 2]);
        const uint32_t ww[2] = {w.x, w.y};
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = __fmul_rn((float) (int8_t) ((ww[i >> 2] >> (8 * (i & 3))) & 0xff), d);
    } else {
        const int blk = c >> 2, sub = c & 3;
        const uint2 w = *reinterpret_cast<const uint2*>(row + blk * 16 + (sub & 1) * 8);
        const float d = __half2float(reinterpret_cast<const __half*>(row + 128)[blk]);
        const int sh = sub >= 2 ? 4 : 0;
        const uint32_t ww[2] = {w.x, w.y};
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = __fmul_rn((float) ((int) (((ww[i >> 2] >> (8 * (i & 3))) >> sh) & 15) - 8), d);
    }
}

// S[h][j] = (q_h . k_j) / 16: a warp a key of one key head, a lane 8 features, the key head's G query heads in turn
__global__ void __launch_bounds__(256) probs_scores_kernel(int kt, const float* __restrict__ q, const uint8_t* __restrict__ kc, int G, int64_t cap, int64_t n,
                                                           int64_t rb, float* __restrict__ S) {
    const int hk = blockIdx.y, lane = threadIdx.x & 31;
    const int64_t j = (int64_t) blockIdx.x * 8 + (threadIdx.x >> 5);
    if (j >= n) return;
    float kv[8];
    row_values8(kc + ((int64_t) hk * cap + j) * rb, kt, lane, kv);
    for (int gq = 0; gq < G; ++gq) {
        const float* qh = q + (int64_t) (hk * G + gq) * D + lane * 8;
        float acc = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc += qh[e] * kv[e];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) S[(int64_t) (hk * G + gq) * n + j] = acc * 0.0625f;
    }
}

// a head's maximum and sum of exp(S - max): a block a head
__global__ void __launch_bounds__(1024) probs_stats_kernel(const float* __restrict__ S, int64_t n, float* __restrict__ scratch) {
    __shared__ float red[32];
    const float* s = S + (int64_t) blockIdx.x * n;
    const int tid = threadIdx.x;
    float m = -INFINITY;
    for (int64_t j = tid; j < n; j += 1024) m = fmaxf(m, s[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((tid & 31) == 0) red[tid >> 5] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < 32; ++w) m = fmaxf(m, red[w]);
    __syncthreads();
    float z = 0.f;
    for (int64_t j = tid; j < n; j += 1024) z += expf(s[j] - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
    if ((tid & 31) == 0) red[tid >> 5] = z;
    __syncthreads();
    if (tid == 0) {
        float t = 0.f;
        for (int w = 0; w < 32; ++w) t += red[w];
        scratch[blockIdx.x * 2] = m;
        scratch[blockIdx.x * 2 + 1] = t;
    }
}

// per key: the heads' weights, their mean (mode 0) or largest (mode 1), added to out
__global__ void probs_reduce_kernel(const float* __restrict__ S, const float* __restrict__ scratch, int Hq, int64_t n, int mode, float* __restrict__ out) {
    const int64_t j = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    float acc = 0.f;
    for (int h = 0; h < Hq; ++h) {
        const float p = expf(S[(int64_t) h * n + j] - scratch[h * 2]) / scratch[h * 2 + 1];
        acc = mode == 1 ? fmaxf(acc, p) : acc + p / (float) Hq;
    }
    out[j] += acc;
}

}  // namespace

extern "C" int ns_q35_attn_probs(ns_gpu* g, int kt, const float* q, const void* kc, int64_t Hq, int64_t Hkv, int64_t Dh, int64_t cap, int64_t n, int mode,
                                 float* scratch, float* out) {
    NS_TRY
    const char* name = "ns_q35_attn_probs";
    if (ns_enter(g, name)) return -1;
    if (n <= 0) return 0;
    if (Hkv < 1 || Hq < 1 || n > cap || Hq % Hkv || Dh != D || kt < 0 || kt > 2)
        return ns_fail(std::string(name) + ": keys past the cache, heads that do not share, or not heads of 256");
    if (!q || !kc || !scratch || !out) return ns_fail(std::string(name) + ": a null buffer");
    if (Hq > 65535 || Hkv > 65535 || n >= ((int64_t) 1 << 31)) return ns_fail(std::string(name) + ": too many heads or keys");
    if (((uintptr_t) kc & 15) != 0 || ((uintptr_t) q & 15) != 0) return ns_fail(std::string(name) + ": rows 16-byte aligned");
    void* kept = nullptr;
    if (ns_kept(g, (size_t) (Hq * n * 4), &kept)) return -1;
    float* S = (float*) kept;
    const int64_t rb = kt == 0 ? 512 : kt == 1 ? 272 : 144;
    probs_scores_kernel<<<dim3((unsigned) ((n + 7) / 8), (unsigned) Hkv), 256, 0, g->compute>>>(kt, q, (const uint8_t*) kc, (int) (Hq / Hkv), cap, n, rb, S);
    if (ns_launched(name)) return -1;
    probs_stats_kernel<<<(unsigned) Hq, 1024, 0, g->compute>>>(S, n, scratch);
    if (ns_launched(name)) return -1;
    probs_reduce_kernel<<<(unsigned) ((n + 255) / 256), 256, 0, g->compute>>>(S, scratch, (int) Hq, n, mode, out);
    return ns_launched(name);
    NS_CATCH("ns_q35_attn_probs")
}
