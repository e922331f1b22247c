// lse_merge.cuh: the log-sum-exp merge of split partials, shared by the decode kernels' second stage.
// A partial row is (O[D] unnormalised, m in log2 units, l) - the layout of the reference's decode scratch
// (kernels/llm/qwen35/silo/attn.cpp:261-290); the merge is attn.cpp:352-368's: mx = max m_k,
// A = sum_k O_k 2^(m_k - mx), L = sum_k l_k 2^(m_k - mx).
#pragma once
#include <cuda_runtime.h>

namespace lse {

constexpr int MAX_SPLITS = 1024;

template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int w = 1; w < THREADS / 32; ++w) r = fmaxf(r, red[w]);
    __syncthreads();
    return r;
}
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) r += red[w];
    __syncthreads();
    return r;
}

// Shared memory a block needs, in floats.
template <int D, int THREADS>
__host__ __device__ constexpr int smem_floats() { return MAX_SPLITS + 32 + THREADS * 2; }

// The partials are read past L1 (ld.global.cg): a merge block may run while other split CTAs still write rows that share
// a cache line with its own, and a line an earlier block of the same SM pulled into L1 would be stale.
// One (row, head) by a block of THREADS threads: nsr (<= MAX_SPLITS) partial rows PS floats apart from pp. Every
// thread gets mx and L; threads tid < D/2 get the merged pair (A[2 tid], A[2 tid + 1]).
template <int D, int THREADS>
__device__ __forceinline__ float2 merge_row(const float* __restrict__ pp, int PS, int nsr, float& mx, float& L, float* sm) {
    constexpr int LANES = D / 2, GROUPS = THREADS / LANES;
    static_assert(THREADS % LANES == 0 && GROUPS >= 1, "a whole number of split groups");
    float* w = sm;                       // [MAX_SPLITS] the splits' weights
    float* red = sm + MAX_SPLITS;        // [32]
    float2* acc_s = reinterpret_cast<float2*>(sm + MAX_SPLITS + 32);   // [THREADS]
    const int tid = threadIdx.x;
    const int g = tid / LANES, lane = tid % LANES;
    // the first 8 splits' values are requested before the weights are known, and a thread's own split's (m, l) with them:
    // one memory latency instead of three in a row
    float2 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int k = g + u * GROUPS;
        v[u] = k < nsr ? __ldcg(reinterpret_cast<const float2*>(pp + (size_t) k * PS + 2 * lane)) : make_float2(0.f, 0.f);
    }
    float2 ml0 = make_float2(-INFINITY, 0.f);
    if (tid < nsr) ml0 = __ldcg(reinterpret_cast<const float2*>(pp + (size_t) tid * PS + D));
    float m_loc = ml0.x;
    for (int k = tid + THREADS; k < nsr; k += THREADS) m_loc = fmaxf(m_loc, __ldcg(pp + (size_t) k * PS + D));
    mx = block_max<THREADS>(m_loc, red);
    float l_loc = 0.f;
    if (tid < nsr) {
        const float e = (ml0.x == -INFINITY || mx == -INFINITY) ? 0.f : exp2f(ml0.x - mx);
        w[tid] = e;
        l_loc = ml0.y * e;
    }
    for (int k = tid + THREADS; k < nsr; k += THREADS) {
        const float mk = __ldcg(pp + (size_t) k * PS + D);
        const float e = (mk == -INFINITY || mx == -INFINITY) ? 0.f : exp2f(mk - mx);
        w[k] = e;
        l_loc += __ldcg(pp + (size_t) k * PS + D + 1) * e;
    }
    L = block_sum<THREADS>(l_loc, red);   // its barriers also publish w
    float2 a = make_float2(0.f, 0.f);
    for (int k0 = 0; k0 < nsr; k0 += 8 * GROUPS) {
        if (k0 > 0) {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int k = k0 + g + u * GROUPS;
                v[u] = k < nsr ? __ldcg(reinterpret_cast<const float2*>(pp + (size_t) k * PS + 2 * lane)) : make_float2(0.f, 0.f);
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int k = k0 + g + u * GROUPS;
            const float e = k < nsr ? w[k] : 0.f;
            a.x += v[u].x * e;
            a.y += v[u].y * e;
        }
    }
    if (GROUPS > 1) {
        acc_s[tid] = a;
        __syncthreads();
        if (g == 0) {
#pragma unroll
            for (int gg = 1; gg < GROUPS; ++gg) {
                const float2 o = acc_s[gg * LANES + lane];
                a.x += o.x;
                a.y += o.y;
            }
        }
    }
    return a;
}

}  // namespace lse
