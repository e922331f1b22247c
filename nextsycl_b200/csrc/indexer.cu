// indexer.cu: glm5next's DSA lightning indexer around the attention (kernels/llm/glm5next/glm.cpp:876-1015): the pooled
// keys of completed pools of 4 tokens, a row's pool scores from the heads' products, and the K best pools a row in
// ascending position. The product S = iq . pooled^T between the first two is a plain GEMM (oneMKL in the reference) and
// is not part of this library.
#include "kernels.cuh"

#include <algorithm>

namespace {

// glm.cpp:883-905: a thread a (pool, feature)
__global__ void idx_pool_kernel(const float* __restrict__ ring, const float* __restrict__ ik, const float* __restrict__ ig, const float* __restrict__ ape,
                                float* __restrict__ pooled, int64_t pos0, int64_t j_lo, int64_t npool, int64_t D) {
    const int64_t total = npool * D;
    for (int64_t id = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; id < total; id += (int64_t) gridDim.x * blockDim.x) {
        const int64_t j = j_lo + id / D, c = id % D;
        float lg[4], kv[4], mx = -INFINITY;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int64_t p = 4 * j + m;
            const float* k = p >= pos0 ? ik + (p - pos0) * D : ring + (p % 8) * 2 * D;
            const float* gg = p >= pos0 ? ig + (p - pos0) * D : ring + (p % 8) * 2 * D + D;
            kv[m] = k[c];
            lg[m] = gg[c] + ape[m * D + c];
            mx = fmaxf(mx, lg[m]);
        }
        float s = 0.f, acc = 0.f;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const float e = expf(lg[m] - mx);
            s += e;
            acc += e * kv[m];
        }
        pooled[j * D + c] = acc / s;
    }
}
// glm.cpp:909-915: the ring takes the pass's last (up to 8) tokens - after the pools above have read it
__global__ void idx_ring_kernel(float* __restrict__ ring, const float* __restrict__ ik, const float* __restrict__ ig, int64_t pos0, int64_t first,
                                int64_t rows, int64_t D) {
    const int64_t total = rows * D;
    for (int64_t id = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; id < total; id += (int64_t) gridDim.x * blockDim.x) {
        const int64_t p = first + id / D, c = id % D;
        ring[(p % 8) * 2 * D + c] = ik[(p - pos0) * D + c];
        ring[(p % 8) * 2 * D + D + c] = ig[(p - pos0) * D + c];
    }
}

// glm.cpp:921-936
__global__ void idx_score_kernel(const float* __restrict__ S, const float* __restrict__ w, float* __restrict__ score, int64_t T, int64_t H, int64_t j0,
                                 int64_t n, int64_t ld, int64_t pos0) {
    const int64_t total = T * n;
    for (int64_t id = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; id < total; id += (int64_t) gridDim.x * blockDim.x) {
        const int64_t r = id / n, jj = id % n, j = j0 + jj;
        const int64_t nv = (pos0 + r + 1) / 4;
        float s = -INFINITY;
        if (j < nv) {
            s = 0.f;
            for (int64_t h = 0; h < H; ++h) s += fmaxf(S[(r * H + h) * n + jj], 0.f) * w[r * H + h];
        }
        score[r * ld + j] = s;
    }
}

// a float's order-preserving key: a larger float has a larger key
__device__ __forceinline__ uint32_t order_key(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// glm.cpp:940-1015: a block a row. A radix select over the keys, 8 bits at a time from the top, finds the K-th largest
// key; then every key above it goes and the first of its equals by position, written in ascending position: each thread
// a run of positions, its place from two block-wide exclusive scans - the same selection every run.
constexpr int TK_THREADS = 1024, TK_HIST = 32;
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* warp_sums) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    if (warp == 0) {
        uint32_t s = warp_sums[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t y = __shfl_up_sync(0xffffffffu, s, o);
            if (lane >= o) s += y;
        }
        warp_sums[lane] = s;   // inclusive sums of the warps
    }
    __syncthreads();
    const uint32_t before = warp > 0 ? warp_sums[warp - 1] : 0u;
    __syncthreads();
    return before + x - v;
}
__global__ void __launch_bounds__(TK_THREADS) topk_kernel(const float* __restrict__ score, int32_t* __restrict__ sel, int64_t n, int64_t ld, int64_t K) {
    __shared__ uint32_t hist[TK_HIST * 256];
    __shared__ uint32_t st[3];   // prefix, mask, still needed
    __shared__ uint32_t warp_sums[32];
    const int64_t r = blockIdx.x;
    const int lid = threadIdx.x;
    const float* row = score + r * ld;
    if (lid == 0) st[0] = 0, st[1] = 0, st[2] = (uint32_t) K;
    uint32_t* mine = hist + (lid % TK_HIST) * 256;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int b = lid; b < TK_HIST * 256; b += TK_THREADS) hist[b] = 0;
        __syncthreads();
        const uint32_t prefix = st[0], mask = st[1];
        for (int64_t j = lid; j < n; j += TK_THREADS) {
            const uint32_t k = order_key(row[j]);
            if ((k & mask) == prefix) atomicAdd(mine + ((k >> shift) & 255), 1u);
        }
        __syncthreads();
        if (lid < 256) {
            uint32_t c = 0;
            for (int m = 0; m < TK_HIST; ++m) c += hist[m * 256 + lid];
            hist[lid] = c;
        }
        __syncthreads();
        if (lid == 0) {
            // the digit, from the top, where the count of keys at or above it reaches what is still needed
            uint32_t need = st[2], above = 0;
            int d = 255;
            for (; d > 0; --d) {
                if (above + hist[d] >= need) break;
                above += hist[d];
            }
            st[0] = prefix | ((uint32_t) d << shift);
            st[1] = mask | (255u << shift);
            st[2] = need - above;
        }
        __syncthreads();
    }
    const uint32_t kth = st[0], ties = st[2];
    const int64_t seg = (n + TK_THREADS - 1) / TK_THREADS, j0 = min(n, (int64_t) lid * seg), j1 = min(n, j0 + seg);
    uint32_t gt = 0, eq = 0;
    for (int64_t j = j0; j < j1; ++j) {
        const uint32_t k = order_key(row[j]);
        gt += k > kth;
        eq += k == kth;
    }
    const uint32_t eq_before = block_exclusive_scan(eq, warp_sums);
    const uint32_t eq_take = eq_before >= ties ? 0u : min(eq, ties - eq_before);
    uint32_t at = block_exclusive_scan(gt + eq_take, warp_sums);
    uint32_t eq_left = eq_take;
    for (int64_t j = j0; j < j1; ++j) {
        const uint32_t k = order_key(row[j]);
        if (k > kth || (k == kth && eq_left > 0)) {
            if (k == kth) --eq_left;
            if (at < (uint32_t) K) sel[r * K + at] = (int32_t) j;
            ++at;
        }
    }
}

unsigned blocks_for(int64_t n) { return (unsigned) std::max<int64_t>(1, std::min<int64_t>(8192, (n + 255) / 256)); }

}  // namespace

extern "C" {

int ns_idx_pool(ns_gpu* g, float* ring, const float* ik, const float* ig, const float* ape, float* pooled, int64_t pos0, int64_t T, int64_t D) {
    NS_TRY
    if (ns_enter(g, "ns_idx_pool")) return -1;
    if (T <= 0) return 0;
    if (!ring || !ik || !ig || !ape || !pooled || D < 1 || pos0 < 0) return ns_fail("ns_idx_pool: a null buffer");
    const int64_t j_lo = pos0 / 4, j_hi = (pos0 + T) / 4;
    if (j_hi > j_lo) {
        idx_pool_kernel<<<blocks_for((j_hi - j_lo) * D), 256, 0, g->compute>>>(ring, ik, ig, ape, pooled, pos0, j_lo, j_hi - j_lo, D);
        if (ns_launched("ns_idx_pool")) return -1;
    }
    const int64_t first = std::max<int64_t>(pos0, pos0 + T - 8);
    idx_ring_kernel<<<blocks_for((pos0 + T - first) * D), 256, 0, g->compute>>>(ring, ik, ig, pos0, first, pos0 + T - first, D);
    return ns_launched("ns_idx_pool");
    NS_CATCH("ns_idx_pool")
}

int ns_idx_score(ns_gpu* g, const float* S, const float* w, float* score, int64_t T, int64_t H, int64_t j0, int64_t n, int64_t ld, int64_t pos0) {
    NS_TRY
    if (ns_enter(g, "ns_idx_score")) return -1;
    if (T <= 0 || n <= 0) return 0;
    if (!S || !w || !score || H < 1 || j0 < 0 || ld < j0 + n) return ns_fail("ns_idx_score: score rows at least j0 + n floats apart");
    idx_score_kernel<<<blocks_for(T * n), 256, 0, g->compute>>>(S, w, score, T, H, j0, n, ld, pos0);
    return ns_launched("ns_idx_score");
    NS_CATCH("ns_idx_score")
}

int ns_topk(ns_gpu* g, const float* score, int32_t* sel, int64_t T, int64_t n, int64_t ld, int64_t K) {
    NS_TRY
    if (ns_enter(g, "ns_topk")) return -1;
    if (T <= 0 || K <= 0 || n <= 0) return 0;
    if (!score || !sel || ld < n || n >= ((int64_t) 1 << 31) || K >= ((int64_t) 1 << 31)) return ns_fail("ns_topk: score rows at least n floats apart");
    if (T >= ((int64_t) 1 << 31)) return ns_fail("ns_topk: too many rows");
    topk_kernel<<<(unsigned) T, TK_THREADS, 0, g->compute>>>(score, sel, n, ld, K);
    return ns_launched("ns_topk");
    NS_CATCH("ns_topk")
}

}  // extern "C"
