// ds41_indexer.cu: deepseek41's indexer around its attention (kernels/llm/deepseek41/silo/k41.cpp:96-250,352-483): a key's
// score for a row is sum_h w[h] relu(q[h] . k), over every key the row sees or only over its candidate blocks of 8 keys;
// block maxima, a candidate mask and the map from compact picks back to positions are the index steps between them.
// With 32 heads of 128 (the model's indexer) the products run on the tensor cores in the numerics of the reference's XMX
// form: q rounded to fp16, fp32 sums. Other shapes take the scalar form with fp32 q.
#include "kernels.cuh"

#include <algorithm>

namespace {

constexpr int IXH = 32, IXD = 128;
constexpr int QROW = IXD + 8;   // halves a row of q in shared memory: 16 bytes of padding keep a quad's 16-byte reads off each other's banks

__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One warp: the scores of 16 keys (rows lo[0..8) then hi[0..8); a null row pointer scores 0) against the 32 heads of q_s
// (fp16 [32][QROW] in shared memory). Lane l returns in (s_lo, s_hi) the scores of rows l/4 and l/4 + 8 (the same in the 4
// lanes of a quad). The contraction index is permuted the same way for both operands so that a lane reads 16 contiguous
// bytes of a key row at a time: its 8 halves are the (k, k+1, k+8, k+9) elements of two MMA steps.
__device__ __forceinline__ void score16(const __half* lo_row, const __half* hi_row, const __half* q_s, const float* w_s, float& s_lo, float& s_hi) {
    const int lane = threadIdx.x & 31, c = lane & 3, hq = lane >> 2;
    float acc[IXH / 8][4];
#pragma unroll
    for (int nt = 0; nt < IXH / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
#pragma unroll
    for (int s2 = 0; s2 < IXD / 32; ++s2) {
        const uint4 zero = make_uint4(0, 0, 0, 0);
        const uint4 lo = lo_row ? *reinterpret_cast<const uint4*>(lo_row + s2 * 32 + c * 8) : zero;
        const uint4 hi = hi_row ? *reinterpret_cast<const uint4*>(hi_row + s2 * 32 + c * 8) : zero;
        const uint32_t a0[4] = {lo.x, hi.x, lo.y, hi.y}, a1[4] = {lo.z, hi.z, lo.w, hi.w};
#pragma unroll
        for (int nt = 0; nt < IXH / 8; ++nt) {
            const uint4 b = *reinterpret_cast<const uint4*>(q_s + (nt * 8 + hq) * QROW + s2 * 32 + c * 8);
            mma16816(acc[nt], a0, b.x, b.y);
            mma16816(acc[nt], a1, b.z, b.w);
        }
    }
    s_lo = 0.f, s_hi = 0.f;
#pragma unroll
    for (int nt = 0; nt < IXH / 8; ++nt) {
        const float w0 = w_s[nt * 8 + 2 * c], w1 = w_s[nt * 8 + 2 * c + 1];
        s_lo += fmaxf(acc[nt][0], 0.f) * w0 + fmaxf(acc[nt][1], 0.f) * w1;
        s_hi += fmaxf(acc[nt][2], 0.f) * w0 + fmaxf(acc[nt][3], 0.f) * w1;
    }
    s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 1);
    s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 2);
    s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 1);
    s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 2);
}

__device__ __forceinline__ void stage_q(const float* q, const float* w, int64_t t, __half* q_s, float* w_s) {
    for (int i = threadIdx.x; i < IXH * IXD; i += blockDim.x) q_s[(i / IXD) * QROW + i % IXD] = __float2half_rn(q[t * IXH * IXD + i]);
    if (threadIdx.x < IXH) w_s[threadIdx.x] = w[t * IXH + threadIdx.x];
    __syncthreads();
}

// k41.cpp:107-175 on mma.sync: a block a (row, 128 positions), a warp 16 positions
__global__ void __launch_bounds__(256) idx_score_tc_kernel(const float* __restrict__ q, const float* __restrict__ w, const __half* __restrict__ k,
                                                           float* __restrict__ score, int64_t n, int64_t ld, int64_t pos0, int64_t ratio) {
    __shared__ __align__(16) __half q_s[IXH * QROW];
    __shared__ float w_s[IXH];
    const int64_t t = blockIdx.y;
    stage_q(q, w, t, q_s, w_s);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t nv = min(n, (pos0 + t + 1) / ratio);
    const int64_t j0 = ((int64_t) blockIdx.x * 8 + warp) * 16;
    if (j0 >= ld) return;
    float* out = score + t * ld;
    if (j0 >= nv) {
        if (lane < 16 && j0 + lane < ld) out[j0 + lane] = -INFINITY;
        return;
    }
    const int64_t jl = j0 + (lane >> 2), jh = jl + 8;
    float s_lo, s_hi;
    score16(jl < nv ? k + jl * IXD : nullptr, jh < nv ? k + jh * IXD : nullptr, q_s, w_s, s_lo, s_hi);
    if ((lane & 3) == 0) {
        if (jl < ld) out[jl] = jl < nv ? s_lo : -INFINITY;
        if (jh < ld) out[jh] = jh < nv ? s_hi : -INFINITY;
    }
}

// k41.cpp:181-246 on mma.sync: a warp two candidate blocks of 8 keys
__global__ void __launch_bounds__(256) idx_score_cand_kernel(const float* __restrict__ q, const float* __restrict__ w, const __half* __restrict__ k,
                                                             const int32_t* __restrict__ cand, int64_t K, float* __restrict__ score, int64_t n, int64_t pos0,
                                                             int64_t ratio) {
    __shared__ __align__(16) __half q_s[IXH * QROW];
    __shared__ float w_s[IXH];
    const int64_t t = blockIdx.y;
    stage_q(q, w, t, q_s, w_s);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t nv = min(n, (pos0 + t + 1) / ratio), nb = (n + 7) / 8;
    const int64_t c0 = ((int64_t) blockIdx.x * 8 + warp) * 2;
    if (c0 >= K) return;
    const int e = lane >> 2;
    const int64_t b_lo = cand[t * K + c0], b_hi = c0 + 1 < K ? (int64_t) cand[t * K + c0 + 1] : -1;
    const int64_t jl = b_lo * 8 + e, jh = b_hi * 8 + e;
    const bool ok_lo = b_lo >= 0 && b_lo < nb && jl < nv, ok_hi = b_hi >= 0 && b_hi < nb && jh < nv;
    float s_lo, s_hi;
    score16(ok_lo ? k + jl * IXD : nullptr, ok_hi ? k + jh * IXD : nullptr, q_s, w_s, s_lo, s_hi);
    if ((lane & 3) == 0) {
        float* out = score + t * K * 8;
        out[c0 * 8 + e] = ok_lo ? s_lo : -INFINITY;
        if (c0 + 1 < K) out[(c0 + 1) * 8 + e] = ok_hi ? s_hi : -INFINITY;
    }
}

// k41.cpp:362-398, the scalar form: fp32 q, a thread a position
__global__ void idx_score_scalar_kernel(const float* __restrict__ q, const float* __restrict__ w, const __half* __restrict__ k, float* __restrict__ score,
                                        int64_t T, int64_t H, int64_t D, int64_t n, int64_t ld, int64_t pos0, int64_t ratio) {
    const int64_t total = T * ld;
    for (int64_t id = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; id < total; id += (int64_t) gridDim.x * blockDim.x) {
        const int64_t t = id / ld, j = id % ld, nv = min(n, (pos0 + t + 1) / ratio);
        float s = -INFINITY;
        if (j < nv) {
            s = 0.f;
            for (int64_t h = 0; h < H; ++h) {
                float acc = 0.f;
                for (int64_t c = 0; c < D; ++c) acc += q[(t * H + h) * D + c] * __half2float(k[j * D + c]);
                s += fmaxf(acc, 0.f) * w[t * H + h];
            }
        }
        score[id] = s;
    }
}

// k41.cpp:403-417
__global__ void block_max_kernel(const float* __restrict__ score, float* __restrict__ bmax, int64_t T, int64_t n, int64_t ld, int64_t bs, int64_t nb, int64_t pos0,
                                 int64_t ratio) {
    const int64_t total = T * nb;
    for (int64_t id = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; id < total; id += (int64_t) gridDim.x * blockDim.x) {
        const int64_t t = id / nb, b = id % nb, lens = min(n, (pos0 + t + 1) / ratio);
        float m = -INFINITY;
        for (int64_t j = b * bs; j < min(n, (b + 1) * bs); ++j) m = fmaxf(m, score[t * ld + j]);
        if (lens > 0 && b == (lens - 1) / bs) m = INFINITY;   // the block of the row's newest position: in, whatever it scores
        bmax[id] = m;
    }
}
// k41.cpp:419-436
__global__ void cand_mark_kernel(const int32_t* __restrict__ cand, uint8_t* __restrict__ mark, int64_t T, int64_t K, int64_t nb) {
    const int64_t total = T * K;
    for (int64_t id = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; id < total; id += (int64_t) gridDim.x * blockDim.x) {
        const int32_t b = cand[id];
        if (b >= 0 && b < nb) mark[(id / K) * nb + b] = 1;
    }
}
__global__ void cand_mask_kernel(float* __restrict__ score, const uint8_t* __restrict__ mark, int64_t T, int64_t n, int64_t ld, int64_t bs, int64_t nb) {
    const int64_t total = T * n;
    for (int64_t id = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; id < total; id += (int64_t) gridDim.x * blockDim.x) {
        const int64_t t = id / n, j = id % n;
        if (!mark[t * nb + j / bs]) score[t * ld + j] = -INFINITY;
    }
}
// k41.cpp:475-483
__global__ void cand_pos_kernel(const int32_t* __restrict__ selc, const int32_t* __restrict__ cand, int32_t* __restrict__ sel, int64_t T, int64_t K, int64_t kp,
                                int64_t bs) {
    const int64_t total = T * kp;
    for (int64_t id = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; id < total; id += (int64_t) gridDim.x * blockDim.x) {
        const int64_t t = id / kp;
        const int32_t c = selc[id];
        sel[id] = cand[t * K + c / bs] * (int32_t) bs + c % (int32_t) bs;
    }
}

unsigned blocks_for(int64_t n) { return (unsigned) std::max<int64_t>(1, std::min<int64_t>(8192, (n + 255) / 256)); }

}  // namespace

extern "C" {

int ns_ds41_idx_score(ns_gpu* g, const float* q, const float* w, const uint16_t* k, float* score, int64_t T, int64_t H, int64_t D, int64_t n, int64_t ld,
                      int64_t pos0, int64_t ratio) {
    NS_TRY
    const char* name = "ns_ds41_idx_score";
    if (ns_enter(g, name)) return -1;
    if (T <= 0 || ld <= 0) return 0;
    if (H < 1 || H > 32 || D < 16 || D % 16 != 0 || ratio < 1) return ns_fail(std::string(name) + ": at most 32 heads, dims a multiple of 16");
    if (!q || !w || !k || !score || n < 0 || pos0 < 0 || T > 65535) return ns_fail(std::string(name) + ": a null buffer");
    if (H == IXH && D == IXD && n >= 8 && ((uintptr_t) k & 15) == 0) {
        idx_score_tc_kernel<<<dim3((unsigned) ((ld + 127) / 128), (unsigned) T), 256, 0, g->compute>>>(q, w, (const __half*) k, score, n, ld, pos0, ratio);
    } else {
        idx_score_scalar_kernel<<<blocks_for(T * ld), 256, 0, g->compute>>>(q, w, (const __half*) k, score, T, H, D, n, ld, pos0, ratio);
    }
    return ns_launched(name);
    NS_CATCH("ns_ds41_idx_score")
}

int ns_ds41_idx_score_cand(ns_gpu* g, const float* q, const float* w, const uint16_t* k, const int32_t* cand, int64_t K, float* score, int64_t T, int64_t H,
                           int64_t D, int64_t n, int64_t pos0, int64_t ratio) {
    NS_TRY
    const char* name = "ns_ds41_idx_score_cand";
    if (ns_enter(g, name)) return -1;
    if (T <= 0 || K <= 0) return 0;
    if (H != IXH || D != IXD || n < 8 || ratio < 1) return ns_fail(std::string(name) + ": 32 heads of 128, at least 8 keys");
    if (!q || !w || !k || !cand || !score || pos0 < 0 || T > 65535 || ((uintptr_t) k & 15) != 0) return ns_fail(std::string(name) + ": a null buffer");
    idx_score_cand_kernel<<<dim3((unsigned) ((K + 15) / 16), (unsigned) T), 256, 0, g->compute>>>(q, w, (const __half*) k, cand, K, score, n, pos0, ratio);
    return ns_launched(name);
    NS_CATCH("ns_ds41_idx_score_cand")
}

int ns_ds41_block_max(ns_gpu* g, const float* score, float* bmax, int64_t T, int64_t n, int64_t ld, int64_t bs, int64_t pos0, int64_t ratio) {
    NS_TRY
    if (ns_enter(g, "ns_ds41_block_max")) return -1;
    if (T <= 0 || n <= 0) return 0;
    if (!score || !bmax || bs < 1 || ratio < 1 || ld < n) return ns_fail("ns_ds41_block_max: blocks of at least one position, rows at least n apart");
    const int64_t nb = (n + bs - 1) / bs;
    block_max_kernel<<<blocks_for(T * nb), 256, 0, g->compute>>>(score, bmax, T, n, ld, bs, nb, pos0, ratio);
    return ns_launched("ns_ds41_block_max");
    NS_CATCH("ns_ds41_block_max")
}

int ns_ds41_cand_mask(ns_gpu* g, float* score, const int32_t* cand, uint8_t* mark, int64_t T, int64_t n, int64_t ld, int64_t K, int64_t bs) {
    NS_TRY
    if (ns_enter(g, "ns_ds41_cand_mask")) return -1;
    if (T <= 0 || n <= 0) return 0;
    if (!score || !cand || !mark || bs < 1 || K < 0 || ld < n) return ns_fail("ns_ds41_cand_mask: a null buffer");
    const int64_t nb = (n + bs - 1) / bs;
    NS_CUDA(cudaMemsetAsync(mark, 0, (size_t) (T * nb), g->compute), "ns_ds41_cand_mask");
    if (K > 0) cand_mark_kernel<<<blocks_for(T * K), 256, 0, g->compute>>>(cand, mark, T, K, nb);
    cand_mask_kernel<<<blocks_for(T * n), 256, 0, g->compute>>>(score, mark, T, n, ld, bs, nb);
    return ns_launched("ns_ds41_cand_mask");
    NS_CATCH("ns_ds41_cand_mask")
}

int ns_ds41_cand_pos(ns_gpu* g, const int32_t* selc, const int32_t* cand, int32_t* sel, int64_t T, int64_t K, int64_t kp, int64_t bs) {
    NS_TRY
    if (ns_enter(g, "ns_ds41_cand_pos")) return -1;
    if (T <= 0 || kp <= 0) return 0;
    if (!selc || !cand || !sel || bs < 1 || K < 1) return ns_fail("ns_ds41_cand_pos: a null buffer");
    cand_pos_kernel<<<blocks_for(T * kp), 256, 0, g->compute>>>(selc, cand, sel, T, K, kp, bs);
    return ns_launched("ns_ds41_cand_pos");
    NS_CATCH("ns_ds41_cand_pos")
}

}  // extern "C"
