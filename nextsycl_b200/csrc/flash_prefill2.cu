// flash_prefill2.cu: the 128-wide causal prefill with TWO row blocks per CTA (256 query rows of one head).
//
// Same arithmetic and operand layouts as flash_prefill.cu (the reference's attn_flash, kernels/llm/qwen35/silo/attn.cpp:
// 105-313, on tcgen05 / tensor memory / TMA). What changes is the schedule. With one row block per CTA the softmax of
// tile j (128 threads, 128 exp2 each) and the two products of tile j form one serial chain and the tensor pipe waits for
// the softmax. Here row blocks A and B each have their own chain - S_X(j) -> softmax_X(j) -> P_X(j) V(j) -> S_X(j+1) -
// their own softmax warpgroup, and their own S/P and O columns in tensor memory (4 x 128 = all 512 columns), and the two
// chains interleave on the tensor pipe: while warpgroup A exponentiates, the pipe runs B's products, and the K and V
// tiles in shared memory serve both blocks. The MMA warp issues whichever product has its inputs ready.
//
// The softmax reads its S row twice from tensor memory (once for the maximum, once to exponentiate) instead of holding
// 128 scores in registers: 320 threads leave 204 registers a thread.
#include "kernels.cuh"
#include "tc05.cuh"

#include <cuda.h>

namespace {
using namespace tc05;

constexpr int D = 128;             // head width (keys and values)
constexpr int BM = 128;            // rows a block; two blocks a CTA
constexpr int BN = 128;            // keys a tile
constexpr int NSTAGE = 2;
constexpr int THREADS = 320;       // 2 softmax warpgroups, 1 TMA warp, 1 MMA warp
constexpr float RESCALE_LOG2 = 8.0f;

constexpr int Q_BYTES = BM * D * 2;          // one block's queries: 32 KB
constexpr int K_BYTES = BN * D * 2;          // 32 KB
constexpr int V_BYTES = BN * D * 2;
constexpr int STAGE = K_BYTES + V_BYTES;
constexpr int SMEM_TOTAL = 1024 + 2 * Q_BYTES + NSTAGE * STAGE + 1024;

struct Params {
    void* out;
    int* status;
    int T, Hq, G;
    int out_kind;          // 0 fp32, 1 the operands' 16-bit type
    int64_t p0;
    float scale_log2;
};

template <int BF16>
__global__ void __launch_bounds__(THREADS, 1)
flash_prefill2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    uint8_t* q_s = smem;                          // [2 blocks][2 chunks][128 rows][128 B]
    uint8_t* kv_s = smem + 2 * Q_BYTES;
    uint64_t* bars = (uint64_t*) (kv_s + NSTAGE * STAGE);
    uint64_t* q_full = bars;                      // [1] both blocks' queries
    uint64_t* k_full = q_full + 1;                // [NSTAGE]
    uint64_t* v_full = k_full + NSTAGE;
    uint64_t* k_empty = v_full + NSTAGE;
    uint64_t* v_empty = k_empty + NSTAGE;
    uint64_t* s_full = v_empty + NSTAGE;          // [2] per block
    uint64_t* p_full = s_full + 2;                // [2] per block, 128 arrivals
    uint64_t* pv_done = p_full + 2;               // [2] per block
    uint64_t* o_final = pv_done + 2;              // [2] per block
    uint32_t* tmem_slot = (uint32_t*) (o_final + 2);
    volatile int* abort_flag = (volatile int*) (tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int mblk = (int) gridDim.x - 1 - (int) blockIdx.x;    // heaviest first
    const int h = blockIdx.y, hk = h / p.G;
    const int r0 = mblk * 2 * BM;
    const int64_t last_pos = p.p0 + min((int64_t) r0 + 2 * BM, (int64_t) p.T) - 1;
    const int ntiles = (int) (last_pos / BN) + 1;   // both blocks walk the same tiles; what a block's rows do not see is masked

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(smem_u32(q_full), 1);
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(smem_u32(k_full + s), 1);
            mbar_init(smem_u32(v_full + s), 1);
            mbar_init(smem_u32(k_empty + s), 1);
            mbar_init(smem_u32(v_empty + s), 1);
        }
        for (int x = 0; x < 2; ++x) {
            mbar_init(smem_u32(s_full + x), 1);
            mbar_init(smem_u32(p_full + x), 128);
            mbar_init(smem_u32(pv_done + x), 1);
            mbar_init(smem_u32(o_final + x), 1);
        }
        mbar_fence_init();
    }
    if (warp == 9) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    // tensor-memory columns: S/P of block x at 128 x, O of block x at 256 + 128 x

    if (warp == 8) {
        // ================= TMA producer =================
        if (elect_one()) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
            mbar_expect_tx(smem_u32(q_full), 2 * Q_BYTES);
            for (int x = 0; x < 2; ++x)
                for (int c = 0; c < D / 64; ++c)
                    tma_load_3d(smem_u32(q_s + x * Q_BYTES + c * (BM * 128)), &tm_q, c * 64, h, r0 + x * BM, smem_u32(q_full));
            bool ok = true;
            for (int j = 0; j < ntiles && ok; ++j) {
                const int s = j % NSTAGE;
                const uint32_t ph = (uint32_t) (j / NSTAGE) & 1;
                uint8_t* ks = kv_s + s * STAGE;
                uint8_t* vs = ks + K_BYTES;
                if (j >= NSTAGE) ok = mbar_wait(smem_u32(k_empty + s), ph ^ 1, abort_flag, p.status, 111);
                if (!ok) break;
                mbar_expect_tx(smem_u32(k_full + s), K_BYTES);
                for (int c = 0; c < D / 64; ++c) tma_load_3d(smem_u32(ks + c * (BN * 128)), &tm_k, c * 64, j * BN, hk, smem_u32(k_full + s));
                if (j >= NSTAGE) ok = mbar_wait(smem_u32(v_empty + s), ph ^ 1, abort_flag, p.status, 112);
                if (!ok) break;
                mbar_expect_tx(smem_u32(v_full + s), V_BYTES);
                for (int c = 0; c < D / 64; ++c) tma_load_3d(smem_u32(vs + c * (BN * 128)), &tm_v, c * 64, j * BN, hk, smem_u32(v_full + s));
            }
        }
    } else if (warp == 9) {
        // ================= MMA issuer =================
        if (elect_one()) {
            constexpr uint32_t idesc_qk = idesc_f16(BM, BN, BF16, 0, 0);
            constexpr uint32_t idesc_pv = idesc_f16(BM, D, BF16, 0, 1);
            bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, p.status, 211);
            int qk[2] = {0, 0}, pv[2] = {0, 0};   // next tile of each product, per block
            int k_seen = 0, v_seen = 0;           // K and V tiles known to have landed
            uint32_t idle = 0;
            while (ok && (pv[0] < ntiles || pv[1] < ntiles)) {
                bool did = false;
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    // P_x(j) V(j): P published by the softmax, V landed
                    int j = pv[x];
                    if (j < qk[x]) {
                        if (j == v_seen && mbar_try(smem_u32(v_full + j % NSTAGE), (uint32_t) (j / NSTAGE) & 1)) ++v_seen;
                        if (j < v_seen && mbar_try(smem_u32(p_full + x), (uint32_t) j & 1)) {
                            fence_after_sync();
                            const uint32_t vb = smem_u32(kv_s + (j % NSTAGE) * STAGE + K_BYTES);
                            const uint32_t pa = tmem + (uint32_t) (x * 128);
                            const uint32_t od = tmem + (uint32_t) (256 + x * 128);
#pragma unroll
                            for (int k = 0; k < BN / 16; ++k) {
                                const uint64_t bd = smem_desc_sw128(vb + k * (16 * 128), BN * 128, 1024);
                                mma_ts(od, pa + (uint32_t) (k * 8), bd, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
                            }
                            ++pv[x];
                            mma_commit(smem_u32(pv_done + x));
                            if (pv[0] > j && pv[1] > j) mma_commit(smem_u32(v_empty + j % NSTAGE));   // both blocks are through with V(j)
                            if (j == ntiles - 1) mma_commit(smem_u32(o_final + x));
                            did = true;
                        }
                    }
                    // S_x(j): K landed, and the block's S/P columns free - P_x(j-1) V(j-1) already issued (the pipe runs in order)
                    j = qk[x];
                    if (j < ntiles && pv[x] == j) {
                        if (j == k_seen && mbar_try(smem_u32(k_full + j % NSTAGE), (uint32_t) (j / NSTAGE) & 1)) ++k_seen;
                        if (j < k_seen) {
                            fence_after_sync();
                            const uint32_t kb = smem_u32(kv_s + (j % NSTAGE) * STAGE), qb = smem_u32(q_s + x * Q_BYTES);
                            const uint32_t d = tmem + (uint32_t) (x * 128);
#pragma unroll
                            for (int k = 0; k < D / 16; ++k) {
                                const uint64_t ad = smem_desc_sw128(qb + (k / 4) * (BM * 128) + (k % 4) * 32, 16, 1024);
                                const uint64_t bd = smem_desc_sw128(kb + (k / 4) * (BN * 128) + (k % 4) * 32, 16, 1024);
                                mma_ss(d, ad, bd, idesc_qk, k > 0);
                            }
                            ++qk[x];
                            mma_commit(smem_u32(s_full + x));
                            if (qk[0] > j && qk[1] > j) mma_commit(smem_u32(k_empty + j % NSTAGE));   // both blocks are through with K(j)
                            did = true;
                        }
                    }
                }
                if (did) {
                    idle = 0;
                    continue;
                }
                __nanosleep(40);   // an idle poll must not take issue slots from the softmax warps on this scheduler
                if (*abort_flag || ++idle > WAIT_LIMIT) {
                    if (!*abort_flag) {
                        *abort_flag = 1;
                        if (p.status) {
                            *(volatile int*) p.status = 212;
                            __threadfence_system();
                        }
                    }
                    ok = false;
                }
            }
        }
    } else {
        // ================= softmax: warpgroup x owns block x; its thread r owns row r0 + 128 x + r =================
        const int x = warp >> 2;
        const int r = tid & 127;
        const uint32_t lane_base = (uint32_t) ((warp & 3) * 32) << 16;
        const int row_g = r0 + x * BM + r;
        const int64_t row_pos = p.p0 + row_g;
        const bool row_live = row_g < p.T;
        const uint32_t s_addr = tmem + lane_base + (uint32_t) (x * 128);
        const uint32_t o_addr = tmem + lane_base + (uint32_t) (256 + x * 128);
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < ntiles; ++j) {
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(s_full + x), (uint32_t) j & 1, abort_flag, p.status, 311));
            if (!ok) break;
            fence_after_sync();
            const int64_t k0 = (int64_t) j * BN;
            const bool edge = k0 + BN - 1 > row_pos;   // some of this tile's keys lie past the row's position
            // ---- pass 1: the row maximum
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(s_addr + c * 32, v);
                tmem_wait_ld();
                if (edge) {
#pragma unroll
                    for (int e = 0; e < 32; ++e)
                        if (k0 + c * 32 + e <= row_pos) mx = fmaxf(mx, __uint_as_float(v[e]));
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(v[e]));
                }
            }
            mx *= p.scale_log2;
            float corr = 1.0f;
            bool need = false;
            if (m_ref == -INFINITY) {
                m_ref = mx;   // nothing seen before (first tile; or all of it masked, and then mx is -inf as well)
            } else if (mx > m_ref + RESCALE_LOG2) {
                corr = ex2(m_ref - mx);
                m_ref = mx;
                need = true;
            }
            if (__any_sync(0xffffffffu, need)) {
                ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(pv_done + x), (uint32_t) (j - 1) & 1, abort_flag, p.status, 312));
                if (!ok) break;
                fence_after_sync();
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld32(o_addr + c * 32, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * corr);
                    tmem_st32(o_addr + c * 32, v);
                }
                tmem_wait_st();
                l *= corr;
            }
            // ---- pass 2: P = exp2(S * scale - m_ref), written over the first 64 columns of the S it came from
            const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(s_addr + c * 32, v);
                tmem_wait_ld();
                uint32_t w[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    float a = ex2(fmaf(__uint_as_float(v[2 * e]), p.scale_log2, neg_m));
                    float b = ex2(fmaf(__uint_as_float(v[2 * e + 1]), p.scale_log2, neg_m));
                    if (edge) {
                        if (k0 + c * 32 + 2 * e > row_pos) a = 0.f;
                        if (k0 + c * 32 + 2 * e + 1 > row_pos) b = 0.f;
                    }
                    sum += a + b;
                    if (BF16) {
                        __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
                        w[e] = *reinterpret_cast<uint32_t*>(&t);
                    } else {
                        __half2 t = __floats2half2_rn(a, b);
                        w[e] = *reinterpret_cast<uint32_t*>(&t);
                    }
                }
                tmem_st16(s_addr + c * 16, w);   // columns 16c .. 16c+15: behind every S column still to be read
            }
            l += sum;
            tmem_wait_st();
            fence_before_sync();
            mbar_arrive(smem_u32(p_full + x));
        }
        // ---- epilogue: O / l
        if (ok) ok = mbar_wait(smem_u32(o_final + x), 0, abort_flag, p.status, 313);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            fence_after_sync();
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            const int64_t row = (int64_t) row_g * p.Hq + h;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(o_addr + c * 32, v);
                tmem_wait_ld();
                if (row_live) {
                    if (p.out_kind == 0) {
                        float4* dst = reinterpret_cast<float4*>((float*) p.out + row * D + c * 32);
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            dst[e] = make_float4(__uint_as_float(v[4 * e]) * inv, __uint_as_float(v[4 * e + 1]) * inv, __uint_as_float(v[4 * e + 2]) * inv,
                                                 __uint_as_float(v[4 * e + 3]) * inv);
                    } else {
                        uint32_t w[16];
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            const float a = __uint_as_float(v[2 * e]) * inv, b = __uint_as_float(v[2 * e + 1]) * inv;
                            if (BF16) {
                                __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
                                w[e] = *reinterpret_cast<uint32_t*>(&t);
                            } else {
                                __half2 t = __floats2half2_rn(a, b);
                                w[e] = *reinterpret_cast<uint32_t*>(&t);
                            }
                        }
                        uint4* dst = reinterpret_cast<uint4*>((uint16_t*) p.out + row * D + c * 32);
#pragma unroll
                        for (int e = 0; e < 4; ++e) dst[e] = make_uint4(w[4 * e], w[4 * e + 1], w[4 * e + 2], w[4 * e + 3]);
                    }
                }
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 9) {
        fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_map(CUtensorMap* m, const void* base, int bf16, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2, uint32_t box1, uint32_t box2,
             const char* where) {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled) ptr;
    }
    if (!fn) return ns_fail(std::string(where) + ": cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {s1, s2};
    cuuint32_t box[3] = {64, box1, box2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ns_fail(std::string(where) + ": tensor map rejected (code " + std::to_string((int) r) + ")");
    return 0;
}

template <int BF16>
int launch(ns_gpu* g, const FlashPrefillArgs& a, const char* where) {
    static_assert(SMEM_TOTAL <= 232448, "shared memory of one CTA");
    CUtensorMap tq, tk, tv;
    if (make_map(&tq, a.q, BF16, D, (uint64_t) a.Hq, (uint64_t) a.T, (uint64_t) D * 2, (uint64_t) a.q_row * 2, 1, BM, where)) return -1;
    if (make_map(&tk, a.k, BF16, D, (uint64_t) a.kv_len, (uint64_t) a.Hkv, (uint64_t) a.k_key * 2, (uint64_t) a.k_head * 2, BN, 1, where)) return -1;
    if (make_map(&tv, a.v, BF16, D, (uint64_t) a.kv_len, (uint64_t) a.Hkv, (uint64_t) a.v_key * 2, (uint64_t) a.v_head * 2, BN, 1, where)) return -1;
    Params p;
    p.out = a.out;
    p.status = a.status;
    p.T = (int) a.T;
    p.Hq = (int) a.Hq;
    p.G = (int) (a.Hq / a.Hkv);
    p.out_kind = a.out_f32 ? 0 : 1;
    p.p0 = a.p0;
    p.scale_log2 = a.scale_log2;
    auto kern = flash_prefill2_kernel<BF16>;
    static bool set[64] = {};
    if (!set[g->dev & 63]) {
        NS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL), where);
        set[g->dev & 63] = true;
    }
    dim3 grid((unsigned) ((a.T + 2 * BM - 1) / (2 * BM)), (unsigned) a.Hq, 1);
    kern<<<grid, THREADS, SMEM_TOTAL, g->compute>>>(tq, tk, tv, p);
    return ns_launched(where);
}

}  // namespace

int ns_launch_flash_prefill2(ns_gpu* g, const FlashPrefillArgs& a, const char* where) {
    return a.bf16 ? launch<1>(g, a, where) : launch<0>(g, a, where);
}
