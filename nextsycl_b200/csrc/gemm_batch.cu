// gemm_batch.cu: ns_gemm_batch_h - independent fp16 x fp16 -> fp32 products, y_b [T, N] (+)= x_b [T, K] . op(w_b)
// (kernels/llm/glm5next/glm.cpp:264-277, where it is one oneMKL gemm_batch call). The glm5next engine's prompt path is
// its user: per block of 32 rows, scores [64 heads, cells] = q~ . G^T (op = transpose) and latents [64, 512] = P . G
// (no transpose) over each row's own gathered cells (llm/glm5next/src/engine.rs:1925,1930).
//
// How: persistent CTAs, one an SM, walk the 128 x 128 output tiles of all the products. Warp 0 issues TMA loads of 64-wide K slices (x as a K-major
// tile; w as a K-major tile when it is transposed, as an MN-major tile - rows of 64 contiguous n - when it is not) into
// a 6-stage ring and never stops between tiles, warp 1 issues tcgen05.mma into one of two fp32 accumulators in tensor
// memory, warps 2-5 read the finished accumulator back (a warp the 32 lanes it may touch) and store, or add to, the rows of
// y while the next tile's MMAs fill the other. Rows past T, columns past N and K's tail are
// zeros from TMA's out-of-bounds fill, never read from memory. Every wait is bounded (status codes 6xx).
// Operands TMA cannot address (a base or stride that is not a multiple of 16 bytes) take a plain shared-memory kernel.
#include "kernels.cuh"
#include "tc05.cuh"

#include <cuda.h>

#include <algorithm>

namespace {
using namespace tc05;

constexpr int BM = 128, BN = 128, BK = 64, NSTAGE = 6;   // 192 KB of stages: one CTA an SM with a deep ring (see the launch)
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE = A_BYTES + B_BYTES;
constexpr int SMEM_TOTAL = 1024 + NSTAGE * STAGE + 256;
constexpr int THREADS = 192;

struct GemmParams {
    float* y;
    int64_t ldy, sy;
    int T, N, K, batch;
    int accumulate;
    int* status;
};

template <int TRANS_W>
__global__ void __launch_bounds__(THREADS, 1)
gemm_batch_h_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    uint64_t* bars = (uint64_t*) (smem + NSTAGE * STAGE);
    uint64_t* full = bars;                   // [NSTAGE]
    uint64_t* empty = bars + NSTAGE;         // [NSTAGE]
    uint64_t* acc_full = empty + NSTAGE;     // [2] a tile's accumulator complete
    uint64_t* acc_empty = acc_full + 2;      // [2] the epilogue has read it (4 arrivals: one a warp)
    uint32_t* tmem_slot = (uint32_t*) (acc_empty + 2);
    volatile int* abort_flag = (volatile int*) (tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nk = (p.K + BK - 1) / BK;
    // The CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...: column tiles of one product fastest (they share its rows of
    // x), then row tiles, then products. The loads never stop between tiles, and a tile's epilogue runs under the next
    // tile's MMAs (two accumulators in tensor memory).
    const int ntn = (p.N + BN - 1) / BN, ntm = (p.T + BM - 1) / BM;
    const long long ntiles = (long long) ntn * ntm * p.batch;
    auto tile_of = [&](long long t, int& n0, int& m0, int& b) {
        n0 = (int) (t % ntn) * BN;
        m0 = (int) ((t / ntn) % ntm) * BM;
        b = (int) (t / ((long long) ntn * ntm));
    };

    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(smem_u32(full + s), 1);
            mbar_init(smem_u32(empty + s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(acc_full + s), 1);
            mbar_init(smem_u32(acc_empty + s), 4);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 2 * BN);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (elect_one()) {
            tma_prefetch_desc(&tm_x);
            tma_prefetch_desc(&tm_w);
            bool ok = true;
            uint32_t it = 0;   // k-steps issued so far, over all of this CTA's tiles
            for (long long t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
                int n0, m0, b;
                tile_of(t, n0, m0, b);
                // Each tile starts its walk over K at another slice and wraps around: CTAs that run in step would otherwise all
                // ask for the same 128-byte window of every 1 KB row at the same time, and such a stride lands on a few of the
                // memory channels only. (The order of a tile's sum moves with it; it is the same every run.)
                const int rot = (int) (t % nk);
                for (int k0 = 0; k0 < nk && ok; ++k0, ++it) {
                    const int kt = k0 + rot < nk ? k0 + rot : k0 + rot - nk;
                    const int s = (int) (it % NSTAGE);
                    if (it >= NSTAGE) ok = mbar_wait(smem_u32(empty + s), ((it / NSTAGE) & 1) ^ 1, abort_flag, p.status, 601);
                    if (!ok) break;
                    uint8_t* a_s = smem + s * STAGE;
                    uint8_t* b_s = a_s + A_BYTES;
                    mbar_expect_tx(smem_u32(full + s), STAGE);
                    tma_load_3d(smem_u32(a_s), &tm_x, kt * BK, m0, b, smem_u32(full + s));
                    if (TRANS_W) {
                        tma_load_3d(smem_u32(b_s), &tm_w, kt * BK, n0, b, smem_u32(full + s));
                    } else {
                        // two chunks of 64 columns, each [64 k][64 n]
                        tma_load_3d(smem_u32(b_s), &tm_w, n0, kt * BK, b, smem_u32(full + s));
                        tma_load_3d(smem_u32(b_s + BK * 128), &tm_w, n0 + 64, kt * BK, b, smem_u32(full + s));
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc = idesc_f16(BM, BN, 0, 0, TRANS_W ? 0 : 1);
            bool ok = true;
            uint32_t it = 0, tc = 0;   // k-steps and tiles so far
            for (long long t = blockIdx.x; t < ntiles && ok; t += gridDim.x, ++tc) {
                const int ab = (int) (tc & 1);
                const uint32_t use = tc >> 1;   // how often this accumulator was used before
                if (use > 0) ok = mbar_wait(smem_u32(acc_empty + ab), (use & 1) ^ 1, abort_flag, p.status, 604);
                if (!ok) break;
                fence_after_sync();
                const uint32_t d = tmem + (uint32_t) (ab * BN);
                for (int kt = 0; kt < nk && ok; ++kt, ++it) {
                    const int s = (int) (it % NSTAGE);
                    ok = mbar_wait(smem_u32(full + s), (it / NSTAGE) & 1, abort_flag, p.status, 602);
                    if (!ok) break;
                    fence_after_sync();
                    const uint32_t ab_s = smem_u32(smem + s * STAGE), bb = ab_s + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = smem_desc_sw128(ab_s + k * 32, 16, 1024);
                        const uint64_t bd = TRANS_W ? smem_desc_sw128(bb + k * 32, 16, 1024) : smem_desc_sw128(bb + k * (16 * 128), BK * 128, 1024);
                        mma_ss(d, ad, bd, idesc, (kt > 0 || k > 0) ? 1u : 0u);
                    }
                    mma_commit(smem_u32(empty + s));
                }
                if (ok) mma_commit(smem_u32(acc_full + ab));
            }
        }
    } else {
        // ---- epilogue: warp w may read tensor-memory lanes 32 (w % 4) ..; a thread owns one row of the tile
        const int quarter = warp & 3;
        const bool vec = (p.ldy % 4 == 0) && (p.sy % 4 == 0) && (((uintptr_t) p.y & 15) == 0);
        bool ok = true;
        uint32_t tc = 0;
        for (long long t = blockIdx.x; t < ntiles && ok; t += gridDim.x, ++tc) {
            int n0, m0, b;
            tile_of(t, n0, m0, b);
            const int ab = (int) (tc & 1);
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(acc_full + ab), (tc >> 1) & 1, abort_flag, p.status, 603));
            if (!ok) break;
            fence_after_sync();
            const int row = m0 + quarter * 32 + lane;
            float* yr = p.y + (int64_t) b * p.sy + (int64_t) row * p.ldy;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t) (quarter * 32) << 16) + (uint32_t) (ab * BN + c * 32), v);
                tmem_wait_ld();
                if (row >= p.T) continue;
                const int col0 = n0 + c * 32;
                if (vec && col0 + 32 <= p.N) {
#pragma unroll
                    for (int e = 0; e < 32; e += 4) {
                        float4 o = make_float4(__uint_as_float(v[e]), __uint_as_float(v[e + 1]), __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
                        float4* dst = reinterpret_cast<float4*>(yr + col0 + e);
                        if (p.accumulate) {
                            const float4 old = *dst;
                            o.x += old.x, o.y += old.y, o.z += old.z, o.w += old.w;
                        }
                        *dst = o;
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e)
                        if (col0 + e < p.N) yr[col0 + e] = (p.accumulate ? yr[col0 + e] : 0.f) + __uint_as_float(v[e]);
                }
            }
            // the accumulator is read: the MMA warp may start the tile after next in it
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(acc_empty + ab));
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        fence_after_sync();
        tmem_dealloc(tmem, 2 * BN);
    }
}

// operands TMA cannot address: 32 x 32 output tiles through shared memory, fp32 accumulation in k order
__global__ void __launch_bounds__(256) gemm_batch_h_plain_kernel(int trans_w, int T, int N, int K, const __half* __restrict__ x, int64_t ldx, int64_t sx,
                                                                 const __half* __restrict__ w, int64_t ldw, int64_t sw, float* __restrict__ y, int64_t ldy,
                                                                 int64_t sy, int accumulate) {
    __shared__ float xs[32][33], ws[32][33];   // ws[k][n]
    const int b = blockIdx.z, n0 = blockIdx.x * 32, m0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 8 rows of threads: a thread 4 rows of the tile
    const __half* xb = x + (int64_t) b * sx;
    const __half* wb = w + (int64_t) b * sw;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < K; k0 += 32) {
        for (int r = ty; r < 32; r += 8) {
            const int m = m0 + r, k = k0 + tx;
            xs[r][tx] = (m < T && k < K) ? __half2float(xb[(int64_t) m * ldx + k]) : 0.f;
            if (trans_w) {   // w [N][K]: row r of the tile's columns, element k
                const int n = n0 + r;
                ws[tx][r] = (n < N && k < K) ? __half2float(wb[(int64_t) n * ldw + k]) : 0.f;
            } else {         // w [K][N]
                const int kk = k0 + r, n = n0 + tx;
                ws[r][tx] = (kk < K && n < N) ? __half2float(wb[(int64_t) kk * ldw + n]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < 32; ++k)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] = fmaf(xs[ty + 8 * i][k], ws[k][tx], acc[i]);
        __syncthreads();
    }
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty + 8 * i, n = n0 + tx;
        if (m < T && n < N) {
            float* dst = y + (int64_t) b * sy + (int64_t) m * ldy + n;
            *dst = (accumulate ? *dst : 0.f) + acc[i];
        }
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled) p;
    }
    return fn;
}

// fp16 rank-3 map: dims (inner, rows, batch), byte strides for rows and batch, box (64, box_rows, 1), 128-byte swizzle
int make_map(CUtensorMap* m, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2, uint32_t box_rows, const char* where) {
    EncodeTiled fn = encode_fn();
    if (!fn) return ns_fail(std::string(where) + ": cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {s1, s2};
    cuuint32_t box[3] = {64, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ns_fail(std::string(where) + ": tensor map rejected (code " + std::to_string((int) r) + ")");
    return 0;
}

bool tma_ok(const void* base, int64_t ld, int64_t stride, int64_t batch) {
    return ((uintptr_t) base & 15) == 0 && ld % 8 == 0 && (batch == 1 || stride % 8 == 0) && ld * 2 < ((int64_t) 1 << 40) && stride * 2 < ((int64_t) 1 << 40);
}

}  // namespace

extern "C" int ns_gemm_batch_h(ns_gpu* g, int64_t batch, int trans_w, int64_t T, int64_t N, int64_t K, const uint16_t* x, int64_t ldx, int64_t sx,
                               const uint16_t* w, int64_t ldw, int64_t sw, float* y, int64_t ldy, int64_t sy, int accumulate) {
    NS_TRY
    const char* name = "ns_gemm_batch_h";
    if (ns_enter(g, name)) return -1;
    if (batch <= 0 || T <= 0 || N <= 0) return 0;
    if (K < 0 || !x || !w || !y) return ns_fail(std::string(name) + ": a null buffer");
    if (ldx < K || ldw < (trans_w ? K : N) || ldy < N) return ns_fail(std::string(name) + ": a leading dimension shorter than its rows");
    if (batch > 65535 || T >= ((int64_t) 1 << 31) || N >= ((int64_t) 1 << 31) || K >= ((int64_t) 1 << 31))
        return ns_fail(std::string(name) + ": at most 65,535 products of fewer than 2^31 rows, columns and terms");
    if (K > 0 && tma_ok(x, ldx, sx, batch) && tma_ok(w, ldw, sw, batch)) {
        CUtensorMap tx, tw;
        // a batch stride of one product's own extent when there is one product (TMA wants a valid stride all the same)
        const uint64_t sxb = (uint64_t) (batch == 1 ? T * ldx : sx) * 2;
        const uint64_t swb = (uint64_t) (batch == 1 ? (trans_w ? N : K) * ldw : sw) * 2;
        if (make_map(&tx, x, (uint64_t) K, (uint64_t) T, (uint64_t) batch, (uint64_t) ldx * 2, sxb, BM, name)) return -1;
        if (trans_w) {
            if (make_map(&tw, w, (uint64_t) K, (uint64_t) N, (uint64_t) batch, (uint64_t) ldw * 2, swb, BN, name)) return -1;
        } else {
            if (make_map(&tw, w, (uint64_t) N, (uint64_t) K, (uint64_t) batch, (uint64_t) ldw * 2, swb, BK, name)) return -1;
        }
        GemmParams p;
        p.y = y, p.ldy = ldy, p.sy = sy, p.T = (int) T, p.N = (int) N, p.K = (int) K, p.batch = (int) batch, p.accumulate = accumulate ? 1 : 0, p.status = g->status_dev;
        static bool set[64][2] = {};
        if (!set[g->dev & 63][trans_w ? 1 : 0]) {
            if (trans_w) NS_CUDA(cudaFuncSetAttribute(gemm_batch_h_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL), name);
            else NS_CUDA(cudaFuncSetAttribute(gemm_batch_h_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL), name);
            set[g->dev & 63][trans_w ? 1 : 0] = true;
        }
        // Persistent CTAs, one an SM, walking the tiles through a six-stage ring. Measured at the glm5next prompt shapes (the
        // pair of products): a CTA a tile, two an SM, three stages 43.5 us; the same persistent 40.1; one an SM with six
        // stages 35.1 (seven: 35.8) - one deep pipeline an SM beats two shallow ones holding the same bytes in flight.
        const int64_t ntiles = ((N + BN - 1) / BN) * ((T + BM - 1) / BM) * batch;
        const unsigned grid = (unsigned) std::min<int64_t>(ntiles, (int64_t) g->sms);
        if (trans_w) gemm_batch_h_kernel<1><<<grid, THREADS, SMEM_TOTAL, g->compute>>>(tx, tw, p);
        else gemm_batch_h_kernel<0><<<grid, THREADS, SMEM_TOTAL, g->compute>>>(tx, tw, p);
        return ns_launched(name);
    }
    dim3 grid((unsigned) ((N + 31) / 32), (unsigned) ((T + 31) / 32), (unsigned) batch);
    if (grid.y > 65535) return ns_fail(std::string(name) + ": too many rows for one launch");
    gemm_batch_h_plain_kernel<<<grid, 256, 0, g->compute>>>(trans_w ? 1 : 0, (int) T, (int) N, (int) K, (const __half*) x, ldx, sx, (const __half*) w, ldw, sw, y,
                                                            ldy, sy, accumulate ? 1 : 0);
    return ns_launched(name);
    NS_CATCH("ns_gemm_batch_h")
}
