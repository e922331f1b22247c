// flash_prefill.cu: causal flash-attention prefill on the Blackwell tensor path (tcgen05.mma, accumulators in tensor
// memory, K/V tiles staged by TMA).
//
// What it computes is the reference's prompt kernel attn_flash (kernels/llm/qwen35/silo/attn.cpp:105-313; D=128 form
// kernels/llm/nemotronh/silo/attn.cpp): out[t,h,:] = softmax_{j <= p0+t}(q k_j * scale) v_j with 16-bit operands, exp2,
// weights rounded to the operand type before they meet V, fp32 sums. Also instantiated for the shape the reference has
// no kernel for: bf16 with 192-wide keys and 128-wide values (non-absorbed MLA prefill).
//
// How: a CTA takes 128 query rows of one head. Warp 0 issues the MMAs, warp 1 the TMA loads (Q once; K and V tiles of
// BN keys through a ring of stages, 128-byte swizzle), warps 4 and up are the softmax. The MMAs: S = Q K^T into one of
// two S buffers in tensor memory, then O += P V with P read from tensor memory (it overlays the S buffer it came from)
// and V as an MN-major shared-memory operand; the order on the pipe is S(0) S(1) PV(0) S(2) PV(1) S(3) ... A softmax
// thread owns row r (= tensor-memory lane r), so row max and sum need no shuffles; it reads its S row, writes P back as
// packed 16-bit pairs, and rescales its O row only when the running maximum grew by more than 2^8 (the final 1/l uses
// the same reference maximum, so the result is unchanged).
// With NG = 2 there are two softmax groups (warps 4-7 and 8-11): group g owns keys [g BN/2, (g+1) BN/2) of every tile
// with its own running maximum, sum and O accumulator in tensor memory (O_g += P_g V_g), so the groups never exchange
// anything inside the loop and two warps a scheduler share the exponentials; the epilogue adds the two accumulators
// under a common maximum. (The 256-wide instance keeps one group: two accumulators of 256 columns do not fit.)
// Every mbarrier wait is bounded; on a timeout the CTA records a status code and runs to its teardown.
// The file holds two kernels of the same arithmetic: flash_prefill_kernel, a CTA a (row block, head) item, and, for the
// 128-wide heads, flash_prefill_stream_kernel, a CTA an SM that works through several items as one stream of key tiles (taken
// for prompts of a few rounds of items; see the launch function).
#include "kernels.cuh"
#include "tc05.cuh"

#include <cuda.h>

#include <cstdlib>

namespace {
using namespace tc05;

constexpr int BM = 128;           // query rows a CTA
constexpr int SOFTMAX_THREADS = 128;   // a softmax group: thread r owns query row r
constexpr float RESCALE_LOG2 = 8.0f;

struct Params {
    void* out;             // [T][Hq*DV] fp32, fp16 or bf16
    int* status;           // a wait that gave up records its code here
    int T, Hq, G;
    int nblk, chunk;       // row blocks; heads whose CTAs are issued together, longest first
    // (streaming kernel) divisions of the item number by the items of a chunk, the heads of a full chunk, of the last chunk,
    // and a key head's query heads, as multiplications (floor(2^32 / d): the quotient comes out right or one short)
    uint32_t inv_per_chunk, inv_chunk, inv_tail, inv_G;
    int out_kind;          // 0 fp32, 1 same 16-bit type as the operands
    int64_t p0, kv_len;    // row t sees keys 0 .. p0+t; kv_len = p0 + T
    float scale_log2;      // multiplies S before exp2 (1 when the queries are pre-scaled)
};

template <int DQK, int DV, int BN, int NSTAGE>
struct Smem {
    static constexpr int Q_BYTES = BM * DQK * 2;
    static constexpr int K_BYTES = BN * DQK * 2;
    static constexpr int V_BYTES = BN * DV * 2;
    static constexpr int STAGE = K_BYTES + V_BYTES;
    static constexpr int BARS = 256;    // mbarriers, the tensor-memory base slot, the flags
    static constexpr int TOTAL = 1024 /* alignment slack */ + Q_BYTES + NSTAGE * STAGE + BARS;
};

// P = exp2(S * scale - m_ref) of one thread's HC keys, rounded to the operand type and written to tensor memory at p_addr
// (16-bit pairs); returns the sum of the unrounded weights. A tile's exponentials are exactly what the special-function
// unit does in the time the tensor pipe takes for the tile's products (16 a clock against 128 x 128 x 256 flops), so
// EMU_OF_16 of every 16 pairs take the FMA pipe instead (tc05::ex2_pair_fma), and the scaling and the sum run as packed pairs.
#ifndef NS_PREFILL_EMU_OF_16
#define NS_PREFILL_EMU_OF_16 4
#endif
template <int HC, int BF16>
__device__ __forceinline__ float softmax_weights(const float* s, float scale_log2, float neg_m, uint32_t p_addr) {
    constexpr int EMU = NS_PREFILL_EMU_OF_16;
    const uint64_t sc2 = pack2(scale_log2, scale_log2), nm2 = pack2(neg_m, neg_m);
    uint64_t sum2 = pack2(0.f, 0.f);
#pragma unroll
    for (int c = 0; c < HC / 32; ++c) {
        uint32_t w[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const uint64_t x2 = fma2(pack2(s[c * 32 + 2 * e], s[c * 32 + 2 * e + 1]), sc2, nm2);
            float a, b;
            // which pairs: spread evenly over the 16, so that both pipes have work all along the unrolled loop
            if (((e + 1) * EMU) / 16 != (e * EMU) / 16) {
                ex2_pair_fma(x2, a, b);
            } else {
                float xa, xb;
                unpack2(x2, xa, xb);
                a = ex2(xa);
                b = ex2(xb);
            }
            sum2 = add2(sum2, pack2(a, b));
            if (BF16) {
                __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
                w[e] = *reinterpret_cast<uint32_t*>(&t);
            } else {
                __half2 t = __floats2half2_rn(a, b);
                w[e] = *reinterpret_cast<uint32_t*>(&t);
            }
        }
        tmem_st16(p_addr + c * 16, w);
    }
    float sa, sb;
    unpack2(sum2, sa, sb);
    return sa + sb;
}

template <int DQK, int DV, int BN, int NSTAGE, int BF16, int NG>
__global__ void __launch_bounds__(SOFTMAX_THREADS * (NG + 1), 1)
flash_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                     const Params p) {
    using L = Smem<DQK, DV, BN, NSTAGE>;
    constexpr int S_COLS = BN;                   // fp32 columns of one S buffer
    constexpr int HC = BN / NG;                  // keys of a tile a softmax thread owns
    constexpr int O_COL = 2 * S_COLS;            // the groups' O accumulators after the two S buffers
    constexpr int TMEM_COLS = (O_COL + NG * DV) <= 256 ? 256 : 512;
    // The MMA warp shares its scheduler with softmax warps and must not starve behind them: it is warp 0, the TMA
    // warp is warp 1, warps 2 and 3 only wait for the teardown, and the softmax warps follow (a warp reads the
    // tensor-memory lanes 32 (warp % 4) .. + 31, so a group is four consecutive warps starting at a multiple of four).
    constexpr int MMA_WARP = 0, TMA_WARP = 1, SOFTMAX_WARP0 = 4;
    static_assert(NG == 1 || NG == 2, "one or two softmax groups");
    static_assert(O_COL + NG * DV <= 512, "tensor memory holds 512 columns");
    static_assert(DQK % 64 == 0 && DV % 64 == 0 && HC % 32 == 0, "tiles in 64-element swizzle chunks");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);   // 128-byte swizzle wants 1024-byte tile bases
    uint8_t* q_s = smem;
    uint8_t* kv_s = smem + L::Q_BYTES;
    uint64_t* bars = (uint64_t*) (kv_s + NSTAGE * L::STAGE);
    // barrier map
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;                 // [2] the first two key tiles, one use each
    uint64_t* f_full = k_full + 2;               // [NSTAGE] what pass j of the MMA warp reads: V(j) and K(j+2)
    uint64_t* k_empty = f_full + NSTAGE;         // [NSTAGE]
    uint64_t* v_empty = k_empty + NSTAGE;        // [NSTAGE]
    uint64_t* s_full = v_empty + NSTAGE;         // [2]
    uint64_t* p_full = s_full + 2;               // [2] every softmax thread of every group arrives
    uint64_t* pv_done = p_full + 2;              // [1]
    uint64_t* o_final = pv_done + 1;             // [1] the last P V done
    uint32_t* tmem_slot = (uint32_t*) (o_final + 1);
    volatile int* abort_flag = (volatile int*) (tmem_slot + 1);
    volatile int* gave_up = abort_flag + 1;                   // a softmax thread left its loop early
    float2* ml_s = (float2*) q_s;   // [NG][128] the groups' (maximum, sum) in the epilogue, when no product reads Q any more

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // CTAs start in the order of their length: within a chunk of heads the row block with the most keys first, for every
    // head of the chunk, then the next shorter one, so the last CTAs to start are the shortest (head by head, the last
    // heads' long blocks started late: 30 against 20 tile times for 2,048 rows of 16 heads on 148 SMs). A chunk is as
    // many heads as keep their keys and values in L2 together: with all 128 heads of the MLA shape in one chunk every
    // CTA streamed its own head from HBM and the kernel took half as long again.
    const int per_chunk = p.chunk * p.nblk;
    const int c0 = ((int) blockIdx.x / per_chunk) * p.chunk, rem = (int) blockIdx.x % per_chunk;
    const int heads_c = min(p.chunk, p.Hq - c0);
    const int mblk = p.nblk - 1 - rem / heads_c;
    const int h = c0 + rem % heads_c, hk = h / p.G;
    const int r0 = mblk * BM;
    // keys this row block sees: up to the position of its last row
    const int64_t last_pos = p.p0 + min((int64_t) r0 + BM, (int64_t) p.T) - 1;
    const int ntiles = (int) (last_pos / BN) + 1;

    if (tid == 0) {
        *abort_flag = 0;
        *gave_up = 0;
        mbar_init(smem_u32(q_full), 1);
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(smem_u32(f_full + s), 1);
            mbar_init(smem_u32(k_empty + s), 1);
            mbar_init(smem_u32(v_empty + s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(k_full + s), 1);
            mbar_init(smem_u32(s_full + s), 1);
            mbar_init(smem_u32(p_full + s), SOFTMAX_THREADS * NG);
        }
        mbar_init(smem_u32(pv_done), 1);
        mbar_init(smem_u32(o_final), 1);
        mbar_fence_init();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == TMA_WARP) {
        // ================= TMA producer: keys two tiles ahead of the values (S(j+2) is issued with P(j) V(j)); what one
        // pass of the MMA warp reads, V(j) and K(j+2), lands on one barrier =================
        if (elect_one()) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
            mbar_expect_tx(smem_u32(q_full), L::Q_BYTES);
            for (int c = 0; c < DQK / 64; ++c) tma_load_3d(smem_u32(q_s + c * (BM * 128)), &tm_q, c * 64, h, r0, smem_u32(q_full));
            bool ok = true;
            // a key tile and a value tile that signal `bar`, after their stages are free (either may be absent: j < 0)
            auto load = [&](int jk, int jv, uint64_t* bar) {
                if (jk >= NSTAGE) ok = mbar_wait(smem_u32(k_empty + jk % NSTAGE), ((uint32_t) (jk / NSTAGE) & 1) ^ 1, abort_flag, p.status, 101);
                if (ok && jv >= NSTAGE) ok = mbar_wait(smem_u32(v_empty + jv % NSTAGE), ((uint32_t) (jv / NSTAGE) & 1) ^ 1, abort_flag, p.status, 102);
                if (!ok) return;
                mbar_expect_tx(smem_u32(bar), (jk >= 0 ? L::K_BYTES : 0) + (jv >= 0 ? L::V_BYTES : 0));
                if (jk >= 0) {
                    uint8_t* ks = kv_s + (jk % NSTAGE) * L::STAGE;
                    for (int c = 0; c < DQK / 64; ++c) tma_load_3d(smem_u32(ks + c * (BN * 128)), &tm_k, c * 64, jk * BN, hk, smem_u32(bar));
                }
                if (jv >= 0) {
                    uint8_t* vs = kv_s + (jv % NSTAGE) * L::STAGE + L::K_BYTES;
                    for (int c = 0; c < DV / 64; ++c) tma_load_3d(smem_u32(vs + c * (BN * 128)), &tm_v, c * 64, jv * BN, hk, smem_u32(bar));
                }
            };
            for (int j = 0; j < 2 && j < ntiles && ok; ++j) load(j, -1, k_full + j);
            for (int j = 0; j < ntiles && ok; ++j) load(j + 2 < ntiles ? j + 2 : -1, j, f_full + j % NSTAGE);
        }
    } else if (warp == MMA_WARP) {
        // ================= MMA issuer =================
        // Order on the tensor pipe: S(0) S(1) PV(0) S(2) PV(1) S(3) ... - S(j+2) goes into the buffer P(j) lived in, behind
        // P(j) V(j) of the same thread, and runs while the softmax works on S(j+1). A wait on a barrier that is already
        // complete still costs this thread over a hundred clocks, so between P(j) becoming ready and S(j+2) being in the
        // pipe there is one wait only: the loads a pass needs were waited for at the end of the pass before.
        if (elect_one()) {
            constexpr uint32_t idesc_qk = idesc_f16(BM, BN, BF16, 0, 0);
            constexpr uint32_t idesc_pv = idesc_f16(BM, DV, BF16, 0, 1);
            auto issue_qk = [&](int j) {
                const int s = j % NSTAGE;
                const uint32_t kb = smem_u32(kv_s + s * L::STAGE), qb = smem_u32(q_s);
                const uint32_t d = tmem + (uint32_t) ((j & 1) * S_COLS);
#pragma unroll
                for (int k = 0; k < DQK / 16; ++k) {
                    const uint64_t ad = smem_desc_sw128(qb + (k / 4) * (BM * 128) + (k % 4) * 32, 16, 1024);
                    const uint64_t bd = smem_desc_sw128(kb + (k / 4) * (BN * 128) + (k % 4) * 32, 16, 1024);
                    mma_ss(d, ad, bd, idesc_qk, k > 0);
                }
                mma_commit(smem_u32(k_empty + s));       // the K stage is free once these MMAs have read it
                mma_commit(smem_u32(s_full + (j & 1)));  // and S is ready for the softmax
            };
            auto wait_f = [&](int j) { return mbar_wait(smem_u32(f_full + j % NSTAGE), (uint32_t) (j / NSTAGE) & 1, abort_flag, p.status, 204); };
            bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, p.status, 201);
            for (int j = 0; j < 2 && j < ntiles && ok; ++j) {
                ok = mbar_wait(smem_u32(k_full + j), 0, abort_flag, p.status, 202);
                if (ok) {
                    fence_after_sync();
                    issue_qk(j);
                }
            }
            if (ok) ok = wait_f(0);
            for (int j = 0; j < ntiles && ok; ++j) {
                const int s = j % NSTAGE;
                ok = mbar_wait(smem_u32(p_full + (j & 1)), (uint32_t) (j >> 1) & 1, abort_flag, p.status, 205);
                if (!ok) break;
                fence_after_sync();
                const uint32_t vb = smem_u32(kv_s + s * L::STAGE + L::K_BYTES);
#pragma unroll
                for (int g = 0; g < NG; ++g) {
                    // group g's keys of the tile: its P (over its own part of the S buffer) into its own accumulator
                    const uint32_t pa = tmem + (uint32_t) ((j & 1) * S_COLS + g * HC);
                    const uint32_t od = tmem + (uint32_t) (O_COL + g * DV);
#pragma unroll
                    for (int k = 0; k < HC / 16; ++k) {
                        // V tile: DV/64 chunks of [BN keys][64] 128 bytes a key; 16 keys a step
                        const uint64_t bd = smem_desc_sw128(vb + (g * (HC / 16) + k) * (16 * 128), BN * 128, 1024);
                        mma_ts(od, pa + (uint32_t) (k * 8), bd, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
                    }
                }
                mma_commit(smem_u32(pv_done));
                // the V stage is free after these products: with two stages its reload is the next thing the ring needs,
                // with three it can wait until S(j+2) is out
                if (NSTAGE < 3) mma_commit(smem_u32(v_empty + s));
                if (j + 2 < ntiles) issue_qk(j + 2);
                if (NSTAGE >= 3) mma_commit(smem_u32(v_empty + s));
                if (j == ntiles - 1) mma_commit(smem_u32(o_final));
                // off the critical path: what the next pass reads
                if (j + 1 < ntiles) ok = wait_f(j + 1);
            }
        }
    } else if (warp >= SOFTMAX_WARP0) {
        // ================= softmax: thread r of group grp owns query row r0 + r and HC keys of every tile ==========
        const int grp = (warp - SOFTMAX_WARP0) >> 2;
        const int r = tid & (SOFTMAX_THREADS - 1);          // 0..127 = tensor-memory lane
        const uint32_t lane_base = (uint32_t) ((warp & 3) * 32) << 16;
        const int64_t row_pos = p.p0 + r0 + r;              // last key this row sees
        const bool row_live = r0 + r < p.T;
        float m_ref = -INFINITY, l = 0.f;                   // m_ref in units of S * scale_log2
        bool ok = true;
        for (int j = 0; j < ntiles; ++j) {
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(s_full + (j & 1)), (uint32_t) (j >> 1) & 1, abort_flag, p.status, 301));
            if (!ok) break;
            fence_after_sync();
            const uint32_t s_addr = tmem + lane_base + (uint32_t) ((j & 1) * S_COLS + grp * HC);
            float s[HC];
            {
                uint32_t v[HC / 32][32];
#pragma unroll
                for (int c = 0; c < HC / 32; ++c) tmem_ld32(s_addr + c * 32, v[c]);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < HC / 32; ++c)
#pragma unroll
                    for (int e = 0; e < 32; ++e) s[c * 32 + e] = __uint_as_float(v[c][e]);
            }
            const int64_t k0 = (int64_t) j * BN + grp * HC;
            // mask: keys past the row's position (the causal edge; it also covers keys past kv_len)
            if (k0 + HC - 1 > row_pos) {
#pragma unroll
                for (int e = 0; e < HC; ++e)
                    if (k0 + e > row_pos) s[e] = -INFINITY;
            }
            float mx = -INFINITY;
#pragma unroll
            for (int e = 0; e < HC; e += 2) mx = max3(mx, s[e], s[e + 1]);
            mx *= p.scale_log2;
            // lazy rescale: move the reference maximum only when it would grow by more than 2^8
            float corr = 1.0f;
            bool need = false;
            if (j == 0 || m_ref == -INFINITY) {
                m_ref = mx;   // nothing weighed yet: O and l are zero, whatever the reference was
            } else if (mx > m_ref + RESCALE_LOG2) {
                corr = ex2(m_ref - mx);
                m_ref = mx;
                need = true;
            }
            if (__any_sync(0xffffffffu, need)) {
                // O must be at rest: P(j-1) V(j-1) done
                ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(pv_done), (uint32_t) (j - 1) & 1, abort_flag, p.status, 302));
                if (!ok) break;
                fence_after_sync();
                const uint32_t o_addr = tmem + lane_base + (uint32_t) (O_COL + grp * DV);
#pragma unroll
                for (int c = 0; c < DV / 32; ++c) {
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
            // P = exp2(S * scale - m_ref), the sum from the unrounded weights, P rounded to the operand type
            const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
            const uint32_t p_addr = s_addr;   // P overlays the first half of the S columns it came from
            l += softmax_weights<HC, BF16>(s, p.scale_log2, neg_m, p_addr);
            tmem_wait_st();
            fence_before_sync();
            mbar_arrive(smem_u32(p_full + (j & 1)));
        }
        // ---- epilogue: O / l to global memory
        // (pv_done cannot serve here: a parity wait only tells the current phase from the one before it, and this thread
        // has not followed its phases; o_final completes exactly once, after the last product)
        if (ok) ok = mbar_wait(smem_u32(o_final), 0, abort_flag, p.status, 303);
        ok = __all_sync(0xffffffffu, ok);
        // two groups: each writes half of the row's columns from both accumulators under the common maximum
        float wgt[NG];
        wgt[0] = 1.0f;
        if (NG > 1) {
            ml_s[grp * SOFTMAX_THREADS + r] = make_float2(m_ref, l);
            if (!ok) *gave_up = 1;
            named_bar_sync(1, SOFTMAX_THREADS * NG);   // every softmax thread gets here: its waits are bounded
            ok = *gave_up == 0;
            float mx = -INFINITY;
#pragma unroll
            for (int g = 0; g < NG; ++g) mx = fmaxf(mx, ml_s[g * SOFTMAX_THREADS + r].x);
            l = 0.f;
#pragma unroll
            for (int g = 0; g < NG; ++g) {
                const float2 ml = ml_s[g * SOFTMAX_THREADS + r];
                wgt[g] = ml.x == -INFINITY ? 0.f : ex2(ml.x - mx);
                l += ml.y * wgt[g];
            }
        }
        if (ok) {
            fence_after_sync();
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            const uint32_t o_addr = tmem + lane_base + (uint32_t) O_COL;
            const int64_t row = (int64_t) (r0 + r) * p.Hq + h;
#pragma unroll
            for (int cc = 0; cc < DV / 32 / NG; ++cc) {
                const int c = grp * (DV / 32 / NG) + cc;
                uint32_t v[32];
                tmem_ld32(o_addr + c * 32, v);
                tmem_wait_ld();
                if (NG > 1) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * wgt[0]);
#pragma unroll
                    for (int g = 1; g < NG; ++g) {
                        uint32_t u[32];
                        tmem_ld32(o_addr + g * DV + c * 32, u);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(fmaf(__uint_as_float(u[e]), wgt[g], __uint_as_float(v[e])));
                    }
                }
                if (row_live) {
                    if (p.out_kind == 0) {
                        float4* dst = reinterpret_cast<float4*>((float*) p.out + row * DV + c * 32);
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
                        uint4* dst = reinterpret_cast<uint4*>((uint16_t*) p.out + row * DV + c * 32);
#pragma unroll
                        for (int e = 0; e < 4; ++e) dst[e] = make_uint4(w[4 * e], w[4 * e + 1], w[4 * e + 2], w[4 * e + 3]);
                    }
                }
            }
        }
    }
    // ---- teardown: every role is out of its loops (all waits are bounded); tensor memory goes back
    fence_before_sync();
    __syncthreads();
    if (warp == MMA_WARP) {
        fence_after_sync();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// ---- the streaming form ---------------------------------------------------------------------------------------------
// The same arithmetic, tile for tile, for prompts whose (row block, head) items are a few times the SMs: there a CTA an item
// leaves the SMs idle between items (a CTA's fixed part - set-up, the first loads, the epilogue - is four tile times) and,
// with fewer than two waves, at the end. Here one CTA an SM works through its share of the items as ONE stream of key tiles.

template <int DQK, int DV, int BN, int NSTAGE, int NG>
struct StreamSmem {
    static constexpr int Q_BYTES = BM * DQK * 2;
    static constexpr int K_BYTES = BN * DQK * 2;
    static constexpr int V_BYTES = BN * DV * 2;
    static constexpr int STAGE = K_BYTES + V_BYTES;
    static constexpr int BARS = 256;    // mbarriers, the tensor-memory base slot, the flags
    static constexpr int ML_BYTES = NG > 1 ? NG * SOFTMAX_THREADS * 8 : 0;   // the groups' (maximum, sum) in the epilogue
    static constexpr int USED = Q_BYTES + NSTAGE * STAGE + BARS + ML_BYTES;
    // the 128-byte swizzle wants tile bases on 1,024-byte boundaries. Where there is room the kernel asks for 1,024 bytes
    // more and rounds its base up; the largest instance has no room, asks for an aligned array and checks what it got.
    static constexpr int SLACK = USED + 1024 <= 232448 ? 1024 : 0;
    static constexpr int TOTAL = USED + SLACK;
};

// n / d for n < 2^31, with inv = floor(2^32 / d) (2^32 - 1 for d = 1)
__device__ __forceinline__ int fast_div(int n, int d, uint32_t inv) {
    int q = (int) __umulhi((uint32_t) n, inv);
    return n - q * d >= d ? q + 1 : q;
}

// one (row block, head) of the CTA's list, and a position in the tiles of the list
struct Cursor {
    int rnd, j;                // the round of the deal the item came from (the number of rounds: the list is at its end); the item's tile
    int h, r0, ntiles;         // query head, first row, key tiles the row block sees
};

template <int DQK, int DV, int BN, int NSTAGE, int BF16, int NG>
__global__ void __launch_bounds__(SOFTMAX_THREADS * (NG + 1), 1)
flash_prefill_stream_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                     const Params p) {
    using L = StreamSmem<DQK, DV, BN, NSTAGE, NG>;
    constexpr int S_COLS = BN;                   // fp32 columns of one S buffer
    constexpr int HC = BN / NG;                  // keys of a tile a softmax thread owns
    constexpr int O_COL = 2 * S_COLS;            // the groups' O accumulators after the two S buffers
    constexpr int TMEM_COLS = (O_COL + NG * DV) <= 256 ? 256 : 512;
    // The MMA warp shares its scheduler with softmax warps and must not starve behind them: it is warp 0, the TMA
    // warp is warp 1, warps 2 and 3 only wait for the teardown, and the softmax warps follow (a warp reads the
    // tensor-memory lanes 32 (warp % 4) .. + 31, so a group is four consecutive warps starting at a multiple of four).
    constexpr int MMA_WARP = 0, TMA_WARP = 1, SOFTMAX_WARP0 = 4;
    static_assert(NG == 1 || NG == 2, "one or two softmax groups");
    static_assert(O_COL + NG * DV <= 512, "tensor memory holds 512 columns");
    static_assert(DQK % 64 == 0 && DV % 64 == 0 && HC % 32 == 0, "tiles in 64-element swizzle chunks");

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    if (L::SLACK == 0 && smem != smem_raw) {      // the same for every thread: nothing has been set up yet
        if (threadIdx.x == 0 && p.status) *(volatile int*) p.status = 104;
        return;
    }
    uint8_t* q_s = smem;
    uint8_t* kv_s = smem + L::Q_BYTES;
    uint64_t* bars = (uint64_t*) (kv_s + NSTAGE * L::STAGE);
    // barrier map
    uint64_t* q_full = bars + 0;                 // Q of the next item landed
    uint64_t* q_empty = bars + 1;                // the item's last S is done: Q may be overwritten
    uint64_t* k_full = bars + 2;                 // [2] the CTA's first two key tiles, one use each
    uint64_t* f_full = k_full + 2;               // [NSTAGE] what pass t of the MMA warp reads: V(t) and K(t+2)
    uint64_t* k_empty = f_full + NSTAGE;         // [NSTAGE]
    uint64_t* v_empty = k_empty + NSTAGE;        // [NSTAGE]
    uint64_t* s_full = v_empty + NSTAGE;         // [2]
    uint64_t* p_full = s_full + 2;               // [2] every softmax thread of every group arrives
    uint64_t* pv_done = p_full + 2;              // [1] once a pass
    uint64_t* o_final = pv_done + 1;             // [1] the item's last P V done
    uint64_t* o_free = o_final + 1;              // [1] every softmax thread has read the item's O
    uint32_t* tmem_slot = (uint32_t*) (o_free + 1);
    volatile int* abort_flag = (volatile int*) (tmem_slot + 1);
    volatile int* gave_up = abort_flag + 1;                   // a softmax thread left its loop early
    float2* ml_s = (float2*) ((uint8_t*) bars + L::BARS);     // [NG][128]

    const int tid = threadIdx.x, warp = tid >> 5;

    // ---- the CTA's list of work. A CTA works through several (row block, head) items as ONE stream of key tiles: the
    // loads, the S products and the softmax of an item's first tiles run while the item before is still in its last
    // products, and between two items the tensor pipe waits only for the epilogue to have read O. Items are numbered in
    // the order of their length - within a chunk of heads the row block with the most keys first, for every head of the
    // chunk, then the next shorter one (a chunk is as many heads as keep their keys and values in L2 together: with all
    // 128 heads of the MLA shape in one chunk every CTA streamed its own head from HBM and the kernel took half as long
    // again) - and dealt to the G CTAs back and forth (CTA c takes items c, 2 G - 1 - c, 2 G + c, ...), so that the CTA
    // with the longest item of one round gets the shortest of the next. Every role walks the same list on its own.
    const int nitems = p.nblk * p.Hq, G = (int) gridDim.x, nrounds = (nitems + G - 1) / G;
    auto next_item = [&](Cursor& c) {
        for (++c.rnd; c.rnd < nrounds; ++c.rnd) {
            const int item = c.rnd * G + ((c.rnd & 1) ? G - 1 - (int) blockIdx.x : (int) blockIdx.x);
            if (item >= nitems) continue;
            const int per_chunk = p.chunk * p.nblk;
            const int ch = fast_div(item, per_chunk, p.inv_per_chunk), c0 = ch * p.chunk, rem = item - ch * per_chunk;
            const bool tail = p.Hq - c0 < p.chunk;
            const int heads_c = tail ? p.Hq - c0 : p.chunk;
            const int blk = fast_div(rem, heads_c, tail ? p.inv_tail : p.inv_chunk);
            const int mblk = p.nblk - 1 - blk;
            c.h = c0 + rem - blk * heads_c;
            c.r0 = mblk * BM;
            // keys this row block sees: up to the position of its last row
            const int64_t last_pos = p.p0 + min((int64_t) c.r0 + BM, (int64_t) p.T) - 1;
            c.ntiles = (int) (last_pos / BN) + 1;
            c.j = 0;
            return;
        }
    };
    auto live = [&](const Cursor& c) { return c.rnd < nrounds; };
    auto advance = [&](Cursor& c) {
        if (++c.j >= c.ntiles) next_item(c);
    };

    if (tid == 0) {
        *abort_flag = 0;
        *gave_up = 0;
        mbar_init(smem_u32(q_full), 1);
        mbar_init(smem_u32(q_empty), 1);
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(smem_u32(f_full + s), 1);
            mbar_init(smem_u32(k_empty + s), 1);
            mbar_init(smem_u32(v_empty + s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(k_full + s), 1);
            mbar_init(smem_u32(s_full + s), 1);
            mbar_init(smem_u32(p_full + s), SOFTMAX_THREADS * NG);
        }
        mbar_init(smem_u32(pv_done), 1);
        mbar_init(smem_u32(o_final), 1);
        mbar_init(smem_u32(o_free), SOFTMAX_THREADS * NG);
        mbar_fence_init();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    Cursor first;        // every thread works the CTA's first item out for itself
    first.rnd = -1;
    next_item(first);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    // Tiles are counted through the whole list: tile t uses stage t % NSTAGE of the ring and S buffer t & 1, whatever
    // item it belongs to, so every barrier's phases run on without a break.
    if (warp == TMA_WARP) {
        // ================= TMA producer: keys two tiles ahead of the values (S(t+2) is issued with P(t) V(t)); what one
        // pass of the MMA warp reads, V(t) and K(t+2), lands on one barrier. Q of an item goes out before the item's first
        // key tile, once the last S of the item before has read the old one =================
        if (elect_one()) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
            bool ok = true;
            Cursor ck = first, cv = first;
            int tk = 0, tv = 0, mq = 0;   // key tiles, value tiles, items' queries requested so far
            // the key tile at ck onto `bar` (whose byte count the caller has announced); Q of an item follows the item's first
            // key tile (which shares its barrier with a value tile of the item before and must not wait for Q's buffer)
            auto load_k = [&](uint64_t* bar) {
                if (tk >= NSTAGE) ok = mbar_wait(smem_u32(k_empty + tk % NSTAGE), ((uint32_t) (tk / NSTAGE) & 1) ^ 1, abort_flag, p.status, 101);
                if (!ok) return;
                uint8_t* ks = kv_s + (tk % NSTAGE) * L::STAGE;
                const int hk = fast_div(ck.h, p.G, p.inv_G);
                for (int c = 0; c < DQK / 64; ++c) tma_load_3d(smem_u32(ks + c * (BN * 128)), &tm_k, c * 64, ck.j * BN, hk, smem_u32(bar));
                if (ck.j == 0) {
                    if (mq > 0) ok = mbar_wait(smem_u32(q_empty), (uint32_t) (mq - 1) & 1, abort_flag, p.status, 103);
                    if (!ok) return;
                    mbar_expect_tx(smem_u32(q_full), L::Q_BYTES);
                    for (int c = 0; c < DQK / 64; ++c) tma_load_3d(smem_u32(q_s + c * (BM * 128)), &tm_q, c * 64, ck.h, ck.r0, smem_u32(q_full));
                    ++mq;
                }
                ++tk;
                advance(ck);
            };
            for (int i = 0; i < 2 && live(ck) && ok; ++i) {
                mbar_expect_tx(smem_u32(k_full + i), L::K_BYTES);
                load_k(k_full + i);
            }
            while (live(cv) && ok) {
                // the value tile first: its stage came free with the product before last, the key stage only once the S
                // issued behind that product has run
                uint64_t* bar = f_full + tv % NSTAGE;
                if (tv >= NSTAGE) ok = mbar_wait(smem_u32(v_empty + tv % NSTAGE), ((uint32_t) (tv / NSTAGE) & 1) ^ 1, abort_flag, p.status, 102);
                if (!ok) break;
                mbar_expect_tx(smem_u32(bar), L::V_BYTES + (live(ck) ? L::K_BYTES : 0));
                uint8_t* vs = kv_s + (tv % NSTAGE) * L::STAGE + L::K_BYTES;
                const int hk = fast_div(cv.h, p.G, p.inv_G);
                for (int c = 0; c < DV / 64; ++c) tma_load_3d(smem_u32(vs + c * (BN * 128)), &tm_v, c * 64, cv.j * BN, hk, smem_u32(bar));
                ++tv;
                advance(cv);
                if (live(ck)) load_k(bar);
            }
        }
    } else if (warp == MMA_WARP) {
        // ================= MMA issuer =================
        // Order on the tensor pipe: S(0) S(1) PV(0) S(2) PV(1) S(3) ... - S(t+2) goes into the buffer P(t) lived in, behind
        // P(t) V(t) of the same thread, and runs while the softmax works on S(t+1). A wait on a barrier that is already
        // complete still costs this thread over a hundred clocks, so between P(t) becoming ready and S(t+2) being in the
        // pipe there is one wait only (two where an item begins): the loads a pass needs were waited for at the end of the
        // pass before.
        if (elect_one()) {
            constexpr uint32_t idesc_qk = idesc_f16(BM, BN, BF16, 0, 0);
            constexpr uint32_t idesc_pv = idesc_f16(BM, DV, BF16, 0, 1);
            bool ok = true;
            Cursor cs = first, cp = first;
            int ts = 0, tp = 0, ms = 0, mp = 0;   // S tiles issued, passes done, items whose S has begun, items finished
            auto issue_qk = [&]() {
                if (ts < 2) {   // the CTA's first two key tiles have barriers of their own
                    ok = mbar_wait(smem_u32(k_full + ts), 0, abort_flag, p.status, 202);
                    if (!ok) return;
                    fence_after_sync();
                }
                if (cs.j == 0) {
                    ok = mbar_wait(smem_u32(q_full), (uint32_t) ms & 1, abort_flag, p.status, 201);
                    if (!ok) return;
                    fence_after_sync();
                    ++ms;
                }
                const int s = ts % NSTAGE;
                const uint32_t kb = smem_u32(kv_s + s * L::STAGE), qb = smem_u32(q_s);
                const uint32_t d = tmem + (uint32_t) ((ts & 1) * S_COLS);
#pragma unroll
                for (int k = 0; k < DQK / 16; ++k) {
                    const uint64_t ad = smem_desc_sw128(qb + (k / 4) * (BM * 128) + (k % 4) * 32, 16, 1024);
                    const uint64_t bd = smem_desc_sw128(kb + (k / 4) * (BN * 128) + (k % 4) * 32, 16, 1024);
                    mma_ss(d, ad, bd, idesc_qk, k > 0);
                }
                mma_commit(smem_u32(k_empty + s));        // the K stage is free once these MMAs have read it
                mma_commit(smem_u32(s_full + (ts & 1)));  // and S is ready for the softmax
                if (cs.j == cs.ntiles - 1) mma_commit(smem_u32(q_empty));   // and, behind the item's last S, Q
                ++ts;
                advance(cs);
            };
            auto wait_f = [&](int t) { return mbar_wait(smem_u32(f_full + t % NSTAGE), (uint32_t) (t / NSTAGE) & 1, abort_flag, p.status, 204); };
            while (live(cs) && cs.rnd == cp.rnd && ts < 2 && ok) issue_qk();
            if (ok) ok = wait_f(0);
            while (live(cp) && ok) {
                const int s = tp % NSTAGE;
                ok = mbar_wait(smem_u32(p_full + (tp & 1)), (uint32_t) (tp >> 1) & 1, abort_flag, p.status, 205);
                // an item's first product overwrites O: the epilogue of the item before must have read it
                if (ok && cp.j == 0 && mp > 0) ok = mbar_wait(smem_u32(o_free), (uint32_t) (mp - 1) & 1, abort_flag, p.status, 207);
                if (!ok) break;
                fence_after_sync();
                const uint32_t vb = smem_u32(kv_s + s * L::STAGE + L::K_BYTES);
#pragma unroll
                for (int g = 0; g < NG; ++g) {
                    // group g's keys of the tile: its P (over its own part of the S buffer) into its own accumulator
                    const uint32_t pa = tmem + (uint32_t) ((tp & 1) * S_COLS + g * HC);
                    const uint32_t od = tmem + (uint32_t) (O_COL + g * DV);
#pragma unroll
                    for (int k = 0; k < HC / 16; ++k) {
                        // V tile: DV/64 chunks of [BN keys][64] 128 bytes a key; 16 keys a step
                        const uint64_t bd = smem_desc_sw128(vb + (g * (HC / 16) + k) * (16 * 128), BN * 128, 1024);
                        mma_ts(od, pa + (uint32_t) (k * 8), bd, idesc_pv, (cp.j > 0 || k > 0) ? 1u : 0u);
                    }
                }
                mma_commit(smem_u32(pv_done));
                // the V stage is free after these products: with two stages its reload is the next thing the ring needs,
                // with three it can wait until S(t+2) is out
                if (NSTAGE < 3) mma_commit(smem_u32(v_empty + s));
                if (live(cs) && cs.rnd == cp.rnd) issue_qk();
                if (NSTAGE >= 3) mma_commit(smem_u32(v_empty + s));
                if (cp.j == cp.ntiles - 1) {
                    mma_commit(smem_u32(o_final));
                    ++mp;
                    // the next item's first two S: here and not two passes early, where the wait for its Q (asked for only
                    // once this item's last S had read the old one) would have held back this item's last products; the
                    // softmax gets to them after this item's epilogue
                    while (live(cs) && ts < tp + 3 && ok) issue_qk();
                }
                ++tp;
                advance(cp);
                // off the critical path: what the next pass reads
                if (live(cp) && ok) ok = wait_f(tp);
            }
        }
    } else if (warp >= SOFTMAX_WARP0) {
        // ================= softmax: thread r of group grp owns query row r0 + r and HC keys of every tile ==========
        const int grp = (warp - SOFTMAX_WARP0) >> 2;
        const int r = tid & (SOFTMAX_THREADS - 1);          // 0..127 = tensor-memory lane
        const uint32_t lane_base = (uint32_t) ((warp & 3) * 32) << 16;
        Cursor ci = first;
        int t = 0, m = 0;                                   // tiles and items done
        bool ok = true;
        while (live(ci)) {
        const int r0 = ci.r0, h = ci.h, ntiles = ci.ntiles;
        const int64_t row_pos = p.p0 + r0 + r;              // last key this row sees
        const bool row_live = r0 + r < p.T;
        float m_ref = -INFINITY, l = 0.f;                   // m_ref in units of S * scale_log2
        for (int j = 0; j < ntiles; ++j, ++t) {
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(s_full + (t & 1)), (uint32_t) (t >> 1) & 1, abort_flag, p.status, 301));
            if (!ok) break;
            fence_after_sync();
            const uint32_t s_addr = tmem + lane_base + (uint32_t) ((t & 1) * S_COLS + grp * HC);
            float s[HC];
            {
                uint32_t v[HC / 32][32];
#pragma unroll
                for (int c = 0; c < HC / 32; ++c) tmem_ld32(s_addr + c * 32, v[c]);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < HC / 32; ++c)
#pragma unroll
                    for (int e = 0; e < 32; ++e) s[c * 32 + e] = __uint_as_float(v[c][e]);
            }
            const int64_t k0 = (int64_t) j * BN + grp * HC;
            // mask: keys past the row's position (the causal edge; it also covers keys past kv_len)
            if (k0 + HC - 1 > row_pos) {
#pragma unroll
                for (int e = 0; e < HC; ++e)
                    if (k0 + e > row_pos) s[e] = -INFINITY;
            }
            float mx = -INFINITY;
#pragma unroll
            for (int e = 0; e < HC; e += 2) mx = max3(mx, s[e], s[e + 1]);
            mx *= p.scale_log2;
            // lazy rescale: move the reference maximum only when it would grow by more than 2^8
            float corr = 1.0f;
            bool need = false;
            if (j == 0 || m_ref == -INFINITY) {
                m_ref = mx;   // nothing weighed yet: O and l are zero, whatever the reference was
            } else if (mx > m_ref + RESCALE_LOG2) {
                corr = ex2(m_ref - mx);
                m_ref = mx;
                need = true;
            }
            if (__any_sync(0xffffffffu, need)) {
                // O must be at rest: P(t-1) V(t-1) done (a tile of this item: need is never set on an item's first tile)
                ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(pv_done), (uint32_t) (t - 1) & 1, abort_flag, p.status, 302));
                if (!ok) break;
                fence_after_sync();
                const uint32_t o_addr = tmem + lane_base + (uint32_t) (O_COL + grp * DV);
#pragma unroll
                for (int c = 0; c < DV / 32; ++c) {
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
            // P = exp2(S * scale - m_ref), the sum from the unrounded weights, P rounded to the operand type
            const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
            const uint32_t p_addr = s_addr;   // P overlays the first half of the S columns it came from
            l += softmax_weights<HC, BF16>(s, p.scale_log2, neg_m, p_addr);
            tmem_wait_st();
            fence_before_sync();
            mbar_arrive(smem_u32(p_full + (t & 1)));
        }
        // ---- the item's epilogue: O / l to global memory
        // (pv_done cannot serve here: a parity wait only tells the current phase from the one before it, and this thread
        // has not followed its phases; o_final completes exactly once an item, and every thread waits for every one)
        if (ok) ok = mbar_wait(smem_u32(o_final), (uint32_t) m & 1, abort_flag, p.status, 303);
        ok = __all_sync(0xffffffffu, ok);
        // two groups: each writes half of the row's columns from both accumulators under the common maximum
        float wgt[NG];
        wgt[0] = 1.0f;
        if (NG > 1) {
            ml_s[grp * SOFTMAX_THREADS + r] = make_float2(m_ref, l);
            if (!ok) *gave_up = 1;
            named_bar_sync(1, SOFTMAX_THREADS * NG);   // every softmax thread gets here, in every item: its waits are bounded
            ok = *gave_up == 0;
            float mx = -INFINITY;
#pragma unroll
            for (int g = 0; g < NG; ++g) mx = fmaxf(mx, ml_s[g * SOFTMAX_THREADS + r].x);
            l = 0.f;
#pragma unroll
            for (int g = 0; g < NG; ++g) {
                const float2 ml = ml_s[g * SOFTMAX_THREADS + r];
                wgt[g] = ml.x == -INFINITY ? 0.f : ex2(ml.x - mx);
                l += ml.y * wgt[g];
            }
        }
        if (!ok) break;
        {
            fence_after_sync();
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            const uint32_t o_addr = tmem + lane_base + (uint32_t) O_COL;
            const int64_t row = (int64_t) (r0 + r) * p.Hq + h;
#pragma unroll
            for (int cc = 0; cc < DV / 32 / NG; ++cc) {
                const int c = grp * (DV / 32 / NG) + cc;
                uint32_t v[32];
                tmem_ld32(o_addr + c * 32, v);
                tmem_wait_ld();
                if (NG > 1) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * wgt[0]);
#pragma unroll
                    for (int g = 1; g < NG; ++g) {
                        uint32_t u[32];
                        tmem_ld32(o_addr + g * DV + c * 32, u);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(fmaf(__uint_as_float(u[e]), wgt[g], __uint_as_float(v[e])));
                    }
                }
                if (cc == DV / 32 / NG - 1) {
                    // this thread's last read of O: the next item's first product may overwrite it
                    fence_before_sync();
                    mbar_arrive(smem_u32(o_free));
                }
                if (row_live) {
                    if (p.out_kind == 0) {
                        float4* dst = reinterpret_cast<float4*>((float*) p.out + row * DV + c * 32);
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
                                __nv_bfloat162 t2 = __floats2bfloat162_rn(a, b);
                                w[e] = *reinterpret_cast<uint32_t*>(&t2);
                            } else {
                                __half2 t2 = __floats2half2_rn(a, b);
                                w[e] = *reinterpret_cast<uint32_t*>(&t2);
                            }
                        }
                        uint4* dst = reinterpret_cast<uint4*>((uint16_t*) p.out + row * DV + c * 32);
#pragma unroll
                        for (int e = 0; e < 4; ++e) dst[e] = make_uint4(w[4 * e], w[4 * e + 1], w[4 * e + 2], w[4 * e + 3]);
                    }
                }
            }
        }
        ++m;
        next_item(ci);
        }   // the CTA's items
    }
    // ---- teardown: every role is out of its loops (all waits are bounded); tensor memory goes back
    fence_before_sync();
    __syncthreads();
    if (warp == MMA_WARP) {
        fence_after_sync();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// ---- host side: tensor maps and launch --------------------------------------------------------------------------------

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

// rank-3 map over 16-bit elements: dims (inner, mid, outer) with byte strides for mid and outer; box (64, box_mid, box_outer)
int make_map(CUtensorMap* m, const void* base, int bf16, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes,
             uint32_t box1, uint32_t box2, const char* where) {
    EncodeTiled fn = encode_fn();
    if (!fn) return ns_fail(std::string(where) + ": cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
    cuuint32_t box[3] = {64, box1, box2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ns_fail(std::string(where) + ": tensor map rejected (code " + std::to_string((int) r) + ")");
    return 0;
}

template <int DQK, int DV, int BN, int NSTAGE, int BF16, int NG, bool STREAM>
int launch(ns_gpu* g, const FlashPrefillArgs& a, const char* where) {
    using L = Smem<DQK, DV, BN, NSTAGE>;
    static_assert(L::TOTAL <= 232448, "shared memory of one CTA");
    CUtensorMap tq, tk, tv;
    // Q [T][Hq][DQK]: a box = 128 rows of one head, 64 features
    if (make_map(&tq, a.q, BF16, DQK, (uint64_t) a.Hq, (uint64_t) a.T, (uint64_t) DQK * 2, (uint64_t) a.q_row * 2, 1, BM, where)) return -1;
    // K, V: (feature, key, head); keys past kv_len read as zeros (whatever the buffer holds there is never loaded)
    if (make_map(&tk, a.k, BF16, DQK, (uint64_t) a.kv_len, (uint64_t) a.Hkv, (uint64_t) a.k_key * 2, (uint64_t) a.k_head * 2, BN, 1, where)) return -1;
    if (make_map(&tv, a.v, BF16, DV, (uint64_t) a.kv_len, (uint64_t) a.Hkv, (uint64_t) a.v_key * 2, (uint64_t) a.v_head * 2, BN, 1, where)) return -1;
    Params p;
    p.out = a.out;
    p.status = a.status;
    p.T = (int) a.T;
    p.Hq = (int) a.Hq;
    p.G = (int) (a.Hq / a.Hkv);
    p.out_kind = a.out_f32 ? 0 : 1;
    p.p0 = a.p0;
    p.kv_len = a.kv_len;
    p.scale_log2 = a.scale_log2;
    auto kern = flash_prefill_kernel<DQK, DV, BN, NSTAGE, BF16, NG>;
    static bool set[64] = {};
    if (!set[g->dev & 63]) {
        NS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL), where);
        set[g->dev & 63] = true;
    }
    p.nblk = (int) ((a.T + BM - 1) / BM);
    {
        // key heads whose K and V (kv_len rows each) stay in L2 together: 32 MB of its 126
        const int64_t per_head = a.kv_len * (int64_t) (DQK + DV) * 2;
        const int64_t kvh = std::max<int64_t>(1, std::min<int64_t>(a.Hkv, (32ll << 20) / std::max<int64_t>(per_head, 1)));
        p.chunk = (int) (kvh * p.G);
    }
    if ((int64_t) p.nblk * a.Hq > 0x7fffffffll) return ns_fail(std::string(where) + ": too many row blocks");
    // Short rows, three to eight rounds of items, all of one chunk: the streaming kernel, a CTA an SM (dealt back and forth the
    // items come out even). Up to one round there is nothing to stream; with many rounds, or several chunks (whose lengths
    // start over, which the deal does not even out), a CTA an item, started by the hardware as SMs come free, is as fast or
    // faster; and with long rows an item's fixed part no longer counts while the streaming loop's pass is the longer one
    // (16,384 rows x 2 heads: 134 us streamed, 119 a CTA an item; 2,048 rows x 32 / 64 heads: 47.0 / 86.2 against 48.8 / 90.5).
    const int64_t nitems = (int64_t) p.nblk * a.Hq;
    if constexpr (STREAM) if (p.nblk <= 16 && nitems >= 3ll * g->sms && nitems <= 8ll * g->sms && p.chunk >= a.Hq) {
        using LS = StreamSmem<DQK, DV, BN, NSTAGE, NG>;
        static_assert(LS::TOTAL <= 232448, "shared memory of one CTA");
        auto inv = [](int64_t d) { return d <= 1 ? 0xffffffffu : (uint32_t) ((1ull << 32) / (uint64_t) d); };
        p.inv_per_chunk = inv((int64_t) p.chunk * p.nblk);
        p.inv_chunk = inv(p.chunk);
        p.inv_tail = inv(a.Hq % p.chunk);
        p.inv_G = inv(p.G);
        auto skern = flash_prefill_stream_kernel<DQK, DV, BN, NSTAGE, BF16, NG>;
        static bool sset[64] = {};
        if (!sset[g->dev & 63]) {
            NS_CUDA(cudaFuncSetAttribute(skern, cudaFuncAttributeMaxDynamicSharedMemorySize, LS::TOTAL), where);
            sset[g->dev & 63] = true;
        }
        skern<<<dim3((unsigned) g->sms), SOFTMAX_THREADS * (NG + 1), LS::TOTAL, g->compute>>>(tq, tk, tv, p);
        return ns_launched(where);
    }
    dim3 grid((unsigned) nitems, 1, 1);
    kern<<<grid, SOFTMAX_THREADS * (NG + 1), L::TOTAL, g->compute>>>(tq, tk, tv, p);
    return ns_launched(where);
}

}  // namespace

int ns_launch_flash_prefill(ns_gpu* g, const FlashPrefillArgs& a, const char* where) {
    if (a.T <= 0) return 0;
    if (a.Dqk == 128 && a.Dv == 128 && !a.bf16) return launch<128, 128, 128, 3, 0, 2, true>(g, a, where);
    if (a.Dqk == 128 && a.Dv == 128 && a.bf16) return launch<128, 128, 128, 3, 1, 2, true>(g, a, where);
    if (a.Dqk == 192 && a.Dv == 128 && a.bf16) return launch<192, 128, 128, 2, 1, 2, false>(g, a, where);
    if (a.Dqk == 192 && a.Dv == 128 && !a.bf16) return launch<192, 128, 128, 2, 0, 2, false>(g, a, where);
    if (a.Dqk == 256 && a.Dv == 256 && !a.bf16) return launch<256, 256, 64, 2, 0, 1, false>(g, a, where);
    return ns_fail(std::string(where) + ": head widths 128/128, 192/128 or 256/256");
}
