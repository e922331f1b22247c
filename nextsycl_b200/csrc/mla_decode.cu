// mla_decode.cu: absorbed MLA latent attention at decode widths on the Blackwell tensor path.
//
// What it computes is the middle stage of the reference's fused kernel mla_decode_t (kernels/llm/deepseek2/ds2.cpp:
// 186-235) in the numerics of its GEMM form (llm/deepseek2/src/engine.rs:1204-1224): per (row t, head h) over the
// latent cache [n][576] fp16 (512 latent + 64 rotated), score = (q . c) * scale with q rounded to fp16, softmax over the
// row's cells 0 .. pos0+t, u = sum_p p * c[:512] with p rounded to fp16, fp32 sums.
//
// How: the 128 heads of a row are the M = 128 rows of a tcgen05 tile, so every cell is read once for all heads, and the
// tile is worked on by a PAIR of SMs: the two CTAs of a key split are a cluster of two and share one MMA
// (tcgen05.mma.cta_group::2), each holding 64 of the heads. Grid = (2 x key splits, head tiles, rows). Per CTA: its 64 heads
// of Q in shared memory (72 KB), its heads' whole 512-wide output rows in tensor memory (256 columns in the pair's
// accumulator layout) beside two S buffers, a ring of key slots (its 32 cells of a 64-cell tile, every feature, K-major:
// the pair's halves are the columns of S = Q C^T) and a ring of value slots (every cell, its 256 of the 512 latent
// features, MN-major, for O += P C), P through shared memory. Splits are merged by a second kernel (log-sum-exp combine).
// Every mbarrier wait is bounded; a wait that gives up records a status code and the CTA runs to its teardown.
#include "kernels.cuh"
#include "tc05.cuh"
#include "lse_merge.cuh"

#include <cuda.h>

namespace {
using namespace tc05;

constexpr int L = 512;                         // latent width; a cache row is CR = 512 + rotated part (64 or 0)
constexpr int BM = 128;                        // heads a tile
constexpr int BN = 64;                         // cells a tile
constexpr int DVH = 256;                       // output columns a merge block takes
constexpr int THREADS = 192;
constexpr int PS = 516;                        // floats a partial row: O[512], m, l, 2 pad
constexpr float RESCALE_LOG2 = 8.0f;


// Programmatic dependent launch: the merge kernel's blocks may be placed on SMs as this kernel's CTAs leave; they run
// once this grid has completed and its partials are visible.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// Cells a key split for a row that sees n cells, when `units` (head tiles x rows sharing the launch) such rows are to fill
// `sms` SMs once with pairs of CTAs: whole tiles, at least two of them (a partial costs 2 KB a head).
__host__ __device__ inline int64_t mla_split(int64_t n, int64_t units, int sms) {
    // cell counts are below 2^31 (the callers check): 32-bit divisions, which the device does in a few instructions
    uint32_t want = (uint32_t) sms / (2u * (uint32_t) units);
    if (want < 1) want = 1;
    uint32_t kb = ((uint32_t) n + want - 1) / want;
    kb = (kb + BN - 1) / BN * BN;
    return kb < 2 * BN ? 2 * BN : (int64_t) kb;
}
// Decode widths (at most 8 rows, as the reference's decode kernels): a row's split size comes from its own cells alone,
// so a row of a verify pass sums exactly as the one-row pass at its position does
// (kernels/llm/deepseek41/silo/attn.cpp:316-319). More rows: one size for the pass, from its longest row.
constexpr int64_t DECODE_ROWS = 8;

struct Params {
    const __half* q;       // [T][H][CR] fp16
    const float* sinks;    // per head, natural-log units, or null: a sink joins the denominator only (deepseek41)
    const int* counts;     // per row: cells it attends to (null: pos0 + t + 1)
    int zmul;              // 1: row t has its own cell matrix (third tensor-map coordinate t); 0: one shared cache
    float* out;            // [T][H][512]
    float* part;           // [T][H][ns][PS]
    int* status;
    int T, H, ns;          // ns: splits the partials are laid out for
    int per_row, units, sms;   // per_row: each row's split size from its own cells (mla_split(n, units, sms)); else kb
    int64_t pos0, kb;      // cells a split
    float scale_log2;
    // a context split over several GPUs: this rank's cells only (cap of them; pos0 relative to the first), partials always kept
    int64_t cap;           // 0: no bound beyond the row's own position
    float* const* mailboxes;
    int rank, nranks;
    long long epoch;
};

// cells of the (rank's) cache row t attends to
__device__ __forceinline__ int64_t row_cells(const Params& p, int t) {
    int64_t n = p.counts ? (int64_t) p.counts[t] : p.pos0 + t + 1;
    if (p.cap > 0) n = min(n, p.cap);
    return n > 0 ? n : 0;
}

// ---- the kernel ----------------------------------------------------------------------------------------------------------
// mla_decode_pair_kernel: the two CTAs of a key split are a cluster and share ONE MMA (tcgen05.mma.cta_group::2, M = 128):
// each CTA holds 64 of the tile's 128 heads, S is computed once for the pair, each CTA keeps its heads' whole 512-wide
// output row in tensor memory and reads only its own 64 rows of Q. What a CTA stages of a
// 64-cell tile: for S its 32 cells with all features (K-major; the pair's two halves are the 64 columns of S), for O all 64
// cells with its 256 of the 512 latent features (MN-major; rank 0 features 0-127 and 256-383, rank 1 the others: the two
// N = 256 products take half of their columns from each CTA) - 68 KB against the 72 KB of a whole tile. A pair's accumulator
// of 64 rows a CTA lies in tensor memory as lanes 0-63 = columns [0, N/2), lanes 64-127 = columns [N/2, N): a softmax thread
// owns (head, half of the tile's cells) for S and (head, 256 of the 512 output features) for O; the two threads of a head
// swap their maxima through shared memory once a tile. P cannot stay in tensor memory (a pair's A operand there has to
// be written twice, by warps that do not hold it): it goes through shared memory as a K-major tile, 8 KB a buffer.
// Leader = the CTA of cluster rank 0: its MMA thread issues every product; TMA loads of both CTAs count on its barriers;
// products are committed to both CTAs' barriers (two commits, one address each).
constexpr int PAIR_S_COL = 256;                // tensor-memory columns: O 0..255, two S buffers of 32 columns
template <int CR>
struct PairGeo {
    static constexpr int NCH = CR / 64;                      // feature chunks of a cell row: 9 or 8
    static constexpr int NK = 2, NV = 2;                     // slots of the key ring and of the value ring
    static constexpr int Q_BYTES = 64 * CR * 2;              // this CTA's 64 heads
    static constexpr int KS_BYTES = 32 * CR * 2;             // its 32 cells of a tile, every feature
    static constexpr int VS_BYTES = BN * 256 * 2;            // every cell of the tile, its 256 latent features
    static constexpr int P_BYTES = 64 * 128;                 // 64 heads x 64 cells fp16
    static constexpr int MISC = 2048;                        // the maxima swap (2 x 128 floats), barriers, flags
    static constexpr int SMEM_TOTAL = 1024 + Q_BYTES + NK * KS_BYTES + NV * VS_BYTES + 2 * P_BYTES + MISC;
    static_assert(SMEM_TOTAL <= 232448, "shared memory of one CTA");
};

template <int CR>
__global__ void __launch_bounds__(THREADS, 1)
mla_decode_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_c, const __grid_constant__ CUtensorMap tm_v,
                       const Params p) {
    using G = PairGeo<CR>;
    constexpr int NCH = G::NCH, NK = G::NK, NV = G::NV;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    uint8_t* q_s = smem;                                   // NCH chunks of [64 heads][64 features]
    uint8_t* k_s = q_s + G::Q_BYTES;                       // key ring: slots of NCH chunks of [32 cells][64 features]
    uint8_t* v_s = k_s + NK * G::KS_BYTES;                 // value ring: slots of 4 chunks of [64 cells][64 features]
    uint8_t* p_s = v_s + NV * G::VS_BYTES;                 // two P tiles [64 heads][64 cells]
    float* ex_s = (float*) (p_s + 2 * G::P_BYTES);         // [2][128]: a thread's maximum of the tile, for the head's other thread
    uint64_t* bars = (uint64_t*) (ex_s + 256);
    // The two products have rings of their own, so neither waits for the other's loads: S(j) needs key slot j % NK and S
    // buffer j & 1 (free once the softmax has READ S(j-2): P lives in shared memory, not over S), P(j) V(j) needs value
    // slot j % NV and P(j). "(leader's)": the barrier of the CTA of rank 0 is the one waited on; TMA bytes of both CTAs and
    // the arrivals of both CTAs' softmax threads go there.
    uint64_t* q_full = bars + 0;                 // (leader's) both CTAs' Q landed
    uint64_t* k_full = bars + 1;                 // [NK] (leader's)
    uint64_t* k_empty = k_full + NK;             // [NK] S of the tile done: this CTA's slot is free
    uint64_t* v_full = k_empty + NK;             // [NV] (leader's)
    uint64_t* v_empty = v_full + NV;             // [NV] P V of the tile done
    uint64_t* s_full = v_empty + NV;             // [2]
    uint64_t* s_free = s_full + 2;               // [2] (leader's) 8 arrivals: every softmax warp of the pair has read the buffer
    uint64_t* p_full = s_free + 2;               // [2] (leader's) 8 arrivals: every softmax warp has written its part of P
    uint64_t* p_free = p_full + 2;               // [2] P V of the tile done: the P buffer may be rewritten, O is at rest
    uint64_t* o_final = p_free + 2;              // [1]
    uint32_t* tmem_slot = (uint32_t*) (o_final + 1);
    volatile int* abort_flag = (volatile int*) (tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5;
    const uint32_t rank = cluster_rank();        // = blockIdx.x & 1 for clusters of (2, 1, 1)
    const int split = blockIdx.x >> 1;
    const int h0 = blockIdx.y * BM, t = blockIdx.z;
    const int64_t n = row_cells(p, t);
    const int64_t kb = p.per_row ? mla_split(n, p.units, p.sms) : p.kb;
    const int64_t jbeg = (int64_t) split * kb, jend = min(n, (int64_t) (split + 1) * kb);
    const int ntiles = jbeg < jend ? (int) ((jend - jbeg + BN - 1) / BN) : 0;
    if (ntiles == 0) return;                     // both CTAs of the pair: the split holds none of the row's cells

    if (tid == 0) {
        abort_flag[0] = abort_flag[1] = abort_flag[2] = abort_flag[3] = 0;   // the flag and the softmax threads' bad[3]
        mbar_init(smem_u32(q_full), 1);
        for (int s = 0; s < NK; ++s) {
            mbar_init(smem_u32(k_full + s), 1);
            mbar_init(smem_u32(k_empty + s), 1);
        }
        for (int s = 0; s < NV; ++s) {
            mbar_init(smem_u32(v_full + s), 1);
            mbar_init(smem_u32(v_empty + s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(s_full + s), 1);
            mbar_init(smem_u32(s_free + s), 8);      // a warp's lane 0 arrives for the warp: 4 warps of either CTA
            mbar_init(smem_u32(p_full + s), 8);
            mbar_init(smem_u32(p_free + s), 1);
        }
        mbar_init(smem_u32(o_final), 1);
        mbar_fence_init();
    }
    if (warp == 5) {
        tmem_alloc_pair(smem_u32(tmem_slot), 512);
        tmem_relinquish_pair();
    }
    fence_before_sync();
    __syncthreads();
    cluster_sync();          // the other CTA's barriers are set up before anything of this one counts on them
    fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    pdl_launch_dependents();

    // a thread that polls several barriers in turn gives up after this many idle rounds
    auto idle_out = [&](uint32_t& idle, int code) {
        __nanosleep(40);
        if (*abort_flag || ++idle > WAIT_LIMIT) {
            if (!*abort_flag) {
                *abort_flag = 1;
                if (p.status) {
                    *(volatile int*) p.status = code;
                    __threadfence_system();
                }
            }
            return true;
        }
        return false;
    };

    if (warp == 4) {
        // ================= TMA producer (both CTAs: each loads its own parts; the bytes count on the leader's barriers) ==========
        if (elect_one()) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_c);
            tma_prefetch_desc(&tm_v);
            if (rank == 0) mbar_expect_tx(smem_u32(q_full), 2 * G::Q_BYTES);
            for (int c = 0; c < NCH; ++c) tma_load_3d_pair(smem_u32(q_s + c * (64 * 128)), &tm_q, c * 64, h0 + 64 * (int) rank, t, smem_u32(q_full));
            // the two rings are fed as their slots come free, whichever first
            int jk = 0, jv = 0;
            uint32_t idle = 0;
            while (jk < ntiles || jv < ntiles) {
                bool did = false;
                if (jk < ntiles && (jk < NK || mbar_try(smem_u32(k_empty + jk % NK), ((uint32_t) (jk / NK) & 1) ^ 1))) {
                    const int s = jk % NK;
                    if (rank == 0) mbar_expect_tx(smem_u32(k_full + s), 2 * G::KS_BYTES);
                    uint8_t* ks = k_s + s * G::KS_BYTES;
                    const int cell0 = (int) (jbeg + (int64_t) jk * BN) + 32 * (int) rank;
                    for (int c = 0; c < NCH; ++c) tma_load_3d_pair(smem_u32(ks + c * (32 * 128)), &tm_c, c * 64, cell0, t * p.zmul, smem_u32(k_full + s));
                    ++jk;
                    did = true;
                }
                if (jv < ntiles && (jv < NV || mbar_try(smem_u32(v_empty + jv % NV), ((uint32_t) (jv / NV) & 1) ^ 1))) {
                    const int s = jv % NV;
                    if (rank == 0) mbar_expect_tx(smem_u32(v_full + s), 2 * G::VS_BYTES);
                    uint8_t* vs = v_s + s * G::VS_BYTES;
                    const int cell0 = (int) (jbeg + (int64_t) jv * BN);
                    for (int i = 0; i < 4; ++i) {
                        const int chunk = (i < 2 ? 0 : 4) + 2 * (int) rank + (i & 1);
                        tma_load_3d_pair(smem_u32(vs + i * (BN * 128)), &tm_v, chunk * 64, cell0, t * p.zmul, smem_u32(v_full + s));
                    }
                    ++jv;
                    did = true;
                }
                if (did) {
                    idle = 0;
                    continue;
                }
                if (idle_out(idle, 401)) break;
            }
        }
    } else if (warp == 5) {
        // ================= MMA issuer: the leader's, for the pair =================
        if (rank == 0 && elect_one()) {
            constexpr uint32_t idesc_qk = idesc_f16(BM, BN, 0, 0, 0);
            constexpr uint32_t idesc_pv = idesc_f16(BM, 256, 0, 0, 1);
            // a product's completion is signalled to the same barrier of both CTAs
            auto commit_both = [&](uint64_t* bar) {
                mma_commit_pair(cluster_map(smem_u32(bar), 0));
                mma_commit_pair(cluster_map(smem_u32(bar), 1));
            };
            bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, p.status, 501);
            const uint64_t q_desc0 = smem_desc_sw128(smem_u32(q_s), 16, 1024);
            auto issue_qk = [&](int j) {
                const uint64_t k_desc0 = smem_desc_sw128(smem_u32(k_s + (j % NK) * G::KS_BYTES), 16, 1024);
                const uint32_t d = tmem + (uint32_t) (PAIR_S_COL + (j & 1) * 32);
#pragma unroll
                for (int k = 0; k < CR / 16; ++k) {
                    const int chunk = k / 4, step = k % 4;
                    mma_ss_pair(d, q_desc0 + (uint64_t) ((chunk * (64 * 128) + step * 32) >> 4), k_desc0 + (uint64_t) ((chunk * (32 * 128) + step * 32) >> 4), idesc_qk,
                                k > 0);
                }
                commit_both(k_empty + j % NK);
                commit_both(s_full + (j & 1));
            };
            auto issue_pv = [&](int j) {
                const uint64_t p_desc0 = smem_desc_sw128(smem_u32(p_s + (j & 1) * G::P_BYTES), 16, 1024);
                // the value operand: MN-major, a CTA's 128 features of each product are two chunks of [64 cells][64 features]
                const uint32_t vs = smem_u32(v_s + (j % NV) * G::VS_BYTES);
                const uint64_t va_desc0 = smem_desc_sw128(vs, BN * 128, 1024), vb_desc0 = smem_desc_sw128(vs + 2 * (BN * 128), BN * 128, 1024);
#pragma unroll
                for (int k = 0; k < BN / 16; ++k) {
                    const uint64_t pa = p_desc0 + (uint64_t) ((k * 32) >> 4);
                    const uint32_t acc = (j > 0 || k > 0) ? 1u : 0u;
                    mma_ss_pair(tmem, pa, va_desc0 + (uint64_t) ((k * (16 * 128)) >> 4), idesc_pv, acc);          // features 0..255
                    mma_ss_pair(tmem + 128, pa, vb_desc0 + (uint64_t) ((k * (16 * 128)) >> 4), idesc_pv, acc);    // features 256..511
                }
                commit_both(v_empty + j % NV);
                commit_both(p_free + (j & 1));
                if (j == ntiles - 1) commit_both(o_final);
            };
            // The two products are issued in whatever order their inputs arrive, P V first (it is short, and it is what the
            // softmax's next P buffer and the value ring wait for). A fixed order would queue it behind an S that waits for a load.
            int qk = 0, pv = 0;
            bool v_ready = false;      // value slot of tile pv seen full (a barrier's phase is tested once it can be the wanted one)
            uint32_t idle = 0;
            while (ok && pv < ntiles) {
                bool did = false;
                if (pv < qk) {
                    if (!v_ready) v_ready = mbar_try(smem_u32(v_full + pv % NV), (uint32_t) (pv / NV) & 1);
                    if (v_ready && mbar_try(smem_u32(p_full + (pv & 1)), (uint32_t) (pv >> 1) & 1)) {
                        fence_after_sync();
                        issue_pv(pv);
                        ++pv;
                        v_ready = false;
                        did = true;
                    }
                }
                if (qk < ntiles && (qk < 2 || mbar_try(smem_u32(s_free + (qk & 1)), ((uint32_t) (qk >> 1) & 1) ^ 1)) &&
                    mbar_try(smem_u32(k_full + qk % NK), (uint32_t) (qk / NK) & 1)) {
                    fence_after_sync();
                    issue_qk(qk);
                    ++qk;
                    did = true;
                }
                if (did) {
                    idle = 0;
                    continue;
                }
                if (idle_out(idle, 504)) ok = false;
            }
        }
    } else {
        // ================= softmax: thread L owns head h0 + 64 rank + (L & 63), the cells 32 (L >> 6) .. + 31 of a tile and the
        // output features 128 (L >> 6) .. + 127 and 256 + 128 (L >> 6) .. + 127 =================
        const int row = tid & 63, ch = tid >> 6;
        const int head = h0 + 64 * (int) rank + row;
        const uint32_t lane_base = (uint32_t) (warp * 32) << 16;
        const bool head_live = head < p.H;
        const uint32_t p_full_leader[2] = {cluster_map(smem_u32(p_full), 0), cluster_map(smem_u32(p_full + 1), 0)};
        const uint32_t s_free_leader[2] = {cluster_map(smem_u32(s_free), 0), cluster_map(smem_u32(s_free + 1), 0)};
        float m_ref = -INFINITY, l = 0.f;
        // The 128 threads meet at a named barrier once a tile, so none may leave the loop alone: a thread whose wait gave up (or
        // that sees the CTA's abort flag) says so in bad[] BEFORE the barrier, and everybody decides on bad[] AFTER it - the
        // same value for all, so all leave at the same barrier.
        volatile int* bad = abort_flag + 1;     // [3]: tiles of either parity, the epilogue
        bool ok = true, left = false;
        for (int j = 0; j < ntiles; ++j) {
            // this tile's P buffer was last read by P(j-2) V(j-2): waited for here, where the thread waits for S anyway
            if (j >= 2) ok = ok && mbar_wait(smem_u32(p_free + (j & 1)), ((uint32_t) (j >> 1) & 1) ^ 1, abort_flag, p.status, 604);
            ok = __all_sync(0xffffffffu, ok && mbar_wait(smem_u32(s_full + (j & 1)), (uint32_t) (j >> 1) & 1, abort_flag, p.status, 601));
            float s[32];
            float mx = -INFINITY;
            if (ok) {
                fence_after_sync();
                uint32_t v[32];
                tmem_ld32(tmem + lane_base + (uint32_t) (PAIR_S_COL + (j & 1) * 32), v);
                tmem_wait_ld();
                // the buffer is read: S of two tiles on may overwrite it
                fence_before_sync();
                __syncwarp();
                if ((tid & 31) == 0) mbar_arrive_cluster(s_free_leader[j & 1]);
#pragma unroll
                for (int e = 0; e < 32; ++e) s[e] = __uint_as_float(v[e]);
                const int64_t c0 = jbeg + (int64_t) j * BN + 32 * ch;
                if (c0 + 32 > jend) {
#pragma unroll
                    for (int e = 0; e < 32; ++e)
                        if (c0 + e >= jend) s[e] = -INFINITY;
                }
#pragma unroll
                for (int e = 0; e < 32; ++e) mx = fmaxf(mx, s[e]);
            } else {
#pragma unroll
                for (int e = 0; e < 32; ++e) s[e] = 0.f;
            }
            // the head's other thread holds the tile's other 32 cells
            ex_s[(j & 1) * 128 + tid] = mx;
            if (!ok || *abort_flag) bad[j & 1] = 1;
            named_bar_sync(1, 128);
            if (bad[j & 1]) {
                left = true;
                break;
            }
            mx = fmaxf(mx, ex_s[(j & 1) * 128 + (tid ^ 64)]);
            mx *= p.scale_log2;
            float corr = 1.0f;
            bool need = false;
            if (j == 0) {
                m_ref = mx;
            } else if (mx > m_ref + RESCALE_LOG2) {
                corr = ex2(m_ref - mx);
                m_ref = mx;
                need = true;
            }
            if (__any_sync(0xffffffffu, need)) {
                // O must be at rest: P(j-1) V(j-1) done, the use of its P buffer number (j-1) / 2
                ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(p_free + ((j - 1) & 1)), (uint32_t) ((j - 1) >> 1) & 1, abort_flag, p.status, 602));
                if (ok) {
                    fence_after_sync();
#pragma unroll
                    for (int c = 0; c < 256 / 32; ++c) {
                        uint32_t v[32];
                        tmem_ld32(tmem + lane_base + (uint32_t) (c * 32), v);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * corr);
                        tmem_st32(tmem + lane_base + (uint32_t) (c * 32), v);
                    }
                    tmem_wait_st();
                }
                l *= corr;
            }
            const float neg_m = -m_ref;   // finite: the first cell of the first tile is always inside the split
            float sum = 0.f;
            // P as a K-major operand tile: head `row` is row `row` of 128 bytes, its 16-byte chunks swizzled by the row
            uint8_t* prow = p_s + (j & 1) * G::P_BYTES + row * 128;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float a = ex2(fmaf(s[q * 8 + 2 * e], p.scale_log2, neg_m));
                    const float b = ex2(fmaf(s[q * 8 + 2 * e + 1], p.scale_log2, neg_m));
                    sum += a + b;
                    __half2 hh = __floats2half2_rn(a, b);
                    w[e] = *reinterpret_cast<uint32_t*>(&hh);
                }
                if (ok) *reinterpret_cast<uint4*>(prow + (((4 * ch + q) ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            l += sum;
            fence_proxy_async();
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive_cluster(p_full_leader[j & 1]);
        }
        // ---- epilogue
        if (ok && !left) ok = mbar_wait(smem_u32(o_final), 0, abort_flag, p.status, 603);
        // the head's sum: both threads' shares (under the same maximum)
        ex_s[(ntiles & 1) * 128 + tid] = l;
        if (!ok || left || *abort_flag) bad[2] = 1;
        named_bar_sync(1, 128);
        ok = bad[2] == 0;
        if (ok) {
            fence_after_sync();
            l += ex_s[(ntiles & 1) * 128 + (tid ^ 64)];
            const int64_t grow = (int64_t) t * p.H + head;
            const bool direct = n <= kb && !p.mailboxes;   // the row's only split: normalised and written as the result
            float inv = 1.0f;
            if (direct) {
                float f = 1.0f, den = l;
                if (p.sinks && head_live) {
                    const float sk = p.sinks[head] * 1.4426950408889634f, mx = fmaxf(m_ref, sk);
                    f = ex2(m_ref - mx);
                    den = l * f + ex2(sk - mx);
                }
                inv = den > 0.f ? f / den : 0.f;
            }
            // A thread holds one row of O; written as it lies, a warp's store would touch 32 rows. Each block of 64 columns
            // goes through a padded [32][68] tile in shared memory (the rings are idle by now), so that a warp instruction
            // writes 256 contiguous bytes of each of two rows, 16 bytes a lane.
            float* tile = reinterpret_cast<float*>(k_s) + warp * (32 * 68);
            const int lane = tid & 31, half = lane >> 4, l16 = lane & 15;
            const int head_w = h0 + 64 * (int) rank + (warp & 1) * 32;     // the warp's first head
            const int64_t row_w = (int64_t) t * p.H + head_w;
            const int rows_w = max(0, min(32, p.H - head_w));
            float* dst0 = direct ? p.out + row_w * L : p.part + (row_w * p.ns + split) * PS;
            const int64_t dst_row = direct ? L : (int64_t) p.ns * PS;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                const int fb = (c < 2 ? 0 : 256) + 128 * ch + (c & 1) * 64;     // the features these 64 columns hold
                uint32_t v0[32], v1[32];
                tmem_ld32(tmem + lane_base + (uint32_t) (c * 64), v0);
                tmem_ld32(tmem + lane_base + (uint32_t) (c * 64 + 32), v1);
                tmem_wait_ld();
                float4* trow = reinterpret_cast<float4*>(tile + lane * 68);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    trow[e] = make_float4(__uint_as_float(v0[4 * e]) * inv, __uint_as_float(v0[4 * e + 1]) * inv, __uint_as_float(v0[4 * e + 2]) * inv,
                                          __uint_as_float(v0[4 * e + 3]) * inv);
                    trow[8 + e] = make_float4(__uint_as_float(v1[4 * e]) * inv, __uint_as_float(v1[4 * e + 1]) * inv, __uint_as_float(v1[4 * e + 2]) * inv,
                                              __uint_as_float(v1[4 * e + 3]) * inv);
                }
                __syncwarp();
#pragma unroll
                for (int rr = 0; rr < 32; rr += 2) {
                    const int ri = rr + half;
                    if (ri < rows_w)
                        *reinterpret_cast<float4*>(dst0 + ri * dst_row + fb + l16 * 4) = *reinterpret_cast<const float4*>(tile + ri * 68 + l16 * 4);
                }
                __syncwarp();
            }
            if (head_live && !direct && ch == 0) {
                float* st = p.part + (grow * p.ns + split) * PS + L;
                st[0] = m_ref;
                st[1] = l;
            }
        }
    }
    // ---- teardown: neither CTA leaves while the other may still read its shared memory or signal its barriers
    fence_before_sync();
    __syncthreads();
    cluster_sync();
    if (warp == 5) {
        fence_after_sync();
        tmem_dealloc_pair(tmem, 512);
    }
}

// The splits of each (row, head) merged (a split past the row's cells wrote nothing and is not read): a block takes one
// half of the 512 columns, 8 groups of 64 lanes x 16 bytes; group g takes the splits k = g, g + 8, ... with 10 loads in
// flight a thread, the first of them issued before the weights are known.
constexpr int MERGE_THREADS = 512, MERGE_GROUPS = 8, MERGE_FLIGHT = 10;
__global__ void __launch_bounds__(MERGE_THREADS) mla_merge_kernel(const Params p) {
    __shared__ float w_s[lse::MAX_SPLITS];
    __shared__ float red[32];
    __shared__ float4 acc_s[MERGE_THREADS];
    const int64_t row = blockIdx.x;   // (t, h)
    const int t = (int) (row / p.H);
    const int tid = threadIdx.x, g = tid >> 6, lane = tid & 63;
    pdl_wait();   // the split kernel's partials
    const int64_t n = row_cells(p, t);
    const int64_t kb = p.per_row ? mla_split(n, p.units, p.sms) : p.kb;
    const int nsr = (int) (((uint32_t) n + (uint32_t) kb - 1) / (uint32_t) kb);
    if (nsr <= 1) return;   // the whole block: the row's one split wrote the result itself
    const float* pp = p.part + row * p.ns * PS;
    const float* src = pp + blockIdx.y * DVH + lane * 4;
    float4 v[MERGE_FLIGHT];
#pragma unroll
    for (int u = 0; u < MERGE_FLIGHT; ++u) {
        const int k = g + MERGE_GROUPS * u;
        v[u] = k < nsr ? *reinterpret_cast<const float4*>(src + (size_t) k * PS) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // a thread's own split's (m, l) travel with the first loads; splits past the block's width (rare) are re-read
    float2 ml0 = make_float2(-INFINITY, 0.f);
    if (tid < nsr) ml0 = *reinterpret_cast<const float2*>(pp + (size_t) tid * PS + L);
    float m_loc = ml0.x;
    for (int k = tid + MERGE_THREADS; k < nsr; k += MERGE_THREADS) m_loc = fmaxf(m_loc, pp[(size_t) k * PS + L]);
    float mx = lse::block_max<MERGE_THREADS>(m_loc, red);
    float l_loc = 0.f;
    if (tid < nsr) {
        const float e = (ml0.x == -INFINITY || mx == -INFINITY) ? 0.f : exp2f(ml0.x - mx);
        w_s[tid] = e;
        l_loc = ml0.y * e;
    }
    for (int k = tid + MERGE_THREADS; k < nsr; k += MERGE_THREADS) {
        const float mk = pp[(size_t) k * PS + L];
        const float e = (mk == -INFINITY || mx == -INFINITY) ? 0.f : exp2f(mk - mx);
        w_s[k] = e;
        l_loc += pp[(size_t) k * PS + L + 1] * e;
    }
    float den = lse::block_sum<MERGE_THREADS>(l_loc, red);   // its barriers also publish w_s
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k0 = 0; k0 < nsr; k0 += MERGE_GROUPS * MERGE_FLIGHT) {
        if (k0 > 0) {
#pragma unroll
            for (int u = 0; u < MERGE_FLIGHT; ++u) {
                const int k = k0 + g + MERGE_GROUPS * u;
                v[u] = k < nsr ? *reinterpret_cast<const float4*>(src + (size_t) k * PS) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int u = 0; u < MERGE_FLIGHT; ++u) {
            const int k = k0 + g + MERGE_GROUPS * u;
            const float e = k < nsr ? w_s[k] : 0.f;
            a.x += v[u].x * e, a.y += v[u].y * e, a.z += v[u].z * e, a.w += v[u].w * e;
        }
    }
    acc_s[tid] = a;
    __syncthreads();
    if (g == 0) {
#pragma unroll
        for (int gg = 1; gg < MERGE_GROUPS; ++gg) {
            const float4 o = acc_s[gg * 64 + lane];
            a.x += o.x, a.y += o.y, a.z += o.z, a.w += o.w;
        }
        float f = 1.0f;
        if (p.sinks) {
            const float sk = p.sinks[row % p.H] * 1.4426950408889634f, m2 = fmaxf(mx, sk);
            f = mx == -INFINITY ? 0.f : exp2f(mx - m2);
            den = den * f + exp2f(sk - m2);
        }
        const float inv = den > 0.f ? f / den : 0.f;
        *reinterpret_cast<float4*>(p.out + row * L + blockIdx.y * DVH + lane * 4) = make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
    }
}


// A context split over several GPUs by cell ranges, this rank's side: its splits merged into one partial (O [512], m in log2
// units, l) per (row, head), stored - plain stores over NVLink - into slot `rank` of EVERY rank's mailbox (the GQA
// KV-split's mailbox with rows of 512 + 2 floats); the last block publishes the step in every mailbox's flag for this rank
// after one system fence. A rank that holds none of a row's cells pushes (0, -inf, 0).
__global__ void __launch_bounds__(256) mla_merge_push_kernel(const Params p) {
    __shared__ float sm[lse::smem_floats<L, 256>()];
    pdl_wait();
    const int64_t rh = blockIdx.x;   // (t, h)
    const int t = (int) (rh / p.H);
    const int64_t n = row_cells(p, t);
    const int64_t kb = p.per_row ? mla_split(n, p.units, p.sms) : p.kb;
    const int nsr = n > 0 ? (int) (((uint32_t) n + (uint32_t) kb - 1) / (uint32_t) kb) : 0;
    float mx, den;
    const float2 a = lse::merge_row<L, 256>(p.part + rh * p.ns * PS, PS, nsr < p.ns ? nsr : p.ns, mx, den, sm);
    const int64_t rows = (int64_t) p.T * p.H;
    const long long epoch = p.epoch ? p.epoch : *ns_mbox_epoch(p.mailboxes[p.rank], p.nranks, rows, L) + 1;
    const int buf = (int) (epoch & 1);
    for (int r = 0; r < p.nranks; ++r) {
        float* slot = p.mailboxes[r] + ns_mbox_slot(buf, p.rank, p.nranks, rows, L) + rh * (L + 2);
        *reinterpret_cast<float2*>(slot + 2 * threadIdx.x) = a;
        if (threadIdx.x == 0) *reinterpret_cast<float2*>(slot + L) = make_float2(mx, den);
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* counter = reinterpret_cast<int*>(p.mailboxes[p.rank] + ns_mbox_flags_off(p.nranks, rows, L)) + 4 * p.nranks;
        if (atomicAdd(counter, 1) + 1 == (int) gridDim.x) {
            *counter = 0;
            __threadfence_system();
            for (int r = 0; r < p.nranks; ++r) {
                long long* flag = reinterpret_cast<long long*>(p.mailboxes[r] + ns_mbox_flags_off(p.nranks, rows, L)) + buf * p.nranks + p.rank;
                asm volatile("st.relaxed.sys.global.s64 [%0], %1;\n" ::"l"(flag), "l"(epoch) : "memory");
            }
        }
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_map(CUtensorMap* m, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2, uint32_t box1, const char* where) {
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
    cuuint32_t box[3] = {64, box1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ns_fail(std::string(where) + ": tensor map rejected (code " + std::to_string((int) r) + ")");
    return 0;
}

}  // namespace

// the split size of a pass of T rows whose longest row sees n cells, and the splits its partials are laid out for
static void mla_layout(int64_t n, int64_t T, int64_t H, int sms, int& per_row, int& units, int64_t& kb, int64_t& ns) {
    const int64_t head_tiles = (H + BM - 1) / BM;
    per_row = T <= DECODE_ROWS ? 1 : 0;
    units = (int) (per_row ? head_tiles : head_tiles * T);
    kb = mla_split(n, units, sms);
    if (T == 1) per_row = 0;   // one row: its own size is the pass's size, and the kernel need not work it out
    if (per_row) {
        // every row's own count is at most n: its splits number at most sms / (2 units), and at most n / 128 rounded up
        int64_t want = sms / (2 * units);
        if (want < 1) want = 1;
        ns = std::min<int64_t>(want, (n + 2 * BN - 1) / (2 * BN));
        if (ns < 1) ns = 1;
    } else {
        ns = (n + kb - 1) / kb;
    }
}

// the split form keeps every row's partial, also where a rank's cells make one split
int64_t ns_mla_partial_floats_split(int64_t n, int64_t T, int64_t H, int sms) {
    if (n < 1) return 0;
    int per_row, units;
    int64_t kb, ns;
    mla_layout(n, T, H, sms, per_row, units, kb, ns);
    return T * H * (ns > 1 ? ns : 1) * PS;
}

int64_t ns_mla_partial_floats(int64_t n, int64_t T, int64_t H, int sms) {
    int per_row, units;
    int64_t kb, ns;
    mla_layout(n, T, H, sms, per_row, units, kb, ns);
    return ns > 1 ? T * H * ns * PS : 0;
}

namespace {
template <int CR>
int launch(ns_gpu* g, const MlaDecodeArgs& a, const char* where) {
    const int64_t n = a.n_max;                   // the most cells any row sees
    Params p;
    p.q = (const __half*) a.q;
    p.counts = a.counts;
    p.sinks = a.sinks;
    p.zmul = a.cache_rows_apart > 0 ? 1 : 0;
    p.out = a.out;
    p.part = a.part;
    p.status = g->status_dev;
    p.T = (int) a.T;
    p.H = (int) a.H;
    p.pos0 = a.pos0;
    int64_t ns = 1;
    mla_layout(n > 0 ? n : 1, a.T, a.H, g->sms, p.per_row, p.units, p.kb, ns);
    p.ns = (int) (ns > 1 ? ns : 1);
    p.sms = g->sms;
    if (p.ns > 1 && !a.part) return ns_fail(std::string(where) + ": no scratch for the key splits");
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.cap = a.mailboxes ? n : 0;
    p.mailboxes = a.mailboxes;
    p.rank = a.rank;
    p.nranks = a.nranks;
    p.epoch = a.epoch;
    if (a.mailboxes && ((n > 0 && !a.part) || a.sinks || a.counts || a.cache_rows_apart > 0)) return ns_fail(std::string(where) + ": the split form takes scratch, one shared cache and no sinks");
    if (p.ns > lse::MAX_SPLITS) return ns_fail(std::string(where) + ": more key splits than the merge holds");
    CUtensorMap tq, tc, tv;
    if (n > 0) {
        // Q [T][H][CR]: a box = a CTA's 64 heads x 64 features of one row
        if (make_map(&tq, a.q, CR, (uint64_t) a.H, (uint64_t) a.T, CR * 2, (uint64_t) a.H * CR * 2, 64, where)) return -1;
        // cells [Z][n][CR]: boxes of 64 features x 32 cells (a CTA's half of a tile for S) and x 64 cells (the whole tile, for
        // the CTA's output features); cells past n read as zeros
        const uint64_t z = p.zmul ? (uint64_t) a.T : 1, zs = p.zmul ? (uint64_t) a.cache_rows_apart * 2 : (uint64_t) n * CR * 2;
        if (make_map(&tc, a.cache, CR, (uint64_t) n, z, CR * 2, zs, 32, where)) return -1;
        if (make_map(&tv, a.cache, CR, (uint64_t) n, z, CR * 2, zs, BN, where)) return -1;
    }
    auto kern = mla_decode_pair_kernel<CR>;
    static bool set[64] = {};
    if (!set[g->dev & 63]) {
        NS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairGeo<CR>::SMEM_TOTAL), where);
        set[g->dev & 63] = true;
    }
    dim3 grid((unsigned) (2 * p.ns), (unsigned) ((a.H + BM - 1) / BM), (unsigned) a.T);
    if (n > 0) {
        // the two CTAs of a key split are a cluster: one MMA over both SMs
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = PairGeo<CR>::SMEM_TOTAL;
        cfg.stream = g->compute;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        NS_CUDA(cudaLaunchKernelEx(&cfg, kern, tq, tc, tv, p), where);
    }
    if (a.mailboxes) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned) (a.T * a.H));
        cfg.blockDim = dim3(256);
        cfg.stream = g->compute;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        NS_CUDA(cudaLaunchKernelEx(&cfg, mla_merge_push_kernel, p), where);
        return 0;
    }
    if (p.ns > 1) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned) (a.T * a.H), 2);
        cfg.blockDim = dim3(MERGE_THREADS);
        cfg.stream = g->compute;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        NS_CUDA(cudaLaunchKernelEx(&cfg, mla_merge_kernel, p), where);
    }
    return 0;
}

}  // namespace

int ns_launch_mla_decode(ns_gpu* g, const MlaDecodeArgs& a, const char* where) {
    if (a.rope == 64) return launch<576>(g, a, where);
    if (a.rope == 0) return launch<512>(g, a, where);
    return ns_fail(std::string(where) + ": a rotated part of 64 or none");
}
