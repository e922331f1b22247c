// gqa_decode.cu: split-KV GQA decode for sm_100a - the bandwidth-bound kernel of the path.
//
// What it computes is the SPLIT form of the reference's flash kernel (kernels/llm/qwen35/silo/attn.cpp:105-313 with
// the decode driver :321-370): for 1..8 rows at positions p0+t, out = softmax(q k^T / sqrt(D)) v over the fp16 caches,
// the query scaled by 1/sqrt(D) log2(e) and rounded to fp16, weights exp2 and rounded to fp16 before they meet V,
// fp32 sums, partials (O, m in log2 units, l) per key split merged by attn.cpp:352-368's formula.
//
// How: a CTA takes one (key split, key head, group of <= 32 query rows = rows x the key head's query heads). Its 4
// warps each stream every 4th 16-key tile of the split through a private cp.async pipeline (16-byte, fully coalesced
// loads; 256 B a key row, XOR-swizzled in shared memory), compute S = Q K^T and O += P V on mma.sync m16n8k16 (the
// rows are too few for a tcgen05 tile; the kernel is HBM-bound), keep their own online softmax (quad shuffles for
// the row max and sum) and merge once at the end through shared memory. No block-wide barrier in the key loop.
//
// The same file holds what follows the split kernel: the merge of a row's splits (a programmatic dependent that starts on a
// key head as soon as that head's split CTAs have counted themselves in), and, for one context split over several GPUs by
// key ranges, the exchange of the ranks' partials over NVLink - as a merge-push kernel plus a combine kernel, as a
// merge that leaves the partial for a caller-run all-gather, or (FUSED) as the split kernel's own tail, the whole step
// one launch.
#include "kernels.cuh"
#include "lse_merge.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int KT = 16;   // keys a warp tile

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;   // 0: the 16 bytes are zero-filled, nothing is read
    asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
// 16 rows of 16 bytes, transposed: lane (g, t) gets the bytes of rows 4t .. 4t+3 in column g (r0) and in column g + 8 (r1).
// Lanes 0-15 give the rows' addresses (16-byte aligned).
__device__ __forceinline__ void ldsm_b8_t(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m16n16.x1.trans.shared.b8 {%0, %1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}
// D (fp32 16x8) += A (fp16 16x16, row) x B (fp16 16x8, col)
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// A kernel that follows another on the stream and starts with pdl_wait(): its blocks may be placed on SMs while the
// first kernel drains, and run once that kernel has completed and its writes are visible (programmatic dependent launch).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

struct Params {
    const void* q;
    int64_t qs, q_seq;
    const ns_b200_seq* seqs;
    ns_b200_seq one;
    void* out;
    float* part;
    int T, Hq, Hkv, G, ns_max, groups;
    int q_f32, out_f32;
    float qscale;
    // KV-split over several GPUs: every row's partial is kept (never normalised here) and the merge pushes this
    // rank's (O, m, l) into every rank's mailbox
    int force_part;
    int rank, nranks;
    float* const* mailboxes;   // device array [nranks]: each rank's mailbox as this GPU sees it (peer-mapped)
    long long epoch;
    // completion counters (null: the merge waits for the whole split grid instead): sync[(b, key head)] counts the split
    // kernel's CTAs of that pair that have written their partials, sync[NS_DEC_SYNC_SLOTS + ...] the merge blocks done with them
    unsigned int* sync;
    int* status;
    long long spins;       // fused KV-split step: polls (100 ns apart) a wait on the peers' flags may take; 0: not that step
    float* mailboxes_host_own;   // this rank's own mailbox as the host knows it (the step's fallback launches the combine on it)
    float* local_part;     // [T*Hq][D+2]: the merge keeps the rank's partial here instead of pushing it (no mailboxes)
};

// keys row t of a sequence sees: its causal length, bounded by what the cache slice holds
__device__ __forceinline__ int64_t row_keys(const ns_b200_seq& s, int t) { return min(s.p0 + t + 1, s.cap); }

// byte offset of 16-byte chunk c of row r in a tile whose rows are ROWB bytes: chunks XOR-swizzled by the row
template <int ROWB>
__device__ __forceinline__ uint32_t swz(int r, int c) {
    return (uint32_t) (r * ROWB + ((c ^ (r & 7)) << 4));
}

// ---- quantised caches (heads of 256; kernels/llm/qwen35/silo/attn.cpp:44-78): a head's row is q8_0 - 256 int8 then 8
// fp16 scales, 272 bytes - or q4_0 - 8 blocks of 16 bytes (byte j: value j low nibble, value j + 16 high) then 8 fp16
// scales, 144 bytes. A key's features enter S as the halves the reference's reader produces, half(float(q) * float(d)):
// q becomes an exact half by placing its (biased) byte in the mantissa of 1024 and subtracting the bias, and the half
// product of two halves is the exact product rounded once, as the reference's float product rounded to half is.
template <int QF>
__host__ __device__ constexpr int raw_row_bytes(int D) { return QF == 0 ? D * 2 : QF == 1 ? D + D / 16 : D / 2 + D / 16; }

__device__ __forceinline__ uint32_t scaled_pair(uint32_t biased, uint32_t sel, __half2 bias, __half2 d2) {
    const uint32_t w = __byte_perm(biased, 0x64646464u, sel);   // halves (1024 + b_lo, 1024 + b_hi)
    __half2 h = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&w), bias), d2);
    return *reinterpret_cast<uint32_t*>(&h);
}
// the two halves (b_lo - bias', b_hi - bias') of the bytes `sel` picks: the quantised values themselves, exact
__device__ __forceinline__ uint32_t value_pair(uint32_t biased, uint32_t sel, __half2 bias) {
    const uint32_t w = __byte_perm(biased, 0x64646464u, sel);
    __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&w), bias);
    return *reinterpret_cast<uint32_t*>(&h);
}
// S = Q K^T over a quantised cache takes its key fragments straight from the raw rows: lane (g, t) of a warp reads
// 16-byte chunks of key g's row and expands them in registers, so the keys never pass through an fp16 tile. A 16-byte
// chunk is 16 (q8_0) or 32 (q4_0) consecutive features, not the (2t, 2t+1, 2t+8, 2t+9) a k-step's fragment holds, so the
// contraction index is permuted: k-step ks, fragment pair `half` of lane t stands for the features frag_feature() names,
// and the queries are staged in shared memory in the same order (a sum does not care about the order of its terms).
// Chunk order: lane t takes chunks 2t + (i & 1) + 8 (i >> 1), i = 0..3 (q8_0, row stride 17 chunks) or 2t + i, i = 0..1
// (q4_0, 9 chunks): the eight lanes of a quarter warp then touch eight different 16-byte bank groups.
// O += P V takes the value fragments from the raw rows too, through the transposing 8-bit ldmatrix: lane (g, t) gets the
// bytes of four consecutive keys 4t .. 4t+3 in feature column g, so fragment positions (2t, 2t+1 | 2t+8, 2t+9) of the
// contraction stand for keys (4t, 4t+1 | 4t+2, 4t+3) of the tile, and S is computed with its key columns in that order
// (column n of n-tile nt is key 4 (n / 2) + 2 nt + n % 2). A value's scale depends on its key and its block of 32
// features, so it goes onto the weights: per block, P' = half(P d[key][block]), and the values enter as the exact small
// integers they are. The weights carry a factor (so do the sums, it cancels in O / l) to keep P' out of the fp16
// subnormals without leaving its range: 2^6 for q8_0 (d <= 65504 / 127: P' <= 33,024), 2^2 for q4_0 (d <= 65504 / 8:
// P' <= 32,752).
template <int QF>
__host__ __device__ constexpr int frag_chunk(int t, int i) { return QF == 1 ? 2 * t + (i & 1) + 8 * (i >> 1) : 2 * t + i; }
// first of the two consecutive features in pair `half` (0: fragment k 2t, 2t+1; 1: k 2t+8, 2t+9) of lane t in k-step ks
template <int QF>
__host__ __device__ constexpr int frag_feature(int ks, int t, int half) {
    return QF == 1 ? 16 * frag_chunk<1>(t, ks / 4) + 4 * (ks % 4) + 2 * half
                   : 32 * frag_chunk<2>(t, ks / 8) + 16 * (ks % 2) + 4 * ((ks % 8) / 2) + 2 * half;
}

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* ptr) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.u32 %0, [%1];\n" : "=r"(v) : "l"(ptr) : "memory");
    return v;
}
// A row's split count as the merge may use it: never more than the partial buffer was laid out for. A row that needs
// more (a sequence longer than the max_kv the caller promised) raises status 802 - its keys past the layout were never
// streamed - instead of reading its neighbours' partials.
__device__ __forceinline__ int clamp_splits(const Params& p, int64_t nsr) {
    if (nsr <= p.ns_max) return (int) nsr;
    if (threadIdx.x == 0 && p.status) {
        *(volatile int*) p.status = 802;
        __threadfence_system();
    }
    return p.ns_max;
}
template <int D>
__device__ void fused_split_tail(const Params& p, const ns_b200_seq& seq, int hk, float* sm);

// QF: the caches' form, 0 fp16, 1 q8_0, 2 q4_0. A quantised tile travels as it lies (cp.async of the raw rows into a ring
// of raw stages) and both products take their fragments from the raw rows, expanding them in registers (above). The
// expansion is several hundred dependent instructions a tile and a warp, so these instances are sized for two CTAs an SM
// (two warps a scheduler to hide each other's latencies).
template <int D, int MT, int NSTAGE, int QF, bool FUSED = false>
__global__ void __launch_bounds__(THREADS, QF == 0 ? 1 : 2) gqa_decode_kernel(const Params p) {
    constexpr int RG = 16 * MT;          // query rows a CTA
    constexpr int ROWB = D * 2;          // bytes a key row
    constexpr int CPR = ROWB / 16;       // 16-byte chunks a row
    constexpr int TILE = KT * ROWB;      // bytes a K (or V) tile
    constexpr int NT = D / 8;            // output n-tiles
    constexpr int KS = D / 16;           // k-steps of S = Q K^T
    constexpr int RAWB = raw_row_bytes<QF>(D);      // bytes a key row as the cache holds it
    constexpr int RAW_CPR = RAWB / 16;
    constexpr int RAW_TILE = KT * RAWB;
    constexpr int WARP_BYTES = QF == 0 ? NSTAGE * 2 * TILE : NSTAGE * 2 * RAW_TILE;
    static_assert(QF == 0 || D == 256, "quantised caches have heads of 256: a row's 32 chunks are a warp's lanes");
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int row_flag[8];
    uint8_t* q_s = smem;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint8_t* w_s = smem + RG * ROWB + warp * WARP_BYTES;   // NSTAGE (K, V) tile pairs, fp16 or raw

    // the row groups of one (split, key head) are neighbours in the grid: they run at the same time, and the second
    // to read a key tile finds it in L2
    pdl_launch_dependents();   // the merge kernel's blocks may take SMs as they free up; they wait for this grid to finish
    const int split = blockIdx.x / p.groups, rg = blockIdx.x % p.groups, hk = blockIdx.y;
    const int b = blockIdx.z;
    const ns_b200_seq seq = p.seqs ? p.seqs[b] : p.one;
    const int T = p.T, G = p.G, R = T * G, row0 = rg * RG;
    const int64_t p0 = seq.p0;
    const int t_lo = row0 / G, t_hi = min(T - 1, (row0 + RG - 1) / G);

    // ---- the group's queries, scaled and rounded to fp16, swizzled like the key tiles (rows past R: zeros). Run after the
    // first key and value tiles have been requested (they do not depend on it), so its latency hides under theirs.
    auto stage_q = [&]() {
    for (int i = tid; i < RG * CPR; i += THREADS) {
        const int r = i / CPR, c = i % CPR, rho = row0 + r;
        uint4 w = make_uint4(0, 0, 0, 0);
        if (rho < R) {
            const int t = rho / G, gq = rho % G;
            const int64_t at = (int64_t) b * p.q_seq + (int64_t) t * p.qs + (int64_t) (hk * G + gq) * D + c * 8;
            float f[8];
            if (QF != 0) {
                // column 16 ks + pos of the staged row holds the feature that fragment position stands for
                const int64_t base = at - c * 8;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int d = frag_feature<QF>(c / 2, e, c % 2);
                    if (p.q_f32) {
                        const float2 x = *reinterpret_cast<const float2*>((const float*) p.q + base + d);
                        f[2 * e] = x.x, f[2 * e + 1] = x.y;
                    } else {
                        const float2 x = __half22float2(*reinterpret_cast<const __half2*>((const __half*) p.q + base + d));
                        f[2 * e] = x.x, f[2 * e + 1] = x.y;
                    }
                }
            } else if (p.q_f32) {
                const float4 a = *reinterpret_cast<const float4*>((const float*) p.q + at);
                const float4 bb = *reinterpret_cast<const float4*>((const float*) p.q + at + 4);
                f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = bb.x, f[5] = bb.y, f[6] = bb.z, f[7] = bb.w;
            } else {
                const uint4 a = *reinterpret_cast<const uint4*>((const __half*) p.q + at);
                const __half2* h = reinterpret_cast<const __half2*>(&a);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 x = __half22float2(h[e]);
                    f[2 * e] = x.x, f[2 * e + 1] = x.y;
                }
            }
            w.x = pack_h2(f[0] * p.qscale, f[1] * p.qscale);
            w.y = pack_h2(f[2] * p.qscale, f[3] * p.qscale);
            w.z = pack_h2(f[4] * p.qscale, f[5] * p.qscale);
            w.w = pack_h2(f[6] * p.qscale, f[7] * p.qscale);
        }
        *reinterpret_cast<uint4*>(q_s + swz<ROWB>(r, c)) = w;
    }
    };
    bool q_staged = false;

    // rows of one pass share a split size; where the rows' own sizes differ (a row's context crosses a step of the
    // split function) the rows go one at a time, each with its own - the same arithmetic either way
    bool same = true;
    for (int t = t_lo; t <= t_hi; ++t) same = same && ns_dec_split(row_keys(seq, t), p.Hkv) == ns_dec_split(row_keys(seq, t_lo), p.Hkv);
    const int npass = same ? 1 : t_hi - t_lo + 1;

    const uint8_t* kbase = (const uint8_t*) seq.kc + (int64_t) hk * seq.cap * RAWB;
    const uint8_t* vbase = (const uint8_t*) seq.vc + (int64_t) hk * seq.cap * RAWB;

    for (int pass = 0; pass < npass; ++pass) {
        const int t_a = same ? t_lo : t_lo + pass, t_b = same ? t_hi : t_a;
        const int64_t kb = ns_dec_split(row_keys(seq, t_a), p.Hkv);
        const int64_t kv_end = row_keys(seq, t_b);
        const int64_t jbeg = (int64_t) split * kb, jend = min(kv_end, (int64_t) (split + 1) * kb);
        if (jbeg >= jend) continue;   // the whole CTA
        const int ntiles = (int) ((jend - jbeg + KT - 1) / KT);

        // this thread's rows: (mt, lane/4) and 8 below; a row outside the pass sees no key
        int lim_rel[MT][2];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int rho = row0 + mt * 16 + hh * 8 + (lane >> 2), t = rho / G;
                const int64_t last = (rho < R && t >= t_a && t <= t_b) ? min(p0 + t, jend - 1) : jbeg - 1;
                lim_rel[mt][hh] = (int) max(last - jbeg, (int64_t) -1);
            }

        float o[MT][NT][4];
        float m[MT][2], l[MT][2];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) o[mt][nt][e] = 0.f;
            m[mt][0] = m[mt][1] = -INFINITY;
            l[mt][0] = l[mt][1] = 0.f;
        }

        // a tile's loads: 16 keys x ROWB bytes of K and of V, 16 bytes a lane a step (two whole rows a warp step)
        auto issue = [&](int tile, int stage) {
            if (tile < ntiles) {
                const int64_t j0 = jbeg + (int64_t) tile * KT;
                if (QF == 0) {
                    uint8_t* ks = w_s + stage * (2 * TILE);
                    uint8_t* vs = ks + TILE;
#pragma unroll
                    for (int i = 0; i < KT * CPR / 32; ++i) {
                        const int idx = i * 32 + lane, r = idx / CPR, c = idx % CPR;
                        const bool ok = j0 + r < jend;
                        const int64_t off = ok ? (j0 + r) * ROWB + c * 16 : 0;
                        cp_async16(smem_u32(ks + swz<ROWB>(r, c)), kbase + off, ok);
                        cp_async16(smem_u32(vs + swz<ROWB>(r, c)), vbase + off, ok);
                    }
                } else {
                    // a tile's raw rows are one run of KT * RAWB bytes in the cache and in the stage alike
                    uint8_t* kr = w_s + stage * (2 * RAW_TILE);
                    uint8_t* vr = kr + RAW_TILE;
                    const int64_t at = j0 * RAWB;
                    const int valid = (int) min((int64_t) RAW_TILE, (jend - j0) * RAWB);   // rows past the split: zeros (scale 0)
#pragma unroll
                    for (int i = 0; i < (KT * RAW_CPR + 31) / 32; ++i) {
                        const int off = (i * 32 + lane) * 16;
                        if (off < RAW_TILE) {
                            const bool ok = off < valid;
                            cp_async16(smem_u32(kr + off), kbase + at + (ok ? off : 0), ok);
                            cp_async16(smem_u32(vr + off), vbase + at + (ok ? off : 0), ok);
                        }
                    }
                }
            }
            cp_async_commit();
        };

#pragma unroll
        for (int s = 0; s < NSTAGE - 1; ++s) issue(warp + s * WARPS, s);
        if (!q_staged) {   // once, by the CTA's first pass that has keys (the condition is the same for all its threads)
            stage_q();
            __syncthreads();
            q_staged = true;
        }

        int stage = 0;
        for (int tile = warp; tile < ntiles; tile += WARPS) {
            {
                int ps = stage + NSTAGE - 1;
                if (ps >= NSTAGE) ps -= NSTAGE;
                issue(tile + (NSTAGE - 1) * WARPS, ps);
            }
            cp_async_wait<NSTAGE - 1>();
            __syncwarp();
            const uint8_t* ks = QF == 0 ? w_s + stage * (2 * TILE) : w_s;
            const uint8_t* vs = QF == 0 ? ks + TILE : w_s;
            const int64_t j0 = jbeg + (int64_t) tile * KT;

            // ---- S = Q K^T: MT x (16 rows x 16 keys)
            float s[MT][2][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[mt][nt][e] = 0.f;
            if (QF == 0) {
#pragma unroll
                for (int k = 0; k < KS; ++k) {
                    uint32_t kf[4];
                    ldsm_x4(smem_u32(ks + swz<ROWB>((lane & 7) + (lane >> 4) * 8, 2 * k + ((lane >> 3) & 1))), kf);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        uint32_t qf[4];
                        ldsm_x4(smem_u32(q_s + swz<ROWB>(mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * k + (lane >> 4))), qf);
                        mma16816(s[mt][0], qf, kf[0], kf[1]);
                        mma16816(s[mt][1], qf, kf[2], kf[3]);
                    }
                }
            } else {
                // key fragments from the raw rows (see frag_feature): keys g and g + 8 of the tile, this lane's chunks
                const uint8_t* kr = w_s + stage * (2 * RAW_TILE);
                const int g = lane >> 2, t = lane & 3;
                const uint8_t* row0p = kr + (4 * (g >> 1) + (g & 1)) * RAWB;   // n-tile 0: key 4 (g / 2) + g % 2
                const uint8_t* row1p = row0p + 2 * RAWB;                        // n-tile 1: two keys on
                constexpr int NI = QF == 1 ? 4 : 2;           // chunks a lane reads of a row
                constexpr int KPC = KS / NI;                   // k-steps a chunk feeds
                const __half2 bias = QF == 1 ? __floats2half2_rn(1152.f, 1152.f) : __floats2half2_rn(1032.f, 1032.f);
                // the blocks' scales: q8_0 chunks 2t + (i & 1) + 8 (i >> 1) lie in blocks t and t + 4, q4_0 chunk = block
                __half2 d0[2], d1[2];
                if (QF == 1) {
                    d0[0] = __half2half2(*reinterpret_cast<const __half*>(row0p + 256 + 2 * t));
                    d0[1] = __half2half2(*reinterpret_cast<const __half*>(row0p + 256 + 2 * (t + 4)));
                    d1[0] = __half2half2(*reinterpret_cast<const __half*>(row1p + 256 + 2 * t));
                    d1[1] = __half2half2(*reinterpret_cast<const __half*>(row1p + 256 + 2 * (t + 4)));
                } else {
                    const __half2 a = *reinterpret_cast<const __half2*>(row0p + 128 + 4 * t);
                    const __half2 c = *reinterpret_cast<const __half2*>(row1p + 128 + 4 * t);
                    d0[0] = __half2half2(__low2half(a)), d0[1] = __half2half2(__high2half(a));
                    d1[0] = __half2half2(__low2half(c)), d1[1] = __half2half2(__high2half(c));
                }
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    const int ch = frag_chunk<QF>(t, i);
                    const uint4 c0 = *reinterpret_cast<const uint4*>(row0p + 16 * ch);
                    const uint4 c1 = *reinterpret_cast<const uint4*>(row1p + 16 * ch);
                    const uint32_t w0[4] = {c0.x, c0.y, c0.z, c0.w}, w1[4] = {c1.x, c1.y, c1.z, c1.w};
                    const __half2 s0 = QF == 1 ? d0[i >> 1] : d0[i], s1 = QF == 1 ? d1[i >> 1] : d1[i];
#pragma unroll
                    for (int kk = 0; kk < KPC; ++kk) {
                        const int k = i * KPC + kk;
                        uint32_t x0, x1;
                        if (QF == 1) {
                            x0 = w0[kk] ^ 0x80808080u, x1 = w1[kk] ^ 0x80808080u;
                        } else {
                            const int sh = (kk & 1) * 4;   // k-steps in turn: the low nibbles (values j), the high ones (j + 16)
                            x0 = (w0[kk >> 1] >> sh) & 0x0F0F0F0Fu, x1 = (w1[kk >> 1] >> sh) & 0x0F0F0F0Fu;
                        }
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            uint32_t qf[4];
                            ldsm_x4(smem_u32(q_s + swz<ROWB>(mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * k + (lane >> 4))), qf);
                            mma16816(s[mt][0], qf, scaled_pair(x0, 0x4140, bias, s0), scaled_pair(x0, 0x4342, bias, s0));
                            mma16816(s[mt][1], qf, scaled_pair(x1, 0x4140, bias, s1), scaled_pair(x1, 0x4342, bias, s1));
                        }
                    }
                }
            }
            // ---- mask, online softmax (a row's 16 scores sit in its quad: 4 a lane)
            uint32_t pf[MT][4];
            float cs[MT][2];
            bool moved = false;
            const int rel0 = (int) (j0 - jbeg);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int last = lim_rel[mt][hh];   // the row's last visible key, relative to the split's first
                    float x[4];
                    float mx = -INFINITY;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int nt = e >> 1;
                        const int key = QF == 0 ? rel0 + nt * 8 + 2 * (lane & 3) + (e & 1) : rel0 + 4 * (lane & 3) + 2 * nt + (e & 1);
                        x[e] = key <= last ? s[mt][nt][hh * 2 + (e & 1)] : -INFINITY;
                        mx = fmaxf(mx, x[e]);
                    }
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                    const float mo = m[mt][hh], mn = fmaxf(mo, mx);
                    const float ref = mn == -INFINITY ? 0.f : mn;   // nothing seen yet: every weight below is 2^-inf = 0
                    const float c = mo == mn ? 1.0f : ex2_approx(mo - ref);
                    float pv[4], sum = 0.f;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        // quantised values: weights and sums times 2^6 (q8_0) or 2^2 (q4_0), see frag_feature
                        pv[e] = ex2_approx(x[e] - (QF == 0 ? ref : QF == 1 ? ref - 6.0f : ref - 2.0f));
                        sum += pv[e];
                    }
                    l[mt][hh] = l[mt][hh] * c + sum;   // this lane's share; the quad's shares are added at the end
                    m[mt][hh] = mn;
                    pf[mt][hh] = pack_h2(pv[0], pv[1]);       // keys 0..7 of the tile -> A fragment k 0..7
                    pf[mt][2 + hh] = pack_h2(pv[2], pv[3]);   // keys 8..15 -> k 8..15
                    cs[mt][hh] = c;
                    moved = moved || c != 1.0f;
                }
            }
            // the running maxima settle after a few tiles: O is rescaled only when some row's maximum moved
            if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            o[mt][nt][hh * 2] *= cs[mt][hh];
                            o[mt][nt][hh * 2 + 1] *= cs[mt][hh];
                        }
            }
            // ---- O += P V
            if (QF == 0) {
#pragma unroll
                for (int jj = 0; jj < NT / 2; ++jj) {
                    uint32_t vf[4];
                    ldsm_x4_t(smem_u32(vs + swz<ROWB>((lane & 7) + ((lane >> 3) & 1) * 8, 2 * jj + (lane >> 4))), vf);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        mma16816(o[mt][2 * jj], pf[mt], vf[0], vf[1]);
                        mma16816(o[mt][2 * jj + 1], pf[mt], vf[2], vf[3]);
                    }
                }
            } else {
                const uint8_t* vr = w_s + stage * (2 * RAW_TILE) + RAW_TILE;
                const int t = lane & 3;
                constexpr int SC_OFF = QF == 1 ? 256 : 128;   // the 8 fp16 scales behind the values
                const __half2 bias = QF == 1 ? __floats2half2_rn(1152.f, 1152.f) : __floats2half2_rn(1032.f, 1032.f);
                uint4 sk[4];   // the scales of this lane's keys 4t .. 4t+3
#pragma unroll
                for (int q = 0; q < 4; ++q) sk[q] = *reinterpret_cast<const uint4*>(vr + (4 * t + q) * RAWB + SC_OFF);
                const uint32_t ld_addr = smem_u32(vr + (lane & 15) * RAWB);
#pragma unroll
                for (int blk = 0; blk < 8; ++blk) {
                    const uint32_t sel = (blk & 1) ? 0x7632u : 0x5410u;
                    const uint32_t w0 = (&sk[0].x)[blk >> 1], w1 = (&sk[1].x)[blk >> 1], w2 = (&sk[2].x)[blk >> 1], w3 = (&sk[3].x)[blk >> 1];
                    const uint32_t s01 = __byte_perm(w0, w1, sel), s23 = __byte_perm(w2, w3, sel);   // (d[4t], d[4t+1]), (d[4t+2], d[4t+3])
                    uint32_t pa[MT][4];
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __half2 h = __hmul2(*reinterpret_cast<const __half2*>(&pf[mt][e]), *reinterpret_cast<const __half2*>(e < 2 ? &s01 : &s23));
                            pa[mt][e] = *reinterpret_cast<const uint32_t*>(&h);
                        }
                    if (QF == 1) {
#pragma unroll
                        for (int c2 = 0; c2 < 2; ++c2) {
                            const int ch = 2 * blk + c2;   // 16 features: n-tiles 2 ch and 2 ch + 1
                            uint32_t r0, r1;
                            ldsm_b8_t(ld_addr + 16 * ch, r0, r1);
                            const uint32_t x0 = r0 ^ 0x80808080u, x1 = r1 ^ 0x80808080u;
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt) {
                                mma16816(o[mt][2 * ch], pa[mt], value_pair(x0, 0x4140, bias), value_pair(x0, 0x4342, bias));
                                mma16816(o[mt][2 * ch + 1], pa[mt], value_pair(x1, 0x4140, bias), value_pair(x1, 0x4342, bias));
                            }
                        }
                    } else {
                        // a block's 16 bytes: byte j holds value j (low nibble) and value j + 16 (high)
                        uint32_t r0, r1;
                        ldsm_b8_t(ld_addr + 16 * blk, r0, r1);
                        const uint32_t x[4] = {r0 & 0x0F0F0F0Fu, r1 & 0x0F0F0F0Fu, (r0 >> 4) & 0x0F0F0F0Fu, (r1 >> 4) & 0x0F0F0F0Fu};
#pragma unroll
                        for (int q = 0; q < 4; ++q)
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt)
                                mma16816(o[mt][4 * blk + q], pa[mt], value_pair(x[q], 0x4140, bias), value_pair(x[q], 0x4342, bias));
                    }
                }
            }
            __syncwarp();
            if (++stage == NSTAGE) stage = 0;
        }
        cp_async_wait<0>();
        __syncthreads();   // every warp's tiles are consumed: the stage memory becomes the merge buffer

        // ---- the 4 warps' (m, l, O) merged: [WARPS][RG] m, l and [WARPS][RG][D] O over the stage memory
        float* ms = reinterpret_cast<float*>(smem + RG * ROWB);
        float* ls = ms + WARPS * RG;
        float* os = ls + WARPS * RG;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                float lt = l[mt][hh];
                lt += __shfl_xor_sync(0xffffffffu, lt, 1);
                lt += __shfl_xor_sync(0xffffffffu, lt, 2);
                const int r = mt * 16 + hh * 8 + (lane >> 2);
                if ((lane & 3) == 0) {
                    ms[warp * RG + r] = m[mt][hh];
                    ls[warp * RG + r] = lt;
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    *reinterpret_cast<float2*>(os + ((size_t) (warp * RG + r)) * D + nt * 8 + 2 * (lane & 3)) =
                        make_float2(o[mt][nt][hh * 2], o[mt][nt][hh * 2 + 1]);
            }
        // per row of the pass (at most 8): does this split hold any of its keys, and is it the row's only split - worked
        // out once by one thread each (64-bit divisions are long instruction sequences), not per output element
        if (tid < 8) {
            const int t = t_a + tid;
            int f = 0;
            if (t <= t_b) {
                const int64_t kv = row_keys(seq, t);
                if (jbeg < kv) f = (ns_dec_splits(kv, p.Hkv) == 1 && !p.force_part) ? 2 : 1;
            }
            row_flag[tid] = f;   // 0: not one of the row's splits, 1: partial, 2: the row's output
        }
        __syncthreads();
        for (int r = warp; r < RG; r += WARPS) {   // a warp a row: 32 lanes x D/32 features
            const int rho = row0 + r;
            if (rho >= R) break;
            const int t = rho / G, gq = rho - t * G;
            if (t < t_a || t > t_b) continue;
            const int flag = row_flag[t - t_a];
            if (flag == 0) continue;
            float mx = -INFINITY;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) mx = fmaxf(mx, ms[w * RG + r]);
            float e[WARPS], L = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float mw = ms[w * RG + r];
                e[w] = (mw == -INFINITY || mx == -INFINITY) ? 0.f : ex2_approx(mw - mx);
                L += ls[w * RG + r] * e[w];
            }
            const int hq = hk * G + gq;
            const int64_t row = ((int64_t) b * T + t) * p.Hq + hq;
            const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
            for (int k = 0; k < D / 32; ++k) {
                const int d = k * 32 + lane;
                float A = 0.f;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) A += os[((size_t) (w * RG + r)) * D + d] * e[w];
                if (flag == 2) {
                    if (p.out_f32) ((float*) p.out)[row * D + d] = A * inv;
                    else ((__half*) p.out)[row * D + d] = __float2half_rn(A * inv);
                } else {
                    p.part[(row * p.ns_max + split) * (D + 2) + d] = A;
                }
            }
            if (flag == 1 && lane == 0) {
                float* pr = p.part + (row * p.ns_max + split) * (D + 2);
                pr[D] = mx;
                pr[D + 1] = L;
            }
        }
        __syncthreads();   // the merge buffer is stage memory again for the next pass
    }
    if (FUSED) {
        fused_split_tail<D>(p, seq, hk, reinterpret_cast<float*>(smem));   // the stage memory is free: the merge's scratch
        return;
    }
    if (p.sync) {
        // this CTA's partials are written: one more of its (sequence, key head)'s splits is ready for the merge
        __threadfence();
        __syncthreads();
        if (tid == 0) atomicAdd(p.sync + (b * p.Hkv + hk), 1u);
    }
}

// The KV-split step in ONE kernel (every CTA of the grid resident: a cooperative launch). After its own split's partials
// are out a CTA counts itself in on its key head. The head's (row, head) pairs are dealt over the head's CTAs; a CTA
// that holds pairs waits (bounded, code 801) until the head's count is full, merges each of its pairs' splits
// (attn.cpp:352-368) and stores the pair's (O, m, l) into slot `rank` of EVERY rank's mailbox over NVLink as 16-byte lines
// (value, step tag, value, step tag): a line arrives whole, so the tag is the value's own flag - no fence, no counter, no
// flag round trip. The same CTAs then read their pairs' lines of every rank from their OWN mailbox, polling (bounded, code
// 701) until the tags show this step, merge across the ranks and write the rows. The last of them returns the counters
// to zero and, when the step numbers live on the device (epoch 0), advances the mailbox's. One launch, no gaps.
__device__ __forceinline__ void st_line(uint4* dst, float x, float y, uint32_t tag) {
    asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};\n" ::"l"(dst), "r"(__float_as_uint(x)), "r"(tag), "r"(__float_as_uint(y)), "r"(tag) : "memory");
}
// polls a line until both halves carry `tag`; false when `spins` polls run out
__device__ __forceinline__ bool ld_line(const uint4* src, uint32_t tag, long long spins, float& x, float& y) {
    uint4 v;
    for (long long it = 0;; ++it) {
        asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
        if (v.y == tag && v.w == tag) break;
        if (it > spins) return false;
        __nanosleep(100);
    }
    x = __uint_as_float(v.x), y = __uint_as_float(v.z);
    return true;
}

template <int D>
__device__ void fused_split_tail(const Params& p, const ns_b200_seq& seq, int hk, float* sm) {
    constexpr int LPR = D / 2 + 1;   // lines a row: D values two a line, then (m, l)
    __shared__ int ready_s;
    __shared__ float2 ml_s[64];      // the ranks' (m, l) of the pair being combined
    const int tid = threadIdx.x;
    const int ctas_head = (int) gridDim.x, R = p.T * p.G;
    const int64_t rows = (int64_t) p.T * p.Hq;
    float* own = p.mailboxes[p.rank];
    int* counters = reinterpret_cast<int*>(own + ns_mbox_flags_off(p.nranks, rows, D)) + 4 * p.nranks;   // [1]: pairs combined
    unsigned int* head_cnt = p.sync + hk;
    __threadfence();
    __syncthreads();
    if (tid == 0) atomicAdd(head_cnt, 1u);
    int mine = 0;
    for (int pr = (int) blockIdx.x; pr < R; pr += ctas_head) ++mine;
    if (mine == 0) return;

    long long* epoch_slot = ns_mbox_epoch(own, p.nranks, rows, D);
    const long long epoch = p.epoch ? p.epoch : *epoch_slot + 1;
    const int buf = (int) (epoch & 1);
    const uint32_t tag = (uint32_t) epoch;   // a mailbox starts zeroed and epochs count from 1: a line never written never matches
    if (tid == 0) {
        int ok = 1;
        unsigned int i = 0;
        while (ld_acquire_gpu(head_cnt) < (unsigned int) ctas_head) {
            if (++i > (1u << 21)) {
                ok = 0;
                if (p.status) {
                    *(volatile int*) p.status = 801;
                    __threadfence_system();
                }
                break;
            }
            __nanosleep(100);
        }
        ready_s = ok;
    }
    __syncthreads();
    if (!ready_s) return;   // the peers' combines give up in their turn (code 701)

    // ---- this CTA's pairs: the splits merged, the result into every rank's mailbox
    const int64_t ll_off = ns_mbox_ll_off_bytes(p.nranks, rows, D);
    for (int pr = (int) blockIdx.x; pr < R; pr += ctas_head) {
        const int t = pr / p.G, gq = pr - t * p.G;
        const int64_t rh = (int64_t) t * p.Hq + hk * p.G + gq;
        const int64_t kv = row_keys(seq, t);
        const int nsr = kv > 0 ? clamp_splits(p, ns_dec_splits(kv, p.Hkv)) : 0;
        float mx, L;
        const float2 a = lse::merge_row<D, THREADS>(p.part + rh * p.ns_max * (D + 2), D + 2, nsr, mx, L, sm);
        const int64_t line0 = ns_mbox_ll_line(buf, p.rank, p.nranks, rows, D) + rh * LPR;
        for (int r = 0; r < p.nranks; ++r) {
            uint4* lines = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.mailboxes[r]) + ll_off) + line0;
            if (tid < D / 2) st_line(lines + tid, a.x, a.y, tag);
            if (tid == THREADS - 1) st_line(lines + D / 2, mx, L, tag);
        }
        __syncthreads();   // the merge's scratch is reused by the next pair
    }

    // ---- the pairs again, now across the ranks: every rank's lines for this step, from this rank's own memory
    bool ok = true;
    const uint4* mine_ll = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(own) + ll_off);
    for (int pr = (int) blockIdx.x; pr < R; pr += ctas_head) {
        const int t = pr / p.G, gq = pr - t * p.G;
        const int64_t rh = (int64_t) t * p.Hq + hk * p.G + gq;
        if (tid < p.nranks) {
            float m, l;
            if (ld_line(mine_ll + ns_mbox_ll_line(buf, tid, p.nranks, rows, D) + rh * LPR + D / 2, tag, p.spins, m, l)) ml_s[tid] = make_float2(m, l);
            else ok = false, ml_s[tid] = make_float2(-INFINITY, 0.f);
        }
        __syncthreads();
        float mx = -INFINITY;
        for (int r = 0; r < p.nranks; ++r) mx = fmaxf(mx, ml_s[r].x);
        for (int c = tid; c < D / 2; c += THREADS) {
            float L = 0.f, ax = 0.f, ay = 0.f;
            for (int r = 0; r < p.nranks; ++r) {
                float x, y;
                if (!ld_line(mine_ll + ns_mbox_ll_line(buf, r, p.nranks, rows, D) + rh * LPR + c, tag, p.spins, x, y)) {
                    ok = false;
                    break;
                }
                const float mk = ml_s[r].x;
                const float e = (mk == -INFINITY || mx == -INFINITY) ? 0.f : exp2f(mk - mx);
                L += ml_s[r].y * e;
                ax += x * e, ay += y * e;
            }
            if (ok) {
                const float inv = L > 0.f ? 1.0f / L : 0.f;
                if (p.out_f32) *reinterpret_cast<float2*>((float*) p.out + rh * D + 2 * c) = make_float2(ax * inv, ay * inv);
                else *reinterpret_cast<__half2*>((__half*) p.out + rh * D + 2 * c) = __floats2half2_rn(ax * inv, ay * inv);
            }
        }
        __syncthreads();   // ml_s is reused by the next pair
    }
    if (!ok && p.status) {
        *(volatile int*) p.status = 701;
        __threadfence_system();
    }
    const int all_ok = __syncthreads_and(ok ? 1 : 0);
    if (tid == 0) {
        if (atomicAdd(counters + 1, mine) + mine == (int) rows) {
            // the step's last CTA: every count it returns to zero has been read by all who wait on it
            for (int h = 0; h < p.Hkv; ++h) p.sync[h] = 0u;
            counters[1] = 0;
            if (p.epoch == 0 && all_ok) *epoch_slot = epoch;
            __threadfence();
        }
    }
}

// A merge block's way in and out when the split kernel counts its CTAs. In: wait (bounded) until every split CTA of the
// block's (sequence, key head) has written - the block was placed while the split kernel's last CTAs still ran, so pairs
// that finished early are merged under that tail. Out: the last merge block of the pair returns both counters to zero.
constexpr unsigned int MERGE_WAIT_LIMIT = 1u << 21;
__device__ __forceinline__ void merge_enter(const Params& p, int b, int hk) {
    if (threadIdx.x == 0) {
        const unsigned int expect = (unsigned int) (p.ns_max * p.groups);
        const unsigned int* c = p.sync + (b * p.Hkv + hk);
        unsigned int i = 0;
        while (ld_acquire_gpu(c) < expect) {
            if (++i > MERGE_WAIT_LIMIT) {
                if (p.status) {
                    *(volatile int*) p.status = 801;
                    __threadfence_system();
                }
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
}
__device__ __forceinline__ void merge_leave(const Params& p, int b, int hk) {
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned int* done = p.sync + NS_DEC_SYNC_SLOTS + (b * p.Hkv + hk);
        if (atomicAdd(done, 1u) + 1u == (unsigned int) (p.T * p.G)) {
            p.sync[b * p.Hkv + hk] = 0u;
            *done = 0u;
            __threadfence();
        }
    }
}

// the splits of each (sequence, row, head) merged: attn.cpp:352-368's formula; rows with one split were written by
// the first kernel
constexpr int MERGE_THREADS = 256;

template <int D>
__global__ void __launch_bounds__(MERGE_THREADS) gqa_merge_kernel(const Params p) {
    __shared__ float sm[lse::smem_floats<D, MERGE_THREADS>()];
    const int64_t rh = blockIdx.x;   // (b, t, hq)
    const int t = (int) ((rh / p.Hq) % p.T), b = (int) (rh / ((int64_t) p.Hq * p.T));
    const int hk = (int) (rh % p.Hq) / p.G;
    if (p.sync) merge_enter(p, b, hk);
    else pdl_wait();   // the split kernel's partials
    const ns_b200_seq seq = p.seqs ? p.seqs[b] : p.one;
    const int nsr = clamp_splits(p, ns_dec_splits(row_keys(seq, t), p.Hkv));
    if (nsr == 1) {
        if (p.sync) merge_leave(p, b, hk);
        return;
    }
    float mx, L;
    const float2 a = lse::merge_row<D, MERGE_THREADS>(p.part + rh * p.ns_max * (D + 2), D + 2, nsr, mx, L, sm);
    if (threadIdx.x < D / 2) {
        const float inv = L > 0.f ? 1.0f / L : 0.f;
        const int d = 2 * threadIdx.x;
        if (p.out_f32) *reinterpret_cast<float2*>((float*) p.out + rh * D + d) = make_float2(a.x * inv, a.y * inv);
        else *reinterpret_cast<__half2*>((__half*) p.out + rh * D + d) = __floats2half2_rn(a.x * inv, a.y * inv);
    }
    if (p.sync) merge_leave(p, b, hk);
}

// KV split over several GPUs, this rank's side: its key splits merged into one partial (O, m, l) per (row, head), which
// is stored - with plain stores over NVLink - into slot `rank` of EVERY rank's mailbox; the last block to finish
// publishes the epoch in every mailbox's flag for this rank (release at system scope). One sequence.
template <int D>
__global__ void __launch_bounds__(MERGE_THREADS) gqa_merge_push_kernel(const Params p) {
    __shared__ float sm[lse::smem_floats<D, MERGE_THREADS>()];
    pdl_wait();   // the split kernel's partials
    const int64_t rh = blockIdx.x;   // (t, hq)
    const int t = (int) (rh / p.Hq);
    const ns_b200_seq seq = p.seqs ? p.seqs[0] : p.one;
    const int64_t kv = row_keys(seq, t);
    const int nsr = kv > 0 ? clamp_splits(p, ns_dec_splits(kv, p.Hkv)) : 0;
    float mx, L;
    const float2 a = lse::merge_row<D, MERGE_THREADS>(p.part + rh * p.ns_max * (D + 2), D + 2, nsr, mx, L, sm);
    const int64_t rows = (int64_t) p.T * p.Hq;
    if (p.local_part) {
        // no mailboxes: the rank's partial stays here, for an exchange the caller runs itself (a library all-gather)
        if (threadIdx.x < D / 2) {
            float* slot = p.local_part + rh * (D + 2);
            *reinterpret_cast<float2*>(slot + 2 * threadIdx.x) = a;
            if (threadIdx.x == 0) *reinterpret_cast<float2*>(slot + D) = make_float2(mx, L);
        }
        return;
    }
    // epoch 0: the step number lives in this rank's own mailbox (the combine advances it), so a recorded graph of the
    // step can be replayed
    const long long epoch = p.epoch ? p.epoch : *ns_mbox_epoch(p.mailboxes[p.rank], p.nranks, rows, D) + 1;
    const int buf = (int) (epoch & 1);
    if (threadIdx.x < D / 2) {
        for (int r = 0; r < p.nranks; ++r) {
            float* slot = p.mailboxes[r] + ns_mbox_slot(buf, p.rank, p.nranks, rows, D) + rh * (D + 2);
            *reinterpret_cast<float2*>(slot + 2 * threadIdx.x) = a;
            if (threadIdx.x == 0) *reinterpret_cast<float2*>(slot + D) = make_float2(mx, L);
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        // the counter lives in this rank's own mailbox and returns to zero for the next call
        int* counter = reinterpret_cast<int*>(p.mailboxes[p.rank] + ns_mbox_flags_off(p.nranks, rows, D)) + 4 * p.nranks;
        const int done = atomicAdd(counter, 1) + 1;
        if (done == (int) gridDim.x) {
            *counter = 0;
            __threadfence_system();
            for (int r = 0; r < p.nranks; ++r) {
                long long* flag = reinterpret_cast<long long*>(p.mailboxes[r] + ns_mbox_flags_off(p.nranks, rows, D)) + buf * p.nranks + p.rank;
                // the fence above is the release; a release on each of these stores would wait out an NVLink round trip
                // per rank, one after the other
                asm volatile("st.relaxed.sys.global.s64 [%0], %1;\n" ::"l"(flag), "l"(epoch) : "memory");
            }
        }
    }
}

struct CombineParams {
    float* mailbox;         // this rank's own mailbox (local memory)
    void* out;              // [T][Hq*D] fp16 or fp32
    int* status;
    int nranks, D, out_f32;
    long long rows, epoch, spins;
};

// The other side: waits - with a bounded poll of LOCAL memory - until every rank's flag shows this epoch, then merges
// the ranks' partials (attn.cpp:352-368's formula across ranks). A wait that runs out writes status code 701 and the
// block leaves without touching the output.
template <int D>
__global__ void __launch_bounds__(D) gqa_combine_kernel(const CombineParams c) {
    __shared__ int ready;
    const int64_t rh = blockIdx.x;
    const int d = threadIdx.x;
    long long* epoch_slot = ns_mbox_epoch(c.mailbox, c.nranks, c.rows, D);
    const long long epoch = c.epoch ? c.epoch : *epoch_slot + 1;
    const int buf = (int) (epoch & 1);
    if (d == 0) {
        const long long* flags = reinterpret_cast<const long long*>(c.mailbox + ns_mbox_flags_off(c.nranks, c.rows, D)) + buf * c.nranks;
        int ok = 1;
        for (int r = 0; r < c.nranks && ok; ++r) {
            long long v = 0, it = 0;
            for (;;) {
                asm volatile("ld.acquire.sys.global.s64 %0, [%1];\n" : "=l"(v) : "l"(flags + r) : "memory");
                if (v >= epoch) break;
                if (++it > c.spins) {
                    ok = 0;
                    break;
                }
                __nanosleep(100);
            }
        }
        if (!ok && c.status) {
            *(volatile int*) c.status = 701;
            __threadfence_system();
        }
        ready = ok;
    }
    __syncthreads();
    if (c.epoch == 0) {
        // the last block to have read the step number advances it (every block read it before arriving here)
        if (d == 0) {
            int* counter = reinterpret_cast<int*>(c.mailbox + ns_mbox_flags_off(c.nranks, c.rows, D)) + 4 * c.nranks + 1;
            if (atomicAdd(counter, 1) + 1 == (int) gridDim.x) {
                *counter = 0;
                if (ready) *epoch_slot = epoch;
                __threadfence();
            }
        }
    }
    if (!ready) return;
    const float* base = c.mailbox + ns_mbox_slot(buf, 0, c.nranks, c.rows, D) + rh * (D + 2);
    const int64_t stride = c.rows * (D + 2);
    float mx = -INFINITY;
    for (int r = 0; r < c.nranks; ++r) mx = fmaxf(mx, base[r * stride + D]);
    float L = 0.f, A = 0.f;
    if (mx != -INFINITY) {
        for (int r = 0; r < c.nranks; ++r) {
            const float mk = base[r * stride + D];
            const float e = mk == -INFINITY ? 0.f : exp2f(mk - mx);
            L += base[r * stride + D + 1] * e;
            A += base[r * stride + d] * e;
        }
    }
    const float v = L > 0.f ? A / L : 0.f;
    if (c.out_f32) ((float*) c.out)[rh * D + d] = v;
    else ((__half*) c.out)[rh * D + d] = __float2half_rn(v);
}

// The ranks' partials side by side in this GPU's memory ([nranks][rows][D+2], however they got there) merged into the rows:
// the combine without mailbox or wait.
template <int D>
__global__ void __launch_bounds__(D) gqa_merge_ranks_kernel(const float* __restrict__ parts, int nranks, long long rows, void* out, int out_f32) {
    const int64_t rh = blockIdx.x;
    const int d = threadIdx.x;
    const float* base = parts + rh * (D + 2);
    const int64_t stride = rows * (D + 2);
    float mx = -INFINITY;
    for (int r = 0; r < nranks; ++r) mx = fmaxf(mx, base[r * stride + D]);
    float L = 0.f, A = 0.f;
    if (mx != -INFINITY) {
        for (int r = 0; r < nranks; ++r) {
            const float mk = base[r * stride + D];
            const float e = mk == -INFINITY ? 0.f : exp2f(mk - mx);
            L += base[r * stride + D + 1] * e;
            A += base[r * stride + d] * e;
        }
    }
    const float v = L > 0.f ? A / L : 0.f;
    if (out_f32) ((float*) out)[rh * D + d] = v;
    else ((__half*) out)[rh * D + d] = __float2half_rn(v);
}

template <class K, class P>
cudaError_t launch_dependent(K kernel, unsigned blocks, unsigned threads, cudaStream_t stream, const P& params) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, params);
}

template <int D, int MT, int NSTAGE, int QF = 0>
int launch(ns_gpu* g, const Params& p, int64_t B, const char* where) {
    constexpr int RG = 16 * MT;
    constexpr size_t tile = (size_t) KT * D * 2, raw_tile = (size_t) KT * raw_row_bytes<QF>(D);
    constexpr size_t smem = (size_t) RG * D * 2 + (size_t) WARPS * (QF == 0 ? NSTAGE * 2 * tile : NSTAGE * 2 * raw_tile);
    static_assert(QF == 0 || 2 * (smem + 1024) <= 227 * 1024, "two CTAs of a quantised instance share an SM");
    static_assert(smem >= (size_t) RG * D * 2 + (size_t) WARPS * RG * (D + 2) * 4, "the merge buffer fits the stage memory");
    auto kern = gqa_decode_kernel<D, MT, NSTAGE, QF>;
    static bool set[64] = {};
    if (!set[g->dev & 63]) {
        NS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem), where);
        set[g->dev & 63] = true;
    }
    dim3 grid((unsigned) (p.ns_max * p.groups), (unsigned) p.Hkv, (unsigned) B);
    if constexpr (QF == 0) {
        if (p.spins > 0) {
            // the whole KV-split step as one kernel, when every CTA of the grid can be resident at once (its CTAs wait on
            // one another)
            auto fused = gqa_decode_kernel<D, MT, NSTAGE, QF, true>;
            static bool fset[64] = {};
            static int per_sm[64] = {};
            if (!fset[g->dev & 63]) {
                NS_CUDA(cudaFuncSetAttribute(fused, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem), where);
                NS_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm[g->dev & 63], fused, THREADS, smem), where);
                fset[g->dev & 63] = true;
            }
            if ((int64_t) grid.x * grid.y <= (int64_t) per_sm[g->dev & 63] * g->sms) {
                // a cooperative launch: the driver guarantees what the kernel relies on. (Measured against a plain launch of
                // the same grid: 37.7 against 45.7 us a step at 32,768 keys a rank, 70.7 against 104 at 131,072.)
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = grid;
                cfg.blockDim = dim3(THREADS);
                cfg.dynamicSmemBytes = smem;
                cfg.stream = g->compute;
                cudaLaunchAttribute attr[1];
                attr[0].id = cudaLaunchAttributeCooperative;
                attr[0].val.cooperative = 1;
                cfg.attrs = attr;
                cfg.numAttrs = 1;
                NS_CUDA(cudaLaunchKernelEx(&cfg, fused, p), where);
                return ns_launched(where);
            }
            // too many CTAs to be resident together: the three launches below
            Params q = p;
            q.sync = nullptr;
            kern<<<grid, THREADS, smem, g->compute>>>(q);
            if (ns_launched(where)) return -1;
            NS_CUDA(launch_dependent(gqa_merge_push_kernel<D>, (unsigned) (p.T * p.Hq), MERGE_THREADS, g->compute, q), where);
            if (ns_launched(where)) return -1;
            return ns_launch_gqa_combine(g, p.mailboxes_host_own, p.nranks, p.T, p.Hq, D, p.epoch, p.spins, p.out, p.out_f32, where);
        }
    }
    kern<<<grid, THREADS, smem, g->compute>>>(p);
    if (ns_launched(where)) return -1;
    if (p.mailboxes || p.local_part) {
        NS_CUDA(launch_dependent(gqa_merge_push_kernel<D>, (unsigned) (p.T * p.Hq), MERGE_THREADS, g->compute, p), where);
        if (ns_launched(where)) return -1;
    } else if (p.ns_max > 1) {
        NS_CUDA(launch_dependent(gqa_merge_kernel<D>, (unsigned) (B * p.T * p.Hq), MERGE_THREADS, g->compute, p), where);
        if (ns_launched(where)) return -1;
    }
    return 0;
}

}  // namespace

int ns_launch_gqa_decode(ns_gpu* g, const GqaDecodeArgs& a, const char* where) {
    Params p;
    p.q = a.q;
    p.qs = a.qs;
    p.q_seq = a.q_seq;
    p.seqs = a.seqs;
    p.one = a.one;
    p.out = a.out;
    p.part = a.part;
    p.T = (int) a.T;
    p.Hq = (int) a.Hq;
    p.Hkv = (int) a.Hkv;
    p.G = (int) (a.Hq / a.Hkv);
    p.ns_max = (int) a.ns_max;
    p.q_f32 = a.q_f32;
    p.out_f32 = a.out_f32;
    p.qscale = 1.0f / sqrtf((float) a.D) * 1.4426950408889634f;
    p.force_part = (a.mailboxes || a.local_part) ? 1 : 0;
    p.local_part = a.local_part;
    p.rank = a.rank;
    p.nranks = a.nranks;
    p.mailboxes = a.mailboxes;
    p.epoch = a.epoch;
    // the counted hand-over to the merge: one sequence-and-key-head pair a counter; the KV-split path keeps the plain dependent
    p.sync = (!a.mailboxes && !a.local_part && a.ns_max > 1 && a.B * a.Hkv <= NS_DEC_SYNC_SLOTS) ? g->dec_sync : nullptr;
    p.status = g->status_dev;
    p.spins = 0;
    p.mailboxes_host_own = nullptr;
    if (a.mailboxes && a.fused_spins > 0) {
        if (a.kt != 0 || a.Hkv > NS_DEC_SYNC_SLOTS) return ns_fail(std::string(where) + ": the one-kernel step takes fp16 caches");
        p.sync = g->dec_sync;      // [Hkv] CTAs of a key head done; the step's last CTA returns them to zero
        p.spins = a.fused_spins;
        p.mailboxes_host_own = a.own_mailbox;
    }
    const int R = p.T * p.G;
    if (a.B > 65535) return ns_fail(std::string(where) + ": too many sequences for one launch");
    if (a.kt != 0) {
        if (a.D != 256 || (a.kt != 1 && a.kt != 2)) return ns_fail(std::string(where) + ": quantised caches are q8_0 (1) or q4_0 (2) with heads of 256");
        p.groups = (R + 15) / 16;
        return a.kt == 1 ? launch<256, 1, 3, 1>(g, p, a.B, where) : launch<256, 1, 4, 2>(g, p, a.B, where);
    }
    if (a.D == 128) {
        if (R <= 16) {
            p.groups = 1;
            return launch<128, 1, 3>(g, p, a.B, where);
        }
        // 32-row CTAs: measured faster than pairs of 16-row CTAs sharing tiles through L2 (119 vs 142 us on 512 MiB)
        p.groups = (R + 31) / 32;
        return launch<128, 2, 3>(g, p, a.B, where);
    }
    if (a.D == 256) {
        p.groups = (R + 15) / 16;
        return launch<256, 1, 3>(g, p, a.B, where);
    }
    return ns_fail(std::string(where) + ": heads of 128 or 256");
}

// ---- decode without caller scratch -----------------------------------------------------------------------------------
// Some callers cannot hand the library a scratch buffer and must not cause an allocation either: an engine whose
// memory plan is fixed when the model is loaded (every byte of the GPU already assigned to weights and caches, so a
// later cudaMalloc may fail, and in any case synchronises the device in the middle of serving), or a decode loop that
// runs with its arena frozen. For them the split partials live in this fixed array instead. It costs
// NS_B200_STATIC_SCRATCH_FLOATS * 4 bytes on every GPU the library is used on, for the life of the process.
namespace {
static __device__ __align__(256) float g_static_scratch[NS_B200_STATIC_SCRATCH_FLOATS];

// touches the array from device code once a device (also keeps the symbol alive in the device image)
__global__ void static_scratch_setup() { g_static_scratch[0] = 0.f; }

std::mutex g_static_mu;
float* g_static_ptr[64] = {};   // per device ordinal: the array's DEVICE address (the host-side name is only a handle)

// the device address of g_static_scratch on g's device, looked up once per device with that device current
int static_scratch(ns_gpu* g, float** out, const char* where) {
    if (g->dev < 0 || g->dev >= 64) return ns_fail(std::string(where) + ": device ordinal out of range");
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_ptr[g->dev]) {
        float* p = nullptr;
        NS_CUDA(cudaGetSymbolAddress((void**) &p, g_static_scratch), where);
        if (!p) return ns_fail(std::string(where) + ": the static scratch has no device address");
        static_scratch_setup<<<1, 1, 0, g->compute>>>();
        if (ns_launched(where)) return -1;
        g_static_ptr[g->dev] = p;
    }
    *out = g_static_ptr[g->dev];
    return 0;
}
}  // namespace

extern "C" int ns_b200_gqa_decode_static(ns_gpu* g, const void* q, int64_t qs, int64_t q_seq, const ns_b200_seq* seqs, int64_t B, int64_t T,
                                         int64_t Hq, int64_t Hkv, int64_t D, int64_t max_kv, void* out) {
    NS_TRY
    const char* name = "ns_b200_gqa_decode_static";
    if (ns_enter(g, name)) return -1;
    if (B < 1) return 0;
    if (T < 1 || T > 8 || (D != 128 && D != 256) || Hkv < 1 || Hq < 1 || Hq % Hkv != 0 || Hq / Hkv > 16)
        return ns_fail(std::string(name) + ": 1..8 rows, heads of 128 or 256, 1..16 query heads a key head");
    if (max_kv < T || max_kv >= ((int64_t) 1 << 31)) return ns_fail(std::string(name) + ": max_kv between T and 2^31");
    if (qs % 8 != 0 || q_seq % 8 != 0 || ((uintptr_t) q & 15) != 0) return ns_fail(std::string(name) + ": query rows 16-byte aligned");
    if (!q || !seqs || !out) return ns_fail(std::string(name) + ": a null buffer");
    const int64_t ns = ns_dec_splits_bound(max_kv, Hkv);   // as ns_b200_gqa_decode lays its partials out
    const int64_t need = ns > 1 ? B * T * Hq * ns * (D + 2) : 0;
    if (need > (int64_t) NS_B200_STATIC_SCRATCH_FLOATS)
        return ns_fail(std::string(name) + ": this batch needs " + std::to_string(need) + " floats of split partials, the built-in scratch holds " +
                       std::to_string((int64_t) NS_B200_STATIC_SCRATCH_FLOATS) + "; use ns_b200_gqa_decode with caller scratch");
    float* part = nullptr;
    if (static_scratch(g, &part, name)) return -1;
    GqaDecodeArgs a{};
    a.q = q;
    a.qs = qs;
    a.q_seq = q_seq;
    a.seqs = seqs;
    a.out = out;
    a.part = part;
    a.B = B, a.T = T, a.Hq = Hq, a.Hkv = Hkv, a.D = D;
    a.ns_max = ns;
    a.q_f32 = 0, a.out_f32 = 0;
    return ns_launch_gqa_decode(g, a, name);
    NS_CATCH("ns_b200_gqa_decode_static")
}

int ns_launch_gqa_merge_ranks(ns_gpu* g, const float* parts, int nranks, int64_t T, int64_t Hq, int64_t D, void* out, int out_f32, const char* where) {
    if (D == 128) gqa_merge_ranks_kernel<128><<<(unsigned) (T * Hq), 128, 0, g->compute>>>(parts, nranks, T * Hq, out, out_f32);
    else if (D == 256) gqa_merge_ranks_kernel<256><<<(unsigned) (T * Hq), 256, 0, g->compute>>>(parts, nranks, T * Hq, out, out_f32);
    else return ns_fail(std::string(where) + ": heads of 128 or 256");
    return ns_launched(where);
}

int ns_launch_gqa_combine(ns_gpu* g, float* mailbox, int nranks, int64_t T, int64_t Hq, int64_t D, int64_t epoch, int64_t spins, void* out,
                          int out_f32, const char* where) {
    CombineParams c;
    c.mailbox = mailbox;
    c.out = out;
    c.status = g->status_dev;
    c.nranks = nranks;
    c.D = (int) D;
    c.out_f32 = out_f32;
    c.rows = T * Hq;
    c.epoch = epoch;
    c.spins = spins;
    if (D == 128) gqa_combine_kernel<128><<<(unsigned) (T * Hq), 128, 0, g->compute>>>(c);
    else if (D == 256) gqa_combine_kernel<256><<<(unsigned) (T * Hq), 256, 0, g->compute>>>(c);
    else if (D == 512) gqa_combine_kernel<512><<<(unsigned) (T * Hq), 512, 0, g->compute>>>(c);   // absorbed MLA's latent rows
    else return ns_fail(std::string(where) + ": rows of 128, 256 or 512");
    return ns_launched(where);
}
