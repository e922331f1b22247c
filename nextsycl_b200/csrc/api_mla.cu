// api_mla.cu: the C-ABI entry points of absorbed MLA attention: deepseek2's fused decode under its own name
// (kernels/llm/deepseek2/ds2.h:33-37) and the native middle stage.
#include "kernels.cuh"

namespace {

constexpr int L = 512, R = 64, NOPE = 128, V = 128, KL = NOPE + R, CR = L + R;

// q~[t,h,:512] = k_b[h] . q_nope[t,h] (k_b [H][512][128] fp16, fp32 sums: ds2.cpp:176-183), the rotated 64 copied
// behind it; written as fp16 [T][H][576], the operand of the tensor-core stage.
// 8 warps a block, a warp a row of the weight matrix at a time, ROWS_IN_FLIGHT rows' loads issued before the first is used
// (one row a time waits out a memory latency a row: 20 us for the 16.8 MB of k_b).
constexpr int ABSORB_SPLIT = 4;        // blocks a (row, head): 128 of k_b's 512 rows each
__global__ void __launch_bounds__(256) mla_absorb_kernel(const float* __restrict__ q, const __half* __restrict__ kb, __half* __restrict__ qa, int T, int H) {
    __shared__ float qn[NOPE];
    const int th = blockIdx.x / ABSORB_SPLIT, part = blockIdx.x % ABSORB_SPLIT, h = th % H;
    const float* qr = q + (int64_t) th * KL;
    if (threadIdx.x < NOPE) qn[threadIdx.x] = qr[threadIdx.x];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __half* dst = qa + (int64_t) th * CR;
    const float q0 = qn[lane * 4], q1 = qn[lane * 4 + 1], q2 = qn[lane * 4 + 2], q3 = qn[lane * 4 + 3];
    constexpr int ROWS = L / ABSORB_SPLIT / 8;   // rows a warp: 16
    const int r0 = part * (L / ABSORB_SPLIT) + warp * ROWS;
    uint2 w[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) w[i] = reinterpret_cast<const uint2*>(kb + ((int64_t) h * L + r0 + i) * NOPE)[lane];   // 4 halves a lane
    float acc[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
        const __half2* hh = reinterpret_cast<const __half2*>(&w[i]);
        const float2 a = __half22float2(hh[0]), b = __half22float2(hh[1]);
        acc[i] = a.x * q0 + a.y * q1 + b.x * q2 + b.y * q3;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int i = 0; i < ROWS; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
    if (lane < ROWS) {
        float v = acc[0];
#pragma unroll
        for (int i = 1; i < ROWS; ++i) v = lane == i ? acc[i] : v;
        dst[r0 + lane] = __float2half_rn(v);
    }
    if (part == 0 && threadIdx.x < R) dst[L + threadIdx.x] = __float2half_rn(qr[NOPE + threadIdx.x]);
}

// out[t,h,:128] = v_b[h] . u[t,h] (v_b [H][128][512] fp16, fp32 sums: ds2.cpp:237-255). A warp 4 rows of v_b at a time.
constexpr int UNABSORB_SPLIT = 4;      // blocks a (row, head): 32 of v_b's 128 rows each
__global__ void __launch_bounds__(256) mla_unabsorb_kernel(const float* __restrict__ u, const __half* __restrict__ vb, float* __restrict__ out, int T, int H) {
    __shared__ float us[L];
    const int th = blockIdx.x / UNABSORB_SPLIT, part = blockIdx.x % UNABSORB_SPLIT, h = th % H;
    for (int i = threadIdx.x; i < L; i += blockDim.x) us[i] = u[(int64_t) th * L + i];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int ROWS = V / UNABSORB_SPLIT / 8;   // rows a warp: 4
    const int r0 = part * (V / UNABSORB_SPLIT) + warp * ROWS;
    uint4 w[ROWS][2];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
        const uint4* vr = reinterpret_cast<const uint4*>(vb + ((int64_t) h * V + r0 + i) * L);
        w[i][0] = vr[lane];
        w[i][1] = vr[32 + lane];
    }
    float acc[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
        float a = 0.f;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const __half2* hh = reinterpret_cast<const __half2*>(&w[i][k]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 x = __half22float2(hh[e]);
                a += x.x * us[(k * 32 + lane) * 8 + 2 * e] + x.y * us[(k * 32 + lane) * 8 + 2 * e + 1];
            }
        }
        acc[i] = a;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int i = 0; i < ROWS; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
    if (lane < ROWS) {
        float v = acc[0];
#pragma unroll
        for (int i = 1; i < ROWS; ++i) v = lane == i ? acc[i] : v;
        out[(int64_t) th * V + r0 + lane] = v;
    }
}

// ---- kv_b as the model file stores it: Q6_K rows of 512 values (two 210-byte blocks: ql [128], qh [64], scales [16] int8,
// d half; kernels/llm/deepseek2/ds2.cpp:117-137), per head its 128 k rows then its 128 v rows. A warp decodes one row at a
// time: lane = (block, half n, group l4 of four l) takes the 16 values (quarter g 0..3) x (l = 4 l4 .. 4 l4 + 3), i.e.
// columns 256 block + 128 n + 32 g + 4 l4 + e, from four bytes of ql's low part, four of its high part, four of qh and
// the four scales of its half - read as 16-bit words, the blocks being only 2-byte aligned. Value = d * scale * (q - 32)
// in fp32, the reference's order.
constexpr int Q6_ROW_BYTES = 2 * 210;
__device__ __forceinline__ uint32_t ld_u32_2(const uint8_t* p) {
    const uint16_t* h = reinterpret_cast<const uint16_t*>(p);
    return (uint32_t) h[0] | ((uint32_t) h[1] << 16);
}
__device__ __forceinline__ int q6_col(int lane, int g, int e) { return 256 * (lane >> 4) + 128 * ((lane >> 3) & 1) + 32 * g + 4 * (lane & 7) + e; }
__device__ __forceinline__ void q6_decode16(const uint8_t* row, int lane, float (&v)[16]) {
    const uint8_t* blk = row + (lane >> 4) * 210;
    const int n = (lane >> 3) & 1, l4 = lane & 7;
    const uint32_t qa = ld_u32_2(blk + 64 * n + 4 * l4), qb = ld_u32_2(blk + 64 * n + 32 + 4 * l4), qh = ld_u32_2(blk + 128 + 32 * n + 4 * l4);
    const float d = __half2float(*reinterpret_cast<const __half*>(blk + 208));
    const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192) + 8 * n + (l4 >> 2);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const float ds = __fmul_rn(d, (float) sc[2 * g]);
        const uint32_t ql = (g & 1) ? qb : qa;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t lb = (ql >> (8 * e)) & 0xFF, hb = (qh >> (8 * e)) & 0xFF;
            const int lo = g < 2 ? (int) (lb & 0xF) : (int) (lb >> 4);
            const int q = (lo | (int) (((hb >> (2 * g)) & 3) << 4)) - 32;
            v[4 * g + e] = __fmul_rn(ds, (float) q);
        }
    }
}

// q~[t,h,c] = sum_i q_nope[i] k_i[c] over the head's 128 Q6_K k rows (ds2.cpp:172-183), the rotated 64 copied behind it,
// as fp16 [T][H][576]. A block a (row, head): its 8 warps each take every 8th k row, the sums meet in shared memory.
__global__ void __launch_bounds__(256) mla_absorb_q6k_kernel(const float* __restrict__ q, const uint8_t* __restrict__ kvb, __half* __restrict__ qa, int H) {
    __shared__ float qn[NOPE];
    __shared__ float part[8][L];
    const int th = blockIdx.x, h = th % H;
    const float* qr = q + (int64_t) th * KL;
    if (threadIdx.x < NOPE) qn[threadIdx.x] = qr[threadIdx.x];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint8_t* rows = kvb + (int64_t) h * (NOPE + V) * Q6_ROW_BYTES;
    float acc[16];
#pragma unroll
    for (int f = 0; f < 16; ++f) acc[f] = 0.f;
    for (int i = warp; i < NOPE; i += 8) {
        float v[16];
        q6_decode16(rows + (int64_t) i * Q6_ROW_BYTES, lane, v);
        const float qi = qn[i];
#pragma unroll
        for (int f = 0; f < 16; ++f) acc[f] = fmaf(qi, v[f], acc[f]);
    }
#pragma unroll
    for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int e = 0; e < 4; ++e) part[warp][q6_col(lane, g, e)] = acc[4 * g + e];
    __syncthreads();
    __half* dst = qa + (int64_t) th * CR;
    for (int c = threadIdx.x; c < L; c += 256) {
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) a += part[w][c];
        dst[c] = __float2half_rn(a);
    }
    if (threadIdx.x < R) dst[L + threadIdx.x] = __float2half_rn(qr[NOPE + threadIdx.x]);
}

// out[t,h,r] = sum_c v_r[c] u[c] over the head's 128 Q6_K v rows (ds2.cpp:237-255). A block a (row, head), a warp a v row at a time.
__global__ void __launch_bounds__(256) mla_unabsorb_q6k_kernel(const float* __restrict__ u, const uint8_t* __restrict__ kvb, float* __restrict__ out, int H) {
    __shared__ float us[L];
    const int th = blockIdx.x, h = th % H;
    for (int i = threadIdx.x; i < L; i += 256) us[i] = u[(int64_t) th * L + i];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint8_t* rows = kvb + ((int64_t) h * (NOPE + V) + NOPE) * Q6_ROW_BYTES;
    float mine[16];
#pragma unroll
    for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int e = 0; e < 4; ++e) mine[4 * g + e] = us[q6_col(lane, g, e)];
    for (int r = warp; r < V; r += 8) {
        float v[16];
        q6_decode16(rows + (int64_t) r * Q6_ROW_BYTES, lane, v);
        float a = 0.f;
#pragma unroll
        for (int f = 0; f < 16; ++f) a = fmaf(v[f], mine[f], a);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (lane == 0) out[(int64_t) th * V + r] = a;
    }
}

int check_rows(const char* name, int64_t T, int64_t H, int64_t pos0) {
    if (T < 1 || T > 64) return ns_fail(std::string(name) + ": 1..64 rows");
    if (H < 1 || H > 1024) return ns_fail(std::string(name) + ": 1..1024 heads");
    if (pos0 < 0 || pos0 + T >= ((int64_t) 1 << 31)) return ns_fail(std::string(name) + ": positions below 2^31");
    return 0;
}

}  // namespace

extern "C" {

int64_t ns_b200_mla_decode_scratch(ns_gpu* g, int64_t T, int64_t H, int64_t pos0) {
    if (!g || T < 1 || H < 1 || pos0 < 0) return 0;
    return ns_mla_partial_floats(pos0 + T, T, H, g->sms);
}

int ns_b200_mla_decode(ns_gpu* g, const void* q, const void* cache, int64_t T, int64_t H, int64_t pos0, float scale, float* out, float* scratch) {
    NS_TRY
    const char* name = "ns_b200_mla_decode";
    if (ns_enter(g, name)) return -1;
    if (check_rows(name, T, H, pos0)) return -1;
    if (!q || !cache || !out) return ns_fail(std::string(name) + ": a null buffer");
    if (((uintptr_t) q & 15) != 0 || ((uintptr_t) cache & 15) != 0 || ((uintptr_t) out & 15) != 0 || ((uintptr_t) scratch & 15) != 0)
        return ns_fail(std::string(name) + ": buffers 16-byte aligned");
    if (ns_mla_partial_floats(pos0 + T, T, H, g->sms) > 0 && !scratch) return ns_fail(std::string(name) + ": no scratch");
    MlaDecodeArgs a{q, cache, out, scratch, T, H, pos0, scale, 64, pos0 + T, nullptr, 0, nullptr};
    return ns_launch_mla_decode(g, a, name);
    NS_CATCH("ns_b200_mla_decode")
}

// kernels/llm/deepseek2/ds2.h:33-37: q [T][H][192] fp32 (rope part rotated), k_b [H][512][128], v_b [H][128][512] and the
// cache fp16 -> out [T][H][128]. Three stages on the compute stream: absorb (q~ = k_b q_nope), the tensor-core latent
// attention, un-absorb (out = v_b u); q~, u and the split partials live in the GPU's kept buffer.
int ns_ds2_mla_decode(ns_gpu* g, const float* q, const uint16_t* kb, const uint16_t* vb, const uint16_t* cache, float* out, int64_t T, int64_t H,
                      int64_t pos0, float scale) {
    NS_TRY
    const char* name = "ns_ds2_mla_decode";
    if (ns_enter(g, name)) return -1;
    if (check_rows(name, T, H, pos0)) return -1;
    if (!q || !kb || !vb || !cache || !out) return ns_fail(std::string(name) + ": a null buffer");
    if (((uintptr_t) kb & 15) != 0 || ((uintptr_t) vb & 15) != 0 || ((uintptr_t) cache & 15) != 0) return ns_fail(std::string(name) + ": buffers 16-byte aligned");
    const int64_t qa_bytes = (T * H * CR * 2 + 255) / 256 * 256, u_bytes = (T * H * L * 4 + 255) / 256 * 256;
    const int64_t part_floats = ns_mla_partial_floats(pos0 + T, T, H, g->sms);
    void* kept = nullptr;
    if (ns_kept(g, (size_t) (qa_bytes + u_bytes + part_floats * 4), &kept)) return -1;
    __half* qa = (__half*) kept;
    float* u = (float*) ((uint8_t*) kept + qa_bytes);
    float* part = part_floats ? (float*) ((uint8_t*) kept + qa_bytes + u_bytes) : nullptr;
    mla_absorb_kernel<<<(unsigned) (T * H * ABSORB_SPLIT), 256, 0, g->compute>>>(q, (const __half*) kb, qa, (int) T, (int) H);
    if (ns_launched(name)) return -1;
    MlaDecodeArgs a{qa, cache, u, part, T, H, pos0, scale, 64, pos0 + T, nullptr, 0, nullptr};
    if (ns_launch_mla_decode(g, a, name)) return -1;
    mla_unabsorb_kernel<<<(unsigned) (T * H * UNABSORB_SPLIT), 256, 0, g->compute>>>(u, (const __half*) vb, out, (int) T, (int) H);
    return ns_launched(name);
    NS_CATCH("ns_ds2_mla_decode")
}

// ---- one context's latent cache split over several GPUs by cell ranges -------------------------------------------------
int64_t ns_b200_mla_kvsplit_scratch(ns_gpu* g, int64_t T, int64_t H, int64_t cells_local) {
    if (!g || T < 1 || H < 1 || cells_local < 1) return 0;
    return ns_mla_partial_floats_split(cells_local, T, H, g->sms);
}

int ns_b200_mla_kvsplit_decode(ns_gpu* g, const void* q, const void* cache, int64_t T, int64_t H, int64_t cells_local, int64_t cell_base, int64_t pos0,
                               float scale, float* scratch, int64_t rank, int64_t nranks, void* const* mailboxes, int64_t epoch) {
    NS_TRY
    const char* name = "ns_b200_mla_kvsplit_decode";
    if (ns_enter(g, name)) return -1;
    if (check_rows(name, T, H, pos0)) return -1;
    if (T > 8) return ns_fail(std::string(name) + ": 1..8 rows");
    if (nranks < 1 || nranks > 64 || rank < 0 || rank >= nranks) return ns_fail(std::string(name) + ": rank within 1..64 ranks");
    if (cells_local < 0 || cells_local >= ((int64_t) 1 << 31) || cell_base < 0 || epoch < 0) return ns_fail(std::string(name) + ": a cell range of 0 .. 2^31 cells, epochs from 1");
    if (!q || !mailboxes || (cells_local > 0 && (!cache || !scratch))) return ns_fail(std::string(name) + ": a null buffer");
    if (((uintptr_t) q & 15) != 0 || ((uintptr_t) cache & 15) != 0 || ((uintptr_t) scratch & 15) != 0) return ns_fail(std::string(name) + ": buffers 16-byte aligned");
    MlaDecodeArgs a{q, cache, nullptr, scratch, T, H, pos0 - cell_base, scale, 64, cells_local, nullptr, 0, nullptr};
    a.mailboxes = (float* const*) mailboxes;
    a.rank = (int) rank;
    a.nranks = (int) nranks;
    a.epoch = epoch;
    return ns_launch_mla_decode(g, a, name);
    NS_CATCH("ns_b200_mla_kvsplit_decode")
}

int ns_b200_mla_kvsplit_combine(ns_gpu* g, void* mailbox, int64_t nranks, int64_t T, int64_t H, int64_t epoch, int64_t wait_us, float* out) {
    NS_TRY
    const char* name = "ns_b200_mla_kvsplit_combine";
    if (ns_enter(g, name)) return -1;
    if (!mailbox || !out) return ns_fail(std::string(name) + ": a null buffer");
    if (nranks < 1 || nranks > 64 || T < 1 || T > 8 || H < 1 || epoch < 0) return ns_fail(std::string(name) + ": 1..64 ranks, 1..8 rows, epochs from 1");
    if (wait_us < 1 || wait_us > 2000000) return ns_fail(std::string(name) + ": a wait of 1 us .. 2 s");
    return ns_launch_gqa_combine(g, (float*) mailbox, (int) nranks, T, H, L, epoch, wait_us * 10, out, 1, name);
    NS_CATCH("ns_b200_mla_kvsplit_combine")
}

// kernels/llm/deepseek2/ds2.h:38-41: the same with kv_b as the model file stores it - Q6_K, [H x (128 + 128)] rows of 512: per
// head its 128 k rows (row i = k_i[0..511], so q~ = sum_i q_nope[i] k_i), then its 128 v rows - decoded where it is read.
int ns_ds2_mla_decode_q6k(ns_gpu* g, const float* q, const void* kvb, const uint16_t* cache, float* out, int64_t T, int64_t H, int64_t pos0, float scale) {
    NS_TRY
    const char* name = "ns_ds2_mla_decode_q6k";
    if (ns_enter(g, name)) return -1;
    if (check_rows(name, T, H, pos0)) return -1;
    if (!q || !kvb || !cache || !out) return ns_fail(std::string(name) + ": a null buffer");
    if (((uintptr_t) kvb & 1) != 0 || ((uintptr_t) cache & 15) != 0) return ns_fail(std::string(name) + ": kv_b 2-byte aligned, the cache 16-byte aligned");
    const int64_t qa_bytes = (T * H * CR * 2 + 255) / 256 * 256, u_bytes = (T * H * L * 4 + 255) / 256 * 256;
    const int64_t part_floats = ns_mla_partial_floats(pos0 + T, T, H, g->sms);
    void* kept = nullptr;
    if (ns_kept(g, (size_t) (qa_bytes + u_bytes + part_floats * 4), &kept)) return -1;
    __half* qa = (__half*) kept;
    float* u = (float*) ((uint8_t*) kept + qa_bytes);
    float* part = part_floats ? (float*) ((uint8_t*) kept + qa_bytes + u_bytes) : nullptr;
    mla_absorb_q6k_kernel<<<(unsigned) (T * H), 256, 0, g->compute>>>(q, (const uint8_t*) kvb, qa, (int) H);
    if (ns_launched(name)) return -1;
    MlaDecodeArgs a{qa, cache, u, part, T, H, pos0, scale, 64, pos0 + T, nullptr, 0, nullptr};
    if (ns_launch_mla_decode(g, a, name)) return -1;
    mla_unabsorb_q6k_kernel<<<(unsigned) (T * H), 256, 0, g->compute>>>(u, (const uint8_t*) kvb, out, (int) H);
    return ns_launched(name);
    NS_CATCH("ns_ds2_mla_decode_q6k")
}

}  // extern "C"
