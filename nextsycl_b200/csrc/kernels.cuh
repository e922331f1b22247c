// kernels.cuh: launchers of the attention kernels, as the C-ABI wrappers (api_*.cu) call them. Each queues work on the
// given stream and returns 0, or -1 through ns_fail.
#pragma once
#include "ns_internal.cuh"
#include "ns_attn.h"

// ---- GQA decode (gqa_decode.cu) -------------------------------------------------------------------------------------
// Keys a split for a row that sees `kv` keys: enough splits that key heads x splits fill two CTAs per SM, in
// multiples of 64 keys. A function of the row's own length only, so a row's arithmetic does not depend on what else
// shares its launch (the property of kernels/llm/qwen35/silo/attn.cpp:100-104).
constexpr int NS_DEC_TARGET_CTAS = 296;
__host__ __device__ inline int64_t ns_dec_split(int64_t kv, int64_t Hkv) {
    const int64_t want = (kv * Hkv + NS_DEC_TARGET_CTAS - 1) / NS_DEC_TARGET_CTAS;
    const int64_t kb = (want + 63) / 64 * 64;
    return kb < 64 ? 64 : kb;
}
__host__ __device__ inline int64_t ns_dec_splits(int64_t kv, int64_t Hkv) {
    const int64_t kb = ns_dec_split(kv, Hkv);
    return (kv + kb - 1) / kb;
}
// The most splits any row of 1 .. max_kv keys can have. ns_dec_splits is not monotone in kv (each 64-key step of the
// split size lowers the count), so a partial buffer shared by rows of several lengths is laid out for this bound, never
// for the longest row's own count: kb >= 64 gives ceil(max_kv / 64), kb >= kv Hkv / 296 gives ceil(296 / Hkv).
__host__ __device__ inline int64_t ns_dec_splits_bound(int64_t max_kv, int64_t Hkv) {
    const int64_t a = (max_kv + 63) / 64, b = (NS_DEC_TARGET_CTAS + Hkv - 1) / Hkv;
    return a < b ? a : b;
}

struct GqaDecodeArgs {
    const void* q;             // [B][T] rows of Hq*D, fp32 or fp16
    int64_t qs;                // elements between rows
    int64_t q_seq;             // elements between sequences
    const ns_b200_seq* seqs;   // device array [B], or null: `one`
    ns_b200_seq one;
    void* out;                 // [B][T][Hq*D], fp32 or fp16
    float* part;               // [B][T][Hq][ns_max][D+2]
    int64_t B, T, Hq, Hkv, D;
    int64_t ns_max;            // splits the partial buffer is laid out for
    int q_f32, out_f32;
    // KV split over several GPUs (null mailboxes: a whole sequence on this GPU)
    float* const* mailboxes;   // device array [nranks] of mailbox bases as this GPU addresses them
    int rank, nranks;
    int64_t epoch;
    int kt = 0;                // the caches' form: 0 fp16, 1 q8_0, 2 q4_0 (heads of 256; rows of 272 / 144 bytes)
    // the whole KV-split step (decode, push, combine) in one kernel: polls a wait on the peers may take (0: the decode and
    // push only), and this rank's own mailbox as the host addresses it
    int64_t fused_spins = 0;
    float* own_mailbox = nullptr;
    float* local_part = nullptr;   // [T*Hq][D+2]: keep the rank's merged partial here (no mailboxes, nothing pushed)
};

// A rank's mailbox for the KV-split combine, in floats from its base: partials [2 buffers][nranks][rows][D+2], then
// (16-float aligned) the flags [2][nranks] as 64-bit epochs and a block counter.
__host__ __device__ inline int64_t ns_mbox_slot(int buf, int rank, int nranks, int64_t rows, int64_t D) {
    return ((int64_t) (buf * nranks + rank) * rows) * (D + 2);
}
__host__ __device__ inline int64_t ns_mbox_flags_off(int nranks, int64_t rows, int64_t D) {
    return (2 * (int64_t) nranks * rows * (D + 2) + 15) / 16 * 16;
}
__host__ __device__ inline int64_t ns_mbox_bytes(int nranks, int64_t rows, int64_t D);
// Behind all that, 16-byte aligned, the lines of the one-kernel step: [2 buffers][nranks][rows][D/2 + 1] lines of 16 bytes
// = (value, step tag, value, step tag) - a row's D values two a line, then (m, l). A line is written by ONE 16-byte store,
// and each of its 8-byte halves carries its own tag, so a reader that sees the tag has the value: data and flag in one
// transfer, no fence and no second round trip over NVLink.
__host__ __device__ inline int64_t ns_mbox_ll_off_bytes(int nranks, int64_t rows, int64_t D) {
    return (ns_mbox_flags_off(nranks, rows, D) * 4 + 2 * (int64_t) nranks * 8 + 64 + 15) / 16 * 16;
}
__host__ __device__ inline int64_t ns_mbox_ll_line(int buf, int rank, int nranks, int64_t rows, int64_t D) {
    return ((int64_t) (buf * nranks + rank) * rows) * (D / 2 + 1);
}
__host__ __device__ inline int64_t ns_mbox_bytes(int nranks, int64_t rows, int64_t D) {
    return ns_mbox_ll_off_bytes(nranks, rows, D) + 2 * (int64_t) nranks * rows * (D / 2 + 1) * 16;
}
// after the flags: two block counters (ints), then the rank's own step number (used when a call passes epoch 0)
__host__ __device__ inline long long* ns_mbox_epoch(float* mailbox, int nranks, int64_t rows, int64_t D) {
    return reinterpret_cast<long long*>(reinterpret_cast<int*>(mailbox + ns_mbox_flags_off(nranks, rows, D)) + 4 * nranks + 2);
}
int ns_launch_gqa_combine(ns_gpu* g, float* mailbox, int nranks, int64_t T, int64_t Hq, int64_t D, int64_t epoch, int64_t spins, void* out,
                          int out_f32, const char* where);
int ns_launch_gqa_decode(ns_gpu* g, const GqaDecodeArgs& a, const char* where);
int ns_launch_gqa_merge_ranks(ns_gpu* g, const float* parts, int nranks, int64_t T, int64_t Hq, int64_t D, void* out, int out_f32, const char* where);

// ---- cache writers (kv_store.cu) ------------------------------------------------------------------------------------
int ns_launch_kv_store(ns_gpu* g, const float* k, int64_t ks, const float* v, int64_t vs, int64_t T, int64_t Hkv, int64_t D, int64_t cap, int64_t p0,
                       void* kc, void* vc);

int ns_launch_kv_store_batch(ns_gpu* g, const float* k, int64_t ks, int64_t k_seq, const float* v, int64_t vs, int64_t v_seq, const ns_b200_seq* seqs,
                             int64_t B, int64_t T, int64_t Hkv, int64_t D);

// rows [0, n) of each head of a quantised cache (kt 1: q8_0, 2: q4_0; heads of 256) as fp16 [Hkv][n][256] (kv_quant.cu)
int ns_launch_kv_dequant(ns_gpu* g, int kt, const void* c, int64_t Hkv, int64_t cap, int64_t n, void* out, const char* where);

// fp32 rows -> 16-bit rows scaled by `scale` (one rounding, as the reference stages its queries: silo/attn.cpp:147)
int ns_launch_scale_to_f16(ns_gpu* g, const float* src, int64_t src_row, void* dst, int64_t dst_row, int64_t rows, int64_t cols, float scale);

// ---- flash prefill on tcgen05 (flash_prefill.cu) -------------------------------------------------------------------------
struct FlashPrefillArgs {
    const void* q;          // [T] rows of Hq*Dqk 16-bit elements, q_row elements apart
    int64_t q_row;
    const void* k;          // element (key, head, d) at key*k_key + head*k_head + d
    int64_t k_key, k_head;
    const void* v;
    int64_t v_key, v_head;
    void* out;              // [T][Hq*Dv] dense; fp32 when out_f32, else the operands' type
    int* status;            // device-visible status word
    int64_t T, Hq, Hkv, Dqk, Dv;
    int64_t p0, kv_len;     // kv_len = p0 + T keys exist
    float scale_log2;       // softmax scale times log2(e); 1 when q is pre-scaled
    int bf16, out_f32;
};
int ns_launch_flash_prefill(ns_gpu* g, const FlashPrefillArgs& a, const char* where);

// ---- absorbed MLA decode on tcgen05 (mla_decode.cu) --------------------------------------------------------------------
struct MlaDecodeArgs {
    const void* q;            // [T][H][512 + rope] fp16: the absorbed query, then the rotated part
    const void* cache;        // cells [n][512 + rope] fp16 - one matrix for all rows, or one per row (cache_rows_apart > 0)
    float* out;               // [T][H][512] fp32
    float* part;              // ns_mla_partial_floats floats (may be null when that is 0)
    int64_t T, H, pos0;
    float scale;
    int rope;                 // 64 (deepseek2's 576-wide rows) or 0 (glm5next's 512-wide rows)
    int64_t n_max;            // the most cells any row attends to (sizes the grid and the partials)
    const int* counts;        // device [T]: cells each row attends to; null: pos0 + t + 1 (causal over one shared cache)
    int64_t cache_rows_apart; // elements between the rows' own cell matrices; 0: one shared cache
    const float* sinks;       // device [H] or null: a per-head sink (natural-log units) that joins the denominator only
    // One context split over several GPUs by cell ranges (null mailboxes: the whole context on this GPU). `cache` then holds
    // this rank's cells only, n_max of them, and pos0 is the first row's position RELATIVE to the rank's first cell (it may be
    // negative or beyond the slice: a row sees min(pos0 + t + 1, n_max) of the rank's cells, none when that is <= 0). Every
    // row's partial is kept, merged over the rank's splits and pushed into slot `rank` of every rank's mailbox.
    float* const* mailboxes = nullptr;
    int rank = 0, nranks = 0;
    int64_t epoch = 0;
};
// floats of partials for a pass of T rows that see up to n cells, on a GPU of `sms` SMs
int64_t ns_mla_partial_floats(int64_t n, int64_t T, int64_t H, int sms);
int64_t ns_mla_partial_floats_split(int64_t n, int64_t T, int64_t H, int sms);
int ns_launch_mla_decode(ns_gpu* g, const MlaDecodeArgs& a, const char* where);
