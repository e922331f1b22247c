// api_gqa.cu: the C-ABI entry points of GQA attention (include/ns_attn.h): argument checks, then the launchers.
#include "kernels.cuh"

#include <algorithm>
#include <cstring>

int ns_prefill_f32(ns_gpu* g, const char* name, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv,
                   int64_t D, int64_t cap, int64_t p0, float* out);

namespace {

bool shape_ok(int64_t Hq, int64_t Hkv, int64_t D) {
    return (D == 128 || D == 256) && Hkv > 0 && Hq > 0 && Hq % Hkv == 0 && Hq / Hkv <= 16;
}

int64_t decode_ns_max(int64_t T, int64_t Hkv, int64_t p0) {
    int64_t ns = 1;
    for (int64_t r = 0; r < T; ++r) ns = std::max(ns, ns_dec_splits(p0 + r + 1, Hkv));
    return ns;
}

// rows 1..8 at p0.., fp32 in and out, one sequence: what ns_q35_attn_decode and its namesakes share
int decode_f32(ns_gpu* g, const char* name, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv,
               int64_t D, int64_t cap, int64_t p0, float* out, float* scratch, int kt = 0) {
    if (ns_enter(g, name)) return -1;
    if (T < 1 || T > 8 || !shape_ok(Hq, Hkv, D)) return ns_fail(std::string(name) + ": 1..8 rows, heads of 128 or 256, 1..16 query heads a key head");
    if (p0 < 0 || p0 + T > cap) return ns_fail(std::string(name) + ": past the cache's capacity");
    if (p0 + T >= ((int64_t) 1 << 31)) return ns_fail(std::string(name) + ": positions below 2^31");
    if (qs % 4 != 0 || ((uintptr_t) q & 15) != 0) return ns_fail(std::string(name) + ": query rows 16-byte aligned");
    if (!q || !kc || !vc || !out) return ns_fail(std::string(name) + ": a null buffer");
    const int64_t ns = decode_ns_max(T, Hkv, p0);
    if (ns > 1 && !scratch) return ns_fail(std::string(name) + ": no scratch");
    GqaDecodeArgs a{};
    a.q = q;
    a.qs = qs;
    a.q_seq = 0;
    a.seqs = nullptr;
    a.one = ns_b200_seq{kc, vc, cap, p0};
    a.out = out;
    a.part = scratch;
    a.B = 1, a.T = T, a.Hq = Hq, a.Hkv = Hkv, a.D = D;
    a.ns_max = ns;
    a.q_f32 = 1, a.out_f32 = 1;
    a.kt = kt;
    return ns_launch_gqa_decode(g, a, name);
}

int64_t decode_scratch(int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t p0) {
    if (T < 1 || Hkv < 1) return 0;
    const int64_t ns = decode_ns_max(T, Hkv, p0);
    return ns > 1 ? T * Hq * ns * (D + 2) : 0;
}

// any number of rows: up to 8 through the decode kernel, more through the tensor-core prompt kernel (api_prefill.cu)
int64_t rows_scratch(int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t p0) {
    return T <= 8 ? decode_scratch(T, Hq, Hkv, D, p0) : 0;
}
int rows_f32(ns_gpu* g, const char* name, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
             int64_t cap, int64_t p0, float* out, float* scratch) {
    if (T <= 0) return 0;
    if (p0 + T > cap) return ns_fail(std::string(name) + ": past the cache's capacity");
    if (T <= 8) return decode_f32(g, name, q, qs, kc, vc, T, Hq, Hkv, D, cap, p0, out, scratch);
    return ns_prefill_f32(g, name, q, qs, kc, vc, T, Hq, Hkv, D, cap, p0, out);
}

}  // namespace

extern "C" {

int ns_q35_kv_store(ns_gpu* g, const float* k, int64_t ks, const float* v, int64_t vs, int64_t T, int64_t Hkv, int64_t D, int64_t cap, int64_t p0,
                    void* kc, void* vc) {
    NS_TRY
    if (ns_enter(g, "ns_q35_kv_store")) return -1;
    if (T <= 0) return 0;
    if (p0 < 0 || p0 + T > cap) return ns_fail("ns_q35_kv_store: past the cache's capacity");
    if (D % 8 != 0 || ks % 4 != 0 || vs % 4 != 0) return ns_fail("ns_q35_kv_store: head width a multiple of 8, rows 16-byte aligned");
    return ns_launch_kv_store(g, k, ks, v, vs, T, Hkv, D, cap, p0, kc, vc);
    NS_CATCH("ns_q35_kv_store")
}

int64_t ns_q35_attn_scratch(int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t p0) { return rows_scratch(T, Hq, Hkv, D, p0); }

int ns_q35_attn(ns_gpu* g, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t cap,
                int64_t p0, float* out, float* scratch) {
    NS_TRY
    return rows_f32(g, "ns_q35_attn", q, qs, kc, vc, T, Hq, Hkv, D, cap, p0, out, scratch);
    NS_CATCH("ns_q35_attn")
}

int ns_q35_attn_decode_supported(int64_t T, int64_t Hq, int64_t Hkv, int64_t D) { return T >= 1 && T <= 8 && shape_ok(Hq, Hkv, D); }

int64_t ns_q35_attn_decode_scratch(int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t p0) { return decode_scratch(T, Hq, Hkv, D, p0); }

int ns_q35_attn_decode(ns_gpu* g, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                       int64_t cap, int64_t p0, float* out, float* scratch) {
    NS_TRY
    return decode_f32(g, "ns_q35_attn_decode", q, qs, kc, vc, T, Hq, Hkv, D, cap, p0, out, scratch);
    NS_CATCH("ns_q35_attn_decode")
}

int ns_q35_attn_decode_kv(ns_gpu* g, int kt, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv,
                          int64_t D, int64_t cap, int64_t p0, float* out, float* scratch) {
    NS_TRY
    if (kt == 0) return decode_f32(g, "ns_q35_attn_decode_kv", q, qs, kc, vc, T, Hq, Hkv, D, cap, p0, out, scratch);
    // q8_0 / q4_0 caches (heads of 256): the decode kernel streams the rows as they lie and expands them in registers to
    // the fp16 values the reference's reader hands its tensor cores (silo/attn.cpp:49-78)
    const char* name = "ns_q35_attn_decode_kv";
    if (kt != 1 && kt != 2) return ns_fail(std::string(name) + ": a cache form 0 (half), 1 (q8_0) or 2 (q4_0)");
    if (D != 256) return ns_fail(std::string(name) + ": quantised caches have heads of 256");
    if (((uintptr_t) kc & 15) != 0 || ((uintptr_t) vc & 15) != 0) return ns_fail(std::string(name) + ": caches 16-byte aligned");
    return decode_f32(g, name, q, qs, kc, vc, T, Hq, Hkv, D, cap, p0, out, scratch, kt);
    NS_CATCH("ns_q35_attn_decode_kv")
}

int64_t ns_nh_attn_scratch(int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t p0) { return rows_scratch(T, Hq, Hkv, D, p0); }

int ns_nh_attn(ns_gpu* g, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t cap,
               int64_t p0, float* out, float* scratch) {
    NS_TRY
    return rows_f32(g, "ns_nh_attn", q, qs, kc, vc, T, Hq, Hkv, D, cap, p0, out, scratch);
    NS_CATCH("ns_nh_attn")
}

int ns_nhs_attn_decode_supported(int64_t T, int64_t Hq, int64_t Hkv, int64_t D) { return T >= 1 && T <= 8 && D == 128 && shape_ok(Hq, Hkv, D); }

int64_t ns_nhs_attn_decode_scratch(int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t p0) { return decode_scratch(T, Hq, Hkv, D, p0); }

int ns_nhs_attn_decode(ns_gpu* g, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                       int64_t cap, int64_t p0, float* out, float* scratch) {
    NS_TRY
    return decode_f32(g, "ns_nhs_attn_decode", q, qs, kc, vc, T, Hq, Hkv, D, cap, p0, out, scratch);
    NS_CATCH("ns_nhs_attn_decode")
}

int ns_b200_kv_store_batch(ns_gpu* g, const float* k, int64_t ks, int64_t k_seq, const float* v, int64_t vs, int64_t v_seq, const ns_b200_seq* seqs,
                           int64_t B, int64_t T, int64_t Hkv, int64_t D) {
    NS_TRY
    const char* name = "ns_b200_kv_store_batch";
    if (ns_enter(g, name)) return -1;
    if (B < 1 || T < 1) return 0;
    if (!k || !v || !seqs || Hkv < 1) return ns_fail(std::string(name) + ": a null buffer");
    if (D % 8 != 0 || ks % 4 != 0 || vs % 4 != 0 || k_seq % 4 != 0 || v_seq % 4 != 0 || ((uintptr_t) k & 15) != 0 || ((uintptr_t) v & 15) != 0)
        return ns_fail(std::string(name) + ": head width a multiple of 8, rows 16-byte aligned");
    return ns_launch_kv_store_batch(g, k, ks, k_seq, v, vs, v_seq, seqs, B, T, Hkv, D);
    NS_CATCH("ns_b200_kv_store_batch")
}

int64_t ns_b200_gqa_decode_scratch(int64_t B, int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t max_kv) {
    if (B < 1 || T < 1 || Hkv < 1 || max_kv < 1) return 0;
    const int64_t ns = ns_dec_splits_bound(max_kv, Hkv);   // shorter sequences of the batch may need more splits than the longest
    return ns > 1 ? B * T * Hq * ns * (D + 2) : 0;
}

int ns_b200_gqa_decode(ns_gpu* g, const void* q, int64_t qs, int64_t q_seq, const ns_b200_seq* seqs, int64_t B, int64_t T, int64_t Hq, int64_t Hkv,
                       int64_t D, int64_t max_kv, void* out, float* scratch) {
    NS_TRY
    const char* name = "ns_b200_gqa_decode";
    if (ns_enter(g, name)) return -1;
    if (B < 1) return 0;
    if (T < 1 || T > 8 || !shape_ok(Hq, Hkv, D)) return ns_fail(std::string(name) + ": 1..8 rows, heads of 128 or 256, 1..16 query heads a key head");
    if (max_kv < T || max_kv >= ((int64_t) 1 << 31)) return ns_fail(std::string(name) + ": max_kv between T and 2^31");
    if (qs % 8 != 0 || q_seq % 8 != 0 || ((uintptr_t) q & 15) != 0) return ns_fail(std::string(name) + ": query rows 16-byte aligned");
    if (!q || !seqs || !out) return ns_fail(std::string(name) + ": a null buffer");
    const int64_t ns = ns_dec_splits_bound(max_kv, Hkv);
    if (ns > 1 && !scratch) return ns_fail(std::string(name) + ": no scratch");
    GqaDecodeArgs a{};
    a.q = q;
    a.qs = qs;
    a.q_seq = q_seq;
    a.seqs = seqs;
    a.out = out;
    a.part = scratch;
    a.B = B, a.T = T, a.Hq = Hq, a.Hkv = Hkv, a.D = D;
    a.ns_max = ns;
    a.q_f32 = 0, a.out_f32 = 0;
    return ns_launch_gqa_decode(g, a, name);
    NS_CATCH("ns_b200_gqa_decode")
}

// ---- one long context split over several GPUs by key ranges (the log-sum-exp combine is the path's one exchange) -------

int64_t ns_b200_kvsplit_mailbox_bytes(int64_t nranks, int64_t T, int64_t Hq, int64_t D) {
    if (nranks < 1 || T < 1 || Hq < 1 || D < 1) return 0;
    return ns_mbox_bytes((int) nranks, T * Hq, D);
}

int64_t ns_b200_kvsplit_scratch(int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t kv_local) {
    if (T < 1 || Hkv < 1 || kv_local < 1) return 0;   // a rank without keys needs none
    // every row keeps its partial, also with one split; rows below the last see fewer keys of the last rank's slice and
    // may need more splits than kv_local itself does, hence the bound
    return T * Hq * ns_dec_splits_bound(kv_local, Hkv) * (D + 2);
}

int ns_b200_kvsplit_decode(ns_gpu* g, const void* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                           int64_t kv_local, int64_t key_base, int64_t p0, float* scratch, int64_t rank, int64_t nranks, void* const* mailboxes,
                           int64_t epoch) {
    NS_TRY
    const char* name = "ns_b200_kvsplit_decode";
    if (ns_enter(g, name)) return -1;
    if (T < 1 || T > 8 || !shape_ok(Hq, Hkv, D)) return ns_fail(std::string(name) + ": 1..8 rows, heads of 128 or 256, 1..16 query heads a key head");
    if (nranks < 1 || nranks > 64 || rank < 0 || rank >= nranks) return ns_fail(std::string(name) + ": rank within 1..64 ranks");
    if (kv_local < 0 || kv_local >= ((int64_t) 1 << 31) || key_base < 0 || p0 < 0 || p0 + T >= ((int64_t) 1 << 40))
        return ns_fail(std::string(name) + ": a key range of 0 .. 2^31 keys");
    if (epoch < 0) return ns_fail(std::string(name) + ": epochs count from 1 (0: the mailbox's own counter)");
    if (qs % 8 != 0 || ((uintptr_t) q & 15) != 0) return ns_fail(std::string(name) + ": query rows 16-byte aligned");
    // a rank past the end of a short context (kv_local 0) streams nothing and still publishes its empty partials, so the
    // others' combines do not wait for it; it needs no caches and no scratch
    if (!q || !mailboxes || (kv_local > 0 && (!kc || !vc || !scratch))) return ns_fail(std::string(name) + ": a null buffer");
    GqaDecodeArgs a{};
    a.q = q;
    a.qs = qs;
    a.q_seq = 0;
    a.seqs = nullptr;
    a.one = ns_b200_seq{kc, vc, kv_local, p0 - key_base};   // the slice's capacity bounds what each row sees of it
    a.out = nullptr;
    a.part = scratch;
    a.B = 1, a.T = T, a.Hq = Hq, a.Hkv = Hkv, a.D = D;
    a.ns_max = std::max<int64_t>(1, ns_dec_splits_bound(kv_local, Hkv));
    a.q_f32 = 0, a.out_f32 = 0;
    a.mailboxes = (float* const*) mailboxes;
    a.rank = (int) rank;
    a.nranks = (int) nranks;
    a.epoch = epoch;
    return ns_launch_gqa_decode(g, a, name);
    NS_CATCH("ns_b200_kvsplit_decode")
}

int ns_b200_kvsplit_partial(ns_gpu* g, const void* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                            int64_t kv_local, int64_t key_base, int64_t p0, float* scratch, float* part) {
    NS_TRY
    const char* name = "ns_b200_kvsplit_partial";
    if (ns_enter(g, name)) return -1;
    if (T < 1 || T > 8 || !shape_ok(Hq, Hkv, D)) return ns_fail(std::string(name) + ": 1..8 rows, heads of 128 or 256, 1..16 query heads a key head");
    if (kv_local < 0 || kv_local >= ((int64_t) 1 << 31) || key_base < 0 || p0 < 0 || p0 + T >= ((int64_t) 1 << 40))
        return ns_fail(std::string(name) + ": a key range of 0 .. 2^31 keys");
    if (qs % 8 != 0 || ((uintptr_t) q & 15) != 0 || ((uintptr_t) part & 7) != 0) return ns_fail(std::string(name) + ": query rows 16-byte aligned");
    if (!q || !part || (kv_local > 0 && (!kc || !vc || !scratch))) return ns_fail(std::string(name) + ": a null buffer");
    GqaDecodeArgs a{};
    a.q = q;
    a.qs = qs;
    a.one = ns_b200_seq{kc, vc, kv_local, p0 - key_base};
    a.part = scratch;
    a.B = 1, a.T = T, a.Hq = Hq, a.Hkv = Hkv, a.D = D;
    a.ns_max = std::max<int64_t>(1, ns_dec_splits_bound(kv_local, Hkv));
    a.local_part = part;
    return ns_launch_gqa_decode(g, a, name);
    NS_CATCH("ns_b200_kvsplit_partial")
}

int ns_b200_kvsplit_merge(ns_gpu* g, const float* parts, int64_t nranks, int64_t T, int64_t Hq, int64_t D, void* out) {
    NS_TRY
    const char* name = "ns_b200_kvsplit_merge";
    if (ns_enter(g, name)) return -1;
    if (!parts || !out) return ns_fail(std::string(name) + ": a null buffer");
    if (nranks < 1 || nranks > 64 || T < 1 || T > 8 || Hq < 1) return ns_fail(std::string(name) + ": 1..64 ranks, 1..8 rows");
    return ns_launch_gqa_merge_ranks(g, parts, (int) nranks, T, Hq, D, out, 0, name);
    NS_CATCH("ns_b200_kvsplit_merge")
}

int ns_b200_kvsplit_step(ns_gpu* g, const void* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                         int64_t kv_local, int64_t key_base, int64_t p0, float* scratch, int64_t rank, int64_t nranks, void* const* mailboxes,
                         void* own_mailbox, int64_t epoch, int64_t wait_us, void* out) {
    NS_TRY
    const char* name = "ns_b200_kvsplit_step";
    if (ns_enter(g, name)) return -1;
    if (T < 1 || T > 8 || !shape_ok(Hq, Hkv, D)) return ns_fail(std::string(name) + ": 1..8 rows, heads of 128 or 256, 1..16 query heads a key head");
    if (nranks < 1 || nranks > 64 || rank < 0 || rank >= nranks) return ns_fail(std::string(name) + ": rank within 1..64 ranks");
    if (kv_local < 0 || kv_local >= ((int64_t) 1 << 31) || key_base < 0 || p0 < 0 || p0 + T >= ((int64_t) 1 << 40))
        return ns_fail(std::string(name) + ": a key range of 0 .. 2^31 keys");
    if (epoch < 0) return ns_fail(std::string(name) + ": epochs count from 1 (0: the mailbox's own counter)");
    // a line's tag is the step number's low 32 bits, and a mailbox starts zeroed: a step whose tag would be 0 could take a
    // line nobody wrote for one that arrived
    if (epoch != 0 && (uint32_t) epoch == 0) return ns_fail(std::string(name) + ": a step number whose low 32 bits are zero (restart the epochs from 1)");
    if (wait_us < 1 || wait_us > 2000000) return ns_fail(std::string(name) + ": a wait of 1 us .. 2 s");
    if (qs % 8 != 0 || ((uintptr_t) q & 15) != 0) return ns_fail(std::string(name) + ": query rows 16-byte aligned");
    if (!q || !mailboxes || !own_mailbox || !out || (kv_local > 0 && (!kc || !vc || !scratch))) return ns_fail(std::string(name) + ": a null buffer");
    GqaDecodeArgs a{};
    a.q = q;
    a.qs = qs;
    a.q_seq = 0;
    a.seqs = nullptr;
    a.one = ns_b200_seq{kc, vc, kv_local, p0 - key_base};
    a.out = out;
    a.part = scratch;
    a.B = 1, a.T = T, a.Hq = Hq, a.Hkv = Hkv, a.D = D;
    a.ns_max = std::max<int64_t>(1, ns_dec_splits_bound(kv_local, Hkv));
    a.q_f32 = 0, a.out_f32 = 0;
    a.mailboxes = (float* const*) mailboxes;
    a.rank = (int) rank;
    a.nranks = (int) nranks;
    a.epoch = epoch;
    a.fused_spins = wait_us * 10;
    a.own_mailbox = (float*) own_mailbox;
    return ns_launch_gqa_decode(g, a, name);
    NS_CATCH("ns_b200_kvsplit_step")
}

int ns_b200_kvsplit_combine(ns_gpu* g, void* mailbox, int64_t nranks, int64_t T, int64_t Hq, int64_t D, int64_t epoch, int64_t wait_us,
                            void* out) {
    NS_TRY
    const char* name = "ns_b200_kvsplit_combine";
    if (ns_enter(g, name)) return -1;
    if (!mailbox || !out) return ns_fail(std::string(name) + ": a null buffer");
    if (nranks < 1 || nranks > 64 || T < 1 || T > 8 || Hq < 1 || epoch < 0) return ns_fail(std::string(name) + ": 1..64 ranks, 1..8 rows, epochs from 1");
    if (wait_us < 1 || wait_us > 2000000) return ns_fail(std::string(name) + ": a wait of 1 us .. 2 s");
    return ns_launch_gqa_combine(g, (float*) mailbox, (int) nranks, T, Hq, D, epoch, wait_us * 10, out, 0, name);
    NS_CATCH("ns_b200_kvsplit_combine")
}

int ns_b200_ipc_export(ns_gpu* g, void* ptr, void* handle64) {
    if (ns_enter(g, "ns_b200_ipc_export")) return -1;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    if (!ptr || !handle64) return ns_fail("ns_b200_ipc_export: a null argument");
    NS_CUDA(cudaIpcGetMemHandle((cudaIpcMemHandle_t*) handle64, ptr), "ns_b200_ipc_export");
    return 0;
}

int ns_b200_ipc_open(ns_gpu* g, const void* handle64, void** out) {
    if (ns_enter(g, "ns_b200_ipc_open")) return -1;
    if (!handle64 || !out) return ns_fail("ns_b200_ipc_open: a null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    NS_CUDA(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess), "ns_b200_ipc_open");
    return 0;
}

int ns_b200_ipc_close(ns_gpu* g, void* ptr) {
    if (ns_enter(g, "ns_b200_ipc_close")) return -1;
    if (ptr) NS_CUDA(cudaIpcCloseMemHandle(ptr), "ns_b200_ipc_close");
    return 0;
}

}  // extern "C"
