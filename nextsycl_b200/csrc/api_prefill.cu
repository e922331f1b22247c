// api_prefill.cu: the C-ABI entry points of prompt (prefill) attention: the reference's names with fp32 rows, and the
// native 16-bit ones. Argument checks, then flash_prefill.cu's launcher.
#include "kernels.cuh"

namespace {

const float LOG2E = 1.4426950408889634f;

bool prefill_shape(int64_t Hq, int64_t Hkv, int64_t D) { return (D == 128 || D == 256) && Hkv > 0 && Hq > 0 && Hq % Hkv == 0; }

}  // namespace

// fp32 rows in, fp32 rows out, fp16 caches [Hkv][cap][D]: the queries are scaled by 1/sqrt(D) log2(e) and rounded to
// fp16 into the GPU's kept staging buffer (what the reference does as it stages them, silo/attn.cpp:112,147), then the
// tensor-core kernel runs with a unit softmax scale.
int ns_prefill_f32(ns_gpu* g, const char* name, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv,
                   int64_t D, int64_t cap, int64_t p0, float* out) {
    if (ns_enter(g, name)) return -1;
    if (T <= 0) return 0;
    if (!prefill_shape(Hq, Hkv, D)) return ns_fail(std::string(name) + ": heads of 128 or 256, a whole number of query heads a key head");
    if (p0 < 0 || p0 + T > cap) return ns_fail(std::string(name) + ": past the cache's capacity");
    if (p0 + T >= ((int64_t) 1 << 31) || T * Hq * D >= ((int64_t) 1 << 40)) return ns_fail(std::string(name) + ": positions below 2^31");
    if (!q || !kc || !vc || !out) return ns_fail(std::string(name) + ": a null buffer");
    if (qs % 4 != 0 || ((uintptr_t) q & 15) != 0 || ((uintptr_t) kc & 15) != 0 || ((uintptr_t) vc & 15) != 0 || ((uintptr_t) out & 15) != 0)
        return ns_fail(std::string(name) + ": rows 16-byte aligned");
    void* qh = nullptr;
    if (ns_kept(g, (size_t) (T * Hq * D * 2), &qh)) return -1;
    if (ns_launch_scale_to_f16(g, q, qs, qh, Hq * D, T, Hq * D, 1.0f / sqrtf((float) D) * LOG2E)) return -1;
    FlashPrefillArgs a{};
    a.q = qh;
    a.q_row = Hq * D;
    a.k = kc;
    a.k_key = D;
    a.k_head = cap * D;
    a.v = vc;
    a.v_key = D;
    a.v_head = cap * D;
    a.out = out;
    a.status = g->status_dev;
    a.T = T, a.Hq = Hq, a.Hkv = Hkv, a.Dqk = D, a.Dv = D;
    a.p0 = p0;
    a.kv_len = p0 + T;
    a.scale_log2 = 1.0f;
    a.bf16 = 0;
    a.out_f32 = 1;
    return ns_launch_flash_prefill(g, a, name);
}

extern "C" {

int ns_q35_attn_prompt_supported(int64_t T, int64_t Hq, int64_t Hkv, int64_t D) { return T > 8 && prefill_shape(Hq, Hkv, D); }

int ns_q35_attn_prompt(ns_gpu* g, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                       int64_t cap, int64_t p0, float* out) {
    NS_TRY
    if (!ns_q35_attn_prompt_supported(T, Hq, Hkv, D)) return ns_fail("ns_q35_attn_prompt: more than 8 rows, heads of 128 or 256");
    return ns_prefill_f32(g, "ns_q35_attn_prompt", q, qs, kc, vc, T, Hq, Hkv, D, cap, p0, out);
    NS_CATCH("ns_q35_attn_prompt")
}

int ns_q35_attn_prompt_kv(ns_gpu* g, int kt, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv,
                          int64_t D, int64_t cap, int64_t p0, float* out) {
    NS_TRY
    const char* name = "ns_q35_attn_prompt_kv";
    if (!ns_q35_attn_prompt_supported(T, Hq, Hkv, D)) return ns_fail(std::string(name) + ": more than 8 rows, heads of 128 or 256");
    if (kt == 0) return ns_prefill_f32(g, name, q, qs, kc, vc, T, Hq, Hkv, D, cap, p0, out);
    // q8_0 / q4_0 caches (heads of 256): expanded to the fp16 values the reference's reader produces (silo/attn.cpp:49-78)
    // in a kept buffer [Hkv][p0+T][256] each; a prompt pass is bound by its products, so the extra pass over the cache is small
    if (kt != 1 && kt != 2) return ns_fail(std::string(name) + ": a cache form 0 (half), 1 (q8_0) or 2 (q4_0)");
    if (ns_enter(g, name)) return -1;
    if (D != 256) return ns_fail(std::string(name) + ": quantised caches have heads of 256");
    if (!kc || !vc || p0 < 0 || p0 + T > cap) return ns_fail(std::string(name) + ": past the cache's capacity");
    const int64_t n = p0 + T, one = (Hkv * n * 256 * 2 + 255) / 256 * 256;
    void* kept = nullptr;
    if (ns_kept_kv(g, (size_t) (2 * one), &kept)) return -1;
    void* kh = kept;
    void* vh = (uint8_t*) kept + one;
    if (ns_launch_kv_dequant(g, kt, kc, Hkv, cap, n, kh, name) || ns_launch_kv_dequant(g, kt, vc, Hkv, cap, n, vh, name)) return -1;
    return ns_prefill_f32(g, name, q, qs, kh, vh, T, Hq, Hkv, D, n, p0, out);
    NS_CATCH("ns_q35_attn_prompt_kv")
}

int ns_nhs_attn_prompt_supported(int64_t T, int64_t Hq, int64_t Hkv, int64_t D) { return T > 8 && D == 128 && prefill_shape(Hq, Hkv, D); }

int ns_nhs_attn_prompt(ns_gpu* g, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                       int64_t cap, int64_t p0, float* out) {
    NS_TRY
    if (!ns_nhs_attn_prompt_supported(T, Hq, Hkv, D)) return ns_fail("ns_nhs_attn_prompt: more than 8 rows, heads of 128");
    return ns_prefill_f32(g, "ns_nhs_attn_prompt", q, qs, kc, vc, T, Hq, Hkv, D, cap, p0, out);
    NS_CATCH("ns_nhs_attn_prompt")
}

int ns_b200_gqa_prefill(ns_gpu* g, int dtype, const void* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                        int64_t cap, int64_t p0, void* out) {
    NS_TRY
    const char* name = "ns_b200_gqa_prefill";
    if (ns_enter(g, name)) return -1;
    if (T <= 0) return 0;
    if (dtype != 0 && dtype != 1) return ns_fail(std::string(name) + ": dtype 0 (fp16) or 1 (bf16)");
    if (!prefill_shape(Hq, Hkv, D) || (D == 256 && dtype == 1)) return ns_fail(std::string(name) + ": heads of 128 (fp16, bf16) or 256 (fp16)");
    if (p0 < 0 || p0 + T > cap || p0 + T >= ((int64_t) 1 << 31)) return ns_fail(std::string(name) + ": past the cache's capacity");
    if (!q || !kc || !vc || !out) return ns_fail(std::string(name) + ": a null buffer");
    if (qs % 8 != 0 || ((uintptr_t) q & 15) != 0 || ((uintptr_t) kc & 15) != 0 || ((uintptr_t) vc & 15) != 0 || ((uintptr_t) out & 15) != 0)
        return ns_fail(std::string(name) + ": rows 16-byte aligned");
    FlashPrefillArgs a{};
    a.q = q;
    a.q_row = qs;
    a.k = kc;
    a.k_key = D;
    a.k_head = cap * D;
    a.v = vc;
    a.v_key = D;
    a.v_head = cap * D;
    a.out = out;
    a.status = g->status_dev;
    a.T = T, a.Hq = Hq, a.Hkv = Hkv, a.Dqk = D, a.Dv = D;
    a.p0 = p0;
    a.kv_len = p0 + T;
    a.scale_log2 = 1.0f / sqrtf((float) D) * LOG2E;
    a.bf16 = dtype;
    a.out_f32 = 0;
    return ns_launch_flash_prefill(g, a, name);
    NS_CATCH("ns_b200_gqa_prefill")
}

int ns_b200_mla_prefill(ns_gpu* g, const void* q, int64_t q_tok, const void* k, int64_t k_tok, const void* v, int64_t v_tok, int64_t T, int64_t H,
                        int64_t p0, float scale, void* out) {
    NS_TRY
    const char* name = "ns_b200_mla_prefill";
    if (ns_enter(g, name)) return -1;
    if (T <= 0) return 0;
    if (H < 1) return ns_fail(std::string(name) + ": at least one head");
    if (p0 < 0 || p0 + T >= ((int64_t) 1 << 31)) return ns_fail(std::string(name) + ": positions below 2^31");
    if (!q || !k || !v || !out) return ns_fail(std::string(name) + ": a null buffer");
    if (q_tok % 8 != 0 || k_tok % 8 != 0 || v_tok % 8 != 0 || q_tok < H * 192 || k_tok < H * 192 || v_tok < H * 128)
        return ns_fail(std::string(name) + ": token strides of at least H heads, multiples of 8 elements");
    if (((uintptr_t) q & 15) != 0 || ((uintptr_t) k & 15) != 0 || ((uintptr_t) v & 15) != 0 || ((uintptr_t) out & 15) != 0)
        return ns_fail(std::string(name) + ": rows 16-byte aligned");
    FlashPrefillArgs a{};
    a.q = q;
    a.q_row = q_tok;
    a.k = k;
    a.k_key = k_tok;
    a.k_head = 192;
    a.v = v;
    a.v_key = v_tok;
    a.v_head = 128;
    a.out = out;
    a.status = g->status_dev;
    a.T = T, a.Hq = H, a.Hkv = H, a.Dqk = 192, a.Dv = 128;
    a.p0 = p0;
    a.kv_len = p0 + T;
    a.scale_log2 = scale * LOG2E;
    a.bf16 = 1;
    a.out_f32 = 0;
    return ns_launch_flash_prefill(g, a, name);
    NS_CATCH("ns_b200_mla_prefill")
}

}  // extern "C"
