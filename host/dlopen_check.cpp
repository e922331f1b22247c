// dlopen_check.cpp: opens the library the way the reference's loader does and binds, by name, every symbol the engines'
// tables ask for on the attention path (crates/sys/src/lib.rs:200-236; llm/qwen35/src/ffi.rs:111-121,155-160,204-208;
// llm/glm5next/src/ffi.rs:33-54; llm/deepseek2/src/ffi.rs:37-39) plus the native entry points. Exit code 0 when all bind.
// With a GPU present (argument "--run") it also runs a 4-element round trip through ns_alloc / ns_copy_*.
#include <cstdio>
#include <cstring>

#include "nextsycl_host.hpp"

static const char* kCore[] = {"ns_last_error", "ns_version",   "ns_gpu_count", "ns_gpu_name",    "ns_gpu_pci",  "ns_gpu_units", "ns_gpu_open",
                              "ns_gpu_close",  "ns_gpu_queue", "ns_gpu_memory", "ns_alloc",      "ns_free",     "ns_alloc_host", "ns_free_host",
                              "ns_copy_to",    "ns_copy_from", "ns_copy_dev",  "ns_copy_2d",     "ns_mark",     "ns_stream_copy", "ns_await",
                              "ns_stamp",      "ns_elapsed",   "ns_fill",      "ns_sync",        "ns_copy_peer"};
static const char* kEngines[] = {
    // qwen35 (and its silo)
    "ns_q35_kv_store", "ns_q35_attn_scratch", "ns_q35_attn", "ns_q35_attn_prompt_supported", "ns_q35_attn_prompt", "ns_q35_attn_prompt_kv",
    "ns_q35_attn_decode_supported", "ns_q35_attn_decode_scratch", "ns_q35_attn_decode", "ns_q35_attn_decode_kv", "ns_q35_graph_begin",
    "ns_q35_graph_end", "ns_q35_graph_launch", "ns_q35_graph_free",
    // nemotronh (the D = 128 copies)
    "ns_nh_attn_scratch", "ns_nh_attn", "ns_nhs_attn_prompt_supported", "ns_nhs_attn_prompt", "ns_nhs_attn_decode_supported",
    "ns_nhs_attn_decode_scratch", "ns_nhs_attn_decode",
    // glm5next
    "ns_mla_attend", "ns_mla_attend_sel", "ns_mla_attend_sel_q8", "ns_mla_cells", "ns_softmax_masked", "ns_to_f16", "ns_to_q8row", "ns_gather_q8_h",
    "ns_gather_h", "ns_gemm_batch_h", "ns_idx_pool", "ns_idx_score", "ns_topk",
    // deepseek2
    "ns_ds2_mla_decode", "ns_ds2_mla_decode_q6k", "ns_ds2_rope", "ns_ds2_kv_store",
    // qwen35: the step before attention
    "ns_q35_qk_norm_rope", "ns_q35_qk_norm_rope_pos", "ns_q35_rope", "ns_b200_qkv_prepare",
    // qwen35 quantised caches
    "ns_q35_kv_store_q", "ns_q35_fwht32", "ns_q35_attn_probs",
    // deepseek41
    "ns_ds41_attend", "ns_ds41_attend_xmx_supported", "ns_ds41_attend_xmx", "ns_ds41_ring_put", "ns_ds41_rows_f16", "ns_ds41_kv_post", "ns_ds41_att_post", "ns_ds41_idx_score", "ns_ds41_block_max", "ns_ds41_idx_score_cand",
    "ns_ds41_cand_pos", "ns_ds41_cand_mask",
    // native
    "ns_b200_gqa_decode_scratch", "ns_b200_gqa_decode", "ns_b200_gqa_prefill", "ns_b200_mla_prefill", "ns_b200_mla_decode_scratch", "ns_b200_mla_decode",
    "ns_b200_kvsplit_mailbox_bytes", "ns_b200_kvsplit_scratch", "ns_b200_kvsplit_decode", "ns_b200_kvsplit_combine", "ns_b200_kvsplit_step", "ns_b200_mla_kvsplit_scratch", "ns_b200_mla_kvsplit_decode", "ns_b200_mla_kvsplit_combine", "ns_b200_kvsplit_partial", "ns_b200_kvsplit_merge", "ns_b200_ipc_export",
    "ns_b200_ipc_open", "ns_b200_ipc_close", "ns_b200_kv_store_batch", "ns_b200_gqa_decode_static"};

int main(int argc, char** argv) {
    try {
        nextsycl::Api api(argc > 1 && std::strcmp(argv[1], "--run") != 0 ? argv[1] : "dist/libnextsycl-llm.so");
        int missing = 0;
        for (const char* n : kCore)
            if (!api.symbol(n)) std::printf("missing core symbol %s\n", n), ++missing;
        for (const char* n : kEngines)
            if (!api.symbol(n)) std::printf("missing engine symbol %s\n", n), ++missing;
        std::printf("%s: %zu core + %zu engine symbols, %d missing; %d GPU(s)\n", api.path().c_str(), sizeof(kCore) / sizeof(*kCore),
                    sizeof(kEngines) / sizeof(*kEngines), missing, api.gpu_count());
        if (missing) return 1;
        // a size query needs no device: the reference's own shape answers with scratch for a long context
        auto scratch = api.need<int64_t (*)(int64_t, int64_t, int64_t, int64_t, int64_t)>("ns_q35_attn_decode_scratch");
        if (scratch(1, 24, 4, 256, 100000) <= 0 || scratch(1, 24, 4, 256, 10) != 0) return std::printf("scratch query wrong\n"), 1;
        bool run = false;
        for (int i = 1; i < argc; ++i) run = run || std::strcmp(argv[i], "--run") == 0;
        if (run) {
            nextsycl::Gpu gpu(api, 0);
            nextsycl::Arena arena(gpu, 1 << 20);
            nextsycl::DevBuf b = arena.f32(4);
            const float in[4] = {1, 2, 3, 4};
            float out[4] = {};
            b.write(in, sizeof(in));
            b.read(out, sizeof(out));
            if (std::memcmp(in, out, sizeof(in)) != 0) return std::printf("round trip differs\n"), 1;
            try {
                b.bounds(8, 16);
                return std::printf("bounds not checked\n"), 1;
            } catch (const std::runtime_error&) {
            }
            std::printf("round trip ok\n");
        }
        return 0;
    } catch (const std::exception& e) {
        std::printf("error: %s\n", e.what());
        return 2;
    }
}
