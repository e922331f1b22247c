/* ns_attn.h: the attention entry points of libnextsycl-llm.so on CUDA (sm_100a).
 *
 * Two groups:
 *  1. The reference's own symbols, with identical signatures, so the per-model engines' dlsym tables
 *     (llm/qwen35/src/ffi.rs:155-160,204-208; llm/glm5next/src/ffi.rs:33-54; llm/deepseek2/src/ffi.rs:37-39) bind
 *     unchanged: float32 queries and outputs, fp16 caches, every size an int64_t, work queued on the ns_gpu's compute
 *     stream, 0 or -1 (+ ns_last_error).
 *  2. Native ns_b200_* entry points: fp16 / bf16 queries and outputs, a batch dimension, lengths read from device
 *     memory (so a decode step can be replayed as a CUDA graph), and the multi-GPU split-KV combine.
 *
 * Cache layouts are the reference's: GQA keys and values in separate fp16 buffers [Hkv][cap][D], element
 * (h*cap + pos)*D + d (kernels/llm/qwen35/q35.cpp:580-584); the deepseek2 latent cache one fp16 row
 * [512 latent | 64 rotated] per token (kernels/llm/deepseek2/ds2.cpp:99-107).
 */
#ifndef NS_ATTN_H
#define NS_ATTN_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ns_gpu ns_gpu;

/* ================= 1. reference-compatible symbols ================= */

/* kernels/llm/qwen35/q35.h:55-57 - fp32 rows k [T][Hkv*D] (ks floats apart) and v (vs apart) into the fp16 caches at
 * positions p0 .. p0+T-1. -1 when p0+T > cap. */
int ns_q35_kv_store(ns_gpu* g, const float* k, int64_t ks, const float* v, int64_t vs, int64_t T, int64_t Hkv, int64_t D, int64_t cap, int64_t p0,
                    void* kc, void* vc);

/* kernels/llm/qwen35/q35.h:62-66 - causal attention of rows q [T][Hq*D] (qs floats apart) at positions p0.. against the
 * caches; out [T][Hq*D]; scratch of ns_q35_attn_scratch floats (0: none needed, may be null). The reference covers
 * D 256 with 2/4/6/8 query heads a key head and D 128 with one; this library covers D 128 and 256 with any whole
 * number of query heads a key head up to 16. */
int64_t ns_q35_attn_scratch(int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t p0);
int ns_q35_attn(ns_gpu* g, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t cap,
                int64_t p0, float* out, float* scratch);

/* kernels/llm/qwen35/silo/silo.h:43-48 - prompt rows (more than 8) on the tensor cores: out [T][Hq*D] = causal
 * softmax(q k^T / sqrt(D)) v for rows at positions p0.. against the fp16 caches. `_supported` is widened from the
 * reference's (D 256, 6 query heads a key head) to D 128 and 256 with any whole number of query heads a key head. */
int ns_q35_attn_prompt_supported(int64_t T, int64_t Hq, int64_t Hkv, int64_t D);
int ns_q35_attn_prompt(ns_gpu* g, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                       int64_t cap, int64_t p0, float* out);
int ns_q35_attn_prompt_kv(ns_gpu* g, int kt, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv,
                          int64_t D, int64_t cap, int64_t p0, float* out);

/* kernels/llm/qwen35/silo/silo.h:49-59 - decode rows (1..8), each at its own position p0+t; a row's result is the same
 * whatever rows share its pass. `_supported` is widened from the reference's (D 256, 6 heads a key head) to D 128 / 256
 * with 1..16 query heads a key head. kt (both _kv entry points): the cache's form, 0 fp16, 1 q8_0, 2 q4_0 (heads of 256;
 * rows as ns_q35_kv_store_q writes them). Decode streams a quantised cache as it lies and expands the raw rows in
 * registers, on their way into the tensor-core fragments, to exactly the fp16 values the reference's reader kv_load8
 * produces (silo/attn.cpp:49-78); a prompt pass, bound by its products, first expands the rows it reads into a buffer
 * the library keeps and runs the fp16 kernel on that. */
int ns_q35_attn_decode_supported(int64_t T, int64_t Hq, int64_t Hkv, int64_t D);
int64_t ns_q35_attn_decode_scratch(int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t p0);
int ns_q35_attn_decode(ns_gpu* g, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                       int64_t cap, int64_t p0, float* out, float* scratch);
int ns_q35_attn_decode_kv(ns_gpu* g, int kt, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv,
                          int64_t D, int64_t cap, int64_t p0, float* out, float* scratch);

/* kernels/llm/qwen35/q35.h:34-38 - one query row q [Hq*D] over the first n keys of the key cache (its form kt: 0 fp16, 1 q8_0,
 * 2 q4_0; heads of 256): each head's softmax weights (scale 1/sqrt(D)), per key their mean over the heads (mode 0) or their
 * largest (mode 1), ADDED to out [n]; scratch [Hq][2] receives each head's (maximum, sum). */
int ns_q35_attn_probs(ns_gpu* g, int kt, const float* q, const void* kc, int64_t Hq, int64_t Hkv, int64_t D, int64_t cap, int64_t n, int mode,
                      float* scratch, float* out);

/* kernels/llm/qwen35/q35.h:39-46 - the quantised caches' writer and rotation. ns_q35_kv_store_q: fp32 rows k, v
 * [T][Hkv*256] into caches [Hkv][cap][272 or 144 bytes] as q8_0 (kt 1: 256 int8 then 8 fp16 scales) or q4_0 (kt 2: 8
 * blocks of 16 bytes, value j low / j+16 high, then 8 fp16 scales; ggml's quantize_row_q4_0), q35.cpp:281-326.
 * ns_q35_fwht32: each block of 32 of rows x [rows][n] (stride floats apart) through the normalised 32-point
 * Walsh-Hadamard transform, its own inverse (q35.cpp:328-348): the rotation applied to q and k (and undone on the output
 * for v) when a quantised cache is rotated. */
int ns_q35_kv_store_q(ns_gpu* g, int kt, const float* k, int64_t ks, const float* v, int64_t vs, int64_t T, int64_t Hkv, int64_t D, int64_t cap,
                      int64_t p0, void* kc, void* vc);
int ns_q35_fwht32(ns_gpu* g, float* x, int64_t rows, int64_t n, int64_t stride);

/* kernels/llm/qwen35/q35.h:16-24,59-61 - the step before attention. Per (row t, head h): x = src[t*ss + h*hs .. + D] RMS-normed
 * (weight w [D], eps), then rotate-half rotary positions on its first n_rot features (pairs i, i + n_rot/2; angle (p0 + t)
 * theta^(-2i / n_rot)), into dst[t*ds + h*D]. _pos: each row at its own positions pos [T][3] (t, h, w), pair k turning by
 * the one Qwen3-VL's interleaved sections (s0, s1, s2) choose. ns_q35_rope: the same without the norm. fp32 throughout;
 * src and dst may be the same rows. */
int ns_q35_qk_norm_rope(ns_gpu* g, const float* src, int64_t ss, int64_t hs, float* dst, int64_t ds, int64_t T, int64_t H, int64_t D, const float* w,
                        float eps, int64_t n_rot, float theta, int64_t p0);
int ns_q35_qk_norm_rope_pos(ns_gpu* g, const float* src, int64_t ss, int64_t hs, float* dst, int64_t ds, int64_t T, int64_t H, int64_t D, const float* w,
                            float eps, int64_t n_rot, float theta, const int32_t* pos, int64_t s0, int64_t s1, int64_t s2);
int ns_q35_rope(ns_gpu* g, const float* src, int64_t ss, int64_t hs, float* dst, int64_t ds, int64_t T, int64_t H, int64_t D, int64_t n_rot, float theta,
                int64_t p0);

/* kernels/llm/deepseek2/ds2.h:20-31 - deepseek2's step before attention. ns_ds2_rope: YaRN rotary positions (ggml's
 * rope_yarn, pairs of adjacent values) in place on x: T rows `row` floats apart, H heads `head` apart, the rotated part
 * n_dims values from float `off` of each head, row t at position pos0 + t; `out` (nullable) also receives the rotated part.
 * ns_ds2_kv_store: the latent cache's rows pos0 .. pos0+T-1 (fp16 [L + R] each) from kv [T][L + R] fp32 - the first L
 * RMS-normed with w (eps), the last R rotated as ns_ds2_rope does at the row's position. */
int ns_ds2_rope(ns_gpu* g, float* x, int64_t T, int64_t H, int64_t row, int64_t head, int64_t off, int64_t n_dims, int64_t pos0, float freq_base,
                float freq_scale, float ext_factor, float mscale, float corr0, float corr1, float* out, int64_t out_row, int64_t out_head);
int ns_ds2_kv_store(ns_gpu* g, const float* kv, const float* w, float eps, uint16_t* cache, int64_t T, int64_t L, int64_t R, int64_t pos0, float freq_base,
                    float freq_scale, float ext_factor, float mscale, float corr0, float corr1);

/* kernels/llm/nemotronh/nh.h:39-44 and silo/nhs.h:63-69 - the same kernels under the nemotronh engine's names (D 128) */
int64_t ns_nh_attn_scratch(int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t p0);
int ns_nh_attn(ns_gpu* g, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t cap,
               int64_t p0, float* out, float* scratch);
int ns_nhs_attn_prompt_supported(int64_t T, int64_t Hq, int64_t Hkv, int64_t D);
int ns_nhs_attn_prompt(ns_gpu* g, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                       int64_t cap, int64_t p0, float* out);
int ns_nhs_attn_decode_supported(int64_t T, int64_t Hq, int64_t Hkv, int64_t D);
int64_t ns_nhs_attn_decode_scratch(int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t p0);
int ns_nhs_attn_decode(ns_gpu* g, const float* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                       int64_t cap, int64_t p0, float* out, float* scratch);

/* kernels/llm/qwen35/q35.h:47-52 - what is queued on the GPU's queue between begin and end is recorded (it does not
 * run), finished by end, replayed by launch as one submission, released by free. Here a CUDA graph captured from the
 * compute stream. Calls that take positions by value bake them in; the native entry points read lengths and step numbers
 * from device memory so that a recorded step stays valid. */
int ns_q35_graph_begin(ns_gpu* g, void** out);
int ns_q35_graph_end(ns_gpu* g, void* h);
int ns_q35_graph_launch(ns_gpu* g, void* h);
void ns_q35_graph_free(void* h);

/* ================= 2. native entry points ================= */

/* One sequence of a decode batch, resident in device memory: its caches ([Hkv][cap][D] fp16 each), their capacity in
 * tokens and the position of the pass's first row (row t sees keys 0 .. p0+t). */
typedef struct ns_b200_seq {
    const void* kc;
    const void* vc;
    int64_t cap;
    int64_t p0;
} ns_b200_seq;

/* A layer's projected rows made ready for attention in one launch (the reference queues ns_q35_qk_norm_rope for q, for k,
 * and ns_q35_kv_store: llm/qwen35/src/engine.rs:1553-1585): q [T][Hq*D] (qs floats apart) and k [T][Hkv*D] (ks apart) are
 * RMS-normed per head (weights wq, wk [D]; null: no norm) and rotated at positions p0 + t; q leaves as fp16 rows q_out
 * [T][Hq*D] (what ns_b200_gqa_decode / ns_b200_gqa_prefill read), k and v [T][Hkv*D] (vs apart) land in the fp16 caches
 * [Hkv][cap][D] at positions p0 .. p0+T-1. The arithmetic is that of the three calls it replaces. */
int ns_b200_qkv_prepare(ns_gpu* g, const float* q, int64_t qs, const float* k, int64_t ks, const float* v, int64_t vs, int64_t T, int64_t Hq, int64_t Hkv,
                        int64_t D, const float* wq, const float* wk, float eps, int64_t n_rot, float theta, int64_t p0, int64_t cap, void* q_out, void* kc,
                        void* vc);

/* The cache writer for a batch in one launch (replaces one ns_q35_kv_store call per sequence, kernels/llm/qwen35/q35.h:55-57,
 * llm/qwen35/src/engine.rs:1577-1585): fp32 rows k, v [B][T][Hkv*D] (ks / vs floats between rows, k_seq / v_seq between
 * sequences) go to positions p0 .. p0+T-1 of each sequence's own fp16 caches, both taken from the DEVICE table seqs [B] that
 * ns_b200_gqa_decode reads, so a recorded step stays valid as the positions advance. One rounding to fp16, as ns_q35_kv_store.
 * A row past its cache's capacity is skipped and the next ns_sync returns -1 (code 803). */
int ns_b200_kv_store_batch(ns_gpu* g, const float* k, int64_t ks, int64_t k_seq, const float* v, int64_t vs, int64_t v_seq, const ns_b200_seq* seqs,
                           int64_t B, int64_t T, int64_t Hkv, int64_t D);

/* Split-KV GQA decode of a batch (replaces one ns_q35_attn_decode call per sequence, llm/qwen35/src/engine.rs:1535,
 * 1596-1600). q [B][T][Hq*D] fp16 (qs elements between rows, q_seq between sequences), seqs a DEVICE array [B],
 * out [B][T][Hq*D] fp16 dense. max_kv bounds every p0+T (it sizes the grid and the scratch; the lengths themselves
 * are read on the device). T 1..8, D 128 or 256, Hq/Hkv 1..16. scratch: ns_b200_gqa_decode_scratch floats. */
int64_t ns_b200_gqa_decode_scratch(int64_t B, int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t max_kv);
int ns_b200_gqa_decode(ns_gpu* g, const void* q, int64_t qs, int64_t q_seq, const ns_b200_seq* seqs, int64_t B, int64_t T, int64_t Hq, int64_t Hkv,
                       int64_t D, int64_t max_kv, void* out, float* scratch);

/* Causal GQA prefill with 16-bit rows in and out (replaces ns_q35_attn_prompt_kv plus the fp32 staging around it,
 * llm/qwen35/src/engine.rs:1586-1593). dtype 0 fp16, 1 bf16: q [T][Hq*D] (qs elements between rows), caches
 * [Hkv][cap][D] and out [T][Hq*D] all of that type; D 128 (both types) or 256 (fp16); row t sees keys 0 .. p0+t. */
int ns_b200_gqa_prefill(ns_gpu* g, int dtype, const void* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                        int64_t cap, int64_t p0, void* out);

/* Non-absorbed MLA prefill in bf16 (no counterpart in the reference, which always runs the absorbed form): q
 * [T][H][192] (128 nope + 64 rope, rotation applied), k [p0+T][H][192], v [p0+T][H][128], out [T][H][128] dense; the
 * token strides q_tok, k_tok, v_tok in elements let a rank pass its slice of heads of a larger tensor. Causal over
 * the p0 cached tokens plus the chunk; `scale` is the softmax scale (1/sqrt(192)). */
int ns_b200_mla_prefill(ns_gpu* g, const void* q, int64_t q_tok, const void* k, int64_t k_tok, const void* v, int64_t v_tok, int64_t T, int64_t H,
                        int64_t p0, float scale, void* out);

/* kernels/llm/deepseek2/ds2.h:33-37 - MLA at decode widths: q [T][H][128 nope + 64 rope] fp32 (the rope part rotated),
 * k_b [H][512][128] and v_b [H][128][512] fp16, the latent cache [n][512 + 64] fp16 (row t sees cells 0 .. pos0+t)
 * -> out [T][H][128]: q~ = k_b q_nope, softmax((q~ . c + q_pe . k_pe) * scale) over the cells, u = sum p c[:512],
 * out = v_b u. Here the middle stage runs on the tensor cores for any context length (the reference switches to a GEMM
 * form past NS_DS2_MLA_FUSED_MAX cells, llm/deepseek2/src/engine.rs:1150-1224); q~ and p are rounded to fp16 as in
 * that GEMM form. Intermediate buffers are the library's own. */
int ns_ds2_mla_decode(ns_gpu* g, const float* q, const uint16_t* kb, const uint16_t* vb, const uint16_t* cache, float* out, int64_t T, int64_t H,
                      int64_t pos0, float scale);

/* kernels/llm/deepseek2/ds2.h:38-41 - the same with kv_b as the model file stores it (Q6_K: 210-byte blocks of 256 values;
 * [H x (128 + 128)] rows of 512: per head its 128 k rows - row i holds k_i[0..511], q~ = sum_i q_nope[i] k_i - then its 128 v
 * rows), decoded where it is read; no fp16 k_b / v_b is kept. The engine takes this form whenever the model keeps kv_b
 * quantised (llm/deepseek2/src/engine.rs:1155). */
int ns_ds2_mla_decode_q6k(ns_gpu* g, const float* q, const void* kvb, const uint16_t* cache, float* out, int64_t T, int64_t H, int64_t pos0, float scale);

/* kernels/llm/glm5next/glm.h:47 - dense causal absorbed MLA over fp32 latents: qa [T][H][L], c [n][L], u [T][H][L] =
 * sum_s softmax(qa . c_s * scale) c_s over s <= pos0+t; exact two-pass softmax in fp32 (L up to 512). */
int ns_mla_attend(ns_gpu* g, const float* qa, const float* c, float* u, int64_t T, int64_t H, int64_t L, int64_t pos0, float scale);
/* kernels/llm/glm5next/glm.h:65-66,79-80 - MLA over each row's selection of cells of the fp16 latent cache [n][512]
 * (or, _q8, of q8 rows: 16 fp16 scales then 512 int8 = 544 bytes): sel_cnt null or sel_cnt[t] < 0 - every earlier
 * token; else 4 tokens of each selected pool sel[t][0 .. sel_cnt[t]) then the row's incomplete pool. qa, u fp32
 * [T][H][512]. The reference runs this on vector units for at most 8 rows and 2,560 cells and falls back to gathers plus
 * oneMKL GEMMs for prompt rows (llm/glm5next/src/engine.rs:1905-1938); here any number of rows takes one path: the
 * rows' cells gathered to fp16, then the tensor-core latent-attention kernel (qa and the weights rounded to fp16). */
int ns_mla_attend_sel(ns_gpu* g, const float* qa, const uint16_t* c, float* u, int64_t T, int64_t H, int64_t L, int64_t pos0, float scale,
                      const int32_t* sel, const int32_t* sel_cnt, int64_t K);
int ns_mla_attend_sel_q8(ns_gpu* g, const float* qa, const void* c, float* u, int64_t T, int64_t H, int64_t L, int64_t pos0, float scale,
                         const int32_t* sel, const int32_t* sel_cnt, int64_t K);
/* kernels/llm/glm5next/glm.h:58-62,70,72,76-78 - the helper steps of the reference's GEMM-form prompt MLA, under their own
 * names: each row's cell indices and count; the masked row softmax; fp32 -> fp16; fp32 rows -> q8 latent rows; rows
 * gathered by index from an fp16 matrix or from q8 rows. Together with ns_gemm_batch_h below they are the whole call
 * sequence of llm/glm5next/src/engine.rs:1908-1938; ns_mla_attend_sel does the same in one call for any number of rows. */
int ns_mla_cells(ns_gpu* g, const int32_t* sel, const int32_t* sel_cnt, int64_t T, int64_t K, int64_t pos0, int32_t* idx, int32_t* n, int64_t NC);
int ns_softmax_masked(ns_gpu* g, float* S, int64_t R, int64_t H, int64_t NC, const int32_t* n, float scale);
int ns_to_f16(ns_gpu* g, const float* x, uint16_t* y, int64_t n);
int ns_to_q8row(ns_gpu* g, const float* x, void* y, int64_t n, int64_t L);
int ns_gather_q8_h(ns_gpu* g, const void* src, const int32_t* idx, uint16_t* out, int64_t n, int64_t L);
int ns_gather_h(ns_gpu* g, const uint16_t* src, const int32_t* idx, uint16_t* out, int64_t n, int64_t C);

/* kernels/llm/glm5next/glm.h:63-64 (glm.cpp:264-277, a oneMKL gemm_batch there) - `batch` independent products in fp16 with
 * fp32 results: y_b [T, N] (+)= x_b [T, K] . op(w_b), op(w) = w^T (w [N, K], rows ldw apart) with trans_w, else w ([K, N]);
 * x_b = x + b*sx (rows ldx apart), w_b = w + b*sw, y_b = y + b*sy (rows ldy apart), strides in elements; accumulate 0
 * overwrites y. Here a tcgen05 kernel (operands staged by TMA, the accumulator in tensor memory) whenever x and w are
 * 16-byte aligned with ldx, ldw, sx, sw multiples of 8 - the engine's shapes are - and a plain kernel otherwise. The order
 * of the fp32 sums is the tensor cores' (oneMKL's is unspecified as well). */
int ns_gemm_batch_h(ns_gpu* g, int64_t batch, int trans_w, int64_t T, int64_t N, int64_t K, const uint16_t* x, int64_t ldx, int64_t sx,
                    const uint16_t* w, int64_t ldw, int64_t sw, float* y, int64_t ldy, int64_t sy, int accumulate);

/* kernels/llm/deepseek41/silo/ds41.h:28-36 - deepseek41's MQA with heads of 512 where a key is its own value. A row at
 * position p = pos0 + t reads its last min(window, p+1) raw keys from the ring (fp16 [R][512], slot pos % R) and then the
 * compressed cells it sees (comp fp16 [n][512], j < (p+1)/ratio; with sel [T][K], the K it lists once it sees more than
 * K); sinks [H] joins each head's softmax denominator only. q, out fp32 [T][H][512]. The reference has a vector-unit
 * kernel (silo/ds41.cpp:139-229, at most ~12K cells a row) and an XMX one (silo/attn.cpp:64-310, H a multiple of 8);
 * both names run the same path here for any H and any cell count: the rows' cells gathered to dense fp16 in bounded
 * blocks of rows, then the tensor-core latent-attention kernel with the XMX kernel's numerics (q scaled by
 * scale*log2(e) and rounded to fp16, exp2, fp16 weights) and the sink folded into its normalisation (attn.cpp:266-285).
 * A sel index outside [0, (p+1)/ratio) is clamped into it rather than read. */
int ns_ds41_attend(ns_gpu* g, const float* q, const uint16_t* raw, int64_t R, const uint16_t* comp, int64_t ratio, const int32_t* sel, int64_t K,
                   const float* sinks, float* out, int64_t T, int64_t H, int64_t pos0, int64_t window, float scale);
int ns_ds41_attend_xmx_supported(int64_t H, int64_t D);   /* 1 when D == 512 (the reference also wants H % 8 == 0) */
int ns_ds41_attend_xmx(ns_gpu* g, const float* q, const uint16_t* raw, int64_t R, const uint16_t* comp, int64_t ratio, const int32_t* sel, int64_t K,
                       const float* sinks, float* out, int64_t T, int64_t H, int64_t pos0, int64_t window, float scale);
/* kernels/llm/deepseek41/silo/ds41.h:76-79,90-93 (k41.cpp:616-662,776-808) - either side of that attention.
 * ns_ds41_kv_post: a layer's window keys kv [T][D] (D <= 512) RMS-normed by w, the last rd values rotated at their
 * positions (YaRN, adjacent pairs), then the model's E4M3 simulation in blocks of 32 (a power-of-two scale a block);
 * kv keeps the simulated values and ring slot (pos0 + t) % R receives them as fp16.
 * ns_ds41_att_post: the attention's output x [T][H][D]: each head's last rd values rotated back, then the same simulation. */
int ns_ds41_kv_post(ns_gpu* g, float* kv, const float* w, int64_t T, int64_t D, float eps, int64_t rd, int64_t pos0, float freq_base, float freq_scale,
                    float ext_factor, float mscale, float corr0, float corr1, uint16_t* ring, int64_t R);
int ns_ds41_att_post(ns_gpu* g, float* x, int64_t T, int64_t H, int64_t D, int64_t rd, int64_t pos0, float freq_base, float freq_scale, float ext_factor,
                     float mscale, float corr0, float corr1);
/* kernels/llm/deepseek41/silo/ds41.h:57-71 (k41.cpp:96-250,352-483) - the indexer that produces `sel` for that attention.
 * ns_ds41_idx_score: score [T][ld] = sum_h w[t][h] relu(q[t][h] . k_j) for j < min(n, (pos0+t+1)/ratio), -inf from there to
 * ld; q [T][H][D] fp32, k fp16 [n][D]. With 32 heads of 128 and at least 8 keys the products run on the tensor cores in
 * the numerics of the reference's XMX form (q rounded to fp16); otherwise the scalar form (fp32 q), as the reference picks.
 * ns_ds41_block_max: bmax [T][ceil(n/bs)] = the best score of each bs positions; the block of a row's newest position +inf.
 * ns_ds41_cand_mask: score to -inf outside the blocks cand [T][K] lists (mark: scratch of T x ceil(n/bs) bytes).
 * ns_ds41_idx_score_cand: scores only over each row's candidate blocks (cand [T][K]: ids of blocks of 8 keys) into score
 * [T][K*8], -inf where the row sees no key. ns_ds41_cand_pos: picks' compact indices selc [T][kp] back to positions. */
int ns_ds41_idx_score(ns_gpu* g, const float* q, const float* w, const uint16_t* k, float* score, int64_t T, int64_t H, int64_t D, int64_t n, int64_t ld,
                      int64_t pos0, int64_t ratio);
int ns_ds41_block_max(ns_gpu* g, const float* score, float* bmax, int64_t T, int64_t n, int64_t ld, int64_t bs, int64_t pos0, int64_t ratio);
int ns_ds41_idx_score_cand(ns_gpu* g, const float* q, const float* w, const uint16_t* k, const int32_t* cand, int64_t K, float* score, int64_t T, int64_t H,
                           int64_t D, int64_t n, int64_t pos0, int64_t ratio);
int ns_ds41_cand_pos(ns_gpu* g, const int32_t* selc, const int32_t* cand, int32_t* sel, int64_t T, int64_t K, int64_t kp, int64_t bs);
int ns_ds41_cand_mask(ns_gpu* g, float* score, const int32_t* cand, uint8_t* mark, int64_t T, int64_t n, int64_t ld, int64_t K, int64_t bs);
/* silo/ds41.cpp:116-133 - the writers of those caches: T fp32 rows [T][D] into ring slots (pos0 + t) % R as fp16; n fp32
 * rows into rows j0.. of an fp16 matrix */
int ns_ds41_ring_put(ns_gpu* g, const float* kv, uint16_t* ring, int64_t T, int64_t pos0, int64_t R, int64_t D);
int ns_ds41_rows_f16(ns_gpu* g, const float* x, uint16_t* cache, int64_t n, int64_t j0, int64_t D);

/* kernels/llm/glm5next/glm.h:47-55 - the DSA lightning indexer that produces `sel` for the selections above.
 * ns_idx_pool: the pooled keys of the pools (4 consecutive tokens) completed by tokens [pos0, pos0+T): pooled[j][c] =
 * sum_m softmax_m(ig_m[c] + ape[m][c]) ik_m[c] (ik, ig [T][D]; ape [4][D]; pooled indexed by pool); members before pos0
 * come from ring [8][2D] (ik | ig at slot pos % 8), which then takes this pass's last tokens.
 * ns_idx_score: from S [T*H][n] = iq . pooled^T (the caller's GEMM) and w [T][H]: score[r][j0+jj] = sum_h relu(S[r*H+h][jj])
 * w[r][h] for the pools row r sees (j < (pos0+r+1)/4), else -inf; score rows ld floats apart.
 * ns_topk: per row the K highest of score[r][0, n) into sel[r][0, K) in ascending position; ties at the K-th value go to the
 * lowest positions; the same selection every run. With K > n the n positions fill the front of the row and the rest stays. */
int ns_idx_pool(ns_gpu* g, float* ring, const float* ik, const float* ig, const float* ape, float* pooled, int64_t pos0, int64_t T, int64_t D);
int ns_idx_score(ns_gpu* g, const float* S, const float* w, float* score, int64_t T, int64_t H, int64_t j0, int64_t n, int64_t ld, int64_t pos0);
int ns_topk(ns_gpu* g, const float* score, int32_t* sel, int64_t T, int64_t n, int64_t ld, int64_t K);

/* The middle stage alone (the benchmark's absorbed-MLA decode): q [T][H][576] fp16 = absorbed query (512) then rotated
 * part (64); cache [n][576] fp16; out u [T][H][512] fp32. scratch: ns_b200_mla_decode_scratch floats (it depends on
 * the GPU's SM count, hence the handle), 0 when the row is not split. */
int64_t ns_b200_mla_decode_scratch(ns_gpu* g, int64_t T, int64_t H, int64_t pos0);
int ns_b200_mla_decode(ns_gpu* g, const void* q, const void* cache, int64_t T, int64_t H, int64_t pos0, float scale, float* out, float* scratch);

/* One long context split over several GPUs by contiguous key ranges, with a log-sum-exp combine (no counterpart in
 * the reference, which runs a context on one GPU and moves activations between GPUs through host memory,
 * kernels/ns/ns.cpp:244-250). Rank r holds the keys [key_base, key_base + kv_local) of every key head in its own caches
 * [Hkv][kv_local][D] fp16; q [T][Hq*D] fp16 is the same on all ranks; row t sees global keys 0 .. p0+t.
 *   ns_b200_kvsplit_decode  - this rank's keys: split-KV decode, then its (O, m, l) per (row, head) is stored into slot
 *     `rank` of EVERY rank's mailbox (mailboxes: a DEVICE array of nranks mailbox addresses as this GPU sees them -
 *     its own and the peers' IPC-opened ones) and the epoch is published in each (release, system scope).
 *   ns_b200_kvsplit_combine - waits on the device, polling this rank's OWN mailbox for at most wait_us microseconds,
 *     until all ranks published `epoch`, then merges them into out [T][Hq*D] fp16. If the wait runs out the kernel
 *     leaves, nothing is written, and the next ns_sync returns -1 ("gave up a bounded wait (code 701)").
 * Epochs count from 1 and must increase by one per step on every rank (two buffers alternate by epoch parity, so a rank
 * may run one step ahead of its peers, never two). With epoch 0 in both calls the step number is kept in the rank's own
 * mailbox and advanced by the combine, so the pair can be recorded once (ns_q35_graph_begin/end) and replayed.
 * A rank whose range is empty (kv_local 0: a context shorter than the ranks' share) still calls ns_b200_kvsplit_decode -
 * caches and scratch may be null - so that its (empty) partial and its flag reach the others. After a combine gave up
 * (code 701) the ranks' step numbers no longer agree: zero every mailbox and restart the epochs before the next step.
 * A mailbox is ns_b200_kvsplit_mailbox_bytes bytes, zeroed once. */
int64_t ns_b200_kvsplit_mailbox_bytes(int64_t nranks, int64_t T, int64_t Hq, int64_t D);
int64_t ns_b200_kvsplit_scratch(int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t kv_local);
int ns_b200_kvsplit_decode(ns_gpu* g, const void* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                           int64_t kv_local, int64_t key_base, int64_t p0, float* scratch, int64_t rank, int64_t nranks, void* const* mailboxes,
                           int64_t epoch);
int ns_b200_kvsplit_combine(ns_gpu* g, void* mailbox, int64_t nranks, int64_t T, int64_t Hq, int64_t D, int64_t epoch, int64_t wait_us,
                            void* out);
/* The same step as ONE kernel launch: this rank's split-KV decode, the push of its partials into every mailbox and the
 * combine of what arrives in its own (own_mailbox: this rank's mailbox as the host addresses it, also entry `rank` of
 * mailboxes), rows written to out [T][Hq*D] fp16. The kernel's CTAs hand work to one another, so it is launched
 * cooperatively (every CTA resident) - which the benchmark's long-context shape and anything up to two CTAs an SM allows;
 * larger grids run the three launches of the two calls above instead, with the same result. Arguments and epochs as above;
 * a wait that runs out raises code 701 (peers) or 801 (this GPU's own CTAs) at the next ns_sync. */
int ns_b200_kvsplit_step(ns_gpu* g, const void* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                         int64_t kv_local, int64_t key_base, int64_t p0, float* scratch, int64_t rank, int64_t nranks, void* const* mailboxes,
                         void* own_mailbox, int64_t epoch, int64_t wait_us, void* out);
/* The exchange left to the caller (the baseline the mailbox forms are measured against): ns_b200_kvsplit_partial runs this
 * rank's split-KV decode and leaves its merged partial - (O [D], m in log2 units, l) per (row, head), [T*Hq][D+2] floats -
 * in `part`; the caller gathers the ranks' partials side by side (a library all-gather such as ncclAllGather) into
 * [nranks][T*Hq][D+2]; ns_b200_kvsplit_merge merges them into out [T][Hq*D] fp16. */
int ns_b200_kvsplit_partial(ns_gpu* g, const void* q, int64_t qs, const void* kc, const void* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                            int64_t kv_local, int64_t key_base, int64_t p0, float* scratch, float* part);
int ns_b200_kvsplit_merge(ns_gpu* g, const float* parts, int64_t nranks, int64_t T, int64_t Hq, int64_t D, void* out);
/* The same split for the absorbed-MLA latent cache (the middle stage, ns_b200_mla_decode's arguments): rank r holds the cells
 * [cell_base, cell_base + cells_local) as cache [cells_local][576] fp16; q [T][H][576] fp16 is the same on all ranks; row t
 * sees global cells 0 .. pos0+t. ns_b200_mla_kvsplit_decode runs this rank's cells on the tensor cores, merges its splits and
 * pushes (O [512], m, l) per (row, head) into every rank's mailbox (ns_b200_kvsplit_mailbox_bytes(nranks, T, H, 512) bytes
 * each, the same protocol, epochs and flags as above); ns_b200_mla_kvsplit_combine polls this rank's own mailbox (bounded,
 * code 701) and writes u [T][H][512] fp32. No reference counterpart. */
int64_t ns_b200_mla_kvsplit_scratch(ns_gpu* g, int64_t T, int64_t H, int64_t cells_local);
int ns_b200_mla_kvsplit_decode(ns_gpu* g, const void* q, const void* cache, int64_t T, int64_t H, int64_t cells_local, int64_t cell_base, int64_t pos0,
                               float scale, float* scratch, int64_t rank, int64_t nranks, void* const* mailboxes, int64_t epoch);
int ns_b200_mla_kvsplit_combine(ns_gpu* g, void* mailbox, int64_t nranks, int64_t T, int64_t H, int64_t epoch, int64_t wait_us, float* out);
/* Device memory shared between processes of one machine (CUDA IPC): a 64-byte handle for ptr (the start of an
 * ns_alloc allocation), opened in another process as a peer-mapped address, closed when done. */
int ns_b200_ipc_export(ns_gpu* g, void* ptr, void* handle64);
int ns_b200_ipc_open(ns_gpu* g, const void* handle64, void** out);
int ns_b200_ipc_close(ns_gpu* g, void* ptr);

/* No counterpart in the reference. ns_b200_gqa_decode for callers that can neither pass scratch nor tolerate an
 * allocation: an engine whose device memory was planned to the last byte at load time, or a serving loop that must
 * not hit the device-wide synchronisation a cudaMalloc brings. The split partials go to an array built into the
 * library (NS_B200_STATIC_SCRATCH_FLOATS floats = 16 MiB, resident on every GPU the library is used on until the
 * process exits). The call allocates nothing, on the device or through any library. Arguments as ns_b200_gqa_decode;
 * -1 with a message when B*T*Hq*S*(D+2) floats exceed the array, S = min(ceil(max_kv/64), ceil(296/Hkv)): the most key
 * splits any sequence of up to max_kv keys has.
 * The first call on each device looks up the array's device address and queues a one-thread set-up kernel: make that
 * first call before starting any stream capture. All calls share the one array, which keeps whatever the last call
 * left in it (nothing in it needs to start at zero: each call writes every partial before reading it); two calls
 * whose kernels overlap on the GPU - different streams or different ns_gpu handles of one device - race on it. */
#define NS_B200_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)
int ns_b200_gqa_decode_static(ns_gpu* g, const void* q, int64_t qs, int64_t q_seq, const ns_b200_seq* seqs, int64_t B, int64_t T, int64_t Hq,
                              int64_t Hkv, int64_t D, int64_t max_kv, void* out);

#ifdef __cplusplus
}
#endif
#endif
