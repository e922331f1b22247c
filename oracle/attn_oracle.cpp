// attn_oracle.cpp: CPU restatement of the numerics of nextsycl's attention kernels.
//
// TEST INFRASTRUCTURE ONLY. Nothing in the shipped library calls into this file; it is the checker the GPU parity
// tests, the smoke test and the benchmark's CPU-baseline leg compare against.
//
// PARITY: PINNED TO THE REFERENCE'S OWN KERNELS RUN FROM SOURCE, except where the reference calls oneMKL. The reference tree
// holds no golden vector, known-answer test or fixture for any attention kernel, and its SYCL tree cannot be built without a
// oneAPI toolchain. Two pins stand in:
//   1. its one importable CPU implementation of arithmetic on this path, reference/deepseek41/ds41ref.py:
//      tests/golden/make_ref_fixtures.py runs that code (its fp8_sim, rms, freqs, rope and its Ref.attention, on seeded weights)
//      and tests/test_oracle.py holds to its output orc_ds41_attend (both numerics), orc_ds41_kv_post and orc_ds41_att_post (bit
//      for bit), the E4M3 simulation (bit for bit), the YaRN rotation, orc_ds41_idx_score, orc_ds41_block_max and orc_topk;
//   2. its own C++ kernels, compiled for the CPU behind a host stand-in for the SYCL names they use - work-groups as
//      cooperative fibers with barriers, sub-groups, group reductions and shuffles, local memory, and joint_matrix with a
//      tile's 16 products added in ascending k (oracle/ref_shim/; oracle/ref_build.py takes the kernels' lines out of a
//      checkout at build time, nothing of them is kept here). tests/test_ref_compiled.py holds to them, bit for bit:
//      orc_gqa_flash_prefill and orc_gqa_flash_decode (attn_flash / flash_decode of qwen35's and nemotronh's silo/attn.cpp,
//      fp16, q8_0 and q4_0 caches), orc_gqa_plain (attn of q35.cpp and nh.cpp), orc_ds41_attend mode 1 (attend_xmx,
//      attend_merge), orc_ds41_idx_score(_cand) (k41.cpp, both forms), orc_kv_store, orc_kv_store_q, orc_kv_dequant,
//      orc_fwht32, orc_q6k_rows, orc_to_q8row, orc_topk's selections; and within 2e-5 of the largest magnitude:
//      orc_mla_fused (ds2.cpp's fused decode), orc_mla_attend_f32, orc_mla_dec512 (glm.cpp), orc_ds41_attend mode 0,
//      orc_qk_norm_rope, orc_ds2_rope, orc_ds2_kv_store, orc_q35_attn_probs, orc_idx_pool, orc_idx_score, the deepseek41
//      steps around attention.
// UNPINNED: orc_gemm_batch_h and orc_mla_gemm - the reference computes these with oneMKL (closed source, not in the image) from
// its Rust engine; they restate fp16 operands with wide accumulation and the engine's sequence of calls. The order in which
// the matrix unit adds a tile's 16 products is not published either; it is ascending k here and in the stand-in.
//
// Storage: fp16 / bf16 values travel as raw uint16_t bit patterns. All functions are pure (no global state) and
// parallelise over (row, head) with OpenMP only, so a result does not depend on the thread count.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

typedef _Float16 h16;

inline float h2f(uint16_t b) {
    h16 h;
    std::memcpy(&h, &b, 2);
    return (float) h;
}
inline uint16_t f2h(float f) {
    h16 h = (h16) f;   // round to nearest even
    uint16_t b;
    std::memcpy(&b, &h, 2);
    return b;
}
inline float round_h(float f) { return (float) (h16) f; }
inline float bf2f(uint16_t b) {
    uint32_t w = (uint32_t) b << 16;
    float f;
    std::memcpy(&f, &w, 4);
    return f;
}
inline uint16_t f2bf(float f) {
    uint32_t w;
    std::memcpy(&w, &f, 4);
    if ((w & 0x7fffffffu) > 0x7f800000u) return (uint16_t) ((w >> 16) | 0x40);
    w += 0x7fffu + ((w >> 16) & 1u);
    return (uint16_t) (w >> 16);
}
inline float round_bf(float f) { return bf2f(f2bf(f)); }

const float LOG2E = 1.4426950408889634f;
const float NEG_INF = -INFINITY;

// ---- split sizes -------------------------------------------------------------------------------------------------
// kernels/llm/qwen35/silo/attn.cpp:325-331 (XMX decode: multiples of 64 keys, ~512 work-groups)
int64_t flash_split(int64_t kv, int64_t Hkv) {
    const int64_t want = (kv * Hkv + 511) / 512;
    return std::max<int64_t>(64, (want + 63) / 64 * 64);
}
int64_t flash_splits(int64_t kv, int64_t Hkv) {
    const int64_t kb = flash_split(kv, Hkv);
    return (kv + kb - 1) / kb;
}
// kernels/llm/qwen35/q35.cpp:34-42 and kernels/llm/nemotronh/nh.cpp:22-30 (vector-unit kernel: only a single row
// is split, in multiples of 32 keys)
int64_t plain_split(int64_t S, int64_t kv, int64_t groups) {
    if (S != 1) return kv;
    const int64_t want = (kv * groups + 511) / 512;
    return std::max<int64_t>(32, (want + 31) / 32 * 32);
}
int64_t plain_splits(int64_t S, int64_t kv, int64_t groups) {
    const int64_t kb = plain_split(S, kv, groups);
    return kv > kb ? (kv + kb - 1) / kb : 1;
}

// ---- GQA, "flash numerics": kernels/llm/qwen35/silo/attn.cpp:105-313 ---------------------------------------------
// One (row, head) over keys [jbeg, jend), visited in ascending chunks of 16 (attn.cpp:163); keys past `lim` (the
// row's own position, attn.cpp:206,213) are masked. qh is the query already scaled and rounded to fp16
// (attn.cpp:112,147). State (m in log2 units, l, O[D]) is updated in place.
void flash_range(const float* qh, const uint16_t* K, const uint16_t* V, int D, int64_t jbeg, int64_t jend, int64_t lim, float& m, float& l,
                 float* O) {
    const int half_d = D / 2;
    for (int64_t j0 = jbeg; j0 < jend; j0 += 16) {
        float s[16];
        float mx = NEG_INF;
        for (int n = 0; n < 16; ++n) {
            const int64_t j = j0 + n;
            if (j <= lim && j < jend) {
                const uint16_t* kr = K + j * D;
                float lo = 0.f, hi = 0.f;   // two sub-groups, each half of the features, summed after (attn.cpp:213)
                for (int d = 0; d < half_d; ++d) lo += qh[d] * h2f(kr[d]);
                for (int d = half_d; d < D; ++d) hi += qh[d] * h2f(kr[d]);
                s[n] = lo + hi;
            } else {
                s[n] = NEG_INF;
            }
            mx = std::fmax(mx, s[n]);
        }
        const float mn = std::fmax(m, mx);
        const float c = mn == NEG_INF ? 1.0f : std::exp2(m - mn);   // attn.cpp:219-220
        float part[4] = {0.f, 0.f, 0.f, 0.f};   // 4 lanes a row, 4 keys a lane, then the lanes' sums pairwise (attn.cpp:224-231)
        float p16[16];
        for (int n = 0; n < 16; ++n) {
            const float pv = s[n] == NEG_INF ? 0.f : std::exp2(s[n] - mn);
            part[n / 4] += pv;       // the denominator takes the unrounded weight (attn.cpp:225-233)
            p16[n] = round_h(pv);    // the numerator the fp16 one (attn.cpp:227)
        }
        const float sum = (part[0] + part[1]) + (part[2] + part[3]);
        l = l * c + sum;
        for (int d = 0; d < D; ++d) O[d] *= c;   // attn.cpp:244
        for (int n = 0; n < 16; ++n) {
            if (p16[n] == 0.f) continue;
            const uint16_t* vr = V + (j0 + n) * D;
            for (int d = 0; d < D; ++d) O[d] += p16[n] * h2f(vr[d]);
        }
        m = mn;
    }
}

void scale_query_h(const float* q, int D, float qscale, float* qh) {
    for (int d = 0; d < D; ++d) qh[d] = round_h(q[d] * qscale);
}

}  // namespace

extern "C" {

int orc_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// sets the number of OpenMP threads later calls use (an inherited OMP_NUM_THREADS=1, as process launchers export it,
// would otherwise make every timing a one-core figure); returns what is in force
int orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void) n;
    return 1;
#endif
}

int64_t orc_flash_split(int64_t kv, int64_t Hkv) { return flash_split(kv, Hkv); }
int64_t orc_flash_splits(int64_t kv, int64_t Hkv) { return flash_splits(kv, Hkv); }
int64_t orc_plain_split(int64_t S, int64_t kv, int64_t groups) { return plain_split(S, kv, groups); }
int64_t orc_plain_splits(int64_t S, int64_t kv, int64_t groups) { return plain_splits(S, kv, groups); }

// Causal GQA attention in flash numerics, one split a row (the prompt kernel, attn.cpp:379-400, and a decode row with
// one split). q [T][qs] fp32 (row t's head h at h*D), caches fp16 [Hkv][cap][D], out fp32 [T][Hq*D].
void orc_gqa_flash_prefill(const float* q, int64_t qs, const uint16_t* kc, const uint16_t* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                           int64_t cap, int64_t p0, float* out) {
    const int64_t G = Hq / Hkv;
    const float qscale = 1.0f / std::sqrt((float) D) * LOG2E;
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
    for (int64_t t = 0; t < T; ++t) {
        for (int64_t h = 0; h < Hq; ++h) {
            std::vector<float> qh(D), O(D, 0.f);
            scale_query_h(q + t * qs + h * D, (int) D, qscale, qh.data());
            float m = NEG_INF, l = 0.f;
            const int64_t hk = h / G;
            flash_range(qh.data(), kc + hk * cap * D, vc + hk * cap * D, (int) D, 0, p0 + t + 1, p0 + t, m, l, O.data());
            float* o = out + (t * Hq + h) * D;
            for (int64_t d = 0; d < D; ++d) o[d] = l > 0.f ? O[d] / l : 0.f;   // attn.cpp:300
        }
    }
}

// Decode rows (T <= 8) in flash numerics with the reference's own key splits and merge: split size from each row's
// own position (attn.cpp:325-350), partial (O, m in log2 units, l), merge attn.cpp:352-368. part (nullable) receives
// [T][Hq][ns][D+2] as the reference's scratch would, ns = the largest split count of the rows.
void orc_gqa_flash_decode(const float* q, int64_t qs, const uint16_t* kc, const uint16_t* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D,
                          int64_t cap, int64_t p0, float* out, float* part) {
    const int64_t G = Hq / Hkv;
    const float qscale = 1.0f / std::sqrt((float) D) * LOG2E;
    int64_t ns = 1;
    for (int64_t r = 0; r < T; ++r) ns = std::max(ns, flash_splits(p0 + r + 1, Hkv));
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t t = 0; t < T; ++t) {
        for (int64_t h = 0; h < Hq; ++h) {
            const int64_t kv = p0 + t + 1, kb = flash_split(kv, Hkv), nsr = flash_splits(kv, Hkv), hk = h / G;
            std::vector<float> qh(D), P((size_t) nsr * (D + 2));
            scale_query_h(q + t * qs + h * D, (int) D, qscale, qh.data());
            for (int64_t s = 0; s < nsr; ++s) {
                float* O = P.data() + s * (D + 2);
                std::fill(O, O + D, 0.f);
                float m = NEG_INF, l = 0.f;
                flash_range(qh.data(), kc + hk * cap * D, vc + hk * cap * D, (int) D, s * kb, std::min(kv, (s + 1) * kb), kv - 1, m, l, O);
                O[D] = m;
                O[D + 1] = l;
            }
            float* o = out + (t * Hq + h) * D;
            if (nsr == 1) {
                for (int64_t d = 0; d < D; ++d) o[d] = P[D + 1] > 0.f ? P[d] / P[D + 1] : 0.f;   // attn.cpp:276-277
            } else {
                float mx = NEG_INF;
                for (int64_t s = 0; s < nsr; ++s) mx = std::fmax(mx, P[s * (D + 2) + D]);
                for (int64_t d = 0; d < D; ++d) {
                    float Ls = 0.f, A = 0.f;
                    if (mx != NEG_INF) {
                        for (int64_t s = 0; s < nsr; ++s) {
                            const float e = std::exp2(P[s * (D + 2) + D] - mx);
                            Ls += P[s * (D + 2) + D + 1] * e;
                            A += P[s * (D + 2) + d] * e;
                        }
                    }
                    o[d] = Ls > 0.f ? A / Ls : 0.f;
                }
                if (part) std::memcpy(part + ((t * Hq + h) * ns) * (D + 2), P.data(), sizeof(float) * nsr * (D + 2));
            }
        }
    }
}

// Causal GQA attention in "plain" numerics, the vector-unit kernel attn<DL,G> (kernels/llm/qwen35/q35.cpp:44-148;
// D=128 instance kernels/llm/nemotronh/nh.cpp:32-37): fp32 q * 1/sqrt(D), natural exp, fp32 weights; 4 sub-groups
// each take every 4th key of the split (q35.cpp:76), each lane D/16 features (the score a 16-lane reduction); merged
// with q35.cpp:104-128; a single row (S == 1) is split over keys and merged by q35.cpp:131-147. `groups` is what the
// split size is computed from: Hkv for q35.cpp, Hq/8 for nh.cpp.
void orc_gqa_plain(const float* q, int64_t qs, const uint16_t* kc, const uint16_t* vc, int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t cap,
                   int64_t p0, int64_t groups, float* out) {
    const int64_t G = Hq / Hkv;
    const int DL = (int) (D / 16);
    const float scale = 1.0f / std::sqrt((float) D);
    const int64_t ns = plain_splits(T, p0 + T, groups), KB = plain_split(T, p0 + T, groups);
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t t = 0; t < T; ++t) {
        for (int64_t h = 0; h < Hq; ++h) {
            const int64_t hk = h / G, kv_end = p0 + t + 1;
            const uint16_t* K = kc + hk * cap * D;
            const uint16_t* V = vc + hk * cap * D;
            std::vector<float> qv(D), P((size_t) ns * (D + 2)), sub((size_t) 4 * (D + 2));
            for (int64_t d = 0; d < D; ++d) qv[d] = q[t * qs + h * D + d] * scale;
            for (int64_t sp = 0; sp < ns; ++sp) {
                const int64_t j0 = sp * (ns > 1 ? KB : kv_end), j1 = std::min(kv_end, ns > 1 ? (sp + 1) * KB : kv_end);
                for (int sg = 0; sg < 4; ++sg) {
                    float* acc = sub.data() + sg * (D + 2);
                    std::fill(acc, acc + D, 0.f);
                    float m = NEG_INF, l = 0.f;
                    for (int64_t j = j0 + sg; j < j1; j += 4) {
                        float sc = 0.f;
                        for (int lane = 0; lane < 16; ++lane) {   // a lane's DL features, then the lanes
                            float d = 0.f;
                            for (int i = 0; i < DL; ++i) d += qv[lane * DL + i] * h2f(K[j * D + lane * DL + i]);
                            sc += d;
                        }
                        const float mn = std::fmax(m, sc);
                        const float c = std::exp(m - mn), e = std::exp(sc - mn);
                        for (int64_t d = 0; d < D; ++d) acc[d] = acc[d] * c + e * h2f(V[j * D + d]);
                        l = l * c + e;
                        m = mn;
                    }
                    acc[D] = m;
                    acc[D + 1] = l;
                }
                float mx = NEG_INF;
                for (int k = 0; k < 4; ++k) mx = std::fmax(mx, sub[k * (D + 2) + D]);
                float* o = P.data() + sp * (D + 2);
                float L = 0.f;
                for (int64_t d = 0; d < D; ++d) {
                    float A = 0.f;
                    L = 0.f;
                    if (mx != NEG_INF) {
                        for (int k = 0; k < 4; ++k) {
                            const float e = std::exp(sub[k * (D + 2) + D] - mx);
                            L += sub[k * (D + 2) + D + 1] * e;
                            A += sub[k * (D + 2) + d] * e;
                        }
                    }
                    o[d] = A;
                }
                o[D] = mx;
                o[D + 1] = L;
            }
            float* o = out + (t * Hq + h) * D;
            if (ns == 1) {
                for (int64_t d = 0; d < D; ++d) o[d] = P[D + 1] > 0.f ? P[d] / P[D + 1] : 0.f;
            } else {
                float mx = NEG_INF;
                for (int64_t k = 0; k < ns; ++k) mx = std::fmax(mx, P[k * (D + 2) + D]);
                for (int64_t d = 0; d < D; ++d) {
                    float L = 0.f, A = 0.f;
                    if (mx != NEG_INF) {
                        for (int64_t k = 0; k < ns; ++k) {
                            const float e = std::exp(P[k * (D + 2) + D] - mx);
                            L += P[k * (D + 2) + D + 1] * e;
                            A += P[k * (D + 2) + d] * e;
                        }
                    }
                    o[d] = L > 0.f ? A / L : 0.f;
                }
            }
        }
    }
}

// Exact causal attention in fp64 over already-rounded inputs: the yardstick both numerics modes are measured
// against. q fp32 [T][qs]; K [Hkv][cap][Dqk], V [Hkv][cap][Dv] as fp16 (kind 0) or bf16 (kind 1) bit patterns;
// out fp64 [T][Hq*Dv]. Row t sees keys 0 .. p0+t.
void orc_attn_exact(const float* q, int64_t qs, const uint16_t* kc, const uint16_t* vc, int kind, int64_t T, int64_t Hq, int64_t Hkv, int64_t Dqk,
                    int64_t Dv, int64_t cap, int64_t p0, double scale, double* out) {
    const int64_t G = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t t = 0; t < T; ++t) {
        for (int64_t h = 0; h < Hq; ++h) {
            const int64_t hk = h / G, n = p0 + t + 1;
            const uint16_t* K = kc + hk * cap * Dqk;
            const uint16_t* V = vc + hk * cap * Dv;
            std::vector<double> s((size_t) n), acc((size_t) Dv, 0.0);
            double mx = -INFINITY;
            for (int64_t j = 0; j < n; ++j) {
                double d = 0.0;
                for (int64_t i = 0; i < Dqk; ++i) d += (double) q[t * qs + h * Dqk + i] * (double) (kind ? bf2f(K[j * Dqk + i]) : h2f(K[j * Dqk + i]));
                s[j] = d * scale;
                mx = std::max(mx, s[j]);
            }
            double sum = 0.0;
            for (int64_t j = 0; j < n; ++j) {
                const double p = std::exp(s[j] - mx);
                sum += p;
                for (int64_t i = 0; i < Dv; ++i) acc[i] += p * (double) (kind ? bf2f(V[j * Dv + i]) : h2f(V[j * Dv + i]));
            }
            for (int64_t i = 0; i < Dv; ++i) out[(t * Hq + h) * Dv + i] = acc[i] / sum;
        }
    }
}

// Generic causal multi-head attention in "tensor-core numerics" for shapes the reference has no kernel for (bf16 MLA
// prefill with 192-wide keys and 128-wide values): the flash restatement above with the storage type a parameter
// (kind 0 fp16, 1 bf16): q rounded to the type after scaling by scale*log2e, weights rounded to the type before
// they meet V, fp32 sums. K [Hkv][cap][Dqk], V [Hkv][cap][Dv].
void orc_attn_tc(const float* q, int64_t qs, const uint16_t* kc, const uint16_t* vc, int kind, int64_t T, int64_t Hq, int64_t Hkv, int64_t Dqk,
                 int64_t Dv, int64_t cap, int64_t p0, float scale, float* out) {
    const int64_t G = Hq / Hkv;
    const float qscale = scale * LOG2E;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t t = 0; t < T; ++t) {
        for (int64_t h = 0; h < Hq; ++h) {
            const int64_t hk = h / G, n = p0 + t + 1;
            const uint16_t* K = kc + hk * cap * Dqk;
            const uint16_t* V = vc + hk * cap * Dv;
            std::vector<float> qh((size_t) Dqk), O((size_t) Dv, 0.f);
            for (int64_t i = 0; i < Dqk; ++i) {
                const float x = q[t * qs + h * Dqk + i] * qscale;
                qh[i] = kind ? round_bf(x) : round_h(x);
            }
            float m = NEG_INF, l = 0.f;
            for (int64_t j0 = 0; j0 < n; j0 += 16) {
                float s[16], mx = NEG_INF;
                for (int c = 0; c < 16; ++c) {
                    const int64_t j = j0 + c;
                    s[c] = NEG_INF;
                    if (j < n) {
                        float d = 0.f;
                        for (int64_t i = 0; i < Dqk; ++i) d += qh[i] * (kind ? bf2f(K[j * Dqk + i]) : h2f(K[j * Dqk + i]));
                        s[c] = d;
                    }
                    mx = std::fmax(mx, s[c]);
                }
                const float mn = std::fmax(m, mx), cf = mn == NEG_INF ? 1.f : std::exp2(m - mn);
                float sum = 0.f;
                for (int64_t i = 0; i < Dv; ++i) O[i] *= cf;
                for (int c = 0; c < 16; ++c) {
                    if (s[c] == NEG_INF) continue;
                    const float pv = std::exp2(s[c] - mn);
                    sum += pv;
                    const float pr = kind ? round_bf(pv) : round_h(pv);
                    for (int64_t i = 0; i < Dv; ++i) O[i] += pr * (kind ? bf2f(V[(j0 + c) * Dv + i]) : h2f(V[(j0 + c) * Dv + i]));
                }
                l = l * cf + sum;
                m = mn;
            }
            for (int64_t i = 0; i < Dv; ++i) out[(t * Hq + h) * Dv + i] = l > 0.f ? O[i] / l : 0.f;
        }
    }
}

// ---- absorbed MLA ------------------------------------------------------------------------------------------------

// The middle stage of the fused decode kernel mla_decode_t (kernels/llm/deepseek2/ds2.cpp:186-235): q [T][H][L+R]
// fp32 (the absorbed query, then the rotated part), cache fp16 [n][L+R], row t sees cells 0 .. pos0+t;
// u [T][H][L]. 16 sub-groups stride the cells by 16, each with its own online (m, sum, acc) using natural exp
// (ds2.cpp:193-216); a lane owns L/16 latent and R/16 rope features and the score is the 16 lanes' sum times scale
// (ds2.cpp:198-209); final merge ds2.cpp:218-235.
void orc_mla_fused(const float* q, const uint16_t* cache, int64_t T, int64_t H, int64_t L, int64_t R, int64_t pos0, float scale, float* u) {
    const int64_t CR = L + R;
    const int DL = (int) (L / 16), DR = (int) (R / 16);
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t t = 0; t < T; ++t) {
        for (int64_t h = 0; h < H; ++h) {
            const float* qr = q + (t * H + h) * CR;
            const int64_t n = pos0 + t + 1;
            std::vector<float> acc((size_t) 16 * L, 0.f), x((size_t) L);
            float m[16], sum[16];
            for (int sg = 0; sg < 16; ++sg) {
                m[sg] = NEG_INF;
                sum[sg] = 0.f;
                float* a = acc.data() + sg * L;
                for (int64_t i = sg; i < n; i += 16) {
                    const uint16_t* row = cache + i * CR;
                    float d = 0.f;
                    for (int lane = 0; lane < 16; ++lane) {
                        float dl = 0.f;
                        for (int f = 0; f < DL; ++f) {
                            x[lane * DL + f] = h2f(row[lane * DL + f]);
                            dl += qr[lane * DL + f] * x[lane * DL + f];
                        }
                        for (int f = 0; f < DR; ++f) dl += qr[L + lane * DR + f] * h2f(row[L + lane * DR + f]);
                        d += dl;
                    }
                    d *= scale;
                    const float mn = std::fmax(m[sg], d);
                    const float ca = std::exp(m[sg] - mn), cb = std::exp(d - mn);
                    sum[sg] = sum[sg] * ca + cb;
                    for (int64_t f = 0; f < L; ++f) a[f] = a[f] * ca + cb * x[f];
                    m[sg] = mn;
                }
            }
            float mx = NEG_INF;
            for (int k = 0; k < 16; ++k) mx = std::fmax(mx, m[k]);
            float tot = 0.f;
            for (int k = 0; k < 16; ++k) tot += m[k] == NEG_INF ? 0.f : sum[k] * std::exp(m[k] - mx);
            float* o = u + (t * H + h) * L;
            for (int64_t f = 0; f < L; ++f) {
                float v = 0.f;
                for (int k = 0; k < 16; ++k) v += acc[k * L + f] * (m[k] == NEG_INF ? 0.f : std::exp(m[k] - mx));
                o[f] = v / tot;
            }
        }
    }
}

// The GEMM form the deepseek2 engine uses past NS_DS2_MLA_FUSED_MAX cells and for prompt rows
// (llm/deepseek2/src/engine.rs:1204-1224 with ns_softmax_masked, kernels/llm/glm5next/glm.cpp:1042-1060):
// qh = fp16(q); S = qh . cache^T in fp32; P = exp(S*scale - max) / sum over the row's first pos0+t+1 cells, fp32;
// P16 = fp16(P); u = P16 . cache[:, :L] in fp32.
void orc_mla_gemm(const float* q, const uint16_t* cache, int64_t T, int64_t H, int64_t L, int64_t R, int64_t pos0, float scale, float* u) {
    const int64_t CR = L + R;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t t = 0; t < T; ++t) {
        for (int64_t h = 0; h < H; ++h) {
            const int64_t n = pos0 + t + 1;
            std::vector<float> qh((size_t) CR), s((size_t) n), acc((size_t) L, 0.f);
            for (int64_t f = 0; f < CR; ++f) qh[f] = round_h(q[(t * H + h) * CR + f]);
            float mx = NEG_INF;
            for (int64_t i = 0; i < n; ++i) {
                const uint16_t* row = cache + i * CR;
                float d = 0.f;
                for (int64_t f = 0; f < CR; ++f) d += qh[f] * h2f(row[f]);
                s[i] = d;
                mx = std::fmax(mx, d * scale);
            }
            float sum = 0.f;
            for (int64_t i = 0; i < n; ++i) sum += std::exp(s[i] * scale - mx);
            for (int64_t i = 0; i < n; ++i) {
                const float p = round_h(std::exp(s[i] * scale - mx) / sum);
                if (p == 0.f) continue;
                const uint16_t* row = cache + i * CR;
                for (int64_t f = 0; f < L; ++f) acc[f] += p * h2f(row[f]);
            }
            std::memcpy(u + (t * H + h) * L, acc.data(), sizeof(float) * L);
        }
    }
}

// Q6_K rows as deepseek2's decode reads kv_b (kernels/llm/deepseek2/ds2.cpp:117-137; ggml's block_q6_K, kernels/ns/ns_gguf.h:
// 210 bytes a 256 values: ql [128], qh [64], scales [16] int8, d half). Value l (0..31) of quarter g (0..3) of half n (0..1)
// of a block: ((low or high nibble of ql[64 n + 32 (g & 1) + l]) | 2 bits of qh[32 n + l] at 2 g) << 4) - 32, times
// d x scales[8 n + 2 g + l / 16] - the product taken as float(d) * float(scale) * float(q), left to right.
// rows [nrows] of `cols` values (cols a multiple of 256) -> out fp32 [nrows][cols]
void orc_q6k_rows(const uint8_t* blocks, int64_t nrows, int64_t cols, float* out) {
    const int64_t nb = cols / 256;
    for (int64_t r = 0; r < nrows; ++r)
        for (int64_t b = 0; b < nb; ++b) {
            const uint8_t* blk = blocks + (r * nb + b) * 210;
            const uint8_t* ql = blk;
            const uint8_t* qh = blk + 128;
            const int8_t* sc = (const int8_t*) (blk + 192);
            uint16_t dbits;
            std::memcpy(&dbits, blk + 208, 2);
            const float d = h2f(dbits);
            for (int n = 0; n < 2; ++n)
                for (int g = 0; g < 4; ++g)
                    for (int l = 0; l < 32; ++l) {
                        const uint8_t lb = ql[64 * n + 32 * (g & 1) + l];
                        const int lo = g < 2 ? (lb & 0xF) : (lb >> 4);
                        const int q = (lo | (((qh[32 * n + l] >> (2 * g)) & 3) << 4)) - 32;
                        out[r * cols + b * 256 + 128 * n + 32 * g + l] = d * (float) sc[8 * n + 2 * g + l / 16] * (float) q;
                    }
        }
}

// fp64 yardstick for absorbed MLA over the fp16 cache (q fp32 as given).
void orc_mla_exact(const float* q, const uint16_t* cache, int64_t T, int64_t H, int64_t L, int64_t R, int64_t pos0, double scale, double* u) {
    const int64_t CR = L + R;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t t = 0; t < T; ++t) {
        for (int64_t h = 0; h < H; ++h) {
            const int64_t n = pos0 + t + 1;
            std::vector<double> s((size_t) n), acc((size_t) L, 0.0);
            double mx = -INFINITY;
            for (int64_t i = 0; i < n; ++i) {
                double d = 0.0;
                for (int64_t f = 0; f < CR; ++f) d += (double) q[(t * H + h) * CR + f] * (double) h2f(cache[i * CR + f]);
                s[i] = d * scale;
                mx = std::max(mx, s[i]);
            }
            double sum = 0.0;
            for (int64_t i = 0; i < n; ++i) {
                const double p = std::exp(s[i] - mx);
                sum += p;
                for (int64_t f = 0; f < L; ++f) acc[f] += p * (double) h2f(cache[i * CR + f]);
            }
            for (int64_t f = 0; f < L; ++f) u[(t * H + h) * L + f] = acc[f] / sum;
        }
    }
}

// ns_mla_attend (kernels/llm/glm5next/glm.cpp:782-812): dense causal absorbed MLA over fp32 latents, exact two-pass
// softmax with natural exp; the dot product is 256 work-items' strided partial sums (glm.cpp:795) added together.
void orc_mla_attend_f32(const float* qa, const float* c, float* u, int64_t T, int64_t H, int64_t L, int64_t pos0, float scale) {
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t t = 0; t < T; ++t) {
        for (int64_t h = 0; h < H; ++h) {
            const float* qr = qa + (t * H + h) * L;
            const int64_t n = pos0 + t + 1;
            std::vector<float> s((size_t) n), acc((size_t) L, 0.f);
            float mx = NEG_INF;
            for (int64_t i = 0; i < n; ++i) {
                float part[256];
                for (int w = 0; w < 256; ++w) {
                    float d = 0.f;
                    for (int64_t r = w; r < L; r += 256) d += qr[r] * c[i * L + r];
                    part[w] = d;
                }
                float d = 0.f;
                for (int w = 0; w < 256; ++w) d += part[w];
                s[i] = d * scale;
                mx = std::fmax(mx, s[i]);
            }
            float sum = 0.f;
            for (int64_t i = 0; i < n; ++i) {
                const float p = std::exp(s[i] - mx);
                sum += p;
                for (int64_t f = 0; f < L; ++f) acc[f] += p * c[i * L + f];
            }
            for (int64_t f = 0; f < L; ++f) u[(t * H + h) * L + f] = acc[f] / sum;
        }
    }
}

// q8 latent rows (kernels/llm/glm5next/glm.cpp:1282-1299): a row of 512 = 16 fp16 scales then 512 int8; block scale
// fp16(amax/127), values round(x / scale) clamped to +-127. y holds n rows of 544 bytes.
void orc_to_q8row(const float* x, uint8_t* y, int64_t n) {
    for (int64_t r = 0; r < n; ++r) {
        uint8_t* row = y + r * 544;
        for (int b = 0; b < 16; ++b) {
            const float* xr = x + r * 512 + b * 32;
            float amax = 0.f;
            for (int e = 0; e < 32; ++e) amax = std::fmax(amax, std::fabs(xr[e]));
            const uint16_t dh = f2h(amax / 127.f);
            const float d = h2f(dh), inv = d > 0.f ? 1.f / d : 0.f;
            std::memcpy(row + 2 * b, &dh, 2);
            int8_t* qs = reinterpret_cast<int8_t*>(row + 32 + b * 32);
            for (int e = 0; e < 32; ++e) qs[e] = (int8_t) std::min(127.f, std::max(-127.f, std::round(xr[e] * inv)));
        }
    }
}

// mla_dec<512,Q8> (kernels/llm/glm5next/glm.cpp:1079-1186): decode rows over the row's cells - every earlier token
// when sel_cnt is null or negative, else 4 tokens of each selected pool then the incomplete pool (glm.cpp:1094-1102).
// Pass 1 scores (a lane's 32 features, 16 lanes, times scale) and the max; pass 2 natural exp, each of 16 sub-groups
// sums every 16th cell, then the sub-groups are added in order (glm.cpp:1173-1183). c is fp16 [n][512] (q8 == 0) or
// q8 rows of 544 bytes (q8 == 1).
void orc_mla_dec512(const float* qa, const void* cv, float* u, int64_t T, int64_t H, int64_t pos0, float scale, const int32_t* sel,
                    const int32_t* sel_cnt, int64_t K, int q8) {
    const int64_t L = 512;
    const uint16_t* c16 = static_cast<const uint16_t*>(cv);
    const uint8_t* c8 = static_cast<const uint8_t*>(cv);
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t t = 0; t < T; ++t) {
        for (int64_t h = 0; h < H; ++h) {
            const int64_t p = pos0 + t;
            const int32_t ns = sel_cnt ? sel_cnt[t] : -1;
            const int64_t tail0 = 4 * ((p + 1) / 4);
            const int64_t n = ns < 0 ? p + 1 : 4 * (int64_t) ns + (p + 1 - tail0);
            auto cell = [&](int64_t i) -> int64_t {
                if (ns < 0) return i;
                if (i < 4 * (int64_t) ns) return 4 * (int64_t) sel[t * K + i / 4] + i % 4;
                return tail0 + (i - 4 * (int64_t) ns);
            };
            auto load = [&](int64_t i, float* x) {
                if (q8) {
                    const uint8_t* row = c8 + cell(i) * 544;
                    for (int b = 0; b < 16; ++b) {
                        uint16_t dh;
                        std::memcpy(&dh, row + 2 * b, 2);
                        const float d = h2f(dh);
                        const int8_t* qs = reinterpret_cast<const int8_t*>(row + 32 + b * 32);
                        for (int e = 0; e < 32; ++e) x[b * 32 + e] = d * (float) qs[e];
                    }
                } else {
                    const uint16_t* row = c16 + cell(i) * L;
                    for (int64_t f = 0; f < L; ++f) x[f] = h2f(row[f]);
                }
            };
            const float* qr = qa + (t * H + h) * L;
            std::vector<float> sc((size_t) n), x((size_t) L), acc((size_t) 16 * L, 0.f);
            float mx = NEG_INF;
            for (int64_t i = 0; i < n; ++i) {
                load(i, x.data());
                float d = 0.f;
                for (int lane = 0; lane < 16; ++lane) {
                    float dl = 0.f;
                    for (int f = 0; f < 32; ++f) dl += qr[lane * 32 + f] * x[lane * 32 + f];
                    d += dl;
                }
                sc[i] = d * scale;
                mx = std::fmax(mx, sc[i]);
            }
            float sk[16] = {};
            for (int64_t i = 0; i < n; ++i) {
                const int sg = (int) (i % 16);
                const float w = std::exp(sc[i] - mx);
                sk[sg] += w;
                load(i, x.data());
                float* a = acc.data() + sg * L;
                for (int64_t f = 0; f < L; ++f) a[f] += w * x[f];
            }
            float sum = 0.f;
            for (int k = 0; k < 16; ++k) sum += sk[k];
            for (int64_t f = 0; f < L; ++f) {
                float v = 0.f;
                for (int k = 0; k < 16; ++k) v += acc[k * L + f];
                u[(t * H + h) * L + f] = v / sum;
            }
        }
    }
}

// ---- deepseek41: MQA over a window ring and compressed cells, with sinks ------------------------------------------

// ns_ds41_attend. A row at position p = pos0+t reads n_raw = min(window, p+1) raw keys from the ring [R][512] (slot
// (p - n_raw + 1 + i) % R) and then compressed cells comp [n][512]: the first vis = (p+1)/ratio of them, or - when sel is
// given and vis > K - the K cells sel[t][0..K) (kernels/llm/deepseek41/silo/attn.cpp:83-94). A key is its own value.
// The sink of a head joins the denominator only.
//   mode 0, the vector kernel (kernels/llm/deepseek41/silo/ds41.cpp:139-229): fp32 q, scores (q . c) * scale, the
//     maximum starts from the sink, natural exp, denominator sum + exp(sink - mx).
//   mode 1, the XMX kernel (silo/attn.cpp:64-259 and the merge :266-285): q scaled by scale*log2(e) and rounded to fp16,
//     chunks of 16 cells ascending, exp2, weights rounded to fp16 for the numerator; as ns_ds41_attend_xmx runs it
//     (attn.cpp:307-352): more than 8 rows, a row's cells in one pass and out = O / (l + 2^(sink*log2e - m)); up to 8
//     rows, the cells in splits and out = sum_k O_k 2^(m_k - mx) / (2^(sink*log2e - mx) + sum_k l_k 2^(m_k - mx)),
//     mx = max(sink*log2e, m_k).
void orc_ds41_attend(const float* q, const uint16_t* raw, int64_t R, const uint16_t* comp, int64_t ratio, const int32_t* sel, int64_t K,
                     const float* sinks, float* out, int64_t T, int64_t H, int64_t pos0, int64_t window, float scale, int mode) {
    const int64_t D = 512;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t t = 0; t < T; ++t) {
        for (int64_t h = 0; h < H; ++h) {
            const int64_t p = pos0 + t;
            const int64_t n_raw = std::min<int64_t>(window, p + 1);
            const int64_t vis = comp ? (p + 1) / ratio : 0;
            const bool pick = sel && vis > K;
            const int64_t n = n_raw + (pick ? K : vis);
            auto cell = [&](int64_t i) -> const uint16_t* {
                if (i < n_raw) return raw + ((p - n_raw + 1 + i) % R) * D;
                const int64_t k = i - n_raw;
                return comp + (pick ? (int64_t) sel[t * K + k] : k) * D;
            };
            const float* qr = q + (t * H + h) * D;
            float* o = out + (t * H + h) * D;
            if (mode == 0) {
                std::vector<float> sc((size_t) n), acc((size_t) D, 0.f);
                float mx = sinks[h];
                for (int64_t i = 0; i < n; ++i) {
                    const uint16_t* c = cell(i);
                    float d = 0.f;
                    for (int64_t r = 0; r < D; ++r) d += qr[r] * h2f(c[r]);
                    sc[i] = d * scale;
                    mx = std::fmax(mx, sc[i]);
                }
                float sum = 0.f;
                for (int64_t i = 0; i < n; ++i) {
                    sc[i] = std::exp(sc[i] - mx);
                    sum += sc[i];
                }
                sum += std::exp(sinks[h] - mx);
                for (int64_t i = 0; i < n; ++i) {
                    const uint16_t* c = cell(i);
                    for (int64_t r = 0; r < D; ++r) acc[r] += sc[i] * h2f(c[r]);
                }
                for (int64_t r = 0; r < D; ++r) o[r] = acc[r] / sum;
            } else {
                std::vector<float> qh((size_t) D);
                for (int64_t r = 0; r < D; ++r) qh[r] = round_h(qr[r] * (scale * LOG2E));
                // cells [jbeg, jend) in chunks of 16 from jbeg: a score the sum of its four quarters' partial dot products
                // (attn.cpp:182), the chunk's sum 8 lanes of 2 cells each, then pairwise (attn.cpp:197-204)
                auto range = [&](int64_t jbeg, int64_t jend, float& m, float& l, float* O) {
                    for (int64_t j0 = jbeg; j0 < jend; j0 += 16) {
                        float s[16], mxc = NEG_INF;
                        for (int c = 0; c < 16; ++c) {
                            s[c] = NEG_INF;
                            if (j0 + c < jend) {
                                const uint16_t* cc = cell(j0 + c);
                                float v = 0.f;
                                for (int q4 = 0; q4 < 4; ++q4) {
                                    float d = 0.f;
                                    for (int64_t r = 128 * q4; r < 128 * (q4 + 1); ++r) d += qh[r] * h2f(cc[r]);
                                    v += d;
                                }
                                s[c] = v;
                            }
                            mxc = std::fmax(mxc, s[c]);
                        }
                        const float mn = std::fmax(m, mxc), cf = mn == NEG_INF ? 1.f : std::exp2(m - mn);
                        for (int64_t r = 0; r < D; ++r) O[r] *= cf;
                        float lane[8];
                        for (int c = 0; c < 16; ++c) {
                            const float pv = s[c] == NEG_INF ? 0.f : std::exp2(s[c] - mn);
                            lane[c / 2] = c % 2 ? lane[c / 2] + pv : pv;
                            if (s[c] == NEG_INF) continue;
                            const float pr = round_h(pv);
                            const uint16_t* cc = cell(j0 + c);
                            for (int64_t r = 0; r < D; ++r) O[r] += pr * h2f(cc[r]);
                        }
                        const float sum = ((lane[0] + lane[1]) + (lane[2] + lane[3])) + ((lane[4] + lane[5]) + (lane[6] + lane[7]));
                        l = l * cf + sum;
                        m = mn;
                    }
                };
                const float sk = sinks[h] * LOG2E;
                if (T > 8) {
                    // a prompt pass: one work-group a row's head group, all its cells; the sink joins the sum (attn.cpp:247-255)
                    std::vector<float> O((size_t) D, 0.f);
                    float m = NEG_INF, l = 0.f;
                    range(0, n, m, l, O.data());
                    l += std::exp2(sk - m);
                    for (int64_t r = 0; r < D; ++r) o[r] = O[r] / l;
                } else {
                    // decode rows (at most 8): the row's cells in splits sized from its own count alone - at most 64 of them,
                    // at least 32 cells, a multiple of 16 (attn.cpp:325-329) -, then the merge with the sink (attn.cpp:266-285)
                    int64_t kb = std::max<int64_t>(32, (n + 63) / 64);
                    kb = (kb + 15) / 16 * 16;
                    const int64_t nsr = (n + kb - 1) / kb;
                    std::vector<float> P((size_t) nsr * (D + 2), 0.f);
                    float mx = sk;
                    for (int64_t k = 0; k < nsr; ++k) {
                        float* O = P.data() + k * (D + 2);
                        float m = NEG_INF, l = 0.f;
                        range(k * kb, std::min(n, (k + 1) * kb), m, l, O);
                        O[D] = m;
                        O[D + 1] = l;
                        mx = std::fmax(mx, m);
                    }
                    float Ls = std::exp2(sk - mx);
                    std::vector<float> e((size_t) nsr);
                    for (int64_t k = 0; k < nsr; ++k) {
                        e[k] = std::exp2(P[k * (D + 2) + D] - mx);
                        Ls += P[k * (D + 2) + D + 1] * e[k];
                    }
                    for (int64_t r = 0; r < D; ++r) {
                        float A = 0.f;
                        for (int64_t k = 0; k < nsr; ++k) A += P[k * (D + 2) + r] * e[k];
                        o[r] = A / Ls;
                    }
                }
            }
        }
    }
}

// ---- quantised caches (heads of 256): kernels/llm/qwen35/q35.cpp:281-326, reader silo/attn.cpp:49-78 --------------------
// A head's row: q8_0 (kt 1) 256 int8 values then 8 fp16 scales = 272 bytes; q4_0 (kt 2) 8 blocks of 16 bytes (byte j of a
// block: value j low nibble, value j + 16 high) then 8 fp16 scales = 144 bytes. Blocks of 32 values.
static inline int64_t q_row_bytes(int kt) { return kt == 1 ? 272 : 144; }

static void quant_block(int kt, const float* x, uint8_t* row, int b) {
    if (kt == 1) {
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) amax = std::fmax(amax, std::fabs(x[j]));
        const float d = amax / 127.0f, id = d != 0.0f ? 1.0f / d : 0.0f;
        for (int j = 0; j < 32; ++j) row[b * 32 + j] = (uint8_t) (int8_t) std::round(x[j] * id);   // half away from zero
        const uint16_t dh = f2h(d);
        std::memcpy(row + 256 + 2 * b, &dh, 2);
    } else {
        // ggml's quantize_row_q4_0: the value of the largest magnitude (the first of a tie), d = it / -8
        float m = 0.0f, am = 0.0f;
        for (int j = 0; j < 32; ++j)
            if (std::fabs(x[j]) > am) {
                am = std::fabs(x[j]);
                m = x[j];
            }
        const float d = m / -8.0f, id = d != 0.0f ? 1.0f / d : 0.0f;
        for (int j = 0; j < 16; ++j) {
            const int lo = std::min(15, (int) (x[j] * id + 8.5f)), hi = std::min(15, (int) (x[j + 16] * id + 8.5f));
            row[b * 16 + j] = (uint8_t) (lo | (hi << 4));
        }
        const uint16_t dh = f2h(d);
        std::memcpy(row + 128 + 2 * b, &dh, 2);
    }
}

// ns_q35_kv_store_q: rows k, v [T][Hkv*256] fp32 (ks, vs floats apart) into the quantised caches [Hkv][cap][row bytes]
void orc_kv_store_q(int kt, const float* k, int64_t ks, const float* v, int64_t vs, int64_t T, int64_t Hkv, int64_t cap, int64_t p0, uint8_t* kc,
                    uint8_t* vc) {
    const int64_t rb = q_row_bytes(kt);
    for (int64_t t = 0; t < T; ++t)
        for (int64_t h = 0; h < Hkv; ++h)
            for (int b = 0; b < 8; ++b) {
                quant_block(kt, k + t * ks + h * 256 + b * 32, kc + (h * cap + p0 + t) * rb, b);
                quant_block(kt, v + t * vs + h * 256 + b * 32, vc + (h * cap + p0 + t) * rb, b);
            }
}

// What kv_load8<KT> hands the tensor cores (silo/attn.cpp:49-78): value = half((float) q * (float) d). Rows [0, n) of each
// head of a cache [Hkv][cap][row bytes] to fp16 [Hkv][n][256].
void orc_kv_dequant(int kt, const uint8_t* c, int64_t Hkv, int64_t cap, int64_t n, uint16_t* out) {
    const int64_t rb = q_row_bytes(kt);
#pragma omp parallel for collapse(2)
    for (int64_t h = 0; h < Hkv; ++h)
        for (int64_t j = 0; j < n; ++j) {
            const uint8_t* row = c + (h * cap + j) * rb;
            uint16_t* o = out + (h * n + j) * 256;
            for (int i = 0; i < 256; ++i) {
                const int b = i / 32, e = i % 32;
                uint16_t dh;
                float q;
                if (kt == 1) {
                    std::memcpy(&dh, row + 256 + 2 * b, 2);
                    q = (float) (int8_t) row[i];
                } else {
                    std::memcpy(&dh, row + 128 + 2 * b, 2);
                    const uint8_t byte = row[b * 16 + (e & 15)];
                    q = (float) ((int) ((e < 16 ? byte : byte >> 4) & 15) - 8);
                }
                o[i] = f2h(q * h2f(dh));
            }
        }
}

// ns_q35_fwht32 (q35.cpp:328-348): each block of 32 of rows [rows][n] through a normalised Walsh-Hadamard transform
void orc_fwht32(float* x, int64_t rows, int64_t n, int64_t stride) {
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t b = 0; b < n / 32; ++b) {
            float* p = x + r * stride + b * 32;
            float v[32];
            for (int i = 0; i < 32; ++i) v[i] = p[i];
            for (int o = 1; o < 32; o <<= 1)
                for (int i = 0; i < 32; ++i)
                    if (!(i & o)) {
                        const float a = v[i], c = v[i + o];
                        v[i] = a + c;
                        v[i + o] = a - c;
                    }
            for (int i = 0; i < 32; ++i) p[i] = v[i] * 0.17677669529663687f;
        }
}

// ---- the step before attention: RMS norm and rotary positions of q and k (kernels/llm/qwen35/q35.cpp:220-254,256-279,350-385)
// Per (row t, head h): x = src[t*ss + h*hs .. + D]; with w: x * rsqrt(mean(x^2) + eps) * w (the squares summed as the
// reference's 16 lanes do: lane l takes i = l, l+16, ..; the lanes' sums added in order); then rotate-half over the first
// n_rot features: pair (i, i + n_rot/2) turned by angle pos * theta^(-2i/n_rot); into dst[t*ds + h*D]. pos = p0 + t, or
// with pos3 [T][3] the one of (t, h, w) that pair k's interleaved section picks (sections s0, s1, s2).
void orc_qk_norm_rope(const float* src, int64_t ss, int64_t hs, float* dst, int64_t ds, int64_t T, int64_t H, int64_t D, const float* w, float eps,
                      int64_t n_rot, float theta, int64_t p0, const int32_t* pos3, int64_t s0, int64_t s1, int64_t s2) {
    const int64_t half_rot = n_rot / 2, sect = s0 + s1 + s2;
    for (int64_t t = 0; t < T; ++t)
        for (int64_t h = 0; h < H; ++h) {
            const float* x = src + t * ss + h * hs;
            float* y = dst + t * ds + h * D;
            float inv = 1.0f;
            if (w) {
                float lane[16] = {};
                for (int64_t i = 0; i < D; ++i) lane[i % 16] += x[i] * x[i];
                float sum = 0.0f;
                for (int l = 0; l < 16; ++l) sum += lane[l];
                inv = 1.0f / std::sqrt(sum / (float) D + eps);
            }
            std::vector<float> v((size_t) D);
            for (int64_t i = 0; i < D; ++i) v[i] = w ? x[i] * inv * w[i] : x[i];
            for (int64_t i = 0; i < D; ++i) {
                if (i >= n_rot) {
                    y[i] = v[i];
                    continue;
                }
                const int64_t k = i < half_rot ? i : i - half_rot;
                float p = (float) (p0 + t);
                if (pos3) {
                    const int64_t sec = k % sect;
                    const int c = (sec % 3 == 1 && sec < 3 * s1) ? 1 : (sec % 3 == 2 && sec < 3 * s2) ? 2 : 0;
                    p = (float) pos3[t * 3 + c];
                }
                const float a = p * std::pow(theta, -2.0f * (float) k / (float) n_rot);
                const float c_ = std::cos(a), sn = std::sin(a);
                const float other = v[i < half_rot ? i + half_rot : i - half_rot];
                y[i] = i < half_rot ? v[i] * c_ - other * sn : v[i] * c_ + other * sn;
            }
        }
}

// ---- deepseek2: YaRN rotary positions and the latent cache's writer (kernels/llm/deepseek2/ds2.cpp:15-34,58-112) ----------
// cos and sin of pair i0 (of n_dims) at position p as ggml's rope cache computes them: the angle by repeated products
static void yarn_cs(float p, int i0, int n_dims, float freq_base, float freq_scale, float ext_factor, float mscale, float corr0, float corr1, float& c,
                    float& s) {
    const float theta_scale = std::pow(freq_base, -2.0f / (float) n_dims);
    float theta_extrap = p;
    for (int k = 0; k < i0 / 2; ++k) theta_extrap *= theta_scale;
    const float theta_interp = freq_scale * theta_extrap;
    float theta = theta_interp;
    if (ext_factor != 0.0f) {
        const float y = ((float) (i0 / 2) - corr0) / std::fmax(0.001f, corr1 - corr0);
        const float ramp_mix = (1.0f - std::fmin(1.0f, std::fmax(0.0f, y))) * ext_factor;
        theta = theta_interp * (1 - ramp_mix) + theta_extrap * ramp_mix;
    }
    c = std::cos(theta) * mscale;
    s = std::sin(theta) * mscale;
}

// ns_ds2_rope: adjacent pairs of the n_dims values from float `off` of each head, in place; `out` (nullable) gets them too
void orc_ds2_rope(float* x, int64_t T, int64_t H, int64_t row, int64_t head, int64_t off, int64_t n_dims, int64_t pos0, float freq_base, float freq_scale,
                  float ext_factor, float mscale, float corr0, float corr1, float* out, int64_t out_row, int64_t out_head) {
    for (int64_t t = 0; t < T; ++t)
        for (int64_t h = 0; h < H; ++h)
            for (int64_t i = 0; i < n_dims / 2; ++i) {
                const int i0 = (int) (2 * i);
                float c, s;
                yarn_cs((float) (pos0 + t), i0, (int) n_dims, freq_base, freq_scale, ext_factor, mscale, corr0, corr1, c, s);
                float* v = x + t * row + h * head + off + i0;
                const float x0 = v[0], x1 = v[1];
                const float y0 = x0 * c - x1 * s, y1 = x0 * s + x1 * c;
                v[0] = y0, v[1] = y1;
                if (out) {
                    out[t * out_row + h * out_head + i0] = y0;
                    out[t * out_row + h * out_head + i0 + 1] = y1;
                }
            }
}

// ns_ds2_kv_store: kv [T][L+R] fp32 -> cache rows pos0.. fp16: the first L RMS-normed with w (the squares summed as the
// reference's 256 work-items do, item l taking i = l, l+256, ..; their sums added in order), the last R rotated
void orc_ds2_kv_store(const float* kv, const float* w, float eps, uint16_t* cache, int64_t T, int64_t L, int64_t R, int64_t pos0, float freq_base,
                      float freq_scale, float ext_factor, float mscale, float corr0, float corr1) {
    for (int64_t t = 0; t < T; ++t) {
        const float* xr = kv + t * (L + R);
        float item[256] = {};
        for (int64_t i = 0; i < L; ++i) item[i % 256] += xr[i] * xr[i];
        float ss = 0.f;
        for (int l = 0; l < 256; ++l) ss += item[l];
        const float inv = 1.f / std::sqrt(ss / (float) L + eps);
        uint16_t* o = cache + (pos0 + t) * (L + R);
        for (int64_t i = 0; i < L; ++i) o[i] = f2h(xr[i] * inv * w[i]);
        for (int64_t i = 0; i < R / 2; ++i) {
            const int i0 = (int) (2 * i);
            float c, s;
            yarn_cs((float) (pos0 + t), i0, (int) R, freq_base, freq_scale, ext_factor, mscale, corr0, corr1, c, s);
            const float x0 = xr[L + i0], x1 = xr[L + i0 + 1];
            o[L + i0] = f2h(x0 * c - x1 * s);
            o[L + i0 + 1] = f2h(x0 * s + x1 * c);
        }
    }
}

// ---- deepseek41: the window key's writer and the attention output's post step (kernels/llm/deepseek41/silo/k41.cpp:16-35,
// 250-270,616-662,776-808): YaRN rotation of a row's last rd values, then the model's E4M3 simulation in blocks of 32
static float pow2_ceil(float x) {   // 2^ceil(log2 x), x > 0
    int e;
    const float m = std::frexp(x, &e);
    if (m == 0.5f) e -= 1;
    return std::ldexp(1.0f, e);
}
static float e4m3_round(float x) {   // the nearest E4M3FN value (ties to even), |x| <= 448
    const float a = std::fabs(x);
    if (a == 0.f) return x;
    int e;
    std::frexp(a, &e);
    int be = e - 1;
    if (be < -6) be = -6;
    const float step = std::ldexp(1.0f, be - 3);
    float q = std::rint(a / step) * step;
    q = std::fmin(q, 448.f);
    return x < 0 ? -q : q;
}
static void e4m3_sim32(const float* v, float* out) {   // a block of 32: a power-of-two scale from its largest magnitude
    float amax = 0.f;
    for (int j = 0; j < 32; ++j) amax = std::fmax(amax, std::fabs(v[j]));
    const float sc = pow2_ceil(std::fmax(amax, 1e-4f) / 448.f);
    for (int j = 0; j < 32; ++j) out[j] = e4m3_round(std::fmin(std::fmax(v[j] / sc, -448.f), 448.f)) * sc;
}

// ns_ds41_kv_post: kv [T][D] RMS-normed by w (256 items' partial sums, added in order), the last rd values rotated at
// pos0 + t, the E4M3 simulation in 32s; kv keeps the simulated values, the ring slot (pos0 + t) % R gets them as fp16
void orc_ds41_kv_post(float* kv, const float* w, int64_t T, int64_t D, float eps, int64_t rd, int64_t pos0, float freq_base, float freq_scale,
                      float ext_factor, float mscale, float corr0, float corr1, uint16_t* ring, int64_t R) {
    for (int64_t t = 0; t < T; ++t) {
        float* xr = kv + t * D;
        float item[256] = {};
        for (int64_t c = 0; c < D; ++c) item[c % 256] += xr[c] * xr[c];
        float s = 0.f;
        for (int l = 0; l < 256; ++l) s += item[l];
        const float inv = 1.f / std::sqrt(s / (float) D + eps);
        std::vector<float> y((size_t) D);
        for (int64_t c = 0; c < D; ++c) y[c] = xr[c] * inv * w[c];
        const int64_t off = D - rd;
        for (int64_t i = 0; i < rd / 2; ++i) {
            const int i0 = (int) (2 * i);
            float cs, sn;
            yarn_cs((float) (pos0 + t), i0, (int) rd, freq_base, freq_scale, ext_factor, mscale, corr0, corr1, cs, sn);
            const float x0 = y[off + i0], x1 = y[off + i0 + 1];
            y[off + i0] = x0 * cs - x1 * sn;
            y[off + i0 + 1] = x0 * sn + x1 * cs;
        }
        for (int64_t c0 = 0; c0 < D; c0 += 32) {
            e4m3_sim32(y.data() + c0, xr + c0);
            for (int j = 0; j < 32; ++j) ring[((pos0 + t) % R) * D + c0 + j] = f2h(xr[c0 + j]);
        }
    }
}

// ns_ds41_att_post: x [T][H][D], each head's last rd values rotated back at the row's position, then the simulation in 32s
void orc_ds41_att_post(float* x, int64_t T, int64_t H, int64_t D, int64_t rd, int64_t pos0, float freq_base, float freq_scale, float ext_factor,
                       float mscale, float corr0, float corr1) {
    const int64_t off = D - rd;
    for (int64_t t = 0; t < T; ++t)
        for (int64_t h = 0; h < H; ++h) {
            float* xr = x + (t * H + h) * D;
            std::vector<float> y(xr, xr + D);
            for (int64_t c = off; c < D; ++c) {
                const int i0 = (int) ((c - off) & ~int64_t(1));
                float cs, sn;
                yarn_cs((float) (pos0 + t), i0, (int) rd, freq_base, freq_scale, ext_factor, mscale, corr0, corr1, cs, sn);
                sn = -sn;
                const float v = xr[c], o = xr[c ^ 1];   // off is even (D a multiple of 32, rd even): the pair's other value
                y[c] = (c - off) % 2 == 0 ? v * cs - o * sn : o * sn + v * cs;
            }
            for (int64_t c0 = 0; c0 < D; c0 += 32) e4m3_sim32(y.data() + c0, xr + c0);
        }
}

// ---- ns_q35_attn_probs (kernels/llm/qwen35/q35.cpp:464-506): one query row's softmax weights over the cache's first n keys
// (its form kt: 0 half, 1 q8_0, 2 q4_0; heads of 256; the value of a quantised element is float(q) * float(d), q35.cpp:19-25),
// per key their mean over the heads (mode 0) or their largest (mode 1), added to out [n]; scratch [Hq][2] gets (max, sum)
void orc_q35_attn_probs(int kt, const float* q, const uint8_t* kc, int64_t Hq, int64_t Hkv, int64_t cap, int64_t n, int mode, float* scratch, float* out) {
    const int64_t D = 256, G = Hq / Hkv, rb = kt == 0 ? 512 : kt == 1 ? 272 : 144;
    const float scale = 1.0f / std::sqrt((float) D);
    std::vector<float> S((size_t) (Hq * n));
#pragma omp parallel for collapse(2)
    for (int64_t h = 0; h < Hq; ++h)
        for (int64_t j = 0; j < n; ++j) {
            const uint8_t* row = kc + ((h / G) * cap + j) * rb;
            float acc = 0.0f;
            for (int64_t i = 0; i < D; ++i) {
                float v;
                if (kt == 0) {
                    uint16_t b;
                    std::memcpy(&b, row + 2 * i, 2);
                    v = h2f(b);
                } else {
                    const int blk = (int) (i / 32), e = (int) (i % 32);
                    uint16_t db;
                    std::memcpy(&db, row + (kt == 1 ? 256 : 128) + 2 * blk, 2);
                    const float d = h2f(db);
                    if (kt == 1) v = (float) (int8_t) row[i] * d;
                    else {
                        const uint8_t w = row[blk * 16 + (e & 15)];
                        v = (float) ((int) (e < 16 ? w & 15 : w >> 4) - 8) * d;
                    }
                }
                acc += q[h * D + i] * v;
            }
            S[h * n + j] = acc * scale;
        }
    for (int64_t h = 0; h < Hq; ++h) {
        float m = NEG_INF, z = 0.0f;
        for (int64_t j = 0; j < n; ++j) m = std::fmax(m, S[h * n + j]);
        for (int64_t j = 0; j < n; ++j) z += std::exp(S[h * n + j] - m);
        scratch[h * 2] = m;
        scratch[h * 2 + 1] = z;
    }
    for (int64_t j = 0; j < n; ++j) {
        float acc = 0.0f;
        for (int64_t h = 0; h < Hq; ++h) {
            const float p = std::exp(S[h * n + j] - scratch[h * 2]) / scratch[h * 2 + 1];
            acc = mode == 1 ? std::fmax(acc, p) : acc + p / (float) Hq;
        }
        out[j] += acc;
    }
}

// ---- glm5next's DSA indexer (kernels/llm/glm5next/glm.cpp:876-1015): pooled keys, pool scores, the K best pools a row ----
// ns_idx_pool: the pools completed by tokens [pos0, pos0+T): pooled[j][c] = sum_m softmax_m(ig_m[c] + ape[m][c]) ik_m[c] over
// the pool's 4 members (positions 4j+m); a member before pos0 comes from ring [8][2D] (ik | ig at slot pos % 8); then the
// ring takes this pass's last (up to 8) tokens.
void orc_idx_pool(float* ring, const float* ik, const float* ig, const float* ape, float* pooled, int64_t pos0, int64_t T, int64_t D) {
    const int64_t j_lo = pos0 / 4, j_hi = (pos0 + T) / 4;
    for (int64_t j = j_lo; j < j_hi; ++j)
        for (int64_t c = 0; c < D; ++c) {
            float lg[4], kv[4], mx = NEG_INF;
            for (int m = 0; m < 4; ++m) {
                const int64_t p = 4 * j + m;
                const float* k = p >= pos0 ? ik + (p - pos0) * D : ring + (p % 8) * 2 * D;
                const float* gg = p >= pos0 ? ig + (p - pos0) * D : ring + (p % 8) * 2 * D + D;
                kv[m] = k[c];
                lg[m] = gg[c] + ape[m * D + c];
                mx = std::fmax(mx, lg[m]);
            }
            float sum = 0.f, acc = 0.f;
            for (int m = 0; m < 4; ++m) {
                const float e = std::exp(lg[m] - mx);
                sum += e;
                acc += e * kv[m];
            }
            pooled[j * D + c] = acc / sum;   // pooled is the whole pooled-key matrix: pool j's row
        }
    const int64_t first = std::max<int64_t>(pos0, pos0 + T - 8);
    for (int64_t p = first; p < pos0 + T; ++p)
        for (int64_t c = 0; c < D; ++c) {
            ring[(p % 8) * 2 * D + c] = ik[(p - pos0) * D + c];
            ring[(p % 8) * 2 * D + D + c] = ig[(p - pos0) * D + c];
        }
}

// ns_idx_score: S [T*H][n] (heads as rows), w [T][H]: score[r][j0+jj] = sum_h relu(S[r*H+h][jj]) w[r][h] for the pools row r
// sees (j < (pos0+r+1)/4), else -inf; score rows ld floats apart
void orc_idx_score(const float* S, const float* w, float* score, int64_t T, int64_t H, int64_t j0, int64_t n, int64_t ld, int64_t pos0) {
    for (int64_t r = 0; r < T; ++r)
        for (int64_t jj = 0; jj < n; ++jj) {
            const int64_t j = j0 + jj, nv = (pos0 + r + 1) / 4;
            float sc = NEG_INF;
            if (j < nv) {
                sc = 0.f;
                for (int64_t h = 0; h < H; ++h) sc += std::fmax(S[(r * H + h) * n + jj], 0.f) * w[r * H + h];
            }
            score[r * ld + j] = sc;
        }
}

// ns_topk: per row the K highest of score[r][0, n) into sel[r][0, K) in ascending position; ties at the K-th value go to
// the lowest positions. Order by the float's order-preserving key (sign bit flipped, negatives complemented).
void orc_topk(const float* score, int32_t* sel, int64_t T, int64_t n, int64_t ld, int64_t K) {
    for (int64_t r = 0; r < T; ++r) {
        std::vector<std::pair<uint32_t, int32_t>> v((size_t) n);
        for (int64_t j = 0; j < n; ++j) {
            uint32_t u;
            std::memcpy(&u, score + r * ld + j, 4);
            v[j] = {(u & 0x80000000u) ? ~u : (u | 0x80000000u), (int32_t) j};
        }
        std::sort(v.begin(), v.end(), [](const std::pair<uint32_t, int32_t>& a, const std::pair<uint32_t, int32_t>& b) {
            return a.first != b.first ? a.first > b.first : a.second < b.second;
        });
        const int64_t k = std::min(K, n);
        std::vector<int32_t> pos((size_t) k);
        for (int64_t i = 0; i < k; ++i) pos[i] = v[i].second;
        std::sort(pos.begin(), pos.end());
        for (int64_t i = 0; i < k; ++i) sel[r * K + i] = pos[i];
    }
}

// ---- deepseek41's indexer (kernels/llm/deepseek41/silo/k41.cpp:96-250,352-483) ---------------------------------------
// score of key j for row t: sum_h w[t][h] relu(q[t][h] . k_j); q fp32 [T][H][D], k fp16 [n][D].
//   the scalar form (k41.cpp:363-398): fp32 q; a head's dot product the sum of its 16-dim chunks' sums; the heads in order.
//   half_q, the matrix-unit form (k41.cpp:106-179; 32 heads): q rounded to fp16 as it is staged (k41.cpp:125-128); a head's
//   dot product one running sum over the dims; lane l takes heads l and l + 16 (k41.cpp:155-162), the 16 lanes' sums added
//   in lane order.
static float ds41_key_score(const float* q, const float* w, const uint16_t* k, int64_t t, int64_t j, int64_t H, int64_t D, bool half_q) {
    std::vector<float> term((size_t) H);
    for (int64_t h = 0; h < H; ++h) {
        float acc = 0.f;
        if (half_q) {
            for (int64_t c = 0; c < D; ++c) acc += round_h(q[(t * H + h) * D + c]) * h2f(k[j * D + c]);
        } else {
            for (int64_t c0 = 0; c0 < D; c0 += 16) {
                float part = 0.f;
                for (int64_t c = c0; c < c0 + 16; ++c) part += q[(t * H + h) * D + c] * h2f(k[j * D + c]);
                acc += part;
            }
        }
        term[h] = std::fmax(acc, 0.f) * w[t * H + h];
    }
    float s = 0.f;
    if (half_q && H % 16 == 0) {
        for (int l = 0; l < 16; ++l) {
            float sv = 0.f;
            for (int64_t h = l; h < H; h += 16) sv += term[h];
            s = l == 0 ? sv : s + sv;
        }
    } else {
        for (int64_t h = 0; h < H; ++h) s += term[h];
    }
    return s;
}
// ns_ds41_idx_score: score [T][ld], -inf from min(n, (pos0+t+1)/ratio) to ld
void orc_ds41_idx_score(const float* q, const float* w, const uint16_t* k, float* score, int64_t T, int64_t H, int64_t D, int64_t n, int64_t ld,
                        int64_t pos0, int64_t ratio, int half_q) {
#pragma omp parallel for collapse(2)
    for (int64_t t = 0; t < T; ++t)
        for (int64_t j = 0; j < ld; ++j) {
            const int64_t nv = std::min<int64_t>(n, (pos0 + t + 1) / ratio);
            score[t * ld + j] = j < nv ? ds41_key_score(q, w, k, t, j, H, D, half_q != 0) : NEG_INF;
        }
}
// ns_ds41_idx_score_cand: only over each row's candidate blocks of 8 keys (cand [T][K] block ids): score [T][K*8] compact
void orc_ds41_idx_score_cand(const float* q, const float* w, const uint16_t* k, const int32_t* cand, int64_t K, float* score, int64_t T, int64_t H,
                             int64_t D, int64_t n, int64_t pos0, int64_t ratio) {
    const int64_t nb = (n + 7) / 8;
    for (int64_t t = 0; t < T; ++t) {
        const int64_t nv = std::min<int64_t>(n, (pos0 + t + 1) / ratio);
        for (int64_t c = 0; c < K; ++c) {
            const int64_t b = cand[t * K + c];
            for (int e = 0; e < 8; ++e) {
                const int64_t j = b * 8 + e;
                score[t * K * 8 + c * 8 + e] = (b >= 0 && b < nb && j < nv) ? ds41_key_score(q, w, k, t, j, H, D, true) : NEG_INF;
            }
        }
    }
}
// ns_ds41_block_max: bmax [T][nb] = the best score of each bs positions; the block of the row's newest position +inf
void orc_ds41_block_max(const float* score, float* bmax, int64_t T, int64_t n, int64_t ld, int64_t bs, int64_t pos0, int64_t ratio) {
    const int64_t nb = (n + bs - 1) / bs;
    for (int64_t t = 0; t < T; ++t)
        for (int64_t b = 0; b < nb; ++b) {
            const int64_t lens = std::min<int64_t>(n, (pos0 + t + 1) / ratio);
            float m = NEG_INF;
            for (int64_t j = b * bs; j < std::min<int64_t>(n, (b + 1) * bs); ++j) m = std::fmax(m, score[t * ld + j]);
            if (lens > 0 && b == (lens - 1) / bs) m = INFINITY;
            bmax[t * nb + b] = m;
        }
}
// ns_ds41_cand_mask: score to -inf outside the blocks cand [T][K] lists
void orc_ds41_cand_mask(float* score, const int32_t* cand, int64_t T, int64_t n, int64_t ld, int64_t K, int64_t bs) {
    const int64_t nb = (n + bs - 1) / bs;
    for (int64_t t = 0; t < T; ++t) {
        std::vector<uint8_t> mark((size_t) nb, 0);
        for (int64_t c = 0; c < K; ++c) {
            const int32_t b = cand[t * K + c];
            if (b >= 0 && b < nb) mark[b] = 1;
        }
        for (int64_t j = 0; j < n; ++j)
            if (!mark[j / bs]) score[t * ld + j] = NEG_INF;
    }
}
// ns_ds41_cand_pos: the picks' compact indices (selc [T][kp], into the K*bs candidate keys) back to positions
void orc_ds41_cand_pos(const int32_t* selc, const int32_t* cand, int32_t* sel, int64_t T, int64_t K, int64_t kp, int64_t bs) {
    for (int64_t t = 0; t < T; ++t)
        for (int64_t i = 0; i < kp; ++i) {
            const int32_t c = selc[t * kp + i];
            sel[t * kp + i] = cand[t * K + c / bs] * (int32_t) bs + c % bs;
        }
}

// ---- cache writers -----------------------------------------------------------------------------------------------

// ns_q35_kv_store (kernels/llm/qwen35/q35.cpp:573-588): fp32 rows k [T][ks], v [T][vs] -> fp16 caches [Hkv][cap][D]
// at positions p0 ..
void orc_kv_store(const float* k, int64_t ks, const float* v, int64_t vs, int64_t T, int64_t Hkv, int64_t D, int64_t cap, int64_t p0, uint16_t* kc,
                  uint16_t* vc) {
    for (int64_t t = 0; t < T; ++t)
        for (int64_t h = 0; h < Hkv; ++h)
            for (int64_t d = 0; d < D; ++d) {
                const int64_t at = (h * cap + p0 + t) * D + d;
                kc[at] = f2h(k[t * ks + h * D + d]);
                vc[at] = f2h(v[t * vs + h * D + d]);
            }
}

// Merge of per-split partials (O unnormalised, m in log2 units, l), optionally with a per-head sink that joins the
// denominator only (kernels/llm/qwen35/silo/attn.cpp:352-368; sink form kernels/llm/deepseek41/silo/attn.cpp:266-285).
// part [rows][ns][PS] with O at 0..D-1, m at D, l at D+1; sinks (nullable) [rows] in natural-log units.
void orc_merge(const float* part, int64_t rows, int64_t ns, int64_t D, int64_t PS, const float* sinks, float* out) {
    for (int64_t r = 0; r < rows; ++r) {
        const float* pp = part + r * ns * PS;
        float mx = NEG_INF;
        for (int64_t k = 0; k < ns; ++k) mx = std::fmax(mx, pp[k * PS + D]);
        if (sinks) mx = std::fmax(mx, sinks[r] * LOG2E);
        for (int64_t d = 0; d < D; ++d) {
            float Ls = 0.f, A = 0.f;
            if (mx != NEG_INF) {
                for (int64_t k = 0; k < ns; ++k) {
                    const float e = std::exp2(pp[k * PS + D] - mx);
                    Ls += pp[k * PS + D + 1] * e;
                    A += pp[k * PS + d] * e;
                }
                if (sinks) Ls += std::exp2(sinks[r] * LOG2E - mx);
            }
            out[r * D + d] = Ls > 0.f ? A / Ls : 0.f;
        }
    }
}

}  // extern "C"
