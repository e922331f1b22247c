"""Builds oracle/_ref/lib*.so: the reference's own attention kernels, compiled for the CPU as a check on the oracle.

    python oracle/ref_build.py <path of a nextsycl checkout>

The reference's kernels are SYCL; its tree cannot be built without a SYCL toolchain and oneMKL. A kernel, though, is C++
once the SYCL names it uses exist. This script takes the kernels' source lines out of the checkout (nothing of them is kept
in this repository: the generated translation units live under oracle/_ref/, which is not committed), puts them behind a
host stand-in for those names (oracle/ref_shim/: work-groups as cooperative fibers, sub-groups, group collectives, local
memory, joint_matrix), and compiles the result with g++: libref.so (qwen35's q35.cpp, deepseek2, glm5next, deepseek41's
vector kernels and indexer), libref_nh.so (nemotronh's nh.cpp), and the three matrix-unit attention files, which share
names, as libref_q35x.so, libref_nhx.so and libref_ds41x.so. tests/test_ref_compiled.py then holds the oracle to the
reference's own code. Test infrastructure only."""
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

# (file within the checkout, first line of the piece as a regular expression, how the piece ends)
#   "brace": through the first following line that is a lone "}" (a function or template at file level)
#   "line": that one line; "brace2": two lines; a number: that many lines; "struct": through the first lone "};"
PIECES = [
    ("kernels/llm/qwen35/q35.cpp", r"^constexpr int SG = 16;", "line"),
    ("kernels/llm/qwen35/q35.cpp", r"^inline float kv_value\(", "brace"),
    ("kernels/llm/qwen35/q35.cpp", r"^constexpr int NSG_A = 4;", "line"),
    ("kernels/llm/qwen35/q35.cpp", r"^int64_t split_keys\(", "brace"),
    ("kernels/llm/qwen35/q35.cpp", r"^int64_t splits\(", "brace"),
    ("kernels/llm/qwen35/q35.cpp", (r"^template <int DL, int G>$", r"^void attn\("), "brace"),   # the decode / short-pass attention kernel and its merge
    ("kernels/llm/qwen35/q35.cpp", r"^int64_t ns_q35_attn_scratch\(", "brace"),
    ("kernels/llm/qwen35/q35.cpp", r"^int ns_q35_attn\(", "brace"),
    ("kernels/llm/qwen35/q35.cpp", r"^int ns_q35_qk_norm_rope\(", "brace"),
    ("kernels/llm/qwen35/q35.cpp", r"^int ns_q35_rope\(", "brace"),
    ("kernels/llm/qwen35/q35.cpp", r"^int ns_q35_qk_norm_rope_pos\(", "brace"),
    ("kernels/llm/qwen35/q35.cpp", r"^int ns_q35_attn_probs\(", "brace"),
    ("kernels/llm/qwen35/q35.cpp", r"^int ns_q35_kv_store_q\(", "brace"),
    ("kernels/llm/qwen35/q35.cpp", r"^int ns_q35_fwht32\(", "brace"),
    ("kernels/llm/qwen35/q35.cpp", r"^int ns_q35_kv_store\(", "brace"),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^template <int KT> constexpr int64_t kv_row\(\)", "line"),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^template <int KT>$", "brace"),          # kv_load8: the reader of a cache row
    ("kernels/llm/deepseek2/ds2.cpp", r"^inline float yarn_ramp\(", "brace"),
    ("kernels/llm/deepseek2/ds2.cpp", r"^inline void yarn_cs\(", "brace"),
    ("kernels/llm/deepseek2/ds2.cpp", r"^int ns_ds2_rope\(", "brace"),
    ("kernels/llm/deepseek2/ds2.cpp", r"^int ns_ds2_kv_store\(", "brace"),
    ("kernels/llm/deepseek2/ds2.cpp", r"^struct Q6KBlock ", "line"),
    ("kernels/llm/deepseek2/ds2.cpp", r"^inline void q6k_cols32\(", "brace"),
    ("kernels/llm/deepseek2/ds2.cpp", (r"^template <bool Q6>$", r"^void mla_decode_t\("), "brace"),   # the fused absorbed-MLA decode kernel
    ("kernels/llm/deepseek2/ds2.cpp", r"^int ns_ds2_mla_decode\(", "brace"),
    ("kernels/llm/deepseek2/ds2.cpp", r"^int ns_ds2_mla_decode_q6k\(", "brace"),
    ("kernels/llm/glm5next/glm.cpp", r"^template <int L>$", "brace2"),               # q8_row_bytes: two lines
    ("kernels/llm/glm5next/glm.cpp", r"^int ns_mla_attend\(", "brace"),
    ("kernels/llm/glm5next/glm.cpp", r"^int ns_gather_h\(", "brace"),
    ("kernels/llm/glm5next/glm.cpp", r"^int ns_idx_pool\(", "brace"),
    ("kernels/llm/glm5next/glm.cpp", r"^int ns_idx_score\(", "brace"),
    ("kernels/llm/glm5next/glm.cpp", r"^int ns_topk\(", "brace"),
    ("kernels/llm/glm5next/glm.cpp", r"^int ns_mla_cells\(", "brace"),
    ("kernels/llm/glm5next/glm.cpp", r"^int ns_softmax_masked\(", "brace"),
    ("kernels/llm/glm5next/glm.cpp", (r"^template <int L, bool Q8 = false>$", r"^static void mla_dec\("), "brace"),   # the selected-cell decode kernel
    ("kernels/llm/glm5next/glm.cpp", (r"^template <int HG>$", r"^static void mla_sel\("), "brace"),
    ("kernels/llm/glm5next/glm.cpp", r"^int ns_mla_attend_sel\(", "brace"),
    ("kernels/llm/glm5next/glm.cpp", r"^int ns_mla_attend_sel_q8\(", "brace"),
    ("kernels/llm/glm5next/glm.cpp", r"^int ns_to_f16\(", "brace"),
    ("kernels/llm/glm5next/glm.cpp", r"^int ns_to_q8row\(", "brace"),
    ("kernels/llm/glm5next/glm.cpp", r"^int ns_gather_q8_h\(", "brace"),
    ("kernels/llm/deepseek41/silo/ds41.cpp", r"^int ns_ds41_rows_f16\(", "brace"),
    ("kernels/llm/deepseek41/silo/ds41.cpp", r"^int ns_ds41_ring_put\(", "brace"),
    ("kernels/llm/deepseek41/silo/ds41.cpp", (r"^template <int HG>$", r"^void attend\("), "brace"),   # the vector form of the MQA-512 attention with sinks
    ("kernels/llm/deepseek41/silo/ds41.cpp", r"^int ns_ds41_attend\(", "brace"),
    ("kernels/llm/deepseek41/silo/k41.cpp", r"^inline float pow2_ceil\(", "brace"),
    ("kernels/llm/deepseek41/silo/k41.cpp", r"^inline float e4m3_round\(", "brace"),
    ("kernels/llm/deepseek41/silo/k41.cpp", r"^namespace jmi = ", "line"),
    ("kernels/llm/deepseek41/silo/k41.cpp", r"^constexpr int IXD = 128, IXH = 32,", "line"),
    ("kernels/llm/deepseek41/silo/k41.cpp", (r"^template <typename T>$", r"^inline auto ix_lp\("), "brace"),
    ("kernels/llm/deepseek41/silo/k41.cpp", (r"^template <typename T>$", r"^inline auto ix_gp\("), "brace"),
    ("kernels/llm/deepseek41/silo/k41.cpp", r"^void idx_score_xmx\(", "brace"),          # the indexer's scores on the matrix units
    ("kernels/llm/deepseek41/silo/k41.cpp", r"^void idx_score_cand_xmx\(", "brace"),
    ("kernels/llm/deepseek41/silo/k41.cpp", r"^int ns_ds41_idx_score\(", "brace"),       # and their scalar form
    ("kernels/llm/deepseek41/silo/k41.cpp", r"^int ns_ds41_idx_score_cand\(", "brace"),
    ("kernels/llm/deepseek41/silo/k41.cpp", r"^inline float kv_yarn_ramp\(", "brace"),
    ("kernels/llm/deepseek41/silo/k41.cpp", r"^inline void kv_yarn_cs\(", "brace"),
    ("kernels/llm/deepseek41/silo/k41.cpp", r"^int ns_ds41_kv_post\(", "brace"),
    ("kernels/llm/deepseek41/silo/k41.cpp", r"^int ns_ds41_att_post\(", "brace"),
    ("kernels/llm/deepseek41/silo/k41.cpp", r"^int ns_ds41_block_max\(", "brace"),
    ("kernels/llm/deepseek41/silo/k41.cpp", r"^int ns_ds41_cand_mask\(", "brace"),
    ("kernels/llm/deepseek41/silo/k41.cpp", r"^int ns_ds41_cand_pos\(", "brace"),
]

# a second translation unit: nemotronh's attention carries the same names as qwen35's
PIECES_NH = [
    ("kernels/llm/nemotronh/nh.cpp", r"^constexpr int SG = 16;", "line"),
    ("kernels/llm/nemotronh/nh.cpp", r"^constexpr int NSG_A = 4;", "line"),
    ("kernels/llm/nemotronh/nh.cpp", r"^int64_t split_keys\(", "brace"),
    ("kernels/llm/nemotronh/nh.cpp", r"^int64_t splits\(", "brace"),
    ("kernels/llm/nemotronh/nh.cpp", (r"^template <int DL, int G>$", r"^void attn\("), "brace"),
    ("kernels/llm/nemotronh/nh.cpp", r"^constexpr int GA = 8;", "line"),
    ("kernels/llm/nemotronh/nh.cpp", r"^int64_t ns_nh_attn_scratch\(", "brace"),
    ("kernels/llm/nemotronh/nh.cpp", r"^int ns_nh_attn\(", "brace"),
]

# the matrix-unit form of qwen35's attention (prompt blocks of 8 rows, and decode rows split over the keys), on the host's
# joint_matrix stand-in
PIECES_Q35X = [
    ("kernels/llm/qwen35/silo/attn.cpp", r"^namespace jm = ", "line"),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^#ifndef Q35_ATTN_CH", 3),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^#ifndef Q35_ATTN_KPAD", 3),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^constexpr int D = 256, HALF_D = 128, SG = 16, M = 8,", "line"),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^template <int KT> constexpr int64_t kv_row\(\)", "line"),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^template <int KT>$", "brace"),
    ("kernels/llm/qwen35/silo/attn.cpp", (r"^template <typename T>$", r"^inline auto lp\("), "brace"),
    ("kernels/llm/qwen35/silo/attn.cpp", (r"^template <typename T>$", r"^inline auto gp\("), "brace"),
    ("kernels/llm/qwen35/silo/attn.cpp", (r"^template <int G>$", r"^struct Slm \{"), "struct"),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^int64_t dec_splits\(int64_t kv, int64_t Hkv\);", "line"),
    ("kernels/llm/qwen35/silo/attn.cpp", (r"^template <int G, bool SPLIT, int KT>$", r"^void attn_flash\("), "brace"),
    ("kernels/llm/qwen35/silo/attn.cpp", (r"^template <int G, int KT>$", r"^void attn_prompt\("), "brace"),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^constexpr int KEYS_D = 64;", "line"),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^int64_t dec_split\(", "brace"),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^int64_t dec_splits\(int64_t kv, int64_t Hkv\) \{", "brace"),
    ("kernels/llm/qwen35/silo/attn.cpp", (r"^template <int G, int KT>$", r"^void flash_decode\("), "brace"),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^int ns_q35_attn_prompt_supported\(", "brace"),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^int ns_q35_attn_prompt\(", "brace"),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^int ns_q35_attn_prompt_kv\(", "brace"),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^int ns_q35_attn_decode_supported\(", "brace"),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^int64_t ns_q35_attn_decode_scratch\(", "brace"),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^int ns_q35_attn_decode\(", "brace"),
    ("kernels/llm/qwen35/silo/attn.cpp", r"^int ns_q35_attn_decode_kv\(", "brace"),
]

# nemotronh's attention on the matrix units: heads of 128, 16 query heads a key head
_NHX = "kernels/llm/nemotronh/silo/attn.cpp"
PIECES_NHX = [
    (_NHX, r"^namespace jm = ", "line"),
    (_NHX, r"^#ifndef NH_ATTN_CH$", 3),
    (_NHX, r"^#ifndef NH_ATTN_KPAD$", 3),
    (_NHX, r"^constexpr int D = 128, HALF_D = 64, SG = 16, M = 8,", "line"),
    (_NHX, (r"^template <typename T>$", r"^inline auto lp\("), "brace"),
    (_NHX, (r"^template <typename T>$", r"^inline auto gp\("), "brace"),
    (_NHX, (r"^template <int G>$", r"^struct Slm \{"), "struct"),
    (_NHX, r"^int64_t dec_splits\(int64_t kv, int64_t Hkv\);", "line"),
    (_NHX, (r"^template <int G, bool SPLIT>$", r"^void attn_flash\("), "brace"),
    (_NHX, (r"^template <int G>$", r"^void attn_prompt\("), "brace"),
    (_NHX, r"^constexpr int KEYS_D = 64;", "line"),
    (_NHX, r"^int64_t dec_split\(", "brace"),
    (_NHX, r"^int64_t dec_splits\(int64_t kv, int64_t Hkv\) \{", "brace"),
    (_NHX, (r"^template <int G>$", r"^void flash_decode\("), "brace"),
    (_NHX, r"^int ns_nhs_attn_prompt_supported\(", "brace"),
    (_NHX, r"^int ns_nhs_attn_prompt\(", "brace"),
    (_NHX, r"^int ns_nhs_attn_decode_supported\(", "brace"),
    (_NHX, r"^int64_t ns_nhs_attn_decode_scratch\(", "brace"),
    (_NHX, r"^int ns_nhs_attn_decode\(", "brace"),
]

# deepseek41's attention on the matrix units: the prompt form and decode's split form with its merge
PIECES_DS41X = [
    ("kernels/llm/deepseek41/silo/attn.cpp", r"^namespace jm = ", "line"),
    ("kernels/llm/deepseek41/silo/attn.cpp", r"^#ifndef DS4_ATTN_CH$", 3),
    ("kernels/llm/deepseek41/silo/attn.cpp", r"^#ifndef DS4_ATTN_CH_DEC$", 3),
    ("kernels/llm/deepseek41/silo/attn.cpp", r"^constexpr int D = 512, QD = 128,", "line"),
    ("kernels/llm/deepseek41/silo/attn.cpp", r"^constexpr float LOG2E = ", "line"),
    ("kernels/llm/deepseek41/silo/attn.cpp", (r"^template <typename T>$", r"^inline auto lp\("), "brace"),
    ("kernels/llm/deepseek41/silo/attn.cpp", (r"^template <typename T>$", r"^inline auto gp\("), "brace"),
    ("kernels/llm/deepseek41/silo/attn.cpp", (r"^template <int G, int C>$", r"^struct Slm \{"), "struct"),
    ("kernels/llm/deepseek41/silo/attn.cpp", r"^constexpr int PS = D \+ 16;", "line"),
    ("kernels/llm/deepseek41/silo/attn.cpp", (r"^template <int G, bool SPLIT, int C = CH>$", r"^void attend_xmx\("), "brace"),
    ("kernels/llm/deepseek41/silo/attn.cpp", r"^void attend_q16\(", "brace"),
    ("kernels/llm/deepseek41/silo/attn.cpp", r"^void attend_merge\(", "brace"),
    ("kernels/llm/deepseek41/silo/attn.cpp", r"^float\* part_buf\(", "brace"),
    ("kernels/llm/deepseek41/silo/attn.cpp", r"^int ns_ds41_attend_xmx_supported\(", "brace"),
    ("kernels/llm/deepseek41/silo/attn.cpp", r"^int ns_ds41_attend_xmx\(", "brace"),
]

HEAD = r'''// GENERATED by oracle/ref_build.py from a nextsycl checkout: the reference's own lines between the markers. Not committed.
#include <sycl/sycl.hpp>
#include <sycl/ext/oneapi/matrix/matrix.hpp>
#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <string>
#include <vector>
using half = sycl::half;
struct ns_gpu { sycl::queue q; };
static std::string ref_last_error;
static int ns_fail(const std::string& what) { ref_last_error = what; return -1; }
#define NS_TRY
#define NS_CATCH
'''
# ns_ds41_attend asks whether the matrix-unit form may take the call: in its unit it may not (that form is a unit of its own)
HEAD_VECTOR_ONLY = r'''static int ns_ds41_attend_xmx_supported(int64_t, int64_t) { return 0; }
template <class... A> static int ns_ds41_attend_xmx(A...) { return -1; }
'''

TAIL = r'''
// ---- entry points for what the reference keeps internal (this file's own lines) ----
extern "C" {
const char* ref_error() { return ref_last_error.c_str(); }
// the sub-group size of the launches that follow (the kernels' [[sycl::reqd_sub_group_size]] means nothing to g++)
int ref_sub_group_size = 16;
void* ref_gpu() { static ns_gpu g; sycl::detail::sub_group_size_setting() = &ref_sub_group_size; return &g; }
// features 8c .. 8c + 7 of a cache row of form kt (1 q8_0, 2 q4_0) as the reference's reader returns them: 8 halves
void ref_kv_load8(int kt, const uint8_t* row, int c, uint16_t* out8) {
    const sycl::uint4 w = kt == 1 ? kv_load8<1>(row, c) : kv_load8<2>(row, c);
    const uint32_t v[4] = {w.x(), w.y(), w.z(), w.w()};
    for (int i = 0; i < 4; ++i) { out8[2 * i] = (uint16_t) (v[i] & 0xffff); out8[2 * i + 1] = (uint16_t) (v[i] >> 16); }
}
int64_t ref_kv_row(int kt) { return kt == 0 ? kv_row<0>() : kt == 1 ? kv_row<1>() : kv_row<2>(); }
// columns [32 k, 32 k + 32) of a 512-wide Q6_K row (two 210-byte blocks)
void ref_q6k_cols32(const void* row, int k, float* v32) {
    float v[32];
    q6k_cols32(reinterpret_cast<const Q6KBlock*>(row), k, v);
    for (int i = 0; i < 32; ++i) v32[i] = v[i];
}
int64_t ref_q8_row_bytes_512() { return q8_row_bytes<512>(); }
}
'''


def take(lines, start_re, how, path):
    # start_re: one expression for the piece's first line, or a pair for its first two lines
    first, second = (start_re, None) if isinstance(start_re, str) else start_re
    rx, rx2 = re.compile(first), re.compile(second) if second else None
    for i, ln in enumerate(lines):
        if rx.search(ln) and (rx2 is None or (i + 1 < len(lines) and rx2.search(lines[i + 1]))):
            if how == "line":
                return lines[i:i + 1]
            if how == "brace2":
                return lines[i:i + 2]
            if isinstance(how, int):
                return lines[i:i + how]
            for j in range(i + 1, len(lines)):
                if lines[j].rstrip() == ("};" if how == "struct" else "}"):
                    return lines[i:j + 1]
            break
    raise SystemExit(f"ref_build: the piece {start_re!r} was not found in {path} (the checkout differs from the one this was written against)")


def build_unit(checkout, pieces, tail, name, head=""):
    os.makedirs(OUT, exist_ok=True)
    parts = [HEAD, head, 'extern "C++" {\n']
    for rel, start_re, how in pieces:
        path = os.path.join(checkout, rel)
        with open(path, encoding="utf-8") as f:
            lines = f.read().split("\n")
        piece = take(lines, start_re, how, rel)
        linkage = 'extern "C" ' if re.match(r"^int(64_t)? ns_", piece[0]) else ""
        parts.append(f"// ---- {rel}\n{linkage}" + "\n".join(piece) + "\n")
    parts.append("}\n" + tail)
    src = os.path.join(OUT, name + ".cpp")
    with open(src, "w", encoding="utf-8") as f:
        f.write("".join(parts))
    so = os.path.join(OUT, "lib" + name + ".so")
    cmd = ["g++", "-O2", "-march=x86-64-v3", "-ffp-contract=off", "-std=c++17", "-fPIC", "-shared", "-Wno-attributes", "-Wno-unknown-pragmas",
           "-I", os.path.join(HERE, "ref_shim"), "-o", so, src]
    subprocess.check_call(cmd)
    return so


TAIL_NH = r'''
extern "C" {
const char* ref_error() { return ref_last_error.c_str(); }
void* ref_gpu() { static ns_gpu g; return &g; }
}
'''


def build(checkout):
    build_unit(checkout, PIECES_NH, TAIL_NH, "ref_nh")
    build_unit(checkout, PIECES_Q35X, TAIL_NH, "ref_q35x")
    build_unit(checkout, PIECES_DS41X, TAIL_NH, "ref_ds41x")
    build_unit(checkout, PIECES_NHX, TAIL_NH, "ref_nhx")
    return build_unit(checkout, PIECES, TAIL, "ref", HEAD_VECTOR_ONLY)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(build(sys.argv[1]))
