"""ctypes front of the CPU oracle (oracle/attn_oracle.cpp -> oracle/liboracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke test and by the benchmark's CPU-baseline leg, never by the
library. Parity: the deepseek41 functions are pinned to fixtures produced by running the reference's own Python
(tests/golden/make_ref_fixtures.py), and every function whose reference kernel has its source in the tree to that kernel,
compiled for the CPU behind a host stand-in for SYCL work-groups, sub-groups and joint_matrix (`build_ref`, `ref_lib`,
`ref_nh_lib`, `ref_unit`; tests/test_ref_compiled.py); the steps the reference computes with oneMKL are unpinned (see
attn_oracle.cpp's header).

Arrays are numpy: fp32 as float32, fp16 / bf16 storage as uint16 bit patterns (`np.float16.view(np.uint16)` for fp16;
`to_bf16_bits` below for bf16).
"""
import ctypes as C
import os
import subprocess
import sys

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")
_lib = None

i64 = C.c_int64
_pf = C.POINTER(C.c_float)
_pd = C.POINTER(C.c_double)
_ph = C.POINTER(C.c_uint16)
_pi = C.POINTER(C.c_int32)


def build(force=False):
    """Compiles the oracle with its Makefile (g++, OpenMP)."""
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(os.path.join(_HERE, "attn_oracle.cpp")):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _SO


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.orc_threads.restype = C.c_int
        for n in ("orc_flash_split", "orc_flash_splits"):
            getattr(_lib, n).restype = i64
            getattr(_lib, n).argtypes = [i64, i64]
        for n in ("orc_plain_split", "orc_plain_splits"):
            getattr(_lib, n).restype = i64
            getattr(_lib, n).argtypes = [i64, i64, i64]
    return _lib


_REF_SO = os.path.join(_HERE, "_ref", "libref.so")
_ref = None


def build_ref(checkout):
    """Compiles oracle/_ref/libref.so - a few of the reference's own kernels for the CPU - from a nextsycl checkout
    (oracle/ref_build.py). Returns the path, or None when the checkout is not there."""
    if not os.path.isdir(os.path.join(checkout, "kernels", "llm")):
        return None
    sys_path = os.path.join(_HERE, "ref_build.py")
    subprocess.check_call([sys.executable, sys_path, checkout], stdout=subprocess.DEVNULL)
    return _REF_SO


def ref_lib():
    """The reference's own kernels compiled for the CPU (see build_ref), or None when they were not built."""
    global _ref
    if _ref is None and os.path.exists(_REF_SO):
        _ref = C.CDLL(_REF_SO)
        _ref.ref_gpu.restype = C.c_void_p
        _ref.ref_error.restype = C.c_char_p
        _ref.ref_kv_row.restype = i64
        _ref.ref_q8_row_bytes_512.restype = i64
    return _ref


_REF_NH_SO = os.path.join(_HERE, "_ref", "libref_nh.so")
_ref_nh = None


def ref_nh_lib():
    """nemotronh's attention kernel compiled for the CPU (a unit of its own: it carries the same names as qwen35's)."""
    global _ref_nh
    if _ref_nh is None and os.path.exists(_REF_NH_SO):
        _ref_nh = C.CDLL(_REF_NH_SO)
        _ref_nh.ref_gpu.restype = C.c_void_p
        _ref_nh.ref_error.restype = C.c_char_p
        _ref_nh.ns_nh_attn_scratch.restype = i64
    return _ref_nh


_units = {}


def ref_unit(name):
    """Another unit of the reference's kernels compiled for the CPU (oracle/_ref/lib<name>.so), or None when not built."""
    if name not in _units:
        so = os.path.join(_HERE, "_ref", "lib" + name + ".so")
        if not os.path.exists(so):
            return None
        u = C.CDLL(so)
        u.ref_gpu.restype = C.c_void_p
        u.ref_error.restype = C.c_char_p
        _units[name] = u
    return _units[name]


def threads():
    return int(lib().orc_threads())


def use_all_cores():
    """Makes later calls use every core this process may run on, whatever OMP_NUM_THREADS said; returns the count."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_threads.restype = C.c_int
    return int(lib().orc_set_threads(C.c_int(n)))


def _f(a):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_pf)


def _h(a):
    assert a.dtype == np.uint16 and a.flags.c_contiguous
    return a.ctypes.data_as(_ph)


def to_f16_bits(x):
    return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def to_bf16_bits(x):
    """fp32 -> bf16 bit patterns, round to nearest even."""
    w = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    w = w + 0x7FFF + ((w >> 16) & 1)
    return (w >> 16).astype(np.uint16)


def from_bf16_bits(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def flash_split(kv, hkv):
    return int(lib().orc_flash_split(kv, hkv))


def flash_splits(kv, hkv):
    return int(lib().orc_flash_splits(kv, hkv))


def gqa_flash_prefill(q, kc, vc, T, Hq, Hkv, D, cap, p0):
    """q fp32 [T, Hq*D]; kc, vc uint16 [Hkv, cap, D] -> fp32 [T, Hq*D] (flash numerics, one split a row)."""
    out = np.empty((T, Hq * D), np.float32)
    lib().orc_gqa_flash_prefill(_f(q), i64(q.shape[1]), _h(kc), _h(vc), i64(T), i64(Hq), i64(Hkv), i64(D), i64(cap), i64(p0), _f(out))
    return out


def gqa_flash_decode(q, kc, vc, T, Hq, Hkv, D, cap, p0):
    """Decode rows (T <= 8) with the reference's own key splits and merge."""
    out = np.empty((T, Hq * D), np.float32)
    lib().orc_gqa_flash_decode(_f(q), i64(q.shape[1]), _h(kc), _h(vc), i64(T), i64(Hq), i64(Hkv), i64(D), i64(cap), i64(p0), _f(out), None)
    return out


def gqa_plain(q, kc, vc, T, Hq, Hkv, D, cap, p0, groups=None):
    out = np.empty((T, Hq * D), np.float32)
    lib().orc_gqa_plain(_f(q), i64(q.shape[1]), _h(kc), _h(vc), i64(T), i64(Hq), i64(Hkv), i64(D), i64(cap), i64(p0),
                        i64(Hkv if groups is None else groups), _f(out))
    return out


def attn_exact(q, kc, vc, T, Hq, Hkv, Dqk, Dv, cap, p0, scale, kind=0):
    """fp64 yardstick. kind 0: fp16 caches, 1: bf16. -> float64 [T, Hq*Dv]."""
    out = np.empty((T, Hq * Dv), np.float64)
    lib().orc_attn_exact(_f(q), i64(q.shape[1]), _h(kc), _h(vc), C.c_int(kind), i64(T), i64(Hq), i64(Hkv), i64(Dqk), i64(Dv), i64(cap), i64(p0),
                         C.c_double(scale), out.ctypes.data_as(_pd))
    return out


def attn_tc(q, kc, vc, T, Hq, Hkv, Dqk, Dv, cap, p0, scale, kind=0):
    """Tensor-core numerics with the storage type a parameter (0 fp16, 1 bf16) -> fp32 [T, Hq*Dv]."""
    out = np.empty((T, Hq * Dv), np.float32)
    lib().orc_attn_tc(_f(q), i64(q.shape[1]), _h(kc), _h(vc), C.c_int(kind), i64(T), i64(Hq), i64(Hkv), i64(Dqk), i64(Dv), i64(cap), i64(p0),
                      C.c_float(scale), _f(out))
    return out


def mla_fused(q, cache, T, H, L, R, pos0, scale):
    """q fp32 [T, H, L+R]; cache uint16 [n, L+R] -> fp32 [T, H, L] (deepseek2's fused decode kernel, middle stage)."""
    u = np.empty((T, H, L), np.float32)
    lib().orc_mla_fused(_f(q), _h(cache), i64(T), i64(H), i64(L), i64(R), i64(pos0), C.c_float(scale), _f(u))
    return u


def mla_gemm(q, cache, T, H, L, R, pos0, scale):
    u = np.empty((T, H, L), np.float32)
    lib().orc_mla_gemm(_f(q), _h(cache), i64(T), i64(H), i64(L), i64(R), i64(pos0), C.c_float(scale), _f(u))
    return u


def mla_exact(q, cache, T, H, L, R, pos0, scale):
    u = np.empty((T, H, L), np.float64)
    lib().orc_mla_exact(_f(q), _h(cache), i64(T), i64(H), i64(L), i64(R), i64(pos0), C.c_double(scale), u.ctypes.data_as(_pd))
    return u


def mla_attend_f32(qa, c, T, H, L, pos0, scale):
    u = np.empty((T, H, L), np.float32)
    lib().orc_mla_attend_f32(_f(qa), _f(c), _f(u), i64(T), i64(H), i64(L), i64(pos0), C.c_float(scale))
    return u


def to_q8row(x):
    """fp32 [n, 512] -> uint8 [n, 544] (16 fp16 scales then 512 int8)."""
    n = x.shape[0]
    y = np.empty((n, 544), np.uint8)
    lib().orc_to_q8row(_f(x), y.ctypes.data_as(C.POINTER(C.c_uint8)), i64(n))
    return y


def mla_dec512(qa, c, T, H, pos0, scale, sel=None, sel_cnt=None, K=0, q8=False):
    u = np.empty((T, H, 512), np.float32)
    lib().orc_mla_dec512(_f(qa), c.ctypes.data_as(C.c_void_p), _f(u), i64(T), i64(H), i64(pos0), C.c_float(scale),
                         None if sel is None else sel.ctypes.data_as(_pi), None if sel_cnt is None else sel_cnt.ctypes.data_as(_pi), i64(K),
                         C.c_int(1 if q8 else 0))
    return u


def kv_store(k, v, T, Hkv, D, cap, p0, kc, vc):
    lib().orc_kv_store(_f(k), i64(k.shape[1]), _f(v), i64(v.shape[1]), i64(T), i64(Hkv), i64(D), i64(cap), i64(p0), _h(kc), _h(vc))


def merge(part, rows, ns, D, PS, sinks=None):
    out = np.empty((rows, D), np.float32)
    lib().orc_merge(_f(part), i64(rows), i64(ns), i64(D), i64(PS), None if sinks is None else _f(sinks), _f(out))
    return out


def ds41_attend(q, raw, R, comp, ratio, sel, K, sinks, T, H, pos0, window, scale, mode=1):
    """deepseek41's MQA-512 with sinks. q fp32 [T, H, 512]; raw uint16 [R, 512]; comp uint16 [n, 512] or None; sel int32
    [T, K] or None; sinks fp32 [H]. mode 0: the vector kernel's numerics, 1: the XMX kernel's."""
    out = np.empty((T, H, 512), np.float32)
    lib().orc_ds41_attend(_f(q), _h(raw), i64(R), None if comp is None else _h(comp), i64(ratio), None if sel is None else sel.ctypes.data_as(_pi),
                          i64(K), _f(sinks), _f(out), i64(T), i64(H), i64(pos0), i64(window), C.c_float(scale), C.c_int(mode))
    return out


def q_row_bytes(kt):
    return {0: 512, 1: 272, 2: 144}[kt]


def kv_store_q(kt, k, v, T, Hkv, cap, p0, kc, vc):
    """fp32 rows k, v [T, Hkv*256] into quantised caches kc, vc uint8 [Hkv, cap, row bytes] (kt 1: q8_0, 2: q4_0)."""
    u8 = C.POINTER(C.c_uint8)
    lib().orc_kv_store_q(C.c_int(kt), _f(k), i64(k.shape[1]), _f(v), i64(v.shape[1]), i64(T), i64(Hkv), i64(cap), i64(p0), kc.ctypes.data_as(u8),
                         vc.ctypes.data_as(u8))


def kv_dequant(kt, c, Hkv, cap, n):
    """Rows [0, n) of each head of a quantised cache as the fp16 values the reference's reader produces -> uint16 [Hkv, n, 256]."""
    out = np.empty((Hkv, n, 256), np.uint16)
    lib().orc_kv_dequant(C.c_int(kt), c.ctypes.data_as(C.POINTER(C.c_uint8)), i64(Hkv), i64(cap), i64(n), _h(out))
    return out


def fwht32(x):
    """In place: each block of 32 of the rows of x [rows, n] fp32 through the normalised Walsh-Hadamard transform."""
    lib().orc_fwht32(_f(x), i64(x.shape[0]), i64(x.shape[1]), i64(x.shape[1]))
    return x


def qk_norm_rope(x, T, H, D, w, eps, n_rot, theta, p0=0, pos3=None, sections=(0, 0, 0)):
    """x fp32 [T, H*D] -> fp32 [T, H*D]: RMS norm (w None: none) then rotate-half rotary positions over the first n_rot features."""
    y = np.empty((T, H * D), np.float32)
    lib().orc_qk_norm_rope(_f(x), i64(x.shape[1]), i64(D), _f(y), i64(H * D), i64(T), i64(H), i64(D), None if w is None else _f(w), C.c_float(eps),
                           i64(n_rot), C.c_float(theta), i64(p0), None if pos3 is None else pos3.ctypes.data_as(_pi), i64(sections[0]), i64(sections[1]),
                           i64(sections[2]))
    return y


def ds2_rope(x, T, H, row, head, off, n_dims, pos0, freq_base, freq_scale, ext_factor, mscale, corr0, corr1, out=None, out_row=0, out_head=0):
    """YaRN rotary positions in place on x (fp32, flat); `out` (fp32, flat) also receives the rotated part."""
    f = C.c_float
    lib().orc_ds2_rope(_f(x), i64(T), i64(H), i64(row), i64(head), i64(off), i64(n_dims), i64(pos0), f(freq_base), f(freq_scale), f(ext_factor), f(mscale),
                       f(corr0), f(corr1), None if out is None else _f(out), i64(out_row), i64(out_head))
    return x


def ds2_kv_store(kv, w, eps, cache, T, L, R, pos0, freq_base, freq_scale, ext_factor, mscale, corr0, corr1):
    """kv fp32 [T, L+R] into rows pos0.. of the latent cache (uint16 [n, L+R]): L RMS-normed with w, R rotated."""
    f = C.c_float
    lib().orc_ds2_kv_store(_f(kv), _f(w), f(eps), _h(cache), i64(T), i64(L), i64(R), i64(pos0), f(freq_base), f(freq_scale), f(ext_factor), f(mscale), f(corr0),
                           f(corr1))


def ds41_kv_post(kv, w, T, D, eps, rd, pos0, yarn, ring, R):
    """In place on kv fp32 [T, D] and into ring (uint16 [R, D]); yarn = (freq_base, freq_scale, ext_factor, mscale, corr0, corr1)."""
    f = C.c_float
    lib().orc_ds41_kv_post(_f(kv), _f(w), i64(T), i64(D), f(eps), i64(rd), i64(pos0), *[f(v) for v in yarn], _h(ring), i64(R))


def ds41_att_post(x, T, H, D, rd, pos0, yarn):
    """In place on x fp32 [T, H, D]."""
    f = C.c_float
    lib().orc_ds41_att_post(_f(x), i64(T), i64(H), i64(D), i64(rd), i64(pos0), *[f(v) for v in yarn])


def q35_attn_probs(kt, q, kc, Hq, Hkv, cap, n, mode, out):
    """One query row q fp32 [Hq*256] over the first n keys of a cache of form kt (uint8 view); adds to out fp32 [n]; -> scratch [Hq, 2]."""
    scratch = np.zeros((Hq, 2), np.float32)
    lib().orc_q35_attn_probs(C.c_int(kt), _f(q), kc.ctypes.data_as(C.POINTER(C.c_uint8)), i64(Hq), i64(Hkv), i64(cap), i64(n), C.c_int(mode), _f(scratch), _f(out))
    return scratch


def idx_pool(ring, ik, ig, ape, pooled, pos0, T, D):
    """Writes rows pos0//4 .. (pos0+T)//4 - 1 of pooled (fp32 [pools, D], indexed by pool); ring fp32 [8, 2D] is read, then updated."""
    lib().orc_idx_pool(_f(ring), _f(ik), _f(ig), _f(ape), _f(pooled), i64(pos0), i64(T), i64(D))


def idx_score(S, w, score, T, H, j0, n, pos0):
    """S fp32 [T*H, n], w fp32 [T, H]; writes score[r, j0:j0+n] (score fp32 [T, ld])."""
    lib().orc_idx_score(_f(S), _f(w), _f(score), i64(T), i64(H), i64(j0), i64(n), i64(score.shape[1]), i64(pos0))


def topk(score, n, K):
    """score fp32 [T, ld] -> sel int32 [T, K] (entries past min(K, n) stay -1)."""
    T = score.shape[0]
    sel = np.full((T, K), -1, np.int32)
    lib().orc_topk(_f(score), sel.ctypes.data_as(_pi), i64(T), i64(n), i64(score.shape[1]), i64(K))
    return sel


def ds41_idx_score(q, w, k, T, H, D, n, ld, pos0, ratio, half_q=True):
    score = np.empty((T, ld), np.float32)
    lib().orc_ds41_idx_score(_f(q), _f(w), _h(k), _f(score), i64(T), i64(H), i64(D), i64(n), i64(ld), i64(pos0), i64(ratio), C.c_int(1 if half_q else 0))
    return score


def ds41_idx_score_cand(q, w, k, cand, K, T, H, D, n, pos0, ratio):
    score = np.empty((T, K * 8), np.float32)
    lib().orc_ds41_idx_score_cand(_f(q), _f(w), _h(k), cand.ctypes.data_as(_pi), i64(K), _f(score), i64(T), i64(H), i64(D), i64(n), i64(pos0), i64(ratio))
    return score


def ds41_block_max(score, n, bs, pos0, ratio):
    T, ld = score.shape
    bmax = np.empty((T, -(-n // bs)), np.float32)
    lib().orc_ds41_block_max(_f(score), _f(bmax), i64(T), i64(n), i64(ld), i64(bs), i64(pos0), i64(ratio))
    return bmax


def ds41_cand_mask(score, cand, n, bs):
    T, ld = score.shape
    lib().orc_ds41_cand_mask(_f(score), cand.ctypes.data_as(_pi), i64(T), i64(n), i64(ld), i64(cand.shape[1]), i64(bs))
    return score


def ds41_cand_pos(selc, cand, bs):
    T, kp = selc.shape
    sel = np.empty((T, kp), np.int32)
    lib().orc_ds41_cand_pos(selc.ctypes.data_as(_pi), cand.ctypes.data_as(_pi), sel.ctypes.data_as(_pi), i64(T), i64(cand.shape[1]), i64(kp), i64(bs))
    return sel


def gemm_batch_h(batch, trans_w, T, N, K, x, ldx, sx, w, ldw, sw, y=None, ldy=None, sy=None):
    """kernels/llm/glm5next/glm.cpp:264-277 (a oneMKL gemm_batch in the reference; its summation order is unspecified, so the
    checker sums in float64): y_b [T, N] (+)= x_b [T, K] . op(w_b) over flat fp16 arrays x, w (uint16 bit patterns) with
    the call's strides; y (flat float32, or None for zeros) supplies what is accumulated onto. -> float64 [batch, T, N]."""
    xf, wf = x.view(np.float16).astype(np.float64), w.view(np.float16).astype(np.float64)
    out = np.zeros((batch, T, N))
    for b in range(batch):
        xb = np.lib.stride_tricks.as_strided(xf[b * sx:], (T, K), (ldx * 8, 8))
        if trans_w:
            wb = np.lib.stride_tricks.as_strided(wf[b * sw:], (N, K), (ldw * 8, 8)).T
        else:
            wb = np.lib.stride_tricks.as_strided(wf[b * sw:], (K, N), (ldw * 8, 8))
        out[b] = xb @ wb
        if y is not None:
            out[b] += np.lib.stride_tricks.as_strided(y[b * sy:], (T, N), (ldy * 4, 4))
    return out


def q6k_rows(blocks, nrows, cols):
    """Q6_K rows (uint8 [nrows, cols/256 * 210]) -> fp32 [nrows, cols], as deepseek2's decode expands kv_b (ds2.cpp:117-137)."""
    out = np.empty((nrows, cols), np.float32)
    lib().orc_q6k_rows(blocks.ctypes.data_as(C.POINTER(C.c_uint8)), i64(nrows), i64(cols), _f(out))
    return out
