"""The oracle against the reference's OWN kernels, compiled for the CPU (oracle/ref_build.py: the cache writers and
readers, the 32-point rotation, the Q6_K row reader, the fp16 and q8 latent-row conversions - the reference's source lines
behind a host stand-in for the SYCL names they use). Bit for bit: all of it is byte, integer or single-rounding work.

Skipped where oracle/_ref/libref.so was not built (no checkout of the reference beside the repository)."""
import ctypes as C

import numpy as np
import pytest

from nextsycl_b200 import workloads as W
from oracle import oracle as O

ref = O.ref_lib()
pytestmark = pytest.mark.skipif(ref is None, reason="oracle/_ref/libref.so not built (no reference checkout)")

u8p = C.POINTER(C.c_uint8)
f32p = C.POINTER(C.c_float)
u16p = C.POINTER(C.c_uint16)
i64 = C.c_int64


def g():
    return C.c_void_p(ref.ref_gpu())


def rows_with_edges(seed, shape):
    """Seeded N(0, 1) rows with the cases a quantiser can get wrong worked in: a block of zeros, a block whose largest
    magnitude occurs twice with opposite signs, values that land on .5 after scaling, a huge and a tiny block."""
    x = W.rng(seed, 0).standard_normal(shape).astype(np.float32)
    flat = x.reshape(-1, 32)
    flat[1] = 0.0
    flat[2, 3], flat[2, 17] = 4.0, -4.0
    flat[2, :3] = np.float32(0.1)
    flat[3] = np.arange(32, dtype=np.float32) * np.float32(0.5) - np.float32(7.75)    # amax 7.75: x * 127 / amax hits halves
    flat[4] *= np.float32(3.0e4)
    flat[5] *= np.float32(1.0e-6)
    flat[6, 0] = -0.0
    return x


@pytest.mark.parametrize("kt", [1, 2])
def test_quantising_cache_writer(kt):
    """ns_q35_kv_store_q (kernels/llm/qwen35/q35.cpp) - the reference's lines - against orc_kv_store_q."""
    T, Hkv, cap, p0 = 5, 3, 11, 4
    k = rows_with_edges(11, (T, Hkv * 256))
    v = rows_with_edges(12, (T, Hkv * 256))
    rb = O.q_row_bytes(kt)
    assert ref.ref_kv_row(kt) == rb
    want_k, want_v = (np.full((Hkv, cap, rb), 0xA5, np.uint8) for _ in range(2))
    got_k, got_v = want_k.copy(), want_v.copy()
    rc = ref.ns_q35_kv_store_q(g(), C.c_int(kt), k.ctypes.data_as(f32p), i64(Hkv * 256), v.ctypes.data_as(f32p), i64(Hkv * 256), i64(T), i64(Hkv), i64(256),
                               i64(cap), i64(p0), want_k.ctypes.data_as(u8p), want_v.ctypes.data_as(u8p))
    assert rc == 0, ref.ref_error()
    O.kv_store_q(kt, k, v, T, Hkv, cap, p0, got_k, got_v)
    assert np.array_equal(got_k, want_k)
    assert np.array_equal(got_v, want_v)


@pytest.mark.parametrize("kt", [1, 2])
def test_quantised_row_reader(kt):
    """kv_load8 (kernels/llm/qwen35/silo/attn.cpp), what the reference's attention sees of a q8_0 / q4_0 row, against
    orc_kv_dequant - over rows the reference's own writer produced and over rows of random bytes with finite scales."""
    Hkv, cap, n = 2, 9, 9
    rb = O.q_row_bytes(kt)
    k = rows_with_edges(13, (n, Hkv * 256))
    cache = np.zeros((Hkv, cap, rb), np.uint8)
    junk = cache.copy()
    O.kv_store_q(kt, k, k, n, Hkv, cap, 0, cache, junk)
    rnd = W.rng(14, kt).integers(0, 256, size=(Hkv, cap, rb), dtype=np.uint8)
    scales = W.rng(15, kt).standard_normal((Hkv, cap, 8)).astype(np.float16)
    rnd[:, :, rb - 16:] = scales.view(np.uint8).reshape(Hkv, cap, 16)
    for c in (cache, rnd):
        got = O.kv_dequant(kt, c, Hkv, cap, n)
        want = np.empty((Hkv, n, 256), np.uint16)
        out8 = (C.c_uint16 * 8)()
        for h in range(Hkv):
            for r in range(n):
                row = np.ascontiguousarray(c[h, r])
                for ch in range(32):
                    ref.ref_kv_load8(C.c_int(kt), row.ctypes.data_as(u8p), C.c_int(ch), out8)
                    want[h, r, 8 * ch:8 * ch + 8] = np.frombuffer(out8, np.uint16)
        assert np.array_equal(got, want)


def test_rotation():
    """ns_q35_fwht32 (kernels/llm/qwen35/q35.cpp) against orc_fwht32."""
    x = rows_with_edges(16, (7, 256))
    want = x.copy()
    assert ref.ns_q35_fwht32(g(), want.ctypes.data_as(f32p), i64(7), i64(256), i64(256)) == 0
    got = O.fwht32(x.copy())
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_fp16_cache_writer():
    """ns_q35_kv_store (kernels/llm/qwen35/q35.cpp) against orc_kv_store."""
    T, Hkv, D, cap, p0 = 4, 3, 128, 9, 2
    k = rows_with_edges(17, (T, Hkv * D))
    v = rows_with_edges(18, (T, Hkv * D))
    want_k, want_v = (np.full((Hkv, cap, D), 0x7E01, np.uint16) for _ in range(2))
    got_k, got_v = want_k.copy(), want_v.copy()
    assert ref.ns_q35_kv_store(g(), k.ctypes.data_as(f32p), i64(Hkv * D), v.ctypes.data_as(f32p), i64(Hkv * D), i64(T), i64(Hkv), i64(D), i64(cap), i64(p0),
                               want_k.ctypes.data_as(u16p), want_v.ctypes.data_as(u16p)) == 0
    O.kv_store(k, v, T, Hkv, D, cap, p0, got_k, got_v)
    assert np.array_equal(got_k, want_k)
    assert np.array_equal(got_v, want_v)


def test_q6k_row_reader():
    """q6k_cols32 (kernels/llm/deepseek2/ds2.cpp), the reference's Q6_K decoder, against orc_q6k_rows: random blocks with
    finite block scales, the sub-block scales over all of int8."""
    nrows, cols = 6, 512
    r = W.rng(19, 0)
    blocks = r.integers(0, 256, size=(nrows, 2, 210), dtype=np.uint8)
    blocks[:, :, 208:210] = (r.standard_normal((nrows, 2, 1)) * 0.01).astype(np.float16).view(np.uint8).reshape(nrows, 2, 2)
    blocks[0, 0, 192:208] = np.array([-128, 127, 0, 1, -1, 64, -64, 5] * 2, np.int8).view(np.uint8)
    blocks = np.ascontiguousarray(blocks.reshape(nrows, 420))
    got = O.q6k_rows(blocks, nrows, cols)
    want = np.empty((nrows, cols), np.float32)
    v32 = (C.c_float * 32)()
    for i in range(nrows):
        for k in range(16):
            ref.ref_q6k_cols32(blocks[i].ctypes.data_as(C.c_void_p), C.c_int(k), v32)
            want[i, 32 * k:32 * k + 32] = np.frombuffer(v32, np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_q8_latent_rows():
    """ns_to_q8row and ns_gather_q8_h (kernels/llm/glm5next/glm.cpp) against orc_to_q8row and the gathered rows' statement
    in the CUDA tests (half(scale * q))."""
    n = 9
    x = rows_with_edges(20, (n, 512))
    assert ref.ref_q8_row_bytes_512() == 544
    want = np.zeros((n, 544), np.uint8)
    assert ref.ns_to_q8row(g(), x.ctypes.data_as(f32p), want.ctypes.data_as(C.c_void_p), i64(n), i64(512)) == 0, ref.ref_error()
    got = O.to_q8row(x)
    assert np.array_equal(got, want)
    idx = np.array([8, 0, 3, 3, 5], np.int32)
    rows = np.zeros((len(idx), 512), np.uint16)
    assert ref.ns_gather_q8_h(g(), want.ctypes.data_as(C.c_void_p), idx.ctypes.data_as(C.POINTER(C.c_int32)), rows.ctypes.data_as(u16p), i64(len(idx)), i64(512)) == 0
    d = want[:, :32].copy().view(np.float16).astype(np.float32)            # [n, 16]
    q = want[:, 32:].view(np.int8).astype(np.float32).reshape(n, 16, 32)
    stated = (d[:, :, None] * q).astype(np.float16).reshape(n, 512)[idx]
    assert np.array_equal(rows, stated.view(np.uint16))


def test_fp16_rows():
    """ns_to_f16 (glm.cpp) and ns_ds41_rows_f16 (kernels/llm/deepseek41/silo/ds41.cpp) against the oracle's rounding."""
    x = rows_with_edges(21, (6, 512))
    x[0, :4] = [65504.0, 65520.0, 1e-8, -6.1e-5]      # the largest half, the first float that rounds to infinity, an underflow, a subnormal
    want = np.zeros(x.shape, np.uint16)
    assert ref.ns_to_f16(g(), x.ctypes.data_as(f32p), want.ctypes.data_as(u16p), i64(x.size)) == 0
    with np.errstate(over="ignore"):
        assert np.array_equal(O.to_f16_bits(x), want)
    cache = np.full((10, 512), 0x7E01, np.uint16)
    assert ref.ns_ds41_rows_f16(g(), x.ctypes.data_as(f32p), cache.ctypes.data_as(u16p), i64(6), i64(3), i64(512)) == 0
    assert np.array_equal(cache[3:9], want) and (cache[:3] == 0x7E01).all() and (cache[9:] == 0x7E01).all()


# ---- kernels with work-groups: the reference's own attention and rotation kernels, run as cooperative fibers -------------

def close(got, want, tol, what):
    d = np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64))
    lim = tol * (1.0 + np.abs(np.asarray(want, np.float64)))
    assert (d <= lim).all(), f"{what}: max abs {d.max():.3e} against {tol:g} (1 + |want|)"


@pytest.mark.parametrize("T,Hq,Hkv,D,kv", [(1, 12, 2, 256, 700), (1, 12, 2, 256, 5000), (1, 8, 2, 256, 40), (3, 8, 2, 256, 300), (2, 4, 4, 128, 200),
                                            (1, 16, 2, 256, 1), (8, 4, 2, 256, 64)])
def test_decode_attention_kernel(T, Hq, Hkv, D, kv):
    """ns_q35_attn (kernels/llm/qwen35/q35.cpp: the kernel `attn`, its key splits and its merge kernel) - the reference's
    lines, sub-groups of 16 - against orc_gqa_plain. Equal to the bit: the oracle sums a sub-group's partial dot products
    in lane order and its sub-groups' and splits' shares in their order, as this runs them."""
    q, k, v, p0 = W.gqa_case(950, T, Hq, Hkv, D, kv)
    qf = q.astype(np.float32)
    ref.ns_q35_attn_scratch.restype = i64
    n = ref.ns_q35_attn_scratch(i64(T), i64(Hq), i64(Hkv), i64(D), i64(p0))
    assert n == (O.lib().orc_plain_splits(i64(T), i64(p0 + T), i64(Hkv)) > 1) * T * Hq * O.lib().orc_plain_splits(i64(T), i64(p0 + T), i64(Hkv)) * (D + 2)
    sc = np.zeros(max(1, n), np.float32)
    got = np.zeros((T, Hq * D), np.float32)
    rc = ref.ns_q35_attn(g(), qf.ctypes.data_as(f32p), i64(Hq * D), k.view(np.uint16).ctypes.data_as(u16p), v.view(np.uint16).ctypes.data_as(u16p), i64(T),
                         i64(Hq), i64(Hkv), i64(D), i64(kv), i64(p0), got.ctypes.data_as(f32p), sc.ctypes.data_as(f32p))
    assert rc == 0, ref.ref_error()
    want = O.gqa_plain(qf, k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, kv, p0)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("D,n_rot,p0", [(256, 64, 0), (256, 64, 4097), (128, 128, 33)])
def test_norm_and_rotary_kernels(D, n_rot, p0):
    """ns_q35_qk_norm_rope, ns_q35_rope and ns_q35_qk_norm_rope_pos (q35.cpp) against orc_qk_norm_rope."""
    T, H = 3, 5
    x = W.rng(951, D).standard_normal((T, H * D)).astype(np.float32)
    w = (1.0 + 0.1 * W.rng(951, 1).standard_normal(D)).astype(np.float32)
    theta, eps = np.float32(1.0e6), np.float32(1e-6)
    got = np.zeros((T, H * D), np.float32)
    assert ref.ns_q35_qk_norm_rope(g(), x.ctypes.data_as(f32p), i64(H * D), i64(D), got.ctypes.data_as(f32p), i64(H * D), i64(T), i64(H), i64(D),
                                   w.ctypes.data_as(f32p), C.c_float(eps), i64(n_rot), C.c_float(theta), i64(p0)) == 0, ref.ref_error()
    close(got, O.qk_norm_rope(x, T, H, D, w, eps, n_rot, theta, p0), 2e-6, "norm + rotation")
    got2 = np.zeros((T, H * D), np.float32)
    assert ref.ns_q35_rope(g(), x.ctypes.data_as(f32p), i64(H * D), i64(D), got2.ctypes.data_as(f32p), i64(H * D), i64(T), i64(H), i64(D), i64(n_rot),
                           C.c_float(theta), i64(p0)) == 0, ref.ref_error()
    close(got2, O.qk_norm_rope(x, T, H, D, None, eps, n_rot, theta, p0), 2e-6, "rotation alone")
    pos3 = np.stack([np.arange(T) + p0, np.arange(T) * 2 + 7, np.arange(T) * 3 + 1]).astype(np.int32)      # [3, T]
    sections = (n_rot // 4 - 3, 2, 1)
    got3 = np.zeros((T, H * D), np.float32)
    assert ref.ns_q35_qk_norm_rope_pos(g(), x.ctypes.data_as(f32p), i64(H * D), i64(D), got3.ctypes.data_as(f32p), i64(H * D), i64(T), i64(H), i64(D),
                                       w.ctypes.data_as(f32p), C.c_float(eps), i64(n_rot), C.c_float(theta), pos3.ctypes.data_as(C.POINTER(C.c_int32)),
                                       i64(sections[0]), i64(sections[1]), i64(sections[2])) == 0, ref.ref_error()
    close(got3, O.qk_norm_rope(x, T, H, D, w, eps, n_rot, theta, 0, pos3=np.ascontiguousarray(pos3), sections=sections), 2e-6, "sectioned positions")


YARN = dict(freq_base=np.float32(10000.0), freq_scale=np.float32(0.025), ext_factor=np.float32(1.0), mscale=np.float32(1.0 + 0.1 * np.log(40.0)),
            corr0=np.float32(10.0), corr1=np.float32(23.0))
YK = ("freq_base", "freq_scale", "ext_factor", "mscale", "corr0", "corr1")


@pytest.mark.parametrize("ext", [0.0, 1.0])
def test_ds2_rotation_and_cache_writer(ext):
    """ns_ds2_rope and ns_ds2_kv_store (kernels/llm/deepseek2/ds2.cpp: YaRN, the latent cache's writer) against orc_ds2_rope
    and orc_ds2_kv_store."""
    f = C.c_float
    T, H, head, off, n_dims, pos0 = 4, 6, 192, 128, 64, 3000
    y = dict(YARN, ext_factor=np.float32(ext))
    x = W.rng(952, 0).standard_normal((T, H * head)).astype(np.float32)
    got, gout = x.copy().ravel(), np.zeros(T * H * n_dims, np.float32)
    assert ref.ns_ds2_rope(g(), got.ctypes.data_as(f32p), i64(T), i64(H), i64(H * head), i64(head), i64(off), i64(n_dims), i64(pos0), *[f(y[k]) for k in YK],
                           gout.ctypes.data_as(f32p), i64(H * n_dims), i64(n_dims)) == 0, ref.ref_error()
    want, wout = x.copy().ravel(), np.zeros(T * H * n_dims, np.float32)
    O.ds2_rope(want, T, H, H * head, head, off, n_dims, pos0, *[float(y[k]) for k in YK], out=wout, out_row=H * n_dims, out_head=n_dims)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)) and np.array_equal(gout.view(np.uint32), wout.view(np.uint32))
    L, R = 512, 64
    kv = W.rng(952, 1).standard_normal((T, L + R)).astype(np.float32)
    w = (1.0 + 0.1 * W.rng(952, 2).standard_normal(L)).astype(np.float32)
    gc, wc = (np.full((pos0 % 7 + T + 2, L + R), 0x7E01, np.uint16) for _ in range(2))
    p = pos0 % 7
    assert ref.ns_ds2_kv_store(g(), kv.ctypes.data_as(f32p), w.ctypes.data_as(f32p), f(1e-6), gc.ctypes.data_as(u16p), i64(T), i64(L), i64(R), i64(p),
                               *[f(y[k]) for k in YK]) == 0, ref.ref_error()
    O.ds2_kv_store(kv, w, np.float32(1e-6), wc, T, L, R, p, *[float(y[k]) for k in YK])
    # the 256 work-items' shares of a row's sum of squares meet in another order than the oracle's: the normed values may
    # differ in the last place before they are rounded to fp16
    a, b = gc[p:p + T].view(np.float16).astype(np.float32), wc[p:p + T].view(np.float16).astype(np.float32)
    close(a, b, 1.0e-3, "latent rows")
    assert (gc[p:p + T] != wc[p:p + T]).mean() < 0.01
    assert np.array_equal(gc[:p], wc[:p]) and np.array_equal(gc[p + T:], wc[p + T:])


def _q6k_blocks(rng, nrows):
    blocks = rng.integers(0, 256, size=(nrows, 2, 210), dtype=np.uint8)
    blocks[:, :, 192:208] = rng.integers(-40, 41, size=(nrows, 2, 16)).astype(np.int8).view(np.uint8)
    blocks[:, :, 208:210] = (np.abs(rng.standard_normal((nrows, 2, 1))) * 2.0e-4 + 1.0e-4).astype(np.float16).view(np.uint8).reshape(nrows, 2, 2)
    return np.ascontiguousarray(blocks.reshape(nrows, 420))


@pytest.mark.parametrize("T,H,n", [(1, 3, 300), (2, 2, 77), (1, 2, 1)])
def test_ds2_fused_decode_kernel(T, H, n):
    """ns_ds2_mla_decode and ns_ds2_mla_decode_q6k (ds2.cpp: mla_decode_t, one work-group of 256 a (row, head): absorb, online
    softmax over the cache, un-absorb) against the same three stages stated with the oracle: q~ = k_b q_nope, orc_mla_fused over
    the latent cache, out = v_b u. The stages' fp32 sums meet in other orders: 2e-5 (1 + |want|)."""
    pos0 = n - T
    scale = np.float32(1.0 / np.sqrt(192.0))
    q = W.rng(953, T).standard_normal((T, H, 192)).astype(np.float32)
    cache = W.normal_f16(953, 3, (n, 576), 0.5)
    kb = W.normal_f16(953, 1, (H, 512, 128), 0.1)
    vb = W.normal_f16(953, 2, (H, 128, 512), 0.1)
    got = np.zeros((T, H, 128), np.float32)
    assert ref.ns_ds2_mla_decode(g(), q.ctypes.data_as(f32p), kb.view(np.uint16).ctypes.data_as(u16p), vb.view(np.uint16).ctypes.data_as(u16p),
                                 cache.view(np.uint16).ctypes.data_as(u16p), got.ctypes.data_as(f32p), i64(T), i64(H), i64(pos0), C.c_float(scale)) == 0

    def stated(k_rows, v_rows):      # k_rows [H, 512, 128] (q~[c] = sum_i k[c][i] q[i]), v_rows [H, 128, 512], float64
        qa = np.einsum("hci,thi->thc", k_rows, q[:, :, :128].astype(np.float64)).astype(np.float32)
        qfull = np.ascontiguousarray(np.concatenate([qa, q[:, :, 128:]], axis=2))
        u = O.mla_fused(qfull, cache.view(np.uint16), T, H, 512, 64, pos0, scale)
        return np.einsum("hvl,thl->thv", v_rows, u.astype(np.float64))
    close(got, stated(kb.astype(np.float64), vb.astype(np.float64)), 2e-5, "fp16 weights")
    kvb = _q6k_blocks(W.rng(953, 9), H * 256)
    vals = O.q6k_rows(kvb, H * 256, 512).reshape(H, 256, 512).astype(np.float64)
    got6 = np.zeros((T, H, 128), np.float32)
    assert ref.ns_ds2_mla_decode_q6k(g(), q.ctypes.data_as(f32p), kvb.ctypes.data_as(C.c_void_p), cache.view(np.uint16).ctypes.data_as(u16p),
                                     got6.ctypes.data_as(f32p), i64(T), i64(H), i64(pos0), C.c_float(scale)) == 0
    # Q6_K: per head 128 k rows (row i = k_i[0..511]) then 128 v rows
    close(got6, stated(np.transpose(vals[:, :128], (0, 2, 1)), vals[:, 128:]), 2e-5, "Q6_K weights")
