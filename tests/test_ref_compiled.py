"""The oracle against the reference's OWN kernels, compiled for the CPU (oracle/ref_build.py: the reference's source lines
behind a host stand-in for the SYCL names they use - work-groups as fibers, sub-groups, group collectives, joint_matrix).
Bit for bit for the byte, integer and single-rounding work and wherever the oracle follows a kernel's summation order (the
flash, plain and deepseek41 matrix-unit attention, the indexer scores); a stated tolerance elsewhere.

Skipped where oracle/_ref/ was not built (no checkout of the reference beside the repository)."""
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


i32p = C.POINTER(C.c_int32)
GSCALE = np.float32(1.0 / 16.0)


def test_glm_exact_attention_kernel():
    """ns_mla_attend (kernels/llm/glm5next/glm.cpp: fp32 latents, two passes) against orc_mla_attend_f32."""
    T, H, L, n = 3, 4, 512, 200
    qa = W.rng(960, 0).standard_normal((T, H, L)).astype(np.float32)
    c = (0.5 * W.rng(960, 1).standard_normal((n, L))).astype(np.float32)
    got = np.zeros((T, H, L), np.float32)
    assert ref.ns_mla_attend(g(), qa.ctypes.data_as(f32p), c.ctypes.data_as(f32p), got.ctypes.data_as(f32p), i64(T), i64(H), i64(L), i64(n - T), C.c_float(GSCALE)) == 0
    close(got, O.mla_attend_f32(qa, c, T, H, L, n - T, GSCALE), 1e-5, "exact attention over fp32 latents")


@pytest.mark.parametrize("T,H,n,q8", [(1, 8, 300, False), (3, 8, 900, False), (2, 8, 500, True), (12, 4, 400, False)])
def test_glm_selected_cell_kernels(T, H, n, q8):
    """ns_mla_attend_sel and ns_mla_attend_sel_q8 (glm.cpp: mla_dec for passes of at most 8 rows, mla_sel above) - dense,
    selected and mixed rows - against orc_mla_dec512."""
    qa = W.rng(961, 0).standard_normal((T, H, 512)).astype(np.float32)
    lat = (0.5 * W.rng(961, 1).standard_normal((n, 512))).astype(np.float32)
    c16 = lat.astype(np.float16)
    cache = O.to_q8row(lat) if q8 else c16.view(np.uint16)
    pos0, K = n - T, 24
    rng = W.rng(961, 2)
    sel, cnt = np.zeros((T, K), np.int32), np.zeros(T, np.int32)
    for t in range(T):
        pools = (pos0 + t + 1) // 4
        cnt[t] = min(K, pools) - (t % 3)
        sel[t, :cnt[t]] = np.sort(rng.choice(pools, size=cnt[t], replace=False))
    fn = ref.ns_mla_attend_sel_q8 if q8 else ref.ns_mla_attend_sel

    def run(selp, cntp, k):
        got = np.zeros((T, H, 512), np.float32)
        rc = fn(g(), qa.ctypes.data_as(f32p), cache.ctypes.data_as(C.c_void_p), got.ctypes.data_as(f32p), i64(T), i64(H), i64(512), i64(pos0), C.c_float(GSCALE),
                None if selp is None else selp.ctypes.data_as(i32p), None if cntp is None else cntp.ctypes.data_as(i32p), i64(k))
        assert rc == 0, ref.ref_error()
        return got
    close(run(sel, cnt, K), O.mla_dec512(qa, cache, T, H, pos0, GSCALE, sel=sel, sel_cnt=cnt, K=K, q8=q8), 2e-5, "selected cells")
    if not q8:
        close(run(None, None, 0), O.mla_dec512(qa, cache, T, H, pos0, GSCALE), 2e-5, "every earlier token")
        cnt2 = cnt.copy()
        cnt2[0] = -1
        close(run(sel, cnt2, K), O.mla_dec512(qa, cache, T, H, pos0, GSCALE, sel=sel, sel_cnt=cnt2, K=K), 2e-5, "a dense row among selected ones")


def test_glm_indexer_kernels():
    """ns_idx_pool, ns_idx_score and ns_topk (glm.cpp) against orc_idx_pool, orc_idx_score and orc_topk (the selection bit for bit)."""
    D = 128
    for pos0, T in ((0, 11), (7, 1), (13, 5), (1021, 9)):
        rng = W.rng(1420, pos0)
        ik, ig = rng.standard_normal((T, D)).astype(np.float32), rng.standard_normal((T, D)).astype(np.float32)
        ape = rng.standard_normal((4, D)).astype(np.float32)
        ring = rng.standard_normal((8, 2 * D)).astype(np.float32)
        pools = (pos0 + T) // 4 + 2
        gring, gp = ring.copy(), np.full((pools, D), 9.0, np.float32)
        wring, wp = ring.copy(), gp.copy()
        assert ref.ns_idx_pool(g(), gring.ctypes.data_as(f32p), ik.ctypes.data_as(f32p), ig.ctypes.data_as(f32p), ape.ctypes.data_as(f32p), gp.ctypes.data_as(f32p),
                               i64(pos0), i64(T), i64(D)) == 0
        O.idx_pool(wring, ik, ig, ape, wp, pos0, T, D)
        close(gp, wp, 2e-6, "pooled keys")
        assert np.array_equal(gring, wring)
    T, H, n, j0, pos0 = 5, 32, 300, 100, 1590
    ld = j0 + n + 7
    S = W.rng(1410, 0).standard_normal((T * H, n)).astype(np.float32)
    w = W.rng(1410, 1).standard_normal((T, H)).astype(np.float32)
    got, want = (np.full((T, ld), 3.0, np.float32) for _ in range(2))
    assert ref.ns_idx_score(g(), S.ctypes.data_as(f32p), w.ctypes.data_as(f32p), got.ctypes.data_as(f32p), i64(T), i64(H), i64(j0), i64(n), i64(ld), i64(pos0)) == 0
    O.idx_score(S, w, want, T, H, j0, n, pos0)
    assert np.array_equal(np.isneginf(got), np.isneginf(want))
    fin = np.isfinite(want)
    close(got[fin], want[fin], 2e-6, "pool scores")
    for (T, n, ld, K, kind) in ((1, 1000, 1000, 64, "normal"), (3, 4097, 4100, 512, "ties"), (4, 700, 800, 700, "ties"), (2, 3000, 3000, 100, "masked"),
                                (1, 50, 64, 80, "normal"), (2, 2048, 2048, 300, "constant")):
        rng = W.rng(1400, n + K)
        score = np.full((T, ld), 7.0, np.float32)
        x = rng.standard_normal((T, n)).astype(np.float32)
        if kind == "ties":
            x = np.round(x * 2) / 2
        if kind == "constant":
            x[:] = -1.5
        if kind == "masked":
            x[:, n // 3:] = -np.inf
            x[1, :10] = 0.0
            x[1, 5] = -0.0
        score[:, :n] = x
        sel = np.full((T, K), -1, np.int32)
        assert ref.ns_topk(g(), score.ctypes.data_as(f32p), sel.ctypes.data_as(i32p), i64(T), i64(n), i64(ld), i64(K)) == 0, ref.ref_error()
        assert np.array_equal(sel, O.topk(score, n, K)), kind


def test_glm_cell_lists_masked_softmax_and_gather():
    """ns_mla_cells, ns_softmax_masked and ns_gather_h (glm.cpp), the reference's lines, against the statements the CUDA tests
    hold the library's kernels to (tests/test_glm_mla_gpu.py::test_helper_kernels)."""
    T, K, pos0, NC = 3, 4, 50, 64
    sel = np.array([[1, 3, 7, 0], [2, 4, 6, 8], [0, 0, 0, 0]], np.int32)
    cnt = np.array([3, 4, -1], np.int32)
    gi, gn = np.full((T, NC), -7, np.int32), np.zeros(T, np.int32)
    assert ref.ns_mla_cells(g(), sel.ctypes.data_as(i32p), cnt.ctypes.data_as(i32p), i64(T), i64(K), i64(pos0), gi.ctypes.data_as(i32p), gn.ctypes.data_as(i32p),
                            i64(NC)) == 0
    for t in range(T):
        p = pos0 + t
        tail0 = 4 * ((p + 1) // 4)
        cells = list(range(p + 1)) if cnt[t] < 0 else [4 * sel[t, i // 4] + i % 4 for i in range(4 * cnt[t])] + list(range(tail0, p + 1))
        assert gn[t] == min(len(cells), NC)
        assert list(gi[t, :gn[t]]) == cells[:NC]
    S = W.rng(962, 5).standard_normal((T * 2, NC)).astype(np.float32)
    got = S.copy()
    assert ref.ns_softmax_masked(g(), got.ctypes.data_as(f32p), i64(T), i64(2), i64(NC), gn.ctypes.data_as(i32p), C.c_float(0.3)) == 0
    got = got.reshape(T, 2, NC)
    for t in range(T):
        m = gn[t]
        z = S.reshape(T, 2, NC)[t, :, :m].astype(np.float64) * 0.3
        e = np.exp(z - z.max(-1, keepdims=True))
        assert np.allclose(got[t, :, :m], e / e.sum(-1, keepdims=True), atol=1e-6)
        assert not got[t, :, m:].any()
    x = W.normal_f16(962, 0, (37, 512), 0.5)
    idx = np.array([5, 0, 36, 5, 17], np.int32)
    out = np.zeros((len(idx), 512), np.uint16)
    assert ref.ns_gather_h(g(), x.view(np.uint16).ctypes.data_as(u16p), idx.ctypes.data_as(i32p), out.ctypes.data_as(u16p), i64(len(idx)), i64(512)) == 0
    assert np.array_equal(out, x.view(np.uint16)[idx])


DSCALE = np.float32(512 ** -0.5)


def _ds41_case(seed, T, H, pos0, window, R, ratio, K, with_comp=True):
    rng = W.rng(seed, 0)
    q = rng.standard_normal((T, H, 512)).astype(np.float32)
    raw = O.to_f16_bits((0.5 * rng.standard_normal((R, 512))).astype(np.float32))
    ncomp = (pos0 + T) // ratio if with_comp else 0
    comp = O.to_f16_bits((0.5 * rng.standard_normal((ncomp, 512))).astype(np.float32)) if ncomp else None
    sel = None
    if K and comp is not None:
        sel = np.zeros((T, K), np.int32)
        for t in range(T):
            vis = (pos0 + t + 1) // ratio
            if vis > K:
                sel[t] = np.sort(rng.choice(vis, size=K, replace=False))
    return q, raw, comp, sel, rng.standard_normal(H).astype(np.float32)


@pytest.mark.parametrize("T,H,pos0,window,R,ratio,K,with_comp", [
    (1, 8, 5, 128, 128, 4, 0, False),        # fewer tokens than the window, no compressed cells
    (1, 8, 1000, 128, 128, 4, 0, False),     # a full window, the ring wrapped many times
    (1, 4, 2047, 128, 128, 4, 0, True),      # window + every compressed cell
    (1, 4, 4095, 128, 160, 4, 256, True),    # the indexer's picks, a ring longer than the window
    (4, 4, 1020, 128, 128, 4, 256, True),    # rows either side of the point where picks start
    (3, 8, 0, 16, 16, 128, 0, True),         # the first tokens; comp given but nothing visible yet
    (2, 3, 300, 64, 64, 4, 0, True),         # a head count that is no multiple of four: one head a work-group
])
def test_ds41_vector_attention_kernel(T, H, pos0, window, R, ratio, K, with_comp):
    """ns_ds41_attend (kernels/llm/deepseek41/silo/ds41.cpp: `attend`, the vector form - window ring, compressed cells, picks,
    per-head sinks) against orc_ds41_attend in that form's numerics (mode 0)."""
    q, raw, comp, sel, sinks = _ds41_case(980 + T, T, H, pos0, window, R, ratio, K, with_comp)
    if comp is None and with_comp:
        comp = np.zeros((1, 512), np.uint16)
    got = np.zeros((T, H, 512), np.float32)
    rc = ref.ns_ds41_attend(g(), q.ctypes.data_as(f32p), raw.ctypes.data_as(u16p), i64(R), None if comp is None else comp.ctypes.data_as(u16p), i64(ratio),
                            None if sel is None else sel.ctypes.data_as(i32p), i64(K), sinks.ctypes.data_as(f32p), got.ctypes.data_as(f32p), i64(T), i64(H),
                            i64(pos0), i64(window), C.c_float(DSCALE))
    assert rc == 0, ref.ref_error()
    close(got, O.ds41_attend(q, raw, R, comp, ratio, sel, K, sinks, T, H, pos0, window, DSCALE, mode=0), 1e-5, "MQA-512 with sinks")


def test_ds41_steps_around_attention():
    """ns_ds41_ring_put, ns_ds41_kv_post, ns_ds41_att_post (norm, YaRN rotation, the model's E4M3 simulation), ns_ds41_block_max,
    ns_ds41_cand_mask and ns_ds41_cand_pos (ds41.cpp, k41.cpp) against the oracle's functions."""
    f = C.c_float
    T, R, D, pos0 = 7, 16, 512, 13
    kv = W.rng(993, 0).standard_normal((T, D)).astype(np.float32)
    before = W.rng(993, 1).integers(0, 1 << 15, size=(R, D), dtype=np.uint16)
    ring = before.copy()
    assert ref.ns_ds41_ring_put(g(), kv.ctypes.data_as(f32p), ring.ctypes.data_as(u16p), i64(T), i64(pos0), i64(R), i64(D)) == 0
    want = before.copy()
    for t in range(T):
        want[(pos0 + t) % R] = kv[t].astype(np.float16).view(np.uint16)
    assert np.array_equal(ring, want)

    def grid_close(got, want, what):     # values on the E4M3 grid: equal but for inputs next to a rounding boundary
        same = got == want
        assert same.mean() > 0.995, f"{what}: {1 - same.mean():.4f} of the values differ"
        assert np.all(np.abs(got.astype(np.float64) - want) <= 0.13 * np.abs(want) + 2e-6), what
    yarn = [float(YARN[k]) for k in YK]
    T, D, rd, pos0, R = 9, 512, 64, 250, 128
    kv = W.rng(1360, 0).standard_normal((T, D)).astype(np.float32)
    w = (1.0 + 0.1 * W.rng(1360, 1).standard_normal(D)).astype(np.float32)
    before = W.rng(1360, 2).integers(0, 1 << 15, size=(R, D), dtype=np.uint16)
    gkv, gring = kv.copy(), before.copy()
    sycl_sg = C.c_int.in_dll(ref, "ref_sub_group_size")
    sycl_sg.value = 32            # these two kernels ask for sub-groups of 32
    try:
        assert ref.ns_ds41_kv_post(g(), gkv.ctypes.data_as(f32p), w.ctypes.data_as(f32p), i64(T), i64(D), f(1e-6), i64(rd), i64(pos0), *[f(v) for v in yarn],
                                   gring.ctypes.data_as(u16p), i64(R)) == 0, ref.ref_error()
        wkv, wring = kv.copy(), before.copy()
        O.ds41_kv_post(wkv, w, T, D, 1e-6, rd, pos0, yarn, wring, R)
        grid_close(gkv, wkv, "kv_post")
        slots = [(pos0 + t) % R for t in range(T)]
        others = [s for s in range(R) if s not in slots]
        assert np.array_equal(gring[others], before[others])
        assert np.array_equal(gring[slots].view(np.float16), gkv.astype(np.float16))
        T, H, D, rd, pos0 = 3, 8, 512, 64, 777
        x = W.rng(1370, 0).standard_normal((T, H, D)).astype(np.float32)
        gx = x.copy()
        assert ref.ns_ds41_att_post(g(), gx.ctypes.data_as(f32p), i64(T), i64(H), i64(D), i64(rd), i64(pos0), *[f(v) for v in yarn]) == 0, ref.ref_error()
        wx = x.copy()
        O.ds41_att_post(wx, T, H, D, rd, pos0, yarn)
        grid_close(gx, wx, "att_post")
    finally:
        sycl_sg.value = 16
    T, n, ld, bs, pos0, ratio, K = 3, 1003, 1008, 8, 4100, 4, 20
    nb = -(-n // bs)
    rng = W.rng(1441, 0)
    score = rng.standard_normal((T, ld)).astype(np.float32)
    vis = [(pos0 + t + 1) // ratio for t in range(T)]
    for t in range(T):
        score[t, min(vis[t], n):] = -np.inf
    bm = np.zeros((T, nb), np.float32)
    assert ref.ns_ds41_block_max(g(), score.ctypes.data_as(f32p), bm.ctypes.data_as(f32p), i64(T), i64(n), i64(ld), i64(bs), i64(pos0), i64(ratio)) == 0
    assert np.array_equal(bm.view(np.uint32), O.ds41_block_max(score, n, bs, pos0, ratio).view(np.uint32))
    cand = np.stack([np.sort(rng.choice(nb, size=K, replace=False)) for _ in range(T)]).astype(np.int32)
    cand[1, 0] = -1
    cand[2, -1] = nb - 1
    gs, mark = score.copy(), np.zeros((T, nb), np.uint8)
    assert ref.ns_ds41_cand_mask(g(), gs.ctypes.data_as(f32p), cand.ctypes.data_as(i32p), mark.ctypes.data_as(u8p), i64(T), i64(n), i64(ld), i64(K), i64(bs)) == 0
    assert np.array_equal(gs.view(np.uint32), O.ds41_cand_mask(score.copy(), cand, n, bs).view(np.uint32))
    kp = 33
    selc = np.stack([np.sort(rng.choice(K * 8, size=kp, replace=False)) for _ in range(T)]).astype(np.int32)
    cand_ok = np.where(cand < 0, 0, cand).astype(np.int32)
    gsel = np.zeros((T, kp), np.int32)
    assert ref.ns_ds41_cand_pos(g(), selc.ctypes.data_as(i32p), cand_ok.ctypes.data_as(i32p), gsel.ctypes.data_as(i32p), i64(T), i64(K), i64(kp), i64(bs)) == 0
    assert np.array_equal(gsel, O.ds41_cand_pos(selc, cand_ok, bs))


@pytest.mark.parametrize("T,Hq,Hkv,kv", [(1, 16, 2, 900), (1, 64, 8, 3000), (4, 32, 4, 700), (8, 8, 1, 40)])
def test_nemotronh_attention_kernel(T, Hq, Hkv, kv):
    """ns_nh_attn (kernels/llm/nemotronh/nh.cpp: attn<8, 8>, heads of 128, eight query heads a work-group) - the only reference
    kernel there is for the head width of benchmark configurations 2 and 5 - against orc_gqa_plain with its grouping. To the bit."""
    nh = O.ref_nh_lib()
    D = 128
    q, k, v, p0 = W.gqa_case(951, T, Hq, Hkv, D, kv)
    qf = q.astype(np.float32)
    n = nh.ns_nh_attn_scratch(i64(T), i64(Hq), i64(Hkv), i64(D), i64(p0))
    sc = np.zeros(max(1, n), np.float32)
    got = np.zeros((T, Hq * D), np.float32)
    rc = nh.ns_nh_attn(C.c_void_p(nh.ref_gpu()), qf.ctypes.data_as(f32p), i64(Hq * D), k.view(np.uint16).ctypes.data_as(u16p),
                       v.view(np.uint16).ctypes.data_as(u16p), i64(T), i64(Hq), i64(Hkv), i64(D), i64(kv), i64(p0), got.ctypes.data_as(f32p), sc.ctypes.data_as(f32p))
    assert rc == 0, nh.ref_error()
    want = O.gqa_plain(qf, k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, kv, p0, groups=Hq // 8)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("kt,mode", [(0, 0), (1, 0), (2, 1), (0, 1)])
def test_attention_weights_kernel(kt, mode):
    """ns_q35_attn_probs (q35.cpp: one row's softmax weights per key over a cache of any form) against orc_q35_attn_probs."""
    Hq, Hkv, cap, n = 12, 2, 300, 270
    rb = O.q_row_bytes(kt)
    k = W.rng(1280, kt).standard_normal((cap, Hkv * 256)).astype(np.float32)
    if kt == 0:
        kc = np.ascontiguousarray(k.reshape(cap, Hkv, 256).transpose(1, 0, 2)).astype(np.float16).view(np.uint8).reshape(Hkv, cap, 512)
    else:
        kc, junk = np.zeros((Hkv, cap, rb), np.uint8), np.zeros((Hkv, cap, rb), np.uint8)
        O.kv_store_q(kt, k, k, cap, Hkv, cap, 0, kc, junk)
    q = W.rng(1285, kt).standard_normal(Hq * 256).astype(np.float32)
    before = W.rng(1286, 0).random(n).astype(np.float32)
    got, gsc = before.copy(), np.zeros((Hq, 2), np.float32)
    rc = ref.ns_q35_attn_probs(g(), C.c_int(kt), q.ctypes.data_as(f32p), kc.ctypes.data_as(C.c_void_p), i64(Hq), i64(Hkv), i64(256), i64(cap), i64(n), C.c_int(mode),
                               gsc.ctypes.data_as(f32p), got.ctypes.data_as(f32p))
    assert rc == 0, ref.ref_error()
    want = before.copy()
    wsc = O.q35_attn_probs(kt, q, kc, Hq, Hkv, cap, n, mode, want)
    close(got, want, 2e-6, "weights")
    close(gsc, wsc, 2e-5, "the heads' maxima and sums")


# ---- the matrix-unit kernels (joint_matrix on the host stand-in: a product row summed over its 16 terms in order) ----
q35x = O.ref_unit("ref_q35x")
needs_q35x = pytest.mark.skipif(q35x is None, reason="oracle/_ref/libref_q35x.so not built (no reference checkout)")


def _gqa256(seed, T, Hkv, p0, spare=3):
    Hq, cap = 6 * Hkv, p0 + T + spare
    r = W.rng(seed, T * 1000 + p0)
    q = r.standard_normal((T, Hq * 256), dtype=np.float32)
    k = (r.standard_normal((Hkv, cap, 256)) * 0.5).astype(np.float16)
    v = (r.standard_normal((Hkv, cap, 256)) * 0.5).astype(np.float16)
    return q, k, v, Hq, cap


@needs_q35x
@pytest.mark.parametrize("T,Hkv,p0", [(9, 1, 0), (16, 1, 0), (13, 2, 37), (24, 1, 100), (40, 2, 5)])
def test_matrix_unit_prompt_kernel(T, Hkv, p0):
    """ns_q35_attn_prompt (kernels/llm/qwen35/silo/attn.cpp: attn_flash<6, false, 0>, blocks of 8 rows over chunks of 16
    keys) - the reference's lines - against orc_gqa_flash_prefill. Equal to the bit: whole and partial row blocks, rows
    whose chunks run past their own last key, a prefix already in the cache."""
    q, k, v, Hq, cap = _gqa256(960, T, Hkv, p0)
    assert q35x.ns_q35_attn_prompt_supported(i64(T), i64(Hq), i64(Hkv), i64(256)) == 1
    got = np.full((T, Hq * 256), np.nan, np.float32)
    rc = q35x.ns_q35_attn_prompt(C.c_void_p(q35x.ref_gpu()), q.ctypes.data_as(f32p), i64(Hq * 256), k.ctypes.data_as(u16p), v.ctypes.data_as(u16p), i64(T),
                                 i64(Hq), i64(Hkv), i64(256), i64(cap), i64(p0), got.ctypes.data_as(f32p))
    assert rc == 0, q35x.ref_error()
    want = O.gqa_flash_prefill(q, k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, 256, cap, p0)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@needs_q35x
@pytest.mark.parametrize("T,Hkv,p0", [(1, 1, 0), (1, 2, 299), (3, 1, 1000), (8, 2, 60), (2, 1, 63), (4, 1, 126), (1, 4, 2500)])
def test_matrix_unit_decode_kernel(T, Hkv, p0):
    """ns_q35_attn_decode (silo/attn.cpp: flash_decode - attn_flash<6, true, 0> a (key head, split), the merge kernel)
    against orc_gqa_flash_decode, to the bit, scratch size and scratch contents included: one split and many, rows whose
    split sizes differ (a context crossing a split step: the row-at-a-time form), a verify pass of 8 rows."""
    q, k, v, Hq, cap = _gqa256(961, T, Hkv, p0)
    q35x.ns_q35_attn_decode_scratch.restype = i64
    n = q35x.ns_q35_attn_decode_scratch(i64(T), i64(Hq), i64(Hkv), i64(256), i64(p0))
    ns = max(O.flash_splits(p0 + r + 1, Hkv) for r in range(T))
    assert n == (T * Hq * ns * 258 if ns > 1 else 0)
    sc = np.zeros(max(1, n), np.float32)
    got = np.full((T, Hq * 256), np.nan, np.float32)
    rc = q35x.ns_q35_attn_decode(C.c_void_p(q35x.ref_gpu()), q.ctypes.data_as(f32p), i64(Hq * 256), k.ctypes.data_as(u16p), v.ctypes.data_as(u16p), i64(T),
                                 i64(Hq), i64(Hkv), i64(256), i64(cap), i64(p0), got.ctypes.data_as(f32p), sc.ctypes.data_as(f32p))
    assert rc == 0, q35x.ref_error()
    want = O.gqa_flash_decode(q, k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, 256, cap, p0)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@needs_q35x
@pytest.mark.parametrize("kt", [1, 2])
def test_matrix_unit_kernels_over_quantised_caches(kt):
    """ns_q35_attn_prompt_kv and ns_q35_attn_decode_kv with q8_0 and q4_0 caches: the kernel reads a row through kv_load8,
    so it equals - to the bit - the oracle over orc_kv_dequant's fp16 values of the same cache bytes."""
    Hkv, Hq = 2, 12
    for T, p0, fn in [(11, 20, "prompt"), (2, 150, "decode")]:
        cap = p0 + T
        r = W.rng(962, kt * 10 + T)
        q = r.standard_normal((T, Hq * 256), dtype=np.float32)
        rows = r.standard_normal((cap, Hkv * 256), dtype=np.float32)
        rb = O.q_row_bytes(kt)
        kc, vc = (np.zeros((Hkv, cap, rb), np.uint8) for _ in range(2))
        O.kv_store_q(kt, rows, np.ascontiguousarray(rows[::-1]), cap, Hkv, cap, 0, kc, vc)
        got = np.full((T, Hq * 256), np.nan, np.float32)
        gq = C.c_void_p(q35x.ref_gpu())
        if fn == "prompt":
            rc = q35x.ns_q35_attn_prompt_kv(gq, C.c_int(kt), q.ctypes.data_as(f32p), i64(Hq * 256), kc.ctypes.data_as(u8p), vc.ctypes.data_as(u8p), i64(T), i64(Hq),
                                            i64(Hkv), i64(256), i64(cap), i64(p0), got.ctypes.data_as(f32p))
        else:
            q35x.ns_q35_attn_decode_scratch.restype = i64
            sc = np.zeros(max(1, q35x.ns_q35_attn_decode_scratch(i64(T), i64(Hq), i64(Hkv), i64(256), i64(p0))), np.float32)
            rc = q35x.ns_q35_attn_decode_kv(gq, C.c_int(kt), q.ctypes.data_as(f32p), i64(Hq * 256), kc.ctypes.data_as(u8p), vc.ctypes.data_as(u8p), i64(T), i64(Hq),
                                            i64(Hkv), i64(256), i64(cap), i64(p0), got.ctypes.data_as(f32p), sc.ctypes.data_as(f32p))
        assert rc == 0, q35x.ref_error()
        kd, vd = O.kv_dequant(kt, kc, Hkv, cap, cap), O.kv_dequant(kt, vc, Hkv, cap, cap)
        want = (O.gqa_flash_prefill if fn == "prompt" else O.gqa_flash_decode)(q, kd, vd, T, Hq, Hkv, 256, cap, p0)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), fn


ds41x = O.ref_unit("ref_ds41x")


@pytest.mark.skipif(ds41x is None, reason="oracle/_ref/libref_ds41x.so not built (no reference checkout)")
@pytest.mark.parametrize("T,H,pos0,window,R,ratio,K,with_comp", [
    (1, 8, 700, 128, 128, 4, 0, False),       # decode, the window alone: splits of 32 cells
    (1, 16, 2047, 128, 128, 4, 0, True),      # window + every compressed cell: 640 cells in 20 splits
    (1, 8, 4095, 128, 160, 4, 256, True),     # the indexer's picks, a ring longer than the window
    (4, 8, 1020, 128, 128, 4, 256, True),     # a verify pass whose rows' split sizes agree, either side of where picks start
    (3, 8, 0, 16, 16, 128, 0, True),          # the first tokens: 1, 2, 3 cells, one split
    (8, 8, 8180, 128, 128, 4, 0, True),       # rows whose split sizes differ: a launch a row
    (9, 8, 300, 64, 64, 4, 0, True),          # more than 8 rows: the prompt form, 2 head groups a work-group -> 1
    (12, 16, 40, 128, 128, 4, 0, True),       # the prompt form, two head groups a work-group
    (64, 64, 0, 32, 32, 4, 8, True),          # 64 rows of 64 heads: a work-group all heads; picks from row 35 on
])
def test_ds41_matrix_unit_attention(T, H, pos0, window, R, ratio, K, with_comp):
    """ns_ds41_attend_xmx (kernels/llm/deepseek41/silo/attn.cpp: attend_xmx in its prompt and split forms, attend_q16,
    attend_merge) - the reference's lines - against orc_ds41_attend in that kernel's numerics (mode 1), to the bit."""
    q, raw, comp, sel, sinks = _ds41_case(990 + T, T, H, pos0, window, R, ratio, K, with_comp)
    if comp is None and with_comp:
        comp = np.zeros((1, 512), np.uint16)
    assert ds41x.ns_ds41_attend_xmx_supported(i64(H), i64(512)) == 1
    got = np.full((T, H, 512), np.nan, np.float32)
    rc = ds41x.ns_ds41_attend_xmx(C.c_void_p(ds41x.ref_gpu()), q.ctypes.data_as(f32p), raw.ctypes.data_as(u16p), i64(R),
                                  None if comp is None else comp.ctypes.data_as(u16p), i64(ratio), None if sel is None else sel.ctypes.data_as(i32p), i64(K),
                                  sinks.ctypes.data_as(f32p), got.ctypes.data_as(f32p), i64(T), i64(H), i64(pos0), i64(window), C.c_float(DSCALE))
    assert rc == 0, ds41x.ref_error()
    want = O.ds41_attend(q, raw, R, comp, ratio, sel, K, sinks, T, H, pos0, window, DSCALE, mode=1)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"max abs difference {np.abs(got - want).max():.3e}"


nhx = O.ref_unit("ref_nhx")


@pytest.mark.skipif(nhx is None, reason="oracle/_ref/libref_nhx.so not built (no reference checkout)")
@pytest.mark.parametrize("T,Hkv,p0", [(9, 1, 0), (21, 2, 50), (1, 1, 0), (1, 2, 700), (8, 1, 60), (3, 1, 4000)])
def test_nemotronh_matrix_unit_kernels(T, Hkv, p0):
    """ns_nhs_attn_prompt and ns_nhs_attn_decode (kernels/llm/nemotronh/silo/attn.cpp: the flash kernel for heads of 128,
    16 query heads a key head) - the reference's lines - against orc_gqa_flash_prefill / orc_gqa_flash_decode, to the bit."""
    Hq, D, cap = 16 * Hkv, 128, p0 + T + 2
    r = W.rng(963, T * 1000 + p0)
    q = r.standard_normal((T, Hq * D), dtype=np.float32)
    k = (r.standard_normal((Hkv, cap, D)) * 0.5).astype(np.float16)
    v = (r.standard_normal((Hkv, cap, D)) * 0.5).astype(np.float16)
    got = np.full((T, Hq * D), np.nan, np.float32)
    gq = C.c_void_p(nhx.ref_gpu())
    if T > 8:
        rc = nhx.ns_nhs_attn_prompt(gq, q.ctypes.data_as(f32p), i64(Hq * D), k.ctypes.data_as(u16p), v.ctypes.data_as(u16p), i64(T), i64(Hq), i64(Hkv), i64(D),
                                    i64(cap), i64(p0), got.ctypes.data_as(f32p))
        want = O.gqa_flash_prefill(q, k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, cap, p0)
    else:
        nhx.ns_nhs_attn_decode_scratch.restype = i64
        sc = np.zeros(max(1, nhx.ns_nhs_attn_decode_scratch(i64(T), i64(Hq), i64(Hkv), i64(D), i64(p0))), np.float32)
        rc = nhx.ns_nhs_attn_decode(gq, q.ctypes.data_as(f32p), i64(Hq * D), k.ctypes.data_as(u16p), v.ctypes.data_as(u16p), i64(T), i64(Hq), i64(Hkv), i64(D),
                                    i64(cap), i64(p0), got.ctypes.data_as(f32p), sc.ctypes.data_as(f32p))
        want = O.gqa_flash_decode(q, k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, cap, p0)
    assert rc == 0, nhx.ref_error()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"max abs difference {np.abs(got - want).max():.3e}"


@pytest.mark.parametrize("T,H,n,ld,pos0,ratio", [
    (3, 32, 77, 80, 400, 4),       # the matrix-unit form: a last tile read shifted back, keys past the cache's
    (2, 32, 300, 300, 20, 4),      # rows that see only the first few keys
    (1, 32, 8, 8, 100, 4),         # one tile
    (2, 32, 5, 16, 100, 4),        # fewer than 8 keys: the scalar form
    (2, 16, 90, 96, 1000, 4),      # 16 heads: the scalar form
])
def test_ds41_indexer_score_kernels(T, H, n, ld, pos0, ratio):
    """ns_ds41_idx_score (kernels/llm/deepseek41/silo/k41.cpp: idx_score_xmx for 32 heads of 128 and at least 8 keys, else the
    scalar kernel) and ns_ds41_idx_score_cand (idx_score_cand_xmx) - the reference's lines - against orc_ds41_idx_score and
    orc_ds41_idx_score_cand, to the bit."""
    D = 128
    r = W.rng(995, n * 10 + T)
    q = r.standard_normal((T, H, D), dtype=np.float32)
    w = r.standard_normal((T, H), dtype=np.float32)
    k = (r.standard_normal((n, D)) * 0.5).astype(np.float16)
    got = np.full((T, ld), np.nan, np.float32)
    rc = ref.ns_ds41_idx_score(g(), q.ctypes.data_as(f32p), w.ctypes.data_as(f32p), k.ctypes.data_as(u16p), got.ctypes.data_as(f32p), i64(T), i64(H), i64(D),
                               i64(n), i64(ld), i64(pos0), i64(ratio))
    assert rc == 0, ref.ref_error()
    xmx = H == 32 and n >= 8
    want = O.ds41_idx_score(q, w, k.view(np.uint16), T, H, D, n, ld, pos0, ratio, half_q=xmx)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"max abs difference {np.nanmax(np.abs(got - want)):.3e}"
    if not xmx:
        return
    nb = (n + 7) // 8
    K = min(6, nb + 2)
    cand = np.stack([np.sort(r.choice(nb + 2, size=K, replace=False)).astype(np.int32) - 1 for _ in range(T)])     # -1 and nb among them: no block
    cand = np.ascontiguousarray(cand)
    gotc = np.full((T, K * 8), np.nan, np.float32)
    rc = ref.ns_ds41_idx_score_cand(g(), q.ctypes.data_as(f32p), w.ctypes.data_as(f32p), k.ctypes.data_as(u16p), cand.ctypes.data_as(i32p), i64(K),
                                    gotc.ctypes.data_as(f32p), i64(T), i64(H), i64(D), i64(n), i64(pos0), i64(ratio))
    assert rc == 0, ref.ref_error()
    wantc = O.ds41_idx_score_cand(q, w, k.view(np.uint16), cand, K, T, H, D, n, pos0, ratio)
    assert np.array_equal(gotc.view(np.uint32), wantc.view(np.uint32))
