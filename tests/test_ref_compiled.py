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
