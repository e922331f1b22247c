"""The quantised GQA caches (q8_0 / q4_0, heads of 256) on the GPU against the CPU oracle, through the C ABI
(kernels/llm/qwen35/q35.cpp:281-348 and the reader silo/attn.cpp:49-78 restated). The writer and the rotation are
bit-exact; attention over a quantised cache is held to |got - want| <= 2e-3 + 1e-2 |want| against the reference's flash
numerics on the values its reader produces."""
import numpy as np
import pytest

from nextsycl_b200 import DevBuf
from nextsycl_b200 import workloads as W
from nextsycl_b200.core import check
from oracle import oracle as O

pytestmark = pytest.mark.gpu
ABS, REL = 2e-3, 1e-2


def assert_close(got, want, what):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert np.isfinite(got).all(), what
    d = np.abs(got - want)
    bad = d > ABS + REL * np.abs(want)
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside tolerance, max abs {d.max():.3e}"


def rows(seed, T, Hkv, scale=1.0):
    rng = W.rng(seed, 0)
    k = (scale * rng.standard_normal((T, Hkv * 256), dtype=np.float32)).astype(np.float32)
    v = (scale * rng.standard_normal((T, Hkv * 256), dtype=np.float32)).astype(np.float32)
    return k, v


def store(gpu, kt, k, v, T, Hkv, cap, p0, kc0=None, vc0=None):
    rb = O.q_row_bytes(kt)
    kc0 = np.zeros((Hkv, cap, rb), np.uint8) if kc0 is None else kc0
    vc0 = np.zeros((Hkv, cap, rb), np.uint8) if vc0 is None else vc0
    dk, dv, dkc, dvc = DevBuf.of(gpu, k), DevBuf.of(gpu, v), DevBuf.of(gpu, kc0), DevBuf.of(gpu, vc0)
    check(gpu.api, gpu.api.ns_q35_kv_store_q(gpu.raw, kt, dk.ptr, k.shape[1], dv.ptr, v.shape[1], T, Hkv, 256, cap, p0, dkc.ptr, dvc.ptr), "ns_q35_kv_store_q")
    gpu.sync()
    return dkc, dvc


@pytest.mark.parametrize("kt", [1, 2])
def test_store_bit_exact(gpu, kt):
    T, Hkv, cap, p0 = 37, 4, 64, 11
    k, v = rows(1200 + kt, T, Hkv, 2.0)
    k[0, :32] = 0.0                          # a zero block
    k[1, 32:64] = np.float32(1.25)           # a constant block: every value ties for the largest
    v[2, 0:32] = np.arange(32, dtype=np.float32) - 16.0
    v[3, 5] = np.float32(1e4)                # one large value: the rest of its block quantises to (almost) nothing
    rb = O.q_row_bytes(kt)
    before = W.rng(1210, kt).integers(0, 255, size=(Hkv, cap, rb), dtype=np.uint8)
    dkc, dvc = store(gpu, kt, k, v, T, Hkv, cap, p0, before.copy(), before.copy())
    wk, wv = before.copy(), before.copy()
    O.kv_store_q(kt, k, v, T, Hkv, cap, p0, wk, wv)
    assert np.array_equal(dkc.read(np.uint8).reshape(Hkv, cap, rb), wk)   # rows outside p0 .. p0+T-1 untouched
    assert np.array_equal(dvc.read(np.uint8).reshape(Hkv, cap, rb), wv)


def test_fwht32_bit_exact(gpu):
    x = W.rng(1220, 0).standard_normal((9, 512), dtype=np.float32)
    stride = 520
    buf = np.zeros((9, stride), np.float32)
    buf[:, :512] = x
    buf[:, 512:] = 7.0
    d = DevBuf.of(gpu, buf)
    check(gpu.api, gpu.api.ns_q35_fwht32(gpu.raw, d.ptr, 9, 512, stride), "ns_q35_fwht32")
    gpu.sync()
    got = d.read(np.float32).reshape(9, stride)
    assert np.array_equal(got[:, :512], O.fwht32(x.copy()))
    assert np.all(got[:, 512:] == 7.0)
    assert gpu.api.ns_q35_fwht32(gpu.raw, d.ptr, 9, 500, stride) == -1


@pytest.mark.parametrize("kt,T,kv", [(1, 1, 700), (2, 1, 700), (1, 4, 3000), (2, 8, 1029), (1, 1, 17)])
def test_decode_over_a_quantised_cache(gpu, kt, T, kv):
    Hq, Hkv, D = 24, 4, 256
    cap, p0 = kv + 5, kv - T
    k, v = rows(1230 + kt + T, kv, Hkv)
    dkc, dvc = store(gpu, kt, k, v, kv, Hkv, cap, 0)
    q = W.rng(1240, T).standard_normal((T, Hq * D), dtype=np.float32)
    dq, out = DevBuf.of(gpu, q), DevBuf(gpu, T * Hq * D * 4)
    n = int(gpu.api.ns_q35_attn_decode_scratch(T, Hq, Hkv, D, p0))
    sc = DevBuf(gpu, max(n, 1) * 4)
    check(gpu.api, gpu.api.ns_q35_attn_decode_kv(gpu.raw, kt, dq.ptr, Hq * D, dkc.ptr, dvc.ptr, T, Hq, Hkv, D, cap, p0, out.ptr, sc.ptr), "decode_kv")
    gpu.sync()
    got = out.read(np.float32).reshape(T, Hq * D)
    rb = O.q_row_bytes(kt)
    kq = O.kv_dequant(kt, dkc.read(np.uint8).reshape(Hkv, cap, rb), Hkv, cap, kv)
    vq = O.kv_dequant(kt, dvc.read(np.uint8).reshape(Hkv, cap, rb), Hkv, cap, kv)
    assert_close(got, O.gqa_flash_decode(q, kq, vq, T, Hq, Hkv, D, kv, p0), f"kt {kt} against the reference numerics")
    assert_close(got, O.attn_exact(q, kq, vq, T, Hq, Hkv, D, D, kv, p0, 1.0 / 16.0), f"kt {kt} against fp64 on the same values")


@pytest.mark.parametrize("kt", [1, 2])
@pytest.mark.parametrize("kv", [1, 2, 3, 15, 16, 17, 31, 33, 64, 65, 130])
def test_decode_short_contexts_and_tile_edges(gpu, kt, kv):
    """The quantised decode takes a tile's keys in a permuted order (four consecutive keys a lane): contexts that end
    anywhere inside a 16-key tile, and verify rows whose last visible key differs, must mask exactly the right ones."""
    T = min(kv, 3)
    Hq, Hkv, D = 12, 2, 256
    cap, p0 = kv + 2, kv - T
    k, v = rows(1300 + kt + kv, kv, Hkv)
    dkc, dvc = store(gpu, kt, k, v, kv, Hkv, cap, 0)
    q = W.rng(1301, kv).standard_normal((T, Hq * D), dtype=np.float32)
    dq, out = DevBuf.of(gpu, q), DevBuf(gpu, T * Hq * D * 4)
    sc = DevBuf(gpu, max(int(gpu.api.ns_q35_attn_decode_scratch(T, Hq, Hkv, D, p0)), 1) * 4)
    check(gpu.api, gpu.api.ns_q35_attn_decode_kv(gpu.raw, kt, dq.ptr, Hq * D, dkc.ptr, dvc.ptr, T, Hq, Hkv, D, cap, p0, out.ptr, sc.ptr), "decode_kv")
    gpu.sync()
    got = out.read(np.float32).reshape(T, Hq * D)
    rb = O.q_row_bytes(kt)
    kq = O.kv_dequant(kt, dkc.read(np.uint8).reshape(Hkv, cap, rb), Hkv, cap, kv)
    vq = O.kv_dequant(kt, dvc.read(np.uint8).reshape(Hkv, cap, rb), Hkv, cap, kv)
    assert_close(got, O.gqa_flash_decode(q, kq, vq, T, Hq, Hkv, D, kv, p0), f"kt {kt} kv {kv}")


@pytest.mark.parametrize("kt", [1, 2])
@pytest.mark.parametrize("amp", [5000.0, 0.05])
def test_decode_with_large_and_small_values(gpu, kt, amp):
    """The decode kernel puts a value's scale onto the softmax weight (times 2^6) as a half: values near the top of the
    fp16 range must not overflow that product, small ones must not lose it to subnormals. Relative tolerance only."""
    T, Hq, Hkv, D, kv = 1, 24, 4, 256, 2100
    cap, p0 = kv, kv - T
    k, v = rows(1290 + kt, kv, Hkv)
    v *= np.float32(amp)
    dkc, dvc = store(gpu, kt, k, v, kv, Hkv, cap, 0)
    q = W.rng(1291, kt).standard_normal((T, Hq * D), dtype=np.float32)
    dq, out = DevBuf.of(gpu, q), DevBuf(gpu, T * Hq * D * 4)
    sc = DevBuf(gpu, max(int(gpu.api.ns_q35_attn_decode_scratch(T, Hq, Hkv, D, p0)), 1) * 4)
    check(gpu.api, gpu.api.ns_q35_attn_decode_kv(gpu.raw, kt, dq.ptr, Hq * D, dkc.ptr, dvc.ptr, T, Hq, Hkv, D, cap, p0, out.ptr, sc.ptr), "decode_kv")
    gpu.sync()
    got = out.read(np.float32).reshape(T, Hq * D).astype(np.float64)
    rb = O.q_row_bytes(kt)
    kq = O.kv_dequant(kt, dkc.read(np.uint8).reshape(Hkv, cap, rb), Hkv, cap, kv)
    vq = O.kv_dequant(kt, dvc.read(np.uint8).reshape(Hkv, cap, rb), Hkv, cap, kv)
    want = np.asarray(O.gqa_flash_decode(q, kq, vq, T, Hq, Hkv, D, kv, p0), np.float64)
    assert np.isfinite(got).all()
    d = np.abs(got - want)
    assert (d <= ABS * amp + REL * np.abs(want)).all(), f"amp {amp}: max abs {d.max():.3e} against values of {np.abs(want).max():.3e}"


@pytest.mark.parametrize("kt", [1, 2])
def test_prompt_over_a_quantised_cache(gpu, kt):
    T, Hq, Hkv, D, p0 = 70, 12, 2, 256, 130
    kv, cap = p0 + T, p0 + T + 9
    k, v = rows(1250 + kt, kv, Hkv)
    dkc, dvc = store(gpu, kt, k, v, kv, Hkv, cap, 0)
    q = W.rng(1260, kt).standard_normal((T, Hq * D), dtype=np.float32)
    dq, out = DevBuf.of(gpu, q), DevBuf(gpu, T * Hq * D * 4)
    check(gpu.api, gpu.api.ns_q35_attn_prompt_kv(gpu.raw, kt, dq.ptr, Hq * D, dkc.ptr, dvc.ptr, T, Hq, Hkv, D, cap, p0, out.ptr), "prompt_kv")
    gpu.sync()
    got = out.read(np.float32).reshape(T, Hq * D)
    rb = O.q_row_bytes(kt)
    kq = O.kv_dequant(kt, dkc.read(np.uint8).reshape(Hkv, cap, rb), Hkv, cap, kv)
    vq = O.kv_dequant(kt, dvc.read(np.uint8).reshape(Hkv, cap, rb), Hkv, cap, kv)
    assert_close(got, O.gqa_flash_prefill(q, kq, vq, T, Hq, Hkv, D, kv, p0), f"kt {kt}")


def test_rejects(gpu):
    api = gpu.api
    k, v = rows(1270, 2, 2)
    dk, dv = DevBuf.of(gpu, k), DevBuf.of(gpu, v)
    c = DevBuf(gpu, 2 * 8 * 272)
    assert api.ns_q35_kv_store_q(gpu.raw, 3, dk.ptr, 512, dv.ptr, 512, 2, 2, 256, 8, 0, c.ptr, c.ptr) == -1    # no such form
    assert api.ns_q35_kv_store_q(gpu.raw, 1, dk.ptr, 512, dv.ptr, 512, 2, 2, 128, 8, 0, c.ptr, c.ptr) == -1    # heads of 256 only
    assert api.ns_q35_kv_store_q(gpu.raw, 1, dk.ptr, 512, dv.ptr, 512, 2, 2, 256, 8, 7, c.ptr, c.ptr) == -1    # past the capacity
    q = DevBuf(gpu, 24 * 256 * 4)
    assert api.ns_q35_attn_decode_kv(gpu.raw, 5, q.ptr, 24 * 256, c.ptr, c.ptr, 1, 24, 4, 256, 8, 0, q.ptr, None) == -1


@pytest.mark.parametrize("kt,mode", [(0, 0), (1, 0), (2, 1), (0, 1)])
def test_attn_probs(gpu, kt, mode):
    """ns_q35_attn_probs against the oracle (kernels/llm/qwen35/q35.cpp:464-506 restated): fp32 arithmetic, the sums in
    another order: 1e-6 absolute on weights that sum to one, 1e-4 relative."""
    api = gpu.api
    Hq, Hkv, cap, n = 12, 2, 700, 650
    rb = O.q_row_bytes(kt)
    k, v = rows(1280 + kt, cap, Hkv)
    if kt == 0:
        kc = np.ascontiguousarray(k.reshape(cap, Hkv, 256).transpose(1, 0, 2)).astype(np.float16).view(np.uint8).reshape(Hkv, cap, 512)
        dkc = DevBuf.of(gpu, kc)
    else:
        dkc, _ = store(gpu, kt, k, v, cap, Hkv, cap, 0)
        kc = dkc.read(np.uint8).reshape(Hkv, cap, rb)
    q = W.rng(1285, kt).standard_normal(Hq * 256, dtype=np.float32)
    before = W.rng(1286, 0).random(n, dtype=np.float32)
    dq, dout, dsc = DevBuf.of(gpu, q), DevBuf.of(gpu, before), DevBuf(gpu, Hq * 2 * 4)
    check(api, api.ns_q35_attn_probs(gpu.raw, kt, dq.ptr, dkc.ptr, Hq, Hkv, 256, cap, n, mode, dsc.ptr, dout.ptr), "ns_q35_attn_probs")
    gpu.sync()
    want = before.copy()
    wsc = O.q35_attn_probs(kt, q, kc, Hq, Hkv, cap, n, mode, want)
    got = dout.read(np.float32)
    assert np.all(np.abs(got - want) <= 1e-6 + 1e-4 * np.abs(want)), float(np.abs(got - want).max())
    gsc = dsc.read(np.float32).reshape(Hq, 2)
    assert np.allclose(gsc, wsc, rtol=1e-4, atol=1e-5)
    if mode == 0:
        assert abs(float((got - before).sum()) - 1.0) < 1e-3      # the heads' mean weights sum to one over the keys
    assert api.ns_q35_attn_probs(gpu.raw, kt, dq.ptr, dkc.ptr, Hq, Hkv, 128, cap, n, mode, dsc.ptr, dout.ptr) == -1
