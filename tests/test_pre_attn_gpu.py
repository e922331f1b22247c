"""The step before attention on the GPU against the CPU oracle, through the C ABI (kernels/llm/qwen35/q35.cpp:220-279,
350-385 restated). fp32 arithmetic with device sin / cos / pow against libm's: |got - want| <= 1e-4 + 1e-4 |want|, plus - the
angle being an fp32 product position x frequency - what one unit in the last place of the largest angle turns a value by,
p 2^-23 max|x| (0.06 at position 100,000; nothing at small positions). The fused entry point is held bit-exact to the three
calls it replaces."""
import numpy as np
import pytest

from nextsycl_b200 import DevBuf
from nextsycl_b200 import workloads as W
from nextsycl_b200.core import check
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def close(got, want, abs_tol=1e-4, rel_tol=1e-4):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert np.isfinite(got).all()
    d = np.abs(got - want)
    assert np.all(d <= abs_tol + rel_tol * np.abs(want)), float(d.max())


@pytest.mark.parametrize("T,H,D,n_rot,p0", [(1, 24, 256, 64, 0), (7, 4, 256, 64, 4093), (3, 16, 128, 128, 100000), (2, 2, 64, 0, 5)])
def test_qk_norm_rope(gpu, T, H, D, n_rot, p0):
    api = gpu.api
    theta, eps = np.float32(1e6), np.float32(1e-6)
    x = W.rng(1300, T).standard_normal((T, H * D), dtype=np.float32)
    w = (1.0 + 0.1 * W.rng(1300, 50).standard_normal(D, dtype=np.float32)).astype(np.float32)
    dx, dw, dy = DevBuf.of(gpu, x), DevBuf.of(gpu, w), DevBuf(gpu, T * H * D * 4)
    check(api, api.ns_q35_qk_norm_rope(gpu.raw, dx.ptr, H * D, D, dy.ptr, H * D, T, H, D, dw.ptr, eps, n_rot, theta, p0), "qk_norm_rope")
    gpu.sync()
    want = O.qk_norm_rope(x, T, H, D, w, eps, n_rot, theta, p0)
    ulp = float(p0 + T) * 2.0 ** -23 * float(np.abs(want).max())
    close(dy.read(np.float32).reshape(T, H * D), want, abs_tol=1e-4 + ulp)
    # the rotation alone
    check(api, api.ns_q35_rope(gpu.raw, dx.ptr, H * D, D, dy.ptr, H * D, T, H, D, n_rot, theta, p0), "rope")
    gpu.sync()
    close(dy.read(np.float32).reshape(T, H * D), O.qk_norm_rope(x, T, H, D, None, 0.0, n_rot, theta, p0), abs_tol=1e-4 + ulp)
    # in place
    check(api, api.ns_q35_qk_norm_rope(gpu.raw, dx.ptr, H * D, D, dx.ptr, H * D, T, H, D, dw.ptr, eps, n_rot, theta, p0), "in place")
    gpu.sync()
    close(dx.read(np.float32).reshape(T, H * D), want, abs_tol=1e-4 + ulp)


def test_qk_norm_rope_pos_sections(gpu):
    api = gpu.api
    T, H, D, n_rot = 6, 4, 128, 64
    theta, eps = np.float32(1e6), np.float32(1e-6)
    x = W.rng(1310, 0).standard_normal((T, H * D), dtype=np.float32)
    w = np.ones(D, np.float32)
    pos = W.rng(1310, 1).integers(0, 5000, size=(T, 3)).astype(np.int32)
    pos[0] = 77                                   # a text row: all three positions equal
    dx, dw, dp, dy = DevBuf.of(gpu, x), DevBuf.of(gpu, w), DevBuf.of(gpu, pos), DevBuf(gpu, T * H * D * 4)
    check(api, api.ns_q35_qk_norm_rope_pos(gpu.raw, dx.ptr, H * D, D, dy.ptr, H * D, T, H, D, dw.ptr, eps, n_rot, theta, dp.ptr, 11, 11, 10), "pos")
    gpu.sync()
    got = dy.read(np.float32).reshape(T, H * D)
    close(got, O.qk_norm_rope(x, T, H, D, w, eps, n_rot, theta, 0, pos, (11, 11, 10)), abs_tol=1e-4 + 5000 * 2.0 ** -23 * 5.0)
    close(got[:1], O.qk_norm_rope(x[:1], 1, H, D, w, eps, n_rot, theta, 77))
    assert api.ns_q35_qk_norm_rope_pos(gpu.raw, dx.ptr, H * D, D, dy.ptr, H * D, T, H, D, dw.ptr, eps, n_rot, theta, dp.ptr, 0, 0, 0) == -1


def test_strided_source(gpu):
    """q, k and v of a layer usually sit in one projected row: heads hs apart inside rows ss apart."""
    api = gpu.api
    T, H, D, n_rot, p0 = 3, 4, 128, 64, 9
    ss, hs = 2 * H * D + 64, 2 * D
    buf = W.rng(1320, 0).standard_normal((T, ss), dtype=np.float32)
    x = np.stack([np.concatenate([buf[t, h * hs:h * hs + D] for h in range(H)]) for t in range(T)])
    w = (1.0 + 0.1 * W.rng(1320, 1).standard_normal(D, dtype=np.float32)).astype(np.float32)
    db, dw, dy = DevBuf.of(gpu, buf), DevBuf.of(gpu, w), DevBuf(gpu, T * H * D * 4)
    check(api, api.ns_q35_qk_norm_rope(gpu.raw, db.ptr, ss, hs, dy.ptr, H * D, T, H, D, dw.ptr, np.float32(1e-6), n_rot, np.float32(1e4), p0), "strided")
    gpu.sync()
    close(dy.read(np.float32).reshape(T, H * D), O.qk_norm_rope(x, T, H, D, w, 1e-6, n_rot, 1e4, p0))


def test_fused_prepare_equals_the_three_calls(gpu):
    api = gpu.api
    T, Hq, Hkv, D, n_rot, p0, cap = 5, 24, 4, 256, 64, 37, 64
    theta, eps = np.float32(1e6), np.float32(1e-6)
    q = W.rng(1330, 0).standard_normal((T, Hq * D), dtype=np.float32)
    k = W.rng(1330, 1).standard_normal((T, Hkv * D), dtype=np.float32)
    v = W.rng(1330, 2).standard_normal((T, Hkv * D), dtype=np.float32)
    wq = (1.0 + 0.1 * W.rng(1330, 3).standard_normal(D, dtype=np.float32)).astype(np.float32)
    wk = (1.0 + 0.1 * W.rng(1330, 4).standard_normal(D, dtype=np.float32)).astype(np.float32)
    before = W.rng(1330, 5).integers(0, 1 << 15, size=(Hkv, cap, D), dtype=np.uint16)
    dq, dk, dv, dwq, dwk = DevBuf.of(gpu, q), DevBuf.of(gpu, k), DevBuf.of(gpu, v), DevBuf.of(gpu, wq), DevBuf.of(gpu, wk)
    # the reference's sequence: norm + rope of q, of k, then the cache store
    qn, kn = DevBuf(gpu, q.nbytes), DevBuf(gpu, k.nbytes)
    kc1, vc1 = DevBuf.of(gpu, before), DevBuf.of(gpu, before)
    check(api, api.ns_q35_qk_norm_rope(gpu.raw, dq.ptr, Hq * D, D, qn.ptr, Hq * D, T, Hq, D, dwq.ptr, eps, n_rot, theta, p0), "q")
    check(api, api.ns_q35_qk_norm_rope(gpu.raw, dk.ptr, Hkv * D, D, kn.ptr, Hkv * D, T, Hkv, D, dwk.ptr, eps, n_rot, theta, p0), "k")
    check(api, api.ns_q35_kv_store(gpu.raw, kn.ptr, Hkv * D, dv.ptr, Hkv * D, T, Hkv, D, cap, p0, kc1.ptr, vc1.ptr), "store")
    # one launch
    q16, kc2, vc2 = DevBuf(gpu, T * Hq * D * 2), DevBuf.of(gpu, before), DevBuf.of(gpu, before)
    check(api, api.ns_b200_qkv_prepare(gpu.raw, dq.ptr, Hq * D, dk.ptr, Hkv * D, dv.ptr, Hkv * D, T, Hq, Hkv, D, dwq.ptr, dwk.ptr, eps, n_rot, theta, p0, cap,
                                       q16.ptr, kc2.ptr, vc2.ptr), "prepare")
    gpu.sync()
    assert np.array_equal(kc2.read(np.uint16), kc1.read(np.uint16))
    assert np.array_equal(vc2.read(np.uint16), vc1.read(np.uint16))
    assert np.array_equal(q16.read(np.float16), qn.read(np.float32).astype(np.float16))
    # and against the oracle
    want_k = O.qk_norm_rope(k, T, Hkv, D, wk, eps, n_rot, theta, p0).reshape(T, Hkv, D).astype(np.float16)
    got_k = kc2.read(np.float16).reshape(Hkv, cap, D)[:, p0:p0 + T].transpose(1, 0, 2)
    close(got_k, want_k, abs_tol=2e-3, rel_tol=2e-3)    # one fp16 rounding apart at most
    assert api.ns_b200_qkv_prepare(gpu.raw, dq.ptr, Hq * D, dk.ptr, Hkv * D, dv.ptr, Hkv * D, T, Hq, Hkv, D, dwq.ptr, dwk.ptr, eps, n_rot, theta, cap - 2, cap,
                                   q16.ptr, kc2.ptr, vc2.ptr) == -1


YARN = dict(freq_base=np.float32(10000.0), freq_scale=np.float32(0.025), ext_factor=np.float32(1.0), mscale=np.float32(1.0 + 0.1 * np.log(40.0)),
            corr0=np.float32(10.0), corr1=np.float32(23.0))


@pytest.mark.parametrize("ext", [0.0, 1.0])
def test_ds2_rope(gpu, ext):
    """deepseek2's q rows [T][H][128 nope | 64 rope]: the rope part of each head turned in place and copied out."""
    api = gpu.api
    T, H, head, off, n_dims, pos0 = 4, 16, 192, 128, 64, 3000
    x = W.rng(1340, 0).standard_normal((T, H * head), dtype=np.float32)
    y = dict(YARN, ext_factor=np.float32(ext))
    dx, dout = DevBuf.of(gpu, x), DevBuf(gpu, T * H * n_dims * 4)
    check(api, api.ns_ds2_rope(gpu.raw, dx.ptr, T, H, H * head, head, off, n_dims, pos0, y["freq_base"], y["freq_scale"], y["ext_factor"], y["mscale"],
                               y["corr0"], y["corr1"], dout.ptr, H * n_dims, n_dims), "ns_ds2_rope")
    gpu.sync()
    want, wout = x.copy().ravel(), np.zeros(T * H * n_dims, np.float32)
    O.ds2_rope(want, T, H, H * head, head, off, n_dims, pos0, *[float(y[k]) for k in ("freq_base", "freq_scale", "ext_factor", "mscale", "corr0", "corr1")],
               out=wout, out_row=H * n_dims, out_head=n_dims)
    # the angle is built from identical single-rounded products on both sides; sin / cos differ by the libraries' last places
    ulp = (pos0 + T) * 2.0 ** -23 * 5.0
    close(dx.read(np.float32), want, abs_tol=1e-5 + ulp)
    close(dout.read(np.float32), wout, abs_tol=1e-5 + ulp)
    got = dx.read(np.float32).reshape(T, H, head)
    assert np.array_equal(got[..., :off], x.reshape(T, H, head)[..., :off])      # the nope part is untouched


def test_ds2_kv_store(gpu):
    api = gpu.api
    T, L, R, pos0, n = 6, 512, 64, 1021, 1100
    kv = W.rng(1350, 0).standard_normal((T, L + R), dtype=np.float32)
    w = (1.0 + 0.1 * W.rng(1350, 1).standard_normal(L, dtype=np.float32)).astype(np.float32)
    before = W.rng(1350, 2).integers(0, 1 << 15, size=(n, L + R), dtype=np.uint16)
    dkv, dw, dc = DevBuf.of(gpu, kv), DevBuf.of(gpu, w), DevBuf.of(gpu, before)
    y = YARN
    check(api, api.ns_ds2_kv_store(gpu.raw, dkv.ptr, dw.ptr, np.float32(1e-6), dc.ptr, T, L, R, pos0, y["freq_base"], y["freq_scale"], y["ext_factor"], y["mscale"],
                                   y["corr0"], y["corr1"]), "ns_ds2_kv_store")
    gpu.sync()
    want = before.copy()
    O.ds2_kv_store(kv, w, 1e-6, want, T, L, R, pos0, *[float(y[k]) for k in ("freq_base", "freq_scale", "ext_factor", "mscale", "corr0", "corr1")])
    got = dc.read(np.uint16).reshape(n, L + R)
    assert np.array_equal(got[:pos0], before[:pos0]) and np.array_equal(got[pos0 + T:], before[pos0 + T:])
    # fp16 rows one rounding apart at most: the norm's sum order and sin / cos differ in the last place
    close(got[pos0:pos0 + T].view(np.float16), want[pos0:pos0 + T].view(np.float16), abs_tol=2e-3, rel_tol=2e-3)
    # a cache written here is what the decode kernel reads: the row count and layout of ns_ds2_mla_decode's cache
    assert got.shape[1] == 576


def sim_close(got, want, what):
    """Values on the E4M3 grid: equal but for the few whose input sat next to a rounding boundary (the norm's sum order and
    sin / cos differ in the last place between the two sides), and those within one grid step (an eighth of the value)."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert np.isfinite(got).all(), what
    same = got == want
    assert same.mean() > 0.995, f"{what}: {1 - same.mean():.4f} of the values differ"
    assert np.all(np.abs(got - want) <= 0.13 * np.abs(want) + 2e-6), what


def test_ds41_kv_post(gpu):
    api = gpu.api
    T, D, rd, pos0, R = 9, 512, 64, 250, 128      # slots 250 % 128 = 122 .. wrap past 127
    kv = W.rng(1360, 0).standard_normal((T, D), dtype=np.float32)
    w = (1.0 + 0.1 * W.rng(1360, 1).standard_normal(D, dtype=np.float32)).astype(np.float32)
    before = W.rng(1360, 2).integers(0, 1 << 15, size=(R, D), dtype=np.uint16)
    yarn = [float(YARN[k]) for k in ("freq_base", "freq_scale", "ext_factor", "mscale", "corr0", "corr1")]
    dkv, dw, dr = DevBuf.of(gpu, kv), DevBuf.of(gpu, w), DevBuf.of(gpu, before)
    check(api, api.ns_ds41_kv_post(gpu.raw, dkv.ptr, dw.ptr, T, D, np.float32(1e-6), rd, pos0, *[np.float32(v) for v in yarn], dr.ptr, R), "ns_ds41_kv_post")
    gpu.sync()
    want_kv, want_ring = kv.copy(), before.copy()
    O.ds41_kv_post(want_kv, w, T, D, 1e-6, rd, pos0, yarn, want_ring, R)
    got_kv, got_ring = dkv.read(np.float32).reshape(T, D), dr.read(np.uint16).reshape(R, D)
    sim_close(got_kv, want_kv, "kv")
    slots = [(pos0 + t) % R for t in range(T)]
    others = [s for s in range(R) if s not in slots]
    assert np.array_equal(got_ring[others], before[others])
    assert np.array_equal(got_ring[slots].view(np.float16), got_kv.astype(np.float16))    # the ring holds what kv keeps
    # every value is on the E4M3 grid of its block: value / scale has at most 4 significant bits
    blocks = got_kv.reshape(T, D // 32, 32).astype(np.float64)
    sc = 2.0 ** np.ceil(np.log2(np.maximum(np.abs(blocks).max(-1, keepdims=True), 1e-4) / 448.0))
    m, _ = np.frexp(blocks / sc)
    assert np.all(m * 16 == np.round(m * 16))


def test_ds41_att_post(gpu):
    api = gpu.api
    T, H, D, rd, pos0 = 3, 8, 512, 64, 777
    x = W.rng(1370, 0).standard_normal((T, H, D), dtype=np.float32)
    yarn = [float(YARN[k]) for k in ("freq_base", "freq_scale", "ext_factor", "mscale", "corr0", "corr1")]
    dx = DevBuf.of(gpu, x)
    check(api, api.ns_ds41_att_post(gpu.raw, dx.ptr, T, H, D, rd, pos0, *[np.float32(v) for v in yarn]), "ns_ds41_att_post")
    gpu.sync()
    want = x.copy()
    O.ds41_att_post(want, T, H, D, rd, pos0, yarn)
    got = dx.read(np.float32).reshape(T, H, D)
    sim_close(got, want, "att_post")
    assert np.array_equal(got[..., :D - rd - 32], want[..., :D - rd - 32])      # blocks without rotated values: exact
    assert api.ns_ds41_att_post(gpu.raw, dx.ptr, T, H, 500, rd, pos0, *[np.float32(v) for v in yarn]) == -1
