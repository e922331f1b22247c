"""The deepseek41 engine's attention symbols on the GPU against the CPU oracle (kernels/llm/deepseek41/silo/attn.cpp and
silo/ds41.cpp restated), through the C ABI. Tolerance: |got - want| <= 2e-3 + 1e-2 |want| against both of the reference's
numerics (its XMX kernel's, which this path shares: fp16 q and weights, exp2; and its vector kernel's fp32 ones - the bar
the benchmark sets for fp16 tensor-core numerics); bit-exact for the two cache writers."""
import numpy as np
import pytest

from nextsycl_b200 import DevBuf
from nextsycl_b200 import workloads as W
from nextsycl_b200.core import check
from oracle import oracle as O

pytestmark = pytest.mark.gpu
SCALE = np.float32(512 ** -0.5)


def close(got, want, abs_tol=2e-3, rel_tol=1e-2):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert np.isfinite(got).all()
    d = np.abs(got - want)
    assert np.all(d <= abs_tol + rel_tol * np.abs(want)), float(d.max())


def case(seed, T, H, pos0, window, R, ratio, K, with_comp=True):
    rng = W.rng(seed, 0)
    q = rng.standard_normal((T, H, 512), dtype=np.float32)
    raw = O.to_f16_bits(0.5 * rng.standard_normal((R, 512), dtype=np.float32))
    ncomp = (pos0 + T) // ratio if with_comp else 0
    comp = O.to_f16_bits(0.5 * rng.standard_normal((ncomp, 512), dtype=np.float32)) if ncomp else None
    sel = None
    if K and comp is not None:
        # each row lists K of the cells it sees (rows that see at most K never read theirs)
        sel = np.zeros((T, K), np.int32)
        for t in range(T):
            vis = (pos0 + t + 1) // ratio
            if vis > K:
                sel[t] = np.sort(rng.choice(vis, size=K, replace=False))
    sinks = rng.standard_normal(H).astype(np.float32)
    return q, raw, comp, sel, sinks


def run(gpu, fn, q, raw, R, comp, ratio, sel, K, sinks, T, H, pos0, window):
    dq, draw, dsk = DevBuf.of(gpu, q), DevBuf.of(gpu, raw), DevBuf.of(gpu, sinks)   # named: a buffer lives as long as its object
    dcomp = DevBuf.of(gpu, comp) if comp is not None else None
    dsel = DevBuf.of(gpu, sel) if sel is not None else None
    out = DevBuf(gpu, T * H * 512 * 4)
    check(gpu.api, fn(gpu.raw, dq.ptr, draw.ptr, R, dcomp.ptr if dcomp else None, ratio, dsel.ptr if dsel else None, K, dsk.ptr, out.ptr, T, H,
                      pos0, window, SCALE), "ns_ds41_attend")
    gpu.sync()
    return out.read(np.float32).reshape(T, H, 512)


@pytest.mark.parametrize("T,H,pos0,window,R,ratio,K,with_comp", [
    (1, 64, 5, 128, 128, 4, 0, False),        # fewer tokens than the window, no compressed cells
    (1, 64, 1000, 128, 128, 4, 0, False),     # a full window, the ring wrapped many times
    (1, 64, 4095, 128, 128, 4, 0, True),      # window + every compressed cell (1024): several key splits
    (1, 64, 8191, 128, 160, 4, 512, True),    # the indexer's picks (sees 2048 > K), a ring longer than the window
    (4, 64, 2044, 128, 128, 4, 512, True),    # rows either side of the point where picks start (vis 511..512 -> 512 = K)
    (5, 16, 2100, 64, 64, 4, 128, True),      # several rows, all picking
    (3, 8, 0, 16, 16, 128, 0, True),          # the first tokens: one, two, three cells; comp given but nothing visible yet
    (40, 64, 0, 128, 128, 4, 0, True),        # prompt rows from position 0
])
def test_attend_against_both_numerics(gpu, T, H, pos0, window, R, ratio, K, with_comp):
    q, raw, comp, sel, sinks = case(980 + T, T, H, pos0, window, R, ratio, K, with_comp)
    if comp is None and with_comp:
        comp = np.zeros((1, 512), np.uint16)   # a valid pointer with no cell visible
    for fn in (gpu.api.ns_ds41_attend_xmx, gpu.api.ns_ds41_attend):
        got = run(gpu, fn, q, raw, R, comp, ratio, sel, K, sinks, T, H, pos0, window)
        close(got, O.ds41_attend(q, raw, R, comp, ratio, sel, K, sinks, T, H, pos0, window, SCALE, mode=1))
        close(got, O.ds41_attend(q, raw, R, comp, ratio, sel, K, sinks, T, H, pos0, window, SCALE, mode=0))


def test_sink_limits(gpu):
    """A sink far below every score leaves the plain softmax; far above, the output vanishes (silo/attn.cpp:266-285)."""
    T, H, pos0, window, R, ratio = 2, 64, 3000, 128, 128, 4
    q, raw, comp, _, sinks = case(990, T, H, pos0, window, R, ratio, 0)
    low = np.full(H, -1e4, np.float32)
    got = run(gpu, gpu.api.ns_ds41_attend_xmx, q, raw, R, comp, ratio, None, 0, low, T, H, pos0, window)
    close(got, O.ds41_attend(q, raw, R, comp, ratio, None, 0, low, T, H, pos0, window, SCALE, mode=1))
    high = np.full(H, 1e4, np.float32)
    got = run(gpu, gpu.api.ns_ds41_attend_xmx, q, raw, R, comp, ratio, None, 0, high, T, H, pos0, window)
    assert np.abs(got).max() < 1e-30


def test_a_row_of_a_verify_pass_equals_the_one_row_pass(gpu):
    """Decode widths (at most 8 rows): a row's split size comes from its own cells, so row t of a pass equals the same
    position run alone bit for bit (kernels/llm/deepseek41/silo/attn.cpp:316-319)."""
    T, H, pos0, window, R, ratio, K = 3, 64, 5000, 128, 128, 4, 256
    q, raw, comp, sel, sinks = case(991, T, H, pos0, window, R, ratio, K)
    whole = run(gpu, gpu.api.ns_ds41_attend_xmx, q, raw, R, comp, ratio, sel, K, sinks, T, H, pos0, window)
    for t in range(T):
        alone = run(gpu, gpu.api.ns_ds41_attend_xmx, q[t:t + 1].copy(), raw, R, comp, ratio, sel[t:t + 1].copy(), K, sinks, 1, H, pos0 + t, window)
        assert np.array_equal(alone[0], whole[t])
    # rows whose cell counts differ (no picks: every compressed cell): 8 rows across a step of the compressed count
    T, pos0 = 8, 4090
    q, raw, comp, _, sinks = case(994, T, H, pos0, window, R, ratio, 0)
    whole = run(gpu, gpu.api.ns_ds41_attend_xmx, q, raw, R, comp, ratio, None, 0, sinks, T, H, pos0, window)
    for t in (0, 5, 7):
        alone = run(gpu, gpu.api.ns_ds41_attend_xmx, q[t:t + 1].copy(), raw, R, comp, ratio, None, 0, sinks, 1, H, pos0 + t, window)
        assert np.array_equal(alone[0], whole[t])


def test_rejects_bad_arguments(gpu):
    api = gpu.api
    q, raw, comp, sel, sinks = case(992, 1, 8, 10, 8, 8, 4, 0)
    dq, draw, dsk, out = DevBuf.of(gpu, q), DevBuf.of(gpu, raw), DevBuf.of(gpu, sinks), DevBuf(gpu, 8 * 512 * 4)
    assert api.ns_ds41_attend(gpu.raw, dq.ptr, draw.ptr, 8, None, 4, None, 0, dsk.ptr, out.ptr, 1, 8, 10, 16, SCALE) == -1   # window > ring
    assert b"window" in api.ns_last_error()
    assert api.ns_ds41_attend(gpu.raw, dq.ptr, None, 8, None, 4, None, 0, dsk.ptr, out.ptr, 1, 8, 10, 8, SCALE) == -1       # no ring
    assert api.ns_ds41_attend(gpu.raw, dq.ptr, draw.ptr, 8, None, 4, None, 0, dsk.ptr, out.ptr, 0, 8, 10, 8, SCALE) == 0     # no rows: nothing to do
    assert api.ns_ds41_attend_xmx_supported(64, 512) == 1 and api.ns_ds41_attend_xmx_supported(64, 128) == 0


def test_cache_writers_bit_exact(gpu):
    api = gpu.api
    T, R, D, pos0 = 7, 16, 512, 13   # wraps: slots 13, 14, 15, 0, 1, 2, 3
    kv = W.rng(993, 0).standard_normal((T, D), dtype=np.float32)
    before = W.rng(993, 1).integers(0, 1 << 15, size=(R, D), dtype=np.uint16)
    dkv, ring = DevBuf.of(gpu, kv), DevBuf.of(gpu, before)
    check(api, api.ns_ds41_ring_put(gpu.raw, dkv.ptr, ring.ptr, T, pos0, R, D), "ring_put")
    gpu.sync()
    want = before.copy()
    for t in range(T):
        want[(pos0 + t) % R] = kv[t].astype(np.float16).view(np.uint16)
    assert np.array_equal(ring.read(np.uint16).reshape(R, D), want)
    n, j0 = 5, 3
    x = W.rng(993, 2).standard_normal((n, D), dtype=np.float32)
    cb = W.rng(993, 3).integers(0, 1 << 15, size=(12, D), dtype=np.uint16)
    dx, cache = DevBuf.of(gpu, x), DevBuf.of(gpu, cb)
    check(api, api.ns_ds41_rows_f16(gpu.raw, dx.ptr, cache.ptr, n, j0, D), "rows_f16")
    gpu.sync()
    want = cb.copy()
    want[j0:j0 + n] = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(cache.read(np.uint16).reshape(12, D), want)
