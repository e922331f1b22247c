"""glm5next's DSA indexer on the GPU against the CPU oracle, through the C ABI (kernels/llm/glm5next/glm.cpp:876-1015
restated). ns_topk is index work: bit-exact. ns_idx_pool and ns_idx_score are fp32 with device exp and another order of
sums: 1e-5 absolute, 1e-5 relative; the ring ns_idx_pool leaves behind is a copy: bit-exact."""
import numpy as np
import pytest

from nextsycl_b200 import DevBuf
from nextsycl_b200 import workloads as W
from nextsycl_b200.core import check
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def run_topk(gpu, score, n, K):
    T, ld = score.shape
    ds, dsel = DevBuf.of(gpu, score), DevBuf.of(gpu, np.full((T, K), -1, np.int32))
    check(gpu.api, gpu.api.ns_topk(gpu.raw, ds.ptr, dsel.ptr, T, n, ld, K), "ns_topk")
    gpu.sync()
    return dsel.read(np.int32).reshape(T, K)


@pytest.mark.parametrize("T,n,ld,K,kind", [
    (1, 1000, 1000, 64, "normal"), (3, 4097, 4100, 512, "ties"), (2, 65536, 65536, 2048, "normal"), (4, 700, 800, 700, "ties"),
    (1, 5000, 5000, 1, "normal"), (2, 3000, 3000, 100, "masked"), (1, 50, 64, 80, "normal"), (2, 2048, 2048, 300, "constant"),
])
def test_topk_bit_exact(gpu, T, n, ld, K, kind):
    rng = W.rng(1400, n + K)
    score = np.full((T, ld), 7.0, np.float32)                      # what lies past n is not looked at
    x = rng.standard_normal((T, n), dtype=np.float32)
    if kind == "ties":
        x = np.round(x * 2) / 2
    if kind == "constant":
        x[:] = -1.5
    if kind == "masked":
        x[:, n // 3:] = -np.inf                                    # pools the row does not see yet
        x[1, :10] = 0.0
        x[1, 5] = -0.0
    score[:, :n] = x
    got = run_topk(gpu, score, n, K)
    assert np.array_equal(got, O.topk(score, n, K))


def test_idx_score(gpu):
    T, H, n, j0, pos0 = 5, 32, 300, 100, 1590
    ld = j0 + n + 7
    S = W.rng(1410, 0).standard_normal((T * H, n), dtype=np.float32)
    w = W.rng(1410, 1).standard_normal((T, H), dtype=np.float32)
    before = np.full((T, ld), 3.0, np.float32)
    dS, dw, dsc = DevBuf.of(gpu, S), DevBuf.of(gpu, w), DevBuf.of(gpu, before)
    check(gpu.api, gpu.api.ns_idx_score(gpu.raw, dS.ptr, dw.ptr, dsc.ptr, T, H, j0, n, ld, pos0), "ns_idx_score")
    gpu.sync()
    want = before.copy()
    O.idx_score(S, w, want, T, H, j0, n, pos0)
    got = dsc.read(np.float32).reshape(T, ld)
    assert np.array_equal(np.isneginf(got), np.isneginf(want))     # the pools a row does not see: (pos0 + r + 1) / 4 on
    fin = np.isfinite(want)
    assert np.all(np.abs(got[fin] - want[fin]) <= 1e-5 + 1e-5 * np.abs(want[fin]))
    assert np.array_equal(got[:, :j0], before[:, :j0]) and np.array_equal(got[:, j0 + n:], before[:, j0 + n:])


@pytest.mark.parametrize("pos0,T", [(0, 11), (6, 1), (7, 1), (13, 5), (1021, 40)])
def test_idx_pool_and_its_ring(gpu, pos0, T):
    D = 128
    rng = W.rng(1420, pos0)
    ik, ig = rng.standard_normal((T, D), dtype=np.float32), rng.standard_normal((T, D), dtype=np.float32)
    ape = rng.standard_normal((4, D), dtype=np.float32)
    ring = rng.standard_normal((8, 2 * D), dtype=np.float32)       # the previous pass's last tokens
    pools = (pos0 + T) // 4 + 2
    before = np.full((pools, D), 9.0, np.float32)
    dring, dik, dig, dape, dp = DevBuf.of(gpu, ring), DevBuf.of(gpu, ik), DevBuf.of(gpu, ig), DevBuf.of(gpu, ape), DevBuf.of(gpu, before)
    check(gpu.api, gpu.api.ns_idx_pool(gpu.raw, dring.ptr, dik.ptr, dig.ptr, dape.ptr, dp.ptr, pos0, T, D), "ns_idx_pool")
    gpu.sync()
    wring, wp = ring.copy(), before.copy()
    O.idx_pool(wring, ik, ig, ape, wp, pos0, T, D)
    got = dp.read(np.float32).reshape(pools, D)
    assert np.all(np.abs(got - wp) <= 1e-5 + 1e-5 * np.abs(wp))
    lo, hi = pos0 // 4, (pos0 + T) // 4
    assert np.array_equal(got[:lo], before[:lo]) and np.array_equal(got[hi:], before[hi:])     # only the completed pools
    assert np.array_equal(dring.read(np.float32).reshape(8, 2 * D), wring)
