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


def _ds41_case(T, H, D, n, seed):
    rng = W.rng(seed, 0)
    q = rng.standard_normal((T, H, D), dtype=np.float32)
    w = rng.standard_normal((T, H), dtype=np.float32)
    k = O.to_f16_bits(rng.standard_normal((n, D), dtype=np.float32))
    return q, w, k


@pytest.mark.parametrize("T,H,D,n,ld,pos0,ratio", [(1, 32, 128, 5000, 5008, 19999, 4), (5, 32, 128, 777, 800, 3000, 4), (3, 32, 128, 8, 16, 30, 4),
                                                   (2, 16, 64, 300, 300, 1100, 4), (2, 32, 128, 5, 8, 100, 4)])
def test_ds41_idx_score(gpu, T, H, D, n, ld, pos0, ratio):
    """32 heads of 128 with at least 8 keys: the tensor-core form (q rounded to fp16); else the scalar form (fp32 q). fp32
    sums of 128 x 32 products in another order: 1e-3 absolute on scores of size ~100, 1e-4 relative."""
    q, w, k = _ds41_case(T, H, D, n, 1430 + n)
    dq, dw, dk, ds = DevBuf.of(gpu, q), DevBuf.of(gpu, w), DevBuf.of(gpu, k), DevBuf(gpu, T * ld * 4)
    ds.fill(0x55)
    check(gpu.api, gpu.api.ns_ds41_idx_score(gpu.raw, dq.ptr, dw.ptr, dk.ptr, ds.ptr, T, H, D, n, ld, pos0, ratio), "ns_ds41_idx_score")
    gpu.sync()
    got = ds.read(np.float32).reshape(T, ld)
    tensor = H == 32 and D == 128 and n >= 8
    want = O.ds41_idx_score(q, w, k, T, H, D, n, ld, pos0, ratio, half_q=tensor)
    assert np.array_equal(np.isneginf(got), np.isneginf(want))
    fin = np.isfinite(want)
    assert np.all(np.abs(got[fin] - want[fin]) <= 1e-3 + 1e-4 * np.abs(want[fin])), float(np.abs(got[fin] - want[fin]).max())


def test_ds41_candidate_steps(gpu):
    api = gpu.api
    T, H, D, n, pos0, ratio, bs, K = 3, 32, 128, 1003, 4100, 4, 8, 20
    ld = 1008
    q, w, k = _ds41_case(T, H, D, n, 1440)
    score = O.ds41_idx_score(q, w, k, T, H, D, n, ld, pos0, ratio)
    nb = -(-n // bs)
    # block maxima: exact
    dsc, dbm = DevBuf.of(gpu, score), DevBuf(gpu, T * nb * 4)
    check(api, api.ns_ds41_block_max(gpu.raw, dsc.ptr, dbm.ptr, T, n, ld, bs, pos0, ratio), "ns_ds41_block_max")
    gpu.sync()
    assert np.array_equal(dbm.read(np.float32).reshape(T, nb), O.ds41_block_max(score, n, bs, pos0, ratio))
    # the candidate blocks: the best K by block maximum (ns_topk), ascending - then the mask, exact
    rng = W.rng(1441, 0)
    cand = np.stack([np.sort(rng.choice(nb, size=K, replace=False)) for _ in range(T)]).astype(np.int32)
    cand[1, 0] = -1                                   # an empty slot
    cand[2, -1] = nb - 1                              # the last, partly filled block
    dcand, dmark = DevBuf.of(gpu, cand), DevBuf(gpu, T * nb)
    check(api, api.ns_ds41_cand_mask(gpu.raw, dsc.ptr, dcand.ptr, dmark.ptr, T, n, ld, K, bs), "ns_ds41_cand_mask")
    gpu.sync()
    assert np.array_equal(dsc.read(np.float32).reshape(T, ld), O.ds41_cand_mask(score.copy(), cand, n, bs))
    # scores over the candidate blocks only
    dq, dw, dk, dcs = DevBuf.of(gpu, q), DevBuf.of(gpu, w), DevBuf.of(gpu, k), DevBuf(gpu, T * K * 8 * 4)
    check(api, api.ns_ds41_idx_score_cand(gpu.raw, dq.ptr, dw.ptr, dk.ptr, dcand.ptr, K, dcs.ptr, T, H, D, n, pos0, ratio), "ns_ds41_idx_score_cand")
    gpu.sync()
    got = dcs.read(np.float32).reshape(T, K * 8)
    want = O.ds41_idx_score_cand(q, w, k, cand, K, T, H, D, n, pos0, ratio)
    assert np.array_equal(np.isneginf(got), np.isneginf(want))
    fin = np.isfinite(want)
    assert np.all(np.abs(got[fin] - want[fin]) <= 1e-3 + 1e-4 * np.abs(want[fin]))
    # compact picks back to positions: exact
    kp = 33
    selc = np.stack([np.sort(rng.choice(K * 8, size=kp, replace=False)) for _ in range(T)]).astype(np.int32)
    cand_ok = np.where(cand < 0, 0, cand).astype(np.int32)
    dselc, dc2, dsel = DevBuf.of(gpu, selc), DevBuf.of(gpu, cand_ok), DevBuf(gpu, T * kp * 4)
    check(api, api.ns_ds41_cand_pos(gpu.raw, dselc.ptr, dc2.ptr, dsel.ptr, T, K, kp, bs), "ns_ds41_cand_pos")
    gpu.sync()
    assert np.array_equal(dsel.read(np.int32).reshape(T, kp), O.ds41_cand_pos(selc, cand_ok, bs))
    assert api.ns_ds41_idx_score_cand(gpu.raw, dq.ptr, dw.ptr, dk.ptr, dcand.ptr, K, dcs.ptr, T, 16, D, n, pos0, ratio) == -1
