"""Absorbed MLA decode on the tensor path against the CPU oracle, through the C ABI.

Tolerance: the benchmark's bar, |got - want| <= 2e-3 + 1e-2 |want|, against the oracle's GEMM-form numerics (q and p rounded
to fp16: llm/deepseek2/src/engine.rs:1204-1224), against the fused kernel's fp32 numerics
(kernels/llm/deepseek2/ds2.cpp:186-235) and against fp64."""
import numpy as np
import pytest

from nextsycl_b200 import DevBuf
from nextsycl_b200 import workloads as W
from oracle import oracle as O

pytestmark = pytest.mark.gpu
ABS, REL = 2e-3, 1e-2
SCALE = float(1.0 / np.sqrt(192.0))


def assert_close(got, want, what, abs_tol=ABS, rel_tol=REL):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    d = np.abs(got - want)
    bad = d > abs_tol + rel_tol * np.abs(want)
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside tolerance, max abs {d.max():.3e}"


def run(gpu, ops, q16, cache, T, H, pos0):
    dq, dc = DevBuf.of(gpu, q16), DevBuf.of(gpu, cache)
    out = DevBuf(gpu, T * H * 512 * 4)
    out.fill(0xFF)
    n = ops.mla_decode_scratch(T, H, pos0)
    sc = DevBuf(gpu, n * 4) if n else None
    if sc is not None:
        sc.fill(0xFF)
    ops.mla_decode(dq, dc, T, H, pos0, SCALE, out, sc)
    gpu.sync()
    return out.read(np.float32).reshape(T, H, 512)


@pytest.mark.parametrize("T,H,n", [(1, 128, 1), (1, 128, 100), (1, 16, 1000), (3, 128, 333), (1, 128, 5000), (2, 200, 700), (1, 128, 4096)])
def test_mla_decode_matches_oracle(gpu, ops, T, H, n):
    q = W.normal_f16(940, 0, (T, H, 576))
    cache = W.normal_f16(940, 1, (n, 576), 0.5)
    got = run(gpu, ops, q, cache, T, H, n - T)
    qf, cb = q.astype(np.float32), cache.view(np.uint16)
    assert_close(got, O.mla_gemm(qf, cb, T, H, 512, 64, n - T, np.float32(SCALE)), "vs GEMM-form numerics")
    assert_close(got, O.mla_fused(qf, cb, T, H, 512, 64, n - T, np.float32(SCALE)), "vs fused-kernel numerics")
    assert_close(got, O.mla_exact(qf, cb, T, H, 512, 64, n - T, SCALE), "vs fp64")


def test_ds2_whole_decode(gpu, ops):
    """ns_ds2_mla_decode: absorb, latent attention, un-absorb, against the same three stages in numpy + the oracle."""
    T, H, n = 2, 128, 900
    q = W.rng(941, 0).standard_normal((T, H, 192), dtype=np.float32)
    kb = W.normal_f16(941, 1, (H, 512, 128), 0.1)
    vb = W.normal_f16(941, 2, (H, 128, 512), 0.1)
    cache = W.normal_f16(941, 3, (n, 576), 0.5)
    out = DevBuf(gpu, T * H * 128 * 4)
    ops.ds2_mla_decode(DevBuf.of(gpu, q), DevBuf.of(gpu, kb), DevBuf.of(gpu, vb), DevBuf.of(gpu, cache), out, T, H, n - T, SCALE)
    gpu.sync()
    got = out.read(np.float32).reshape(T, H, 128)
    # q~ = k_b q_nope (fp32), then [q~ | q_pe] as the oracle's input (it rounds it to fp16 as the kernel does)
    qa = np.einsum("hrc,thc->thr", kb.astype(np.float32), q[:, :, :128]).astype(np.float32)
    qfull = np.ascontiguousarray(np.concatenate([qa, q[:, :, 128:]], axis=2))
    u = O.mla_gemm(qfull, cache.view(np.uint16), T, H, 512, 64, n - T, np.float32(SCALE))
    want = np.einsum("hvl,thl->thv", vb.astype(np.float64), u.astype(np.float64))
    assert_close(got, want, "whole decode")


@pytest.mark.parametrize("n", [32768, 131072])
def test_config_3_full_size(gpu, ops, n):
    """benchmark configuration 3: 128 heads, latent cache ~N(0, 0.5), query ~N(0, 1), scale 1/sqrt(192). All 128 heads run on the
    GPU; the oracle checks 16 of them: the first and last head of each run of 32 (a softmax warp's 32 tensor-memory lanes;
    heads 0-63 are the pair's first CTA, 64-127 its second) and 8 more in between; every checked row spans all 512 output
    columns, i.e. both lane halves of the accumulator and both threads of a head."""
    T, H = 1, 128
    q = W.normal_f16(3, 0, (T, H, 576))
    cache = W.normal_f16(3, 1, (n, 576), 0.5)
    got = run(gpu, ops, q, cache, T, H, n - 1)
    heads = [0, 31, 32, 63, 64, 95, 96, 127, 7, 16, 45, 50, 77, 88, 101, 120]
    qs = np.ascontiguousarray(q[:, heads].astype(np.float32))
    assert_close(got[:, heads], O.mla_gemm(qs, cache.view(np.uint16), T, len(heads), 512, 64, n - 1, np.float32(SCALE)), f"config 3, heads {heads}")
    assert np.isfinite(got).all()


def test_a_verify_row_equals_the_one_row_pass(gpu, ops):
    """At decode widths a row's key splits come from its own cell count alone: row t of a pass of T rows is the one-row
    pass at its position, bit for bit (the property kernels/llm/deepseek41/silo/attn.cpp:316-319 states for its decode)."""
    T, H, n = 4, 128, 9000
    q = W.normal_f16(941, 0, (T, H, 576))
    cache = W.normal_f16(941, 1, (n, 576), 0.5)
    whole = run(gpu, ops, q, cache, T, H, n - T)
    for t in range(T):
        alone = run(gpu, ops, q[t:t + 1].copy(), cache, 1, H, n - T + t)
        assert np.array_equal(alone[0], whole[t])
    # more rows than a decode pass: one split size for the pass; still within tolerance of the oracle
    T = 12
    q = W.normal_f16(941, 2, (T, H, 576))
    got = run(gpu, ops, q, cache, T, H, n - T)
    assert_close(got, O.mla_gemm(q.astype(np.float32), cache.view(np.uint16), T, H, 512, 64, n - T, np.float32(SCALE)), "12 rows")


def _q6k_blocks(rng, nrows, cols=512):
    """Random Q6_K rows: any bytes are a valid block; d a small half so the values are O(0.1)."""
    nb = cols // 256
    blk = rng.integers(0, 256, size=(nrows, nb, 210), dtype=np.uint8)
    blk[:, :, 192:208] = rng.integers(-32, 32, size=(nrows, nb, 16)).astype(np.int8).view(np.uint8)
    d = (rng.uniform(2e-4, 6e-4, size=(nrows, nb)).astype(np.float32) * rng.choice([-1.0, 1.0], size=(nrows, nb)).astype(np.float32)).astype(np.float16)
    blk[:, :, 208:210] = d.view(np.uint8).reshape(nrows, nb, 2)
    return np.ascontiguousarray(blk.reshape(nrows, nb * 210))


def _run_q6k(gpu, q, kvb, cache, T, H, pos0):
    from nextsycl_b200.core import check
    dq, dk, dc = DevBuf.of(gpu, q), DevBuf.of(gpu, kvb), DevBuf.of(gpu, cache)
    out = DevBuf(gpu, T * H * 128 * 4)
    out.fill(0xFF)
    check(gpu.api, gpu.api.need("ns_ds2_mla_decode_q6k")(gpu.raw, dq.ptr, dk.ptr, dc.ptr, out.ptr, T, H, pos0, np.float32(SCALE)), "ns_ds2_mla_decode_q6k")
    gpu.sync()
    return out.read(np.float32).reshape(T, H, 128)


def test_ds2_q6k_decoder_bit_exact(gpu):
    """The Q6_K reader of ns_ds2_mla_decode_q6k, read out exactly: one cell whose latent is a one-hot column c, under a zero
    query (score 0, weight exactly 1, sum exactly 1), makes the attention's u that one-hot, so out[h][r] = v_r[c] as the
    decoder produced it - equal to the oracle's decode of the same blocks (kernels/llm/deepseek2/ds2.cpp:123-137) exactly,
    for columns in every (block, half, quarter, scale half)."""
    H = 4
    rng = W.rng(945, 0)
    kvb = _q6k_blocks(rng, H * 256)
    vals = O.q6k_rows(kvb, H * 256, 512).reshape(H, 256, 512)
    q = np.zeros((1, H, 192), np.float32)
    cols = [256 * b + 128 * n + 32 * g + l for b in (0, 1) for n in (0, 1) for g in (0, 1, 2, 3) for l in (0, 15, 16, 31)][::3] + [0, 511]
    for c in cols:
        cache = np.zeros((1, 576), np.float16)
        cache[0, c] = 1.0
        got = _run_q6k(gpu, q, kvb, cache, 1, H, 0)
        assert np.array_equal(got[0], vals[:, 128:, c]), c      # equal as values (a zero code times a negative scale is -0 in the decoder, +0 once summed)


@pytest.mark.parametrize("T,H,n", [(1, 128, 700), (3, 16, 2500)])
def test_ds2_q6k_whole_decode(gpu, T, H, n):
    """ns_ds2_mla_decode_q6k against the same three stages on the CPU: kv_b expanded by the oracle's Q6_K reader, q~ = sum_i
    q_nope[i] k_i, the oracle's latent attention (GEMM-form numerics), out = v . u."""
    rng = W.rng(946, T)
    kvb = _q6k_blocks(rng, H * 256)
    vals = O.q6k_rows(kvb, H * 256, 512).reshape(H, 256, 512).astype(np.float64)
    q = rng.standard_normal((T, H, 192), dtype=np.float32)
    cache = W.normal_f16(946, 3, (n, 576), 0.5)
    got = _run_q6k(gpu, q, kvb, cache, T, H, n - T)
    qa = np.einsum("thi,hic->thc", q[:, :, :128].astype(np.float64), vals[:, :128]).astype(np.float32)
    qfull = np.ascontiguousarray(np.concatenate([qa, q[:, :, 128:]], axis=2))
    u = O.mla_gemm(qfull, cache.view(np.uint16), T, H, 512, 64, n - T, np.float32(SCALE))
    want = np.einsum("hrc,thc->thr", vals[:, 128:], u.astype(np.float64))
    assert_close(got, want, "q6k whole decode")
