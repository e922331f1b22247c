"""The glm5next engine's MLA symbols on the GPU against the CPU oracle (kernels/llm/glm5next/glm.cpp restated), through
the C ABI. Tolerance: |got - want| <= 2e-3 + 1e-2 |want| for the tensor-core path (fp16 q and weights, where the
reference's vector kernels keep fp32: the bar the benchmark sets for fp16 tensor-core numerics); 1e-5 for the fp32 kernel;
bit-exact for the integer / fp16 helper kernels."""
import numpy as np
import pytest

from nextsycl_b200 import DevBuf
from nextsycl_b200 import workloads as W
from nextsycl_b200.core import check
from oracle import oracle as O

pytestmark = pytest.mark.gpu
SCALE = np.float32(1.0 / 16.0)   # glm5next: 1/sqrt(256)


def close(got, want, abs_tol=2e-3, rel_tol=1e-2):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert np.isfinite(got).all()
    d = np.abs(got - want)
    assert np.all(d <= abs_tol + rel_tol * np.abs(want)), float(d.max())


def test_mla_attend_fp32(gpu):
    T, H, L, n = 3, 8, 512, 200
    qa = W.rng(960, 0).standard_normal((T, H, L), dtype=np.float32)
    c = (0.5 * W.rng(960, 1).standard_normal((n, L), dtype=np.float32)).astype(np.float32)
    u = DevBuf(gpu, T * H * L * 4)
    dqa, dc = DevBuf.of(gpu, qa), DevBuf.of(gpu, c)   # named: a buffer lives as long as its Python object
    check(gpu.api, gpu.api.ns_mla_attend(gpu.raw, dqa.ptr, dc.ptr, u.ptr, T, H, L, n - T, SCALE), "ns_mla_attend")
    gpu.sync()
    got = u.read(np.float32).reshape(T, H, L)
    close(got, O.mla_attend_f32(qa, c, T, H, L, n - T, SCALE), abs_tol=1e-4, rel_tol=1e-3)   # fp32 both sides; the order of the sums differs


@pytest.mark.parametrize("T,H,n,q8", [(1, 64, 300, False), (3, 64, 2000, False), (2, 64, 700, True), (12, 16, 900, False)])
def test_mla_attend_sel_dense_and_selected(gpu, T, H, n, q8):
    api = gpu.api
    qa = W.rng(961, 0).standard_normal((T, H, 512), dtype=np.float32)
    lat = (0.5 * W.rng(961, 1).standard_normal((n, 512), dtype=np.float32)).astype(np.float32)
    c16 = lat.astype(np.float16)
    rows8 = O.to_q8row(lat)
    cache = rows8 if q8 else c16
    dq, dc = DevBuf.of(gpu, qa), DevBuf.of(gpu, cache)
    u = DevBuf(gpu, T * H * 512 * 4)
    fn = api.ns_mla_attend_sel_q8 if q8 else api.ns_mla_attend_sel
    pos0 = n - T
    # a selection: K pools per row (4 tokens each), all complete pools before the row; counts differ per row
    K = 40
    rng = W.rng(961, 2)
    sel = np.zeros((T, K), np.int32)
    cnt = np.zeros(T, np.int32)
    for t in range(T):
        pools = (pos0 + t + 1) // 4
        cnt[t] = min(K, pools) - (t % 3)
        sel[t, :cnt[t]] = np.sort(rng.choice(pools, size=cnt[t], replace=False))
    dsel, dcnt = DevBuf.of(gpu, sel), DevBuf.of(gpu, cnt)
    check(api, fn(gpu.raw, dq.ptr, dc.ptr, u.ptr, T, H, 512, pos0, SCALE, dsel.ptr, dcnt.ptr, K), "sel")
    gpu.sync()
    got = u.read(np.float32).reshape(T, H, 512)
    want = O.mla_dec512(qa, cache if q8 else c16.view(np.uint16), T, H, pos0, SCALE, sel=sel, sel_cnt=cnt, K=K, q8=q8)
    close(got, want)
    if not q8:
        # no selection: every earlier token
        check(api, fn(gpu.raw, dq.ptr, dc.ptr, u.ptr, T, H, 512, pos0, SCALE, None, None, 0), "dense")
        gpu.sync()
        close(u.read(np.float32).reshape(T, H, 512), O.mla_dec512(qa, c16.view(np.uint16), T, H, pos0, SCALE))
        # a negative count for one row: that row is dense, the others selected
        cnt2 = cnt.copy()
        cnt2[0] = -1
        dcnt2 = DevBuf.of(gpu, cnt2)
        check(api, fn(gpu.raw, dq.ptr, dc.ptr, u.ptr, T, H, 512, pos0, SCALE, dsel.ptr, dcnt2.ptr, K), "mixed")
        gpu.sync()
        close(u.read(np.float32).reshape(T, H, 512), O.mla_dec512(qa, c16.view(np.uint16), T, H, pos0, SCALE, sel=sel, sel_cnt=cnt2, K=K))


def test_helper_kernels(gpu):
    api = gpu.api
    n = 37
    x = (0.5 * W.rng(962, 0).standard_normal((n, 512), dtype=np.float32)).astype(np.float32)
    # q8 rows: bit-exact against the oracle's encoder
    y = DevBuf(gpu, n * 544)
    dx = DevBuf.of(gpu, x)
    check(api, api.ns_to_q8row(gpu.raw, dx.ptr, y.ptr, n, 512), "to_q8row")
    want8 = O.to_q8row(x)
    assert np.array_equal(y.read(np.uint8).reshape(n, 544), want8)
    # fp32 -> fp16: one rounding
    h = DevBuf(gpu, n * 512 * 2)
    check(api, api.ns_to_f16(gpu.raw, dx.ptr, h.ptr, n * 512), "to_f16")
    assert np.array_equal(h.read(np.float16).reshape(n, 512), x.astype(np.float16))
    # gathers
    idx = np.array([5, 0, 36, 5, 17], np.int32)
    out = DevBuf(gpu, len(idx) * 512 * 2)
    didx0 = DevBuf.of(gpu, idx)
    check(api, api.ns_gather_h(gpu.raw, h.ptr, didx0.ptr, out.ptr, len(idx), 512), "gather_h")
    assert np.array_equal(out.read(np.float16).reshape(len(idx), 512), x.astype(np.float16)[idx])
    check(api, api.ns_gather_q8_h(gpu.raw, y.ptr, didx0.ptr, out.ptr, len(idx), 512), "gather_q8_h")
    scales = want8[:, :32].copy().view(np.float16).astype(np.float32)
    vals = want8[:, 32:].copy().view(np.int8).astype(np.float32).reshape(n, 16, 32)
    deq = (vals * scales[:, :, None]).reshape(n, 512).astype(np.float16)
    assert np.array_equal(out.read(np.float16).reshape(len(idx), 512), deq[idx])
    # cells and the masked softmax
    T, K, pos0, NC = 3, 4, 50, 64
    sel = np.array([[1, 3, 7, 0], [2, 4, 6, 8], [0, 0, 0, 0]], np.int32)
    cnt = np.array([3, 4, -1], np.int32)
    didx, dn = DevBuf(gpu, T * NC * 4), DevBuf(gpu, T * 4)
    dsel, dcnt = DevBuf.of(gpu, sel), DevBuf.of(gpu, cnt)
    check(api, api.ns_mla_cells(gpu.raw, dsel.ptr, dcnt.ptr, T, K, pos0, didx.ptr, dn.ptr, NC), "cells")
    gi, gn = didx.read(np.int32).reshape(T, NC), dn.read(np.int32)
    for t in range(T):
        p = pos0 + t
        tail0 = 4 * ((p + 1) // 4)
        if cnt[t] < 0:
            cells = list(range(p + 1))
        else:
            cells = [4 * sel[t, i // 4] + i % 4 for i in range(4 * cnt[t])] + list(range(tail0, p + 1))
        assert gn[t] == min(len(cells), NC)
        assert list(gi[t, :gn[t]]) == cells[:NC]
    S = W.rng(962, 5).standard_normal((T * 2, NC), dtype=np.float32)
    dS = DevBuf.of(gpu, S)
    check(api, api.ns_softmax_masked(gpu.raw, dS.ptr, T, 2, NC, dn.ptr, np.float32(0.3)), "softmax_masked")
    got = dS.read(np.float32).reshape(T, 2, NC)
    for t in range(T):
        m = gn[t]
        z = S.reshape(T, 2, NC)[t, :, :m].astype(np.float64) * 0.3
        e = np.exp(z - z.max(-1, keepdims=True))
        assert np.allclose(got[t, :, :m], e / e.sum(-1, keepdims=True), atol=1e-6)
        assert not got[t, :, m:].any()


def _gemm(gpu, batch, trans_w, T, N, K, x, ldx, sx, w, ldw, sw, y, ldy, sy, accumulate):
    dx, dw, dy = DevBuf.of(gpu, x), DevBuf.of(gpu, w), DevBuf.of(gpu, y)
    check(gpu.api, gpu.api.ns_gemm_batch_h(gpu.raw, batch, trans_w, T, N, K, dx.ptr, ldx, sx, dw.ptr, ldw, sw, dy.ptr, ldy, sy, accumulate), "ns_gemm_batch_h")
    gpu.sync()
    return dy.read(np.float32)


@pytest.mark.parametrize("batch,trans_w,T,N,K,pad,acc", [
    (32, 1, 64, 2112, 512, 0, 0),     # the engine's score product at its largest cell count (llm/glm5next/src/engine.rs:1925)
    (32, 0, 64, 512, 2112, 0, 0),     # and its value product (:1930)
    (3, 1, 64, 64, 512, 0, 0),        # the smallest padded cell count
    (3, 0, 64, 512, 64, 0, 1),        # accumulating
    (2, 1, 200, 300, 136, 8, 1),      # ragged tiles in every dimension, padded rows, accumulating
    (2, 0, 130, 72, 200, 16, 0),
    (1, 1, 1, 8, 8, 0, 0),            # one row
    (2, 1, 33, 50, 70, 3, 0),         # odd strides: the plain kernel
    (2, 0, 33, 50, 70, 5, 1),
    (2, 1, 5, 7, 0, 0, 1),            # nothing to sum: y stays (accumulate) ...
    (2, 0, 5, 7, 0, 0, 0),            # ... or becomes zero
])
def test_gemm_batch_h(gpu, batch, trans_w, T, N, K, pad, acc):
    """ns_gemm_batch_h against float64 products of the same fp16 values. Tolerance: fp32 accumulation of K products of
    magnitude ~1: |got - want| <= 1e-3 + 1e-4 |want| sqrt(K) is generous; the sums are exact to ~1e-5 in practice."""
    rng = W.rng(963, batch * 1000 + T + N + K + trans_w)
    ldx, ldy = K + pad, N + pad
    wr, wc = (N, K) if trans_w else (K, N)
    ldw = wc + pad
    sx, sw, sy = T * ldx + pad, wr * ldw + pad, T * ldy + pad
    x = (rng.standard_normal(batch * sx, dtype=np.float32)).astype(np.float16).view(np.uint16)
    w = (rng.standard_normal(batch * sw, dtype=np.float32)).astype(np.float16).view(np.uint16)
    y0 = rng.standard_normal(batch * sy, dtype=np.float32)
    got = _gemm(gpu, batch, trans_w, T, N, K, x, ldx, sx, w, ldw, sw, y0.copy(), ldy, sy, acc)
    want = O.gemm_batch_h(batch, trans_w, T, N, K, x, ldx, sx, w, ldw, sw, y0 if acc else None, ldy, sy)
    keep = np.ones(batch * sy, bool)      # everything outside the [T, N] blocks must be untouched
    for b in range(batch):
        g = np.lib.stride_tricks.as_strided(got[b * sy:], (T, N), (ldy * 4, 4))
        d = np.abs(g - want[b])
        assert np.all(d <= 1e-3 + 1e-4 * np.abs(want[b]) * np.sqrt(K)), (b, float(d.max()))
        for t in range(T):
            keep[b * sy + t * ldy: b * sy + t * ldy + N] = False
    assert np.array_equal(got[keep], y0[keep])


def test_prompt_block_as_the_engine_calls_it(gpu):
    """The reference engine's prompt path for one block of rows, call for call (llm/glm5next/src/engine.rs:1908-1938):
    ns_mla_cells, ns_gather_h, ns_to_f16, ns_gemm_batch_h (scores), ns_softmax_masked, ns_to_f16, ns_gemm_batch_h (values) -
    against the oracle's statement of the same attention (glm.cpp's mla_dec<512> numerics restated) and against
    ns_mla_attend_sel, the one-call form."""
    api = gpu.api
    tr, H, L, pos0, K = 5, 64, 512, 300, 16
    NC = -(-(4 * K + 3) // 64) * 64
    rng = W.rng(964, 0)
    qa = rng.standard_normal((tr, H, L), dtype=np.float32)
    c16 = (0.5 * rng.standard_normal((pos0 + tr, L), dtype=np.float32)).astype(np.float16)
    sel = np.stack([np.sort(rng.choice((pos0 + t + 1) // 4, size=K, replace=False)) for t in range(tr)]).astype(np.int32)
    cnt = np.full(tr, K, np.int32)
    scale = np.float32(1 / 16.0)
    dq, dc, dsel, dcnt = DevBuf.of(gpu, qa), DevBuf.of(gpu, c16), DevBuf.of(gpu, sel), DevBuf.of(gpu, cnt)
    didx, dn = DevBuf(gpu, tr * NC * 4), DevBuf(gpu, tr * 4)
    gh, qh = DevBuf(gpu, tr * NC * L * 2), DevBuf(gpu, tr * H * L * 2)
    sb, ph, u = DevBuf(gpu, tr * H * NC * 4), DevBuf(gpu, tr * H * NC * 2), DevBuf(gpu, tr * H * L * 4)
    check(api, api.ns_mla_cells(gpu.raw, dsel.ptr, dcnt.ptr, tr, K, pos0, didx.ptr, dn.ptr, NC), "cells")
    check(api, api.ns_gather_h(gpu.raw, dc.ptr, didx.ptr, gh.ptr, tr * NC, L), "gather")
    check(api, api.ns_to_f16(gpu.raw, dq.ptr, qh.ptr, tr * H * L), "to_f16")
    check(api, api.ns_gemm_batch_h(gpu.raw, tr, 1, H, NC, L, qh.ptr, L, H * L, gh.ptr, L, NC * L, sb.ptr, NC, H * NC, 0), "scores")
    check(api, api.ns_softmax_masked(gpu.raw, sb.ptr, tr, H, NC, dn.ptr, scale), "softmax")
    check(api, api.ns_to_f16(gpu.raw, sb.ptr, ph.ptr, tr * H * NC), "to_f16")
    check(api, api.ns_gemm_batch_h(gpu.raw, tr, 0, H, L, NC, ph.ptr, NC, H * NC, gh.ptr, L, NC * L, u.ptr, L, H * L, 0), "values")
    gpu.sync()
    got = u.read(np.float32).reshape(tr, H, L)
    want = O.mla_dec512(qa, c16.view(np.uint16), tr, H, pos0, scale, sel=sel, sel_cnt=cnt, K=K)
    close(got, want)
    one = DevBuf(gpu, tr * H * L * 4)
    check(api, api.ns_mla_attend_sel(gpu.raw, dq.ptr, dc.ptr, one.ptr, tr, H, L, pos0, scale, dsel.ptr, dcnt.ptr, K), "attend_sel")
    gpu.sync()
    close(one.read(np.float32).reshape(tr, H, L), got)
