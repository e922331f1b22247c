"""The CPU oracle checked on the CPU: against an independent numpy statement of causal softmax attention (the form
the reference's own Python models use, reference/ricursive-65b/ripple_ref.py:279-294), against its fp64 mode, and
against the committed known-answer file. Parity with the reference itself is unpinned (no golden vectors exist for
attention in the reference tree); these tests pin the oracle to the mathematics and to itself."""
import os

import numpy as np
import pytest

from nextsycl_b200 import workloads as W
from oracle import oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "oracle_kat.npz")
# the benchmark's tolerance for fp16 tensor-core numerics against exact arithmetic
ABS, REL = 2e-3, 1e-2


def numpy_attention(q, k, v, T, Hq, Hkv, D, p0):
    G = Hq // Hkv
    out = np.zeros((T, Hq, D))
    for t in range(T):
        n = p0 + t + 1
        for h in range(Hq):
            s = (k[h // G, :n].astype(np.float64) @ q[t, h * D:(h + 1) * D].astype(np.float64)) / np.sqrt(D)
            p = np.exp(s - s.max())
            p /= p.sum()
            out[t, h] = p @ v[h // G, :n].astype(np.float64)
    return out.reshape(T, Hq * D)


def close(a, b, abs_tol=ABS, rel_tol=REL):
    d = np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64))
    return bool(np.all(d <= abs_tol + rel_tol * np.abs(b)))


@pytest.mark.parametrize("T,Hq,Hkv,D,kv", [(1, 8, 2, 128, 1), (5, 8, 2, 128, 37), (3, 12, 2, 256, 100), (9, 16, 4, 128, 64), (2, 64, 8, 128, 500)])
def test_gqa_modes_agree_with_numpy(T, Hq, Hkv, D, kv):
    q, k, v, p0 = W.gqa_case(910, T, Hq, Hkv, D, kv)
    qf, kb, vb = q.astype(np.float32), k.view(np.uint16), v.view(np.uint16)
    ref = numpy_attention(qf, k, v, T, Hq, Hkv, D, p0)
    ex = O.attn_exact(qf, kb, vb, T, Hq, Hkv, D, D, kv, p0, 1 / np.sqrt(D))
    assert np.abs(ex - ref).max() < 1e-12
    assert np.abs(O.gqa_plain(qf, kb, vb, T, Hq, Hkv, D, kv, p0) - ex).max() < 5e-6
    assert close(O.gqa_flash_prefill(qf, kb, vb, T, Hq, Hkv, D, kv, p0), ex)
    assert close(O.attn_tc(qf, kb, vb, T, Hq, Hkv, D, D, kv, p0, 1 / np.sqrt(D), 0), ex)
    if T <= 8:
        assert close(O.gqa_flash_decode(qf, kb, vb, T, Hq, Hkv, D, kv, p0), ex)


def test_flash_decode_splits_match_the_reference_formula():
    # kernels/llm/qwen35/silo/attn.cpp:325-331: ~512 work-groups, multiples of 64 keys
    assert O.flash_split(32768, 8) == 512 and O.flash_splits(32768, 8) == 64
    assert O.flash_split(262144, 4) == 2048 and O.flash_splits(262144, 4) == 128
    assert O.flash_split(100, 8) == 64 and O.flash_splits(100, 8) == 2
    assert O.flash_splits(64, 8) == 1


def test_flash_decode_row_does_not_depend_on_its_pass():
    """A verify row equals the one-row pass at its position, bit for bit (kernels/llm/qwen35/silo/attn.cpp:100-104)."""
    T, Hq, Hkv, D, kv = 4, 8, 2, 128, 700
    q, k, v, p0 = W.gqa_case(911, T, Hq, Hkv, D, kv)
    qf, kb, vb = q.astype(np.float32), k.view(np.uint16), v.view(np.uint16)
    all_rows = O.gqa_flash_decode(qf, kb, vb, T, Hq, Hkv, D, kv, p0)
    for t in range(T):
        one = O.gqa_flash_decode(qf[t:t + 1].copy(), kb, vb, 1, Hq, Hkv, D, kv, p0 + t)
        assert np.array_equal(one[0], all_rows[t])


def test_empty_and_single_key():
    # one key: the output is that key's value row
    q, k, v, p0 = W.gqa_case(912, 1, 4, 1, 128, 1)
    out = O.gqa_flash_prefill(q.astype(np.float32), k.view(np.uint16), v.view(np.uint16), 1, 4, 1, 128, 1, 0)
    assert np.allclose(out.reshape(4, 128), np.broadcast_to(v[0, 0].astype(np.float32), (4, 128)), atol=1e-3)


def test_bf16_generic_attention_192_128():
    """The shape the reference has no kernel for (bf16, 192-wide keys, 128-wide values): tensor-core numerics against fp64."""
    T, H, kv = 6, 4, 90
    q = O.from_bf16_bits(W.normal_bf16_bits(913, 0, (T, H * 192)))
    kb = W.normal_bf16_bits(913, 1, (H, kv, 192))
    vb = W.normal_bf16_bits(913, 2, (H, kv, 128))
    sc = 1 / np.sqrt(192.0)
    ex = O.attn_exact(q, kb, vb, T, H, H, 192, 128, kv, kv - T, sc, kind=1)
    tc = O.attn_tc(q, kb, vb, T, H, H, 192, 128, kv, kv - T, np.float32(sc), kind=1)
    # bf16 weights carry 8 mantissa bits: the band is wider than fp16's
    assert np.abs(tc - ex).max() < 2e-2


@pytest.mark.parametrize("T,H,n", [(1, 4, 1), (1, 16, 130), (3, 8, 777)])
def test_mla_modes(T, H, n):
    q = W.rng(914, 0).standard_normal((T, H, 576), dtype=np.float32)
    c = W.normal_f16(914, 1, (n, 576), 0.5).view(np.uint16)
    sc = 1 / np.sqrt(192.0)
    ex = O.mla_exact(q, c, T, H, 512, 64, n - T, sc)
    assert np.abs(O.mla_fused(q, c, T, H, 512, 64, n - T, np.float32(sc)) - ex).max() < 5e-6
    assert close(O.mla_gemm(q, c, T, H, 512, 64, n - T, np.float32(sc)), ex)


def test_mla_glm_kernels():
    T, H, n = 2, 4, 300
    qa = W.rng(915, 0).standard_normal((T, H, 512), dtype=np.float32)
    c32 = (0.5 * W.rng(915, 1).standard_normal((n, 512), dtype=np.float32)).astype(np.float16)
    sc = np.float32(1 / 16.0)
    dense = O.mla_attend_f32(qa, c32.astype(np.float32), T, H, 512, n - T, sc)
    dec = O.mla_dec512(qa, c32.view(np.uint16), T, H, n - T, sc)
    assert np.abs(dense - dec).max() < 5e-6
    # q8 rows: 544 bytes, values within half a quantisation step of the fp32 source
    x = c32.astype(np.float32)
    rows = O.to_q8row(x)
    assert rows.shape == (n, 544)
    scales = rows[:, :32].copy().view(np.float16).astype(np.float32)          # [n, 16]
    vals = rows[:, 32:].copy().view(np.int8).astype(np.float32).reshape(n, 16, 32)
    deq = (vals * scales[:, :, None]).reshape(n, 512)
    assert np.all(np.abs(deq - x) <= 0.5 * np.repeat(scales, 32, axis=1) + 1e-6)
    dq8 = O.mla_dec512(qa, rows, T, H, n - T, sc, q8=True)
    assert np.abs(dq8 - dec).max() < 2e-2
    # a selection: pools 0 and 5 (4 tokens each) plus the incomplete pool
    sel = np.array([[0, 5], [0, 5]], np.int32)
    cnt = np.array([2, 2], np.int32)
    s = O.mla_dec512(qa, c32.view(np.uint16), T, H, n - T, sc, sel=sel, sel_cnt=cnt, K=2)
    assert np.isfinite(s).all() and np.abs(s - dec).max() > 0


def test_merge_with_and_without_sink():
    rng = np.random.default_rng(3)
    rows, ns, D = 5, 3, 16
    part = rng.standard_normal((rows, ns, D + 2)).astype(np.float32)
    part[:, :, D + 1] = np.abs(part[:, :, D + 1]) + 0.1
    out = O.merge(part, rows, ns, D, D + 2)
    m, l, o = part[:, :, D].astype(np.float64), part[:, :, D + 1].astype(np.float64), part[:, :, :D].astype(np.float64)
    w = np.exp2(m - m.max(1, keepdims=True))
    ref = (o * w[:, :, None]).sum(1) / (l * w).sum(1)[:, None]
    assert np.allclose(out, ref, rtol=1e-5, atol=1e-6)
    sinks = rng.standard_normal(rows).astype(np.float32)
    outs = O.merge(part, rows, ns, D, D + 2, sinks)
    mx = np.maximum(m.max(1), sinks * np.log2(np.e))
    w = np.exp2(m - mx[:, None])
    ref = (o * w[:, :, None]).sum(1) / ((l * w).sum(1) + np.exp2(sinks * np.log2(np.e) - mx))[:, None]
    assert np.allclose(outs, ref, rtol=1e-5, atol=1e-6)


def test_kv_store_layout():
    T, Hkv, D, cap, p0 = 3, 2, 128, 10, 4
    k = W.rng(916, 0).standard_normal((T, Hkv * D), dtype=np.float32)
    v = W.rng(916, 1).standard_normal((T, Hkv * D), dtype=np.float32)
    kc = np.zeros((Hkv, cap, D), np.uint16)
    vc = np.zeros((Hkv, cap, D), np.uint16)
    O.kv_store(k, v, T, Hkv, D, cap, p0, kc, vc)
    assert np.array_equal(kc[:, p0:p0 + T].view(np.float16), k.reshape(T, Hkv, D).transpose(1, 0, 2).astype(np.float16))
    assert not kc[:, :p0].any() and not vc[:, p0 + T:].any()


def test_known_answers():
    g = np.load(GOLD)
    for name in ("gqa_a", "gqa_b", "gqa_c", "gqa_d"):
        T, Hq, Hkv, D, cap, p0 = [int(x) for x in g[name + "_meta"]]
        qf = g[name + "_q"].astype(np.float32)
        kb, vb = g[name + "_k"].view(np.uint16), g[name + "_v"].view(np.uint16)
        assert np.allclose(O.gqa_flash_prefill(qf, kb, vb, T, Hq, Hkv, D, cap, p0), g[name + "_flash"], rtol=0, atol=1e-6)
        assert np.allclose(O.gqa_plain(qf, kb, vb, T, Hq, Hkv, D, cap, p0), g[name + "_plain"], rtol=0, atol=1e-6)
        if T <= 8:
            assert np.allclose(O.gqa_flash_decode(qf, kb, vb, T, Hq, Hkv, D, cap, p0), g[name + "_flash_decode"], rtol=0, atol=1e-6)
    for name in ("mla_a", "mla_b"):
        T, H, pos0 = [int(x) for x in g[name + "_meta"]]
        sc = np.float32(1.0 / np.sqrt(192.0))
        c = g[name + "_c"].view(np.uint16)
        assert np.allclose(O.mla_fused(g[name + "_q"], c, T, H, 512, 64, pos0, sc), g[name + "_fused"], rtol=0, atol=1e-6)
        assert np.allclose(O.mla_gemm(g[name + "_q"], c, T, H, 512, 64, pos0, sc), g[name + "_gemm"], rtol=0, atol=1e-6)


def ds41_numpy(q, raw, R, comp, ratio, sel, K, sinks, T, H, pos0, window, scale):
    """The attention of reference/deepseek41/ds41ref.py:241-250 (scores, the maximum with the sink, exp, a denominator that
    also holds exp(sink - m)) over the cells kernels/llm/deepseek41/silo/attn.cpp:83-94 lists for a row, in float64."""
    out = np.zeros((T, H, 512))
    for t in range(T):
        p = pos0 + t
        n_raw = min(window, p + 1)
        cells = [raw[(p - n_raw + 1 + i) % R] for i in range(n_raw)]
        vis = (p + 1) // ratio if comp is not None else 0
        if sel is not None and vis > K:
            cells += [comp[j] for j in sel[t]]
        else:
            cells += [comp[j] for j in range(vis)]
        kk = np.stack(cells).view(np.float16).astype(np.float64)
        s = q[t].astype(np.float64) @ kk.T * scale
        m = np.maximum(s.max(-1), sinks)
        pr = np.exp(s - m[:, None])
        out[t] = (pr @ kk) / (pr.sum(-1) + np.exp(sinks - m))[:, None]
    return out


@pytest.mark.parametrize("T,pos0,window,R,ncomp,ratio,K", [(1, 5, 8, 8, 0, 4, 0), (1, 300, 128, 128, 75, 4, 0), (2, 299, 64, 96, 75, 4, 16),
                                                           (3, 0, 16, 16, 0, 4, 0)])
def test_ds41_attend_both_numerics(T, pos0, window, R, ncomp, ratio, K):
    H = 8
    rng = W.rng(970, T * 1000 + pos0)
    q = rng.standard_normal((T, H, 512), dtype=np.float32)
    raw = O.to_f16_bits(0.5 * rng.standard_normal((R, 512), dtype=np.float32))
    comp = O.to_f16_bits(0.5 * rng.standard_normal((ncomp, 512), dtype=np.float32)) if ncomp else None
    sel = None
    if K:
        sel = np.stack([np.sort(rng.choice((pos0 + t + 1) // ratio, size=K, replace=False)) for t in range(T)]).astype(np.int32)
    sinks = rng.standard_normal(H).astype(np.float32)
    scale = np.float32(512 ** -0.5)
    want = ds41_numpy(q, raw, R, comp, ratio, sel, K, sinks, T, H, pos0, window, scale)
    vec = O.ds41_attend(q, raw, R, comp, ratio, sel, K, sinks, T, H, pos0, window, scale, mode=0)
    xmx = O.ds41_attend(q, raw, R, comp, ratio, sel, K, sinks, T, H, pos0, window, scale, mode=1)
    assert np.abs(vec - want).max() < 1e-5
    assert close(xmx, want)
    # a sink far below every score leaves a plain softmax; far above, it takes the whole denominator
    low = O.ds41_attend(q, raw, R, comp, ratio, sel, K, np.full(H, -1e4, np.float32), T, H, pos0, window, scale, mode=1)
    high = O.ds41_attend(q, raw, R, comp, ratio, sel, K, np.full(H, 1e4, np.float32), T, H, pos0, window, scale, mode=1)
    assert close(low, ds41_numpy(q, raw, R, comp, ratio, sel, K, np.full(H, -1e4), T, H, pos0, window, scale))
    assert np.abs(high).max() < 1e-30


@pytest.mark.parametrize("kt", [1, 2])
def test_quantised_cache_rows(kt):
    """kernels/llm/qwen35/q35.cpp:281-326 and silo/attn.cpp:49-78 restated in numpy: blocks of 32, llama.cpp's q8_0 / q4_0
    with the scales behind the values; the reader's value is half(q * d)."""
    T, Hkv, cap, p0 = 5, 2, 16, 3
    rng = W.rng(975, kt)
    k = rng.standard_normal((T, Hkv * 256), dtype=np.float32)
    v = (3.0 * rng.standard_normal((T, Hkv * 256), dtype=np.float32)).astype(np.float32)
    k[0, :32] = 0.0                      # an all-zero block: scale 0, values 0 (q8_0) or 8 (q4_0)
    k[1, 32:64] = np.float32(-2.5)       # a constant block
    rb = O.q_row_bytes(kt)
    kc = np.zeros((Hkv, cap, rb), np.uint8)
    vc = np.zeros((Hkv, cap, rb), np.uint8)
    O.kv_store_q(kt, k, v, T, Hkv, cap, p0, kc, vc)
    for src, cache in ((k, kc), (v, vc)):
        x = src.reshape(T, Hkv, 8, 32)
        for t in range(T):
            for h in range(Hkv):
                row = cache[h, p0 + t]
                for b in range(8):
                    xb = x[t, h, b]
                    if kt == 1:
                        d = np.float32(np.abs(xb).max()) / np.float32(127.0)
                        inv = np.float32(1.0) / d if d != 0 else np.float32(0.0)
                        y = xb * inv
                        want = (np.sign(y) * np.floor(np.abs(y) + np.float32(0.5))).astype(np.int8)   # round half away from zero
                        assert np.array_equal(row[b * 32:(b + 1) * 32].view(np.int8), want)
                        assert row[256 + 2 * b:258 + 2 * b].view(np.float16)[0] == np.float16(d)
                    else:
                        m = xb[np.argmax(np.abs(xb))] if np.abs(xb).max() > 0 else np.float32(0.0)
                        d = np.float32(m) / np.float32(-8.0)
                        inv = np.float32(1.0) / d if d != 0 else np.float32(0.0)
                        qv = np.minimum(15, (xb * inv + np.float32(8.5)).astype(np.int32))
                        want = (qv[:16] | (qv[16:] << 4)).astype(np.uint8)
                        assert np.array_equal(row[b * 16:(b + 1) * 16], want)
                        assert row[128 + 2 * b:130 + 2 * b].view(np.float16)[0] == np.float16(d)
        deq = O.kv_dequant(kt, cache, Hkv, cap, cap).view(np.float16).astype(np.float32)
        back = deq[:, p0:p0 + T].transpose(1, 0, 2).reshape(T, Hkv, 8, 32)
        # a block is within half a step of its scale (q8_0), a step (q4_0: the codes stop at 15), plus the fp16 rounding of the scale
        step = np.abs(x).max(-1, keepdims=True) / (127.0 if kt == 1 else 8.0)
        assert np.all(np.abs(back - x) <= (0.51 if kt == 1 else 1.01) * step + 1e-3 * np.abs(x).max())
    assert np.all(kc[:, :p0] == 0) and np.all(kc[:, p0 + T:] == 0)


def test_fwht32_is_its_own_inverse():
    x = W.rng(976, 0).standard_normal((7, 256), dtype=np.float32)
    y = O.fwht32(x.copy())
    h = np.array([[(-1) ** bin(i & j).count("1") for j in range(32)] for i in range(32)], np.float64) / np.sqrt(32.0)
    assert np.allclose(y.reshape(7, 8, 32), x.reshape(7, 8, 32).astype(np.float64) @ h, atol=1e-5)
    assert np.allclose(O.fwht32(y.copy()), x, atol=1e-5)


def test_qk_norm_rope_against_numpy():
    """kernels/llm/qwen35/q35.cpp:220-254 in float64 numpy: RMS norm, then rotate-half over the first n_rot features."""
    T, H, D, n_rot, theta, eps, p0 = 5, 3, 128, 64, 1e6, 1e-6, 1000
    x = W.rng(977, 0).standard_normal((T, H * D), dtype=np.float32)
    w = (1.0 + 0.1 * W.rng(977, 1).standard_normal(D, dtype=np.float32)).astype(np.float32)
    y = O.qk_norm_rope(x, T, H, D, w, eps, n_rot, theta, p0)
    xd = x.astype(np.float64).reshape(T, H, D)
    v = xd / np.sqrt((xd ** 2).mean(-1, keepdims=True) + eps) * w
    k = np.arange(n_rot // 2)
    ang = (p0 + np.arange(T))[:, None] * theta ** (-2.0 * k / n_rot)
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    want = v.copy()
    want[..., :n_rot // 2] = v[..., :n_rot // 2] * c - v[..., n_rot // 2:n_rot] * s
    want[..., n_rot // 2:n_rot] = v[..., n_rot // 2:n_rot] * c + v[..., :n_rot // 2] * s
    assert np.abs(y.reshape(T, H, D) - want).max() < 2e-3      # fp32 angles at position 1,000: ~1e-4 rad
    # positions given per row, all three equal: the same as the plain form at that position
    pos3 = np.repeat((p0 + np.arange(T, dtype=np.int32))[:, None], 3, 1).copy()
    assert np.array_equal(O.qk_norm_rope(x, T, H, D, w, eps, n_rot, theta, 0, pos3, (11, 11, 10)), y)
    # without weights: the rotation alone keeps each pair's length
    r = O.qk_norm_rope(x, T, H, D, None, 0.0, n_rot, theta, p0).reshape(T, H, D)
    xr = x.reshape(T, H, D)
    assert np.allclose(r[..., :32] ** 2 + r[..., 32:64] ** 2, xr[..., :32] ** 2 + xr[..., 32:64] ** 2, rtol=1e-4, atol=1e-6)
    assert np.array_equal(r[..., n_rot:], xr[..., n_rot:])


def test_topk_selection_rule():
    """kernels/llm/glm5next/glm.cpp:940-1015: the K highest a row, ties at the K-th value to the lowest positions, ascending."""
    rng = W.rng(978, 0)
    T, n, ld, K = 3, 500, 512, 37
    score = np.full((T, ld), 123.0, np.float32)
    score[:, :n] = np.round(rng.standard_normal((T, n), dtype=np.float32) * 4) / 4      # many ties
    score[1, :50] = -np.inf
    sel = O.topk(score, n, K)
    for r in range(T):
        order = np.lexsort((np.arange(n), -score[r, :n].astype(np.float64)))           # value descending, then position ascending
        assert np.array_equal(sel[r], np.sort(order[:K]))
    assert np.array_equal(O.topk(score, 20, 30)[0, :20], np.arange(20)) and np.all(O.topk(score, 20, 30)[0, 20:] == -1)


def test_ds41_indexer_steps():
    """kernels/llm/deepseek41/silo/k41.cpp:352-483 against numpy: scores, block maxima, candidate mask, compact picks."""
    T, H, D, n, pos0, ratio = 3, 32, 128, 100, 390, 4          # rows see (391, 392, 393) // 4 = 97, 98, 98 keys
    ld = 104
    rng = W.rng(979, 0)
    q = rng.standard_normal((T, H, D), dtype=np.float32)
    w = rng.standard_normal((T, H), dtype=np.float32)
    k = O.to_f16_bits(rng.standard_normal((n, D), dtype=np.float32))
    kf = k.view(np.float16).astype(np.float64)
    for half_q in (False, True):
        qq = (q.astype(np.float16) if half_q else q).astype(np.float64)
        want = np.einsum("th,thj->tj", w.astype(np.float64), np.maximum(np.einsum("thd,jd->thj", qq, kf), 0.0))
        got = O.ds41_idx_score(q, w, k, T, H, D, n, ld, pos0, ratio, half_q)
        for t in range(T):
            nv = min(n, (pos0 + t + 1) // ratio)
            assert np.allclose(got[t, :nv], want[t, :nv], rtol=1e-4, atol=1e-3) and np.all(np.isneginf(got[t, nv:]))
    score = O.ds41_idx_score(q, w, k, T, H, D, n, ld, pos0, ratio)
    bmax = O.ds41_block_max(score, n, 8, pos0, ratio)
    assert bmax.shape == (T, 13) and np.isposinf(bmax[0, 96 // 8]) and np.isposinf(bmax[1, 97 // 8])
    assert bmax[0, 3] == score[0, 24:32].max()
    cand = np.array([[0, 5, 12, -1], [1, 2, 3, 40], [12, 11, 10, 9]], np.int32)
    masked = O.ds41_cand_mask(score.copy(), cand, n, 8)
    assert np.array_equal(masked[0, 40:48], score[0, 40:48]) and np.all(np.isneginf(masked[0, 8:40]))
    sc = O.ds41_idx_score_cand(q, w, k, cand, 4, T, H, D, n, pos0, ratio)
    assert np.array_equal(sc[0, 8:16], score[0, 40:48]) and np.all(np.isneginf(sc[0, 24:32])) and np.all(np.isneginf(sc[1, 24:32]))
    selc = np.array([[0, 9, 17], [8, 1, 2], [31, 0, 7]], np.int32)
    sel = O.ds41_cand_pos(selc, cand, 8)
    assert np.array_equal(sel[0], [0, 41, 97]) and np.array_equal(sel[2], [9 * 8 + 7, 96, 103])


# ---- the oracle pinned to values produced by the reference's own CPU code ------------------------------------------------
# tests/golden/ds41ref_fixtures.npz was written by tests/golden/make_ref_fixtures.py, which imports
# reference/deepseek41/ds41ref.py and runs its functions and its Ref.attention as written (seeded weights through a stub of
# Ref.w). The oracle functions below are therefore held to reference output, not to a restatement.
import ref_fixtures as RF  # noqa: E402


def test_ref_pin_e4m3_simulation_bit_exact():
    """ds41ref.fp8_sim (:42-52) == the simulation inside orc_ds41_att_post (no rotation: rd 0), bit for bit, ties included."""
    g = RF.load()
    x = g["fp8_in"].reshape(1, 1, 512).copy()
    O.ds41_att_post(x, 1, 1, 512, 0, 0, (10000.0, 1.0, 0.0, 1.0, 0.0, 0.0))
    assert np.array_equal(x.reshape(16, 32).view(np.uint32), g["fp8_out"].view(np.uint32))


def test_ref_pin_rms_norm():
    """ds41ref.rms (:88-90) against the oracle's per-head RMS norm (no rotation: n_rot 0)."""
    g = RF.load()
    y = O.qk_norm_rope(g["rms_in"], 5, 1, 96, g["rms_w"], 1e-6, 0, 10000.0)
    assert np.allclose(y, g["rms_out"], rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize("name", ["plain", "yarn"])
def test_ref_pin_rotation(name):
    """ds41ref.freqs + rope (:93-113) against the oracle's YaRN rotation with the engine's parameter mapping. The reference
    takes the angle in float64, the kernels in float32: a value may turn by one unit in the last place of the angle."""
    g = RF.load()
    y = RF.yarn_of(g[f"rope_{name}_cfg"])
    for i, p in enumerate(g[f"rope_{name}_pos"]):
        x = g[f"rope_{name}_in"][i].copy().reshape(-1)          # 3 heads of 64
        O.ds2_rope(x, 1, 3, 192, 64, 0, 64, int(p), *y)
        want = g[f"rope_{name}_out"][i]
        tol = 2e-6 + float(p) * 2.0 ** -23 * float(np.abs(want).max()) * 1.5
        assert np.abs(x.reshape(3, 64) - want).max() <= tol, (name, int(p))


@pytest.mark.parametrize("L", [0, 1])
def test_ref_pin_kv_post_and_att_post_bit_exact(L):
    """Either side of the attention, as Ref.attention runs it (:187-191 norm, rotation, simulation of the window keys;
    :251-253 the output's rotation undone and simulated): the oracle's results equal the reference's bit for bit."""
    d = RF.layer(RF.load(), L)
    kv = d["kv_in"].copy()
    ring = np.zeros((64, d["HD"]), np.uint16)
    O.ds41_kv_post(kv, d["kv_w"], d["T"], d["HD"], 1e-6, d["RD"], 0, d["yarn"], ring, 64)
    assert np.array_equal(kv.astype(np.float16).view(np.uint16), d["kv_f16"])
    assert np.array_equal(kv, d["kv_f16"].view(np.float16).astype(np.float32))
    assert np.array_equal(ring[:d["T"]], d["kv_f16"])
    for i, r in enumerate(d["qrows"]):
        x = d["attn_out"][i:i + 1].copy()
        O.ds41_att_post(x, 1, d["H"], d["HD"], d["RD"], int(r), d["yarn"])
        assert np.array_equal(x[0], d["att_post_out"][i]), (L, int(r))


@pytest.mark.parametrize("L", [0, 1])
def test_ref_pin_attention_with_sinks(L):
    """Ref.attention's scores, sink and weighted sum (:236-250) over the window and the compressed keys it picks: the
    oracle's vector-kernel numerics (fp32 throughout) to 1e-5, its XMX numerics (fp16 q and weights) within the path's bar."""
    d = RF.layer(RF.load(), L)
    scale = np.float32(d["HD"] ** -0.5)
    for i in range(len(d["qrows"])):
        r, ring, comp, sel, K = RF.row_inputs(d, i)
        want = d["attn_out"][i]
        vec = O.ds41_attend(d["q"][i:i + 1].copy(), ring, 64, comp, max(d["ratio"], 1), sel, K, d["sinks"], 1, d["H"], r, d["WIN"], scale, mode=0)[0]
        xmx = O.ds41_attend(d["q"][i:i + 1].copy(), ring, 64, comp, max(d["ratio"], 1), sel, K, d["sinks"], 1, d["H"], r, d["WIN"], scale, mode=1)[0]
        assert np.abs(vec - want).max() < 1e-5, (L, r)
        assert np.all(np.abs(xmx - want) <= RF.ABS + RF.REL * np.abs(want)), (L, r)


def test_ref_pin_indexer_scores_candidates_and_picks():
    """The indexer of Ref.attention (:212-231): scores sum_h w relu(q . k), -inf past what the row sees; block maxima with
    the newest block forced in; the top blocks kept; the K best keys in ascending position."""
    d = RF.layer(RF.load(), 1)
    iq, w, k = d["idx_q"], d["idx_w"], d["idx_k_f16"]
    n, (IH, ID) = k.shape[0], iq.shape[1:]
    for i, r in enumerate(d["qrows"]):
        r = int(r)
        vis = (r + 1) // d["ratio"]
        sc = O.ds41_idx_score(iq[i:i + 1].copy(), w[i:i + 1].copy(), k, 1, IH, ID, n, n, r, d["ratio"], half_q=False)
        assert np.allclose(sc[0, :vis], d["idx_score"][i, :vis], rtol=1e-6, atol=1e-6) and np.all(np.isneginf(sc[0, vis:]))
        if vis == 0:
            continue      # nothing to pick; (the reference's kernel leaves such a row's blocks at -inf, its Python keeps block 0: k41.cpp:412)
        bm = O.ds41_block_max(sc, n, d["cand_bs"], r, d["ratio"])
        nb = bm.shape[1]
        keep = np.zeros(nb, bool)
        for b in O.topk(bm, nb, min(d["cand_top"], nb))[0]:
            keep[b] = b >= 0 and bm[0, b] > -np.inf
        assert np.array_equal(np.repeat(keep, d["cand_bs"])[:n], d["cand"][i].astype(bool)), r
        sel = O.topk(sc, n, min(d["ITOP"], n))[0]
        want = d["topk"][i]
        assert np.array_equal(sel[:min(vis, d["ITOP"])], want[want >= 0]), r


def test_q6k_reader_is_ggml_block_layout():
    """orc_q6k_rows (kernels/llm/deepseek2/ds2.cpp:117-137) against ggml's published block_q6_K layout written out in numpy."""
    rng = np.random.default_rng(7)
    blk = rng.integers(0, 256, size=(3, 420), dtype=np.uint8)
    d = np.array([1e-3, -2e-3], np.float16)
    for b in range(2):
        blk[:, b * 210 + 208:b * 210 + 210] = d[b:b + 1].view(np.uint8)
    got = O.q6k_rows(blk, 3, 512)
    want = np.zeros((3, 512), np.float32)
    for r in range(3):
        for b in range(2):
            x = blk[r, b * 210:(b + 1) * 210]
            ql, qh, sc, dd = x[:128].astype(np.int32), x[128:192].astype(np.int32), x[192:208].view(np.int8), np.float32(x[208:210].view(np.float16)[0])
            for n in range(2):
                for l in range(32):
                    h = qh[32 * n + l]
                    qs = [(ql[64 * n + l] & 0xF) | ((h & 3) << 4), (ql[64 * n + l + 32] & 0xF) | (((h >> 2) & 3) << 4),
                          (ql[64 * n + l] >> 4) | (((h >> 4) & 3) << 4), (ql[64 * n + l + 32] >> 4) | (((h >> 6) & 3) << 4)]
                    for g in range(4):
                        want[r, b * 256 + 128 * n + 32 * g + l] = dd * np.float32(sc[8 * n + l // 16 + 2 * g]) * np.float32(qs[g] - 32)
    assert np.array_equal(got, want)
