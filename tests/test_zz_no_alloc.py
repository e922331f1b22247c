"""ns_b200_gqa_decode_static: split-KV decode for callers that cannot allocate (a memory plan fixed at load, a serving
loop that must not stall on cudaMalloc). Its partials live in an array inside the library; the result must equal the
entry point that takes caller scratch. Runs last so that a failure here cannot hide another test's."""
import numpy as np
import pytest

from nextsycl_b200 import DevBuf
from nextsycl_b200 import workloads as W

pytestmark = pytest.mark.gpu
ABS, REL = 2e-3, 1e-2


def _case(gpu, ops, seed, B, T, Hq, Hkv, D, kvs, cap):
    qs, seqs, keep = [], [], []
    for b, kv in enumerate(kvs):
        q, k, v, p0 = W.gqa_case(seed, T, Hq, Hkv, D, kv, cap=cap, seq=b)
        qs.append(q)
        dk, dv = DevBuf.of(gpu, k), DevBuf.of(gpu, v)
        keep += [dk, dv]
        seqs.append((dk, dv, cap, p0))
    return DevBuf.of(gpu, np.stack(qs)), ops.seq_table(seqs), keep


def test_static_scratch_decode_equals_caller_scratch_twice(gpu, ops):
    api = gpu.api
    f = api.need("ns_b200_gqa_decode_static")
    shapes = [(3, 2, 16, 2, 128, [700, 3000, 1234], 3008), (2, 1, 64, 8, 128, [9000, 5000], 9000)]   # two calls in a row, different shapes
    for i, (B, T, Hq, Hkv, D, kvs, cap) in enumerate(shapes):
        dq, table, keep = _case(gpu, ops, 990 + i, B, T, Hq, Hkv, D, kvs, cap)
        n = B * T * Hq * D
        want = DevBuf(gpu, n * 2)
        sc = DevBuf(gpu, max(4, 4 * ops.gqa_decode_scratch(B, T, Hq, Hkv, D, max(kvs))))
        ops.gqa_decode(dq, Hq * D, T * Hq * D, table, B, T, Hq, Hkv, D, max(kvs), want, sc)
        w = want.read(np.float16).astype(np.float32)
        for call in range(2):
            got = DevBuf(gpu, n * 2)
            got.fill(0xFF)
            rc = f(gpu.raw, dq.ptr, Hq * D, T * Hq * D, table.ptr, B, T, Hq, Hkv, D, max(kvs), got.ptr)
            assert rc == 0, api.last_error()
            o = got.read(np.float16).astype(np.float32)
            assert np.isfinite(o).all()
            assert np.all(np.abs(o - w) <= ABS + REL * np.abs(w)), (i, call, float(np.abs(o - w).max()))


def test_static_scratch_rejects_what_does_not_fit(gpu, ops):
    api = gpu.api
    d = DevBuf(gpu, 4096)
    # 64 sequences x 8 rows x 64 heads x ~37 splits x 130 floats: far beyond 4 Mi floats
    rc = api.need("ns_b200_gqa_decode_static")(gpu.raw, d.ptr, 64 * 128, 8 * 64 * 128, d.ptr, 64, 8, 64, 8, 128, 32768, d.ptr)
    assert rc == -1
    assert "built-in scratch holds" in api.last_error()
    gpu.sync()
