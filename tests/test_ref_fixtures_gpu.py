"""The CUDA kernels held DIRECTLY to values the reference's own CPU code produced (tests/golden/ds41ref_fixtures.npz,
written by tests/golden/make_ref_fixtures.py from reference/deepseek41/ds41ref.py): the attention with sinks, the steps
either side of it, and the indexer. No oracle in between. Tolerance: the path's bar, |got - want| <= 2e-3 + 1e-2 |want|,
for the attention (fp16 q and weights on the tensor cores against the reference's float32); for the E4M3 simulation,
whose output is a step function of values computed with device sin / cos against float64 tables, "equal except where a
value sat on a rounding boundary" (at least 99.5% bit-equal, the rest one grid step away)."""
import numpy as np
import pytest

import ref_fixtures as RF
from nextsycl_b200 import DevBuf
from nextsycl_b200.core import check

pytestmark = pytest.mark.gpu


def sim_close(got, want, what):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert np.isfinite(got).all(), what
    same = got == want
    assert same.mean() > 0.995, f"{what}: {1 - same.mean():.4f} of the values differ"
    assert np.all(np.abs(got - want) <= 0.13 * np.abs(want) + 2e-6), what


@pytest.mark.parametrize("L", [0, 1])
def test_attend_equals_the_reference_python(gpu, L):
    d = RF.layer(RF.load(), L)
    api = gpu.api
    scale = np.float32(d["HD"] ** -0.5)
    dsk = DevBuf.of(gpu, d["sinks"])
    for i in range(len(d["qrows"])):
        r, ring, comp, sel, K = RF.row_inputs(d, i)
        dq, dring = DevBuf.of(gpu, d["q"][i:i + 1].copy()), DevBuf.of(gpu, ring)
        dcomp = DevBuf.of(gpu, comp) if comp is not None else None
        dsel = DevBuf.of(gpu, sel) if sel is not None else None
        out = DevBuf(gpu, d["H"] * 512 * 4)
        for fn in (api.ns_ds41_attend_xmx, api.ns_ds41_attend):
            out.fill(0xFF)
            check(api, fn(gpu.raw, dq.ptr, dring.ptr, 64, dcomp.ptr if dcomp else None, max(d["ratio"], 1), dsel.ptr if dsel else None, K, dsk.ptr,
                          out.ptr, 1, d["H"], r, d["WIN"], scale), "ns_ds41_attend")
            gpu.sync()
            got = out.read(np.float32).reshape(d["H"], 512)
            want = d["attn_out"][i]
            assert np.isfinite(got).all()
            assert np.all(np.abs(got - want) <= RF.ABS + RF.REL * np.abs(want)), (L, r, float(np.abs(got - want).max()))


@pytest.mark.parametrize("L", [0, 1])
def test_kv_post_and_att_post_equal_the_reference_python(gpu, L):
    d = RF.layer(RF.load(), L)
    api = gpu.api
    y = [np.float32(v) for v in d["yarn"]]
    T, D, R = d["T"], d["HD"], 64
    dkv, dw, dr = DevBuf.of(gpu, d["kv_in"]), DevBuf.of(gpu, d["kv_w"]), DevBuf(gpu, R * D * 2)
    dr.fill(0)
    check(api, api.ns_ds41_kv_post(gpu.raw, dkv.ptr, dw.ptr, T, D, np.float32(1e-6), d["RD"], 0, *y, dr.ptr, R), "ns_ds41_kv_post")
    gpu.sync()
    want = d["kv_f16"].view(np.float16).astype(np.float32)
    sim_close(dkv.read(np.float32).reshape(T, D), want, "kv_post")
    sim_close(dr.read(np.uint16).reshape(R, D)[:T].view(np.float16).astype(np.float32), want, "kv_post ring")
    for i, r in enumerate(d["qrows"]):
        dx = DevBuf.of(gpu, d["attn_out"][i:i + 1].copy())
        check(api, api.ns_ds41_att_post(gpu.raw, dx.ptr, 1, d["H"], D, d["RD"], int(r), *y), "ns_ds41_att_post")
        gpu.sync()
        sim_close(dx.read(np.float32).reshape(d["H"], D), d["att_post_out"][i], f"att_post row {int(r)}")


def test_indexer_scores_equal_the_reference_python(gpu):
    d = RF.layer(RF.load(), 1)
    api = gpu.api
    iq, w, k = d["idx_q"], d["idx_w"], d["idx_k_f16"]
    n, (IH, ID) = k.shape[0], iq.shape[1:]
    dk = DevBuf.of(gpu, k)
    for i, r in enumerate(d["qrows"]):
        r = int(r)
        vis = (r + 1) // d["ratio"]
        dq, dw, ds = DevBuf.of(gpu, iq[i:i + 1].copy()), DevBuf.of(gpu, w[i:i + 1].copy()), DevBuf(gpu, n * 4)
        check(api, api.ns_ds41_idx_score(gpu.raw, dq.ptr, dw.ptr, dk.ptr, ds.ptr, 1, IH, ID, n, n, r, d["ratio"]), "ns_ds41_idx_score")
        gpu.sync()
        sc = ds.read(np.float32)
        assert np.allclose(sc[:vis], d["idx_score"][i, :vis], rtol=1e-5, atol=1e-5) and np.all(np.isneginf(sc[vis:])), r
        if vis == 0:
            continue
        K = min(d["ITOP"], n)
        dsel = DevBuf(gpu, K * 4)
        dsel.fill(0xFF)
        check(api, api.ns_topk(gpu.raw, ds.ptr, dsel.ptr, 1, n, n, K), "ns_topk")
        gpu.sync()
        want = d["topk"][i]
        assert np.array_equal(dsel.read(np.int32)[:min(vis, K)], want[want >= 0]), r
