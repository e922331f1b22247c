"""GQA split-KV decode on the GPU against the CPU oracle, through the C ABI.

Tolerance: the benchmark's bar for this path, max-abs 2e-3 / max-rel 1e-2 against the reference numerics (the oracle's
flash mode restates kernels/llm/qwen35/silo/attn.cpp), checked as |got - want| <= 2e-3 + 1e-2 |want|; the fp64 exact
result is reported beside it with the same bar."""
import numpy as np
import pytest

from nextsycl_b200 import DevBuf
from nextsycl_b200 import workloads as W
from oracle import oracle as O

pytestmark = pytest.mark.gpu
ABS, REL = 2e-3, 1e-2


def assert_close(got, want, what):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    d = np.abs(got - want)
    bad = d > ABS + REL * np.abs(want)
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside tolerance, max abs {d.max():.3e}"


def run_compat(gpu, ops, q, k, v, T, Hq, Hkv, D, cap, p0, name="ns_q35_attn_decode", qs=None):
    qs = qs or Hq * D
    qf = np.zeros((T, qs), np.float32)
    qf[:, :Hq * D] = q.astype(np.float32)
    dq, dk, dv = DevBuf.of(gpu, qf), DevBuf.of(gpu, k), DevBuf.of(gpu, v)
    out = DevBuf(gpu, T * Hq * D * 4)
    out.fill(0xFF)
    n = int(gpu.api.need(name + "_scratch")(T, Hq, Hkv, D, p0))
    sc = DevBuf(gpu, n * 4) if n else None
    if sc is not None:
        sc.fill(0xFF)   # the arena hands out whatever was there before (NaN patterns here)
    if name.endswith("decode"):
        ops.attn_decode(dq, qs, dk, dv, T, Hq, Hkv, D, cap, p0, out, sc, name=name)
    else:
        ops.attn(dq, qs, dk, dv, T, Hq, Hkv, D, cap, p0, out, sc, name=name)
    return out.read(np.float32).reshape(T, Hq * D)


CASES = [
    # T, Hq, Hkv, D, kv
    (1, 8, 2, 128, 1),          # a single key
    (1, 8, 2, 128, 15),         # less than one tile
    (1, 64, 8, 128, 100),       # ragged, two splits
    (4, 32, 4, 128, 1000),      # the verify shape, 32 rows a key head
    (8, 16, 4, 128, 333),       # 8 rows x 4 heads
    (3, 16, 1, 128, 2049),      # 16 heads a key head, 48 rows: two row groups
    (1, 4, 4, 128, 4097),       # one query head a key head
    (2, 24, 4, 256, 700),       # the qwen35 shape (D 256, 6 heads a key head)
    (8, 24, 4, 256, 65),        # 48 rows of 256: three row groups
    (1, 64, 8, 128, 5000),
]


@pytest.mark.parametrize("T,Hq,Hkv,D,kv", CASES)
def test_decode_matches_oracle(gpu, ops, T, Hq, Hkv, D, kv):
    cap = kv + 3
    q, k, v, p0 = W.gqa_case(920, T, Hq, Hkv, D, kv, cap=cap)
    got = run_compat(gpu, ops, q, k, v, T, Hq, Hkv, D, cap, p0)
    qf, kb, vb = q.astype(np.float32), k.view(np.uint16), v.view(np.uint16)
    assert_close(got, O.gqa_flash_decode(qf, kb, vb, T, Hq, Hkv, D, cap, p0), "vs flash numerics")
    assert_close(got, O.attn_exact(qf, kb, vb, T, Hq, Hkv, D, D, cap, p0, 1 / np.sqrt(D)), "vs fp64")


def test_query_row_stride_and_other_names(gpu, ops):
    T, Hq, Hkv, D, kv = 2, 16, 2, 128, 300
    q, k, v, p0 = W.gqa_case(921, T, Hq, Hkv, D, kv)
    want = O.gqa_flash_decode(q.astype(np.float32), k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, kv, p0)
    assert_close(run_compat(gpu, ops, q, k, v, T, Hq, Hkv, D, kv, p0, qs=Hq * D + 64), want, "strided q")
    assert_close(run_compat(gpu, ops, q, k, v, T, Hq, Hkv, D, kv, p0, name="ns_nhs_attn_decode"), want, "nhs name")
    assert_close(run_compat(gpu, ops, q, k, v, T, Hq, Hkv, D, kv, p0, name="ns_nh_attn"), want, "nh name")


def test_a_row_does_not_depend_on_its_pass(gpu, ops):
    """Verify rows equal one-row passes bit for bit, also where the rows' split sizes differ
    (the invariant of kernels/llm/qwen35/silo/attn.cpp:100-104 that `spec-check` tests, cli/nextsycl/src/main.rs:967-989)."""
    Hq, Hkv, D = 32, 4, 128
    for kv in (900, 4739):   # 4739: rows 4736 | 4737.. sit either side of a step of the split size (4 key heads)
        T = 4
        q, k, v, p0 = W.gqa_case(922, T, Hq, Hkv, D, kv)
        rows = run_compat(gpu, ops, q, k, v, T, Hq, Hkv, D, kv, p0)
        for t in range(T):
            one = run_compat(gpu, ops, q[t:t + 1], k, v, 1, Hq, Hkv, D, kv, p0 + t)
            assert np.array_equal(one[0], rows[t]), (kv, t)


def test_rows_path_any_T(gpu, ops):
    """ns_q35_attn with more than 8 rows."""
    T, Hq, Hkv, D, kv = 19, 8, 2, 128, 140
    q, k, v, p0 = W.gqa_case(923, T, Hq, Hkv, D, kv)
    got = run_compat(gpu, ops, q, k, v, T, Hq, Hkv, D, kv, p0, name="ns_q35_attn")
    assert_close(got, O.gqa_flash_prefill(q.astype(np.float32), k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, kv, p0), "rows")


def test_kv_store_then_decode(gpu, ops):
    T, Hkv, D, cap, p0 = 3, 4, 128, 64, 40
    k = W.rng(924, 0).standard_normal((T, Hkv * D), dtype=np.float32)
    v = W.rng(924, 1).standard_normal((T, Hkv * D), dtype=np.float32)
    kc, vc = DevBuf(gpu, Hkv * cap * D * 2), DevBuf(gpu, Hkv * cap * D * 2)
    kc.fill(0), vc.fill(0)
    dkr, dvr = DevBuf.of(gpu, k), DevBuf.of(gpu, v)
    ops.kv_store(dkr, Hkv * D, dvr, Hkv * D, T, Hkv, D, cap, p0, kc, vc)
    hk, hv = np.zeros((Hkv, cap, D), np.uint16), np.zeros((Hkv, cap, D), np.uint16)
    O.kv_store(k, v, T, Hkv, D, cap, p0, hk, hv)
    assert np.array_equal(kc.read(np.uint16).reshape(Hkv, cap, D), hk)      # bit-exact: one rounding to fp16
    assert np.array_equal(vc.read(np.uint16).reshape(Hkv, cap, D), hv)
    from nextsycl_b200 import Error
    with pytest.raises(Error, match="capacity"):
        ops.kv_store(dkr, Hkv * D, dvr, Hkv * D, T, Hkv, D, cap, cap - 1, kc, vc)


def test_argument_errors(gpu, ops):
    api = gpu.api
    d = DevBuf(gpu, 1 << 20)
    assert api.ns_q35_attn_decode(gpu.raw, d.ptr, 1024, d.ptr, d.ptr, 9, 8, 2, 128, 100, 0, d.ptr, None) == -1
    assert "1..8 rows" in api.last_error()
    assert api.ns_q35_attn_decode(gpu.raw, d.ptr, 1024, d.ptr, d.ptr, 1, 8, 2, 128, 100, 100, d.ptr, None) == -1
    assert "capacity" in api.last_error()
    assert api.ns_q35_attn_decode(gpu.raw, d.ptr, 8 * 128, d.ptr, d.ptr, 1, 8, 2, 128, 100000, 50000, d.ptr, None) == -1
    assert "scratch" in api.last_error()
    assert api.ns_q35_attn_decode_kv(gpu.raw, 1, d.ptr, 1024, d.ptr, d.ptr, 1, 8, 2, 128, 100, 0, d.ptr, None) == -1
    gpu.sync()


def test_native_batch_fp16(gpu, ops):
    """ns_b200_gqa_decode: 3 sequences of different lengths in one launch equal their own one-sequence results."""
    B, T, Hq, Hkv, D = 3, 2, 16, 2, 128
    kvs = [50, 1500, 777]
    cap = 1600
    qs, seqs, want = [], [], []
    keep = []
    for b, kv in enumerate(kvs):
        q, k, v, p0 = W.gqa_case(925, T, Hq, Hkv, D, kv, cap=cap, seq=b)
        qs.append(q)
        dk, dv = DevBuf.of(gpu, k), DevBuf.of(gpu, v)
        keep += [dk, dv]
        seqs.append((dk, dv, cap, p0))
        want.append(O.gqa_flash_decode(q.astype(np.float32), k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, cap, p0))
    dq = DevBuf.of(gpu, np.stack(qs))
    table = ops.seq_table(seqs)
    out = DevBuf(gpu, B * T * Hq * D * 2)
    n = ops.gqa_decode_scratch(B, T, Hq, Hkv, D, max(kvs))
    sc = DevBuf(gpu, n * 4)
    sc.fill(0xFF)
    ops.gqa_decode(dq, Hq * D, T * Hq * D, table, B, T, Hq, Hkv, D, max(kvs), out, sc)
    got = out.read(np.float16).reshape(B, T, Hq * D).astype(np.float32)
    for b in range(B):
        # fp16 output: half an ulp of fp16 on top of the kernel's own error
        assert_close(got[b], want[b], f"sequence {b}")


def _batch(gpu, ops, seed, T, Hq, Hkv, D, kvs, cap):
    qs, seqs, want, keep = [], [], [], []
    for b, kv in enumerate(kvs):
        q, k, v, p0 = W.gqa_case(seed, T, Hq, Hkv, D, kv, cap=cap, seq=b)
        qs.append(q)
        dk, dv = DevBuf.of(gpu, k), DevBuf.of(gpu, v)
        keep += [dk, dv]
        seqs.append((dk, dv, cap, p0))
        want.append(O.gqa_flash_decode(q.astype(np.float32), k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, cap, p0))
    return DevBuf.of(gpu, np.stack(qs)), ops.seq_table(seqs), want, keep


@pytest.mark.parametrize("Hq,Hkv,kvs", [(64, 8, [9000, 4736]), (32, 4, [4737, 4736, 9472]), (16, 2, [20000, 9473, 64, 18944])])
def test_ragged_batch_where_a_shorter_sequence_needs_more_splits(gpu, ops, Hq, Hkv, kvs):
    """The split count is not monotone in the length (8 key heads: 4,736 keys make 37 splits, 9,000 make 36), so the
    partials are laid out for the most any length up to max_kv can need; each sequence against the oracle."""
    T, D = 1, 128
    cap = max(kvs)
    dq, table, want, keep = _batch(gpu, ops, 927, T, Hq, Hkv, D, kvs, cap)
    B = len(kvs)
    out = DevBuf(gpu, B * T * Hq * D * 2)
    sc = DevBuf(gpu, 4 * ops.gqa_decode_scratch(B, T, Hq, Hkv, D, cap))
    sc.fill(0xFF)
    ops.gqa_decode(dq, Hq * D, T * Hq * D, table, B, T, Hq, Hkv, D, cap, out, sc)
    got = out.read(np.float16).reshape(B, T, Hq * D).astype(np.float32)
    for b in range(B):
        assert_close(got[b], want[b], f"sequence {b} of {kvs}")


def test_a_sequence_longer_than_max_kv_is_reported_not_misread(gpu, ops):
    """max_kv sizes the partials; a longer sequence makes the merge stop at the layout and the next sync fail (code 802)."""
    from nextsycl_b200 import Error
    T, Hq, Hkv, D = 1, 16, 2, 128
    dq, table, want, keep = _batch(gpu, ops, 928, T, Hq, Hkv, D, [1000], 1000)
    out = DevBuf(gpu, T * Hq * D * 2)
    sc = DevBuf(gpu, 4 * ops.gqa_decode_scratch(1, T, Hq, Hkv, D, 100))
    ops.gqa_decode(dq, Hq * D, T * Hq * D, table, 1, T, Hq, Hkv, D, 100, out, sc)
    with pytest.raises(Error, match="802"):
        gpu.sync()
    gpu.sync()   # the status is cleared; the GPU is usable
    sc = DevBuf(gpu, 4 * ops.gqa_decode_scratch(1, T, Hq, Hkv, D, 1000))
    ops.gqa_decode(dq, Hq * D, T * Hq * D, table, 1, T, Hq, Hkv, D, 1000, out, sc)
    assert_close(out.read(np.float16).reshape(T, Hq * D).astype(np.float32), want[0], "after the report")


@pytest.mark.parametrize("B", [1, 2])
def test_full_size_config_2(gpu, ops, B):
    """benchmark configuration 2 at full size: 64 query heads, 8 key heads, 32,768 cached tokens, batch of sequences."""
    T, Hq, Hkv, D, kv = 1, 64, 8, 128, 32768
    seqs, want, qs, keep = [], [], [], []
    for b in range(B):
        q, k, v, p0 = W.gqa_case(2, T, Hq, Hkv, D, kv, seq=b)
        qs.append(q)
        dk, dv = DevBuf.of(gpu, k), DevBuf.of(gpu, v)
        keep += [dk, dv]
        seqs.append((dk, dv, kv, p0))
        want.append(O.gqa_flash_decode(q.astype(np.float32), k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, kv, p0))
    dq = DevBuf.of(gpu, np.stack(qs))
    out = DevBuf(gpu, B * T * Hq * D * 2)
    sc = DevBuf(gpu, 4 * ops.gqa_decode_scratch(B, T, Hq, Hkv, D, kv))
    ops.gqa_decode(dq, Hq * D, T * Hq * D, ops.seq_table(seqs), B, T, Hq, Hkv, D, kv, out, sc)
    got = out.read(np.float16).reshape(B, T, Hq * D).astype(np.float32)
    for b in range(B):
        assert_close(got[b], want[b], f"sequence {b}")


@pytest.mark.parametrize("T,Hq,Hkv,kv", [(1, 64, 8, 32768), (4, 32, 4, 262144)])
def test_nh_attn_against_the_plain_numerics_at_full_size(gpu, ops, T, Hq, Hkv, kv):
    """Configurations 2 and 5 through ns_nh_attn, held to the numerics of the ONLY reference kernel that exists for heads of
    128 - the vector-unit attn<8,8> (kernels/llm/nemotronh/nh.cpp:575-585: fp32 query times scale, natural exp, fp32
    weights; the oracle's plain mode) - within the path's bar."""
    D = 128
    q, k, v, p0 = W.gqa_case(2 if T == 1 else 5, T, Hq, Hkv, D, kv)
    got = run_compat(gpu, ops, q, k, v, T, Hq, Hkv, D, kv, p0, name="ns_nh_attn")
    assert_close(got, O.gqa_plain(q.astype(np.float32), k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, kv, p0), "vs plain numerics")


def test_full_size_config_5(gpu, ops):
    """benchmark configuration 5 on one GPU at full size: 4 verify rows, 32 query / 4 key heads of 128, 262,144 cached tokens
    (512 MiB of K and V). Each row against the oracle's flash numerics, and row t against the one-row pass at its position
    (bit for bit: a row's splits come from its own length)."""
    T, Hq, Hkv, D, kv = 4, 32, 4, 128, 262144
    q, k, v, p0 = W.gqa_case(5, T, Hq, Hkv, D, kv)
    dk, dv, dq = DevBuf.of(gpu, k), DevBuf.of(gpu, v), DevBuf.of(gpu, q)
    out = DevBuf(gpu, T * Hq * D * 2)
    sc = DevBuf(gpu, 4 * ops.gqa_decode_scratch(1, T, Hq, Hkv, D, kv))
    ops.gqa_decode(dq, Hq * D, T * Hq * D, ops.seq_table([(dk, dv, kv, p0)]), 1, T, Hq, Hkv, D, kv, out, sc)
    got = out.read(np.float16).reshape(T, Hq * D)
    want = O.gqa_flash_decode(q.astype(np.float32), k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, kv, p0)
    assert_close(got.astype(np.float32), want, "config 5")
    one = DevBuf(gpu, Hq * D * 2)
    for t in (0, T - 1):
        dq1 = DevBuf.of(gpu, q[t:t + 1].copy())
        ops.gqa_decode(dq1, Hq * D, Hq * D, ops.seq_table([(dk, dv, kv, p0 + t)]), 1, 1, Hq, Hkv, D, kv, one, sc)
        assert np.array_equal(one.read(np.float16).reshape(Hq * D).view(np.uint16), got[t].view(np.uint16)), f"row {t}"


def test_batched_cache_writer_equals_the_per_sequence_one(gpu, ops):
    """ns_b200_kv_store_batch: one launch writes every sequence's new rows at its own position, bit for bit what one
    ns_q35_kv_store a sequence writes; a row past a cache's capacity is skipped and reported."""
    from nextsycl_b200 import Error
    B, T, Hkv, D, cap = 3, 2, 4, 128, 40
    p0s = [0, 17, 38]
    k = W.rng(929, 0).standard_normal((B, T, Hkv * D), dtype=np.float32)
    v = W.rng(929, 1).standard_normal((B, T, Hkv * D), dtype=np.float32)
    dk, dv = DevBuf.of(gpu, k), DevBuf.of(gpu, v)
    one, batch = [], []
    for b in range(B):
        for dst in (one, batch):
            kc, vc = DevBuf(gpu, Hkv * cap * D * 2), DevBuf(gpu, Hkv * cap * D * 2)
            kc.fill(0x11), vc.fill(0x22)
            dst.append((kc, vc))
        ops.kv_store(dk.view(b * T * Hkv * D * 4, T * Hkv * D * 4), Hkv * D, dv.view(b * T * Hkv * D * 4, T * Hkv * D * 4), Hkv * D, T, Hkv, D, cap, p0s[b],
                     one[b][0], one[b][1])
    table = ops.seq_table([(batch[b][0], batch[b][1], cap, p0s[b]) for b in range(B)])
    ops.kv_store_batch(dk, Hkv * D, T * Hkv * D, dv, Hkv * D, T * Hkv * D, table, B, T, Hkv, D)
    gpu.sync()
    for b in range(B):
        assert np.array_equal(batch[b][0].read(np.uint16), one[b][0].read(np.uint16)), b
        assert np.array_equal(batch[b][1].read(np.uint16), one[b][1].read(np.uint16)), b
    table = ops.seq_table([(batch[0][0], batch[0][1], cap, cap - 1)])      # two rows at the last position: the second does not fit
    ops.kv_store_batch(dk, Hkv * D, T * Hkv * D, dv, Hkv * D, T * Hkv * D, table, 1, T, Hkv, D)
    with pytest.raises(Error, match="803"):
        gpu.sync()
    gpu.sync()
