"""Writes tests/golden/ds41ref_fixtures.npz by RUNNING the reference's own CPU statement of DeepSeek-V4.1 attention.

The reference tree holds one importable, weight-free CPU implementation of arithmetic on this path:
reference/deepseek41/ds41ref.py (PyTorch float32). Its module-level functions - pow2_ceil, fp8_sim (:32-55), rms, freqs,
rope (:88-113) - are what ns_ds41_kv_post / ns_ds41_att_post compute, and Ref.attention (:168-262) is the model's
attention: window keys, compressed keys, the indexer's scores, block candidates and top-k picks, masked scores, the
per-head sink in the denominator only (:241-250), the rotation undone on the output and its E4M3 simulation.

This script imports that module from the reference checkout, builds a Ref WITHOUT a model file (its weights come from a
seeded generator through a stub of Ref.w; every other line of Ref.attention runs as written), and records the inputs
and outputs of the steps the CPU oracle restates - through the reference's own `tap` callback and by wrapping the
module-level functions it calls. Nothing is retyped: every expected value in the fixture file was produced by
the reference's code. tests/test_oracle.py holds the oracle to these fixtures.

Run where the reference checkout is available (not on the GPU machines):
    python tests/golden/make_ref_fixtures.py /path/to/the/nextsycl/checkout
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) != 2:
    raise SystemExit("usage: python tests/golden/make_ref_fixtures.py /path/to/the/nextsycl/checkout")
REF = sys.argv[1]
sys.path.insert(0, os.path.join(REF, "reference", "deepseek41"))
os.environ.setdefault("NS_REF_THREADS", "4")
import ds41ref as R  # noqa: E402

OUT = os.path.join(HERE, "ds41ref_fixtures.npz")
fx = {}


def f32(t):
    return np.ascontiguousarray(t.detach().to(torch.float32).numpy())


def f16_bits_exact(t, what):
    """fp16 bit patterns of values the caches hold; the simulated values must survive the cast unchanged."""
    a = f32(t)
    h = a.astype(np.float16)
    assert np.array_equal(h.astype(np.float32), a), what + ": not exact in fp16"
    return h.view(np.uint16)


# ---------------------------------------------------------------------------------------------------------------------
# 1. the module-level functions on their own
# ---------------------------------------------------------------------------------------------------------------------
g = torch.Generator().manual_seed(0x6E73 + 41)

# E4M3 simulation in blocks of 32: ordinary blocks, a block of zeros, one below the amax floor, one with a lone spike,
# one whose values sit on rounding ties of the E4M3 grid, one of large values
v = torch.randn(16, 32, generator=g)
v[1] = 0.0
v[2] = 3e-5 * torch.randn(32, generator=g)
v[3] = 1e-3 * torch.randn(32, generator=g)
v[3, 7] = 200.0
tie = torch.tensor([1.0625, 1.1875, 1.3125, 2.125, 2.375, 0.53125, 17.0, 19.0, 0.001953125 * 0.5, 0.001953125 * 1.5])
v[4, :10] = tie
v[4, 10] = 448.0       # amax 448: scale exactly 1, the ties above are ties on the grid
v[4, 11:] = 0.0
v[5] = 1e4 * torch.randn(32, generator=g)
v[6] = -v[4]
fx["fp8_in"], fx["fp8_out"] = f32(v), f32(R.fp8_sim(v.clone()))

xr = torch.randn(5, 96, generator=g) * 3.0
wr = 1.0 + 0.1 * torch.randn(96, generator=g)
fx["rms_in"], fx["rms_w"], fx["rms_out"] = f32(xr), f32(wr), f32(R.rms(xr, wr, 1e-6))

# the rotation's table: plain (orig 0) and YaRN. (dim, n, orig, base, factor, beta_fast, beta_slow)
YARN = dict(dim=64, orig=4096, base=160000.0, factor=16.0, beta_fast=32.0, beta_slow=1.0)
PLAIN = dict(dim=64, orig=0, base=10000.0, factor=16.0, beta_fast=32.0, beta_slow=1.0)
NPOS = 3000
for name, cfg in (("yarn", YARN), ("plain", PLAIN)):
    c, s = R.freqs(cfg["dim"], NPOS, cfg["orig"], cfg["base"], cfg["factor"], cfg["beta_fast"], cfg["beta_slow"])
    pos = torch.tensor([0, 1, 2, 17, 255, 1024, 2999])
    xx = torch.randn(len(pos), 3, 64, generator=g)
    fx[f"rope_{name}_cfg"] = np.array([cfg["dim"], cfg["orig"], cfg["base"], cfg["factor"], cfg["beta_fast"], cfg["beta_slow"]], np.float64)
    fx[f"rope_{name}_pos"] = pos.numpy().astype(np.int64)
    fx[f"rope_{name}_cos"], fx[f"rope_{name}_sin"] = f32(c[pos]), f32(s[pos])
    fx[f"rope_{name}_in"] = f32(xx)
    fx[f"rope_{name}_out"] = f32(R.rope(xx, (c, s), pos))
    fx[f"rope_{name}_inv"] = f32(R.rope(xx, (c, s), pos, inverse=True))

# ---------------------------------------------------------------------------------------------------------------------
# 2. Ref.attention as written, on seeded weights
# ---------------------------------------------------------------------------------------------------------------------
ref = R.Ref.__new__(R.Ref)      # no model file: the fields __init__ reads from the file are set here
ref.D, ref.L = 96, 2
ref.H, ref.HD, ref.RD = 4, 512, 64
ref.QL, ref.OG, ref.OL = 48, 2, 16
ref.WIN = 16
ref.IH, ref.ID, ref.ITOP = 4, 128, 5
ref.ratio = [0, 4]
ref.kv_src, ref.idx_src = [1], [1]
ref.cand_src, ref.cand_top, ref.cand_bs = 1, 2, 4
ref.eps = 1e-6
ref.rope_base, ref.comp_base = PLAIN["base"], YARN["base"]
ref.yarn = (YARN["orig"], YARN["factor"], YARN["beta_fast"], YARN["beta_slow"])

SHAPES = {
    "attn_q_a.weight": (ref.QL, ref.D), "attn_q_a_norm.weight": (ref.QL,), "attn_q_b.weight": (ref.H * ref.HD, ref.QL),
    "attn_kv.weight": (ref.HD, ref.D), "attn_kv_a_norm.weight": (ref.HD,),
    "attn_compressor_kv.weight": (ref.HD, ref.D), "attn_compressor_gate.weight": (ref.HD, ref.D), "attn_compressor_norm.weight": (ref.HD,),
    "indexer.wk.weight": (ref.ID, ref.HD), "indexer.k_norm.weight": (ref.ID,), "indexer.attn_q_b.weight": (ref.IH * ref.ID, ref.QL),
    "indexer.proj.weight": (ref.IH, ref.D), "attn_sinks.weight": (ref.H,),
    "attn_output_a.weight": (ref.OG * ref.OL, ref.H * ref.HD // ref.OG), "attn_output_b.weight": (ref.D, ref.OG * ref.OL),
}
weights = {}


def stub_w(l, r):
    if (l, r) not in weights:
        shape = SHAPES[r]
        gen = torch.Generator().manual_seed(1000 * l + sorted(SHAPES).index(r))
        if r.endswith("norm.weight"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=gen)
        elif r == "attn_sinks.weight":
            t = torch.randn(shape, generator=gen)
        elif r == "attn_q_b.weight":
            t = torch.randn(shape, generator=gen) * (2.0 / shape[1] ** 0.5)     # scores a few units wide: a softmax that is neither flat nor one-hot
        else:
            t = torch.randn(shape, generator=gen) / shape[1] ** 0.5
        weights[(l, r)] = t
    return weights[(l, r)].clone()


ref.w = stub_w

calls = []
orig = {n: getattr(R, n) for n in ("rope", "fp8_sim", "fp4_sim", "rms")}


def recorder(name):
    def wrapped(*a, **k):
        ins = [t.clone() if torch.is_tensor(t) else t for t in a]
        out = orig[name](*a, **k)
        calls.append((name, ins, dict(k), out.clone()))
        return out
    return wrapped


for n in orig:
    setattr(R, n, recorder(n))

for layer, T, qrows in ((0, 40, [0, 1, 5, 15, 16, 23, 39]), (1, 48, [0, 2, 3, 11, 19, 20, 31, 47])):
    calls.clear()
    taps = {}
    xin = torch.randn(T, ref.D, generator=torch.Generator().manual_seed(77 + layer))
    xin = xin / xin.square().mean(-1, keepdim=True).sqrt()      # "x [T, D] normed"
    sh = {}
    out = ref.attention(layer, xin, sh, lambda n, t: taps.__setitem__(n, t.clone()), torch.tensor(qrows))
    p = f"L{layer}_"
    fx[p + "qrows"] = np.array(qrows, np.int64)
    fx[p + "meta"] = np.array([T, ref.H, ref.HD, ref.RD, ref.WIN, ref.ratio[layer], ref.ITOP, ref.cand_bs, ref.cand_top], np.int64)
    fx[p + "q"] = f32(taps[f"q-{layer}"])                                    # [rows, H, 512], rotated
    fx[p + "sinks"] = f32(stub_w(layer, "attn_sinks.weight"))
    # the window keys' step: rms (its input, weight) -> rope -> fp8_sim == tap kv
    rms_kv = [c for c in calls if c[0] == "rms" and c[1][1] is not None and c[1][1].shape == (ref.HD,)][0]
    fx[p + "kv_in"], fx[p + "kv_w"] = f32(rms_kv[1][0]), f32(rms_kv[1][1])
    fx[p + "kv_f16"] = f16_bits_exact(taps[f"kv-{layer}"], "window keys")       # the simulated keys: exact in fp16, so these bits are kv_post's output
    # the attention proper: the values before the rotation is undone = the inverse rope call's input beside the untouched part
    inv = [c for c in calls if c[0] == "rope" and c[2].get("inverse")][0]
    derope = taps[f"attn_derope-{layer}"]
    o = derope.clone()
    o[..., -ref.RD:] = inv[1][0]
    fx[p + "attn_out"] = f32(o)                                              # [rows, H, 512] = softmax-with-sink weighted keys
    fx[p + "attn_derope"] = f32(derope)
    sims = [c for c in calls if c[0] == "fp8_sim"]
    fx[p + "att_post_out"] = f32(sims[-1][3].reshape(len(qrows), ref.H, ref.HD))    # fp8_sim of the de-rotated output
    if ref.ratio[layer]:
        fx[p + "comp_f16"] = f16_bits_exact(sh["comp"], "compressed keys")
        fx[p + "idx_k_f16"] = f16_bits_exact(sh["idx_k"], "indexer keys")
        fp4 = [c for c in calls if c[0] == "fp4_sim"]
        iq = [c for c in fp4 if c[3].dim() == 3][0][3]                           # [rows, IH, ID] after its simulation
        fx[p + "idx_q"] = f32(iq)
        wt = (xin[torch.tensor(qrows)] @ stub_w(layer, "indexer.proj.weight").T) * (ref.ID ** -0.5 * ref.IH ** -0.5)
        fx[p + "idx_w"] = f32(wt)
        fx[p + "topk"] = sh["topk"].numpy().astype(np.int32)                    # [rows, K] ascending, -1 where the row sees fewer
        fx[p + "cand"] = sh["cand"].numpy().astype(np.uint8)                    # [rows, ncomp] the kept candidate blocks, per key
        # the scores themselves, recomputed with the reference's own expression (ds41ref.py:214-215) from the recorded operands
        score = (torch.einsum("thd,jd->thj", iq, sh["idx_k"]).relu() * wt[..., None]).sum(1)
        fx[p + "idx_score"] = f32(score)

for n in orig:
    setattr(R, n, orig[n])

np.savez_compressed(OUT, **fx)
print(OUT, os.path.getsize(OUT), "bytes;", len(fx), "arrays")
