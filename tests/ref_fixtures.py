"""Reading tests/golden/ds41ref_fixtures.npz: values produced by running the reference's own CPU code
(reference/deepseek41/ds41ref.py, driven by tests/golden/make_ref_fixtures.py), and the engine's mapping from the model's
rotation settings to the six numbers the kernels take (llm/deepseek41/src/model.rs:669-684)."""
import math
import os

import numpy as np

PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ds41ref_fixtures.npz")
ABS, REL = 2e-3, 1e-2      # the path's parity bar: |got - want| <= 2e-3 + 1e-2 |want|


def load():
    return np.load(PATH)


def yarn_of(cfg):
    """(dim, orig, base, factor, beta_fast, beta_slow) as ds41ref.freqs takes them -> (freq_base, freq_scale, ext_factor,
    mscale, corr0, corr1) as the engine derives them, in float32 like the engine."""
    dim, orig, base, factor, bf, bs = [float(v) for v in cfg]
    if orig == 0:
        return (base, 1.0, 0.0, 1.0, 0.0, 0.0)
    f = np.float32

    def corr(beta):
        return float(f(dim) * np.log(f(orig) / (f(beta) * f(2.0) * f(np.pi))) / (f(2.0) * np.log(f(base))))
    return (base, 1.0 / factor, 1.0, 1.0, max(math.floor(corr(bf)), 0.0), min(math.ceil(corr(bs)), dim - 1.0))


def layer(g, L):
    """The recorded attention of layer L (0: window keys only, plain rotation; 1: compressed keys, indexer picks, YaRN)."""
    p = f"L{L}_"
    T, H, HD, RD, WIN, ratio, ITOP, cand_bs, cand_top = [int(v) for v in g[p + "meta"]]
    d = dict(T=T, H=H, HD=HD, RD=RD, WIN=WIN, ratio=ratio, ITOP=ITOP, cand_bs=cand_bs, cand_top=cand_top,
             yarn=yarn_of(g["rope_plain_cfg" if L == 0 else "rope_yarn_cfg"]))
    for k in g.files:
        if k.startswith(p) and k != p + "meta":
            d[k[len(p):]] = g[k]
    return d


def row_inputs(d, i, R=64):
    """What the kernel of row i sees: the ring as of that row (slot pos % R), the compressed keys, its picks (the
    reference's -1 'no pick' entries become index 0: a row that sees at most K cells reads them all and ignores sel)."""
    r = int(d["qrows"][i])
    ring = np.zeros((R, d["HD"]), np.uint16)
    lo = max(0, r + 1 - R)
    for pos in range(lo, r + 1):
        ring[pos % R] = d["kv_f16"][pos]
    comp = d.get("comp_f16") if d["ratio"] else None
    sel, K = None, 0
    if d["ratio"]:
        K = d["ITOP"]
        s = d["topk"][i:i + 1]
        sel = np.ascontiguousarray(np.where(s < 0, 0, s).astype(np.int32))
    return r, ring, comp, sel, K
