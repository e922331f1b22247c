"""The cubic the prefill softmax uses for a quarter of its exponentials (nextsycl_b200/csrc/tc05.cuh: ex2_pair_fma), restated
in numpy float32 operation for operation: x = n + r by the magic-number addition, 2^r by the cubic, n added into the exponent
field. Its relative error must stay under what a 16-bit weight's own rounding hides (fp16: 2^-11 = 4.9e-4)."""
import re
from pathlib import Path

import numpy as np

SRC = Path(__file__).resolve().parent.parent / "nextsycl_b200" / "csrc" / "tc05.cuh"


def coefficients():
    """c3, c2, c1, c0 as the header holds them (the test follows the source, not a copy of its numbers)."""
    text = SRC.read_text()
    body = text[text.index("ex2_pair_fma"):]
    body = body[:body.index("\n}\n")]
    vals = [np.float32(v) for v in re.findall(r"pack2\((0\.\d+)f,", body)]
    assert len(vals) == 4, vals
    return vals


def ex2_cubic(x):
    f = np.float32
    c3, c2, c1, c0 = coefficients()
    x = np.maximum(x.astype(f), f(-125.0))
    magic = f(12582912.0)
    t = (x + magic).astype(f)                 # round(x) in the low mantissa bits
    n = (t - magic).astype(f)
    r = (x - n).astype(f)
    q = (c3 * r + c2).astype(f)
    q = (q * r + c1).astype(f)
    q = (q * r + c0).astype(f)
    bits = q.view(np.uint32) + (t.view(np.uint32) << np.uint32(23))
    return bits.view(f)


def test_cubic_is_within_a_16_bit_weights_rounding():
    x = np.linspace(-60.0, 8.0, 2_000_001).astype(np.float32)
    got = ex2_cubic(x).astype(np.float64)
    want = np.exp2(x.astype(np.float64))
    rel = np.abs(got / want - 1.0)
    assert rel.max() < 1.0e-4, rel.max()


def test_edges():
    f = np.float32
    x = np.array([0.0, -0.5, 0.5, -1.0, 8.0, -124.6, -125.0, -126.0, -1.0e4, -np.inf], f)
    got = ex2_cubic(x)
    assert np.all(np.isfinite(got)) and np.all(got > 0)
    assert abs(float(got[0]) - 1.0) < 1e-4 and abs(float(got[4]) - 256.0) < 256e-4
    # everything at or below -125 comes out as 2^-125: a weight of zero once rounded to 16 bits
    assert np.all(got[6:] == got[6]) and float(got[6]) < 3e-38
    assert np.float16(got[6]) == 0
