"""Writes tests/golden/oracle_kat.npz: small seeded inputs and the CPU oracle's outputs for them.

The reference holds no golden vectors for attention, so these are the repository's own known-answer set: they pin the
oracle (oracle/attn_oracle.cpp) against later edits, not the oracle against the reference. Run from the repository
root: `python tests/golden/make_golden.py`.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from nextsycl_b200 import workloads as W  # noqa: E402
from oracle import oracle as O  # noqa: E402


def cases():
    out = {}
    # GQA: (name, T, Hq, Hkv, D, kv)
    for name, T, Hq, Hkv, D, kv in [("gqa_a", 3, 8, 2, 128, 77), ("gqa_b", 1, 16, 2, 128, 300), ("gqa_c", 20, 4, 1, 128, 41), ("gqa_d", 2, 12, 2, 256, 130)]:
        q, k, v, p0 = W.gqa_case(900, T, Hq, Hkv, D, kv, cap=kv + 5, seq=len(out))
        qf = q.astype(np.float32)
        kb, vb = k.view(np.uint16), v.view(np.uint16)
        cap = kv + 5
        out[name + "_q"], out[name + "_k"], out[name + "_v"] = q, k, v
        out[name + "_meta"] = np.array([T, Hq, Hkv, D, cap, p0], np.int64)
        out[name + "_flash"] = O.gqa_flash_prefill(qf, kb, vb, T, Hq, Hkv, D, cap, p0)
        out[name + "_plain"] = O.gqa_plain(qf, kb, vb, T, Hq, Hkv, D, cap, p0)
        if T <= 8:
            out[name + "_flash_decode"] = O.gqa_flash_decode(qf, kb, vb, T, Hq, Hkv, D, cap, p0)
    # MLA 576-d
    for name, T, H, n in [("mla_a", 1, 8, 100), ("mla_b", 2, 16, 150)]:
        q = W.rng(901, len(out)).standard_normal((T, H, 576), dtype=np.float32)
        c = W.normal_f16(901, len(out) + 1, (n, 576), 0.5)
        out[name + "_q"], out[name + "_c"] = q, c
        out[name + "_meta"] = np.array([T, H, n - T], np.int64)
        sc = np.float32(1.0 / np.sqrt(192.0))
        out[name + "_fused"] = O.mla_fused(q, c.view(np.uint16), T, H, 512, 64, n - T, sc)
        out[name + "_gemm"] = O.mla_gemm(q, c.view(np.uint16), T, H, 512, 64, n - T, sc)
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_kat.npz")
    np.savez_compressed(path, **cases())
    print(path, os.path.getsize(path))
