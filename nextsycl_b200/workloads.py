"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

The reference measures attention inside whole-model runs and names no dataset for this path; these tensors are the
workload. Every tensor has its own counter-based generator, seed = 0x6E73 + 1000*config + tensor id; values are drawn
as fp32 N(0, sigma) and rounded to the storage type, and the rounded values are what both the kernels and the checker
receive.
"""
import numpy as np


def rng(config, tensor):
    return np.random.Generator(np.random.Philox(0x6E73 + 1000 * int(config) + int(tensor)))


def normal_f16(config, tensor, shape, sigma=1.0):
    """fp16 array of N(0, sigma) values."""
    x = rng(config, tensor).standard_normal(shape, dtype=np.float32)
    if sigma != 1.0:
        x *= np.float32(sigma)
    return x.astype(np.float16)


def normal_f32(config, tensor, shape, sigma=1.0):
    """fp32 array of N(0, sigma) values."""
    x = rng(config, tensor).standard_normal(shape, dtype=np.float32)
    if sigma != 1.0:
        x *= np.float32(sigma)
    return x


def normal_bf16_bits(config, tensor, shape, sigma=1.0):
    """bf16 bit patterns (uint16) of N(0, sigma) values, round to nearest even."""
    x = rng(config, tensor).standard_normal(shape, dtype=np.float32)
    if sigma != 1.0:
        x *= np.float32(sigma)
    w = x.view(np.uint32).astype(np.uint64)
    w = w + 0x7FFF + ((w >> 16) & 1)
    return (w >> 16).astype(np.uint16)


def gqa_case(config, T, Hq, Hkv, D, kv, cap=None, seq=0):
    """q fp16 [T, Hq*D], K and V caches fp16 [Hkv, cap, D] filled up to kv (zeros after), p0 = kv - T."""
    cap = cap or kv
    q = normal_f16(config, 10 * seq + 0, (T, Hq * D))
    k = np.zeros((Hkv, cap, D), np.float16)
    v = np.zeros((Hkv, cap, D), np.float16)
    k[:, :kv] = normal_f16(config, 10 * seq + 1, (Hkv, kv, D))
    v[:, :kv] = normal_f16(config, 10 * seq + 2, (Hkv, kv, D))
    return q, k, v, kv - T
