"""Bounds-checked wrappers over the attention entry points: the engine side of the boundary, in the manner of the
reference's `ops.rs` (`need!` size checks before every FFI call, llm/glm5next/src/ops.rs:20-26; the qwen35 engine's
call sites llm/qwen35/src/engine.rs:1577-1608).

Every method takes `DevBuf`s, checks that the kernel's reads and writes fit them, queues the call on the GPU's compute
stream and returns; `gpu.sync()` waits. A failing call raises `core.Error` with the library's message.
"""
import ctypes as C

import numpy as np

from . import api as _api
from .core import DevBuf, Error, check


def _need(buf, nbytes, what):
    if buf is None or buf.len < nbytes:
        raise Error(f"{what}: {nbytes} bytes needed, the buffer holds {0 if buf is None else buf.len}")


class Ops:
    def __init__(self, gpu):
        self.gpu = gpu
        self.api = gpu.api

    # ---- caches -------------------------------------------------------------------------------------------------
    def kv_store(self, k, ks, v, vs, T, Hkv, D, cap, p0, kc, vc):
        """fp32 rows k, v [T][Hkv*D] into the fp16 caches at p0.. (ns_q35_kv_store)."""
        _need(k, ((T - 1) * ks + Hkv * D) * 4, "kv_store k")
        _need(v, ((T - 1) * vs + Hkv * D) * 4, "kv_store v")
        _need(kc, Hkv * cap * D * 2, "kv_store key cache")
        _need(vc, Hkv * cap * D * 2, "kv_store value cache")
        check(self.api, self.api.need("ns_q35_kv_store")(self.gpu.raw, k.ptr, ks, v.ptr, vs, T, Hkv, D, cap, p0, kc.ptr, vc.ptr), "kv_store")

    # ---- GQA decode, the reference's call (fp32 in and out, one sequence) ------------------------------------------
    def attn_decode_supported(self, T, Hq, Hkv, D):
        return bool(self.api.need("ns_q35_attn_decode_supported")(T, Hq, Hkv, D))

    def attn_decode_scratch(self, T, Hq, Hkv, D, p0):
        return int(self.api.need("ns_q35_attn_decode_scratch")(T, Hq, Hkv, D, p0))

    def attn_decode(self, q, qs, kc, vc, T, Hq, Hkv, D, cap, p0, out, scratch=None, name="ns_q35_attn_decode"):
        _need(q, ((T - 1) * qs + Hq * D) * 4, "attn_decode q")
        _need(kc, Hkv * cap * D * 2, "attn_decode key cache")
        _need(vc, Hkv * cap * D * 2, "attn_decode value cache")
        _need(out, T * Hq * D * 4, "attn_decode out")
        sc = int(self.api.need(name + "_scratch")(T, Hq, Hkv, D, p0))
        if sc > 0:
            _need(scratch, sc * 4, "attn_decode scratch")
        check(self.api, self.api.need(name)(self.gpu.raw, q.ptr, qs, kc.ptr, vc.ptr, T, Hq, Hkv, D, cap, p0, out.ptr,
                                            scratch.ptr if scratch is not None else None), name)

    def attn(self, q, qs, kc, vc, T, Hq, Hkv, D, cap, p0, out, scratch=None, name="ns_q35_attn"):
        """Any number of rows (ns_q35_attn / ns_nh_attn)."""
        _need(q, ((T - 1) * qs + Hq * D) * 4, "attn q")
        _need(kc, Hkv * cap * D * 2, "attn key cache")
        _need(vc, Hkv * cap * D * 2, "attn value cache")
        _need(out, T * Hq * D * 4, "attn out")
        sc = int(self.api.need(name + "_scratch")(T, Hq, Hkv, D, p0))
        if sc > 0:
            _need(scratch, sc * 4, "attn scratch")
        check(self.api, self.api.need(name)(self.gpu.raw, q.ptr, qs, kc.ptr, vc.ptr, T, Hq, Hkv, D, cap, p0, out.ptr,
                                            scratch.ptr if scratch is not None else None), name)

    # ---- GQA decode, native: a batch of sequences, fp16 in and out -------------------------------------------------
    def seq_table(self, seqs):
        """The device array of ns_b200_seq for [(kc, vc, cap, p0), ...] (DevBufs and ints); waits for the copy."""
        arr = (_api.Seq * len(seqs))()
        for i, (kc, vc, cap, p0) in enumerate(seqs):
            arr[i] = _api.Seq(kc.ptr, vc.ptr, cap, p0)
        host = np.frombuffer(bytes(arr), dtype=np.uint8)
        return DevBuf.of(self.gpu, host)

    def gqa_decode_scratch(self, B, T, Hq, Hkv, D, max_kv):
        return int(self.api.need("ns_b200_gqa_decode_scratch")(B, T, Hq, Hkv, D, max_kv))

    def gqa_decode(self, q, qs, q_seq, table, B, T, Hq, Hkv, D, max_kv, out, scratch=None):
        _need(q, ((B - 1) * q_seq + (T - 1) * qs + Hq * D) * 2, "gqa_decode q")
        _need(table, B * C.sizeof(_api.Seq), "gqa_decode sequence table")
        _need(out, B * T * Hq * D * 2, "gqa_decode out")
        sc = self.gqa_decode_scratch(B, T, Hq, Hkv, D, max_kv)
        if sc > 0:
            _need(scratch, sc * 4, "gqa_decode scratch")
        check(self.api, self.api.need("ns_b200_gqa_decode")(self.gpu.raw, q.ptr, qs, q_seq, table.ptr, B, T, Hq, Hkv, D, max_kv, out.ptr,
                                                            scratch.ptr if scratch is not None else None), "ns_b200_gqa_decode")
