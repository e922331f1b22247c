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

    def kv_store_batch(self, k, ks, k_seq, v, vs, v_seq, table, B, T, Hkv, D):
        """fp32 rows k, v [B][T][Hkv*D] into each sequence's caches at its own p0.. in one launch (ns_b200_kv_store_batch)."""
        _need(k, ((B - 1) * k_seq + (T - 1) * ks + Hkv * D) * 4, "kv_store_batch k")
        _need(v, ((B - 1) * v_seq + (T - 1) * vs + Hkv * D) * 4, "kv_store_batch v")
        _need(table, B * C.sizeof(_api.Seq), "kv_store_batch sequence table")
        check(self.api, self.api.need("ns_b200_kv_store_batch")(self.gpu.raw, k.ptr, ks, k_seq, v.ptr, vs, v_seq, table.ptr, B, T, Hkv, D),
              "ns_b200_kv_store_batch")

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

    # ---- prompt attention -------------------------------------------------------------------------------------------
    def attn_prompt_supported(self, T, Hq, Hkv, D):
        return bool(self.api.need("ns_q35_attn_prompt_supported")(T, Hq, Hkv, D))

    def attn_prompt(self, q, qs, kc, vc, T, Hq, Hkv, D, cap, p0, out, name="ns_q35_attn_prompt"):
        """fp32 rows in and out against the fp16 caches (ns_q35_attn_prompt / ns_nhs_attn_prompt)."""
        _need(q, ((T - 1) * qs + Hq * D) * 4, "attn_prompt q")
        _need(kc, Hkv * cap * D * 2, "attn_prompt key cache")
        _need(vc, Hkv * cap * D * 2, "attn_prompt value cache")
        _need(out, T * Hq * D * 4, "attn_prompt out")
        check(self.api, self.api.need(name)(self.gpu.raw, q.ptr, qs, kc.ptr, vc.ptr, T, Hq, Hkv, D, cap, p0, out.ptr), name)

    def gqa_prefill(self, dtype, q, qs, kc, vc, T, Hq, Hkv, D, cap, p0, out):
        """16-bit rows in and out (dtype 0 fp16, 1 bf16)."""
        _need(q, ((T - 1) * qs + Hq * D) * 2, "gqa_prefill q")
        _need(kc, Hkv * cap * D * 2, "gqa_prefill key cache")
        _need(vc, Hkv * cap * D * 2, "gqa_prefill value cache")
        _need(out, T * Hq * D * 2, "gqa_prefill out")
        check(self.api, self.api.need("ns_b200_gqa_prefill")(self.gpu.raw, dtype, q.ptr, qs, kc.ptr, vc.ptr, T, Hq, Hkv, D, cap, p0, out.ptr),
              "ns_b200_gqa_prefill")

    def mla_prefill(self, q, q_tok, k, k_tok, v, v_tok, T, H, p0, scale, out):
        """bf16 q [T][H][192], k [p0+T][H][192], v [p0+T][H][128] -> out [T][H][128]."""
        n = p0 + T
        _need(q, ((T - 1) * q_tok + H * 192) * 2, "mla_prefill q")
        _need(k, ((n - 1) * k_tok + H * 192) * 2, "mla_prefill k")
        _need(v, ((n - 1) * v_tok + H * 128) * 2, "mla_prefill v")
        _need(out, T * H * 128 * 2, "mla_prefill out")
        check(self.api, self.api.need("ns_b200_mla_prefill")(self.gpu.raw, q.ptr, q_tok, k.ptr, k_tok, v.ptr, v_tok, T, H, p0, scale, out.ptr),
              "ns_b200_mla_prefill")

    # ---- absorbed MLA decode ----------------------------------------------------------------------------------------
    def mla_decode_scratch(self, T, H, pos0):
        return int(self.api.need("ns_b200_mla_decode_scratch")(self.gpu.raw, T, H, pos0))

    def mla_decode(self, q, cache, T, H, pos0, scale, out, scratch=None):
        """q fp16 [T][H][576], cache fp16 [n][576] -> out fp32 [T][H][512] (the middle stage of deepseek2's MLA)."""
        _need(q, T * H * 576 * 2, "mla_decode q")
        _need(cache, (pos0 + T) * 576 * 2, "mla_decode cache")
        _need(out, T * H * 512 * 4, "mla_decode out")
        sc = self.mla_decode_scratch(T, H, pos0)
        if sc > 0:
            _need(scratch, sc * 4, "mla_decode scratch")
        check(self.api, self.api.need("ns_b200_mla_decode")(self.gpu.raw, q.ptr, cache.ptr, T, H, pos0, scale, out.ptr,
                                                            scratch.ptr if scratch is not None else None), "ns_b200_mla_decode")

    def ds2_mla_decode(self, q, kb, vb, cache, out, T, H, pos0, scale):
        """deepseek2's whole decode attention: q fp32 [T][H][192], k_b [H][512][128], v_b [H][128][512] fp16 -> out fp32 [T][H][128]."""
        _need(q, T * H * 192 * 4, "ds2_mla_decode q")
        _need(kb, H * 512 * 128 * 2, "ds2_mla_decode k_b")
        _need(vb, H * 128 * 512 * 2, "ds2_mla_decode v_b")
        _need(cache, (pos0 + T) * 576 * 2, "ds2_mla_decode cache")
        _need(out, T * H * 128 * 4, "ds2_mla_decode out")
        check(self.api, self.api.need("ns_ds2_mla_decode")(self.gpu.raw, q.ptr, kb.ptr, vb.ptr, cache.ptr, out.ptr, T, H, pos0, scale), "ns_ds2_mla_decode")
