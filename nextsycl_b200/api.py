"""The loader of libnextsycl-llm.so: the Python mirror of the reference's `nextsycl_sys::Api`
(crates/sys/src/lib.rs:26-60, :138-151, :181-250).

The same search order - NEXTSYCL_LIB, else dist/ beside the package - the same flags (RTLD_NOW | RTLD_GLOBAL), one
function pointer per ns.h symbol bound at load with an error naming the missing one, and `symbol(name)` for the
engines' own tables, which bind by name and fail at first use (llm/qwen35/src/ffi.rs:72-86).

There is no CPU fallback: if the library is missing, `load()` raises.
"""
import ctypes as C
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

i64 = C.c_int64
vp = C.c_void_p

# the 26 symbols of include/ns.h, in the order crates/sys/src/lib.rs:200-236 binds them; ns_copy_2d is optional there
CORE = {
    "ns_last_error": (C.c_char_p, []),
    "ns_version": (C.c_char_p, []),
    "ns_gpu_count": (C.c_int, []),
    "ns_gpu_name": (C.c_int, [C.c_int, C.c_char_p, C.c_size_t]),
    "ns_gpu_pci": (C.c_int, [C.c_int, C.c_char_p, C.c_size_t]),
    "ns_gpu_units": (C.c_int, [C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "ns_gpu_open": (C.c_int, [C.c_int, C.POINTER(vp)]),
    "ns_gpu_close": (None, [vp]),
    "ns_gpu_queue": (vp, [vp]),
    "ns_gpu_memory": (C.c_int, [vp, C.POINTER(C.c_uint64), C.POINTER(i64)]),
    "ns_alloc": (C.c_int, [vp, C.c_size_t, C.POINTER(vp)]),
    "ns_free": (C.c_int, [vp, vp]),
    "ns_alloc_host": (C.c_int, [vp, C.c_size_t, C.POINTER(vp)]),
    "ns_free_host": (C.c_int, [vp, vp]),
    "ns_copy_to": (C.c_int, [vp, vp, vp, C.c_size_t]),
    "ns_copy_from": (C.c_int, [vp, vp, vp, C.c_size_t]),
    "ns_copy_dev": (C.c_int, [vp, vp, vp, C.c_size_t]),
    "ns_copy_2d": (C.c_int, [vp, vp, C.c_size_t, vp, C.c_size_t, C.c_size_t, C.c_size_t]),
    "ns_mark": (C.c_int, [vp, C.POINTER(i64)]),
    "ns_stream_copy": (C.c_int, [vp, vp, vp, C.c_size_t, C.POINTER(i64), C.c_int, C.c_int, C.POINTER(i64)]),
    "ns_await": (C.c_int, [vp, i64]),
    "ns_stamp": (C.c_int, [vp, C.POINTER(i64)]),
    "ns_elapsed": (C.c_int, [vp, i64, i64, C.POINTER(C.c_double)]),
    "ns_fill": (C.c_int, [vp, vp, C.c_uint8, C.c_size_t]),
    "ns_sync": (C.c_int, [vp]),
    "ns_copy_peer": (C.c_int, [vp, vp, vp, vp, C.c_size_t, vp]),
}

_ATTN_ARGS = [vp, vp, i64, vp, vp, i64, i64, i64, i64, i64, i64, vp]          # g q qs kc vc T Hq Hkv D cap p0 out
_SCRATCH_ARGS = [i64, i64, i64, i64, i64]                                      # T Hq Hkv D p0


class Seq(C.Structure):
    """ns_b200_seq (include/ns_attn.h): one sequence of a decode batch, as it lies in device memory."""
    _fields_ = [("kc", vp), ("vc", vp), ("cap", i64), ("p0", i64)]


# every attention symbol include/ns_attn.h declares: name -> (restype, argtypes)
ATTN = {
    "ns_q35_kv_store": (C.c_int, [vp, vp, i64, vp, i64, i64, i64, i64, i64, i64, vp, vp]),
    "ns_q35_attn_scratch": (i64, _SCRATCH_ARGS),
    "ns_q35_attn": (C.c_int, _ATTN_ARGS + [vp]),
    "ns_q35_attn_decode_supported": (C.c_int, [i64, i64, i64, i64]),
    "ns_q35_attn_decode_scratch": (i64, _SCRATCH_ARGS),
    "ns_q35_attn_decode": (C.c_int, _ATTN_ARGS + [vp]),
    "ns_q35_attn_decode_kv": (C.c_int, [vp, C.c_int] + _ATTN_ARGS[1:] + [vp]),
    "ns_nh_attn_scratch": (i64, _SCRATCH_ARGS),
    "ns_nh_attn": (C.c_int, _ATTN_ARGS + [vp]),
    "ns_nhs_attn_decode_supported": (C.c_int, [i64, i64, i64, i64]),
    "ns_nhs_attn_decode_scratch": (i64, _SCRATCH_ARGS),
    "ns_nhs_attn_decode": (C.c_int, _ATTN_ARGS + [vp]),
    "ns_q35_attn_prompt_supported": (C.c_int, [i64, i64, i64, i64]),
    "ns_q35_attn_prompt": (C.c_int, _ATTN_ARGS),
    "ns_q35_attn_prompt_kv": (C.c_int, [vp, C.c_int] + _ATTN_ARGS[1:]),
    "ns_nhs_attn_prompt_supported": (C.c_int, [i64, i64, i64, i64]),
    "ns_nhs_attn_prompt": (C.c_int, _ATTN_ARGS),
    "ns_b200_gqa_prefill": (C.c_int, [vp, C.c_int, vp, i64, vp, vp, i64, i64, i64, i64, i64, i64, vp]),
    "ns_b200_mla_prefill": (C.c_int, [vp, vp, i64, vp, i64, vp, i64, i64, i64, i64, C.c_float, vp]),
    "ns_ds2_mla_decode": (C.c_int, [vp, vp, vp, vp, vp, vp, i64, i64, i64, C.c_float]),
    "ns_ds2_mla_decode_q6k": (C.c_int, [vp, vp, vp, vp, vp, i64, i64, i64, C.c_float]),
    "ns_mla_attend": (C.c_int, [vp, vp, vp, vp, i64, i64, i64, i64, C.c_float]),
    "ns_mla_attend_sel": (C.c_int, [vp, vp, vp, vp, i64, i64, i64, i64, C.c_float, vp, vp, i64]),
    "ns_mla_attend_sel_q8": (C.c_int, [vp, vp, vp, vp, i64, i64, i64, i64, C.c_float, vp, vp, i64]),
    "ns_mla_cells": (C.c_int, [vp, vp, vp, i64, i64, i64, vp, vp, i64]),
    "ns_softmax_masked": (C.c_int, [vp, vp, i64, i64, i64, vp, C.c_float]),
    "ns_to_f16": (C.c_int, [vp, vp, vp, i64]),
    "ns_to_q8row": (C.c_int, [vp, vp, vp, i64, i64]),
    "ns_gather_q8_h": (C.c_int, [vp, vp, vp, vp, i64, i64]),
    "ns_gather_h": (C.c_int, [vp, vp, vp, vp, i64, i64]),
    "ns_gemm_batch_h": (C.c_int, [vp, i64, C.c_int, i64, i64, i64, vp, i64, i64, vp, i64, i64, vp, i64, i64, C.c_int]),
    "ns_q35_qk_norm_rope": (C.c_int, [vp, vp, i64, i64, vp, i64, i64, i64, i64, vp, C.c_float, i64, C.c_float, i64]),
    "ns_q35_qk_norm_rope_pos": (C.c_int, [vp, vp, i64, i64, vp, i64, i64, i64, i64, vp, C.c_float, i64, C.c_float, vp, i64, i64, i64]),
    "ns_q35_rope": (C.c_int, [vp, vp, i64, i64, vp, i64, i64, i64, i64, i64, C.c_float, i64]),
    "ns_b200_qkv_prepare": (C.c_int, [vp, vp, i64, vp, i64, vp, i64, i64, i64, i64, i64, vp, vp, C.c_float, i64, C.c_float, i64, i64, vp, vp, vp]),
    "ns_ds41_idx_score": (C.c_int, [vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64]),
    "ns_ds41_block_max": (C.c_int, [vp, vp, vp, i64, i64, i64, i64, i64, i64]),
    "ns_ds41_idx_score_cand": (C.c_int, [vp, vp, vp, vp, vp, i64, vp, i64, i64, i64, i64, i64, i64]),
    "ns_ds41_cand_pos": (C.c_int, [vp, vp, vp, vp, i64, i64, i64, i64]),
    "ns_ds41_cand_mask": (C.c_int, [vp, vp, vp, vp, i64, i64, i64, i64, i64]),
    "ns_ds41_kv_post": (C.c_int, [vp, vp, vp, i64, i64, C.c_float, i64, i64, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, vp, i64]),
    "ns_ds41_att_post": (C.c_int, [vp, vp, i64, i64, i64, i64, i64, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float]),
    "ns_ds2_rope": (C.c_int, [vp, vp, i64, i64, i64, i64, i64, i64, i64, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, vp, i64, i64]),
    "ns_ds2_kv_store": (C.c_int, [vp, vp, vp, C.c_float, vp, i64, i64, i64, i64, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float]),
    "ns_idx_pool": (C.c_int, [vp, vp, vp, vp, vp, vp, i64, i64, i64]),
    "ns_idx_score": (C.c_int, [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64]),
    "ns_topk": (C.c_int, [vp, vp, vp, i64, i64, i64, i64]),
    "ns_q35_attn_probs": (C.c_int, [vp, C.c_int, vp, vp, i64, i64, i64, i64, i64, C.c_int, vp, vp]),
    "ns_q35_kv_store_q": (C.c_int, [vp, C.c_int, vp, i64, vp, i64, i64, i64, i64, i64, i64, vp, vp]),
    "ns_q35_fwht32": (C.c_int, [vp, vp, i64, i64, i64]),
    "ns_ds41_attend": (C.c_int, [vp, vp, vp, i64, vp, i64, vp, i64, vp, vp, i64, i64, i64, i64, C.c_float]),
    "ns_ds41_attend_xmx_supported": (C.c_int, [i64, i64]),
    "ns_ds41_attend_xmx": (C.c_int, [vp, vp, vp, i64, vp, i64, vp, i64, vp, vp, i64, i64, i64, i64, C.c_float]),
    "ns_ds41_ring_put": (C.c_int, [vp, vp, vp, i64, i64, i64, i64]),
    "ns_ds41_rows_f16": (C.c_int, [vp, vp, vp, i64, i64, i64]),
    "ns_b200_mla_decode_scratch": (i64, [vp, i64, i64, i64]),
    "ns_b200_mla_decode": (C.c_int, [vp, vp, vp, i64, i64, i64, C.c_float, vp, vp]),
    "ns_b200_kv_store_batch": (C.c_int, [vp, vp, i64, i64, vp, i64, i64, vp, i64, i64, i64, i64]),
    "ns_b200_gqa_decode_scratch": (i64, [i64, i64, i64, i64, i64, i64]),
    "ns_b200_gqa_decode": (C.c_int, [vp, vp, i64, i64, vp, i64, i64, i64, i64, i64, i64, vp, vp]),
    "ns_q35_graph_begin": (C.c_int, [vp, C.POINTER(vp)]),
    "ns_q35_graph_end": (C.c_int, [vp, vp]),
    "ns_q35_graph_launch": (C.c_int, [vp, vp]),
    "ns_q35_graph_free": (None, [vp]),
    "ns_b200_kvsplit_mailbox_bytes": (i64, [i64, i64, i64, i64]),
    "ns_b200_kvsplit_scratch": (i64, [i64, i64, i64, i64, i64]),
    "ns_b200_kvsplit_decode": (C.c_int, [vp, vp, i64, vp, vp, i64, i64, i64, i64, i64, i64, i64, vp, i64, i64, vp, i64]),
    "ns_b200_kvsplit_partial": (C.c_int, [vp, vp, i64, vp, vp, i64, i64, i64, i64, i64, i64, i64, vp, vp]),
    "ns_b200_kvsplit_merge": (C.c_int, [vp, vp, i64, i64, i64, i64, vp]),
    "ns_b200_kvsplit_step": (C.c_int, [vp, vp, i64, vp, vp, i64, i64, i64, i64, i64, i64, i64, vp, i64, i64, vp, vp, i64, i64, vp]),
    "ns_b200_kvsplit_combine": (C.c_int, [vp, vp, i64, i64, i64, i64, i64, i64, vp]),
    "ns_b200_mla_kvsplit_scratch": (i64, [vp, i64, i64, i64]),
    "ns_b200_mla_kvsplit_decode": (C.c_int, [vp, vp, vp, i64, i64, i64, i64, i64, C.c_float, vp, i64, i64, vp, i64]),
    "ns_b200_mla_kvsplit_combine": (C.c_int, [vp, vp, i64, i64, i64, i64, i64, vp]),
    "ns_b200_ipc_export": (C.c_int, [vp, vp, vp]),
    "ns_b200_ipc_open": (C.c_int, [vp, vp, C.POINTER(vp)]),
    "ns_b200_ipc_close": (C.c_int, [vp, vp]),
    "ns_b200_gqa_decode_static": (C.c_int, [vp, vp, i64, i64, vp, i64, i64, i64, i64, i64, i64, vp]),
}


class LoadError(RuntimeError):
    pass


def library_path():
    """NEXTSYCL_LIB when set, else dist/libnextsycl-llm.so of this repository (crates/sys/src/lib.rs:138-151)."""
    return os.environ.get("NEXTSYCL_LIB") or os.path.join(ROOT, "dist", "libnextsycl-llm.so")


class Api:
    """One opened kernel library. Attributes are the bound functions (`api.ns_alloc(...)`)."""

    def __init__(self, path):
        self.path = path
        try:
            self.dll = C.CDLL(path, mode=os.RTLD_NOW | os.RTLD_GLOBAL)
        except OSError as e:
            raise LoadError(f"{path}: {e}") from e
        for name, (res, args) in CORE.items():
            self._bind(name, res, args, optional=(name == "ns_copy_2d"))
        for name, (res, args) in ATTN.items():
            self._bind(name, res, args, optional=True)   # engines' symbols: missing ones fail at first use

    def _bind(self, name, res, args, optional=False):
        try:
            f = getattr(self.dll, name)
        except AttributeError:
            if optional:
                return
            raise LoadError(f"{self.path}: {name} is missing") from None
        f.restype = res
        f.argtypes = args
        setattr(self, name, f)

    def symbol(self, name):
        """The address of `name`, or None (crates/sys/src/lib.rs:246-250)."""
        try:
            return C.cast(getattr(self.dll, name), vp).value
        except AttributeError:
            return None

    def need(self, name):
        """The bound function, or an error naming it (llm/qwen35/src/ffi.rs:76-79)."""
        f = getattr(self, name, None)
        if f is None:
            raise LoadError(f"{self.path}: {name} is missing")
        return f

    def last_error(self):
        m = self.ns_last_error()
        return m.decode("utf-8", "replace") if m else ""


_api = None


def load(path=None):
    """The process's library, opened once (crates/core/src/lib.rs:58-60)."""
    global _api
    if _api is None or (path and path != _api.path):
        _api = Api(path or library_path())
    return _api
