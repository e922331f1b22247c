"""CPU-side checks of the drop-in boundary: the library loads the way the reference's loader opens it
(dlopen RTLD_NOW | RTLD_GLOBAL, crates/sys/src/lib.rs:181-187), exports every symbol include/*.h declares, and its
pure size queries answer without a device."""
import ctypes as C
import glob
import os
import re

import pytest

from nextsycl_b200 import api as A

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(h).read(), flags=re.S)
        names.update(re.findall(r"\b(ns_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol(api):
    missing = [n for n in declared_symbols() if api.symbol(n) is None]
    assert not missing, missing


def test_python_tables_cover_the_headers():
    declared = set(declared_symbols())
    bound = set(A.CORE) | set(A.ATTN)
    assert declared == bound, (sorted(declared - bound), sorted(bound - declared))


def test_core_symbols_are_the_reference_loader_set():
    # the 26 names crates/sys/src/lib.rs:200-236 binds
    assert len(A.CORE) == 26
    assert "ns_copy_peer" in A.CORE and "ns_stream_copy" in A.CORE


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(A.LoadError):
        A.Api(str(tmp_path / "libnextsycl-llm.so"))


def test_version_and_error_string(api):
    assert b"nextsycl" in api.ns_version()
    assert api.ns_last_error() is not None


def test_decode_supported_widened(api):
    f = api.ns_q35_attn_decode_supported
    assert f(1, 24, 4, 256) == 1        # the reference's own shape (silo/attn.cpp:402-404)
    assert f(1, 64, 8, 128) == 1 and f(4, 32, 4, 128) == 1 and f(8, 16, 4, 128) == 1
    assert f(9, 64, 8, 128) == 0 and f(0, 64, 8, 128) == 0
    assert f(1, 64, 8, 64) == 0 and f(1, 63, 8, 128) == 0


def test_decode_scratch_follows_each_rows_own_splits(api):
    """Scratch = T*Hq*ns*(D+2) floats with ns the largest split count of the rows, 0 when no row is split
    (the contract of kernels/llm/qwen35/silo/attn.cpp:406-410)."""
    f = api.ns_q35_attn_decode_scratch
    assert f(1, 64, 8, 128, 10) == 0              # 11 keys: one split
    s = f(1, 64, 8, 128, 32767)
    assert s > 0 and s % (64 * 130) == 0
    ns = s // (64 * 130)
    assert 32 <= ns <= 40                          # ~296 CTAs over 8 key heads
    s4 = f(4, 32, 4, 128, 262140)
    assert s4 % (4 * 32 * 130) == 0
    assert api.ns_b200_gqa_decode_scratch(8, 1, 64, 8, 128, 32768) == 8 * s


def test_seq_struct_layout():
    assert C.sizeof(A.Seq) == 32
