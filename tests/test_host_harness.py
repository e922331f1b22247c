"""The C++ stand-in for the reference's Rust loader (host/): it opens the library with dlopen(RTLD_NOW | RTLD_GLOBAL) and
binds every core and engine symbol by name, the way crates/sys and the engines' ffi.rs tables do. The reference's own
host language cannot be compiled here (no Rust toolchain), so this is the check that the C ABI is complete."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build(tmp_path):
    exe = str(tmp_path / "dlopen_check")
    env = {k: v for k, v in os.environ.items() if k not in ("CXX", "CC")}
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-Wall", "-o", exe, os.path.join(ROOT, "host", "dlopen_check.cpp"), "-ldl"], env=env)
    return exe


def test_every_symbol_binds_by_name(tmp_path):
    exe = build(tmp_path)
    r = subprocess.run([exe, os.path.join(ROOT, "dist", "libnextsycl-llm.so")], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 missing" in r.stdout


def test_missing_library_is_an_error(tmp_path):
    exe = build(tmp_path)
    r = subprocess.run([exe, str(tmp_path / "nothing.so")], capture_output=True, text=True)
    assert r.returncode == 2 and "error" in r.stdout


@pytest.mark.gpu
def test_round_trip_through_the_cpp_foundation(tmp_path):
    exe = build(tmp_path)
    r = subprocess.run([exe, os.path.join(ROOT, "dist", "libnextsycl-llm.so"), "--run"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "round trip ok" in r.stdout
