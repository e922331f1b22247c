"""nextsycl_b200: the attention path of nextsycl (causal GQA prefill, split-KV decode, absorbed MLA) as hand-written
sm_100a CUDA kernels behind the reference's own C ABI.

The product is dist/libnextsycl-llm.so (sources in nextsycl_b200/csrc, headers in include/). This package is the
host-side mirror of the reference's Rust foundation for tests, benchmarks and Python callers:

  api   - the dlopen/dlsym loader (crates/sys)
  core  - Gpu, DevBuf, HostBuf, Arena (crates/core)
  ops   - bounds-checked wrappers over the attention entry points (the engines' ops.rs / call sites)
  build - compiles the library with nvcc for sm_100a
"""
from . import api, core, ops  # noqa: F401
from .core import Arena, DevBuf, Error, Gpu, HostBuf  # noqa: F401
from .ops import Ops  # noqa: F401
