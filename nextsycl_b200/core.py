"""Device foundation: the Python mirror of the reference's `nextsycl_core` (crates/core/src/lib.rs): `Gpu`
(:133-156), `DevBuf` with its bounds checks (:217-304), `HostBuf`, and the bump `Arena` (:446-503).

Buffers are raw device pointers owned through the C ABI (ns_alloc / ns_free); host arrays are numpy. Nothing here
touches torch: the library's own streams carry the work, and `Gpu.sync()` is the only wait.
"""
import ctypes as C

import numpy as np

from . import api as _api


class Error(RuntimeError):
    """A failed library call; `is_no_room` as crates/core/src/lib.rs:39-43 classifies it."""

    @property
    def is_no_room(self):
        s = str(self)
        return "device allocation of" in s and "failed" in s


def check(api, rc, what):
    if rc != 0:
        raise Error(f"{what}: {api.last_error()}")


class Gpu:
    """One opened GPU: its own compute stream, two copy lanes, tickets."""

    def __init__(self, index=0, api=None):
        self.api = api or _api.load()
        self.index = index
        h = C.c_void_p()
        check(self.api, self.api.ns_gpu_open(index, C.byref(h)), f"opening GPU {index}")
        self.raw = h
        buf = C.create_string_buffer(256)
        check(self.api, self.api.ns_gpu_name(index, buf, 256), "naming the GPU")
        self.name = buf.value.decode()
        self.pci = buf.value.decode() if self.api.ns_gpu_pci(index, buf, 256) == 0 else None
        u, m = C.c_int(), C.c_int()
        check(self.api, self.api.ns_gpu_units(index, C.byref(u), C.byref(m)), "asking the GPU's units")
        self.units, self.mhz = u.value, m.value

    def close(self):
        if self.raw:
            self.api.ns_gpu_close(self.raw)
            self.raw = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def sync(self):
        check(self.api, self.api.ns_sync(self.raw), "waiting for the GPU")

    def memory(self):
        t, f = C.c_uint64(), C.c_int64()
        check(self.api, self.api.ns_gpu_memory(self.raw, C.byref(t), C.byref(f)), "asking the GPU's memory")
        return t.value, f.value

    def stamp(self):
        t = C.c_int64()
        check(self.api, self.api.ns_stamp(self.raw, C.byref(t)), "stamping")
        return t.value

    def elapsed_ns(self, t0, t1):
        ns = C.c_double()
        check(self.api, self.api.ns_elapsed(self.raw, t0, t1, C.byref(ns)), "reading stamps")
        return ns.value

    def record(self, fn):
        """Records what `fn` queues on the compute stream (it does not run) and returns a Graph to replay it."""
        h = C.c_void_p()
        check(self.api, self.api.need("ns_q35_graph_begin")(self.raw, C.byref(h)), "starting a recording")
        try:
            fn()
        finally:
            rc = self.api.need("ns_q35_graph_end")(self.raw, h)
        check(self.api, rc, "finishing a recording")
        return Graph(self, h)

    def stream(self):
        """The compute cudaStream_t as an integer (ns_gpu_queue returns a pointer to it)."""
        p = self.api.ns_gpu_queue(self.raw)
        return C.cast(p, C.POINTER(C.c_void_p))[0]


class Graph:
    """A recorded stretch of the compute stream (ns_q35_graph_*)."""

    def __init__(self, gpu, handle):
        self.gpu, self.h = gpu, handle

    def launch(self):
        check(self.gpu.api, self.gpu.api.ns_q35_graph_launch(self.gpu.raw, self.h), "replaying a recording")

    def free(self):
        if self.h:
            self.gpu.api.ns_q35_graph_free(self.h)
            self.h = None


class DevBuf:
    """Device memory of one GPU; a view (`view`) does not own it."""

    def __init__(self, gpu, nbytes, _ptr=None, _owner=None):
        self.gpu = gpu
        self.len = int(nbytes)
        if _ptr is None:
            p = C.c_void_p()
            check(gpu.api, gpu.api.ns_alloc(gpu.raw, self.len, C.byref(p)), "allocating device memory")
            self.ptr = p.value
            self.owned = True
        else:
            self.ptr = _ptr
            self.owned = False
            self._owner = _owner

    def free(self):
        if self.owned and self.ptr and self.gpu.raw:
            self.gpu.api.ns_free(self.gpu.raw, self.ptr)
        self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def bounds(self, at, n):
        if at < 0 or n < 0 or at + n > self.len:
            raise Error(f"bytes {at}..{at + n} of a {self.len}-byte buffer")

    def view(self, at, n):
        self.bounds(at, n)
        return DevBuf(self.gpu, n, _ptr=self.ptr + at, _owner=self)

    def write(self, arr, at=0):
        """Host array into the buffer at byte `at`, queued; the array must stay alive until the next sync."""
        a = np.ascontiguousarray(arr)
        self.bounds(at, a.nbytes)
        check(self.gpu.api, self.gpu.api.ns_copy_to(self.gpu.raw, self.ptr + at, a.ctypes.data, a.nbytes), "copying to the GPU")
        return a

    def read(self, dtype, count=None, at=0):
        """The buffer's bytes from `at` as a numpy array; waits."""
        dt = np.dtype(dtype)
        n = (self.len - at) // dt.itemsize if count is None else int(count)
        self.bounds(at, n * dt.itemsize)
        out = np.empty(n, dt)
        check(self.gpu.api, self.gpu.api.ns_copy_from(self.gpu.raw, out.ctypes.data, self.ptr + at, out.nbytes), "copying from the GPU")
        self.gpu.sync()
        return out

    def fill(self, v=0):
        check(self.gpu.api, self.gpu.api.ns_fill(self.gpu.raw, self.ptr, v, self.len), "filling")

    @classmethod
    def of(cls, gpu, arr):
        """A new buffer holding `arr` (waits for the copy)."""
        a = np.ascontiguousarray(arr)
        b = cls(gpu, max(1, a.nbytes))
        b.write(a)
        gpu.sync()
        return b


class HostBuf:
    """Pinned host memory (ns_alloc_host): the fast side of the GPU's copies, as a numpy array."""

    def __init__(self, gpu, nbytes):
        self.gpu = gpu
        self.len = int(nbytes)
        p = C.c_void_p()
        check(gpu.api, gpu.api.ns_alloc_host(gpu.raw, self.len, C.byref(p)), "allocating pinned memory")
        self.ptr = p.value
        self.bytes = np.ctypeslib.as_array(C.cast(self.ptr, C.POINTER(C.c_uint8)), shape=(self.len,))

    def array(self, dtype, shape=None, at=0):
        dt = np.dtype(dtype)
        n = (self.len - at) // dt.itemsize if shape is None else int(np.prod(shape))
        a = self.bytes[at:at + n * dt.itemsize].view(dt)
        return a if shape is None else a.reshape(shape)

    def free(self):
        if self.ptr and self.gpu.raw:
            self.bytes = None
            self.gpu.api.ns_free_host(self.gpu.raw, self.ptr)
        self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Arena:
    """A bump allocator over one device allocation, 256-byte aligned (crates/core/src/lib.rs:474-485); requests
    that do not fit get an allocation of their own and count as spills."""

    def __init__(self, gpu, nbytes):
        self.buf = DevBuf(gpu, nbytes)
        self.off = 0
        self.peak = 0
        self.spills = 0

    def bytes(self, n):
        at = (self.off + 255) // 256 * 256
        if at + n > self.buf.len:
            self.spills += 1
            return DevBuf(self.buf.gpu, n)
        self.off = at + n
        self.peak = max(self.peak, self.off)
        return self.buf.view(at, min(max(n, 1), self.buf.len - at))

    def f32(self, n):
        return self.bytes(n * 4)

    def reset(self):
        self.off = 0

    def mark(self):
        return self.off

    def rewind(self, mark):
        if mark < self.off:
            self.off = mark
