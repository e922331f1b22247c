"""The ns.h core on a real GPU: memory, ordered copies, tickets, stamps and the error convention
(kernels/ns/ns.h:18-56 semantics)."""
import ctypes as C

import numpy as np
import pytest

from nextsycl_b200 import Arena, DevBuf, Error, HostBuf

pytestmark = pytest.mark.gpu


def test_device_is_a_b200_class_gpu(api, gpu):
    assert api.ns_gpu_count() >= 1
    assert gpu.units >= 100 and gpu.mhz > 0
    total, free = gpu.memory()
    assert total > 100 << 30 and 0 < free <= total
    assert gpu.stream() is not None


def test_copy_round_trip_and_fill(gpu):
    x = np.arange(1 << 20, dtype=np.float32)
    b = DevBuf.of(gpu, x)
    assert np.array_equal(b.read(np.float32), x)
    b.fill(0)
    assert not b.read(np.float32).any()
    c = DevBuf(gpu, x.nbytes)
    b.write(x)
    from nextsycl_b200.core import check
    check(gpu.api, gpu.api.ns_copy_dev(gpu.raw, c.ptr, b.ptr, x.nbytes), "copy_dev")
    assert np.array_equal(c.read(np.float32), x)


def test_copy_2d(gpu):
    src = np.arange(64 * 48, dtype=np.uint8).reshape(64, 48)
    a = DevBuf.of(gpu, src)
    b = DevBuf(gpu, 64 * 32)
    from nextsycl_b200.core import check
    check(gpu.api, gpu.api.ns_copy_2d(gpu.raw, b.ptr, 32, a.ptr, 48, 20, 64), "copy_2d")
    got = b.read(np.uint8).reshape(64, 32)[:, :20]
    assert np.array_equal(got, src[:, :20])


def test_pinned_host_memory_and_lanes(gpu):
    h = HostBuf(gpu, 1 << 20)
    h.array(np.uint8)[:] = 7
    d = DevBuf(gpu, 1 << 20)
    t0, t1 = C.c_int64(), C.c_int64()
    api = gpu.api
    assert api.ns_mark(gpu.raw, C.byref(t0)) == 0
    deps = (C.c_int64 * 1)(t0.value)
    assert api.ns_stream_copy(gpu.raw, d.ptr, h.ptr, 1 << 20, deps, 1, 0, C.byref(t1)) == 0
    assert api.ns_await(gpu.raw, t1.value) == 0
    assert (d.read(np.uint8) == 7).all()
    assert api.ns_stream_copy(gpu.raw, d.ptr, h.ptr, 16, deps, 1, 2, C.byref(t1)) == -1
    assert "lane" in api.last_error()
    assert api.ns_await(gpu.raw, 1 << 40) == -1
    h.free()


def test_stamps_measure_time(gpu):
    d = DevBuf(gpu, 256 << 20)
    a = gpu.stamp()
    d.fill(1)
    b = gpu.stamp()
    ns = gpu.elapsed_ns(a, b)
    assert 1e3 < ns < 1e9


def test_allocation_failure_is_no_room(gpu):
    with pytest.raises(Error) as e:
        DevBuf(gpu, 1 << 50)
    assert e.value.is_no_room
    # the context is still usable
    assert DevBuf.of(gpu, np.ones(4, np.float32)).read(np.float32).sum() == 4


def test_arena_alignment_and_spill(gpu):
    a = Arena(gpu, 4096)
    x = a.bytes(10)
    y = a.f32(100)
    assert (y.ptr - x.ptr) == 256 and a.peak == 256 + 400
    m = a.mark()
    z = a.bytes(8192)
    assert a.spills == 1 and z.owned
    a.rewind(m)
    assert a.mark() == m
    with pytest.raises(Error):
        x.bounds(0, 11)


def test_errors_are_per_call_and_null_gpu_is_rejected(api):
    assert api.ns_sync(None) == -1
    assert "no gpu" in api.last_error()
    out = C.c_void_p()
    assert api.ns_gpu_open(10_000, C.byref(out)) == -1
    assert "no GPU" in api.last_error()


def test_a_ticket_older_than_the_ring_is_refused(gpu):
    """Tickets index a ring of 65,536 events (kernels/ns/ns_internal.hpp:14): a ticket more than a ring older than the newest
    names an event slot a newer mark has taken, so it is refused instead of standing for that newer event."""
    api = gpu.api
    first, t = C.c_int64(), C.c_int64()
    assert api.ns_mark(gpu.raw, C.byref(first)) == 0
    for _ in range(65536):
        assert api.ns_mark(gpu.raw, C.byref(t)) == 0
    gpu.sync()
    assert api.ns_await(gpu.raw, t.value) == 0
    assert api.ns_await(gpu.raw, first.value) == -1 and "older" in api.last_error()
    ns = C.c_double()
    assert api.ns_elapsed(gpu.raw, first.value, t.value, C.byref(ns)) == -1
    assert api.ns_elapsed(gpu.raw, t.value - 5, t.value, C.byref(ns)) == 0 and ns.value >= 0
