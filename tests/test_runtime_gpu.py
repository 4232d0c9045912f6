"""Vendor runtime on a real device: devapis primitives, stream / event pools and the caching allocator
(semantics pinned by dipu/tests/python/individual_scripts/test_memory_stats.py:6-82, test_allocator.py:6-90,
test_rt_tensor.py:109-124, unittests/test_get_device_properties.py:5-13)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_device_queries(devapis):
    assert devapis.getDeviceCount() >= 1
    p = devapis.getDeviceProperties(0)
    assert p.name.decode().startswith("NVIDIA") and p.major >= 10 and p.multiProcessorCount > 0 and p.totalGlobalMem >= 256 << 20
    free, total = devapis.getDeviceStatus(0)
    assert 0 < free <= total
    devapis.setDevice(0)
    assert devapis.current_device() == 0
    assert devapis.getDriverVersion() > 0 and devapis.getRuntimeVersion() > 0
    devapis.checkLastError()


def test_streams_events_copies(devapis):
    devapis.setDevice(0)
    s = devapis.createStream()
    assert devapis.streamNotNull(s) and not devapis.streamNotNull(None)
    e0, e1 = devapis.createEvent(), devapis.createEvent()
    n = 64 << 20
    st, d0 = devapis.mallocDevice(n)
    st2, d1 = devapis.mallocDevice(n)
    assert st == devapis.OpStatus.SUCCESS and st2 == devapis.OpStatus.SUCCESS
    h = devapis.mallocHost(n)
    assert devapis.isPinnedPtr(h)
    ctypes.memset(h, 0x5a, n)
    devapis.recordEvent(e0, s)
    devapis.memCopyH2DAsync(s, n, d0, h)
    devapis.memCopyD2DAsync(s, n, 0, d1, 0, d0)
    devapis.memSetAsync(s, d0, 0, n)
    devapis.recordEvent(e1, s)
    devapis.waitEvent(e1)
    assert devapis.getEventStatus(e1) == devapis.EventStatus.READY
    assert devapis.eventElapsedTime(e0, e1) > 0
    assert devapis.isStreamEmpty(s)
    back = (ctypes.c_ubyte * 16)()
    devapis.memCopyD2H(16, ctypes.addressof(back), d1)
    assert bytes(back) == b"\x5a" * 16
    devapis.memCopyD2H(16, ctypes.addressof(back), d0)
    assert bytes(back) == b"\x00" * 16
    s2 = devapis.getStreamFromPool(0)
    devapis.streamWaitEvent(s2, e1)
    devapis.syncStream(s2)
    assert devapis.getDefaultStream(0) == devapis.getDefaultStream(0)
    pool = {devapis.getStreamFromPool(0) for _ in range(16)}
    assert len(pool) == 8  # eight pool streams handed out round-robin
    ev = devapis.getEventFromPool()
    devapis.restoreEventToPool(ev)
    assert devapis.getEventFromPool() == ev  # recycled
    devapis.restoreEventToPool(ev)
    devapis.freeDevice(d0)
    devapis.freeDevice(d1)
    devapis.freeHost(h)
    devapis.destroyEvent(e0)
    devapis.destroyEvent(e1)
    devapis.destroyStream(s)


def test_large_async_copies_of_ragged_size_arrive_bit_exact(devapis):
    """memCopyH2DAsync / memCopyD2HAsync issue a transfer above 1 MiB as a train of 256 KiB pieces: a size that is no multiple
    of the piece (and an odd one) must arrive whole, from pinned and from pageable host memory, at an offset into both buffers."""
    devapis.setDevice(0)
    s = devapis.createStream()
    # 3 MiB + 12345: pieces of 256 KiB; 17 MiB + 7: more than 64 such pieces, so the pieces grow to a sixty-fourth of the transfer
    for n, pinned in (((3 << 20) + 12345, True), ((3 << 20) + 12345, False), ((17 << 20) + 7, True)):
        src = torch.randint(0, 256, (n + 64,), dtype=torch.uint8)
        h_in = src.pin_memory() if pinned else src.clone()
        h_out = torch.zeros(n + 64, dtype=torch.uint8)
        h_out = h_out.pin_memory() if pinned else h_out
        st, d = devapis.mallocDevice(n + 64)
        assert st == devapis.OpStatus.SUCCESS
        devapis.memSetAsync(s, d, 0, n + 64)
        devapis.memCopyH2DAsync(s, n, d + 16, h_in.data_ptr() + 3)
        devapis.memCopyD2HAsync(s, n, h_out.data_ptr() + 5, d + 16)
        devapis.syncStream(s)
        assert torch.equal(h_out[5:5 + n], h_in[3:3 + n])
        assert int(h_out[:5].sum()) == 0 and int(h_out[5 + n:].sum()) == 0  # nothing written beyond the requested bytes
        devapis.freeDevice(d)
    devapis.destroyStream(s)


def test_malloc_device_reports_nomem_without_raising(devapis):
    devapis.setDevice(0)
    _, total = devapis.getDeviceStatus(0)
    st, p = devapis.mallocDevice(total * 4, throwExcepion=False)  # larger than the device: refused by the driver up front
    assert st == devapis.OpStatus.ERR_NOMEM and p is None
    devapis.checkLastError()  # the error state was cleared
    with pytest.raises(devapis.VendorError):
        devapis.mallocDevice(total * 4)


def test_caching_allocator_on_device(devapis):
    A = devapis.CachingAllocator
    A.useFakeBackend(0)  # make sure the CUDA backend is active
    devapis.setDevice(0)
    s = devapis.getDefaultStream(0)
    A.emptyCache()
    base = A.stats(0)
    ptrs = []
    expect = 0
    for numel in (1, 100, 1000, 300000, 5 << 20, 40 << 20):
        nbytes = 4 * numel
        ptrs.append(A.allocate(nbytes, 0, s))
        expect += ((nbytes - 1) | 511) + 1
        st = A.stats(0)
        assert st["allocated_bytes"] - base["allocated_bytes"] >= expect - 0  # rounded to 512 B, never less
        assert st["reserved_bytes"] >= st["allocated_bytes"]
    # memory is usable
    torch.cuda.synchronize()
    devapis.memSetAsync(s, ptrs[-1], 1, 160 << 20)
    devapis.syncStream(s)
    for p in ptrs:
        A.free(p)
    st = A.stats(0)
    assert st["allocated_bytes"] == base["allocated_bytes"] and st["reserved_bytes"] > 0
    # a second round of the same sizes is served from the cache
    mallocs = st["num_device_mallocs"]
    again = [A.allocate(4 * n, 0, s) for n in (1, 100, 1000, 300000, 5 << 20, 40 << 20)]
    assert A.stats(0)["num_device_mallocs"] == mallocs
    for p in again:
        A.free(p)
    # cross-stream use defers the reuse until the other stream's work is done
    p = A.allocate(1 << 20, 0, s)
    other = devapis.getStreamFromPool(0)
    A.recordStream(p, other)
    A.free(p)
    devapis.syncStream(other)
    q = A.allocate(1 << 20, 0, s)
    A.free(q)
    A.emptyCache()
    assert A.stats(0)["reserved_bytes"] == 0
    assert A.stats(0)["allocated_bytes_peak"] >= expect
    A.resetPeakStats(0)
    assert A.stats(0)["allocated_bytes_peak"] == 0


def test_allocator_every_small_size(devapis):
    # dipu/tests/python/individual_scripts/test_allocator.py:6-90 sweeps 0..32 KiB byte by byte; a stride keeps this quick
    A = devapis.CachingAllocator
    devapis.setDevice(0)
    s = devapis.getDefaultStream(0)
    live = []
    for n in list(range(0, 2050)) + list(range(2050, 32768, 97)):
        p = A.allocate(n, 0, s)
        if n == 0:
            assert p is None
        else:
            assert p % 512 == 0
            live.append(p)
        if len(live) > 64:
            A.free(live.pop(0))
    for p in live:
        A.free(p)
    hp = devapis.CachingHostAllocator.allocate(1000)
    assert devapis.isPinnedPtr(hp)
    devapis.CachingHostAllocator.recordStream(hp, s)
    devapis.CachingHostAllocator.free(hp)
    devapis.CachingHostAllocator.emptyCache()
    A.emptyCache()


def _fill_and_check(devapis, stream, ptr, nbytes, value):
    devapis.memSetAsync(stream, ptr, value, nbytes)
    devapis.syncStream(stream)
    for off in (0, nbytes // 2 - 8, nbytes - 16):
        back = (ctypes.c_ubyte * 16)()
        devapis.memCopyD2H(16, ctypes.addressof(back), ptr + off)
        assert bytes(back) == bytes([value]) * 16


def test_expandable_segment_maps_and_unmaps_pages(devapis):
    """The vendor's ExpandableSegment on the real driver: address reservation, page-wise map / unmap, data survives growth."""
    MiB = 1 << 20
    devapis.setDevice(0)
    s = devapis.getDefaultStream(0)
    seg = devapis.ExpandableSegment(0, s, 2 * MiB)
    try:
        base = seg.ptr()
        assert base and base % (2 * MiB) == 0 and seg.size() >= devapis.getDeviceProperties(0).totalGlobalMem
        assert seg.mappedBytes() == 0
        p, n = seg.map(base, 5 * MiB)                 # three 2 MiB pages
        assert p == base and n == 6 * MiB and seg.mappedBytes() == 6 * MiB
        _fill_and_check(devapis, s, base, 6 * MiB, 0x11)
        p2, n2 = seg.map(base + 6 * MiB, 2 * MiB)     # grow at the end: the old pages keep their content
        assert p2 == base + 6 * MiB and n2 == 2 * MiB
        _fill_and_check(devapis, s, base + 6 * MiB, 2 * MiB, 0x22)
        back = (ctypes.c_ubyte * 16)()
        devapis.memCopyD2H(16, ctypes.addressof(back), base + 6 * MiB - 16)
        assert bytes(back) == b"\x11" * 16
        # a copy that crosses a page boundary
        h = devapis.mallocHost(4 * MiB)
        ctypes.memset(h, 0x33, 4 * MiB)
        devapis.memCopyH2D(4 * MiB, base + 3 * MiB, h)
        devapis.memCopyD2H(16, ctypes.addressof(back), base + 5 * MiB)
        assert bytes(back) == b"\x33" * 16
        devapis.freeHost(h)
        # unmap: only whole pages inside the range go away
        p3, n3 = seg.unmap(base + 1 * MiB, 4 * MiB)   # covers page 1 wholly, pages 0 and 2 partly
        assert p3 == base + 2 * MiB and n3 == 2 * MiB and seg.mappedBytes() == 6 * MiB
        p4, n4 = seg.unmap(base + 1 * MiB, 512 * 1024)
        assert n4 == 0
        p5, n5 = seg.map(base + 2 * MiB, 2 * MiB)     # the hole can be mapped again
        assert p5 == base + 2 * MiB and n5 == 2 * MiB
        _fill_and_check(devapis, s, base, 8 * MiB, 0x44)
    finally:
        seg.close()
    devapis.checkLastError()


def test_caching_allocator_with_expandable_segments(devapis):
    """expandable_segments:True on the device: blocks of one growing segment hold their data, free pages go back."""
    MiB = 1 << 20
    A = devapis.CachingAllocator
    devapis.setDevice(0)
    s = devapis.createStream()
    A.emptyCache()
    before = A.stats(0)["reserved_bytes"]
    A.configure("expandable_segments:True")
    try:
        a = A.allocate(30 * MiB, 0, s)
        b = A.allocate(50 * MiB, 0, s)
        assert b == a + 30 * MiB                       # same segment, contiguous
        assert A.stats(0)["reserved_bytes"] - before == 80 * MiB
        devapis.memSetAsync(s, a, 0x5c, 30 * MiB)
        devapis.memSetAsync(s, b, 0xa7, 50 * MiB)
        c = A.allocate(100 * MiB, 0, s)                # grows the segment by five more pages
        assert c == b + 50 * MiB
        devapis.memSetAsync(s, c, 0x01, 100 * MiB)
        devapis.syncStream(s)
        back = (ctypes.c_ubyte * 16)()
        for ptr, n, val in ((a, 30 * MiB, 0x5c), (b, 50 * MiB, 0xa7), (c, 100 * MiB, 0x01)):
            for off in (0, n - 16):
                devapis.memCopyD2H(16, ctypes.addressof(back), ptr + off)
                assert bytes(back) == bytes([val]) * 16
        small = [A.allocate(4096, 0, s) for _ in range(8)]   # the small pool has its own segment with 2 MiB pages
        assert A.stats(0)["reserved_bytes"] - before == 182 * MiB
        for p in small + [a, b, c]:
            A.free(p)
        A.emptyCache()
        assert A.stats(0)["reserved_bytes"] == before
    finally:
        A.configure("expandable_segments:False")
        devapis.destroyStream(s)
    devapis.checkLastError()


def test_memory_stats_identities(devapis):
    """dipu/tests/python/individual_scripts/test_memory_stats.py:6-82: every tensor of numel float32 elements raises
    `allocated` by at least ((4 * numel - 1) | 511) + 1, reserved >= allocated throughout; once everything is freed
    allocated == 0 while reserved > 0, until empty_cache() brings reserved to 0 as well; peaks hold and reset."""
    A = devapis.CachingAllocator
    A.useFakeBackend(0)
    devapis.setDevice(0)
    s = devapis.getDefaultStream(0)
    devapis.syncDevice()
    A.emptyCache()
    assert A.stats(0)["allocated_bytes"] == 0 and A.stats(0)["reserved_bytes"] == 0
    A.resetPeakStats(0)
    ptrs, expect = [], 0
    for numel in [1, 7, 128, 129, 1000, 4096, 100000, 1 << 20, 3 << 20, (10 << 20) + 1, 50 << 20]:
        before = A.stats(0)["allocated_bytes"]
        ptrs.append(A.allocate(4 * numel, 0, s))
        nbytes = ((4 * numel - 1) | 511) + 1
        expect += nbytes
        st = A.stats(0)
        assert st["allocated_bytes"] - before >= nbytes
        assert st["allocated_bytes"] >= expect
        assert st["reserved_bytes"] >= st["allocated_bytes"]
        assert st["allocated_bytes_peak"] >= st["allocated_bytes"] and st["reserved_bytes_peak"] >= st["reserved_bytes"]
    peak = A.stats(0)["allocated_bytes_peak"]
    for p in ptrs:
        A.free(p)
    st = A.stats(0)
    assert st["allocated_bytes"] == 0 and st["reserved_bytes"] > 0
    assert st["allocated_bytes_peak"] == peak      # the peak outlives the tensors
    A.resetPeakStats(0)
    assert A.stats(0)["allocated_bytes_peak"] == 0
    A.emptyCache()
    st = A.stats(0)
    assert st["allocated_bytes"] == 0 and st["reserved_bytes"] == 0


def test_one_thread_per_device_with_its_own_current_device(devapis):
    """dipu/tests/python/individual_scripts/test_multi_thread.py:6-16: one thread per device, each setting its device and
    working there; the current device is per thread, so no thread disturbs another or the main thread."""
    import threading
    n = devapis.getDeviceCount()
    devapis.setDevice(0)
    errors = []
    barrier = threading.Barrier(max(n, 2))

    def worker(num):
        try:
            index = num % n
            devapis.setDevice(index)
            barrier.wait(timeout=30)   # every thread has chosen its device before any of them works
            assert devapis.current_device() == index
            stream = devapis.getDefaultStream(index)
            st, p = devapis.mallocDevice(1 << 20)
            assert st == devapis.OpStatus.SUCCESS
            devapis.memSetAsync(stream, p, 0x40 + num, 1 << 20)
            devapis.syncStream(stream)
            back = (ctypes.c_ubyte * 8)()
            devapis.memCopyD2H(8, ctypes.addressof(back), p)
            assert bytes(back) == bytes([0x40 + num]) * 8
            assert devapis.current_device() == index
            devapis.freeDevice(p)
        except Exception as exc:  # reported by the main thread
            errors.append((num, repr(exc)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(max(n, 2))]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=60)
    assert not errors, errors
    assert devapis.current_device() == 0


def test_vendor_contract_by_its_mangled_names_on_the_device():
    """libdipu_vendor_b200_torchabi.so carries the functions DIPU links (namespace dipu::devapis, DIPU's exact C++
    signatures: runtime/device/deviceapis.h:23-124). They are driven here by their mangled names the way DIPU's proxy layer
    calls them: stream, device memory, asynchronous copies both ways, events and their status."""
    import os
    import torch  # noqa: F401  (libc10 / libtorch_cpu are dependencies of the library)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lib = ctypes.CDLL(os.path.join(root, "deeplink.framework_b200", "lib", "libdipu_vendor_b200_torchabi.so"))
    vp, sz = ctypes.c_void_p, ctypes.c_size_t

    def fn(name, restype, *argtypes):
        f = getattr(lib, name)
        f.restype, f.argtypes = restype, list(argtypes)
        return f

    setDevice = fn("_ZN4dipu7devapis9setDeviceEa", None, ctypes.c_int8)
    current_device = fn("_ZN4dipu7devapis14current_deviceEv", ctypes.c_int8)
    createStream = fn("_ZN4dipu7devapis12createStreamEPP11CUstream_stb", None, ctypes.POINTER(vp), ctypes.c_bool)
    destroyStream = fn("_ZN4dipu7devapis13destroyStreamEP11CUstream_st", None, vp)
    syncStream = fn("_ZN4dipu7devapis10syncStreamEP11CUstream_st", None, vp)
    createEvent = fn("_ZN4dipu7devapis11createEventEPP10CUevent_st", None, ctypes.POINTER(vp))
    destroyEvent = fn("_ZN4dipu7devapis12destroyEventEP10CUevent_st", None, vp)
    recordEvent = fn("_ZN4dipu7devapis11recordEventEP10CUevent_stP11CUstream_st", None, vp, vp)
    getEventStatus = fn("_ZN4dipu7devapis14getEventStatusEP10CUevent_st", ctypes.c_int32, vp)
    mallocDevice = fn("_ZN4dipu7devapis12mallocDeviceEPPvmb", ctypes.c_int32, ctypes.POINTER(vp), sz, ctypes.c_bool)
    freeDevice = fn("_ZN4dipu7devapis10freeDeviceEPv", None, vp)
    h2d = fn("_ZN4dipu7devapis15memCopyH2DAsyncEP11CUstream_stmPvPKv", None, vp, sz, vp, vp)
    d2h = fn("_ZN4dipu7devapis15memCopyD2HAsyncEP11CUstream_stmPvPKv", None, vp, sz, vp, vp)

    setDevice(0)
    assert current_device() == 0
    stream, event, dptr = vp(), vp(), vp()
    createStream(ctypes.byref(stream), False)
    createEvent(ctypes.byref(event))
    assert stream.value and event.value
    n = 1 << 20
    assert mallocDevice(ctypes.byref(dptr), n, True) == 0 and dptr.value      # OpStatus::SUCCESS
    src = (ctypes.c_ubyte * n)()
    ctypes.memset(src, 0xA5, n)
    dst = (ctypes.c_ubyte * n)()
    h2d(stream, n, dptr, ctypes.addressof(src))
    d2h(stream, n, ctypes.addressof(dst), dptr)
    recordEvent(event, stream)
    syncStream(stream)
    assert getEventStatus(event) == 3                                          # EventStatus::READY
    assert bytes(dst[:64]) == b"\xa5" * 64 and bytes(dst[-64:]) == b"\xa5" * 64
    # an impossible request reports ERR_NOMEM instead of throwing when asked to
    huge = vp()
    assert mallocDevice(ctypes.byref(huge), 1 << 50, False) == 2 and not huge.value
    freeDevice(dptr)
    destroyEvent(event)
    destroyStream(stream)
