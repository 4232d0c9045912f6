"""Policy of the caching device allocator on a host-side fake backend (no GPU): size classes, split / coalesce, cache
hits, the out-of-memory ladder (host-side fault injection: the pretend device simply runs out), event-deferred reuse
after record_stream, statistics. Semantics pinned by the reference's tests/python/individual_scripts/test_memory_stats.py."""
import pytest

MiB = 1 << 20


@pytest.fixture()
def A(pkg):
    alloc = pkg.devapis.CachingAllocator
    alloc.useFakeBackend(8 << 30)
    yield alloc
    alloc.useFakeBackend(0)


def test_rounding_and_stats(A):
    base = A.stats(0)
    assert base["allocated_bytes"] == 0 and base["reserved_bytes"] == 0
    ptrs, expect = [], 0
    for numel in (1, 10, 100, 1000, 100000):
        nbytes = 4 * numel
        ptrs.append(A.allocate(nbytes, 0, 1))
        expect += ((nbytes - 1) | 511) + 1
        st = A.stats(0)
        assert st["allocated_bytes"] == expect  # exactly the 512-byte rounding, as for the reference's BF/BS/RAW allocators
        assert st["reserved_bytes"] >= st["allocated_bytes"]
    assert A.stats(0)["segments"] == 1  # all small requests share one 2 MiB segment
    for p in ptrs:
        A.free(p)
    st = A.stats(0)
    assert st["allocated_bytes"] == 0 and st["reserved_bytes"] == 2 * MiB and st["allocated_bytes_peak"] == expect
    A.emptyCache()
    assert A.stats(0)["reserved_bytes"] == 0
    A.resetPeakStats(0)
    assert A.stats(0)["allocated_bytes_peak"] == 0
    assert A.allocate(0, 0, 1) is None


def test_size_classes(A):
    a = A.allocate(3 * MiB, 0, 1)      # mid: carved from a 256 MiB arena
    assert A.stats(0)["reserved_bytes"] == 256 * MiB
    b = A.allocate(20 * MiB, 0, 1)     # same arena
    assert A.stats(0)["reserved_bytes"] == 256 * MiB and A.stats(0)["num_device_mallocs"] == 1
    c = A.allocate(2049 * MiB + 5, 0, 1)  # large: own segment rounded to 2 MiB
    assert A.stats(0)["reserved_bytes"] == 256 * MiB + 2050 * MiB
    for p in (a, b, c):
        A.free(p)
    # a freed 2 GiB block serves the next request of that size without touching the driver
    n = A.stats(0)["num_device_mallocs"]
    d = A.allocate(2048 * MiB, 0, 1)
    assert A.stats(0)["num_device_mallocs"] == n and A.stats(0)["num_cache_hits"] >= 1
    A.free(d)


def test_split_and_coalesce(A):
    a = A.allocate(100 * MiB, 0, 1)
    A.free(a)
    parts = [A.allocate(25 * MiB, 0, 1) for _ in range(4)]  # carved out of the cached 100 MiB block
    assert A.stats(0)["segments"] == 1
    assert sorted(parts) == [parts[0] + i * 25 * MiB for i in range(4)]
    for p in (parts[1], parts[3], parts[0], parts[2]):
        A.free(p)
    again = A.allocate(100 * MiB, 0, 1)  # neighbours merged back into one block
    assert again == a and A.stats(0)["segments"] == 1
    A.free(again)


def test_blocks_are_only_reused_on_their_stream(A):
    a = A.allocate(64 * MiB, 0, 1)
    A.free(a)
    b = A.allocate(64 * MiB, 0, 2)  # other stream: must not get stream 1's cached block
    assert b != a and A.stats(0)["segments"] == 2
    c = A.allocate(64 * MiB, 0, 1)
    assert c == a
    A.free(b)
    A.free(c)


def test_out_of_memory_ladder(pkg):
    A = pkg.devapis.CachingAllocator
    A.useFakeBackend(1 << 30)  # a 1 GiB device
    try:
        a = A.allocate(600 * MiB, 0, 1)
        A.free(a)                           # cached, still reserved
        b = A.allocate(700 * MiB, 0, 1)     # does not fit beside the cached block: cache is released, then it fits
        st = A.stats(0)
        assert st["num_alloc_retries"] >= 1 and st["num_ooms"] == 0 and st["reserved_bytes"] == 700 * MiB
        with pytest.raises(MemoryError) as e:
            A.allocate(600 * MiB, 0, 1)     # genuinely out of memory
        assert "out of memory" in str(e.value)
        assert A.stats(0)["num_ooms"] == 1
        A.free(b)
        c = A.allocate(900 * MiB, 0, 1)     # after the failure the allocator still works
        A.free(c)
    finally:
        A.useFakeBackend(0)


def test_record_stream_defers_reuse_until_events_complete(pkg):
    A = pkg.devapis.CachingAllocator
    A.useFakeBackend(4 << 30, pending_events=True)
    try:
        a = A.allocate(64 * MiB, 0, 1)
        A.recordStream(a, 2)    # e.g. a collective on the communication stream reads the block
        A.free(a)
        b = A.allocate(64 * MiB, 0, 1)
        assert b != a           # the event on stream 2 has not completed: the block is parked
        A.free(b)
        A.fakeCompleteEvents()
        c = A.allocate(64 * MiB, 0, 1)
        d = A.allocate(64 * MiB, 0, 1)
        assert a in (c, d)      # parked block came back once its event completed
        A.free(c)
        A.free(d)
        with pytest.raises(pkg.devapis.VendorError):
            A.free(12345)       # foreign pointer
    finally:
        A.useFakeBackend(0)


def test_configuration_strings(A, pkg):
    A.configure("max_split_size_mb:64,garbage_collection_threshold:0.8")
    a = A.allocate(200 * MiB, 0, 1)
    A.free(a)
    b = A.allocate(30 * MiB, 0, 1)  # the oversize cached block is not split for a small request
    assert b != a
    A.free(b)
    with pytest.raises(pkg.devapis.VendorError):
        A.configure("no_such_option:1")
    with pytest.raises(pkg.devapis.VendorError):
        A.configure("max_split_size_mb:10")


# ---- expandable segments (expandable_segments:True): one growing segment per pool and stream ----------------------------
def test_expandable_segment_grows_in_place(A):
    A.configure("expandable_segments:True")
    a = A.allocate(10 * MiB, 0, 1)
    st = A.stats(0)
    assert st["segments"] == 1 and st["reserved_bytes"] == 20 * MiB   # one 20 MiB page of the large pool
    b = A.allocate(30 * MiB, 0, 1)
    # the free 10 MiB tail of the first page plus one more page: the segment grew at its end, contiguously
    assert b == a + 10 * MiB
    st = A.stats(0)
    assert st["segments"] == 1 and st["reserved_bytes"] == 40 * MiB and st["allocated_bytes"] == 40 * MiB
    A.free(a)
    A.free(b)
    n = A.stats(0)["num_device_mallocs"]
    c = A.allocate(40 * MiB, 0, 1)   # the two freed blocks coalesced: a cache hit, nothing mapped
    assert c == a and A.stats(0)["num_device_mallocs"] == n
    A.free(c)
    A.emptyCache()
    st = A.stats(0)
    assert st["reserved_bytes"] == 0 and st["segments"] == 0


def test_expandable_small_pool_and_streams(A):
    A.configure("expandable_segments:True")
    small = [A.allocate(64 * 1024, 0, 1) for _ in range(100)]   # 6.25 MiB in 2 MiB pages
    st = A.stats(0)
    assert st["segments"] == 1 and st["reserved_bytes"] == 8 * MiB
    assert sorted(small) == small and small[-1] - small[0] == 99 * 64 * 1024   # one contiguous run
    other = A.allocate(64 * 1024, 0, 2)   # another stream: its own segment
    assert A.stats(0)["segments"] == 2
    big = A.allocate(5 * MiB, 0, 1)       # large pool of stream 1: a third one
    assert A.stats(0)["segments"] == 3
    for p in small + [other, big]:
        A.free(p)
    A.emptyCache()
    assert A.stats(0)["reserved_bytes"] == 0 and A.stats(0)["segments"] == 0


def test_expandable_unmaps_free_pages_when_memory_is_short(pkg):
    A = pkg.devapis.CachingAllocator
    A.useFakeBackend(100 * MiB)
    try:
        A.configure("expandable_segments:True")
        a = A.allocate(60 * MiB, 0, 1)
        A.free(a)                                  # 60 MiB stay mapped in stream 1's segment
        assert A.stats(0)["reserved_bytes"] == 60 * MiB
        b = A.allocate(60 * MiB, 0, 2)             # stream 2 needs 60 MiB, only 40 are left: stream 1's free pages go back
        st = A.stats(0)
        assert st["num_alloc_retries"] >= 1 and st["reserved_bytes"] == 60 * MiB and st["num_ooms"] == 0
        with pytest.raises(MemoryError):
            A.allocate(60 * MiB, 0, 1)
        assert A.stats(0)["num_ooms"] == 1
        A.free(b)
    finally:
        A.useFakeBackend(0)


def test_expandable_refills_gaps_at_the_lowest_address(A):
    A.configure("expandable_segments:True")
    x, y, z = (A.allocate(20 * MiB, 0, 1) for _ in range(3))
    assert y == x + 20 * MiB and z == y + 20 * MiB
    A.free(y)
    A.emptyCache()                                  # y's page is unmapped: a hole between x and z
    assert A.stats(0)["reserved_bytes"] == 40 * MiB
    w = A.allocate(15 * MiB, 0, 1)
    assert w == y                                   # the hole is mapped again before the segment grows at its end
    v = A.allocate(30 * MiB, 0, 1)                  # does not fit the 5 MiB left in the hole: goes behind z
    assert v == z + 20 * MiB
    for p in (x, z, w, v):
        A.free(p)
    A.emptyCache()
    assert A.stats(0)["reserved_bytes"] == 0


def test_expandable_config_is_validated(A):
    with pytest.raises(Exception, match="True or False"):
        A.configure("expandable_segments:yes")
    A.configure("expandable_segments:False")
