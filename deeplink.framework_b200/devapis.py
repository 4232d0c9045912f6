"""Python mirror of DIPU's vendor interface (namespace dipu::devapis) over the vendor runtime's C-ABI.

Function names, argument meaning and error behaviour follow the reference declarations in
dipu/torch_dipu/csrc_dipu/runtime/device/deviceapis.h:23-124 and diclapis.h:20-82: void functions raise on any driver
error (the reference throws c10::Error through TORCH_CHECK), mallocDevice returns OpStatus.ERR_NOMEM instead of
raising when throwExcepion is False, getEventStatus maps "not ready" to PENDING. Streams, events and communicators are
opaque integer handles.
"""
import ctypes
import enum

from . import _native

_v = _native.vendor


class OpStatus(enum.IntEnum):
    SUCCESS = 0
    ERR_UNKNOWN = 1
    ERR_NOMEM = 2


class EventStatus(enum.IntEnum):
    PENDING = 0
    RUNNING = 1
    DEFERRED = 2
    READY = 3


class diclResult_t(enum.IntEnum):
    DICL_SUCCESS = 0
    DICL_ERR_UNDEF = 0x1000


class ReduceOp(enum.IntEnum):  # same order as c10d::ReduceOp
    SUM = 0
    AVG = 1
    PRODUCT = 2
    MIN = 3
    MAX = 4


class VendorError(RuntimeError):
    pass


class DeviceProperties(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 256), ("totalGlobalMem", ctypes.c_size_t), ("major", ctypes.c_int32), ("minor", ctypes.c_int32),
                ("multiProcessorCount", ctypes.c_int32)]


class AllocStats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in ("allocated_bytes", "allocated_bytes_peak", "reserved_bytes", "reserved_bytes_peak",
                                              "active_blocks", "segments", "num_alloc_retries", "num_ooms", "num_device_mallocs",
                                              "num_cache_hits")]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


class UniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_char * 128)]


_v.b200_last_error.restype = ctypes.c_char_p
_vp, _sz, _i = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
_SIGS = {
    "b200_initialize_vendor": [], "b200_finalize_vendor": [], "b200_current_device": [ctypes.POINTER(_i)],
    "b200_get_device_properties": [_i, ctypes.POINTER(DeviceProperties)],
    "b200_get_device_status": [_i, ctypes.POINTER(_sz), ctypes.POINTER(_sz)],
    "b200_set_device": [_i], "b200_reset_device": [_i], "b200_sync_device": [], "b200_check_last_error": [],
    "b200_get_device_count": [ctypes.POINTER(_i)], "b200_get_driver_version": [ctypes.POINTER(_i)],
    "b200_get_runtime_version": [ctypes.POINTER(_i)],
    "b200_create_stream": [ctypes.POINTER(_vp), _i], "b200_destroy_stream": [_vp], "b200_destroy_stream_on": [_vp, _i],
    "b200_release_stream": [], "b200_sync_stream": [_vp], "b200_stream_wait_event": [_vp, _vp],
    "b200_create_event": [ctypes.POINTER(_vp)], "b200_destroy_event": [_vp], "b200_wait_event": [_vp], "b200_record_event": [_vp, _vp],
    "b200_event_elapsed_time": [ctypes.POINTER(ctypes.c_float), _vp, _vp], "b200_get_event_status": [_vp, ctypes.POINTER(_i)],
    "b200_malloc_host": [ctypes.POINTER(_vp), _sz], "b200_free_host": [_vp], "b200_malloc_device": [ctypes.POINTER(_vp), _sz],
    "b200_free_device": [_vp], "b200_memset_async": [_vp, _vp, _i, _sz],
    "b200_memcpy_d2d": [_sz, _i, _vp, _i, _vp], "b200_memcpy_h2d": [_sz, _vp, _vp], "b200_memcpy_d2h": [_sz, _vp, _vp],
    "b200_memcpy_d2d_async": [_vp, _sz, _i, _vp, _i, _vp], "b200_memcpy_h2d_async": [_vp, _sz, _vp, _vp],
    "b200_memcpy_d2h_async": [_vp, _sz, _vp, _vp],
    "b200_cache_alloc": [ctypes.POINTER(_vp), _sz, _i, _vp], "b200_cache_free": [_vp], "b200_cache_record_stream": [_vp, _vp],
    "b200_cache_empty": [], "b200_cache_stats": [_i, ctypes.POINTER(AllocStats)], "b200_cache_reset_peak": [_i],
    "b200_cache_configure": [ctypes.c_char_p], "b200_cache_use_fake_backend": [_sz, _i], "b200_cache_fake_complete_events": [],
    "b200_host_cache_alloc": [ctypes.POINTER(_vp), _sz], "b200_host_cache_free": [_vp], "b200_host_cache_record_stream": [_vp, _vp],
    "b200_host_cache_empty": [],
    "b200_default_stream": [_i, ctypes.POINTER(_vp)], "b200_stream_from_pool": [_i, ctypes.POINTER(_vp)],
    "b200_event_from_pool": [ctypes.POINTER(_vp)], "b200_event_to_pool": [_vp], "b200_release_all_pools": [],
    "b200_graph_begin_capture": [_vp], "b200_graph_end_capture": [_vp, ctypes.POINTER(_vp)], "b200_graph_launch": [_vp, _vp],
    "b200_graph_destroy": [_vp],
    "b200_dicl_get_unique_id": [ctypes.POINTER(UniqueId)],
    "b200_dicl_comm_init_rank": [ctypes.POINTER(_vp), _i, ctypes.POINTER(UniqueId), _i, _i], "b200_dicl_comm_destroy": [_vp],
    "b200_dicl_get_comm_async_error": [_vp],
    "b200_dicl_all_reduce": [_vp, _vp, _sz, _i, _i, _vp, _vp], "b200_dicl_broadcast": [_vp, _vp, _sz, _i, _i, _vp, _vp],
    "b200_dicl_all_gather": [_vp, _vp, _sz, _i, _vp, _vp], "b200_dicl_reduce": [_vp, _vp, _sz, _i, _i, _i, _vp, _vp],
    "b200_dicl_reduce_scatter": [_vp, _vp, _sz, _i, _i, _vp, _vp], "b200_dicl_send": [_vp, _sz, _i, _i, _vp, _vp],
    "b200_dicl_recv": [_vp, _sz, _i, _i, _vp, _vp],
    "b200_dicl_all_to_all_equal_split": [_vp, _vp, _sz, _i, _vp, _vp],
    "b200_dicl_all_to_all_unequal_split": [_vp, ctypes.POINTER(_sz), ctypes.POINTER(_sz), _vp, ctypes.POINTER(_sz), ctypes.POINTER(_sz), _i, _vp,
                                           _vp],
    "b200_dicl_get_comm_name": [ctypes.c_char_p, _sz, _vp],
    "b200_dicl_comm_rank": [_vp, ctypes.POINTER(_i), ctypes.POINTER(_i)],
    "b200_dicl_peer_reduce_create": [ctypes.POINTER(_vp), _vp, _sz, _vp], "b200_dicl_peer_all_reduce": [_vp, _vp, _vp, _sz, _i, _vp],
    "b200_dicl_peer_reduce_destroy": [_vp], "b200_dicl_peer_reduce_reset_status": [_vp],
    "b200_dicl_peer_space_check": [_vp], "b200_dicl_peer_space_reset_status": [_vp],
    "b200_dicl_peer_space_create": [ctypes.POINTER(_vp), _vp, _sz, _i, _vp],
    "b200_dicl_peer_space_create_emulated": [ctypes.POINTER(_vp), _i, _sz, _i],
    "b200_dicl_peer_space_describe": [_vp, _vp],
    "b200_dicl_peer_reduce_gather": [_vp, _i, ctypes.c_uint32, _vp, ctypes.c_int64, ctypes.c_int64, _i, _i, _vp],
    "b200_dicl_peer_space_destroy": [_vp],
    "b200_expandable_create": [ctypes.POINTER(_vp), _i, _vp, _sz, ctypes.POINTER(_i), _i], "b200_expandable_destroy": [_vp],
    "b200_expandable_map": [_vp, _vp, _sz, ctypes.POINTER(_vp), ctypes.POINTER(_sz)],
    "b200_expandable_unmap": [_vp, _vp, _sz, ctypes.POINTER(_vp), ctypes.POINTER(_sz)], "b200_expandable_add_peer": [_vp, _i],
}
for _n, _a in _SIGS.items():
    getattr(_v, _n).argtypes = _a
    getattr(_v, _n).restype = ctypes.c_int
for _n in ("b200_stream_not_null", "b200_is_stream_empty", "b200_is_pinned_ptr", "b200_dicl_unique_id_bytes"):
    getattr(_v, _n).restype = ctypes.c_int
_v.b200_dicl_peer_reduce_status.argtypes = [_vp]
_v.b200_dicl_peer_reduce_status.restype = ctypes.c_int
_v.b200_dicl_peer_space_status.argtypes = [_vp]
_v.b200_dicl_peer_space_status.restype = ctypes.c_int
_v.b200_dicl_peer_set_wait_limit_ns.argtypes = [ctypes.c_ulonglong]
_v.b200_dicl_peer_set_wait_limit_ns.restype = None
_v.b200_dicl_peer_space_result.argtypes = [_vp, _i]
_v.b200_dicl_peer_space_result.restype = _vp
_v.b200_expandable_ptr.argtypes = [_vp]
_v.b200_expandable_ptr.restype = _vp
_v.b200_expandable_size.argtypes = [_vp]
_v.b200_expandable_size.restype = _sz
_v.b200_expandable_mapped_bytes.argtypes = [_vp]
_v.b200_expandable_mapped_bytes.restype = _sz
_v.b200_stream_not_null.argtypes = [_vp]
_v.b200_is_stream_empty.argtypes = [_vp]
_v.b200_is_pinned_ptr.argtypes = [_vp]

C_SYMBOLS = sorted(list(_SIGS) + ["b200_stream_not_null", "b200_is_stream_empty", "b200_is_pinned_ptr", "b200_dicl_unique_id_bytes",
                                  "b200_last_error", "b200_dicl_peer_set_wait_limit_ns", "b200_dicl_peer_reduce_status", "b200_dicl_peer_space_status", "b200_dicl_peer_space_result", "b200_expandable_ptr", "b200_expandable_size", "b200_expandable_mapped_bytes"])


def last_error():
    return _v.b200_last_error().decode()


def _check(rc, what):
    if rc != 0:
        raise VendorError("%s failed (status %d): %s" % (what, rc, last_error()))


# ---- device --------------------------------------------------------------------------------------------------
def initializeVendor():
    _check(_v.b200_initialize_vendor(), "initializeVendor")


def finalizeVendor():
    _check(_v.b200_finalize_vendor(), "finalizeVendor")


def current_device():
    d = _i()
    _check(_v.b200_current_device(ctypes.byref(d)), "current_device")
    return d.value


def getDeviceProperties(device_index):
    p = DeviceProperties()
    _check(_v.b200_get_device_properties(device_index, ctypes.byref(p)), "getDeviceProperties")
    return p


def getDeviceStatus(device_index):
    f, t = _sz(), _sz()
    _check(_v.b200_get_device_status(device_index, ctypes.byref(f), ctypes.byref(t)), "getDeviceStatus")
    return f.value, t.value


def setDevice(dev):
    _check(_v.b200_set_device(dev), "setDevice")


def resetDevice(dev=0):
    _check(_v.b200_reset_device(dev), "resetDevice")


def syncDevice():
    _check(_v.b200_sync_device(), "syncDevice")


def checkLastError():
    _check(_v.b200_check_last_error(), "checkLastError")


def getDeviceCount():
    n = _i()
    _check(_v.b200_get_device_count(ctypes.byref(n)), "getDeviceCount")
    return n.value


def getDriverVersion():
    n = _i()
    _check(_v.b200_get_driver_version(ctypes.byref(n)), "getDriverVersion")
    return n.value


def getRuntimeVersion():
    n = _i()
    _check(_v.b200_get_runtime_version(ctypes.byref(n)), "getRuntimeVersion")
    return n.value


# ---- streams / events ---------------------------------------------------------------------------------------------
def createStream(prior=False):
    s = _vp()
    _check(_v.b200_create_stream(ctypes.byref(s), int(prior)), "createStream")
    return s.value


def destroyStream(stream, devId=None):
    if devId is None:
        _check(_v.b200_destroy_stream(stream), "destroyStream")
    else:
        _check(_v.b200_destroy_stream_on(stream, devId), "destroyStream")


def releaseStream():
    _check(_v.b200_release_stream(), "releaseStream")


def syncStream(stream):
    _check(_v.b200_sync_stream(stream), "syncStream")


def streamNotNull(stream):
    return bool(_v.b200_stream_not_null(stream))


def streamWaitEvent(stream, event):
    _check(_v.b200_stream_wait_event(stream, event), "streamWaitEvent")


def isStreamEmpty(stream):
    return bool(_v.b200_is_stream_empty(stream))


def createEvent():
    e = _vp()
    _check(_v.b200_create_event(ctypes.byref(e)), "createEvent")
    return e.value


def destroyEvent(event):
    _check(_v.b200_destroy_event(event), "destroyEvent")


def waitEvent(event):
    _check(_v.b200_wait_event(event), "waitEvent")


def recordEvent(event, stream):
    _check(_v.b200_record_event(event, stream), "recordEvent")


def eventElapsedTime(start, end):
    ms = ctypes.c_float()
    _check(_v.b200_event_elapsed_time(ctypes.byref(ms), start, end), "eventElapsedTime")
    return ms.value


def getEventStatus(event):
    st = _i()
    _check(_v.b200_get_event_status(event, ctypes.byref(st)), "getEventStatus")
    return EventStatus(st.value)


def getDefaultStream(device):
    s = _vp()
    _check(_v.b200_default_stream(device, ctypes.byref(s)), "getDefaultStream")
    return s.value


def getStreamFromPool(device):
    s = _vp()
    _check(_v.b200_stream_from_pool(device, ctypes.byref(s)), "getStreamFromPool")
    return s.value


def getEventFromPool():
    e = _vp()
    _check(_v.b200_event_from_pool(ctypes.byref(e)), "getEventFromPool")
    return e.value


def restoreEventToPool(event):
    _check(_v.b200_event_to_pool(event), "restoreEventToPool")


# ---- stream capture (no counterpart in dipu::devapis) -------------------------------------------------------------------
def graphBeginCapture(stream):
    _check(_v.b200_graph_begin_capture(stream), "graphBeginCapture")


def graphEndCapture(stream):
    g = _vp()
    _check(_v.b200_graph_end_capture(stream, ctypes.byref(g)), "graphEndCapture")
    return g.value


def graphLaunch(graph_exec, stream):
    _check(_v.b200_graph_launch(graph_exec, stream), "graphLaunch")


def graphDestroy(graph_exec):
    _check(_v.b200_graph_destroy(graph_exec), "graphDestroy")


# ---- memory --------------------------------------------------------------------------------------------------------
def mallocHost(nbytes):
    p = _vp()
    _check(_v.b200_malloc_host(ctypes.byref(p), nbytes), "mallocHost")
    return p.value


def freeHost(p):
    _check(_v.b200_free_host(p), "freeHost")


def mallocDevice(nbytes, throwExcepion=True):
    """Returns (OpStatus, pointer). With throwExcepion=False an out-of-memory condition is reported, not raised."""
    p = _vp()
    rc = _v.b200_malloc_device(ctypes.byref(p), nbytes)
    if rc == OpStatus.ERR_NOMEM and not throwExcepion:
        return OpStatus.ERR_NOMEM, None
    _check(rc, "mallocDevice")
    return OpStatus.SUCCESS, p.value


def freeDevice(p):
    _check(_v.b200_free_device(p), "freeDevice")


def isPinnedPtr(p):
    return bool(_v.b200_is_pinned_ptr(p))


def memSetAsync(stream, ptr, val, size):
    _check(_v.b200_memset_async(stream, ptr, val, size), "memSetAsync")


def memCopyD2D(nbytes, dstDevId, dst, srcDevId, src):
    _check(_v.b200_memcpy_d2d(nbytes, dstDevId, dst, srcDevId, src), "memCopyD2D")


def memCopyH2D(nbytes, dst, src):
    _check(_v.b200_memcpy_h2d(nbytes, dst, src), "memCopyH2D")


def memCopyD2H(nbytes, dst, src):
    _check(_v.b200_memcpy_d2h(nbytes, dst, src), "memCopyD2H")


def memCopyD2DAsync(stream, nbytes, dstDevId, dst, srcDevId, src):
    _check(_v.b200_memcpy_d2d_async(stream, nbytes, dstDevId, dst, srcDevId, src), "memCopyD2DAsync")


def memCopyH2DAsync(stream, nbytes, dst, src):
    _check(_v.b200_memcpy_h2d_async(stream, nbytes, dst, src), "memCopyH2DAsync")


def memCopyD2HAsync(stream, nbytes, dst, src):
    _check(_v.b200_memcpy_d2h_async(stream, nbytes, dst, src), "memCopyD2HAsync")


# ---- caching allocator (what dipu::getAllocator(DIPU) offers) -----------------------------------------------------------
class CachingAllocator:
    @staticmethod
    def allocate(nbytes, device, stream):
        p = _vp()
        rc = _v.b200_cache_alloc(ctypes.byref(p), nbytes, device, stream)
        if rc == OpStatus.ERR_NOMEM:
            raise MemoryError(last_error())
        _check(rc, "allocate")
        return p.value

    @staticmethod
    def free(p):
        _check(_v.b200_cache_free(p), "free")

    @staticmethod
    def recordStream(p, stream):
        _check(_v.b200_cache_record_stream(p, stream), "recordStream")

    @staticmethod
    def emptyCache():
        _check(_v.b200_cache_empty(), "emptyCache")

    @staticmethod
    def stats(device):
        s = AllocStats()
        _check(_v.b200_cache_stats(device, ctypes.byref(s)), "stats")
        return s.as_dict()

    @staticmethod
    def resetPeakStats(device):
        _check(_v.b200_cache_reset_peak(device), "resetPeakStats")

    @staticmethod
    def configure(conf):
        _check(_v.b200_cache_configure(conf.encode()), "configure")

    @staticmethod
    def useFakeBackend(capacity, pending_events=False):
        _check(_v.b200_cache_use_fake_backend(capacity, int(pending_events)), "useFakeBackend")

    @staticmethod
    def fakeCompleteEvents():
        _check(_v.b200_cache_fake_complete_events(), "fakeCompleteEvents")


class ExpandableSegment:
    """dipu::ExpandableSegment as the vendor implements it (runtime/core/allocator/ExpandableSegment.h:105-136): a
    reservation of virtual addresses into which pages of `page_size` bytes are mapped and unmapped. map / unmap return
    (ptr, size) of the affected whole pages; size 0 from map means the device is out of memory."""

    def __init__(self, device, stream, page_size, peers=()):
        h = _vp()
        arr = (ctypes.c_int * max(len(peers), 1))(*peers)
        _check(_v.b200_expandable_create(ctypes.byref(h), device, stream, page_size, arr, len(peers)), "vendorCreateExpandableSegment")
        self.handle = h.value

    def map(self, ptr, size):
        p, n = _vp(), _sz()
        _check(_v.b200_expandable_map(self.handle, ptr, size, ctypes.byref(p), ctypes.byref(n)), "ExpandableSegment.map")
        return (p.value or 0), n.value

    def unmap(self, ptr, size):
        p, n = _vp(), _sz()
        _check(_v.b200_expandable_unmap(self.handle, ptr, size, ctypes.byref(p), ctypes.byref(n)), "ExpandableSegment.unmap")
        return (p.value or 0), n.value

    def addPeer(self, device):
        _check(_v.b200_expandable_add_peer(self.handle, device), "ExpandableSegment.addPeer")

    def ptr(self):
        return _v.b200_expandable_ptr(self.handle)

    def size(self):
        return _v.b200_expandable_size(self.handle)

    def mappedBytes(self):
        return _v.b200_expandable_mapped_bytes(self.handle)

    def close(self):
        if self.handle:
            _check(_v.b200_expandable_destroy(self.handle), "ExpandableSegment destroy")
            self.handle = None


class CachingHostAllocator:
    @staticmethod
    def allocate(nbytes):
        p = _vp()
        _check(_v.b200_host_cache_alloc(ctypes.byref(p), nbytes), "host allocate")
        return p.value

    @staticmethod
    def free(p):
        _check(_v.b200_host_cache_free(p), "host free")

    @staticmethod
    def recordStream(p, stream):
        _check(_v.b200_host_cache_record_stream(p, stream), "host recordStream")

    @staticmethod
    def emptyCache():
        _check(_v.b200_host_cache_empty(), "host emptyCache")


# ---- DICL ------------------------------------------------------------------------------------------------------------------
DICL_UNIQUE_ID_BYTES_SIZE = _v.b200_dicl_unique_id_bytes()


def _dicl(rc, what):
    if rc != 0:
        raise VendorError("call dicl error, expr = %s, status %d: %s" % (what, rc, last_error()))
    return diclResult_t.DICL_SUCCESS


def diclGetUniqueId():
    uid = UniqueId()
    _dicl(_v.b200_dicl_get_unique_id(ctypes.byref(uid)), "diclGetUniqueId")
    return bytes(ctypes.string_at(ctypes.byref(uid), 128))


def diclCommInitRank(nranks, uniqueId, rank, localDeviceId=-1):
    uid = UniqueId()
    ctypes.memmove(ctypes.byref(uid), uniqueId, 128)
    comm = _vp()
    _dicl(_v.b200_dicl_comm_init_rank(ctypes.byref(comm), nranks, ctypes.byref(uid), rank, localDeviceId), "diclCommInitRank")
    return comm.value


def diclCommDestroy(comm):
    return _dicl(_v.b200_dicl_comm_destroy(comm), "diclCommDestroy")


def diclGetCommAsyncError(comm):
    rc = _v.b200_dicl_get_comm_async_error(comm)
    return diclResult_t.DICL_SUCCESS if rc == 0 else diclResult_t.DICL_ERR_UNDEF


def diclAllReduce(sendBuf, recvBuf, count, datatype, reduceOp, comm, stream):
    return _dicl(_v.b200_dicl_all_reduce(sendBuf, recvBuf, count, datatype, int(reduceOp), comm, stream), "diclAllReduce")


def diclCommRank(comm):
    r, n = ctypes.c_int(), ctypes.c_int()
    _check(_v.b200_dicl_comm_rank(comm, ctypes.byref(r), ctypes.byref(n)), "diclCommRank")
    return r.value, n.value


class PeerAllReduce:
    """SUM all-reduce of small messages in one kernel over peer memory (no reference counterpart; see
    b200_dicl_peer_reduce_* in include/dipu_b200/vendor_c_api.h). Creation is collective over the communicator."""

    def __init__(self, comm, max_bytes, stream):
        h = _vp()
        _check(_v.b200_dicl_peer_reduce_create(ctypes.byref(h), comm, max_bytes, stream), "peer reduce create")
        self.handle, self.max_bytes = h.value, max_bytes

    def all_reduce(self, sendBuf, recvBuf, count, datatype, stream):
        _check(_v.b200_dicl_peer_all_reduce(self.handle, sendBuf, recvBuf, count, datatype, stream), "peer all-reduce")

    def status(self):
        return _v.b200_dicl_peer_reduce_status(self.handle)

    def reset_status(self):
        _check(_v.b200_dicl_peer_reduce_reset_status(self.handle), "peer reduce reset status")

    def close(self):
        """Collective: every rank drains its device and meets the others in a one-element all-reduce inside the call,
        so no peer can still be reading this rank's staging or writing its flags when they are freed."""
        if self.handle:
            _check(_v.b200_dicl_peer_reduce_destroy(self.handle), "peer reduce destroy")
            self.handle = None


def setPeerWaitLimitNs(ns):
    """Limit of every flag wait in the peer-memory kernels (PeerAllReduce, PeerSpace.reduce_gather) launched from now on;
    0 restores the default of one second."""
    _v.b200_dicl_peer_set_wait_limit_ns(int(ns))


class _DeviceBytes:
    """A device address range in the form torch.as_tensor() accepts (CUDA array interface, version 2)."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False), "version": 2}


def tensorFromDevicePtr(ptr, shape, dtype, device):
    """A torch tensor that views `shape` elements of `dtype` at device address `ptr` (no copy; the memory's owner must
    outlive the tensor)."""
    import torch
    n = 1
    for d in shape:
        n *= int(d)
    raw = torch.as_tensor(_DeviceBytes(ptr, n * torch.empty((), dtype=dtype).element_size()), device=device)
    return raw.view(dtype).view(*shape)


class _PeerSpaceDesc(ctypes.Structure):
    """b200PeerSpace (include/dipu_b200/peer_space.h)."""
    _fields_ = [("rank", ctypes.c_int32), ("nranks", ctypes.c_int32), ("slots", ctypes.c_int32), ("max_units", ctypes.c_uint32),
                ("ctas", ctypes.c_uint32), ("pad_", ctypes.c_uint32), ("slot_bytes", ctypes.c_uint64),
                ("stage", ctypes.c_void_p * 8), ("gout", ctypes.c_void_p * 8), ("flags", ctypes.c_void_p * 8)]


class PeerSpace:
    """Staging / result slots shared by a communicator's ranks for row-parallel linears whose all-reduce is fused into the
    compute kernels (no reference counterpart; b200_dicl_peer_space_* in include/dipu_b200/vendor_c_api.h). Creation is
    collective. One fused linear is `diopi.diopiB200MmPush(ctx, x, w_t, space, slot, epoch, prev)` followed by
    `space.reduce_gather(slot, epoch, residual, rows, cols, dtype, stream)`; begin() hands out (epoch, prev) for a slot."""

    def __init__(self, comm, slot_bytes, slots, stream, _handle=None):
        if _handle is None:
            h = _vp()
            _check(_v.b200_dicl_peer_space_create(ctypes.byref(h), comm, slot_bytes, int(slots), stream), "peer space create")
            _handle = h.value
        self.handle, self.slot_bytes, self.slots = _handle, slot_bytes, slots
        self.desc = _PeerSpaceDesc()
        _check(_v.b200_dicl_peer_space_describe(self.handle, ctypes.addressof(self.desc)), "peer space describe")
        self.epoch = 0
        self.last = [0] * slots  # epoch of the last call on each slot
        self.final_wait = 1

    @classmethod
    def emulated(cls, nranks, slot_bytes, slots):
        """A group of `nranks` in this process on the current device (tests): returns one PeerSpace per rank. Enqueue the
        products of all ranks first, then the reductions, on one stream."""
        arr = (ctypes.c_void_p * nranks)()
        _check(_v.b200_dicl_peer_space_create_emulated(arr, int(nranks), slot_bytes, int(slots)), "peer space create (emulated)")
        out = [cls(None, slot_bytes, slots, None, _handle=arr[r]) for r in range(nranks)]
        for s in out:
            s.final_wait = 0
        return out

    def begin(self, slot):
        """Numbers for the next fused linear on `slot`: (epoch, epoch of the previous call on that slot). Every rank must
        call this in the same order."""
        self.epoch += 1
        prev, self.last[slot] = self.last[slot], self.epoch
        return self.epoch, prev

    def result_ptr(self, slot):
        return _v.b200_dicl_peer_space_result(self.handle, int(slot))

    def reduce_gather(self, slot, epoch, residual_ptr, rows, cols, datatype, stream):
        _check(_v.b200_dicl_peer_reduce_gather(self.handle, int(slot), int(epoch), residual_ptr or None, int(rows), int(cols), int(datatype),
                                               int(self.final_wait), stream), "peer reduce-gather")

    def status(self):
        return _v.b200_dicl_peer_space_status(self.handle)

    def check(self):
        """diclResult_t.DICL_SUCCESS while every bounded wait completed, DICL_ERR_UNDEF once one ran out (the failed call's
        result is incomplete on every rank; last_error() says so). OR the value over the ranks before trusting a result."""
        return diclResult_t.DICL_SUCCESS if _v.b200_dicl_peer_space_check(self.handle) == 0 else diclResult_t.DICL_ERR_UNDEF

    def reset_status(self):
        _check(_v.b200_dicl_peer_space_reset_status(self.handle), "peer space reset status")

    def close(self):
        if self.handle:
            _check(_v.b200_dicl_peer_space_destroy(self.handle), "peer space destroy")
            self.handle = None


def diclBroadcast(sendBuf, recvBuf, count, datatype, root, comm, stream):
    return _dicl(_v.b200_dicl_broadcast(sendBuf, recvBuf, count, datatype, root, comm, stream), "diclBroadcast")


def diclAllGather(sendBuf, recvBuf, sendCount, datatype, comm, stream):
    return _dicl(_v.b200_dicl_all_gather(sendBuf, recvBuf, sendCount, datatype, comm, stream), "diclAllGather")


def diclReduce(sendBuf, recvBuf, count, datatype, reduceOp, root, comm, stream):
    return _dicl(_v.b200_dicl_reduce(sendBuf, recvBuf, count, datatype, int(reduceOp), root, comm, stream), "diclReduce")


def diclReduceScatter(sendBuf, recvBuf, recvCount, datatype, op, comm, stream):
    return _dicl(_v.b200_dicl_reduce_scatter(sendBuf, recvBuf, recvCount, datatype, int(op), comm, stream), "diclReduceScatter")


def diclSend(sendBuf, count, datatype, peer, comm, stream):
    return _dicl(_v.b200_dicl_send(sendBuf, count, datatype, peer, comm, stream), "diclSend")


def diclRecv(recvBuf, count, datatype, peer, comm, stream):
    return _dicl(_v.b200_dicl_recv(recvBuf, count, datatype, peer, comm, stream), "diclRecv")


def diclAllToAllEqualSplit(sendBuf, recvBuf, count, dataType, comm, stream):
    return _dicl(_v.b200_dicl_all_to_all_equal_split(sendBuf, recvBuf, count, dataType, comm, stream), "diclAllToAllEqualSplit")


def diclAllToAllUnequalSplit(sendBuf, sendCounts, sendDisplacements, recvBuf, recvCounts, recvDisplacements, dataType, comm, stream):
    n = len(sendCounts)
    arr = lambda v: (ctypes.c_size_t * n)(*v)  # noqa: E731
    return _dicl(_v.b200_dicl_all_to_all_unequal_split(sendBuf, arr(sendCounts), arr(sendDisplacements), recvBuf, arr(recvCounts),
                                                       arr(recvDisplacements), dataType, comm, stream), "diclAllToAllUnequalSplit")


def diclGetCommName(comm):
    buf = ctypes.create_string_buffer(64)
    _dicl(_v.b200_dicl_get_comm_name(buf, 64, comm), "diclGetCommName")
    return buf.value.decode()
