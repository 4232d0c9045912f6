"""ctypes binding of the DIOPI C-ABI (include/diopi/functions.h, functions_ext.h) through the minihost.

Tensors are torch tensors used purely as memory holders: a handle records data pointer, shape, strides, dtype and
device, exactly the metadata DIPU's diopirt callbacks expose. Every diopiXxx function of the library is callable as
`diopi.diopiXxx(ctx, ...)` with torch tensors, Python numbers and lists in the argument order of the C prototype;
a non-zero return code raises DiopiError carrying diopiGetLastErrorString().
"""
import ctypes

import torch

from . import _native

_lib = _native.diopi
_host = _native.host

# ---- enums (include/diopi/diopirt.h) -------------------------------------------------------------------------
diopi_host, diopi_device = 0, 1
DTYPE = {
    torch.int8: 0, torch.uint8: 1, torch.int16: 2, torch.int32: 4, torch.int64: 6, torch.float16: 8, torch.float32: 9,
    torch.float64: 10, torch.bool: 11, torch.bfloat16: 12,
}
RoundModeNone, RoundModeTrunc, RoundModeFloor = 0, 1, 2


class DiopiError(RuntimeError):
    pass


class _Size(ctypes.Structure):
    _fields_ = [("data", ctypes.POINTER(ctypes.c_int64)), ("len", ctypes.c_int64)]


class _ScalarU(ctypes.Union):
    _fields_ = [("fval", ctypes.c_double), ("ival", ctypes.c_int64)]


class _Scalar(ctypes.Structure):
    _anonymous_ = ("u",)
    _fields_ = [("stype", ctypes.c_int), ("u", _ScalarU)]


def _scalar(v):
    s = _Scalar()
    if isinstance(v, bool) or isinstance(v, int):
        s.stype = 6  # diopi_dtype_int64 (bools travel as int64, reference diopi_helper.cpp:74-119)
        s.ival = int(v)
    else:
        s.stype = 10  # diopi_dtype_float64
        s.fval = float(v)
    return s


_host.minihostMakeTensor.restype = ctypes.c_void_p
_host.minihostMakeTensor.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64),
                                     ctypes.c_int, ctypes.c_int, ctypes.c_int]
_host.minihostFreeTensor.argtypes = [ctypes.c_void_p]
_host.minihostMakeContext.restype = ctypes.c_void_p
_host.minihostMakeContext.argtypes = [ctypes.c_void_p, ctypes.c_int]
_host.minihostResetContext.argtypes = [ctypes.c_void_p]
_host.minihostFreeContext.argtypes = [ctypes.c_void_p]
_host.minihostWorkspaceCount.restype = ctypes.c_int64
_host.minihostWorkspaceCount.argtypes = [ctypes.c_void_p]
_lib.diopiGetLastErrorString.restype = ctypes.c_char_p
_lib.diopiGetVendorName.restype = ctypes.c_char_p
_lib.diopiGetImplVersion.restype = ctypes.c_char_p
_lib.diopiB200GemmStatus.restype = ctypes.c_int
_lib.diopiB200Init.restype = ctypes.c_int
_lib.diopiB200SetPushWaitLimitNs.argtypes = [ctypes.c_ulonglong]
_lib.diopiB200SetPushWaitLimitNs.restype = None
_INITIALISED = set()


def init_device(device):
    """What a host does where it initialises a device: the library's one-time set-up (diopiB200Init) with that device
    current, so that the first operator call neither allocates nor synchronises."""
    if device in _INITIALISED or not torch.cuda.is_available():
        return
    with torch.cuda.device(device):
        if _lib.diopiB200Init() != 0:
            raise DiopiError("diopiB200Init failed: %s" % _lib.diopiGetLastErrorString().decode())
    _INITIALISED.add(device)


class Handle:
    """A diopiTensorHandle_t describing a torch tensor's memory. Keeps the tensor alive."""

    __slots__ = ("tensor", "ptr")

    def __init__(self, t, keep=True):
        if t.dtype not in DTYPE:
            raise DiopiError("dtype %s has no diopi counterpart" % t.dtype)
        nd = t.dim()
        shape = (ctypes.c_int64 * max(nd, 1))(*t.shape)
        stride = (ctypes.c_int64 * max(nd, 1))(*t.stride())
        dev = diopi_device if t.is_cuda else diopi_host
        idx = t.device.index if t.is_cuda else 0
        self.tensor = t if keep else None
        self.ptr = _host.minihostMakeTensor(ctypes.c_void_p(t.data_ptr()), nd, shape, stride, DTYPE[t.dtype], dev, idx or 0)
        if not self.ptr:
            raise DiopiError("could not create a tensor handle")

    def __del__(self):
        if getattr(self, "ptr", None) and _host is not None:  # at interpreter exit the module globals may already be gone
            _host.minihostFreeTensor(self.ptr)
            self.ptr = None


_HANDLE_CACHE = {}


def handle(t):
    """Handle for a torch tensor. Handles are pure metadata (pointer, shape, strides, dtype, device), so one is kept per
    distinct description and re-used: with a caching allocator a steady-state loop sees the same descriptions every step.
    Cached handles do not keep the tensor alive; the caller's reference does for the duration of the call."""
    if isinstance(t, Handle):
        return t
    key = (t.data_ptr(), t.dtype, tuple(t.shape), t.stride(), t.device.index if t.is_cuda else -1)
    h = _HANDLE_CACHE.get(key)
    if h is None:
        if len(_HANDLE_CACHE) >= 8192:
            _HANDLE_CACHE.clear()
        h = Handle(t, keep=False)
        _HANDLE_CACHE[key] = h
    return h


class Context:
    """diopiContext: the stream every op of a call is enqueued on, plus the workspace the op requested."""

    def __init__(self, stream=None, device=None):
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream if torch.cuda.is_available() else 0
        if device is None:
            device = torch.cuda.current_device() if torch.cuda.is_available() else 0
        self.stream = int(stream)
        self.device = int(device)
        init_device(self.device)
        self.ptr = _host.minihostMakeContext(ctypes.c_void_p(self.stream), self.device)

    def release_workspace(self):
        """What the DIPU wrapper does when it returns: workspace tensors go back to the caching allocator."""
        _host.minihostResetContext(self.ptr)

    def workspace_count(self):
        return _host.minihostWorkspaceCount(self.ptr)

    def __del__(self):
        if getattr(self, "ptr", None) and _host is not None:  # at interpreter exit the module globals may already be gone
            _host.minihostFreeContext(self.ptr)
            self.ptr = None


# ---- signatures ---------------------------------------------------------------------------------------------
# T: tensor handle   t: tensor handle or None   s: const diopiScalar_t*   i: int64   d: double   b: bool
# z: diopiSize_t by value   L: (const handle*, int64 count)   r: diopiRoundMode_t
# I: const int64_t* or None   P: const bool* or None   G: generator handle (Generator or None)
SIGNATURES = {
    "diopiCopyInp": "tT", "diopiCastDtype": "Tt", "diopiFill": "Ts", "diopiZeroInp": "T", "diopiOnes": "Tz", "diopiZeros": "Tz",
    "diopiArange": "Tsss",
    "diopiAdd": "Ttts", "diopiAddInp": "Tts", "diopiAddScalar": "Ttss", "diopiAddInpScalar": "Tss",
    "diopiSub": "Ttts", "diopiSubInp": "Tts", "diopiSubScalar": "Ttss", "diopiSubInpScalar": "Tss",
    "diopiMul": "Ttt", "diopiMulInp": "Tt", "diopiMulScalar": "Tts", "diopiMulInpScalar": "Ts",
    "diopiDiv": "Tttr", "diopiDivInp": "Ttr", "diopiDivScalar": "Ttsr", "diopiDivInpScalar": "Tsr",
    "diopiPow": "Tts", "diopiPowInp": "Ts", "diopiPowTensor": "Ttt", "diopiPowScalar": "Tst",
    "diopiNeg": "Tt", "diopiNegInp": "T", "diopiRsqrt": "Tt", "diopiRsqrtInp": "T", "diopiSqrt": "Tt", "diopiReciprocal": "Tt",
    "diopiExp": "Tt", "diopiSin": "Tt", "diopiSinInp": "T", "diopiCos": "Tt", "diopiCosInp": "T", "diopiSilu": "Tt", "diopiSiluInp": "T",
    "diopiSigmoid": "Tt", "diopiRelu": "Tt", "diopiTanh": "Tt",
    "diopiTriu": "Tti", "diopiTriuInp": "Ti", "diopiMaskedFill": "Tttt", "diopiMaskedFillInp": "Ttt", "diopiMaskedFillScalar": "Ttts",
    "diopiMaskedFillInpScalar": "Tts", "diopiWhere": "Tttt", "diopiCat": "TLi", "diopiIndexSelect": "Ttit", "diopiEmbedding": "Tttibb",
    "diopiMean": "Ttz", "diopiSum": "Ttz", "diopiSoftmax": "Tti", "diopiLayerNorm": "TTTtttzd",
    "diopiMm": "Ttt", "diopiAddmm": "Ttttss", "diopiBmm": "Ttt", "diopiBaddbmm": "Ttttdd", "diopiBaddbmmInp": "Tttdd", "diopiMatmul": "Ttt",
    "diopiLinear": "Tttt",
    "diopiRMSNorm": "TTtzttd", "diopiRotaryEmbedding": "Ttttbb",
    "diopiMultiHeadAttention": "TTTdbbdTttt",
    "diopiArgmax": "TtIb", "diopiSort": "TTtibP", "diopiTopk": "TTtiibb", "diopiCumsum": "Tti", "diopiGather": "Ttit",
    "diopiMultinomial": "TtibG", "diopiIndexPutInp": "TtLb",
    # additions of this library (include/diopi/functions_b200.h): fused steps of a decode iteration
    "diopiB200MmSwiGLU": "TTT", "diopiB200AddRMSNorm": "TTTTtd", "diopiB200RopeAppendKV": "TTTTTTi",
}

_CTYPES = {"T": ctypes.c_void_p, "t": ctypes.c_void_p, "s": ctypes.POINTER(_Scalar), "i": ctypes.c_int64, "d": ctypes.c_double,
           "b": ctypes.c_bool, "z": _Size, "r": ctypes.c_int, "I": ctypes.POINTER(ctypes.c_int64), "P": ctypes.POINTER(ctypes.c_bool),
           "G": ctypes.c_void_p}


def _bind(name):
    fn = getattr(_lib, name)
    sig = SIGNATURES[name]
    argtypes = [ctypes.c_void_p]
    for c in sig:
        if c == "L":
            argtypes += [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int64]
        else:
            argtypes.append(_CTYPES[c])
    fn.argtypes = argtypes
    fn.restype = ctypes.c_int

    def call(ctx, *args):
        if len(args) != len(sig):
            raise TypeError("%s expects %d arguments after ctx, got %d" % (name, len(sig), len(args)))
        cargs = [ctx.ptr]
        keep = []
        for c, a in zip(sig, args):
            if c in "Tt":
                if a is None:
                    cargs.append(None)
                else:
                    h = handle(a)
                    keep.append(h)
                    cargs.append(h.ptr)
            elif c == "s":
                if a is None:
                    cargs.append(None)
                else:
                    s = _scalar(a)
                    keep.append(s)
                    cargs.append(ctypes.byref(s))
            elif c == "z":
                vals = list(a) if a is not None else []
                arr = (ctypes.c_int64 * max(len(vals), 1))(*vals)
                keep.append(arr)
                cargs.append(_Size(ctypes.cast(arr, ctypes.POINTER(ctypes.c_int64)), len(vals)))
            elif c == "L":
                hs = [None if x is None else handle(x) for x in a]   # None: an absent optional tensor (NULL handle)
                keep.append(hs)
                arr = (ctypes.c_void_p * max(len(hs), 1))(*[None if h is None else h.ptr for h in hs])
                keep.append(arr)
                cargs += [arr, len(hs)]
            elif c == "I":
                if a is None:
                    cargs.append(None)
                else:
                    v = ctypes.c_int64(int(a))
                    keep.append(v)
                    cargs.append(ctypes.byref(v))
            elif c == "P":
                if a is None:
                    cargs.append(None)
                else:
                    v = ctypes.c_bool(bool(a))
                    keep.append(v)
                    cargs.append(ctypes.byref(v))
            elif c == "G":
                cargs.append(None if a is None else a.ptr)
            elif c == "b":
                cargs.append(bool(a))
            elif c == "d":
                cargs.append(float(a))
            else:
                cargs.append(int(a))
        rc = fn(*cargs)
        if rc != 0:
            raise DiopiError("%s failed with code %d: %s" % (name, rc, last_error()))
        return rc

    call.__name__ = name
    return call


class Generator:
    """The host's RNG state the library reads and advances (diopiGeneratorGetSeedAndOffset / SetSeedAndOffset)."""

    def __init__(self, seed=67280421310721):
        _host.minihostMakeGenerator.restype = ctypes.c_void_p
        _host.minihostMakeGenerator.argtypes = [ctypes.c_uint64]
        self.ptr = _host.minihostMakeGenerator(seed)

    def state(self):
        seed, off = ctypes.c_uint64(), ctypes.c_uint64()
        _host.diopiGeneratorGetSeedAndOffset(ctypes.c_void_p(self.ptr), ctypes.byref(seed), ctypes.byref(off))
        return seed.value, off.value

    def set_state(self, seed, offset):
        _host.diopiGeneratorSetSeedAndOffset(ctypes.c_void_p(self.ptr), ctypes.c_uint64(seed), ctypes.c_uint64(offset))

    def __del__(self):
        if getattr(self, "ptr", None):
            _host.minihostFreeGenerator(ctypes.c_void_p(self.ptr))
            self.ptr = None


def diopiIndex(ctx, self_tensor, indices):
    """diopiIndex allocates its result through diopiRequireTensor (the reference's wrapper passes `&out_ptr`); here the
    result is copied out of the context's workspace into a torch tensor before the workspace is released."""
    fn = _lib.diopiIndex
    fn.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int64]
    fn.restype = ctypes.c_int
    hs = [None if x is None else handle(x) for x in indices]   # None: the whole dimension (torch's `:` before an index)
    arr = (ctypes.c_void_p * max(len(hs), 1))(*[None if h is None else h.ptr for h in hs])
    out = ctypes.c_void_p()
    hself = handle(self_tensor)
    rc = fn(ctx.ptr, ctypes.byref(out), hself.ptr, arr, len(hs))
    if rc != 0:
        raise DiopiError("diopiIndex failed with code %d: %s" % (rc, last_error()))
    size = _Size()
    _host.diopiGetTensorShape(out, ctypes.byref(size))
    shape = [size.data[i] for i in range(size.len)]
    data = ctypes.c_void_p()
    _host.diopiGetTensorData(out, ctypes.byref(data))
    result = torch.empty(shape, dtype=self_tensor.dtype, device=self_tensor.device)
    nbytes = result.numel() * result.element_size()
    if nbytes:
        from . import devapis
        devapis.memCopyD2DAsync(ctx.stream, nbytes, ctx.device, result.data_ptr(), ctx.device, data.value)
    return result


def diopiB200MmPush(ctx, mat1, mat2, space, slot, epoch, prev_epoch):
    """This rank's partial product mat1 [M, K] x mat2 [K, N], pushed piece by piece into the peers' staging slots (see
    include/diopi/functions_b200.h). `space` is a devapis.PeerSpace; pair every call with space.reduce_gather()."""
    fn = _lib.diopiB200MmPush
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_uint32, ctypes.c_uint32]
    fn.restype = ctypes.c_int
    h1, h2 = handle(mat1), handle(mat2)
    rc = fn(ctx.ptr, h1.ptr, h2.ptr, ctypes.addressof(space.desc), int(slot), int(epoch), int(prev_epoch))
    if rc != 0:
        raise DiopiError("diopiB200MmPush failed with code %d: %s" % (rc, last_error()))
    return rc


def last_error():
    return _lib.diopiGetLastErrorString().decode()


def vendor_name():
    return _lib.diopiGetVendorName().decode()


def gemm_status():
    """0 unless a bounded wait inside a tensor-core kernel ever timed out on the current device (synchronises)."""
    return _lib.diopiB200GemmStatus()


def __getattr__(name):
    if name in SIGNATURES:
        f = _bind(name)
        globals()[name] = f
        return f
    raise AttributeError(name)


def exported_functions():
    return sorted(SIGNATURES)
