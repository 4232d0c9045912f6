"""Loads the three native libraries. There is no fallback: a missing library is an ImportError."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(_HERE, "lib")

VENDOR_LIB = os.path.join(LIB_DIR, "libdipu_vendor_b200.so")
HOST_LIB = os.path.join(LIB_DIR, "libdiopirt_minihost.so")
DIOPI_LIB = os.path.join(LIB_DIR, "libdiopi_impl.so")


def _point_at_bundled_nccl():
    """The DICL layer dlopens NCCL lazily; prefer the copy that ships with the installed torch wheels."""
    if os.environ.get("B200_NCCL_LIBRARY"):
        return
    try:
        import nvidia.nccl as _n
        for p in _n.__path__:
            cand = os.path.join(p, "lib", "libnccl.so.2")
            if os.path.exists(cand):
                os.environ["B200_NCCL_LIBRARY"] = cand
                return
    except Exception:
        pass


def _load(path):
    if not os.path.exists(path):
        raise ImportError(
            "%s is missing: build the native code first (python __graft_entry__.py build, or "
            "python deeplink.framework_b200/build.py). This package has no CPU or PyTorch fallback." % path)
    # RTLD_GLOBAL: the operator library resolves the diopirt callbacks against the host library, as it would against DIPU
    return ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)


_point_at_bundled_nccl()
vendor = _load(VENDOR_LIB)
host = _load(HOST_LIB)
diopi = _load(DIOPI_LIB)
