"""Eager adapter in DIPU's shape: `import` this module and an unmodified torch program runs its hot-path ops on
`torch.device("dipu")` through the DIOPI C-ABI.

What DIPU does with its generated wrappers (reference dipu/scripts/autogen_diopi_wrapper/diopi_wrapper_template.py:100-142:
per aten op a C++ function registered on DIPU's dispatch key that allocates the outputs, builds a diopiContext on the
current stream and calls ::diopiXxx) is done here by `lib/libtorch_dipu_b200.so` for the ops of the transformer-inference
path, on torch's PrivateUse1 key renamed to "dipu" (the device name of the reference's python package,
dipu/torch_dipu/__init__.py). Memory comes from the vendor runtime's caching allocator, copies go through the vendor's
copy calls and diopiCopyInp. There is no CPU fallback: an aten op without a wrapper raises torch's NotImplementedError.
"""
import ctypes
import os

import torch

from . import _native  # noqa: F401  (loads the vendor runtime, the minimal DIOPI host and the operator library)

_LIB = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libtorch_dipu_b200.so")
if not os.path.exists(_LIB):
    raise ImportError("libtorch_dipu_b200.so is not built: run `python __graft_entry__.py` (build) first")
torch.ops.load_library(_LIB)
_handle = ctypes.CDLL(_LIB)
_handle.dipu_b200_adapter_stats.argtypes = [ctypes.POINTER(ctypes.c_int64)] * 3


class _DeviceModule:
    """What torch expects of `torch.<backend name>`: a few queries used by tensor printing, `.to()` and generators."""

    @staticmethod
    def is_available():
        from . import devapis
        try:
            return devapis.getDeviceCount() > 0
        except Exception:
            return False

    @staticmethod
    def device_count():
        from . import devapis
        return devapis.getDeviceCount()

    @staticmethod
    def current_device():
        from . import devapis
        return devapis.current_device()

    @staticmethod
    def set_device(index):
        from . import devapis
        devapis.setDevice(int(index))

    @staticmethod
    def synchronize(device=None):
        from . import devapis
        devapis.syncDevice()

    @staticmethod
    def is_initialized():
        return True

    @staticmethod
    def _is_in_bad_fork():
        return False

    @staticmethod
    def manual_seed_all(seed):
        return None


torch._register_device_module("dipu", _DeviceModule)
torch.utils.generate_methods_for_privateuse1_backend(for_tensor=True, for_module=True, for_storage=False)


def _load_c10d():
    import glob
    import importlib.util
    paths = glob.glob(os.path.join(os.path.dirname(_LIB), "dipu_b200_c10d*.so"))
    if not paths:
        return None
    spec = importlib.util.spec_from_file_location("dipu_b200_c10d", paths[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


_c10d = _load_c10d()
if _c10d is not None:
    import torch.distributed as _dist

    def _create_dicl(store, rank, size, timeout):
        """What the reference's torch_dipu/dipu/distributed.py:22-27 registers: the creator of the "dicl" backend."""
        return _c10d.create_process_group_dicl(store, rank, size, timeout)

    if not hasattr(_dist.Backend, "DICL"):
        _dist.Backend.register_backend("dicl", _create_dicl, devices=["dipu"])


def stats():
    """(DIOPI calls issued, device allocations served, host<->device copies) since the library was loaded."""
    a, b, c = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
    _handle.dipu_b200_adapter_stats(ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))
    return {"diopi_calls": a.value, "allocations": b.value, "host_copies": c.value}
