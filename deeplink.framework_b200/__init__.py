"""B200-native DIPU vendor backend: vendor runtime (devapis / DICL) and DIOPI operator library for sm_100a.

The directory name contains a dot, so the package is imported under the name `dipu_b200`
(see load_package() in __graft_entry__.py at the repository root).

    devapis   mirror of dipu::devapis (device, stream, event, memory, caching allocator, DICL communicator)
    diopi     the DIOPI C-ABI functions, called through a minimal DIOPI host
    layer     the Llama decoder layer as the stream of DIOPI calls DIPU dispatches (harness, not a model zoo)

Importing the package loads the native libraries; it fails if they have not been built.
"""
from . import _native  # noqa: F401  (raises ImportError when the libraries are missing)
from . import devapis, diopi  # noqa: F401

__all__ = ["devapis", "diopi", "install_caching_allocator"]

_allocator_installed = False


def install_caching_allocator():
    """Makes torch allocate every CUDA tensor through this runtime's caching allocator (what DIPU does with
    c10::SetAllocator). Must run before the process allocates any CUDA memory through torch."""
    global _allocator_installed
    if _allocator_installed:
        return
    import torch
    alloc = torch.cuda.memory.CUDAPluggableAllocator(_native.VENDOR_LIB, "b200_torch_alloc", "b200_torch_free")
    torch.cuda.memory.change_current_allocator(alloc)
    _allocator_installed = True
