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

__all__ = ["devapis", "diopi"]
