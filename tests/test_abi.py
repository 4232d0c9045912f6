"""The C-ABI libraries load without a GPU and export every symbol the headers in include/ declare (no compute calls here)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "include")


def _declared(path, api_macro, prefix):
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set()
    for m in re.finditer(r"%s\s+[\w\s\*]+?\b(%s\w+)\s*\(" % (api_macro, prefix), text):
        names.add(m.group(1))
    return names


def test_operator_library_exports_declared_functions(pkg):
    lib = pkg._native.diopi
    declared = set()
    for h in ("functions.h", "functions_ext.h", "functions_b200.h"):
        declared |= _declared(os.path.join(INC, "diopi", h), "DIOPI_API", "diopi")
    declared |= {"diopiGetVendorName", "diopiGetImplVersion", "diopiGetLastErrorString"}
    assert len(declared) > 70
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, missing
    # and the Python binding knows every DIOPI function of the two DIOPI headers
    for h in ("functions.h", "functions_ext.h"):
        for n in _declared(os.path.join(INC, "diopi", h), "DIOPI_API", "diopi"):
            assert n in pkg.diopi.SIGNATURES or callable(getattr(pkg.diopi, n, None)), n   # diopiIndex has a hand-written binding


def test_host_library_exports_the_diopirt_callbacks(pkg):
    host = pkg._native.host
    text = open(os.path.join(INC, "diopi", "diopirt.h")).read()
    names = set(re.findall(r"DIOPI_RT_API\s+[\w\s\*]+?\b(diopi\w+)\s*\(", text))
    assert "diopiRequireTensor" in names and "diopiGetStream" in names
    missing = [n for n in sorted(names) if not hasattr(host, n)]
    assert not missing, missing


def test_vendor_library_exports_declared_functions(pkg):
    lib = pkg._native.vendor
    declared = _declared(os.path.join(INC, "dipu_b200", "vendor_c_api.h"), "B200_API", "b200_")
    assert len(declared) > 70
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, missing
    assert pkg.devapis.DICL_UNIQUE_ID_BYTES_SIZE == 128
    assert isinstance(pkg.devapis.getDeviceCount(), int)  # works without a GPU (0 devices)


def test_product_does_not_import_the_oracle():
    pkg_dir = os.path.join(ROOT, "deeplink.framework_b200")
    for dp, _, fs in os.walk(pkg_dir):
        for f in fs:
            if f.endswith((".py", ".cpp", ".cu", ".h", ".cuh")):
                assert "oracle" not in open(os.path.join(dp, f)).read(), os.path.join(dp, f)


def test_missing_library_is_an_import_error(tmp_path):
    import importlib.util
    src = os.path.join(ROOT, "deeplink.framework_b200", "_native.py")
    code = open(src).read().replace('os.path.join(_HERE, "lib")', repr(str(tmp_path)))
    p = tmp_path / "_native_copy.py"
    p.write_text(code)
    spec = importlib.util.spec_from_file_location("_native_copy", str(p))
    mod = importlib.util.module_from_spec(spec)
    try:
        spec.loader.exec_module(mod)
    except ImportError as e:
        assert "no CPU or PyTorch fallback" in str(e)
    else:
        raise AssertionError("loading without the libraries must fail")
    assert ctypes.sizeof(ctypes.c_void_p) == 8


def test_torch_abi_library_has_dipu_devapis_signatures(pkg):
    """The wrappers carry DIPU's mangled names: what `libtorch_dipu.so` links when built with -DDEVICE=b200."""
    import subprocess
    import torch  # noqa: F401  (libc10 / libtorch_cpu must be loadable)
    lib = os.path.join(ROOT, "deeplink.framework_b200", "lib", "libdipu_vendor_b200_torchabi.so")
    assert os.path.exists(lib), "build first"
    syms = subprocess.run(["nm", "-DC", "--defined-only", lib], capture_output=True, text=True, check=True).stdout
    for want in ("dipu::devapis::mallocDevice(void**, unsigned long, bool)",
                 "dipu::devapis::createStream(CUstream_st**, bool)",
                 "dipu::devapis::destroyStream(CUstream_st*, signed char)",
                 "dipu::devapis::getEventStatus(CUevent_st*)",
                 "dipu::devapis::memCopyD2DAsync(CUstream_st*, unsigned long, signed char, void*, signed char, void const*)",
                 "dipu::devapis::diclAllReduce(void const*, void*, unsigned long, c10::ScalarType, c10d::ReduceOp const&, b200Comm*, CUstream_st*)",
                 "dipu::devapis::diclCommInitRank(b200Comm**, int, b200UniqueId, int, int)",
                 "dipu::devapis::diclAllToAllUnequalSplit(", "dipu::devapis::diclGetCommName(", "dipu::devapis::DICL_UNIQUE_ID_BYTES_SIZE",
                 "dipu::vendorCreateExpandableSegment(int, CUstream_st*, unsigned long, std::vector<int",
                 "dipu::vendorMakeGenerator(signed char)"):
        assert want in syms, want
    handle = ctypes.CDLL(lib)
    count = getattr(handle, "_ZN4dipu7devapis14getDeviceCountEv")
    count.restype = ctypes.c_int
    assert count() >= 0
    # the RNG state container behind vendorMakeGenerator: seed / offset round trip, clone, offset rule (all host-side)
    selftest = handle.b200_torchabi_generator_selftest
    selftest.restype = ctypes.c_int
    assert selftest() == 0
    # the copy_ policy object registered with setDipuCopyInstance: which path each kind of copy takes (metadata-only tensors)
    copytest = handle.b200_torchabi_copy_selftest
    copytest.restype = ctypes.c_int
    assert copytest() == 0
