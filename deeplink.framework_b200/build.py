"""Build recipe for the three native libraries (nvcc, sm_100a only).

    lib/libdipu_vendor_b200.so   vendor runtime: device / stream / event / memory API, caching allocators,
                                 stream and event pools, DICL communicator (NCCL bound at run time)
    lib/libdiopirt_minihost.so   a small DIOPI host (the diopirt callbacks over plain tensor structs)
    lib/libdiopi_impl.so         the DIOPI operator library: hand-written sm_100a kernels
    lib/libtorch_dipu_b200.so             hot-path aten ops on the PrivateUse1 key ("dipu"), each wrapper calling ::diopiXxx
    lib/dipu_b200_c10d.<abi>.so           the c10d backend "dicl" (torch.distributed on dipu tensors) as a Python extension module
    lib/libdipu_vendor_b200_torchabi.so   the vendor contract with DIPU's exact C++ signatures (namespace dipu::devapis, torch
                                 types in the arguments): thin wrappers over the C-ABI runtime, built when torch's headers are present

Objects go to build/ (ignored by git), libraries to lib/ next to this file so that they travel with the tree.
Run as a script or call build().
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(ROOT, "build", "obj")
LIB = os.path.join(HERE, "lib")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", os.path.join(ROOT, "include"),
          "-diag-suppress", "177"]


def _nccl_include():
    try:
        import nvidia.nccl  # noqa: F401  (namespace package shipped with torch's wheels)
        for p in nvidia.nccl.__path__:
            inc = os.path.join(p, "include")
            if os.path.exists(os.path.join(inc, "nccl.h")):
                return inc
    except Exception:
        pass
    for inc in ("/usr/include", "/usr/local/cuda/include"):
        if os.path.exists(os.path.join(inc, "nccl.h")):
            return inc
    raise RuntimeError("nccl.h not found")


def _sources(sub):
    d = os.path.join(CSRC, sub)
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith((".cu", ".cpp")))


def _headers():
    out = []
    for base in (CSRC, os.path.join(ROOT, "include")):
        for dp, _, fs in os.walk(base):
            out += [os.path.join(dp, f) for f in fs if f.endswith((".h", ".cuh", ".hpp"))]
    return out


def _compile(src, extra):
    rel = os.path.relpath(src, CSRC).replace(os.sep, "_")
    obj = os.path.join(OBJ, rel + ".o")
    newest = max([os.path.getmtime(src), os.path.getmtime(__file__)] + [os.path.getmtime(h) for h in _headers()])
    if os.path.exists(obj) and os.path.getmtime(obj) >= newest:
        return obj
    cmd = [NVCC] + ARCH + COMMON + extra + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    return obj


def _link(name, objs, extra):
    out = os.path.join(LIB, name)
    if os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(o) for o in objs):
        return out
    cmd = [NVCC] + ARCH + ["-shared", "-o", out] + objs + extra
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed for %s:\n%s\n%s" % (name, r.stdout, r.stderr))
    return out


def _build_torch_abi(vendor_lib, verbose):
    """csrc/torch_abi/*.cpp: the files a DIPU tree would compile as csrc_dipu/vendor/b200/. Needs torch's C++ headers."""
    return _build_torch_lib("torch_abi", "libdipu_vendor_b200_torchabi.so", ["-l:libdipu_vendor_b200.so"], verbose)


def _build_torch_adapter(verbose):
    """csrc/torch_adapter/*.cpp: hot-path aten ops on the PrivateUse1 key ("dipu"), each wrapper calling ::diopiXxx."""
    return _build_torch_lib("torch_adapter", "libtorch_dipu_b200.so",
                            ["-l:libdipu_vendor_b200.so", "-l:libdiopirt_minihost.so", "-l:libdiopi_impl.so"], verbose)


def _build_torch_c10d(verbose):
    """csrc/torch_c10d/*.cpp: the c10d backend "dicl" as a Python extension module (pybind11 from torch's headers)."""
    import sysconfig
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    py_inc = sysconfig.get_paths()["include"]
    if not os.path.exists(os.path.join(py_inc, "Python.h")):
        return None
    return _build_torch_lib("torch_c10d", "dipu_b200_c10d" + suffix, ["-l:libtorch_dipu_b200.so", "-l:libdipu_vendor_b200.so"], verbose,
                            extra_cflags=["-DTORCH_EXTENSION_NAME=dipu_b200_c10d", "-I", py_inc], extra_link=["-ltorch_python", "-ltorch"])


def _build_torch_lib(sub, out_name, link_libs, verbose, extra_cflags=(), extra_link=()):
    try:
        import torch
        from torch.utils.cpp_extension import include_paths
        incs = include_paths()
        torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    except Exception:
        return None
    srcs = sorted(os.path.join(CSRC, sub, f) for f in os.listdir(os.path.join(CSRC, sub)) if f.endswith(".cpp"))
    objs = []
    newest_hdr = max(os.path.getmtime(h) for h in _headers())
    for src in srcs:
        obj = os.path.join(OBJ, sub + "_" + os.path.basename(src) + ".o")
        if not (os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), newest_hdr, os.path.getmtime(__file__))):
            cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-fvisibility=hidden", "-c", src, "-o", obj, "-I", os.path.join(ROOT, "include"),
                   "-I", "/usr/local/cuda/include"] + ["-I" + p for p in incs] + list(extra_cflags)
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError("g++ failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
            if verbose:
                print("compiled", os.path.relpath(src, ROOT), flush=True)
        objs.append(obj)
    out = os.path.join(LIB, out_name)
    if not (os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(o) for o in objs)):
        cmd = ["g++", "-shared", "-o", out] + objs + ["-L", LIB] + link_libs + ["-L", torch_lib] + list(extra_link) + ["-lc10", "-ltorch_cpu",
                                                       "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + torch_lib]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed for %s:\n%s\n%s" % (out, r.stdout, r.stderr))
    return out


def build(verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB, exist_ok=True)
    jobs = []
    for sub, extra in (("vendor", ["-I", _nccl_include()]), ("minihost", []), ("diopi", [])):
        for src in _sources(sub):
            jobs.append((sub, src, extra))
    # csrc/torch_abi is compiled separately (g++ against torch's headers), see _build_torch_abi
    objs = {"vendor": [], "minihost": [], "diopi": []}
    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, os.cpu_count() or 1)) as ex:
        futs = {ex.submit(_compile, src, extra): (sub, src) for sub, src, extra in jobs}
        for f in concurrent.futures.as_completed(futs):
            sub, src = futs[f]
            objs[sub].append(f.result())
            if verbose:
                print("compiled", os.path.relpath(src, ROOT), flush=True)
    for k in objs:
        objs[k].sort()
    vendor = _link("libdipu_vendor_b200.so", objs["vendor"], ["-ldl", "-lpthread"])
    _link("libdiopirt_minihost.so", objs["minihost"],
          ["-L", LIB, "-l:libdipu_vendor_b200.so", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"])
    # the diopirt callbacks stay undefined here: the host that loads this library provides them (DIPU, or the minihost)
    _link("libdiopi_impl.so", objs["diopi"], [])
    built = [vendor, os.path.join(LIB, "libdiopirt_minihost.so"), os.path.join(LIB, "libdiopi_impl.so")]
    abi = _build_torch_abi(vendor, verbose)
    if abi:
        built.append(abi)
    adapter = _build_torch_adapter(verbose)
    if adapter:
        built.append(adapter)
        c10d = _build_torch_c10d(verbose)
        if c10d:
            built.append(c10d)
    return built


if __name__ == "__main__":
    for p in build(verbose=True):
        print("built", p)
