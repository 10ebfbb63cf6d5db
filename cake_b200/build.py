"""Builds libcake_b200.so in-tree with nvcc for sm_100a (the only target; no fallbacks).

    python -m cake_b200.build            # or: from cake_b200.build import build; build()
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SO = os.path.join(HERE, "libcake_b200.so")
SRC = os.path.join(HERE, "csrc", "cake_b200.cu")


def _nccl_include() -> str:
    try:
        import nvidia.nccl  # type: ignore
        return os.path.join(os.path.dirname(nvidia.nccl.__file__), "include")
    except Exception:
        for p in sys.path:
            cand = os.path.join(p, "nvidia", "nccl", "include")
            if os.path.exists(os.path.join(cand, "nccl.h")):
                return cand
    return "/usr/include"


def sources():
    d = os.path.join(HERE, "csrc")
    return [os.path.join(d, f) for f in sorted(os.listdir(d)) if f.endswith((".cu", ".cuh"))] + \
           [os.path.join(ROOT, "include", "cake_b200.h")]


def stale() -> bool:
    if not os.path.exists(SO):
        return True
    t = os.path.getmtime(SO)
    return any(os.path.getmtime(s) > t for s in sources())


# translation units of the library: object file -> (source, the files it depends on besides itself; None = everything in csrc/)
UNITS = {
    "cake_b200.o": ("cake_b200.cu", None),
    "mixers.o": ("mixers.cu", ("mixers.cuh", "common.cuh")),
    "mixers_window.o": ("mixers_window.cu", ("mixers.cuh", "common.cuh")),
}


def _unit_stale(obj: str, src: str, deps) -> bool:
    d = os.path.join(HERE, "csrc")
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    others = {os.path.join(d, s_) for _, (s_, _) in UNITS.items() if s_ != src}   # another unit's .cu is not a dependency
    files = [f for f in sources() if f not in others] if deps is None else [os.path.join(d, src)] + [os.path.join(d, x) for x in deps]
    return any(os.path.getmtime(f) > t for f in files)


def build(force: bool = False, verbose: bool = False, host: bool = True, quiet: bool = False) -> str:
    """``host=False``: only the library (what the Python host needs); ``quiet``: the compiler's output goes to stderr.
    Every translation unit is compiled to an object file beside its source (stale ones only, side by side), then linked."""
    if not force and not stale():
        if host:
            build_host()
        return SO
    from concurrent.futures import ThreadPoolExecutor
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
             "-ccbin", "/usr/bin/g++", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
             "-I", _nccl_include(), "-I", os.path.join(ROOT, "include")]
    if verbose:
        flags = ["-Xptxas", "-v"] + flags
    out = sys.stderr if quiet else None
    d = os.path.join(HERE, "csrc")

    def compile_unit(item):
        obj, (src, deps) = item
        obj = os.path.join(d, obj)
        if force or _unit_stale(obj, src, deps):
            tmp = obj + f".{os.getpid()}.tmp"
            subprocess.check_call([nvcc, *flags, "-c", os.path.join(d, src), "-o", tmp], stdout=out)
            os.replace(tmp, obj)
        return obj

    with ThreadPoolExecutor(max_workers=len(UNITS)) as ex:
        objs = list(ex.map(compile_unit, UNITS.items()))
    tmp = SO + f".{os.getpid()}.tmp"   # written beside the target and renamed: a concurrent reader never maps half a library
    subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-ccbin", "/usr/bin/g++", "-o", tmp, *objs, "-ldl"],
                          stdout=out)
    os.replace(tmp, SO)
    if host:
        build_host(force=True)
    return SO


def build_trace(defines=("-DMK_TRACE=1",), name="libcake_b200_trace.so") -> str:
    """A/B builds of the same library with extra -D switches, written next to the product library (selected at run time with
    CAKE_B200_LIB=<path>, bench_tools/ab.sh).  Profiling aid only; nothing in the product uses it."""
    out = os.path.join(HERE, name)
    if os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(s) for s in sources()):
        return out
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", *defines,
                           "-ccbin", "/usr/bin/g++", "-Xcompiler", "-fPIC", "-shared", "--expt-relaxed-constexpr",
                           "-I", _nccl_include(), "-I", os.path.join(ROOT, "include"), "-o", out, SRC,
                           os.path.join(HERE, "csrc", "mixers.cu"), os.path.join(HERE, "csrc", "mixers_window.cu"), "-ldl"])
    return out


def build_host(force: bool = False) -> str:
    """The C++ host side (cake_b200/host/cake_host.hpp, cake_wire.hpp) + its drivers `cake_run` and `cake_worker`,
    linked against the C ABI."""
    hdrs = [os.path.join(HERE, "host", "cake_host.hpp"), os.path.join(HERE, "host", "cake_wire.hpp"),
            os.path.join(ROOT, "include", "cake_b200.h")]
    for name in ("cake_run", "cake_worker"):
        out = os.path.join(HERE, "host", name)
        src = out + ".cc"
        if not force and os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(d) for d in [src] + hdrs):
            continue
        subprocess.check_call(["/usr/bin/g++", "-std=c++17", "-O2", "-Wall", "-o", out, src, "-I", os.path.join(ROOT, "include"),
                               "-L", HERE, "-lcake_b200", "-pthread", "-Wl,-rpath,$ORIGIN/.."])
    return os.path.join(HERE, "host", "cake_run")


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
