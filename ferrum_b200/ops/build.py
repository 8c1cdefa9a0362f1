"""Builds the two native libraries of the package, in the source tree.

`libferrum_kernels.so`: the sm_100a kernels (csrc/kernels/*.cu), plain C entry points,
compiled with nvcc.  `_host*.so`: the C++ cache manager and scheduler (csrc/host/*.cpp),
a pybind11 module compiled with g++.  Both are rebuilt when a source is newer than the
library, so a fresh checkout compiles what it needs at its first call and later calls
start at once.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
import sysconfig
import threading
import time

from ..errors import KernelError

PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PKG, "csrc")
KERNEL_LIB = os.path.join(PKG, "libferrum_kernels.so")
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _host_lib_path():
    return os.path.join(PKG, "_host" + sysconfig.get_config_var("EXT_SUFFIX"))


def _newer(sources, target):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _find(tool, extra=()):
    p = shutil.which(tool)
    if p:
        return p
    for d in extra:
        q = os.path.join(d, tool)
        if os.path.exists(q):
            return q
    raise KernelError(f"{tool} not found: the native code of ferrum_b200 cannot be built")


class _Progress:
    """Prints a line now and then while a long compile runs."""

    def __init__(self, what):
        self.what, self._stop = what, threading.Event()
        self._t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        t0 = time.time()
        while not self._stop.wait(10.0):
            print(f"[ferrum_b200] still compiling {self.what} ({time.time() - t0:.0f}s)", file=sys.stderr, flush=True)

    def __enter__(self):
        print(f"[ferrum_b200] compiling {self.what} (first call only)", file=sys.stderr, flush=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()


def _run_all(cmds, what):
    """Run the compile commands in parallel (they are independent translation units)."""
    with _Progress(what):
        procs = [(c, subprocess.Popen(c, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)) for c in cmds]
        for c, p in procs:
            out, _ = p.communicate()
            if p.returncode != 0:
                for _, q in procs:
                    if q.poll() is None:
                        q.kill()
                raise KernelError(f"build failed: {' '.join(c)}\n{out}")


def trace_build():
    """FERRUM_KERNEL_TRACE=1 selects a second library, built with -DFERRUM_TRACE, whose kernels
    record a timeline (see csrc/kernels/common.cuh and `kernel_bench.py timeline`)."""
    return os.environ.get("FERRUM_KERNEL_TRACE", "0") == "1"


def build_kernels(force=False, verbose_ptxas=False):
    srcs = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")))
    hdrs = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cuh")) + glob.glob(os.path.join(CSRC, "kernels", "*.h")))
    if not srcs:
        raise KernelError("no kernel sources found")
    trace = trace_build()
    target = KERNEL_LIB[:-3] + "_trace.so" if trace else KERNEL_LIB
    if not force and not _newer(srcs + hdrs, target):
        return target
    nvcc = _find("nvcc", ["/usr/local/cuda/bin"])
    bdir = os.path.join(PKG, "_build", "trace") if trace else os.path.join(PKG, "_build")
    os.makedirs(bdir, exist_ok=True)
    objs, cmds = [], []
    for s in srcs:
        o = os.path.join(bdir, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer([s] + hdrs, o):
            cmd = [nvcc, *NVCC_ARCH, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden",
                   "-c", s, "-o", o]
            if verbose_ptxas:
                cmd[1:1] = ["-Xptxas", "-v"]
            if trace:
                cmd[1:1] = ["-DFERRUM_TRACE"]
            cmds.append(cmd)
    if cmds:
        _run_all(cmds, f"{len(cmds)} CUDA source(s) for sm_100a")
    tmp = target + f".tmp{os.getpid()}"
    link = [nvcc, *NVCC_ARCH, "-shared", "-o", tmp, *objs]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise KernelError(f"link failed: {' '.join(link)}\n{r.stdout}")
    os.replace(tmp, target)
    return target


def build_host(force=False):
    srcs = sorted(glob.glob(os.path.join(CSRC, "host", "*.cpp")))
    hdrs = sorted(glob.glob(os.path.join(CSRC, "host", "*.hpp")))
    target = _host_lib_path()
    if not force and not _newer(srcs + hdrs, target):
        return target
    import pybind11
    gxx = _find("g++")
    tmp = target + f".tmp{os.getpid()}"
    cmd = [gxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
           "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], *srcs, "-o", tmp]
    _run_all([cmd], "the C++ cache manager and scheduler")
    os.replace(tmp, target)
    return target


def build_all(force=False):
    return build_host(force), build_kernels(force)
