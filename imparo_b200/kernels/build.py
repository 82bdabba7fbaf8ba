"""Compiles the engine's native code in the source tree, at first use.

Two libraries: the sm_100a kernels (nvcc, csrc/kernels/*.cu) and the host runtime (g++,
csrc/host/*.cpp).  Objects and libraries go to imparo_b200/_build/; when that folder
cannot be written, to a per-user folder under the temporary directory.  A library is
rebuilt only when a source, a header or a flag changed.  Progress goes to stderr, one
line per file and one now and then while a compiler runs.
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(_PKG, "csrc")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-cudart", "shared"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[imparo_b200 build] {msg}", file=sys.stderr, flush=True)


def _find_nvcc() -> str:
    for cand in (os.environ.get("IMPARO_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc not found (looked at $IMPARO_NVCC, PATH and /usr/local/cuda/bin): "
                     "the CUDA kernels cannot be compiled and there is no other path")


def build_dir() -> str:
    d = os.environ.get("IMPARO_BUILD_DIR") or os.path.join(_PKG, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"imparo_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _sources(sub: str, ext: str):
    folder = os.path.join(CSRC, sub)
    srcs = sorted(os.path.join(folder, f) for f in os.listdir(folder) if f.endswith(ext))
    hdrs = sorted(os.path.join(folder, f) for f in os.listdir(folder) if f.endswith((".cuh", ".h", ".hpp")))
    return srcs, hdrs


def _digest(paths, flags) -> str:
    h = hashlib.sha256()
    for p in paths:
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    # the checkout's own path (it is in the include flags) is no part of what was compiled:
    # a tree that was built and then copied elsewhere stays built
    h.update(" ".join(flags).replace(_PKG, "<package>").encode())
    return h.hexdigest()


def _run(cmd, what: str) -> None:
    done = threading.Event()

    def beat():
        t0 = time.time()
        while not done.wait(15.0):
            _say(f"... still compiling {what} ({int(time.time() - t0)} s)")
    th = threading.Thread(target=beat, daemon=True)
    th.start()
    try:
        env = dict(os.environ)
        env.setdefault("TMPDIR", tempfile.gettempdir())
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    finally:
        done.set()
    if r.returncode != 0:
        raise BuildError(f"compiling {what} failed:\n$ {' '.join(cmd)}\n{r.stdout}")


def _build(name: str, sub: str, ext: str, compiler: str, cflags, link_cmd_tail, variant: str = "") -> str:
    out_dir = build_dir()
    lib = os.path.join(out_dir, f"lib{name}.so")
    srcs, hdrs = _sources(sub, ext)
    if not srcs:
        raise BuildError(f"no {ext} sources under {os.path.join(CSRC, sub)}")
    digest = _digest(srcs + hdrs, [compiler] + list(cflags) + list(link_cmd_tail))
    stamp = lib + ".stamp"

    def fresh() -> bool:
        try:
            with open(stamp) as f:
                return f.read().strip() == digest and os.path.isfile(lib)
        except OSError:
            return False
    if fresh():
        return lib
    with open(os.path.join(out_dir, f".{name}.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if fresh():
            return lib
        t0 = time.time()
        _say(f"compiling {len(srcs)} files for lib{name}.so into {out_dir}")
        objs = []

        def one(src):
            obj = os.path.join(out_dir, os.path.basename(src) + variant + ".o")
            # per-file digest: only changed files are recompiled
            d = _digest([src] + hdrs, [compiler] + list(cflags))
            ostamp = obj + ".stamp"
            try:
                with open(ostamp) as f:
                    if f.read().strip() == d and os.path.isfile(obj):
                        return obj
            except OSError:
                pass
            _run([compiler] + list(cflags) + ["-c", src, "-o", obj], os.path.basename(src))
            with open(ostamp, "w") as f:
                f.write(d)
            _say(f"compiled {os.path.basename(src)}")
            return obj
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            objs = list(pool.map(one, srcs))
        tmp = lib + f".tmp{os.getpid()}"
        _run([compiler, "-shared", "-o", tmp] + objs + list(link_cmd_tail), f"lib{name}.so (link)")
        os.replace(tmp, lib)
        with open(stamp, "w") as f:
            f.write(digest)
        _say(f"lib{name}.so ready in {time.time() - t0:.0f} s")
    return lib


def timeline_build() -> bool:
    """IMPARO_TIMELINE=1 selects a second build of the kernels that stamps a device timeline
    (kernels/timeline.py); it has its own objects and library name."""
    return os.environ.get("IMPARO_TIMELINE", "") not in ("", "0")


def build_kernels() -> str:
    """-> path of the CUDA kernel library (sm_100a)."""
    nvcc = _find_nvcc()
    cuda_lib = os.path.join(os.path.dirname(os.path.dirname(nvcc)), "lib64")
    tail = ["-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "shared", "-Xcompiler", "-fPIC",
            f"-L{cuda_lib}", "-lcublas", "-Xlinker", f"-rpath={cuda_lib}"]
    flags = NVCC_FLAGS + ["-I", os.path.join(CSRC, "kernels")]
    if timeline_build():
        return _build("imparo_b200_kernels_timeline", "kernels", ".cu", nvcc, flags + ["-DIMPARO_TIMELINE"], tail, variant=".tl")
    return _build("imparo_b200_kernels", "kernels", ".cu", nvcc, flags, tail)


def build_host() -> str:
    """-> path of the host runtime library (cache manager, scheduler)."""
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise BuildError("no C++ compiler found for the host runtime (g++)")
    return _build("imparo_b200_host", "host", ".cpp", cxx, CXX_FLAGS + ["-I", os.path.join(CSRC, "host")], [])


def build_all():
    return build_host(), build_kernels()
