"""Compiles the CUDA sources of this folder for sm_100a into two shared libraries and loads them.

``core`` (``_build/libtitan_b200.so``): what every model needs in either dtype (element-wise kernels,
the CUDA-core matrix product and attention, sampling).  ``tensor``
(``_build/libtitan_b200_tensor.so``): the tcgen05 / TMA / mma.sync kernels that bfloat16 runs use; it
is built and loaded when the first of them is asked for, so a float32 run never compiles it.  Each is
built in-tree by calling nvcc directly: one object per source, in parallel, then one link.  A stamp
of the sources' contents decides whether a build is current, so a fresh checkout compiles at its
first call and later calls only load.  If the tree cannot be
written, the build goes to a per-user folder under the system's temporary
directory.  Progress is printed to stderr, a line per file and one every few
seconds while nvcc runs.

There is no fallback: without nvcc or with a failing build, ``load`` raises.
berniehans/titan compiles its kernels at run time too, through NVRTC for
compute_86 (engine/engine-cuda/src/batched_gemm.rs:324-336).
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
LIBS = {"core": "libtitan_b200.so", "tensor": "libtitan_b200_tensor.so"}
TENSOR_SOURCES = ("gemm_tc.cu", "attention_mma.cu", "attention_tc.cu", "tma_host.cu")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fvisibility=default"]

_libs = {}
_lock = threading.RLock()


class BuildError(RuntimeError):
    pass


def sources(which: Optional[str] = None) -> List[str]:
    """The sources of one library ("core", "tensor") or of both (None)."""
    every = sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))
    if which is None:
        return every
    return [f for f in every if (f in TENSOR_SOURCES) == (which == "tensor")]


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def find_nvcc() -> str:
    for cand in (os.environ.get("TITAN_B200_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (CUDA_HOME, /usr/local/cuda/bin, PATH); the kernels cannot be built")


def _extra_flags() -> List[str]:
    """More nvcc flags from the environment (TITAN_B200_NVCC_FLAGS), for experiments such as -DNAME."""
    return os.environ.get("TITAN_B200_NVCC_FLAGS", "").split()


def _stamp(which: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + _extra_flags()).encode())
    for f in sources(which) + _headers():
        h.update(f.encode())
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _writable(d: str) -> bool:
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    d = os.environ.get("TITAN_B200_BUILD_DIR") or os.path.join(HERE, "_build")
    if _writable(d):
        return d
    d = os.path.join(tempfile.gettempdir(), f"titan_b200_build_{os.getuid()}")
    if _writable(d):
        return d
    raise BuildError("no writable folder for the build (tried the source tree and the temporary directory)")


def _say(msg: str) -> None:
    print(f"[titan_b200] {msg}", file=sys.stderr, flush=True)


def _run(cmd: List[str], what: str) -> None:
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=HERE)
    if p.returncode != 0:
        raise BuildError(f"{what} failed:\n{' '.join(cmd)}\n{p.stdout}")


def build(force: bool = False, verbose_ptxas: bool = False, which: Optional[str] = None) -> str:
    """Build what is missing or stale of one library (or of both, ``which=None``); return the path of the last."""
    if which is None:
        build(force, verbose_ptxas, "core")
        return build(force, verbose_ptxas, "tensor")
    out = build_dir()
    lib = os.path.join(out, LIBS[which])
    stamp_file = os.path.join(out, f"stamp_{which}.txt")
    stamp = _stamp(which)
    if not force and os.path.isfile(lib) and os.path.isfile(stamp_file) and open(stamp_file).read().strip() == stamp:
        return lib
    nvcc = find_nvcc()
    srcs = sources(which)
    _say(f"compiling {len(srcs)} CUDA sources ({which} kernels) for sm_100a into {out} (first call only)")
    t0 = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _say(f"... still compiling ({time.time() - t0:.0f} s)")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    extra = (["-Xptxas", "-v"] if verbose_ptxas else []) + _extra_flags()

    def one(src: str) -> str:
        obj = os.path.join(out, src[:-3] + ".o")
        _run([nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *extra, "-c", src, "-o", obj], f"compiling {src}")
        _say(f"compiled {src} ({time.time() - t0:.0f} s)")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
            objs = list(pool.map(one, srcs))
        tmp = lib + f".{os.getpid()}.tmp"
        _run([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs], "linking")     # the tensor library's few outside symbols resolve against core at load time
        os.replace(tmp, lib)
        with open(stamp_file, "w") as f:
            f.write(stamp)
    finally:
        done.set()
    _say(f"built {LIBS[which]} in {time.time() - t0:.0f} s")
    return lib


def load(which: str = "core") -> ctypes.CDLL:
    """The loaded library; builds it first if need be.  Raises if that fails.  ``tensor`` loads ``core``
    first (with global symbols: error reporting, launch settings and the merge kernel live there)."""
    with _lock:
        if which not in _libs:
            if which == "tensor":
                load("core")
            path = build(which=which)
            try:
                _libs[which] = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
            except OSError as e:
                raise BuildError(f"{path} was built but cannot be loaded: {e}") from None
        return _libs[which]
