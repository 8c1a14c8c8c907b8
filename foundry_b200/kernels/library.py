"""Building and loading the kernel library (`csrc/*.cu` -> one shared object).

The kernels are compiled with nvcc for sm_100a only and loaded through their
`extern "C"` launchers with ctypes. The library is built in the source tree
(`csrc/_build/`) when that is writable, else under `$FOUNDRY_B200_BUILD_DIR`
or a per-user temporary folder; nothing is written to `$HOME`. It is rebuilt
when a source or a flag changed. There is no other implementation to fall back
to: if the library can be neither found nor built, importing the kernels
fails with the compiler's message.
"""
from __future__ import annotations

import ctypes
import glob
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

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
LIB_NAME = "libfoundry_b200.so"
ABI_VERSION = 2
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
] + os.environ.get("FOUNDRY_B200_NVCC_EXTRA", "").split()


class KernelLibraryError(RuntimeError):
    """The CUDA kernel library is missing and cannot be built, or is unusable."""


def sources() -> List[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _headers() -> List[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")))


def source_digest() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for path in sources() + _headers():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as handle:
            h.update(handle.read())
    return h.hexdigest()[:16]


def _find_nvcc() -> Optional[str]:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    return None


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe-{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    override = os.environ.get("FOUNDRY_B200_BUILD_DIR")
    if override:
        os.makedirs(override, exist_ok=True)
        return override
    in_tree = os.path.join(CSRC, "_build")
    if _writable_dir(in_tree):
        return in_tree
    fallback = os.path.join(tempfile.gettempdir(), f"foundry_b200-build-{os.getuid()}")
    os.makedirs(fallback, exist_ok=True)
    return fallback


def _log(message: str) -> None:
    print(f"[foundry_b200] {message}", file=sys.stderr, flush=True)


def build(force: bool = False, verbose: bool = True) -> str:
    """Compile every `.cu` for sm_100a and link the shared object; returns its
    path. A build that is already up to date returns at once."""
    out_dir = build_dir()
    lib_path = os.path.join(out_dir, LIB_NAME)
    stamp_path = lib_path + ".stamp"
    digest = source_digest()
    if not force and os.path.exists(lib_path) and os.path.exists(stamp_path):
        with open(stamp_path) as handle:
            if handle.read().strip() == digest:
                return lib_path
    nvcc = _find_nvcc()
    if nvcc is None:
        raise KernelLibraryError(
            f"{lib_path} is absent or stale and nvcc was not found (set NVCC or PATH); "
            "the CUDA kernels have no substitute")
    srcs = sources()
    if verbose:
        _log(f"compiling {len(srcs)} CUDA sources for sm_100a into {out_dir} ...")
    started = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _log(f"still compiling ({time.time() - started:.0f} s)")

    beat = threading.Thread(target=heartbeat, daemon=True)
    if verbose:
        beat.start()

    def compile_one(src: str) -> str:
        obj = os.path.join(out_dir, os.path.basename(src)[:-3] + f".{os.getpid()}.o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise KernelLibraryError(f"nvcc failed on {src}:\n{proc.stdout}\n{proc.stderr}")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            objects = list(pool.map(compile_one, srcs))
        tmp_lib = f"{lib_path}.{os.getpid()}.tmp"
        proc = subprocess.run([nvcc, "-shared", "-o", tmp_lib, *objects, "-gencode",
                               "arch=compute_100a,code=sm_100a"], capture_output=True, text=True)
        if proc.returncode != 0:
            raise KernelLibraryError(f"linking failed:\n{proc.stdout}\n{proc.stderr}")
        os.replace(tmp_lib, lib_path)
        with open(stamp_path, "w") as handle:
            handle.write(digest)
    finally:
        done.set()
        # also the objects of sources that compiled before another one failed
        for src in srcs:
            try:
                os.remove(os.path.join(out_dir, os.path.basename(src)[:-3] + f".{os.getpid()}.o"))
            except OSError:
                pass
    if verbose:
        _log(f"built {LIB_NAME} in {time.time() - started:.0f} s")
    return lib_path


_LIB: Optional[ctypes.CDLL] = None
_LOCK = threading.Lock()


def load() -> ctypes.CDLL:
    """The loaded library; built first if needed."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is None:
            path = build()
            try:
                lib = ctypes.CDLL(path)
            except OSError as exc:
                raise KernelLibraryError(f"cannot load {path}: {exc}") from exc
            lib.fb_last_error.restype = ctypes.c_char_p
            lib.fb_abi_version.restype = ctypes.c_int
            if lib.fb_abi_version() != ABI_VERSION:
                raise KernelLibraryError(
                    f"{path} has ABI version {lib.fb_abi_version()}, expected {ABI_VERSION}")
            _LIB = lib
    return _LIB
