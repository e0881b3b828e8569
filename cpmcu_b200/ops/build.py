"""Compiles the CUDA sources under ``csrc/`` for sm_100a into one shared library.

The library is built in the source tree (``cpmcu_b200/_lib``) with plain nvcc, one
object per source in parallel, and rebuilt when a source, a header or a flag
changes.  Where the tree cannot be written, a per-user folder under the system's
temporary folder is used.  The reference builds one torch extension with
setuptools (setup.py:292-379); this library has no torch headers in it, so a cold
build is a matter of seconds per file.
"""
from __future__ import annotations

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

PACKAGE_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC_DIR = os.path.join(PACKAGE_DIR, "csrc")
LIB_NAME = "libcpmcu_b200_kernels.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("CPMCU_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $CPMCU_NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin); "
                     "the kernels of this library are compiled at first use and need it")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


# The checked build: every page number taken from a page table is checked before use (csrc/common.cuh).
BOUNDS_FLAG = "-DCPM_CHECK_BOUNDS"


def _fingerprint(check_bounds: bool = False) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + ([BOUNDS_FLAG] if check_bounds else [])).encode())
    for name in sorted(os.listdir(CSRC_DIR)):
        if name.endswith((".cu", ".cuh", ".h")):
            h.update(name.encode())
            with open(os.path.join(CSRC_DIR, name), "rb") as f:
                h.update(f.read())
    return h.hexdigest()


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe-{os.getpid()}")
        with open(probe, "w") as f:
            f.write("x")
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dirs(check_bounds: bool = False) -> List[str]:
    sub = "_lib_checked" if check_bounds else "_lib"
    dirs = []
    if os.environ.get("CPMCU_BUILD_DIR"):
        dirs.append(os.path.join(os.environ["CPMCU_BUILD_DIR"], "checked") if check_bounds else os.environ["CPMCU_BUILD_DIR"])
    dirs.append(os.path.join(PACKAGE_DIR, "_lib", "checked") if check_bounds else os.path.join(PACKAGE_DIR, "_lib"))
    dirs.append(os.path.join(tempfile.gettempdir(), f"cpmcu_b200-{os.getuid()}", sub))
    return dirs


def _say(msg: str) -> None:
    print(f"[cpmcu_b200 build] {msg}", file=sys.stderr, flush=True)


def existing_library(check_bounds: bool = False) -> Optional[str]:
    """Path of an up-to-date library, or None."""
    fp = _fingerprint(check_bounds)
    for d in build_dirs(check_bounds):
        lib, stamp = os.path.join(d, LIB_NAME), os.path.join(d, "fingerprint")
        try:
            if os.path.isfile(lib) and open(stamp).read().strip() == fp:
                return lib
        except OSError:
            continue
    return None


def build(force: bool = False, verbose: bool = True, check_bounds: bool = False) -> str:
    """Returns the path of the shared library, compiling it if it is stale or absent.  ``check_bounds``: the
    checked build (a library of its own beside the ordinary one)."""
    if not force:
        lib = existing_library(check_bounds)
        if lib:
            return lib
    nvcc = find_nvcc()
    out_dir = next((d for d in build_dirs(check_bounds) if _writable_dir(d)), None)
    if out_dir is None:
        raise BuildError(f"no writable folder to build in (tried {build_dirs(check_bounds)})")
    flags = NVCC_FLAGS + ([BOUNDS_FLAG] if check_bounds else [])
    obj_dir = os.path.join(out_dir, "_build")
    os.makedirs(obj_dir, exist_ok=True)
    srcs = sources()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {out_dir}" + (" (checked build)" if check_bounds else ""))
    t0 = time.time()
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _say(f"still compiling ... {time.time() - t0:.0f} s")

    if verbose:
        threading.Thread(target=ticker, daemon=True).start()

    def compile_one(name: str) -> str:
        obj = os.path.join(obj_dir, name[:-3] + ".o")
        cmd = [nvcc, *flags, "-I", CSRC_DIR, "-c", os.path.join(CSRC_DIR, name), "-o", obj]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise BuildError(f"nvcc failed on {name}:\n{' '.join(cmd)}\n{p.stdout}\n{p.stderr}")
        if verbose:
            _say(f"compiled {name} ({time.time() - t0:.0f} s)")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2, max(1, len(srcs)))) as pool:
            objs = list(pool.map(compile_one, srcs))
        tmp_lib = os.path.join(out_dir, f".{LIB_NAME}.{os.getpid()}")
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp_lib, *objs]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise BuildError(f"link failed:\n{' '.join(cmd)}\n{p.stdout}\n{p.stderr}")
        os.replace(tmp_lib, os.path.join(out_dir, LIB_NAME))
        with open(os.path.join(out_dir, "fingerprint"), "w") as f:
            f.write(_fingerprint(check_bounds))
    finally:
        done.set()
    if verbose:
        _say(f"built {LIB_NAME} in {time.time() - t0:.0f} s")
    return os.path.join(out_dir, LIB_NAME)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, check_bounds="--check-bounds" in sys.argv))
