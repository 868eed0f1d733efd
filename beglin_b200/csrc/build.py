"""Compiling the CUDA sources of this folder into one shared library for sm_100a, and loading it.

`nvcc` compiles every `.cu` file to an object (in parallel) and links `libbeglin_b200.so`.  The
library has a C interface and includes no framework headers, so a fresh checkout builds in well
under a minute.  It is built at the first call that needs it: into `_build/` beside the sources,
or, when that folder cannot be written, into a per-user folder under the system's temporary
directory.  A stamp with a hash of the sources and flags decides whether a build is current.  While
it compiles it prints a line per file to stderr.
"""
from __future__ import annotations

import ctypes
import fcntl
import glob
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libbeglin_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--threads", "2"] + ARCH_FLAGS

_lib: Optional[ctypes.CDLL] = None


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    cands = [os.environ.get("NVCC"), shutil.which("nvcc")]
    for home in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if home:
            cands.append(os.path.join(home, "bin", "nvcc"))
    for c in cands:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc not found (looked at $NVCC, PATH, $CUDA_HOME/bin and /usr/local/cuda/bin); "
                     "the CUDA kernels of beglin_b200 cannot be built")


def sources() -> List[str]:
    return sorted(glob.glob(os.path.join(HERE, "*.cu")))


def _source_hash() -> str:
    h = hashlib.sha1()
    for path in sources() + sorted(glob.glob(os.path.join(HERE, "*.cuh"))) + sorted(glob.glob(os.path.join(HERE, "*.h"))):
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    forced = os.environ.get("BEGLIN_B200_BUILD_DIR")
    if forced:
        os.makedirs(forced, exist_ok=True)
        return forced
    local = os.path.join(HERE, "_build")
    if _writable_dir(local):
        return local
    fallback = os.path.join(tempfile.gettempdir(), f"beglin_b200_build_{os.getuid()}")
    if _writable_dir(fallback):
        return fallback
    raise BuildError(f"no writable folder for the build: tried {local} and {fallback}")


def _say(msg: str) -> None:
    print(f"[beglin_b200] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: str, obj: str) -> None:
    _say(f"compiling {os.path.basename(src)} for sm_100a ...")
    t0 = time.time()
    cmd = [nvcc] + NVCC_FLAGS + ["-I", HERE, "-c", src, "-o", obj]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{r.stdout}")
    _say(f"compiled {os.path.basename(src)} in {time.time() - t0:.1f} s")


def build(verbose: bool = True) -> str:
    """Build the library if it is not current; return its path."""
    out = build_dir()
    lib = os.path.join(out, LIB_NAME)
    stamp = os.path.join(out, "stamp")
    want = _source_hash()
    lock_path = os.path.join(out, "lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.exists(lib) and os.path.exists(stamp):
                with open(stamp) as f:
                    if f.read().strip() == want:
                        return lib
            nvcc = find_nvcc()
            srcs = sources()
            _say(f"building {LIB_NAME} from {len(srcs)} CUDA files in {out} (first call only)")
            objs = [os.path.join(out, os.path.basename(s)[:-3] + ".o") for s in srcs]
            workers = max(1, min(len(srcs), (os.cpu_count() or 2)))
            with ThreadPoolExecutor(max_workers=workers) as pool:
                list(pool.map(lambda so: _compile_one(nvcc, so[0], so[1]), zip(srcs, objs)))
            tmp = lib + f".{os.getpid()}.tmp"
            r = subprocess.run([nvcc, "-shared", "-o", tmp] + objs + ARCH_FLAGS,
                               stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if r.returncode != 0:
                raise BuildError(f"linking {LIB_NAME} failed:\n{r.stdout}")
            os.replace(tmp, lib)
            with open(stamp, "w") as f:
                f.write(want)
            _say(f"built {lib}")
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def load() -> ctypes.CDLL:
    """The library, built if need be.  Raises if it cannot be built or loaded: there is no fallback."""
    global _lib
    if _lib is None:
        path = build()
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise BuildError(f"could not load {path}: {e}") from e
    return _lib
