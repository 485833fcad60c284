"""Builds the CUDA kernel library for sm_100a with nvcc and returns its path.

The library is built in-tree (``celeg_b200/csrc/_build/libceleg_b200.so``) the first time it is
needed and again whenever a source changes; objects are cached per source file. If the package
folder cannot be written, a per-user folder under the system's temporary directory is used.
``CELEG_B200_BUILD_DIR`` overrides the place. Progress lines go to stderr so a first call that
compiles for a minute does not look hung.
"""
from __future__ import annotations

import concurrent.futures
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import List, Optional

SOURCE_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libceleg_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


class BuildError(RuntimeError):
    pass


def _log(message: str) -> None:
    print(f"[celeg_b200] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for candidate in (os.environ.get("CELEG_B200_NVCC"),
                      os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                      shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise BuildError("nvcc was not found (looked at CELEG_B200_NVCC, CUDA_HOME, PATH, /usr/local/cuda/bin); "
                     "the CUDA kernels of celeg_b200 cannot be built")


def sources() -> List[str]:
    return sorted(name for name in os.listdir(SOURCE_DIR) if name.endswith(".cu"))


def _headers_digest() -> bytes:
    digest = hashlib.sha256()
    for name in sorted(os.listdir(SOURCE_DIR)):
        if name.endswith((".cuh", ".h")):
            with open(os.path.join(SOURCE_DIR, name), "rb") as handle:
                digest.update(name.encode() + b"\0" + handle.read())
    digest.update(" ".join(NVCC_FLAGS).encode())
    return digest.digest()


def _source_digest(name: str, headers: bytes) -> str:
    digest = hashlib.sha256(headers)
    with open(os.path.join(SOURCE_DIR, name), "rb") as handle:
        digest.update(handle.read())
    return digest.hexdigest()[:24]


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
    override = os.environ.get("CELEG_B200_BUILD_DIR")
    if override:
        if not _writable_dir(override):
            raise BuildError(f"CELEG_B200_BUILD_DIR={override} cannot be written")
        return override
    in_tree = os.path.join(SOURCE_DIR, "_build")
    if _writable_dir(in_tree):
        return in_tree
    fallback = os.path.join(tempfile.gettempdir(), f"celeg_b200_build_{os.getuid()}")
    if _writable_dir(fallback):
        return fallback
    raise BuildError(f"neither {in_tree} nor {fallback} can be written; set CELEG_B200_BUILD_DIR")


def _compile_one(nvcc: str, name: str, obj: str) -> None:
    started = time.time()
    _log(f"compiling {name} for sm_100a ...")
    tmp = obj + f".tmp{os.getpid()}"
    result = subprocess.run([nvcc, *NVCC_FLAGS, "-I", SOURCE_DIR, "-c", os.path.join(SOURCE_DIR, name), "-o", tmp],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if result.returncode != 0:
        raise BuildError(f"nvcc failed on {name}:\n{result.stdout}")
    os.replace(tmp, obj)
    _log(f"compiled {name} in {time.time() - started:.0f} s")


def ensure_built(verbose: bool = True) -> str:
    """Path of an up-to-date library; compiles what is missing."""
    out_dir = build_dir()
    headers = _headers_digest()
    names = sources()
    objects = {name: os.path.join(out_dir, f"{os.path.splitext(name)[0]}.{_source_digest(name, headers)}.o")
               for name in names}
    link_digest = hashlib.sha256("\n".join(sorted(os.path.basename(o) for o in objects.values())).encode()).hexdigest()[:24]
    library = os.path.join(out_dir, LIB_NAME)
    stamp = os.path.join(out_dir, "link.stamp")

    def current() -> bool:
        try:
            with open(stamp, "r") as handle:
                return handle.read().strip() == link_digest and os.path.isfile(library)
        except OSError:
            return False

    if current():
        return library
    with open(os.path.join(out_dir, "build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if current():
                return library
            nvcc = find_nvcc()
            todo = [name for name in names if not os.path.isfile(objects[name])]
            if todo:
                _log(f"building the kernel library in {out_dir}: {len(todo)} file(s) to compile")
                workers = max(1, min(len(todo), os.cpu_count() or 1, 8))
                with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
                    for future in [pool.submit(_compile_one, nvcc, name, objects[name]) for name in todo]:
                        future.result()
            _log("linking " + LIB_NAME)
            tmp = library + f".tmp{os.getpid()}"
            result = subprocess.run([nvcc, "-shared", "-o", tmp, *objects.values(), "-lcudart"],
                                    stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if result.returncode != 0:
                raise BuildError(f"linking {LIB_NAME} failed:\n{result.stdout}")
            os.replace(tmp, library)
            with open(stamp, "w") as handle:
                handle.write(link_digest)
            keep = set(objects.values())
            for name in os.listdir(out_dir):          # objects of older source versions
                path = os.path.join(out_dir, name)
                if name.endswith(".o") and path not in keep:
                    try:
                        os.remove(path)
                    except OSError:
                        pass
            _log("kernel library is ready")
            return library
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


if __name__ == "__main__":
    print(ensure_built())
