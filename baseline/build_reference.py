#!/usr/bin/env python3
"""Builds celsowm/celeg's own shared library (its C API over its CPU and CUDA backends) out of tree
into ``baseline/_ref``, for ``bench.py --impl reference``.

celeg is a CMake project; its configure step needs libcurl (for downloads from the hub) and fetches
server dependencies from the network, neither of which is available offline. What the benchmark
needs is ``libceleg`` alone, so this script compiles the source lists of celeg's own manifests
(cmake/sources/{base_runtime,cpu_backend,cuda_backend,api}.cmake plus the two service files that
CMakeLists.txt links into ``celeg``) with g++ and nvcc directly, unmodified, from the read-only
checkout, and links them with cudart, cuBLAS and cuBLASLt, as CMakeLists.txt does. One file is not
compiled: src/checkpoint/hf_http.cpp (the libcurl transport). Its three functions are replaced by a
stub that throws "no network", written next to the objects; the benchmark loads a local folder and
never reaches them. Nothing of this repository's package is compiled or linked here.

  python baseline/build_reference.py /path/to/celeg [--jobs N] [--arch sm_100]
"""
from __future__ import annotations

import argparse
import concurrent.futures
import hashlib
import os
import re
import shutil
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
MANIFESTS = ("base_runtime", "cpu_backend", "cuda_backend", "api")
EXTRA_SOURCES = ("src/serve/cpu_inference_service.cpp", "src/serve/cuda_inference_service.cpp",
                 "src/serve/generation_dispatcher.cpp")
LEFT_OUT = ("src/checkpoint/hf_http.cpp",)
STUB = """// Stand-in for celeg's src/checkpoint/hf_http.cpp (libcurl transport): there is no network here.
#include "hf_http.hpp"
#include <stdexcept>
namespace celeg::hf_internal {
std::string url_encode(const std::string& value) { return value; }
HttpResponse http_request(const std::string&, const std::string&, bool) {
    throw std::runtime_error("no network: the HuggingFace transport is not built");
}
void http_download_file(const std::string&, const std::filesystem::path&, size_t, bool) {
    throw std::runtime_error("no network: the HuggingFace transport is not built");
}
}
"""


def manifest_sources(root: str) -> list:
    found = []
    for name in MANIFESTS:
        with open(os.path.join(root, "cmake", "sources", f"{name}.cmake"), "r", encoding="utf-8") as handle:
            found += re.findall(r"^\s+(src/\S+\.(?:cpp|cu|c))\s*$", handle.read(), flags=re.M)
    found += list(EXTRA_SOURCES)
    return [s for s in dict.fromkeys(found) if s not in LEFT_OUT]


def compile_one(root: str, source: str, arch: str, objects: str, log) -> str:
    tag = hashlib.sha256(source.encode()).hexdigest()[:10]
    obj = os.path.join(objects, f"{os.path.basename(source)}.{tag}.o")
    if os.path.isfile(obj):
        return obj
    path = source if os.path.isabs(source) else os.path.join(root, source)
    include = ["-I", os.path.join(root, "include"), "-I", os.path.join(root, "src"),
               "-I", os.path.join(root, "src", "backend", "cpu"), "-I", os.path.join(root, "src", "checkpoint")]
    defines = [f'-DCELEG_DESCRIPTOR_DIRECTORY="{os.path.join(root, "descriptors")}"',
               f'-DCELEG_DESCRIPTOR_INSTALL_DIRECTORY="{os.path.join(OUT, "descriptors")}"', "-DCELEG_API_BUILD=1", "-DCELEG_API_WITH_CUDA=1"]
    if source.endswith(".cu"):
        command = ["nvcc", "-std=c++20", "-O3", "-gencode", f"arch=compute_{arch[3:]},code={arch}",
                   "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", *include, *defines, "-c", path, "-o", obj + ".tmp"]
    else:
        command = ["g++", "-std=c++20", "-O2", "-fPIC", "-pthread", "-I", "/usr/local/cuda/include", *include, *defines,
                   "-c", path, "-o", obj + ".tmp"]
    started = time.time()
    result = subprocess.run(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"{source}: compiler exit {result.returncode}\n{result.stdout[-4000:]}")
    os.replace(obj + ".tmp", obj)
    log(f"compiled {source} in {time.time() - started:.0f} s")
    return obj


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("checkout", help="celeg's source tree (read only)")
    parser.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    parser.add_argument("--arch", default="sm_100")
    args = parser.parse_args()
    root = os.path.abspath(args.checkout)
    objects = os.path.join(OUT, "obj")
    os.makedirs(objects, exist_ok=True)
    stub = os.path.join(OUT, "hf_http_stub.cpp")
    with open(stub, "w", encoding="utf-8") as handle:
        handle.write(STUB)
    # celeg looks for architecture descriptors in its checkout, then in its install directory: a copy beside the
    # library serves where the checkout is not mounted
    shutil.copytree(os.path.join(root, "descriptors"), os.path.join(OUT, "descriptors"), dirs_exist_ok=True)
    sources = manifest_sources(root) + [stub]

    def log(message: str) -> None:
        print(f"[reference build] {message}", file=sys.stderr, flush=True)

    log(f"{len(sources)} sources, {args.jobs} jobs, {args.arch}")
    with concurrent.futures.ThreadPoolExecutor(max_workers=args.jobs) as pool:
        futures = [pool.submit(compile_one, root, source, args.arch, objects, log) for source in sources]
        built = [future.result() for future in futures]
    library = os.path.join(OUT, "libceleg.so")
    link = ["g++", "-shared", "-o", library + ".tmp", *built, "-L/usr/local/cuda/lib64", "-Wl,-rpath,/usr/local/cuda/lib64",
            "-lcudart", "-lcublas", "-lcublasLt", "-lpthread", "-ldl"]
    result = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if result.returncode != 0:
        print(result.stdout[-6000:], file=sys.stderr)
        return 1
    os.replace(library + ".tmp", library)
    log(f"linked {library}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
