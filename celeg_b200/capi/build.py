"""Builds the C interface library (include/celeg_b200/api.h) with g++ against this interpreter's headers:
``celeg_b200/capi/_build/libceleg_b200_api.so``. ``python -m celeg_b200.capi.build`` prints its path."""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libceleg_b200_api.so"


class ApiBuildError(RuntimeError):
    pass


def ensure_built() -> str:
    out_dir = os.path.join(HERE, "_build")
    os.makedirs(out_dir, exist_ok=True)
    source = os.path.join(HERE, "api.cpp")
    header = os.path.join(HERE, os.pardir, os.pardir, "include", "celeg_b200", "api.h")
    digest = hashlib.sha256()
    for path in (source, header):
        with open(path, "rb") as handle:
            digest.update(handle.read())
    digest.update((sys.version + sys.prefix).encode())
    stamp = os.path.join(out_dir, "api.stamp")
    library = os.path.join(out_dir, LIB_NAME)
    try:
        with open(stamp, "r") as handle:
            if handle.read().strip() == digest.hexdigest() and os.path.isfile(library):
                return library
    except OSError:
        pass
    include = sysconfig.get_config_var("INCLUDEPY")
    libdir = sysconfig.get_config_var("LIBDIR")
    version = sysconfig.get_config_var("LDVERSION")
    if not include or not os.path.isfile(os.path.join(include, "Python.h")):
        raise ApiBuildError(f"Python.h was not found under {include}: the C interface needs the interpreter's headers")
    print("[celeg_b200] compiling the C interface library ...", file=sys.stderr, flush=True)
    import site
    folders = ":".join(dict.fromkeys([*site.getsitepackages(), *(p for p in sys.path if p.endswith("site-packages"))]))
    command = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-I", include,
               f'-DCELEG_B200_SITE_PACKAGES="{folders}"', source,
               "-o", library + f".tmp{os.getpid()}", f"-L{libdir}", f"-Wl,-rpath,{libdir}", f"-lpython{version}",
               "-ldl", "-lpthread"]
    result = subprocess.run(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if result.returncode != 0:
        raise ApiBuildError("building the C interface failed:\n" + result.stdout)
    os.replace(library + f".tmp{os.getpid()}", library)
    with open(stamp, "w") as handle:
        handle.write(digest.hexdigest())
    return library


if __name__ == "__main__":
    print(ensure_built())
