"""In-tree build of the native extension ``grace_b200/_C*.so``.

Every ``.cu`` under ``csrc/`` is compiled for sm_100a only with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` (nvcc cross-compiles
without a GPU), ``bindings.cpp`` / ``runtime.cpp`` with the host compiler
through nvcc, and everything is linked into one shared object that sits beside
the Python sources.  A content hash of the sources is stored next to the
library; ``ensure_built()`` rebuilds only when it differs.

Run ``python -m grace_b200.ops.build`` to build explicitly.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
CSRC = PKG / "csrc"
BUILD = PKG / "_build"
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
TARGET = PKG / ("_C" + EXT_SUFFIX)
HASH_FILE = BUILD / "sources.sha256"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
              "-diag-suppress", "550"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def _sources():
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp"))


def _headers():
    return sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh"))


def source_hash() -> str:
    h = hashlib.sha256()
    for f in _sources() + _headers():
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    return TARGET.exists() and HASH_FILE.exists() and HASH_FILE.read_text().strip() == source_hash()


def _includes():
    import pybind11

    return ["-I", str(CSRC), "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]


def _compile(src: Path, verbose: bool) -> Path:
    obj = BUILD / (src.name + ".o")
    cmd = [_nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, *_includes(), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src.name, res.stdout, res.stderr))
    if verbose and src.suffix == ".cu":
        sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and is_current():
        return TARGET
    BUILD.mkdir(exist_ok=True)
    srcs = _sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), srcs))
    tmp = BUILD / ("_C.tmp" + EXT_SUFFIX)
    cmd = [_nvcc(), "-shared", "-cudart", "shared", *ARCH_FLAGS, "-o", str(tmp), *map(str, objs)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (res.stdout, res.stderr))
    os.replace(tmp, TARGET)
    HASH_FILE.write_text(source_hash())
    return TARGET


def ensure_built() -> Path:
    """Build if the library is missing or older than its sources.  Several
    ranks may start at once: an exclusive file lock makes one of them build
    while the others wait and then find the library current."""
    if is_current():
        return TARGET
    import fcntl

    BUILD.mkdir(exist_ok=True)
    with open(BUILD / "build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if is_current():
                return TARGET
            return build()
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
