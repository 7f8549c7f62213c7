"""In-tree build of the native extension ``grace_b200/_C*.so``.

Every ``.cu`` under ``csrc/`` is compiled for sm_100a only with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` (nvcc cross-compiles
without a GPU), ``bindings.cpp`` / ``runtime.cpp`` with the host compiler
through nvcc, and everything is linked into one shared object that sits beside
the Python sources.  A content hash of the sources is stored next to the
library; ``ensure_built()`` rebuilds only when it differs.

A second, *checked* variant (``_C_checked``) is the same sources compiled with
``-DGRACE_CHECKED``: index and offset checks in the kernels that record
``(kernel, source line, index)`` in the status block and skip the access instead
of faulting.  ``GRACE_CHECKED=1`` in the environment makes ``native()`` load it.

Run ``python -m grace_b200.ops.build`` to build explicitly (``--checked`` for
the checked variant, ``--all`` for both).
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
TARGET_CHECKED = PKG / ("_C_checked" + EXT_SUFFIX)
BUILD_CHECKED = PKG / "_build_checked"
HASH_FILE_CHECKED = BUILD_CHECKED / "sources.sha256"

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


def is_current(checked: bool = False) -> bool:
    target, hash_file = (TARGET_CHECKED, HASH_FILE_CHECKED) if checked else (TARGET, HASH_FILE)
    return target.exists() and hash_file.exists() and hash_file.read_text().strip() == source_hash()


def _includes():
    import pybind11

    return ["-I", str(CSRC), "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]


def _compile(src: Path, verbose: bool, checked: bool = False) -> Path:
    obj = (BUILD_CHECKED if checked else BUILD) / (src.name + ".o")
    extra = ["-DGRACE_CHECKED", "-DGRACE_MODULE_NAME=_C_checked"] if checked else []
    cmd = [_nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, *extra, *_includes(), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src.name, res.stdout, res.stderr))
    if verbose and src.suffix == ".cu":
        sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False, checked: bool = False) -> Path:
    target, build_dir, hash_file = (TARGET_CHECKED, BUILD_CHECKED, HASH_FILE_CHECKED) if checked else (TARGET, BUILD, HASH_FILE)
    if not force and is_current(checked):
        return target
    build_dir.mkdir(exist_ok=True)
    srcs = _sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose, checked), srcs))
    tmp = build_dir / ("_C.tmp" + EXT_SUFFIX)
    cmd = [_nvcc(), "-shared", "-cudart", "shared", *ARCH_FLAGS, "-o", str(tmp), *map(str, objs)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (res.stdout, res.stderr))
    os.replace(tmp, target)
    hash_file.write_text(source_hash())
    return target


def ensure_built(checked: bool = False) -> Path:
    """Build if the library is missing or older than its sources.  Several
    ranks may start at once: an exclusive file lock makes one of them build
    while the others wait and then find the library current."""
    if is_current(checked):
        return TARGET_CHECKED if checked else TARGET
    import fcntl

    build_dir = BUILD_CHECKED if checked else BUILD
    build_dir.mkdir(exist_ok=True)
    with open(build_dir / "build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if is_current(checked):
                return TARGET_CHECKED if checked else TARGET
            return build(checked=checked)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


if __name__ == "__main__":
    variants = [False, True] if "--all" in sys.argv else ["--checked" in sys.argv]
    for variant in variants:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, checked=variant))
