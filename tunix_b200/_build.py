"""In-tree native build: nvcc (sm_100a) for the CUDA library, g++ for the host extensions.

The shared objects are written next to this file so they travel with a snapshot of
the source tree and are found by `ctypes` without an install step.

  libtunix_b200_cuda.so   every .cu under csrc/ (extern "C" entry points, loaded by `_lib.py`)
  libtunix_b200_host.so   csrc/host/*.cc (sequence packing, trajectory JSON; C ABI)
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR / "csrc" / "build"
CUDA_LIB = PKG_DIR / "libtunix_b200_cuda.so"
HOST_LIB = PKG_DIR / "libtunix_b200_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _digest(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(str(p.name).encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("build failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), res.stdout, res.stderr))
    return res.stdout + res.stderr


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    """Compile every csrc/*.cu for sm_100a and link one shared library."""
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh"))
    stamp = BUILD_DIR / "cuda.stamp"
    digest = _digest(sources + headers, " ".join(NVCC_FLAGS))
    if not force and CUDA_LIB.exists() and stamp.exists() and stamp.read_text() == digest:
        return CUDA_LIB
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    hdr_digest = _digest(headers, " ".join(NVCC_FLAGS))

    def compile_one(src: Path) -> Path:
        obj = BUILD_DIR / (src.stem + ".o")
        ostamp = BUILD_DIR / (src.stem + ".stamp")
        d = _digest([src], hdr_digest)
        if not force and obj.exists() and ostamp.exists() and ostamp.read_text() == d:
            return obj
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        out = _run(cmd)
        if verbose:
            print(out, file=sys.stderr)
        ostamp.write_text(d)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources) or 1)) as ex:
        objs = list(ex.map(compile_one, sources))
    _run([nvcc, "-shared", "-o", str(CUDA_LIB), *map(str, objs), "-lcudart", "-Xcompiler", "-fPIC"])
    stamp.write_text(digest)
    return CUDA_LIB


def build_host(force: bool = False) -> Path:
    """Compile the C++ host extensions (no CUDA, no Python headers: plain C ABI)."""
    sources = sorted((CSRC / "host").glob("*.cc"))
    headers = sorted((CSRC / "host").glob("*.h"))
    stamp = BUILD_DIR / "host.stamp"
    digest = _digest(sources + headers, " ".join(CXX_FLAGS))
    if not force and HOST_LIB.exists() and stamp.exists() and stamp.read_text() == digest:
        return HOST_LIB
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    _run([cxx, *CXX_FLAGS, "-shared", "-o", str(HOST_LIB), *map(str, sources)])
    stamp.write_text(digest)
    return HOST_LIB


def build_host_sanitized(force: bool = False) -> Path:
    """The host extensions once more with AddressSanitizer and UndefinedBehaviorSanitizer, for the test that runs the
    packing suite against them (the process that loads this library must have libasan preloaded)."""
    sources = sorted((CSRC / "host").glob("*.cc"))
    out = BUILD_DIR / "libtunix_b200_host_asan.so"
    stamp = BUILD_DIR / "host_asan.stamp"
    flags = ["-O1", "-g", "-std=c++17", "-fPIC", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
             "-fno-sanitize-recover=all"]
    digest = _digest(sources, " ".join(flags))
    if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
        return out
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    cxx, _ = sanitizer_toolchain()
    _run([cxx, *flags, "-shared", "-o", str(out), *map(str, sources)])
    stamp.write_text(digest)
    return out


def sanitizer_toolchain():
    """(compiler, path of its libasan.so): the first g++ that ships the sanitizer run-time."""
    seen = []
    for cxx in (os.environ.get("CXX"), "/usr/bin/g++", shutil.which("g++")):
        if not cxx or cxx in seen or not os.path.exists(cxx):
            continue
        seen.append(cxx)
        res = subprocess.run([cxx, "-print-file-name=libasan.so"], capture_output=True, text=True)
        path = res.stdout.strip()
        if res.returncode == 0 and os.path.isabs(path) and os.path.exists(path):
            return cxx, path
    raise RuntimeError("no g++ with libasan on this machine")


TRAJJSON_LIB = PKG_DIR / "utils" / "_trajjson.so"


def build_pyext(force: bool = False) -> Path:
    """Compile the CPython extension modules under csrc/pyext (need Python.h)."""
    import sysconfig
    src = CSRC / "pyext" / "trajjson.cc"
    stamp = BUILD_DIR / "pyext.stamp"
    digest = _digest([src], " ".join(CXX_FLAGS) + sys.version)
    if not force and TRAJJSON_LIB.exists() and stamp.exists() and stamp.read_text() == digest:
        return TRAJJSON_LIB
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    inc = sysconfig.get_paths()["include"]
    if not os.path.exists(os.path.join(inc, "Python.h")):
        raise RuntimeError("Python.h not found; the pure-Python serializer will be used")
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    _run([cxx, *CXX_FLAGS, "-fvisibility=default", "-shared", "-I", inc, "-o", str(TRAJJSON_LIB), str(src)])
    stamp.write_text(digest)
    return TRAJJSON_LIB


def build_pyext_sanitized(force: bool = False) -> Path:
    """`_trajjson` with AddressSanitizer and UndefinedBehaviorSanitizer, beside the build products (not in the
    package); `TUNIX_B200_TRAJJSON_LIB` makes `utils.trajectory_logger` load it."""
    import sysconfig
    src = CSRC / "pyext" / "trajjson.cc"
    out = BUILD_DIR / "asan" / "_trajjson.so"
    stamp = BUILD_DIR / "pyext_asan.stamp"
    flags = ["-O1", "-g", "-std=c++17", "-fPIC", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
             "-fno-sanitize-recover=all", "-fvisibility=default"]
    digest = _digest([src], " ".join(flags) + sys.version)
    if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
        return out
    out.parent.mkdir(parents=True, exist_ok=True)
    inc = sysconfig.get_paths()["include"]
    if not os.path.exists(os.path.join(inc, "Python.h")):
        raise RuntimeError("Python.h not found")
    cxx, _ = sanitizer_toolchain()
    _run([cxx, *flags, "-shared", "-I", inc, "-o", str(out), str(src)])
    stamp.write_text(digest)
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_host(force)
    try:
        build_pyext(force)
    except RuntimeError as e:  # optional: a Python fallback exists
        print(f"[tunix_b200 build] pyext skipped: {e}", file=sys.stderr)
    build_cuda(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", CUDA_LIB, HOST_LIB)
