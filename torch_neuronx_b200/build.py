"""In-tree build of ``libb200_sdpa.so`` (sm_100a only) with plain ``nvcc``, and of the C++
operator layer ``libb200_sdpa_ops.so`` (``csrc_ops/aten_ops.cpp``: the dispatcher kernels of the
two ATen ops, linked against the first library and against torch) with ``g++``.

``python -m torch_neuronx_b200.build`` compiles every ``csrc/*.cu`` to an object
file and links them into one shared library next to this file.  Objects are
rebuilt only when their source (or a header) changed; the key is a hash of the
sources, the flags and the nvcc version, which plays the role of the upstream
compile cache (``torch_neuronx/nki_kernel.py:57-115``) for an ahead-of-time
build.  There is no JIT and no fallback: if the library is missing the package
refuses to run.
"""

from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(CSRC, "build")
LIB_PATH = os.path.join(HERE, "libb200_sdpa.so")
OPS_SRC = os.path.join(HERE, "csrc_ops", "aten_ops.cpp")
OPS_LIB_PATH = os.path.join(HERE, "libb200_sdpa_ops.so")
# the checked build: the same sources with -DB200_SDPA_DEBUG (index, scratch-slot and tensor-memory column
# checks that report through the status word; csrc/debug.cuh)
CHECKED_OBJ_DIR = os.path.join(CSRC, "build_checked")
CHECKED_LIB_PATH = os.path.join(HERE, "libb200_sdpa_checked.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put CUDA 12.8+ on PATH")


def _sources():
    cu = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    hdr = sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    hdr_paths = [os.path.join(CSRC, h) for h in hdr] + [os.path.join(HERE, "..", "include", "b200_sdpa.h")]
    return cu, hdr_paths


def _digest(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def build(verbose: bool = False, force: bool = False, checked: bool = False) -> str:
    """Build (if needed) and return the path of the shared library.  ``checked`` builds the bounds-checking
    variant ``libb200_sdpa_checked.so`` instead (same ABI; loaded when ``B200_SDPA_CHECKED=1``)."""
    if checked:
        return _build(verbose, force, CHECKED_OBJ_DIR, CHECKED_LIB_PATH, ["-DB200_SDPA_DEBUG"], with_ops=False)
    return _build(verbose, force, OBJ_DIR, LIB_PATH, [], with_ops=True)


def _build(verbose: bool, force: bool, OBJ_DIR: str, LIB_PATH: str, extra_flags, with_ops: bool) -> str:
    nvcc = find_nvcc()
    version = subprocess.run([nvcc, "--version"], capture_output=True, text=True, check=True).stdout
    cu, hdrs = _sources()
    os.makedirs(OBJ_DIR, exist_ok=True)
    stamp_path = os.path.join(OBJ_DIR, "stamps.json")
    try:
        with open(stamp_path) as f:
            stamps = json.load(f)
    except (OSError, ValueError):
        stamps = {}
    flags = NVCC_FLAGS + list(extra_flags)
    flag_key = " ".join(flags) + version

    def compile_one(name: str):
        src = os.path.join(CSRC, name)
        obj = os.path.join(OBJ_DIR, name[:-3] + ".o")
        key = _digest([src] + hdrs, flag_key)
        if not force and stamps.get(name) == key and os.path.exists(obj):
            return name, key, False, ""
        cmd = [nvcc] + flags + ["-c", src, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {name}:\n{res.stdout}\n{res.stderr}")
        return name, key, True, res.stderr

    rebuilt = False
    with ThreadPoolExecutor(max_workers=min(8, len(cu))) as pool:
        for name, key, did, log in pool.map(compile_one, cu):
            stamps[name] = key
            rebuilt |= did
            if did and verbose:
                sys.stderr.write(f"--- {name}\n{log}\n")
    objs = [os.path.join(OBJ_DIR, n[:-3] + ".o") for n in cu]
    if rebuilt or not os.path.exists(LIB_PATH):
        # -Bsymbolic: the library's own calls (kernel launch stubs included) bind to its own definitions, so a
        # process may hold the normal and the checked build side by side without one interposing on the other
        cmd = [nvcc, "-shared", "-o", LIB_PATH] + objs + ["-cudart", "static", "-Xlinker", "-Bsymbolic",
                                                          "-lpthread", "-ldl", "-lrt"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    if with_ops:
        build_ops(stamps, force=force or rebuilt, verbose=verbose)
    with open(stamp_path, "w") as f:
        json.dump(stamps, f)
    return LIB_PATH


def build_ops(stamps: dict, force: bool = False, verbose: bool = False) -> str:
    """Build (if needed) the C++ operator layer against the installed torch; returns its path."""
    import torch
    from torch.utils import cpp_extension

    gxx = os.environ.get("CXX") or shutil.which("g++")
    if gxx is None:
        raise RuntimeError("g++ not found; set CXX")
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    flags = ["-O2", "-std=c++17", "-fPIC", "-shared", "-Wno-deprecated-declarations",
             f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for inc in cpp_extension.include_paths() + [os.path.join(cuda_home, "include")]:
        flags += ["-isystem", inc]
    key = _digest([OPS_SRC, os.path.join(HERE, "..", "include", "b200_sdpa.h")], " ".join(flags) + torch.__version__)
    if not force and stamps.get("aten_ops.cpp") == key and os.path.exists(OPS_LIB_PATH):
        return OPS_LIB_PATH
    cmd = [gxx] + flags + [OPS_SRC, "-o", OPS_LIB_PATH, f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10", "-lc10_cuda",
                           f"-L{HERE}", "-lb200_sdpa", "-Wl,-rpath,$ORIGIN"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"g++ failed for aten_ops.cpp:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(f"--- aten_ops.cpp\n{res.stderr}\n")
    stamps["aten_ops.cpp"] = key
    return OPS_LIB_PATH


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv, checked="--checked" in sys.argv)
    print(path)
