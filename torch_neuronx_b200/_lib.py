"""ctypes binding of ``libb200_sdpa.so`` (the C ABI in ``include/b200_sdpa.h``).

This replaces the upstream kernel-registration layer
(``torch_neuronx/nki_hop.py:880-1039`` ``NKIHOPCaller`` ->
``_C._nki_dispatch_eager``, ``torch_neuronx/csrc/core/NeuronBindings.cpp:900``)
with a direct launch: no lowering cache, no IR, one foreign call per op.

There is no fallback of any kind.  If the shared library has not been built the
import of the compute entry points raises, and every compute call requires a
CUDA device.
"""

from __future__ import annotations

import ctypes as C
import os
import threading

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200_sdpa.so")
OPS_LIB_PATH = os.path.join(HERE, "libb200_sdpa_ops.so")   # C++ operator layer (dispatcher kernels of the ATen ops)
# B200_SDPA_CHECKED=1 runs everything on the bounds-checking build of the library (csrc/debug.cuh;
# `python -m torch_neuronx_b200.build --checked`); the C++ operator layer is linked against the normal library, so
# the ATen ops then go through the Python implementations and the same checked kernels.
CHECKED = os.environ.get("B200_SDPA_CHECKED", "0") not in ("", "0")
if CHECKED:
    LIB_PATH = os.path.join(HERE, "libb200_sdpa_checked.so")

ABI_VERSION = 6
STATIC_SCRATCH_BYTES = 16 << 20  # B200_SDPA_STATIC_SCRATCH_BYTES

# b200_sdpa_status
OK = 0
ERR_NULL, ERR_STRUCT, ERR_DTYPE, ERR_SHAPE, ERR_UNSUPPORTED = 1, 2, 3, 4, 5
ERR_WORKSPACE, ERR_ALIGNMENT, ERR_CUDA, ERR_DEVICE, ERR_TIMEOUT, ERR_TOO_LARGE, ERR_CACHE_FULL, ERR_BOUNDS = 6, 7, 8, 9, 10, 11, 12, 13

# b200_sdpa_dtype
F32, F16, BF16 = 0, 1, 2

# b200_sdpa_path
PATH_AUTO, PATH_GENERIC, PATH_PREFILL, PATH_DECODE = 0, 1, 2, 3
PATH_NAMES = {PATH_AUTO: "auto", PATH_GENERIC: "generic", PATH_PREFILL: "prefill", PATH_DECODE: "decode"}

# launch-counter ids
KID_GENERIC, KID_PREFILL, KID_DECODE, KID_COMBINE, KID_MERGE, KID_BWD_DQ, KID_BWD_DKV, KID_BWD_PREP = range(8)
KERNEL_NAMES = ("generic", "prefill", "decode_partial", "decode_combine", "merge", "bwd_dq", "bwd_dkv", "bwd_prep")


class Params(C.Structure):
    """Mirror of ``B200SdpaParams``."""

    _fields_ = [
        ("struct_size", C.c_uint32),
        ("dtype", C.c_int32),
        ("device", C.c_int32),
        ("force_path", C.c_int32),
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("out", C.c_void_p),
        ("lse", C.c_void_p),
        ("q_stride", C.c_int64 * 4),
        ("k_stride", C.c_int64 * 4),
        ("v_stride", C.c_int64 * 4),
        ("out_stride", C.c_int64 * 4),
        ("lse_stride", C.c_int64 * 3),
        ("B", C.c_int32),
        ("Hq", C.c_int32),
        ("Hkv", C.c_int32),
        ("L", C.c_int32),
        ("S", C.c_int32),
        ("E", C.c_int32),
        ("Dv", C.c_int32),
        ("scale", C.c_float),
        ("is_causal", C.c_int32),
        ("q_offset", C.c_int64),
        ("k_offset", C.c_int64),
        ("kv_lens", C.c_void_p),
        ("bias", C.c_void_p),
        ("bias_dtype", C.c_int32),
        ("kv_chunk", C.c_int32),
        ("bias_stride", C.c_int64 * 4),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_uint64),
        ("status", C.c_void_p),
        ("block_table", C.c_void_p),
        ("block_table_stride", C.c_int32),
        ("page_size", C.c_int32),
        ("k_new", C.c_void_p),
        ("v_new", C.c_void_p),
        ("k_new_stride", C.c_int64 * 2),
        ("v_new_stride", C.c_int64 * 2),
        ("kv_lens_out", C.c_void_p),
        ("rope_cos", C.c_void_p),
        ("rope_sin", C.c_void_p),
        ("rope_stride", C.c_int32),
        ("rope_interleaved", C.c_int32),
        ("rope_positions", C.c_int32),
        ("acc_mode", C.c_int32),
        ("acc", C.c_void_p),
        ("acc_lse", C.c_void_p),
        ("acc_stride", C.c_int64 * 3),
        ("acc_lse_stride", C.c_int64 * 3),
    ]


class Plan(C.Structure):
    """Mirror of ``B200SdpaPlan``."""

    _fields_ = [
        ("struct_size", C.c_uint32),
        ("path", C.c_int32),
        ("block_m", C.c_int32),
        ("block_n", C.c_int32),
        ("grid_x", C.c_int32),
        ("grid_y", C.c_int32),
        ("grid_z", C.c_int32),
        ("threads", C.c_int32),
        ("smem_bytes", C.c_int32),
        ("kv_splits", C.c_int32),
        ("launches", C.c_int32),
        ("workspace_bytes", C.c_uint64),
    ]


class MergeParams(C.Structure):
    """Mirror of ``B200SdpaMergeParams``."""

    _fields_ = [
        ("struct_size", C.c_uint32),
        ("dtype", C.c_int32),
        ("device", C.c_int32),
        ("first", C.c_int32),
        ("acc", C.c_void_p),
        ("acc_lse", C.c_void_p),
        ("part", C.c_void_p),
        ("part_lse", C.c_void_p),
        ("final_out", C.c_void_p),
        ("part_stride", C.c_int64 * 4),
        ("part_lse_stride", C.c_int64 * 3),
        ("final_stride", C.c_int64 * 4),
        ("B", C.c_int32),
        ("Hq", C.c_int32),
        ("L", C.c_int32),
        ("Dv", C.c_int32),
        ("acc_stride", C.c_int64 * 3),
        ("acc_lse_stride", C.c_int64 * 3),
    ]


class BwdParams(C.Structure):
    """Mirror of ``B200SdpaBwdParams``."""

    _fields_ = [
        ("struct_size", C.c_uint32),
        ("dtype", C.c_int32),
        ("device", C.c_int32),
        ("force_path", C.c_int32),
        ("grad_out", C.c_void_p),
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("out", C.c_void_p),
        ("lse", C.c_void_p),
        ("grad_q", C.c_void_p),
        ("grad_k", C.c_void_p),
        ("grad_v", C.c_void_p),
        ("grad_bias", C.c_void_p),
        ("grad_out_stride", C.c_int64 * 4),
        ("q_stride", C.c_int64 * 4),
        ("k_stride", C.c_int64 * 4),
        ("v_stride", C.c_int64 * 4),
        ("out_stride", C.c_int64 * 4),
        ("lse_stride", C.c_int64 * 3),
        ("grad_q_stride", C.c_int64 * 4),
        ("grad_k_stride", C.c_int64 * 4),
        ("grad_v_stride", C.c_int64 * 4),
        ("grad_bias_stride", C.c_int64 * 4),
        ("B", C.c_int32),
        ("Hq", C.c_int32),
        ("Hkv", C.c_int32),
        ("L", C.c_int32),
        ("S", C.c_int32),
        ("E", C.c_int32),
        ("Dv", C.c_int32),
        ("scale", C.c_float),
        ("is_causal", C.c_int32),
        ("bias_dtype", C.c_int32),
        ("q_offset", C.c_int64),
        ("k_offset", C.c_int64),
        ("kv_lens", C.c_void_p),
        ("bias", C.c_void_p),
        ("bias_stride", C.c_int64 * 4),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_uint64),
        ("status", C.c_void_p),
    ]


# Every symbol include/b200_sdpa.h declares: name -> (restype, argtypes)
EXPORTS = {
    "b200_sdpa_abi_version": (C.c_int, []),
    "b200_sdpa_strerror": (C.c_char_p, [C.c_int]),
    "b200_sdpa_query_plan": (C.c_int, [C.POINTER(Params), C.POINTER(Plan)]),
    "b200_sdpa_fwd": (C.c_int, [C.POINTER(Params), C.c_void_p]),
    "b200_sdpa_decode": (C.c_int, [C.POINTER(Params), C.c_void_p]),
    "b200_sdpa_decode_static": (C.c_int, [C.POINTER(Params), C.c_void_p]),
    "b200_sdpa_bwd_query_plan": (C.c_int, [C.POINTER(BwdParams), C.POINTER(Plan)]),
    "b200_sdpa_bwd": (C.c_int, [C.POINTER(BwdParams), C.c_void_p]),
    "b200_sdpa_merge": (C.c_int, [C.POINTER(MergeParams), C.c_void_p]),
    "b200_sdpa_launch_count": (C.c_uint64, [C.c_int]),
    "b200_sdpa_reset_launch_counts": (None, []),
    "b200_sdpa_checked_build": (C.c_int, []),
    "b200_sdpa_debug_selftest": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p]),
}

_lib = None
_lock = threading.Lock()


class LibraryMissing(RuntimeError):
    pass


def load():
    """Load the shared library once; raise loudly if it is not there."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise LibraryMissing(
                f"{LIB_PATH} not found: build it with `python -m torch_neuronx_b200.build` "
                "(there is no CPU or PyTorch fallback for this path)"
            )
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in EXPORTS.items():
            fn = getattr(lib, name)  # AttributeError names the missing symbol
            fn.restype = res
            fn.argtypes = args
        got = lib.b200_sdpa_abi_version()
        if got != ABI_VERSION:
            raise RuntimeError(f"libb200_sdpa.so has ABI version {got}, this package expects {ABI_VERSION}")
        _lib = lib
    return _lib


_ops_loaded = None


def load_ops() -> bool:
    """Load the C++ operator layer (``csrc_ops/aten_ops.cpp``): it registers the CUDA kernels of the two
    ATen ops with the dispatcher, as upstream's native dispatcher does
    (``torch_neuronx/csrc/core/dispatch/NeuronDispatcher.cpp:2370-2582``).  Returns False when the
    library has not been built; the same kernels are then reached through the ctypes binding."""
    global _ops_loaded
    if _ops_loaded is not None:
        return _ops_loaded
    with _lock:
        if _ops_loaded is None:
            _ops_loaded = False
            if not CHECKED and os.path.exists(OPS_LIB_PATH) and os.path.exists(LIB_PATH):
                import torch

                try:
                    C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)   # the layer links against it by name
                    torch.ops.load_library(OPS_LIB_PATH)
                    _ops_loaded = True
                except OSError as exc:
                    # a library from an interrupted or outdated build: importing the package must still work
                    # (the build itself runs as a module of it); any compute call will report the real problem
                    import warnings

                    warnings.warn(f"libb200_sdpa_ops.so could not be loaded ({exc}); rebuild with "
                                  "`python -m torch_neuronx_b200.build`")
    return _ops_loaded


def strerror(code: int) -> str:
    return load().b200_sdpa_strerror(int(code)).decode()


def launch_counts() -> dict:
    lib = load()
    return {name: int(lib.b200_sdpa_launch_count(i)) for i, name in enumerate(KERNEL_NAMES)}


def reset_launch_counts() -> None:
    load().b200_sdpa_reset_launch_counts()
