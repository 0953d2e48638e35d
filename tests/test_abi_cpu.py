"""CPU-side checks of the C ABI: the library loads, exports every symbol the header
declares, rejects malformed parameter blocks, and plans kernels -- no GPU needed
(``b200_sdpa_query_plan`` is host-only)."""

import ctypes as C
import os
import re

import pytest

from torch_neuronx_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200_sdpa.h")


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_sdpa_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = C.CDLL(_lib.LIB_PATH)
    names = _declared_symbols()
    assert "b200_sdpa_fwd" in names and "b200_sdpa_decode" in names and "b200_sdpa_merge" in names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/b200_sdpa.h but not exported"
    assert set(names) == set(_lib.EXPORTS), "python binding table and header disagree"


def test_checked_build_exports_the_same_abi():
    """The bounds-checking variant of the library is the same ABI with the checks compiled in."""
    import os

    checked = os.path.join(os.path.dirname(_lib.LIB_PATH), "libb200_sdpa_checked.so")
    normal = C.CDLL(_lib.LIB_PATH)
    normal.b200_sdpa_checked_build.restype = C.c_int
    assert normal.b200_sdpa_checked_build() == 0
    # without the checks the self-test entry point declines before touching any device
    normal.b200_sdpa_debug_selftest.restype = C.c_int
    normal.b200_sdpa_debug_selftest.argtypes = [C.c_int, C.c_void_p, C.c_void_p]
    assert normal.b200_sdpa_debug_selftest(0, None, None) == _lib.ERR_UNSUPPORTED
    if not os.path.exists(checked):
        import pytest

        pytest.skip("checked library not built (python -m torch_neuronx_b200.build --checked)")
    lib = C.CDLL(checked)
    for n in _declared_symbols():
        assert hasattr(lib, n), f"{n} missing from the checked build"
    lib.b200_sdpa_checked_build.restype = C.c_int
    lib.b200_sdpa_abi_version.restype = C.c_int
    assert lib.b200_sdpa_checked_build() == 1
    assert lib.b200_sdpa_abi_version() == _lib.ABI_VERSION


def test_abi_version_and_strerror():
    lib = _lib.load()
    assert lib.b200_sdpa_abi_version() == _lib.ABI_VERSION
    assert _lib.strerror(0) == "ok"
    for code in range(1, 14):
        assert _lib.strerror(code) not in ("ok", "unknown status")
    assert _lib.strerror(999) == "unknown status"


def _params(B=1, Hq=8, Hkv=2, L=256, S=256, E=128, Dv=128, dtype=_lib.BF16, contiguous=True, **kw):
    p = _lib.Params()
    p.struct_size = C.sizeof(_lib.Params)
    p.dtype, p.device = dtype, -1
    fake = 0x7F0000000000  # never dereferenced by the planner
    p.q, p.k, p.v, p.out = fake, fake + (1 << 30), fake + (2 << 30), fake + (3 << 30)
    p.B, p.Hq, p.Hkv, p.L, p.S, p.E, p.Dv = B, Hq, Hkv, L, S, E, Dv
    p.q_stride[:] = [Hq * L * E, L * E, E, 1]
    p.k_stride[:] = [Hkv * S * E, S * E, E, 1]
    p.v_stride[:] = [Hkv * S * Dv, S * Dv, Dv, 1]
    p.out_stride[:] = [Hq * L * Dv, L * Dv, Dv, 1]
    p.lse_stride[:] = [Hq * L, L, 1]
    p.scale = 0.1
    for k_, v_ in kw.items():
        setattr(p, k_, v_)
    return p


def _plan(p):
    plan = _lib.Plan()
    plan.struct_size = C.sizeof(_lib.Plan)
    rc = _lib.load().b200_sdpa_query_plan(C.byref(p), C.byref(plan))
    return rc, plan


def test_planner_picks_the_expected_kernel():
    rc, plan = _plan(_params(B=4, Hq=32, Hkv=8, L=4096, S=4096))
    assert rc == 0 and plan.path == _lib.PATH_PREFILL
    # 16 * 32 * 4 = 2048 items of two 128-row tiles at head dim 128: the persistent form, one CTA per SM; 16 bytes
    # of (optional) scratch hold the counter the items are drawn from
    assert plan.block_m == 256 and plan.block_n == 128 and plan.threads == 512
    assert plan.grid_x == 148 and 190 * 1024 < plan.smem_bytes <= 195 * 1024 and plan.workspace_bytes == 16
    # fewer than three items per SM, or head dim 64: one item per CTA, no scratch
    rc, small = _plan(_params(B=1, Hq=32, Hkv=8, L=2048, S=2048))
    assert rc == 0 and small.path == _lib.PATH_PREFILL and small.threads == 320
    assert small.grid_x == 8 * 32 and small.workspace_bytes == 0
    rc, d64 = _plan(_params(B=4, Hq=32, Hkv=8, L=4096, S=4096, E=64, Dv=64))
    assert rc == 0 and d64.path == _lib.PATH_PREFILL and d64.threads == 320 and d64.grid_x == 16 * 32 * 4
    rc, plan = _plan(_params(B=64, Hq=32, Hkv=8, L=1, S=8192))
    assert rc == 0 and plan.path == _lib.PATH_DECODE and plan.launches == 2
    assert plan.workspace_bytes == 64 * 32 * plan.kv_splits * (128 + 2) * 4
    rc, plan = _plan(_params(dtype=_lib.F32, E=64, Dv=64))
    assert rc == 0 and plan.path == _lib.PATH_GENERIC
    rc, plan = _plan(_params(E=96, Dv=96))  # head dim the tensor-core kernel is not built for
    assert rc == 0 and plan.path == _lib.PATH_GENERIC
    rc, plan = _plan(_params(scale=-1.0))
    assert rc == 0 and plan.path == _lib.PATH_GENERIC
    # head dims beyond 128: the one-tile-per-CTA tensor-core kernel
    p = _params(E=192, Dv=128)
    p.q_stride[:] = [8 * 256 * 192, 256 * 192, 192, 1]
    p.k_stride[:] = [2 * 256 * 192, 256 * 192, 192, 1]
    rc, plan = _plan(p)
    assert rc == 0 and plan.path == _lib.PATH_PREFILL and plan.block_m == 128 and plan.threads == 192
    assert plan.grid_x == 2 * 8 * 1 and plan.smem_bytes > 200 * 1024
    p = _params(E=256, Dv=256)
    for st, h in ((p.q_stride, 8), (p.k_stride, 2), (p.v_stride, 2), (p.out_stride, 8)):
        st[:] = [h * 256 * 256, 256 * 256, 256, 1]
    rc, plan = _plan(p)
    assert rc == 0 and plan.path == _lib.PATH_PREFILL and plan.threads == 192
    rc, plan = _plan(_params(E=192, Dv=192))   # not a shape the wide kernel is built for
    assert rc == 0 and plan.path == _lib.PATH_GENERIC


def test_planner_rejects_bad_blocks():
    lib = _lib.load()
    p = _params()
    p.struct_size = 12
    assert _plan(p)[0] == _lib.ERR_STRUCT
    assert _plan(_params(dtype=7))[0] == _lib.ERR_DTYPE
    assert _plan(_params(Hq=6, Hkv=4))[0] == _lib.ERR_SHAPE
    assert _plan(_params(L=0))[0] == _lib.ERR_SHAPE
    p = _params()
    p.q = None
    assert _plan(p)[0] == _lib.ERR_NULL
    # forcing the tensor-core path on a misaligned base is an alignment error, not a crash
    p = _params(force_path=_lib.PATH_PREFILL)
    p.q = 0x7F0000000002
    assert _plan(p)[0] == _lib.ERR_ALIGNMENT
    assert _plan(_params(force_path=_lib.PATH_DECODE))[0] == _lib.ERR_UNSUPPORTED  # L != 1
    assert lib.b200_sdpa_query_plan(None, None) == _lib.ERR_NULL
    assert lib.b200_sdpa_fwd(None, None) == _lib.ERR_NULL
    assert lib.b200_sdpa_merge(None, None) == _lib.ERR_NULL


def test_struct_layout_matches_the_header():
    """Offsets computed by the C compiler for the header must equal ctypes' (guards the
    binding against silent drift)."""
    import shutil
    import subprocess
    import tempfile

    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    src = r"""
#include <stdio.h>
#include <stddef.h>
#include "b200_sdpa.h"
int main(void) {
  printf("%zu %zu %zu %zu %zu %zu %zu\n", sizeof(B200SdpaParams), offsetof(B200SdpaParams, q_offset),
         offsetof(B200SdpaParams, kv_lens), offsetof(B200SdpaParams, bias_stride), offsetof(B200SdpaParams, status),
         sizeof(B200SdpaPlan), sizeof(B200SdpaMergeParams));
  printf("%zu %zu %zu %zu %zu %zu\n", sizeof(B200SdpaBwdParams), offsetof(B200SdpaBwdParams, grad_bias),
         offsetof(B200SdpaBwdParams, lse_stride), offsetof(B200SdpaBwdParams, scale),
         offsetof(B200SdpaBwdParams, q_offset), offsetof(B200SdpaBwdParams, status));
  return 0;
}
"""
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "t.c"), "w").write(src)
        subprocess.run([cc, "-I", os.path.join(ROOT, "include"), os.path.join(d, "t.c"), "-o", os.path.join(d, "t")],
                       check=True)
        got = [int(x) for x in subprocess.run([os.path.join(d, "t")], capture_output=True, text=True,
                                              check=True).stdout.split()]
    P = _lib.Params
    want = [C.sizeof(P), P.q_offset.offset, P.kv_lens.offset, P.bias_stride.offset, P.status.offset,
            C.sizeof(_lib.Plan), C.sizeof(_lib.MergeParams)]
    W = _lib.BwdParams
    want += [C.sizeof(W), W.grad_bias.offset, W.lse_stride.offset, W.scale.offset, W.q_offset.offset,
             W.status.offset]
    assert got == want


def test_backward_entry_rejects_bad_blocks():
    lib = _lib.load()
    assert lib.b200_sdpa_bwd(None, None) == _lib.ERR_NULL
    p = _lib.BwdParams()
    p.struct_size = 16
    assert lib.b200_sdpa_bwd(C.byref(p), None) == _lib.ERR_STRUCT
    p.struct_size = C.sizeof(_lib.BwdParams)
    p.dtype = 9
    assert lib.b200_sdpa_bwd(C.byref(p), None) == _lib.ERR_DTYPE
    p.dtype = _lib.BF16
    assert lib.b200_sdpa_bwd(C.byref(p), None) == _lib.ERR_SHAPE
    p.B, p.Hq, p.Hkv, p.L, p.S, p.E, p.Dv = 1, 6, 4, 8, 8, 16, 16
    assert lib.b200_sdpa_bwd(C.byref(p), None) == _lib.ERR_SHAPE
    p.Hkv = 2
    assert lib.b200_sdpa_bwd(C.byref(p), None) == _lib.ERR_NULL  # no pointers given


def _bwd_params(B=2, Hq=8, Hkv=2, L=300, S=300, D=128, dtype=_lib.BF16, **kw):
    p = _lib.BwdParams()
    p.struct_size = C.sizeof(_lib.BwdParams)
    p.dtype, p.device = dtype, -1
    fake = 0x7F0000000000  # never dereferenced by the planner
    names = ("grad_out", "q", "k", "v", "out", "lse", "grad_q", "grad_k", "grad_v")
    for i, n in enumerate(names):
        setattr(p, n, fake + (i << 30))
    p.B, p.Hq, p.Hkv, p.L, p.S, p.E, p.Dv = B, Hq, Hkv, L, S, D, D
    qs = [Hq * L * D, L * D, D, 1]
    ks = [Hkv * S * D, S * D, D, 1]
    for n in ("grad_out_stride", "q_stride", "out_stride", "grad_q_stride"):
        getattr(p, n)[:] = qs
    for n in ("k_stride", "v_stride", "grad_k_stride", "grad_v_stride"):
        getattr(p, n)[:] = ks
    p.lse_stride[:] = [Hq * L, L, 1]
    p.scale = 0.1
    for k_, v_ in kw.items():
        setattr(p, k_, v_)
    return p


def _bwd_plan(p):
    plan = _lib.Plan()
    plan.struct_size = C.sizeof(_lib.Plan)
    return _lib.load().b200_sdpa_bwd_query_plan(C.byref(p), C.byref(plan)), plan


def test_backward_planner():
    rc, plan = _bwd_plan(_bwd_params())
    assert rc == 0 and plan.path == _lib.PATH_PREFILL and plan.launches == 3 and plan.threads == 320
    assert plan.workspace_bytes == 2 * 4 * 2 * 8 * 384            # two fp32 rows statistics, L padded to 128
    assert plan.grid_x == 3 * 8 * 2 and plan.grid_y == 3 * 2 * 2  # query tiles x Hq x B, key tiles x Hkv x B
    rc, plan = _bwd_plan(_bwd_params(dtype=_lib.F32, D=64))
    assert rc == 0 and plan.path == _lib.PATH_GENERIC and plan.workspace_bytes == 0 and plan.launches == 2
    rc, plan = _bwd_plan(_bwd_params(D=96))          # head dim the tensor-core kernels are not built for
    assert rc == 0 and plan.path == _lib.PATH_GENERIC
    rc, plan = _bwd_plan(_bwd_params(force_path=_lib.PATH_GENERIC))
    assert rc == 0 and plan.path == _lib.PATH_GENERIC
    p = _bwd_params(force_path=_lib.PATH_PREFILL)
    p.grad_k = 0x7F0000000002                         # misaligned gradient buffer
    assert _bwd_plan(p)[0] == _lib.ERR_ALIGNMENT
    assert _bwd_plan(_bwd_params(force_path=_lib.PATH_PREFILL, dtype=_lib.F32))[0] == _lib.ERR_UNSUPPORTED
    assert _bwd_plan(_bwd_params(force_path=_lib.PATH_DECODE))[0] == _lib.ERR_UNSUPPORTED
    assert _bwd_plan(_bwd_params(D=300))[0] == _lib.ERR_UNSUPPORTED   # beyond the CUDA-core kernels too


def test_paged_cache_planning():
    def paged(**kw):
        p = _params(B=4, Hq=32, Hkv=8, L=1, S=64 * 16, E=128, Dv=128)
        p.k_stride[:] = [16 * 8 * 128, 128, 8 * 128, 1]   # (page, head, row, element) of a (pages, 16, 8, 128) pool
        p.v_stride[:] = [16 * 8 * 128, 128, 8 * 128, 1]
        p.block_table, p.block_table_stride, p.page_size = 0x7F0000400000, 64, 16
        p.kv_lens = 0x7F0000500000
        for k_, v_ in kw.items():
            setattr(p, k_, v_)
        return p

    rc, plan = _plan(paged())
    assert rc == 0 and plan.path == _lib.PATH_DECODE and plan.launches == 2 and plan.workspace_bytes > 0
    assert _plan(paged(page_size=12))[0] == _lib.ERR_SHAPE          # not a power of two
    assert _plan(paged(kv_lens=None))[0] == _lib.ERR_NULL           # lengths are required with a block table
    assert _plan(paged(S=64 * 16 + 1))[0] == _lib.ERR_SHAPE         # more context than the table can address
    assert _plan(paged(L=2))[0] == _lib.ERR_UNSUPPORTED             # only the decode kernel reads pages
    assert _plan(paged(dtype=_lib.F32))[0] == _lib.ERR_UNSUPPORTED
    assert _plan(paged(force_path=_lib.PATH_GENERIC))[0] == _lib.ERR_UNSUPPORTED


def test_append_planning():
    def dec(**kw):
        p = _params(B=4, Hq=32, Hkv=8, L=1, S=2048, E=128, Dv=128)
        p.kv_lens = 0x7F0000500000
        p.k_new, p.v_new = 0x7F0000600000, 0x7F0000700000
        p.k_new_stride[:] = [8 * 128, 128]
        p.v_new_stride[:] = [8 * 128, 128]
        for k_, v_ in kw.items():
            setattr(p, k_, v_)
        return p

    rc, plan = _plan(dec())
    assert rc == 0 and plan.path == _lib.PATH_DECODE
    assert _plan(dec(v_new=None))[0] == _lib.ERR_NULL                     # the two rows go together
    assert _plan(dec(kv_lens=None))[0] == _lib.ERR_NULL                   # the position comes from kv_lens
    assert _plan(dec(kv_lens_out=0x7F0000500000))[0] == _lib.ERR_UNSUPPORTED   # must not alias kv_lens
    assert _plan(dec(L=2))[0] == _lib.ERR_UNSUPPORTED                     # decode only
    assert _plan(dec(dtype=_lib.F32))[0] == _lib.ERR_UNSUPPORTED
    p = dec()
    p.k_new_stride[:] = [8 * 128 + 4, 128]                                # rows not 16-byte aligned
    assert _plan(p)[0] == _lib.ERR_UNSUPPORTED
    # rotary tables: both or none, only together with an appended row, at least E/2 columns
    # and a stated number of table rows
    rope = dict(rope_cos=0x7F0000800000, rope_sin=0x7F0000900000, rope_stride=64, rope_positions=2048)
    assert _plan(dec(**rope))[0] == 0
    assert _plan(dec(rope_cos=0x7F0000800000, rope_stride=64, rope_positions=2048))[0] == _lib.ERR_NULL
    assert _plan(dec(k_new=None, v_new=None, **rope))[0] == _lib.ERR_UNSUPPORTED
    assert _plan(dec(**{**rope, "rope_stride": 32}))[0] == _lib.ERR_UNSUPPORTED
    assert _plan(dec(**{**rope, "rope_positions": 0}))[0] == _lib.ERR_SHAPE


def test_bias_planning():
    """An additive bias stays on the tcgen05 kernel when its softmax threads can read it as 16-byte
    pieces of a row: the query's dtype, unit stride along the keys, S % 8 == 0, aligned rows."""
    fake_bias = 0x7F4000000000
    L = S = 512
    full = dict(bias=fake_bias, bias_dtype=_lib.BF16)

    def plan_with(stride, **kw):
        p = _params(L=L, S=kw.pop("S", S), **{**full, **kw})
        p.bias_stride[:] = stride
        return _plan(p)

    rc, plan = plan_with([8 * L * S, L * S, S, 1])
    assert rc == 0 and plan.path == _lib.PATH_PREFILL
    rc, plan = plan_with([0, 0, S, 1])                       # broadcast over batch and heads
    assert rc == 0 and plan.path == _lib.PATH_PREFILL
    rc, plan = plan_with([S, 0, 0, 1])                       # per batch and key
    assert rc == 0 and plan.path == _lib.PATH_PREFILL
    rc, plan = plan_with([8 * L * S, L * S, S, 1], E=64, Dv=64)
    assert rc == 0 and plan.path == _lib.PATH_PREFILL
    # everything else is served by the CUDA-core kernel
    rc, plan = plan_with([8 * L * S, L * S, S, 1], bias_dtype=_lib.F32)
    assert rc == 0 and plan.path == _lib.PATH_GENERIC
    rc, plan = plan_with([8 * L * S, L * S, S, 1], bias_dtype=_lib.F16)
    assert rc == 0 and plan.path == _lib.PATH_GENERIC       # not the query's dtype
    rc, plan = plan_with([8 * L * 2 * S, L * 2 * S, 2 * S, 2])
    assert rc == 0 and plan.path == _lib.PATH_GENERIC       # strided along the keys
    rc, plan = plan_with([8 * L * 500, L * 500, 500, 1], S=500)
    assert rc == 0 and plan.path == _lib.PATH_GENERIC       # S % 8 != 0
    rc, plan = plan_with([8 * L * S, L * S, S + 4, 1])
    assert rc == 0 and plan.path == _lib.PATH_GENERIC       # rows off the 16-byte grid
    rc, plan = plan_with([8 * L * S, L * S, S, 1], bias=fake_bias + 2)
    assert rc == 0 and plan.path == _lib.PATH_GENERIC
    rc, plan = plan_with([8 * L * S, L * S, S, 1], E=192, Dv=128)
    assert rc == 0 and plan.path == _lib.PATH_PREFILL       # the wide kernel reads it the same way


def test_cpp_operator_layer_loads_and_registers():
    """The C++ operator layer is an in-tree shared library next to the kernel library; loading it registers the
    CUDA kernels of the two ATen ops and the status-word accessor (no GPU needed to load)."""
    import torch

    import torch_neuronx_b200 as T

    assert os.path.exists(_lib.OPS_LIB_PATH), "build it with python -m torch_neuronx_b200.build"
    assert T.ops.native_op_layer()
    assert hasattr(torch.ops.b200_sdpa_native, "status_word")
    q = torch.randn(1, 2, 8, 16)
    with pytest.raises(NotImplementedError):        # CPU tensors never reach the CUDA kernel
        torch.ops.aten._scaled_dot_product_fused_attention_overrideable(q, q, q)


def test_accumulating_form_planning():
    """The accumulating form (one ring step folded into a running fp32 result) is served by the tensor-core
    prefill kernels at head dim 128 (the one with one item per CTA unless B200_SDPA_PREFILL says otherwise);
    everything else is declined so that the caller merges separately."""
    acc = dict(acc_mode=2, acc=0x7F5000000000, acc_lse=0x7F5100000000)

    def plan_acc(**kw):
        p = _params(**{**dict(B=1, Hq=8, Hkv=2, L=512, S=512), **acc, **kw})
        p.acc_stride[:] = [8 * 512 * 128, 512 * 128, 128]
        p.acc_lse_stride[:] = [8 * 512, 512, 1]
        return _plan(p)

    rc, plan = plan_acc()
    assert rc == 0 and plan.path == _lib.PATH_PREFILL and plan.threads == 320      # a small problem: one item per CTA
    rc, plan = plan_acc(B=4, Hq=32, Hkv=8, L=4096, S=4096)
    assert rc == 0 and plan.threads == 320          # also where the plain call would take persistent CTAs: ring
    rc, plan = plan_acc(Hq=64, Hkv=8, L=16384, S=16384)                            # steps run under the power cap,
    assert rc == 0 and plan.threads == 320                                         # where one item per CTA is faster
    assert plan_acc(E=64, Dv=64)[0] == _lib.ERR_UNSUPPORTED
    assert plan_acc(dtype=_lib.F32)[0] == _lib.ERR_UNSUPPORTED
    assert plan_acc(L=1)[0] == 0                                                   # one row still goes to that kernel
    assert plan_acc(acc=None)[0] == _lib.ERR_NULL
    assert plan_acc(acc=0x7F5000000004)[0] == _lib.ERR_UNSUPPORTED                 # rows not 16-byte aligned
    assert plan_acc(acc_mode=3)[0] == _lib.ERR_UNSUPPORTED
    assert plan_acc(force_path=_lib.PATH_GENERIC)[0] == _lib.ERR_UNSUPPORTED
    p = _params(B=1, Hq=8, Hkv=2, L=512, S=512, **acc)
    p.out = None                                                                   # no output tensor in this form
    p.acc_stride[:] = [8 * 512 * 128, 512 * 128, 128]
    p.acc_lse_stride[:] = [8 * 512, 512, 1]
    assert _plan(p)[0] == 0
