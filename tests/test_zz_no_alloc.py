"""The decode entry point with built-in scratch, called straight through the C ABI.

Some hosts cannot hand the library a workspace: a serving process that gave all device
memory to its own pool at start-up (a later cudaMalloc fails or is forbidden), or code on
a path where allocator calls are not allowed.  ``b200_sdpa_decode_static`` serves them
from a fixed array inside the library.  Here it must give the same answer as the regular
entry point on two calls in a row (the array is shared and keeps old contents), and must
refuse a request whose partials do not fit.

The file name sorts last so that a run stopping at the first failure has already run
every other test.
"""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _params(lib_mod, q, k, v, out, lse, lens, kv_chunk, workspace=None):
    p = lib_mod.Params()
    p.struct_size = C.sizeof(lib_mod.Params)
    p.dtype = lib_mod.BF16
    p.device = q.device.index
    p.force_path = lib_mod.PATH_AUTO
    p.q, p.k, p.v, p.out, p.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    p.q_stride[:] = q.stride()
    p.k_stride[:] = k.stride()
    p.v_stride[:] = v.stride()
    p.out_stride[:] = out.stride()
    p.lse_stride[:] = lse.stride()
    p.B, p.Hq, p.L, p.E = q.shape
    p.Hkv, p.S, p.Dv = k.shape[1], k.shape[2], v.shape[3]
    p.scale = q.shape[3] ** -0.5
    p.kv_lens = lens.data_ptr()
    p.kv_chunk = kv_chunk
    if workspace is not None:
        p.workspace, p.workspace_bytes = workspace.data_ptr(), workspace.numel()
    return p


def test_static_scratch_decode_matches_the_workspace_entry_point_twice():
    from torch_neuronx_b200 import _lib

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    g = torch.Generator().manual_seed(99)
    for call, (B, S, chunk) in enumerate([(5, 3000, 512), (3, 1200, 256)]):
        q = torch.randn(B, 32, 1, 128, generator=g).to(torch.bfloat16).to(dev)
        k = torch.randn(B, 8, S, 128, generator=g).to(torch.bfloat16).to(dev)
        v = torch.randn(B, 8, S, 128, generator=g).to(torch.bfloat16).to(dev)
        lens = torch.randint(1, S + 1, (B,), generator=g).to(torch.int32).to(dev)
        want_o = torch.full((B, 32, 1, 128), float("nan"), dtype=torch.bfloat16, device=dev)
        want_l = torch.full((B, 32, 1), float("nan"), dtype=torch.float32, device=dev)
        got_o, got_l = want_o.clone(), want_l.clone()

        plan = _lib.Plan()
        plan.struct_size = C.sizeof(_lib.Plan)
        ref_p = _params(_lib, q, k, v, want_o, want_l, lens, chunk)
        assert lib.b200_sdpa_query_plan(C.byref(ref_p), C.byref(plan)) == _lib.OK
        assert plan.path == _lib.PATH_DECODE and plan.workspace_bytes <= _lib.STATIC_SCRATCH_BYTES
        ws = torch.empty(int(plan.workspace_bytes), dtype=torch.uint8, device=dev)
        ref_p = _params(_lib, q, k, v, want_o, want_l, lens, chunk, workspace=ws)
        assert lib.b200_sdpa_decode(C.byref(ref_p), stream) == _lib.OK

        new_p = _params(_lib, q, k, v, got_o, got_l, lens, chunk)  # no workspace at all
        rc = lib.b200_sdpa_decode_static(C.byref(new_p), stream)
        assert rc == _lib.OK, _lib.strerror(rc)
        torch.cuda.synchronize()
        assert not torch.isnan(got_o.float()).any() and not torch.isnan(got_l).any(), f"call {call}"
        # same kernels, same split geometry, a fixed merge order: the two entry points agree bit for bit
        assert torch.equal(got_o, want_o), f"call {call}: {(got_o.float() - want_o.float()).abs().max().item()}"
        assert torch.equal(got_l, want_l), f"call {call}: {(got_l - want_l).abs().max().item()}"


def test_static_scratch_decode_rejects_what_does_not_fit():
    from torch_neuronx_b200 import _lib

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    B, Hq, S = 64, 64, 8192  # 64 * 64 * 32 splits * 130 floats > 16 MiB
    q = torch.zeros(B, Hq, 1, 128, dtype=torch.bfloat16, device=dev)
    k = torch.zeros(1, 8, S, 128, dtype=torch.bfloat16, device=dev).expand(B, 8, S, 128)
    out = torch.zeros_like(q)
    lse = torch.zeros(B, Hq, 1, dtype=torch.float32, device=dev)
    lens = torch.full((B,), S, dtype=torch.int32, device=dev)
    p = _params(_lib, q, k, k, out, lse, lens, 256)
    rc = lib.b200_sdpa_decode_static(C.byref(p), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    assert rc == _lib.ERR_TOO_LARGE
    assert "capacity" in _lib.strerror(rc)
