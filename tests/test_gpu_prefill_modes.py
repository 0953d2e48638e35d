"""The two forms of the tensor-core prefill kernel -- one work item per CTA, and persistent CTAs that walk a
list of items with a dedicated epilogue warpgroup -- do the same arithmetic in the same order for every query
row, so wherever both can serve a request they must agree BIT FOR BIT, and both must meet the oracle's bar.
``B200_SDPA_PREFILL`` selects the form (read at every launch)."""

import os

import pytest
import torch

from tests.util import check_against_oracle, make_qkv

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(mode, q, k, v, **kw):
    import torch_neuronx_b200 as T

    old = os.environ.get("B200_SDPA_PREFILL")
    os.environ["B200_SDPA_PREFILL"] = mode
    try:
        out = torch.full((q.shape[0], q.shape[1], q.shape[2], v.shape[3]), float("nan"), dtype=q.dtype, device=DEV)
        lse = torch.full(q.shape[:3], float("nan"), dtype=torch.float32, device=DEV)
        for name in ("attn_bias", "kv_lens"):
            if kw.get(name) is not None:
                kw[name] = kw[name].to(DEV)
        T.reset_launch_counts()
        T.sdpa_forward(q.to(DEV), k.to(DEV), v.to(DEV), out=out, lse=lse, **kw)
        torch.cuda.synchronize()
        T.check_device_status()
        assert T.launch_counts()["prefill"] == 1
        plan = dict(T.ops.last_plan)
    finally:
        if old is None:
            os.environ.pop("B200_SDPA_PREFILL", None)
        else:
            os.environ["B200_SDPA_PREFILL"] = old
    return out.cpu(), lse.cpu(), plan


CASES = [
    # B, Hq, Hkv, L, S, causal, lens, q_offset
    (1, 4, 4, 128, 128, False, None, 0),
    (2, 8, 2, 300, 300, True, [300, 170], 0),            # ragged tiles, pair-of-heads layout
    (1, 2, 1, 640, 512, True, None, 0),                   # L > S: rows beyond the keys' triangle
    (2, 4, 4, 257, 1000, False, [1000, 1], 0),            # one visible key
    (1, 6, 2, 384, 384, True, [0], 0),                    # nothing visible at all
    (1, 4, 2, 512, 768, True, None, 256),                 # a ring block: global row offset
    (3, 3, 3, 129, 129, True, None, 0),                   # group of one: row-block layout, second tile almost empty
    (1, 16, 4, 1024, 1024, True, None, 0),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", CASES, ids=[f"c{i}" for i in range(len(CASES))])
def test_both_forms_agree_bit_for_bit_and_with_the_oracle(case, dtype):
    B, Hq, Hkv, L, S, causal, lens, q_off = case
    q, k, v = make_qkv(100 + L + S, B, Hq, Hkv, L, S, 128, dtype)
    kv_lens = None if lens is None else torch.tensor(lens, dtype=torch.int32)
    kw = dict(is_causal=causal, kv_lens=kv_lens, q_offset=q_off)
    o1, l1, plan1 = _run("per_cta", q, k, v, **dict(kw))
    o2, l2, plan2 = _run("persistent", q, k, v, **dict(kw))
    assert plan1["threads"] == 320 and plan2["threads"] == 512, (plan1, plan2)   # the two kernels did run
    assert torch.equal(o1, o2), f"outputs differ: {(o1.float() - o2.float()).abs().max().item()}"
    assert torch.equal(l1, l2), "lse differs"
    check_against_oracle(q, k, v, o2, l2, is_causal=causal, kv_lens=kv_lens, q_offset=q_off, tag=f"persistent {case}")


def test_persistent_form_with_an_additive_bias_and_many_items():
    # 4 x 16 heads x 8 blocks of 256 rows = 512 items (more than three per SM: the automatic choice) with a
    # bias read by the softmax threads; bit-identical to the per-CTA form
    q, k, v = make_qkv(7, 4, 16, 4, 2048, 2048, 128, torch.bfloat16)
    bias = torch.randn(2048, 2048, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16)
    o0, l0, plan0 = _run("auto", q, k, v, attn_bias=bias)
    assert plan0["threads"] == 512 and plan0["grid"][0] == 148
    o1, l1, plan1 = _run("per_cta", q, k, v, attn_bias=bias)
    assert plan1["threads"] == 320
    assert torch.equal(o0, o1) and torch.equal(l0, l1)
    check_against_oracle(q[:1, :4], k[:1, :1], v[:1, :1], o0[:1, :4], l0[:1, :4], attn_mask=bias, tag="persistent + bias")


def test_persistent_form_without_scratch_takes_items_in_a_fixed_order():
    # straight through the C ABI without a workspace: no counter, every CTA walks items c, c + grid, ...
    import ctypes as C

    from torch_neuronx_b200 import _lib

    lib = _lib.load()
    q, k, v = make_qkv(9, 1, 8, 8, 8192, 8192, 128, torch.bfloat16)   # 8 x 32 = 256 items of 256 rows
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    ref_o, ref_l, plan = _run("persistent", q, k, v, is_causal=True)
    assert plan["threads"] == 512
    out = torch.full_like(qd, float("nan"))
    lse = torch.full((1, 8, 8192), float("nan"), dtype=torch.float32, device=DEV)
    p = _lib.Params()
    p.struct_size = C.sizeof(_lib.Params)
    p.dtype, p.device, p.force_path = _lib.BF16, 0, _lib.PATH_PREFILL
    p.q, p.k, p.v, p.out, p.lse = qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), out.data_ptr(), lse.data_ptr()
    p.q_stride[:], p.k_stride[:], p.v_stride[:], p.out_stride[:] = qd.stride(), kd.stride(), vd.stride(), out.stride()
    p.lse_stride[:] = lse.stride()
    p.B, p.Hq, p.Hkv, p.L, p.S, p.E, p.Dv = 1, 8, 8, 8192, 8192, 128, 128
    p.scale, p.is_causal = 128 ** -0.5, 1
    os.environ["B200_SDPA_PREFILL"] = "persistent"
    try:
        rc = lib.b200_sdpa_fwd(C.byref(p), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    finally:
        os.environ.pop("B200_SDPA_PREFILL", None)
    assert rc == _lib.OK, _lib.strerror(rc)
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), ref_o) and torch.equal(lse.cpu(), ref_l)
