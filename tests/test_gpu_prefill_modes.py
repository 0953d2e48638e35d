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


@pytest.mark.parametrize("causal", [False, True])
def test_accumulating_form_folds_key_blocks_into_a_running_result(causal):
    """Three key blocks attended one after the other with the merge done in the kernel's epilogue give the
    attention over all keys (the ring step, ``cp_ring_handler.py:308-318``); rows that see nothing in a block
    (causal: the block lies after them) keep what they had."""
    import torch_neuronx_b200 as T
    from oracle import sdpa_oracle as O

    B, Hq, Hkv, L, S, D = 2, 8, 2, 384, 3 * 256, 128
    q, k, v = make_qkv(21, B, Hq, Hkv, L, S, D, torch.bfloat16)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    big = torch.full((B, Hq, L + 64, D), float("nan"), dtype=torch.float32, device=DEV)   # the accumulator is a view
    acc, acc_lse = big[:, :, 32:32 + L], torch.full((B, Hq, L), float("nan"), dtype=torch.float32, device=DEV)
    q_off = 300                                                     # global position of query row 0
    results = {}
    for form, threads in (("per_cta", 320), ("persistent", 512)):   # both prefill kernels have the form
        os.environ["B200_SDPA_PREFILL"] = form
        try:
            big.fill_(float("nan"))
            acc_lse.fill_(float("nan"))
            T.reset_launch_counts()
            for blk in range(3):
                ok = T.sdpa_forward_accumulate(qd, kd[:, :, blk * 256:(blk + 1) * 256], vd[:, :, blk * 256:(blk + 1) * 256],
                                               acc, acc_lse, first=blk == 0, is_causal=causal, scale=0.1, q_offset=q_off,
                                               k_offset=blk * 256)
                assert ok and T.ops.last_plan["threads"] == threads
            torch.cuda.synchronize()
            T.check_device_status()
        finally:
            os.environ.pop("B200_SDPA_PREFILL", None)
        assert T.launch_counts()["prefill"] == 3 and T.launch_counts()["merge"] == 0
        results[form] = (acc.clone(), acc_lse.clone())
    # the same arithmetic in both kernels
    assert torch.equal(results["per_cta"][0], results["persistent"][0])
    assert torch.equal(results["per_cta"][1], results["persistent"][1])
    ref_o, ref_l = O.sdpa_forward(q, k, v, is_causal=causal, scale=0.1, q_offset=q_off, compute_dtype=torch.float32)
    assert torch.isnan(big[:, :, :32]).all() and torch.isnan(big[:, :, 32 + L:]).all()       # nothing outside the view
    err = (acc.cpu() - ref_o).abs()
    assert err.max().item() <= 2e-2 and err.mean().item() <= 2e-3, err.max().item()
    assert (acc_lse.cpu() - ref_l).abs().max().item() <= 1e-3
    # what the accumulating kernel does not serve is declined, not half done
    q64, k64, v64 = (t.to(DEV) for t in make_qkv(22, 1, 4, 4, 256, 256, 64, torch.bfloat16))
    a64 = torch.zeros(1, 4, 256, 64, device=DEV)
    assert T.sdpa_forward_accumulate(q64, k64, v64, a64, torch.zeros(1, 4, 256, device=DEV), first=True) is False


@pytest.mark.parametrize("layout", ["zigzag", "contiguous"])
def test_ring_with_the_merge_fused_into_the_attention_kernel(layout):
    """The ring driver with every step folded into the accumulator by the attention kernel itself (the default):
    four virtual ranks on one GPU against full attention, no merge kernel launched."""
    import torch_neuronx_b200 as T
    from oracle import sdpa_oracle as O

    world, S = 4, 2048
    q, k, v = make_qkv(31, 1, 8, 2, S, S, 128, torch.bfloat16)
    qs = [T.shard_sequence(q, r, world, layout).contiguous().to(DEV) for r in range(world)]
    ks = [T.shard_sequence(k, r, world, layout).contiguous().to(DEV) for r in range(world)]
    vs = [T.shard_sequence(v, r, world, layout).contiguous().to(DEV) for r in range(world)]
    os.environ["B200_SDPA_RING_FUSED"] = "1"
    try:
        T.reset_launch_counts()
        outs, lses, calls = T.ring_attention_virtual(qs, ks, vs, is_causal=True, layout=layout)
        torch.cuda.synchronize()
        T.check_device_status()
    finally:
        os.environ.pop("B200_SDPA_RING_FUSED", None)
    counts = T.launch_counts()
    assert counts["merge"] == 0 and counts["prefill"] == calls, (counts, calls)
    out = T.unshard_sequence([o.cpu() for o in outs], layout)
    lse = T.unshard_sequence([l.unsqueeze(-1).cpu() for l in lses], layout).squeeze(-1)
    check_against_oracle(q, k, v, out, lse, is_causal=True, tag=f"fused ring {layout}")
