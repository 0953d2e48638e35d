"""Full-size configurations: sampled rows against the chunked oracle plus
size-independent properties (probabilities rebuilt from lse sum to one, splitting the
keys and merging reproduces the unsplit result, run-to-run identity)."""

import math

import pytest
import torch

from oracle import sdpa_oracle as O
from tests.util import HALF_LSE_ABS, HALF_MAX_ABS, HALF_MEAN_ABS

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _sample_check(q, k, v, out, lse, slices, **kw):
    ref_o, ref_l = O.sdpa_forward_chunked(q, k, v, row_slices=slices, compute_dtype=torch.float32, **kw)
    for r0, r1 in slices:
        err = (out[:, :, r0:r1].float() - ref_o[:, :, r0:r1]).abs()
        assert err.max().item() <= HALF_MAX_ABS, (r0, r1, err.max().item())
        assert err.mean().item() <= HALF_MEAN_ABS
        assert (lse[:, :, r0:r1] - ref_l[:, :, r0:r1]).abs().max().item() <= HALF_LSE_ABS


def test_config2_gpt2_shape():
    import torch_neuronx_b200 as T

    g = torch.Generator().manual_seed(1)
    q, k, v = ((torch.randn(8, 12, 1024, 64, generator=g) * 0.5).to(torch.bfloat16) for _ in range(3))
    out, lse = T.sdpa_forward(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=True, scale=0.125)
    torch.cuda.synchronize()
    T.check_device_status()
    assert T.ops.last_plan["path"] == "prefill"
    ref_o, ref_l = O.sdpa_forward(q[:2], k[:2], v[:2], is_causal=True, scale=0.125, compute_dtype=torch.float32)
    err = (out[:2].cpu().float() - ref_o).abs()
    assert err.max().item() <= HALF_MAX_ABS and err.mean().item() <= HALF_MEAN_ABS
    assert (lse[:2].cpu() - ref_l).abs().max().item() <= HALF_LSE_ABS


def test_config3_llama_gqa_prefill_with_padding():
    import torch_neuronx_b200 as T

    g = torch.Generator().manual_seed(2)
    q = torch.randn(4, 32, 4096, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(4, 8, 4096, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(4, 8, 4096, 128, generator=g).to(torch.bfloat16)
    lens = torch.randint(2048, 4097, (4,), generator=g).to(torch.int32)
    scale = 1 / math.sqrt(128)
    qd, kd, vd, ld = q.to(DEV), k.to(DEV), v.to(DEV), lens.to(DEV)
    out, lse = T.sdpa_forward(qd, kd, vd, is_causal=True, scale=scale, kv_lens=ld)
    out2, lse2 = T.sdpa_forward(qd, kd, vd, is_causal=True, scale=scale, kv_lens=ld)
    torch.cuda.synchronize()
    T.check_device_status()
    assert T.ops.last_plan["path"] == "prefill"
    assert torch.equal(out, out2) and torch.equal(lse, lse2)
    slices = [(0, 64), (1000, 1064), (2040, 2104), (3000, 3032), (4064, 4096)]
    _sample_check(q, k, v, out.cpu(), lse.cpu(), slices, is_causal=True, scale=scale, kv_lens=lens)
    # property: probabilities rebuilt from the returned lse sum to one (upstream test_sdpa_math.py:30-41)
    b, h, r = 1, 5, 3333
    n = min(int(lens[b]), r + 1)
    logits = (q[b, h, r].float() @ k[b, h // 4, :n].float().T) * scale
    assert abs(torch.exp(logits - lse[b, h, r].cpu()).sum().item() - 1.0) < 5e-3
    # the on-GPU generic kernel agrees on one batch (independent arithmetic path)
    o3, l3 = T.sdpa_forward(qd[3:], kd[3:], vd[3:], is_causal=True, scale=scale, kv_lens=ld[3:], force_path=1)
    torch.cuda.synchronize()
    assert (o3.float() - out[3:].float()).abs().max().item() <= HALF_MAX_ABS
    assert (l3 - lse[3:]).abs().max().item() <= HALF_LSE_ABS


def test_config4_llama_gqa_decode_ragged_cache():
    import torch_neuronx_b200 as T

    g = torch.Generator().manual_seed(3)
    q = torch.randn(64, 32, 1, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(64, 8, 8192, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(64, 8, 8192, 128, generator=g).to(torch.bfloat16)
    lens = torch.randint(512, 8193, (64,), generator=g).to(torch.int32)
    scale = 1 / math.sqrt(128)
    out, lse = T.sdpa_forward(q.to(DEV), k.to(DEV), v.to(DEV), scale=scale, kv_lens=lens.to(DEV))
    torch.cuda.synchronize()
    T.check_device_status()
    assert T.ops.last_plan["path"] == "decode"
    ref_o, ref_l = O.sdpa_forward(q[:16], k[:16], v[:16], scale=scale, kv_lens=lens[:16], compute_dtype=torch.float32)
    err = (out[:16].cpu().float() - ref_o).abs()
    assert err.max().item() <= HALF_MAX_ABS and err.mean().item() <= HALF_MEAN_ABS
    assert (lse[:16].cpu() - ref_l).abs().max().item() <= HALF_LSE_ABS
    # property: splitting the keys differently changes nothing beyond rounding
    out_b, lse_b = T.sdpa_forward(q.to(DEV), k.to(DEV), v.to(DEV), scale=scale, kv_lens=lens.to(DEV), kv_chunk=2048)
    torch.cuda.synchronize()
    assert (out_b.float() - out.float()).abs().max().item() <= 1e-2
    assert (lse_b - lse).abs().max().item() <= 1e-4


@pytest.mark.parametrize("layout", ["zigzag", "contiguous"])
@pytest.mark.parametrize("world", [2, 4])
def test_ring_schedule_on_one_device(layout, world):
    """All ranks of a ring emulated in this process: the per-rank step logic, offsets and
    merges must reproduce full causal attention; and (negative guard, upstream
    tests/distributed/dtensor/test_scaled_dot_product_attention.py:624-628) must differ
    from attention over the local shard only."""
    import torch_neuronx_b200 as T

    g = torch.Generator().manual_seed(4)
    S = 2048
    q = torch.randn(1, 8, S, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(1, 2, S, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(1, 2, S, 128, generator=g).to(torch.bfloat16)
    qs = [T.shard_sequence(q, r, world, layout).contiguous().to(DEV) for r in range(world)]
    ks = [T.shard_sequence(k, r, world, layout).contiguous().to(DEV) for r in range(world)]
    vs = [T.shard_sequence(v, r, world, layout).contiguous().to(DEV) for r in range(world)]
    outs, lses, calls = T.ring_attention_virtual(qs, ks, vs, is_causal=True, layout=layout)
    torch.cuda.synchronize()
    T.check_device_status()
    out = T.unshard_sequence([o.cpu() for o in outs], layout)
    lse = T.unshard_sequence([l.cpu().unsqueeze(-1) for l in lses], layout).squeeze(-1)
    ref_o, ref_l = O.sdpa_forward(q, k, v, is_causal=True, compute_dtype=torch.float32)
    err = (out.float() - ref_o).abs()
    assert err.max().item() <= HALF_MAX_ABS and err.mean().item() <= HALF_MEAN_ABS
    assert (lse - ref_l).abs().max().item() <= HALF_LSE_ABS
    local_only, _ = T.sdpa_forward(qs[world - 1], ks[world - 1], vs[world - 1], is_causal=True)
    assert (local_only.cpu().float() - outs[world - 1].cpu().float()).abs().max().item() > 1e-2


@pytest.mark.parametrize(
    "B,Hq,Hkv,L,E,Dv",
    [
        (3, 7, 7, 4096, 128, 128),    # 21 key/value streams of 2 MB: a full wave and a ragged one
        (5, 12, 3, 8192, 128, 128),   # grouped heads (head-pair layout), 15 streams of 4 MB
        (3, 9, 9, 2048, 64, 64),      # head dim 64
        (2, 9, 9, 4096, 192, 128),    # the wide kernel: 18 streams of 2.6 MB
    ],
)
@pytest.mark.parametrize("causal", [True, False])
def test_many_kv_streams_every_cta_lands_on_its_rows(B, Hq, Hkv, L, E, Dv, causal):
    """Problems whose key/value streams do not fit the L2 budget together are issued in waves of
    streams (the last wave ragged here).  The CUDA-core kernels map rows to CTAs independently, so
    agreement of every (batch, head, row) of the output, lse and gradients checks the tensor-core
    kernels' CTA-to-work mapping at sizes the CPU oracle cannot reach."""
    import torch_neuronx_b200 as T
    from torch_neuronx_b200 import _lib

    g = torch.Generator().manual_seed(B * 1000 + Hq)
    q = torch.randn(B, Hq, L, E, generator=g).to(torch.bfloat16).to(DEV)
    k = torch.randn(B, Hkv, L, E, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(B, Hkv, L, Dv, generator=g).to(torch.bfloat16).to(DEV)
    lens = torch.randint(L // 2, L + 1, (B,), generator=g).to(torch.int32).to(DEV)
    out, lse = T.sdpa_forward(q, k, v, is_causal=causal, kv_lens=lens)
    assert T.ops.last_plan["path"] == "prefill"
    ref_o, ref_l = T.sdpa_forward(q, k, v, is_causal=causal, kv_lens=lens, force_path=_lib.PATH_GENERIC)
    torch.cuda.synchronize()
    T.check_device_status()
    assert (out.float() - ref_o.float()).abs().max().item() <= HALF_MAX_ABS
    assert (lse - ref_l).abs().max().item() <= HALF_LSE_ABS
    if E != Dv:
        return   # the backward of unequal head dims has one implementation (CUDA cores)
    go = torch.randn(B, Hq, L, Dv, generator=g).to(torch.bfloat16).to(DEV)
    grads = T.sdpa_backward(go, q, k, v, out, lse, is_causal=causal, kv_lens=lens)
    assert T.ops.last_bwd_plan["path"] == "prefill"
    refs = T.sdpa_backward(go, q, k, v, out, lse, is_causal=causal, kv_lens=lens, force_path=_lib.PATH_GENERIC)
    torch.cuda.synchronize()
    T.check_device_status()
    for name, a, b in zip(("dq", "dk", "dv"), grads, refs):
        err = (a.float() - b.float()).abs()
        scale = b.float().abs().max().item()
        assert err.max().item() <= 2e-2 * max(1.0, scale), (name, err.max().item(), scale)
        assert err.mean().item() <= 2e-3 * max(1.0, scale), (name, err.mean().item())
