"""Host logic of the structured-mask recognition and the meta kernels of the custom ops
(no GPU: the classification runs on whatever device holds the mask)."""

import pytest
import torch

from torch_neuronx_b200 import masks
from torch_neuronx_b200.masks import classify_mask

L = S = 12
TRIL = torch.ones(L, S, dtype=torch.bool).tril()


def _pad(lens, n_q=1):
    lens = torch.as_tensor(lens)
    return (torch.arange(S).view(1, 1, 1, S) < lens.view(-1, 1, 1, 1)).expand(-1, 1, n_q, S).clone()


def test_causal_triangle_is_recognised_in_every_rank():
    for m in (TRIL.clone(), TRIL[None].clone(), TRIL[None, None].clone()):
        got = classify_mask(m, 2, L, S)
        assert got.recognised and got.is_causal and got.kv_lens is None


def test_rectangular_triangles_are_top_left_aligned():
    for n_q, n_k in ((5, 12), (12, 5)):
        m = torch.ones(n_q, n_k, dtype=torch.bool).tril()
        got = classify_mask(m, 1, n_q, n_k)
        assert got.recognised and got.is_causal and got.kv_lens is None
    # bottom-right alignment is a different mask
    m = torch.ones(5, 12, dtype=torch.bool).tril(diagonal=7)
    assert not classify_mask(m, 1, 5, 12).recognised


def test_all_true_mask_disappears():
    got = classify_mask(torch.ones(1, 1, L, S, dtype=torch.bool), 3, L, S)
    assert got.recognised and not got.is_causal and got.kv_lens is None


@pytest.mark.parametrize("n_q", [1, L])
def test_right_padding_becomes_key_lengths(n_q):
    got = classify_mask(_pad([12, 5, 0], n_q), 3, L, S)
    assert got.recognised and not got.is_causal
    assert got.kv_lens.dtype == torch.int32 and got.kv_lens.tolist() == [12, 5, 0]


def test_one_padding_row_broadcasts_over_the_batch():
    got = classify_mask(_pad([7]), 4, L, S)
    assert got.recognised and got.kv_lens.tolist() == [7, 7, 7, 7]


def test_causal_with_right_padding():
    m = _pad([12, 5, 1], L) & TRIL
    got = classify_mask(m, 3, L, S)
    assert got.recognised and got.is_causal and got.kv_lens.tolist() == [12, 5, 1]


@pytest.mark.parametrize("kind", ["window", "key_offset", "left_pad", "per_head", "hole", "float"])
def test_other_masks_are_kept(kind):
    if kind == "window":
        m = TRIL & ~torch.ones(L, S, dtype=torch.bool).tril(-4)
    elif kind == "key_offset":
        m = torch.ones(L, S, dtype=torch.bool).tril(diagonal=2)
    elif kind == "left_pad":
        m = torch.ones(1, 1, 1, S, dtype=torch.bool)
        m[..., :3] = False
    elif kind == "per_head":
        m = TRIL[None, None].expand(1, 2, L, S).clone()
    elif kind == "hole":
        m = TRIL.clone()
        m[7, 3] = False
    else:
        m = torch.zeros(L, S)
    got = classify_mask(m, 1, L, S)
    assert not got.recognised and got.residual is m and not got.is_causal and got.kv_lens is None


def test_verdict_is_cached_per_tensor_and_version():
    m = TRIL.clone()
    before = dict(masks.stats)
    assert classify_mask(m, 1, L, S).is_causal
    assert classify_mask(m, 1, L, S).is_causal
    assert masks.stats["examined"] == before["examined"] + 1
    assert masks.stats["cache_hits"] == before["cache_hits"] + 1
    m[0, 5] = True  # in-place edit bumps the version counter: examined again, and no longer causal
    assert not classify_mask(m, 1, L, S).recognised
    assert masks.stats["examined"] == before["examined"] + 2
    # an equal but different tensor is its own entry
    assert classify_mask(TRIL.clone(), 1, L, S).is_causal
    assert masks.stats["examined"] == before["examined"] + 3


def test_custom_ops_have_meta_kernels():
    """Shape propagation without running anything (what tracing needs): the kernel-level
    forward and backward ops and the ATen op under fake tensors."""
    import torch_neuronx_b200  # noqa: F401  (registers the ops)
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        q = torch.empty(2, 8, 64, 64, dtype=torch.bfloat16, device="cuda")
        k = torch.empty(2, 2, 96, 64, dtype=torch.bfloat16, device="cuda")
        v = torch.empty(2, 2, 96, 32, dtype=torch.bfloat16, device="cuda")
        qt = torch.empty(2, 64, 8, 64, dtype=torch.bfloat16, device="cuda").transpose(1, 2)
        out = torch.ops.b200_sdpa.fwd(q, k, v, True, 0.0, None, False, None, None)
        assert out.shape == (2, 8, 64, 32) and out.dtype == torch.bfloat16
        out_t = torch.ops.b200_sdpa.fwd(qt, k, v, True, 0.0, None, False, None, None)
        assert out_t.shape == (2, 8, 64, 32) and out_t.stride(1) < out_t.stride(2)  # query's dimension order
        lse = torch.empty(2, 8, 64, device="cuda")
        gq, gk, gv = torch.ops.b200_sdpa.bwd(out, q, k, v, out, lse, True)
        assert gq.shape == q.shape and gk.shape == k.shape and gv.shape == v.shape
        res = torch.ops.aten._scaled_dot_product_fused_attention_overrideable(q, k, v, None, 0.0, True)
        assert res[0].shape == (2, 8, 64, 32) and res[1].shape == (2, 8, 64)
