"""Dense boolean masks that only say "causal" / "right padding" must reach the
tensor-core kernels, give the same numbers as the explicit form, and train."""

import pytest
import torch

from oracle import sdpa_oracle as O
from tests.util import check_against_oracle

pytestmark = pytest.mark.gpu


def _qkv(seed, B, Hq, Hkv, L, S, D, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(B, Hq, L, D, generator=g).to(dtype), torch.randn(B, Hkv, S, D, generator=g).to(dtype),
            torch.randn(B, Hkv, S, D, generator=g).to(dtype))


def test_dense_causal_mask_runs_the_tensor_core_kernel():
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    q, k, v = (t.to(dev) for t in _qkv(1, 2, 8, 2, 512, 512, 128))
    mask = torch.ones(512, 512, dtype=torch.bool, device=dev).tril()
    want = T.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
    T.reset_launch_counts()
    got = T.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=True)
    again = T.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=True)  # cached verdict
    torch.cuda.synchronize()
    counts = T.launch_counts()
    assert counts["prefill"] == 2 and counts["generic"] == 0
    assert torch.equal(got, want) and torch.equal(again, want)
    T.set_mask_recognition(False)
    try:
        T.reset_launch_counts()
        literal = T.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=True)
        torch.cuda.synchronize()
        # taken literally the mask is an additive bias: still the tensor-core kernel (its bias
        # variant), but every key tile is visited
        counts = T.launch_counts()
        assert counts["prefill"] == 1 and counts["generic"] == 0
    finally:
        T.set_mask_recognition(True)
    assert (literal.float() - want.float()).abs().max().item() <= 2e-2


@pytest.mark.parametrize("causal", [False, True])
def test_padding_mask_becomes_key_lengths(causal):
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    q, k, v = _qkv(2, 3, 8, 2, 256, 256, 64)
    lens = torch.tensor([256, 100, 1])
    mask = (torch.arange(256).view(1, 1, 1, 256) < lens.view(3, 1, 1, 1)).expand(3, 1, 256, 256)
    if causal:
        mask = mask & torch.ones(256, 256, dtype=torch.bool).tril()
    mask = mask.contiguous()
    T.reset_launch_counts()
    out = T.scaled_dot_product_attention(q.to(dev), k.to(dev), v.to(dev), attn_mask=mask.to(dev), enable_gqa=True)
    torch.cuda.synchronize()
    counts = T.launch_counts()
    assert counts["prefill"] == 1 and counts["generic"] == 0
    _, lse = O.sdpa_forward(q, k, v, attn_mask=mask, compute_dtype=torch.float32)
    check_against_oracle(q, k, v, out.cpu(), lse, attn_mask=mask, tag=f"padding mask causal={causal}")


def test_recognised_masks_train():
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    q, k, v = _qkv(3, 2, 4, 4, 128, 128, 64, torch.float32)
    go = torch.randn(2, 4, 128, 64, generator=torch.Generator().manual_seed(4))
    lens = torch.tensor([128, 77])
    mask = ((torch.arange(128).view(1, 1, 1, 128) < lens.view(2, 1, 1, 1)) & torch.ones(128, 128, dtype=torch.bool).tril())
    qr, kr, vr = (t.clone().double().requires_grad_() for t in (q, k, v))
    torch.nn.functional.scaled_dot_product_attention(qr, kr, vr, attn_mask=mask).backward(go.double())
    qd, kd, vd = (t.to(dev).requires_grad_() for t in (q, k, v))
    T.reset_launch_counts()
    T.scaled_dot_product_attention(qd, kd, vd, attn_mask=mask.to(dev)).backward(go.to(dev))
    torch.cuda.synchronize()
    counts = T.launch_counts()
    assert counts["bwd_dq"] == 1 and counts["bwd_dkv"] == 1
    for got, want in ((qd.grad, qr.grad), (kd.grad, kr.grad), (vd.grad, vr.grad)):
        torch.testing.assert_close(got.cpu().double(), want, rtol=1e-4, atol=1e-5)


def test_kernel_level_backward_op():
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    q, k, v = (t.to(dev) for t in _qkv(5, 1, 4, 2, 96, 96, 64, torch.float32))
    go = torch.randn(1, 4, 96, 64, generator=torch.Generator().manual_seed(6)).to(dev)
    lse = torch.empty(1, 4, 96, device=dev)
    out = T.scaled_dot_product_attention_kernel(q, k, v, is_causal=True, training=True, lse=lse)
    gq, gk, gv = T.scaled_dot_product_attention_backward_kernel(go, q, k, v, out, lse, is_causal=True)
    want = O.sdpa_backward(go.cpu(), q.cpu(), k.cpu(), v.cpu(), out.cpu(), lse.cpu(), is_causal=True)
    for got, w in zip((gq, gk, gv), want[:3]):
        torch.testing.assert_close(got.cpu(), w, rtol=1e-4, atol=1e-5)
