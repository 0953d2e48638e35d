"""Helpers shared by the GPU parity tests."""

import math

import torch

from oracle import sdpa_oracle as O

HALF_MAX_ABS = 2e-2   # bf16/fp16 output vs the fp32 oracle: max-abs
HALF_MEAN_ABS = 2e-3  # ... and mean-abs
HALF_LSE_ABS = 1e-3   # lse of half inputs: abs 1e-3 plus 1e-6 relative (fp32 spacing at large |lse|)
HALF_LSE_REL = 1e-6
FP32_RTOL = 1e-5      # fp32 output vs the fp32 oracle
FP32_ATOL = 1e-5


def make_qkv(seed, B, Hq, Hkv, L, S, D, dtype, scale_in=1.0, Dv=None):
    g = torch.Generator().manual_seed(seed)
    Dv = Dv or D
    q = (torch.randn(B, Hq, L, D, generator=g) * scale_in).to(dtype)
    k = (torch.randn(B, Hkv, S, D, generator=g) * scale_in).to(dtype)
    v = (torch.randn(B, Hkv, S, Dv, generator=g) * scale_in).to(dtype)
    return q, k, v


def run_cuda(q, k, v, *, poison=True, **kw):
    """Run the CUDA path on copies of CPU tensors; outputs are NaN-poisoned first so
    an unwritten element cannot pass."""
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    qc, kc, vc = q.to(dev), k.to(dev), v.to(dev)
    for name in ("attn_bias", "kv_lens"):
        if kw.get(name) is not None:
            kw[name] = kw[name].to(dev)
    B, Hq, L, _ = q.shape
    out = T.alloc_like_query(qc, (B, Hq, L, v.shape[3]))
    lse = torch.empty(B, Hq, L, dtype=torch.float32, device=dev)
    if poison:
        out.fill_(float("nan"))
        lse.fill_(float("nan"))
    o, l = T.sdpa_forward(qc, kc, vc, out=out, lse=lse, **kw)
    torch.cuda.synchronize()
    T.check_device_status()
    return o.cpu(), l.cpu()


def check_against_oracle(q, k, v, out, lse, *, attn_mask=None, is_causal=False, scale=None, kv_lens=None,
                         q_offset=0, k_offset=0, tag=""):
    """Parity bar: fp32 within 1e-5; half types within max-abs 2e-2 / mean-abs 2e-3 of
    the fp32 oracle; -inf positions of lse must coincide exactly."""
    ref_o, ref_l = O.sdpa_forward(q, k, v, attn_mask=attn_mask, is_causal=is_causal, scale=scale, kv_lens=kv_lens,
                                  q_offset=q_offset, k_offset=k_offset, compute_dtype=torch.float32)
    assert out.shape == ref_o.shape and lse.shape == ref_l.shape, tag
    assert not torch.isnan(out.float()).any(), f"{tag}: NaN in out (unwritten or bad arithmetic)"
    dead = ref_l == float("-inf")
    assert torch.equal(lse == float("-inf"), dead), f"{tag}: -inf pattern of lse differs"
    assert not torch.isnan(lse).any(), f"{tag}: NaN in lse"
    if dead.any():
        assert torch.all(out[dead] == 0), f"{tag}: dead rows must be exactly zero"
    live = ~dead
    if q.dtype == torch.float32:
        torch.testing.assert_close(out, ref_o, rtol=FP32_RTOL, atol=FP32_ATOL, msg=lambda m: f"{tag}: {m}")
        torch.testing.assert_close(lse[live], ref_l[live], rtol=FP32_RTOL, atol=FP32_ATOL,
                                   msg=lambda m: f"{tag} lse: {m}")
    else:
        err = (out.float() - ref_o).abs()
        assert err.max().item() <= HALF_MAX_ABS, f"{tag}: max-abs {err.max().item():.3e}"
        assert err.mean().item() <= HALF_MEAN_ABS, f"{tag}: mean-abs {err.mean().item():.3e}"
        if live.any():
            lerr = ((lse[live] - ref_l[live]).abs() - HALF_LSE_REL * ref_l[live].abs()).max().item()
            assert lerr <= HALF_LSE_ABS, f"{tag}: lse abs err {lerr:.3e}"
    return ref_o, ref_l


def default_scale(D):
    return 1.0 / math.sqrt(D)
