"""Seeded random problems on the tensor-core kernels while another stream saturates the memory
system, so that loads land at other times than in a quiet run.  The CUDA-core kernels (an
independent arithmetic path with no hand-offs between roles) are the reference; repeated calls
must agree bit for bit.  A hand-off that relies on timing instead of a barrier shows up here as a
wrong or irreproducible row (this is how a missing wait in the head-dim-64 forward was caught)."""

import random

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(rnd, case):
    D = rnd.choice([64, 128, 64, 128, (192, 128), 256])
    E, Dv = D if isinstance(D, tuple) else (D, D)
    group = rnd.choice([1, 1, 2, 4, 8])
    Hkv = rnd.choice([1, 2, 3, 4])
    B = rnd.choice([1, 2, 3])
    L = rnd.choice([64, 128, 200, 256, 384, 520, 1024, 1536, 2048])
    S = rnd.choice([L, L, 8 * rnd.randint(8, 256)])
    causal = rnd.random() < 0.5
    use_bias = (not causal) and rnd.random() < 0.5
    use_lens = rnd.random() < 0.4
    g = torch.Generator().manual_seed(case)
    Hq = Hkv * group
    q = torch.randn(B, Hq, L, E, generator=g).to(torch.bfloat16).to(DEV)
    k = torch.randn(B, Hkv, S, E, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(B, Hkv, S, Dv, generator=g).to(torch.bfloat16).to(DEV)
    go = torch.randn(B, Hq, L, Dv, generator=g).to(torch.bfloat16).to(DEV)
    bias = None
    if use_bias:
        shape = rnd.choice([(B, Hq, L, S), (L, S), (B, 1, 1, S), (1, Hq, L, S)])
        bias = (torch.randn(shape, generator=g) * 2).to(torch.bfloat16)
        bias = bias.masked_fill(torch.rand(shape, generator=g) < 0.05, float("-inf")).to(DEV)
    lens = torch.randint(1, S + 1, (B,), generator=g).to(torch.int32).to(DEV) if use_lens else None
    return q, k, v, go, dict(attn_bias=bias, is_causal=causal, kv_lens=lens), (E, Dv)


@pytest.mark.parametrize("seed", [1, 2])
def test_tensor_core_kernels_under_background_traffic(seed):
    import torch_neuronx_b200 as T
    from torch_neuronx_b200 import _lib

    rnd = random.Random(seed)
    hog_a = torch.empty(512 << 20, dtype=torch.uint8, device=DEV)
    hog_b = torch.empty_like(hog_a)
    side = torch.cuda.Stream()

    def disturb():
        with torch.cuda.stream(side):
            for _ in range(6):
                hog_b.copy_(hog_a, non_blocking=True)

    for case in range(60):
        q, k, v, go, kw, (E, Dv) = _case(rnd, seed * 1000 + case)
        tag = f"seed {seed} case {case}: q{tuple(q.shape)} k{tuple(k.shape)} v{tuple(v.shape)} " \
              f"causal={kw['is_causal']} bias={None if kw['attn_bias'] is None else tuple(kw['attn_bias'].shape)} " \
              f"lens={kw['kv_lens'] is not None}"
        ref_o, ref_l = T.sdpa_forward(q, k, v, force_path=_lib.PATH_GENERIC, **kw)
        torch.cuda.synchronize()
        if rnd.random() < 0.7:
            disturb()
        outs = [T.sdpa_forward(q, k, v, **kw) for _ in range(3)]
        assert T.ops.last_plan["path"] == "prefill", tag
        torch.cuda.synchronize()
        T.check_device_status()
        live = torch.isfinite(ref_l)
        for o, l in outs:
            assert torch.equal(torch.isfinite(l), live), tag
            # (two 16-bit results may differ by a unit in the last place, which grows with the magnitude)
            assert (o.float() - ref_o.float()).abs().max().item() <= 3e-2 * max(1.0, ref_o.float().abs().max().item() / 2), tag
            if live.any():
                assert (l[live] - ref_l[live]).abs().max().item() <= 2e-3, tag
            assert torch.equal(o, outs[0][0]) and torch.equal(l, outs[0][1]), tag + " (forward not reproducible)"
        if E != Dv or E > 128:
            continue   # one backward implementation for these head dims
        o, l = outs[0]
        refs = T.sdpa_backward(go, q, k, v, o, l, force_path=_lib.PATH_GENERIC, **kw)[:3]
        torch.cuda.synchronize()
        if rnd.random() < 0.7:
            disturb()
        grads = [T.sdpa_backward(go, q, k, v, o, l, **kw)[:3] for _ in range(2)]
        assert T.ops.last_bwd_plan["path"] == "prefill", tag
        torch.cuda.synchronize()
        T.check_device_status()
        for gr in grads:
            for name, a, b, first in zip(("dq", "dk", "dv"), gr, refs, grads[0]):
                scale = max(1.0, b.float().abs().max().item())
                assert (a.float() - b.float()).abs().max().item() <= 4e-2 * scale, f"{tag} {name}"
                assert torch.equal(a, first), f"{tag} {name} (backward not reproducible)"
    torch.cuda.synchronize()
