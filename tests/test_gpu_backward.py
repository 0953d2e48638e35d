"""Backward parity on the GPU: ``b200_sdpa_bwd`` through the C ABI against the golden
vectors made by upstream's ``compute_attention_backward``, against the oracle on a
matrix of shapes and layouts, through autograd, and -- at full size -- through
identities that hold whatever the size.

Bars: fp32 gradients ``rtol 1e-4 / atol 1e-5`` (upstream's own bar for its backward
formula, ``tests/neuron_dynamo_backend/unit/test_decompositions.py:8742``); half types
``rtol 5e-2 / atol 5e-3`` (upstream's device bar,
``tests/python_ops/test_scaled_dot_product_attention.py:301``) against the fp32 oracle
GIVEN THE SAME forward output and log-sum-exp as the kernel: the backward reads the
half-precision ``out`` through ``delta = sum(dO * out)``, so two backwards fed two
differently rounded ``out`` tensors differ by that rounding, not by their own
arithmetic.  The tests that go forward and backward on the GPU and compare with CPU
autograd carry that rounding and use the forward's half-precision bar (max-abs 2e-2
beside the relative term, mean-abs 2e-3)."""

import math

import pytest
import torch

from oracle import sdpa_oracle as O
from tests.golden_cases import backward_inputs_for

pytestmark = pytest.mark.gpu

FP32_GRAD = dict(rtol=1e-4, atol=1e-5)
HALF_GRAD = dict(rtol=5e-2, atol=5e-3)
# The tensor-core kernels round P and dS to the 16-bit type before their second product (the
# CUDA-core kernels keep them fp32): the forward's half-precision max-abs bar beside the relative term.
HALF_GRAD_TC = dict(rtol=5e-2, atol=2e-2)


def _names():
    import os

    path = os.path.join(os.path.dirname(__file__), "golden", "sdpa_bwd_golden.pt")
    return sorted(torch.load(path, weights_only=False)["cases"].keys())


def _cuda_backward(go, q, k, v, *, mask=None, is_causal=False, scale=None, kv_lens=None, need_grad_bias=False,
                   out=None, lse=None, layout=None, force_path=0):
    """Forward (unless out/lse are given) and backward on the GPU; gradient buffers are
    NaN-poisoned first so that an unwritten element cannot pass."""
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)

    def put(t):
        t = t.to(dev)
        if layout == "bshd":  # (B,S,H,D) storage seen as (B,H,S,D)
            t = t.transpose(1, 2).contiguous().transpose(1, 2)
        return t

    qc, kc, vc, gc = put(q), put(k), put(v), put(go)
    bias = None
    if mask is not None:
        bias = mask.to(dev)
        if bias.dtype == torch.bool:
            bias = torch.where(bias, 0.0, float("-inf")).to(qc.dtype)
    lens = kv_lens.to(dev).to(torch.int32) if kv_lens is not None else None
    if out is None:
        oc, lc = T.sdpa_forward(qc, kc, vc, attn_bias=bias, is_causal=is_causal, scale=scale, kv_lens=lens)
    else:
        oc, lc = put(out), lse.to(dev)
    gq = torch.full_like(qc, float("nan"))
    gk = torch.full_like(kc, float("nan"))
    gv = torch.full_like(vc, float("nan"))
    T.reset_launch_counts()
    gq, gk, gv, gb = T.sdpa_backward(gc, qc, kc, vc, oc, lc, attn_bias=bias, is_causal=is_causal, scale=scale,
                                     kv_lens=lens, need_grad_bias=need_grad_bias, grad_q=gq, grad_k=gk, grad_v=gv,
                                     force_path=force_path)
    torch.cuda.synchronize()
    T.check_device_status()
    counts = T.launch_counts()
    assert counts["bwd_dq"] == 1 and counts["bwd_dkv"] == (1 if k.shape[2] > 0 else 0)
    from torch_neuronx_b200 import ops as _ops
    assert counts["bwd_prep"] == (1 if _ops.last_bwd_plan["path"] == "prefill" else 0)
    _cuda_backward.path = _ops.last_bwd_plan["path"]
    assert gq.stride() == qc.stride() and gk.stride() == kc.stride() and gv.stride() == vc.stride()
    _cuda_backward.forward = (oc.cpu(), lc.cpu())
    return gq.cpu(), gk.cpu(), gv.cpu(), (gb.cpu() if gb is not None else None)


def _close(got, want, dtype, tag, tol=None):
    assert not torch.isnan(got.float()).any(), f"{tag}: NaN (unwritten or bad arithmetic)"
    if tol is None:
        tensor_core = getattr(_cuda_backward, "path", "generic") == "prefill"
        tol = FP32_GRAD if dtype == torch.float32 else (HALF_GRAD_TC if tensor_core else HALF_GRAD)
    torch.testing.assert_close(got.float(), want.float(), msg=lambda m: f"{tag}: {m}", **tol)


@pytest.mark.parametrize("name", _names())
def test_backward_matches_upstream_golden(golden_bwd, name):
    case = golden_bwd[name]
    q, k, v, mask, go = backward_inputs_for(name, case)
    # the forward results upstream's backward was given (the oracle reproduces them bit for bit)
    out, lse = O.sdpa_forward(q, k, v, attn_mask=mask, is_causal=case["causal"], scale=case["scale"])
    gq, gk, gv, _ = _cuda_backward(go, q, k, v, mask=mask, is_causal=case["causal"], scale=case["scale"],
                                   out=out, lse=lse)
    tol = None
    if name.startswith("gqa_") and q.dtype != torch.float32:
        # upstream rounds each head's dK/dV to bf16 and then sums the group in bf16; the kernel sums the
        # group in fp32 and rounds once.  Where a group's terms of size ~1 cancel, upstream's intermediate
        # roundings (2^-8 each) remain: allow the forward's half-precision max-abs bar beside the relative term.
        tol = dict(rtol=5e-2, atol=2e-2)
    for got, key in ((gq, "dq"), (gk, "dk"), (gv, "dv")):
        _close(got, case[key], q.dtype, f"{name} {key}", tol if key != "dq" else None)


def test_backward_dead_rows_are_exact_zero(golden_bwd):
    case = golden_bwd["dead_rows_leftpad10"]
    gq, gk, gv, _ = _cuda_backward(case["grad_out"], case["q"], case["k"], case["v"], mask=case["mask"],
                                   scale=case["scale"])
    assert torch.all(gq[..., :10, :] == 0) and torch.all(gk[..., :10, :] == 0) and torch.all(gv[..., :10, :] == 0)


def _oracle_backward(go, q, k, v, forward=None, **kw):
    """fp32 oracle backward.  ``forward`` = the (out, lse) the kernel under test was given;
    without it the oracle's own fp32 forward is used."""
    f32 = torch.float32
    if forward is None:
        forward = O.sdpa_forward(q, k, v, compute_dtype=f32, **kw)
    return O.sdpa_backward(go, q, k, v, forward[0], forward[1], compute_dtype=f32, **kw)


SHAPES = [
    # B, Hq, Hkv, L,   S,   E,   Dv
    (2, 4, 4, 64, 64, 64, 64),
    (1, 8, 2, 130, 97, 128, 128),    # ragged tails, grouped heads
    (2, 6, 1, 33, 200, 32, 32),      # multi-query
    (1, 2, 2, 77, 77, 16, 48),       # E != Dv
    (1, 4, 2, 96, 160, 192, 128),    # upstream's asymmetric head dims (qk 192 / v 128)
    (1, 2, 1, 50, 70, 256, 256),     # largest head dim served
    (3, 4, 4, 1, 150, 64, 64),       # single query row
    (1, 3, 3, 200, 1, 80, 80),       # single key
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_backward_against_oracle(shape, causal, dtype):
    B, Hq, Hkv, L, S, E, Dv = shape
    g = torch.Generator().manual_seed(hash(shape) % 1000 + (7 if causal else 0))
    q = torch.randn(B, Hq, L, E, generator=g).to(dtype)
    k = torch.randn(B, Hkv, S, E, generator=g).to(dtype)
    v = torch.randn(B, Hkv, S, Dv, generator=g).to(dtype)
    go = torch.randn(B, Hq, L, Dv, generator=g).to(dtype)
    got = _cuda_backward(go, q, k, v, is_causal=causal)
    want = _oracle_backward(go, q, k, v, forward=_cuda_backward.forward, is_causal=causal)
    for a, b, n in zip(got[:3], want[:3], ("dq", "dk", "dv")):
        _close(a, b, dtype, f"{shape} causal={causal} {n}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_backward_transposed_storage_and_kv_lens(dtype):
    g = torch.Generator().manual_seed(21)
    B, Hq, Hkv, L, S, D = 3, 8, 2, 100, 140, 64
    q = torch.randn(B, Hq, L, D, generator=g).to(dtype)
    k = torch.randn(B, Hkv, S, D, generator=g).to(dtype)
    v = torch.randn(B, Hkv, S, D, generator=g).to(dtype)
    go = torch.randn(B, Hq, L, D, generator=g).to(dtype)
    lens = torch.tensor([140, 0, 61])
    got = _cuda_backward(go, q, k, v, is_causal=True, kv_lens=lens, layout="bshd")
    want = _oracle_backward(go, q, k, v, forward=_cuda_backward.forward, is_causal=True, kv_lens=lens)
    for a, b, n in zip(got[:3], want[:3], ("dq", "dk", "dv")):
        _close(a, b, dtype, f"bshd kv_lens {n}")
    assert torch.all(got[0][1] == 0) and torch.all(got[1][1] == 0) and torch.all(got[2][1] == 0)  # batch without keys
    assert torch.all(got[1][2, :, 61:] == 0) and torch.all(got[2][2, :, 61:] == 0)                # padded keys


@pytest.mark.parametrize("bias_shape", [(2, 4, 40, 56), (2, 1, 40, 56), (1, 1, 1, 56), (40, 56)])
def test_backward_with_bias_and_logit_gradient(bias_shape):
    g = torch.Generator().manual_seed(5)
    q = torch.randn(2, 4, 40, 32, generator=g)
    k = torch.randn(2, 2, 56, 32, generator=g)
    v = torch.randn(2, 2, 56, 32, generator=g)
    go = torch.randn(2, 4, 40, 32, generator=g)
    bias = torch.randn(bias_shape, generator=g)
    want = _oracle_backward(go, q, k, v, attn_mask=bias)
    got = _cuda_backward(go, q, k, v, mask=bias, need_grad_bias=True)
    for a, b, n in zip(got, want, ("dq", "dk", "dv", "dbias")):
        assert a.shape == b.shape
        _close(a, b, torch.float32, f"bias {bias_shape} {n}")


def test_logit_gradient_is_written_beyond_the_causal_frontier():
    # a float bias together with a causal frontier expressed through offsets: the logit
    # gradient buffer must be fully written (zeros where masked)
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(9)
    q, k, v, go = (torch.randn(1, 2, 70, 16, generator=g).to(dev) for _ in range(4))
    bias = torch.zeros(1, 1, 70, 70, device=dev)
    out, lse = T.sdpa_forward(q, k, v, attn_bias=bias, is_causal=True)
    _, _, _, gb = T.sdpa_backward(go, q, k, v, out, lse, attn_bias=bias, is_causal=True, need_grad_bias=True)
    torch.cuda.synchronize()
    upper = torch.ones(70, 70, dtype=torch.bool, device=dev).triu(1)
    assert not torch.isnan(gb).any() and torch.all(gb[..., upper] == 0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float64])
@pytest.mark.parametrize("gqa", [False, True])
def test_autograd_through_the_aten_op(dtype, gqa):
    # upstream tests/python_ops/test_scaled_dot_product_attention.py:56-97: CPU autograd vs device autograd,
    # and both device ops must have run
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(42)
    Hq, Hkv = (8, 2) if gqa else (4, 4)
    q = torch.randn(2, Hq, 96, 64, generator=g, dtype=torch.float32)
    k = torch.randn(2, Hkv, 96, 64, generator=g, dtype=torch.float32)
    v = torch.randn(2, Hkv, 96, 64, generator=g, dtype=torch.float32)
    go = torch.randn(2, Hq, 96, 64, generator=g, dtype=torch.float32)
    qr, kr, vr = (t.clone().double().requires_grad_() for t in (q.to(dtype), k.to(dtype), v.to(dtype)))
    ref = torch.nn.functional.scaled_dot_product_attention(qr, kr, vr, is_causal=True, enable_gqa=gqa)
    ref.backward(go.to(dtype).double())

    qd, kd, vd = (t.to(dtype).to(dev).requires_grad_() for t in (q, k, v))
    T.reset_launch_counts()
    out = T.scaled_dot_product_attention(qd, kd, vd, is_causal=True, enable_gqa=gqa)
    out.backward(go.to(dtype).to(dev))
    torch.cuda.synchronize()
    counts = T.launch_counts()
    assert counts["bwd_dq"] == 1 and counts["bwd_dkv"] == 1
    for got, want, n in ((qd.grad, qr.grad, "dq"), (kd.grad, kr.grad, "dk"), (vd.grad, vr.grad, "dv")):
        assert got.shape == want.shape and got.dtype == dtype
        if dtype == torch.bfloat16:
            err = (got.cpu().double() - want).abs()
            assert bool((err <= 2e-2 + 5e-2 * want.abs()).all()), f"autograd bf16 {n}: {err.max().item():.3e}"
            assert err.mean().item() <= 2e-3, f"autograd bf16 {n}: mean {err.mean().item():.3e}"
        else:
            _close(got.cpu(), want, torch.float32, f"autograd {dtype} {n}")


def test_autograd_reduces_the_logit_gradient_to_a_broadcast_bias():
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(3)
    q, k, v, go = (torch.randn(2, 4, 24, 32, generator=g) for _ in range(4))
    bias = torch.randn(2, 1, 24, 24, generator=g)
    qr, kr, vr, br = (t.clone().double().requires_grad_() for t in (q, k, v, bias))
    torch.nn.functional.scaled_dot_product_attention(qr, kr, vr, attn_mask=br).backward(go.double())
    qd, kd, vd, bd = (t.to(dev).requires_grad_() for t in (q, k, v, bias))
    T.scaled_dot_product_attention(qd, kd, vd, attn_mask=bd).backward(go.to(dev))
    torch.cuda.synchronize()
    assert bd.grad.shape == bias.shape
    _close(bd.grad.cpu(), br.grad, torch.float32, "dbias (broadcast over heads)")
    _close(qd.grad.cpu(), qr.grad, torch.float32, "dq with bias")


def test_routed_functional_call_trains():
    import torch_neuronx_b200 as T

    T.enable_sdpa_routing()
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(8)
    q, k, v = (torch.randn(1, 4, 128, 64, generator=g).to(torch.bfloat16).to(dev).requires_grad_() for _ in range(3))
    T.reset_launch_counts()
    out = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    out.float().square().mean().backward()
    torch.cuda.synchronize()
    counts = T.launch_counts()
    assert counts["prefill"] + counts["generic"] == 1 and counts["bwd_dq"] == 1 and counts["bwd_dkv"] == 1
    assert all(torch.isfinite(t.grad.float()).all() for t in (q, k, v))


def test_saturated_softmax_backward_tracks_float32():
    # upstream tests/python_ops/test_sdpa_math.py:44-63: a bf16 backward keeps the fp32 gradient magnitude
    for sat in (8, 32, 64):
        amp = {}
        for dtype in (torch.bfloat16, torch.float32):
            torch.manual_seed(0)
            q = (torch.randn(1, 4, 512, 128) * sat).to(dtype)
            k = (torch.randn(1, 4, 512, 128) * sat).to(dtype)
            v = torch.randn(1, 4, 512, 128).to(dtype)
            go = torch.full((1, 4, 512, 128), 1e-7).to(dtype)
            gq, gk, _, _ = _cuda_backward(go, q, k, v, is_causal=True, scale=128 ** -0.5)
            assert torch.isfinite(gq.float()).all() and torch.isfinite(gk.float()).all()
            amp[dtype] = (gq.float().abs().max().item() / 1e-7, gk.float().abs().max().item() / 1e-7)
        for a, b in zip(amp[torch.bfloat16], amp[torch.float32]):
            assert a == pytest.approx(b, rel=0.25)


def test_backward_full_size_identities():
    """Third benchmark configuration (bf16, 4 x 32/8 heads x 4096 x 128, causal, ragged
    lengths).  Identities that need no reference: every probability row sums to one, so
    the key-summed value gradient equals the row-summed upstream gradient per feature;
    dS enters dQ and dK symmetrically, so sum(q * dq) == sum(k * dk) per kv-head group.
    One (batch, kv head) group is also compared with the oracle."""
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(2)
    B, Hq, Hkv, L, D = 4, 32, 8, 4096, 128
    q = torch.randn(B, Hq, L, D, generator=g).to(torch.bfloat16).to(dev)
    k = torch.randn(B, Hkv, L, D, generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn(B, Hkv, L, D, generator=g).to(torch.bfloat16).to(dev)
    go = torch.randn(B, Hq, L, D, generator=g).to(torch.bfloat16).to(dev)
    lens = torch.tensor([4096, 3500, 2048, 4001], dtype=torch.int32, device=dev)
    out, lse = T.sdpa_forward(q, k, v, is_causal=True, kv_lens=lens)
    gq, gk, gv, _ = T.sdpa_backward(go, q, k, v, out, lse, is_causal=True, kv_lens=lens)
    torch.cuda.synchronize()
    T.check_device_status()
    assert all(torch.isfinite(t.float()).all() for t in (gq, gk, gv))
    # rows of batch b beyond lens[b] still see keys [0, lens[b]) -> all rows are live
    # tolerances: the stored gradients carry one bf16 rounding each (relative 2^-9, random sign), so a
    # sum of n of them is off by about 2^-9 * the 2-norm of the terms; eight such sigmas plus a small floor
    eps = 8 * 2.0 ** -9
    lhs = gv.float().sum(dim=2)
    rhs = go.float().sum(dim=2).view(B, Hkv, Hq // Hkv, D).sum(dim=2)
    tol = eps * gv.float().square().sum(dim=2).sqrt() + 1.0
    assert bool(((lhs - rhs).abs() <= tol).all()), (lhs - rhs).abs().max().item()
    qa, kb = q.float() * gq.float(), k.float() * gk.float()
    a = qa.sum(dim=(2, 3)).view(B, Hkv, Hq // Hkv).sum(dim=2)
    b = kb.sum(dim=(2, 3))
    tol = eps * (qa.square().sum(dim=(2, 3)).view(B, Hkv, Hq // Hkv).sum(dim=2).sqrt()
                 + kb.square().sum(dim=(2, 3)).sqrt()) + 1.0
    assert bool(((a - b).abs() <= tol).all()), (a - b).abs().max().item()
    # one group against the oracle (fp32 on the CPU)
    bi, hk = 1, 5
    hs = slice(hk * 4, hk * 4 + 4)
    qs, ks, vs, gs = q[bi:bi + 1, hs].cpu(), k[bi:bi + 1, hk:hk + 1].cpu(), v[bi:bi + 1, hk:hk + 1].cpu(), go[bi:bi + 1, hs].cpu()
    want = _oracle_backward(gs, qs, ks, vs, forward=(out[bi:bi + 1, hs].cpu(), lse[bi:bi + 1, hs].cpu()),
                            is_causal=True, kv_lens=lens[bi:bi + 1].cpu())
    _close(gq[bi:bi + 1, hs].cpu(), want[0], torch.bfloat16, "full-size dq")
    _close(gk[bi:bi + 1, hk:hk + 1].cpu(), want[1], torch.bfloat16, "full-size dk")
    _close(gv[bi:bi + 1, hk:hk + 1].cpu(), want[2], torch.bfloat16, "full-size dv")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout", ["zigzag", "contiguous"])
def test_ring_backward_with_virtual_ranks(layout, dtype):
    """Four virtual ranks on one GPU: the per-block backward calls (global offsets, the
    final out/lse as normalisers) must add up to the gradients of full attention."""
    import torch_neuronx_b200 as T
    from torch_neuronx_b200 import ring

    dev = torch.device("cuda", 0)
    world = 4
    g = torch.Generator().manual_seed(12)
    S = 128 * world
    q = torch.randn(1, 8, S, 64, generator=g).to(dtype)
    k = torch.randn(1, 2, S, 64, generator=g).to(dtype)
    v = torch.randn(1, 2, S, 64, generator=g).to(dtype)
    go = torch.randn(1, 8, S, 64, generator=g).to(dtype)
    sh = lambda t: [ring.shard_sequence(t, r, world, layout).contiguous().to(dev) for r in range(world)]  # noqa: E731
    qs, ks, vs, gos = sh(q), sh(k), sh(v), sh(go)
    outs, lses, _ = T.ring_attention_virtual(qs, ks, vs, is_causal=True, layout=layout)
    dq, dk, dv, calls = ring.ring_attention_backward_virtual(gos, qs, ks, vs, outs, lses, is_causal=True, layout=layout)
    torch.cuda.synchronize()
    T.check_device_status()
    out = ring.unshard_sequence([o.cpu() for o in outs], layout)
    lse = ring.unshard_sequence([l.cpu().unsqueeze(-1) for l in lses], layout).squeeze(-1)
    want = _oracle_backward(go, q, k, v, forward=(out, lse), is_causal=True)
    for got, w, n in zip((dq, dk, dv), want[:3], ("dq", "dk", "dv")):
        _close(ring.unshard_sequence([t.cpu() for t in got], layout), w, dtype, f"ring {layout} {n}",
               None if dtype == torch.float32 else dict(rtol=5e-2, atol=2e-2))
    assert calls == (world * (world + 1) // 2 if layout == "contiguous" else world * world + world)


TC_SHAPES = [
    # B, Hq, Hkv, L,    S,    D
    (1, 2, 2, 128, 128, 128),
    (2, 4, 2, 256, 384, 128),
    (1, 8, 2, 130, 97, 128),      # ragged tails on both axes, grouped heads
    (1, 4, 1, 333, 517, 64),      # multi-query, head dim 64
    (2, 2, 2, 1, 300, 64),        # single query row
    (1, 2, 2, 300, 1, 128),       # single key
    (1, 4, 4, 1024, 1024, 128),   # eight tiles each way
    (1, 8, 2, 640, 256, 64),      # more rows than keys
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", TC_SHAPES)
def test_tensor_core_backward_against_oracle(shape, causal, dtype):
    from torch_neuronx_b200 import _lib

    B, Hq, Hkv, L, S, D = shape
    g = torch.Generator().manual_seed(sum(shape) + (3 if causal else 0))
    q = torch.randn(B, Hq, L, D, generator=g).to(dtype)
    k = torch.randn(B, Hkv, S, D, generator=g).to(dtype)
    v = torch.randn(B, Hkv, S, D, generator=g).to(dtype)
    go = torch.randn(B, Hq, L, D, generator=g).to(dtype)
    got = _cuda_backward(go, q, k, v, is_causal=causal, force_path=_lib.PATH_PREFILL)
    assert _cuda_backward.path == "prefill"
    fwd = _cuda_backward.forward
    want = _oracle_backward(go, q, k, v, forward=fwd, is_causal=causal)
    ref = _cuda_backward(go, q, k, v, is_causal=causal, force_path=_lib.PATH_GENERIC, out=fwd[0], lse=fwd[1])
    assert _cuda_backward.path == "generic"
    for a, b, c, n in zip(got[:3], want[:3], ref[:3], ("dq", "dk", "dv")):
        # P and dS are rounded to the 16-bit type before their second product: allow the
        # forward's half-precision max-abs bar beside the relative term
        _close(a, b, dtype, f"tc {shape} causal={causal} {n}", dict(rtol=5e-2, atol=2e-2))
        err = (a.float() - b.float()).abs().mean().item()
        assert err <= 2e-3 * max(1.0, b.float().abs().mean().item() * 10), f"{n}: mean-abs {err:.3e}"
        _close(a, c, dtype, f"tc vs cuda-core {shape} causal={causal} {n}", dict(rtol=5e-2, atol=2e-2))


@pytest.mark.parametrize("causal", [False, True])
def test_tensor_core_backward_ragged_lengths_and_transposed_storage(causal):
    from torch_neuronx_b200 import _lib

    g = torch.Generator().manual_seed(31)
    B, Hq, Hkv, L, S, D = 3, 8, 2, 200, 260, 128
    q = torch.randn(B, Hq, L, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, Hkv, S, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, Hkv, S, D, generator=g).to(torch.bfloat16)
    go = torch.randn(B, Hq, L, D, generator=g).to(torch.bfloat16)
    lens = torch.tensor([260, 0, 131])
    got = _cuda_backward(go, q, k, v, is_causal=causal, kv_lens=lens, layout="bshd", force_path=_lib.PATH_PREFILL)
    want = _oracle_backward(go, q, k, v, forward=_cuda_backward.forward, is_causal=causal, kv_lens=lens)
    for a, b, n in zip(got[:3], want[:3], ("dq", "dk", "dv")):
        _close(a, b, torch.bfloat16, f"tc bshd kv_lens {n}", dict(rtol=5e-2, atol=2e-2))
    assert all(torch.all(t[1] == 0) for t in got[:3])                                  # batch without keys
    assert torch.all(got[1][2, :, 131:] == 0) and torch.all(got[2][2, :, 131:] == 0)   # padded keys


def test_tensor_core_backward_is_deterministic():
    from torch_neuronx_b200 import _lib

    g = torch.Generator().manual_seed(77)
    q, k, v, go = (torch.randn(1, 4, 512, 128, generator=g).to(torch.bfloat16) for _ in range(4))
    a = _cuda_backward(go, q, k, v, is_causal=True, force_path=_lib.PATH_PREFILL)
    b = _cuda_backward(go, q, k, v, is_causal=True, force_path=_lib.PATH_PREFILL, out=_cuda_backward.forward[0],
                       lse=_cuda_backward.forward[1])
    assert all(torch.equal(x, y) for x, y in zip(a[:3], b[:3]))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kind", ["full", "query_key", "batch_key", "head"])
@pytest.mark.parametrize("shape", [(2, 4, 2, 300, 304, 128), (1, 8, 8, 520, 1024, 64), (2, 6, 3, 129, 136, 128)])
def test_tensor_core_backward_with_additive_bias(shape, kind, dtype):
    """The forward's additive bias (query dtype, unit stride along the keys) is re-read by both
    tcgen05 backward kernels: row-wise by the grad_q kernel, column-wise (lanes = keys) by the
    grad_k / grad_v kernel; -inf entries and a dead row included."""
    from torch_neuronx_b200 import _lib

    B, Hq, Hkv, L, S, D = shape
    g = torch.Generator().manual_seed(L * 5 + S + D)
    q = torch.randn(B, Hq, L, D, generator=g).to(dtype)
    k = torch.randn(B, Hkv, S, D, generator=g).to(dtype)
    v = torch.randn(B, Hkv, S, D, generator=g).to(dtype)
    go = torch.randn(B, Hq, L, D, generator=g).to(dtype)
    bshape = {"full": (B, Hq, L, S), "query_key": (L, S), "batch_key": (B, 1, 1, S), "head": (1, Hq, L, S)}[kind]
    bias = (torch.randn(bshape, generator=g) * 2).to(dtype)
    bias = bias.masked_fill(torch.rand(bshape, generator=g) < 0.1, float("-inf"))
    if kind == "full":
        bias[0, 0, min(5, L - 1)] = float("-inf")
    got = _cuda_backward(go, q, k, v, mask=bias)
    assert _cuda_backward.path == "prefill"
    fwd = _cuda_backward.forward
    want = _oracle_backward(go, q, k, v, forward=fwd, attn_mask=bias)
    ref = _cuda_backward(go, q, k, v, mask=bias, force_path=_lib.PATH_GENERIC, out=fwd[0], lse=fwd[1])
    assert _cuda_backward.path == "generic"
    for a, b, c, n in zip(got[:3], want[:3], ref[:3], ("dq", "dk", "dv")):
        _close(a, b, dtype, f"tc bias {kind} {shape} {n}", dict(rtol=5e-2, atol=2e-2))
        err = (a.float() - b.float()).abs().mean().item()
        assert err <= 2e-3 * max(1.0, b.float().abs().mean().item() * 10), f"{n}: mean-abs {err:.3e}"
        _close(a, c, dtype, f"tc bias vs cuda-core {kind} {shape} {n}", dict(rtol=5e-2, atol=2e-2))
    if kind == "full":
        assert torch.all(got[0][0, 0, min(5, L - 1)] == 0)
    # the logit gradient is written by the CUDA-core kernels only
    _cuda_backward(go, q, k, v, mask=bias, need_grad_bias=True)
    assert _cuda_backward.path == "generic"


def test_one_element_bias_takes_part_in_the_backward():
    # A (1,1,1,1) bias shifts every logit and therefore lse; only None / an empty tensor mean "no bias"
    # (upstream scaled_dot_product_fused_attention.py:178).  Gradients must match CPU autograd.
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(11)
    q, k, v, go = (torch.randn(2, 3, 20, 32, generator=g) for _ in range(4))
    bias = torch.full((1, 1, 1, 1), 1.5)
    qr, kr, vr, br = (t.clone().double().requires_grad_() for t in (q, k, v, bias))
    torch.nn.functional.scaled_dot_product_attention(qr, kr, vr, attn_mask=br).backward(go.double())
    qd, kd, vd, bd = (t.to(dev).requires_grad_() for t in (q, k, v, bias))
    T.scaled_dot_product_attention(qd, kd, vd, attn_mask=bd).backward(go.to(dev))
    torch.cuda.synchronize()
    _close(qd.grad.cpu(), qr.grad, torch.float32, "dq with a one-element bias")
    _close(kd.grad.cpu(), kr.grad, torch.float32, "dk with a one-element bias")
    _close(vd.grad.cpu(), vr.grad, torch.float32, "dv with a one-element bias")
    assert bd.grad.shape == bias.shape
    assert abs(float(bd.grad.cpu()) - float(br.grad)) <= 1e-4   # the logit gradients sum to zero per row
    # and with B = Hq = L = S = 1 a full-shape bias is a one-element tensor too
    q1, k1, v1, go1 = (torch.randn(1, 1, 1, 32, generator=g) for _ in range(4))
    b1 = torch.full((1, 1, 1, 1), -0.75)
    qd, kd, vd, bd = (t.to(dev).requires_grad_() for t in (q1, k1, v1, b1))
    out = T.scaled_dot_product_attention(qd, kd, vd, attn_mask=bd)
    out.backward(go1.to(dev))
    torch.cuda.synchronize()
    torch.testing.assert_close(out.detach().cpu(), v1, rtol=1e-6, atol=1e-6)          # one key: out = v
    torch.testing.assert_close(vd.grad.cpu(), go1, rtol=1e-6, atol=1e-6)
    assert float(qd.grad.abs().max()) <= 1e-6 and float(kd.grad.abs().max()) <= 1e-6
