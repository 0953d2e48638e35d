"""GPU tests of the operator layer: the ATen override, the kernel-level custom op and
the user-facing function, modelled on upstream's
tests/python_ops/test_scaled_dot_product_attention.py and test_cpp_dispatch.py."""

import math

import pytest
import torch
import torch.nn.functional as F

from oracle import sdpa_oracle as O
from tests.util import HALF_MAX_ABS, check_against_oracle, make_qkv

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float16, 2e-2), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("heads", [(8, 8), (24, 6), (8, 1)])
def test_accuracy_matrix(dtype, tol, heads):
    # upstream test_scaled_dot_product_attention.py:220-302: [1,H,512,64], seed 42, MHA/GQA/MQA
    import torch_neuronx_b200 as T

    hq, hkv = heads
    q, k, v = make_qkv(42, 1, hq, hkv, 512, 512, 64, dtype)
    out = T.scaled_dot_product_attention(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=True, enable_gqa=True)
    ref, _ = O.sdpa_forward(q, k, v, is_causal=True, compute_dtype=torch.float32)
    assert out.dtype == dtype
    assert (out.cpu().float() - ref).abs().max().item() <= tol


def test_aten_op_returns_the_nine_tuple():
    import torch_neuronx_b200  # noqa: F401  (registers the CUDA kernel)

    q, k, v = make_qkv(1, 2, 4, 2, 96, 80, 64, torch.bfloat16)
    res = torch.ops.aten._scaled_dot_product_fused_attention_overrideable(
        q.to(DEV), k.to(DEV), v.to(DEV), None, 0.0, False, False, scale=0.1)
    assert len(res) == 9
    out, lse, cq, ck, max_q, max_k, seed, off, dbg = res
    assert out.shape == (2, 4, 96, 64) and out.dtype == torch.bfloat16
    assert lse.shape == (2, 4, 96) and lse.dtype == torch.float32  # upstream :847-883
    assert max_q == 96 and max_k == 80
    assert cq is None or cq.numel() == 0
    assert dbg is None or dbg.numel() == 0
    # dropout is off: the philox slots are int32 scalar zeros (upstream decompositions.py:2310-2311)
    for slot in (seed, off):
        assert slot.dtype == torch.int32 and slot.dim() == 0 and slot.device.type == "cuda" and int(slot) == 0
    ref_o, ref_l = O.sdpa_forward(q, k, v, scale=0.1, compute_dtype=torch.float32)
    assert (out.cpu().float() - ref_o).abs().max().item() <= HALF_MAX_ABS
    assert (lse.cpu() - ref_l).abs().max().item() <= 1e-3


def test_lse_is_produced_with_grad_disabled():
    # upstream :886-930
    import torch_neuronx_b200  # noqa: F401

    q, k, v = make_qkv(2, 1, 2, 2, 64, 64, 64, torch.float32)
    with torch.no_grad():
        res = torch.ops.aten._scaled_dot_product_fused_attention_overrideable(q.to(DEV), k.to(DEV), v.to(DEV))
    assert res[1].shape == (1, 2, 64) and torch.isfinite(res[1]).all()


def test_bool_and_float_masks_through_the_aten_op():
    import torch_neuronx_b200  # noqa: F401

    q, k, v = make_qkv(3, 2, 4, 4, 51, 51, 48, torch.float32)
    g = torch.Generator().manual_seed(3)
    keep = torch.rand(2, 1, 51, 51, generator=g) > 0.3
    keep[..., 0] = True
    fmask = torch.randn(2, 1, 51, 51, generator=g)
    for m in (keep, fmask):
        out = torch.ops.aten._scaled_dot_product_fused_attention_overrideable(
            q.to(DEV), k.to(DEV), v.to(DEV), m.to(DEV))[0]
        ref, _ = O.sdpa_forward(q, k, v, attn_mask=m)
        torch.testing.assert_close(out.cpu(), ref, rtol=1e-5, atol=1e-5)


def test_error_messages():
    # upstream :305-359 and NeuronDispatcher.cpp:2380-2458
    import torch_neuronx_b200 as T

    q, k, v = (t.to(DEV) for t in make_qkv(4, 1, 4, 4, 16, 16, 32, torch.float32))
    op = torch.ops.aten._scaled_dot_product_fused_attention_overrideable
    with pytest.raises(NotImplementedError, match="return_debug_mask"):
        op(q, k, v, None, 0.0, False, True)
    with pytest.raises(RuntimeError, match="Explicit attn_mask should not be set when is_causal=True"):
        op(q, k, v, torch.zeros(16, 16, device=DEV), 0.0, True)
    with pytest.raises(RuntimeError, match="same dtype"):
        op(q, k.half(), v)
    with pytest.raises(RuntimeError, match="must divide the number of heads in query"):
        op(q, k[:, :3], v[:, :3])
    with pytest.raises(RuntimeError, match="batch sizes must match"):
        op(q, k.repeat(2, 1, 1, 1), v.repeat(2, 1, 1, 1))
    with pytest.raises(RuntimeError, match="4D"):
        op(q[0], k[0], v[0])
    with pytest.raises(ValueError, match="outside"):
        T.scaled_dot_product_attention(q, k, v, dropout_p=1.5)
    with pytest.raises(NotImplementedError, match="dropout"):
        T.scaled_dot_product_attention(q, k, v, dropout_p=0.1)
    with pytest.raises(ValueError, match="Expected CUDA device"):
        T.scaled_dot_product_attention(q.cpu(), k.cpu(), v.cpu())


def test_fp64_is_computed_in_fp32_and_cast_back():
    # upstream :1288-1335
    import torch_neuronx_b200 as T

    q, k, v = make_qkv(5, 1, 2, 2, 40, 40, 32, torch.float64)
    out = T.scaled_dot_product_attention(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=True)
    assert out.dtype == torch.float64
    ref = F.scaled_dot_product_attention(q, k, v, is_causal=True)
    assert (out.cpu() - ref).abs().max().item() < 1e-5


@pytest.mark.parametrize("make_view", ["chunk", "transpose", "as_strided", "expand_kv"])
def test_output_strides_follow_the_query(make_view):
    # upstream :943-1000 (views) and :1123-1221 (stride-0 K/V from repeat_kv)
    import torch_neuronx_b200 as T

    B, H, L, D = 2, 4, 64, 64
    g = torch.Generator().manual_seed(6)
    if make_view == "chunk":
        qkv = torch.randn(B, H, L, 3 * D, generator=g).to(torch.bfloat16)
        q, k, v = qkv.chunk(3, dim=-1)
    elif make_view == "transpose":
        q, k, v = (torch.randn(B, L, H, D, generator=g).to(torch.bfloat16).transpose(1, 2) for _ in range(3))
    elif make_view == "as_strided":
        base = torch.randn(B * H * L * D * 2, generator=g).to(torch.bfloat16)
        q = base.as_strided((B, H, L, D), (H * L * D * 2, L * D * 2, D * 2, 1))
        k, v = (torch.randn(B, H, L, D, generator=g).to(torch.bfloat16) for _ in range(2))
    else:
        q = torch.randn(B, H, L, D, generator=g).to(torch.bfloat16)
        k, v = (torch.randn(B, 1, L, D, generator=g).to(torch.bfloat16).expand(B, H, L, D) for _ in range(2))
    ref_cpu = F.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=True)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    if make_view == "chunk":
        qkv_d = qkv.to(DEV)
        qd, kd, vd = qkv_d.chunk(3, dim=-1)
    elif make_view == "transpose":
        qd, kd, vd = (t.transpose(1, 2).contiguous().to(DEV).transpose(1, 2) for t in (q, k, v))
    elif make_view == "expand_kv":
        kd, vd = (t[:, :1].contiguous().to(DEV).expand(B, H, L, D) for t in (k, v))
    out = T.scaled_dot_product_attention(qd, kd, vd, is_causal=True)
    expect = torch.empty_like(qd).stride()
    assert out.stride() == expect, (out.stride(), expect)
    assert (out.cpu().float() - ref_cpu).abs().max().item() <= HALF_MAX_ABS


def test_kernel_level_op_signature_and_optional_lse():
    # nki_kernels/scaled_dot_product_attention.py:9-41: training=True writes lse, False does not
    import torch_neuronx_b200 as T

    q, k, v = make_qkv(7, 1, 8, 2, 130, 130, 128, torch.bfloat16)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    lse = torch.full((1, 8, 130), float("nan"), device=DEV)
    out = torch.ops.b200_sdpa.fwd(qd, kd, vd, True, 0.0, None, True, None, lse)
    ref_o, ref_l = O.sdpa_forward(q, k, v, is_causal=True, compute_dtype=torch.float32)
    assert (out.cpu().float() - ref_o).abs().max().item() <= HALF_MAX_ABS
    assert (lse.cpu() - ref_l).abs().max().item() <= 1e-3
    out2 = T.scaled_dot_product_attention_kernel(qd, kd, vd, is_causal=True, training=False)
    assert torch.equal(out, out2)
    assert hasattr(torch.ops.b200_sdpa.fwd, "default")  # upstream tests/nki/test_nki_op.py:107-121


def test_functional_sdpa_routing_opt_in():
    import torch_neuronx_b200 as T

    T.enable_sdpa_routing()
    q, k, v = make_qkv(8, 2, 8, 8, 256, 256, 64, torch.bfloat16)
    T.reset_launch_counts()
    out = F.scaled_dot_product_attention(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=True)
    torch.cuda.synchronize()
    assert T.launch_counts()["prefill"] == 1, "plain F.scaled_dot_product_attention must reach the fused kernel"
    ref, _ = O.sdpa_forward(q, k, v, is_causal=True, compute_dtype=torch.float32)
    assert (out.cpu().float() - ref).abs().max().item() <= HALF_MAX_ABS


def test_host_overhead_smoke():
    # upstream :839-844 bounds the median eager call at 10 ms for [1,8,512,64] fp32
    import time

    import torch_neuronx_b200 as T

    q, k, v = (t.to(DEV) for t in make_qkv(9, 1, 8, 8, 512, 512, 64, torch.float32))
    for _ in range(3):
        T.scaled_dot_product_attention(q, k, v, is_causal=True)
    torch.cuda.synchronize()
    times = []
    for _ in range(20):
        t0 = time.perf_counter()
        T.scaled_dot_product_attention(q, k, v, is_causal=True)
        torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
    assert sorted(times)[len(times) // 2] < 10e-3


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,causal", [(torch.float32, False), (torch.float32, True), (torch.bfloat16, True)])
def test_native_multi_head_attn_mid(dtype, causal):
    # upstream tests/python_ops/test_native_multi_head_attn_mid.py:27-62: [B, H, D, S] operands, [B, H, S, D] result
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(4)
    B, H, D, S = 1, 8, 128, 512
    q, k, v = (torch.randn(B, H, D, S, generator=g).to(dtype) for _ in range(3))
    T.reset_launch_counts()
    got = T.native_multi_head_attn_mid(q.to(dev), k.to(dev), v.to(dev), use_causal_mask=causal, dropout_p=0.0,
                                       training=False)
    torch.cuda.synchronize()
    assert got.shape == (B, H, S, D) and got.dtype == dtype
    counts = T.launch_counts()
    assert counts["prefill" if dtype == torch.bfloat16 else "generic"] == 1
    qt, kt, vt = (t.transpose(-2, -1) for t in (q, k, v))
    _, lse = O.sdpa_forward(qt, kt, vt, is_causal=causal, compute_dtype=torch.float32)
    check_against_oracle(qt, kt, vt, got.cpu(), lse, is_causal=causal, tag=f"mha mid {dtype}")
    # out variant: written in place, same storage returned
    out = torch.empty(B, H, S, D, dtype=dtype, device=dev)
    ptr = out.data_ptr()
    res = T.native_multi_head_attn_mid(q.to(dev), k.to(dev), v.to(dev), use_causal_mask=causal, out=out)
    torch.cuda.synchronize()
    assert res.data_ptr() == ptr and torch.equal(res, got)
    with pytest.raises(RuntimeError, match="do not support empty tensors"):
        T.native_multi_head_attn_mid(q[:0].to(dev), k[:0].to(dev), v[:0].to(dev))


@pytest.mark.gpu
def test_traced_training_step_runs_the_same_kernels():
    """``torch.compile`` with the ``aot_eager`` backend: Dynamo + AOTAutograd trace forward and backward
    through the ATen ops (meta kernels for shapes, the derivative formula for the backward graph) and the
    compiled graph then launches the same CUDA kernels."""
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(13)
    q, k, v = (torch.randn(2, 4, 256, 64, generator=g).to(torch.bfloat16).to(dev).requires_grad_() for _ in range(3))

    def step(q, k, v):
        out = torch.ops.aten._scaled_dot_product_fused_attention_overrideable(q, k, v, None, 0.0, True)[0]
        return out.float().square().mean()

    eager = step(q, k, v)
    eager.backward()
    want = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    T.reset_launch_counts()
    compiled = torch.compile(step, backend="aot_eager", fullgraph=True)
    loss = compiled(q, k, v)
    loss.backward()
    torch.cuda.synchronize()
    counts = T.launch_counts()
    assert counts["prefill"] == 1 and counts["bwd_dq"] == 1 and counts["bwd_dkv"] == 1
    assert torch.equal(loss, eager)
    for t, w in zip((q, k, v), want):
        assert torch.equal(t.grad, w)


def test_aten_ops_are_served_by_the_cpp_layer_with_upstream_error_behaviour():
    # upstream checks in its native dispatcher (NeuronDispatcher.cpp:2380-2458); same messages and classes here
    import torch_neuronx_b200 as T

    assert T.ops.native_op_layer(), "libb200_sdpa_ops.so was not built / loaded"
    op = torch.ops.aten._scaled_dot_product_fused_attention_overrideable
    q, k, v = (t.to(DEV) for t in make_qkv(5, 1, 4, 2, 64, 64, 64, torch.bfloat16))
    mask = torch.ones(64, 64, dtype=torch.bool, device=DEV)
    with pytest.raises(RuntimeError, match="Explicit attn_mask should not be set when is_causal=True"):
        op(q, k, v, mask, 0.0, True)
    with pytest.raises(NotImplementedError, match="dropout_p != 0 is not supported"):
        op(q, k, v, None, 0.1)
    with pytest.raises(ValueError, match=r"outside \[0, 1\]"):
        op(q, k, v, None, 1.5)
    with pytest.raises(NotImplementedError, match="return_debug_mask=True is not supported"):
        op(q, k, v, None, 0.0, False, True)
    with pytest.raises(RuntimeError, match="Number of heads in key and value must divide the number of heads in query"):
        op(q[:, :3], k, v)
    with pytest.raises(RuntimeError, match="same dtype"):
        op(q, k.float(), v)
    with pytest.raises(RuntimeError, match="must be 4D tensors"):
        op(q[0], k[0], v[0])
    # float64 is computed in float32 and cast back; a bool mask becomes 0 / -inf
    qd, kd, vd = (t.double() for t in (q, k, v))
    out = op(qd, kd, vd, mask.tril())[0]
    assert out.dtype == torch.float64
    ref, _ = O.sdpa_forward(qd.cpu().float(), kd.cpu().float(), vd.cpu().float(), is_causal=True)
    assert (out.cpu().float() - ref).abs().max().item() <= 1e-5
    # the status word is the one the Python layer reads
    assert T.ops._status_word(0).data_ptr() == torch.ops.b200_sdpa_native.status_word(0).data_ptr()


def test_the_native_layer_runs_from_several_threads():
    # dispatcher kernels run without the interpreter lock; concurrent callers on their own streams get their own
    # scratch from the caching allocator
    import threading

    import torch_neuronx_b200  # noqa: F401

    op = torch.ops.aten._scaled_dot_product_fused_attention_overrideable
    q, k, v = make_qkv(6, 2, 8, 2, 256, 256, 128, torch.bfloat16)
    ref, _ = O.sdpa_forward(q, k, v, is_causal=True, compute_dtype=torch.float32)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    errs = [None] * 4

    def work(i):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.default_stream())
        with torch.cuda.stream(s):
            worst = 0.0
            for _ in range(50):
                out = op(qd, kd, vd, None, 0.0, True)[0]
                worst = max(worst, (out.float().cpu() - ref).abs().max().item())
        errs[i] = worst

    threads = [threading.Thread(target=work, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert all(e is not None and e <= HALF_MAX_ABS for e in errs), errs
