"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle.

Bars (stated once in tests/util.py): fp32 rtol/atol 1e-5; bf16/fp16 max-abs <= 2e-2 and
mean-abs <= 2e-3 against the fp32 oracle; lse abs <= 1e-3 (half) / 1e-5 (fp32); rows
without a visible key exactly 0 / -inf.
"""

import math

import pytest
import torch

from tests.golden_cases import expected_for, inputs_for
from tests.util import check_against_oracle, make_qkv, run_cuda

pytestmark = pytest.mark.gpu

GENERIC, PREFILL, DECODE = 1, 2, 3


def _golden_names():
    import os

    path = os.path.join(os.path.dirname(__file__), "golden", "sdpa_golden.pt")
    return sorted(torch.load(path, weights_only=False)["cases"].keys())


@pytest.mark.parametrize("name", _golden_names())
def test_golden_cases(golden, name):
    """Every committed upstream vector, through the automatic kernel choice."""
    case = golden[name]
    q, k, v, mask = inputs_for(name, case)
    bias = None
    if mask is not None:
        bias = torch.where(mask, 0.0, float("-inf")).to(q.dtype) if mask.dtype == torch.bool else mask
    out, lse = run_cuda(q, k, v, attn_bias=bias, is_causal=case["causal"], scale=case["scale"])
    check_against_oracle(q, k, v, out, lse, attn_mask=mask, is_causal=case["causal"], scale=case["scale"], tag=name)
    # and against the stored upstream output itself (computed in the input dtype)
    for got, want in expected_for(name, case, out, lse):
        finite = torch.isfinite(want.float())
        tol = 1e-5 if q.dtype == torch.float32 else 2e-2
        assert (got.float()[finite] - want.float()[finite]).abs().max().item() <= tol * max(
            1.0, want.float()[finite].abs().max().item()), name


SHAPES = [
    # B, Hq, Hkv, L, S, D
    (1, 1, 1, 1, 1, 64),
    (2, 2, 2, 7, 7, 64),
    (1, 4, 1, 64, 64, 128),
    (1, 2, 2, 127, 127, 64),
    (2, 8, 2, 128, 128, 128),
    (1, 4, 4, 129, 129, 64),
    (1, 8, 1, 577, 577, 128),
    (2, 4, 2, 300, 45, 128),
    (1, 4, 2, 45, 300, 64),
    (1, 2, 1, 512, 1024, 128),
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("path", [GENERIC, PREFILL])
def test_half_paths(shape, causal, dtype, path):
    B, Hq, Hkv, L, S, D = shape
    q, k, v = make_qkv(11, B, Hq, Hkv, L, S, D, dtype)
    out, lse = run_cuda(q, k, v, is_causal=causal, force_path=path)
    check_against_oracle(q, k, v, out, lse, is_causal=causal, tag=f"{shape} causal={causal} path={path}")


@pytest.mark.parametrize("shape", SHAPES[:8])
@pytest.mark.parametrize("causal", [False, True])
def test_fp32_generic(shape, causal):
    B, Hq, Hkv, L, S, D = shape
    q, k, v = make_qkv(12, B, Hq, Hkv, L, S, D, torch.float32)
    out, lse = run_cuda(q, k, v, is_causal=causal)
    check_against_oracle(q, k, v, out, lse, is_causal=causal, tag=f"fp32 {shape}")


@pytest.mark.parametrize("path", [GENERIC, PREFILL])
@pytest.mark.parametrize("causal", [False, True])
def test_right_padding_lengths(path, causal):
    q, k, v = make_qkv(13, 4, 8, 2, 384, 384, 128, torch.bfloat16)
    lens = torch.tensor([384, 1, 200, 0], dtype=torch.int32)
    out, lse = run_cuda(q, k, v, is_causal=causal, kv_lens=lens, force_path=path)
    check_against_oracle(q, k, v, out, lse, is_causal=causal, kv_lens=lens, tag=f"kv_lens path={path}")


@pytest.mark.parametrize("path", [GENERIC, PREFILL])
@pytest.mark.parametrize("offsets", [(256, 0), (0, 256), (128, 64), (100, 300), (64, 128)])
def test_block_offsets(path, offsets):
    """Causal rule between blocks of a longer sequence (ring steps), incl. blocks the
    rule hides completely."""
    qo, ko = offsets
    q, k, v = make_qkv(14, 1, 4, 2, 256, 256, 64, torch.bfloat16)
    out, lse = run_cuda(q, k, v, is_causal=True, q_offset=qo, k_offset=ko, force_path=path)
    check_against_oracle(q, k, v, out, lse, is_causal=True, q_offset=qo, k_offset=ko, tag=f"offsets {offsets}")


def test_explicit_scale_and_head_dims_generic():
    for D, Dv in ((48, 48), (32, 80), (256, 256), (512, 64)):
        q, k, v = make_qkv(15, 1, 2, 1, 70, 90, D, torch.float32, Dv=Dv)
        out, lse = run_cuda(q, k, v, scale=0.2)
        check_against_oracle(q, k, v, out, lse, scale=0.2, tag=f"D={D} Dv={Dv}")
    q, k, v = make_qkv(15, 1, 2, 2, 64, 64, 64, torch.bfloat16)
    out, lse = run_cuda(q, k, v, scale=-0.3)  # negative scale is served by the generic kernel
    check_against_oracle(q, k, v, out, lse, scale=-0.3, tag="negative scale")


@pytest.mark.parametrize("path", [GENERIC, PREFILL])
def test_transposed_storage_and_output_layout(path):
    """(B,S,H,D) storage seen through transpose(1,2): no copies in, and the output takes
    the query's strides (upstream tests/python_ops/test_cpp_dispatch.py:283-297)."""
    import torch_neuronx_b200 as T

    B, H, Hkv, L, D = 2, 8, 2, 320, 128
    g = torch.Generator().manual_seed(16)
    qs = torch.randn(B, L, H, D, generator=g).to(torch.bfloat16)
    ks = torch.randn(B, L, Hkv, D, generator=g).to(torch.bfloat16)
    vs = torch.randn(B, L, Hkv, D, generator=g).to(torch.bfloat16)
    dev = torch.device("cuda", 0)
    q, k, v = (t.to(dev).transpose(1, 2) for t in (qs, ks, vs))
    assert not q.is_contiguous()
    out, lse = T.sdpa_forward(q, k, v, is_causal=True, force_path=path)
    torch.cuda.synchronize()
    T.check_device_status()
    assert out.stride() == q.stride() and out.shape == q.shape
    check_against_oracle(qs.transpose(1, 2), ks.transpose(1, 2), vs.transpose(1, 2), out.cpu(), lse.cpu(),
                         is_causal=True, tag="transposed")


def test_bias_paths_and_dead_rows(golden):
    case = golden["dead_rows_leftpad10"]
    q, k, v, mask = case["q"], case["k"], case["v"], case["mask"]
    bias = torch.where(mask, 0.0, float("-inf"))
    out, lse = run_cuda(q, k, v, attn_bias=bias, scale=case["scale"])
    assert torch.all(out[..., :10, :] == 0) and torch.all(lse[..., :10] == float("-inf"))
    check_against_oracle(q, k, v, out, lse, attn_mask=mask, scale=case["scale"], tag="dead rows")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("group,D", [(1, 64), (4, 128), (8, 128), (3, 64), (16, 128)])
def test_decode_ragged(dtype, group, D):
    import torch_neuronx_b200 as T

    B, Hkv, S = 6, 2, 1500
    q, k, v = make_qkv(17, B, Hkv * group, Hkv, 1, S, D, dtype)
    lens = torch.tensor([1500, 1, 0, 777, 256, 1023], dtype=torch.int32)
    T.reset_launch_counts()
    out, lse = run_cuda(q, k, v, kv_lens=lens, kv_chunk=256)
    counts = T.launch_counts()
    assert counts["decode_partial"] == 1 and counts["decode_combine"] == 1 and counts["prefill"] == 0
    assert T.ops.last_plan["path"] == "decode" and T.ops.last_plan["kv_splits"] == 6
    check_against_oracle(q, k, v, out, lse, kv_lens=lens, tag=f"decode g={group} D={D} {dtype}")
    out2, lse2 = run_cuda(q, k, v, kv_lens=lens, kv_chunk=256)
    assert torch.equal(out, out2) and torch.equal(lse, lse2), "decode must be run-to-run identical"


def test_decode_default_chunk_and_no_lens():
    q, k, v = make_qkv(18, 3, 32, 8, 1, 4096, 128, torch.bfloat16)
    out, lse = run_cuda(q, k, v)
    check_against_oracle(q, k, v, out, lse, tag="decode dense")


def test_kernel_choice_is_observable():
    """Launch counters prove which kernel served a call (upstream:
    tests/utils/neuron_test_utils.py:18-135 assert_op_runs_on_neuron)."""
    import torch_neuronx_b200 as T

    q, k, v = make_qkv(19, 1, 4, 4, 256, 256, 128, torch.bfloat16)
    T.reset_launch_counts()
    run_cuda(q, k, v, is_causal=True)
    assert T.launch_counts()["prefill"] == 1 and T.launch_counts()["generic"] == 0
    qf, kf, vf = make_qkv(19, 1, 4, 4, 256, 256, 128, torch.float32)
    run_cuda(qf, kf, vf, is_causal=True)
    assert T.launch_counts()["generic"] == 1


def test_run_to_run_identical_prefill():
    q, k, v = make_qkv(20, 2, 8, 2, 640, 640, 128, torch.bfloat16)
    a = run_cuda(q, k, v, is_causal=True, force_path=PREFILL)
    b = run_cuda(q, k, v, is_causal=True, force_path=PREFILL)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_merge_kernel_matches_oracle():
    import torch_neuronx_b200 as T
    from oracle import sdpa_oracle as O

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(21)
    B, H, L, D = 2, 3, 50, 64
    pa = torch.randn(B, H, L, D, generator=g).to(torch.bfloat16)
    pb = torch.randn(B, H, L, D, generator=g).to(torch.bfloat16)
    la = torch.randn(B, H, L, generator=g) * 3
    lb = torch.randn(B, H, L, generator=g) * 3
    la[0, 0, :5] = float("-inf")
    lb[0, 0, 3:8] = float("-inf")
    acc = torch.empty(B, H, L, D, dtype=torch.float32, device=dev)
    acc_l = torch.empty(B, H, L, dtype=torch.float32, device=dev)
    fin = torch.full((B, H, L, D), float("nan"), dtype=torch.bfloat16, device=dev)
    T.merge_partials(acc, acc_l, pa.to(dev), la.to(dev), first=True)
    T.merge_partials(acc, acc_l, pb.to(dev), lb.to(dev), first=False, final_out=fin)
    torch.cuda.synchronize()
    ref_o, ref_l = O.merge_partials(pa, la, pb, lb)
    assert torch.equal(acc_l.cpu() == float("-inf"), ref_l == float("-inf"))
    live = ref_l != float("-inf")
    torch.testing.assert_close(acc_l.cpu()[live], ref_l[live], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(acc.cpu(), ref_o, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(fin.cpu().float(), ref_o, rtol=1e-2, atol=1e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(1, 4, 2, 300, 300), (2, 8, 8, 130, 517), (1, 24, 24, 1024, 1024), (2, 4, 1, 1, 200)])
def test_unequal_head_dims_run_on_tensor_cores(shape, causal, dtype):
    # upstream tests/python_ops/test_scaled_dot_product_attention.py:46-97,117-180: qk head dim 192, v head dim 128
    import torch_neuronx_b200 as T

    B, Hq, Hkv, L, S = shape
    g = torch.Generator().manual_seed(L + S + (1 if causal else 0))
    q = torch.randn(B, Hq, L, 192, generator=g).to(dtype)
    k = torch.randn(B, Hkv, S, 192, generator=g).to(dtype)
    v = torch.randn(B, Hkv, S, 128, generator=g).to(dtype)
    lens = torch.randint(1, S + 1, (B,), generator=g).to(torch.int32) if B > 1 else None
    T.reset_launch_counts()
    out, lse = run_cuda(q, k, v, is_causal=causal, kv_lens=lens)
    assert out.shape == (B, Hq, L, 128)
    counts = T.launch_counts()
    assert counts["prefill"] == 1 and counts["generic"] == 0, counts
    check_against_oracle(q, k, v, out, lse, is_causal=causal, kv_lens=lens, tag=f"192/128 {shape} causal={causal}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(1, 4, 2, 300, 300), (2, 2, 2, 130, 517), (1, 8, 8, 1024, 1024)])
def test_head_dim_256_runs_on_tensor_cores(shape, causal, dtype):
    import torch_neuronx_b200 as T

    B, Hq, Hkv, L, S = shape
    q, k, v = make_qkv(L + S, B, Hq, Hkv, L, S, 256, dtype)
    lens = torch.tensor([S, max(1, S // 3)][:B], dtype=torch.int32) if B > 1 else None
    T.reset_launch_counts()
    out, lse = run_cuda(q, k, v, is_causal=causal, kv_lens=lens)
    counts = T.launch_counts()
    assert counts["prefill"] == 1 and counts["generic"] == 0, counts
    check_against_oracle(q, k, v, out, lse, is_causal=causal, kv_lens=lens, tag=f"D=256 {shape} causal={causal}")


def _make_bias(kind, B, Hq, L, S, dtype, g):
    shape = {"full": (B, Hq, L, S), "query_key": (L, S), "batch_key": (B, 1, 1, S), "head": (1, Hq, L, S)}[kind]
    bias = (torch.randn(shape, generator=g) * 2).to(dtype)
    drop = torch.rand(shape, generator=g) < 0.1
    bias = bias.masked_fill(drop, float("-inf"))
    if kind == "full":
        bias[0, 0, min(5, L - 1)] = float("-inf")        # a row without a visible key
    if kind == "batch_key":
        bias[-1, ..., S // 2:] = float("-inf")          # right padding written as a bias
    return bias


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kind", ["full", "query_key", "batch_key", "head"])
@pytest.mark.parametrize("shape", [(2, 4, 2, 300, 304, 128), (1, 8, 8, 520, 1024, 64), (2, 6, 3, 129, 136, 128),
                                   (1, 4, 2, 300, 520, (192, 128)), (1, 2, 2, 260, 264, 256)])
def test_additive_bias_runs_on_tensor_cores(shape, kind, dtype):
    """An additive bias in the query's dtype (what the SDPA front end makes of every mask it does not
    recognise) is read by the softmax threads of the tcgen05 kernel: full, broadcast over batch and
    heads, over heads and queries, and over the batch; -inf entries and a dead row included."""
    import torch_neuronx_b200 as T

    B, Hq, Hkv, L, S, D = shape
    E, Dv = D if isinstance(D, tuple) else (D, D)
    g = torch.Generator().manual_seed(L * 7 + S + E)
    q = torch.randn(B, Hq, L, E, generator=g).to(dtype)
    k = torch.randn(B, Hkv, S, E, generator=g).to(dtype)
    v = torch.randn(B, Hkv, S, Dv, generator=g).to(dtype)
    bias = _make_bias(kind, B, Hq, L, S, dtype, g)
    out, lse = run_cuda(q, k, v, attn_bias=bias)
    assert T.ops.last_plan["path"] == "prefill"
    check_against_oracle(q, k, v, out, lse, attn_mask=bias, tag=f"bias {kind}")
    if kind == "full":
        r = min(5, L - 1)
        assert torch.all(out[0, 0, r] == 0) and lse[0, 0, r] == float("-inf")


def test_additive_bias_with_key_lengths_and_fallbacks():
    import torch_neuronx_b200 as T

    g = torch.Generator().manual_seed(77)
    B, Hq, Hkv, L, S, D = 2, 4, 4, 256, 512, 128
    q = torch.randn(B, Hq, L, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, Hkv, S, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, Hkv, S, D, generator=g).to(torch.bfloat16)
    bias = torch.randn(B, Hq, L, S, generator=g).to(torch.bfloat16)
    lens = torch.tensor([300, 512], dtype=torch.int32)
    out, lse = run_cuda(q, k, v, attn_bias=bias, kv_lens=lens)
    assert T.ops.last_plan["path"] == "prefill"
    check_against_oracle(q, k, v, out, lse, attn_mask=bias, kv_lens=lens, tag="bias + lengths")
    # what the tensor-core kernel cannot read as 16-byte pieces goes to the CUDA-core kernel:
    # a key count that is not a multiple of 8, a bias of another dtype, a strided last dimension
    out, lse = run_cuda(q, k[:, :, :500], v[:, :, :500], attn_bias=bias[..., :500].contiguous())
    assert T.ops.last_plan["path"] == "generic"
    check_against_oracle(q, k[:, :, :500], v[:, :, :500], out, lse, attn_mask=bias[..., :500], tag="S % 8")
    out, lse = run_cuda(q, k, v, attn_bias=bias.float())
    assert T.ops.last_plan["path"] == "generic"
    check_against_oracle(q, k, v, out, lse, attn_mask=bias.float(), tag="fp32 bias")
    wide = torch.randn(B, Hq, L, 2 * S, generator=g).to(torch.bfloat16)
    strided = wide.to("cuda:0")[..., ::2]
    out, lse = T.sdpa_forward(q.to("cuda:0"), k.to("cuda:0"), v.to("cuda:0"), attn_bias=strided)
    torch.cuda.synchronize()
    assert T.ops.last_plan["path"] == "generic"
    check_against_oracle(q, k, v, out.cpu(), lse.cpu(), attn_mask=wide[..., ::2], tag="strided bias")
