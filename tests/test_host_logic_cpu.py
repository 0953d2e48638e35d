"""Host-side logic that needs no GPU: argument validation and messages, output layout
rule, work partitioning, the ring schedule, and the registered op schemas."""

import pytest
import torch

import torch_neuronx_b200 as T
from torch_neuronx_b200 import ops, ring


def test_validation_messages_match_upstream_wording():
    q = torch.randn(1, 4, 8, 16)
    with pytest.raises(ValueError, match="Expected CUDA device"):
        T.scaled_dot_product_attention(q, q, q)
    with pytest.raises(RuntimeError, match="same dtype"):
        ops._validate(q, q.half(), q, None, 0.0, False, False)
    with pytest.raises(RuntimeError, match="Explicit attn_mask should not be set when is_causal=True"):
        ops._validate(q, q, q, torch.zeros(8, 8), 0.0, True, False)
    with pytest.raises(NotImplementedError, match="return_debug_mask"):
        ops._validate(q, q, q, None, 0.0, False, True)
    with pytest.raises(ValueError, match=r"outside \[0, 1\]"):
        ops._validate(q, q, q, None, -0.1, False, False)


def test_output_layout_rule_equals_torch_meta_kernel():
    from torch._meta_registrations import alloc_with_matching_layout

    cases = [
        torch.empty(2, 4, 16, 8),
        torch.empty(2, 16, 4, 8).transpose(1, 2),
        torch.empty(2, 4, 16, 24).chunk(3, dim=-1)[1],
        torch.empty(16, 2, 4, 8).permute(1, 2, 0, 3),
    ]
    for q in cases:
        for dv in (8, 6):
            shape = (q.shape[0], q.shape[1], q.shape[2], dv)
            a = T.alloc_like_query(q, shape)
            b = alloc_with_matching_layout(q, shape)
            assert a.shape == b.shape and a.stride() == b.stride(), (q.stride(), dv)


def test_bias_stride_broadcasting():
    b = torch.zeros(2, 1, 1, 7)
    assert ops._bias_strides(b, (2, 4, 5, 7)) == [7, 0, 0, 1]
    assert ops._bias_strides(torch.zeros(5, 7), (2, 4, 5, 7)) == [0, 0, 7, 1]
    with pytest.raises(RuntimeError, match="not broadcastable"):
        ops._bias_strides(torch.zeros(3, 7), (2, 4, 5, 7))


def test_partition_units_is_exact_and_balanced():
    for n in (1, 7, 32, 96, 512):
        for w in (1, 2, 4, 8):
            parts = T.partition_units(n, w)
            assert parts[0][0] == 0 and parts[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
            sizes = [e - s for s, e in parts]
            assert max(sizes) - min(sizes) <= 1
    g = torch.Generator().manual_seed(0)
    costs = torch.randint(512, 8193, (512,), generator=g).tolist()
    parts = T.partition_units(512, 8, costs)
    loads = [sum(costs[s:e]) for s, e in parts]
    assert parts[-1][1] == 512 and max(loads) / (sum(loads) / 8) < 1.05


def test_units_view_roundtrip():
    q = torch.arange(2 * 8 * 3 * 4, dtype=torch.float32).reshape(2, 8, 3, 4)
    k = torch.randn(2, 2, 5, 4)
    v = torch.randn(2, 2, 5, 4)
    lens = torch.tensor([5, 2], dtype=torch.int32)
    qu, ku, vu, lu = T.as_units(q, k, v, lens)
    assert qu.shape == (4, 4, 3, 4) and ku.shape == (4, 1, 5, 4) and lu.tolist() == [5, 5, 2, 2]
    assert torch.equal(qu[3], q[1, 4:8]) and torch.equal(ku[3, 0], k[1, 1])
    assert torch.equal(T.from_units(qu, 2, 2), q)


@pytest.mark.parametrize("layout", [ring.ZIGZAG, ring.CONTIGUOUS])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_ring_schedule_covers_exactly_the_causal_pairs(layout, world):
    """Union over steps of the (query, key) pairs each rank computes == the causal
    triangle restricted to its rows, each pair exactly once."""
    n_local = 16
    S = n_local * world
    pos = torch.arange(S).view(1, 1, S, 1)
    for rank in range(world):
        my_pos = ring.shard_sequence(pos, rank, world, layout).flatten()
        seen = torch.zeros(n_local, S, dtype=torch.int32)
        for step in range(world):
            src = (rank - step) % world
            src_pos = ring.shard_sequence(pos, src, world, layout).flatten()
            for c in ring.ring_schedule(rank, src, world, n_local, layout, True):
                for i in range(c.q0, c.q1):
                    for j in range(c.k0, c.k1):
                        vis = (not c.causal) or (c.k_offset + (j - c.k0) <= c.q_offset + (i - c.q0))
                        if vis:
                            seen[i, src_pos[j]] += 1
        want = (torch.arange(S).view(1, S) <= my_pos.view(n_local, 1)).to(torch.int32)
        assert torch.equal(seen, want), (layout, world, rank)


def test_zigzag_balances_causal_work():
    world, n_local = 8, 64
    work = []
    for rank in range(world):
        w = 0
        for step in range(world):
            for c in ring.ring_schedule(rank, (rank - step) % world, world, n_local, ring.ZIGZAG, True):
                w += (c.q1 - c.q0) * (c.k1 - c.k0) // (2 if c.causal else 1)
        work.append(w)
    assert max(work) / min(work) < 1.01


def test_shard_unshard_roundtrip():
    x = torch.arange(64).view(1, 1, 64, 1)
    for layout in (ring.ZIGZAG, ring.CONTIGUOUS):
        parts = [ring.shard_sequence(x, r, 4, layout) for r in range(4)]
        assert torch.equal(ring.unshard_sequence(parts, layout), x)


def test_ops_are_registered_like_upstream_registers_its_own():
    # kernel-level op visible under torch.ops.<ns>.<name>.default (upstream tests/nki/test_nki_op.py:107-121)
    assert hasattr(torch.ops.b200_sdpa, "fwd") and hasattr(torch.ops.b200_sdpa.fwd, "default")
    schema = str(torch.ops.b200_sdpa.fwd.default._schema)
    assert "bool is_causal, float dropout_p, float? scale, bool training, int? seed" in schema
    # fake/meta execution gives the query-matching layout
    q = torch.empty(2, 16, 4, 8, device="meta").transpose(1, 2)
    out = torch.ops.b200_sdpa.fwd(q, q, q, True, 0.0, None, False, None, None)
    assert out.shape == q.shape and out.stride() == q.stride()
    # the ATen op has a CUDA kernel registered by this package
    assert torch._C._dispatch_has_kernel_for_dispatch_key(
        "aten::_scaled_dot_product_fused_attention_overrideable", "CUDA")


def test_missing_library_is_loud(monkeypatch, tmp_path):
    from torch_neuronx_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.LibraryMissing, match="no CPU or PyTorch fallback"):
        _lib.load()
