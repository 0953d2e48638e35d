"""DTensor placements and the context-parallel handler among CPU ranks (gloo, world 2).
The per-block compute is replaced by the oracle; everything else -- strategy
registration, dispatch through torch's context-parallel table, ring forward and backward,
wrapping of the results -- is the code the GPUs run."""

import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.test_ring_gloo_cpu import _oracle_attn, _oracle_bwd, _oracle_merge

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torch.distributed.device_mesh import init_device_mesh
        from torch.distributed.tensor import DTensor, Shard
        from torch.distributed.tensor.experimental._context_parallel import _attention as cp

        from oracle import sdpa_oracle as O
        from torch_neuronx_b200 import dtensor as D
        from torch_neuronx_b200 import ring

        mesh = init_device_mesh("cpu", (world,))
        assert D.install_context_parallel_handler()
        D.set_block_functions(_oracle_attn, _oracle_merge, _oracle_bwd)
        D.set_sequence_layout(ring.CONTIGUOUS)
        g = torch.Generator().manual_seed(0)
        S = 16 * world
        q = torch.randn(1, 4, S, 16, generator=g)
        k = torch.randn(1, 2, S, 16, generator=g)
        v = torch.randn(1, 2, S, 16, generator=g)
        go = torch.randn(1, 4, S, 16, generator=g)
        ref_o, ref_l = O.sdpa_forward(q, k, v, is_causal=True, scale=0.25)
        ref_g = O.sdpa_backward(go, q, k, v, ref_o, ref_l, is_causal=True, scale=0.25)

        def dt(t, dim=2):
            return DTensor.from_local(ring.shard_sequence(t, rank, world, ring.CONTIGUOUS, dim=dim).contiguous(),
                                      mesh, [Shard(dim)])

        cp._enable_cp_dtensor_dispatcher()
        try:
            res = torch.ops.aten._scaled_dot_product_fused_attention_overrideable(
                dt(q), dt(k), dt(v), None, 0.0, True, False, scale=0.25)
            out, lse = res[0], res[1]
            zero = torch.zeros((), dtype=torch.int64)
            grads = torch.ops.aten._scaled_dot_product_fused_attention_overrideable_backward(
                dt(go), dt(q), dt(k), dt(v), None, [True, True, True, False], out, lse, None, None, S, S, 0.0, True,
                zero, zero, scale=0.25)
        finally:
            cp._disable_cp_dtensor_dispatcher()
        ok = isinstance(out, DTensor) and out.placements == (Shard(2),) and lse.placements == (Shard(2),)
        ok = ok and (out.full_tensor() - ref_o).abs().max().item() < 1e-5
        ok = ok and (lse.full_tensor() - ref_l).abs().max().item() < 1e-5
        for got, want in zip(grads[:3], ref_g[:3]):
            ok = ok and isinstance(got, DTensor) and got.placements == (Shard(2),)
            ok = ok and (got.full_tensor() - want).abs().max().item() < 2e-5
        torch.save(dict(ok=bool(ok)), os.path.join(result_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_context_parallel_handler_over_gloo(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert torch.load(tmp_path / f"r{r}.pt")["ok"], f"rank {r}"


def test_strategies_cover_replicate_heads_batch_and_sequence():
    """Placement tables by themselves (no process group): one row per placement, outputs
    first, and the sequence row only after the handler was installed."""
    from torch_neuronx_b200 import dtensor as D

    D._sequence_placement = False
    assert [str(p) for p in D._placements()] == ["R", "S(1)", "S(0)"]
    D._sequence_placement = True
    try:
        assert [str(p) for p in D._placements()] == ["R", "S(1)", "S(0)", "S(2)"]
    finally:
        D._sequence_placement = False
