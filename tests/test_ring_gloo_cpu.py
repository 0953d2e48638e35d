"""World-size-2 and -4 ring attention among CPU ranks (gloo): the same orchestration
code the GPUs run -- schedule, send/recv rotation, merges -- with the block kernel and
the merge replaced by the CPU oracle.  Also a host-side failure: a rank that never joins
makes the others' rendezvous end with an error instead of hanging."""

import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_attn(q, k, v, *, is_causal, scale, q_offset, k_offset):
    from oracle import sdpa_oracle as O

    return O.sdpa_forward(q, k, v, is_causal=is_causal, scale=scale, q_offset=q_offset, k_offset=k_offset)


def _oracle_merge(acc, acc_lse, part, part_lse, first):
    from oracle import sdpa_oracle as O

    if first:
        acc.copy_(part.float())
        acc_lse.copy_(part_lse)
    else:
        o, l = O.merge_partials(acc, acc_lse, part, part_lse)
        acc.copy_(o)
        acc_lse.copy_(l)


def _worker(rank, world, port, layout, causal, result_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import sdpa_oracle as O
        from torch_neuronx_b200 import ring

        g = torch.Generator().manual_seed(0)  # every rank draws the same full tensors
        S = 32 * world
        q = torch.rand(1, 8, S, 32, generator=g)
        k = torch.rand(1, 2, S, 32, generator=g)
        v = torch.rand(1, 2, S, 32, generator=g)
        ql, kl, vl = (ring.shard_sequence(t, rank, world, layout).contiguous() for t in (q, k, v))
        out, lse = ring.ring_attention(ql, kl, vl, is_causal=causal, scale=0.2, layout=layout,
                                       attn_fn=_oracle_attn, merge_fn=_oracle_merge)
        ref_o, ref_l = O.sdpa_forward(q, k, v, is_causal=causal, scale=0.2)
        want_o = ring.shard_sequence(ref_o, rank, world, layout)
        want_l = ring.shard_sequence(ref_l.unsqueeze(-1), rank, world, layout).squeeze(-1)
        ok = (out - want_o).abs().max().item() < 1e-5 and (lse - want_l).abs().max().item() < 1e-5
        local_o, _ = O.sdpa_forward(ql, kl, vl, is_causal=causal, scale=0.2)
        differs = (local_o - out).abs().max().item() > 1e-3  # negative guard: not local-only attention
        torch.save(dict(ok=ok, differs=differs), os.path.join(result_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,layout,causal", [(2, "zigzag", True), (2, "contiguous", True),
                                                 (4, "zigzag", True), (2, "zigzag", False)])
def test_ring_attention_over_gloo(tmp_path, world, layout, causal):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, layout, causal, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(tmp_path / f"r{r}.pt")
        assert res["ok"], f"rank {r}: ring result differs from full attention"
        if r == world - 1:  # (rank 0 of a contiguous causal ring legitimately sees only itself)
            assert res["differs"], f"rank {r}: ring result equals local-only attention"


def _lonely_worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime

    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
        outcome = "joined"
    except Exception as e:  # the missing rank surfaces as an error on the host
        outcome = type(e).__name__
    open(os.path.join(result_dir, f"r{rank}.txt"), "w").write(outcome)


def test_missing_rank_is_detected_on_the_host(tmp_path):
    """Rank 1 of 2 never starts: rank 0 must get an exception within the timeout."""
    port = _free_port()
    ctx = mp.get_context("spawn")
    p = ctx.Process(target=_lonely_worker, args=(0, 2, port, str(tmp_path)))
    p.start()
    p.join(60)
    assert not p.is_alive()
    assert open(tmp_path / "r0.txt").read() != "joined"
