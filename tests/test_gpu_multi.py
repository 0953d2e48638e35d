"""Two real GPUs (skipped on a single-GPU box): ring attention over NCCL against the
oracle, and the (batch x kv-head) partition with every rank computing its own units."""

import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    import torch_neuronx_b200 as T
    from oracle import sdpa_oracle as O

    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        g = torch.Generator().manual_seed(0)
        S = 1024 * world
        q = torch.rand(1, 8, S, 128, generator=g).to(torch.bfloat16)
        k = torch.rand(1, 2, S, 128, generator=g).to(torch.bfloat16)
        v = torch.rand(1, 2, S, 128, generator=g).to(torch.bfloat16)
        res = {}
        for layout in ("zigzag", "contiguous"):
            ql, kl, vl = (T.shard_sequence(t, rank, world, layout).contiguous().to(dev) for t in (q, k, v))
            out, lse = T.ring_attention(ql, kl, vl, is_causal=True, scale=0.2, layout=layout)
            torch.cuda.synchronize()
            T.check_device_status()
            ref_o, ref_l = O.sdpa_forward(q, k, v, is_causal=True, scale=0.2, compute_dtype=torch.float32)
            want_o = T.shard_sequence(ref_o, rank, world, layout)
            want_l = T.shard_sequence(ref_l.unsqueeze(-1), rank, world, layout).squeeze(-1)
            res[layout] = ((out.cpu().float() - want_o).abs().max().item(), (lse.cpu() - want_l).abs().max().item())
        # partition of independent units: each rank computes its share, results gathered on the host
        qb = torch.randn(2, 8, 256, 128, generator=g).to(torch.bfloat16)
        kb = torch.randn(2, 2, 256, 128, generator=g).to(torch.bfloat16)
        vb = torch.randn(2, 2, 256, 128, generator=g).to(torch.bfloat16)
        qu, ku, vu, _, (s, e) = T.local_units(qb, kb, vb, rank, world)
        ou, _ = T.sdpa_forward(qu.contiguous().to(dev), ku.contiguous().to(dev), vu.contiguous().to(dev), is_causal=True)
        torch.cuda.synchronize()
        ref_u, _ = O.sdpa_forward(qb, kb, vb, is_causal=True, compute_dtype=torch.float32)
        ref_units = ref_u.reshape(2, 2, 4, 256, 128).flatten(0, 1)[s:e]
        res["units"] = (ou.cpu().float() - ref_units).abs().max().item()
        torch.save(res, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ring_and_partition_on_two_gpus(tmp_path):
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(tmp_path / f"r{r}.pt")
        for layout in ("zigzag", "contiguous"):
            assert res[layout][0] <= 2e-2 and res[layout][1] <= 1e-3, (r, layout, res[layout])
        assert res["units"] <= 2e-2
