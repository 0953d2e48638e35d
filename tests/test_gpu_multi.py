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


def _train_worker(rank, world, port, out_dir):
    """Forward + backward of a sequence-sharded attention through torch's context-parallel
    dispatch (DTensor inputs) and through the ring driver directly."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import DTensor, Shard
    from torch.distributed.tensor.experimental._context_parallel import _attention as cp

    import torch_neuronx_b200 as T
    from oracle import sdpa_oracle as O
    from torch_neuronx_b200 import dtensor as D

    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        mesh = init_device_mesh("cuda", (world,))
        assert D.install_context_parallel_handler()
        g = torch.Generator().manual_seed(0)
        S = 256 * world
        q = torch.randn(1, 8, S, 64, generator=g)
        k = torch.randn(1, 2, S, 64, generator=g)
        v = torch.randn(1, 2, S, 64, generator=g)
        go = torch.randn(1, 8, S, 64, generator=g)
        ref_o, ref_l = O.sdpa_forward(q, k, v, is_causal=True)
        ref_g = O.sdpa_backward(go, q, k, v, ref_o, ref_l, is_causal=True)
        res = {}
        for layout in ("zigzag", "contiguous"):
            D.set_sequence_layout(layout)
            loc = [T.shard_sequence(t, rank, world, layout).contiguous().to(dev) for t in (q, k, v, go)]
            qd, kd, vd = (DTensor.from_local(t, mesh, [Shard(2)]).requires_grad_() for t in loc[:3])
            cp._enable_cp_dtensor_dispatcher()
            try:
                out = torch.ops.aten._scaled_dot_product_fused_attention_overrideable(qd, kd, vd, None, 0.0, True)[0]
                out.backward(DTensor.from_local(loc[3], mesh, [Shard(2)]))
            finally:
                cp._disable_cp_dtensor_dispatcher()
            torch.cuda.synchronize()
            T.check_device_status()
            errs = [(out.to_local().detach().cpu() - T.shard_sequence(ref_o, rank, world, layout)).abs().max().item()]
            for got, want in zip((qd.grad, kd.grad, vd.grad), ref_g[:3]):
                errs.append((got.to_local().cpu() - T.shard_sequence(want, rank, world, layout)).abs().max().item())
            res[layout] = errs
        # head- and batch-sharded DTensors need no exchange: DTensor's ordinary dispatch runs the op on the
        # local shards with the placements registered in torch_neuronx_b200.dtensor
        qb = torch.randn(2, 8, 128, 64, generator=g)
        kb = torch.randn(2, 2, 128, 64, generator=g)
        vb = torch.randn(2, 2, 128, 64, generator=g)
        gob = torch.randn(2, 8, 128, 64, generator=g)
        rb_o, rb_l = O.sdpa_forward(qb, kb, vb, is_causal=True)
        rb_g = O.sdpa_backward(gob, qb, kb, vb, rb_o, rb_l, is_causal=True)
        for dim in (0, 1):
            parts = [t.chunk(world, dim=dim)[rank].contiguous().to(dev) for t in (qb, kb, vb, gob)]
            qd, kd, vd = (DTensor.from_local(t, mesh, [Shard(dim)]).requires_grad_() for t in parts[:3])
            outd = torch.ops.aten._scaled_dot_product_fused_attention_overrideable(qd, kd, vd, None, 0.0, True)[0]
            outd.backward(DTensor.from_local(parts[3], mesh, [Shard(dim)]))
            torch.cuda.synchronize()
            errs = [(outd.to_local().detach().cpu() - rb_o.chunk(world, dim=dim)[rank]).abs().max().item()]
            for got, want in zip((qd.grad, kd.grad, vd.grad), rb_g[:3]):
                errs.append((got.to_local().cpu() - want.chunk(world, dim=dim)[rank]).abs().max().item())
            assert outd.placements == (Shard(dim),)
            res[f"shard{dim}"] = errs
        torch.save(res, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_context_parallel_training_step_on_two_gpus(tmp_path):
    import torch.multiprocessing as mp

    mp.spawn(_train_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(tmp_path / f"r{r}.pt")
        for layout, errs in res.items():
            assert errs[0] <= 1e-5 and max(errs[1:]) <= 1e-4, (r, layout, errs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_drives_two_devices_and_keeps_its_current_device():
    """Every kernel family on cuda:0 and then on cuda:1 from one process: the opt-in to large dynamic
    shared memory is a per-device attribute, and a call naming another device must leave the caller's
    current device as it found it."""
    import torch_neuronx_b200 as T
    from oracle import sdpa_oracle as O
    from tests.util import make_qkv

    q, k, v = make_qkv(3, 1, 8, 2, 300, 300, 128, torch.bfloat16)
    go = torch.randn(q.shape, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16)
    ref_o, ref_l = O.sdpa_forward(q, k, v, is_causal=True, compute_dtype=torch.float32)
    torch.cuda.set_device(0)
    for index in (0, 1):
        dev = torch.device("cuda", index)
        T.reset_launch_counts()
        out, lse = T.sdpa_forward(q.to(dev), k.to(dev), v.to(dev), is_causal=True)
        gq, gk, gv, _ = T.sdpa_backward(go.to(dev), q.to(dev), k.to(dev), v.to(dev), out, lse, is_causal=True)
        torch.cuda.synchronize(dev)
        T.check_device_status()
        assert torch.cuda.current_device() == 0, "a call on another device changed the caller's device"
        counts = T.launch_counts()
        assert counts["prefill"] == 1 and counts["bwd_dq"] == 1 and counts["bwd_dkv"] == 1, counts
        assert (out.cpu().float() - ref_o).abs().max().item() <= 2e-2
        assert (lse.cpu() - ref_l).abs().max().item() <= 1e-3
        want = O.sdpa_backward(go, q, k, v, out.cpu(), lse.cpu(), is_causal=True, compute_dtype=torch.float32)
        for got, ref in zip((gq, gk, gv), want[:3]):
            torch.testing.assert_close(got.cpu().float(), ref, rtol=5e-2, atol=2e-2)


def _long_context_worker(rank, world, port, out_dir):
    """Configuration 5 at its own size (one causal 131072-token sequence) over two ranks: forward and backward
    of the ring, then the sampled-row check the benchmark also runs (independent CUDA-core kernels on the
    all-gathered tensors, a few rows on the CPU oracle, the negative guard)."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import math

    import torch.distributed as dist

    import bench
    import torch_neuronx_b200 as T
    from torch_neuronx_b200 import _lib, ring as R

    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        S, Hq, Hkv, D = 131072, 64, 8, 128
        n_local = S // world
        g = torch.Generator(device=dev).manual_seed(4000 + rank)
        q = torch.randn(1, Hq, n_local, D, generator=g, device=dev, dtype=torch.bfloat16)
        k = torch.randn(1, Hkv, n_local, D, generator=g, device=dev, dtype=torch.bfloat16)
        v = torch.randn(1, Hkv, n_local, D, generator=g, device=dev, dtype=torch.bfloat16)
        go = torch.randn(q.shape, generator=g, device=dev, dtype=torch.bfloat16)
        scale = 1.0 / math.sqrt(D)
        out, lse = T.ring_attention(q, k, v, is_causal=True, scale=scale, layout="zigzag")
        dq, dk, dv = T.ring_attention_backward(go, q, k, v, out, lse, is_causal=True, scale=scale, layout="zigzag")
        torch.cuda.synchronize()
        T.check_device_status()
        res = bench.ring_check(T, R, _lib, dist, dev, rank, world, "zigzag", q, k, v, go, out, lse, dq, dk, dv, scale,
                               True)
        torch.save(res, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_long_context_ring_at_full_size_on_two_gpus(tmp_path):
    import torch.multiprocessing as mp

    mp.spawn(_long_context_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(tmp_path / f"r{r}.pt")
        assert res["ok"], res
        assert res["max_abs_out"] <= 2e-2 and res["max_abs_lse"] <= 1e-3 and res["guard_diff"] > 0.1, res
        assert res["max_abs_out_cpu"] <= 2e-2 and res["max_abs_lse_cpu"] <= 1e-3, res
