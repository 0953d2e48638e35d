"""The launches are plain stream work: they can be captured into a CUDA graph and replayed, which is how
a serving loop runs its decode steps.  Replays must follow new data in the captured buffers."""

import pytest
import torch

from oracle import sdpa_oracle as O
from tests.util import check_against_oracle

pytestmark = pytest.mark.gpu


def test_prefill_and_decode_replay_from_a_cuda_graph():
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(23)
    # static buffers a graph works on
    q = torch.zeros(2, 8, 256, 128, dtype=torch.bfloat16, device=dev)
    k = torch.zeros(2, 2, 256, 128, dtype=torch.bfloat16, device=dev)
    v = torch.zeros_like(k)
    q1 = torch.zeros(2, 8, 1, 128, dtype=torch.bfloat16, device=dev)
    lens = torch.tensor([256, 100], dtype=torch.int32, device=dev)
    out, lse = torch.empty_like(q), torch.empty(2, 8, 256, device=dev)
    out1, lse1 = torch.empty_like(q1), torch.empty(2, 8, 1, device=dev)

    def work():
        T.sdpa_forward(q, k, v, is_causal=True, kv_lens=lens, out=out, lse=lse)
        T.sdpa_forward(q1, k, v, kv_lens=lens, out=out1, lse=lse1)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):      # warm-up outside the capture (scratch buffers, first-use set-up)
        work()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        work()
    for trial in range(2):             # new data in the same buffers, replay, compare
        hq = torch.randn(2, 8, 256, 128, generator=g).to(torch.bfloat16)
        hk = torch.randn(2, 2, 256, 128, generator=g).to(torch.bfloat16)
        hv = torch.randn(2, 2, 256, 128, generator=g).to(torch.bfloat16)
        hq1 = torch.randn(2, 8, 1, 128, generator=g).to(torch.bfloat16)
        hl = torch.tensor([256, 100 + 50 * trial], dtype=torch.int32)
        q.copy_(hq), k.copy_(hk), v.copy_(hv), q1.copy_(hq1), lens.copy_(hl)
        out.fill_(float("nan")), out1.fill_(float("nan"))
        T.reset_launch_counts()
        graph.replay()
        torch.cuda.synchronize()
        T.check_device_status()
        assert sum(T.launch_counts().values()) == 0      # nothing was launched from the host: the graph did the work
        check_against_oracle(hq, hk, hv, out.cpu(), lse.cpu(), is_causal=True, kv_lens=hl, tag=f"graph prefill {trial}")
        check_against_oracle(hq1, hk, hv, out1.cpu(), lse1.cpu(), kv_lens=hl, tag=f"graph decode {trial}")


def test_generation_steps_replay_from_a_cuda_graph():
    """decode_append captured once; each replay appends the row found in the static k_new / v_new buffers and
    the lengths travel between replays through a device-side copy."""
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(29)
    B, Hq, Hkv, D, S = 2, 8, 2, 128, 128
    k_full = torch.randn(B, Hkv, S, D, generator=g).to(torch.bfloat16)
    v_full = torch.randn(B, Hkv, S, D, generator=g).to(torch.bfloat16)
    kc = torch.zeros(B, Hkv, S, D, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    start = [5, 40]
    for b in range(B):
        kc[b, :, :start[b]] = k_full[b, :, :start[b]].to(dev)
        vc[b, :, :start[b]] = v_full[b, :, :start[b]].to(dev)
    lens = torch.tensor(start, dtype=torch.int32, device=dev)
    q = torch.zeros(B, Hq, 1, D, dtype=torch.bfloat16, device=dev)
    kn = torch.zeros(B, Hkv, D, dtype=torch.bfloat16, device=dev)
    vn = torch.zeros_like(kn)
    holder = {}

    def step():
        o, l, new = T.decode_append(q, kn, vn, kc, vc, lens, need_lse=True)
        lens.copy_(new)                      # ordered after the kernels on the same stream
        holder["out"], holder["lse"] = o, l

    # warm-up on copies of the state so that the captured run starts from the same point
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    saved = (kc.clone(), vc.clone(), lens.clone())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    kc.copy_(saved[0]), vc.copy_(saved[1]), lens.copy_(saved[2])
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    kc.copy_(saved[0]), vc.copy_(saved[1]), lens.copy_(saved[2])   # capture does not execute; be explicit anyway
    cur = list(start)
    for _ in range(4):
        hq = torch.randn(B, Hq, 1, D, generator=g).to(torch.bfloat16)
        q.copy_(hq)
        kn.copy_(torch.stack([k_full[b, :, cur[b]] for b in range(B)]))
        vn.copy_(torch.stack([v_full[b, :, cur[b]] for b in range(B)]))
        graph.replay()
        torch.cuda.synchronize()
        cur = [c + 1 for c in cur]
        assert lens.tolist() == cur
        check_against_oracle(hq, k_full, v_full, holder["out"].cpu(), holder["lse"].cpu(),
                             kv_lens=torch.tensor(cur, dtype=torch.int32), tag="graphed generation step")
    for b in range(B):
        assert torch.equal(kc[b, :, :cur[b]].cpu(), k_full[b, :, :cur[b]])
