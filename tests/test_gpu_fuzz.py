"""Seeded random shapes through the automatic kernel choice: forward (and, for a third of the cases,
backward) against the oracle.  The draw covers grouped heads, ragged tile tails, right padding, both
storage orders, the head dimensions of every kernel family and the three dtypes."""

import random

import pytest
import torch

from oracle import sdpa_oracle as O
from tests.util import check_against_oracle

pytestmark = pytest.mark.gpu

HEAD_DIMS = [(64, 64), (128, 128), (192, 128), (256, 256), (32, 32), (80, 80), (16, 48)]


def _case(seed):
    rng = random.Random(seed)
    e, dv = rng.choice(HEAD_DIMS)
    group = rng.choice([1, 1, 2, 4, 8])
    hkv = rng.choice([1, 2, 3])
    return dict(
        B=rng.choice([1, 2, 3]), Hq=hkv * group, Hkv=hkv, L=rng.choice([1, 7, 64, 129, 200, 333]),
        S=rng.choice([1, 50, 128, 257, 400]), E=e, Dv=dv, dtype=rng.choice([torch.bfloat16, torch.float16, torch.float32]),
        causal=rng.random() < 0.5, lens=rng.random() < 0.5, bshd=rng.random() < 0.3, backward=seed % 3 == 0,
    )


@pytest.mark.parametrize("seed", range(120))
def test_random_shapes_match_the_oracle(seed):
    import torch_neuronx_b200 as T

    c = _case(seed)
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(1000 + seed)
    q = torch.randn(c["B"], c["Hq"], c["L"], c["E"], generator=g).to(c["dtype"])
    k = torch.randn(c["B"], c["Hkv"], c["S"], c["E"], generator=g).to(c["dtype"])
    v = torch.randn(c["B"], c["Hkv"], c["S"], c["Dv"], generator=g).to(c["dtype"])
    lens = torch.randint(0, c["S"] + 1, (c["B"],), generator=g).to(torch.int32) if c["lens"] else None

    def put(t):
        t = t.to(dev)
        return t.transpose(1, 2).contiguous().transpose(1, 2) if c["bshd"] else t

    qd, kd, vd = put(q), put(k), put(v)
    ld = lens.to(dev) if lens is not None else None
    out, lse = T.sdpa_forward(qd, kd, vd, is_causal=c["causal"], kv_lens=ld)
    torch.cuda.synchronize()
    T.check_device_status()
    check_against_oracle(q, k, v, out.cpu(), lse.cpu(), is_causal=c["causal"], kv_lens=lens, tag=str(c))
    if not c["backward"] or c["E"] > 256 or c["Dv"] > 256:
        return
    go = torch.randn(c["B"], c["Hq"], c["L"], c["Dv"], generator=g).to(c["dtype"])
    gq, gk, gv, _ = T.sdpa_backward(put(go), qd, kd, vd, out, lse, is_causal=c["causal"], kv_lens=ld)
    torch.cuda.synchronize()
    T.check_device_status()
    want = O.sdpa_backward(go, q, k, v, out.cpu(), lse.cpu(), is_causal=c["causal"], kv_lens=lens,
                           compute_dtype=torch.float32)
    tol = dict(rtol=1e-4, atol=1e-5) if c["dtype"] == torch.float32 else dict(rtol=5e-2, atol=2e-2)
    for got, ref, n in zip((gq, gk, gv), want[:3], ("dq", "dk", "dv")):
        assert not torch.isnan(got.float()).any(), f"{n} {c}"
        torch.testing.assert_close(got.cpu().float(), ref.float(), msg=lambda m: f"{n} {c}: {m}", **tol)
