"""Partition of independent attention work over GPUs.

Attention is independent per (batch, kv head): upstream declares exactly these
two placements for the op -- ``Shard(0)`` on batch and ``Shard(1)`` on heads for
q, k, v, out and lse (``torch_neuronx/distributed/tensor/register_sharding.py:
111-157``).  Here the flattened (batch x kv head) index space is cut into one
contiguous range per rank, balanced by cost, and each unit keeps its ``Hq/Hkv``
query heads with its kv head so no rank ever needs another rank's K/V.  No
collective is involved.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch


def partition_units(n_units: int, world: int, costs: Optional[Sequence[float]] = None) -> List[Tuple[int, int]]:
    """Contiguous ``[start, end)`` ranges, one per rank.  Without costs the ranges
    differ by at most one unit; with costs each cut is placed where the running
    cost crosses the next multiple of ``total / world``."""
    if world <= 0:
        raise ValueError("world must be positive")
    if costs is None:
        base, extra = divmod(n_units, world)
        out, s = [], 0
        for r in range(world):
            e = s + base + (1 if r < extra else 0)
            out.append((s, e))
            s = e
        return out
    if len(costs) != n_units:
        raise ValueError("one cost per unit expected")
    total = float(sum(costs))
    out, s, run = [], 0, 0.0
    for r in range(world):
        target = total * (r + 1) / world
        e = s
        while e < n_units and (run + costs[e] / 2.0 <= target or e == s) and (n_units - e) > (world - 1 - r):
            run += costs[e]
            e += 1
        if r == world - 1:
            while e < n_units:
                run += costs[e]
                e += 1
        out.append((s, e))
        s = e
    return out


def as_units(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kv_lens: Optional[torch.Tensor] = None):
    """View ``(B,Hq,L,E)``, ``(B,Hkv,S,E)``, ``(B,Hkv,S,Dv)`` as independent units:
    ``(B*Hkv, Hq/Hkv, L, E)``, ``(B*Hkv, 1, S, E)``, ``(B*Hkv, 1, S, Dv)`` plus the
    per-unit key lengths.  Views when the batch and head strides allow, else copies."""
    B, Hq, L, E = q.shape
    Hkv = k.shape[1]
    if Hq % Hkv:
        raise RuntimeError("Number of heads in key and value must divide the number of heads in query")
    g = Hq // Hkv
    qu = q.reshape(B, Hkv, g, L, E).flatten(0, 1)
    ku = k.reshape(B * Hkv, 1, k.shape[2], k.shape[3])
    vu = v.reshape(B * Hkv, 1, v.shape[2], v.shape[3])
    lens = None if kv_lens is None else kv_lens.repeat_interleave(Hkv)
    return qu, ku, vu, lens


def from_units(out_units: torch.Tensor, B: int, Hkv: int) -> torch.Tensor:
    """Inverse of :func:`as_units` for an output ``(B*Hkv, g, L, Dv)`` -> ``(B, Hq, L, Dv)``."""
    n, g, L, Dv = out_units.shape
    return out_units.reshape(B, Hkv, g, L, Dv).reshape(B, Hkv * g, L, Dv)


def local_units(q, k, v, rank: int, world: int, kv_lens=None, costs=None):
    """This rank's share of the (batch x kv head) units and its ``[start, end)``."""
    qu, ku, vu, lens = as_units(q, k, v, kv_lens)
    s, e = partition_units(qu.shape[0], world, costs)[rank]
    return qu[s:e], ku[s:e], vu[s:e], (None if lens is None else lens[s:e]), (s, e)
