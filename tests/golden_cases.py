"""Rebuild the inputs of the committed golden cases.

The fixture file keeps inputs only for tiny cases; the rest are regenerated
from the seed with the same draw order as ``tests/golden/make_golden.py`` and
checked against the stored checksum.
"""

import torch


def _checksum(*tensors):
    return float(sum(t.double().sum().item() for t in tensors))


def inputs_for(name, case):
    """Return ``(q, k, v, mask)`` for one golden case."""
    if "q" in case:
        return case["q"], case["k"], case["v"], case.get("mask")
    if name.startswith("small_"):
        g = torch.Generator().manual_seed(case["seed"])
        dtype, lq, lk = case["dtype"], case["lq"], case["lk"]
        q = torch.randn(2, 2, lq, 48, generator=g).to(dtype)
        k = torch.randn(2, 2, lk, 48, generator=g).to(dtype)
        v = torch.randn(2, 2, lk, 48, generator=g).to(dtype)
        mask = None
        if case["mask_kind"] == "float":
            mask = torch.randn(2, 1, lq, lk, generator=g).to(dtype)
        elif case["mask_kind"] == "bool":
            mask = torch.rand(2, 1, lq, lk, generator=g) > 0.3
            mask[..., 0] = True
    elif name.startswith("saturated_"):
        torch.manual_seed(case["seed"])
        sat = case["sat"]
        q = (torch.randn(1, 4, 512, 128) * sat).to(torch.bfloat16)
        k = (torch.randn(1, 4, 512, 128) * sat).to(torch.bfloat16)
        v = torch.randn(1, 4, 512, 128).to(torch.bfloat16)
        mask = None
    elif name == "config1_fp32":
        g = torch.Generator().manual_seed(case["seed"])
        q = torch.randn(2, 8, 512, 64, generator=g)
        k = torch.randn(2, 8, 512, 64, generator=g)
        v = torch.randn(2, 8, 512, 64, generator=g)
        mask = None
    else:
        raise KeyError(name)
    got = _checksum(q, k, v)
    assert abs(got - case["input_sum"]) <= 1e-9 * max(1.0, abs(case["input_sum"])), (
        f"{name}: seeded inputs differ from the ones the fixture was made with"
    )
    return q, k, v, mask


def expected_for(name, case, out, lse):
    """Pair up (actual, expected) tensors: full outputs or the stored row subsample."""
    pairs = [(lse, case["lse"])]
    if "out" in case:
        pairs.append((out, case["out"]))
    else:
        step = 64 if name.startswith("saturated_") else 37
        pairs.append((out[:, :, ::step], case["out_rows"]))
    return pairs


def backward_inputs_for(name, case):
    """Return ``(q, k, v, mask, grad_out)`` for one case of the backward fixture."""
    if "q" in case:
        return case["q"], case["k"], case["v"], case.get("mask"), case["grad_out"]
    g = torch.Generator().manual_seed(case["seed"])
    dtype = case["dtype"]
    if name.startswith("small_"):
        lq, lk = case["lq"], case["lk"]
        q = torch.randn(2, 2, lq, 48, generator=g).to(dtype)
        k = torch.randn(2, 2, lk, 48, generator=g).to(dtype)
        v = torch.randn(2, 2, lk, 48, generator=g).to(dtype)
        mask = None
        if case["mask_kind"] == "float":
            mask = torch.randn(2, 1, lq, lk, generator=g).to(dtype)
        elif case["mask_kind"] == "bool":
            mask = torch.rand(2, 1, lq, lk, generator=g) > 0.3
            mask[..., 0] = True
        go = torch.randn(2, 2, lq, 48, generator=g).to(dtype)
    elif name.startswith("gqa_"):
        q = torch.randn(1, case["hq"], 40, 64, generator=g).to(dtype)
        k = torch.randn(1, case["hkv"], 77, 64, generator=g).to(dtype)
        v = torch.randn(1, case["hkv"], 77, 64, generator=g).to(dtype)
        go = torch.randn(1, case["hq"], 40, 64, generator=g).to(dtype)
        mask = None
    else:
        raise KeyError(name)
    got = _checksum(q, k, v, go)
    assert abs(got - case["input_sum"]) <= 1e-9 * max(1.0, abs(case["input_sum"])), (
        f"{name}: seeded inputs differ from the ones the fixture was made with"
    )
    return q, k, v, mask, go
