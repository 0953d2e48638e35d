"""CPU oracle for the fused scaled-dot-product-attention forward and backward.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package may import this
module; it exists so that the parity tests, the smoke check and the CPU leg of
the benchmark have an independent statement of what the CUDA path must
produce.

Parity status: PINNED.  ``tests/golden/`` holds outputs produced by the
upstream file ``torch_neuronx/_sdpa_math.py`` (``compute_attention`` and
``compute_attention_backward``) and ``tests/test_oracle_golden.py`` requires
this restatement to reproduce them bit for bit on the same seeded inputs.

What is restated, and where it lives upstream:

* ``torch_neuronx/_sdpa_math.py:51-95`` ``compute_attention`` -- accumulate in
  fp32 for half inputs, ``logits = q @ k^T * scale``, causal mask (top-left
  aligned lower triangle, ``:15-28``), additive bias after the causal mask
  (``:30-31``), row max with a guard for rows without any visible key
  (``:85-91``), ``lse = max + log(sum)``, probabilities rounded to the input
  dtype before the second matmul (``:94``).
* ``torch_neuronx/_sdpa_math.py:98-176`` ``compute_attention_backward`` --
  probabilities rebuilt from the saved log-sum-exp, ``dV = P^T dO``,
  ``dP = dO V^T``, softmax Jacobian, ``dQ = dS K``, ``dK = dS^T Q``.
* ``torch_neuronx/neuron_dynamo_backend/decompositions.py:2083-2128`` --
  how the op drives that function: grouped-query heads expanded with
  ``repeat_interleave`` (``:2088-2091``), default scale ``1/sqrt(E)``
  (``:2094-2095``), boolean masks turned into ``0 / -inf`` additive biases in
  the query dtype (``:2101-2102``).

Extensions that the upstream function does not have but the kernels do are
expressed through those same primitives, so the oracle never grows new
arithmetic: per-batch valid key lengths become a ``[B,1,1,S]`` ``0/-inf``
bias, and global row/key offsets (used by ring blocks) become a ``[L,S]``
``0/-inf`` bias with ``is_causal=False``.
"""

from __future__ import annotations

import math

import torch

NEG_INF = float("-inf")


def accumulator_dtype(dtype: torch.dtype) -> torch.dtype:
    """fp16/bf16 inputs accumulate in fp32, everything else in its own type
    (``_sdpa_math.py:6-7``)."""
    if dtype in (torch.float16, torch.bfloat16):
        return torch.float32
    return dtype


def masked_logits(scores: torch.Tensor, bias: torch.Tensor | None, causal: bool) -> torch.Tensor:
    """Apply the causal triangle first and the additive bias second
    (``_sdpa_math.py:15-33``).  The triangle is anchored at the top-left
    corner: query row ``i`` sees keys ``j <= i`` whatever the two lengths."""
    if causal:
        n_q, n_k = scores.shape[-2], scores.shape[-1]
        rows = torch.arange(n_q).unsqueeze(-1)
        cols = torch.arange(n_k).unsqueeze(0)
        scores = scores.masked_fill(cols > rows, NEG_INF)
    if bias is not None and bias.numel() > 0:
        scores = scores + bias
    return scores


def attention_core(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    bias: torch.Tensor | None,
    scale: float,
    causal: bool,
) -> tuple[torch.Tensor, torch.Tensor]:
    """The forward arithmetic of ``compute_attention`` at ``dropout_p == 0``
    (``_sdpa_math.py:79-95``); k and v already carry as many heads as q.

    Returns ``(out, lse)`` with ``out`` in q's dtype and ``lse`` in fp32.
    """
    in_dtype = q.dtype
    acc = accumulator_dtype(in_dtype)
    scores = torch.matmul(q.to(acc), k.to(acc).transpose(-2, -1))
    scores = masked_logits(scores * scale, bias, causal)

    row_max = scores.amax(dim=-1, keepdim=True)
    dead = row_max == NEG_INF  # rows that see no key at all
    shift = torch.where(dead, 0.0, row_max)
    weights = torch.exp(scores - shift)
    denom = weights.sum(dim=-1, keepdim=True)
    lse = row_max.squeeze(-1) + torch.log(denom.squeeze(-1))
    denom = torch.where(dead, 1.0, denom)
    probs = weights / denom
    out = torch.matmul(probs.to(in_dtype), v)
    return out, lse.to(torch.float32)


def expand_kv_heads(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
    """Grouped-query layout: query head ``h`` reads kv head ``h // group``
    (``decompositions.py:2088-2091``)."""
    hq, hkv = q.shape[1], k.shape[1]
    if hq != hkv:
        if hkv == 0 or hq % hkv != 0:
            raise RuntimeError(
                "Number of heads in key and value must divide the number of heads in query"
            )
        g = hq // hkv
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
    return k, v


def additive_bias(mask: torch.Tensor | None, like: torch.Tensor) -> torch.Tensor | None:
    """``None`` stays absent, a boolean mask (True = keep) becomes ``0/-inf``
    in the query dtype, anything else is taken as an additive bias
    (``decompositions.py:2099-2104``)."""
    if mask is None:
        return None
    if mask.dtype == torch.bool:
        return torch.where(mask, 0.0, NEG_INF).to(like.dtype)
    return mask


def key_length_bias(kv_lens: torch.Tensor, n_keys: int, dtype: torch.dtype) -> torch.Tensor:
    """Right padding: batch ``b`` sees keys ``j < kv_lens[b]`` -> ``[B,1,1,S]``."""
    cols = torch.arange(n_keys).view(1, 1, 1, n_keys)
    keep = cols < kv_lens.view(-1, 1, 1, 1).to(torch.int64)
    return torch.where(keep, 0.0, NEG_INF).to(dtype)


def offset_causal_bias(n_q: int, n_k: int, q_offset: int, k_offset: int, dtype) -> torch.Tensor:
    """Causal predicate between blocks of a longer sequence: query row ``i``
    (global position ``q_offset + i``) sees key ``j`` iff
    ``k_offset + j <= q_offset + i``."""
    rows = torch.arange(n_q).unsqueeze(-1) + q_offset
    cols = torch.arange(n_k).unsqueeze(0) + k_offset
    return torch.where(cols <= rows, 0.0, NEG_INF).to(dtype)


def sdpa_forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    attn_mask: torch.Tensor | None = None,
    is_causal: bool = False,
    scale: float | None = None,
    kv_lens: torch.Tensor | None = None,
    q_offset: int = 0,
    k_offset: int = 0,
    compute_dtype: torch.dtype | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """The op as the upstream decomposition drives it, plus the two kernel
    extensions (``kv_lens`` and block offsets).

    ``compute_dtype=torch.float32`` upcasts q, k and v first: that is the
    "fp32 reference" the half-precision tolerances are stated against.
    """
    if compute_dtype is not None:
        q, k, v = q.to(compute_dtype), k.to(compute_dtype), v.to(compute_dtype)
        if attn_mask is not None and attn_mask.dtype != torch.bool:
            attn_mask = attn_mask.to(compute_dtype)
    n_q, n_k, e = q.shape[2], k.shape[2], q.shape[3]
    if scale is None:
        scale = 1.0 / math.sqrt(e)
    k, v = expand_kv_heads(q, k, v)

    bias = additive_bias(attn_mask, q)
    if kv_lens is not None:
        pad = key_length_bias(kv_lens.cpu(), n_k, q.dtype)
        bias = pad if bias is None else bias + pad
    causal = bool(is_causal)
    if causal and (q_offset != 0 or k_offset != 0):
        tri = offset_causal_bias(n_q, n_k, q_offset, k_offset, q.dtype)
        bias = tri if bias is None else bias + tri
        causal = False
    return attention_core(q, k, v, bias, float(scale), causal)


def sdpa_forward_chunked(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    is_causal: bool = False,
    scale: float | None = None,
    kv_lens: torch.Tensor | None = None,
    rows_per_chunk: int = 1024,
    compute_dtype: torch.dtype | None = None,
    row_slices: list[tuple[int, int]] | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Same result as :func:`sdpa_forward` without ever holding the full
    ``[L,S]`` score matrix: one (batch, kv head) group and one block of query
    rows at a time, the causal rule carried by the row offset.

    With ``row_slices`` only those ``[r0, r1)`` row ranges are evaluated (the
    rest of ``out`` / ``lse`` stays NaN) -- the sampled check used for shapes
    whose full oracle would take minutes.
    """
    b_, hq, n_q, _ = q.shape
    hkv, n_k, dv = k.shape[1], k.shape[2], v.shape[3]
    g = hq // hkv
    out_dtype = compute_dtype or q.dtype
    out = torch.full((b_, hq, n_q, dv), float("nan"), dtype=out_dtype)
    lse = torch.full((b_, hq, n_q), float("nan"), dtype=torch.float32)
    if row_slices is None:
        row_slices = [(r, min(r + rows_per_chunk, n_q)) for r in range(0, n_q, rows_per_chunk)]
    for b in range(b_):
        for h in range(hkv):
            qs = q[b : b + 1, h * g : (h + 1) * g]
            for r0, r1 in row_slices:
                k_hi = min(n_k, r1) if is_causal else n_k
                lens = None if kv_lens is None else kv_lens[b : b + 1].clamp(max=k_hi)
                o, l = sdpa_forward(
                    qs[:, :, r0:r1],
                    k[b : b + 1, h : h + 1, :k_hi],
                    v[b : b + 1, h : h + 1, :k_hi],
                    is_causal=is_causal,
                    scale=scale,
                    kv_lens=lens,
                    q_offset=r0,
                    k_offset=0,
                    compute_dtype=compute_dtype,
                )
                out[b, h * g : (h + 1) * g, r0:r1] = o[0]
                lse[b, h * g : (h + 1) * g, r0:r1] = l[0]
    return out, lse


def merge_partials(out_a, lse_a, out_b, lse_b):
    """Combine two attention results over disjoint key sets for the same
    queries: ``lse = logaddexp(lse_a, lse_b)`` and outputs weighted by
    ``exp(lse_x - lse)``, all in fp32.  Rows dead on both sides stay
    ``(0, -inf)``."""
    lse_a = lse_a.float()
    lse_b = lse_b.float()
    lse = torch.logaddexp(lse_a, lse_b)
    dead = lse == NEG_INF
    wa = torch.where(dead, 0.0, torch.exp(lse_a - torch.where(dead, 0.0, lse)))
    wb = torch.where(dead, 0.0, torch.exp(lse_b - torch.where(dead, 0.0, lse)))
    out = out_a.float() * wa.unsqueeze(-1) + out_b.float() * wb.unsqueeze(-1)
    return out, lse


def attention_backward_core(
    grad_out: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    lse: torch.Tensor,
    bias: torch.Tensor | None,
    scale: float,
    causal: bool,
):
    """The backward arithmetic of ``compute_attention_backward`` at ``dropout_p == 0``
    (``_sdpa_math.py:130-176``); k and v already carry as many heads as q.

    Probabilities are rebuilt from the forward's log-sum-exp (rows whose lse is -inf
    get zero probabilities), ``dV = P^T dO``, ``dP = dO V^T``, and the softmax
    Jacobian is applied with the row term ``sum_j dP_j P_j + sum_d dO_d (out_d -
    (P V)_d)`` -- which is ``sum_d dO_d out_d`` with the forward's own ``out``.
    Returns ``(dq, dk, dv, dbias)`` in the input dtype; ``dbias`` is the gradient
    of the logits, ``[B,H,L,S]`` without any reduction over broadcast bias
    dimensions, or ``None`` when no bias took part (``:169``).
    """
    in_dtype = q.dtype
    acc = accumulator_dtype(in_dtype)
    g, qa, ka, va, oa = (t.to(acc) for t in (grad_out, q, k, v, out))
    la = lse.to(acc)
    if bias is not None and bias.numel() > 1:
        bias = bias.to(acc)
    else:
        bias = None
    scores = masked_logits(torch.matmul(qa, ka.transpose(-2, -1)) * scale, bias, causal)
    dead = la == NEG_INF
    probs = torch.exp(scores - torch.where(dead, 0.0, la).unsqueeze(-1))
    probs = torch.where(dead.unsqueeze(-1), 0.0, probs)
    dv = torch.matmul(probs.transpose(-2, -1), g)
    dp = torch.matmul(g, va.transpose(-2, -1))
    row = (dp * probs).sum(dim=-1, keepdim=True) + (g * (oa - torch.matmul(probs, va))).sum(dim=-1, keepdim=True)
    dlogits = probs * (dp - row)
    ds = dlogits * scale
    dq = torch.matmul(ds, ka)
    dk = torch.matmul(ds.transpose(-2, -1), qa)
    dbias = dlogits.to(in_dtype) if bias is not None else None
    return dq.to(in_dtype), dk.to(in_dtype), dv.to(in_dtype), dbias


def sdpa_backward(
    grad_out, q, k, v, out, lse, attn_mask=None, is_causal=False, scale=None, kv_lens=None,
    compute_dtype: torch.dtype | None = None,
):
    """Backward of :func:`sdpa_forward` the way upstream drives it: grouped heads are
    expanded before the math and the key/value gradients of a group are summed back
    in the gradient dtype (``_prepare_backward_inputs`` / ``_reduce_gqa_gradients``,
    ``neuron_dynamo_backend/decompositions.py:2535-2598``)."""
    if compute_dtype is not None:
        grad_out, q, k, v, out = (t.to(compute_dtype) for t in (grad_out, q, k, v, out))
        if attn_mask is not None and attn_mask.dtype != torch.bool:
            attn_mask = attn_mask.to(compute_dtype)
    hq, hkv, n_k, e = q.shape[1], k.shape[1], k.shape[2], q.shape[3]
    if scale is None:
        scale = 1.0 / math.sqrt(e)
    ke, ve = expand_kv_heads(q, k, v)
    bias = additive_bias(attn_mask, q)
    if kv_lens is not None:
        pad = key_length_bias(kv_lens.cpu(), n_k, q.dtype)
        bias = pad if bias is None else bias + pad
    dq, dk, dv, dbias = attention_backward_core(grad_out, q, ke, ve, out, lse, bias, float(scale), bool(is_causal))
    if attn_mask is None or attn_mask.dtype == torch.bool:
        dbias = None
    if hq != hkv:
        g = hq // hkv
        b_, _, s_, _ = dk.shape
        dk = dk.view(b_, hkv, g, s_, dk.shape[-1]).sum(dim=2)
        dv = dv.view(b_, hkv, g, s_, dv.shape[-1]).sum(dim=2)
    return dq, dk, dv, dbias
