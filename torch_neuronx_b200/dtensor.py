"""DTensor integration of the fused-attention ops: sharding strategies and the
context-parallel (ring) handler.

Upstream registers four placements for the forward and backward overrideable ops --
replicated, head-sharded, batch-sharded, sequence-sharded
(``torch_neuronx/distributed/tensor/register_sharding.py:49-186,189-420``) -- and puts a
ring handler for the two ops into torch's context-parallel dispatch table so that
``context_parallel(...)`` reaches it (``distributed/tensor/cp_ring_handler.py:460-534``).
The same two steps here, for CUDA tensors:

* :func:`register_sharding_strategies` -- replicated / head / batch placements.  These
  need no exchange: every rank runs the kernel on its own heads or batches.
* :func:`install_context_parallel_handler` -- adds the sequence placement and routes the
  two ops, while torch's context-parallel dispatcher is enabled, to
  :func:`ring.ring_attention` / :func:`ring.ring_attention_backward`.  The sequence
  placement is only correct together with the ring (a rank that attended to its own
  chunk alone would be wrong, not slow), which is why it is installed here and not with
  the other three.

Nothing here computes: placements are host logic and the ring driver launches the
kernels.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch

from . import ring

aten = torch.ops.aten
FWD_OP = aten._scaled_dot_product_fused_attention_overrideable.default
BWD_OP = aten._scaled_dot_product_fused_attention_overrideable_backward.default

_sequence_placement = False   # set by install_context_parallel_handler()
_registered = False
_block_functions: dict = {}   # optional replacements of the per-block compute (CPU tests)
_layout_override: Optional[str] = None


def _tensor_slot(schema_args, idx) -> bool:
    from torch.distributed.tensor._op_schema import OpStrategy

    return idx < len(schema_args) and isinstance(schema_args[idx], OpStrategy)


def _placements():
    from torch.distributed.tensor.placement_types import Replicate, Shard

    rows = [Replicate(), Shard(1), Shard(0)]   # nothing / heads / batch
    if _sequence_placement:
        rows.append(Shard(2))
    return rows


def _forward_strategy(op_schema):
    """Outputs ``(out, lse, cum_seq_q, cum_seq_k, max_q, max_k, philox_seed, philox_offset,
    debug_mask)`` then the tensor inputs ``q, k, v[, attn_bias]``: out and lse follow the
    placement of q/k/v (lse is ``(B, Hq, L)``, the same first three dimensions)."""
    from torch.distributed.tensor._ops.utils import expand_to_full_mesh_op_strategy
    from torch.distributed.tensor.placement_types import Replicate

    args = op_schema.args_schema
    has_bias = _tensor_slot(args, 3)
    debug = len(args) > 6 and bool(args[6])
    table = []
    for p in _placements():
        row = [p, p, None, None, None, None, Replicate(), Replicate(), p if debug else None, p, p, p]
        if has_bias:
            row.append(p)
        table.append(row)
    return expand_to_full_mesh_op_strategy(op_schema.get_mesh_from_args(), op_schema, table, input_index=9)


def _backward_strategy(op_schema):
    """Outputs ``(grad_q, grad_k, grad_v, grad_bias)`` then every tensor input in schema
    order: grad_out, q, k, v, [attn_bias], out, lse, [cum_seq_q, cum_seq_k], [philox_seed,
    philox_offset] -- the bracketed ones only when they arrive as tensors."""
    from torch.distributed.tensor._ops.utils import expand_to_full_mesh_op_strategy
    from torch.distributed.tensor.placement_types import Replicate

    args = op_schema.args_schema
    has_bias = _tensor_slot(args, 4)
    table = []
    for p in _placements():
        row = [p, p, p, p if has_bias else None]                # gradients
        row += [p, p, p, p]                                     # grad_out, q, k, v
        if has_bias:
            row.append(p)
        row += [p, p]                                           # out, lse
        row += [Replicate() for i in (8, 9, 14, 15) if _tensor_slot(args, i)]
        table.append(row)
    return expand_to_full_mesh_op_strategy(op_schema.get_mesh_from_args(validate=False), op_schema, table,
                                           input_index=4)


def register_sharding_strategies() -> None:
    """Register (or refresh) the placements of the two ops with DTensor."""
    global _registered
    from torch.distributed.tensor._op_schema import RuntimeSchemaInfo
    from torch.distributed.tensor._ops.utils import register_op_strategy

    register_op_strategy(FWD_OP, schema_info=RuntimeSchemaInfo(4))(_forward_strategy)
    register_op_strategy(BWD_OP)(_backward_strategy)
    _registered = True


# ----------------------------------------------------------------------------
# context parallel
# ----------------------------------------------------------------------------


def set_block_functions(attn_fn: Optional[Callable] = None, merge_fn: Optional[Callable] = None,
                        bwd_fn: Optional[Callable] = None) -> None:
    """Replace the per-block compute of the ring driver (``None`` = the CUDA kernels).
    Exists so the orchestration can be exercised among CPU ranks."""
    _block_functions.clear()
    for name, fn in (("attn_fn", attn_fn), ("merge_fn", merge_fn), ("bwd_fn", bwd_fn)):
        if fn is not None:
            _block_functions[name] = fn


def set_sequence_layout(layout: Optional[str]) -> None:
    """Force ``ring.ZIGZAG`` or ``ring.CONTIGUOUS``; ``None`` follows torch's
    context-parallel load-balancing option."""
    global _layout_override
    _layout_override = layout


def _sequence_layout() -> str:
    if _layout_override is not None:
        return _layout_override
    try:
        from torch.distributed.tensor.experimental._context_parallel import _attention as cp

        balanced = bool(getattr(cp._cp_options, "enable_load_balance", False))
    except (ImportError, AttributeError):
        balanced = False
    # torch's head-tail balancer gives rank r chunks r and 2N-1-r: the zigzag placement
    return ring.ZIGZAG if balanced else ring.CONTIGUOUS


def _ring_forward(mesh, query, key, value, attn_bias=None, dropout_p=0.0, is_causal=False, return_debug_mask=False,
                  *, scale=None):
    if attn_bias is not None and attn_bias.numel() != 0:
        raise NotImplementedError("context-parallel attention takes no attn_bias; use is_causal")
    if dropout_p != 0.0 or return_debug_mask:
        raise NotImplementedError("context-parallel attention supports neither dropout nor a debug mask")
    kw = {k: v for k, v in _block_functions.items() if k in ("attn_fn", "merge_fn")}
    out, lse = ring.ring_attention(query, key, value, group=mesh.get_group(), is_causal=is_causal, scale=scale,
                                   layout=_sequence_layout(), **kw)
    zero = torch.zeros((), dtype=torch.int32, device=query.device)
    return out, lse, None, None, query.shape[2], key.shape[2], zero, zero, None


def _ring_backward(mesh, grad_out, query, key, value, attn_bias, grad_input_mask, out, logsumexp, cum_seq_q,
                   cum_seq_k, max_q, max_k, dropout_p, is_causal, philox_seed, philox_offset, *, scale=None):
    if attn_bias is not None and attn_bias.numel() != 0:
        raise NotImplementedError("context-parallel attention takes no attn_bias; use is_causal")
    if dropout_p != 0.0:
        raise NotImplementedError("context-parallel attention supports no dropout")
    kw = {k: v for k, v in _block_functions.items() if k == "bwd_fn"}
    gq, gk, gv = ring.ring_attention_backward(grad_out, query, key, value, out, logsumexp, group=mesh.get_group(),
                                              is_causal=is_causal, scale=scale, layout=_sequence_layout(), **kw)
    return gq, gk, gv, None


def _context_parallel_handler(op_call, args, kwargs):
    """Custom DTensor handler for the two ops while context parallelism is enabled: the
    inputs must already be sequence-sharded (a redistribution would defeat the ring), the
    local shards go to the ring driver, the results are wrapped with the propagated
    placements."""
    from torch.distributed.tensor import DTensor

    dispatcher = DTensor._op_dispatcher
    op_info = dispatcher.unwrap_to_op_info(op_call, args, kwargs)
    dispatcher.sharding_propagator.propagate(op_info)
    sharding = op_info.output_sharding
    if sharding is None:
        raise RuntimeError(f"context-parallel handler: no output sharding for {op_call}")
    if sharding.needs_redistribute:
        raise RuntimeError("context-parallel handler: q, k and v must already be sharded on the sequence dimension")
    fn = _ring_forward if op_call is FWD_OP else _ring_backward
    local = fn(op_info.compute_mesh, *op_info.local_args, **op_info.local_kwargs)
    return dispatcher.wrap(local, sharding.output_spec)


def install_context_parallel_handler() -> bool:
    """Add the sequence placement and put the ring handler into torch's context-parallel
    dispatch table.  Returns False (and changes nothing) when torch's private
    context-parallel module is not where this build expects it."""
    global _sequence_placement
    try:
        from torch.distributed.tensor.experimental._context_parallel import _attention as cp

        table = cp.custom_ops
    except (ImportError, AttributeError):
        return False
    _sequence_placement = True
    register_sharding_strategies()
    table[FWD_OP] = _context_parallel_handler
    table[BWD_OP] = _context_parallel_handler
    return True
