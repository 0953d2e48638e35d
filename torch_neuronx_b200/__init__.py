"""B200-native fused scaled-dot-product attention behind torch-neuronx's op API.

Importing the package registers the CUDA implementation of
``aten::_scaled_dot_product_fused_attention_overrideable`` (and of its ``_backward``
companion) and the kernel-level op
``b200_sdpa::fwd``.  Compute needs ``libb200_sdpa.so`` (``python -m
torch_neuronx_b200.build``) and a B200; nothing here falls back to another
implementation.
"""

from . import _lib
from .ops import (
    alloc_like_query,
    check_device_status,
    decode_append,
    enable_sdpa_routing,
    fused_attention_overrideable,
    fused_attention_overrideable_backward,
    merge_partials,
    native_multi_head_attn_mid,
    paged_decode,
    register_aten_override,
    scaled_dot_product_attention,
    scaled_dot_product_attention_backward_kernel,
    scaled_dot_product_attention_kernel,
    set_mask_recognition,
    sdpa_backward,
    sdpa_forward,
    sdpa_forward_accumulate,
)
from .masks import MaskStructure, classify_mask
from .ring import (
    ring_attention,
    ring_attention_backward,
    ring_attention_backward_virtual,
    ring_attention_virtual,
    shard_sequence,
    unshard_sequence,
)
from .sharding import as_units, from_units, local_units, partition_units

register_aten_override()

launch_counts = _lib.launch_counts
reset_launch_counts = _lib.reset_launch_counts

__all__ = [
    "MaskStructure", "alloc_like_query", "as_units", "check_device_status", "classify_mask", "decode_append", "enable_sdpa_routing",
    "from_units", "fused_attention_overrideable", "fused_attention_overrideable_backward", "launch_counts",
    "local_units", "merge_partials", "native_multi_head_attn_mid", "paged_decode", "partition_units", "register_aten_override", "reset_launch_counts",
    "ring_attention", "ring_attention_backward", "ring_attention_backward_virtual", "ring_attention_virtual", "scaled_dot_product_attention",
    "scaled_dot_product_attention_backward_kernel", "scaled_dot_product_attention_kernel", "sdpa_backward",
    "sdpa_forward", "sdpa_forward_accumulate", "set_mask_recognition", "shard_sequence", "unshard_sequence",
]
