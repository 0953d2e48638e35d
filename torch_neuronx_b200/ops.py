"""Operator layer: the fused SDPA forward on B200 behind upstream's op API.

Three entry levels, mirroring upstream:

``scaled_dot_product_attention(...)``
    same keyword arguments as ``torch.nn.functional.scaled_dot_product_attention``;
    what a model calls.

``aten::_scaled_dot_product_fused_attention_overrideable`` (CUDA key)
    the ATen op upstream registers for its device
    (``torch_neuronx/python_ops/__init__.py:86-95``,
    ``torch_neuronx/python_ops/scaled_dot_product_fused_attention.py:458-508``);
    returns the same 9-tuple (``:366-376``).  Argument checks and messages follow
    ``torch_neuronx/csrc/core/dispatch/NeuronDispatcher.cpp:2380-2458`` and
    ``torch_neuronx/python_ops/base.py:1036-1111``.

``b200_sdpa::fwd``
    the kernel-level custom op with the positional signature of
    ``nki_kernels::scaled_dot_product_attention_kernel``
    (``torch_neuronx/python_ops/nki_kernels/scaled_dot_product_attention.py:9-41``)
    plus one optional extension, ``kv_lens`` (valid keys per batch).

All of them end in one foreign call into ``libb200_sdpa.so``.  There is no
fallback: non-CUDA tensors are rejected and a missing library raises.
"""

from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch
import torch.overrides

from . import _lib, masks

_DTYPE_CODE = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}

# ----------------------------------------------------------------------------
# per-device scratch and status words
# ----------------------------------------------------------------------------

_status_words: dict[int, torch.Tensor] = {}
_zero_scalars: dict[int, tuple] = {}
_workspaces: dict[tuple[int, int], torch.Tensor] = {}
_retired_workspaces: list = []
last_plan: dict = {}
last_bwd_plan: dict = {}


def _device_index(t: torch.Tensor) -> int:
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def _status_word(dev: int) -> torch.Tensor:
    """The device's status word (int32[4]); one per device, shared with the C++ operator layer."""
    w = _status_words.get(dev)
    if w is None:
        if _lib.load_ops():
            w = torch.ops.b200_sdpa_native.status_word(dev)
        else:
            w = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", dev))
        _status_words[dev] = w
    return w


def _philox_zeros(dev: int):
    """The philox seed / offset slots of the 9-tuple when dropout is off: int32 scalar zeros, as
    upstream returns them (``decompositions.py:2310-2311``).  One pair per device."""
    z = _zero_scalars.get(dev)
    if z is None:
        d = torch.device("cuda", dev)
        z = (torch.zeros((), dtype=torch.int32, device=d), torch.zeros((), dtype=torch.int32, device=d))
        _zero_scalars[dev] = z
    return z


def _workspace(dev: int, nbytes: int) -> torch.Tensor:
    """Scratch for the decode partials and the backward's row statistics.

    Eager calls share one buffer per (device, stream): work on one stream is ordered, so
    reuse across calls is safe.  When a larger request arrives the old buffer is kept alive
    (never handed back to the allocator) because a CUDA graph captured earlier on that
    stream may have its address baked in.  While the stream is being captured the call gets
    a buffer of its own from the graph's pool, and that buffer is not put into the eager
    cache: memory of a graph's private pool must not be reused by eager work."""
    if torch.cuda.is_current_stream_capturing():
        return torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=torch.device("cuda", dev))
    key = (dev, torch.cuda.current_stream(dev).cuda_stream)
    w = _workspaces.get(key)
    if w is None or w.numel() < nbytes:
        if w is not None:
            _retired_workspaces.append(w)
        w = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=torch.device("cuda", dev))
        _workspaces[key] = w
    return w


def release_workspaces() -> None:
    """Drop every cached scratch buffer (also the retired ones).  Only safe when no CUDA graph
    that was captured through this module will be replayed again."""
    _workspaces.clear()
    _retired_workspaces.clear()


def check_device_status(device=None) -> None:
    """Synchronise and raise if any kernel reported a device-side error (a bounded
    wait that gave up).  Cheap enough for tests; not called on the hot path."""
    if device is None:
        devs = list(range(torch.cuda.device_count())) if _lib.load_ops() else list(_status_words)
    else:
        devs = [torch.device(device).index or 0]
    for dev in devs:
        w = _status_word(dev) if _lib.load_ops() else _status_words.get(dev)
        if w is None:
            continue
        vals = w.cpu().tolist()
        if vals[0] != 0:
            w.zero_()
            raise RuntimeError(
                f"b200_sdpa device status {vals[0]} ({_lib.strerror(vals[0])}); role={vals[1]} step={vals[2]} "
                f"extra={vals[3]}"
            )


# ----------------------------------------------------------------------------
# validation (same rules and messages as upstream's dispatcher)
# ----------------------------------------------------------------------------


def _validate(query, key, value, attn_bias, dropout_p, is_causal, return_debug_mask):
    if return_debug_mask:
        raise NotImplementedError("return_debug_mask=True is not supported: the fused kernel keeps no attention matrix")
    if attn_bias is not None and is_causal:
        raise RuntimeError(
            "_scaled_dot_product_fused_attention_overrideable: Explicit attn_mask should not be set when is_causal=True"
        )
    for name, t in (("query", query), ("key", key), ("value", value)):
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{name} must be a Tensor")
    if not (query.device.type == key.device.type == value.device.type):
        raise RuntimeError("Expected query, key, and value to have the same device type")
    if query.dtype not in (torch.float32, torch.float16, torch.bfloat16, torch.float64):
        raise RuntimeError(f"SDPA: query dtype must be float32, float16, or bfloat16, got {query.dtype}")
    if not (query.dtype == key.dtype == value.dtype):
        raise RuntimeError("Expected query, key, and value to have the same dtype")
    if query.dim() != 4 or key.dim() != 4 or value.dim() != 4:
        raise RuntimeError("SDPA: query, key and value must be 4D tensors (B, H, S, D)")
    if not (query.shape[0] == key.shape[0] == value.shape[0]):
        raise RuntimeError("SDPA: batch sizes must match")
    if key.shape[1] != value.shape[1]:
        raise RuntimeError("SDPA: key and value must have the same number of heads")
    if key.shape[2] != value.shape[2]:
        raise RuntimeError("SDPA: key and value must have the same sequence length")
    if query.shape[3] != key.shape[3]:
        raise RuntimeError("SDPA: query and key must have the same embedding dimension")
    if key.shape[1] == 0 or query.shape[1] % key.shape[1] != 0:
        raise RuntimeError("SDPA: Number of heads in key and value must divide the number of heads in query")
    if dropout_p < 0.0 or dropout_p > 1.0:
        raise ValueError(f"dropout_p={dropout_p} is outside [0, 1]. Pass a value in [0, 1].")
    if dropout_p != 0.0:
        raise NotImplementedError("dropout_p != 0 is not supported by the B200 fused attention path")
    if query.device.type != "cuda":
        raise ValueError(f"Expected CUDA device, got {query.device}")
    if not (query.device == key.device == value.device):
        raise RuntimeError("Expected query, key, and value to be on the same device")


def alloc_like_query(query: torch.Tensor, shape) -> torch.Tensor:
    """Output buffer laid out like the query: identical strides when the shapes agree,
    otherwise dense strides in the query's dimension order (the rule of torch's own
    meta kernel for this op, which upstream also follows:
    ``scaled_dot_product_fused_attention.py:357-358``).  The kernels store with these
    strides directly, so no re-layout copy follows."""
    shape = tuple(int(s) for s in shape)
    if tuple(query.shape) == shape:
        return torch.empty_like(query)
    order = sorted(range(4), key=lambda i: query.stride(i), reverse=True)
    permuted = [shape[i] for i in order]
    back = [order.index(i) for i in range(4)]
    return torch.empty(permuted, dtype=query.dtype, device=query.device).permute(back)


def _bias_strides(bias: torch.Tensor, target):
    """Strides of ``bias`` viewed as broadcast to ``target`` (0 where broadcast)."""
    if bias.dim() > 4:
        raise RuntimeError("attn_mask must have at most 4 dimensions")
    shape = (1,) * (4 - bias.dim()) + tuple(bias.shape)
    stride = (0,) * (4 - bias.dim()) + tuple(bias.stride())
    out = []
    for s, st, t in zip(shape, stride, target):
        if s == t:
            out.append(st if s != 1 else 0)
        elif s == 1:
            out.append(0)
        else:
            raise RuntimeError(f"attn_mask of shape {tuple(bias.shape)} is not broadcastable to {tuple(target)}")
    return out


# ----------------------------------------------------------------------------
# the one foreign call
# ----------------------------------------------------------------------------


def sdpa_forward(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    *,
    attn_bias: Optional[torch.Tensor] = None,
    is_causal: bool = False,
    scale: Optional[float] = None,
    kv_lens: Optional[torch.Tensor] = None,
    q_offset: int = 0,
    k_offset: int = 0,
    need_lse: bool = True,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    force_path: int = _lib.PATH_AUTO,
    kv_chunk: int = 0,
):
    """Launch the forward on the current CUDA stream; returns ``(out, lse)``
    (``lse`` is ``None`` when ``need_lse`` is false and no buffer was passed).

    Inputs must already satisfy :func:`_validate`; dtype is fp32/fp16/bf16.
    ``attn_bias`` is additive (bool masks are converted by the callers)."""
    lib = _lib.load()
    dev = _device_index(query)
    B, Hq, L, E = query.shape
    Hkv, S, Dv = key.shape[1], key.shape[2], value.shape[3]
    if scale is None:
        scale = 1.0 / math.sqrt(E)
    if out is None:
        out = alloc_like_query(query, (B, Hq, L, Dv))
    if lse is None and need_lse:
        lse = torch.empty((B, Hq, L), dtype=torch.float32, device=query.device)

    p = _lib.Params()
    p.struct_size = C.sizeof(_lib.Params)
    p.dtype = _DTYPE_CODE[query.dtype]
    p.device = dev
    p.force_path = force_path
    p.q, p.k, p.v, p.out = query.data_ptr(), key.data_ptr(), value.data_ptr(), out.data_ptr()
    p.lse = lse.data_ptr() if lse is not None else None
    p.q_stride[:] = query.stride()
    p.k_stride[:] = key.stride()
    p.v_stride[:] = value.stride()
    p.out_stride[:] = out.stride()
    if lse is not None:
        p.lse_stride[:] = lse.stride()
    p.B, p.Hq, p.Hkv, p.L, p.S, p.E, p.Dv = B, Hq, Hkv, L, S, E, Dv
    p.scale = float(scale)
    p.is_causal = 1 if is_causal else 0
    p.q_offset, p.k_offset = int(q_offset), int(k_offset)
    if kv_lens is not None:
        if kv_lens.dtype != torch.int32 or kv_lens.device != query.device or kv_lens.shape != (B,):
            raise RuntimeError("kv_lens must be an int32 CUDA tensor of shape (B,) on the query's device")
        if not kv_lens.is_contiguous():
            kv_lens = kv_lens.contiguous()
        p.kv_lens = kv_lens.data_ptr()
    if attn_bias is not None:
        if attn_bias.dtype not in _DTYPE_CODE:
            attn_bias = attn_bias.to(torch.float32)
        p.bias = attn_bias.data_ptr()
        p.bias_dtype = _DTYPE_CODE[attn_bias.dtype]
        p.bias_stride[:] = _bias_strides(attn_bias, (B, Hq, L, S))
    p.kv_chunk = int(kv_chunk)
    p.status = _status_word(dev).data_ptr()

    plan = _lib.Plan()
    plan.struct_size = C.sizeof(_lib.Plan)
    rc = lib.b200_sdpa_query_plan(C.byref(p), C.byref(plan))
    if rc != _lib.OK:
        raise RuntimeError(f"b200_sdpa_query_plan: {_lib.strerror(rc)}")
    ws = None
    if plan.workspace_bytes:
        ws = _workspace(dev, int(plan.workspace_bytes))
        p.workspace = ws.data_ptr()
        p.workspace_bytes = ws.numel()
    stream = torch.cuda.current_stream(dev).cuda_stream
    rc = lib.b200_sdpa_fwd(C.byref(p), C.c_void_p(stream))
    if rc != _lib.OK:
        raise RuntimeError(f"b200_sdpa_fwd: {_lib.strerror(rc)}")
    last_plan.clear()
    last_plan.update(
        path=_lib.PATH_NAMES.get(plan.path, str(plan.path)), block_m=plan.block_m, block_n=plan.block_n,
        grid=(plan.grid_x, plan.grid_y, plan.grid_z), threads=plan.threads, smem_bytes=plan.smem_bytes,
        kv_splits=plan.kv_splits, launches=plan.launches, workspace_bytes=int(plan.workspace_bytes),
    )
    return out, lse


def sdpa_forward_accumulate(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    acc: torch.Tensor,
    acc_lse: torch.Tensor,
    *,
    first: bool,
    is_causal: bool = False,
    scale: Optional[float] = None,
    q_offset: int = 0,
    k_offset: int = 0,
) -> bool:
    """One step of a ring over key/value blocks with the merge fused into the attention kernel's
    epilogue: the result of ``query`` against this block is folded into the running fp32 ``acc``
    ``(B, Hq, L, Dv)`` / ``acc_lse`` ``(B, Hq, L)`` (overwritten when ``first``) -- no partial in the
    storage dtype, no separate merge launch (upstream merges in Python between per-block calls,
    ``cp_ring_handler.py:308-318``).  Returns False, having done nothing, when the request is not one
    the accumulating kernels serve (the tensor-core prefill kernels: f16/bf16, head dim 128, no bias,
    TMA-legal strides); the caller then runs the plain forward and :func:`merge_partials`."""
    if query.dtype not in (torch.float16, torch.bfloat16) or not query.is_cuda:
        return False
    lib = _lib.load()
    dev = _device_index(query)
    B, Hq, L, E = query.shape
    Hkv, S, Dv = key.shape[1], key.shape[2], value.shape[3]
    if acc.dtype != torch.float32 or tuple(acc.shape) != (B, Hq, L, Dv) or acc.stride(3) != 1:
        raise RuntimeError("acc must be an fp32 (B, Hq, L, Dv) tensor with unit inner stride")
    if acc_lse.dtype != torch.float32 or tuple(acc_lse.shape) != (B, Hq, L):
        raise RuntimeError("acc_lse must be an fp32 (B, Hq, L) tensor")
    if scale is None:
        scale = 1.0 / math.sqrt(E)
    p = _lib.Params()
    p.struct_size = C.sizeof(_lib.Params)
    p.dtype = _DTYPE_CODE[query.dtype]
    p.device = dev
    p.force_path = _lib.PATH_AUTO
    p.q, p.k, p.v = query.data_ptr(), key.data_ptr(), value.data_ptr()
    p.q_stride[:] = query.stride()
    p.k_stride[:] = key.stride()
    p.v_stride[:] = value.stride()
    p.out_stride[:] = (Hq * L * Dv, L * Dv, Dv, 1)     # no output tensor in this form
    p.B, p.Hq, p.Hkv, p.L, p.S, p.E, p.Dv = B, Hq, Hkv, L, S, E, Dv
    p.scale = float(scale)
    p.is_causal = 1 if is_causal else 0
    p.q_offset, p.k_offset = int(q_offset), int(k_offset)
    p.acc_mode = 1 if first else 2
    p.acc, p.acc_lse = acc.data_ptr(), acc_lse.data_ptr()
    p.acc_stride[:] = acc.stride()[:3]
    p.acc_lse_stride[:] = acc_lse.stride()
    p.status = _status_word(dev).data_ptr()
    plan = _lib.Plan()
    plan.struct_size = C.sizeof(_lib.Plan)
    rc = lib.b200_sdpa_query_plan(C.byref(p), C.byref(plan))
    if rc in (_lib.ERR_UNSUPPORTED, _lib.ERR_ALIGNMENT):
        return False
    if rc != _lib.OK:
        raise RuntimeError(f"b200_sdpa_query_plan: {_lib.strerror(rc)}")
    if plan.workspace_bytes:
        ws = _workspace(dev, int(plan.workspace_bytes))
        p.workspace = ws.data_ptr()
        p.workspace_bytes = ws.numel()
    rc = lib.b200_sdpa_fwd(C.byref(p), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    if rc != _lib.OK:
        raise RuntimeError(f"b200_sdpa_fwd: {_lib.strerror(rc)}")
    last_plan.clear()
    last_plan.update(path=_lib.PATH_NAMES.get(plan.path, str(plan.path)), grid=(plan.grid_x, plan.grid_y, plan.grid_z),
                     threads=plan.threads, launches=plan.launches, accumulate=True)
    return True


def paged_decode(
    query: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    block_table: torch.Tensor,
    kv_lens: torch.Tensor,
    *,
    scale: Optional[float] = None,
    layout: str = "NHD",
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    need_lse: bool = False,
    kv_chunk: int = 0,
    k_new: Optional[torch.Tensor] = None,
    v_new: Optional[torch.Tensor] = None,
    rope_cos: Optional[torch.Tensor] = None,
    rope_sin: Optional[torch.Tensor] = None,
    rope_interleaved: bool = False,
):
    """One decode step against a paged key/value cache; returns ``(out, lse)`` -- or, with
    ``k_new`` / ``v_new`` (``(B, Hkv, D)``, the rows of the token being decoded),
    ``(out, lse, new_lens)``: the new row is attended to as key ``kv_lens[b]`` and written
    into its page by the kernel that reads it (see :func:`decode_append`).

    ``query`` is ``(B, Hq, 1, D)``; ``k_pages`` / ``v_pages`` are page pools,
    ``(pages, page_size, Hkv, D)`` for ``layout="NHD"`` or ``(pages, Hkv, page_size, D)``
    for ``"HND"`` (any strides with a unit inner stride); ``block_table`` is int32
    ``(B, max_pages)`` and ``kv_lens`` int32 ``(B,)``.  Key ``s`` of sequence ``b`` is row
    ``s % page_size`` of page ``block_table[b, s // page_size]``.  The split-KV decode
    kernel reads the pages in place -- no gather into a dense cache.  Upstream's decode
    runs the same op on a dense cache (``torch_mlir/ops/scaled_dot_product_attention.py:64-68``);
    the paged layout is what a serving loop around that op keeps."""
    lib = _lib.load()
    if layout not in ("NHD", "HND"):
        raise ValueError("layout must be 'NHD' or 'HND'")
    if query.dim() != 4 or query.shape[2] != 1 or k_pages.dim() != 4 or v_pages.dim() != 4:
        raise RuntimeError("paged_decode: query must be (B, Hq, 1, D) and the page pools 4-D")
    if query.dtype not in (torch.float16, torch.bfloat16) or k_pages.dtype != query.dtype or v_pages.dtype != query.dtype:
        raise RuntimeError("paged_decode: query and the page pools must share a float16 or bfloat16 dtype")
    if not (query.is_cuda and k_pages.device == query.device and v_pages.device == query.device):
        raise ValueError(f"Expected CUDA tensors on one device, got {query.device}, {k_pages.device}, {v_pages.device}")
    dev = _device_index(query)
    B, Hq, _, E = query.shape
    hd, rd = (2, 1) if layout == "NHD" else (1, 2)
    Hkv, page_size = k_pages.shape[hd], k_pages.shape[rd]
    if k_pages.shape != v_pages.shape or k_pages.shape[3] != E:
        raise RuntimeError("paged_decode: k_pages and v_pages must have the same shape and the query's head dim")
    if Hkv == 0 or Hq % Hkv != 0:
        raise RuntimeError("SDPA: Number of heads in key and value must divide the number of heads in query")
    if block_table.dtype != torch.int32 or block_table.dim() != 2 or block_table.shape[0] != B or block_table.device != query.device:
        raise RuntimeError("paged_decode: block_table must be an int32 CUDA tensor of shape (B, max_pages)")
    if kv_lens.dtype != torch.int32 or kv_lens.shape != (B,) or kv_lens.device != query.device:
        raise RuntimeError("kv_lens must be an int32 CUDA tensor of shape (B,) on the query's device")
    block_table = block_table.contiguous()
    kv_lens = kv_lens.contiguous()
    if scale is None:
        scale = 1.0 / math.sqrt(E)
    if out is None:
        out = torch.empty_like(query)
    if lse is None and need_lse:
        lse = torch.empty((B, Hq, 1), dtype=torch.float32, device=query.device)

    p = _lib.Params()
    p.struct_size = C.sizeof(_lib.Params)
    p.dtype = _DTYPE_CODE[query.dtype]
    p.device = dev
    p.force_path = _lib.PATH_DECODE
    p.q, p.k, p.v, p.out = query.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr()
    p.lse = lse.data_ptr() if lse is not None else None
    p.q_stride[:] = query.stride()
    p.k_stride[:] = [k_pages.stride(0), k_pages.stride(hd), k_pages.stride(rd), k_pages.stride(3)]
    p.v_stride[:] = [v_pages.stride(0), v_pages.stride(hd), v_pages.stride(rd), v_pages.stride(3)]
    p.out_stride[:] = out.stride()
    if lse is not None:
        p.lse_stride[:] = lse.stride()
    p.B, p.Hq, p.Hkv, p.L, p.E, p.Dv = B, Hq, Hkv, 1, E, E
    p.S = block_table.shape[1] * page_size
    p.scale = float(scale)
    p.kv_lens = kv_lens.data_ptr()
    p.block_table = block_table.data_ptr()
    p.block_table_stride = block_table.shape[1]
    p.page_size = page_size
    rope = (rope_cos, rope_sin, rope_interleaved) if rope_cos is not None else None
    new_lens = _attach_new_rows(p, k_new, v_new, query, Hkv, kv_lens, rope, capacity=int(p.S))
    _launch_decode(lib, p, dev, kv_chunk)
    return (out, lse) if new_lens is None else (out, lse, new_lens)


def _launch_decode(lib, p, dev: int, kv_chunk: int) -> None:
    """Plan, attach the scratch and enqueue a decode parameter block on the current stream."""
    p.kv_chunk = int(kv_chunk)
    p.status = _status_word(dev).data_ptr()
    plan = _lib.Plan()
    plan.struct_size = C.sizeof(_lib.Plan)
    rc = lib.b200_sdpa_query_plan(C.byref(p), C.byref(plan))
    if rc != _lib.OK:
        raise RuntimeError(f"b200_sdpa_query_plan: {_lib.strerror(rc)}")
    ws = _workspace(dev, int(plan.workspace_bytes))
    p.workspace = ws.data_ptr()
    p.workspace_bytes = ws.numel()
    rc = lib.b200_sdpa_decode(C.byref(p), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    if rc != _lib.OK:
        raise RuntimeError(f"b200_sdpa_decode: {_lib.strerror(rc)}")


def _attach_new_rows(p, k_new, v_new, query, Hkv, kv_lens, rope=None, capacity=None):
    """Fill the append (and rotary) fields of a parameter block; returns the tensor that will receive the
    new lengths.  ``rope`` = ``(cos, sin, interleaved)`` with fp32 ``(positions, >= D/2)`` tables that
    must cover every position of the cache (``positions >= capacity``)."""
    if k_new is None and v_new is None:
        if rope is not None:
            raise RuntimeError("decode append: the rotary embedding is applied together with an appended row")
        return None
    if k_new is None or v_new is None:
        raise RuntimeError("decode append: k_new and v_new go together")
    B, _, _, E = query.shape
    for name, t in (("k_new", k_new), ("v_new", v_new)):
        if tuple(t.shape) != (B, Hkv, E) or t.dtype != query.dtype or t.device != query.device or t.stride(2) != 1:
            raise RuntimeError(f"decode append: {name} must be (B, Hkv, D) in the query dtype with unit inner stride")
    p.k_new, p.v_new = k_new.data_ptr(), v_new.data_ptr()
    p.k_new_stride[:] = k_new.stride()[:2]
    p.v_new_stride[:] = v_new.stride()[:2]
    if rope is not None:
        cos, sin, interleaved = rope
        for name, t in (("rope_cos", cos), ("rope_sin", sin)):
            if t.dtype != torch.float32 or t.dim() != 2 or t.shape[1] < E // 2 or t.stride(1) != 1 or t.device != query.device:
                raise RuntimeError(f"decode append: {name} must be an fp32 (positions, >= D/2) CUDA tensor with unit inner stride")
        if cos.stride(0) != sin.stride(0) or cos.shape[0] != sin.shape[0]:
            raise RuntimeError("decode append: rope_cos and rope_sin must have the same rows and row stride")
        if cos.shape[0] < 1 or (capacity is not None and cos.shape[0] < capacity):
            raise RuntimeError(
                f"decode append: the rotary tables hold {cos.shape[0]} positions but the cache has room for {capacity}"
            )
        p.rope_cos, p.rope_sin = cos.data_ptr(), sin.data_ptr()
        p.rope_positions = cos.shape[0]
        p.rope_stride = cos.stride(0)
        p.rope_interleaved = 1 if interleaved else 0
    new_lens = torch.empty_like(kv_lens)
    p.kv_lens_out = new_lens.data_ptr()
    return new_lens


def decode_append(
    query: torch.Tensor,
    k_new: torch.Tensor,
    v_new: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    kv_lens: torch.Tensor,
    *,
    scale: Optional[float] = None,
    need_lse: bool = False,
    kv_chunk: int = 0,
    rope_cos: Optional[torch.Tensor] = None,
    rope_sin: Optional[torch.Tensor] = None,
    rope_interleaved: bool = False,
):
    """One decode step of a generation loop against a dense ``(B, Hkv, S, D)`` cache, with the
    cache append fused into the attention kernel: batch ``b`` attends keys ``[0, kv_lens[b]]``
    where key ``kv_lens[b]`` is the new row ``k_new[b]`` / ``v_new[b]`` (``(B, Hkv, D)``), and
    the CTA that reads that row also writes it into ``k_cache`` / ``v_cache`` at that position.
    Returns ``(out, lse, new_lens)`` with ``new_lens = min(kv_lens + 1, S)`` in a fresh tensor.
    A sequence whose cache is full appends nothing (its new token is neither stored nor attended
    to) and the device status word reports it: :func:`check_device_status` then raises.  With ``rope_cos`` / ``rope_sin`` (fp32
    ``(positions, >= D/2)``) the rotary embedding of position ``kv_lens[b]`` is applied to the query
    and to the new key inside the same kernel (fp32 arithmetic, one rounding; ``rope_interleaved``
    selects the (2i, 2i+1) pairing instead of (i, i + D/2)) and the key is cached rotated.  (Upstream's loop appends with separate ops
    before the attention op: ``tests/blocks/block_def/llama.py:110-119`` is the caller shape.)"""
    lib = _lib.load()
    if query.dim() != 4 or query.shape[2] != 1 or k_cache.dim() != 4 or v_cache.shape != k_cache.shape:
        raise RuntimeError("decode_append: query must be (B, Hq, 1, D) and the caches (B, Hkv, S, D)")
    if query.dtype not in (torch.float16, torch.bfloat16) or k_cache.dtype != query.dtype or v_cache.dtype != query.dtype:
        raise RuntimeError("decode_append: query and caches must share a float16 or bfloat16 dtype")
    dev = _device_index(query)
    B, Hq, _, E = query.shape
    Hkv, S = k_cache.shape[1], k_cache.shape[2]
    if Hkv == 0 or Hq % Hkv != 0:
        raise RuntimeError("SDPA: Number of heads in key and value must divide the number of heads in query")
    if kv_lens.dtype != torch.int32 or kv_lens.shape != (B,) or kv_lens.device != query.device:
        raise RuntimeError("kv_lens must be an int32 CUDA tensor of shape (B,) on the query's device")
    kv_lens = kv_lens.contiguous()
    if scale is None:
        scale = 1.0 / math.sqrt(E)
    out = torch.empty_like(query)
    lse = torch.empty((B, Hq, 1), dtype=torch.float32, device=query.device) if need_lse else None
    p = _lib.Params()
    p.struct_size = C.sizeof(_lib.Params)
    p.dtype = _DTYPE_CODE[query.dtype]
    p.device = dev
    p.force_path = _lib.PATH_DECODE
    p.q, p.k, p.v, p.out = query.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr()
    p.lse = lse.data_ptr() if lse is not None else None
    p.q_stride[:] = query.stride()
    p.k_stride[:] = k_cache.stride()
    p.v_stride[:] = v_cache.stride()
    p.out_stride[:] = out.stride()
    if lse is not None:
        p.lse_stride[:] = lse.stride()
    p.B, p.Hq, p.Hkv, p.L, p.S, p.E, p.Dv = B, Hq, Hkv, 1, S, E, E
    p.scale = float(scale)
    p.kv_lens = kv_lens.data_ptr()
    rope = (rope_cos, rope_sin, rope_interleaved) if rope_cos is not None else None
    new_lens = _attach_new_rows(p, k_new, v_new, query, Hkv, kv_lens, rope, capacity=S)
    _launch_decode(lib, p, dev, kv_chunk)
    return out, lse, new_lens


def sdpa_backward(
    grad_out: torch.Tensor,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    out: torch.Tensor,
    lse: torch.Tensor,
    *,
    attn_bias: Optional[torch.Tensor] = None,
    is_causal: bool = False,
    scale: Optional[float] = None,
    kv_lens: Optional[torch.Tensor] = None,
    q_offset: int = 0,
    k_offset: int = 0,
    need_grad_bias: bool = False,
    grad_q: Optional[torch.Tensor] = None,
    grad_k: Optional[torch.Tensor] = None,
    grad_v: Optional[torch.Tensor] = None,
    force_path: int = _lib.PATH_AUTO,
):
    """Launch the backward on the current CUDA stream; returns ``(grad_q, grad_k,
    grad_v, grad_bias)``.  Each gradient is allocated with the layout of the tensor
    it belongs to (what upstream's ``DispatchSdpaBwdImpl`` does with
    ``alloc_with_matching_layout``, ``NeuronDispatcher.cpp:2560-2575``) and the
    kernels store with those strides.  ``grad_bias`` is the gradient of the logits,
    ``(B, Hq, L, S)`` in the query dtype, or ``None`` unless asked for."""
    lib = _lib.load()
    dev = _device_index(query)
    B, Hq, L, E = query.shape
    Hkv, S, Dv = key.shape[1], key.shape[2], value.shape[3]
    if tuple(grad_out.shape) != (B, Hq, L, Dv) or tuple(out.shape) != (B, Hq, L, Dv):
        raise RuntimeError("SDPA backward: grad_out and out must have shape (B, Hq, L, Dv)")
    if grad_out.dtype != query.dtype or out.dtype != query.dtype:
        raise RuntimeError("SDPA backward: grad_out and out must have the dtype of query")
    if lse.dtype != torch.float32 or tuple(lse.shape) != (B, Hq, L):
        raise RuntimeError("SDPA backward: logsumexp must be a float32 tensor of shape (B, Hq, L)")
    if scale is None:
        scale = 1.0 / math.sqrt(E)
    if grad_out.stride(3) != 1 or any((st * grad_out.element_size()) % 16 for st in grad_out.stride()[:3]):
        grad_out = grad_out.contiguous()   # e.g. the expanded gradient of a reduction: stride 0 everywhere
    grad_q = torch.empty_like(query) if grad_q is None else grad_q
    grad_k = torch.empty_like(key) if grad_k is None else grad_k
    grad_v = torch.empty_like(value) if grad_v is None else grad_v
    for g, like in ((grad_q, query), (grad_k, key), (grad_v, value)):
        if g.shape != like.shape or g.dtype != like.dtype or g.device != like.device:
            raise RuntimeError("SDPA backward: a gradient buffer must match its tensor in shape, dtype and device")
    grad_bias = None
    if need_grad_bias:
        grad_bias = torch.empty((B, Hq, L, S), dtype=query.dtype, device=query.device)

    p = _lib.BwdParams()
    p.struct_size = C.sizeof(_lib.BwdParams)
    p.dtype = _DTYPE_CODE[query.dtype]
    p.device = dev
    p.grad_out, p.q, p.k, p.v = grad_out.data_ptr(), query.data_ptr(), key.data_ptr(), value.data_ptr()
    p.out, p.lse = out.data_ptr(), lse.data_ptr()
    p.grad_q, p.grad_k, p.grad_v = grad_q.data_ptr(), grad_k.data_ptr(), grad_v.data_ptr()
    p.grad_out_stride[:] = grad_out.stride()
    p.q_stride[:] = query.stride()
    p.k_stride[:] = key.stride()
    p.v_stride[:] = value.stride()
    p.out_stride[:] = out.stride()
    p.lse_stride[:] = lse.stride()
    p.grad_q_stride[:] = grad_q.stride()
    p.grad_k_stride[:] = grad_k.stride()
    p.grad_v_stride[:] = grad_v.stride()
    if grad_bias is not None:
        p.grad_bias = grad_bias.data_ptr()
        p.grad_bias_stride[:] = grad_bias.stride()
    p.B, p.Hq, p.Hkv, p.L, p.S, p.E, p.Dv = B, Hq, Hkv, L, S, E, Dv
    p.scale = float(scale)
    p.is_causal = 1 if is_causal else 0
    p.q_offset, p.k_offset = int(q_offset), int(k_offset)
    if kv_lens is not None:
        if kv_lens.dtype != torch.int32 or kv_lens.device != query.device or kv_lens.shape != (B,):
            raise RuntimeError("kv_lens must be an int32 CUDA tensor of shape (B,) on the query's device")
        kv_lens = kv_lens.contiguous()
        p.kv_lens = kv_lens.data_ptr()
    if attn_bias is not None:
        if attn_bias.dtype not in _DTYPE_CODE:
            attn_bias = attn_bias.to(torch.float32)
        p.bias = attn_bias.data_ptr()
        p.bias_dtype = _DTYPE_CODE[attn_bias.dtype]
        p.bias_stride[:] = _bias_strides(attn_bias, (B, Hq, L, S))
    p.status = _status_word(dev).data_ptr()
    p.force_path = force_path
    plan = _lib.Plan()
    plan.struct_size = C.sizeof(_lib.Plan)
    rc = lib.b200_sdpa_bwd_query_plan(C.byref(p), C.byref(plan))
    if rc != _lib.OK:
        raise RuntimeError(f"b200_sdpa_bwd_query_plan: {_lib.strerror(rc)}")
    ws = None
    if plan.workspace_bytes:
        ws = _workspace(dev, int(plan.workspace_bytes))
        p.workspace = ws.data_ptr()
        p.workspace_bytes = ws.numel()
    rc = lib.b200_sdpa_bwd(C.byref(p), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    if rc != _lib.OK:
        raise RuntimeError(f"b200_sdpa_bwd: {_lib.strerror(rc)}")
    last_bwd_plan.clear()
    last_bwd_plan.update(path=_lib.PATH_NAMES.get(plan.path, str(plan.path)), launches=plan.launches,
                         workspace_bytes=int(plan.workspace_bytes))
    return grad_q, grad_k, grad_v, grad_bias


def merge_partials(acc, acc_lse, part, part_lse, *, first=False, final_out=None):
    """One ring-step merge on the current stream: fold ``(part, part_lse)`` into the
    fp32 running ``(acc, acc_lse)`` in place; optionally also write the merged rows
    to ``final_out`` in the partial's dtype."""
    lib = _lib.load()
    B, Hq, L, Dv = part.shape
    if acc.dtype != torch.float32 or acc.stride(3) != 1 or tuple(acc.shape) != (B, Hq, L, Dv):
        raise RuntimeError("acc must be an fp32 tensor shaped like the partial with unit inner stride")
    if acc_lse.dtype != torch.float32 or tuple(acc_lse.shape) != (B, Hq, L):
        raise RuntimeError("acc_lse must be an fp32 tensor of shape (B, Hq, L)")
    m = _lib.MergeParams()
    m.struct_size = C.sizeof(_lib.MergeParams)
    m.dtype = _DTYPE_CODE[part.dtype]
    m.device = _device_index(part)
    m.first = 1 if first else 0
    m.acc, m.acc_lse = acc.data_ptr(), acc_lse.data_ptr()
    m.part, m.part_lse = part.data_ptr(), part_lse.data_ptr()
    m.part_stride[:] = part.stride()
    m.part_lse_stride[:] = part_lse.stride()
    if final_out is not None:
        m.final_out = final_out.data_ptr()
        m.final_stride[:] = final_out.stride()
    m.B, m.Hq, m.L, m.Dv = B, Hq, L, Dv
    m.acc_stride[:] = acc.stride()[:3]
    m.acc_lse_stride[:] = acc_lse.stride()
    rc = lib.b200_sdpa_merge(C.byref(m), C.c_void_p(torch.cuda.current_stream(m.device).cuda_stream))
    if rc != _lib.OK:
        raise RuntimeError(f"b200_sdpa_merge: {_lib.strerror(rc)}")


# ----------------------------------------------------------------------------
# ATen-level op
# ----------------------------------------------------------------------------


def _additive_bias(attn_mask: Optional[torch.Tensor], query: torch.Tensor):
    """Bool mask (True = keep) -> 0 / -inf in the query dtype; float masks are used as
    they are (``decompositions.py:2099-2104``)."""
    if attn_mask is None:
        return None
    if attn_mask.dtype == torch.bool:
        return torch.where(attn_mask, 0.0, float("-inf")).to(query.dtype)
    return attn_mask


def fused_attention_overrideable(
    query, key, value, attn_bias=None, dropout_p=0.0, is_causal=False, return_debug_mask=False, *, scale=None
):
    """CUDA implementation of ``aten::_scaled_dot_product_fused_attention_overrideable``.

    Returns ``(output, logsumexp, cum_seq_q, cum_seq_k, max_q, max_k, philox_seed,
    philox_offset, debug_attn_mask)``: output in the query dtype with the query's
    layout, logsumexp fp32 ``(B, Hq, L)`` always (the ATen contract upstream keeps,
    ``scaled_dot_product_fused_attention.py:291-295``), the unused slots ``None`` and
    the philox slots zero scalars since dropout is not offered."""
    _validate(query, key, value, attn_bias, dropout_p, is_causal, return_debug_mask)
    B, Hq, L, _ = query.shape
    S, Dv = key.shape[2], value.shape[3]
    if query.numel() == 0 or key.shape[3] == 0 or Dv == 0:
        raise RuntimeError("SDPA: zero-size inputs are not routed to the fused kernel")
    in_dtype = query.dtype
    if in_dtype == torch.float64:  # computed in fp32 and cast back (NeuronDispatcher.cpp:2418-2434)
        query, key, value = query.float(), key.float(), value.float()
        if attn_bias is not None and attn_bias.dtype == torch.float64:
            attn_bias = attn_bias.float()
    bias = _additive_bias(attn_bias, query)
    out, lse = sdpa_forward(query, key, value, attn_bias=bias, is_causal=is_causal, scale=scale, need_lse=True)
    if in_dtype == torch.float64:
        out = out.double()
    seed, offset = _philox_zeros(_device_index(query))
    return out, lse, None, None, L, S, seed, offset, None


def fused_attention_overrideable_backward(
    grad_out, query, key, value, attn_bias, grad_input_mask, out, logsumexp, cum_seq_q, cum_seq_k, max_q, max_k,
    dropout_p, is_causal, philox_seed, philox_offset, *, scale=None
):
    """CUDA implementation of ``aten::_scaled_dot_product_fused_attention_overrideable_backward``
    (upstream: ``scaled_dot_product_fused_attention.py:717-781`` and
    ``NeuronDispatcher.cpp:2523-2582``).  Returns ``(grad_query, grad_key, grad_value,
    grad_attn_bias)``; the sequence metadata and philox slots are ignored as upstream
    ignores them, and the bias gradient is the logit gradient in full ``(B, Hq, L, S)``
    shape (``_sdpa_math.py:169``) -- autograd reduces it to a broadcast bias's shape --
    or an undefined tensor when no bias took part."""
    if query.device.type != "cuda":
        raise ValueError(f"Expected CUDA device, got {query.device}")
    if key.shape[1] == 0 or query.shape[1] % key.shape[1] != 0:
        raise RuntimeError("SDPA: Number of heads in key and value must divide the number of heads in query")
    if dropout_p != 0.0:
        raise NotImplementedError("dropout_p != 0 is not supported by the B200 fused attention path")
    in_dtype = query.dtype
    if in_dtype == torch.float64:
        grad_out, query, key, value, out = (t.float() for t in (grad_out, query, key, value, out))
    # only None or an empty tensor mean "no bias" (upstream: scaled_dot_product_fused_attention.py:178);
    # a one-element bias shifted every logit in the forward and is part of lse
    has_bias = attn_bias is not None and attn_bias.numel() != 0
    bias = None
    if has_bias:
        bias = attn_bias.float() if attn_bias.dtype == torch.float64 else attn_bias
    want_bias_grad = has_bias and (grad_input_mask is None or len(grad_input_mask) < 4 or bool(grad_input_mask[3]))
    gq, gk, gv, gb = sdpa_backward(
        grad_out, query, key, value, out, logsumexp, attn_bias=bias, is_causal=is_causal, scale=scale,
        need_grad_bias=want_bias_grad,
    )
    if in_dtype == torch.float64:
        gq, gk, gv = gq.double(), gk.double(), gv.double()
        gb = gb.double() if gb is not None else None
    return gq, gk, gv, gb


def _overrideable_backward_meta(
    grad_out, query, key, value, attn_bias, grad_input_mask, out, logsumexp, cum_seq_q, cum_seq_k, max_q, max_k,
    dropout_p, is_causal, philox_seed, philox_offset, *, scale=None
):
    grad_bias = None
    if attn_bias is not None and attn_bias.numel() != 0 and (len(grad_input_mask) < 4 or grad_input_mask[3]):
        grad_bias = query.new_empty((query.shape[0], query.shape[1], query.shape[2], key.shape[2]))
    return torch.empty_like(query), torch.empty_like(key), torch.empty_like(value), grad_bias


# ----------------------------------------------------------------------------
# kernel-level custom op (signature of upstream's nki_kernels op)
# ----------------------------------------------------------------------------

_LIB_DEF = torch.library.Library("b200_sdpa", "DEF")
_LIB_DEF.define(
    "fwd(Tensor q, Tensor k, Tensor v, bool is_causal, float dropout_p, float? scale, bool training, "
    "int? seed, Tensor(a!)? lse, *, Tensor? kv_lens=None) -> Tensor"
)


def _fwd_cuda(q, k, v, is_causal, dropout_p, scale, training, seed, lse, *, kv_lens=None):
    _validate(q, k, v, None, dropout_p, False, False)
    B, Hq, L, _ = q.shape
    buf = None
    if training:
        if lse is not None and lse.dtype == torch.float32 and tuple(lse.shape) == (B, Hq, L) and lse.is_cuda:
            buf = lse  # written in place: no copy as upstream's lse.copy_() needs
    out, got = sdpa_forward(q, k, v, is_causal=is_causal, scale=scale, kv_lens=kv_lens, need_lse=training, lse=buf)
    if training and lse is not None and buf is None:
        lse.copy_(got.reshape(lse.shape))
    return out


def _fwd_meta(q, k, v, is_causal, dropout_p, scale, training, seed, lse, *, kv_lens=None):
    return alloc_like_query(q, (q.shape[0], q.shape[1], q.shape[2], v.shape[3]))


_LIB_IMPL = torch.library.Library("b200_sdpa", "IMPL")
_LIB_IMPL.impl("fwd", _fwd_cuda, "CUDA")
_LIB_IMPL.impl("fwd", _fwd_meta, "Meta")


_LIB_DEF.define(
    "bwd(Tensor grad_out, Tensor q, Tensor k, Tensor v, Tensor out, Tensor lse, bool is_causal=False, "
    "float dropout_p=0.0, float? scale=None, int? seed=None, *, Tensor? kv_lens=None) -> (Tensor, Tensor, Tensor)"
)


def _bwd_cuda(grad_out, q, k, v, out, lse, is_causal=False, dropout_p=0.0, scale=None, seed=None, *, kv_lens=None):
    _validate(q, k, v, None, dropout_p, False, False)
    gq, gk, gv, _ = sdpa_backward(grad_out, q, k, v, out, lse, is_causal=is_causal, scale=scale, kv_lens=kv_lens)
    return gq, gk, gv


def _bwd_meta(grad_out, q, k, v, out, lse, is_causal=False, dropout_p=0.0, scale=None, seed=None, *, kv_lens=None):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


_LIB_IMPL.impl("bwd", _bwd_cuda, "CUDA")
_LIB_IMPL.impl("bwd", _bwd_meta, "Meta")


def scaled_dot_product_attention_backward_kernel(
    grad_out, q, k, v, out, lse, is_causal=False, dropout_p=0.0, scale=None, seed=None, kv_lens=None
):
    """Same call shape as upstream's ``scaled_dot_product_attention_backward_kernel``
    (``nki_kernels/scaled_dot_product_attention_backward.py:9-50``): gradients for q, k
    and v from the forward's output and fp32 ``(B, Hq, L)`` log-sum-exp."""
    return torch.ops.b200_sdpa.bwd(grad_out, q, k, v, out, lse, is_causal, dropout_p, scale, seed, kv_lens=kv_lens)


def scaled_dot_product_attention_kernel(
    q, k, v, is_causal=False, dropout_p=0.0, scale=None, training=False, seed=None, lse=None, kv_lens=None
):
    """Same call shape as upstream's ``scaled_dot_product_attention_kernel``
    (``nki_kernels/scaled_dot_product_attention.py:44-86``): returns the attention
    output; with ``training=True`` the fp32 log-sum-exp is written into ``lse``."""
    return torch.ops.b200_sdpa.fwd(q, k, v, is_causal, dropout_p, scale, training, seed, lse, kv_lens=kv_lens)


# ----------------------------------------------------------------------------
# middle stage of native multi-head attention (inference caller of the same kernels)
# ----------------------------------------------------------------------------


def native_multi_head_attn_mid(query, key, value, *, use_causal_mask=False, dropout_p=0.0, training=False, out=None):
    """The attention stage of upstream's split ``native_multi_head_attention``
    (``python_ops/native_multi_head_attn_mid.py:66-157``,
    ``python_ops/torch_mlir/ops/native_multi_head_attn_mid.py:58-114``): q, k and v arrive
    in ``[B, H, D, S]`` layout, the result is ``[B, Hq, S_q, D_v]``; no log-sum-exp is
    produced, ``training`` does not change the computation, and ``out`` (if given) is
    written in place and returned.

    The ``[B, H, D, S]`` operands are the ``[B, H, S, D]`` operands seen through a
    transpose, which the kernels take as strides.  Half-precision inputs with a head
    dimension the tensor-core kernels serve are first re-laid out with the head dimension
    innermost (one streaming copy, far cheaper than leaving the call on CUDA cores)."""
    for name, t in (("query", query), ("key", key), ("value", value)):
        if not isinstance(t, torch.Tensor) or t.dim() != 4:
            raise RuntimeError(f"native_multi_head_attn_mid: {name} must be a 4-D tensor [B, H, D, S]")
    if query.numel() == 0 or key.numel() == 0 or value.numel() == 0:
        raise RuntimeError(
            "Attention operations do not support empty tensors. Please ensure all input tensors have non-zero elements."
        )
    q, k, v = query.transpose(-2, -1), key.transpose(-2, -1), value.transpose(-2, -1)
    _validate(q, k, v, None, dropout_p, use_causal_mask, False)
    if q.dtype in (torch.float16, torch.bfloat16) and q.shape[3] == v.shape[3] and q.shape[3] in (64, 128):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, Hq, L, _ = q.shape
    if out is not None:
        if tuple(out.shape) != (B, Hq, L, v.shape[3]) or out.dtype != q.dtype or out.device != q.device:
            raise RuntimeError("native_multi_head_attn_mid: out must be [B, Hq, S_q, D_v] in the input dtype on the input device")
    result, _ = sdpa_forward(q, k, v, is_causal=bool(use_causal_mask), need_lse=False, out=out)
    return result


# ----------------------------------------------------------------------------
# registration with ATen
# ----------------------------------------------------------------------------

_ATEN_IMPL = None
_ROUTING = None
_SDP_OVERRIDEABLE = 4  # at::SDPBackend::overrideable


def register_aten_override() -> None:
    """Register the CUDA kernel of the overrideable fused-attention op (upstream does the
    same for its device key at import, ``python_ops/__init__.py:86-95``)."""
    global _ATEN_IMPL
    if _ATEN_IMPL is not None:
        return
    lib = torch.library.Library("aten", "IMPL")
    if not _lib.load_ops():
        # the C++ operator layer (which registers these two kernels natively, so that a call runs without
        # the interpreter lock) has not been built: the same kernels through the ctypes binding
        lib.impl("_scaled_dot_product_fused_attention_overrideable", fused_attention_overrideable, "CUDA")
        lib.impl(
            "_scaled_dot_product_fused_attention_overrideable_backward", fused_attention_overrideable_backward, "CUDA"
        )
    # torch ships a meta kernel for the forward op only; tracing and DTensor's sharding propagation need
    # the backward's output shapes too
    lib.impl("_scaled_dot_product_fused_attention_overrideable_backward", _overrideable_backward_meta, "Meta")
    _ATEN_IMPL = lib


def native_op_layer() -> bool:
    """Whether the ATen ops are served by the C++ operator layer (``libb200_sdpa_ops.so``)."""
    return _lib.load_ops()


def _supported_by_fused_path(query, key, value, attn_mask, dropout_p, is_causal) -> bool:
    """Same decision shape as upstream's backend choice
    (``torch_neuronx/csrc/aten/SdpBackendSelection.cpp:14-68``): 4-D, non-empty, and
    additionally what this build serves (dtype, no dropout)."""
    if query.dim() != 4 or key.dim() != 4 or value.dim() != 4:
        return False
    if query.numel() == 0 or key.numel() == 0 or value.numel() == 0:
        return False
    if query.dtype not in _DTYPE_CODE or dropout_p != 0.0:
        return False
    if attn_mask is not None and is_causal:
        return False
    return True


class _SdpaRouting(torch.overrides.TorchFunctionMode):
    """Sends ``F.scaled_dot_product_attention`` calls this build serves to the fused op
    and leaves every other call to torch."""

    def __torch_function__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func is torch.nn.functional.scaled_dot_product_attention:
            names = ("query", "key", "value", "attn_mask", "dropout_p", "is_causal", "scale", "enable_gqa")
            bound = dict(zip(names, args))
            bound.update(kwargs)
            q, k, v = bound.get("query"), bound.get("key"), bound.get("value")
            mask, drop = bound.get("attn_mask"), bound.get("dropout_p", 0.0)
            causal = bound.get("is_causal", False)
            if (
                isinstance(q, torch.Tensor) and isinstance(k, torch.Tensor) and isinstance(v, torch.Tensor)
                and q.is_cuda and k.is_cuda and v.is_cuda
                and _supported_by_fused_path(q, k, v, mask, drop, causal)
                and q.dtype == k.dtype == v.dtype
                and (q.shape[1] == k.shape[1] or bound.get("enable_gqa", False))
            ):
                return scaled_dot_product_attention(q, k, v, mask, drop, causal, bound.get("scale"), True)
        return func(*args, **kwargs)


def enable_sdpa_routing() -> None:
    """Make plain ``F.scaled_dot_product_attention`` on CUDA tensors reach the fused op
    for inputs this build serves -- the role upstream's ``_fused_sdp_choice`` stub plays
    for its device (``SdpBackendSelection.cpp:14-75``).  For CUDA tensors torch asks its
    built-in choice function directly and never the dispatcher, so the decision is made
    one level up, in a torch-function mode installed for the rest of the process.
    Opt-in.  Tensors that need autograd are routed as well: the ATen op's derivative
    formula calls the backward op registered beside the forward."""
    global _ROUTING
    register_aten_override()
    if _ROUTING is not None:
        return
    mode = _SdpaRouting()
    mode.__enter__()
    _ROUTING = mode


# ----------------------------------------------------------------------------
# user-facing function
# ----------------------------------------------------------------------------


class _AttentionWithKeyLengths(torch.autograd.Function):
    """Autograd for the one call shape the ATen op cannot express: per-batch valid key
    counts instead of a mask.  Forward and backward are the same two foreign calls the
    ATen ops make."""

    @staticmethod
    def forward(ctx, query, key, value, kv_lens, is_causal, scale):
        out, lse = sdpa_forward(query, key, value, is_causal=is_causal, scale=scale, kv_lens=kv_lens, need_lse=True)
        ctx.save_for_backward(query, key, value, out, lse, kv_lens)
        ctx.is_causal, ctx.scale = is_causal, scale
        return out

    @staticmethod
    def backward(ctx, grad_out):
        query, key, value, out, lse, kv_lens = ctx.saved_tensors
        gq, gk, gv, _ = sdpa_backward(grad_out, query, key, value, out, lse, is_causal=ctx.is_causal,
                                      scale=ctx.scale, kv_lens=kv_lens)
        return gq, gk, gv, None, None, None


_recognise_masks = True


def set_mask_recognition(enabled: bool) -> None:
    """Switch the examination of dense boolean masks (see ``masks.classify_mask``) on or
    off for :func:`scaled_dot_product_attention` and the routed functional call."""
    global _recognise_masks
    _recognise_masks = bool(enabled)


def scaled_dot_product_attention(
    query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False, *, kv_lens=None
):
    """Drop-in for ``torch.nn.functional.scaled_dot_product_attention`` on CUDA tensors.

    ``enable_gqa`` is accepted for signature parity; grouped heads are detected from
    the shapes (``Hq % Hkv == 0``) and never expanded in memory.  ``kv_lens``
    (int32 ``(B,)``) is the one extension: valid keys per batch for right padding or
    a ragged cache, instead of a dense mask."""
    _validate(query, key, value, attn_mask, dropout_p, is_causal, False)
    if not enable_gqa and query.shape[1] != key.shape[1]:
        raise RuntimeError("SDPA: number of heads differ between query and key; pass enable_gqa=True")
    if (
        _recognise_masks and attn_mask is not None and attn_mask.dtype == torch.bool and kv_lens is None
        and not torch.cuda.is_current_stream_capturing()
    ):
        # a dense mask that only says "causal" and/or "right padding" keeps the tensor-core kernels
        found = masks.classify_mask(attn_mask, query.shape[0], query.shape[2], key.shape[2])
        if found.recognised:
            attn_mask, is_causal, kv_lens = None, found.is_causal, found.kv_lens
    if kv_lens is None:
        return torch.ops.aten._scaled_dot_product_fused_attention_overrideable(
            query, key, value, attn_mask, dropout_p, is_causal, False, scale=scale
        )[0]
    in_dtype = query.dtype
    if in_dtype == torch.float64:
        query, key, value = query.float(), key.float(), value.float()
    if attn_mask is None:
        out = _AttentionWithKeyLengths.apply(query, key, value, kv_lens, bool(is_causal), scale)
    else:
        if torch.is_grad_enabled() and (query.requires_grad or key.requires_grad or value.requires_grad):
            raise NotImplementedError("kv_lens together with attn_mask is forward-only; fold the lengths into the mask")
        bias = _additive_bias(attn_mask, query)
        out, _ = sdpa_forward(query, key, value, attn_bias=bias, is_causal=is_causal, scale=scale, kv_lens=kv_lens,
                              need_lse=False)
    return out.double() if in_dtype == torch.float64 else out
