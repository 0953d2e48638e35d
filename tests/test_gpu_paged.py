"""Decode against a paged key/value cache: same numbers as the dense cache it was cut
from (the kernel arithmetic is identical, only row addresses differ), oracle parity, both
pool layouts, ragged lengths, pages in random order."""

import pytest
import torch

from oracle import sdpa_oracle as O
from tests.util import check_against_oracle

pytestmark = pytest.mark.gpu


def _paged_copy(k, v, lens, page_size, layout, seed):
    """Scatter a dense (B, Hkv, S, D) cache into shuffled pages; returns pools + block table."""
    B, Hkv, S, D = k.shape
    max_pages = (S + page_size - 1) // page_size
    g = torch.Generator().manual_seed(seed)
    n_pages = B * max_pages + 3
    order = torch.randperm(n_pages, generator=g)[: B * max_pages].view(B, max_pages).to(torch.int32)
    kp = torch.full((n_pages, page_size, Hkv, D), float("nan"), dtype=k.dtype)
    vp = torch.full((n_pages, page_size, Hkv, D), float("nan"), dtype=k.dtype)
    for b in range(B):
        for pg in range((int(lens[b]) + page_size - 1) // page_size):
            rows = slice(pg * page_size, min((pg + 1) * page_size, S))
            n = rows.stop - rows.start
            kp[order[b, pg], :n] = k[b, :, rows].transpose(0, 1)
            vp[order[b, pg], :n] = v[b, :, rows].transpose(0, 1)
    if layout == "HND":
        kp, vp = kp.transpose(1, 2).contiguous(), vp.transpose(1, 2).contiguous()
    return kp, vp, order


@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("page_size", [16, 128])
@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float16, 64)])
def test_paged_decode_matches_dense_and_oracle(dtype, D, page_size, layout):
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(5)
    B, Hq, Hkv, S = 5, 16, 4, 1000
    q = torch.randn(B, Hq, 1, D, generator=g).to(dtype)
    k = torch.randn(B, Hkv, S, D, generator=g).to(dtype)
    v = torch.randn(B, Hkv, S, D, generator=g).to(dtype)
    lens = torch.tensor([1000, 1, 517, 0, 256], dtype=torch.int32)
    kp, vp, table = _paged_copy(k, v, lens, page_size, layout, seed=9)
    T.reset_launch_counts()
    out, lse = T.paged_decode(q.to(dev), kp.to(dev), vp.to(dev), table.to(dev), lens.to(dev), layout=layout,
                              need_lse=True)
    torch.cuda.synchronize()
    T.check_device_status()
    counts = T.launch_counts()
    assert counts["decode_partial"] == 1 and counts["decode_combine"] == 1 and counts["generic"] == 0
    check_against_oracle(q, k, v, out.cpu(), lse.cpu(), kv_lens=lens, tag=f"paged {layout} page={page_size}")
    # the dense cache with the same split geometry gives the same bits
    S_table = table.shape[1] * page_size
    kd = torch.zeros(B, Hkv, S_table, D, dtype=dtype)
    vd = torch.zeros(B, Hkv, S_table, D, dtype=dtype)
    kd[:, :, :S], vd[:, :, :S] = k, v
    dense_o, dense_l = T.sdpa_forward(q.to(dev), kd.to(dev), vd.to(dev), kv_lens=lens.to(dev))
    torch.cuda.synchronize()
    assert torch.equal(out, dense_o) and torch.equal(lse.nan_to_num(neginf=-1.0), dense_l.nan_to_num(neginf=-1.0))


def test_paged_decode_rejects_what_it_cannot_serve():
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    q = torch.zeros(2, 8, 1, 128, dtype=torch.bfloat16, device=dev)
    pool = torch.zeros(4, 16, 2, 128, dtype=torch.bfloat16, device=dev)
    table = torch.zeros(2, 2, dtype=torch.int32, device=dev)
    lens = torch.tensor([5, 7], dtype=torch.int32, device=dev)
    with pytest.raises(RuntimeError, match="float16 or bfloat16"):
        T.paged_decode(q.float(), pool.float(), pool.float(), table, lens)
    with pytest.raises(RuntimeError, match="block_table"):
        T.paged_decode(q, pool, pool, table.long(), lens)
    with pytest.raises(RuntimeError):   # page size that is not a power of two
        T.paged_decode(q, pool[:, :12], pool[:, :12], table, lens)


@pytest.mark.parametrize("paged", [False, True])
def test_decode_with_fused_append(paged):
    """A short generation loop: every step attends to the cache plus the new token's row and the kernel
    itself writes that row into the cache.  Outputs must match the oracle on the grown cache, and after
    the loop the cache must hold exactly the rows that were appended."""
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(17)
    B, Hq, Hkv, D, S, page = 4, 16, 4, 128, 320, 16
    lens = torch.tensor([0, 63, 200, 318], dtype=torch.int32)
    k_full = torch.randn(B, Hkv, S, D, generator=g).to(torch.bfloat16)   # the rows the sequence will have
    v_full = torch.randn(B, Hkv, S, D, generator=g).to(torch.bfloat16)
    k_cache, v_cache = k_full.clone(), v_full.clone()
    for b in range(B):                                                   # not yet appended: poison
        k_cache[b, :, int(lens[b]):] = float("nan")
        v_cache[b, :, int(lens[b]):] = float("nan")
    if paged:
        max_pages = S // page
        table = torch.randperm(B * max_pages, generator=g).view(B, max_pages).to(torch.int32)
        kp = torch.empty(B * max_pages, page, Hkv, D, dtype=torch.bfloat16)
        vp = torch.empty_like(kp)
        for b in range(B):
            for pg in range(max_pages):
                kp[table[b, pg]] = k_cache[b, :, pg * page:(pg + 1) * page].transpose(0, 1)
                vp[table[b, pg]] = v_cache[b, :, pg * page:(pg + 1) * page].transpose(0, 1)
        kc, vc, tb = kp.to(dev), vp.to(dev), table.to(dev)
    else:
        kc, vc = k_cache.to(dev), v_cache.to(dev)
    cur = lens.clone().to(dev)
    for step in range(3):
        q = torch.randn(B, Hq, 1, D, generator=g).to(torch.bfloat16)
        pos = cur.cpu().long().clamp(max=S - 1)
        k_new = torch.stack([k_full[b, :, pos[b]] for b in range(B)])   # (B, Hkv, D)
        v_new = torch.stack([v_full[b, :, pos[b]] for b in range(B)])
        if paged:
            out, lse, new = T.paged_decode(q.to(dev), kc, vc, tb, cur, need_lse=True, k_new=k_new.to(dev),
                                           v_new=v_new.to(dev))
        else:
            out, lse, new = T.decode_append(q.to(dev), k_new.to(dev), v_new.to(dev), kc, vc, cur, need_lse=True)
        torch.cuda.synchronize()
        if bool((cur.cpu() >= S).any()):
            # a sequence whose cache is full drops its new row; the status word says which one
            with pytest.raises(RuntimeError, match=r"cache is full.*role=3 step=320 extra=320"):
                T.check_device_status()
        else:
            T.check_device_status()
        want_lens = (cur.cpu() + 1).clamp(max=S)
        assert torch.equal(new.cpu(), want_lens)
        check_against_oracle(q, k_full, v_full, out.cpu(), lse.cpu(), kv_lens=want_lens, tag=f"append step {step}")
        cur = new
    final = cur.cpu()
    assert final.tolist() == [3, 66, 203, 320]      # the last sequence filled its cache after two steps
    if paged:
        dense_k = torch.stack([torch.cat([kc[tb[b, pg]].transpose(0, 1) for pg in range(S // page)], dim=1)
                               for b in range(B)]).cpu()
    else:
        dense_k = kc.cpu()
    for b in range(B):
        n = int(final[b])
        assert torch.equal(dense_k[b, :, :n], k_full[b, :, :n])          # appended rows are in the cache
        assert torch.isnan(dense_k[b, :, n:].float()).all()               # and nothing beyond them was touched


def _rope(x, cos, sin, interleaved):
    """fp32 rotary embedding of the last dimension; cos/sin are (..., D/2) broadcastable."""
    x = x.float()
    if interleaved:
        a, b = x[..., 0::2], x[..., 1::2]
        out = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1).flatten(-2)
    else:
        h = x.shape[-1] // 2
        a, b = x[..., :h], x[..., h:]
        out = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
    return out


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float16, 64)])
def test_decode_append_with_fused_rotary_embedding(dtype, D, interleaved):
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(31)
    B, Hq, Hkv, S = 3, 8, 2, 200
    lens = torch.tensor([0, 77, 150], dtype=torch.int32)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.arange(S).float()[:, None] * inv_freq[None, :]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()                 # (S, D/2) fp32
    q = torch.randn(B, Hq, 1, D, generator=g).to(dtype)
    k_cache = torch.randn(B, Hkv, S, D, generator=g).to(dtype)                 # already rotated rows, as a cache holds
    v_cache = torch.randn(B, Hkv, S, D, generator=g).to(dtype)
    k_new = torch.randn(B, Hkv, D, generator=g).to(dtype)
    v_new = torch.randn(B, Hkv, D, generator=g).to(dtype)
    kc, vc = k_cache.to(dev), v_cache.to(dev)
    out, lse, new = T.decode_append(q.to(dev), k_new.to(dev), v_new.to(dev), kc, vc, lens.to(dev), need_lse=True,
                                    rope_cos=cos.to(dev), rope_sin=sin.to(dev), rope_interleaved=interleaved)
    torch.cuda.synchronize()
    T.check_device_status()
    # reference: rotate in fp32, round once, append, attend
    pos = lens.long()
    q_rot = _rope(q, cos[pos][:, None, None, :], sin[pos][:, None, None, :], interleaved).to(dtype)
    k_rot = _rope(k_new, cos[pos][:, None, :], sin[pos][:, None, :], interleaved).to(dtype)
    k_ref, v_ref = k_cache.clone(), v_cache.clone()
    for b in range(B):
        k_ref[b, :, pos[b]] = k_rot[b]
        v_ref[b, :, pos[b]] = v_new[b]
    check_against_oracle(q_rot, k_ref, v_ref, out.cpu(), lse.cpu(), kv_lens=lens + 1, tag=f"rope interleaved={interleaved}")
    assert new.cpu().tolist() == (lens + 1).tolist()
    for b in range(B):
        assert torch.equal(kc[b, :, pos[b]].cpu(), k_rot[b])                    # the cache holds the rotated key
        assert torch.equal(vc[b, :, pos[b]].cpu(), v_new[b])


def test_rotary_tables_must_cover_the_cache():
    """The rotary tables are indexed by the sequence length: the host layer refuses tables shorter than
    the cache, and through the C ABI a length beyond the tables uses their last row instead of reading
    past them."""
    import ctypes as C

    import torch_neuronx_b200 as T
    from torch_neuronx_b200 import _lib

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(5)
    B, Hq, Hkv, S, D = 2, 4, 2, 64, 64
    q = torch.randn(B, Hq, 1, D, generator=g).to(torch.bfloat16).to(dev)
    kc = torch.randn(B, Hkv, S, D, generator=g).to(torch.bfloat16).to(dev)
    vc = torch.randn(B, Hkv, S, D, generator=g).to(torch.bfloat16).to(dev)
    kn = torch.randn(B, Hkv, D, generator=g).to(torch.bfloat16).to(dev)
    vn = torch.randn(B, Hkv, D, generator=g).to(torch.bfloat16).to(dev)
    lens = torch.tensor([10, 40], dtype=torch.int32, device=dev)
    short = torch.randn(32, D // 2, generator=g).to(dev)           # 32 positions for a 64-row cache
    with pytest.raises(RuntimeError, match="rotary tables hold 32 positions"):
        T.decode_append(q, kn, vn, kc, vc, lens, rope_cos=short, rope_sin=short)

    # straight through the C ABI with the short tables: sequence 1 (length 40) is rotated by row 31
    lib = _lib.load()
    cos, sin = short.cos().contiguous(), short.sin().contiguous()
    out = torch.full_like(q, float("nan"))
    new_lens = torch.empty_like(lens)
    p = _lib.Params()
    p.struct_size = C.sizeof(_lib.Params)
    p.dtype, p.device, p.force_path = _lib.BF16, 0, _lib.PATH_DECODE
    p.q, p.k, p.v, p.out = q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr()
    p.q_stride[:], p.k_stride[:], p.v_stride[:], p.out_stride[:] = q.stride(), kc.stride(), vc.stride(), out.stride()
    p.B, p.Hq, p.Hkv, p.L, p.S, p.E, p.Dv = B, Hq, Hkv, 1, S, D, D
    p.scale = D ** -0.5
    p.kv_lens, p.kv_lens_out = lens.data_ptr(), new_lens.data_ptr()
    p.k_new, p.v_new = kn.data_ptr(), vn.data_ptr()
    p.k_new_stride[:], p.v_new_stride[:] = kn.stride()[:2], vn.stride()[:2]
    p.rope_cos, p.rope_sin, p.rope_stride, p.rope_positions = cos.data_ptr(), sin.data_ptr(), cos.stride(0), 32
    plan = _lib.Plan()
    plan.struct_size = C.sizeof(_lib.Plan)
    assert lib.b200_sdpa_query_plan(C.byref(p), C.byref(plan)) == _lib.OK
    ws = torch.empty(max(int(plan.workspace_bytes), 16), dtype=torch.uint8, device=dev)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    assert lib.b200_sdpa_decode(C.byref(p), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)) == _lib.OK
    torch.cuda.synchronize()
    rows = torch.tensor([10, 31])
    k_rot = _rope(kn.cpu(), cos.cpu()[rows][:, None, :], sin.cpu()[rows][:, None, :], False).to(torch.bfloat16)
    for b, pos in enumerate((10, 40)):
        assert torch.equal(kc[b, :, pos].cpu(), k_rot[b])
    p.rope_positions = 0
    assert lib.b200_sdpa_query_plan(C.byref(p), C.byref(plan)) == _lib.ERR_SHAPE
