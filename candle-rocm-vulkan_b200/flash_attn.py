"""Attention over dense (uncompressed) K / V: the host mirror of `candle-nn/src/flash_attn.rs` and of
the `candle-flash-attn` shim (candle-flash-attn/src/lib.rs:149-520) on top of b200_flash_attn.

Layouts follow the reference: `q: (batch, seq_q, heads_q, head_dim)`, `k` / `v: (batch, seq_kv,
heads_kv, head_dim)`; varlen: `(total, heads, head_dim)` with cumulative u32 offsets. Tensors may be
strided views (only the last dim must be contiguous); the result is contiguous in `q`'s layout.
There is no unfused fallback here: a call the kernel does not cover raises (the behaviour of the
reference under `strict`, flash_attn.rs:529-540).
"""
import ctypes as C
from typing import Optional

import numpy as np
import torch

from . import _abi as A
from .turbo_quant import FlashAttnConfig, TurboQuantizer, _dtype_id, _need_cuda, _stream, _workspace

_FP8 = getattr(torch, "float8_e4m3fn", None)


def _kv_dtype_id(t: torch.Tensor) -> int:
    if _FP8 is not None and t.dtype == _FP8:
        return A.FP8
    if t.dtype == torch.uint8:  # raw E4M3 bytes
        return A.FP8
    return _dtype_id(t)


def _alibi(cfg: FlashAttnConfig, q: torch.Tensor, b: int, hq: int):
    if cfg.alibi_slopes is None:
        return None, 0
    al = cfg.alibi_slopes.to(device=q.device, dtype=torch.float32).contiguous()
    if al.shape == (hq,):
        return al, 0
    if al.shape == (b, hq):
        return al, hq
    raise ValueError(f"flash-attn: alibi slopes must be ({hq}) or ({b}, {hq}), got {tuple(al.shape)}")


def _fa_args(q, k, v, cfg: FlashAttnConfig, cu_q=None, cu_k=None, max_q=0, max_k=0):
    for t, what in ((q, "q"), (k, "k"), (v, "v")):
        _need_cuda(t, what)
    varlen = cu_q is not None
    if varlen:
        if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
            raise ValueError("flash-attn varlen: q, k, v must be (total, heads, head_dim)")
        total_q, hq, d = q.shape
        total_k, hkv, dk = k.shape
        b = cu_q.numel() - 1
        if cu_k.numel() != b + 1 or b < 1:
            raise ValueError("flash-attn varlen: seqlens_q and seqlens_k must both have batch + 1 entries")
        lq, lk = int(max_q), int(max_k)
        qs = (0, q.stride(0), q.stride(1))
        ks = (0, k.stride(0), k.stride(1))
        vs = (0, v.stride(0), v.stride(1))
        out = torch.empty((total_q, hq, d), dtype=q.dtype, device=q.device)
    else:
        if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
            raise ValueError("flash-attn: q, k, v must be (batch, seq, heads, head_dim)")
        b, lq, hq, d = q.shape
        bk, lk, hkv, dk = k.shape
        if bk != b or v.shape[0] != b:
            raise ValueError(f"flash-attn: batch sizes differ: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}")
        total_q = b * lq
        qs, ks, vs = q.stride()[:3], k.stride()[:3], v.stride()[:3]
        out = torch.empty((b, lq, hq, d), dtype=q.dtype, device=q.device)
    if tuple(v.shape) != tuple(k.shape) or dk != d:
        raise ValueError(f"flash-attn: shapes do not match: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}")
    if hkv == 0 or hq % hkv != 0:
        raise ValueError(f"flash-attn: {hq} query heads are not a multiple of {hkv} kv heads")
    if cfg.softcap is not None and not cfg.softcap > 0.0:
        raise ValueError("flash-attn: softcap must be > 0")
    if q.stride(-1) != 1:
        q = q.contiguous()
        qs = (0, q.stride(0), q.stride(1)) if varlen else q.stride()[:3]
    if k.stride(-1) != 1 or v.stride(-1) != 1:
        raise ValueError("flash-attn: k and v must be contiguous along the head dim")
    alibi, abs_ = _alibi(cfg, q, b, hq)
    wl, wr = cfg.window_i32()
    a = A.FaArgs()
    a.q, a.k, a.v, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.q_dtype, a.kv_dtype = _dtype_id(q), _kv_dtype_id(k)
    if varlen:
        cu_q = cu_q.to(device=q.device, dtype=torch.int32).contiguous()  # same bits as u32 below 2^31
        cu_k = cu_k.to(device=q.device, dtype=torch.int32).contiguous()
        a.cu_q, a.cu_k = cu_q.data_ptr(), cu_k.data_ptr()
    a.b, a.lq, a.lk, a.hq, a.hkv, a.d = b, lq, lk, hq, hkv, d
    a.q_strides, a.k_strides, a.v_strides = A.u64x3(*qs), A.u64x3(*ks), A.u64x3(*vs)
    a.scale, a.softcap = cfg.softmax_scale, cfg.softcap or 0.0
    a.wl, a.wr = wl, wr
    a.k_descale, a.v_descale = cfg.k_descale, cfg.v_descale
    a.alibi, a.alibi_bstride = (alibi.data_ptr() if alibi is not None else None), abs_
    a.varlen, a.total_q = int(varlen), total_q
    nbytes = A.lib().b200_flash_attn_workspace_bytes(C.byref(a))
    ws = _workspace(q.device, nbytes) if nbytes else None
    a.workspace, a.workspace_bytes = (ws.data_ptr(), ws.numel()) if ws is not None else (None, 0)
    keep = (q, k, v, cu_q, cu_k, alibi, ws)
    return a, out, keep


def flash_attn_with_config(q, k, v, cfg: FlashAttnConfig) -> torch.Tensor:
    """candle-nn/src/flash_attn.rs:544-551."""
    a, out, _keep = _fa_args(q, k, v, cfg)
    A.check(A.lib().b200_flash_attn(C.byref(a), _stream(q.device)))
    return out


def flash_attn(q, k, v, softmax_scale: float, causal: bool) -> torch.Tensor:
    """candle-flash-attn/src/lib.rs:149-157."""
    cfg = FlashAttnConfig(softmax_scale)
    return flash_attn_with_config(q, k, v, cfg.causal() if causal else cfg)


def flash_attn_windowed(q, k, v, softmax_scale: float, window_size_left: Optional[int], window_size_right: Optional[int]):
    """candle-flash-attn/src/lib.rs:161-178 (`None` = unbounded; left None + right 0 = causal)."""
    return flash_attn_with_config(q, k, v, FlashAttnConfig(softmax_scale).window(window_size_left, window_size_right))


def flash_attn_alibi(q, k, v, alibi_slopes, softmax_scale: float, causal: bool):
    """candle-flash-attn/src/lib.rs:181-198."""
    cfg = FlashAttnConfig(softmax_scale, alibi_slopes=alibi_slopes)
    return flash_attn_with_config(q, k, v, cfg.causal() if causal else cfg)


def flash_attn_alibi_windowed(q, k, v, alibi_slopes, softmax_scale: float, window_size_left, window_size_right):
    """candle-flash-attn/src/lib.rs:201-220."""
    cfg = FlashAttnConfig(softmax_scale, alibi_slopes=alibi_slopes).window(window_size_left, window_size_right)
    return flash_attn_with_config(q, k, v, cfg)


def flash_attn_alibi_windowed_softcap(q, k, v, alibi_slopes, softmax_scale: float, window_size_left, window_size_right,
                                      softcap: float):
    """candle-flash-attn/src/lib.rs:223-260: softcap 0 disables the cap."""
    cfg = FlashAttnConfig(softmax_scale, alibi_slopes=alibi_slopes, softcap=softcap if softcap > 0.0 else None)
    return flash_attn_with_config(q, k, v, cfg.window(window_size_left, window_size_right))


def flash_attn_bhsd(q, k, v, cfg: FlashAttnConfig) -> torch.Tensor:
    """(batch, heads, seq, head_dim) in and out, through transposed views (flash_attn.rs:583-596)."""
    return flash_attn_with_config(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), cfg).transpose(1, 2)


def flash_attn_varlen_with_config(q, k, v, seqlens_q, seqlens_k, max_seqlen_q: int, max_seqlen_k: int, cfg: FlashAttnConfig):
    """candle-nn/src/flash_attn.rs:841-862."""
    a, out, _keep = _fa_args(q, k, v, cfg, seqlens_q, seqlens_k, max_seqlen_q, max_seqlen_k)
    A.check(A.lib().b200_flash_attn(C.byref(a), _stream(q.device)))
    return out


def flash_attn_varlen(q, k, v, seqlens_q, seqlens_k, max_seqlen_q: int, max_seqlen_k: int, softmax_scale: float, causal: bool):
    """candle-flash-attn/src/lib.rs:278-303."""
    cfg = FlashAttnConfig(softmax_scale)
    return flash_attn_varlen_with_config(q, k, v, seqlens_q, seqlens_k, max_seqlen_q, max_seqlen_k, cfg.causal() if causal else cfg)


def flash_attn_varlen_windowed(q, k, v, seqlens_q, seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale,
                               window_size_left, window_size_right):
    """candle-flash-attn/src/lib.rs:306-340."""
    cfg = FlashAttnConfig(softmax_scale).window(window_size_left, window_size_right)
    return flash_attn_varlen_with_config(q, k, v, seqlens_q, seqlens_k, max_seqlen_q, max_seqlen_k, cfg)


def flash_attn_varlen_alibi(q, k, v, alibi_slopes, seqlens_q, seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal):
    """candle-flash-attn/src/lib.rs:424-450."""
    cfg = FlashAttnConfig(softmax_scale, alibi_slopes=alibi_slopes)
    return flash_attn_varlen_with_config(q, k, v, seqlens_q, seqlens_k, max_seqlen_q, max_seqlen_k, cfg.causal() if causal else cfg)


def _check_blocks(blocks, batch: int, what: str):
    """Shapes of paged blocks against (batch, kv_heads, _, row) of the first one; returns (kv_heads, total rows)
    (candle-nn/src/flash_attn.rs:650-689)."""
    if len(blocks) == 0:
        raise ValueError(f"{what}: no blocks")
    _, hkv, _, kw = blocks[0].k.shape
    vw = blocks[0].v.shape[3]
    lk = 0
    for i, blk in enumerate(blocks):
        bk, hk, ck, wk = blk.k.shape
        bv, hv, cv, wv = blk.v.shape
        if bk != batch or bv != batch or hk != hkv or hv != hkv or wk != kw or wv != vw:
            raise ValueError(f"{what}: block {i} k {tuple(blk.k.shape)} / v {tuple(blk.v.shape)} do not match batch {batch}, "
                             f"{hkv} kv heads, rows of {kw} / {vw}")
        if blk.rows > ck or blk.rows > cv:
            raise ValueError(f"{what}: block {i} has {blk.rows} rows but capacities {ck} / {cv}")
        if blk.k.dtype != blocks[0].k.dtype or blk.v.dtype != blocks[0].v.dtype:
            raise ValueError(f"{what}: block {i} has another dtype than block 0")
        lk += blk.rows
    if lk == 0:
        raise ValueError(f"{what}: the blocks hold no keys")
    return hkv, lk


def flash_attn_blocks(q, blocks, cfg: FlashAttnConfig) -> torch.Tensor:
    """Attention of `q: (batch, q_heads, seq_q, head_dim)` over the dense K / V of paged cache blocks (`KvBlockRef` with
    (batch, kv_heads, capacity, head_dim) tensors of which the first `rows` positions are valid); masks, soft-capping
    and ALiBi are bottom-right aligned over the concatenated keys; output (batch, q_heads, seq_q, head_dim) in the query
    dtype (candle-nn/src/flash_attn.rs:691-727). The blocks are read where they are (b200_flash_attn_paged: a block table
    in device memory, any number of blocks and of query tokens; the reference's in-place kernel serves up to 4 query
    tokens and 128 blocks and concatenates otherwise). Blocks that the kernel cannot read in place (rows that are not
    contiguous along the head dim or do not start on 16-byte boundaries, row strides that differ between blocks) are
    concatenated on the device and the call runs `flash_attn_bhsd`."""
    if q.dim() != 4:
        raise ValueError(f"flash-attn blocks: q must be (batch, q_heads, seq_q, head_dim), got {tuple(q.shape)}")
    b, hq, lq, d = q.shape
    hkv, lk = _check_blocks(blocks, b, "flash-attn blocks")
    if blocks[0].k.shape[3] != d or blocks[0].v.shape[3] != d:
        raise ValueError(f"flash-attn blocks: k {tuple(blocks[0].k.shape)} / v {tuple(blocks[0].v.shape)} do not match the head dim {d} of q")
    live = [blk for blk in blocks if blk.rows > 0]

    def in_place(t, ref):
        # layout of paged_block_layout (flash_attn.rs:618-646): contiguous last dim, head stride = whole rows, batch
        # stride = kv_heads head strides, one row stride for all blocks
        return (t.is_cuda and t.device == q.device and t.stride(3) == 1 and t.stride(2) == ref.stride(2)
                and t.stride(1) == t.shape[2] * t.stride(2) and t.stride(0) == t.shape[1] * t.stride(1)
                and t.data_ptr() % 16 == 0 and (t.stride(2) * t.element_size()) % 16 == 0)

    if not all(in_place(blk.k, live[0].k) and in_place(blk.v, live[0].v) for blk in live) or hq % hkv != 0:
        if len(live) == 1:
            k, v = live[0].k[:, :, : live[0].rows], live[0].v[:, :, : live[0].rows]
        else:
            k = torch.cat([blk.k[:, :, : blk.rows].to(q.device) for blk in live], dim=2)
            v = torch.cat([blk.v[:, :, : blk.rows].to(q.device) for blk in live], dim=2)
        return flash_attn_bhsd(q, k, v, cfg)
    _need_cuda(q, "q")
    if cfg.softcap is not None and not cfg.softcap > 0.0:
        raise ValueError("flash-attn: softcap must be > 0")
    qt = q.transpose(1, 2)  # (batch, seq, heads, head_dim) view, as the C ABI describes queries
    if qt.stride(-1) != 1:
        qt = qt.contiguous()
    out = torch.empty((b, lq, hq, d), dtype=q.dtype, device=q.device)
    table = np.zeros(len(live), dtype=np.dtype([("k", "<u8"), ("v", "<u8"), ("rows", "<u4"), ("k_cap", "<u4"), ("v_cap", "<u4"), ("pad", "<u4")]))
    for n, blk in enumerate(live):
        table[n] = (blk.k.data_ptr(), blk.v.data_ptr(), blk.rows, blk.k.shape[2], blk.v.shape[2], 0)
    pages = torch.from_numpy(table.view(np.uint8)).to(q.device)
    alibi, abs_ = _alibi(cfg, qt, b, hq)
    wl, wr = cfg.window_i32()
    a = A.FaArgs()
    a.q, a.k, a.v, a.o = qt.data_ptr(), None, None, out.data_ptr()
    a.q_dtype, a.kv_dtype = _dtype_id(qt), _kv_dtype_id(live[0].k)
    a.b, a.lq, a.lk, a.hq, a.hkv, a.d = b, lq, lk, hq, hkv, d
    a.q_strides = A.u64x3(*qt.stride()[:3])
    a.k_strides, a.v_strides = A.u64x3(0, live[0].k.stride(2), 0), A.u64x3(0, live[0].v.stride(2), 0)
    a.scale, a.softcap = cfg.softmax_scale, cfg.softcap or 0.0
    a.wl, a.wr = wl, wr
    a.k_descale, a.v_descale = cfg.k_descale, cfg.v_descale
    a.alibi, a.alibi_bstride = (alibi.data_ptr() if alibi is not None else None), abs_
    a.varlen, a.total_q = 0, b * lq
    nbytes = A.lib().b200_flash_attn_paged_workspace_bytes(C.byref(a), len(live))
    if nbytes == 0:
        A.check(A.lib().b200_flash_attn_paged(C.byref(a), pages.data_ptr(), len(live), _stream(q.device)))  # raises with the reason
    ws = _workspace(q.device, nbytes)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    A.check(A.lib().b200_flash_attn_paged(C.byref(a), pages.data_ptr(), len(live), _stream(q.device)))
    return out.transpose(1, 2)


def flash_attn_varlen_paged_windowed(q, k, v, seqlens_q, seqlens_k, block_table, mm_prefix_ranges, max_seqlen_q: int, max_seqlen_k: int,
                                     softmax_scale: float, window_size_left: Optional[int], window_size_right: Optional[int],
                                     page_block_size: int, softcap: Optional[float] = None) -> torch.Tensor:
    """Variable length attention over a paged KV cache: `k`, `v` are (num_blocks, page_block_size, kv_heads, head_dim) and
    `block_table` (batch, max_blocks_per_seq) lists the blocks of each sequence; `seqlens_q` / `seqlens_k` are the
    cumulative lengths of the varlen calls. The pages of every sequence are gathered, then the varlen kernel runs
    (candle-flash-attn/src/lib.rs:341-420, which gathers on the host sequence by sequence; here one index over all
    tokens is built on the device). `mm_prefix_ranges` is not supported, as in the reference."""
    if mm_prefix_ranges is not None:
        raise ValueError("flash-attn: mm_prefix_ranges is not supported by this implementation")
    if k.dim() != 4 or v.shape != k.shape:
        raise ValueError(f"flash-attn: paged k / v must be (num_blocks, page, kv_heads, head_dim), got {tuple(k.shape)} / {tuple(v.shape)}")
    nblk, page, hkv, d = k.shape
    if page != page_block_size:
        raise ValueError(f"flash-attn: k has pages of {page} tokens, page_block_size is {page_block_size}")
    batch = seqlens_k.numel() - 1
    if block_table.dim() != 2 or block_table.shape[0] < batch:
        raise ValueError(f"flash-attn: block_table has {block_table.shape[0] if block_table.dim() == 2 else 0} rows for {batch} sequences")
    cu = seqlens_k.to(device=k.device, dtype=torch.int64).clamp_min(0)
    lens = cu[1:] - cu[:-1]
    total, longest = (int(x) for x in torch.stack([cu[-1], lens.max() if batch > 0 else cu[-1]]).tolist())
    need = (longest + page - 1) // page
    if need > block_table.shape[1]:
        raise ValueError(f"flash-attn: a sequence needs {need} blocks, block_table has {block_table.shape[1]}")
    pos = torch.arange(total, device=k.device, dtype=torch.int64)
    seq = torch.searchsorted(cu[1:].contiguous(), pos, right=True)
    off = pos - cu[seq]
    blk = block_table.to(device=k.device, dtype=torch.int64)[seq, off // page]
    rows = blk * page + off % page
    kf = k.reshape(nblk * page, hkv, d).index_select(0, rows)
    vf = v.reshape(nblk * page, hkv, d).index_select(0, rows)
    cfg = FlashAttnConfig(softmax_scale, softcap=softcap if softcap is not None and softcap > 0.0 else None)
    cfg = cfg.window(window_size_left, window_size_right)
    return flash_attn_varlen_with_config(q, kf, vf, seqlens_q, seqlens_k, max_seqlen_q, max_seqlen_k, cfg)


def flash_attn_fp8(q, k, v, cfg: FlashAttnConfig) -> torch.Tensor:
    """K and V rounded to E4M3 with one scale per tensor (amax / 448), queries kept in their dtype
    (candle-nn/src/flash_attn.rs:867-894, without the optional Hadamard pre-rotation)."""
    if _FP8 is None:
        raise RuntimeError("flash_attn_fp8 needs torch.float8_e4m3fn")

    def quant(x):
        x32 = x.float()
        amax = float(x32.abs().max())
        scale = amax / 448.0 if amax > 0.0 else 1.0
        return (x32 / scale).to(_FP8), scale

    k8, ks = quant(k)
    v8, vs = quant(v)
    c = FlashAttnConfig(cfg.softmax_scale, cfg.window_size_left, cfg.window_size_right, cfg.softcap, cfg.alibi_slopes,
                        cfg.k_descale * ks, cfg.v_descale * vs, cfg.splits)
    return flash_attn_with_config(q, k8, v8, c)


def prefill_append(q, k, v, cfg: FlashAttnConfig, k_cache, v_cache, kq: TurboQuantizer, vq: TurboQuantizer, pos):
    """One call for a prefill chunk: attention of `q` over the uncompressed `k` / `v` ((batch, seq,
    heads, head_dim)) and the packed rows of `k` / `v` written at `pos` of the (batch, kv_heads,
    capacity, words) caches. Replaces `flash_attn(q, k, v, scale, causal)` followed by
    `TurboKvCache::append` (candle-nn/src/turbo_quant.rs:916-945)."""
    a, out, _keep = _fa_args(q, k, v, cfg)
    b, t, hkv, d = k.shape
    kt, vt = k.transpose(1, 2), v.transpose(1, 2)  # (b, hkv, t, d) views of the same memory
    pos_t = pos if isinstance(pos, torch.Tensor) else None
    ap = A.KvAppendArgs(
        kt.data_ptr(), vt.data_ptr(), A.u64x3(*kt.stride()[:3]), A.u64x3(*vt.stride()[:3]),
        k_cache.data_ptr(), v_cache.data_ptr(), A.u64x3(*k_cache.stride()[:3]), A.u64x3(*v_cache.stride()[:3]),
        pos_t.data_ptr() if pos_t is not None else None, 0 if pos_t is not None else int(pos),
        b, hkv, t, d, _dtype_id(k), kq.side(), vq.side())
    A.check(A.lib().b200_fa_prefill_append(C.byref(a), C.byref(ap), _stream(q.device)))
    return out
