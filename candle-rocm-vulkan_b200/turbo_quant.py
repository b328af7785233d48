"""Host-side mirror of the reference's compressed KV cache API over libb200attn.so.

Names, argument meaning and error behaviour follow candle-nn/src/turbo_quant.rs
(`TurboQuantizer`, `QuantizedTensor`, `TurboKvCache`, `attention_packed`) and
candle-nn/src/flash_attn.rs (`FlashAttnConfig`), so tests written against the reference read the
same here. torch only provides device memory and streams; every computation is a call through
the C ABI (include/b200attn.h). There is no CPU path: tensors must live on a CUDA device.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional, Tuple

import numpy as np
import torch

from . import _abi as A


class QuantFormat:
    """A quantization format: `QuantFormat.parse("mxfp4")`, `QuantFormat.turbo_mse(4)` ...
    (candle-core/src/accel/formats.rs:21-135)."""

    def __init__(self, mode: int, bits: int = 4):
        self.mode, self.bits = mode, bits

    @staticmethod
    def turbo_mse(bits=4):
        return QuantFormat(A.TURBO_MSE, bits)

    @staticmethod
    def parse(s: str) -> "QuantFormat":
        t = s.strip().lower().replace("-", "").replace("_", "").replace(" ", "")
        digits = "".join(ch for ch in t if ch.isdigit())
        name = "".join(ch for ch in t if not ch.isdigit())
        bits = int(digits) if digits else 0
        if name in ("turbo", "tq", "mse", "turbomse", "tqmse", "turboquant", "lloydmax"):
            f = QuantFormat(A.TURBO_MSE, bits or 4)
        elif name in ("prod", "turboprod", "tqprod", "qjl", "turboqjl"):
            f = QuantFormat(A.TURBO_PROD, bits or 4)
        elif name == "nvfp" and digits == "4":
            f = QuantFormat(A.NVFP4)
        elif name == "mxfp" and digits == "4":
            f = QuantFormat(A.MXFP4)
        elif name == "mxfp" and digits == "8":
            f = QuantFormat(A.MXFP8)
        elif (name in ("fp", "nvfp") and digits == "8") or (name == "em" and digits == "43"):
            f = QuantFormat(A.FP8_ROW)
        else:
            raise ValueError(f"unknown quantization format {s!r} (turbo[1-4], prod[2-5], nvfp4, mxfp4, mxfp8, fp8)")
        return f

    def name(self) -> str:
        return {A.TURBO_MSE: f"turbo-mse{self.bits}", A.TURBO_PROD: f"turbo-prod{self.bits}", A.NVFP4: "nvfp4",
                A.MXFP4: "mxfp4", A.MXFP8: "mxfp8", A.FP8_ROW: "fp8"}[self.mode]

    def is_turbo(self) -> bool:
        return self.mode <= A.TURBO_PROD

    def __repr__(self):
        return self.name()


_DTYPES = {torch.float32: A.F32, torch.float16: A.F16, torch.bfloat16: A.BF16}


def _dtype_id(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {t.dtype} (f32, f16, bf16)") from None


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _need_cuda(t: torch.Tensor, what: str):
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be on a CUDA device: this library has no CPU path")


@dataclass
class FlashAttnConfig:
    """Options of one attention call (candle-nn/src/flash_attn.rs:26-123)."""
    softmax_scale: float
    window_size_left: Optional[int] = None
    window_size_right: Optional[int] = None
    softcap: Optional[float] = None
    alibi_slopes: Optional[torch.Tensor] = None
    k_descale: float = 1.0
    v_descale: float = 1.0
    splits: int = 0  # key splits per sequence (SplitKv::Fixed), 0 = chosen by the library

    def causal(self):
        self.window_size_right = 0
        return self

    def window(self, left, right):
        self.window_size_left, self.window_size_right = left, right
        return self

    def window_i32(self) -> Tuple[int, int]:
        cv = lambda w: -1 if w is None else min(int(w), 2**31 - 1)
        return cv(self.window_size_left), cv(self.window_size_right)


@dataclass
class QuantizedTensor:
    """A tensor quantized row by row along its last dimension (turbo_quant.rs:39-53)."""
    data: torch.Tensor
    shape: torch.Size
    dtype: torch.dtype

    def size_in_bytes(self) -> int:
        return self.data.numel() * 4


class TurboQuantizer:
    """Quantizes vectors of a fixed length in one format (turbo_quant.rs:57-321). `rotation`: "none", "hadamard",
    "dense" or "auto"; auto resolves to hadamard for powers of two and to dense otherwise, hadamard to dense for
    lengths that are not powers of two (RotationKind::resolve, accel/config.rs:131-138). The Hadamard rotation is
    fused into the quantize and attention kernels; the dense one (a matrix product with a seeded orthonormal matrix)
    runs as its own launch before / after them, as every rotation does in the reference."""

    def __init__(self, format: QuantFormat, dim: int, rotation: str = "auto", seed: int = 42, device="cuda"):
        self.format, self.dim, self.device = format, dim, torch.device(device)
        self.layout = A.row_layout(format.mode, format.bits, dim)
        pow2 = dim & (dim - 1) == 0
        if rotation not in ("none", "hadamard", "dense", "auto"):
            raise ValueError("rotation must be none, hadamard, dense or auto")
        if rotation == "auto":
            rotation = "hadamard" if pow2 else "dense"
        if rotation == "hadamard" and not pow2:
            rotation = "dense"
        self.rotation = rotation
        self.seed = seed
        tab = (C.c_float * 32)()
        if format.is_turbo():
            # prod rows spend one of their bits on the sketch: codes of bits - 1 bits (formats.rs code_bits)
            A.check(A.lib().b200_codebook(dim, self.layout.code_bits, tab))
        self.tab = torch.tensor(list(tab), dtype=torch.float32, device=self.device)
        # prod rows: S and S^T of the 1-bit sketch of the residual (turbo_quant.rs:111-118)
        self.qjl = None
        if format.mode == A.TURBO_PROD:
            m = (C.c_float * (dim * dim))()
            A.check(A.lib().b200_qjl_matrix(dim, seed, m))
            s_mat = torch.frombuffer(m, dtype=torch.float32).view(dim, dim).to(self.device)
            self.qjl = (s_mat, s_mat.t().contiguous())
        self.pi = None
        if rotation == "dense":
            m = (C.c_float * (dim * dim))()
            A.check(A.lib().b200_rotation_matrix(dim, seed, m))
            self.pi = torch.frombuffer(m, dtype=torch.float32).view(dim, dim).to(self.device)
        self.signs = None
        if rotation == "hadamard":
            s = (C.c_float * dim)()
            A.check(A.lib().b200_hadamard_signs(dim, seed, s))
            self.signs = torch.tensor(list(s), dtype=torch.float32, device=self.device)

    def row_words(self) -> int:
        return self.layout.row_words

    def side(self) -> A.QuantSide:
        return A.QuantSide(self.format.mode, self.format.bits, self.tab.data_ptr(),
                           A.ROT_HADAMARD if self.rotation == "hadamard" else A.ROT_NONE,
                           self.signs.data_ptr() if self.signs is not None else None)

    def rotate(self, x: torch.Tensor) -> torch.Tensor:
        """`x Pi^T` in f32 (turbo_quant.rs:182-188)."""
        x = x.to(torch.float32).contiguous()
        if self.rotation == "none":
            return x
        out = torch.empty_like(x)
        if self.rotation == "dense":
            A.check(A.lib().b200_tq_rotate_dense(x.data_ptr(), out.data_ptr(), self.pi.data_ptr(), x.numel() // self.dim,
                                                 self.dim, 0, _stream(x.device)))
            return out
        A.check(A.lib().b200_tq_rotate(x.data_ptr(), out.data_ptr(), self.signs.data_ptr(), x.numel() // self.dim,
                                       self.dim, 0, _stream(x.device)))
        return out

    def unrotate(self, y: torch.Tensor) -> torch.Tensor:
        """`y Pi` (turbo_quant.rs:191-196)."""
        if self.rotation == "none":
            return y
        y = y.to(torch.float32).contiguous()
        out = torch.empty_like(y)
        if self.rotation == "dense":
            A.check(A.lib().b200_tq_rotate_dense(y.data_ptr(), out.data_ptr(), self.pi.data_ptr(), y.numel() // self.dim,
                                                 self.dim, 1, _stream(y.device)))
            return out
        A.check(A.lib().b200_tq_rotate(y.data_ptr(), out.data_ptr(), self.signs.data_ptr(), y.numel() // self.dim,
                                       self.dim, 1, _stream(y.device)))
        return out

    def quantize_rotated_rows(self, y: torch.Tensor) -> torch.Tensor:
        """Rows that are already in the rotated domain -> packed rows (the reference's TqQuant op)."""
        _need_cuda(y, "rows")
        rows, d = y.shape
        if d != self.dim:
            raise ValueError(f"turbo-quant: expected rows of {self.dim} values, got {d}")
        if y.stride(1) != 1:
            y = y.contiguous()
        out = torch.empty((rows, self.layout.row_words), dtype=torch.int32, device=y.device)
        args = A.TqQuantArgs(y.data_ptr(), out.data_ptr(), self.tab.data_ptr(), rows, d, y.stride(0), 0,
                             _dtype_id(y), self.format.mode, self.format.bits)
        A.check(A.lib().b200_tq_quantize(C.byref(args), _stream(y.device)))
        return out

    def quantize_rows(self, x: torch.Tensor) -> torch.Tensor:
        """Packs `x: (rows, dim)` into `(rows, row_words)` rows, rotation included
        (turbo_quant.rs:199-212); one launch."""
        _need_cuda(x, "rows")
        rows, d = x.shape
        if d != self.dim:
            raise ValueError(f"turbo-quant: expected rows of {self.dim} values, got {d}")
        if self.qjl is not None:
            # prod rows (turbo_quant.rs:214-236): stage one, residual, projection with S^T (the host's matmul), sign bits
            y = self.rotate(x)
            packed = self.quantize_rotated_rows(y)
            resid = torch.empty((rows, d), dtype=torch.float32, device=x.device)
            ra = A.TqResidArgs(y.data_ptr(), packed.data_ptr(), self.tab.data_ptr(), resid.data_ptr(), rows, d, y.stride(0), 0,
                               A.F32, self.format.bits)
            A.check(A.lib().b200_tq_residual(C.byref(ra), _stream(x.device)))
            proj = resid.matmul(self.qjl[1])
            sa = A.TqSignsArgs(packed.data_ptr(), proj.data_ptr(), resid.data_ptr(), packed.data_ptr(), rows, d, self.format.bits)
            A.check(A.lib().b200_tq_signs(C.byref(sa), _stream(x.device)))
            return packed
        if self.rotation == "none":
            return self.quantize_rotated_rows(x)
        if self.rotation == "dense":
            return self.quantize_rotated_rows(self.rotate(x))
        out = torch.empty((1, 1, rows, self.layout.row_words), dtype=torch.int32, device=x.device)
        _kv_append(x.view(1, 1, rows, d), x.view(1, 1, rows, d), out, out.clone(), self, self, 0)
        return out.view(rows, self.layout.row_words)

    def dequantize_rows(self, data: torch.Tensor) -> torch.Tensor:
        """`(rows, row_words)` -> `(rows, dim)` f32 in the original domain (turbo_quant.rs:250-270)."""
        _need_cuda(data, "rows")
        rows, rw = data.shape
        if rw != self.layout.row_words:
            raise ValueError(f"turbo-quant: expected rows of {self.layout.row_words} words, got {rw}")
        data = data.contiguous()
        out = torch.empty((rows, self.dim), dtype=torch.float32, device=data.device)
        zs = torch.empty_like(out) if self.qjl is not None else None
        args = A.TqDequantArgs(data.data_ptr(), out.data_ptr(), self.tab.data_ptr(), rows, self.dim, 0,
                               self.format.mode, self.format.bits, zs.data_ptr() if zs is not None else None)
        A.check(A.lib().b200_tq_dequantize(C.byref(args), _stream(data.device)))
        if zs is not None:
            out = out + zs.matmul(self.qjl[0])  # the sketch's part of the estimate (turbo_quant.rs:281-284)
        return self.unrotate(out)

    def quantize(self, x: torch.Tensor) -> QuantizedTensor:
        d = x.shape[-1]
        if d != self.dim:
            raise ValueError(f"turbo-quant: expected a last dim of {self.dim}, got {d}")
        return QuantizedTensor(self.quantize_rows(x.reshape(-1, d)), x.shape, x.dtype)

    def dequantize(self, q: QuantizedTensor) -> torch.Tensor:
        return self.dequantize_rows(q.data).reshape(q.shape).to(q.dtype)


def _kv_append(k, v, k_cache, v_cache, kq: TurboQuantizer, vq: TurboQuantizer, pos, pos_add: int = 0, status=None, after_prev: bool = False):
    """b200_kv_append over (b, hkv, t, d) tensors and (b, hkv, cap, words) caches. `pos`: int or an
    int32 device tensor with one position per batch entry, to which `pos_add` is added. Rows whose
    device position falls outside the cache are skipped (`status`, an int32 device tensor, is set to 3)."""
    b, h, t, d = k.shape
    # the dense rotation is not fused: rows rotated by their own launch (f32), then appended with rotation none
    if kq.rotation == "dense":
        k = kq.rotate(k.reshape(-1, d)).view(b, h, t, d)
    if vq.rotation == "dense":
        v = vq.rotate(v.reshape(-1, d)).view(b, h, t, d)
    if k.dtype != v.dtype:
        k, v = k.to(torch.float32), v.to(torch.float32)
    if k.stride(3) != 1:
        k = k.contiguous()
    if v.stride(3) != 1:
        v = v.contiguous()
    pos_t = pos if isinstance(pos, torch.Tensor) else None
    args = A.KvAppendArgs(
        k.data_ptr(), v.data_ptr(), A.u64x3(*k.stride()[:3]), A.u64x3(*v.stride()[:3]),
        k_cache.data_ptr(), v_cache.data_ptr(), A.u64x3(*k_cache.stride()[:3]), A.u64x3(*v_cache.stride()[:3]),
        pos_t.data_ptr() if pos_t is not None else None, int(pos_add) if pos_t is not None else int(pos) + int(pos_add),
        b, h, t, d, _dtype_id(k), kq.side(), vq.side(), min(k_cache.shape[2], v_cache.shape[2]),
        status.data_ptr() if status is not None else None,
        # B200_KV_AFTER_PREV: the stream's previous kernel neither reads the rows written here nor writes k, v or pos
        A.KV_AFTER_PREV if after_prev else 0, 0)
    A.check(A.lib().b200_kv_append(C.byref(args), _stream(k.device)))


_WORKSPACES = {}


def _workspace(device, nbytes: int) -> torch.Tensor:
    """One growing scratch buffer per (device, stream): calls on one stream are ordered, so they
    can share it; the reference allocates the split buffers per call (accel.rs:190-199)."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


class OutputGather:
    """Buffers for b200_tq_attention_gather on one rank of a `torch.distributed` group: the gathered outputs of all
    ranks (two slots) and the step flags live in symmetric memory, so every rank can store into every other rank's copy.
    `rows` = batch * q_heads * seq_q of one rank (all ranks alike)."""

    def __init__(self, rows: int, d: int, dtype, device, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as sm
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.buf = sm.empty((2, self.world, rows, d), dtype=dtype, device=device)
        self.flags = sm.empty((max(self.world, 4),), dtype=torch.int32, device=device)
        self._h_buf = sm.rendezvous(self.buf, group)
        self._h_flags = sm.rendezvous(self.flags, group)
        self.buf.zero_()
        self.flags.zero_()
        self.state = torch.zeros(2, dtype=torch.int32, device=device)  # step, block counter
        torch.cuda.synchronize(device)
        dist.barrier(group)
        self.args = A.PeerGather(int(self._h_buf.buffer_ptrs_dev), int(self._h_flags.buffer_ptrs_dev), self.world, self.rank,
                                 self.state.data_ptr(), self.state.data_ptr() + 4)

    def steps_done(self) -> int:
        return int(self.state[0].item())

    def gathered(self) -> torch.Tensor:
        """(world, rows, d): the rows of all ranks after the last completed call (synchronizes to read the step)."""
        return self.buf[self.steps_done() & 1]


class _DenseRotationIO:
    """Queries rotated before and outputs rotated back after an attention call whose quantizers use the dense rotation
    (not fused into the kernels): f32 staging tensors that the kernel reads / writes instead of the caller's."""

    def __init__(self, q: torch.Tensor, out: torch.Tensor, kq: TurboQuantizer, vq: TurboQuantizer):
        self.kq = kq if (kq.rotation == "dense" and kq.qjl is None) else None  # prod keys rotate their query themselves
        self.vq = vq if vq.rotation == "dense" else None
        self.q_user, self.out_user = q, out
        self.q32 = torch.empty(q.shape, dtype=torch.float32, device=q.device) if self.kq is not None else None
        self.o32 = torch.empty(out.shape, dtype=torch.float32, device=q.device) if self.vq is not None else None

    def before(self):
        if self.kq is not None:
            src = self.q_user.to(torch.float32).contiguous()
            A.check(A.lib().b200_tq_rotate_dense(src.data_ptr(), self.q32.data_ptr(), self.kq.pi.data_ptr(), src.numel() // self.kq.dim,
                                                 self.kq.dim, 0, _stream(src.device)))

    def after(self):
        if self.vq is not None:
            back = self.vq.unrotate(self.o32.view(-1, self.vq.dim))
            self.out_user.copy_(back.view(self.out_user.shape))


class PackedAttention:
    """A prepared `attention_packed` call: arguments checked and marshalled once, `run()` only
    launches (a few microseconds of host time, and capturable in a CUDA graph after one warm-up
    call). The tensors given here are read / written by every `run()`; keep them alive."""

    def __init__(self, q: torch.Tensor, k_rows: torch.Tensor, v_rows: torch.Tensor, kv_len, kq: TurboQuantizer,
                 vq: TurboQuantizer, cfg: FlashAttnConfig, out: Optional[torch.Tensor] = None,
                 gather: Optional["OutputGather"] = None, after_prev: bool = False, kv_len_add: int = 0,
                 fresh_rows: Optional[int] = None, status: Optional[torch.Tensor] = None, outputs_free: bool = False):
        # after_prev: B200_TQ_AFTER_PREV of include/b200attn.h (the call may start while the stream's previous kernel
        # still runs; only for callers whose kv_len is not written by that kernel). fresh_rows (with after_prev):
        # B200_TQ_INPUTS_FINAL, the previous kernel writes none of the inputs but at most that many rows at the end
        # of every sequence (q included: it must be final before that kernel starts).
        # outputs_free (with after_prev): B200_TQ_OUTPUTS_FREE, no kernel that may still be running on the stream reads or
        # writes `out` or this call's workspace (consecutive calls with different outputs and their own workspaces).
        # status: an int32 device word that the kernels set when a bounded device wait runs out.
        _need_cuda(q, "q")
        b, hq, lq, d = q.shape
        kside = kq.side()
        if kq.qjl is not None:
            # prod keys (turbo_quant.rs:1161-1168): the rotated query followed by S q, f32; the keys' side of the call
            # then says "not rotated"
            qr = kq.rotate(q.reshape(-1, d)).view(b, hq, lq, d)
            q_out_dtype = q.dtype
            q = torch.cat([qr, qr.matmul(kq.qjl[1])], dim=3).contiguous()
            kside.rotation, kside.signs = A.ROT_NONE, None
            if out is None:
                out = torch.empty((b, hq, lq, d), dtype=q_out_dtype, device=q.device)
        bk, hkv, cap, kw = k_rows.shape
        bv, hv, capv, vw = v_rows.shape
        ragged = isinstance(kv_len, torch.Tensor)
        lk = cap if ragged else int(kv_len)
        if bk != b or bv != b or hv != hkv or capv < lk or cap < lk or (not ragged and lk == 0):
            raise ValueError(f"turbo-quant attention: q {tuple(q.shape)} / k {tuple(k_rows.shape)} / v {tuple(v_rows.shape)}"
                             f" / kv_len {kv_len} do not match")
        if kw < kq.row_words() or vw < vq.row_words() or d != kq.dim or d != vq.dim:
            raise ValueError(f"turbo-quant attention: rows of {kw} / {vw} words and head dim {d} do not match the "
                             f"quantizers ({kq.row_words()} / {vq.row_words()} words, dim {kq.dim})")
        if q.stride(3) != 1:
            q = q.contiguous()
        if k_rows.stride(3) != 1 or v_rows.stride(3) != 1:
            raise ValueError("turbo-quant attention: packed rows must be contiguous along the words")
        if out is None:
            out = torch.empty((b, hq, lq, d), dtype=q.dtype, device=q.device)
        self._dense = _DenseRotationIO(q, out, kq, vq)
        user_out = out
        if self._dense.q32 is not None:
            q = self._dense.q32
        if self._dense.o32 is not None:
            out = self._dense.o32
        wl, wr = cfg.window_i32()
        alibi, abs_ = None, 0
        if cfg.alibi_slopes is not None:
            alibi = cfg.alibi_slopes.to(device=q.device, dtype=torch.float32).contiguous()
            if alibi.shape == (hq,):
                abs_ = 0
            elif alibi.shape == (b, hq):
                abs_ = hq
            else:
                raise ValueError(f"flash-attn: alibi slopes must be ({hq}) or ({b}, {hq}), got {tuple(alibi.shape)}")
        args = A.TqAttnArgs()
        args.q, args.out = q.data_ptr(), out.data_ptr()
        args.q_dtype, args.out_dtype = _dtype_id(q), _dtype_id(out)
        args.q_strides, args.out_strides = A.u64x3(*q.stride()[:3]), A.u64x3(*out.stride()[:3])
        args.k_rows, args.v_rows = k_rows.data_ptr(), v_rows.data_ptr()
        args.k_strides, args.v_strides = A.u64x3(*k_rows.stride()[:3]), A.u64x3(*v_rows.stride()[:3])
        args.pages, args.n_pages = None, 0
        args.kv_len_dev = kv_len.data_ptr() if ragged else None
        args.b, args.lq, args.lk, args.hq, args.hkv, args.d = b, lq, lk, hq, hkv, d
        args.kq, args.vq = kside, vq.side()
        args.scale, args.softcap = cfg.softmax_scale, cfg.softcap or 0.0
        args.wl, args.wr = wl, wr
        args.alibi, args.alibi_bstride = (alibi.data_ptr() if alibi is not None else None), abs_
        args.splits = cfg.splits
        args.flags = A.TQ_AFTER_PREV if after_prev else 0
        if after_prev and fresh_rows is not None:
            args.flags |= A.TQ_INPUTS_FINAL
            args.fresh_rows = int(fresh_rows)
        if after_prev and outputs_free:
            args.flags |= A.TQ_OUTPUTS_FREE
        nbytes = A.lib().b200_tq_attention_workspace_bytes(C.byref(args))  # the plan, and with it the size, depends on the flags
        if nbytes == 0:
            A.check(A.lib().b200_tq_attention(C.byref(args), None))  # reports why the call cannot be planned
        # calls of a stream share one scratch buffer, which stream order keeps apart; a call that does not wait for the one
        # before (outputs_free) has a buffer of its own
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device) if (after_prev and outputs_free) else _workspace(q.device, nbytes)
        args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
        args.status = status.data_ptr() if status is not None else None
        args.kv_len_add = int(kv_len_add) if ragged else 0  # tokens appended since the device lengths were written
        self.args, self.out, self.device = args, user_out, q.device
        self._keep = (q, out, k_rows, v_rows, kv_len, kq, vq, alibi, ws, status)
        self.workspace = ws  # the scratch buffer of the call (shared by the calls of one stream unless outputs_free)
        self._fn, self._ref = A.lib().b200_tq_attention, C.byref(args)
        self._gather = gather
        if gather is not None and self._dense.o32 is not None:
            raise ValueError("OutputGather: the gathered rows are stored by the attention kernel, before a dense rotation back")
        if gather is not None:
            # outputs also stored into every rank's gathered buffer by the kernel that merges the key splits
            if out.numel() != gather.buf.shape[2] * gather.buf.shape[3] or out.dtype != gather.buf.dtype:
                raise ValueError("OutputGather was sized for other outputs")
            fn, gref = A.lib().b200_tq_attention_gather, C.byref(gather.args)
            self._fn = lambda ref, stream: fn(ref, gref, stream)

    def run(self) -> torch.Tensor:
        self._dense.before()
        rc = self._fn(self._ref, torch.cuda.current_stream(self.device).cuda_stream)
        if rc:
            A.check(rc)
        self._dense.after()
        return self.out


def attention_packed(q: torch.Tensor, k_rows: torch.Tensor, v_rows: torch.Tensor, kv_len, kq: TurboQuantizer,
                     vq: TurboQuantizer, cfg: FlashAttnConfig, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of `q: (batch, q_heads, seq_q, head_dim)` over packed rows `k_rows: (batch,
    kv_heads, capacity, k_words)`, `v_rows: (..., v_words)` (turbo_quant.rs:993-1072). `kv_len`: the
    number of valid rows, an int (all sequences) or an int32 device tensor with one length per
    batch entry (ragged batch). Output in `q`'s dtype and layout."""
    return PackedAttention(q, k_rows, v_rows, kv_len, kq, vq, cfg, out).run()


@dataclass
class KvBlockRef:
    """One block of a paged cache: `k` / `v` are (batch, kv_heads, capacity, words) int32 tensors of packed rows of
    which the first `rows` positions of the third axis are valid (candle-nn/src/flash_attn.rs:608-613)."""
    k: torch.Tensor
    v: torch.Tensor
    rows: int


class PackedBlocksAttention:
    """A prepared `attention_packed_blocks` call: the block table is built and copied to the device once, `run()` only
    launches (capturable in a CUDA graph after one warm-up call). The tensors given here are read / written by every
    `run()`; keep them alive. Arguments as `attention_packed_blocks`."""

    def __init__(self, q: torch.Tensor, blocks, kq: TurboQuantizer, vq: TurboQuantizer, cfg: FlashAttnConfig, in_place: bool = False,
                 kv_len: Optional[torch.Tensor] = None, after_prev: bool = False, out: Optional[torch.Tensor] = None):
        _need_cuda(q, "q")
        if len(blocks) == 0:
            raise ValueError("turbo-quant blocks: no blocks")
        b, hq, lq, d = q.shape
        hkv = blocks[0].k.shape[1]
        kw, vw = blocks[0].k.shape[3], blocks[0].v.shape[3]
        if kw != kq.row_words() or vw != vq.row_words() or d != kq.dim or d != vq.dim:
            raise ValueError(f"turbo-quant blocks: rows of {kw} / {vw} words and head dim {d} do not match the quantizers "
                             f"({kq.row_words()} / {vq.row_words()} words, dim {kq.dim})")
        table = np.zeros(len(blocks), dtype=np.dtype([("k", "<u8"), ("v", "<u8"), ("rows", "<u4"), ("k_cap", "<u4"), ("v_cap", "<u4"), ("pad", "<u4")]))
        lk = 0
        for n, blk in enumerate(blocks):
            for t, w, what in ((blk.k, kw, "k"), (blk.v, vw, "v")):
                # paged_block_layout (flash_attn.rs:618-646): contiguous rows, head stride = whole rows, batch stride = hkv heads
                if t.dtype != torch.int32 or t.dim() != 4 or t.shape[0] != b or t.shape[1] != hkv or t.shape[3] != w or not t.is_contiguous():
                    raise ValueError(f"turbo-quant blocks: block {n} ({what}) must be a contiguous int32 ({b}, {hkv}, capacity, {w}) tensor")
                if t.device != q.device:
                    raise ValueError("turbo-quant blocks: blocks live on another device")
            if not 0 <= blk.rows <= min(blk.k.shape[2], blk.v.shape[2]):
                raise ValueError(f"turbo-quant blocks: block {n} holds {blk.rows} rows, capacity {blk.k.shape[2]} / {blk.v.shape[2]}")
            table[n] = (blk.k.data_ptr(), blk.v.data_ptr(), blk.rows, blk.k.shape[2], blk.v.shape[2], 0)
            lk += blk.rows
        if lk == 0:
            raise ValueError("turbo-quant blocks: no valid rows")
        pages = torch.from_numpy(table.view(np.uint8)).to(q.device)
        if q.stride(3) != 1:
            q = q.contiguous()
        if out is None:
            out = torch.empty((b, hq, lq, d), dtype=q.dtype, device=q.device)
        self._dense = _DenseRotationIO(q, out, kq, vq)
        user_out = out
        if self._dense.q32 is not None:
            q = self._dense.q32
        if self._dense.o32 is not None:
            out = self._dense.o32
        wl, wr = cfg.window_i32()
        alibi, abs_ = None, 0
        if cfg.alibi_slopes is not None:
            alibi = cfg.alibi_slopes.to(device=q.device, dtype=torch.float32).contiguous()
            if alibi.shape not in ((hq,), (b, hq)):
                raise ValueError(f"flash-attn: alibi slopes must be ({hq}) or ({b}, {hq}), got {tuple(alibi.shape)}")
            abs_ = hq if alibi.dim() == 2 else 0
        args = A.TqAttnArgs()
        args.q, args.out = q.data_ptr(), out.data_ptr()
        args.q_dtype, args.out_dtype = _dtype_id(q), _dtype_id(out)
        args.q_strides, args.out_strides = A.u64x3(*q.stride()[:3]), A.u64x3(*out.stride()[:3])
        args.k_rows = args.v_rows = None
        args.k_strides, args.v_strides = A.u64x3(0, 0, kw), A.u64x3(0, 0, vw)  # only the row stride is common to the blocks
        args.pages, args.n_pages = pages.data_ptr(), len(blocks)
        args.kv_len_dev = kv_len.data_ptr() if kv_len is not None else None
        args.flags = (A.TQ_AFTER_PREV if after_prev else 0) | (A.TQ_IN_PLACE if in_place else 0)
        args.b, args.lq, args.lk, args.hq, args.hkv, args.d = b, lq, lk, hq, hkv, d
        args.kq, args.vq = kq.side(), vq.side()
        args.scale, args.softcap = cfg.softmax_scale, cfg.softcap or 0.0
        args.wl, args.wr = wl, wr
        args.alibi, args.alibi_bstride = (alibi.data_ptr() if alibi is not None else None), abs_
        args.workspace, args.workspace_bytes, args.status = None, 0, None
        # with the workspace the library asks for, the tensor-core kernel walks the table (or the blocks are compacted
        # into the workspace first); `in_place=True` (B200_TQ_IN_PLACE) keeps the general kernel that reads the blocks
        # where they are
        need = int(A.lib().b200_tq_attention_workspace_bytes(C.byref(args)))
        if need == 0:
            A.check(A.lib().b200_tq_attention(C.byref(args), _stream(q.device)))  # raises with the library's reason
        ws = _workspace(q.device, need)
        args.workspace, args.workspace_bytes = ws.data_ptr(), need
        self.args, self.out, self.device = args, user_out, q.device
        self._keep = (q, out, blocks, pages, kv_len, kq, vq, alibi, ws)
        self._ref = C.byref(args)

    def run(self) -> torch.Tensor:
        self._dense.before()
        rc = A.lib().b200_tq_attention(self._ref, torch.cuda.current_stream(self.device).cuda_stream)
        if rc:
            A.check(rc)
        self._dense.after()
        return self.out


def attention_packed_blocks(q: torch.Tensor, blocks, kq: TurboQuantizer, vq: TurboQuantizer, cfg: FlashAttnConfig, in_place: bool = False,
                            kv_len: Optional[torch.Tensor] = None, after_prev: bool = False) -> torch.Tensor:
    """Attention of `q: (batch, q_heads, seq_q, head_dim)` over packed rows that live in paged cache blocks, given as
    a block table in device memory (candle-nn/src/turbo_quant.rs:1074-1114; no limit of 128 blocks). The keys are the
    valid rows of the blocks, one block after the other; masks are bottom-right aligned over them. Keys and values in
    one format of the tensor-core kernel: that kernel walks the block table itself (tiles end where blocks end). Other
    format pairs of that kernel: the blocks are compacted into the workspace by one copy kernel first; everything else,
    and `in_place=True`: the general kernel reads the blocks where they are. `kv_len` (int32 device tensor, one entry
    per batch entry; only where the kernel walks the table): sequence b attends to the first kv_len[b] keys."""
    return PackedBlocksAttention(q, blocks, kq, vq, cfg, in_place, kv_len, after_prev).run()


class TurboKvCache:
    """A KV cache that stores keys and values compressed and attends over them without
    decompressing them (turbo_quant.rs:786-991). Layouts: `append(k, v)` with `(batch, kv_heads,
    seq, head_dim)`, `attention(q)` with `(batch, q_heads, seq_q, head_dim)`.

    The capacity buffers grow like the reference's `Cache` (candle-nn/src/kv_cache.rs:60-96):
    allocated at the first append, grown by max(grow_by, capacity / 2) when full."""

    def __init__(self, key: QuantFormat, value: QuantFormat, dim: int, rotation: str = "auto", seed: int = 42,
                 grow_by: int = 1, device="cuda"):
        if value.mode == A.TURBO_PROD:
            raise ValueError("turbo-quant: values use the MSE codebooks, not the prod (QJL) format")
        self.kq = TurboQuantizer(key, dim, rotation, seed, device)
        self.vq = TurboQuantizer(value, dim, rotation, (seed + 2) & (2**64 - 1), device)
        self.dim, self.grow_by = dim, max(int(grow_by), 1)
        self.k: Optional[torch.Tensor] = None
        self.v: Optional[torch.Tensor] = None
        self.cap = self.grow_by
        self.len = 0
        self.dtype: Optional[torch.dtype] = None

    @classmethod
    def with_formats(cls, key, value, dim, rotation, seed, grow_by, device="cuda"):
        return cls(key, value, dim, rotation, seed, grow_by, device)

    def formats(self):
        return self.kq.format, self.vq.format

    def seq_len(self) -> int:
        return self.len

    def reset(self):
        self.k = self.v = None
        self.len = 0
        self.cap = self.grow_by

    def storage_bytes(self) -> int:
        return sum(t.numel() * 4 for t in (self.k, self.v) if t is not None)

    def _grown(self, need: int) -> int:
        cap = self.cap
        while cap < need:
            cap += max(self.grow_by, cap // 2, 1)
        return cap

    def append(self, k: torch.Tensor, v: torch.Tensor):
        _need_cuda(k, "k")
        b, h, t, d = k.shape
        if d != self.dim or tuple(v.shape) != (b, h, t, d):
            raise ValueError(f"turbo-quant cache: k {tuple(k.shape)} / v {tuple(v.shape)} do not match head dim {self.dim}")
        if self.dtype is None:
            self.dtype = k.dtype
        if self.k is None:
            self.cap = self._grown(t)
            self.k = torch.zeros((b, h, self.cap, self.kq.row_words()), dtype=torch.int32, device=k.device)
            self.v = torch.zeros((b, h, self.cap, self.vq.row_words()), dtype=torch.int32, device=k.device)
        need = self.len + t
        cap = self._grown(need)
        if cap > self.cap:
            nk = torch.zeros((b, h, cap, self.kq.row_words()), dtype=torch.int32, device=k.device)
            nv = torch.zeros((b, h, cap, self.vq.row_words()), dtype=torch.int32, device=k.device)
            nk[:, :, : self.cap] = self.k
            nv[:, :, : self.cap] = self.v
            self.k, self.v, self.cap = nk, nv, cap
        if self.kq.qjl is not None:
            # prod keys are finished in stages (quantize, residual, sketch): rows first, then copied to their place;
            # the values go through the fused append
            rows = self.kq.quantize_rows(k.reshape(-1, d).contiguous() if k.is_contiguous() else k.contiguous().view(-1, d))
            self.k[:, :, self.len:self.len + t] = rows.view(b, h, t, -1)
            scratch = torch.empty_like(self.v)
            _kv_append(v, v, scratch, self.v, self.vq, self.vq, self.len)
        else:
            _kv_append(k, v, self.k, self.v, self.kq, self.vq, self.len)
        self.len += t

    def keys_values(self):
        """Keys and values `(batch, kv_heads, seq, head_dim)`, dequantized (turbo_quant.rs:947-966)."""
        if self.k is None:
            return None
        b, h, _, _ = self.k.shape
        dt = self.dtype or torch.float32
        deq = lambda q, x: q.dequantize_rows(x[:, :, : self.len].reshape(b * h * self.len, -1)).reshape(
            b, h, self.len, self.dim).to(dt)
        return deq(self.kq, self.k), deq(self.vq, self.v)

    # query rows per kv head (tokens x heads of the group) from which a chunk of prefill over the cache goes through
    # the dequantized rows and the tensor-core prefill tiles instead of the decode kernel, which re-reads the packed
    # rows once per pack of eight query rows
    PREFILL_ROWS = 512

    def attention(self, q: torch.Tensor, cfg: FlashAttnConfig) -> torch.Tensor:
        """Attention of `q: (batch, q_heads, seq_q, head_dim)` over the cache (turbo_quant.rs:968-990). Decode and
        short chunks: the fused kernel over the packed rows. Long chunks (chunked prefill over an already compressed
        cache): the reference's own second route, `keys_values()` + `flash_attn_bhsd` (turbo_quant.rs:986-990), whose
        attention here runs on the tcgen05 prefill tiles."""
        if self.k is None:
            raise RuntimeError("turbo-quant cache: attention on an empty cache")
        b, hq, lq, d = q.shape
        hkv = self.k.shape[1]
        if (d == 128 and q.dtype in (torch.float16, torch.bfloat16) and hkv and hq % hkv == 0
                and lq * (hq // hkv) >= self.PREFILL_ROWS and self.kq.qjl is None):
            from .flash_attn import flash_attn_bhsd
            k, v = self.keys_values()
            return flash_attn_bhsd(q, k.to(q.dtype), v.to(q.dtype), cfg)
        return attention_packed(q, self.k, self.v, self.len, self.kq, self.vq, cfg)
