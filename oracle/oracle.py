"""numpy front end of the CPU oracle (oracle/tq_oracle.c) and of the reference's own kernel
sources compiled as plain C++ (oracle/_ref/accel_host_test).

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this module; it is the checker
used by tests/, by the smoke check and by the CPU baseline leg of bench.py.
"""
from __future__ import annotations

import ctypes as C
import os
import struct
import subprocess
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
MSE, PROD, MXFP4, NVFP4, MXFP8, FP8 = range(6)
MODE_NAMES = {MSE: "turbo-mse", PROD: "turbo-prod", MXFP4: "mxfp4", NVFP4: "nvfp4", MXFP8: "mxfp8", FP8: "fp8"}

_lib = None


def build():
    """Compiles liboracle.so (and oracle/_ref when the reference tree is present)."""
    subprocess.run(["make", "-s", "-C", str(HERE)], check=True)


def lib():
    global _lib
    if _lib is None:
        so = HERE / "liboracle.so"
        if not so.exists():
            build()
        _lib = C.CDLL(str(so))
        _lib.orc_h2f.restype = C.c_float
        _lib.orc_h2f.argtypes = [C.c_uint16]
        _lib.orc_f2h.restype = C.c_uint16
        _lib.orc_f2h.argtypes = [C.c_float]
        _lib.orc_bf2f.restype = C.c_float
        _lib.orc_bf2f.argtypes = [C.c_uint16]
        _lib.orc_f2bf.restype = C.c_uint16
        _lib.orc_f2bf.argtypes = [C.c_float]
        for n in ("orc_e4m3_to_f32", "orc_fp4_to_f32", "orc_e8m0_to_f32"):
            getattr(_lib, n).restype = C.c_float
            getattr(_lib, n).argtypes = [C.c_uint32]
        for n in ("orc_f32_to_e4m3", "orc_f32_to_fp4"):
            getattr(_lib, n).restype = C.c_uint32
            getattr(_lib, n).argtypes = [C.c_float]
        _lib.orc_mx_scale_code.restype = C.c_uint32
        _lib.orc_mx_scale_code.argtypes = [C.c_float, C.c_int]
        _lib.orc_normal_fill.argtypes = [C.c_uint64, C.c_float, C.c_void_p, C.c_size_t]
        _lib.orc_u64_fill.argtypes = [C.c_uint64, C.c_void_p, C.c_size_t]
        _lib.orc_rotate_rows.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
        _lib.orc_quantize_rows.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
        _lib.orc_dequantize_rows.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        _lib.orc_combine.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_void_p]
        _lib.orc_split_count_grouped.argtypes = [C.c_longlong, C.c_int, C.c_longlong, C.c_int]
        _lib.orc_rotation_matrix.argtypes = [C.c_int, C.c_int, C.c_uint64, C.c_void_p]
        _lib.orc_hadamard_signs.argtypes = [C.c_int, C.c_uint64, C.c_void_p]
        _lib.orc_codebook.argtypes = [C.c_int, C.c_int, C.c_void_p]
    return _lib


class AttnParams(C.Structure):
    _fields_ = [("b", C.c_int), ("lq", C.c_int), ("lk", C.c_int), ("hq", C.c_int), ("hkv", C.c_int),
                ("d", C.c_int), ("scale", C.c_float), ("softcap", C.c_float), ("wl", C.c_int),
                ("wr", C.c_int), ("k_descale", C.c_float), ("v_descale", C.c_float)]


class PackedSides(C.Structure):
    _fields_ = [("k_mode", C.c_int), ("k_bits", C.c_int), ("v_mode", C.c_int), ("v_bits", C.c_int),
                ("k_sb", C.c_size_t), ("k_sh", C.c_size_t), ("k_ss", C.c_size_t),
                ("v_sb", C.c_size_t), ("v_sh", C.c_size_t), ("v_ss", C.c_size_t)]


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


# ------------------------------------------------------------------ element codecs

def f32_to_e4m3(x):
    l = lib()
    return np.array([l.orc_f32_to_e4m3(float(v)) for v in np.ravel(x)], dtype=np.uint32).reshape(np.shape(x))


def e4m3_to_f32(c):
    l = lib()
    return np.array([l.orc_e4m3_to_f32(int(v)) for v in np.ravel(c)], dtype=np.float32).reshape(np.shape(c))


def f32_to_fp4(x):
    l = lib()
    return np.array([l.orc_f32_to_fp4(float(v)) for v in np.ravel(x)], dtype=np.uint32).reshape(np.shape(x))


def fp4_to_f32(c):
    l = lib()
    return np.array([l.orc_fp4_to_f32(int(v)) for v in np.ravel(c)], dtype=np.float32).reshape(np.shape(c))


def f32_to_f16_bits(x):
    """Round to nearest even f16 (same bits as accel_common.h ax_f2h for finite values)."""
    return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def f32_to_bf16_bits(x):
    """accel_common.h:156-161 vectorized."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    r = np.where(nan, (u >> 16) | 0x40, r)
    return r.astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_to(x, dtype: str):
    """f32 values rounded through a storage dtype ('f32', 'f16', 'bf16')."""
    x = np.asarray(x, dtype=np.float32)
    if dtype == "f16":
        return x.astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        return bf16_bits_to_f32(f32_to_bf16_bits(x))
    return x


# ------------------------------------------------------------------ layout, tables, RNG

def row_layout(mode: int, bits: int, dim: int):
    out = (C.c_int * 5)()
    if lib().orc_row_layout(mode, bits, dim, out):
        raise ValueError(f"format mode {mode} bits {bits} does not fit vectors of {dim}")
    return dict(code_bits=out[0], code_words=out[1], aux_words=out[2], row_words=out[3], rsc_offset=out[4])


def normal(seed: int, n: int, scale: float = 1.0):
    out = np.empty(n, dtype=np.float32)
    lib().orc_normal_fill(C.c_uint64(seed), C.c_float(scale), _p(out), n)
    return out


def u64s(seed: int, n: int):
    out = np.empty(n, dtype=np.uint64)
    lib().orc_u64_fill(C.c_uint64(seed), _p(out), n)
    return out


def codebook(dim: int, bits: int):
    tab = np.zeros(32, dtype=np.float32)
    if lib().orc_codebook(dim, bits, _p(tab)):
        raise ValueError("codebooks have 1 to 4 bits and dim >= 2")
    return tab


def hadamard_signs(dim: int, seed: int):
    s = np.zeros(dim, dtype=np.float32)
    if lib().orc_hadamard_signs(dim, C.c_uint64(seed), _p(s)):
        raise ValueError("hadamard needs a power of two")
    return s


def rotation_matrix(dim: int, kind: int, seed: int):
    m = np.zeros((dim, dim), dtype=np.float32)
    if lib().orc_rotation_matrix(dim, kind, C.c_uint64(seed), _p(m)):
        raise ValueError("bad rotation")
    return m


def rotate_rows(x, pi, transpose=False):
    """transpose False: y = x Pi^T (into the rotated domain); True: x = y Pi (back)."""
    x = _c(x, np.float32)
    d = x.shape[-1]
    y = np.empty_like(x)
    lib().orc_rotate_rows(_p(x), x.size // d, d, _p(_c(pi, np.float32)), int(transpose), _p(y))
    return y


# ------------------------------------------------------------------ row codec

def quantize_rows(y, mode, bits=4, tab=None, norm_order=1):
    y = _c(y, np.float32)
    rows, d = y.shape
    lay = row_layout(mode, bits, d)
    tab = _c(tab if tab is not None else np.zeros(32), np.float32)
    out = np.empty((rows, lay["row_words"]), dtype=np.uint32)
    assert lib().orc_quantize_rows(_p(y), rows, d, mode, bits, _p(tab), norm_order, _p(out)) == 0
    return out


def qjl_matrix(dim: int, seed: int):
    """Row-major dim x dim matrix of standard normals: the QJL projection S of prod rows (turbo.rs:236-239)."""
    m = np.empty((dim, dim), dtype=np.float32)
    lib().orc_qjl_matrix(dim, C.c_uint64(seed), _p(m))
    return m


def tq_residual(y, data, bits, tab):
    """resid = y / rsc0 - centroid[code] of prod rows after stage one (turbo_quant_impl.h:161-177)."""
    y, data = _c(y, np.float32), _c(data, np.uint32)
    rows, d = y.shape
    out = np.empty((rows, d), dtype=np.float32)
    assert lib().orc_tq_residual(_p(y), _p(data), C.c_size_t(rows), d, bits, _p(_c(tab, np.float32)), _p(out)) == 0
    return out


def tq_signs(data, proj, resid, bits):
    """Sign bits of proj = S resid and rsc1 = |resid| filled into prod rows (turbo_quant_impl.h:179-206)."""
    data, proj, resid = _c(data, np.uint32), _c(proj, np.float32), _c(resid, np.float32)
    rows, d = proj.shape
    out = np.empty_like(data)
    assert lib().orc_tq_signs(_p(data), _p(proj), _p(resid), C.c_size_t(rows), d, bits, _p(out)) == 0
    return out


def quantize_rows_prod(y, bits, tab, s_matrix, norm_order=1):
    """Prod rows of rotated vectors y: stage one (codes of bits - 1 bits, norm), residual, projection with S, sign bits
    and residual norm (candle-nn/src/turbo_quant.rs:214-236)."""
    y = _c(y, np.float32)
    stage1 = quantize_rows(y, PROD, bits, tab, norm_order)
    resid = tq_residual(y, stage1, bits, tab)
    proj = resid @ np.ascontiguousarray(s_matrix.T)
    return tq_signs(stage1, proj, resid, bits)


def dequantize_qjl(data, dim, bits):
    """QJL coefficients of prod rows: +-(rsc0 rsc1 sqrt(pi / 2) / dim) by sign bit (turbo_quant_impl.h:219-222)."""
    data = _c(data, np.uint32)
    out = np.empty((data.shape[0], dim), dtype=np.float32)
    assert lib().orc_dequantize_qjl(_p(data), C.c_size_t(data.shape[0]), dim, bits, _p(out)) == 0
    return out


def ref_tq_signs(data, proj, resid, bits, gx=3):
    """tq_signs on the host emulator of the reference's kernels."""
    data, proj, resid = _c(data, np.uint32), _c(proj, np.float32), _c(resid, np.float32)
    rows, d = proj.shape
    lay = row_layout(PROD, bits, d)
    params = np.array([rows, d, lay["code_words"], lay["row_words"], gx], dtype=np.uint32)
    out = ref_run({"op": "tq_signs", "data": data.ravel(), "proj": proj.ravel(), "resid": resid.ravel(), "params": params})
    return out["out"].reshape(rows, lay["row_words"])


def dequantize_rows(data, dim, mode, bits=4, tab=None):
    data = _c(data, np.uint32)
    rows, rw = data.shape
    tab = _c(tab if tab is not None else np.zeros(32), np.float32)
    out = np.empty((rows, dim), dtype=np.float32)
    assert lib().orc_dequantize_rows(_p(data), rows, rw, dim, mode, bits, _p(tab), _p(out)) == 0
    return out


# ------------------------------------------------------------------ attention

def _params(b, lq, lk, hq, hkv, d, scale, softcap=0.0, wl=-1, wr=-1, k_descale=1.0, v_descale=1.0):
    return AttnParams(b, lq, lk, hq, hkv, d, scale, softcap, wl, wr, k_descale, v_descale)


def reference_attention(q, k, v, scale, wl=-1, wr=-1, softcap=0.0, alibi=None, cu_q=None, cu_k=None,
                        k_descale=1.0, v_descale=1.0, max_q=0, max_k=0):
    """Dense: q (b, lq, hq, d), k / v (b, lk, hkv, d). Varlen: q (tq, hq, d), k / v (tk, hkv, d)."""
    q, k, v = _c(q, np.float32), _c(k, np.float32), _c(v, np.float32)
    if cu_q is None:
        b, lq, hq, d = q.shape
        lk, hkv = k.shape[1], k.shape[2]
    else:
        cu_q, cu_k = _c(cu_q, np.uint32), _c(cu_k, np.uint32)
        b = len(cu_q) - 1
        hq, d = q.shape[1], q.shape[2]
        hkv = k.shape[1]
        lq, lk = max_q, max_k
    abs_ = 0
    if alibi is not None:
        alibi = _c(alibi, np.float32)
        abs_ = hq if alibi.ndim == 2 else 0
    p = _params(b, lq, lk, hq, hkv, d, scale, softcap, wl, wr, k_descale, v_descale)
    out = np.empty(q.shape, dtype=np.float32)
    lib().orc_reference_attention(_p(q), _p(k), _p(v), _p(cu_q), _p(cu_k), _p(alibi), abs_, C.byref(p), _p(out))
    return out


def tq_attention(q, kd, vd, lk, k_fmt, v_fmt, scale, tab=None, kv_len=None, wl=-1, wr=-1, softcap=0.0,
                 alibi=None):
    """q (b, hq, lq, d) f32; kd / vd (b, hkv, cap, words) u32; *_fmt = (mode, bits). Out (b, hq, lq, d)."""
    q, kd, vd = _c(q, np.float32), _c(kd, np.uint32), _c(vd, np.uint32)
    b, hq, lq, d = q.shape
    if k_fmt[0] == PROD:
        d //= 2  # prod keys: the rotated query followed by S q
    _, hkv, kcap, kw = kd.shape
    _, _, vcap, vw = vd.shape
    tab = _c(tab if tab is not None else np.zeros(64), np.float32)
    abs_ = 0
    if alibi is not None:
        alibi = _c(alibi, np.float32)
        abs_ = hq if alibi.ndim == 2 else 0
    if kv_len is not None:
        kv_len = _c(kv_len, np.int32)
    p = _params(b, lq, lk, hq, hkv, d, scale, softcap, wl, wr)
    sd = PackedSides(k_fmt[0], k_fmt[1], v_fmt[0], v_fmt[1], hkv * kcap * kw, kcap * kw, kw,
                     hkv * vcap * vw, vcap * vw, vw)
    out = np.empty((b, hq, lq, d), dtype=np.float32)
    assert lib().orc_tq_attention(_p(q), _p(kd), _p(vd), _p(kv_len), _p(tab), _p(alibi), abs_, C.byref(p),
                                  C.byref(sd), _p(out)) == 0
    return out


def unfused_attention(q, k, v, scale, wl=-1, wr=-1, softcap=0.0, k_descale=1.0, v_descale=1.0):
    q, k, v = _c(q, np.float32), _c(k, np.float32), _c(v, np.float32)
    b, lq, hq, d = q.shape
    lk, hkv = k.shape[1], k.shape[2]
    p = _params(b, lq, lk, hq, hkv, d, scale, softcap, wl, wr, k_descale, v_descale)
    out = np.empty(q.shape, dtype=np.float32)
    lib().orc_unfused_attention(_p(q), _p(k), _p(v), C.byref(p), _p(out))
    return out


def combine(part_o, part_lse):
    part_o, part_lse = _c(part_o, np.float32), _c(part_lse, np.float32)
    s, rows, d = part_o.shape
    o = np.empty((rows, d), dtype=np.float32)
    lib().orc_combine(_p(part_o), _p(part_lse), rows, d, s, _p(o))
    return o


def split_count_grouped(rows, group, lk, compute_units):
    return lib().orc_split_count_grouped(rows, group, lk, compute_units)


def row_group(hq, hkv):
    return lib().orc_row_group(hq, hkv)


def cpu_decode_step(k_rows, v_rows, q, mode, bits, k_tab, v_tab, cache_dtype: str, scale: float):
    """The reference's CPU path for one decode step of one sequence, all in one C call: k_rows / v_rows (hkv, L, words)
    packed rows, q (hq, d) f32 -> (hq, d) f32. Dequantizes the cached rows to `cache_dtype`, then unfused attention."""
    k_rows, v_rows, q = _c(k_rows, np.uint32), _c(v_rows, np.uint32), _c(q, np.float32)
    hkv, L, _ = k_rows.shape
    hq, d = q.shape
    out = np.empty((hq, d), dtype=np.float32)
    dt = {"f32": 0, "f16": 1, "bf16": 2}[cache_dtype]
    rc = lib().orc_cpu_decode_step(_p(k_rows), _p(v_rows), C.c_size_t(L), hkv, hq, d, mode, bits, _p(_c(k_tab, np.float32)),
                                   _p(_c(v_tab, np.float32)), dt, _p(q), C.c_float(scale), _p(out))
    assert rc == 0
    return out


def num_threads():
    return lib().orc_num_threads()


def set_num_threads(n: int):
    lib().orc_set_num_threads(int(n))


# ------------------------------------------------------------------ the reference's own kernels (oracle/_ref)

REF_BIN = HERE / "_ref" / "accel_host_test"
_KINDS = {np.dtype(np.float32): 0, np.dtype(np.uint32): 1, np.dtype(np.uint64): 2, np.dtype(np.int32): 3}
_DT = {0: np.float32, 1: np.uint32, 2: np.uint64, 3: np.int32}


def ref_available() -> bool:
    return REF_BIN.exists() and os.access(REF_BIN, os.X_OK)


def ref_run(arrays: dict) -> dict:
    """Runs one operation of the reference's host test driver. File protocol:
    repeated [u32 name_len][name][u8 kind][u64 bytes][bytes]
    (candle-core/kernels/tests/accel_host_test.cpp:19-61)."""
    with tempfile.TemporaryDirectory() as td:
        fin, fout = os.path.join(td, "in"), os.path.join(td, "out")
        with open(fin, "wb") as f:
            for name, a in arrays.items():
                if isinstance(a, str):
                    kind, raw = 4, a.encode()
                else:
                    a = np.ascontiguousarray(a)
                    kind, raw = _KINDS[a.dtype], a.tobytes()
                f.write(struct.pack("<I", len(name)) + name.encode() + struct.pack("<BQ", kind, len(raw)) + raw)
        subprocess.run([str(REF_BIN), fin, fout], check=True)
        out = {}
        with open(fout, "rb") as f:
            buf = f.read()
        pos = 0
        while pos < len(buf):
            (nl,) = struct.unpack_from("<I", buf, pos)
            pos += 4
            name = buf[pos:pos + nl].decode()
            pos += nl
            kind, nb = struct.unpack_from("<BQ", buf, pos)
            pos += 9
            out[name] = np.frombuffer(buf[pos:pos + nb], dtype=_DT[kind]).copy()
            pos += nb
        return out


def ref_tq_quant(x, mode, bits, tab, src_dtype=0, gx=5):
    """tq_quant_{f32,f16,bf16} on the host emulator; x (rows, d) f32 (rounded to the source dtype by
    the driver). Returns (rows, row_words) u32."""
    x = _c(x, np.float32)
    rows, d = x.shape
    lay = row_layout(mode, bits, d)
    params = np.array([rows, d, mode, lay["code_bits"], lay["code_words"], lay["aux_words"], lay["row_words"],
                       gx, src_dtype], dtype=np.uint32)
    out = ref_run({"op": "tq_quant", "x": x.ravel(), "tab": _c(tab, np.float32), "params": params})
    return out["out"].reshape(rows, lay["row_words"])


def ref_tq_dequant(data, dim, mode, bits, tab, gx=3):
    data = _c(data, np.uint32)
    rows = data.shape[0]
    lay = row_layout(mode, bits, dim)
    params = np.array([rows, dim, mode, lay["code_bits"], lay["code_words"], lay["row_words"], lay["rsc_offset"],
                       gx, 0], dtype=np.uint32)
    out = ref_run({"op": "tq_dequant", "data": data.ravel(), "tab": _c(tab, np.float32), "params": params})
    return out["out"].reshape(rows, dim)


def ref_tq_attn(q, kd, vd, lk, k_fmt, v_fmt, scale, tab, splits=1, group=1, wl=-1, wr=-1, softcap=0.0,
                alibi=None, fp8=False, gx=None):
    """tq_attn / tq_attn_fp8 / tq_attng{G}[_fp8] (+ tq_combine) on the host emulator."""
    q, kd, vd = _c(q, np.float32), _c(kd, np.uint32), _c(vd, np.uint32)
    b, hq, lq, w = q.shape
    d = w // 2 if k_fmt[0] == PROD else w  # prod keys: the rotated query followed by S q
    _, hkv, kcap, kw = kd.shape
    _, _, vcap, vw = vd.shape
    kl, vl = row_layout(k_fmt[0], k_fmt[1], d), row_layout(v_fmt[0], v_fmt[1], d)
    if gx is None:
        gx = lq * hq // group
    abs_ = 0
    arrays = {"op": "tq_attn", "q": q.ravel(), "kd": kd.ravel(), "vd": vd.ravel(), "tab": _c(tab, np.float32)}
    if alibi is not None:
        alibi = _c(alibi, np.float32)
        abs_ = hq if alibi.ndim == 2 else 0
        arrays["alibi"] = alibi.ravel()
    arrays["uparams"] = np.array([b, lq, lk, hq, hkv, d, k_fmt[0], kl["code_bits"], kl["code_words"],
                                  kl["rsc_offset"], v_fmt[0], vl["code_bits"], vl["code_words"],
                                  vl["rsc_offset"], splits, gx, abs_, int(fp8), group], dtype=np.uint32)
    arrays["strides"] = np.array([hq * lq * w, lq * w, w, hkv * kcap * kw, kcap * kw, kw,
                                  hkv * vcap * vw, vcap * vw, vw], dtype=np.uint64)
    arrays["fparams"] = np.array([scale, softcap], dtype=np.float32)
    arrays["iparams"] = np.array([wl, wr], dtype=np.int32)
    return ref_run(arrays)["o"].reshape(b, hq, lq, d)


def ref_fa(q, k, v, scale, q_dtype=0, kv_dtype=0, kind=0, version=2, splits=1, group=1, wl=-1, wr=-1,
           softcap=0.0, kd=1.0, vd=1.0, cu_q=None, cu_k=None, alibi=None):
    """fa_row* / fa{2,3}_d* on the host emulator. Dense q (b, lq, hq, d), k / v (b, lk, hkv, d);
    varlen q (tq, hq, d) with cu_q / cu_k. q_dtype 0 f32 / 1 f16 / 2 bf16; kv_dtype 0 same / 1 fp8 /
    2 f16 / 3 bf16 (with f32 queries). kind 0 row kernel, 1 tile kernel. Returns f32 in q's shape."""
    q, k, v = _c(q, np.float32), _c(k, np.float32), _c(v, np.float32)
    varlen = cu_q is not None
    if varlen:
        cu_q, cu_k = _c(cu_q, np.uint32), _c(cu_k, np.uint32)
        b = len(cu_q) - 1
        tq, hq, d = q.shape
        hkv = k.shape[1]
        lq = int(np.max(np.diff(cu_q.astype(np.int64))))
        lk = int(np.max(np.diff(cu_k.astype(np.int64))))
        strides = [0, hq * d, d, 0, hkv * d, d, 0, hkv * d, d]
        total_q = tq
    else:
        b, lq, hq, d = q.shape
        lk, hkv = k.shape[1], k.shape[2]
        strides = [lq * hq * d, hq * d, d, lk * hkv * d, hkv * d, d, lk * hkv * d, hkv * d, d]
        total_q = b * lq
    dmax = 64 if d <= 64 else (128 if d <= 128 else 256)
    tiles = {(2, 64): 32, (2, 128): 16, (2, 256): 8, (3, 64): 64, (3, 128): 32, (3, 256): 16}
    gx = lq * hq // group if kind == 0 else -(-lq // tiles[(version, dmax)])
    abs_ = 0
    arrays = {"op": "fa", "q": q.ravel(), "k": k.ravel(), "v": v.ravel()}
    if alibi is not None:
        alibi = _c(alibi, np.float32)
        abs_ = hq if alibi.ndim == 2 else 0
        arrays["alibi"] = alibi.ravel()
    if varlen:
        arrays["cu_q"], arrays["cu_k"] = cu_q, cu_k
    arrays["dims"] = np.array([b, lq, lk, hq, hkv, d, total_q], dtype=np.uint32)
    arrays["strides"] = np.array(strides, dtype=np.uint64)
    arrays["fparams"] = np.array([scale, softcap, kd, vd], dtype=np.float32)
    arrays["iparams"] = np.array([wl, wr], dtype=np.int32)
    arrays["cfg"] = np.array([kind, dmax, version, splits, int(varlen), max(gx, 1), abs_, group], dtype=np.uint32)
    arrays["dtypes"] = np.array([q_dtype, kv_dtype], dtype=np.uint32)
    return ref_run(arrays)["o"].reshape(q.shape)
