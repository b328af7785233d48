"""Generates the golden fixtures in this folder from the reference's own kernel sources.

Run where the reference tree is mounted (it is compiled, unmodified, into oracle/_ref by
oracle/Makefile):

    python tests/golden/make_golden.py

Every fixture holds the seeded inputs' parameters and the outputs of the reference's host-emulated
kernels (candle-core/kernels/tests/accel_host_test.cpp driving turbo_quant_impl.h and
flash_attn_impl.h). Inputs are regenerated from the seeds by the oracle's SplitMix64 / Box-Muller
generator (candle-core/src/accel/turbo.rs:148-176), so only outputs are stored. The test suite
never needs the reference tree: it reads these files.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle as O  # noqa: E402

HERE = Path(__file__).resolve().parent

# (mode, bits, dim): the list of candle-core/tests/accel_kernels_host.rs:965-975 without the prod
# rows, plus every format at the head dim of the benchmark configurations.
QUANT_CASES = [
    (O.MSE, 4, 128), (O.MSE, 3, 96), (O.MSE, 1, 64), (O.MSE, 2, 128), (O.NVFP4, 4, 128), (O.MXFP4, 4, 64),
    (O.MXFP8, 4, 256), (O.FP8, 4, 80), (O.MXFP4, 4, 128), (O.MXFP8, 4, 128), (O.FP8, 4, 128),
    (O.NVFP4, 4, 64), (O.MSE, 4, 256), (O.FP8, 4, 256),
]


def quant_input(mode, bits, dim, rows=37, seed=77):
    """Rows with exact zeros, an all-zero row, an outlier row and a tiny row
    (accel_kernels_host.rs:980-984 plus edge rows)."""
    x = O.normal(seed + 1000 * mode + dim + bits, rows * dim).reshape(rows, dim).copy()
    x[0, 3] = 0.0
    x[1] = 0.0
    x[2] *= 1e-3
    x[3, 5] = 300.0
    x[4] *= 50.0
    x[5, ::7] = 0.0
    x[6] = 2.0 ** -130  # subnormal block maxima: MX scale code 0
    return x


def tab_for(mode, bits, dim):
    return O.codebook(dim, bits) if mode <= O.PROD else np.zeros(32, np.float32)


def gen_quant():
    out = {}
    for mode, bits, dim in QUANT_CASES:
        x = quant_input(mode, bits, dim)
        tab = tab_for(mode, bits, dim)
        for sd, name in ((0, "f32"), (1, "f16"), (2, "bf16")):
            key = f"m{mode}_b{bits}_d{dim}_{name}"
            words = O.ref_tq_quant(x, mode, bits, tab, src_dtype=sd)
            out[key] = words
            if sd == 0:
                out[key + "_deq"] = O.ref_tq_dequant(words, dim, mode, bits, tab)
        out[f"tab_m{mode}_b{bits}_d{dim}"] = tab
    np.savez_compressed(HERE / "tq_quant.npz", **out)
    print("tq_quant.npz", len(out), "arrays")


# (name, k_fmt, v_fmt, b, lq, lk, hq, hkv, d, splits, group, wl, wr, softcap, alibi, fp8)
ATTN_CASES = [
    ("fp8_g4_s3", (O.FP8, 4), (O.FP8, 4), 1, 1, 300, 8, 2, 128, 3, 4, -1, 0, 0.0, False, True),
    ("fp8_plain", (O.FP8, 4), (O.FP8, 4), 2, 1, 150, 4, 2, 128, 1, 1, -1, 0, 0.0, False, False),
    ("mxfp4_g4_s4", (O.MXFP4, 4), (O.MXFP4, 4), 2, 1, 517, 8, 2, 128, 4, 4, -1, 0, 0.0, False, False),
    ("mxfp8_g4_s2", (O.MXFP8, 4), (O.MXFP8, 4), 1, 1, 260, 8, 2, 128, 2, 4, -1, 0, 0.0, False, False),
    ("nvfp4_g8_s2", (O.NVFP4, 4), (O.NVFP4, 4), 1, 1, 200, 8, 1, 128, 2, 8, -1, 0, 0.0, False, False),
    ("turbo4_g8_s3", (O.MSE, 4), (O.MSE, 4), 1, 1, 333, 8, 1, 128, 3, 8, -1, 0, 0.0, False, False),
    ("turbo3_2_lq3", (O.MSE, 3), (O.MSE, 2), 1, 3, 70, 2, 1, 128, 3, 1, -1, 0, 0.0, False, False),
    ("nvfp4_mxfp4_cap", (O.NVFP4, 4), (O.MXFP4, 4), 1, 2, 64, 2, 2, 64, 2, 1, -1, -1, 20.0, False, False),
    ("fp8_mxfp8_d256", (O.FP8, 4), (O.MXFP8, 4), 1, 4, 33, 4, 1, 256, 1, 1, -1, 0, 0.0, False, False),
    ("mxfp4_window", (O.MXFP4, 4), (O.MXFP4, 4), 1, 2, 190, 4, 2, 128, 2, 2, 40, 0, 0.0, False, False),
    ("fp8_alibi", (O.FP8, 4), (O.FP8, 4), 2, 1, 97, 4, 2, 128, 1, 2, -1, 0, 0.0, True, True),
    ("mxfp4_d64", (O.MXFP4, 4), (O.MXFP4, 4), 2, 1, 130, 4, 1, 64, 2, 4, -1, 0, 0.0, False, False),
]


def attn_inputs(case):
    name, kf, vf, b, lq, lk, hq, hkv, d = case[:9]
    seed = 4000 + sum(ord(c) for c in name)
    n = b * hkv * lk
    kx = O.normal(seed, n * d, 1.5).reshape(n, d)
    vx = O.normal(seed + 1, n * d, 1.0).reshape(n, d)
    q = O.normal(seed + 2, b * hq * lq * d).reshape(b, hq, lq, d)
    tab = np.zeros(64, np.float32)
    tab[:32] = tab_for(kf[0], kf[1], d)
    tab[32:] = tab_for(vf[0], vf[1], d)
    kd = O.quantize_rows(kx, kf[0], kf[1], tab[:32]).reshape(b, hkv, lk, -1)
    vd = O.quantize_rows(vx, vf[0], vf[1], tab[32:]).reshape(b, hkv, lk, -1)
    alibi = (0.05 * (1 + np.arange(b * hq, dtype=np.float32))).reshape(b, hq) if case[14] else None
    return q, kd, vd, tab, alibi


def gen_attn():
    out = {}
    for case in ATTN_CASES:
        name, kf, vf, b, lq, lk, hq, hkv, d, splits, group, wl, wr, softcap, _, fp8 = case
        q, kd, vd, tab, alibi = attn_inputs(case)
        scale = 1.0 / np.sqrt(d)
        out[name] = O.ref_tq_attn(q, kd, vd, lk, kf, vf, scale, tab, splits=splits, group=group, wl=wl,
                                  wr=wr, softcap=softcap, alibi=alibi, fp8=fp8)
        print(" attn", name, out[name].shape)
    np.savez_compressed(HERE / "tq_attn.npz", **out)


# (name, q_dtype, kv_dtype, kind, version, b, lq, lk, hq, hkv, d, splits, group, wl, wr, softcap, varlen)
FA_CASES = [
    ("row_f32", 0, 0, 0, 2, 2, 1, 200, 4, 2, 128, 2, 1, -1, 0, 0.0, False),
    ("row_f16_g4", 1, 0, 0, 2, 1, 1, 300, 8, 2, 128, 3, 4, -1, 0, 0.0, False),
    ("row_bf16_fp8", 2, 1, 0, 2, 1, 2, 150, 4, 2, 64, 1, 2, -1, 0, 0.0, False),
    ("tile3_bf16", 2, 0, 1, 3, 1, 100, 100, 4, 2, 128, 1, 1, -1, 0, 0.0, False),
    ("tile2_f16_win", 1, 0, 1, 2, 1, 70, 90, 2, 1, 64, 1, 1, 20, 0, 30.0, False),
    ("tile3_f32_full", 0, 0, 1, 3, 2, 40, 40, 2, 2, 128, 1, 1, -1, -1, 0.0, False),
    ("varlen_bf16", 2, 0, 1, 3, 3, 0, 0, 4, 2, 128, 1, 1, -1, 0, 0.0, True),
]
VARLEN_Q = np.array([0, 37, 38, 90], dtype=np.uint32)
VARLEN_K = np.array([0, 50, 120, 172], dtype=np.uint32)


def fa_inputs(case):
    name, qd, kvd, kind, version, b, lq, lk, hq, hkv, d = case[:11]
    seed = 9000 + sum(ord(c) for c in name)
    if case[16]:
        tq, tk = int(VARLEN_Q[-1]), int(VARLEN_K[-1])
        q = O.normal(seed, tq * hq * d).reshape(tq, hq, d)
        k = O.normal(seed + 1, tk * hkv * d).reshape(tk, hkv, d)
        v = O.normal(seed + 2, tk * hkv * d).reshape(tk, hkv, d)
    else:
        q = O.normal(seed, b * lq * hq * d).reshape(b, lq, hq, d)
        k = O.normal(seed + 1, b * lk * hkv * d).reshape(b, lk, hkv, d)
        v = O.normal(seed + 2, b * lk * hkv * d).reshape(b, lk, hkv, d)
    return q, k, v


def gen_fa():
    out = {}
    for case in FA_CASES:
        name, qd, kvd, kind, version, b, lq, lk, hq, hkv, d, splits, group, wl, wr, softcap, varlen = case
        q, k, v = fa_inputs(case)
        kw = dict(cu_q=VARLEN_Q, cu_k=VARLEN_K) if varlen else {}
        kdesc = 0.5 if kvd == 1 else 1.0
        out[name] = O.ref_fa(q, k, v, 1.0 / np.sqrt(d), q_dtype=qd, kv_dtype=kvd, kind=kind, version=version,
                             splits=splits, group=group, wl=wl, wr=wr, softcap=softcap, kd=kdesc, vd=1.0, **kw)
        print(" fa", name, out[name].shape)
    np.savez_compressed(HERE / "flash_attn.npz", **out)


# prod (QJL) rows: (bits, dim); the sketch uses the quantizer's seed
PROD_CASES = [(4, 128), (2, 64), (5, 256), (3, 96)]
PROD_SEED = 42
# (name, bits, b, lq, lk, hq, hkv, d, splits, group, wl, wr): prod keys, 4-bit codebook values
PROD_ATTN_CASES = [("prod4_g2_s3", 4, 1, 2, 150, 4, 2, 128, 3, 2, -1, 0), ("prod3_window", 3, 2, 1, 77, 4, 1, 64, 1, 1, 30, 0)]


def prod_rows(y, bits, dim):
    """Stage one by the reference's tq_quant kernel, the residual and its projection by the oracle (the reference
    computes them with tensor operations on the host side), sign bits and residual norm by the reference's tq_signs."""
    tab = O.codebook(dim, bits - 1)
    s = O.qjl_matrix(dim, PROD_SEED)
    stage1 = O.ref_tq_quant(y, O.PROD, bits, tab)
    resid = O.tq_residual(y, stage1, bits, tab)
    proj = (resid.astype(np.float64) @ s.T.astype(np.float64)).astype(np.float32)
    return stage1, resid, proj, O.ref_tq_signs(stage1, proj, resid, bits), tab, s


def prod_attn_inputs(case):
    name, bits, b, lq, lk, hq, hkv, d = case[:8]
    seed = 6000 + sum(ord(c) for c in name)
    kx = O.normal(seed, b * hkv * lk * d, 1.5).reshape(-1, d)
    vx = O.normal(seed + 1, b * hkv * lk * d).reshape(-1, d)
    q = O.normal(seed + 2, b * hq * lq * d).reshape(b, hq, lq, d)
    _, _, _, kd, ktab, s = prod_rows(kx, bits, d)
    vtab = O.codebook(d, 4)
    vd = O.quantize_rows(vx, O.MSE, 4, vtab)
    tab = np.zeros(64, np.float32)
    tab[:32], tab[32:] = ktab, vtab
    qx = np.concatenate([q, (q.astype(np.float64) @ s.T.astype(np.float64)).astype(np.float32)], axis=-1)
    return qx, kd.reshape(b, hkv, lk, -1), vd.reshape(b, hkv, lk, -1), tab


def prod_attn_inputs_from(kd, case):
    """The inputs of a prod attention case with the key rows taken from the fixture (the reference's own rows): needs
    neither the reference tree nor a bit-identical host matmul for the keys."""
    name, bits, b, lq, lk, hq, hkv, d = case[:8]
    seed = 6000 + sum(ord(c) for c in name)
    vx = O.normal(seed + 1, b * hkv * lk * d).reshape(-1, d)
    q = O.normal(seed + 2, b * hq * lq * d).reshape(b, hq, lq, d)
    s = O.qjl_matrix(d, PROD_SEED)
    vtab = O.codebook(d, 4)
    tab = np.zeros(64, np.float32)
    tab[:32], tab[32:] = O.codebook(d, bits - 1), vtab
    qx = np.concatenate([q, (q.astype(np.float64) @ s.T.astype(np.float64)).astype(np.float32)], axis=-1)
    return qx, kd, O.quantize_rows(vx, O.MSE, 4, vtab).reshape(b, hkv, lk, -1), tab


def gen_prod():
    out = {}
    for bits, dim in PROD_CASES:
        y = quant_input(O.PROD, bits, dim)
        stage1, resid, proj, rows, tab, s = prod_rows(y, bits, dim)
        key = f"b{bits}_d{dim}"
        out[key + "_stage1"], out[key + "_resid"], out[key + "_proj"], out[key + "_rows"] = stage1, resid, proj, rows
    for case in PROD_ATTN_CASES:
        name, bits, b, lq, lk, hq, hkv, d, splits, group, wl, wr = case
        qx, kd, vd, tab = prod_attn_inputs(case)
        out[name + "_kd"] = kd
        out[name] = O.ref_tq_attn(qx, kd, vd, lk, (O.PROD, bits), (O.MSE, 4), 1.0 / np.sqrt(d), tab, splits=splits, group=group, wl=wl, wr=wr)
        print(" prod attn", name, out[name].shape)
    np.savez_compressed(HERE / "tq_prod.npz", **out)
    print("tq_prod.npz", len(out), "arrays")


def gen_misc():
    dec = O.ref_run({"op": "decoders"})
    rows, d, s = 5, 128, 4
    po = O.normal(31, s * rows * d).reshape(s, rows, d)
    pl = O.normal(32, s * rows, 3.0).reshape(s, rows).copy()
    pl[1, 2] = -np.inf
    pl[:, 4] = -np.inf
    comb = O.ref_run({"op": "combine", "part_o": po.ravel(), "part_lse": pl.ravel(),
                      "params": np.array([rows, d, s], dtype=np.uint32)})
    np.savez_compressed(HERE / "misc.npz", e4m3=dec["e4m3_ref"].view(np.uint32), e4m3_fast=dec["e4m3_fast"].view(np.uint32),
                        h2f=dec["h2f"].view(np.uint32), combine_t=comb["t"].reshape(rows, d),
                        combine_o=comb["o"].reshape(rows, d))
    print("misc.npz")


if __name__ == "__main__":
    if not O.ref_available():
        O.build()
    assert O.ref_available(), "oracle/_ref is not built (needs the reference tree)"
    gen_quant()
    gen_attn()
    gen_fa()
    gen_prod()
    gen_misc()
