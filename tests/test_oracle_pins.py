"""Pins the CPU oracle (oracle/tq_oracle.c) to the reference: the golden fixtures produced by the
reference's own kernel sources (tests/golden/make_golden.py) and the known-answer values asserted by
the reference's unit tests (candle-core/src/accel/formats.rs:414-504, turbo.rs:585-597,
attention.rs:741-877)."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
spec = importlib.util.spec_from_file_location("make_golden", ROOT / "tests" / "golden" / "make_golden.py")
MG = importlib.util.module_from_spec(spec)
spec.loader.exec_module(MG)


def test_e4m3_all_codes_roundtrip(oracle, golden):
    # formats.rs:414-432 and the exhaustive decoder check of accel_kernels_host.rs:650-681
    codes = np.arange(256, dtype=np.uint32)
    vals = oracle.e4m3_to_f32(codes)
    assert np.array_equal(vals.view(np.uint32), golden["misc"]["e4m3"])
    assert np.array_equal(golden["misc"]["e4m3"], golden["misc"]["e4m3_fast"])
    for c in range(256):
        v = vals[c]
        if np.isnan(v):
            continue
        back = int(oracle.f32_to_e4m3(np.float32(v)))
        if v == 0:
            assert back & 0x7F == 0
        else:
            assert back == c
    assert oracle.e4m3_to_f32(0x7E) == 448.0
    assert oracle.f32_to_e4m3(np.float32(1000.0)) == 0x7E
    assert oracle.f32_to_e4m3(np.float32(-1000.0)) == 0xFE
    assert oracle.e4m3_to_f32(0x01) == 0.001953125


def test_f16_decoder_all_codes(oracle, golden):
    l = oracle.lib()
    got = np.array([l.orc_h2f(h) for h in range(65536)], dtype=np.float32).view(np.uint32)
    want = golden["misc"]["h2f"]
    nan = (want & 0x7FFFFFFF) > 0x7F800000  # NaN payloads are quieted when ctypes widens the return value
    assert np.array_equal(got[~nan], want[~nan])
    assert np.array_equal(got[nan] | 0x00400000, want[nan] | 0x00400000)
    # and the encoder inverts it on every finite code
    h = np.arange(65536, dtype=np.uint16)
    f = h.view(np.float16).astype(np.float32)
    fin = np.isfinite(f)
    back = np.array([l.orc_f2h(float(x)) for x in f[fin][::37]], dtype=np.uint16)
    assert np.array_equal(back, h[fin][::37])


def test_fp4_codes(oracle):
    # formats.rs:447-458
    vals = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for c, v in enumerate(vals):
        assert oracle.fp4_to_f32(c) == v
        assert oracle.fp4_to_f32(c | 8) == -v
        assert oracle.f32_to_fp4(np.float32(v)) == c
    assert oracle.f32_to_fp4(np.float32(0.75)) == 2
    assert oracle.f32_to_fp4(np.float32(2.5)) == 4
    assert oracle.f32_to_fp4(np.float32(5.0)) == 6
    assert oracle.f32_to_fp4(np.float32(100.0)) == 7


def test_mx_scales_and_layouts(oracle):
    l = oracle.lib()
    # formats.rs:461-465
    assert l.orc_mx_scale_code(6.0, 2) == 127
    assert l.orc_e8m0_to_f32(l.orc_mx_scale_code(12.0, 2)) == 2.0
    assert l.orc_mx_scale_code(0.0, 2) == 0
    # formats.rs:468-477
    lay = oracle.row_layout(oracle.MSE, 3, 128)
    assert (lay["code_words"], lay["aux_words"], lay["row_words"]) == (12, 0, 14)
    lay = oracle.row_layout(oracle.PROD, 4, 128)
    assert (lay["code_words"], lay["aux_words"], lay["row_words"]) == (12, 4, 18)
    lay = oracle.row_layout(oracle.MXFP4, 4, 64)
    assert (lay["code_words"], lay["aux_words"]) == (8, 1)
    lay = oracle.row_layout(oracle.NVFP4, 4, 128)
    assert (lay["code_words"], lay["aux_words"]) == (16, 2)
    with pytest.raises(ValueError):
        oracle.row_layout(oracle.MXFP8, 4, 48)
    # row sizes at the head dim of the benchmark configurations
    assert [oracle.row_layout(m, 4, 128)["row_words"] for m in (5, 4, 2, 3, 0)] == [34, 35, 19, 20, 18]


def test_codebook_known_values(oracle):
    # turbo.rs:585-597 (the only pin available for the Lloyd-Max table)
    d = 128
    s = np.sqrt(np.float32(d))
    c = oracle.codebook(d, 2)[:4] * s
    assert abs(c[2] - 0.4528) < 0.01 and abs(c[3] - 1.5104) < 0.02 and abs(c[0] + c[3]) < 1e-6
    assert abs(oracle.codebook(d, 1)[1] * s - 0.7979) < 0.01
    t = oracle.codebook(d, 4)
    assert np.all(np.diff(t[:16]) > 0) and np.all(np.isinf(t[31:]))
    assert np.allclose(t[16:31], 0.5 * (t[:15] + t[1:16]), atol=1e-7)


def test_rotations_orthogonal(oracle):
    # turbo.rs:600-615
    for d, kind in ((64, 1), (48, 2), (16, 0)):
        m = oracle.rotation_matrix(d, kind, 7).astype(np.float64)
        assert np.allclose(m @ m.T, np.eye(d), atol=1e-4)
    s = oracle.hadamard_signs(128, 42)
    assert set(np.unique(s)) <= {-1.0, 1.0}
    m = oracle.rotation_matrix(128, 1, 42)
    assert np.array_equal(np.sign(m[0]), s)  # row 0 of H is all +


def test_known_answers_of_the_reference_unit_tests(oracle):
    # words produced by the reference's tq_quant kernels for a closed-form input
    i = np.arange(512)
    x = (((i * 37) % 101 - 50) / 10).astype(np.float32).reshape(4, 128)
    x[1] = 0
    w = oracle.quantize_rows(x, oracle.MXFP4)
    assert [int(v) for v in w[0, :4]] == [0x1D59E4BE, 0x0E5AE3C6, 0x9E4B62D6, 0xB63C61D5]
    assert int(w[0, 16]) == 0x7F7F7F7F and int(w[0, 17]) == 0x3F800000 and int(w[3, 0]) == 0xD60E5AE4
    w = oracle.quantize_rows(x, oracle.NVFP4)
    assert [int(v) for v in w[0, 16:19]] == [0x7E7D7E7E, 0x7D7E7D7E, 0x3AF3CF3D]
    w = oracle.quantize_rows(x, oracle.FP8)
    assert int(w[0, 0]) == 0xFB75EFFE and int(w[0, 32]) == 0x3C36DB6E
    assert np.all(w[1, :32] == 0) and int(w[1, 32]) == 0x3F800000
    w = oracle.quantize_rows(x, oracle.MXFP8)
    assert int(w[0, 0]) == 0xF872EAFA and int(w[0, 32]) == 0x79797979


@pytest.mark.parametrize("case", MG.QUANT_CASES, ids=lambda c: f"m{c[0]}b{c[1]}d{c[2]}")
def test_quantize_matches_reference_kernels(oracle, golden, case):
    mode, bits, dim = case
    g = golden["tq_quant"]
    x = MG.quant_input(mode, bits, dim)
    tab = g[f"tab_m{mode}_b{bits}_d{dim}"]
    assert np.array_equal(tab.view(np.uint32), MG.tab_for(mode, bits, dim).view(np.uint32))
    for name in ("f32", "f16", "bf16"):
        want = g[f"m{mode}_b{bits}_d{dim}_{name}"]
        got = oracle.quantize_rows(oracle.round_to(x, name), mode, bits, tab, norm_order=1)
        assert np.array_equal(got, want), f"{name}: {(got != want).sum()} words differ"
    deq = oracle.dequantize_rows(g[f"m{mode}_b{bits}_d{dim}_f32"], dim, mode, bits, tab)
    assert np.array_equal(deq.view(np.uint32), g[f"m{mode}_b{bits}_d{dim}_f32_deq"].view(np.uint32))
    if mode <= oracle.PROD:
        # the CPU codec sums the norm sequentially: rare code flips only (accel_kernels_host.rs:1022-1027)
        seq = oracle.quantize_rows(x, mode, bits, tab, norm_order=0)
        lay = oracle.row_layout(mode, bits, dim)
        want = g[f"m{mode}_b{bits}_d{dim}_f32"]
        flips = 0
        for j in range(dim):
            pos = j * bits
            a = (seq[:, pos >> 5] >> (pos & 31)) & ((1 << min(bits, 32 - (pos & 31))) - 1)
            b = (want[:, pos >> 5] >> (pos & 31)) & ((1 << min(bits, 32 - (pos & 31))) - 1)
            flips += int((a != b).sum())
        assert flips <= x.size // 1000 + 1
        r0s, r0t = seq[:, lay["rsc_offset"]].view(np.float32), g[f"m{mode}_b{bits}_d{dim}_f32"][:, lay["rsc_offset"]].view(np.float32)
        assert np.allclose(r0s, r0t, rtol=1e-5)


@pytest.mark.parametrize("case", MG.ATTN_CASES, ids=lambda c: c[0])
def test_packed_attention_matches_reference_kernels(oracle, golden, case):
    name, kf, vf, b, lq, lk, hq, hkv, d, splits, group, wl, wr, softcap, _, _ = case
    q, kd, vd, tab, alibi = MG.attn_inputs(case)
    got = oracle.tq_attention(q, kd, vd, lk, kf, vf, 1.0 / np.sqrt(d), tab, wl=wl, wr=wr, softcap=softcap, alibi=alibi)
    want = golden["tq_attn"][name]
    # the reference's own bar between its kernels and its CPU code (accel_kernels_host.rs:405-410)
    assert np.allclose(got, want, atol=2e-5, rtol=1e-4), np.abs(got - want).max()


@pytest.mark.parametrize("case", MG.FA_CASES, ids=lambda c: c[0])
def test_dense_attention_matches_reference_kernels(oracle, golden, case):
    name, qd, kvd, kind, version, b, lq, lk, hq, hkv, d, splits, group, wl, wr, softcap, varlen = case
    q, k, v = MG.fa_inputs(case)
    qn = {0: "f32", 1: "f16", 2: "bf16"}[qd]
    q = oracle.round_to(q, qn)
    kdesc = 1.0
    if kvd == 1:
        k = oracle.e4m3_to_f32(oracle.f32_to_e4m3(k))
        v = oracle.e4m3_to_f32(oracle.f32_to_e4m3(v))
        kdesc = 0.5
    else:
        k, v = oracle.round_to(k, qn), oracle.round_to(v, qn)
    kw = dict(cu_q=MG.VARLEN_Q, cu_k=MG.VARLEN_K, max_q=52, max_k=70) if varlen else {}
    got = oracle.reference_attention(q, k, v, 1.0 / np.sqrt(d), wl=wl, wr=wr, softcap=softcap, k_descale=kdesc, **kw)
    got = oracle.round_to(got, qn)
    want = golden["flash_attn"][name]
    atol, rtol = {"f32": (2e-5, 1e-4), "f16": (2e-3, 2e-3), "bf16": (1.6e-2, 1.6e-2)}[qn]
    assert np.allclose(got, want, atol=atol, rtol=rtol), np.abs(got - want).max()


def test_combine_matches_reference_kernels(oracle, golden):
    rows, d, s = 5, 128, 4
    po = oracle.normal(31, s * rows * d).reshape(s, rows, d)
    pl = oracle.normal(32, s * rows, 3.0).reshape(s, rows).copy()
    pl[1, 2] = -np.inf
    pl[:, 4] = -np.inf
    got = oracle.combine(po, pl)
    assert np.array_equal(got.view(np.uint32), golden["misc"]["combine_t"].view(np.uint32))
    assert np.array_equal(golden["misc"]["combine_t"], golden["misc"]["combine_o"])


def test_split_heuristic_known_values(oracle):
    # attention.rs:486-506 evaluated by hand for a 148 SM device
    assert oracle.row_group(32, 8) == 4 and oracle.row_group(64, 8) == 8 and oracle.row_group(6, 2) == 1
    assert oracle.split_count_grouped(32, 4, 2048, 148) == 32
    assert oracle.split_count_grouped(256, 8, 32768, 148) == 64
    assert oracle.split_count_grouped(4096, 4, 16384, 148) == 10
    assert oracle.split_count_grouped(16, 1, 100, 16) == 1


def test_unfused_path_equals_reference_attention(oracle):
    # candle-nn/src/flash_attn.rs:1027-1050: fused CPU vs unfused < 1e-5
    b, lq, lk, hq, hkv, d = 2, 5, 40, 4, 2, 64
    q = oracle.normal(1, b * lq * hq * d).reshape(b, lq, hq, d)
    k = oracle.normal(2, b * lk * hkv * d).reshape(b, lk, hkv, d)
    v = oracle.normal(3, b * lk * hkv * d).reshape(b, lk, hkv, d)
    for wl, wr in ((-1, 0), (-1, -1), (3, 0)):
        a = oracle.reference_attention(q, k, v, 0.125, wl=wl, wr=wr)
        u = oracle.unfused_attention(q, k, v, 0.125, wl=wl, wr=wr)
        assert np.allclose(a, u, atol=1e-5)


@pytest.mark.parametrize("bits,dim", MG.PROD_CASES)
def test_prod_rows_pinned_to_reference_kernels(oracle, golden, bits, dim):
    """TurboProd rows: stage one against the reference's tq_quant kernel, sign bits and residual norm against its
    tq_signs kernel (on the fixture's residual and projection, so that no host matmul sits in the comparison)."""
    g, key = golden["tq_prod"], f"b{bits}_d{dim}"
    y = MG.quant_input(oracle.PROD, bits, dim)
    tab = oracle.codebook(dim, bits - 1)
    stage1 = oracle.quantize_rows(y, oracle.PROD, bits, tab)
    assert np.array_equal(stage1, g[key + "_stage1"])
    resid = oracle.tq_residual(y, stage1, bits, tab)
    assert np.array_equal(resid.view(np.uint32), g[key + "_resid"].view(np.uint32))
    assert np.array_equal(oracle.tq_signs(stage1, g[key + "_proj"], resid, bits), g[key + "_rows"])
    # the whole chain (with this machine's matmul): sign bits may differ only where a projection is at rounding distance of zero
    rows = oracle.quantize_rows_prod(y, bits, tab, oracle.qjl_matrix(dim, MG.PROD_SEED))
    lay = oracle.row_layout(oracle.PROD, bits, dim)
    flips = np.unpackbits((rows ^ g[key + "_rows"])[:, lay["code_words"]:lay["code_words"] + (dim + 31) // 32].view(np.uint8)).sum()
    assert flips <= 2
    # QJL coefficients: +-c by sign bit
    zs = oracle.dequantize_qjl(g[key + "_rows"], dim, bits)
    c = g[key + "_rows"][:, lay["rsc_offset"]].view(np.float32) * g[key + "_rows"][:, lay["rsc_offset"] + 1].view(np.float32)
    assert np.allclose(np.abs(zs), (c * np.float32(1.2533141) / np.float32(dim))[:, None], rtol=1e-6)


@pytest.mark.parametrize("case", MG.PROD_ATTN_CASES, ids=lambda c: c[0])
def test_prod_attention_pinned_to_reference_kernels(oracle, golden, case):
    name, bits, b, lq, lk, hq, hkv, d, splits, group, wl, wr = case
    qx, kd, vd, tab = MG.prod_attn_inputs_from(golden["tq_prod"][name + "_kd"], case)
    got = oracle.tq_attention(qx, kd, vd, lk, (oracle.PROD, bits), (oracle.MSE, 4), 1.0 / np.sqrt(d), tab, wl=wl, wr=wr)
    assert np.allclose(got, golden["tq_prod"][name], atol=1e-4, rtol=2e-5)
