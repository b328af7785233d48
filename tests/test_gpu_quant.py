"""GPU parity of the row quantizer, dequantizer and fused append through the C ABI: bit-exact
against the golden words of the reference's tq_quant kernels and against the CPU oracle."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest
import torch

from gpu_util import fmt, pkg, rows_dev, to_dev, words

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
spec = importlib.util.spec_from_file_location("make_golden", ROOT / "tests" / "golden" / "make_golden.py")
MG = importlib.util.module_from_spec(spec)
spec.loader.exec_module(MG)


@pytest.fixture(scope="module")
def P():
    return pkg()


@pytest.mark.parametrize("case", MG.QUANT_CASES, ids=lambda c: f"m{c[0]}b{c[1]}d{c[2]}")
def test_quantize_bit_exact_with_reference_kernels(P, golden, case):
    mode, bits, dim = case
    g = golden["tq_quant"]
    x = MG.quant_input(mode, bits, dim)
    qz = P.TurboQuantizer(fmt(P, mode, bits), dim, "none", 5)
    assert np.array_equal(qz.tab.cpu().numpy().view(np.uint32), g[f"tab_m{mode}_b{bits}_d{dim}"].view(np.uint32))
    for name in ("f32", "f16", "bf16"):
        got = words(qz.quantize_rows(to_dev(x, name)))
        want = g[f"m{mode}_b{bits}_d{dim}_{name}"]
        assert np.array_equal(got, want), f"{name}: {(got != want).sum()} words differ"
    deq = qz.dequantize_rows(rows_dev(g[f"m{mode}_b{bits}_d{dim}_f32"]))
    assert np.array_equal(deq.cpu().numpy().view(np.uint32), g[f"m{mode}_b{bits}_d{dim}_f32_deq"].view(np.uint32))


@pytest.mark.parametrize("mode,bits,dim", [(5, 4, 128), (4, 4, 128), (2, 4, 128), (3, 4, 128), (0, 4, 128), (0, 3, 128),
                                           (2, 4, 1024), (3, 4, 48), (5, 4, 33), (0, 2, 512)])
def test_quantize_bit_exact_with_oracle_many_rows(P, oracle, mode, bits, dim):
    rows = 4099  # not a multiple of the rows per block
    x = oracle.normal(900 + mode + dim, rows * dim).reshape(rows, dim)
    x[:, :3] *= 8.0  # outlier channels
    x[17] = 0.0
    qz = P.TurboQuantizer(fmt(P, mode, bits), dim, "none", 5)
    for name in ("bf16", "f32"):
        got = words(qz.quantize_rows(to_dev(x, name)))
        want = oracle.quantize_rows(oracle.round_to(x, name), mode, bits, qz.tab.cpu().numpy(), norm_order=1)
        assert np.array_equal(got, want), f"{name}: {(got != want).sum()} words differ"
    back = qz.dequantize_rows(rows_dev(want)).cpu().numpy()
    assert np.array_equal(back.view(np.uint32), oracle.dequantize_rows(want, dim, mode, bits, qz.tab.cpu().numpy()).view(np.uint32))


def test_quantize_edge_rows(P, oracle):
    dim = 128
    x = np.zeros((6, dim), np.float32)
    x[1] = 3.0e38  # (infinite inputs give NaN codes whose sign is platform defined: not compared)
    x[2, 0] = np.nan
    x[3] = 1e38
    x[4] = -2.0 ** -140
    x[5, ::2] = 448.0
    for mode in (5, 4, 2, 3):
        qz = P.TurboQuantizer(fmt(P, mode), dim, "none", 5)
        got = words(qz.quantize_rows(to_dev(x)))
        want = oracle.quantize_rows(x, mode)
        assert np.array_equal(got, want), mode
    empty = P.TurboQuantizer(fmt(P, 5), dim, "none", 5).quantize_rows(torch.empty((0, dim), device="cuda:0"))
    assert tuple(empty.shape) == (0, 34)


def boundary_rows(mode, dim=128):
    """Rows whose effective scale is exactly 1, filled with every midpoint between two neighbouring codes and the floats on
    either side of it, both signs: the ties-to-even cases of the 4-bit and 8-bit element codecs."""
    up = lambda a: np.nextafter(a, np.float32(np.inf), dtype=np.float32)
    dn = lambda a: np.nextafter(a, np.float32(0), dtype=np.float32)
    if mode in (2, 3):
        vals, top = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32), 6.0
    else:  # every non-negative finite e4m3 value: subnormals m / 512, normals (1 + m / 8) 2^(e - 7)
        vals = np.array([m / 512.0 for m in range(8)] + [(1 + m / 8.0) * 2.0 ** (e - 7) for e in range(1, 16) for m in range(8)][:-1], np.float32)
        top = 448.0
    mids = ((vals[:-1].astype(np.float64) + vals[1:].astype(np.float64)) / 2).astype(np.float32)
    pts = np.concatenate([mids, up(mids), dn(mids), vals, up(vals), dn(np.maximum(vals, np.float32(1e-30)))])
    pts = np.clip(np.concatenate([pts, -pts]), -top, top).astype(np.float32)
    # NVFP4: element 0 makes the global scale 1 and blocks 1-3 (block maximum 6) get a block scale of 1; the others:
    # element 0 makes the scale of the row (FP8) or of block 0 (MX) exactly 1
    slots = [16 * blk + j for blk in (1, 2, 3) for j in range(1, 16)] if mode == 3 else list(range(1, 32))
    nrow = (len(pts) + len(slots) - 1) // len(slots)
    x = np.zeros((nrow, dim), np.float32)
    x[:, 0] = 2688.0 if mode == 3 else top
    if mode == 3:
        x[:, 16:64:16] = top
    flat = np.zeros(nrow * len(slots), np.float32)
    flat[: len(pts)] = pts
    x[:, slots] = flat.reshape(nrow, len(slots))
    return x


@pytest.mark.parametrize("mode", [2, 3, 4, 5])
def test_quantize_rounding_boundaries(P, oracle, mode):
    x = boundary_rows(mode)
    qz = P.TurboQuantizer(fmt(P, mode), 128, "none", 5)
    got = words(qz.quantize_rows(to_dev(x)))
    want = oracle.quantize_rows(x, mode)
    assert np.array_equal(got, want), f"mode {mode}: {(got != want).sum()} words differ"


def test_append_positions_strides_and_growth(P, oracle):
    b, h, d = 3, 2, 128
    cache = P.TurboKvCache(fmt(P, 2), fmt(P, 4), d, "none", 42, 4)
    allk, allv = [], []
    for step, t in enumerate((5, 1, 1, 30, 1)):
        k = oracle.normal(100 + step, b * h * t * d).reshape(b, h, t, d)
        v = oracle.normal(200 + step, b * h * t * d).reshape(b, h, t, d)
        # (b, t, h, d) storage viewed as (b, h, t, d): the strides of a model's k / v projections
        kt = to_dev(k.transpose(0, 2, 1, 3), "f16").transpose(1, 2)
        vt = to_dev(v.transpose(0, 2, 1, 3), "f16").transpose(1, 2)
        cache.append(kt, vt)
        allk.append(k)
        allv.append(v)
    n = cache.seq_len()
    assert n == 38 and cache.cap >= 38
    K = oracle.round_to(np.concatenate(allk, axis=2), "f16")
    V = oracle.round_to(np.concatenate(allv, axis=2), "f16")
    assert np.array_equal(words(cache.k[:, :, :n]), oracle.quantize_rows(K.reshape(-1, d), 2).reshape(b, h, n, -1))
    assert np.array_equal(words(cache.v[:, :, :n]), oracle.quantize_rows(V.reshape(-1, d), 4).reshape(b, h, n, -1))
    assert int(cache.k[:, :, n:].abs().sum()) == 0  # spare capacity stays zero
    kk, vv = cache.keys_values()
    want = oracle.round_to(oracle.dequantize_rows(words(cache.k[:, :, :n]).reshape(-1, 19), d, 2), "f16")
    assert np.array_equal(kk.float().cpu().numpy().reshape(-1, d), want)
    cache.reset()
    assert cache.seq_len() == 0 and cache.storage_bytes() == 0


def test_append_per_sequence_positions(P, oracle):
    from candle_rocm_vulkan_b200.turbo_quant import _kv_append
    b, h, d, cap = 4, 2, 128, 16
    kq, vq = P.TurboQuantizer(fmt(P, 3), d, "none", 1), P.TurboQuantizer(fmt(P, 5), d, "none", 3)
    kc = torch.zeros((b, h, cap, kq.row_words()), dtype=torch.int32, device="cuda:0")
    vc = torch.zeros((b, h, cap, vq.row_words()), dtype=torch.int32, device="cuda:0")
    pos = torch.tensor([0, 3, 15, 7], dtype=torch.int32, device="cuda:0")
    k = oracle.normal(1, b * h * d).reshape(b, h, 1, d)
    v = oracle.normal(2, b * h * d).reshape(b, h, 1, d)
    _kv_append(to_dev(k, "bf16"), to_dev(v, "bf16"), kc, vc, kq, vq, pos)
    wk = oracle.quantize_rows(oracle.round_to(k, "bf16").reshape(-1, d), 3).reshape(b, h, -1)
    wv = oracle.quantize_rows(oracle.round_to(v, "bf16").reshape(-1, d), 5).reshape(b, h, -1)
    for bi, p_ in enumerate((0, 3, 15, 7)):
        assert np.array_equal(words(kc[bi, :, p_]), wk[bi]) and np.array_equal(words(vc[bi, :, p_]), wv[bi])
    assert int((kc != 0).any(dim=-1).sum()) == b * h


@pytest.mark.parametrize("mode", [0, 2])  # the general kernel (codebook rows) and the 128-element fast path
def test_append_positions_outside_the_cache_write_nothing(P, oracle, mode):
    """A device position below zero or at / past the capacity (a stale length word) must not make the kernel
    store outside its slab: the row is skipped and the status word says so; host positions are refused."""
    import ctypes as C
    from candle_rocm_vulkan_b200.turbo_quant import _kv_append
    A = P._abi
    b, h, d, cap = 4, 2, 128, 8
    kq, vq = P.TurboQuantizer(fmt(P, mode), d, "none", 1), P.TurboQuantizer(fmt(P, mode), d, "none", 3)
    rw = kq.row_words()
    # guard rows before and after every cache catch a store outside of it
    big_k = torch.full((b * h * cap + 2 * cap, rw), 0x5a5a5a5a, dtype=torch.int32, device="cuda:0")
    big_v = torch.full_like(big_k, 0x5a5a5a5a)
    kc = big_k[cap:cap + b * h * cap].view(b, h, cap, rw)
    vc = big_v[cap:cap + b * h * cap].view(b, h, cap, rw)
    kc.zero_()
    vc.zero_()
    pos = torch.tensor([2, cap, -1, cap + 1000], dtype=torch.int32, device="cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    k = oracle.normal(1, b * h * d).reshape(b, h, 1, d)
    v = oracle.normal(2, b * h * d).reshape(b, h, 1, d)
    _kv_append(to_dev(k, "bf16"), to_dev(v, "bf16"), kc, vc, kq, vq, pos, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 3
    tab = kq.tab.cpu().numpy()
    wk = oracle.quantize_rows(oracle.round_to(k, "bf16").reshape(-1, d), mode, 4, tab).reshape(b, h, -1)
    assert np.array_equal(words(kc[0, :, 2]), wk[0])            # the one valid position was written
    assert int((kc != 0).any(dim=-1).sum()) == h and int((vc != 0).any(dim=-1).sum()) == h   # and nothing else
    for big in (big_k, big_v):
        assert bool((big[:cap] == 0x5a5a5a5a).all()) and bool((big[cap + b * h * cap:] == 0x5a5a5a5a).all())
    # positions in range leave the status alone
    status.zero_()
    _kv_append(to_dev(k, "bf16"), to_dev(v, "bf16"), kc, vc, kq, vq, torch.tensor([0, 1, 7, 3], dtype=torch.int32, device="cuda:0"),
               status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # a host position past the end is refused before any launch
    with pytest.raises(A.B200Error):
        _kv_append(to_dev(k, "bf16"), to_dev(v, "bf16"), kc, vc, kq, vq, cap)


@pytest.mark.parametrize("mode,bits", [(0, 4), (3, 4), (2, 4), (5, 4)])
def test_hadamard_append_stages(P, oracle, mode, bits):
    """With rotation on, parity is per stage: the butterflies agree with the reference's matmul to
    rounding, and the quantizer is bit-exact on the rows it is given."""
    rows, d = 2048, 128
    x = oracle.normal(31 + mode, rows * d).reshape(rows, d)
    qz = P.TurboQuantizer(fmt(P, mode, bits), d, "hadamard", 42)
    assert np.array_equal(qz.signs.cpu().numpy(), oracle.hadamard_signs(d, 42))
    pi = oracle.rotation_matrix(d, 1, 42)
    y_gpu = qz.rotate(to_dev(x, "bf16")).cpu().numpy()
    y_ref = oracle.rotate_rows(oracle.round_to(x, "bf16"), pi)
    assert np.allclose(y_gpu, y_ref, atol=2e-5, rtol=1e-5)
    back = qz.unrotate(to_dev(y_gpu)).cpu().numpy()
    assert np.allclose(back, oracle.round_to(x, "bf16"), atol=2e-5)
    tab = qz.tab.cpu().numpy()
    fused = words(qz.quantize_rows(to_dev(x, "bf16")))
    assert np.array_equal(fused, oracle.quantize_rows(y_gpu, mode, bits, tab, norm_order=1))
    # end to end against the matmul rotation: rare flips where a value sits on a rounding boundary
    ref = oracle.quantize_rows(y_ref, mode, bits, tab, norm_order=1)
    lay = oracle.row_layout(mode, bits, d)
    diff_codes = np.unpackbits((fused[:, : lay["code_words"]] ^ ref[:, : lay["code_words"]]).view(np.uint8)).sum()
    assert diff_codes <= rows * d * lay["code_bits"] // 500


@pytest.mark.parametrize("bits,dim", [(4, 128), (2, 64), (5, 256), (3, 96)])
def test_prod_rows_bit_exact_with_reference_kernels(P, oracle, golden, bits, dim):
    """TurboProd (QJL) rows, stage by stage through the C ABI: stage one against the reference's tq_quant kernel, the
    residual against the oracle's bits, sign bits and residual norm against the reference's tq_signs kernel (on the
    fixture's projection, so that no matmul sits in the comparison); then the whole chain with the device's matmul."""
    import ctypes as C
    A = P._abi
    g, key = golden["tq_prod"], f"b{bits}_d{dim}"
    y = MG.quant_input(oracle.PROD, bits, dim)
    qz = P.TurboQuantizer(P.QuantFormat(A.TURBO_PROD, bits), dim, "none", MG.PROD_SEED)
    assert np.array_equal(qz.tab.cpu().numpy(), oracle.codebook(dim, bits - 1))
    assert np.array_equal(qz.qjl[0].cpu().numpy(), oracle.qjl_matrix(dim, MG.PROD_SEED))
    yd = to_dev(y)
    stage1 = qz.quantize_rotated_rows(yd)
    assert np.array_equal(words(stage1), g[key + "_stage1"])
    rows = y.shape[0]
    resid = torch.empty((rows, dim), dtype=torch.float32, device="cuda:0")
    ra = A.TqResidArgs(yd.data_ptr(), stage1.data_ptr(), qz.tab.data_ptr(), resid.data_ptr(), rows, dim, dim, 0, A.F32, bits)
    A.check(A.lib().b200_tq_residual(C.byref(ra), None))
    assert np.array_equal(resid.cpu().numpy().view(np.uint32), g[key + "_resid"].view(np.uint32))
    proj = to_dev(g[key + "_proj"])
    out = torch.empty_like(stage1)
    sa = A.TqSignsArgs(stage1.data_ptr(), proj.data_ptr(), resid.data_ptr(), out.data_ptr(), rows, dim, bits)
    A.check(A.lib().b200_tq_signs(C.byref(sa), None))
    assert np.array_equal(words(out), g[key + "_rows"])
    # the whole chain: sign bits may differ only where a projection is at rounding distance of zero
    full = words(qz.quantize_rows(yd))
    lay = oracle.row_layout(oracle.PROD, bits, dim)
    sw = slice(lay["code_words"], lay["code_words"] + (dim + 31) // 32)
    assert np.unpackbits((full ^ g[key + "_rows"])[:, sw].view(np.uint8)).sum() <= 3
    rest = np.ones(lay["row_words"], bool)
    rest[sw] = False
    assert np.array_equal(full[:, rest], g[key + "_rows"][:, rest])
    # dequantized estimate: codebook part + sketch part, against the oracle on the same rows
    want = (oracle.dequantize_rows(g[key + "_rows"], dim, oracle.PROD, bits, oracle.codebook(dim, bits - 1))
            + oracle.dequantize_qjl(g[key + "_rows"], dim, bits) @ oracle.qjl_matrix(dim, MG.PROD_SEED))
    got = qz.dequantize_rows(rows_dev(g[key + "_rows"])).cpu().numpy()
    assert np.allclose(got, want, atol=2e-5 * max(1.0, float(np.abs(want).max())), rtol=1e-5)
