"""GPU parity of the attention over dense K / V (b200_flash_attn, b200_fa_prefill_append) through the C
ABI: against the outputs of the reference's fa_row / fa2 / fa3 kernels (golden fixtures), against the
CPU oracle on seeded inputs, and through properties at prefill sizes."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest
import torch

from gpu_util import assert_close, fmt, pkg, to_dev, words

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
spec = importlib.util.spec_from_file_location("make_golden", ROOT / "tests" / "golden" / "make_golden.py")
MG = importlib.util.module_from_spec(spec)
spec.loader.exec_module(MG)
QN = {0: "f32", 1: "f16", 2: "bf16"}


@pytest.fixture(scope="module")
def P():
    return pkg()


def fp8_dev(oracle, x):
    """f32 -> E4M3 codes on the device (uint8) and the values they decode to."""
    codes = oracle.f32_to_e4m3(x).astype(np.uint8).reshape(x.shape)
    return torch.from_numpy(codes).to("cuda:0"), oracle.e4m3_to_f32(codes).reshape(x.shape)


def cfg_of(P, d, wl=-1, wr=-1, softcap=0.0, alibi=None, kd=1.0, vd=1.0, scale=None):
    c = P.FlashAttnConfig(scale if scale is not None else 1.0 / np.sqrt(d))
    c.window_size_left = None if wl < 0 else wl
    c.window_size_right = None if wr < 0 else wr
    c.softcap = softcap or None
    c.k_descale, c.v_descale = kd, vd
    if alibi is not None:
        c.alibi_slopes = to_dev(alibi)
    return c


@pytest.mark.parametrize("case", MG.FA_CASES, ids=lambda c: c[0])
def test_against_reference_kernel_outputs(P, oracle, golden, case):
    name, qd, kvd, kind, version, b, lq, lk, hq, hkv, d, splits, group, wl, wr, softcap, varlen = case
    q, k, v = MG.fa_inputs(case)
    qn = QN[qd]
    F = P.flash_attn
    qt = to_dev(q, qn)
    kdesc = 1.0
    if kvd == 1:
        kt, _ = fp8_dev(oracle, k)
        vt, _ = fp8_dev(oracle, v)
        kdesc = 0.5
    else:
        kt, vt = to_dev(k, qn), to_dev(v, qn)
    c = cfg_of(P, d, wl, wr, softcap, kd=kdesc)
    if varlen:
        cu_q = torch.from_numpy(MG.VARLEN_Q.astype(np.int32)).to("cuda:0")
        cu_k = torch.from_numpy(MG.VARLEN_K.astype(np.int32)).to("cuda:0")
        out = F.flash_attn_varlen_with_config(qt, kt, vt, cu_q, cu_k, 52, 70, c)
    else:
        out = F.flash_attn_with_config(qt, kt, vt, c)
    torch.cuda.synchronize()
    assert out.dtype == qt.dtype and out.shape == qt.shape
    # the fixture holds the reference kernel's output rounded to the output dtype: one more half ulp
    assert_close(out.float().cpu().numpy(), golden["flash_attn"][name], what=name, out=qn,
                 rtol=2e-3 + {"f32": 0.0, "f16": 2.0 ** -12, "bf16": 2.0 ** -9}[qn])


ORACLE_CASES = [
    # name, qdt, b, lq, lk, hq, hkv, d, wl, wr, softcap, alibi, fp8
    ("decode_split", "bf16", 2, 1, 3000, 8, 2, 128, -1, 0, 0.0, False, False),
    ("decode_lq3_g8", "f16", 1, 3, 1500, 16, 2, 128, -1, 0, 0.0, False, False),
    ("prefill_causal", "bf16", 2, 300, 300, 8, 2, 128, -1, 0, 0.0, False, False),
    ("prefill_chunk", "f16", 1, 130, 450, 4, 4, 64, -1, 0, 0.0, False, False),
    ("window_left", "bf16", 1, 200, 260, 4, 2, 128, 33, 0, 0.0, False, False),
    ("window_both", "f16", 1, 150, 150, 2, 1, 64, 10, 7, 0.0, False, False),
    ("softcap_alibi", "f16", 2, 70, 90, 4, 2, 128, -1, 0, 20.0, True, False),
    ("full_noncausal", "f32", 1, 65, 129, 6, 3, 128, -1, -1, 0.0, False, False),
    ("fp8_prefill", "bf16", 1, 100, 164, 8, 2, 128, -1, 0, 0.0, False, True),
    ("fp8_decode_d64", "f16", 3, 1, 2100, 4, 1, 64, -1, 0, 0.0, False, True),
    ("lq_longer_than_lk", "f16", 1, 80, 50, 2, 2, 64, -1, 0, 0.0, False, False),
    # 512 packed rows and more with head dim 128: the tcgen05 tiles (many key tiles, windows, ragged ends)
    ("tc_chunked_prefill", "bf16", 2, 333, 1000, 8, 2, 128, -1, 0, 0.0, False, False),
    ("tc_f16_noncausal", "f16", 1, 130, 777, 4, 1, 128, -1, -1, 0.0, False, False),
    ("tc_window", "bf16", 1, 700, 700, 2, 2, 128, 100, 0, 0.0, False, False),
    ("tc_lq_longer", "f16", 1, 600, 450, 4, 4, 128, -1, 0, 0.0, False, False),
    # 1024 packed rows and more: blocks of two row tiles
    ("tc2_ragged_rows", "bf16", 1, 530, 900, 4, 2, 128, -1, 0, 0.0, False, False),
    ("tc2_window", "f16", 2, 300, 640, 8, 2, 128, 70, 0, 0.0, False, False),
    # every head dim that is a multiple of 8 up to 256 (the reference takes any d <= 256): buckets 64 / 128 / 256
    ("d256_decode", "bf16", 2, 1, 2200, 8, 2, 256, -1, 0, 0.0, False, False),
    ("d256_prefill", "f16", 1, 140, 200, 4, 2, 256, -1, 0, 0.0, False, False),
    ("d256_fp8_window", "bf16", 1, 70, 300, 4, 1, 256, 50, 0, 0.0, False, True),
    ("d192_f32_alibi", "f32", 1, 66, 130, 6, 3, 192, -1, 0, 15.0, True, False),
    ("d96_prefill", "f16", 2, 90, 90, 4, 2, 96, -1, 0, 0.0, False, False),
    ("d40_decode", "bf16", 1, 2, 1300, 4, 4, 40, -1, 0, 0.0, False, False),
    ("d8_noncausal", "f16", 1, 33, 47, 2, 1, 8, -1, -1, 0.0, False, False),
    # decode calls (at most 16 packed rows per kv head): the warps share the keys of a tile and merge at the end
    ("dec_16_rows_exactly", "bf16", 2, 4, 1000, 8, 2, 128, -1, 0, 0.0, False, False),
    ("dec_window_softcap_alibi", "f16", 3, 2, 777, 8, 4, 128, 300, 0, 25.0, True, False),
    ("dec_f32_q_short", "f32", 1, 1, 37, 4, 1, 64, -1, 0, 0.0, False, False),
    ("dec_many_blocks", "bf16", 38, 1, 1030, 8, 8, 64, -1, 0, 0.0, False, False),
    ("dec_lq_longer_than_lk", "f16", 1, 5, 3, 2, 1, 128, -1, 0, 0.0, False, False),
]


@pytest.mark.parametrize("case", ORACLE_CASES, ids=lambda c: c[0])
def test_against_oracle(P, oracle, case):
    name, qn, b, lq, lk, hq, hkv, d, wl, wr, softcap, use_alibi, fp8 = case
    seed = 500 + sum(ord(ch) for ch in name)
    q = oracle.round_to(oracle.normal(seed, b * lq * hq * d).reshape(b, lq, hq, d), qn)
    k = oracle.normal(seed + 1, b * lk * hkv * d).reshape(b, lk, hkv, d)
    v = oracle.normal(seed + 2, b * lk * hkv * d).reshape(b, lk, hkv, d)
    alibi = (0.05 * np.abs(oracle.normal(seed + 3, b * hq))).reshape(b, hq).astype(np.float32) if use_alibi else None
    kd, vd = (0.75, 1.5) if fp8 else (1.0, 1.0)
    if fp8:
        kt, k = fp8_dev(oracle, k)
        vt, v = fp8_dev(oracle, v)
    else:
        k, v = oracle.round_to(k, qn), oracle.round_to(v, qn)
        kt, vt = to_dev(k, qn), to_dev(v, qn)
    want = oracle.reference_attention(q, k, v, 1.0 / np.sqrt(d), wl=wl, wr=wr, softcap=softcap, alibi=alibi, k_descale=kd, v_descale=vd)
    out = P.flash_attn.flash_attn_with_config(to_dev(q, qn), kt, vt, cfg_of(P, d, wl, wr, softcap, alibi, kd, vd))
    torch.cuda.synchronize()
    assert_close(out.float().cpu().numpy(), want, what=name, out=qn)


def test_rows_without_visible_keys_are_zero(P, oracle):
    # lq > lk under a causal window: the first lq - lk query rows see no key (flash_attn_impl.h: zeros)
    b, lq, lk, hq, hkv, d = 1, 80, 50, 2, 2, 64
    q = torch.randn((b, lq, hq, d), device="cuda:0", dtype=torch.float16)
    k = torch.randn((b, lk, hkv, d), device="cuda:0", dtype=torch.float16)
    v = torch.randn((b, lk, hkv, d), device="cuda:0", dtype=torch.float16)
    out = P.flash_attn.flash_attn(q, k, v, 0.125, True)
    torch.cuda.synchronize()
    assert torch.count_nonzero(out[:, : lq - lk]) == 0
    assert torch.isfinite(out).all()


def test_bhsd_views_and_named_entry_points(P, oracle):
    b, s, hq, hkv, d = 2, 96, 4, 2, 128
    q = oracle.round_to(oracle.normal(1, b * hq * s * d).reshape(b, hq, s, d), "bf16")
    k = oracle.round_to(oracle.normal(2, b * hkv * s * d).reshape(b, hkv, s, d), "bf16")
    v = oracle.round_to(oracle.normal(3, b * hkv * s * d).reshape(b, hkv, s, d), "bf16")
    F = P.flash_attn
    qt, kt, vt = to_dev(q, "bf16"), to_dev(k, "bf16"), to_dev(v, "bf16")
    want = oracle.reference_attention(q.transpose(0, 2, 1, 3), k.transpose(0, 2, 1, 3), v.transpose(0, 2, 1, 3), 0.1, wr=0)
    got = F.flash_attn_bhsd(qt, kt, vt, P.FlashAttnConfig(0.1).causal())
    torch.cuda.synchronize()
    assert got.shape == qt.shape
    assert_close(got.float().cpu().numpy().transpose(0, 2, 1, 3), want, what="bhsd", out="bf16")
    a = F.flash_attn(qt.transpose(1, 2), kt.transpose(1, 2), vt.transpose(1, 2), 0.1, True)
    w = F.flash_attn_windowed(qt.transpose(1, 2), kt.transpose(1, 2), vt.transpose(1, 2), 0.1, None, 0)
    torch.cuda.synchronize()
    assert torch.equal(a, w) and torch.equal(a, got.transpose(1, 2))


def test_varlen_equals_per_sequence_calls(P):
    torch.manual_seed(5)
    hq, hkv, d = 8, 2, 128
    lens_q, lens_k = [5, 130, 1, 64], [70, 130, 900, 64]
    cu_q = torch.tensor([0] + list(np.cumsum(lens_q)), dtype=torch.int32, device="cuda:0")
    cu_k = torch.tensor([0] + list(np.cumsum(lens_k)), dtype=torch.int32, device="cuda:0")
    q = torch.randn((sum(lens_q), hq, d), device="cuda:0", dtype=torch.bfloat16)
    k = torch.randn((sum(lens_k), hkv, d), device="cuda:0", dtype=torch.bfloat16)
    v = torch.randn((sum(lens_k), hkv, d), device="cuda:0", dtype=torch.bfloat16)
    F = P.flash_attn
    out = F.flash_attn_varlen(q, k, v, cu_q, cu_k, max(lens_q), max(lens_k), d ** -0.5, True)
    for i in range(len(lens_q)):
        qs, ks = slice(int(cu_q[i]), int(cu_q[i + 1])), slice(int(cu_k[i]), int(cu_k[i + 1]))
        one = F.flash_attn(q[qs][None], k[ks][None], v[ks][None], d ** -0.5, True)[0]
        assert_close(out[qs].float().cpu().numpy(), one.float().cpu().numpy(), atol=2e-3, what=f"sequence {i}", out="bf16")


def test_blocks_match_the_oracle_on_the_concatenated_rows(P, oracle):
    """Dense K / V in paged blocks (decode of 2 tokens and a chunk of 70): the keys are the valid rows of the blocks in
    order; capacity rows past `rows` hold garbage that must not be read."""
    b, hq, hkv, d = 2, 8, 2, 128
    rows = [37, 0, 128, 5]
    caps = [64, 16, 128, 8]
    lk = sum(rows)
    k = oracle.round_to(oracle.normal(11, b * hkv * lk * d).reshape(b, hkv, lk, d), "bf16")
    v = oracle.round_to(oracle.normal(12, b * hkv * lk * d).reshape(b, hkv, lk, d), "bf16")
    blocks, at = [], 0
    for r, c in zip(rows, caps):
        kb = torch.full((b, hkv, c, d), 1e4, device="cuda:0", dtype=torch.bfloat16)
        vb = torch.full((b, hkv, c, d), -1e4, device="cuda:0", dtype=torch.bfloat16)
        kb[:, :, :r] = to_dev(k[:, :, at : at + r], "bf16")
        vb[:, :, :r] = to_dev(v[:, :, at : at + r], "bf16")
        blocks.append(P.KvBlockRef(kb, vb, r))
        at += r
    for lq in (2, 70):
        q = oracle.round_to(oracle.normal(13 + lq, b * hq * lq * d).reshape(b, hq, lq, d), "bf16")
        want = oracle.reference_attention(q.transpose(0, 2, 1, 3), k.transpose(0, 2, 1, 3), v.transpose(0, 2, 1, 3), d ** -0.5, wr=0)
        got = P.flash_attn.flash_attn_blocks(to_dev(q, "bf16"), blocks, P.FlashAttnConfig(d ** -0.5).causal())
        torch.cuda.synchronize()
        assert got.shape == (b, hq, lq, d)
        assert_close(got.float().cpu().numpy().transpose(0, 2, 1, 3), want, what=f"blocks lq={lq}", out="bf16")


@pytest.mark.parametrize("dt,d,page,nblk,lq,wl", [(torch.bfloat16, 128, 16, 300, 1, -1), (torch.float16, 64, 32, 70, 3, 500),
                                                   (torch.float32, 256, 8, 90, 1, -1), ("fp8", 128, 16, 150, 2, -1),
                                                   (torch.bfloat16, 128, 64, 40, 300, -1)])
def test_many_blocks_read_in_place_equal_the_concatenated_call(P, dt, d, page, nblk, lq, wl):
    """b200_flash_attn_paged over hundreds of blocks of one page each, carved out of one pool in shuffled order (so
    that consecutive keys live far apart), the last block partly filled, one block empty: decode with key splits, a
    few query tokens, a chunk of prefill. Against b200_flash_attn on the same rows concatenated, which reads the same
    values in the same tiles: identical bits. Rows of the pool are wider than the head dim (a row stride of its own)."""
    F = P.flash_attn
    b, hq, hkv = 3, 8, 2
    g = torch.Generator(device="cuda:0").manual_seed(nblk)
    fp8 = dt == "fp8"
    store = torch.float32 if fp8 else dt
    pool_k = torch.randn((nblk, b, hkv, page, d + 16), generator=g, device="cuda:0").to(store)
    pool_v = torch.randn((nblk, b, hkv, page, d + 16), generator=g, device="cuda:0").to(store)
    if fp8:
        pool_k, pool_v = (pool_k * 0.5).to(torch.float8_e4m3fn), (pool_v * 0.5).to(torch.float8_e4m3fn)
    order = torch.randperm(nblk, generator=g, device="cuda:0").tolist()
    blocks = []
    for n, i in enumerate(order):
        rows = page if n < nblk - 1 else max(1, page // 3)
        if n == nblk // 2:
            rows = 0
        blocks.append(P.KvBlockRef(pool_k[i, :, :, :, :d], pool_v[i, :, :, :, :d], rows))
    qdt = torch.bfloat16 if fp8 else dt
    q = torch.randn((b, hq, lq, d), generator=g, device="cuda:0").to(qdt)
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    if wl >= 0:
        cfg = cfg.window(wl, 0)
    if fp8:
        cfg.k_descale, cfg.v_descale = 2.0, 2.0
    got = F.flash_attn_blocks(q, blocks, cfg)
    k = torch.cat([blk.k[:, :, : blk.rows] for blk in blocks], dim=2)
    v = torch.cat([blk.v[:, :, : blk.rows] for blk in blocks], dim=2)
    want = F.flash_attn_bhsd(q, k, v, cfg)
    torch.cuda.synchronize()
    assert got.shape == want.shape and torch.isfinite(got.float()).all()
    if lq * (hq // hkv) >= 512 and d == 128:
        # the concatenated call of this size runs on the tcgen05 tiles, the paged one on the general kernel
        assert_close(got.float().cpu().numpy(), want.float().cpu().numpy(), what="paged prefill chunk", out="bf16")
    else:
        assert torch.equal(got, want)


def test_paged_varlen_equals_varlen_on_gathered_pages(P):
    torch.manual_seed(9)
    hq, hkv, d, page, nblk = 8, 2, 128, 16, 40
    lens_q, lens_k = [3, 40, 1], [33, 40, 130]
    cu_q = torch.tensor([0] + list(np.cumsum(lens_q)), dtype=torch.int32, device="cuda:0")
    cu_k = torch.tensor([0] + list(np.cumsum(lens_k)), dtype=torch.int32, device="cuda:0")
    kp = torch.randn((nblk, page, hkv, d), device="cuda:0", dtype=torch.float16)
    vp = torch.randn((nblk, page, hkv, d), device="cuda:0", dtype=torch.float16)
    perm = torch.randperm(nblk)[: sum((n + page - 1) // page for n in lens_k)].tolist()
    table = torch.zeros((3, 9), dtype=torch.int32)
    ks, vs, at = [], [], 0
    for i, n in enumerate(lens_k):
        nb = (n + page - 1) // page
        ids = perm[at : at + nb]
        at += nb
        table[i, :nb] = torch.tensor(ids, dtype=torch.int32)
        ks.append(kp[ids].reshape(nb * page, hkv, d)[:n])
        vs.append(vp[ids].reshape(nb * page, hkv, d)[:n])
    q = torch.randn((sum(lens_q), hq, d), device="cuda:0", dtype=torch.float16)
    F = P.flash_attn
    got = F.flash_attn_varlen_paged_windowed(q, kp, vp, cu_q, cu_k, table.to("cuda:0"), None, max(lens_q), max(lens_k), d ** -0.5, 64, 0, page)
    want = F.flash_attn_varlen_windowed(q, torch.cat(ks), torch.cat(vs), cu_q, cu_k, max(lens_q), max(lens_k), d ** -0.5, 64, 0)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    with pytest.raises(ValueError, match="needs 9 blocks"):
        F.flash_attn_varlen_paged_windowed(q, kp, vp, cu_q, cu_k, table[:, :8].to("cuda:0"), None, 40, 130, 0.1, None, 0, page)
    with pytest.raises(ValueError, match="page_block_size"):
        F.flash_attn_varlen_paged_windowed(q, kp, vp, cu_q, cu_k, table.to("cuda:0"), None, 40, 130, 0.1, None, 0, 32)


def test_fp8_helper_close_to_bf16_attention(P):
    torch.manual_seed(6)
    q = torch.randn((1, 64, 8, 128), device="cuda:0", dtype=torch.bfloat16)
    k = torch.randn((1, 256, 2, 128), device="cuda:0", dtype=torch.bfloat16)
    v = torch.randn((1, 256, 2, 128), device="cuda:0", dtype=torch.bfloat16)
    F = P.flash_attn
    cfg = P.FlashAttnConfig(128 ** -0.5).causal()
    a, b8 = F.flash_attn_with_config(q, k, v, cfg), F.flash_attn_fp8(q, k, v, cfg)
    assert (a.float() - b8.float()).abs().max() < 0.08  # E4M3 rounding of K and V: 2^-4 relative per element


def test_prefill_at_full_size_matches_sampled_rows(P, oracle):
    """The prefill chunk of the third benchmark configuration at a quarter of its batch: rows sampled
    over the sequence are compared with the oracle run on exactly those query rows."""
    b, s, hq, hkv, d = 1, 4096, 32, 8, 128
    torch.manual_seed(7)
    q = torch.randn((b, s, hq, d), device="cuda:0", dtype=torch.bfloat16)
    k = torch.randn((b, s, hkv, d), device="cuda:0", dtype=torch.bfloat16)
    v = torch.randn((b, s, hkv, d), device="cuda:0", dtype=torch.bfloat16)
    out = P.flash_attn.flash_attn(q, k, v, d ** -0.5, True)
    torch.cuda.synchronize()
    kn, vn = k.float().cpu().numpy(), v.float().cpu().numpy()
    for i in (0, 1, 63, 64, 1000, 2047, 4095):
        # query row i sees keys 0..=i: one query over lk = i + 1 keys, causal
        want = oracle.reference_attention(q[:, i:i + 1].float().cpu().numpy(), kn[:, : i + 1], vn[:, : i + 1], d ** -0.5, wr=0)
        assert_close(out[:, i:i + 1].float().cpu().numpy(), want, what=f"row {i}", out="bf16")


@pytest.mark.parametrize("rotation", ["none", "hadamard"])
def test_prefill_append_gives_both_reference_results(P, oracle, rotation):
    b, s, hq, hkv, d = 2, 200, 8, 2, 128
    q = oracle.round_to(oracle.normal(11, b * s * hq * d).reshape(b, s, hq, d), "bf16")
    k = oracle.round_to(oracle.normal(12, b * s * hkv * d).reshape(b, s, hkv, d), "bf16")
    v = oracle.round_to(oracle.normal(13, b * s * hkv * d).reshape(b, s, hkv, d), "bf16")
    nv = fmt(P, 3)
    kq, vq = P.TurboQuantizer(nv, d, rotation, 42), P.TurboQuantizer(nv, d, rotation, 44)
    cap, pos = 256, 16
    kc = torch.zeros((b, hkv, cap, kq.row_words()), dtype=torch.int32, device="cuda:0")
    vc = torch.zeros_like(kc)
    out = P.flash_attn.prefill_append(to_dev(q, "bf16"), to_dev(k, "bf16"), to_dev(v, "bf16"), P.FlashAttnConfig(d ** -0.5).causal(),
                                      kc, vc, kq, vq, pos)
    torch.cuda.synchronize()
    want = oracle.reference_attention(q, k, v, d ** -0.5, wr=0)
    assert_close(out.float().cpu().numpy(), want, what="prefill output", out="bf16")
    # cache rows: bit-exact with the reference's quantizer on the same (rotated) rows
    # (with the Hadamard rotation: on the rows the device butterflies give, which agree with the
    # reference's matmul to rounding; tests/test_gpu_quant.py checks that stage by itself)
    for t, cache, qz in ((k, kc, kq), (v, vc, vq)):
        rows = t.transpose(0, 2, 1, 3).reshape(-1, d)
        if rotation == "hadamard":
            rows = qz.rotate(to_dev(rows, "bf16")).cpu().numpy()
        want_rows = oracle.quantize_rows(rows, 3).reshape(b, hkv, s, -1)
        got = words(cache)
        assert np.array_equal(got[:, :, pos:pos + s], want_rows)
        assert not got[:, :, :pos].any() and not got[:, :, pos + s:].any()


def test_prefill_append_from_two_host_threads(P, oracle):
    """b200_fa_prefill_append is re-entrant: two host threads, each on its own stream and its own caches, call it side
    by side many times; every call's output and cache rows are those of the same call made alone."""
    import threading
    b, s, hq, hkv, d = 1, 1024, 8, 2, 128
    nv = fmt(P, 3)
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    work = []
    for t in range(2):
        g = torch.Generator(device="cuda:0").manual_seed(50 + t)
        q = torch.randn((b, s, hq, d), generator=g, device="cuda:0", dtype=torch.bfloat16)
        k = torch.randn((b, s, hkv, d), generator=g, device="cuda:0", dtype=torch.bfloat16)
        v = torch.randn((b, s, hkv, d), generator=g, device="cuda:0", dtype=torch.bfloat16)
        kq, vq = P.TurboQuantizer(nv, d, "none", 42), P.TurboQuantizer(nv, d, "none", 44)
        kc = torch.zeros((b, hkv, s, kq.row_words()), dtype=torch.int32, device="cuda:0")
        vc = torch.zeros_like(kc)
        want = P.flash_attn.prefill_append(q, k, v, cfg, kc, vc, kq, vq, 0).clone()
        torch.cuda.synchronize()
        work.append(dict(q=q, k=k, v=v, kq=kq, vq=vq, kc=kc, vc=vc, want=want, want_k=kc.clone(), want_v=vc.clone(),
                         stream=torch.cuda.Stream("cuda:0"), bad=[]))
    torch.cuda.synchronize()
    start = threading.Barrier(2)

    def run(w):
        with torch.cuda.stream(w["stream"]):
            start.wait()
            for it in range(40):
                w["kc"].zero_()
                w["vc"].zero_()
                out = P.flash_attn.prefill_append(w["q"], w["k"], w["v"], cfg, w["kc"], w["vc"], w["kq"], w["vq"], 0)
                w["stream"].synchronize()
                if not (torch.equal(out, w["want"]) and torch.equal(w["kc"], w["want_k"]) and torch.equal(w["vc"], w["want_v"])):
                    w["bad"].append(it)

    threads = [threading.Thread(target=run, args=(w,)) for w in work]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not work[0]["bad"] and not work[1]["bad"], (work[0]["bad"], work[1]["bad"])
    assert P._abi.lib().b200_device_wait_status() == 0


def test_argument_errors(P):
    A = P._abi
    F = P.flash_attn
    q = torch.zeros((1, 4, 6, 128), device="cuda:0", dtype=torch.float16)
    k = torch.zeros((1, 4, 4, 128), device="cuda:0", dtype=torch.float16)
    with pytest.raises(ValueError, match="not a multiple"):
        F.flash_attn(q, k, k, 1.0, False)
    for d_bad in (100, 264):  # not a multiple of 8; above 256
        qb = torch.zeros((1, 4, 4, d_bad), device="cuda:0", dtype=torch.float16)
        with pytest.raises(A.B200Error) as e:
            F.flash_attn(qb, qb, qb, 1.0, False)
        assert e.value.code == A.ERR_UNSUPPORTED_SHAPE
    with pytest.raises(A.B200Error, match="must match q"):
        F.flash_attn(q[:, :, :4], k.to(torch.bfloat16), k.to(torch.bfloat16), 1.0, False)
    with pytest.raises(RuntimeError, match="no CPU path"):
        F.flash_attn(q.cpu(), k.cpu(), k.cpu(), 1.0, False)


def test_no_device_wait_ran_out(P):
    """Collected after the attention tests of this file: the bounded waits of the tcgen05 prefill tiles all completed."""
    assert P._abi.lib().b200_device_wait_status() == 0
