"""GPU parity of the attention over packed rows through the C ABI: against the outputs of the
reference's tq_attn kernels (golden fixtures), against the CPU oracle on seeded inputs, and through
size-independent properties at the sizes of the benchmark configurations."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest
import torch

from gpu_util import assert_close, fmt, pkg, rows_dev, to_dev, words

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
spec = importlib.util.spec_from_file_location("make_golden", ROOT / "tests" / "golden" / "make_golden.py")
MG = importlib.util.module_from_spec(spec)
spec.loader.exec_module(MG)


@pytest.fixture(scope="module")
def P():
    return pkg()


def run_packed(P, q, kd, vd, kv_len, kf, vf, scale, qdt="f32", rotation="none", seed=42, **cfg):
    d = q.shape[-1]
    kq = P.TurboQuantizer(fmt(P, *kf), d, rotation, seed)
    vq = P.TurboQuantizer(fmt(P, *vf), d, rotation, seed + 2)
    c = P.FlashAttnConfig(scale)
    c.window_size_left = None if cfg.get("wl", -1) < 0 else cfg["wl"]
    c.window_size_right = None if cfg.get("wr", -1) < 0 else cfg["wr"]
    c.softcap = cfg.get("softcap") or None
    c.splits = cfg.get("splits", 0)
    if cfg.get("alibi") is not None:
        c.alibi_slopes = to_dev(cfg["alibi"])
    kl = kv_len if isinstance(kv_len, int) else torch.from_numpy(np.asarray(kv_len, np.int32)).to("cuda:0")
    out = P.attention_packed(to_dev(q, qdt), rows_dev(kd), rows_dev(vd),
                             kl, kq, vq, c)
    torch.cuda.synchronize()
    return out.float().cpu().numpy()


SUPPORTED = list(MG.ATTN_CASES)  # codebook rows with 1-3 bit codes run on the general kernel


@pytest.mark.parametrize("case", SUPPORTED, ids=lambda c: c[0])
def test_against_reference_kernel_outputs(P, golden, case):
    name, kf, vf, b, lq, lk, hq, hkv, d, splits, group, wl, wr, softcap, _, _ = case
    q, kd, vd, tab, alibi = MG.attn_inputs(case)
    for s in (0, 1, splits):
        got = run_packed(P, q, kd, vd, lk, kf, vf, 1.0 / np.sqrt(d), wl=wl, wr=wr, softcap=softcap, alibi=alibi, splits=s)
        assert_close(got, golden["tq_attn"][name], what=f"{name} splits={s}")


def test_unsupported_formats_are_reported(P):
    A = P._abi
    d = 512  # above both kernels
    kq = P.TurboQuantizer(fmt(P, 0, 3), d, "none", 1)
    rows = torch.zeros((1, 1, 8, kq.row_words()), dtype=torch.int32, device="cuda:0")
    with pytest.raises(A.B200Error) as e:
        P.attention_packed(torch.zeros((1, 2, 1, d), device="cuda:0"), rows, rows, 8, kq, kq, P.FlashAttnConfig(1.0))
    assert e.value.code == A.ERR_UNSUPPORTED_SHAPE


GENERAL_CASES = [
    # name, key format, value format, b, lq, lk, hq, hkv, d, wl, wr, softcap, rotation
    ("turbo2_turbo3_ragged", (0, 2), (0, 3), 3, 1, 300, 8, 2, 128, -1, 0, 0.0, "none"),
    ("turbo3_hadamard_gqa", (0, 3), (0, 3), 2, 2, 150, 8, 2, 128, -1, 0, 0.0, "hadamard"),
    ("turbo1_turbo4_d64", (0, 1), (0, 4), 1, 3, 90, 2, 1, 64, 20, 0, 0.0, "none"),
    ("mxfp4_d96", (2, 4), (2, 4), 2, 1, 200, 4, 2, 96, -1, 0, 15.0, "none"),
    ("fp8_nvfp4_d32", (5, 4), (3, 4), 1, 2, 77, 2, 2, 32, -1, -1, 0.0, "none"),
    # few output rows over many keys: the call is split along the keys and a second kernel merges the partial rows
    ("split_turbo2_hadamard", (0, 2), (0, 2), 2, 1, 2600, 4, 2, 128, -1, 0, 0.0, "hadamard"),
    ("split_mxfp8_d96_window", (4, 4), (4, 4), 3, 2, 1500, 2, 1, 96, 700, 0, 0.0, "none"),
    ("split_turbo3_softcap", (0, 3), (0, 1), 1, 1, 5000, 8, 8, 64, -1, 0, 10.0, "none"),
]


@pytest.mark.parametrize("case", GENERAL_CASES, ids=lambda c: c[0])
def test_general_kernel_against_oracle(P, oracle, case):
    """Formats and head dims outside the tensor-core kernel: 1-3 bit codebook rows, head dims 32 and 96."""
    name, kf, vf, b, lq, lk, hq, hkv, d, wl, wr, softcap, rotation = case
    seed = 300 + sum(ord(ch) for ch in name)
    kx = oracle.normal(seed, b * hkv * lk * d).reshape(-1, d)
    vx = oracle.normal(seed + 1, b * hkv * lk * d).reshape(-1, d)
    q = oracle.normal(seed + 2, b * hq * lq * d).reshape(b, hq, lq, d)
    kq = P.TurboQuantizer(fmt(P, *kf), d, rotation, 42)
    vq = P.TurboQuantizer(fmt(P, *vf), d, rotation, 44)
    kd = kq.quantize_rows(to_dev(kx)).view(b, hkv, lk, -1)
    vd = vq.quantize_rows(to_dev(vx)).view(b, hkv, lk, -1)
    lens = np.array([lk, max(1, lk // 3), lk - 1][:b], np.int32)
    c = P.FlashAttnConfig(d ** -0.5)
    c.window_size_left = None if wl < 0 else wl
    c.window_size_right = None if wr < 0 else wr
    c.softcap = softcap or None
    got = P.attention_packed(to_dev(q), kd, vd, torch.from_numpy(lens).to("cuda:0"), kq, vq, c).cpu().numpy()
    # the oracle attends in the rotated space over the same packed rows, then rotates back
    tab = np.zeros(64, np.float32)
    tab[:32] = MG.tab_for(kf[0], kf[1], d)
    tab[32:] = MG.tab_for(vf[0], vf[1], d)
    qr = q
    if rotation == "hadamard":
        qr = oracle.rotate_rows(q.reshape(-1, d), oracle.rotation_matrix(d, 1, 42)).reshape(q.shape)
    want = oracle.tq_attention(qr, words(kd), words(vd), lk, kf, vf, d ** -0.5, tab, kv_len=lens, wl=wl, wr=wr, softcap=softcap)
    if rotation == "hadamard":
        want = oracle.rotate_rows(want.reshape(-1, d), oracle.rotation_matrix(d, 1, 44), transpose=True).reshape(want.shape)
    assert_close(got, want, what=name)


def make_rows(oracle, seed, b, hkv, lk, d, kf, vf, outliers=False, cap=None):
    n = b * hkv * lk
    kx = oracle.normal(seed, n * d, 1.0).reshape(b, hkv, lk, d)
    vx = oracle.normal(seed + 1, n * d, 1.0).reshape(b, hkv, lk, d)
    if outliers:  # 1% of the (kv head, channel) pairs scaled by 8
        rng = np.random.default_rng(seed)
        for idx in rng.choice(hkv * d, size=max(1, hkv * d // 100), replace=False):
            kx[:, idx // d, :, idx % d] *= 8
            vx[:, idx // d, :, idx % d] *= 8
    tab = np.zeros(64, np.float32)
    tab[:32] = MG.tab_for(kf[0], kf[1], d)
    tab[32:] = MG.tab_for(vf[0], vf[1], d)
    kd = oracle.quantize_rows(kx.reshape(-1, d), kf[0], kf[1], tab[:32]).reshape(b, hkv, lk, -1)
    vd = oracle.quantize_rows(vx.reshape(-1, d), vf[0], vf[1], tab[32:]).reshape(b, hkv, lk, -1)
    if cap and cap > lk:
        pad = lambda a: np.concatenate([a, np.full((b, hkv, cap - lk, a.shape[-1]), 0xDEADBEEF, np.uint32)], axis=2)
        kd, vd = pad(kd), pad(vd)
    return kd, vd, tab


FORMATS = [(5, 4), (4, 4), (2, 4), (3, 4), (0, 4)]


@pytest.mark.parametrize("kf", FORMATS, ids=lambda f: f"k{f[0]}")
@pytest.mark.parametrize("vf", FORMATS, ids=lambda f: f"v{f[0]}")
def test_all_format_pairs_d128(P, oracle, kf, vf):
    b, hq, hkv, d, lk = 2, 8, 2, 128, 777
    kd, vd, tab = make_rows(oracle, 50 + 7 * kf[0] + vf[0], b, hkv, lk, d, kf, vf, outliers=True)
    q = oracle.normal(77, b * hq * d).reshape(b, hq, 1, d)
    want = oracle.tq_attention(oracle.round_to(q, "bf16"), kd, vd, lk, kf, vf, 0.0884, tab, wr=0)
    got = run_packed(P, q, kd, vd, lk, kf, vf, 0.0884, qdt="bf16", wr=0)
    assert_close(got, want, what=f"k{kf} v{vf}", out="bf16")


@pytest.mark.parametrize("d", [64, 256])
@pytest.mark.parametrize("f", FORMATS, ids=lambda f: f"m{f[0]}")
def test_other_head_dims(P, oracle, d, f):
    b, hq, hkv, lk = 1, 4, 2, 300
    kd, vd, tab = make_rows(oracle, 300 + d + f[0], b, hkv, lk, d, f, f)
    q = oracle.normal(78, b * hq * 2 * d).reshape(b, hq, 2, d)
    want = oracle.tq_attention(oracle.round_to(q, "f16"), kd, vd, lk, f, f, d ** -0.5, tab, wr=0)
    got = run_packed(P, q, kd, vd, lk, f, f, d ** -0.5, qdt="f16", wr=0)
    assert_close(got, want, what=f"d{d} m{f}", out="f16")


@pytest.mark.parametrize("lk", [1, 2, 15, 16, 17, 31, 32, 33, 127, 128, 129, 255, 257, 511, 640, 1025])
def test_every_tail_length(P, oracle, lk):
    b, hq, hkv, d = 1, 8, 2, 128
    kd, vd, tab = make_rows(oracle, 1000 + lk, b, hkv, lk, d, (2, 4), (2, 4), cap=lk + 3)
    q = oracle.normal(79, b * hq * d).reshape(b, hq, 1, d)
    want = oracle.tq_attention(q, kd, vd, lk, (2, 4), (2, 4), 0.0884, tab, wr=0)
    for splits in (0, 1, 3):
        got = run_packed(P, q, kd, vd, lk, (2, 4), (2, 4), 0.0884, wr=0, splits=splits)
        assert_close(got, want, what=f"lk{lk} splits{splits}")


def test_ragged_batch_is_per_sequence_attention(P, oracle):
    """One launch over a ragged batch == the reference semantics applied per sequence."""
    b, hq, hkv, d, cap = 6, 32, 8, 128, 1500
    lens = np.array([512, 1500, 1, 777, 1024, 130], np.int32)
    kd, vd, tab = make_rows(oracle, 2002, b, hkv, cap, d, (2, 4), (2, 4), outliers=True)
    q = oracle.normal(80, b * hq * d).reshape(b, hq, 1, d)
    got = run_packed(P, q, kd, vd, lens, (2, 4), (2, 4), 0.0884, qdt="bf16", wr=0)
    want = oracle.tq_attention(oracle.round_to(q, "bf16"), kd, vd, cap, (2, 4), (2, 4), 0.0884, tab, kv_len=lens, wr=0)
    assert_close(got, want, what="ragged", out="bf16")
    for bi in (0, 2, 5):  # and each sequence alone gives the same bits as inside the batch
        one = run_packed(P, q[bi:bi + 1], kd[bi:bi + 1], vd[bi:bi + 1], int(lens[bi]), (2, 4), (2, 4), 0.0884, qdt="bf16", wr=0)
        assert_close(one, got[bi:bi + 1], atol=1e-2, rtol=8e-3, what=f"sequence {bi}")  # one bf16 ulp


@pytest.mark.parametrize("d,qdt", [(64, "f16"), (128, "bf16"), (128, "f32"), (256, "bf16")])
def test_many_short_columns_take_the_row_per_warp_combine(P, oracle, d, qdt):
    """More columns than an eighth of the decode grid's warps: the combine runs one warp per output row (every other
    case in this file has few columns and takes the block per row). Ragged lengths with an empty sequence."""
    b, hq, hkv = 96, 8, 4
    rng = np.random.default_rng(d)
    lens = rng.integers(1, 200, size=b).astype(np.int32)
    lens[5], lens[17] = 0, 199
    lk = int(lens.max())
    kd, vd, tab = make_rows(oracle, 7000 + d, b, hkv, lk, d, (2, 4), (5, 4), cap=lk + 2)
    q = oracle.normal(81, b * hq * d).reshape(b, hq, 1, d)
    want = oracle.tq_attention(oracle.round_to(q, qdt), kd, vd, lk, (2, 4), (5, 4), d ** -0.5, tab, kv_len=lens, wr=0)
    got = run_packed(P, q, kd, vd, lens, (2, 4), (5, 4), d ** -0.5, qdt=qdt, wr=0)
    assert np.all(got[5] == 0)
    assert_close(got, want, what=f"many columns d{d} {qdt}", out=qdt)


def test_many_short_columns_with_a_rotated_cache(P, oracle):
    """The row-per-warp combine rotates the merged rows back (Hadamard cache, 192 columns of 100 keys)."""
    b, hq, hkv, d, lk = 48, 8, 4, 128, 100
    kx = oracle.normal(15, b * hkv * lk * d).reshape(b, hkv, lk, d)
    vx = oracle.normal(16, b * hkv * lk * d).reshape(b, hkv, lk, d)
    q = oracle.normal(17, b * hq * d).reshape(b, hq, 1, d)
    f = (0, 4)
    cache = P.TurboKvCache(fmt(P, *f), fmt(P, *f), d, "hadamard", 42, lk)
    cache.append(to_dev(kx, "bf16"), to_dev(vx, "bf16"))
    got = cache.attention(to_dev(q, "bf16"), P.FlashAttnConfig(0.0884).causal()).float().cpu().numpy()
    pk, pv = oracle.rotation_matrix(d, 1, 42), oracle.rotation_matrix(d, 1, 44)
    tab = MG.tab_for(f[0], f[1], d)
    kd = oracle.quantize_rows(oracle.rotate_rows(oracle.round_to(kx, "bf16").reshape(-1, d), pk), f[0], f[1], tab).reshape(b, hkv, lk, -1)
    vd = oracle.quantize_rows(oracle.rotate_rows(oracle.round_to(vx, "bf16").reshape(-1, d), pv), f[0], f[1], tab).reshape(b, hkv, lk, -1)
    qr = oracle.rotate_rows(oracle.round_to(q, "bf16").reshape(-1, d), pk).reshape(q.shape)
    o = oracle.tq_attention(qr, kd, vd, lk, f, f, 0.0884, np.concatenate([tab, tab]), wr=0)
    want = oracle.rotate_rows(o.reshape(-1, d), pv, transpose=True).reshape(o.shape)
    assert_close(got, want, what="hadamard, many columns", out="bf16")


def test_launch_behind_a_running_kernel_gives_the_same_rows(P, oracle):
    """B200_TQ_AFTER_PREV: the attention takes its place while the stream's previous kernel still runs and waits for
    it before reading the query and the rows. Here that kernel is the append that writes the very rows (and a copy
    that writes the query): the outputs must be those of the plain launch, call after call."""
    b, hq, hkv, d, lk = 8, 16, 4, 128, 2000
    f = fmt(P, 2, 4)
    kq, vq = P.TurboQuantizer(f, d, "none", 42), P.TurboQuantizer(f, d, "none", 44)
    g = torch.Generator(device="cuda:0").manual_seed(5)
    kx = torch.randn((b, hkv, lk, d), generator=g, device="cuda:0", dtype=torch.bfloat16)
    vx = torch.randn((b, hkv, lk, d), generator=g, device="cuda:0", dtype=torch.bfloat16)
    kc = torch.zeros((b, hkv, lk, kq.row_words()), dtype=torch.int32, device="cuda:0")
    vc = torch.zeros_like(kc)
    lens = torch.tensor([2000, 1, 777, 1500, 64, 1999, 33, 1024], dtype=torch.int32, device="cuda:0")
    q_src = [torch.randn((b, hq, 1, d), generator=g, device="cuda:0", dtype=torch.bfloat16) for _ in range(3)]
    q = torch.empty_like(q_src[0])
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    plain = P.PackedAttention(q, kc, vc, lens, kq, vq, cfg)
    behind = P.PackedAttention(q, kc, vc, lens, kq, vq, cfg, out=torch.empty_like(plain.out), after_prev=True)
    from candle_rocm_vulkan_b200.turbo_quant import _kv_append
    for it in range(3):
        scale = float(it + 1)
        kc.zero_(); vc.zero_()
        q.copy_(q_src[it])
        _kv_append(kx * scale, vx, kc, vc, kq, vq, 0)
        plain.run()
        torch.cuda.synchronize()
        want = plain.out.clone()
        kc.zero_(); vc.zero_(); q.zero_()
        torch.cuda.synchronize()
        q.copy_(q_src[it])                          # the kernels right before the attention write what it reads
        _kv_append(kx * scale, vx, kc, vc, kq, vq, 0)
        behind.run()
        behind.run()                                # and once more behind its own combine
        torch.cuda.synchronize()
        assert torch.equal(behind.out, want), f"call {it}"
    assert P._abi.lib().b200_device_wait_status() == 0


@pytest.mark.parametrize("f", [(2, 4), (0, 4)])
def test_calls_that_overlap_their_predecessors_give_the_same_rows(P, oracle, f):
    """B200_TQ_AFTER_PREV | B200_TQ_INPUTS_FINAL | B200_TQ_OUTPUTS_FREE: calls over caches nobody writes, each with an
    output and a workspace of its own, neither read nor stored behind the call before. A chain of them, eager and as a
    CUDA graph, gives the rows of the plain calls (ragged lengths; such calls merge their columns inside the grid where a
    plain call of this shape runs a combine grid, so the sums differ in their last bits)."""
    b, hq, hkv, d, cap = 16, 16, 4, 128, 3000
    fm = fmt(P, *f)
    kq, vq = P.TurboQuantizer(fm, d, "none", 42), P.TurboQuantizer(fm, d, "none", 44)
    g = torch.Generator(device="cuda:0").manual_seed(6)
    lens = torch.randint(1, cap, (b,), generator=g, device="cuda:0", dtype=torch.int32)
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    n = 4
    caches, qs = [], []
    for i in range(n):
        kx = torch.randn((b * hkv * cap, d), generator=g, device="cuda:0")
        vx = torch.randn((b * hkv * cap, d), generator=g, device="cuda:0")
        caches.append((kq.quantize_rows(kx).view(b, hkv, cap, -1), vq.quantize_rows(vx).view(b, hkv, cap, -1)))
        qs.append(torch.randn((b, hq, 1, d), generator=g, device="cuda:0", dtype=torch.bfloat16))
    plain = [P.PackedAttention(qs[i], caches[i][0], caches[i][1], lens, kq, vq, cfg) for i in range(n)]
    for c in plain:
        c.run()
    torch.cuda.synchronize()
    want = [c.out.clone() for c in plain]
    chain = [P.PackedAttention(qs[i], caches[i][0], caches[i][1], lens, kq, vq, cfg, after_prev=True, fresh_rows=0, outputs_free=True)
             for i in range(n)]
    for rounds in range(2):
        for c in chain:
            c.out.fill_(float("nan"))
        for c in chain:
            c.run()
        torch.cuda.synchronize()
        for i, c in enumerate(chain):
            torch.testing.assert_close(c.out.float(), want[i].float(), rtol=1.6e-2, atol=2e-3, msg=f"eager chain, round {rounds}, call {i}")
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        for c in chain:
            c.run()
    for c in chain:
        c.out.fill_(float("nan"))
    gr.replay()
    torch.cuda.synchronize()
    for i, c in enumerate(chain):
        torch.testing.assert_close(c.out.float(), want[i].float(), rtol=1.6e-2, atol=2e-3, msg=f"graph chain, call {i}")
    assert P._abi.lib().b200_device_wait_status() == 0


def test_overlapping_calls_with_one_length_and_several_query_tokens(P, oracle):
    """The same chain over caches of one length, TurboQuant-4 rows and two query tokens per sequence
    (a combine-free call whose columns are split over many workers), against the oracle and against the plain calls."""
    b, hq, hkv, d, lk, lq = 2, 8, 1, 128, 5000, 2
    f = (0, 4)
    kd, vd, tab = make_rows(oracle, 3500, b, hkv, lk, d, f, f)
    fm = fmt(P, *f)
    kq, vq = P.TurboQuantizer(fm, d, "none", 42), P.TurboQuantizer(fm, d, "none", 44)
    cfg = P.FlashAttnConfig(0.0884).causal()
    n = 3
    qs = [oracle.normal(86 + i, b * hq * lq * d).reshape(b, hq, lq, d) for i in range(n)]
    want = [oracle.tq_attention(q, kd, vd, lk, f, f, 0.0884, tab, wr=0) for q in qs]
    k_dev, v_dev = rows_dev(kd), rows_dev(vd)
    chain = [P.PackedAttention(to_dev(qs[i]), k_dev, v_dev, lk, kq, vq, cfg, after_prev=i > 0, fresh_rows=0 if i > 0 else None,
                               outputs_free=i > 0) for i in range(n)]
    for rounds in range(2):
        for c in chain:
            c.out.fill_(float("nan"))
        for c in chain:
            c.run()
        torch.cuda.synchronize()
        for i, c in enumerate(chain):
            assert_close(c.out.float().cpu().numpy(), want[i], what=f"round {rounds}, call {i}")
    assert P._abi.lib().b200_device_wait_status() == 0


def test_length_and_position_offsets(P, oracle):
    """kv_len_add / pos0 with device positions: a step that appends at lens + j and attends to lens + j + 1 keys gives
    the rows and outputs of the same step run with the lengths updated on the device."""
    from candle_rocm_vulkan_b200.turbo_quant import _kv_append
    b, hq, hkv, d, cap = 6, 8, 2, 128, 700
    f = fmt(P, 2, 4)
    kq, vq = P.TurboQuantizer(f, d, "none", 42), P.TurboQuantizer(f, d, "none", 44)
    g = torch.Generator(device="cuda:0").manual_seed(9)
    kx = torch.randn((b, hkv, cap, d), generator=g, device="cuda:0", dtype=torch.bfloat16)
    vx = torch.randn((b, hkv, cap, d), generator=g, device="cuda:0", dtype=torch.bfloat16)
    q = torch.randn((b, hq, 1, d), generator=g, device="cuda:0", dtype=torch.bfloat16)
    lens0 = torch.tensor([600, 0, 33, 257, 1, 512], dtype=torch.int32, device="cuda:0")
    cfg = P.FlashAttnConfig(d ** -0.5).causal()

    def fresh():
        kc = torch.zeros((b, hkv, cap, kq.row_words()), dtype=torch.int32, device="cuda:0")
        vc = torch.zeros_like(kc)
        _kv_append(kx, vx, kc, vc, kq, vq, 0)
        return kc, vc

    kn = torch.randn((3, b, hkv, 1, d), generator=g, device="cuda:0", dtype=torch.bfloat16)
    vn = torch.randn((3, b, hkv, 1, d), generator=g, device="cuda:0", dtype=torch.bfloat16)
    # lengths updated on the device before every step
    kc1, vc1 = fresh()
    lens = lens0.clone()
    want = []
    for j in range(3):
        _kv_append(kn[j], vn[j], kc1, vc1, kq, vq, lens)
        lens.add_(1)
        want.append(P.PackedAttention(q, kc1, vc1, lens, kq, vq, cfg).run().clone())
    # lengths left alone, offsets in the arguments
    kc2, vc2 = fresh()
    for j in range(3):
        _kv_append(kn[j], vn[j], kc2, vc2, kq, vq, lens0, pos_add=j)
        got = P.PackedAttention(q, kc2, vc2, lens0, kq, vq, cfg, kv_len_add=j + 1, after_prev=True).run()
        torch.cuda.synchronize()
        assert torch.equal(got, want[j]), f"step {j}"
    assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)


def test_rows_copied_while_the_append_of_the_step_still_runs(P, oracle):
    """B200_TQ_INPUTS_FINAL with fresh_rows = 1: behind the append of a decode step, the attention may copy every row but
    the sequence's last one before that kernel has finished. Poison sits where the new rows go until the append writes
    them, so a tile copied too early would show in the outputs. Several steps in a row, ragged lengths among which a
    sequence of one key, one that ends exactly on a tile boundary and one that starts a tile."""
    from candle_rocm_vulkan_b200.turbo_quant import _kv_append
    b, hq, hkv, d, cap = 8, 16, 4, 128, 2100
    f = fmt(P, 2, 4)
    kq, vq = P.TurboQuantizer(f, d, "none", 42), P.TurboQuantizer(f, d, "none", 44)
    g = torch.Generator(device="cuda:0").manual_seed(11)
    kx = torch.randn((b, hkv, cap, d), generator=g, device="cuda:0", dtype=torch.bfloat16)
    vx = torch.randn((b, hkv, cap, d), generator=g, device="cuda:0", dtype=torch.bfloat16)
    lens0 = torch.tensor([2000, 0, 31, 32, 63, 1999, 640, 1024], dtype=torch.int32, device="cuda:0")
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    steps = 4
    kn = torch.randn((steps, b, hkv, 1, d), generator=g, device="cuda:0", dtype=torch.bfloat16)
    vn = torch.randn((steps, b, hkv, 1, d), generator=g, device="cuda:0", dtype=torch.bfloat16)
    qs = torch.randn((steps, b, hq, 1, d), generator=g, device="cuda:0", dtype=torch.bfloat16)

    def fresh():
        kc = torch.zeros((b, hkv, cap, kq.row_words()), dtype=torch.int32, device="cuda:0")
        vc = torch.zeros_like(kc)
        _kv_append(kx, vx, kc, vc, kq, vq, 0)
        for bi in range(b):  # rows past the lengths: NaN scales until a step writes them
            kc[bi, :, int(lens0[bi]):] = 0x7fc00000
            vc[bi, :, int(lens0[bi]):] = 0x7fc00000
        return kc, vc

    kc1, vc1 = fresh()
    want = []
    for j in range(steps):
        _kv_append(kn[j], vn[j], kc1, vc1, kq, vq, lens0, pos_add=j)
        want.append(P.PackedAttention(qs[j], kc1, vc1, lens0, kq, vq, cfg, kv_len_add=j + 1).run().clone())
    kc2, vc2 = fresh()
    torch.cuda.synchronize()
    for j in range(steps):
        _kv_append(kn[j], vn[j], kc2, vc2, kq, vq, lens0, pos_add=j)
        got = P.PackedAttention(qs[j], kc2, vc2, lens0, kq, vq, cfg, kv_len_add=j + 1, after_prev=True, fresh_rows=1).run()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all(), f"step {j}"
        assert torch.equal(got, want[j]), f"step {j}"
    # the whole loop without a host synchronization, the append of every step but the first launched behind the
    # previous step's attention as well (B200_KV_AFTER_PREV): steps chase one another on the device, eagerly and
    # replayed from a CUDA graph; the outputs are those of the plain loop, bit for bit
    def chained(kc, vc, outs):
        for j in range(steps):
            _kv_append(kn[j], vn[j], kc, vc, kq, vq, lens0, pos_add=j, after_prev=(j > 0))
            P.PackedAttention(qs[j], kc, vc, lens0, kq, vq, cfg, out=outs[j], kv_len_add=j + 1, after_prev=True, fresh_rows=1).run()

    kc3, vc3 = fresh()
    outs = [torch.empty_like(want[0]) for _ in range(steps)]
    chained(kc3, vc3, outs)
    torch.cuda.synchronize()
    for j in range(steps):
        assert torch.equal(outs[j], want[j]), f"chained step {j}"
    assert torch.equal(kc3, kc1) and torch.equal(vc3, vc1)
    kc4, vc4 = fresh()
    outs4 = [torch.zeros_like(want[0]) for _ in range(steps)]
    chained(kc4, vc4, outs4)  # warm-up: what a first call allocates is allocated outside the capture
    torch.cuda.synchronize()
    k0, v0 = fresh()
    kc4.copy_(k0)
    vc4.copy_(v0)
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        chained(kc4, vc4, outs4)
    for o in outs4:
        o.zero_()
    gr.replay()
    torch.cuda.synchronize()
    for j in range(steps):
        assert torch.equal(outs4[j], want[j]), f"graph step {j}"
    # and layer after layer over caches nobody writes (fresh_rows = 0), each call behind the one before
    out = [torch.empty_like(want[0]) for _ in range(3)]
    calls = [P.PackedAttention(qs[i], kc2, vc2, lens0, kq, vq, cfg, out=out[i], kv_len_add=steps, after_prev=True, fresh_rows=0) for i in range(3)]
    ref = [P.PackedAttention(qs[i], kc2, vc2, lens0, kq, vq, cfg, kv_len_add=steps).run().clone() for i in range(3)]
    torch.cuda.synchronize()
    for _ in range(3):
        for c in calls:
            c.run()
    torch.cuda.synchronize()
    for i in range(3):
        assert torch.equal(out[i], ref[i]), f"layer {i}"
    assert P._abi.lib().b200_device_wait_status() == 0


@pytest.mark.parametrize("b", [3, 120])  # few columns: the combine grid merges; many: the decode grid itself
def test_far_more_workers_than_tiles(P, oracle, b):
    """A capacity of thousands of rows sizes the grid, but the sequences hold a handful of keys: most workers own no
    tile, and the segments of a column must still be the consecutive workers that own one (a merge that counted the idle
    workers in between would read partial results that nobody wrote). Poisoned workspace, ragged lengths."""
    hq, hkv, d, cap = 16, 2, 128, 6000
    lens = np.array([70, 1, 33], np.int32) if b == 3 else np.random.default_rng(b).integers(0, 71, size=b).astype(np.int32)
    kd, vd, tab = make_rows(oracle, 911, b, hkv, 80, d, (2, 4), (2, 4), cap=cap)
    q = oracle.normal(912, b * hq * d).reshape(b, hq, 1, d)
    kq, vq = P.TurboQuantizer(fmt(P, 2, 4), d, "none", 42), P.TurboQuantizer(fmt(P, 2, 4), d, "none", 44)
    from candle_rocm_vulkan_b200 import turbo_quant as TQ
    for key, ws in list(TQ._WORKSPACES.items()):
        ws.view(torch.int32).fill_(0x7fc00000)  # NaN in every partial result left over from earlier calls
    torch.cuda.synchronize()
    want = oracle.tq_attention(oracle.round_to(q, "bf16"), kd, vd, cap, (2, 4), (2, 4), d ** -0.5, tab, kv_len=lens, wr=0)
    for splits in (0, 1, 7):
        cfg = P.FlashAttnConfig(d ** -0.5).causal()
        cfg.splits = splits
        call = P.PackedAttention(to_dev(q, "bf16"), rows_dev(kd), rows_dev(vd), torch.from_numpy(lens).to("cuda:0"), kq, vq, cfg)
        call.workspace.view(torch.int32).fill_(0x7fc00000)
        got = call.run().float().cpu().numpy()
        assert_close(got, want, what=f"sparse work, splits={splits}", out="bf16")


@pytest.mark.parametrize("lq,wl,wr,softcap,use_alibi", [(3, -1, 0, 0.0, False), (4, 50, 0, 0.0, False), (2, -1, -1, 15.0, False),
                                                         (1, -1, 0, 0.0, True), (5, 20, 3, 30.0, True), (3, 0, 0, 0.0, False)])
def test_masks_softcap_alibi_multi_query(P, oracle, lq, wl, wr, softcap, use_alibi):
    b, hq, hkv, d, lk = 2, 8, 2, 128, 333
    kd, vd, tab = make_rows(oracle, 3000 + lq, b, hkv, lk, d, (5, 4), (3, 4))
    q = oracle.normal(81, b * hq * lq * d).reshape(b, hq, lq, d)
    alibi = (0.02 * (1 + np.arange(b * hq, dtype=np.float32))).reshape(b, hq) if use_alibi else None
    want = oracle.tq_attention(q, kd, vd, lk, (5, 4), (3, 4), 0.0884, tab, wl=wl, wr=wr, softcap=softcap, alibi=alibi)
    got = run_packed(P, q, kd, vd, lk, (5, 4), (3, 4), 0.0884, wl=wl, wr=wr, softcap=softcap, alibi=alibi)
    assert_close(got, want, what="masks")


@pytest.mark.parametrize("lq,wl,wr,softcap,use_alibi", [(1, -1, 0, 0.0, False), (2, 37, 0, 0.0, False), (1, -1, 0, 20.0, True), (4, 5, 2, 0.0, False)])
@pytest.mark.parametrize("lk", [333, 1000])
def test_masks_on_codebook_rows_in_the_cache_layout(P, oracle, lq, wl, wr, softcap, use_alibi, lk):
    """TurboQuant-4 keys and values packed back to back take the kernel of warp pairs, which deals the keys of a tile
    to its lanes in an order of its own: windows, tails, soft-capping and ALiBi must still see every key at its place."""
    b, hq, hkv, d = 3, 16, 2, 128
    f = (0, 4)
    kd, vd, tab = make_rows(oracle, 3400 + lq, b, hkv, lk, d, f, f)
    q = oracle.normal(85, b * hq * lq * d).reshape(b, hq, lq, d)
    alibi = (0.02 * (1 + np.arange(b * hq, dtype=np.float32))).reshape(b, hq) if use_alibi else None
    lens = np.array([lk, lk - 17, 40], np.int32)
    want = oracle.tq_attention(q, kd, vd, lk, f, f, 0.0884, tab, kv_len=lens, wl=wl, wr=wr, softcap=softcap, alibi=alibi)
    got = run_packed(P, q, kd, vd, lens, f, f, 0.0884, wl=wl, wr=wr, softcap=softcap, alibi=alibi)
    assert_close(got, want, what="masks on codebook rows")


def test_queries_longer_than_keys_give_zero_rows(P, oracle):
    b, hq, hkv, d, lk, lq = 1, 2, 1, 128, 3, 6
    kd, vd, tab = make_rows(oracle, 3100, b, hkv, lk, d, (4, 4), (4, 4))
    q = oracle.normal(82, b * hq * lq * d).reshape(b, hq, lq, d)
    want = oracle.tq_attention(q, kd, vd, lk, (4, 4), (4, 4), 0.0884, tab, wr=0)
    got = run_packed(P, q, kd, vd, lk, (4, 4), (4, 4), 0.0884, wr=0)
    assert np.all(got[:, :, :3] == 0) and np.all(want[:, :, :3] == 0)
    assert_close(got, want, what="lq > lk")


def test_unaligned_views_and_row_padding(P, oracle):
    """Rows that start at any word offset and rows padded to a common stride (the reference's tests
    use the larger of the K / V row sizes for both sides)."""
    b, hq, hkv, d, lk = 2, 4, 2, 128, 200
    kf, vf = (3, 4), (2, 4)
    kd, vd, tab = make_rows(oracle, 3200, b, hkv, lk, d, kf, vf)
    q = oracle.normal(83, b * hq * d).reshape(b, hq, 1, d)
    want = oracle.tq_attention(q, kd, vd, lk, kf, vf, 0.0884, tab, wr=0)
    kq = P.TurboQuantizer(fmt(P, *kf), d, "none", 1)
    vq = P.TurboQuantizer(fmt(P, *vf), d, "none", 3)
    for off in (0, 1, 2, 3):
        rw = 23  # padded row stride (words)
        kbuf = torch.full((off + b * hkv * lk * rw,), 0x7FC00000, dtype=torch.int32, device="cuda:0")
        vbuf = torch.full((off + b * hkv * lk * rw,), 0x7FC00000, dtype=torch.int32, device="cuda:0")
        kv = kbuf[off:].view(b, hkv, lk, rw)
        vv = vbuf[off:].view(b, hkv, lk, rw)
        kv[..., : kd.shape[-1]] = rows_dev(kd)
        vv[..., : vd.shape[-1]] = rows_dev(vd)
        got = P.attention_packed(to_dev(q), kv, vv, lk, kq, vq, P.FlashAttnConfig(0.0884).causal())
        assert_close(got.cpu().numpy(), want, what=f"offset {off}")


@pytest.mark.parametrize("f", [(0, 4), (3, 4), (5, 8)])
def test_native_rows_at_any_word_offset(P, oracle, f):
    """Rows packed back to back (the cache's own layout) whose first row sits at any word offset: rows of 72, 80 or
    136 bytes are read with 8- or 16-byte loads only where every row is aligned to that, so an odd offset must take
    the other instantiation and give the same rows."""
    b, hq, hkv, d, lk = 2, 8, 2, 128, 333
    kd, vd, tab = make_rows(oracle, 3300 + f[0], b, hkv, lk, d, f, f)
    q = oracle.normal(84, b * hq * d).reshape(b, hq, 1, d)
    want = oracle.tq_attention(q, kd, vd, lk, f, f, 0.0884, tab, wr=0)
    kq = P.TurboQuantizer(fmt(P, *f), d, "none", 1)
    vq = P.TurboQuantizer(fmt(P, *f), d, "none", 3)
    rw = kd.shape[-1]
    first = None
    for off in (0, 1, 2, 3, 4):
        kbuf = torch.full((off + b * hkv * lk * rw,), 0x7FC00000, dtype=torch.int32, device="cuda:0")
        vbuf = torch.full((off + b * hkv * lk * rw,), 0x7FC00000, dtype=torch.int32, device="cuda:0")
        kv = kbuf[off:].view(b, hkv, lk, rw)
        vv = vbuf[off:].view(b, hkv, lk, rw)
        kv.copy_(rows_dev(kd))
        vv.copy_(rows_dev(vd))
        got = P.attention_packed(to_dev(q), kv, vv, lk, kq, vq, P.FlashAttnConfig(0.0884).causal()).cpu().numpy()
        assert_close(got, want, what=f"format {f}, offset {off}")
        if first is None:
            first = got
        # codebook rows: the aligned instantiation deals a tile's keys to its lanes in another order (sums in another order)
        if f[0] != 0:
            assert np.array_equal(got, first), f"format {f}: offset {off} changes the bits"


def test_value_scales_of_any_magnitude(P, oracle):
    """The per-key value scale is folded into the exponent of the second product: rows whose scale
    is far outside the f16 range must not lose accuracy."""
    b, hq, hkv, d, lk = 1, 8, 1, 128, 96
    for mag in (1e-20, 3e-6, 1.0, 7e4, 1e18):
        kx = oracle.normal(1, lk * d).reshape(lk, d)
        vx = oracle.normal(2, lk * d).reshape(lk, d) * mag
        vx[::3] *= 1e-3
        for f in ((5, 4), (2, 4), (3, 4)):
            kd = oracle.quantize_rows(kx, f[0]).reshape(b, hkv, lk, -1)
            vd = oracle.quantize_rows(vx.astype(np.float32), f[0]).reshape(b, hkv, lk, -1)
            q = oracle.normal(84, hq * d).reshape(b, hq, 1, d)
            want = oracle.tq_attention(q, kd, vd, lk, f, f, 0.0884, wr=0)
            got = run_packed(P, q, kd, vd, lk, f, f, 0.0884, wr=0)
            assert_close(got / mag, want / mag, what=f"magnitude {mag} format {f}")


@pytest.mark.parametrize("f", [(0, 4), (3, 4), (5, 4)], ids=lambda f: f"m{f[0]}")
def test_hadamard_cache_end_to_end(P, oracle, f):
    """Rotated cache (the reference's default): append + attention through the cache object
    against the oracle run with the reference's matmul rotation."""
    b, hq, hkv, d, lk = 2, 16, 2, 128, 500
    kx = oracle.normal(5, b * hkv * lk * d).reshape(b, hkv, lk, d)
    vx = oracle.normal(6, b * hkv * lk * d).reshape(b, hkv, lk, d)
    q = oracle.normal(7, b * hq * d).reshape(b, hq, 1, d)
    cache = P.TurboKvCache(fmt(P, *f), fmt(P, *f), d, "hadamard", 42, lk)
    cache.append(to_dev(kx, "bf16"), to_dev(vx, "bf16"))
    got = cache.attention(to_dev(q, "bf16"), P.FlashAttnConfig(0.0884).causal()).float().cpu().numpy()
    pk, pv = oracle.rotation_matrix(d, 1, 42), oracle.rotation_matrix(d, 1, 44)
    tab = MG.tab_for(f[0], f[1], d)
    kd = oracle.quantize_rows(oracle.rotate_rows(oracle.round_to(kx, "bf16").reshape(-1, d), pk), f[0], f[1], tab).reshape(b, hkv, lk, -1)
    vd = oracle.quantize_rows(oracle.rotate_rows(oracle.round_to(vx, "bf16").reshape(-1, d), pv), f[0], f[1], tab).reshape(b, hkv, lk, -1)
    qr = oracle.rotate_rows(oracle.round_to(q, "bf16").reshape(-1, d), pk).reshape(q.shape)
    o = oracle.tq_attention(qr, kd, vd, lk, f, f, 0.0884, np.concatenate([tab, tab]), wr=0)
    want = oracle.rotate_rows(o.reshape(-1, d), pv, transpose=True).reshape(o.shape)
    assert_close(got, want, what=f"hadamard {f}", out="bf16")


@pytest.mark.parametrize("f,rot", [((3, 4), "hadamard"), ((4, 4), "none")])
def test_chunked_prefill_over_the_compressed_cache(P, oracle, f, rot):
    """A chunk of 160 query tokens (640 rows per kv head) over 900 cached keys: the cache serves it from its dequantized
    rows on the prefill tiles (the reference's keys_values + flash_attn_bhsd route, turbo_quant.rs:986-990). Against the
    fused kernel over the packed rows, which computes the same attention pack by pack; the two differ by the rounding
    of the dequantized rows and of the rotated queries to bf16."""
    b, hq, hkv, d, lk, lq = 1, 8, 2, 128, 900, 160
    g = torch.Generator(device="cuda:0").manual_seed(3)
    k = torch.randn((b, hkv, lk, d), generator=g, device="cuda:0").to(torch.bfloat16)
    v = torch.randn((b, hkv, lk, d), generator=g, device="cuda:0").to(torch.bfloat16)
    q = torch.randn((b, hq, lq, d), generator=g, device="cuda:0").to(torch.bfloat16)
    cache = P.TurboKvCache(fmt(P, *f), fmt(P, *f), d, rot, 42, lk)
    cache.append(k, v)
    c = P.FlashAttnConfig(d ** -0.5).causal()
    assert lq * (hq // hkv) >= cache.PREFILL_ROWS
    got = cache.attention(q, c).float().cpu().numpy()
    want = P.attention_packed(q, cache.k, cache.v, cache.seq_len(), cache.kq, cache.vq, c).float().cpu().numpy()
    assert_close(got, want, atol=3e-2, rtol=2e-2, what=f"chunked prefill {f} {rot}", out="bf16")
    # and a short chunk stays on the fused kernel: identical to the direct call
    assert torch.equal(cache.attention(q[:, :, -4:], c), P.attention_packed(q[:, :, -4:].contiguous(), cache.k, cache.v, lk, cache.kq, cache.vq, c))


@pytest.mark.parametrize("f,d", [((0, 4), 96), ((2, 4), 96), ((0, 3), 160)])
def test_dense_rotation_for_head_dims_that_are_not_powers_of_two(P, oracle, f, d):
    """RotationKind::Auto at a head dim that is not a power of two: the seeded dense rotation (turbo.rs:204-229). The
    rotated rows have the oracle's bits (sums in index order), so the packed rows are bit-exact; the attention through
    the cache object (rotate q, kernel, rotate back) against the oracle's matmul rotation."""
    b, hq, hkv, lk = 2, 4, 2, 300
    kx = oracle.normal(15, b * hkv * lk * d).reshape(b, hkv, lk, d)
    vx = oracle.normal(16, b * hkv * lk * d).reshape(b, hkv, lk, d)
    q = oracle.normal(17, b * hq * d).reshape(b, hq, 1, d)
    cache = P.TurboKvCache(fmt(P, *f), fmt(P, *f), d, "auto", 42, lk)
    assert cache.kq.rotation == "dense" and cache.vq.rotation == "dense"
    cache.append(to_dev(kx), to_dev(vx))
    pk, pv = oracle.rotation_matrix(d, 2, 42), oracle.rotation_matrix(d, 2, 44)
    tab = MG.tab_for(f[0], f[1], d)
    kd = oracle.quantize_rows(oracle.rotate_rows(kx.reshape(-1, d), pk), f[0], f[1], tab).reshape(b, hkv, lk, -1)
    vd = oracle.quantize_rows(oracle.rotate_rows(vx.reshape(-1, d), pv), f[0], f[1], tab).reshape(b, hkv, lk, -1)
    assert np.array_equal(words(cache.k[:, :, :lk]), kd) and np.array_equal(words(cache.v[:, :, :lk]), vd)
    got = cache.attention(to_dev(q), P.FlashAttnConfig(d ** -0.5).causal()).cpu().numpy()
    qr = oracle.rotate_rows(q.reshape(-1, d), pk).reshape(q.shape)
    o = oracle.tq_attention(qr, kd, vd, lk, f, f, d ** -0.5, np.concatenate([tab, tab]), wr=0)
    want = oracle.rotate_rows(o.reshape(-1, d), pv, transpose=True).reshape(o.shape)
    assert_close(got, want, what=f"dense rotation {f} d={d}")
    # dequantized keys come back in the original domain
    k_back, _ = cache.keys_values()
    assert_close(k_back.float().cpu().numpy(), oracle.rotate_rows(oracle.dequantize_rows(kd.reshape(-1, kd.shape[-1]), d, f[0], f[1], tab), pk, transpose=True).reshape(b, hkv, lk, d),
                 atol=1e-5, rtol=1e-5, what="keys_values")


def test_config1_fp8_single_decode(P, oracle):
    """B=1, Hq=32, Hkv=8, D=128, 2048 keys, f16, FP8 rows with one f32 scale per token and head."""
    b, hq, hkv, d, lk = 1, 32, 8, 128, 2048
    kx = oracle.normal(1002, b * hkv * lk * d).reshape(b, hkv, lk, d)
    vx = oracle.normal(1003, b * hkv * lk * d).reshape(b, hkv, lk, d)
    q = oracle.normal(1001, b * hq * d).reshape(b, hq, 1, d)
    cache = P.TurboKvCache(fmt(P, 5), fmt(P, 5), d, "none", 42, lk)
    cache.append(to_dev(kx, "f16"), to_dev(vx, "f16"))
    got = cache.attention(to_dev(q, "f16"), P.FlashAttnConfig(d ** -0.5).causal()).float().cpu().numpy()
    kd = oracle.quantize_rows(oracle.round_to(kx, "f16").reshape(-1, d), 5).reshape(b, hkv, lk, -1)
    vd = oracle.quantize_rows(oracle.round_to(vx, "f16").reshape(-1, d), 5).reshape(b, hkv, lk, -1)
    assert np.array_equal(words(cache.k), kd) and np.array_equal(words(cache.v), vd)
    want = oracle.tq_attention(oracle.round_to(q, "f16"), kd, vd, lk, (5, 4), (5, 4), d ** -0.5, wr=0)
    assert_close(got, want, what="config 1", out="f16")
    # the unfused CPU path of the reference: dequantize to the cache dtype, then matmul softmax matmul
    kdq = oracle.round_to(oracle.dequantize_rows(kd.reshape(-1, 34), d, 5), "f16").reshape(b, hkv, lk, d).transpose(0, 2, 1, 3)
    vdq = oracle.round_to(oracle.dequantize_rows(vd.reshape(-1, 34), d, 5), "f16").reshape(b, hkv, lk, d).transpose(0, 2, 1, 3)
    unf = oracle.unfused_attention(oracle.round_to(q, "f16").transpose(0, 2, 1, 3), kdq, vdq, d ** -0.5, wr=0).transpose(0, 2, 1, 3)
    assert_close(got, unf, what="config 1 vs the unfused path", out="f16")


def test_full_size_properties_config2(P, oracle):
    """At the full size of the ragged MXFP4 configuration (B=64, lengths in [512, 8192]): a slice is
    checked against the oracle, the rest through properties that do not depend on the size."""
    b, hq, hkv, d = 64, 32, 8, 128
    lens = (512 + oracle.u64s(2002, b) % np.uint64(7681)).astype(np.int32)
    cap = int(lens.max())
    g = torch.Generator(device="cuda:0").manual_seed(5)
    # the configuration's value distribution: N(0, 1) with 1 % of the (kv head, channel) pairs scaled by 8
    chan = torch.ones(hkv * d, device="cuda:0", dtype=torch.bfloat16)
    chan[torch.from_numpy(np.random.default_rng(2003).choice(hkv * d, size=(hkv * d + 99) // 100, replace=False)).to("cuda:0")] = 8
    chan = chan.view(1, hkv, 1, d)
    k = torch.randn((b, hkv, cap, d), generator=g, device="cuda:0", dtype=torch.bfloat16) * chan
    v = torch.randn((b, hkv, cap, d), generator=g, device="cuda:0", dtype=torch.bfloat16) * chan
    q = torch.randn((b, hq, 1, d), generator=g, device="cuda:0", dtype=torch.bfloat16)
    cache = P.TurboKvCache(fmt(P, 2), fmt(P, 2), d, "none", 42, cap)
    cache.append(k, v)
    kvl = torch.from_numpy(lens).to("cuda:0")
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    out = P.attention_packed(q, cache.k, cache.v, kvl, cache.kq, cache.vq, cfg)
    # 1. slice parity: three sequences (shortest, longest, first), all heads, full context
    for bi in sorted({int(lens.argmin()), int(lens.argmax()), 0}):
        L = int(lens[bi])
        kd, vd = words(cache.k[bi:bi + 1, :, :L]), words(cache.v[bi:bi + 1, :, :L])
        kx = k[bi, :, :L].float().cpu().numpy().reshape(-1, d)
        assert np.array_equal(kd.reshape(-1, 19), oracle.quantize_rows(kx, 2))
        want = oracle.tq_attention(q[bi:bi + 1].float().cpu().numpy(), kd, vd, L, (2, 4), (2, 4), d ** -0.5, wr=0)
        assert_close(out[bi:bi + 1].float().cpu().numpy(), want, what=f"sequence {bi}", out="bf16")
    # 2. the split count does not change the result beyond rounding
    cfg2 = P.FlashAttnConfig(d ** -0.5).causal()
    cfg2.splits = 3
    out2 = P.attention_packed(q, cache.k, cache.v, kvl, cache.kq, cache.vq, cfg2)
    assert_close(out2.float().cpu().numpy(), out.float().cpu().numpy(), atol=4e-3, rtol=8e-3, what="split invariance")
    # 3. keys beyond kv_len are never read: poisoning them changes nothing
    for bi in range(b):
        cache.k[bi, :, int(lens[bi]):] = 0x7FC07FC0
        cache.v[bi, :, int(lens[bi]):] = 0x7FC07FC0
    out3 = P.attention_packed(q, cache.k, cache.v, kvl, cache.kq, cache.vq, cfg)
    assert torch.equal(out3, out)
    # 4. linearity in V: every E8M0 block scale of the value rows one step up (word 16 of a row holds the four scale
    # bytes) doubles every value exactly, so the outputs double (to the rounding of the weights, whose running maxima
    # move by one)
    assert torch.isfinite(out).all()
    cache.v[:, :, :, 16] += 0x01010101
    out4 = P.attention_packed(q, cache.k, cache.v, kvl, cache.kq, cache.vq, cfg)
    assert_close(out4.float().cpu().numpy(), 2.0 * out.float().cpu().numpy(), atol=2e-3, rtol=8e-3, what="linearity in V")


def _fill_cache(P, cache, b, hkv, ctx, d, dtype, seed):
    """Synthetic keys / values generated and quantized on the device in slabs (the caches of configs 4 and 5 are too
    large to come from the host); returns the slabs of the first two sequences for the oracle."""
    g = torch.Generator(device="cuda:0").manual_seed(seed)
    keep_k, keep_v = [], []
    for p0 in range(0, ctx, 2048):
        t = min(2048, ctx - p0)
        k = torch.randn((b, hkv, t, d), generator=g, device="cuda:0", dtype=dtype)
        v = torch.randn((b, hkv, t, d), generator=g, device="cuda:0", dtype=dtype)
        cache.append(k, v)
        keep_k.append(k[:2].float().cpu().numpy())
        keep_v.append(v[:2].float().cpu().numpy())
    return np.concatenate(keep_k, axis=2), np.concatenate(keep_v, axis=2)


def test_full_size_config4_turboquant(P, oracle):
    """One GPU's share of the long-context TurboQuant configuration (one kv head of B=32, Hq=64/8, context 32768,
    4-bit codebook rows, seeded Hadamard rotation): two sequences over the full context against the oracle on the
    rows copied back, the batch through split invariance."""
    b, hq, hkv, d, ctx = 32, 8, 1, 128, 32768
    cache = P.TurboKvCache(fmt(P, 0, 4), fmt(P, 0, 4), d, "hadamard", 42, ctx)
    kx, vx = _fill_cache(P, cache, b, hkv, ctx, d, torch.bfloat16, 41)
    assert cache.seq_len() == ctx
    q = torch.randn((b, hq, 1, d), generator=torch.Generator(device="cuda:0").manual_seed(3), device="cuda:0", dtype=torch.bfloat16)
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    out = cache.attention(q, cfg)
    kd, vd = words(cache.k[:2]), words(cache.v[:2])
    # rows: bit-exact with the reference quantizer on the rows the device butterflies give
    rot = cache.kq.rotate(to_dev(kx[:, :, :256].reshape(-1, d), "bf16")).cpu().numpy()
    tab = MG.tab_for(0, 4, d)
    assert np.array_equal(kd[:, :, :256].reshape(-1, 18), oracle.quantize_rows(rot, 0, 4, tab))
    # attention in the rotated space over the same rows, rotated back
    qr = oracle.rotate_rows(q[:2].float().cpu().numpy().reshape(-1, d), oracle.rotation_matrix(d, 1, 42)).reshape(2, hq, 1, d)
    tabs = np.zeros(64, np.float32)
    tabs[:32] = tab
    tabs[32:] = tab
    want = oracle.tq_attention(qr, kd, vd, ctx, (0, 4), (0, 4), d ** -0.5, tabs, wr=0)
    want = oracle.rotate_rows(want.reshape(-1, d), oracle.rotation_matrix(d, 1, 44), transpose=True).reshape(want.shape)
    assert_close(out[:2].float().cpu().numpy(), want, what="config 4, two sequences", out="bf16")
    cfg2 = P.FlashAttnConfig(d ** -0.5).causal()
    cfg2.splits = 5
    out2 = cache.attention(q, cfg2)
    assert_close(out2.float().cpu().numpy(), out.float().cpu().numpy(), atol=4e-3, rtol=8e-3, what="split invariance")


def test_full_size_config5_mxfp8_layer(P, oracle):
    """One layer of the MXFP8 sweep (B=128, Hq=32, Hkv=8, context 16384, f16): 4.7 GB of packed rows on the device; two
    sequences against the oracle on the rows copied back, all of them finite and independent of the split count."""
    b, hq, hkv, d, ctx = 128, 32, 8, 128, 16384
    cache = P.TurboKvCache(fmt(P, 4), fmt(P, 4), d, "none", 42, ctx)
    kx, vx = _fill_cache(P, cache, b, hkv, ctx, d, torch.float16, 51)
    q = torch.randn((b, hq, 1, d), generator=torch.Generator(device="cuda:0").manual_seed(4), device="cuda:0", dtype=torch.float16)
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    out = cache.attention(q, cfg)
    kd, vd = words(cache.k[:2]), words(cache.v[:2])
    assert np.array_equal(kd[0, 0, :512], oracle.quantize_rows(kx[0, 0, :512], 4))
    want = oracle.tq_attention(q[:2].float().cpu().numpy(), kd, vd, ctx, (4, 4), (4, 4), d ** -0.5, wr=0)
    assert_close(out[:2].float().cpu().numpy(), want, what="config 5, two sequences", out="f16")
    assert torch.isfinite(out).all()
    cfg2 = P.FlashAttnConfig(d ** -0.5).causal()
    cfg2.splits = 2
    out2 = cache.attention(q, cfg2)
    assert_close(out2.float().cpu().numpy(), out.float().cpu().numpy(), atol=4e-3, rtol=8e-3, what="split invariance")
    del cache
    torch.cuda.empty_cache()


def test_gather_epilogue_on_one_rank(P, oracle):
    """b200_tq_attention_gather with a world of one: the rows land in slot (step & 1) of the gathered buffer, the step
    and the flag advance, and the regular output is unchanged. (The exchange between
    ranks is exercised by `bench.py --gpus N`, which checks the gathered rows against an NCCL all-gather.)"""
    import ctypes as C
    A = P._abi
    dev = torch.device("cuda:0")
    b, hq, hkv, d, cap = 3, 8, 2, 128, 700
    kq = P.TurboQuantizer(fmt(P, A.MXFP4), d, "none", 42, dev)
    vq = P.TurboQuantizer(fmt(P, A.MXFP4), d, "none", 44, dev)
    k_rows = kq.quantize_rows(to_dev(oracle.normal(5, b * hkv * cap * d).reshape(-1, d), "bf16")).view(b, hkv, cap, -1)
    v_rows = vq.quantize_rows(to_dev(oracle.normal(6, b * hkv * cap * d).reshape(-1, d), "bf16")).view(b, hkv, cap, -1)
    kv_len = torch.tensor([700, 33, 512], dtype=torch.int32, device=dev)
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    buf = torch.full((2, 1, b * hq, d), 7.0, dtype=torch.bfloat16, device=dev)
    flags = torch.zeros(4, dtype=torch.int32, device=dev)
    state = torch.zeros(2, dtype=torch.int32, device=dev)
    ptrs = torch.tensor([buf.data_ptr(), flags.data_ptr()], dtype=torch.int64, device=dev)

    class G:  # what OutputGather provides, without symmetric memory
        pass
    g = G()
    g.buf = buf
    g.args = A.PeerGather(ptrs.data_ptr(), ptrs.data_ptr() + 8, 1, 0, state.data_ptr(), state.data_ptr() + 4)
    for step in (1, 2, 3):
        q = to_dev(oracle.normal(90 + step, b * hq * d).reshape(b, hq, 1, d), "bf16")
        want = P.attention_packed(q, k_rows, v_rows, kv_len, kq, vq, cfg)
        got = P.PackedAttention(q, k_rows, v_rows, kv_len, kq, vq, cfg, gather=g).run()
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert state.tolist() == [step, 0] and flags.tolist()[0] == step
        assert torch.equal(buf[step & 1, 0].view(b, hq, 1, d), want)
    with pytest.raises(A.B200Error, match="world"):
        g.args.world = 0
        P.PackedAttention(q, k_rows, v_rows, kv_len, kq, vq, cfg, gather=g).run()


@pytest.mark.parametrize("case", MG.PROD_ATTN_CASES, ids=lambda c: c[0])
def test_prod_keys_against_reference_kernel_outputs(P, oracle, golden, case):
    """TurboProd keys (codebook codes + the 1-bit sketch of the residual): the attention over the reference's own rows
    against the outputs of its tq_attn kernels; then a cache that quantizes the keys itself against the oracle."""
    A = P._abi
    name, bits, b, lq, lk, hq, hkv, d, splits, group, wl, wr = case
    qx, kd, vd, tab = MG.prod_attn_inputs_from(golden["tq_prod"][name + "_kd"], case)
    kq = P.TurboQuantizer(P.QuantFormat(A.TURBO_PROD, bits), d, "none", MG.PROD_SEED)
    vq = P.TurboQuantizer(fmt(P, 0, 4), d, "none", MG.PROD_SEED + 2)
    c = P.FlashAttnConfig(d ** -0.5)
    c.window_size_left = None if wl < 0 else wl
    c.window_size_right = None if wr < 0 else wr
    got = P.attention_packed(to_dev(qx[..., :d]), rows_dev(kd), rows_dev(vd), lk, kq, vq, c).cpu().numpy()
    assert_close(got, golden["tq_prod"][name], what=name)
    # end to end: rows written by the cache (device matmuls in the sketch), attention against the oracle on those rows
    cache = P.TurboKvCache(P.QuantFormat(A.TURBO_PROD, bits), fmt(P, 0, 4), d, "none", MG.PROD_SEED, lk)
    g = torch.Generator(device="cuda:0").manual_seed(bits)
    kx = torch.randn((b, hkv, lk, d), generator=g, device="cuda:0")
    vx = torch.randn((b, hkv, lk, d), generator=g, device="cuda:0")
    cache.append(kx, vx)
    q = torch.randn((b, hq, lq, d), generator=g, device="cuda:0")
    got = cache.attention(q, c).cpu().numpy()
    s = oracle.qjl_matrix(d, MG.PROD_SEED)
    qn = q.cpu().numpy()
    qxx = np.concatenate([qn, qn @ s.T], axis=-1)
    want = oracle.tq_attention(qxx, words(cache.k[:, :, :lk]), words(cache.v[:, :, :lk]), lk, (oracle.PROD, bits), (oracle.MSE, 4), d ** -0.5,
                               tab, wl=wl, wr=wr)
    assert_close(got, want, what=name + " cache")
    # and the estimate is the unbiased one: far closer to exact attention than the codebook part alone
    lay = oracle.row_layout(oracle.PROD, bits, d)
    k0 = words(cache.k[:, :, :lk]).copy()
    k0[..., lay["rsc_offset"] + 1] = 0
    no_sketch = oracle.tq_attention(qxx, k0, words(cache.v[:, :, :lk]), lk, (oracle.PROD, bits), (oracle.MSE, 4), d ** -0.5, tab, wl=wl, wr=wr)
    assert np.abs(no_sketch - want).max() > 1e-3


def _local_gather(P, world, rows, d, dev, max_polls=0):
    """What OutputGather provides, without symmetric memory: every rank's buffer and flags are plain local allocations."""
    A = P._abi

    class G:
        pass
    g = G()
    g.buf = torch.full((2, world, rows, d), 7.0, dtype=torch.bfloat16, device=dev)
    g.peer_bufs = [g.buf] + [torch.full_like(g.buf, 9.0) for _ in range(world - 1)]
    g.flags = [torch.zeros(max(world, 4), dtype=torch.int32, device=dev) for _ in range(world)]
    g.state = torch.zeros(2, dtype=torch.int32, device=dev)
    g.ptrs = torch.tensor([t.data_ptr() for t in g.peer_bufs] + [t.data_ptr() for t in g.flags], dtype=torch.int64, device=dev)
    g.args = A.PeerGather(g.ptrs.data_ptr(), g.ptrs.data_ptr() + 8 * world, world, 0, g.state.data_ptr(), g.state.data_ptr() + 4, max_polls, 0)
    return g


def test_gather_epilogue_inside_the_decode_grid(P, oracle):
    """Many columns: the decode grid merges its segments itself and the workers that finish the rows store them into
    the gathered buffer; the worker that finishes the call's last column publishes the step. Ragged lengths with empty
    sequences (their zero rows are gathered too)."""
    A = P._abi
    dev = torch.device("cuda:0")
    b, hq, hkv, d, cap = 96, 8, 2, 128, 300
    kq = P.TurboQuantizer(fmt(P, A.MXFP4), d, "none", 42, dev)
    vq = P.TurboQuantizer(fmt(P, A.MXFP4), d, "none", 44, dev)
    g0 = torch.Generator(device=dev).manual_seed(3)
    k_rows = kq.quantize_rows(torch.randn((b * hkv * cap, d), generator=g0, device=dev, dtype=torch.bfloat16)).view(b, hkv, cap, -1)
    v_rows = vq.quantize_rows(torch.randn((b * hkv * cap, d), generator=g0, device=dev, dtype=torch.bfloat16)).view(b, hkv, cap, -1)
    lens = np.random.default_rng(1).integers(1, cap + 1, size=b).astype(np.int32)
    lens[3] = lens[40] = 0
    kv_len = torch.from_numpy(lens).to(dev)
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    g = _local_gather(P, 1, b * hq, d, dev)
    for step in (1, 2, 3):
        q = torch.randn((b, hq, 1, d), generator=g0, device=dev, dtype=torch.bfloat16)
        want = P.attention_packed(q, k_rows, v_rows, kv_len, kq, vq, cfg)
        got = P.PackedAttention(q, k_rows, v_rows, kv_len, kq, vq, cfg, gather=g).run()
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert g.state.tolist() == [step, 0] and g.flags[0].tolist()[0] == step
        assert torch.equal(g.buf[step & 1, 0].view(b, hq, 1, d), want)
        assert bool((got[3] == 0).all())


@pytest.mark.parametrize("b", [3, 96])  # the publish step as a grid of its own behind the combine grid / inside the decode grid
def test_gather_wait_for_a_rank_that_never_answers(P, oracle, b):
    """Failure detection without a fault: a world of two whose second rank does not exist (its buffer and flags are
    local allocations that nobody writes). The wait for its flag runs out after max_polls polls: the call returns, the
    status word says 2, the library-wide flag is raised, this rank's own rows are complete, and the next call (a world
    of one on the same state words) works."""
    A = P._abi
    dev = torch.device("cuda:0")
    hq, hkv, d, cap = 8, 2, 128, 300
    kq = P.TurboQuantizer(fmt(P, A.MXFP4), d, "none", 42, dev)
    vq = P.TurboQuantizer(fmt(P, A.MXFP4), d, "none", 44, dev)
    g0 = torch.Generator(device=dev).manual_seed(4)
    k_rows = kq.quantize_rows(torch.randn((b * hkv * cap, d), generator=g0, device=dev, dtype=torch.bfloat16)).view(b, hkv, cap, -1)
    v_rows = vq.quantize_rows(torch.randn((b * hkv * cap, d), generator=g0, device=dev, dtype=torch.bfloat16)).view(b, hkv, cap, -1)
    kv_len = torch.from_numpy(np.random.default_rng(2).integers(1, cap + 1, size=b).astype(np.int32)).to(dev)
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    q = torch.randn((b, hq, 1, d), generator=g0, device=dev, dtype=torch.bfloat16)
    want = P.attention_packed(q, k_rows, v_rows, kv_len, kq, vq, cfg)
    assert A.lib().b200_device_wait_check(1) == A.OK
    g = _local_gather(P, 2, b * hq, d, dev, max_polls=2000)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    got = P.PackedAttention(q, k_rows, v_rows, kv_len, kq, vq, cfg, gather=g, status=status).run()
    torch.cuda.synchronize()                                   # returns: the wait is bounded
    assert int(status.item()) == 2
    assert torch.equal(got, want)                              # the attention itself is complete
    assert torch.equal(g.buf[1, 0].view(b, hq, 1, d), want)    # and so are this rank's rows, in both ranks' buffers
    assert torch.equal(g.peer_bufs[1][1, 0].view(b, hq, 1, d), want)
    assert g.flags[1].tolist()[0] == 1 and g.flags[0].tolist()[1] == 0
    assert g.state.tolist() == [1, 0]                          # the step advanced, the column counter is back at zero
    assert A.lib().b200_device_wait_status() == 1
    assert A.lib().b200_device_wait_check(1) == A.ERR_DEVICE_WAIT and b"wait" in A.lib().b200_last_error()
    assert A.lib().b200_device_wait_status() == 0
    # the same state words, a world of one: works, and takes the next step's slot
    g.args.world = 1
    status.zero_()
    got = P.PackedAttention(q, k_rows, v_rows, kv_len, kq, vq, cfg, gather=g, status=status).run()
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and torch.equal(got, want)
    assert g.state.tolist() == [2, 0] and torch.equal(g.buf[0, 0].view(b, hq, 1, d), want)
    assert A.lib().b200_device_wait_status() == 0


@pytest.mark.parametrize("kf,vf", [((2, 4), (2, 4)), ((0, 4), (0, 3)), ((5, 4), (4, 4))])
def test_paged_blocks_equal_the_concatenated_rows(P, oracle, kf, vf):
    """attention_packed_blocks over four cache blocks of different capacities and fill levels (one of them empty)
    against the oracle on the concatenated valid rows (candle-nn/src/turbo_quant.rs:1536-1563 tests the same way)."""
    b, hq, hkv, d, lq = 2, 4, 2, 128, 2
    kq = P.TurboQuantizer(fmt(P, *kf), d, "none", 42)
    vq = P.TurboQuantizer(fmt(P, *vf), d, "none", 44)
    caps, fills = [16, 64, 8, 128], [16, 9, 0, 100]
    blocks, kcat, vcat = [], [], []
    for n, (cap, rows) in enumerate(zip(caps, fills)):
        kx = oracle.normal(700 + n, b * hkv * cap * d).reshape(-1, d)
        vx = oracle.normal(800 + n, b * hkv * cap * d).reshape(-1, d)
        kb = kq.quantize_rows(to_dev(kx)).view(b, hkv, cap, -1).contiguous()
        vb = vq.quantize_rows(to_dev(vx)).view(b, hkv, cap, -1).contiguous()
        blocks.append(P.KvBlockRef(kb, vb, rows))
        kcat.append(words(kb)[:, :, :rows])
        vcat.append(words(vb)[:, :, :rows])
    kd, vd = np.concatenate(kcat, axis=2), np.concatenate(vcat, axis=2)
    lk = sum(fills)
    q = oracle.normal(9, b * hq * lq * d).reshape(b, hq, lq, d)
    tab = np.zeros(64, np.float32)
    tab[:32] = MG.tab_for(kf[0], kf[1], d)
    tab[32:] = MG.tab_for(vf[0], vf[1], d)
    for wl, wr in ((-1, 0), (30, 0), (-1, -1)):
        c = P.FlashAttnConfig(d ** -0.5)
        c.window_size_left = None if wl < 0 else wl
        c.window_size_right = None if wr < 0 else wr
        want = oracle.tq_attention(q, np.ascontiguousarray(kd), np.ascontiguousarray(vd), lk, kf, vf, d ** -0.5, tab, wl=wl, wr=wr)
        # blocks compacted into the workspace for the tensor-core kernel (where the format has one), and read in place
        for in_place in (False, True):
            got = P.attention_packed_blocks(to_dev(q), blocks, kq, vq, c, in_place=in_place).cpu().numpy()
            assert_close(got, want, what=f"paged wl={wl} wr={wr} in_place={in_place}")
    with pytest.raises(ValueError, match="no blocks"):
        P.attention_packed_blocks(to_dev(q), [], kq, vq, c)
    # B200_TQ_AFTER_PREV on a paged call: the kernels that prepare the table run right before the attention, which
    # must not start as their programmatic dependent; the rows are those of the plain call
    c = P.FlashAttnConfig(d ** -0.5).causal()
    plain = P.attention_packed_blocks(to_dev(q), blocks, kq, vq, c)
    for _ in range(3):
        assert torch.equal(P.attention_packed_blocks(to_dev(q), blocks, kq, vq, c, after_prev=True), plain)


def test_long_paged_rows_in_place_on_the_general_kernel(P, oracle):
    """B200_TQ_IN_PLACE: keys and values in different formats over 30 blocks, read where they are by the general kernel,
    which splits the 2 400 keys of the few output rows; against the oracle on the concatenated rows, and the same
    call without a workspace (one block per row) within rounding of it."""
    b, hq, hkv, d, lq = 1, 4, 2, 128, 1
    kf, vf = (5, 4), (2, 4)
    kq, vq = P.TurboQuantizer(fmt(P, *kf), d, "none", 42), P.TurboQuantizer(fmt(P, *vf), d, "none", 44)
    blocks, kcat, vcat = [], [], []
    g = torch.Generator(device="cuda:0").manual_seed(5)
    for n in range(30):
        cap, rows = 96, 96 - (n % 5) * 8
        kb = kq.quantize_rows(torch.randn((b * hkv * cap, d), generator=g, device="cuda:0")).view(b, hkv, cap, -1).contiguous()
        vb = vq.quantize_rows(torch.randn((b * hkv * cap, d), generator=g, device="cuda:0")).view(b, hkv, cap, -1).contiguous()
        blocks.append(P.KvBlockRef(kb, vb, rows))
        kcat.append(words(kb)[:, :, :rows])
        vcat.append(words(vb)[:, :, :rows])
    kd, vd = np.concatenate(kcat, axis=2), np.concatenate(vcat, axis=2)
    lk = kd.shape[2]
    q = oracle.normal(19, b * hq * lq * d).reshape(b, hq, lq, d)
    c = P.FlashAttnConfig(d ** -0.5).causal()
    want = oracle.tq_attention(q, np.ascontiguousarray(kd), np.ascontiguousarray(vd), lk, kf, vf, d ** -0.5, np.zeros(64, np.float32), wr=0)
    call = P.PackedBlocksAttention(to_dev(q), blocks, kq, vq, c, in_place=True)
    assert call.args.workspace_bytes > 16  # partial rows of the key splits
    got = call.run().cpu().numpy()
    assert_close(got, want, what="paged in place, split")
    call.args.workspace_bytes = 16  # too small for the splits: one block per output row
    assert_close(call.run().cpu().numpy(), want, what="paged in place, no split")


@pytest.mark.parametrize("f,d", [((2, 4), 128), ((4, 4), 128), ((0, 4), 64), ((5, 4), 256), ((3, 4), 128)])
def test_paged_rows_read_where_they_are(P, oracle, f, d):
    """The tensor-core kernel walking the block table: blocks of odd fill levels (tiles end where blocks end, so most
    blocks end in a short tile), an empty block, a full one whose last row is the last row of its allocation, a batch
    with per-sequence lengths (one of them zero, one ending inside the first block, one taking every key), windows.
    Against the oracle on the concatenated rows with the same lengths."""
    b, hq, hkv, lq = 5, 8, 2, 1
    kq, vq = P.TurboQuantizer(fmt(P, *f), d, "none", 42), P.TurboQuantizer(fmt(P, *f), d, "none", 44)
    caps, fills = [40, 64, 8, 32, 200, 33], [37, 64, 0, 32, 131, 1]
    blocks, kcat, vcat = [], [], []
    g = torch.Generator(device="cuda:0").manual_seed(d + f[0])
    for cap, rows in zip(caps, fills):
        kb = kq.quantize_rows(torch.randn((b * hkv * cap, d), generator=g, device="cuda:0")).view(b, hkv, cap, -1).contiguous()
        vb = vq.quantize_rows(torch.randn((b * hkv * cap, d), generator=g, device="cuda:0")).view(b, hkv, cap, -1).contiguous()
        blocks.append(P.KvBlockRef(kb, vb, rows))
        kcat.append(words(kb)[:, :, :rows])
        vcat.append(words(vb)[:, :, :rows])
    kd, vd = np.ascontiguousarray(np.concatenate(kcat, axis=2)), np.ascontiguousarray(np.concatenate(vcat, axis=2))
    lk = sum(fills)
    tab = np.zeros(64, np.float32)
    tab[:32] = tab[32:] = MG.tab_for(f[0], f[1], d)
    q = torch.randn((b, hq, lq, d), generator=g, device="cuda:0")
    lens = np.array([lk, 0, 20, 102, 265], np.int32)
    for wl, wr in ((-1, 0), (70, 0)):
        c = P.FlashAttnConfig(d ** -0.5)
        c.window_size_left = None if wl < 0 else wl
        c.window_size_right = None if wr < 0 else wr
        want = oracle.tq_attention(q.cpu().numpy(), kd, vd, lk, f, f, d ** -0.5, tab, wl=wl, wr=wr)
        got = P.attention_packed_blocks(q, blocks, kq, vq, c).cpu().numpy()
        assert_close(got, want, what=f"paged walk wl={wl}")
        want = oracle.tq_attention(q.cpu().numpy(), kd, vd, lk, f, f, d ** -0.5, tab, kv_len=lens, wl=wl, wr=wr)
        got = P.attention_packed_blocks(q, blocks, kq, vq, c, kv_len=torch.from_numpy(lens).to("cuda:0")).cpu().numpy()
        assert np.all(got[1] == 0)
        assert_close(got, want, what=f"ragged paged walk wl={wl}")
    # several query tokens per sequence (chunked prefill over a paged cache)
    q3 = torch.randn((b, hq, 3, d), generator=g, device="cuda:0")
    c = P.FlashAttnConfig(d ** -0.5).causal()
    want = oracle.tq_attention(q3.cpu().numpy(), kd, vd, lk, f, f, d ** -0.5, tab, wr=0)
    assert_close(P.attention_packed_blocks(q3, blocks, kq, vq, c).cpu().numpy(), want, what="paged walk lq=3")


def test_paged_rows_with_whole_tiles_give_the_bits_of_the_dense_call(P, oracle):
    """Blocks whose fill levels are multiples of the tile (512 rows): the walk over the table cuts the keys into the
    same tiles as the call over the concatenated rows, so the outputs are the same bits."""
    b, hq, hkv, d, nblk, rows = 16, 32, 8, 128, 8, 512
    f = fmt(P, 2, 4)
    kq, vq = P.TurboQuantizer(f, d, "none", 42), P.TurboQuantizer(f, d, "none", 44)
    g = torch.Generator(device="cuda:0").manual_seed(77)
    blocks = []
    for _ in range(nblk):
        kb = kq.quantize_rows(torch.randn((b * hkv * rows, d), generator=g, device="cuda:0", dtype=torch.bfloat16)).view(b, hkv, rows, -1)
        vb = vq.quantize_rows(torch.randn((b * hkv * rows, d), generator=g, device="cuda:0", dtype=torch.bfloat16)).view(b, hkv, rows, -1)
        blocks.append(P.KvBlockRef(kb, vb, rows))
    q = torch.randn((b, hq, 1, d), generator=g, device="cuda:0", dtype=torch.bfloat16)
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    dense_k = torch.cat([blk.k for blk in blocks], dim=2).contiguous()
    dense_v = torch.cat([blk.v for blk in blocks], dim=2).contiguous()
    want = P.attention_packed(q, dense_k, dense_v, nblk * rows, kq, vq, cfg)
    got = P.attention_packed_blocks(q, blocks, kq, vq, cfg)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
