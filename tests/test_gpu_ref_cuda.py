"""The CUDA path against the reference's own GPU kernels on the same device and the same packed rows.

baseline/_ref_cuda/libref_cuda.so is the reference's kernel headers compiled for sm_100a with the instantiation lines and
the launch plan of the reference (baseline/ref_cuda.cu); it is built where the reference tree is present and travels as a
built file. Without it these tests are skipped: the other parity tests (CPU oracle, golden vectors) do not depend on it."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from baseline import ref_cuda as R  # noqa: E402
from gpu_util import assert_close, pkg  # noqa: E402

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not R.available(), reason="baseline/_ref_cuda/libref_cuda.so was not built")]

CASES = [
    # fmt, rotation, q dtype, b, hq, hkv, lens
    ("mxfp4", "none", torch.bfloat16, 6, 32, 8, [512, 1999, 8192, 3000, 77, 4097]),
    ("fp8", "none", torch.float16, 1, 32, 8, [2048]),
    ("mxfp8", "none", torch.float16, 4, 32, 8, [4096] * 4),
    ("nvfp4", "hadamard", torch.bfloat16, 3, 16, 8, [1000, 129, 2500]),
    ("turbo4", "hadamard", torch.bfloat16, 2, 16, 2, [6000, 6000]),
    ("turbo4", "hadamard", torch.bfloat16, 3, 8, 8, [100, 3333, 1024]),
]


@pytest.mark.parametrize("fmt,rot,dt,b,hq,hkv,lens", CASES, ids=[f"{c[0]}-{c[1]}-b{c[3]}-g{c[4] // c[5]}" for c in CASES])
def test_attention_matches_the_reference_kernels_on_this_gpu(fmt, rot, dt, b, hq, hkv, lens):
    P = pkg()
    dev = torch.device("cuda:0")
    d, cap = 128, max(lens)
    g = torch.Generator(device=dev).manual_seed(7)
    kq = P.TurboQuantizer(P.QuantFormat.parse(fmt), d, rot, 42, dev)
    vq = P.TurboQuantizer(P.QuantFormat.parse(fmt), d, rot, 44, dev)
    k = torch.randn((b * hkv * cap, d), generator=g, device=dev, dtype=torch.float32)
    v = torch.randn((b * hkv * cap, d), generator=g, device=dev, dtype=torch.float32)
    k[:, 5] *= 8  # an outlier channel
    kc = kq.quantize_rows(k).view(b, hkv, cap, -1)
    vc = vq.quantize_rows(v).view(b, hkv, cap, -1)
    q = torch.randn((b, hq, 1, d), generator=g, device=dev, dtype=torch.float32).to(dt)
    kv_len = torch.tensor(lens, dtype=torch.int32, device=dev)
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    got = P.attention_packed(q, kc, vc, kv_len, kq, vq, cfg)

    # the reference rotates the queries before its kernel and the outputs after it (candle-nn/src/turbo_quant.rs:1161,1033)
    q32 = kq.rotate(q.reshape(-1, d)).view(b, hq, 1, d)
    tab = torch.cat([kq.tab, vq.tab])
    ref = R.TqAttention(torch, q32, kc, vc, lens, kq.layout, vq.layout, kq.format.mode, vq.format.mode, tab, d ** -0.5, 148)
    want = ref.run(torch.cuda.current_stream(dev).cuda_stream)
    want = vq.unrotate(want.reshape(-1, d)).view(b, hq, 1, d)
    torch.cuda.synchronize()
    assert torch.isfinite(want).all()
    assert_close(got.float().cpu().numpy(), want.cpu().numpy(), what=f"{fmt} vs reference kernels",
                 out={torch.bfloat16: "bf16", torch.float16: "f16"}[dt])


def test_quantized_rows_are_the_bits_of_the_reference_kernel():
    """tq_quant_f32 of the reference on this GPU against b200_tq_quantize, every format, bit for bit."""
    P = pkg()
    dev = torch.device("cuda:0")
    d, rows = 128, 4096
    g = torch.Generator(device=dev).manual_seed(11)
    x = torch.randn((rows, d), generator=g, device=dev, dtype=torch.float32)
    x[::7, 3] *= 50
    x[5] = 0
    for fmt in ("fp8", "mxfp8", "mxfp4", "nvfp4", "turbo4", "turbo2"):
        tq = P.TurboQuantizer(P.QuantFormat.parse(fmt), d, "none", 42, dev)
        ours = tq.quantize_rotated_rows(x)
        L = tq.layout
        theirs = torch.zeros_like(ours)
        rc = R.lib().refcu_tq_quant(x.data_ptr(), 0, theirs.data_ptr(), tq.tab.data_ptr(), rows, d, d, tq.format.mode, L.code_bits,
                                    L.code_words, L.aux_words, L.row_words, torch.cuda.current_stream(dev).cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        same = (ours == theirs).all(dim=1)
        if fmt.startswith("turbo"):
            # the norm is a sum of squares: the reference itself allows a small share of flipped codes between its
            # implementations (candle-core/tests/accel_kernels_host.rs:1022-1027)
            assert same.float().mean().item() >= 0.999, f"{fmt}: {(~same).sum().item()} of {rows} rows differ"
        else:
            assert same.all(), f"{fmt}: {(~same).sum().item()} of {rows} rows differ"
