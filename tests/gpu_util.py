"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import __graft_entry__ as G

TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
# tolerance of attention outputs against the reference arithmetic: 2e-3 relative, 1e-2 absolute
ATOL, RTOL = 1e-2, 2e-3


def pkg():
    G.build()
    return G.load_package()


def to_dev(x, dtype="f32"):
    return torch.from_numpy(np.ascontiguousarray(x)).to("cuda:0").to(TORCH_DT[dtype])


def rows_dev(a):
    """Packed u32 rows (numpy) -> int32 device tensor with the same bits."""
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int32)).to("cuda:0")


def words(t):
    return t.detach().cpu().numpy().view(np.uint32)


def fmt(P, mode, bits=4):
    return P.QuantFormat(mode, bits)


# half an ulp of the output dtype, relative: the kernels round their f32 result once to that dtype
HALF_ULP = {"f32": 0.0, "f16": 2.0 ** -12, "bf16": 2.0 ** -9}


def assert_close(got, want, atol=ATOL, rtol=RTOL, what="", out="f32"):
    """|got - want| <= atol + rtol |want| on the f32 result, plus the final rounding to `out`."""
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    err = np.abs(got - want)
    # "not (err <= tol)" rather than "err > tol": a NaN (an output row that was never written, or a broken one) fails
    bad = ~(err <= atol + (rtol + HALF_ULP[out]) * np.abs(want))
    bad &= ~(np.isnan(got) & np.isnan(want))
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} out of tolerance or not finite, max abs err {np.nanmax(err):.3e}"
    return float(np.nanmax(err)) if err.size else 0.0
