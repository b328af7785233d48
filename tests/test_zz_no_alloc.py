"""The entry point for hosts that cannot allocate device memory, b200_tq_attention_static.

Some callers of this library have no way to give it a workspace: the process gave all of HBM to
its own pool at start-up, or it sits in a decode loop where cudaMalloc / cudaFree are forbidden
because they synchronize the device. For them the library carries a fixed scratch buffer. This
test drives that entry point through the C ABI, twice in a row (the buffer keeps the first call's
contents, so the second call shows that stale contents do no harm), and compares each result with
the regular entry point, whose workspace the caller provides. It also checks the refusal of a
call that needs more scratch than the buffer holds. The file sorts last on purpose: if it fails,
every other test has already run.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import ATOL, RTOL, assert_close, fmt, pkg, rows_dev, to_dev

pytestmark = pytest.mark.gpu


def build_args(P, q, out, k_rows, v_rows, kv_len, kq, vq, scale):
    """The argument block of both entry points for a causal decode call (no workspace set)."""
    A = P._abi
    b, hq, lq, d = q.shape
    args = A.TqAttnArgs()
    args.q, args.out = q.data_ptr(), out.data_ptr()
    args.q_dtype = args.out_dtype = {torch.float32: A.F32, torch.float16: A.F16, torch.bfloat16: A.BF16}[q.dtype]
    args.q_strides, args.out_strides = A.u64x3(*q.stride()[:3]), A.u64x3(*out.stride()[:3])
    args.k_rows, args.v_rows = k_rows.data_ptr(), v_rows.data_ptr()
    args.k_strides, args.v_strides = A.u64x3(*k_rows.stride()[:3]), A.u64x3(*v_rows.stride()[:3])
    args.kv_len_dev = kv_len.data_ptr()
    args.b, args.lq, args.lk, args.hq, args.hkv, args.d = b, lq, k_rows.shape[2], hq, k_rows.shape[1], d
    args.kq, args.vq = kq.side(), vq.side()
    args.scale, args.softcap, args.wl, args.wr = scale, 0.0, -1, 0
    return args


def test_static_scratch_entry_matches_the_regular_one(oracle):
    P = pkg()
    A = P._abi
    lib = A.lib()
    dev = torch.device("cuda:0")
    b, hq, hkv, d, cap = 8, 32, 8, 128, 3000
    lens = np.array([3000, 17, 1024, 2999, 512, 1, 2048, 777], np.int32)
    kq = P.TurboQuantizer(fmt(P, A.MXFP4), d, "none", 42, dev)
    vq = P.TurboQuantizer(fmt(P, A.MXFP8), d, "none", 44, dev)
    kx = oracle.normal(71, b * hkv * cap * d).reshape(b * hkv * cap, d)
    vx = oracle.normal(72, b * hkv * cap * d).reshape(b * hkv * cap, d)
    k_rows = kq.quantize_rows(to_dev(kx, "bf16")).view(b, hkv, cap, -1)
    v_rows = vq.quantize_rows(to_dev(vx, "bf16")).view(b, hkv, cap, -1)
    kv_len = torch.from_numpy(lens).to(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    for call in range(2):  # two calls in a row share the built-in buffer
        q = to_dev(oracle.normal(80 + call, b * hq * d).reshape(b, hq, 1, d), "bf16")
        want_out = torch.empty_like(q)
        args = build_args(P, q, want_out, k_rows, v_rows, kv_len, kq, vq, d ** -0.5)
        need = lib.b200_tq_attention_workspace_bytes(C.byref(args))
        assert 0 < need <= A.STATIC_SCRATCH_BYTES
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        args.workspace, args.workspace_bytes = ws.data_ptr(), need
        A.check(lib.b200_tq_attention(C.byref(args), stream))
        got_out = torch.full_like(q, float("nan"))
        sargs = build_args(P, q, got_out, k_rows, v_rows, kv_len, kq, vq, d ** -0.5)
        A.check(lib.b200_tq_attention_static(C.byref(sargs), stream))
        torch.cuda.synchronize()
        assert_close(got_out.float().cpu().numpy(), want_out.float().cpu().numpy(), atol=ATOL, rtol=RTOL, what=f"call {call}")
        if call == 0:  # and against the CPU oracle once, so that both entry points are not wrong together
            want = oracle.tq_attention(q.float().cpu().numpy(), k_rows.cpu().numpy().view(np.uint32),
                                       v_rows.cpu().numpy().view(np.uint32), cap, (2, 4), (4, 4), d ** -0.5, kv_len=lens, wr=0)
            assert_close(got_out.float().cpu().numpy(), want, what="oracle", out="bf16")


def test_static_scratch_entry_refuses_oversized_calls():
    P = pkg()
    A = P._abi
    lib = A.lib()
    dev = torch.device("cuda:0")
    b, hq, hkv, d, cap = 4096, 8, 8, 128, 1  # many columns: the column table and partials outgrow the buffer
    kq = P.TurboQuantizer(fmt(P, A.FP8_ROW), d, "none", 42, dev)
    rows = torch.zeros((b, hkv, cap, kq.row_words()), dtype=torch.int32, device=dev)
    q = torch.zeros((b, hq, 1, d), dtype=torch.float16, device=dev)
    out = torch.empty_like(q)
    kv_len = torch.ones(b, dtype=torch.int32, device=dev)
    args = build_args(P, q, out, rows, rows, kv_len, kq, kq, 1.0)
    assert lib.b200_tq_attention_workspace_bytes(C.byref(args)) > A.STATIC_SCRATCH_BYTES
    rc = lib.b200_tq_attention_static(C.byref(args), torch.cuda.current_stream(dev).cuda_stream)
    assert rc == A.ERR_WORKSPACE
    msg = lib.b200_last_error().decode()
    assert str(A.STATIC_SCRATCH_BYTES) in msg and "b200_tq_attention" in msg
