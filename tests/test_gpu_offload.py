"""Pinned host buffers and the copy stream (candle-core/src/cuda_backend/offload.rs): ordering against the compute
stream in both directions, range checks, reuse of a staging buffer, and packed KV blocks that live in host memory and
are uploaded behind another layer's attention."""
import numpy as np
import pytest
import torch

from gpu_util import fmt, pkg

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def P():
    return pkg()


def test_upload_and_download_are_ordered_with_the_compute_stream(P):
    dev = torch.device("cuda:0")
    copy = P.CopyStream(dev)
    n = 8 << 20
    host = P.PinnedHostBuffer(n)
    assert len(host) == n
    rng = np.random.default_rng(1)
    data = rng.integers(0, 256, n, dtype=np.uint8)
    host.numpy()[:] = data
    slot = torch.zeros(n + 4096, dtype=torch.uint8, device=dev)
    # a long chain of kernels on the compute stream that writes the slot: the upload must start after it
    for _ in range(50):
        slot.add_(1)
    ev = copy.upload(host, 0, slot, 4096, n)
    ev.wait_on_compute()
    got = slot[4096:].clone()          # queued after the wait: sees the uploaded bytes
    head = slot[:4096].clone()
    torch.cuda.synchronize()
    assert ev.is_complete()
    assert np.array_equal(got.cpu().numpy(), data)
    assert (head == 50).all()          # bytes outside the copied range keep the kernels' result
    # download: starts after the kernels queued before it, read through the buffer (which waits for the copy)
    back = P.PinnedHostBuffer(n)
    x = torch.zeros(n, dtype=torch.uint8, device=dev)
    for _ in range(37):
        x.add_(1)
    ev3 = copy.download(x, 16, back, 32, 1000)
    ev3.wait_on_compute()              # the source may be overwritten by work queued after this wait
    x.zero_()
    ev3.synchronize()
    assert (back.numpy()[32:1032] == 37).all()
    copy.synchronize()
    for e in (ev, ev3):
        e.close()
    host.close()
    back.close()


def test_ranges_and_devices_are_checked(P):
    A = P._abi
    dev = torch.device("cuda:0")
    copy = P.CopyStream(dev)
    host = P.PinnedHostBuffer(1024)
    t = torch.zeros(256, dtype=torch.float32, device=dev)
    for args in ((host, 1000, t, 0, 100), (host, 0, t, 1000, 100)):
        with pytest.raises(A.B200Error) as e:
            copy.upload(*args)
        assert e.value.code == A.ERR_BAD_ARG and "exceeds" in str(e.value)
    with pytest.raises(A.B200Error, match="exceeds"):
        copy.download(t, 1020, host, 0, 8)
    with pytest.raises(A.B200Error, match="exceeds"):
        copy.download(t, 0, host, 1020, 8)
    with pytest.raises(ValueError, match="another device"):
        copy.upload(host, 0, torch.zeros(4), 0, 4)
    with pytest.raises(ValueError, match="contiguous"):
        copy.upload(host, 0, torch.zeros((4, 4), device=dev).t(), 0, 4)
    # empty buffers and empty copies are fine
    empty = P.PinnedHostBuffer(0)
    assert len(empty) == 0 and empty.numpy().size == 0
    copy.upload(host, 0, t, 0, 0).close()


def test_a_staging_buffer_is_not_rewritten_under_a_running_copy(P):
    """Two uploads through one staging buffer: the second fill goes through numpy(), which waits for the first copy."""
    dev = torch.device("cuda:0")
    copy = P.CopyStream(dev)
    n = 64 << 20
    host = P.PinnedHostBuffer(n)
    a, b = torch.empty(n, dtype=torch.uint8, device=dev), torch.empty(n, dtype=torch.uint8, device=dev)
    host.numpy()[:] = 7
    e1 = copy.upload(host, 0, a, 0, n)
    host.numpy()[:] = 9                # must not reach the first copy
    e2 = copy.upload(host, 0, b, 0, n)
    e1.wait_on_compute()
    e2.wait_on_compute()
    torch.cuda.synchronize()
    assert (a == 7).all() and (b == 9).all()
    # an event nobody waited on: closing it orders the compute stream behind the copy
    host.numpy()[:] = 3
    copy.upload(host, 0, a, 0, n).close()
    s = a.sum(dtype=torch.int64)       # queued after the close: sees the copy
    assert int(s.item()) == 3 * n


def test_blocks_uploaded_from_host_memory_behind_another_layers_attention(P):
    """Packed KV blocks of a layer live in pinned host memory; they are uploaded into device slots on the copy stream
    while the attention of another (resident) layer runs, and attended over in place once the copy event was waited
    for. The result has the bits of the same call over blocks that never left the device."""
    dev = torch.device("cuda:0")
    b, hq, hkv, d, nblk, cap = 4, 16, 4, 128, 24, 256
    kq, vq = P.TurboQuantizer(fmt(P, 2), d, "none", 42), P.TurboQuantizer(fmt(P, 2), d, "none", 44)
    g = torch.Generator(device=dev).manual_seed(21)
    rw = kq.row_words()
    blk_bytes = b * hkv * cap * rw * 4
    resident, fills = [], []
    for n in range(nblk):
        kb = kq.quantize_rows(torch.randn((b * hkv * cap, d), generator=g, device=dev)).view(b, hkv, cap, rw).contiguous()
        vb = vq.quantize_rows(torch.randn((b * hkv * cap, d), generator=g, device=dev)).view(b, hkv, cap, rw).contiguous()
        resident.append((kb, vb))
        fills.append(cap if n < nblk - 1 else 100)
    q = torch.randn((b, hq, 1, d), generator=g, device=dev).to(torch.bfloat16)
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    want = P.attention_packed_blocks(q, [P.KvBlockRef(k, v, r) for (k, v), r in zip(resident, fills)], kq, vq, cfg)
    # offload: every block's K and V bytes into one pinned buffer
    copy = P.CopyStream(dev)
    host = P.PinnedHostBuffer(2 * nblk * blk_bytes)
    down = []
    for n, (kb, vb) in enumerate(resident):
        down.append(copy.download(kb, 0, host, (2 * n) * blk_bytes, blk_bytes))
        down.append(copy.download(vb, 0, host, (2 * n + 1) * blk_bytes, blk_bytes))
    for e in down:
        e.synchronize()
    # the "other layer": a resident cache whose attention runs while the blocks come back
    other_k = kq.quantize_rows(torch.randn((b * hkv * 8192, d), generator=g, device=dev)).view(b, hkv, 8192, rw)
    other_v = vq.quantize_rows(torch.randn((b * hkv * 8192, d), generator=g, device=dev)).view(b, hkv, 8192, rw)
    slots = [(torch.zeros_like(k), torch.zeros_like(v)) for k, v in resident]
    ups = []
    for n, (ks, vs) in enumerate(slots):
        ups.append(copy.upload(host, (2 * n) * blk_bytes, ks, 0, blk_bytes))
        ups.append(copy.upload(host, (2 * n + 1) * blk_bytes, vs, 0, blk_bytes))
    for _ in range(8):
        P.attention_packed(q, other_k, other_v, 8192, kq, vq, cfg)     # runs beside the uploads
    for e in ups:
        e.wait_on_compute()
    got = P.attention_packed_blocks(q, [P.KvBlockRef(k, v, r) for (k, v), r in zip(slots, fills)], kq, vq, cfg)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    assert P._abi.lib().b200_device_wait_status() == 0
