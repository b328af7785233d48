"""Pinned host buffers and the device's copy stream, for packed KV blocks that live in host memory (or on disk) and are
uploaded while other layers compute. Mirrors candle-core/src/cuda_backend/offload.rs (`PinnedHostBuffer`, `CopyStream`,
`CopyEvent`, `CudaDevice::alloc_pinned` / `copy_stream`) over the C ABI (b200_pinned_*, b200_copy_*).

    copy = CopyStream(device)
    host = PinnedHostBuffer(nbytes)                    # once
    host.numpy()[:n] = block_bytes                     # waits for earlier copies of `host`
    ev = copy.upload(host, 0, slot, 0, n)              # slot: a device tensor; starts after the work queued so far
    ...                                                # other layers run while the DMA engine copies
    ev.wait_on_compute()                               # before the kernels that read `slot`
"""
import ctypes as C
from typing import Optional

import numpy as np
import torch

from . import _abi as A


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class PinnedHostBuffer:
    """Page-locked host memory usable with the copy stream of every device (offload.rs:122-213)."""

    def __init__(self, nbytes: int):
        h = C.c_void_p()
        A.check(A.lib().b200_pinned_alloc(int(nbytes), C.byref(h)))
        self._h = h

    def __len__(self) -> int:
        return int(A.lib().b200_pinned_len(self._h))

    def wait_idle(self):
        """Blocks until every copy queued on this buffer has completed."""
        A.check(A.lib().b200_pinned_wait_idle(self._h))

    def numpy(self) -> np.ndarray:
        """The bytes as a uint8 array (a view, not a copy), after the copies queued on this buffer completed."""
        n = len(self)
        if n == 0:
            return np.empty(0, np.uint8)
        ptr = A.lib().b200_pinned_ptr(self._h)
        if not ptr:
            A.check(A.ERR_LAUNCH)
        return np.ctypeslib.as_array((C.c_uint8 * n).from_address(ptr))

    def close(self):
        if self._h is not None and self._h.value:
            A.lib().b200_pinned_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class CopyEvent:
    """Completion of a copy queued on a `CopyStream` (offload.rs:215-266)."""

    def __init__(self, handle, device, keep):
        self._h, self.device, self._keep = handle, device, keep

    def wait_on_compute(self):
        """The current stream of the device waits (on the GPU) for the copy: work queued afterwards sees the uploaded
        bytes and may overwrite or free the source of a download."""
        A.check(A.lib().b200_copy_event_wait_on_compute(self._h, _stream(self.device)))

    def synchronize(self):
        """Blocks the calling thread until the copy completed."""
        A.check(A.lib().b200_copy_event_synchronize(self._h))

    def is_complete(self) -> bool:
        return bool(A.lib().b200_copy_event_is_complete(self._h))

    def close(self):
        if self._h is not None:
            with torch.cuda.device(self.device):
                A.lib().b200_copy_event_free(self._h, _stream(self.device))
            self._h, self._keep = None, None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _bytes_of(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


class CopyStream:
    """The copy stream of a device: all instances for one device share one stream, so copies run in issue order
    (offload.rs:268-426)."""

    def __init__(self, device="cuda"):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("copy stream: a CUDA device is needed (no CPU path)")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())

    def _check(self, t: torch.Tensor, what: str):
        if not t.is_cuda or t.device != self.device:
            raise ValueError(f"copy stream: the {what} lives on another device than the copy stream")
        if not t.is_contiguous():
            raise ValueError(f"copy stream: the {what} must be contiguous")

    def upload(self, src: PinnedHostBuffer, src_off: int, dst: torch.Tensor, dst_off: int, nbytes: int) -> CopyEvent:
        """Queues the copy of `src[src_off : src_off + nbytes]` into `dst` at byte offset `dst_off`; it starts after the
        work queued so far on the device's current stream. Wait for the returned event on the compute stream before
        reading `dst`."""
        self._check(dst, "destination")
        ev = C.c_void_p()
        with torch.cuda.device(self.device):
            A.check(A.lib().b200_copy_upload(src._h, int(src_off), dst.data_ptr(), _bytes_of(dst), int(dst_off), int(nbytes),
                                             _stream(self.device), C.byref(ev)))
        return CopyEvent(ev, self.device, (src, dst))

    def download(self, src: torch.Tensor, src_off: int, dst: PinnedHostBuffer, dst_off: int, nbytes: int) -> CopyEvent:
        """Queues the copy of `nbytes` bytes of `src` from byte offset `src_off` into `dst[dst_off : ...]`; it starts after
        the work queued so far on the device's current stream (it sees the results of earlier kernels). Read `dst` after
        `CopyEvent.synchronize()` or through `PinnedHostBuffer.numpy()`, which waits."""
        self._check(src, "source")
        ev = C.c_void_p()
        with torch.cuda.device(self.device):
            A.check(A.lib().b200_copy_download(src.data_ptr(), _bytes_of(src), int(src_off), dst._h, int(dst_off), int(nbytes),
                                               _stream(self.device), C.byref(ev)))
        return CopyEvent(ev, self.device, (src, dst))

    def synchronize(self):
        with torch.cuda.device(self.device):
            A.check(A.lib().b200_copy_stream_synchronize())
