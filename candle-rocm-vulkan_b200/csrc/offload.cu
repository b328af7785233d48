// Pinned host buffers and the copy stream of a device: host <-> device transfers of offloaded packed KV blocks
// (host-memory or SSD resident) that run beside the attention kernels.
//
// Same contract as candle-core/src/cuda_backend/offload.rs: a copy is queued on a non-blocking stream of its own
// (one per device, shared by all callers, so copies run in issue order); it starts after the work queued so far on
// the caller's compute stream (the buffer's allocation and the kernels that still use it are ordered there) and
// returns an event; the compute stream waits for that event before it reads uploaded bytes (or overwrites the source
// of a download), the host waits for it before it reads downloaded bytes. A pinned buffer remembers the events of the
// copies queued on it: touching its bytes waits for them, so a staging buffer is never rewritten under a running copy.
// No kernel is involved; the ordering is events only, and every call can be captured in a CUDA graph except the ones
// that block the host.
#include <memory>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace b200 {

struct CopyStreamState {
    cudaStream_t stream = nullptr;
    std::mutex mu;
};
static CopyStreamState g_copy[16];

// the copy stream of the current device (created on first use)
static int copy_stream(cudaStream_t &out, int &dev) {
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return set_error(B200_ERR_LAUNCH, "copy stream: no current device");
    CopyStreamState &c = g_copy[dev];
    std::lock_guard<std::mutex> lock(c.mu);
    if (!c.stream && cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking) != cudaSuccess) {
        c.stream = nullptr;
        return set_error(B200_ERR_LAUNCH, "copy stream: %s", cudaGetErrorString(cudaGetLastError()));
    }
    out = c.stream;
    return B200_OK;
}

struct SharedEvent {
    cudaEvent_t ev = nullptr;
    ~SharedEvent() {
        if (ev) cudaEventDestroy(ev);
    }
};

}  // namespace b200

using namespace b200;

struct B200PinnedBuffer {
    void *ptr = nullptr;
    size_t len = 0;
    std::mutex mu;
    std::vector<std::shared_ptr<SharedEvent>> pending;  // copies queued on this buffer that may still run
};

struct B200CopyEvent {
    std::shared_ptr<SharedEvent> ev;
    bool waited = false;  // the compute stream was told to wait, or the host did
};

static int wait_idle(B200PinnedBuffer *b) {
    std::lock_guard<std::mutex> lock(b->mu);
    for (auto &e : b->pending)
        if (cudaEventSynchronize(e->ev) != cudaSuccess) return set_error(B200_ERR_LAUNCH, "pinned buffer: %s", cudaGetErrorString(cudaGetLastError()));
    b->pending.clear();
    return B200_OK;
}

extern "C" int b200_pinned_alloc(size_t bytes, B200PinnedBuffer **out) {
    if (!out) return set_error(B200_ERR_BAD_ARG, "pinned_alloc: null result pointer");
    *out = nullptr;
    auto *b = new B200PinnedBuffer();
    // portable: usable with the copy streams of every device
    if (bytes && cudaHostAlloc(&b->ptr, bytes, cudaHostAllocPortable) != cudaSuccess) {
        delete b;
        return set_error(B200_ERR_LAUNCH, "pinned_alloc: %zu bytes: %s", bytes, cudaGetErrorString(cudaGetLastError()));
    }
    b->len = bytes;
    *out = b;
    return B200_OK;
}

extern "C" int b200_pinned_free(B200PinnedBuffer *b) {
    if (!b) return B200_OK;
    const int rc = wait_idle(b);  // the DMA engine must not read freed pages
    if (b->ptr) cudaFreeHost(b->ptr);
    delete b;
    return rc;
}

extern "C" size_t b200_pinned_len(const B200PinnedBuffer *b) { return b ? b->len : 0; }

extern "C" int b200_pinned_wait_idle(B200PinnedBuffer *b) {
    if (!b) return set_error(B200_ERR_BAD_ARG, "pinned buffer: null");
    return wait_idle(b);
}

// The bytes, after the copies queued on the buffer have completed.
extern "C" void *b200_pinned_ptr(B200PinnedBuffer *b) {
    if (!b || wait_idle(b)) return nullptr;
    return b->ptr;
}

// the copy stream waits for what is queued on `compute`; then the copy; then the event
static int queue_copy(void *dst, const void *src, size_t bytes, cudaMemcpyKind kind, B200PinnedBuffer *host, cudaStream_t compute,
                      B200CopyEvent **ev_out, const char *what) {
    cudaStream_t cs;
    int dev;
    int rc = copy_stream(cs, dev);
    if (rc) return rc;
    auto after = std::make_shared<SharedEvent>();
    auto done = std::make_shared<SharedEvent>();
    if (cudaEventCreateWithFlags(&after->ev, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&done->ev, cudaEventDisableTiming) != cudaSuccess)
        return set_error(B200_ERR_LAUNCH, "%s: event: %s", what, cudaGetErrorString(cudaGetLastError()));
    // one caller at a time between the wait and the record, so that the event marks this copy
    std::lock_guard<std::mutex> lock(g_copy[dev].mu);
    if (cudaEventRecord(after->ev, compute) != cudaSuccess || cudaStreamWaitEvent(cs, after->ev, 0) != cudaSuccess)
        return set_error(B200_ERR_LAUNCH, "%s: ordering after the compute stream: %s", what, cudaGetErrorString(cudaGetLastError()));
    if (bytes && cudaMemcpyAsync(dst, src, bytes, kind, cs) != cudaSuccess)
        return set_error(B200_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(cudaGetLastError()));
    if (cudaEventRecord(done->ev, cs) != cudaSuccess) return set_error(B200_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(cudaGetLastError()));
    {
        std::lock_guard<std::mutex> hl(host->mu);
        // forget the copies that have finished, remember this one
        auto &p = host->pending;
        for (size_t i = 0; i < p.size();) {
            if (cudaEventQuery(p[i]->ev) == cudaSuccess) {
                p[i] = p.back();
                p.pop_back();
            } else {
                ++i;
            }
        }
        (void)cudaGetLastError();  // cudaErrorNotReady of the queries above is not an error
        p.push_back(done);
    }
    auto *e = new B200CopyEvent();
    e->ev = done;
    *ev_out = e;
    return B200_OK;
}

static bool range_ok(size_t off, size_t bytes, size_t len) { return off <= len && bytes <= len - off; }

extern "C" int b200_copy_upload(B200PinnedBuffer *src, size_t src_off, void *dst, size_t dst_len, size_t dst_off, size_t bytes,
                                b200_stream_t compute, B200CopyEvent **ev) {
    if (!src || !ev || (!dst && bytes)) return set_error(B200_ERR_BAD_ARG, "copy stream upload: null argument");
    *ev = nullptr;
    if (!range_ok(src_off, bytes, src->len))
        return set_error(B200_ERR_BAD_ARG, "copy stream upload: source range %zu+%zu exceeds the %zu byte pinned buffer", src_off, bytes, src->len);
    if (!range_ok(dst_off, bytes, dst_len))
        return set_error(B200_ERR_BAD_ARG, "copy stream upload: destination range %zu+%zu exceeds %zu bytes", dst_off, bytes, dst_len);
    return queue_copy(static_cast<char *>(dst) + dst_off, static_cast<const char *>(src->ptr) + src_off, bytes, cudaMemcpyHostToDevice, src,
                      (cudaStream_t)compute, ev, "copy stream upload");
}

extern "C" int b200_copy_download(const void *src, size_t src_len, size_t src_off, B200PinnedBuffer *dst, size_t dst_off, size_t bytes,
                                  b200_stream_t compute, B200CopyEvent **ev) {
    if (!dst || !ev || (!src && bytes)) return set_error(B200_ERR_BAD_ARG, "copy stream download: null argument");
    *ev = nullptr;
    if (!range_ok(src_off, bytes, src_len))
        return set_error(B200_ERR_BAD_ARG, "copy stream download: source range %zu+%zu exceeds %zu bytes", src_off, bytes, src_len);
    if (!range_ok(dst_off, bytes, dst->len))
        return set_error(B200_ERR_BAD_ARG, "copy stream download: destination range %zu+%zu exceeds the %zu byte pinned buffer", dst_off, bytes,
                         dst->len);
    return queue_copy(static_cast<char *>(dst->ptr) + dst_off, static_cast<const char *>(src) + src_off, bytes, cudaMemcpyDeviceToHost, dst,
                      (cudaStream_t)compute, ev, "copy stream download");
}

extern "C" int b200_copy_event_wait_on_compute(B200CopyEvent *e, b200_stream_t compute) {
    if (!e) return set_error(B200_ERR_BAD_ARG, "copy event: null");
    if (cudaStreamWaitEvent((cudaStream_t)compute, e->ev->ev, 0) != cudaSuccess)
        return set_error(B200_ERR_LAUNCH, "copy event: %s", cudaGetErrorString(cudaGetLastError()));
    e->waited = true;
    return B200_OK;
}

extern "C" int b200_copy_event_synchronize(B200CopyEvent *e) {
    if (!e) return set_error(B200_ERR_BAD_ARG, "copy event: null");
    if (cudaEventSynchronize(e->ev->ev) != cudaSuccess) return set_error(B200_ERR_LAUNCH, "copy event: %s", cudaGetErrorString(cudaGetLastError()));
    e->waited = true;
    return B200_OK;
}

extern "C" int b200_copy_event_is_complete(B200CopyEvent *e) {
    if (!e) return 0;
    const cudaError_t q = cudaEventQuery(e->ev->ev);
    if (q != cudaSuccess) (void)cudaGetLastError();
    return q == cudaSuccess ? 1 : 0;
}

// An event that nobody waited on: the compute stream is made to wait for the copy, which orders the frees and the
// writes issued afterwards (the reference's Drop of CopyEvent does the same).
extern "C" int b200_copy_event_free(B200CopyEvent *e, b200_stream_t compute) {
    if (!e) return B200_OK;
    int rc = B200_OK;
    if (!e->waited && cudaStreamWaitEvent((cudaStream_t)compute, e->ev->ev, 0) != cudaSuccess)
        rc = set_error(B200_ERR_LAUNCH, "copy event: %s", cudaGetErrorString(cudaGetLastError()));
    delete e;
    return rc;
}

extern "C" int b200_copy_stream_synchronize(void) {
    cudaStream_t cs;
    int dev;
    const int rc = copy_stream(cs, dev);
    if (rc) return rc;
    if (cudaStreamSynchronize(cs) != cudaSuccess) return set_error(B200_ERR_LAUNCH, "copy stream: %s", cudaGetErrorString(cudaGetLastError()));
    return B200_OK;
}
