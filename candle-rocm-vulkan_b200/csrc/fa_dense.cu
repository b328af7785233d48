// Attention over dense (uncompressed) K / V: placeholder entry points until the kernels land.
#include "common.cuh"

using namespace b200;

extern "C" size_t b200_flash_attn_workspace_bytes(const B200FaArgs *) { return 0; }

extern "C" int b200_flash_attn(const B200FaArgs *, b200_stream_t) {
    return set_error(B200_ERR_UNSUPPORTED_SHAPE, "flash_attn: dense K/V kernels are not built yet");
}

extern "C" int b200_fa_prefill_append(const B200FaArgs *, const B200KvAppendArgs *, b200_stream_t) {
    return set_error(B200_ERR_UNSUPPORTED_SHAPE, "fa_prefill_append: dense K/V kernels are not built yet");
}
