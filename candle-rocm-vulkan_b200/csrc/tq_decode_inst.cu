// Instantiations of the decode kernel for one key format (B200_KM is given on the command line so
// that the formats compile in parallel).
#include "tq_decode.cuh"

#ifndef B200_KM
#error "define B200_KM (key format id)"
#endif

namespace b200 {

template <int KM, int VM, int HD, bool NAT, bool PAGED>
int launch_decode(const DecodeParams &p, dim3 grid, size_t smem, cudaStream_t stream) {
    auto kern = tq_decode_kernel<KM, VM, HD, NAT, PAGED>;
    static thread_local size_t configured[16] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && configured[dev] < smem) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return set_error(B200_ERR_LAUNCH, "tq_attention: shared memory opt-in of %zu bytes: %s", smem, cudaGetErrorString(e));
        configured[dev] = smem;
    }
    if (p.after_prev) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(DW * 32);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
        if (e != cudaSuccess) return set_error(B200_ERR_LAUNCH, "tq_attention: %s", cudaGetErrorString(e));
        return check_launch("tq_attention");
    }
    kern<<<grid, DW * 32, smem, stream>>>(p);
    return check_launch("tq_attention");
}

#define INST(VM)                                                                                       \
    template int launch_decode<B200_KM, VM, 64, false, false>(const DecodeParams &, dim3, size_t, cudaStream_t);  \
    template int launch_decode<B200_KM, VM, 128, false, false>(const DecodeParams &, dim3, size_t, cudaStream_t); \
    template int launch_decode<B200_KM, VM, 256, false, false>(const DecodeParams &, dim3, size_t, cudaStream_t);

template <int KM, int VM, int HD, bool NAT>
int launch_decode_pair(const DecodeParams &p, dim3 grid, size_t smem, cudaStream_t stream) {
    auto kern = tq_decode_pair_kernel<KM, VM, HD, NAT>;
    static thread_local size_t configured[16] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && configured[dev] < smem) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return set_error(B200_ERR_LAUNCH, "tq_attention: shared memory opt-in of %zu bytes: %s", smem, cudaGetErrorString(e));
        configured[dev] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(PW * 64);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.after_prev ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    if (e != cudaSuccess) return set_error(B200_ERR_LAUNCH, "tq_attention: %s", cudaGetErrorString(e));
    return check_launch("tq_attention");
}

#ifdef B200_ONLY_SAME_FORMAT  // measurement builds only
#if B200_KM == B200_TURBO_MSE
template int launch_decode_pair<B200_KM, B200_KM, 128, true>(const DecodeParams &, dim3, size_t, cudaStream_t);
#endif
#else
INST(B200_TURBO_MSE)
INST(B200_MXFP4)
INST(B200_NVFP4)
INST(B200_MXFP8)
INST(B200_FP8_ROW)
#define INST_PAIR(VM)                                                                                       \
    template int launch_decode_pair<B200_KM, VM, 64, false>(const DecodeParams &, dim3, size_t, cudaStream_t);  \
    template int launch_decode_pair<B200_KM, VM, 128, false>(const DecodeParams &, dim3, size_t, cudaStream_t); \
    template int launch_decode_pair<B200_KM, VM, 256, false>(const DecodeParams &, dim3, size_t, cudaStream_t);
// the pairs of pair_formats()
#if B200_KM == B200_TURBO_MSE
INST_PAIR(B200_TURBO_MSE)
INST_PAIR(B200_MXFP4)
INST_PAIR(B200_NVFP4)
template int launch_decode_pair<B200_KM, B200_KM, 128, true>(const DecodeParams &, dim3, size_t, cudaStream_t);
#elif B200_KM == B200_MXFP4 || B200_KM == B200_NVFP4
INST_PAIR(B200_TURBO_MSE)
#endif
#endif
// rows packed back to back, keys and values in the same format, head dim 128: row strides as compile-time constants
template int launch_decode<B200_KM, B200_KM, 128, true, false>(const DecodeParams &, dim3, size_t, cudaStream_t);
// rows in the blocks of a page table, read where they are: keys and values in the same format
template int launch_decode<B200_KM, B200_KM, 64, false, true>(const DecodeParams &, dim3, size_t, cudaStream_t);
template int launch_decode<B200_KM, B200_KM, 128, false, true>(const DecodeParams &, dim3, size_t, cudaStream_t);
template int launch_decode<B200_KM, B200_KM, 256, false, true>(const DecodeParams &, dim3, size_t, cudaStream_t);

}  // namespace b200
