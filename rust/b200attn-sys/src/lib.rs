//! `repr(C)` mirror of `include/b200attn.h`, field by field and export by export. Not compiled in the image this
//! library was built in (no Rust toolchain there): the struct sizes and offsets are kept in step with the header by
//! `tests/test_abi_cpu.py`, which checks the ctypes mirror of the same declarations against sizes computed from the
//! header's layout rules; a maintainer runs `cargo test` (the size assertions at the end) once with the toolchain.
#![allow(non_camel_case_types, non_snake_case)]

use std::os::raw::{c_char, c_int, c_void};

pub type b200_stream_t = *mut c_void; // cudaStream_t

pub const B200_OK: c_int = 0;
pub const B200_ERR_BAD_ARG: c_int = -1;
pub const B200_ERR_UNSUPPORTED_SHAPE: c_int = -2;
pub const B200_ERR_LAUNCH: c_int = -3;
pub const B200_ERR_WORKSPACE: c_int = -4;
pub const B200_ERR_DEVICE_WAIT: c_int = -5;

pub const B200_F32: i32 = 0;
pub const B200_F16: i32 = 1;
pub const B200_BF16: i32 = 2;
pub const B200_FP8: i32 = 3;

pub const B200_TURBO_MSE: i32 = 0;
pub const B200_TURBO_PROD: i32 = 1;
pub const B200_MXFP4: i32 = 2;
pub const B200_NVFP4: i32 = 3;
pub const B200_MXFP8: i32 = 4;
pub const B200_FP8_ROW: i32 = 5;

pub const B200_ROT_NONE: i32 = 0;
pub const B200_ROT_HADAMARD: i32 = 1;

pub const B200_KV_AFTER_PREV: u32 = 1;
pub const B200_TQ_AFTER_PREV: u32 = 1;
pub const B200_TQ_INPUTS_FINAL: u32 = 2;
pub const B200_TQ_IN_PLACE: u32 = 4;
pub const B200_TQ_OUTPUTS_FREE: u32 = 8;
pub const B200_STATIC_SCRATCH_BYTES: usize = 8 << 20;

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct B200RowLayout {
    pub dim: i32,
    pub code_bits: i32,
    pub code_words: i32,
    pub aux_words: i32,
    pub row_words: i32,
    pub rsc_offset: i32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct B200Profile {
    pub cc_major: i32,
    pub cc_minor: i32,
    pub sm_count: i32,
    pub max_smem_optin: i32,
    pub total_mem: i64,
    pub name: [c_char; 64],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct B200QuantSide {
    pub mode: i32,
    pub bits: i32,
    pub tab: *const f32,
    pub rotation: i32,
    pub signs: *const f32,
}

#[repr(C)]
pub struct B200TqQuantArgs {
    pub src: *const c_void,
    pub out: *mut u32,
    pub tab: *const f32,
    pub rows: u64,
    pub dim: u32,
    pub src_stride: u64,
    pub out_stride: u64,
    pub src_dtype: i32,
    pub mode: i32,
    pub bits: i32,
}

#[repr(C)]
pub struct B200TqDequantArgs {
    pub data: *const u32,
    pub out: *mut f32,
    pub tab: *const f32,
    pub rows: u64,
    pub dim: u32,
    pub data_stride: u64,
    pub mode: i32,
    pub bits: i32,
    pub zs: *mut f32,
}

#[repr(C)]
pub struct B200TqResidArgs {
    pub src: *const c_void,
    pub data: *const u32,
    pub tab: *const f32,
    pub resid: *mut f32,
    pub rows: u64,
    pub dim: u32,
    pub src_stride: u64,
    pub data_stride: u64,
    pub src_dtype: i32,
    pub bits: i32,
}

#[repr(C)]
pub struct B200TqSignsArgs {
    pub input: *const u32, // `in` in the header
    pub proj: *const f32,
    pub resid: *const f32,
    pub out: *mut u32,
    pub rows: u64,
    pub dim: u32,
    pub bits: i32,
}

#[repr(C)]
pub struct B200KvAppendArgs {
    pub k: *const c_void,
    pub v: *const c_void,
    pub k_strides: [u64; 3],
    pub v_strides: [u64; 3],
    pub k_cache: *mut u32,
    pub v_cache: *mut u32,
    pub k_cache_strides: [u64; 3],
    pub v_cache_strides: [u64; 3],
    pub pos: *const i32,
    pub pos0: i32,
    pub b: u32,
    pub hkv: u32,
    pub t: u32,
    pub d: u32,
    pub src_dtype: i32,
    pub kq: B200QuantSide,
    pub vq: B200QuantSide,
    pub cap: u32,
    pub status: *mut i32,
    pub flags: u32,
    pub pad: u32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct B200Page {
    pub k: *const c_void,
    pub v: *const c_void,
    pub rows: u32,
    pub k_cap: u32,
    pub v_cap: u32,
    pub pad: u32,
}

#[repr(C)]
pub struct B200TqAttnArgs {
    pub q: *const c_void,
    pub out: *mut c_void,
    pub q_dtype: i32,
    pub out_dtype: i32,
    pub q_strides: [u64; 3],
    pub out_strides: [u64; 3],
    pub k_rows: *const u32,
    pub v_rows: *const u32,
    pub k_strides: [u64; 3],
    pub v_strides: [u64; 3],
    pub pages: *const B200Page,
    pub n_pages: u32,
    pub kv_len_dev: *const i32,
    pub b: u32,
    pub lq: u32,
    pub lk: u32,
    pub hq: u32,
    pub hkv: u32,
    pub d: u32,
    pub kq: B200QuantSide,
    pub vq: B200QuantSide,
    pub scale: f32,
    pub softcap: f32,
    pub wl: i32,
    pub wr: i32,
    pub alibi: *const f32,
    pub alibi_bstride: u32,
    pub splits: i32,
    pub workspace: *mut c_void,
    pub workspace_bytes: usize,
    pub status: *mut i32,
    pub flags: u32,
    pub kv_len_add: i32,
    pub fresh_rows: u32,
}

#[repr(C)]
pub struct B200PeerGather {
    pub peer_bufs: *const *mut c_void,
    pub peer_flags: *const *mut u32,
    pub world: u32,
    pub rank: u32,
    pub step: *mut u32,
    pub done_ctr: *mut u32,
    pub max_polls: u32,
    pub pad: u32,
}

#[repr(C)]
pub struct B200FaArgs {
    pub q: *const c_void,
    pub k: *const c_void,
    pub v: *const c_void,
    pub o: *mut c_void,
    pub q_dtype: i32,
    pub kv_dtype: i32,
    pub cu_q: *const u32,
    pub cu_k: *const u32,
    pub b: u32,
    pub lq: u32,
    pub lk: u32,
    pub hq: u32,
    pub hkv: u32,
    pub d: u32,
    pub q_strides: [u64; 3],
    pub k_strides: [u64; 3],
    pub v_strides: [u64; 3],
    pub scale: f32,
    pub softcap: f32,
    pub wl: i32,
    pub wr: i32,
    pub k_descale: f32,
    pub v_descale: f32,
    pub alibi: *const f32,
    pub alibi_bstride: u32,
    pub varlen: u32,
    pub total_q: u64,
    pub workspace: *mut c_void,
    pub workspace_bytes: usize,
}

/// Opaque: page-locked host memory (`b200_pinned_*`).
#[repr(C)]
pub struct B200PinnedBuffer {
    _private: [u8; 0],
}
/// Opaque: completion of one queued copy (`b200_copy_event_*`).
#[repr(C)]
pub struct B200CopyEvent {
    _private: [u8; 0],
}

#[link(name = "b200attn")]
extern "C" {
    // host-side tables and plans (candle-core/src/accel/{formats,turbo,attention}.rs)
    pub fn b200_row_layout(mode: c_int, bits: c_int, dim: c_int, out: *mut B200RowLayout) -> c_int;
    pub fn b200_codebook(dim: c_int, bits: c_int, tab: *mut f32) -> c_int;
    pub fn b200_hadamard_signs(dim: c_int, seed: u64, signs: *mut f32) -> c_int;
    pub fn b200_qjl_matrix(dim: c_int, seed: u64, s: *mut f32) -> c_int;
    pub fn b200_row_group(hq: c_int, hkv: c_int) -> c_int;
    pub fn b200_split_count_grouped(rows: i64, group: c_int, lk: i64, compute_units: c_int) -> c_int;
    pub fn b200_describe(device: c_int, out: *mut B200Profile) -> c_int;
    pub fn b200_last_error() -> *const c_char;

    // quantizer (CudaStorage::tq_quantize / tq_residual / tq_signs / tq_dequantize)
    pub fn b200_tq_quantize(args: *const B200TqQuantArgs, stream: b200_stream_t) -> c_int;
    pub fn b200_tq_dequantize(args: *const B200TqDequantArgs, stream: b200_stream_t) -> c_int;
    pub fn b200_tq_residual(args: *const B200TqResidArgs, stream: b200_stream_t) -> c_int;
    pub fn b200_tq_signs(args: *const B200TqSignsArgs, stream: b200_stream_t) -> c_int;
    pub fn b200_tq_rotate(input: *const f32, out: *mut f32, signs: *const f32, rows: u64, dim: u32, inverse: c_int,
                          stream: b200_stream_t) -> c_int;
    pub fn b200_rotation_matrix(dim: c_int, seed: u64, pi: *mut f32) -> c_int;
    pub fn b200_tq_rotate_dense(input: *const f32, out: *mut f32, pi: *const f32, rows: u64, dim: u32, inverse: c_int,
                                stream: b200_stream_t) -> c_int;
    pub fn b200_kv_append(args: *const B200KvAppendArgs, stream: b200_stream_t) -> c_int;

    // attention over packed rows (CudaStorage::tq_attention / tq_attention_paged)
    pub fn b200_tq_attention_workspace_bytes(args: *const B200TqAttnArgs) -> usize;
    pub fn b200_tq_attention(args: *const B200TqAttnArgs, stream: b200_stream_t) -> c_int;
    pub fn b200_tq_attention_static(args: *const B200TqAttnArgs, stream: b200_stream_t) -> c_int;
    pub fn b200_tq_attention_gather(args: *const B200TqAttnArgs, gather: *const B200PeerGather, stream: b200_stream_t) -> c_int;

    // dense attention (CudaStorage::flash_attn / flash_attn_paged) and prefill with the cache write
    pub fn b200_flash_attn_workspace_bytes(args: *const B200FaArgs) -> usize;
    pub fn b200_flash_attn(args: *const B200FaArgs, stream: b200_stream_t) -> c_int;
    pub fn b200_flash_attn_paged_workspace_bytes(args: *const B200FaArgs, n_pages: u32) -> usize;
    pub fn b200_flash_attn_paged(args: *const B200FaArgs, pages: *const B200Page, n_pages: u32, stream: b200_stream_t) -> c_int;
    pub fn b200_fa_prefill_append(fa: *const B200FaArgs, append: *const B200KvAppendArgs, stream: b200_stream_t) -> c_int;

    // health of the bounded device waits
    pub fn b200_device_wait_status() -> c_int;
    pub fn b200_device_wait_check(clear: c_int) -> c_int;

    // offloaded KV blocks (candle-core/src/cuda_backend/offload.rs)
    pub fn b200_pinned_alloc(bytes: usize, out: *mut *mut B200PinnedBuffer) -> c_int;
    pub fn b200_pinned_free(buf: *mut B200PinnedBuffer) -> c_int;
    pub fn b200_pinned_len(buf: *const B200PinnedBuffer) -> usize;
    pub fn b200_pinned_wait_idle(buf: *mut B200PinnedBuffer) -> c_int;
    pub fn b200_pinned_ptr(buf: *mut B200PinnedBuffer) -> *mut c_void;
    pub fn b200_copy_upload(src: *mut B200PinnedBuffer, src_off: usize, dst: *mut c_void, dst_len: usize, dst_off: usize, bytes: usize,
                            compute: b200_stream_t, event: *mut *mut B200CopyEvent) -> c_int;
    pub fn b200_copy_download(src: *const c_void, src_len: usize, src_off: usize, dst: *mut B200PinnedBuffer, dst_off: usize, bytes: usize,
                              compute: b200_stream_t, event: *mut *mut B200CopyEvent) -> c_int;
    pub fn b200_copy_event_wait_on_compute(event: *mut B200CopyEvent, compute: b200_stream_t) -> c_int;
    pub fn b200_copy_event_synchronize(event: *mut B200CopyEvent) -> c_int;
    pub fn b200_copy_event_is_complete(event: *mut B200CopyEvent) -> c_int;
    pub fn b200_copy_event_free(event: *mut B200CopyEvent, compute: b200_stream_t) -> c_int;
    pub fn b200_copy_stream_synchronize() -> c_int;
}

/// The message of the calling thread's last failed call.
pub fn last_error() -> String {
    // SAFETY: the library returns a NUL-terminated thread-local buffer that stays valid until the thread's next call.
    unsafe { std::ffi::CStr::from_ptr(b200_last_error()) }.to_string_lossy().into_owned()
}

#[cfg(test)]
mod tests {
    use super::*;
    use std::mem::size_of;

    // sizes on LP64 (x86-64 and aarch64 Linux), the same numbers tests/test_abi_cpu.py asserts for the ctypes mirror
    #[test]
    fn struct_sizes_match_the_header() {
        assert_eq!(size_of::<B200RowLayout>(), 24);
        assert_eq!(size_of::<B200Profile>(), 88);
        assert_eq!(size_of::<B200QuantSide>(), 32);
        assert_eq!(size_of::<B200Page>(), 32);
        assert_eq!(size_of::<B200PeerGather>(), 48);
    }
}
