"""ctypes binding of libb200attn.so (declarations: include/b200attn.h).

The structures mirror the C header field by field; nothing here computes. Loading fails loudly
when the library is missing: there is no CPU path behind these calls.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libb200attn.so"

OK, ERR_BAD_ARG, ERR_UNSUPPORTED_SHAPE, ERR_LAUNCH, ERR_WORKSPACE, ERR_DEVICE_WAIT = 0, -1, -2, -3, -4, -5
F32, F16, BF16, FP8 = 0, 1, 2, 3
TURBO_MSE, TURBO_PROD, MXFP4, NVFP4, MXFP8, FP8_ROW = range(6)
ROT_NONE, ROT_HADAMARD = 0, 1
STATIC_SCRATCH_BYTES = 8 << 20

u64x3 = C.c_uint64 * 3


class RowLayout(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("dim", "code_bits", "code_words", "aux_words", "row_words", "rsc_offset")]


class Profile(C.Structure):
    _fields_ = [("cc_major", C.c_int32), ("cc_minor", C.c_int32), ("sm_count", C.c_int32),
                ("max_smem_optin", C.c_int32), ("total_mem", C.c_int64), ("name", C.c_char * 64)]


class QuantSide(C.Structure):
    _fields_ = [("mode", C.c_int32), ("bits", C.c_int32), ("tab", C.c_void_p), ("rotation", C.c_int32),
                ("signs", C.c_void_p)]


class TqQuantArgs(C.Structure):
    _fields_ = [("src", C.c_void_p), ("out", C.c_void_p), ("tab", C.c_void_p), ("rows", C.c_uint64),
                ("dim", C.c_uint32), ("src_stride", C.c_uint64), ("out_stride", C.c_uint64),
                ("src_dtype", C.c_int32), ("mode", C.c_int32), ("bits", C.c_int32)]


class TqDequantArgs(C.Structure):
    _fields_ = [("data", C.c_void_p), ("out", C.c_void_p), ("tab", C.c_void_p), ("rows", C.c_uint64),
                ("dim", C.c_uint32), ("data_stride", C.c_uint64), ("mode", C.c_int32), ("bits", C.c_int32), ("zs", C.c_void_p)]


class TqResidArgs(C.Structure):
    _fields_ = [("src", C.c_void_p), ("data", C.c_void_p), ("tab", C.c_void_p), ("resid", C.c_void_p), ("rows", C.c_uint64),
                ("dim", C.c_uint32), ("src_stride", C.c_uint64), ("data_stride", C.c_uint64), ("src_dtype", C.c_int32),
                ("bits", C.c_int32)]


class TqSignsArgs(C.Structure):
    _fields_ = [("in_", C.c_void_p), ("proj", C.c_void_p), ("resid", C.c_void_p), ("out", C.c_void_p), ("rows", C.c_uint64),
                ("dim", C.c_uint32), ("bits", C.c_int32)]


class KvAppendArgs(C.Structure):
    _fields_ = [("k", C.c_void_p), ("v", C.c_void_p), ("k_strides", u64x3), ("v_strides", u64x3),
                ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("k_cache_strides", u64x3),
                ("v_cache_strides", u64x3), ("pos", C.c_void_p), ("pos0", C.c_int32), ("b", C.c_uint32),
                ("hkv", C.c_uint32), ("t", C.c_uint32), ("d", C.c_uint32), ("src_dtype", C.c_int32),
                ("kq", QuantSide), ("vq", QuantSide), ("cap", C.c_uint32), ("status", C.c_void_p),
                ("flags", C.c_uint32), ("pad", C.c_uint32)]


class Page(C.Structure):
    _fields_ = [("k", C.c_void_p), ("v", C.c_void_p), ("rows", C.c_uint32), ("k_cap", C.c_uint32),
                ("v_cap", C.c_uint32), ("pad", C.c_uint32)]


KV_AFTER_PREV = 1  # B200_KV_AFTER_PREV
TQ_AFTER_PREV = 1  # B200_TQ_AFTER_PREV
TQ_INPUTS_FINAL = 2  # B200_TQ_INPUTS_FINAL
TQ_IN_PLACE = 4  # B200_TQ_IN_PLACE
TQ_OUTPUTS_FREE = 8  # B200_TQ_OUTPUTS_FREE


class TqAttnArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("out", C.c_void_p), ("q_dtype", C.c_int32), ("out_dtype", C.c_int32),
                ("q_strides", u64x3), ("out_strides", u64x3), ("k_rows", C.c_void_p), ("v_rows", C.c_void_p),
                ("k_strides", u64x3), ("v_strides", u64x3), ("pages", C.c_void_p), ("n_pages", C.c_uint32),
                ("kv_len_dev", C.c_void_p), ("b", C.c_uint32), ("lq", C.c_uint32), ("lk", C.c_uint32),
                ("hq", C.c_uint32), ("hkv", C.c_uint32), ("d", C.c_uint32), ("kq", QuantSide), ("vq", QuantSide),
                ("scale", C.c_float), ("softcap", C.c_float), ("wl", C.c_int32), ("wr", C.c_int32),
                ("alibi", C.c_void_p), ("alibi_bstride", C.c_uint32), ("splits", C.c_int32),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("status", C.c_void_p), ("flags", C.c_uint32), ("kv_len_add", C.c_int32),
                ("fresh_rows", C.c_uint32)]


class PeerGather(C.Structure):
    _fields_ = [("peer_bufs", C.c_void_p), ("peer_flags", C.c_void_p), ("world", C.c_uint32), ("rank", C.c_uint32),
                ("step", C.c_void_p), ("done_ctr", C.c_void_p), ("max_polls", C.c_uint32), ("pad", C.c_uint32)]


class FaArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
                ("q_dtype", C.c_int32), ("kv_dtype", C.c_int32), ("cu_q", C.c_void_p), ("cu_k", C.c_void_p),
                ("b", C.c_uint32), ("lq", C.c_uint32), ("lk", C.c_uint32), ("hq", C.c_uint32), ("hkv", C.c_uint32),
                ("d", C.c_uint32), ("q_strides", u64x3), ("k_strides", u64x3), ("v_strides", u64x3),
                ("scale", C.c_float), ("softcap", C.c_float), ("wl", C.c_int32), ("wr", C.c_int32),
                ("k_descale", C.c_float), ("v_descale", C.c_float), ("alibi", C.c_void_p),
                ("alibi_bstride", C.c_uint32), ("varlen", C.c_uint32), ("total_q", C.c_uint64),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


# every symbol that include/b200attn.h declares
SYMBOLS = [
    "b200_row_layout", "b200_codebook", "b200_hadamard_signs", "b200_qjl_matrix", "b200_row_group", "b200_split_count_grouped",
    "b200_tq_residual", "b200_tq_signs", "b200_rotation_matrix", "b200_tq_rotate_dense",
    "b200_describe", "b200_last_error", "b200_tq_rotate", "b200_tq_quantize", "b200_tq_dequantize", "b200_kv_append",
    "b200_tq_attention_workspace_bytes", "b200_tq_attention", "b200_tq_attention_static", "b200_tq_attention_gather",
    "b200_flash_attn_workspace_bytes", "b200_flash_attn_paged_workspace_bytes", "b200_flash_attn_paged",
    "b200_flash_attn", "b200_fa_prefill_append", "b200_device_wait_status", "b200_device_wait_check",
    "b200_pinned_alloc", "b200_pinned_free", "b200_pinned_len", "b200_pinned_wait_idle", "b200_pinned_ptr",
    "b200_copy_upload", "b200_copy_download", "b200_copy_event_wait_on_compute", "b200_copy_event_synchronize",
    "b200_copy_event_is_complete", "b200_copy_event_free", "b200_copy_stream_synchronize",
]

_lib = None


class B200Error(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"b200attn error {code}: {msg}")
        self.code = code


def lib():
    """The loaded library. Raises if it has not been built (run __graft_entry__.build())."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `make -C {HERE / 'csrc'}`; "
                               "there is no CPU fallback for the CUDA kernels")
        l = C.CDLL(str(LIB_PATH))
        l.b200_last_error.restype = C.c_char_p
        l.b200_row_layout.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(RowLayout)]
        l.b200_codebook.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_float)]
        l.b200_hadamard_signs.argtypes = [C.c_int, C.c_uint64, C.POINTER(C.c_float)]
        l.b200_qjl_matrix.argtypes = [C.c_int, C.c_uint64, C.POINTER(C.c_float)]
        l.b200_rotation_matrix.argtypes = [C.c_int, C.c_uint64, C.POINTER(C.c_float)]
        l.b200_tq_rotate_dense.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint32, C.c_int, C.c_void_p]
        l.b200_tq_residual.argtypes = [C.POINTER(TqResidArgs), C.c_void_p]
        l.b200_tq_signs.argtypes = [C.POINTER(TqSignsArgs), C.c_void_p]
        l.b200_row_group.argtypes = [C.c_int, C.c_int]
        l.b200_split_count_grouped.argtypes = [C.c_int64, C.c_int, C.c_int64, C.c_int]
        l.b200_describe.argtypes = [C.c_int, C.POINTER(Profile)]
        l.b200_tq_rotate.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint32, C.c_int, C.c_void_p]
        l.b200_tq_quantize.argtypes = [C.POINTER(TqQuantArgs), C.c_void_p]
        l.b200_tq_dequantize.argtypes = [C.POINTER(TqDequantArgs), C.c_void_p]
        l.b200_kv_append.argtypes = [C.POINTER(KvAppendArgs), C.c_void_p]
        l.b200_tq_attention_workspace_bytes.argtypes = [C.POINTER(TqAttnArgs)]
        l.b200_tq_attention_workspace_bytes.restype = C.c_size_t
        l.b200_tq_attention.argtypes = [C.POINTER(TqAttnArgs), C.c_void_p]
        l.b200_tq_attention_static.argtypes = [C.POINTER(TqAttnArgs), C.c_void_p]
        l.b200_tq_attention_gather.argtypes = [C.POINTER(TqAttnArgs), C.POINTER(PeerGather), C.c_void_p]
        l.b200_flash_attn_workspace_bytes.argtypes = [C.POINTER(FaArgs)]
        l.b200_flash_attn_workspace_bytes.restype = C.c_size_t
        l.b200_flash_attn.argtypes = [C.POINTER(FaArgs), C.c_void_p]
        l.b200_flash_attn_paged_workspace_bytes.argtypes = [C.POINTER(FaArgs), C.c_uint32]
        l.b200_flash_attn_paged_workspace_bytes.restype = C.c_size_t
        l.b200_flash_attn_paged.argtypes = [C.POINTER(FaArgs), C.c_void_p, C.c_uint32, C.c_void_p]
        l.b200_fa_prefill_append.argtypes = [C.POINTER(FaArgs), C.POINTER(KvAppendArgs), C.c_void_p]
        l.b200_device_wait_check.argtypes = [C.c_int]
        l.b200_pinned_alloc.argtypes = [C.c_size_t, C.POINTER(C.c_void_p)]
        l.b200_pinned_free.argtypes = [C.c_void_p]
        l.b200_pinned_len.argtypes = [C.c_void_p]
        l.b200_pinned_len.restype = C.c_size_t
        l.b200_pinned_wait_idle.argtypes = [C.c_void_p]
        l.b200_pinned_ptr.argtypes = [C.c_void_p]
        l.b200_pinned_ptr.restype = C.c_void_p
        l.b200_copy_upload.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.POINTER(C.c_void_p)]
        l.b200_copy_download.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.POINTER(C.c_void_p)]
        l.b200_copy_event_wait_on_compute.argtypes = [C.c_void_p, C.c_void_p]
        l.b200_copy_event_synchronize.argtypes = [C.c_void_p]
        l.b200_copy_event_is_complete.argtypes = [C.c_void_p]
        l.b200_copy_event_free.argtypes = [C.c_void_p, C.c_void_p]
        _lib = l
    return _lib


def check(rc: int):
    if rc != OK:
        raise B200Error(rc, lib().b200_last_error().decode())


def row_layout(mode: int, bits: int, dim: int) -> RowLayout:
    out = RowLayout()
    check(lib().b200_row_layout(mode, bits, dim, C.byref(out)))
    return out
