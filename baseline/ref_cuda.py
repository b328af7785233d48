"""ctypes binding of baseline/_ref_cuda/libref_cuda.so: the reference's own GPU kernels compiled for sm_100a from its
kernel headers (see ref_cuda.cu), launched with the reference's launch plan. Bench and test infrastructure only.

The plan restated here: heads per workgroup `row_group` (candle-core/src/accel/attention.rs:586-592), key splits
`split_count_grouped` with the Auto policy (:486-506; 64 workgroups per compute unit, one 128-key window per split, 64 keys
for packed workgroups, at most 64 splits), FP8 specialisation when both sides are FP8 rows
(candle-core/src/accel/turbo.rs:537-552)."""
import ctypes as C
import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB = HERE / "_ref_cuda" / "libref_cuda.so"
# the reference tree is expected beside the repository (or where REFERENCE points)
KERNELS = Path(os.environ.get("REFERENCE", HERE.parent.parent / "reference")) / "candle-core" / "kernels"
FA_MAX_SPLITS, SPLIT_WORKGROUPS_PER_CU, THREADS = 64, 64, 128
MODE_FP8 = 5


class RefTqCall(C.Structure):
    _fields_ = [("q", C.c_void_p), ("kd", C.c_void_p), ("vd", C.c_void_p), ("tab", C.c_void_p), ("out", C.c_void_p),
                ("part_o", C.c_void_p), ("part_lse", C.c_void_p),
                ("b", C.c_uint32), ("lq", C.c_uint32), ("lk", C.c_uint32), ("hq", C.c_uint32), ("hkv", C.c_uint32), ("d", C.c_uint32),
                ("k_strides", C.c_uint64 * 3), ("v_strides", C.c_uint64 * 3),
                ("k_side", C.c_uint32 * 4), ("v_side", C.c_uint32 * 4),
                ("scale", C.c_float), ("splits", C.c_uint32), ("group", C.c_uint32), ("fp8", C.c_uint32), ("pad", C.c_uint32)]


def build(kernels: Path = KERNELS) -> bool:
    """Compiles the library where the reference's kernel headers are present; keeps a prebuilt one otherwise."""
    if not (kernels / "turbo_quant_impl.h").is_file():
        return LIB.is_file()
    src = HERE / "ref_cuda.cu"
    if LIB.is_file() and LIB.stat().st_mtime >= max(src.stat().st_mtime, *(p.stat().st_mtime for p in kernels.glob("*.h"))):
        return True
    LIB.parent.mkdir(exist_ok=True)
    subprocess.run(["nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-shared",
                    "-Xcompiler", "-fPIC", f"-I{kernels}", "-o", str(LIB), str(src)], check=True)
    return True


def available() -> bool:
    return LIB.is_file()


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(LIB))
        _lib.refcu_tq_attention.argtypes = [C.POINTER(RefTqCall), C.c_void_p]
        _lib.refcu_tq_attention_many.argtypes = [C.POINTER(RefTqCall), C.c_int, C.c_void_p]
        _lib.refcu_tq_quant.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint64,
                                        C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p]
        _lib.refcu_fa_prefill_bf16.argtypes = [C.c_void_p] * 4 + [C.c_uint32] * 4 + [C.c_float, C.c_void_p]
    return _lib


def row_group(hq, hkv):
    g = hq // max(hkv, 1)
    for c in (8, 4, 2):
        if g >= c and g % c == 0:
            return c
    return 1


def split_count_grouped(rows, group, lk, compute_units):
    group = max(group, 1)
    workgroups = max(rows // group, 1)
    by_occupancy = -(-SPLIT_WORKGROUPS_PER_CU * max(compute_units, 1) // workgroups)
    keys = THREADS // 2 if group > 1 else THREADS
    by_keys = max(-(-lk // keys), 1)
    return max(1, min(by_occupancy, by_keys, FA_MAX_SPLITS))


class TqAttention:
    """The reference's fused attention over packed rows `(b, hkv, cap, row_words)`: one call per entry of `lens` when
    the lengths differ (the reference's cache has one length), one call for the whole batch when they are equal."""

    def __init__(self, torch, q32, kc, vc, lens, k_layout, v_layout, k_mode, v_mode, tab, scale, compute_units):
        b, hq, lq, d = q32.shape
        _, hkv, cap, kw = kc.shape
        vw = vc.shape[3]
        self.out = torch.empty((b, hq, lq, d), dtype=torch.float32, device=q32.device)
        group = row_group(hq, hkv)
        uniform = len(set(int(x) for x in lens)) == 1
        spans = [(0, b, int(lens[0]))] if uniform else [(i, 1, int(lens[i])) for i in range(b)]
        self.calls = (RefTqCall * len(spans))()
        self.keep = [q32, kc, vc, tab]
        self.splits = []
        for c, (b0, nb, lk) in zip(self.calls, spans):
            rows = nb * hq * lq
            splits = split_count_grouped(rows, group, lk, compute_units)
            self.splits.append(splits)
            po = torch.empty(splits * rows * d, dtype=torch.float32, device=q32.device) if splits > 1 else None
            pl = torch.empty(splits * rows, dtype=torch.float32, device=q32.device) if splits > 1 else None
            self.keep += [po, pl]
            c.q, c.kd, c.vd = q32[b0].data_ptr(), kc[b0].data_ptr(), vc[b0].data_ptr()
            c.tab, c.out = tab.data_ptr(), self.out[b0].data_ptr()
            c.part_o, c.part_lse = (po.data_ptr(), pl.data_ptr()) if splits > 1 else (None, None)
            c.b, c.lq, c.lk, c.hq, c.hkv, c.d = nb, lq, lk, hq, hkv, d
            c.k_strides[:] = [hkv * cap * kw, cap * kw, kw]
            c.v_strides[:] = [hkv * cap * vw, cap * vw, vw]
            c.k_side[:] = [k_mode, k_layout.code_bits, k_layout.code_words, k_layout.rsc_offset]
            c.v_side[:] = [v_mode, v_layout.code_bits, v_layout.code_words, v_layout.rsc_offset]
            c.scale, c.splits, c.group = scale, splits, group
            c.fp8 = 1 if (k_mode == MODE_FP8 and v_mode == MODE_FP8) else 0
        self.launches = sum(2 if s > 1 else 1 for s in self.splits)
        self.group = group

    def run(self, stream):
        rc = lib().refcu_tq_attention_many(self.calls, len(self.calls), stream)
        if rc:
            raise RuntimeError(f"reference kernels: launch failed ({rc})")
        return self.out
