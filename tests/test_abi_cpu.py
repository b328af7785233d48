"""CPU-side checks of the C ABI: the library loads, exports every declared symbol, and its host-only
helpers agree with the oracle. No kernel is launched here."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import __graft_entry__ as G

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def pkg():
    G.build()
    return G.load_package()


def test_exports_every_declared_symbol(pkg):
    header = (ROOT / "include" / "b200attn.h").read_text()
    declared = set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", header))
    assert declared == set(pkg._abi.SYMBOLS), declared ^ set(pkg._abi.SYMBOLS)
    lib = pkg._abi.lib()
    for s in declared:
        assert hasattr(lib, s), s


def test_struct_sizes_match_header(pkg):
    # a C compiler's view of the header, against the ctypes mirror
    import subprocess, tempfile, os
    A = pkg._abi
    names = {"B200RowLayout": A.RowLayout, "B200Profile": A.Profile, "B200QuantSide": A.QuantSide,
             "B200TqQuantArgs": A.TqQuantArgs, "B200TqDequantArgs": A.TqDequantArgs, "B200KvAppendArgs": A.KvAppendArgs,
             "B200Page": A.Page, "B200TqAttnArgs": A.TqAttnArgs, "B200FaArgs": A.FaArgs, "B200PeerGather": A.PeerGather,
             "B200TqResidArgs": A.TqResidArgs, "B200TqSignsArgs": A.TqSignsArgs}
    src = '#include <stdio.h>\n#include "b200attn.h"\nint main(void){' + "".join(
        f'printf("{n} %zu\\n", sizeof({n}));' for n in names) + "return 0;}"
    with tempfile.TemporaryDirectory() as td:
        c = os.path.join(td, "s.c")
        open(c, "w").write(src)
        subprocess.run(["gcc", "-I", str(ROOT / "include"), c, "-o", os.path.join(td, "s")], check=True)
        out = subprocess.run([os.path.join(td, "s")], check=True, capture_output=True, text=True).stdout
    for line in out.splitlines():
        n, sz = line.split()
        assert C.sizeof(names[n]) == int(sz), n


def test_rust_sys_crate_mirrors_the_header():
    """rust/b200attn-sys/src/lib.rs (not compiled here: no Rust toolchain) against the header, as text: every export,
    every struct with its fields in order, every constant, and the struct sizes its own tests assert."""
    import subprocess, tempfile, os
    header = (ROOT / "include" / "b200attn.h").read_text()
    rust = (ROOT / "rust" / "b200attn-sys" / "src" / "lib.rs").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    assert set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", header)) == set(re.findall(r"pub fn (b200_[a-z0-9_]+)\s*\(", rust))
    for name, value in re.findall(r"#define (B200_[A-Z0-9_]+) \(?(-?\d+)u?\)?\s*$", header, flags=re.M):
        m = re.search(rf"pub const {name}: [a-z_0-9]+ = (-?\d+);", rust)
        assert m and int(m.group(1)) == int(value), name
    rename = {"in": "input"}  # a Rust keyword
    for name, body in re.findall(r"typedef struct (B200\w+) \{(.*?)\} \1;", header, flags=re.S):
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            # "const void *k, *v" / "uint64_t q_strides[3], out_strides[3]" / "char name[64]"
            first, *rest = decl.split(",")
            fields.append(re.findall(r"(\w+)(?:\[\d+\])?$", first.strip())[0])
            fields += [re.findall(r"(\w+)(?:\[\d+\])?$", r.strip())[0] for r in rest]
        m = re.search(rf"pub struct {name} \{{(.*?)\n\}}", rust, flags=re.S)
        assert m, name
        got = re.findall(r"pub (\w+):", m.group(1))
        assert got == [rename.get(f, f) for f in fields], (name, got, fields)
    sizes = dict(re.findall(r"size_of::<(B200\w+)>\(\), (\d+)\)", rust))
    src = '#include <stdio.h>\n#include "b200attn.h"\nint main(void){' + "".join(
        f'printf("{n} %zu\\n", sizeof({n}));' for n in sizes) + "return 0;}"
    with tempfile.TemporaryDirectory() as td:
        c = os.path.join(td, "s.c")
        open(c, "w").write(src)
        subprocess.run(["gcc", "-I", str(ROOT / "include"), c, "-o", os.path.join(td, "s")], check=True)
        out = subprocess.run([os.path.join(td, "s")], check=True, capture_output=True, text=True).stdout
    for line in out.splitlines():
        n, sz = line.split()
        assert int(sizes[n]) == int(sz), n


def test_python_constants_mirror_the_header(pkg):
    """Every B200_* constant of the header that the Python side names (without the prefix) has the header's value."""
    header = re.sub(r"/\*.*?\*/", "", (ROOT / "include" / "b200attn.h").read_text(), flags=re.S)
    defs = {n: int(v) for n, v in re.findall(r"#define B200_([A-Z0-9_]+) \(?(-?\d+)u?\)?\s*$", header, flags=re.M)}
    A = pkg._abi
    seen = 0
    for name, value in defs.items():
        if hasattr(A, name):
            assert getattr(A, name) == value, name
            seen += 1
    for name in ("TQ_AFTER_PREV", "TQ_INPUTS_FINAL", "TQ_IN_PLACE", "TQ_OUTPUTS_FREE", "KV_AFTER_PREV"):
        assert name in defs and getattr(A, name) == defs[name], name
    assert seen >= 10


def test_row_layouts_and_errors(pkg, oracle):
    A = pkg._abi
    for mode in (0, 2, 3, 4, 5):
        for dim in (64, 96, 128, 256, 1024):
            for bits in (1, 2, 3, 4):
                try:
                    want = oracle.row_layout(mode, bits, dim)
                except ValueError:
                    with pytest.raises(A.B200Error):
                        A.row_layout(mode, bits, dim)
                    continue
                got = A.row_layout(mode, bits, dim)
                assert (got.code_bits, got.code_words, got.aux_words, got.row_words, got.rsc_offset) == tuple(
                    want[k] for k in ("code_bits", "code_words", "aux_words", "row_words", "rsc_offset"))
    with pytest.raises(A.B200Error) as e:
        A.row_layout(A.MXFP8, 4, 48)
    assert "multiple of the 32 element block" in str(e.value)
    with pytest.raises(A.B200Error):
        A.row_layout(A.TURBO_MSE, 9, 128)
    with pytest.raises(A.B200Error):
        A.row_layout(A.FP8_ROW, 4, 2048)


def test_codebook_signs_heuristics_match_oracle(pkg, oracle):
    lib = pkg._abi.lib()
    for dim, bits in ((128, 4), (128, 2), (64, 1), (96, 3), (256, 4)):
        tab = (C.c_float * 32)()
        assert lib.b200_codebook(dim, bits, tab) == 0
        assert np.array_equal(np.array(tab, dtype=np.float32).view(np.uint32), oracle.codebook(dim, bits).view(np.uint32))
    for dim, seed in ((128, 42), (128, 44), (64, 7)):
        s = (C.c_float * dim)()
        assert lib.b200_hadamard_signs(dim, seed, s) == 0
        assert np.array_equal(np.array(s, dtype=np.float32), oracle.hadamard_signs(dim, seed))
    assert lib.b200_hadamard_signs(96, 1, (C.c_float * 96)()) != 0
    for hq, hkv in ((32, 8), (64, 8), (6, 2), (8, 8), (16, 1)):
        assert lib.b200_row_group(hq, hkv) == oracle.row_group(hq, hkv)
    for rows, g, lk, cu in ((32, 4, 2048, 148), (256, 8, 32768, 148), (4096, 4, 16384, 148), (16, 1, 100, 16)):
        assert lib.b200_split_count_grouped(rows, g, lk, cu) == oracle.split_count_grouped(rows, g, lk, cu)


def test_dense_rotation_matrix_matches_the_oracle(pkg, oracle):
    """b200_rotation_matrix (Gaussian rows + two passes of modified Gram-Schmidt in f64, turbo.rs:204-229) against the
    oracle's restatement, bit for bit, and orthonormal to f32 precision."""
    lib = pkg._abi.lib()
    for dim, seed in ((96, 42), (80, 7), (33, 2**63 + 5), (192, 44)):
        m = (C.c_float * (dim * dim))()
        assert lib.b200_rotation_matrix(dim, seed, m) == 0
        got = np.frombuffer(m, dtype=np.float32).reshape(dim, dim)
        want = oracle.rotation_matrix(dim, 2, seed)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (dim, seed)
        assert np.abs(got.astype(np.float64) @ got.astype(np.float64).T - np.eye(dim)).max() < 1e-6
    assert lib.b200_rotation_matrix(0, 1, (C.c_float * 1)()) == pkg._abi.ERR_BAD_ARG


def test_argument_errors_without_gpu(pkg):
    A = pkg._abi
    lib = A.lib()
    assert lib.b200_tq_quantize(None, None) == A.ERR_BAD_ARG
    args = A.TqAttnArgs()
    args.hq, args.hkv, args.d = 6, 4, 128
    assert lib.b200_tq_attention(C.byref(args), None) == A.ERR_BAD_ARG
    assert b"not a multiple" in lib.b200_last_error()
    args.hq, args.hkv, args.d = 8, 2, 100
    assert lib.b200_tq_attention(C.byref(args), None) == A.ERR_UNSUPPORTED_SHAPE
    assert lib.b200_tq_attention_workspace_bytes(C.byref(args)) == 0


def test_paged_dense_attention_argument_errors_without_gpu(pkg):
    """The checks of the paged entry points run before anything touches the device (candle-nn/src/flash_attn.rs:650-689,
    candle-flash-attn/src/lib.rs:357-392)."""
    import pytest
    import torch
    F, Ref = pkg.flash_attn, pkg.KvBlockRef
    q = torch.zeros((2, 4, 1, 64))
    kv = lambda b=2, h=2, c=8, d=64: torch.zeros((b, h, c, d))
    with pytest.raises(ValueError, match="no blocks"):
        F.flash_attn_blocks(q, [], pkg.FlashAttnConfig(0.1))
    with pytest.raises(ValueError, match="do not match batch"):
        F.flash_attn_blocks(q, [Ref(kv(), kv(), 4), Ref(kv(b=3), kv(b=3), 4)], pkg.FlashAttnConfig(0.1))
    with pytest.raises(ValueError, match="rows but capacities"):
        F.flash_attn_blocks(q, [Ref(kv(), kv(), 9)], pkg.FlashAttnConfig(0.1))
    with pytest.raises(ValueError, match="hold no keys"):
        F.flash_attn_blocks(q, [Ref(kv(), kv(), 0)], pkg.FlashAttnConfig(0.1))
    with pytest.raises(ValueError, match="head dim"):
        F.flash_attn_blocks(q, [Ref(kv(d=32), kv(d=32), 4)], pkg.FlashAttnConfig(0.1))
    with pytest.raises(RuntimeError, match="CUDA"):  # valid blocks: the call reaches the device check
        F.flash_attn_blocks(q, [Ref(kv(), kv(), 4)], pkg.FlashAttnConfig(0.1))
    pages = torch.zeros((4, 16, 2, 64))
    cu = torch.tensor([0, 20], dtype=torch.int32)
    with pytest.raises(ValueError, match="mm_prefix_ranges"):
        F.flash_attn_varlen_paged_windowed(q, pages, pages, cu, cu, torch.zeros((1, 2), dtype=torch.int32), cu, 1, 20, 0.1, None, None, 16)
    with pytest.raises(ValueError, match="needs 2 blocks"):
        F.flash_attn_varlen_paged_windowed(q, pages, pages, cu, cu, torch.zeros((1, 1), dtype=torch.int32), None, 1, 20, 0.1, None, None, 16)
    with pytest.raises(ValueError, match="rows for 1 sequences"):
        F.flash_attn_varlen_paged_windowed(q, pages, pages, cu, cu, torch.zeros((0, 2), dtype=torch.int32), None, 1, 20, 0.1, None, None, 16)


def test_product_does_not_import_the_oracle():
    for p in (ROOT / "candle-rocm-vulkan_b200").glob("*.py"):
        assert "oracle" not in p.read_text().replace("no CPU path", ""), p
