"""Switches of the fused attention and TurboQuant paths, and the per-architecture choices that hang on them: the
host-side layer of candle-core/src/accel/{config,profile,mod}.rs (env parsing, `AccelConfig`, `AccelProfile::cuda`,
automatic formats, `describe`). Nothing here reaches the kernels: the C ABI takes plain fields, and a host that binds
the library keeps its own copy of this layer (the reference keeps it on the Rust side of the boundary)."""
import copy
import ctypes as C
import os
import sys
import threading
from dataclasses import dataclass, field
from typing import Optional, Tuple

from . import _abi as A


def parse_bool(s: str) -> Optional[bool]:
    """config.rs:320-326."""
    t = s.strip().lower()
    if t in ("1", "on", "true", "yes", "y", "enable", "enabled"):
        return True
    if t in ("0", "off", "false", "no", "n", "disable", "disabled"):
        return False
    return None


def parse_version(s: str) -> Optional[str]:
    """`1`, `v1`, `fa1`, `flash-attention1`, ... -> "v1" / "v2" / "v3"; `auto` -> None (config.rs:47-64)."""
    t = s.strip().lower().replace("-", "").replace("_", "").replace(" ", "")
    for prefix in ("flashattention", "flashattn", "fa", "v"):
        while prefix and t.startswith(prefix):
            t = t[len(prefix):]
            if prefix != "v":
                break
    if t in ("", "auto", "uto"):
        return None
    if t in ("1", "2"):
        return "v" + t
    if t in ("3", "4"):
        return "v3"
    raise ValueError(f"unknown flash-attention version {s!r} (auto, 1, 2, 3)")


def parse_split_kv(s: str):
    """"auto" | "off" | number of splits (config.rs:86-103)."""
    t = s.strip().lower()
    if t in ("", "auto"):
        return "auto"
    b = parse_bool(t)
    if b is not None:
        return "auto" if b else "off"
    try:
        n = int(t)
    except ValueError:
        raise ValueError(f"invalid split-kv value {s!r} (auto, off, or a number)") from None
    if n < 0:
        raise ValueError(f"invalid split-kv value {s!r} (auto, off, or a number)")
    return "off" if n <= 1 else min(n, 64)


def parse_rotation(s: str) -> str:
    """config.rs:119-129."""
    t = s.strip().lower()
    if t in ("", "auto"):
        return "auto"
    if t in ("hadamard", "had", "wht", "fwht"):
        return "hadamard"
    if t in ("dense", "orthogonal", "qr", "random"):
        return "dense"
    if t in ("none", "off", "0", "false", "no", "identity"):
        return "none"
    raise ValueError(f"unknown rotation {s!r} (auto, hadamard, dense, none)")


def resolve_rotation(kind: str, d: int) -> str:
    """config.rs:131-138."""
    pow2 = d > 0 and d & (d - 1) == 0
    if kind == "auto":
        return "hadamard" if pow2 else "dense"
    if kind == "hadamard" and not pow2:
        return "dense"
    return kind


BACKENDS = ("cuda", "rocm", "vulkan", "cpu", "metal")
_BACKEND_NAMES = {"cuda": "cuda", "nvidia": "cuda", "rocm": "rocm", "hip": "rocm", "amd": "rocm", "vulkan": "vulkan", "vk": "vulkan",
                  "cpu": "cpu", "metal": "metal", "mps": "metal", "apple": "metal"}


def parse_backends(s: str) -> frozenset:
    """`all`, `none`, or a list such as `cuda,rocm` (config.rs:181-201)."""
    t = s.strip().lower()
    if t in ("", "all", "auto"):
        return frozenset(BACKENDS)
    if t in ("none", "off"):
        return frozenset()
    out = set()
    for part in t.replace(";", ",").replace(" ", ",").replace("+", ",").split(","):
        if not part:
            continue
        if part not in _BACKEND_NAMES:
            raise ValueError(f"unknown backend {part!r} in {s!r}")
        out.add(_BACKEND_NAMES[part])
    return frozenset(out)


def parse_bits(s: str) -> int:
    try:
        b = int(s.strip())
    except ValueError:
        b = 0
    if not 1 <= b <= 8:
        raise ValueError(f"expected a bit width in 1..=8, got {s!r}")
    return b


def parse_format(s: str) -> Optional[Tuple[int, int]]:
    """(mode, bits) with bits 0 = not given, None for `auto` (formats.rs:53-96)."""
    t = s.strip().lower().replace("-", "").replace("_", "").replace(" ", "")
    digits = "".join(ch for ch in t if ch.isdigit())
    name = "".join(ch for ch in t if not ch.isdigit())
    if (name == "" and not digits) or name == "auto":
        return None
    bits = int(digits) if digits else 0
    if name in ("turbo", "tq", "mse", "turbomse", "tqmse", "turboquant", "lloydmax"):
        if bits > 4:
            raise ValueError(f"turbo (mse) supports 1-4 bits, got {bits}")
        return (A.TURBO_MSE, bits)
    if name in ("prod", "turboprod", "tqprod", "qjl", "turboqjl"):
        if bits == 1 or bits > 5:
            raise ValueError(f"turbo prod supports 2-5 bits, got {bits}")
        return (A.TURBO_PROD, bits)
    if name == "nvfp" and digits == "4":
        return (A.NVFP4, 4)
    if name == "mxfp" and digits == "4":
        return (A.MXFP4, 4)
    if name == "mxfp" and digits == "8":
        return (A.MXFP8, 8)
    if (name in ("fp", "nvfp") and digits == "8") or (name == "em" and digits == "43"):
        return (A.FP8_ROW, 8)
    raise ValueError(f"unknown quantization format {s!r} (auto, turbo[1-4], prod[2-5], nvfp4, mxfp4, mxfp8, fp8)")


def with_default_bits(f: Tuple[int, int], bits: int) -> Tuple[int, int]:
    """formats.rs:99-109."""
    mode, b = f
    if mode == A.TURBO_MSE and b == 0:
        return (mode, min(max(bits, 1), 4))
    if mode == A.TURBO_PROD and b == 0:
        return (mode, min(max(bits, 2), 5))
    return f


@dataclass
class FlashAttnOptions:
    """config.rs:218-256; the environment variable of each field in `AccelConfig.apply_env`."""
    enabled: bool = True
    version: Optional[str] = None
    split_kv: object = "auto"
    fp8_kv: bool = True
    hadamard: bool = True
    gqa_decode: bool = True
    backends: frozenset = frozenset(BACKENDS)
    debug: bool = False


@dataclass
class TurboQuantOptions:
    """config.rs:258-311."""
    enabled: bool = True
    key_format: Optional[Tuple[int, int]] = None
    value_format: Optional[Tuple[int, int]] = None
    key_bits: int = 4
    value_bits: int = 4
    rotation: str = "auto"
    qjl: bool = False
    fused_attention: bool = True
    fp8_fast_path: bool = True
    seed: int = 42
    backends: frozenset = frozenset(BACKENDS)
    debug: bool = False


def _warn(var, msg):
    print(f"candle accel: ignoring {var}: {msg}", file=sys.stderr)


@dataclass
class AccelConfig:
    flash_attn: FlashAttnOptions = field(default_factory=FlashAttnOptions)
    turbo_quant: TurboQuantOptions = field(default_factory=TurboQuantOptions)

    @classmethod
    def from_env(cls, environ=None) -> "AccelConfig":
        c = cls()
        c.apply_env(environ)
        return c

    def apply_env(self, environ=None):
        """The `CANDLE_FLASH_ATTN*` / `CANDLE_TURBO_QUANT*` variables (config.rs:374-446); a value that does not parse is
        reported on stderr and ignored."""
        environ = os.environ if environ is None else environ

        def env(var):
            v = environ.get(var)
            return v if v is not None and v.strip() else None

        def env_bool(var, obj, name):
            v = env(var)
            if v is not None:
                b = parse_bool(v)
                if b is None:
                    _warn(var, f"expected on/off, got {v!r}")
                else:
                    setattr(obj, name, b)

        def env_parse(var, obj, names, f):
            v = env(var)
            if v is not None:
                try:
                    x = f(v)
                except ValueError as e:
                    _warn(var, str(e))
                    return
                for n in names:
                    setattr(obj, n, x)

        fa, tq = self.flash_attn, self.turbo_quant
        env_bool("CANDLE_FLASH_ATTN", fa, "enabled")
        env_parse("CANDLE_FLASH_ATTN_VERSION", fa, ["version"], parse_version)
        env_parse("CANDLE_FLASH_ATTN_SPLIT_KV", fa, ["split_kv"], parse_split_kv)
        env_bool("CANDLE_FLASH_ATTN_FP8_KV", fa, "fp8_kv")
        env_bool("CANDLE_FLASH_ATTN_HADAMARD", fa, "hadamard")
        env_bool("CANDLE_FLASH_ATTN_GQA", fa, "gqa_decode")
        env_parse("CANDLE_FLASH_ATTN_BACKENDS", fa, ["backends"], parse_backends)
        env_bool("CANDLE_FLASH_ATTN_DEBUG", fa, "debug")
        env_bool("CANDLE_TURBO_QUANT", tq, "enabled")
        env_parse("CANDLE_TURBO_QUANT_FORMAT", tq, ["key_format", "value_format"], parse_format)
        env_parse("CANDLE_TURBO_QUANT_K_FORMAT", tq, ["key_format"], parse_format)
        env_parse("CANDLE_TURBO_QUANT_V_FORMAT", tq, ["value_format"], parse_format)
        env_parse("CANDLE_TURBO_QUANT_BITS", tq, ["key_bits", "value_bits"], parse_bits)
        env_parse("CANDLE_TURBO_QUANT_K_BITS", tq, ["key_bits"], parse_bits)
        env_parse("CANDLE_TURBO_QUANT_V_BITS", tq, ["value_bits"], parse_bits)
        env_parse("CANDLE_TURBO_QUANT_ROTATION", tq, ["rotation"], parse_rotation)
        env_bool("CANDLE_TURBO_QUANT_QJL", tq, "qjl")
        env_bool("CANDLE_TURBO_QUANT_FUSED", tq, "fused_attention")
        env_bool("CANDLE_TURBO_QUANT_FP8_FAST", tq, "fp8_fast_path")

        def seed(s):
            v = int(s.strip())
            if not 0 <= v < 2 ** 64:
                raise ValueError("number too large to fit in target type")
            return v

        env_parse("CANDLE_TURBO_QUANT_SEED", tq, ["seed"], seed)
        env_parse("CANDLE_TURBO_QUANT_BACKENDS", tq, ["backends"], parse_backends)
        env_bool("CANDLE_TURBO_QUANT_DEBUG", tq, "debug")

    def flash_attn_allowed(self, backend: str = "cuda") -> bool:
        return self.flash_attn.enabled and backend in self.flash_attn.backends

    def turbo_quant_kernels_allowed(self, backend: str = "cuda") -> bool:
        return backend in self.turbo_quant.backends and backend != "metal"


_lock = threading.RLock()
_config: Optional[AccelConfig] = None


def config() -> AccelConfig:
    """The current configuration: the environment on first use, then programmatic changes (config.rs:466-478)."""
    global _config
    with _lock:
        if _config is None:
            _config = AccelConfig.from_env()
        return copy.deepcopy(_config)


def set_config(c: AccelConfig):
    global _config
    with _lock:
        _config = copy.deepcopy(c)


def update_config(f):
    """`update_config(lambda c: setattr(c.flash_attn, "version", "v2"))` (config.rs:489-495)."""
    with _lock:
        c = config()
        f(c)
        set_config(c)


def reset_config():
    """Drops programmatic changes; the environment is read again on next use."""
    global _config
    with _lock:
        _config = None


@dataclass
class AccelProfile:
    """What the kernels' dispatch depends on for an NVIDIA GPU (profile.rs:30-94)."""
    backend: str
    arch: str
    flash_attn_version: str
    native_fp8: bool
    native_fp4: bool
    native_mx: bool
    fp4_format: Tuple[int, int]
    fp8_format: Tuple[int, int]
    max_shared_mem: int
    compute_units: int

    @classmethod
    def cuda(cls, major: int, minor: int, max_shared_mem: int, compute_units: int) -> "AccelProfile":
        cc = major * 10 + minor
        version = "v1" if cc < 80 else ("v3" if 90 <= cc < 120 else "v2")
        blackwell = cc >= 100
        return cls("cuda", f"sm_{cc}", version, cc >= 89, blackwell, blackwell, (A.NVFP4, 4),
                   (A.MXFP8, 8) if blackwell else (A.FP8_ROW, 8), max_shared_mem, compute_units)

    def auto_format(self, bits: int, keys: bool, qjl: bool) -> Tuple[int, int]:
        """Native FP4 / FP8 when the GPU has it, else codebooks up to 5 bits and FP8 above (profile.rs:181-193)."""
        if bits >= 6:
            return self.fp8_format
        if bits == 4 and self.native_fp4:
            return self.fp4_format
        if keys and qjl and bits >= 2:
            return (A.TURBO_PROD, min(bits, 5))
        return (A.TURBO_MSE, min(bits, 4))

    def turbo_formats(self, o: TurboQuantOptions):
        """Resolved key and value formats (profile.rs:196-213): values never use the QJL stage, and with QJL off the
        prod format degrades to the codebook of the same width."""
        def resolve(f, bits, keys):
            f = f if f is not None else self.auto_format(bits, keys, o.qjl)
            f = with_default_bits(f, bits)
            if f[0] == A.TURBO_PROD and (not o.qjl or not keys):
                return (A.TURBO_MSE, min(f[1], 4))
            return f
        return resolve(o.key_format, o.key_bits, True), resolve(o.value_format, o.value_bits, False)


def profile(device: int = 0) -> AccelProfile:
    """The profile of a CUDA device, from b200_describe."""
    p = A.Profile()
    A.check(A.lib().b200_describe(int(device), C.byref(p)))
    return AccelProfile.cuda(p.cc_major, p.cc_minor, p.max_smem_optin, p.sm_count)


def format_name(f: Tuple[int, int]) -> str:
    mode, bits = f
    return {A.TURBO_MSE: f"turbo{bits}", A.TURBO_PROD: f"prod{bits}", A.NVFP4: "nvfp4", A.MXFP4: "mxfp4", A.MXFP8: "mxfp8",
            A.FP8_ROW: "fp8"}[mode]


def describe(device: int = 0) -> str:
    """One paragraph for logs: what runs fused on `device`, with which formats (mod.rs:41-99)."""
    c, p = config(), profile(device)
    kf, vf = p.turbo_formats(c.turbo_quant)
    fa_on = c.flash_attn_allowed("cuda")
    tq_k = c.turbo_quant_kernels_allowed("cuda")
    return (f"flash-attn: {'on' if fa_on else 'off'} (version {c.flash_attn.version or p.flash_attn_version}, split-kv {c.flash_attn.split_kv}, "
            f"fp8 kv {c.flash_attn.fp8_kv}, hadamard {c.flash_attn.hadamard}) on {p.arch}, {p.compute_units} SMs, "
            f"{p.max_shared_mem} B shared memory per block\n"
            f"turbo-quant: {'on' if c.turbo_quant.enabled else 'off'} (gpu kernels {tq_k}, k {format_name(kf)}, v {format_name(vf)}, "
            f"rotation {c.turbo_quant.rotation}, fused attention {c.turbo_quant.fused_attention})")
