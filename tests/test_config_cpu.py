"""The switch layer (candle-core/src/accel/{config,profile}.rs): parsers, environment, per-architecture formats. The
expected values are those of the reference's own unit tests (config.rs:509-536, profile.rs:250-343)."""
import pytest

import __graft_entry__ as G


@pytest.fixture(scope="module")
def cfg():
    G.build()
    return G.load_package().config


def test_parse_versions(cfg):
    assert cfg.parse_version("auto") is None
    assert cfg.parse_version("2") == "v2"
    assert cfg.parse_version("FA3") == "v3"
    assert cfg.parse_version("flash-attention1") == "v1"
    assert cfg.parse_version("v4") == "v3"
    with pytest.raises(ValueError):
        cfg.parse_version("7")


def test_parse_switches(cfg):
    assert cfg.parse_split_kv("off") == "off"
    assert cfg.parse_split_kv("8") == 8
    # "1" and "0" are read as on / off before they are read as numbers (config.rs:91-93)
    assert cfg.parse_split_kv("1") == "auto" and cfg.parse_split_kv("0") == "off"
    assert cfg.parse_split_kv("200") == 64 and cfg.parse_split_kv("on") == "auto"
    b = cfg.parse_backends("rocm,vulkan")
    assert "rocm" in b and "vulkan" in b and "cuda" not in b and "cpu" not in b
    assert cfg.parse_backends("all") == frozenset(cfg.BACKENDS) and cfg.parse_backends("none") == frozenset()
    with pytest.raises(ValueError):
        cfg.parse_backends("cuda,tpu")
    assert cfg.parse_rotation("none") == "none" and cfg.parse_rotation("WHT") == "hadamard"
    assert cfg.resolve_rotation("auto", 128) == "hadamard"
    assert cfg.resolve_rotation("auto", 96) == "dense"
    assert cfg.resolve_rotation("hadamard", 96) == "dense" and cfg.resolve_rotation("none", 96) == "none"


def test_dispatch_tables(cfg):
    A = G.load_package()._abi
    P = cfg.AccelProfile
    assert P.cuda(7, 5, 64 << 10, 40).flash_attn_version == "v1"
    assert P.cuda(8, 6, 99 << 10, 80).flash_attn_version == "v2"
    h100 = P.cuda(9, 0, 227 << 10, 132)
    assert h100.flash_attn_version == "v3" and h100.native_fp8 and not h100.native_fp4
    b200 = P.cuda(10, 0, 227 << 10, 148)
    assert b200.arch == "sm_100" and b200.native_fp4 and b200.native_mx
    assert b200.auto_format(4, False, True) == (A.NVFP4, 4)
    assert b200.auto_format(8, False, True) == (A.MXFP8, 8)
    assert b200.auto_format(3, True, True) == (A.TURBO_PROD, 3) and b200.auto_format(3, True, False) == (A.TURBO_MSE, 3)
    assert P.cuda(12, 0, 99 << 10, 84).flash_attn_version == "v2"
    assert h100.auto_format(8, True, True) == (A.FP8_ROW, 8) and h100.auto_format(4, True, True) == (A.TURBO_PROD, 4)


def test_turbo_resolution(cfg):
    A = G.load_package()._abi
    p = cfg.AccelProfile.cuda(8, 6, 99 << 10, 80)  # no native FP4: the codebook formats, like the reference's gfx1100 case
    o = cfg.TurboQuantOptions()
    assert p.turbo_formats(o) == ((A.TURBO_MSE, 4), (A.TURBO_MSE, 4))
    o = cfg.TurboQuantOptions(qjl=True)
    assert p.turbo_formats(o) == ((A.TURBO_PROD, 4), (A.TURBO_MSE, 4))
    o = cfg.TurboQuantOptions(qjl=False, key_bits=3)
    assert p.turbo_formats(o)[0] == (A.TURBO_MSE, 3)
    o = cfg.TurboQuantOptions(key_format=(A.NVFP4, 4), value_format=(A.TURBO_PROD, 3))
    assert p.turbo_formats(o) == ((A.NVFP4, 4), (A.TURBO_MSE, 3))  # values never use the QJL stage
    # a B200 picks NVFP4 at 4 bits and MXFP8 at 8
    b200 = cfg.AccelProfile.cuda(10, 0, 227 << 10, 148)
    assert b200.turbo_formats(cfg.TurboQuantOptions()) == ((A.NVFP4, 4), (A.NVFP4, 4))
    assert b200.turbo_formats(cfg.TurboQuantOptions(key_bits=8, value_bits=8)) == ((A.MXFP8, 8), (A.MXFP8, 8))


def test_environment_layer(cfg, capsys):
    A = G.load_package()._abi
    env = {"CANDLE_FLASH_ATTN": "off", "CANDLE_FLASH_ATTN_VERSION": "fa2", "CANDLE_FLASH_ATTN_SPLIT_KV": "16",
           "CANDLE_FLASH_ATTN_GQA": "no", "CANDLE_FLASH_ATTN_BACKENDS": "cuda",
           "CANDLE_TURBO_QUANT_FORMAT": "mxfp4", "CANDLE_TURBO_QUANT_V_FORMAT": "turbo3", "CANDLE_TURBO_QUANT_BITS": "5",
           "CANDLE_TURBO_QUANT_K_BITS": "2", "CANDLE_TURBO_QUANT_ROTATION": "none", "CANDLE_TURBO_QUANT_QJL": "yes",
           "CANDLE_TURBO_QUANT_SEED": "7", "CANDLE_TURBO_QUANT_FP8_FAST": "maybe", "CANDLE_TURBO_QUANT_DEBUG": " "}
    c = cfg.AccelConfig.from_env(env)
    fa, tq = c.flash_attn, c.turbo_quant
    assert (fa.enabled, fa.version, fa.split_kv, fa.gqa_decode, fa.backends) == (False, "v2", 16, False, frozenset({"cuda"}))
    assert tq.key_format == (A.MXFP4, 4) and tq.value_format == (A.TURBO_MSE, 3)
    assert (tq.key_bits, tq.value_bits, tq.rotation, tq.qjl, tq.seed) == (2, 5, "none", True, 7)
    assert tq.fp8_fast_path is True and tq.debug is False      # an unparsable value and a blank one are ignored
    assert "CANDLE_TURBO_QUANT_FP8_FAST" in capsys.readouterr().err
    assert not c.flash_attn_allowed("cuda") and c.turbo_quant_kernels_allowed("cuda") and not c.turbo_quant_kernels_allowed("metal")
    with pytest.raises(ValueError):
        cfg.parse_format("turbo7")
    assert cfg.parse_format("auto") is None and cfg.parse_format("E4M3") == (A.FP8_ROW, 8) and cfg.parse_format("prod") == (A.TURBO_PROD, 0)


def test_process_wide_configuration(cfg):
    cfg.reset_config()
    base = cfg.config()
    cfg.update_config(lambda c: setattr(c.flash_attn, "version", "v2"))
    assert cfg.config().flash_attn.version == "v2" and base.flash_attn.version is None  # config() hands out copies
    c = cfg.config()
    c.turbo_quant.qjl = True
    assert cfg.config().turbo_quant.qjl is False
    cfg.set_config(c)
    assert cfg.config().turbo_quant.qjl is True
    cfg.reset_config()
    assert cfg.config().flash_attn.version is None and cfg.config().turbo_quant.qjl is False
