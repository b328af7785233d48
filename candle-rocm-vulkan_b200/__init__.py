"""B200-native fused attention over a compressed KV cache (drop-in for the quantized-KV attention
path of Qntology/candle-rocm-vulkan).

`csrc/` holds the CUDA kernels and the C ABI (include/b200attn.h, built into libb200attn.so);
`turbo_quant` mirrors the reference's host API on top of it. The directory name carries a hyphen,
so load it with `__graft_entry__.load_package()`, which registers it as `candle_rocm_vulkan_b200`.
"""
from . import _abi  # noqa: F401
from . import config  # noqa: F401
from . import flash_attn  # noqa: F401
from . import offload  # noqa: F401
from .offload import CopyEvent, CopyStream, PinnedHostBuffer  # noqa: F401
from .turbo_quant import (FlashAttnConfig, KvBlockRef, OutputGather, PackedAttention, PackedBlocksAttention, QuantFormat,  # noqa: F401
                          QuantizedTensor, TurboKvCache, TurboQuantizer, attention_packed, attention_packed_blocks)
