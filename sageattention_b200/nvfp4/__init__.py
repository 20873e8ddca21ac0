"""Public surface of the NVFP4 attention path, name-for-name with ``sageattention.nvfp4``.

Reference: sageattention/nvfp4/__init__.py:7-36 (the eight public names plus the private
helpers its tests import).
"""

from .flash import (  # noqa: F401
    _NVFP4FlashAttn,
    _gqa_reduce_cast_dkdv,
    _run_bwd,
    _run_bwd_hp,
    nvfp4_flash_attn_func,
    rope_quant_nvfp4,
    vproj_quant_nvfp4,
    _next_mult,
    _quant_nvfp4,
    _quant_nvfp4_dual,
    _resolve_fwd_tiles,
    _run_flash_packed,
    convert_fp32_to_fp4_packed,
    nvfp4_flash_attention,
    nvfp4_flash_attention_packed,
    nvfp4_flash_decode,
    nvfp4_flash_decode_prequant,
    nvfp4_quant_kv_decode,
)
from .kv_cache import NVFP4KVCache  # noqa: F401

__all__ = [
    "nvfp4_flash_attn_func",
    "nvfp4_flash_attention",
    "nvfp4_flash_attention_packed",
    "nvfp4_flash_decode",
    "nvfp4_flash_decode_prequant",
    "nvfp4_quant_kv_decode",
    "NVFP4KVCache",
    "convert_fp32_to_fp4_packed",
]
