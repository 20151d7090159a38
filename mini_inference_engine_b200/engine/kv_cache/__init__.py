"""KV-cache operators of the hot path, under the reference's names."""

from .decode_metadata import validate_decode_metadata
from .triton_flash_prefill import triton_flash_prefill_attention
from .triton_packed_attention import can_use_triton_packed_prefill, triton_packed_prefill_attention
from .triton_packed_kv import can_use_triton_packed_kv_write, triton_write_packed_kv
from .triton_paged_attention import (
    SPLIT_KV_BLOCK_TOKENS,
    can_use_triton_paged_decode,
    select_decode_block_tokens,
    select_decode_split_count,
    select_split_kv_decode,
    triton_is_available,
    triton_paged_decode_attention,
)
from .triton_paged_kv import can_use_triton_decode_kv_write, triton_write_decode_kv
from .triton_tc_decode import select_tensor_core_decode, tensor_core_decode_attention

__all__ = [
    "SPLIT_KV_BLOCK_TOKENS",
    "can_use_triton_decode_kv_write",
    "can_use_triton_packed_kv_write",
    "can_use_triton_packed_prefill",
    "can_use_triton_paged_decode",
    "select_decode_block_tokens",
    "select_decode_split_count",
    "select_split_kv_decode",
    "select_tensor_core_decode",
    "tensor_core_decode_attention",
    "triton_flash_prefill_attention",
    "triton_is_available",
    "triton_packed_prefill_attention",
    "triton_paged_decode_attention",
    "triton_write_decode_kv",
    "triton_write_packed_kv",
    "validate_decode_metadata",
]
