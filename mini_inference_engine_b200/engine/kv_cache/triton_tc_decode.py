"""Grouped-query decode entry point (reference: engine/kv_cache/triton_tc_decode.py:34-229).

The reference keeps a second, tensor-core Triton kernel for GQA decode; here
both entry points run the same CUDA kernel, which always shares each K/V read
across the query heads of a group.
"""

from __future__ import annotations

import torch

from .triton_paged_attention import launch_decode_attention

TILE_TOKENS = 64
_SMALL_BATCH = 2
_SMALL_BATCH_SPLITS = 4


def select_tensor_core_decode(max_sequence_length: int, batch_size: int) -> tuple[int, int]:
    """``(split_count, tile_tokens)`` the reference measured on the L4 (triton_tc_decode.py:34-45)."""

    if int(batch_size) < 1:
        raise ValueError("batch_size must be positive")
    if int(batch_size) <= _SMALL_BATCH and int(max_sequence_length) >= _SMALL_BATCH_SPLITS * TILE_TOKENS:
        return _SMALL_BATCH_SPLITS, TILE_TOKENS
    return 1, TILE_TOKENS


def tensor_core_decode_attention(
    query: torch.Tensor,
    key_blocks: torch.Tensor,
    value_blocks: torch.Tensor,
    block_tables: torch.Tensor,
    sequence_lengths: torch.Tensor,
    output: torch.Tensor,
    *,
    position_buffer: torch.Tensor,
    has_query_positions: bool,
    scale: float,
    split_count: int,
    split_span: int,
    tile_tokens: int,
) -> None:
    """Write attention into ``output`` (the query's shape); the caller has checked the inputs."""

    del split_count, tile_tokens  # the device picks the split-KV partition
    batch = int(query.shape[0])
    capacity = int(block_tables.shape[1]) * int(key_blocks.shape[2])
    bound = min(capacity, int(split_span) * 8) if split_span < 2**30 else capacity
    launch_decode_attention(
        query, output, key_blocks, value_blocks, block_tables, sequence_lengths,
        position_buffer if has_query_positions else None,
        scale=scale, max_total_tokens=batch * max(bound, 1),
    )


__all__ = ["select_tensor_core_decode", "tensor_core_decode_attention", "TILE_TOKENS"]
