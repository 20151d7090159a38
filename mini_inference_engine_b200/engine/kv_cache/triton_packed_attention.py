"""Packed whole-prompt prefill attention addressed by per-token metadata
(reference: engine/kv_cache/triton_packed_attention.py:156-259).

The reference runs one Triton program per (token, head) and re-reads K/V for every
token; here the per-token metadata is folded into per-request ``cu_seqlens`` /
``kv_lens`` on the device (no host read) and the tiled kernel of
``triton_flash_prefill`` does the work.  Rows must be packed request by request
in position order, which is how every caller of the reference builds them
(engine/kv_cache/packed.py:89).
"""

from __future__ import annotations

import torch

from ... import _lib
from .triton_flash_prefill import triton_flash_prefill_attention
from .triton_paged_kv import triton_is_available


def can_use_triton_packed_prefill(
    query: torch.Tensor,
    key_blocks: torch.Tensor,
    value_blocks: torch.Tensor,
    token_to_sequence: torch.Tensor,
    token_positions: torch.Tensor,
    block_tables: torch.Tensor,
) -> bool:
    """Device/shape contract (triton_packed_attention.py:156-183)."""

    tensors = (query, key_blocks, value_blocks, token_to_sequence, token_positions, block_tables)
    if not all(t.is_cuda for t in tensors) or not triton_is_available():
        return False
    return bool(
        query.ndim == 3
        and query.dtype in _lib.DTYPE_CODES
        and key_blocks.dtype == value_blocks.dtype == query.dtype
        and token_to_sequence.ndim == 1
        and token_positions.ndim == 1
        and token_to_sequence.shape[0] == token_positions.shape[0] == query.shape[0]
        and block_tables.ndim == 2
    )


def triton_packed_prefill_attention(
    query: torch.Tensor,
    key_blocks: torch.Tensor,
    value_blocks: torch.Tensor,
    token_to_sequence: torch.Tensor,
    token_positions: torch.Tensor,
    block_tables: torch.Tensor,
    *,
    scale: float,
) -> torch.Tensor:
    """Causal varlen attention for flat ``[tokens, heads, dim]`` Q; row ``t`` sees keys ``0..position[t]``."""

    if not can_use_triton_packed_prefill(query, key_blocks, value_blocks, token_to_sequence, token_positions,
                                         block_tables):
        raise ValueError("inputs do not satisfy the Triton packed-prefill contract")
    if key_blocks.shape != value_blocks.shape:
        raise ValueError("key and value page tensors must have identical shapes")
    total_tokens, num_heads, _ = (int(v) for v in query.shape)
    requests = int(block_tables.shape[0])
    if requests < 1:
        raise ValueError("block_tables must contain at least one request")
    if num_heads % int(key_blocks.shape[1]) != 0:
        raise ValueError("query heads must be divisible by KV heads")
    if not 1 <= int(key_blocks.shape[2]) <= 128:
        raise ValueError("Triton packed prefill supports block sizes from 1 to 128")
    if total_tokens < 1:
        raise ValueError("packed prefill requires at least one token")
    sequences = token_to_sequence.long()
    counts = torch.zeros(requests, dtype=torch.int64, device=query.device)
    counts.scatter_add_(0, sequences, torch.ones_like(sequences))
    cu_seqlens = torch.zeros(requests + 1, dtype=torch.int32, device=query.device)
    cu_seqlens[1:] = counts.cumsum(0)
    kv_lens = torch.zeros(requests, dtype=torch.int64, device=query.device)
    kv_lens.scatter_reduce_(0, sequences, token_positions.long() + 1, reduce="amax")
    return triton_flash_prefill_attention(query, key_blocks, value_blocks, block_tables, cu_seqlens,
                                          kv_lens.to(torch.int32), max_query_len=total_tokens, scale=scale)


__all__ = ["can_use_triton_packed_prefill", "triton_is_available", "triton_packed_prefill_attention"]
