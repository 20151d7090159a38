"""Packed-prefill KV-cache writer (reference: engine/kv_cache/triton_packed_kv.py:113-208).

Row ``t`` of the packed K/V states lands in slot
``block_tables[token_to_sequence[t], pos // page] * page + pos % page`` with
``pos = token_positions[t]``: the reference's slot mapping.  The copy is
``mie_write_packed_kv`` in ``csrc/kv_scatter.cu``.
"""

from __future__ import annotations

import torch

from ... import _lib
from .triton_paged_kv import triton_is_available


def can_use_triton_packed_kv_write(
    key_states: torch.Tensor,
    value_states: torch.Tensor,
    token_to_sequence: torch.Tensor,
    token_positions: torch.Tensor,
    block_tables: torch.Tensor,
    key_blocks: torch.Tensor,
    value_blocks: torch.Tensor,
) -> bool:
    """Shape/device contract of the packed writer (triton_packed_kv.py:113-143)."""

    tensors = (key_states, value_states, token_to_sequence, token_positions, block_tables, key_blocks, value_blocks)
    if not all(t.is_cuda for t in tensors) or not triton_is_available():
        return False
    return bool(
        key_states.ndim == 4
        and value_states.shape == key_states.shape
        and key_states.shape[0] == 1
        and key_states.dtype == value_states.dtype == key_blocks.dtype == value_blocks.dtype
        and key_states.dtype in _lib.DTYPE_CODES
        and token_to_sequence.ndim == 1
        and token_positions.ndim == 1
        and token_to_sequence.shape == token_positions.shape
        and block_tables.ndim == 2
        and key_blocks.ndim == 4
        and key_blocks.shape == value_blocks.shape
    )


def triton_write_packed_kv(
    key_states: torch.Tensor,
    value_states: torch.Tensor,
    token_to_sequence: torch.Tensor,
    token_positions: torch.Tensor,
    block_tables: torch.Tensor,
    key_blocks: torch.Tensor,
    value_blocks: torch.Tensor,
) -> None:
    """Scatter flat current-layer K/V rows into their physical pages."""

    if not can_use_triton_packed_kv_write(
        key_states, value_states, token_to_sequence, token_positions, block_tables, key_blocks, value_blocks
    ):
        raise ValueError("inputs do not satisfy the Triton packed K/V write contract")
    if int(key_states.shape[2]) != int(token_to_sequence.shape[0]):
        raise ValueError("packed K/V token count must match token metadata")
    if int(key_states.shape[1]) != int(key_blocks.shape[1]):
        raise ValueError("packed K/V head count must match the cache")
    if int(key_states.shape[3]) != int(key_blocks.shape[3]):
        raise ValueError("packed K/V head_dim must match the cache")
    _, kv_heads, tokens, head_dim = (int(v) for v in key_states.shape)
    num_blocks, _, block_size, _ = (int(v) for v in key_blocks.shape)
    device = key_states.device
    _lib.check(_lib.load().mie_write_packed_kv(
        _lib.view4_arg(key_states), _lib.view4_arg(value_states), _lib.index_arg(token_to_sequence),
        _lib.index_arg(token_positions), _lib.index_arg(block_tables),
        _lib.view4_arg(key_blocks), _lib.view4_arg(value_blocks),
        tokens, kv_heads, head_dim, block_size, num_blocks,
        int(block_tables.shape[0]), int(block_tables.shape[1]),
        key_states.element_size(), _lib.ptr(_lib.status_word(device)), _lib.stream_arg(device),
    ))


__all__ = ["can_use_triton_packed_kv_write", "triton_is_available", "triton_write_packed_kv"]
