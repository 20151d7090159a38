"""One-token KV-cache writer (reference: engine/kv_cache/triton_paged_kv.py:116-223).

The module keeps the reference's name so importers need no change; there is
no Triton here.  The copy itself is ``mie_write_decode_kv`` in
``csrc/kv_scatter.cu``.
"""

from __future__ import annotations

import torch

from ... import _lib
from .decode_metadata import validate_decode_metadata


def triton_is_available() -> bool:
    """Whether the CUDA library and a CUDA device are usable (name kept from the reference)."""

    if not torch.cuda.is_available():
        return False
    _lib.load()  # a missing library on a GPU box is an error, not a reason to fall back
    return True


def can_use_triton_decode_kv_write(
    key_states: torch.Tensor,
    value_states: torch.Tensor,
    block_tables: torch.Tensor | None,
    sequence_lengths: torch.Tensor | None,
    key_blocks: torch.Tensor,
    value_blocks: torch.Tensor,
) -> bool:
    """Shape/device contract of the one-token writer (triton_paged_kv.py:116-151)."""

    tensors = (key_states, value_states, key_blocks, value_blocks, block_tables, sequence_lengths)
    if any(t is None for t in tensors) or not all(t.is_cuda for t in tensors):
        return False
    if len({t.device for t in tensors}) != 1 or not triton_is_available():
        return False
    return bool(
        key_states.ndim == 4
        and key_blocks.ndim == value_blocks.ndim == 4
        and key_blocks.shape == value_blocks.shape
        and value_states.shape == key_states.shape
        and key_states.shape[2] == 1
        and key_states.dtype == value_states.dtype == key_blocks.dtype == value_blocks.dtype
        and key_states.dtype in _lib.DTYPE_CODES
        and block_tables.ndim == 2
        and sequence_lengths.ndim == 1
        and key_states.shape[0] == block_tables.shape[0] == sequence_lengths.shape[0]
        and key_states.shape[1] == key_blocks.shape[1]
        and key_states.shape[3] == key_blocks.shape[3]
        and 1 <= key_blocks.shape[2] <= 128
    )


def triton_write_decode_kv(
    key_states: torch.Tensor,
    value_states: torch.Tensor,
    block_tables: torch.Tensor,
    sequence_lengths: torch.Tensor,
    key_blocks: torch.Tensor,
    value_blocks: torch.Tensor,
    *,
    query_start_positions: torch.Tensor | None = None,
    _validate_metadata: bool = True,
) -> None:
    """Write each request's new K/V row at its explicit position, or at the KV tail."""

    if not can_use_triton_decode_kv_write(
        key_states, value_states, block_tables, sequence_lengths, key_blocks, value_blocks
    ):
        raise ValueError("inputs do not satisfy the Triton decode KV-write contract")
    batch, kv_heads, _, head_dim = (int(v) for v in key_states.shape)
    num_blocks, _, block_size, _ = (int(v) for v in key_blocks.shape)
    if _validate_metadata:
        validate_decode_metadata(
            block_tables, sequence_lengths, device=key_states.device, batch_size=batch,
            num_blocks=num_blocks, block_size=block_size, query_positions=query_start_positions,
        )
    device = key_states.device
    _lib.check(_lib.load().mie_write_decode_kv(
        _lib.view4_arg(key_states), _lib.view4_arg(value_states), _lib.index_arg(block_tables),
        _lib.index_arg(sequence_lengths), _lib.index_arg(query_start_positions),
        _lib.view4_arg(key_blocks), _lib.view4_arg(value_blocks),
        batch, kv_heads, head_dim, block_size, num_blocks, int(block_tables.shape[1]),
        key_states.element_size(), _lib.ptr(_lib.status_word(device)), _lib.stream_arg(device),
    ))


__all__ = ["can_use_triton_decode_kv_write", "triton_is_available", "triton_write_decode_kv"]
