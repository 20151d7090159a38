"""Ragged one-token paged decode attention
(reference: engine/kv_cache/triton_paged_attention.py:576-985).

Same names and call signatures as the reference module (which is why the file
keeps "triton" in its name); the work is done by ``mie_paged_decode_attention``
in ``csrc/decode_attention.cu``.  The reference's L4 knobs that only pick a
Triton tile (``block_tokens``, ``use_gqa_reuse``) are validated and otherwise
ignored; ``split_count`` keeps its validation rules, but how a context is cut
into split-KV chunks is decided on the device from the batch's real lengths
(``MIE_DECODE_SPLIT_POLICY`` = ``auto`` | ``none`` | a chunk length overrides it).
``sdpa_compat`` (bit-matching the L4's FlashAttention rounding) is accepted
and not emulated: results stay within the 2e-2 bf16 tolerance of the torch
block-wise reference.
"""

from __future__ import annotations

import os

import torch

from ... import _lib
from .decode_metadata import validate_decode_metadata
from .triton_paged_kv import triton_is_available

SPLIT_KV_BLOCK_TOKENS = 64  # the reference's tile for opt-in split-KV on the L4 (kept for importers)

_SPLIT_COUNTS = (1, 2, 4, 8)


def select_decode_split_count(max_sequence_length: int, batch_size: int | None = None) -> int:
    """Split count of a fixed decode-graph shape (triton_paged_attention.py:582-614).

    The values are the reference's L4 table, kept because its callers and
    tests read them; this library's own kernel partitions by length on the device.
    """

    length = int(max_sequence_length)
    batch = None if batch_size is None else int(batch_size)
    if batch is not None and batch < 1:
        raise ValueError("batch_size must be positive")
    if length < 1024:
        return 1
    if length > 4096:
        return 8
    if batch is None:
        return 2 if length <= 2048 else 4
    if length <= 2048:
        return 8 if batch <= 2 else 4 if batch <= 4 else 1
    return 1 if batch >= 8 else 8


def select_split_kv_decode(max_sequence_length: int, batch_size: int) -> int:
    """Opt-in split-KV count, or 1 (triton_paged_attention.py:620-637)."""

    length, batch = int(max_sequence_length), int(batch_size)
    if batch <= 1 and length >= 1024:
        return 8
    if batch <= 2 and length >= 2048:
        return 4
    return 1


def select_decode_block_tokens(max_sequence_length: int) -> int:
    """Token-reduction tile the reference profiled on the L4 (triton_paged_attention.py:640-643)."""

    return 64 if int(max_sequence_length) >= 1024 else 16


def can_use_triton_paged_decode(
    query: torch.Tensor,
    key_blocks: torch.Tensor,
    value_blocks: torch.Tensor,
    block_tables: torch.Tensor | None,
    sequence_lengths: torch.Tensor | None,
) -> bool:
    """Device/shape contract of the decode kernel (triton_paged_attention.py:646-677)."""

    if block_tables is None or sequence_lengths is None:
        return False
    tensors = (query, key_blocks, value_blocks, block_tables, sequence_lengths)
    if not all(t.is_cuda for t in tensors) or len({t.device for t in tensors}) != 1:
        return False
    if not triton_is_available():
        return False
    return bool(
        query.ndim == 4
        and key_blocks.ndim == value_blocks.ndim == 4
        and key_blocks.shape[1] > 0
        and key_blocks.shape[3] == query.shape[3]
        and query.shape[2] == 1
        and query.dtype in _lib.DTYPE_CODES
        and key_blocks.dtype == value_blocks.dtype == query.dtype
        and block_tables.ndim == 2
        and sequence_lengths.ndim == 1
    )


def _split_policy() -> int:
    raw = os.environ.get("MIE_DECODE_SPLIT_POLICY", "auto").strip().lower()
    if raw in ("", "auto"):
        return 1
    if raw == "none":
        return 0
    return max(16, int(raw))


def decode_scratch(batch: int, q_heads: int, kv_heads: int, head_dim: int, max_total_tokens: int,
                   device: torch.device) -> torch.Tensor:
    """Uninitialised scratch (work plan + split-KV partials) for one decode-attention call."""

    size = int(_lib.load().mie_decode_scratch_bytes(batch, q_heads, kv_heads, head_dim, int(max_total_tokens)))
    return torch.empty(size, dtype=torch.uint8, device=device)


def launch_decode_attention(
    query: torch.Tensor,
    output: torch.Tensor,
    key_blocks: torch.Tensor,
    value_blocks: torch.Tensor,
    block_tables: torch.Tensor,
    sequence_lengths: torch.Tensor,
    query_positions: torch.Tensor | None,
    *,
    scale: float,
    max_total_tokens: int,
    scratch: torch.Tensor | None = None,
    split_policy: int | None = None,
    plan_only: bool = False,
    use_plan: bool = False,
    plan_slot: int = 0,
    status: torch.Tensor | None = None,
    quantized_out: tuple[torch.Tensor, torch.Tensor] | None = None,
) -> None:
    """Thin call into ``mie_paged_decode_attention``; ``output`` has the query's shape.  ``quantized_out`` =
    ``(e4m3 [batch, q_heads * 128], scales [q_heads, batch])`` also receives the output quantised for o_proj."""

    batch, q_heads, _, head_dim = (int(v) for v in query.shape)
    num_blocks, kv_heads, block_size, _ = (int(v) for v in key_blocks.shape)
    device = query.device
    if scratch is None:
        scratch = decode_scratch(batch, q_heads, kv_heads, head_dim, max_total_tokens, device)
    word = status if status is not None else _lib.status_word(device)
    q8, q_scales = quantized_out if quantized_out is not None else (None, None)
    _lib.check(_lib.load().mie_paged_decode_attention(
        _lib.view4_arg(query), _lib.view4_arg(output), _lib.view4_arg(key_blocks), _lib.view4_arg(value_blocks),
        _lib.index_arg(block_tables), _lib.index_arg(sequence_lengths), _lib.index_arg(query_positions),
        batch, q_heads, kv_heads, head_dim, block_size, num_blocks, int(block_tables.shape[1]),
        _lib.DTYPE_CODES[query.dtype], float(scale),
        _split_policy() if split_policy is None else int(split_policy),
        int(max_total_tokens), _lib.ptr(scratch), scratch.numel(), int(plan_only), int(use_plan), int(plan_slot),
        _lib.ptr(q8), 0 if q8 is None else q8.stride(0), _lib.ptr(q_scales), 0 if q_scales is None else q_scales.stride(0),
        _lib.ptr(word), _lib.stream_arg(device),
    ))


def triton_paged_decode_attention(
    query: torch.Tensor,
    key_blocks: torch.Tensor,
    value_blocks: torch.Tensor,
    block_tables: torch.Tensor,
    sequence_lengths: torch.Tensor,
    *,
    scale: float,
    split_count: int = 1,
    max_sequence_length: int | None = None,
    use_gqa_reuse: bool | None = False,
    block_tokens: int = 16,
    query_start_positions: torch.Tensor | None = None,
    sdpa_compat: bool = False,
    _validate_metadata: bool = True,
    _reserved_lengths: tuple[int, ...] | None = None,
) -> torch.Tensor:
    """Decode one token per request straight from physical KV pages.

    ``query`` is ``[batch, query_heads, 1, head_dim]``, pages are
    ``[physical_blocks, kv_heads, block_size, head_dim]``; the result has the
    attention-interface layout ``[batch, 1, query_heads, head_dim]``.  With
    query positions, row ``b`` reads only its first
    ``min(sequence_length, position + 1)`` tokens; device positions may change
    between CUDA-graph replays.
    """

    if not can_use_triton_paged_decode(query, key_blocks, value_blocks, block_tables, sequence_lengths):
        raise ValueError("inputs do not satisfy the Triton paged-decode contract")
    batch, q_heads, _, head_dim = (int(v) for v in query.shape)
    num_blocks, kv_heads, block_size, _ = (int(v) for v in key_blocks.shape)
    if value_blocks.shape != key_blocks.shape:
        raise ValueError("key and value page tensors must have identical shapes")
    if int(block_tables.shape[0]) != batch:
        raise ValueError("block-table batch does not match query batch")
    if int(sequence_lengths.shape[0]) != batch:
        raise ValueError("sequence lengths do not match query batch")
    if query_start_positions is not None and (
        query_start_positions.ndim != 1
        or int(query_start_positions.shape[0]) != batch
        or query_start_positions.device != query.device
        or query_start_positions.dtype not in (torch.int32, torch.int64)
    ):
        raise ValueError(
            "query positions must be an integer vector on the query device with one value per row"
        )
    if q_heads % kv_heads != 0:
        raise ValueError("query heads must be divisible by KV heads")
    if use_gqa_reuse is True and q_heads // kv_heads not in (2, 4):
        raise ValueError("GQA-reuse decode currently supports 2 or 4 query heads per KV head")
    if not 1 <= block_size <= 128:
        raise ValueError("Triton paged decode supports block sizes from 1 to 128")
    allowed_tiles = (8, 16, 32, 64, 128) if sdpa_compat else (8, 16, 32, 64)
    if int(block_tokens) not in allowed_tiles:
        raise ValueError("block_tokens must be 8, 16, 32, or 64 (128 only in SDPA-compatible mode)")
    split_count = int(split_count)
    if split_count not in _SPLIT_COUNTS:
        raise ValueError("split_count must be one of 1, 2, 4, or 8")
    if sdpa_compat and split_count != 1:
        raise ValueError("SDPA-compatible decode requires a single KV split")
    if split_count > 1:
        if max_sequence_length is None or int(max_sequence_length) < 1:
            raise ValueError("max_sequence_length is required when split-KV is enabled")
        max_sequence_length = int(max_sequence_length)
        if max_sequence_length < split_count:
            raise ValueError("max_sequence_length must cover every requested split")

    if _validate_metadata:
        validate_decode_metadata(
            block_tables, sequence_lengths, device=query.device, batch_size=batch, num_blocks=num_blocks,
            block_size=block_size, query_positions=query_start_positions,
            max_sequence_length=max_sequence_length if split_count > 1 else None,
            reserved_lengths=_reserved_lengths,
        )

    capacity = int(block_tables.shape[1]) * block_size
    bound = capacity if max_sequence_length is None else min(capacity, int(max_sequence_length))
    output = torch.empty_like(query)
    launch_decode_attention(
        query, output, key_blocks, value_blocks, block_tables, sequence_lengths, query_start_positions,
        scale=scale, max_total_tokens=batch * max(bound, 1),
    )
    return output.transpose(1, 2)


__all__ = [
    "can_use_triton_paged_decode",
    "select_decode_block_tokens",
    "select_decode_split_count",
    "select_split_kv_decode",
    "SPLIT_KV_BLOCK_TOKENS",
    "triton_is_available",
    "triton_paged_decode_attention",
]
