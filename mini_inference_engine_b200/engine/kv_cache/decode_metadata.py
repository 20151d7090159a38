"""Decode-metadata validation (reference: engine/kv_cache/decode_metadata.py:10-91).

Eager calls copy the small metadata tensors to the host and raise ``ValueError``
with the reference's messages before any kernel touches a page.  While a CUDA
graph is being captured nothing may be read on the host, so one small kernel
applies the same predicates on every replay and ORs the outcome into a device
status word; ``raise_for_status`` turns a non-zero word into the same
``ValueError`` after the step's results were copied back.  The reference uses
device asserts there, which lose the CUDA context; this library never traps.
"""

from __future__ import annotations

from collections.abc import Sequence

import torch

from ... import _lib


def _host_rows(tensor: torch.Tensor) -> list:
    return tensor.detach().to("cpu").tolist()


def validate_decode_metadata(
    block_tables: torch.Tensor,
    sequence_lengths: torch.Tensor,
    *,
    device: torch.device,
    batch_size: int,
    num_blocks: int,
    block_size: int,
    query_positions: torch.Tensor | None = None,
    max_sequence_length: int | None = None,
    reserved_lengths: Sequence[int] | None = None,
    status: torch.Tensor | None = None,
) -> None:
    """Check live block-table entries, lengths and positions of one decode batch."""

    integer = (torch.int32, torch.int64)
    for name, tensor, ndim in (("block_tables", block_tables, 2), ("sequence_lengths", sequence_lengths, 1)):
        if tensor.ndim != ndim or tensor.shape[0] != batch_size:
            raise ValueError(f"{name} has an invalid shape for the decode batch")
        if tensor.device != device or tensor.dtype not in integer:
            raise ValueError(f"{name} must be an integer tensor on the query device")
    if query_positions is not None and (
        query_positions.ndim != 1
        or query_positions.shape[0] != batch_size
        or query_positions.device != device
        or query_positions.dtype not in integer
    ):
        raise ValueError("query positions must be an integer vector on the query device")
    if reserved_lengths is not None and len(reserved_lengths) != batch_size:
        raise ValueError("reserved lengths must contain one value per sequence")

    capturing = device.type == "cuda" and torch.cuda.is_current_stream_capturing()
    if capturing:
        word = status if status is not None else _lib.status_word(device)
        _lib.check(_lib.load().mie_validate_decode_metadata(
            _lib.index_arg(block_tables), _lib.index_arg(sequence_lengths), _lib.index_arg(query_positions),
            batch_size, int(block_tables.shape[1]), block_size, num_blocks,
            -1 if max_sequence_length is None else int(max_sequence_length),
            _lib.ptr(word), _lib.stream_arg(device),
        ))
        return

    width = int(block_tables.shape[1])
    lengths = _host_rows(sequence_lengths)
    positions = None if query_positions is None else _host_rows(query_positions)
    tables = _host_rows(block_tables)
    for row, length in enumerate(lengths):
        if not 1 <= length <= width * block_size:
            raise ValueError("sequence_lengths exceed the available block-table capacity")
        if reserved_lengths is not None and length > reserved_lengths[row]:
            raise ValueError("sequence_lengths exceed the reserved KV length")
        position = length - 1 if positions is None else positions[row]
        if not 0 <= position < length:
            raise ValueError("query position must satisfy 0 <= position < sequence_length")
        read_length = length if positions is None else position + 1
        if max_sequence_length is not None and read_length > max_sequence_length:
            raise ValueError("max_sequence_length does not cover the attention read length")
        live_pages = -(-length // block_size)
        if any(not 0 <= page < num_blocks for page in tables[row][:live_pages]):
            raise ValueError("block_tables contain an invalid physical block ID")


__all__ = ["validate_decode_metadata"]
