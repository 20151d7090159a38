"""Tiled varlen causal prefill attention over KV pages
(reference: engine/kv_cache/triton_flash_prefill.py:154-202).

Same name and signature as the reference; the kernel is
``mie_flash_prefill_attention`` in ``csrc/prefill_attention.cu``.
"""

from __future__ import annotations

import torch

from ... import _lib


def triton_flash_prefill_attention(
    query: torch.Tensor,
    key_blocks: torch.Tensor,
    value_blocks: torch.Tensor,
    block_tables: torch.Tensor,
    cu_seqlens: torch.Tensor,
    kv_lens: torch.Tensor,
    *,
    max_query_len: int,
    scale: float,
) -> torch.Tensor:
    """Causal varlen attention for flat ``[tokens, heads, dim]`` Q over KV pages.

    ``key_blocks`` / ``value_blocks`` are ``[physical_blocks, kv_heads, page, dim]`` and already hold every
    request's K/V (new tokens included).  ``cu_seqlens`` (``[requests + 1]``) splits the flat query rows per
    request, ``kv_lens`` is each request's total K/V length, and ``max_query_len`` is a host int that sizes
    the grid, so nothing is read back from the device.
    """

    if not query.is_cuda:
        raise RuntimeError("flash prefill needs CUDA tensors")
    if query.ndim != 3 or key_blocks.ndim != 4 or key_blocks.shape != value_blocks.shape:
        raise ValueError("expected query [tokens, heads, dim] and pages [blocks, kv_heads, page, dim]")
    tokens, heads, head_dim = (int(x) for x in query.shape)
    num_blocks, kv_heads, page, _ = (int(x) for x in key_blocks.shape)
    if heads % kv_heads or head_dim & (head_dim - 1) or page & (page - 1):
        raise ValueError("needs heads divisible by KV heads and power-of-two head_dim and page size")
    if query.stride(2) != 1 or key_blocks.stride(3) != 1 or value_blocks.stride(3) != 1:
        raise ValueError("the last (head_dim) dimension must be contiguous")
    if query.dtype not in (torch.bfloat16, torch.float16) or key_blocks.dtype != query.dtype:
        raise ValueError("flash prefill supports bf16/fp16 queries and pages of the same dtype")
    out = torch.empty_like(query)
    launch_flash_prefill(query, out, key_blocks, value_blocks, block_tables, cu_seqlens, kv_lens,
                         max_query_len=max_query_len, scale=scale)
    return out


def launch_flash_prefill(query, out, key_blocks, value_blocks, block_tables, cu_seqlens, kv_lens, *,
                         max_query_len: int, scale: float, status: torch.Tensor | None = None) -> None:
    """Thin call into ``mie_flash_prefill_attention`` writing into ``out`` (``[tokens, heads, dim]``, same
    dtype as the query, last dimension contiguous).  Rows of ``query`` that no ``cu_seqlens`` range covers
    are left untouched in ``out``."""

    tokens, heads, head_dim = (int(x) for x in query.shape)
    num_blocks, kv_heads, page, _ = (int(x) for x in key_blocks.shape)
    requests = int(cu_seqlens.shape[0]) - 1
    if tokens == 0 or requests <= 0:
        return
    device = query.device
    word = status if status is not None else _lib.status_word(device)
    _lib.check(_lib.load().mie_flash_prefill_attention(
        _lib.ptr(query), query.stride(0), query.stride(1), tokens, _lib.ptr(out), out.stride(0), out.stride(1),
        _lib.view4_arg(key_blocks), _lib.view4_arg(value_blocks), _lib.index_arg(block_tables),
        _lib.index_arg(cu_seqlens), _lib.index_arg(kv_lens), requests, int(max_query_len), heads, kv_heads,
        head_dim, page, num_blocks, int(block_tables.shape[1]), _lib.DTYPE_CODES[query.dtype], float(scale),
        _lib.ptr(word), _lib.stream_arg(device),
    ))


__all__ = ["triton_flash_prefill_attention"]  # launch_flash_prefill is this package's own lower-level entry
