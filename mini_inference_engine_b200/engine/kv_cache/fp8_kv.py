"""FP8 (e4m3) KV cache: pool layout, the decode-attention call over it and a torch quantiser.

The reference keeps K/V in bf16 and only names an FP8 cache as the lever left for its HBM-bound decode
(docs/phase_notes/roofline.md:76); there is no reference function to mirror, so the names here are this
package's own.  Layout per layer (page size 16, head_dim 128)::

    data   [pages, kv_heads, 2, 16, 128] uint8   K rows then V rows of one (page, head): one 4 KiB TMA box
    scales [pages, kv_heads, 2, 16]      float32 one scale per (token, KV head) for K and for V

``scale = amax / 448`` of the row and ``row / max(scale, 1e-12)`` rounded to e4m3, the rule of the activation
quantiser.  2,112 bytes per token and layer at 8 KV heads instead of 4,096.
"""

from __future__ import annotations

import torch

from ... import _lib

PAGE = 16
HEAD_DIM = 128


class Fp8KvPool:
    """``[layers, pages, kv_heads, 2, 16, 128]`` e4m3 bytes and their scales on one device."""

    def __init__(self, layers: int, num_pages: int, kv_heads: int, device: torch.device) -> None:
        self.layers, self.num_pages, self.kv_heads = layers, num_pages, kv_heads
        self.data = torch.zeros(layers, num_pages, kv_heads, 2, PAGE, HEAD_DIM, dtype=torch.uint8, device=device)
        self.scales = torch.zeros(layers, num_pages, kv_heads, 2, PAGE, dtype=torch.float32, device=device)
        if self.data.data_ptr() % 1024 or self.scales.data_ptr() % 128:
            raise RuntimeError("the allocator returned an unaligned FP8 KV pool")

    @property
    def page_stride_bytes(self) -> int:
        return self.kv_heads * 2 * PAGE * HEAD_DIM

    def bytes_per_token(self) -> int:
        """K + V bytes one context token costs per layer, scales included."""

        return self.kv_heads * 2 * (HEAD_DIM + 4)

    def fill_from(self, layer: int, key_blocks: torch.Tensor, value_blocks: torch.Tensor) -> None:
        """Quantise bf16 pages ``[pages, kv_heads, 16, 128]`` into layer ``layer`` (tests, benchmarks)."""

        for which, pages in enumerate((key_blocks, value_blocks)):
            quantized, scales = quantize_kv_rows(pages)
            self.data[layer, :, :, which].copy_(quantized)
            self.scales[layer, :, :, which].copy_(scales)


    def dequantized_pages(self, layer: int, page_ids: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """The pages ``page_ids`` (int64, on the pool's device) of layer ``layer`` as two contiguous bf16 tensors
        ``[len(page_ids), kv_heads, 16, 128]``: ``e4m3 * scale`` rounded to bf16, what a reader of the cache sees.
        The prompt-chunk attention kernel reads bf16 pages, so a chunk step stages its requests' pages this way."""

        staged = []
        for which in (0, 1):
            data = self.data[layer, :, :, which].index_select(0, page_ids)
            scales = self.scales[layer, :, :, which].index_select(0, page_ids)
            staged.append((data.view(torch.float8_e4m3fn).float() * scales.unsqueeze(-1)).to(torch.bfloat16))
        return staged[0], staged[1]


def quantize_kv_rows(rows: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``[..., 128]`` bf16/fp16 rows -> (e4m3 bytes as uint8, fp32 scales ``[...]``), with torch ops on the
    rows' device.  The CUDA writer (``mie_qkv_norm_rope_write_kv8``) produces the same bits."""

    values = rows.float()
    # A tensor divisor: dividing by a Python scalar lets the CUDA backend multiply by 1/448 instead, which
    # is not the correctly rounded quotient the writer kernel and the CPU compute.
    scales = values.abs().amax(dim=-1) / torch.full((), 448.0, dtype=torch.float32, device=rows.device)
    quantized = (values / scales.clamp_min(1e-12).unsqueeze(-1)).to(torch.float8_e4m3fn)
    return quantized.view(torch.uint8), scales


def launch_decode_attention_kv8(
    query: torch.Tensor,
    output: torch.Tensor,
    pool_data: torch.Tensor,
    pool_scales: torch.Tensor,
    block_tables: torch.Tensor,
    sequence_lengths: torch.Tensor,
    query_positions: torch.Tensor | None,
    *,
    scale: float,
    scratch: torch.Tensor,
    split_policy: int = 1,
    plan_only: bool = False,
    use_plan: bool = False,
    plan_slot: int = 0,
    status: torch.Tensor | None = None,
    quantized_out: tuple[torch.Tensor, torch.Tensor] | None = None,
) -> None:
    """Ragged paged decode attention over ONE layer of an FP8 pool (``pool_data`` ``[pages, kv_heads, 2, 16, 128]``
    uint8, ``pool_scales`` ``[pages, kv_heads, 2, 16]`` fp32); ``query`` / ``output`` ``[batch, heads, 1, 128]``.
    Thin call into ``mie_paged_decode_attention_kv8``."""

    batch, q_heads, _, head_dim = (int(v) for v in query.shape)
    num_blocks, kv_heads = int(pool_data.shape[0]), int(pool_data.shape[1])
    if head_dim != HEAD_DIM or tuple(pool_data.shape[2:]) != (2, PAGE, HEAD_DIM) or pool_data.dtype != torch.uint8:
        raise ValueError("the FP8 KV path needs head_dim 128 and a [pages, kv_heads, 2, 16, 128] uint8 pool")
    if not pool_data[0].is_contiguous() or not pool_scales.is_contiguous():
        raise ValueError("pages of the FP8 pool must be contiguous")
    device = query.device
    word = status if status is not None else _lib.status_word(device)
    q8, q_scales = quantized_out if quantized_out is not None else (None, None)
    _lib.check(_lib.load().mie_paged_decode_attention_kv8(
        _lib.view4_arg(query), _lib.view4_arg(output), _lib.ptr(pool_data), int(pool_data.stride(0)),
        _lib.ptr(pool_scales), _lib.index_arg(block_tables), _lib.index_arg(sequence_lengths),
        _lib.index_arg(query_positions), batch, q_heads, kv_heads, num_blocks, int(block_tables.shape[1]),
        _lib.DTYPE_CODES[query.dtype], float(scale), int(split_policy), _lib.ptr(scratch), scratch.numel(),
        int(plan_only), int(use_plan), int(plan_slot), _lib.ptr(q8), 0 if q8 is None else q8.stride(0),
        _lib.ptr(q_scales), 0 if q_scales is None else q_scales.stride(0), _lib.ptr(word), _lib.stream_arg(device),
    ))


__all__ = ["Fp8KvPool", "launch_decode_attention_kv8", "quantize_kv_rows"]
