"""Seeded synthetic inputs for the hot path's benchmark and parity configurations.

All tensors are generated on the CPU from a ``torch.Generator`` so the CPU
oracle and the GPU kernels see identical bits; callers move them to a device.
Shapes follow Qwen3-4B (32 query / 8 KV heads, head_dim 128, hidden 2560,
MLP 9728, 16-token pages).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

Q_HEADS = 32
KV_HEADS = 8
HEAD_DIM = 128
HIDDEN = 2560
INTERMEDIATE = 9728
VOCAB = 151936
LAYERS = 36
PAGE = 16
RMS_EPS = 1e-6
ROPE_THETA = 5_000_000.0

# (N, K) of the four merged projections of one layer.
GEMM_SHAPES = {
    "qkv": (Q_HEADS * HEAD_DIM + 2 * KV_HEADS * HEAD_DIM, HIDDEN),
    "o": (HIDDEN, Q_HEADS * HEAD_DIM),
    "gate_up": (2 * INTERMEDIATE, HIDDEN),
    "down": (HIDDEN, INTERMEDIATE),
}
GEMM_M_SWEEP = (1, 8, 64, 256, 2048)


def _generator(seed: int) -> torch.Generator:
    generator = torch.Generator(device="cpu")
    generator.manual_seed(seed)
    return generator


@dataclass
class DecodeCase:
    """One ragged paged-decode problem: per-request K/V, a shared page pool and random block tables."""

    query: torch.Tensor            # [batch, q_heads, 1, dim]
    key_blocks: torch.Tensor       # [pages, kv_heads, page, dim]
    value_blocks: torch.Tensor
    block_tables: torch.Tensor     # [batch, width] int32, -1 padded
    sequence_lengths: torch.Tensor  # [batch] int32
    scale: float
    lengths: tuple[int, ...] = field(default_factory=tuple)

    def to(self, device) -> "DecodeCase":
        return DecodeCase(self.query.to(device), self.key_blocks.to(device), self.value_blocks.to(device),
                          self.block_tables.to(device), self.sequence_lengths.to(device), self.scale, self.lengths)


def sequence_kv(seed: int, length: int, kv_heads: int = KV_HEADS, head_dim: int = HEAD_DIM,
                dtype: torch.dtype = torch.bfloat16) -> tuple[torch.Tensor, torch.Tensor]:
    """K and V of one sequence, ``[1, kv_heads, length, dim]`` ~ N(0, 1)."""

    generator = _generator(seed)
    keys = torch.randn(1, kv_heads, length, head_dim, generator=generator).to(dtype)
    values = torch.randn(1, kv_heads, length, head_dim, generator=generator).to(dtype)
    return keys, values


def decode_case(lengths=(17, 128, 513, 2048), *, seed: int = 0, num_pages: int = 256, page: int = PAGE,
                q_heads: int = Q_HEADS, kv_heads: int = KV_HEADS, head_dim: int = HEAD_DIM,
                dtype: torch.dtype = torch.bfloat16, shuffle_pages: bool = True) -> DecodeCase:
    """BASELINE configuration 0 by default: ragged batch, pool of 256 pages, random page permutation.

    Sequence ``i`` draws its K/V from seed ``seed * 1000 + i + 1``; the query from ``seed``.
    """

    generator = _generator(seed)
    batch = len(lengths)
    query = torch.randn(batch, q_heads, 1, head_dim, generator=generator).to(dtype)
    needed = [-(-n // page) for n in lengths]
    if sum(needed) > num_pages:
        raise ValueError("page pool too small for the requested lengths")
    order = torch.randperm(num_pages, generator=generator) if shuffle_pages else torch.arange(num_pages)
    key_blocks = torch.zeros(num_pages, kv_heads, page, head_dim, dtype=dtype)
    value_blocks = torch.zeros_like(key_blocks)
    width = max(needed)
    tables = torch.full((batch, width), -1, dtype=torch.int32)
    cursor = 0
    for i, (length, pages) in enumerate(zip(lengths, needed)):
        ids = order[cursor : cursor + pages]
        cursor += pages
        tables[i, :pages] = ids.to(torch.int32)
        keys, values = sequence_kv(seed * 1000 + i + 1, length, kv_heads, head_dim, dtype)
        padded = pages * page
        k_pad = torch.zeros(kv_heads, padded, head_dim, dtype=dtype)
        v_pad = torch.zeros_like(k_pad)
        k_pad[:, :length] = keys[0]
        v_pad[:, :length] = values[0]
        key_blocks[ids] = k_pad.view(kv_heads, pages, page, head_dim).permute(1, 0, 2, 3)
        value_blocks[ids] = v_pad.view(kv_heads, pages, page, head_dim).permute(1, 0, 2, 3)
    return DecodeCase(query, key_blocks, value_blocks, tables,
                      torch.tensor(lengths, dtype=torch.int32), 1.0 / math.sqrt(head_dim), tuple(lengths))


def lognormal_contexts(count: int, *, seed: int, median: float = 2048.0, sigma: float = 1.0,
                       low: int = 16, high: int = 32768) -> torch.Tensor:
    """Context lengths of BASELINE configuration 4: round(exp(N(ln median, sigma))) clipped to [low, high]."""

    generator = _generator(seed)
    raw = torch.exp(torch.randn(count, generator=generator) * sigma + math.log(median))
    return raw.round().clamp(low, high).to(torch.int64)


def random_block_tables(lengths: torch.Tensor, *, num_pages: int, page: int = PAGE, seed: int = 0,
                        extra_tokens: int = 0) -> torch.Tensor:
    """Block tables ``[batch, width]`` int32 drawn from one random permutation of the pool.

    ``extra_tokens`` reserves room for tokens appended later (decode steps).
    """

    needed = [-(-(int(n) + extra_tokens) // page) for n in lengths.tolist()]
    if sum(needed) > num_pages:
        raise ValueError(f"page pool of {num_pages} too small: {sum(needed)} pages needed")
    order = torch.randperm(num_pages, generator=_generator(seed)).to(torch.int32)
    tables = torch.full((len(needed), max(needed)), -1, dtype=torch.int32)
    cursor = 0
    for row, pages in enumerate(needed):
        tables[row, :pages] = order[cursor : cursor + pages]
        cursor += pages
    return tables


def gemm_case(name: str, m: int, *, seed: int = 0, dtype: torch.dtype = torch.bfloat16):
    """BASELINE configuration 1: ``(x [m, K] bf16 ~ N(0,1), W [N, K] fp32 ~ N(0, 0.02))``."""

    n, k = GEMM_SHAPES[name]
    generator = _generator(seed * 7919 + m * 13 + sum(map(ord, name)))
    weight = torch.randn(n, k, generator=generator) * 0.02
    x = torch.randn(m, k, generator=generator).to(dtype)
    return x, weight


@dataclass
class PrefillCase:
    """BASELINE configuration 2: chunks over cached prefixes, packed into one varlen stream."""

    prefix_lengths: tuple[int, ...]
    chunk_lengths: tuple[int, ...]
    query: torch.Tensor            # [tokens, q_heads, dim]
    new_keys: torch.Tensor         # [1, kv_heads, tokens, dim]
    new_values: torch.Tensor
    key_blocks: torch.Tensor       # prefix already written
    value_blocks: torch.Tensor
    block_tables: torch.Tensor     # [requests, width] int32
    cu_seqlens: torch.Tensor       # [requests + 1] int32
    kv_lens: torch.Tensor          # [requests] int32
    token_to_sequence: torch.Tensor  # [tokens] int32
    token_positions: torch.Tensor    # [tokens] int32
    scale: float

    def to(self, device) -> "PrefillCase":
        moved = {name: (value.to(device) if isinstance(value, torch.Tensor) else value)
                 for name, value in self.__dict__.items()}
        return PrefillCase(**moved)


def prefill_case(*, requests: int = 6, seed: int = 0, max_prefix: int = 4096, max_chunk: int = 512,
                 page: int = PAGE, q_heads: int = Q_HEADS, kv_heads: int = KV_HEADS, head_dim: int = HEAD_DIM,
                 prefix_lengths=None, chunk_lengths=None, spare_pages: int = 8,
                 dtype: torch.dtype = torch.bfloat16) -> PrefillCase:
    generator = _generator(seed)
    if prefix_lengths is None:
        prefix_lengths = torch.randint(0, max_prefix + 1, (requests,), generator=generator).tolist()
    if chunk_lengths is None:
        chunk_lengths = torch.randint(1, max_chunk + 1, (requests,), generator=generator).tolist()
    requests = len(prefix_lengths)
    totals = [p + c for p, c in zip(prefix_lengths, chunk_lengths)]
    needed = [-(-t // page) for t in totals]
    num_pages = sum(needed) + spare_pages
    order = torch.randperm(num_pages, generator=generator)
    key_blocks = torch.zeros(num_pages, kv_heads, page, head_dim, dtype=dtype)
    value_blocks = torch.zeros_like(key_blocks)
    tables = torch.full((requests, max(needed)), -1, dtype=torch.int32)
    cursor = 0
    for r, (prefix, pages) in enumerate(zip(prefix_lengths, needed)):
        ids = order[cursor : cursor + pages]
        cursor += pages
        tables[r, :pages] = ids.to(torch.int32)
        if prefix:
            keys, values = sequence_kv(seed * 1000 + 500 + r, prefix, kv_heads, head_dim, dtype)
            full = -(-prefix // page)
            k_pad = torch.zeros(kv_heads, full * page, head_dim, dtype=dtype)
            v_pad = torch.zeros_like(k_pad)
            k_pad[:, :prefix] = keys[0]
            v_pad[:, :prefix] = values[0]
            key_blocks[ids[:full]] = k_pad.view(kv_heads, full, page, head_dim).permute(1, 0, 2, 3)
            value_blocks[ids[:full]] = v_pad.view(kv_heads, full, page, head_dim).permute(1, 0, 2, 3)
    tokens = sum(chunk_lengths)
    query = torch.randn(tokens, q_heads, head_dim, generator=generator).to(dtype)
    new_keys = torch.randn(1, kv_heads, tokens, head_dim, generator=generator).to(dtype)
    new_values = torch.randn(1, kv_heads, tokens, head_dim, generator=generator).to(dtype)
    cu = torch.zeros(requests + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(chunk_lengths, dtype=torch.int32).cumsum(0)
    tok2seq = torch.cat([torch.full((c,), r, dtype=torch.int32) for r, c in enumerate(chunk_lengths)])
    tokpos = torch.cat([torch.arange(p, p + c, dtype=torch.int32) for p, c in zip(prefix_lengths, chunk_lengths)])
    return PrefillCase(tuple(prefix_lengths), tuple(chunk_lengths), query, new_keys, new_values, key_blocks,
                       value_blocks, tables, cu, torch.tensor(totals, dtype=torch.int32), tok2seq, tokpos,
                       1.0 / math.sqrt(head_dim))
