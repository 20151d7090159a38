"""Flat-token Qwen3 forward over the sm_100a kernels, with a CUDA-graph decode step.

Takes the place of the captured decode forward of the reference
(engine/serving/chunked_prefill.py:206-298: ``_graph_decode_call`` /
``_capture_decode_graph`` / ``_decode``) and of the flat layer loops
(engine/model_runner/qwen3_mixed.py:125, qwen3_packed.py:29).  The reference
drives Hugging Face's ``Qwen3ForCausalLM`` and monkey-patches its modules; this
runner owns plain weight tensors and calls the kernels directly, so one decode
layer is a dozen launches of this library's kernels:

  add+RMSNorm(+quant) -> FP8 GEMM (merged qkv) -> q/k-norm + RoPE + KV write ->
  paged decode attention -> quant -> FP8 GEMM (o) [all-reduce] ->
  add+RMSNorm(+quant) -> FP8 GEMM (merged gate_up) -> SiLU*up(+quant) ->
  FP8 GEMM (down) [all-reduce]

Tensor parallelism is by heads: rank r of t owns query heads [32r/t, 32(r+1)/t)
and KV heads [8r/t, 8(r+1)/t) with its own K/V page pool, the merged qkv and
gate_up projections are column-parallel, o and down are row-parallel.  Their
partial sums are combined by ``mie_tp_reduce_rms_norm`` (one kernel per rank
over IPC-mapped peer memory that also does the residual add, the RMSNorm and
the FP8 quantisation for the next GEMM; ``MIE_TP_EXCHANGE=nccl`` selects a
plain NCCL all-reduce instead).  The tied lm_head is vocabulary-sharded and
greedy sampling exchanges one (value, index) pair per row over NCCL.  The
library is reached through its C-ABI with ``ctypes``; PyTorch owns tensors,
streams and CUDA graphs only.
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass

import torch

from ... import _lib
from ..kernels import sm89_fp8
from .peer_exchange import PeerExchange
from ..kv_cache.fp8_kv import Fp8KvPool, launch_decode_attention_kv8
from ..kv_cache.triton_flash_prefill import launch_flash_prefill
from ..kv_cache.triton_paged_attention import decode_scratch, launch_decode_attention


# A decode work plan carries 64 work counters, one per attention launch that reuses it; deeper models
# rebuild the plan every 64 layers.
PLAN_SLOTS = 64


@dataclass(frozen=True)
class Qwen3Shape:
    """Architecture constants (defaults: Qwen3-4B)."""

    layers: int = 36
    hidden: int = 2560
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 9728
    vocab: int = 151936
    rms_eps: float = 1e-6
    rope_theta: float = 5_000_000.0
    page: int = 16


def quantize_weight_blocks(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """e4m3 weight + one fp32 scale per 128x128 block (``amax / 448``), on the weight's device."""

    n, k = weight.shape
    nb, kb = -(-n // 128), -(-k // 128)
    padded = torch.zeros(nb * 128, kb * 128, dtype=torch.float32, device=weight.device)
    padded[:n, :k] = weight.float()
    blocks = padded.view(nb, 128, kb, 128)
    scales = blocks.abs().amax(dim=(1, 3)) / 448.0
    quantized = (blocks / scales.clamp_min(1e-12)[:, None, :, None]).view(nb * 128, kb * 128)[:n, :k]
    return quantized.to(torch.float8_e4m3fn).contiguous(), scales.contiguous()


@dataclass
class LayerWeights:
    qkv: torch.Tensor
    qkv_scale: torch.Tensor
    o: torch.Tensor
    o_scale: torch.Tensor
    gate_up: torch.Tensor
    gate_up_scale: torch.Tensor
    down: torch.Tensor
    down_scale: torch.Tensor
    input_norm: torch.Tensor
    post_norm: torch.Tensor
    q_norm: torch.Tensor
    k_norm: torch.Tensor


def shard_bounds(n: int, tp_size: int, tp_rank: int) -> tuple[int, int]:
    """Rows ``[start, stop)`` of an ``n``-row dimension that rank ``tp_rank`` of ``tp_size`` owns."""

    return n // tp_size * tp_rank, n // tp_size * (tp_rank + 1)


def scale_window(start: int, stop: int, block: int = 128) -> tuple[int, int]:
    """The smallest range of whole scale blocks ``[base, end)`` that covers ``[start, stop)``."""

    return start // block * block, -(-stop // block) * block


def _window_rows(w8: torch.Tensor, scales: torch.Tensor, start: int, stop: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Rows ``[start, stop)`` of a block-quantised ``[N, K]`` weight, placed inside their scale window: the
    result has ``end - base`` rows (zeros outside the shard) and the window's rows of the scale grid, so a
    shard that starts in the middle of a 128-row scale block keeps the unsharded block's scale."""

    base, end = scale_window(start, stop)
    out = torch.zeros(end - base, w8.shape[1], dtype=torch.uint8, device=w8.device)
    out[start - base:stop - base] = w8[start:stop].view(torch.uint8)
    rows = scales[base // 128:end // 128]
    if rows.shape[0] < (end - base) // 128:  # the window runs past the last (partial) block
        rows = torch.cat([rows, rows.new_zeros((end - base) // 128 - rows.shape[0], rows.shape[1])])
    return out.view(torch.float8_e4m3fn), rows.contiguous()


class Qwen3Weights:
    """Seeded random-init weights in the checkpoint's format, sharded for one tensor-parallel rank.

    Every rank draws the full tensors from the same per-layer seed, quantises them on the UNSHARDED
    128x128 block grid (what a checkpoint holds) and keeps its slice of the e4m3 values and of the scale
    grid, so all ranks of a group hold consistent shards and a shard is bit for bit a slice of the
    single-GPU model.  Head shards are whole scale blocks (head_dim 128).  An MLP shard need not be: at 8
    ranks 9728 / 8 = 1216 = 9.5 blocks, so odd ranks start 64 rows into a block.  Such a shard is stored
    inside its window of whole scale blocks (``inter_window`` wide, the shard at ``inter_offset``, zeros
    around it): gate and up each occupy one window of the merged gate_up weight, and down_proj's K
    dimension is the window, so every kernel keeps seeing 128-aligned scale blocks and the zero rows /
    columns contribute exact zeros.
    """

    def __init__(self, shape: Qwen3Shape, device: torch.device, *, seed: int = 0, tp_rank: int = 0,
                 tp_size: int = 1, layers: int | None = None) -> None:
        if shape.kv_heads % tp_size or shape.q_heads % tp_size or shape.vocab % tp_size:
            raise ValueError("tensor-parallel size must divide the head counts and the vocabulary")
        self.shape, self.device, self.tp_rank, self.tp_size = shape, device, tp_rank, tp_size
        d, hd = shape.hidden, shape.head_dim
        q_rows, kv_rows, inter = shape.q_heads * hd, shape.kv_heads * hd, shape.intermediate
        if inter % tp_size or (inter // tp_size) % 16:
            raise ValueError("tensor-parallel size must divide the MLP width into multiples of 16")
        if (q_rows // tp_size) % 128 or (kv_rows // tp_size) % 128:
            raise ValueError("a rank's query / KV head rows must be whole 128-row scale blocks")
        q_lo, q_hi = shard_bounds(q_rows, tp_size, tp_rank)
        kv_lo, kv_hi = shard_bounds(kv_rows, tp_size, tp_rank)
        i_lo, i_hi = shard_bounds(inter, tp_size, tp_rank)
        base, end = scale_window(i_lo, i_hi)
        self.inter_window, self.inter_offset, self.inter_width = end - base, i_lo - base, i_hi - i_lo

        def draw(generator: torch.Generator, rows: int, cols: int) -> torch.Tensor:
            return torch.randn(rows, cols, generator=generator, device=device, dtype=torch.float32) * 0.02

        def norm_weight(generator: torch.Generator, width: int) -> torch.Tensor:
            noise = torch.randn(width, generator=generator, device=device, dtype=torch.float32)
            return (1.0 + 0.1 * noise).to(torch.bfloat16)

        self.layers: list[LayerWeights] = []
        for index in range(shape.layers if layers is None else layers):
            generator = torch.Generator(device=device).manual_seed(seed * 100003 + index)
            wq, wk, wv = draw(generator, q_rows, d), draw(generator, kv_rows, d), draw(generator, kv_rows, d)
            wo = draw(generator, d, q_rows)
            wg, wu = draw(generator, inter, d), draw(generator, inter, d)
            wd = draw(generator, d, inter)
            (q8, q_s), (k8, k_s), (v8, v_s) = (quantize_weight_blocks(w) for w in (wq, wk, wv))
            o8, o_s = quantize_weight_blocks(wo)
            (g8, g_s), (u8, u_s) = quantize_weight_blocks(wg), quantize_weight_blocks(wu)
            d8, d_s = quantize_weight_blocks(wd)
            del wq, wk, wv, wo, wg, wu, wd
            qkv8 = torch.cat([q8[q_lo:q_hi], k8[kv_lo:kv_hi], v8[kv_lo:kv_hi]]).contiguous()
            qkv_s = torch.cat([q_s[q_lo // 128:q_hi // 128], k_s[kv_lo // 128:kv_hi // 128],
                               v_s[kv_lo // 128:kv_hi // 128]]).contiguous()
            o_local = o8[:, q_lo:q_hi].contiguous()
            o_local_s = o_s[:, q_lo // 128:q_hi // 128].contiguous()
            gate8, gate_s = _window_rows(g8, g_s, i_lo, i_hi)
            up8, up_s = _window_rows(u8, u_s, i_lo, i_hi)
            gu8, gu_s = torch.cat([gate8, up8]).contiguous(), torch.cat([gate_s, up_s]).contiguous()
            down8 = torch.zeros(d, end - base, dtype=torch.uint8, device=device)
            down8[:, i_lo - base:i_hi - base] = d8[:, i_lo:i_hi].view(torch.uint8)
            down_s = d_s[:, base // 128:end // 128]
            if down_s.shape[1] < (end - base) // 128:
                down_s = torch.cat([down_s, down_s.new_zeros(down_s.shape[0], (end - base) // 128 - down_s.shape[1])],
                                   dim=1)
            self.layers.append(LayerWeights(
                qkv8, qkv_s, o_local, o_local_s, gu8, gu_s, down8.view(torch.float8_e4m3fn), down_s.contiguous(),
                norm_weight(generator, d), norm_weight(generator, d),
                norm_weight(generator, hd), norm_weight(generator, hd),
            ))
            del q8, k8, v8, o8, g8, u8, d8
        generator = torch.Generator(device=device).manual_seed(seed * 100003 + 99991)
        self.embedding = (torch.randn(shape.vocab, d, generator=generator, device=device, dtype=torch.float32)
                          * 0.02).to(torch.bfloat16)
        self.final_norm = norm_weight(generator, d)
        # Tied lm_head, vocabulary-sharded: this rank scores rows [vocab_start, vocab_start + vocab / tp).
        v_lo, v_hi = shard_bounds(shape.vocab, tp_size, tp_rank)
        self.vocab_start = v_lo
        self.lm_head = self.embedding[v_lo:v_hi]

    def to(self, device: torch.device) -> "Qwen3Weights":
        """The same weights on another device (a CPU-drawn model is bit-identical on every host, a
        CUDA-drawn one follows the GPU's generator)."""

        import copy

        clone = copy.copy(self)
        clone.device = device
        clone.layers = [LayerWeights(*[getattr(layer, name).to(device) for name in layer.__dataclass_fields__])
                        for layer in self.layers]
        clone.embedding, clone.final_norm = self.embedding.to(device), self.final_norm.to(device)
        lo = self.vocab_start
        clone.lm_head = clone.embedding[lo:lo + self.lm_head.shape[0]]
        return clone

    def weight_bytes(self) -> int:
        total = self.lm_head.numel() * 2
        for layer in self.layers:
            for t in (layer.qkv, layer.o, layer.gate_up, layer.down):
                total += t.numel()
            for t in (layer.qkv_scale, layer.o_scale, layer.gate_up_scale, layer.down_scale):
                total += t.numel() * 4
        return total


def rope_table(shape: Qwen3Shape, max_positions: int, device: torch.device) -> torch.Tensor:
    """``[max_positions, 2, head_dim]`` bf16: cos row and sin row per position, built as HF's
    ``Qwen3RotaryEmbedding`` does (fp32 angles, cast at the end)."""

    inv_freq = 1.0 / (shape.rope_theta ** (torch.arange(0, shape.head_dim, 2, dtype=torch.int64,
                                                         device=device).float() / shape.head_dim))
    angles = torch.arange(max_positions, device=device, dtype=torch.float32).unsqueeze(1) * inv_freq
    emb = torch.cat((angles, angles), dim=-1)
    return torch.stack((emb.cos(), emb.sin()), dim=1).to(torch.bfloat16).contiguous()


DEFAULT_DECODE_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)


def select_bucket(rows: int, buckets: tuple[int, ...]) -> int | None:
    """Smallest bucket that holds ``rows`` (reference: engine/serving/decode_graph.py:29-32)."""

    if rows < 1:
        return None
    return next((size for size in buckets if size >= rows), None)


class _Padding:
    """Owner of a row that carries no request."""

    def __repr__(self) -> str:  # pragma: no cover - debugging aid
        return "<padding row>"


PADDING = _Padding()


class DecodeBuffers:
    """Static buffers of one decode-graph bucket (reference: engine/serving/decode_graph.py:36-96): ids,
    lengths (including the new token), block tables and output tokens keep their addresses across replays.

    Rows ``[0, live)`` carry requests, the rest are padding rows: token 0, length 1 and a one-entry table
    pointing at the row's OWN scratch page, so a padding row writes and reads offset 0 of a page no request
    and no other padding row uses.  ``scratch_pages`` must hold ``batch`` distinct page ids.

    Host side.  Ids and lengths (12 bytes a row) are copied whole every step.  The block tables are not:
    a pinned host mirror remembers, per row, who owns it and how many table entries the device already
    holds, and ``pack_rows`` copies only what changed - a whole row when its owner changed, the new tail
    when a request grew into another page, the scratch entry when a row became padding.  Block lists are
    append-only per owner.  The copies are asynchronous reads of the pinned mirror, so the caller must have
    synchronised with the previous step's copies before packing again (reading the step's tokens does).
    """

    def __init__(self, batch: int, table_width: int, device: torch.device, scratch_pages=None,
                 page: int = 16) -> None:
        self.batch, self.table_width, self.page = batch, table_width, page
        self.advance = False  # True when the captured graph feeds its tokens back and bumps the lengths
        self.scratch_pages = None if scratch_pages is None else tuple(int(p) for p in scratch_pages[:batch])
        if self.scratch_pages is not None and (len(self.scratch_pages) != batch
                                               or len(set(self.scratch_pages)) != batch
                                               or min(self.scratch_pages) < 0):
            raise ValueError("each graph row requires a distinct non-negative scratch page")
        self.input_ids = torch.zeros(batch, dtype=torch.int64, device=device)
        self.sequence_lengths = torch.ones(batch, dtype=torch.int32, device=device)
        self.block_tables = torch.full((batch, table_width), -1, dtype=torch.int32, device=device)
        self.output_tokens = torch.zeros(batch, dtype=torch.int64, device=device)
        pin = device.type == "cuda"

        def host(shape, dtype, fill):
            tensor = torch.full(shape, fill, dtype=dtype)
            return tensor.pin_memory() if pin else tensor

        # Host mirrors for the end-to-end path.
        self.host_ids = host((batch,), torch.int64, 0)
        self.host_lengths = host((batch,), torch.int32, 1)
        self.host_tables = host((batch, table_width), torch.int32, -1)
        self.host_tokens = host((batch,), torch.int64, 0)
        self._owners: list[object] = [None] * batch  # None: the device row is in an unknown state
        self._held: list[int] = [0] * batch          # table entries of the row that the device holds
        self.table_bytes_copied = 0                  # running total, for the measurement of the host step
        if self.scratch_pages is not None:
            self.pack_rows((), (), (), ())           # a valid all-padding batch for warm-up and capture

    def pack(self, ids, lengths, tables=None) -> int:
        """Copy one step's host metadata to the device whole (async, pinned). Returns the bytes copied."""

        self.host_ids.copy_(torch.as_tensor(ids, dtype=torch.int64))
        self.host_lengths.copy_(torch.as_tensor(lengths, dtype=torch.int32))
        self.input_ids.copy_(self.host_ids, non_blocking=True)
        self.sequence_lengths.copy_(self.host_lengths, non_blocking=True)
        copied = self.host_ids.numel() * 8 + self.host_lengths.numel() * 4
        if tables is not None:
            self.host_tables.copy_(torch.as_tensor(tables, dtype=torch.int32))
            self.block_tables.copy_(self.host_tables, non_blocking=True)
            copied += self.host_tables.numel() * 4
            self._owners = [None] * self.batch
        return copied

    def pack_rows(self, owners, ids, lengths, block_rows) -> int:
        """One step's rows: ``owners[i]`` (any hashable identity of the request in row i), its input token,
        its length INCLUDING the new token and its page ids.  Rows beyond ``len(owners)`` become padding.
        Only table entries that changed since the previous call are copied.  Returns the bytes copied."""

        live = len(owners)
        if not (len(ids) == len(lengths) == len(block_rows) == live) or live > self.batch:
            raise ValueError("real row counts must agree and fit the graph bucket")
        if self.scratch_pages is None and live < self.batch:
            raise ValueError("padding rows need scratch pages")
        page, width = self.page, self.table_width
        # Ids and lengths: two vectorised writes into the pinned mirrors.
        if live:
            self.host_ids[:live] = torch.as_tensor(ids, dtype=torch.int64)
            self.host_lengths[:live] = torch.as_tensor(lengths, dtype=torch.int32)
        if live < self.batch:
            self.host_ids[live:] = 0
            self.host_lengths[live:] = 1
        # Tables: plain Python comparisons per row, tensor writes only for what changed.
        scratch = None
        dirty: list[tuple[int, int, int]] = []  # (row, first entry, end entry)
        owners_now, held = self._owners, self._held
        for row in range(live):
            blocks, length = block_rows[row], int(lengths[row])
            count = len(blocks)
            if length < 1 or count > width or count * page < length:
                raise ValueError("decode position/block row exceeds the fixed graph table capacity")
            previous = owners_now[row]
            same_owner = previous is not None and previous is not PADDING and previous == owners[row]
            first = held[row] if same_owner else 0
            if count == first:
                continue
            if count < first:
                raise ValueError("a request's block list may only grow")
            fresh = [int(b) for b in blocks[first:]]
            if scratch is None:
                scratch = set(self.scratch_pages or ())
            if min(fresh) < 0 or not scratch.isdisjoint(fresh):
                raise ValueError("real rows must use valid blocks disjoint from scratch pages")
            self.host_tables[row, first:count] = torch.tensor(fresh, dtype=torch.int32)
            dirty.append((row, first, count))
            owners_now[row], held[row] = owners[row], count
        for row in range(live, self.batch):
            if owners_now[row] is not PADDING:
                self.host_tables[row, 0] = self.scratch_pages[row]
                dirty.append((row, 0, 1))
                owners_now[row], held[row] = PADDING, 1
        self.input_ids.copy_(self.host_ids, non_blocking=True)
        self.sequence_lengths.copy_(self.host_lengths, non_blocking=True)
        copied = self.batch * 12
        entries = sum(end - first for _, first, end in dirty)
        if len(dirty) > 32 or entries * 4 > self.host_tables.numel():
            self.block_tables.copy_(self.host_tables, non_blocking=True)
            table_bytes = self.host_tables.numel() * 4
        else:
            for row, first, end in dirty:
                self.block_tables[row, first:end].copy_(self.host_tables[row, first:end], non_blocking=True)
            table_bytes = entries * 4
        self.table_bytes_copied += table_bytes
        return copied + table_bytes


def sharded_greedy_tokens(local_logits: torch.Tensor, vocab_start: int, tp_size: int, group=None) -> torch.Tensor:
    """Greedy token ids from vocabulary-sharded logits ``[batch, vocab / tp]``.

    Every rank contributes its best (value, global index) pair per row; one all-gather later each rank
    picks the pair with the largest value (lowest rank wins ties, which is also the lowest index).
    """

    batch = local_logits.shape[0]
    best_value, best_index = local_logits.float().max(dim=-1)
    if tp_size == 1:
        return best_index + vocab_start
    pair = torch.stack((best_value, (best_index + vocab_start).float()), dim=-1).contiguous()
    flat = torch.empty(tp_size * batch, 2, dtype=torch.float32, device=local_logits.device)
    torch.distributed.all_gather_into_tensor(flat, pair, group=group)
    gathered = flat.view(tp_size, batch, 2)
    winner = gathered[:, :, 0].argmax(dim=0)
    return gathered[winner, torch.arange(batch, device=local_logits.device), 1].long()


def sharded_greedy_from_pairs(tokens: torch.Tensor, values: torch.Tensor, tp_size: int, group=None) -> torch.Tensor:
    """Global greedy tokens from every rank's local winner: ``tokens`` are global vocabulary indices, ``values``
    order-preserving keys of the winning bf16 logits (``mie_lm_head_argmax``).  The largest value wins; among
    equal values the lowest rank, whose shard holds the lower indices."""

    if tp_size == 1:
        return tokens
    rows = tokens.shape[0]
    pair = torch.stack((values.long(), tokens), dim=-1).contiguous()
    flat = torch.empty(tp_size * rows, 2, dtype=torch.int64, device=tokens.device)
    torch.distributed.all_gather_into_tensor(flat, pair, group=group)
    gathered = flat.view(tp_size, rows, 2)
    winner = gathered[:, :, 0].argmax(dim=0)
    return gathered[winner, torch.arange(rows, device=tokens.device), 1]


class MixedBuffers:
    """Static buffers of one captured mixed step: ``decode`` decode rows followed by ``chunk`` prompt-chunk
    tokens in one flat stream (reference: engine/kv_cache/mixed.py:44 ``MixedBatchMetadata``, built per step by
    engine/model_runner/qwen3_mixed.py:41-122; here the tensors are fixed so that the step can be replayed).

    Table rows ``[0, decode)`` belong to the decode rows, rows ``[decode, decode + chunks)`` to the prompt
    chunks, the last row to the padding "request" that owns every unused chunk token (its pages are scratch).
    """

    def __init__(self, decode: int, chunk: int, chunks: int, table_width: int, device: torch.device,
                 decode_scratch: tuple[int, ...], chunk_scratch: tuple[int, ...], page: int) -> None:
        self.decode, self.chunk, self.chunks, self.table_width, self.page = decode, chunk, chunks, table_width, page
        pad_pages = -(-chunk // page)  # pages the padding tokens of this bucket can spread over
        if len(decode_scratch) < decode or len(chunk_scratch) < pad_pages:
            raise ValueError("not enough scratch pages for this mixed bucket")
        if pad_pages > table_width:
            raise ValueError(f"a chunk bucket of {chunk} tokens needs block tables at least {pad_pages} pages wide")
        self.decode_scratch, self.chunk_scratch = decode_scratch[:decode], tuple(chunk_scratch[:pad_pages])
        tokens, rows = decode + chunk, decode + chunks + 1
        self.tokens, self.rows = tokens, rows
        pin = device.type == "cuda"

        def pair(shape, dtype):
            host = torch.zeros(shape, dtype=dtype)
            return torch.zeros(shape, dtype=dtype, device=device), (host.pin_memory() if pin else host)

        self.input_ids, self.host_ids = pair((tokens,), torch.int64)
        self.token_to_sequence, self.host_tok2seq = pair((tokens,), torch.int32)
        self.token_positions, self.host_tokpos = pair((tokens,), torch.int32)
        self.block_tables, self.host_tables = pair((rows, table_width), torch.int32)
        self.decode_lengths, self.host_lengths = pair((max(decode, 1),), torch.int32)
        self.cu_seqlens, self.host_cu = pair((chunks + 2,), torch.int32)
        self.kv_lens, self.host_kv = pair((chunks + 1,), torch.int32)
        self.logit_rows, self.host_logit_rows = pair((decode + chunks,), torch.int64)
        self.output_tokens = torch.zeros(decode + chunks, dtype=torch.int64, device=device)
        self.host_tokens = torch.zeros(decode + chunks, dtype=torch.int64)
        if pin:
            self.host_tokens = self.host_tokens.pin_memory()
        self.pack([], [], [], [])

    def pack(self, decode_ids, decode_lengths, decode_blocks, chunks) -> int:
        """``decode_*``: the live decode rows (token, length including it, page ids).  ``chunks``: a list of
        ``(token ids, start position, page ids)`` with at most ``self.chunks`` entries and ``self.chunk``
        tokens in total.  Everything else becomes padding.  Returns the bytes copied to the device."""

        live, page = len(decode_ids), self.page
        total = sum(len(c[0]) for c in chunks)
        if live > self.decode or len(chunks) > self.chunks or total > self.chunk:
            raise ValueError("the step does not fit this mixed bucket")
        ids, seq, pos = self.host_ids, self.host_tok2seq, self.host_tokpos
        tables, lengths = self.host_tables, self.host_lengths
        tables.fill_(-1)
        for row in range(self.decode):
            if row < live:
                blocks, length = decode_blocks[row], int(decode_lengths[row])
                if length < 1 or len(blocks) > self.table_width or len(blocks) * page < length:
                    raise ValueError("decode position/block row exceeds the fixed table capacity")
                ids[row], seq[row], pos[row], lengths[row] = int(decode_ids[row]), row, length - 1, length
                tables[row, :len(blocks)] = torch.tensor([int(b) for b in blocks], dtype=torch.int32)
            else:
                ids[row], seq[row], pos[row], lengths[row] = 0, row, 0, 1
                tables[row, 0] = self.decode_scratch[row]
        cursor = self.decode
        self.host_cu[0] = 0
        for index in range(self.chunks):
            if index < len(chunks):
                tokens, start, blocks = chunks[index]
                count = len(tokens)
                if count < 1 or len(blocks) > self.table_width or len(blocks) * page < start + count:
                    raise ValueError("chunk position/block row exceeds the fixed table capacity")
                ids[cursor:cursor + count] = torch.tensor([int(t) for t in tokens], dtype=torch.int64)
                seq[cursor:cursor + count] = self.decode + index
                pos[cursor:cursor + count] = torch.arange(start, start + count, dtype=torch.int32)
                tables[self.decode + index, :len(blocks)] = torch.tensor([int(b) for b in blocks], dtype=torch.int32)
                self.host_kv[index] = start + count
                cursor += count
                self.host_logit_rows[self.decode + index] = cursor - 1
            else:
                self.host_kv[index] = 0
                self.host_logit_rows[self.decode + index] = 0
            self.host_cu[index + 1] = cursor - self.decode
        padding = self.tokens - cursor
        pad_row = self.decode + self.chunks
        ids[cursor:] = 0
        seq[cursor:] = pad_row
        pos[cursor:] = torch.arange(padding, dtype=torch.int32)
        tables[pad_row, :len(self.chunk_scratch)] = torch.tensor(self.chunk_scratch, dtype=torch.int32)
        self.host_kv[self.chunks] = padding
        self.host_cu[self.chunks + 1] = self.tokens - self.decode
        self.host_logit_rows[:self.decode] = torch.arange(self.decode, dtype=torch.int64)
        copied = 0
        for device_tensor, host_tensor in ((self.input_ids, ids), (self.token_to_sequence, seq),
                                           (self.token_positions, pos), (self.block_tables, tables),
                                           (self.decode_lengths, lengths), (self.cu_seqlens, self.host_cu),
                                           (self.kv_lens, self.host_kv), (self.logit_rows, self.host_logit_rows)):
            device_tensor.copy_(host_tensor, non_blocking=True)
            copied += host_tensor.numel() * host_tensor.element_size()
        return copied


class Qwen3DecodeRunner:
    """Steps of a Qwen3-shaped FP8 model over paged KV: decode rows, packed prompt chunks or both in one
    flat forward, eager or replayed from CUDA graphs captured per bucket.

    The K/V pool holds ``num_pages`` request pages followed by scratch pages that only padding rows of a
    captured bucket touch (reference: engine/serving/chunked_prefill.py:133-148 - the extra pages are
    exclusively scratch, the request capacity is unchanged): one page per row of the largest decode bucket
    and enough pages for the padding tokens of the largest prompt-chunk bucket.
    """

    def __init__(self, weights: Qwen3Weights, *, num_pages: int, max_batch: int, max_context: int,
                 process_group=None, kv_init: str = "zeros", fused_exchange: bool | None = None,
                 decode_buckets: tuple[int, ...] | None = None, chunk_buckets: tuple[int, ...] = (128, 512),
                 max_chunks: int = 4, kv_dtype: str = "bf16") -> None:
        self.weights, self.shape = weights, weights.shape
        self.device, self.group = weights.device, process_group
        self.tp = weights.tp_size
        shape = self.shape
        self.local_q_heads = shape.q_heads // self.tp
        self.local_kv_heads = shape.kv_heads // self.tp
        self.local_inter = weights.inter_window  # the MLP shard inside its window of whole scale blocks
        self.num_pages, self.max_batch, self.max_context = num_pages, max_batch, max_context
        if decode_buckets is None:
            decode_buckets = tuple(b for b in DEFAULT_DECODE_BUCKETS if b < max_batch) + (max_batch,)
        if not decode_buckets or tuple(sorted(set(decode_buckets))) != tuple(decode_buckets) or decode_buckets[0] < 1:
            raise ValueError("decode_buckets must be non-empty, strictly increasing positive integers")
        self.decode_buckets = tuple(int(b) for b in decode_buckets)
        self.chunk_buckets = tuple(sorted(int(c) for c in chunk_buckets))
        self.max_chunks = int(max_chunks)
        chunk_scratch = -(-max(self.chunk_buckets, default=0) // shape.page)
        self.decode_scratch_pages = tuple(range(num_pages, num_pages + self.decode_buckets[-1]))
        self.chunk_scratch_pages = tuple(range(num_pages + self.decode_buckets[-1],
                                               num_pages + self.decode_buckets[-1] + chunk_scratch))
        self.total_pages = num_pages + self.decode_buckets[-1] + chunk_scratch
        self.table_width = -(-max_context // shape.page)
        layers = len(weights.layers)
        if kv_dtype not in ("bf16", "fp8"):
            raise ValueError("kv_dtype must be 'bf16' or 'fp8'")
        self.kv_dtype = kv_dtype
        self.kv8 = None
        if kv_dtype == "fp8":
            # Opt-in e4m3 K/V pool (one fp32 scale per token and KV head).  Decode rows read it directly;
            # prompt chunks attend bf16 staging copies of their pages.  bf16 stays the default and the parity path.
            if shape.page != 16 or shape.head_dim != 128:
                raise ValueError("the FP8 KV cache needs 16-token pages and head_dim 128")
            self.kv8 = Fp8KvPool(layers, self.total_pages, self.local_kv_heads, self.device)
            self.key_blocks = self.value_blocks = None
            if kv_init == "normal":
                for layer in range(layers):
                    # random e4m3 bytes with the exponent capped (no NaN / huge values) and scales near 1 / 448
                    self.kv8.data[layer].random_(0, 256).bitwise_and_(0xBF)
                    self.kv8.scales[layer].uniform_(0.004, 0.012)
        else:
            pool_shape = (layers, self.total_pages, self.local_kv_heads, shape.page, shape.head_dim)
            self.key_blocks = torch.empty(pool_shape, dtype=torch.bfloat16, device=self.device)
            self.value_blocks = torch.empty(pool_shape, dtype=torch.bfloat16, device=self.device)
            if kv_init == "zeros":
                self.key_blocks.zero_()
                self.value_blocks.zero_()
            elif kv_init == "normal":
                for pool in (self.key_blocks, self.value_blocks):
                    for layer in range(layers):
                        pool[layer].normal_()
        self.rope = rope_table(shape, max_context, self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.scratch = decode_scratch(max(max_batch, self.decode_buckets[-1]), self.local_q_heads,
                                      self.local_kv_heads, shape.head_dim, max_batch * max_context, self.device)
        # (kind, bucket...) -> (graph, buffers): ("decode", rows, advance) or ("mixed", rows, chunk tokens)
        self._graphs: dict[tuple, tuple[torch.cuda.CUDAGraph, object]] = {}
        self._generation = 0  # distinguishes the rows of successive generate() calls
        self.launches_per_step = 0
        # lm_head + greedy sampling: one pass over the tied embedding that never writes the logits
        # (mie_lm_head_argmax) unless MIE_LM_HEAD=cublas; its per-row keys are zero between calls.
        self.fused_lm_head = os.environ.get("MIE_LM_HEAD", "fused") != "cublas"
        self._lm_keys = torch.zeros(256, dtype=torch.int64, device=self.device)
        # Tensor parallel decode: the all-reduce after o_proj / down_proj is fused into the residual add +
        # RMSNorm + quantisation kernel over peer memory unless MIE_TP_EXCHANGE=nccl (or fused_exchange=False).
        if fused_exchange is None:
            fused_exchange = os.environ.get("MIE_TP_EXCHANGE", "fused") != "nccl"
        self.exchange = None
        if self.tp > 1 and fused_exchange:
            # Rows for the largest decode bucket plus the largest prompt-chunk bucket of a mixed step; a longer
            # flat forward (a whole-prompt prefill) sums its partial rows with NCCL instead.
            exchange_rows = max(max_batch, self.decode_buckets[-1]) + max(self.chunk_buckets, default=0)
            self.exchange = PeerExchange(self.tp, weights.tp_rank, exchange_rows, shape.hidden, self.device,
                                         process_group)

    # -- small helpers ------------------------------------------------------------------------

    def _quant_buffers(self, rows: int, width: int) -> tuple[torch.Tensor, torch.Tensor]:
        padded = (width + 15) // 16 * 16
        q = torch.empty(rows, padded, dtype=torch.float8_e4m3fn, device=self.device)
        if padded != width:
            q.view(torch.uint8)[:, width:].zero_()
        return q, torch.empty((width + 127) // 128, rows, dtype=torch.float32, device=self.device)

    def _norm(self, x, weight, residual=None, *, quantize: bool):
        """(normed bf16 or None, summed or None, quantised pair or None)."""

        rows, cols = x.shape
        lib, stream = _lib.load(), _lib.stream_arg(self.device)
        summed = torch.empty_like(x) if residual is not None else None
        if quantize:
            q, scales = self._quant_buffers(rows, cols)
            _lib.check(lib.mie_rms_norm(_lib.ptr(x), x.stride(0), _lib.ptr(residual), _lib.ptr(summed),
                                        _lib.ptr(weight), None, _lib.ptr(q), q.stride(0), _lib.ptr(scales),
                                        scales.stride(0), rows, cols, self.shape.rms_eps, stream))
            return None, summed, (q, scales)
        out = torch.empty_like(x)
        _lib.check(lib.mie_rms_norm(_lib.ptr(x), x.stride(0), _lib.ptr(residual), _lib.ptr(summed),
                                    _lib.ptr(weight), _lib.ptr(out), None, 0, None, 0, rows, cols,
                                    self.shape.rms_eps, stream))
        return out, summed, None

    def _gemm(self, quantized, weight, weight_scale, rows: int, k: int, out: torch.Tensor | None = None) -> torch.Tensor:
        if out is None:
            out = torch.empty(rows, weight.shape[0], dtype=torch.bfloat16, device=self.device)
        sm89_fp8.launch_fp8_gemm(quantized[0], quantized[1], weight, weight_scale, out, rows, k, status=self.status)
        return out

    def _quantize(self, x: torch.Tensor):
        return sm89_fp8.quantize_activation_kmajor(x)

    def _all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp > 1:
            torch.distributed.all_reduce(x, group=self.group)
        return x

    def _silu_mul_quantized(self, gate_up: torch.Tensor, rows: int):
        """SiLU(gate) * up over the two windows of the merged gate_up output, quantised for down_proj."""

        inter = self.local_inter
        q, scales = self._quant_buffers(rows, inter)
        _lib.check(_lib.load().mie_silu_mul(_lib.ptr(gate_up), _lib.ptr(gate_up[:, inter:]), gate_up.stride(0), None,
                                            _lib.ptr(q), q.stride(0), _lib.ptr(scales), scales.stride(0), rows,
                                            inter, _lib.stream_arg(self.device)))
        return q, scales

    def _row_parallel_then_norm(self, quantized, weight, weight_scale, rows: int, k: int, residual, norm_weight,
                                *, quantize: bool):
        """Row-parallel projection, sum over the ranks, residual add and RMSNorm of the sum.  Returns
        ``(normed bf16 or None, new residual, quantised pair or None)`` like ``_norm``.  With the fused exchange
        the new residual is only valid in the rows this rank owns (the only rows it reads again)."""

        ex = self.exchange
        if ex is None or rows > ex.max_rows:
            out = self._all_reduce(self._gemm(quantized, weight, weight_scale, rows, k))
            return self._norm(out, norm_weight, residual, quantize=quantize)
        self._gemm(quantized, weight, weight_scale, rows, k, out=ex.partial[:rows])
        summed = torch.empty_like(residual)
        ex.reduce_norm(rows, residual, summed, norm_weight, self.shape.rms_eps, quantized=quantize, status=self.status)
        if quantize:
            return None, summed, (ex.q[:rows], ex.scales[:, :rows])
        return ex.normed[:rows], summed, None

    def _qkv_post(self, layer_index: int, layer, qkv, queries, positions, token_to_sequence, block_tables,
                  tokens: int, table_rows: int) -> None:
        """q/k RMSNorm + RoPE on the merged qkv rows, K/V rows to their page slots, q rows to ``queries``."""

        shape = self.shape
        if self.kv8 is not None:
            _lib.check(_lib.load().mie_qkv_norm_rope_write_kv8(
                _lib.ptr(qkv), qkv.stride(0), _lib.ptr(layer.q_norm), _lib.ptr(layer.k_norm), _lib.ptr(self.rope),
                int(self.rope.shape[0]), _lib.index_arg(positions), _lib.index_arg(token_to_sequence),
                _lib.index_arg(block_tables), _lib.ptr(queries), _lib.ptr(self.kv8.data[layer_index]),
                self.kv8.page_stride_bytes, _lib.ptr(self.kv8.scales[layer_index]), tokens, self.local_q_heads,
                self.local_kv_heads, self.total_pages, table_rows, int(block_tables.shape[1]), shape.rms_eps,
                _lib.ptr(self.status), _lib.stream_arg(self.device)))
            return
        _lib.check(_lib.load().mie_qkv_norm_rope_write(
            _lib.ptr(qkv), qkv.stride(0), _lib.ptr(layer.q_norm), _lib.ptr(layer.k_norm), _lib.ptr(self.rope),
            int(self.rope.shape[0]), _lib.index_arg(positions), _lib.index_arg(token_to_sequence),
            _lib.index_arg(block_tables), _lib.ptr(queries), _lib.view4_arg(self.key_blocks[layer_index]),
            _lib.view4_arg(self.value_blocks[layer_index]), tokens, self.local_q_heads, self.local_kv_heads,
            shape.page, self.total_pages, table_rows, int(block_tables.shape[1]), shape.rms_eps,
            _lib.ptr(self.status), _lib.stream_arg(self.device)))

    # -- the decode forward -------------------------------------------------------------------

    def decode_forward(self, input_ids: torch.Tensor, sequence_lengths: torch.Tensor,
                       block_tables: torch.Tensor, return_logits: bool = False):
        """One token per request.  ``sequence_lengths`` already counts the new token, which is
        written at position ``length - 1``.  Returns the greedy next token ids ``[batch]`` (int64)."""

        shape, lib = self.shape, _lib.load()
        batch = int(input_ids.shape[0])
        launches_before = lib.mie_launch_count()
        hd, lq = shape.head_dim, self.local_q_heads
        hidden = self.weights.embedding.index_select(0, input_ids)
        positions = sequence_lengths - 1
        scale = 1.0 / math.sqrt(hd)
        layers = self.weights.layers
        _, _, quantized = self._norm(hidden, layers[0].input_norm, quantize=True)
        residual, final = hidden, None
        for index, layer in enumerate(layers):
            qkv = self._gemm(quantized, layer.qkv, layer.qkv_scale, batch, shape.hidden)
            queries = torch.empty(batch, lq, 1, hd, dtype=torch.bfloat16, device=self.device)
            self._qkv_post(index, layer, qkv, queries, positions, None, block_tables, batch, batch)
            attended = torch.empty_like(queries)
            attn_q = self._quant_buffers(batch, lq * hd)
            if self.kv8 is not None:
                launch_decode_attention_kv8(queries, attended, self.kv8.data[index], self.kv8.scales[index],
                                            block_tables, sequence_lengths, None, scale=scale, scratch=self.scratch,
                                            split_policy=1, use_plan=index % PLAN_SLOTS != 0,
                                            plan_slot=index % PLAN_SLOTS, status=self.status, quantized_out=attn_q)
            else:
                launch_decode_attention(queries, attended, self.key_blocks[index], self.value_blocks[index],
                                        block_tables, sequence_lengths, None, scale=scale,
                                        max_total_tokens=batch * self.max_context, scratch=self.scratch,
                                        split_policy=1, use_plan=index % PLAN_SLOTS != 0,
                                        plan_slot=index % PLAN_SLOTS, status=self.status,
                                        quantized_out=attn_q)
            _, residual, quantized = self._row_parallel_then_norm(attn_q, layer.o, layer.o_scale, batch, lq * hd,
                                                                  residual, layer.post_norm, quantize=True)
            gate_up = self._gemm(quantized, layer.gate_up, layer.gate_up_scale, batch, shape.hidden)
            act_q = self._silu_mul_quantized(gate_up, batch)
            last = index + 1 == len(layers)
            next_norm = self.weights.final_norm if last else layers[index + 1].input_norm
            final, residual, quantized = self._row_parallel_then_norm(act_q, layer.down, layer.down_scale, batch,
                                                                      self.local_inter, residual, next_norm,
                                                                      quantize=not last)
        if self.fused_lm_head and not return_logits and batch <= 256:
            tokens = self.greedy_tokens(final)
            self.launches_per_step = int(lib.mie_launch_count() - launches_before)
            return tokens
        logits = torch.matmul(final, self.weights.lm_head.t())
        self.launches_per_step = int(lib.mie_launch_count() - launches_before)
        if self.tp == 1:
            tokens = logits.argmax(dim=-1)
            return (tokens, logits) if return_logits else tokens
        return sharded_greedy_tokens(logits, self.weights.vocab_start, self.tp, self.group)

    def greedy_tokens(self, final: torch.Tensor) -> torch.Tensor:
        """Greedy next tokens of normed hidden rows ``[rows, hidden]`` (rows <= 256): the bf16 product with the
        tied lm_head and its argmax in one pass (reference: engine/model_runner/qwen3_mixed.py:164-174)."""

        lib = _lib.load()
        rows = int(final.shape[0])
        if final.stride(1) != 1 or final.stride(0) % 8 != 0 or final.data_ptr() % 16 != 0:
            final = final.contiguous()
        head = self.weights.lm_head
        tokens = torch.empty(rows, dtype=torch.int64, device=self.device)
        values = torch.empty(rows, dtype=torch.int32, device=self.device) if self.tp > 1 else None
        _lib.check(lib.mie_lm_head_argmax(_lib.ptr(final), final.stride(0), _lib.ptr(head), head.stride(0), rows,
                                          head.shape[0], head.shape[1], self.weights.vocab_start,
                                          _lib.ptr(self._lm_keys), _lib.ptr(tokens), _lib.ptr(values),
                                          _lib.ptr(self.status), _lib.stream_arg(self.device)))
        return sharded_greedy_from_pairs(tokens, values, self.tp, self.group) if self.tp > 1 else tokens

    # -- flat forward: decode rows and packed prompt chunks in one token stream --------------------------

    def mixed_forward(self, input_ids: torch.Tensor, token_to_sequence: torch.Tensor,
                      token_positions: torch.Tensor, block_tables: torch.Tensor, *, decode_rows: int,
                      decode_lengths: torch.Tensor | None, cu_seqlens: torch.Tensor, kv_lens: torch.Tensor,
                      max_query_len: int, logit_rows: torch.Tensor, return_logits: bool = False):
        """One flat ``[tokens]`` forward (reference: engine/model_runner/qwen3_mixed.py:125-178 and the mixed
        branch of the attention adapter, engine/kv_cache/qwen3_paged.py:221-330).

        Tokens ``[0, decode_rows)`` are decode tokens, one per request: token ``i`` belongs to table row ``i``
        and sits at position ``decode_lengths[i] - 1``.  The remaining tokens are prompt chunks packed back to
        back; ``cu_seqlens`` (relative to the first chunk token) and ``kv_lens`` describe them, their table rows
        follow the decode rows, ``token_to_sequence`` / ``token_positions`` place every token's K/V.  Per layer
        the K/V rows of ALL tokens are scattered first, then the decode rows run the paged decode kernel and
        the chunk rows the tiled prefill kernel (causal within the chunk, over the request's cached prefix);
        all other operators run once over the whole stream.  ``logit_rows`` selects the rows that are
        projected to logits; their greedy tokens are returned in that order."""

        shape, lib = self.shape, _lib.load()
        stream = _lib.stream_arg(self.device)
        tokens = int(input_ids.shape[0])
        table_rows = int(block_tables.shape[0])
        chunk_tokens = tokens - decode_rows
        hd, lq = shape.head_dim, self.local_q_heads
        launches_before = lib.mie_launch_count()
        hidden = self.weights.embedding.index_select(0, input_ids)
        scale = 1.0 / math.sqrt(hd)
        layers = self.weights.layers
        # Same layer structure as the decode forward: every residual add + RMSNorm (+ quantisation) is fused
        # with the sum over the ranks that precedes it (the peer-memory exchange when the token count fits its
        # buffers, NCCL all-reduce + the norm kernel otherwise).
        _, _, quantized = self._norm(hidden, layers[0].input_norm, quantize=True)
        residual, normed = hidden, None
        chunk_tables = block_tables[decode_rows:]
        if self.kv8 is not None and chunk_tokens:
            # The chunk kernel reads bf16 pages: per layer, after the writer has quantised the new rows into the
            # FP8 pool, the chunk requests' pages (cached prefix and the chunk itself) are dequantised into a
            # staging set of bf16 pages addressed by a renumbered table, so a chunk attends exactly what the
            # cache holds, as the decode steps after it will.
            staged_ids = chunk_tables.clamp_min(0).flatten().long()
            numbering = torch.arange(staged_ids.numel(), dtype=chunk_tables.dtype, device=self.device)
            chunk_tables = torch.where(chunk_tables >= 0, numbering.view_as(chunk_tables),
                                       torch.full_like(chunk_tables, -1))
        for index, layer in enumerate(layers):
            qkv = self._gemm(quantized, layer.qkv, layer.qkv_scale, tokens, shape.hidden)
            queries = torch.empty(tokens, lq, hd, dtype=torch.bfloat16, device=self.device)
            self._qkv_post(index, layer, qkv, queries, token_positions, token_to_sequence, block_tables, tokens,
                           table_rows)
            attended = torch.empty_like(queries)
            if decode_rows and self.kv8 is not None:
                launch_decode_attention_kv8(queries[:decode_rows].unsqueeze(2), attended[:decode_rows].unsqueeze(2),
                                            self.kv8.data[index], self.kv8.scales[index], block_tables[:decode_rows],
                                            decode_lengths, None, scale=scale, scratch=self.scratch, split_policy=1,
                                            use_plan=index % PLAN_SLOTS != 0, plan_slot=index % PLAN_SLOTS,
                                            status=self.status)
            elif decode_rows:
                launch_decode_attention(queries[:decode_rows].unsqueeze(2), attended[:decode_rows].unsqueeze(2),
                                        self.key_blocks[index], self.value_blocks[index],
                                        block_tables[:decode_rows], decode_lengths, None, scale=scale,
                                        max_total_tokens=decode_rows * self.max_context, scratch=self.scratch,
                                        split_policy=1, use_plan=index % PLAN_SLOTS != 0,
                                        plan_slot=index % PLAN_SLOTS, status=self.status)
            if chunk_tokens:
                if self.kv8 is not None:
                    key_pages, value_pages = self.kv8.dequantized_pages(index, staged_ids)
                else:
                    key_pages, value_pages = self.key_blocks[index], self.value_blocks[index]
                launch_flash_prefill(queries[decode_rows:], attended[decode_rows:], key_pages, value_pages,
                                     chunk_tables, cu_seqlens, kv_lens, max_query_len=max_query_len, scale=scale,
                                     status=self.status)
            attn_q = self._quantize(attended.view(tokens, lq * hd))
            _, residual, quantized = self._row_parallel_then_norm(attn_q, layer.o, layer.o_scale, tokens, lq * hd,
                                                                  residual, layer.post_norm, quantize=True)
            gate_up = self._gemm(quantized, layer.gate_up, layer.gate_up_scale, tokens, shape.hidden)
            act_q = self._silu_mul_quantized(gate_up, tokens)
            last = index + 1 == len(layers)
            next_norm = self.weights.final_norm if last else layers[index + 1].input_norm
            normed, residual, quantized = self._row_parallel_then_norm(act_q, layer.down, layer.down_scale, tokens,
                                                                       self.local_inter, residual, next_norm,
                                                                       quantize=not last)
        final = normed.index_select(0, logit_rows)
        if self.fused_lm_head and not return_logits and final.shape[0] <= 256:
            picked = self.greedy_tokens(final)
            self.launches_per_step = int(lib.mie_launch_count() - launches_before)
            return picked
        logits = torch.matmul(final, self.weights.lm_head.t())
        self.launches_per_step = int(lib.mie_launch_count() - launches_before)
        picked = sharded_greedy_tokens(logits, self.weights.vocab_start, self.tp, self.group)
        return (picked, logits) if return_logits else picked

    def prefill_forward(self, input_ids: torch.Tensor, token_to_sequence: torch.Tensor,
                        token_positions: torch.Tensor, block_tables: torch.Tensor, cu_seqlens: torch.Tensor,
                        kv_lens: torch.Tensor, max_query_len: int, return_logits: bool = False):
        """Flat ``[tokens]`` forward of packed prompt chunks only (reference: engine/model_runner/qwen3_packed.py:29):
        the mixed forward without decode rows; each request's last row is projected to logits.
        Returns the greedy next token of every request ``[requests]``."""

        last_rows = (cu_seqlens[1:].long() - 1).clamp_min(0)
        return self.mixed_forward(input_ids, token_to_sequence, token_positions, block_tables, decode_rows=0,
                                  decode_lengths=None, cu_seqlens=cu_seqlens, kv_lens=kv_lens,
                                  max_query_len=max_query_len, logit_rows=last_rows, return_logits=return_logits)

    def generate(self, prompts: list[list[int]], max_new_tokens: int, *, use_graph: bool = True) -> list[list[int]]:
        """Greedy generation for requests that arrive together (BASELINE configuration 3): one packed
        whole-prompt prefill, then one decode step per new token (a CUDA graph of the bucket that holds the
        batch when ``use_graph``).  Pages are handed out in order from the start of the pool.  Requests that
        arrive and finish at different times go through ``ContinuousBatcher`` instead."""

        shape, device = self.shape, self.device
        batch = len(prompts)
        lengths = [len(p) for p in prompts]
        needed = [-(-(n + max_new_tokens) // shape.page) for n in lengths]
        if sum(needed) > self.num_pages:
            raise ValueError("the KV pool is too small for these requests")
        if max(n + max_new_tokens for n in lengths) > self.max_context:
            raise ValueError("a request is longer than max_context")
        width = self.table_width
        tables = torch.full((batch, width), -1, dtype=torch.int32)
        cursor = 0
        for row, pages in enumerate(needed):
            tables[row, :pages] = torch.arange(cursor, cursor + pages, dtype=torch.int32)
            cursor += pages
        tables_dev = tables.to(device)
        flat = torch.tensor([t for p in prompts for t in p], dtype=torch.int64, device=device)
        tok2seq = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, n in enumerate(lengths)]).to(device)
        tokpos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lengths]).to(device)
        cu = torch.zeros(batch + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(lengths, dtype=torch.int32).cumsum(0)
        kv_lens = torch.tensor(lengths, dtype=torch.int32, device=device)
        bucket = select_bucket(batch, self.decode_buckets) if use_graph and max_new_tokens > 1 else None
        buffers = None
        if bucket is not None:
            # A serving engine captures its buckets once at start-up; capture only touches scratch pages.
            buffers = self.capture(bucket, advance=True)
        next_ids = self.prefill_forward(flat, tok2seq, tokpos, tables_dev, cu.to(device), kv_lens, max(lengths))
        outputs = [[int(t)] for t in next_ids.tolist()]
        current = kv_lens.clone()
        if buffers is not None:
            # The graph feeds its own tokens back, so the steps are queued back to back; every step's tokens
            # are kept on the device and read in one copy at the end (no host round trip between steps).
            # Rows beyond the batch stay padding rows: their length grows with every replay but stays inside
            # their scratch page for up to `page` replays, after which they are reset.
            self._generation += 1
            buffers.pack_rows([(self._generation, row) for row in range(batch)], [0] * batch,
                              [n + 1 for n in lengths],
                              [tables[row, :needed[row]].tolist() for row in range(batch)])
            buffers.input_ids[:batch].copy_(next_ids)
            history = torch.empty(max_new_tokens - 1, batch, dtype=torch.int64, device=device)
            for step in range(max_new_tokens - 1):
                if bucket > batch and step and step % (shape.page - 1) == 0:
                    buffers.sequence_lengths[batch:].fill_(1)
                self.replay(bucket, advance=True)
                history[step].copy_(buffers.output_tokens[:batch])
            for step_tokens in history.tolist():
                for row, token in enumerate(step_tokens):
                    outputs[row].append(int(token))
        else:
            for _ in range(max_new_tokens - 1):
                current = current + 1
                next_ids = self.decode_forward(next_ids, current, tables_dev)
                for row, token in enumerate(next_ids.tolist()):
                    outputs[row].append(int(token))
        self.check_status()
        return outputs

    # -- CUDA graphs -----------------------------------------------------------------------------

    def capture(self, batch: int, table_width: int | None = None, *, advance: bool = False) -> DecodeBuffers:
        """Capture (once) the decode step for a bucket of ``batch`` rows (reference:
        engine/serving/chunked_prefill.py:231-262).  Warm-up and capture run on an all-padding batch, so
        they only touch scratch pages.  With ``advance`` the graph also feeds the sampled tokens back as the
        next inputs and bumps the lengths, so replays need no host work."""

        key = ("decode", batch, bool(advance))
        if key in self._graphs and (table_width is None or self._graphs[key][1].table_width == table_width):
            return self._graphs[key][1]
        if batch > len(self.decode_scratch_pages):
            raise ValueError(f"bucket {batch} exceeds the largest decode bucket {len(self.decode_scratch_pages)}")
        buffers = DecodeBuffers(batch, table_width or self.table_width, self.device, self.decode_scratch_pages,
                                self.shape.page)
        buffers.advance = advance
        self._capture(key, buffers, lambda: self.decode_forward(buffers.input_ids, buffers.sequence_lengths,
                                                                buffers.block_tables), advance)
        return buffers

    def capture_mixed(self, decode: int, chunk: int) -> MixedBuffers:
        """Capture (once) the mixed step for ``decode`` decode rows plus ``chunk`` prompt-chunk tokens."""

        key = ("mixed", decode, chunk)
        if key in self._graphs:
            return self._graphs[key][1]
        buffers = MixedBuffers(decode, chunk, self.max_chunks, self.table_width, self.device,
                               self.decode_scratch_pages, self.chunk_scratch_pages, self.shape.page)

        def forward():
            return self.mixed_forward(buffers.input_ids, buffers.token_to_sequence, buffers.token_positions,
                                      buffers.block_tables, decode_rows=decode,
                                      decode_lengths=buffers.decode_lengths if decode else None,
                                      cu_seqlens=buffers.cu_seqlens, kv_lens=buffers.kv_lens, max_query_len=chunk,
                                      logit_rows=buffers.logit_rows)

        self._capture(key, buffers, forward, False)
        return buffers

    def _capture(self, key, buffers, forward, advance: bool) -> None:
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                forward()
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            tokens = forward()
            buffers.output_tokens.copy_(tokens)
            if advance:
                buffers.input_ids.copy_(tokens)
                buffers.sequence_lengths.add_(1)
        self._graphs[key] = (graph, buffers)

    def replay(self, batch: int, *, advance: bool = False) -> None:
        self._graphs[("decode", batch, bool(advance))][0].replay()

    def step_host(self, batch: int, ids, lengths, tables=None) -> tuple[torch.Tensor, int, int]:
        """End-to-end step from host metadata: H2D, graph replay, D2H of the sampled tokens.
        Returns ``(host tokens, h2d bytes, d2h bytes)``; synchronises the stream."""

        graph, buffers = self._graphs[("decode", batch, False)]
        h2d = buffers.pack(ids, lengths, tables)
        graph.replay()
        buffers.host_tokens.copy_(buffers.output_tokens, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return buffers.host_tokens, h2d, buffers.host_tokens.numel() * 8

    def decode_rows(self, owners, ids, lengths, block_rows) -> tuple[list[int], int, int]:
        """One decode step for the live rows of a continuous batch: the smallest bucket that holds them is
        captured on first use, the rows are packed (padding rows reset, block tables updated incrementally),
        the bucket's graph is replayed and the live rows' tokens are read back (reference:
        engine/serving/chunked_prefill.py:264-298).  Returns ``(tokens, h2d bytes, d2h bytes)``."""

        live = len(owners)
        bucket = select_bucket(live, self.decode_buckets)
        if bucket is None:
            raise ValueError(f"{live} rows exceed the largest decode bucket {self.decode_buckets[-1]}")
        buffers = self.capture(bucket)
        h2d = buffers.pack_rows(owners, ids, lengths, block_rows)
        self._graphs[("decode", bucket, False)][0].replay()
        buffers.host_tokens[:live].copy_(buffers.output_tokens[:live], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return buffers.host_tokens[:live].tolist(), h2d, live * 8

    def mixed_rows(self, decode_ids, decode_lengths, decode_blocks, chunks) -> tuple[list[int], list[int]]:
        """One captured mixed step (see ``MixedBuffers.pack``).  Returns the decode rows' tokens and, per
        chunk, the greedy token after its last row (meaningful when the chunk completes its prompt)."""

        live, total = len(decode_ids), sum(len(c[0]) for c in chunks)
        decode = select_bucket(live, self.decode_buckets) if live else 0
        chunk = next((c for c in self.chunk_buckets if c >= total), None)
        if decode is None or chunk is None or len(chunks) > self.max_chunks:
            raise ValueError("the step exceeds the largest mixed bucket")
        buffers = self.capture_mixed(decode, chunk)
        buffers.pack(decode_ids, decode_lengths, decode_blocks, chunks)
        self._graphs[("mixed", decode, chunk)][0].replay()
        buffers.host_tokens.copy_(buffers.output_tokens, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        tokens = buffers.host_tokens.tolist()
        return tokens[:live], tokens[decode:decode + len(chunks)]

    def release_graphs(self) -> None:
        """Drop every captured graph (they hold pointers into the pools, the exchange and NCCL)."""

        self._graphs.clear()

    def check_status(self) -> None:
        _lib.raise_for_status(self.status)


__all__ = ["DEFAULT_DECODE_BUCKETS", "DecodeBuffers", "LayerWeights", "MixedBuffers", "PADDING", "Qwen3DecodeRunner",
           "Qwen3Shape", "Qwen3Weights", "scale_window", "select_bucket", "shard_bounds",
           "quantize_weight_blocks", "rope_table", "sharded_greedy_from_pairs", "sharded_greedy_tokens"]
