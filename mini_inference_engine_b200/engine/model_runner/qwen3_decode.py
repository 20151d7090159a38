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


class Qwen3Weights:
    """Seeded random-init weights in the checkpoint's format, sharded for one tensor-parallel rank.

    Every rank draws the full tensors from the same per-layer seed and keeps its
    slice, so all ranks of a group hold consistent shards.  Shards are quantised
    on their own 128x128 block grid.
    """

    def __init__(self, shape: Qwen3Shape, device: torch.device, *, seed: int = 0, tp_rank: int = 0,
                 tp_size: int = 1, layers: int | None = None) -> None:
        if shape.kv_heads % tp_size or shape.q_heads % tp_size or shape.vocab % tp_size:
            raise ValueError("tensor-parallel size must divide the head counts and the vocabulary")
        self.shape, self.device, self.tp_rank, self.tp_size = shape, device, tp_rank, tp_size
        d, hd = shape.hidden, shape.head_dim
        q_rows, kv_rows, inter = shape.q_heads * hd, shape.kv_heads * hd, shape.intermediate
        if inter % tp_size or (inter // tp_size) % 8:
            raise ValueError("tensor-parallel size must divide the MLP width into multiples of 8")

        def shard(n: int) -> slice:
            return slice(n // tp_size * tp_rank, n // tp_size * (tp_rank + 1))

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
            qkv = torch.cat([wq[shard(q_rows)], wk[shard(kv_rows)], wv[shard(kv_rows)]])
            gate_up = torch.cat([wg[shard(inter)], wu[shard(inter)]])
            qkv8, qkv_s = quantize_weight_blocks(qkv)
            o8, o_s = quantize_weight_blocks(wo[:, shard(q_rows)])
            gu8, gu_s = quantize_weight_blocks(gate_up)
            d8, d_s = quantize_weight_blocks(wd[:, shard(inter)])
            self.layers.append(LayerWeights(
                qkv8, qkv_s, o8, o_s, gu8, gu_s, d8, d_s,
                norm_weight(generator, d), norm_weight(generator, d),
                norm_weight(generator, hd), norm_weight(generator, hd),
            ))
            del wq, wk, wv, wo, wg, wu, wd, qkv, gate_up
        generator = torch.Generator(device=device).manual_seed(seed * 100003 + 99991)
        self.embedding = (torch.randn(shape.vocab, d, generator=generator, device=device, dtype=torch.float32)
                          * 0.02).to(torch.bfloat16)
        self.final_norm = norm_weight(generator, d)
        # Tied lm_head, vocabulary-sharded: this rank scores rows [vocab_start, vocab_start + vocab / tp).
        self.vocab_start = shape.vocab // tp_size * tp_rank
        self.lm_head = self.embedding[shard(shape.vocab)]

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


class DecodeBuffers:
    """Static device buffers of one decode-graph bucket (reference: engine/serving/decode_graph.py:36-96):
    ids, lengths (including the new token), block tables and output tokens keep their addresses across replays."""

    def __init__(self, batch: int, table_width: int, device: torch.device) -> None:
        self.batch, self.table_width = batch, table_width
        self.advance = False  # True when the captured graph feeds its tokens back and bumps the lengths
        self.input_ids = torch.zeros(batch, dtype=torch.int64, device=device)
        self.sequence_lengths = torch.ones(batch, dtype=torch.int32, device=device)
        self.block_tables = torch.zeros(batch, table_width, dtype=torch.int32, device=device)
        self.output_tokens = torch.zeros(batch, dtype=torch.int64, device=device)
        # Pinned host mirrors for the end-to-end path.
        self.host_ids = torch.zeros(batch, dtype=torch.int64).pin_memory()
        self.host_lengths = torch.ones(batch, dtype=torch.int32).pin_memory()
        self.host_tables = torch.zeros(batch, table_width, dtype=torch.int32).pin_memory()
        self.host_tokens = torch.zeros(batch, dtype=torch.int64).pin_memory()

    def pack(self, ids, lengths, tables=None) -> int:
        """Copy one step's host metadata to the device (async, pinned). Returns the bytes copied."""

        self.host_ids.copy_(torch.as_tensor(ids, dtype=torch.int64))
        self.host_lengths.copy_(torch.as_tensor(lengths, dtype=torch.int32))
        self.input_ids.copy_(self.host_ids, non_blocking=True)
        self.sequence_lengths.copy_(self.host_lengths, non_blocking=True)
        copied = self.host_ids.numel() * 8 + self.host_lengths.numel() * 4
        if tables is not None:
            self.host_tables.copy_(torch.as_tensor(tables, dtype=torch.int32))
            self.block_tables.copy_(self.host_tables, non_blocking=True)
            copied += self.host_tables.numel() * 4
        return copied


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


class Qwen3DecodeRunner:
    """Decode steps of a Qwen3-shaped FP8 model over paged KV, eager or as a CUDA graph."""

    def __init__(self, weights: Qwen3Weights, *, num_pages: int, max_batch: int, max_context: int,
                 process_group=None, kv_init: str = "zeros", fused_exchange: bool | None = None) -> None:
        self.weights, self.shape = weights, weights.shape
        self.device, self.group = weights.device, process_group
        self.tp = weights.tp_size
        shape = self.shape
        self.local_q_heads = shape.q_heads // self.tp
        self.local_kv_heads = shape.kv_heads // self.tp
        self.local_inter = shape.intermediate // self.tp
        self.num_pages, self.max_batch, self.max_context = num_pages, max_batch, max_context
        layers = len(weights.layers)
        pool_shape = (layers, num_pages, self.local_kv_heads, shape.page, shape.head_dim)
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
        self.scratch = decode_scratch(max_batch, self.local_q_heads, self.local_kv_heads, shape.head_dim,
                                      max_batch * max_context, self.device)
        self._graphs: dict[int, tuple[torch.cuda.CUDAGraph, DecodeBuffers]] = {}
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
            self.exchange = PeerExchange(self.tp, weights.tp_rank, max_batch, shape.hidden, self.device, process_group)

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

    def _row_parallel_then_norm(self, quantized, weight, weight_scale, rows: int, k: int, residual, norm_weight,
                                *, quantize: bool):
        """Row-parallel projection, sum over the ranks, residual add and RMSNorm of the sum.  Returns
        ``(normed bf16 or None, new residual, quantised pair or None)`` like ``_norm``.  With the fused exchange
        the new residual is only valid in the rows this rank owns (the only rows it reads again)."""

        ex = self.exchange
        if ex is None:
            out = self._all_reduce(self._gemm(quantized, weight, weight_scale, rows, k))
            return self._norm(out, norm_weight, residual, quantize=quantize)
        self._gemm(quantized, weight, weight_scale, rows, k, out=ex.partial[:rows])
        summed = torch.empty_like(residual)
        ex.reduce_norm(rows, residual, summed, norm_weight, self.shape.rms_eps, quantized=quantize, status=self.status)
        if quantize:
            return None, summed, (ex.q[:rows], ex.scales[:, :rows])
        return ex.normed[:rows], summed, None

    # -- the decode forward -------------------------------------------------------------------

    def decode_forward(self, input_ids: torch.Tensor, sequence_lengths: torch.Tensor,
                       block_tables: torch.Tensor, return_logits: bool = False):
        """One token per request.  ``sequence_lengths`` already counts the new token, which is
        written at position ``length - 1``.  Returns the greedy next token ids ``[batch]`` (int64)."""

        shape, lib = self.shape, _lib.load()
        stream = _lib.stream_arg(self.device)
        batch = int(input_ids.shape[0])
        launches_before = lib.mie_launch_count()
        hd, lq, lkv = shape.head_dim, self.local_q_heads, self.local_kv_heads
        hidden = self.weights.embedding.index_select(0, input_ids)
        positions = sequence_lengths - 1
        scale = 1.0 / math.sqrt(hd)
        layers = self.weights.layers
        _, _, quantized = self._norm(hidden, layers[0].input_norm, quantize=True)
        residual, final = hidden, None
        for index, layer in enumerate(layers):
            qkv = self._gemm(quantized, layer.qkv, layer.qkv_scale, batch, shape.hidden)
            queries = torch.empty(batch, lq, 1, hd, dtype=torch.bfloat16, device=self.device)
            _lib.check(lib.mie_qkv_norm_rope_write(
                _lib.ptr(qkv), qkv.stride(0), _lib.ptr(layer.q_norm), _lib.ptr(layer.k_norm), _lib.ptr(self.rope),
                int(self.rope.shape[0]), _lib.index_arg(positions), _lib.index_arg(None),
                _lib.index_arg(block_tables), _lib.ptr(queries), _lib.view4_arg(self.key_blocks[index]),
                _lib.view4_arg(self.value_blocks[index]), batch, lq, lkv, shape.page, self.num_pages, batch,
                int(block_tables.shape[1]), shape.rms_eps, _lib.ptr(self.status), stream))
            attended = torch.empty_like(queries)
            attn_q = self._quant_buffers(batch, lq * hd)
            launch_decode_attention(queries, attended, self.key_blocks[index], self.value_blocks[index],
                                    block_tables, sequence_lengths, None, scale=scale,
                                    max_total_tokens=batch * self.max_context, scratch=self.scratch,
                                    split_policy=1, use_plan=index % PLAN_SLOTS != 0,
                                    plan_slot=index % PLAN_SLOTS, status=self.status,
                                    quantized_out=attn_q)
            _, residual, quantized = self._row_parallel_then_norm(attn_q, layer.o, layer.o_scale, batch, lq * hd,
                                                                  residual, layer.post_norm, quantize=True)
            gate_up = self._gemm(quantized, layer.gate_up, layer.gate_up_scale, batch, shape.hidden)
            inter = self.local_inter
            if inter % 128 == 0:
                q, scales = self._quant_buffers(batch, inter)
                _lib.check(lib.mie_silu_mul(_lib.ptr(gate_up), _lib.ptr(gate_up[:, inter:]), gate_up.stride(0), None,
                                            _lib.ptr(q), q.stride(0), _lib.ptr(scales), scales.stride(0), batch,
                                            inter, stream))
                act_q = (q, scales)
            else:
                act = torch.empty(batch, inter, dtype=torch.bfloat16, device=self.device)
                _lib.check(lib.mie_silu_mul(_lib.ptr(gate_up), _lib.ptr(gate_up[:, inter:]), gate_up.stride(0),
                                            _lib.ptr(act), None, 0, None, 0, batch, inter, stream))
                act_q = self._quantize(act)
            last = index + 1 == len(layers)
            next_norm = self.weights.final_norm if last else layers[index + 1].input_norm
            final, residual, quantized = self._row_parallel_then_norm(act_q, layer.down, layer.down_scale, batch, inter,
                                                                      residual, next_norm, quantize=not last)
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

    # -- packed prefill (whole prompts or chunks over a cached prefix) ----------------------------------

    def prefill_forward(self, input_ids: torch.Tensor, token_to_sequence: torch.Tensor,
                        token_positions: torch.Tensor, block_tables: torch.Tensor, cu_seqlens: torch.Tensor,
                        kv_lens: torch.Tensor, max_query_len: int, return_logits: bool = False):
        """Flat ``[tokens]`` forward of packed prompt chunks (reference: engine/model_runner/qwen3_packed.py:29,
        qwen3_mixed.py:125): K/V of every token are scattered to their pages, attention is causal within a chunk
        and sees the request's cached prefix, and only each request's last row is projected to logits.
        Returns the greedy next token of every request ``[requests]``."""

        from ..kv_cache.triton_flash_prefill import triton_flash_prefill_attention

        shape, lib = self.shape, _lib.load()
        stream = _lib.stream_arg(self.device)
        tokens = int(input_ids.shape[0])
        requests = int(kv_lens.shape[0])
        hd, lq, lkv = shape.head_dim, self.local_q_heads, self.local_kv_heads
        hidden = self.weights.embedding.index_select(0, input_ids)
        residual, mlp_out = None, None
        scale = 1.0 / math.sqrt(hd)
        for index, layer in enumerate(self.weights.layers):
            if index == 0:
                _, _, quantized = self._norm(hidden, layer.input_norm, quantize=True)
                residual = hidden
            else:
                _, residual, quantized = self._norm(mlp_out, layer.input_norm, residual, quantize=True)
            qkv = self._gemm(quantized, layer.qkv, layer.qkv_scale, tokens, shape.hidden)
            queries = torch.empty(tokens, lq, hd, dtype=torch.bfloat16, device=self.device)
            _lib.check(lib.mie_qkv_norm_rope_write(
                _lib.ptr(qkv), qkv.stride(0), _lib.ptr(layer.q_norm), _lib.ptr(layer.k_norm), _lib.ptr(self.rope),
                int(self.rope.shape[0]), _lib.index_arg(token_positions), _lib.index_arg(token_to_sequence),
                _lib.index_arg(block_tables), _lib.ptr(queries), _lib.view4_arg(self.key_blocks[index]),
                _lib.view4_arg(self.value_blocks[index]), tokens, lq, lkv, shape.page, self.num_pages, requests,
                int(block_tables.shape[1]), shape.rms_eps, _lib.ptr(self.status), stream))
            attended = triton_flash_prefill_attention(queries, self.key_blocks[index], self.value_blocks[index],
                                                      block_tables, cu_seqlens, kv_lens,
                                                      max_query_len=max_query_len, scale=scale)
            attn_q = self._quantize(attended.view(tokens, lq * hd))
            attn_out = self._all_reduce(self._gemm(attn_q, layer.o, layer.o_scale, tokens, lq * hd))
            _, residual, quantized = self._norm(attn_out, layer.post_norm, residual, quantize=True)
            gate_up = self._gemm(quantized, layer.gate_up, layer.gate_up_scale, tokens, shape.hidden)
            inter = self.local_inter
            act = torch.empty(tokens, inter, dtype=torch.bfloat16, device=self.device)
            _lib.check(lib.mie_silu_mul(_lib.ptr(gate_up), _lib.ptr(gate_up[:, inter:]), gate_up.stride(0),
                                        _lib.ptr(act), None, 0, None, 0, tokens, inter, stream))
            mlp_out = self._all_reduce(self._gemm(self._quantize(act), layer.down, layer.down_scale, tokens, inter))
        last_rows = (cu_seqlens[1:].long() - 1).clamp_min(0)
        final, _, _ = self._norm(mlp_out.index_select(0, last_rows), self.weights.final_norm,
                                 residual.index_select(0, last_rows), quantize=False)
        if self.fused_lm_head and not return_logits and final.shape[0] <= 256:
            return self.greedy_tokens(final)
        logits = torch.matmul(final, self.weights.lm_head.t())
        picked = sharded_greedy_tokens(logits, self.weights.vocab_start, self.tp, self.group)
        return (picked, logits) if return_logits else picked

    def generate(self, prompts: list[list[int]], max_new_tokens: int, *, use_graph: bool = True) -> list[list[int]]:
        """Greedy continuous-batching generation for requests that arrive together (BASELINE configuration 3):
        one packed whole-prompt prefill, then one decode step per new token (a CUDA graph when ``use_graph``).
        Pages are handed out in order from the start of the pool."""

        shape, device = self.shape, self.device
        batch = len(prompts)
        lengths = [len(p) for p in prompts]
        needed = [-(-(n + max_new_tokens) // shape.page) for n in lengths]
        if sum(needed) > self.num_pages:
            raise ValueError("the KV pool is too small for these requests")
        width = max(needed)
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
        buffers = None
        if use_graph and max_new_tokens > 1:
            # A graph captured for this batch size and table width by an earlier call is reused (a serving
            # engine captures once at start-up).  Capture runs throw-away steps that write position 0 of page
            # 0, so it happens before the prompt is written.
            cached = self._graphs.get(batch)
            if cached is not None and cached[1].advance and cached[1].block_tables.shape[1] == width:
                buffers = cached[1]
            else:
                buffers = self.capture(batch, width, advance=True)
        next_ids = self.prefill_forward(flat, tok2seq, tokpos, tables_dev, cu.to(device), kv_lens, max(lengths))
        outputs = [[int(t)] for t in next_ids.tolist()]
        current = kv_lens.clone()
        if buffers is not None:
            buffers.input_ids.copy_(next_ids)
            buffers.block_tables.copy_(tables_dev)
            buffers.sequence_lengths.copy_(current + 1)
        if buffers is not None:
            # The graph feeds its own tokens back, so the steps are queued back to back; every step's tokens
            # are kept on the device and read in one copy at the end (no host round trip between steps).
            history = torch.empty(max_new_tokens - 1, batch, dtype=torch.int64, device=device)
            for step in range(max_new_tokens - 1):
                self.replay(batch)
                history[step].copy_(buffers.output_tokens)
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

    # -- CUDA graph ------------------------------------------------------------------------------

    def capture(self, batch: int, table_width: int, *, advance: bool = False) -> DecodeBuffers:
        """Capture the decode step for ``batch`` rows.  With ``advance`` the graph also feeds the
        sampled tokens back as the next inputs and bumps the lengths, so replays need no host work."""

        buffers = DecodeBuffers(batch, table_width, self.device)
        buffers.advance = advance
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                self.decode_forward(buffers.input_ids, buffers.sequence_lengths, buffers.block_tables)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            tokens = self.decode_forward(buffers.input_ids, buffers.sequence_lengths, buffers.block_tables)
            buffers.output_tokens.copy_(tokens)
            if advance:
                buffers.input_ids.copy_(tokens)
                buffers.sequence_lengths.add_(1)
        self._graphs[batch] = (graph, buffers)
        return buffers

    def replay(self, batch: int) -> None:
        self._graphs[batch][0].replay()

    def step_host(self, batch: int, ids, lengths, tables=None) -> tuple[torch.Tensor, int, int]:
        """End-to-end step from host metadata: H2D, graph replay, D2H of the sampled tokens.
        Returns ``(host tokens, h2d bytes, d2h bytes)``; synchronises the stream."""

        graph, buffers = self._graphs[batch]
        h2d = buffers.pack(ids, lengths, tables)
        graph.replay()
        buffers.host_tokens.copy_(buffers.output_tokens, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return buffers.host_tokens, h2d, buffers.host_tokens.numel() * 8

    def check_status(self) -> None:
        _lib.raise_for_status(self.status)


__all__ = ["DecodeBuffers", "LayerWeights", "Qwen3DecodeRunner", "Qwen3Shape", "Qwen3Weights",
           "quantize_weight_blocks", "rope_table", "sharded_greedy_from_pairs", "sharded_greedy_tokens"]
