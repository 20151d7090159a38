"""CPU oracle of one Qwen3 decode step over paged KV.  TEST INFRASTRUCTURE ONLY.

Restates, with the functions of ``oracle.hot_path``, what the reference engine
computes for a one-token step through Hugging Face's Qwen3 modules with its
paged attention adapter (engine/kv_cache/qwen3_paged.py:191-219: project qkv,
per-head q/k RMSNorm, RoPE, KV write, paged attention, o_proj; decoder layer
order of engine/kernels/fused.py:286-303; logits of the last row and greedy
argmax, engine/serving/chunked_prefill.py:224-229), with every linear replaced
by the FP8 block-scaled restatement.  Only tests, ``smoke()`` and ``bench.py``'s
CPU baseline may import it.
"""

from __future__ import annotations

import math

import torch

from . import hot_path


def decode_step(weights, key_blocks, value_blocks, input_ids, sequence_lengths, block_tables, *, q_heads, kv_heads,
                head_dim, eps, theta, return_hidden=False, all_reduce=None, pick_tokens=None, kv_image=None):
    """``weights``: object with ``layers`` (each with qkv/o/gate_up/down e4m3 weights, ``*_scale`` block
    scales and the four norm vectors), ``embedding`` and ``final_norm``, all on the CPU.
    ``key_blocks`` / ``value_blocks``: ``[layers, pages, kv_heads, page, dim]``, updated in place.
    ``sequence_lengths`` counts the new token.  Returns greedy tokens (and the final hidden rows).

    For a tensor-parallel shard pass the LOCAL head counts, ``all_reduce`` (sums a tensor over the ranks,
    applied after o_proj and down_proj, the only two exchange points) and ``pick_tokens`` (turns this
    rank's vocabulary-sharded logits into global greedy tokens).

    ``kv_image`` (FP8 KV cache, which the reference does not have): a function applied to the new K and V
    rows before they are stored, e.g. quantise -> dequantise, so that the cache holds what an FP8 pool would
    give back."""

    batch = input_ids.shape[0]
    hidden = weights.embedding.index_select(0, input_ids)
    positions = (sequence_lengths - 1).long()
    cos, sin = hot_path.rope_cos_sin(positions.view(batch, 1), head_dim, theta)
    q_width, kv_width = q_heads * head_dim, kv_heads * head_dim
    for index, layer in enumerate(weights.layers):
        residual = hidden
        normed = hot_path.rms_norm(hidden, layer.input_norm, eps)
        qkv = hot_path.fp8_linear(normed, layer.qkv, layer.qkv_scale)
        q, k, v = qkv.split((q_width, kv_width, kv_width), dim=-1)
        q = hot_path.rms_norm(q.reshape(batch, 1, q_heads, head_dim), layer.q_norm, eps).transpose(1, 2)
        k = hot_path.rms_norm(k.reshape(batch, 1, kv_heads, head_dim), layer.k_norm, eps).transpose(1, 2)
        v = v.reshape(batch, 1, kv_heads, head_dim).transpose(1, 2)
        q, k = hot_path.apply_rotary_pos_emb(q, k, cos, sin)
        if kv_image is not None:
            k, v = kv_image(k), kv_image(v)
        hot_path.write_decode_kv(k, v, block_tables, sequence_lengths, key_blocks[index], value_blocks[index])
        attended = hot_path.paged_decode_attention(q, key_blocks[index], value_blocks[index], block_tables,
                                                   sequence_lengths, 1.0 / math.sqrt(head_dim))
        attn_out = hot_path.fp8_linear(attended.reshape(batch, q_width), layer.o, layer.o_scale)
        if all_reduce is not None:
            attn_out = all_reduce(attn_out)
        normed, residual = hot_path.rms_norm(attn_out, layer.post_norm, eps, residual=residual)
        gate_up = hot_path.fp8_linear(normed, layer.gate_up, layer.gate_up_scale)
        inter = gate_up.shape[-1] // 2
        act = hot_path.silu_mul(gate_up[:, :inter], gate_up[:, inter:])
        mlp_out = hot_path.fp8_linear(act, layer.down, layer.down_scale)
        if all_reduce is not None:
            mlp_out = all_reduce(mlp_out)
        hidden = residual + mlp_out
    final = hot_path.rms_norm(hidden, weights.final_norm, eps)
    logits = final @ (weights.lm_head if pick_tokens is not None else weights.embedding).t()
    tokens = logits.argmax(dim=-1) if pick_tokens is None else pick_tokens(logits)
    return (tokens, final, logits) if return_hidden else tokens


def prefill_step(weights, key_blocks, value_blocks, input_ids, token_to_sequence, token_positions, block_tables,
                 cu_seqlens, kv_lens, *, q_heads, kv_heads, head_dim, eps, theta, return_hidden=False, kv_image=None):
    """Packed prompt chunks through the model (engine/model_runner/qwen3_packed.py:29-113; attention adapter
    packed branch engine/kv_cache/qwen3_paged.py:102-189): per layer the new K/V rows are scattered to their
    pages, attention is causal within a chunk over the whole cached prefix, and each request's last row is
    projected to logits.  Returns the greedy next token of every request.  ``kv_image``: as in
    ``decode_step`` (the chunk then attends what an FP8 cache holds of its own rows too)."""

    tokens = input_ids.shape[0]
    hidden = weights.embedding.index_select(0, input_ids)
    cos, sin = hot_path.rope_cos_sin(token_positions.view(1, tokens).long(), head_dim, theta)
    q_width, kv_width = q_heads * head_dim, kv_heads * head_dim
    for index, layer in enumerate(weights.layers):
        residual = hidden
        normed = hot_path.rms_norm(hidden, layer.input_norm, eps)
        qkv = hot_path.fp8_linear(normed, layer.qkv, layer.qkv_scale)
        q, k, v = qkv.split((q_width, kv_width, kv_width), dim=-1)
        q = hot_path.rms_norm(q.reshape(1, tokens, q_heads, head_dim), layer.q_norm, eps).transpose(1, 2)
        k = hot_path.rms_norm(k.reshape(1, tokens, kv_heads, head_dim), layer.k_norm, eps).transpose(1, 2)
        v = v.reshape(1, tokens, kv_heads, head_dim).transpose(1, 2)
        q, k = hot_path.apply_rotary_pos_emb(q, k, cos, sin)
        if kv_image is not None:
            k, v = kv_image(k), kv_image(v)
        hot_path.write_packed_kv(k, v, token_to_sequence, token_positions, block_tables, key_blocks[index],
                                 value_blocks[index])
        attended = hot_path.chunked_prefill_attention(q[0].transpose(0, 1).contiguous(), key_blocks[index],
                                                      value_blocks[index], block_tables, cu_seqlens, kv_lens,
                                                      1.0 / math.sqrt(head_dim))
        attn_out = hot_path.fp8_linear(attended.reshape(tokens, q_width), layer.o, layer.o_scale)
        normed, residual = hot_path.rms_norm(attn_out, layer.post_norm, eps, residual=residual)
        gate_up = hot_path.fp8_linear(normed, layer.gate_up, layer.gate_up_scale)
        inter = gate_up.shape[-1] // 2
        act = hot_path.silu_mul(gate_up[:, :inter], gate_up[:, inter:])
        hidden = residual + hot_path.fp8_linear(act, layer.down, layer.down_scale)
    last_rows = cu_seqlens[1:].long() - 1
    final = hot_path.rms_norm(hidden.index_select(0, last_rows), weights.final_norm, eps)
    logits = final @ weights.embedding.t()
    picked = logits.argmax(dim=-1)
    return (picked, final, logits) if return_hidden else picked

