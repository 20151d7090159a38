"""CPU oracle for the continuous-batching hot path.  TEST INFRASTRUCTURE ONLY.

A restatement, in plain PyTorch on the CPU, of the algorithms the reference
engine (Makireddyvighnesh/mini-inference-engine, paths below are relative to
that project) runs on its torch/CPU path for: paged decode attention, the
KV-cache scatter and block-table gather, chunked-prefill attention over pages,
the FP8 128x128 block-scaled linear, and the fused RMSNorm / SiLU*up / RoPE
glue.  Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU
baseline may import this package; nothing under ``mini_inference_engine_b200``
does, and the product has no CPU fallback.

Pinning: the attention, scatter/gather and glue functions are checked against
outputs of the reference's own code (imported from a checkout of the reference
by ``tests/golden/make_golden.py``; the vectors are committed under
``tests/golden/``) and against the known answers in the reference's tests
(1.5 / 76.0 for causal positions, tests/test_paged_attention.py:178-270).
The FP8 linear has no CPU implementation in the reference (its arithmetic
exists only inside Triton kernels, engine/kernels/sm89_fp8.py:220-398, and the
fallback ``transformers.integrations.finegrained_fp8.fp8_linear`` of the pinned
transformers 5.14.1 is GPU-only and absent from the installed 5.5.0), so
``fp8_linear`` below restates those kernels' arithmetic and is pinned only
against the double-precision dequantised product the reference's kernel benchmark checks against
(benchmarks/commands/run_kernel_track.py:210-217): parity unpinned for the
bit pattern of the FP8 product, pinned for the 1e-2 tolerance.
"""

from __future__ import annotations

import math

import torch

FP8_MAX = 448.0
BLOCK = 128


# ---------------------------------------------------------------------------
# KV scatter / gather  (exact copies)
# ---------------------------------------------------------------------------

def write_decode_kv(key_states, value_states, block_tables, sequence_lengths, key_blocks, value_blocks,
                    query_positions=None):
    """One new K/V row per request -> page ``table[b][pos // page]``, slot ``pos % page``.

    Follows engine/kv_cache/triton_paged_kv.py:20-107 (position from the
    explicit buffer, else ``length - 1``) and, for the destination arithmetic,
    PagedKvCache.write_layer_segment (engine/kv_cache/paged.py:691-740).
    """

    page = key_blocks.shape[2]
    for b in range(key_states.shape[0]):
        pos = int(sequence_lengths[b]) - 1 if query_positions is None else int(query_positions[b])
        block = int(block_tables[b, pos // page])
        key_blocks[block, :, pos % page, :] = key_states[b, :, 0, :]
        value_blocks[block, :, pos % page, :] = value_states[b, :, 0, :]


def write_packed_kv(key_states, value_states, token_to_sequence, token_positions, block_tables, key_blocks,
                    value_blocks):
    """Packed rows -> pages (engine/kv_cache/triton_packed_kv.py:18-104)."""

    page = key_blocks.shape[2]
    for t in range(key_states.shape[2]):
        seq, pos = int(token_to_sequence[t]), int(token_positions[t])
        block = int(block_tables[seq, pos // page])
        key_blocks[block, :, pos % page, :] = key_states[0, :, t, :]
        value_blocks[block, :, pos % page, :] = value_states[0, :, t, :]


def gather_kv(key_blocks, value_blocks, table_row, length):
    """Dense ``[kv_heads, length, dim]`` K and V of one sequence (engine/kv_cache/paged.py:910-944)."""

    page = key_blocks.shape[2]
    pages = -(-length // page)
    ids = table_row[:pages].long()
    keys = key_blocks[ids].permute(1, 0, 2, 3).reshape(key_blocks.shape[1], pages * page, -1)[:, :length]
    values = value_blocks[ids].permute(1, 0, 2, 3).reshape(value_blocks.shape[1], pages * page, -1)[:, :length]
    return keys.contiguous(), values.contiguous()


# ---------------------------------------------------------------------------
# Attention
# ---------------------------------------------------------------------------

def _attend_one_query(query_token, key_blocks, value_blocks, table_row, valid_tokens, scale, groups):
    """Block-wise online softmax of engine/kv_cache/paged_attention.py:147-216.

    QK^T stays in the activation dtype (bf16 bmm), scores/softmax/PV are fp32,
    one page at a time.
    """

    heads, dim = query_token.shape
    page = key_blocks.shape[2]
    kv_for_head = torch.arange(heads) // groups
    running_max = torch.full((heads,), -torch.inf, dtype=torch.float32)
    running_sum = torch.zeros((heads,), dtype=torch.float32)
    running_out = torch.zeros((heads, dim), dtype=torch.float32)
    for logical, start in enumerate(range(0, valid_tokens, page)):
        count = min(page, valid_tokens - start)
        block = int(table_row[logical])
        keys = key_blocks[block, :, :count, :].index_select(0, kv_for_head)
        values = value_blocks[block, :, :count, :].float().index_select(0, kv_for_head)
        scores = torch.bmm(query_token.unsqueeze(1), keys.transpose(1, 2)).squeeze(1).float() * scale
        new_max = torch.maximum(running_max, scores.max(dim=-1).values)
        old_weight = torch.exp(running_max - new_max)
        weights = torch.exp(scores - new_max.unsqueeze(-1))
        running_sum = running_sum * old_weight + weights.sum(dim=-1)
        running_out = running_out * old_weight.unsqueeze(-1) + torch.bmm(weights.unsqueeze(1), values).squeeze(1)
        running_max = new_max
    return running_out / running_sum.clamp_min(torch.finfo(torch.float32).tiny).unsqueeze(-1)


def paged_decode_attention(query, key_blocks, value_blocks, block_tables, sequence_lengths, scale,
                           query_positions=None):
    """``[batch, heads, 1, dim]`` query -> ``[batch, 1, heads, dim]`` (paged_attention.py:221-365, torch backend).

    Row ``b`` reads ``min(length, position + 1)`` tokens
    (engine/kv_cache/triton_paged_attention.py:234-236).
    """

    batch, heads, _, _ = query.shape
    groups = heads // key_blocks.shape[1]
    rows = []
    for b in range(batch):
        length = int(sequence_lengths[b])
        valid = length if query_positions is None else min(length, int(query_positions[b]) + 1)
        rows.append(_attend_one_query(query[b, :, 0, :], key_blocks, value_blocks, block_tables[b], valid,
                                      float(scale), groups).to(query.dtype))
    return torch.stack(rows, dim=0).unsqueeze(1)


def chunked_prefill_attention(query, key_blocks, value_blocks, block_tables, cu_seqlens, kv_lens, scale):
    """Packed varlen causal attention over pages, lower-right aligned.

    Query row ``i`` of request ``r`` sits at position ``kv_len - q_len + i``
    and sees keys ``0..position`` (engine/kv_cache/triton_flash_prefill.py:18-23).
    Computed as the reference's test oracle does: gather the request's K/V and
    take a masked fp32 softmax (tests/test_triton_flash_prefill.py:17-27), which
    is also what gather_layer + aligned_prefill_sdpa compute
    (engine/generation/chunked_prefill.py:23-61) up to bf16 rounding.
    """

    tokens, heads, dim = query.shape
    groups = heads // key_blocks.shape[1]
    out = torch.empty_like(query)
    for r in range(len(kv_lens)):
        start, end = int(cu_seqlens[r]), int(cu_seqlens[r + 1])
        q_len, kv_len = end - start, int(kv_lens[r])
        if q_len == 0:
            continue
        keys, values = gather_kv(key_blocks, value_blocks, block_tables[r], kv_len)
        keys = keys.float().repeat_interleave(groups, dim=0)
        values = values.float().repeat_interleave(groups, dim=0)
        q = query[start:end].float().transpose(0, 1)  # [heads, q_len, dim]
        scores = torch.matmul(q, keys.transpose(1, 2)) * float(scale)
        positions = torch.arange(kv_len - q_len, kv_len).unsqueeze(1)
        mask = torch.arange(kv_len).unsqueeze(0) > positions
        scores = scores.masked_fill(mask.unsqueeze(0), -torch.inf)
        out[start:end] = torch.matmul(torch.softmax(scores, dim=-1), values).transpose(0, 1).to(query.dtype)
    return out


# ---------------------------------------------------------------------------
# FP8 128x128 block-scaled linear
# ---------------------------------------------------------------------------

def quantize_weight(weight_fp32):
    """Per 128x128 block: ``scale = amax / 448``, ``w8 = (w / scale).to(e4m3)`` (the checkpoint's format)."""

    n, k = weight_fp32.shape
    nb, kb = -(-n // BLOCK), -(-k // BLOCK)
    padded = torch.zeros(nb * BLOCK, kb * BLOCK, dtype=torch.float32)
    padded[:n, :k] = weight_fp32
    blocks = padded.view(nb, BLOCK, kb, BLOCK)
    scales = blocks.abs().amax(dim=(1, 3)) / FP8_MAX
    safe = scales.clamp_min(1e-12)
    quantized = (blocks / safe[:, None, :, None]).view(nb * BLOCK, kb * BLOCK)[:n, :k]
    return quantized.to(torch.float8_e4m3fn), scales.contiguous()


def quantize_activation(x2d):
    """Per token, per 128-column group (engine/kernels/sm89_fp8.py:303-332).

    Returns the e4m3 tensor and the RAW fp32 scales (zero for an all-zero group);
    the division uses ``max(scale, 1e-12)``.
    """

    m, k = x2d.shape
    groups = -(-k // BLOCK)
    padded = torch.zeros(m, groups * BLOCK, dtype=torch.float32)
    padded[:, :k] = x2d.float()
    tiles = padded.view(m, groups, BLOCK)
    scales = tiles.abs().amax(dim=-1) / FP8_MAX
    quantized = (tiles / scales.clamp_min(1e-12).unsqueeze(-1)).view(m, groups * BLOCK)[:, :k]
    return quantized.to(torch.float8_e4m3fn), scales.contiguous()


def fp8_linear(x, weight_fp8, weight_scale_inv, bias=None, output_dtype=None):
    """``acc += dot(a8, w8) * a_scale * w_scale`` per 128-wide K block, fp32 accumulate.

    Restates engine/kernels/sm89_fp8.py:265-300 (fused) == :304-332 + :371-398
    (split): K blocks in increasing order, both scales applied to each block's
    fp32 dot, result cast to the activation dtype, bias added afterwards (:528).
    """

    k = x.shape[-1]
    x2d = x.reshape(-1, k)
    a8, a_scale = quantize_activation(x2d)
    n = weight_fp8.shape[0]
    a32, w32 = a8.float(), weight_fp8.float()
    acc = torch.zeros(x2d.shape[0], n, dtype=torch.float32)
    w_scale_rows = weight_scale_inv.repeat_interleave(BLOCK, dim=0)[:n]  # [n, k_blocks]
    for kb in range(-(-k // BLOCK)):
        cols = slice(kb * BLOCK, min(k, (kb + 1) * BLOCK))
        dot = a32[:, cols] @ w32[:, cols].T
        acc += dot * a_scale[:, kb : kb + 1] * w_scale_rows[:, kb].unsqueeze(0)
    out = acc.to(output_dtype or x.dtype).reshape(*x.shape[:-1], n)
    return out if bias is None else out + bias


def dense_fp8_reference(x, weight_fp8, weight_scale_inv):
    """Double-precision product of the bf16 activation with the dequantised weight.

    The accuracy reference BASELINE's GEMM tolerance names
    (benchmarks/commands/run_kernel_track.py:210-217).
    """

    n, k = weight_fp8.shape
    scales = weight_scale_inv.double().repeat_interleave(BLOCK, dim=0)[:n].repeat_interleave(BLOCK, dim=1)[:, :k]
    return x.reshape(-1, k).double() @ (weight_fp8.double() * scales).T


# ---------------------------------------------------------------------------
# Fused glue (the unfused PyTorch / Hugging Face ops the reference replaces)
# ---------------------------------------------------------------------------

def rms_norm(x, weight, eps, residual=None):
    """``Qwen3RMSNorm`` (fp32 variance, ``weight * x.to(input dtype)``); with ``residual``
    returns ``(norm(x + residual), x + residual)`` as engine/kernels/fused.py:165-203 does."""

    summed = x if residual is None else x + residual
    h = summed.float()
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    out = weight * h.to(x.dtype)
    return out if residual is None else (out, summed)


def silu_mul(gate, up):
    """``F.silu(gate) * up`` (engine/kernels/fused.py:217-233)."""

    return torch.nn.functional.silu(gate) * up


def rotate_half(x):
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim=1):
    """Hugging Face rotate-half RoPE (transformers modeling_qwen3.apply_rotary_pos_emb;
    engine/kernels/fused.py:247-262 reproduces it)."""

    cos, sin = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)
    return q * cos + rotate_half(q) * sin, k * cos + rotate_half(k) * sin


def rope_cos_sin(positions, head_dim, theta, dtype=torch.bfloat16):
    """cos/sin tables as HF's ``Qwen3RotaryEmbedding`` builds them (fp32 math, cast at the end)."""

    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    freqs = positions.float().unsqueeze(-1) * inv_freq
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def quantize_kv_rows(rows):
    """FP8 KV cache: one scale per 128-wide K or V row, ``scale = amax / 448`` (raw scale kept, 0 for a zero
    row), ``row / max(scale, 1e-12)`` rounded to e4m3 - the activation quantiser's rule (``quantize_activation``
    above) applied per (token, KV head).  PARITY UNPINNED: the reference has no FP8 KV cache, it only names
    the idea (docs/phase_notes/roofline.md:76).  ``rows``: ``[..., 128]`` bf16.  Returns (e4m3 bytes as uint8
    ``[..., 128]``, fp32 scales ``[...]``)."""

    values = rows.float()
    scales = values.abs().amax(dim=-1) / 448.0
    quantized = (values / scales.clamp_min(1e-12).unsqueeze(-1)).to(torch.float8_e4m3fn)
    return quantized.view(torch.uint8), scales


def dequantize_kv_rows(quantized_u8, scales, dtype=torch.bfloat16):
    """What a reader of the FP8 cache sees, in the cache's former dtype: ``e4m3 * scale`` rounded to ``dtype``."""

    return (quantized_u8.view(torch.float8_e4m3fn).float() * scales.unsqueeze(-1)).to(dtype)


def paged_decode_attention_fp8_kv(query, key_blocks, value_blocks, block_tables, sequence_lengths, scale,
                                  query_positions=None):
    """Oracle of decode attention over an FP8 KV cache: the reference's torch path (``paged_decode_attention``)
    fed the quantise -> dequantise image of the bf16 pages.  Returns the output and the two dequantised pools."""

    k8, k_scales = quantize_kv_rows(key_blocks)
    v8, v_scales = quantize_kv_rows(value_blocks)
    keys = dequantize_kv_rows(k8, k_scales, key_blocks.dtype)
    values = dequantize_kv_rows(v8, v_scales, value_blocks.dtype)
    out = paged_decode_attention(query, keys, values, block_tables, sequence_lengths, scale, query_positions)
    return out, keys, values


def default_scale(head_dim):
    return 1.0 / math.sqrt(head_dim)
