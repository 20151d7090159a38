"""Greedy generation of one request with the CPU oracle (helper of the GPU tests, not a test itself)."""

from __future__ import annotations

import torch

from oracle import qwen3_model


def oracle_generate(cpu_weights, shape, prompt, new_tokens: int, kv_image=None):
    """Whole-prompt prefill then ``new_tokens - 1`` decode steps of ONE request on a private page pool.
    Returns ``(tokens, margin)``: ``margin`` is the smallest, over the steps, of the oracle's top-2 logit gap
    divided by the magnitude of its top logit - how decisively the oracle's own arithmetic picks each token.
    ``kv_image`` is handed to both oracle steps (an FP8 KV cache: quantise -> dequantise of every stored row)."""

    page = shape.page
    pages = -(-(len(prompt) + new_tokens) // page)
    layers = len(cpu_weights.layers)
    keys = torch.zeros(layers, pages, shape.kv_heads, page, shape.head_dim, dtype=torch.bfloat16)
    values = torch.zeros_like(keys)
    tables = torch.arange(pages, dtype=torch.int32).view(1, pages)
    n = len(prompt)
    kwargs = dict(q_heads=shape.q_heads, kv_heads=shape.kv_heads, head_dim=shape.head_dim, eps=shape.rms_eps,
                  theta=shape.rope_theta, return_hidden=True, kv_image=kv_image)
    picked, _, logits = qwen3_model.prefill_step(
        cpu_weights, keys, values, torch.tensor(prompt), torch.zeros(n, dtype=torch.int32),
        torch.arange(n, dtype=torch.int32), tables, torch.tensor([0, n], dtype=torch.int32),
        torch.tensor([n], dtype=torch.int32), **kwargs)
    tokens, margin = [int(picked[0])], _margin(logits)
    length = n
    for _ in range(new_tokens - 1):
        length += 1
        picked, _, logits = qwen3_model.decode_step(cpu_weights, keys, values, torch.tensor([tokens[-1]]),
                                                    torch.tensor([length], dtype=torch.int32), tables, **kwargs)
        tokens.append(int(picked[0]))
        margin = min(margin, _margin(logits))
    return tokens, margin


def _margin(logits: torch.Tensor) -> float:
    top2 = logits.float().topk(2, dim=-1).values
    return float(((top2[:, 0] - top2[:, 1]) / top2[:, 0].abs().clamp_min(1e-30)).min())
