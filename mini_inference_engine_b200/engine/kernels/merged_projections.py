"""Merged FP8 projections: q/k/v as one N=6144 GEMM, gate/up as one N=19456 GEMM
(reference: engine/kernels/merged_projections.py).

Weights and block scales are concatenated along N (split points are multiples
of 128, so no scale block straddles a projection); the original modules'
weights become views of the merged storage and the q/k/v and gate/up results
are column views of one GEMM output.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from . import sm89_fp8

QKV = ("q_proj", "k_proj", "v_proj")
GATE_UP = ("gate_proj", "up_proj")
_ATTRS = {QKV: "_minillm_qkv", GATE_UP: "_minillm_gate_up"}


@dataclass(frozen=True)
class MergedLinear:
    weight: torch.Tensor
    weight_scale_inv: torch.Tensor
    splits: tuple[int, ...]
    block_size: tuple[int, int]
    allow_deepgemm: bool = False


def merge_weights(weights, scales, block_size=(128, 128)) -> MergedLinear:
    """Concatenate ``[N_i, K]`` e4m3 weights and their ``[N_i/128, K/128]`` scales along N."""

    if any(int(w.shape[0]) % block_size[0] for w in weights):
        raise ValueError("every merged projection must have a multiple of 128 output rows")
    return MergedLinear(torch.cat(list(weights)).contiguous(), torch.cat(list(scales)).contiguous(),
                        tuple(int(w.shape[0]) for w in weights), tuple(block_size))


def _mergeable(linears: list[Any]) -> bool:
    first = linears[0]
    block = tuple(getattr(first, "block_size", None) or ())
    if len(block) != 2:
        return False
    for linear in linears:
        weight, scales = getattr(linear, "weight", None), getattr(linear, "weight_scale_inv", None)
        if (weight is None or weight.dtype != torch.float8_e4m3fn or not isinstance(scales, torch.Tensor)
                or getattr(linear, "bias", None) is not None or getattr(linear, "activation_scale", None) is not None
                or tuple(linear.block_size) != block or weight.shape[1] != first.weight.shape[1]
                or weight.shape[0] % block[0] or weight.device != first.weight.device):
            return False
    return True


def _rebind(linear: Any, name: str, value: torch.Tensor) -> None:
    if name in linear._parameters:
        linear._parameters[name] = torch.nn.Parameter(value, requires_grad=False)
    else:
        linear._buffers[name] = value


def _merge(module: Any, names: tuple[str, ...]) -> MergedLinear | None:
    linears = [getattr(module, name, None) for name in names]
    if any(linear is None for linear in linears) or not _mergeable(linears):
        return None
    block = tuple(int(b) for b in linears[0].block_size)
    merged = merge_weights([l.weight.data for l in linears], [l.weight_scale_inv.data for l in linears], block)
    start = 0
    for linear, rows in zip(linears, merged.splits):
        _rebind(linear, "weight", merged.weight[start : start + rows])
        _rebind(linear, "weight_scale_inv", merged.weight_scale_inv[start // block[0] : (start + rows) // block[0]])
        start += rows
    return merged


def _linear(merged: MergedLinear, x: torch.Tensor) -> torch.Tensor:
    return sm89_fp8.sm89_fp8_linear(x, merged.weight, merged.weight_scale_inv, block_size=list(merged.block_size))


def project_qkv(attention: Any, hidden_states: torch.Tensor) -> tuple[torch.Tensor, ...]:
    """``(q_proj(x), k_proj(x), v_proj(x))``; column views of one GEMM when merged."""

    merged = getattr(attention, "_minillm_qkv", None)
    if merged is None:
        return attention.q_proj(hidden_states), attention.k_proj(hidden_states), attention.v_proj(hidden_states)
    return _linear(merged, hidden_states).split(merged.splits, dim=-1)


def project_gate_up(mlp: Any, x: torch.Tensor) -> tuple[torch.Tensor, ...]:
    """``(gate_proj(x), up_proj(x))``; column views of one GEMM when merged."""

    merged = getattr(mlp, "_minillm_gate_up", None)
    if merged is None:
        return mlp.gate_proj(x), mlp.up_proj(x)
    return _linear(merged, x).split(merged.splits, dim=-1)


def install_merged_projections(model: Any, pretune_tokens: int | None = None) -> int:
    """Merge every Qwen3 attention's q/k/v and MLP's gate/up; returns the merge count."""

    del pretune_tokens  # nothing is autotuned
    from transformers.models.qwen3 import modeling_qwen3

    count = 0
    for module in model.modules():
        if isinstance(module, modeling_qwen3.Qwen3Attention):
            names = QKV
        elif isinstance(module, modeling_qwen3.Qwen3MLP):
            names = GATE_UP
        else:
            continue
        if getattr(module, _ATTRS[names], None) is not None:
            continue
        merged = _merge(module, names)
        if merged is not None:
            object.__setattr__(module, _ATTRS[names], merged)
            count += 1
    return count


def uninstall_merged_projections(model: Any) -> None:
    for module in model.modules():
        for attr in _ATTRS.values():
            if attr in module.__dict__:
                object.__delattr__(module, attr)


def merged_linears(model: Any) -> list[MergedLinear]:
    return [module.__dict__[attr] for module in model.modules() for attr in _ATTRS.values()
            if attr in module.__dict__]


__all__ = [
    "MergedLinear", "install_merged_projections", "merge_weights", "merged_linears", "project_gate_up",
    "project_qkv", "uninstall_merged_projections",
]
