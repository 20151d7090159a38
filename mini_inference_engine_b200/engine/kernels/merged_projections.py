"""Merged FP8 projections: q/k/v as one N=6144 GEMM, gate/up as one N=19456 GEMM
(reference: engine/kernels/merged_projections.py:33-170).

The sibling projections of a module read the same activation, so their e4m3
weights and 128x128 block scales are stacked along N once (every piece is a
whole number of 128-row scale blocks, so no scale block straddles two
projections), the activation is quantised once, one GEMM runs, and the
callers get column views of its output.  The original ``nn.Linear``-like
modules keep working: their ``weight`` / ``weight_scale_inv`` become row views
of the stacked storage, so the separate and the merged computation read the
very same bytes and produce the very same bits.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Iterable

import torch

from . import sm89_fp8

QKV = ("q_proj", "k_proj", "v_proj")
GATE_UP = ("gate_proj", "up_proj")

# Which sibling projections are stacked, the attribute the stack is parked under on the owning module, and
# the Transformers class that owns them.
_GROUPS = (
    {"names": QKV, "slot": "_minillm_qkv", "owner": "Qwen3Attention"},
    {"names": GATE_UP, "slot": "_minillm_gate_up", "owner": "Qwen3MLP"},
)
_ATTRS = {group["names"]: group["slot"] for group in _GROUPS}


@dataclass(frozen=True)
class MergedLinear:
    """Stacked weight ``[sum(splits), K]`` e4m3, its scales ``[sum(splits) / 128, K / 128]`` and the rows of
    every piece."""

    weight: torch.Tensor
    weight_scale_inv: torch.Tensor
    splits: tuple[int, ...]
    block_size: tuple[int, int]
    allow_deepgemm: bool = False

    def __call__(self, x: torch.Tensor) -> tuple[torch.Tensor, ...]:
        out = sm89_fp8.sm89_fp8_linear(x, self.weight, self.weight_scale_inv, block_size=list(self.block_size))
        return out.split(self.splits, dim=-1)

    def row_views(self) -> Iterable[tuple[torch.Tensor, torch.Tensor]]:
        """(weight rows, scale rows) of every piece, as views of the stacked storage."""

        row, rows_per_scale = 0, self.block_size[0]
        for rows in self.splits:
            yield (self.weight[row:row + rows],
                   self.weight_scale_inv[row // rows_per_scale:(row + rows) // rows_per_scale])
            row += rows


def merge_weights(weights, scales, block_size=(128, 128)) -> MergedLinear:
    """Concatenate ``[N_i, K]`` e4m3 weights and their ``[N_i/128, K/128]`` scales along N."""

    if any(int(w.shape[0]) % block_size[0] for w in weights):
        raise ValueError("every merged projection must have a multiple of 128 output rows")
    return MergedLinear(torch.cat(list(weights)).contiguous(), torch.cat(list(scales)).contiguous(),
                        tuple(int(w.shape[0]) for w in weights), tuple(block_size))


def _why_not(pieces: list[Any]) -> str | None:
    """Reason the sibling projections cannot be stacked, or None when they can."""

    if any(piece is None for piece in pieces):
        return "a projection is missing"
    lead = pieces[0]
    block = tuple(getattr(lead, "block_size", None) or ())
    if len(block) != 2:
        return "no 2-D scale block size"
    for piece in pieces:
        weight = getattr(piece, "weight", None)
        if weight is None or weight.dtype != torch.float8_e4m3fn:
            return "weight is not e4m3"
        if not isinstance(getattr(piece, "weight_scale_inv", None), torch.Tensor):
            return "no block scales"
        if getattr(piece, "bias", None) is not None or getattr(piece, "activation_scale", None) is not None:
            return "bias or static activation scale"
        if tuple(piece.block_size) != block:
            return "mixed block sizes"
        if weight.shape[1] != lead.weight.shape[1] or weight.device != lead.weight.device:
            return "different input width or device"
        if weight.shape[0] % block[0]:
            return "rows are not whole scale blocks"
    return None


def _point_at(piece: Any, name: str, view: torch.Tensor) -> None:
    """Make ``piece.<name>`` (a parameter or a buffer) the given view."""

    if name in piece._parameters:
        piece._parameters[name] = torch.nn.Parameter(view, requires_grad=False)
    else:
        piece._buffers[name] = view


def _stack(owner: Any, names: tuple[str, ...]) -> MergedLinear | None:
    pieces = [getattr(owner, name, None) for name in names]
    if _why_not(pieces) is not None:
        return None
    merged = merge_weights([piece.weight.data for piece in pieces],
                           [piece.weight_scale_inv.data for piece in pieces],
                           tuple(int(b) for b in pieces[0].block_size))
    for piece, (weight_rows, scale_rows) in zip(pieces, merged.row_views()):
        _point_at(piece, "weight", weight_rows)
        _point_at(piece, "weight_scale_inv", scale_rows)
    return merged


def _project(owner: Any, names: tuple[str, ...], x: torch.Tensor) -> tuple[torch.Tensor, ...]:
    merged = owner.__dict__.get(_ATTRS[names])
    if merged is not None:
        return merged(x)
    return tuple(getattr(owner, name)(x) for name in names)


def project_qkv(attention: Any, hidden_states: torch.Tensor) -> tuple[torch.Tensor, ...]:
    """``(q_proj(x), k_proj(x), v_proj(x))``; column views of one GEMM when merged."""

    return _project(attention, QKV, hidden_states)


def project_gate_up(mlp: Any, x: torch.Tensor) -> tuple[torch.Tensor, ...]:
    """``(gate_proj(x), up_proj(x))``; column views of one GEMM when merged."""

    return _project(mlp, GATE_UP, x)


def install_merged_projections(model: Any, pretune_tokens: int | None = None) -> int:
    """Stack q/k/v of every Qwen3 attention and gate/up of every Qwen3 MLP of ``model``; returns how many
    stacks were made (``pretune_tokens`` is accepted for the reference's signature; nothing is autotuned)."""

    del pretune_tokens
    from transformers.models.qwen3 import modeling_qwen3

    made = 0
    for group in _GROUPS:
        owner_class = getattr(modeling_qwen3, group["owner"])
        for module in model.modules():
            if not isinstance(module, owner_class) or group["slot"] in module.__dict__:
                continue
            merged = _stack(module, group["names"])
            if merged is not None:
                module.__dict__[group["slot"]] = merged  # not a submodule, parameter or buffer
                made += 1
    return made


def uninstall_merged_projections(model: Any) -> None:
    """Forget the stacks (the pieces keep pointing into the stacked storage, which stays valid)."""

    for module in model.modules():
        for group in _GROUPS:
            module.__dict__.pop(group["slot"], None)


def merged_linears(model: Any) -> list[MergedLinear]:
    return [module.__dict__[group["slot"]] for module in model.modules() for group in _GROUPS
            if group["slot"] in module.__dict__]


__all__ = [
    "MergedLinear", "install_merged_projections", "merge_weights", "merged_linears", "project_gate_up",
    "project_qkv", "uninstall_merged_projections",
]
