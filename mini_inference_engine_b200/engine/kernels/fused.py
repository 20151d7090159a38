"""Fused RMSNorm / SiLU*up / RoPE (reference: engine/kernels/fused.py).

Same function names and call signatures as the reference; the kernels are in
``csrc/fused_glue.cu``.  The bf16 rounding points are PyTorch's (fp32 math in
between); the row-sum order of RMSNorm is a plain warp/CTA tree rather than
ATen's, so results agree with the unfused ops to within one bf16 ulp on rare
elements instead of bit for bit.
"""

from __future__ import annotations

from typing import Any

import torch

from ... import _lib


def fused_kernels_available(device: torch.device | str | None = None) -> bool:
    if not torch.cuda.is_available() or (device is not None and torch.device(device).type != "cuda"):
        return False
    _lib.load()
    return True


def _rows_2d(x: torch.Tensor, n_cols: int) -> torch.Tensor | None:
    """``x`` as ``[rows, n_cols]`` without a copy, or None when the rows are not evenly strided."""

    try:
        rows = x.view(-1, n_cols)
    except RuntimeError:
        return None
    return rows if rows.stride(-1) == 1 and rows.stride(0) % 8 == 0 and rows.data_ptr() % 16 == 0 else None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float,
             residual: torch.Tensor | None = None) -> torch.Tensor | tuple[torch.Tensor, torch.Tensor]:
    """``Qwen3RMSNorm(x)``, or ``(norm(x + residual), x + residual)`` (engine/kernels/fused.py:165-203)."""

    n_cols = int(x.shape[-1])
    if n_cols % 4 or n_cols < 128:
        raise ValueError("rms_norm reproduces PyTorch's vectorized reduction: width must be a multiple of 4, >= 128")
    if x.dtype != torch.bfloat16 or not x.is_cuda:
        raise ValueError("rms_norm expects a CUDA bf16 tensor")
    lib = _lib.load()
    stream = _lib.stream_arg(x.device)
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    weight = weight.contiguous()
    rows = _rows_2d(x, n_cols)
    if rows is None and residual is None and n_cols == 128 and x.dim() >= 3 and x.stride(-1) == 1:
        # Per-head rows of a [..., heads, 128] column view of a merged q/k/v output.
        view = x.reshape(-1, int(x.shape[-2]), n_cols) if x.dim() > 3 else x
        if view.stride(-1) == 1 and view.stride(0) % 8 == 0 and view.stride(1) % 8 == 0 and view.data_ptr() % 16 == 0:
            _lib.check(lib.mie_head_rms_norm(_lib.ptr(view), view.stride(0), view.stride(1), int(view.shape[1]),
                                             _lib.ptr(weight), _lib.ptr(out), view.shape[0] * view.shape[1],
                                             float(eps), stream))
            return out
    if rows is None or n_cols % 8 or n_cols > 8192:
        rows = x.contiguous().view(-1, n_cols)
        if n_cols % 8 or n_cols > 8192:
            raise ValueError("rms_norm supports widths that are multiples of 8 up to 8192")
    num_rows = int(rows.shape[0])
    if residual is None:
        _lib.check(lib.mie_rms_norm(_lib.ptr(rows), rows.stride(0), None, None, _lib.ptr(weight), _lib.ptr(out),
                                    None, 0, None, 0, num_rows, n_cols, float(eps), stream))
        return out
    residual_rows = residual.reshape(-1, n_cols).contiguous()
    summed = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    _lib.check(lib.mie_rms_norm(_lib.ptr(rows), rows.stride(0), _lib.ptr(residual_rows), _lib.ptr(summed),
                                _lib.ptr(weight), _lib.ptr(out), None, 0, None, 0, num_rows, n_cols, float(eps),
                                stream))
    return out, summed


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``F.silu(gate) * up`` in one pass (engine/kernels/fused.py:217-233)."""

    n_cols = int(gate.shape[-1])
    gate_rows, up_rows = _rows_2d(gate, n_cols), _rows_2d(up, n_cols)
    if gate_rows is None or up_rows is None or gate_rows.stride() != up_rows.stride() or n_cols % 8:
        gate_rows, up_rows = gate.contiguous().view(-1, n_cols), up.contiguous().view(-1, n_cols)
        if n_cols % 8:
            raise ValueError("silu_mul supports widths that are multiples of 8")
    out = torch.empty(gate.shape, dtype=gate.dtype, device=gate.device)
    _lib.check(_lib.load().mie_silu_mul(_lib.ptr(gate_rows), _lib.ptr(up_rows), gate_rows.stride(0), _lib.ptr(out),
                                        None, 0, None, 0, int(gate_rows.shape[0]), n_cols,
                                        _lib.stream_arg(gate.device)))
    return out


def _rope_one(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    batch, heads, seq, dim = x.shape
    out = torch.empty_like(x)
    _lib.check(_lib.load().mie_rope(_lib.view4_arg(x), _lib.ptr(cos), _lib.ptr(sin),
                                    cos.stride(0) if cos.shape[0] > 1 else 0, cos.stride(1), _lib.view4_arg(out),
                                    batch, heads, seq, dim, _lib.stream_arg(x.device)))
    return out


def _rope_supported(q, k, cos, sin, unsqueeze_dim) -> bool:
    return bool(
        unsqueeze_dim == 1 and q.is_cuda and q.dim() == 4 and k.dim() == 4 and cos.dim() == 3
        and q.dtype == k.dtype == cos.dtype == sin.dtype == torch.bfloat16
        and q.stride(-1) == 1 and k.stride(-1) == 1 and cos.stride(-1) == 1 and sin.stride() == cos.stride()
        and q.shape[-1] % 2 == 0 and cos.shape[0] in (1, q.shape[0]) and cos.shape[1] == q.shape[2]
    )


def apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim=1):
    """Drop-in for ``transformers.models.qwen3.modeling_qwen3.apply_rotary_pos_emb`` (fused.py:247-262)."""

    if not _rope_supported(q, k, cos, sin, unsqueeze_dim):
        raise ValueError("apply_rotary_pos_emb: unsupported layout (bf16 CUDA [B, H, T, D] with [B|1, T, D] cos/sin)")
    return _rope_one(q, cos, sin), _rope_one(k, cos, sin)


# --- Installation on a Hugging Face Qwen3 model -------------------------------------------------
#
# A model is switched over by giving each norm / MLP / decoder-layer module a subclass of its own class
# whose ``forward`` calls the kernels above (``module.__class__`` is swapped, nothing is copied), and is
# switched back by restoring the class.  RoPE is a module-level function in Transformers, bound by name in
# every module that imported it, so it is replaced process-wide in each such module while at least one
# model is installed.

_INSTALLED_FLAG = "_minillm_fused_kernels"


def _width_ok(hidden_states: torch.Tensor) -> bool:
    width = int(hidden_states.shape[-1])
    return hidden_states.is_cuda and hidden_states.dtype == torch.bfloat16 and width % 8 == 0 and 128 <= width <= 8192


class _FusedNorm:
    def forward(self, hidden_states):
        if _width_ok(hidden_states):
            return rms_norm(hidden_states, self.weight, self.variance_epsilon)
        return super().forward(hidden_states)


class _FusedMlp:
    def forward(self, x):
        from .merged_projections import project_gate_up

        if not (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16)):
            return super().forward(x)
        gate, up = project_gate_up(self, x)
        return self.down_proj(silu_mul(gate, up))


class _FusedDecoderLayer:
    """The decoder layer with its post-attention residual add folded into the RMSNorm that follows it."""

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_values=None,
                use_cache=False, position_embeddings=None, **kwargs):
        attended, _ = self.self_attn(
            hidden_states=self.input_layernorm(hidden_states), attention_mask=attention_mask,
            position_ids=position_ids, past_key_values=past_key_values, use_cache=use_cache,
            position_embeddings=position_embeddings, **kwargs)
        norm = self.post_attention_layernorm
        if _width_ok(attended):
            normed, stream = rms_norm(attended, norm.weight, norm.variance_epsilon, residual=hidden_states)
        else:
            stream = hidden_states + attended
            normed = norm(stream)
        return stream + self.mlp(normed)


_SUBCLASS_CACHE: dict[tuple[type, type], type] = {}


def _fused_class(base: type, mixin: type) -> type:
    key = (base, mixin)
    if key not in _SUBCLASS_CACHE:
        _SUBCLASS_CACHE[key] = type(f"Fused{base.__name__}", (mixin, base), {"_mie_plain_class": base})
    return _SUBCLASS_CACHE[key]


def _mixins() -> dict[type, type]:
    from transformers.models.qwen3 import modeling_qwen3 as hf

    return {hf.Qwen3RMSNorm: _FusedNorm, hf.Qwen3MLP: _FusedMlp, hf.Qwen3DecoderLayer: _FusedDecoderLayer}


class _RopeSwitch:
    """Process-wide, reference-counted replacement of ``apply_rotary_pos_emb`` in every module that binds it
    by name: Transformers' Qwen3 module and the paged-attention adapter of whichever reference package is
    imported (its ``engine/kv_cache/qwen3_paged.py`` does ``from ...modeling_qwen3 import apply_rotary_pos_emb``)."""

    def __init__(self) -> None:
        self.users = 0
        self.displaced: list[tuple[Any, Any]] = []  # (module, the function it had)
        self.original: Any = None

    def _targets(self) -> list[Any]:
        import sys

        from transformers.models.qwen3 import modeling_qwen3 as hf

        adapters = [module for name, module in list(sys.modules.items())
                    if name.endswith("engine.kv_cache.qwen3_paged") and module is not None
                    and hasattr(module, "apply_rotary_pos_emb")]
        return [hf, *adapters]

    def entry(self, q, k, cos, sin, unsqueeze_dim=1):
        # Calls this library's kernel cannot take (other dtypes or layouts, tensors of other devices: the
        # patch is process-wide and other models share the symbol) stay with the function that was displaced.
        if _rope_supported(q, k, cos, sin, unsqueeze_dim):
            return apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim)
        return self.original(q, k, cos, sin, unsqueeze_dim)

    def acquire(self) -> None:
        if self.users == 0:
            targets = self._targets()
            self.original = targets[0].apply_rotary_pos_emb
            entry = self.entry  # one function object for every module that binds the name
            for module in targets:
                self.displaced.append((module, module.apply_rotary_pos_emb))
                module.apply_rotary_pos_emb = entry
        self.users += 1

    def release(self) -> None:
        self.users -= 1
        if self.users == 0:
            for module, function in self.displaced:
                module.apply_rotary_pos_emb = function
            self.displaced.clear()


_ROPE = _RopeSwitch()


def warm_fused_kernels(model: Any) -> None:
    """Nothing is compiled at run time here; kept so callers of the reference API need no change."""

    del model
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def install_fused_kernels(model: Any) -> bool:
    """Route a HF Qwen3 model's norms, MLPs, layer adds and RoPE through these kernels
    (reference: engine/kernels/fused.py:350-382).  False, and nothing changed, without a CUDA device."""

    if getattr(model, _INSTALLED_FLAG, False):
        return True
    if not fused_kernels_available(next(model.parameters()).device):
        return False
    mixins = _mixins()
    for module in model.modules():
        if hasattr(type(module), "_mie_plain_class"):
            continue  # shared with a model that is installed already
        for base, mixin in mixins.items():
            if isinstance(module, base):
                module.__class__ = _fused_class(type(module), mixin)
                break
    _ROPE.acquire()
    setattr(model, _INSTALLED_FLAG, True)
    return True


def uninstall_fused_kernels(model: Any) -> None:
    if not getattr(model, _INSTALLED_FLAG, False):
        return
    for module in model.modules():
        plain = getattr(type(module), "_mie_plain_class", None)
        if plain is not None:
            module.__class__ = plain
    _ROPE.release()
    setattr(model, _INSTALLED_FLAG, False)


__all__ = [
    "apply_rotary_pos_emb", "fused_kernels_available", "install_fused_kernels",
    "rms_norm", "silu_mul", "uninstall_fused_kernels", "warm_fused_kernels",
]
