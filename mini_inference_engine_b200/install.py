"""Rebind the reference engine's hot-path operators to this library.

The reference has no plugin registry: its kernels are plain functions that callers import by name
(``from .triton_paged_attention import triton_paged_decode_attention`` and so on), so a drop-in has to
replace the attribute in the defining module AND in every module that imported it by name.
``install(minillm_l4)`` walks that list; ``uninstall`` restores the originals.

    import minillm_l4                       # the reference package
    import mini_inference_engine_b200 as mie
    mie.install.install(minillm_l4)

After this the reference's model runner, KV cache, step planner and serving scheduler run unchanged on the
sm_100a kernels.
"""

from __future__ import annotations

import importlib
import sys
from types import ModuleType

from .engine.kernels import fused, merged_projections, sm89_fp8
from .engine.kv_cache import (
    decode_metadata,
    triton_flash_prefill,
    triton_packed_attention,
    triton_packed_kv,
    triton_paged_attention,
    triton_paged_kv,
    triton_tc_decode,
)

# reference module (relative to the package) -> replacement module and the names it takes over
_DEFINING = {
    "engine.kv_cache.triton_paged_attention": (triton_paged_attention, triton_paged_attention.__all__),
    "engine.kv_cache.triton_tc_decode": (triton_tc_decode, triton_tc_decode.__all__),
    "engine.kv_cache.triton_paged_kv": (triton_paged_kv, triton_paged_kv.__all__),
    "engine.kv_cache.triton_packed_kv": (triton_packed_kv, triton_packed_kv.__all__),
    "engine.kv_cache.triton_flash_prefill": (triton_flash_prefill, triton_flash_prefill.__all__),
    "engine.kv_cache.triton_packed_attention": (triton_packed_attention, triton_packed_attention.__all__),
    "engine.kv_cache.decode_metadata": (decode_metadata, decode_metadata.__all__),
    "engine.kernels.sm89_fp8": (sm89_fp8, sm89_fp8.__all__),
    "engine.kernels.fused": (fused, ["rms_norm", "silu_mul", "apply_rotary_pos_emb", "fused_kernels_available"]),
    "engine.kernels.merged_projections": (merged_projections, ["project_qkv", "project_gate_up"]),
}

# Modules of the reference that bind those operators by name at import time
# (engine/kv_cache/paged_attention.py:27-34, kv_cache/__init__.py:22-31, qwen3_paged.py:13-26,
#  serving/chunked_prefill.py:14-22, serving/continuous_prefix.py:12-16, serving/prefix_cache.py:11-17,
#  engine/kernels/__init__.py:3).
_IMPORTERS = (
    "engine.kv_cache",
    "engine.kv_cache.paged_attention",
    "engine.kv_cache.qwen3_paged",
    "engine.kernels",
    "engine.serving.chunked_prefill",
    "engine.serving.continuous_prefix",
    "engine.serving.prefix_cache",
)

_saved: list[tuple[ModuleType, str, object]] = []


def _module(package: ModuleType, relative: str) -> ModuleType | None:
    name = f"{package.__name__}.{relative}"
    if name in sys.modules:
        return sys.modules[name]
    try:
        return importlib.import_module(name)
    except ImportError:
        return None


def install(reference_package: ModuleType) -> int:
    """Point every hot-path operator of ``reference_package`` at this library; returns the rebind count."""

    if _saved:
        return len(_saved)
    replacements: dict[int, object] = {}
    for relative, (ours, names) in _DEFINING.items():
        module = _module(reference_package, relative)
        if module is None:
            continue
        for name in names:
            if hasattr(module, name) and hasattr(ours, name):
                original = getattr(module, name)
                replacements[id(original)] = getattr(ours, name)
                _saved.append((module, name, original))
                setattr(module, name, getattr(ours, name))
    for relative in _IMPORTERS:
        module = _module(reference_package, relative)
        if module is None:
            continue
        for name, value in list(vars(module).items()):
            if callable(value) and id(value) in replacements:
                _saved.append((module, name, value))
                setattr(module, name, replacements[id(value)])
    return len(_saved)


def uninstall() -> None:
    while _saved:
        module, name, original = _saved.pop()
        setattr(module, name, original)


__all__ = ["install", "uninstall"]
