"""Dynamic block-scaled FP8 linear (reference: engine/kernels/sm89_fp8.py).

The module and function names are the reference's (its callers import
``sm89_fp8_linear`` and friends by name), but the kernels behind them are the
sm_100a tcgen05 GEMM and the activation quantiser of ``csrc/fp8_gemm.cu``.
The contract is the reference's: e4m3 weights ``[N, K]`` with one fp32 inverse
scale per 128x128 block, bf16/fp16 activations quantised per token and per 128
columns (``scale = amax / 448``, raw scale kept), every 128-wide K block's dot
product multiplied by both scales and accumulated in fp32, bias added
afterwards.  By default a shape with too few output tiles for the GPU has the
K range of a tile cut into parts that are summed separately and then added in
a fixed order, so the last bit of a row can depend on the batch size;
``set_batch_invariant(True)`` (or ``MIE_FP8_BATCH_INVARIANT=1``) keeps the
single increasing-K order of the reference for every row at every batch size.

The reference's ``path="fused" | "split"`` and ``gemm_config`` choose between
Triton kernels that are bit-identical by construction; here every call runs
the same two kernels (quantise, GEMM), so the arguments are validated and
otherwise ignored.  There is no fallback to Transformers: an unsupported call
raises.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any

import torch

from ... import _lib

SUPPORTED_BLOCK_SIZE = (128, 128)
MAX_M_BUCKET = 16384
SPLIT_M_THRESHOLD = 256
QUANT_BLOCK_M = 16


@dataclass(frozen=True)
class FP8GemmConfig:
    """Tile description kept for API compatibility (engine/kernels/sm89_fp8.py:38-65)."""

    block_m: int
    block_n: int
    num_warps: int
    num_stages: int
    group_m: int = 8
    block_k: int = 128

    @property
    def kwargs(self) -> dict[str, int]:
        return {"BLOCK_M": self.block_m, "BLOCK_N": self.block_n, "BLOCK_K": self.block_k,
                "GROUP_M": self.group_m, "PIPELINE_STAGES": self.num_stages}

    @property
    def label(self) -> str:
        return f"{self.block_m}x{self.block_n}x{self.block_k}/w{self.num_warps}/s{self.num_stages}/g{self.group_m}"

    def launch_kwargs(self) -> dict[str, int]:
        return {**self.kwargs, "num_warps": self.num_warps, "num_stages": self.num_stages}


SPLIT_GEMM_CONFIGS = tuple(
    FP8GemmConfig(*spec) if len(spec) == 4 else FP8GemmConfig(*spec[:4], group_m=spec[4])
    for spec in (
        (64, 64, 4, 3), (64, 64, 4, 4), (64, 64, 4, 5), (64, 128, 4, 3), (64, 128, 4, 4), (128, 64, 4, 3),
        (128, 64, 4, 4), (128, 128, 4, 3), (128, 128, 8, 3), (128, 128, 8, 4), (64, 256, 4, 3), (64, 256, 8, 3),
        (128, 256, 8, 3), (128, 128, 8, 3, 16),
    )
)


def m_bucket(rows: int) -> int:
    """Ceiling power of two of ``rows``, capped at ``MAX_M_BUCKET``."""

    if rows < 0:
        raise ValueError("rows must be nonnegative")
    return min(1 << (max(1, rows) - 1).bit_length(), MAX_M_BUCKET)


def select_fp8_path(rows: int, path: str = "auto") -> str:
    """Resolve ``auto`` as the reference does (inclusive threshold); no CUDA involved."""

    if path not in {"auto", "fused", "split"}:
        raise ValueError(f"Unknown SM89 FP8 path: {path!r}")
    if rows < 0:
        raise ValueError("rows must be nonnegative")
    if path != "auto":
        return path
    return "split" if rows >= SPLIT_M_THRESHOLD else "fused"


def pretune_row_buckets(max_tokens: int) -> tuple[int, ...]:
    return tuple(1 << i for i in range(m_bucket(max(1, max_tokens)).bit_length()))


def sm89_available(device: torch.device | str | None = None) -> bool:
    """Whether the FP8 kernels can run: a CUDA device of compute capability 10.x.

    The name is the reference's (it gates on 8.9); this build targets sm_100a.
    """

    if not torch.cuda.is_available():
        return False
    if torch.cuda.get_device_capability(device)[0] != 10:
        return False
    _lib.load()
    return True


def _supports_call(input, weight, weight_scale_inv, block_size, activation_scale) -> bool:
    return bool(
        input.is_cuda and weight.is_cuda and weight_scale_inv.is_cuda
        and input.dtype in {torch.float16, torch.bfloat16}
        and weight.dtype == torch.float8_e4m3fn
        and weight_scale_inv.dtype == torch.float32
        and input.ndim >= 2 and weight.ndim == 2 and weight_scale_inv.ndim == 2
        and block_size is not None and tuple(block_size) == SUPPORTED_BLOCK_SIZE
        and activation_scale is None
        and input.shape[-1] == weight.shape[1]
        and tuple(weight_scale_inv.shape) == ((weight.shape[0] + 127) // 128, (weight.shape[1] + 127) // 128)
        and sm89_available(weight.device)
    )


def _padded_width(k: int) -> int:
    return (k + 15) // 16 * 16


def quantize_activation_kmajor(input_2d: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Quantise ``[M, K]`` activations; scales come back K-group major ``[groups, M]``
    (the layout the GEMM reads).  The e4m3 rows are padded to a multiple of 16 bytes."""

    m, k = input_2d.shape
    if input_2d.stride(1) != 1:
        input_2d = input_2d.contiguous()
    groups = (k + 127) // 128
    width = _padded_width(k)
    quantized = torch.empty((m, width), device=input_2d.device, dtype=torch.float8_e4m3fn)
    if width != k:
        quantized.view(torch.uint8)[:, k:].zero_()
    scales = torch.empty((groups, max(m, 1)), device=input_2d.device, dtype=torch.float32)
    _lib.check(_lib.load().mie_fp8_quantize(
        _lib.ptr(input_2d), input_2d.stride(0), _lib.DTYPE_CODES[input_2d.dtype], _lib.ptr(quantized), width,
        _lib.ptr(scales), scales.stride(0), m, k, _lib.stream_arg(input_2d.device),
    ))
    return quantized, scales


def quantize_sm89_fp8_activation(input_2d: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``(e4m3 [M, K], raw fp32 scales [M, ceil(K/128)])`` (engine/kernels/sm89_fp8.py:401-424)."""

    if input_2d.ndim != 2 or input_2d.dtype not in {torch.bfloat16, torch.float16}:
        raise ValueError("Expected a 2D bf16/fp16 activation")
    if not input_2d.is_cuda or not sm89_available(input_2d.device):
        raise RuntimeError("Activation quantization requires a CUDA device and the mie_b200 library")
    if input_2d.shape[1] == 0:
        raise ValueError("Activation width must be positive")
    quantized, scales = quantize_activation_kmajor(input_2d)
    return quantized[:, : input_2d.shape[1]], scales[:, : input_2d.shape[0]].t()


# Weights whose layout the GEMM cannot read in place (K not a multiple of 16, unaligned base or rows) are
# copied into a padded buffer.  The copy is remembered ON the tensor object that was passed (an attribute,
# together with the tensor's version counter), so a module's parameter is copied once, while a temporary is
# copied on every call; nothing is keyed by address, which an allocator may hand to another tensor.
_PADDED_ATTR = "_mie_padded_weight"

# Process-wide default of ``max_split`` for every GEMM launched through this module: 0 lets the library cut
# the K range of a tile across a thread-block cluster where that is faster; 1 never cuts, which makes every
# output row the plain increasing-K sum whatever batch it is computed in (the reference's row-independence
# and path-independence promise, tests/test_sm89_fp8_exact.py).  MIE_FP8_BATCH_INVARIANT=1 selects 1.
_DEFAULT_MAX_SPLIT = 1 if os.environ.get("MIE_FP8_BATCH_INVARIANT", "0") == "1" else 0


def set_batch_invariant(enabled: bool) -> bool:
    """Make FP8 linear results independent of the batch they are computed in (``max_split = 1``).
    Returns the previous setting."""

    global _DEFAULT_MAX_SPLIT
    previous = _DEFAULT_MAX_SPLIT == 1
    _DEFAULT_MAX_SPLIT = 1 if enabled else 0
    return previous


def _gemm_weight(weight: torch.Tensor) -> tuple[torch.Tensor, bool]:
    """The weight as the GEMM needs it (rows contiguous, 16-byte aligned base and row stride) and whether
    a copy was written just now on the current stream.

    Model weights (K a multiple of 16) pass through untouched.  Odd shapes are copied into a padded buffer
    the first time they are seen; the GEMM that follows that copy must not request weight tiles ahead of
    its launch-chain wait (``MIE_GEMM_NO_WEIGHT_PREFETCH``), later calls reuse the buffer.
    """

    k = weight.shape[1]
    if weight.stride(1) == 1 and weight.stride(0) % 16 == 0 and weight.data_ptr() % 16 == 0:
        return weight, False
    capturing = torch.cuda.is_current_stream_capturing()
    cached = getattr(weight, _PADDED_ATTR, None)
    if cached is not None and cached[1] == weight._version and not capturing:
        return cached[0], False
    padded = torch.zeros((weight.shape[0], _padded_width(k)), dtype=torch.uint8, device=weight.device)
    padded[:, :k] = weight.contiguous().view(torch.uint8)
    if not capturing:
        try:
            setattr(weight, _PADDED_ATTR, (padded, weight._version))
        except (AttributeError, RuntimeError):
            pass
    return padded, True


def launch_fp8_gemm(quantized: torch.Tensor, scales_kmajor: torch.Tensor, weight: torch.Tensor,
                    weight_scale_inv: torch.Tensor, output: torch.Tensor, m: int, k: int,
                    status: torch.Tensor | None = None, max_split: int | None = None) -> None:
    """``output[m, n] = fp8 block-scaled product``; thin call into ``mie_fp8_gemm``."""

    device = output.device
    w, fresh_copy = _gemm_weight(weight)
    scales_w = weight_scale_inv if weight_scale_inv.stride(1) == 1 else weight_scale_inv.contiguous()
    word = status if status is not None else _lib.status_word(device)
    _lib.check(_lib.load().mie_fp8_gemm(
        _lib.ptr(quantized), quantized.stride(0), _lib.ptr(scales_kmajor), scales_kmajor.stride(0),
        _lib.ptr(w), w.stride(0), _lib.ptr(scales_w), scales_w.stride(0),
        _lib.ptr(output), output.stride(0), _lib.DTYPE_CODES[output.dtype], m, int(weight.shape[0]), k,
        int(_DEFAULT_MAX_SPLIT if max_split is None else max_split),
        _lib.GEMM_NO_WEIGHT_PREFETCH if fresh_copy else 0, _lib.ptr(word), _lib.stream_arg(device),
    ))


def _launch_split_gemm(activation, weight, output, activation_scales, weight_scales, config=None):
    """GEMM over pre-quantised activations with ``[M, groups]`` scales (engine/kernels/sm89_fp8.py:427-441)."""

    del config
    m, k = activation.shape
    width = _padded_width(k)
    if activation.stride(1) != 1 or activation.stride(0) % 16 or activation.data_ptr() % 16:
        padded = torch.zeros((m, width), dtype=torch.float8_e4m3fn, device=activation.device)
        padded[:, :k] = activation
        activation = padded
    launch_fp8_gemm(activation, activation_scales.t().contiguous(), weight, weight_scales, output, m, k)


def sm89_fp8_linear(
    input: torch.Tensor,
    weight: torch.Tensor,
    weight_scale_inv: torch.Tensor,
    block_size: list[int] | tuple[int, int] | None = None,
    bias: torch.Tensor | None = None,
    activation_scale: torch.Tensor | None = None,
    output_dtype: torch.dtype | None = None,
    allow_deepgemm: bool = True,
    *,
    path: str = "auto",
    gemm_config: FP8GemmConfig | None = None,
) -> torch.Tensor:
    """Transformers-compatible FP8 linear (engine/kernels/sm89_fp8.py:444-528)."""

    del allow_deepgemm
    select_fp8_path(0, path)
    if gemm_config is not None and (path != "split" or gemm_config not in SPLIT_GEMM_CONFIGS):
        raise ValueError("gemm_config must be a listed split config with path='split'")
    if not _supports_call(input, weight, weight_scale_inv, block_size, activation_scale):
        raise RuntimeError("Unsupported FP8 linear call and this library has no fallback")
    if output_dtype is not None and output_dtype not in {torch.float16, torch.bfloat16}:
        raise TypeError("SM89 FP8 output must be float16 or bfloat16")

    k = int(input.shape[-1])
    m = int(input.numel() // k) if k else 0
    n = int(weight.shape[0])
    output = torch.empty((m, n), device=input.device, dtype=output_dtype or input.dtype)
    if m and n:
        input_2d = input.reshape(m, k)
        quantized, scales = quantize_activation_kmajor(input_2d)
        launch_fp8_gemm(quantized, scales, weight, weight_scale_inv, output, m, k)
    result = output.reshape(*input.shape[:-1], n)
    return result if bias is None else result + bias


def pretune_sm89_fp8(model: Any, max_tokens: int = MAX_M_BUCKET) -> int:
    """Warm every FP8 shape of ``model`` (engine/kernels/sm89_fp8.py:531-558).

    Nothing is autotuned here; the call only creates the TMA descriptors
    ahead of the first request.  Returns shape/bucket pairs.
    """

    shapes = {
        (module.weight, module.weight_scale_inv, tuple(getattr(module, "block_size", SUPPORTED_BLOCK_SIZE)))
        for module in model.modules()
        if getattr(getattr(module, "weight", None), "dtype", None) == torch.float8_e4m3fn
        and isinstance(getattr(module, "weight_scale_inv", None), torch.Tensor)
    }
    dtype = next(p.dtype for p in model.parameters() if p.dtype in {torch.bfloat16, torch.float16})
    return pretune_sm89_fp8_shapes(shapes, dtype, max_tokens)


def pretune_sm89_fp8_shapes(shapes: Any, dtype: torch.dtype, max_tokens: int = MAX_M_BUCKET) -> int:
    unique = {}
    for weight, scales, block in shapes:
        unique.setdefault(tuple(weight.shape), (weight, scales, tuple(block)))
    buckets = pretune_row_buckets(int(max_tokens))
    with torch.inference_mode():
        for weight, scales, block in unique.values():
            for rows in (1, 256):
                activation = torch.zeros((rows, weight.shape[1]), dtype=dtype, device=weight.device)
                sm89_fp8_linear(activation, weight, scales, block_size=list(block))
    torch.cuda.synchronize()
    return len(unique) * len(buckets)


_original_fp8_linear = None


def install_sm89_fp8_dispatch() -> dict[str, Any]:
    """Route ``transformers.integrations.finegrained_fp8.fp8_linear`` to this kernel
    (engine/kernels/sm89_fp8.py:579-610)."""

    if not sm89_available():
        capability = list(torch.cuda.get_device_capability()) if torch.cuda.is_available() else None
        raise RuntimeError(
            f"The FP8 kernel requires an NVIDIA compute-capability 10.x GPU; detected capability={capability}"
        )
    from transformers.integrations import finegrained_fp8

    global _original_fp8_linear
    if getattr(finegrained_fp8, "fp8_linear", None) is not sm89_fp8_linear:
        _original_fp8_linear = getattr(finegrained_fp8, "fp8_linear", None)
        finegrained_fp8.fp8_linear = sm89_fp8_linear
    return {
        "installed": True,
        "backend": "mie_b200_tcgen05_fp8",
        "compute_capability_required": [10, 0],
        "block_size": [128, 128],
        "fused_operations": [
            "dynamic activation scaling",
            "FP8 E4M3 activation quantization",
            "block-scaled FP8 matrix multiplication",
        ],
        "fallback": None,
    }


__all__ = [
    "FP8GemmConfig", "MAX_M_BUCKET", "SPLIT_GEMM_CONFIGS", "SPLIT_M_THRESHOLD", "install_sm89_fp8_dispatch",
    "m_bucket", "pretune_sm89_fp8", "pretune_sm89_fp8_shapes", "quantize_sm89_fp8_activation",
    "select_fp8_path", "set_batch_invariant", "sm89_available", "sm89_fp8_linear",
]
