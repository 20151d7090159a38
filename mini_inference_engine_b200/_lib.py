"""ctypes binding of ``libmie_b200.so`` (the C-ABI in ``include/mie_b200.h``).

There is no CPU fallback: if the shared library is missing or cannot be
loaded, every operator of this package raises ``MieLibraryError``.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int32, c_int64, c_void_p
from pathlib import Path

import torch

from .build import LIB_PATH

STATUS_BAD_LENGTH = 1
STATUS_BAD_POSITION = 2
STATUS_BAD_PAGE = 4
STATUS_BAD_SEQUENCE = 8
STATUS_WAIT_TIMEOUT = 16
STATUS_MAX_LENGTH = 32
STATUS_CAPACITY = 64
STATUS_NO_TOKEN = 128

GEMM_NO_WEIGHT_PREFETCH = 1

STATUS_MESSAGES = {
    STATUS_BAD_LENGTH: "sequence_lengths exceed the available block-table capacity",
    STATUS_BAD_POSITION: "query position must satisfy 0 <= position < sequence_length",
    STATUS_BAD_PAGE: "block_tables contain an invalid physical block ID",
    STATUS_BAD_SEQUENCE: "token_to_sequence contains an invalid sequence index",
    STATUS_WAIT_TIMEOUT: "a bounded device-side wait timed out",
    STATUS_MAX_LENGTH: "max_sequence_length does not cover the attention read length",
    STATUS_CAPACITY: "decode work plan exceeded its scratch capacity",
    STATUS_NO_TOKEN: "greedy sampling found no candidate for a row (token 0 was substituted)",
}

DTYPE_CODES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


class MieLibraryError(RuntimeError):
    """The CUDA library is missing, failed to load, or rejected a call."""


class IndexT(Structure):
    _fields_ = [("ptr", c_void_p), ("is64", c_int32), ("stride0", c_int64), ("stride1", c_int64)]


class View4T(Structure):
    _fields_ = [("ptr", c_void_p), ("stride", c_int64 * 4)]


TP_MAX_RANKS = 8
IPC_HANDLE_BYTES = 64


class TpPeersT(ctypes.Structure):
    """``mie_tp_peers_t``: per-rank addresses of the buffers of the fused tensor-parallel exchange."""

    _fields_ = [("partial", c_void_p * TP_MAX_RANKS), ("q", c_void_p * TP_MAX_RANKS),
                ("scales", c_void_p * TP_MAX_RANKS), ("normed", c_void_p * TP_MAX_RANKS),
                ("flags", c_void_p * TP_MAX_RANKS)]


_SIGNATURES: dict[str, tuple[object, list[object]]] = {
    "mie_last_error": (c_char_p, []),
    "mie_version": (ctypes.c_int, []),
    "mie_sm_count": (ctypes.c_int, []),
    "mie_launch_count": (c_int64, []),
    "mie_write_decode_kv": (ctypes.c_int, [View4T, View4T, IndexT, IndexT, IndexT, View4T, View4T, c_int32, c_int32,
                                           c_int32, c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p]),
    "mie_write_packed_kv": (ctypes.c_int, [View4T, View4T, IndexT, IndexT, IndexT, View4T, View4T, c_int32, c_int32,
                                           c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_void_p,
                                           c_void_p]),
    "mie_gather_kv": (ctypes.c_int, [View4T, View4T, IndexT, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32,
                                     c_int32, c_int32, c_void_p, c_void_p]),
    "mie_validate_decode_metadata": (ctypes.c_int, [IndexT, IndexT, IndexT, c_int32, c_int32, c_int32, c_int32,
                                                    c_int64, c_void_p, c_void_p]),
    "mie_decode_scratch_bytes": (c_int64, [c_int32, c_int32, c_int32, c_int32, c_int64]),
    "mie_paged_decode_attention": (ctypes.c_int, [View4T, View4T, View4T, View4T, IndexT, IndexT, IndexT, c_int32,
                                                  c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                                                  c_float, c_int32, c_int64, c_void_p, c_int64, c_int32, c_int32,
                                                  c_int32, c_void_p, c_int64, c_void_p, c_int32, c_void_p, c_void_p]),
    "mie_paged_decode_attention_kv8": (ctypes.c_int, [View4T, View4T, c_void_p, c_int64, c_void_p, IndexT, IndexT,
                                                      IndexT, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                                                      c_float, c_int32, c_void_p, c_int64, c_int32, c_int32,
                                                      c_int32, c_void_p, c_int64, c_void_p, c_int32, c_void_p,
                                                      c_void_p]),
    "mie_qkv_norm_rope_write_kv8": (ctypes.c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int32, IndexT,
                                                   IndexT, IndexT, c_void_p, c_void_p, c_int64, c_void_p, c_int32,
                                                   c_int32, c_int32, c_int32, c_int32, c_int32, c_float, c_void_p,
                                                   c_void_p]),
    "mie_decode_builtin_scratch_bytes": (c_int64, []),
    "mie_paged_decode_attention_static": (ctypes.c_int, [View4T, View4T, View4T, View4T, IndexT, IndexT, IndexT,
                                                         c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                                                         c_int32, c_int32, c_float, c_int32, c_int64, c_void_p,
                                                         c_void_p]),
    "mie_flash_prefill_attention": (ctypes.c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, View4T,
                                                   View4T, IndexT, IndexT, IndexT, c_int32, c_int32, c_int32,
                                                   c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_float,
                                                   c_void_p, c_void_p]),
    "mie_fp8_quantize": (ctypes.c_int, [c_void_p, c_int64, c_int32, c_void_p, c_int64, c_void_p, c_int32, c_int32,
                                        c_int32, c_void_p]),
    "mie_fp8_gemm": (ctypes.c_int, [c_void_p, c_int64, c_void_p, c_int32, c_void_p, c_int64, c_void_p, c_int32,
                                    c_void_p, c_int64, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                                    c_void_p, c_void_p]),
    "mie_rms_norm": (ctypes.c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                    c_void_p, c_int32, c_int32, c_int32, c_float, c_void_p]),
    "mie_head_rms_norm": (ctypes.c_int, [c_void_p, c_int64, c_int64, c_int32, c_void_p, c_void_p, c_int64, c_float,
                                         c_void_p]),
    "mie_silu_mul": (ctypes.c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int32,
                                    c_int32, c_int32, c_void_p]),
    "mie_rope": (ctypes.c_int, [View4T, c_void_p, c_void_p, c_int64, c_int64, View4T, c_int32, c_int32, c_int32,
                                c_int32, c_void_p]),
    "mie_qkv_norm_rope_write": (ctypes.c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int32, IndexT,
                                               IndexT, IndexT, c_void_p, View4T, View4T, c_int32, c_int32, c_int32,
                                               c_int32, c_int32, c_int32, c_int32, c_float, c_void_p, c_void_p]),
    "mie_lm_head_argmax": (ctypes.c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int32, c_int32, c_int32, c_int64,
                                          c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "mie_ipc_export": (ctypes.c_int, [c_void_p, c_void_p, ctypes.POINTER(c_int64)]),
    "mie_ipc_open": (ctypes.c_int, [c_void_p, c_int64, ctypes.POINTER(c_void_p)]),
    "mie_ipc_close": (ctypes.c_int, [c_void_p, c_int64]),
    "mie_tp_reduce_rms_norm": (ctypes.c_int, [ctypes.POINTER(TpPeersT), c_int32, c_int32, c_int64, c_void_p, c_void_p,
                                              c_void_p, c_int64, c_int32, c_int32, c_int32, c_float, c_void_p,
                                              ctypes.c_uint32, c_void_p, c_void_p]),
}

_lib: ctypes.CDLL | None = None


def exported_symbols() -> tuple[str, ...]:
    """Names that ``include/mie_b200.h`` declares and this module binds."""

    return tuple(_SIGNATURES)


def library_path() -> Path:
    """The shared library to load: ``$MIE_LIBRARY_PATH`` when set (a build kept elsewhere), else the in-tree one."""

    override = os.environ.get("MIE_LIBRARY_PATH")
    return Path(override) if override else LIB_PATH


def load() -> ctypes.CDLL:
    """Load the shared library (once) and attach argument types."""

    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        raise MieLibraryError(
            f"{path} is missing: run `python -m mini_inference_engine_b200.build` (needs nvcc). "
            "This package has no CPU or PyTorch fallback."
        )
    try:
        lib = ctypes.CDLL(str(path))
    except OSError as error:
        raise MieLibraryError(f"cannot load {path}: {error}") from error
    for name, (restype, argtypes) in _SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as error:
            raise MieLibraryError(f"{path} does not export {name}; rebuild it") from error
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(code: int) -> None:
    """Raise for a negative return code of a C-ABI call."""

    if code == 0:
        return
    message = load().mie_last_error().decode("utf-8", "replace")
    if code == -1:
        raise ValueError(message)
    raise MieLibraryError(f"mie_b200 call failed ({code}): {message}")


def index_arg(tensor: torch.Tensor | None) -> IndexT:
    """Describe an int32/int64 metadata tensor (1-D or 2-D, any strides)."""

    if tensor is None:
        return IndexT(None, 0, 0, 0)
    if tensor.dtype not in (torch.int32, torch.int64):
        raise ValueError("metadata tensors must be int32 or int64")
    strides = tensor.stride()
    return IndexT(tensor.data_ptr(), int(tensor.dtype == torch.int64), strides[0] if strides else 1,
                  strides[1] if len(strides) > 1 else 0)


def view4_arg(tensor: torch.Tensor) -> View4T:
    if tensor.ndim != 4:
        raise ValueError("expected a 4-D tensor")
    return View4T(tensor.data_ptr(), (c_int64 * 4)(*tensor.stride()))


def stream_arg(device: torch.device | None = None) -> c_void_p:
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def ptr(tensor: torch.Tensor | None) -> c_void_p:
    return c_void_p(None if tensor is None else tensor.data_ptr())


# One status word per device, reused by every call that does not bring its own.
_status_words: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    index = device.index if device.index is not None else torch.cuda.current_device()
    word = _status_words.get(index)
    if word is None:
        # Created outside inference mode even when the first caller is inside it (the reference's engine runs
        # under torch.inference_mode()): an inference tensor could not be cleared from ordinary code later.
        with torch.inference_mode(False):
            word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
        _status_words[index] = word
    return word


def raise_for_status(word: torch.Tensor) -> None:
    """Read a status word back (synchronises) and raise ``ValueError`` if any bit is set."""

    bits = int(word.item())
    if bits == 0:
        return
    word.zero_()
    messages = [text for bit, text in STATUS_MESSAGES.items() if bits & bit]
    raise ValueError("; ".join(messages) or f"device status {bits}")
