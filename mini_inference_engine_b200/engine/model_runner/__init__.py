"""Flat-token model loops of the hot path."""

from .qwen3_decode import DecodeBuffers, Qwen3DecodeRunner, Qwen3Shape, Qwen3Weights

__all__ = ["DecodeBuffers", "Qwen3DecodeRunner", "Qwen3Shape", "Qwen3Weights"]
