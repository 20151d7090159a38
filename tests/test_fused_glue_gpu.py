"""Fused RMSNorm / SiLU*up / RoPE kernels against the Hugging Face ops' outputs (tests/golden/glue.pt).

The reference promises bit-equality with PyTorch on its L4 by replaying ATen's
reduction tree; here the rounding points are the same but the row sum uses a
different order, so the bound is one bf16 ulp (2^-7 relative) on the few elements that differ.
"""

from __future__ import annotations

import pytest
import torch

from mini_inference_engine_b200 import _lib
from mini_inference_engine_b200.engine.kernels import fused
from oracle import hot_path

pytestmark = pytest.mark.gpu


def _close(got: torch.Tensor, want: torch.Tensor, max_mismatch: float = 0.02) -> None:
    got, want = got.cpu().float(), want.float()
    assert got.shape == want.shape
    ulp = want.abs().clamp_min(1e-30) * 2.0 ** -7
    assert ((got - want).abs() <= ulp).all(), (got - want).abs().max().item()
    assert (got != want).float().mean().item() <= max_mismatch


def test_rms_norm_plain_residual_and_heads(golden, device):
    g = golden("glue")
    w = g["weight"].to(device)
    _close(fused.rms_norm(g["hidden"].to(device), w, 1e-6), g["rms_plain"])
    normed, summed = fused.rms_norm(g["hidden"].to(device), w, 1e-6, residual=g["residual"].to(device))
    assert torch.equal(summed.cpu(), g["rms_summed"])
    _close(normed, g["rms_fused"])
    _close(fused.rms_norm(g["heads"].to(device), g["head_weight"].to(device), 1e-6), g["head_norm"])


def test_rms_norm_on_strided_head_views_of_merged_qkv(golden, device):
    """q/k norm reads column views of a merged projection output (engine/kernels/fused.py:178-189)."""

    g = golden("glue")
    heads = g["heads"]  # [5, 8, 128]
    merged = torch.randn(5, 6144).to(torch.bfloat16)
    merged[:, 4096:5120] = heads.reshape(5, 1024)
    view = merged.to(device)[:, 4096:5120].view(5, 8, 128)
    assert not view.is_contiguous()
    _close(fused.rms_norm(view, g["head_weight"].to(device), 1e-6), g["head_norm"])
    with pytest.raises(ValueError, match="width"):
        fused.rms_norm(torch.zeros(2, 64, dtype=torch.bfloat16, device=device), torch.ones(64, device=device), 1e-6)


def test_silu_mul_contiguous_and_column_views(golden, device):
    g = golden("glue")
    _close(fused.silu_mul(g["gate"].to(device), g["up"].to(device)), g["silu_mul"], max_mismatch=0.01)
    merged = torch.cat((g["gate"], g["up"]), dim=-1).to(device)
    gate, up = merged.split(9728, dim=-1)
    _close(fused.silu_mul(gate, up), g["silu_mul"], max_mismatch=0.01)


def test_rope_matches_hf_bitwise(golden, device):
    g = golden("glue")
    q = g["q"].to(device).transpose(1, 2).contiguous().transpose(1, 2)  # [B, H, T, D] view of [B, T, H, D]
    q_rot, k_rot = fused.apply_rotary_pos_emb(q, g["k"].to(device), g["cos"].to(device), g["sin"].to(device))
    assert torch.equal(q_rot.cpu(), g["q_rot"]) and torch.equal(k_rot.cpu(), g["k_rot"])
    with pytest.raises(ValueError, match="unsupported layout"):
        fused.apply_rotary_pos_emb(q.float(), g["k"].to(device), g["cos"].to(device), g["sin"].to(device))


def test_fused_quantisation_equals_norm_then_quantiser(device):
    """RMSNorm and SiLU*up with fused e4m3 output == the bf16 result pushed through the standalone quantiser."""

    from mini_inference_engine_b200.engine.kernels import sm89_fp8

    torch.manual_seed(4)
    lib, stream = _lib.load(), _lib.stream_arg(device)
    x = torch.randn(37, 2560, device=device).to(torch.bfloat16)
    res = torch.randn(37, 2560, device=device).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(2560, device=device)).to(torch.bfloat16)
    normed, _ = fused.rms_norm(x, w, 1e-6, residual=res)
    q_ref, s_ref = sm89_fp8.quantize_activation_kmajor(normed)
    q = torch.empty(37, 2560, dtype=torch.float8_e4m3fn, device=device)
    s = torch.empty(20, 37, dtype=torch.float32, device=device)
    summed = torch.empty_like(x)
    _lib.check(lib.mie_rms_norm(_lib.ptr(x), 2560, _lib.ptr(res), _lib.ptr(summed), _lib.ptr(w), None, _lib.ptr(q),
                                2560, _lib.ptr(s), 37, 37, 2560, 1e-6, stream))
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(s, s_ref)
    gate_up = torch.randn(37, 2 * 9728, device=device).to(torch.bfloat16)
    act = fused.silu_mul(gate_up[:, :9728], gate_up[:, 9728:])
    q_ref, s_ref = sm89_fp8.quantize_activation_kmajor(act)
    q = torch.empty(37, 9728, dtype=torch.float8_e4m3fn, device=device)
    s = torch.empty(76, 37, dtype=torch.float32, device=device)
    _lib.check(lib.mie_silu_mul(_lib.ptr(gate_up), _lib.ptr(gate_up[:, 9728:]), 2 * 9728, None, _lib.ptr(q), 9728,
                                _lib.ptr(s), 37, 37, 9728, stream))
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(s, s_ref)


def test_qkv_norm_rope_write_equals_the_unfused_chain(device):
    """One pass over the merged qkv output == head norm -> RoPE -> packed KV write (oracle ops)."""

    torch.manual_seed(5)
    tokens, q_heads, kv_heads, page = 9, 8, 2, 16
    qkv = torch.randn(tokens, (q_heads + 2 * kv_heads) * 128).to(torch.bfloat16)
    qw = (1 + 0.1 * torch.randn(128)).to(torch.bfloat16)
    kw = (1 + 0.1 * torch.randn(128)).to(torch.bfloat16)
    positions = torch.tensor([0, 1, 2, 3, 40, 41, 100, 15, 16], dtype=torch.int32)
    tok2seq = torch.tensor([0, 0, 0, 0, 1, 1, 2, 3, 3], dtype=torch.int32)
    tables = torch.tensor([[3, -1, -1, -1, -1, -1, -1], [0, 5, 7, -1, -1, -1, -1], [1, 2, 4, 6, 8, 9, 10],
                           [11, 12, -1, -1, -1, -1, -1]], dtype=torch.int32)
    pages = 13
    theta = 5_000_000.0
    q, k, v = qkv.split((q_heads * 128, kv_heads * 128, kv_heads * 128), dim=-1)
    qn = hot_path.rms_norm(q.reshape(1, tokens, q_heads, 128), qw, 1e-6).transpose(1, 2)
    kn = hot_path.rms_norm(k.reshape(1, tokens, kv_heads, 128), kw, 1e-6).transpose(1, 2)
    cos, sin = hot_path.rope_cos_sin(positions.view(1, tokens), 128, theta)
    q_ref, k_ref = hot_path.apply_rotary_pos_emb(qn, kn, cos, sin)
    kb_ref = torch.zeros(pages, kv_heads, page, 128, dtype=torch.bfloat16)
    vb_ref = torch.zeros_like(kb_ref)
    hot_path.write_packed_kv(k_ref, v.reshape(1, tokens, kv_heads, 128).transpose(1, 2), tok2seq, positions, tables,
                             kb_ref, vb_ref)

    from mini_inference_engine_b200.engine.model_runner.qwen3_decode import Qwen3Shape, rope_table

    table = rope_table(Qwen3Shape(rope_theta=theta), 128, device)
    kb = torch.zeros(pages, kv_heads, page, 128, dtype=torch.bfloat16, device=device)
    vb = torch.zeros_like(kb)
    q_out = torch.empty(tokens, q_heads, 128, dtype=torch.bfloat16, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    qkv_dev, qw_dev, kw_dev = qkv.to(device), qw.to(device), kw.to(device)
    pos_dev, seq_dev, tab_dev = positions.to(device), tok2seq.to(device), tables.to(device)
    _lib.check(_lib.load().mie_qkv_norm_rope_write(
        _lib.ptr(qkv_dev), qkv_dev.stride(0), _lib.ptr(qw_dev), _lib.ptr(kw_dev), _lib.ptr(table), 128,
        _lib.index_arg(pos_dev), _lib.index_arg(seq_dev), _lib.index_arg(tab_dev),
        _lib.ptr(q_out), _lib.view4_arg(kb), _lib.view4_arg(vb), tokens, q_heads, kv_heads, page, pages, 4, 7, 1e-6,
        _lib.ptr(status), _lib.stream_arg(device)))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(vb.cpu(), vb_ref)  # V is a pure copy
    _close(q_out, q_ref[0].transpose(0, 1), max_mismatch=0.05)
    _close(kb, kb_ref, max_mismatch=0.05)
