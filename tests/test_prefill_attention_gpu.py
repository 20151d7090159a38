"""Chunked-prefill attention over pages on the GPU: golden outputs of the reference's exact path
(gather + aligned SDPA) and the fp32 oracle, 2e-2 max-abs as in tests/test_triton_flash_prefill.py:30-66."""

from __future__ import annotations

import pytest
import torch

from mini_inference_engine_b200 import workloads
from mini_inference_engine_b200.engine.kv_cache import (
    triton_flash_prefill_attention,
    triton_packed_prefill_attention,
    triton_write_packed_kv,
)
from oracle import hot_path

pytestmark = pytest.mark.gpu
ATOL = 2e-2


def _run(case, device):
    dev = case.to(device)
    triton_write_packed_kv(dev.new_keys, dev.new_values, dev.token_to_sequence, dev.token_positions,
                           dev.block_tables, dev.key_blocks, dev.value_blocks)
    out = triton_flash_prefill_attention(dev.query, dev.key_blocks, dev.value_blocks, dev.block_tables,
                                         dev.cu_seqlens, dev.kv_lens, max_query_len=max(case.chunk_lengths),
                                         scale=case.scale)
    torch.cuda.synchronize()
    return dev, out.cpu()


def _oracle(case):
    kb, vb = case.key_blocks.clone(), case.value_blocks.clone()
    hot_path.write_packed_kv(case.new_keys, case.new_values, case.token_to_sequence, case.token_positions,
                             case.block_tables, kb, vb)
    return kb, vb, hot_path.chunked_prefill_attention(case.query, kb, vb, case.block_tables, case.cu_seqlens,
                                                      case.kv_lens, case.scale)


def test_matches_reference_golden_chunks(golden, device, status_clean):
    meta = golden("prefill_chunks")
    case = workloads.prefill_case(seed=meta["seed"], prefix_lengths=meta["prefixes"], chunk_lengths=meta["chunks"],
                                  q_heads=meta["q_heads"], kv_heads=meta["kv_heads"], head_dim=meta["head_dim"],
                                  page=meta["page"])
    _, out = _run(case, device)
    assert (out.float() - meta["output"].float()).abs().max().item() <= ATOL


def test_configuration_2_scatter_then_attention(device, status_clean):
    """BASELINE configuration 2: 6 sequences, prefixes U[0, 4096], chunks U[1, 512], 32 q / 8 kv heads."""

    case = workloads.prefill_case(requests=6, seed=0)
    kb, vb, expected = _oracle(case)
    dev, out = _run(case, device)
    assert torch.equal(dev.key_blocks.cpu(), kb) and torch.equal(dev.value_blocks.cpu(), vb)  # scatter: bit-exact
    assert (out.float() - expected.float()).abs().max().item() <= ATOL


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("page", [16, 32, 64])
def test_edge_shapes(dtype, page, device, status_clean):
    """One-token chunks, empty prefixes, chunk ends on tile edges, an empty request in the middle."""

    prefixes = (0, 77, 0, 63, 1024, 5)
    chunks = (1, 1, 16, 65, 17, 0)
    case = workloads.prefill_case(seed=3, prefix_lengths=prefixes[:5], chunk_lengths=chunks[:5], page=page,
                                  q_heads=8, kv_heads=2, dtype=dtype)
    _, _, expected = _oracle(case)
    _, out = _run(case, device)
    assert (out.float() - expected.float()).abs().max().item() <= ATOL


def test_packed_metadata_entry_point(device, status_clean):
    """Whole prompts addressed by (token_to_sequence, token_positions) (triton_packed_attention.py:186-259)."""

    case = workloads.prefill_case(seed=9, prefix_lengths=(0, 0, 0), chunk_lengths=(40, 1, 130), q_heads=8, kv_heads=2)
    _, _, expected = _oracle(case)
    dev = case.to(device)
    triton_write_packed_kv(dev.new_keys, dev.new_values, dev.token_to_sequence, dev.token_positions,
                           dev.block_tables, dev.key_blocks, dev.value_blocks)
    out = triton_packed_prefill_attention(dev.query, dev.key_blocks, dev.value_blocks, dev.token_to_sequence,
                                          dev.token_positions, dev.block_tables, scale=case.scale)
    assert (out.cpu().float() - expected.float()).abs().max().item() <= ATOL
    with pytest.raises(ValueError, match="contract"):
        triton_packed_prefill_attention(dev.query.cpu(), dev.key_blocks, dev.value_blocks, dev.token_to_sequence,
                                        dev.token_positions, dev.block_tables, scale=case.scale)


def test_decode_is_the_one_row_special_case(device, status_clean):
    """A one-token chunk over a prefix equals paged decode attention on the same pages."""

    from mini_inference_engine_b200.engine.kv_cache import triton_paged_decode_attention

    case = workloads.prefill_case(seed=4, prefix_lengths=(300, 31), chunk_lengths=(1, 1))
    dev, out = _run(case, device)
    decoded = triton_paged_decode_attention(dev.query.view(2, 1, 32, 128).transpose(1, 2), dev.key_blocks,
                                            dev.value_blocks, dev.block_tables, dev.kv_lens, scale=case.scale)
    assert (out.float() - decoded.cpu().view(2, 32, 128).float()).abs().max().item() <= 1e-2
