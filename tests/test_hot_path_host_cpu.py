"""Host-side logic of the operators (no GPU): selector tables, metadata validation, FP8 dispatch helpers.

Expected values are the ones the reference's own CPU tests pin (tests/test_paged_attention.py:132-175,394-415;
tests/test_decode_metadata.py; tests/test_sm89_fp8_cpu.py).
"""

from __future__ import annotations

import pytest
import torch

from mini_inference_engine_b200.engine.kernels import merged_projections, sm89_fp8
from mini_inference_engine_b200.engine.kv_cache import (
    select_decode_block_tokens,
    select_decode_split_count,
    select_split_kv_decode,
    select_tensor_core_decode,
    validate_decode_metadata,
)


@pytest.mark.parametrize(("length", "expected"), [(128, 1), (1024, 2), (2048, 2), (2049, 4), (4096, 4), (4097, 8)])
def test_split_count_fixed_graph_buckets(length, expected):
    assert select_decode_split_count(length) == expected


@pytest.mark.parametrize(("length", "batch", "expected"),
                         [(2048, 1, 8), (2048, 4, 4), (2048, 8, 1), (3072, 1, 8), (3072, 4, 8), (3072, 8, 1),
                          (4096, 8, 1), (4097, 8, 8)])
def test_split_count_by_batch_shape(length, batch, expected):
    assert select_decode_split_count(length, batch_size=batch) == expected
    with pytest.raises(ValueError):
        select_decode_split_count(length, batch_size=0)


def test_other_selectors():
    assert [select_decode_block_tokens(n) for n in (1023, 1024, 4608)] == [16, 64, 64]
    assert select_split_kv_decode(4096, 1) == 8 and select_split_kv_decode(1023, 1) == 1
    assert select_split_kv_decode(2048, 2) == 4 and select_split_kv_decode(8192, 32) == 1
    assert select_tensor_core_decode(2048, 1) == (4, 64) and select_tensor_core_decode(100, 1) == (1, 64)
    assert select_tensor_core_decode(2048, 4) == (1, 64)
    with pytest.raises(ValueError):
        select_tensor_core_decode(2048, 0)


def _metadata(lengths, tables, positions=None):
    device = torch.device("cpu")
    return dict(block_tables=torch.tensor(tables, dtype=torch.int32), sequence_lengths=torch.tensor(lengths, dtype=torch.int32),
                device=device, batch_size=len(lengths), num_blocks=4, block_size=16,
                query_positions=None if positions is None else torch.tensor(positions, dtype=torch.int64))


def test_metadata_validation_messages():
    good = _metadata([17, 3], [[0, 1], [2, -1]])
    validate_decode_metadata(**good)
    with pytest.raises(ValueError, match="block-table capacity"):
        validate_decode_metadata(**_metadata([33, 3], [[0, 1], [2, -1]]))
    with pytest.raises(ValueError, match="invalid physical block ID"):
        validate_decode_metadata(**_metadata([17, 3], [[0, 4], [2, -1]]))
    with pytest.raises(ValueError, match="position"):
        validate_decode_metadata(**_metadata([17, 3], [[0, 1], [2, -1]], positions=[17, 0]))
    with pytest.raises(ValueError, match="max_sequence_length"):
        validate_decode_metadata(**good, max_sequence_length=16)
    with pytest.raises(ValueError, match="reserved KV length"):
        validate_decode_metadata(**good, reserved_lengths=(16, 3))
    with pytest.raises(ValueError, match="one value per sequence"):
        validate_decode_metadata(**good, reserved_lengths=(16,))
    bad_dtype = dict(good, sequence_lengths=torch.tensor([17.0, 3.0]))
    with pytest.raises(ValueError, match="integer tensor"):
        validate_decode_metadata(**bad_dtype)
    # Dead table entries (past the length) are never inspected.
    validate_decode_metadata(**_metadata([16, 3], [[0, 99], [2, -7]]))


def test_fp8_dispatch_helpers():
    assert [sm89_fp8.m_bucket(n) for n in (0, 1, 2, 3, 17, 16384, 20000)] == [1, 1, 2, 4, 32, 16384, 16384]
    assert sm89_fp8.select_fp8_path(255) == "fused" and sm89_fp8.select_fp8_path(256) == "split"
    assert sm89_fp8.select_fp8_path(1, "split") == "split"
    with pytest.raises(ValueError):
        sm89_fp8.select_fp8_path(1, "fast")
    with pytest.raises(ValueError):
        sm89_fp8.m_bucket(-1)
    assert sm89_fp8.pretune_row_buckets(100) == (1, 2, 4, 8, 16, 32, 64, 128)
    assert len(sm89_fp8.SPLIT_GEMM_CONFIGS) == 14 and all(c.block_k == 128 for c in sm89_fp8.SPLIT_GEMM_CONFIGS)
    assert sm89_fp8.SPLIT_GEMM_CONFIGS[-1].label == "128x128x128/w8/s3/g16"
    assert sm89_fp8.sm89_available() is False  # no CUDA device on this host


def test_merge_weights_concatenates_on_block_boundaries():
    q = torch.zeros(256, 128, dtype=torch.float8_e4m3fn)
    k = torch.ones(128, 128).to(torch.float8_e4m3fn)
    merged = merged_projections.merge_weights([q, k], [torch.full((2, 1), 2.0), torch.full((1, 1), 3.0)])
    assert merged.weight.shape == (384, 128) and merged.splits == (256, 128)
    assert merged.weight_scale_inv.flatten().tolist() == [2.0, 2.0, 3.0]
    with pytest.raises(ValueError, match="multiple of 128"):
        merged_projections.merge_weights([torch.zeros(100, 128, dtype=torch.float8_e4m3fn)], [torch.ones(1, 1)])
