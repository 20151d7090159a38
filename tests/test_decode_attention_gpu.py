"""Paged decode attention on the GPU against the CPU oracle and the reference's golden outputs.

Tolerance: 2e-2 max-abs in bf16, the bound BASELINE and the reference's own
GPU tests use (tests/test_paged_attention.py:273-351).
"""

from __future__ import annotations

import pytest
import torch

from mini_inference_engine_b200 import _lib, workloads
from mini_inference_engine_b200.engine.kv_cache import (
    triton_paged_decode_attention,
    tensor_core_decode_attention,
)
from mini_inference_engine_b200.engine.kv_cache.triton_paged_attention import launch_decode_attention
from oracle import hot_path

pytestmark = pytest.mark.gpu
ATOL = 2e-2


def _run(case, device, positions=None, **kwargs):
    dev = case.to(device)
    out = triton_paged_decode_attention(
        dev.query, dev.key_blocks, dev.value_blocks, dev.block_tables, dev.sequence_lengths, scale=case.scale,
        query_start_positions=None if positions is None else positions.to(device), **kwargs)
    torch.cuda.synchronize()
    return out.cpu()


@pytest.mark.parametrize("name", ["decode_cfg0", "decode_positions", "decode_page32"])
def test_matches_reference_golden_outputs(name, golden, device, status_clean):
    meta = golden(name)
    case = workloads.decode_case(meta["lengths"], seed=meta["seed"], num_pages=meta["num_pages"], page=meta["page"],
                                 q_heads=meta["q_heads"], kv_heads=meta["kv_heads"], head_dim=meta["head_dim"])
    positions = None if meta["positions"] is None else torch.tensor(meta["positions"])
    out = _run(case, device, positions)
    assert out.shape == meta["output"].shape and out.dtype == torch.bfloat16
    assert (out.float() - meta["output"].float()).abs().max().item() <= ATOL


@pytest.mark.parametrize("policy", [0, 1, 64, 256])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_split_policies_agree_with_oracle(policy, dtype, device, status_clean):
    lengths = (1, 15, 16, 17, 300, 1025, 4096, 2049)
    case = workloads.decode_case(lengths, seed=11, num_pages=512, dtype=dtype)
    expected = hot_path.paged_decode_attention(case.query, case.key_blocks, case.value_blocks, case.block_tables,
                                               case.sequence_lengths, case.scale)
    dev = case.to(device)
    out = torch.empty_like(dev.query)
    launch_decode_attention(dev.query, out, dev.key_blocks, dev.value_blocks, dev.block_tables,
                            dev.sequence_lengths, None, scale=case.scale, max_total_tokens=sum(lengths),
                            split_policy=policy)
    torch.cuda.synchronize()
    got = out.transpose(1, 2).cpu()
    assert (got.float() - expected.float()).abs().max().item() <= ATOL


@pytest.mark.parametrize("page", [8, 16, 32, 64])
@pytest.mark.parametrize("split_count", [1, 2, 4])
@pytest.mark.parametrize("use_gqa_reuse", [False, True])
def test_page_sizes_and_reference_knobs(page, split_count, use_gqa_reuse, device, status_clean):
    """Shapes of the reference's sweep (tests/test_paged_attention.py:273-351)."""

    lengths = (page * 2 + 3, page + 1)
    case = workloads.decode_case(lengths, seed=37, num_pages=32, page=page, q_heads=4, kv_heads=2)
    expected = hot_path.paged_decode_attention(case.query, case.key_blocks, case.value_blocks, case.block_tables,
                                               case.sequence_lengths, case.scale)
    out = _run(case, device, split_count=split_count, max_sequence_length=max(lengths),
               use_gqa_reuse=use_gqa_reuse, block_tokens=64)
    assert (out.float() - expected.float()).abs().max().item() <= ATOL


@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64])
def test_causal_position_known_answers(index_dtype, device, status_clean):
    """A position-1 query must not see positions 2/3: exactly 1.5, and 76.0 at position 3
    (tests/test_paged_attention.py:178-233)."""

    values = torch.tensor([[1.0, 2.0, 100.0, 200.0], [4.0, 8.0, 16.0, 32.0]], dtype=torch.bfloat16)
    value_blocks = values.reshape(2, 2, 1, 2, 1).expand(2, 2, 1, 2, 64).reshape(4, 1, 2, 64).contiguous().to(device)
    key_blocks = torch.zeros_like(value_blocks)
    query = torch.ones(2, 2, 1, 64, dtype=torch.bfloat16, device=device)
    tables = torch.tensor([[0, 1], [2, 3]], dtype=index_dtype, device=device)
    lengths = torch.tensor([4, 4], dtype=torch.int32, device=device)
    positions = torch.tensor([[1, 99], [3, 99]], dtype=index_dtype, device=device)[:, 0]
    out = triton_paged_decode_attention(query, key_blocks, value_blocks, tables, lengths, scale=0.125,
                                        query_start_positions=positions)
    assert out.shape == (2, 1, 2, 64)
    assert torch.equal(out[0].cpu(), torch.full((1, 2, 64), 1.5, dtype=torch.bfloat16))
    assert torch.equal(out[1].cpu(), torch.full((1, 2, 64), 15.0, dtype=torch.bfloat16))
    assert torch.equal(lengths.cpu(), torch.tensor([4, 4], dtype=torch.int32))


def test_positions_update_between_graph_replays(device, status_clean):
    """Device positions are read at run time (tests/test_paged_attention.py:236-270), TMA path."""

    case = workloads.decode_case((64,), seed=5, num_pages=8, q_heads=4, kv_heads=1)
    dev = case.to(device)
    positions = torch.tensor([9], dtype=torch.int64, device=device)
    kwargs = dict(scale=case.scale, query_start_positions=positions, _validate_metadata=False)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            triton_paged_decode_attention(dev.query, dev.key_blocks, dev.value_blocks, dev.block_tables,
                                          dev.sequence_lengths, **kwargs)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = triton_paged_decode_attention(dev.query, dev.key_blocks, dev.value_blocks, dev.block_tables,
                                            dev.sequence_lengths, **kwargs)
    for position in (9, 40, 63):
        positions.fill_(position)
        graph.replay()
        torch.cuda.synchronize()
        expected = hot_path.paged_decode_attention(case.query, case.key_blocks, case.value_blocks,
                                                   case.block_tables, case.sequence_lengths, case.scale,
                                                   torch.tensor([position]))
        assert (out.cpu().float() - expected.float()).abs().max().item() <= ATOL, position


def test_ragged_lognormal_batch_with_long_contexts(device, status_clean):
    """Configuration-4 shaped lengths (log-normal, clipped at 32768) incl. one maximum-length context."""

    lengths = workloads.lognormal_contexts(24, seed=9).tolist()
    lengths[3], lengths[7] = 32768, 16
    pages = sum(-(-n // 16) for n in lengths) + 5
    case = workloads.decode_case(tuple(lengths), seed=21, num_pages=pages)
    out = _run(case, device, max_sequence_length=32768, split_count=8)
    rows = (3, 7, 0, 11)
    for row in rows:
        expected = hot_path.paged_decode_attention(case.query[row : row + 1], case.key_blocks, case.value_blocks,
                                                   case.block_tables[row : row + 1],
                                                   case.sequence_lengths[row : row + 1], case.scale)
        assert (out[row : row + 1].float() - expected.float()).abs().max().item() <= ATOL, row
    # Size-independent property on every row: the chunked result equals the unsplit result.
    dev = case.to(device)
    whole = torch.empty_like(dev.query)
    launch_decode_attention(dev.query, whole, dev.key_blocks, dev.value_blocks, dev.block_tables,
                            dev.sequence_lengths, None, scale=case.scale, max_total_tokens=sum(lengths),
                            split_policy=0)
    torch.cuda.synchronize()
    assert (whole.transpose(1, 2).cpu().float() - out.float()).abs().max().item() <= 1e-2


def test_large_keys_at_least_as_accurate_as_reference_path(device, status_clean):
    """Keys near 280 (Qwen3 layer 0): error vs fp64 no worse than the torch path
    (tests/test_paged_attention.py:354-391)."""

    torch.manual_seed(11)
    tokens = 129
    keys = torch.randn(1, 2, tokens, 128) * 4
    keys[..., 7] = 280.0 * torch.sign(torch.randn(1, 2, tokens))
    keys = keys.to(torch.bfloat16)
    values = torch.randn(1, 2, tokens, 128).to(torch.bfloat16)
    query = (torch.randn(1, 4, 1, 128) * 0.6).to(torch.bfloat16)
    pages = -(-tokens // 16)
    kb = torch.zeros(pages, 2, 16, 128, dtype=torch.bfloat16)
    vb = torch.zeros_like(kb)
    tables = torch.arange(pages, dtype=torch.int32).flip(0).unsqueeze(0).contiguous()
    hot_path.write_packed_kv(keys, values, torch.zeros(tokens, dtype=torch.int32), torch.arange(tokens), tables,
                             kb, vb)
    lengths = torch.tensor([tokens], dtype=torch.int32)
    exact = torch.nn.functional.scaled_dot_product_attention(query.double(), keys.double(), values.double(),
                                                             enable_gqa=True)
    reference = hot_path.paged_decode_attention(query, kb, vb, tables, lengths, 128 ** -0.5)
    out = triton_paged_decode_attention(query.to(device), kb.to(device), vb.to(device), tables.to(device),
                                        lengths.to(device), scale=128 ** -0.5).cpu()
    ref_err = (reference.transpose(1, 2).double() - exact).abs().max().item()
    got_err = (out.transpose(1, 2).double() - exact).abs().max().item()
    assert got_err <= ref_err + 1e-3


def test_tensor_core_entry_point_writes_into_output(device, status_clean):
    case = workloads.decode_case((100, 31), seed=8, num_pages=16)
    dev = case.to(device)
    output = torch.empty_like(dev.query)
    tensor_core_decode_attention(dev.query, dev.key_blocks, dev.value_blocks, dev.block_tables,
                                 dev.sequence_lengths, output, position_buffer=dev.sequence_lengths,
                                 has_query_positions=False, scale=case.scale, split_count=1, split_span=2 ** 30,
                                 tile_tokens=64)
    expected = hot_path.paged_decode_attention(case.query, case.key_blocks, case.value_blocks, case.block_tables,
                                               case.sequence_lengths, case.scale)
    assert (output.transpose(1, 2).cpu().float() - expected.float()).abs().max().item() <= ATOL


def test_contract_errors_match_the_reference(device):
    case = workloads.decode_case((20,), seed=1, num_pages=4).to(device)
    args = (case.query, case.key_blocks, case.value_blocks, case.block_tables, case.sequence_lengths)
    with pytest.raises(ValueError, match="split_count"):
        triton_paged_decode_attention(*args, scale=1.0, split_count=3)
    with pytest.raises(ValueError, match="max_sequence_length"):
        triton_paged_decode_attention(*args, scale=1.0, split_count=2)
    with pytest.raises(ValueError, match="single KV split"):
        triton_paged_decode_attention(*args, scale=1.0, split_count=2, max_sequence_length=32, sdpa_compat=True)
    with pytest.raises(ValueError, match="block_tokens"):
        triton_paged_decode_attention(*args, scale=1.0, block_tokens=128)
    with pytest.raises(ValueError, match="integer"):
        triton_paged_decode_attention(*args, scale=1.0,
                                      query_start_positions=torch.zeros(1, device=device))
    with pytest.raises(ValueError, match="contract"):
        triton_paged_decode_attention(case.query.cpu(), *args[1:], scale=1.0)


def test_bad_page_id_sets_status_and_keeps_the_context(device):
    """An out-of-range page id under _validate_metadata=False is clamped and flagged, never a fault."""

    case = workloads.decode_case((40,), seed=1, num_pages=4).to(device)
    tables = case.block_tables.clone()
    tables[0, 1] = 1000
    out = triton_paged_decode_attention(case.query, case.key_blocks, case.value_blocks, tables,
                                        case.sequence_lengths, scale=case.scale, _validate_metadata=False)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    word = _lib.status_word(device)
    assert int(word.item()) & _lib.STATUS_BAD_PAGE
    word.zero_()
    with pytest.raises(ValueError, match="invalid physical block ID"):
        triton_paged_decode_attention(case.query, case.key_blocks, case.value_blocks, tables,
                                      case.sequence_lengths, scale=case.scale)


def test_fused_quantised_output_equals_the_standalone_quantiser(device, status_clean):
    """The e4m3 + per-head scales written by the attention epilogue (single-chunk and merged rows) are
    bit-identical to pushing the bf16 output through the activation quantiser."""

    from mini_inference_engine_b200.engine.kernels import sm89_fp8

    lengths = (9, 700, 64, 5000, 2048, 31)
    case = workloads.decode_case(lengths, seed=13, num_pages=512).to(device)
    batch = len(lengths)
    for policy in (0, 1, 64):
        out = torch.empty_like(case.query)
        q8 = torch.zeros(batch, 32 * 128, dtype=torch.float8_e4m3fn, device=device)
        scales = torch.full((32, batch), -1.0, dtype=torch.float32, device=device)
        launch_decode_attention(case.query, out, case.key_blocks, case.value_blocks, case.block_tables,
                                case.sequence_lengths, None, scale=case.scale, max_total_tokens=sum(lengths),
                                split_policy=policy, quantized_out=(q8, scales))
        q_ref, s_ref = sm89_fp8.quantize_activation_kmajor(out.view(batch, 32 * 128))
        torch.cuda.synchronize()
        assert torch.equal(q8.view(torch.uint8), q_ref.view(torch.uint8)), policy
        assert torch.equal(scales, s_ref), policy


def test_plan_reuse_across_layers_leaves_counters_clean(device, status_clean):
    """One plan, several launches on different pools (as the model step does per layer)."""

    lengths = (3000, 40, 1500)
    cases = [workloads.decode_case(lengths, seed=20 + i, num_pages=300) for i in range(3)]
    from mini_inference_engine_b200.engine.kv_cache.triton_paged_attention import decode_scratch

    scratch = decode_scratch(3, 32, 8, 128, sum(lengths), device)
    dev0 = cases[0].to(device)
    for layer, case in enumerate(cases):
        dev = case.to(device)
        out = torch.empty_like(dev.query)
        launch_decode_attention(dev.query, out, dev.key_blocks, dev.value_blocks, dev0.block_tables,
                                dev0.sequence_lengths, None, scale=case.scale, max_total_tokens=sum(lengths),
                                scratch=scratch, split_policy=64, use_plan=layer > 0, plan_slot=layer)
        torch.cuda.synchronize()
        host = workloads.DecodeCase(case.query, case.key_blocks, case.value_blocks, cases[0].block_tables,
                                    case.sequence_lengths, case.scale)
        expected = hot_path.paged_decode_attention(host.query, host.key_blocks, host.value_blocks, host.block_tables,
                                                   host.sequence_lengths, host.scale)
        assert (out.transpose(1, 2).cpu().float() - expected.float()).abs().max().item() <= ATOL, layer
