"""The CPU oracle against vectors produced by the reference's own code (tests/golden/make_golden.py)."""

from __future__ import annotations

import hashlib

import torch

from mini_inference_engine_b200 import workloads
from oracle import hot_path


def _digest(*tensors):
    digest = hashlib.sha256()
    for tensor in tensors:
        digest.update(tensor.contiguous().view(torch.uint8).numpy().tobytes())
    return digest.hexdigest()


def _decode_case(meta):
    return workloads.decode_case(meta["lengths"], seed=meta["seed"], num_pages=meta["num_pages"], page=meta["page"],
                                 q_heads=meta["q_heads"], kv_heads=meta["kv_heads"], head_dim=meta["head_dim"])


def test_decode_oracle_matches_reference_bitwise(golden):
    for name in ("decode_cfg0", "decode_positions", "decode_page32"):
        meta = golden(name)
        case = _decode_case(meta)
        assert _digest(case.query) == meta["query_digest"]
        positions = None if meta["positions"] is None else torch.tensor(meta["positions"])
        out = hot_path.paged_decode_attention(case.query, case.key_blocks, case.value_blocks, case.block_tables,
                                              case.sequence_lengths, case.scale, positions)
        # Same per-page arithmetic on the same bytes: placement of pages must not matter.
        assert torch.equal(out, meta["output"]), name


def test_decode_oracle_known_answers():
    """Causal-position known answers of the reference's tests (tests/test_paged_attention.py:178-270)."""

    values = torch.tensor([1.0, 2.0, 100.0, 200.0], dtype=torch.bfloat16).reshape(1, 1, 4, 1).expand(1, 1, 4, 64)
    key_blocks = torch.zeros(2, 1, 2, 64, dtype=torch.bfloat16)
    value_blocks = values.reshape(1, 2, 2, 64).permute(1, 0, 2, 3).contiguous()
    query = torch.ones(1, 2, 1, 64, dtype=torch.bfloat16)
    tables = torch.tensor([[0, 1]], dtype=torch.int32)
    lengths = torch.tensor([4], dtype=torch.int32)
    for position, expected in ((1, 1.5), (3, 75.75)):
        out = hot_path.paged_decode_attention(query, key_blocks, value_blocks, tables, lengths, 0.125,
                                              torch.tensor([position]))
        assert torch.equal(out, torch.full_like(out, expected).to(torch.bfloat16)), position


def test_scatter_gather_oracle_matches_reference(golden):
    meta = golden("scatter_gather")
    page, kv_heads, head_dim = meta["page"], meta["kv_heads"], meta["head_dim"]
    key_blocks = torch.zeros(meta["num_pages"], kv_heads, page, head_dim, dtype=torch.bfloat16)
    value_blocks = torch.zeros_like(key_blocks)
    tables = meta["tables"]
    rows, seqs, poss = [], [], []
    for i, length in enumerate(meta["lengths"]):
        keys, values = workloads.sequence_kv(meta["kv_seed_base"] + i, length, kv_heads, head_dim)
        rows.append((keys, values))
        seqs += [i] * length
        poss += list(range(length))
    keys = torch.cat([k for k, _ in rows], dim=2)
    values = torch.cat([v for _, v in rows], dim=2)
    hot_path.write_packed_kv(keys, values, torch.tensor(seqs), torch.tensor(poss), tables, key_blocks, value_blocks)
    assert torch.equal(key_blocks, meta["key_blocks"])
    assert torch.equal(value_blocks, meta["value_blocks"])
    for i, length in enumerate(meta["lengths"]):
        k, v = hot_path.gather_kv(key_blocks, value_blocks, tables[i], length)
        assert torch.equal(k.unsqueeze(0), meta["gathered"][i][0])
        assert torch.equal(v.unsqueeze(0), meta["gathered"][i][1])
    # One-token writer: re-write the last token of each sequence through the decode path.
    kb2, vb2 = key_blocks.clone(), value_blocks.clone()
    last_k = torch.stack([k[0, :, -1:, :] for k, _ in rows])
    last_v = torch.stack([v[0, :, -1:, :] for _, v in rows])
    for i, length in enumerate(meta["lengths"]):
        block = int(tables[i, (length - 1) // page])
        kb2[block, :, (length - 1) % page] = 0
        vb2[block, :, (length - 1) % page] = 0
    hot_path.write_decode_kv(last_k, last_v, tables, torch.tensor(meta["lengths"]), kb2, vb2)
    assert torch.equal(kb2, key_blocks) and torch.equal(vb2, value_blocks)


def test_prefill_oracle_matches_reference_sdpa(golden):
    meta = golden("prefill_chunks")
    case = workloads.prefill_case(seed=meta["seed"], prefix_lengths=meta["prefixes"], chunk_lengths=meta["chunks"],
                                  q_heads=meta["q_heads"], kv_heads=meta["kv_heads"], head_dim=meta["head_dim"],
                                  page=meta["page"])
    assert _digest(case.query) == meta["query_digest"]
    hot_path.write_packed_kv(case.new_keys, case.new_values, case.token_to_sequence, case.token_positions,
                             case.block_tables, case.key_blocks, case.value_blocks)
    out = hot_path.chunked_prefill_attention(case.query, case.key_blocks, case.value_blocks, case.block_tables,
                                             case.cu_seqlens, case.kv_lens, case.scale)
    # The reference's SDPA path rounds differently from an fp32 softmax; its own
    # test bound for this comparison is 2e-2 max-abs (tests/test_triton_flash_prefill.py:30-66).
    assert (out.float() - meta["output"].float()).abs().max().item() < 2e-2


def test_glue_oracle_matches_hf_ops_bitwise(golden):
    meta = golden("glue")
    assert torch.equal(hot_path.rms_norm(meta["hidden"], meta["weight"], 1e-6), meta["rms_plain"])
    fused, summed = hot_path.rms_norm(meta["hidden"], meta["weight"], 1e-6, residual=meta["residual"])
    assert torch.equal(summed, meta["rms_summed"]) and torch.equal(fused, meta["rms_fused"])
    assert torch.equal(hot_path.rms_norm(meta["heads"], meta["head_weight"], 1e-6), meta["head_norm"])
    assert torch.equal(hot_path.silu_mul(meta["gate"], meta["up"]), meta["silu_mul"])
    cos, sin = hot_path.rope_cos_sin(meta["positions"], 128, 5_000_000.0)
    assert torch.equal(cos, meta["cos"]) and torch.equal(sin, meta["sin"])
    q_rot, k_rot = hot_path.apply_rotary_pos_emb(meta["q"], meta["k"], cos, sin)
    assert torch.equal(q_rot, meta["q_rot"]) and torch.equal(k_rot, meta["k_rot"])


def test_fp8_oracle_within_tolerance_of_dequantised_product():
    """The FP8 restatement against the double-precision dequantised product (1e-2 relative)."""

    for name, m in (("o", 8), ("qkv", 3)):
        x, weight = workloads.gemm_case(name, m, seed=1)
        w8, scales = hot_path.quantize_weight(weight)
        out = hot_path.fp8_linear(x, w8, scales).double()
        exact = hot_path.dense_fp8_reference(x, w8, scales)
        rel = (out - exact).norm(dim=1) / exact.norm(dim=1)
        assert rel.max().item() < 1e-2 * 5, rel.max().item()  # activation quantisation adds ~3% per element, <5e-2 in L2


def test_fp8_quantiser_raw_scales_and_zero_rows():
    """Raw scale stored (zero for a zero group), division by max(scale, 1e-12)
    (engine/kernels/sm89_fp8.py:320-326; tests/test_sm89_fp8_exact.py:55-63)."""

    x = torch.zeros(3, 256, dtype=torch.bfloat16)
    x[1, :128] = 448.0
    x[2, 130] = -1.0
    q, s = hot_path.quantize_activation(x)
    assert s[0].tolist() == [0.0, 0.0]
    assert s[1].tolist() == [1.0, 0.0]
    assert q[1, :128].float().eq(448.0).all() and q[0].float().eq(0).all()
    assert q[2, 130].float().item() == -448.0
    assert s[2, 1].item() == (torch.tensor(1.0) / 448.0).item()
