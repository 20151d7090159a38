"""KV scatter / gather kernels through the reference-named operators: bit-exact against the oracle."""

from __future__ import annotations

import pytest
import torch

from mini_inference_engine_b200 import _lib, workloads
from mini_inference_engine_b200.engine.kv_cache import triton_write_decode_kv, triton_write_packed_kv
from oracle import hot_path

pytestmark = pytest.mark.gpu


def test_packed_writer_matches_reference_pages_bitwise(golden, device, status_clean):
    meta = golden("scatter_gather")
    page, kv_heads, head_dim = meta["page"], meta["kv_heads"], meta["head_dim"]
    key_blocks = torch.zeros(meta["num_pages"], kv_heads, page, head_dim, dtype=torch.bfloat16, device=device)
    value_blocks = torch.zeros_like(key_blocks)
    ks, vs, seqs, poss = [], [], [], []
    for i, length in enumerate(meta["lengths"]):
        k, v = workloads.sequence_kv(meta["kv_seed_base"] + i, length, kv_heads, head_dim)
        ks.append(k)
        vs.append(v)
        seqs += [i] * length
        poss += list(range(length))
    keys, values = torch.cat(ks, dim=2).to(device), torch.cat(vs, dim=2).to(device)
    triton_write_packed_kv(keys, values, torch.tensor(seqs, dtype=torch.int32, device=device),
                           torch.tensor(poss, dtype=torch.int32, device=device), meta["tables"].to(device),
                           key_blocks, value_blocks)
    assert torch.equal(key_blocks.cpu(), meta["key_blocks"])
    assert torch.equal(value_blocks.cpu(), meta["value_blocks"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64])
def test_packed_writer_strided_value_view(dtype, index_dtype, device, status_clean):
    """V as a column view of a merged qkv output, K/V with independent strides
    (reference: tests/test_triton_packed_kv.py:13-33)."""

    torch.manual_seed(1)
    tokens, kv_heads, head_dim, page, pages = 37, 4, 128, 16, 8
    merged = torch.randn(tokens, (8 + 2 * kv_heads) * head_dim, device=device).to(dtype)
    k = merged[:, 8 * head_dim : (8 + kv_heads) * head_dim].view(1, tokens, kv_heads, head_dim).transpose(1, 2)
    v = merged[:, (8 + kv_heads) * head_dim :].view(1, tokens, kv_heads, head_dim).transpose(1, 2)
    lengths = (20, 17)
    tables = torch.tensor([[5, 2, 7], [0, 6, -1]], dtype=index_dtype, device=device)
    tok2seq = torch.tensor([0] * 20 + [1] * 17, dtype=index_dtype, device=device)
    tokpos = torch.tensor(list(range(20)) + list(range(17)), dtype=index_dtype, device=device)
    kb = torch.zeros(pages, kv_heads, page, head_dim, dtype=dtype, device=device)
    vb = torch.zeros_like(kb)
    triton_write_packed_kv(k, v, tok2seq, tokpos, tables, kb, vb)
    kb_ref, vb_ref = torch.zeros_like(kb).cpu(), torch.zeros_like(vb).cpu()
    hot_path.write_packed_kv(k.cpu(), v.cpu(), tok2seq.cpu(), tokpos.cpu(), tables.cpu(), kb_ref, vb_ref)
    assert torch.equal(kb.cpu(), kb_ref) and torch.equal(vb.cpu(), vb_ref)
    del lengths


@pytest.mark.parametrize("explicit_positions", [False, True])
def test_decode_writer_matches_oracle_bitwise(explicit_positions, device, status_clean):
    torch.manual_seed(2)
    batch, kv_heads, head_dim, page, pages = 5, 8, 128, 16, 40
    lengths = torch.tensor([1, 16, 17, 100, 33], dtype=torch.int32)
    tables = workloads.random_block_tables(lengths, num_pages=pages, page=page, seed=4)
    # Sliced (strided) metadata, as in tests/test_decode_metadata.py:141-153.
    wide = torch.full((batch, tables.shape[1] * 2), -1, dtype=torch.int32, device=device)
    wide[:, ::2] = tables.to(device)
    tables_dev = wide[:, ::2]
    lengths_wide = torch.zeros(batch * 3, dtype=torch.int32, device=device)
    lengths_wide[::3] = lengths.to(device)
    lengths_dev = lengths_wide[::3]
    positions = (lengths - 1 - torch.tensor([0, 3, 0, 50, 32])).clamp_min(0) if explicit_positions else None
    k = torch.randn(batch, kv_heads, 1, head_dim, device=device).to(torch.bfloat16)
    v = torch.randn(batch, 1, kv_heads, head_dim, device=device).to(torch.bfloat16).transpose(1, 2)
    kb = torch.zeros(pages, kv_heads, page, head_dim, dtype=torch.bfloat16, device=device)
    vb = torch.zeros_like(kb)
    triton_write_decode_kv(k, v, tables_dev, lengths_dev, kb, vb,
                           query_start_positions=None if positions is None else positions.to(device).long())
    kb_ref, vb_ref = torch.zeros_like(kb).cpu(), torch.zeros_like(vb).cpu()
    hot_path.write_decode_kv(k.cpu(), v.cpu(), tables, lengths, kb_ref, vb_ref, positions)
    assert torch.equal(kb.cpu(), kb_ref) and torch.equal(vb.cpu(), vb_ref)


def test_decode_writer_rejects_bad_metadata_before_touching_pages(device, status_clean):
    """Invalid metadata raises on the host and leaves the pages and the context alone
    (reference: tests/test_decode_metadata.py:156-176)."""

    kb = torch.zeros(4, 2, 16, 128, dtype=torch.bfloat16, device=device)
    vb = torch.zeros_like(kb)
    k = torch.ones(1, 2, 1, 128, dtype=torch.bfloat16, device=device)
    tables = torch.tensor([[9, 0]], dtype=torch.int32, device=device)
    with pytest.raises(ValueError, match="invalid physical block ID"):
        triton_write_decode_kv(k, k, tables, torch.tensor([3], dtype=torch.int32, device=device), kb, vb)
    with pytest.raises(ValueError, match="position"):
        triton_write_decode_kv(k, k, torch.tensor([[1, 0]], dtype=torch.int32, device=device),
                               torch.tensor([3], dtype=torch.int32, device=device), kb, vb,
                               query_start_positions=torch.tensor([3], device=device))
    assert not kb.any() and not vb.any()
    # Without host validation the kernel itself refuses the row and reports through the status word.
    triton_write_decode_kv(k, k, tables, torch.tensor([3], dtype=torch.int32, device=device), kb, vb,
                           _validate_metadata=False)
    torch.cuda.synchronize()
    assert not kb.any()
    word = _lib.status_word(device)
    assert int(word.item()) == _lib.STATUS_BAD_PAGE
    with pytest.raises(ValueError, match="invalid physical block ID"):
        _lib.raise_for_status(word)


def test_gather_matches_reference_bitwise(golden, device, status_clean):
    meta = golden("scatter_gather")
    kb, vb = meta["key_blocks"].to(device), meta["value_blocks"].to(device)
    lib = _lib.load()
    for i, length in enumerate(meta["lengths"]):
        k_out = torch.empty(meta["kv_heads"], length, meta["head_dim"], dtype=torch.bfloat16, device=device)
        v_out = torch.empty_like(k_out)
        row = meta["tables"][i].to(device)
        _lib.check(lib.mie_gather_kv(_lib.view4_arg(kb), _lib.view4_arg(vb), _lib.index_arg(row), _lib.ptr(k_out),
                                     _lib.ptr(v_out), length, meta["kv_heads"], meta["head_dim"], meta["page"],
                                     meta["num_pages"], 2, _lib.ptr(_lib.status_word(device)),
                                     _lib.stream_arg(device)))
        assert torch.equal(k_out.cpu().unsqueeze(0), meta["gathered"][i][0])
        assert torch.equal(v_out.cpu().unsqueeze(0), meta["gathered"][i][1])
