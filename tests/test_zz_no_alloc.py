"""The allocation-free decode-attention entry point against the regular one.

Some hosts of this library have no way to allocate device memory for the kernel's scratch (a bare C-ABI
binding, or a server whose HBM was all given to the KV pool), so ``mie_paged_decode_attention_static`` keeps
the work plan and split-KV partials in an array inside the library.  This file is named to be collected
last: if it fails, a run that stops at the first failure has already run everything else.
"""

from __future__ import annotations

import pytest
import torch

from mini_inference_engine_b200 import _lib, workloads
from mini_inference_engine_b200.engine.kv_cache.triton_paged_attention import launch_decode_attention

pytestmark = pytest.mark.gpu
ATOL = 2e-2  # the decode-attention tolerance used throughout tests/test_decode_attention_gpu.py


def _static_call(case, out, *, max_total_tokens, split_policy=1):
    lib = _lib.load()
    batch, q_heads, _, head_dim = (int(v) for v in case.query.shape)
    num_blocks, kv_heads, block_size, _ = (int(v) for v in case.key_blocks.shape)
    device = case.query.device
    return lib.mie_paged_decode_attention_static(
        _lib.view4_arg(case.query), _lib.view4_arg(out), _lib.view4_arg(case.key_blocks),
        _lib.view4_arg(case.value_blocks), _lib.index_arg(case.block_tables), _lib.index_arg(case.sequence_lengths),
        _lib.index_arg(None), batch, q_heads, kv_heads, head_dim, block_size, num_blocks,
        int(case.block_tables.shape[1]), _lib.DTYPE_CODES[case.query.dtype], float(case.scale), split_policy,
        int(max_total_tokens), _lib.ptr(_lib.status_word(device)), _lib.stream_arg(device))


def test_static_scratch_entry_matches_the_regular_entry_twice_in_a_row(device):
    assert _lib.load().mie_decode_builtin_scratch_bytes() == 16 << 20
    # Two different batches back to back: the second call finds the first call's plan and partials in the
    # shared array and must not be affected by them.  Both entry points build the same plan and run the same
    # kernels, only the scratch address differs, so the outputs are compared bit for bit.
    for lengths, seed in (((17, 128, 513, 2048), 0), ((4096, 33, 1000, 16, 700, 2500), 5)):
        case = workloads.decode_case(lengths, seed=seed, num_pages=640).to(device)
        total = sum(lengths)
        expected = torch.empty_like(case.query)
        launch_decode_attention(case.query, expected, case.key_blocks, case.value_blocks, case.block_tables,
                                case.sequence_lengths, None, scale=case.scale, max_total_tokens=total)
        got = torch.full_like(case.query, float("nan"))
        _lib.check(_static_call(case, got, max_total_tokens=total))
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, expected)
    word = _lib.status_word(device)
    assert int(word.item()) == 0


def test_static_scratch_entry_matches_the_reference_golden_output(golden, device):
    """Not a self-comparison: BASELINE configuration 0 against the output the reference's torch path gave."""

    meta = golden("decode_cfg0")
    case = workloads.decode_case(meta["lengths"], seed=meta["seed"], num_pages=meta["num_pages"], page=meta["page"],
                                 q_heads=meta["q_heads"], kv_heads=meta["kv_heads"],
                                 head_dim=meta["head_dim"]).to(device)
    for _ in range(2):
        got = torch.full_like(case.query, float("nan"))
        _lib.check(_static_call(case, got, max_total_tokens=sum(meta["lengths"])))
        torch.cuda.synchronize()
        result = got.transpose(1, 2).cpu()
        assert result.shape == meta["output"].shape
        assert (result.float() - meta["output"].float()).abs().max().item() <= ATOL
    assert int(_lib.status_word(device).item()) == 0


def test_static_scratch_entry_rejects_batches_beyond_its_array(device):
    case = workloads.decode_case((64, 64), seed=1, num_pages=16).to(device)
    out = torch.zeros_like(case.query)
    code = _static_call(case, out, max_total_tokens=1 << 26)
    assert code == -1
    with pytest.raises(ValueError, match="built-in buffer holds"):
        _lib.check(code)
    torch.cuda.synchronize()
    assert not out.any()  # nothing was launched
