"""Fused lm_head + greedy sampling (``mie_lm_head_argmax``) against the bf16 matmul + argmax it replaces
(engine/model_runner/qwen3_mixed.py:164-174, engine/serving/chunked_prefill.py:224-229)."""

from __future__ import annotations

import pytest
import torch

from mini_inference_engine_b200 import _lib

pytestmark = pytest.mark.gpu


def _fused(x, w, *, vocab_offset=0, values=False, keys=None):
    lib = _lib.load()
    rows = x.shape[0]
    keys = torch.zeros(256, dtype=torch.int64, device=x.device) if keys is None else keys
    tokens = torch.empty(rows, dtype=torch.int64, device=x.device)
    vals = torch.empty(rows, dtype=torch.int32, device=x.device) if values else None
    status = torch.zeros(1, dtype=torch.int32, device=x.device)
    _lib.check(lib.mie_lm_head_argmax(_lib.ptr(x), x.stride(0), _lib.ptr(w), w.stride(0), rows, w.shape[0], w.shape[1],
                                      vocab_offset, _lib.ptr(keys), _lib.ptr(tokens), _lib.ptr(vals), _lib.ptr(status),
                                      _lib.stream_arg(x.device)))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert not keys.any()  # left clear for the next call
    return (tokens, vals) if values else tokens


@pytest.mark.parametrize("rows", [1, 8, 33, 130, 256])
@pytest.mark.parametrize("vocab,k", [(128, 64), (1000, 200), (4099, 2560)])
def test_exact_integer_logits_and_lowest_index_ties(rows, vocab, k, device):
    """Integer operands: every fp32 sum is exact, bf16 rounding makes ties, the lowest index must win."""

    generator = torch.Generator().manual_seed(rows * 31 + vocab)
    x = torch.randint(-1, 2, (rows, k), generator=generator).to(torch.bfloat16)
    w = torch.randint(-1, 2, (vocab, k), generator=generator).to(torch.bfloat16)
    w[vocab // 2] = w[3]  # an exact duplicate row further down never beats the first one
    logits = (x.float() @ w.float().t()).to(torch.bfloat16)
    expected = logits.argmax(dim=-1)
    got = _fused(x.to(device), w.to(device))
    assert torch.equal(got.cpu(), expected)


def test_model_shape_matches_bf16_matmul_argmax(device):
    """Qwen3-4B head: 151,936 x 2,560, 256 rows of N(0,1) hidden states, two calls in a row on shared keys."""

    generator = torch.Generator(device=device).manual_seed(0)
    w = (torch.randn(151936, 2560, device=device, generator=generator) * 0.02).to(torch.bfloat16)
    keys = torch.zeros(256, dtype=torch.int64, device=device)
    for rows in (256, 8):
        x = torch.randn(rows, 2560, device=device, generator=generator).to(torch.bfloat16)
        logits32 = x.float() @ w.float().t()
        reference = logits32.to(torch.bfloat16)
        got = _fused(x, w, keys=keys)
        best = reference.float().max(dim=-1).values
        picked = reference.float().gather(1, got.view(-1, 1)).view(-1)
        # fp32 summation order may move a logit by one bf16 step: the pick must be a maximum to within it.
        assert ((best - picked) <= best.abs() * 2 ** -7).all()
        same = got == reference.argmax(dim=-1)
        top2 = reference.float().topk(2, dim=-1).values
        clear = (top2[:, 0] - top2[:, 1]) > top2[:, 0].abs() * 2 ** -6
        assert same[clear].all()


def test_sharded_head_reports_global_indices_and_values(device):
    generator = torch.Generator().manual_seed(5)
    x = torch.randint(-1, 2, (16, 256), generator=generator).to(torch.bfloat16).to(device)
    w = torch.randint(-1, 2, (2048, 256), generator=generator).to(torch.bfloat16).to(device)
    full = _fused(x, w)
    lo, lo_val = _fused(x, w[:1024], values=True)
    hi, hi_val = _fused(x, w[1024:], vocab_offset=1024, values=True)
    merged = torch.where(hi_val > lo_val, hi, lo)  # equal values: the lower shard holds the lower index
    assert torch.equal(merged, full)
    assert (hi >= 1024).all() and (lo < 1024).all()


def test_rejects_bad_arguments(device):
    lib = _lib.load()
    x = torch.zeros(300, 64, dtype=torch.bfloat16, device=device)
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device=device)
    keys = torch.zeros(512, dtype=torch.int64, device=device)
    tokens = torch.zeros(300, dtype=torch.int64, device=device)
    code = lib.mie_lm_head_argmax(_lib.ptr(x), 64, _lib.ptr(w), 64, 300, 128, 64, 0, _lib.ptr(keys), _lib.ptr(tokens),
                                  None, None, _lib.stream_arg(device))
    assert code < 0
