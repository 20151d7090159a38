"""Continuous batching through bucketed CUDA graphs on the GPU, token for token against the CPU oracle.

Short configuration (2 layers, width 512, 4 query / 2 KV heads of 128, vocabulary 2048).  The weight and
prompt seeds were chosen so that the ORACLE's own top-2 logit gap is at least 5 % of its top logit at every
step of every request (the tests re-check that with the oracle before trusting it): far outside the bf16
noise of two forwards, so greedy tokens must be identical, and they are compared with ``==``.
"""

from __future__ import annotations

import pytest
import torch

from mini_inference_engine_b200.engine.model_runner.continuous import ContinuousBatcher
from mini_inference_engine_b200.engine.model_runner.qwen3_decode import Qwen3DecodeRunner, Qwen3Shape, Qwen3Weights
from oracle_generation import oracle_generate

pytestmark = pytest.mark.gpu

SHAPE = Qwen3Shape(layers=2, hidden=512, q_heads=4, kv_heads=2, head_dim=128, intermediate=1024, vocab=2048)
DECISIVE = 0.045  # smallest accepted oracle margin (top-2 gap / |top logit|); bf16 noise is below 2**-6


def _requests(plan, prompt_seed):
    generator = torch.Generator().manual_seed(prompt_seed)
    return [(f"r{i}", torch.randint(0, SHAPE.vocab, (n,), generator=generator).tolist(), new)
            for i, (n, new) in enumerate(plan)]


def _oracle(cpu, requests):
    expected = {}
    for rid, prompt, new in requests:
        tokens, margin = oracle_generate(cpu, SHAPE, prompt, new)
        assert margin >= DECISIVE, f"the oracle itself is not decisive for {rid}: margin {margin:.4f}"
        expected[rid] = tokens
    return expected


@pytest.mark.parametrize("use_graphs", [True, False])
def test_requests_finish_at_different_times_through_shrinking_buckets(use_graphs, device):
    """Five requests with different ``max_new_tokens``: the live rows are compacted as requests finish and
    the decode bucket goes 8 -> 4 -> 2 -> 1; every request's tokens equal the oracle's; padding rows only
    ever touch offset 0 of their own scratch pages; pages nobody was given stay untouched."""

    cpu_weights = Qwen3Weights(SHAPE, torch.device("cpu"), seed=36)
    weights = cpu_weights.to(device)
    requests = _requests([(37, 3), (5, 6), (130, 9), (20, 14), (64, 20)], prompt_seed=1)
    expected = _oracle(cpu_weights, requests)
    runner = Qwen3DecodeRunner(weights, num_pages=48, max_batch=8, max_context=256, max_chunks=8)
    assert runner.decode_buckets == (1, 2, 4, 8) and runner.total_pages > runner.num_pages
    batcher = ContinuousBatcher(runner, max_prefill_tokens=512, use_graphs=use_graphs)
    for rid, prompt, new in requests:
        batcher.submit(rid, prompt, new)
    results = batcher.run()
    for rid, _, _ in requests:
        assert results[rid] == expected[rid], rid
    assert int(runner.status.item()) == 0
    assert batcher.pool.free_pages == runner.num_pages
    if use_graphs:
        buckets = [r["bucket"] for r in batcher.records if "bucket" in r]
        assert buckets[0] == 8 and buckets[-1] == 1 and buckets == sorted(buckets, reverse=True)
        assert set(buckets) == {8, 4, 2, 1}
        # Steady-state steps copy no table entries at all; a step only pays for pages that were appended.
        small = [r["h2d_bytes"] for r in batcher.records if "h2d_bytes" in r]
        assert min(small) == min(b * 12 for b in (1, 2, 4, 8) if b in buckets)
    torch.cuda.synchronize()
    used_pages = 5 * 0 + sum(-(-(len(p) + n) // 16) for _, p, n in requests)
    for pool in (runner.key_blocks, runner.value_blocks):
        assert not pool[:, used_pages:runner.num_pages].any()          # canary: pages nobody owned
        assert not pool[:, runner.num_pages:, :, 1:, :].any()          # scratch pages: only offset 0 is written


def test_late_arrivals_and_page_reuse(device):
    """Requests submitted while others decode, with a pool so small that later requests reuse the pages
    earlier ones gave back."""

    cpu_weights = Qwen3Weights(SHAPE, torch.device("cpu"), seed=36)
    weights = cpu_weights.to(device)
    requests = _requests([(37, 3), (5, 6), (130, 9), (20, 14), (64, 20)], prompt_seed=1)
    expected = _oracle(cpu_weights, requests)
    runner = Qwen3DecodeRunner(weights, num_pages=16, max_batch=4, max_context=256, kv_init="normal")
    batcher = ContinuousBatcher(runner, max_prefill_tokens=64)
    pending = list(requests)
    for _ in range(2):
        batcher.submit(*pending.pop(0))
    for iteration in range(400):
        if pending and iteration % 3 == 2:
            batcher.submit(*pending.pop(0))
        batcher.step()
        if not pending and not batcher.live and not batcher.waiting:
            break
    runner.check_status()
    assert {rid: batcher.results[rid] for rid, _, _ in requests} == expected


@pytest.mark.parametrize("use_graphs", [True, False])
def test_prompt_chunks_ride_along_with_decode_rows(use_graphs, device):
    """Mixed steps: three requests decode while a 300-token prompt is admitted and advances in bounded
    chunks inside the SAME forward (captured per (decode bucket, chunk-token bucket) when ``use_graphs``)."""

    cpu_weights = Qwen3Weights(SHAPE, torch.device("cpu"), seed=63)
    weights = cpu_weights.to(device)
    requests = _requests([(9, 24), (33, 24), (17, 24), (300, 4)], prompt_seed=1)
    expected = _oracle(cpu_weights, requests)
    runner = Qwen3DecodeRunner(weights, num_pages=64, max_batch=4, max_context=512, chunk_buckets=(32, 128))
    batcher = ContinuousBatcher(runner, max_prefill_tokens=128, mixed=True, use_graphs=use_graphs)
    for request in requests[:3]:
        batcher.submit(*request)
    for _ in range(4):
        batcher.step()
    assert all(r.decoding for r in batcher.live) and len(batcher.live) == 3
    batcher.submit(*requests[3])
    results = batcher.run()
    assert {rid: results[rid] for rid, _, _ in requests} == expected
    mixed = [r for r in batcher.records if r["kind"] == "mixed"]
    # The long prompt needed at least three steps, each of which also advanced the three decode rows.
    long_steps = [r for r in mixed if r["decode_rows"] == 3]
    assert len(long_steps) >= 3 and all(r["chunk_tokens"] + r["decode_rows"] <= 128 for r in long_steps)
    assert sum(r["chunk_tokens"] for r in long_steps) == 300
    assert int(runner.status.item()) == 0 and batcher.pool.free_pages == runner.num_pages
    if use_graphs:
        assert ("mixed", 4, 128) in runner._graphs


def test_bucket_graph_equals_the_eager_step_bit_for_bit(device):
    """A bucket's replay (3 live rows in a bucket of 4, one padding row) gives the tokens of the eager step
    on the 3 rows alone, and the pages of the live rows are byte-identical."""

    cpu_weights = Qwen3Weights(SHAPE, torch.device("cpu"), seed=5)
    weights = cpu_weights.to(device)
    runner = Qwen3DecodeRunner(weights, num_pages=24, max_batch=4, max_context=128, kv_init="normal")
    eager = Qwen3DecodeRunner(weights, num_pages=24, max_batch=4, max_context=128)
    eager.key_blocks.copy_(runner.key_blocks)
    eager.value_blocks.copy_(runner.value_blocks)
    blocks = [[3, 7], [1], [9, 4, 11]]
    lengths, ids = [20, 5, 40], [17, 900, 2047]
    tokens, h2d, d2h = runner.decode_rows(["a", "b", "c"], ids, lengths, blocks)
    tables = torch.full((3, runner.table_width), -1, dtype=torch.int32)
    for row, pages in enumerate(blocks):
        tables[row, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
    want = eager.decode_forward(torch.tensor(ids, device=device), torch.tensor(lengths, dtype=torch.int32, device=device),
                                tables.to(device))
    assert tokens == want.tolist() and d2h == 24 and h2d == 4 * 12 + (2 + 1 + 3) * 4
    live = torch.tensor(sorted(p for pages in blocks for p in pages), device=device)
    assert torch.equal(runner.key_blocks.index_select(1, live), eager.key_blocks.index_select(1, live))
    assert torch.equal(runner.value_blocks.index_select(1, live), eager.value_blocks.index_select(1, live))
    runner.check_status()


@pytest.mark.parametrize("mixed", [False, True])
def test_requests_sharing_prefix_pages_run_through_the_captured_steps(mixed, device):
    """Prefix reuse with the graphs ON (the reference turns its decode graphs off under prefix reuse,
    engine/serving/chunked_prefill.py:126-127): "b" and "c" arrive while "a" decodes, borrow the whole pages of
    the prompt prefix they have in common with it - the same page ids in several block-table rows of the
    bucket graphs and of the captured mixed steps - and prefill only their tails.  Tokens equal the oracle's."""

    cpu_weights = Qwen3Weights(SHAPE, torch.device("cpu"), seed=36)
    generator = torch.Generator().manual_seed(0)
    common = torch.randint(0, SHAPE.vocab, (48,), generator=generator).tolist()
    requests = [("a", common + torch.randint(0, SHAPE.vocab, (9,), generator=generator).tolist(), 10),
                ("b", common + torch.randint(0, SHAPE.vocab, (20,), generator=generator).tolist(), 6),
                ("c", common[:16] + torch.randint(0, SHAPE.vocab, (30,), generator=generator).tolist(), 5)]
    expected = _oracle(cpu_weights, requests)
    runner = Qwen3DecodeRunner(cpu_weights.to(device), num_pages=24, max_batch=4, max_context=128, max_chunks=4,
                               chunk_buckets=(128,))
    batcher = ContinuousBatcher(runner, max_prefill_tokens=128, mixed=mixed, prefix_cache=True)
    batcher.submit(*requests[0])
    for _ in range(3):
        batcher.step()
    donor = batcher.live[0]
    assert donor.decoding and donor.published == 3
    batcher.submit(*requests[1])
    batcher.submit(*requests[2])
    batcher.step()
    by_id = {r.rid: r for r in batcher.live}
    assert by_id["b"].pages[:3] == donor.pages[:3] and by_id["c"].pages[:1] == donor.pages[:1]
    assert batcher.prefix_hits == 48 + 16
    results = batcher.run()
    for rid, _, _ in requests:
        assert results[rid] == expected[rid], rid
    assert int(runner.status.item()) == 0
    kinds = {r["kind"] for r in batcher.records}
    assert ("mixed" in kinds) if mixed else ("decode+prefill" in kinds)
    batcher.drop_prefix_cache()
    assert batcher.pool.free_pages == runner.num_pages

