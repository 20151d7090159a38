"""Host logic of the bucketed decode graphs and of continuous batching, on the CPU.

Static buffers (padding rows on private scratch pages, incremental block-table updates), the mixed-step
packer, bucket selection, the page pool and the batcher's bookkeeping need no GPU: the buffers live on the
CPU device here and the model is replaced by a stub whose "next token" is a function of its inputs.
"""

from __future__ import annotations

import pytest
import torch

from mini_inference_engine_b200.engine.model_runner.continuous import ContinuousBatcher, PagePool, PagePoolExhausted
from mini_inference_engine_b200.engine.model_runner.qwen3_decode import (
    DEFAULT_DECODE_BUCKETS,
    PADDING,
    DecodeBuffers,
    MixedBuffers,
    Qwen3Shape,
    scale_window,
    select_bucket,
    shard_bounds,
)

CPU = torch.device("cpu")


def test_bucket_selection_matches_the_reference_contract():
    # engine/serving/decode_graph.py:29-32 and tests/test_serving_cuda_graphs.py of the reference.
    assert [select_bucket(n, (1, 2, 4, 8)) for n in (1, 2, 3, 5, 8)] == [1, 2, 4, 8, 8]
    assert select_bucket(9, (1, 2, 4, 8)) is None and select_bucket(0, (1, 2)) is None
    assert DEFAULT_DECODE_BUCKETS[-1] == 256


def test_padding_rows_sit_on_their_own_scratch_pages():
    scratch = tuple(range(100, 108))
    buffers = DecodeBuffers(4, 6, CPU, scratch, page=16)
    assert buffers.block_tables[:, 0].tolist() == [100, 101, 102, 103]
    assert buffers.sequence_lengths.tolist() == [1, 1, 1, 1] and buffers.input_ids.tolist() == [0, 0, 0, 0]
    buffers.pack_rows(["a", "b"], [7, 9], [17, 3], [[5, 6], [2]])
    assert buffers.input_ids.tolist() == [7, 9, 0, 0]
    assert buffers.sequence_lengths.tolist() == [17, 3, 1, 1]
    assert buffers.block_tables[0, :2].tolist() == [5, 6] and buffers.block_tables[1, 0].item() == 2
    assert buffers.block_tables[2:, 0].tolist() == [102, 103]
    with pytest.raises(ValueError, match="distinct"):
        DecodeBuffers(2, 4, CPU, (7, 7))
    with pytest.raises(ValueError, match="capacity"):
        buffers.pack_rows(["a"], [1], [40], [[5, 6]])  # 40 tokens need 3 pages
    with pytest.raises(ValueError, match="disjoint from scratch"):
        buffers.pack_rows(["z"], [1], [3], [[101]])
    with pytest.raises(ValueError, match="fit the graph bucket"):
        buffers.pack_rows(list("abcde"), [1] * 5, [1] * 5, [[1]] * 5)


def test_block_tables_are_updated_incrementally():
    buffers = DecodeBuffers(4, 8, CPU, tuple(range(50, 54)), page=4)
    base = buffers.table_bytes_copied
    buffers.pack_rows(["a", "b"], [1, 2], [5, 2], [[10, 11], [12]])
    assert buffers.table_bytes_copied - base == (2 + 1) * 4  # two fresh rows, nothing for the padding rows
    base = buffers.table_bytes_copied
    buffers.pack_rows(["a", "b"], [3, 4], [6, 3], [[10, 11], [12]])
    assert buffers.table_bytes_copied == base  # nobody crossed a page boundary: no table traffic at all
    buffers.pack_rows(["a", "b"], [3, 4], [9, 4], [[10, 11, 13], [12]])
    assert buffers.table_bytes_copied - base == 4  # one appended page id
    assert buffers.block_tables[0, :3].tolist() == [10, 11, 13]
    # "a" finishes: "b" is compacted into row 0 (whole row rewritten), row 1 becomes padding.
    base = buffers.table_bytes_copied
    buffers.pack_rows(["b"], [5], [5], [[12, 14]])
    assert buffers.table_bytes_copied - base == 2 * 4 + 4
    assert buffers.block_tables[0, :2].tolist() == [12, 14] and buffers.block_tables[1, 0].item() == 51
    assert buffers._owners[1] is PADDING
    with pytest.raises(ValueError, match="only grow"):
        buffers.pack_rows(["b"], [5], [3], [[12]])
    # The device copy always equals the host mirror in every live entry.
    generator = torch.Generator().manual_seed(0)
    owners, pages = ["p", "q", "r"], {"p": [1], "q": [2], "r": [3]}
    lengths = {"p": 1, "q": 2, "r": 3}
    fresh = 20
    for step in range(40):
        for name in owners:
            lengths[name] += 1
            if lengths[name] > len(pages[name]) * 4:
                pages[name].append(fresh)
                fresh += 1
        if step == 15:
            owners.remove("q")
        if step == 25:
            owners.append("s")
            pages["s"], lengths["s"] = [fresh], 2
            fresh += 1
        keep = [n for n in owners if len(pages[n]) <= 8]
        buffers.pack_rows(keep, [int(torch.randint(0, 9, (1,), generator=generator)) for _ in keep],
                          [lengths[n] for n in keep], [pages[n] for n in keep])
        for row, name in enumerate(keep):
            assert buffers.block_tables[row, :len(pages[name])].tolist() == pages[name]
            assert buffers.sequence_lengths[row].item() == lengths[name]
        for row in range(len(keep), 4):
            assert buffers.block_tables[row, 0].item() == 50 + row and buffers.sequence_lengths[row].item() == 1


def test_mixed_step_packer_lays_out_decode_rows_chunks_and_padding():
    buffers = MixedBuffers(decode=4, chunk=16, chunks=2, table_width=4, device=CPU,
                           decode_scratch=(90, 91, 92, 93), chunk_scratch=(94, 95), page=8)
    assert buffers.tokens == 20 and buffers.rows == 7
    # all padding after construction
    assert buffers.token_to_sequence[4:].tolist() == [6] * 16 and buffers.kv_lens.tolist() == [0, 0, 16]
    assert buffers.cu_seqlens.tolist() == [0, 0, 0, 16]
    buffers.pack([11, 12], [9, 3], [[1, 2], [3]], [([21, 22, 23], 8, [4, 5]), ([31], 0, [6])])
    assert buffers.input_ids.tolist()[:8] == [11, 12, 0, 0, 21, 22, 23, 31]
    assert buffers.token_to_sequence.tolist()[:8] == [0, 1, 2, 3, 4, 4, 4, 5]
    assert buffers.token_to_sequence.tolist()[8:] == [6] * 12
    assert buffers.token_positions.tolist()[:8] == [8, 2, 0, 0, 8, 9, 10, 0]
    assert buffers.token_positions.tolist()[8:] == list(range(12))
    assert buffers.decode_lengths.tolist() == [9, 3, 1, 1]
    assert buffers.cu_seqlens.tolist() == [0, 3, 4, 16] and buffers.kv_lens.tolist() == [11, 1, 12]
    assert buffers.logit_rows.tolist() == [0, 1, 2, 3, 6, 7]
    assert buffers.block_tables[2:4, 0].tolist() == [92, 93] and buffers.block_tables[6, :2].tolist() == [94, 95]
    assert buffers.block_tables[4, :2].tolist() == [4, 5] and buffers.block_tables[5, 0].item() == 6
    with pytest.raises(ValueError, match="does not fit"):
        buffers.pack([], [], [], [(list(range(17)), 0, [1, 2, 3])])
    with pytest.raises(ValueError, match="capacity"):
        buffers.pack([], [], [], [([1, 2], 7, [1])])  # positions 7..8 need two pages


def test_shard_windows_keep_the_128_grid():
    assert shard_bounds(9728, 8, 3) == (3648, 4864)
    assert scale_window(3648, 4864) == (3584, 4864)   # starts 64 rows into a block
    assert scale_window(2432, 3648) == (2432, 3712)   # ends 64 rows into a block
    assert scale_window(0, 4864) == (0, 4864)


def test_page_pool_promises_then_hands_out():
    pool = PagePool(4)
    assert pool.can_promise(4) and not pool.can_promise(5)
    pool.promise(3)
    assert not pool.can_promise(2)
    first, second = pool.take(), pool.take()
    assert (first, second) == (0, 1)
    pool.give_back([first, second], unused_promise=1)
    assert pool.free_pages == 4 and pool.can_promise(4)
    with pytest.raises(PagePoolExhausted):
        pool.take()


class _StubRunner:
    """Stands in for Qwen3DecodeRunner: next token = (last token + length) % 97, first token of a prompt =
    (sum of the prompt) % 97.  Records the buckets it was asked for."""

    def __init__(self, num_pages=64, max_batch=8, max_context=256, page=16):
        self.shape = Qwen3Shape(page=page)
        self.num_pages, self.max_batch, self.max_context = num_pages, max_batch, max_context
        self.decode_buckets, self.chunk_buckets, self.max_chunks = (1, 2, 4, 8), (32, 128), 4
        self.table_width = max_context // page
        self.device = CPU
        self.buckets_used, self.mixed_steps, self.seen_pages = [], [], set()
        self.prompt_sums: dict[tuple, int] = {}

    def decode_rows(self, owners, ids, lengths, block_rows):
        self.buckets_used.append(select_bucket(len(owners), self.decode_buckets))
        for pages, length in zip(block_rows, lengths):
            assert len(pages) * self.shape.page >= length
            self.seen_pages.update(pages)
        return [(i + n) % 97 for i, n in zip(ids, lengths)], 0, 0

    def _chunk_tokens(self, chunk_items):
        out = []
        for tokens, start, pages in chunk_items:
            assert len(pages) * self.shape.page >= start + len(tokens)
            key = tuple(pages[:1])
            self.prompt_sums[key] = (self.prompt_sums.get(key, 0) if start else 0) + sum(tokens)
            out.append(self.prompt_sums[key] % 97)
        return out

    def prefill_forward(self, flat, tok2seq, tokpos, tables, cu, kv_lens, max_query_len):
        items = []
        for r in range(len(kv_lens)):
            a, b = int(cu[r]), int(cu[r + 1])
            items.append((flat[a:b].tolist(), int(tokpos[a]), [p for p in tables[r].tolist() if p >= 0]))
        return torch.tensor(self._chunk_tokens(items))

    def mixed_rows(self, ids, lengths, blocks, chunk_items):
        self.mixed_steps.append((len(ids), sum(len(c[0]) for c in chunk_items)))
        return [(i + n) % 97 for i, n in zip(ids, lengths)], self._chunk_tokens(chunk_items)

    def check_status(self):
        pass


def _expected(prompt, new_tokens):
    tokens, last, length = [], sum(prompt) % 97, len(prompt)
    tokens.append(last)
    for _ in range(new_tokens - 1):
        length += 1
        last = (last + length) % 97
        tokens.append(last)
    return tokens


@pytest.mark.parametrize("mixed", [False, True])
def test_batcher_compacts_rows_and_frees_pages(mixed):
    runner = _StubRunner()
    batcher = ContinuousBatcher(runner, max_prefill_tokens=32, mixed=mixed)
    requests = {f"r{i}": (list(range(1, 4 + 7 * i)), new) for i, new in enumerate((2, 5, 9, 17, 30))}
    for rid, (prompt, new) in requests.items():
        batcher.submit(rid, prompt, new)
    batcher.submit("late", [5] * 40, 3)
    results = batcher.run()
    for rid, (prompt, new) in requests.items():
        assert results[rid] == _expected(prompt, new), rid
    assert results["late"] == _expected([5] * 40, 3)
    assert batcher.pool.free_pages == runner.num_pages and batcher.pool.can_promise(runner.num_pages)
    # The decode bucket follows the number of live rows down to one.
    used = runner.buckets_used
    peak = used.index(max(used))  # rows ramp up while prompts are admitted, then only shrink
    assert used[-1] == 1 and used[peak:] == sorted(used[peak:], reverse=True) and {4, 2, 1} <= set(used)
    if not mixed:
        assert max(used) == 8
    if mixed:
        assert runner.mixed_steps and all(tokens <= 32 for _, tokens in runner.mixed_steps)
    with pytest.raises(ValueError, match="max_context"):
        batcher.submit("huge", [1] * 300, 8)


def test_batcher_waits_for_pages_in_fifo_order():
    runner = _StubRunner(num_pages=4)
    batcher = ContinuousBatcher(runner, max_prefill_tokens=64)
    batcher.submit("a", [1] * 30, 20)   # 50 tokens -> 4 pages: takes the whole pool
    batcher.submit("b", [2] * 10, 4)    # must wait until "a" is done
    batcher.step()
    assert [r.rid for r in batcher.live] == ["a"] and len(batcher.waiting) == 1
    results = batcher.run()
    assert results["a"] == _expected([1] * 30, 20) and results["b"] == _expected([2] * 10, 4)
    runner2 = _StubRunner(num_pages=2)
    stuck = ContinuousBatcher(runner2)
    stuck.submit("never", [1] * 40, 8)  # needs 3 pages, the pool has 2
    with pytest.raises(PagePoolExhausted):
        stuck.run()


class _PrefixStubRunner(_StubRunner):
    """Tokens do not matter here; records every chunk it is asked to prefill."""

    def __init__(self, **kwargs):
        super().__init__(**kwargs)
        self.chunks = []

    def _chunk_tokens(self, chunk_items):
        for tokens, start, pages in chunk_items:
            assert len(pages) * self.shape.page >= start + len(tokens)
            self.chunks.append((start, len(tokens), tuple(pages)))
        return [1] * len(chunk_items)


@pytest.mark.parametrize("mixed", [False, True])
def test_prefix_cache_shares_whole_prompt_pages_and_counts_references(mixed):
    runner = _PrefixStubRunner(num_pages=16, max_batch=4, max_context=128)
    batcher = ContinuousBatcher(runner, max_prefill_tokens=32, mixed=mixed, prefix_cache=True)
    common = list(range(100, 140))                      # 40 tokens: two whole pages and a half
    batcher.submit("a", common + [1, 2, 3], 6)
    while not any(r.rid == "a" and r.decoding for r in batcher.live):
        batcher.step()
    donor = next(r for r in batcher.live if r.rid == "a")
    assert donor.published == 2 and donor.borrowed == 0
    batcher.submit("b", common + [7, 8], 3)            # same first two pages, another tail
    batcher.submit("c", common[:16] + [9] * 20, 2)     # only the first page in common
    batcher.submit("d", common[:32], 2)                # the prompt IS two whole pages: one token is left to prefill
    batcher.step()
    taker = {r.rid: r for r in batcher.live}
    assert taker["b"].pages[:2] == donor.pages[:2] and taker["b"].borrowed == 2
    assert taker["c"].pages[:1] == donor.pages[:1] and taker["c"].borrowed == 1
    assert taker["d"].pages[:1] == donor.pages[:1] and taker["d"].borrowed == 1
    assert batcher.prefix_hits == 32 + 16 + 16
    # The borrowed tokens were never prefilled again: b, c and d start their first chunk behind the shared pages.
    starts = {pages[:1] + (start,) for start, _, pages in runner.chunks}
    assert (donor.pages[0], 32) in starts and (donor.pages[0], 16) in starts
    # Nobody ever writes a position inside a page it borrowed.
    for request in taker.values():
        assert request.prefilled >= request.borrowed * 16
    results = batcher.run()
    assert set(results) == {"a", "b", "c", "d"}
    # Private pages are free again; the published prefix pages stay cached until dropped or evicted.
    cached = set(batcher._prefix_pages.values())
    assert donor.pages[0] in cached and donor.pages[1] in cached
    assert batcher.pool.free_pages == runner.num_pages - len(cached)
    assert all(count == 0 for count in batcher._refs.values())
    batcher.drop_prefix_cache()
    assert batcher.pool.free_pages == runner.num_pages and not batcher._prefix_pages


def test_cached_prefix_pages_are_evicted_when_the_pool_needs_them():
    runner = _PrefixStubRunner(num_pages=8, max_batch=2, max_context=128)
    batcher = ContinuousBatcher(runner, max_prefill_tokens=64, prefix_cache=True)
    batcher.submit("a", list(range(48)) + [5], 2)       # 4 pages, 3 of them whole prompt pages
    batcher.run()
    assert batcher.pool.free_pages == 8 - 3 and len(batcher._prefix_pages) == 3
    batcher.submit("big", [7] * 100, 20)                # 8 pages: only fits once the cache lets go
    results = batcher.run()
    assert "big" in results and len(results["big"]) == 20
    assert not any(key[1] == tuple(range(16)) for key in batcher._prefix_pages)  # a's pages were reclaimed
    batcher.drop_prefix_cache()
    assert batcher.pool.free_pages == 8

