"""Continuous batching over the captured steps of ``Qwen3DecodeRunner``.

The small serving loop that the hot path needs around it (reference: engine/serving/chunked_prefill.py -
``ChunkedPrefillPagedRunner``: admission while a slot and enough pages for the request's full length are free
``:46-57``, one decode step for all live rows per iteration through a bucketed CUDA graph ``:264-298``, prompt
work in bounded chunks ``:314-455``).  It owns request bookkeeping and a page free list and nothing else:
the reference's admission scheduler, prefix cache, step planner and event recorder stay the reference's.

Two step policies:

* ``mixed=False``  every iteration runs one graph decode step for the decoding rows (the bucket is the
  smallest that holds them: rows are compacted when a request finishes, so the bucket shrinks with the
  batch), then spends up to ``max_prefill_tokens`` of prompt work in one eager packed prefill forward.
* ``mixed=True``   every iteration is ONE captured forward that carries the decode rows and the prompt chunks
  in one flat token stream (token-count buckets), so a long prompt advances a bounded chunk per step
  instead of stalling decode.

``prefix_cache=True`` lets a request borrow the whole pages of a prompt prefix that another request has already
written (the reference switches its decode graphs OFF when prefix reuse is on,
engine/serving/chunked_prefill.py:126-127; here a shared page is just the same id in two block-table rows, so
the captured decode and mixed steps run unchanged).  Pages are reference-counted; a prefix page nobody uses
stays cached until the pool needs it back.
"""

from __future__ import annotations

from collections import OrderedDict, deque
from dataclasses import dataclass, field

import torch

from .qwen3_decode import Qwen3DecodeRunner


class PagePoolExhausted(RuntimeError):
    """No free KV page is left for a request that was admitted against a reservation."""


class PagePool:
    """Free list of the runner's request pages with per-request reservations: a request is admitted only
    when pages for its FULL length (prompt + new tokens) can be promised, and then takes them one at a time
    as it grows, so its block list is append-only."""

    def __init__(self, num_pages: int) -> None:
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))  # pop() hands out page 0 first
        self._promised = 0

    @property
    def free_pages(self) -> int:
        return len(self._free)

    def can_promise(self, pages: int) -> bool:
        return pages <= len(self._free) - self._promised

    def promise(self, pages: int) -> None:
        if not self.can_promise(pages):
            raise PagePoolExhausted(f"cannot reserve {pages} pages")
        self._promised += pages

    def take(self) -> int:
        """One page out of an earlier promise."""

        if not self._free or self._promised < 1:
            raise PagePoolExhausted("no reserved page left")
        self._promised -= 1
        return self._free.pop()

    def give_back(self, pages: list[int], unused_promise: int) -> None:
        self._free.extend(reversed(pages))
        self._promised -= unused_promise


@dataclass
class _Request:
    rid: object
    prompt: list[int]
    max_new_tokens: int
    pages: list[int] = field(default_factory=list)
    promised: int = 0          # pages promised and not taken yet
    prefilled: int = 0         # prompt tokens whose K/V are in the cache
    generated: list[int] = field(default_factory=list)
    borrowed: int = 0          # leading pages taken over from the prefix cache at admission
    published: int = 0         # leading whole prompt pages already offered to the prefix cache

    @property
    def decoding(self) -> bool:
        return self.prefilled == len(self.prompt)

    @property
    def finished(self) -> bool:
        return len(self.generated) >= self.max_new_tokens


class ContinuousBatcher:
    """Greedy continuous-batching generation: requests may be submitted at any iteration and finish at
    different times.  ``step()`` runs one iteration and returns the ``(request id, token)`` pairs it produced;
    ``run()`` drains everything and returns each request's tokens."""

    def __init__(self, runner: Qwen3DecodeRunner, *, max_prefill_tokens: int = 512, mixed: bool = False,
                 use_graphs: bool = True, prefix_cache: bool = False) -> None:
        if max_prefill_tokens < 1:
            raise ValueError("max_prefill_tokens must be positive")
        self.runner, self.mixed, self.use_graphs = runner, bool(mixed), bool(use_graphs)
        self.prefix_cache = bool(prefix_cache)
        # Prefix cache: key of a whole-page prompt prefix -> the page that holds its last 16 tokens.  A key is the
        # nested tuple (key of the prefix one page shorter, this page's tokens): equal keys mean equal prefixes.
        self._prefix_pages: OrderedDict[tuple, int] = OrderedDict()
        self._page_key: dict[int, tuple] = {}
        self._refs: dict[int, int] = {}  # page -> live requests that have it in their block list
        self.prefix_hits = 0             # prompt tokens that were not prefilled again
        self.max_prefill_tokens = int(max_prefill_tokens)
        if self.mixed:
            self.max_prefill_tokens = min(self.max_prefill_tokens, max(runner.chunk_buckets))
        self.pool = PagePool(runner.num_pages)
        self.waiting: deque[_Request] = deque()
        self.live: list[_Request] = []   # admission order; decode rows are the decoding ones, in this order
        self.results: dict[object, list[int]] = {}
        self.records: list[dict] = []    # one per iteration: rows, bucket, chunk tokens, bytes copied

    # -- requests -----------------------------------------------------------------------------------

    def submit(self, rid, prompt, max_new_tokens: int) -> None:
        prompt = [int(t) for t in prompt]
        if not prompt or max_new_tokens < 1:
            raise ValueError("a request needs a prompt and at least one new token")
        if len(prompt) + max_new_tokens > self.runner.max_context:
            raise ValueError("prompt + new tokens exceed the runner's max_context")
        if rid in self.results or any(r.rid == rid for r in (*self.waiting, *self.live)):
            raise ValueError(f"duplicate request id {rid!r}")
        self.waiting.append(_Request(rid, prompt, int(max_new_tokens)))

    def _prefix_keys(self, request: _Request, pages: int):
        """Keys of the request's first ``pages`` whole prompt pages, shortest prefix first."""

        page, key = self.runner.shape.page, ()
        for k in range(pages):
            key = (key, tuple(request.prompt[k * page:(k + 1) * page]))
            yield key

    def _cached_prefix(self, request: _Request) -> list[int]:
        """Pages of the longest cached whole-page prefix of the prompt.  At least one prompt token is left to
        prefill: its logits give the request's first new token."""

        hits = []
        for key in self._prefix_keys(request, (len(request.prompt) - 1) // self.runner.shape.page):
            cached = self._prefix_pages.get(key)
            if cached is None:
                break
            hits.append(cached)
        return hits

    def _evict(self, wanted: int, keep: set[int]) -> None:
        """Hand cached prefix pages nobody uses back to the pool, oldest first, until ``wanted`` can be promised."""

        for key, cached in list(self._prefix_pages.items()):
            if self.pool.can_promise(wanted):
                return
            if self._refs.get(cached, 0) == 0 and cached not in keep:
                del self._prefix_pages[key]
                del self._page_key[cached]
                self._refs.pop(cached, None)
                self.pool.give_back([cached], 0)

    def _admit(self) -> None:
        page = self.runner.shape.page
        while self.waiting and len(self.live) < self.runner.max_batch:
            request = self.waiting[0]
            hits = self._cached_prefix(request) if self.prefix_cache else []
            needed = -(-(len(request.prompt) + request.max_new_tokens) // page) - len(hits)
            if not self.pool.can_promise(needed):
                self._evict(needed, set(hits))
            if not self.pool.can_promise(needed):
                break  # FIFO: a large request at the head waits for pages, nothing overtakes it
            self.pool.promise(needed)
            request.promised = needed
            for cached in hits:
                self._refs[cached] = self._refs.get(cached, 0) + 1
                self._prefix_pages.move_to_end(self._page_key[cached])
            request.pages = list(hits)
            request.borrowed = request.published = len(hits)
            request.prefilled = len(hits) * page
            self.prefix_hits += request.prefilled
            self.live.append(self.waiting.popleft())

    def _grow(self, request: _Request, tokens: int) -> None:
        """Make sure the request holds pages for ``tokens`` tokens."""

        page = self.runner.shape.page
        while len(request.pages) * page < tokens:
            fresh = self.pool.take()
            request.pages.append(fresh)
            self._refs[fresh] = 1
            request.promised -= 1

    def _publish(self, request: _Request) -> None:
        """Offer the whole prompt pages this request has finished writing to the prefix cache."""

        whole = min(request.prefilled, len(request.prompt)) // self.runner.shape.page
        if whole <= request.published:
            return
        for k, key in enumerate(self._prefix_keys(request, whole)):
            if k >= request.published and key not in self._prefix_pages:
                self._prefix_pages[key] = request.pages[k]
                self._page_key[request.pages[k]] = key
        request.published = whole

    def _retire(self) -> None:
        still = []
        for request in self.live:
            if request.decoding and request.finished:
                self.results[request.rid] = list(request.generated)
                private = []
                for used in request.pages:
                    self._refs[used] -= 1
                    if self._refs[used] == 0 and used not in self._page_key:
                        del self._refs[used]
                        private.append(used)  # cached prefix pages stay out of the free list until evicted
                self.pool.give_back(private, request.promised)
            else:
                still.append(request)
        self.live = still  # order kept: rows are compacted, not shuffled

    def drop_prefix_cache(self) -> None:
        """Give every cached prefix page that no live request uses back to the pool."""

        for key, cached in list(self._prefix_pages.items()):
            if self._refs.get(cached, 0) == 0:
                del self._prefix_pages[key]
                del self._page_key[cached]
                self._refs.pop(cached, None)
                self.pool.give_back([cached], 0)

    # -- one iteration ------------------------------------------------------------------------------

    def _plan_chunks(self, budget: int) -> list[tuple[_Request, int, int]]:
        """(request, start, count) for the partial prompts, shortest remaining first, inside the budget."""

        chunks = []
        partial = sorted((r for r in self.live if not r.decoding), key=lambda r: len(r.prompt) - r.prefilled)
        for request in partial:
            if budget <= 0 or len(chunks) >= self.runner.max_chunks:
                break
            count = min(len(request.prompt) - request.prefilled, budget)
            chunks.append((request, request.prefilled, count))
            budget -= count
        return chunks

    def step(self) -> list[tuple[object, int]]:
        self._admit()
        produced: list[tuple[object, int]] = []
        decoding = [r for r in self.live if r.decoding and not r.finished]
        for request in decoding:
            self._grow(request, len(request.prompt) + len(request.generated))
        budget = self.max_prefill_tokens
        if self.mixed:
            budget = max(self.max_prefill_tokens - len(decoding), self.runner.shape.page)
            budget = min(budget, max(self.runner.chunk_buckets))
        chunks = self._plan_chunks(budget)
        for request, start, count in chunks:
            self._grow(request, start + count)
        record = {"decode_rows": len(decoding), "chunk_tokens": sum(c for _, _, c in chunks), "kind": "idle"}
        if not decoding and not chunks:
            self.records.append(record)
            return produced

        decode_ids = [r.generated[-1] for r in decoding]
        decode_lengths = [len(r.prompt) + len(r.generated) for r in decoding]
        decode_blocks = [r.pages for r in decoding]
        chunk_items = [(r.prompt[start:start + count], start, r.pages) for r, start, count in chunks]
        if self.mixed and chunks:
            record["kind"] = "mixed"
            decode_tokens, chunk_tokens = self._mixed(decode_ids, decode_lengths, decode_blocks, chunk_items)
        else:
            decode_tokens, chunk_tokens = [], []
            if decoding:
                record["kind"] = "decode"
                decode_tokens = self._decode(decoding, decode_ids, decode_lengths, decode_blocks, record)
            if chunks:
                record["kind"] = "decode+prefill" if decoding else "prefill"
                chunk_tokens = self._prefill(chunk_items)
        for request, token in zip(decoding, decode_tokens):
            request.generated.append(int(token))
            produced.append((request.rid, int(token)))
        for (request, start, count), token in zip(chunks, chunk_tokens):
            request.prefilled = start + count
            if self.prefix_cache:
                self._publish(request)
            if request.decoding:  # the chunk completed the prompt: its last row gave the first new token
                request.generated.append(int(token))
                produced.append((request.rid, int(token)))
        self.records.append(record)
        self._retire()
        return produced

    def _decode(self, decoding, ids, lengths, blocks, record) -> list[int]:
        runner = self.runner
        if self.use_graphs:
            tokens, h2d, _ = runner.decode_rows([r.rid for r in decoding], ids, lengths, blocks)
            record["h2d_bytes"] = h2d
            record["bucket"] = next(b for b in runner.decode_buckets if b >= len(decoding))
            return tokens
        device = runner.device
        width = runner.table_width
        tables = torch.full((len(decoding), width), -1, dtype=torch.int32)
        for row, pages in enumerate(blocks):
            tables[row, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        out = runner.decode_forward(torch.tensor(ids, dtype=torch.int64, device=device),
                                    torch.tensor(lengths, dtype=torch.int32, device=device), tables.to(device))
        return out.tolist()

    def _prefill(self, chunk_items) -> list[int]:
        runner, device = self.runner, self.runner.device
        width = runner.table_width
        counts = [len(tokens) for tokens, _, _ in chunk_items]
        flat = torch.tensor([t for tokens, _, _ in chunk_items for t in tokens], dtype=torch.int64, device=device)
        tok2seq = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(counts)]).to(device)
        tokpos = torch.cat([torch.arange(start, start + n, dtype=torch.int32)
                            for (_, start, _), n in zip(chunk_items, counts)]).to(device)
        tables = torch.full((len(chunk_items), width), -1, dtype=torch.int32)
        for row, (_, _, pages) in enumerate(chunk_items):
            tables[row, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        cu = torch.zeros(len(counts) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(counts, dtype=torch.int32).cumsum(0)
        kv_lens = torch.tensor([start + n for (_, start, _), n in zip(chunk_items, counts)], dtype=torch.int32)
        out = runner.prefill_forward(flat, tok2seq, tokpos, tables.to(device), cu.to(device), kv_lens.to(device),
                                     max(counts))
        return out.tolist()

    def _mixed(self, ids, lengths, blocks, chunk_items) -> tuple[list[int], list[int]]:
        runner = self.runner
        if self.use_graphs:
            return runner.mixed_rows(ids, lengths, blocks, chunk_items)
        device, width = runner.device, runner.table_width
        live, counts = len(ids), [len(tokens) for tokens, _, _ in chunk_items]
        flat = torch.tensor(list(ids) + [t for tokens, _, _ in chunk_items for t in tokens], dtype=torch.int64)
        tok2seq = torch.cat([torch.arange(live, dtype=torch.int32),
                             *[torch.full((n,), live + i, dtype=torch.int32) for i, n in enumerate(counts)]])
        tokpos = torch.cat([torch.tensor(lengths, dtype=torch.int32) - 1,
                            *[torch.arange(start, start + n, dtype=torch.int32)
                              for (_, start, _), n in zip(chunk_items, counts)]])
        tables = torch.full((live + len(chunk_items), width), -1, dtype=torch.int32)
        for row, pages in enumerate(list(blocks) + [pages for _, _, pages in chunk_items]):
            tables[row, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        cu = torch.zeros(len(counts) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(counts, dtype=torch.int32).cumsum(0)
        kv_lens = torch.tensor([start + n for (_, start, _), n in zip(chunk_items, counts)], dtype=torch.int32)
        logit_rows = torch.cat([torch.arange(live, dtype=torch.int64), live + cu[1:].long() - 1])
        out = runner.mixed_forward(flat.to(device), tok2seq.to(device), tokpos.to(device), tables.to(device),
                                   decode_rows=live,
                                   decode_lengths=torch.tensor(lengths, dtype=torch.int32, device=device) if live else None,
                                   cu_seqlens=cu.to(device), kv_lens=kv_lens.to(device), max_query_len=max(counts),
                                   logit_rows=logit_rows.to(device)).tolist()
        return out[:live], out[live:]

    def run(self, max_iterations: int = 100000) -> dict[object, list[int]]:
        for _ in range(max_iterations):
            if not self.waiting and not self.live:
                break
            before = (len(self.waiting), len(self.live), sum(r.prefilled + len(r.generated) for r in self.live))
            self.step()
            after = (len(self.waiting), len(self.live), sum(r.prefilled + len(r.generated) for r in self.live))
            if before == after and not self.live:
                raise PagePoolExhausted("the request at the head of the queue can never be admitted")
        self.runner.check_status()
        return self.results


__all__ = ["ContinuousBatcher", "PagePool", "PagePoolExhausted"]
