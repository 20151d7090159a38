"""Head-sharded tensor parallelism, host side, on CPU with gloo (world sizes 2 and 4).

Checks what does not need a GPU: shard layout of the merged projections, the two all-reduce points, and the
vocabulary-sharded greedy exchange.  Each rank runs the CPU oracle's decode step on its shard; the group's
tokens must equal the unsharded oracle's.
"""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mini_inference_engine_b200 import workloads
from mini_inference_engine_b200.engine.model_runner.qwen3_decode import (
    Qwen3Shape,
    Qwen3Weights,
    sharded_greedy_from_pairs,
    sharded_greedy_tokens,
)
from oracle import qwen3_model

SHAPE = Qwen3Shape(layers=2, hidden=512, q_heads=4, kv_heads=2, head_dim=128, intermediate=1024, vocab=2048)
# Four ranks whose MLP shard (768 / 4 = 192 columns) is one and a half scale blocks: odd ranks start 64
# rows into a 128-row block, as the 4B model's 9728 / 8 = 1216 does at eight ranks.
SHAPE4 = Qwen3Shape(layers=2, hidden=512, q_heads=8, kv_heads=4, head_dim=128, intermediate=768, vocab=2048)


def _free_port() -> int:
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _step(weights, tp, pools, ids, lengths, tables, shape=SHAPE, **kwargs):
    return qwen3_model.decode_step(weights, pools[0], pools[1], ids, lengths, tables, q_heads=shape.q_heads // tp,
                                   kv_heads=shape.kv_heads // tp, head_dim=shape.head_dim, eps=shape.rms_eps,
                                   theta=shape.rope_theta, **kwargs)


def _inputs(shape=SHAPE):
    lengths = torch.tensor([6, 40, 17], dtype=torch.int32)
    tables = workloads.random_block_tables(lengths, num_pages=12, page=16, seed=3, extra_tokens=4)
    ids = torch.tensor([5, 900, 2000])
    generator = torch.Generator().manual_seed(11)
    keys = torch.randn(shape.layers, 12, shape.kv_heads, 16, shape.head_dim, generator=generator).to(torch.bfloat16)
    values = torch.randn(shape.layers, 12, shape.kv_heads, 16, shape.head_dim, generator=generator).to(torch.bfloat16)
    return ids, lengths, tables, keys, values


def _worker(rank: int, world: int, port: int, queue, shape=SHAPE, seed=4) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        weights = Qwen3Weights(shape, torch.device("cpu"), seed=seed, tp_rank=rank, tp_size=world)
        ids, lengths, tables, keys, values = _inputs(shape)
        local = shape.kv_heads // world
        pools = (keys[:, :, rank * local:(rank + 1) * local].contiguous(),
                 values[:, :, rank * local:(rank + 1) * local].contiguous())

        def all_reduce(tensor):
            summed = tensor.float()
            dist.all_reduce(summed)
            return summed.to(tensor.dtype)

        seen = {}

        def pick(logits):
            # The fused lm_head reports (global index, order key of the bf16 logit) per row; its exchange must
            # choose the same tokens as the exchange of the logits themselves.
            best = logits.to(torch.bfloat16).float().max(dim=-1)
            bits = best.values.to(torch.bfloat16).view(torch.int16).int() & 0xFFFF
            keys = torch.where((bits & 0x8000) != 0, ~bits & 0xFFFF, bits | 0x8000).to(torch.int32)
            seen["pairs"] = sharded_greedy_from_pairs(best.indices + weights.vocab_start, keys, world)
            return sharded_greedy_tokens(logits, weights.vocab_start, world)

        tokens = _step(weights, world, pools, ids, lengths, tables, shape, all_reduce=all_reduce, pick_tokens=pick)
        assert torch.equal(seen["pairs"], tokens)
        queue.put((rank, tokens.tolist()))
    finally:
        dist.destroy_process_group()


def _run_group(world, shape, seed):
    ids, lengths, tables, keys, values = _inputs(shape)
    full = Qwen3Weights(shape, torch.device("cpu"), seed=seed)
    expected, _, logits = _step(full, 1, (keys.clone(), values.clone()), ids, lengths, tables, shape,
                                return_hidden=True)
    top2 = logits.float().topk(2, dim=-1).values
    context = mp.get_context("spawn")
    queue = context.Queue()
    port = _free_port()
    workers = [context.Process(target=_worker, args=(rank, world, port, queue, shape, seed)) for rank in range(world)]
    for worker in workers:
        worker.start()
    results = dict(queue.get(timeout=240) for _ in workers)
    for worker in workers:
        worker.join(timeout=60)
        assert worker.exitcode == 0
    return results, expected, top2


def test_two_rank_oracle_step_matches_single_rank():
    results, expected, top2 = _run_group(2, SHAPE, 4)
    clear = (top2[:, 0] - top2[:, 1]) > top2[:, 0].abs() * 2.0 ** -6
    assert results[0] == results[1]  # both ranks agree on the sampled tokens
    for row in range(3):
        if clear[row]:  # activation groups align with the shard boundaries, so only fp32 summation order differs
            assert results[0][row] == int(expected[row])


def test_four_ranks_with_half_scale_block_shards_match_single_rank():
    """MLP shards of 192 columns: ranks 1 and 3 start 64 rows into a scale block.  Their weights are still
    slices of the unsharded quantisation (the shard sits inside its window of whole blocks), only the
    activation groups of the two half blocks are scaled per rank; tokens with a clear oracle margin agree."""

    results, expected, top2 = _run_group(4, SHAPE4, 4)
    assert results[0] == results[1] == results[2] == results[3]
    clear = (top2[:, 0] - top2[:, 1]) > top2[:, 0].abs() * 2.0 ** -4
    assert bool(clear.any())
    for row in range(3):
        if clear[row]:
            assert results[0][row] == int(expected[row])


def test_half_block_shards_are_slices_of_the_unsharded_quantisation():
    full = Qwen3Weights(SHAPE4, torch.device("cpu"), seed=4, layers=1).layers[0]
    inter = SHAPE4.intermediate
    for rank in range(4):
        shard_weights = Qwen3Weights(SHAPE4, torch.device("cpu"), seed=4, tp_rank=rank, tp_size=4, layers=1)
        shard = shard_weights.layers[0]
        window, offset, width = shard_weights.inter_window, shard_weights.inter_offset, shard_weights.inter_width
        assert (window, offset, width) == (256, 64 * (rank % 2), 192)
        lo = rank * 192
        base = lo - offset
        gate, up = shard.gate_up[:window].view(torch.uint8), shard.gate_up[window:].view(torch.uint8)
        assert torch.equal(gate[offset:offset + width], full.gate_up[lo:lo + width].view(torch.uint8))
        assert torch.equal(up[offset:offset + width], full.gate_up[inter + lo:inter + lo + width].view(torch.uint8))
        assert not gate[:offset].any() and not gate[offset + width:].any() and not up[:offset].any()
        assert torch.equal(shard.gate_up_scale[:2], full.gate_up_scale[base // 128:base // 128 + 2])
        assert torch.equal(shard.gate_up_scale[2:], full.gate_up_scale[inter // 128 + base // 128:][:2])
        down = shard.down.view(torch.uint8)
        assert torch.equal(down[:, offset:offset + width], full.down[:, lo:lo + width].view(torch.uint8))
        assert not down[:, :offset].any() and not down[:, offset + width:].any()
        assert torch.equal(shard.down_scale, full.down_scale[:, base // 128:base // 128 + 2])


def test_shards_are_slices_of_the_unsharded_weights():
    """With 128-aligned shard boundaries the per-shard block quantisation equals slicing the full one."""

    full = Qwen3Weights(SHAPE, torch.device("cpu"), seed=4, layers=1).layers[0]
    q_rows, kv_rows, inter = SHAPE.q_heads * 128, SHAPE.kv_heads * 128, SHAPE.intermediate
    for rank in range(2):
        shard = Qwen3Weights(SHAPE, torch.device("cpu"), seed=4, tp_rank=rank, tp_size=2, layers=1).layers[0]
        q = slice(rank * q_rows // 2, (rank + 1) * q_rows // 2)
        k = slice(q_rows + rank * kv_rows // 2, q_rows + (rank + 1) * kv_rows // 2)
        v = slice(q_rows + kv_rows + rank * kv_rows // 2, q_rows + kv_rows + (rank + 1) * kv_rows // 2)
        expected_qkv = torch.cat([full.qkv[q], full.qkv[k], full.qkv[v]])
        assert torch.equal(shard.qkv.view(torch.uint8), expected_qkv.view(torch.uint8))
        cols = slice(rank * q_rows // 2, (rank + 1) * q_rows // 2)
        assert torch.equal(shard.o.view(torch.uint8), full.o[:, cols].contiguous().view(torch.uint8))
        assert torch.equal(shard.o_scale, full.o_scale[:, rank * q_rows // 256:(rank + 1) * q_rows // 256])
        g = slice(rank * inter // 2, (rank + 1) * inter // 2)
        u = slice(inter + rank * inter // 2, inter + (rank + 1) * inter // 2)
        assert torch.equal(shard.gate_up.view(torch.uint8), torch.cat([full.gate_up[g], full.gate_up[u]]).view(torch.uint8))
        assert torch.equal(shard.down.view(torch.uint8), full.down[:, g].contiguous().view(torch.uint8))
    with pytest.raises(ValueError, match="tensor-parallel size"):
        Qwen3Weights(SHAPE, torch.device("cpu"), tp_size=3)


def test_sharded_greedy_single_rank_adds_the_offset():
    logits = torch.tensor([[0.1, 0.9, 0.3], [0.5, 0.2, 0.4]])
    assert sharded_greedy_tokens(logits, 100, 1).tolist() == [101, 100]


def test_peer_exchange_block_layout_and_row_ownership():
    """Host logic of the fused exchange: region offsets are aligned and disjoint, every row has one owner."""

    from mini_inference_engine_b200.engine.model_runner.peer_exchange import PeerExchange

    offsets, size = PeerExchange.layout(256, 2560)
    names = ["partial", "q", "scales", "normed", "flags"]
    assert list(offsets) == names and all(offsets[n] % 256 == 0 for n in names)
    extents = {"partial": 256 * 2560 * 2, "q": 256 * 2560, "scales": 20 * 256 * 4, "normed": 256 * 2560 * 2, "flags": 64}
    for first, second in zip(names, names[1:]):
        assert offsets[first] + extents[first] <= offsets[second]
    assert offsets["flags"] + extents["flags"] <= size
    for tp, rows in ((2, 256), (4, 37), (8, 5), (8, 256), (3, 1)):
        owners = []
        for rank in range(tp):
            ex = PeerExchange.__new__(PeerExchange)
            ex.tp, ex.rank = tp, rank
            owners.extend(ex.owned_rows(rows))
        assert owners == list(range(rows))
