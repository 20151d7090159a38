"""Head-sharded tensor parallelism on real GPUs: one process per GPU, the fused peer-memory exchange with
its NVLink flag protocol, CUDA-graph replays, and every rank's tokens against the UNSHARDED CPU oracle.

Needs 2 GPUs (runs again at 4 and 8 when they are visible).  The model is the short configuration widened
to 8 query / 8 KV heads so that it shards 8 ways; its MLP width 1536 gives 192-wide shards at 8 ranks
(1.5 scale blocks: odd ranks start 64 rows into a 128-row scale block, the case of the 4B model's 9728 / 8).
The seeds make the oracle's own top-2 logit gap at least 8 % of its top logit at every step, far outside
what fp32 summation order (and, at 8 ranks, the per-rank activation-scale groups of the half blocks) can
move, so the tokens are compared with ``==``.  NVLS is off and the exchange kernel uses plain peer loads.
"""

from __future__ import annotations

import os
import socket

import pytest
import torch

from mini_inference_engine_b200.engine.model_runner.qwen3_decode import Qwen3Shape, Qwen3Weights
from oracle_generation import oracle_generate

pytestmark = pytest.mark.gpu

SHAPE = Qwen3Shape(layers=2, hidden=512, q_heads=8, kv_heads=8, head_dim=128, intermediate=1536, vocab=2048)
WEIGHT_SEED, PROMPT_SEED = 82, 0
PLAN = ((21, 8), (70, 6), (9, 10))


def _requests(prompt_seed: int = PROMPT_SEED):
    generator = torch.Generator().manual_seed(prompt_seed)
    return [(f"r{i}", torch.randint(0, SHAPE.vocab, (n,), generator=generator).tolist(), new)
            for i, (n, new) in enumerate(PLAN)]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results, mixed: bool, kv_dtype: str = "bf16",
            weight_seed: int = WEIGHT_SEED, prompt_seed: int = PROMPT_SEED) -> None:
    import torch.distributed as dist

    from mini_inference_engine_b200.engine.model_runner.continuous import ContinuousBatcher
    from mini_inference_engine_b200.engine.model_runner.qwen3_decode import Qwen3DecodeRunner

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    outcome = None
    try:
        # Drawn on the CPU so that the shards are slices of exactly the model the parent's oracle runs.
        weights = Qwen3Weights(SHAPE, torch.device("cpu"), seed=weight_seed, tp_rank=rank, tp_size=world).to(device)
        runner = Qwen3DecodeRunner(weights, num_pages=32, max_batch=4, max_context=128,
                                   process_group=dist.group.WORLD, kv_dtype=kv_dtype)
        assert runner.exchange is not None
        batcher = ContinuousBatcher(runner, max_prefill_tokens=128, mixed=mixed)
        first, late, third = _requests(prompt_seed)
        batcher.submit(*first)
        batcher.submit(*third)
        for _ in range(3):
            batcher.step()
        batcher.submit(*late)  # its 70-token prompt arrives while the other two decode
        tokens = batcher.run()
        replays = sum(1 for record in batcher.records if "bucket" in record or record["kind"] == "mixed")
        mixed_steps = sum(1 for record in batcher.records if record["kind"] == "mixed" and record["decode_rows"])
        status = int(runner.status.item())
        outcome = {"tokens": {rid: list(t) for rid, t in tokens.items()}, "replays": replays, "status": status,
                   "mixed_steps": mixed_steps,
                   "window": (weights.inter_window, weights.inter_offset, weights.inter_width)}
        runner.release_graphs()
        torch.cuda.synchronize(device)
        dist.barrier()
        torch.cuda.synchronize(device)
        runner.exchange.close()
    except Exception as error:  # reported to the parent instead of a bare exit code
        outcome = {"error": repr(error)}
    finally:
        results[rank] = outcome
        os._exit(0 if outcome and "error" not in outcome else 1)


def _run_ranks(world: int, worker_args: tuple) -> list:
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(rank, world, port, results, *worker_args)) for rank in range(world)]
    for proc in procs:
        proc.start()
    for proc in procs:
        proc.join(timeout=300)
    for proc in procs:
        if proc.is_alive():
            proc.kill()  # this exact child, by handle
            pytest.fail("a rank did not finish in time")
    outcomes = [results.get(rank) for rank in range(world)]
    assert all(o is not None and "error" not in o for o in outcomes), outcomes
    return outcomes


@pytest.mark.parametrize("mixed", [False, True])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_every_rank_matches_the_unsharded_oracle(world, mixed):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    cpu = Qwen3Weights(SHAPE, torch.device("cpu"), seed=WEIGHT_SEED)
    expected = {}
    for rid, prompt, new in _requests():
        tokens, margin = oracle_generate(cpu, SHAPE, prompt, new)
        assert margin >= 0.08, f"the oracle itself is not decisive: margin {margin:.4f}"
        expected[rid] = tokens

    outcomes = _run_ranks(world, (mixed,))
    for rank, outcome in enumerate(outcomes):
        assert outcome["status"] == 0, (rank, outcome["status"])
        assert outcome["replays"] >= 4
        # With mixed steps the late prompt rides along with the two decoding rows through the fused exchange.
        assert (outcome["mixed_steps"] >= 1) == mixed
        assert outcome["tokens"] == expected, (rank, outcome["tokens"], expected)
    if world == 8:  # odd ranks start in the middle of a scale block
        assert outcomes[1]["window"] == (256, 64, 192) and outcomes[0]["window"] == (256, 0, 192)


KV8_WEIGHT_SEED, KV8_PROMPT_SEED, KV8_MARGIN = 226, 0, 0.1


@pytest.mark.parametrize("mixed", [False, True])
@pytest.mark.parametrize("world", [2, 4])
def test_fp8_kv_cache_under_tensor_parallelism(world, mixed):
    """The opt-in FP8 KV cache with sharded KV heads: every rank quantises the rows of its own heads (one scale
    per token and KV head, so sharding does not change a single byte), prompt chunks attend the staged pages,
    decode rows the FP8 kernel.  Expected tokens: the unsharded oracle storing every K/V row through the
    quantise -> dequantise image; its own margin is re-checked before the tokens are compared with ``==``."""

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from oracle import hot_path

    def image(rows):
        return hot_path.dequantize_kv_rows(*hot_path.quantize_kv_rows(rows))

    cpu = Qwen3Weights(SHAPE, torch.device("cpu"), seed=KV8_WEIGHT_SEED)
    expected = {}
    for rid, prompt, new in _requests(KV8_PROMPT_SEED):
        tokens, margin = oracle_generate(cpu, SHAPE, prompt, new, kv_image=image)
        assert margin >= KV8_MARGIN, f"the oracle itself is not decisive: margin {margin:.4f}"
        expected[rid] = tokens
    outcomes = _run_ranks(world, (mixed, "fp8", KV8_WEIGHT_SEED, KV8_PROMPT_SEED))
    for rank, outcome in enumerate(outcomes):
        assert outcome["status"] == 0, (rank, outcome["status"])
        assert outcome["tokens"] == expected, (rank, outcome["tokens"], expected)
