"""The CUDA-graph decode step of a small Qwen3-shaped FP8 model against the CPU oracle.

Short configuration (2 layers, width 512, 4 query / 2 KV heads of 128, vocab 2048).

* ``test_generation_tokens_equal_the_oracle``: whole generations (packed prefill + graph decode steps) on
  seeds for which the oracle's own top-2 logit gap is at least 4.5 % of its top logit at every step; the
  tokens are compared with ``==`` - the bit-exact bar for greedy tokens of the short configurations.
* ``test_tokens_within_the_noise_band_on_random_state``: decode steps from an arbitrary random cache, where
  the oracle's own logits can sit a few bf16 ulps apart; there equality is demanded wherever the oracle's
  margin exceeds the bf16 noise of two forwards, and a near-maximal token inside that band.
"""

from __future__ import annotations

import copy

import pytest
import torch

from mini_inference_engine_b200 import workloads
from mini_inference_engine_b200.engine.model_runner.qwen3_decode import (
    Qwen3DecodeRunner,
    Qwen3Shape,
    Qwen3Weights,
)
from oracle import qwen3_model

pytestmark = pytest.mark.gpu

SHAPE = Qwen3Shape(layers=2, hidden=512, q_heads=4, kv_heads=2, head_dim=128, intermediate=1024, vocab=2048)


def _cpu_weights(weights):
    clone = copy.copy(weights)
    clone.layers = [type(layer)(*[getattr(layer, f).cpu() for f in layer.__dataclass_fields__])
                    for layer in weights.layers]
    clone.embedding, clone.final_norm = weights.embedding.cpu(), weights.final_norm.cpu()
    return clone


@pytest.mark.parametrize("use_graph", [False, True])
def test_tokens_within_the_noise_band_on_random_state(use_graph, device):
    torch.manual_seed(0)
    weights = Qwen3Weights(SHAPE, device, seed=1)
    lengths = torch.tensor([5, 33, 130], dtype=torch.int32)
    steps, pages = 6, 40
    runner = Qwen3DecodeRunner(weights, num_pages=pages, max_batch=3, max_context=256, kv_init="normal")
    tables = workloads.random_block_tables(lengths, num_pages=pages, page=16, seed=2, extra_tokens=steps + 1)
    key_cpu, value_cpu = runner.key_blocks.cpu(), runner.value_blocks.cpu()
    cpu = _cpu_weights(weights)
    ids = torch.tensor([7, 1000, 2047])
    lengths_dev, tables_dev = lengths.to(device), tables.to(device)
    if use_graph:
        buffers = runner.capture(3, tables.shape[1], advance=True)
        buffers.block_tables.copy_(tables_dev)
        buffers.sequence_lengths.copy_(lengths_dev + 1)
        # Capture ran warm-up steps on the same pages: restore the pool the oracle starts from.
        runner.key_blocks.copy_(key_cpu)
        runner.value_blocks.copy_(value_cpu)
    current = lengths.clone()
    decided = 0
    for step in range(steps):
        current = current + 1  # the new token is part of the sequence
        expected, final_ref, logits_ref = qwen3_model.decode_step(
            cpu, key_cpu, value_cpu, ids, current, tables, q_heads=SHAPE.q_heads, kv_heads=SHAPE.kv_heads,
            head_dim=SHAPE.head_dim, eps=SHAPE.rms_eps, theta=SHAPE.rope_theta, return_hidden=True)
        if use_graph:
            buffers.input_ids.copy_(ids.to(device))  # keep both sides on the oracle's token stream
            runner.replay(3, advance=True)
            got, logits = buffers.output_tokens.cpu(), None
        else:
            got, logits = runner.decode_forward(ids.to(device), current.to(device), tables_dev, return_logits=True)
            got, logits = got.cpu(), logits.cpu().float()
        torch.cuda.synchronize()
        runner.check_status()
        # bf16 logits of a random tied-embedding model sit a few ulps apart, so "identical greedy tokens"
        # is asserted wherever the oracle's margin exceeds the bf16 noise of two whole forwards (4 ulps of
        # the top logit); inside that band the token must still be one of the oracle's near-maximal ones.
        reference_logits = logits_ref.float()
        top2 = reference_logits.topk(2, dim=-1).values
        noise = top2[:, 0].abs() * 2.0 ** -6
        if logits is not None:
            assert (logits - reference_logits).abs().max().item() <= 2.0 * noise.max().item()
        for row in range(3):
            if top2[row, 0] - top2[row, 1] > noise[row]:
                assert got[row] == expected[row], (step, row, got, expected)
            else:
                assert reference_logits[row, got[row]] >= top2[row, 0] - noise[row], (step, row, got, expected)
            decided += int(top2[row, 0] - top2[row, 1] > noise[row])
        ids = expected
    assert decided >= steps  # most rows are decided by a clear margin
    # The pages the step wrote equal the oracle's within rounding of the projections.
    assert (runner.key_blocks.cpu().float() - key_cpu.float()).abs().max().item() < 0.1


def test_launch_count_is_reported(device):
    weights = Qwen3Weights(SHAPE, device, seed=1)
    runner = Qwen3DecodeRunner(weights, num_pages=8, max_batch=1, max_context=64)
    tables = torch.arange(4, dtype=torch.int32, device=device).view(1, 4)
    runner.decode_forward(torch.tensor([1], device=device), torch.tensor([3], dtype=torch.int32, device=device),
                          tables)
    # Per layer: add+RMSNorm(+quant) x2, SiLU*up(+quant), 4 GEMMs, q/k-norm + RoPE + KV write, decode attention
    # and its merge (o_proj quantisation fused into both); once per step: the split-KV plan, the final norm and
    # the two launches of the fused lm_head + greedy sampling.
    assert runner.launches_per_step == 2 * 10 + 2 + 2


def test_generation_tokens_equal_the_oracle(device):
    """Short form of BASELINE configuration 3: requests arrive together, one packed whole-prompt prefill, then
    greedy decode steps (eager, then replayed from the bucket's graph that feeds its own tokens back); every
    token of every request equals the CPU oracle's."""

    from oracle_generation import oracle_generate

    cpu = Qwen3Weights(SHAPE, torch.device("cpu"), seed=31)  # drawn on the CPU: the same model on every host
    weights = cpu.to(device)
    generator = torch.Generator().manual_seed(1)
    new_tokens = 12
    prompts = [torch.randint(0, SHAPE.vocab, (n,), generator=generator).tolist() for n in (37, 5, 130)]
    expected = []
    for prompt in prompts:
        tokens, margin = oracle_generate(cpu, SHAPE, prompt, new_tokens)
        assert margin >= 0.045, f"the oracle itself is not decisive: margin {margin:.4f}"
        expected.append(tokens)
    runner = Qwen3DecodeRunner(weights, num_pages=32, max_batch=3, max_context=256)
    for use_graph in (False, True, True):  # the third run reuses the captured bucket
        runner.key_blocks.zero_()
        runner.value_blocks.zero_()
        assert runner.generate(prompts, new_tokens, use_graph=use_graph) == expected
    assert int(runner.status.item()) == 0
    assert ("decode", 3, True) in runner._graphs


