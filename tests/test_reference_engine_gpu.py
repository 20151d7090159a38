"""The reference's OWN serving engine running on this library's kernels (the drop-in claim, end to end).

Needs a copy of the reference (Makireddyvighnesh/mini-inference-engine) that can be imported as
``minillm_l4``; looked for, in this order, at ``$MIE_REFERENCE_CHECKOUT`` (a checkout: the directory that
holds ``engine/``), ``<repository>/baseline/_ref`` (a ``pip install --target`` of it) and a directory named
``reference`` beside the repository.  Skipped when none is there.

What runs: the reference's ``ChunkedPrefillPagedRunner`` (its scheduler, page allocator, Hugging Face Qwen3
model with ``PagedQwen3Attention`` adapters, its CUDA-graph decode buckets and its mixed batches) on a tiny
random Qwen3 with head_dim 128 on the GPU, after ``install.install(minillm_l4)`` pointed every hot-path operator
at this library - as in the reference's tests/test_chunked_prefill.py:127-152, which compares the runner's
tokens with dense greedy decoding.  The model seed makes the dense model's top-2 logit gap at least 8 % of the
top logit at every step (re-checked below), so the tokens are compared with ``==``.
"""

from __future__ import annotations

import os
import sys
import tempfile
from copy import deepcopy
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def _reference_path() -> tuple[Path, bool] | None:
    """(directory to put on sys.path, whether it must first be linked as ``minillm_l4``)."""

    env = os.environ.get("MIE_REFERENCE_CHECKOUT")
    if env and (Path(env) / "engine" / "kv_cache").is_dir():
        return Path(env), True
    installed = ROOT / "baseline" / "_ref"
    if (installed / "minillm_l4" / "engine" / "kv_cache").is_dir():
        return installed, False
    beside = ROOT.parent / "reference"
    if (beside / "engine" / "kv_cache").is_dir():
        return beside, True
    return None


REFERENCE = _reference_path()
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(REFERENCE is None, reason="no copy of the reference engine on this host")]

MODEL_SEED = 149
REQUESTS = (("short", tuple(range(1, 8)), 6),
            ("long", tuple(((i * 7) % 23) + 1 for i in range(45)), 5),
            ("later", (5, 6, 7, 8, 9, 13, 2), 8))


@pytest.fixture(scope="module")
def reference():
    path, needs_link = REFERENCE
    if needs_link:
        link_dir = Path(tempfile.mkdtemp(prefix="minillm_ref_"))
        (link_dir / "minillm_l4").symlink_to(path)
        path = link_dir
    sys.path.insert(0, str(path))
    try:
        import minillm_l4  # noqa: F401
        import minillm_l4.engine.serving.chunked_prefill  # noqa: F401

        yield sys.modules["minillm_l4"]
    finally:
        sys.path.remove(str(path))


def _model():
    from transformers import Qwen3Config, Qwen3ForCausalLM

    torch.manual_seed(MODEL_SEED)
    return Qwen3ForCausalLM(Qwen3Config(
        vocab_size=24, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=2,
        num_key_value_heads=1, head_dim=128, max_position_embeddings=256, use_sliding_window=False,
        sliding_window=None, initializer_range=0.08, tie_word_embeddings=True)).eval().to(torch.bfloat16)


def _dense_greedy(model, prompt, new_tokens):
    ids, out, margin = torch.tensor([list(prompt)]), [], float("inf")
    with torch.inference_mode():
        for _ in range(new_tokens):
            logits = model(input_ids=ids).logits[0, -1].float()
            top2 = logits.topk(2).values
            margin = min(margin, float((top2[0] - top2[1]) / top2[0].abs().clamp_min(1e-30)))
            out.append(int(logits.argmax()))
            ids = torch.cat([ids, torch.tensor([[out[-1]]])], dim=1)
    return out, margin


def _run(reference, model, device, **runner_kwargs):
    from minillm_l4.benchmarks.core.harness import BenchmarkHarness
    from minillm_l4.benchmarks.core.schemas import HarnessConfig, RequestSpec, WorkloadSpec
    from minillm_l4.engine.serving.chunked_prefill import ChunkedPrefillPagedRunner

    requests = tuple(RequestSpec(rid, prompt, new, scheduled_arrival_ms=0.1 * i)
                     for i, (rid, prompt, new) in enumerate(REQUESTS))
    runner = ChunkedPrefillPagedRunner(deepcopy(model).to(device), block_size=16, num_blocks=40, max_batch_size=3,
                                       device=str(device), enable_prefix=False, **runner_kwargs)
    result = BenchmarkHarness(HarnessConfig(
        repetitions=1, warmup_repetitions=0, respect_arrival_schedule=True, collect_gpu=False,
        collect_system_telemetry=False)).run_trace(
        WorkloadSpec(name="drop-in", seed=47, device=device.type, requests=requests, arrival_pattern="fixed_rate"),
        runner)
    tokens = {row["request_id"]: row["outcome"]["generated_token_ids"] for row in result.runs[0]["requests"]}
    summary = runner.last_summary
    runner.close()
    return tokens, summary


@pytest.fixture(scope="module")
def expected(reference):
    model = _model()
    tokens = {}
    for rid, prompt, new in REQUESTS:
        tokens[rid], margin = _dense_greedy(model, prompt, new)
        assert margin >= 0.08, f"the dense model itself is not decisive for {rid}: margin {margin:.4f}"
    # The reference's own CPU path (torch backend) gives the same tokens: its published exactness claim.
    cpu_tokens, _ = _run(reference, model, torch.device("cpu"), max_prefill_tokens=16, prefill_chunk_size=16,
                         decode_backend="torch")
    assert cpu_tokens == tokens
    return tokens


@pytest.fixture()
def installed(reference):
    from mini_inference_engine_b200 import _lib, install

    count = install.install(reference)
    assert count > 20
    before = int(_lib.load().mie_launch_count())
    yield lambda: int(_lib.load().mie_launch_count()) - before
    install.uninstall()


@pytest.mark.parametrize("variant", ["chunked_graphs", "packed_flash", "mixed_batch", "mixed_graph_decode"])
def test_reference_runner_on_installed_kernels(variant, reference, expected, installed, device, status_clean):
    kwargs = {
        "chunked_graphs": dict(max_prefill_tokens=16, prefill_chunk_size=16, decode_backend="triton",
                               cuda_graphs=True, graph_batch_sizes=(1, 2, 4)),
        "packed_flash": dict(max_prefill_tokens=64, prefill_chunk_size=None, decode_backend="triton",
                             packed_attention_backend="triton_flash"),
        "mixed_batch": dict(max_prefill_tokens=24, prefill_chunk_size=None, decode_backend="triton",
                            mixed_batch=True),
        "mixed_graph_decode": dict(max_prefill_tokens=24, prefill_chunk_size=None, decode_backend="triton",
                                   mixed_batch=True, cuda_graphs=True, graph_mixed_decode=True,
                                   graph_batch_sizes=(1, 2, 4)),
    }[variant]
    paged = sys.modules["minillm_l4.engine.kv_cache.paged_attention"]
    assert paged.triton_paged_decode_attention.__module__.startswith("mini_inference_engine_b200")
    tokens, summary = _run(reference, _model(), device, **kwargs)
    assert tokens == expected
    assert installed() > 0  # kernels of this library were launched
    if "cuda_graphs" in kwargs:
        # The reference captured ITS decode graphs over the rebound operators and replayed them.
        assert summary["graph_replays"] > 0, summary.get("graph_fallback_reason")


def test_reference_fused_installer_over_rebound_operators(reference, expected, installed, device, status_clean):
    """The reference's ``install_fused_kernels`` resolves ``rms_norm`` / ``silu_mul`` / ``apply_rotary_pos_emb``
    in its own module at call time, so after ``install()`` it wires the model to this library's kernels
    (including the RoPE of the paged attention adapter)."""

    from minillm_l4.engine.kernels import fused as reference_fused
    from transformers.models.qwen3 import modeling_qwen3

    from mini_inference_engine_b200.engine.kernels import fused as ours

    assert reference_fused.rms_norm is ours.rms_norm and reference_fused.apply_rotary_pos_emb is ours.apply_rotary_pos_emb
    model = _model().to(device)
    adapter = sys.modules["minillm_l4.engine.kv_cache.qwen3_paged"]
    original_rope = modeling_qwen3.apply_rotary_pos_emb
    assert reference_fused.install_fused_kernels(model)
    try:
        assert adapter.apply_rotary_pos_emb is ours.apply_rotary_pos_emb
        tokens, _ = _run(reference, model, device, max_prefill_tokens=16, prefill_chunk_size=16,
                         decode_backend="triton")
        assert tokens == expected
    finally:
        reference_fused.uninstall_fused_kernels(model)
    assert modeling_qwen3.apply_rotary_pos_emb is original_rope


def test_own_fused_installer_patches_the_adapter_rope(reference, device):
    from transformers.models.qwen3 import modeling_qwen3

    from mini_inference_engine_b200.engine.kernels import fused as ours

    adapter = sys.modules["minillm_l4.engine.kv_cache.qwen3_paged"]
    before = (modeling_qwen3.apply_rotary_pos_emb, adapter.apply_rotary_pos_emb)
    model = _model().to(device)
    assert ours.install_fused_kernels(model)
    try:
        assert modeling_qwen3.apply_rotary_pos_emb is adapter.apply_rotary_pos_emb
        assert adapter.apply_rotary_pos_emb is not before[1]
        ids = torch.tensor([[1, 2, 3, 4, 5]], device=device)
        fused_logits = model(input_ids=ids).logits
    finally:
        ours.uninstall_fused_kernels(model)
    assert (modeling_qwen3.apply_rotary_pos_emb, adapter.apply_rotary_pos_emb) == before
    plain_logits = model(input_ids=ids).logits
    assert (fused_logits.float() - plain_logits.float()).abs().max().item() <= 0.05 * plain_logits.float().abs().max().item()
