"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own CPU code.

Usage (needs a checkout of Makireddyvighnesh/mini-inference-engine; it is only
read, never copied):

    python tests/golden/make_golden.py --reference /path/to/mini-inference-engine

The reference imports itself as ``minillm_l4``; a temporary symlink of that
name is put on ``sys.path``.  Inputs are regenerated from seeds by
``mini_inference_engine_b200.workloads``, so each fixture stores only the
reference's outputs (plus a checksum of the inputs they belong to).
"""

from __future__ import annotations

import argparse
import hashlib
import sys
import tempfile
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from mini_inference_engine_b200 import workloads  # noqa: E402

OUT = Path(__file__).resolve().parent


def tensor_digest(*tensors: torch.Tensor) -> str:
    digest = hashlib.sha256()
    for tensor in tensors:
        digest.update(tensor.contiguous().view(torch.uint8).numpy().tobytes())
    return digest.hexdigest()


def import_reference(path: Path):
    link_dir = Path(tempfile.mkdtemp(prefix="minillm_ref_"))
    (link_dir / "minillm_l4").symlink_to(path)
    sys.path.insert(0, str(link_dir))
    import minillm_l4  # noqa: F401


def build_cache(lengths, *, seed, num_pages, page, kv_heads, head_dim, dtype=torch.bfloat16):
    """A reference PagedKvCache holding the same per-sequence K/V that workloads.decode_case writes."""

    from minillm_l4.engine.kv_cache.paged import PagedKvAllocator, PagedKvCache

    allocator = PagedKvAllocator(num_blocks=num_pages, block_size=page)
    cache = PagedKvCache(allocator, num_layers=1, num_kv_heads=kv_heads, head_dim=head_dim, dtype=dtype,
                         device="cpu")
    cache.key_blocks.zero_()
    cache.value_blocks.zero_()
    ids = tuple(f"s{i}" for i in range(len(lengths)))
    for i, (sid, length) in enumerate(zip(ids, lengths)):
        allocator.allocate(sid, token_count=length)
        keys, values = workloads.sequence_kv(seed * 1000 + i + 1, length, kv_heads, head_dim, dtype)
        cache.write_layer_segment(sid, 0, keys, values, start_token=0)
    return cache, ids


def golden_decode(name, lengths, *, seed, num_pages, page=16, q_heads=32, kv_heads=8, head_dim=128,
                  positions=None):
    from minillm_l4.engine.kv_cache.paged_attention import paged_attention

    case = workloads.decode_case(lengths, seed=seed, num_pages=num_pages, page=page, q_heads=q_heads,
                                 kv_heads=kv_heads, head_dim=head_dim)
    cache, ids = build_cache(lengths, seed=seed, num_pages=num_pages, page=page, kv_heads=kv_heads,
                             head_dim=head_dim)
    starts = tuple(n - 1 for n in lengths) if positions is None else tuple(positions)
    out = paged_attention(case.query, cache, ids, layer_index=0, query_start_positions=starts,
                          scale=case.scale, num_key_value_groups=q_heads // kv_heads, backend="torch")
    torch.save({
        "lengths": tuple(lengths), "seed": seed, "num_pages": num_pages, "page": page, "q_heads": q_heads,
        "kv_heads": kv_heads, "head_dim": head_dim, "positions": None if positions is None else tuple(positions),
        "query_digest": tensor_digest(case.query),
        "reference_tables": cache.block_table_tensor(ids).to(torch.int32),
        "output": out.clone(),
    }, OUT / f"{name}.pt")
    print(name, tuple(out.shape), out.dtype)


def golden_scatter_gather():
    """write_layer_segment / gather_layer on a small pool, appended in two segments."""

    from minillm_l4.engine.kv_cache.paged import PagedKvAllocator, PagedKvCache

    page, kv_heads, head_dim, num_pages = 4, 2, 8, 12
    lengths = (9, 5, 14)
    allocator = PagedKvAllocator(num_blocks=num_pages, block_size=page)
    cache = PagedKvCache(allocator, num_layers=1, num_kv_heads=kv_heads, head_dim=head_dim,
                         dtype=torch.bfloat16, device="cpu")
    cache.key_blocks.zero_()
    cache.value_blocks.zero_()
    ids = tuple(f"s{i}" for i in range(len(lengths)))
    gathered = []
    for i, (sid, length) in enumerate(zip(ids, lengths)):
        allocator.allocate(sid, token_count=length)
        keys, values = workloads.sequence_kv(77 + i, length, kv_heads, head_dim)
        first = length // 2
        cache.write_layer_segment(sid, 0, keys[:, :, :first], values[:, :, :first], start_token=0)
        cache.write_layer_segment(sid, 0, keys[:, :, first:], values[:, :, first:], start_token=first)
    for sid in ids:
        k, v = cache.gather_layer(sid, 0)
        gathered.append((k.clone(), v.clone()))
    torch.save({
        "page": page, "kv_heads": kv_heads, "head_dim": head_dim, "num_pages": num_pages, "lengths": lengths,
        "kv_seed_base": 77, "tables": cache.block_table_tensor(ids).to(torch.int32),
        "key_blocks": cache.key_blocks[0].clone(), "value_blocks": cache.value_blocks[0].clone(),
        "gathered": gathered,
    }, OUT / "scatter_gather.pt")
    print("scatter_gather")


def golden_prefill():
    """Chunk-over-prefix attention through the reference's exact path: gather_layer + aligned_prefill_sdpa."""

    from types import SimpleNamespace

    from minillm_l4.engine.generation.chunked_prefill import aligned_prefill_sdpa

    q_heads, kv_heads, head_dim, page = 4, 2, 128, 16
    prefixes, chunks = (300, 0, 77, 1290), (37, 130, 1, 256)
    case = workloads.prefill_case(seed=5, prefix_lengths=prefixes, chunk_lengths=chunks, q_heads=q_heads,
                                  kv_heads=kv_heads, head_dim=head_dim, page=page)
    from oracle import hot_path

    kb, vb = case.key_blocks.clone(), case.value_blocks.clone()
    hot_path.write_packed_kv(case.new_keys, case.new_values, case.token_to_sequence, case.token_positions,
                             case.block_tables, kb, vb)
    module = SimpleNamespace(num_key_value_groups=q_heads // kv_heads, training=False, is_causal=True)
    outputs = []
    for r, (prefix, chunk) in enumerate(zip(prefixes, chunks)):
        keys, values = hot_path.gather_kv(kb, vb, case.block_tables[r], prefix + chunk)
        start = int(case.cu_seqlens[r])
        q = case.query[start : start + chunk].transpose(0, 1).unsqueeze(0)  # [1, heads, chunk, dim]
        out, _ = aligned_prefill_sdpa(module, q, keys.unsqueeze(0), values.unsqueeze(0), None,
                                      scaling=case.scale, dropout=0.0, is_causal=True)
        outputs.append(out[0, -chunk:].clone())  # [chunk, heads, dim]
    torch.save({
        "seed": 5, "prefixes": prefixes, "chunks": chunks, "q_heads": q_heads, "kv_heads": kv_heads,
        "head_dim": head_dim, "page": page, "query_digest": tensor_digest(case.query),
        "output": torch.cat(outputs, dim=0),
    }, OUT / "prefill_chunks.pt")
    print("prefill_chunks", tuple(torch.cat(outputs, dim=0).shape))


def golden_glue():
    """The unfused Hugging Face / PyTorch ops that the reference's fused kernels reproduce bit for bit."""

    from transformers.models.qwen3 import modeling_qwen3

    generator = torch.Generator().manual_seed(3)
    hidden = torch.randn(5, 2560, generator=generator).to(torch.bfloat16)
    residual = torch.randn(5, 2560, generator=generator).to(torch.bfloat16)
    weight = (1.0 + 0.1 * torch.randn(2560, generator=generator)).to(torch.bfloat16)
    norm = modeling_qwen3.Qwen3RMSNorm(2560, eps=1e-6)
    norm.weight.data = weight.clone()
    norm = norm.to(torch.bfloat16)
    plain = norm(hidden)
    summed = hidden + residual
    fused = norm(summed)
    heads = torch.randn(5, 8, 128, generator=generator).to(torch.bfloat16)
    head_weight = (1.0 + 0.1 * torch.randn(128, generator=generator)).to(torch.bfloat16)
    head_norm = modeling_qwen3.Qwen3RMSNorm(128, eps=1e-6)
    head_norm.weight.data = head_weight.clone()
    head_norm = head_norm.to(torch.bfloat16)
    gate = torch.randn(5, 9728, generator=generator).to(torch.bfloat16)
    up = torch.randn(5, 9728, generator=generator).to(torch.bfloat16)
    q = torch.randn(2, 32, 3, 128, generator=generator).to(torch.bfloat16)
    k = torch.randn(2, 8, 3, 128, generator=generator).to(torch.bfloat16)
    positions = torch.tensor([[0, 1, 2], [4095, 4096, 40000]])
    inv_freq = 1.0 / (5_000_000.0 ** (torch.arange(0, 128, 2, dtype=torch.int64).float() / 128))
    freqs = positions.float().unsqueeze(-1) * inv_freq
    emb = torch.cat((freqs, freqs), dim=-1)
    cos, sin = emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)
    q_rot, k_rot = modeling_qwen3.apply_rotary_pos_emb(q, k, cos, sin)
    torch.save({
        "seed": 3, "hidden": hidden, "residual": residual, "weight": weight, "rms_plain": plain,
        "rms_summed": summed, "rms_fused": fused, "heads": heads, "head_weight": head_weight,
        "head_norm": head_norm(heads), "gate": gate, "up": up,
        "silu_mul": torch.nn.functional.silu(gate) * up, "q": q, "k": k, "positions": positions,
        "cos": cos, "sin": sin, "q_rot": q_rot, "k_rot": k_rot,
    }, OUT / "glue.pt")
    print("glue")


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", type=Path, required=True)
    args = parser.parse_args()
    import_reference(args.reference.resolve())
    torch.manual_seed(0)
    # BASELINE configuration 0.
    golden_decode("decode_cfg0", (17, 128, 513, 2048), seed=0, num_pages=256)
    # Explicit causal positions shorter than the stored length; odd page size; GQA 2.
    golden_decode("decode_positions", (40, 9, 33), seed=2, num_pages=16, page=8, q_heads=4, kv_heads=2,
                  head_dim=64, positions=(12, 8, 0))
    golden_decode("decode_page32", (70, 33, 200), seed=3, num_pages=16, page=32, q_heads=8, kv_heads=2,
                  head_dim=128)
    golden_scatter_gather()
    golden_prefill()
    golden_glue()


if __name__ == "__main__":
    main()
