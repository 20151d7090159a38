"""FP8 (e4m3) KV cache on the GPU: the decode kernel over the quantised pool and the writer that fills it.

Oracle (``oracle.hot_path.paged_decode_attention_fp8_kv``): the reference's torch decode path fed the
quantise -> dequantise image of the bf16 pages.  PARITY UNPINNED against the reference itself: it has no FP8
KV cache (it names one as future work, docs/phase_notes/roofline.md:76).  Bounds: the kernel against that
oracle within 2e-2 max-abs, the bound of the bf16 path (the kernel works on the exact e4m3 x scale products,
the oracle on their bf16 roundings); the quantised pages themselves bit-exact against the oracle's quantiser.
"""

from __future__ import annotations

import pytest
import torch

from mini_inference_engine_b200 import _lib, workloads
from mini_inference_engine_b200.engine.kv_cache.fp8_kv import Fp8KvPool, launch_decode_attention_kv8, quantize_kv_rows
from mini_inference_engine_b200.engine.kv_cache.triton_paged_attention import decode_scratch
from oracle import hot_path

pytestmark = pytest.mark.gpu
ATOL = 2e-2


def _pool_from_case(case, device):
    pages, kv_heads = int(case.key_blocks.shape[0]), int(case.key_blocks.shape[1])
    pool = Fp8KvPool(1, pages, kv_heads, device)
    pool.fill_from(0, case.key_blocks.to(device), case.value_blocks.to(device))
    return pool


def _run(case, pool, device, *, policy=1, positions=None, quantized=False):
    dev = case.to(device)
    batch, q_heads = int(dev.query.shape[0]), int(dev.query.shape[1])
    out = torch.full_like(dev.query, float("nan"))
    total = int(case.sequence_lengths.sum())
    scratch = decode_scratch(batch, q_heads, pool.kv_heads, 128, total, device)
    q_out = None
    if quantized:
        q_out = (torch.zeros(batch, q_heads * 128, dtype=torch.float8_e4m3fn, device=device),
                 torch.zeros(q_heads, batch, dtype=torch.float32, device=device))
    launch_decode_attention_kv8(dev.query, out, pool.data[0], pool.scales[0], dev.block_tables, dev.sequence_lengths,
                                None if positions is None else positions.to(device), scale=case.scale,
                                scratch=scratch, split_policy=policy, quantized_out=q_out)
    torch.cuda.synchronize()
    return out.transpose(1, 2).cpu(), q_out


def test_torch_quantiser_matches_the_oracle_quantiser(device):
    rows = torch.randn(5, 3, 16, 128, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16)
    rows[0, 0, 0] = 0
    rows[1, 1, 1] *= 1e4
    q_ref, s_ref = hot_path.quantize_kv_rows(rows)
    q, s = quantize_kv_rows(rows.to(device))
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)
    assert s_ref[0, 0, 0] == 0 and not q_ref[0, 0, 0].any()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("policy", [0, 1, 64])
def test_decode_over_fp8_pages_matches_the_dequantised_oracle(dtype, policy, device, status_clean):
    lengths = (1, 15, 16, 17, 300, 1025, 4096, 2049)
    case = workloads.decode_case(lengths, seed=11, num_pages=512, dtype=dtype)
    expected, _, _ = hot_path.paged_decode_attention_fp8_kv(case.query, case.key_blocks, case.value_blocks,
                                                            case.block_tables, case.sequence_lengths, case.scale)
    pool = _pool_from_case(case, device)
    got, _ = _run(case, pool, device, policy=policy)
    assert torch.isfinite(got.float()).all()
    assert (got.float() - expected.float()).abs().max().item() <= ATOL


def test_baseline_configuration_0_on_fp8_pages(golden, device, status_clean):
    """BASELINE configuration 0's shapes; also against the bf16 golden output with the quantisation error
    of e4m3 rows (3 mantissa bits) allowed for."""

    meta = golden("decode_cfg0")
    case = workloads.decode_case(meta["lengths"], seed=meta["seed"], num_pages=meta["num_pages"], page=meta["page"],
                                 q_heads=meta["q_heads"], kv_heads=meta["kv_heads"], head_dim=meta["head_dim"])
    expected, _, _ = hot_path.paged_decode_attention_fp8_kv(case.query, case.key_blocks, case.value_blocks,
                                                            case.block_tables, case.sequence_lengths, case.scale)
    pool = _pool_from_case(case, device)
    got, _ = _run(case, pool, device)
    assert (got.float() - expected.float()).abs().max().item() <= ATOL
    assert (got.float() - meta["output"].float()).abs().max().item() <= 0.15


def test_positions_garbage_tails_gqa_groups_and_quantised_output(device, status_clean):
    # Explicit query positions shorten the read; pages past the read length hold NaN bytes and huge scales.
    lengths = (40, 7, 130)
    case = workloads.decode_case(lengths, seed=3, num_pages=64, q_heads=16, kv_heads=2)  # 8 query heads per KV head
    positions = torch.tensor([20, 6, 64])
    expected, _, _ = hot_path.paged_decode_attention_fp8_kv(case.query, case.key_blocks, case.value_blocks,
                                                            case.block_tables, case.sequence_lengths, case.scale,
                                                            query_positions=positions)
    pool = _pool_from_case(case, device)
    table = case.block_tables
    for row, (length, position) in enumerate(zip(lengths, positions.tolist())):
        read = min(length, position + 1)
        page, slot = int(table[row, read // 16]), read % 16
        pool.data[0, page, :, :, slot:] = 0x7F       # e4m3 NaN
        pool.scales[0, page, :, :, slot:] = float("inf")
    got, q_out = _run(case, pool, device, positions=positions, quantized=True)
    assert torch.isfinite(got.float()).all()
    assert (got.float() - expected.float()).abs().max().item() <= ATOL
    # The e4m3 copy for o_proj is the quantisation of the bf16 rows that were written.
    q8, scales = q_out
    rows = got.reshape(3, 16, 128)
    want_q, want_s = hot_path.quantize_kv_rows(rows)
    assert torch.equal(scales.t().cpu(), want_s)
    assert torch.equal(q8.cpu().view(torch.uint8).view(3, 16, 128), want_q)


def test_writer_fills_the_pool_like_the_oracle_quantiser(device, status_clean):
    """``mie_qkv_norm_rope_write_kv8``: q rows equal the bf16 writer's, the K/V bytes and scales equal the
    quantisation of the K/V rows the bf16 writer stores."""

    torch.manual_seed(0)
    tokens, q_heads, kv_heads, pages = 37, 4, 2, 8
    qkv = torch.randn(tokens, (q_heads + 2 * kv_heads) * 128, device=device).to(torch.bfloat16)
    qkv[3] = 0
    q_w = (1 + 0.1 * torch.randn(128, device=device)).to(torch.bfloat16)
    k_w = (1 + 0.1 * torch.randn(128, device=device)).to(torch.bfloat16)
    from mini_inference_engine_b200.engine.model_runner.qwen3_decode import Qwen3Shape, rope_table

    rope = rope_table(Qwen3Shape(), 128, device)
    positions = torch.arange(tokens, dtype=torch.int32, device=device) + 5
    seq = torch.zeros(tokens, dtype=torch.int32, device=device)
    tables = torch.tensor([[5, 2, 7, 0]], dtype=torch.int32, device=device)
    lib, stream = _lib.load(), _lib.stream_arg(device)
    status = _lib.status_word(device)
    q_ref = torch.empty(tokens, q_heads, 128, dtype=torch.bfloat16, device=device)
    keys = torch.zeros(pages, kv_heads, 16, 128, dtype=torch.bfloat16, device=device)
    values = torch.zeros_like(keys)
    _lib.check(lib.mie_qkv_norm_rope_write(
        _lib.ptr(qkv), qkv.stride(0), _lib.ptr(q_w), _lib.ptr(k_w), _lib.ptr(rope), 128, _lib.index_arg(positions),
        _lib.index_arg(seq), _lib.index_arg(tables), _lib.ptr(q_ref), _lib.view4_arg(keys), _lib.view4_arg(values),
        tokens, q_heads, kv_heads, 16, pages, 1, 4, 1e-6, _lib.ptr(status), stream))
    pool = Fp8KvPool(1, pages, kv_heads, device)
    q_got = torch.empty_like(q_ref)
    _lib.check(lib.mie_qkv_norm_rope_write_kv8(
        _lib.ptr(qkv), qkv.stride(0), _lib.ptr(q_w), _lib.ptr(k_w), _lib.ptr(rope), 128, _lib.index_arg(positions),
        _lib.index_arg(seq), _lib.index_arg(tables), _lib.ptr(q_got), _lib.ptr(pool.data[0]),
        pool.page_stride_bytes, _lib.ptr(pool.scales[0]), tokens, q_heads, kv_heads, pages, 1, 4, 1e-6,
        _lib.ptr(status), stream))
    torch.cuda.synchronize()
    assert torch.equal(q_got, q_ref)
    for which, dense in enumerate((keys, values)):
        want_q, want_s = hot_path.quantize_kv_rows(dense.cpu())
        assert torch.equal(pool.data[0, :, :, which].cpu(), want_q)
        assert torch.equal(pool.scales[0, :, :, which].cpu(), want_s)


def test_arguments_are_checked(device):
    case = workloads.decode_case((20,), seed=1, num_pages=8).to(device)
    pool = Fp8KvPool(1, 8, 8, device)
    out = torch.empty_like(case.query)
    scratch = decode_scratch(1, 32, 8, 128, 64, device)
    with pytest.raises(ValueError, match="head_dim 128"):
        launch_decode_attention_kv8(case.query[..., :64], out[..., :64], pool.data[0], pool.scales[0],
                                    case.block_tables, case.sequence_lengths, None, scale=1.0, scratch=scratch)
    shifted = pool.data[0].view(-1)[128:128 + 7 * 8 * 4096].view(7, 8, 2, 16, 128)  # base 128 bytes off the grid
    with pytest.raises(ValueError, match="1 KiB aligned"):
        launch_decode_attention_kv8(case.query, out, shifted, pool.scales[0][:7], case.block_tables,
                                    case.sequence_lengths, None, scale=1.0, scratch=scratch)


def test_decode_step_over_the_fp8_cache(device):
    """The runner's decode step with ``kv_dtype="fp8"`` (writer + attention over the quantised pool, eager and
    as a bucket graph) against the oracle's step over the dequantised image of the same cache."""

    from mini_inference_engine_b200.engine.model_runner.qwen3_decode import Qwen3DecodeRunner, Qwen3Shape, Qwen3Weights
    from oracle import qwen3_model

    shape = Qwen3Shape(layers=2, hidden=512, q_heads=4, kv_heads=2, head_dim=128, intermediate=1024, vocab=2048)
    cpu = Qwen3Weights(shape, torch.device("cpu"), seed=36)
    runner = Qwen3DecodeRunner(cpu.to(device), num_pages=24, max_batch=4, max_context=128, kv_dtype="fp8")
    generator = torch.Generator().manual_seed(2)
    pages = runner.total_pages
    keys = torch.randn(2, pages, 2, 16, 128, generator=generator).to(torch.bfloat16)
    values = torch.randn(2, pages, 2, 16, 128, generator=generator).to(torch.bfloat16)
    for layer in range(2):
        runner.kv8.fill_from(layer, keys[layer].to(device), values[layer].to(device))
    blocks = [[3, 7], [1], [9, 4, 11]]
    lengths, ids = [20, 5, 40], [17, 900, 2047]
    tables = torch.full((3, runner.table_width), -1, dtype=torch.int32)
    for row, page_ids in enumerate(blocks):
        tables[row, :len(page_ids)] = torch.tensor(page_ids, dtype=torch.int32)
    got, logits = runner.decode_forward(torch.tensor(ids, device=device),
                                        torch.tensor(lengths, dtype=torch.int32, device=device), tables.to(device),
                                        return_logits=True)
    runner.check_status()
    # Oracle: the dequantised image of the cache; the new token's rows go through the same image.
    key_image = torch.stack([hot_path.dequantize_kv_rows(*hot_path.quantize_kv_rows(keys[l])) for l in range(2)])
    value_image = torch.stack([hot_path.dequantize_kv_rows(*hot_path.quantize_kv_rows(values[l])) for l in range(2)])
    expected, _, want = qwen3_model.decode_step(cpu, key_image, value_image, torch.tensor(ids),
                                                torch.tensor(lengths, dtype=torch.int32), tables, q_heads=4, kv_heads=2,
                                                head_dim=128, eps=shape.rms_eps, theta=shape.rope_theta,
                                                return_hidden=True,
                                                kv_image=lambda rows: hot_path.dequantize_kv_rows(
                                                    *hot_path.quantize_kv_rows(rows)))
    want = want.float()
    # Two layers of e4m3 activation quantisation sit behind the attention: a last-bit difference in an
    # attention row can flip the rounding of an activation, so logits agree to the quantisation noise of the
    # model (the bf16-cache step is held to 2 * 2**-6 of the top logit), not to attention tolerance.
    assert (logits.cpu().float() - want).abs().max().item() <= 0.08 * want.abs().max().item()
    top2 = want.topk(2, dim=-1).values
    for row in range(3):
        if (top2[row, 0] - top2[row, 1]) > 0.1 * top2[row, 0].abs():
            assert int(got[row]) == int(expected[row])
    # The written rows: position length-1 of every request holds the quantisation of the oracle's bf16 row.
    for row, (length, page_ids) in enumerate(zip(lengths, blocks)):
        page, slot = page_ids[(length - 1) // 16], (length - 1) % 16
        want_q, want_s = hot_path.quantize_kv_rows(key_image[0, page, :, slot])
        assert torch.equal(runner.kv8.scales[0, page, :, 0, slot].cpu(), want_s)
        assert torch.equal(runner.kv8.data[0, page, :, 0, slot].cpu(), want_q)
    # The same rows through a bucket graph give the same tokens.
    tokens, _, _ = runner.decode_rows(["a", "b", "c"], ids, lengths, blocks)
    assert tokens == got.tolist()


def _image(rows):
    return hot_path.dequantize_kv_rows(*hot_path.quantize_kv_rows(rows))


def test_prompt_chunks_over_the_fp8_cache(device):
    """A prompt in two chunks (the second over a cached prefix) next to a whole prompt: the writer quantises
    the new rows, the chunk kernel attends the dequantised pages.  Against the oracle's packed step whose
    stored rows go through the same quantise -> dequantise image."""

    from mini_inference_engine_b200.engine.model_runner.qwen3_decode import Qwen3DecodeRunner, Qwen3Shape, Qwen3Weights
    from oracle import qwen3_model

    shape = Qwen3Shape(layers=2, hidden=512, q_heads=4, kv_heads=2, head_dim=128, intermediate=1024, vocab=2048)
    cpu = Qwen3Weights(shape, torch.device("cpu"), seed=36)
    runner = Qwen3DecodeRunner(cpu.to(device), num_pages=24, max_batch=4, max_context=128, kv_dtype="fp8")
    generator = torch.Generator().manual_seed(4)
    prompt_a = torch.randint(0, shape.vocab, (45,), generator=generator)
    prompt_b = torch.randint(0, shape.vocab, (19,), generator=generator)
    blocks = [[5, 2, 9], [7, 1]]
    tables = torch.full((2, runner.table_width), -1, dtype=torch.int32)
    for row, page_ids in enumerate(blocks):
        tables[row, :len(page_ids)] = torch.tensor(page_ids, dtype=torch.int32)
    keys = torch.zeros(2, runner.total_pages, 2, 16, 128, dtype=torch.bfloat16)
    values = torch.zeros_like(keys)
    kwargs = dict(q_heads=4, kv_heads=2, head_dim=128, eps=shape.rms_eps, theta=shape.rope_theta, return_hidden=True,
                  kv_image=_image)
    # step 1: the first 30 tokens of A; step 2: the last 15 of A (prefix 30) packed with all of B
    steps = [
        (prompt_a[:30], [0] * 30, list(range(30)), [0, 30], [30]),
        (torch.cat([prompt_a[30:], prompt_b]), [0] * 15 + [1] * 19, list(range(30, 45)) + list(range(19)),
         [0, 15, 34], [45, 19]),
    ]
    for ids, owners, positions, cu, kv in steps:
        meta = [torch.tensor(x, dtype=torch.int32) for x in (owners, positions, cu, kv)]
        expected, _, want = qwen3_model.prefill_step(cpu, keys, values, ids, meta[0], meta[1], tables, meta[2],
                                                     meta[3], **kwargs)
        got, logits = runner.prefill_forward(ids.to(device), meta[0].to(device), meta[1].to(device),
                                             tables.to(device), meta[2].to(device), meta[3].to(device),
                                             max(b - a for a, b in zip(cu, cu[1:])), return_logits=True)
        runner.check_status()
        want = want.float()
        assert (logits.cpu().float() - want).abs().max().item() <= 0.08 * want.abs().max().item()
        top2 = want.topk(2, dim=-1).values
        for row in range(len(kv)):
            if (top2[row, 0] - top2[row, 1]) > 0.1 * top2[row, 0].abs():
                assert int(got[row]) == int(expected[row])
    # Layer 0 sees the same inputs on both sides, so its cache rows are the oracle's rows quantised, bit for bit
    # (the oracle's pool holds the bf16 image; quantising an image again reproduces its bytes and scales).
    for row, length in ((0, 45), (1, 19)):
        for position in (0, 15, 16, length - 1):
            page, slot = blocks[row][position // 16], position % 16
            for which, pool in enumerate((keys, values)):
                want_q, want_s = hot_path.quantize_kv_rows(pool[0, page, :, slot])
                assert torch.equal(runner.kv8.scales[0, page, :, which, slot].cpu(), want_s)
                assert torch.equal(runner.kv8.data[0, page, :, which, slot].cpu(), want_q)


@pytest.mark.parametrize("mixed", [False, True])
def test_generation_over_the_fp8_cache_equals_the_oracle(mixed, device):
    """Continuous batching with ``kv_dtype="fp8"`` (chunked prompts, bucket graphs, and with ``mixed`` the captured
    prefill + decode steps) against the oracle generating over the quantise -> dequantise image of its cache.
    Seeds chosen so that the oracle's top-2 gap is at least 10 % of its top logit at every step (re-checked
    here): outside the noise of e4m3 rows, so the tokens are compared with ``==``."""

    from mini_inference_engine_b200.engine.model_runner.continuous import ContinuousBatcher
    from mini_inference_engine_b200.engine.model_runner.qwen3_decode import Qwen3DecodeRunner, Qwen3Shape, Qwen3Weights
    from oracle_generation import oracle_generate

    shape = Qwen3Shape(layers=2, hidden=512, q_heads=4, kv_heads=2, head_dim=128, intermediate=1024, vocab=2048)
    cpu = Qwen3Weights(shape, torch.device("cpu"), seed=33)
    generator = torch.Generator().manual_seed(0)
    requests = [(f"r{i}", torch.randint(0, shape.vocab, (n,), generator=generator).tolist(), new)
                for i, (n, new) in enumerate([(37, 4), (150, 8), (20, 12)])]
    expected = {}
    for rid, prompt, new in requests:
        expected[rid], margin = oracle_generate(cpu, shape, prompt, new, kv_image=_image)
        assert margin >= 0.1, f"the oracle itself is not decisive for {rid}: margin {margin:.4f}"
    runner = Qwen3DecodeRunner(cpu.to(device), num_pages=48, max_batch=4, max_context=256, max_chunks=4,
                               chunk_buckets=(128,), kv_dtype="fp8")
    batcher = ContinuousBatcher(runner, max_prefill_tokens=128, mixed=mixed)
    for rid, prompt, new in requests:
        batcher.submit(rid, prompt, new)
    results = batcher.run()
    assert int(runner.status.item()) == 0
    for rid, _, _ in requests:
        assert results[rid] == expected[rid], rid
