"""Single-kernel micro-benchmarks of the hot path (also the small cases profiled with ncu).

    python microbench.py decode --concurrency 64
    python microbench.py gemm --shape qkv --rows 256
    python microbench.py prefill --requests 6
    python microbench.py lm_head --rows 8

Each prints one JSON line with the CUDA-event time per launch (median of the repeats, L2 flushed by a
256 MiB fill between repeats) and the algorithmic bytes / FLOPs of the launch.
"""

from __future__ import annotations

import argparse
import json
import statistics

import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from mini_inference_engine_b200 import _lib, workloads  # noqa: E402
from mini_inference_engine_b200.engine.kernels import sm89_fp8  # noqa: E402
from mini_inference_engine_b200.engine.kv_cache import (  # noqa: E402
    triton_flash_prefill_attention,
    triton_write_packed_kv,
)
from mini_inference_engine_b200.engine.kv_cache.triton_paged_attention import (  # noqa: E402
    decode_scratch,
    launch_decode_attention,
)


def _time(run, repeats: int, device: torch.device) -> float:
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    for _ in range(3):
        run()
    torch.cuda.synchronize(device)
    samples = []
    for _ in range(repeats):
        flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        run()
        end.record()
        torch.cuda.synchronize(device)
        samples.append(start.elapsed_time(end))
    return statistics.median(samples)


def decode(args, device) -> dict:
    if getattr(args, "lengths", None):
        lengths = torch.tensor([int(n) for n in args.lengths])  # e.g. BASELINE configuration 0: 17,128,513,2048
        args.concurrency = len(lengths)
    else:
        lengths = workloads.lognormal_contexts(args.concurrency, seed=args.concurrency)
    total = int(lengths.sum())
    pages = sum(-(-int(n) // workloads.PAGE) for n in lengths) + 8
    tables = workloads.random_block_tables(lengths, num_pages=pages, seed=1)
    if getattr(args, "sequential_tables", False):
        # Every request's pages in ascending order, requests back to back: the placement a fresh allocator gives,
        # against the random placement the benchmark (and the reference's own benchmarks) use.
        live = tables >= 0
        tables[live] = torch.arange(int(live.sum()), dtype=tables.dtype)
    tables = tables.to(device)
    kv_heads, q_heads = workloads.KV_HEADS // args.tp, workloads.Q_HEADS // args.tp
    query = torch.randn(args.concurrency, q_heads, 1, 128, device=device).to(torch.bfloat16)
    out = torch.empty_like(query)
    lens = lengths.to(torch.int32).to(device)
    scratch = decode_scratch(args.concurrency, q_heads, kv_heads, 128, total, device)
    if args.kv_dtype == "fp8":
        from mini_inference_engine_b200.engine.kv_cache.fp8_kv import Fp8KvPool, launch_decode_attention_kv8

        pool = Fp8KvPool(1, pages, kv_heads, device)
        pool.data.random_(0, 256).bitwise_and_(0xBF)  # random e4m3 bytes without NaN patterns
        pool.scales.uniform_(0.004, 0.012)
        bytes_per_token = pool.bytes_per_token()

        def run(**plan):
            launch_decode_attention_kv8(query, out, pool.data[0], pool.scales[0], tables, lens, None,
                                        scale=128 ** -0.5, scratch=scratch, split_policy=args.split_policy, **plan)
    else:
        key_blocks = torch.randn(pages, kv_heads, workloads.PAGE, 128, device=device).to(torch.bfloat16)
        value_blocks = torch.randn(pages, kv_heads, workloads.PAGE, 128, device=device).to(torch.bfloat16)
        bytes_per_token = 2 * kv_heads * 128 * 2

        def run(**plan):
            launch_decode_attention(query, out, key_blocks, value_blocks, tables, lens, None, scale=128 ** -0.5,
                                    max_total_tokens=total, scratch=scratch, split_policy=args.split_policy, **plan)

    if getattr(args, "reuse_plan", False):
        # As inside a model step: the split-KV plan is built once (layer 0) and every later layer's launch
        # reuses it with its own work counter, so the timed call is decode + merge only.
        def run_reused():
            run(use_plan=True, plan_slot=next_slot())

        counter = {"n": 0}

        def next_slot():
            counter["n"] = counter["n"] % 63 + 1
            return counter["n"]

        run(plan_only=True)
        samples = []
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
        for rep in range(args.repeats + 3):
            if counter["n"] == 63:
                run(plan_only=True)
                counter["n"] = 0
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run_reused()
            e1.record()
            torch.cuda.synchronize(device)
            if rep >= 3:
                samples.append(e0.elapsed_time(e1))
        ms = statistics.median(samples)
    else:
        ms = _time(run, args.repeats, device)
    algorithmic = total * bytes_per_token + 2 * query.numel() * 2
    return {"kernel": f"paged decode attention (plan + decode + merge), {args.kv_dtype} KV",
            "concurrency": args.concurrency, "total_context_tokens": total, "us_per_launch": ms * 1e3,
            "kv_bytes_per_token": bytes_per_token, "algorithmic_bytes": algorithmic,
            "gb_per_s": algorithmic / ms / 1e6}


def gemm(args, device) -> dict:
    n, k = workloads.GEMM_SHAPES[args.shape]
    weights = [(torch.randn(n, k, device=device) * 32).clamp(-448, 448).to(torch.float8_e4m3fn)
               for _ in range(args.copies)]
    scales = torch.rand((n + 127) // 128, (k + 127) // 128, device=device) * 0.09 + 0.001
    x = torch.randn(args.rows, k, device=device).to(torch.bfloat16)
    quantized, a_scales = sm89_fp8.quantize_activation_kmajor(x)
    out = torch.empty(args.rows, n, dtype=torch.bfloat16, device=device)

    def run_all():
        for weight in weights:
            sm89_fp8.launch_fp8_gemm(quantized, a_scales, weight, scales, out, args.rows, k)

    run_all()
    torch.cuda.synchronize(device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run_all()
    ms = _time(graph.replay, args.repeats, device) / args.copies
    flops = 2.0 * args.rows * n * k
    traffic = n * k + args.rows * k + 2 * args.rows * n
    return {"kernel": "fp8 block-scaled gemm", "shape": args.shape, "m": args.rows, "n": n, "k": k,
            "us_per_launch": ms * 1e3, "tflops": flops / ms / 1e9, "gb_per_s": traffic / ms / 1e6}


def prefill(args, device) -> dict:
    case = workloads.prefill_case(requests=args.requests, seed=0).to(device)
    triton_write_packed_kv(case.new_keys, case.new_values, case.token_to_sequence, case.token_positions,
                           case.block_tables, case.key_blocks, case.value_blocks)

    def run():
        triton_flash_prefill_attention(case.query, case.key_blocks, case.value_blocks, case.block_tables,
                                       case.cu_seqlens, case.kv_lens, max_query_len=max(case.chunk_lengths),
                                       scale=case.scale)

    ms = _time(run, args.repeats, device)
    flops = sum(4 * workloads.Q_HEADS * 128 * (c * p + c * (c + 1) / 2)
                for p, c in zip(case.prefix_lengths, case.chunk_lengths))
    return {"kernel": "chunked prefill attention", "prefixes": case.prefix_lengths, "chunks": case.chunk_lengths,
            "us_per_launch": ms * 1e3, "tflops": flops / ms / 1e9}


def lm_head(args, device) -> dict:
    vocab, hidden = 151936, 2560
    weight = (torch.randn(vocab, hidden, device=device) * 0.02).to(torch.bfloat16)
    x = torch.randn(args.rows, hidden, device=device).to(torch.bfloat16)
    keys = torch.zeros(256, dtype=torch.int64, device=device)
    tokens = torch.empty(args.rows, dtype=torch.int64, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    lib = _lib.load()

    def run():
        _lib.check(lib.mie_lm_head_argmax(_lib.ptr(x), x.stride(0), _lib.ptr(weight), weight.stride(0), args.rows,
                                          vocab, hidden, 0, _lib.ptr(keys), _lib.ptr(tokens), None, _lib.ptr(status),
                                          _lib.stream_arg(device)))

    ms = _time(run, args.repeats, device)
    algorithmic = vocab * hidden * 2 + args.rows * hidden * 2 + args.rows * 8
    return {"kernel": "lm_head + greedy sampling", "rows": args.rows, "us_per_launch": ms * 1e3,
            "algorithmic_bytes": algorithmic, "gb_per_s": algorithmic / ms / 1e6}


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    sub = parser.add_subparsers(dest="command", required=True)
    p = sub.add_parser("decode")
    p.add_argument("--concurrency", type=int, default=64)
    p.add_argument("--tp", type=int, default=1)
    p.add_argument("--split-policy", type=int, default=1)
    p.add_argument("--kv-dtype", default="bf16", choices=["bf16", "fp8"])
    p.add_argument("--sequential-tables", action="store_true",
                   help="pages of a request in ascending order instead of randomly placed")
    p.add_argument("--reuse-plan", action="store_true",
                   help="time decode + merge only, with the plan built once as inside a model step")
    p.add_argument("--lengths", type=lambda text: [int(n) for n in text.split(",")], default=None,
                   help="explicit context lengths instead of the log-normal draw, e.g. 17,128,513,2048")
    p = sub.add_parser("gemm")
    p.add_argument("--shape", default="qkv", choices=list(workloads.GEMM_SHAPES))
    p.add_argument("--rows", type=int, default=256)
    p.add_argument("--copies", type=int, default=4)
    p = sub.add_parser("prefill")
    p.add_argument("--requests", type=int, default=6)
    p = sub.add_parser("lm_head")
    p.add_argument("--rows", type=int, default=8)
    for name in ("decode", "gemm", "prefill", "lm_head"):
        sub.choices[name].add_argument("--repeats", type=int, default=9)
    args = parser.parse_args()
    device = torch.device("cuda", 0)
    result = {"decode": decode, "gemm": gemm, "prefill": prefill, "lm_head": lm_head}[args.command](args, device)
    print(json.dumps(result))


if __name__ == "__main__":
    main()
