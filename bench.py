"""Benchmark of the continuous-batching decode hot path on B200.

Metric (BASELINE.json): decode tok/s of a random-init Qwen3-4B-shaped FP8 model on a
ragged batch, with the paged-attention HBM GB/s as a fraction of peak.

Workload (BASELINE configuration 4): C concurrent sequences (default 256) whose
contexts are log-normal (median 2048, sigma 1.0, clipped to [16, 32768]), random
block tables over a KV pool of about 80% of free HBM, split-KV decode attention,
one CUDA-graph decode step per "step"; tensor-parallel over --gpus ranks.

    python bench.py --gpus 1 --steps 200 --warmup 3
    python -m torch.distributed.run --nproc-per-node 8 ... bench.py --gpus 8 ...
    python bench.py --impl reference        # the reference's torch/CPU path on host cores

Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

FALLBACK_HBM_GBS = 6650.0
METRIC = "decode tok/s (Qwen3-4B FP8 shape, ragged batch); paged-attn HBM GB/s % peak"


def parse_args() -> argparse.Namespace:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--concurrency", type=int, default=256)
    parser.add_argument("--kv-fraction", type=float, default=0.8)
    parser.add_argument("--layers", type=int, default=None, help="debug: fewer layers (invalid as a result)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-e2e", action="store_true")
    parser.add_argument("--workload", default="config4", choices=["config4", "config3"],
                        help="config4: ragged decode sweep point (the headline); config3: 8 x (2048 prompt + 128 new)")
    parser.add_argument("--no-extras", action="store_true",
                        help="skip the extra keys measured after the headline (configs 0-3, FP8 KV cache)")
    parser.add_argument("--breakdown", action="store_true",
                        help="instead of the benchmark: CUDA-event time per kernel class of the eager decode step")
    parser.add_argument("--watchdog", type=int, default=900,
                        help="seconds after which every rank dumps its Python stacks and exits (0 = off)")
    return parser.parse_args()


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except (ValueError, KeyError):
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ----------------------------------------------------------------------------------------------
# Clock sampling during the timed region
# ----------------------------------------------------------------------------------------------

class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int) -> None:
        self.device_index, self.process, self.path = device_index, None, None

    def start(self) -> None:
        try:
            import tempfile

            handle = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = handle.name
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.device_index)], stdout=handle, stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        clocks, max_clock, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        try:
            for line in Path(self.path).read_text().splitlines():
                fields = [f.strip() for f in line.split(",")]
                if len(fields) < 9:
                    continue
                try:
                    clocks.append(float(fields[1]))
                    max_clock = float(fields[2])
                except ValueError:
                    continue
                for name, value in zip(names, fields[5:9]):
                    if value.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


# ----------------------------------------------------------------------------------------------
# CPU baseline: the reference's torch/CPU path (oracle port) on a bounded sample
# ----------------------------------------------------------------------------------------------

def cpu_decode_baseline(sample_sequences: int = 4, max_context: int = 4096, repeats: int = 1,
                        layer_source=None, embedding=None, final_norm=None) -> dict:
    """Time one decode step of ONE layer (+ the tied lm_head) of the Qwen3-4B-shaped FP8 model on the host
    cores with the CPU oracle, and extrapolate to the 36-layer model: tok/s = S / (36 * t_layer + t_head)."""

    from mini_inference_engine_b200 import workloads
    from mini_inference_engine_b200.engine.model_runner.qwen3_decode import Qwen3Shape, Qwen3Weights
    from oracle import hot_path, qwen3_model

    shape = Qwen3Shape()
    threads = torch.get_num_threads()
    contexts = workloads.lognormal_contexts(256, seed=256)[:sample_sequences].clamp(max=max_context)
    if layer_source is None:
        weights = Qwen3Weights(shape, torch.device("cpu"), seed=0, layers=1)
    else:
        class _W:  # one layer copied from the device model
            pass
        weights = _W()
        weights.layers = [type(layer_source)(*[getattr(layer_source, f).cpu()
                                                for f in layer_source.__dataclass_fields__])]
        weights.embedding, weights.final_norm = embedding.cpu(), final_norm.cpu()
    pages = int(sum(-(-(int(n) + 2) // 16) for n in contexts)) + 4
    tables = workloads.random_block_tables(contexts, num_pages=pages, seed=3, extra_tokens=2)
    key_blocks = torch.randn(1, pages, shape.kv_heads, 16, shape.head_dim).to(torch.bfloat16)
    value_blocks = torch.randn(1, pages, shape.kv_heads, 16, shape.head_dim).to(torch.bfloat16)
    ids = torch.randint(0, shape.vocab, (sample_sequences,))
    lengths = (contexts + 1).to(torch.int32)

    def one_layer_step():
        # decode_step over a 1-layer model = one layer + final norm + lm_head + argmax.
        return qwen3_model.decode_step(weights, key_blocks, value_blocks, ids, lengths, tables,
                                       q_heads=shape.q_heads, kv_heads=shape.kv_heads, head_dim=shape.head_dim,
                                       eps=shape.rms_eps, theta=shape.rope_theta)

    def head_only():
        final = hot_path.rms_norm(weights.embedding[:sample_sequences], weights.final_norm, shape.rms_eps)
        return (final @ weights.embedding.t()).argmax(dim=-1)

    one_layer_step()
    t0 = time.perf_counter()
    for _ in range(repeats):
        one_layer_step()
    t_step = (time.perf_counter() - t0) / repeats
    t0 = time.perf_counter()
    head_only()
    t_head = time.perf_counter() - t0
    t_layer = max(t_step - t_head, 1e-6)
    full = shape.layers * t_layer + t_head
    return {
        "value": sample_sequences / full, "unit": "tok/s", "cores": threads, "kind": "port",
        "sample": (f"{sample_sequences} sequences (contexts {contexts.tolist()}), one decode step of 1 layer + "
                   f"lm_head timed with the CPU oracle ({t_layer * 1e3:.0f} ms/layer, {t_head * 1e3:.0f} ms head), "
                   f"extrapolated to 36 layers"),
        "seconds_per_step_extrapolated": full,
    }


def use_all_host_cores() -> int:
    """Let torch's CPU kernels use every core this process may run on; returns the thread count."""

    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    torch.set_num_threads(max(cores, 1))
    return torch.get_num_threads()


def cpu_baseline_in_clean_process(args: argparse.Namespace) -> dict:
    """Run ``bench.py --impl reference`` in a child process whose environment carries no thread limits and no
    rendezvous variables, and return its JSON line.  A multi-process launcher exports ``OMP_NUM_THREADS=1``
    before Python starts; raising the thread count afterwards leaves the OpenMP pool of that process pinned
    the way it was initialised (measured: 40x slower than a clean process, not 1x), so the baseline that has
    to be the same at every N is taken in a process of its own."""

    drop = ("OMP_NUM_THREADS", "MKL_NUM_THREADS", "OPENBLAS_NUM_THREADS", "RANK", "LOCAL_RANK", "WORLD_SIZE",
            "LOCAL_WORLD_SIZE", "GROUP_RANK", "ROLE_RANK", "MASTER_ADDR", "MASTER_PORT", "TORCHELASTIC_RUN_ID")
    env = {k: v for k, v in os.environ.items() if k not in drop and not k.startswith("TORCHELASTIC")}
    env["MIE_BENCH_CPU_CHILD"] = "1"
    env["CUDA_VISIBLE_DEVICES"] = ""
    done = subprocess.run([sys.executable, str(Path(__file__).resolve()), "--impl", "reference", "--gpus",
                           str(args.gpus), "--steps", str(args.steps), "--warmup", str(args.warmup)],
                          env=env, capture_output=True, text=True, timeout=900)
    lines = [line for line in done.stdout.splitlines() if line.startswith("{")]
    if done.returncode != 0 or not lines:
        raise RuntimeError(f"CPU baseline child failed ({done.returncode}): {done.stderr[-400:]}")
    return json.loads(lines[-1])


def launched_with_thread_limit() -> bool:
    return "OMP_NUM_THREADS" in os.environ and os.environ.get("MIE_BENCH_CPU_CHILD") != "1"


def run_reference_arm(args: argparse.Namespace) -> None:
    """The reference's own CPU path for this metric: its torch block-wise attention and the FP8 linear
    restated on the CPU (the reference has no CPU FP8 kernel), on all host threads."""

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # A multi-process launcher exports OMP_NUM_THREADS=1 to its workers; the baseline uses every host core
    # at every N so that all runs share one denominator.
    if launched_with_thread_limit():
        emit(cpu_baseline_in_clean_process(args))
        return
    use_all_host_cores()
    repeats = max(1, min(args.steps, 2))
    started = time.perf_counter()
    base = cpu_decode_baseline(repeats=repeats)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["seconds_per_step_extrapolated"] * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3/bf16",
        "data": "synthetic",
        "config": {"workload": "config4 ragged decode, CPU sample", "sample": base["sample"],
                   "timed_repeats": repeats},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_seconds": time.perf_counter() - started,
    }
    emit(line)


# ----------------------------------------------------------------------------------------------
# Our arm
# ----------------------------------------------------------------------------------------------

def run_config3(args, shape, device, rank, world, group) -> None:
    """BASELINE configuration 3: 8 requests arrive together, 2048 random prompt ids each, 128 new tokens,
    greedy, paged KV, CUDA graph for decode.  Output tok/s = new tokens / wall time of the whole generation
    (the reference's definition, docs/metric_definitions.md:25-27).  One timed generation after one warm-up
    generation of the same shape, which also captures the decode graph as a serving engine does at start-up."""

    from mini_inference_engine_b200.engine.model_runner.qwen3_decode import Qwen3DecodeRunner, Qwen3Weights

    weights = Qwen3Weights(shape, device, seed=0, tp_rank=rank, tp_size=world, layers=args.layers)
    requests, prompt_len, new_tokens = 8, 2048, 128
    pages = requests * (-(-(prompt_len + new_tokens) // shape.page)) + 8
    runner = Qwen3DecodeRunner(weights, num_pages=pages, max_batch=requests, max_context=prompt_len + new_tokens + 8,
                               process_group=group)
    generator = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, shape.vocab, (prompt_len,), generator=generator).tolist() for _ in range(requests)]
    runner.generate(prompts, new_tokens)  # warm-up: tensor maps, cuBLAS, and the decode graph of this bucket
    torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    outputs = runner.generate(prompts, new_tokens)
    torch.cuda.synchronize(device)
    wall = time.perf_counter() - t0
    if rank == 0:
        emit({
            "metric": "output tok/s, 8 requests x 2048-token prompts, 128 new tokens (configuration 3)",
            "value": requests * new_tokens / wall, "unit": "tok/s", "n_gpus": world, "seconds": wall,
            "vs_baseline": requests * new_tokens / wall / 160.6,  # the reference's published L4 number
            "higher_is_better": True, "data": "synthetic", "dtype": "fp8_e4m3 GEMM / bf16 KV+activations",
            "config": {"workload": "config3", "requests": requests, "prompt_tokens": prompt_len,
                       "new_tokens": new_tokens, "includes": "packed prefill + 127 graph decode steps (the graph was captured by the warm-up generation)"},
            "tokens_first_request": outputs[0][:8],
        })
    if world > 1:
        leave_together(runner, device)


def run_breakdown(runner, buffers, steps: int, device, rank: int, world: int, concurrency: int) -> None:
    """CUDA-event time per kernel class of the decode step, run eagerly (no graph) with the stream kept busy
    ahead of the launches so that the intervals hold device time, not launch gaps.  Under tensor parallelism
    the exchange kernels wait for their peers, so their time includes the skew between ranks; every rank
    measures, rank 0 prints its own figures."""

    from mini_inference_engine_b200.engine.model_runner import qwen3_decode

    spans: dict[str, list] = {}

    def timed(name_of, fn):
        def wrapper(*args, **kwargs):
            name = name_of(*args, **kwargs)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*args, **kwargs)
            e1.record()
            spans.setdefault(name, []).append((e0, e1))
            return out
        return wrapper

    layer0 = runner.weights.layers[0]
    shapes = {tuple(layer0.qkv.shape): "gemm qkv", tuple(layer0.o.shape): "gemm o",
              tuple(layer0.gate_up.shape): "gemm gate_up", tuple(layer0.down.shape): "gemm down"}
    runner._gemm = timed(lambda q, w, *a, **k: shapes.get(tuple(w.shape), "gemm other"), runner._gemm)
    runner._norm = timed(lambda *a, **k: "add + rms_norm (+quant)", runner._norm)
    runner._qkv_post = timed(lambda *a, **k: "q/k norm + rope + kv write", runner._qkv_post)
    runner._silu_mul_quantized = timed(lambda *a, **k: "silu*up + quant", runner._silu_mul_quantized)
    runner.greedy_tokens = timed(lambda *a, **k: "lm_head + greedy sampling", runner.greedy_tokens)
    qwen3_decode.launch_decode_attention = timed(lambda *a, **k: "decode attention (plan + decode + merge)",
                                                 qwen3_decode.launch_decode_attention)
    if runner.exchange is not None:
        runner.exchange.reduce_norm = timed(lambda *a, **k: "peer exchange + add + rms_norm + quant",
                                            runner.exchange.reduce_norm)
    totals = []
    for step in range(steps + 1):
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(device)
        spans.clear()
        torch.cuda._sleep(40_000_000)  # ~20 ms of device time: the host queues the whole step behind it
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        runner.decode_forward(buffers.input_ids, buffers.sequence_lengths, buffers.block_tables)
        s1.record()
        torch.cuda.synchronize(device)
        if step:  # the first pass warms up
            totals.append((s0.elapsed_time(s1), {n: [a.elapsed_time(b) for a, b in v] for n, v in spans.items()}))
    runner.check_status()
    if rank == 0:
        classes = {}
        for name in totals[0][1]:
            per_call = [t for _, per in totals for t in per[name]]
            classes[name] = {"calls_per_step": len(totals[0][1][name]),
                             "us_per_call": sum(per_call) / len(per_call) * 1e3,
                             "ms_per_step": sum(per_call) / len(totals)}
        step_ms = sum(t for t, _ in totals) / len(totals)
        emit({"breakdown": "eager decode step, CUDA events per kernel class", "n_gpus": world,
              "concurrency": concurrency, "eager_step_ms": step_ms,
              "sum_of_classes_ms": sum(c["ms_per_step"] for c in classes.values()),
              "classes": dict(sorted(classes.items(), key=lambda kv: -kv[1]["ms_per_step"]))})


def measure_configs(weights, shape, device) -> dict:
    """BASELINE configurations 0-3 next to the headline (configuration 4), each a few hundred milliseconds:
    0 = paged decode attention on the 4-sequence ragged batch, 1 = the FP8 GEMMs at M = 256 / 2048,
    2 = packed chunked-prefill attention, 3 = 8 requests x (2048-token prompt + 128 new tokens)."""

    import types

    import microbench
    from mini_inference_engine_b200.engine.model_runner.qwen3_decode import Qwen3DecodeRunner

    out = {}
    ns = types.SimpleNamespace
    d0 = microbench.decode(ns(concurrency=4, lengths=[17, 128, 513, 2048], tp=1, split_policy=1, kv_dtype="bf16",
                              repeats=15), device)
    out["config0"] = {"us_per_launch": d0["us_per_launch"], "gb_per_s": d0["gb_per_s"],
                      "note": "4 sequences, 2,706 context tokens: launch-latency bound (11 MB of K/V)"}
    gemms = {}
    for name in ("qkv", "o", "gate_up", "down"):
        for rows in (256, 2048):
            g = microbench.gemm(ns(shape=name, rows=rows, copies=4, repeats=7), device)
            gemms[f"{name}_m{rows}"] = {"us": g["us_per_launch"], "tflops": g["tflops"]}
    out["config1"] = gemms
    p2 = microbench.prefill(ns(requests=6, repeats=9), device)
    out["config2"] = {"us_per_launch": p2["us_per_launch"], "tflops": p2["tflops"]}
    requests, prompt_len, new_tokens = 8, 2048, 128
    pages = requests * (-(-(prompt_len + new_tokens) // shape.page)) + 8
    small = Qwen3DecodeRunner(weights, num_pages=pages, max_batch=requests, max_context=prompt_len + new_tokens + 8)
    generator = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, shape.vocab, (prompt_len,), generator=generator).tolist() for _ in range(requests)]
    small.generate(prompts, new_tokens)  # warm-up; also captures the bucket's graph, as a server does at start-up
    torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    small.generate(prompts, new_tokens)
    torch.cuda.synchronize(device)
    wall = time.perf_counter() - t0
    out["config3"] = {"output_tok_s": requests * new_tokens / wall, "seconds": wall,
                      "includes": "packed prefill of 8 x 2048 tokens + 127 graph decode steps"}
    small.release_graphs()
    return out


def measure_fp8_kv(weights, shape, device, contexts, tables, ids0, num_pages, max_context, steps, warmup, peak) -> dict:
    """The headline workload again over the opt-in FP8 (e4m3) KV cache: same contexts, same block tables,
    same graph step, K/V read as 2,112 bytes per token and layer instead of 4,096.  Not the headline: the
    reference's cache precision is bf16."""

    from mini_inference_engine_b200.engine.kv_cache.fp8_kv import launch_decode_attention_kv8
    from mini_inference_engine_b200.engine.model_runner.qwen3_decode import Qwen3DecodeRunner

    concurrency = int(contexts.numel())
    runner = Qwen3DecodeRunner(weights, num_pages=num_pages, max_batch=concurrency, max_context=max_context,
                               kv_init="normal", kv_dtype="fp8")
    buffers = runner.capture(concurrency, tables.shape[1], advance=True)
    buffers.input_ids.copy_(ids0.to(device))
    buffers.block_tables.copy_(tables.to(device))
    buffers.sequence_lengths.copy_((contexts + 1).to(torch.int32).to(device))
    for _ in range(warmup):
        runner.replay(concurrency, advance=True)
    torch.cuda.synchronize(device)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        runner.replay(concurrency, advance=True)
    end.record()
    torch.cuda.synchronize(device)
    runner.check_status()
    step_ms = start.elapsed_time(end) / steps
    lengths_now = (contexts + 1 + warmup + steps).to(torch.int32).to(device)
    query = torch.randn(concurrency, shape.q_heads, 1, shape.head_dim, device=device).to(torch.bfloat16)
    out = torch.empty_like(query)
    durations = []
    for layer in range(min(len(weights.layers), 12)):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        launch_decode_attention_kv8(query, out, runner.kv8.data[layer], runner.kv8.scales[layer],
                                    buffers.block_tables, lengths_now, None, scale=shape.head_dim ** -0.5,
                                    scratch=runner.scratch, split_policy=1, status=runner.status)
        e1.record()
        if layer:
            durations.append((e0, e1))
    torch.cuda.synchronize(device)
    attn_ms = statistics.mean(a.elapsed_time(b) for a, b in durations)
    bytes_per_token = runner.kv8.bytes_per_token()
    algorithmic = int(lengths_now.sum().item()) * bytes_per_token + 2 * query.numel() * 2
    result = {"value": concurrency * steps / (step_ms * steps / 1e3), "unit": "tok/s", "ms_per_step": step_ms,
              "kv_bytes_per_token_per_layer": bytes_per_token,
              "attention": {"kernel": "decode_kv8_kernel<bf16>", "ms_per_launch": attn_ms,
                            "algorithmic_bytes_per_launch": algorithmic,
                            "achieved": algorithmic / (attn_ms / 1e3) / 1e9, "unit": "GB/s",
                            "frac": algorithmic / (attn_ms / 1e3) / 1e9 / peak},
              "note": "opt-in e4m3 KV cache with one fp32 scale per (token, KV head); bf16 KV stays the headline"}
    runner.release_graphs()
    return result


def leave_together(runner, device) -> None:
    """End a multi-rank run: drop the captured graphs (they hold NCCL kernels and peer-memory pointers), wait
    for the device and for every rank, unmap the peers' exchange blocks, then exit without running the
    communicator's destructor (destroying a communicator that graphs had captured blocked one earlier run;
    with the graphs gone and NVLS off nothing is bound to a peer when the process exits)."""

    runner.release_graphs()
    torch.cuda.synchronize(device)
    torch.distributed.barrier()
    torch.cuda.synchronize(device)
    if runner.exchange is not None:
        runner.exchange.close()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


_RESULT_OUT = None


def emit(line: dict) -> None:
    """Print the one JSON line on the process's original stdout."""

    out = _RESULT_OUT if _RESULT_OUT is not None else sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main() -> None:
    # Libraries (NCCL with NCCL_DEBUG set, for one) write banners to file descriptor 1; the contract is ONE
    # JSON line on stdout, so everything else that goes to fd 1 is sent to stderr.
    global _RESULT_OUT
    sys.stdout.flush()
    _RESULT_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    args = parse_args()
    if args.watchdog > 0:
        import faulthandler

        faulthandler.dump_traceback_later(args.watchdog, exit=True)
    if args.impl == "reference":
        run_reference_arm(args)
        return

    from mini_inference_engine_b200 import workloads
    from mini_inference_engine_b200.engine.kv_cache.triton_paged_attention import launch_decode_attention
    from mini_inference_engine_b200.engine.model_runner.qwen3_decode import (
        Qwen3DecodeRunner,
        Qwen3Shape,
        Qwen3Weights,
    )

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    group = None
    early_cpu = None
    if world > 1 and rank == 0 and not args.no_cpu_baseline and not args.breakdown:
        # The CPU baseline of a multi-rank run is taken FIRST, while the other ranks block (without spinning)
        # in the rendezvous below: ranks that wait for rank 0 inside a collective poll on the host and take the
        # cores the baseline needs (measured: 16 s per layer instead of 0.1 s).
        try:
            base = (cpu_baseline_in_clean_process(args)["cpu_baseline"] if launched_with_thread_limit()
                    else cpu_decode_baseline())
            early_cpu = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        except Exception as error:  # the baseline is reported, never required
            early_cpu = {"value": None, "unit": "tok/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"failed: {error!r}"}
    if world > 1:
        # No NVLink multicast (NVLS) objects: a rank that leaves while its memory is bound to one can raise
        # NVLink faults on its peers, and the exchange kernels of this library use plain peer loads anyway.
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.distributed.init_process_group("nccl", device_id=device)
        group = torch.distributed.group.WORLD
    tp = world

    def barrier() -> None:
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(device)

    def max_over_ranks(value: float) -> float:
        if world == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64, device=device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item())

    shape = Qwen3Shape()
    if args.workload == "config3":
        run_config3(args, shape, device, rank, world, group)
        return
    concurrency, steps, warmup = args.concurrency, args.steps, max(args.warmup, 0)
    weights = Qwen3Weights(shape, device, seed=0, tp_rank=rank, tp_size=tp, layers=args.layers)
    layers = len(weights.layers)
    contexts = workloads.lognormal_contexts(concurrency, seed=concurrency)
    e2e_steps = 0 if args.no_e2e else steps
    planned_steps = 2 * (warmup + steps) + 16
    max_context = int(contexts.max()) + planned_steps + 1
    local_kv = shape.kv_heads // tp
    page_bytes = layers * 2 * local_kv * shape.page * shape.head_dim * 2
    needed_pages = int(sum(-(-(int(n) + planned_steps + 1) // shape.page) for n in contexts)) + 8
    torch.cuda.synchronize(device)
    free_bytes, _ = torch.cuda.mem_get_info(device)
    # Leave room for logits, graph pools and scratch.
    pool_pages = int(max(free_bytes - (6 << 30), 0) * args.kv_fraction) // page_bytes
    if world > 1:
        t = torch.tensor([pool_pages], dtype=torch.int64, device=device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MIN)
        pool_pages = int(t.item())
    num_pages = max(pool_pages, needed_pages)
    runner = Qwen3DecodeRunner(weights, num_pages=num_pages, max_batch=concurrency, max_context=max_context,
                               process_group=group, kv_init="normal")
    tables = workloads.random_block_tables(contexts, num_pages=num_pages, page=shape.page, seed=concurrency,
                                           extra_tokens=planned_steps + 1)
    width = tables.shape[1]
    ids0 = torch.randint(0, shape.vocab, (concurrency,), generator=torch.Generator().manual_seed(1))

    # ---- device-resident measurement: the graph feeds its tokens back and bumps the lengths ----
    buffers = runner.capture(concurrency, width, advance=True)
    launches_per_step = runner.launches_per_step
    buffers.input_ids.copy_(ids0.to(device))
    buffers.block_tables.copy_(tables.to(device))
    buffers.sequence_lengths.copy_((contexts + 1).to(torch.int32).to(device))
    if args.breakdown:
        run_breakdown(runner, buffers, max(1, min(steps, 5)), device, rank, world, concurrency)
        if world > 1:
            leave_together(runner, device)
        return
    for _ in range(warmup):
        runner.replay(concurrency, advance=True)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()  # lets `ncu --profile-from-start off` list only the timed launches
    start.record()
    for _ in range(steps):
        runner.replay(concurrency, advance=True)
    end.record()
    barrier()
    torch.cuda.profiler.stop()
    clocks = sampler.stop() if rank == 0 else {}
    elapsed_ms = max_over_ranks(start.elapsed_time(end))
    runner.check_status()
    tokens_per_s = concurrency * steps / (elapsed_ms / 1e3)
    grown = warmup + steps  # tokens every context has gained so far

    # ---- end to end: host metadata in, H2D, replay, D2H of the sampled tokens, every step ----
    e2e = None
    if e2e_steps:
        # Same workload as the device-resident loop: every context starts again at its drawn length (the
        # pool's contents are random either way), so the two numbers differ only by the host round trip.
        # Each step hands the runner plain host data (request ids, last tokens, lengths, page lists); it packs
        # them into pinned mirrors, copies ids and lengths and whatever block-table entries changed, replays
        # the bucket's graph and reads the tokens back.
        grown = 0
        owners = list(range(concurrency))
        block_rows = [row[row >= 0].tolist() for row in tables]  # pages reserved for the whole run
        host_lengths = (contexts + 1).tolist()
        host_ids = buffers.output_tokens.cpu().tolist()
        first_h2d = None
        for _ in range(max(warmup, 1)):
            host_ids, h2d, _ = runner.decode_rows(owners, host_ids, host_lengths, block_rows)
            first_h2d = h2d if first_h2d is None else first_h2d
            host_lengths = [n + 1 for n in host_lengths]
        barrier()
        h2d = d2h = 0
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            host_ids, h2d, d2h = runner.decode_rows(owners, host_ids, host_lengths, block_rows)
            host_lengths = [n + 1 for n in host_lengths]
        torch.cuda.synchronize(device)
        wall = max_over_ranks(time.perf_counter() - t0)
        barrier()
        runner.check_status()
        e2e = {"value": concurrency * e2e_steps / wall, "unit": "tok/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": wall / e2e_steps * 1e3,
               "h2d_bytes_first_step": first_h2d,
               "note": "block tables are copied when a row changes owner or grows into a page, not every step"}
        grown = max(warmup, 1) + e2e_steps
        host_ids = torch.tensor(host_ids, dtype=torch.int64)

    # ---- roofline of the dominant kernel: paged decode attention, timed alone with CUDA events ----
    lengths_now = (contexts + 1 + grown).to(torch.int32).to(device)
    tables_dev = buffers.block_tables
    lq = shape.q_heads // tp
    query = torch.randn(concurrency, lq, 1, shape.head_dim, device=device).to(torch.bfloat16)
    out = torch.empty_like(query)
    launch_decode_attention(query, out, runner.key_blocks[0], runner.value_blocks[0], tables_dev, lengths_now, None,
                            scale=shape.head_dim ** -0.5, max_total_tokens=concurrency * max_context,
                            scratch=runner.scratch, split_policy=1, plan_only=True, status=runner.status)
    durations = []
    for rep in range(3):
        for layer in range(layers):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            launch_decode_attention(query, out, runner.key_blocks[layer], runner.value_blocks[layer], tables_dev,
                                    lengths_now, None, scale=shape.head_dim ** -0.5,
                                    max_total_tokens=concurrency * max_context, scratch=runner.scratch,
                                    split_policy=1, use_plan=True, plan_slot=layer,
                                    status=runner.status)
            e1.record()
            if rep > 0:
                durations.append((e0, e1))
            if layer == layers - 1:
                # Work counters are consumed by a launch: rebuild the plan before the next sweep.
                launch_decode_attention(query, out, runner.key_blocks[0], runner.value_blocks[0], tables_dev,
                                        lengths_now, None, scale=shape.head_dim ** -0.5,
                                        max_total_tokens=concurrency * max_context, scratch=runner.scratch,
                                        split_policy=1, plan_only=True, status=runner.status)
    torch.cuda.synchronize(device)
    attn_ms = statistics.mean(a.elapsed_time(b) for a, b in durations)
    total_tokens = int(lengths_now.sum().item())
    kv_bytes_per_token = 2 * (shape.kv_heads // tp) * shape.head_dim * 2
    algorithmic = total_tokens * kv_bytes_per_token + 2 * concurrency * lq * shape.head_dim * 2
    peak, peak_kind = measured_peaks()
    achieved = algorithmic / (attn_ms / 1e3) / 1e9
    traffic = None
    ratio_file = ROOT / "profiles" / "decode_attention_dram_ratio.json"
    if ratio_file.exists():
        try:
            traffic = algorithmic * float(json.loads(ratio_file.read_text())["dram_bytes_per_algorithmic_byte"])
        except (ValueError, KeyError):
            traffic = None
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "peak_kind": peak_kind, "kernel": "decode_kernel<bf16>",
                "algorithmic_bytes_per_launch": algorithmic, "ms_per_launch": attn_ms}
    runner.check_status()

    # Every rank holds the tokens of the last replayed step; under tensor parallelism they must be identical.
    tokens_agree = None
    if world > 1:
        mine = [buffers.output_tokens.clone()]
        if e2e is not None:
            mine.append(host_ids.to(device))
        mine = torch.cat(mine)
        gathered = torch.empty(world, mine.numel(), dtype=torch.int64, device=device)
        torch.distributed.all_gather_into_tensor(gathered, mine)
        tokens_agree = bool((gathered == gathered[0:1]).all().item())

    cpu = early_cpu
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        use_all_host_cores()
        try:
            cpu_all = cpu_decode_baseline(layer_source=weights.layers[0], embedding=weights.embedding,
                                          final_norm=weights.final_norm)
            cpu = {k: cpu_all[k] for k in ("value", "unit", "cores", "kind", "sample")}
        except Exception as error:  # the baseline is reported, never required
            cpu = {"value": None, "unit": "tok/s", "cores": torch.get_num_threads(), "kind": "port",
                   "sample": f"failed: {error!r}"}

    extra_configs = extra_fp8 = None
    if world == 1 and not args.no_extras and args.layers is None:
        try:
            extra_configs = measure_configs(weights, shape, device)
        except Exception as error:  # extras are reported, never required
            extra_configs = {"failed": repr(error)}
        try:
            import gc

            tables_cpu, ids_cpu = tables, ids0
            runner.release_graphs()
            runner.key_blocks = runner.value_blocks = None
            del buffers, tables_dev
            gc.collect()
            torch.cuda.empty_cache()
            extra_fp8 = measure_fp8_kv(weights, shape, device, contexts, tables_cpu, ids_cpu, num_pages, max_context,
                                       min(steps, 50), warmup, peak)
        except Exception as error:
            extra_fp8 = {"failed": repr(error)}

    if rank == 0:
        step_bytes = weights.weight_bytes() + total_tokens * kv_bytes_per_token * layers
        line = {
            "metric": METRIC, "value": tokens_per_s, "unit": "tok/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": elapsed_ms / steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3 GEMM / bf16 KV+activations", "data": "synthetic",
            "config": {
                "workload": "config4: ragged decode sweep point", "concurrency": concurrency,
                "context": "lognormal(median 2048, sigma 1.0) clipped [16, 32768]",
                "total_context_tokens": total_tokens, "layers": layers, "parallelism": f"tp{tp}",
                "kv_pool_pages": num_pages, "kv_pool_gb_per_gpu": num_pages * page_bytes / 1e9,
                "split_kv": "length-proportional chunks chosen on the device",
                "l2": "inputs larger than L2 (KV pool and weights are re-read from HBM every step)",
                "graph": "one CUDA graph per decode step",
                "tp_exchange": ("none" if tp == 1 else "fused reduce+norm over peer memory"
                                if runner.exchange is not None else "nccl all-reduce"),
            },
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": launches_per_step * steps, "clocks": clocks, "tp_tokens_agree": tokens_agree,
            "step_hbm_bytes_per_gpu": step_bytes,
            "step_hbm_frac_of_peak": step_bytes / (elapsed_ms / steps / 1e3) / 1e9 / peak,
            "configs": extra_configs, "fp8_kv": extra_fp8,
        }
        if args.layers is not None:
            line["invalid"] = "debug run with fewer layers"
        emit(line)
    if world > 1:
        leave_together(runner, device)


if __name__ == "__main__":
    main()
