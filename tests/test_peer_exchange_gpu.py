"""The fused tensor-parallel exchange (all-reduce + residual add + RMSNorm + quantisation over peer memory).

On ONE GPU the ranks are emulated: every rank's block lives on the same device, the flags every kernel would
wait for are written beforehand, and the ranks' kernels run one after the other (no launch ever waits for
another launch).  The reference for the arithmetic is the plain formulation: fp32 sum of the partial rows in
rank order rounded once to bf16, then the residual add + RMSNorm (+ quantiser) of ``oracle.hot_path``.
The two-GPU test maps the blocks through CUDA IPC in two processes and needs two devices.
"""

from __future__ import annotations

import os
import socket

import pytest
import torch

from mini_inference_engine_b200 import _lib
from mini_inference_engine_b200.engine.model_runner.peer_exchange import PeerExchange
from oracle import hot_path

pytestmark = pytest.mark.gpu

EPS = 1e-6


def _reference(partials, residual, weight):
    total = torch.zeros_like(partials[0], dtype=torch.float32)
    for part in partials:
        total += part.float()
    reduced = total.to(torch.bfloat16)
    normed, summed = hot_path.rms_norm(reduced, weight, EPS, residual=residual)
    q, scales = hot_path.quantize_activation(normed)
    return normed, summed, q, scales


def _close(got: torch.Tensor, want: torch.Tensor, max_mismatch: float = 0.02) -> None:
    got, want = got.cpu().float(), want.float()
    ulp = want.abs().clamp_min(1e-30) * 2.0 ** -7
    assert ((got - want).abs() <= ulp).all(), (got - want).abs().max().item()
    assert (got != want).float().mean().item() <= max_mismatch


def _emulated(tp: int, rows: int, cols: int, device):
    nbytes = PeerExchange.layout(rows, cols)[1]
    blocks = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for _ in range(tp)]
    return [PeerExchange(tp, r, rows, cols, device, emulated_blocks=blocks) for r in range(tp)]


@pytest.mark.parametrize("tp,rows", [(2, 8), (4, 37), (8, 256), (8, 5)])
def test_emulated_ranks_match_the_plain_formulation(device, tp, rows):
    cols = 2560
    torch.manual_seed(tp * 1000 + rows)
    ranks = _emulated(tp, rows, cols, device)
    weight = (torch.randn(cols) * 0.1 + 1.0).to(torch.bfloat16)
    residual = torch.randn(rows, cols).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    for step in range(2):  # two epochs through the same flags
        partials = [(torch.randn(rows, cols) * (0.5 + r)).to(torch.bfloat16) for r in range(tp)]
        want_normed, want_summed, want_q, want_scales = _reference(partials, residual, weight)
        for quantized in (True, False):
            for ex, part in zip(ranks, partials):
                ex.partial[:rows].copy_(part.to(device))
                ex.flags.fill_(1 << 20)  # every peer "has signalled" both phases of any epoch used here
            summed = [torch.zeros(rows, cols, dtype=torch.bfloat16, device=device) for _ in range(tp)]
            for r, ex in enumerate(ranks):
                ex.reduce_norm(rows, residual.to(device), summed[r], weight.to(device), EPS, quantized=quantized,
                               status=status)
            torch.cuda.synchronize(device)
            assert int(status.item()) == 0
            for r, ex in enumerate(ranks):
                owned = ex.owned_rows(rows)
                assert torch.equal(summed[r][owned.start:owned.stop].cpu(), want_summed[owned.start:owned.stop])
                if quantized:
                    # the quantiser is exact given the normed row; rows whose norm differs by an ulp differ in q too
                    got = ex.q[:rows].cpu().float() * ex.scales[:, :rows].cpu().t().repeat_interleave(128, dim=1)
                    want = want_q.float() * want_scales.repeat_interleave(128, dim=1)
                    assert (got - want).abs().max().item() <= 0.07 * want.abs().max().item()
                    assert (ex.q[:rows].cpu().view(torch.uint8) != want_q.view(torch.uint8)).float().mean().item() < 0.02
                    assert torch.equal(ex.q[:rows].cpu().view(torch.uint8), ranks[0].q[:rows].cpu().view(torch.uint8))
                    assert torch.equal(ex.scales[:, :rows].cpu(), ranks[0].scales[:, :rows].cpu())
                else:
                    _close(ex.normed[:rows], want_normed)
                    assert torch.equal(ex.normed[:rows].cpu(), ranks[0].normed[:rows].cpu())
        residual = want_summed


def test_fused_exchange_equals_library_norm_of_the_reduced_rows_bitwise(device):
    """Same rounding points as ``mie_rms_norm`` with fused quantisation applied to the all-reduced rows."""

    tp, rows, cols = 4, 64, 2560
    torch.manual_seed(7)
    ranks = _emulated(tp, rows, cols, device)
    weight = (torch.randn(cols) * 0.1 + 1.0).to(torch.bfloat16).to(device)
    residual = torch.randn(rows, cols).to(torch.bfloat16).to(device)
    partials = [torch.randn(rows, cols).to(torch.bfloat16).to(device) for _ in range(tp)]
    total = torch.zeros(rows, cols, dtype=torch.float32, device=device)
    for part in partials:
        total += part.float()
    reduced = total.to(torch.bfloat16)
    lib, stream = _lib.load(), _lib.stream_arg(device)
    want_summed = torch.empty_like(reduced)
    want_q = torch.empty(rows, cols, dtype=torch.float8_e4m3fn, device=device)
    want_scales = torch.empty(cols // 128, rows, dtype=torch.float32, device=device)
    _lib.check(lib.mie_rms_norm(_lib.ptr(reduced), cols, _lib.ptr(residual), _lib.ptr(want_summed), _lib.ptr(weight),
                                None, _lib.ptr(want_q), cols, _lib.ptr(want_scales), rows, rows, cols, EPS, stream))
    for ex, part in zip(ranks, partials):
        ex.partial[:rows].copy_(part)
        ex.flags.fill_(1 << 20)
    summed = torch.zeros(rows, cols, dtype=torch.bfloat16, device=device)
    for ex in ranks:
        ex.reduce_norm(rows, residual, summed, weight, EPS, quantized=True)  # disjoint owned rows of one tensor
    torch.cuda.synchronize(device)
    assert torch.equal(summed, want_summed)
    for ex in ranks:
        assert torch.equal(ex.q[:rows].view(torch.uint8), want_q.view(torch.uint8))
        assert torch.equal(ex.scales[:, :rows], want_scales)


def test_a_wait_that_runs_out_sets_the_status_bit_and_returns(device):
    """Nothing ever sets the peer's flag: the bounded wait gives up, the status word says so, the context lives."""

    tp, rows, cols = 2, 4, 256
    ranks = _emulated(tp, rows, cols, device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    weight = torch.ones(cols, dtype=torch.bfloat16, device=device)
    residual = torch.zeros(rows, cols, dtype=torch.bfloat16, device=device)
    summed = torch.zeros_like(residual)
    ranks[0].reduce_norm(rows, residual, summed, weight, EPS, quantized=True, status=status, max_polls=64)
    torch.cuda.synchronize(device)
    assert int(status.item()) & _lib.STATUS_WAIT_TIMEOUT
    with pytest.raises(ValueError, match="timed out"):
        _lib.raise_for_status(status)
    assert torch.ones(4, device=device).sum().item() == 4.0


def test_argument_checks(device):
    ex = _emulated(2, 4, 256, device)[0]
    good = torch.zeros(4, 256, dtype=torch.bfloat16, device=device)
    with pytest.raises(ValueError, match="capacity"):
        ex.reduce_norm(5, good, good, good[0], EPS, quantized=True)
    with pytest.raises(ValueError, match="contiguous bf16"):
        ex.reduce_norm(4, good.float(), good, good[0], EPS, quantized=True)
    with pytest.raises(ValueError, match="multiple of 128"):
        PeerExchange(2, 0, 4, 200, device, emulated_blocks=[])
    with pytest.raises(ValueError, match="out of range"):
        PeerExchange(9, 0, 4, 256, device, emulated_blocks=[])


# ---------------------------------------------------------------------------------------------
# Two processes, two GPUs: blocks mapped through CUDA IPC, flags really cross NVLink.
# ---------------------------------------------------------------------------------------------

def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _two_gpu_worker(rank: int, world: int, port: int, results) -> None:
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        rows, cols = 96, 2560
        ex = PeerExchange(world, rank, rows, cols, device, dist.group.WORLD)
        gen = torch.Generator().manual_seed(11)
        weight = (torch.randn(cols, generator=gen) * 0.1 + 1.0).to(torch.bfloat16)
        residual = torch.randn(rows, cols, generator=gen).to(torch.bfloat16)
        status = torch.zeros(1, dtype=torch.int32, device=device)
        ok = True
        for step in range(3):
            partials = [torch.randn(rows, cols, generator=gen).to(torch.bfloat16) for _ in range(world)]
            want_normed, want_summed, want_q, want_scales = _reference(partials, residual, weight)
            ex.partial[:rows].copy_(partials[rank].to(device))
            summed = torch.zeros(rows, cols, dtype=torch.bfloat16, device=device)
            ex.reduce_norm(rows, residual.to(device), summed, weight.to(device), EPS, quantized=step != 2,
                           status=status)
            torch.cuda.synchronize(device)
            owned = ex.owned_rows(rows)
            ok &= torch.equal(summed[owned.start:owned.stop].cpu(), want_summed[owned.start:owned.stop])
            if step != 2:
                mismatch = (ex.q[:rows].cpu().view(torch.uint8) != want_q.view(torch.uint8)).float().mean().item()
                ok &= mismatch < 0.02
                gathered = [torch.empty_like(ex.q[:rows].view(torch.uint8)) for _ in range(world)]
                dist.all_gather(gathered, ex.q[:rows].view(torch.uint8).contiguous())
                ok &= all(torch.equal(g, gathered[0]) for g in gathered)
            else:
                diff = (ex.normed[:rows].cpu().float() - want_normed.float()).abs()
                ok &= bool((diff <= want_normed.float().abs().clamp_min(1e-30) * 2.0 ** -7).all())
            residual = want_summed
        ok &= int(status.item()) == 0
        results[rank] = bool(ok)
        dist.barrier()
        torch.cuda.synchronize(device)
        ex.close()
    finally:
        os._exit(0 if results.get(rank) else 1)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_exchange_over_ipc_mapped_peer_memory():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_two_gpu_worker, args=(rank, 2, port, results)) for rank in range(2)]
    for proc in procs:
        proc.start()
    for proc in procs:
        proc.join(timeout=240)
    for proc in procs:
        if proc.is_alive():
            proc.kill()  # this exact child, by handle
            pytest.fail("a rank did not finish in time")
    assert [results.get(r) for r in range(2)] == [True, True]
