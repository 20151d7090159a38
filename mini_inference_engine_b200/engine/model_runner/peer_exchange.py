"""Buffers and peer mappings of the fused tensor-parallel exchange (``mie_tp_reduce_rms_norm``).

Under head-sharded tensor parallelism the two row-parallel projections of a layer (o_proj, down_proj) leave
partial sums on every rank.  The reference runs on one GPU and has no counterpart; the plain formulation is
``all_reduce`` followed by the residual add + RMSNorm + quantisation.  Here each rank keeps ONE device block
that its peers map through CUDA IPC::

    partial [rows, cols] bf16 | q [rows, cols] e4m3 | scales [cols/128, rows] f32 | normed [rows, cols] bf16 | flags
    | landing [tp, rows, cols] bf16

and one kernel per rank does the exchange and the norm together (see ``csrc/peer_reduce.cu``).  Two forms:

* pull - the row-parallel GEMM writes into the local ``partial``; the exchange kernel tells the peers, waits for
  them and loads their partial rows over NVLink (``reduce_norm``);
* push - the GEMM's epilogue stores every output row straight into slot ``[own rank]`` of the owner's
  ``landing`` area and counts it into the owner's arrival counter (``push_gemm``, ``mie_fp8_gemm_tp_push``);
  the exchange kernel then waits on its local counter and reads local memory only (``reduce_norm(pushed=True)``).

Either way the next column-parallel GEMM reads ``q`` / ``scales`` (or the lm_head reads ``normed``), which every
rank's kernel has filled for the rows it owns, and the sums are formed in the same rank order: same bits.
"""

from __future__ import annotations

import ctypes

import torch

from ... import _lib


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class PeerExchange:
    """One rank's block, the mapped blocks of its peers, and the call into the fused kernel.

    ``group``: a ``torch.distributed`` process group whose ranks are the tensor-parallel ranks of ONE node
    (handles travel with ``all_gather_object``).  ``emulated_blocks``: instead of a group, a list of ``tp``
    uint8 tensors on this device standing in for the ranks' blocks (single-process tests; entry ``rank`` is
    used as the local block)."""

    def __init__(self, tp: int, rank: int, max_rows: int, cols: int, device: torch.device, group=None, *,
                 emulated_blocks: list[torch.Tensor] | None = None) -> None:
        if not 1 <= tp <= _lib.TP_MAX_RANKS or not 0 <= rank < tp:
            raise ValueError(f"rank {rank} of {tp} is out of range (at most {_lib.TP_MAX_RANKS} ranks)")
        if cols % 128 != 0:
            raise ValueError("cols must be a multiple of 128")
        self.tp, self.rank, self.max_rows, self.cols, self.device = tp, rank, max_rows, cols, device
        groups = cols // 128
        self._offsets, cursor = self.layout(max_rows, cols, tp)
        self.block_bytes = cursor
        self._mapped: list[tuple[int, int]] = []  # (mapped address, offset) of peers' blocks, for close()
        if emulated_blocks is not None:
            if len(emulated_blocks) != tp or any(b.numel() < cursor or b.dtype != torch.uint8 for b in emulated_blocks):
                raise ValueError(f"need {tp} uint8 blocks of at least {cursor} bytes")
            self.block = emulated_blocks[rank]
            bases = [int(b.data_ptr()) for b in emulated_blocks]
        else:
            self.block = torch.zeros(cursor, dtype=torch.uint8, device=device)
            bases = self._exchange_handles(group)
        if any(base % 256 for base in bases):
            raise ValueError("exchange blocks must be 256-byte aligned")
        self._bases = bases
        self.state = torch.zeros(4, dtype=torch.int32, device=device)  # epoch, CTA arrivals, rows landed (local only)
        block = self.block
        self.partial = self._view(block, "partial", torch.bfloat16, (max_rows, cols))
        self.q = self._view(block, "q", torch.float8_e4m3fn, (max_rows, cols))
        self.scales = self._view(block, "scales", torch.float32, (groups, max_rows))
        self.normed = self._view(block, "normed", torch.bfloat16, (max_rows, cols))
        self.flags = self._view(block, "flags", torch.int32, (2 * _lib.TP_MAX_RANKS,))
        self.landing = self._view(block, "landing", torch.bfloat16, (tp, max_rows, cols))

    ARRIVED_WORD = _lib.TP_MAX_RANKS + 1  # flags[0..8): epochs, [8]: rows landed, [9]: pushed elements arrived

    @staticmethod
    def layout(max_rows: int, cols: int, tp: int = 0) -> tuple[dict[str, int], int]:
        """Byte offsets of the regions inside a rank's block, and the block size (``tp`` landing slots)."""

        offsets, cursor = {}, 0
        for name, nbytes in (("partial", max_rows * cols * 2), ("q", max_rows * cols),
                             ("scales", cols // 128 * max_rows * 4), ("normed", max_rows * cols * 2),
                             ("flags", 2 * _lib.TP_MAX_RANKS * 4), ("landing", tp * max_rows * cols * 2)):
            offsets[name] = cursor
            cursor = _align(cursor + nbytes)
        return offsets, cursor

    def _view(self, block: torch.Tensor, name: str, dtype: torch.dtype, shape: tuple[int, ...]) -> torch.Tensor:
        nbytes = torch.empty((), dtype=dtype).element_size()
        for extent in shape:
            nbytes *= extent
        start = self._offsets[name]
        return block[start:start + nbytes].view(dtype).view(shape)

    def _exchange_handles(self, group) -> list[int]:
        import torch.distributed as dist

        lib = _lib.load()
        handle = (ctypes.c_uint8 * _lib.IPC_HANDLE_BYTES)()
        offset = ctypes.c_int64(0)
        torch.cuda.synchronize(self.device)  # the zero fill has landed before anyone maps the block
        _lib.check(lib.mie_ipc_export(_lib.ptr(self.block), handle, ctypes.byref(offset)))
        mine = (bytes(handle), int(offset.value))
        gathered: list = [None] * self.tp
        dist.all_gather_object(gathered, mine, group=group)
        bases = []
        for peer, (peer_handle, peer_offset) in enumerate(gathered):
            if peer == self.rank:
                bases.append(int(self.block.data_ptr()))
                continue
            raw = (ctypes.c_uint8 * _lib.IPC_HANDLE_BYTES).from_buffer_copy(peer_handle)
            mapped = ctypes.c_void_p()
            _lib.check(lib.mie_ipc_open(raw, peer_offset, ctypes.byref(mapped)))
            self._mapped.append((int(mapped.value), peer_offset))
            bases.append(int(mapped.value))
        dist.barrier(group=group)  # every rank has mapped every block before the first kernel uses one
        return bases

    def _peers(self, quantized: bool) -> _lib.TpPeersT:
        peers = _lib.TpPeersT()
        for r in range(self.tp):
            base = self._bases[r]
            peers.partial[r] = base + self._offsets["partial"]
            peers.flags[r] = base + self._offsets["flags"]
            if quantized:
                peers.q[r] = base + self._offsets["q"]
                peers.scales[r] = base + self._offsets["scales"]
            else:
                peers.normed[r] = base + self._offsets["normed"]
        return peers

    def push_gemm(self, quantized: tuple[torch.Tensor, torch.Tensor], weight: torch.Tensor, weight_scale: torch.Tensor,
                  rows: int, k: int, *, status: torch.Tensor | None = None, max_split: int | None = None) -> None:
        """The row-parallel projection of ``rows`` quantised rows whose output goes straight to the owners'
        landing areas (``mie_fp8_gemm_tp_push``); follow it with ``reduce_norm(rows, ..., pushed=True)``."""

        from ..kernels import sm89_fp8

        if rows > self.max_rows or int(weight.shape[0]) != self.cols:
            raise ValueError(f"{rows} rows x {int(weight.shape[0])} columns do not fit the exchange "
                             f"({self.max_rows} x {self.cols})")
        push = _lib.TpPushT()
        slot_bytes = self.max_rows * self.cols * 2
        for r in range(self.tp):
            push.rows[r] = self._bases[r] + self._offsets["landing"] + self.rank * slot_bytes
            push.arrived[r] = self._bases[r] + self._offsets["flags"] + 4 * self.ARRIVED_WORD
        push.ld, push.tp, push.rows_per_rank = self.cols, self.tp, max(1, -(-rows // self.tp))
        sm89_fp8.launch_fp8_gemm_push(quantized[0], quantized[1], weight, weight_scale, push, rows, k, self.device,
                                      status=status, max_split=max_split)

    def owned_rows(self, rows: int) -> range:
        per_rank = (rows + self.tp - 1) // self.tp
        begin = min(per_rank * self.rank, rows)
        return range(begin, min(begin + per_rank, rows))

    def reduce_norm(self, rows: int, residual: torch.Tensor, summed: torch.Tensor, weight: torch.Tensor, eps: float,
                    *, quantized: bool, status: torch.Tensor | None = None, max_polls: int = 0,
                    pushed: bool = False) -> None:
        """``partial[:rows]`` of all ranks (``pushed``: the local landing slots ``push_gemm`` filled) -> ``summed``
        (owned rows) and ``q``/``scales`` or ``normed`` on every rank.  ``residual`` and ``summed`` are local
        ``[rows, cols]`` tensors of which only the owned rows are used."""

        if rows > self.max_rows:
            raise ValueError(f"{rows} rows exceed the exchange capacity {self.max_rows}")
        for name, tensor in (("residual", residual), ("summed", summed)):
            if tensor.dtype != torch.bfloat16 or tensor.shape[-1] != self.cols or not tensor.is_contiguous():
                raise ValueError(f"{name} must be contiguous bf16 [rows, {self.cols}]")
        word = status if status is not None else _lib.status_word(self.device)
        peers = self._peers(quantized)
        if pushed:
            _lib.check(_lib.load().mie_tp_reduce_rms_norm_pushed(
                ctypes.byref(peers), self.tp, self.rank, _lib.ptr(self.landing), self.cols, self.max_rows * self.cols,
                _lib.ptr(self.flags[self.ARRIVED_WORD:]), _lib.ptr(residual), _lib.ptr(summed), _lib.ptr(weight),
                self.cols, self.max_rows, rows, self.cols, float(eps), _lib.ptr(self.state), int(max_polls),
                _lib.ptr(word), _lib.stream_arg(self.device)))
            return
        _lib.check(_lib.load().mie_tp_reduce_rms_norm(
            ctypes.byref(peers), self.tp, self.rank, self.cols, _lib.ptr(residual), _lib.ptr(summed), _lib.ptr(weight),
            self.cols, self.max_rows, rows, self.cols, float(eps), _lib.ptr(self.state), int(max_polls), _lib.ptr(word),
            _lib.stream_arg(self.device)))

    def close(self) -> None:
        lib = _lib.load()
        for mapped, offset in self._mapped:
            lib.mie_ipc_close(mapped, offset)
        self._mapped = []
