"""Buffers and peer mappings of the fused tensor-parallel exchange (``mie_tp_reduce_rms_norm``).

Under head-sharded tensor parallelism the two row-parallel projections of a layer (o_proj, down_proj) leave
partial sums on every rank.  The reference runs on one GPU and has no counterpart; the plain formulation is
``all_reduce`` followed by the residual add + RMSNorm + quantisation.  Here each rank keeps ONE device block
that its peers map through CUDA IPC::

    partial [rows, cols] bf16 | q [rows, cols] e4m3 | scales [cols/128, rows] f32 | normed [rows, cols] bf16 | flags

and one kernel per rank does the exchange and the norm together (see ``csrc/peer_reduce.cu``).  The row-parallel
GEMM writes straight into ``partial``; the next column-parallel GEMM reads ``q`` / ``scales`` (or the lm_head
reads ``normed``), which every rank's kernel has filled for the rows it owns.
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
        self._offsets, cursor = self.layout(max_rows, cols)
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

    @staticmethod
    def layout(max_rows: int, cols: int) -> tuple[dict[str, int], int]:
        """Byte offsets of the five regions inside a rank's block, and the block size."""

        offsets, cursor = {}, 0
        for name, nbytes in (("partial", max_rows * cols * 2), ("q", max_rows * cols),
                             ("scales", cols // 128 * max_rows * 4), ("normed", max_rows * cols * 2),
                             ("flags", 2 * _lib.TP_MAX_RANKS * 4)):
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

    def owned_rows(self, rows: int) -> range:
        per_rank = (rows + self.tp - 1) // self.tp
        begin = min(per_rank * self.rank, rows)
        return range(begin, min(begin + per_rank, rows))

    def reduce_norm(self, rows: int, residual: torch.Tensor, summed: torch.Tensor, weight: torch.Tensor, eps: float,
                    *, quantized: bool, status: torch.Tensor | None = None, max_polls: int = 0) -> None:
        """``partial[:rows]`` of all ranks -> ``summed`` (owned rows) and ``q``/``scales`` or ``normed`` on every
        rank.  ``residual`` and ``summed`` are local ``[rows, cols]`` tensors of which only the owned rows are used."""

        if rows > self.max_rows:
            raise ValueError(f"{rows} rows exceed the exchange capacity {self.max_rows}")
        for name, tensor in (("residual", residual), ("summed", summed)):
            if tensor.dtype != torch.bfloat16 or tensor.shape[-1] != self.cols or not tensor.is_contiguous():
                raise ValueError(f"{name} must be contiguous bf16 [rows, {self.cols}]")
        word = status if status is not None else _lib.status_word(self.device)
        peers = self._peers(quantized)
        _lib.check(_lib.load().mie_tp_reduce_rms_norm(
            ctypes.byref(peers), self.tp, self.rank, self.cols, _lib.ptr(residual), _lib.ptr(summed), _lib.ptr(weight),
            self.cols, self.max_rows, rows, self.cols, float(eps), _lib.ptr(self.state), int(max_polls), _lib.ptr(word),
            _lib.stream_arg(self.device)))

    def close(self) -> None:
        lib = _lib.load()
        for mapped, offset in self._mapped:
            lib.mie_ipc_close(mapped, offset)
        self._mapped = []
