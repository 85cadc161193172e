"""Sequence-sharded decode over one NVLink/NVSwitch box.

The reference has no multi-GPU path; this extends its packed decode to a cache
whose logical sequence is split contiguously over the ranks of a process group.
Every rank owns a ThreePrecisionCache over its slice (pages and 32-token key
blocks never straddle a boundary, so per-shard packing is bit-identical to a
single cache), runs the local decode to an un-normalised (max, sum-exp, out)
state per query head, and the states are combined with ONE all-gather of
``B*Hq*130`` floats followed by the exact merge of
r2omni/sspa/kernels/triton_fourq_attention.py:58-69 on every rank.  The residual
window and the flush live on the last rank only.

``fused=True`` replaces the all-gather and the merge launch by peer stores inside
the decode kernel: every rank's last CTA of a (request, kv head) writes its state
rows into every rank's exchange buffer over NVLink as (value, step) words, waits
(bounded) until every rank's words of the step have landed in its own buffer and
merges in place (``r2k_decode_exchange``).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib as L
from .cache import _stream_ptr, dtype_code
from .executor import SplitKExecutor


def shard_token_range(total_tokens: int, world: int, rank: int, *, align: int = 128) -> tuple[int, int]:
    """Contiguous slice [start, end) of rank ``rank``: as even as possible in units of
    ``align`` tokens (a multiple of the page size and of the key block), the remainder on the last rank."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank must lie in [0, world)")
    if align < 1 or total_tokens < 0:
        raise ValueError("align must be positive and total_tokens non-negative")
    units = total_tokens // align
    base, extra = divmod(units, world)
    start_units = rank * base + min(rank, extra)
    end_units = start_units + base + (1 if rank < extra else 0)
    start, end = start_units * align, end_units * align
    if rank == world - 1:
        end = total_tokens
    return start, end


class SequenceShardedExecutor:
    """``executor(query, append=None)`` over a sequence-sharded cache.

    ``local`` is this rank's SplitKExecutor.  ``append`` is honoured on the last
    rank (which owns the residual window) and ignored elsewhere, so every rank can
    make the same call.
    """

    def __init__(self, local: SplitKExecutor, group=None, *, fused: bool = False, device_step_counter: bool = False,
                 wait_us: int = 0):
        import torch.distributed as dist
        self._dist = dist
        self.local, self.group = local, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.fused = bool(fused) and self.world > 1
        # the step counter of the fused merge lives on the host (one integer per call) or, for calls that are
        # captured into a CUDA graph and replayed, on the device
        self.device_step_counter = bool(device_step_counter)
        # microseconds the fused merge waits for the other ranks' rows before it reports a device timeout (0: the
        # library's default, about a second)
        self.wait_us = int(wait_us)
        self._exchange, self._mapped, self._own = None, [], None
        if self.fused:
            self._open_exchange()
        a = local.arenas
        shape = (a.batch, local.num_query_heads, 130)
        self.state = torch.empty(shape, device=a.device, dtype=torch.float32)
        self.gathered = torch.empty((self.world * a.batch, local.num_query_heads, 130), device=a.device, dtype=torch.float32)
        self.output = torch.empty((a.batch, local.num_query_heads, 128), device=a.device, dtype=torch.bfloat16)
        self._staging = None if a.dtype == torch.bfloat16 else torch.empty(self.output.shape, device=a.device,
                                                                           dtype=torch.float32)

    def _open_exchange(self) -> None:
        """One exchange buffer per rank, created here and mapped into every other rank through its 64-byte
        inter-process handle (exchanged with one all_gather_object)."""
        if self.world > L.MAX_RANKS:
            raise ValueError(f"the fused merge supports at most {L.MAX_RANKS} ranks")
        lib, a = L.lib(), self.local.arenas
        geom = a.geom(self.local.num_query_heads)
        need = C.c_size_t(0)
        L.check(lib.r2k_exchange_bytes(C.byref(geom), self.world, C.byref(need)), "r2k_exchange_bytes")
        own, handle = C.c_void_p(0), (C.c_ubyte * 64)()
        with torch.cuda.device(a.device):
            L.check(lib.r2k_exchange_create(C.c_size_t(need.value), C.byref(own), handle), "r2k_exchange_create")
            handles = [None] * self.world
            self._dist.all_gather_object(handles, (self.rank, bytes(handle)), group=self.group)
            ex = L.Exchange()
            ex.rank, ex.world, ex.seq, ex.wait_us = self.rank, self.world, 0, self.wait_us
            for r, raw in handles:
                if r == self.rank:
                    ex.buffers[r] = own.value
                    continue
                ptr = C.c_void_p(0)
                L.check(lib.r2k_exchange_open((C.c_ubyte * 64).from_buffer_copy(raw), C.byref(ptr)), "r2k_exchange_open")
                ex.buffers[r] = ptr.value
                self._mapped.append(ptr.value)
        self._own, self._exchange = own.value, ex
        self._dist.barrier(group=self.group)   # nobody starts a step before every mapping exists

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's (call on every rank, after the last step completed)."""
        if self._exchange is None:
            return
        torch.cuda.synchronize(self.local.arenas.device)
        self._dist.barrier(group=self.group)
        lib = L.lib()
        for ptr in self._mapped:
            lib.r2k_exchange_close(C.c_void_p(ptr), 1)
        self._dist.barrier(group=self.group)
        lib.r2k_exchange_close(C.c_void_p(self._own), 0)
        self._exchange, self._mapped, self._own, self.fused = None, [], None, False

    def __call__(self, query: torch.Tensor, append=None) -> torch.Tensor:
        ex = self.local
        a = ex.arenas
        mine = append if self.rank == self.world - 1 else None
        if self.fused:
            self._exchange.seq = 0 if self.device_step_counter else ((self._exchange.seq + 1) & 0xFFFFFFFF or 1)
            return ex.decode_exchange(query, self._exchange, self.output, append=mine)
        ex.decode_state(query, out=self.state, append=mine)
        if self.world > 1:
            self._dist.all_gather_into_tensor(self.gathered, self.state, group=self.group)
            states = self.gathered
        else:
            states = self.state
        rows = a.batch * ex.num_query_heads
        flags = L.FLAG_OUTPUT_HADAMARD if ex.output_hadamard else 0
        out = self.output if self._staging is None else self._staging
        if self._staging is not None:
            flags |= L.FLAG_OUT_F32
        L.check(L.lib().r2k_merge_states(
            C.c_void_p(states.data_ptr()), self.world, C.c_int64(rows * 130), rows, dtype_code(a.dtype),
            C.c_void_p(out.data_ptr()), C.c_uint32(flags), C.c_void_p(_stream_ptr(a.device))), "r2k_merge_states")
        if self._staging is not None:
            self.output.copy_(self._staging)
        return self.output
