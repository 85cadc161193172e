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

    def __init__(self, local: SplitKExecutor, group=None):
        import torch.distributed as dist
        self._dist = dist
        self.local, self.group = local, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        a = local.arenas
        shape = (a.batch, local.num_query_heads, 130)
        self.state = torch.empty(shape, device=a.device, dtype=torch.float32)
        self.gathered = torch.empty((self.world * a.batch, local.num_query_heads, 130), device=a.device, dtype=torch.float32)
        self.output = torch.empty((a.batch, local.num_query_heads, 128), device=a.device, dtype=torch.bfloat16)
        self._staging = None if a.dtype == torch.bfloat16 else torch.empty(self.output.shape, device=a.device,
                                                                           dtype=torch.float32)

    def __call__(self, query: torch.Tensor, append=None) -> torch.Tensor:
        ex = self.local
        a = ex.arenas
        mine = append if self.rank == self.world - 1 else None
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
