"""Append / flush state machine of the residual window.

Mirrors r2omni/sspa/runtime/dynamic_fourq_cache.py:16-24, 172-267.  The flush
(quantize-and-pack of the oldest 128 tokens into the INT4 key arena and the INT2
value arena, metadata append, ring slide) is three launches on the current
stream with no host synchronisation; arenas are preallocated, so no device
pointer changes and no executor has to be rebuilt afterwards.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from .. import _lib as L
from .cache import PackedArenas, ThreePrecisionCache, _stream_ptr
from .executor import append_recent_fp_triton


@dataclass
class DynamicCacheStats:
    """dynamic_fourq_cache.py:16-24."""

    appended_tokens: int = 0
    flushed_superblocks: int = 0
    flushed_tokens: int = 0
    flushed_int4_value_tokens: int = 0
    recent_reallocation_count: int = 0
    local_tail_dequant_tokens: int = 0
    full_dequant_tensor_count: int = 0


def flush_recent(arenas: PackedArenas, stats: DynamicCacheStats | None = None) -> int:
    """Flush the oldest ``arenas.flush`` ring tokens of every request.  Returns
    the number of already-packed key rows that were re-quantised with them."""
    n = arenas.flush
    if arenas.recent_len < n:
        raise RuntimeError("Recent-FP pool holds fewer tokens than one flush")
    if arenas.k_active + n > arenas.k_capacity:
        raise RuntimeError("compact INT4 K capacity exhausted")
    if arenas.i2_active + n > arenas.i2_capacity:
        raise RuntimeError(
            f"compact INT2 V capacity exhausted: need {arenas.i2_active + n}, have {arenas.i2_capacity}")
    if arenas.i2_active + n > arenas.i2_global.shape[1]:
        raise RuntimeError("compact INT2 token metadata capacity exhausted")
    tail = arenas.k_active % arenas.k_block
    geom = arenas.geom(arenas.num_kv_heads)
    meta = arenas.i2_global
    L.check(L.lib().r2k_flush_recent(
        C.byref(geom), C.byref(arenas.view()), C.c_int32(arenas.recent_len), C.c_int32(n),
        C.c_int64(arenas.k_active), C.c_int64(arenas.i2_active),
        C.c_void_p(arenas.i2_global.data_ptr()), C.c_void_p(arenas.i2_logical.data_ptr()),
        C.c_int64(0 if arenas.batch == 1 else meta.stride(0) * 8), C.c_int64(arenas.i2_active),
        C.c_void_p(_stream_ptr(arenas.device))), "r2k_flush_recent")
    arenas.k_active += n
    arenas.i2_active += n
    arenas.recent_len -= n
    if stats is not None:
        stats.local_tail_dequant_tokens += tail
        stats.flushed_superblocks += 1
        stats.flushed_tokens += n
    return tail


def append_generated_token(
    cache,
    new_key: torch.Tensor,
    new_value: torch.Tensor,
    *,
    global_token_index: int,
    logical_position: int,
    stats: DynamicCacheStats,
) -> bool:
    """Append to fixed Recent-FP storage; flush one configured old-token chunk
    first when the ring is full (dynamic_fourq_cache.py:172-267).  ``cache`` is a
    ThreePrecisionCache, or the PackedArenas of a stacked executor."""
    arenas = cache.arenas if isinstance(cache, ThreePrecisionCache) else cache
    if arenas.recent_capacity < arenas.flush:
        raise RuntimeError("Recent-FP pool was not preallocated for dynamic generation")
    if new_key.ndim == 4 and arenas.batch == 1:
        new_key, new_value = new_key[0], new_value[0]
    if new_key.shape != new_value.shape or new_key.numel() != arenas.batch * arenas.num_kv_heads * 128:
        raise ValueError("new K/V must be [Hkv,1,D] or [1,Hkv,1,D]")
    flushed = False
    if arenas.recent_len == arenas.recent_capacity:
        flush_recent(arenas, stats)
        flushed = True
    append_recent_fp_triton(arenas, new_key, new_value, global_token_index=global_token_index,
                            logical_position=logical_position)
    stats.appended_tokens += 1
    return flushed
