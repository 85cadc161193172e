"""Split-K decode executor: the reference's operator API over one CUDA launch.

Mirrors r2omni/sspa/kernels/triton_fourq_splitk.py:1158-2256 (SplitKWorkspace,
SplitKExecutor, allocate_splitk_workspace, required_splitk_blocks,
prepare_splitk_executor, stack_homogeneous_splitk_executors,
append_recent_fp_triton, allocated_workspace_bytes).  Tuning keywords of the
Triton implementation (warps, stages, tensor-core switches, block_n, ...) are
accepted and ignored: the CUDA kernel chooses its own tiling.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Sequence

import torch

from .. import _lib as L
from .cache import PackedArenas, ThreePrecisionCache, _stream_ptr, dtype_code, stack_arenas


@dataclass
class SplitKWorkspace:
    """Scratch of one decode launch plus the aliased output tensor."""

    buffer: torch.Tensor          # u8, partial (max, sum-exp, out) slots + arrival counters
    output: torch.Tensor          # bf16 [B,Hq,128]; overwritten by every call
    staging: torch.Tensor | None  # f32 [B,Hq,128], only when the cache dtype is not bf16
    block_n: int
    total_blocks: int
    num_query_heads: int


def _workspace_bytes(arenas: PackedArenas, num_query_heads: int) -> int:
    need = C.c_size_t(0)
    geom = arenas.geom(num_query_heads, full_capacity=True)
    L.check(L.lib().r2k_decode_workspace_bytes(C.byref(geom), C.byref(need)), "r2k_decode_workspace_bytes")
    return int(need.value)


def required_splitk_blocks(cache: ThreePrecisionCache, *, block_n: int = 128, reserve_tokens: int = 0) -> int:
    """triton_fourq_splitk.py:1679-1692 (kept for callers that size shared workspaces)."""
    if block_n < 1:
        raise ValueError("block_n must be positive")
    a = cache.arenas
    counts = (a.n_fp, a.recent_capacity, a.n_i4, a.i2_active)
    return sum(-(-c // block_n) for c in counts) + -(-max(0, int(reserve_tokens)) // block_n)


def _allocate(arenas: PackedArenas, num_query_heads: int, block_n: int, total_blocks: int) -> SplitKWorkspace:
    dev = arenas.device
    nbytes = _workspace_bytes(arenas, num_query_heads)
    buffer = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    L.check(L.lib().r2k_decode_workspace_init(C.c_void_p(buffer.data_ptr()), C.c_size_t(nbytes),
                                              C.c_void_p(_stream_ptr(dev))), "r2k_decode_workspace_init")
    shape = (arenas.batch, num_query_heads, 128)
    staging = None if arenas.dtype == torch.bfloat16 else torch.empty(shape, device=dev, dtype=torch.float32)
    return SplitKWorkspace(buffer, torch.empty(shape, device=dev, dtype=torch.bfloat16), staging, int(block_n),
                           int(total_blocks), int(num_query_heads))


def allocate_splitk_workspace(
    cache: ThreePrecisionCache,
    *,
    num_query_heads: int = 16,
    block_n: int = 128,
    reserve_tokens: int = 0,
    device: torch.device | None = None,
    partial_output_dtype: torch.dtype = torch.float32,
    hierarchical_group_blocks: int = 64,
) -> SplitKWorkspace:
    """triton_fourq_splitk.py:1607-1676.  Sized for the cache's full append
    capacity, so flushes never require a new workspace."""
    if partial_output_dtype not in {torch.float16, torch.float32}:
        raise ValueError("partial_output_dtype must be float16 or float32")
    if hierarchical_group_blocks not in {16, 32, 64}:
        raise ValueError("hierarchical_group_blocks must be 16, 32, or 64")
    if int(num_query_heads) < 1:
        raise ValueError("num_query_heads must be positive")
    required = required_splitk_blocks(cache, block_n=block_n, reserve_tokens=reserve_tokens)
    if required <= 0:
        raise ValueError("cannot allocate workspace for an empty cache")
    if device is not None and torch.device(device) != cache.arenas.device:
        raise ValueError("workspace device must be the cache device")
    return _allocate(cache.arenas, int(num_query_heads), block_n, required)


def allocated_workspace_bytes(workspace: SplitKWorkspace) -> int:
    """triton_fourq_splitk.py:2244-2256."""
    extra = 0 if workspace.staging is None else workspace.staging.numel() * 4
    return int(workspace.buffer.numel() + workspace.output.numel() * 2 + extra)


class SplitKExecutor:
    """``executor(query, append=None) -> Tensor[B,Hq,128]`` (bf16, aliased).

    With ``append=(k, v, global_index, logical_position)`` the new token takes
    part in the attention and is written to the Recent-FP ring by the same
    launch (triton_fourq_splitk.py:1243-1547).  As in the reference, a B == 1
    caller bumps ``cache.recent_fp_pool.active_length`` itself after the call;
    a stacked (B > 1) executor advances its own host mirror.
    """

    def __init__(self, arenas: PackedArenas, workspace: SplitKWorkspace, *, output_hadamard: bool = False,
                 cache: ThreePrecisionCache | None = None, sm_scale: float = 0.0):
        self.arenas, self.workspace, self.cache = arenas, workspace, cache
        self.output_hadamard = bool(output_hadamard)
        self.num_query_heads = workspace.num_query_heads
        self.num_key_value_heads = arenas.num_kv_heads
        self.head_dim = 128
        self.block_n = workspace.block_n
        self.sm_scale = float(sm_scale)
        self._append = L.Append()
        self._lib = L.lib()
        self._geom = arenas.geom(self.num_query_heads, sm_scale=self.sm_scale)
        self._idx = None
        # per-step constants of the launch, built once
        self._decode = self._lib.r2k_decode
        self._decode_host = self._lib.r2k_decode_host
        self._geom_ref = C.byref(self._geom)
        self._append_ref = C.byref(self._append)
        self._view_obj, self._view_ref = None, None
        self._ws_ptr, self._ws_size = workspace.buffer.data_ptr(), workspace.buffer.numel()
        self._qshape = (arenas.batch, self.num_query_heads, 128)
        self._host_staging, self._host_pair = None, None

    @property
    def batched(self) -> bool:
        return self.arenas.batch > 1

    def _launch(self, query, append, out_ptr, flags) -> None:
        a = self.arenas
        geom = self._geom
        geom.n_i2 = a.i2_active   # the only extent that moves during generation (flushes)
        view = a.view()
        if view is not self._view_obj:
            self._view_obj, self._view_ref = view, C.byref(view)
        status = self._decode(self._geom_ref, self._view_ref, query.data_ptr(), append, self._ws_ptr, self._ws_size, out_ptr,
                              flags, _stream_ptr(a.device))
        if status:
            L.check(status, "r2k_decode")

    def _check_query(self, query: torch.Tensor) -> torch.Tensor:
        if query.ndim == 4:
            query = query[:, :, 0]
        a = self.arenas
        if (query.shape != self._qshape or query.device != a.device or not query.is_contiguous()
                or query.dtype != a.dtype):
            raise ValueError("query does not match prepared split-K executor")
        return query

    def _make_append(self, append, query):
        a = self.arenas
        if append is None:
            return None
        k, v, global_index, logical_position = append
        n = a.batch * a.num_kv_heads * 128
        if (k.numel() != n or v.numel() != n or k.device != query.device or v.device != query.device
                or not k.is_contiguous() or not v.is_contiguous() or k.dtype != a.dtype or v.dtype != a.dtype):
            raise ValueError("append K/V must be contiguous [B,Hkv,1,D] or [B,Hkv,D]")
        if a.recent_len >= a.recent_capacity:
            raise RuntimeError("prepared executor cannot fuse an append into a full Recent-FP pool")
        ap = self._append
        ap.k, ap.v = k.data_ptr(), v.data_ptr()
        if isinstance(global_index, int) and isinstance(logical_position, int):
            ap.indices, ap.global_index, ap.logical_position = None, global_index, logical_position
            self._idx = None
        elif logical_position is None:
            # a ready device table [B,2] of (global index, logical position): read by the launch in place, so a
            # caller that replays captured steps only has to advance it on the stream
            t = global_index
            if (not torch.is_tensor(t) or t.dtype != torch.int64 or tuple(t.shape) != (a.batch, 2) or t.device != query.device
                    or not t.is_contiguous()):
                raise ValueError("append index table must be a contiguous int64 [B,2] tensor on the cache device")
            self._idx = t
            ap.indices, ap.global_index, ap.logical_position = t.data_ptr(), 0, 0
        else:
            cols = []
            for value in (global_index, logical_position):
                t = torch.as_tensor(value, device=query.device, dtype=torch.int64).reshape(-1)
                if t.numel() == 1:
                    t = t.expand(a.batch)
                elif t.numel() != a.batch:
                    raise ValueError("batched append indices must contain one value per request")
                cols.append(t)
            self._idx = torch.stack(cols, dim=1).contiguous()
            ap.indices, ap.global_index, ap.logical_position = self._idx.data_ptr(), 0, 0
        return self._append_ref

    def __call__(self, query: torch.Tensor, append=None) -> torch.Tensor:
        query = self._check_query(query)
        a = self.arenas
        if append is None and a.n_fp + a.n_i4 + a.i2_active + a.recent_len == 0:
            raise ValueError("four-quadrant cache has no surviving tokens")
        ap = self._make_append(append, query)
        flags = L.FLAG_OUTPUT_HADAMARD if self.output_hadamard else 0
        ws = self.workspace
        if ws.staging is None:
            self._launch(query, ap, ws.output.data_ptr(), flags)
        else:
            # fp16 caches: the kernel's element type is fp16, the operator's output is bf16
            self._launch(query, ap, ws.staging.data_ptr(), flags | L.FLAG_OUT_F32)
            ws.output.copy_(ws.staging)
        if append is not None and self.batched:
            a.recent_len += 1
        return ws.output

    def step_host(self, host_in: torch.Tensor, host_out: torch.Tensor, append_indices=None) -> torch.Tensor:
        """One decode step for a caller whose tensors live in host memory (r2k_decode_host): ``host_in`` is the
        query [B,Hq,128] followed, when ``append_indices = (global_index, logical_position)`` (two ints) is given,
        by the new key and value rows [B,Hkv,128] each, in one contiguous CPU tensor of the cache's element type
        (pinned for asynchronous copies); the result is written to ``host_out`` [B,Hq,128] (same type) and can be
        read on return: the call copies in, launches the decode with its fused append, copies out and waits."""
        a = self.arenas
        if a.dtype != torch.bfloat16:
            raise ValueError("step_host supports bf16 caches")
        nq, nkv = a.batch * self.num_query_heads * 128, a.batch * a.num_kv_heads * 128
        need = nq + (2 * nkv if append_indices is not None else 0)
        if self._host_pair is not None and host_in is self._host_pair[0] and host_out is self._host_pair[1] \
                and need == self._host_pair[2]:
            pass   # the same buffers as in the last call: already checked
        elif (host_in.device.type != "cpu" or host_out.device.type != "cpu" or host_in.dtype != a.dtype
                or host_out.dtype != a.dtype or not host_in.is_contiguous() or not host_out.is_contiguous()
                or host_in.numel() < need or host_out.numel() != nq):
            raise ValueError("host buffers do not match the prepared split-K executor")
        else:
            self._host_pair = (host_in, host_out, need, host_in.data_ptr(), host_out.data_ptr())
        if append_indices is None and a.n_fp + a.n_i4 + a.i2_active + a.recent_len == 0:
            raise ValueError("four-quadrant cache has no surviving tokens")
        ap = None
        if append_indices is not None:
            if a.recent_len >= a.recent_capacity:
                raise RuntimeError("prepared executor cannot fuse an append into a full Recent-FP pool")
            ap = self._append
            ap.k, ap.v, ap.indices = None, None, None
            ap.global_index, ap.logical_position = int(append_indices[0]), int(append_indices[1])
            ap = self._append_ref
        if self._host_staging is None:
            n = C.c_size_t()
            L.check(self._lib.r2k_decode_host_staging_bytes(self._geom_ref, C.byref(n)), "r2k_decode_host_staging_bytes")
            self._host_staging = torch.empty(n.value, device=a.device, dtype=torch.uint8)
            self._host_staging_ptr, self._host_staging_size = self._host_staging.data_ptr(), n.value
        geom = self._geom
        geom.n_i2 = a.i2_active
        view = a.view()
        if view is not self._view_obj:
            self._view_obj, self._view_ref = view, C.byref(view)
        flags = L.FLAG_OUTPUT_HADAMARD if self.output_hadamard else 0
        pair = self._host_pair
        status = self._decode_host(self._geom_ref, self._view_ref, pair[3], ap, self._ws_ptr, self._ws_size,
                                   self._host_staging_ptr, self._host_staging_size, pair[4], flags, _stream_ptr(a.device))
        if status:
            L.check(status, "r2k_decode_host")
        if append_indices is not None and self.batched:
            a.recent_len += 1
        return host_out

    def decode_f32(self, query: torch.Tensor, append=None) -> torch.Tensor:
        """Same launch with an un-rounded float32 result (parity checks)."""
        query = self._check_query(query)
        ap = self._make_append(append, query)
        out = torch.empty((self.arenas.batch, self.num_query_heads, 128), device=query.device, dtype=torch.float32)
        flags = L.FLAG_OUT_F32 | (L.FLAG_OUTPUT_HADAMARD if self.output_hadamard else 0)
        self._launch(query, ap, out.data_ptr(), flags)
        if append is not None and self.batched:
            self.arenas.recent_len += 1
        return out

    def decode_state(self, query: torch.Tensor, out: torch.Tensor | None = None, append=None) -> torch.Tensor:
        """Un-normalised (max, sum-exp, weighted V) per query head, float32
        [B,Hq,130] in natural-log units: the per-shard half of a sequence-sharded decode.
        A shard without any token yields (-inf, 0, 0)."""
        query = self._check_query(query)
        ap = self._make_append(append, query)
        if out is None:
            out = torch.empty((self.arenas.batch, self.num_query_heads, 130), device=query.device, dtype=torch.float32)
        self._launch(query, ap, out.data_ptr(), L.FLAG_OUT_STATE)
        if append is not None and self.batched:
            self.arenas.recent_len += 1
        return out

    def decode_exchange(self, query: torch.Tensor, exchange, out: torch.Tensor, append=None) -> torch.Tensor:
        """Sequence-sharded step with the cross-rank merge fused into the launch (``r2k_decode_exchange``):
        ``exchange`` is the rank's ``R2KExchange`` with this step's counter, ``out`` receives the merged output."""
        query = self._check_query(query)
        a = self.arenas
        if a.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
            raise ValueError("the fused sharded step writes bf16 output for a bf16 cache")
        ap = self._make_append(append, query)
        self._geom.n_i2 = a.i2_active
        view = a.view()
        flags = L.FLAG_OUTPUT_HADAMARD if self.output_hadamard else 0
        status = self._lib.r2k_decode_exchange(C.byref(self._geom), C.byref(view), query.data_ptr(), ap, self._ws_ptr,
                                               self._ws_size, out.data_ptr(), flags, C.byref(exchange), _stream_ptr(a.device))
        if status:
            L.check(status, "r2k_decode_exchange")
        if append is not None and self.batched:
            a.recent_len += 1
        return out

    def device_status(self) -> int:
        status = C.c_int32(0)
        L.check(self._lib.r2k_decode_device_status(C.c_void_p(self.workspace.buffer.data_ptr()), C.byref(status),
                                                   C.c_void_p(_stream_ptr(self.arenas.device))))
        return int(status.value)


def prepare_splitk_executor(
    cache: ThreePrecisionCache,
    workspace: SplitKWorkspace,
    *,
    block_n: int = 128,
    num_warps: int = 8,
    num_stages: int = 2,
    reduce_num_warps: int = 8,
    use_tensor_cores_qk: bool = True,
    use_tensor_cores_pv: bool = False,
    broadcast_k_metadata: bool = False,
    single_request_fastpath: bool | None = None,
    tight_metadata_rows: bool | None = None,
    output_hadamard: bool = False,
    hierarchical_reduce: bool = True,
) -> SplitKExecutor:
    """triton_fourq_splitk.py:1695-1907."""
    if not isinstance(cache, ThreePrecisionCache):
        raise TypeError("prepare_splitk_executor expects a ThreePrecisionCache")
    if workspace.block_n != block_n:
        raise ValueError("cache/workspace is incompatible with a mixed split-K executor")
    a = cache.arenas
    if workspace.num_query_heads % a.num_kv_heads:
        raise ValueError("query heads must be divisible by key/value heads")
    if workspace.num_query_heads // a.num_kv_heads > 8:
        raise ValueError("the B200 split-K executor supports at most 8 GQA heads per KV head")
    if tuple(workspace.output.shape) != (a.batch, workspace.num_query_heads, 128):
        raise ValueError("split-K workspace geometry is inconsistent")
    if workspace.buffer.numel() < _workspace_bytes(a, workspace.num_query_heads):
        raise ValueError("workspace block capacity is smaller than the active cache")
    if workspace.buffer.device != a.device:
        raise ValueError("workspace device must be the cache device")
    return SplitKExecutor(a, workspace, output_hadamard=output_hadamard, cache=cache)


def stack_homogeneous_splitk_executors(
    executors: Sequence[SplitKExecutor],
    *,
    workspace: SplitKWorkspace | None = None,
    throughput_use_tensor_cores_pv: bool = False,
    throughput_direct_reduce_max_splits: int = 0,
) -> SplitKExecutor:
    """Combine independent B == 1 cache snapshots into one throughput executor
    (triton_fourq_splitk.py:1995-2241): payloads are copied once into
    request-major arenas that then own the generated Recent-FP state."""
    executors = tuple(executors)
    if len(executors) < 2:
        raise ValueError("stacking split-K executors requires at least two requests")
    first = executors[0]
    if any(e.arenas.batch != 1 for e in executors):
        raise ValueError("source split-K executors must use batch=1 workspaces")
    if int(throughput_direct_reduce_max_splits) not in {0, 16, 32, 64, 128}:
        raise ValueError("throughput_direct_reduce_max_splits must be 0/16/32/64/128")
    for i, e in enumerate(executors[1:], start=1):
        if (e.num_query_heads, e.output_hadamard) != (first.num_query_heads, first.output_hadamard):
            raise ValueError(f"split-K request {i} is outside the homogeneous bucket: num_query_heads/output_hadamard")
    arenas = stack_arenas([ThreePrecisionCache(e.arenas) for e in executors])
    if workspace is None or tuple(workspace.output.shape) != (arenas.batch, first.num_query_heads, 128) \
            or workspace.buffer.numel() < _workspace_bytes(arenas, first.num_query_heads):
        workspace = _allocate(arenas, first.num_query_heads, first.block_n, first.workspace.total_blocks)
    return SplitKExecutor(arenas, workspace, output_hadamard=first.output_hadamard, cache=None)


def append_recent_fp_triton(cache, new_key, new_value, *, global_token_index: int, logical_position: int) -> None:
    """Append one decode token to Recent-FP with one CUDA launch
    (triton_fourq_splitk.py:1557-1604).  The name is the reference's; the launch is CUDA."""
    a = cache.arenas if isinstance(cache, ThreePrecisionCache) else cache
    if new_key.ndim == 4 and a.batch == 1:
        new_key, new_value = new_key[0], new_value[0]
    n = a.batch * a.num_kv_heads * 128
    if new_key.shape != new_value.shape or new_key.numel() != n:
        raise ValueError("new K/V must be [Hkv,1,D] or [1,Hkv,1,D]")
    if a.recent_len >= a.recent_capacity:
        raise RuntimeError("Recent-FP staging buffer has no append capacity")
    if not new_key.is_cuda or new_key.dtype != a.dtype:
        raise RuntimeError("fused Recent-FP append requires CUDA tensors of the cache dtype")
    new_key, new_value = new_key.contiguous(), new_value.contiguous()
    ap = L.Append()
    ap.k, ap.v, ap.indices = new_key.data_ptr(), new_value.data_ptr(), None
    ap.global_index, ap.logical_position = int(global_token_index), int(logical_position)
    geom = a.geom(a.num_kv_heads)
    L.check(L.lib().r2k_append_recent(C.byref(geom), C.byref(a.view()), C.byref(ap), C.c_void_p(_stream_ptr(a.device))),
            "r2k_append_recent")
    a.recent_len += 1


append_recent_fp = append_recent_fp_triton
