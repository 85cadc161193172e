"""The decode-time attention path of the reference's attention manager, on this library's kernels.

Mirrors what ``QwenSSPAAttentionManager`` does for a layer whose cache has been packed
(r2omni/sspa/integration/qwen_sspa_attention.py): ``_prepare_executor`` (:1108-1200), ``_project_qkv``
(:1202-1248), ``_run_fourq`` (:1633-1647), ``_append_generated_token`` (:1649-1678) and the decode branch of
``_active_forward`` (:1778-1847), with ``kernel_backend = "cuda_sm100"`` in place of the reference's
``"triton_mixed_fused_splitk"``.  What the reference's manager does around that path -- installing forward hooks on
a Hugging Face model, the prefill-time policy that assigns page precisions, statistics -- is not here: a caller
hands over packed caches (``build_three_precision_cache`` or ``adopt_reference_cache``) and any attention module
object with ``q_proj / k_proj / v_proj / o_proj`` callables.

Differences that follow from the kernels: one launch per step instead of three; a flush never invalidates the
executor (arenas are preallocated and the flush runs on the stream), so nothing is rebuilt after it; the fused
append takes its indices from a device tensor when asked to, so that a whole decode step can be replayed from a CUDA
graph.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

from .cache import ThreePrecisionCache
from .dynamic import DynamicCacheStats, append_generated_token, flush_recent
from .executor import (SplitKExecutor, allocate_splitk_workspace, prepare_splitk_executor,
                       stack_homogeneous_splitk_executors)
from .hadamard import qwen_qk_mrope, qwen_qkv_prologue, triton_fwht_128

KERNEL_BACKEND = "cuda_sm100"


@dataclass
class LayerState:
    """The fields of the reference's per-layer state that the decode path touches
    (r2omni/sspa/integration/qwen_sspa_runtime.py:15-50)."""

    layer_id: int
    fourq_executor: SplitKExecutor
    fourq_cache: ThreePrecisionCache | None     # None for a stacked (batch > 1) executor: it owns the arenas
    original_seq_len: int
    num_heads: int
    dynamic_stats: DynamicCacheStats = field(default_factory=DynamicCacheStats)
    calls: int = 0
    kernel_calls: int = 0
    append_count: int = 0
    generated_recompress_count: int = 0
    flush_decode_steps: list = field(default_factory=list)
    last_cache_position: int = -1
    migrated: bool = True


class PackedKVAttentionManager:
    """Decode-time attention over packed caches, one state per layer.

    ``manager.adopt_layer(layer_id, caches, seq_len)`` plays the role of the end of ``_finalize_prefill_layer``
    (a list of per-request caches becomes one stacked executor, as ``enable_homogeneous_decode_batch`` does);
    ``manager.active_forward(layer_id, module, hidden_states, position_embeddings, cache_position)`` is one decode
    step of that layer: project, rotate, append (fused into the decode launch while the residual window has room,
    quantize-and-pack flush first when it is full), attend, project out.
    """

    kernel_backend = KERNEL_BACKEND

    def __init__(self, *, num_query_heads: int, mrope_section=(16, 24, 24), key_hadamard: bool = False,
                 value_hadamard: bool = False, validate_kernel_output: bool = False, device_positions: bool = False):
        self.num_query_heads = int(num_query_heads)
        self.mrope_section = tuple(int(v) for v in mrope_section)
        self.key_hadamard, self.value_hadamard = bool(key_hadamard), bool(value_hadamard)
        self.validate_kernel_output = bool(validate_kernel_output)
        # append indices from a device tensor [B,2] that the caller advances on the stream (graph replay), instead
        # of two Python integers per step
        self.device_positions = bool(device_positions)
        self._states: dict[int, LayerState] = {}
        self._throughput_batch_size = 1

    # ---- set-up --------------------------------------------------------------------------------------------
    def _prepare_executor(self, caches) -> tuple[SplitKExecutor, ThreePrecisionCache | None]:
        """qwen_sspa_attention.py:1108-1200: workspace + executor per cache, stacked when there are several
        requests.  The output Hadamard runs in the decode epilogue when values were rotated before packing."""
        singles = []
        for cache in caches:
            if not isinstance(cache, ThreePrecisionCache):
                raise TypeError("adopt_layer expects ThreePrecisionCache objects of this library")
            ws = allocate_splitk_workspace(cache, num_query_heads=self.num_query_heads)
            singles.append(prepare_splitk_executor(cache, ws, output_hadamard=self.value_hadamard))
        if len(singles) == 1:
            return singles[0], caches[0]
        return stack_homogeneous_splitk_executors(singles), None

    def adopt_layer(self, layer_id: int, caches, seq_len: int) -> LayerState:
        caches = list(caches) if isinstance(caches, (list, tuple)) else [caches]
        executor, cache = self._prepare_executor(caches)
        if self._states and executor.arenas.batch != self._throughput_batch_size:
            raise ValueError("every layer must hold the same number of requests")
        self._throughput_batch_size = executor.arenas.batch
        state = LayerState(int(layer_id), executor, cache, int(seq_len), self.num_query_heads)
        self._states[int(layer_id)] = state
        return state

    # ---- one decode step -----------------------------------------------------------------------------------
    def _project_qkv(self, module: Any, hidden_states: torch.Tensor, position_embeddings):
        """qwen_sspa_attention.py:1202-1248 (the Qwen2.5-Omni branch: fused multimodal RoPE, optional Hadamard).
        Returns (q, k, v, value_ready): with a fused ``qkv_proj`` on the module the value rows come back already
        rotated when ``value_hadamard`` is on."""
        batch_size = int(hidden_states.shape[0])
        if int(hidden_states.shape[1]) != 1:
            raise ValueError("compact fused mRoPE decode requires one token per request")
        if batch_size != self._throughput_batch_size:
            raise ValueError("decode batch does not match the active throughput cache arena: "
                             f"hidden={batch_size}, cache={self._throughput_batch_size}")
        if position_embeddings is None or len(position_embeddings) != 2:
            raise ValueError("Qwen position_embeddings are required")
        d = int(module.head_dim)
        cos, sin = position_embeddings
        fused = getattr(module, "qkv_proj", None)
        if fused is not None:
            # one projection for the three (not in the reference's modules; serving stacks fuse them): its output is
            # read in place by the prologue launch, which also brings the value rows along, rotated when asked to
            qkv = fused(hidden_states)
            nq = self.num_query_heads * d
            nkv = (int(qkv.shape[-1]) - nq) // 2
            return qwen_qkv_prologue(qkv[..., :nq], qkv[..., nq : nq + nkv], qkv[..., nq + nkv :], cos, sin, self.mrope_section,
                                     key_hadamard=self.key_hadamard, value_hadamard=self.value_hadamard) + (True,)
        q = module.q_proj(hidden_states).view(batch_size, 1, -1, d).transpose(1, 2).contiguous()
        k = module.k_proj(hidden_states).view(batch_size, 1, -1, d).transpose(1, 2).contiguous()
        v = module.v_proj(hidden_states).view(batch_size, 1, -1, d).transpose(1, 2).contiguous()
        q, k = qwen_qk_mrope(q, k, cos, sin, self.mrope_section, apply_hadamard=self.key_hadamard)
        return q, k, v, False

    def _kernel_value(self, value: torch.Tensor) -> torch.Tensor:
        return triton_fwht_128(value) if self.value_hadamard else value

    def _run_fourq(self, state: LayerState, q: torch.Tensor, append=None) -> torch.Tensor:
        """qwen_sspa_attention.py:1633-1647."""
        state.kernel_calls += 1
        return state.fourq_executor(q, append=append)

    def _append_generated_token(self, state: LayerState, new_k, new_v, current_position: int) -> bool:
        """qwen_sspa_attention.py:1649-1678, the branch taken when the residual window is full."""
        target = state.fourq_cache if state.fourq_cache is not None else state.fourq_executor.arenas
        return append_generated_token(target, new_k, new_v, global_token_index=current_position,
                                      logical_position=current_position, stats=state.dynamic_stats)

    def flush_if_full(self, layer_id: int) -> bool:
        """Quantize-and-pack the residual window of a layer when it is full (the flush half of
        ``_append_generated_token``), so that the step that follows can fuse its append.  A caller that replays
        decode steps from a CUDA graph calls this between replays."""
        state = self._states[int(layer_id)]
        arenas = state.fourq_executor.arenas
        if arenas.recent_len < arenas.recent_capacity:
            return False
        flush_recent(arenas, state.dynamic_stats)
        state.generated_recompress_count += 1
        state.flush_decode_steps.append(state.append_count + 1)
        return True

    def active_forward(self, layer_id: int, module: Any, hidden_states: torch.Tensor, position_embeddings,
                       cache_position=None, append_indices: torch.Tensor | None = None) -> torch.Tensor:
        """The decode branch of ``_active_forward`` (qwen_sspa_attention.py:1778-1847) for one layer: returns the
        attention block's output ``[B,1,hidden]``.  ``cache_position`` is the append position (default: the
        layer's sequence length); with ``device_positions`` the launch reads its indices from ``append_indices``
        (device i64 ``[B,2]``) instead."""
        state = self._states[int(layer_id)]
        state.calls += 1
        q, new_k, new_v, value_ready = self._project_qkv(module, hidden_states, position_embeddings)
        kernel_new_k, kernel_new_v = new_k, (new_v if value_ready else self._kernel_value(new_v))
        current_position = state.original_seq_len if cache_position is None else int(cache_position)
        arenas = state.fourq_executor.arenas
        fused_append = None
        if current_position == state.last_cache_position:
            pass   # the same position twice: the token is already in the window
        else:
            if current_position != state.original_seq_len:
                raise RuntimeError(f"cache position {current_position} is not append position {state.original_seq_len}")
            if arenas.recent_len < arenas.recent_capacity:
                if self.device_positions:
                    if append_indices is None:
                        raise ValueError("device_positions needs the append_indices tensor")
                    fused_append = (kernel_new_k, kernel_new_v, append_indices, None)
                else:
                    fused_append = (kernel_new_k, kernel_new_v, current_position, current_position)
            elif self._append_generated_token(state, kernel_new_k, kernel_new_v, current_position):
                state.generated_recompress_count += 1       # flushed; the executor stays valid
                state.flush_decode_steps.append(state.append_count + 1)
            state.append_count += 1
            state.original_seq_len += 1
            state.last_cache_position = current_position
        mixed = self._run_fourq(state, q, append=fused_append)
        if fused_append is not None:
            if not state.fourq_executor.batched:    # a stacked executor advances its own mirror
                arenas.recent_len += 1
            state.dynamic_stats.appended_tokens += 1
        if self.validate_kernel_output:
            torch._assert_async(torch.isfinite(mixed).all(), "four-quadrant attention produced NaN/Inf")
        return module.o_proj(mixed.reshape(int(hidden_states.shape[0]), 1, -1).to(hidden_states.dtype))

    # ---- bookkeeping ---------------------------------------------------------------------------------------
    def get_stats(self) -> dict:
        """Per-layer counters in the shape of the reference's ``get_stats`` entries for the decode path."""
        out = {}
        for layer_id, s in self._states.items():
            a = s.fourq_executor.arenas
            out[layer_id] = {
                "kernel_backend": self.kernel_backend, "calls": s.calls, "kernel_calls": s.kernel_calls,
                "append_count": s.append_count, "generated_recompress_count": s.generated_recompress_count,
                "flush_decode_steps": list(s.flush_decode_steps), "flushed_tokens": s.dynamic_stats.flushed_tokens,
                "sequence_length": s.original_seq_len, "recent_fp_tokens": a.recent_len,
                "int2_tokens": a.i2_active, "requests": a.batch,
            }
        return out
