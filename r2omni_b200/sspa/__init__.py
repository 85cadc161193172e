"""Host-side mirror of the reference's ``r2omni.sspa`` packed/active cache API."""
from .cache import (
    CompactInt2ValueArena,
    CompactInt4KeyArena,
    LayerCompressionPlan,
    PackedArenas,
    PageClass,
    PhysicalPageIndex,
    PrecisionPool,
    ThreePrecisionCache,
    adopt_reference_cache,
    build_three_precision_cache,
    precision_cache_active_storage_breakdown,
    precision_cache_storage_breakdown,
)
from .dynamic import DynamicCacheStats, append_generated_token, flush_recent
from .hadamard import normalized_fwht, qwen_qk_mrope, qwen_qkv_prologue, triton_fwht_128
from .integration import KERNEL_BACKEND, LayerState, PackedKVAttentionManager
from .sharded import SequenceShardedExecutor, shard_token_range
from .executor import (
    SplitKExecutor,
    SplitKWorkspace,
    allocate_splitk_workspace,
    allocated_workspace_bytes,
    append_recent_fp,
    append_recent_fp_triton,
    prepare_splitk_executor,
    required_splitk_blocks,
    stack_homogeneous_splitk_executors,
)

__all__ = [
    "CompactInt2ValueArena", "CompactInt4KeyArena", "LayerCompressionPlan", "PackedArenas", "PageClass",
    "PhysicalPageIndex", "PrecisionPool", "ThreePrecisionCache", "adopt_reference_cache", "build_three_precision_cache",
    "precision_cache_active_storage_breakdown", "precision_cache_storage_breakdown",
    "DynamicCacheStats", "append_generated_token", "flush_recent",
    "SplitKExecutor", "SplitKWorkspace", "allocate_splitk_workspace", "allocated_workspace_bytes",
    "append_recent_fp", "append_recent_fp_triton", "prepare_splitk_executor", "required_splitk_blocks",
    "stack_homogeneous_splitk_executors", "SequenceShardedExecutor", "shard_token_range",
    "triton_fwht_128", "normalized_fwht", "qwen_qk_mrope", "qwen_qkv_prologue", "KERNEL_BACKEND", "LayerState", "PackedKVAttentionManager",
]
