"""Generate golden fixtures for the SSPA packed-KV path FROM THE REFERENCE ITSELF.

Run once, in a container that has the reference checkout (read-only):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/R2-Omni

It imports the unmodified reference (CPU torch path), builds small caches from
seeded inputs, appends tokens through the reference's own flush state machine,
runs the reference's dequantise-then-attend decoder and stores inputs and
results as compressed ``.npz`` files next to this script.  The tests load only
those files; nothing here runs at test time.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

if len(sys.argv) < 2 and "R2OMNI_REFERENCE" not in os.environ:
    raise SystemExit("usage: make_golden.py /path/to/R2-Omni   (or set R2OMNI_REFERENCE)")
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ["R2OMNI_REFERENCE"]
sys.path.insert(0, REF)
sys.dont_write_bytecode = True

from r2omni.sspa.kernels.triton_fourq_attention import triton_mixed_reference  # noqa: E402
from r2omni.sspa.runtime.cache_plan import LayerCompressionPlan  # noqa: E402
from r2omni.sspa.runtime.dynamic_fourq_cache import DynamicCacheStats, append_generated_token  # noqa: E402
from r2omni.sspa.runtime.int2_reference import normalized_fwht  # noqa: E402
from r2omni.sspa.runtime.precision_pool import build_three_precision_cache  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from recipe import digest, make_inputs  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16/fp16 tensors are stored as their raw 16-bit patterns."""
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.detach().clone().contiguous().view(torch.int16).numpy()
    return t.detach().clone().contiguous().numpy()


def make_plan(classes: torch.Tensor, page: int, recent_capacity: int) -> LayerCompressionPlan:
    n = int(classes.numel())
    pos = torch.arange(n * page)
    sel = lambda c: (classes == c).nonzero().flatten()  # noqa: E731
    return LayerCompressionPlan(
        layer_id=0, fp_pages=sel(1), int4_pages=sel(2), int2_pages=sel(5), evicted_pages=sel(0),
        protected_pages=torch.empty(0, dtype=torch.long), recent_fp_capacity=recent_capacity,
        logical_positions=pos, global_token_indices=pos.clone(),
        page_offsets=torch.arange(n) * page, page_lengths=torch.full((n,), page), page_classes=classes,
    )


def snapshot(cache, prefix: str, out: dict, ring: bool = True, full: bool = True) -> None:
    if not full:
        tmp: dict = {}
        snapshot(cache, "", tmp, ring=True, full=True)
        for name, array in tmp.items():
            if array.ndim == 0 or array.size <= 8:
                out[prefix + name] = array
            else:
                out[prefix + name + "_digest"] = np.asarray(digest(array))
        return
    ck, cv = cache.compact_key, cache.compact_value
    out[prefix + "k_packed"] = bits(ck.packed)
    out[prefix + "k_scale"] = bits(ck.scale)
    out[prefix + "k_zero"] = bits(ck.zero_point)
    out[prefix + "k_active"] = np.int64(ck.active_length)
    out[prefix + "k_offsets"] = np.asarray(ck.segment_offsets, dtype=np.int64)
    n2 = cv.active_length
    out[prefix + "i2_packed"] = bits(cv.packed[:, :n2])
    out[prefix + "i2_scale"] = bits(cv.scale[:, :n2])
    out[prefix + "i2_zero"] = bits(cv.zero_point[:, :n2])
    out[prefix + "i2_active"] = np.int64(n2)
    out[prefix + "i2_capacity"] = np.int64(cv.capacity)
    p4 = cache.int4_pool.packed_v
    n4 = cache.int4_pool.token_count
    h = ck.packed.shape[0]
    if n4:
        out[prefix + "i4_packed"] = bits(p4.packed.reshape(h, n4, 64))
        out[prefix + "i4_scale"] = bits(p4.scale)
    out[prefix + "fp_v"] = bits(cache.fp_pool.fp_v) if cache.fp_pool.token_count else np.zeros((h, 0, 128), np.int16)
    r = cache.recent_fp_pool
    if ring:
        out[prefix + "recent_k"] = bits(r.fp_k)
        out[prefix + "recent_v"] = bits(r.fp_v)
    out[prefix + "recent_len"] = np.int64(r.active_length)
    out[prefix + "recent_len_device"] = np.int64(int(r.length_device))
    out[prefix + "recent_global"] = bits(r.global_index_buffer)
    out[prefix + "recent_logical"] = bits(r.logical_position_buffer)
    out[prefix + "recent_page_lengths"] = bits(r.page_index.lengths)
    out[prefix + "i2_global"] = bits(cache.int2_pool.page_index.global_token_indices[: cache.int2_pool.token_count])
    out[prefix + "i2_logical"] = bits(cache.int2_pool.page_index.logical_positions[: cache.int2_pool.token_count])
    out[prefix + "fp_global"] = bits(cache.fp_pool.page_index.global_token_indices)
    out[prefix + "i4_global"] = bits(cache.int4_pool.page_index.global_token_indices[:n4])
    out[prefix + "evicted_global"] = bits(cache.evicted_global_indices)


def case(name, *, hq, hkv, page, classes, recent_capacity, appends, seed, k_block=32, group=32,
         append_capacity=None, dtype=torch.bfloat16, outliers=True, snapshots=()):
    classes = torch.as_tensor(classes, dtype=torch.long)
    s = int(classes.numel()) * page
    key, value, new_k, new_v, queries = make_inputs(
        seed=seed, hq=hq, hkv=hkv, tokens=s, appends=appends, n_queries=len(snapshots) + 2,
        dtype=dtype, outliers=outliers)

    cache = build_three_precision_cache(
        key, value, make_plan(classes, page, recent_capacity), page_size=page,
        key_quantization_superblock=k_block, int2_group_size=group,
        compact_key_append_capacity=append_capacity, recent_flush_size=128,
    )
    out = {
        "hq": np.int64(hq), "hkv": np.int64(hkv), "page": np.int64(page), "classes": classes.numpy(),
        "recent_capacity": np.int64(recent_capacity), "k_block": np.int64(k_block), "group": np.int64(group),
        "append_capacity": np.int64(-1 if append_capacity is None else append_capacity),
        "is_bf16": np.int64(dtype == torch.bfloat16),
        "seed": np.int64(seed), "appends": np.int64(appends), "outliers": np.int64(outliers),
        "input_digest": np.asarray(digest(key, value, new_k, new_v, queries)),
        "snapshots": np.asarray(list(snapshots) + [appends], dtype=np.int64),
    }
    snapshot(cache, "s0_", out, ring=False)
    has_tokens = cache.survivor_count > 0
    if has_tokens:
        out["s0_out"] = triton_mixed_reference(queries[0].float(), cache).numpy()
        out["s0_out_lowp"] = bits(triton_mixed_reference(queries[0], cache))
        out["s0_out_hadamard"] = bits(normalized_fwht(triton_mixed_reference(queries[0], cache)).to(dtype))
    stats = DynamicCacheStats()
    flush_steps, tails = [], []
    marks = list(snapshots) + [appends]
    for i in range(appends):
        before = stats.local_tail_dequant_tokens
        if append_generated_token(cache, new_k[i].unsqueeze(1), new_v[i].unsqueeze(1),
                                  global_token_index=s + i, logical_position=s + i, stats=stats):
            flush_steps.append(i)
            tails.append(stats.local_tail_dequant_tokens - before)
        if i + 1 in marks:
            j = marks.index(i + 1) + 1
            snapshot(cache, f"s{j}_", out, full=(i + 1 == appends))
            out[f"s{j}_out"] = triton_mixed_reference(queries[j].float(), cache).numpy()
            out[f"s{j}_out_lowp"] = bits(triton_mixed_reference(queries[j], cache))
    out["flush_steps"] = np.asarray(flush_steps, dtype=np.int64)
    out["flush_tails"] = np.asarray(tails, dtype=np.int64)
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **out)
    print(name, "S", s, "pools", cache.fp_pool.token_count, cache.int4_pool.token_count, cache.int2_pool.token_count,
          "flushes", flush_steps, "tails", tails, "bytes", os.path.getsize(path))


def seeded_classes(n, seed, p_fp=0.25, p_i4=0.5):
    r = torch.rand(n, generator=torch.Generator().manual_seed(seed))
    return [1 if x < p_fp else 2 if x < p_fp + p_i4 else 5 for x in r.tolist()]


if __name__ == "__main__":
    torch.set_num_threads(4)
    # every tier plus an evicted page, page 32, one flush
    case("tiers_page32", hq=16, hkv=2, page=32, classes=[1, 2, 5, 0, 2, 5, 1, 2], recent_capacity=128,
         appends=130, seed=11, snapshots=(5, 128))
    # the benchmark's mix at page 64, two flushes
    case("mixed_page64", hq=16, hkv=2, page=64, classes=seeded_classes(12, 5), recent_capacity=128,
         appends=258, seed=12, append_capacity=384, snapshots=(127, 129))
    # page 16: pool origins are not multiples of the key block, and each flush re-quantises a 16-token tail
    case("page16_tail", hq=16, hkv=2, page=16, classes=[1, 2, 2, 5, 5, 5, 1, 2, 5], recent_capacity=128,
         appends=257, seed=13, append_capacity=256, snapshots=(129,))
    # 7B head shape (GQA 7), fp16 inputs, no outliers
    case("gqa7_fp16", hq=28, hkv=4, page=64, classes=seeded_classes(6, 9), recent_capacity=128,
         appends=129, seed=14, dtype=torch.float16, outliers=False)
    # wider calibration blocks; residual window larger than one flush
    case("kblock64_group64", hq=16, hkv=2, page=32, classes=[2, 5, 1, 5, 2, 2], recent_capacity=256,
         appends=300, seed=15, k_block=64, group=64, append_capacity=512, snapshots=(256, 257))
    # a cache with a single tier and nothing else (INT4 only: the reference's own CPU-runnable configuration)
    case("int4_only", hq=16, hkv=2, page=32, classes=[2] * 8, recent_capacity=128, appends=128, seed=16)
