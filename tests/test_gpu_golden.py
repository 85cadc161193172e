"""CUDA path against the fixtures produced by the reference itself: packing and
indexing bit-exact, attention within max-abs 2e-3 / rel 1e-2.  Calls go through
the C ABI (ctypes) of libr2k_b200.so."""
import numpy as np
import pytest
import torch

import r2omni_b200 as R
from golden_cases import CASES, GoldenCase, compare_snapshot
from gpu_helpers import GRID_CAPS, apply_grid_cap, assert_close, build_gpu_cache, image, make_executor

pytestmark = pytest.mark.gpu


def _kwargs(case):
    return dict(page_size=case.page, recent_capacity=case.recent_capacity, k_block=case.k_block, v2_group=case.group,
                append_capacity=case.append_capacity)


@pytest.mark.parametrize("name", CASES)
@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("grid_cap", GRID_CAPS)
def test_fixture_pack_append_flush_and_decode(name, fused, grid_cap, monkeypatch):
    case = GoldenCase(name)
    apply_grid_cap(monkeypatch, grid_cap, case.hkv)
    cache = build_gpu_cache(case.key, case.value, case.classes, **_kwargs(case))
    compare_snapshot(case, "s0_", image(cache, "s0_"), skip=("recent_k", "recent_v"))
    ex = make_executor(cache, case.hq)
    if case.has("s0_out"):
        q = case.queries[0].cuda()
        assert_close(ex.decode_f32(q), torch.from_numpy(case.z["s0_out"]), f"{name} s0 f32")
        want = torch.from_numpy(case.z["s0_out_lowp"]).view(case.dtype)
        assert_close(ex(q), want, f"{name} s0 lowp")
    stats = R.DynamicCacheStats()
    s = int(case.classes.numel()) * case.page
    new_k, new_v = case.new_k.cuda(), case.new_v.cuda()
    flushes = []
    dummy_q = case.queries[0].cuda()
    for i in range(case.appends):
        ring = cache.recent_fp_pool
        if fused and ring.active_length < ring.capacity:
            # the decode launch itself appends the token (SplitKExecutor append=...)
            ex(dummy_q, append=(new_k[i].unsqueeze(0).contiguous(), new_v[i].unsqueeze(0).contiguous(), s + i, s + i))
            ring.active_length += 1
            stats.appended_tokens += 1
        elif R.append_generated_token(cache, new_k[i].unsqueeze(1), new_v[i].unsqueeze(1), global_token_index=s + i,
                                      logical_position=s + i, stats=stats):
            flushes.append(i)
        if i + 1 in case.marks:
            j = case.marks.index(i + 1) + 1
            compare_snapshot(case, f"s{j}_", image(cache, f"s{j}_"))
            assert int(cache.arenas.recent_len_device[0]) == int(case.z[f"s{j}_recent_len_device"])
            q = case.queries[j].cuda()
            assert_close(ex.decode_f32(q), torch.from_numpy(case.z[f"s{j}_out"]), f"{name} s{j} f32")
    assert flushes == [int(v) for v in case.z["flush_steps"]]
    assert stats.appended_tokens == case.appends
    assert stats.local_tail_dequant_tokens == int(np.sum(case.z["flush_tails"]))
    assert ex.device_status() == 0


def test_hadamard_epilogue_matches_reference_fixture():
    case = GoldenCase("tiers_page32")
    cache = build_gpu_cache(case.key, case.value, case.classes, **_kwargs(case))
    ex = make_executor(cache, case.hq, output_hadamard=True)
    want = torch.from_numpy(case.z["s0_out_hadamard"]).view(case.dtype)
    got = ex(case.queries[0].cuda())
    # one bf16 ulp of slack on top of the attention tolerance: the transform runs after a bf16 rounding
    assert_close(got, want, "hadamard")


def test_capacity_exhaustion_raises_runtime_error():
    case = GoldenCase("tiers_page32")
    cache = build_gpu_cache(case.key, case.value, case.classes, **_kwargs(case))
    stats = R.DynamicCacheStats()
    k, v = case.new_k.cuda(), case.new_v.cuda()
    with pytest.raises(RuntimeError):
        for i in range(300):
            R.append_generated_token(cache, k[i % case.appends].unsqueeze(1), v[i % case.appends].unsqueeze(1),
                                     global_token_index=i, logical_position=i, stats=stats)
