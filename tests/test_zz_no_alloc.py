"""The allocation-free decode entry point (r2k_decode_static).

Some callers may not allocate device memory at all: a plugin that a host runtime hands nothing but its
input and output buffers, or a latency path that must stay away from the allocator.  For them the
library keeps the split-K scratch in a static device array and exposes r2k_decode_static, which takes
no workspace.  This test calls it through the C ABI twice in a row on the same stream (the second call
finds the first call's leftovers in the shared array) and checks both results against r2k_decode with a
caller-provided workspace, within the attention tolerance of the other GPU tests (max-abs 2e-3 + rel 1e-2;
in practice the two are the same kernel and agree bit for bit).  It also checks that an oversized
geometry is refused, that two geometries can take turns on the array, and the status / reset calls.  The file sorts last so that a failure here cannot hide another test's result.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _static_decode(ex, query, append=None, flags=0):
    """r2k_decode_static through ctypes: inputs and outputs from the caller, no workspace argument."""
    from r2omni_b200 import _lib as L
    from r2omni_b200.sspa.cache import _stream_ptr
    a = ex.arenas
    out = torch.empty((a.batch, ex.num_query_heads, 128), device=query.device, dtype=torch.float32)
    geom = a.geom(ex.num_query_heads)
    ap = ex._make_append(append, query)
    status = L.lib().r2k_decode_static(C.byref(geom), C.byref(a.view()), C.c_void_p(query.data_ptr()), ap,
                                       C.c_void_p(out.data_ptr()), C.c_uint32(flags | L.FLAG_OUT_F32),
                                       C.c_void_p(_stream_ptr(a.device)))
    return status, out


def test_static_scratch_decode_matches_workspace_decode_twice_in_a_row():
    import r2omni_b200 as R
    from r2omni_b200 import _lib as L
    from gpu_helpers import assert_close, build_gpu_cache, make_executor
    from recipe import make_inputs

    torch.manual_seed(0)
    r = torch.rand(48, generator=torch.Generator().manual_seed(9))
    classes = torch.where(r < 0.25, 1, torch.where(r < 0.75, 2, 5))
    key, value, new_k, new_v, queries = make_inputs(seed=70, hq=16, hkv=2, tokens=48 * 64, appends=2, n_queries=2)
    cache = build_gpu_cache(key, value, classes, page_size=64)
    ex = make_executor(cache, 16)
    for i in range(2):
        q = queries[i].cuda()
        want = ex.decode_f32(q).clone()                  # existing entry point, caller-provided workspace
        status, got = _static_decode(ex, q)              # new entry point, library-owned static scratch
        assert status == L.OK, L.lib().r2k_status_string(status)
        torch.cuda.synchronize()
        assert_close(got, want, f"static-scratch decode, call {i}")
        assert torch.equal(got, want), "same kernel, same order of operations: expected identical bits"
    # with a fused append as well: the ring row, length and indices must end up as with the workspace variant
    twin = build_gpu_cache(key, value, classes, page_size=64)
    ex2 = make_executor(twin, 16)
    k, v = new_k[0].unsqueeze(0).contiguous().cuda(), new_v[0].unsqueeze(0).contiguous().cuda()
    want = ex.decode_f32(queries[0].cuda(), append=(k, v, 7, 7))
    status, got = _static_decode(ex2, queries[0].cuda(), append=(k, v, 7, 7))
    assert status == L.OK
    assert_close(got, want, "static-scratch decode with append")
    assert int(twin.arenas.recent_len_device[0]) == int(cache.arenas.recent_len_device[0]) == 1
    assert torch.equal(twin.arenas.recent_k[0, :, 0], cache.arenas.recent_k[0, :, 0])


def test_static_scratch_decode_rejects_oversized_geometry():
    from r2omni_b200 import _lib as L
    g = L.Geom()
    g.batch, g.num_q_heads, g.num_kv_heads, g.head_dim = 256, 64, 8, 128    # 2048 (request, head) pairs of partial slots
    g.page_size, g.k_block, g.v2_group = 64, 32, 32
    g.n_i4 = g.i4_capacity = g.k_off_i2 = 4096
    g.k_capacity, g.recent_capacity = 4096 + 128, 128
    need = C.c_size_t(0)
    assert L.lib().r2k_decode_workspace_bytes(C.byref(g), C.byref(need)) == L.OK
    assert need.value > (4 << 20)
    dummy = torch.zeros(16, device="cuda")
    view = L.CacheView()
    status = L.lib().r2k_decode_static(C.byref(g), C.byref(view), C.c_void_p(dummy.data_ptr()), None,
                                       C.c_void_p(dummy.data_ptr()), C.c_uint32(0), None)
    assert status == L.ERR_WORKSPACE


def test_static_scratch_serves_alternating_geometries_and_reports_its_status():
    """Two geometries whose counters and partial slots would sit at different offsets take turns on the one static
    array (one request with 2 kv heads, then a stacked batch of 8 requests with 8 kv heads): every result must
    equal the workspace variant's.  The status word of the static scratch is readable and clearable without the
    caller ever seeing its address."""
    import r2omni_b200 as R
    from r2omni_b200 import _lib as L
    from r2omni_b200.sspa.cache import _stream_ptr
    from gpu_helpers import build_gpu_cache, make_executor
    from recipe import make_inputs

    classes = torch.tensor([2, 5, 1, 2, 5, 2, 1, 5])
    key, value, _, _, queries = make_inputs(seed=71, hq=16, hkv=2, tokens=512, appends=1, n_queries=2)
    small = make_executor(build_gpu_cache(key, value, classes, page_size=64), 16)
    singles = []
    for b in range(8):
        k8, v8, _, _, q8 = make_inputs(seed=72 + b, hq=16, hkv=8, tokens=512, appends=1, n_queries=2)
        singles.append(make_executor(build_gpu_cache(k8, v8, classes, page_size=64), 16))
    wide = R.stack_homogeneous_splitk_executors(singles)
    q_wide = torch.randn(2, 8, 16, 128, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda()
    stream = C.c_void_p(_stream_ptr(small.arenas.device))
    assert L.lib().r2k_decode_static_reset(stream) == L.OK
    for turn in range(2):
        for ex, q in ((small, queries[turn].cuda()), (wide, q_wide[turn])):
            want = ex.decode_f32(q).clone()
            status, got = _static_decode(ex, q)
            assert status == L.OK, L.lib().r2k_status_string(status)
            torch.cuda.synchronize()
            assert torch.equal(got, want), f"turn {turn}, batch {ex.arenas.batch}"
    word = C.c_int32(-1)
    assert L.lib().r2k_decode_static_status(C.byref(word), stream) == L.OK and word.value == 0
    assert L.lib().r2k_decode_static_reset(stream) == L.OK
    status, got = _static_decode(small, queries[0].cuda())
    torch.cuda.synchronize()
    assert status == L.OK and torch.equal(got, small.decode_f32(queries[0].cuda()))
