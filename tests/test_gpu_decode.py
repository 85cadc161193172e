"""CUDA decode / append / flush against the CPU oracle on seeded inputs at sizes
the oracle finishes in seconds, plus the error behaviour of the operator API."""
import ctypes as C

import pytest
import torch

import r2omni_b200 as R
from r2omni_b200 import _lib as L
from gpu_helpers import GRID_CAPS, apply_grid_cap, assert_close, build_gpu_cache, image, make_executor
from oracle import sspa_oracle as O
from recipe import make_inputs

pytestmark = pytest.mark.gpu


def seeded_classes(n, seed, p_fp=0.25, p_i4=0.5):
    r = torch.rand(n, generator=torch.Generator().manual_seed(seed))
    return torch.tensor([1 if x < p_fp else 2 if x < p_fp + p_i4 else 5 for x in r.tolist()])


def both_caches(seed, *, hq, hkv, tokens, page, classes, appends, dtype=torch.bfloat16, n_queries=2, **kw):
    key, value, new_k, new_v, queries = make_inputs(seed=seed, hq=hq, hkv=hkv, tokens=tokens, appends=appends,
                                                    n_queries=n_queries, dtype=dtype)
    ocache = O.build_cache(key, value, classes, page_size=page, **kw)
    gcache = build_gpu_cache(key, value, classes, page_size=page, **kw)
    return ocache, gcache, new_k, new_v, queries


def arena_equal(ocache, gcache):
    a, r = gcache.arenas, gcache._r
    n2 = ocache.i2_active
    pairs = [(ocache.k_packed, a.k_packed[r]), (ocache.k_scale, a.k_scale[r]), (ocache.k_zero, a.k_zero[r]),
             (ocache.fp_v, a.fp_v[r]), (ocache.i4_packed, a.i4_packed[r]), (ocache.i4_scale, a.i4_scale[r]),
             (ocache.i2_packed[:, :n2], a.i2_packed[r][:, :n2]), (ocache.i2_scale[:, :n2], a.i2_scale[r][:, :n2]),
             (ocache.i2_zero[:, :n2], a.i2_zero[r][:, :n2]),
             (ocache.recent_k[:, : ocache.recent_len], a.recent_k[r][:, : ocache.recent_len]),
             (ocache.recent_v[:, : ocache.recent_len], a.recent_v[r][:, : ocache.recent_len])]
    assert (ocache.k_active, ocache.i2_active, ocache.recent_len) == (a.k_active, a.i2_active, a.recent_len)
    for i, (want, got) in enumerate(pairs):
        got = got.cpu()
        if want.dtype in (torch.bfloat16, torch.float16):
            want, got = want.view(torch.int16), got.view(torch.int16)
        assert torch.equal(want, got), f"arena tensor {i} differs in {(want != got).sum().item()} elements"


def test_int4_only_4096_tokens_with_full_residual_window():
    """The reference's CPU-runnable configuration: B1, 16/2 heads, 4096 INT4-value tokens (page 32) + 128 residual."""
    classes = torch.full((128,), 2)
    ocache, gcache, new_k, new_v, queries = both_caches(21, hq=16, hkv=2, tokens=4096, page=32, classes=classes, appends=129)
    stats = R.DynamicCacheStats()
    k, v = new_k.cuda(), new_v.cuda()
    for i in range(128):
        O.append_token(ocache, new_k[i], new_v[i], 4096 + i, 4096 + i)
        R.append_generated_token(gcache, k[i].unsqueeze(1), v[i].unsqueeze(1), global_token_index=4096 + i,
                                 logical_position=4096 + i, stats=stats)
    arena_equal(ocache, gcache)
    ex = make_executor(gcache, 16)
    q = queries[0]
    assert_close(ex.decode_f32(q.cuda()), O.decode_fp32(q.float(), ocache), "int4-only f32")
    assert_close(ex(q.cuda()), O.decode(q, ocache), "int4-only bf16")
    # ring is full: a fused append must be refused, the flush path must take over
    with pytest.raises(RuntimeError):
        ex(q.cuda(), append=(k[128].unsqueeze(0).contiguous(), v[128].unsqueeze(0).contiguous(), 0, 0))
    assert O.append_token(ocache, new_k[128], new_v[128], 4224, 4224)
    assert R.append_generated_token(gcache, k[128].unsqueeze(1), v[128].unsqueeze(1), global_token_index=4224,
                                    logical_position=4224, stats=stats)
    arena_equal(ocache, gcache)
    assert_close(ex.decode_f32(queries[1].cuda()), O.decode_fp32(queries[1].float(), ocache), "after flush")
    assert ex.device_status() == 0


@pytest.mark.parametrize("hq,hkv", [(16, 2), (28, 4)])
@pytest.mark.parametrize("grid_cap", GRID_CAPS)
def test_mixed_pools_fused_append_every_step(hq, hkv, grid_cap, monkeypatch):
    """Mixed bf16/INT4/INT2 pages (25/50/25), one fused append per decode step across a flush; with a grid limit
    a CTA streams up to 30 tiles of three pools through the shared-memory ring and carries its softmax state across."""
    apply_grid_cap(monkeypatch, grid_cap, hkv)
    classes = seeded_classes(96, 3)
    ocache, gcache, new_k, new_v, queries = both_caches(22 + hq, hq=hq, hkv=hkv, tokens=96 * 64, page=64, classes=classes,
                                                        appends=140, n_queries=140, append_capacity=256)
    ex = make_executor(gcache, hq)
    stats = R.DynamicCacheStats()
    k, v = new_k.cuda(), new_v.cuda()
    s = 96 * 64
    for i in range(140):
        ring = gcache.recent_fp_pool
        q = queries[i]
        if ring.active_length == ring.capacity:
            assert R.append_generated_token(gcache, k[i].unsqueeze(1), v[i].unsqueeze(1), global_token_index=s + i,
                                            logical_position=s + i, stats=stats)
            out = ex.decode_f32(q.cuda())
        else:
            out = ex.decode_f32(q.cuda(), append=(k[i].unsqueeze(0).contiguous(), v[i].unsqueeze(0).contiguous(), s + i, s + i))
            ring.active_length += 1
        O.append_token(ocache, new_k[i], new_v[i], s + i, s + i)
        if i % 23 == 0 or i in (127, 128, 129, 139):
            assert_close(out, O.decode_fp32(q.float(), ocache), f"step {i}")
    arena_equal(ocache, gcache)
    assert torch.equal(gcache.arenas.recent_global[0].cpu()[: ocache.recent_len], ocache.recent_global[: ocache.recent_len])
    assert torch.equal(gcache.arenas.recent_page_lengths[0].cpu(), ocache.recent_page_lengths)
    assert int(gcache.arenas.recent_len_device[0]) == ocache.recent_len
    assert ex.device_status() == 0


@pytest.mark.parametrize("hq,hkv", [(3, 3), (4, 2), (3, 1), (8, 2), (5, 1), (12, 2), (7, 1), (8, 1)])
def test_every_group_width(hq, hkv):
    """Query heads per kv head from 1 (no grouping) to 8, a single kv head included: the MMA's eight head columns
    are padded for narrower groups and the padding must reach neither the output nor the appended rows.  Mixed pages,
    fused appends, the Hadamard epilogue and the state output."""
    classes = seeded_classes(24, 60 + hq)
    s = 24 * 64
    ocache, gcache, new_k, new_v, queries = both_caches(70 + 8 * hq + hkv, hq=hq, hkv=hkv, tokens=s, page=64, classes=classes,
                                                        appends=6, n_queries=8, append_capacity=256)
    ex = make_executor(gcache, hq)
    exh = make_executor(gcache, hq, output_hadamard=True)
    k, v = new_k.cuda(), new_v.cuda()
    for i in range(6):
        q = queries[i]
        out = ex.decode_f32(q.cuda(), append=(k[i].unsqueeze(0).contiguous(), v[i].unsqueeze(0).contiguous(), s + i, s + i))
        gcache.recent_fp_pool.active_length += 1
        O.append_token(ocache, new_k[i], new_v[i], s + i, s + i)
        assert_close(out, O.decode_fp32(q.float(), ocache), f"group of {hq // hkv}, step {i}")
    arena_equal(ocache, gcache)
    q = queries[6]
    got = ex(q.cuda())
    assert got.shape == (1, hq, 128) and got.dtype == torch.bfloat16
    assert_close(got, O.decode(q, ocache), "element-type output")
    # the epilogue rotates the rounded output: checked against the oracle's transform of this very output, so that
    # the attention tolerance (which a rounding before a 128-term sum amplifies) stays out of it; one ulp of slack
    rotated = O.fwht128(got.float().cpu()).to(torch.bfloat16).float()
    assert ((exh(q.cuda()).float().cpu() - rotated).abs() <= 2.0 ** -7 * rotated.abs() + 1e-6).all()
    top, den, acc = O.decode_state(queries[7].float(), ocache)
    st = ex.decode_state(queries[7].cuda()).cpu()
    assert st.shape == (1, hq, 130)
    assert torch.allclose(st[..., 0] + torch.log(st[..., 1]), top + torch.log(den), atol=2e-3)
    assert_close(st[..., 2:] / st[..., 1:2], acc / den.unsqueeze(-1), "state output")
    assert ex.device_status() == 0


@pytest.mark.parametrize("grid_cap", (None, "heads", "3"))
def test_stacked_batch_matches_per_request_oracle(grid_cap, monkeypatch):
    """Homogeneous batch (B=3): stacked arenas, per-request oracle; fused append and a batched flush."""
    apply_grid_cap(monkeypatch, grid_cap, 6)
    classes = seeded_classes(40, 8)
    hq, hkv, s = 16, 2, 40 * 64
    oc, ex1, ks, vs, qs = [], [], [], [], []
    for b in range(3):
        o, g, nk, nv, q = both_caches(40 + b, hq=hq, hkv=hkv, tokens=s, page=64, classes=classes, appends=130,
                                      n_queries=3, append_capacity=256)
        oc.append(o); ex1.append(make_executor(g, hq)); ks.append(nk); vs.append(nv); qs.append(q)
    ex = R.stack_homogeneous_splitk_executors(ex1)
    new_k = torch.stack(ks, 1).cuda()   # [appends, B, Hkv, 128]
    new_v = torch.stack(vs, 1).cuda()
    stats = R.DynamicCacheStats()

    def check(qi, tag, append=None):
        q = torch.cat([qs[b][qi] for b in range(3)], 0)
        out = ex.decode_f32(q.cuda(), append=append)
        for b in range(3):
            assert_close(out[b : b + 1], O.decode_fp32(qs[b][qi].float(), oc[b]), f"{tag} request {b}")

    check(0, "static")
    for i in range(130):
        for b in range(3):
            O.append_token(oc[b], ks[b][i], vs[b][i], s + i, s + i)
        if i == 64:   # one step through the fused path
            check(1, "fused", append=(new_k[i].contiguous(), new_v[i].contiguous(), s + i, s + i))
        else:
            R.append_generated_token(ex.arenas, new_k[i].contiguous(), new_v[i].contiguous(), global_token_index=s + i,
                                     logical_position=s + i, stats=stats)
    assert stats.flushed_tokens == 128 and ex.arenas.recent_len == 2
    check(2, "after batched flush")
    for b in range(3):
        arena_equal(oc[b], R.ThreePrecisionCache(ex.arenas, b))
    assert ex.device_status() == 0


def test_fp16_cache_and_wide_blocks():
    classes = torch.tensor([2, 5, 1, 5, 2, 2, 1, 5])
    ocache, gcache, new_k, new_v, queries = both_caches(31, hq=16, hkv=2, tokens=8 * 32, page=32, classes=classes, appends=40,
                                                        dtype=torch.float16, k_block=64, v2_group=128, append_capacity=256)
    ex = make_executor(gcache, 16)
    k, v = new_k.cuda(), new_v.cuda()
    for i in range(40):
        O.append_token(ocache, new_k[i], new_v[i], i, i)
        ex(queries[0].cuda(), append=(k[i].unsqueeze(0).contiguous(), v[i].unsqueeze(0).contiguous(), i, i))
        gcache.recent_fp_pool.active_length += 1
    arena_equal(ocache, gcache)
    assert_close(ex.decode_f32(queries[1].cuda()), O.decode_fp32(queries[1].float(), ocache), "fp16 f32")
    assert ex(queries[1].cuda()).dtype == torch.bfloat16


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("k_block,v2_group", [(32, 32), (32, 64), (64, 32), (64, 64), (128, 32), (128, 128), (32, 128)])
def test_block_and_group_sizes_through_a_flush(k_block, v2_group, dtype):
    """Key calibration blocks of 32 / 64 / 128 tokens and INT2 groups of 32 / 64 / 128 channels, both element types:
    a history that does not end on a key block (the flush re-quantises the tail block), 130 appends through one
    flush, arenas bit for bit, decode within tolerance before and after."""
    classes = torch.tensor([2, 1, 5, 2, 5, 1, 2])
    s = 7 * 32
    ocache, gcache, new_k, new_v, queries = both_caches(90 + k_block + v2_group, hq=16, hkv=2, tokens=s, page=32, classes=classes,
                                                        appends=130, n_queries=3, dtype=dtype, k_block=k_block,
                                                        v2_group=v2_group, append_capacity=256)
    ex = make_executor(gcache, 16)
    stats = R.DynamicCacheStats()
    k, v = new_k.cuda(), new_v.cuda()

    def check(qi, what):
        # 350 tokens of seeded noise make peaked attention: single INT4-value tokens carry most of a head's weight.
        # The reference's CPU decoder rounds code * scale of INT4 values to the element type, its GPU kernel and
        # this one do not; with weights like these that rounding alone moves the CPU result by more than the
        # tolerance.  So: within tolerance of the unrounded form, and of the rounded form once its own shift is allowed.
        q = queries[qi]
        got = ex.decode_f32(q.cuda())
        plain = O.decode_fp32(q.float(), ocache, round_int4_values=False)
        assert_close(got, plain, what)
        rounded = O.decode_fp32(q.float(), ocache)
        slack = (rounded - plain).abs()
        assert ((got.cpu() - rounded).abs() <= 2e-3 + 1e-2 * rounded.abs() + slack).all(), what

    check(0, "before the appends")
    flushed = 0
    for i in range(130):
        O.append_token(ocache, new_k[i], new_v[i], s + i, s + i)
        flushed += bool(R.append_generated_token(gcache, k[i].unsqueeze(1), v[i].unsqueeze(1), global_token_index=s + i,
                                                 logical_position=s + i, stats=stats))
        if i == 126:
            check(1, "full window")
    assert flushed == 1
    arena_equal(ocache, gcache)
    check(2, "after the flush")
    assert ex.device_status() == 0


@pytest.mark.parametrize("p_fp,p_i4", [(0.25, 0.5), (0.0, 1.0), (0.0, 0.0), (1.0, 0.0)])
def test_peaked_attention(p_fp, p_i4):
    """Queries three times as long as usual: a few tokens take most of every head's weight, so nothing averages
    out and every rounding of a probability or a value shows.  Mixed pages and each value format alone, six seeds."""
    for seed in range(6):
        classes = seeded_classes(32, 200 + seed, p_fp=p_fp, p_i4=p_i4)
        ocache, gcache, new_k, new_v, queries = both_caches(300 + seed, hq=16, hkv=2, tokens=32 * 64, page=64, classes=classes,
                                                            appends=3, n_queries=1)
        for i in range(3):
            O.append_token(ocache, new_k[i], new_v[i], 2048 + i, 2048 + i)
            R.append_generated_token(gcache, new_k[i].cuda().unsqueeze(1), new_v[i].cuda().unsqueeze(1),
                                     global_token_index=2048 + i, logical_position=2048 + i, stats=R.DynamicCacheStats())
        q = (queries[0].float() * 3.0).to(torch.bfloat16)
        got = make_executor(gcache, 16).decode_f32(q.cuda())
        plain = O.decode_fp32(q.float(), ocache, round_int4_values=False)
        assert_close(got, plain, f"seed {seed}")
        # the CPU decoder's rounding of INT4 values moves its own result by `slack` (see the test above)
        rounded = O.decode_fp32(q.float(), ocache)
        slack = (rounded - plain).abs()
        assert ((got.cpu() - rounded).abs() <= 2e-3 + 1e-2 * rounded.abs() + slack).all(), f"seed {seed}, rounded form"


def test_explicit_softmax_scale_and_four_dimensional_query():
    """A softmax scale other than 128 ** -0.5 (the executor's constructor takes one), and the query given as
    [B, Hq, 1, 128], the form the attention manager hands over."""
    classes = seeded_classes(16, 77)
    ocache, gcache, new_k, new_v, queries = both_caches(78, hq=16, hkv=2, tokens=16 * 64, page=64, classes=classes, appends=2)
    for i in range(2):
        O.append_token(ocache, new_k[i], new_v[i], 1024 + i, 1024 + i)
        R.append_generated_token(gcache, new_k[i].cuda().unsqueeze(1), new_v[i].cuda().unsqueeze(1),
                                 global_token_index=1024 + i, logical_position=1024 + i, stats=R.DynamicCacheStats())
    ws = R.allocate_splitk_workspace(gcache, num_query_heads=16)
    q = queries[0]
    for scale in (0.03, 0.2):
        ex = R.SplitKExecutor(gcache.arenas, ws, cache=gcache, sm_scale=scale)
        assert_close(ex.decode_f32(q.cuda()), O.decode_fp32(q.float(), ocache, sm_scale=scale), f"scale {scale}")
    ex = make_executor(gcache, 16)
    flat = ex(q.cuda()).clone()
    assert torch.equal(ex(q.cuda().unsqueeze(2)), flat)
    assert_close(flat, O.decode(q, ocache), "default scale")


def test_only_residual_window_and_only_history():
    classes = torch.tensor([0, 0])       # every page evicted: attention over the residual window alone
    ocache, gcache, new_k, new_v, queries = both_caches(33, hq=16, hkv=2, tokens=64, page=32, classes=classes, appends=5)
    ex = make_executor(gcache, 16)
    with pytest.raises(ValueError):
        ex(queries[0].cuda())           # no surviving token at all
    k, v = new_k.cuda(), new_v.cuda()
    for i in range(5):
        O.append_token(ocache, new_k[i], new_v[i], i, i)
        out = ex.decode_f32(queries[0].cuda(), append=(k[i].unsqueeze(0).contiguous(), v[i].unsqueeze(0).contiguous(), i, i))
        gcache.recent_fp_pool.active_length += 1
        assert_close(out, O.decode_fp32(queries[0].float(), ocache), f"residual only, {i + 1} tokens")
    classes = torch.tensor([5, 1, 2])    # history only, empty residual window, ragged tile tails
    ocache, gcache, _, _, queries = both_caches(34, hq=16, hkv=2, tokens=48, page=16, classes=classes, appends=1)
    ex = make_executor(gcache, 16)
    assert_close(ex.decode_f32(queries[0].cuda()), O.decode_fp32(queries[0].float(), ocache), "history only")


def test_sharded_states_merge_to_the_single_cache_result():
    """Two contiguous sequence shards -> per-shard un-normalised states -> r2k_merge_states."""
    classes = seeded_classes(32, 5, p_fp=0.0, p_i4=0.5)
    key, value, new_k, new_v, queries = make_inputs(seed=50, hq=16, hkv=2, tokens=32 * 64, appends=3, n_queries=1)
    whole = O.build_cache(key, value, classes, page_size=64)
    for i in range(3):
        O.append_token(whole, new_k[i], new_v[i], i, i)
    states = []
    for r in range(2):
        sl = slice(r * 1024, (r + 1) * 1024)
        g = build_gpu_cache(key[:, sl].contiguous(), value[:, sl].contiguous(), classes[r * 16 : (r + 1) * 16], page_size=64)
        if r == 1:   # the residual window lives on the last shard
            st = R.DynamicCacheStats()
            for i in range(3):
                R.append_generated_token(g, new_k[i].cuda().unsqueeze(1), new_v[i].cuda().unsqueeze(1),
                                         global_token_index=i, logical_position=i, stats=st)
        states.append(make_executor(g, 16).decode_state(queries[0].cuda()))
    stacked = torch.stack(states).contiguous()
    out = torch.empty(1, 16, 128, device="cuda", dtype=torch.float32)
    L.check(L.lib().r2k_merge_states(C.c_void_p(stacked.data_ptr()), 2, C.c_int64(16 * 130), 16, L.DTYPE_BF16,
                                     C.c_void_p(out.data_ptr()), C.c_uint32(L.FLAG_OUT_F32),
                                     C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    assert_close(out, O.decode_fp32(queries[0].float(), whole), "two-shard merge")
    # the per-shard state itself, against the oracle's partial state of the same tokens
    top, den, acc = O.decode_state(queries[0].float(), O.build_cache(key[:, :1024].contiguous(), value[:, :1024].contiguous(),
                                                                      classes[:16], page_size=64))
    s0 = states[0].cpu()
    # the state's reference point need not be the true maximum (it moves lazily); its log-sum-exp is what is defined
    assert torch.allclose(s0[..., 0] + torch.log(s0[..., 1]), top + torch.log(den), atol=2e-3)
    assert_close(s0[..., 2:] / s0[..., 1:2], acc / den.unsqueeze(-1), "shard-0 state")


def test_operator_argument_errors():
    classes = torch.tensor([2, 5])
    _, gcache, new_k, new_v, queries = both_caches(35, hq=16, hkv=2, tokens=64, page=32, classes=classes, appends=1)
    ex = make_executor(gcache, 16)
    q = queries[0].cuda()
    with pytest.raises(ValueError):
        ex(q[:, :8].contiguous())                       # wrong head count
    with pytest.raises(ValueError):
        ex(q.float())                                   # wrong dtype
    with pytest.raises(ValueError):
        ex(q, append=(new_k[0].cuda()[:1], new_v[0].cuda()[:1], 0, 0))   # wrong append shape
    with pytest.raises(ValueError):
        R.prepare_splitk_executor(gcache, ex.workspace, block_n=64)      # workspace/block mismatch
    with pytest.raises(TypeError):
        R.prepare_splitk_executor(object(), ex.workspace)
    with pytest.raises(ValueError):
        R.build_three_precision_cache(queries[0][0].cuda(), queries[0][0].cuda(), None, cache_variant="v_fourq_k_bf16")


def test_host_buffer_step_matches_device_call_and_oracle():
    """r2k_decode_host (SplitKExecutor.step_host): pinned host query / new rows in, host result out, one call per
    step.  Same bits as the device-tensor call on a twin cache, same ring afterwards, oracle parity."""
    classes = seeded_classes(24, 5)
    hq, hkv, s = 16, 2, 24 * 64
    twins = [both_caches(77, hq=hq, hkv=hkv, tokens=s, page=64, classes=classes, appends=6, n_queries=6) for _ in range(2)]
    ocache, new_k, new_v, queries = twins[0][0], twins[0][2], twins[0][3], twins[0][4]
    ex_dev, ex_host = make_executor(twins[0][1], hq), make_executor(twins[1][1], hq)
    host_in = torch.empty(hq * 128 + 2 * hkv * 128, dtype=torch.bfloat16).pin_memory()
    host_out = torch.empty(1, hq, 128, dtype=torch.bfloat16).pin_memory()
    for i in range(6):
        q = queries[i].reshape(1, hq, 128)
        host_in[: hq * 128] = q.flatten()
        host_in[hq * 128 : hq * 128 + hkv * 128] = new_k[i].flatten()
        host_in[hq * 128 + hkv * 128 :] = new_v[i].flatten()
        want = ex_dev(q.cuda(), append=(new_k[i].unsqueeze(0).contiguous().cuda(), new_v[i].unsqueeze(0).contiguous().cuda(),
                                        s + i, s + i)).cpu()
        got = ex_host.step_host(host_in, host_out, append_indices=(s + i, s + i))
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"step {i}"
        O.append_token(ocache, new_k[i], new_v[i], s + i, s + i)
        assert_close(got.float(), O.decode_fp32(q.float(), ocache), f"host step {i}")
    # without an append: the query alone travels
    want = ex_dev(queries[0].reshape(1, hq, 128).cuda()).cpu()
    host_in[: hq * 128] = queries[0].flatten()
    got = ex_host.step_host(host_in, host_out)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    a_dev, a_host = twins[0][1].arenas, twins[1][1].arenas   # the ring after six fused appends: device state of the twins
    for name in ("recent_k", "recent_v", "recent_len_device", "recent_global", "recent_logical", "recent_page_lengths"):
        assert torch.equal(getattr(a_dev, name), getattr(a_host, name)), name
    assert int(a_host.recent_len_device[0]) == ocache.recent_len == 6
    assert torch.equal(a_host.recent_k[0][:, :6].cpu().view(torch.int16), ocache.recent_k[:, :6].view(torch.int16))
    assert torch.equal(a_host.recent_v[0][:, :6].cpu().view(torch.int16), ocache.recent_v[:, :6].view(torch.int16))
    assert ex_host.device_status() == 0
    with pytest.raises(ValueError):
        ex_host.step_host(host_in[: hq * 128], host_out, append_indices=(0, 0))   # rows missing
    with pytest.raises(ValueError):
        ex_host.step_host(host_in.cuda(), host_out)
