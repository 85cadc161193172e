"""Parity at the sizes the benchmark times: every CTA of these launches streams many tiles (the shared-memory ring
is refilled again and again, its barrier phases flip, online-softmax state is carried across whole pools), which the
small cases of the other files never reach.  Inputs, seeds and page mixes are the benchmark's own (bench.py)."""
import pytest
import torch

import r2omni_b200 as R
from bench import K_BLOCK, PAGE, RING, V2_GROUP, page_classes, synth_kv
from gpu_helpers import assert_close, make_executor, make_plan
from oracle import sspa_oracle as O
from test_gpu_decode import arena_equal

pytestmark = pytest.mark.gpu


def _pair(tokens, kv_seed, classes, hkv, device="cuda"):
    """The product cache on the GPU and the oracle cache on the host from the same seeded K/V."""
    key, value = synth_kv(tokens, kv_seed, device, hkv=hkv)
    gcache = R.build_three_precision_cache(key, value, make_plan(classes, PAGE, RING), page_size=PAGE,
                                           key_quantization_superblock=K_BLOCK, int2_group_size=V2_GROUP,
                                           compact_key_append_capacity=RING, recent_flush_size=RING)
    ocache = O.build_cache(key.cpu(), value.cpu(), classes, page_size=PAGE, recent_capacity=RING, k_block=K_BLOCK,
                           v2_group=V2_GROUP, append_capacity=RING)
    return gcache, ocache


def test_batch8_32k_mixed_pages_across_a_flush():
    """The default benchmark workload itself: 8 requests x 32768 tokens, bf16/INT4/INT2 pages 25/50/25 from the
    benchmark's seeds, one fused append per step, through the flush of the full residual window."""
    batch, tokens, hq, hkv = 8, 32768, 16, 2
    classes = page_classes(tokens // PAGE, 11, 0.25, 0.5)
    pairs = [_pair(tokens, 11 * 1000 + b, classes, hkv) for b in range(batch)]
    oc = [p[1] for p in pairs]
    ex = R.stack_homogeneous_splitk_executors([make_executor(p[0], hq) for p in pairs])
    del pairs
    g = torch.Generator().manual_seed(5)
    steps = RING + 3
    qs = torch.randn(steps, batch, hq, 128, generator=g).to(torch.bfloat16)
    ks = torch.randn(steps, batch, hkv, 128, generator=g).to(torch.bfloat16)
    vs = torch.randn(steps, batch, hkv, 128, generator=g).to(torch.bfloat16)
    stats = R.DynamicCacheStats()
    checked = 0
    for i in range(steps):
        q, k, v = qs[i].cuda(), ks[i].cuda(), vs[i].cuda()
        flushed = ex.arenas.recent_len == RING
        if flushed:   # the window is full: quantize-and-pack it, then append; decode without a fused append
            assert R.append_generated_token(ex.arenas, k, v, global_token_index=tokens + i, logical_position=tokens + i,
                                            stats=stats)
            out = ex.decode_f32(q)
        else:
            out = ex.decode_f32(q, append=(k, v, tokens + i, tokens + i))
        for b in range(batch):
            O.append_token(oc[b], ks[i, b], vs[i, b], tokens + i, tokens + i)
        if i in (0, 63, RING - 1) or flushed or i == steps - 1:
            for b in range(batch):
                assert_close(out[b : b + 1], O.decode_fp32(qs[i, b : b + 1].float(), oc[b]), f"step {i} request {b}")
            checked += 1
    assert checked >= 5 and stats.flushed_tokens == RING      # counted per call (all requests flush together)
    for b in range(batch):
        arena_equal(oc[b], R.ThreePrecisionCache(ex.arenas, b))
    assert ex.device_status() == 0


def test_batch16_65k_seven_query_heads_per_kv_head():
    """One layer of the 28-query / 4-KV-head shape at 16 requests x 65536 tokens; three of the requests are held
    against the oracle (the others share the launch and the page mix)."""
    batch, tokens, hq, hkv = 16, 65536, 28, 4
    classes = page_classes(tokens // PAGE, 13, 0.25, 0.5)
    held = (0, 7, 15)
    execs, oc = [], {}
    for b in range(batch):
        if b in held:
            gcache, oc[b] = _pair(tokens, 13 * 1000 + b, classes, hkv)
        else:
            key, value = synth_kv(tokens, 13 * 1000 + b, "cuda", hkv=hkv)
            gcache = R.build_three_precision_cache(key, value, make_plan(classes, PAGE, RING), page_size=PAGE,
                                                   key_quantization_superblock=K_BLOCK, int2_group_size=V2_GROUP,
                                                   compact_key_append_capacity=RING, recent_flush_size=RING)
            del key, value
        execs.append(make_executor(gcache, hq))
    ex = R.stack_homogeneous_splitk_executors(execs)
    del execs
    g = torch.Generator().manual_seed(6)
    for i in range(3):
        q = torch.randn(batch, hq, 128, generator=g).to(torch.bfloat16)
        k = torch.randn(batch, hkv, 128, generator=g).to(torch.bfloat16)
        v = torch.randn(batch, hkv, 128, generator=g).to(torch.bfloat16)
        out = ex.decode_f32(q.cuda(), append=(k.cuda(), v.cuda(), tokens + i, tokens + i))
        for b in held:
            O.append_token(oc[b], k[b], v[b], tokens + i, tokens + i)
            assert_close(out[b : b + 1], O.decode_fp32(q[b : b + 1].float(), oc[b]), f"step {i} request {b}")
    assert ex.device_status() == 0


def test_single_request_128k_shard_two_level_merge():
    """One request of 131072 tokens (an eighth of a million-token cache, INT4/INT2 value pages 50/50): every CTA of a
    kv head holds one of ~74 partials, merged in two levels."""
    tokens, hq, hkv = 131072, 16, 2
    classes = page_classes(tokens // PAGE, 77, 0.0, 0.5)
    gcache, ocache = _pair(tokens, 900, classes, hkv)
    ex = make_executor(gcache, hq)
    g = torch.Generator().manual_seed(7)
    for i in range(2):
        q = torch.randn(1, hq, 128, generator=g).to(torch.bfloat16)
        k = torch.randn(1, hkv, 128, generator=g).to(torch.bfloat16)
        v = torch.randn(1, hkv, 128, generator=g).to(torch.bfloat16)
        out = ex.decode_f32(q.cuda(), append=(k.cuda(), v.cuda(), tokens + i, tokens + i))
        gcache.recent_fp_pool.active_length += 1
        O.append_token(ocache, k[0], v[0], tokens + i, tokens + i)
        top, den, acc = O.decode_state(q.float(), ocache, chunk=16384)
        assert_close(out, acc / den.unsqueeze(-1), f"step {i}")
    # the un-normalised state: its first entry is the kernel's reference point (it trails the true maximum by up
    # to 8 binary orders), so what must agree is the total weight max + log(sum) and the normalised values
    state = ex.decode_state(q.cuda()).cpu()
    assert torch.allclose(state[..., 0] + state[..., 1].log(), top + den.log(), atol=2e-3)
    assert_close(state[..., 2:] / state[..., 1:2], acc / den.unsqueeze(-1), "un-normalised state")
    assert ex.device_status() == 0


@pytest.mark.parametrize("tokens,batch", [(32768, 4), (131072, 1)])
def test_repeated_launches_give_the_same_bits(tokens, batch):
    """Which CTA of a head arrives last at the merge differs from launch to launch; the result must not: partials
    are folded in slot order whoever folds them.  Sixty launches of the same step (nine partials per head merged in
    one level; 74 per head merged in two), every output bit for bit the first one."""
    hq, hkv = 16, 2
    classes = page_classes(tokens // PAGE, 31, 0.25 if batch > 1 else 0.0, 0.5)
    singles = []
    for b in range(batch):
        key, value = synth_kv(tokens, 4000 + b, "cuda", hkv=hkv)
        singles.append(make_executor(R.build_three_precision_cache(
            key, value, make_plan(classes, PAGE, RING), page_size=PAGE, key_quantization_superblock=K_BLOCK,
            int2_group_size=V2_GROUP, compact_key_append_capacity=RING, recent_flush_size=RING), hq))
        del key, value
    ex = singles[0] if batch == 1 else R.stack_homogeneous_splitk_executors(singles)
    g = torch.Generator().manual_seed(3)
    q = torch.randn(batch, hq, 128, generator=g).to(torch.bfloat16).cuda()
    first = ex.decode_f32(q).clone()
    state = ex.decode_state(q).clone()
    assert torch.isfinite(first).all()
    for i in range(60):
        assert torch.equal(ex.decode_f32(q), first), f"launch {i}"
    for i in range(10):
        assert torch.equal(ex.decode_state(q), state), f"state, launch {i}"
    assert ex.device_status() == 0
