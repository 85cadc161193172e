"""A cache built by the reference itself, decoded in place by this library.

Needs the unmodified reference under baseline/_ref (oracle/install_reference.py puts it there; it is not part of the
repository) and skips without it.  The reference builds a ThreePrecisionCache on the GPU with its own (Triton) pack
kernels; PackedArenas.from_reference_cache wraps the very same tensors, so both decoders read identical bytes:
this library's output must match the reference's dequantise-then-attend decoder on that cache within the attention
tolerance, a fused append must land in the reference's ring, and the reference's Triton decoder must agree as well.
"""
import os
import sys

import pytest
import torch

import r2omni_b200 as R
from gpu_helpers import assert_close, make_executor
from recipe import make_inputs

pytestmark = pytest.mark.gpu

REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")


@pytest.fixture(scope="module")
def ref():
    if not os.path.isdir(os.path.join(REF, "r2omni")):
        pytest.skip("the reference is not installed under baseline/_ref")
    import bench
    ns, why = bench.load_reference()
    if ns is None:
        pytest.skip(why)
    return ns


def _reference_cache(ref, key, value, classes, page):
    import bench
    dev = key.device
    return ref.build_three_precision_cache(
        key, value, bench.reference_plan(ref, classes, page, 128, dev), page_size=page, key_quantization_superblock=32,
        int2_group_size=32, compact_key_append_capacity=256, recent_flush_size=128)


def test_decode_of_a_reference_built_cache_in_place(ref):
    r = torch.rand(64, generator=torch.Generator().manual_seed(4))
    classes = torch.where(r < 0.25, 1, torch.where(r < 0.75, 2, 5))
    key, value, new_k, new_v, queries = make_inputs(seed=81, hq=16, hkv=2, tokens=64 * 64, appends=4, n_queries=5)
    cache = _reference_cache(ref, key.cuda(), value.cuda(), classes, 64)
    adopted = R.adopt_reference_cache(cache)
    a = adopted.arenas
    assert a.k_packed.data_ptr() == cache.compact_key.packed.data_ptr()              # views, not copies
    assert a.recent_k.data_ptr() == cache.recent_fp_pool.fp_k.data_ptr()
    assert a.i2_packed.data_ptr() == cache.int2_pool.packed_v.packed.data_ptr()
    ex = make_executor(adopted, 16)
    q = queries[0].cuda()
    assert_close(ex.decode_f32(q), ref.triton_mixed_reference(q.float(), cache), "static cache, fp32")
    assert_close(ex(q), ref.triton_mixed_reference(q, cache), "static cache, bf16")
    for i in range(4):   # fused appends through this library land in the reference's ring
        q = queries[i + 1].cuda()
        k, v = new_k[i].unsqueeze(0).contiguous().cuda(), new_v[i].unsqueeze(0).contiguous().cuda()
        out = ex.decode_f32(q, append=(k, v, 4096 + i, 4096 + i))
        a.recent_len += 1
        cache.recent_fp_pool.active_length += 1       # the reference object's host mirror, as its own caller bumps it
        assert int(cache.recent_fp_pool.length_device) == i + 1
        assert torch.equal(cache.recent_fp_pool.fp_k[:, i], new_k[i].cuda())
        assert_close(out, ref.triton_mixed_reference(q.float(), cache), f"after append {i}")
    assert ex.device_status() == 0


def test_reference_triton_decoder_agrees_on_the_same_cache(ref):
    from r2omni.sspa.kernels import triton_fourq_splitk as T
    classes = torch.tensor([1, 2, 5, 2] * 8)
    key, value, _, _, queries = make_inputs(seed=82, hq=16, hkv=2, tokens=32 * 64, appends=1, n_queries=1)
    cache = _reference_cache(ref, key.cuda(), value.cuda(), classes, 64)
    ws = T.allocate_splitk_workspace(cache, block_n=128, num_query_heads=16, partial_output_dtype=torch.float32)
    theirs = T.prepare_splitk_executor(cache, ws, block_n=128, broadcast_k_metadata=True)(queries[0].cuda()).float().clone()
    ours = make_executor(R.adopt_reference_cache(cache), 16)(queries[0].cuda()).float()
    # both are bf16 outputs of the same cache: one bf16 ulp of slack on top of the attention tolerance
    assert_close(ours, theirs, "this library against the reference's Triton decoder")


@pytest.mark.parametrize("hadamard", [False, True])
@pytest.mark.parametrize("rot_dtype", [torch.bfloat16, torch.float32])
def test_mrope_prologue_against_the_reference_kernel(ref, hadamard, rot_dtype):
    """The reference's fused multimodal-RoPE kernel (Triton, run here on the GPU) and this library's give the same
    bits (the library computes x*cos + rot*sin as the reference's compiled kernel does: one product rounded, the
    other fused into the addition)."""
    from r2omni.sspa.kernels.triton_qwen_mrope import qwen_qk_mrope as reference_mrope
    g = torch.Generator().manual_seed(17)
    q = torch.randn(8, 16, 1, 128, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(8, 2, 1, 128, generator=g).to(torch.bfloat16).cuda()
    angle = torch.rand(3, 8, 1, 128, generator=g) * 6.2831853
    cos, sin = torch.cos(angle).to(rot_dtype).cuda(), torch.sin(angle).to(rot_dtype).cuda()
    want_q, want_k = reference_mrope(q, k, cos, sin, [16, 24, 24], apply_hadamard=hadamard)
    got_q, got_k = R.qwen_qk_mrope(q, k, cos, sin, (16, 24, 24), apply_hadamard=hadamard)
    assert torch.equal(got_q.view(torch.int16), want_q.view(torch.int16))
    assert torch.equal(got_k.view(torch.int16), want_k.view(torch.int16))
