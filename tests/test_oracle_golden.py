"""The CPU oracle restatement, pinned against fixtures produced by the reference itself."""
import numpy as np
import pytest
import torch

from golden_cases import CASES, GoldenCase, compare_snapshot, snapshot_arrays
from oracle import sspa_oracle as O


def image(cache: O.OracleCache, prefix: str) -> dict:
    return snapshot_arrays(
        prefix, k_packed=cache.k_packed, k_scale=cache.k_scale, k_zero=cache.k_zero, k_active=cache.k_active,
        k_offsets=cache.k_offsets, i2_packed=cache.i2_packed, i2_scale=cache.i2_scale, i2_zero=cache.i2_zero,
        i2_active=cache.i2_active, i4_packed=cache.i4_packed, i4_scale=cache.i4_scale, fp_v=cache.fp_v,
        recent_k=cache.recent_k, recent_v=cache.recent_v, recent_len=cache.recent_len,
        recent_global=cache.recent_global, recent_logical=cache.recent_logical,
        recent_page_lengths=cache.recent_page_lengths, i2_global=cache.i2_global, i2_logical=cache.i2_logical)


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_reference_fixture(name):
    case = GoldenCase(name)
    cache = O.build_cache(case.key, case.value, case.classes, **case.build_kwargs())
    compare_snapshot(case, "s0_", image(cache, "s0_"), skip=("recent_k", "recent_v"))
    assert int(case.z["s0_i2_capacity"]) == cache.i2_capacity
    if case.has("s0_out"):
        q = case.queries[0]
        assert np.array_equal(O.decode(q.float(), cache).numpy(), case.z["s0_out"])
        assert np.array_equal(O.decode(q, cache).view(torch.int16).numpy(), case.z["s0_out_lowp"])
        assert np.array_equal(O.decode(q, cache, output_hadamard=True).view(torch.int16).numpy(),
                              case.z["s0_out_hadamard"])
    flushes, tails = [], []
    for i in range(case.appends):
        before = cache.flushes
        prefix_len = cache.k_active % cache.k_block
        if O.append_token(cache, case.new_k[i], case.new_v[i], cache_len(case) + i, cache_len(case) + i):
            flushes.append(i)
            tails.append(prefix_len)
        assert cache.flushes - before == (1 if flushes and flushes[-1] == i else 0)
        if i + 1 in case.marks:
            j = case.marks.index(i + 1) + 1
            compare_snapshot(case, f"s{j}_", image(cache, f"s{j}_"))
            q = case.queries[j]
            assert np.array_equal(O.decode(q.float(), cache).numpy(), case.z[f"s{j}_out"])
            assert np.array_equal(O.decode(q, cache).view(torch.int16).numpy(), case.z[f"s{j}_out_lowp"])
    assert flushes == [int(v) for v in case.z["flush_steps"]]
    assert tails == [int(v) for v in case.z["flush_tails"]]


def cache_len(case):
    return int(case.classes.numel()) * case.page


def test_capacity_exhaustion_raises():
    case = GoldenCase("tiers_page32")
    cache = O.build_cache(case.key, case.value, case.classes, **case.build_kwargs())
    with pytest.raises(RuntimeError):
        for i in range(300):
            O.append_token(cache, case.new_k[i % case.appends], case.new_v[i % case.appends], i, i)


def test_chunked_state_equals_whole_pool_state():
    case = GoldenCase("mixed_page64")
    cache = O.build_cache(case.key, case.value, case.classes, **case.build_kwargs())
    q = case.queries[0].float()
    whole = O.decode(q, cache)
    chunked = O.decode(q, cache, chunk=96)
    assert torch.allclose(whole, chunked, atol=2e-6, rtol=1e-5)


def test_fwht_is_orthonormal_involution():
    x = torch.randn(5, 128, generator=torch.Generator().manual_seed(0))
    assert torch.allclose(O.fwht128(O.fwht128(x)), x, atol=1e-5)


def test_oracle_mrope_reproduces_the_reference_kernel_outputs():
    """tests/golden/mrope_reference.npz holds the outputs of the reference's own multimodal-RoPE kernel (made on a
    GPU by tests/golden/make_mrope_golden.py): the oracle must give the same 16-bit patterns."""
    import os

    import numpy as np
    from make_mrope_golden import CASES, SECTIONS, mrope_inputs
    from recipe import digest
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "mrope_reference.npz"))
    for name, batch, hq, hkv, tokens, dtype, rot_dtype, hadamard in CASES:
        q, k, cos, sin = mrope_inputs(name, batch, hq, hkv, tokens, dtype, rot_dtype)
        assert digest(q, k, cos.float(), sin.float()) == str(z[name + "_digest"]), name
        got_q, got_k = O.qk_mrope(q, k, cos, sin, SECTIONS, hadamard)
        assert np.array_equal(got_q.contiguous().view(torch.int16).numpy(), z[name + "_q"]), name
        assert np.array_equal(got_k.contiguous().view(torch.int16).numpy(), z[name + "_k"]), name
