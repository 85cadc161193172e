"""CPU-side checks: the C ABI library loads and exports every symbol the header declares, its
structs have the layout the ctypes binding assumes, argument validation works without a GPU,
and the host logic (tier sort, work partition, shard ranges) is right."""
import ctypes as C
import os
import re
import shutil
import subprocess
import sys

import pytest
import torch

import r2omni_b200 as R
from r2omni_b200 import _lib as L
from r2omni_b200.build import build_library
from r2omni_b200.sspa.cache import tier_sorted_tokens
from gpu_helpers import make_plan
from oracle import sspa_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "r2k_b200.h")
NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


@pytest.fixture(scope="module")
def lib():
    build_library()
    return L.lib()


def test_library_exports_every_declared_symbol(lib):
    text = open(HEADER).read()
    declared = set(re.findall(r"\b(r2k_[a-z0-9_]+)\s*\(", text))
    assert declared == set(L.EXPORTS), declared ^ set(L.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_struct_layouts_match_the_header(tmp_path):
    src = tmp_path / "sizes.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "r2k_b200.h"\nint main(void){printf("%zu %zu %zu %zu %zu %zu %zu %zu\\n",'
                   "sizeof(R2KGeom), sizeof(R2KCacheView), sizeof(R2KAppend), offsetof(R2KGeom, sm_scale),"
                   "offsetof(R2KCacheView, k_packed_bstride), offsetof(R2KAppend, global_index),"
                   "sizeof(R2KExchange), offsetof(R2KExchange, seq));return 0;}\n")
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), "-o", str(exe), str(src)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    want = [C.sizeof(L.Geom), C.sizeof(L.CacheView), C.sizeof(L.Append), L.Geom.sm_scale.offset,
            L.CacheView.k_packed_bstride.offset, L.Append.global_index.offset, C.sizeof(L.Exchange), L.Exchange.seq.offset]
    assert got == want


def test_status_strings_and_validation_without_a_gpu(lib):
    assert lib.r2k_status_string(0) == b"ok"
    assert b"capacity" in lib.r2k_status_string(L.ERR_CAPACITY)
    need = C.c_size_t(0)
    assert lib.r2k_decode_workspace_bytes(None, C.byref(need)) == L.ERR_NULL
    g = L.Geom()
    g.batch, g.num_q_heads, g.num_kv_heads, g.head_dim = 1, 16, 2, 64            # head_dim must be 128
    assert lib.r2k_decode_workspace_bytes(C.byref(g), C.byref(need)) == L.ERR_GEOMETRY
    g.head_dim, g.num_q_heads = 128, 40                                          # 20 query heads per kv head
    g.page_size, g.k_block, g.v2_group = 32, 32, 32
    assert lib.r2k_decode_workspace_bytes(C.byref(g), C.byref(need)) == L.ERR_GEOMETRY
    g.num_q_heads, g.k_capacity, g.n_i4, g.i4_capacity = 16, 128, 256, 256       # pool larger than the key arena
    assert lib.r2k_decode_workspace_bytes(C.byref(g), C.byref(need)) == L.ERR_GEOMETRY
    assert lib.r2k_pack_k_int4(None, 0, 2, C.c_int64(4), None, C.c_int64(4), None, None, None, C.c_int64(128), 32,
                               C.c_int64(0), None) == L.ERR_NULL
    with pytest.raises(ValueError):
        L.check(L.ERR_GEOMETRY, "x")
    with pytest.raises(RuntimeError):
        L.check(L.ERR_CAPACITY, "x")


def test_exchange_entry_points_validate_without_a_gpu(lib):
    g = L.Geom()
    g.batch, g.num_q_heads, g.num_kv_heads, g.head_dim, g.dtype = 2, 16, 2, 128, L.DTYPE_BF16
    g.page_size, g.k_block, g.v2_group, g.recent_capacity, g.sm_scale = 64, 32, 32, 128, 0.0
    need = C.c_size_t(0)
    assert lib.r2k_exchange_bytes(C.byref(g), 4, C.byref(need)) == L.OK
    states = 2 * 4 * 2 * 16 * 130 * 8   # two halves x ranks x rows x (value, step) words
    assert need.value == (states + 127) // 128 * 128 + 128          # + the device-side step counter
    assert lib.r2k_exchange_bytes(C.byref(g), 9, C.byref(need)) == L.ERR_GEOMETRY
    assert lib.r2k_exchange_bytes(C.byref(g), 2, None) == L.ERR_NULL
    assert lib.r2k_decode_exchange(C.byref(g), None, None, None, None, 0, None, 0, None, None) == L.ERR_NULL
    assert lib.r2k_exchange_close(None, 0) == L.OK


def test_host_buffer_entry_points_validate_without_a_gpu(lib):
    g = L.Geom()
    g.batch, g.num_q_heads, g.num_kv_heads, g.head_dim, g.dtype = 8, 16, 2, 128, L.DTYPE_BF16
    need = C.c_size_t(0)
    assert lib.r2k_decode_host_staging_bytes(C.byref(g), C.byref(need)) == L.OK
    inputs = 8 * 16 * 128 * 2 + 2 * 8 * 2 * 128 * 2            # q | k | v
    result = 8 * 16 * 130 * 4                                    # the largest output form (state rows)
    assert need.value == (inputs + 255) // 256 * 256 + (result + 255) // 256 * 256
    assert lib.r2k_decode_host_staging_bytes(C.byref(g), None) == L.ERR_NULL
    assert lib.r2k_decode_host_staging_bytes(None, C.byref(need)) == L.ERR_GEOMETRY
    buf = (C.c_uint8 * 64)()
    assert lib.r2k_decode_host(C.byref(g), None, None, None, None, 0, None, 0, None, 0, None) == L.ERR_NULL
    # staging too small: refused before any CUDA call
    assert lib.r2k_decode_host(C.byref(g), None, buf, None, None, 0, buf, 64, buf, 0, None) == L.ERR_WORKSPACE


def test_missing_library_is_a_loud_error(monkeypatch):
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB", "/nonexistent/libr2k_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or Triton fallback"):
        L.lib()


def test_cache_build_refuses_cpu_tensors_and_unsupported_variants():
    classes = torch.tensor([1, 2, 5, 0])
    key = torch.zeros(2, 128, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        R.build_three_precision_cache(key, key, make_plan(classes, 32, 128))
    for kw in (dict(cache_variant="v_fourq_k_int2_compact"), dict(matched_fp=True), dict(generated_value_precision="int4"),
               dict(page_size=48), dict(key_quantization_superblock=16), dict(recent_flush_size=96)):
        with pytest.raises(ValueError):
            R.build_three_precision_cache(key, key, make_plan(classes, 32, 128), **kw)
    with pytest.raises(ValueError):
        R.build_three_precision_cache(key, key[:, :64], make_plan(classes, 32, 128))


def test_tier_sort_matches_the_oracle():
    g = torch.Generator().manual_seed(4)
    for page in (16, 32, 64):
        classes = torch.randint(0, 6, (37,), generator=g)
        plan = make_plan(classes, page, 128)
        got = tier_sorted_tokens(plan)
        want = O.tier_sort(classes, plan.page_offsets, plan.page_lengths)
        for a, b in zip(got, want):
            assert torch.equal(a, b)


def test_shard_ranges_tile_the_sequence():
    for total, world, align in ((1 << 20, 8, 128), (1000, 3, 128), (128, 4, 128), (0, 2, 64), (65536 + 64, 5, 64)):
        ranges = [R.shard_token_range(total, world, r, align=align) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == total
        for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
            assert a1 == b0 and a0 <= a1 and a1 % align == 0
        sizes = [b - a for a, b in ranges[:-1]]
        assert not sizes or max(sizes) - min(sizes) <= align
    with pytest.raises(ValueError):
        R.shard_token_range(10, 2, 2)


@pytest.mark.skipif(not os.path.exists(NVCC), reason="nvcc not available")
def test_work_partition_covers_every_tile_exactly_once(tmp_path):
    exe = tmp_path / "partition_check"
    subprocess.run([NVCC, "-O2", "-std=c++17", "-Wno-deprecated-gpu-targets", "-I", os.path.join(ROOT, "include"), "-I",
                    os.path.join(ROOT, "r2omni_b200", "csrc"), "-o", str(exe), os.path.join(ROOT, "tests", "partition_check.cu")],
                   check=True, capture_output=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.startswith("OK"), out.stdout


def test_step_byte_model_counts_every_stream():
    classes = torch.tensor([1, 2, 2, 5])
    key = torch.randn(2, 256, 128).to(torch.bfloat16)
    cache = O.build_cache(key, key, classes, page_size=64)
    want = 2 * (256 * 76 + 64 * 256 + 128 * 68 + 64 * 44) + 4 * 16 * 128
    assert O.step_bytes(cache, 16, append=False) == want
    sys.path.insert(0, ROOT)
    import bench
    assert bench.algorithmic_bytes(64, 128, 64, 0, 1, append=False) == want
