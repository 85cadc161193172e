"""Shared helpers of the GPU parity tests: build product caches from seeded
inputs and lay their arenas out under the golden fixtures' key names."""
from __future__ import annotations

import torch

import r2omni_b200 as R
from golden_cases import snapshot_arrays

ATOL, RTOL = 2e-3, 1e-2   # attention tolerance of the packed-KV path: max-abs 2e-3 / rel 1e-2

# Decode-grid limits for small inputs (environment variable R2K_GRID_CAP, read by the library at every call):
# one CTA per (request, kv head) streams every tile of every pool through the shared-memory ring; two CTAs per
# head add the cross-CTA merge; three CTAs in all make a CTA cross from one head into the next.
GRID_CAPS = (None, "heads", "2x_heads", "3")


def apply_grid_cap(monkeypatch, mode, heads: int) -> None:
    if mode is None:
        monkeypatch.delenv("R2K_GRID_CAP", raising=False)
    else:
        monkeypatch.setenv("R2K_GRID_CAP", str({"heads": heads, "2x_heads": 2 * heads, "3": 3}[mode]))


def make_plan(classes: torch.Tensor, page: int, recent_capacity: int) -> R.LayerCompressionPlan:
    n = int(classes.numel())
    pos = torch.arange(n * page)
    sel = lambda c: (classes == c).nonzero().flatten()  # noqa: E731
    return R.LayerCompressionPlan(
        layer_id=0, fp_pages=sel(1), int4_pages=sel(2), int2_pages=sel(5), evicted_pages=sel(0),
        protected_pages=torch.empty(0, dtype=torch.long), recent_fp_capacity=recent_capacity,
        logical_positions=pos, global_token_indices=pos.clone(),
        page_offsets=torch.arange(n) * page, page_lengths=torch.full((n,), page), page_classes=classes)


def build_gpu_cache(key, value, classes, *, page_size, recent_capacity=128, k_block=32, v2_group=32,
                    append_capacity=None, device="cuda"):
    return R.build_three_precision_cache(
        key.to(device), value.to(device), make_plan(classes, page_size, recent_capacity), page_size=page_size,
        key_quantization_superblock=k_block, int2_group_size=v2_group,
        compact_key_append_capacity=append_capacity, recent_flush_size=128)


def image(cache, prefix: str, request: int = 0) -> dict:
    a = cache.arenas if hasattr(cache, "arenas") else cache
    c = lambda t: t[request].cpu()  # noqa: E731
    return snapshot_arrays(
        prefix, k_packed=c(a.k_packed), k_scale=c(a.k_scale), k_zero=c(a.k_zero), k_active=a.k_active,
        k_offsets=a.k_offsets, i2_packed=c(a.i2_packed), i2_scale=c(a.i2_scale), i2_zero=c(a.i2_zero),
        i2_active=a.i2_active, i4_packed=c(a.i4_packed), i4_scale=c(a.i4_scale), fp_v=c(a.fp_v),
        recent_k=c(a.recent_k), recent_v=c(a.recent_v), recent_len=a.recent_len,
        recent_global=c(a.recent_global), recent_logical=c(a.recent_logical),
        recent_page_lengths=c(a.recent_page_lengths), i2_global=c(a.i2_global)[: a.i2_active],
        i2_logical=c(a.i2_logical)[: a.i2_active])


def make_executor(cache, hq, **kw):
    ws = R.allocate_splitk_workspace(cache, num_query_heads=hq)
    return R.prepare_splitk_executor(cache, ws, **kw)


def assert_close(got: torch.Tensor, want: torch.Tensor, what: str = "") -> None:
    got, want = got.float().cpu(), want.float().cpu()
    err = (got - want).abs()
    bound = ATOL + RTOL * want.abs()
    worst = (err - bound).max().item()
    assert torch.isfinite(got).all(), f"{what}: non-finite output"
    assert worst <= 0, f"{what}: max-abs err {err.max().item():.3e}, exceeds atol {ATOL} + rtol {RTOL} by {worst:.3e}"
