"""CPU restatement of R2-Omni's SSPA packed-KV path (torch on CPU, fp32).

TEST INFRASTRUCTURE ONLY: this module is the parity checker.  It is imported by
the tests, by the smoke run and by the CPU-baseline leg of the benchmark, never
by the product package, and it never touches a GPU.

Every routine restates one reference routine and cites it by the reference's
own path.  The restatement is pinned against outputs produced by the reference
itself (fixtures under ``tests/golden``, produced by
``tests/golden/make_golden.py``).

Covered (cache variant ``v_fourq_k_int4_compact``, generated values -> INT2):

* per-channel affine INT4 key blocks       r2omni/sspa/runtime/compact_int4_key.py:83-110
* per-token symmetric INT4 values          r2omni/sspa/runtime/quantization.py:19-50, 77-102
* per-token-group affine INT2 values       r2omni/sspa/runtime/int2_reference.py:96-151
* tier sort of pages into pools            r2omni/sspa/runtime/precision_pool.py:611-669
* cache assembly                           r2omni/sspa/runtime/precision_pool.py:787-984
* one-token append and 128-token flush     r2omni/sspa/runtime/dynamic_fourq_cache.py:172-267
* dequantise-then-attend decode            r2omni/sspa/kernels/triton_fourq_attention.py:41-125
* orthonormal 128-point Walsh-Hadamard     r2omni/sspa/runtime/int2_reference.py:18-31
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

# r2omni/sspa/policy/four_quadrant.py:6-12
EVICTED_PAGE, FP_PAGE, INT4_PAGE, RECENT_FP_PAGE, PROTECTED_FP_PAGE, INT2_PAGE = 0, 1, 2, 3, 4, 5

_EPS = 1.0e-6


def _ceil_to(value: int, multiple: int) -> int:
    return -(-int(value) // int(multiple)) * int(multiple)


# --------------------------------------------------------------------------- #
# quantisers (the bit-exact packing authority is the reference's CPU torch path)
# --------------------------------------------------------------------------- #
def quantize_k_int4(key: torch.Tensor, block: int = 32):
    """Affine INT4 per (head, ``block``-token block, channel).

    compact_int4_key.py:83-110.  The calibrated range is widened to contain 0,
    the step is clamped to 1e-6, codes use the fp32 step while the stored step
    is rounded to fp16.  Returns (packed u8 [H,S,D/2], scale fp16 [H,nb,D],
    zero u8 [H,nb,D]) with ``nb = max(1, ceil(S/block))``.
    """
    h, s, d = key.shape
    nb = max(1, -(-s // block))
    x = key.float()
    pad = nb * block - s
    # pad with +inf / -inf surrogates so a ragged last block calibrates on real rows only
    lo_src = torch.cat((x, x.new_full((h, pad, d), float("inf"))), 1).view(h, nb, block, d)
    hi_src = torch.cat((x, x.new_full((h, pad, d), float("-inf"))), 1).view(h, nb, block, d)
    if s == 0:
        lo = x.new_zeros(h, nb, d)
        hi = x.new_zeros(h, nb, d)
    else:
        lo = lo_src.amin(2).clamp_max(0.0)
        hi = hi_src.amax(2).clamp_min(0.0)
    step = ((hi - lo) / 15.0).clamp_min(_EPS)
    zero = (-lo / step).round().clamp(0, 15)
    owner = torch.arange(s) // block
    codes = (x / step[:, owner] + zero[:, owner]).round().clamp(0, 15).to(torch.uint8)
    packed = codes[..., 0::2] | (codes[..., 1::2] << 4)
    if s == 0:
        step = torch.zeros_like(step)
        zero = torch.zeros_like(zero)
    return packed.contiguous(), step.to(torch.float16), zero.to(torch.uint8)


def dequantize_k_int4(packed, scale, zero, start: int, length: int, block: int):
    """compact_int4_key.py:175-195 -- ``(code - zero) * scale`` in fp32."""
    rows = packed[:, start : start + length]
    codes = torch.stack((rows & 15, rows >> 4), -1).flatten(-2).float()
    owner = torch.arange(start, start + length) // block
    return (codes - zero[:, owner].float()) * scale[:, owner].float()


def quantize_v_int4(value: torch.Tensor):
    """Symmetric INT4 per token: quantization.py:19-50 with ``dim=2`` and the
    nibble packing of quantization.py:77-102 (two's complement, even dim low).

    Returns (packed u8 [H,S,D/2], scale fp32 [H,S,1]).
    """
    x = value.float()
    scale = (x.abs().amax(2, keepdim=True) / 7.0).clamp_min(_EPS)
    q = (x / scale).round().clamp(-7, 7).to(torch.int16)
    nib = (q & 15).to(torch.uint8)
    return (nib[..., 0::2] | (nib[..., 1::2] << 4)).contiguous(), scale


def dequantize_v_int4(packed, scale, round_to=None):
    """``code * scale`` in fp32 (fused_value_pack.py:236-250).  The reference's
    static INT4-V pool is a PackedTensor whose ``dequantize`` additionally
    rounds to the cache dtype (packed_kv_layout.py:30-32); pass ``round_to``
    to reproduce that."""
    nib = torch.stack((packed & 15, packed >> 4), -1).flatten(-2).to(torch.int16)
    out = torch.where(nib >= 8, nib - 16, nib).float() * scale.float()
    return out if round_to is None else out.to(round_to).float()


def quantize_v_int2(value: torch.Tensor, group: int = 32):
    """Affine INT2 per (token, ``group``-wide slice of head_dim).

    int2_reference.py:96-151 (axis ``per_token_group``).  Returns (packed u8
    [H,S,D/4], scale fp16 [H,S,G,1], zero u8 [H,S,G,1]).
    """
    h, s, d = value.shape
    x = value.float().view(h, s, d // group, group)
    lo = x.amin(3, keepdim=True).clamp_max(0.0)
    hi = x.amax(3, keepdim=True).clamp_min(0.0)
    scale = ((hi - lo) / 3.0).clamp_min(_EPS)
    zero = (-lo / scale).round().clamp(0, 3)
    codes = (x / scale + zero).round().clamp(0, 3).to(torch.uint8).view(h, s, d)
    packed = codes[..., 0::4] | (codes[..., 1::4] << 2) | (codes[..., 2::4] << 4) | (codes[..., 3::4] << 6)
    return packed.contiguous(), scale.to(torch.float16), zero.to(torch.uint8)


def dequantize_v_int2(packed, scale, zero, group: int = 32):
    """fused_value_pack.py:445-469."""
    h, s, d4 = packed.shape
    codes = torch.stack((packed & 3, (packed >> 2) & 3, (packed >> 4) & 3, packed >> 6), -1)
    grouped = codes.view(h, s, d4 * 4 // group, group).float()
    return ((grouped - zero.float()) * scale.float()).view(h, s, d4 * 4)


def fwht128(x: torch.Tensor) -> torch.Tensor:
    """Orthonormal Walsh-Hadamard over the last axis (int2_reference.py:18-31)."""
    n = x.shape[-1]
    out = x.float().contiguous()
    span = 1
    while span < n:
        pair = out.view(*out.shape[:-1], -1, 2, span)
        a, b = pair[..., 0, :], pair[..., 1, :]
        out = torch.stack((a + b, a - b), -2).reshape(x.shape)
        span *= 2
    return out * n ** -0.5


def qk_mrope(query: torch.Tensor, key: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, sections,
             apply_hadamard: bool = False):
    """Qwen multimodal RoPE of q [B,Hq,T,128] and k [B,Hkv,T,128] with cos / sin [3,B,T,128], then optionally the
    Hadamard transform; restatement of _qwen_qk_mrope_kernel
    (r2omni/sspa/kernels/triton_qwen_mrope.py:44-212): out[d] = x[d]*cos[axis(d)] + rot(x)[d]*sin[axis(d)],
    rot(x)[d] = -x[d+64] for d < 64 and x[d-64] above, axis by the section of d mod 64, fp32, rounded to the
    input type.  The reference's kernel is compiled code: its sum is one rounded product (rot*sin) fused into a
    multiply-add with the other (x*cos), which is what this computes (the fused step in float64, rounded once more
    to float32).  Pinned by tests/golden/mrope_reference.npz, which holds that kernel's own outputs."""
    d = torch.arange(128)
    sd = d % 64
    axis = torch.where(sd < sections[0], 0, torch.where(sd < sections[0] + sections[1], 1, 2))
    c = cos.float()[axis, :, :, d].permute(1, 2, 0)      # [B,T,128]
    s = sin.float()[axis, :, :, d].permute(1, 2, 0)
    outs = []
    for x in (query, key):
        xf = x.float()
        rot = torch.cat((-xf[..., 64:], xf[..., :64]), dim=-1)
        y = (xf.double() * c[:, None].double() + (rot * s[:, None]).double()).float()
        if apply_hadamard:
            y = fwht128(y)
        outs.append(y.to(x.dtype))
    return outs[0], outs[1]


# --------------------------------------------------------------------------- #
# cache
# --------------------------------------------------------------------------- #
@dataclass
class OracleCache:
    """Plain-tensor image of the reference's ThreePrecisionCache
    (precision_pool.py:210-274) for the INT4-K / tiered-V variant."""

    page_size: int
    k_block: int
    v2_group: int
    flush: int
    dtype: torch.dtype
    # key arena (compact_int4_key.py:113-125)
    k_packed: torch.Tensor
    k_scale: torch.Tensor
    k_zero: torch.Tensor
    k_active: int
    k_offsets: tuple
    # pools
    fp_v: torch.Tensor
    i4_packed: torch.Tensor
    i4_scale: torch.Tensor
    i2_packed: torch.Tensor
    i2_scale: torch.Tensor
    i2_zero: torch.Tensor
    i2_active: int
    # residual window (precision_pool.py:747-784)
    recent_k: torch.Tensor
    recent_v: torch.Tensor
    recent_len: int
    recent_global: torch.Tensor
    recent_logical: torch.Tensor
    recent_page_lengths: torch.Tensor
    # token bookkeeping per pool
    fp_global: torch.Tensor = None
    i4_global: torch.Tensor = None
    i2_global: torch.Tensor = None
    i2_logical: torch.Tensor = None
    evicted_global: torch.Tensor = None
    flushes: int = 0
    appended: int = 0
    stats: dict = field(default_factory=dict)

    @property
    def n_fp(self):
        return int(self.fp_v.shape[1])

    @property
    def n_i4(self):
        return int(self.i4_packed.shape[1])

    @property
    def k_capacity(self):
        return int(self.k_packed.shape[1])

    @property
    def i2_capacity(self):
        return int(self.i2_packed.shape[1])

    @property
    def recent_capacity(self):
        return int(self.recent_k.shape[1])


def tier_sort(page_classes, page_offsets, page_lengths):
    """Stable reorder of pages into (bf16-V, INT4-V, INT2-V, evicted) token lists.

    precision_pool.py:611-669: FP, protected-FP and recent-FP pages form tier 0,
    INT4 pages tier 1, INT2 pages tier 2, everything else is evicted.
    """
    tier = torch.full_like(page_classes, 3)
    for cls in (FP_PAGE, PROTECTED_FP_PAGE, RECENT_FP_PAGE):
        tier[page_classes == cls] = 0
    tier[page_classes == INT4_PAGE] = 1
    tier[page_classes == INT2_PAGE] = 2
    out = []
    for t in range(4):
        pages = (tier == t).nonzero().flatten()
        pieces = [torch.arange(int(page_offsets[p]), int(page_offsets[p]) + int(page_lengths[p])) for p in pages]
        out.append(torch.cat(pieces) if pieces else torch.empty(0, dtype=torch.long))
    return out


def build_cache(
    key,
    value,
    page_classes,
    *,
    page_size=32,
    page_offsets=None,
    page_lengths=None,
    global_token_indices=None,
    logical_positions=None,
    recent_capacity=128,
    k_block=32,
    v2_group=32,
    append_capacity=None,
    flush=128,
):
    """precision_pool.py:787-984 for ``cache_variant="v_fourq_k_int4_compact"``,
    ``generated_value_precision="int2"``, ``matched_fp=False``."""
    h, s, d = key.shape
    n_pages = int(page_classes.numel())
    if page_offsets is None:
        page_offsets = torch.arange(n_pages) * page_size
    if page_lengths is None:
        page_lengths = torch.full((n_pages,), page_size, dtype=torch.long)
    if global_token_indices is None:
        global_token_indices = torch.arange(s)
    if logical_positions is None:
        logical_positions = torch.arange(s)
    if append_capacity is None:
        append_capacity = recent_capacity
    fp_t, i4_t, i2_t, ev_t = tier_sort(page_classes, page_offsets, page_lengths)
    assert fp_t.numel() + i4_t.numel() + i2_t.numel() + ev_t.numel() == s

    # keys: one arena over the concatenated tier order (compact_int4_key.py:223-281)
    order = torch.cat((fp_t, i4_t, i2_t))
    active = int(order.numel())
    k_cap = max(128, _ceil_to(active + append_capacity, 128))
    k_packed = torch.zeros(h, k_cap, d // 2, dtype=torch.uint8)
    k_scale = torch.zeros(h, k_cap // k_block, d, dtype=torch.float16)
    k_zero = torch.zeros(h, k_cap // k_block, d, dtype=torch.uint8)
    if active:
        p, sc, z = quantize_k_int4(key[:, order], k_block)
        k_packed[:, :active] = p
        k_scale[:, : sc.shape[1]] = sc
        k_zero[:, : z.shape[1]] = z

    # values
    fp_v = value[:, fp_t].contiguous()
    i4_packed, i4_scale = quantize_v_int4(value[:, i4_t])
    i2_active = int(i2_t.numel())
    i2_cap = max(128, _ceil_to(i2_active + append_capacity, 128))
    groups = d // v2_group
    i2_packed = torch.zeros(h, i2_cap, d // 4, dtype=torch.uint8)
    i2_scale = torch.zeros(h, i2_cap, groups, 1, dtype=torch.float16)
    i2_zero = torch.zeros(h, i2_cap, groups, 1, dtype=torch.uint8)
    if i2_active:
        p, sc, z = quantize_v_int2(value[:, i2_t], v2_group)
        i2_packed[:, :i2_active], i2_scale[:, :i2_active], i2_zero[:, :i2_active] = p, sc, z

    return OracleCache(
        page_size=page_size, k_block=k_block, v2_group=v2_group, flush=flush, dtype=key.dtype,
        k_packed=k_packed, k_scale=k_scale, k_zero=k_zero, k_active=active,
        k_offsets=(0, int(fp_t.numel()), int(fp_t.numel() + i4_t.numel())),
        fp_v=fp_v, i4_packed=i4_packed, i4_scale=i4_scale,
        i2_packed=i2_packed, i2_scale=i2_scale, i2_zero=i2_zero, i2_active=i2_active,
        recent_k=torch.zeros(h, recent_capacity, d, dtype=key.dtype),
        recent_v=torch.zeros(h, recent_capacity, d, dtype=key.dtype),
        recent_len=0,
        recent_global=torch.full((recent_capacity,), -1, dtype=torch.long),
        recent_logical=torch.full((recent_capacity,), -1, dtype=torch.long),
        recent_page_lengths=torch.zeros(recent_capacity // page_size, dtype=torch.long),
        fp_global=global_token_indices[fp_t], i4_global=global_token_indices[i4_t],
        i2_global=global_token_indices[i2_t].clone(), i2_logical=logical_positions[i2_t].clone(),
        evicted_global=global_token_indices[ev_t],
    )


def flush_recent(cache: OracleCache) -> int:
    """Quantize-and-pack the oldest ``flush`` residual tokens
    (dynamic_fourq_cache.py:195-254).  Returns the re-quantised key tail length
    (compact_int4_key.py:210-220)."""
    n = cache.flush
    kb, vb = cache.recent_k[:, :n].clone(), cache.recent_v[:, :n].clone()
    if cache.k_active + n > cache.k_capacity:
        raise RuntimeError("compact INT4 K capacity exhausted")
    if cache.i2_active + n > cache.i2_capacity:
        raise RuntimeError("compact INT2 V capacity exhausted")
    # keys: re-quantise the partial block in front of the append point together with the new rows
    prefix = cache.k_active // cache.k_block * cache.k_block
    tail = cache.k_active - prefix
    old = dequantize_k_int4(cache.k_packed, cache.k_scale, cache.k_zero, prefix, tail, cache.k_block).to(kb.dtype)
    p, sc, z = quantize_k_int4(torch.cat((old, kb), 1), cache.k_block)
    cache.k_packed[:, prefix : prefix + tail + n] = p
    b0 = prefix // cache.k_block
    cache.k_scale[:, b0 : b0 + sc.shape[1]] = sc
    cache.k_zero[:, b0 : b0 + z.shape[1]] = z
    cache.k_active += n
    # values -> INT2 arena (fused_value_pack.py:474-516)
    p, sc, z = quantize_v_int2(vb, cache.v2_group)
    a = cache.i2_active
    cache.i2_packed[:, a : a + n], cache.i2_scale[:, a : a + n], cache.i2_zero[:, a : a + n] = p, sc, z
    cache.i2_active += n
    cache.i2_global = torch.cat((cache.i2_global, cache.recent_global[:n]))
    cache.i2_logical = torch.cat((cache.i2_logical, cache.recent_logical[:n]))
    # slide the unflushed remainder to the front (dynamic_fourq_cache.py:248-253)
    rest = cache.recent_len - n
    for buf in (cache.recent_k, cache.recent_v):
        buf[:, :rest] = buf[:, n : cache.recent_len].clone()
    for buf in (cache.recent_global, cache.recent_logical):
        buf[:rest] = buf[n : cache.recent_len].clone()
    cache.recent_len = rest
    cache.flushes += 1
    return tail


def append_token(cache: OracleCache, new_k, new_v, global_index: int, logical_position: int) -> bool:
    """dynamic_fourq_cache.py:172-267.  ``new_k``/``new_v``: [H,1,D] or [H,D]."""
    flushed = False
    if cache.recent_len == cache.recent_capacity:
        flush_recent(cache)
        flushed = True
    pos = cache.recent_len
    cache.recent_k[:, pos] = new_k.reshape(cache.recent_k.shape[0], -1)
    cache.recent_v[:, pos] = new_v.reshape(cache.recent_v.shape[0], -1)
    cache.recent_global[pos] = int(global_index)
    cache.recent_logical[pos] = int(logical_position)
    cache.recent_len += 1
    starts = torch.arange(cache.recent_page_lengths.numel()) * cache.page_size
    cache.recent_page_lengths.copy_((cache.recent_len - starts).clamp(0, cache.page_size))
    cache.appended += 1
    return flushed


# --------------------------------------------------------------------------- #
# attention
# --------------------------------------------------------------------------- #
def partial_state(query, key, value, sm_scale):
    """(max, sum-exp, weighted-V) of one pool.  triton_fourq_attention.py:41-55.

    ``query`` [1,Hq,D] (any float dtype), ``key``/``value`` fp32 [Hkv,S,D].
    """
    hq, hkv = query.shape[1], key.shape[0]
    owner = torch.arange(hq) // (hq // hkv)
    logits = torch.einsum("bhd,hsd->bhs", query.float(), key[owner]) * sm_scale
    top = logits.amax(-1)
    w = torch.exp(logits - top.unsqueeze(-1))
    return top, w.sum(-1), torch.einsum("bhs,hsd->bhd", w, value[owner])


def merge_state(a, b):
    """triton_fourq_attention.py:58-69."""
    top = torch.maximum(a[0], b[0])
    wa, wb = torch.exp(a[0] - top), torch.exp(b[0] - top)
    return top, a[1] * wa + b[1] * wb, a[2] * wa.unsqueeze(-1) + b[2] * wb.unsqueeze(-1)


def pool_tensors(cache: OracleCache, round_int4_values: bool = True):
    """Dequantised fp32 (K, V) of the four pools in the reference's merge order
    (bf16-V, INT4-V, INT2-V, residual); triton_fourq_attention.py:17-38, 91-121.

    The reference's CPU decoder takes the INT4 values through ``PackedTensor.dequantize``, which rounds
    ``code * scale`` to the cache's element type (packed_kv_layout.py:30-32); its GPU kernel multiplies in fp32
    and does not round (triton_fourq_splitk.py:789-795).  ``round_int4_values=False`` gives the second form, which
    a test uses to tell a kernel's own error from that rounding."""
    n_i2 = cache.i2_active
    spans = ((cache.k_offsets[0], cache.n_fp), (cache.k_offsets[1], cache.n_i4), (cache.k_offsets[2], n_i2))
    values = (
        cache.fp_v.float(),
        dequantize_v_int4(cache.i4_packed, cache.i4_scale, round_to=cache.dtype if round_int4_values else None),
        dequantize_v_int2(cache.i2_packed[:, :n_i2], cache.i2_scale[:, :n_i2], cache.i2_zero[:, :n_i2], cache.v2_group),
    )
    out = []
    for (start, count), v in zip(spans, values):
        if count:
            out.append((dequantize_k_int4(cache.k_packed, cache.k_scale, cache.k_zero, start, count, cache.k_block), v))
    if cache.recent_len:
        out.append((cache.recent_k[:, : cache.recent_len].float(), cache.recent_v[:, : cache.recent_len].float()))
    return out


def decode_state(query, cache: OracleCache, sm_scale=None, chunk=None, round_int4_values: bool = True):
    """Un-normalised merged (max, sum-exp, weighted-V) over every pool.

    ``chunk`` bounds memory for very long caches by applying the same
    partial/merge functions to sequence chunks of each pool.
    """
    if query.ndim == 4:
        query = query[:, :, 0]
    scale = float(sm_scale) if sm_scale is not None else query.shape[-1] ** -0.5
    state = None
    for k, v in pool_tensors(cache, round_int4_values):
        step = k.shape[1] if chunk is None else int(chunk)
        for s0 in range(0, k.shape[1], step):
            part = partial_state(query, k[:, s0 : s0 + step], v[:, s0 : s0 + step], scale)
            state = part if state is None else merge_state(state, part)
    if state is None:
        raise ValueError("cache has no surviving tokens")
    return state


def decode(query, cache: OracleCache, sm_scale=None, output_hadamard=False, chunk=None):
    """triton_fourq_attention.py:72-125: ``[1,Hq,D]`` in, ``[1,Hq,D]`` out in the
    query dtype.  With ``output_hadamard`` the result is rounded to the query
    dtype first and then transformed (triton_fourq_splitk.py:999-1005)."""
    top, den, acc = decode_state(query, cache, sm_scale, chunk)
    out = (acc / den.unsqueeze(-1)).to(query.dtype)
    if output_hadamard:
        out = fwht128(out.float()).to(query.dtype)
    return out


def decode_fp32(query, cache: OracleCache, sm_scale=None, round_int4_values: bool = True):
    """Same as :func:`decode` without the final rounding to the query dtype."""
    top, den, acc = decode_state(query, cache, sm_scale, round_int4_values=round_int4_values)
    return acc / den.unsqueeze(-1)


def step_bytes(cache: OracleCache, hq: int, append: bool = True) -> int:
    """Algorithmic bytes one decode step must move for this cache (one request)."""
    h, d = cache.k_packed.shape[0], cache.k_packed.shape[2] * 2
    hist = cache.n_fp + cache.n_i4 + cache.i2_active
    per_head = (
        hist * (d // 2 + 3 * d // cache.k_block)
        + cache.n_fp * 2 * d
        + cache.n_i4 * (d // 2 + 4)
        + cache.i2_active * (d // 4 + 3 * d // cache.v2_group)
        + cache.recent_len * 4 * d
    )
    return h * per_head + 4 * hq * d + (8 * h * d if append else 0)
