"""Packed/active cache objects of the SSPA path, built on the device.

Mirrors the reference's cache API (r2omni/sspa/runtime/precision_pool.py,
compact_int4_key.py, fused_value_pack.py, cache_plan.py) for the INT4-key /
tiered-value variant.  All storage lives in one :class:`PackedArenas` whose
tensors carry a leading request axis, so that a single cache (B == 1) and a
homogeneous batch share every kernel and every host routine; the
reference-shaped objects (``ThreePrecisionCache``, ``PrecisionPool``,
``CompactInt4KeyArena`` ...) are thin views onto it.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from enum import IntEnum
from typing import Literal

import torch

from .. import _lib as L


class PageClass(IntEnum):
    """r2omni/sspa/policy/four_quadrant.py:6-12."""

    EVICTED_PAGE = 0
    FP_PAGE = 1
    INT4_PAGE = 2
    RECENT_FP_PAGE = 3
    PROTECTED_FP_PAGE = 4
    INT2_PAGE = 5


@dataclass(frozen=True)
class LayerCompressionPlan:
    """r2omni/sspa/runtime/cache_plan.py:11-24."""

    layer_id: int
    fp_pages: torch.Tensor
    int4_pages: torch.Tensor
    int2_pages: torch.Tensor
    evicted_pages: torch.Tensor
    protected_pages: torch.Tensor
    recent_fp_capacity: int
    logical_positions: torch.Tensor
    global_token_indices: torch.Tensor
    page_offsets: torch.Tensor
    page_lengths: torch.Tensor
    page_classes: torch.Tensor


def _ceil_to(value: int, multiple: int) -> int:
    return -(-int(value) // int(multiple)) * int(multiple)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_ptr(device) -> int:
    """Handle of torch's current stream on `device` (the raw accessor costs a fraction of the Stream object)."""
    if _raw_stream is not None and device.index is not None:
        return _raw_stream(device.index)
    return int(torch.cuda.current_stream(device).cuda_stream)


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return L.DTYPE_BF16
    if dtype == torch.float16:
        return L.DTYPE_FP16
    raise ValueError("the packed-KV path stores bfloat16 or float16 keys/values")


def _ptr(t: torch.Tensor | None):
    return None if t is None or t.numel() == 0 else C.c_void_p(t.data_ptr())


# --------------------------------------------------------------------------- #
# pack routines (C ABI)
# --------------------------------------------------------------------------- #
def pack_k_int4_into(src, index, packed, scale, zero, *, k_block: int, dst_start: int) -> None:
    """Quantise ``src[:, index]`` ([H,S,128]) into key-arena rows starting at
    ``dst_start`` (compact_int4_key.py:83-110, 200-220)."""
    h, rows, _ = src.shape
    count = int(rows if index is None else index.numel())
    L.check(L.lib().r2k_pack_k_int4(
        _ptr(src), dtype_code(src.dtype), h, C.c_int64(rows), _ptr(index), C.c_int64(count),
        _ptr(packed), _ptr(scale), _ptr(zero), C.c_int64(packed.shape[-2]), k_block, C.c_int64(dst_start),
        C.c_void_p(_stream_ptr(src.device))), "r2k_pack_k_int4")


def pack_v_int4_into(src, index, packed, scale, *, dst_start: int) -> None:
    """fused_value_pack.py:25-70 / quantization.py:19-50."""
    h, rows, _ = src.shape
    count = int(rows if index is None else index.numel())
    L.check(L.lib().r2k_pack_v_int4(
        _ptr(src), dtype_code(src.dtype), h, C.c_int64(rows), _ptr(index), C.c_int64(count),
        _ptr(packed), _ptr(scale), C.c_int64(packed.shape[-2]), C.c_int64(dst_start),
        C.c_void_p(_stream_ptr(src.device))), "r2k_pack_v_int4")


def pack_v_int2_into(src, index, packed, scale, zero, *, group: int, dst_start: int) -> None:
    """fused_value_pack.py:72-149 / int2_reference.py:96-151."""
    h, rows, _ = src.shape
    count = int(rows if index is None else index.numel())
    L.check(L.lib().r2k_pack_v_int2(
        _ptr(src), dtype_code(src.dtype), h, C.c_int64(rows), _ptr(index), C.c_int64(count),
        _ptr(packed), _ptr(scale), _ptr(zero), C.c_int64(packed.shape[-2]), group, C.c_int64(dst_start),
        C.c_void_p(_stream_ptr(src.device))), "r2k_pack_v_int2")


def gather_rows_into(src, index, dst, *, dst_start: int = 0) -> None:
    h, rows, _ = src.shape
    count = int(index.numel())
    L.check(L.lib().r2k_gather_rows(
        _ptr(src), h, C.c_int64(rows), _ptr(index), C.c_int64(count), _ptr(dst), C.c_int64(dst.shape[-2]),
        C.c_int64(dst_start), C.c_void_p(_stream_ptr(src.device))), "r2k_gather_rows")


# --------------------------------------------------------------------------- #
# storage
# --------------------------------------------------------------------------- #
@dataclass
class PackedArenas:
    """Every device tensor of B homogeneous caches; axis 0 is the request."""

    dtype: torch.dtype
    page_size: int
    k_block: int
    v2_group: int
    flush: int
    k_packed: torch.Tensor      # u8  [B,H,k_cap,64]
    k_scale: torch.Tensor       # f16 [B,H,k_cap/k_block,128]
    k_zero: torch.Tensor        # u8  [B,H,k_cap/k_block,128]
    k_active: int
    k_offsets: tuple
    fp_v: torch.Tensor          # T   [B,H,n_fp,128]
    i4_packed: torch.Tensor     # u8  [B,H,n_i4,64]
    i4_scale: torch.Tensor      # f32 [B,H,n_i4,1]
    i2_packed: torch.Tensor     # u8  [B,H,i2_cap,32]
    i2_scale: torch.Tensor      # f16 [B,H,i2_cap,G,1]
    i2_zero: torch.Tensor       # u8  [B,H,i2_cap,G,1]
    i2_active: int
    recent_k: torch.Tensor      # T   [B,H,cap,128]
    recent_v: torch.Tensor
    recent_len_device: torch.Tensor    # i32 [B]
    recent_global: torch.Tensor        # i64 [B,cap]
    recent_logical: torch.Tensor
    recent_page_lengths: torch.Tensor  # i64 [B,cap/page]
    recent_len: int                    # host mirror (same for every request)
    i2_global: torch.Tensor            # i64 [B, i2 token capacity]
    i2_logical: torch.Tensor
    fp_global: torch.Tensor
    fp_logical: torch.Tensor
    i4_global: torch.Tensor
    i4_logical: torch.Tensor
    evicted_global: torch.Tensor
    generated_k_offset: int = 0
    static_i2_tokens: int = 0
    _view: L.CacheView | None = field(default=None, repr=False)

    # ---- shapes ----
    @property
    def batch(self) -> int:
        return int(self.k_packed.shape[0])

    @property
    def num_kv_heads(self) -> int:
        return int(self.k_packed.shape[1])

    @property
    def k_capacity(self) -> int:
        return int(self.k_packed.shape[2])

    @property
    def n_fp(self) -> int:
        return int(self.fp_v.shape[2])

    @property
    def n_i4(self) -> int:
        return int(self.i4_packed.shape[2])

    @property
    def i2_capacity(self) -> int:
        return int(self.i2_packed.shape[2])

    @property
    def recent_capacity(self) -> int:
        return int(self.recent_k.shape[2])

    @property
    def device(self) -> torch.device:
        return self.k_packed.device

    def tensors(self) -> dict:
        return {k: v for k, v in self.__dict__.items() if isinstance(v, torch.Tensor)}

    # ---- C ABI images ----
    def geom(self, num_q_heads: int, *, full_capacity: bool = False, sm_scale: float = 0.0) -> L.Geom:
        g = L.Geom()
        g.batch, g.num_q_heads, g.num_kv_heads, g.head_dim = self.batch, int(num_q_heads), self.num_kv_heads, 128
        g.dtype, g.page_size, g.k_block, g.v2_group = dtype_code(self.dtype), self.page_size, self.k_block, self.v2_group
        g.n_fp, g.n_i4 = self.n_fp, self.n_i4
        g.n_i2 = min(self.i2_capacity, self.k_capacity - self.k_offsets[2]) if full_capacity else self.i2_active
        g.k_capacity = self.k_capacity
        g.k_off_fp, g.k_off_i4, g.k_off_i2 = self.k_offsets
        g.fp_capacity, g.i4_capacity, g.i2_capacity = self.n_fp, self.n_i4, self.i2_capacity
        g.recent_capacity = self.recent_capacity
        g.sm_scale = float(sm_scale)
        return g

    @classmethod
    def from_reference_cache(cls, cache) -> "PackedArenas":
        """Adopt, without copying any payload, a cache object built by the reference's own
        ``build_three_precision_cache`` on a CUDA device (r2omni/sspa/runtime/precision_pool.py:210-274, 787-984):
        the arenas here are views of the very tensors the reference's executor binds
        (r2omni/sspa/kernels/triton_fourq_splitk.py:1772-1811, 1833-1907), so a decode through this library reads
        the reference's bytes in place and a fused append lands in the reference's residual ring.  The object is
        read by attribute only; nothing of the reference is imported.  Supported: the INT4-key / tiered-value
        variant with generated values going to the INT2 pool; anything else raises ValueError.  Token bookkeeping
        arrays (global / logical indices of the packed pools) are copied, they are not payload."""
        ck = getattr(cache, "compact_key", None)
        if ck is None or int(getattr(ck, "bit_width", 0)) != 4 or getattr(cache, "matched_fp", False):
            raise ValueError("only caches with a compact INT4 key arena can be adopted")
        if getattr(cache, "generated_value_precision", "int2") != "int2":
            raise ValueError("only caches whose generated values go to the INT2 pool can be adopted")
        i2 = cache.int2_pool.packed_v
        if i2 is None or not hasattr(i2, "capacity"):
            raise ValueError("the INT2-value pool must be a preallocated arena")
        ring = cache.recent_fp_pool
        if ring.length_device is None or ring.fp_k is None or ring.capacity <= 0:
            raise ValueError("the residual ring must be preallocated with a device-side length")
        dev, dtype = ck.packed.device, ring.fp_k.dtype
        if dev.type != "cuda":
            raise RuntimeError("only CUDA-resident caches can be adopted; there is no CPU path")
        h, d = int(ck.packed.shape[0]), 128
        n_fp, n_i4 = int(cache.fp_pool.token_count), int(cache.int4_pool.token_count)

        def empty(*shape, dtype):
            return torch.zeros((1, *shape), device=dev, dtype=dtype)

        fp_v = cache.fp_pool.fp_v.unsqueeze(0) if n_fp else empty(h, 0, d, dtype=dtype)
        if n_i4:
            i4 = cache.int4_pool.packed_v
            i4_packed = i4.packed.view(1, h, n_i4, d // 2)
            i4_scale = i4.scale.view(1, h, n_i4, 1)
            if i4_scale.dtype != torch.float32:
                raise ValueError("INT4-value scales must be float32")
        else:
            i4_packed, i4_scale = empty(h, 0, d // 2, dtype=torch.uint8), empty(h, 0, 1, dtype=torch.float32)

        def meta(pool, capacity=None):
            src = pool.page_index.global_token_indices, pool.page_index.logical_positions
            n = int(src[0].numel())
            cap = n if capacity is None else max(int(capacity), n)
            out = [torch.full((1, cap), -1, device=dev, dtype=torch.long) for _ in src]
            for o, t in zip(out, src):
                o[0, :n] = t.to(dev)
            return out

        i2_active = int(i2.active_length)
        fp_g, fp_l = meta(cache.fp_pool)
        i4_g, i4_l = meta(cache.int4_pool)
        i2_g, i2_l = meta(cache.int2_pool, int(i2.capacity))
        return cls(
            dtype=dtype, page_size=int(cache.page_size), k_block=int(ck.superblock_size), v2_group=int(i2.group_size),
            flush=int(cache.recent_flush_size),
            k_packed=ck.packed.unsqueeze(0), k_scale=ck.scale.unsqueeze(0), k_zero=ck.zero_point.unsqueeze(0),
            k_active=int(ck.active_length), k_offsets=tuple(int(v) for v in ck.segment_offsets),
            fp_v=fp_v, i4_packed=i4_packed, i4_scale=i4_scale,
            i2_packed=i2.packed.unsqueeze(0), i2_scale=i2.scale.unsqueeze(0), i2_zero=i2.zero_point.unsqueeze(0),
            i2_active=i2_active,
            recent_k=ring.fp_k.unsqueeze(0), recent_v=ring.fp_v.unsqueeze(0),
            recent_len_device=ring.length_device.view(1),
            recent_global=ring.global_index_buffer.unsqueeze(0), recent_logical=ring.logical_position_buffer.unsqueeze(0),
            recent_page_lengths=ring.page_index.lengths.unsqueeze(0), recent_len=int(ring.active_length or 0),
            i2_global=i2_g, i2_logical=i2_l, fp_global=fp_g, fp_logical=fp_l, i4_global=i4_g, i4_logical=i4_l,
            evicted_global=cache.evicted_global_indices.to(dev).reshape(1, -1).long(),
            generated_k_offset=int(getattr(cache, "generated_k_offset", 0)) or int(ck.active_length),
            static_i2_tokens=i2_active,
        )

    def view(self) -> L.CacheView:
        if self._view is None:
            v = L.CacheView()
            for name in L._PTRS:
                t = {"recent_len": self.recent_len_device}.get(name, getattr(self, name, None))
                setattr(v, name, None if t is None or t.numel() == 0 else t.data_ptr())
                stride = 0 if t is None or t.numel() == 0 or t.shape[0] == 1 else t.stride(0) * t.element_size()
                setattr(v, name + "_bstride", stride)
            self._view = v
        return self._view


# --------------------------------------------------------------------------- #
# reference-shaped views
# --------------------------------------------------------------------------- #
@dataclass(frozen=True)
class PhysicalPageIndex:
    """precision_pool.py:35-41."""

    original_page_ids: torch.Tensor
    physical_offsets: torch.Tensor
    lengths: torch.Tensor
    global_token_indices: torch.Tensor
    logical_positions: torch.Tensor


class CompactInt4KeyArena:
    """View with the attributes of compact_int4_key.py:113-220."""

    bit_width = 4

    def __init__(self, arenas: PackedArenas, request: int = 0):
        self._a, self._r = arenas, request

    packed = property(lambda s: s._a.k_packed[s._r])
    scale = property(lambda s: s._a.k_scale[s._r])
    zero_point = property(lambda s: s._a.k_zero[s._r])
    active_length = property(lambda s: s._a.k_active)
    capacity = property(lambda s: s._a.k_capacity)
    segment_offsets = property(lambda s: tuple(s._a.k_offsets))
    superblock_size = property(lambda s: s._a.k_block)
    original_dtype = property(lambda s: s._a.dtype)
    head_count = property(lambda s: s._a.num_kv_heads)
    head_dim = 128
    superblock_count = property(lambda s: int(s._a.k_scale.shape[2]))

    def allocation_tensors(self):
        return self.packed, self.scale, self.zero_point

    @property
    def nbytes(self) -> int:
        return int(sum(t.numel() * t.element_size() for t in self.allocation_tensors()))

    @property
    def active_nbytes(self) -> int:
        n = self.active_length
        if n <= 0:
            return 0
        blocks = -(-n // self.superblock_size)
        return int(self.head_count * (n * 64 + blocks * 128 * 3))

    def dequantize_range(self, start: int, length: int) -> torch.Tensor:
        """Verification helper (torch ops): ``(code - zero) * scale`` in fp32."""
        start, length = int(start), int(length)
        if start < 0 or length < 0 or start + length > self.active_length:
            raise ValueError("compact INT4 K range is outside the active payload")
        rows = self.packed[:, start : start + length]
        codes = torch.stack((rows & 15, rows >> 4), -1).flatten(-2).float()
        owner = torch.arange(start, start + length, device=rows.device) // self.superblock_size
        return (codes - self.zero_point[:, owner].float()) * self.scale[:, owner].float()

    def dequantize(self) -> torch.Tensor:
        return self.dequantize_range(0, self.active_length)


class CompactInt2ValueArena:
    """View with the attributes of fused_value_pack.py:401-516."""

    axis = "per_token_group"
    superblock_size = 128

    def __init__(self, arenas: PackedArenas, request: int = 0):
        self._a, self._r = arenas, request

    packed = property(lambda s: s._a.i2_packed[s._r])
    scale = property(lambda s: s._a.i2_scale[s._r])
    zero_point = property(lambda s: s._a.i2_zero[s._r])
    active_length = property(lambda s: s._a.i2_active)
    capacity = property(lambda s: s._a.i2_capacity)
    group_size = property(lambda s: s._a.v2_group)
    original_dtype = property(lambda s: s._a.dtype)
    original_shape = property(lambda s: (s._a.num_kv_heads, s._a.i2_active, 128))

    def allocation_tensors(self):
        return self.packed, self.scale, self.zero_point

    @property
    def nbytes(self) -> int:
        return int(sum(t.numel() * t.element_size() for t in self.allocation_tensors()))

    @property
    def active_nbytes(self) -> int:
        groups = 128 // self.group_size
        return int(self._a.num_kv_heads * self.active_length * (32 + 3 * groups))

    def dequantize_range(self, start: int, length: int) -> torch.Tensor:
        start, length = int(start), int(length)
        if start < 0 or length < 0 or start + length > self.active_length:
            raise ValueError("compact INT2 V dequantization range is outside active storage")
        p = self.packed[:, start : start + length]
        codes = torch.stack((p & 3, (p >> 2) & 3, (p >> 4) & 3, p >> 6), -1)
        h = p.shape[0]
        grouped = codes.view(h, length, 128 // self.group_size, self.group_size).float()
        scale = self.scale[:, start : start + length].float()
        zero = self.zero_point[:, start : start + length].float()
        return ((grouped - zero) * scale).view(h, length, 128)

    def dequantize(self) -> torch.Tensor:
        return self.dequantize_range(0, self.active_length)


class PackedInt4Values:
    """Static INT4-value pool with the fields of PackedTensor (packed_kv_layout.py:11-32)."""

    num_bits = 4
    quant_scheme = "per_token"
    zero_point = None

    def __init__(self, arenas: PackedArenas, request: int = 0):
        self._a, self._r = arenas, request

    packed = property(lambda s: s._a.i4_packed[s._r].flatten())
    scale = property(lambda s: s._a.i4_scale[s._r])
    original_shape = property(lambda s: (s._a.num_kv_heads, s._a.n_i4, 128))
    dtype = property(lambda s: s._a.dtype)

    @property
    def nbytes(self) -> int:
        return int(self._a.i4_packed[self._r].numel() + self._a.i4_scale[self._r].numel() * 4)

    def dequantize(self) -> torch.Tensor:
        p = self._a.i4_packed[self._r]
        nib = torch.stack((p & 15, p >> 4), -1).flatten(-2).to(torch.int16)
        return (torch.where(nib >= 8, nib - 16, nib).float() * self.scale.float()).to(self.dtype)


class PrecisionPool:
    """View with the attributes of precision_pool.py:152-207."""

    def __init__(self, arenas: PackedArenas, name: str, request: int = 0):
        self._a, self.name, self._r = arenas, name, request

    @property
    def token_count(self) -> int:
        a = self._a
        return {"fp": a.n_fp, "int4": a.n_i4, "int2": a.i2_active, "recent_fp": a.recent_len}[self.name]

    @property
    def active_length(self):
        return self._a.recent_len if self.name == "recent_fp" else None

    @active_length.setter
    def active_length(self, value) -> None:
        if self.name != "recent_fp":
            raise AttributeError("only the Recent-FP pool has a mutable active length")
        self._a.recent_len = int(value)

    @property
    def capacity(self) -> int:
        return self._a.recent_capacity if self.name == "recent_fp" else 0

    @property
    def fp_k(self):
        return self._a.recent_k[self._r] if self.name == "recent_fp" else None

    @property
    def fp_v(self):
        if self.name == "recent_fp":
            return self._a.recent_v[self._r]
        return self._a.fp_v[self._r] if self.name == "fp" and self._a.n_fp else None

    packed_k = None

    @property
    def packed_v(self):
        if self.name == "int4":
            return PackedInt4Values(self._a, self._r) if self._a.n_i4 else None
        if self.name == "int2":
            return CompactInt2ValueArena(self._a, self._r)
        return None

    @property
    def length_device(self):
        return self._a.recent_len_device[self._r : self._r + 1] if self.name == "recent_fp" else None

    @property
    def global_index_buffer(self):
        return self._a.recent_global[self._r] if self.name == "recent_fp" else None

    @property
    def logical_position_buffer(self):
        return self._a.recent_logical[self._r] if self.name == "recent_fp" else None

    @property
    def page_index(self) -> PhysicalPageIndex:
        a, r, n = self._a, self._r, self.token_count
        page = a.page_size
        if self.name == "recent_fp":
            pages = a.recent_capacity // page
            return PhysicalPageIndex(
                torch.full((pages,), -1, device=a.device, dtype=torch.long),
                torch.arange(pages, device=a.device, dtype=torch.long) * page,
                a.recent_page_lengths[r], a.recent_global[r], a.recent_logical[r])
        glob, logi = {"fp": (a.fp_global, a.fp_logical), "int4": (a.i4_global, a.i4_logical),
                      "int2": (a.i2_global, a.i2_logical)}[self.name]
        pages = -(-n // page)
        offsets = torch.arange(pages, device=a.device, dtype=torch.long) * page
        lengths = (n - offsets).clamp(max=page)
        return PhysicalPageIndex(torch.full((pages,), -1, device=a.device, dtype=torch.long), offsets, lengths,
                                 glob[r][:n], logi[r][:n])

    @property
    def payload_bytes(self) -> int:
        """Allocated payload bytes of the pool, reserved capacity included (precision_pool.py:170-176): what the
        reference's attention manager sums for its storage statistics."""
        a, h = self._a, self._a.num_kv_heads
        if self.name == "fp":
            return int(h * a.n_fp * 256)
        if self.name == "int4":
            return int(h * a.n_i4 * 68)
        if self.name == "int2":
            return int(h * a.i2_capacity * (32 + 3 * (128 // a.v2_group)))
        return int(2 * h * a.recent_capacity * 256)

    @property
    def active_payload_bytes(self) -> int:
        a, n = self._a, self.token_count
        h = a.num_kv_heads
        return int({"fp": h * n * 256, "int4": h * n * 68, "int2": h * n * (32 + 3 * (128 // a.v2_group)),
                    "recent_fp": h * n * 512}[self.name])


class ThreePrecisionCache:
    """The packed/active cache of one request (precision_pool.py:210-274)."""

    matched_fp = False
    cache_variant = "v_fourq_k_int4_compact"
    quantization_superblock = 128
    generated_value_precision = "int2"
    uniform_int4_key = True
    uniform_int2_key = False
    full_precision_key = False
    compact_int4_key = True
    compact_int2_key = False
    compact_int2_value = True
    compact_int4_value = None

    def __init__(self, arenas: PackedArenas, request: int = 0):
        self.arenas, self._r = arenas, request
        self.fp_pool = PrecisionPool(arenas, "fp", request)
        self.int4_pool = PrecisionPool(arenas, "int4", request)
        self.int2_pool = PrecisionPool(arenas, "int2", request)
        self.recent_fp_pool = PrecisionPool(arenas, "recent_fp", request)
        self.compact_key = CompactInt4KeyArena(arenas, request)
        self.compact_value = CompactInt2ValueArena(arenas, request)

    page_size = property(lambda s: s.arenas.page_size)
    recent_flush_size = property(lambda s: s.arenas.flush)
    static_int4_tokens = property(lambda s: s.arenas.n_i4)
    generated_k_offset = property(lambda s: s.arenas.generated_k_offset)
    evicted_global_indices = property(lambda s: s.arenas.evicted_global[s._r])

    @property
    def survivor_count(self) -> int:
        a = self.arenas
        return a.n_fp + a.n_i4 + a.i2_active + a.recent_len

    @property
    def payload_bytes(self) -> int:
        a = self.arenas
        names = ("k_packed", "k_scale", "k_zero", "fp_v", "i4_packed", "i4_scale", "i2_packed", "i2_scale", "i2_zero",
                 "recent_k", "recent_v")
        return int(sum(getattr(a, n)[self._r].numel() * getattr(a, n).element_size() for n in names))

    @property
    def storage_bytes(self) -> int:
        return precision_cache_storage_breakdown(self)["persistent_cache_bytes"]


def precision_cache_storage_breakdown(cache: ThreePrecisionCache) -> dict:
    """Allocated bytes, reserved capacity included (precision_pool.py:296-338)."""
    a, r = cache.arenas, cache._r
    meta_names = ("recent_len_device", "recent_global", "recent_logical", "recent_page_lengths", "i2_global", "i2_logical",
                  "fp_global", "fp_logical", "i4_global", "i4_logical", "evicted_global")
    meta = sum(getattr(a, n)[r].numel() * getattr(a, n).element_size() for n in meta_names)
    payload = cache.payload_bytes
    return {"kv_payload_bytes": int(payload), "metadata_bytes": int(meta), "persistent_cache_bytes": int(payload + meta)}


def precision_cache_active_storage_breakdown(cache: ThreePrecisionCache) -> dict:
    """Populated bytes only (precision_pool.py:341-397)."""
    pools = (cache.fp_pool, cache.int4_pool, cache.int2_pool, cache.recent_fp_pool)
    payload = sum(p.active_payload_bytes for p in pools) + cache.compact_key.active_nbytes
    page = cache.page_size
    meta = cache.evicted_global_indices.numel() * 8
    for p in pools:
        n = p.token_count
        meta += 3 * 8 * (-(-n // page)) + 2 * 8 * n
    meta += 4
    return {"kv_payload_bytes": int(payload), "metadata_bytes": int(meta), "persistent_cache_bytes": int(payload + meta)}


# --------------------------------------------------------------------------- #
# builder
# --------------------------------------------------------------------------- #
def tier_sorted_tokens(plan: LayerCompressionPlan):
    """Stable reorder of pages into (bf16-V, INT4-V, INT2-V, evicted) token lists
    (precision_pool.py:611-669), computed on the host from the small page table."""
    classes = plan.page_classes.detach().cpu().long()
    offsets = plan.page_offsets.detach().cpu().long()
    lengths = plan.page_lengths.detach().cpu().long()
    tier = torch.full_like(classes, 3)
    for cls in (PageClass.FP_PAGE, PageClass.PROTECTED_FP_PAGE, PageClass.RECENT_FP_PAGE):
        tier[classes == int(cls)] = 0
    tier[classes == int(PageClass.INT4_PAGE)] = 1
    tier[classes == int(PageClass.INT2_PAGE)] = 2
    order = torch.argsort(tier, stable=True)
    o_len, o_start, o_tier = lengths[order], offsets[order], tier[order]
    total = int(o_len.sum())
    starts = torch.repeat_interleave(o_start, o_len)
    firsts = torch.repeat_interleave(o_len.cumsum(0) - o_len, o_len)
    tokens = starts + torch.arange(total) - firsts
    token_tier = torch.repeat_interleave(o_tier, o_len)
    return tuple(tokens[token_tier == t] for t in range(4))


def build_three_precision_cache(
    key: torch.Tensor,
    value: torch.Tensor,
    plan: LayerCompressionPlan,
    *,
    page_size: int = 32,
    quantization_superblock: int = 128,
    key_quantization_superblock: int = 32,
    int2_group_size: int = 32,
    generated_value_precision: Literal["int2", "int4"] = "int2",
    matched_fp: bool = False,
    preallocate_recent: bool = True,
    cache_variant: str = "v_fourq_k_int4_compact",
    compact_key_append_capacity: int | None = None,
    recent_flush_size: int = 128,
) -> ThreePrecisionCache:
    """Stable page reorder into contiguous bf16/INT4/INT2 value pools over one
    INT4 key arena, plus the residual ring (precision_pool.py:787-984), packed on
    the device by this library's kernels."""
    if key.shape != value.shape or key.ndim != 3:
        raise ValueError("key/value must be logical [Hkv,S,D]")
    if int(key.shape[1]) != int(plan.logical_positions.numel()):
        raise ValueError("K/V sequence length must match the static plan")
    if int(key.shape[2]) != 128:
        raise ValueError("the packed-KV path requires head_dim=128")
    if page_size not in {16, 32, 64}:
        raise ValueError("page_size must be 16, 32, or 64")
    if quantization_superblock != 128:
        raise ValueError("formal precision pools use 128-token quantization superblocks")
    if key_quantization_superblock not in {32, 64, 128}:
        raise ValueError("K quantization superblock must be 32, 64, or 128")
    if int2_group_size not in {32, 64, 128}:
        raise ValueError("compact INT2 V requires group_size 32, 64, or 128")
    if (recent_flush_size not in {32, 64, 128} or recent_flush_size % page_size
            or recent_flush_size % key_quantization_superblock):
        raise ValueError("recent_flush_size must be 32/64/128 and align to page/K blocks")
    if not preallocate_recent:
        raise ValueError("the B200 path always preallocates the Recent-FP ring")
    if plan.recent_fp_capacity < recent_flush_size:
        raise ValueError("Recent-FP capacity must cover one configured flush")
    if plan.recent_fp_capacity % page_size:
        raise ValueError("Recent-FP capacity must be positive and page aligned")
    if cache_variant != "v_fourq_k_int4_compact" or matched_fp:
        raise ValueError(f"unsupported cache_variant for the B200 path: {cache_variant} (matched_fp={matched_fp})")
    if generated_value_precision != "int2":
        raise ValueError("the B200 path flushes generated values to the INT2 pool (generated_value_precision='int2')")
    if not key.is_cuda:
        raise RuntimeError("build_three_precision_cache packs on a CUDA device; there is no CPU path")
    dtype_code(key.dtype)
    dev = key.device
    key, value = key.contiguous(), value.contiguous()
    h, s, d = key.shape

    fp_t, i4_t, i2_t, ev_t = tier_sorted_tokens(plan)
    if fp_t.numel() + i4_t.numel() + i2_t.numel() + ev_t.numel() != s:
        raise ValueError("compact physical pools must cover every logical token")
    append_capacity = plan.recent_fp_capacity if compact_key_append_capacity is None else int(compact_key_append_capacity)
    n_fp, n_i4, n_i2 = int(fp_t.numel()), int(i4_t.numel()), int(i2_t.numel())
    active = n_fp + n_i4 + n_i2
    k_cap = max(128, _ceil_to(active + append_capacity, 128))
    i2_cap = max(128, _ceil_to(n_i2 + append_capacity, 128))
    groups = d // int2_group_size
    cap = int(plan.recent_fp_capacity)
    glob = plan.global_token_indices.detach().cpu().long()
    logi = plan.logical_positions.detach().cpu().long()
    meta_cap = n_i2 + max(0, min(i2_cap - n_i2, k_cap - active)) // page_size * page_size

    def z(*shape, dtype):
        return torch.zeros((1, *shape), device=dev, dtype=dtype)

    def meta(src, extra=0):
        out = torch.full((1, src.numel() + extra), -1, device=dev, dtype=torch.long)
        out[0, : src.numel()] = src.to(dev)
        return out

    arenas = PackedArenas(
        dtype=key.dtype, page_size=int(page_size), k_block=int(key_quantization_superblock), v2_group=int(int2_group_size),
        flush=int(recent_flush_size),
        k_packed=z(h, k_cap, 64, dtype=torch.uint8),
        k_scale=z(h, k_cap // key_quantization_superblock, d, dtype=torch.float16),
        k_zero=z(h, k_cap // key_quantization_superblock, d, dtype=torch.uint8),
        k_active=active, k_offsets=(0, n_fp, n_fp + n_i4),
        fp_v=z(h, n_fp, d, dtype=key.dtype),
        i4_packed=z(h, n_i4, 64, dtype=torch.uint8), i4_scale=z(h, n_i4, 1, dtype=torch.float32),
        i2_packed=z(h, i2_cap, 32, dtype=torch.uint8), i2_scale=z(h, i2_cap, groups, 1, dtype=torch.float16),
        i2_zero=z(h, i2_cap, groups, 1, dtype=torch.uint8), i2_active=n_i2,
        recent_k=z(h, cap, d, dtype=key.dtype), recent_v=z(h, cap, d, dtype=key.dtype),
        recent_len_device=torch.zeros(1, device=dev, dtype=torch.int32),
        recent_global=torch.full((1, cap), -1, device=dev, dtype=torch.long),
        recent_logical=torch.full((1, cap), -1, device=dev, dtype=torch.long),
        recent_page_lengths=torch.zeros((1, cap // page_size), device=dev, dtype=torch.long),
        recent_len=0,
        i2_global=meta(glob[i2_t], meta_cap - n_i2), i2_logical=meta(logi[i2_t], meta_cap - n_i2),
        fp_global=meta(glob[fp_t]), fp_logical=meta(logi[fp_t]),
        i4_global=meta(glob[i4_t]), i4_logical=meta(logi[i4_t]),
        evicted_global=meta(glob[ev_t]),
        generated_k_offset=active, static_i2_tokens=n_i2,
    )
    if active:
        order = torch.cat((fp_t, i4_t, i2_t)).to(dev)
        pack_k_int4_into(key, order, arenas.k_packed[0], arenas.k_scale[0], arenas.k_zero[0],
                         k_block=arenas.k_block, dst_start=0)
    if n_fp:
        gather_rows_into(value, fp_t.to(dev), arenas.fp_v[0])
    if n_i4:
        pack_v_int4_into(value, i4_t.to(dev), arenas.i4_packed[0], arenas.i4_scale[0], dst_start=0)
    if n_i2:
        pack_v_int2_into(value, i2_t.to(dev), arenas.i2_packed[0], arenas.i2_scale[0], arenas.i2_zero[0],
                         group=arenas.v2_group, dst_start=0)
    return ThreePrecisionCache(arenas)


def adopt_reference_cache(cache) -> ThreePrecisionCache:
    """This library's cache object over the tensors of a cache the reference built (zero copy, see
    PackedArenas.from_reference_cache): hand it to allocate_splitk_workspace / prepare_splitk_executor as usual."""
    return ThreePrecisionCache(PackedArenas.from_reference_cache(cache))


def stack_arenas(caches) -> PackedArenas:
    """Copy B identical-geometry caches into request-major arenas
    (triton_fourq_splitk.py:1975-1992, 2114-2160)."""
    first = caches[0].arenas
    scalars = ("dtype", "page_size", "k_block", "v2_group", "flush", "k_active", "k_offsets", "i2_active", "recent_len",
               "generated_k_offset", "static_i2_tokens")
    for i, c in enumerate(caches[1:], start=1):
        bad = [n for n in scalars if getattr(c.arenas, n) != getattr(first, n)]
        bad += [n for n, t in first.tensors().items() if tuple(getattr(c.arenas, n).shape) != tuple(t.shape)]
        if bad:
            raise ValueError(f"split-K request {i} is outside the homogeneous bucket: " + ", ".join(bad))
    fields = {n: getattr(first, n) for n in scalars}
    for name in first.tensors():
        fields[name] = torch.cat([getattr(c.arenas, name) for c in caches], dim=0).contiguous()
    return PackedArenas(**fields)
