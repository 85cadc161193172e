// Quantize-and-pack kernels, bit-exact with the reference's CPU torch routines:
// IEEE divisions (__fdiv_rn), round-half-even (rintf), no fused multiply-add
// across the divide/add, steps stored as fp16 while codes use the fp32 step.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "device_utils.cuh"

namespace r2k {

template <bool BF16>
__device__ __forceinline__ float raw_to_float(uint16_t raw) {
  if (BF16) return __uint_as_float((uint32_t)raw << 16);
  return __half2float(__ushort_as_half(raw));
}
template <bool BF16>
__device__ __forceinline__ float round_through_elem(float x) {
  if (BF16) return __bfloat162float(__float2bfloat16_rn(x));
  return __half2float(__float2half_rn(x));
}

struct PackArgs {
  const uint16_t* src;      // [B][H, src_rows, 128] 16-bit elements
  int64_t src_bstride;      // bytes
  int64_t src_rows;
  const int64_t* index;     // optional [count] source rows (shared by every request)
  int64_t count;
  int64_t capacity;         // destination rows per head
  int64_t dst_start;
  int num_heads;
};

// ---- keys: per (head, block, channel) affine INT4 -------------------------
// One CTA of 64 threads per (block, head, request); thread c owns channels 2c, 2c+1.
// compact_int4_key.py:83-110 (quantiser), :210-220 (tail re-quantisation).
template <bool BF16>
__global__ void __launch_bounds__(64) pack_k_int4_kernel(PackArgs a, uint8_t* packed, __half* scale, uint8_t* zero,
                                                         int64_t packed_bstride, int64_t scale_bstride, int64_t zero_bstride,
                                                         int k_block, int64_t first_block) {
  // A flush launches the value pack behind this kernel with programmatic stream serialization: the two read
  // different halves of the residual window and write different arenas, so they may run side by side.
  launch_dependents();
  const int64_t blk = first_block + blockIdx.x;
  const int head = blockIdx.y, req = blockIdx.z, c = threadIdx.x;
  const int64_t blocks_per_head = a.capacity / k_block;
  const uint16_t* src = reinterpret_cast<const uint16_t*>(reinterpret_cast<const uint8_t*>(a.src) + req * a.src_bstride) +
                        (int64_t)head * a.src_rows * 128;
  uint8_t* prow = packed + req * packed_bstride + ((int64_t)head * a.capacity) * 64;
  __half* srow = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(scale) + req * scale_bstride) +
                 ((int64_t)head * blocks_per_head + blk) * 128;
  uint8_t* zrow = zero + req * zero_bstride + ((int64_t)head * blocks_per_head + blk) * 128;

  const int64_t r_begin = blk * k_block;
  const int64_t r_end = min(r_begin + (int64_t)k_block, a.dst_start + a.count);
  // rows in front of dst_start are already packed: they are re-quantised from their dequantised, element-rounded values
  const float old_s0 = __half2float(srow[2 * c]), old_s1 = __half2float(srow[2 * c + 1]);
  const float old_z0 = (float)zrow[2 * c], old_z1 = (float)zrow[2 * c + 1];

  // The block's values (raw 16-bit pairs: re-quantised rows are element-rounded, so nothing is lost) are staged in
  // shared memory by the first pass: its loads are independent and run several at a time, and the second pass
  // reads no global memory, so its stores do not wait behind loads that might alias them.
  extern __shared__ uint32_t staged_words[];   // k_block rows of 64 words (dynamic: k_block * 256 bytes)
  uint32_t (*staged)[64] = reinterpret_cast<uint32_t (*)[64]>(staged_words);
  auto fetch_raw = [&](int64_t r) -> uint32_t {
    if (r < a.dst_start) {
      const uint8_t byte = prow[r * 64 + c];
      const float x0 = __fmul_rn(__fsub_rn((float)(byte & 15), old_z0), old_s0);
      const float x1 = __fmul_rn(__fsub_rn((float)(byte >> 4), old_z1), old_s1);
      if (BF16) return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x0)) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x1)) << 16);
      return (uint32_t)__half_as_ushort(__float2half_rn(x0)) | ((uint32_t)__half_as_ushort(__float2half_rn(x1)) << 16);
    }
    const int64_t i = r - a.dst_start;
    const int64_t s = a.index ? a.index[i] : i;
    return *reinterpret_cast<const uint32_t*>(src + s * 128 + 2 * c);
  };

  float lo0 = INFINITY, hi0 = -INFINITY, lo1 = INFINITY, hi1 = -INFINITY;
  const int rows = (int)(r_end - r_begin);
#pragma unroll 8
  for (int i = 0; i < rows; ++i) {
    const uint32_t w = fetch_raw(r_begin + i);
    staged[i][c] = w;
    const float x0 = raw_to_float<BF16>((uint16_t)(w & 0xffffu)), x1 = raw_to_float<BF16>((uint16_t)(w >> 16));
    lo0 = fminf(lo0, x0); hi0 = fmaxf(hi0, x0);
    lo1 = fminf(lo1, x1); hi1 = fmaxf(hi1, x1);
  }
  lo0 = fminf(lo0, 0.f); hi0 = fmaxf(hi0, 0.f);
  lo1 = fminf(lo1, 0.f); hi1 = fmaxf(hi1, 0.f);
  const float st0 = fmaxf(__fdiv_rn(__fsub_rn(hi0, lo0), 15.f), 1.0e-6f);
  const float st1 = fmaxf(__fdiv_rn(__fsub_rn(hi1, lo1), 15.f), 1.0e-6f);
  const float zp0 = fminf(fmaxf(rintf(__fdiv_rn(-lo0, st0)), 0.f), 15.f);
  const float zp1 = fminf(fmaxf(rintf(__fdiv_rn(-lo1, st1)), 0.f), 15.f);
#pragma unroll 4
  for (int i = 0; i < rows; ++i) {
    const uint32_t w = staged[i][c];   // written by this very thread
    const float x0 = raw_to_float<BF16>((uint16_t)(w & 0xffffu)), x1 = raw_to_float<BF16>((uint16_t)(w >> 16));
    const float q0 = fminf(fmaxf(rintf(__fadd_rn(__fdiv_rn(x0, st0), zp0)), 0.f), 15.f);
    const float q1 = fminf(fmaxf(rintf(__fadd_rn(__fdiv_rn(x1, st1), zp1)), 0.f), 15.f);
    prow[(r_begin + i) * 64 + c] = (uint8_t)((uint32_t)q0 | ((uint32_t)q1 << 4));
  }
  srow[2 * c] = __float2half_rn(st0);
  srow[2 * c + 1] = __float2half_rn(st1);
  zrow[2 * c] = (uint8_t)zp0;
  zrow[2 * c + 1] = (uint8_t)zp1;
}

// ---- values: per-token symmetric INT4 -------------------------------------
// One warp per (token, head, request); lane owns dims 4l..4l+3.
// quantization.py:19-50, 77-102; fused_value_pack.py:25-70.
template <bool BF16>
__global__ void __launch_bounds__(128) pack_v_int4_kernel(PackArgs a, uint8_t* packed, float* scale, int64_t packed_bstride,
                                                          int64_t scale_bstride) {
  const int64_t i = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (i >= a.count) return;
  const int head = blockIdx.y, req = blockIdx.z, lane = threadIdx.x & 31;
  const int64_t s = a.index ? a.index[i] : i;
  const uint16_t* src = reinterpret_cast<const uint16_t*>(reinterpret_cast<const uint8_t*>(a.src) + req * a.src_bstride) +
                        ((int64_t)head * a.src_rows + s) * 128;
  const uint2 w = *reinterpret_cast<const uint2*>(src + 4 * lane);
  float x[4] = {raw_to_float<BF16>((uint16_t)(w.x & 0xffffu)), raw_to_float<BF16>((uint16_t)(w.x >> 16)),
                raw_to_float<BF16>((uint16_t)(w.y & 0xffffu)), raw_to_float<BF16>((uint16_t)(w.y >> 16))};
  float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
  const float sc = fmaxf(__fdiv_rn(amax, 7.f), 1.0e-6f);
  uint32_t out = 0;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int q = (int)fminf(fmaxf(rintf(__fdiv_rn(x[e], sc)), -7.f), 7.f);
    out |= (uint32_t)(q & 15) << (4 * e);
  }
  const int64_t row = (int64_t)head * a.capacity + a.dst_start + i;
  *reinterpret_cast<uint16_t*>(packed + req * packed_bstride + row * 64 + 2 * lane) = (uint16_t)out;
  if (lane == 0) *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scale) + req * scale_bstride + row * 4) = sc;
}

// ---- values: per-token, per-group affine INT2 ------------------------------
// One warp per (token, head, request); lane owns dims 4l..4l+3 (one output byte).
// int2_reference.py:96-151; fused_value_pack.py:72-149.
template <bool BF16>
__global__ void __launch_bounds__(128) pack_v_int2_kernel(PackArgs a, uint8_t* packed, __half* scale, uint8_t* zero,
                                                          int64_t packed_bstride, int64_t scale_bstride, int64_t zero_bstride,
                                                          int group) {
  launch_dependents();   // in a flush the ring kernel follows; it waits for this grid before it touches the ring
  const int64_t i = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (i < a.count) {
    const int head = blockIdx.y, req = blockIdx.z, lane = threadIdx.x & 31;
    const int64_t s = a.index ? a.index[i] : i;
    const uint16_t* src = reinterpret_cast<const uint16_t*>(reinterpret_cast<const uint8_t*>(a.src) + req * a.src_bstride) +
                          ((int64_t)head * a.src_rows + s) * 128;
    const uint2 w = *reinterpret_cast<const uint2*>(src + 4 * lane);
    float x[4] = {raw_to_float<BF16>((uint16_t)(w.x & 0xffffu)), raw_to_float<BF16>((uint16_t)(w.x >> 16)),
                  raw_to_float<BF16>((uint16_t)(w.y & 0xffffu)), raw_to_float<BF16>((uint16_t)(w.y >> 16))};
    float lo = fminf(fminf(x[0], x[1]), fminf(x[2], x[3]));
    float hi = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
    const int lanes = group / 4;  // lanes per group: 8, 16 or 32
    for (int d = 1; d < lanes; d <<= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, d));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, d));
    }
    lo = fminf(lo, 0.f);
    hi = fmaxf(hi, 0.f);
    const float sc = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), 3.f), 1.0e-6f);
    const float zp = fminf(fmaxf(rintf(__fdiv_rn(-lo, sc)), 0.f), 3.f);
    uint32_t out = 0;
  #pragma unroll
    for (int e = 0; e < 4; ++e) {
      const uint32_t q = (uint32_t)fminf(fmaxf(rintf(__fadd_rn(__fdiv_rn(x[e], sc), zp)), 0.f), 3.f);
      out |= q << (2 * e);
    }
    const int64_t row = (int64_t)head * a.capacity + a.dst_start + i;
    packed[req * packed_bstride + row * 32 + lane] = (uint8_t)out;
    if ((lane & (lanes - 1)) == 0) {
      const int groups = 128 / group;
      const int64_t m = row * groups + lane / lanes;
      reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(scale) + req * scale_bstride)[m] = __float2half_rn(sc);
      zero[req * zero_bstride + m] = (uint8_t)zp;
    }
  }
  // In a flush this grid runs beside the key pack in front of it.  The ring kernel behind it waits for this
  // grid only, so this grid must not complete before the key pack has: every thread passes here on its way out.
  grid_dependency_wait();
}

// ---- row gather (bf16-value pool) ------------------------------------------
__global__ void __launch_bounds__(128) gather_rows_kernel(const uint16_t* src, int64_t src_rows, const int64_t* index,
                                                          int64_t count, uint16_t* dst, int64_t dst_rows, int64_t dst_start) {
  const int64_t i = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (i >= count) return;
  const int head = blockIdx.y, lane = threadIdx.x & 31;
  const int64_t s = index ? index[i] : i;
  const uint2 w = *reinterpret_cast<const uint2*>(src + ((int64_t)head * src_rows + s) * 128 + 4 * lane);
  *reinterpret_cast<uint2*>(dst + ((int64_t)head * dst_rows + dst_start + i) * 128 + 4 * lane) = w;
}

// ---- host block copy ---------------------------------------------------------
// Brings a block of page-locked, device-mapped host memory into device memory with plain loads over PCIe, 16 bytes
// per thread.  A decode launched behind it with programmatic stream serialization runs its prologue and starts
// streaming the packed pools meanwhile; it reads the block only after this grid has completed.
__global__ void __launch_bounds__(256) host_block_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int n16) {
  launch_dependents();
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i < n16) dst[i] = src[i];
}

// ---- residual ring ----------------------------------------------------------
struct RingArgs {
  uint8_t* recent_k; uint8_t* recent_v; int32_t* recent_len;
  int64_t* recent_global; int64_t* recent_logical; int64_t* recent_page_lengths;
  int64_t k_bstride, v_bstride, len_bstride, global_bstride, logical_bstride, page_bstride;
  int num_heads, capacity, page_size;
};

// One-token append (triton_fourq_splitk.py:413-447).  grid (B), block 256: K/V rows of every head, then metadata.
__global__ void append_recent_kernel(RingArgs r, const uint8_t* new_k, const uint8_t* new_v, const int64_t* idx,
                                     int64_t global_index, int64_t logical_position) {
  const int b = blockIdx.x;
  int32_t* len_ptr = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(r.recent_len) + b * r.len_bstride);
  const int pos = *len_ptr;
  __syncthreads();  // everybody has read the length before thread 0 bumps it
  if (pos < r.capacity) {
    for (int i = threadIdx.x; i < r.num_heads * 16; i += blockDim.x) {  // 16-byte pieces
      const int h = i >> 4, piece = i & 15;
      const size_t s = ((size_t)b * r.num_heads + h) * 256 + 16 * piece;
      const size_t d = ((size_t)h * r.capacity + pos) * 256 + 16 * piece;
      *reinterpret_cast<uint4*>(r.recent_k + b * r.k_bstride + d) = *reinterpret_cast<const uint4*>(new_k + s);
      *reinterpret_cast<uint4*>(r.recent_v + b * r.v_bstride + d) = *reinterpret_cast<const uint4*>(new_v + s);
    }
    if (threadIdx.x == 0) {
      reinterpret_cast<int64_t*>(reinterpret_cast<uint8_t*>(r.recent_global) + b * r.global_bstride)[pos] = idx ? idx[2 * b] : global_index;
      reinterpret_cast<int64_t*>(reinterpret_cast<uint8_t*>(r.recent_logical) + b * r.logical_bstride)[pos] = idx ? idx[2 * b + 1] : logical_position;
      *len_ptr = pos + 1;
      reinterpret_cast<int64_t*>(reinterpret_cast<uint8_t*>(r.recent_page_lengths) + b * r.page_bstride)[pos / r.page_size] =
          pos % r.page_size + 1;
    }
  }
}

// After a flush: copy the flushed tokens' indices to the INT2 pool's metadata, slide the remaining rows
// to the front (each thread owns one 16-byte column and walks the rows in order, so overlapping
// ranges are safe), and refresh length and page lengths (dynamic_fourq_cache.py:108-117, 248-253).
__global__ void flush_ring_kernel(RingArgs r, int ring_tokens, int flush_tokens, int64_t* i2_global, int64_t* i2_logical,
                                  int64_t meta_bstride, int64_t meta_dst) {
  const int b = blockIdx.x;
  const int rest = ring_tokens - flush_tokens;
  int64_t* gl = reinterpret_cast<int64_t*>(reinterpret_cast<uint8_t*>(r.recent_global) + b * r.global_bstride);
  int64_t* lg = reinterpret_cast<int64_t*>(reinterpret_cast<uint8_t*>(r.recent_logical) + b * r.logical_bstride);
  if (i2_global != nullptr) {
    int64_t* dg = reinterpret_cast<int64_t*>(reinterpret_cast<uint8_t*>(i2_global) + b * meta_bstride) + meta_dst;
    int64_t* dl = reinterpret_cast<int64_t*>(reinterpret_cast<uint8_t*>(i2_logical) + b * meta_bstride) + meta_dst;
    for (int i = threadIdx.x; i < flush_tokens; i += blockDim.x) { dg[i] = gl[i]; dl[i] = lg[i]; }
  }
  grid_dependency_wait();   // the pack kernels read the rows that are moved and the length that is reset below
  __syncthreads();
  for (int col = threadIdx.x; col < r.num_heads * 16; col += blockDim.x) {
    const int h = col >> 4, piece = col & 15;
    uint8_t* kb = r.recent_k + b * r.k_bstride + (size_t)h * r.capacity * 256 + 16 * piece;
    uint8_t* vb = r.recent_v + b * r.v_bstride + (size_t)h * r.capacity * 256 + 16 * piece;
    for (int row = 0; row < rest; ++row) {
      *reinterpret_cast<uint4*>(kb + (size_t)row * 256) = *reinterpret_cast<const uint4*>(kb + (size_t)(row + flush_tokens) * 256);
      *reinterpret_cast<uint4*>(vb + (size_t)row * 256) = *reinterpret_cast<const uint4*>(vb + (size_t)(row + flush_tokens) * 256);
    }
  }
  if (threadIdx.x == 0) {
    for (int row = 0; row < rest; ++row) { gl[row] = gl[row + flush_tokens]; lg[row] = lg[row + flush_tokens]; }
    *reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(r.recent_len) + b * r.len_bstride) = rest;
    int64_t* pl = reinterpret_cast<int64_t*>(reinterpret_cast<uint8_t*>(r.recent_page_lengths) + b * r.page_bstride);
    for (int pg = 0; pg < r.capacity / r.page_size; ++pg) {
      const int v = rest - pg * r.page_size;
      pl[pg] = v < 0 ? 0 : (v > r.page_size ? r.page_size : v);
    }
  }
}

// ---------------------------------------------------------------------------
// Normalised 128-point Walsh-Hadamard transform of 16-bit rows, fp32 butterflies in the reference's stage order
// (stride 1, 2, ..., 64), result rounded to the element type.  One warp per row, four consecutive channels per
// lane: two stages in registers, five through shuffles.  In place when out == in.
// ---------------------------------------------------------------------------
template <bool BF16>
__global__ void fwht128_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, int64_t rows) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const uint2 raw = *reinterpret_cast<const uint2*>(in + row * 128 + 4 * lane);
  float r[4];
  if (BF16) {
    r[0] = __uint_as_float(raw.x << 16); r[1] = __uint_as_float(raw.x & 0xffff0000u);
    r[2] = __uint_as_float(raw.y << 16); r[3] = __uint_as_float(raw.y & 0xffff0000u);
  } else {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    r[0] = a.x; r[1] = a.y; r[2] = b.x; r[3] = b.y;
  }
  const float a = __fadd_rn(r[0], r[1]), b = __fsub_rn(r[0], r[1]), c = __fadd_rn(r[2], r[3]), d = __fsub_rn(r[2], r[3]);
  r[0] = __fadd_rn(a, c); r[1] = __fadd_rn(b, d); r[2] = __fsub_rn(a, c); r[3] = __fsub_rn(b, d);
#pragma unroll
  for (int sft = 1; sft < 32; sft <<= 1) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float o = __shfl_xor_sync(0xffffffffu, r[e], sft);
      r[e] = (lane & sft) ? __fsub_rn(o, r[e]) : __fadd_rn(r[e], o);
    }
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) r[e] = __fmul_rn(r[e], 0.08838834764831845f);
  uint2 pk;
  if (BF16) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(r[0], r[1]), hi = __floats2bfloat162_rn(r[2], r[3]);
    pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
  } else {
    __half2 lo = __floats2half2_rn(r[0], r[1]), hi = __floats2half2_rn(r[2], r[3]);
    pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
  }
  *reinterpret_cast<uint2*>(out + row * 128 + 4 * lane) = pk;
}

// ---------------------------------------------------------------------------
// Qwen multimodal rotary embedding of the query and key rows of a step, optionally followed by the 128-point
// Hadamard transform, in one launch: row (request, head, token) of q or k, out[d] = x[d] * cos[axis(d)] +
// rot(x)[d] * sin[axis(d)] with rot(x)[d] = -x[d + 64] (d < 64), x[d - 64] (d >= 64) and axis(d) chosen by the
// section of d mod 64.  fp32 arithmetic, products and sum rounded separately (as the elementwise CPU form),
// result rounded to the element type.  One warp per row, four consecutive channels per lane.
// ---------------------------------------------------------------------------
struct MropeArgs {
  const uint16_t* q; const uint16_t* k; uint16_t* q_out; uint16_t* k_out;
  const void* cos; const void* sin;
  int64_t cos_stride[4], sin_stride[4];   // elements: axis, request, token, channel
  int batch, hq, hkv, tokens, section0, section1, rot_dtype, hadamard;   // rot_dtype: R2K_DTYPE_* or 2 for float32
  // The whole prologue of a decode step (v != nullptr): the value rows pass through the same launch (copied, or
  // Hadamard-transformed when v_hadamard), and the three inputs may be slices of one fused projection: elements
  // between two requests' rows (a request's heads and tokens stay contiguous); the outputs are contiguous.
  const uint16_t* v; uint16_t* v_out;
  int64_t q_bstride, k_bstride, v_bstride;
  int v_hadamard;
};

__device__ __forceinline__ float load_rot(const void* base, int64_t index, int dtype) {
  if (dtype == 2) return reinterpret_cast<const float*>(base)[index];
  const uint16_t raw = reinterpret_cast<const uint16_t*>(base)[index];
  return dtype == R2K_DTYPE_BF16 ? __uint_as_float((uint32_t)raw << 16) : __half2float(__ushort_as_half(raw));
}

template <bool BF16>
__global__ void mrope_rows_kernel(MropeArgs a) {
  // The decode launch that follows on the stream may start its CTAs and prefetch pool tiles right away (it is
  // launched with programmatic stream serialization); it reads the rows written here only after its own
  // dependency wait, i.e. after this grid has completed.
  launch_dependents();
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = a.hq + a.hkv + (a.v != nullptr ? a.hkv : 0);
  if (row >= (int64_t)a.batch * heads * a.tokens) return;
  const int request = (int)(row / ((int64_t)heads * a.tokens));
  const int local = (int)(row - (int64_t)request * heads * a.tokens);
  const int head = local / a.tokens, token = local - head * a.tokens;
  const int which = head < a.hq ? 0 : (head < a.hq + a.hkv ? 1 : 2);   // query, key or value row
  const int h = which == 0 ? head : (which == 1 ? head - a.hq : head - a.hq - a.hkv);
  const int nh = which == 0 ? a.hq : a.hkv;
  const int64_t in_row = ((int64_t)h * a.tokens + token) * 128;
  const int64_t off = (((int64_t)request * nh + h) * a.tokens + token) * 128;   // in the contiguous output
  const uint16_t* src = which == 0 ? a.q + request * a.q_bstride : (which == 1 ? a.k + request * a.k_bstride : a.v + request * a.v_bstride);
  uint16_t* dst = which == 0 ? a.q_out : (which == 1 ? a.k_out : a.v_out);
  const uint2 raw = *reinterpret_cast<const uint2*>(src + in_row + 4 * lane);
  if (which == 2 && !a.v_hadamard) {   // a value row that is only brought into place
    *reinterpret_cast<uint2*>(dst + off + 4 * lane) = raw;
    return;
  }
  float x[4];
  if (BF16) {
    x[0] = __uint_as_float(raw.x << 16); x[1] = __uint_as_float(raw.x & 0xffff0000u);
    x[2] = __uint_as_float(raw.y << 16); x[3] = __uint_as_float(raw.y & 0xffff0000u);
  } else {
    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    x[0] = lo.x; x[1] = lo.y; x[2] = hi.x; x[3] = hi.y;
  }
  float r[4];
  if (which == 2) {
#pragma unroll
    for (int e = 0; e < 4; ++e) r[e] = x[e];
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int d = 4 * lane + e, sd = d & 63;
      const float other = __shfl_xor_sync(0xffffffffu, x[e], 16);   // channel d +- 64 lives 16 lanes away
      const float rotated = lane < 16 ? -other : other;
      const int axis = sd < a.section0 ? 0 : (sd < a.section0 + a.section1 ? 1 : 2);
      const float c = load_rot(a.cos, axis * a.cos_stride[0] + request * a.cos_stride[1] + token * a.cos_stride[2] + d * a.cos_stride[3],
                               a.rot_dtype);
      const float s = load_rot(a.sin, axis * a.sin_stride[0] + request * a.sin_stride[1] + token * a.sin_stride[2] + d * a.sin_stride[3],
                               a.rot_dtype);
      r[e] = __fmaf_rn(x[e], c, __fmul_rn(rotated, s));   // the reference's compiled form of x*cos + rot*sin: one product rounded, one fused
    }
  }
  if (which == 2 || a.hadamard) {
    const float p = __fadd_rn(r[0], r[1]), m = __fsub_rn(r[0], r[1]), c = __fadd_rn(r[2], r[3]), d = __fsub_rn(r[2], r[3]);
    r[0] = __fadd_rn(p, c); r[1] = __fadd_rn(m, d); r[2] = __fsub_rn(p, c); r[3] = __fsub_rn(m, d);
#pragma unroll
    for (int sft = 1; sft < 32; sft <<= 1) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float o = __shfl_xor_sync(0xffffffffu, r[e], sft);
        r[e] = (lane & sft) ? __fsub_rn(o, r[e]) : __fadd_rn(r[e], o);
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) r[e] = __fmul_rn(r[e], 0.08838834764831845f);
  }
  uint2 pk;
  if (BF16) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(r[0], r[1]), hi = __floats2bfloat162_rn(r[2], r[3]);
    pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
  } else {
    __half2 lo = __floats2half2_rn(r[0], r[1]), hi = __floats2half2_rn(r[2], r[3]);
    pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
  }
  *reinterpret_cast<uint2*>(dst + off + 4 * lane) = pk;
}

}  // namespace r2k
