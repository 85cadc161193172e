// Packed-KV GQA decode for sm_100a: one launch per decode step.
//
// Replaces the reference's three launches (tile partials, 64-way group
// reduce, final reduce + Hadamard + fused append;
// r2omni/sspa/kernels/triton_fourq_splitk.py:449-1020, 1243-1547).
//
// Shape of the kernel
//   * grid = one CTA per SM (rounded down to a whole number of CTAs per (request, kv head) when there are at
//     least two per head); every CTA owns a contiguous range of the flat tile list (request, kv head, pool,
//     tile), balanced by measured per-tile cost, and keeps ONE running (max, sum-exp, out) state per
//     (request, kv head) it crosses.
//   * warp 8 is the producer: one of its lanes streams each tile's key nibbles, key scale/zero rows, value bytes
//     and value metadata into a 4-stage shared-memory ring with bulk copies (TMA; a swizzled tensor map for
//     bf16 values) completing on mbarriers.  Warps 0-7 consume, one 32-token key block per warp and tile.
//   * tokens sit on the M axis of mma.sync.m16n8k16 and the (<= 8) query heads
//     of the GQA group on N, so no MMA lane is padding:
//       S^T[tok,head] = K[tok,ch] Q'^T[ch,head],  O^T[dim,head] += V^T[dim,tok] P^T[tok,head].
//   * INT4 codes are fed to the tensor core as fp16 *subnormals* (code * 2^-24
//     or code * 2^-20 straight out of an AND), so a key nibble costs 5/8 of an
//     ALU instruction.  Per-channel key scales are folded into Q' once per
//     32-token block as an exact two-term fp16 sum (hi + lo = q * scale), the zero points
//     are subtracted from the codes with one exact HSUB2 per register, per-token INT4-value scales are
//     folded into P, INT2 values are dequantised in registers.
//   * partial states go to a small workspace; the last CTA to finish a group of nine partials merges them, the
//     last group of a (request, kv head) merges the group results, writes the output, applies the optional
//     Hadamard epilogue and the fused append.
//   * the residual window is read in 64-token tiles, 16 tokens per warp, two tiles in work at once.
//
// Every wait is bounded: a wait that gives up records R2K_ERR_DEVICE_TIMEOUT in
// the workspace, the warp stops consuming and the kernel still terminates.
#pragma once

#include "decode.cuh"
#include "decode_consumer.cuh"
#include "device_utils.cuh"

namespace r2k {

namespace {

struct Tile {
  int pool;   // 0 bf16-V, 1 INT4-V, 2 INT2-V, 3 residual
  int win;    // first key-arena row of the window (pool 3: first ring row)
  int lo, hi; // valid rows of the window, [lo, hi) relative to win
};

__device__ __forceinline__ Tile tile_of(const DecodeParams& p, int u) {
  Tile t;
  int a0, a1, len;
  if (u < p.nF) {
    t.pool = 0; t.win = p.wF0 + u * kTF; a0 = p.g.k_off_fp; a1 = a0 + p.g.n_fp; len = kTF;
  } else if (u < p.nF + p.n4) {
    t.pool = 1; t.win = p.w40 + (u - p.nF) * kTQ; a0 = p.g.k_off_i4; a1 = a0 + p.g.n_i4; len = kTQ;
  } else if (u < p.nF + p.n4 + p.n2) {
    t.pool = 2; t.win = p.w20 + (u - p.nF - p.n4) * kTQ; a0 = p.g.k_off_i2; a1 = a0 + p.g.n_i2; len = kTQ;
  } else {
    t.pool = 3; t.win = (u - p.nF - p.n4 - p.n2) * kTR; a0 = 0; a1 = p.g.recent_capacity; len = kTR;
  }
  t.lo = max(a0 - t.win, 0);
  t.hi = min(a1 - t.win, len);
  return t;
}

// The unit range [u0,u1) of (request,kv head) `bh` inside a CTA's cost interval [c0, c1).
__device__ __forceinline__ void unit_range(const DecodeParams& p, const CostPos& c0, const CostPos& c1, int bh, int& u0, int& u1) {
  const uint32_t lo = bh == c0.bh ? c0.r : 0u;
  const uint32_t hi = bh == c1.bh ? c1.r : p.c_bh;
  u0 = units_before(p, lo);
  u1 = units_before(p, hi);
}

template <bool BF16>
__device__ __forceinline__ float elem_to_float(uint16_t raw) {
  if (BF16) return __uint_as_float((uint32_t)raw << 16);
  return __half2float(__ushort_as_half(raw));
}

// ---------------------------------------------------------------------------
// producer
// ---------------------------------------------------------------------------
__device__ __forceinline__ void copy_piece(uint8_t* dst, const uint8_t* src, int bytes, uint64_t* bar, int lane,
                                           uint32_t& tx) {
  if (bytes <= 0) return;
  if ((((uintptr_t)src | (uintptr_t)smem_u32(dst) | (uint32_t)bytes) & 15u) == 0) {
    if (lane == 0) { bulk_g2s(dst, src, (uint32_t)bytes, bar); tx += (uint32_t)bytes; }
  } else {  // ragged edge: plain loads
    for (int i = lane; i < bytes; i += 32) dst[i] = src[i];
  }
}
__device__ __forceinline__ void zero_piece(uint8_t* dst, int bytes, int lane) {
  for (int i = lane; i < bytes; i += 32) dst[i] = 0;
}

// Rows [lo, hi) of a bf16-value tile written into the swizzled half boxes by plain loads (ragged tiles, unaligned
// pools): `src` addresses row lo.  Rows outside [lo, hi) are cleared, so a masked row never feeds a NaN.
__device__ __forceinline__ void copy_fp_rows(uint8_t* vreg, const uint8_t* src, int lo, int hi, int len, int lane) {
  const int chunks = (hi - lo) * 16;
  if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
    for (int i = lane; i < chunks; i += 32)
      *reinterpret_cast<uint4*>(vreg + fp_box_offset(lo + (i >> 4), i & 15)) = __ldg(reinterpret_cast<const uint4*>(src) + i);
  } else {
    for (int i = lane; i < chunks * 16; i += 32) vreg[fp_box_offset(lo + (i >> 8), (i >> 4) & 15) + (i & 15)] = src[i];
  }
  for (int half = 0; half < 2; ++half) {
    zero_piece(vreg + half * kFpHalfBytes, lo * 128, lane);
    zero_piece(vreg + half * kFpHalfBytes + hi * 128, (len - hi) * 128, lane);
  }
}

__device__ __forceinline__ void produce_tile(const DecodeParams& p, const Tile& tl, int b, int h, uint8_t* stage,
                                             uint64_t* bar, int lane) {
  uint32_t tx = 0;
  const R2KCacheView& v = p.v;
  const int nvalid = tl.hi - tl.lo;
  if (tl.pool == 3) {
    const size_t row = ((size_t)h * p.g.recent_capacity + tl.win) * 256;
    copy_piece(stage + kOffV, (const uint8_t*)v.recent_k + (size_t)b * v.recent_k_bstride + row, nvalid * 256, bar, lane, tx);
    copy_piece(stage + kOffV + kOffRecentV, (const uint8_t*)v.recent_v + (size_t)b * v.recent_v_bstride + row, nvalid * 256,
               bar, lane, tx);
    if (nvalid < kTR) {
      zero_piece(stage + kOffV + nvalid * 256, (kTR - nvalid) * 256, lane);
      zero_piece(stage + kOffV + kOffRecentV + nvalid * 256, (kTR - nvalid) * 256, lane);
    }
  } else {
    const int len = tl.pool == 0 ? kTF : kTQ;
    // keys: the whole window, clipped to the arena (its capacity is a multiple of 128 rows, not of the tile)
    const int krows = min(len, p.g.k_capacity - tl.win);
    copy_piece(stage + off_k(tl.pool), v.k_packed + (size_t)b * v.k_packed_bstride + ((size_t)h * p.g.k_capacity + tl.win) * 64,
               krows * 64, bar, lane, tx);
    const int blk0 = tl.win >> p.kblock_shift;
    const int nblk = min(max(1, len >> p.kblock_shift), (p.g.k_capacity >> p.kblock_shift) - blk0);
    const size_t meta = (size_t)h * (p.g.k_capacity >> p.kblock_shift) + blk0;
    copy_piece(stage + off_ks(tl.pool), (const uint8_t*)v.k_scale + (size_t)b * v.k_scale_bstride + meta * 256, nblk * 256, bar, lane, tx);
    copy_piece(stage + off_kz(tl.pool), v.k_zero + (size_t)b * v.k_zero_bstride + meta * 128, nblk * 128, bar, lane, tx);
    // values: only rows of this pool; rows of the window outside it are cleared
    uint8_t* vreg = stage + kOffV;
    if (tl.pool == 0) {
      const size_t row = (size_t)h * p.g.fp_capacity + (tl.win + tl.lo - p.g.k_off_fp);
      copy_fp_rows(vreg, (const uint8_t*)v.fp_v + (size_t)b * v.fp_v_bstride + row * 256, tl.lo, tl.hi, len, lane);
    } else if (tl.pool == 1) {
      const size_t row = (size_t)h * p.g.i4_capacity + (tl.win + tl.lo - p.g.k_off_i4);
      copy_piece(vreg + tl.lo * 64, v.i4_packed + (size_t)b * v.i4_packed_bstride + row * 64, nvalid * 64, bar, lane, tx);
      copy_piece(vreg + kOffI4Scale + tl.lo * 4, (const uint8_t*)v.i4_scale + (size_t)b * v.i4_scale_bstride + row * 4,
                 nvalid * 4, bar, lane, tx);
      if (nvalid < len) {
        zero_piece(vreg + kOffI4Scale, tl.lo * 4, lane);
        zero_piece(vreg + kOffI4Scale + tl.hi * 4, (len - tl.hi) * 4, lane);
      }
    } else {
      const size_t row = (size_t)h * p.g.i2_capacity + (tl.win + tl.lo - p.g.k_off_i2);
      const int g2 = p.groups2;
      copy_piece(vreg + tl.lo * 32, v.i2_packed + (size_t)b * v.i2_packed_bstride + row * 32, nvalid * 32, bar, lane, tx);
      copy_piece(vreg + kOffI2Scale + tl.lo * g2 * 2, (const uint8_t*)v.i2_scale + (size_t)b * v.i2_scale_bstride + row * g2 * 2,
                 nvalid * g2 * 2, bar, lane, tx);
      copy_piece(vreg + kOffI2Zero + tl.lo * g2, v.i2_zero + (size_t)b * v.i2_zero_bstride + row * g2, nvalid * g2, bar, lane, tx);
      if (nvalid < len) {
        zero_piece(vreg + kOffI2Scale, tl.lo * g2 * 2, lane);
        zero_piece(vreg + kOffI2Scale + tl.hi * g2 * 2, (len - tl.hi) * g2 * 2, lane);
      }
    }
  }
  __syncwarp();
  if (lane == 0) mbar_arrive_expect_tx(bar, tx);
}

// Per-(request, kv head) source bases, biased so that a key-arena row index addresses every array of its pool.
struct TileSources {
  const uint8_t* kp; const uint8_t* ks; const uint8_t* kz;
  const uint8_t* v0; const uint8_t* v1; const uint8_t* v2;   // value payload of pools 0..2
  const uint8_t* s1;       // INT4-value scales
  const uint8_t* s2;       // INT2-value scales
  const uint8_t* z2;       // INT2-value zero points
  bool fast1, fast2;       // every full tile of the pool can go through 16-byte-aligned bulk copies
};

__device__ __forceinline__ TileSources tile_sources(const DecodeParams& p, int b, int h) {
  const R2KCacheView& v = p.v;
  TileSources s;
  const int64_t hb = h;
  s.kp = v.k_packed + (int64_t)b * v.k_packed_bstride + hb * p.g.k_capacity * 64;
  s.ks = (const uint8_t*)v.k_scale + (int64_t)b * v.k_scale_bstride + hb * (p.g.k_capacity >> p.kblock_shift) * 256;
  s.kz = v.k_zero + (int64_t)b * v.k_zero_bstride + hb * (p.g.k_capacity >> p.kblock_shift) * 128;
  const int64_t r0 = hb * p.g.fp_capacity - p.g.k_off_fp, r1 = hb * p.g.i4_capacity - p.g.k_off_i4,
                r2 = hb * p.g.i2_capacity - p.g.k_off_i2;
  s.v0 = (const uint8_t*)v.fp_v + (int64_t)b * v.fp_v_bstride + r0 * 256;
  s.v1 = v.i4_packed + (int64_t)b * v.i4_packed_bstride + r1 * 64;
  s.v2 = v.i2_packed + (int64_t)b * v.i2_packed_bstride + r2 * 32;
  s.s1 = (const uint8_t*)v.i4_scale + (int64_t)b * v.i4_scale_bstride + r1 * 4;
  s.s2 = (const uint8_t*)v.i2_scale + (int64_t)b * v.i2_scale_bstride + r2 * p.groups2 * 2;
  s.z2 = v.i2_zero + (int64_t)b * v.i2_zero_bstride + r2 * p.groups2;
  // full tiles start at multiples of 64 rows, so base alignment decides everything
  s.fast1 = ((((uintptr_t)s.v1) | ((uintptr_t)s.s1)) & 15) == 0;
  s.fast2 = ((((uintptr_t)s.v2) | ((uintptr_t)s.s2) | ((uintptr_t)s.z2)) & 15) == 0 && p.groups2 == 4;
  return s;
}

// A full, aligned tile: one lane issues the bulk copies; no per-lane work, no 64-bit multiplies.
__device__ __forceinline__ void produce_full_tile(const DecodeParams& p, const TileSources& src, int pool, int win, int b,
                                                  int h, uint8_t* stage, uint64_t* bar) {
  const int len = pool == 0 ? kTF : kTQ;
  const int nblk = max(1, len >> p.kblock_shift);
  const int blk0 = win >> p.kblock_shift;
  uint32_t tx = (uint32_t)(len * 64 + nblk * 384);
  tx += pool == 0 ? (uint32_t)(len * 256) : pool == 1 ? (uint32_t)(len * 68) : (uint32_t)(len * 44);
  mbar_arrive_expect_tx(bar, tx);
  bulk_g2s(stage + off_k(pool), src.kp + (size_t)win * 64, (uint32_t)(len * 64), bar);
  bulk_g2s(stage + off_ks(pool), src.ks + (size_t)blk0 * 256, (uint32_t)(nblk * 256), bar);
  bulk_g2s(stage + off_kz(pool), src.kz + (size_t)blk0 * 128, (uint32_t)(nblk * 128), bar);
  if (pool == 0) {   // two 64-channel boxes of kTF rows, 128-byte swizzle
    const int row = win - p.g.k_off_fp;
    tensor_g2s_4d(stage + kOffV, &p.fp_map, 0, row, h, b, bar);
    tensor_g2s_4d(stage + kOffV + kFpHalfBytes, &p.fp_map, 64, row, h, b, bar);
  } else if (pool == 1) {
    bulk_g2s(stage + kOffV, src.v1 + (size_t)win * 64, (uint32_t)(len * 64), bar);
    bulk_g2s(stage + kOffV + kOffI4Scale, src.s1 + (size_t)win * 4, (uint32_t)(len * 4), bar);
  } else {
    bulk_g2s(stage + kOffV, src.v2 + (size_t)win * 32, (uint32_t)(len * 32), bar);
    bulk_g2s(stage + kOffV + kOffI2Scale, src.s2 + (size_t)win * 8, (uint32_t)(len * 8), bar);
    bulk_g2s(stage + kOffV + kOffI2Zero, src.z2 + (size_t)win * 4, (uint32_t)(len * 4), bar);
  }
}

}  // namespace

// Exact merge of `count` partial rows (max, sum, out[128]) of head hh; this thread owns dims 8*sub .. 8*sub+7.
// Row `own` (or -1) is not loaded: the caller still holds it in registers (om, ol, oacc), which saves the merging
// CTA a dependent round trip to memory for the common nine-partial head.  Rows are folded in slot order in
// batches of nine slots, whoever merges, so the result does not depend on which CTA arrived last.
constexpr int kMergeBatch = kMergeGroup;
__device__ __forceinline__ void merge_rows(const float* base, int count, int own, float om, float ol, const float (&oacc)[8],
                                           int hh, int sub, float& mx, float& lsum, float (&acc)[8]) {
  mx = -INFINITY;
  lsum = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  for (int q0 = 0; q0 < count; q0 += kMergeBatch) {
    float2 ml[kMergeBatch];
    float4 va[kMergeBatch], vb[kMergeBatch];
#pragma unroll
    for (int k = 0; k < kMergeBatch; ++k) {
      const int q = q0 + k;
      if (q == own) {
        ml[k] = make_float2(om, ol);
        va[k] = make_float4(oacc[0], oacc[1], oacc[2], oacc[3]);
        vb[k] = make_float4(oacc[4], oacc[5], oacc[6], oacc[7]);
      } else {
        const float* row = base + (size_t)min(q, count - 1) * kSlotFloats + hh * kRowFloats;
        ml[k] = __ldcg(reinterpret_cast<const float2*>(row));
        va[k] = __ldcg(reinterpret_cast<const float4*>(row + 4 + 8 * sub));
        vb[k] = __ldcg(reinterpret_cast<const float4*>(row + 8 + 8 * sub));
      }
    }
    float bm = mx;   // running reference point: rescale what is already accumulated when a batch raises it
#pragma unroll
    for (int k = 0; k < kMergeBatch; ++k) bm = fmaxf(bm, (q0 + k < count) ? ml[k].x : -INFINITY);
    if (bm > mx) {
      const float f = mx == -INFINITY ? 0.f : ex2_approx(mx - bm);
      lsum *= f;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] *= f;
      mx = bm;
    }
#pragma unroll
    for (int k = 0; k < kMergeBatch; ++k) {
      const float w = (q0 + k < count && ml[k].x != -INFINITY) ? ex2_approx(ml[k].x - mx) : 0.f;
      acc[0] += w * va[k].x; acc[1] += w * va[k].y; acc[2] += w * va[k].z; acc[3] += w * va[k].w;
      acc[4] += w * vb[k].x; acc[5] += w * vb[k].y; acc[6] += w * vb[k].z; acc[7] += w * vb[k].w;
      lsum += w * ml[k].y;
    }
  }
}

__device__ __forceinline__ void store_row(float* slot, int hh, int sub, float mx, float lsum, const float (&acc)[8]) {
  float* orow = slot + hh * kRowFloats;
  __stcg(reinterpret_cast<float4*>(orow + 4 + 8 * sub), make_float4(acc[0], acc[1], acc[2], acc[3]));
  __stcg(reinterpret_cast<float4*>(orow + 8 + 8 * sub), make_float4(acc[4], acc[5], acc[6], acc[7]));
  if (sub == 0) __stcg(reinterpret_cast<float2*>(orow), make_float2(mx, lsum));
}

// Normalise (or emit the raw state), optional Hadamard, store.  16 threads per head, 8 dims each.
template <bool BF16>
__device__ __forceinline__ void write_output(const DecodeParams& p, size_t orow, bool valid, int sub, float mx, float lsum,
                                             const float (&acc)[8]) {
  // every lane takes part in the shuffles below; `valid` only guards the stores (padding heads of GQA < 8)
  if (p.flags & R2K_FLAG_OUT_STATE) {
    if (!valid) return;
    float* o = reinterpret_cast<float*>(p.out) + orow * 130;
    if (sub == 0) { o[0] = mx * kLn2; o[1] = lsum; }
#pragma unroll
    for (int e = 0; e < 8; e += 2) *reinterpret_cast<float2*>(o + 2 + 8 * sub + e) = make_float2(acc[e], acc[e + 1]);
    return;
  }
  const float inv = 1.f / lsum;
  float r[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) r[e] = acc[e] * inv;
  if (p.flags & R2K_FLAG_OUTPUT_HADAMARD) {
#pragma unroll
    for (int e = 0; e < 8; ++e)  // round through the element type first, as the reference does
      r[e] = BF16 ? __bfloat162float(__float2bfloat16_rn(r[e])) : __half2float(__float2half_rn(r[e]));
#pragma unroll
    for (int span = 1; span < 8; span <<= 1) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if ((e & span) == 0) { const float a = r[e], c = r[e + span]; r[e] = a + c; r[e + span] = a - c; }
      }
    }
#pragma unroll
    for (int sft = 1; sft < 16; sft <<= 1) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float o2 = __shfl_xor_sync(0xffffffffu, r[e], sft);
        r[e] = (sub & sft) ? (o2 - r[e]) : (r[e] + o2);
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) r[e] *= 0.08838834764831845f;
  }
  if (!valid) return;
  if (p.flags & R2K_FLAG_OUT_F32) {
    float* o = reinterpret_cast<float*>(p.out) + orow * kD + 8 * sub;
    *reinterpret_cast<float4*>(o) = make_float4(r[0], r[1], r[2], r[3]);
    *reinterpret_cast<float4*>(o + 4) = make_float4(r[4], r[5], r[6], r[7]);
  } else {
    uint4 pk;
    if (BF16) { pk.x = pack_bf16x2(r[0], r[1]); pk.y = pack_bf16x2(r[2], r[3]); pk.z = pack_bf16x2(r[4], r[5]); pk.w = pack_bf16x2(r[6], r[7]); }
    else { pk.x = pack_f16x2(r[0], r[1]); pk.y = pack_f16x2(r[2], r[3]); pk.z = pack_f16x2(r[4], r[5]); pk.w = pack_f16x2(r[6], r[7]); }
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.out) + orow * kD + 8 * sub) = pk;
  }
}

// Step counter of the fused cross-rank merge: given by the host, or (xseq == 0) kept on the device behind the
// state words of this rank's exchange buffer, so that a captured graph can be replayed.  Every reader sees the value
// of the previous step; the CTA that counts in last moves it on (exchange_count_in).
__device__ __forceinline__ uint32_t* exchange_counter(const DecodeParams& p) {
  return reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(p.xbuf[p.xrank]) + p.xflags_off);
}
__device__ __forceinline__ uint32_t exchange_step(const DecodeParams& p) {
  if (p.xseq != 0) return p.xseq;
  const uint32_t s = *reinterpret_cast<volatile uint32_t*>(exchange_counter(p)) + 1u;
  return s == 0 ? 1u : s;
}

// Hand-over of the device-side step counter: every CTA has read the counter (after the previous launch completed)
// before it counts in, so the CTA that counts in last may move the counter on for the next launch while this one
// is still streaming -- nothing of it is left for the end of the kernel.
__device__ __forceinline__ void exchange_count_in(const DecodeParams& p, uint32_t step) {
  uint32_t* ctr = exchange_counter(p);
  if (atomicAdd(ctr + 1, 1u) == (uint32_t)p.grid - 1u) {
    ctr[1] = 0u;
    ctr[0] = step;
  }
}

// Fused cross-rank merge of one (request, kv head), run by the head's last-arriving CTA on every rank.  Every
// state value travels as an 8-byte (value, step) word: the CTA stores this rank's rows into every rank's
// exchange buffer (plain peer stores over NVLink), then polls the ranks' rows in the local buffer until every
// word carries this step's tag (bounded), and the 128 workers fold the rows in rank order.  No fence, no
// separate flag, no barrier.  A buffer holds two halves (step parity) of [world][rows][130] words; the tag makes a
// stale word of an older step unmistakable.  On return (lsum, acc) hold the merged state; the caller normalises
// and stores as usual.
// Not inlined: it runs once per (request, kv head) and must not cost the streaming loop any registers.
static_assert(R2K_MAX_RANKS * 8 * 130 * 4 <= kScratchBytes, "every rank's rows of one head group fit the merge scratch");
__device__ __noinline__ void exchange_merge(const DecodeParams& p, uint32_t seq, size_t orow, int hh, bool worker, int sub,
                                               float* staging, float mx, float& lsum, float (&acc)[8]) {
  const bool valid = hh < p.gqa;
  const uint32_t par = seq & 1u;
  const size_t rows = (size_t)p.g.batch * p.g.num_q_heads;
  // Send side.  The workers lay this head group's rows out in shared memory as [gqa][130] floats; then all
  // consumer threads copy them to every rank, consecutive threads writing consecutive 16-byte pairs of tagged
  // words: a warp's store covers four whole 128-byte lines of the peer's buffer.  (Stores of one thread's own
  // eight channels would touch sixteen lines per instruction and take several times as long to leave the SM.)
  if (worker && valid) {
    float* r = staging + hh * 130;
    if (sub == 0) *reinterpret_cast<float2*>(r) = make_float2(mx * kLn2, lsum);
#pragma unroll
    for (int e = 0; e < 8; e += 2) *reinterpret_cast<float2*>(r + 2 + 8 * sub + e) = make_float2(acc[e], acc[e + 1]);
  }
  named_bar_sync(1, kConsumers);
  {
    const uint32_t pairs = (uint32_t)p.gqa * 65u;   // 16-byte pairs of tagged words per rank
    const size_t first = ((size_t)(par * p.xw + p.xrank) * rows + (orow - hh)) * 130;
    const float2* src = reinterpret_cast<const float2*>(staging);
#pragma unroll 4
    for (uint32_t i = threadIdx.x; i < pairs * (uint32_t)p.xw; i += kConsumers) {
      const uint32_t r = i / pairs, c = i - r * pairs;
      const float2 v = src[c];
      st_tagged2_sys(reinterpret_cast<uint2*>(p.xbuf[r]) + first + 2 * c, __float_as_uint(v.x), __float_as_uint(v.y), seq);
    }
  }
  // Receive side.  All consumer threads bring the ranks' rows of this head group from the local exchange buffer
  // into shared memory, eight 16-byte loads in flight per thread and poll; a pair counts when both of its words
  // carry this step's tag.  Polls are bounded: kExchangePolls rounds with p.xnap nanoseconds of sleep between them (about
  // 1.3 s by default: ranks may be skewed by host work).
  named_bar_sync(1, kConsumers);   // the send loop has read the staged rows: the space is reused
  {
    const uint32_t pairs = (uint32_t)p.gqa * 65u, total = pairs * (uint32_t)p.xw;
    const uint2* base = reinterpret_cast<const uint2*>(p.xbuf[p.xrank]) + ((size_t)(par * p.xw) * rows + (orow - hh)) * 130;
    const size_t pitch = rows * 130;   // words between two ranks' copies of a row
    float2* dst = reinterpret_cast<float2*>(staging);
    bool timed_out = false;
    const uint32_t nap = p.xnap;   // nanoseconds between two polls once the first 256 quick ones are spent
#pragma unroll 1
    for (uint32_t i0 = threadIdx.x; i0 < total; i0 += 8 * kConsumers) {
      uint4 w[8];
      bool ok = false;
      for (uint32_t it = 0; it < kExchangePolls && !ok; ++it) {
        if (it) __nanosleep(it < 256 ? 100 : nap);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t i = min(i0 + k * kConsumers, total - 1u), r = i / pairs, c = i - r * pairs;
          w[k] = ld_tagged2_sys(base + r * pitch + 2 * c);
        }
        ok = true;
#pragma unroll
        for (int k = 0; k < 8; ++k) ok = ok && w[k].y == seq && w[k].w == seq;
      }
      timed_out = timed_out || !ok;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t i = i0 + k * kConsumers;
        if (i < total) dst[i] = make_float2(__uint_as_float(w[k].x), __uint_as_float(w[k].z));
      }
      if (!ok) {
        // A pair that never arrived (the wait ran out) is taken as the state of a rank without tokens:
        // (max, sum) = (-inf, 0), values 0.  The output then is the merge of the ranks that did arrive: finite.
#pragma unroll 1
        for (int k = 0; k < 8; ++k) {
          const uint32_t i = i0 + k * kConsumers;
          if (i >= total) break;
          const uint32_t r = i / pairs, c = i - r * pairs;
          const uint4 v = ld_tagged2_sys(base + r * pitch + 2 * c);
          if (v.y != seq || v.w != seq) dst[i] = (c % 65u == 0u) ? make_float2(-INFINITY, 0.f) : make_float2(0.f, 0.f);
          else dst[i] = make_float2(__uint_as_float(v.x), __uint_as_float(v.z));
        }
      }
    }
    if (timed_out) atomicExch(p.err, R2K_ERR_DEVICE_TIMEOUT);
  }
  named_bar_sync(1, kConsumers);
  if (!worker || !valid) return;
  // fold the ranks' rows in rank order around the common maximum
  const int rank_floats = p.gqa * 130;
  const float* mine = staging + hh * 130;
  float m_all = -INFINITY, l = 0.f;
  for (int r = 0; r < p.xw; ++r) m_all = fmaxf(m_all, mine[r * rank_floats]);
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  for (int r = 0; r < p.xw; ++r) {
    const float* row = mine + r * rank_floats;
    const float mk = row[0];
    const float wgt = (mk == -INFINITY) ? 0.f : __expf(mk - m_all);
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
      const float2 v = *reinterpret_cast<const float2*>(row + 2 + 8 * sub + e);
      acc[e] += wgt * v.x;
      acc[e + 1] += wgt * v.y;
    }
    l += wgt * row[1];
  }
  lsum = l;
}

// One warp's 32-token key block of a tile: scores, softmax update, value accumulation.
template <int POOL, bool PARTIAL, bool BF16>
__device__ __forceinline__ void consume_block(WarpState& st, uint32_t sb, const LaneOffsets& o, const uint32_t (&qh)[16],
                                              float alpha, int t, int pg, int step, int lo, int hi) {
  float s[2][4];
  qk_int4(sb, o, qh, alpha, s);
  if (PARTIAL) { mask_scores(s[0], pg, lo, hi); mask_scores(s[1], 16 + pg, lo, hi); }
  softmax_update<2>(st, s);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    if (POOL == 0) pv_fp<BF16, true>(st, sb, o.va, o.vb, j, s[j]);
    else if (POOL == 1) pv_int4<PARTIAL>(st, sb, o, j, s[j], pg, lo, hi);
    else pv_int2<PARTIAL>(st, sb, o, j, s[j], t, step, lo, hi);
  }
}

// All tiles [ua, ub) of one value pool for one (request, kv head): the lane offsets are computed once here.
// INT4-/INT2-value tiles hold kTQ tokens, one key block per warp.  bf16-value tiles hold kTF = kTQ/2 tokens;
// the lower half of the warps takes even tiles and the upper half odd ones, so every warp still works on 32
// tokens at a time and pays the per-block work (Q' and the zero-point chain) once per 32 tokens.
template <int POOL, bool BF16>
__device__ __forceinline__ void consume_pool(WarpState& st, const DecodeParams& p, int ua, int ub, int first, uint32_t stage0,
                                             uint64_t* full_bar, uint64_t* empty_bar, int& stage, uint32_t& phase, bool& alive,
                                             const uint32_t (&qh)[16], int warp, int lane) {
  if (ua >= ub) return;
  const int g = lane >> 2, t = lane & 3, pg = pi_row(g);
  constexpr int kLen = POOL == 0 ? kTF : kTQ;
  constexpr int kHalf = kNW / 2;
  const int a0 = POOL == 0 ? p.g.k_off_fp : POOL == 1 ? p.g.k_off_i4 : p.g.k_off_i2;
  const int a1 = a0 + (POOL == 0 ? p.g.n_fp : POOL == 1 ? p.g.n_i4 : p.g.n_i2);
  const int w0 = POOL == 0 ? p.wF0 : POOL == 1 ? p.w40 : p.w20;
  const int slice = 32 * (POOL == 0 ? warp % kHalf : warp);
  const int t0 = 2 * t + (t & 1), t1 = 2 * t + 1 - (t & 1);
  const int blk = slice >> p.kblock_shift;   // windows start on multiples of the largest key block
  LaneOffsets o;
  o.k = off_k(POOL) + (slice + pg) * 64 + 16 * t;
  o.ks = off_ks(POOL) + blk * 256 + 64 * t;
  o.kz = off_kz(POOL) + blk * 128 + 32 * t;
  int step = 0;
  if (POOL == 0) {
    o.va = kOffV + fp_box_offset(slice + t0, 2 * g);   // swizzled half boxes
    o.vb = kOffV + fp_box_offset(slice + t1, 2 * g);
    o.m0 = o.m1 = 0;
  } else if (POOL == 1) {
    o.va = kOffV + (slice + t0) * 64 + 8 * g; o.vb = kOffV + (slice + t1) * 64 + 8 * g;
    o.m0 = kOffV + kOffI4Scale + (slice + pg) * 4; o.m1 = 0;
  } else {
    step = 2 * p.groups2;
    const int grp = (16 * g) >> p.group2_shift;
    o.va = kOffV + (slice + t0) * 32 + 4 * g; o.vb = kOffV + (slice + t1) * 32 + 4 * g;
    o.m0 = kOffV + kOffI2Scale + (slice + t0) * step + 2 * grp;
    o.m1 = kOffV + kOffI2Zero + (slice + t0) * (step >> 1) + grp;
  }
  set_units(st, POOL == 1 ? 1 : 0);
  const int parity = warp >= kHalf ? 1 : 0;
  int lo_edge = a0 - (w0 + (ua - first) * kLen) - slice;   // validity window of this warp's slice, slides with the tile
  int hi_edge = a1 - (w0 + (ua - first) * kLen) - slice;
  for (int u = ua; u < ub; ++u, lo_edge -= kLen, hi_edge -= kLen) {
    if (alive && !mbar_wait(&full_bar[stage], phase)) {
      if (lane == 0) atomicExch(p.err, R2K_ERR_DEVICE_TIMEOUT);
      alive = false;
    }
    if (alive) {
      if (POOL != 0 || ((u & 1) == parity)) {
        const uint32_t sb = stage0 + stage * kStageBytes;
        if (lo_edge <= 0 && hi_edge >= 32) consume_block<POOL, false, BF16>(st, sb, o, qh, p.qscale, t, pg, step, 0, 32);
        else if (min(hi_edge, 32) > max(lo_edge, 0))
          consume_block<POOL, true, BF16>(st, sb, o, qh, p.qscale, t, pg, step, max(lo_edge, 0), min(hi_edge, 32));
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
    }
    if (++stage == kStages) { stage = 0; phase ^= 1u; }
  }
}

// ---------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------
template <bool BF16>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) decode_kernel(const __grid_constant__ DecodeParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* stages = smem;
  float* scratch = reinterpret_cast<float*>(smem + kStages * kStageBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes + kScratchBytes);
  uint64_t* empty_bar = full_bar + kStages;
  int* flags = reinterpret_cast<int*>(empty_bar + kStages);  // [0] last-arriver flag

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  // The packed pools are never written by a decode launch, so the next decode of the stream may start streaming
  // them as soon as SMs fall free.  Everything a previous kernel can have written (query, appended rows, residual
  // window and its length, split-K workspace) is read only after grid_dependency_wait().
  launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], kNW); }
    mbar_fence_init();
  }
  __syncthreads();

  const CostPos c0 = cta_pos(p, cta), c1 = cta_pos(p, cta + 1);
  const int bh_lo = c0.bh;
  int bh_hi = c1.r > 0 ? c1.bh : c1.bh - 1;
  if (bh_hi > p.bh_total - 1) bh_hi = p.bh_total - 1;
  const bool has_append = p.app_k != nullptr;

  int stage = 0;
  uint32_t phase = 0;

  if (warp == kNW) {
    // ------------------------------ producer ------------------------------
    bool alive = true;
    for (int bh = bh_lo; bh <= bh_hi && alive; ++bh) {
      const int b = bh / p.g.num_kv_heads, h = bh - b * p.g.num_kv_heads;
      int u0, u1;
      unit_range(p, c0, c1, bh, u0, u1);
      int rlen = -1;   // read only when a residual-window tile comes up: keeps the load off the path to the first copy
      const TileSources src = tile_sources(p, b, h);
      for (int u = u0; u < u1; ++u) {
        const Tile tl = tile_of(p, u);
        if (tl.pool == 3) {
          if (rlen < 0) {
            grid_dependency_wait();   // the ring and its length belong to the previous step until it has completed
            rlen = *reinterpret_cast<const int*>((const uint8_t*)p.v.recent_len + (size_t)b * p.v.recent_len_bstride) +
                   (has_append ? 1 : 0);
          }
          if (tl.win >= rlen) continue;
        }
        if (!mbar_wait_relaxed(&empty_bar[stage], phase ^ 1u)) {
          if (lane == 0) atomicExch(p.err, R2K_ERR_DEVICE_TIMEOUT);
          alive = false;
          break;
        }
        uint8_t* sb = stages + stage * kStageBytes;
        const bool full = tl.pool < 3 && tl.lo == 0 && tl.hi == (tl.pool == 0 ? kTF : kTQ) &&
                          (tl.pool == 0 ? p.fp_tma != 0 : tl.pool == 1 ? src.fast1 : src.fast2);
        if (full) {
          if (lane == 0) produce_full_tile(p, src, tl.pool, tl.win, b, h, sb, &full_bar[stage]);
        } else {
          produce_tile(p, tl, b, h, sb, &full_bar[stage], lane);
        }
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
    return;
  }

  // -------------------------------- consumers --------------------------------
  const int g = lane >> 2, t = lane & 3, pg = pi_row(g);
  bool alive = true;
  WarpState st;
  // the partition arithmetic of the first (request, kv head) needs nothing a previous kernel wrote: done while
  // that kernel is still finishing, it is off the path from the dependency wait to the first tile
  int first_u0 = 0, first_u1 = 0, first_part0 = 0, first_nparts = 1;
  if (bh_lo <= bh_hi) {
    unit_range(p, c0, c1, bh_lo, first_u0, first_u1);
    first_part0 = first_cta_of(p, bh_lo);
    first_nparts = last_cta_of(p, bh_lo) - first_part0 + 1;
  }
  grid_dependency_wait();
  // step tag of the fused cross-rank merge: read once, here, by everybody (see the counter hand-over below)
  const uint32_t xstep = p.xw > 1 ? exchange_step(p) : 0u;
  const bool xcount = p.xw > 1 && p.xseq == 0 && threadIdx.x == 0;

  for (int bh = bh_lo; bh <= bh_hi; ++bh) {
    const int b = bh / p.g.num_kv_heads, h = bh - b * p.g.num_kv_heads;
    int u0 = first_u0, u1 = first_u1;
    // who else works on this head: known before the first tile arrives, so it is off the path to the merge
    int part0 = first_part0, nparts = first_nparts;
    if (bh != bh_lo) {
      unit_range(p, c0, c1, bh, u0, u1);
      part0 = first_cta_of(p, bh);
      nparts = last_cta_of(p, bh) - part0 + 1;
    }
    const int rlen0 = *reinterpret_cast<const int*>((const uint8_t*)p.v.recent_len + (size_t)b * p.v.recent_len_bstride);
    const int rlen = rlen0 + (has_append ? 1 : 0);
    state_reset(st);

    // query fragments of head g of this KV group, channels 32t..32t+31
    const uint16_t* qrow = nullptr;
    uint32_t qh[16];
    if (g < p.gqa) qrow = reinterpret_cast<const uint16_t*>(p.q) + ((size_t)b * p.g.num_q_heads + h * p.gqa + g) * kD;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (qrow != nullptr) raw = __ldg(reinterpret_cast<const uint4*>(qrow + 32 * t + 8 * i));
      const uint32_t wv[4] = {raw.x, raw.y, raw.z, raw.w};
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = elem_to_float<BF16>((uint16_t)(wv[e >> 1] >> (16 * (e & 1))));
#pragma unroll
      for (int k = 0; k < 4; ++k) qh[4 * i + k] = pack_f16x2(f[k], f[k + 4]);
    }

    const uint32_t stage0 = smem_u32(stages);
    consume_pool<0, BF16>(st, p, max(u0, 0), min(u1, p.nF), 0, stage0, full_bar, empty_bar, stage, phase, alive, qh, warp, lane);
    consume_pool<1, BF16>(st, p, max(u0, p.nF), min(u1, p.nF + p.n4), p.nF, stage0, full_bar, empty_bar, stage, phase, alive,
                          qh, warp, lane);
    consume_pool<2, BF16>(st, p, max(u0, p.nF + p.n4), min(u1, p.nF + p.n4 + p.n2), p.nF + p.n4, stage0, full_bar, empty_bar,
                          stage, phase, alive, qh, warp, lane);
    // residual window: kTR-token tiles, 16 tokens per warp; the lower half of the warps takes even tiles and the
    // upper half odd ones, so two tiles (the whole 128-token window) are in work at once
    set_units(st, 0);
    for (int u = max(u0, p.nF + p.n4 + p.n2); u < u1; ++u) {
      const int ur = u - p.nF - p.n4 - p.n2;
      const int win = ur * kTR;
      if (win >= rlen) continue;
      if (alive && !mbar_wait(&full_bar[stage], phase)) {
        if (lane == 0) atomicExch(p.err, R2K_ERR_DEVICE_TIMEOUT);
        alive = false;
      }
      if (alive) {
        uint8_t* sbp = stages + stage * kStageBytes;
        const uint32_t sb = stage0 + stage * kStageBytes;
        if ((warp >= kNW / 2 ? 1 : 0) == (ur & 1)) {
          const int r0 = 16 * (warp % (kNW / 2));
          const int hi = min(rlen - win - r0, 16);
          if (hi > 0) {
            const int app_row = rlen0 - win - r0;  // ring row that receives the appended token, relative to this slice
            if (has_append && app_row >= 0 && app_row < 16) {
              const size_t off = ((size_t)b * p.g.num_kv_heads + h) * 256 + 8 * lane;
              *reinterpret_cast<uint2*>(sbp + kOffV + (r0 + app_row) * 256 + 8 * lane) =
                  __ldg(reinterpret_cast<const uint2*>((const uint8_t*)p.app_k + off));
              *reinterpret_cast<uint2*>(sbp + kOffV + kOffRecentV + (r0 + app_row) * 256 + 8 * lane) =
                  __ldg(reinterpret_cast<const uint2*>((const uint8_t*)p.app_v + off));
              __syncwarp();
            }
            const int t0 = 2 * t + (t & 1), t1 = 2 * t + 1 - (t & 1);
            float s[1][4];
            qk_fp<BF16>(sb + kOffV + (r0 + pg) * 256 + 64 * t, qrow, t, p.qscale, s[0]);
            if (hi < 16) mask_scores(s[0], pg, 0, hi);
            softmax_update<1>(st, s);
            pv_fp<BF16, false>(st, sb, kOffV + kOffRecentV + (r0 + t0) * 256 + 32 * g, kOffV + kOffRecentV + (r0 + t1) * 256 + 32 * g, 0,
                               s[0]);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
      }
      if (++stage == kStages) { stage = 0; phase ^= 1u; }
    }

    // ---- this CTA's partial for (b, h): merge the eight warps through shared memory ----
    set_units(st, 0);
#pragma unroll
    for (int d = 4; d < 32; d <<= 1) {
      st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], d);
      st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], d);
    }
    {
      float* mine = scratch + warp * kSlotFloats;
      float* r0 = mine + (2 * t) * kRowFloats;
      float* r1 = r0 + kRowFloats;
      const float c0 = st.corr[0] * k2p24, c1 = st.corr[1] * k2p24;  // INT4 value codes were fed as code+8
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        *reinterpret_cast<float2*>(r0 + 4 + 16 * g + 2 * j) = make_float2(st.o[j][0] - c0, st.o[j][2] - c0);
        *reinterpret_cast<float2*>(r1 + 4 + 16 * g + 2 * j) = make_float2(st.o[j][1] - c1, st.o[j][3] - c1);
      }
      if (g == 0) { r0[0] = st.m[0]; r0[1] = st.l[0]; r1[0] = st.m[1]; r1[1] = st.l[1]; }
    }
    named_bar_sync(1, kConsumers);
    float* slot = p.partials + ((size_t)bh * p.parts_cap + (cta - part0)) * kSlotFloats;
    static_assert(kNW >= 6, "warps 4 and 5 carry the request counter and the appended rows");
    const bool worker = threadIdx.x < 128;   // warps 0-3 carry the merge protocol; the others only meet the barriers
    float own_m = -INFINITY, own_l = 0.f, own_acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};   // this CTA's partial
    if (worker) {
      const int hh = threadIdx.x >> 4, sub = threadIdx.x & 15;  // 16 threads per head, 8 dims each
      float mw[kNW], mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < kNW; ++w) { mw[w] = scratch[w * kSlotFloats + hh * kRowFloats]; mx = fmaxf(mx, mw[w]); }
      float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
      float lsum = 0.f;
#pragma unroll
      for (int w = 0; w < kNW; ++w) {
        const float wgt = (mw[w] == -INFINITY) ? 0.f : ex2_approx(mw[w] - mx);
        const float* row = scratch + w * kSlotFloats + hh * kRowFloats;
        const float4 v0 = *reinterpret_cast<const float4*>(row + 4 + 8 * sub);
        const float4 v1 = *reinterpret_cast<const float4*>(row + 8 + 8 * sub);
        a0.x += wgt * v0.x; a0.y += wgt * v0.y; a0.z += wgt * v0.z; a0.w += wgt * v0.w;
        a1.x += wgt * v1.x; a1.y += wgt * v1.y; a1.z += wgt * v1.z; a1.w += wgt * v1.w;
        lsum += wgt * row[1];
      }
      float* orow = slot + hh * kRowFloats;
      __stcg(reinterpret_cast<float4*>(orow + 4 + 8 * sub), a0);
      __stcg(reinterpret_cast<float4*>(orow + 8 + 8 * sub), a1);
      if (sub == 0) __stcg(reinterpret_cast<float2*>(orow), make_float2(mx, lsum));
      own_m = mx; own_l = lsum;
      own_acc[0] = a0.x; own_acc[1] = a0.y; own_acc[2] = a0.z; own_acc[3] = a0.w;
      own_acc[4] = a1.x; own_acc[5] = a1.y; own_acc[6] = a1.z; own_acc[7] = a1.w;
    }
    // ---- two-level exact merge: groups of kMergeGroup partials, then the group results ----
    // Release pattern: the CTA barrier orders every thread's partial stores before thread 0's fence, whose
    // cumulativity publishes them before the ticket; the reader side mirrors it (ticket, fence, barrier).
    const int hh = (threadIdx.x >> 4) & 7, sub = threadIdx.x & 15;
    const int part = cta - part0, grp = part / kMergeGroup, ngroups = (nparts + kMergeGroup - 1) / kMergeGroup;
    const int gsize = min(kMergeGroup, nparts - kMergeGroup * grp);
    float mx, lsum, acc[8];
    named_bar_sync(1, kConsumers);
    if (threadIdx.x == 0) {
      __threadfence();
      const int ticket = atomicAdd(&p.group_counter[bh * p.groups_cap + grp], 1);
      if (xcount && bh == bh_lo) exchange_count_in(p, xstep);   // in flight together with the ticket
      flags[0] = (ticket == gsize - 1);
      if (flags[0]) p.group_counter[bh * p.groups_cap + grp] = 0;
      __threadfence();
    }
    named_bar_sync(1, kConsumers);
    bool last = flags[0] != 0;
    if (last) {
      if (worker)
        merge_rows(p.partials + ((size_t)bh * p.parts_cap + kMergeGroup * grp) * kSlotFloats, gsize, part - kMergeGroup * grp, own_m, own_l,
                   own_acc, hh,
                   sub, mx, lsum, acc);
      if (ngroups > 1) {
        if (worker) store_row(p.group_partials + ((size_t)bh * p.groups_cap + grp) * kSlotFloats, hh, sub, mx, lsum, acc);
        named_bar_sync(1, kConsumers);
        if (threadIdx.x == 0) {
          __threadfence();
          const int ticket = atomicAdd(&p.bh_counter[bh], 1);
          flags[1] = (ticket == ngroups - 1);
          if (flags[1]) p.bh_counter[bh] = 0;
          __threadfence();
        }
        named_bar_sync(1, kConsumers);
        last = flags[1] != 0;
        if (last && worker) {   // this CTA's own group result is still in (mx, lsum, acc)
          const float gm = mx, gl = lsum;
          float gacc[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) gacc[e] = acc[e];
          merge_rows(p.group_partials + (size_t)bh * p.groups_cap * kSlotFloats, ngroups, grp, gm, gl, gacc, hh, sub, mx, lsum, acc);
        }
      }
    }
    if (last) {
      // ---- last arriver of (b, h): epilogue and fused append ----
      // Every CTA of this head has arrived, so none of them reads recent_len[b] any more.  One thread outside
      // the merge workers counts the head in; the last head of the request moves the ring metadata.  This runs
      // beside the merge below, not after it.
      if (threadIdx.x == 128) {
        __threadfence();
        const int done = atomicAdd(&p.req_counter[b], 1);
        if (done == p.g.num_kv_heads - 1) {
          p.req_counter[b] = 0;
          if (has_append) {
            const int64_t gi = p.app_idx ? p.app_idx[2 * b] : p.app_global;
            const int64_t lp = p.app_idx ? p.app_idx[2 * b + 1] : p.app_logical;
            *reinterpret_cast<int64_t*>((uint8_t*)p.v.recent_global + (size_t)b * p.v.recent_global_bstride + 8 * (size_t)rlen0) = gi;
            *reinterpret_cast<int64_t*>((uint8_t*)p.v.recent_logical + (size_t)b * p.v.recent_logical_bstride + 8 * (size_t)rlen0) = lp;
            *reinterpret_cast<int*>((uint8_t*)p.v.recent_len + (size_t)b * p.v.recent_len_bstride) = rlen0 + 1;
            *reinterpret_cast<int64_t*>((uint8_t*)p.v.recent_page_lengths + (size_t)b * p.v.recent_page_lengths_bstride +
                                        8 * (size_t)(rlen0 / p.g.page_size)) = rlen0 % p.g.page_size + 1;
          }
        }
      }
      if (has_append && warp == 5) {  // ring row rlen0 of head h
        const size_t src = ((size_t)b * p.g.num_kv_heads + h) * 256 + 8 * lane;
        const size_t dst = ((size_t)h * p.g.recent_capacity + rlen0) * 256 + 8 * lane;
        *reinterpret_cast<uint2*>((uint8_t*)p.v.recent_k + (size_t)b * p.v.recent_k_bstride + dst) =
            __ldg(reinterpret_cast<const uint2*>((const uint8_t*)p.app_k + src));
        *reinterpret_cast<uint2*>((uint8_t*)p.v.recent_v + (size_t)b * p.v.recent_v_bstride + dst) =
            __ldg(reinterpret_cast<const uint2*>((const uint8_t*)p.app_v + src));
      }
      const size_t orow = (size_t)b * p.g.num_q_heads + h * p.gqa + hh;
      if (p.xw > 1) exchange_merge(p, xstep, orow, hh, worker, sub, scratch, mx, lsum, acc);
      if (worker) write_output<BF16>(p, orow, hh < p.gqa, sub, mx, lsum, acc);
    }
    named_bar_sync(1, kConsumers);  // scratch and flags are reused by the next (request, kv head)
  }
  if (xcount && bh_lo > bh_hi) { __threadfence(); exchange_count_in(p, xstep); }   // a CTA without work counts in too
}

// ---------------------------------------------------------------------------
// cross-shard merge of un-normalised states
// ---------------------------------------------------------------------------
__global__ void merge_states_kernel(const float* __restrict__ states, int num_states, int64_t state_stride, int rows,
                                    int dtype, void* out, uint32_t flags) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float mx = -INFINITY;
  for (int s = 0; s < num_states; ++s) mx = fmaxf(mx, states[s * state_stride + (int64_t)row * 130]);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float lsum = 0.f;
  for (int s = 0; s < num_states; ++s) {
    const float* st = states + s * state_stride + (int64_t)row * 130;
    const float wgt = (st[0] == -INFINITY) ? 0.f : __expf(st[0] - mx);
    const float2 v0 = *reinterpret_cast<const float2*>(st + 2 + 4 * lane);
    const float2 v1 = *reinterpret_cast<const float2*>(st + 4 + 4 * lane);
    acc.x += wgt * v0.x; acc.y += wgt * v0.y; acc.z += wgt * v1.x; acc.w += wgt * v1.y;
    lsum += wgt * st[1];
  }
  const float inv = 1.f / lsum;
  float r[4] = {acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv};
  const bool bf16 = dtype == R2K_DTYPE_BF16;
  if (flags & R2K_FLAG_OUTPUT_HADAMARD) {
#pragma unroll
    for (int e = 0; e < 4; ++e) r[e] = bf16 ? __bfloat162float(__float2bfloat16_rn(r[e])) : __half2float(__float2half_rn(r[e]));
    float a = r[0] + r[1], bq = r[0] - r[1], c = r[2] + r[3], d = r[2] - r[3];
    r[0] = a + c; r[1] = bq + d; r[2] = a - c; r[3] = bq - d;
#pragma unroll
    for (int sft = 1; sft < 32; sft <<= 1) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float o2 = __shfl_xor_sync(0xffffffffu, r[e], sft);
        r[e] = (lane & sft) ? (o2 - r[e]) : (r[e] + o2);
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) r[e] *= 0.08838834764831845f;
  }
  if (flags & R2K_FLAG_OUT_F32) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + (int64_t)row * kD + 4 * lane) = make_float4(r[0], r[1], r[2], r[3]);
  } else {
    uint2 pk;
    if (bf16) { pk.x = pack_bf16x2(r[0], r[1]); pk.y = pack_bf16x2(r[2], r[3]); }
    else { pk.x = pack_f16x2(r[0], r[1]); pk.y = pack_f16x2(r[2], r[3]); }
    *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(out) + (int64_t)row * kD + 4 * lane) = pk;
  }
}

}  // namespace r2k
