// Geometry shared by the host launcher and the decode kernel.
#pragma once

#include <cuda.h>
#include <stdint.h>

#include "r2k_b200.h"

namespace r2k {

constexpr int kD = 128;                     // head_dim
constexpr int kNW = 8;                      // consumer warps per CTA
constexpr int kThreads = (kNW + 1) * 32;    // plus one producer warp
constexpr int kConsumers = kNW * 32;
constexpr int kTQ = kNW * 32;               // tokens per tile: INT4-/INT2-value pools (one key block per warp)
constexpr int kTF = kNW * 16;               // tokens per tile: bf16-value pool
constexpr int kTR = (kNW / 2) * 16;         // tokens per tile: residual window (16 per warp of one half of the warps)
constexpr int kStages = 4;
constexpr int kCtasPerSm = 1;

// Shared-memory stage: [value region | key payload | key scales | key zeros].  The value region of a pool is as
// large as that pool needs (bf16 values: kTF rows of 256 bytes; INT4 / INT2 values: kTQ rows of 64 bytes + scales),
// and the key rows follow it directly, so that a stage is no larger than its largest tile and four of them fit.
constexpr int kOffV = 0;
// value region, per pool
// bf16-value tiles are stored as two half boxes (channels 0-63, 64-127) of kTF rows x 128 bytes; inside every
// row the 16-byte chunks are XOR-swizzled by (row & 7) -- the layout of a 128-byte-swizzled tensor copy.
constexpr int kFpHalfBytes = kTF * 128;
constexpr int kOffI4Scale = kTQ * 64;            // f32 per token after the nibble rows
constexpr int kOffI2Scale = kTQ * 32;            // f16 x groups per token after the crumb rows
constexpr int kOffI2Zero = kOffI2Scale + kTQ * 8;
constexpr int kOffRecentV = kTR * 256;           // residual tile: K rows then V rows
constexpr int kVBytesFp = kTF * 256;
constexpr int kVBytesPacked = kTQ * 68;
static_assert(kOffI2Zero + kTQ * 4 <= kVBytesPacked && kOffI4Scale + kTQ * 4 <= kVBytesPacked, "value region");
__host__ __device__ constexpr int tile_tokens(int pool) { return pool == 0 ? kTF : kTQ; }
__host__ __device__ constexpr int off_k(int pool) { return pool == 0 ? kVBytesFp : kVBytesPacked; }       // key nibble rows
__host__ __device__ constexpr int off_ks(int pool) { return off_k(pool) + tile_tokens(pool) * 64; }          // key scales
__host__ __device__ constexpr int off_kz(int pool) { return off_ks(pool) + (tile_tokens(pool) / 32) * 256; }  // key zeros
__host__ __device__ constexpr int stage_end(int pool) { return off_kz(pool) + (tile_tokens(pool) / 32) * 128; }
constexpr int kStageBytes = ((stage_end(0) > stage_end(1) ? stage_end(0) : stage_end(1)) + 1023) / 1024 * 1024;
static_assert(kStageBytes % 1024 == 0, "the swizzled value boxes want 1024-byte alignment");
static_assert(off_k(0) % 128 == 0 && off_k(1) % 128 == 0, "bulk copies want 16-byte aligned destinations");
static_assert(2 * kTR * 256 <= kStageBytes, "residual tile: key rows and value rows");
static_assert(kTF % 128 == 0 && kTQ % 128 == 0, "tile windows must start on multiples of the largest key block");

constexpr int kRowFloats = 132;                  // (max, sum, pad, pad, out[128]) per head
constexpr int kSlotFloats = 8 * kRowFloats;      // one partial: 8 heads of a KV group
constexpr int kScratchBytes = kNW * kSlotFloats * 4;
constexpr int kSmemBytes = kStages * kStageBytes + kScratchBytes + 256;

// Partials of a (request, kv head) are merged in groups of kMergeGroup by each group's last-arriving CTA, then the
// group results by the head's last arriver.  A group is one batch of loads for the merging CTA (merge_rows), so
// both levels cost one dependent round trip to memory for up to kMergeGroup * kMergeGroup CTAs per head.
constexpr int kMergeGroup = 9;
constexpr int kWsHeaderBytes = 256;
// The arrival counters sit in a block of fixed size behind the header, so that the partial slots start at the
// same offset for every geometry whose counters fit: launches of different geometries may then share one
// workspace (each launch leaves the counters it used at zero, and no launch writes floats where another expects
// a counter).  Only a geometry with more counters than this gets a larger block.
constexpr size_t kWsCounterBlockBytes = 64u << 10;
constexpr uint32_t kExchangePolls = 1u << 16;     // polls of the cross-rank wait before it gives up
constexpr uint32_t kExchangeNapNs = 20000;        // default sleep between polls: about 1.3 s in all

struct DecodeParams {
  R2KGeom g;
  R2KCacheView v;
  const void* q;
  const void* app_k;
  const void* app_v;
  const int64_t* app_idx;
  int64_t app_global, app_logical;
  void* out;
  uint32_t flags;
  // workspace
  int* err;
  int* bh_counter;
  int* req_counter;
  int* group_counter;
  float* partials;
  float* group_partials;
  int parts_cap, groups_cap;
  // derived
  int gqa, bh_total, grid;
  int nF, n4, n2, nR, units;      // tiles per (request, kv head) and their sum
  int wF0, w40, w20;              // arena row of the first window of each pool
  uint32_t cF, c4, c2, cR, c_bh;  // tile cost weights and their sum per (request, kv head); c_bh < 2^22
  int groups2, group2_shift, kblock_shift;
  float qscale;                   // sm_scale * log2(e)
  // bf16-value pool as a 4-D tensor {128, fp_capacity, kv heads, requests} with 64-element boxes and 128-byte
  // swizzle: full value tiles arrive bank-conflict-free for the value MMA's loads (valid when fp_tma != 0)
  int fp_tma;
  // fused cross-rank merge (xw > 1): every rank's exchange buffer, this rank, the world size and the step counter.
  // A buffer holds two halves (step parity) of [world][rows][130] (value, step) words, then the device-side step
  // counter at byte offset xflags_off.
  int xw, xrank;
  uint32_t xseq, xflags_off;
  uint32_t xnap;                  // nanoseconds the cross-rank wait sleeps between two polls
  float* xbuf[R2K_MAX_RANKS];
  alignas(64) CUtensorMap fp_map;
};

// Work is laid out on a cost axis: (request, kv head) bh owns [bh*c_bh, (bh+1)*c_bh), a tile owns its cost
// weight inside it.  CTA i owns [pos(i), pos(i+1)) with pos(i) = ceil(i * BH * c_bh / grid), kept as a
// (bh, remainder) pair so that everything stays in 32-bit arithmetic.
struct CostPos {
  int bh;
  uint32_t r;
};
__host__ __device__ inline CostPos cta_pos(const DecodeParams& p, int i) {
  const uint32_t a = (uint32_t)i * (uint32_t)p.bh_total, g = (uint32_t)p.grid;
  CostPos c;
  c.bh = (int)(a / g);
  c.r = ((a % g) * p.c_bh + g - 1) / g;
  if (c.r >= p.c_bh) { c.bh += 1; c.r = 0; }
  return c;
}
// Number of tiles of one (request, kv head) whose cost coordinate starts before r.
__host__ __device__ inline int units_before(const DecodeParams& p, uint32_t r) {
  int n = 0;
  const uint32_t cnt[4] = {(uint32_t)p.nF, (uint32_t)p.n4, (uint32_t)p.n2, (uint32_t)p.nR};
  const uint32_t cost[4] = {p.cF, p.c4, p.c2, p.cR};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (r == 0) return n;
    const uint32_t span = cnt[k] * cost[k];
    if (r >= span) { n += (int)cnt[k]; r -= span; }
    else { n += (int)((r + cost[k] - 1) / cost[k]); return n; }
  }
  return n;
}
// First and last CTA whose cost interval intersects bh's (a CTA with an empty interval strictly inside counts).
__host__ __device__ inline int first_cta_of(const DecodeParams& p, int bh) {
  return (int)(((uint32_t)bh * (uint32_t)p.grid) / (uint32_t)p.bh_total);
}
__host__ __device__ inline int last_cta_of(const DecodeParams& p, int bh) {
  int i = (int)((((uint32_t)bh + 1u) * (uint32_t)p.grid) / (uint32_t)p.bh_total);
  if (i > p.grid - 1) i = p.grid - 1;
  while (i > 0 && cta_pos(p, i).bh > bh) --i;
  return i;
}

}  // namespace r2k
