// Geometry shared by the host launcher and the decode kernel.
#pragma once

#include <stdint.h>

#include "r2k_b200.h"

namespace r2k {

constexpr int kD = 128;                     // head_dim
constexpr int kNW = 4;                      // consumer warps per CTA
constexpr int kThreads = (kNW + 1) * 32;    // plus one producer warp
constexpr int kConsumers = kNW * 32;
constexpr int kTQ = kNW * 32;               // tokens per tile: INT4-/INT2-value pools (one key block per warp)
constexpr int kTF = kNW * 16;               // tokens per tile: bf16-value pool
constexpr int kTR = 32;                     // tokens per tile: residual window (two warps)
constexpr int kStages = 3;
constexpr int kCtasPerSm = 2;

// shared-memory stage: [value region | key payload | key scales | key zeros]
constexpr int kOffV = 0;
constexpr int kVBytes = 16384;
constexpr int kOffK = kOffV + kVBytes;
constexpr int kOffKS = kOffK + kTQ * 64;
constexpr int kOffKZ = kOffKS + (kTQ / 32) * 256;
constexpr int kStageBytes = kOffKZ + (kTQ / 32) * 128;
static_assert(kStageBytes % 128 == 0, "stage must stay 128-byte aligned");
// value region, per pool
constexpr int kOffI4Scale = kTQ * 64;            // f32 per token after the nibble rows
constexpr int kOffI2Scale = kTQ * 32;            // f16 x groups per token after the crumb rows
constexpr int kOffI2Zero = kOffI2Scale + kTQ * 8;
constexpr int kOffRecentV = kTR * 256;           // residual tile: K rows then V rows
static_assert(kTF * 256 <= kVBytes && kOffI2Zero + kTQ * 4 <= kVBytes && 2 * kTR * 256 <= kVBytes, "value region");

constexpr int kRowFloats = 132;                  // (max, sum, pad, pad, out[128]) per head
constexpr int kSlotFloats = 8 * kRowFloats;      // one partial: 8 heads of a KV group
constexpr int kScratchBytes = kNW * kSlotFloats * 4;
constexpr int kSmemBytes = kStages * kStageBytes + kScratchBytes + 256;

constexpr int kWsHeaderBytes = 256;

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
  float* partials;
  int parts_cap;
  // derived
  int gqa, bh_total, grid;
  int nF, n4, n2, nR, units;      // tiles per (request, kv head) and their sum
  int wF0, w40, w20;              // arena row of the first window of each pool
  int64_t cF, c4, c2, cR, c_bh, c_total;
  int groups2, group2_shift, kblock_shift;
  float qscale;                   // sm_scale * log2(e)
};

// Number of tiles of one (request, kv head) whose cost coordinate starts before r.
__host__ __device__ inline int units_before(const DecodeParams& p, int64_t r) {
  int n = 0;
  const int cnt[4] = {p.nF, p.n4, p.n2, p.nR};
  const int64_t cost[4] = {p.cF, p.c4, p.c2, p.cR};
  for (int k = 0; k < 4; ++k) {
    if (r <= 0) return n;
    int64_t a = (r + cost[k] - 1) / cost[k];
    n += a < cnt[k] ? (int)a : cnt[k];
    r -= (int64_t)cnt[k] * cost[k];
  }
  return n;
}
__host__ __device__ inline int64_t cta_cost_begin(const DecodeParams& p, int i) {
  return ((int64_t)i * p.c_total + p.grid - 1) / p.grid;
}
__host__ __device__ inline int first_cta_of(const DecodeParams& p, int bh) {
  return (int)(((int64_t)bh * p.c_bh * p.grid) / p.c_total);
}
__host__ __device__ inline int last_cta_of(const DecodeParams& p, int bh) {
  return (int)(((((int64_t)bh + 1) * p.c_bh - 1) * p.grid) / p.c_total);
}

}  // namespace r2k
