// Consumer-side math of the packed-KV decode kernel: scores, online softmax and value accumulation of one
// warp's 32-token key block, on data staged in shared memory.
//
// Every shared-memory operand is addressed as `base + compile-time offset`, where `base` is a 32-bit shared
// address (stage base + a per-lane offset that is computed once per pool, not per tile): the hot loop carries
// half a dozen address registers instead of recomputing ~40 lane addresses per tile.
#pragma once

#include "decode.cuh"
#include "device_utils.cuh"

namespace r2k {

constexpr float kLn2 = 0.69314718055994531f;
constexpr float k2p24 = 16777216.0f;
constexpr float k2p20 = 1048576.0f;
constexpr float k2m24 = 1.0f / 16777216.0f;
constexpr float k2m20 = 1.0f / 1048576.0f;
constexpr uint32_t kMaskLo = 0x000F000Fu;  // nibble 0 of each half-word -> code * 2^-24 as fp16
constexpr uint32_t kMaskHi = 0x00F000F0u;  // nibble 1 of each half-word -> code * 2^-20 as fp16

// ---- shared-memory loads by 32-bit address (volatile: never hoisted above the stage's barrier wait) ----
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
  uint32_t v;
  asm volatile("{\n.reg .u16 h;\nld.shared.u16 h, [%1];\ncvt.u32.u16 %0, h;\n}\n" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t a) {
  uint32_t v;
  asm volatile("{\n.reg .u16 h;\nld.shared.u8 h, [%1];\ncvt.u32.u16 %0, h;\n}\n" : "=r"(v) : "r"(a));
  return v;
}

// Row permutation inside a 16-token MMA tile: MMA row/k-slot r reads token pi(r).  It keeps a thread's two key
// rows in one 128-byte line and makes the four tokens of one value load alternate 64-byte halves (2-way
// instead of 4-way shared-memory conflicts).
__device__ __forceinline__ int pi_row(int r) {  // r in 0..7
  return (r & ~1) + ((r & 1) ^ ((r >> 1) & 1));
}

struct WarpState {
  float m[2];      // running reference point (log2 units) of heads 2t, 2t+1
  float l[2];      // this lane's share of sum-exp
  float corr[4];   // 8 * 2^-24 * sum of fp16(p * scale) over INT4-value tokens (the +8 code offset), accumulated by
                   // one MMA per tile whose A rows are all 8: complete per lane, [0],[2] head 2t and [1],[3] head 2t+1
  float o[8][4];   // O^T fragments: block j <-> dims 16g+2j (c0,c1) and 16g+2j+1 (c2,c3); columns = heads 2t,2t+1
  int units;       // 0: true units; 1: INT4 units (even dims * 2^-24, odd dims * 2^-20)
};

__device__ __forceinline__ void state_reset(WarpState& s) {
  s.m[0] = s.m[1] = -INFINITY;
  s.l[0] = s.l[1] = 0.f;
  s.corr[0] = s.corr[1] = s.corr[2] = s.corr[3] = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) s.o[j][0] = s.o[j][1] = s.o[j][2] = s.o[j][3] = 0.f;
  s.units = 0;
}

__device__ __forceinline__ void set_units(WarpState& s, int units) {
  if (s.units == units) return;
  const float fe = units ? k2m24 : k2p24, fo = units ? k2m20 : k2p20;  // exact power-of-two rescale
#pragma unroll
  for (int j = 0; j < 8; ++j) { s.o[j][0] *= fe; s.o[j][1] *= fe; s.o[j][2] *= fo; s.o[j][3] *= fo; }
  s.units = units;
}

// Online-softmax update for NT 16-token tiles of scores (log2 units, already masked with -inf); returns
// probabilities in place.  Lazy reference point: it only moves when a score exceeds it by more than 2^8, so
// probabilities stay below 256 and most blocks skip the rescale of the accumulators.
template <int NT>
__device__ __forceinline__ void softmax_update(WarpState& st, float (&s)[NT][4]) {
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][2]));
    mx1 = fmaxf(mx1, fmaxf(s[j][1], s[j][3]));
  }
  // The reference point is the same in all eight lanes that share a head pair, so each lane can test its own
  // scores against it; the cross-lane maximum is only needed when some lane asks for a move (about one block in
  // ten), which keeps six shuffles and their latency out of the common path.
  if (__any_sync(0xffffffffu, (mx0 > st.m[0] + 8.f) | (mx1 > st.m[1] + 8.f))) {
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 4));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 4));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 8));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 8));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 16));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 16));
    const float n0 = fmaxf(st.m[0], mx0), n1 = fmaxf(st.m[1], mx1);
    const float f0 = ex2_approx(st.m[0] - n0), f1 = ex2_approx(st.m[1] - n1);  // m = -inf -> 0
    st.l[0] *= f0; st.l[1] *= f1;
    st.corr[0] *= f0; st.corr[1] *= f1; st.corr[2] *= f0; st.corr[3] *= f1;
#pragma unroll
    for (int j = 0; j < 8; ++j) { st.o[j][0] *= f0; st.o[j][1] *= f1; st.o[j][2] *= f0; st.o[j][3] *= f1; }
    st.m[0] = n0; st.m[1] = n1;
  }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    s[j][0] = ex2_approx(s[j][0] - st.m[0]);
    s[j][1] = ex2_approx(s[j][1] - st.m[1]);
    s[j][2] = ex2_approx(s[j][2] - st.m[0]);
    s[j][3] = ex2_approx(s[j][3] - st.m[1]);
    st.l[0] += s[j][0] + s[j][2];
    st.l[1] += s[j][1] + s[j][3];
  }
}

__device__ __forceinline__ void mask_scores(float (&s)[4], int row_a, int lo, int hi) {
  if (row_a < lo || row_a >= hi) s[0] = s[1] = -INFINITY;
  if (row_a + 8 < lo || row_a + 8 >= hi) s[2] = s[3] = -INFINITY;
}

// Byte offset, inside the value region of a bf16-value tile, of 16-byte chunk c (0..15) of row r: half box
// c / 8, row pitch 128 bytes, chunk index XOR (r & 7).  This is where a 128-byte-swizzled tensor copy of the two
// 64-channel boxes puts it (the region is 1024-byte aligned), and what the plain-load path reproduces.
__host__ __device__ __forceinline__ uint32_t fp_box_offset(int r, int c) {
  return (uint32_t)((c >> 3) * kFpHalfBytes + r * 128 + (((c & 7) ^ (r & 7)) * 16));
}

// Per-lane shared-memory offsets (relative to the stage base) of one warp's 32-token slice.
struct LaneOffsets {
  uint32_t k;    // key rows: (slice + pi(g)) * 64 + 16 t        (+ (16 j + 8 e) * 64)
  uint32_t ks;   // key scales of the slice's block + 64 t       (+ 16 i)
  uint32_t kz;   // key zeros of the slice's block + 32 t        (+ 16)
  uint32_t va;   // value rows of token t0 (see pv_*), vb of token t1
  uint32_t vb;
  uint32_t m0;   // first value metadata address (INT4: scale of row pi(g); INT2: scale of token t0's group)
  uint32_t m1;   // INT2: zero of token t0's group
};

// Scores of two 16-token tiles against INT4 keys.  Q' = q * scale is held as an exact two-term fp16 sum
// (hi = RN(q*s), lo = fma(q, s, -hi)), so every product the tensor core sees is exact and the fp32
// accumulation is the only rounding.  Codes minus zero points are fed as signed fp16 subnormals (AND, HSUB2).
__device__ __forceinline__ void qk_int4(uint32_t sb, const LaneOffsets& o, const uint32_t (&qh)[16], float alpha,
                                        float (&s)[2][4]) {
  uint32_t qp[16], ql[16];  // paired (c0,c4) (c1,c5) (c2,c6) (c3,c7) per 8-channel word
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 w = lds128(sb + o.ks + 16 * i);
    const uint32_t sp[4] = {__byte_perm(w.x, w.z, 0x5410), __byte_perm(w.x, w.z, 0x7632), __byte_perm(w.y, w.w, 0x5410),
                            __byte_perm(w.y, w.w, 0x7632)};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      qp[4 * i + k] = hmul2_u32(qh[4 * i + k], sp[k]);
      ql[4 * i + k] = hfma2_neg_u32(qh[4 * i + k], sp[k], qp[4 * i + k]);
    }
  }
  // Zero points as fp16 subnormal pairs in the two code domains: (z0,z4), (z2,z6) scaled 2^-24 for the low
  // nibbles and (z1,z5), (z3,z7) scaled 2^-20 for the high ones.  code - zero is then one exact HSUB2 per
  // register (subnormal arithmetic is exact on integers), and the tensor core sees signed integers.
  uint32_t zl[8], zh[8];
  {
    const uint4 za = lds128(sb + o.kz), zb = lds128(sb + o.kz + 16);
    const uint32_t z[8] = {za.x, za.y, za.z, za.w, zb.x, zb.y, zb.z, zb.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t x = __byte_perm(z[2 * i], z[2 * i + 1], 0x5410);  // z0 z1 z4 z5
      const uint32_t y = __byte_perm(z[2 * i], z[2 * i + 1], 0x7632);  // z2 z3 z6 z7
      zl[2 * i] = x & 0x00FF00FFu;     zh[2 * i] = (x >> 4) & 0x0FF00FF0u;
      zl[2 * i + 1] = y & 0x00FF00FFu; zh[2 * i + 1] = (y >> 4) & 0x0FF00FF0u;
    }
  }
  const float f24 = k2p24 * alpha, f20 = k2p20 * alpha;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const uint4 ka = lds128(sb + o.k + 16 * j * 64);
    const uint4 kb = lds128(sb + o.k + (16 * j + 8) * 64);
    const uint32_t wa[4] = {ka.x, ka.y, ka.z, ka.w}, wb[4] = {kb.x, kb.y, kb.z, kb.w};
    float lo[4] = {0.f, 0.f, 0.f, 0.f}, hi[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t a8 = wa[i] >> 8, b8 = wb[i] >> 8;
      const uint32_t l0 = hsub2_u32(wa[i] & kMaskLo, zl[2 * i]), l1 = hsub2_u32(wb[i] & kMaskLo, zl[2 * i]);
      const uint32_t l2 = hsub2_u32(a8 & kMaskLo, zl[2 * i + 1]), l3 = hsub2_u32(b8 & kMaskLo, zl[2 * i + 1]);
      const uint32_t h0 = hsub2_u32(wa[i] & kMaskHi, zh[2 * i]), h1 = hsub2_u32(wb[i] & kMaskHi, zh[2 * i]);
      const uint32_t h2 = hsub2_u32(a8 & kMaskHi, zh[2 * i + 1]), h3 = hsub2_u32(b8 & kMaskHi, zh[2 * i + 1]);
      mma_f16(lo, l0, l1, l2, l3, qp[4 * i + 0], qp[4 * i + 2]);
      mma_f16(hi, h0, h1, h2, h3, qp[4 * i + 1], qp[4 * i + 3]);
      mma_f16(lo, l0, l1, l2, l3, ql[4 * i + 0], ql[4 * i + 2]);
      mma_f16(hi, h0, h1, h2, h3, ql[4 * i + 1], ql[4 * i + 3]);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) s[j][c] = fmaf(lo[c], f24, hi[c] * f20);
  }
}

// O^T += V^T P^T for 16-token tile j of INT4 values: codes as fp16 subnormals (the two's-complement fix
// code ^ 8 rides in the same LOP3 as the mask), per-token scale folded into P.
template <bool PARTIAL>
__device__ __forceinline__ void pv_int4(WarpState& st, uint32_t sb, const LaneOffsets& o, int j, float (&p)[4], int pg,
                                        int lo, int hi) {
  float sa = __uint_as_float(lds32(sb + o.m0 + 64 * j)), sc = __uint_as_float(lds32(sb + o.m0 + 64 * j + 32));
  if (PARTIAL) {
    if (16 * j + pg < lo || 16 * j + pg >= hi) sa = 0.f;
    if (16 * j + pg + 8 < lo || 16 * j + pg + 8 >= hi) sc = 0.f;
  }
  const uint32_t ha = pack_f16x2(p[0] * sa, p[1] * sa), hb = pack_f16x2(p[2] * sc, p[3] * sc);
  const uint32_t b0 = movmatrix_trans(ha), b1 = movmatrix_trans(hb);
  mma_f16(st.corr, 0x00080008u, 0x00080008u, 0x00080008u, 0x00080008u, b0, b1);   // the offset the codes carry below
  const uint2 w0 = lds64(sb + o.va + 1024 * j), w1 = lds64(sb + o.vb + 1024 * j);
  const uint2 w2 = lds64(sb + o.va + 1024 * j + 512), w3 = lds64(sb + o.vb + 1024 * j + 512);
  constexpr uint32_t kFixLo = 0x00080008u, kFixHi = 0x00800080u;
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const uint32_t c0 = hf ? w0.y : w0.x, c1 = hf ? w1.y : w1.x, c2 = hf ? w2.y : w2.x, c3 = hf ? w3.y : w3.x;
    const uint32_t xa = __byte_perm(c0, c1, 0x5410), ya = __byte_perm(c0, c1, 0x7632);
    const uint32_t xb = __byte_perm(c2, c3, 0x5410), yb = __byte_perm(c2, c3, 0x7632);
    const uint32_t xa8 = xa >> 8, xb8 = xb >> 8, ya8 = ya >> 8, yb8 = yb >> 8;
    mma_f16(st.o[4 * hf + 0], (xa & kMaskLo) ^ kFixLo, (xa & kMaskHi) ^ kFixHi, (xb & kMaskLo) ^ kFixLo, (xb & kMaskHi) ^ kFixHi, b0, b1);
    mma_f16(st.o[4 * hf + 1], (xa8 & kMaskLo) ^ kFixLo, (xa8 & kMaskHi) ^ kFixHi, (xb8 & kMaskLo) ^ kFixLo, (xb8 & kMaskHi) ^ kFixHi, b0, b1);
    mma_f16(st.o[4 * hf + 2], (ya & kMaskLo) ^ kFixLo, (ya & kMaskHi) ^ kFixHi, (yb & kMaskLo) ^ kFixLo, (yb & kMaskHi) ^ kFixHi, b0, b1);
    mma_f16(st.o[4 * hf + 3], (ya8 & kMaskLo) ^ kFixLo, (ya8 & kMaskHi) ^ kFixHi, (yb8 & kMaskLo) ^ kFixLo, (yb8 & kMaskHi) ^ kFixHi, b0, b1);
  }
}

// (code - zero) * scale for the eight 2-bit fields of each half-word of x -> eight half2.
__device__ __forceinline__ void dequant_crumbs(uint32_t x, const uint32_t (&zm)[5], const uint32_t (&sk)[5],
                                               uint32_t (&v)[8]) {
#pragma unroll
  for (int i = 0; i < 5; ++i)
    v[i] = hmul2_u32(hsub2_u32((x & (0x00030003u << (2 * i))) | 0x64006400u, zm[i]), sk[i]);
  const uint32_t y = x >> 10;
#pragma unroll
  for (int i = 0; i < 3; ++i)
    v[5 + i] = hmul2_u32(hsub2_u32((y & (0x00030003u << (2 * i))) | 0x64006400u, zm[i]), sk[i]);
}

// O^T += V^T P^T for 16-token tile j of INT2 values, dequantised in registers ((code - zero) exactly, then one
// fp16 multiply by the scale).  `step` = bytes between consecutive tokens of the scale array (2 * groups);
// the zero array has half that pitch.  Token t1 sits one token after (t even) or before (t odd) token t0.
template <bool PARTIAL>
__device__ __forceinline__ void pv_int2(WarpState& st, uint32_t sb, const LaneOffsets& o, int j, float (&pr)[4], int t,
                                        int step, int lo, int hi) {
  const uint32_t b0 = movmatrix_trans(pack_f16x2(pr[0], pr[1])), b1 = movmatrix_trans(pack_f16x2(pr[2], pr[3]));
  const int d1 = (t & 1) ? -step : step;   // scale offset of token t1 relative to token t0
  uint32_t w[4], sc[4], zp[4];
  w[0] = lds32(sb + o.va + 512 * j);       w[1] = lds32(sb + o.vb + 512 * j);
  w[2] = lds32(sb + o.va + 512 * j + 256); w[3] = lds32(sb + o.vb + 512 * j + 256);
  const uint32_t s0 = sb + o.m0 + 16 * j * step, z0 = sb + o.m1 + 8 * j * step;
  sc[0] = lds16(s0);            sc[1] = lds16(s0 + d1);
  sc[2] = lds16(s0 + 8 * step); sc[3] = lds16(s0 + 8 * step + d1);
  zp[0] = lds8(z0);             zp[1] = lds8(z0 + (d1 >> 1));
  zp[2] = lds8(z0 + 4 * step);  zp[3] = lds8(z0 + 4 * step + (d1 >> 1));
  if (PARTIAL) {
    const int t0 = 2 * t + (t & 1), t1 = 2 * t + 1 - (t & 1);
    const int tok[4] = {16 * j + t0, 16 * j + t1, 16 * j + t0 + 8, 16 * j + t1 + 8};
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (tok[i] < lo || tok[i] >= hi) { sc[i] = 0u; zp[i] = 0u; }
  }
  uint32_t va[16], vb[16];
#pragma unroll
  for (int pr2 = 0; pr2 < 2; ++pr2) {
    const uint32_t s2 = sc[2 * pr2] | (sc[2 * pr2 + 1] << 16), z2 = zp[2 * pr2] | (zp[2 * pr2 + 1] << 16);
    uint32_t zm[5], sk[5];
    const uint32_t quarter[5] = {0x3C003C00u, 0x34003400u, 0x2C002C00u, 0x24002400u, 0x1C001C00u};  // 4^-i as half2
#pragma unroll
    for (int i = 0; i < 5; ++i) { zm[i] = 0x64006400u + (z2 << (2 * i)); sk[i] = i ? hmul2_u32(s2, quarter[i]) : s2; }
    const uint32_t x = __byte_perm(w[2 * pr2], w[2 * pr2 + 1], 0x5410), y = __byte_perm(w[2 * pr2], w[2 * pr2 + 1], 0x7632);
    uint32_t lo8[8], hi8[8];
    dequant_crumbs(x, zm, sk, lo8);
    dequant_crumbs(y, zm, sk, hi8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (pr2 == 0) { va[i] = lo8[i]; va[8 + i] = hi8[i]; } else { vb[i] = lo8[i]; vb[8 + i] = hi8[i]; }
    }
  }
#pragma unroll
  for (int jb = 0; jb < 8; ++jb) mma_f16(st.o[jb], va[2 * jb], va[2 * jb + 1], vb[2 * jb], vb[2 * jb + 1], b0, b1);
}

// O^T += V^T P^T for 16-token tile j of 16-bit values (rows of 256 bytes): prmt pair-transposes; for bf16 the
// probabilities go in as two bf16 terms (P = P_hi + P_lo, two MMAs) to keep ~16 mantissa bits of P.
// SWZ: rows of a swizzled half box (128-byte pitch, see fp_box_offset): va / vb carry the swizzled offset of the
// lane's first 16-byte chunk and the second chunk is its neighbour (offset ^ 16).  Plain 256-byte rows (the
// residual window) cost a 4-way bank conflict on every load here, which does not matter for 32 tokens.
template <bool BF16, bool SWZ>
__device__ __forceinline__ void pv_fp(WarpState& st, uint32_t sb, uint32_t va, uint32_t vb, int j, float (&pr)[4]) {
  constexpr int kPitch = SWZ ? 128 : 256;
  uint32_t bh0, bh1, bl0 = 0, bl1 = 0;
  if (BF16) {
    const uint32_t ha = pack_bf16x2(pr[0], pr[1]), hb = pack_bf16x2(pr[2], pr[3]);
    const uint32_t la = pack_bf16x2(pr[0] - __uint_as_float(ha << 16), pr[1] - __uint_as_float(ha & 0xffff0000u));
    const uint32_t lb = pack_bf16x2(pr[2] - __uint_as_float(hb << 16), pr[3] - __uint_as_float(hb & 0xffff0000u));
    bh0 = movmatrix_trans(ha); bh1 = movmatrix_trans(hb);
    bl0 = movmatrix_trans(la); bl1 = movmatrix_trans(lb);
  } else {
    bh0 = movmatrix_trans(pack_f16x2(pr[0], pr[1])); bh1 = movmatrix_trans(pack_f16x2(pr[2], pr[3]));
  }
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const uint32_t xa = SWZ ? ((va + 16 * kPitch * j) ^ (16 * hf)) : (va + 16 * kPitch * j + 16 * hf);
    const uint32_t xb = SWZ ? ((vb + 16 * kPitch * j) ^ (16 * hf)) : (vb + 16 * kPitch * j + 16 * hf);
    const uint4 r0 = lds128(sb + xa), r1 = lds128(sb + xb);
    const uint4 r2 = lds128(sb + xa + 8 * kPitch), r3 = lds128(sb + xb + 8 * kPitch);
    const uint32_t a[4] = {r0.x, r0.y, r0.z, r0.w}, b[4] = {r1.x, r1.y, r1.z, r1.w};
    const uint32_t c[4] = {r2.x, r2.y, r2.z, r2.w}, d[4] = {r3.x, r3.y, r3.z, r3.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t a0 = __byte_perm(a[q], b[q], 0x5410), a1 = __byte_perm(a[q], b[q], 0x7632);
      const uint32_t a2 = __byte_perm(c[q], d[q], 0x5410), a3 = __byte_perm(c[q], d[q], 0x7632);
      if (BF16) {
        mma_bf16(st.o[4 * hf + q], a0, a1, a2, a3, bh0, bh1);
        mma_bf16(st.o[4 * hf + q], a0, a1, a2, a3, bl0, bl1);
      } else {
        mma_f16(st.o[4 * hf + q], a0, a1, a2, a3, bh0, bh1);
      }
    }
  }
}

// Scores of one 16-token tile of 16-bit keys (residual window): exact products, fp32 accumulation.
// `ka` addresses key row pi(g) of the tile at byte 64 t.
template <bool BF16>
__device__ __forceinline__ void qk_fp(uint32_t ka, const uint16_t* qrow, int t, float scale, float (&s)[4]) {
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 ra = lds128(ka + 16 * i), rb = lds128(ka + 8 * 256 + 16 * i);
    uint4 qq = make_uint4(0u, 0u, 0u, 0u);
    if (qrow != nullptr) qq = __ldg(reinterpret_cast<const uint4*>(qrow + 32 * t + 8 * i));
    if (BF16) {
      mma_bf16(acc, ra.x, rb.x, ra.y, rb.y, qq.x, qq.y);
      mma_bf16(acc, ra.z, rb.z, ra.w, rb.w, qq.z, qq.w);
    } else {
      mma_f16(acc, ra.x, rb.x, ra.y, rb.y, qq.x, qq.y);
      mma_f16(acc, ra.z, rb.z, ra.w, rb.w, qq.z, qq.w);
    }
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) s[c] = acc[c] * scale;
}

}  // namespace r2k
