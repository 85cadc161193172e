// Host-only brute-force check of the decode kernel's work partition (compiled with nvcc, runs on the CPU):
// every tile of every (request, kv head) is owned by exactly one CTA, CTAs own contiguous ranges, and the
// closed-form first/last CTA of a (request, kv head) agree with the enumeration the CTAs perform.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "decode.cuh"

using namespace r2k;

static int check(int bh_total, int nF, int n4, int n2, int nR, int grid, unsigned cF, unsigned c4, unsigned c2, unsigned cR) {
  DecodeParams p{};
  p.bh_total = bh_total; p.nF = nF; p.n4 = n4; p.n2 = n2; p.nR = nR; p.units = nF + n4 + n2 + nR;
  p.cF = cF; p.c4 = c4; p.c2 = c2; p.cR = cR;
  p.c_bh = nF * cF + n4 * c4 + n2 * c2 + nR * cR;
  p.grid = grid;
  std::vector<int> owner((size_t)bh_total * p.units, -1);
  std::vector<int> first(bh_total, 1 << 30), last(bh_total, -1);
  for (int cta = 0; cta < grid; ++cta) {
    const CostPos c0 = cta_pos(p, cta), c1 = cta_pos(p, cta + 1);
    int bh_hi = c1.r > 0 ? c1.bh : c1.bh - 1;
    if (bh_hi > bh_total - 1) bh_hi = bh_total - 1;
    for (int bh = c0.bh; bh <= bh_hi; ++bh) {
      const unsigned lo = bh == c0.bh ? c0.r : 0u, hi = bh == c1.bh ? c1.r : p.c_bh;
      const int u0 = units_before(p, lo), u1 = units_before(p, hi);
      if (u1 < u0) return 1;
      for (int u = u0; u < u1; ++u) {
        if (owner[(size_t)bh * p.units + u] != -1) return 2;   // owned twice
        owner[(size_t)bh * p.units + u] = cta;
      }
      if (cta < first[bh]) first[bh] = cta;
      if (cta > last[bh]) last[bh] = cta;
    }
  }
  for (size_t i = 0; i < owner.size(); ++i) if (owner[i] < 0) return 3;            // orphan tile
  for (size_t i = 1; i < owner.size(); ++i) if (owner[i] < owner[i - 1]) return 4; // not contiguous / ordered
  for (int bh = 0; bh < bh_total; ++bh) {
    if (first[bh] != first_cta_of(p, bh)) return 5;
    if (last[bh] != last_cta_of(p, bh)) return 6;
    if (last[bh] - first[bh] + 1 > (grid + bh_total - 1) / bh_total + 1) return 7;   // workspace bound
  }
  const CostPos end = cta_pos(p, grid);
  if (end.bh != bh_total || end.r != 0) return 8;
  return 0;
}

int main() {
  long cases = 0;
  unsigned seed = 12345u;
  auto rnd = [&](int n) { seed = seed * 1664525u + 1013904223u; return (int)((seed >> 8) % (unsigned)n); };
  for (int it = 0; it < 20000; ++it) {
    const int bh = 1 + rnd(it % 3 == 0 ? 64 : 8);
    const int nF = rnd(4) ? rnd(200) : 0, n4 = rnd(4) ? rnd(300) : 0, n2 = rnd(4) ? rnd(300) : 0, nR = rnd(6);
    const int units = nF + n4 + n2 + nR;
    if (units == 0) continue;
    const long total = (long)units * bh;
    int grid = 1 + rnd(444);
    if (grid > total) grid = (int)total;
    const unsigned cF = 1 + rnd(40), c4 = 1 + rnd(40), c2 = 1 + rnd(40), cR = 1 + rnd(40);
    const int rc = check(bh, nF, n4, n2, nR, grid, cF, c4, c2, cR);
    if (rc) {
      std::printf("FAIL rc=%d bh=%d tiles=%d/%d/%d/%d grid=%d costs=%u/%u/%u/%u\n", rc, bh, nF, n4, n2, nR, grid, cF, c4, c2, cR);
      return 1;
    }
    ++cases;
  }
  // the benchmark geometries (tiles of 128 bf16-value / 256 INT4- or INT2-value / 64 residual tokens; grids of one
  // CTA per SM, rounded down to a whole number of CTAs per (request, kv head)): 8 x 32768 tokens on 2 kv heads,
  // 1M tokens of one request, 16 x 65536 tokens on 4 kv heads, 4096 INT4-value tokens of one request
  if (check(16, 64, 64, 33, 2, 144, 14, 21, 24, 5) || check(2, 0, 2048, 2049, 2, 148, 14, 21, 24, 5) ||
      check(64, 128, 128, 65, 2, 128, 14, 21, 24, 5) || check(2, 0, 16, 0, 2, 18, 14, 21, 24, 5))
    return 2;
  std::printf("OK %ld cases\n", cases + 4);
  return 0;
}
