// extern "C" surface of libr2k_b200.so: validation, launch geometry, launches.
// No torch types, no allocation, no synchronisation (except r2k_decode_device_status).
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "decode_kernel.cuh"
#include "pack_kernels.cuh"
#include "r2k_b200.h"

namespace r2k {
namespace {

std::atomic<uint64_t> g_launches{0};

struct DeviceInfo {
  int sms = 0;
  bool ready = false;
  bool pdl = true;   // R2K_DISABLE_PDL=1 in the environment turns programmatic dependent launch off (debugging)
};
DeviceInfo g_dev[64];
std::mutex g_dev_mutex;

// Per-device facts and the kernels' function attributes, set up once per device under a lock: the first calls of
// two host threads may race here.
int device_info(DeviceInfo** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return R2K_ERR_CUDA;
  DeviceInfo& d = g_dev[dev];
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!d.ready) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return R2K_ERR_CUDA;
    if (cudaFuncSetAttribute(decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
      return R2K_ERR_CUDA;
    cudaFuncSetAttribute(decode_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(decode_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    d.sms = sms;
    const char* off = std::getenv("R2K_DISABLE_PDL");
    d.pdl = !(off != nullptr && off[0] == '1');
    d.ready = true;
  }
  *out = &d;
  return R2K_OK;
}

// R2K_GRID_CAP=<n> in the environment (read at every call, so a test can change it inside one process) limits
// the decode grid to n CTAs: small caches then put many tiles on one CTA, which is how the tests reach the
// pipeline's stage reuse, phase flips and head crossings without benchmark-sized inputs.
int grid_cap_from_env() {
  const char* cap = std::getenv("R2K_GRID_CAP");
  if (cap == nullptr || cap[0] == 0) return 0;
  const int v = std::atoi(cap);
  return v > 0 ? v : 0;
}

inline bool pow2_in(int v, int a, int b, int c) { return v == a || v == b || v == c; }
inline int ilog2(int v) { int s = 0; while ((1 << s) < v) ++s; return s; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_geom(const R2KGeom* g) {
  if (g == nullptr) return R2K_ERR_NULL;
  if (g->head_dim != kD || g->batch < 1 || g->num_kv_heads < 1 || g->num_q_heads < 1) return R2K_ERR_GEOMETRY;
  if (g->num_q_heads % g->num_kv_heads || g->num_q_heads / g->num_kv_heads > 8) return R2K_ERR_GEOMETRY;
  if (g->dtype != R2K_DTYPE_BF16 && g->dtype != R2K_DTYPE_FP16) return R2K_ERR_GEOMETRY;
  if (!pow2_in(g->k_block, 32, 64, 128) || !pow2_in(g->v2_group, 32, 64, 128) || !pow2_in(g->page_size, 16, 32, 64))
    return R2K_ERR_GEOMETRY;
  if (g->n_fp < 0 || g->n_i4 < 0 || g->n_i2 < 0 || g->recent_capacity < 0) return R2K_ERR_GEOMETRY;
  if (g->k_capacity < 0 || g->k_capacity % 128) return R2K_ERR_GEOMETRY;
  if (g->k_off_fp < 0 || g->k_off_i4 < g->k_off_fp + g->n_fp || g->k_off_i2 < g->k_off_i4 + g->n_i4 ||
      g->k_off_i2 + g->n_i2 > g->k_capacity)
    return R2K_ERR_GEOMETRY;
  if (g->n_fp > g->fp_capacity || g->n_i4 > g->i4_capacity || g->n_i2 > g->i2_capacity) return R2K_ERR_CAPACITY;
  if (g->recent_capacity % g->page_size) return R2K_ERR_GEOMETRY;
  return R2K_OK;
}

int windows(int a0, int n, int tile, int* first) {
  *first = a0 / tile * tile;
  if (n <= 0) return 0;
  return (a0 + n + tile - 1) / tile - a0 / tile;
}

// Everything the kernel derives from the geometry; shared by workspace sizing and the launch.
int derive(const R2KGeom* g, DecodeParams* p) {
  DeviceInfo* dev;
  int rc = device_info(&dev);
  if (rc) return rc;
  std::memset(p, 0, sizeof(*p));
  p->g = *g;
  p->gqa = g->num_q_heads / g->num_kv_heads;
  p->bh_total = g->batch * g->num_kv_heads;
  p->nF = windows(g->k_off_fp, g->n_fp, kTF, &p->wF0);
  p->n4 = windows(g->k_off_i4, g->n_i4, kTQ, &p->w40);
  p->n2 = windows(g->k_off_i2, g->n_i2, kTQ, &p->w20);
  p->nR = (g->recent_capacity + kTR - 1) / kTR;
  p->units = p->nF + p->n4 + p->n2 + p->nR;
  if (p->units == 0) return R2K_ERR_EMPTY;
  const int g2 = kD / g->v2_group;
  // Tile costs balance the CTAs' work.  The kernel is instruction-bound rather than byte-bound, so the weights
  // are measured per-tile times (ns of one CTA slot on B200, pure-pool caches), scaled down until a whole
  // (request, kv head) fits in 22 bits: the kernel's partition arithmetic is 32-bit.
  (void)g2;
  double ns[4] = {1400.0, 2110.0, 2400.0, 500.0};
  // R2K_TILE_NS="bf16,int4,int2,residual" in the environment overrides the weights (tuning runs)
  static const char* tile_ns_env = std::getenv("R2K_TILE_NS");
  if (tile_ns_env != nullptr) {
    double v[4];
    if (std::sscanf(tile_ns_env, "%lf,%lf,%lf,%lf", &v[0], &v[1], &v[2], &v[3]) == 4 && v[0] > 0 && v[1] > 0 && v[2] > 0 && v[3] > 0)
      for (int k = 0; k < 4; ++k) ns[k] = v[k];
  }
  const int64_t cnt[4] = {p->nF, p->n4, p->n2, p->nR};
  double scale = 100.0;
  uint32_t w[4];
  for (;;) {
    int64_t sum = 0;
    for (int k = 0; k < 4; ++k) {
      const double v = ns[k] / scale;
      w[k] = v < 1.0 ? 1u : (uint32_t)(v + 0.5);
      sum += cnt[k] * (int64_t)w[k];
    }
    if (sum < (1 << 22)) { p->c_bh = (uint32_t)sum; break; }
    if (w[0] == 1 && w[1] == 1 && w[2] == 1 && w[3] == 1) return R2K_ERR_GEOMETRY;  // > 4M tiles per head
    scale *= 2.0;
  }
  p->cF = w[0]; p->c4 = w[1]; p->c2 = w[2]; p->cR = w[3];
  const int64_t total_units = (int64_t)p->units * p->bh_total;
  int64_t cap = (int64_t)dev->sms * kCtasPerSm;
  const int env_cap = grid_cap_from_env();
  if (env_cap > 0 && env_cap < cap) cap = env_cap;
  p->grid = (int)(total_units < cap ? total_units : cap);
  // A whole number of CTAs per (request, kv head) -- no CTA then pays the partial/merge protocol twice -- when that
  // leaves at most one SM in twenty idle.  With many heads (64 heads on 148 SMs would use 128) the idle SMs cost
  // more than the CTAs that cross from one head into the next: measured 205 -> 193 us per launch for 16 requests
  // x 4 kv heads x 65536 tokens, against 31.7 -> 39 us for 8 x 2 x 32768 where rounding only idles 4 SMs.
  if (p->grid >= 2 * p->bh_total) {
    const int rounded = p->grid / p->bh_total * p->bh_total;
    if (rounded * 20 >= p->grid * 19) p->grid = rounded;
  }
  // More than kMergeGroup CTAs on a (request, kv head) pay a second merge level (a store, a ticket and one more
  // round of loads: ~2.6 us).  A head with so few tiles that kMergeGroup CTAs stream them in less extra time than
  // that gets kMergeGroup CTAs: measured 11.3 -> 10.0 us per launch for one request x 2 kv heads x 4096 tokens
  // (18 -> 9 CTAs per head).  The tile weights include fixed costs (about 1.5x the streaming time), hence 3 us.
  if (p->grid > kMergeGroup * p->bh_total) {
    double head_ns = 0.0;
    for (int k = 0; k < 4; ++k) head_ns += (double)cnt[k] * ns[k];
    const double per_head = (double)p->grid / p->bh_total;
    if (head_ns / kMergeGroup - head_ns / per_head < 3000.0) p->grid = kMergeGroup * p->bh_total;
  }
  if ((int64_t)p->grid * p->bh_total >= (int64_t)1 << 31) return R2K_ERR_GEOMETRY;
  p->parts_cap = (p->grid + p->bh_total - 1) / p->bh_total + 1;
  p->groups_cap = (p->parts_cap + kMergeGroup - 1) / kMergeGroup;
  p->groups2 = g2;
  p->group2_shift = ilog2(g->v2_group);
  p->kblock_shift = ilog2(g->k_block);
  const float sm = g->sm_scale > 0.f ? g->sm_scale : 0.08838834764831845f;
  p->qscale = sm * 1.4426950408889634f;
  return R2K_OK;
}

size_t counters_bytes(const DecodeParams& p) {
  const size_t n = ((size_t)(p.bh_total + p.g.batch + p.bh_total * p.groups_cap) * sizeof(int) + 255) / 256 * 256;
  return n < kWsCounterBlockBytes ? kWsCounterBlockBytes : n;
}
size_t workspace_need(const DecodeParams& p) {
  return kWsHeaderBytes + counters_bytes(p) +
         (size_t)p.bh_total * (p.parts_cap + p.groups_cap) * kSlotFloats * sizeof(float);
}

// ---- tensor map of the bf16-value pool -------------------------------------------------------------------
// Encoded through the driver entry point (no link against the driver library); the last few maps are kept,
// keyed by everything that goes into them, because callers decode with the same cache many times.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
struct FpMapKey {
  const void* base; int64_t bstride; int32_t capacity, heads, batch;
  bool operator==(const FpMapKey& o) const {
    return base == o.base && bstride == o.bstride && capacity == o.capacity && heads == o.heads && batch == o.batch;
  }
};
struct FpMapEntry { FpMapKey key; CUtensorMap map; bool used = false; };
std::mutex g_map_mutex;
FpMapEntry g_maps[8];
int g_map_next = 0;

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &res) != cudaSuccess ||
        res != cudaDriverEntryPointSuccess)
      sym = nullptr;
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}

// Fills p->fp_map / p->fp_tma.  Any reason the map cannot be built (no pool, unaligned base or stride, no driver
// entry point) leaves fp_tma = 0 and the kernel on its plain-load path for bf16-value tiles.
void bind_fp_map(DecodeParams* p) {
  p->fp_tma = 0;
  const R2KGeom& g = p->g;
  if (g.n_fp <= 0 || g.fp_capacity <= 0 || p->v.fp_v == nullptr) return;
  const int64_t bstride = g.batch > 1 ? p->v.fp_v_bstride : (int64_t)g.fp_capacity * g.num_kv_heads * 256;
  if ((reinterpret_cast<uintptr_t>(p->v.fp_v) & 15u) || bstride <= 0 || (bstride & 15)) return;
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return;
  const FpMapKey key{p->v.fp_v, bstride, g.fp_capacity, g.num_kv_heads, g.batch};
  std::lock_guard<std::mutex> lock(g_map_mutex);
  for (const FpMapEntry& e : g_maps)
    if (e.used && e.key == key) { p->fp_map = e.map; p->fp_tma = 1; return; }
  const cuuint64_t dims[4] = {128, (cuuint64_t)g.fp_capacity, (cuuint64_t)g.num_kv_heads, (cuuint64_t)g.batch};
  const cuuint64_t strides[3] = {256, (cuuint64_t)g.fp_capacity * 256, (cuuint64_t)bstride};
  const cuuint32_t box[4] = {64, (cuuint32_t)kTF, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMap map;
  if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void*>(p->v.fp_v), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return;
  FpMapEntry& slot = g_maps[g_map_next];
  g_map_next = (g_map_next + 1) % 8;
  slot.key = key; slot.map = map; slot.used = true;
  p->fp_map = map;
  p->fp_tma = 1;
}

template <bool BF16>
int launch_pack_k(const PackArgs& a, int batch, uint8_t* packed, void* scale, uint8_t* zero, int64_t pb, int64_t sb, int64_t zb,
                  int k_block, cudaStream_t st) {
  const int64_t first = a.dst_start / k_block, last = (a.dst_start + a.count - 1) / k_block;
  dim3 grid((unsigned)(last - first + 1), (unsigned)a.num_heads, (unsigned)batch);
  pack_k_int4_kernel<BF16><<<grid, 64, (size_t)k_block * 256, st>>>(a, packed, reinterpret_cast<__half*>(scale), zero, pb, sb, zb, k_block, first);
  ++g_launches;
  return cudaGetLastError() == cudaSuccess ? R2K_OK : R2K_ERR_CUDA;
}
// A launch that may start while the kernel in front of it on the stream is still running, once that kernel has
// let its dependents go (programmatic stream serialization); `overlap` false gives an ordinary launch.
template <typename... Params, typename... Args>
cudaError_t launch_behind(void (*kernel)(Params...), dim3 grid, dim3 block, cudaStream_t st, bool overlap, Args... args) {
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = overlap ? 1 : 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

template <bool BF16>
int launch_pack_v2(const PackArgs& a, int batch, uint8_t* packed, void* scale, uint8_t* zero, int64_t pb, int64_t sb, int64_t zb,
                   int group, cudaStream_t st, bool overlap = false) {
  dim3 grid((unsigned)((a.count + 3) / 4), (unsigned)a.num_heads, (unsigned)batch);
  const cudaError_t err = launch_behind(pack_v_int2_kernel<BF16>, grid, dim3(128), st, overlap, a, packed,
                                        reinterpret_cast<__half*>(scale), zero, pb, sb, zb, group);
  ++g_launches;
  return err == cudaSuccess ? R2K_OK : R2K_ERR_CUDA;
}

RingArgs ring_args(const R2KGeom* g, const R2KCacheView* v) {
  RingArgs r;
  r.recent_k = reinterpret_cast<uint8_t*>(v->recent_k);
  r.recent_v = reinterpret_cast<uint8_t*>(v->recent_v);
  r.recent_len = v->recent_len;
  r.recent_global = v->recent_global;
  r.recent_logical = v->recent_logical;
  r.recent_page_lengths = v->recent_page_lengths;
  r.k_bstride = v->recent_k_bstride; r.v_bstride = v->recent_v_bstride; r.len_bstride = v->recent_len_bstride;
  r.global_bstride = v->recent_global_bstride; r.logical_bstride = v->recent_logical_bstride;
  r.page_bstride = v->recent_page_lengths_bstride;
  r.num_heads = g->num_kv_heads; r.capacity = g->recent_capacity; r.page_size = g->page_size;
  return r;
}

int check_ring(const R2KGeom* g, const R2KCacheView* v) {
  if (!v->recent_k || !v->recent_v || !v->recent_len || !v->recent_global || !v->recent_logical || !v->recent_page_lengths)
    return R2K_ERR_NULL;
  if (!aligned16(v->recent_k) || !aligned16(v->recent_v) || (v->recent_k_bstride & 15) || (v->recent_v_bstride & 15))
    return R2K_ERR_ALIGNMENT;
  if ((v->recent_len_bstride & 3) || (v->recent_global_bstride & 7) || (v->recent_logical_bstride & 7) ||
      (v->recent_page_lengths_bstride & 7))
    return R2K_ERR_ALIGNMENT;
  (void)g;
  return R2K_OK;
}

}  // namespace
}  // namespace r2k

using namespace r2k;

extern "C" {

const char* r2k_status_string(int status) {
  switch (status) {
    case R2K_OK: return "ok";
    case R2K_ERR_NULL: return "required pointer is NULL";
    case R2K_ERR_GEOMETRY: return "unsupported or inconsistent geometry";
    case R2K_ERR_ALIGNMENT: return "pointer or stride is not sufficiently aligned";
    case R2K_ERR_CAPACITY: return "capacity exhausted";
    case R2K_ERR_WORKSPACE: return "workspace too small";
    case R2K_ERR_CUDA: return "CUDA runtime error";
    case R2K_ERR_DEVICE_TIMEOUT: return "bounded device-side wait timed out";
    case R2K_ERR_EMPTY: return "cache holds no tokens";
    default: return "unknown status";
  }
}

uint64_t r2k_launch_count(void) { return g_launches.load(); }

int r2k_decode_workspace_bytes(const R2KGeom* geom, size_t* bytes) {
  if (bytes == nullptr) return R2K_ERR_NULL;
  int rc = check_geom(geom);
  if (rc) return rc;
  DecodeParams p;
  rc = derive(geom, &p);
  if (rc) return rc;
  *bytes = workspace_need(p);
  return R2K_OK;
}

int r2k_decode_workspace_init(void* workspace, size_t bytes, void* stream) {
  if (workspace == nullptr) return R2K_ERR_NULL;
  if (bytes < (size_t)kWsHeaderBytes) return R2K_ERR_WORKSPACE;
  // header + counters: clear everything in front of the partial slots that this workspace could ever hold
  size_t n = bytes < (size_t)(1 << 20) ? bytes : (size_t)(1 << 20);
  return cudaMemsetAsync(workspace, 0, n, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess ? R2K_OK : R2K_ERR_CUDA;
}

static size_t exchange_states_bytes(const R2KGeom* g, int world) {
  const size_t n = (size_t)2 * world * g->batch * g->num_q_heads * 130 * sizeof(uint2);   // (value, step) words
  return (n + 127) / 128 * 128;
}

static int decode_impl(const R2KGeom* geom, const R2KCacheView* view, const void* q, const R2KAppend* append, void* workspace,
                       size_t workspace_bytes, void* out, uint32_t flags, const R2KExchange* ex, void* stream) {
  if (view == nullptr || q == nullptr || workspace == nullptr || out == nullptr) return R2K_ERR_NULL;
  int rc = check_geom(geom);
  if (rc) return rc;
  DecodeParams p;
  rc = derive(geom, &p);
  if (rc) return rc;
  if (workspace_bytes < workspace_need(p)) return R2K_ERR_WORKSPACE;
  if (!aligned16(workspace) || !aligned16(q) || !aligned16(out)) return R2K_ERR_ALIGNMENT;
  const bool need_k = geom->n_fp + geom->n_i4 + geom->n_i2 > 0;
  if (need_k && (!view->k_packed || !view->k_scale || !view->k_zero)) return R2K_ERR_NULL;
  if (geom->n_fp && !view->fp_v) return R2K_ERR_NULL;
  if (geom->n_i4 && (!view->i4_packed || !view->i4_scale)) return R2K_ERR_NULL;
  if (geom->n_i2 && (!view->i2_packed || !view->i2_scale || !view->i2_zero)) return R2K_ERR_NULL;
  if (geom->recent_capacity > 0) {
    rc = check_ring(geom, view);
    if (rc) return rc;
  } else if (!view->recent_len) {
    return R2K_ERR_NULL;
  }
  if (!aligned16(view->k_packed) || !aligned16(view->k_scale) || !aligned16(view->k_zero) || !aligned16(view->fp_v) ||
      !aligned16(view->i4_packed) || !aligned16(view->i2_packed))
    return R2K_ERR_ALIGNMENT;
  if ((view->k_packed_bstride | view->k_scale_bstride | view->k_zero_bstride | view->fp_v_bstride | view->i4_packed_bstride |
       view->i2_packed_bstride) & 15)
    return R2K_ERR_ALIGNMENT;
  p.v = *view;
  p.q = q;
  if (append != nullptr && append->k != nullptr) {
    if (append->v == nullptr) return R2K_ERR_NULL;
    if (geom->recent_capacity <= 0) return R2K_ERR_CAPACITY;
    if (!aligned16(append->k) || !aligned16(append->v)) return R2K_ERR_ALIGNMENT;
    p.app_k = append->k; p.app_v = append->v; p.app_idx = append->indices;
    p.app_global = append->global_index; p.app_logical = append->logical_position;
  }
  p.out = out;
  p.flags = flags;
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  p.err = reinterpret_cast<int*>(ws);
  p.bh_counter = reinterpret_cast<int*>(ws + kWsHeaderBytes);
  p.req_counter = p.bh_counter + p.bh_total;
  p.group_counter = p.req_counter + p.g.batch;
  p.partials = reinterpret_cast<float*>(ws + kWsHeaderBytes + counters_bytes(p));
  p.group_partials = p.partials + (size_t)p.bh_total * p.parts_cap * kSlotFloats;
  bind_fp_map(&p);
  if (ex != nullptr && ex->world > 1) {
    if (ex->world > R2K_MAX_RANKS || ex->rank < 0 || ex->rank >= ex->world || (flags & R2K_FLAG_OUT_STATE)) return R2K_ERR_GEOMETRY;
    for (int r = 0; r < ex->world; ++r) {
      if (ex->buffers[r] == nullptr) return R2K_ERR_NULL;
      if (!aligned16(ex->buffers[r])) return R2K_ERR_ALIGNMENT;
      p.xbuf[r] = reinterpret_cast<float*>(ex->buffers[r]);
    }
    p.xw = ex->world; p.xrank = ex->rank; p.xseq = ex->seq;
    // wait budget -> sleep between polls (the number of polls is fixed); a poll itself takes about a microsecond
    p.xnap = kExchangeNapNs;
    if (ex->wait_us != 0) {
      const uint64_t nap = (uint64_t)ex->wait_us * 1000u / kExchangePolls;
      p.xnap = nap > 1000000u ? 1000000u : (uint32_t)nap;
    }
    p.xflags_off = (uint32_t)exchange_states_bytes(geom, ex->world);
  }

  DeviceInfo* dev;
  rc = device_info(&dev);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // Programmatic stream serialization: when the previous kernel of the stream signals early (a decode launch
  // does), this grid's CTAs may start on free SMs and prefetch pool tiles; the kernel itself waits for the
  // previous kernel's completion before it reads anything that kernel can have written.
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = dev->pdl ? 1 : 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)p.grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t err = geom->dtype == R2K_DTYPE_BF16 ? cudaLaunchKernelEx(&cfg, decode_kernel<true>, p)
                                                        : cudaLaunchKernelEx(&cfg, decode_kernel<false>, p);
  ++g_launches;
  return err == cudaSuccess ? R2K_OK : R2K_ERR_CUDA;
}

int r2k_decode(const R2KGeom* geom, const R2KCacheView* view, const void* q, const R2KAppend* append, void* workspace,
               size_t workspace_bytes, void* out, uint32_t flags, void* stream) {
  return decode_impl(geom, view, q, append, workspace, workspace_bytes, out, flags, nullptr, stream);
}

namespace {
constexpr int kHostZeroCopyDefault = 6;   // inputs brought in by a copy kernel, result written in place: measured fastest
// q | k | v | out, each rounded up to 256 bytes
struct HostStaging { size_t q, kv, in_bytes, out_off, out_max, total; };
bool host_staging(const R2KGeom* g, HostStaging& s) {
  if (g == nullptr || g->batch < 1 || g->num_q_heads < 1 || g->num_kv_heads < 1) return false;
  s.q = (size_t)g->batch * g->num_q_heads * 128 * 2;
  s.kv = (size_t)g->batch * g->num_kv_heads * 128 * 2;
  s.in_bytes = s.q + 2 * s.kv;
  s.out_off = (s.in_bytes + 255) & ~(size_t)255;
  s.out_max = (size_t)g->batch * g->num_q_heads * 130 * 4;
  s.total = s.out_off + ((s.out_max + 255) & ~(size_t)255);
  return true;
}
}  // namespace

int r2k_decode_host_staging_bytes(const R2KGeom* geom, size_t* bytes) {
  HostStaging s;
  if (bytes == nullptr) return R2K_ERR_NULL;
  if (!host_staging(geom, s)) return R2K_ERR_GEOMETRY;
  *bytes = s.total;
  return R2K_OK;
}

int r2k_decode_host(const R2KGeom* geom, const R2KCacheView* view, const void* host_in, const R2KAppend* append,
                    void* workspace, size_t workspace_bytes, void* staging, size_t staging_bytes, void* host_out,
                    uint32_t flags, void* stream) {
  if (geom == nullptr || host_in == nullptr || host_out == nullptr || staging == nullptr) return R2K_ERR_NULL;
  HostStaging s;
  if (!host_staging(geom, s)) return R2K_ERR_GEOMETRY;
  if (staging_bytes < s.total) return R2K_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(staging) & 15u) return R2K_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* dev = static_cast<uint8_t*>(staging);
  const size_t rows = (size_t)geom->batch * geom->num_q_heads;
  const size_t out_bytes = (flags & R2K_FLAG_OUT_STATE) ? rows * 130 * 4 : (flags & R2K_FLAG_OUT_F32) ? rows * 128 * 4 : rows * 128 * 2;
  // Page-locked, device-mapped host buffers can be used by the kernel in place (its accesses to q, the new rows
  // and the result are plain loads and stores): bit 0 of R2K_HOST_ZERO_COPY lets it read host_in over PCIe, bit 1
  // lets it write host_out; bit 2 brings host_in into `staging` with a small copy kernel instead of a memcpy, so
  // that the decode launch behind it (programmatic stream serialization) overlaps the transfer with its prologue.
  // A buffer that is not mapped (or pageable) takes the memcpy.
  static const int zero_copy = [] { const char* e = getenv("R2K_HOST_ZERO_COPY"); return e ? atoi(e) : kHostZeroCopyDefault; }();
  auto mapped = [](const void* p) -> uint8_t* {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return a.type == cudaMemoryTypeHost ? static_cast<uint8_t*>(a.devicePointer) : nullptr;
  };
  uint8_t* in = (zero_copy & 1) ? mapped(host_in) : nullptr;
  uint8_t* out = (zero_copy & 2) ? mapped(host_out) : nullptr;
  if (in != nullptr && (reinterpret_cast<uintptr_t>(in) & 15u)) in = nullptr;
  if (out != nullptr && (reinterpret_cast<uintptr_t>(out) & 15u)) out = nullptr;
  if (in == nullptr) {
    const size_t in_bytes = append ? s.in_bytes : s.q;
    uint8_t* src = (zero_copy & 4) ? mapped(host_in) : nullptr;
    if (src != nullptr && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {   // bit 2: a copy kernel the decode launch overlaps
      const int n16 = (int)(in_bytes / 16);
      host_block_copy_kernel<<<(n16 + 255) / 256, 256, 0, st>>>(reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dev), n16);
      ++g_launches;
      if (cudaGetLastError() != cudaSuccess) return R2K_ERR_CUDA;
    } else if (cudaMemcpyAsync(dev, host_in, in_bytes, cudaMemcpyHostToDevice, st) != cudaSuccess) {
      return R2K_ERR_CUDA;
    }
    in = dev;
  }
  R2KAppend dev_append;
  if (append != nullptr) {
    dev_append = *append;
    dev_append.k = in + s.q;
    dev_append.v = in + s.q + s.kv;
  }
  const int status = decode_impl(geom, view, in, append ? &dev_append : nullptr, workspace, workspace_bytes,
                                 out ? out : dev + s.out_off, flags, nullptr, stream);
  if (status != R2K_OK) return status;
  if (out == nullptr && cudaMemcpyAsync(host_out, dev + s.out_off, out_bytes, cudaMemcpyDeviceToHost, st) != cudaSuccess)
    return R2K_ERR_CUDA;
  return cudaStreamSynchronize(st) == cudaSuccess ? R2K_OK : R2K_ERR_CUDA;
}

int r2k_decode_exchange(const R2KGeom* geom, const R2KCacheView* view, const void* q, const R2KAppend* append, void* workspace,
                        size_t workspace_bytes, void* out, uint32_t flags, const R2KExchange* exchange, void* stream) {
  if (exchange == nullptr) return R2K_ERR_NULL;
  if (exchange->world < 1) return R2K_ERR_GEOMETRY;
  return decode_impl(geom, view, q, append, workspace, workspace_bytes, out, flags, exchange, stream);
}

int r2k_exchange_bytes(const R2KGeom* geom, int32_t world, size_t* bytes) {
  if (bytes == nullptr) return R2K_ERR_NULL;
  int rc = check_geom(geom);
  if (rc) return rc;
  if (world < 1 || world > R2K_MAX_RANKS) return R2K_ERR_GEOMETRY;
  *bytes = exchange_states_bytes(geom, world) + 128;   // + device step counter
  return R2K_OK;
}

int r2k_exchange_create(size_t bytes, void** buffer, unsigned char handle[64]) {
  if (buffer == nullptr || handle == nullptr) return R2K_ERR_NULL;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "inter-process handle size");
  if (bytes == 0) return R2K_ERR_GEOMETRY;
  void* ptr = nullptr;
  if (cudaMalloc(&ptr, bytes) != cudaSuccess) return R2K_ERR_CUDA;
  cudaIpcMemHandle_t h;
  if (cudaMemset(ptr, 0, bytes) != cudaSuccess || cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) {
    cudaFree(ptr);
    return R2K_ERR_CUDA;
  }
  std::memcpy(handle, &h, 64);
  *buffer = ptr;
  return R2K_OK;
}

int r2k_exchange_open(const unsigned char handle[64], void** buffer) {
  if (buffer == nullptr || handle == nullptr) return R2K_ERR_NULL;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  void* ptr = nullptr;
  if (cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return R2K_ERR_CUDA;
  *buffer = ptr;
  return R2K_OK;
}

int r2k_exchange_close(void* buffer, int32_t opened) {
  if (buffer == nullptr) return R2K_OK;
  const cudaError_t e = opened ? cudaIpcCloseMemHandle(buffer) : cudaFree(buffer);
  return e == cudaSuccess ? R2K_OK : R2K_ERR_CUDA;
}

}  // extern "C"

// Scratch of r2k_decode_static.  In host code this name is only a handle: the device address comes from
// cudaGetSymbolAddress, per device (device code may name the array directly).
static __device__ __align__(256) unsigned char g_static_workspace[R2K_STATIC_WORKSPACE_BYTES];

namespace {
std::mutex g_static_mutex;
void* g_static_ptr[64] = {};
constexpr size_t kStaticHeadBytes = kWsHeaderBytes + kWsCounterBlockBytes;   // status word + arrival counters

// Device address of the static scratch on the current device.  The first call on a device resolves it
// (cudaGetSymbolAddress with that device current) and clears the status word and the counters on `stream`.
int static_workspace(void** out, cudaStream_t stream) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return R2K_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_workspace) != cudaSuccess || p == nullptr) return R2K_ERR_CUDA;
    if (cudaMemsetAsync(p, 0, kStaticHeadBytes, stream) != cudaSuccess) return R2K_ERR_CUDA;
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return R2K_OK;
}
}  // namespace

extern "C" {

int r2k_decode_static(const R2KGeom* geom, const R2KCacheView* view, const void* q, const R2KAppend* append, void* out,
                      uint32_t flags, void* stream) {
  size_t need = 0;
  int rc = r2k_decode_workspace_bytes(geom, &need);
  if (rc) return rc;
  if (need > (size_t)R2K_STATIC_WORKSPACE_BYTES) return R2K_ERR_WORKSPACE;
  void* ptr = nullptr;
  rc = static_workspace(&ptr, reinterpret_cast<cudaStream_t>(stream));
  if (rc) return rc;
  return r2k_decode(geom, view, q, append, ptr, (size_t)R2K_STATIC_WORKSPACE_BYTES, out, flags, stream);
}

int r2k_decode_static_status(int32_t* status, void* stream) {
  void* ptr = nullptr;
  const int rc = static_workspace(&ptr, reinterpret_cast<cudaStream_t>(stream));
  if (rc) return rc;
  return r2k_decode_device_status(ptr, status, stream);
}

int r2k_decode_static_reset(void* stream) {
  void* ptr = nullptr;
  const int rc = static_workspace(&ptr, reinterpret_cast<cudaStream_t>(stream));
  if (rc) return rc;
  return cudaMemsetAsync(ptr, 0, kStaticHeadBytes, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess ? R2K_OK : R2K_ERR_CUDA;
}

int r2k_decode_device_status(void* workspace, int32_t* status, void* stream) {
  if (workspace == nullptr || status == nullptr) return R2K_ERR_NULL;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(status, workspace, sizeof(int32_t), cudaMemcpyDeviceToHost, st) != cudaSuccess) return R2K_ERR_CUDA;
  return cudaStreamSynchronize(st) == cudaSuccess ? R2K_OK : R2K_ERR_CUDA;
}

int r2k_merge_states(const float* states, int32_t num_states, int64_t state_stride, int32_t rows, int32_t dtype, void* out,
                     uint32_t flags, void* stream) {
  if (states == nullptr || out == nullptr) return R2K_ERR_NULL;
  if (num_states < 1 || rows < 1 || (dtype != R2K_DTYPE_BF16 && dtype != R2K_DTYPE_FP16)) return R2K_ERR_GEOMETRY;
  if ((reinterpret_cast<uintptr_t>(states) & 7u) || (state_stride & 1) || !aligned16(out)) return R2K_ERR_ALIGNMENT;
  merge_states_kernel<<<(rows + 3) / 4, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(states, num_states, state_stride, rows,
                                                                                         dtype, out, flags);
  ++g_launches;
  return cudaGetLastError() == cudaSuccess ? R2K_OK : R2K_ERR_CUDA;
}

static int check_pack(const void* src, int32_t dtype, int32_t heads, int64_t src_rows, int64_t count, int64_t capacity,
                      int64_t dst_start) {
  if (src == nullptr) return R2K_ERR_NULL;
  if (dtype != R2K_DTYPE_BF16 && dtype != R2K_DTYPE_FP16) return R2K_ERR_GEOMETRY;
  if (heads < 1 || src_rows < 0 || count < 0 || dst_start < 0) return R2K_ERR_GEOMETRY;
  if (dst_start + count > capacity) return R2K_ERR_CAPACITY;
  if (reinterpret_cast<uintptr_t>(src) & 7u) return R2K_ERR_ALIGNMENT;
  return R2K_OK;
}

int r2k_pack_k_int4(const void* src, int32_t dtype, int32_t num_kv_heads, int64_t src_rows, const int64_t* index, int64_t count,
                    uint8_t* k_packed, void* k_scale, uint8_t* k_zero, int64_t k_capacity, int32_t k_block, int64_t dst_start,
                    void* stream) {
  int rc = check_pack(src, dtype, num_kv_heads, src_rows, count, k_capacity, dst_start);
  if (rc) return rc;
  if (!k_packed || !k_scale || !k_zero) return R2K_ERR_NULL;
  if (!pow2_in(k_block, 32, 64, 128) || k_capacity % k_block) return R2K_ERR_GEOMETRY;
  if (count == 0) return R2K_OK;
  PackArgs a{reinterpret_cast<const uint16_t*>(src), 0, src_rows, index, count, k_capacity, dst_start, num_kv_heads};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return dtype == R2K_DTYPE_BF16 ? launch_pack_k<true>(a, 1, k_packed, k_scale, k_zero, 0, 0, 0, k_block, st)
                                 : launch_pack_k<false>(a, 1, k_packed, k_scale, k_zero, 0, 0, 0, k_block, st);
}

int r2k_pack_v_int4(const void* src, int32_t dtype, int32_t num_kv_heads, int64_t src_rows, const int64_t* index, int64_t count,
                    uint8_t* packed, float* scale, int64_t capacity, int64_t dst_start, void* stream) {
  int rc = check_pack(src, dtype, num_kv_heads, src_rows, count, capacity, dst_start);
  if (rc) return rc;
  if (!packed || !scale) return R2K_ERR_NULL;
  if (count == 0) return R2K_OK;
  PackArgs a{reinterpret_cast<const uint16_t*>(src), 0, src_rows, index, count, capacity, dst_start, num_kv_heads};
  dim3 grid((unsigned)((count + 3) / 4), (unsigned)num_kv_heads, 1);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == R2K_DTYPE_BF16) pack_v_int4_kernel<true><<<grid, 128, 0, st>>>(a, packed, scale, 0, 0);
  else pack_v_int4_kernel<false><<<grid, 128, 0, st>>>(a, packed, scale, 0, 0);
  ++g_launches;
  return cudaGetLastError() == cudaSuccess ? R2K_OK : R2K_ERR_CUDA;
}

int r2k_pack_v_int2(const void* src, int32_t dtype, int32_t num_kv_heads, int64_t src_rows, const int64_t* index, int64_t count,
                    uint8_t* packed, void* scale, uint8_t* zero, int64_t capacity, int32_t group, int64_t dst_start, void* stream) {
  int rc = check_pack(src, dtype, num_kv_heads, src_rows, count, capacity, dst_start);
  if (rc) return rc;
  if (!packed || !scale || !zero) return R2K_ERR_NULL;
  if (!pow2_in(group, 32, 64, 128)) return R2K_ERR_GEOMETRY;
  if (count == 0) return R2K_OK;
  PackArgs a{reinterpret_cast<const uint16_t*>(src), 0, src_rows, index, count, capacity, dst_start, num_kv_heads};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return dtype == R2K_DTYPE_BF16 ? launch_pack_v2<true>(a, 1, packed, scale, zero, 0, 0, 0, group, st)
                                 : launch_pack_v2<false>(a, 1, packed, scale, zero, 0, 0, 0, group, st);
}

int r2k_gather_rows(const void* src, int32_t num_kv_heads, int64_t src_rows, const int64_t* index, int64_t count, void* dst,
                    int64_t dst_rows, int64_t dst_start, void* stream) {
  if (src == nullptr || dst == nullptr) return R2K_ERR_NULL;
  if (num_kv_heads < 1 || count < 0 || dst_start < 0) return R2K_ERR_GEOMETRY;
  if (dst_start + count > dst_rows) return R2K_ERR_CAPACITY;
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 7u) return R2K_ERR_ALIGNMENT;
  if (count == 0) return R2K_OK;
  dim3 grid((unsigned)((count + 3) / 4), (unsigned)num_kv_heads, 1);
  gather_rows_kernel<<<grid, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint16_t*>(src), src_rows, index, count, reinterpret_cast<uint16_t*>(dst), dst_rows, dst_start);
  ++g_launches;
  return cudaGetLastError() == cudaSuccess ? R2K_OK : R2K_ERR_CUDA;
}

int r2k_fwht128(const void* in, void* out, int32_t dtype, int64_t rows, void* stream) {
  if (in == nullptr || out == nullptr) return R2K_ERR_NULL;
  if (rows < 0 || (dtype != R2K_DTYPE_BF16 && dtype != R2K_DTYPE_FP16)) return R2K_ERR_GEOMETRY;
  if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 7u) return R2K_ERR_ALIGNMENT;
  if (rows == 0) return R2K_OK;
  const unsigned grid = (unsigned)((rows + 3) / 4);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == R2K_DTYPE_BF16)
    fwht128_kernel<true><<<grid, 128, 0, st>>>(reinterpret_cast<const uint16_t*>(in), reinterpret_cast<uint16_t*>(out), rows);
  else
    fwht128_kernel<false><<<grid, 128, 0, st>>>(reinterpret_cast<const uint16_t*>(in), reinterpret_cast<uint16_t*>(out), rows);
  ++g_launches;
  return cudaGetLastError() == cudaSuccess ? R2K_OK : R2K_ERR_CUDA;
}

int r2k_qk_mrope(const void* q, const void* k, void* q_out, void* k_out, int32_t dtype, int32_t batch, int32_t num_q_heads,
                 int32_t num_kv_heads, int32_t tokens, const void* cos, const void* sin, int32_t rot_dtype,
                 const int64_t cos_strides[4], const int64_t sin_strides[4], int32_t section0, int32_t section1,
                 int32_t apply_hadamard, void* stream) {
  if (!q || !k || !q_out || !k_out || !cos || !sin || !cos_strides || !sin_strides) return R2K_ERR_NULL;
  if ((dtype != R2K_DTYPE_BF16 && dtype != R2K_DTYPE_FP16) || (rot_dtype != R2K_DTYPE_BF16 && rot_dtype != R2K_DTYPE_FP16 && rot_dtype != 2))
    return R2K_ERR_GEOMETRY;
  if (batch < 1 || num_q_heads < 1 || num_kv_heads < 1 || tokens < 1) return R2K_ERR_GEOMETRY;
  if (section0 < 0 || section1 < 0 || section0 + section1 > 64) return R2K_ERR_GEOMETRY;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(q_out) |
       reinterpret_cast<uintptr_t>(k_out)) & 7u)
    return R2K_ERR_ALIGNMENT;
  MropeArgs a;
  a.q = reinterpret_cast<const uint16_t*>(q); a.k = reinterpret_cast<const uint16_t*>(k);
  a.q_out = reinterpret_cast<uint16_t*>(q_out); a.k_out = reinterpret_cast<uint16_t*>(k_out);
  a.cos = cos; a.sin = sin;
  for (int i = 0; i < 4; ++i) { a.cos_stride[i] = cos_strides[i]; a.sin_stride[i] = sin_strides[i]; }
  a.batch = batch; a.hq = num_q_heads; a.hkv = num_kv_heads; a.tokens = tokens;
  a.section0 = section0; a.section1 = section1; a.rot_dtype = rot_dtype; a.hadamard = apply_hadamard ? 1 : 0;
  a.v = nullptr; a.v_out = nullptr; a.v_hadamard = 0; a.v_bstride = 0;
  a.q_bstride = (int64_t)num_q_heads * tokens * 128; a.k_bstride = (int64_t)num_kv_heads * tokens * 128;
  const int64_t rows = (int64_t)batch * (num_q_heads + num_kv_heads) * tokens;
  const unsigned grid = (unsigned)((rows + 3) / 4);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == R2K_DTYPE_BF16) mrope_rows_kernel<true><<<grid, 128, 0, st>>>(a);
  else mrope_rows_kernel<false><<<grid, 128, 0, st>>>(a);
  ++g_launches;
  return cudaGetLastError() == cudaSuccess ? R2K_OK : R2K_ERR_CUDA;
}

int r2k_qkv_prologue(const void* q, int64_t q_bstride, const void* k, int64_t k_bstride, const void* v, int64_t v_bstride,
                     void* q_out, void* k_out, void* v_out, int32_t dtype, int32_t batch, int32_t num_q_heads,
                     int32_t num_kv_heads, const void* cos, const void* sin, int32_t rot_dtype, const int64_t cos_strides[4],
                     const int64_t sin_strides[4], int32_t section0, int32_t section1, int32_t key_hadamard,
                     int32_t value_hadamard, void* stream) {
  if (!q || !k || !v || !q_out || !k_out || !v_out || !cos || !sin || !cos_strides || !sin_strides) return R2K_ERR_NULL;
  if ((dtype != R2K_DTYPE_BF16 && dtype != R2K_DTYPE_FP16) || (rot_dtype != R2K_DTYPE_BF16 && rot_dtype != R2K_DTYPE_FP16 && rot_dtype != 2))
    return R2K_ERR_GEOMETRY;
  if (batch < 1 || num_q_heads < 1 || num_kv_heads < 1) return R2K_ERR_GEOMETRY;
  if (section0 < 0 || section1 < 0 || section0 + section1 > 64) return R2K_ERR_GEOMETRY;
  if (q_bstride < (int64_t)num_q_heads * 128 || k_bstride < (int64_t)num_kv_heads * 128 || v_bstride < (int64_t)num_kv_heads * 128)
    return R2K_ERR_GEOMETRY;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_out) | reinterpret_cast<uintptr_t>(v_out)) & 7u)
    return R2K_ERR_ALIGNMENT;
  if ((q_bstride | k_bstride | v_bstride) & 3) return R2K_ERR_ALIGNMENT;   // 8-byte loads of four channels
  MropeArgs a;
  a.q = reinterpret_cast<const uint16_t*>(q); a.k = reinterpret_cast<const uint16_t*>(k); a.v = reinterpret_cast<const uint16_t*>(v);
  a.q_out = reinterpret_cast<uint16_t*>(q_out); a.k_out = reinterpret_cast<uint16_t*>(k_out); a.v_out = reinterpret_cast<uint16_t*>(v_out);
  a.q_bstride = q_bstride; a.k_bstride = k_bstride; a.v_bstride = v_bstride;
  a.cos = cos; a.sin = sin;
  for (int i = 0; i < 4; ++i) { a.cos_stride[i] = cos_strides[i]; a.sin_stride[i] = sin_strides[i]; }
  a.batch = batch; a.hq = num_q_heads; a.hkv = num_kv_heads; a.tokens = 1;
  a.section0 = section0; a.section1 = section1; a.rot_dtype = rot_dtype;
  a.hadamard = key_hadamard ? 1 : 0; a.v_hadamard = value_hadamard ? 1 : 0;
  const int64_t rows = (int64_t)batch * (num_q_heads + 2 * num_kv_heads);
  const unsigned grid = (unsigned)((rows + 3) / 4);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == R2K_DTYPE_BF16) mrope_rows_kernel<true><<<grid, 128, 0, st>>>(a);
  else mrope_rows_kernel<false><<<grid, 128, 0, st>>>(a);
  ++g_launches;
  return cudaGetLastError() == cudaSuccess ? R2K_OK : R2K_ERR_CUDA;
}

int r2k_append_recent(const R2KGeom* geom, const R2KCacheView* view, const R2KAppend* append, void* stream) {
  if (view == nullptr || append == nullptr || append->k == nullptr || append->v == nullptr) return R2K_ERR_NULL;
  int rc = check_geom(geom);
  if (rc) return rc;
  if (geom->recent_capacity <= 0) return R2K_ERR_CAPACITY;
  rc = check_ring(geom, view);
  if (rc) return rc;
  if (!aligned16(append->k) || !aligned16(append->v)) return R2K_ERR_ALIGNMENT;
  append_recent_kernel<<<geom->batch, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      ring_args(geom, view), reinterpret_cast<const uint8_t*>(append->k), reinterpret_cast<const uint8_t*>(append->v),
      append->indices, append->global_index, append->logical_position);
  ++g_launches;
  return cudaGetLastError() == cudaSuccess ? R2K_OK : R2K_ERR_CUDA;
}

int r2k_flush_recent(const R2KGeom* geom, const R2KCacheView* view, int32_t ring_tokens, int32_t flush_tokens, int64_t k_dst,
                     int64_t v_dst, int64_t* i2_global, int64_t* i2_logical, int64_t meta_bstride, int64_t v_meta_dst,
                     void* stream) {
  if (view == nullptr) return R2K_ERR_NULL;
  int rc = check_geom(geom);
  if (rc) return rc;
  rc = check_ring(geom, view);
  if (rc) return rc;
  if (flush_tokens < 1 || ring_tokens < flush_tokens || ring_tokens > geom->recent_capacity) return R2K_ERR_GEOMETRY;
  if (k_dst < 0 || v_dst < 0 || k_dst + flush_tokens > geom->k_capacity || v_dst + flush_tokens > geom->i2_capacity)
    return R2K_ERR_CAPACITY;
  if (!view->k_packed || !view->k_scale || !view->k_zero || !view->i2_packed || !view->i2_scale || !view->i2_zero)
    return R2K_ERR_NULL;
  if ((i2_global == nullptr) != (i2_logical == nullptr)) return R2K_ERR_NULL;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  DeviceInfo* dev;
  rc = device_info(&dev);
  if (rc) return rc;
  const bool bf16 = geom->dtype == R2K_DTYPE_BF16;
  PackArgs ka{reinterpret_cast<const uint16_t*>(view->recent_k), view->recent_k_bstride, geom->recent_capacity, nullptr,
              flush_tokens, geom->k_capacity, k_dst, geom->num_kv_heads};
  uint8_t* kp = const_cast<uint8_t*>(view->k_packed);
  void* ks = const_cast<void*>(view->k_scale);
  uint8_t* kz = const_cast<uint8_t*>(view->k_zero);
  rc = bf16 ? launch_pack_k<true>(ka, geom->batch, kp, ks, kz, view->k_packed_bstride, view->k_scale_bstride, view->k_zero_bstride,
                                  geom->k_block, st)
            : launch_pack_k<false>(ka, geom->batch, kp, ks, kz, view->k_packed_bstride, view->k_scale_bstride, view->k_zero_bstride,
                                   geom->k_block, st);
  if (rc) return rc;
  PackArgs va{reinterpret_cast<const uint16_t*>(view->recent_v), view->recent_v_bstride, geom->recent_capacity, nullptr,
              flush_tokens, geom->i2_capacity, v_dst, geom->num_kv_heads};
  uint8_t* vp = const_cast<uint8_t*>(view->i2_packed);
  void* vs = const_cast<void*>(view->i2_scale);
  uint8_t* vz = const_cast<uint8_t*>(view->i2_zero);
  // The three launches overlap where they may: the value pack runs beside the key pack (different halves of the
  // ring, different arenas) and only completes after it; the ring kernel copies the flushed tokens' indices, then
  // waits for both packs before it moves rows and resets the length.  The ring kernel does not let ITS dependents go
  // early: a decode launch behind a flush must find the pools complete.
  rc = bf16 ? launch_pack_v2<true>(va, geom->batch, vp, vs, vz, view->i2_packed_bstride, view->i2_scale_bstride,
                                   view->i2_zero_bstride, geom->v2_group, st, dev->pdl)
            : launch_pack_v2<false>(va, geom->batch, vp, vs, vz, view->i2_packed_bstride, view->i2_scale_bstride,
                                    view->i2_zero_bstride, geom->v2_group, st, dev->pdl);
  if (rc) return rc;
  const cudaError_t err = launch_behind(flush_ring_kernel, dim3((unsigned)geom->batch), dim3(256), st, dev->pdl,
                                        ring_args(geom, view), (int)ring_tokens, (int)flush_tokens, i2_global, i2_logical,
                                        meta_bstride, v_meta_dst);
  ++g_launches;
  return err == cudaSuccess ? R2K_OK : R2K_ERR_CUDA;
}

}  // extern "C"
