/*
 * r2k_b200 -- C ABI of the B200 (sm_100a) SSPA packed-KV decode path.
 *
 * Plain pointers and sizes only; no torch types.  Every entry point returns an
 * int status (R2K_OK == 0), never throws, never synchronises the device and
 * never allocates device memory (workspaces are caller-provided).  All device
 * work is enqueued on the stream passed as `stream` (a cudaStream_t cast to
 * void*; NULL is the legacy default stream).
 *
 * Each declaration names the routine of the reference implementation
 * (Fabulous1496/R2-Omni, paths relative to that project) that it replaces.
 */
#ifndef R2K_B200_H
#define R2K_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------ */
enum {
  R2K_OK = 0,
  R2K_ERR_NULL = 1,          /* a required pointer is NULL                           */
  R2K_ERR_GEOMETRY = 2,      /* unsupported or inconsistent shapes                   */
  R2K_ERR_ALIGNMENT = 3,     /* a base pointer or stride is not 16-byte aligned      */
  R2K_ERR_CAPACITY = 4,      /* an arena or the residual ring has no room            */
  R2K_ERR_WORKSPACE = 5,     /* workspace too small                                  */
  R2K_ERR_CUDA = 6,          /* a CUDA runtime call failed (launch, attribute, ...)  */
  R2K_ERR_DEVICE_TIMEOUT = 7,/* a bounded device-side wait gave up (see r2k_decode_device_status) */
  R2K_ERR_EMPTY = 8          /* the cache holds no token to attend to                */
};

/* element type of queries, bf16-value pages, the residual window and the output */
enum { R2K_DTYPE_BF16 = 0, R2K_DTYPE_FP16 = 1 };

/* r2k_decode flags */
enum {
  R2K_FLAG_OUTPUT_HADAMARD = 1, /* round to the element type, then 128-point orthonormal WHT
                                   (r2omni/sspa/kernels/triton_fourq_splitk.py:999-1005)   */
  R2K_FLAG_OUT_F32 = 2,         /* `out` is float32 [B,Hq,128] instead of the element type  */
  R2K_FLAG_OUT_STATE = 4        /* `out` is float32 [B,Hq,130]: (max, sum-exp, un-normalised
                                   weighted V[128]) in natural-log units, for cross-shard merge */
};

/*
 * Geometry of one homogeneous batch of caches (every request has the same
 * extents; only the residual-window length differs per request).  Mirrors the
 * scalar fields r2omni/sspa/kernels/triton_fourq_splitk.py:1833-1907
 * (prepare_splitk_executor) extracts from a ThreePrecisionCache.
 */
typedef struct R2KGeom {
  int32_t batch;            /* B                                                        */
  int32_t num_q_heads;      /* Hq                                                       */
  int32_t num_kv_heads;     /* Hkv; Hq % Hkv == 0 and Hq / Hkv <= 8                     */
  int32_t head_dim;         /* must be 128                                              */
  int32_t dtype;            /* R2K_DTYPE_*                                              */
  int32_t page_size;        /* 16, 32 or 64 (residual page-length bookkeeping)          */
  int32_t k_block;          /* tokens per key calibration block: 32, 64 or 128          */
  int32_t v2_group;         /* INT2-value group width along head_dim: 32, 64 or 128     */
  int32_t n_fp;             /* tokens in the bf16-value pool                            */
  int32_t n_i4;             /* tokens in the INT4-value pool                            */
  int32_t n_i2;             /* tokens in the INT2-value pool (static + flushed)         */
  int32_t k_capacity;       /* token rows per head of the key arena (multiple of 128)   */
  int32_t k_off_fp;         /* key-arena row of the first token of each pool            */
  int32_t k_off_i4;
  int32_t k_off_i2;
  int32_t fp_capacity;      /* token rows per head of the bf16-value array              */
  int32_t i4_capacity;      /* token rows per head of the INT4-value arrays             */
  int32_t i2_capacity;      /* token rows per head of the INT2-value arena              */
  int32_t recent_capacity;  /* token rows per head of the residual ring                 */
  float sm_scale;           /* softmax scale; <= 0 selects head_dim^-0.5                */
} R2KGeom;

/*
 * Device pointers of one batch of caches.  Each pointer addresses request 0;
 * request b lives `*_bstride` BYTES further (0 is fine for B == 1).  Layouts
 * are the reference's storage formats, bit for bit:
 *   k_packed  u8  [Hkv, k_capacity, 64]   byte j = code(2j) | code(2j+1) << 4
 *   k_scale   f16 [Hkv, k_capacity/k_block, 128], k_zero u8 same shape
 *             (r2omni/sspa/runtime/compact_int4_key.py:95-109, 241-249)
 *   fp_v      T   [Hkv, fp_capacity, 128]
 *   i4_packed u8  [Hkv, i4_capacity, 64]  two's-complement nibbles, even dim low
 *   i4_scale  f32 [Hkv, i4_capacity]      (r2omni/sspa/runtime/fused_value_pack.py:52-70)
 *   i2_packed u8  [Hkv, i2_capacity, 32]  byte j = c(4j)|c(4j+1)<<2|c(4j+2)<<4|c(4j+3)<<6
 *   i2_scale  f16 [Hkv, i2_capacity, 128/v2_group], i2_zero u8 same shape
 *             (r2omni/sspa/runtime/fused_value_pack.py:107-149)
 *   recent_k/v T  [Hkv, recent_capacity, 128], recent_len i32 [1] per request,
 *   recent_global / recent_logical i64 [recent_capacity],
 *   recent_page_lengths i64 [recent_capacity / page_size]
 *             (r2omni/sspa/runtime/precision_pool.py:747-784)
 * Pointers of an empty pool may be NULL.
 */
typedef struct R2KCacheView {
  const uint8_t* k_packed;  const void* k_scale;  const uint8_t* k_zero;
  const void* fp_v;
  const uint8_t* i4_packed; const float* i4_scale;
  const uint8_t* i2_packed; const void* i2_scale; const uint8_t* i2_zero;
  void* recent_k; void* recent_v; int32_t* recent_len;
  int64_t* recent_global; int64_t* recent_logical; int64_t* recent_page_lengths;
  int64_t k_packed_bstride, k_scale_bstride, k_zero_bstride;
  int64_t fp_v_bstride;
  int64_t i4_packed_bstride, i4_scale_bstride;
  int64_t i2_packed_bstride, i2_scale_bstride, i2_zero_bstride;
  int64_t recent_k_bstride, recent_v_bstride, recent_len_bstride;
  int64_t recent_global_bstride, recent_logical_bstride, recent_page_lengths_bstride;
} R2KCacheView;

/* One token appended in the same launch as the decode it takes part in. */
typedef struct R2KAppend {
  const void* k;              /* T [B, Hkv, 128]; NULL = no append                      */
  const void* v;              /* T [B, Hkv, 128]                                        */
  const int64_t* indices;     /* optional device i64 [B,2] (global index, logical position)
                                 per request; NULL = use the two scalars for every request */
  int64_t global_index;
  int64_t logical_position;
} R2KAppend;

/* ---- decode ------------------------------------------------------------ */

/* Bytes of scratch r2k_decode needs for this geometry on the current device.
 * Replaces allocate_splitk_workspace / required_splitk_blocks
 * (r2omni/sspa/kernels/triton_fourq_splitk.py:1607-1692). */
int r2k_decode_workspace_bytes(const R2KGeom* geom, size_t* bytes);

/* Clears the status word and the arrival counters at the head of a workspace.
 * Call once after allocating it (and after any decode that reported a device
 * timeout).  One workspace may serve launches of different geometries one after
 * another on a stream, as long as it is large enough for each of them.          */
int r2k_decode_workspace_init(void* workspace, size_t bytes, void* stream);

/*
 * One decode step over a batch of packed caches: split-K partial attention over
 * the INT4 keys and bf16/INT4/INT2 value pools plus the residual window, exact
 * (max, sum-exp, out) merge, optional Hadamard epilogue and optional fused
 * one-token append into the residual ring -- a single launch.
 *   q   : T [B, Hq, 128] contiguous;  out: see R2K_FLAG_OUT_*.
 * With `append`, the new token takes part in the attention and is then written
 * to ring row recent_len[b]; recent_len, the two index arrays and the page
 * length are updated on the device.  The ring must have room (host-checked by
 * the caller, as in the reference).
 * Replaces SplitKExecutor.__call__ and its three launches
 * (r2omni/sspa/kernels/triton_fourq_splitk.py:1243-1547: _fourq_page_partial_kernel
 * :449-931, _fourq_hierarchical_group_reduce_kernel :1023-1086,
 * _fourq_partial_reduce_kernel :936-1020).
 */
int r2k_decode(const R2KGeom* geom, const R2KCacheView* view, const void* q, const R2KAppend* append,
               void* workspace, size_t workspace_bytes, void* out, uint32_t flags, void* stream);

/*
 * r2k_decode for callers that are not allowed to allocate device memory: it takes no workspace.
 * (No counterpart in the reference, which allocates its split-K scratch with torch.)
 *
 * Meant for code that runs where cudaMalloc is off limits -- a plugin handed only its input and
 * output buffers by a host runtime that owns every allocation and forbids others, or a latency
 * path that must never touch the allocator (cudaMalloc may synchronise the whole device).
 * The split-K scratch (arrival counters and partial (max, sum-exp, out) slots) lives in a
 * file-scope `static __device__` array of R2K_STATIC_WORKSPACE_BYTES inside the library, so every GPU
 * that loads the library holds that much memory until the process exits.
 *
 *  - A geometry whose scratch need (r2k_decode_workspace_bytes) exceeds R2K_STATIC_WORKSPACE_BYTES is
 *    rejected with R2K_ERR_WORKSPACE; nothing is launched.
 *  - The first call on each device resolves the array's device address (cudaGetSymbolAddress, with
 *    that device current) and clears its counters; make that first call outside any stream capture.
 *  - Every call on a device shares the one array, which keeps the previous call's contents.  The
 *    arrival counters live in a block of fixed size and position and every launch leaves the ones it
 *    used at zero, so back-to-back calls on ONE stream are fine, also when their geometries differ;
 *    calls that may overlap on the GPU (different streams, or graphs replayed concurrently) race on it
 *    and must be serialised by the caller, or use r2k_decode with separate workspaces.
 *  - Inputs, outputs, flags and results are exactly those of r2k_decode.
 *  - r2k_decode_static_status reads the device-side status word of the static scratch (what
 *    r2k_decode_device_status is for a caller-provided workspace; it synchronises `stream`), and
 *    r2k_decode_static_reset clears that word and the arrival counters on `stream` (what
 *    r2k_decode_workspace_init is for a workspace: call it after a reported device timeout).  Neither
 *    allocates; either may be the first call on a device.
 */
#define R2K_STATIC_WORKSPACE_BYTES (4u << 20)
int r2k_decode_static(const R2KGeom* geom, const R2KCacheView* view, const void* q, const R2KAppend* append,
                      void* out, uint32_t flags, void* stream);
int r2k_decode_static_status(int32_t* status, void* stream);
int r2k_decode_static_reset(void* stream);

/*
 * r2k_decode for a caller whose query, appended rows and result live in HOST memory: ONE call copies the
 * inputs to the device, launches the decode (with its fused append), copies the result back and waits for
 * the stream, so that `host_out` can be read on return.  This is the call a host runtime binds when its
 * tensors are not device-resident (the reference's operator receives torch CUDA tensors, so there the copies
 * are the caller's `.to(device)` / `.cpu()` around SplitKExecutor.__call__,
 * r2omni/sspa/kernels/triton_fourq_splitk.py:1739-1850).
 *
 *   host_in  : q [B,Hq,128] of T, followed -- only if append != NULL -- by k [B,Hkv,128] and v [B,Hkv,128]
 *              of T, contiguous.  Page-locked memory makes the copies asynchronous; pageable memory works.
 *   append   : NULL, or the indices / scalars of R2KAppend; its k and v pointers are ignored.
 *   staging  : device scratch of at least r2k_decode_host_staging_bytes() bytes, 16-byte aligned.
 *   host_out : as `out` of r2k_decode (R2K_FLAG_OUT_* honoured).
 * A page-locked, device-mapped `host_out` is written by the kernel in place (no copy back); environment variable
 * R2K_HOST_ZERO_COPY selects otherwise (bit 0: read `host_in` in place, bit 1: write `host_out` in place, bit 2:
 * bring a mapped `host_in` into `staging` with a copy kernel that the decode launch overlaps; default 6).
 * Returns the decode's status; a CUDA failure of a copy or of the wait is R2K_ERR_CUDA.
 */
int r2k_decode_host_staging_bytes(const R2KGeom* geom, size_t* bytes);
int r2k_decode_host(const R2KGeom* geom, const R2KCacheView* view, const void* host_in, const R2KAppend* append,
                    void* workspace, size_t workspace_bytes, void* staging, size_t staging_bytes, void* host_out,
                    uint32_t flags, void* stream);

/* Copies the device-side status word of the last decodes that used `workspace`
 * into *status (R2K_OK or R2K_ERR_DEVICE_TIMEOUT).  Synchronises `stream`.     */
int r2k_decode_device_status(void* workspace, int32_t* status, void* stream);

/* Number of kernels of this library launched by this process so far. */
uint64_t r2k_launch_count(void);

/*
 * Merge `num_states` un-normalised attention states (each float32 [rows,130] as
 * written by R2K_FLAG_OUT_STATE, `state_stride` floats apart) into the final
 * output [rows,128] (element type, or float32 with R2K_FLAG_OUT_F32; Hadamard
 * flag honoured).  rows = B*Hq.  This is the cross-GPU step of the
 * sequence-sharded path; the arithmetic is _merge_state of
 * r2omni/sspa/kernels/triton_fourq_attention.py:58-69.
 */
int r2k_merge_states(const float* states, int32_t num_states, int64_t state_stride, int32_t rows,
                     int32_t dtype, void* out, uint32_t flags, void* stream);

/* ---- sequence-sharded decode with the merge fused over peer memory -------- */

/*
 * One exchange buffer per rank (GPU), mapped into every rank's address space.
 * A decode launched through r2k_decode_exchange ends, for every (request, kv
 * head), by storing this rank's un-normalised state rows into EVERY rank's
 * buffer over NVLink (plain peer stores of 8-byte (value, step) words), waiting
 * (bounded) until all ranks' words of this step have landed in its own buffer
 * and merging them there -- the exact merge of r2k_merge_states.  Every rank ends
 * with the same output; there is no collective launch and no merge launch.
 * No counterpart in the reference (it has no multi-GPU path); the arithmetic
 * is _merge_state, r2omni/sspa/kernels/triton_fourq_attention.py:58-69.
 *
 * Rules: world <= R2K_MAX_RANKS, one process per GPU, every rank makes the
 * call for every step with the same `seq` (1, 2, 3, ...; or 0 on every rank and
 * every step: the kernel then counts the steps itself in the exchange buffer,
 * which is what a captured CUDA graph needs; two steps in flight
 * never share a buffer half because a rank cannot finish step n+1 before every
 * rank has finished step n).  A rank that is missing makes the others give up
 * after a bounded wait (about a second, see wait_us) and report
 * R2K_ERR_DEVICE_TIMEOUT through r2k_decode_device_status; nothing hangs.  Rows
 * that never arrived count as the state of a rank without tokens, so `out` then
 * holds the finite merge of the ranks that did arrive.
 */
#define R2K_MAX_RANKS 8
typedef struct R2KExchange {
  void*    buffers[R2K_MAX_RANKS]; /* rank r's exchange buffer as mapped in this process */
  int32_t  rank, world;
  uint32_t seq;                    /* step counter 1, 2, 3, ... or 0: use the counter kept in the buffer */
  uint32_t wait_us;                /* budget, in microseconds, of the wait for the other ranks' rows before it
                                      gives up (65536 polls share it; a poll itself takes about a microsecond, so
                                      the shortest wait is some 70 ms); 0 selects the default, about 1.3 s   */
} R2KExchange;

/* Bytes of one rank's exchange buffer for this geometry and world size. */
int r2k_exchange_bytes(const R2KGeom* geom, int32_t world, size_t* bytes);
/* Set-up only (these three allocate / map device memory; nothing else in this
 * library does): a zeroed device buffer plus its 64-byte inter-process handle;
 * a mapping of another rank's buffer (peer access is enabled on the way); and
 * their release (`opened` != 0 for a mapping obtained from r2k_exchange_open). */
int r2k_exchange_create(size_t bytes, void** buffer, unsigned char handle[64]);
int r2k_exchange_open(const unsigned char handle[64], void** buffer);
int r2k_exchange_close(void* buffer, int32_t opened);
/* r2k_decode plus the fused cross-rank merge described above.  `out` receives
 * the merged, normalised output; R2K_FLAG_OUT_STATE is not accepted. */
int r2k_decode_exchange(const R2KGeom* geom, const R2KCacheView* view, const void* q, const R2KAppend* append,
                        void* workspace, size_t workspace_bytes, void* out, uint32_t flags,
                        const R2KExchange* exchange, void* stream);

/* ---- quantize and pack -------------------------------------------------- */

/*
 * Per-channel affine INT4 key blocks.  Gathers `count` rows src[h, index[i], :]
 * (index == NULL: rows 0..count-1) of a T [Hkv, src_rows, 128] tensor into arena
 * rows dst_start .. dst_start+count-1 and calibrates every k_block-token block
 * those rows touch.  When dst_start is not a multiple of k_block, the rows
 * already stored in front of it inside that block are dequantised, rounded to T
 * and re-quantised together with the new rows, exactly as
 * CompactInt4KeyArena.append_superblock does.
 * Replaces quantize_int4_key_per_channel / _gather_pack_int4_key_kernel /
 * CompactInt4KeyArena._write / append_superblock
 * (r2omni/sspa/runtime/compact_int4_key.py:21-110, 200-220).
 */
int r2k_pack_k_int4(const void* src, int32_t dtype, int32_t num_kv_heads, int64_t src_rows,
                    const int64_t* index, int64_t count,
                    uint8_t* k_packed, void* k_scale, uint8_t* k_zero,
                    int64_t k_capacity, int32_t k_block, int64_t dst_start, void* stream);

/* Per-token symmetric INT4 values (scale = max(amax/7, 1e-6), codes -7..7).
 * Replaces _gather_pack_int4_value_kernel and make_packed_tensor(.,4,"per_token",2)
 * (r2omni/sspa/runtime/fused_value_pack.py:25-70, r2omni/sspa/runtime/quantization.py:19-50, 77-102). */
int r2k_pack_v_int4(const void* src, int32_t dtype, int32_t num_kv_heads, int64_t src_rows,
                    const int64_t* index, int64_t count,
                    uint8_t* packed, float* scale, int64_t capacity, int64_t dst_start, void* stream);

/* Per-token, per-group affine INT2 values (range widened to contain 0).
 * Replaces _gather_pack_int2_value_kernel and quantize_int2_value
 * (r2omni/sspa/runtime/fused_value_pack.py:72-149, r2omni/sspa/runtime/int2_reference.py:96-151). */
int r2k_pack_v_int2(const void* src, int32_t dtype, int32_t num_kv_heads, int64_t src_rows,
                    const int64_t* index, int64_t count,
                    uint8_t* packed, void* scale, uint8_t* zero, int64_t capacity, int32_t group,
                    int64_t dst_start, void* stream);

/* Row gather dst[h, dst_start+i, :] = src[h, index[i], :] for 128-wide T rows
 * (the bf16-value pool of build_three_precision_cache,
 * r2omni/sspa/runtime/precision_pool.py:708, 733-735). */
int r2k_gather_rows(const void* src, int32_t num_kv_heads, int64_t src_rows, const int64_t* index,
                    int64_t count, void* dst, int64_t dst_rows, int64_t dst_start, void* stream);

/* Normalised 128-point Walsh-Hadamard transform of `rows` 128-wide rows of the
 * given 16-bit type (fp32 butterflies, stages of stride 1..64, times 128^-1/2,
 * rounded to the element type); in place when out == in.  Replaces
 * triton_fwht_128 / _fwht_128_kernel (r2omni/sspa/kernels/triton_qwen_mrope.py:
 * 13-42, 325-346; CPU form normalized_fwht, r2omni/sspa/runtime/int2_reference.py:18-31):
 * the pre-conditioning of new key/value rows when key_hadamard / value_hadamard is on. */
int r2k_fwht128(const void* in, void* out, int32_t dtype, int64_t rows, void* stream);

/* Qwen multimodal rotary embedding of q [B,Hq,T,128] and k [B,Hkv,T,128] (contiguous, 16-bit type `dtype`) in
 * one launch, optionally followed by the 128-point Hadamard transform of every row.  cos / sin are addressed as
 * [axis(3), request, token, channel] with the given element strides; rot_dtype is R2K_DTYPE_BF16, R2K_DTYPE_FP16
 * or 2 for float32; axis(d) is 0 for (d mod 64) < section0, 1 below section0 + section1, else 2.  Outputs may
 * alias the inputs.  Replaces qwen_qk_mrope / _qwen_qk_mrope_kernel / _qwen_batched_qk_mrope_kernel
 * (r2omni/sspa/kernels/triton_qwen_mrope.py:44-124, 126-212, 214-322), the prologue that produces the query and
 * the new key row of a decode step (r2omni/sspa/integration/qwen_sspa_attention.py:1239-1247). */
int r2k_qk_mrope(const void* q, const void* k, void* q_out, void* k_out, int32_t dtype, int32_t batch,
                 int32_t num_q_heads, int32_t num_kv_heads, int32_t tokens, const void* cos, const void* sin,
                 int32_t rot_dtype, const int64_t cos_strides[4], const int64_t sin_strides[4], int32_t section0,
                 int32_t section1, int32_t apply_hadamard, void* stream);

/* The whole prologue of a decode step in one launch: query rows [B,Hq,128] and new key rows [B,Hkv,128] rotated as
 * by r2k_qk_mrope (one token per request; Hadamard when key_hadamard), new value rows [B,Hkv,128] brought along
 * (copied, or Hadamard-transformed as by r2k_fwht128 when value_hadamard).  The three inputs may be slices of one
 * fused projection output: `*_bstride` is the number of elements between two requests' rows (a request's heads are
 * contiguous; a multiple of 4); the outputs are contiguous and are what r2k_decode takes as q and as the rows to
 * append.  The launch lets the decode launch behind it start early, like r2k_qk_mrope.  Same arithmetic, bit for
 * bit, as the two calls it replaces.  Covers what _project_qkv does after the projections
 * (r2omni/sspa/integration/qwen_sspa_attention.py:1216-1249, and the value rotation of :1780). */
int r2k_qkv_prologue(const void* q, int64_t q_bstride, const void* k, int64_t k_bstride, const void* v, int64_t v_bstride,
                     void* q_out, void* k_out, void* v_out, int32_t dtype, int32_t batch, int32_t num_q_heads,
                     int32_t num_kv_heads, const void* cos, const void* sin, int32_t rot_dtype,
                     const int64_t cos_strides[4], const int64_t sin_strides[4], int32_t section0, int32_t section1,
                     int32_t key_hadamard, int32_t value_hadamard, void* stream);

/* ---- residual window ---------------------------------------------------- */

/*
 * Standalone one-token append into the residual ring of every request of the
 * batch (row recent_len[b]; updates recent_len, index arrays, page length).
 * Replaces append_recent_fp_triton / _append_recent_fp_kernel
 * (r2omni/sspa/kernels/triton_fourq_splitk.py:413-447, 1557-1604).
 */
int r2k_append_recent(const R2KGeom* geom, const R2KCacheView* view, const R2KAppend* append, void* stream);

/*
 * Flush: quantize-and-pack the oldest `flush_tokens` rows of the residual ring
 * of every request into key-arena rows k_dst.. (with tail re-quantisation) and
 * INT2-value rows v_dst.., copy their global/logical indices to
 * i2_global/i2_logical (i64 arrays, row v_meta_dst.., may be NULL), slide the
 * remaining `ring_tokens - flush_tokens` rows to the front and set recent_len
 * and the page lengths accordingly.  `ring_tokens` is the host mirror of the
 * ring length.  All on `stream`, no host synchronisation.
 * Replaces the flush branch of append_generated_token
 * (r2omni/sspa/runtime/dynamic_fourq_cache.py:195-254).
 */
int r2k_flush_recent(const R2KGeom* geom, const R2KCacheView* view, int32_t ring_tokens, int32_t flush_tokens,
                     int64_t k_dst, int64_t v_dst,
                     int64_t* i2_global, int64_t* i2_logical, int64_t meta_bstride, int64_t v_meta_dst,
                     void* stream);

const char* r2k_status_string(int status);

#ifdef __cplusplus
}
#endif
#endif /* R2K_B200_H */
