/*
 * b200kv.h — C ABI of the B200 (sm_100a) int8-KV-cache attention kernels.
 *
 * Drop-in boundary for the attention half of kbwal/inference-engine's Qwen3-1.7B engine:
 * each entry point replaces one host wrapper + Triton kernel pair of the reference file
 * qwen3-1.7b/kernels.py (cited per function).  A Python binding (ctypes) calls these with
 * raw device pointers taken from torch tensors; nothing here knows about torch.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless the name ends in _host.
 *   - Strides are in ELEMENTS of the pointed-to type.  The innermost (head_dim) stride is 1.
 *   - bf16 tensors are passed as `const void*` / `void*` (2-byte elements).
 *   - `stream` is a cudaStream_t passed as void* (0 = legacy default stream).  All work is
 *     enqueued on it; no entry point synchronises, allocates, frees or keeps a pointer after
 *     it returns, and every grid is a function of the shape arguments only, so calls may be
 *     captured in a CUDA graph (the reference engine does: engine.py:376-449).
 *   - An empty batch (zero entries / zero rows) is valid: the call returns B200KV_OK at once, whatever the
 *     pointers are (empty tensors have no storage).
 *   - Return value: B200KV_OK, or a negative B200KV_E_* code, in which case NOTHING was
 *     launched.  `status` (optional, may be NULL) is a device int32 the kernels OR error bits
 *     into when device-side data is inconsistent (a page id or token position out of range):
 *     the offending access is skipped, never performed.
 *
 * Cache layout (reference: LayerKVCache, kernels.py:11-17; allocation engine.py:472-492)
 *   k, v          int8  [num_pages, Hkv, page_size, D]
 *   k_scale, v_scale fp32 [num_pages, Hkv, page_size]
 *   k_calibration fp32  [num_pages, Hkv, 1, D]
 *   The reference's layout is the special case page_size = max_len, one page per sequence
 *   slot, table = slot_ids.  Token t of entry b lives in page table[b*table_stride + t/page_size]
 *   at row t % page_size; an entry's calibration row is that of its first page.
 */
#ifndef B200KV_H
#define B200KV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200KV_VERSION 2

enum {
  B200KV_OK = 0,
  B200KV_E_NULL = -1,      /* a required pointer is NULL */
  B200KV_E_SHAPE = -2,     /* unsupported geometry (head_dim, head counts, page size) */
  B200KV_E_ALIGN = -3,     /* pointer or stride not aligned as the kernels need */
  B200KV_E_WORKSPACE = -4, /* caller-provided workspace too small */
  B200KV_E_LAUNCH = -5,    /* the CUDA runtime rejected a launch (see cudaGetLastError) */
  B200KV_E_RANGE = -6,     /* a size argument is out of the supported range */
  B200KV_E_STATIC_LIMIT = -7 /* b200kv_decode_attn_static: the call needs more scratch than the built-in array holds */
};

/* Bits OR-ed into the optional device status word. */
enum {
  B200KV_S_BAD_PAGE = 1,    /* block-table entry outside [0, num_pages) */
  B200KV_S_BAD_POSITION = 2, /* token position outside the entry's table (>= max_pages*page_size) */
  B200KV_S_TIMEOUT = 4,      /* a bounded wait inside a kernel ran out; that CTA's output rows are not written */
  B200KV_S_BAD_PLAN = 8      /* b200kv_decode_attn_planned: the plan was not made for this batch (other lengths, head
                                counts, page size or SM count); the warps that saw it wrote nothing */
};

/* One layer's cache, by value.  Mirrors LayerKVCache (kernels.py:11-17). */
typedef struct b200kv_cache {
  int8_t* k;
  int8_t* v;
  float* k_scale;
  float* v_scale;
  float* k_calibration;
  int64_t stride_page;  /* codes: elements between pages (k and v share strides, kernels.py:284-287) */
  int64_t stride_head;  /* codes: elements between kv heads */
  int64_t stride_tok;   /* codes: elements between token rows (>= D) */
  int64_t sstride_page; /* scales: elements between pages */
  int64_t sstride_head; /* scales: elements between kv heads */
  int64_t cstride_page; /* calibration: elements between pages */
  int64_t cstride_head; /* calibration: elements between kv heads */
  int32_t num_pages;
  int32_t num_kv_heads;
  int32_t page_size;
  int32_t head_dim;
} b200kv_cache;

/* Page table of a batch: `ids` int32 [num_entries, max_pages] with row stride `stride`.
 * The reference's `slot_ids [B]` is {ids = slot_ids, stride = 1, max_pages = 1}. */
typedef struct b200kv_table {
  const int32_t* ids;
  int32_t stride;
  int32_t max_pages;
} b200kv_table;

int b200kv_version(void);
const char* b200kv_error_string(int code);

/* Replaces fused_rope_kv_decode (kernels.py:364-544).
 * For every entry b < *num_decoding: per-head RMSNorm + half-split RoPE of q[b] and k[b] in
 * fp32; q_out[b] = bf16(q * calibration); k / calibration and v are quantized per head to int8
 * with scale = max(absmax,1e-6)/127 and written at token position cached_lens[b].
 * q [B,Hq,D], k,v [B,Hkv,D] bf16 with the given entry/head strides (views of the fused QKV
 * row are fine); cos,sin bf16 [B, D/2] with row stride; q_out bf16 [B,Hq,D].
 * Codes, scales and q_out are bit-identical to the reference arithmetic evaluated in IEEE fp32
 * without FMA (sum of squares in numpy pairwise order). */
int b200kv_write_decode(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                        const void* k, int64_t k_stride_b, int64_t k_stride_h,
                        const void* v, int64_t v_stride_b, int64_t v_stride_h,
                        const void* q_norm_w, const void* k_norm_w,
                        const void* cos, int64_t cos_stride_b, const void* sin, int64_t sin_stride_b,
                        const b200kv_cache* cache, const b200kv_table* table,
                        const int32_t* cached_lens, const int32_t* num_decoding,
                        void* q_out, int64_t o_stride_b, int64_t o_stride_h,
                        int32_t B, int32_t Hq, float eps, int32_t* status, void* stream);

/* Replaces fused_norm_rope_prefill (kernels.py:547-714): norm + rope of all N packed rows,
 * bf16 outputs q_out [N,Hq,D], k_out [N,Hkv,D] (strides given). */
int b200kv_norm_rope_prefill(const void* q, int64_t q_stride_n, int64_t q_stride_h,
                             const void* k, int64_t k_stride_n, int64_t k_stride_h,
                             const void* q_norm_w, const void* k_norm_w,
                             const void* cos, int64_t cos_stride_n, const void* sin, int64_t sin_stride_n,
                             void* q_out, int64_t qo_stride_n, int64_t qo_stride_h,
                             void* k_out, int64_t ko_stride_n, int64_t ko_stride_h,
                             int32_t N, int32_t Hq, int32_t Hkv, int32_t D, float eps, void* stream);

/* Replaces quantize_kv_prefill (kernels.py:717-865).  k (bf16, output of norm_rope_prefill)
 * and v [N,Hkv,D] packed rows; entry b >= *num_decoding owns rows [cu_seqlens[b], cu_seqlens[b+1]).
 * First chunk (cached_lens[b] == 0): calibration = max(1e-3, max_t |k[t,d]|) is computed and
 * stored; otherwise loaded.  Rows are written at token positions cached_lens[b] + t. */
int b200kv_quantize_prefill(const void* k, int64_t k_stride_n, int64_t k_stride_h,
                            const void* v, int64_t v_stride_n, int64_t v_stride_h,
                            const int32_t* cu_seqlens, int32_t num_entries,
                            const b200kv_cache* cache, const b200kv_table* table,
                            const int32_t* cached_lens, const int32_t* num_decoding,
                            int32_t N, int32_t* status, void* stream);

/* fused_norm_rope_prefill and quantize_kv_prefill in one call (kernels.py:547-714 followed by :717-865), for callers
 * that need not keep the two as separate steps: q_out / k_out receive the normed + roped rows of all N packed rows
 * exactly as b200kv_norm_rope_prefill writes them, and the rows of prefilling entries are quantized from the
 * bf16-rounded k_out (the reference stores k as bf16 between its two kernels, so the codes depend on that rounding)
 * and from v, with the calibration rule of b200kv_quantize_prefill.  Same bits as the two calls made one after the
 * other; two launches instead of three, none of which waits for a serial pass over the chunk. */
int b200kv_write_prefill(const void* q, int64_t q_stride_n, int64_t q_stride_h,
                         const void* k, int64_t k_stride_n, int64_t k_stride_h,
                         const void* v, int64_t v_stride_n, int64_t v_stride_h,
                         const void* q_norm_w, const void* k_norm_w,
                         const void* cos, int64_t cos_stride_n, const void* sin, int64_t sin_stride_n,
                         const int32_t* cu_seqlens, int32_t num_entries,
                         const b200kv_cache* cache, const b200kv_table* table,
                         const int32_t* cached_lens, const int32_t* num_decoding,
                         void* q_out, int64_t qo_stride_n, int64_t qo_stride_h,
                         void* k_out, int64_t ko_stride_n, int64_t ko_stride_h,
                         int32_t N, int32_t Hq, float eps, int32_t* status, void* stream);

/* Replaces dequantize_kv_prefix (kernels.py:868-970): rows [cu_cached[b], cu_cached[b+1]) of
 * k_out/v_out bf16 [Hkv, capacity, D] receive bf16(code*k_scale*calibration) / bf16(code*v_scale)
 * of entry b's first cached tokens. */
int b200kv_dequant_prefix(const b200kv_cache* cache, const b200kv_table* table,
                          const int32_t* cu_cached, int32_t num_entries,
                          void* k_out, void* v_out, int64_t o_stride_h, int64_t o_stride_n,
                          int32_t capacity, int32_t* status, void* stream);

/* Replaces prefill_attention (kernels.py:973-1175): packed varlen causal attention of the
 * prefilling entries over [dequantized prefix | own chunk].  tile_start [num_tiles] gives the
 * first packed row of each block_m-row query tile (-1 = idle), seq_ids [N] the entry of each row.
 * k_prefix / v_prefix may be NULL when the step has no cached prefix at all (empty tensors have no storage); prefix
 * lengths in cu_cached are then ignored. */
int b200kv_prefill_attn(const void* q, int64_t q_stride_n, int64_t q_stride_h,
                        const void* k, int64_t k_stride_n, int64_t k_stride_h,
                        const void* v, int64_t v_stride_n, int64_t v_stride_h,
                        const int32_t* seq_ids, const int32_t* cu_seqlens, const int32_t* tile_start,
                        int32_t num_tiles, int32_t block_m,
                        const void* k_prefix, const void* v_prefix, int64_t p_stride_h, int64_t p_stride_n,
                        const int32_t* cu_cached,
                        void* out, int64_t o_stride_n, int64_t o_stride_h,
                        int32_t N, int32_t Hq, int32_t Hkv, int32_t D, void* stream);

/* The same operation with the kernel chosen by the caller and an optional status word.
 * variant 0 = automatic (what b200kv_prefill_attn does: the tcgen05 kernel when block_m >= 64,
 * else the mma.sync kernel), 1 = the mma.sync kernel (64-row CTAs, register accumulators),
 * 2 = the tcgen05 kernel (128-row CTAs, accumulators in tensor memory).  Both give results within
 * the attention tolerance of each other; they differ in summation order.  3 = a test mode of the tcgen05
 * kernel: its issuing warps stay idle and every wait gives up after a few thousand polls, so all of the
 * kernel's bounded waits run out; the call must come back with B200KV_S_TIMEOUT in the status word and
 * no output row written (the time-out path, exercised without faulting the GPU).  prefix_rows = rows each
 * kv head of k_prefix / v_prefix holds (their shape[1]); it bounds the tensor-map copies of the
 * tcgen05 kernel.  0 = unknown: prefix tiles are then fetched with plain asynchronous copies. */
int b200kv_prefill_attn_variant(const void* q, int64_t q_stride_n, int64_t q_stride_h,
                                const void* k, int64_t k_stride_n, int64_t k_stride_h,
                                const void* v, int64_t v_stride_n, int64_t v_stride_h,
                                const int32_t* seq_ids, const int32_t* cu_seqlens, const int32_t* tile_start,
                                int32_t num_tiles, int32_t block_m,
                                const void* k_prefix, const void* v_prefix, int64_t p_stride_h, int64_t p_stride_n,
                                int32_t prefix_rows, const int32_t* cu_cached,
                                void* out, int64_t o_stride_n, int64_t o_stride_h,
                                int32_t N, int32_t Hq, int32_t Hkv, int32_t D,
                                int32_t variant, int32_t* status, void* stream);

/* The two element-wise ops of the decoder block either side of the attention path.
 * b200kv_silu_mul replaces silu_mul (kernels.py:1178-1212): out[n, d] = bf16((g * sigmoid(g)) * u) with
 * g = gate_up[n, d], u = gate_up[n, D + d], fp32 arithmetic.  bf16 [N, 2D] -> bf16 [N, D]; D a multiple
 * of 8, rows 16-byte aligned.
 * b200kv_add_rms_norm replaces add_rms_norm (kernels.py:1215-1285): new_residual = bf16(residual + delta);
 * normed = bf16((new_residual * rsqrt(mean(new_residual^2) + eps)) * weight), the mean over the rounded new
 * residual.  bf16 [N, D] each, D a multiple of 8 and at most 8192. */
int b200kv_silu_mul(const void* gate_up, int64_t in_stride, void* out, int64_t out_stride,
                    int32_t N, int32_t D, void* stream);
int b200kv_add_rms_norm(const void* residual, int64_t r_stride, const void* delta, int64_t d_stride,
                        const void* weight, void* new_residual, int64_t nr_stride,
                        void* normed, int64_t nn_stride, int32_t N, int32_t D, float eps, void* stream);

/* Replaces sample (kernels.py:1286-1370): Gumbel-max sampling, two kernels.  token[b] = the first index
 * attaining max_v (logits[b,v] + tau * -log(-log(u))), u = clamp(U(seed, b*V + v), 1e-10, 1 - 1e-7) with the
 * Philox-4x32-10 uniform of the reference; tau = 0 is greedy argmax.  logits bf16 (elem_bytes 2) or fp32 (4),
 * row stride in elements; seed = device int64, advanced by one by the call; out = device int64 [B] with stride
 * out_stride; workspace = b200kv_sample_workspace_bytes(B, V) bytes of device memory (the reference's two
 * partial buffers). */
size_t b200kv_sample_workspace_bytes(int32_t B, int32_t V);
int b200kv_sample(const void* logits, int64_t stride, int32_t elem_bytes, int64_t* seed, float tau,
                  void* workspace, size_t workspace_bytes, int64_t* out, int64_t out_stride,
                  int32_t B, int32_t V, void* stream);

/* Replaces skinny_matmul (kernels.py:1373-1455), the matmul `linear` uses for the few rows of a decode step, where
 * reading the weight once from HBM is the whole cost: y[M, N] = x[M, K] . w[N, K]^T, bf16 in, fp32 accumulate, bf16
 * out; w in the layout of nn.Linear.weight.  M <= 64 (the reference's bound), N a multiple of 128, K a multiple of
 * 64; x and w 16-byte aligned with row strides (ldx, ldw, elements) that are multiples of 8.  `splits` in
 * {1, 2, 4, 8}: the CTAs of a cluster of that size share a block of 128 weight rows and split K (at most
 * max(16, M rounded up to a power of two) / 2 and at most K / 64); the caller picks it so that (N / 128) * splits
 * fills the SMs (b200kv_skinny_linear is what tune_linear times against cuBLAS per shape, as the reference does).
 * The fp32 summation order differs from the reference's (as its own does between autotuned block sizes), so results
 * agree to the last bf16 bit, not bit for bit. */
int b200kv_skinny_linear(const void* x, int64_t ldx, const void* w, int64_t ldw, void* y, int64_t ldy,
                         int32_t M, int32_t N, int32_t K, int32_t splits, int32_t* status, void* stream);

/* Chained launches (off by default).  While enabled, every kernel of this library except decode attention
 * (which is chained per call, through bit 2 of its `variant`) and b200kv_decode_plan (never chained) is launched
 * with programmatic stream serialization: it may be brought up while the kernel launched just before it on
 * the same stream is still running, reads only caller-provided metadata (cu_seqlens, cu_cached,
 * cached_lens, num_decoding, block table, tile_start, seq_ids) until that kernel has completed, and
 * touches everything else afterwards.  Enable it only if no kernel that precedes a call of this
 * library on its stream writes those metadata arrays - true for the reference engine, which uploads
 * them once per step before the first layer (engine.py:347-356).  Process-wide; has no counterpart
 * in the reference. */
void b200kv_set_chained_launch(int enabled);
int b200kv_get_chained_launch(void);

/* Bytes of fp32 workspace b200kv_decode_attn needs for a batch of B entries on a device with
 * `sm_count` SMs (replaces the three partial buffers of kernels.py:305-311).
 * Contract: the workspace must be ZERO-filled once when it is allocated.  It holds, besides the
 * split partials, one arrival counter per (entry, kv head); the kernel returns every counter to
 * zero, so the same workspace can serve any number of stream-ordered calls WITH THE SAME B AND
 * HEAD COUNTS (the counters' place depends on them; zero-fill again before changing shape).  Two
 * calls that overlap on the GPU must not share a workspace. */
size_t b200kv_decode_attn_workspace_bytes(int32_t B, int32_t Hq, int32_t Hkv, int32_t D, int32_t sm_count);
/* The part of that workspace that has to be zero: its first b200kv_decode_attn_workspace_zero_bytes(B, Hkv) bytes
 * (the arrival counters).  What lies behind them (the split partials) is written before it is read in every call
 * and may hold anything, NaNs included. */
size_t b200kv_decode_attn_workspace_zero_bytes(int32_t B, int32_t Hkv);

/* Replaces decode_attention (kernels.py:272-361): split-K GQA decode attention over the int8
 * cache with in-kernel dequantization, one new token per entry, followed by the cross-split
 * log-sum-exp reduction.  Entry b < *num_decoding attends tokens [0, cached_lens[b]] and its
 * result is written to out[b] (bf16 [>=B,Hq,D]); other rows of `out` are not touched.
 * q bf16 [B,Hq,D] is the q_out of b200kv_write_decode.  `variant` bit 0: 0 = tensor-core kernel
 * (the product path), 1 = scalar CUDA-core kernel kept for cross-checking; bit 1: 0 = the
 * cross-split reduction is fused into the attention kernel (the warp delivering the last piece of
 * an (entry, head) merges them), 1 = it runs as a second kernel like the reference's; bit 2: 1 =
 * early start: the kernel may be scheduled while the kernel launched just before it on `stream`
 * is still running, and reads cached_lens, num_decoding and the block table before waiting for
 * it (cache, q and workspace are read after the wait).  Set it only when that preceding kernel
 * does not write those three arrays - true for b200kv_write_decode, the call the engine makes
 * right before (architecture.py:101-123). */
int b200kv_decode_attn(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                       const b200kv_cache* cache, const b200kv_table* table,
                       const int32_t* cached_lens, const int32_t* num_decoding, float scale,
                       void* out, int64_t o_stride_b, int64_t o_stride_h,
                       void* workspace, size_t workspace_bytes,
                       int32_t B, int32_t Hq, int32_t sm_count, int32_t variant,
                       int32_t* status, void* stream);

/* Per-step plan of decode attention.  No counterpart in the reference, whose kernel re-derives its work split
 * from cached_lens in every program of every layer (compute_piece / assign_work, kernels.py:20-70).
 *
 * The work split of b200kv_decode_attn depends only on cached_lens, *num_decoding and the block table, which a
 * decoder step uploads once and then uses for all of its layers (engine.py:347-356, 451-470).
 * b200kv_decode_plan computes the split once (one small kernel on `stream`) into `plan`
 * (b200kv_decode_plan_bytes(sm_count) bytes of device memory, 16-byte aligned): for every warp of the persistent
 * grid the position of its first tile and the page ids of its first tiles.  b200kv_decode_attn_planned is
 * b200kv_decode_attn reading that plan: same arguments, same result bit for bit, but each CTA starts its copies
 * after one round of loads instead of a length scan, a search and a dependent page-table read.
 * Contract: between b200kv_decode_plan and the last planned call that uses the plan, cached_lens, *num_decoding
 * and the table must not change, and B, Hkv, page_size and sm_count must be the ones the plan was made with (B counts
 * the entries of cached_lens; q and out are only touched in the rows of decoding entries, so a caller that packs
 * tokens may hold fewer rows than B there).  A
 * plan that does not fit (checked per warp against the header and the lengths) sets B200KV_S_BAD_PLAN in the
 * status word and the warps that saw it write nothing; zero-fill the workspace again after that.
 * `variant` as for b200kv_decode_attn, except bit 1 (the two-kernel reduction), which is refused.  With bit 2
 * (early start) the plan counts as metadata: it is read before the wait, which is safe because the plan kernel
 * never releases a chained successor before it has finished. */
size_t b200kv_decode_plan_bytes(int32_t sm_count);
int b200kv_decode_plan(const b200kv_table* table, const int32_t* cached_lens, const int32_t* num_decoding,
                       int32_t B, int32_t num_kv_heads, int32_t page_size, int32_t sm_count,
                       void* plan, size_t plan_bytes, void* stream);
int b200kv_decode_attn_planned(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                               const b200kv_cache* cache, const b200kv_table* table,
                               const int32_t* cached_lens, const int32_t* num_decoding, float scale,
                               void* out, int64_t o_stride_b, int64_t o_stride_h,
                               void* workspace, size_t workspace_bytes,
                               const void* plan, size_t plan_bytes,
                               int32_t B, int32_t Hq, int32_t sm_count, int32_t variant,
                               int32_t* status, void* stream);

/* b200kv_decode_attn for callers that must not allocate.  It has no counterpart in the reference
 * (whose wrapper allocates three partial buffers per call, kernels.py:305-311).
 *
 * Same computation and same result as b200kv_decode_attn with variant 0, but the caller passes
 * no workspace: the scratch (arrival counters and fp32 split partials) is a fixed 8 MiB array
 * inside the library's device image, so this call reaches neither cudaMalloc/cudaFree nor any
 * allocating library routine.  Meant for hosts that cannot allocate where they call attention:
 * a server whose own pool already owns all device memory, code running inside another
 * component's stream capture, or a loop that cannot afford the device-wide synchronisation an
 * allocation implies.
 *
 * Limit: the call is rejected with B200KV_E_STATIC_LIMIT (nothing launched) when
 * b200kv_decode_attn_workspace_bytes(B, Hq, Hkv, D, sm_count) exceeds
 * b200kv_decode_attn_static_limit() = 8 MiB.  On a 148-SM device with 8 KV heads that admits
 * Hq/Hkv = 2 up to B of about 130,000 entries and Hq/Hkv = 4 up to about 25,000; Hq/Hkv = 8 does
 * not fit.  Every GPU that loads the library keeps the 8 MiB until the process ends.
 *
 * The first call on each device looks up the array's device address (one cudaGetSymbolAddress,
 * with that device current); make that first call before any stream capture begins.
 * All calls on a device share the one array: each call clears the counters it needs on `stream`
 * before its kernel, and calls that overlap on the GPU (different streams, no dependency between
 * them) race on it - order them, or use b200kv_decode_attn with separate workspaces. */
size_t b200kv_decode_attn_static_limit(void);
int b200kv_decode_attn_static(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                              const b200kv_cache* cache, const b200kv_table* table,
                              const int32_t* cached_lens, const int32_t* num_decoding, float scale,
                              void* out, int64_t o_stride_b, int64_t o_stride_h,
                              int32_t B, int32_t Hq, int32_t sm_count, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200KV_H */
