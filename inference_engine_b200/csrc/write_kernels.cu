// Quantize-on-write kernels of the int8 KV-cache path: fused QK-RMSNorm + RoPE + int8
// quantization (decode and prefill flavours) and the prefix dequantizer.
//
// Bit-exactness contract: int8 codes, fp32 scales, calibration and bf16 outputs equal the
// reference arithmetic (qwen3-1.7b/kernels.py:410-480, 579-670, 764-823, 918-932) evaluated
// in IEEE fp32 with separately rounded operations.  Hence: explicit __f*_rn intrinsics (never
// contracted into FMA), IEEE sqrt and divide, and a fixed order for the sum of squares.
// This translation unit is additionally compiled with -fmad=false.
//
// Mapping: one warp per (token, head).  Lane l holds elements d = 4l..4l+3 of the 128-wide
// head, so lanes 0-15 own the first rotary half and lanes 16-31 the second; the rotation
// partner of a lane is lane ^ 16.  A warp reads one 256-byte bf16 head row with 8-byte loads
// (fully coalesced) and writes one 128-byte int8 row with 4-byte stores.
#include "common.cuh"

namespace b200kv {

constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ void load4_bf16(const void* base, int lane, float (&x)[4]) {
  uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(base) + 4 * lane);
  x[0] = bf16_bits_to_float(raw.x & 0xFFFFu);
  x[1] = bf16_bits_to_float(raw.x >> 16);
  x[2] = bf16_bits_to_float(raw.y & 0xFFFFu);
  x[3] = bf16_bits_to_float(raw.y >> 16);
}

__device__ __forceinline__ void store4_bf16(void* base, int lane, const float (&x)[4]) {
  uint2 raw;
  raw.x = float_to_bf16_bits(x[0]) | (float_to_bf16_bits(x[1]) << 16);
  raw.y = float_to_bf16_bits(x[2]) | (float_to_bf16_bits(x[3]) << 16);
  *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(base) + 4 * lane) = raw;
}

__device__ __forceinline__ void load4_f32(const float* base, int lane, float (&x)[4]) {
  float4 raw = *reinterpret_cast<const float4*>(base + 4 * lane);
  x[0] = raw.x; x[1] = raw.y; x[2] = raw.z; x[3] = raw.w;
}

// Sum of squares of the 128 elements spread over the warp, in the order the reference's
// `tl.sum(x1*x1) + tl.sum(x2*x2)` has under numpy: per 64-element half, eight strided running
// sums r[j] += a[8i+j] (i ascending), then ((r0+r1)+(r2+r3)) + ((r4+r5)+(r6+r7)); halves added
// first-half first.  `sq` is this warp's 128-float shared scratch.
__device__ __forceinline__ float sum_squares_ordered(const float (&x)[4], float* sq, int lane) {
  float4 s;
  s.x = __fmul_rn(x[0], x[0]); s.y = __fmul_rn(x[1], x[1]);
  s.z = __fmul_rn(x[2], x[2]); s.w = __fmul_rn(x[3], x[3]);
  __syncwarp();
  *reinterpret_cast<float4*>(sq + 4 * lane) = s;
  __syncwarp();
  const int l16 = lane & 15;
  const float* a = sq + (l16 >> 3) * kHalfD + (l16 & 7);
  float r = a[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) r = __fadd_rn(r, a[8 * i]);
  r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, 1));
  r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, 2));
  r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, 4));
  float first = __shfl_sync(0xffffffffu, r, 0);
  float second = __shfl_sync(0xffffffffu, r, 8);
  return __fadd_rn(first, second);
}

// RMSNorm + half-split rotation of one head row; result elements d = 4*lane + c.
// kernels.py:414-436 / 583-633.
__device__ __forceinline__ void norm_rope_head(const void* x_row, const void* w, const void* cos_row,
                                               const void* sin_row, float eps, float* sq, int lane, float (&out)[4]) {
  float x[4], wv[4], c[4], s[4];
  load4_bf16(x_row, lane, x);
  load4_bf16(w, lane, wv);
  load4_bf16(cos_row, lane & 15, c);
  load4_bf16(sin_row, lane & 15, s);
  float ss = sum_squares_ordered(x, sq, lane);
  float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)kD), eps)));
  const bool first_half = lane < 16;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float y = __fmul_rn(__fmul_rn(x[i], rstd), wv[i]);
    float other = __shfl_xor_sync(0xffffffffu, y, 16);
    float y1 = first_half ? y : other;
    float y2 = first_half ? other : y;
    out[i] = first_half ? __fsub_rn(__fmul_rn(y1, c[i]), __fmul_rn(y2, s[i]))
                        : __fadd_rn(__fmul_rn(y1, s[i]), __fmul_rn(y2, c[i]));
  }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Per-row absmax int8 quantizer (kernels.py:460-470, 475-480, 798-811): writes the 128 codes
// of one head row (4 per lane) and its scale.
__device__ __forceinline__ void quantize_store(const float (&x)[4], int8_t* code_row, float* scale_ptr, int lane) {
  float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
  amax = warp_max(amax);
  float scale = __fdiv_rn(fmaxf(amax, 1e-6f), 127.0f);
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float r = rintf(__fdiv_rn(x[i], scale));
    r = fminf(fmaxf(r, -127.0f), 127.0f);
    packed |= (static_cast<uint32_t>(static_cast<int>(r)) & 0xFFu) << (8 * i);
  }
  *reinterpret_cast<uint32_t*>(code_row + 4 * lane) = packed;
  if (lane == 0) *scale_ptr = scale;
}

// ------------------------------------------------------------------ decode write
// grid (B, ceil((Hq + 2*Hkv) / 8)), 256 threads.  Warp job j: [0,Hq) q heads, [Hq,Hq+Hkv) k
// heads, [Hq+Hkv, Hq+2Hkv) v heads.  kernels.py:364-480.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
write_decode_kernel(const uint16_t* __restrict__ q, long long q_sb, long long q_sh,
                    const uint16_t* __restrict__ k, long long k_sb, long long k_sh,
                    const uint16_t* __restrict__ v, long long v_sb, long long v_sh,
                    const uint16_t* __restrict__ qw, const uint16_t* __restrict__ kw,
                    const uint16_t* __restrict__ cosp, long long cos_sb,
                    const uint16_t* __restrict__ sinp, long long sin_sb,
                    CacheView c, const int32_t* __restrict__ cached_lens, const int32_t* __restrict__ num_decoding,
                    uint16_t* __restrict__ q_out, long long o_sb, long long o_sh, int Hq, float eps, int32_t* status) {
  __shared__ __align__(16) float sq_all[kWarpsPerBlock][kD];
  pdl_enter();
  const int b = blockIdx.x;
  if (b >= *num_decoding) return;
  pdl_wait();  // q, k, v come from the kernel before this one
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int job = blockIdx.y * kWarpsPerBlock + warp;
  const int Hkv = c.Hkv;
  if (job >= Hq + 2 * Hkv) return;
  float* sq = sq_all[warp];

  const int pos = cached_lens[b];
  if (job < Hq) {
    float r[4], cal[4];
    norm_rope_head(q + b * q_sb + job * q_sh, qw, cosp + b * cos_sb, sinp + b * sin_sb, eps, sq, lane, r);
    int page0 = lookup_page(c, b, 0, status);
    if (page0 < 0) return;
    const int hk = job / (Hq / Hkv);
    load4_f32(c.k_cal + page0 * c.cstride_page + hk * c.cstride_head, lane, cal);
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = __fmul_rn(r[i], cal[i]);
    store4_bf16(q_out + b * o_sb + job * o_sh, lane, r);
    return;
  }
  const int page = lookup_page(c, b, pos, status);
  if (page < 0) return;
  const int row = pos % c.page_size;
  if (job < Hq + Hkv) {
    const int j = job - Hq;
    float r[4], cal[4];
    norm_rope_head(k + b * k_sb + j * k_sh, kw, cosp + b * cos_sb, sinp + b * sin_sb, eps, sq, lane, r);
    int page0 = lookup_page(c, b, 0, status);
    if (page0 < 0) return;
    load4_f32(c.k_cal + page0 * c.cstride_page + j * c.cstride_head, lane, cal);
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = __fdiv_rn(r[i], cal[i]);
    quantize_store(r, c.k + page * c.stride_page + j * c.stride_head + row * c.stride_tok,
                   c.k_scale + page * c.sstride_page + j * c.sstride_head + row, lane);
  } else {
    const int j = job - Hq - Hkv;
    float x[4];
    load4_bf16(v + b * v_sb + j * v_sh, lane, x);
    quantize_store(x, c.v + page * c.stride_page + j * c.stride_head + row * c.stride_tok,
                   c.v_scale + page * c.sstride_page + j * c.sstride_head + row, lane);
  }
}

// ------------------------------------------------------------------ prefill norm + rope
// grid (N, ceil((Hq+Hkv)/8)); kernels.py:547-670.  Outputs rounded to bf16 (nearest even).
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
norm_rope_prefill_kernel(const uint16_t* __restrict__ q, long long q_sn, long long q_sh,
                         const uint16_t* __restrict__ k, long long k_sn, long long k_sh,
                         const uint16_t* __restrict__ qw, const uint16_t* __restrict__ kw,
                         const uint16_t* __restrict__ cosp, long long cos_sn,
                         const uint16_t* __restrict__ sinp, long long sin_sn,
                         uint16_t* __restrict__ q_out, long long qo_sn, long long qo_sh,
                         uint16_t* __restrict__ k_out, long long ko_sn, long long ko_sh,
                         int Hq, int Hkv, float eps) {
  __shared__ __align__(16) float sq_all[kWarpsPerBlock][kD];
  pdl_enter();
  const int n = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int job = blockIdx.y * kWarpsPerBlock + warp;
  if (job >= Hq + Hkv) return;
  pdl_wait();  // q and k come from the kernel before this one
  float r[4];
  if (job < Hq) {
    norm_rope_head(q + n * q_sn + job * q_sh, qw, cosp + n * cos_sn, sinp + n * sin_sn, eps, sq_all[warp], lane, r);
    store4_bf16(q_out + n * qo_sn + job * qo_sh, lane, r);
  } else {
    const int j = job - Hq;
    norm_rope_head(k + n * k_sn + j * k_sh, kw, cosp + n * cos_sn, sinp + n * sin_sn, eps, sq_all[warp], lane, r);
    store4_bf16(k_out + n * ko_sn + j * ko_sh, lane, r);
  }
}

// ------------------------------------------------------------------ prefill quantize
// Entry of packed row r, found by a whole warp: every lane tests one entry per round, so the answer costs one or
// two rounds of memory latency instead of log2(entries) dependent ones.  The entry holding row r is the one
// with cu[e] <= r < cu[e+1] (an empty entry never matches).  Returns -1 when r is past the last entry.
__device__ __forceinline__ int entry_of_row_warp(const int32_t* cu, int num_entries, int r, int lane) {
  for (int e0 = 0; e0 < num_entries; e0 += 32) {
    const int e = e0 + lane;
    const bool hit = e < num_entries && cu[e] <= r && r < cu[e + 1];
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    if (m) return e0 + __ffs(m) - 1;
  }
  return -1;
}

__device__ __forceinline__ bool is_first_chunk(int b, int nd, const int32_t* cu, const int32_t* cached_lens) {
  return b >= nd && cu[b + 1] > cu[b] && cached_lens[b] == 0;
}

// Phase 1: calibration of first-chunk entries: cal[d] = max(1e-3, max_t |k[t,d]|) over the chunk's rows
// (kernels.py:764-780).  max is exact and order-independent, so any split of the rows reproduces the serial
// result.  grid (num_entries, Hkv), 1024 threads: 32 row groups x 32 lanes of 4 channels (8-byte loads, eight
// rows in flight per thread), reduced through shared memory; entries that are not on their first chunk leave
// at once.
constexpr int kCalibGroups = 32;
__global__ void __launch_bounds__(kCalibGroups * 32)
calibrate_kernel(const uint16_t* __restrict__ k, long long k_sn, long long k_sh, CacheView c,
                 const int32_t* __restrict__ cu, const int32_t* __restrict__ cached_lens,
                 const int32_t* __restrict__ num_decoding, int N, int32_t* status) {
  pdl_enter();
  const int b = blockIdx.x, h = blockIdx.y;
  if (!is_first_chunk(b, *num_decoding, cu, cached_lens)) return;
  pdl_wait();  // k comes from the kernel before this one
  const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int s0 = cu[b], s1 = min(cu[b + 1], N);
  float m[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
  for (int t = s0 + g; t < s1; t += kCalibGroups) {
    float x[4];
    load4_bf16(k + t * k_sn + h * k_sh, lane, x);
#pragma unroll
    for (int i = 0; i < 4; ++i) m[i] = fmaxf(m[i], fabsf(x[i]));
  }
  __shared__ float part[kCalibGroups][kD];
#pragma unroll
  for (int i = 0; i < 4; ++i) part[g][4 * lane + i] = m[i];
  __syncthreads();
  if (threadIdx.x < kD) {
    float r = 1e-3f;
#pragma unroll
    for (int i = 0; i < kCalibGroups; ++i) r = fmaxf(r, part[i][threadIdx.x]);
    const int page0 = lookup_page(c, b, 0, status);
    if (page0 >= 0) c.k_cal[page0 * c.cstride_page + h * c.cstride_head + threadIdx.x] = r;
  }
}

// Phase 2: quantize every prefill row (kernels.py:786-823).  grid (N, ceil(2*Hkv/8)); warp job
// j: [0,Hkv) k heads, [Hkv,2Hkv) v heads.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
quantize_prefill_kernel(const uint16_t* __restrict__ k, long long k_sn, long long k_sh,
                        const uint16_t* __restrict__ v, long long v_sn, long long v_sh, CacheView c,
                        const int32_t* __restrict__ cu, int num_entries, const int32_t* __restrict__ cached_lens,
                        const int32_t* __restrict__ num_decoding, int32_t* status) {
  pdl_enter();
  const int r = blockIdx.x;
  if (r >= cu[num_entries]) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int job = blockIdx.y * kWarpsPerBlock + warp;
  if (job >= 2 * c.Hkv) return;
  const int b = entry_of_row_warp(cu, num_entries, r, lane);
  if (b < 0 || b < *num_decoding) return;
  pdl_wait();  // k, v and the calibration come from the kernels before this one
  float x[4];
  if (job < c.Hkv) load4_bf16(k + r * k_sn + job * k_sh, lane, x);  // in flight during the page lookups
  else load4_bf16(v + r * v_sn + (job - c.Hkv) * v_sh, lane, x);
  const int pos = cached_lens[b] + (r - cu[b]);
  const int page = lookup_page(c, b, pos, status);
  if (page < 0) return;
  const int row = pos % c.page_size;
  if (job < c.Hkv) {
    const int page0 = lookup_page(c, b, 0, status);
    if (page0 < 0) return;
    float cal[4];
    load4_f32(c.k_cal + page0 * c.cstride_page + job * c.cstride_head, lane, cal);
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = __fdiv_rn(x[i], cal[i]);
    quantize_store(x, c.k + page * c.stride_page + job * c.stride_head + row * c.stride_tok,
                   c.k_scale + page * c.sstride_page + job * c.sstride_head + row, lane);
  } else {
    const int j = job - c.Hkv;
    quantize_store(x, c.v + page * c.stride_page + j * c.stride_head + row * c.stride_tok,
                   c.v_scale + page * c.sstride_page + j * c.sstride_head + row, lane);
  }
}

// ------------------------------------------------------------------ prefix dequant
// kernels.py:868-932.  The output rows are packed end to end (cu_cached), so the grid runs over OUTPUT rows: one warp per row, all
// kv heads (a grid over (entry, token tile) would launch one mostly idle CTA column per entry of the batch).
// The warp finds the row's entry and page once; the loads of the heads are independent of one another, so they
// are all in flight together.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
dequant_prefix_kernel(CacheView c, const int32_t* __restrict__ cu_cached, int num_entries, uint16_t* __restrict__ k_out,
                      uint16_t* __restrict__ v_out, long long o_sh, long long o_sn, int capacity, int32_t* status) {
  pdl_enter();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * kWarpsPerBlock + warp;
  if (r >= min(cu_cached[num_entries], capacity)) return;
  // the entry b with cu_cached[b] <= r < cu_cached[b+1] (entries without a prefix never match)
  int b = -1, start = 0;
  for (int e0 = 0; e0 < num_entries && b < 0; e0 += 32) {
    const int e = e0 + lane;
    const int lo = e < num_entries ? cu_cached[e] : 0, hi = e < num_entries ? cu_cached[e + 1] : 0;
    const unsigned hit = __ballot_sync(0xffffffffu, e < num_entries && lo <= r && r < hi);
    if (hit) {
      const int src = __ffs(hit) - 1;
      b = e0 + src;
      start = __shfl_sync(0xffffffffu, lo, src);
    }
  }
  if (b < 0) return;
  const int t = r - start;
  const int page0 = lookup_page(c, b, 0, status);
  const int page = lookup_page(c, b, t, status);
  if (page0 < 0 || page < 0) return;
  const int row = t % c.page_size;
  pdl_wait();  // the cache is written by the kernels before this one
  constexpr int kHeadsAtOnce = 4;
  for (int h0 = 0; h0 < c.Hkv; h0 += kHeadsAtOnce) {
    uint32_t kc[kHeadsAtOnce], vc[kHeadsAtOnce];
    float ks[kHeadsAtOnce], vs[kHeadsAtOnce], cal[kHeadsAtOnce][4];
#pragma unroll
    for (int i = 0; i < kHeadsAtOnce; ++i) {
      const int h = min(h0 + i, c.Hkv - 1);
      const long long coff = page * c.stride_page + h * c.stride_head + row * c.stride_tok + 4 * lane;
      const long long soff = page * c.sstride_page + h * c.sstride_head + row;
      kc[i] = *reinterpret_cast<const uint32_t*>(c.k + coff);
      vc[i] = *reinterpret_cast<const uint32_t*>(c.v + coff);
      ks[i] = c.k_scale[soff];
      vs[i] = c.v_scale[soff];
      load4_f32(c.k_cal + page0 * c.cstride_page + h * c.cstride_head, lane, cal[i]);
    }
#pragma unroll
    for (int i = 0; i < kHeadsAtOnce; ++i) {
      const int h = h0 + i;
      if (h >= c.Hkv) break;
      float ko[4], vo[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float kf = (float)(int)(int8_t)((kc[i] >> (8 * j)) & 0xFFu);
        const float vf = (float)(int)(int8_t)((vc[i] >> (8 * j)) & 0xFFu);
        ko[j] = __fmul_rn(__fmul_rn(kf, ks[i]), cal[i][j]);
        vo[j] = __fmul_rn(vf, vs[i]);
      }
      const long long ooff = h * o_sh + (long long)r * o_sn;
      store4_bf16(k_out + ooff, lane, ko);
      store4_bf16(v_out + ooff, lane, vo);
    }
  }
}

static inline int launch_status() { return cudaGetLastError() == cudaSuccess ? B200KV_OK : B200KV_E_LAUNCH; }
static inline bool stride_ok4(long long s) { return (s % 4) == 0; }

}  // namespace b200kv

using namespace b200kv;

extern "C" int b200kv_write_decode(const void* q, int64_t q_sb, int64_t q_sh, const void* k, int64_t k_sb, int64_t k_sh,
                                   const void* v, int64_t v_sb, int64_t v_sh, const void* qw, const void* kw,
                                   const void* cosp, int64_t cos_sb, const void* sinp, int64_t sin_sb,
                                   const b200kv_cache* cache, const b200kv_table* table, const int32_t* cached_lens,
                                   const int32_t* num_decoding, void* q_out, int64_t o_sb, int64_t o_sh, int32_t B,
                                   int32_t Hq, float eps, int32_t* status, void* stream) {
  // an empty batch is valid and has nothing to launch (its tensors have no storage, so their pointers are NULL)
  if (B == 0) return B200KV_OK;
  if (!q || !k || !v || !qw || !kw || !cosp || !sinp || !cached_lens || !num_decoding || !q_out) return B200KV_E_NULL;
  int rc = check_cache(cache, table);
  if (rc) return rc;
  const int Hkv = cache->num_kv_heads;
  if (B < 0 || Hq < 1 || Hq % Hkv) return B200KV_E_SHAPE;
  if (!aligned(q, 8) || !aligned(k, 8) || !aligned(v, 8) || !aligned(qw, 8) || !aligned(kw, 8) || !aligned(cosp, 8) ||
      !aligned(sinp, 8) || !aligned(q_out, 8))
    return B200KV_E_ALIGN;
  if (!stride_ok4(q_sb) || !stride_ok4(q_sh) || !stride_ok4(k_sb) || !stride_ok4(k_sh) || !stride_ok4(v_sb) ||
      !stride_ok4(v_sh) || !stride_ok4(cos_sb) || !stride_ok4(sin_sb) || !stride_ok4(o_sb) || !stride_ok4(o_sh))
    return B200KV_E_ALIGN;
  if (B == 0) return B200KV_OK;
  dim3 grid(B, (Hq + 2 * Hkv + kWarpsPerBlock - 1) / kWarpsPerBlock);
  launch_chained(write_decode_kernel, grid, dim3(kWarpsPerBlock * 32), 0, (cudaStream_t)stream,
      (const uint16_t*)q, q_sb, q_sh, (const uint16_t*)k, k_sb, k_sh, (const uint16_t*)v, v_sb, v_sh,
      (const uint16_t*)qw, (const uint16_t*)kw, (const uint16_t*)cosp, cos_sb, (const uint16_t*)sinp, sin_sb,
      make_view(cache, table), cached_lens, num_decoding, (uint16_t*)q_out, o_sb, o_sh, Hq, eps, status);
  return launch_status();
}

extern "C" int b200kv_norm_rope_prefill(const void* q, int64_t q_sn, int64_t q_sh, const void* k, int64_t k_sn,
                                        int64_t k_sh, const void* qw, const void* kw, const void* cosp, int64_t cos_sn,
                                        const void* sinp, int64_t sin_sn, void* q_out, int64_t qo_sn, int64_t qo_sh,
                                        void* k_out, int64_t ko_sn, int64_t ko_sh, int32_t N, int32_t Hq, int32_t Hkv,
                                        int32_t D, float eps, void* stream) {
  // an empty batch is valid and has nothing to launch (its tensors have no storage, so their pointers are NULL)
  if (N == 0) return B200KV_OK;
  if (!q || !k || !qw || !kw || !cosp || !sinp || !q_out || !k_out) return B200KV_E_NULL;
  if (D != kD || Hq < 1 || Hkv < 1 || N < 0) return B200KV_E_SHAPE;
  if (!aligned(q, 8) || !aligned(k, 8) || !aligned(qw, 8) || !aligned(kw, 8) || !aligned(cosp, 8) || !aligned(sinp, 8) ||
      !aligned(q_out, 8) || !aligned(k_out, 8))
    return B200KV_E_ALIGN;
  if (!stride_ok4(q_sn) || !stride_ok4(q_sh) || !stride_ok4(k_sn) || !stride_ok4(k_sh) || !stride_ok4(cos_sn) ||
      !stride_ok4(sin_sn) || !stride_ok4(qo_sn) || !stride_ok4(qo_sh) || !stride_ok4(ko_sn) || !stride_ok4(ko_sh))
    return B200KV_E_ALIGN;
  if (N == 0) return B200KV_OK;
  dim3 grid(N, (Hq + Hkv + kWarpsPerBlock - 1) / kWarpsPerBlock);
  launch_chained(norm_rope_prefill_kernel, grid, dim3(kWarpsPerBlock * 32), 0, (cudaStream_t)stream,
      (const uint16_t*)q, q_sn, q_sh, (const uint16_t*)k, k_sn, k_sh, (const uint16_t*)qw, (const uint16_t*)kw,
      (const uint16_t*)cosp, cos_sn, (const uint16_t*)sinp, sin_sn, (uint16_t*)q_out, qo_sn, qo_sh, (uint16_t*)k_out,
      ko_sn, ko_sh, Hq, Hkv, eps);
  return launch_status();
}

extern "C" int b200kv_quantize_prefill(const void* k, int64_t k_sn, int64_t k_sh, const void* v, int64_t v_sn,
                                       int64_t v_sh, const int32_t* cu_seqlens, int32_t num_entries,
                                       const b200kv_cache* cache, const b200kv_table* table, const int32_t* cached_lens,
                                       const int32_t* num_decoding, int32_t N, int32_t* status, void* stream) {
  // an empty batch is valid and has nothing to launch (its tensors have no storage, so their pointers are NULL)
  if (N == 0 || num_entries == 0) return B200KV_OK;
  if (!k || !v || !cu_seqlens || !cached_lens || !num_decoding) return B200KV_E_NULL;
  int rc = check_cache(cache, table);
  if (rc) return rc;
  if (N < 0 || num_entries < 0) return B200KV_E_SHAPE;
  if (!aligned(k, 8) || !aligned(v, 8) || !stride_ok4(k_sn) || !stride_ok4(k_sh) || !stride_ok4(v_sn) || !stride_ok4(v_sh))
    return B200KV_E_ALIGN;
  if (N == 0 || num_entries == 0) return B200KV_OK;
  const int Hkv = cache->num_kv_heads;
  CacheView view = make_view(cache, table);
  cudaStream_t s = (cudaStream_t)stream;
  launch_chained(calibrate_kernel, dim3(num_entries, Hkv), dim3(kCalibGroups * 32), 0, s, (const uint16_t*)k, k_sn, k_sh, view,
                 cu_seqlens, cached_lens, num_decoding, N, status);
  launch_chained(quantize_prefill_kernel, dim3(N, (2 * Hkv + kWarpsPerBlock - 1) / kWarpsPerBlock), dim3(kWarpsPerBlock * 32), 0, s,
      (const uint16_t*)k, k_sn, k_sh, (const uint16_t*)v, v_sn, v_sh, view, cu_seqlens, num_entries, cached_lens,
      num_decoding, status);
  return launch_status();
}

extern "C" int b200kv_dequant_prefix(const b200kv_cache* cache, const b200kv_table* table, const int32_t* cu_cached,
                                     int32_t num_entries, void* k_out, void* v_out, int64_t o_sh, int64_t o_sn,
                                     int32_t capacity, int32_t* status, void* stream) {
  // an empty batch is valid and has nothing to launch (its tensors have no storage, so their pointers are NULL)
  if (num_entries == 0 || capacity == 0) return B200KV_OK;
  if (!cu_cached || !k_out || !v_out) return B200KV_E_NULL;
  int rc = check_cache(cache, table);
  if (rc) return rc;
  if (num_entries < 0 || capacity < 0) return B200KV_E_SHAPE;
  if (!aligned(k_out, 8) || !aligned(v_out, 8) || !stride_ok4(o_sh) || !stride_ok4(o_sn)) return B200KV_E_ALIGN;
  if (num_entries == 0 || capacity == 0) return B200KV_OK;
  dim3 grid((unsigned)((capacity + kWarpsPerBlock - 1) / kWarpsPerBlock));
  launch_chained(dequant_prefix_kernel, grid, dim3(kWarpsPerBlock * 32), 0, (cudaStream_t)stream,
      make_view(cache, table), cu_cached, num_entries, (uint16_t*)k_out, (uint16_t*)v_out, o_sh, o_sn, capacity, status);
  return launch_status();
}
