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
// kernels.py:414-436 / 583-633.  The operands are already in registers, so that a caller can put all of its
// loads (this row, the page table, the calibration) in flight before the first arithmetic instruction needs one.
struct HeadRow {
  uint2 x, w, c, s;  // 4 bf16 each: the row, the norm weight, cos and sin of this lane's rotary columns
};
__device__ __forceinline__ HeadRow load_head_row(const void* x_row, const void* w, const void* cos_row,
                                                 const void* sin_row, int lane) {
  HeadRow r;
  r.x = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(x_row) + 4 * lane);
  r.w = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(w) + 4 * lane);
  r.c = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(cos_row) + 4 * (lane & 15));
  r.s = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(sin_row) + 4 * (lane & 15));
  return r;
}
__device__ __forceinline__ void unpack4(uint2 raw, float (&x)[4]) {
  x[0] = bf16_bits_to_float(raw.x & 0xFFFFu);
  x[1] = bf16_bits_to_float(raw.x >> 16);
  x[2] = bf16_bits_to_float(raw.y & 0xFFFFu);
  x[3] = bf16_bits_to_float(raw.y >> 16);
}
__device__ __forceinline__ void norm_rope_regs(const HeadRow& row, float eps, float* sq, int lane, float (&out)[4]);

__device__ __forceinline__ void norm_rope_head(const void* x_row, const void* w, const void* cos_row,
                                               const void* sin_row, float eps, float* sq, int lane, float (&out)[4]) {
  norm_rope_regs(load_head_row(x_row, w, cos_row, sin_row, lane), eps, sq, lane, out);
}

__device__ __forceinline__ void norm_rope_regs(const HeadRow& row, float eps, float* sq, int lane, float (&out)[4]) {
  float x[4], wv[4], c[4], s[4];
  unpack4(row.x, x);
  unpack4(row.w, wv);
  unpack4(row.c, c);
  unpack4(row.s, s);
  float ss = sum_squares_ordered(x, sq, lane);
  // ss / 128 as a product with 2^-7: both are the correctly rounded value of the same real number
  static_assert(kD == 128, "the mean is taken with a power-of-two factor");
  float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(ss, 0.0078125f), eps)));
  // First half: y1*c - y2*s with y1 = mine, y2 = the partner's; second half: y1*s + y2*c with y1 = the partner's,
  // y2 = mine.  Both are mine*c + partner*(-+s): subtracting is adding the negated product and the sum commutes,
  // so one expression with a signed sine gives the same bits as the two of the reference.
  const bool first_half = lane < 16;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float y = __fmul_rn(__fmul_rn(x[i], rstd), wv[i]);
    float other = __shfl_xor_sync(0xffffffffu, y, 16);
    out[i] = __fadd_rn(__fmul_rn(y, c[i]), __fmul_rn(other, first_half ? -s[i] : s[i]));
  }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Per-row absmax int8 quantizer (kernels.py:460-470, 475-480, 798-811): writes the 128 codes
// of one head row (4 per lane) and its scale.  code = rint(x / scale) with the IEEE quotient: the quotient is
// first estimated as x * (127 / amax) with an approximate reciprocal (2 ulp), which is within 6e-5 of it for
// |x / scale| <= 127.5 (the rounding of scale itself, the approximate division, the product); only when that
// estimate lies within 2e-4 of a rounding boundary (k + 0.5) can the two round to different integers, and only
// then is the division carried out.  The estimate does not wait for the division that produces the stored scale.
__device__ __forceinline__ void quantize_store(const float (&x)[4], int8_t* code_row, float* scale_ptr, int lane) {
  float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
  amax = warp_max(amax);
  const float floor_max = fmaxf(amax, 1e-6f);
  const float scale = __fdiv_rn(floor_max, 127.0f);
  // (the approximate division returns 0 for divisors above 2^126: rows with such values divide every element)
  const float inv = __fdividef(127.0f, floor_max);
  const float band = amax < 1e30f ? 2e-4f : __int_as_float(0x7f800000);
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float est = __fmul_rn(x[i], inv);
    float r = rintf(est);
    if (fabsf(fabsf(__fsub_rn(est, r)) - 0.5f) < band) r = rintf(__fdiv_rn(x[i], scale));
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
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int job = blockIdx.y * kWarpsPerBlock + warp;
  const int Hkv = c.Hkv;
  if (job >= Hq + 2 * Hkv) return;
  float* sq = sq_all[warp];
  // Round one of loads (metadata, allowed before the wait): where the new token goes and the page that holds the
  // sequence's calibration row.
  const int32_t* trow = c.table + (long long)b * c.table_stride;
  const int pos = cached_lens[b];
  int page0 = trow[0];
  pdl_wait();  // q, k, v come from the kernel before this one
  // ... and this warp's head row with its norm weight and rotary columns
  const bool is_q = job < Hq, is_k = !is_q && job < Hq + Hkv;
  const int j = is_q ? job : (is_k ? job - Hq : job - Hq - Hkv);
  HeadRow row;
  if (is_q) row = load_head_row(q + act_offset(b, q_sb, j, q_sh), qw, cosp + (long long)b * (int)cos_sb, sinp + (long long)b * (int)sin_sb, lane);
  else if (is_k) row = load_head_row(k + act_offset(b, k_sb, j, k_sh), kw, cosp + (long long)b * (int)cos_sb, sinp + (long long)b * (int)sin_sb, lane);
  else row.x = *reinterpret_cast<const uint2*>(v + act_offset(b, v_sb, j, v_sh) + 4 * lane);
  // Round two, issued as soon as round one's metadata is there: the page of the new token and the calibration.
  int slot, prow;
  split_pos(c, pos, slot, prow);
  const bool pos_ok = pos >= 0 && slot < c.max_pages;
  int page = (!is_q && pos_ok) ? trow[slot] : 0;
  const bool page0_ok = page0 >= 0 && page0 < c.num_pages;
  float cal[4] = {1.f, 1.f, 1.f, 1.f};
  if ((is_q || is_k) && page0_ok)
    load4_f32(c.k_cal + cal_offset(c, page0, is_q ? j / (Hq / Hkv) : j), lane, cal);
  if ((is_q || is_k) && !page0_ok) {
    if (lane == 0 && status) atomicOr(status, B200KV_S_BAD_PAGE);
    return;
  }
  if (!is_q) {
    if (!pos_ok) {
      if (lane == 0 && status) atomicOr(status, B200KV_S_BAD_POSITION);
      return;
    }
    if (page < 0 || page >= c.num_pages) {
      if (lane == 0 && status) atomicOr(status, B200KV_S_BAD_PAGE);
      return;
    }
  }
  float r[4];
  if (is_q) {
    norm_rope_regs(row, eps, sq, lane, r);
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = __fmul_rn(r[i], cal[i]);
    store4_bf16(q_out + act_offset(b, o_sb, j, o_sh), lane, r);
  } else if (is_k) {
    norm_rope_regs(row, eps, sq, lane, r);
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = __fdiv_rn(r[i], cal[i]);
    quantize_store(r, c.k + code_offset(c, page, j, prow), c.k_scale + scale_offset(c, page, j, prow), lane);
  } else {
    unpack4(row.x, r);
    quantize_store(r, c.v + code_offset(c, page, j, prow), c.v_scale + scale_offset(c, page, j, prow), lane);
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
    norm_rope_head(q + act_offset(n, q_sn, job, q_sh), qw, cosp + (long long)n * (int)cos_sn, sinp + (long long)n * (int)sin_sn, eps, sq_all[warp], lane, r);
    store4_bf16(q_out + act_offset(n, qo_sn, job, qo_sh), lane, r);
  } else {
    const int j = job - Hq;
    norm_rope_head(k + act_offset(n, k_sn, j, k_sh), kw, cosp + (long long)n * (int)cos_sn, sinp + (long long)n * (int)sin_sn, eps, sq_all[warp], lane, r);
    store4_bf16(k_out + act_offset(n, ko_sn, j, ko_sh), lane, r);
  }
}

// ------------------------------------------------------------------ prefill quantize
__device__ __forceinline__ bool is_first_chunk(int b, int nd, const int32_t* cu, const int32_t* cached_lens) {
  return b >= nd && cu[b + 1] > cu[b] && cached_lens[b] == 0;
}

// ------------------------------------------------------------------ prefill write
// Two kernels that do not depend on one another replace the reference's serial loop over a chunk (8 programs per
// chunk, kernels.py:717-823):
//   rows kernel        one warp per (packed row, head): V of every prefilling row, and K of the rows whose entry
//                      already has a calibration (not its first chunk): k / calibration -> codes + scale;
//   first-chunk kernel K of entries on their first chunk, which need the column maxima of the WHOLE chunk before
//                      any row can be quantized (kernels.py:764-780): a cluster of kFirstCtas CTAs per kv head
//                      shares the rows, exchanges its 128 column maxima through distributed shared memory between
//                      two cluster barriers (no global round trip, no spinning) and quantizes its rows from registers.
// The fused entry point runs the rows kernel with the norm + rope of q and k folded in (one launch does what
// fused_norm_rope_prefill and the row part of quantize_kv_prefill do), then the first-chunk kernel.

// Which entry owns packed row r, with that entry's first row, cached length and first page, found by the whole
// warp in one round of loads (lane e tests entry e0 + e).  b = -1: the row lies behind the last entry.
struct RowEntry {
  int b, start, cached, page0;
};
__device__ __forceinline__ RowEntry find_row_entry(const int32_t* __restrict__ cu, int num_entries,
                                                   const int32_t* __restrict__ cached_lens, const CacheView& c, int r, int lane) {
  RowEntry re{-1, 0, 0, -1};
  for (int e0 = 0; e0 < num_entries; e0 += 32) {
    const int e = e0 + lane;
    const bool in = e < num_entries;
    const int lo = in ? cu[e] : 0, hi = in ? cu[e + 1] : 0;
    const int cl = in ? cached_lens[e] : 0;
    const int p0 = in ? c.table[(long long)e * c.table_stride] : -1;
    const unsigned m = __ballot_sync(0xffffffffu, in && lo <= r && r < hi);
    if (m) {
      const int src = __ffs(m) - 1;
      re.b = e0 + src;
      re.start = __shfl_sync(0xffffffffu, lo, src);
      re.cached = __shfl_sync(0xffffffffu, cl, src);
      re.page0 = __shfl_sync(0xffffffffu, p0, src);
      break;
    }
  }
  return re;
}

// The cache row of token position `pos` of entry b: page id from the table (bounds-checked, status bit on failure).
__device__ __forceinline__ int page_of(const CacheView& c, int b, int pos, int32_t* status, int lane) {
  int slot, prow;
  split_pos(c, pos, slot, prow);
  if (pos < 0 || slot >= c.max_pages) {
    if (lane == 0 && status) atomicOr(status, B200KV_S_BAD_POSITION);
    return -1;
  }
  const int page = c.table[(long long)b * c.table_stride + slot];
  if (page < 0 || page >= c.num_pages) {
    if (lane == 0 && status) atomicOr(status, B200KV_S_BAD_PAGE);
    return -1;
  }
  return page;
}

// kFusedNorm = true: q, k are the raw projections; the kernel norms and ropes every row of them into q_out / k_out
// (what fused_norm_rope_prefill does, kernels.py:547-670) and quantizes from the bf16-rounded k it just produced.
// kFusedNorm = false: k is already normed + roped bf16 (the argument of quantize_kv_prefill), q is not touched.
// grid (N, ceil(jobs / 8)); warp job: [0, Hq) q heads (fused only), then Hkv k heads, then Hkv v heads.
template <bool kFusedNorm>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
prefill_rows_kernel(const uint16_t* __restrict__ q, long long q_sn, long long q_sh,
                    const uint16_t* __restrict__ k, long long k_sn, long long k_sh,
                    const uint16_t* __restrict__ v, long long v_sn, long long v_sh,
                    const uint16_t* __restrict__ qw, const uint16_t* __restrict__ kw,
                    const uint16_t* __restrict__ cosp, long long cos_sn, const uint16_t* __restrict__ sinp, long long sin_sn,
                    uint16_t* __restrict__ q_out, long long qo_sn, long long qo_sh,
                    uint16_t* __restrict__ k_out, long long ko_sn, long long ko_sh,
                    CacheView c, const int32_t* __restrict__ cu, int num_entries, const int32_t* __restrict__ cached_lens,
                    const int32_t* __restrict__ num_decoding, int Hq, float eps, int32_t* status) {
  __shared__ __align__(16) float sq_all[kFusedNorm ? kWarpsPerBlock : 1][kD];
  pdl_enter();
  const int r = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int job = blockIdx.y * kWarpsPerBlock + warp;
  const int Hkv = c.Hkv, nq = kFusedNorm ? Hq : 0;
  if (job >= nq + 2 * Hkv) return;
  const bool is_q = job < nq, is_k = !is_q && job < nq + Hkv;
  const int j = is_q ? job : (is_k ? job - nq : job - nq - Hkv);
  // round one (metadata, readable before the wait): the row's entry
  const int nd = *num_decoding;
  const RowEntry re = find_row_entry(cu, num_entries, cached_lens, c, r, lane);
  const bool prefilling = re.b >= 0 && re.b >= nd;
  const bool first_chunk = prefilling && re.cached == 0;
  if (!kFusedNorm && (!prefilling || (is_k && first_chunk))) return;  // nothing to quantize here
  if (kFusedNorm && !is_q && !is_k && !prefilling) return;
  pdl_wait();  // q, k, v come from the kernel before this one
  HeadRow row;
  if (kFusedNorm && is_q) row = load_head_row(q + act_offset(r, q_sn, j, q_sh), qw, cosp + (long long)r * (int)cos_sn, sinp + (long long)r * (int)sin_sn, lane);
  else if (kFusedNorm && is_k) row = load_head_row(k + act_offset(r, k_sn, j, k_sh), kw, cosp + (long long)r * (int)cos_sn, sinp + (long long)r * (int)sin_sn, lane);
  else row.x = *reinterpret_cast<const uint2*>((is_k ? k + act_offset(r, k_sn, j, k_sh) : v + act_offset(r, v_sn, j, v_sh)) + 4 * lane);
  // round two: the page of this row's token and the entry's calibration
  const bool quantizes = prefilling && !is_q && !(is_k && first_chunk);
  const int pos = re.cached + (r - re.start);
  int page = -1;
  float cal[4] = {1.f, 1.f, 1.f, 1.f};
  if (quantizes) {
    page = page_of(c, re.b, pos, status, lane);
    if (is_k) {
      if (re.page0 < 0 || re.page0 >= c.num_pages) {
        if (lane == 0 && status) atomicOr(status, B200KV_S_BAD_PAGE);
        page = -1;
      } else {
        load4_f32(c.k_cal + cal_offset(c, re.page0, j), lane, cal);
      }
    }
  }
  float x[4];
  if (kFusedNorm && (is_q || is_k)) {
    norm_rope_regs(row, eps, sq_all[kFusedNorm ? warp : 0], lane, x);
    if (is_q) {
      store4_bf16(q_out + act_offset(r, qo_sn, j, qo_sh), lane, x);
      return;
    }
    store4_bf16(k_out + act_offset(r, ko_sn, j, ko_sh), lane, x);
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = bf16_bits_to_float(float_to_bf16_bits(x[i]));  // the quantizer reads the stored bf16
  } else {
    unpack4(row.x, x);
  }
  if (!quantizes || page < 0) return;
  int slot_unused, prow;
  split_pos(c, pos, slot_unused, prow);
  if (is_k) {
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = __fdiv_rn(x[i], cal[i]);
    quantize_store(x, c.k + code_offset(c, page, j, prow), c.k_scale + scale_offset(c, page, j, prow), lane);
  } else {
    quantize_store(x, c.v + code_offset(c, page, j, prow), c.v_scale + scale_offset(c, page, j, prow), lane);
  }
}

// K of first-chunk entries.  grid (Hkv, kFirstLanes, kFirstCtas), cluster (1, 1, kFirstCtas), kFirstWarps warps.
// Cluster (h, y) walks the entries b = y, y + kFirstLanes, ... that are on their first chunk; its CTAs share the
// chunk's rows round-robin by warp.  Per entry: every warp takes the column maxima of its rows (the first
// kKeepRows stay in registers), the CTA folds its warps' maxima in shared memory, the cluster's CTAs read one
// another's 128 maxima through distributed shared memory between two cluster barriers, calibration =
// max(1e-3, column max) (exact and order-independent, kernels.py:764-780) is stored by CTA 0, and every warp
// quantizes its rows as k / calibration (kernels.py:786-811).
constexpr int kFirstCtas = 8, kFirstWarps = 16, kFirstLanes = 4, kKeepRows = 8;
__global__ void __launch_bounds__(kFirstWarps * 32)
first_chunk_k_kernel(const uint16_t* __restrict__ k, long long k_sn, long long k_sh, CacheView c,
                     const int32_t* __restrict__ cu, int num_entries, const int32_t* __restrict__ cached_lens,
                     const int32_t* __restrict__ num_decoding, int N, int32_t* status) {
  __shared__ __align__(16) float part[kFirstWarps][kD];
  __shared__ float cta_max[kD];
  __shared__ __align__(16) float cal_s[kD];
  pdl_enter();
  const int h = blockIdx.x, y = blockIdx.y;
  unsigned crank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nd = *num_decoding;
  const int wid = (int)crank * kFirstWarps + warp, nw = kFirstCtas * kFirstWarps;  // this warp among the cluster's
  bool waited = false;
  for (int e0 = 0; e0 < num_entries; e0 += 32) {
    // the entries of this cluster's lane that are on their first chunk, 32 candidates per round of loads; every
    // thread of the cluster sees the same mask, so the barriers below are reached by all or by none
    const int e = e0 + lane;
    unsigned mask = __ballot_sync(0xffffffffu, e < num_entries && (e % kFirstLanes) == y && is_first_chunk(e, nd, cu, cached_lens));
    while (mask) {
      const int b = e0 + __ffs(mask) - 1;
      mask &= mask - 1;
      if (!waited) {
        pdl_wait();  // k comes from the kernel before this one
        waited = true;
      }
      const int s0 = cu[b], s1 = min(cu[b + 1], N);
      const uint16_t* kcol = k + h * k_sh + 4 * lane;
      uint2 keep[kKeepRows];
      int keep_page[kKeepRows];  // table entries of the kept rows, fetched in the same round as the rows
      float m[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < kKeepRows; ++i) {  // independent loads: all in flight together
        const int t = s0 + wid + i * nw;
        keep[i] = t < s1 ? *reinterpret_cast<const uint2*>(kcol + (long long)t * (int)k_sn) : make_uint2(0u, 0u);
        int slot, prow_unused;
        split_pos(c, t - s0, slot, prow_unused);
        keep_page[i] = (t < s1 && slot < c.max_pages) ? c.table[(long long)b * c.table_stride + slot] : -2;
      }
#pragma unroll
      for (int i = 0; i < kKeepRows; ++i) {
        float x[4];
        unpack4(keep[i], x);
#pragma unroll
        for (int j = 0; j < 4; ++j) m[j] = fmaxf(m[j], fabsf(x[j]));
      }
      for (int t = s0 + wid + kKeepRows * nw; t < s1; t += nw) {  // chunks beyond kKeepRows * 128 rows
        float x[4];
        unpack4(*reinterpret_cast<const uint2*>(kcol + (long long)t * (int)k_sn), x);
#pragma unroll
        for (int j = 0; j < 4; ++j) m[j] = fmaxf(m[j], fabsf(x[j]));
      }
      *reinterpret_cast<float4*>(&part[warp][4 * lane]) = make_float4(m[0], m[1], m[2], m[3]);
      __syncthreads();
      if (threadIdx.x < kD) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kFirstWarps; ++w) v = fmaxf(v, part[w][threadIdx.x]);
        cta_max[threadIdx.x] = v;
      }
      asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
      if (threadIdx.x < kD) {
        float v = 1e-3f;
        const uint32_t mine = (uint32_t)__cvta_generic_to_shared(&cta_max[threadIdx.x]);
#pragma unroll
        for (int p = 0; p < kFirstCtas; ++p) {
          uint32_t remote;
          float pv;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(mine), "r"(p));
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(pv) : "r"(remote) : "memory");
          v = fmaxf(v, pv);
        }
        cal_s[threadIdx.x] = v;
      }
      // nobody may overwrite cta_max (next entry) or leave while a peer still reads it
      asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
      __syncthreads();
      const int page0 = c.table[(long long)b * c.table_stride];
      const bool page0_ok = page0 >= 0 && page0 < c.num_pages;
      if (!page0_ok && crank == 0 && threadIdx.x == 0 && status) atomicOr(status, B200KV_S_BAD_PAGE);
      if (crank == 0 && threadIdx.x < kD && page0_ok)
        c.k_cal[cal_offset(c, page0, h) + threadIdx.x] = cal_s[threadIdx.x];
      float cal[4];
      load4_f32(cal_s, lane, cal);
      auto quantize_row = [&](int t, uint2 raw, int page) {
        float x[4];
        unpack4(raw, x);
#pragma unroll
        for (int j = 0; j < 4; ++j) x[j] = __fdiv_rn(x[j], cal[j]);
        const int pos = t - s0;  // first chunk: the entry's cached length is zero
        if (page < 0 || page >= c.num_pages) {
          if (lane == 0 && status) atomicOr(status, page == -2 ? B200KV_S_BAD_POSITION : B200KV_S_BAD_PAGE);
          return;
        }
        int slot_unused, prow;
        split_pos(c, pos, slot_unused, prow);
        quantize_store(x, c.k + code_offset(c, page, h, prow), c.k_scale + scale_offset(c, page, h, prow), lane);
      };
#pragma unroll
      for (int i = 0; i < kKeepRows; ++i) {
        const int t = s0 + wid + i * nw;
        if (t < s1) quantize_row(t, keep[i], keep_page[i]);
      }
      for (int t = s0 + wid + kKeepRows * nw; t < s1; t += nw) {
        int slot, prow_unused;
        split_pos(c, t - s0, slot, prow_unused);
        quantize_row(t, *reinterpret_cast<const uint2*>(kcol + (long long)t * (int)k_sn),
                     slot < c.max_pages ? c.table[(long long)b * c.table_stride + slot] : -2);
      }
      __syncthreads();  // part / cal_s are reused by the next entry
    }
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
  int slot_unused, row;
  split_pos(c, t, slot_unused, row);
  pdl_wait();  // the cache is written by the kernels before this one
  constexpr int kHeadsAtOnce = 4;
  for (int h0 = 0; h0 < c.Hkv; h0 += kHeadsAtOnce) {
    uint32_t kc[kHeadsAtOnce], vc[kHeadsAtOnce];
    float ks[kHeadsAtOnce], vs[kHeadsAtOnce], cal[kHeadsAtOnce][4];
#pragma unroll
    for (int i = 0; i < kHeadsAtOnce; ++i) {
      const int h = min(h0 + i, c.Hkv - 1);
      const long long coff = code_offset(c, page, h, row) + 4 * lane;
      const long long soff = scale_offset(c, page, h, row);
      kc[i] = *reinterpret_cast<const uint32_t*>(c.k + coff);
      vc[i] = *reinterpret_cast<const uint32_t*>(c.v + coff);
      ks[i] = c.k_scale[soff];
      vs[i] = c.v_scale[soff];
      load4_f32(c.k_cal + cal_offset(c, page0, h), lane, cal[i]);
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
// strides of bf16 tensors: whole 8-byte groups, and below 2^31 elements (the kernels multiply them in 32 bits)
static inline bool stride_ok4(long long s) { return (s % 4) == 0 && s >= 0 && s <= 0x7fffffffLL; }

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

// The first-chunk kernel: a cluster of kFirstCtas CTAs per (kv head, entry lane), chained like the others.
static cudaError_t launch_first_chunk(const uint16_t* k, long long k_sn, long long k_sh, const CacheView& view,
                                      const int32_t* cu, int num_entries, const int32_t* cached_lens,
                                      const int32_t* num_decoding, int N, int32_t* status, cudaStream_t s) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(view.Hkv, kFirstLanes, kFirstCtas);
  cfg.blockDim = dim3(kFirstWarps * 32);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = kFirstCtas;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chained_launch_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, first_chunk_k_kernel, k, k_sn, k_sh, view, cu, num_entries, cached_lens, num_decoding, N,
                            status);
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
  const int Hkv = cache->num_kv_heads;
  CacheView view = make_view(cache, table);
  cudaStream_t s = (cudaStream_t)stream;
  launch_chained(prefill_rows_kernel<false>, dim3(N, (2 * Hkv + kWarpsPerBlock - 1) / kWarpsPerBlock), dim3(kWarpsPerBlock * 32), 0, s,
                 (const uint16_t*)nullptr, 0LL, 0LL, (const uint16_t*)k, (long long)k_sn, (long long)k_sh, (const uint16_t*)v,
                 (long long)v_sn, (long long)v_sh, (const uint16_t*)nullptr, (const uint16_t*)nullptr, (const uint16_t*)nullptr,
                 0LL, (const uint16_t*)nullptr, 0LL, (uint16_t*)nullptr, 0LL, 0LL, (uint16_t*)nullptr, 0LL, 0LL, view,
                 cu_seqlens, (int)num_entries, cached_lens, num_decoding, 0, 0.f, status);
  if (cudaGetLastError() != cudaSuccess) return B200KV_E_LAUNCH;
  if (launch_first_chunk((const uint16_t*)k, k_sn, k_sh, view, cu_seqlens, num_entries, cached_lens, num_decoding, N, status,
                         s) != cudaSuccess)
    return B200KV_E_LAUNCH;
  return launch_status();
}

extern "C" int b200kv_write_prefill(const void* q, int64_t q_sn, int64_t q_sh, const void* k, int64_t k_sn, int64_t k_sh,
                                    const void* v, int64_t v_sn, int64_t v_sh, const void* qw, const void* kw,
                                    const void* cosp, int64_t cos_sn, const void* sinp, int64_t sin_sn,
                                    const int32_t* cu_seqlens, int32_t num_entries, const b200kv_cache* cache,
                                    const b200kv_table* table, const int32_t* cached_lens, const int32_t* num_decoding,
                                    void* q_out, int64_t qo_sn, int64_t qo_sh, void* k_out, int64_t ko_sn, int64_t ko_sh,
                                    int32_t N, int32_t Hq, float eps, int32_t* status, void* stream) {
  if (N == 0) return B200KV_OK;
  if (!q || !k || !v || !qw || !kw || !cosp || !sinp || !cu_seqlens || !cached_lens || !num_decoding || !q_out || !k_out)
    return B200KV_E_NULL;
  int rc = check_cache(cache, table);
  if (rc) return rc;
  const int Hkv = cache->num_kv_heads;
  if (N < 0 || num_entries < 1 || Hq < 1 || Hq % Hkv) return B200KV_E_SHAPE;
  if (!aligned(q, 8) || !aligned(k, 8) || !aligned(v, 8) || !aligned(qw, 8) || !aligned(kw, 8) || !aligned(cosp, 8) ||
      !aligned(sinp, 8) || !aligned(q_out, 8) || !aligned(k_out, 8))
    return B200KV_E_ALIGN;
  if (!stride_ok4(q_sn) || !stride_ok4(q_sh) || !stride_ok4(k_sn) || !stride_ok4(k_sh) || !stride_ok4(v_sn) ||
      !stride_ok4(v_sh) || !stride_ok4(cos_sn) || !stride_ok4(sin_sn) || !stride_ok4(qo_sn) || !stride_ok4(qo_sh) ||
      !stride_ok4(ko_sn) || !stride_ok4(ko_sh))
    return B200KV_E_ALIGN;
  CacheView view = make_view(cache, table);
  cudaStream_t s = (cudaStream_t)stream;
  launch_chained(prefill_rows_kernel<true>, dim3(N, (Hq + 2 * Hkv + kWarpsPerBlock - 1) / kWarpsPerBlock),
                 dim3(kWarpsPerBlock * 32), 0, s, (const uint16_t*)q, (long long)q_sn, (long long)q_sh, (const uint16_t*)k,
                 (long long)k_sn, (long long)k_sh, (const uint16_t*)v, (long long)v_sn, (long long)v_sh, (const uint16_t*)qw,
                 (const uint16_t*)kw, (const uint16_t*)cosp, (long long)cos_sn, (const uint16_t*)sinp, (long long)sin_sn,
                 (uint16_t*)q_out, (long long)qo_sn, (long long)qo_sh, (uint16_t*)k_out, (long long)ko_sn, (long long)ko_sh, view,
                 cu_seqlens, (int)num_entries, cached_lens, num_decoding, (int)Hq, eps, status);
  if (cudaGetLastError() != cudaSuccess) return B200KV_E_LAUNCH;
  if (launch_first_chunk((const uint16_t*)k_out, ko_sn, ko_sh, view, cu_seqlens, num_entries, cached_lens, num_decoding, N,
                         status, s) != cudaSuccess)
    return B200KV_E_LAUNCH;
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
