// Packed variable-length causal attention for prefilling entries (chunked prefill):
// every query row of an entry's chunk attends the entry's dequantized prefix (bf16, in full)
// and the rows of its own chunk up to itself.  Replaces prefill_attention_kernel
// (qwen3-1.7b/kernels.py:987-1126).
//
// This first version is a straightforward CUDA-core kernel (fp32 FMAs, one warp per query row):
// grid (num_tiles, Hq), 4 warps; warp w takes rows w, w+4, ... of its tile.  Keys are consumed
// 32 at a time: each lane scores one key (q broadcast from shared memory), the warp does the
// online-softmax update, then accumulates P.V with lane l owning channels 4l..4l+3.
#include "common.cuh"

namespace b200kv {

constexpr int kPfWarps = 4;

__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct KeySource {
  const uint16_t* k;
  const uint16_t* v;
  long long k_stride, v_stride;  // elements between consecutive keys
};

// Consume keys [0, count) of `src` (key j's row at base + j*stride); keys j > limit are masked.
__device__ __forceinline__ void consume(const KeySource& src, int count, int limit, const float* q_s, float scale_log2,
                                        float& m, float& l, float (&acc)[4], int lane) {
  for (int base = 0; base < count; base += 32) {
    const int j = base + lane;
    const bool live = j < count && j <= limit;
    float s = -INFINITY;
    if (live) {
      const uint4* row = reinterpret_cast<const uint4*>(src.k + j * src.k_stride);
      float dot = 0.f;
#pragma unroll 4
      for (int c = 0; c < 16; ++c) {
        uint4 raw = row[c];
        uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          dot = fmaf(q_s[8 * c + 2 * i], bf16_bits_to_float(w[i] & 0xFFFFu), dot);
          dot = fmaf(q_s[8 * c + 2 * i + 1], bf16_bits_to_float(w[i] >> 16), dot);
        }
      }
      s = dot * scale_log2;
    }
    const float mx = warp_max_f(s);
    if (mx == -INFINITY) continue;  // every key of this group is masked (warp-uniform)
    const float m_new = fmaxf(m, mx);
    const float alpha = exp2f(m - m_new);
    // the reference rounds P to bf16 before P.V (kernels.py:1068,1113); keep fp32 here (closer to exact)
    const float p = live ? exp2f(s - m_new) : 0.f;
    l = l * alpha + warp_sum_f(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] *= alpha;
    const int nk = min(32, count - base);
    for (int jj = 0; jj < nk; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      if (pj == 0.f) continue;
      uint2 raw = *reinterpret_cast<const uint2*>(src.v + (long long)(base + jj) * src.v_stride + 4 * lane);
      acc[0] = fmaf(pj, bf16_bits_to_float(raw.x & 0xFFFFu), acc[0]);
      acc[1] = fmaf(pj, bf16_bits_to_float(raw.x >> 16), acc[1]);
      acc[2] = fmaf(pj, bf16_bits_to_float(raw.y & 0xFFFFu), acc[2]);
      acc[3] = fmaf(pj, bf16_bits_to_float(raw.y >> 16), acc[3]);
    }
  }
}

__global__ void __launch_bounds__(kPfWarps * 32)
prefill_attn_kernel(const uint16_t* __restrict__ q, long long q_sn, long long q_sh, const uint16_t* __restrict__ k,
                    long long k_sn, long long k_sh, const uint16_t* __restrict__ v, long long v_sn, long long v_sh,
                    const int32_t* __restrict__ seq_ids, const int32_t* __restrict__ cu_seqlens,
                    const int32_t* __restrict__ tile_start, int block_m, const uint16_t* __restrict__ k_prefix,
                    const uint16_t* __restrict__ v_prefix, long long p_sh, long long p_sn,
                    const int32_t* __restrict__ cu_cached, uint16_t* __restrict__ out, long long o_sn, long long o_sh,
                    int N, int G, float scale_log2) {
  __shared__ __align__(16) float q_all[kPfWarps][kD];
  const int row_start = tile_start[blockIdx.x];
  if (row_start < 0 || row_start >= N) return;
  const int hq = blockIdx.y, hk = hq / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = seq_ids[row_start];
  const int prefix_start = cu_cached[seq], prefix_len = cu_cached[seq + 1] - prefix_start;
  const int seq_start = cu_seqlens[seq], seq_end = min(cu_seqlens[seq + 1], N);
  const int row_end = min(row_start + block_m, seq_end);
  float* q_s = q_all[warp];
  KeySource pre{k_prefix + hk * p_sh + (long long)prefix_start * p_sn, v_prefix + hk * p_sh + (long long)prefix_start * p_sn, p_sn, p_sn};
  KeySource own{k + (long long)seq_start * k_sn + hk * k_sh, v + (long long)seq_start * v_sn + hk * v_sh, k_sn, v_sn};
  for (int r = row_start + warp; r < row_end; r += kPfWarps) {
    __syncwarp();
    {
      uint2 raw = *reinterpret_cast<const uint2*>(q + r * q_sn + hq * q_sh + 4 * lane);
      q_s[4 * lane] = bf16_bits_to_float(raw.x & 0xFFFFu);
      q_s[4 * lane + 1] = bf16_bits_to_float(raw.x >> 16);
      q_s[4 * lane + 2] = bf16_bits_to_float(raw.y & 0xFFFFu);
      q_s[4 * lane + 3] = bf16_bits_to_float(raw.y >> 16);
    }
    __syncwarp();
    float m = -INFINITY, l = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
    consume(pre, prefix_len, prefix_len, q_s, scale_log2, m, l, acc, lane);
    consume(own, r - seq_start + 1, r - seq_start, q_s, scale_log2, m, l, acc, lane);
    const float inv = l != 0.f ? 1.f / l : 0.f;
    uint2 w;
    w.x = float_to_bf16_bits(acc[0] * inv) | (float_to_bf16_bits(acc[1] * inv) << 16);
    w.y = float_to_bf16_bits(acc[2] * inv) | (float_to_bf16_bits(acc[3] * inv) << 16);
    *reinterpret_cast<uint2*>(out + r * o_sn + hq * o_sh + 4 * lane) = w;
  }
}

}  // namespace b200kv

using namespace b200kv;

extern "C" int b200kv_prefill_attn(const void* q, int64_t q_sn, int64_t q_sh, const void* k, int64_t k_sn, int64_t k_sh,
                                   const void* v, int64_t v_sn, int64_t v_sh, const int32_t* seq_ids,
                                   const int32_t* cu_seqlens, const int32_t* tile_start, int32_t num_tiles, int32_t block_m,
                                   const void* k_prefix, const void* v_prefix, int64_t p_sh, int64_t p_sn,
                                   const int32_t* cu_cached, void* out, int64_t o_sn, int64_t o_sh, int32_t N, int32_t Hq,
                                   int32_t Hkv, int32_t D, void* stream) {
  if (!q || !k || !v || !seq_ids || !cu_seqlens || !tile_start || !k_prefix || !v_prefix || !cu_cached || !out)
    return B200KV_E_NULL;
  if (D != kD || Hq < 1 || Hkv < 1 || Hq % Hkv || N < 0 || num_tiles < 0 || block_m < 1) return B200KV_E_SHAPE;
  if (!aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16) || !aligned(k_prefix, 16) || !aligned(v_prefix, 16) ||
      !aligned(out, 16))
    return B200KV_E_ALIGN;
  const int64_t strides[] = {q_sn, q_sh, k_sn, k_sh, v_sn, v_sh, p_sh, p_sn, o_sn, o_sh};
  for (int64_t s : strides)
    if (s % 8) return B200KV_E_ALIGN;
  if (N == 0 || num_tiles == 0) return B200KV_OK;
  const float scale_log2 = (1.0f / sqrtf((float)D)) * 1.4426950408889634f;
  prefill_attn_kernel<<<dim3(num_tiles, Hq), kPfWarps * 32, 0, (cudaStream_t)stream>>>(
      (const uint16_t*)q, q_sn, q_sh, (const uint16_t*)k, k_sn, k_sh, (const uint16_t*)v, v_sn, v_sh, seq_ids, cu_seqlens,
      tile_start, block_m, (const uint16_t*)k_prefix, (const uint16_t*)v_prefix, p_sh, p_sn, cu_cached, (uint16_t*)out,
      o_sn, o_sh, N, Hq / Hkv, scale_log2);
  return cudaGetLastError() == cudaSuccess ? B200KV_OK : B200KV_E_LAUNCH;
}
