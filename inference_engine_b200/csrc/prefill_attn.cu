// Packed variable-length causal attention for prefilling entries (chunked prefill): every query
// row of an entry's chunk attends the entry's dequantized prefix (bf16, in full) and the rows of
// its own chunk up to itself.  Replaces prefill_attention_kernel (qwen3-1.7b/kernels.py:987-1126).
//
// Tensor-core flash attention: a CTA of 4 warps owns 64 query rows of one q head (a 128-row tile
// of the caller is two such CTAs); each warp owns 16 rows.  Keys are consumed 64 at a time from
// a double-buffered shared-memory ring filled with 16-byte cp.async copies (rows padded to 272
// bytes so that ldmatrix reads are conflict-free).  S = Q K^T and O += P V run as bf16
// mma.m16n8k16 with fp32 accumulation; K fragments come from ldmatrix, V fragments from
// ldmatrix.trans; P is rounded to bf16 before P.V exactly as the reference does
// (kernels.py:1068,1113); softmax in fp32 registers with exp2 and log2(e) folded into the scale
// (kernels.py:1167-1168).  The score accumulator layout of one k16 slice is the A-fragment layout
// of the second product, so P never leaves registers.
#include "common.cuh"

namespace b200kv {

constexpr int kPfWarps = 4;
constexpr int kPfRows = 16 * kPfWarps;   // query rows per CTA
constexpr int kPfKeys = 64;              // keys per block
constexpr int kPfRowBytes = kD * 2 + 16; // 272: padded bf16 row
constexpr int kPfTileBytes = kPfKeys * kPfRowBytes;

__device__ __forceinline__ uint32_t pf_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void pf_cp16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void pf_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void pf_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float pf_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  return float_to_bf16_bits(lo) | (float_to_bf16_bits(hi) << 16);
}

// Copy `count` (<= 64) key rows of 128 bf16 (row j at src + j*stride elements) into a padded
// tile; rows past `count` are zero-filled.
__device__ __forceinline__ void load_tile(uint32_t dst, const uint16_t* src, long long stride, int count, int tid) {
#pragma unroll
  for (int i = 0; i < (kPfKeys * 16) / (kPfWarps * 32); ++i) {
    const int c = tid + i * kPfWarps * 32, r = c >> 4, col = c & 15;
    const bool valid = r < count;
    pf_cp16(dst + r * kPfRowBytes + col * 16, valid ? src + r * stride + col * 8 : src, valid ? 16 : 0);
  }
}

__global__ void __launch_bounds__(kPfWarps * 32)
prefill_attn_kernel(const uint16_t* __restrict__ q, long long q_sn, long long q_sh, const uint16_t* __restrict__ k,
                    long long k_sn, long long k_sh, const uint16_t* __restrict__ v, long long v_sn, long long v_sh,
                    const int32_t* __restrict__ seq_ids, const int32_t* __restrict__ cu_seqlens,
                    const int32_t* __restrict__ tile_start, int block_m, int subs, const uint16_t* __restrict__ k_prefix,
                    const uint16_t* __restrict__ v_prefix, long long p_sh, long long p_sn,
                    const int32_t* __restrict__ cu_cached, uint16_t* __restrict__ out, long long o_sn, long long o_sh,
                    int N, int G, float scale_log2) {
  extern __shared__ __align__(128) uint8_t pf_smem[];
  pdl_enter();
  // heads run fastest in the grid: the caller's real tiles come first in tile_start, so every CTA with work
  // is dispatched before the idle ones behind them
  const int tile = blockIdx.y / subs, sub = blockIdx.y - tile * subs;
  const int tile_row = tile_start[tile];
  if (tile_row < 0 || tile_row >= N) return;
  const int hq = blockIdx.x, hk = hq / G;
  const int seq = seq_ids[tile_row];
  // a step in which no entry has a cached prefix may pass empty prefix tensors (no storage: NULL pointers)
  const int prefix_start = cu_cached[seq], prefix_len = (k_prefix && v_prefix) ? cu_cached[seq + 1] - prefix_start : 0;
  const int seq_start = cu_seqlens[seq], seq_end = min(cu_seqlens[seq + 1], N);
  const int row_end = min(tile_row + block_m, seq_end);
  const int row0 = tile_row + sub * kPfRows;  // first query row of this CTA
  if (row0 >= row_end) return;
  const int cta_last = min(row0 + kPfRows, row_end) - 1;  // last query row of this CTA
  const int own_keys = cta_last - seq_start + 1;          // causal: keys up to the last query
  const int nb_pre = (prefix_len + kPfKeys - 1) / kPfKeys, nb_own = (own_keys + kPfKeys - 1) / kPfKeys;
  const int nb = nb_pre + nb_own;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const uint32_t smem0 = pf_smem_u32(pf_smem);
  pdl_wait();  // q, k, v and the prefix come from the kernels before this one; only metadata was read so far
  const uint16_t* kpre = k_prefix + hk * p_sh + (long long)prefix_start * p_sn;
  const uint16_t* vpre = v_prefix + hk * p_sh + (long long)prefix_start * p_sn;
  const uint16_t* kown = k + (long long)seq_start * k_sn + hk * k_sh;
  const uint16_t* vown = v + (long long)seq_start * v_sn + hk * v_sh;

  auto issue = [&](int kb) {
    const uint32_t sk = smem0 + (kb & 1) * 2 * kPfTileBytes, sv = sk + kPfTileBytes;
    if (kb < nb_pre) {
      const int j0 = kb * kPfKeys, cnt = min(kPfKeys, prefix_len - j0);
      load_tile(sk, kpre + (long long)j0 * p_sn, p_sn, cnt, tid);
      load_tile(sv, vpre + (long long)j0 * p_sn, p_sn, cnt, tid);
    } else {
      const int j0 = (kb - nb_pre) * kPfKeys, cnt = min(kPfKeys, own_keys - j0);
      load_tile(sk, kown + (long long)j0 * k_sn, k_sn, cnt, tid);
      load_tile(sv, vown + (long long)j0 * v_sn, v_sn, cnt, tid);
    }
    pf_commit();
  };
  issue(0);

  // Q fragments of this warp's 16 rows (rows past the end are read from a valid row and never stored)
  const int qr0 = row0 + warp * 16 + g, qr1 = qr0 + 8;
  const uint16_t* q0 = q + (long long)min(qr0, row_end - 1) * q_sn + hq * q_sh;
  const uint16_t* q1 = q + (long long)min(qr1, row_end - 1) * q_sn + hq * q_sh;
  uint32_t qa[8][4];
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    qa[s][0] = *reinterpret_cast<const uint32_t*>(q0 + 16 * s + 2 * t);
    qa[s][1] = *reinterpret_cast<const uint32_t*>(q1 + 16 * s + 2 * t);
    qa[s][2] = *reinterpret_cast<const uint32_t*>(q0 + 16 * s + 8 + 2 * t);
    qa[s][3] = *reinterpret_cast<const uint32_t*>(q1 + 16 * s + 8 + 2 * t);
  }
  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows g and g+8 (l: this lane's share)
  // ldmatrix lane addressing inside a tile (see the fragment notes at the top of the file)
  const uint32_t k_lane = ((lane >> 4) * 8 + (lane & 7)) * kPfRowBytes + ((lane >> 3) & 1) * 16;
  const uint32_t v_lane = (((lane >> 3) & 1) * 8 + (lane & 7)) * kPfRowBytes + (lane >> 4) * 16;

  for (int kb = 0; kb < nb; ++kb) {
    if (kb + 1 < nb) { issue(kb + 1); pf_wait<1>(); } else { pf_wait<0>(); }
    __syncthreads();
    const uint32_t sk = smem0 + (kb & 1) * 2 * kPfTileBytes, sv = sk + kPfTileBytes;
    // ---- S = Q K^T for 64 keys: 8 n-tiles of 8 keys
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {     // 16 channels per step
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {   // 16 keys per ldmatrix.x4
        uint32_t b[4];
        ldsm_x4(b, sk + k_lane + jp * 16 * kPfRowBytes + ks * 32);
        mma_bf16(s[2 * jp], qa[ks], b[0], b[1]);
        mma_bf16(s[2 * jp + 1], qa[ks], b[2], b[3]);
      }
    }
    // ---- mask + online softmax.  s[j][0..1]: row g, keys 8j+2t, +1;  s[j][2..3]: row g+8
    const bool pre = kb < nb_pre;
    const int j0 = pre ? kb * kPfKeys : (kb - nb_pre) * kPfKeys;
    // visible key count per row inside this block
    const int lim0 = pre ? prefix_len - j0 : min(own_keys, qr0 - seq_start + 1) - j0;
    const int lim1 = pre ? prefix_len - j0 : min(own_keys, qr1 - seq_start + 1) - j0;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int kk = 8 * j + 2 * t;
      s[j][0] = kk < lim0 ? s[j][0] * scale_log2 : -INFINITY;
      s[j][1] = kk + 1 < lim0 ? s[j][1] * scale_log2 : -INFINITY;
      s[j][2] = kk < lim1 ? s[j][2] * scale_log2 : -INFINITY;
      s[j][3] = kk + 1 < lim1 ? s[j][3] * scale_log2 : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
      mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float sm0 = mn0 == -INFINITY ? 0.f : mn0, sm1 = mn1 == -INFINITY ? 0.f : mn1;  // kernels.py:1062
    const float al0 = pf_exp2(m0 - sm0), al1 = pf_exp2(m1 - sm1);
    m0 = mn0; m1 = mn1;
    uint32_t pa[4][4];  // P as A fragments of the 4 k16 slices
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p0 = pf_exp2(s[j][0] - sm0), p1 = pf_exp2(s[j][1] - sm0);
      const float p2 = pf_exp2(s[j][2] - sm1), p3 = pf_exp2(s[j][3] - sm1);
      ps0 += p0 + p1; ps1 += p2 + p3;
      pa[j >> 1][(j & 1) * 2] = pack_bf16x2(p0, p1);      // a0 / a2: row g
      pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16x2(p2, p3);  // a1 / a3: row g+8
    }
    l0 = l0 * al0 + ps0; l1 = l1 * al1 + ps1;
#pragma unroll
    for (int j = 0; j < 16; ++j) { o[j][0] *= al0; o[j][1] *= al0; o[j][2] *= al1; o[j][3] *= al1; }
    // ---- O += P V: 4 k16 slices of keys x 16 n-tiles of 8 channels
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {   // 16 channels per ldmatrix.x4.trans
        uint32_t b[4];
        ldsm_x4_trans(b, sv + v_lane + kk * 16 * kPfRowBytes + dp * 32);
        mma_bf16(o[2 * dp], pa[kk], b[0], b[1]);
        mma_bf16(o[2 * dp + 1], pa[kk], b[2], b[3]);
      }
    }
    __syncthreads();  // everyone is done with this stage before it is refilled
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = l0 != 0.f ? 1.f / l0 : 0.f, i1 = l1 != 0.f ? 1.f / l1 : 0.f;  // kernels.py:1118
  if (qr0 < row_end) {
    uint16_t* dst = out + (long long)qr0 * o_sn + hq * o_sh + 2 * t;
#pragma unroll
    for (int j = 0; j < 16; ++j) *reinterpret_cast<uint32_t*>(dst + 8 * j) = pack_bf16x2(o[j][0] * i0, o[j][1] * i0);
  }
  if (qr1 < row_end) {
    uint16_t* dst = out + (long long)qr1 * o_sn + hq * o_sh + 2 * t;
#pragma unroll
    for (int j = 0; j < 16; ++j) *reinterpret_cast<uint32_t*>(dst + 8 * j) = pack_bf16x2(o[j][2] * i1, o[j][3] * i1);
  }
}

}  // namespace b200kv

using namespace b200kv;

namespace b200kv {
int launch_prefill_attn_tc5(const uint16_t* q, long long q_sn, long long q_sh, const uint16_t* k, long long k_sn,
                            long long k_sh, const uint16_t* v, long long v_sn, long long v_sh, const int32_t* seq_ids,
                            const int32_t* cu_seqlens, const int32_t* tile_start, int num_tiles, int block_m,
                            const uint16_t* k_prefix, const uint16_t* v_prefix, long long p_sh, long long p_sn,
                            int prefix_rows, const int32_t* cu_cached, uint16_t* out, long long o_sn, long long o_sh, int N,
                            int Hq, int Hkv, float scale_log2, int32_t* status, int idle_issuers, cudaStream_t stream);
}

extern "C" int b200kv_prefill_attn_variant(const void* q, int64_t q_sn, int64_t q_sh, const void* k, int64_t k_sn,
                                           int64_t k_sh, const void* v, int64_t v_sn, int64_t v_sh, const int32_t* seq_ids,
                                           const int32_t* cu_seqlens, const int32_t* tile_start, int32_t num_tiles,
                                           int32_t block_m, const void* k_prefix, const void* v_prefix, int64_t p_sh,
                                           int64_t p_sn, int32_t prefix_rows, const int32_t* cu_cached, void* out,
                                           int64_t o_sn, int64_t o_sh, int32_t N, int32_t Hq, int32_t Hkv, int32_t D,
                                           int32_t variant, int32_t* status, void* stream) {
  // an empty batch is valid and has nothing to launch (its tensors have no storage, so their pointers are NULL)
  if (N == 0 || num_tiles == 0) return B200KV_OK;
  // k_prefix / v_prefix may be NULL (empty tensors): the step then has no cached prefix to attend
  if (!q || !k || !v || !seq_ids || !cu_seqlens || !tile_start || !cu_cached || !out) return B200KV_E_NULL;
  if (!k_prefix || !v_prefix) prefix_rows = 0;
  if (D != kD || Hq < 1 || Hkv < 1 || Hq % Hkv || N < 0 || num_tiles < 0 || block_m < 1 || prefix_rows < 0)
    return B200KV_E_SHAPE;
  if (variant < 0 || variant > 3) return B200KV_E_RANGE;
  if (!aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16) || !aligned(k_prefix, 16) || !aligned(v_prefix, 16) ||
      !aligned(out, 16))
    return B200KV_E_ALIGN;
  const int64_t strides[] = {q_sn, q_sh, k_sn, k_sh, v_sn, v_sh, p_sh, p_sn, o_sn, o_sh};
  for (int64_t s : strides)
    if (s % 8) return B200KV_E_ALIGN;
  if (N == 0 || num_tiles == 0) return B200KV_OK;
  if ((long long)num_tiles * ((block_m + kPfRows - 1) / kPfRows) > 65535) return B200KV_E_RANGE;  // grid.y
  const float scale_log2 = (1.0f / sqrtf((float)D)) * 1.4426950408889634f;
  // Query tiles of at least 64 rows fill a 128-row tcgen05 tile well enough to pay; smaller ones stay
  // on the 64-row mma.sync kernel.
  const bool tc5 = variant >= 2 || (variant == 0 && block_m >= 64);
  if (tc5)
    return launch_prefill_attn_tc5((const uint16_t*)q, q_sn, q_sh, (const uint16_t*)k, k_sn, k_sh, (const uint16_t*)v, v_sn,
                                   v_sh, seq_ids, cu_seqlens, tile_start, num_tiles, block_m, (const uint16_t*)k_prefix,
                                   (const uint16_t*)v_prefix, p_sh, p_sn, prefix_rows, cu_cached, (uint16_t*)out, o_sn, o_sh, N,
                                   Hq, Hkv, scale_log2, status, variant == 3 ? 1 : 0, (cudaStream_t)stream);
  const int subs = (block_m + kPfRows - 1) / kPfRows;
  const size_t smem = 4 * (size_t)kPfTileBytes;
  if (cudaFuncSetAttribute(prefill_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return B200KV_E_LAUNCH;
  launch_chained(prefill_attn_kernel, dim3(Hq, num_tiles * subs), dim3(kPfWarps * 32), smem, (cudaStream_t)stream,
      (const uint16_t*)q, q_sn, q_sh, (const uint16_t*)k, k_sn, k_sh, (const uint16_t*)v, v_sn, v_sh, seq_ids, cu_seqlens,
      tile_start, block_m, subs, (const uint16_t*)k_prefix, (const uint16_t*)v_prefix, p_sh, p_sn, cu_cached,
      (uint16_t*)out, o_sn, o_sh, N, Hq / Hkv, scale_log2);
  return cudaGetLastError() == cudaSuccess ? B200KV_OK : B200KV_E_LAUNCH;
}

extern "C" int b200kv_prefill_attn(const void* q, int64_t q_sn, int64_t q_sh, const void* k, int64_t k_sn, int64_t k_sh,
                                   const void* v, int64_t v_sn, int64_t v_sh, const int32_t* seq_ids,
                                   const int32_t* cu_seqlens, const int32_t* tile_start, int32_t num_tiles, int32_t block_m,
                                   const void* k_prefix, const void* v_prefix, int64_t p_sh, int64_t p_sn,
                                   const int32_t* cu_cached, void* out, int64_t o_sn, int64_t o_sh, int32_t N, int32_t Hq,
                                   int32_t Hkv, int32_t D, void* stream) {
  // no row count in this signature: 0 = unknown (the tcgen05 kernel then copies prefix tiles with cp.async)
  return b200kv_prefill_attn_variant(q, q_sn, q_sh, k, k_sn, k_sh, v, v_sn, v_sh, seq_ids, cu_seqlens, tile_start, num_tiles,
                                     block_m, k_prefix, v_prefix, p_sh, p_sn, 0, cu_cached, out, o_sn, o_sh, N, Hq, Hkv, D, 0,
                                     nullptr, stream);
}
