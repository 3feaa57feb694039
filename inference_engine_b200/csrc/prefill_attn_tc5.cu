// Chunked-prefill attention on the 5th-generation tensor cores (tcgen05 + tensor memory).
// Same contract as prefill_attn_kernel (prefill_attn.cu): packed variable-length causal
// attention of the prefilling entries over [dequantized prefix | own chunk], replacing
// prefill_attention_kernel (qwen3-1.7b/kernels.py:987-1126).
//
// One CTA of 128 threads owns 128 query rows of one q head.  Thread t owns row t, which is lane
// t of tensor memory, so every row-wise softmax quantity lives in one thread and needs no
// shuffle.  Per block of 128 keys:
//   S = Q K^T     8 x tcgen05.mma (M128 N128 K16, bf16 -> fp32), Q and K from shared memory,
//                 S in tensor memory columns [0,128)
//   softmax       two passes of tcgen05.ld over the thread's row (max, then exp2 / sum);
//                 P is rounded to bf16 exactly as the reference does (kernels.py:1068,1113)
//                 and stored back into tensor memory over the columns of S it has consumed
//   PV = P V      8 x tcgen05.mma with P read from tensor memory and V from shared memory
//                 (channel-contiguous, i.e. N-major B operand), into columns [128,256)
//   O = O*a + PV  in fp32 registers (one row of 128 channels per thread)
// Q, K and V tiles are laid out in shared memory as the canonical 128-byte-swizzled layout the
// matrix descriptors name: two blocks of 64 channels, each [row][128 bytes] with the 16-byte
// chunk index XOR-ed with (row & 7).  K and V use the same physical layout; only their
// descriptors differ (K: K-major, rows = N; V: N-major, rows = K).  Tiles are filled with
// cp.async; K is refilled as soon as S is complete and V as soon as PV is complete, so the loads
// of the next block run under the softmax of this one.  Two CTAs fit one SM (96 KB of shared
// memory and 256 of the 512 tensor-memory columns each), so one CTA's softmax overlaps the
// other's matrix products.
//
// Every wait on an mbarrier is bounded: if a completion never arrives the CTA records
// B200KV_S_TIMEOUT in the status word, stops issuing work, frees its tensor memory and returns.
#include "common.cuh"

namespace b200kv {

constexpr int kT5Threads = 128;
constexpr int kT5Tile = 128;                        // query rows per CTA = keys per block
constexpr uint32_t kT5TileBytes = kT5Tile * kD * 2; // 32 KB
constexpr uint32_t kT5BlockBytes = kT5Tile * 128;   // one 64-channel block of a tile: 16 KB
constexpr uint32_t kT5Smem = 3 * kT5TileBytes + 1024 /* alignment slack */ + 64 /* barriers, tmem slot */;
constexpr uint32_t kT5Cols = 256;                   // tensor-memory columns: S/P [0,128), PV [128,256)
constexpr uint32_t kT5SpinLimit = 1u << 20;

__device__ __forceinline__ uint32_t t5_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void t5_cp16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void t5_commit_group() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void t5_wait_group() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
__device__ __forceinline__ void t5_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void t5_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void t5_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

__device__ __forceinline__ void t5_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
// Bounded wait for the phase with the given parity; false when the limit ran out.
__device__ __forceinline__ bool t5_mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < kT5SpinLimit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
// Arrive on `bar` when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void t5_mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}

// Shared-memory matrix descriptor: 128-byte swizzle, start address / leading / stride byte offsets
// in units of 16 bytes, descriptor version 1.
__device__ __forceinline__ uint64_t t5_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::f16: fp32 accumulator, bf16 A and B, M = 128, N = 128.
constexpr uint32_t kT5IdescBase = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kT5IdescQK = kT5IdescBase;              // A (Q) K-major, B (K tile) K-major
constexpr uint32_t kT5IdescPV = kT5IdescBase | (1u << 16); // B (V tile) N-major

__device__ __forceinline__ void t5_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void t5_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}

// This thread's lane, 32 consecutive columns starting at taddr's column.
__device__ __forceinline__ void t5_ld32(uint32_t taddr, float (&r)[32]) {
  uint32_t u[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
        "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
        "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]),
        "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) r[i] = __uint_as_float(u[i]);
}
__device__ __forceinline__ void t5_st16(uint32_t taddr, const uint32_t (&u)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
      ::"r"(taddr), "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]), "r"(u[8]),
        "r"(u[9]), "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]) : "memory");
}
__device__ __forceinline__ float t5_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t t5_pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;\n" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// `count` (<= 128) rows of 128 bf16 (row j at src + j*stride elements) into a swizzled tile; rows past
// `count` are zero-filled.
__device__ __forceinline__ void t5_load_tile(uint32_t dst, const uint16_t* src, long long stride, int count, int tid) {
#pragma unroll
  for (int i = 0; i < (kT5Tile * 16) / kT5Threads; ++i) {
    const int c = tid + i * kT5Threads, r = c >> 4, col = c & 15;
    const bool valid = r < count;
    const uint32_t d = dst + (col >> 3) * kT5BlockBytes + r * 128 + (((col & 7) ^ (r & 7)) << 4);
    t5_cp16(d, valid ? src + r * stride + col * 8 : src, valid ? 16 : 0);
  }
}

__global__ void __launch_bounds__(kT5Threads, 2)
prefill_attn_tc5_kernel(const uint16_t* __restrict__ q, long long q_sn, long long q_sh, const uint16_t* __restrict__ k,
                        long long k_sn, long long k_sh, const uint16_t* __restrict__ v, long long v_sn, long long v_sh,
                        const int32_t* __restrict__ seq_ids, const int32_t* __restrict__ cu_seqlens,
                        const int32_t* __restrict__ tile_start, int block_m, int subs,
                        const uint16_t* __restrict__ k_prefix, const uint16_t* __restrict__ v_prefix, long long p_sh,
                        long long p_sn, const int32_t* __restrict__ cu_cached, uint16_t* __restrict__ out, long long o_sn,
                        long long o_sh, int N, int G, float scale_log2, int32_t* status) {
  extern __shared__ uint8_t t5_raw[];
  const int tile = blockIdx.x / subs, sub = blockIdx.x - tile * subs;
  const int tile_row = tile_start[tile];
  if (tile_row < 0 || tile_row >= N) return;
  const int hq = blockIdx.y, hk = hq / G;
  const int seq = seq_ids[tile_row];
  const int prefix_start = cu_cached[seq], prefix_len = cu_cached[seq + 1] - prefix_start;
  const int seq_start = cu_seqlens[seq], seq_end = min(cu_seqlens[seq + 1], N);
  const int row_end = min(tile_row + block_m, seq_end);
  const int row0 = tile_row + sub * kT5Tile;  // first query row of this CTA
  if (row0 >= row_end) return;
  const int cta_last = min(row0 + kT5Tile, row_end) - 1;
  const int own_keys = cta_last - seq_start + 1;  // causal: keys up to the CTA's last query
  const int nb_pre = (prefix_len + kT5Tile - 1) / kT5Tile, nb_own = (own_keys + kT5Tile - 1) / kT5Tile;
  const int nb = nb_pre + nb_own;

  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t base = (t5_smem_u32(t5_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base, sK = base + kT5TileBytes, sV = base + 2 * kT5TileBytes;
  const uint32_t bar_s = base + 3 * kT5TileBytes, bar_o = bar_s + 8, slot = bar_s + 16;

  if (tid == 0) {
    t5_mbar_init(bar_s, 1);
    t5_mbar_init(bar_o, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot), "r"(kT5Cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }

  const uint16_t* kpre = k_prefix + hk * p_sh + (long long)prefix_start * p_sn;
  const uint16_t* vpre = v_prefix + hk * p_sh + (long long)prefix_start * p_sn;
  const uint16_t* kown = k + (long long)seq_start * k_sn + hk * k_sh;
  const uint16_t* vown = v + (long long)seq_start * v_sn + hk * v_sh;
  auto load_keys = [&](uint32_t dst, int kb, bool is_v) {
    if (kb < nb_pre) {
      const int j0 = kb * kT5Tile;
      t5_load_tile(dst, (is_v ? vpre : kpre) + (long long)j0 * p_sn, p_sn, min(kT5Tile, prefix_len - j0), tid);
    } else {
      const int j0 = (kb - nb_pre) * kT5Tile;
      if (is_v) t5_load_tile(dst, vown + (long long)j0 * v_sn, v_sn, min(kT5Tile, own_keys - j0), tid);
      else      t5_load_tile(dst, kown + (long long)j0 * k_sn, k_sn, min(kT5Tile, own_keys - j0), tid);
    }
  };
  // Q rows past the end of the packed batch are zero-filled; rows of other entries inside the tile are
  // read and computed but never stored.
  t5_load_tile(sQ, q + (long long)row0 * q_sn + hq * q_sh, q_sn, min(kT5Tile, N - row0), tid);
  load_keys(sK, 0, false);
  t5_commit_group();
  load_keys(sV, 0, true);
  t5_commit_group();

  t5_fence_before();
  __syncthreads();
  t5_fence_after();
  uint32_t tmem;
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(tmem) : "r"(slot));
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  const uint32_t tS = tmem + lane_base, tO = tmem + lane_base + 128;

  const int my_row = row0 + tid;
  const int my_keys = min(own_keys, my_row - seq_start + 1);  // own-chunk keys this row may see
  float o[kD];
#pragma unroll
  for (int i = 0; i < kD; ++i) o[i] = 0.f;
  float m = -INFINITY, l = 0.f;  // running max of the raw scores, running sum
  bool alive = true;

  for (int kb = 0; kb < nb; ++kb) {
    const uint32_t parity = kb & 1;
    // ---- K block kb has landed (groups in flight: [K kb][V kb])
    t5_wait_group<1>();
    t5_fence_async_smem();
    t5_fence_before();
    __syncthreads();
    if (tid == 0 && alive) {
      t5_fence_after();
#pragma unroll
      for (int j = 0; j < 8; ++j) {  // 16 channels per instruction
        const uint32_t off = (j >> 2) * kT5BlockBytes + (j & 3) * 32;
        t5_mma_ss(tmem, t5_desc(sQ + off, 16, 1024), t5_desc(sK + off, 16, 1024), kT5IdescQK, j > 0);
      }
      t5_mma_commit(bar_s);
    }
    if (alive && !t5_mbar_wait(bar_s, parity)) alive = false;
    alive = __syncthreads_and(alive);
    if (!alive) break;
    t5_fence_after();
    // K is free: refill it for the next block (an empty group keeps the group count uniform)
    if (kb + 1 < nb) load_keys(sK, kb + 1, false);
    t5_commit_group();

    // ---- softmax of this thread's row
    const bool pre = kb < nb_pre;
    const int j0 = pre ? kb * kT5Tile : (kb - nb_pre) * kT5Tile;
    const int lim = (pre ? prefix_len : my_keys) - j0;  // keys [0, lim) of this block are visible
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float s[32];
      t5_ld32(tS + 32 * c, s);
#pragma unroll
      for (int i = 0; i < 32; ++i) mx = fmaxf(mx, 32 * c + i < lim ? s[i] : -INFINITY);
    }
    const float m_new = fmaxf(m, mx);
    const float m_use = m_new == -INFINITY ? 0.f : m_new * scale_log2;  // kernels.py:1062
    const float alpha = t5_exp2(m * scale_log2 - m_use);
    m = m_new;
    float psum = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float s[32];
      t5_ld32(tS + 32 * c, s);
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int kk = 32 * c + 2 * i;
        const float p0 = kk < lim ? t5_exp2(fmaf(s[2 * i], scale_log2, -m_use)) : 0.f;
        const float p1 = kk + 1 < lim ? t5_exp2(fmaf(s[2 * i + 1], scale_log2, -m_use)) : 0.f;
        psum += p0 + p1;
        pk[i] = t5_pack_bf16x2(p0, p1);
      }
      t5_st16(tS + 16 * c, pk);  // P over the columns of S already consumed
    }
    l = l * alpha + psum;
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");

    // ---- V block kb has landed (groups in flight: [V kb][K kb+1]); P is complete
    t5_wait_group<1>();
    t5_fence_async_smem();
    t5_fence_before();
    __syncthreads();
    if (tid == 0) {
      t5_fence_after();
#pragma unroll
      for (int j = 0; j < 8; ++j)  // 16 keys per instruction: 8 columns of packed P, 2 KB of V rows
        t5_mma_ts(tmem + 128, tmem + 8 * j, t5_desc(sV + j * 2048, kT5BlockBytes, 1024), kT5IdescPV, j > 0);
      t5_mma_commit(bar_o);
    }
    if (!t5_mbar_wait(bar_o, parity)) alive = false;
    alive = __syncthreads_and(alive);
    if (!alive) break;
    t5_fence_after();
    if (kb + 1 < nb) load_keys(sV, kb + 1, true);
    t5_commit_group();

    // ---- O = O * alpha + PV
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float pv[32];
      t5_ld32(tO + 32 * c, pv);
#pragma unroll
      for (int i = 0; i < 32; ++i) o[32 * c + i] = fmaf(o[32 * c + i], alpha, pv[i]);
    }
  }
  t5_wait_group<0>();
  if (!alive && tid == 0 && status) atomicOr(status, B200KV_S_TIMEOUT);

  if (alive && my_row < row_end) {
    const float inv = l != 0.f ? 1.f / l : 0.f;  // kernels.py:1118
    uint4* dst = reinterpret_cast<uint4*>(out + (long long)my_row * o_sn + hq * o_sh);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      uint4 w;
      w.x = t5_pack_bf16x2(o[8 * i] * inv, o[8 * i + 1] * inv);
      w.y = t5_pack_bf16x2(o[8 * i + 2] * inv, o[8 * i + 3] * inv);
      w.z = t5_pack_bf16x2(o[8 * i + 4] * inv, o[8 * i + 5] * inv);
      w.w = t5_pack_bf16x2(o[8 * i + 6] * inv, o[8 * i + 7] * inv);
      dst[i] = w;
    }
  }
  t5_fence_before();
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kT5Cols) : "memory");
}

int launch_prefill_attn_tc5(const uint16_t* q, long long q_sn, long long q_sh, const uint16_t* k, long long k_sn,
                            long long k_sh, const uint16_t* v, long long v_sn, long long v_sh, const int32_t* seq_ids,
                            const int32_t* cu_seqlens, const int32_t* tile_start, int num_tiles, int block_m,
                            const uint16_t* k_prefix, const uint16_t* v_prefix, long long p_sh, long long p_sn,
                            const int32_t* cu_cached, uint16_t* out, long long o_sn, long long o_sh, int N, int Hq,
                            int Hkv, float scale_log2, int32_t* status, cudaStream_t stream) {
  // the opt-in is a per-device attribute of the function: set it on every call (it is cheap)
  if (cudaFuncSetAttribute(prefill_attn_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kT5Smem) !=
      cudaSuccess)
    return B200KV_E_LAUNCH;
  const int subs = (block_m + kT5Tile - 1) / kT5Tile;
  prefill_attn_tc5_kernel<<<dim3(num_tiles * subs, Hq), kT5Threads, kT5Smem, stream>>>(
      q, q_sn, q_sh, k, k_sn, k_sh, v, v_sn, v_sh, seq_ids, cu_seqlens, tile_start, block_m, subs, k_prefix, v_prefix, p_sh,
      p_sn, cu_cached, out, o_sn, o_sh, N, Hq / Hkv, scale_log2, status);
  return cudaGetLastError() == cudaSuccess ? B200KV_OK : B200KV_E_LAUNCH;
}

}  // namespace b200kv
