// Chunked-prefill attention on the 5th-generation tensor cores (tcgen05 + tensor memory).
// Same contract as prefill_attn_kernel (prefill_attn.cu): packed variable-length causal
// attention of the prefilling entries over [dequantized prefix | own chunk], replacing
// prefill_attention_kernel (qwen3-1.7b/kernels.py:987-1126).
//
// One CTA owns 128 query rows of one q head and runs two warpgroups of 128 threads.  The key
// blocks (128 keys each) of the tile are dealt alternately to the two warpgroups; each keeps its
// own running (max, sum, O) and the two are merged at the end, so while one warpgroup is in its
// softmax the tensor core works for the other.  Inside a warpgroup, thread t owns query row t =
// lane t of tensor memory: every row-wise softmax quantity lives in one thread, no shuffles.
// Per key block of a warpgroup:
//   S = Q K^T     8 x tcgen05.mma (M128 N128 K16, bf16 -> fp32), Q and K from shared memory,
//                 S in the warpgroup's tensor-memory columns [0,128)
//   softmax       one tcgen05.ld of the thread's 128 scores, max, exp2, sum; P rounded to bf16 as
//                 the reference does (kernels.py:1068,1113) and stored over the first 64 columns of S
//   O += P V      8 x tcgen05.mma with P read from tensor memory and V from shared memory
//                 (channel-contiguous: N-major B operand), accumulating in columns [128,256)
// O stays in tensor memory for the whole tile.  Its rescaling is lazy: the reference offset of the
// exponentials only moves when the row maximum has grown by more than 2^8 since it was set (then O
// and the sum are multiplied by the correction, a tensor-memory round trip); otherwise P is simply
// computed against the older offset, which is the same mathematics.  The product S of the next
// block is issued right behind P V of this one, so the tensor core never waits for the softmax
// threads of its own warpgroup to come back.
//
// Q, K and V tiles are laid out in shared memory as the canonical 128-byte-swizzled layout the
// matrix descriptors name: two blocks of 64 channels, each [row][128 bytes] with the 16-byte
// chunk index XOR-ed with (row & 7).  K and V use the same physical layout; only their
// descriptors differ (K: K-major, rows = N; V: N-major, rows = K).  Each warpgroup fills its own
// tiles with cp.async (one K tile, two V tiles; rows past the visible range are zero-filled, so
// uninitialised memory behind a prefix never reaches the tensor core).  The tensor core executes
// one thread's products in issue order, so the completion of S of block i also means that P V of
// block i-1 is complete: at that one wait per block the K tile and the other V tile are free and
// block i+1 is fetched into them, under the softmax of block i.
//
// Every wait on an mbarrier is bounded: if a completion never arrives the warpgroup records
// B200KV_S_TIMEOUT in the status word, stops issuing work and skips its stores; the CTA still
// frees its tensor memory and returns.
#include "common.cuh"
#include "tmem_ldst.cuh"

namespace b200kv {

constexpr int kT5Threads = 256;
constexpr int kT5Tile = 128;                        // query rows per CTA = keys per block
constexpr uint32_t kT5TileBytes = kT5Tile * kD * 2; // 32 KB
constexpr uint32_t kT5BlockBytes = kT5Tile * 128;   // one 64-channel block of a tile: 16 KB
constexpr uint32_t kT5WgBytes = 3 * kT5TileBytes;   // per warpgroup: K, V0, V1
constexpr uint32_t kT5Smem = kT5TileBytes + 2 * kT5WgBytes + 1024 /* alignment slack */ + 64 /* barriers, flags */;
constexpr uint32_t kT5Cols = 512;                   // tensor memory: warpgroup w has S/P at 256w, O at 256w+128
constexpr uint32_t kT5SpinLimit = 1u << 20;
constexpr float kT5Lazy = 8.f;                      // log2 of the growth of the row maximum that forces a rescale

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

// Copied by kThreads threads (tid in [0, kThreads)): `count` (<= 128) rows of 128 bf16 (row j at src + j*stride elements) into a swizzled tile; rows past
// `count` are zero-filled.
template <int kThreads>
__device__ __forceinline__ void t5_load_tile(uint32_t dst, const uint16_t* src, long long stride, int count, int tid) {
#pragma unroll
  for (int i = 0; i < (kT5Tile * 16) / kThreads; ++i) {
    const int c = tid + i * kThreads, r = c >> 4, col = c & 15;
    const bool valid = r < count;
    const uint32_t d = dst + (col >> 3) * kT5BlockBytes + r * 128 + (((col & 7) ^ (r & 7)) << 4);
    t5_cp16(d, valid ? src + r * stride + col * 8 : src, valid ? 16 : 0);
  }
}


__device__ __forceinline__ void t5_wg_sync(int wg) { asm volatile("bar.sync %0, 128;\n" ::"r"(wg + 1) : "memory"); }

__global__ void __launch_bounds__(kT5Threads, 1)
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

  const int tid = threadIdx.x, wg = tid >> 7, wt = tid & 127;
  const int n_mine = (nb - wg + 1) >> 1;  // this warpgroup's blocks: wg, wg + 2, ...
  const uint32_t base = (t5_smem_u32(t5_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base;
  const uint32_t sK = base + kT5TileBytes + wg * kT5WgBytes;  // one K tile, then two V tiles
  const uint32_t sV = sK + kT5TileBytes;
  const uint32_t bars = base + kT5TileBytes + 2 * kT5WgBytes;
  const uint32_t bar_s = bars + wg * 16, bar_o = bar_s + 8, slot = bars + 32, dead_flag = bars + 40 + wg * 4;

  if (tid == 0) {
    for (int i = 0; i < 4; ++i) t5_mbar_init(bars + 8 * i, 1);
    asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(bars + 40), "r"(0) : "memory");
    asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(bars + 44), "r"(0) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (tid < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot), "r"(kT5Cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }

  const uint16_t* kpre = k_prefix + hk * p_sh + (long long)prefix_start * p_sn;
  const uint16_t* vpre = v_prefix + hk * p_sh + (long long)prefix_start * p_sn;
  const uint16_t* kown = k + (long long)seq_start * k_sn + hk * k_sh;
  const uint16_t* vown = v + (long long)seq_start * v_sn + hk * v_sh;
  // this warpgroup's i-th block is block wg + 2i of the tile
  auto load_keys = [&](uint32_t dst, int i, bool is_v) {
    const int kb = wg + 2 * i;
    if (kb < nb_pre) {
      const int j0 = kb * kT5Tile;
      t5_load_tile<128>(dst, (is_v ? vpre : kpre) + (long long)j0 * p_sn, p_sn, min(kT5Tile, prefix_len - j0), wt);
    } else {
      const int j0 = (kb - nb_pre) * kT5Tile;
      if (is_v) t5_load_tile<128>(dst, vown + (long long)j0 * v_sn, v_sn, min(kT5Tile, own_keys - j0), wt);
      else      t5_load_tile<128>(dst, kown + (long long)j0 * k_sn, k_sn, min(kT5Tile, own_keys - j0), wt);
    }
  };
  // Q rows past the end of the packed batch are zero-filled; rows of other entries inside the tile are
  // read and computed but never stored.
  t5_load_tile<256>(sQ, q + (long long)row0 * q_sn + hq * q_sh, q_sn, min(kT5Tile, N - row0), tid);
  if (n_mine > 0) { load_keys(sK, 0, false); load_keys(sV, 0, true); }
  t5_commit_group();
  t5_wait_group<0>();
  t5_fence_async_smem();
  t5_fence_before();
  __syncthreads();
  t5_fence_after();
  uint32_t tmem;
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(tmem) : "r"(slot));
  const uint32_t tS_all = tmem + 256 * wg, tO_all = tS_all + 128;  // lane 0: what the MMA is given
  const uint32_t lane_base = (uint32_t)(((tid >> 5) & 3) * 32) << 16;
  const uint32_t tS = tS_all + lane_base, tO = tO_all + lane_base;  // this thread's lane

  auto issue_s = [&]() {  // S = Q K^T of the block in the K tile
#pragma unroll
    for (int j = 0; j < 8; ++j) {  // 16 channels per instruction
      const uint32_t off = (j >> 2) * kT5BlockBytes + (j & 3) * 32;
      t5_mma_ss(tS_all, t5_desc(sQ + off, 16, 1024), t5_desc(sK + off, 16, 1024), kT5IdescQK, j > 0);
    }
    t5_mma_commit(bar_s);
  };
  if (wt == 0 && n_mine > 0) issue_s();

  const int my_row = row0 + wt;
  const int my_keys = min(own_keys, my_row - seq_start + 1);  // own-chunk keys this row may see
  const int first_keys = row0 - seq_start + 1;                // ... and the tile's first row
  float m_ref = -INFINITY, l = 0.f;  // offset of the exponentials (log2 units, scaled), running sum
  bool dead = false;

  for (int i = 0; i < n_mine; ++i) {
    const uint32_t parity = i & 1;
    // S of block i is complete, and with it (the tensor core runs one thread's products in order) P V of
    // block i-1: the K tile and the other V tile are free, O is stable.  Fetch block i+1 into them.
    const bool ok = t5_mbar_wait(bar_s, parity);
    t5_fence_after();
    if (ok && i + 1 < n_mine) {
      load_keys(sK, i + 1, false);
      load_keys(sV + ((i + 1) & 1) * kT5TileBytes, i + 1, true);
    }
    t5_commit_group();

    // ---- softmax of this thread's row
    const int kb = wg + 2 * i;
    const bool pre = kb < nb_pre;
    const int j0 = pre ? kb * kT5Tile : (kb - nb_pre) * kT5Tile;
    const int lim = (pre ? prefix_len : my_keys) - j0;                         // keys [0, lim) visible to this row
    const bool full = (pre ? prefix_len : min(own_keys, first_keys)) - j0 >= kT5Tile;  // ... all 128 to every row
    uint32_t u[128];
    t5_ld128(tS, u);
    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains instead of one of 128
    if (full) {
#pragma unroll
      for (int c = 0; c < 128; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(u[c]));
    } else {
#pragma unroll
      for (int c = 0; c < 128; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], c < lim ? __uint_as_float(u[c]) : -INFINITY);
    }
    const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
    const float r = mx * scale_log2;
    const bool move = r > m_ref + kT5Lazy;  // also true for the first visible key of a row (m_ref = -inf)
    if (__any_sync(0xffffffffu, move)) {
      const float alpha = move ? t5_exp2(m_ref - r) : 1.f;  // 0 when nothing was accumulated yet
      if (move) { m_ref = r; l *= alpha; }
      if (i > 0) {  // O of the earlier blocks is complete (see above)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t w[32];
          t5_ld32(tO + 32 * c, w);
#pragma unroll
          for (int e = 0; e < 32; ++e) w[e] = __float_as_uint(__uint_as_float(w[e]) * alpha);
          t5_st32(tO + 32 * c, w);
        }
      }
    }
    const float off = m_ref == -INFINITY ? 0.f : m_ref;  // kernels.py:1062
    float ps4[4] = {0.f, 0.f, 0.f, 0.f};
    uint32_t pk[64];
    if (full) {
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        const float p0 = t5_exp2(fmaf(__uint_as_float(u[2 * c]), scale_log2, -off));
        const float p1 = t5_exp2(fmaf(__uint_as_float(u[2 * c + 1]), scale_log2, -off));
        ps4[c & 3] += p0 + p1;
        pk[c] = t5_pack_bf16x2(p0, p1);
      }
    } else {
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        const float p0 = 2 * c < lim ? t5_exp2(fmaf(__uint_as_float(u[2 * c]), scale_log2, -off)) : 0.f;
        const float p1 = 2 * c + 1 < lim ? t5_exp2(fmaf(__uint_as_float(u[2 * c + 1]), scale_log2, -off)) : 0.f;
        ps4[c & 3] += p0 + p1;
        pk[c] = t5_pack_bf16x2(p0, p1);
      }
    }
    l += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
    t5_st64(tS, pk);  // P over the first 64 columns of S
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");

    // ---- K of block i+1 has landed (V of block i did one iteration ago)
    t5_wait_group<0>();
    t5_fence_async_smem();
    if (!ok) asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(dead_flag), "r"(1) : "memory");
    t5_fence_before();
    t5_wg_sync(wg);
    {
      uint32_t f;
      asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(f) : "r"(dead_flag) : "memory");
      if (f) { dead = true; break; }
    }
    if (wt == 0) {
      t5_fence_after();
#pragma unroll
      for (int j = 0; j < 8; ++j)  // 16 keys per instruction: 8 columns of packed P, 2 KB of V rows
        t5_mma_ts(tO_all, tS_all + 8 * j, t5_desc(sV + (i & 1) * kT5TileBytes + j * 2048, kT5BlockBytes, 1024), kT5IdescPV,
                  (i > 0) || (j > 0));
      if (i + 1 < n_mine) issue_s();  // executes behind P V: it overwrites the columns P is read from
      else t5_mma_commit(bar_o);      // the last P V of this warpgroup
    }
  }
  t5_wait_group<0>();
  if (n_mine > 0 && !dead) {
    if (!t5_mbar_wait(bar_o, 0)) asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(dead_flag), "r"(1) : "memory");
    t5_fence_after();
  }

  // ---- merge the two warpgroups: warpgroup 1 hands its (offset, sum, O) over through shared memory
  // (its K tile and first V tile: 64 KB, [channel][row] fp32 so that both sides touch consecutive banks)
  const uint32_t xO = base + kT5TileBytes + kT5WgBytes, xML = base + kT5TileBytes;  // scalars: warpgroup 0's K tile
  t5_wg_sync(wg);  // every thread of the warpgroup is past its last use of these buffers
  {
    uint32_t f;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(f) : "r"(dead_flag) : "memory");
    dead = dead || f;
  }
  if (wg == 1) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t w[32];
      if (n_mine > 0 && !dead) {
        t5_ld32(tO + 32 * c, w);
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) w[e] = 0u;
      }
#pragma unroll
      for (int e = 0; e < 32; ++e)
        asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(xO + ((32 * c + e) * 128 + wt) * 4), "r"(w[e]) : "memory");
    }
  }
  t5_fence_before();
  __syncthreads();  // (a) warpgroup 0 no longer uses its K tile, (b) warpgroup 1's O is visible
  if (wg == 1) {
    const uint32_t a = xML;
    asm volatile("st.shared.f32 [%0], %1;\n" ::"r"(a + wt * 4), "f"(m_ref) : "memory");
    asm volatile("st.shared.f32 [%0], %1;\n" ::"r"(a + 512 + wt * 4), "f"(l) : "memory");
    asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(a + 1024), "r"(dead ? 1 : 0) : "memory");
  }
  __syncthreads();
  if (wg == 0) {
    float m1, l1;
    uint32_t dead1;
    asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(m1) : "r"(xML + wt * 4) : "memory");
    asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(l1) : "r"(xML + 512 + wt * 4) : "memory");
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(dead1) : "r"(xML + 1024) : "memory");
    dead = dead || dead1;
    if (dead && wt == 0 && status) atomicOr(status, B200KV_S_TIMEOUT);
    if (!dead) {
      t5_fence_after();
      const float mm = fmaxf(m_ref, m1);
      const float a0 = m_ref == -INFINITY ? 0.f : t5_exp2(m_ref - mm), a1 = m1 == -INFINITY ? 0.f : t5_exp2(m1 - mm);
      const float lt = l * a0 + l1 * a1;
      const float inv = lt != 0.f ? 1.f / lt : 0.f;  // kernels.py:1118
      const float f0 = a0 * inv, f1 = a1 * inv;
      uint4* dst = reinterpret_cast<uint4*>(out + (long long)my_row * o_sn + hq * o_sh);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t w[32];
        t5_ld32(tO + 32 * c, w);
        float o[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float o1;
          asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(o1) : "r"(xO + ((32 * c + e) * 128 + wt) * 4) : "memory");
          o[e] = __uint_as_float(w[e]) * f0 + o1 * f1;
        }
        if (my_row < row_end) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint4 x;
            x.x = t5_pack_bf16x2(o[8 * e], o[8 * e + 1]);
            x.y = t5_pack_bf16x2(o[8 * e + 2], o[8 * e + 3]);
            x.z = t5_pack_bf16x2(o[8 * e + 4], o[8 * e + 5]);
            x.w = t5_pack_bf16x2(o[8 * e + 6], o[8 * e + 7]);
            dst[4 * c + e] = x;
          }
        }
      }
    }
  }
  t5_fence_before();
  __syncthreads();
  if (tid < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kT5Cols) : "memory");
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
