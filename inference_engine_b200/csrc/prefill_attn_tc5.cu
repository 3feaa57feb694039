// Chunked-prefill attention on the 5th-generation tensor cores (tcgen05 + tensor memory).
// Same contract as prefill_attn_kernel (prefill_attn.cu): packed variable-length causal
// attention of the prefilling entries over [dequantized prefix | own chunk], replacing
// prefill_attention_kernel (qwen3-1.7b/kernels.py:987-1126).
//
// One CTA owns 128 query rows of one q head and runs twelve warps in three roles:
//   warps 0-3 and 4-7   two softmax warpgroups.  The keys of the tile are cut into blocks of 64 and dealt
//                       alternately to the two; each keeps its own running (offset, sum, O) and the two are
//                       merged at the end.  Thread t of a warpgroup owns query row t = lane t of tensor
//                       memory: every row-wise softmax quantity lives in one thread, no shuffles.
//   warps 8 and 9       one lane of each issues every tcgen05.mma of warpgroup 0 and 1.
//   warps 10 and 11     fetch the K and V tiles of warpgroup 0 and 1 (tensor-map copies started by one lane).
// Per key block h of a warpgroup:
//   S(h) = Q K^T   8 x tcgen05.mma (M128 N64 K16, bf16 -> fp32), Q and K from shared memory, into one of the
//                  warpgroup's two S buffers (64 tensor-memory columns each)
//   softmax        one tcgen05.ld of the thread's 64 scores, max, exp2, sum; P rounded to bf16 as the
//                  reference does (kernels.py:1068,1113) and stored over the first 32 columns of the same
//                  S buffer
//   O += P V       4 x tcgen05.mma (M128 N128 K16) with P read from tensor memory and V from shared memory
//                  (channel-contiguous: N-major B operand), accumulating in the warpgroup's 128 O columns
// The products are software-pipelined against the softmax: when P(h) is stored (128 arrivals on a `ready`
// barrier), the issuing lane queues P V(h) and then S(h+2) into the buffer P(h) occupies (the tensor core
// executes one thread's products in issue order), while S(h+1) is already complete or running in the other
// buffer; the warpgroup goes from one softmax straight into the next.  Completions come back through
// tcgen05.commit on mbarriers: `s_done` to the softmax threads, `kempty` / `vempty` to the fetching warp,
// which refills the ring slot (three K and three V tiles of 16 KB per warpgroup) and reports on `kfull` /
// `vfull`.  Measured on a B200 an M128 N64 K16 product from shared memory takes 49 cycles and an
// M128 N128 K16 one 65 (the latter is the nominal rate; the former is bound by the 128 B/clk the tensor
// core reads shared memory at), so one block pair costs the tensor core about 1300 cycles.
// O stays in tensor memory for the whole tile.  Its rescaling is lazy: the reference offset of the
// exponentials only moves when the row maximum has grown by more than 2^8 since it was set (then, after
// waiting for the one P V that may be in flight, O and the sum are multiplied by the correction, a
// tensor-memory round trip); otherwise P is simply computed against the older offset, which is the same
// mathematics.
//
// Q, K and V tiles are laid out in shared memory as the canonical 128-byte-swizzled layout the matrix
// descriptors name: two blocks of 64 channels, each [row][128 bytes] with the 16-byte chunk index XOR-ed
// with (row & 7) - which is also what a tensor-map copy with the 128-byte swizzle writes.  K and V use the
// same physical layout; only their descriptors differ (K: K-major, rows = N; V: N-major, rows = K).
// A prefix block that is not full is copied with cp.async and zero-filled instead (see the fetching warp).
//
// Every wait on an mbarrier is bounded: if a completion never arrives the waiting role records it, stops
// issuing work and the CTA skips its stores, sets B200KV_S_TIMEOUT in the status word, frees its tensor
// memory and returns.
#include <cuda.h>  // CUtensorMap and the cuTensorMapEncodeTiled prototype only; the entry point is fetched at run time

#include "common.cuh"
#include "tmem_ldst.cuh"

namespace b200kv {

constexpr int kT5Threads = 384;                       // two softmax warpgroups, two warps issuing products, two fetching tiles
constexpr int kT5Tile = 128;                         // query rows per CTA
constexpr int kT5Keys = 64;                          // keys per block
constexpr uint32_t kT5QBytes = kT5Tile * kD * 2;     // Q tile: 32 KB, two 64-channel blocks of 16 KB
constexpr uint32_t kT5KvBytes = kT5Keys * kD * 2;    // K or V tile: 16 KB, two 64-channel blocks of 8 KB
constexpr uint32_t kT5WgBytes = 6 * kT5KvBytes;      // per warpgroup: K ring of 3, V ring of 3
constexpr uint32_t kT5Smem = kT5QBytes + 2 * kT5WgBytes + 1024 /* alignment slack */ + 384 /* barriers, flags */;
constexpr uint32_t kT5Cols = 512;                    // tensor memory: warpgroup w has S0/P0 at 256w, S1/P1 at 256w+64, O at 256w+128
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
__device__ __forceinline__ bool t5_mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit) {
  for (uint32_t spin = 0; spin < limit; ++spin) {
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
__device__ __forceinline__ void t5_mbar_arrive(uint32_t bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}\n" ::"r"(bar) : "memory");
}
// One arrival that also announces `bytes` of bulk-copy traffic the phase has to see before it completes.
__device__ __forceinline__ void t5_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}\n" ::"r"(bar), "r"(bytes) : "memory");
}
// Tensor-map (TMA) tile load of one box into shared memory; completion is counted in bytes on `bar`.
// c0 (the channel coordinate) must keep the 16-byte rule: it is 0 or 64 bf16 here.
__device__ __forceinline__ void t5_tma_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
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
// Instruction descriptor of kind::f16: fp32 accumulator, bf16 A and B, M = 128, N as given.
constexpr uint32_t t5_idesc(uint32_t n) { return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24); }
constexpr uint32_t kT5IdescQK = t5_idesc(kT5Keys);        // A (Q) K-major, B (K tile) K-major, N = 64 keys
constexpr uint32_t kT5IdescPV = t5_idesc(kD) | (1u << 16); // B (V tile) N-major, N = 128 channels

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

// Copied by kThreads threads (tid in [0, kThreads)): `count` (<= kRows) rows of 128 bf16 (row j at
// src + j*stride elements) into a swizzled tile of kRows rows; rows past `count` are zero-filled.
template <int kThreads, int kRows>
__device__ __forceinline__ void t5_load_tile(uint32_t dst, const uint16_t* src, long long stride, int count, int tid) {
#pragma unroll
  for (int i = 0; i < (kRows * 16) / kThreads; ++i) {
    const int c = tid + i * kThreads, r = c >> 4, col = c & 15;
    const bool valid = r < count;
    const uint32_t d = dst + (col >> 3) * (kRows * 128) + r * 128 + (((col & 7) ^ (r & 7)) << 4);
    t5_cp16(d, valid ? src + r * stride + col * 8 : src, valid ? 16 : 0);
  }
}

__device__ __forceinline__ void t5_wg_sync(int wg) { asm volatile("bar.sync %0, 128;\n" ::"r"(wg + 1) : "memory"); }
__device__ __forceinline__ void t5_sts_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t t5_lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr) : "memory");
  return v;
}

__global__ void __launch_bounds__(kT5Threads, 1)
prefill_attn_tc5_kernel(const uint16_t* __restrict__ q, long long q_sn, long long q_sh, const uint16_t* __restrict__ k,
                        long long k_sn, long long k_sh, const uint16_t* __restrict__ v, long long v_sn, long long v_sh,
                        const int32_t* __restrict__ seq_ids, const int32_t* __restrict__ cu_seqlens,
                        const int32_t* __restrict__ tile_start, int block_m, int subs,
                        const uint16_t* __restrict__ k_prefix, const uint16_t* __restrict__ v_prefix, long long p_sh,
                        long long p_sn, const int32_t* __restrict__ cu_cached, uint16_t* __restrict__ out, long long o_sn,
                        long long o_sh, int N, int G, float scale_log2, int32_t* status,
                        const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                        const __grid_constant__ CUtensorMap tm_kp, const __grid_constant__ CUtensorMap tm_vp, int prefix_tma,
                        int idle_issuers) {
  extern __shared__ uint8_t t5_raw[];
  // idle_issuers (a test mode): the issuing warps do nothing and every wait gives up after a few thousand polls,
  // so that all bounded waits of the kernel run out and the time-out path is exercised without a fault
  const uint32_t spin = idle_issuers ? 4096u : kT5SpinLimit;
  // The first CTA waits for the predecessor on every path (a grid in which no CTA waited could complete before
  // it); the trigger for the successor comes late, from the softmax threads when their last block is done: a
  // successor brought up while this kernel is in full swing would only sit on the SMs.
  if ((blockIdx.x | blockIdx.y) == 0) pdl_wait();
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
  const int row0 = tile_row + sub * kT5Tile;  // first query row of this CTA
  if (row0 >= row_end) return;
  const int cta_last = min(row0 + kT5Tile, row_end) - 1;
  const int own_keys = cta_last - seq_start + 1;  // causal: keys up to the CTA's last query
  const int nb_pre = (prefix_len + kT5Keys - 1) / kT5Keys, nb_own = (own_keys + kT5Keys - 1) / kT5Keys;
  const int nb = nb_pre + nb_own;

  float m_ref_keep = -INFINITY, l_keep = 0.f;
  // roles: warps 0-3 and 4-7 = softmax warpgroups 0 and 1, warps 8 and 9 = issue the products of warpgroup 0
  // and 1, warps 10 and 11 = fetch the K and V tiles of warpgroup 0 and 1
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, wg = tid >> 7, wt = tid & 127;
  const int n_blk[2] = {(nb + 1) >> 1, nb >> 1};  // warpgroup w owns blocks w, w + 2, ...
  const uint32_t base = (t5_smem_u32(t5_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base;
  const uint32_t bars = base + kT5QBytes + 2 * kT5WgBytes;
  // per warpgroup w, 18 barriers at bars + 144 w:
  //   s_done[2]  S buffer b holds a complete S (arrival = tcgen05.commit)
  //   o_done[2]  the last-but-one and the last P V are complete (one phase each: a parity wait must never fall
  //              two phases behind, so these two do not share a barrier)
  //   ready[2]   P is stored in S buffer b (128 arrivals)
  //   kfull[3], vfull[3]    ring slot holds its tile (one arrival by the fetching warp, plus the tile's bytes
  //                         when it is a tensor-map copy)
  //   kempty[3], vempty[3]  the product that read the slot is complete (tcgen05.commit)
  auto ring_k = [&](int w) { return base + kT5QBytes + w * kT5WgBytes; };
  auto ring_v = [&](int w) { return ring_k(w) + 3 * kT5KvBytes; };
  auto bar_s = [&](int w, int buf) { return bars + 144 * w + 8 * buf; };
  auto bar_o = [&](int w, int which) { return bars + 144 * w + 16 + 8 * which; };
  auto bar_r = [&](int w, int buf) { return bars + 144 * w + 32 + 8 * buf; };
  auto bar_kf = [&](int w, int sl) { return bars + 144 * w + 48 + 8 * sl; };
  auto bar_vf = [&](int w, int sl) { return bars + 144 * w + 72 + 8 * sl; };
  auto bar_ke = [&](int w, int sl) { return bars + 144 * w + 96 + 8 * sl; };
  auto bar_ve = [&](int w, int sl) { return bars + 144 * w + 120 + 8 * sl; };
  const uint32_t bar_q = bars + 288;  // the Q tile has landed (256 arrivals)
  const uint32_t slot = bars + 296, dead_flag = bars + 304;

  if (tid == 0) {
    for (int w = 0; w < 2; ++w) {
      for (int i = 0; i < 18; ++i) t5_mbar_init(bars + 144 * w + 8 * i, (i == 4 || i == 5) ? 128 : 1);  // 4, 5: ready
    }
    t5_mbar_init(bar_q, 256);
    t5_sts_u32(dead_flag, 0);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (tid < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot), "r"(kT5Cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  t5_fence_before();
  __syncthreads();  // barriers and the tensor-memory base are visible to every role
  t5_fence_after();
  pdl_wait();  // q, k, v and the prefix come from the kernels before this one; only metadata was read so far
  const uint32_t tmem = t5_lds_u32(slot);
  bool dead = false;
  if (wg < 2) {
    // The softmax threads copy the Q tile while the fetching warps already stream K and V.  Q rows past the end
    // of the packed batch are zero-filled; rows of other entries inside the tile are read and computed but
    // never stored.
    t5_load_tile<256, kT5Tile>(sQ, q + (long long)row0 * q_sn + hq * q_sh, q_sn, min(kT5Tile, N - row0), tid);
    t5_commit_group();
    t5_wait_group<0>();
    t5_fence_async_smem();
    t5_mbar_arrive(bar_q);
  }

  if (warp >= 10) {
    // ---- a fetching warp: streams the K and V tiles of warpgroup w into its rings.  Block h of the warpgroup
    // is block w + 2h of the tile and lives in slot h % 3.  Full tiles come by tensor-map copies started by
    // lane 0 (two boxes of 64 rows x 64 channels, swizzled by the copy engine into the layout described
    // above).  A prefix block that is not full is copied by the warp's 32 lanes with cp.async instead, because
    // the rows behind a prefix may be uninitialised memory and have to be zero in shared memory (0 x NaN would
    // poison O); so is every prefix block when the caller gave no row capacity for the prefix tensors.
    const int w = warp - 10, n = n_blk[w];
    const uint16_t* kpre = k_prefix + hk * p_sh + (long long)prefix_start * p_sn;
    const uint16_t* vpre = v_prefix + hk * p_sh + (long long)prefix_start * p_sn;
    const uint16_t* kown = k + (long long)seq_start * k_sn + hk * k_sh;
    const uint16_t* vown = v + (long long)seq_start * v_sn + hk * v_sh;
    bool live = true;
    for (int h = 0; h < n && live; ++h) {
      const int kb = w + 2 * h, sl = h % 3;
      const bool pre = kb < nb_pre;
      const int j0 = pre ? kb * kT5Keys : (kb - nb_pre) * kT5Keys;
      const int count = min(kT5Keys, (pre ? prefix_len : own_keys) - j0);
      const bool tma = !pre || (prefix_tma && count == kT5Keys);
      const int row = pre ? prefix_start + j0 : seq_start + j0;
      for (int is_v = 0; is_v < 2 && live; ++is_v) {
        const uint32_t dst = (is_v ? ring_v(w) : ring_k(w)) + sl * kT5KvBytes;
        const uint32_t full = is_v ? bar_vf(w, sl) : bar_kf(w, sl), empty = is_v ? bar_ve(w, sl) : bar_ke(w, sl);
        // the product that read this slot three blocks ago has completed
        if (h >= 3 && !t5_mbar_wait(empty, (h / 3 - 1) & 1, spin)) { live = false; break; }
        if (tma) {
          if (lane == 0) {
            t5_mbar_expect_tx(full, kT5KvBytes);
            const CUtensorMap* map = pre ? (is_v ? &tm_vp : &tm_kp) : (is_v ? &tm_v : &tm_k);
            t5_tma_3d(dst, map, 0, pre ? row : hk, pre ? hk : row, full);
            t5_tma_3d(dst + kT5Keys * 128, map, 64, pre ? row : hk, pre ? hk : row, full);
          }
        } else {
          const uint16_t* src = pre ? (is_v ? vpre : kpre) + (long long)j0 * p_sn
                                    : (is_v ? vown + (long long)j0 * v_sn : kown + (long long)j0 * k_sn);
          t5_load_tile<32, kT5Keys>(dst, src, pre ? p_sn : (is_v ? v_sn : k_sn), count, lane);
          t5_commit_group();
          t5_wait_group<0>();
          t5_fence_async_smem();
          __syncwarp();
          if (lane == 0) t5_mbar_arrive(full);
        }
      }
    }
    if (!live && lane == 0) t5_sts_u32(dead_flag, 1);
  } else if (warp >= 8) {
    // ---- an issuing warp: one lane queues every product of warpgroup w.  The descriptors are built once; per
    // instruction only the start-address field moves.  The issue of a product blocks while the tensor core's
    // queue is full, and this lane's waits and commits are not hidden behind its own products; with one
    // issuing lane per warpgroup the bookkeeping of one overlaps the products of the other.
    if (lane == 0 && !idle_issuers) {
      const int w = warp - 8, n = n_blk[w];
      const uint64_t dq = t5_desc(sQ, 16, 1024), dk = t5_desc(ring_k(w), 16, 1024);
      const uint64_t dv = t5_desc(ring_v(w), kT5Keys * 128, 1024);
      const uint32_t tw = tmem + 256 * w;
      bool live = t5_mbar_wait(bar_q, 0, spin);
      auto issue_s = [&](int h) {  // S(h) = Q K(h)^T into S buffer h & 1, then the arrivals
        const int sl = h % 3;
        if (!t5_mbar_wait(bar_kf(w, sl), (h / 3) & 1, spin)) { live = false; return; }
        const uint64_t kd = dk + (uint64_t)(sl * (kT5KvBytes >> 4));
        const uint32_t d = tw + 64 * (h & 1);
#pragma unroll
        for (int j = 0; j < 8; ++j)  // 16 channels per instruction
          t5_mma_ss(d, dq + (uint64_t)(((j >> 2) * (kT5Tile * 128) + (j & 3) * 32) >> 4),
                    kd + (uint64_t)(((j >> 2) * (kT5Keys * 128) + (j & 3) * 32) >> 4), kT5IdescQK, j > 0);
        t5_mma_commit(bar_s(w, h & 1));
        t5_mma_commit(bar_ke(w, sl));
      };
      for (int h = 0; h < 2; ++h)
        if (h < n && live) issue_s(h);
      for (int h = 0; h < n && live; ++h) {
        const int sl = h % 3;
        // P(h) is stored and V(h) has landed
        if (!t5_mbar_wait(bar_r(w, h & 1), (h >> 1) & 1, spin) || !t5_mbar_wait(bar_vf(w, sl), (h / 3) & 1, spin)) {
          live = false;
          break;
        }
        t5_fence_after();
        const uint64_t vd = dv + (uint64_t)(sl * (kT5KvBytes >> 4));
#pragma unroll
        for (int j = 0; j < 4; ++j)  // 16 keys per instruction: 8 columns of packed P, 2 KB of V rows
          t5_mma_ts(tw + 128, tw + 64 * (h & 1) + 8 * j, vd + (uint64_t)(j * (2048 >> 4)), kT5IdescPV, (h > 0) || (j > 0));
        t5_mma_commit(bar_ve(w, sl));
        if (h + 2 < n) issue_s(h + 2);  // executes behind P V(h): it overwrites the columns P(h) is read from
        else t5_mma_commit(bar_o(w, h + 1 < n ? 0 : 1));  // the last-but-one / the last P V of the warpgroup
      }
      if (!live) t5_sts_u32(dead_flag, 1);
    }
  } else {
    const int n_mine = n_blk[wg];
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + 256 * wg + lane_base, tO = tS + 128;  // this thread's lane
    const int my_keys = min(own_keys, row0 + wt - seq_start + 1);  // own-chunk keys this row may see
    const int first_keys = min(own_keys, row0 - seq_start + 1);    // ... and the tile's first row
    float m_ref = -INFINITY, l = 0.f;  // offset of the exponentials (log2 units, scaled), running sum
    bool ok = true;
    for (int h = 0; h < n_mine && ok; ++h) {
      ok = t5_mbar_wait(bar_s(wg, h & 1), (h >> 1) & 1, spin);  // S(h) is complete
      t5_fence_after();
      // ---- softmax of this thread's row
      const int kb = wg + 2 * h;
      const bool pre = kb < nb_pre;
      const int j0 = pre ? kb * kT5Keys : (kb - nb_pre) * kT5Keys;
      const int lim = (pre ? prefix_len : my_keys) - j0;                // keys [0, lim) visible to this row
      const bool full = (pre ? prefix_len : first_keys) - j0 >= kT5Keys;  // ... all 64 to every row of the tile
      uint32_t u[64];
      t5_ld64(tS + 64 * (h & 1), u);
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains instead of one of 64
      if (full) {
#pragma unroll
        for (int c = 0; c < 64; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(u[c]));
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], c < lim ? __uint_as_float(u[c]) : -INFINITY);
      }
      const float r = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
      const bool move = r > m_ref + kT5Lazy;  // also true for the first visible key of a row (m_ref = -inf)
      if (__any_sync(0xffffffffu, move)) {
        const float alpha = move ? t5_exp2(m_ref - r) : 1.f;  // 0 when nothing was accumulated yet
        if (move) { m_ref = r; l *= alpha; }
        if (h > 0) {
          // O must be at rest: P V(h-1) may still be queued.  Its completion is what S(h+1)'s barrier (or, for
          // the last block, the barrier of the last-but-one P V) reports; waiting for that phase here and again
          // at the top of the next block is harmless.
          ok = ok && (h + 1 < n_mine ? t5_mbar_wait(bar_s(wg, (h + 1) & 1), ((h + 1) >> 1) & 1, spin) : t5_mbar_wait(bar_o(wg, 0), 0, spin));
          t5_fence_after();
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
      uint32_t pk[32];
      if (full) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float p0 = t5_exp2(fmaf(__uint_as_float(u[2 * c]), scale_log2, -off));
          const float p1 = t5_exp2(fmaf(__uint_as_float(u[2 * c + 1]), scale_log2, -off));
          ps4[c & 3] += p0 + p1;
          pk[c] = t5_pack_bf16x2(p0, p1);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float p0 = 2 * c < lim ? t5_exp2(fmaf(__uint_as_float(u[2 * c]), scale_log2, -off)) : 0.f;
          const float p1 = 2 * c + 1 < lim ? t5_exp2(fmaf(__uint_as_float(u[2 * c + 1]), scale_log2, -off)) : 0.f;
          ps4[c & 3] += p0 + p1;
          pk[c] = t5_pack_bf16x2(p0, p1);
        }
      }
      l += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
      t5_st32(tS + 64 * (h & 1), pk);  // P over the first 32 columns of this S buffer
      asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
      t5_fence_before();
      if (ok) t5_mbar_arrive(bar_r(wg, h & 1));  // hand P(h) to the issuing warp
    }
    pdl_trigger();
    if (n_mine > 0 && ok) ok = t5_mbar_wait(bar_o(wg, 1), 0, spin);  // the last P V
    t5_fence_after();
    if (!ok) t5_sts_u32(dead_flag, 1);
    m_ref_keep = m_ref;
    l_keep = l;
  }

  // ---- merge the two warpgroups: warpgroup 1 hands its (offset, sum, O) over through shared memory
  // (the first 64 KB of its rings, [channel][row] fp32 so that both sides touch consecutive banks)
  const uint32_t xO = base + kT5QBytes + kT5WgBytes, xML = base + kT5QBytes;  // scalars: start of warpgroup 0's rings
  const uint32_t tO = tmem + 256 * (wg & 1) + 128 + ((uint32_t)(((tid >> 5) & 3) * 32) << 16);
  const int my_row = row0 + wt;
  t5_fence_before();
  __syncthreads();  // every product of the CTA is complete (or given up), nobody uses the rings any more
  t5_fence_after();
  dead = t5_lds_u32(dead_flag) != 0;
  if (wg == 1) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t w[32];
      if (n_blk[1] > 0 && !dead) {
        t5_ld32(tO + 32 * c, w);
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) w[e] = 0u;
      }
#pragma unroll
      for (int e = 0; e < 32; ++e) t5_sts_u32(xO + ((32 * c + e) * 128 + wt) * 4, w[e]);
    }
    t5_sts_u32(xML + wt * 4, __float_as_uint(m_ref_keep));
    t5_sts_u32(xML + 512 + wt * 4, __float_as_uint(l_keep));
  }
  __syncthreads();
  if (wg == 0) {
    const float m0 = m_ref_keep, l0 = l_keep;
    const float m1 = __uint_as_float(t5_lds_u32(xML + wt * 4)), l1 = __uint_as_float(t5_lds_u32(xML + 512 + wt * 4));
    if (dead && wt == 0 && status) atomicOr(status, B200KV_S_TIMEOUT);
    if (!dead) {
      const float mm = fmaxf(m0, m1);
      const float a0 = m0 == -INFINITY ? 0.f : t5_exp2(m0 - mm), a1 = m1 == -INFINITY ? 0.f : t5_exp2(m1 - mm);
      const float lt = l0 * a0 + l1 * a1;
      const float inv = lt != 0.f ? 1.f / lt : 0.f;  // kernels.py:1118
      const float f0 = a0 * inv, f1 = a1 * inv;
      uint4* dst = reinterpret_cast<uint4*>(out + (long long)my_row * o_sn + hq * o_sh);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t w[32];
        t5_ld32(tO + 32 * c, w);
        float o[32];
#pragma unroll
        for (int e = 0; e < 32; ++e)
          o[e] = __uint_as_float(w[e]) * f0 + __uint_as_float(t5_lds_u32(xO + ((32 * c + e) * 128 + wt) * 4)) * f1;
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

// cuTensorMapEncodeTiled, fetched from the driver through the runtime (the library links no libcuda).
typedef CUresult (*t5_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static t5_encode_fn t5_encoder() {
  static t5_encode_fn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return (t5_encode_fn)p;
  }();
  return fn;
}
// A bf16 tensor [d2][d1][128 channels] with element strides (s2, s1, 1), read in boxes of 64 channels x b1 x b2
// with the 128-byte swizzle; out-of-range rows read as zero.
static bool t5_make_map(CUtensorMap* map, const void* base, uint64_t d1, uint64_t d2, long long s1, long long s2, uint32_t b1,
                        uint32_t b2) {
  t5_encode_fn enc = t5_encoder();
  if (!enc || d1 == 0 || d2 == 0 || s1 <= 0 || s2 <= 0) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)kD, d1, d2};
  const cuuint64_t strides[2] = {(cuuint64_t)s1 * 2, (cuuint64_t)s2 * 2};
  const cuuint32_t box[3] = {64, b1, b2}, estr[3] = {1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// prefix_rows: rows each kv head of k_prefix / v_prefix holds (0 = not known: prefix tiles are then copied with
// cp.async only).
int launch_prefill_attn_tc5(const uint16_t* q, long long q_sn, long long q_sh, const uint16_t* k, long long k_sn,
                            long long k_sh, const uint16_t* v, long long v_sn, long long v_sh, const int32_t* seq_ids,
                            const int32_t* cu_seqlens, const int32_t* tile_start, int num_tiles, int block_m,
                            const uint16_t* k_prefix, const uint16_t* v_prefix, long long p_sh, long long p_sn,
                            int prefix_rows, const int32_t* cu_cached, uint16_t* out, long long o_sn, long long o_sh, int N,
                            int Hq, int Hkv, float scale_log2, int32_t* status, int idle_issuers, cudaStream_t stream) {
  // the opt-in is a per-device attribute of the function: set it on every call (it is cheap)
  if (cudaFuncSetAttribute(prefill_attn_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kT5Smem) !=
      cudaSuccess)
    return B200KV_E_LAUNCH;
  CUtensorMap tm_k, tm_v, tm_kp, tm_vp;
  // own chunk [N][Hkv][128]: box = 64 rows of one head
  if (!t5_make_map(&tm_k, k, Hkv, N, k_sh, k_sn, 1, kT5Keys) || !t5_make_map(&tm_v, v, Hkv, N, v_sh, v_sn, 1, kT5Keys))
    return B200KV_E_LAUNCH;
  // prefix [Hkv][rows][128]: box = 64 rows of one head; without a row count the maps are placeholders
  int prefix_tma = prefix_rows > 0 && t5_make_map(&tm_kp, k_prefix, prefix_rows, Hkv, p_sn, p_sh, kT5Keys, 1) &&
                   t5_make_map(&tm_vp, v_prefix, prefix_rows, Hkv, p_sn, p_sh, kT5Keys, 1);
  if (!prefix_tma) { tm_kp = tm_k; tm_vp = tm_v; }
  const int subs = (block_m + kT5Tile - 1) / kT5Tile;
  const cudaError_t le = launch_chained(prefill_attn_tc5_kernel, dim3(Hq, num_tiles * subs), dim3(kT5Threads), kT5Smem, stream,
                                        q, q_sn, q_sh, k, k_sn, k_sh, v, v_sn, v_sh, seq_ids, cu_seqlens, tile_start, block_m, subs,
                                        k_prefix, v_prefix, p_sh, p_sn, cu_cached, out, o_sn, o_sh, N, Hq / Hkv, scale_log2, status,
                                        tm_k, tm_v, tm_kp, tm_vp, prefix_tma, idle_issuers);
  return le == cudaSuccess && cudaGetLastError() == cudaSuccess ? B200KV_OK : B200KV_E_LAUNCH;
}

}  // namespace b200kv
