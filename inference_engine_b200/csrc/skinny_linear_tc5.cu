// Weight-streaming matmul for few rows (decode steps): y[M, N] = x[M, K] . W[N, K]^T with M <= 64, on the
// 5th-generation tensor cores (tcgen05 + tensor memory), fed by tensor-map (TMA) copies.  Replaces
// skinny_matmul_kernel / skinny_matmul (qwen3-1.7b/kernels.py:1373-1455).
//
// At these row counts the matmul is bound by reading W once from HBM (2 N K bytes): the tensor core has to do
// 2 M N K flops per 2 N K bytes, i.e. M flops per byte, which CUDA cores cannot deliver at 6+ TB/s beyond a
// handful of rows.  So the roles are swapped: a CTA owns 128 WEIGHT rows as the M dimension of the MMA
// (tcgen05.mma, M128 N{16,32,64} K16, bf16 -> fp32) and the token rows of x, padded to 16 / 32 / 64, are its N
// dimension; the accumulator [128 weight rows x tokens] lives in tensor memory.
//
//   grid (N / 128, S), cluster (1, S): the S CTAs of a cluster share one block of 128 weight rows and split K in
//   units of 64 channels, so that even a [2048 x 2048] weight occupies ~128 SMs with 16 row blocks.
//   warp 0, one lane   producer: per 64-channel step one TMA box of W (128 rows x 128 bytes, 16 KB) and one of x
//                      (tokens x 128 bytes) into a ring of kSkStages slots, both counted in bytes on the slot's
//                      `full` barrier.  W is a constant of the model, so its first slots are requested BEFORE the
//                      wait for the preceding kernel (which produces x); x follows after the wait.
//   warp 1, one lane   issues 4 tcgen05.mma per slot (K = 16 each), then tcgen05.commit on the slot's `empty`
//                      barrier; after the last slot a commit on `done`.
//   warps 2-5          epilogue: each thread owns one weight row = one lane of tensor memory.  S = 1: tcgen05.ld,
//                      round to bf16, store y[m][n] (a warp writes 64 contiguous bytes per token).  S > 1: the
//                      cluster reduces through distributed shared memory: CTA r receives from every CTA the
//                      accumulator columns of tokens [r T/S, (r+1) T/S), between two cluster barriers, sums the S
//                      contributions in a fixed order and stores those tokens.
// Every mbarrier wait is bounded; when one runs out the CTA records B200KV_S_TIMEOUT, keeps taking part in the
// cluster barriers (they are hardware barriers that every CTA of the cluster reaches on every path), stores nothing
// and frees its tensor memory.
#include <cuda.h>

#include "common.cuh"
#include "tmem_ldst.cuh"

namespace b200kv {

constexpr int kSkRows = 128;     // weight rows per CTA
constexpr int kSkStep = 64;      // channels per pipeline slot (128 bytes: one swizzle atom)
constexpr int kSkStages = 4;
constexpr int kSkThreads = 192;  // producer warp, issuing warp, four epilogue warps
constexpr uint32_t kSkWBytes = kSkRows * kSkStep * 2;  // 16 KB
constexpr uint32_t kSkSpin = 1u << 20;

__device__ __forceinline__ uint32_t sk_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void sk_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ bool sk_mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit) {
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
__device__ __forceinline__ void sk_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}\n" ::"r"(bar), "r"(bytes) : "memory");
}
// Tensor-map tile load into this CTA alone (every CTA fetches its own boxes of this GPU's memory).  c0 is a multiple of
// 64 bf16 = 128 bytes, so the 16-byte rule of the innermost coordinate holds.
__device__ __forceinline__ void sk_tma_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void sk_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
// Shared-memory matrix descriptor, K-major operand in the 128-byte-swizzled layout a tensor-map copy writes:
// rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t sk_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(16u >> 4) << 16) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
// kind::f16 instruction descriptor: fp32 accumulator, bf16 A and B (both K-major), M = 128, N = n.
__host__ __device__ constexpr uint32_t sk_idesc(uint32_t n) { return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24); }
__device__ __forceinline__ void sk_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void sk_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
template <int N>
__device__ __forceinline__ void sk_tmem_ld(uint32_t taddr, uint32_t (&u)[N]);
template <>
__device__ __forceinline__ void sk_tmem_ld<64>(uint32_t taddr, uint32_t (&u)[64]) { t5_ld64(taddr, u); }
template <>
__device__ __forceinline__ void sk_tmem_ld<32>(uint32_t taddr, uint32_t (&u)[32]) { t5_ld32(taddr, u); }
template <>
__device__ __forceinline__ void sk_tmem_ld<16>(uint32_t taddr, uint32_t (&u)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;\n"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
        "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
      : "r"(taddr) : "memory");
}

// kT = token columns of the accumulator (M rounded up to 16, 32 or 64).
template <int kT>
__global__ void __launch_bounds__(kSkThreads, 2)
skinny_linear_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                     uint16_t* __restrict__ y, long long ldy, int M, int K, int S, int32_t* status) {
  extern __shared__ uint8_t sk_raw[];
  constexpr uint32_t kXBytes = kT * kSkStep * 2;
  constexpr uint32_t kSlot = kSkWBytes + kXBytes;
  constexpr uint32_t kCols = kT < 32 ? 32 : kT;  // tensor-memory columns: a power of two >= 32
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t base = (sk_smem_u32(sk_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + kSkStages * kSlot;  // full[kSkStages], empty[kSkStages], done
  auto bar_full = [&](int s) { return bars + 8 * s; };
  auto bar_empty = [&](int s) { return bars + 8 * (kSkStages + s); };
  const uint32_t bar_done = bars + 16 * kSkStages, slot_word = bar_done + 8, dead_word = bar_done + 12;
  unsigned crank = 0;
  if (S > 1) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
  // this CTA's share of the K steps: as even as the count allows, earlier ranks take the larger shares
  const int steps_all = K / kSkStep;
  const int step0 = (int)(((long long)steps_all * crank) / S), step1 = (int)(((long long)steps_all * (crank + 1)) / S);
  const int nsteps = step1 - step0;
  const int n0 = blockIdx.x * kSkRows;

  if ((blockIdx.x | blockIdx.y) == 0) pdl_wait();  // a grid in which no CTA waited could complete before its predecessor
  if (tid == 0) {
    for (int s = 0; s < kSkStages; ++s) {
      sk_mbar_init(bar_full(s), 1);
      sk_mbar_init(bar_empty(s), 1);
    }
    sk_mbar_init(bar_done, 1);
    asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(dead_word), "r"(0) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot_word), "r"(kCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  uint32_t tmem;
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(tmem) : "r"(slot_word) : "memory");
  bool dead = false;

  if (warp == 0) {
    if (lane == 0) {
      // weights first (they do not depend on the kernel before this one), then the wait, then x
      const int pre = min(nsteps, kSkStages);
      for (int i = 0; i < pre; ++i) {
        sk_expect_tx(bar_full(i), kSlot);
        sk_tma_2d(base + i * kSlot, &tm_w, (step0 + i) * kSkStep, n0, bar_full(i));
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i) sk_tma_2d(base + i * kSlot + kSkWBytes, &tm_x, (step0 + i) * kSkStep, 0, bar_full(i));
      for (int i = pre; i < nsteps; ++i) {
        const int s = i % kSkStages;
        if (!sk_mbar_wait(bar_empty(s), (i / kSkStages - 1) & 1, kSkSpin)) { dead = true; break; }
        sk_expect_tx(bar_full(s), kSlot);
        sk_tma_2d(base + s * kSlot, &tm_w, (step0 + i) * kSkStep, n0, bar_full(s));
        sk_tma_2d(base + s * kSlot + kSkWBytes, &tm_x, (step0 + i) * kSkStep, 0, bar_full(s));
      }
      pdl_trigger();  // nothing left to fetch: the next kernel may be brought up
      if (dead) asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(dead_word), "r"(1) : "memory");
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = sk_idesc(kT);
      for (int i = 0; i < nsteps; ++i) {
        const int s = i % kSkStages;
        if (!sk_mbar_wait(bar_full(s), (i / kSkStages) & 1, kSkSpin)) { dead = true; break; }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint64_t da = sk_desc(base + s * kSlot), db = sk_desc(base + s * kSlot + kSkWBytes);
#pragma unroll
        for (int j = 0; j < kSkStep / 16; ++j) sk_mma(tmem, da + (uint64_t)((j * 32) >> 4), db + (uint64_t)((j * 32) >> 4), idesc, (i | j) != 0);
        sk_commit(bar_empty(s));
      }
      if (dead) asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(dead_word), "r"(1) : "memory");
      sk_commit(bar_done);  // arrives when every product issued above has completed (at once if there were none)
    }
  }

  // ---- epilogue: warps 2-5; warp w reads tensor-memory lanes 32 (w % 4) .. +31 = weight rows n0 + that
  float acc[kT];
  const int row = 32 * (warp & 3) + lane;
  if (warp >= 2) {
    if (!sk_mbar_wait(bar_done, 0, kSkSpin)) dead = true;
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    uint32_t raw[kT];
    if (!dead && nsteps > 0) {
      sk_tmem_ld<kT>(tmem + ((uint32_t)(32 * (warp & 3)) << 16), raw);
    } else {
#pragma unroll
      for (int m = 0; m < kT; ++m) raw[m] = 0u;
    }
#pragma unroll
    for (int m = 0; m < kT; ++m) acc[m] = __uint_as_float(raw[m]);
  }
  if (S == 1) {
    if (warp >= 2) {
      uint32_t d;
      asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(d) : "r"(dead_word) : "memory");
      dead = dead || d != 0;
      if (dead) {
        if (row == 0 && status) atomicOr(status, B200KV_S_TIMEOUT);
      } else {
#pragma unroll
        for (int m = 0; m < kT; ++m)
          if (m < M) y[(long long)m * ldy + n0 + row] = (uint16_t)float_to_bf16_bits(acc[m]);
      }
    }
  } else {
    // reduce-scatter over the cluster through distributed shared memory.  The pipeline slots are idle now (every
    // product has completed), so the receive area [S senders][kT / S tokens][128 rows] fp32 reuses them.
    const int per = kT / S;  // tokens this CTA finishes; S divides kT (both powers of two, S <= 8 <= kT / 2)
    __syncthreads();         // all roles of this CTA are past their use of the slots
    sk_cluster_sync();       // ... and so are the peers, before anyone writes into them
    if (warp >= 2) {
      const uint32_t mine = base + ((crank * per) * kSkRows + row) * 4;  // [sender = me][token 0][row] in the receiver
#pragma unroll
      for (int m = 0; m < kT; ++m) {
        const uint32_t dst_rank = m / per;
        const uint32_t local = mine + (uint32_t)((m - dst_rank * per) * kSkRows * 4);
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(dst_rank));
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(acc[m]) : "memory");
      }
      uint32_t d;
      asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(d) : "r"(dead_word) : "memory");
      dead = dead || d != 0;
      if (dead && row == 0 && status) atomicOr(status, B200KV_S_TIMEOUT);
    }
    sk_cluster_sync();  // every contribution has landed
    if (warp >= 2) {
      for (int t = 0; t < per; ++t) {
        const int m = crank * per + t;
        float sum = 0.f;
        for (int src = 0; src < S; ++src) {
          float v;
          asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v) : "r"(base + ((src * per + t) * kSkRows + row) * 4) : "memory");
          sum += v;
        }
        if (m < M) y[(long long)m * ldy + n0 + row] = (uint16_t)float_to_bf16_bits(sum);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kCols) : "memory");
}

typedef CUresult (*sk_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static sk_encode_fn sk_encoder() {
  static sk_encode_fn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return (sk_encode_fn)p;
  }();
  return fn;
}
// bf16 matrix [rows][K] with `ld` elements between rows, read in boxes of 64 channels x box_rows with the 128-byte
// swizzle; rows past the end read as zero.
static bool sk_make_map(CUtensorMap* map, const void* basep, uint64_t rows, uint64_t K, long long ld, uint32_t box_rows) {
  sk_encode_fn enc = sk_encoder();
  if (!enc || rows == 0 || K == 0 || ld <= 0) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kSkStep, box_rows}, estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(basep), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int kT>
static int sk_launch(const CUtensorMap& tm_w, const CUtensorMap& tm_x, uint16_t* y, long long ldy, int M, int N, int K, int S,
                     int32_t* status, cudaStream_t stream) {
  constexpr size_t smem = (size_t)kSkStages * (kSkWBytes + kT * kSkStep * 2) + 1024 /* alignment slack */ + 256 /* barriers */;
  static_assert(smem >= (size_t)kT * kSkRows * 4 + 1024, "the receive area of the cluster reduction reuses the slots");
  if (cudaFuncSetAttribute(skinny_linear_kernel<kT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return B200KV_E_LAUNCH;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(N / kSkRows, S);
  cfg.blockDim = dim3(kSkThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (S > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = S;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (chained_launch_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, skinny_linear_kernel<kT>, tm_w, tm_x, y, ldy, M, K, S, status);
  return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? B200KV_OK : B200KV_E_LAUNCH;
}

}  // namespace b200kv

using namespace b200kv;

extern "C" int b200kv_skinny_linear(const void* x, int64_t ldx, const void* w, int64_t ldw, void* y, int64_t ldy, int32_t M,
                                    int32_t N, int32_t K, int32_t splits, int32_t* status, void* stream) {
  if (M == 0 || N == 0) return B200KV_OK;
  if (!x || !w || !y) return B200KV_E_NULL;
  if (M < 0 || M > 64 || N < 0 || (N % kSkRows) || K < kSkStep || (K % kSkStep)) return B200KV_E_SHAPE;
  if (splits != 1 && splits != 2 && splits != 4 && splits != 8) return B200KV_E_SHAPE;
  const int T = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  if (splits > T / 2 || splits > K / kSkStep) return B200KV_E_SHAPE;
  if (!aligned(x, 16) || !aligned(w, 16) || !aligned(y, 2) || (ldx % 8) || (ldw % 8) || ldx < K || ldw < K || ldy < N)
    return B200KV_E_ALIGN;
  CUtensorMap tm_w, tm_x;
  if (!sk_make_map(&tm_w, w, (uint64_t)N, (uint64_t)K, ldw, kSkRows) || !sk_make_map(&tm_x, x, (uint64_t)M, (uint64_t)K, ldx, (uint32_t)T))
    return B200KV_E_LAUNCH;
  cudaStream_t s = (cudaStream_t)stream;
  if (T == 16) return sk_launch<16>(tm_w, tm_x, (uint16_t*)y, ldy, M, N, K, splits, status, s);
  if (T == 32) return sk_launch<32>(tm_w, tm_x, (uint16_t*)y, ldy, M, N, K, splits, status, s);
  return sk_launch<64>(tm_w, tm_x, (uint16_t*)y, ldy, M, N, K, splits, status, s);
}
