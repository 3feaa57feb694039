// Gumbel-max sampling over the vocabulary, two stages like the reference (qwen3-1.7b/kernels.py:1286-1370):
// stage 1 takes the best (value, index) of every block of 2048 columns, stage 2 the best block.  tau = 0 is
// greedy argmax.  token[b] = the FIRST index attaining max_v (logits[b,v] + tau * -log(-log(u))), with
// u = clamp(uniform(seed, b * V + v), 1e-10, 1 - 1e-7).  The uniform is the one Triton's tl.rand gives the
// reference: first word of Philox-4x32-10 (Salmon et al., SC'11) for counter (b * V + v, 0, 0, 0) and the
// 64-bit seed as key, read as a signed int32 x, folded to non-negative (x < 0 -> -x - 1), converted to fp32 and
// multiplied by 4.6566127342e-10.  Products and sums are rounded separately (no FMA contraction), so the
// noisy logits are the fp32 values the reference computes.
#include "common.cuh"

namespace b200kv {

constexpr int kSmThreads = 256;
constexpr int kSmBlock = 2048;  // columns per stage-1 CTA

__device__ __forceinline__ uint32_t philox_first_word(uint32_t c0, uint32_t k0, uint32_t k1) {
  uint32_t c1 = 0, c2 = 0, c3 = 0;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t h0 = __umulhi(0xD2511F53u, c0), l0 = 0xD2511F53u * c0;
    const uint32_t h1 = __umulhi(0xCD9E8D57u, c2), l1 = 0xCD9E8D57u * c2;
    c0 = h1 ^ c1 ^ k0;
    c1 = l1;
    c2 = h0 ^ c3 ^ k1;
    c3 = l0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c0;
}

__device__ __forceinline__ float noisy_logit(float logit, float tau, uint32_t word) {
  int x = (int)word;
  x = x < 0 ? -x - 1 : x;
  float u = __fmul_rn((float)x, 4.6566127342e-10f);
  u = fminf(fmaxf(u, 1e-10f), (float)(1.0 - 1e-7));
  return __fadd_rn(logit, __fmul_rn(tau, -logf(-logf(u))));
}

// the better of two candidates: the larger value, on a tie the smaller index
__device__ __forceinline__ void take_better(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

__device__ __forceinline__ void block_best(float& v, int& i) {
  __shared__ float sv[kSmThreads / 32];
  __shared__ int si[kSmThreads / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) take_better(v, i, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, i, o));
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = v; si[threadIdx.x >> 5] = i; }
  __syncthreads();
  if (threadIdx.x < 32) {
    v = threadIdx.x < kSmThreads / 32 ? sv[threadIdx.x] : -INFINITY;
    i = threadIdx.x < kSmThreads / 32 ? si[threadIdx.x] : 0x7FFFFFFF;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) take_better(v, i, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, i, o));
  }
}

// grid (B, ceil(V / 2048)).  logits bf16 (elem_bytes 2) or fp32 (4), row stride in elements.
__global__ void __launch_bounds__(kSmThreads)
sample_stage1_kernel(const void* __restrict__ logits, long long stride, int elem_bytes, const long long* __restrict__ seed,
                     float tau, float* __restrict__ part_val, int* __restrict__ part_idx, int V) {
  pdl_enter();
  pdl_wait();  // the logits (and the seed, advanced by the previous call) come from the kernels before this one
  const int b = blockIdx.x, nblk = gridDim.y;
  const unsigned long long s = (unsigned long long)*seed;
  const uint32_t k0 = (uint32_t)s, k1 = (uint32_t)(s >> 32);
  float best = -INFINITY;
  int idx = 0x7FFFFFFF;
#pragma unroll
  for (int j = 0; j < kSmBlock / kSmThreads; ++j) {
    const int v = blockIdx.y * kSmBlock + j * kSmThreads + threadIdx.x;
    if (v < V) {
      const float x = elem_bytes == 2
                          ? bf16_bits_to_float(reinterpret_cast<const uint16_t*>(logits)[(long long)b * stride + v])
                          : reinterpret_cast<const float*>(logits)[(long long)b * stride + v];
      const float z = noisy_logit(x, tau, philox_first_word((uint32_t)(b * V + v), k0, k1));
      if (z > best) { best = z; idx = v; }  // columns ascend per thread: the first maximum stays
    }
  }
  block_best(best, idx);
  if (threadIdx.x == 0) { part_val[b * nblk + blockIdx.y] = best; part_idx[b * nblk + blockIdx.y] = idx; }
}

// grid (B).  The seed advances by one per call (kernels.py:1369), here, after every stage-1 CTA has read it.
__global__ void __launch_bounds__(kSmThreads)
sample_stage2_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx, int nblk, long long* __restrict__ out,
                     long long out_stride, long long* __restrict__ seed) {
  pdl_enter();
  pdl_wait();
  const int b = blockIdx.x;
  float best = -INFINITY;
  int idx = 0x7FFFFFFF;
  for (int j = threadIdx.x; j < nblk; j += kSmThreads) take_better(best, idx, part_val[b * nblk + j], part_idx[b * nblk + j]);
  block_best(best, idx);
  if (threadIdx.x == 0) {
    out[b * out_stride] = idx;
    if (b == 0) *seed += 1;
  }
}

}  // namespace b200kv

using namespace b200kv;

extern "C" size_t b200kv_sample_workspace_bytes(int32_t B, int32_t V) {
  const size_t nblk = ((size_t)V + kSmBlock - 1) / kSmBlock;
  return (size_t)B * nblk * 8;  // one fp32 and one int32 per (row, block)
}

extern "C" int b200kv_sample(const void* logits, int64_t stride, int32_t elem_bytes, int64_t* seed, float tau, void* workspace,
                             size_t workspace_bytes, int64_t* out, int64_t out_stride, int32_t B, int32_t V, void* stream) {
  // an empty batch is valid and has nothing to launch (its tensors have no storage, so their pointers are NULL)
  if (B == 0) return B200KV_OK;
  if (!logits || !seed || !workspace || !out) return B200KV_E_NULL;
  if (B < 0 || V < 1 || (elem_bytes != 2 && elem_bytes != 4)) return B200KV_E_SHAPE;
  if ((long long)B * V > 0x7FFFFFFFll) return B200KV_E_RANGE;  // the counter b * V + v is 32-bit, as in the reference
  if (workspace_bytes < b200kv_sample_workspace_bytes(B, V)) return B200KV_E_WORKSPACE;
  if (!aligned(workspace, 8) || !aligned(logits, elem_bytes)) return B200KV_E_ALIGN;
  if (B == 0) return B200KV_OK;
  const int nblk = (V + kSmBlock - 1) / kSmBlock;
  if (nblk > 65535) return B200KV_E_RANGE;
  float* pv = (float*)workspace;
  int* pi = (int*)(pv + (size_t)B * nblk);
  cudaError_t e = launch_chained(sample_stage1_kernel, dim3((unsigned)B, (unsigned)nblk), dim3(kSmThreads), 0,
                                 (cudaStream_t)stream, logits, stride, (int)elem_bytes, (const long long*)seed, tau, pv, pi, (int)V);
  if (e != cudaSuccess || cudaGetLastError() != cudaSuccess) return B200KV_E_LAUNCH;
  e = launch_chained(sample_stage2_kernel, dim3((unsigned)B), dim3(kSmThreads), 0, (cudaStream_t)stream, (const float*)pv,
                     (const int*)pi, nblk, (long long*)out, out_stride, (long long*)seed);
  return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? B200KV_OK : B200KV_E_LAUNCH;
}
