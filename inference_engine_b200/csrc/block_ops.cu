// The two element-wise ops of the decoder block that sit between the attention path and the GEMMs:
// silu_mul (qwen3-1.7b/kernels.py:1178-1212) and add_rms_norm (kernels.py:1215-1285).  Both are
// HBM-bound streaming kernels: 16-byte loads and stores, fp32 arithmetic in the reference's order, results
// rounded to bf16 once.
#include "common.cuh"

namespace b200kv {

constexpr int kBoThreads = 256;
constexpr int kBoVec = 8;        // bf16 per 16-byte access
constexpr int kBoMaxChunks = 4;  // add_rms_norm keeps a row in registers: D <= 256 * 8 * 4 = 8192

__device__ __forceinline__ void bo_unpack(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ uint4 bo_pack(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) w[i] = float_to_bf16_bits(f[2 * i]) | (float_to_bf16_bits(f[2 * i + 1]) << 16);
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// grid (N, ceil(D / 2048)): out[row, d] = bf16((gate * sigmoid(gate)) * up), gate = in[row, d], up = in[row, D + d]
__global__ void __launch_bounds__(kBoThreads)
silu_mul_kernel(const uint16_t* __restrict__ in, long long in_stride, uint16_t* __restrict__ out, long long out_stride,
                int D) {
  pdl_enter();
  const int col = (blockIdx.y * kBoThreads + threadIdx.x) * kBoVec;
  if (col >= D) return;
  pdl_wait();  // the input comes from the kernel before this one
  const uint16_t* row = in + (long long)blockIdx.x * in_stride;
  float g[8], u[8], y[8];
  bo_unpack(*reinterpret_cast<const uint4*>(row + col), g);
  bo_unpack(*reinterpret_cast<const uint4*>(row + D + col), u);
#pragma unroll
  for (int i = 0; i < 8; ++i) y[i] = (g[i] * (1.0f / (1.0f + __expf(-g[i])))) * u[i];
  *reinterpret_cast<uint4*>(out + (long long)blockIdx.x * out_stride + col) = bo_pack(y);
}

// grid (N), one CTA per row: new_residual = bf16(residual + delta); normed = bf16((new_residual * inv_rms) * w)
// with inv_rms = 1 / sqrt(sum(new_residual^2) / D + eps) over the bf16-rounded new residual.
__global__ void __launch_bounds__(kBoThreads)
add_rms_norm_kernel(const uint16_t* __restrict__ residual, long long r_stride, const uint16_t* __restrict__ delta,
                    long long d_stride, const uint16_t* __restrict__ weight, uint16_t* __restrict__ new_residual,
                    long long nr_stride, uint16_t* __restrict__ normed, long long nn_stride, int D, float eps) {
  __shared__ float part[kBoThreads / 32];
  pdl_enter();
  pdl_wait();  // residual and delta come from the kernels before this one
  const long long n = blockIdx.x;
  float r[kBoMaxChunks][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < kBoMaxChunks; ++c) {
    const int col = (c * kBoThreads + threadIdx.x) * kBoVec;
    if (col < D) {
      float a[8], b[8];
      bo_unpack(*reinterpret_cast<const uint4*>(residual + n * r_stride + col), a);
      bo_unpack(*reinterpret_cast<const uint4*>(delta + n * d_stride + col), b);
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] += b[i];
      const uint4 packed = bo_pack(a);
      *reinterpret_cast<uint4*>(new_residual + n * nr_stride + col) = packed;
      bo_unpack(packed, r[c]);  // the sum runs over the rounded values (kernels.py:1245-1249)
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(r[c][i], r[c][i], ss);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kBoThreads / 32; ++i) tot += part[i];
  const float inv = 1.0f / sqrtf(tot / (float)D + eps);
#pragma unroll
  for (int c = 0; c < kBoMaxChunks; ++c) {
    const int col = (c * kBoThreads + threadIdx.x) * kBoVec;
    if (col < D) {
      float w[8], y[8];
      bo_unpack(*reinterpret_cast<const uint4*>(weight + col), w);
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = (r[c][i] * inv) * w[i];
      *reinterpret_cast<uint4*>(normed + n * nn_stride + col) = bo_pack(y);
    }
  }
}

}  // namespace b200kv

using namespace b200kv;

extern "C" int b200kv_silu_mul(const void* gate_up, int64_t in_stride, void* out, int64_t out_stride, int32_t N, int32_t D,
                               void* stream) {
  // an empty batch is valid and has nothing to launch (its tensors have no storage, so their pointers are NULL)
  if (N == 0) return B200KV_OK;
  if (!gate_up || !out) return B200KV_E_NULL;
  if (N < 0 || D < 1 || D % kBoVec) return B200KV_E_SHAPE;
  if (!aligned(gate_up, 16) || !aligned(out, 16) || in_stride % kBoVec || out_stride % kBoVec) return B200KV_E_ALIGN;
  if (N == 0) return B200KV_OK;
  const unsigned gy = (unsigned)((D + kBoThreads * kBoVec - 1) / (kBoThreads * kBoVec));
  if (gy > 65535u) return B200KV_E_RANGE;
  const cudaError_t e = launch_chained(silu_mul_kernel, dim3((unsigned)N, gy), dim3(kBoThreads), 0, (cudaStream_t)stream,
                                       (const uint16_t*)gate_up, in_stride, (uint16_t*)out, out_stride, D);
  return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? B200KV_OK : B200KV_E_LAUNCH;
}

extern "C" int b200kv_add_rms_norm(const void* residual, int64_t r_stride, const void* delta, int64_t d_stride,
                                   const void* weight, void* new_residual, int64_t nr_stride, void* normed,
                                   int64_t nn_stride, int32_t N, int32_t D, float eps, void* stream) {
  // an empty batch is valid and has nothing to launch (its tensors have no storage, so their pointers are NULL)
  if (N == 0) return B200KV_OK;
  if (!residual || !delta || !weight || !new_residual || !normed) return B200KV_E_NULL;
  if (N < 0 || D < 1 || D % kBoVec) return B200KV_E_SHAPE;
  if (D > kBoThreads * kBoVec * kBoMaxChunks) return B200KV_E_RANGE;
  if (!aligned(residual, 16) || !aligned(delta, 16) || !aligned(weight, 16) || !aligned(new_residual, 16) ||
      !aligned(normed, 16) || r_stride % kBoVec || d_stride % kBoVec || nr_stride % kBoVec || nn_stride % kBoVec)
    return B200KV_E_ALIGN;
  if (N == 0) return B200KV_OK;
  const cudaError_t e = launch_chained(add_rms_norm_kernel, dim3((unsigned)N), dim3(kBoThreads), 0, (cudaStream_t)stream,
                                       (const uint16_t*)residual, r_stride, (const uint16_t*)delta, d_stride,
                                       (const uint16_t*)weight, (uint16_t*)new_residual, nr_stride, (uint16_t*)normed,
                                       nn_stride, D, eps);
  return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? B200KV_OK : B200KV_E_LAUNCH;
}
