// Shared device/host helpers for the b200kv kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "b200kv.h"

namespace b200kv {

constexpr int kD = 128;       // head_dim the kernels are specialised for
constexpr int kHalfD = 64;

// Device-side view of the cache + page table, passed to kernels by value.
struct CacheView {
  int8_t* k;
  int8_t* v;
  float* k_scale;
  float* v_scale;
  float* k_cal;
  long long stride_page, stride_head, stride_tok;
  long long sstride_page, sstride_head;
  long long cstride_page, cstride_head;
  int num_pages, Hkv, page_size;
  int page_shift;  // log2(page_size) when that is a power of two, else -1 (split_pos divides)
  const int32_t* table;
  int table_stride, max_pages;
};

inline CacheView make_view(const b200kv_cache* c, const b200kv_table* t) {
  CacheView w;
  w.k = c->k; w.v = c->v; w.k_scale = c->k_scale; w.v_scale = c->v_scale; w.k_cal = c->k_calibration;
  w.stride_page = c->stride_page; w.stride_head = c->stride_head; w.stride_tok = c->stride_tok;
  w.sstride_page = c->sstride_page; w.sstride_head = c->sstride_head;
  w.cstride_page = c->cstride_page; w.cstride_head = c->cstride_head;
  w.num_pages = c->num_pages; w.Hkv = c->num_kv_heads; w.page_size = c->page_size;
  w.page_shift = -1;
  for (int sft = 0; sft < 31; ++sft)
    if (c->page_size == (1 << sft)) w.page_shift = sft;
  w.table = t->ids; w.table_stride = t->stride; w.max_pages = t->max_pages;
  return w;
}

// Chained launches (programmatic dependent launch).  Every kernel of the path (a) waits for the kernel launched
// before it on the stream (pdl_wait) before it reads anything that kernel may have written or writes global
// memory itself, having read at most caller-provided metadata by then, and (b) tells the stream when the next
// kernel may be brought up (pdl_trigger).  Both are no-ops for a kernel launched the ordinary way; the launch
// attribute is only set while b200kv_set_chained_launch(1) is in force.
bool chained_launch_enabled();
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// First statement of every kernel.  The trigger may come this early: the next kernel cannot be brought up before
// every CTA of this grid has executed it (or exited), so it only ever takes resources this grid has no use for
// any more.  The first CTA of the grid waits at once, on every path: a grid in which no CTA waited could
// complete before its predecessor, and the kernel after it only waits for THIS grid.
__device__ __forceinline__ void pdl_enter() {
  pdl_trigger();
  if ((blockIdx.x | blockIdx.y | blockIdx.z) == 0) pdl_wait();
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chained_launch_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Host-side validation shared by the entry points.  Returns B200KV_OK or an error code.
inline int check_cache(const b200kv_cache* c, const b200kv_table* t) {
  if (!c || !t || !c->k || !c->v || !c->k_scale || !c->v_scale || !c->k_calibration || !t->ids) return B200KV_E_NULL;
  if (c->head_dim != kD || c->num_kv_heads < 1 || c->page_size < 1 || c->num_pages < 1) return B200KV_E_SHAPE;
  if (t->max_pages < 1 || t->stride < 0) return B200KV_E_SHAPE;
  // a 16-token tile must not straddle pages; a single page per entry may have any length
  if (t->max_pages > 1 && (c->page_size % 16) != 0) return B200KV_E_SHAPE;
  if (!aligned(c->k, 16) || !aligned(c->v, 16) || !aligned(c->k_scale, 16) || !aligned(c->v_scale, 16) ||
      !aligned(c->k_calibration, 16))
    return B200KV_E_ALIGN;
  if (c->stride_tok < kD || (c->stride_tok % 16) || (c->stride_head % 16) || (c->stride_page % 16)) return B200KV_E_ALIGN;
  if ((c->sstride_head % 4) || (c->sstride_page % 4) || (c->cstride_head % 4) || (c->cstride_page % 4)) return B200KV_E_ALIGN;
  // the kernels multiply ids by strides in 32 x 32 -> 64 bit arithmetic
  const int64_t strides[] = {c->stride_page, c->stride_head, c->stride_tok, c->sstride_page, c->sstride_head,
                             c->cstride_page, c->cstride_head};
  for (int64_t s : strides)
    if (s < 0 || s > 0x7fffffffLL) return B200KV_E_RANGE;
  return B200KV_OK;
}

// Token position -> (table column, row inside the page).
__device__ __forceinline__ void split_pos(const CacheView& c, int pos, int& slot, int& prow) {
  if (c.page_shift >= 0) {
    slot = pos >> c.page_shift;
    prow = pos & (c.page_size - 1);
  } else {
    slot = pos / c.page_size;
    prow = pos - slot * c.page_size;
  }
}
// Element offsets into the cache tensors.  Every stride is below 2^31 (check_cache), so each product is one
// 32 x 32 -> 64 bit multiply-add, and the part inside a page fits 32 bits.
__device__ __forceinline__ long long code_offset(const CacheView& c, int page, int head, int prow) {
  return (long long)page * (int)c.stride_page + (head * (int)c.stride_head + prow * (int)c.stride_tok);
}
__device__ __forceinline__ long long scale_offset(const CacheView& c, int page, int head, int prow) {
  return (long long)page * (int)c.sstride_page + (head * (int)c.sstride_head + prow);
}
__device__ __forceinline__ long long cal_offset(const CacheView& c, int page, int head) {
  return (long long)page * (int)c.cstride_page + head * (int)c.cstride_head;
}
// Row r, head j of a packed activation tensor whose strides (elements) are below 2^31 (checked on the host).
__device__ __forceinline__ long long act_offset(int r, long long s_row, int j, long long s_head) {
  return (long long)r * (int)s_row + j * (int)s_head;
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

__device__ __forceinline__ uint32_t float_to_bf16_bits(float x) {
  return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(x)));
}

// Page id of token position `pos` of entry b, or -1 (and a status bit) when out of range.
__device__ __forceinline__ int lookup_page(const CacheView& c, int b, int pos, int32_t* status) {
  int slot, prow;
  split_pos(c, pos, slot, prow);
  if (pos < 0 || slot >= c.max_pages) {
    if (status) atomicOr(status, B200KV_S_BAD_POSITION);
    return -1;
  }
  int page = c.table[(long long)b * c.table_stride + slot];
  if (page < 0 || page >= c.num_pages) {
    if (status) atomicOr(status, B200KV_S_BAD_PAGE);
    return -1;
  }
  return page;
}

}  // namespace b200kv
