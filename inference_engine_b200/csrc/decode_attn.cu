// Split-K GQA decode attention over the paged int8 KV cache (sm_100a), with in-kernel
// dequantization and a cross-split log-sum-exp reduction.  Replaces the reference's
// decode_attention_kernel + decode_attention_combine_kernel (qwen3-1.7b/kernels.py:83-264).
//
// Work decomposition (device side, from cached_lens/num_decoding only, so the grid is a
// function of shapes and the call is graph-capturable):
//   * the unit of work is a TILE of 16 tokens of one (entry, kv head);
//   * all tiles of the batch are laid end to end in (entry, kv head, tile) order and cut into
//     equal contiguous ranges, one per WARP of a persistent grid (sm_count * kCtasPerSm CTAs of
//     kWarps warps).  Every warp therefore streams the same number of bytes (+-1 tile);
//   * a warp walks its range; whenever it finishes its part of an (entry, head) it either
//     writes the final bf16 output (it saw the whole sequence) or an fp32 partial
//     (acc, m, l) into one of its two workspace slots; the four warps of a CTA that hold pieces
//     of the same (entry, head) add them in shared memory first;
//   * the warp that delivers the last piece of an (entry, head) merges all of them (an arrival
//     counter per (entry, head) in the workspace); `variant` bit 1 leaves the merge to a second
//     small kernel instead, as the reference does;
//   * the split can be read from a per-step plan (decode_plan_kernel) instead of being
//     re-derived by every CTA of every layer's call.
//
// Data movement: every warp owns a private ring of kStages tiles in shared memory, filled
// with 16-byte cp.async copies (K tile 2 KB, V tile 2 KB, 2 x 16 scales) that complete in the
// background; no block-level barrier exists anywhere in the main loop.  Each token row is
// 128 contiguous bytes, a (page, head) tile is 2 KB contiguous, so every copy is coalesced.
//
// Arithmetic (variant 0, the product path): both contractions run on the tensor cores.
//     S[head, tok] = q[head, :] . K[tok, :]   int8 x int8 -> int32, mma.m16n8k32.  q is split once
//                    per segment into two int8 terms (rows 0-7: high term of heads 0-7, rows 8-15:
//                    low term), the RAW code words of 8 tokens are the B fragment, straight from one
//                    16-byte shared-memory read, with no conversion at all.  Lane (g,t) ends up with
//                    the scores of head g for tokens 2t, 2t+1, 2t+8, 2t+9 - exactly the P' fragment
//                    the second contraction wants, so no shuffles sit between the two.
//     O^T[d, head] += V^T[d, tok] . P'[tok, head]   fp16 x fp16 -> fp32, mma.m16n8k16.  Codes are
//                    widened exactly with byte permutes (0x6400 | (code ^ 0x80) == 1152 + code); the
//                    offset is taken out of O every kDebiasTiles tiles as 1152 x the sum of P'
//                    (mma_debias); P' = p * v_scale.
// Softmax state is fp32 in registers; scores use exp2 with log2(e) folded into the scale.
// Variant 1 does the same with fp32 FMAs on the CUDA cores and exists for cross-checking.
#include <algorithm>
#include <type_traits>

#include "common.cuh"

namespace b200kv {

constexpr int kTile = 16;                 // tokens per tile
constexpr int kWarps = 4;                 // warps per CTA
constexpr int kCtasPerSm = 3;
constexpr int kStages = 4;                // tiles in flight per warp
constexpr int kTileBytes = 2 * kTile * kD + 2 * kTile * 4;  // K, V codes + K, V scales = 4224
constexpr int kDeepTiles = 224;           // tiles per warp from which the full look-ahead of the ring pays
constexpr int kShallowFloor = 8;          // ... and up to which a warp's few tiles are all requested at once
constexpr int kMaxG = 8;                  // query heads per kv head the MMA n-dimension can hold
constexpr int kMaxB = 1 << 20;
static_assert((kStages & (kStages - 1)) == 0, "ring indices are masked");

struct Partition {
  int U;        // total tiles over all (entry, head)
  int per;      // tiles per worker
  int W;        // workers (warps in the grid)
};

// ------------------------------------------------------------------ small PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <int kOff>
__device__ __forceinline__ void cp_async16_imm(uint32_t dst, const void* src) {  // both addresses + kOff bytes
  asm volatile("cp.async.cg.shared.global [%0+%2], [%1+%2], 16;\n" ::"r"(dst), "l"(src), "n"(kOff) : "memory");
}
// D += A(16x32, row, s8) * B(32x8, col, s8), s32 accumulate.
__device__ __forceinline__ void imma16832(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// D += A(16x16, row) * B(16x8, col), fp16 inputs, fp32 accumulate.
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Arrival on a counter in global memory with release (my stores before it) and acquire (others' stores after it)
// semantics at device scope, in one instruction.
__device__ __forceinline__ int atom_add_acq_rel(int* addr, int v) {
  int old;
  asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], %2;" : "=r"(old) : "l"(addr), "r"(v) : "memory");
  return old;
}

// ------------------------------------------------------------------ partition (all CTAs agree)
constexpr int kSmemLens = 512;  // token counts of the first entries are kept in shared memory

// Tokens each entry attends (cached_len + 1; 0 past num_decoding), from shared memory for the
// first kSmemLens entries (no global round trip when a warp positions itself), else from global.
struct Lens {
  const int32_t* __restrict__ g;
  const int* s;
  int nd;
  __device__ __forceinline__ int n(int b) const { return b < kSmemLens ? s[b] : (b < nd ? g[b] + 1 : 0); }
  __device__ __forceinline__ int tiles(int b) const { return (n(b) + kTile - 1) / kTile; }
};

// Tiles per kv head of entries [0,B), scanned by the whole CTA.  Thread i owns the `chunk`
// consecutive entries starting at i*chunk; chunk_prefix[i] (shared, blockDim.x+1 ints) is the
// number of tiles before that chunk, chunk_prefix[blockDim.x] the total; lens_s receives the
// token counts of the first kSmemLens entries.  The loads of cached_lens do not wait for
// num_decoding (it only masks them).  When `gprefix` is given (one CTA does this) the per-entry
// exclusive prefix [B+1] is also written to global memory for the separate reduction kernel.
__device__ void scan_tiles(const int32_t* __restrict__ cached_lens, int B, const int32_t* __restrict__ num_decoding,
                           int chunk, int* chunk_prefix, int* lens_s, int* __restrict__ gprefix, int& nd_out) {
  const int tid = threadIdx.x, nt = blockDim.x;
  const int lo = min(tid * chunk, B), hi = min(lo + chunk, B);
  const int nd_raw = *num_decoding;
  int first = lo < hi ? cached_lens[lo] : 0;  // issued together with the load above
  const int nd = min(nd_raw, B);
  int sum = 0;
  for (int b = lo; b < hi; ++b) {
    const int cl = b == lo ? first : cached_lens[b];
    const int n = b < nd ? cl + 1 : 0;
    if (b < kSmemLens) lens_s[b] = n;
    sum += (n + kTile - 1) / kTile;
  }
  chunk_prefix[tid] = sum;
  __syncthreads();
  if (tid < 32) {  // exclusive scan of the nt chunk sums by one warp
    int carry = 0;
    for (int base = 0; base < nt; base += 32) {
      int v = (base + tid < nt) ? chunk_prefix[base + tid] : 0;
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int y = __shfl_up_sync(0xffffffffu, incl, o);
        if (tid >= o) incl += y;
      }
      if (base + tid < nt) chunk_prefix[base + tid] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (tid == 0) chunk_prefix[nt] = carry;
  }
  __syncthreads();
  if (gprefix) {
    int run = chunk_prefix[tid];
    for (int b = lo; b < hi; ++b) {
      gprefix[b] = run;
      run += (b < nd ? (cached_lens[b] + 1 + kTile - 1) / kTile : 0);
    }
    if (tid == 0) gprefix[B] = chunk_prefix[nt];
  }
  nd_out = nd;
}

// `per` = tiles per warp.  Never below the even share; the floor below it trades parallelism against
// hand-offs: a piece that goes through the workspace costs about as much as 8 tiles of work, but the four pieces
// of a CTA that covers exactly one (entry, head) meet in shared memory and cost nothing of the kind.  So short
// sequences (32 tiles or fewer on average) are cut into quarters of the average length (2..8 tiles) when the grid
// has warps to spare for that: in a batch of equal lengths every CTA then owns exactly one (entry, head), and its
// four warps fetch the few tiles side by side instead of one warp streaming all of them (5.8 instead of 10.3 us
// for one 128-token sequence).  When the quarters would not fit the grid, short sequences use pieces of 8 tiles
// (a whole sequence per warp, or exactly a CTA of 4 x 8); longer ones pieces of 4 (64 tokens, the reference's
// MIN_PIECE, kernels.py:295).
__host__ __device__ __forceinline__ Partition make_partition(int total_tiles_one_head, int Hkv, int W, int num_entries) {
  Partition p;
  p.U = total_tiles_one_head * Hkv;
  p.W = W;
  const int share = (p.U + W - 1) / W;
  int min_tiles = 4;
  if (num_entries > 0 && total_tiles_one_head <= 32 * num_entries) {
    int quarter = (total_tiles_one_head + 4 * num_entries - 1) / (4 * num_entries);  // <= 8
    if (quarter < 2) quarter = 2;
    min_tiles = share <= quarter ? quarter : 8;
  }
  p.per = share > min_tiles ? share : min_tiles;
  return p;
}

// Position in the flattened (entry, head, tile) list.  (slot, row0) locate the tile in the
// entry's page table (table column and first row inside that page); they advance incrementally
// so the hot loop never divides.
struct Cursor {
  int b, h, tile, T, n, slot, row0, base;  // base: flat index of (entry b, head 0, tile 0)
  __device__ __forceinline__ void seek(const int* chunk_prefix, int nchunks, int chunk, const Lens& lens, int Hkv,
                                       int page_size, int u) {
    int lo = 0, hi = nchunks;  // largest chunk whose first flat index is <= u
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (Hkv * chunk_prefix[mid] <= u) lo = mid; else hi = mid;
    }
    b = lo * chunk;
    int run = chunk_prefix[lo];
    while (true) {
      T = lens.tiles(b);
      if (Hkv * (run + T) > u) break;
      run += T;
      ++b;
    }
    n = lens.n(b);
    base = Hkv * run;
    int r = u - base;
    h = r / T;
    tile = r - h * T;
    slot = (tile * kTile) / page_size;
    row0 = tile * kTile - slot * page_size;
  }
  // First tile of the next (entry, head); only called while one exists.
  __device__ __forceinline__ void next_segment(const Lens& lens, int Hkv) {
    tile = 0; slot = 0; row0 = 0;
    if (++h < Hkv) return;
    h = 0;
    base += Hkv * T;
    do { ++b; T = lens.tiles(b); } while (T == 0);
    n = lens.n(b);
  }
  // Next tile in flat order; only called while one exists.
  __device__ __forceinline__ void next(const Lens& lens, int Hkv, int page_size) {
    if (++tile < T) {
      row0 += kTile;
      const bool wrap = row0 >= page_size;
      row0 = wrap ? 0 : row0;
      slot += wrap ? 1 : 0;
      return;
    }
    next_segment(lens, Hkv);
  }
};

// ------------------------------------------------------------------ producer: one tile -> smem
// Shared-memory tile (4224 B): K codes [16][128] with 16-byte chunk c of row r stored at chunk
// c ^ (4*(r&1)); V codes [16][128] with chunk c of row r at c ^ (r&6); then k_scale[16],
// v_scale[16].  The swizzles make the consumer's 16-byte fragment reads conflict-free.
struct PageWindow {
  int b, base, reg;  // `reg` of lane i holds table[b][base + i]
};

// Per-lane constants of the copy pattern: a lane moves 16-byte chunk (lane & 7) of rows
// (lane >> 3) + 4i, i = 0..3.  The K swizzle is invariant under row += 4; the V swizzle flips
// chunk bit 2, hence two V offsets (even / odd i).
struct LaneCopy {
  uint32_t k_dst, v_dst[2], s_dst;  // shared-memory byte offsets inside a stage (for i = 0 / 1)
  long long g_off, g_step;          // global byte offsets inside a (page, head) tile
  int r0, srow;
};

__device__ __forceinline__ LaneCopy make_lane_copy(const CacheView& c, int lane) {
  LaneCopy lc;
  lc.r0 = lane >> 3;
  const int col = lane & 7;
  lc.k_dst = lc.r0 * kD + ((col ^ ((lc.r0 & 1) << 2)) << 4);
  lc.v_dst[0] = kTile * kD + lc.r0 * kD + ((col ^ (lc.r0 & 6)) << 4);
  lc.v_dst[1] = kTile * kD + lc.r0 * kD + ((col ^ ((lc.r0 + 4) & 6)) << 4);
  lc.s_dst = 2 * kTile * kD + lane * 4;
  lc.g_off = lc.r0 * c.stride_tok + col * 16;
  lc.g_step = 4 * c.stride_tok;
  lc.srow = lane & 15;
  return lc;
}

// Page id of the cursor's tile from the lane-distributed window of the entry's table row (reloaded when the
// cursor leaves it); -2 when the tile lies beyond the table.
__device__ __forceinline__ void load_window(const CacheView& c, int b, int slot, PageWindow& win, int lane) {
  win.b = b;
  win.base = slot & ~31;
  const int idx = win.base + lane;
  win.reg = (idx < c.max_pages) ? c.table[(long long)b * c.table_stride + idx] : -2;
}
__device__ __forceinline__ int window_page(const CacheView& c, const Cursor& cur, PageWindow& win, int lane) {
  const int slot = cur.slot;
  if (cur.b != win.b || slot < win.base || slot >= win.base + 32) load_window(c, cur.b, slot, win, lane);
  return __shfl_sync(0xffffffffu, win.reg, slot - win.base);
}

__device__ __forceinline__ void issue_tile(const CacheView& c, const Cursor& cur, int page, const LaneCopy& lc,
                                           uint32_t sbase, int lane, int32_t* status) {
  const int nvalid = cur.n - cur.tile * kTile;  // >= 1; >= 16 for every tile but a sequence's last
  const bool ok = page >= 0 && page < c.num_pages;
  if (!ok) {
    if (lane == 0 && status) atomicOr(status, page == -2 ? B200KV_S_BAD_POSITION : B200KV_S_BAD_PAGE);
    page = 0;
  }
  // strides fit 32 bits (checked on the host): each product is one widening multiply-add
  const long long code_off = (long long)page * (int)c.stride_page + (long long)cur.h * (int)c.stride_head +
                             (cur.row0 * (int)c.stride_tok + (int)lc.g_off);
  const int8_t* ksrc = c.k + code_off;
  const int8_t* vsrc = c.v + code_off;
  const float* ssrc = (lane < 16 ? c.k_scale : c.v_scale) +
                      ((long long)page * (int)c.sstride_page + (long long)cur.h * (int)c.sstride_head + cur.row0);
  if (ok && nvalid >= kTile) {  // the common case: a full tile, no predicates
    if (c.stride_tok == kD) {   // rows are contiguous: 4 rows further is +512 bytes on both sides
      cp_async16_imm<0>(sbase + lc.k_dst, ksrc);
      cp_async16_imm<512>(sbase + lc.k_dst, ksrc);
      cp_async16_imm<1024>(sbase + lc.k_dst, ksrc);
      cp_async16_imm<1536>(sbase + lc.k_dst, ksrc);
      cp_async16_imm<0>(sbase + lc.v_dst[0], vsrc);
      cp_async16_imm<512>(sbase + lc.v_dst[1], vsrc);
      cp_async16_imm<1024>(sbase + lc.v_dst[0], vsrc);
      cp_async16_imm<1536>(sbase + lc.v_dst[1], vsrc);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        cp_async16(sbase + lc.k_dst + 512 * i, ksrc + i * lc.g_step, 16);
        cp_async16(sbase + lc.v_dst[i & 1] + 512 * i, vsrc + i * lc.g_step, 16);
      }
    }
    cp_async4(sbase + lc.s_dst, ssrc + lc.srow, 4);
  } else {  // last tile of a sequence (rows past the end are zero-filled, never read) or a bad page
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const bool valid = ok && (lc.r0 + 4 * i) < nvalid;
      cp_async16(sbase + lc.k_dst + 512 * i, valid ? ksrc + i * lc.g_step : c.k, valid ? 16 : 0);
      cp_async16(sbase + lc.v_dst[i & 1] + 512 * i, valid ? vsrc + i * lc.g_step : c.v, valid ? 16 : 0);
    }
    const bool valid = ok && lc.srow < nvalid;
    cp_async4(sbase + lc.s_dst, valid ? ssrc + lc.srow : c.k_scale, valid ? 4 : 0);
  }
}

// ------------------------------------------------------------------ consumer state (tensor-core variant)
// Lane (g = lane>>2, t = lane&3).  Scores: head g, tokens 2t, 2t+1, 2t+8, 2t+9 of the tile.
// Output accumulators: channels 16g+2j (+1), head columns 2t, 2t+1.
struct MmaState {
  uint32_t qa[4][4];  // A fragments of q for the 4 k-steps: {hi, lo, hi', lo'} words (see mma_begin)
  float sfac;         // head g: softmax_scale * log2(e) * s1 / 128
  float m, l;         // head g: running max (log2 domain, uniform over t) and this lane's share of the sum
  float lv;           // head g: this lane's share of the sum of P' = p * v_scale (as rounded to fp16) since the last
                      // mma_debias, see mma_pv
  float o[8][4];      // O^T accumulators: m-tile j, rows d = 16g+2j (+1), columns 2t, 2t+1
  uint32_t k_off[2], v_off;  // lane-constant shared-memory offsets of the fragment reads
};

// Start of an (entry, head) segment: load head g of the GQA group and split it into two int8
// terms (s1 = absmax/127; hi = rint(q/s1), lo = rint((q - hi*s1) * 128/s1), so
// q ~ s1*(hi + lo/128) with an error below absmax * 2^-15), and reset the softmax state.
// k-step s = 2c+jj covers channels 64c + 16t + 8jj + {0..3} (first k half) and +4 (second half).
__device__ __forceinline__ void mma_begin(MmaState& st, const uint16_t* __restrict__ q, long long q_sb, long long q_sh,
                                          int b, int h, int G, float scale_log2, int lane) {
  const int g = lane >> 2, t = lane & 3;
  float f[32];
  float amax = 0.f;
  if (g < G) {
    const uint16_t* row = q + b * q_sb + (long long)(h * G + g) * q_sh;
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint4 raw = *reinterpret_cast<const uint4*>(row + 64 * c + 16 * t + 8 * half);
        uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          f[16 * c + 8 * half + 2 * i] = bf16_bits_to_float(w[i] & 0xFFFFu);
          f[16 * c + 8 * half + 2 * i + 1] = bf16_bits_to_float(w[i] >> 16);
        }
      }
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(f[i]));
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = 0.f;
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  const float s1 = amax > 0.f ? amax * (1.f / 127.f) : 1.f;
  const float inv = 1.f / s1;
#pragma unroll
  for (int w = 0; w < 8; ++w) {  // word w = channels 64(w>>2) + 16t + 4(w&3) + {0..3}
    uint32_t hi_w = 0, lo_w = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float x = f[4 * w + i];
      const float hi = fminf(fmaxf(rintf(x * inv), -127.f), 127.f);
      const float lo = fminf(fmaxf(rintf((x - hi * s1) * (128.f * inv)), -127.f), 127.f);
      hi_w |= ((uint32_t)(int)hi & 0xFFu) << (8 * i);
      lo_w |= ((uint32_t)(int)lo & 0xFFu) << (8 * i);
    }
    // A fragment of k-step w>>1: a0 = (row g: hi, k 4t..), a1 = (row g+8: lo, k 4t..), a2/a3 = k 16+4t..
    st.qa[w >> 1][2 * (w & 1)] = hi_w;
    st.qa[w >> 1][2 * (w & 1) + 1] = lo_w;
  }
  st.sfac = g < G ? scale_log2 * s1 * (1.f / 128.f) : 0.f;
  st.m = -INFINITY;
  st.l = 0.f;
  st.lv = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) st.o[j][i] = 0.f;
}

__device__ __forceinline__ void mma_init_lane(MmaState& st, int lane) {
  const int g = lane >> 2, t = lane & 3;
  st.k_off[0] = g * kD + ((t ^ ((g & 1) << 2)) << 4);
  st.k_off[1] = g * kD + (((t + 4) ^ ((g & 1) << 2)) << 4);
  st.v_off = kTile * kD + 2 * t * kD + ((g ^ (2 * t)) << 4);
}

// One tile is processed in three steps: scores and softmax bookkeeping (int8 tensor cores), the rescaling of O by
// the tile's correction, and the P.V product (fp16 tensor cores).  (Taking the scores of tile k+1 ahead of tile k's
// product, to overlap the two dependency chains, was measured: no gain at 64 sequences x 4096 tokens, and the ring
// slot it ties up costs 3-7 % on larger batches.)
struct Scored {
  uint32_t pb0, pb1;  // P' = p * v_scale as the B fragment of the second contraction: k = 2t, 2t+1 | 2t+8, 2t+9, n = head g
  float alpha;        // exp2(old max - new max): what O has to be multiplied by before this tile's product is added
  float lv;           // this lane's share of the sum of the tile's P' (as rounded to fp16)
};

// S = q . K^T on the int8 tensor cores, running max / sum update, P'.
__device__ __forceinline__ Scored mma_score(MmaState& st, const uint8_t* stage, int nvalid, int lane) {
  const int t = lane & 3;
  const float* sS = reinterpret_cast<const float*>(stage + 2 * kTile * kD);
  // B fragment of lane (g,t): token g (first MMA group) / g+8 (second), raw code words; one 16-byte read feeds
  // two k-steps.
  int c1[4] = {0, 0, 0, 0}, c2[4] = {0, 0, 0, 0};
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const uint4 w0 = *reinterpret_cast<const uint4*>(stage + st.k_off[c]);
    const uint4 w1 = *reinterpret_cast<const uint4*>(stage + st.k_off[c] + 8 * kD);
    imma16832(c1, st.qa[2 * c], w0.x, w0.y);
    imma16832(c2, st.qa[2 * c], w1.x, w1.y);
    imma16832(c1, st.qa[2 * c + 1], w0.z, w0.w);
    imma16832(c2, st.qa[2 * c + 1], w1.z, w1.w);
  }
  // rows g (high term) and g+8 (low term) of head g, tokens 2t, 2t+1 (c1) and 2t+8, 2t+9 (c2)
  const float2 ks_a = *reinterpret_cast<const float2*>(sS + 2 * t), ks_b = *reinterpret_cast<const float2*>(sS + 8 + 2 * t);
  const float2 vs_a = *reinterpret_cast<const float2*>(sS + 16 + 2 * t), vs_b = *reinterpret_cast<const float2*>(sS + 24 + 2 * t);
  float a[4];
  a[0] = (float)(c1[0] * 128 + c1[2]) * (ks_a.x * st.sfac);  // |hi| <= 128*127*127, so no overflow
  a[1] = (float)(c1[1] * 128 + c1[3]) * (ks_a.y * st.sfac);
  a[2] = (float)(c2[0] * 128 + c2[2]) * (ks_b.x * st.sfac);
  a[3] = (float)(c2[1] * 128 + c2[3]) * (ks_b.y * st.sfac);
  if (nvalid < kTile) {  // a sequence's last tile: rows past the end do not exist (their scales were zero-filled)
    if (2 * t >= nvalid) a[0] = -INFINITY;
    if (2 * t + 1 >= nvalid) a[1] = -INFINITY;
    if (2 * t + 8 >= nvalid) a[2] = -INFINITY;
    if (2 * t + 9 >= nvalid) a[3] = -INFINITY;
  }
  float mx = fmaxf(fmaxf(a[0], a[1]), fmaxf(a[2], a[3]));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  const float m_new = fmaxf(st.m, mx);
  Scored r;
  r.alpha = fast_exp2(st.m - m_new);
  const float p0 = fast_exp2(a[0] - m_new), p1 = fast_exp2(a[1] - m_new);  // exp2(-inf) = 0 for masked rows
  const float p2 = fast_exp2(a[2] - m_new), p3 = fast_exp2(a[3] - m_new);
  st.l = st.l * r.alpha + ((p0 + p1) + (p2 + p3));
  st.m = m_new;
  const __half2 h0 = __floats2half2_rn(p0 * vs_a.x, p1 * vs_a.y), h1 = __floats2half2_rn(p2 * vs_b.x, p3 * vs_b.y);
  r.pb0 = *reinterpret_cast<const uint32_t*>(&h0);
  r.pb1 = *reinterpret_cast<const uint32_t*>(&h1);
  // the sum of the fp16 values the tensor core will see: what the +1152 offset of the widened codes adds per channel
  const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
  r.lv = (f0.x + f0.y) + (f1.x + f1.y);
  return r;
}

// Rescale O when some running max moved (warp-uniform test); columns 2t, 2t+1 belong to heads whose state lives
// in lanes 8t.. and 8t+4..
__device__ __forceinline__ void mma_rescale(MmaState& st, float alpha, int lane) {
  const int t = lane & 3;
  if (__any_sync(0xffffffffu, alpha != 1.f)) {
    const float al0 = __shfl_sync(0xffffffffu, alpha, 8 * t), al1 = __shfl_sync(0xffffffffu, alpha, 8 * t + 4);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      st.o[j][0] *= al0; st.o[j][1] *= al1;
      st.o[j][2] *= al0; st.o[j][3] *= al1;
    }
    st.lv *= alpha;  // the offset that O carries is scaled with it
  }
}

// O'^T += (V + 1152)^T . P' : lane reads channels 16g..16g+15 of tokens 2t, 2t+1, 2t+8, 2t+9.  A code is widened to
// fp16 by a byte permute alone: 0x6400 | (code ^ 0x80) is the half 1152 + code, exactly.  The offset is not
// subtracted per element (a third of this function's instructions): every channel of head g collects
// 1152 * sum(P'), which mma_debias takes away again every few tiles.
__device__ __forceinline__ void mma_pv(MmaState& st, const uint8_t* stage, const Scored& s) {
  constexpr uint32_t kMagic = 0x64646464u, kFlip = 0x80808080u;
  const uint32_t pb0 = s.pb0, pb1 = s.pb1;
  st.lv += s.lv;
  uint32_t vw[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 raw = *reinterpret_cast<const uint4*>(stage + st.v_off + (i & 1) * kD + (i >> 1) * 8 * kD);
    vw[i][0] = raw.x ^ kFlip; vw[i][1] = raw.y ^ kFlip; vw[i][2] = raw.z ^ kFlip; vw[i][3] = raw.w ^ kFlip;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t sel = (j & 1) ? 0x7362u : 0x5140u;
    const uint32_t xa = prmt(vw[0][j >> 1], vw[1][j >> 1], sel);  // tokens 2t, 2t+1: (d0,d0',d1,d1')
    const uint32_t xb = prmt(vw[2][j >> 1], vw[3][j >> 1], sel);  // tokens 2t+8, 2t+9
    mma16816(st.o[j], prmt(xa, kMagic, 0x5140u), prmt(xa, kMagic, 0x7362u), prmt(xb, kMagic, 0x5140u),
             prmt(xb, kMagic, 0x7362u), pb0, pb1);
  }
}

// Take the offset of the widened codes out of O: every channel of head `col` has collected 1152 * (sum of P' of that
// head since the last call).  Done every kDebiasTiles tiles, so that the offset never grows far beyond the products
// it rides on and the fp32 accumulation keeps its precision however long the sequence is.
constexpr int kDebiasTiles = 8;
__device__ __forceinline__ void mma_debias(MmaState& st, int lane) {
  const int t = lane & 3;
  float lv = st.lv;
  lv += __shfl_xor_sync(0xffffffffu, lv, 1);
  lv += __shfl_xor_sync(0xffffffffu, lv, 2);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float off = 1152.f * __shfl_sync(0xffffffffu, lv, 4 * (2 * t + j));
#pragma unroll
    for (int i = 0; i < 8; ++i) { st.o[i][j] -= off; st.o[i][2 + j] -= off; }
  }
  st.lv = 0.f;
}

// Finish an (entry, head) segment: final bf16 rows when the warp saw every tile, otherwise an
// fp32 partial (acc[G][128], m[G], l[G]) in the given workspace slot.
__device__ __forceinline__ void mma_end(MmaState& st, bool whole, uint16_t* __restrict__ out, long long o_sb,
                                        long long o_sh, int b, int h, int G, float* __restrict__ part_o,
                                        float* __restrict__ part_ml, int lane) {
  const int g = lane >> 2, t = lane & 3;
  mma_debias(st, lane);
  float l = st.l;
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int col = 2 * t + j;  // this lane's output column; its softmax state lives in lanes 4*col..
    const float l_c = __shfl_sync(0xffffffffu, l, 4 * col), m_c = __shfl_sync(0xffffffffu, st.m, 4 * col);
    if (col >= G) continue;
    if (whole) {
      const float inv = 1.f / l_c;
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)  // channels 16g + 2i, 16g + 2i + 1
        w[i] = float_to_bf16_bits(st.o[i][j] * inv) | (float_to_bf16_bits(st.o[i][2 + j] * inv) << 16);
      uint16_t* dst = out + b * o_sb + (long long)(h * G + col) * o_sh + 16 * g;
      *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
      *reinterpret_cast<uint4*>(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
    } else {
      float* dst = part_o + col * kD + 16 * g;
#pragma unroll
      for (int i = 0; i < 8; i += 2)
        *reinterpret_cast<float4*>(dst + 2 * i) = make_float4(st.o[i][j], st.o[i][2 + j], st.o[i + 1][j], st.o[i + 1][2 + j]);
      if (g == 0) {
        part_ml[col * 2] = m_c;
        part_ml[col * 2 + 1] = l_c;
      }
    }
  }
}

// ------------------------------------------------------------------ consumer state (scalar variant)
// Lane l: scores of token l>>1 over channels 64*(l&1).., output channels 4l..4l+3.
struct ScalarState {
  float m[kMaxG], l[kMaxG];
  float o[kMaxG][4];
  float scale_log2;
};

__device__ __forceinline__ void scalar_begin(ScalarState& st, float* qs, const uint16_t* __restrict__ q, long long q_sb,
                                             long long q_sh, int b, int h, int G, float scale_log2, int lane) {
  __syncwarp();
  for (int i = lane; i < G * kD; i += 32) {
    const int gq = i / kD, d = i - gq * kD;
    qs[i] = bf16_bits_to_float(q[b * q_sb + (long long)(h * G + gq) * q_sh + d]);
  }
  __syncwarp();
#pragma unroll
  for (int gq = 0; gq < kMaxG; ++gq) {
    st.m[gq] = -INFINITY; st.l[gq] = 0.f;
    st.o[gq][0] = st.o[gq][1] = st.o[gq][2] = st.o[gq][3] = 0.f;
  }
  st.scale_log2 = scale_log2;
}

__device__ __forceinline__ void scalar_tile(ScalarState& st, const float* qs, float* ps, const uint8_t* stage, int nvalid,
                                            int G, int lane) {
  const uint8_t* sK = stage;
  const uint8_t* sV = stage + kTile * kD;
  const float* sS = reinterpret_cast<const float*>(stage + 2 * kTile * kD);
  const int tok = lane >> 1, half = lane & 1;
  float dot[kMaxG];
#pragma unroll
  for (int gq = 0; gq < kMaxG; ++gq) dot[gq] = 0.f;
  for (int cc = 0; cc < 4; ++cc) {
    const int chunk = 4 * half + cc;
    uint4 raw = *reinterpret_cast<const uint4*>(sK + tok * kD + ((chunk ^ ((tok & 1) << 2)) << 4));
    uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float kf = (float)(int)(int8_t)((w[i >> 2] >> (8 * (i & 3))) & 0xFFu);
#pragma unroll
      for (int gq = 0; gq < kMaxG; ++gq)
        if (gq < G) dot[gq] = fmaf(qs[gq * kD + 16 * chunk + i], kf, dot[gq]);
    }
  }
  const bool valid = tok < nvalid;
  const float ks = sS[tok], vs = sS[16 + tok];
  float alpha[kMaxG];
  __syncwarp();
#pragma unroll
  for (int gq = 0; gq < kMaxG; ++gq) {
    if (gq >= G) continue;
    float d = dot[gq] + __shfl_xor_sync(0xffffffffu, dot[gq], 1);
    float sc = valid ? d * (ks * st.scale_log2) : -INFINITY;
    float mx = sc;
#pragma unroll
    for (int o = 2; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float m_new = fmaxf(st.m[gq], mx);
    alpha[gq] = fast_exp2(st.m[gq] - m_new);
    const float p = fast_exp2(sc - m_new);
    float psum = half == 0 ? p : 0.f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
    st.l[gq] = st.l[gq] * alpha[gq] + psum;
    st.m[gq] = m_new;
    if (half == 0) ps[gq * kTile + tok] = valid ? p * vs : 0.f;
  }
  __syncwarp();
#pragma unroll
  for (int gq = 0; gq < kMaxG; ++gq)
    if (gq < G) { st.o[gq][0] *= alpha[gq]; st.o[gq][1] *= alpha[gq]; st.o[gq][2] *= alpha[gq]; st.o[gq][3] *= alpha[gq]; }
  for (int r = 0; r < kTile; ++r) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(sV + r * kD + (((lane >> 2) ^ (r & 6)) << 4) + 4 * (lane & 3));
    float vf[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) vf[i] = (float)(int)(int8_t)((w >> (8 * i)) & 0xFFu);
#pragma unroll
    for (int gq = 0; gq < kMaxG; ++gq) {
      if (gq >= G) continue;
      const float pv = ps[gq * kTile + r];
#pragma unroll
      for (int i = 0; i < 4; ++i) st.o[gq][i] = fmaf(pv, vf[i], st.o[gq][i]);
    }
  }
}

__device__ __forceinline__ void scalar_end(ScalarState& st, bool whole, uint16_t* __restrict__ out, long long o_sb,
                                           long long o_sh, int b, int h, int G, float* __restrict__ part_o,
                                           float* __restrict__ part_ml, int lane) {
#pragma unroll
  for (int gq = 0; gq < kMaxG; ++gq) {
    if (gq >= G) continue;
    if (whole) {
      const float inv = 1.f / st.l[gq];
      uint2 w;
      w.x = float_to_bf16_bits(st.o[gq][0] * inv) | (float_to_bf16_bits(st.o[gq][1] * inv) << 16);
      w.y = float_to_bf16_bits(st.o[gq][2] * inv) | (float_to_bf16_bits(st.o[gq][3] * inv) << 16);
      *reinterpret_cast<uint2*>(out + b * o_sb + (long long)(h * G + gq) * o_sh + 4 * lane) = w;
    } else {
      *reinterpret_cast<float4*>(part_o + gq * kD + 4 * lane) = make_float4(st.o[gq][0], st.o[gq][1], st.o[gq][2], st.o[gq][3]);
      if (lane == 0) {
        part_ml[gq * 2] = st.m[gq];
        part_ml[gq * 2 + 1] = st.l[gq];
      }
    }
  }
}

// ------------------------------------------------------------------ main kernel
// Workspace: int32 prefix[B+1] (padded to 256 B; read by the separate reduction kernel) |
// int32 arrivals[B*Hkv] (padded; zero on entry, left zero: counts the partials of each (entry, head)
// when the reduction is fused into this kernel) | float ml[W][2][G][2] | float acc[W][2][G][128]
__host__ __device__ inline size_t ws_prefix_bytes(int B) { return (((size_t)(B + 1) * 4 + 255) / 256) * 256; }
__host__ __device__ inline size_t ws_count_bytes(int B, int Hkv) { return (((size_t)B * Hkv * 4 + 255) / 256) * 256; }
__host__ __device__ inline size_t ws_head_bytes(int B, int Hkv) { return ws_prefix_bytes(B) + ws_count_bytes(B, Hkv); }

// The pieces of one (entry, head) that reached the workspace, in tile order.  Its flat tile range
// [s0, e) is covered by warps w_first..w_last; CTAs c_lo..c_hi-1 lie entirely inside it, each of
// those summed its four pieces in shared memory and left ONE piece in the slot of its first warp.
// So the list is: warps [w_first, kWarps*c_lo), then every kWarps-th warp up to kWarps*c_hi, then
// warps [kWarps*c_hi, w_last].  A warp's piece is in its slot 1 only if it is w_first and the
// (entry, head) starts inside that warp's range.
struct Pieces {
  int w_first, n_a, w_b, n_b, w_c, n, slot_first;
  __device__ __forceinline__ Pieces(const Partition& part, int s0, int e) {
    w_first = s0 / part.per;
    const int w_last = (e - 1) / part.per;
    const int span = kWarps * part.per;
    const int c_lo = (s0 + span - 1) / span, c_hi = min(e, part.U) / span;
    slot_first = s0 > w_first * part.per ? 1 : 0;
    if (c_hi > c_lo) {
      w_b = kWarps * c_lo; w_c = kWarps * c_hi;
      n_a = w_b - w_first; n_b = c_hi - c_lo;
      n = n_a + n_b + (w_last - w_c + 1);
    } else {
      w_b = w_c = w_first; n_a = 0; n_b = 0;
      n = w_last - w_first + 1;
    }
  }
  // workspace slot index (2 * warp + slot) of piece k
  __device__ __forceinline__ int slot_of(int k) const {
    const int w = k < n_a ? w_first + k : (k < n_a + n_b ? w_b + kWarps * (k - n_a) : w_c + (k - n_a - n_b));
    return 2 * w + (w == w_first ? slot_first : 0);
  }
};

// Merge the pieces of one (entry, head) and write the final bf16 rows.  One warp; lane l owns
// channels 4l..4l+3.  Loads bypass L1 (the pieces were written by other SMs).  Sixteen pieces per
// round: lane k fetches (m, l) of piece k while every lane fetches its channels of all sixteen in
// the same round of memory latency (the loads are unconditional and independent; a padded slot
// repeats the last piece and gets weight zero), then an online-softmax update folds the round in.
__device__ __forceinline__ void merge_partials_by_column(const float* __restrict__ ws_ml, const float* __restrict__ ws_o,
                                               const Pieces& pc, int G, uint16_t* __restrict__ out_row, long long o_sh,
                                               int lane) {
  constexpr int kRound = 16;
  for (int col = 0; col < G; ++col) {
    float M = -INFINITY, L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k0 = 0; k0 < pc.n; k0 += kRound) {
      const int nb = min(kRound, pc.n - k0);
      float2 ml = make_float2(-INFINITY, 0.f);
      if (lane < nb) ml = __ldcg(reinterpret_cast<const float2*>(ws_ml + ((size_t)pc.slot_of(k0 + lane) * G + col) * 2));
      float4 buf[kRound];
#pragma unroll
      for (int j = 0; j < kRound; ++j)
        buf[j] = __ldcg(reinterpret_cast<const float4*>(ws_o + ((size_t)pc.slot_of(k0 + min(j, nb - 1)) * G + col) * kD + 4 * lane));
      float mb = ml.x;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, o));
      const float M_new = fmaxf(M, mb);
      const float resc = M == -INFINITY ? 0.f : fast_exp2(M - M_new);
      const float wgt = lane < nb ? fast_exp2(ml.x - M_new) : 0.f;
      float ls = ml.y * wgt;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o);
      L = L * resc + ls;
      acc.x *= resc; acc.y *= resc; acc.z *= resc; acc.w *= resc;
#pragma unroll
      for (int j = 0; j < kRound; ++j) {
        const float wg = __shfl_sync(0xffffffffu, wgt, j);
        acc.x = fmaf(buf[j].x, wg, acc.x); acc.y = fmaf(buf[j].y, wg, acc.y);
        acc.z = fmaf(buf[j].z, wg, acc.z); acc.w = fmaf(buf[j].w, wg, acc.w);
      }
      M = M_new;
    }
    const float inv = 1.f / L;
    uint2 r;
    r.x = float_to_bf16_bits(acc.x * inv) | (float_to_bf16_bits(acc.y * inv) << 16);
    r.y = float_to_bf16_bits(acc.z * inv) | (float_to_bf16_bits(acc.w * inv) << 16);
    *reinterpret_cast<uint2*>(out_row + col * o_sh + 4 * lane) = r;
  }
}

// The same for a GQA group of two heads (the geometry of the path), both heads in ONE round of loads per eight
// pieces: lane 2k + col fetches (m, l) of (piece k, head col) while every lane fetches its channels of both heads of
// all eight pieces (16 independent 16-byte loads), so up to eight pieces cost a single round of memory latency.
__device__ __forceinline__ void merge_partials_pair(const float* __restrict__ ws_ml, const float* __restrict__ ws_o,
                                                    const Pieces& pc, uint16_t* __restrict__ out_row, long long o_sh, int lane) {
  constexpr int kRound = 8, G = 2;
  float M[G] = {-INFINITY, -INFINITY}, L[G] = {0.f, 0.f};
  float4 acc[G] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  for (int k0 = 0; k0 < pc.n; k0 += kRound) {
    const int nb = min(kRound, pc.n - k0);
    float2 ml = make_float2(-INFINITY, 0.f);
    if (lane < 2 * nb) ml = __ldcg(reinterpret_cast<const float2*>(ws_ml + ((size_t)pc.slot_of(k0 + (lane >> 1)) * G + (lane & 1)) * 2));
    float4 buf[kRound][G];
#pragma unroll
    for (int j = 0; j < kRound; ++j) {
      const float* base = ws_o + (size_t)pc.slot_of(k0 + min(j, nb - 1)) * G * kD + 4 * lane;
      buf[j][0] = __ldcg(reinterpret_cast<const float4*>(base));
      buf[j][1] = __ldcg(reinterpret_cast<const float4*>(base + kD));
    }
    // maximum per head: lanes of equal parity among the first sixteen hold that head's pieces
    float mb = lane < 2 * nb ? ml.x : -INFINITY;
#pragma unroll
    for (int o = 2; o < 32; o <<= 1) mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, o));
    const float mb0 = __shfl_sync(0xffffffffu, mb, 0), mb1 = __shfl_sync(0xffffffffu, mb, 1);
    const float Mn[G] = {fmaxf(M[0], mb0), fmaxf(M[1], mb1)};
    const float wgt = lane < 2 * nb ? fast_exp2(ml.x - Mn[lane & 1]) : 0.f;
    float ls = ml.y * wgt;
#pragma unroll
    for (int o = 2; o < 32; o <<= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o);
    const float ls0 = __shfl_sync(0xffffffffu, ls, 0), ls1 = __shfl_sync(0xffffffffu, ls, 1);
#pragma unroll
    for (int c = 0; c < G; ++c) {
      const float resc = M[c] == -INFINITY ? 0.f : fast_exp2(M[c] - Mn[c]);
      L[c] = L[c] * resc + (c ? ls1 : ls0);
      acc[c].x *= resc; acc[c].y *= resc; acc[c].z *= resc; acc[c].w *= resc;
      M[c] = Mn[c];
    }
#pragma unroll
    for (int j = 0; j < kRound; ++j) {
#pragma unroll
      for (int c = 0; c < G; ++c) {
        const float wg = __shfl_sync(0xffffffffu, wgt, 2 * j + c);
        acc[c].x = fmaf(buf[j][c].x, wg, acc[c].x); acc[c].y = fmaf(buf[j][c].y, wg, acc[c].y);
        acc[c].z = fmaf(buf[j][c].z, wg, acc[c].z); acc[c].w = fmaf(buf[j][c].w, wg, acc[c].w);
      }
    }
  }
#pragma unroll
  for (int c = 0; c < G; ++c) {
    const float inv = 1.f / L[c];
    uint2 r;
    r.x = float_to_bf16_bits(acc[c].x * inv) | (float_to_bf16_bits(acc[c].y * inv) << 16);
    r.y = float_to_bf16_bits(acc[c].z * inv) | (float_to_bf16_bits(acc[c].w * inv) << 16);
    *reinterpret_cast<uint2*>(out_row + c * o_sh + 4 * lane) = r;
  }
}

__device__ __forceinline__ void merge_partials(const float* __restrict__ ws_ml, const float* __restrict__ ws_o,
                                               const Pieces& pc, int G, uint16_t* __restrict__ out_row, long long o_sh,
                                               int lane) {
  if (G == 2) merge_partials_pair(ws_ml, ws_o, pc, out_row, o_sh, lane);
  else merge_partials_by_column(ws_ml, ws_o, pc, G, out_row, o_sh, lane);
}

__host__ __device__ inline size_t ws_ml_bytes(int W, int G) { return (((size_t)W * 2 * G * 2 * 4 + 255) / 256) * 256; }

// ------------------------------------------------------------------ per-step plan
// The partition depends only on the step's metadata (cached_lens, num_decoding, the block table), which is
// the same for every layer of a decoder step.  decode_plan_kernel computes it once: a header and, for every
// warp of the persistent grid, the cursor of its first tile and the page ids of its first kStages-1 tiles.
// A planned decode_attn_kernel then needs one round of loads (its plan entry, the lengths, num_decoding)
// before its first copies are in flight, instead of the length scan, a binary search and a dependent
// page-table read in each of its CTAs in each layer.
constexpr int kPlanMagic = 0x6b765031;  // "kvP1"
constexpr int kPlanHeaderInts = 8;      // magic, B, Hkv, W, U, per, num_decoding, page_size
constexpr int kPlanEntryInts = 16;      // b, h, tile, T, n, base, page[0..2], reserved
constexpr int kPlanThreads = 1024;
__host__ __device__ inline size_t plan_bytes(int W) { return ((size_t)kPlanHeaderInts + (size_t)W * kPlanEntryInts) * 4; }

__global__ void __launch_bounds__(kPlanThreads)
decode_plan_kernel(const int32_t* __restrict__ cached_lens, const int32_t* __restrict__ num_decoding,
                   const int32_t* __restrict__ table, int table_stride, int max_pages, int page_size, int B, int Hkv,
                   int W, int* __restrict__ plan) {
  __shared__ int chunk_prefix[kPlanThreads + 1];
  __shared__ int lens_s[kSmemLens];
  // No early trigger here: a kernel chained behind this one is only brought up when every thread of this
  // grid has exited, i.e. after the fence below, so it may read the plan before its own wait.
  pdl_wait();
  const int chunk = (B + kPlanThreads - 1) / kPlanThreads;
  int nd;
  scan_tiles(cached_lens, B, num_decoding, chunk, chunk_prefix, lens_s, nullptr, nd);
  const Lens lens{cached_lens, lens_s, nd};
  const Partition part = make_partition(chunk_prefix[kPlanThreads], Hkv, W, nd);
  if (threadIdx.x == 0) {
    plan[0] = kPlanMagic; plan[1] = B; plan[2] = Hkv; plan[3] = W;
    plan[4] = part.U; plan[5] = part.per; plan[6] = nd; plan[7] = page_size;
  }
  for (int w = threadIdx.x; w < W; w += kPlanThreads) {
    int* e = plan + kPlanHeaderInts + (size_t)w * kPlanEntryInts;
    const long long u_begin = (long long)w * part.per;
    if (u_begin >= part.U) {
      e[0] = -1;
      continue;
    }
    Cursor cur;
    cur.seek(chunk_prefix, kPlanThreads, chunk, lens, Hkv, page_size, (int)u_begin);
    e[0] = cur.b; e[1] = cur.h; e[2] = cur.tile; e[3] = cur.T; e[4] = cur.n; e[5] = cur.base;
    int left = min(part.per, part.U - (int)u_begin);
    for (int i = 0; i < kStages - 1; ++i) {
      int page = -1;
      if (left > 0) {
        page = cur.slot < max_pages ? table[(long long)cur.b * table_stride + cur.slot] : -2;
        if (--left > 0) cur.next(lens, Hkv, page_size);
      }
      e[6 + i] = page;
    }
  }
  __threadfence();
}

#ifdef B200KV_STAMPS
// Instrumented build only: 16 words per warp of the persistent grid.  [0] kernel entry and [5] exit in %globaltimer
// nanoseconds, [1] SM id, [6] tiles, [7] pieces merged; the rest are SM clock cycles since this warp's entry:
// [8] metadata there (plan or scan done), [2] first copies issued, [9] q of the first segment loaded, [3] first tile
// landed, [4] last tile consumed, [10] last piece stored, [11] arrival counter answered (last arriver only),
// [12] merge done (last arriver only), [13] exit.
constexpr int kStampWarps = 4096, kStampWords = 16;
__device__ unsigned long long g_stamps[kStampWarps * kStampWords];
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define STAMP(i, v) do { if (lane == 0 && w < kStampWarps) g_stamps[kStampWords * w + (i)] = (v); } while (0)
#define dclk() ((unsigned long long)(clock64() - c_entry))
#else
#define STAMP(i, v) do { } while (0)
#endif

template <bool kScalar>
__global__ void __launch_bounds__(kWarps * 32, kCtasPerSm)
decode_attn_kernel(const uint16_t* __restrict__ q, long long q_sb, long long q_sh, CacheView c,
                   const int32_t* __restrict__ cached_lens, const int32_t* __restrict__ num_decoding, float scale_log2,
                   uint16_t* __restrict__ out, long long o_sb, long long o_sh, uint8_t* __restrict__ workspace, int B,
                   int G, int W, int fused, int early, const int* __restrict__ plan, int32_t* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring = smem;                                                       // kWarps * kStages * kTileBytes
  float* q_s = reinterpret_cast<float*>(ring + kWarps * kStages * kTileBytes);  // scalar variant: kWarps * (G*128 + G*16)
  int* chunk_prefix = reinterpret_cast<int*>(q_s + (kScalar ? kWarps * (kMaxG * kD + kMaxG * kTile) : 0));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int w = blockIdx.x * kWarps + warp;
#ifdef B200KV_STAMPS
  const unsigned long long t_entry = gtime();
  const long long c_entry = clock64();
#endif

  // The first CTA waits for the predecessor at once, so that this grid can never complete before it.  The
  // trigger for the successor comes late, when a warp has issued its last tile: the CTAs of a successor that is
  // brought up while this kernel still streams sit on the SMs waiting and slow the streaming down (measured:
  // +16 us per call when the trigger was the first statement).
  if (blockIdx.x == 0) pdl_wait();
  int* lens_s = chunk_prefix + kWarps * 32 + 1;
  int* cta_arrive = lens_s + kSmemLens;  // how many of this CTA's warps have parked a piece in shared memory
  if (threadIdx.x == 0) *cta_arrive = 0;  // ordered before any use by the barriers below
  int nd;
  Partition part;
  Cursor pc;  // producer position (runs kStages-1 tiles ahead of the consumer)
  int first_page = -1;  // planned: lane i < kStages-1 holds the page id of the warp's i-th tile
  if (plan != nullptr) {
    // One round of independent loads: the warp's plan entry (lanes 0-15), the header (lanes 16-23),
    // num_decoding and this thread's share of the lengths.
    int pe = 0;
    if (lane < kPlanEntryInts) pe = __ldcg(plan + kPlanHeaderInts + (size_t)w * kPlanEntryInts + lane);
    else if (lane < kPlanEntryInts + kPlanHeaderInts) pe = __ldcg(plan + (lane - kPlanEntryInts));
    const int nd_raw = __ldcg(num_decoding);
    int cl[kSmemLens / (kWarps * 32)];
#pragma unroll
    for (int i = 0; i < kSmemLens / (kWarps * 32); ++i) {
      const int b = threadIdx.x + i * kWarps * 32;
      cl[i] = b < B ? __ldcg(cached_lens + b) : 0;
    }
    nd = min(nd_raw, B);
#pragma unroll
    for (int i = 0; i < kSmemLens / (kWarps * 32); ++i) {
      const int b = threadIdx.x + i * kWarps * 32;
      if (b < B) lens_s[b] = b < nd ? cl[i] + 1 : 0;
    }
    __syncthreads();
    const bool hdr_ok = __shfl_sync(0xffffffffu, pe, 16) == kPlanMagic && __shfl_sync(0xffffffffu, pe, 17) == B &&
                        __shfl_sync(0xffffffffu, pe, 18) == c.Hkv && __shfl_sync(0xffffffffu, pe, 19) == W &&
                        __shfl_sync(0xffffffffu, pe, 22) == nd && __shfl_sync(0xffffffffu, pe, 23) == c.page_size;
    part.U = __shfl_sync(0xffffffffu, pe, 20);
    part.per = __shfl_sync(0xffffffffu, pe, 21);
    part.W = W;
    pc.b = __shfl_sync(0xffffffffu, pe, 0);
    pc.h = __shfl_sync(0xffffffffu, pe, 1);
    pc.tile = __shfl_sync(0xffffffffu, pe, 2);
    pc.T = __shfl_sync(0xffffffffu, pe, 3);
    pc.n = __shfl_sync(0xffffffffu, pe, 4);
    pc.base = __shfl_sync(0xffffffffu, pe, 5);
    first_page = __shfl_sync(0xffffffffu, pe, 6 + (lane < kStages - 1 ? lane : 0));
    if (!hdr_ok) {  // not a plan of this batch on this grid: nothing is read or written through it
      if (lane == 0 && status) atomicOr(status, B200KV_S_BAD_PLAN);
      return;
    }
    if (pc.b < 0) return;  // no work for this warp
    const Lens probe{cached_lens, lens_s, nd};
    if (pc.b >= B || pc.h < 0 || pc.h >= c.Hkv || pc.n != probe.n(pc.b) || pc.T != probe.tiles(pc.b) || pc.tile < 0 ||
        pc.tile >= pc.T || (long long)w * part.per >= part.U) {  // the plan was made from other lengths
      if (lane == 0 && status) atomicOr(status, B200KV_S_BAD_PLAN);
      return;
    }
    pc.slot = (pc.tile * kTile) / c.page_size;
    pc.row0 = pc.tile * kTile - pc.slot * c.page_size;
  } else {
    const int nchunks = blockDim.x, chunk = (B + nchunks - 1) / nchunks;
    scan_tiles(cached_lens, B, num_decoding, chunk, chunk_prefix, lens_s,
               (blockIdx.x == 0 && !fused) ? reinterpret_cast<int*>(workspace) : nullptr, nd);
    part = make_partition(chunk_prefix[nchunks], c.Hkv, W, nd);
    if ((long long)w * part.per >= part.U) return;
    const Lens probe{cached_lens, lens_s, nd};
    pc.seek(chunk_prefix, nchunks, chunk, probe, c.Hkv, c.page_size, w * part.per);
  }
  STAMP(8, dclk());
  const Lens lens{cached_lens, lens_s, nd};
  const int u0 = w * part.per;
  const int ntiles = min(part.per, part.U - u0);

  int* ws_count = reinterpret_cast<int*>(workspace + ws_prefix_bytes(B));
  float* ws_ml = reinterpret_cast<float*>(workspace + ws_head_bytes(B, c.Hkv));
  float* ws_o = reinterpret_cast<float*>(workspace + ws_head_bytes(B, c.Hkv) + ws_ml_bytes(W, G));
  uint8_t* my_ring = ring + warp * kStages * kTileBytes;
  const uint32_t my_ring_s = smem_u32(my_ring);
  float* my_q = q_s + warp * (kMaxG * kD + kMaxG * kTile);

  Cursor cc = pc;  // consumer position, advanced segment by segment
  PageWindow win{-1, 0, -1};
  const LaneCopy lc = make_lane_copy(c, lane);

  // Early start: everything above read only the batch metadata.  q, the workspace and the newest
  // token of every sequence (the last tile) may still be in flight from the kernel launched just
  // before this one (the quantize-on-write of this layer), so those wait for it; older tiles are
  // not touched by it and are fetched right away, hiding the first burst behind that kernel.
  bool must_wait = early != 0;
  int p_left = ntiles;  // tiles not yet issued
#pragma unroll
  for (int i = 0; i < kStages - 1; ++i) {
    if (p_left > 0) {
      if (must_wait && pc.tile == pc.T - 1) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        must_wait = false;
      }
      const int page = plan != nullptr ? __shfl_sync(0xffffffffu, first_page, i) : window_page(c, pc, win, lane);
      issue_tile(c, pc, page, lc, my_ring_s + i * kTileBytes, lane, status);
      if (--p_left > 0) pc.next(lens, c.Hkv, c.page_size);
    }
    cp_async_commit();
  }
  STAMP(2, dclk());
  // planned: the table row of the next tile is requested now and is there when the main loop wants it
  if (plan != nullptr && p_left > 0) load_window(c, pc.b, pc.slot, win, lane);
  if (must_wait) asm volatile("griddepcontrol.wait;" ::: "memory");

  typename std::conditional<kScalar, ScalarState, MmaState>::type st;
  if constexpr (!kScalar) mma_init_lane(st, lane);
  int stage_c = 0, stage_p = kStages - 1;  // ring slots of the tile consumed / issued next
  int done = 0;
  // ... and a warp with only a handful of tiles has nothing to gain from holding one back: the grid is far from
  // loading the memory system and its time is the latency of its few tiles
  const bool deep = part.per > kDeepTiles || part.per <= kShallowFloor;
  while (done < ntiles) {
    // one segment: the tiles [cc.tile, cc.tile + seg) of (entry cc.b, head cc.h)
    const int seg = min(cc.T - cc.tile, ntiles - done);
    if constexpr (kScalar) scalar_begin(st, my_q, q, q_sb, q_sh, cc.b, cc.h, G, scale_log2, lane);
    else mma_begin(st, q, q_sb, q_sh, cc.b, cc.h, G, scale_log2, lane);
#ifdef B200KV_STAMPS
    if (done == 0) STAMP(9, dclk());
#endif
    int remaining = cc.n - cc.tile * kTile;  // tokens from this tile to the end of the sequence
    for (int k = 0; k < seg; ++k) {
      if (p_left > 0) {
        issue_tile(c, pc, window_page(c, pc, win, lane), lc, my_ring_s + stage_p * kTileBytes, lane, status);
        if (--p_left > 0) pc.next(lens, c.Hkv, c.page_size);
      }
      cp_async_commit();
      // Measured on B200: up to about 200 tiles per warp (64-128 sequences of 4096 tokens) the kernel is 3-4 % faster
      // when a warp also waits for the tile AFTER the one it is about to use (fewer requests queued in the memory
      // system at any time); beyond that the deeper look-ahead wins by 5-8 %.
      if (deep) cp_async_wait<kStages - 1>();
      else cp_async_wait<kStages - 2>();
      __syncwarp();
#ifdef B200KV_STAMPS
      if (done == 0 && k == 0) STAMP(3, dclk());
#endif
      const uint8_t* stage = my_ring + stage_c * kTileBytes;
      if constexpr (kScalar) {
        scalar_tile(st, my_q, my_q + kMaxG * kD, stage, min(remaining, kTile), G, lane);
      } else {
        const Scored s = mma_score(st, stage, remaining, lane);
        mma_rescale(st, s.alpha, lane);
        mma_pv(st, stage, s);
        if ((k & (kDebiasTiles - 1)) == kDebiasTiles - 1) mma_debias(st, lane);
      }
      __syncwarp();
      remaining -= kTile;
      stage_c = (stage_c + 1) & (kStages - 1);
      stage_p = (stage_p + 1) & (kStages - 1);
    }
#ifdef B200KV_STAMPS
    if (done + seg >= ntiles) STAMP(4, dclk());
#endif
    // whole iff the segment began at the sequence's first tile and reached its last one
    const bool whole = cc.tile == 0 && seg == cc.T;
    const int slot = done == 0 ? 0 : 1;
    const int s0 = cc.base + cc.h * cc.T;  // flat tile range of this (entry, head): [s0, s0 + T)
    uint16_t* out_row = out + cc.b * o_sb + (long long)(cc.h * G) * o_sh;
    // Do all four warps of this CTA hold pieces of this same (entry, head)?  Then the pieces meet
    // in shared memory and one warp forwards their sum (no global round trip for three of them).
    const int cta_u0 = blockIdx.x * kWarps * part.per, cta_u1 = cta_u0 + kWarps * part.per;
    const bool cta_inside = !whole && s0 <= cta_u0 && cta_u1 <= s0 + cc.T && cta_u1 <= part.U;
    bool deliver = !whole;                       // a piece of mine (or my CTA's sum) goes to the workspace
    float* po = ws_o + ((size_t)w * 2 + slot) * G * kD;
    float* pml = ws_ml + ((size_t)w * 2 + slot) * G * 2;
    if (cta_inside) {
      cp_async_wait<0>();
      __syncwarp();
      float* so = reinterpret_cast<float*>(my_ring);  // [G][128] then [G][2]; the ring is idle now
      if constexpr (kScalar) scalar_end(st, false, out, o_sb, o_sh, cc.b, cc.h, G, so, so + kMaxG * kD, lane);
      else mma_end(st, false, out, o_sb, o_sh, cc.b, cc.h, G, so, so + kMaxG * kD, lane);
      __threadfence_block();
      __syncwarp();
      int t = 0;
      if (lane == 0) t = atomicAdd(cta_arrive, 1);
      t = __shfl_sync(0xffffffffu, t, 0);
      deliver = t == kWarps - 1;
      if (deliver) {  // last of the four: sum them; lane l owns channels 4l..4l+3
        __threadfence_block();
        const bool exact = s0 == cta_u0 && s0 + cc.T == cta_u1;  // the CTA saw the whole sequence
        po = ws_o + ((size_t)(blockIdx.x * kWarps) * 2) * G * kD;  // slot 0 of the CTA's first warp
        pml = ws_ml + ((size_t)(blockIdx.x * kWarps) * 2) * G * 2;
        for (int col = 0; col < G; ++col) {
          float m4[kWarps], M = -INFINITY;
#pragma unroll
          for (int i = 0; i < kWarps; ++i) {
            m4[i] = reinterpret_cast<const float*>(ring + i * kStages * kTileBytes)[kMaxG * kD + col * 2];
            M = fmaxf(M, m4[i]);
          }
          float L = 0.f;
          float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int i = 0; i < kWarps; ++i) {
            const float* sp = reinterpret_cast<const float*>(ring + i * kStages * kTileBytes);
            const float wg = fast_exp2(m4[i] - M);
            L = fmaf(sp[kMaxG * kD + col * 2 + 1], wg, L);
            const float4 o = *reinterpret_cast<const float4*>(sp + col * kD + 4 * lane);
            a.x = fmaf(o.x, wg, a.x); a.y = fmaf(o.y, wg, a.y); a.z = fmaf(o.z, wg, a.z); a.w = fmaf(o.w, wg, a.w);
          }
          if (exact) {
            const float inv = 1.f / L;
            uint2 r;
            r.x = float_to_bf16_bits(a.x * inv) | (float_to_bf16_bits(a.y * inv) << 16);
            r.y = float_to_bf16_bits(a.z * inv) | (float_to_bf16_bits(a.w * inv) << 16);
            *reinterpret_cast<uint2*>(out_row + col * o_sh + 4 * lane) = r;
          } else {
            *reinterpret_cast<float4*>(po + col * kD + 4 * lane) = a;
            if (lane == 0) { pml[col * 2] = M; pml[col * 2 + 1] = L; }
          }
        }
        if (exact) deliver = false;
      }
    } else {
      if constexpr (kScalar) scalar_end(st, whole, out, o_sb, o_sh, cc.b, cc.h, G, po, pml, lane);
      else mma_end(st, whole, out, o_sb, o_sh, cc.b, cc.h, G, po, pml, lane);
    }
#ifdef B200KV_STAMPS
    if (done + seg >= ntiles) STAMP(10, dclk());
#endif
    if (fused && deliver) {
      // Fused cross-split reduction: the warp that delivers the last piece of (entry, head) merges
      // all of them.  Release: partial stores -> warp barrier -> counter; acquire: counter -> warp barrier -> loads.
      const Pieces pieces(part, s0, s0 + cc.T);
      __syncwarp();  // the lanes' partial stores are ordered before lane 0's release below
      int arrived = 0;
      if (lane == 0) arrived = atom_add_acq_rel(ws_count + cc.b * c.Hkv + cc.h, 1) + 1;
      arrived = __shfl_sync(0xffffffffu, arrived, 0);
      if (arrived == pieces.n) {  // the acquire half makes every earlier arriver's stores visible to this warp
        __syncwarp();
        STAMP(11, dclk());
        merge_partials(ws_ml, ws_o, pieces, G, out_row, o_sh, lane);
        if (lane == 0) ws_count[cc.b * c.Hkv + cc.h] = 0;  // leave the counter zero for the next call
#ifdef B200KV_STAMPS
        STAMP(7, (unsigned long long)pieces.n);
        STAMP(12, dclk());
#endif
      }
    }
    done += seg;
    if (done < ntiles) cc.next_segment(lens, c.Hkv);
  }
  // The successor is released only now: its CTAs, brought up while this kernel still streams, would sit on the SMs
  // waiting for it and slow it down (measured: 14-16 us per call with an earlier trigger).
  pdl_trigger();
  cp_async_wait<0>();
#ifdef B200KV_STAMPS
  {
    unsigned sm;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
    STAMP(0, t_entry); STAMP(1, (unsigned long long)sm); STAMP(5, gtime()); STAMP(6, (unsigned long long)ntiles);
    STAMP(13, dclk());
  }
#endif
}

// ------------------------------------------------------------------ cross-split reduction
// grid (B, Hkv), 128 threads.  kernels.py:216-264, with exp2 because the running maxima are kept
// in the log2 domain.  Worker w's piece of (b, h) is in its slot 1 only when it is not the first
// segment of w's range.  Partials are merged up to 128 at a time: thread i fetches (m, l) of
// partial i (one parallel round of loads), the block agrees on the maximum, then the four warps
// each sum every fourth partial with 16-byte loads (lane l owns channels 4l..4l+3) and the four
// sums are added through shared memory - so even a sequence cut into 64 pieces costs a few rounds
// of memory latency, not 64.
__global__ void __launch_bounds__(kD)
decode_combine_kernel(const uint8_t* __restrict__ workspace, const int32_t* __restrict__ num_decoding,
                      uint16_t* __restrict__ out, long long o_sb, long long o_sh, int B, int Hkv, int G, int W) {
  __shared__ float wgt_s[kD];
  __shared__ float red_s[4];
  __shared__ __align__(16) float acc_s[4][kD];
  const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  if (b >= min(*num_decoding, B)) return;
  const int* prefix = reinterpret_cast<const int*>(workspace);
  const int T = prefix[b + 1] - prefix[b];
  if (T == 0) return;
  const Partition part = make_partition(prefix[B], Hkv, W, min(*num_decoding, B));
  const int s = Hkv * prefix[b] + h * T, e = s + T;
  const int w_first = s / part.per, w_last = (e - 1) / part.per;
  if (w_first == w_last) return;  // one warp saw the whole sequence and wrote the output itself
  const Pieces pieces(part, s, e);
  if (pieces.n == 1) return;      // one CTA saw the whole sequence, summed its pieces and wrote the output
  const float* ws_ml = reinterpret_cast<const float*>(workspace + ws_head_bytes(B, Hkv));
  const float* ws_o = reinterpret_cast<const float*>(workspace + ws_head_bytes(B, Hkv) + ws_ml_bytes(W, G));
  const int warp = tid >> 5, lane = tid & 31;

  for (int col = 0; col < G; ++col) {
    float M = -INFINITY, L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k0 = 0; k0 < pieces.n; k0 += kD) {
      const int nb = min(kD, pieces.n - k0);
      float m_i = -INFINITY, l_i = 0.f;
      if (tid < nb) {
        const size_t base = (size_t)pieces.slot_of(k0 + tid) * G + col;
        m_i = ws_ml[base * 2];
        l_i = ws_ml[base * 2 + 1];
      }
      float mx = m_i;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if (lane == 0) red_s[warp] = mx;
      __syncthreads();
      const float M_new = fmaxf(M, fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3])));
      __syncthreads();
      const float w_i = tid < nb ? fast_exp2(m_i - M_new) : 0.f;
      wgt_s[tid] = w_i;
      float ls = l_i * w_i;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o);
      if (lane == 0) red_s[warp] = ls;
      __syncthreads();
      const float rescale = M == -INFINITY ? 0.f : fast_exp2(M - M_new);
      L = L * rescale + ((red_s[0] + red_s[1]) + (red_s[2] + red_s[3]));
      acc.x *= rescale; acc.y *= rescale; acc.z *= rescale; acc.w *= rescale;
#pragma unroll 4
      for (int i = warp; i < nb; i += 4) {
        const size_t base = (size_t)pieces.slot_of(k0 + i) * G + col;
        const float4 o = *reinterpret_cast<const float4*>(ws_o + base * kD + 4 * lane);
        const float wg = wgt_s[i];
        acc.x = fmaf(o.x, wg, acc.x); acc.y = fmaf(o.y, wg, acc.y);
        acc.z = fmaf(o.z, wg, acc.z); acc.w = fmaf(o.w, wg, acc.w);
      }
      M = M_new;
      __syncthreads();  // before wgt_s / red_s are rewritten
    }
    *reinterpret_cast<float4*>(&acc_s[warp][4 * lane]) = acc;
    __syncthreads();
    const float v = (acc_s[0][tid] + acc_s[1][tid]) + (acc_s[2][tid] + acc_s[3][tid]);
    out[b * o_sb + (long long)(h * G + col) * o_sh + tid] = (uint16_t)float_to_bf16_bits(v / L);
    __syncthreads();  // before acc_s is rewritten for the next column
  }
}

static size_t main_smem_bytes(int B, bool scalar) {
  size_t s = (size_t)kWarps * kStages * kTileBytes;
  if (scalar) s += (size_t)kWarps * (kMaxG * kD + kMaxG * kTile) * 4;
  s += (size_t)(kWarps * 32 + 1 + kSmemLens + 1) * 4;
  (void)B;
  return s;
}

}  // namespace b200kv

using namespace b200kv;

extern "C" size_t b200kv_decode_attn_workspace_bytes(int32_t B, int32_t Hq, int32_t Hkv, int32_t D, int32_t sm_count) {
  if (B < 0 || Hq < 1 || Hkv < 1 || Hq % Hkv || D != kD || sm_count < 1) return 0;
  const int G = Hq / Hkv;
  const int W = sm_count * kCtasPerSm * kWarps;
  return ws_head_bytes(B, Hkv) + ws_ml_bytes(W, G) + (size_t)W * 2 * G * kD * 4;
}

extern "C" size_t b200kv_decode_attn_workspace_zero_bytes(int32_t B, int32_t Hkv) {
  if (B < 0 || Hkv < 1) return 0;
  return ws_head_bytes(B, Hkv);
}

// Argument checks shared by the three decode-attention entry points; nothing is enqueued before they pass.
static int check_decode_args(const void* q, int64_t q_sb, int64_t q_sh, const b200kv_cache* cache,
                             const b200kv_table* table, const int32_t* cached_lens, const int32_t* num_decoding,
                             const void* out, int64_t o_sb, int64_t o_sh, const void* workspace, size_t workspace_bytes,
                             int32_t B, int32_t Hq, int32_t sm_count, int32_t variant) {
  if (!q || !cached_lens || !num_decoding || !out || !workspace) return B200KV_E_NULL;
  int rc = check_cache(cache, table);
  if (rc) return rc;
  const int Hkv = cache->num_kv_heads;
  if (B < 0 || Hq < 1 || Hq % Hkv || Hq / Hkv > kMaxG || sm_count < 1 || variant < 0 || variant > 7) return B200KV_E_SHAPE;
  if (B > kMaxB) return B200KV_E_RANGE;
  if (!aligned(q, 16) || !aligned(out, 16) || !aligned(workspace, 256) || (q_sb % 8) || (q_sh % 8) || (o_sb % 8) || (o_sh % 8))
    return B200KV_E_ALIGN;
  if (workspace_bytes < b200kv_decode_attn_workspace_bytes(B, Hq, Hkv, kD, sm_count)) return B200KV_E_WORKSPACE;
  return B200KV_OK;
}

// Launch (arguments already checked).  `clear_bytes` > 0: that many bytes at the head of the workspace are
// zeroed on the stream first (the built-in scratch keeps the previous call's contents).
static int launch_decode(const void* q, int64_t q_sb, int64_t q_sh, const b200kv_cache* cache, const b200kv_table* table,
                         const int32_t* cached_lens, const int32_t* num_decoding, float scale, void* out, int64_t o_sb,
                         int64_t o_sh, void* workspace, size_t clear_bytes, int32_t B, int32_t Hq, int32_t sm_count,
                         int32_t variant, const void* plan, int32_t* status, void* stream) {
  const int Hkv = cache->num_kv_heads;
  const int G = Hq / Hkv;
  const int W = sm_count * kCtasPerSm * kWarps;
  // Only CTAs that can have work are launched.  No entry has more tiles than its table row can address; a warp takes
  // at least 4 tiles, except in a batch of short sequences (32 tiles or fewer on average, make_partition), where it
  // takes at least 2 - and such a batch has at most 32 B Hkv tiles, i.e. 4 B Hkv CTAs.
  const long long max_tiles = (long long)B * Hkv * (((long long)table->max_pages * cache->page_size + kTile - 1) / kTile);
  const long long want_long = (max_tiles + 4 * kWarps - 1) / (4 * kWarps);
  const long long want_short = std::min<long long>((max_tiles + 2 * kWarps - 1) / (2 * kWarps), 4LL * B * Hkv);
  const long long want = std::max(want_long, want_short);
  const int grid = (int)std::max<long long>(1, std::min<long long>(sm_count * kCtasPerSm, want));
  const float scale_log2 = scale * 1.4426950408889634f;
  cudaStream_t s = (cudaStream_t)stream;
  const bool scalar = (variant & 1) != 0;
  const int fused = (variant & 2) ? 0 : 1;
  const int early = ((variant & 4) && fused) ? 1 : 0;  // the separate reduction kernel's prefix array is written before the wait
  const size_t smem = main_smem_bytes(B, scalar);
  // the opt-in to more than 48 KB of dynamic shared memory is per function AND per device: set on every call
  cudaError_t e = scalar ? cudaFuncSetAttribute(decode_attn_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                         : cudaFuncSetAttribute(decode_attn_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return B200KV_E_LAUNCH;
  if (clear_bytes && cudaMemsetAsync(workspace, 0, clear_bytes, s) != cudaSuccess) return B200KV_E_LAUNCH;
  CacheView view = make_view(cache, table);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = early ? 1 : 0;
  cudaError_t le = cudaLaunchKernelEx(&cfg, scalar ? decode_attn_kernel<true> : decode_attn_kernel<false>,
                                      (const uint16_t*)q, (long long)q_sb, (long long)q_sh, view, cached_lens, num_decoding,
                                      scale_log2, (uint16_t*)out, (long long)o_sb, (long long)o_sh, (uint8_t*)workspace,
                                      (int)B, G, W, fused, early, (const int*)plan, status);
  if (le != cudaSuccess) return B200KV_E_LAUNCH;
  if (cudaGetLastError() != cudaSuccess) return B200KV_E_LAUNCH;
  if (fused) return B200KV_OK;
  decode_combine_kernel<<<dim3(B, Hkv), kD, 0, s>>>((const uint8_t*)workspace, num_decoding, (uint16_t*)out, o_sb, o_sh, B,
                                                    Hkv, G, W);
  return cudaGetLastError() == cudaSuccess ? B200KV_OK : B200KV_E_LAUNCH;
}

extern "C" int b200kv_decode_attn(const void* q, int64_t q_sb, int64_t q_sh, const b200kv_cache* cache,
                                  const b200kv_table* table, const int32_t* cached_lens, const int32_t* num_decoding,
                                  float scale, void* out, int64_t o_sb, int64_t o_sh, void* workspace,
                                  size_t workspace_bytes, int32_t B, int32_t Hq, int32_t sm_count, int32_t variant,
                                  int32_t* status, void* stream) {
  // an empty batch is valid and has nothing to launch (its tensors have no storage, so their pointers are NULL)
  if (B == 0) return B200KV_OK;
  const int rc = check_decode_args(q, q_sb, q_sh, cache, table, cached_lens, num_decoding, out, o_sb, o_sh, workspace,
                                   workspace_bytes, B, Hq, sm_count, variant);
  if (rc) return rc;
  return launch_decode(q, q_sb, q_sh, cache, table, cached_lens, num_decoding, scale, out, o_sb, o_sh, workspace, 0, B, Hq,
                       sm_count, variant, nullptr, status, stream);
}

extern "C" size_t b200kv_decode_plan_bytes(int32_t sm_count) {
  return sm_count < 1 ? 0 : plan_bytes(sm_count * kCtasPerSm * kWarps);
}

extern "C" int b200kv_decode_plan(const b200kv_table* table, const int32_t* cached_lens, const int32_t* num_decoding,
                                  int32_t B, int32_t Hkv, int32_t page_size, int32_t sm_count, void* plan,
                                  size_t plan_bytes_given, void* stream) {
  if (!table || !table->ids || !cached_lens || !num_decoding || !plan) return B200KV_E_NULL;
  if (B < 0 || Hkv < 1 || page_size < 1 || sm_count < 1 || table->max_pages < 1 || table->stride < 0) return B200KV_E_SHAPE;
  if (table->max_pages > 1 && (page_size % kTile) != 0) return B200KV_E_SHAPE;
  if (B > kMaxB) return B200KV_E_RANGE;
  if (!aligned(plan, 16)) return B200KV_E_ALIGN;
  if (plan_bytes_given < b200kv_decode_plan_bytes(sm_count)) return B200KV_E_WORKSPACE;
  const int W = sm_count * kCtasPerSm * kWarps;
  decode_plan_kernel<<<1, kPlanThreads, 0, (cudaStream_t)stream>>>(cached_lens, num_decoding, table->ids, table->stride,
                                                                   table->max_pages, page_size, B, Hkv, W, (int*)plan);
  return cudaGetLastError() == cudaSuccess ? B200KV_OK : B200KV_E_LAUNCH;
}

extern "C" int b200kv_decode_attn_planned(const void* q, int64_t q_sb, int64_t q_sh, const b200kv_cache* cache,
                                          const b200kv_table* table, const int32_t* cached_lens,
                                          const int32_t* num_decoding, float scale, void* out, int64_t o_sb, int64_t o_sh,
                                          void* workspace, size_t workspace_bytes, const void* plan, size_t plan_bytes_given,
                                          int32_t B, int32_t Hq, int32_t sm_count, int32_t variant, int32_t* status,
                                          void* stream) {
  if (B == 0) return B200KV_OK;
  if (!plan) return B200KV_E_NULL;
  const int rc = check_decode_args(q, q_sb, q_sh, cache, table, cached_lens, num_decoding, out, o_sb, o_sh, workspace,
                                   workspace_bytes, B, Hq, sm_count, variant);
  if (rc) return rc;
  if (variant & 2) return B200KV_E_SHAPE;  // the two-kernel reduction reads a prefix array only the unplanned kernel writes
  if (!aligned(plan, 16)) return B200KV_E_ALIGN;
  if (plan_bytes_given < b200kv_decode_plan_bytes(sm_count)) return B200KV_E_WORKSPACE;
  return launch_decode(q, q_sb, q_sh, cache, table, cached_lens, num_decoding, scale, out, o_sb, o_sh, workspace, 0, B, Hq,
                       sm_count, variant, plan, status, stream);
}

#ifdef B200KV_STAMPS
extern "C" int b200kv_stamps_read(unsigned long long* host, int clear) {
  cudaError_t e = cudaMemcpyFromSymbol(host, b200kv::g_stamps, sizeof(unsigned long long) * kStampWarps * kStampWords);
  if (e == cudaSuccess && clear) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, b200kv::g_stamps);
    if (e == cudaSuccess) e = cudaMemset(p, 0, sizeof(unsigned long long) * kStampWarps * kStampWords);
  }
  return e == cudaSuccess ? kStampWarps : -1;
}
#endif

// ------------------------------------------------------------------ entry point that allocates nothing
// Some hosts of this library may not create device memory at all when they reach the attention
// call: a serving process that hands the whole HBM budget to its own KV-cache pool at start-up has
// nothing left for cudaMalloc to carve from, a plug-in that runs inside someone else's stream
// capture must not call an allocator (cudaMalloc synchronises the device and is illegal while
// capturing), and latency-critical loops avoid it because its cost is unbounded.  For them the
// scratch of the decode kernel (arrival counters + split partials) lives in a fixed array that is
// part of the library image: every GPU that loads the library holds these bytes until the process
// exits.
namespace b200kv {
constexpr size_t kStaticScratchBytes = 8u << 20;  // 148 SMs, 8 KV heads: Hq/Hkv = 2 to B ~ 130,000, Hq/Hkv = 4 to B ~ 25,000
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
constexpr int kMaxDevices = 64;
static unsigned char* g_static_scratch_ptr[kMaxDevices] = {};  // device address per ordinal, set on first use
}  // namespace b200kv

extern "C" size_t b200kv_decode_attn_static_limit(void) { return kStaticScratchBytes; }

extern "C" int b200kv_decode_attn_static(const void* q, int64_t q_sb, int64_t q_sh, const b200kv_cache* cache,
                                         const b200kv_table* table, const int32_t* cached_lens,
                                         const int32_t* num_decoding, float scale, void* out, int64_t o_sb,
                                         int64_t o_sh, int32_t B, int32_t Hq, int32_t sm_count, int32_t* status,
                                         void* stream) {
  if (!cache) return B200KV_E_NULL;
  const size_t need = b200kv_decode_attn_workspace_bytes(B, Hq, cache->num_kv_heads, cache->head_dim, sm_count);
  if (need == 0) return B200KV_E_SHAPE;
  if (need > kStaticScratchBytes) return B200KV_E_STATIC_LIMIT;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200KV_E_LAUNCH;
  if (!g_static_scratch_ptr[dev]) {
    // In host code the array's name is only a handle; the kernel needs the address the symbol has
    // on the current device.  Done once per device, with that device current.
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) return B200KV_E_LAUNCH;
    g_static_scratch_ptr[dev] = static_cast<unsigned char*>(p);
  }
  unsigned char* scratch = g_static_scratch_ptr[dev];
  if (B == 0) return B200KV_OK;
  const int rc = check_decode_args(q, q_sb, q_sh, cache, table, cached_lens, num_decoding, out, o_sb, o_sh, scratch,
                                   kStaticScratchBytes, B, Hq, sm_count, 0);
  if (rc) return rc;  // nothing has been enqueued
  // The array keeps whatever the previous call (possibly of another batch size) left behind; the
  // prefix + arrival-counter head of THIS call's layout is cleared on the stream ahead of the kernel.
  return launch_decode(q, q_sb, q_sh, cache, table, cached_lens, num_decoding, scale, out, o_sb, o_sh, scratch,
                       ws_head_bytes(B, cache->num_kv_heads), B, Hq, sm_count, 0, nullptr, status, stream);
}
