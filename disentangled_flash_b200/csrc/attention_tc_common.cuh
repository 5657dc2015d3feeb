// Pieces shared by the two tcgen05 attention kernels (scores staged from global memory, and
// scores computed in-kernel): 16-bit packing, mixed-precision adds, and the per-tile softmax tail
// (mask -> running max/sum -> P to TMEM -> O rescale) plus the final normalise-and-store.
#pragma once

#include "dfl_common.cuh"
#include "tcgen05_ptx.cuh"

namespace dfl {
#ifdef DFL_TRACE
// Development aid (not compiled into the product): per-warp event timestamps of CTA (1, 0).
static __device__ long long g_trace[16 * 512];
#define TRACE_DECL int trace_n = 0;
#define TRACE_PARAM , int& trace_n
#define TRACE_ARG , trace_n
#define TRACE(ev)                                                                              \
  do {                                                                                         \
    if (blockIdx.x == 1 && blockIdx.y == 0 && (threadIdx.x & 31) == 0 && trace_n < 512)         \
      g_trace[(threadIdx.x >> 5) * 512 + trace_n++] = (clock64() << 8) | (long long)(ev);       \
  } while (0)
#else
#define TRACE_DECL
#define TRACE_PARAM
#define TRACE_ARG
#define TRACE(ev) do { } while (0)
#endif
namespace attn {

constexpr int BM = 128;  // query rows per CTA (= TMEM lanes)
constexpr int BN = 64;   // keys per tile

template <typename T>
struct Pack2;
template <>
struct Pack2<__half> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  // acc + (float)x with x a raw fp16 bit pattern: one instruction, no separate conversion
  static __device__ __forceinline__ float add(float acc, uint16_t x) {
    float d;
    asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(d) : "h"(x), "f"(acc));
    return d;
  }
  // sum of the two packed values, exactly as the tensor core will read them
  static __device__ __forceinline__ float sum2(uint32_t w) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    return f.x + f.y;
  }
  // both packed values times c, rounded again
  static __device__ __forceinline__ uint32_t scale2(uint32_t w, float c) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    return pack(f.x * c, f.y * c);
  }
};
template <>
struct Pack2<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float add(float acc, uint16_t x) {
    float d;
    asm("add.rn.f32.bf16 %0, %1, %2;" : "=f"(d) : "h"(x), "f"(acc));
    return d;
  }
  static __device__ __forceinline__ float sum2(uint32_t w) {
    return __uint_as_float(w << 16) + __uint_as_float(w & 0xffff0000u);
  }
  static __device__ __forceinline__ uint32_t scale2(uint32_t w, float c) {
    return pack(__uint_as_float(w << 16) * c, __uint_as_float(w & 0xffff0000u) * c);
  }
};

// Per-thread online-softmax state of one query row.
struct RowState {
  float m_run = -INFINITY;  // running maximum, unscaled score units
  float l_run = 0.0f;       // running sum of exp2
};

// Everything after the relative scores have been added to s[]:
//   mask (keys >= L and padded keys -> -inf; padded query row -> 0 on in-range keys),
//   running max / sum in base 2, P rounded to T and written to TMEM at t_p (BN/2 packed columns),
//   O (at t_o, D fp32 columns) rescaled when the maximum of any row of the warp moved,
//   then p_full is signalled.  Returns false if a bounded wait expired.
template <typename T, int D>
__device__ __forceinline__ bool softmax_tile_tail(float (&s)[BN], RowState& st, uint32_t kb0, uint32_t kb1, int n_in,
                                                  bool q_keep, float cscale, int kt, uint32_t t_o, uint32_t t_p,
                                                  uint64_t* o_ready, uint64_t* p_full, volatile int* abort_flag,
                                                  int* status_word) {
  if (!q_keep) {
#pragma unroll
    for (int jj = 0; jj < BN; ++jj) s[jj] = jj < n_in ? 0.0f : -INFINITY;
  } else if ((kb0 & kb1) != 0xffffffffu) {
#pragma unroll
    for (int jj = 0; jj < BN; ++jj) {
      const uint32_t w = jj < 32 ? kb0 : kb1;
      if (!((w >> (jj & 31)) & 1u)) s[jj] = -INFINITY;
    }
  }
  float tile_max = -INFINITY;
#pragma unroll
  for (int jj = 0; jj < BN; ++jj) tile_max = fmaxf(tile_max, s[jj]);
  const float m_new = fmaxf(st.m_run, tile_max);
  const float m_use = m_new == -INFINITY ? 0.0f : m_new;  // nothing attended yet: avoid inf - inf
  const float corr = ptx::ex2_approx((st.m_run - m_use) * cscale);  // 0 when m_run = -inf
  const float neg_m = -m_use * cscale;
  float tile_sum = 0.0f;
  uint32_t packed[BN / 2];
#pragma unroll
  for (int jj = 0; jj < BN; jj += 2) {
    const float p0 = ptx::ex2_approx(fmaf(s[jj], cscale, neg_m));
    const float p1 = ptx::ex2_approx(fmaf(s[jj + 1], cscale, neg_m));
    tile_sum += p0 + p1;
    packed[jj / 2] = Pack2<T>::pack(p0, p1);
  }
  st.l_run = st.l_run * corr + tile_sum;
  st.m_run = m_new;

  // O accumulated so far (tiles < kt) must be complete before it is rescaled or P(kt) is consumed
  if (kt > 0) {
    if (!ptx::mbar_wait(o_ready, (uint32_t)(kt - 1) & 1u, abort_flag, status_word, 9)) return false;
    ptx::tc_fence_after();
    if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t o[32];
        ptx::tmem_ld32(t_o + c0, o);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int x = 0; x < 32; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * corr);
        ptx::tmem_st32(t_o + c0, o);
      }
    }
  }
  {
    uint32_t (&pk)[32] = *reinterpret_cast<uint32_t (*)[32]>(&packed[0]);
    ptx::tmem_st32(t_p, pk);
  }
  ptx::tmem_wait_st();
  ptx::tc_fence_before();
  ptx::mbar_arrive(p_full);
  return true;
}

// ---------------------------------------------------------------------------------------------
// Column-split variant: PARTS threads (in warps w, w+4, ... - same TMEM lane quarter) share one query
// row, each owning W = BN/PARTS keys of every tile and D/PARTS output columns.  The row maximum of a
// tile is agreed through shared memory and a per-quarter mbarrier (bounded wait like every other wait).
// ---------------------------------------------------------------------------------------------
constexpr float kLazyMaxSlack = 8.0f;  // log2 of the largest P that may reach the tensor core

struct RowExchange {
  float* slot;          // [2 (tile parity)][PARTS][BM] floats in shared memory
  uint64_t* bar;        // mbarrier of this lane quarter: one arrival per warp (PARTS per phase)
};

__device__ __forceinline__ void tmem_ld_n(uint32_t taddr, uint32_t (&r)[32]) { ptx::tmem_ld32(taddr, r); }
__device__ __forceinline__ void tmem_ld_n(uint32_t taddr, uint32_t (&r)[16]) { ptx::tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_ld_n(uint32_t taddr, uint32_t (&r)[8]) { ptx::tmem_ld8(taddr, r); }
__device__ __forceinline__ void tmem_st_n(uint32_t taddr, const uint32_t (&r)[32]) { ptx::tmem_st32(taddr, r); }
__device__ __forceinline__ void tmem_st_n(uint32_t taddr, const uint32_t (&r)[16]) { ptx::tmem_st16(taddr, r); }
__device__ __forceinline__ void tmem_st_n(uint32_t taddr, const uint32_t (&r)[8]) { ptx::tmem_st8(taddr, r); }

// s[] holds the thread's W scores (keys part*W ... of the tile) with the relative scores added.
// kb: keep-bits of those keys (bit x = key x of the part).  n_in: in-range keys of the part (may be <= 0).
// t_o_part: TMEM address of the thread's D/PARTS output columns; t_p_part: of its W/2 packed P columns.
template <typename T, int D, int PARTS>
__device__ __forceinline__ bool softmax_part_tail(float (&s)[BN / PARTS], RowState& st, uint32_t kb, int n_in,
                                                  bool q_keep, float cscale, int kt, int part, int row,
                                                  const RowExchange& xc, uint32_t t_o_part, uint32_t t_p_part,
                                                  uint64_t* o_ready, uint64_t* p_full, volatile int* abort_flag,
                                                  int* status_word TRACE_PARAM) {
  constexpr int W = BN / PARTS;
  constexpr uint32_t kAll = W == 32 ? 0xffffffffu : ((1u << W) - 1u);
  if (!q_keep) {
#pragma unroll
    for (int x = 0; x < W; ++x) s[x] = x < n_in ? 0.0f : -INFINITY;
  } else if ((kb & kAll) != kAll) {
#pragma unroll
    for (int x = 0; x < W; ++x)
      if (!(kb & (1u << x))) s[x] = -INFINITY;
  }
  // tree-shaped maximum (a serial chain of W dependent max operations would stall the warp)
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int x = 0; x < W; ++x) mx[x & 3] = fmaxf(mx[x & 3], s[x]);
  const float part_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
  // agree on the tile maximum with the threads that own the other parts of this row
  float* base = xc.slot + (kt & 1) * PARTS * BM + row;
  base[part * BM] = part_max;
  __syncwarp();
  if ((threadIdx.x & 31) == 0) ptx::mbar_arrive(xc.bar);
  if (!ptx::mbar_wait(xc.bar, (uint32_t)kt & 1u, abort_flag, status_word, 22)) return false;
  float tile_max = part_max;
#pragma unroll
  for (int q = 0; q < PARTS; ++q) tile_max = fmaxf(tile_max, base[q * BM]);
  TRACE(51);

  // Lazy reference maximum: st.m_run only moves when the tile maximum exceeds it by more than 2^8 after
  // scaling, so exp2 arguments stay <= 8 (P <= 256, exact range of both 16-bit types) and the O accumulator
  // in TMEM needs rescaling only on those rare tiles.  All threads of a row see the same tile_max and m_run.
  const bool move = tile_max > st.m_run + kLazyMaxSlack / cscale;  // also true for the first finite maximum
  const float m_new = move ? tile_max : st.m_run;
  const float m_use = m_new == -INFINITY ? 0.0f : m_new;
  const float corr = move ? ptx::ex2_approx((st.m_run - m_use) * cscale) : 1.0f;
  const float neg_m = -m_use * cscale;
  float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  uint32_t packed[W / 2];
#pragma unroll
  for (int x = 0; x < W; x += 2) {
    const float p0 = ptx::ex2_approx(fmaf(s[x], cscale, neg_m));
    const float p1 = ptx::ex2_approx(fmaf(s[x + 1], cscale, neg_m));
    sum[(x >> 1) & 3] += p0 + p1;
    packed[x / 2] = Pack2<T>::pack(p0, p1);
  }
  // partial sum over this thread's keys; corr is the same in every part of the row
  st.l_run = st.l_run * corr + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
  st.m_run = m_new;
  TRACE(52);

  // O is rescaled only on the rare tiles where the reference maximum moved; only then does this thread
  // have to see PV(kt-1) complete.  (The P buffer written below was last read by PV(kt-2), which is
  // complete because S(kt), issued after it, has already been observed.)
  if (kt > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {  // same decision in every warp of the row group
    if (!ptx::mbar_wait(o_ready, (uint32_t)(kt - 1) & 1u, abort_flag, status_word, 9)) return false;
    ptx::tc_fence_after();
    {
      uint32_t o[D / PARTS];
      tmem_ld_n(t_o_part, o);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int x = 0; x < D / PARTS; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * corr);
      tmem_st_n(t_o_part, o);
    }
  }
  TRACE(53);
  tmem_st_n(t_p_part, packed);
  ptx::tmem_wait_st();
  TRACE(54);
  ptx::tc_fence_before();
  __syncwarp();
  if ((threadIdx.x & 31) == 0) ptx::mbar_arrive(p_full);
  return true;
}

// Final step of the column-split variant: add the partial row sums, normalise and store the thread's
// D/PARTS output columns to out_part.
template <typename T, int D, int PARTS>
__device__ __forceinline__ void softmax_part_store(const RowState& st, bool ok, bool row_ok, int n_kt, int part, int row,
                                                   const RowExchange& xc, uint32_t t_o_part, T* out_part,
                                                   uint64_t* o_ready, volatile int* abort_flag, int* status_word) {
  float* base = xc.slot + (n_kt & 1) * PARTS * BM + row;
  base[part * BM] = st.l_run;
  __syncwarp();
  if ((threadIdx.x & 31) == 0) ptx::mbar_arrive(xc.bar);
  if (ok) ok = ptx::mbar_wait(xc.bar, (uint32_t)n_kt & 1u, abort_flag, status_word, 23);
  float total = 0.0f;
#pragma unroll
  for (int q = 0; q < PARTS; ++q) total += base[q * BM];
  const float inv = 1.0f / total;
  if (ok) ok = ptx::mbar_wait(o_ready, (uint32_t)(n_kt - 1) & 1u, abort_flag, status_word, 10);
  ptx::tc_fence_after();
  uint32_t o[D / PARTS];
  tmem_ld_n(t_o_part, o);
  ptx::tmem_wait_ld();
  if (ok && row_ok) {
#pragma unroll
    for (int v = 0; v < D / PARTS / 8; ++v) {
      uint4 pk;
      pk.x = Pack2<T>::pack(__uint_as_float(o[v * 8 + 0]) * inv, __uint_as_float(o[v * 8 + 1]) * inv);
      pk.y = Pack2<T>::pack(__uint_as_float(o[v * 8 + 2]) * inv, __uint_as_float(o[v * 8 + 3]) * inv);
      pk.z = Pack2<T>::pack(__uint_as_float(o[v * 8 + 4]) * inv, __uint_as_float(o[v * 8 + 5]) * inv);
      pk.w = Pack2<T>::pack(__uint_as_float(o[v * 8 + 6]) * inv, __uint_as_float(o[v * 8 + 7]) * inv);
      *reinterpret_cast<uint4*>(out_part + v * 8) = pk;
    }
  }
}

// Wait for the last PV, normalise the row and store it to out_row (D contiguous elements).
template <typename T, int D>
__device__ __forceinline__ void softmax_store_row(const RowState& st, bool ok, bool row_ok, int n_kt, uint32_t t_o,
                                                  T* out_row, uint64_t* o_ready, volatile int* abort_flag,
                                                  int* status_word) {
  if (ok) ok = ptx::mbar_wait(o_ready, (uint32_t)(n_kt - 1) & 1u, abort_flag, status_word, 10);
  ptx::tc_fence_after();
  const float inv = 1.0f / st.l_run;
#pragma unroll
  for (int c0 = 0; c0 < D; c0 += 32) {
    uint32_t o[32];
    ptx::tmem_ld32(t_o + c0, o);
    ptx::tmem_wait_ld();
    if (ok && row_ok) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        uint4 pk;
        pk.x = Pack2<T>::pack(__uint_as_float(o[v * 8 + 0]) * inv, __uint_as_float(o[v * 8 + 1]) * inv);
        pk.y = Pack2<T>::pack(__uint_as_float(o[v * 8 + 2]) * inv, __uint_as_float(o[v * 8 + 3]) * inv);
        pk.z = Pack2<T>::pack(__uint_as_float(o[v * 8 + 4]) * inv, __uint_as_float(o[v * 8 + 5]) * inv);
        pk.w = Pack2<T>::pack(__uint_as_float(o[v * 8 + 6]) * inv, __uint_as_float(o[v * 8 + 7]) * inv);
        *reinterpret_cast<uint4*>(out_row + c0 + v * 8) = pk;
      }
    }
  }
}

// Load one S tile row (BN fp32 columns at t_s) into registers.
__device__ __forceinline__ void load_scores(uint32_t t_s, float (&s)[BN]) {
  uint32_t raw[32];
#pragma unroll
  for (int half = 0; half < BN / 32; ++half) {
    ptx::tmem_ld32(t_s + half * 32, raw);
    ptx::tmem_wait_ld();
#pragma unroll
    for (int x = 0; x < 32; ++x) s[half * 32 + x] = __uint_as_float(raw[x]);
  }
}

}  // namespace attn
}  // namespace dfl
