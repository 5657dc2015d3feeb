// Pieces shared by the two tcgen05 attention kernels (scores staged from global memory, and
// scores computed in-kernel): 16-bit packing and mixed-precision adds; for the first kernel also the
// per-tile softmax tail (mask -> running max/sum -> P to TMEM -> O rescale) and the final
// normalise-and-store.
#pragma once

#include "dfl_common.cuh"
#include "tcgen05_ptx.cuh"

namespace dfl {
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

// Slack of the lazy reference maximum used by the relative-table kernel: its running maximum moves only when a tile
// exceeds it by more than 2^kLazyMaxSlack after scaling.
constexpr float kLazyMaxSlack = 8.0f;  // log2 of the largest P that may reach the tensor core

__device__ __forceinline__ void tmem_ld_n(uint32_t taddr, uint32_t (&r)[32]) { ptx::tmem_ld32(taddr, r); }
__device__ __forceinline__ void tmem_ld_n(uint32_t taddr, uint32_t (&r)[16]) { ptx::tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_ld_n(uint32_t taddr, uint32_t (&r)[8]) { ptx::tmem_ld8(taddr, r); }
__device__ __forceinline__ void tmem_st_n(uint32_t taddr, const uint32_t (&r)[32]) { ptx::tmem_st32(taddr, r); }
__device__ __forceinline__ void tmem_st_n(uint32_t taddr, const uint32_t (&r)[16]) { ptx::tmem_st16(taddr, r); }
__device__ __forceinline__ void tmem_st_n(uint32_t taddr, const uint32_t (&r)[8]) { ptx::tmem_st8(taddr, r); }

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
