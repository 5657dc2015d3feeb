// tcgen05 fused disentangled attention over position tables laid out by relative distance.
//
// Same result as dfl_pos_scores + dfl_attention_fwd (reference: the two torch.matmul calls at
// src/disentangled_flash/kernel.py:574-585 followed by the Triton kernel kernel.py:137-345).  The tables
// rel_key / rel_query [H, 2L-1, d] hold, in row e, the position projection every (query i, key j) pair with
// x = j - i = e - (L-1) uses, so the two relative terms of a (128 query x 64 key) tile are
//   C2P[i, j] = q_i . rel_key[x]      P2C[i, j] = k_j . rel_query[x]
// with x running over one contiguous window of 191 table rows.  Both are produced by tcgen05.mma from
// 64-row table blocks (L2 resident), rounded to the input type exactly like the separate score GEMMs round
// their output, and parked in shared memory, where the softmax threads pick them up along diagonals.
//   C2P depends on the query rows only: per query row a ring of four 64-column blocks is kept across key
//       tiles (a key tile needs one new block; the first tile of an item three).
//   P2C is new for every key tile: PT[m, n] = rel_query[x_lo + m] . k_n (two 128x64xd MMAs over a ring of four
//       table blocks, three of them live), so that TMEM lanes are table rows and all lanes convert.
//
// Persistent: one CTA per SM walks (batch, head, query tile) items; every role keeps running counters so that
// the barrier phases carry over from item to item and the loader / MMA issuer run ahead into the next item.
// Sixteen warps:
//   warps 0-3   softmax stream 0: one thread per query row, key tiles 0, 2, 4, ... of the item
//   warps 4-7   softmax stream 1: key tiles 1, 3, 5, ...  Each stream has its own running maximum, row sum and
//               output accumulator in TMEM (no per-tile exchange); the two are merged once per item.
//   warps 8-11  converters: TMEM -> 16-bit -> shared memory for the C2P blocks and the PT tiles
//   warps 12-13 PV issuers, one per stream: O[g] (+)= P[g] V as soon as the stream has stored P
//   warp 14     per-item mask analysis (kept-key bits, skipped key tiles) and TMA producer
//   warp 15     issuer of the "front" MMAs of a tile (new C2P block, PT, S) and TMEM owner
#include <type_traits>

#include "attention_tc_common.cuh"

namespace dfl {

__device__ int g_attn_rel_status = 0;

namespace {

using attn::BM;
using attn::BN;
using attn::Pack2;

constexpr int kSoftmaxWarps = 8;
constexpr int kConvHiWarp0 = 12;      // end of the converter warps
constexpr int kPvWarp0 = 12;
constexpr int kTmaWarp = 14;
constexpr int kMmaWarp = 15;
constexpr int kThreads = 512;
constexpr int kSoftmaxRegs = 176;   // 256 threads x 176 + 256 threads x 80 = 65536 registers
constexpr int kOtherRegs = 80;

constexpr int RING_COLS = 256;                 // four 64-column blocks per query row
constexpr int RING_MIRROR = 16;                // columns 0..15 repeated at 256..271: a 16-key run never wraps
constexpr int RING_PITCH_H = 290;              // halfs per ring row (bank spread of the diagonal reads: 1.5 wavefronts)
constexpr int PT_ROWS = 192;
constexpr int PT_PITCH_H = BN + 2;             // 33 words: the anti-diagonal reads are conflict free
constexpr int kMaxSeqLen = 1024;               // 32 words of kept-key bits per item

// TMEM columns (all 512; one CTA per SM)
constexpr int COL_S = 0;       // 2 x 64   S of stream 0 / 1
constexpr int COL_P = 128;     // 2 x 32   P (16-bit pairs) of stream 0 / 1
constexpr int COL_O = 192;     // 2 x 64   O of stream 0 / 1 (first D columns used)
constexpr int COL_CNEW = 320;  // 64       one C2P block for 128 query rows
constexpr int COL_PT = 384;    // 2 x 64   PT accumulators
constexpr int kTmemCols = 512;

template <int D>
struct RLayout {
  static_assert(D == 32 || D == 64, "head dims 32 and 64");
  static constexpr int kRowBytes = D * 2;
  static constexpr int kQ = BM * kRowBytes;     // Q tile
  static constexpr int kBlk = BN * kRowBytes;   // K tile, V tile, one 64-row table block
  static constexpr int offQ = 0;
  static constexpr int offK = offQ + kQ;              // 2 stages
  static constexpr int offV = offK + 2 * kBlk;        // 2 stages
  static constexpr int offPK = offV + 2 * kBlk;       // 2 rel_key blocks
  static constexpr int offFQ = offPK + 2 * kBlk;      // ring of 4 rel_query blocks
  // The second PT MMA reads 128 operand rows from a 64-row block; the rows past it (the next block, or the start
  // of the C2P ring after the last block) only feed TMEM lanes 64..127, which nobody reads.
  static constexpr int offRing = offFQ + 4 * kBlk;                 // C2P ring [128][RING_PITCH_H]
  static constexpr int offPT = offRing + BM * RING_PITCH_H * 2;    // PT staging, one per stream
  static constexpr int kPTStage = PT_ROWS * PT_PITCH_H * 2;
  static constexpr int offBar = (offPT + 2 * kPTStage + 15) & ~15;
  static constexpr int kBarBytes = 512;
  // two exchange slots (by item parity) of [2 streams][BM] (max, sum); then the mean-of-V scratch: [256] partial
  // sums and the [D] column mean
  static constexpr int offXchg = offBar + kBarBytes;
  static constexpr int kXchgSlot = 2 * BM * 8;
  static constexpr int offMeanV = offXchg + 2 * kXchgSlot;
  static constexpr int kXchgBytes = 2 * kXchgSlot + 1024 + 256;
  static constexpr int offItem = offXchg + kXchgBytes; // 2 item slots
  static constexpr int kItemBytes = 160;
  static constexpr int total = offItem + 2 * kItemBytes + 1024;   // + alignment slack
};

// What the loader warp publishes per item.
struct ItemSlot {
  int t_begin, t_end;   // key tiles [t_begin, t_end) are processed
  int any_kept;         // 0: every query row of the tile is padding -> mean-of-V path, no pipeline work
  int bh, i0;           // batch*heads + head, first query row
  uint32_t kbits[32];   // kept-key bits of the batch row, word w = keys [32w, 32w+32)
};
static_assert(sizeof(ItemSlot) <= 160, "item slot too large");

struct RBarriers {
  uint64_t q_full, q_empty;
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t pk_full[2], pk_empty[2];
  uint64_t fq_full[4], fq_empty[4];
  uint64_t s_full[2], s_free[2], p_full[2], o_ready[2];
  uint64_t cnew_full, cnew_free;
  uint64_t pt_full, pt_free;
  uint64_t c2p_ready[2], ring_release[2];
  uint64_t pt_ready[2], pt_release[2];
  uint64_t item_full[2], item_empty[2];
  uint64_t xbar_a, xbar_b;
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(RBarriers) <= 512, "barrier block too large");

__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
}
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
}

// tcgen05.mma with shared-memory descriptors passed as 32-bit halves (hi is shared by both operands) and the
// accumulate flag as a compile-time constant: the issuing thread spends no instructions on building descriptors.
template <int ACC>
__device__ __forceinline__ void umma_ss_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "n"(ACC)
      : "memory");
}
template <int ACC>
__device__ __forceinline__ void umma_ts_lohi(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t hi, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(hi), "r"(idesc), "n"(ACC)
      : "memory");
}

// 16-bit shared-memory load, zero-extended into a 32-bit register (32-bit destinations keep every value in its
// own register; the address arithmetic of unrolled callers folds into the instruction's immediate offset).
__device__ __forceinline__ uint32_t lds_u16_r32(uint32_t saddr) {
  uint32_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(saddr) : "memory");
  return v;
}

// Kept-key bits of batch row b: lane w returns word w (keys [32w, 32w+32)) built from its own 32 mask elements.
__device__ __forceinline__ uint32_t kept_bits_word(const DflAttnRelParams& p, int b, int lane) {
  const int L = p.seq_len;
  uint32_t kb = 0;
  const int jw = 32 * lane;
  const long long base = (long long)b * L + jw;
  if (jw + 32 <= L && p.mask_elem_size == 1 && ((reinterpret_cast<uintptr_t>(p.mask) + base) & 15) == 0) {
    const uint4* m16 = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(p.mask) + base);
    const uint4 lo = m16[0], hi = m16[1];
    const uint32_t wds[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int x = 0; x < 32; ++x)
      if ((wds[x >> 2] >> ((x & 3) * 8)) & 0xffu) kb |= 1u << x;
  } else if (jw < L) {
#pragma unroll 8
    for (int x = 0; x < 32; ++x)
      if (jw + x < L && mask_keep(p.mask, p.mask_elem_size, base + x)) kb |= 1u << x;
  }
  return kb;
}

// Key tiles before the first and after the last kept key contribute nothing to a kept query row (their
// probabilities are exactly zero) and are skipped; a padded query row attends uniformly to all L keys, so a query
// tile that contains one walks every key tile.  A tile of padded rows only is the column mean of V (any_kept false).
// Warp-collective: kb_mine is the lane's kept-key word of the batch row.
struct TileRange {
  int t_begin, t_end;
  bool any_kept;
};
__device__ __forceinline__ TileRange tile_range(uint32_t kb_mine, int i0, int L, int lane) {
  const int n_kt = (L + BN - 1) / BN;
  const uint32_t nz = __ballot_sync(0xffffffffu, kb_mine != 0u);
  const bool in_q = lane >= (i0 >> 5) && lane < (i0 >> 5) + BM / 32;
  const int rows_here = L - 32 * lane;   // in-range rows of this lane's word
  const uint32_t full = rows_here >= 32 ? 0xffffffffu : (rows_here <= 0 ? 0u : ((1u << rows_here) - 1u));
  const bool any_kept = __ballot_sync(0xffffffffu, in_q && kb_mine != 0u) != 0u;
  const bool any_padded = __ballot_sync(0xffffffffu, in_q && (kb_mine & full) != full) != 0u;
  TileRange r{0, n_kt, any_kept};
  if (!any_padded && nz != 0u) {
    r.t_begin = (__ffs(nz) - 1) >> 1;
    r.t_end = ((31 - __clz(nz)) >> 1) + 1;
  }
  return r;
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads, 1)
attention_rel_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_fk,
                     const __grid_constant__ CUtensorMap tmap_fq, const DflAttnRelParams p, int* status_word,
                     int n_items) {
  using LO = RLayout<D>;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  RBarriers* bars = reinterpret_cast<RBarriers*>(smem + LO::offBar);
  volatile int* abort_flag = &bars->abort_flag;
  ItemSlot* slots = reinterpret_cast<ItemSlot*>(smem + LO::offItem);

  const int L = p.seq_len, H = p.heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool has_c2p = p.rel_key != nullptr, has_p2c = p.rel_query != nullptr;
  TRACE_DECL

  // ------------------------------------------------------------------ setup (once per CTA)
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bars->q_full, 1);
    ptx::mbar_init(&bars->q_empty, 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&bars->k_full[s], 1);
      ptx::mbar_init(&bars->k_empty[s], 1);
      ptx::mbar_init(&bars->v_full[s], 1);
      ptx::mbar_init(&bars->v_empty[s], 1);
      ptx::mbar_init(&bars->pk_full[s], 1);
      ptx::mbar_init(&bars->pk_empty[s], 1);
      ptx::mbar_init(&bars->s_full[s], 1);
      ptx::mbar_init(&bars->s_free[s], 4);        // one elected lane per warp of the stream
      ptx::mbar_init(&bars->p_full[s], 4);
      ptx::mbar_init(&bars->o_ready[s], 1);
      ptx::mbar_init(&bars->c2p_ready[s], 4);     // converter warps 8-11
      ptx::mbar_init(&bars->ring_release[s], 4);
      ptx::mbar_init(&bars->pt_ready[s], 4);      // converter warps 8-11
      ptx::mbar_init(&bars->pt_release[s], 4);
      ptx::mbar_init(&bars->item_full[s], 1);
      ptx::mbar_init(&bars->item_empty[s], 15);   // every warp but the loader
    }
    for (int s = 0; s < 4; ++s) {
      ptx::mbar_init(&bars->fq_full[s], 1);
      ptx::mbar_init(&bars->fq_empty[s], 1);
    }
    ptx::mbar_init(&bars->cnew_full, 1);
    ptx::mbar_init(&bars->cnew_free, 4);
    ptx::mbar_init(&bars->pt_full, 1);
    ptx::mbar_init(&bars->pt_free, 4);
    ptx::mbar_init(&bars->xbar_a, kSoftmaxWarps);
    ptx::mbar_init(&bars->xbar_b, kSoftmaxWarps);
    bars->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kTmaWarp && lane == 0) {
    ptx::prefetch_tensormap(&tmap_q);
    ptx::prefetch_tensormap(&tmap_k);
    ptx::prefetch_tensormap(&tmap_v);
    ptx::prefetch_tensormap(&tmap_fk);
    ptx::prefetch_tensormap(&tmap_fq);
  }
  if (warp == kMmaWarp) {
    ptx::tmem_alloc(&bars->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  // Item order: item = query tile * (batch*heads) + batch*head, so the items of one CTA (stride gridDim) differ in
  // query tile and batch row, which evens out the padding-dependent cost without any bookkeeping.
  const int n_bh = p.batch * H;
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  // Items of this CTA: it = blockIdx.x, blockIdx.x + gridDim.x, ...  item -> (query tile, batch*head)
  // Every role walks the same item sequence and keeps its own running counters.

  // Register budgets are set per warpgroup (warps 0-3, 4-7: softmax; 8-11: converters; 12-15: the rest), at the
  // head of the branch the whole warpgroup takes.
  auto converter_role = [&]() {
    // -------------------------------------------------------------- converters
    // Thread (quarter q4, lane) owns TMEM lane 32*q4 + lane: a query row of a C2P block, a table row of the first
    // PT accumulator and, for lanes 0..63 (warps 8 and 9), a table row of the second PT accumulator.
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    unsigned char* ring_row = smem + LO::offRing + row * (RING_PITCH_H * 2);
    uint32_t c_blk = 0, c_pt = 0, c_win = 0;   // C2P blocks converted, PT tiles converted, table-window position
    uint32_t c_t0 = 0, c_t1 = 0;               // tiles seen per stream
    bool ok = true;

    // 64 fp32 columns of this thread's TMEM lane -> registers (both halves in flight before the single wait: a TMEM
    // round trip costs several hundred cycles), then -> 64 16-bit values at dst (4-byte aligned), rounded like a
    // GEMM epilogue.  Split in two so that the TMEM buffer can be handed back between the two steps.
    auto load_64 = [&](uint32_t t_src, uint32_t (&raw0)[32], uint32_t (&raw1)[32]) {
      ptx::tmem_ld32(t_src, raw0);
      ptx::tmem_ld32(t_src + 32, raw1);
      ptx::tmem_wait_ld();
    };
    auto store_64 = [&](const uint32_t (&raw0)[32], const uint32_t (&raw1)[32], unsigned char* dst, bool mirror) {
#pragma unroll
      for (int x = 0; x < 32; x += 2) {
        const uint32_t w = Pack2<T>::pack(__uint_as_float(raw0[x]), __uint_as_float(raw0[x + 1]));
        *reinterpret_cast<uint32_t*>(dst + x * 2) = w;
        if (x < RING_MIRROR && mirror) *reinterpret_cast<uint32_t*>(dst + RING_COLS * 2 + x * 2) = w;
      }
#pragma unroll
      for (int x = 0; x < 32; x += 2)
        *reinterpret_cast<uint32_t*>(dst + 64 + x * 2) = Pack2<T>::pack(__uint_as_float(raw1[x]), __uint_as_float(raw1[x + 1]));
    };

    int k = 0;
    for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x, ++k) {
      const int slot = k & 1;
      ok = ptx::mbar_wait_inline(&bars->item_full[slot], (uint32_t)(k >> 1) & 1u, abort_flag, status_word, 32);
      if (!ok) break;
      const ItemSlot* sl = &slots[slot];
      const int n = sl->t_end - sl->t_begin;
      const bool any_kept = sl->any_kept != 0;
      for (int u = 0; u < n && ok && any_kept; ++u) {
        const int g = u & 1;
        const uint32_t c_t = g ? c_t1 : c_t0;
        if (has_c2p) {
          const int jobs = u == 0 ? 3 : 1;
          for (int x = 0; x < jobs && ok; ++x, ++c_blk) {
            ok = ptx::mbar_wait_inline(&bars->cnew_full, c_blk & 1u, abort_flag, status_word, 18);
            if (!ok) break;
            TRACE(12);
            ptx::tc_fence_after();
            uint32_t raw0[32], raw1[32];
            load_64(tmem_base + lane_base + COL_CNEW, raw0, raw1);
            // the accumulator is free as soon as it is in registers: the next block's MMA overlaps the stores
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&bars->cnew_free);
            if (x == 0) {
              // The ring position a new block overwrites was last read by the stream's previous tile; the first
              // tile of an item also overwrites positions the other stream's last tile of the previous item read.
              ok = ptx::mbar_wait_inline(&bars->ring_release[g], (c_t & 1u) ^ 1u, abort_flag, status_word, 17);
              if (ok && u == 0) ok = ptx::mbar_wait_inline(&bars->ring_release[1], (c_t1 & 1u) ^ 1u, abort_flag, status_word, 17);
              if (!ok) break;
            }
            const int pos = c_blk & 3;
            store_64(raw0, raw1, ring_row + pos * 128, pos == 0);
            TRACE(13);
          }
          if (!ok) break;
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&bars->c2p_ready[g]);
        }
        if (has_p2c) {
          ok = ptx::mbar_wait_inline(&bars->pt_full, c_pt & 1u, abort_flag, status_word, 19);
          if (!ok) break;
          TRACE(14);
          ptx::tc_fence_after();
          const int pp = c_win & 3;
          unsigned char* stage = smem + LO::offPT + g * LO::kPTStage;
          {
            uint32_t raw0[32], raw1[32];
            load_64(tmem_base + lane_base + COL_PT, raw0, raw1);
            if (q4 >= 2) {   // these warps are done with the accumulators
              ptx::tc_fence_before();
              __syncwarp();
              if (lane == 0) ptx::mbar_arrive(&bars->pt_free);
            }
            // the stream's staging tile must have been gathered by the stream's previous tile
            ok = ptx::mbar_wait_inline(&bars->pt_release[g], (c_t & 1u) ^ 1u, abort_flag, status_word, 20);
            if (!ok) break;
            TRACE(15);
            store_64(raw0, raw1, stage + ((pp == 3 ? 64 : 0) + row) * (PT_PITCH_H * 2), false);
          }
          if (q4 < 2) {
            uint32_t raw0[32], raw1[32];
            load_64(tmem_base + lane_base + COL_PT + BN, raw0, raw1);
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&bars->pt_free);
            store_64(raw0, raw1, stage + ((pp == 3 ? 0 : 128) + row) * (PT_PITCH_H * 2), false);
          }
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&bars->pt_ready[g]);
          ++c_pt;
          c_win += (u == n - 1) ? 3u : 1u;
          TRACE(16);
        }
        if (g) ++c_t1; else ++c_t0;
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bars->item_empty[slot]);
    }
  };

  // Warps 12, 13 (lane 0): PV issuer of stream 0 / 1: O[g] (+)= P[g] . V(tile) once the stream's four warps have stored P.
  auto pv_role = [&]() {
    if (lane != 0) return;
    const int g = warp - kPvWarp0;
    constexpr int is_bf16 = __is_same(T, __nv_bfloat16) ? 1 : 0;
    constexpr uint32_t idesc_pv = ptx::make_idesc_f16(is_bf16, BM, D, 0, 1);   // V is MN-major
    constexpr uint32_t desc_hi = (((8u * LO::kRowBytes) >> 4) & 0x3FFFu) | (1u << 14) |
                                 (ptx::swizzle_mode_for_row_bytes(LO::kRowBytes) << 29);
    constexpr uint32_t kStepUnits = (16u * LO::kRowBytes) >> 4;   // 16 keys further down the V tile
    const uint32_t v_lo = ((ptx::smem_u32(smem + LO::offV) >> 4) & 0x3FFFu) | (((uint32_t)LO::kBlk >> 4) << 16);
    const uint32_t t_o = tmem_base + COL_O + g * 64, t_p = tmem_base + COL_P + g * (BN / 2);
    uint32_t c_t = 0, c_tiles0 = 0;   // tiles of this stream so far; tiles of all earlier items
    bool ok = true;
    int k = 0;
    for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x, ++k) {
      const int slot = k & 1;
      ok = ptx::mbar_wait_inline(&bars->item_full[slot], (uint32_t)(k >> 1) & 1u, abort_flag, status_word, 36);
      if (!ok) break;
      const ItemSlot* sl = &slots[slot];
      if (sl->any_kept != 0) {
        const int n = sl->t_end - sl->t_begin;
        // O[g] is overwritten by the stream's first PV of an item: the previous item's merge (item k-1 of this CTA,
        // whatever its kind) must have read both accumulators
        if (k > 0 && g < n) ok = ptx::mbar_wait_inline(&bars->xbar_b, (uint32_t)(k - 1) & 1u, abort_flag, status_word, 38);
        for (int u = g; u < n && ok; u += 2, ++c_t) {
          const uint32_t tile = c_tiles0 + (uint32_t)u, vb = tile & 1u;
          ok = ptx::mbar_wait_inline(&bars->p_full[g], c_t & 1u, abort_flag, status_word, 7) &&
               ptx::mbar_wait_inline(&bars->v_full[vb], (tile >> 1) & 1u, abort_flag, status_word, 8);
          if (!ok) break;
          TRACE(27);
          ptx::tc_fence_after();
          const uint32_t vt_lo = v_lo + vb * ((uint32_t)LO::kBlk >> 4);
          if (u < 2) umma_ts_lohi<0>(t_o, t_p, vt_lo, desc_hi, idesc_pv);
          else umma_ts_lohi<1>(t_o, t_p, vt_lo, desc_hi, idesc_pv);
#pragma unroll
          for (int kk = 1; kk < BN / 16; ++kk)
            umma_ts_lohi<1>(t_o, t_p + kk * 8, vt_lo + kk * kStepUnits, desc_hi, idesc_pv);
          ptx::umma_commit(&bars->v_empty[vb]);
          ptx::umma_commit(&bars->o_ready[g]);
        }
        c_tiles0 += (uint32_t)n;
      }
      ptx::mbar_arrive(&bars->item_empty[slot]);
    }
  };

  if (warp < kSoftmaxWarps) {
    setmaxnreg_inc();
    // ----------------------------------------------------------------- softmax
    const int g = warp >> 2, q4 = warp & 3;     // stream, lane quarter
    const int r = q4 * 32 + lane;               // query row of the tile = TMEM lane
    const float cscale = p.scale * 1.4426950408889634f;
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    const uint32_t t_s = tmem_base + lane_base + COL_S + g * BN;
    const uint32_t t_p = tmem_base + lane_base + COL_P + g * (BN / 2);
    const uint32_t t_o = tmem_base + lane_base + COL_O + g * 64;
    const uint32_t t_o_other = tmem_base + lane_base + COL_O + (1 - g) * 64;
    const uint32_t ring_addr = ptx::smem_u32(smem + LO::offRing) + (uint32_t)(r * RING_PITCH_H * 2);
    // PT[m][n] with m = n - r + 128: element n of this row sits at pt_addr + n * (pitch + 1) halfs
    const uint32_t pt_addr = ptx::smem_u32(smem + LO::offPT + g * LO::kPTStage) + (uint32_t)((128 - r) * PT_PITCH_H * 2);
    float2* xchg_base = reinterpret_cast<float2*>(smem + LO::offXchg);
    uint32_t c_t = 0, c_o = 0;      // tiles of this stream / of the other stream so far
    uint32_t c_blk0 = 0;            // C2P blocks produced before this item
    uint32_t c_m = 0;               // items merged
    bool ok = true;

    int k = 0;
    for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x, ++k) {
      const int slot = k & 1;
      ok = ptx::mbar_wait_inline(&bars->item_full[slot], (uint32_t)(k >> 1) & 1u, abort_flag, status_word, 33);
      if (!ok) break;
      const ItemSlot* sl = &slots[slot];
      const int t_begin = sl->t_begin, n = sl->t_end - sl->t_begin;
      const bool any_kept = sl->any_kept != 0;
      const int bh = sl->bh, b = bh / H, h = bh - b * H;
      const int i0 = sl->i0;

      if (!any_kept) {
        // Every query row of this tile is padding: each attends uniformly to all L keys, so every output row is
        // the column mean of V.  No score, no softmax: one pass over V by the 256 softmax threads.
        float* part = reinterpret_cast<float*>(smem + LO::offMeanV);         // [groups][D] partial sums
        T* mean = reinterpret_cast<T*>(smem + LO::offMeanV + 1024);          // [D]
        constexpr int kGroups = 256 / D;
        const int tid = threadIdx.x, col = tid % D, grp = tid / D;
        const T* V = reinterpret_cast<const T*>(p.v) + (long long)bh * L * D;
        float sum = 0.0f;
        for (int row = grp; row < L; row += kGroups) sum += Elem<T>::to_f(V[(long long)row * D + col]);
        part[grp * D + col] = sum;
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bars->xbar_a);
        ok = ptx::mbar_wait_inline(&bars->xbar_a, c_m & 1u, abort_flag, status_word, 34);
        if (!ok) break;
        if (tid < D) {
          float total = 0.0f;
          for (int gidx = 0; gidx < kGroups; ++gidx) total += part[gidx * D + tid];
          mean[tid] = Elem<T>::from_f(total / (float)L);
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bars->xbar_b);
        ok = ptx::mbar_wait_inline(&bars->xbar_b, c_m & 1u, abort_flag, status_word, 35);
        if (!ok) break;
        ++c_m;
        const int rows = L - i0 < BM ? L - i0 : BM;
        constexpr int kVec = D / 8;  // 16-byte chunks per output row
        const uint4 mine = *reinterpret_cast<const uint4*>(mean + (tid % kVec) * 8);
        T* out = reinterpret_cast<T*>(p.out) + ((long long)b * L + i0) * ((long long)H * D) + (long long)h * D;
        for (int e = tid; e < rows * kVec; e += 256) {
          const int rr = e / kVec, v = e - rr * kVec;
          *reinterpret_cast<uint4*>(out + (long long)rr * H * D + v * 8) = mine;
        }
      } else {
        const int i = i0 + r;
        const bool row_ok = i < L;
        const bool q_keep = row_ok && ((sl->kbits[i >> 5] >> (i & 31)) & 1u) != 0u;
        float m_run = -INFINITY, l_run = 0.0f;

        for (int u = g; u < n && ok; u += 2) {
          const int t = t_begin + u, j0 = t * BN;
          // The stream's previous PV must be complete before its P operand is overwritten or O is rescaled.
          ok = ptx::mbar_wait_inline(&bars->o_ready[g], (c_t & 1u) ^ 1u, abort_flag, status_word, 22) &&
               ptx::mbar_wait_inline(&bars->s_full[g], c_t & 1u, abort_flag, status_word, 9);
          if (ok && has_c2p) ok = ptx::mbar_wait_inline(&bars->c2p_ready[g], c_t & 1u, abort_flag, status_word, 10);
          if (ok && has_p2c) ok = ptx::mbar_wait_inline(&bars->pt_ready[g], c_t & 1u, abort_flag, status_word, 21);
          if (!ok) break;
          TRACE(1);
          ptx::tc_fence_after();
          // ring column of (row r, key x of the tile): (64 * block index of the tile + 128 - r + x) mod 256
          const uint32_t cb = (64u * (c_blk0 + (uint32_t)u) + 128u - (uint32_t)r) & 255u;
          const uint32_t kb0 = sl->kbits[2 * t], kb1 = sl->kbits[2 * t + 1];
          const bool keys_all_kept = (kb0 & kb1) == 0xffffffffu;
          const int n_in = L - j0;

          // The tile is walked in four chunks of 16 keys by one rolled loop (a small loop body stays in the
          // instruction cache; a fully unrolled 64-key body does not): the two relative terms from shared memory,
          // mask, exp2 against the running reference maximum, P chunk to TMEM.
          // One TMEM round trip per tile (a tcgen05.ld -> wait::ld pair costs several hundred cycles, and wait::ld
          // drains every outstanding load, so per-chunk loads cannot be pipelined): the whole S row is fetched at
          // once - which also frees the S buffer for the MMA of the stream's next tile right away - and the loop
          // consumes the first 16 registers, then rotates the rest down.
          uint32_t raw[BN];
          {
            uint32_t (&lo)[32] = *reinterpret_cast<uint32_t (*)[32]>(&raw[0]);
            uint32_t (&hi)[32] = *reinterpret_cast<uint32_t (*)[32]>(&raw[32]);
            ptx::tmem_ld32(t_s, lo);
            ptx::tmem_ld32(t_s + 32, hi);
            ptx::tmem_wait_ld();
          }
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&bars->s_free[g]);
          TRACE(2);

          // Lazy reference maximum: m_run moves only when a chunk maximum exceeds it by more than 2^8 after scaling,
          // so exp2 arguments stay <= 8 (P <= 256, exact range of both 16-bit types) and O needs rescaling rarely.
          // On a move, everything accumulated against the old reference is rescaled: the row sum, O in TMEM (if the
          // stream already accumulated in this item) and the P chunks of this tile that are already written.
          float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
          for (int q = 0; q < 4; ++q) {
            float s[16];
#pragma unroll
            for (int x = 0; x < 16; ++x) s[x] = __uint_as_float(raw[x]);
#pragma unroll
            for (int x = 0; x < BN - 16; ++x) raw[x] = raw[x + 16];
            // per term: 16 loads issued before the 16 adds that use them (a warp issues in order; a load followed
            // at once by its consumer would expose the shared-memory latency once per element)
            if (has_c2p) {
              const uint32_t base = (cb + 16u * q) & 255u;   // a 16-key run stays inside columns [base, base+16) <= 271
              const uint32_t caddr = ring_addr + 2u * base;
              uint32_t cv[16];
#pragma unroll
              for (int x = 0; x < 16; ++x) cv[x] = lds_u16_r32(caddr + 2u * x);
#pragma unroll
              for (int x = 0; x < 16; ++x) s[x] = Pack2<T>::add(s[x], (uint16_t)cv[x]);
            }
            if (has_p2c) {
              const uint32_t paddr = pt_addr + (uint32_t)(q * 16 * (PT_PITCH_H + 1) * 2);
              uint32_t pv[16];
#pragma unroll
              for (int x = 0; x < 16; ++x) pv[x] = lds_u16_r32(paddr + (uint32_t)(x * (PT_PITCH_H + 1) * 2));
#pragma unroll
              for (int x = 0; x < 16; ++x) s[x] = Pack2<T>::add(s[x], (uint16_t)pv[x]);
            }
            // mask: keys >= L and padded keys -> -inf; a padded query row -> 0 on every in-range key
            if (!q_keep) {
#pragma unroll
              for (int x = 0; x < 16; ++x) s[x] = 16 * q + x < n_in ? 0.0f : -INFINITY;
            } else if (!keys_all_kept) {
              const uint32_t kbq = ((q < 2 ? kb0 : kb1) >> ((q & 1) * 16)) & 0xffffu;
#pragma unroll
              for (int x = 0; x < 16; ++x)
                if (!((kbq >> x) & 1u)) s[x] = -INFINITY;
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int x = 0; x < 16; ++x) mx[x & 3] = fmaxf(mx[x & 3], s[x]);
            const float cmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            const bool move = cmax > m_run + attn::kLazyMaxSlack / cscale;  // also true for the first finite maximum
            if (__any_sync(0xffffffffu, move)) {
              const float m_new = move ? cmax : m_run;
              const float m_use = m_new == -INFINITY ? 0.0f : m_new;
              const float corr = move ? ptx::ex2_approx((m_run - m_use) * cscale) : 1.0f;   // 0 when m_run = -inf
              m_run = m_new;
              l_run *= corr;
              if (u >= 2) {   // the stream already accumulated into O in this item
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 8) {   // rare: small rolled steps keep the register footprint low
                  uint32_t o[8];
                  ptx::tmem_ld8(t_o + c0, o);
                  ptx::tmem_wait_ld();
#pragma unroll
                  for (int x = 0; x < 8; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * corr);
                  ptx::tmem_st8(t_o + c0, o);
                }
              }
              if (q > 0) {    // P chunks 0..q-1 of this tile were formed against the old reference
                sum[0] = sum[1] = sum[2] = sum[3] = 0.0f;
                ptx::tmem_wait_st();
#pragma unroll 1
                for (int j = 0; j < q; ++j) {
                  uint32_t w[8];
                  ptx::tmem_ld8(t_p + 8 * j, w);
                  ptx::tmem_wait_ld();
#pragma unroll
                  for (int x = 0; x < 8; ++x) {
                    w[x] = Pack2<T>::scale2(w[x], corr);
                    sum[x & 3] += Pack2<T>::sum2(w[x]);
                  }
                  ptx::tmem_st8(t_p + 8 * j, w);
                }
              }
            }
            const float neg_m = -(m_run == -INFINITY ? 0.0f : m_run) * cscale;
            uint32_t packed[8];
            // staged by kind of instruction (arguments, exp2, packing, sums): a warp issues in order
#pragma unroll
            for (int x = 0; x < 16; ++x) s[x] = fmaf(s[x], cscale, neg_m);
#pragma unroll
            for (int x = 0; x < 16; ++x) s[x] = ptx::ex2_approx(s[x]);
#pragma unroll
            for (int x = 0; x < 16; x += 2) packed[x / 2] = Pack2<T>::pack(s[x], s[x + 1]);
            // The row sum is taken over P as rounded for the tensor core, so that the weights P/l the output is
            // built from sum to one exactly.  (The reference sums the unrounded values, kernel.py:316-333; with the
            // lazy reference maximum the largest P of a row is not the exactly representable 1.0, and an unrounded
            // sum would leave the rounding error of the dominant key uncompensated.)
#pragma unroll
            for (int x = 0; x < 8; ++x) sum[x & 3] += Pack2<T>::sum2(packed[x]);
            ptx::tmem_st8(t_p + 8 * q, packed);
          }
          l_run += (sum[0] + sum[1]) + (sum[2] + sum[3]);
          TRACE(4);
          ptx::tmem_wait_st();
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (has_c2p) ptx::mbar_arrive(&bars->ring_release[g]);
            if (has_p2c) ptx::mbar_arrive(&bars->pt_release[g]);
            ptx::mbar_arrive(&bars->p_full[g]);
          }
          ++c_t;
          TRACE(5);
        }
        if (!ok) break;

        TRACE(6);
        // ---- merge the two streams of the row and store.  Stream g writes output columns [g*D/2, (g+1)*D/2).
        const int my_tiles = (n - g + 1) / 2, other_tiles = n - my_tiles;
        c_o += (uint32_t)other_tiles;
        if (my_tiles > 0) ok = ptx::mbar_wait_inline(&bars->o_ready[g], (c_t & 1u) ^ 1u, abort_flag, status_word, 23);
        if (ok && other_tiles > 0)
          ok = ptx::mbar_wait_inline(&bars->o_ready[1 - g], (c_o & 1u) ^ 1u, abort_flag, status_word, 24);
        if (!ok) break;
        float2* xchg = xchg_base + (c_m & 1u) * (2 * BM);   // slots alternate: a stream may be one item ahead
        xchg[g * BM + r] = make_float2(m_run, l_run);
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bars->xbar_a);
        ok = ptx::mbar_wait_inline(&bars->xbar_a, c_m & 1u, abort_flag, status_word, 34);
        if (!ok) break;
        ptx::tc_fence_after();
        const float2 other = xchg[(1 - g) * BM + r];
        const float m_all = fmaxf(m_run, other.x);
        const float m_fin = m_all == -INFINITY ? 0.0f : m_all;
        const float a_me = my_tiles > 0 && m_run != -INFINITY ? ptx::ex2_approx((m_run - m_fin) * cscale) : 0.0f;
        const float a_ot = other_tiles > 0 && other.x != -INFINITY ? ptx::ex2_approx((other.x - m_fin) * cscale) : 0.0f;
        const float inv = 1.0f / (l_run * a_me + other.y * a_ot);
        constexpr int HW = D / 2;   // output columns per thread
        uint32_t o_me[HW], o_ot[HW];
        if (my_tiles > 0) attn::tmem_ld_n(t_o + g * HW, o_me);
        if (other_tiles > 0) attn::tmem_ld_n(t_o_other + g * HW, o_ot);
        ptx::tmem_wait_ld();
        // Both accumulators are in registers: the PV issuer may start the next item's accumulation (it waits for the
        // eight arrivals); the streams themselves go on without waiting for each other's stores.
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bars->xbar_b);
        float res[HW];
#pragma unroll
        for (int x = 0; x < HW; ++x) {
          float v = my_tiles > 0 ? __uint_as_float(o_me[x]) * a_me : 0.0f;
          if (other_tiles > 0) v = fmaf(__uint_as_float(o_ot[x]), a_ot, v);
          res[x] = v * inv;
        }
        if (row_ok) {
          T* out = reinterpret_cast<T*>(p.out) + ((long long)b * L + i) * ((long long)H * D) + (long long)h * D + g * HW;
#pragma unroll
          for (int v = 0; v < HW / 8; ++v) {
            uint4 pk;
            pk.x = Pack2<T>::pack(res[v * 8 + 0], res[v * 8 + 1]);
            pk.y = Pack2<T>::pack(res[v * 8 + 2], res[v * 8 + 3]);
            pk.z = Pack2<T>::pack(res[v * 8 + 4], res[v * 8 + 5]);
            pk.w = Pack2<T>::pack(res[v * 8 + 6], res[v * 8 + 7]);
            *reinterpret_cast<uint4*>(out + v * 8) = pk;
          }
        }
        ++c_m;
        TRACE(7);
        if (has_c2p) c_blk0 += (uint32_t)n + 2u;
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bars->item_empty[slot]);
    }
  } else if (warp < kConvHiWarp0) {
    setmaxnreg_dec();
    converter_role();
  } else {
    setmaxnreg_dec();
    if (warp < kTmaWarp) {
      pv_role();
    } else if (warp == kTmaWarp) {
    // ------------------------------------------------- mask analysis + TMA producer
    uint32_t c_q = 0, c_kv = 0, c_pk = 0, c_fq = 0;   // running counts: Q loads, K/V tiles, rel_key / rel_query blocks
    bool ok = true;
    int k = 0;
    for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x, ++k) {
      const int slot = k & 1;
      const int qt = it / n_bh, bh = it - qt * n_bh, b = bh / H, h = bh - b * H;
      const int i0 = qt * BM;
      ItemSlot* sl = &slots[slot];
      TRACE(40);
      ok = ptx::mbar_wait_inline(&bars->item_empty[slot], ((uint32_t)(k >> 1) & 1u) ^ 1u, abort_flag, status_word, 30);
      if (!ok) break;
      const uint32_t kb_mine = kept_bits_word(p, b, lane);
      const TileRange range = tile_range(kb_mine, i0, L, lane);
      const int t_begin = range.t_begin, t_end = range.t_end;
      const bool any_kept = range.any_kept;
      sl->kbits[lane] = kb_mine;
      if (lane == 0) {
        sl->t_begin = t_begin;
        sl->t_end = t_end;
        sl->any_kept = any_kept ? 1 : 0;
        sl->bh = bh;
        sl->i0 = i0;
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bars->item_full[slot]);
      TRACE(41);
      if (!any_kept) continue;

      if (lane == 0) {
        const int n = t_end - t_begin;
        const int e0 = t_begin * BN - i0 - 2 * BN + (L - 1);   // table row of block 0 (x0 = j_begin - i0 - 128)
        auto load_pk = [&](int c) -> bool {
          const int buf = c_pk & 1;
          if (!ptx::mbar_wait_inline(&bars->pk_empty[buf], ((c_pk >> 1) & 1u) ^ 1u, abort_flag, status_word, 11)) return false;
          ptx::mbar_arrive_expect_tx(&bars->pk_full[buf], (uint32_t)LO::kBlk);
          ptx::tma_load_3d(smem + LO::offPK + buf * LO::kBlk, &tmap_fk, &bars->pk_full[buf], 0, e0 + c * BN, h);
          ++c_pk;
          return true;
        };
        auto load_fq = [&](int c) -> bool {
          const int pos = c_fq & 3;
          if (!ptx::mbar_wait_inline(&bars->fq_empty[pos], ((c_fq >> 2) & 1u) ^ 1u, abort_flag, status_word, 12)) return false;
          ptx::mbar_arrive_expect_tx(&bars->fq_full[pos], (uint32_t)LO::kBlk);
          ptx::tma_load_3d(smem + LO::offFQ + pos * LO::kBlk, &tmap_fq, &bars->fq_full[pos], 0, e0 + c * BN, h);
          ++c_fq;
          return true;
        };
        auto load_k = [&](int u) -> bool {
          const int buf = (c_kv + u) & 1;
          if (!ptx::mbar_wait_inline(&bars->k_empty[buf], (((c_kv + u) >> 1) & 1u) ^ 1u, abort_flag, status_word, 1)) return false;
          ptx::mbar_arrive_expect_tx(&bars->k_full[buf], (uint32_t)LO::kBlk);
          ptx::tma_load_3d(smem + LO::offK + buf * LO::kBlk, &tmap_k, &bars->k_full[buf], 0, (t_begin + u) * BN, bh);
          return true;
        };
        auto load_v = [&](int u) -> bool {
          const int buf = (c_kv + u) & 1;
          if (!ptx::mbar_wait_inline(&bars->v_empty[buf], (((c_kv + u) >> 1) & 1u) ^ 1u, abort_flag, status_word, 2)) return false;
          ptx::mbar_arrive_expect_tx(&bars->v_full[buf], (uint32_t)LO::kBlk);
          ptx::tma_load_3d(smem + LO::offV + buf * LO::kBlk, &tmap_v, &bars->v_full[buf], 0, (t_begin + u) * BN, bh);
          return true;
        };
        ok = ptx::mbar_wait_inline(&bars->q_empty, (c_q & 1u) ^ 1u, abort_flag, status_word, 3);
        if (ok) {
          ptx::mbar_arrive_expect_tx(&bars->q_full, (uint32_t)LO::kQ);
          ptx::tma_load_3d(smem + LO::offQ, &tmap_q, &bars->q_full, 0, i0, bh);
          ++c_q;
        }
        // Issue order: what the MMA front of a tile needs (rel_key block, K, rel_query block) first; the V tile,
        // whose stage is released only by the PV two tiles back, trails by one tile so that waiting for it never
        // holds back the next tile's front loads.
        if (ok && has_c2p) ok = load_pk(0) && load_pk(1);
        if (ok) ok = load_k(0);
        if (ok && has_p2c) ok = load_fq(0) && load_fq(1) && load_fq(2);
        if (ok && has_c2p) ok = load_pk(2);
        for (int u = 1; u < n && ok; ++u) {
          if (has_c2p) ok = load_pk(u + 2);
          if (ok) ok = load_k(u);
          if (ok && has_p2c) ok = load_fq(u + 2);
          if (ok) ok = load_v(u - 1);
        }
        if (ok) ok = load_v(n - 1);
        c_kv += (uint32_t)n;
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    }
    } else {
    // -------------------------------------------------------------- MMA issuer
    // One thread issues the "front" of every tile (new C2P block(s), PT, S), so its instruction count per tile bounds
    // the tile rate: descriptors are kept as precomputed 32-bit halves (only the start-address field moves).
    if (lane == 0) {
      constexpr int is_bf16 = __is_same(T, __nv_bfloat16) ? 1 : 0;
      constexpr uint32_t idesc_64 = ptx::make_idesc_f16(is_bf16, BM, BN, 0, 0);  // 128 x 64, both K-major
      constexpr uint32_t mode = ptx::swizzle_mode_for_row_bytes(LO::kRowBytes);
      constexpr uint32_t sbo = 8 * LO::kRowBytes;
      constexpr int kSteps = LO::kRowBytes / 32;  // K=16 steps over d
      // shared-memory descriptor = {lo, hi}: lo = start>>4 | (leading offset>>4) << 16, hi = stride offset>>4 |
      // version 1 << 14 | swizzle << 29; every operand here shares hi
      constexpr uint32_t desc_hi = ((sbo >> 4) & 0x3FFFu) | (1u << 14) | (mode << 29);
      constexpr uint32_t kBlkUnits = (uint32_t)LO::kBlk >> 4;
      auto desc_lo = [](uint32_t addr, uint32_t lbo) { return ((addr >> 4) & 0x3FFFu) | ((lbo >> 4) << 16); };
      const uint32_t q_lo = desc_lo(ptx::smem_u32(smem + LO::offQ), 16);
      const uint32_t pk_lo = desc_lo(ptx::smem_u32(smem + LO::offPK), 16);
      const uint32_t fq_lo = desc_lo(ptx::smem_u32(smem + LO::offFQ), 16);
      const uint32_t k_lo = desc_lo(ptx::smem_u32(smem + LO::offK), 16);
      uint32_t c_q = 0, c_front = 0, c_pk = 0, c_fq = 0, c_pt = 0;
      uint32_t c_s0 = 0, c_s1 = 0;   // per stream: S tiles issued
      bool ok = true;

      // D[128 x 64] = A[128 x d] * B[64 x d]^T, both operands K-major tiles in shared memory
      auto mma_128x64 = [&](uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo) {
#pragma unroll
        for (int kk = 0; kk < kSteps; ++kk) {
          if (kk == 0) umma_ss_lohi<0>(d_tmem, a_lo, b_lo, desc_hi, idesc_64);
          else umma_ss_lohi<1>(d_tmem, a_lo + 2u * kk, b_lo + 2u * kk, desc_hi, idesc_64);
        }
      };

      // everything tile u needs before its softmax: new C2P block(s), PT, S
      auto front = [&](int u, int n) -> bool {
        const int g = u & 1;
        if (u == 0) {
          if (!ptx::mbar_wait_inline(&bars->q_full, c_q & 1u, abort_flag, status_word, 4)) return false;
          ++c_q;
        }
        if (has_c2p) {
          const int jobs = u == 0 ? 3 : 1;
          for (int x = 0; x < jobs; ++x, ++c_pk) {
            const uint32_t buf = c_pk & 1u;
            TRACE(20);
            if (!ptx::mbar_wait_inline(&bars->pk_full[buf], (c_pk >> 1) & 1u, abort_flag, status_word, 13)) return false;
            TRACE(21);
            if (!ptx::mbar_wait_inline(&bars->cnew_free, (c_pk & 1u) ^ 1u, abort_flag, status_word, 14)) return false;
            TRACE(22);
            ptx::tc_fence_after();
            mma_128x64(tmem_base + COL_CNEW, q_lo, pk_lo + buf * kBlkUnits);
            ptx::umma_commit(&bars->pk_empty[buf]);
            ptx::umma_commit(&bars->cnew_full);
          }
        }
        const uint32_t kb = c_front & 1u;
        if (!ptx::mbar_wait_inline(&bars->k_full[kb], (c_front >> 1) & 1u, abort_flag, status_word, 5)) return false;
        TRACE(23);
        const uint32_t kt_lo = k_lo + kb * kBlkUnits;
        if (has_p2c) {
          // window of tile u = table blocks u, u+1, u+2 of the item, at ring positions p, p+1, p+2 (mod 4)
          const int first = u == 0 ? 0 : 2;
          for (int x = first; x < 3; ++x) {
            const uint32_t blk = c_fq + (uint32_t)x;
            if (!ptx::mbar_wait_inline(&bars->fq_full[blk & 3], (blk >> 2) & 1u, abort_flag, status_word, 15)) return false;
          }
          TRACE(24);
          if (!ptx::mbar_wait_inline(&bars->pt_free, (c_pt & 1u) ^ 1u, abort_flag, status_word, 16)) return false;
          TRACE(25);
          ptx::tc_fence_after();
          const uint32_t pp = c_fq & 3u;
          // 128 contiguous operand rows, then the remaining block: positions (p, p+1 | p+2), except p = 3 where
          // the contiguous pair is blocks u+1, u+2 at positions 0, 1 and block u sits alone at position 3
          const uint32_t a1 = pp == 3u ? 0u : pp;
          const uint32_t a2 = pp == 3u ? 3u : (pp + 2u) & 3u;
          mma_128x64(tmem_base + COL_PT, fq_lo + a1 * kBlkUnits, kt_lo);
          mma_128x64(tmem_base + COL_PT + BN, fq_lo + a2 * kBlkUnits, kt_lo);
          ptx::umma_commit(&bars->fq_empty[pp]);   // block u is not part of any later window
          ++c_fq;
          if (u == n - 1) {                         // the item's last two blocks
            ptx::umma_commit(&bars->fq_empty[c_fq & 3]);
            ++c_fq;
            ptx::umma_commit(&bars->fq_empty[c_fq & 3]);
            ++c_fq;
          }
          ptx::umma_commit(&bars->pt_full);
          ++c_pt;
        }
        TRACE(29);
        const uint32_t c_s = g ? c_s1 : c_s0;
        if (!ptx::mbar_wait_inline(&bars->s_free[g], (c_s & 1u) ^ 1u, abort_flag, status_word, 6)) return false;
        TRACE(26);
        ptx::tc_fence_after();
        mma_128x64(tmem_base + COL_S + g * BN, q_lo, kt_lo);
        ptx::umma_commit(&bars->s_full[g]);
        ptx::umma_commit(&bars->k_empty[kb]);
        if (g) ++c_s1; else ++c_s0;
        ++c_front;
        if (u == n - 1) ptx::umma_commit(&bars->q_empty);
        return true;
      };

      // The fronts run ahead of the softmax streams as far as the buffers allow, also into the next item; the PV of
      // a tile is issued by the softmax stream that produced its P.
      int k = 0;
      for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x, ++k) {
        const int slot = k & 1;
        ok = ptx::mbar_wait_inline(&bars->item_full[slot], (uint32_t)(k >> 1) & 1u, abort_flag, status_word, 31);
        if (!ok) break;
        const ItemSlot* sl = &slots[slot];
        if (sl->any_kept != 0) {
          const int n = sl->t_end - sl->t_begin;
          for (int u = 0; u < n && ok; ++u) ok = front(u, n);
        }
        ptx::mbar_arrive(&bars->item_empty[slot]);
      }
    }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) ptx::tmem_dealloc(tmem_base, kTmemCols);
}

// rel[h, e, :] = pos[h, lut[2L-2-e], :]; one thread per 16-byte chunk.
__global__ void expand_rel_tables_kernel(const uint4* __restrict__ pos, const int32_t* __restrict__ lut,
                                         uint4* __restrict__ rel, int heads, int n_active, int n_rows, int chunks) {
  const long long total = (long long)heads * n_rows * chunks;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % chunks);
    const long long he = idx / chunks;
    const int e = (int)(he % n_rows), h = (int)(he / n_rows);
    int slot = lut[n_rows - 1 - e];
    slot = slot < 0 ? 0 : (slot >= n_active ? n_active - 1 : slot);
    rel[idx] = pos[((long long)h * n_active + slot) * chunks + c];
  }
}

template <typename T, int D>
int launch_rel_typed(const DflAttnRelParams& p, cudaStream_t stream) {
  using LO = RLayout<D>;
  const int L = p.seq_len, BH = p.batch * p.heads, R = 2 * L - 1;
  const uint64_t row = (uint64_t)D * sizeof(T), seq = (uint64_t)L * row, table = (uint64_t)R * row;
  CUtensorMap tq, tk, tv, tfk, tfq;
  int rc = encode_tensor_map_3d(&tq, p.q, D, L, BH, row, seq, D, BM, LO::kRowBytes);
  if (rc == DFL_OK) rc = encode_tensor_map_3d(&tk, p.k, D, L, BH, row, seq, D, BN, LO::kRowBytes);
  if (rc == DFL_OK) rc = encode_tensor_map_3d(&tv, p.v, D, L, BH, row, seq, D, BN, LO::kRowBytes);
  // a disabled term reuses the other table's map; it is never dereferenced
  const void* fk = p.rel_key ? p.rel_key : p.rel_query;
  const void* fq = p.rel_query ? p.rel_query : p.rel_key;
  if (rc == DFL_OK) rc = encode_tensor_map_3d(&tfk, fk, D, R, p.heads, row, table, D, BN, LO::kRowBytes);
  if (rc == DFL_OK) rc = encode_tensor_map_3d(&tfq, fq, D, R, p.heads, row, table, D, BN, LO::kRowBytes);
  if (rc != DFL_OK) return rc;

  auto kernel = attention_rel_kernel<T, D>;
  // one-time configuration per device (the opt-in to large dynamic shared memory is a per-device attribute)
  constexpr int kMaxDevices = 64;
  static int sm_counts[kMaxDevices] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fail(DFL_ERR_LAUNCH, "current device: %s", cudaGetErrorString(e));
  if (sm_counts[dev] == 0) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, LO::total);
    if (e != cudaSuccess) return fail(DFL_ERR_LAUNCH, "attention_rel smem opt-in: %s", cudaGetErrorString(e));
    int count = 0;
    e = cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || count < 1) return fail(DFL_ERR_LAUNCH, "SM count: %s", cudaGetErrorString(e));
    sm_counts[dev] = count;
  }
  const int sm_count = sm_counts[dev];
  int* status_word = p.status;
  if (!status_word) {
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&status_word), g_attn_rel_status);
    if (e != cudaSuccess) return fail(DFL_ERR_LAUNCH, "status word: %s", cudaGetErrorString(e));
  }
  const long long n_items = (long long)BH * ((L + BM - 1) / BM);
  if (n_items > 0x7fffffffLL) return fail(DFL_ERR_TOO_LARGE, "too many (batch, head, query tile) items");
  const int grid = n_items < sm_count ? (int)n_items : sm_count;
  kernel<<<grid, kThreads, LO::total, stream>>>(tq, tk, tv, tfk, tfq, p, status_word, (int)n_items);
  return check_launch("attention_rel_kernel");
}

}  // namespace

bool attention_rel_supported(const DflAttnRelParams& p) {
  return p.dtype != DFL_F32 && (p.head_dim == 32 || p.head_dim == 64) && (p.rel_key || p.rel_query) &&
         p.seq_len >= 1 && p.seq_len <= kMaxSeqLen;
}

int launch_attention_rel(const DflAttnRelParams& p, cudaStream_t stream) {
  if (!attention_rel_supported(p)) return fail(DFL_ERR_UNSUPPORTED, "configuration not covered by the relative-table kernel");
  if (p.dtype == DFL_F16)
    return p.head_dim == 64 ? launch_rel_typed<__half, 64>(p, stream) : launch_rel_typed<__half, 32>(p, stream);
  return p.head_dim == 64 ? launch_rel_typed<__nv_bfloat16, 64>(p, stream)
                          : launch_rel_typed<__nv_bfloat16, 32>(p, stream);
}

int launch_expand_rel_tables(const void* pos, const int32_t* lut, void* rel, int heads, int n_active, int seq_len,
                             int head_dim, int dtype, cudaStream_t stream) {
  const int chunks = head_dim * (int)dtype_size(dtype) / 16;
  const int n_rows = 2 * seq_len - 1;
  const long long total = (long long)heads * n_rows * chunks;
  const int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 4096) blocks = 4096;
  expand_rel_tables_kernel<<<(int)blocks, threads, 0, stream>>>(reinterpret_cast<const uint4*>(pos), lut,
                                                                reinterpret_cast<uint4*>(rel), heads, n_active, n_rows,
                                                                chunks);
  return check_launch("expand_rel_tables_kernel");
}

}  // namespace dfl

#ifdef DFL_TRACE
extern "C" int dfl_debug_read_trace_rel(long long* host_buf, int clear) {
  cudaDeviceSynchronize();
  cudaError_t e = cudaMemcpyFromSymbol(host_buf, dfl::g_trace, sizeof(long long) * 16 * 512);
  if (clear) {
    static long long zeros[16 * 512] = {0};
    cudaMemcpyToSymbol(dfl::g_trace, zeros, sizeof(zeros));
  }
  return (int)e;
}
#endif
