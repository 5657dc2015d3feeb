// tcgen05 fused disentangled attention over position tables laid out by relative distance.
//
// Same result as dfl_pos_scores + dfl_attention_fwd (reference: the two torch.matmul calls at
// src/disentangled_flash/kernel.py:574-585 followed by the Triton kernel kernel.py:137-345).  The tables
// rel_key / rel_query [H, 2L-1, d] hold, in row e, the position projection every (query i, key j) pair with
// x = j - i = e - (L-1) uses, so the two relative terms of a (128 query x 128 key) tile are
//   C2P[i, j] = q_i . rel_key[x]      P2C[i, j] = k_j . rel_query[x]
// with x running over one contiguous window of 255 table rows.  Both are produced by tcgen05.mma from 128-row
// table blocks (L2 resident), rounded to the input type exactly like the separate score GEMMs round their output,
// and parked in shared memory, where the softmax threads pick them up along diagonals.
//   C2P depends on the query rows only: D[r, m] = q_r . rel_key[x_lo + m] with TMEM lanes = query rows.  Per query
//       row a shared-memory ring of two 128-column blocks is kept (the window of a key tile is two blocks; the next
//       key tile needs one new block, written in place of the block that left the window).
//   P2C is new for every key tile: D[n, m] = k_n . rel_query[x_lo + m] with TMEM lanes = keys n, computed in two
//       halves of 128 table rows through one 128-column accumulator.  Converter warps round each key's row and
//       store the 136-column span the 128 queries of the tile can reach; a softmax thread then reads, for key n,
//       element (n & 7) + 128 - r of row n: the 32 lanes of a warp read 32 consecutive elements.
//
// Persistent: one CTA per SM walks (batch, head, 128-query tile) items in 128-key tiles; every role keeps running
// counters so that the barrier phases carry over from item to item and the loader / MMA issuer run ahead.
//   warps 0-7   softmax: two threads per query row (warps w and w+4 own the same TMEM lanes; each takes 64 of the
//               128 keys of a tile, 32 of the 64 packed P columns and half of the output columns).  Two passes over
//               the keys in rolled loops of 32: scores + relative terms + mask + maximum, written back to the S
//               columns; then exp2, rounding, row sum and the P store.
//   warps 8-11  converters for the C2P block and P2C accumulators (TMEM -> 16-bit -> shared memory)
//   warp 12     issuer of every MMA (C2P block, S, P2C halves, PV) and TMEM owner
//   warp 13     per-item mask analysis (kept-key bits, skipped key tiles), one item ahead, and TMA producer
// The first MMAs of an item (first C2P block, S and P2C of its first key tile) are issued while the softmax threads
// still work on the last key tile of the previous item; the second C2P block of an item goes through the P and O
// columns, which are idle between the read-out of one item and the first PV of the next.
//   warps 14-15 idle (they complete the fourth warpgroup, whose registers go to the softmax warps)
#include <type_traits>

#include "attention_tc_common.cuh"

namespace dfl {

__device__ int g_attn_rel_status = 0;

namespace {

using attn::Pack2;

constexpr int BM = 128;              // query rows per item (= TMEM lanes)
constexpr int BK = 128;              // keys per tile
constexpr int kSoftmaxWarps = 8;
constexpr int kMmaWarp = 12;
constexpr int kTmaWarp = 13;
constexpr int kThreads = 512;
constexpr int kSoftmaxRegs = 152;    // 256 x 152 + 128 x 120 + 128 x 88 = 65536 registers
constexpr int kConvRegs = 120;
constexpr int kMiscRegs = 88;
// The kernel is launched with 65536 / kThreads = 128 registers per thread.  `setmaxnreg.inc` waits until the pool
// holds what it asks for, so the three budgets must not ask for more than the SM has (a wait that nothing could
// bound); `setmaxnreg.dec` with a value above the launch allocation is an illegal instruction.
constexpr int kLaunchRegs = 65536 / kThreads;
static_assert(8 * 32 * kSoftmaxRegs + 4 * 32 * kConvRegs + 4 * 32 * kMiscRegs <= kThreads * kLaunchRegs,
              "register budgets of the three warpgroup kinds exceed what the launch allocates");
static_assert(kSoftmaxRegs >= kLaunchRegs && kConvRegs <= kLaunchRegs && kMiscRegs <= kLaunchRegs &&
                  kSoftmaxRegs % 8 == 0 && kConvRegs % 8 == 0 && kMiscRegs % 8 == 0,
              "setmaxnreg.inc raises and setmaxnreg.dec lowers the launch allocation, in multiples of 8");
constexpr int kConsumerWarps = 13;   // softmax, converters, MMA issuer: every warp that reads an item slot

constexpr int kItemSlots = 3;        // the loader analyses one item ahead of the one whose tiles it loads
constexpr int kMaxSeqLen = 2048;
constexpr int kMaskWords = kMaxSeqLen / 32;   // kept-key bits per item

// C2P ring: per query row two 128-column blocks and the first 16 columns once more (a 16-key run never wraps).
// 580 bytes = 145 words per row: the diagonal 16-bit reads of a warp and its 32-bit stores are conflict free.
constexpr int RING_COLS = 256;
constexpr int RING_MIRROR = 16;
constexpr int RING_PITCH = 580;
// P2C staging: per key 17 chunks of 8 columns (the chunk-aligned span of table rows its 128 queries reach).
// 272 bytes = 68 words per row: eight consecutive rows cover all 32 banks with their 16-byte stores.
constexpr int STG_CHUNKS = 17;
constexpr int STG_PITCH = STG_CHUNKS * 16;

// TMEM columns (all 512; one CTA per SM)
constexpr int COL_S = 0;      // 128  S = Q K^T of the current tile (fp32)
constexpr int COL_P = 128;    // 64   P of the current tile (16-bit pairs), A operand of the PV MMA
constexpr int COL_O = 192;    // 64   O accumulator (first D columns used)
constexpr int COL_XC = 256;   // 128  one new C2P block for the 128 query rows
constexpr int COL_XP = 384;   // 128  one half (128 table rows) of the P2C accumulator of a key tile
constexpr int kTmemCols = 512;

template <int D>
struct RLayout {
  static_assert(D == 32 || D == 64, "head dims 32 and 64");
  static constexpr int kRowBytes = D * 2;
  static constexpr int kTile = 128 * kRowBytes;        // Q tile, K tile, V tile, one 128-row table block
  static constexpr int kVStages = D == 64 ? 1 : 2;     // d = 64 fills shared memory: V and rel_key blocks are
  static constexpr int kRkStages = D == 64 ? 1 : 2;    // reloaded within the tile time after their single use
  static constexpr int offQ = 0;
  static constexpr int offK = offQ + kTile;                 // 2 stages
  static constexpr int offV = offK + 2 * kTile;
  static constexpr int offRK = offV + kVStages * kTile;
  static constexpr int offRQ = offRK + kRkStages * kTile;   // 2 stages
  static constexpr int offRing = offRQ + 2 * kTile;
  static constexpr int offStg = offRing + BM * RING_PITCH;
  static constexpr int offBar = offStg + BK * STG_PITCH;
  static constexpr int kBarBytes = 512;
  // exchange area: row maxima [2 parities][2 halves][BM], row sums [2 halves][BM], then the mean-of-V scratch
  // ([256 / D groups][D] partial sums, [D] column mean)
  static constexpr int offXmax = offBar + kBarBytes;
  static constexpr int offXsum = offXmax + 2 * 2 * BM * 4;
  static constexpr int offMeanV = offXsum + 2 * BM * 4;
  static constexpr int offItem = offMeanV + 1024 + 256;
  static constexpr int kItemBytes = 288;
  static constexpr int total = offItem + kItemSlots * kItemBytes + 1024;   // + alignment slack
  static_assert(offStg % 16 == 0 && offBar % 16 == 0 && offItem % 16 == 0, "alignment");
  static_assert(total <= 232448, "shared memory budget");
};

// What the loader warp publishes per item.
struct ItemSlot {
  int t_begin, t_end;   // key tiles [t_begin, t_end) are processed
  int any_kept;         // 0: every query row of the tile is padding -> mean-of-V path, no pipeline work
  int bh, i0;           // batch*heads + head, first query row
  uint32_t kbits[kMaskWords];   // kept-key bits of the batch row, word w = keys [32w, 32w+32)
};
static_assert(sizeof(ItemSlot) <= 288, "item slot too large");

struct RBarriers {
  uint64_t q_full, q_empty;
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t rk_full[2], rk_empty[2], rq_full[2], rq_empty[2];
  uint64_t s_full, s_free;          // S accumulator: MMA -> softmax, softmax (8 warps) -> MMA
  uint64_t xc_full, xc_free;        // C2P block accumulator: MMA -> converters (4 warps) -> MMA
  uint64_t b1_full;                 // second C2P block of an item, in the P and O columns
  uint64_t xp_full, xp_free;        // P2C half accumulator: MMA -> converters (4 warps) -> MMA
  uint64_t pt_ready, pt_release;    // P2C staging tile: converters -> softmax -> converters
  uint64_t p_full, o_ready, o_free; // P stored (8 warps); PV complete; output accumulator read out (8 warps)
  uint64_t c2p_ready, ring_release; // C2P ring blocks of a tile: converters -> softmax -> converters
  uint64_t pair2[4];                // the two warps of a lane quarter: row maximum (row sum) posted
  uint64_t item_full[kItemSlots], item_empty[kItemSlots];
  uint64_t xbar;                    // the eight softmax warps (mean-of-V path)
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(RBarriers) <= 512, "barrier block too large");

template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
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
__device__ __forceinline__ void umma_ts_lohi(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 16-bit shared-memory load, zero-extended into a 32-bit register (32-bit destinations keep every value in its
// own register; the address arithmetic of unrolled callers folds into the instruction's immediate offset).
__device__ __forceinline__ uint32_t lds_u16_r32(uint32_t saddr) {
  uint32_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(saddr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t saddr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(saddr) : "memory");
  return v;
}
// low 32 bits of {hi, lo} >> amount (amount 0 or 16: one element of a pair of packed 16-bit values)
__device__ __forceinline__ uint32_t funnel_r(uint32_t lo, uint32_t hi, uint32_t amount) {
  uint32_t v;
  asm("shf.r.wrap.b32 %0, %1, %2, %3;" : "=r"(v) : "r"(lo), "r"(hi), "r"(amount));
  return v;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float m;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(m) : "f"(a), "f"(b), "f"(c));
  return m;
}
__device__ __forceinline__ void sts_u32(uint32_t saddr, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(saddr), "r"(v) : "memory");
}
__device__ __forceinline__ void sts_v4(uint32_t saddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// 32 consecutive fp32 TMEM columns of this thread's lane into arr[off .. off+31] (a register array indexed by
// compile-time constants; no address of the array is taken, so it stays in registers across loop iterations).
#define DFL_TMEM_LD32_F(taddr, arr, off)                                                                            \
  asm volatile(                                                                                                     \
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                                     \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                                     \
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"                     \
      : "=f"(arr[off + 0]), "=f"(arr[off + 1]), "=f"(arr[off + 2]), "=f"(arr[off + 3]), "=f"(arr[off + 4]),          \
        "=f"(arr[off + 5]), "=f"(arr[off + 6]), "=f"(arr[off + 7]), "=f"(arr[off + 8]), "=f"(arr[off + 9]),          \
        "=f"(arr[off + 10]), "=f"(arr[off + 11]), "=f"(arr[off + 12]), "=f"(arr[off + 13]), "=f"(arr[off + 14]),     \
        "=f"(arr[off + 15]), "=f"(arr[off + 16]), "=f"(arr[off + 17]), "=f"(arr[off + 18]), "=f"(arr[off + 19]),     \
        "=f"(arr[off + 20]), "=f"(arr[off + 21]), "=f"(arr[off + 22]), "=f"(arr[off + 23]), "=f"(arr[off + 24]),     \
        "=f"(arr[off + 25]), "=f"(arr[off + 26]), "=f"(arr[off + 27]), "=f"(arr[off + 28]), "=f"(arr[off + 29]),     \
        "=f"(arr[off + 30]), "=f"(arr[off + 31])                                                                     \
      : "r"(taddr)                                                                                                  \
      : "memory")

#define DFL_TMEM_ST32_F(taddr, arr, off)                                                                            \
  asm volatile(                                                                                                     \
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "                                                               \
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "                                    \
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"                            \
      ::"r"(taddr), "f"(arr[off + 0]), "f"(arr[off + 1]), "f"(arr[off + 2]), "f"(arr[off + 3]), "f"(arr[off + 4]),   \
        "f"(arr[off + 5]), "f"(arr[off + 6]), "f"(arr[off + 7]), "f"(arr[off + 8]), "f"(arr[off + 9]),               \
        "f"(arr[off + 10]), "f"(arr[off + 11]), "f"(arr[off + 12]), "f"(arr[off + 13]), "f"(arr[off + 14]),          \
        "f"(arr[off + 15]), "f"(arr[off + 16]), "f"(arr[off + 17]), "f"(arr[off + 18]), "f"(arr[off + 19]),          \
        "f"(arr[off + 20]), "f"(arr[off + 21]), "f"(arr[off + 22]), "f"(arr[off + 23]), "f"(arr[off + 24]),          \
        "f"(arr[off + 25]), "f"(arr[off + 26]), "f"(arr[off + 27]), "f"(arr[off + 28]), "f"(arr[off + 29]),          \
        "f"(arr[off + 30]), "f"(arr[off + 31])                                                                       \
      : "memory")

// s0 += lo half of w, s1 += hi half of w (w = two packed values of type T), in fp32.
template <typename T>
__device__ __forceinline__ void add_pair(float& s0, float& s1, uint32_t w);
template <>
__device__ __forceinline__ void add_pair<__half>(float& s0, float& s1, uint32_t w) {
  asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tadd.rn.f32.f16 %0, lo, %0;\n\tadd.rn.f32.f16 %1, hi, %1;\n\t}"
      : "+f"(s0), "+f"(s1)
      : "r"(w));
}
template <>
__device__ __forceinline__ void add_pair<__nv_bfloat16>(float& s0, float& s1, uint32_t w) {
  asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tadd.rn.f32.bf16 %0, lo, %0;\n\tadd.rn.f32.bf16 %1, hi, %1;\n\t}"
      : "+f"(s0), "+f"(s1)
      : "r"(w));
}

// Kept-key bits of batch row b: word w (keys [32w, 32w+32)) built from its 32 mask elements.
__device__ __forceinline__ uint32_t kept_bits_word(const DflAttnRelParams& p, int b, int w) {
  const int L = p.seq_len;
  uint32_t kb = 0;
  const int jw = 32 * w;
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
// Warp-collective: lane l holds the kept-key words l (kb_lo) and l + 32 (kb_hi) of the batch row.
struct TileRange {
  int t_begin, t_end;
  bool any_kept;
};
__device__ __forceinline__ TileRange tile_range(uint32_t kb_lo, uint32_t kb_hi, int i0, int L, int lane) {
  const int n_kt = (L + BK - 1) / BK;
  const uint32_t nz_lo = __ballot_sync(0xffffffffu, kb_lo != 0u);
  const uint32_t nz_hi = __ballot_sync(0xffffffffu, kb_hi != 0u);
  const int qw = i0 >> 5;                       // first mask word of the query tile (a multiple of 4)
  const bool q_hi = qw >= 32;
  const uint32_t kb = q_hi ? kb_hi : kb_lo;
  const int wl = qw & 31;
  const bool in_q = lane >= wl && lane < wl + BM / 32;
  const int rows_here = L - 32 * (lane + (q_hi ? 32 : 0));   // in-range rows of this lane's word
  const uint32_t full = rows_here >= 32 ? 0xffffffffu : (rows_here <= 0 ? 0u : ((1u << rows_here) - 1u));
  const bool any_kept = __ballot_sync(0xffffffffu, in_q && kb != 0u) != 0u;
  const bool any_padded = __ballot_sync(0xffffffffu, in_q && (kb & full) != full) != 0u;
  TileRange r{0, n_kt, any_kept};
  if (!any_padded && (nz_lo | nz_hi) != 0u) {
    const int first = nz_lo ? __ffs(nz_lo) - 1 : 32 + __ffs(nz_hi) - 1;
    const int last = nz_hi ? 32 + 31 - __clz(nz_hi) : 31 - __clz(nz_lo);
    r.t_begin = first >> 2;
    r.t_end = (last >> 2) + 1;
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
  int fail_code = 0;   // code of the bounded wait of this thread that expired first, if any

  // ------------------------------------------------------------------ setup (once per CTA)
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bars->q_full, 1);
    ptx::mbar_init(&bars->q_empty, 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&bars->k_full[s], 1);
      ptx::mbar_init(&bars->k_empty[s], 1);
      ptx::mbar_init(&bars->v_full[s], 1);
      ptx::mbar_init(&bars->v_empty[s], 1);
      ptx::mbar_init(&bars->rk_full[s], 1);
      ptx::mbar_init(&bars->rk_empty[s], 1);
      ptx::mbar_init(&bars->rq_full[s], 1);
      ptx::mbar_init(&bars->rq_empty[s], 1);
    }
    for (int s = 0; s < kItemSlots; ++s) {
      ptx::mbar_init(&bars->item_full[s], 1);
      ptx::mbar_init(&bars->item_empty[s], kConsumerWarps);
    }
    ptx::mbar_init(&bars->b1_full, 1);
    ptx::mbar_init(&bars->s_full, 1);
    ptx::mbar_init(&bars->s_free, kSoftmaxWarps);   // one elected lane per softmax warp
    ptx::mbar_init(&bars->xc_full, 1);
    ptx::mbar_init(&bars->xc_free, 4);              // converter warps
    ptx::mbar_init(&bars->xp_full, 1);
    ptx::mbar_init(&bars->xp_free, 4);              // converter warps
    ptx::mbar_init(&bars->pt_ready, 4);
    ptx::mbar_init(&bars->pt_release, kSoftmaxWarps);
    ptx::mbar_init(&bars->p_full, kSoftmaxWarps);
    ptx::mbar_init(&bars->o_ready, 1);
    ptx::mbar_init(&bars->o_free, kSoftmaxWarps);
    ptx::mbar_init(&bars->c2p_ready, 4);
    ptx::mbar_init(&bars->ring_release, kSoftmaxWarps);
    for (int s = 0; s < 4; ++s) ptx::mbar_init(&bars->pair2[s], 2);
    ptx::mbar_init(&bars->xbar, kSoftmaxWarps);
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

  // A bounded wait whose verdict is the same in every lane of the warp (the tcgen05.ld/st/wait instructions that
  // follow are warp-collective and must not be reached by part of a warp).
  auto wwait = [&](uint64_t* bar, uint32_t parity, int code) -> bool {
    return __all_sync(0xffffffffu, ptx::mbar_wait_inline(bar, parity, abort_flag, fail_code, code));
  };

  // The set-up above overlaps the tail of the previous kernel of the stream; Q, K, V, the mask and the status word
  // are touched from here on.
  wait_for_predecessor();

  // Every role walks the same item sequence (item number k of this CTA is item blockIdx.x + k * gridDim.x; it uses
  // item slot k % 3 in phase (k / 3) & 1) and keeps its own running counters.  Register budgets are set per
  // warpgroup (warps 0-3, 4-7: softmax; 8-11: converters; 12-15: the rest), at the head of the branch the whole
  // warpgroup takes.  The loops over a tile's keys are rolled on purpose: the kernel is bound by instruction fetch
  // as soon as the code of a tile no longer fits the instruction caches.
  if (warp < kSoftmaxWarps) {
    setmaxnreg_inc<kSoftmaxRegs>();
    // ----------------------------------------------------------------- softmax
    const int hf = warp >> 2, q4 = warp & 3;    // key half of the tile, lane quarter
    const int r = q4 * 32 + lane;               // query row of the tile = TMEM lane
    const float cscale = p.scale * 1.4426950408889634f;
    const float slack = attn::kLazyMaxSlack / cscale;
    constexpr int OW = D / 2;                   // output columns per thread
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    const uint32_t t_s = tmem_base + lane_base + COL_S + hf * 64;
    const uint32_t t_p = tmem_base + lane_base + COL_P + hf * 32;
    const uint32_t t_o = tmem_base + lane_base + COL_O + hf * OW;
    const uint32_t ring_row = ptx::smem_u32(smem + LO::offRing) + (uint32_t)(r * RING_PITCH);
    const uint32_t odd16 = (uint32_t)(r & 1) * 16u;   // a row's window starts on an odd column iff r is odd
    // P2C of (row r, key n) is element (n & 7) + 128 - r of staging row n
    const uint32_t stg_base = ptx::smem_u32(smem + LO::offStg) + (uint32_t)(hf * 64 * STG_PITCH + 2 * (128 - r));
    float* xmax = reinterpret_cast<float*>(smem + LO::offXmax);
    float* xsum = reinterpret_cast<float*>(smem + LO::offXsum);
    uint64_t* pair2 = &bars->pair2[q4];
    // Two running counts give every barrier phase of this role: c_t = key tiles started (all items), c_i = items with
    // kept rows finished.  Per tile one phase each of s_full, c2p_ready, pt_ready and o_ready, per tile and per item
    // one of pair2; an item of padded rows only uses xbar exactly twice (phases 0 and 1).
    uint32_t c_t = 0, c_i = 0;
    bool ok = true;

    int k = 0;
    for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x, ++k) {
      const int slot = k % kItemSlots;
      ok = wwait(&bars->item_full[slot], (uint32_t)(k / kItemSlots) & 1u, 33);
      if (!ok) break;
      const ItemSlot* sl = &slots[slot];
      const int t_begin = sl->t_begin, n = sl->t_end - sl->t_begin;
      const bool any_kept = sl->any_kept != 0;
      const int bh = sl->bh, b = bh / H, h = bh - b * H;
      const int i0 = sl->i0;

      // where the item's rows go: [B,L,H*d], or packed rows of the sequence (see DflAttnRelParams.out_row_base)
      const long long out_row0 = p.out_row_base ? (long long)p.out_row_base[b] : (long long)b * L;
      const int out_rows = p.out_row_base ? p.out_row_count[b] : L;
      if (!any_kept && out_rows <= i0) {
        // a tile of padded positions that the packed output does not hold: nothing to compute, nothing to store
      } else if (!any_kept) {
        // Every query row of this tile is padding: each attends uniformly to all L keys, so every output row is
        // the column mean of V.  No score, no softmax: one pass over V by the 256 softmax threads.
        // 16-byte loads, every thread sums 8 columns over a stride of rows; the row groups of a warp are folded with
        // shuffles and the eight warps through shared memory (the row-exchange words are idle during such an item).
        float* part = xmax;                                                  // [8 warps][D] partial sums
        T* mean = reinterpret_cast<T*>(smem + LO::offMeanV + 1024);          // [D]
        constexpr int kChunks = D / 8;             // 16-byte chunks per row of V
        constexpr int kRowStep = 256 / kChunks;    // rows covered by the 256 threads at once
        const int tid = threadIdx.x, chunk = tid % kChunks, rgrp = tid / kChunks;
        const uint4* V4 = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.v) + (long long)bh * L * D);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int row = rgrp; row < L; row += kRowStep) {
          const uint4 raw = __ldg(V4 + (long long)row * kChunks + chunk);
          const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += Elem<T>::to_f(e[j]);
        }
#pragma unroll
        for (int o = kChunks; o < 32; o <<= 1) {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
        }
        if (lane < kChunks) {
#pragma unroll
          for (int j = 0; j < 8; ++j) part[warp * D + lane * 8 + j] = acc[j];
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bars->xbar);
        ok = wwait(&bars->xbar, 0u, 34);
        if (!ok) break;
        if (tid < D) {
          float total = 0.0f;
#pragma unroll
          for (int w = 0; w < kSoftmaxWarps; ++w) total += part[w * D + tid];
          mean[tid] = Elem<T>::from_f(total / (float)L);
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bars->xbar);
        ok = wwait(&bars->xbar, 1u, 35);
        if (!ok) break;
        const int rows = out_rows - i0 < BM ? out_rows - i0 : BM;
        constexpr int kVec = D / 8;  // 16-byte chunks per output row
        const uint4 mine = *reinterpret_cast<const uint4*>(mean + (tid % kVec) * 8);
        T* out = reinterpret_cast<T*>(p.out) + (out_row0 + i0) * ((long long)H * D) + (long long)h * D;
        for (int e = tid; e < rows * kVec; e += 256) {
          const int rr = e / kVec, v = e - rr * kVec;
          *reinterpret_cast<uint4*>(out + (long long)rr * H * D + v * 8) = mine;
        }
      } else {
        const int i = i0 + r;
        const bool row_ok = i < L;
        const bool q_keep = row_ok && ((sl->kbits[i >> 5] >> (i & 31)) & 1u) != 0u;
        float m_run = -INFINITY, l_run = 0.0f;

        for (int u = 0; u < n && ok; ++u) {
          const int t = t_begin + u;
          const uint32_t kb0 = sl->kbits[4 * t + 2 * hf], kb1 = sl->kbits[4 * t + 2 * hf + 1];
          const int n_in = L - t * BK - hf * 64;   // in-range keys among this thread's 64 (may be <= 0 or >= 64)
          // ring column of (row r, key x of the tile): (128 * (u & 1) + 128 - r + x) mod 256
          const uint32_t cb = (128u * (uint32_t)(u & 1) + 128u - (uint32_t)r + 64u * (uint32_t)hf) & 255u;

          const uint32_t tile_phase = c_t & 1u;
          ++c_t;
          ok = wwait(&bars->s_full, tile_phase, 41);
          if (ok && has_c2p) ok = wwait(&bars->c2p_ready, tile_phase, 42);
          if (ok && has_p2c) ok = wwait(&bars->pt_ready, tile_phase, 44);
          if (!ok) break;
          ptx::tc_fence_after();

          // ---- pass 1 over the thread's 64 keys in two chunks of 32: S from TMEM (the next chunk in flight), the two
          // relative terms from shared memory, mask, running maximum; the biased scores go back to the S columns.
          float cur[32], nxt[32];
          float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
          DFL_TMEM_LD32_F(t_s, nxt, 0);
#pragma unroll 1
          for (int q = 0; q < 2; ++q) {
            ptx::tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 32; ++x) cur[x] = nxt[x];
            if (q == 0) DFL_TMEM_LD32_F(t_s + 32, nxt, 0);
            if (has_p2c) {
              const uint32_t paddr = stg_base + (uint32_t)(q * 32 * STG_PITCH);
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                // per 16 keys: 16 loads issued before the 16 adds that use them (a warp issues in order)
                uint32_t pv[16];
#pragma unroll
                for (int x = 0; x < 16; ++x)
                  pv[x] = lds_u16_r32(paddr + (uint32_t)((16 * j + x) * STG_PITCH + 2 * (x & 7)));
#pragma unroll
                for (int x = 0; x < 16; ++x) cur[16 * j + x] = Pack2<T>::add(cur[16 * j + x], (uint16_t)pv[x]);
              }
              // the staging tile is read: the converters may fill it for the next tile while the C2P terms of this
              // chunk, the mask and pass 2 are still to come
              if (q == 1) {
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&bars->pt_release);
              }
            }
            if (has_c2p) {
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                // 16 keys are read as nine aligned 32-bit words and shifted by one element where the run starts on
                // an odd column; the run stays below column 272 (the first 16 columns are mirrored behind the ring)
                const uint32_t w0 = (cb + 32u * (uint32_t)q + 16u * j) & 255u;
                const uint32_t caddr = ring_row + 2u * (w0 & ~1u);
                uint32_t cw[9];
#pragma unroll
                for (int x = 0; x < 9; ++x) cw[x] = lds_u32(caddr + 4u * x);
#pragma unroll
                for (int x = 0; x < 8; ++x)
                  add_pair<T>(cur[16 * j + 2 * x], cur[16 * j + 2 * x + 1], funnel_r(cw[x], cw[x + 1], odd16));
              }
            }
            // mask: keys >= L and padded keys -> -inf; a padded query row -> 0 on every in-range key
            const uint32_t kbq = q ? kb1 : kb0;
            if (!q_keep) {
              const int n_q = n_in - 32 * q;
#pragma unroll
              for (int x = 0; x < 32; ++x) cur[x] = x < n_q ? 0.0f : -INFINITY;
            } else if (kbq != 0xffffffffu) {
#pragma unroll
              for (int x = 0; x < 32; ++x)
                if (!((kbq >> x) & 1u)) cur[x] = -INFINITY;
            }
#pragma unroll
            for (int x = 0; x < 32; x += 2) mx[(x >> 1) & 3] = max3(mx[(x >> 1) & 3], cur[x], cur[x + 1]);
            DFL_TMEM_ST32_F(t_s + 32 * q, cur, 0);
          }
          // the ring blocks and the staging tile of this tile are read
          __syncwarp();
          if (lane == 0 && has_c2p) ptx::mbar_arrive(&bars->ring_release);
          const float my_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
          // the row maximum of the tile needs the other half of the keys: exchange through shared memory
          const uint32_t pair_phase = (c_t + c_i + 1u) & 1u;   // c_t - 1 tiles and c_i items before this exchange
          float* xm = xmax + pair_phase * (2 * BM);
          xm[hf * BM + r] = my_max;
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(pair2);
          ptx::tmem_wait_st();
          DFL_TMEM_LD32_F(t_s, nxt, 0);   // first chunk of pass 2, in flight during the exchange
          ok = wwait(pair2, pair_phase, 45);
          if (!ok) break;
          const float tile_max = fmaxf(my_max, xm[(1 - hf) * BM + r]);

          // Lazy reference maximum: m_run moves only when the tile maximum exceeds it by more than 2^8 after scaling,
          // so exp2 arguments stay <= 8 (P <= 256, exact range of both 16-bit types) and O needs rescaling rarely.
          // Both threads of a row see the same m_run and tile_max and take the same decision.
          bool pv_seen = false;   // PV(u-1) known complete
          const bool move = tile_max > m_run + slack;   // also true for the first finite maximum
          if (__any_sync(0xffffffffu, move)) {
            const float m_new = move ? tile_max : m_run;
            const float m_use = m_new == -INFINITY ? 0.0f : m_new;
            const float corr = move ? ptx::ex2_approx((m_run - m_use) * cscale) : 1.0f;   // 0 when m_run = -inf
            m_run = m_new;
            l_run *= corr;
            if (u >= 1) {   // O holds the item's earlier tiles: rescale this thread's half of the columns
              ok = wwait(&bars->o_ready, c_t & 1u, 46);   // PV(u-1): c_t - 2 completed before it
              pv_seen = true;
              if (!ok) break;
              ptx::tc_fence_after();
#pragma unroll
              for (int c0 = 0; c0 < OW; c0 += 16) {
                uint32_t o[16];
                ptx::tmem_ld16(t_o + c0, o);
                ptx::tmem_wait_ld();
#pragma unroll
                for (int x = 0; x < 16; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * corr);
                ptx::tmem_st16(t_o + c0, o);
              }
            }
          }
          const float neg_m = -(m_run == -INFINITY ? 0.0f : m_run) * cscale;

          // ---- pass 2: P = exp2(biased score * scale - reference), rounded, to the P columns; row sum.
          // The row sum is taken over P as rounded for the tensor core, so that the weights P/l the output is
          // built from sum to one exactly.  (The reference sums the unrounded values, kernel.py:316-333; with the
          // lazy reference maximum the largest P of a row is not the exactly representable 1.0, and an unrounded
          // sum would leave the rounding error of the dominant key uncompensated.)
          float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
          for (int q = 0; q < 2; ++q) {
            ptx::tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 32; ++x) cur[x] = nxt[x];
            if (q == 0) {
              DFL_TMEM_LD32_F(t_s + 32, nxt, 0);
            } else {
              // the whole S half is in registers: the accumulator is free for the next tile's S
              ptx::tc_fence_before();
              __syncwarp();
              if (lane == 0) ptx::mbar_arrive(&bars->s_free);
            }
#pragma unroll
            for (int x = 0; x < 32; ++x) cur[x] = fmaf(cur[x], cscale, neg_m);
#pragma unroll
            for (int x = 0; x < 32; ++x) cur[x] = ptx::ex2_approx(cur[x]);
            uint32_t packed[16];
#pragma unroll
            for (int x = 0; x < 32; x += 2) packed[x / 2] = Pack2<T>::pack(cur[x], cur[x + 1]);
#pragma unroll
            for (int x = 0; x < 16; ++x) add_pair<T>(sum[(2 * x) & 3], sum[(2 * x + 1) & 3], packed[x]);
            // the P buffer is the A operand of the previous tile's PV until that MMA completes
            if (q == 0 && u >= 1 && !pv_seen) {
              ok = wwait(&bars->o_ready, c_t & 1u, 47);
              if (!ok) break;
              ptx::tc_fence_after();
            }
            ptx::tmem_st16(t_p + 16 * q, packed);
          }
          if (!ok) break;
          l_run += (sum[0] + sum[1]) + (sum[2] + sum[3]);
          ptx::tmem_wait_st();
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&bars->p_full);
        }
        if (!ok) break;

        // ---- the item's last PV, then normalise and store this thread's half of the output columns
        ok = wwait(&bars->o_ready, (c_t & 1u) ^ 1u, 48);   // the item's last PV: c_t - 1 completed before it
        if (!ok) break;
        ptx::tc_fence_after();
        xsum[hf * BM + r] = l_run;
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(pair2);
        ok = wwait(pair2, (c_t + c_i) & 1u, 49);
        ++c_i;
        if (!ok) break;
        const float inv = 1.0f / (l_run + xsum[(1 - hf) * BM + r]);
        uint32_t o[OW];
        attn::tmem_ld_n(t_o, o);
        ptx::tmem_wait_ld();
        // the accumulator is in registers: the next item's second C2P block and first PV may overwrite it
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bars->o_free);
        if (row_ok && i < out_rows) {
          T* out = reinterpret_cast<T*>(p.out) + (out_row0 + i) * ((long long)H * D) + (long long)h * D + hf * OW;
#pragma unroll
          for (int v = 0; v < OW / 8; ++v) {
            uint4 pk;
            pk.x = Pack2<T>::pack(__uint_as_float(o[v * 8 + 0]) * inv, __uint_as_float(o[v * 8 + 1]) * inv);
            pk.y = Pack2<T>::pack(__uint_as_float(o[v * 8 + 2]) * inv, __uint_as_float(o[v * 8 + 3]) * inv);
            pk.z = Pack2<T>::pack(__uint_as_float(o[v * 8 + 4]) * inv, __uint_as_float(o[v * 8 + 5]) * inv);
            pk.w = Pack2<T>::pack(__uint_as_float(o[v * 8 + 6]) * inv, __uint_as_float(o[v * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(out + v * 8) = pk;
          }
        }
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bars->item_empty[slot]);
    }
  } else if (warp < kMmaWarp) {
    setmaxnreg_dec<kConvRegs>();
    // -------------------------------------------------------------- converters
    // Thread (quarter q4, lane) owns TMEM lane 32*q4 + lane of both transit accumulators:
    //   C2P blocks: query row r of the tile; the block's 128 columns are rounded and stored to ring row r.
    //   P2C halves: key n of the tile.  Of the 256 table rows of the tile's window, the 128 queries reach rows
    //     n+1 .. n+128; the chunk-aligned span [8*(n/8), 8*(n/8) + 136) is stored to staging row n.
    // Jobs are taken in the order the MMA issuer produces them.
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    const int c_first = row >> 3;   // first chunk of the staging span (chunks are 8 table rows = 16 bytes)
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    const uint32_t t_xp = tmem_base + lane_base + COL_XP;
    const uint32_t t_xc = tmem_base + lane_base + COL_XC;
    const uint32_t t_b1 = tmem_base + lane_base + COL_P;   // second block of an item: P and O columns
    const uint32_t stg_row = ptx::smem_u32(smem + LO::offStg) + (uint32_t)(row * STG_PITCH) - (uint32_t)(c_first * 16);
    const uint32_t ring_row = ptx::smem_u32(smem + LO::offRing) + (uint32_t)(row * RING_PITCH);
    uint32_t c_xp = 0, c_xc = 0, c_b1 = 0, c_pt = 0;
    uint32_t rel_seen = 0;      // phases of ring_release (one per key tile) waited for so far
    uint32_t tiles_before = 0;  // key tiles of all earlier items
    bool ok = true;

    // One C2P block: TMEM (two pieces of 64 columns) -> 16-bit -> ring block `pos` of this thread's row.  The ring
    // position must be free: `need` key tiles in total must have been read by all softmax warps.
    auto convert_block = [&](uint32_t t_src, uint64_t* full, uint32_t full_parity, bool frees_xc, int pos, uint32_t need) -> bool {
      if (!wwait(full, full_parity, 18)) return false;
      ptx::tc_fence_after();
#pragma unroll 1
      for (int piece = 0; piece < 2; ++piece) {
        uint32_t r0[32], r1[32];
        ptx::tmem_ld32(t_src + piece * 64, r0);
        ptx::tmem_ld32(t_src + piece * 64 + 32, r1);
        ptx::tmem_wait_ld();
        if (piece == 1 && frees_xc) {   // the block is in registers: the accumulator is free for the next block's MMA
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&bars->xc_free);
        }
        if (piece == 0) {
          while (rel_seen < need) {
            if (!wwait(&bars->ring_release, rel_seen & 1u, 17)) return false;
            ++rel_seen;
          }
        }
        const uint32_t dst = ring_row + (uint32_t)(pos * 256 + piece * 128);
#pragma unroll
        for (int x = 0; x < 32; x += 2) {
          const uint32_t w = Pack2<T>::pack(__uint_as_float(r0[x]), __uint_as_float(r0[x + 1]));
          sts_u32(dst + 2 * x, w);
          if (x < RING_MIRROR && pos == 0 && piece == 0) sts_u32(dst + RING_COLS * 2 + 2 * x, w);
        }
#pragma unroll
        for (int x = 0; x < 32; x += 2)
          sts_u32(dst + 64 + 2 * x, Pack2<T>::pack(__uint_as_float(r1[x]), __uint_as_float(r1[x + 1])));
      }
      return true;
    };
    // One half (128 table rows) of a tile's P2C accumulator -> staging.  half 0 also waits for the staging tile.
    auto convert_half = [&](int half) -> bool {
      if (!wwait(&bars->xp_full, c_xp & 1u, 19)) return false;
      ptx::tc_fence_after();
      // A warp's 32 keys reach chunks 4*q4 .. 4*q4 + 19 of the window's 32: quarters 2 and 3 never store anything of
      // the first 64 columns of the first half, quarters 0 and 1 nothing of the last 64 of the second half.
      const int p_begin = (half == 0 && q4 >= 2) ? 1 : 0;
      const int p_end = (half == 1 && q4 <= 1) ? 1 : 2;
#pragma unroll 1
      for (int piece = p_begin; piece < p_end; ++piece) {
        uint32_t r0[32], r1[32];
        ptx::tmem_ld32(t_xp + piece * 64, r0);
        ptx::tmem_ld32(t_xp + piece * 64 + 32, r1);
        ptx::tmem_wait_ld();
        if (piece == p_end - 1) {   // what this warp needs of the half is in registers: its share of xp_free
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&bars->xp_free);
        }
        if (half == 0 && piece == p_begin) {
          // the staging tile must have been read by all softmax warps (previous tile)
          if (!wwait(&bars->pt_release, (c_pt & 1u) ^ 1u, 20)) return false;
        }
        // 8 chunks of 8 table rows; chunk c of the window goes to position c - c_first if that is in [0, 16]
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint32_t (&src)[32] = c < 4 ? r0 : r1;
          const int x = (c & 3) * 8;
          const uint32_t w0 = Pack2<T>::pack(__uint_as_float(src[x + 0]), __uint_as_float(src[x + 1]));
          const uint32_t w1 = Pack2<T>::pack(__uint_as_float(src[x + 2]), __uint_as_float(src[x + 3]));
          const uint32_t w2 = Pack2<T>::pack(__uint_as_float(src[x + 4]), __uint_as_float(src[x + 5]));
          const uint32_t w3 = Pack2<T>::pack(__uint_as_float(src[x + 6]), __uint_as_float(src[x + 7]));
          const int chunk = half * 16 + piece * 8 + c;
          if (chunk >= c_first && chunk <= c_first + (STG_CHUNKS - 1)) sts_v4(stg_row + (uint32_t)(chunk * 16), w0, w1, w2, w3);
        }
      }
      ++c_xp;
      return true;
    };

    int k = 0;
    for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x, ++k) {
      const int slot = k % kItemSlots;
      ok = wwait(&bars->item_full[slot], (uint32_t)(k / kItemSlots) & 1u, 32);
      if (!ok) break;
      const ItemSlot* sl = &slots[slot];
      const int n = sl->t_end - sl->t_begin;
      if (sl->any_kept != 0) {
        // Jobs of the item in production order: block 0 | P2C of tile 0 | block 1 | per further tile u: first half,
        // block u + 1, second half.  One flat loop with one copy of each conversion routine: the converter's code
        // shares the instruction cache with the softmax warps of its scheduler.
        for (int u = 0; u < n && ok; ++u) {
#pragma unroll 1
          for (int jb = 0; jb < 4 && ok; ++jb) {
            // kind: 0 nothing, 1 C2P block from the XC accumulator, 2 C2P block from the P/O columns, 3 P2C half
            int kind, arg;
            if (u == 0) {
              kind = jb == 0 ? 1 : (jb == 3 ? 2 : 3);
              arg = jb == 0 ? 0 : (jb == 3 ? 1 : jb - 1);          // ring position / half
            } else {
              kind = jb == 0 ? 0 : (jb == 2 ? 1 : 3);
              arg = jb == 2 ? ((u + 1) & 1) : (jb == 1 ? 0 : 1);   // block u + 1 replaces block u - 1
            }
            if (kind == 3) {
              if (has_p2c) ok = convert_half(arg);
            } else if (kind != 0 && has_c2p) {
              const bool from_xc = kind == 1;
              ok = convert_block(from_xc ? t_xc : t_b1, from_xc ? &bars->xc_full : &bars->b1_full,
                                 (from_xc ? c_xc : c_b1) & 1u, from_xc, arg, tiles_before + (uint32_t)u);
              if (from_xc) ++c_xc; else ++c_b1;
            }
          }
          if (!ok) break;
          __syncwarp();
          if (lane == 0) {
            if (has_c2p) ptx::mbar_arrive(&bars->c2p_ready);
            if (has_p2c) ptx::mbar_arrive(&bars->pt_ready);
          }
          ++c_pt;
        }
        if (has_c2p) tiles_before += (uint32_t)n;
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bars->item_empty[slot]);
    }
  } else {
    setmaxnreg_dec<kMiscRegs>();
    if (warp == kTmaWarp) {
      // ------------------------------------------------- mask analysis + TMA producer
      // Running counts of loads; stage = count % stages, phase = (count / stages) & 1.  Loads are issued in the
      // order the MMA issuer consumes them (a stage that is still in use blocks only loads needed after its release).
      struct LoadItem {
        int t_begin, n, i0, bh, h;
        bool any_kept;
      };
      uint32_t c_q = 0, c_k = 0, c_v = 0, c_rk = 0, c_rq = 0;
      bool ok = true;

      // Mask analysis of item number k2 (item it2), published through its slot.  Warp-collective.
      auto analyze = [&](int k2, int it2, LoadItem& f) -> bool {
        const int slot = k2 % kItemSlots;
        const int qt = it2 / n_bh, bh = it2 - qt * n_bh, b = bh / H;
        const int i0 = qt * BM;
        ItemSlot* sl = &slots[slot];
        if (!wwait(&bars->item_empty[slot], ((uint32_t)(k2 / kItemSlots) & 1u) ^ 1u, 30)) return false;
        const uint32_t kb_lo = kept_bits_word(p, b, lane);
        const uint32_t kb_hi = L > 1024 ? kept_bits_word(p, b, lane + 32) : 0u;
        const TileRange range = tile_range(kb_lo, kb_hi, i0, L, lane);
        sl->kbits[lane] = kb_lo;
        sl->kbits[lane + 32] = kb_hi;
        if (lane == 0) {
          sl->t_begin = range.t_begin;
          sl->t_end = range.t_end;
          sl->any_kept = range.any_kept ? 1 : 0;
          sl->bh = bh;
          sl->i0 = i0;
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bars->item_full[slot]);
        f.t_begin = range.t_begin;
        f.n = range.t_end - range.t_begin;
        f.i0 = i0;
        f.bh = bh;
        f.h = bh - b * H;
        f.any_kept = range.any_kept;
        return true;
      };
      // table row of column 0 of block 0: pair (row r, key x) of tile u uses column 128 - r + x of blocks u, u+1
      auto table_row0 = [&](const LoadItem& f) { return f.t_begin * BK - f.i0 - BM + (L - 1); };
      auto load_rk = [&](const LoadItem& f, int c) -> bool {
        const uint32_t st = c_rk % LO::kRkStages, ph = (c_rk / LO::kRkStages) & 1u;
        if (!ptx::mbar_wait_inline(&bars->rk_empty[st], ph ^ 1u, abort_flag, fail_code, 11)) return false;
        ptx::mbar_arrive_expect_tx(&bars->rk_full[st], (uint32_t)LO::kTile);
        ptx::tma_load_3d(smem + LO::offRK + st * LO::kTile, &tmap_fk, &bars->rk_full[st], 0, table_row0(f) + c * BK, f.h);
        ++c_rk;
        return true;
      };
      auto load_rq = [&](const LoadItem& f, int c) -> bool {
        const uint32_t st = c_rq & 1u, ph = (c_rq >> 1) & 1u;
        if (!ptx::mbar_wait_inline(&bars->rq_empty[st], ph ^ 1u, abort_flag, fail_code, 12)) return false;
        ptx::mbar_arrive_expect_tx(&bars->rq_full[st], (uint32_t)LO::kTile);
        ptx::tma_load_3d(smem + LO::offRQ + st * LO::kTile, &tmap_fq, &bars->rq_full[st], 0, table_row0(f) + c * BK, f.h);
        ++c_rq;
        return true;
      };
      auto load_k = [&](const LoadItem& f, int u) -> bool {
        const uint32_t st = c_k & 1u, ph = (c_k >> 1) & 1u;
        if (!ptx::mbar_wait_inline(&bars->k_empty[st], ph ^ 1u, abort_flag, fail_code, 1)) return false;
        ptx::mbar_arrive_expect_tx(&bars->k_full[st], (uint32_t)LO::kTile);
        ptx::tma_load_3d(smem + LO::offK + st * LO::kTile, &tmap_k, &bars->k_full[st], 0, (f.t_begin + u) * BK, f.bh);
        ++c_k;
        return true;
      };
      auto load_v = [&](const LoadItem& f, int u) -> bool {
        const uint32_t st = c_v % LO::kVStages, ph = (c_v / LO::kVStages) & 1u;
        if (!ptx::mbar_wait_inline(&bars->v_empty[st], ph ^ 1u, abort_flag, fail_code, 2)) return false;
        ptx::mbar_arrive_expect_tx(&bars->v_full[st], (uint32_t)LO::kTile);
        ptx::tma_load_3d(smem + LO::offV + st * LO::kTile, &tmap_v, &bars->v_full[st], 0, (f.t_begin + u) * BK, f.bh);
        ++c_v;
        return true;
      };
      // what the first MMAs of an item need: Q, first rel_key block, K of the first tile, first two rel_query blocks
      auto prologue_loads = [&](const LoadItem& f) -> bool {
        if (!ptx::mbar_wait_inline(&bars->q_empty, (c_q & 1u) ^ 1u, abort_flag, fail_code, 3)) return false;
        ptx::mbar_arrive_expect_tx(&bars->q_full, (uint32_t)LO::kTile);
        ptx::tma_load_3d(smem + LO::offQ, &tmap_q, &bars->q_full, 0, f.i0, f.bh);
        ++c_q;
        if (has_c2p && !load_rk(f, 0)) return false;
        if (!load_k(f, 0)) return false;
        if (has_p2c && !(load_rq(f, 0) && load_rq(f, 1))) return false;
        return true;
      };

      LoadItem cur{}, nxt{};
      int it = blockIdx.x, k = 0;
      if (it < n_items) {
        ok = analyze(0, it, cur);
        if (ok && cur.any_kept && lane == 0) ok = prologue_loads(cur);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
      for (; it < n_items && ok; it += gridDim.x, ++k) {
        const bool has_next = n_items - it > (int)gridDim.x;
        // what the item needs right at its start goes out before the next item's mask is analysed
        if (cur.any_kept && lane == 0) {
          if (has_c2p) ok = load_rk(cur, 1);
          if (ok && cur.n > 1) {
            ok = load_k(cur, 1);
            if (ok && has_c2p) ok = load_rk(cur, 2);
            if (ok && has_p2c) ok = load_rq(cur, 2);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (ok && has_next) ok = analyze(k + 1, it + (int)gridDim.x, nxt);
        if (!ok) break;
        const bool next_kept = has_next && nxt.any_kept;
        if (lane == 0) {
          if (cur.any_kept) {
            for (int u = 0; u < cur.n && ok; ++u) {
              if (u + 1 < cur.n) {
                if (u > 0) {
                  ok = load_k(cur, u + 1);
                  if (ok && has_c2p) ok = load_rk(cur, u + 2);
                  if (ok && has_p2c) ok = load_rq(cur, u + 2);
                }
              } else if (next_kept) {
                ok = prologue_loads(nxt);
              }
              if (ok) ok = load_v(cur, u);
            }
          } else if (next_kept) {
            ok = prologue_loads(nxt);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        cur = nxt;
      }
    } else if (warp == kMmaWarp) {
      // -------------------------------------------------------------- MMA issuer
      // One thread issues every MMA; descriptors are kept as precomputed 32-bit halves (only the start-address
      // field moves).  Order per key tile u (steady state): the next tile's first P2C half, new C2P block and second
      // P2C half while the softmax threads work on tile u, the next tile's S as soon as they have read S(u), then
      // PV(u) as soon as P(u) is stored.  In the item's last tile the place of the next tile's MMAs is taken by the
      // first MMAs of the next item.
      if (lane == 0) {
        constexpr int is_bf16 = __is_same(T, __nv_bfloat16) ? 1 : 0;
        constexpr uint32_t idesc_nn = ptx::make_idesc_f16(is_bf16, BM, 128, 0, 0);   // 128 x 128, both K-major
        constexpr uint32_t idesc_pv = ptx::make_idesc_f16(is_bf16, BM, D, 0, 1);     // 128 x D, V is MN-major
        constexpr uint32_t mode = ptx::swizzle_mode_for_row_bytes(LO::kRowBytes);
        constexpr uint32_t sbo = 8 * LO::kRowBytes;
        constexpr int kSteps = LO::kRowBytes / 32;   // K=16 steps over d
        // shared-memory descriptor = {lo, hi}: lo = start>>4 | (leading offset>>4) << 16, hi = stride offset>>4 |
        // version 1 << 14 | swizzle << 29; every operand here shares hi
        constexpr uint32_t desc_hi = ((sbo >> 4) & 0x3FFFu) | (1u << 14) | (mode << 29);
        constexpr uint32_t kTileUnits = (uint32_t)LO::kTile >> 4;
        constexpr uint32_t kPvStepUnits = (16u * LO::kRowBytes) >> 4;   // 16 keys further down the V tile
        auto desc_lo = [](uint32_t addr, uint32_t lbo) { return ((addr >> 4) & 0x3FFFu) | ((lbo >> 4) << 16); };
        const uint32_t q_lo = desc_lo(ptx::smem_u32(smem + LO::offQ), 16);
        const uint32_t k_lo = desc_lo(ptx::smem_u32(smem + LO::offK), 16);
        const uint32_t rk_lo = desc_lo(ptx::smem_u32(smem + LO::offRK), 16);
        const uint32_t rq_lo = desc_lo(ptx::smem_u32(smem + LO::offRQ), 16);
        const uint32_t v_lo = ((ptx::smem_u32(smem + LO::offV) >> 4) & 0x3FFFu) | (kTileUnits << 16);
        uint32_t c_q = 0, c_k = 0, c_v = 0, c_rk = 0;   // loads consumed (stage / phase as in the loader)
        uint32_t c_s = 0, c_xc = 0, c_xp = 0, c_p = 0;  // S tiles, C2P blocks through XC, P2C halves, PVs issued
        uint32_t rq_alloc = 0;                          // rel_query blocks handed to items so far
        uint32_t c_items = 0;                           // items with kept rows started so far
        bool ok = true;

        // D[128 x 128] = A[128 x d] * B[128 x d]^T, both operands K-major tiles in shared memory
        auto mma_nn = [&](uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo) {
#pragma unroll
          for (int kk = 0; kk < kSteps; ++kk) {
            if (kk == 0) umma_ss_lohi<0>(d_tmem, a_lo, b_lo, desc_hi, idesc_nn);
            else umma_ss_lohi<1>(d_tmem, a_lo + 2u * kk, b_lo + 2u * kk, desc_hi, idesc_nn);
          }
        };
        auto wait1 = [&](uint64_t* bar, uint32_t parity, int code) -> bool {
          return ptx::mbar_wait_inline(bar, parity, abort_flag, fail_code, code);
        };
        // new C2P block = Q . rel_key block^T, into the block accumulator, or (second block of an item) into the
        // P and O columns, which the caller has made sure are idle
        auto issue_c = [&](bool second_block) -> bool {
          const uint32_t st = c_rk % LO::kRkStages, ph = (c_rk / LO::kRkStages) & 1u;
          if (!wait1(&bars->rk_full[st], ph, 13)) return false;
          if (!second_block && !wait1(&bars->xc_free, (c_xc & 1u) ^ 1u, 14)) return false;
          ptx::tc_fence_after();
          mma_nn(tmem_base + (second_block ? COL_P : COL_XC), q_lo, rk_lo + st * kTileUnits);
          ptx::umma_commit(&bars->rk_empty[st]);
          ptx::umma_commit(second_block ? &bars->b1_full : &bars->xc_full);
          ++c_rk;
          if (!second_block) ++c_xc;
          return true;
        };
        // S = Q . K^T of the tile whose K is in stage kst
        auto issue_s = [&](uint32_t kst) -> bool {
          if (!wait1(&bars->s_free, (c_s & 1u) ^ 1u, 6)) return false;
          ptx::tc_fence_after();
          mma_nn(tmem_base + COL_S, q_lo, k_lo + kst * kTileUnits);
          ptx::umma_commit(&bars->s_full);
          ++c_s;
          return true;
        };
        // one half of the P2C accumulator: XP[n, m] = K . rel_query block^T; `first` = first use of the table block
        // (wait for its load), `last` = last use (release its stage)
        auto issue_pt = [&](uint32_t kst, uint32_t blk, bool first, bool last) -> bool {
          const uint32_t st = blk & 1u, ph = (blk >> 1) & 1u;
          if (first && !wait1(&bars->rq_full[st], ph, 15)) return false;
          if (!wait1(&bars->xp_free, (c_xp & 1u) ^ 1u, 16)) return false;
          ptx::tc_fence_after();
          mma_nn(tmem_base + COL_XP, k_lo + kst * kTileUnits, rq_lo + st * kTileUnits);
          if (last) ptx::umma_commit(&bars->rq_empty[st]);
          ptx::umma_commit(&bars->xp_full);
          ++c_xp;
          return true;
        };
        // The first MMAs of an item with n key tiles: first C2P block, both P2C halves of tile 0, S(0).  rq0 receives
        // the number of the item's first rel_query block (tile u uses blocks rq0 + u and rq0 + u + 1).
        auto item_head = [&](int n, uint32_t& rq0) -> bool {
          if (!wait1(&bars->q_full, c_q & 1u, 4)) return false;
          ++c_q;
          if (has_c2p && !issue_c(false)) return false;
          const uint32_t kst = c_k & 1u;
          if (!wait1(&bars->k_full[kst], (c_k >> 1) & 1u, 5)) return false;
          rq0 = rq_alloc;
          if (has_p2c) {
            if (!(issue_pt(kst, rq0, true, true) && issue_pt(kst, rq0 + 1u, true, n == 1))) return false;
            rq_alloc += (uint32_t)n + 1u;
          }
          if (!issue_s(kst)) return false;
          ptx::umma_commit(&bars->k_empty[kst]);
          ++c_k;
          return true;
        };
        struct ItemInfo {
          bool any_kept;
          int n;
        };
        auto get_item = [&](int k2, ItemInfo& f) -> bool {
          const int slot = k2 % kItemSlots;
          if (!wait1(&bars->item_full[slot], (uint32_t)(k2 / kItemSlots) & 1u, 31)) return false;
          f.any_kept = slots[slot].any_kept != 0;
          f.n = slots[slot].t_end - slots[slot].t_begin;
          return true;
        };

        ItemInfo cur{false, 0}, nxt{false, 0};
        uint32_t cur_rq = 0, nxt_rq = 0;
        int it = blockIdx.x, k = 0;
        if (it < n_items) {
          ok = get_item(0, cur);
          if (ok && cur.any_kept) ok = item_head(cur.n, cur_rq);
        }
        for (; it < n_items && ok; it += gridDim.x, ++k) {
          const bool has_next = n_items - it > (int)gridDim.x;
          // The output accumulator of the previous item with kept rows has been read out (o_free completes one phase per
          // such item; this thread is never more than one phase behind, so parities cannot alias).
          if (cur.any_kept) {
            if (c_items > 0) ok = wait1(&bars->o_free, (c_items - 1u) & 1u, 38);
            ++c_items;
          }
          if (!ok) break;
          if (cur.any_kept) {
            const int n = cur.n;
            if (has_c2p) ok = issue_c(true);
            if (ok && n == 1) ptx::umma_commit(&bars->q_empty);
            for (int u = 0; u < n && ok; ++u) {
              if (u + 1 < n) {
                // ---- front of tile u + 1
                const uint32_t kst = c_k & 1u;
                ok = wait1(&bars->k_full[kst], (c_k >> 1) & 1u, 5);
                if (ok && has_p2c) ok = issue_pt(kst, cur_rq + (uint32_t)(u + 1), false, true);
                if (ok && has_c2p) ok = issue_c(false);
                if (ok && has_p2c) ok = issue_pt(kst, cur_rq + (uint32_t)(u + 2), true, u + 2 == n);
                if (ok) ok = issue_s(kst);   // waits until the softmax threads have read the current tile's S
                if (!ok) break;
                ptx::umma_commit(&bars->k_empty[kst]);
                ++c_k;
                if (u + 2 == n) ptx::umma_commit(&bars->q_empty);   // S(n-1) and the last C2P block are issued
              } else if (has_next) {
                // The next item's slot is read only now: the loader publishes it after loads whose stages this
                // thread's earlier MMAs of the current item release.
                ok = get_item(k + 1, nxt);
                if (ok && nxt.any_kept) ok = item_head(nxt.n, nxt_rq);
                if (!ok) break;
              }
              // ---- PV(u): O (+)= P . V
              const uint32_t vst = c_v % LO::kVStages, vph = (c_v / LO::kVStages) & 1u;
              ok = wait1(&bars->p_full, c_p & 1u, 7) && wait1(&bars->v_full[vst], vph, 8);
              if (!ok) break;
              ptx::tc_fence_after();
              const uint32_t vt_lo = v_lo + vst * kTileUnits;
#pragma unroll
              for (int kk = 0; kk < BK / 16; ++kk)
                umma_ts_lohi(tmem_base + COL_O, tmem_base + COL_P + kk * 8, vt_lo + kk * kPvStepUnits, desc_hi, idesc_pv,
                             (u > 0 || kk > 0) ? 1u : 0u);
              ptx::umma_commit(&bars->v_empty[vst]);
              ptx::umma_commit(&bars->o_ready);
              ++c_v;
              ++c_p;
            }
          } else if (has_next) {
            ok = get_item(k + 1, nxt);
            if (ok && nxt.any_kept) ok = item_head(nxt.n, nxt_rq);
          }
          if (!ok) break;
          ptx::mbar_arrive(&bars->item_empty[k % kItemSlots]);
          cur = nxt;
          cur_rq = nxt_rq;
        }
      }
    }
  }

  if (fail_code != 0 && status_word != nullptr) atomicCAS(status_word, 0, fail_code);
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
  if (rc == DFL_OK) rc = encode_tensor_map_3d(&tk, p.k, D, L, BH, row, seq, D, BK, LO::kRowBytes);
  if (rc == DFL_OK) rc = encode_tensor_map_3d(&tv, p.v, D, L, BH, row, seq, D, BK, LO::kRowBytes);
  // a disabled term reuses the other table's map; it is never dereferenced
  const void* fk = p.rel_key ? p.rel_key : p.rel_query;
  const void* fq = p.rel_query ? p.rel_query : p.rel_key;
  if (rc == DFL_OK) rc = encode_tensor_map_3d(&tfk, fk, D, R, p.heads, row, table, D, BK, LO::kRowBytes);
  if (rc == DFL_OK) rc = encode_tensor_map_3d(&tfq, fq, D, R, p.heads, row, table, D, BK, LO::kRowBytes);
  if (rc != DFL_OK) return rc;

  auto kernel = attention_rel_kernel<T, D>;
  static KernelDeviceConfig config;   // per instantiation
  int sm_count = 0;
  rc = configure_kernel(config, kernel, LO::total, &sm_count, "attention_rel_kernel");
  if (rc != DFL_OK) return rc;
  cudaError_t e;
  int* status_word = p.status;
  if (!status_word) {
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&status_word), g_attn_rel_status);
    if (e != cudaSuccess) return fail(DFL_ERR_LAUNCH, "status word: %s", cudaGetErrorString(e));
  }
  const long long n_items = (long long)BH * ((L + BM - 1) / BM);
  if (n_items > 0x7fffffffLL) return fail(DFL_ERR_TOO_LARGE, "too many (batch, head, query tile) items");
  const int grid = n_items < sm_count ? (int)n_items : sm_count;
  e = launch_after_predecessor(kernel, dim3(grid), dim3(kThreads), LO::total, stream, tq, tk, tv, tfk, tfq, p, status_word,
                               (int)n_items);
  if (e != cudaSuccess) return fail(DFL_ERR_LAUNCH, "attention_rel_kernel: %s", cudaGetErrorString(e));
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
