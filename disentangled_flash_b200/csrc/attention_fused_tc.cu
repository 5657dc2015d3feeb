// tcgen05 fused disentangled attention with the relative scores computed in-kernel.
//
// Same result as dfl_pos_scores + dfl_attention_fwd (reference: the two torch.matmul calls at
// src/disentangled_flash/kernel.py:574-585 followed by the Triton kernel kernel.py:137-345), but the
// C2P and P2C score tensors [B,H,L,A] never exist in global memory: their tiles are produced by
// tcgen05.mma from the small per-head tables posK / posQ [H,A,d] (L2 resident), rounded to the
// input type exactly like the separate GEMMs round their output, and parked in shared memory for
// the softmax threads to gather from.
//
// One CTA = 128 query rows of one (batch, head); key tiles of 64.  The slot table lut is monotone
// with steps 0/1, so the slots a (128 x 64) tile touches form one window [lo, hi] with
// hi - lo <= 190, and the window moves towards lower slots by at most 64 per key tile.
//   C2P: c2p[i, s] = q_i . posK[s] depends on the query rows only, so it is kept across key tiles
//        in a ring of five 64-slot blocks per row; a key tile needs at most one new block
//        (one 128x64x d MMA, the first tile up to four).
//   P2C: p2c[j, s] = k_j . posQ[s] is needed for the 64 keys of the tile and the window's slots:
//        computed transposed, PT[s - lo, j] = posQ[lo + ...] . k_j (one or two 128x64x d MMAs),
//        so that TMEM lanes are slots and all 128 lanes convert.
// Twenty-two warps:
//   warps 0-15  softmax, four threads per query row (warps w, w+4, w+8, w+12 share TMEM lanes 32*(w&3)...):
//               each owns 16 of the 64 keys of a tile and a quarter of the output columns; S from TMEM,
//               gather c2p from the ring row and p2c from PT, agree on the row maximum, then the common tail.
//               Many narrow threads rather than few wide ones: the work is latency bound.
//   warps 16-19 converters: TMEM -> 16-bit -> shared memory for the C2P blocks and the PT tiles.
//   warp 20     TMA producer: Q, K/V ring, posK blocks, posQ windows.
//   warp 21     MMA issuer and TMEM owner: C2P blocks, PT, S = Q K^T, O += P V.
#include "attention_tc_common.cuh"

namespace dfl {

__device__ int g_attn_fused_status = 0;


namespace {

using attn::BM;
using attn::BN;
using attn::Pack2;

constexpr int kParts = 4;                       // softmax threads per query row
constexpr int kSoftmaxWarps = 4 * kParts;
constexpr int kConvWarp0 = kSoftmaxWarps;       // 4 converter warps
constexpr int kTmaWarp = kSoftmaxWarps + 4;
constexpr int kMmaWarp = kSoftmaxWarps + 5;
constexpr int kThreads = (kSoftmaxWarps + 6) * 32;
constexpr int KV_STAGES = 2;
constexpr int RING_BLOCKS = 5;
constexpr int RING_SPAN = RING_BLOCKS * 64;          // 320 ring positions; positions 320..383 mirror 0..63
constexpr int RING_PITCH_H = RING_SPAN + 64 + 2;     // halfs per ring row: 772 bytes = 193 words (odd: conflict free)
constexpr int PT_ROWS = 192;                         // a tile's window has at most 191 slots
constexpr int PT_PITCH_H = BN + 2;                    // halfs per PT row: 132 bytes = 33 words
constexpr int LUT_LO_PAD = BN;
constexpr int LUT_HI_PAD = BM;

// TMEM columns (512 allocated; one CTA per SM is guaranteed by its shared-memory footprint)
constexpr int COL_S = 0;      // 2 x BN
constexpr int COL_P = 128;    // 2 x BN/2
constexpr int COL_CNEW = 192; // BN  (one 64-slot C2P block for 128 rows)
constexpr int COL_PT = 256;   // 2 x BN (slots lo..lo+127 and lo+128..lo+255, 64 keys each)
constexpr int COL_O = 384;    // D
constexpr int kTmemCols = 512;

template <int D>
struct FLayout {
  static constexpr int kRowBytes = D >= 64 ? 128 : D * 2;
  static_assert(D <= 64, "in-kernel relative scores are built for head dims 32 and 64");
  static constexpr int kQ = BM * kRowBytes;            // Q tile; a posQ sub-window has the same shape
  static constexpr int kK = BN * kRowBytes;            // K tile, V tile, posK block
  static constexpr int offQ = 0;
  static constexpr int offKV = offQ + kQ;                      // KV_STAGES x (K, V)
  // posQ window operand: slots lo..lo+127 (kQ bytes) then lo+128..lo+191 (kQ/2 bytes).  The second MMA reads
  // 128 rows from the second part, i.e. runs on into the posK operand that follows; those rows only feed
  // TMEM lanes 64..127, which nobody reads.
  static constexpr int offPQ = offKV + KV_STAGES * 2 * kK;
  static constexpr int offPK = offPQ + kQ + kQ / 2;            // posK block operand (kK = kQ/2 bytes)
  static constexpr int offRing = offPK + kK;                   // C2P ring [128][RING_PITCH_H]
  static constexpr int offPT = offRing + BM * RING_PITCH_H * 2;  // PT staging [256][PT_PITCH_H]
  static constexpr int offBar = (offPT + PT_ROWS * PT_PITCH_H * 2 + 15) & ~15;
  static constexpr int kBarBytes = 512;
  static constexpr int offXchg = offBar + kBarBytes;            // row exchange: [2][kParts][BM] floats
  static constexpr int offTables = offXchg + 2 * kParts * BM * 4;
  // tables: step bits u32[n_lut/32 + 2], lutS u16[n_lut], win_lo/win_hi int16[n_kt] each, kbits u32[2*n_kt]
  static __host__ __device__ constexpr int wbits_bytes(int n_lut) { return (((n_lut + 31) / 32 + 1) * 4 + 15) & ~15; }
  static int total(int L) {
    const int n_lut = 2 * L - 1 + LUT_LO_PAD + LUT_HI_PAD;
    const int n_kt = (L + BN - 1) / BN;
    return offTables + wbits_bytes(n_lut) + ((2 * n_lut + 15) & ~15) + ((4 * n_kt + 15) & ~15) + 8 * n_kt + 1024;
  }
};

struct FBarriers {
  uint64_t q_full;
  uint64_t kv_full[KV_STAGES], kv_empty[KV_STAGES];
  uint64_t s_full[2], s_free[2], p_full[2];
  uint64_t o_ready;
  uint64_t pk_full, pk_empty;        // posK block operand in shared memory
  uint64_t pq_full, pq_empty;        // posQ window operand in shared memory
  uint64_t cnew_full, cnew_free;     // C2P block in TMEM
  uint64_t pt_full, pt_free;         // PT tile in TMEM
  uint64_t c2p_ready[2];             // ring holds everything tile t needs
  uint64_t ring_release[2];          // softmax threads finished gathering C2P of tile t
  uint64_t pt_ready, pt_release;     // PT staging in shared memory
  uint64_t pair[4];                  // per lane quarter: the two softmax warps of a row exchange maxima
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(FBarriers) <= 512, "barrier block too large");

struct FTables {
  const uint32_t* wbits;  // step bits: bit l of word k+1 is slot(32k+l) - slot(32k+l-1) (0 or 1); word 0 is zero
  const uint16_t* lutS;   // slot of each (padded) delta index
  const int16_t* win_lo;  // per key tile: lowest slot touched
  const int16_t* win_hi;  // per key tile: highest slot touched
  const uint32_t* kbits;  // key keep-bits
};

// C2P block jobs of tile t: the first processed tile brings blocks hi>>6 .. lo>>6, later tiles at most one.
struct BlockJobs {
  int first, count;  // blocks first, first-1, ..., first-count+1
};
__device__ __forceinline__ BlockJobs c2p_jobs(const FTables& tb, int t, int t_begin) {
  const int blo = tb.win_lo[t] >> 6;
  if (t == t_begin) return {tb.win_hi[t] >> 6, (tb.win_hi[t] >> 6) - blo + 1};
  const int prev = tb.win_lo[t - 1] >> 6;
  return {blo, blo < prev ? 1 : 0};
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads, 1)
attention_fused_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_pk,
                       const __grid_constant__ CUtensorMap tmap_pq, const __grid_constant__ CUtensorMap tmap_pq64,
                       const DflAttnTablesParams p, int* status_word) {
  using LO = FLayout<D>;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  FBarriers* bars = reinterpret_cast<FBarriers*>(smem + LO::offBar);
  volatile int* abort_flag = &bars->abort_flag;

  const int L = p.seq_len, H = p.heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
  const int i0 = blockIdx.x * BM;
  const int n_kt = (L + BN - 1) / BN;
  const bool has_c2p = p.pos_key != nullptr, has_p2c = p.pos_query != nullptr;
  const int n_lut = 2 * L - 1 + LUT_LO_PAD + LUT_HI_PAD;
  TRACE_DECL
  TRACE(99);

  uint32_t* wbits = reinterpret_cast<uint32_t*>(smem + LO::offTables);          // [(n_lut+31)/32 + 1]
  uint16_t* lutS = reinterpret_cast<uint16_t*>(smem + LO::offTables + LO::wbits_bytes(n_lut));
  int16_t* win_lo = reinterpret_cast<int16_t*>(smem + LO::offTables + LO::wbits_bytes(n_lut) + ((2 * n_lut + 15) & ~15));
  int16_t* win_hi = win_lo + n_kt;
  uint32_t* kbits = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(win_lo) + ((4 * n_kt + 15) & ~15));
  const FTables tb{wbits, lutS, win_lo, win_hi, kbits};

  // ------------------------------------------------------------------ setup
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bars->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      ptx::mbar_init(&bars->kv_full[s], 1);
      ptx::mbar_init(&bars->kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&bars->s_full[s], 1);
      // one elected lane per warp arrives (after __syncwarp): kSoftmaxWarps softmax warps, 4 converter warps
      ptx::mbar_init(&bars->s_free[s], kSoftmaxWarps);
      ptx::mbar_init(&bars->p_full[s], kSoftmaxWarps);
      ptx::mbar_init(&bars->c2p_ready[s], 4);
      ptx::mbar_init(&bars->ring_release[s], kSoftmaxWarps);
    }
    ptx::mbar_init(&bars->o_ready, 1);
    ptx::mbar_init(&bars->pk_full, 1);
    ptx::mbar_init(&bars->pk_empty, 1);
    ptx::mbar_init(&bars->pq_full, 1);
    ptx::mbar_init(&bars->pq_empty, 1);
    ptx::mbar_init(&bars->cnew_full, 1);
    ptx::mbar_init(&bars->cnew_free, 4);
    ptx::mbar_init(&bars->pt_full, 1);
    ptx::mbar_init(&bars->pt_free, 4);
    ptx::mbar_init(&bars->pt_ready, 4);
    ptx::mbar_init(&bars->pt_release, kSoftmaxWarps);
    for (int q = 0; q < 4; ++q) ptx::mbar_init(&bars->pair[q], kParts);
    bars->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kTmaWarp && lane == 0) {
    ptx::prefetch_tensormap(&tmap_q);
    ptx::prefetch_tensormap(&tmap_k);
    ptx::prefetch_tensormap(&tmap_v);
    ptx::prefetch_tensormap(&tmap_pk);
    ptx::prefetch_tensormap(&tmap_pq);
    ptx::prefetch_tensormap(&tmap_pq64);
  }
  if (warp == kMmaWarp) {
    ptx::tmem_alloc(&bars->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  TRACE(97);
  // ---- tables.  All global reads are issued first; two block-wide syncs follow.
  // slot table, edge-replicated so that out-of-range (i, j) pairs resolve inside the tile's window
  for (int e = threadIdx.x; e < n_lut; e += kThreads) {
    int src = e - LUT_LO_PAD;
    src = src < 0 ? 0 : (src > 2 * L - 2 ? 2 * L - 2 : src);
    lutS[e] = (uint16_t)p.lut[src];
  }
  // key keep-mask as bits: word w covers keys [32w, 32w+32); keys >= L are 0
  for (int w = warp; w < 2 * n_kt; w += kThreads / 32) {
    const int j = w * 32 + lane;
    const bool keep = j < L && mask_keep(p.mask, p.mask_elem_size, (long long)b * L + j);
    const uint32_t bits = __ballot_sync(0xffffffffu, keep);
    if (lane == 0) kbits[w] = bits;
  }
  // Key tiles before the first and after the last kept key contribute nothing to a kept query row
  // (their probabilities are exactly zero) and are skipped; a padded query row attends uniformly to all
  // L keys, so a query tile that contains one walks every key tile.
  const bool my_row_in_range = threadIdx.x < BM && i0 + (int)threadIdx.x < L;
  const bool my_row_kept = my_row_in_range && mask_keep(p.mask, p.mask_elem_size, (long long)b * L + i0 + threadIdx.x);
  ptx::tc_fence_before();
  TRACE(96);
  const bool any_padded_row = __syncthreads_or(my_row_in_range && !my_row_kept) != 0;
  TRACE(95);
  // step bit of entry e: slot(e) - slot(e-1) (0 or 1).  One ballot per 32 entries stores them in entry order;
  // a softmax thread later takes the 32-bit window that ends at its entry (see step_mask_at).
  {
    const int n_words = (n_lut + 31) / 32;
    for (int k = warp; k < n_words; k += kThreads / 32) {
      const int e = k * 32 + lane;
      const bool step = e >= 1 && e < n_lut && lutS[e] != lutS[e - 1];
      const uint32_t bits = __ballot_sync(0xffffffffu, step);
      if (lane == 0) wbits[k + 1] = bits;
    }
    if (threadIdx.x == 0) wbits[0] = 0;
  }
  for (int t = threadIdx.x; t < n_kt; t += kThreads) {
    int a = i0 - (t * BN + BN - 1) + (L - 1), z = i0 + (BM - 1) - t * BN + (L - 1);
    a = a < 0 ? 0 : (a > 2 * L - 2 ? 2 * L - 2 : a);
    z = z < 0 ? 0 : (z > 2 * L - 2 ? 2 * L - 2 : z);
    win_lo[t] = (int16_t)lutS[a + LUT_LO_PAD];
    win_hi[t] = (int16_t)lutS[z + LUT_LO_PAD];
  }
  const bool any_kept_row = __syncthreads_or(my_row_kept) != 0;
  ptx::tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  int t_begin = 0, t_end = n_kt;
  if (!any_padded_row) {
    while (t_begin < n_kt - 1 && (kbits[2 * t_begin] | kbits[2 * t_begin + 1]) == 0) ++t_begin;
    while (t_end > t_begin + 1 && (kbits[2 * t_end - 2] | kbits[2 * t_end - 1]) == 0) --t_end;
  }
  const int n_tiles = t_end - t_begin;
  TRACE(98);

  if (!any_kept_row) {
    // Every query row of this tile is padding: each of them attends uniformly to all L keys, so every
    // output row is the column mean of V.  No score, no softmax: one pass over V by the whole CTA.
    float* part = reinterpret_cast<float*>(smem + LO::offRing);   // [groups][D] partial sums, then [D] means
    constexpr int kGroups = kThreads / D;
    const int col = threadIdx.x % D, grp = threadIdx.x / D;
    const T* V = reinterpret_cast<const T*>(p.v) + (long long)bh * L * D;
    float sum = 0.0f;
    if (grp < kGroups)
      for (int row = grp; row < L; row += kGroups) sum += Elem<T>::to_f(V[(long long)row * D + col]);
    if (grp < kGroups) part[grp * D + col] = sum;
    __syncthreads();
    T* mean = reinterpret_cast<T*>(part + kGroups * D);
    if (threadIdx.x < D) {
      float total = 0.0f;
      for (int gidx = 0; gidx < kGroups; ++gidx) total += part[gidx * D + threadIdx.x];
      mean[threadIdx.x] = Elem<T>::from_f(total / (float)L);
    }
    __syncthreads();
    const int rows = L - i0 < BM ? L - i0 : BM;
    constexpr int kVec = D / 8;  // 16-byte chunks per output row
    T* out = reinterpret_cast<T*>(p.out) + ((long long)b * L + i0) * ((long long)H * D) + (long long)h * D;
    for (int e = threadIdx.x; e < rows * kVec; e += kThreads) {
      const int rr = e / kVec, v = e - rr * kVec;
      *reinterpret_cast<uint4*>(out + (long long)rr * H * D + v * 8) = *reinterpret_cast<const uint4*>(mean + v * 8);
    }
  } else

  if (warp == kTmaWarp) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      ptx::mbar_arrive_expect_tx(&bars->q_full, (uint32_t)LO::kQ);
      ptx::tma_load_3d(smem + LO::offQ, &tmap_q, &bars->q_full, 0, i0, bh);
      uint32_t n_job = 0;
      for (int t = t_begin; t < t_end && ok; ++t) {
        const int u = t - t_begin;  // ordinal of the tile among the processed ones: drives stages and parities
        if (has_c2p) {
          const BlockJobs jobs = c2p_jobs(tb, t, t_begin);
          for (int x = 0; x < jobs.count && ok; ++x, ++n_job) {
            ok = ptx::mbar_wait(&bars->pk_empty, (n_job & 1u) ^ 1u, abort_flag, status_word, 11);
            if (!ok) break;
            ptx::mbar_arrive_expect_tx(&bars->pk_full, (uint32_t)LO::kK);
            ptx::tma_load_3d(smem + LO::offPK, &tmap_pk, &bars->pk_full, 0, (jobs.first - x) * 64, h);
          }
          if (!ok) break;
        }
        if (has_p2c) {
          ok = ptx::mbar_wait(&bars->pq_empty, ((uint32_t)u & 1u) ^ 1u, abort_flag, status_word, 12);
          if (!ok) break;
          TRACE(32);
          const int lo = win_lo[t];
          const bool two = win_hi[t] - lo >= 128;
          ptx::mbar_arrive_expect_tx(&bars->pq_full, (uint32_t)(two ? LO::kQ + LO::kQ / 2 : LO::kQ));
          ptx::tma_load_3d(smem + LO::offPQ, &tmap_pq, &bars->pq_full, 0, lo, h);
          if (two) ptx::tma_load_3d(smem + LO::offPQ + LO::kQ, &tmap_pq64, &bars->pq_full, 0, lo + 128, h);
        }
        const int s = u % KV_STAGES;
        ok = ptx::mbar_wait(&bars->kv_empty[s], ((uint32_t)(u / KV_STAGES) & 1u) ^ 1u, abort_flag, status_word, 1);
        if (!ok) break;
        TRACE(33);
        ptx::mbar_arrive_expect_tx(&bars->kv_full[s], (uint32_t)(2 * LO::kK));
        unsigned char* kv = smem + LO::offKV + s * 2 * LO::kK;
        ptx::tma_load_3d(kv, &tmap_k, &bars->kv_full[s], 0, t * BN, bh);
        ptx::tma_load_3d(kv + LO::kK, &tmap_v, &bars->kv_full[s], 0, t * BN, bh);
      }
    }
  } else if (warp == kMmaWarp) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr int is_bf16 = __is_same(T, __nv_bfloat16) ? 1 : 0;
      constexpr uint32_t idesc_64 = ptx::make_idesc_f16(is_bf16, BM, BN, 0, 0);  // 128 x 64, both K-major
      constexpr uint32_t idesc_pv = ptx::make_idesc_f16(is_bf16, BM, D, 0, 1);   // V is MN-major
      constexpr uint32_t mode = ptx::swizzle_mode_for_row_bytes(LO::kRowBytes);
      constexpr uint32_t sbo = 8 * LO::kRowBytes;
      constexpr int kSteps = LO::kRowBytes / 32;  // K=16 steps over d
      const uint32_t q_addr = ptx::smem_u32(smem + LO::offQ);
      const uint32_t pk_addr = ptx::smem_u32(smem + LO::offPK);
      const uint32_t pq_addr = ptx::smem_u32(smem + LO::offPQ);
      uint32_t n_job = 0;
      bool ok = ptx::mbar_wait(&bars->q_full, 0, abort_flag, status_word, 2);

      // D[128 x 64] = A[128 x d] * B[64 x d]^T, both operands K-major tiles in shared memory
      auto mma_128x64 = [&](uint32_t d_col, uint32_t a_addr, uint32_t b_addr) {
#pragma unroll
        for (int k = 0; k < kSteps; ++k) {
          const uint64_t adesc = ptx::make_smem_desc(a_addr + k * 32, 16, sbo, mode);
          const uint64_t bdesc = ptx::make_smem_desc(b_addr + k * 32, 16, sbo, mode);
          ptx::umma_ss_f16(tmem_base + d_col, adesc, bdesc, idesc_64, k != 0 ? 1u : 0u);
        }
      };

      // everything tile t needs before its softmax: new C2P blocks, PT, S
      auto issue_front = [&](int t) -> bool {
        if (has_c2p) {
          const BlockJobs jobs = c2p_jobs(tb, t, t_begin);
          for (int x = 0; x < jobs.count; ++x, ++n_job) {
            if (!ptx::mbar_wait(&bars->pk_full, n_job & 1u, abort_flag, status_word, 13)) return false;
            if (!ptx::mbar_wait(&bars->cnew_free, (n_job & 1u) ^ 1u, abort_flag, status_word, 14)) return false;
            TRACE(22);
            ptx::tc_fence_after();
            mma_128x64(COL_CNEW, q_addr, pk_addr);
            ptx::umma_commit(&bars->pk_empty);
            ptx::umma_commit(&bars->cnew_full);
          }
        }
        const int u = t - t_begin;
        const int s = u % KV_STAGES, sb = u & 1;
        if (!ptx::mbar_wait(&bars->kv_full[s], (uint32_t)(u / KV_STAGES) & 1u, abort_flag, status_word, 3)) return false;
        TRACE(23);
        const uint32_t k_addr = ptx::smem_u32(smem + LO::offKV + s * 2 * LO::kK);
        if (has_p2c) {
          if (!ptx::mbar_wait(&bars->pq_full, (uint32_t)u & 1u, abort_flag, status_word, 15)) return false;
          if (!ptx::mbar_wait(&bars->pt_free, ((uint32_t)u & 1u) ^ 1u, abort_flag, status_word, 16)) return false;
          TRACE(25);
          ptx::tc_fence_after();
          mma_128x64(COL_PT, pq_addr, k_addr);
          if (win_hi[t] - win_lo[t] >= 128) mma_128x64(COL_PT + BN, pq_addr + LO::kQ, k_addr);
          ptx::umma_commit(&bars->pq_empty);
          ptx::umma_commit(&bars->pt_full);
        }
        if (!ptx::mbar_wait(&bars->s_free[sb], ((uint32_t)(u >> 1) & 1u) ^ 1u, abort_flag, status_word, 4)) return false;
        TRACE(26);
        ptx::tc_fence_after();
        mma_128x64(COL_S + sb * BN, q_addr, k_addr);
        ptx::umma_commit(&bars->s_full[sb]);
        return true;
      };

      if (ok) ok = issue_front(t_begin);
      for (int t = t_begin; t < t_end && ok; ++t) {
        if (t + 1 < t_end) ok = issue_front(t + 1);
        if (!ok) break;
        const int u = t - t_begin;
        const int s = u % KV_STAGES, sb = u & 1;
        ok = ptx::mbar_wait(&bars->p_full[sb], (uint32_t)(u >> 1) & 1u, abort_flag, status_word, 5);
        if (!ok) break;
        TRACE(27);
        ptx::tc_fence_after();
        const uint32_t v_addr = ptx::smem_u32(smem + LO::offKV + s * 2 * LO::kK + LO::kK);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint64_t bdesc = ptx::make_smem_desc(v_addr + kk * 16 * LO::kRowBytes, LO::kK, sbo, mode);
          ptx::umma_ts_f16(tmem_base + COL_O, tmem_base + COL_P + sb * (BN / 2) + kk * 8, bdesc, idesc_pv,
                           (u | kk) != 0 ? 1u : 0u);
        }
        ptx::umma_commit(&bars->kv_empty[s]);
        ptx::umma_commit(&bars->o_ready);
        TRACE(28);
      }
    }
  } else if (warp >= kConvWarp0) {
    // -------------------------------------------------------------- converters
    // Thread (quarter q = warp & 3, lane) owns TMEM lane 32q + lane: a query row for C2P blocks,
    // a slot (relative to the window start) for PT tiles.
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    unsigned char* ring_row = smem + LO::offRing + row * (RING_PITCH_H * 2);
    unsigned char* pt_base = smem + LO::offPT;
    uint32_t n_job = 0;
    bool ok = true;

    // 64 fp32 columns at t_src -> 64 16-bit values at dst (4-byte aligned), rounded like a GEMM epilogue
    // (all lanes must execute the TMEM load; `store` and `mirror` only gate the shared-memory writes)
    auto convert_64 = [&](uint32_t t_src, unsigned char* dst, int mirror = 0, bool store = true) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t raw[32];
        ptx::tmem_ld32(t_src + half * 32, raw);
        ptx::tmem_wait_ld();
        if (store) {
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            const uint32_t w = Pack2<T>::pack(__uint_as_float(raw[x]), __uint_as_float(raw[x + 1]));
            *reinterpret_cast<uint32_t*>(dst + half * 64 + x * 2) = w;
            if (mirror) *reinterpret_cast<uint32_t*>(dst + mirror + half * 64 + x * 2) = w;
          }
        }
      }
    };

    for (int t = t_begin; t < t_end && ok; ++t) {
      const int u = t - t_begin;
      if (has_c2p) {
        const BlockJobs jobs = c2p_jobs(tb, t, t_begin);
        // The ring position a new block overwrites was last needed by tile t-2.  The wait is taken even
        // when tile t brings no block: it keeps this role at most two tiles ahead of the softmax, which the
        // two-phase c2p_ready barriers rely on.
        ok = ptx::mbar_wait(&bars->ring_release[u & 1], ((uint32_t)(u >> 1) & 1u) ^ 1u, abort_flag, status_word, 17);
        if (!ok) break;
        TRACE(11);
        for (int x = 0; x < jobs.count && ok; ++x, ++n_job) {
          ok = ptx::mbar_wait(&bars->cnew_full, n_job & 1u, abort_flag, status_word, 18);
          if (!ok) break;
          TRACE(12);
          ptx::tc_fence_after();
          const int blk = jobs.first - x;
          // the block at ring position 0 is mirrored at position 5 so that a row's run never wraps
          convert_64(tmem_base + lane_base + COL_CNEW, ring_row + (blk % RING_BLOCKS) * 128,
                     blk % RING_BLOCKS == 0 ? RING_SPAN * 2 : 0);
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&bars->cnew_free);
          TRACE(13);
        }
        if (!ok) break;
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bars->c2p_ready[u & 1]);
      }
      if (has_p2c) {
        ok = ptx::mbar_wait(&bars->pt_full, (uint32_t)u & 1u, abort_flag, status_word, 19);
        if (!ok) break;
        TRACE(14);
        ptx::tc_fence_after();
        // the staging tile is single-buffered: tile t-1 must have been gathered
        ok = ptx::mbar_wait(&bars->pt_release, ((uint32_t)u & 1u) ^ 1u, abort_flag, status_word, 20);
        if (!ok) break;
        TRACE(15);
        convert_64(tmem_base + lane_base + COL_PT, pt_base + row * (PT_PITCH_H * 2));
        if (win_hi[t] - win_lo[t] >= 128)  // slots lo+128 .. lo+191 sit in lanes 0..63 of the second accumulator
          convert_64(tmem_base + lane_base + COL_PT + BN, pt_base + (128 + (row & 63)) * (PT_PITCH_H * 2), 0, row < 64);
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          ptx::mbar_arrive(&bars->pt_free);
          ptx::mbar_arrive(&bars->pt_ready);
        }
        TRACE(16);
      }
    }
  } else {
    // ----------------------------------------------------------------- softmax
    constexpr int W = BN / kParts;                 // keys per thread and tile
    const int q4 = warp & 3, part = warp >> 2;     // lane quarter, which part of the keys / output columns
    const int r = q4 * 32 + lane;
    const int i = i0 + r;
    const bool row_ok = i < L;
    const bool q_keep = row_ok && mask_keep(p.mask, p.mask_elem_size, (long long)b * L + i);
    const float cscale = p.scale * 1.4426950408889634f;
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    const uint32_t t_o_part = tmem_base + lane_base + COL_O + part * (D / kParts);
    const uint32_t ring_addr = ptx::smem_u32(smem + LO::offRing) + (uint32_t)(r * RING_PITCH_H * 2);
    const uint32_t pt_addr = ptx::smem_u32(smem + LO::offPT);
    const attn::RowExchange xc{reinterpret_cast<float*>(smem + LO::offXchg), &bars->pair[q4]};
    attn::RowState st;
    bool ok = true;

    for (int t = t_begin; t < t_end && ok; ++t) {
      const int u = t - t_begin;
      const int sb = u & 1, j0 = t * BN + part * W;  // first key of this thread's part
      ok = ptx::mbar_wait(&bars->s_full[sb], (uint32_t)(u >> 1) & 1u, abort_flag, status_word, 7);
      if (!ok) break;
      TRACE(1);
      ptx::tc_fence_after();
      float s[W];
      {
        uint32_t raw[W];
        attn::tmem_ld_n(tmem_base + lane_base + COL_S + sb * BN + part * W, raw);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int x = 0; x < W; ++x) s[x] = __uint_as_float(raw[x]);
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bars->s_free[sb]);
      TRACE(2);

      // Slots of this thread's W pairs: s_0 = slot(i, j0) and s_{x+1} = s_x - step bit x (steps are 0 or 1), so the
      // two gathers walk their row with a running address instead of one table lookup per element.
      const int e0 = LUT_LO_PAD + i - j0 + (L - 1);  // table index of pair (i, j0); pair (i, j0+x) is e0 - x
      // bit x of steps = slot(e0 - x) - slot(e0 - x - 1): the bit-reversed 32-entry window ending at e0
      const uint32_t steps = __brev(__funnelshift_rc(wbits[e0 >> 5], wbits[(e0 >> 5) + 1], (e0 & 31) + 1)) & 0x7fffffffu;
      const int s0 = lutS[e0];
      if (has_c2p) {
        ok = ptx::mbar_wait(&bars->c2p_ready[sb], (uint32_t)(u >> 1) & 1u, abort_flag, status_word, 8);
        if (!ok) break;
      }
      if (has_p2c) {
        ok = ptx::mbar_wait(&bars->pt_ready, (uint32_t)u & 1u, abort_flag, status_word, 21);
        if (!ok) break;
      }
      TRACE(3);
      {
        // C2P: ring position of slot s0; the mirror makes pos-(W-1) .. pos contiguous.
        int pos = s0 % RING_SPAN;
        if (pos < W - 1) pos += RING_SPAN;
        uint32_t caddr = ring_addr + 2u * (uint32_t)pos;
        // P2C: PT[slot - lo][key]; the row moves down one pitch whenever the slot steps, the column follows x.
        uint32_t paddr = pt_addr + (uint32_t)((s0 - (int)win_lo[t]) * (PT_PITCH_H * 2) + part * W * 2);
        uint16_t cval[W], pval[W];
#pragma unroll
        for (int x = 0; x < W; ++x) {
          if (has_c2p) cval[x] = ptx::lds_u16(caddr);
          if (has_p2c) pval[x] = ptx::lds_u16(paddr + 2u * x);
          if (steps & (1u << x)) {
            caddr -= 2u;
            paddr -= (uint32_t)(PT_PITCH_H * 2);
          }
        }
        if (has_c2p) {
#pragma unroll
          for (int x = 0; x < W; ++x) s[x] = Pack2<T>::add(s[x], cval[x]);
        }
        if (has_p2c) {
#pragma unroll
          for (int x = 0; x < W; ++x) s[x] = Pack2<T>::add(s[x], pval[x]);
        }
        __syncwarp();
        if (lane == 0) {
          if (has_c2p) ptx::mbar_arrive(&bars->ring_release[sb]);
          if (has_p2c) ptx::mbar_arrive(&bars->pt_release);
        }
      }
      TRACE(6);

      const uint32_t kb = kbits[(j0 >> 5)] >> (j0 & 31);
      ok = attn::softmax_part_tail<T, D, kParts>(s, st, kb, L - j0, q_keep, cscale, u, part, r, xc, t_o_part,
                                                 tmem_base + lane_base + COL_P + sb * (BN / 2) + part * (W / 2),
                                                 &bars->o_ready, &bars->p_full[sb], abort_flag, status_word TRACE_ARG);
      TRACE(7);
    }
    T* out = reinterpret_cast<T*>(p.out) + ((long long)b * L + (row_ok ? i : 0)) * ((long long)H * D) +
             (long long)h * D + part * (D / kParts);
    attn::softmax_part_store<T, D, kParts>(st, ok, row_ok, n_tiles, part, r, xc, t_o_part, out, &bars->o_ready,
                                           abort_flag, status_word);
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) ptx::tmem_dealloc(tmem_base, kTmemCols);
}

template <typename T, int D>
int launch_fused_typed(const DflAttnTablesParams& p, cudaStream_t stream) {
  using LO = FLayout<D>;
  const int L = p.seq_len, BH = p.batch * p.heads, A = p.n_active;
  const uint64_t row = (uint64_t)D * sizeof(T), seq = (uint64_t)L * row, table = (uint64_t)A * row;
  CUtensorMap tq, tk, tv, tpk, tpq, tpq64;
  int rc = encode_tensor_map_3d(&tq, p.q, D, L, BH, row, seq, D, BM, LO::kRowBytes);
  if (rc == DFL_OK) rc = encode_tensor_map_3d(&tk, p.k, D, L, BH, row, seq, D, BN, LO::kRowBytes);
  if (rc == DFL_OK) rc = encode_tensor_map_3d(&tv, p.v, D, L, BH, row, seq, D, BN, LO::kRowBytes);
  // a disabled term reuses the other table's map; it is never dereferenced
  const void* pk = p.pos_key ? p.pos_key : p.pos_query;
  const void* pq = p.pos_query ? p.pos_query : p.pos_key;
  if (rc == DFL_OK) rc = encode_tensor_map_3d(&tpk, pk, D, A, p.heads, row, table, D, BN, LO::kRowBytes);
  if (rc == DFL_OK) rc = encode_tensor_map_3d(&tpq, pq, D, A, p.heads, row, table, D, BM, LO::kRowBytes);
  if (rc == DFL_OK) rc = encode_tensor_map_3d(&tpq64, pq, D, A, p.heads, row, table, D, BM / 2, LO::kRowBytes);
  if (rc != DFL_OK) return rc;

  constexpr int kMaxSmem = 232448;
  const int smem = LO::total(L);
  if (smem > kMaxSmem) return fail(DFL_ERR_TOO_LARGE, "seq_len %d needs %d bytes of shared memory", L, smem);
  // 512 TMEM columns per CTA: exactly one CTA may be resident per SM
  const int smem_request = smem < kMaxSmem / 2 + 1024 ? kMaxSmem / 2 + 1024 : smem;

  auto kernel = attention_fused_kernel<T, D>;
  static int configured_smem = 0;
  if (smem_request > configured_smem) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_request);
    if (e != cudaSuccess) return fail(DFL_ERR_LAUNCH, "attention_fused smem opt-in: %s", cudaGetErrorString(e));
    configured_smem = smem_request;
  }
  int* status_word = p.status;
  if (!status_word) {
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&status_word), g_attn_fused_status);
    if (e != cudaSuccess) return fail(DFL_ERR_LAUNCH, "status word: %s", cudaGetErrorString(e));
  }
  dim3 grid((L + BM - 1) / BM, BH);
  if (grid.y > 65535) return fail(DFL_ERR_TOO_LARGE, "batch*heads > 65535");
  kernel<<<grid, kThreads, smem_request, stream>>>(tq, tk, tv, tpk, tpq, tpq64, p, status_word);
  return check_launch("attention_fused_kernel");
}

}  // namespace

bool attention_fused_supported(const DflAttnTablesParams& p) {
  return p.dtype != DFL_F32 && (p.head_dim == 32 || p.head_dim == 64) && (p.pos_key || p.pos_query) &&
         p.n_active >= 1 && p.n_active <= 4096 && p.seq_len <= 1024;
}

int launch_attention_fused(const DflAttnTablesParams& p, cudaStream_t stream) {
  if (!attention_fused_supported(p)) return fail(DFL_ERR_UNSUPPORTED, "configuration not covered by the fused-score kernel");
  if (p.dtype == DFL_F16)
    return p.head_dim == 64 ? launch_fused_typed<__half, 64>(p, stream) : launch_fused_typed<__half, 32>(p, stream);
  return p.head_dim == 64 ? launch_fused_typed<__nv_bfloat16, 64>(p, stream)
                          : launch_fused_typed<__nv_bfloat16, 32>(p, stream);
}

}  // namespace dfl

#ifdef DFL_TRACE
extern "C" int dfl_debug_read_trace(long long* host_buf, int clear) {
  cudaDeviceSynchronize();
  cudaError_t e = cudaMemcpyFromSymbol(host_buf, dfl::g_trace, sizeof(long long) * 16 * 512);
  if (clear) {
    static long long zeros[16 * 512] = {0};
    cudaMemcpyToSymbol(dfl::g_trace, zeros, sizeof(zeros));
  }
  return (int)e;
}
#endif
