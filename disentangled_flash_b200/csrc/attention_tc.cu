// tcgen05 fused disentangled attention forward for FP16/BF16, head dims 32/64/128.
//
// Replaces the reference's Triton kernel _deberta_attention_forward_kernel and
// its launcher (src/disentangled_flash/kernel.py:137-429):
//   S[i,j] = q_i.k_j + c2p[i, lut[i-j+L-1]] + p2c[j, lut[i-j+L-1]]
//   P = softmax_j(S * scale) under the factorised padding mask, O = P V,
//   out[b, i, h*d:(h+1)*d] = O.  [B,H,L,L] never exists in memory.
//
// One CTA owns 128 query rows of one (batch, head) and walks the keys in tiles
// of 64.  Eight warps, four roles:
//   warps 0-3  softmax: one thread per query row.  S is read from TMEM with
//              tcgen05.ld, the two relative scores are gathered from shared
//              memory, the row is scaled, masked and exponentiated (base 2,
//              online max/sum), P is rounded to the input type and written back
//              to TMEM, the O accumulator in TMEM is rescaled when the row
//              maximum moved, and at the end O/rowsum is stored.
//   warp 4     TMA producer: Q once, then K and V tiles into a 2-stage ring
//              (128-byte swizzle; 64-byte for d=32).
//   warp 5     MMA issuer: S = Q K^T (operands in shared memory, K-major) and
//              O += P V (P from TMEM, V from shared memory, MN-major), both
//              tcgen05.mma with fp32 accumulators in TMEM; also owns the TMEM
//              allocation.
//   warps 6-7  relative-score stagers: per key tile, warp 6 copies for every
//              query row the <=72 contiguous c2p slots that row can touch in
//              this tile, warp 7 copies the p2c slot window of the 64 keys, with
//              16-byte cp.async that signal an mbarrier on completion.
// The slot table lut (delta -> local slot) is monotone with steps of 0 or 1, so
// everything a tile needs from a c2p/p2c row is one contiguous window.
#include "attention_tc_common.cuh"

namespace dfl {

__device__ int g_attn_status = 0;

namespace {

using attn::BM;  // 128 query rows per CTA
using attn::BN;  // 64 keys per tile
using attn::Pack2;
constexpr int kThreads = 256;
constexpr int KV_STAGES = 2;
constexpr int kMaxSmem = 232448;  // 227 KB opt-in limit per block
constexpr int C_CHUNKS = 9;      // 16-byte chunks per staged c2p row: (BN-1+7)/8 + 1
constexpr int P_CHUNKS = 25;     // 16-byte chunks per staged p2c row: (BM+BN-2+7)/8 + 1
constexpr int C_PITCH = C_CHUNKS * 16;   // bytes
constexpr int P_PITCH = P_CHUNKS * 16;   // bytes
constexpr int LUT_LO_PAD = BN;   // replicated entries below index 0
constexpr int LUT_HI_PAD = BM;   // replicated entries above index 2L-2

// TMEM column plan
constexpr int COL_S = 0;             // two S buffers of BN fp32 columns
constexpr int COL_P = 2 * BN;        // two P buffers of BN/2 columns (packed 16-bit pairs)
constexpr int COL_O = 2 * BN + BN;   // D fp32 columns

// NB = relative-score stages: 2 when the shared memory of the sequence length leaves room (the stagers then fill
// the next tile's windows while the softmax warps gather from the current one), else 1.
template <int D, int NB_>
struct Layout {
  static constexpr int kRowBytes = D >= 64 ? 128 : D * 2;      // swizzle span = bytes of one smem row
  static constexpr int kSub = D * 2 / kRowBytes;               // 64-column sub-tiles per row (2 for d=128)
  static constexpr int kQSub = BM * kRowBytes;                  // bytes of one Q sub-tile
  static constexpr int kKSub = BN * kRowBytes;                  // bytes of one K (or V) sub-tile
  static constexpr int kQ = kSub * kQSub;
  static constexpr int kKV = 2 * kSub * kKSub;                  // K then V
  static constexpr int kBias = BM * C_PITCH + BN * P_PITCH;    // one relative-score stage
  static constexpr int kTmemCols = (COL_O + D) <= 256 ? 256 : 512;
  static constexpr int kBiasStages = NB_;
  static constexpr int offQ = 0;
  static constexpr int offKV = offQ + kQ;
  static constexpr int offBias = offKV + KV_STAGES * kKV;
  static constexpr int offBar = offBias + kBiasStages * kBias;  // 8-byte aligned (all sizes are multiples of 16)
  static constexpr int kBarBytes = 256;
  static constexpr int offLut = offBar + kBarBytes;
  static int total(int L) { return offLut + (2 * L - 1 + LUT_LO_PAD + LUT_HI_PAD) * 2 + ((L + 31) / 32 + 4) * 4 + 1024; }
};

struct Barriers {
  uint64_t q_full;
  uint64_t kv_full[KV_STAGES];
  uint64_t kv_empty[KV_STAGES];
  uint64_t s_full[2];
  uint64_t s_free[2];
  uint64_t p_full[2];
  uint64_t o_ready;
  uint64_t bias_full[2];
  uint64_t bias_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(Barriers) <= 256, "barrier block too large");

struct RoleCtx {
  unsigned char* smem;
  Barriers* bars;
  const uint16_t* lut_s;
  const uint32_t* kbits;
  uint32_t tmem_base;
  int* status_word;
  int L, H, b, h, i0, n_kt;
  bool has_c2p, has_p2c;
};

// Softmax role: executed by warps 0-3, thread (warp*32+lane) owns query row i0 + warp*32 + lane,
// which is TMEM lane warp*32+lane of every accumulator.
template <typename T, int D, int NB>
__device__ __forceinline__ void softmax_role(const RoleCtx& c, const DflAttnParams& p, int warp, int lane) {
  using LO = Layout<D, NB>;
  Barriers* bars = c.bars;
  volatile int* abort_flag = &bars->abort_flag;
  const int L = c.L;
  const int r = warp * 32 + lane;
  const int i = c.i0 + r;
  const bool row_ok = i < L;
  const bool q_keep = row_ok && mask_keep(p.mask, p.mask_elem_size, (long long)c.b * L + i);
  const bool has_pos = c.has_c2p || c.has_p2c;
  const float cscale = p.scale * 1.4426950408889634f;  // scores are exponentiated in base 2
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  const uint32_t t_o = c.tmem_base + lane_base + COL_O;

  attn::RowState st;
  bool ok = true;

  for (int kt = 0; kt < c.n_kt && ok; ++kt) {
    const int sb = kt & 1, j0 = kt * BN;
    const uint32_t use = (uint32_t)(kt >> 1) & 1u;
    ok = ptx::mbar_wait(&bars->s_full[sb], use, abort_flag, c.status_word, 7);
    if (!ok) break;
    ptx::tc_fence_after();
    float s[BN];
    attn::load_scores(c.tmem_base + lane_base + COL_S + sb * BN, s);
    ptx::tc_fence_before();
    ptx::mbar_arrive(&bars->s_free[sb]);  // S buffer may be overwritten by the tile after next

    if (has_pos) {
      const int bs = kt % NB;
      ok = ptx::mbar_wait(&bars->bias_full[bs], (uint32_t)(kt / NB) & 1u, abort_flag, c.status_word, 8);
      if (!ok) break;
      const unsigned char* stage = c.smem + LO::offBias + bs * LO::kBias;
      // lut_i[-jj] is the byte offset (2*slot) of pair (i, j0+jj)
      const uint16_t* lut_i = c.lut_s + (LUT_LO_PAD + i - j0 + (L - 1));
      const uint32_t c_lo = lut_i[-(BN - 1)] & ~15u;
      const unsigned char* c_row = stage + r * C_PITCH - c_lo;
      const uint32_t p_lo = c.lut_s[LUT_LO_PAD + c.i0 - j0 + (L - 1) - (BN - 1)] & ~15u;
      const unsigned char* p_row = stage + BM * C_PITCH - p_lo;
      // A slot table of the builder's shape (non-decreasing, steps of 0 or 1) keeps every offset inside the staged
      // window; for any other table the offset is clamped into the window, so that a wrong table gives wrong
      // scores but never a read outside the row's stage.
      auto elem = [](const unsigned char* base, uint32_t lo, uint32_t off, uint32_t pitch) {
        const uint32_t rel = min(off - lo, pitch - 2u);   // off < lo wraps to a huge value and is clamped as well
        return *reinterpret_cast<const uint16_t*>(base + lo + rel);
      };
      if (c.has_c2p && c.has_p2c) {
#pragma unroll
        for (int jj = 0; jj < BN; ++jj) {
          const uint32_t off = lut_i[-jj];
          s[jj] = Pack2<T>::add(Pack2<T>::add(s[jj], elem(c_row, c_lo, off, C_PITCH)),
                                elem(p_row + jj * P_PITCH, p_lo, off, P_PITCH));
        }
      } else if (c.has_c2p) {
#pragma unroll
        for (int jj = 0; jj < BN; ++jj) s[jj] = Pack2<T>::add(s[jj], elem(c_row, c_lo, lut_i[-jj], C_PITCH));
      } else {
#pragma unroll
        for (int jj = 0; jj < BN; ++jj) s[jj] = Pack2<T>::add(s[jj], elem(p_row + jj * P_PITCH, p_lo, lut_i[-jj], P_PITCH));
      }
      ptx::mbar_arrive(&bars->bias_empty[bs]);
    }

    ok = attn::softmax_tile_tail<T, D>(s, st, c.kbits[2 * kt], c.kbits[2 * kt + 1], L - j0, q_keep, cscale, kt, t_o,
                                       c.tmem_base + lane_base + COL_P + sb * (BN / 2), &bars->o_ready,
                                       &bars->p_full[sb], abort_flag, c.status_word);
  }

  T* out = reinterpret_cast<T*>(p.out) + ((long long)c.b * L + (row_ok ? i : 0)) * ((long long)c.H * D) + (long long)c.h * D;
  attn::softmax_store_row<T, D>(st, ok, row_ok, c.n_kt, t_o, out, &bars->o_ready, abort_flag, c.status_word);
}

template <typename T, int D, int NB>
__global__ void __launch_bounds__(kThreads, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const DflAttnParams p, int* status_word) {
  using LO = Layout<D, NB>;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  Barriers* bars = reinterpret_cast<Barriers*>(smem + LO::offBar);
  uint16_t* lut_s = reinterpret_cast<uint16_t*>(smem + LO::offLut);  // byte offsets (2*slot), edge-replicated
  volatile int* abort_flag = &bars->abort_flag;

  const int L = p.seq_len, H = p.heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
  const int i0 = blockIdx.x * BM;
  const int n_kt = (L + BN - 1) / BN;
  const bool has_c2p = p.c2p != nullptr, has_p2c = p.p2c != nullptr;
  const bool has_pos = has_c2p || has_p2c;
  const int n_lut = 2 * L - 1 + LUT_LO_PAD + LUT_HI_PAD;
  uint32_t* kbits = reinterpret_cast<uint32_t*>(smem + LO::offLut + ((n_lut * 2 + 3) & ~3));  // key keep-bits

  // ------------------------------------------------------------------ setup
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bars->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      ptx::mbar_init(&bars->kv_full[s], 1);
      ptx::mbar_init(&bars->kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&bars->s_full[s], 1);
      ptx::mbar_init(&bars->s_free[s], 128);
      ptx::mbar_init(&bars->p_full[s], 128);
      ptx::mbar_init(&bars->bias_full[s], has_pos ? 32 * ((has_c2p ? 1 : 0) + (has_p2c ? 1 : 0)) : 1);
      ptx::mbar_init(&bars->bias_empty[s], 128);
    }
    ptx::mbar_init(&bars->o_ready, 1);
    bars->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 4 && lane == 0) {
    ptx::prefetch_tensormap(&tmap_q);
    ptx::prefetch_tensormap(&tmap_k);
    ptx::prefetch_tensormap(&tmap_v);
  }
  if (warp == 5) {
    ptx::tmem_alloc(&bars->tmem_base, LO::kTmemCols);
    ptx::tmem_relinquish();
  }
  // slot table as byte offsets, replicated at both ends so that out-of-range (i, j) pairs stay in bounds
  if (has_pos) {
    for (int e = threadIdx.x; e < n_lut; e += kThreads) {
      int src = e - LUT_LO_PAD;
      src = src < 0 ? 0 : (src > 2 * L - 2 ? 2 * L - 2 : src);
      // entries outside [0, ld_slots) (a table that did not come from dfl_build_position_lut) are clamped
      int slot = p.lut[src];
      slot = slot < 0 ? 0 : (slot >= p.ld_slots ? p.ld_slots - 1 : slot);
      lut_s[e] = (uint16_t)(2 * slot);
    }
  }
  // key keep-mask as bits: word w covers keys [32w, 32w+32); keys >= L are 0
  for (int w = warp; w < 2 * n_kt; w += kThreads / 32) {
    const int j = w * 32 + lane;
    const bool keep = j < L && mask_keep(p.mask, p.mask_elem_size, (long long)b * L + j);
    const uint32_t bits = __ballot_sync(0xffffffffu, keep);
    if (lane == 0) kbits[w] = bits;
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      ptx::mbar_arrive_expect_tx(&bars->q_full, (uint32_t)LO::kQ);
      for (int c = 0; c < LO::kSub; ++c)
        ptx::tma_load_3d(smem + LO::offQ + c * LO::kQSub, &tmap_q, &bars->q_full, c * 64, i0, bh);
      for (int kt = 0; kt < n_kt; ++kt) {
        const int s = kt % KV_STAGES;
        const uint32_t ph = (uint32_t)(kt / KV_STAGES) & 1u;
        if (!ptx::mbar_wait(&bars->kv_empty[s], ph ^ 1u, abort_flag, status_word, 1)) break;
        ptx::mbar_arrive_expect_tx(&bars->kv_full[s], (uint32_t)LO::kKV);
        unsigned char* kv = smem + LO::offKV + s * LO::kKV;
        for (int c = 0; c < LO::kSub; ++c) {
          ptx::tma_load_3d(kv + c * LO::kKSub, &tmap_k, &bars->kv_full[s], c * 64, kt * BN, bh);
          ptx::tma_load_3d(kv + (LO::kSub + c) * LO::kKSub, &tmap_v, &bars->kv_full[s], c * 64, kt * BN, bh);
        }
      }
    }
  } else if (warp == 5) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr int is_bf16 = __is_same(T, __nv_bfloat16) ? 1 : 0;
      constexpr uint32_t idesc_qk = ptx::make_idesc_f16(is_bf16, BM, BN, 0, 0);
      constexpr uint32_t idesc_pv = ptx::make_idesc_f16(is_bf16, BM, D, 0, 1);  // B (=V) is MN-major
      constexpr uint32_t mode = ptx::swizzle_mode_for_row_bytes(LO::kRowBytes);
      constexpr uint32_t sbo = 8 * LO::kRowBytes;
      constexpr int kPerSub = LO::kRowBytes / 32;  // K=16 MMA steps per 64-column (or 32-column) sub-tile
      const uint32_t q_addr = ptx::smem_u32(smem + LO::offQ);
      bool ok = ptx::mbar_wait(&bars->q_full, 0, abort_flag, status_word, 2);

      auto issue_qk = [&](int kt) -> bool {
        const int s = kt % KV_STAGES, sb = kt & 1;
        if (!ptx::mbar_wait(&bars->kv_full[s], (uint32_t)(kt / KV_STAGES) & 1u, abort_flag, status_word, 3)) return false;
        if (!ptx::mbar_wait(&bars->s_free[sb], ((uint32_t)(kt >> 1) & 1u) ^ 1u, abort_flag, status_word, 4)) return false;
        ptx::tc_fence_after();
        const uint32_t k_addr = ptx::smem_u32(smem + LO::offKV + s * LO::kKV);
#pragma unroll
        for (int c = 0; c < LO::kSub; ++c)
#pragma unroll
          for (int k = 0; k < kPerSub; ++k) {
            const uint64_t adesc = ptx::make_smem_desc(q_addr + c * LO::kQSub + k * 32, 16, sbo, mode);
            const uint64_t bdesc = ptx::make_smem_desc(k_addr + c * LO::kKSub + k * 32, 16, sbo, mode);
            ptx::umma_ss_f16(tmem_base + COL_S + sb * BN, adesc, bdesc, idesc_qk, (c | k) != 0 ? 1u : 0u);
          }
        ptx::umma_commit(&bars->s_full[sb]);
        return true;
      };

      if (ok) ok = issue_qk(0);
      for (int kt = 0; kt < n_kt && ok; ++kt) {
        if (kt + 1 < n_kt) ok = issue_qk(kt + 1);  // next S tile overlaps this tile's softmax
        if (!ok) break;
        const int s = kt % KV_STAGES, sb = kt & 1;
        ok = ptx::mbar_wait(&bars->p_full[sb], (uint32_t)(kt >> 1) & 1u, abort_flag, status_word, 5);
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t v_addr = ptx::smem_u32(smem + LO::offKV + s * LO::kKV + LO::kSub * LO::kKSub);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          // V tile rows are keys: 16 keys = two 8-row swizzle groups; N (=d) chunks of 64 are LO::kKSub apart
          const uint64_t bdesc = ptx::make_smem_desc(v_addr + kk * 16 * LO::kRowBytes, LO::kKSub, sbo, mode);
          ptx::umma_ts_f16(tmem_base + COL_O, tmem_base + COL_P + sb * (BN / 2) + kk * 8, bdesc, idesc_pv,
                           (kt | kk) != 0 ? 1u : 0u);
        }
        ptx::umma_commit(&bars->kv_empty[s]);
        ptx::umma_commit(&bars->o_ready);
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------- relative-score stagers
    const bool mine = warp == 6 ? has_c2p : has_p2c;
    if (mine) {
      const size_t es = sizeof(T);
      const unsigned char* src_base = reinterpret_cast<const unsigned char*>(warp == 6 ? p.c2p : p.p2c) +
                                      (size_t)bh * L * p.ld_slots * es;
      const size_t row_bytes = (size_t)p.ld_slots * es;
      for (int kt = 0; kt < n_kt; ++kt) {
        const int sb = kt % NB, j0 = kt * BN;
        if (!ptx::mbar_wait(&bars->bias_empty[sb], ((uint32_t)(kt / NB) & 1u) ^ 1u, abort_flag, status_word, 6)) break;
        unsigned char* stage = smem + LO::offBias + sb * LO::kBias;
        if (warp == 6) {
          // row r of the tile needs slots lut[i-j] for j in [j0, j0+BN): a window of <= BN slots
          for (int idx = lane; idx < BM * C_CHUNKS; idx += 32) {
            const int r = idx / C_CHUNKS, c = idx - r * C_CHUNKS;
            const int i = i0 + r;
            if (i >= L) continue;
            const int base_idx = LUT_LO_PAD + i - j0 + (L - 1);
            const uint32_t lo = lut_s[base_idx - (BN - 1)] & ~15u;  // byte offset of the aligned window start
            const uint32_t hi = lut_s[base_idx];
            const uint32_t off = lo + 16u * c;
            if (off <= hi) ptx::cp_async_16(stage + r * C_PITCH + 16 * c, src_base + (size_t)i * row_bytes + off);
          }
        } else {
          // all BN keys of the tile share one slot window (the one the whole 128 x 64 tile touches)
          unsigned char* pstage = stage + BM * C_PITCH;
          const int base_idx = LUT_LO_PAD + i0 - j0 + (L - 1);
          const uint32_t lo = lut_s[base_idx - (BN - 1)] & ~15u;
          const uint32_t hi = lut_s[base_idx + (BM - 1)];
          for (int idx = lane; idx < BN * P_CHUNKS; idx += 32) {
            const int r = idx / P_CHUNKS, c = idx - r * P_CHUNKS;
            const int j = j0 + r;
            if (j >= L) continue;
            const uint32_t off = lo + 16u * c;
            if (off <= hi) ptx::cp_async_16(pstage + r * P_PITCH + 16 * c, src_base + (size_t)j * row_bytes + off);
          }
        }
        ptx::cp_async_mbar_arrive_noinc(&bars->bias_full[sb]);
      }
      ptx::cp_async_wait_all();
    }
  } else {
    RoleCtx ctx{smem, bars, lut_s, kbits, tmem_base, status_word, L, H, b, h, i0, n_kt, has_c2p, has_p2c};
    softmax_role<T, D, NB>(ctx, p, warp, lane);
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 5) ptx::tmem_dealloc(tmem_base, LO::kTmemCols);
}

}  // namespace

namespace {

template <typename T, int D, int NB>
int launch_typed(const DflAttnParams& p, cudaStream_t stream) {
  using LO = Layout<D, NB>;
  const int L = p.seq_len;
  const int BH = p.batch * p.heads;
  const uint64_t row = (uint64_t)D * sizeof(T), seq = (uint64_t)L * row;
  const uint32_t box_inner = D < 64 ? D : 64;
  CUtensorMap tq, tk, tv;
  int rc = encode_tensor_map_3d(&tq, p.q, D, L, BH, row, seq, box_inner, BM, LO::kRowBytes);
  if (rc == DFL_OK) rc = encode_tensor_map_3d(&tk, p.k, D, L, BH, row, seq, box_inner, BN, LO::kRowBytes);
  if (rc == DFL_OK) rc = encode_tensor_map_3d(&tv, p.v, D, L, BH, row, seq, box_inner, BN, LO::kRowBytes);
  if (rc != DFL_OK) return rc;

  // Shared memory: what the kernel uses, but never so little that more CTAs could become
  // resident on one SM than the 512 TMEM columns can serve (each CTA allocates kTmemCols).
  constexpr int kMaxCtas = 512 / LO::kTmemCols;
  int smem = LO::total(L);
  const int floor_for_tmem = kMaxSmem / (kMaxCtas + 1) + 1024;
  if (smem < floor_for_tmem) smem = floor_for_tmem;
  if (smem > kMaxSmem) return fail(DFL_ERR_TOO_LARGE, "seq_len %d needs %d bytes of shared memory", L, smem);

  auto kernel = attention_tc_kernel<T, D, NB>;
  static KernelDeviceConfig config;   // per instantiation
  rc = configure_kernel(config, kernel, smem, nullptr, "attention_tc_kernel");
  if (rc != DFL_OK) return rc;
  int* status_word = p.status;
  if (!status_word) {
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&status_word), g_attn_status);
    if (e != cudaSuccess) return fail(DFL_ERR_LAUNCH, "status word: %s", cudaGetErrorString(e));
  }
  dim3 grid((L + BM - 1) / BM, BH);
  if (grid.y > 65535) return fail(DFL_ERR_TOO_LARGE, "batch*heads > 65535");
  kernel<<<grid, kThreads, smem, stream>>>(tq, tk, tv, p, status_word);
  return check_launch("attention_tc_kernel");
}

template <typename T, int D>
int launch_stages(const DflAttnParams& p, cudaStream_t stream) {
  const bool has_pos = p.c2p != nullptr || p.p2c != nullptr;
  if (has_pos && Layout<D, 2>::total(p.seq_len) <= kMaxSmem) return launch_typed<T, D, 2>(p, stream);
  return launch_typed<T, D, 1>(p, stream);
}

template <typename T>
int launch_d(const DflAttnParams& p, cudaStream_t stream) {
  switch (p.head_dim) {
    case 32: return launch_stages<T, 32>(p, stream);
    case 64: return launch_stages<T, 64>(p, stream);
    case 128: return launch_stages<T, 128>(p, stream);
  }
  return fail(DFL_ERR_UNSUPPORTED, "head_dim %d not in {32,64,128}", p.head_dim);
}

}  // namespace

int launch_attention_tc(const DflAttnParams& p, cudaStream_t stream) {
  if (p.seq_len > 16384) return fail(DFL_ERR_TOO_LARGE, "seq_len %d > 16384", p.seq_len);
  if (p.dtype == DFL_F16) return launch_d<__half>(p, stream);
  if (p.dtype == DFL_BF16) return launch_d<__nv_bfloat16>(p, stream);
  return fail(DFL_ERR_UNSUPPORTED, "tcgen05 attention handles FP16/BF16 only");
}

}  // namespace dfl
