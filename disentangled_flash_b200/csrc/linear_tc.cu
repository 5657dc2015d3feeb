// tcgen05 GEMM family for FP16/BF16: fused QKV projection with head-split
// epilogue, relative-embedding projection, and the C2P/P2C position-score GEMMs.
//
// Replaces the library GEMMs on the reference's hot path: F.linear for the
// fused QKV projection plus the three permute().contiguous() copies
// (src/disentangled_flash/_torch.py:284-314), the relative-embedding
// projections (_torch.py:143-158) and torch.matmul x2 for the position scores
// (src/disentangled_flash/kernel.py:574-585).
//
//   C_z[m,n] = sum_k X_z[m,k] * W_{z % w_mod}[n,k] (+ bias[n]),  fp32 accumulation in TMEM
//
// Two kernels, both persistent with one CTA per SM and 320 threads.  A producer warp streams K-blocks of X and W
// into a shared-memory ring with TMA (128-byte swizzle, K-major) and keeps streaming across tile boundaries, one
// elected thread of the MMA warp issues tcgen05.mma into one of two 256-column TMEM accumulators, and eight
// epilogue warps drain the finished accumulator (tcgen05.ld, one row per thread, 128 columns per warp), add the
// bias, apply the activation, round to the output type, stage 32 x 64 blocks in shared memory and write them with
// tiled bulk stores, head-major [B,H,L,d] or row-major - while the MMA warp already fills the other accumulator.
//   * gemm_tc_pair_kernel: clusters of two CTAs on one 256 x 256 tile (cta_group::2), six 32 KB stages per CTA;
//     used whenever M >= 256 and K >= 64.
//   * gemm_tc_kernel: one CTA per 128 x 256 tile, for the small shapes.
#include <cstring>

#include "dfl_common.cuh"
#include "tcgen05_ptx.cuh"

namespace dfl {

// ------------------------------------------------------------------ tensor maps
namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn resolve_encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}
}  // namespace

int encode_tensor_map_3d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t rows, uint64_t batch,
                         uint64_t row_stride_bytes, uint64_t batch_stride_bytes, uint32_t box_inner,
                         uint32_t box_rows, int swizzle_bytes) {
  EncodeTiledFn encode = resolve_encode_tiled();
  if (!encode) return fail(DFL_ERR_DRIVER, "cuTensorMapEncodeTiled entry point not available");
  if ((row_stride_bytes & 15) || (batch_stride_bytes & 15))
    return fail(DFL_ERR_ALIGNMENT, "tensor-map strides must be multiples of 16 bytes");
  const cuuint64_t dims[3] = {inner, rows, batch};
  const cuuint64_t strides[2] = {row_stride_bytes, batch_stride_bytes};
  const cuuint32_t box[3] = {box_inner, box_rows, 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  CUtensorMapSwizzle sw = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), dims, strides, box,
                      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(DFL_ERR_DRIVER, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return DFL_OK;
}

// Library-owned status word for kernels whose caller passes none.
__device__ int g_gemm_status = 0;

namespace {

constexpr int TM = 128, TN = 256;  // 128 x 256 output tile: 87 flop per operand byte staged through shared memory
constexpr int kEpilogueWarps = 8;   // warp w drains TMEM lanes 32*(w&3).. of accumulator columns 128*(w>>2)..
constexpr int kTmaWarp = 8, kMmaWarp = 9;
constexpr int kThreads = 320;
constexpr int kTmemCols = 512;      // two 256-column accumulators: epilogue of tile i overlaps main loop of tile i+1
constexpr int kMaxSmem = 232448;

// Output staging for the tiled-store epilogue: per epilogue warp one buffer of 32 rows x 64 columns (128-byte
// rows in the 128-byte swizzle pattern of the output tensor maps).  Two warps share a scheduler, so one converts
// while the other's store drains its buffer.
constexpr int kStageRows = 32, kStageCols = 64;
constexpr int kStageBufBytes = kStageRows * kStageCols * 2;   // 4 KB
constexpr int kStagingBytes = 8 * kStageBufBytes;              // one buffer per epilogue warp = 32 KB

struct OutMaps {
  CUtensorMap m[3];
};

template <int BK>
struct GemmSmem {
  static constexpr int kRowBytes = BK * 2;
  static constexpr int kTileA = TM * kRowBytes;
  static constexpr int kTileB = TN * kRowBytes;
  static constexpr int kStage = kTileA + kTileB;
  static constexpr int kStages = BK == 64 ? 4 : 6;          // 192 KB / 144 KB of operand ring: one CTA per SM
  static constexpr int kStagingOffset = kStages * kStage;      // output staging of the epilogue warps
  static constexpr int kBarrierOffset = kStagingOffset + kStagingBytes;
  static constexpr int kTotal = kBarrierOffset + 512 + 1024;  // barriers + holder + flags, + alignment slack
};

// Epilogue of one accumulator chunk: 32 consecutive columns [n, n+32) of output row m, as fp32 bit patterns in r.
// Adds the bias, rounds to T and stores 32 (or 16) bytes at a time, head-major or row-major.
template <typename T>
__device__ __forceinline__ void store_chunk(const GemmDesc& g, const uint32_t (&r)[32], int m, int n, int z, int ncols,
                                            int hd, const T* bias) {
  T* dst;
  int valid = 32;
  if (g.head_split) {
    const int which = n / hd, rem = n - which * hd;
    const int h = rem / g.head_dim, dd = rem - h * g.head_dim;
    const int row = g.row_groups ? __ldg(g.row_groups + (m >> 5)) + (m & 31) : m;
    const int b = row / g.rows_per_seq, l = row - b * g.rows_per_seq;
    T* out = reinterpret_cast<T*>(which == 0 ? g.out[0] : (which == 1 ? g.out[1] : g.out[2]));
    dst = out + (((long long)b * g.heads + h) * g.rows_per_seq + l) * g.head_dim + dd;
  } else {
    dst = reinterpret_cast<T*>(g.out[0]) + (long long)z * g.stride_c + (long long)m * g.ldc + n;
    valid = ncols - n < 32 ? ncols - n : 32;  // multiple of 8
  }
  // 32-byte stores (one full sector per thread and instruction) where the destination allows them
  const bool wide = (reinterpret_cast<uintptr_t>(dst) & 31u) == 0;
  uint4 held = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    if (v * 8 >= valid) break;
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
    if (bias) {
      const uint4 braw = __ldg(reinterpret_cast<const uint4*>(bias + n + v * 8));
      const T* bh = reinterpret_cast<const T*>(&braw);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += Elem<T>::to_f(bh[j]);
    }
    if (g.activation == DFL_ACT_GELU) {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = gelu_erf_fast(f[j]);
    }
    uint4 packed;
    T* ph = reinterpret_cast<T*>(&packed);
#pragma unroll
    for (int j = 0; j < 8; ++j) ph[j] = Elem<T>::from_f(f[j]);
    const bool pair_end = (v & 1) != 0, pair_start_last = (v & 1) == 0 && (v + 1) * 8 >= valid;
    if (wide && pair_end) {
      asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst + (v - 1) * 8), "r"(held.x), "r"(held.y),
                   "r"(held.z), "r"(held.w), "r"(packed.x), "r"(packed.y), "r"(packed.z), "r"(packed.w) : "memory");
    } else if (wide && !pair_start_last) {
      held = packed;
    } else {
      *reinterpret_cast<uint4*>(dst + v * 8) = packed;
    }
  }
}

// Whether the output can be written as 32-row x 64-column boxes: row-major always (the tensor map clips at ldc and
// M); head-major when a box neither straddles two heads (head_dim a multiple of 64) nor two sequences.
__host__ __device__ inline bool tiled_store_ok(const GemmDesc& g) {
  return !g.head_split || (g.head_dim % kStageCols == 0 && g.rows_per_seq % kStageRows == 0);
}

// Drains one warp's 32 lanes x 128 columns of an accumulator.  `taddr` = TMEM address of the warp's lane quarter at
// the accumulator's first column, `m_warp` = output row of lane 0, `n0` = first output column of the tile,
// `col_begin` = first accumulator column of this warp (0 or 128).
// With `tiled` the rows go through the warp's staging buffers and leave as tiled bulk stores of full 128-byte
// lines (per-thread stores would write every 32-byte sector in two halves from different instructions, and the
// number of store requests, not the math, then bounds GEMMs with a short K).
// CONV: the epilogue of the convolution branch (padding mask of the output row, tanh) is compiled in; plain GEMMs
// take the instantiation without it (the extra code cost them 7 % when it was shared).
template <typename T, bool CONV>
__device__ __forceinline__ void drain_accumulator(const GemmDesc& g, const CUtensorMap* tmap_out, bool tiled,
                                                  unsigned char* buf, uint32_t taddr, int m_warp, int n0,
                                                  int col_begin, int z, bool ready, int lane) {
  const int ncols = g.head_split ? g.N : g.ldc;
  const T* bias = reinterpret_cast<const T*>(g.bias);
  const int hd = g.heads * g.head_dim;
  if (!tiled) {
    const int m = m_warp + lane;
#pragma unroll 1
    for (int c0 = col_begin; c0 < col_begin + TN / 2; c0 += 32) {
      const int n = n0 + c0;
      if (n >= ncols) break;  // warp-uniform
      uint32_t r[32];
      ptx::tmem_ld32(taddr + (uint32_t)c0, r);
      ptx::tmem_wait_ld();
      if (!ready || m >= g.M) continue;
      store_chunk<T>(g, r, m, n, z, ncols, hd, bias);
    }
    return;
  }
  // padding mask of this thread's output row (convolution epilogue)
  bool keep_row = true;
  if (CONV && g.row_mask && m_warp + lane < g.M) keep_row = mask_keep(g.row_mask, g.row_mask_elem, (long long)z * g.M + m_warp + lane);
#pragma unroll 1
  for (int c0 = col_begin; c0 < col_begin + TN / 2; c0 += kStageCols) {
    const int n = n0 + c0;
    if (n >= ncols) break;  // warp-uniform
    uint32_t r0[32], r1[32];
    ptx::tmem_ld32(taddr + (uint32_t)c0, r0);
    ptx::tmem_ld32(taddr + (uint32_t)c0 + 32u, r1);
    // the previous store of this warp has finished reading the buffer
    if (lane == 0) ptx::bulk_wait_group_read<0>();
    __syncwarp();
    ptx::tmem_wait_ld();
    if (!ready || m_warp >= g.M) continue;  // warp-uniform
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v < 4 ? r0[v * 8 + j] : r1[(v - 4) * 8 + j]);
      if (bias && n + v * 8 < g.N) {
        const uint4 braw = __ldg(reinterpret_cast<const uint4*>(bias + n + v * 8));
        const T* bh = reinterpret_cast<const T*>(&braw);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += Elem<T>::to_f(bh[j]);
      }
      if (CONV && !keep_row) {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = 0.0f;
      }
      if (g.activation == DFL_ACT_GELU) {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = gelu_erf_fast(f[j]);
      } else if (CONV && g.activation == DFL_ACT_TANH) {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = tanh_fast(f[j]);
      }
      uint4 packed;
      T* ph = reinterpret_cast<T*>(&packed);
#pragma unroll
      for (int j = 0; j < 8; ++j) ph[j] = Elem<T>::from_f(f[j]);
      *reinterpret_cast<uint4*>(buf + lane * 128 + ((v ^ (lane & 7)) << 4)) = packed;
    }
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      if (g.head_split) {
        const int which = n / hd, rem = n - which * hd;
        const int h = rem / g.head_dim, dd = rem - h * g.head_dim;
        const int row = g.row_groups ? __ldg(g.row_groups + (m_warp >> 5)) : m_warp;   // a warp's 32 rows: one group
        const int b = row / g.rows_per_seq, l = row - b * g.rows_per_seq;
        ptx::tma_store_3d(&tmap_out[which], buf, dd, l, b * g.heads + h);
      } else {
        ptx::tma_store_3d(&tmap_out[0], buf, n, m_warp, z);
      }
      ptx::bulk_commit_group();
    }
  }
}

// Persistent kernel: grid = number of SMs (or fewer tiles); each CTA walks tiles t = blockIdx.x, + gridDim.x, ...
// Tile order: n fastest, so that CTAs running concurrently share rows of X in L2.
template <typename T, int BK>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
               const __grid_constant__ OutMaps tmap_out, const GemmDesc g, const int num_kb, const int tiles_n,
               const int tiles_m, const int num_tiles, const int tiled) {
  using S = GemmSmem<BK>;
  constexpr int STAGES = S::kStages;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarrierOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;   // [2]
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;   // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&tmem_full_bar[a], 1);
      ptx::mbar_init(&tmem_empty_bar[a], kEpilogueWarps);  // one elected lane of each epilogue warp
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kTmaWarp && lane == 0) {
    ptx::prefetch_tensormap(&tmap_x);
    ptx::prefetch_tensormap(&tmap_w);
  }
  if (warp == kMmaWarp) {
    ptx::tmem_alloc(tmem_holder, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  auto tile_coords = [&](int tile, int& m0, int& n0, int& z) {
    const int per_z = tiles_n * tiles_m;
    z = tile / per_z;
    const int rem = tile - z * per_z;
    const int tm = rem / tiles_n;
    m0 = tm * TM;
    n0 = (rem - tm * tiles_n) * TN;
  };

  if (warp == kTmaWarp) {
    // ---------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m0, n0, z;
        tile_coords(tile, m0, n0, z);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          ok = ptx::mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, g.status, 1);
          if (!ok) break;
          ptx::mbar_arrive_expect_tx(&full_bar[s], (uint32_t)S::kStage);
          unsigned char* a = smem + s * S::kStage;
          ptx::tma_load_3d(a, &tmap_x, &full_bar[s], kb * BK, m0, z);
          ptx::tma_load_3d(a + S::kTileA, &tmap_w, &full_bar[s], kb * BK, n0, z % g.w_mod);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_idesc_f16(__is_same(T, __nv_bfloat16) ? 1 : 0, TM, TN, 0, 0);
      constexpr uint32_t mode = ptx::swizzle_mode_for_row_bytes(S::kRowBytes);
      const uint64_t adesc0 = ptx::make_smem_desc(ptx::smem_u32(smem), 16, 8 * S::kRowBytes, mode);
      const uint64_t bdesc0 = ptx::make_smem_desc(ptx::smem_u32(smem + S::kTileA), 16, 8 * S::kRowBytes, mode);
      uint32_t it = 0;
      bool ok = true;
      int lt = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++lt) {
        const int acc = lt & 1;
        ok = ptx::mbar_wait(&tmem_empty_bar[acc], ((uint32_t)(lt >> 1) & 1u) ^ 1u, abort_flag, g.status, 4);
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          ok = ptx::mbar_wait(&full_bar[s], ph, abort_flag, g.status, 2);
          if (!ok) break;
          ptx::tc_fence_after();
          // descriptors differ from the stage-0 ones only in the 16-byte-granular address field
          const uint64_t adesc = adesc0 + (uint64_t)(s * (S::kStage >> 4));
          const uint64_t bdesc = bdesc0 + (uint64_t)(s * (S::kStage >> 4));
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            ptx::umma_ss_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          ptx::umma_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
        }
        if (!ok) break;
        ptx::umma_commit(&tmem_full_bar[acc]);  // accumulator complete
      }
    }
  } else {
    // -------------------------------------------------------------- epilogue
    unsigned char* staging = smem + S::kStagingOffset + warp * kStageBufBytes;
    const int quarter = warp & 3, col_begin = (warp >> 2) * (TN / 2);
    bool ready = true;
    int lt = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++lt) {
      int m0, n0, z;
      tile_coords(tile, m0, n0, z);
      const int acc = lt & 1;
      if (ready) ready = ptx::mbar_wait(&tmem_full_bar[acc], (uint32_t)(lt >> 1) & 1u, abort_flag, g.status, 3);
      ptx::tc_fence_after();
      drain_accumulator<T, false>(g, tmap_out.m, tiled != 0, staging,
                           tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * TN), m0 + quarter * 32, n0,
                           col_begin, z, ready, lane);
      // this warp has read its lanes of the accumulator: hand it back to the MMA issuer
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&tmem_empty_bar[acc]);
    }
    if (lane == 0) ptx::bulk_wait_group<0>();   // the staging buffers are read until the stores complete
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) ptx::tmem_dealloc(tmem_base, kTmemCols);
}

// ---------------------------------------------------------------------------------------------------------------
// CTA-pair form (clusters of two, `cta_group::2`): one 256 x 256 output tile per pair.  Each CTA loads its own 128
// rows of X and 128 of the tile's 256 rows of W per k-step (32 KB for 128 x 256 x 64 of MMA work, against 48 KB in
// the single-CTA kernel: the operand stream from L2 is what bounds this GEMM), the leader CTA (cluster rank 0)
// issues M=256, N=256 MMAs that read both CTAs' shared memory and write 128 accumulator lanes in each CTA's TMEM,
// and each CTA's epilogue warps drain their own lanes.  Barriers: the loads of both CTAs report to the leader's
// `full` barriers; the leader's commits arrive on the `empty` / `tmem_full` barriers of both CTAs; the epilogue
// warps of both CTAs arrive on the leader's `tmem_empty` barriers.
constexpr int kPairStages = 6;                       // 6 x 32 KB operand ring per CTA
constexpr int kPairStageBytes = (TM + TN / 2) * 128;  // A 128x64 + half of B 128x64, 2-byte elements
constexpr int kPairStagingOffset = kPairStages * kPairStageBytes;
constexpr int kPairBarrierOffset = kPairStagingOffset + kStagingBytes;
constexpr int kPairSmem = kPairBarrierOffset + 512 + 1024;
static_assert(kPairSmem <= kMaxSmem && GemmSmem<64>::kTotal <= kMaxSmem && GemmSmem<32>::kTotal <= kMaxSmem,
              "operand ring + output staging + barriers must fit the 227 KB a CTA can opt in to");

template <typename T, bool CONV>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                    const __grid_constant__ OutMaps tmap_out, const GemmDesc g, const int num_kb, const int tiles_n,
                    const int tiles_m, const int num_tiles, const int tiled) {
  constexpr int BK = 64;
  constexpr int STAGES = kPairStages;
  constexpr int kTileA = TM * BK * 2;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kPairBarrierOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;   // [2]
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;   // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();   // 0 = leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);    // the leader's producer (expect_tx); only the leader's are used
      ptx::mbar_init(&empty_bar[s], 1);   // one commit of the leader's MMA thread, delivered to both CTAs
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&tmem_full_bar[a], 1);
      ptx::mbar_init(&tmem_empty_bar[a], 2 * kEpilogueWarps);  // one lane of each epilogue warp of both CTAs (leader's only)
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kTmaWarp && lane == 0) {
    ptx::prefetch_tensormap(&tmap_x);
    ptx::prefetch_tensormap(&tmap_w);
  }
  if (warp == kMmaWarp) {
    ptx::tmem_alloc_pair(tmem_holder, kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();   // the peer's barriers exist before anything is reported to them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  wait_for_predecessor();    // the set-up above overlaps the previous kernel's tail; its outputs are read from here on

  auto tile_coords = [&](int tile, int& m0, int& n0, int& z) {
    const int per_z = tiles_n * tiles_m;
    z = tile / per_z;
    const int rem = tile - z * per_z;
    const int tm = rem / tiles_n;
    m0 = tm * (2 * TM);
    n0 = (rem - tm * tiles_n) * TN;
  };

  if (warp == kTmaWarp) {
    // ---------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int m0, n0, z;
        tile_coords(tile, m0, n0, z);
        // k-steps: num_kb = taps x (k-blocks per tap); a plain GEMM has one tap with no row shift
        const int taps = CONV && g.taps > 1 ? g.taps : 1;
        const int kb_per_tap = CONV ? num_kb / taps : num_kb;
        const int w_batch = z % g.w_mod;
        int tap = 0, kb = 0;
        for (int step = 0; step < num_kb; ++step, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          ok = ptx::mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, g.status, 11);
          if (!ok) break;
          if (rank == 0) ptx::mbar_arrive_expect_tx(&full_bar[s], 2u * (uint32_t)kPairStageBytes);
          const uint32_t leader_full = ptx::map_to_cta(ptx::smem_u32(&full_bar[s]), 0);
          unsigned char* a = smem + s * kPairStageBytes;
          // rows above the first or below the last row of X_z are filled with zeros by the load
          if constexpr (CONV) {
            ptx::tma_load_3d_pair(a, &tmap_x, leader_full, kb * BK, m0 + (int)rank * TM + tap - (taps >> 1), z);
            ptx::tma_load_3d_pair(a + kTileA, &tmap_w, leader_full, kb * BK, n0 + (int)rank * (TN / 2),
                                  taps > 1 ? tap : w_batch);
            if (++kb == kb_per_tap) {
              kb = 0;
              ++tap;
            }
          } else {
            ptx::tma_load_3d_pair(a, &tmap_x, leader_full, step * BK, m0 + (int)rank * TM, z);
            ptx::tma_load_3d_pair(a + kTileA, &tmap_w, leader_full, step * BK, n0 + (int)rank * (TN / 2), w_batch);
          }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = ptx::make_idesc_f16(__is_same(T, __nv_bfloat16) ? 1 : 0, 2 * TM, TN, 0, 0);
      constexpr uint32_t mode = ptx::swizzle_mode_for_row_bytes(BK * 2);
      const uint64_t adesc0 = ptx::make_smem_desc(ptx::smem_u32(smem), 16, 8 * BK * 2, mode);
      const uint64_t bdesc0 = ptx::make_smem_desc(ptx::smem_u32(smem + kTileA), 16, 8 * BK * 2, mode);
      uint32_t it = 0;
      bool ok = true;
      int lt = 0;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++lt) {
        const int acc = lt & 1;
        ok = ptx::mbar_wait(&tmem_empty_bar[acc], ((uint32_t)(lt >> 1) & 1u) ^ 1u, abort_flag, g.status, 14);
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          ok = ptx::mbar_wait(&full_bar[s], ph, abort_flag, g.status, 12);
          if (!ok) break;
          ptx::tc_fence_after();
          const uint64_t adesc = adesc0 + (uint64_t)(s * (kPairStageBytes >> 4));
          const uint64_t bdesc = bdesc0 + (uint64_t)(s * (kPairStageBytes >> 4));
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            ptx::umma_ss_f16_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          ptx::umma_commit_pair(&empty_bar[s]);  // frees the stage in both CTAs
        }
        if (!ok) break;
        ptx::umma_commit_pair(&tmem_full_bar[acc]);  // accumulator complete, both CTAs' epilogues may read
      }
    }
  } else {
    // -------------------------------------------------------------- epilogue (both CTAs, own lanes)
    unsigned char* staging = smem + kPairStagingOffset + warp * kStageBufBytes;
    const int quarter = warp & 3, col_begin = (warp >> 2) * (TN / 2);
    bool ready = true;
    int lt = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++lt) {
      int m0, n0, z;
      tile_coords(tile, m0, n0, z);
      const int acc = lt & 1;
      if (ready) ready = ptx::mbar_wait(&tmem_full_bar[acc], (uint32_t)(lt >> 1) & 1u, abort_flag, g.status, 13);
      ptx::tc_fence_after();
      drain_accumulator<T, CONV>(g, tmap_out.m, tiled != 0, staging,
                           tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * TN),
                           m0 + (int)rank * TM + quarter * 32, n0, col_begin, z, ready, lane);
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&tmem_empty_bar[acc]), 0));
    }
    if (lane == 0) ptx::bulk_wait_group<0>();   // the staging buffers are read until the stores complete
  }

  // Nothing of this CTA may still be in use by the peer (its shared memory is read by the leader's MMAs, its
  // barriers receive the leader's commits) when it exits or frees its tensor memory.
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();
  ptx::tc_fence_after();
  if (warp == kMmaWarp) ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
}

// Tensor maps of the outputs for the tiled-store epilogue: boxes of 32 rows x 64 columns, 128-byte swizzle.
// Head-major outputs [B, H, L, d] are described as {d, L, B*H}; the row-major output as {ldc, M, batch}.
template <typename T>
int encode_output_maps(const GemmDesc& g, OutMaps* maps, int* tiled) {
  *tiled = tiled_store_ok(g) ? 1 : 0;
  memset(maps, 0, sizeof(*maps));
  if (!*tiled) return DFL_OK;
  const size_t es = sizeof(T);
  if (g.head_split) {
    const uint64_t seqs = (uint64_t)(g.row_groups ? g.out_seqs : g.M / g.rows_per_seq) * g.heads;
    for (int o = 0; o < 3; ++o) {
      if (!g.out[o]) continue;
      int rc = encode_tensor_map_3d(&maps->m[o], g.out[o], g.head_dim, g.rows_per_seq, seqs, (uint64_t)g.head_dim * es,
                                    (uint64_t)g.rows_per_seq * g.head_dim * es, kStageCols, kStageRows, 128);
      if (rc != DFL_OK) return rc;
    }
    return DFL_OK;
  }
  const uint64_t batch_stride = g.batch > 1 ? (uint64_t)g.stride_c * es : (uint64_t)g.M * g.ldc * es;
  return encode_tensor_map_3d(&maps->m[0], g.out[0], g.ldc, g.M, g.batch, (uint64_t)g.ldc * es, batch_stride,
                              kStageCols, kStageRows, 128);
}

template <typename T, bool CONV>
int launch_pair(const GemmDesc& g, cudaStream_t stream) {
  constexpr int BK = 64;
  const size_t es = sizeof(T);
  CUtensorMap tmap_x, tmap_w;
  const uint64_t x_batch_stride = g.batch > 1 ? (uint64_t)g.stride_x * es : (uint64_t)g.M * g.K * es;
  const int taps = g.taps > 1 ? g.taps : 1;
  const int w_batches = taps > 1 ? taps : (g.w_mod > 1 ? g.w_mod : 1);
  const uint64_t w_batch_stride = taps > 1 ? (uint64_t)g.N * g.K * es
                                  : (w_batches > 1 ? (uint64_t)g.stride_w * es : (uint64_t)g.N * g.K * es);
  int rc = encode_tensor_map_3d(&tmap_x, g.x, g.K, g.M, g.batch, (uint64_t)g.K * es, x_batch_stride, BK, TM, BK * 2);
  if (rc != DFL_OK) return rc;
  rc = encode_tensor_map_3d(&tmap_w, g.w, g.K, g.N, w_batches, (uint64_t)g.K * es, w_batch_stride, BK, TN / 2, BK * 2);
  if (rc != DFL_OK) return rc;
  OutMaps tmap_out;
  int tiled = 0;
  rc = encode_output_maps<T>(g, &tmap_out, &tiled);
  if (rc != DFL_OK) return rc;

  auto kernel = gemm_tc_pair_kernel<T, CONV>;
  static KernelDeviceConfig config;   // per template instantiation
  int num_sms = 0;
  rc = configure_kernel(config, kernel, kPairSmem, &num_sms, "gemm_tc_pair_kernel");
  if (rc != DFL_OK) return rc;
  GemmDesc gd = g;
  if (!gd.status) {
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&gd.status), g_gemm_status);
    if (e != cudaSuccess) return fail(DFL_ERR_LAUNCH, "status word: %s", cudaGetErrorString(e));
  }
  const int ncols = g.head_split ? g.N : g.ldc;
  const int tiles_n = (ncols + TN - 1) / TN, tiles_m = (g.M + 2 * TM - 1) / (2 * TM);
  const long long num_tiles = (long long)tiles_n * tiles_m * g.batch;
  if (num_tiles > 0x7fffffff) return fail(DFL_ERR_TOO_LARGE, "gemm_tc: too many tiles");
  const long long max_pairs = num_sms / 2;
  const int pairs = (int)(num_tiles < max_pairs ? num_tiles : max_pairs);
  const int num_kb = taps * ((g.K + BK - 1) / BK);
  cudaError_t le = launch_after_predecessor(kernel, dim3(2 * pairs), dim3(kThreads), kPairSmem, stream, tmap_x, tmap_w,
                                            tmap_out, gd, num_kb, tiles_n, tiles_m, (int)num_tiles, tiled);
  if (le != cudaSuccess) return fail(DFL_ERR_LAUNCH, "gemm_tc_pair_kernel: %s", cudaGetErrorString(le));
  return check_launch("gemm_tc_pair_kernel");
}

template <typename T, int BK>
int launch_bk(const GemmDesc& g, cudaStream_t stream) {
  using S = GemmSmem<BK>;
  const size_t es = sizeof(T);
  CUtensorMap tmap_x, tmap_w;
  const uint64_t x_batch_stride = g.batch > 1 ? (uint64_t)g.stride_x * es : (uint64_t)g.M * g.K * es;
  const int w_batches = g.w_mod > 1 ? g.w_mod : 1;
  const uint64_t w_batch_stride = w_batches > 1 ? (uint64_t)g.stride_w * es : (uint64_t)g.N * g.K * es;
  int rc = encode_tensor_map_3d(&tmap_x, g.x, g.K, g.M, g.batch, (uint64_t)g.K * es, x_batch_stride, BK, TM, BK * 2);
  if (rc != DFL_OK) return rc;
  rc = encode_tensor_map_3d(&tmap_w, g.w, g.K, g.N, w_batches, (uint64_t)g.K * es, w_batch_stride, BK, TN, BK * 2);
  if (rc != DFL_OK) return rc;
  OutMaps tmap_out;
  int tiled = 0;
  rc = encode_output_maps<T>(g, &tmap_out, &tiled);
  if (rc != DFL_OK) return rc;

  auto kernel = gemm_tc_kernel<T, BK>;
  static KernelDeviceConfig config;   // per template instantiation
  int num_sms = 0;
  rc = configure_kernel(config, kernel, S::kTotal, &num_sms, "gemm_tc_kernel");
  if (rc != DFL_OK) return rc;
  GemmDesc gd = g;
  if (!gd.status) {
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&gd.status), g_gemm_status);
    if (e != cudaSuccess) return fail(DFL_ERR_LAUNCH, "status word: %s", cudaGetErrorString(e));
  }
  const int ncols = g.head_split ? g.N : g.ldc;
  const int tiles_n = (ncols + TN - 1) / TN, tiles_m = (g.M + TM - 1) / TM;
  const long long num_tiles = (long long)tiles_n * tiles_m * g.batch;
  if (num_tiles > 0x7fffffff) return fail(DFL_ERR_TOO_LARGE, "gemm_tc: too many tiles");
  const int grid = (int)(num_tiles < num_sms ? num_tiles : num_sms);
  const int num_kb = (g.K + BK - 1) / BK;
  kernel<<<grid, kThreads, S::kTotal, stream>>>(tmap_x, tmap_w, tmap_out, gd, num_kb, tiles_n, tiles_m,
                                                (int)num_tiles, tiled);
  return check_launch("gemm_tc_kernel");
}

template <typename T>
int launch_t(const GemmDesc& g, cudaStream_t stream) {
  if (g.K % 8) return fail(DFL_ERR_ALIGNMENT, "K=%d: rows must be multiples of 16 bytes for TMA", g.K);
  if (g.head_split && (g.head_dim % 32)) return fail(DFL_ERR_UNSUPPORTED, "head_dim must be a multiple of 32");
  if (!g.head_split && (g.ldc % 8)) return fail(DFL_ERR_ALIGNMENT, "ldc must be a multiple of 8");
  if (g.bias && !aligned16(g.bias)) return fail(DFL_ERR_ALIGNMENT, "bias not 16-byte aligned");
  // CTA pairs on 256 x 256 tiles when the problem has at least one full pair tile of rows and a 64-wide k-step
  if (g.K >= 64 && g.M >= 2 * TM) {
    const bool conv = g.taps > 1 || g.row_mask || g.activation == DFL_ACT_TANH;
    return conv ? launch_pair<T, true>(g, stream) : launch_pair<T, false>(g, stream);
  }
  if (g.taps > 1 || g.row_mask) return fail(DFL_ERR_UNSUPPORTED, "taps and row masks need the pair kernel (M >= 256, K >= 64)");
  return g.K >= 64 ? launch_bk<T, 64>(g, stream) : launch_bk<T, 32>(g, stream);
}

}  // namespace

int launch_gemm_tc(const GemmDesc& g, cudaStream_t stream) {
  if (g.dtype == DFL_F16) return launch_t<__half>(g, stream);
  if (g.dtype == DFL_BF16) return launch_t<__nv_bfloat16>(g, stream);
  return fail(DFL_ERR_UNSUPPORTED, "tcgen05 GEMM handles FP16/BF16 only");
}

}  // namespace dfl
