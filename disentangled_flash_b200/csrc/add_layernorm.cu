// Residual add + LayerNorm in one pass over HBM.
//
// Replaces, in the encoder's layer loop (src/disentangled_flash/deberta.py:268-270), the tail of the two output
// blocks of a layer - DebertaV2SelfOutput.forward (_reference.py:108-112) and DebertaV2Output.forward
// (_reference.py:481-485): `LayerNorm(dense_out + residual)`, which PyTorch runs as an elementwise add (read 2,
// write 1) followed by a layer-norm kernel (read 1, write 1).  Here: read 2, write 1.
//
//   out[r, :] = (v - mean(v)) * rsqrt(var(v) + eps) * gamma + beta,   v = x[r, :] + residual[r, :]   (fp32)
//
// One warp per row, the row held in registers as 16-byte vectors (VEC per lane), two-pass statistics (mean, then
// centred variance) with warp shuffles; no shared memory.  HBM bound: algorithmic bytes per row
// (2 reads + 1 write) * hidden * sizeof(T)  (1 read + 1 write without a residual).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "dfl_common.cuh"

namespace dfl {
namespace {

constexpr int kWarpsPerBlock = 8;

template <typename T>
struct Vec16 {
  static constexpr int kElems = 16 / sizeof(T);
};

template <typename T>
__device__ __forceinline__ void unpack(const uint4& raw, float* out);
template <>
__device__ __forceinline__ void unpack<float>(const uint4& raw, float* out) {
  out[0] = __uint_as_float(raw.x); out[1] = __uint_as_float(raw.y);
  out[2] = __uint_as_float(raw.z); out[3] = __uint_as_float(raw.w);
}
template <>
__device__ __forceinline__ void unpack<__half>(const uint4& raw, float* out) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    out[2 * i] = f.x; out[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void unpack<__nv_bfloat16>(const uint4& raw, float* out) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {   // a bf16 is the upper half of an fp32
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <typename T>
__device__ __forceinline__ uint4 pack(const float* in);
template <>
__device__ __forceinline__ uint4 pack<float>(const float* in) {
  return make_uint4(__float_as_uint(in[0]), __float_as_uint(in[1]), __float_as_uint(in[2]), __float_as_uint(in[3]));
}
template <>
__device__ __forceinline__ uint4 pack<__half>(const float* in) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = __floats2half2_rn(in[2 * i], in[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ __forceinline__ uint4 pack<__nv_bfloat16>(const float* in) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Read once: do not keep in L1.  A plain (coherent) load: `out` may be the same buffer as `x` or `residual`, so the
// inputs are not read-only for the lifetime of the kernel.
__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Row gather for the embedding front-end: where the rows of x (and of residual) come from.
struct RowSource {
  const void* x_rows;        // [rows] indices into x (token ids), or null: row r of x is row r
  const void* res_rows;      // [rows] indices into residual (position ids), or null
  int idx_elem;              // 4 or 8: int32 / int64 indices
  long long x_limit;         // rows of the x table
  long long res_limit;       // rows of the residual table
  int* status;               // device word that receives kStatusBadIndex when an index is out of range
};
constexpr int kStatusBadIndex = 98;

__device__ __forceinline__ long long load_index(const void* idx, int elem, long long i) {
  return elem == 8 ? reinterpret_cast<const long long*>(idx)[i] : (long long)reinterpret_cast<const int*>(idx)[i];
}

// Vector j of lane l covers columns (j*32 + l) * E .. +E: a warp reads 512 contiguous bytes per vector index.
template <typename T, int VEC>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
add_layernorm_kernel(const uint4* x, const uint4* residual, const uint4* __restrict__ gamma,
                     const uint4* __restrict__ beta, uint4* out, long long rows, int hidden, float eps,
                     const void* __restrict__ row_mask, int mask_elem, uint4* out2,
                     const int32_t* __restrict__ out2_rows, const RowSource src) {
  constexpr int E = Vec16<T>::kElems;
  const int lane = threadIdx.x & 31;
  const int vecs_per_row = hidden / E;
  const float inv_n = 1.0f / (float)hidden;
  const long long warp0 = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const long long stride = (long long)gridDim.x * kWarpsPerBlock;
  wait_for_predecessor();
  for (long long row = warp0; row < rows; row += stride) {
    // an index outside its table reads as a row of zeros and is reported through the status word
    long long x_row = row, res_row = row;
    if (src.x_rows) {
      x_row = load_index(src.x_rows, src.idx_elem, row);
      if (x_row < 0 || x_row >= src.x_limit) x_row = -1;
    }
    if (src.res_rows) {
      res_row = load_index(src.res_rows, src.idx_elem, row);
      if (res_row < 0 || res_row >= src.res_limit) res_row = -1;
    }
    if ((x_row < 0 || res_row < 0) && src.status && lane == 0) atomicCAS(src.status, 0, kStatusBadIndex);
    const uint4* xr = x + x_row * vecs_per_row;
    const uint4* rr = residual ? residual + res_row * vecs_per_row : nullptr;
    uint4 rx[VEC], rres[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const int c = j * 32 + lane;
      rx[j] = c < vecs_per_row && x_row >= 0 ? ld_stream(xr + c) : make_uint4(0, 0, 0, 0);
    }
    if (rr && res_row < 0) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) rres[j] = make_uint4(0, 0, 0, 0);
    } else if (rr) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const int c = j * 32 + lane;
        rres[j] = c < vecs_per_row ? ld_stream(rr + c) : make_uint4(0, 0, 0, 0);
      }
    }
    float v[VEC * E];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      unpack<T>(rx[j], v + j * E);
      if (rr) {
        float r[E];
        unpack<T>(rres[j], r);
#pragma unroll
        for (int e = 0; e < E; ++e) v[j * E + e] += r[e];
      }
#pragma unroll
      for (int e = 0; e < E; ++e) sum += v[j * E + e];   // out-of-range vectors are zero
    }
    const float mean = warp_sum(sum) * inv_n;
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      if (j * 32 + lane < vecs_per_row) {
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float c = v[j * E + e] - mean;
          sq = fmaf(c, c, sq);
        }
      }
    }
    // rows the mask drops are written as zeros (the convolution branch multiplies its output by the padding mask)
    const float keep = row_mask && !mask_keep(row_mask, mask_elem, row) ? 0.0f : 1.0f;
    const float rstd = rsqrtf(warp_sum(sq) * inv_n + eps) * keep;
    uint4* orow = out + row * vecs_per_row;
    // optional second copy of the row at another row index (the unpacked layout of a packed batch)
    long long row2 = -1;
    if (out2) row2 = out2_rows[row];
    uint4* orow2 = row2 >= 0 ? out2 + row2 * vecs_per_row : nullptr;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const int c = j * 32 + lane;
      if (c < vecs_per_row) {
        float g[E], b[E], y[E];
        unpack<T>(__ldg(gamma + c), g);
        if (beta) unpack<T>(__ldg(beta + c), b);
#pragma unroll
        for (int e = 0; e < E; ++e) y[e] = fmaf((v[j * E + e] - mean) * rstd, g[e], beta ? b[e] * keep : 0.f);
        const uint4 packed = pack<T>(y);
        orow[c] = packed;
        if (orow2) orow2[c] = packed;
      }
    }
  }
}

template <typename T, int VEC>
void launch_one(const void* x, const void* residual, const void* gamma, const void* beta, void* out, long long rows,
                int hidden, float eps, const void* row_mask, int mask_elem, void* out2, const int32_t* out2_rows,
                const RowSource& src, int sm_count, cudaStream_t stream) {
  const long long wanted = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const long long cap = (long long)sm_count * 8;   // 8 CTAs of 8 warps per SM: one wave, grid-stride beyond it
  const int blocks = (int)(wanted < cap ? wanted : cap);
  launch_after_predecessor(add_layernorm_kernel<T, VEC>, dim3(blocks), dim3(kWarpsPerBlock * 32), 0, stream,
                           (const uint4*)x, (const uint4*)residual, (const uint4*)gamma, (const uint4*)beta, (uint4*)out,
                           rows, hidden, eps, row_mask, mask_elem, (uint4*)out2, out2_rows, src);
}

template <typename T>
int launch_typed(const void* x, const void* residual, const void* gamma, const void* beta, void* out, long long rows,
                 int hidden, float eps, const void* row_mask, int mask_elem, void* out2, const int32_t* out2_rows,
                 const RowSource& src, int sm_count, cudaStream_t stream) {
  constexpr int E = Vec16<T>::kElems;
  const int vec = (hidden / E + 31) / 32;
#define DFL_LN_CASE(V)                                                                              \
  if (vec <= V) {                                                                                   \
    launch_one<T, V>(x, residual, gamma, beta, out, rows, hidden, eps, row_mask, mask_elem, out2, out2_rows,   \
                     src, sm_count, stream);                                                                   \
    return check_launch("add_layernorm_kernel");                                                    \
  }
  DFL_LN_CASE(1) DFL_LN_CASE(2) DFL_LN_CASE(3) DFL_LN_CASE(4) DFL_LN_CASE(6) DFL_LN_CASE(8) DFL_LN_CASE(12)
  DFL_LN_CASE(16)
#undef DFL_LN_CASE
  return fail(DFL_ERR_UNSUPPORTED, "hidden size %d exceeds %d for this dtype", hidden, add_layernorm_max_hidden(sizeof(T)));
}

}  // namespace

namespace {
// dst[r, :] = src[rows[r], :] (zeros for a negative entry); one warp per row, 16-byte vectors.
__global__ void __launch_bounds__(256) copy_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                        const int32_t* __restrict__ rows, long long n_rows,
                                                        int vecs_per_row) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const long long stride = (long long)gridDim.x * 8;
  wait_for_predecessor();
  for (long long r = warp0; r < n_rows; r += stride) {
    const long long from = rows[r];
    for (int c = lane; c < vecs_per_row; c += 32)
      dst[r * vecs_per_row + c] = from >= 0 ? src[from * vecs_per_row + c] : make_uint4(0, 0, 0, 0);
  }
}
}  // namespace

int launch_copy_rows(const void* src, void* dst, const int32_t* rows, long long n_rows, int row_bytes,
                     cudaStream_t stream) {
  static KernelDeviceConfig config;
  int sm_count = 0;
  if (int rc = configure_kernel(config, copy_rows_kernel, 0, &sm_count, "copy_rows_kernel")) return rc;
  const long long wanted = (n_rows + 7) / 8, cap = (long long)sm_count * 8;
  const int blocks = (int)(wanted < cap ? wanted : cap);
  cudaError_t e = launch_after_predecessor(copy_rows_kernel, dim3(blocks), dim3(256), 0, stream, (const uint4*)src,
                                           (uint4*)dst, rows, n_rows, row_bytes / 16);
  if (e != cudaSuccess) return fail(DFL_ERR_LAUNCH, "copy_rows_kernel: %s", cudaGetErrorString(e));
  return check_launch("copy_rows_kernel");
}

int add_layernorm_max_hidden(size_t elem_size) { return 16 * 32 * (int)(16 / elem_size); }

namespace {
int launch_rows(const void* x, const void* residual, const void* gamma, const void* beta, void* out, long long rows,
                int hidden, float eps, int dtype, const void* row_mask, int mask_elem, void* out2,
                const int32_t* out2_rows, const RowSource& src, cudaStream_t stream) {
  static KernelDeviceConfig config;   // only the SM count of the current device is needed (no shared memory)
  int sm_count = 0;
  if (int rc = configure_kernel(config, add_layernorm_kernel<float, 1>, 0, &sm_count, "add_layernorm_kernel")) return rc;
  switch (dtype) {
    case DFL_F16: return launch_typed<__half>(x, residual, gamma, beta, out, rows, hidden, eps, row_mask, mask_elem, out2, out2_rows, src, sm_count, stream);
    case DFL_BF16: return launch_typed<__nv_bfloat16>(x, residual, gamma, beta, out, rows, hidden, eps, row_mask, mask_elem, out2, out2_rows, src, sm_count, stream);
    default: return launch_typed<float>(x, residual, gamma, beta, out, rows, hidden, eps, row_mask, mask_elem, out2, out2_rows, src, sm_count, stream);
  }
}
}  // namespace

int launch_add_layernorm(const void* x, const void* residual, const void* gamma, const void* beta, void* out,
                         long long rows, int hidden, float eps, int dtype, const void* row_mask, int mask_elem,
                         void* out2, const int32_t* out2_rows, cudaStream_t stream) {
  const RowSource plain{nullptr, nullptr, 4, 0, 0, nullptr};
  return launch_rows(x, residual, gamma, beta, out, rows, hidden, eps, dtype, row_mask, mask_elem, out2, out2_rows, plain,
                     stream);
}

// Embedding front-end: out[r] = LayerNorm(table[ids[r]] (+ pos_table[pos_ids[r]])), masked rows zero.
int launch_embed_layernorm(const void* ids, const void* table, long long vocab, const void* pos_ids,
                           const void* pos_table, long long positions, int idx_elem, const void* gamma,
                           const void* beta, void* out, long long rows, int hidden, float eps, int dtype,
                           const void* row_mask, int mask_elem, int* status, cudaStream_t stream) {
  const RowSource src{ids, pos_table ? pos_ids : nullptr, idx_elem, vocab, positions, status};
  return launch_rows(table, pos_table, gamma, beta, out, rows, hidden, eps, dtype, row_mask, mask_elem, nullptr, nullptr,
                     src, stream);
}

}  // namespace dfl
