// IEEE-fp32 CUDA-core GEMM family ("strict FP32" path, and the cross-check
// path for 16-bit inputs).
//
// Replaces, for float32 models, the library GEMMs the reference issues with
// TF32 disabled: F.linear for the fused QKV projection (_torch.py:292-296),
// the relative-embedding projections (_torch.py:146-158) and the two
// position-score matmuls (kernel.py:577,583).  tcgen05 has no IEEE-fp32 MMA
// kind, so strict fp32 is FFMA work; its roofline is the fp32 CUDA-core rate.
//
// C_z[m,n] = sum_k X_z[m,k] * W_{z % w_mod}[n,k] (+ bias[n]), fp32 accumulate.
// Tile 128x128x16 (long inner products) or 64x64x16, 256 threads, 8x8 or 4x4 outputs per thread (4-wide groups of
// rows and of columns, 64 apart), operands staged in shared memory as fp32 with the k index outermost so that the
// inner product reads conflict-free float4 (four per k for 64 FMAs with the large tile); the next k-block is fetched from global memory into registers while the current one
// is multiplied.  Every output accumulates its products in ascending k with one fmaf each.
#include "dfl_common.cuh"

namespace dfl {
namespace {

constexpr int BK = 16, PAD = 4;

template <typename T>
__device__ __forceinline__ void load4(const T* p, bool vec_ok, int valid, float (&v)[4]) {
  // Loads up to 4 consecutive elements starting at p (valid in [0,4]).
  if (valid == 4 && vec_ok) {
    if constexpr (sizeof(T) == 4) {
      float4 f = *reinterpret_cast<const float4*>(p);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
      uint2 raw = *reinterpret_cast<const uint2*>(p);
      const T* h = reinterpret_cast<const T*>(&raw);
      v[0] = Elem<T>::to_f(h[0]); v[1] = Elem<T>::to_f(h[1]);
      v[2] = Elem<T>::to_f(h[2]); v[3] = Elem<T>::to_f(h[3]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = i < valid ? Elem<T>::to_f(p[i]) : 0.0f;
  }
}

// G = 4-wide groups of rows and of columns per thread: tile 64*G x 64*G, (4*G)^2 outputs per thread.
template <typename T, int G>
__global__ void __launch_bounds__(256, G > 1 ? 2 : 5)
gemm_simt_kernel(GemmDesc g) {
  constexpr int BM = 64 * G, BN = 64 * G, R = 4 * G;
  __shared__ float As[BK][BM + PAD];
  __shared__ float Bs[BK][BN + PAD];

  const int z = blockIdx.z;
  const T* X = reinterpret_cast<const T*>(g.x) + (long long)z * g.stride_x;
  const T* W = reinterpret_cast<const T*>(g.w) + (long long)(z % g.w_mod) * g.stride_w;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tid = threadIdx.x;
  const int ty = tid / 16, tx = tid % 16;

  // loader mapping: two 4-element k-runs (rows lrow and lrow + 64) per thread, for A and for B
  const int lrow = tid / 4, lk = (tid % 4) * 4;
  // vector loads need K % 4 == 0 (row starts stay aligned) and an aligned base
  const bool vec_ok = (g.K % 4 == 0) && ((reinterpret_cast<uintptr_t>(X) % (4 * sizeof(T))) == 0) &&
                      ((reinterpret_cast<uintptr_t>(W) % (4 * sizeof(T))) == 0);

  float acc[R][R];
#pragma unroll
  for (int i = 0; i < R; ++i)
#pragma unroll
    for (int j = 0; j < R; ++j) acc[i][j] = 0.0f;

  float a[G][4], b[G][4];
  auto fetch = [&](int k0) {
    const int kk = k0 + lk;
    const int kvalid = g.K - kk < 0 ? 0 : (g.K - kk > 4 ? 4 : g.K - kk);
#pragma unroll
    for (int h = 0; h < G; ++h) {
      const int am = m0 + lrow + 64 * h, bn = n0 + lrow + 64 * h;
      load4<T>(X + (long long)am * g.K + kk, vec_ok, am < g.M ? kvalid : 0, a[h]);
      load4<T>(W + (long long)bn * g.K + kk, vec_ok, bn < g.N ? kvalid : 0, b[h]);
    }
  };
  // the large tile fetches the next k-block while it multiplies; the small tile, used for short inner products,
  // keeps its registers for occupancy instead
  constexpr bool kPrefetch = G > 1;
  if (kPrefetch) fetch(0);
  for (int k0 = 0; k0 < g.K; k0 += BK) {
    if (!kPrefetch) fetch(k0);
    __syncthreads();  // previous tile fully consumed
#pragma unroll
    for (int h = 0; h < G; ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        As[lk + i][lrow + 64 * h] = a[h][i];
        Bs[lk + i][lrow + 64 * h] = b[h][i];
      }
    __syncthreads();
    if (kPrefetch && k0 + BK < g.K) fetch(k0 + BK);   // in flight during the multiply
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float ar[R], br[R];
#pragma unroll
      for (int h = 0; h < G; ++h) {
        const float4 av = *reinterpret_cast<const float4*>(&As[k][64 * h + ty * 4]);
        const float4 bv = *reinterpret_cast<const float4*>(&Bs[k][64 * h + tx * 4]);
        ar[4 * h] = av.x; ar[4 * h + 1] = av.y; ar[4 * h + 2] = av.z; ar[4 * h + 3] = av.w;
        br[4 * h] = bv.x; br[4 * h + 1] = bv.y; br[4 * h + 2] = bv.z; br[4 * h + 3] = bv.w;
      }
#pragma unroll
      for (int i = 0; i < R; ++i)
#pragma unroll
        for (int j = 0; j < R; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
    }
  }

  // epilogue: rows ty*4 + i and 64 + ty*4 + i, columns tx*4 + j and 64 + tx*4 + j
  const T* bias = reinterpret_cast<const T*>(g.bias);
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int m = m0 + (i >> 2) * 64 + ty * 4 + (i & 3);
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const int n = n0 + (j >> 2) * 64 + tx * 4 + (j & 3);
      if (g.head_split) {
        if (n >= g.N) continue;
        float v = acc[i][j];
        if (bias) v += Elem<T>::to_f(bias[n]);
        const int hd = g.heads * g.head_dim;
        const int which = n / hd, rem = n % hd;
        const int h = rem / g.head_dim, dd = rem % g.head_dim;
        const int b_ = m / g.rows_per_seq, l = m % g.rows_per_seq;
        T* out = reinterpret_cast<T*>(g.out[which]);
        out[(((long long)b_ * g.heads + h) * g.rows_per_seq + l) * g.head_dim + dd] = Elem<T>::from_f(v);
      } else {
        if (n >= g.ldc) continue;
        float v = n < g.N ? acc[i][j] : 0.0f;
        if (bias && n < g.N) v += Elem<T>::to_f(bias[n]);
        if (g.activation == DFL_ACT_GELU) v = gelu_erf_exact(v);
        T* out = reinterpret_cast<T*>(g.out[0]) + (long long)z * g.stride_c;
        out[(long long)m * g.ldc + n] = Elem<T>::from_f(v);
      }
    }
  }
}

}  // namespace

template <int G>
int launch_tiles(const GemmDesc& g, cudaStream_t stream) {
  const int ncols = g.head_split ? g.N : g.ldc;
  constexpr int TILE = 64 * G;
  dim3 grid((ncols + TILE - 1) / TILE, (g.M + TILE - 1) / TILE, g.batch);
  if (grid.y > 65535 || grid.z > 65535) return fail(DFL_ERR_TOO_LARGE, "gemm_simt grid too large");
  if (g.dtype == DFL_F32) gemm_simt_kernel<float, G><<<grid, 256, 0, stream>>>(g);
  else if (g.dtype == DFL_F16) gemm_simt_kernel<__half, G><<<grid, 256, 0, stream>>>(g);
  else gemm_simt_kernel<__nv_bfloat16, G><<<grid, 256, 0, stream>>>(g);
  return check_launch("gemm_simt_kernel");
}

int launch_gemm_simt(const GemmDesc& g, cudaStream_t stream) {
  // 128 x 128 tiles for long inner products (the projections), 64 x 64 for the short ones (position scores, K = d)
  // and for outputs too small to give every SM two of the large tiles (296 on a 148-SM part)
  const long long big_tiles = (long long)((g.M + 127) / 128) * (((g.head_split ? g.N : g.ldc) + 127) / 128) * g.batch;
  return g.K >= 256 && big_tiles >= 296 ? launch_tiles<2>(g, stream) : launch_tiles<1>(g, stream);
}

}  // namespace dfl
