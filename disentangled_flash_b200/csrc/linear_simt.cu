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
// Tile 64x64x16, 256 threads, 4x4 outputs per thread, operands staged in
// shared memory as fp32 with the k index outermost so that the inner product
// reads two conflict-free float4 per k.
#include "dfl_common.cuh"

namespace dfl {
namespace {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

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

template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(GemmDesc g) {
  __shared__ float As[BK][BM + PAD];
  __shared__ float Bs[BK][BN + PAD];

  const int z = blockIdx.z;
  const T* X = reinterpret_cast<const T*>(g.x) + (long long)z * g.stride_x;
  const T* W = reinterpret_cast<const T*>(g.w) + (long long)(z % g.w_mod) * g.stride_w;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tid = threadIdx.x;
  const int ty = tid / 16, tx = tid % 16;

  // loader mapping: one 4-element k-run of one row per thread, for A and for B
  const int lrow = tid / 4, lk = (tid % 4) * 4;
  // vector loads need K % 4 == 0 (row starts stay aligned) and an aligned base
  const bool vec_ok = (g.K % 4 == 0) && ((reinterpret_cast<uintptr_t>(X) % (4 * sizeof(T))) == 0) &&
                      ((reinterpret_cast<uintptr_t>(W) % (4 * sizeof(T))) == 0);

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < g.K; k0 += BK) {
    float a[4], b[4];
    const int kk = k0 + lk;
    const int kvalid = g.K - kk < 0 ? 0 : (g.K - kk > 4 ? 4 : g.K - kk);
    const int am = m0 + lrow, bn = n0 + lrow;
    load4<T>(X + (long long)am * g.K + kk, vec_ok, am < g.M ? kvalid : 0, a);
    load4<T>(W + (long long)bn * g.K + kk, vec_ok, bn < g.N ? kvalid : 0, b);
    __syncthreads();  // previous tile fully consumed
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      As[lk + i][lrow] = a[i];
      Bs[lk + i][lrow] = b[i];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 bv = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
      const float ar[4] = {av.x, av.y, av.z, av.w};
      const float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
    }
  }

  // epilogue
  const T* bias = reinterpret_cast<const T*>(g.bias);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (g.head_split) {
        if (n >= g.N) continue;
        float v = acc[i][j];
        if (bias) v += Elem<T>::to_f(bias[n]);
        const int hd = g.heads * g.head_dim;
        const int which = n / hd, rem = n % hd;
        const int h = rem / g.head_dim, dd = rem % g.head_dim;
        const int b = m / g.rows_per_seq, l = m % g.rows_per_seq;
        T* out = reinterpret_cast<T*>(g.out[which]);
        out[(((long long)b * g.heads + h) * g.rows_per_seq + l) * g.head_dim + dd] = Elem<T>::from_f(v);
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

int launch_gemm_simt(const GemmDesc& g, cudaStream_t stream) {
  const int ncols = g.head_split ? g.N : g.ldc;
  dim3 grid((ncols + BN - 1) / BN, (g.M + BM - 1) / BM, g.batch);
  if (grid.y > 65535 || grid.z > 65535) return fail(DFL_ERR_TOO_LARGE, "gemm_simt grid too large");
  if (g.dtype == DFL_F32) gemm_simt_kernel<float><<<grid, 256, 0, stream>>>(g);
  else if (g.dtype == DFL_F16) gemm_simt_kernel<__half><<<grid, 256, 0, stream>>>(g);
  else gemm_simt_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(g);
  return check_launch("gemm_simt_kernel");
}

}  // namespace dfl
