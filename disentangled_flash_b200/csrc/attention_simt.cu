// IEEE-fp32 CUDA-core fused disentangled attention.
//
// This is the "strict FP32" implementation of the fused kernel (the reference
// runs its Triton kernel with input_precision="ieee" in that mode,
// src/disentangled_flash/kernel.py:211-217,277-283; tcgen05 offers no IEEE
// fp32 MMA kind) and, for 16-bit inputs, the cross-check path behind
// DFL_ALGO_SIMT.  Semantics follow kernel.py:137-345:
//   S[i,j] = q_i.k_j + c2p[i, lut[i-j+L-1]] + p2c[j, lut[i-j+L-1]]
//   scaled by scale*log2(e); pairs with a padded key -> -inf; a padded query
//   row -> 0 for every in-range key (uniform attention); online softmax in
//   base 2; P rounded to the input dtype before P*V for 16-bit inputs.
//
// Mapping: one thread owns one query row (running max, running sum and the d
// output accumulators live in registers), a CTA owns ROWS consecutive rows
// of one (batch, head), K/V tiles of BN keys are staged in shared memory as
// fp32 and read as warp-wide broadcasts.  [B,H,L,L] is never formed.
#include "dfl_common.cuh"

namespace dfl {
namespace {

constexpr int BN = 32;

template <typename T, int D, int ROWS>
__global__ void __launch_bounds__(ROWS)
attention_simt_kernel(DflAttnParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int QS = D + 4;  // (D+4)/4 is odd: own-row float4 reads are conflict free
  float* Qs = reinterpret_cast<float*>(smem_raw);   // [ROWS][QS]
  float* Ks = Qs + ROWS * QS;                        // [BN][D]
  float* Vs = Ks + BN * D;                           // [BN][D]
  int* keep_s = reinterpret_cast<int*>(Vs + BN * D); // [BN]
  int16_t* lut_s = reinterpret_cast<int16_t*>(keep_s + BN);  // [2L-1]

  const int L = p.seq_len, H = p.heads;
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  const int tid = threadIdx.x;
  const int i0 = blockIdx.x * ROWS;
  const int i = i0 + tid;
  const bool row_ok = i < L;
  const bool has_c2p = p.c2p != nullptr, has_p2c = p.p2c != nullptr;
  const bool has_pos = has_c2p || has_p2c;

  const T* Q = reinterpret_cast<const T*>(p.q) + (long long)bh * L * D;
  const T* K = reinterpret_cast<const T*>(p.k) + (long long)bh * L * D;
  const T* V = reinterpret_cast<const T*>(p.v) + (long long)bh * L * D;
  const T* C2P = has_c2p ? reinterpret_cast<const T*>(p.c2p) + ((long long)bh * L + (row_ok ? i : 0)) * p.ld_slots : nullptr;
  const T* P2C = has_p2c ? reinterpret_cast<const T*>(p.p2c) + (long long)bh * L * p.ld_slots : nullptr;

  // stage Q tile and LUT
  for (int e = tid; e < ROWS * D; e += ROWS) {
    const int r = e / D, dd = e % D;
    Qs[r * QS + dd] = (i0 + r < L) ? Elem<T>::to_f(Q[(long long)(i0 + r) * D + dd]) : 0.0f;
  }
  if (has_pos)
    for (int e = tid; e < 2 * L - 1; e += ROWS) lut_s[e] = (int16_t)p.lut[e];

  const bool q_keep = row_ok && mask_keep(p.mask, p.mask_elem_size, (long long)b * L + i);
  const float scale_log2 = p.scale * 1.4426950408889634f;

  float m_run = -INFINITY, l_run = 0.0f;
  float acc[D];
#pragma unroll
  for (int dd = 0; dd < D; ++dd) acc[dd] = 0.0f;

  for (int j0 = 0; j0 < L; j0 += BN) {
    __syncthreads();  // previous K/V tile consumed (and Q/LUT staged, first time)
    for (int e = tid; e < BN * D; e += ROWS) {
      const int r = e / D, dd = e % D;
      const bool ok = j0 + r < L;
      Ks[e] = ok ? Elem<T>::to_f(K[(long long)(j0 + r) * D + dd]) : 0.0f;
      Vs[e] = ok ? Elem<T>::to_f(V[(long long)(j0 + r) * D + dd]) : 0.0f;
    }
    if (tid < BN) keep_s[tid] = (j0 + tid < L) ? (int)mask_keep(p.mask, p.mask_elem_size, (long long)b * L + j0 + tid) : 0;
    __syncthreads();

    float s[BN];
#pragma unroll
    for (int jj = 0; jj < BN; ++jj) s[jj] = 0.0f;
#pragma unroll 4
    for (int d4 = 0; d4 < D; d4 += 4) {
      const float4 qv = *reinterpret_cast<const float4*>(&Qs[tid * QS + d4]);
#pragma unroll
      for (int jj = 0; jj < BN; ++jj) {
        const float4 kv = *reinterpret_cast<const float4*>(&Ks[jj * D + d4]);
        s[jj] = fmaf(qv.x, kv.x, s[jj]);
        s[jj] = fmaf(qv.y, kv.y, s[jj]);
        s[jj] = fmaf(qv.z, kv.z, s[jj]);
        s[jj] = fmaf(qv.w, kv.w, s[jj]);
      }
    }

    float tile_max = -INFINITY;
#pragma unroll
    for (int jj = 0; jj < BN; ++jj) {
      const int j = j0 + jj;
      const bool in_range = j < L;
      float v = s[jj];
      if (has_pos && row_ok && in_range) {
        const int slot = lut_s[i - j + L - 1];
        if (has_c2p) v += Elem<T>::to_f(C2P[slot]);
        if (has_p2c) v += Elem<T>::to_f(P2C[(long long)j * p.ld_slots + slot]);
      }
      v *= scale_log2;
      if (!in_range) v = -INFINITY;
      else if (!q_keep) v = 0.0f;          // padded query row: uniform over all in-range keys
      else if (!keep_s[jj]) v = -INFINITY; // padded key
      s[jj] = v;
      tile_max = fmaxf(tile_max, v);
    }

    const float m_new = fmaxf(m_run, tile_max);
    const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;  // all-masked so far: avoid inf-inf
    const float corr = exp2f(m_run - m_use);                  // m_run=-inf -> 0
    float tile_sum = 0.0f;
#pragma unroll
    for (int jj = 0; jj < BN; ++jj) {
      const float pr = exp2f(s[jj] - m_use);
      tile_sum += pr;
      s[jj] = round_through<T>(pr);
    }
    l_run = l_run * corr + tile_sum;
    m_run = m_new;
#pragma unroll
    for (int dd = 0; dd < D; ++dd) acc[dd] *= corr;
#pragma unroll
    for (int d4 = 0; d4 < D; d4 += 4) {  // fully unrolled: acc[] must stay in registers
#pragma unroll
      for (int jj = 0; jj < BN; ++jj) {
        const float4 vv = *reinterpret_cast<const float4*>(&Vs[jj * D + d4]);
        acc[d4 + 0] = fmaf(s[jj], vv.x, acc[d4 + 0]);
        acc[d4 + 1] = fmaf(s[jj], vv.y, acc[d4 + 1]);
        acc[d4 + 2] = fmaf(s[jj], vv.z, acc[d4 + 2]);
        acc[d4 + 3] = fmaf(s[jj], vv.w, acc[d4 + 3]);
      }
    }
  }

  if (row_ok) {
    const float inv = 1.0f / l_run;
    T* out = reinterpret_cast<T*>(p.out) + ((long long)b * L + i) * ((long long)H * D) + (long long)h * D;
#pragma unroll
    for (int dd = 0; dd < D; ++dd) out[dd] = Elem<T>::from_f(acc[dd] * inv);
  }
}

template <typename T, int D>
int launch_typed(const DflAttnParams& p, cudaStream_t stream) {
  constexpr int ROWS = D == 128 ? 64 : 128;
  const size_t smem = (size_t)(ROWS * (D + 4) + 2 * BN * D) * sizeof(float) + BN * sizeof(int) +
                      (size_t)(2 * p.seq_len) * sizeof(int16_t);
  auto kernel = attention_simt_kernel<T, D, ROWS>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(DFL_ERR_LAUNCH, "attention_simt smem opt-in: %s", cudaGetErrorString(e));
  }
  dim3 grid((p.seq_len + ROWS - 1) / ROWS, p.batch * p.heads);
  if (grid.y > 65535) return fail(DFL_ERR_TOO_LARGE, "batch*heads > 65535");
  kernel<<<grid, ROWS, smem, stream>>>(p);
  return check_launch("attention_simt_kernel");
}

template <typename T>
int launch_d(const DflAttnParams& p, cudaStream_t stream) {
  switch (p.head_dim) {
    case 32: return launch_typed<T, 32>(p, stream);
    case 64: return launch_typed<T, 64>(p, stream);
    case 128: return launch_typed<T, 128>(p, stream);
  }
  return fail(DFL_ERR_UNSUPPORTED, "head_dim %d not in {32,64,128}", p.head_dim);
}

}  // namespace

int launch_attention_simt(const DflAttnParams& p, cudaStream_t stream) {
  if (p.seq_len > 16384) return fail(DFL_ERR_TOO_LARGE, "seq_len %d > 16384", p.seq_len);
  if (p.dtype == DFL_F32) return launch_d<float>(p, stream);
  if (p.dtype == DFL_F16) return launch_d<__half>(p, stream);
  return launch_d<__nv_bfloat16>(p, stream);
}

}  // namespace dfl
