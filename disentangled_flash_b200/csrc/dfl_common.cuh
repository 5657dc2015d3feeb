// Shared host/device helpers for the B200 disentangled-attention library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "../../include/dfl_b200.h"

namespace dfl {

// ---------------------------------------------------------------- errors ---
// Last error detail, per host thread.  Written only on failure paths.
inline char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

inline int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return status;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DFL_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return DFL_OK;
}

// Launchers keep their one-time configuration (shared-memory opt-in, SM count, symbol addresses) per device.
constexpr int kMaxDevices = 64;

// One-time launch configuration of one kernel instance, kept per device: the opt-in to large dynamic shared
// memory is a per-device attribute of the kernel, and the grid of a persistent kernel follows the device's SM
// count.  One object per kernel instance (a function-local static of its launcher); first calls from several
// host threads are serialised.
struct KernelDeviceConfig {
  std::mutex mutex;
  int smem_opted_in[kMaxDevices] = {0};
  int sm_count[kMaxDevices] = {0};
};
template <typename Kernel>
inline int configure_kernel(KernelDeviceConfig& cfg, Kernel kernel, int smem_bytes, int* sm_count, const char* what) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(DFL_ERR_LAUNCH, "%s: current device: %s", what, cudaGetErrorString(e));
  std::lock_guard<std::mutex> lock(cfg.mutex);
  if (smem_bytes > cfg.smem_opted_in[dev]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return fail(DFL_ERR_LAUNCH, "%s: shared-memory opt-in: %s", what, cudaGetErrorString(e));
    cfg.smem_opted_in[dev] = smem_bytes;
  }
  if (cfg.sm_count[dev] == 0) {
    int count = 0;
    e = cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || count < 1) return fail(DFL_ERR_LAUNCH, "%s: SM count: %s", what, cudaGetErrorString(e));
    cfg.sm_count[dev] = count;
  }
  if (sm_count) *sm_count = cfg.sm_count[dev];
  return DFL_OK;
}

// Launch with programmatic stream serialization: the kernel's CTAs may be scheduled, and run up to their
// `griddepcontrol.wait`, while the previous kernel of the stream is still draining; everything that touches global
// memory comes after that wait, which returns when the previous kernel has completed and its writes are visible.
// This takes the launch latency and the kernel's set-up (barrier initialisation, tensor-memory allocation, descriptor
// prefetch) off the path between two dependent kernels.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_after_predecessor(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                            cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// Device side of the above: wait for the previous kernel of the stream (no-op for a plain launch).
__device__ __forceinline__ void wait_for_predecessor() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline size_t dtype_size(int dtype) { return dtype == DFL_F32 ? 4 : 2; }

// ------------------------------------------------------------ conversions ---
template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct Elem<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// Round an fp32 value through T (identity for float).
template <typename T>
__device__ __forceinline__ float round_through(float v) {
  return Elem<T>::to_f(Elem<T>::from_f(v));
}

// Non-zero test of one mask element of 1, 4 or 8 bytes.
__device__ __forceinline__ bool mask_keep(const void* mask, int elem_size, long long idx) {
  if (elem_size == 1) return reinterpret_cast<const uint8_t*>(mask)[idx] != 0;
  if (elem_size == 4) return reinterpret_cast<const uint32_t*>(mask)[idx] != 0;
  return reinterpret_cast<const unsigned long long*>(mask)[idx] != 0ull;
}

// ------------------------------------------------- kernel launch wrappers ---
// One function per kernel family; defined in the matching .cu file.
int launch_position_lut(int L, int buckets, int max_pos, int span, int uses_bias, int32_t* lut,
                        int64_t* active, int32_t* n_active, cudaStream_t stream);
int launch_gather_slots(const void* src, const int64_t* active, void* dst, int heads, int n_src,
                        int n_active, int d, int dtype, cudaStream_t stream);

// Generic batched "NT" GEMM description used by both GEMM families:
//   C_z[m, n] = sum_k X_z[m, k] * W_{z % w_mod}[n, k] (+ bias[n])
// with either a head-split epilogue (QKV / position projection) or a plain
// row-major epilogue with leading dimension ldc (position scores).
struct GemmDesc {
  const void* x;
  const void* w;
  const void* bias;
  void* out[3];
  int M, N, K;
  int batch;            // grid.z
  long long stride_x;   // elements between X_z
  long long stride_w;   // elements between W_z'
  int w_mod;            // W index = z % w_mod
  long long stride_c;   // elements between C_z (row-major epilogue)
  int ldc;              // row-major epilogue leading dimension; columns [N, ldc) zero-filled
  int head_split;       // 1: head-split epilogue, 0: row-major
  int heads, head_dim, rows_per_seq;
  int dtype;
  int* status;          // device status word of the call, or null (the tcgen05 GEMM then uses the library's word)
  int activation;       // DFL_ACT_*: applied after the bias (row-major epilogue only)
  // 1-D convolution as a GEMM over taps (tensor-core pair kernel only): k-step (tap, kb) multiplies rows
  // m + tap - taps/2 of X_z (rows outside [0, M) read as zero: 'same' padding) with weight matrix W[tap].
  int taps;             // 0 or 1: plain GEMM
  const void* row_mask; // [batch, M] or null: output rows whose element is zero are set to 0 before the activation
  int row_mask_elem;    // element size of row_mask: 1, 4 or 8 bytes
  // Packed input rows (head-split epilogue of the tensor-core kernels only): rows 32g .. 32g+31 of X are written to
  // rows row_groups[g] .. +31 of the [out_seqs * rows_per_seq] output row space.  Null: row m goes to row m.
  const int* row_groups;
  int out_seqs;         // sequences of the output tensors when row_groups is set (else M / rows_per_seq)
};

// tanh for the GEMM epilogues of 16-bit outputs: 1 - 2 / (1 + e^(2x)) with approximate exp2 and reciprocal
// (absolute error ~1e-7; exact limits +-1).
__device__ __forceinline__ float tanh_fast(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * 2.8853900817779268f));   // 2 log2(e)
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return fmaf(-2.0f, r, 1.0f);
}

// GELU, 0.5 x (1 + erf(x / sqrt 2)), for the GEMM epilogues.
// Exact form (strict FP32 kernels): the CUDA library's erff.
__device__ __forceinline__ float gelu_erf_exact(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }
// Fast form (16-bit outputs): erf by the rational approximation 7.1.26 of Abramowitz & Stegun,
// erf(z) = 1 - (a1 t + ... + a5 t^5) exp(-z^2), t = 1 / (1 + p z), z >= 0, absolute error below 1.5e-7 - three
// orders of magnitude under the rounding step of an FP16 or BF16 output - with one approximate reciprocal and one
// approximate exp2 (relative error ~1e-7 each).
__device__ __forceinline__ float gelu_erf_fast(float x) {
  // gelu(x) = max(x, 0) - |x| * q(t) * exp(-z^2),  z = |x| / sqrt 2,  q(t) = 0.5 (a1 t + ... + a5 t^5).
  // With w = z * sqrt(log2 e): exp(-z^2) = exp2(-w^2) and 1 + p z = 1 + (p / sqrt(log2 e)) w.
  const float ax = fabsf(x);
  const float w = ax * 0.84932180028801904f;            // sqrt(log2(e) / 2)
  float t, e;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.27273748088f, w, 1.0f)));   // p / sqrt(log2 e)
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-w * w));
  float q = fmaf(0.5307027145f, t, -0.7265760135f);      // a5 / 2, a4 / 2
  q = fmaf(q, t, 0.7107068705f);                          // a3 / 2
  q = fmaf(q, t, -0.142248368f);                          // a2 / 2
  q = fmaf(q, t, 0.127414796f);                           // a1 / 2
  return fmaf(-(ax * (q * t)), e, fmaxf(x, 0.0f));
}
int launch_gemm_simt(const GemmDesc& g, cudaStream_t stream);
int launch_gemm_tc(const GemmDesc& g, cudaStream_t stream);

int launch_attention_simt(const DflAttnParams& p, cudaStream_t stream);
int launch_attention_tc(const DflAttnParams& p, cudaStream_t stream);
bool attention_rel_supported(const DflAttnRelParams& p);
int launch_attention_rel(const DflAttnRelParams& p, cudaStream_t stream);
int add_layernorm_max_hidden(size_t elem_size);
int launch_add_layernorm(const void* x, const void* residual, const void* gamma, const void* beta, void* out,
                         long long rows, int hidden, float eps, int dtype, const void* row_mask, int mask_elem,
                         void* out2, const int32_t* out2_rows, cudaStream_t stream);
int launch_embed_layernorm(const void* ids, const void* table, long long vocab, const void* pos_ids,
                           const void* pos_table, long long positions, int idx_elem, const void* gamma,
                           const void* beta, void* out, long long rows, int hidden, float eps, int dtype,
                           const void* row_mask, int mask_elem, int* status, cudaStream_t stream);
int launch_copy_rows(const void* src, void* dst, const int32_t* rows, long long n_rows, int row_bytes,
                     cudaStream_t stream);
int launch_selftest_bounded_wait(int* status, uint32_t limit_us, cudaStream_t stream);
int launch_expand_rel_tables(const void* pos, const int32_t* lut, void* rel, int heads, int n_active, int seq_len,
                             int head_dim, int dtype, cudaStream_t stream);

}  // namespace dfl
