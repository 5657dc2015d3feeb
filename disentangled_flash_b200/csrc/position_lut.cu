// Relative-position index builder and active-slot gather (prepare-time kernels).
//
// Reference behaviour reproduced bit for bit:
//   make_log_bucket_position        src/disentangled_flash/_reference.py:115-136
//   SharedPositionPlanCache.compact src/disentangled_flash/position.py:89-128
//   _project_active_positions       src/disentangled_flash/_torch.py:171-186
//
// The reference computes the bucket of every delta in float32 on the CPU,
// clamps it into [0, 2*span), and derives the pruned slot list with
// unique() + searchsorted().  The global slot is a monotone non-decreasing
// function of delta (identity near zero, ceil(log) beyond, clamp at both
// ends), so unique()+searchsorted() is exactly "count the slot changes to the
// left of delta": one block-wide prefix sum, no sort.
#include "dfl_common.cuh"

namespace dfl {
namespace {

// float32 steps of the reference formula.  log() is taken in double and
// rounded to float: that is the correctly rounded float32 logarithm, which is
// what a <=1-ulp CPU logf agrees with everywhere the ceil() argument is not
// within an ulp of an integer.  The one exact-integer case, |delta| ==
// max_position-1, has numerator == denominator and yields exactly 1.0f.
__device__ __forceinline__ long long bucket_of(long long delta, int bucket_size, int max_position) {
  const int mid = bucket_size / 2;
  const bool inside = (delta < mid) && (delta > -mid);
  const long long abs_pos = inside ? (long long)(mid - 1) : (delta < 0 ? -delta : delta);
  if (abs_pos <= mid) return delta;
  const float ratio = __fdiv_rn((float)abs_pos, (float)mid);
  const float denom_arg = (float)((double)(max_position - 1) / (double)mid);
  const float lg = (float)log((double)ratio);
  const float den = (float)log((double)denom_arg);
  float q = __fdiv_rn(lg, den);
  q = __fmul_rn(q, (float)(mid - 1));
  const float log_pos = __fadd_rn(ceilf(q), (float)mid);
  const float sign = delta > 0 ? 1.0f : -1.0f;
  return (long long)(__fmul_rn(log_pos, sign));
}

__device__ __forceinline__ int global_slot(int t, int L, int buckets, int max_pos, int span) {
  long long delta = (long long)t - (L - 1);
  if (buckets > 0) delta = bucket_of(delta, buckets, max_pos);
  long long g = delta + span;
  const long long hi = 2ll * span - 1;
  g = g < 0 ? 0 : (g > hi ? hi : g);
  return (int)g;
}

constexpr int kLutThreads = 1024;

__global__ void __launch_bounds__(kLutThreads)
build_position_lut_kernel(int L, int buckets, int max_pos, int span, int uses_bias,
                          int32_t* __restrict__ lut, int64_t* __restrict__ active,
                          int32_t* __restrict__ n_active) {
  const int n = 2 * L - 1;
  const int tid = threadIdx.x;
  if (!uses_bias) {
    for (int t = tid; t < n; t += kLutThreads) lut[t] = 0;
    if (tid == 0) *n_active = 0;
    return;
  }
  __shared__ int warp_sums[kLutThreads / 32];
  __shared__ int carry_s;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < n; base += kLutThreads) {
    const int t = base + tid;
    int g = -1, flag = 0;
    if (t < n) {
      g = global_slot(t, L, buckets, max_pos, span);
      flag = (t == 0) || (g != global_slot(t - 1, L, buckets, max_pos, span));
    }
    // inclusive block scan of flag
    int v = flag;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      int u = __shfl_up_sync(0xffffffffu, v, off);
      if ((tid & 31) >= off) v += u;
    }
    if ((tid & 31) == 31) warp_sums[tid >> 5] = v;
    __syncthreads();
    if (tid < 32) {
      int w = warp_sums[tid];
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        int u = __shfl_up_sync(0xffffffffu, w, off);
        if (tid >= off) w += u;
      }
      warp_sums[tid] = w;
    }
    __syncthreads();
    const int warp_prefix = (tid >> 5) ? warp_sums[(tid >> 5) - 1] : 0;
    const int carry = carry_s;
    const int local = carry + warp_prefix + v - 1;
    if (t < n) {
      lut[t] = local;
      if (flag) active[local] = (int64_t)g;
    }
    __syncthreads();
    if (tid == 0) carry_s = carry + warp_sums[kLutThreads / 32 - 1];
    __syncthreads();
  }
  if (tid == 0) *n_active = carry_s;
}

template <typename T>
__global__ void gather_slots_kernel(const T* __restrict__ src, const int64_t* __restrict__ active,
                                    T* __restrict__ dst, int heads, int n_src, int n_active, int d) {
  const long long total = (long long)heads * n_active * d;
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    const int dd = (int)(e % d);
    const long long r = e / d;
    const int a = (int)(r % n_active);
    const int h = (int)(r / n_active);
    const long long s = active[a];
    dst[e] = src[((long long)h * n_src + s) * d + dd];
  }
}

}  // namespace

int launch_position_lut(int L, int buckets, int max_pos, int span, int uses_bias, int32_t* lut,
                        int64_t* active, int32_t* n_active, cudaStream_t stream) {
  build_position_lut_kernel<<<1, kLutThreads, 0, stream>>>(L, buckets, max_pos, span, uses_bias, lut,
                                                           active, n_active);
  return check_launch("build_position_lut_kernel");
}

int launch_gather_slots(const void* src, const int64_t* active, void* dst, int heads, int n_src,
                        int n_active, int d, int dtype, cudaStream_t stream) {
  const long long total = (long long)heads * n_active * d;
  if (total == 0) return DFL_OK;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 1184 ? (total + threads - 1) / threads : 1184);
  if (dtype == DFL_F32) {
    gather_slots_kernel<float><<<blocks, threads, 0, stream>>>((const float*)src, active, (float*)dst,
                                                               heads, n_src, n_active, d);
  } else {
    // fp16 and bf16 are both moved as opaque 16-bit words
    gather_slots_kernel<uint16_t><<<blocks, threads, 0, stream>>>(
        (const uint16_t*)src, active, (uint16_t*)dst, heads, n_src, n_active, d);
  }
  return check_launch("gather_slots_kernel");
}

}  // namespace dfl
