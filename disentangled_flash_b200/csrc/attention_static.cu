// Allocation-free variant of the relative-score + fused-attention step.
//
// The regular path computes the C2P/P2C score tensors into buffers that the caller allocates
// (dfl_pos_scores) and then consumes them (dfl_attention_fwd).  Some callers have no allocator to
// give: a serving process that handed the whole device to its own arena at start-up, or a plug-in
// invoked from a host runtime's callback where cudaMalloc (which synchronises the device) is not
// allowed.  For them this entry point keeps the score tensors in a fixed array that lives in the
// library's device image, so the call itself performs no allocation of any kind.
#include <mutex>

#include "dfl_common.cuh"

namespace dfl {
namespace {

constexpr size_t kStaticScratchBytes = DFL_STATIC_SCRATCH_BYTES;

// Lives in every CUDA context that loads the library, until the context is destroyed.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle: the device address has to be asked for, once per
// device, while that device is current.  The address is cached for the life of the process: it stays valid
// until the device's context is destroyed (after cudaDeviceReset the library must be reloaded).
std::mutex g_setup_mutex;
unsigned char* g_scratch_addr[kMaxDevices] = {nullptr};

int scratch_for_current_device(unsigned char** out) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail(DFL_ERR_LAUNCH, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (device < 0 || device >= kMaxDevices) return fail(DFL_ERR_TOO_LARGE, "device ordinal %d >= %d", device, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_addr[device]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || !ptr)
      return fail(DFL_ERR_LAUNCH, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
    g_scratch_addr[device] = static_cast<unsigned char*>(ptr);
  }
  *out = g_scratch_addr[device];
  return DFL_OK;
}

}  // namespace
}  // namespace dfl

using namespace dfl;

extern "C" {

size_t dfl_static_scratch_bytes(void) { return kStaticScratchBytes; }

int dfl_attention_fwd_static(const DflAttnTablesParams* p, void* stream) {
  if (!p) return fail(DFL_ERR_BAD_ARG, "null params");
  // Everything that bounds the scratch size is checked before the size is computed, so that the product below
  // cannot wrap: batch*heads <= 2^16, seq_len <= 2^14, slots <= 2^15, 4 bytes -> below 2^47.
  if (p->dtype != DFL_F16 && p->dtype != DFL_BF16 && p->dtype != DFL_F32) return fail(DFL_ERR_BAD_ARG, "unknown dtype %d", p->dtype);
  if (p->head_dim != 32 && p->head_dim != 64 && p->head_dim != 128)
    return fail(DFL_ERR_UNSUPPORTED, "head_dim %d not in {32,64,128}", p->head_dim);
  if (p->batch < 1 || p->heads < 1 || p->seq_len < 1) return fail(DFL_ERR_BAD_ARG, "non-positive size");
  if (p->seq_len > 16384) return fail(DFL_ERR_TOO_LARGE, "seq_len %d > 16384", p->seq_len);
  if ((long long)p->batch * p->heads > 65535) return fail(DFL_ERR_TOO_LARGE, "batch*heads > 65535");
  const bool has_c2p = p->pos_key != nullptr, has_p2c = p->pos_query != nullptr;
  if ((has_c2p || has_p2c) && p->n_active < 1) return fail(DFL_ERR_BAD_ARG, "n_active must be positive");
  if ((has_c2p || has_p2c) && p->n_active > 2 * p->seq_len)
    return fail(DFL_ERR_BAD_ARG, "n_active %d exceeds the 2*seq_len relative distances", p->n_active);

  const unsigned long long es = p->dtype == DFL_F32 ? 4 : 2;
  const int ld = has_c2p || has_p2c ? (p->n_active + 7) / 8 * 8 : 0;
  unsigned long long one = (unsigned long long)p->batch * (unsigned long long)p->heads * (unsigned long long)p->seq_len *
                           (unsigned long long)ld * es;
  one = (one + 255) / 256 * 256;
  const unsigned long long need = one * ((has_c2p ? 1 : 0) + (has_p2c ? 1 : 0));
  if (need > kStaticScratchBytes)
    return fail(DFL_ERR_TOO_LARGE,
                "relative-score scratch of %llu bytes exceeds the built-in %zu bytes; "
                "use dfl_pos_scores + dfl_attention_fwd with caller-provided buffers",
                need, kStaticScratchBytes);

  unsigned char* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != DFL_OK) return rc;
  void* c2p = has_c2p ? scratch : nullptr;
  void* p2c = has_p2c ? scratch + (has_c2p ? one : 0) : nullptr;

  if (has_c2p || has_p2c) {
    DflPosScoreParams s{};
    s.q = has_c2p ? p->q : nullptr;
    s.k = has_p2c ? p->k : nullptr;
    s.pos_key = p->pos_key;
    s.pos_query = p->pos_query;
    s.c2p = c2p;
    s.p2c = p2c;
    s.batch = p->batch; s.heads = p->heads; s.seq_len = p->seq_len; s.head_dim = p->head_dim;
    s.n_active = p->n_active; s.ld_slots = ld; s.dtype = p->dtype; s.algo = p->algo;
    rc = dfl_pos_scores(&s, stream);  // every element of the used region, padding columns included, is rewritten
    if (rc != DFL_OK) return rc;
  }
  DflAttnParams a{};
  a.q = p->q; a.k = p->k; a.v = p->v; a.c2p = c2p; a.p2c = p2c; a.lut = p->lut; a.mask = p->mask;
  a.out = p->out; a.status = p->status;
  a.batch = p->batch; a.heads = p->heads; a.seq_len = p->seq_len; a.head_dim = p->head_dim;
  a.ld_slots = ld; a.mask_elem_size = p->mask_elem_size; a.scale = p->scale; a.dtype = p->dtype; a.algo = p->algo;
  return dfl_attention_fwd(&a, stream);
}

}  // extern "C"
