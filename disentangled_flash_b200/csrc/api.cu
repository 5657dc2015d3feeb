// extern "C" entry points: argument validation and dispatch only.
#include "dfl_common.cuh"

using namespace dfl;

namespace {

bool valid_dtype(int d) { return d == DFL_F16 || d == DFL_BF16 || d == DFL_F32; }
bool valid_head_dim(int d) { return d == 32 || d == 64 || d == 128; }
bool use_tensor_cores(int dtype, int algo) { return algo == DFL_ALGO_AUTO && dtype != DFL_F32; }

}  // namespace

extern "C" {

int dfl_version(void) { return 100; }

const char* dfl_status_string(int status) {
  switch (status) {
    case DFL_OK: return "ok";
    case DFL_ERR_BAD_ARG: return "bad argument";
    case DFL_ERR_UNSUPPORTED: return "unsupported configuration";
    case DFL_ERR_ALIGNMENT: return "pointer or leading dimension not 16-byte aligned";
    case DFL_ERR_LAUNCH: return "CUDA launch failed";
    case DFL_ERR_DRIVER: return "CUDA driver call failed";
    case DFL_ERR_DEVICE_TIMEOUT: return "device-side bounded wait expired";
    case DFL_ERR_TOO_LARGE: return "size beyond supported maximum";
  }
  return "unknown status";
}

const char* dfl_last_error(void) { return last_error_buffer(); }

int dfl_check_status(int32_t* status_dev, void* stream) {
  if (!status_dev) return fail(DFL_ERR_BAD_ARG, "null status word");
  cudaStream_t s = (cudaStream_t)stream;
  int32_t code = 0;
  cudaError_t e = cudaMemcpyAsync(&code, status_dev, sizeof(code), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return fail(DFL_ERR_LAUNCH, "reading the status word: %s", cudaGetErrorString(e));
  if (code == 0) return DFL_OK;
  e = cudaMemsetAsync(status_dev, 0, sizeof(code), s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return fail(DFL_ERR_LAUNCH, "clearing the status word: %s", cudaGetErrorString(e));
  if (code == 98)   // dfl_embed_layernorm: the one code that is not a wait
    return fail(DFL_ERR_BAD_ARG, "an embedding index was outside its table (that row was read as zeros)");
  return fail(DFL_ERR_DEVICE_TIMEOUT, "a bounded device-side wait expired (wait code %d); outputs since the last check are invalid",
              (int)code);
}

int dfl_selftest_bounded_wait(int32_t* status_dev, uint32_t limit_us, void* stream) {
  if (!status_dev) return fail(DFL_ERR_BAD_ARG, "null status word");
  if (limit_us < 1 || limit_us > 100000) return fail(DFL_ERR_BAD_ARG, "limit_us must be in 1..100000");
  return launch_selftest_bounded_wait(status_dev, limit_us, (cudaStream_t)stream);
}

int dfl_build_position_lut(int seq_len, int position_buckets, int max_relative_positions, int span,
                           int uses_position_bias, int32_t* lut_dev, int64_t* active_dev,
                           int32_t* n_active_dev, void* stream) {
  if (seq_len < 1) return fail(DFL_ERR_BAD_ARG, "sequence_length must be positive");
  if (!lut_dev || !n_active_dev) return fail(DFL_ERR_BAD_ARG, "null output pointer");
  if (uses_position_bias) {
    if (!active_dev) return fail(DFL_ERR_BAD_ARG, "null active_slots pointer");
    if (span < 1) return fail(DFL_ERR_BAD_ARG, "span must be positive");
    if (position_buckets == 1) return fail(DFL_ERR_BAD_ARG, "position_buckets == 1 has no valid bucket map");
    if (position_buckets > 1 && max_relative_positions - 1 <= position_buckets / 2)
      return fail(DFL_ERR_BAD_ARG, "max_relative_positions-1 must exceed position_buckets/2");
  }
  if (seq_len > (1 << 20)) return fail(DFL_ERR_TOO_LARGE, "sequence_length > 2^20");
  return launch_position_lut(seq_len, position_buckets, max_relative_positions, span,
                             uses_position_bias, lut_dev, active_dev, n_active_dev,
                             (cudaStream_t)stream);
}

int dfl_gather_slots(const void* src, const int64_t* active_dev, void* dst, int heads,
                     int n_slots_src, int n_active, int head_dim, int dtype, void* stream) {
  if (!valid_dtype(dtype)) return fail(DFL_ERR_BAD_ARG, "unknown dtype %d", dtype);
  if (heads < 1 || n_slots_src < 1 || n_active < 0 || head_dim < 1)
    return fail(DFL_ERR_BAD_ARG, "non-positive size");
  if (n_active == 0) return DFL_OK;
  if (!src || !active_dev || !dst) return fail(DFL_ERR_BAD_ARG, "null pointer");
  return launch_gather_slots(src, active_dev, dst, heads, n_slots_src, n_active, head_dim, dtype,
                             (cudaStream_t)stream);
}

int dfl_qkv_proj(const DflLinearParams* p, void* stream) {
  if (!p) return fail(DFL_ERR_BAD_ARG, "null params");
  if (!valid_dtype(p->dtype)) return fail(DFL_ERR_BAD_ARG, "unknown dtype %d", p->dtype);
  if (p->n_out < 1 || p->n_out > 3) return fail(DFL_ERR_BAD_ARG, "n_out must be 1..3");
  if (p->M < 1 || p->K < 1 || p->heads < 1 || p->rows_per_seq < 1)
    return fail(DFL_ERR_BAD_ARG, "non-positive size");
  if (!valid_head_dim(p->head_dim))
    return fail(DFL_ERR_UNSUPPORTED, "head_dim %d not in {32,64,128}", p->head_dim);
  if (p->row_groups) {
    // packed rows: groups of 32 input rows with their destination rows; the kernels read one entry per 32 rows
    if (p->M % 32 || p->rows_per_seq % 32) return fail(DFL_ERR_BAD_ARG, "row_groups need M and rows_per_seq in multiples of 32");
    if (p->out_seqs < 1) return fail(DFL_ERR_BAD_ARG, "row_groups need out_seqs >= 1");
    if (!use_tensor_cores(p->dtype, p->algo))
      return fail(DFL_ERR_UNSUPPORTED, "row_groups are served by the tensor-core kernels only (FP16/BF16)");
  } else if (p->M % p->rows_per_seq) {
    return fail(DFL_ERR_BAD_ARG, "M not a multiple of rows_per_seq");
  }
  if (!p->x || !p->w) return fail(DFL_ERR_BAD_ARG, "null input pointer");
  if (!aligned16(p->x) || !aligned16(p->w)) return fail(DFL_ERR_ALIGNMENT, "x/w not 16-byte aligned");
  for (int o = 0; o < p->n_out; ++o) {
    if (!p->out[o]) return fail(DFL_ERR_BAD_ARG, "null output pointer %d", o);
    if (!aligned16(p->out[o])) return fail(DFL_ERR_ALIGNMENT, "output %d not 16-byte aligned", o);
  }
  GemmDesc g{};
  g.x = p->x; g.w = p->w; g.bias = p->bias;
  for (int o = 0; o < 3; ++o) g.out[o] = o < p->n_out ? p->out[o] : nullptr;
  g.M = p->M; g.N = p->n_out * p->heads * p->head_dim; g.K = p->K;
  g.batch = 1; g.stride_x = 0; g.stride_w = 0; g.w_mod = 1; g.stride_c = 0; g.ldc = g.N;
  g.head_split = 1; g.heads = p->heads; g.head_dim = p->head_dim; g.rows_per_seq = p->rows_per_seq;
  g.dtype = p->dtype;
  g.status = p->status;
  g.row_groups = p->row_groups; g.out_seqs = p->out_seqs;
  if (use_tensor_cores(p->dtype, p->algo)) return launch_gemm_tc(g, (cudaStream_t)stream);
  return launch_gemm_simt(g, (cudaStream_t)stream);
}

int dfl_pos_scores(const DflPosScoreParams* p, void* stream) {
  if (!p) return fail(DFL_ERR_BAD_ARG, "null params");
  if (!valid_dtype(p->dtype)) return fail(DFL_ERR_BAD_ARG, "unknown dtype %d", p->dtype);
  if (p->batch < 1 || p->heads < 1 || p->seq_len < 1 || p->n_active < 1)
    return fail(DFL_ERR_BAD_ARG, "non-positive size");
  if (!valid_head_dim(p->head_dim))
    return fail(DFL_ERR_UNSUPPORTED, "head_dim %d not in {32,64,128}", p->head_dim);
  if (p->ld_slots < p->n_active || p->ld_slots % 8)
    return fail(DFL_ERR_ALIGNMENT, "ld_slots must be >= n_active and a multiple of 8");
  if ((long long)p->batch * p->heads > 65535) return fail(DFL_ERR_TOO_LARGE, "batch*heads > 65535");
  int rc = DFL_OK;
  for (int term = 0; term < 2 && rc == DFL_OK; ++term) {
    const void* x = term == 0 ? p->q : p->k;
    const void* w = term == 0 ? p->pos_key : p->pos_query;
    void* out = term == 0 ? p->c2p : p->p2c;
    if (!out) continue;
    if (!x || !w) return fail(DFL_ERR_BAD_ARG, "null input for requested position-score term %d", term);
    if (!aligned16(x) || !aligned16(w) || !aligned16(out))
      return fail(DFL_ERR_ALIGNMENT, "position-score tensor not 16-byte aligned");
    GemmDesc g{};
    g.x = x; g.w = w; g.bias = nullptr; g.out[0] = out;
    g.M = p->seq_len; g.N = p->n_active; g.K = p->head_dim;
    g.batch = p->batch * p->heads;
    g.stride_x = (long long)p->seq_len * p->head_dim;
    g.stride_w = (long long)p->n_active * p->head_dim;
    g.w_mod = p->heads;
    g.stride_c = (long long)p->seq_len * p->ld_slots;
    g.ldc = p->ld_slots;
    g.head_split = 0; g.heads = p->heads; g.head_dim = p->head_dim; g.rows_per_seq = p->seq_len;
    g.dtype = p->dtype;
    g.status = p->status;
    rc = use_tensor_cores(p->dtype, p->algo) ? launch_gemm_tc(g, (cudaStream_t)stream)
                                             : launch_gemm_simt(g, (cudaStream_t)stream);
  }
  return rc;
}

int dfl_attention_fwd(const DflAttnParams* p, void* stream) {
  if (!p) return fail(DFL_ERR_BAD_ARG, "null params");
  if (!valid_dtype(p->dtype)) return fail(DFL_ERR_BAD_ARG, "unknown dtype %d", p->dtype);
  if (p->batch < 1 || p->heads < 1 || p->seq_len < 1) return fail(DFL_ERR_BAD_ARG, "non-positive size");
  if (!valid_head_dim(p->head_dim))
    return fail(DFL_ERR_UNSUPPORTED, "head_dim %d not in {32,64,128}", p->head_dim);
  if (!p->q || !p->k || !p->v || !p->out || !p->mask) return fail(DFL_ERR_BAD_ARG, "null pointer");
  if (p->mask_elem_size != 1 && p->mask_elem_size != 4 && p->mask_elem_size != 8)
    return fail(DFL_ERR_BAD_ARG, "mask_elem_size must be 1, 4 or 8");
  if ((p->c2p || p->p2c) && !p->lut) return fail(DFL_ERR_BAD_ARG, "position scores given without a LUT");
  if ((p->c2p || p->p2c) && (p->ld_slots < 1 || p->ld_slots % 8))
    return fail(DFL_ERR_ALIGNMENT, "ld_slots must be a positive multiple of 8");
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->out) ||
      (p->c2p && !aligned16(p->c2p)) || (p->p2c && !aligned16(p->p2c)))
    return fail(DFL_ERR_ALIGNMENT, "attention tensor not 16-byte aligned");
  if (!(p->scale > 0.0f)) return fail(DFL_ERR_BAD_ARG, "scale must be positive");
  if (use_tensor_cores(p->dtype, p->algo)) return launch_attention_tc(*p, (cudaStream_t)stream);
  return launch_attention_simt(*p, (cudaStream_t)stream);
}

int dfl_expand_rel_tables(const void* pos, const int32_t* lut_dev, void* rel, int heads, int n_active, int seq_len,
                          int head_dim, int dtype, void* stream) {
  if (!valid_dtype(dtype)) return fail(DFL_ERR_BAD_ARG, "unknown dtype %d", dtype);
  if (heads < 1 || n_active < 1 || seq_len < 1 || head_dim < 1) return fail(DFL_ERR_BAD_ARG, "non-positive size");
  if (!pos || !lut_dev || !rel) return fail(DFL_ERR_BAD_ARG, "null pointer");
  if ((head_dim * dtype_size(dtype)) % 16) return fail(DFL_ERR_ALIGNMENT, "table rows must be multiples of 16 bytes");
  if (!aligned16(pos) || !aligned16(rel)) return fail(DFL_ERR_ALIGNMENT, "table not 16-byte aligned");
  return launch_expand_rel_tables(pos, lut_dev, rel, heads, n_active, seq_len, head_dim, dtype, (cudaStream_t)stream);
}

int dfl_dense(const DflDenseParams* p, void* stream) {
  if (!p) return fail(DFL_ERR_BAD_ARG, "null params");
  if (!valid_dtype(p->dtype)) return fail(DFL_ERR_BAD_ARG, "unknown dtype %d", p->dtype);
  if (p->M < 0 || p->N < 1 || p->K < 1) return fail(DFL_ERR_BAD_ARG, "non-positive size");
  if (p->activation != DFL_ACT_NONE && p->activation != DFL_ACT_GELU)
    return fail(DFL_ERR_BAD_ARG, "dfl_dense takes DFL_ACT_NONE or DFL_ACT_GELU, got %d", p->activation);
  if (p->M == 0) return DFL_OK;
  if (!p->x || !p->w || !p->out) return fail(DFL_ERR_BAD_ARG, "null pointer");
  if ((p->N % 8) || (p->K % 8)) return fail(DFL_ERR_ALIGNMENT, "N and K must be multiples of 8 elements");
  if (!aligned16(p->x) || !aligned16(p->w) || !aligned16(p->out) || !aligned16(p->bias))
    return fail(DFL_ERR_ALIGNMENT, "pointers must be 16-byte aligned");
  GemmDesc g{};
  g.x = p->x; g.w = p->w; g.bias = p->bias; g.out[0] = p->out;
  g.M = p->M; g.N = p->N; g.K = p->K;
  g.batch = 1; g.stride_x = 0; g.stride_w = 0; g.w_mod = 1; g.stride_c = 0;
  g.ldc = p->N;
  g.head_split = 0; g.heads = 1; g.head_dim = p->N; g.rows_per_seq = p->M;
  g.dtype = p->dtype;
  g.status = p->status;
  g.activation = p->activation;
  return use_tensor_cores(p->dtype, p->algo) ? launch_gemm_tc(g, (cudaStream_t)stream)
                                             : launch_gemm_simt(g, (cudaStream_t)stream);
}

int dfl_conv1d_supported(const DflConv1dParams* p) {
  if (!p || (p->dtype != DFL_F16 && p->dtype != DFL_BF16)) return 0;
  if (p->taps < 1 || p->taps > 9 || !(p->taps & 1)) return 0;
  if (p->seq_len < 256 || p->c_in < 64 || (p->c_in % 8) || (p->c_out % 8) || p->c_out < 8) return 0;
  return p->activation == DFL_ACT_NONE || p->activation == DFL_ACT_GELU || p->activation == DFL_ACT_TANH;
}

int dfl_conv1d(const DflConv1dParams* p, void* stream) {
  if (!p) return fail(DFL_ERR_BAD_ARG, "null params");
  if (!valid_dtype(p->dtype)) return fail(DFL_ERR_BAD_ARG, "unknown dtype %d", p->dtype);
  if (p->batch < 1 || p->seq_len < 1 || p->c_in < 1 || p->c_out < 1) return fail(DFL_ERR_BAD_ARG, "non-positive size");
  if (!dfl_conv1d_supported(p))
    return fail(DFL_ERR_UNSUPPORTED,
                "conv1d covers F16/BF16, odd taps <= 9, seq_len >= 256, c_in >= 64, channels in multiples of 8");
  if (!p->x || !p->w || !p->out) return fail(DFL_ERR_BAD_ARG, "null pointer");
  if (p->row_mask && p->mask_elem_size != 1 && p->mask_elem_size != 4 && p->mask_elem_size != 8)
    return fail(DFL_ERR_BAD_ARG, "mask_elem_size must be 1, 4 or 8");
  if (!aligned16(p->x) || !aligned16(p->w) || !aligned16(p->out) || !aligned16(p->bias))
    return fail(DFL_ERR_ALIGNMENT, "pointers must be 16-byte aligned");
  if ((long long)p->batch > 65535) return fail(DFL_ERR_TOO_LARGE, "batch beyond 65535");
  GemmDesc g{};
  g.x = p->x; g.w = p->w; g.bias = p->bias; g.out[0] = p->out;
  g.M = p->seq_len; g.N = p->c_out; g.K = p->c_in;
  g.batch = p->batch;
  g.stride_x = (long long)p->seq_len * p->c_in;
  g.stride_w = 0; g.w_mod = 1;
  g.stride_c = (long long)p->seq_len * p->c_out;
  g.ldc = p->c_out;
  g.head_split = 0; g.heads = 1; g.head_dim = p->c_out; g.rows_per_seq = p->seq_len;
  g.dtype = p->dtype;
  g.status = p->status;
  g.activation = p->activation;
  g.taps = p->taps;
  g.row_mask = p->row_mask; g.row_mask_elem = p->mask_elem_size;
  return launch_gemm_tc(g, (cudaStream_t)stream);
}

int dfl_copy_rows(const void* src, void* dst, const int32_t* rows_dev, int64_t n_rows, int32_t row_bytes, void* stream) {
  if (n_rows < 0 || row_bytes < 16 || (row_bytes % 16)) return fail(DFL_ERR_BAD_ARG, "rows of a positive multiple of 16 bytes");
  if (n_rows == 0) return DFL_OK;
  if (!src || !dst || !rows_dev) return fail(DFL_ERR_BAD_ARG, "null pointer");
  if (!aligned16(src) || !aligned16(dst)) return fail(DFL_ERR_ALIGNMENT, "pointers must be 16-byte aligned");
  return launch_copy_rows(src, dst, rows_dev, n_rows, row_bytes, (cudaStream_t)stream);
}

int dfl_add_layernorm_supported(int dtype, int hidden) {
  if (!valid_dtype(dtype) || hidden < 1) return 0;
  const int elems = (int)(16 / dtype_size(dtype));
  return hidden % elems == 0 && hidden <= add_layernorm_max_hidden(dtype_size(dtype)) ? 1 : 0;
}

int dfl_add_layernorm(const DflAddLayerNormParams* p, void* stream) {
  if (!p) return fail(DFL_ERR_BAD_ARG, "null params");
  if (!valid_dtype(p->dtype)) return fail(DFL_ERR_BAD_ARG, "unknown dtype %d", p->dtype);
  if (p->rows < 0 || p->hidden < 1) return fail(DFL_ERR_BAD_ARG, "non-positive size");
  if (!(p->eps >= 0.0f)) return fail(DFL_ERR_BAD_ARG, "eps must be non-negative");
  if (!dfl_add_layernorm_supported(p->dtype, p->hidden))
    return fail(DFL_ERR_UNSUPPORTED, "hidden size %d: rows must be multiples of 16 bytes and at most %d elements",
                p->hidden, add_layernorm_max_hidden(dtype_size(p->dtype)));
  if (p->rows == 0) return DFL_OK;
  if (!p->x || !p->gamma || !p->out) return fail(DFL_ERR_BAD_ARG, "null pointer");
  if (!aligned16(p->x) || !aligned16(p->residual) || !aligned16(p->gamma) || !aligned16(p->beta) || !aligned16(p->out))
    return fail(DFL_ERR_ALIGNMENT, "pointers must be 16-byte aligned");
  if (p->row_mask && p->mask_elem_size != 1 && p->mask_elem_size != 4 && p->mask_elem_size != 8)
    return fail(DFL_ERR_BAD_ARG, "mask_elem_size must be 1, 4 or 8");
  if ((p->out2 != nullptr) != (p->out2_rows != nullptr)) return fail(DFL_ERR_BAD_ARG, "out2 and out2_rows go together");
  if (!aligned16(p->out2)) return fail(DFL_ERR_ALIGNMENT, "out2 must be 16-byte aligned");
  return launch_add_layernorm(p->x, p->residual, p->gamma, p->beta, p->out, p->rows, p->hidden, p->eps, p->dtype,
                              p->row_mask, p->mask_elem_size, p->out2, p->out2_rows, (cudaStream_t)stream);
}

int dfl_embed_layernorm(const DflEmbedLayerNormParams* p, void* stream) {
  if (!p) return fail(DFL_ERR_BAD_ARG, "null params");
  if (!valid_dtype(p->dtype)) return fail(DFL_ERR_BAD_ARG, "unknown dtype %d", p->dtype);
  if (p->rows < 0 || p->hidden < 1 || p->vocab < 1) return fail(DFL_ERR_BAD_ARG, "non-positive size");
  if (!(p->eps >= 0.0f)) return fail(DFL_ERR_BAD_ARG, "eps must be non-negative");
  if (!dfl_add_layernorm_supported(p->dtype, p->hidden))
    return fail(DFL_ERR_UNSUPPORTED, "hidden size %d: rows must be multiples of 16 bytes and at most %d elements",
                p->hidden, add_layernorm_max_hidden(dtype_size(p->dtype)));
  if (p->rows == 0) return DFL_OK;
  if (!p->ids || !p->table || !p->gamma || !p->out) return fail(DFL_ERR_BAD_ARG, "null pointer");
  if (p->id_elem_size != 4 && p->id_elem_size != 8) return fail(DFL_ERR_BAD_ARG, "id_elem_size must be 4 or 8");
  if ((p->pos_ids != nullptr) != (p->pos_table != nullptr)) return fail(DFL_ERR_BAD_ARG, "pos_ids and pos_table go together");
  if (p->pos_table && p->positions < 1) return fail(DFL_ERR_BAD_ARG, "positions must be positive");
  if (p->row_mask && p->mask_elem_size != 1 && p->mask_elem_size != 4 && p->mask_elem_size != 8)
    return fail(DFL_ERR_BAD_ARG, "mask_elem_size must be 1, 4 or 8");
  if (!aligned16(p->table) || !aligned16(p->pos_table) || !aligned16(p->gamma) || !aligned16(p->beta) || !aligned16(p->out))
    return fail(DFL_ERR_ALIGNMENT, "pointers must be 16-byte aligned");
  return launch_embed_layernorm(p->ids, p->table, p->vocab, p->pos_ids, p->pos_table, p->positions, p->id_elem_size,
                                p->gamma, p->beta, p->out, p->rows, p->hidden, p->eps, p->dtype, p->row_mask,
                                p->mask_elem_size, p->status, (cudaStream_t)stream);
}

int dfl_attention_rel_supported(const DflAttnRelParams* p) {
  return p && p->algo == DFL_ALGO_AUTO && attention_rel_supported(*p) ? 1 : 0;
}

int dfl_attention_rel_fwd(const DflAttnRelParams* p, void* stream) {
  if (!p) return fail(DFL_ERR_BAD_ARG, "null params");
  if (!valid_dtype(p->dtype)) return fail(DFL_ERR_BAD_ARG, "unknown dtype %d", p->dtype);
  if (p->batch < 1 || p->heads < 1 || p->seq_len < 1) return fail(DFL_ERR_BAD_ARG, "non-positive size");
  if (!p->q || !p->k || !p->v || !p->out || !p->mask) return fail(DFL_ERR_BAD_ARG, "null pointer");
  if (p->mask_elem_size != 1 && p->mask_elem_size != 4 && p->mask_elem_size != 8)
    return fail(DFL_ERR_BAD_ARG, "mask_elem_size must be 1, 4 or 8");
  if (!(p->scale > 0.0f)) return fail(DFL_ERR_BAD_ARG, "scale must be positive");
  if ((p->out_row_base != nullptr) != (p->out_row_count != nullptr))
    return fail(DFL_ERR_BAD_ARG, "out_row_base and out_row_count go together");
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->out) ||
      (p->rel_key && !aligned16(p->rel_key)) || (p->rel_query && !aligned16(p->rel_query)))
    return fail(DFL_ERR_ALIGNMENT, "attention tensor not 16-byte aligned");
  if (!dfl_attention_rel_supported(p))
    return fail(DFL_ERR_UNSUPPORTED, "not covered by the relative-table kernel; use dfl_pos_scores + dfl_attention_fwd");
  return launch_attention_rel(*p, (cudaStream_t)stream);
}

}  // extern "C"
