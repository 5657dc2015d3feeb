/*
 * dfl_b200.h -- C ABI of the B200 (sm_100a) disentangled-attention library.
 *
 * Every entry point replaces one step of the reference's Triton-backend hot
 * path (paths below are inside the reference project,
 * src/disentangled_flash/...).  The library owns no user-visible memory:
 * every pointer is a borrowed CUDA device pointer unless stated otherwise,
 * every launch goes to the stream that is passed in, and nothing
 * synchronises with the host.  All functions return 0 on success or a
 * negative DFL_ERR_* code; none throws, aborts or prints.
 *
 * Alignment: every tensor base pointer must be 16-byte aligned (TMA and
 * 128-bit vector access); violations return DFL_ERR_ALIGNMENT.
 */
#ifndef DFL_B200_H_
#define DFL_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define DFL_API __attribute__((visibility("default")))
#else
#define DFL_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------ */
#define DFL_OK                   0
#define DFL_ERR_BAD_ARG         -1  /* null pointer, non-positive size, unknown enum      */
#define DFL_ERR_UNSUPPORTED     -2  /* head_dim not in {32,64,128}, dtype/algo mismatch   */
#define DFL_ERR_ALIGNMENT       -3  /* pointer or leading dimension not 16-byte aligned   */
#define DFL_ERR_LAUNCH          -4  /* CUDA runtime reported an error at launch           */
#define DFL_ERR_DRIVER          -5  /* tensor-map encoding / driver entry point failed    */
#define DFL_ERR_DEVICE_TIMEOUT  -6  /* a bounded device-side wait expired (status word)   */
#define DFL_ERR_TOO_LARGE       -7  /* size beyond a documented fixed maximum             */

/* element type of activations and weights */
#define DFL_F16   0
#define DFL_BF16  1
#define DFL_F32   2

/* kernel family selection: AUTO = tcgen05 kernels for F16/BF16, IEEE-fp32
 * CUDA-core kernels for F32.  SIMT forces the CUDA-core kernels for any
 * dtype; it exists so that tests can cross-check the tensor-core kernels at
 * sizes where a CPU oracle is too slow. */
#define DFL_ALGO_AUTO  0
#define DFL_ALGO_SIMT  1

DFL_API int         dfl_version(void);
DFL_API const char* dfl_status_string(int status);
/* Human-readable detail of the last non-zero status returned on this host thread. */
DFL_API const char* dfl_last_error(void);

/*
 * Device status word.  The tcgen05 kernels wait on hardware barriers with a time limit (two seconds); a wait
 * that runs out makes its CTA skip the rest of its work, free its tensor memory and return, after writing a
 * non-zero code (which wait gave up) to the `status` word of the call - a device int32 owned by the caller and
 * zeroed by it before first use; calls given no status word use a word inside the library.  Nothing on the hot
 * path reads the word.  dfl_check_status() is the read-out: it waits for `stream`, copies the word to the host,
 * and if it is non-zero clears it and returns DFL_ERR_DEVICE_TIMEOUT (dfl_last_error() names the code; the
 * outputs of the calls since the previous check are then not valid).  The reference has no counterpart: its
 * Triton kernel has no device-side waits.
 *
 * dfl_selftest_bounded_wait() is a diagnostic for that path: one CTA allocates tensor memory, waits on a
 * barrier nobody arrives at with a limit of `limit_us` microseconds (1..100000), gives up, frees its tensor
 * memory and records code 99 in `status_dev`.  It never traps and never waits without a limit.
 */
DFL_API int dfl_check_status(int32_t* status_dev, void* stream);
DFL_API int dfl_selftest_bounded_wait(int32_t* status_dev, uint32_t limit_us, void* stream);

/*
 * Log-bucket relative-position index builder (bit-exact).
 * Replaces SharedPositionPlanCache.compact (position.py:89-128) and
 * make_log_bucket_position (_reference.py:115-136), which the reference
 * evaluates on the CPU and copies to the device.
 *
 *   lut_dev      int32 [2*seq_len-1]  delta index (i-j+L-1) -> local slot
 *   active_dev   int64 [min(2*seq_len-1, 2*span)] capacity; first *n_active valid
 *   n_active_dev int32 [1]
 * position_buckets <= 0 selects the un-bucketed branch; uses_position_bias == 0
 * writes an all-zero LUT and n_active = 0 (position.py:118-120).
 */
DFL_API int dfl_build_position_lut(int seq_len, int position_buckets, int max_relative_positions,
                           int span, int uses_position_bias,
                           int32_t* lut_dev, int64_t* active_dev, int32_t* n_active_dev,
                           void* stream);

/*
 * Fused projection with head-split epilogue:
 *     Y = X[M,K] * W[N,K]^T + bias[N],   N = n_out * heads * head_dim
 * and column block `o` of Y is written to out[o] in [M/rows_per_seq, heads,
 * rows_per_seq, head_dim] layout.  With n_out = 3 this is the fused QKV
 * projection plus the three head transposes (replaces _project_qkv,
 * _torch.py:284-297, and _reshape_heads x3, _torch.py:299-314).  With
 * n_out = 1, M = rows_per_seq = 2*span it is the relative-embedding
 * projection posK/posQ = transpose_for_scores(proj(rel)) (_torch.py:143-158).
 */
typedef struct DflLinearParams {
  const void* x;        /* [M, K] row-major                                    */
  const void* w;        /* [N, K] row-major (nn.Linear weight layout)          */
  const void* bias;     /* [N] or NULL                                         */
  void*       out[3];   /* n_out tensors, each [M/rows_per_seq, heads, rows_per_seq, head_dim] */
  int32_t M, K;
  int32_t n_out;        /* 1..3                                                */
  int32_t heads, head_dim;
  int32_t rows_per_seq; /* L; M must be a multiple of it                       */
  int32_t dtype;        /* DFL_F16 / DFL_BF16 / DFL_F32                        */
  int32_t algo;         /* DFL_ALGO_*                                          */
  int32_t* status;      /* optional device int32, see dfl_check_status()       */
  /* Optional packed input rows (FP16/BF16 tensor-core kernels; no counterpart in the reference, which projects the
   * padded positions too): X holds only the kept rows, in groups of 32; group g (rows 32g .. 32g+31) is written to
   * rows row_groups[g] .. +31 of the output row space [out_seqs * rows_per_seq] (row = sequence * rows_per_seq +
   * position).  M and rows_per_seq must be multiples of 32, every group must lie inside one sequence, and output
   * rows no group covers are left as they are.  NULL: row m of X is output row m and out_seqs is ignored. */
  const int32_t* row_groups;   /* device int32 [M / 32] or NULL */
  int32_t out_seqs;
} DflLinearParams;
DFL_API int dfl_qkv_proj(const DflLinearParams* p, void* stream);

/*
 * Prune projected position tables to the active slots:
 *   dst[h, a, :] = src[h, active[a], :]      (replaces _project_active_positions,
 *   _torch.py:171-186).  src is [heads, n_slots_src, head_dim], dst is
 *   [heads, n_active, head_dim].
 */
DFL_API int dfl_gather_slots(const void* src, const int64_t* active_dev, void* dst,
                     int heads, int n_slots_src, int n_active, int head_dim, int dtype,
                     void* stream);

/*
 * Content-to-position / position-to-content score GEMMs over the active slots
 * (replaces the two torch.matmul calls at kernel.py:574-585):
 *     c2p[b,h,i,a] = sum_d q[b,h,i,d] * pos_key[h,a,d]
 *     p2c[b,h,j,a] = sum_d k[b,h,j,d] * pos_query[h,a,d]
 * Outputs are [batch, heads, seq_len, ld_slots] with ld_slots >= n_active and
 * ld_slots a multiple of 8 (row starts stay 16-byte aligned); columns
 * [n_active, ld_slots) are written as zero.  Either pair may be NULL.
 */
typedef struct DflPosScoreParams {
  const void* q;          /* [B,H,L,d] or NULL */
  const void* k;          /* [B,H,L,d] or NULL */
  const void* pos_key;    /* [H,A,d]  (needed with q) */
  const void* pos_query;  /* [H,A,d]  (needed with k) */
  void*       c2p;        /* [B,H,L,ld_slots] or NULL */
  void*       p2c;        /* [B,H,L,ld_slots] or NULL */
  int32_t batch, heads, seq_len, head_dim;
  int32_t n_active, ld_slots;
  int32_t dtype, algo;
  int32_t* status;        /* optional device int32, see dfl_check_status() */
} DflPosScoreParams;
DFL_API int dfl_pos_scores(const DflPosScoreParams* p, void* stream);

/*
 * Fused disentangled attention forward (replaces the Triton kernel
 * _deberta_attention_forward_kernel and its launcher, kernel.py:137-429):
 *   S[i,j] = q_i.k_j + c2p[i, lut[i-j+L-1]] + p2c[j, lut[i-j+L-1]]
 *   P      = softmax_j( S * scale ) under the factorised padding mask
 *   out[b,i,h*d:(h+1)*d] = P V
 * Mask rule: pair (i,j) attended iff mask[b,i] && mask[b,j]; a padded query
 * row is uniform over all L keys.  [B,H,L,L] is never written to memory.
 */
typedef struct DflAttnParams {
  const void* q;          /* [B,H,L,d] */
  const void* k;          /* [B,H,L,d] */
  const void* v;          /* [B,H,L,d] */
  const void* c2p;        /* [B,H,L,ld_slots] or NULL (term disabled) */
  const void* p2c;        /* [B,H,L,ld_slots] or NULL (term disabled) */
  const int32_t* lut;     /* [2L-1]; may be NULL when both terms are disabled.  Must come from
                             dfl_build_position_lut or have its shape: non-decreasing in the delta index with
                             steps of 0 or 1 and entries in [0, ld_slots) - the tcgen05 kernel stages one
                             contiguous window of slots per tile and clamps anything outside it */
  const void* mask;       /* [B,L], mask_elem_size bytes per element, non-zero = keep */
  void*       out;        /* [B,L,H*d] */
  int32_t*    status;     /* optional device int32: set non-zero if a bounded wait expired */
  int32_t batch, heads, seq_len, head_dim;
  int32_t ld_slots;
  int32_t mask_elem_size; /* 1, 4 or 8 */
  float   scale;          /* 1/sqrt(head_dim * (1 + has_c2p + has_p2c)), natural units */
  int32_t dtype, algo;
} DflAttnParams;
DFL_API int dfl_attention_fwd(const DflAttnParams* p, void* stream);

/*
 * Allocation-free variant of dfl_pos_scores followed by dfl_attention_fwd.  It has no counterpart
 * in the reference (whose launcher allocates with torch.empty on every call).
 *
 * Who needs it: callers that cannot allocate device memory at the point of the call, e.g. a server
 * that gave the whole device to its own arena at start-up, or a plug-in running inside a host
 * runtime's callback where cudaMalloc (a device-wide synchronisation) is off limits.  The C2P/P2C
 * score tensors, which the regular path keeps in caller-allocated buffers, live here in a fixed
 * array inside the library's device image.  The call performs no cudaMalloc/cudaFree and calls no
 * allocating library routine; inputs and the output are still the caller's.
 *
 * Limit: DFL_STATIC_SCRATCH_BYTES (32 MiB), held by every GPU context that loads the library until
 * it exits.  Needed: (number of enabled terms) * batch*heads*seq_len*ceil8(n_active)*sizeof(element),
 * each term rounded up to 256 bytes; larger requests return DFL_ERR_TOO_LARGE and touch nothing.
 *
 * The first call on each device looks up the array's device address (with that device current) and
 * performs the kernels' one-time configuration; make that first call before any stream capture.
 * All calls on a device share the one array and it keeps the last call's scores: every element a
 * call reads is rewritten by that same call first, so nothing has to be cleared, but two calls whose
 * kernels overlap on the GPU (different streams, or different host threads) race on it.
 */
#define DFL_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)
typedef struct DflAttnTablesParams {
  const void* q;          /* [B,H,L,d] */
  const void* k;          /* [B,H,L,d] */
  const void* v;          /* [B,H,L,d] */
  const void* pos_key;    /* [H,A,d] or NULL (C2P disabled) */
  const void* pos_query;  /* [H,A,d] or NULL (P2C disabled) */
  const int32_t* lut;     /* [2L-1]; may be NULL when both terms are disabled */
  const void* mask;       /* [B,L] */
  void*       out;        /* [B,L,H*d] */
  int32_t*    status;     /* optional device int32, as in DflAttnParams */
  int32_t batch, heads, seq_len, head_dim;
  int32_t n_active;       /* A */
  int32_t mask_elem_size; /* 1, 4 or 8 */
  float   scale;
  int32_t dtype, algo;
} DflAttnTablesParams;
DFL_API int    dfl_attention_fwd_static(const DflAttnTablesParams* p, void* stream);
DFL_API size_t dfl_static_scratch_bytes(void);


/*
 * Fused attention over position tables laid out by relative distance.
 *
 * dfl_expand_rel_tables() is a prepare-time step (once per layer and sequence length, next to the
 * pruning of kernel.py:503-532): it expands a pruned table pos [H,A,d] through the slot table
 * lut [2L-1] into rel [H, 2L-1, d] with rel[h, e] = pos[h, lut[2L-2-e]], i.e. row e holds the
 * projection used by every (query i, key j) pair with j - i = e - (L-1).  No arithmetic: rows are copied.
 *
 * dfl_attention_rel_fwd() is the whole attention core in one launch, equal in result to
 * dfl_pos_scores + dfl_attention_fwd (the two torch.matmul calls kernel.py:574-585 followed by the Triton
 * kernel kernel.py:137-429): S = QK^T + q_i.rel_key[j-i] + k_j.rel_query[j-i], the two relative terms
 * rounded to the input type as the separate score GEMMs round their output, scale, 2-D padding mask,
 * softmax, PV.  The score tensors [B,H,L,A] never exist in global memory.  A persistent kernel: one CTA
 * per SM walks (batch, head, 128-query-tile) items.  Covered: FP16/BF16, head_dim 32 or 64, at least one
 * relative term, seq_len <= 2048; dfl_attention_rel_supported() tells, other configurations return
 * DFL_ERR_UNSUPPORTED (use dfl_pos_scores + dfl_attention_fwd for them).
 */
typedef struct DflAttnRelParams {
  const void* q;          /* [B,H,L,d] */
  const void* k;          /* [B,H,L,d] */
  const void* v;          /* [B,H,L,d] */
  const void* rel_key;    /* [H,2L-1,d] expanded pos_key table, or NULL (C2P disabled) */
  const void* rel_query;  /* [H,2L-1,d] expanded pos_query table, or NULL (P2C disabled) */
  const void* mask;       /* [B,L] */
  void*       out;        /* [B,L,H*d] */
  int32_t*    status;     /* optional device int32, as in DflAttnParams */
  int32_t batch, heads, seq_len, head_dim;
  int32_t mask_elem_size; /* 1, 4 or 8 */
  float   scale;
  int32_t dtype, algo;
  /* Packed output (both NULL: out is [B,L,H*d]).  With both given, out is [T,H*d]: the rows of sequence b start at
   * row out_row_base[b] and only its first out_row_count[b] positions are written (query positions beyond that,
   * padding, are not computed where a whole tile of them can be skipped and never stored).  No counterpart in the
   * reference, which keeps padded positions in every tensor. */
  const int32_t* out_row_base;   /* device [B] or NULL */
  const int32_t* out_row_count;  /* device [B] or NULL */
} DflAttnRelParams;
DFL_API int dfl_expand_rel_tables(const void* pos, const int32_t* lut_dev, void* rel, int heads, int n_active,
                                  int seq_len, int head_dim, int dtype, void* stream);
DFL_API int dfl_attention_rel_supported(const DflAttnRelParams* p);
DFL_API int dfl_attention_rel_fwd(const DflAttnRelParams* p, void* stream);

/*
 * Dense layer with the bias and the activation in the GEMM epilogue:
 *     out[M, N] = act(x[M, K] * w[N, K]^T + bias[N])
 * Replaces DebertaV2Intermediate.forward (_reference.py:461-471: nn.Linear followed by ACT2FN["gelu"], which PyTorch
 * runs as a GEMM and an elementwise kernel that reads and writes the [M, N] intermediate once more).  All tensors
 * row-major, K and N multiples of 8 elements (16-byte rows).  DFL_ACT_GELU is the erf form, 0.5 v (1 + erf(v/sqrt 2)):
 * the F32 kernels use erff, the F16/BF16 kernels a rational approximation of erf with absolute error < 1.5e-7.
 */
#define DFL_ACT_NONE 0
#define DFL_ACT_GELU 1
#define DFL_ACT_TANH 2
typedef struct DflDenseParams {
  const void* x;        /* [M, K] */
  const void* w;        /* [N, K] (nn.Linear weight layout) */
  const void* bias;     /* [N] or NULL */
  void*       out;      /* [M, N] */
  int32_t M, N, K;
  int32_t activation;   /* DFL_ACT_* */
  int32_t dtype;        /* DFL_F16 / DFL_BF16 / DFL_F32 */
  int32_t algo;         /* DFL_ALGO_* */
  int32_t* status;      /* optional device int32, see dfl_check_status() */
} DflDenseParams;
DFL_API int dfl_dense(const DflDenseParams* p, void* stream);

/*
 * 1-D convolution over the sequence with 'same' zero padding, stride 1, one group, as one tensor-core GEMM over the
 * taps, with bias, padding mask and activation in the epilogue:
 *     out[b, l, :] = act(keep[b, l] * (bias + sum_t w[t] * x[b, l + t - taps/2, :]))
 * Replaces, in ConvLayer.forward (_reference.py:534-556), the two permute().contiguous() copies around nn.Conv1d,
 * the convolution, masked_fill_ and the activation.  x is [batch, seq_len, c_in], w is [taps, c_out, c_in] (the
 * nn.Conv1d weight [c_out, c_in, taps] permuted once at prepare time), out is [batch, seq_len, c_out]; row_mask is
 * the [batch, seq_len] padding mask (non-zero = keep) or NULL.  The taps are k-steps of the GEMM: the operand
 * loads of tap t start t - taps/2 rows higher or lower, and rows outside the sequence read as zero.
 * Covered: F16/BF16, taps odd and <= 9, seq_len >= 256, c_in >= 64, c_in and c_out multiples of 8;
 * dfl_conv1d_supported() tells, other configurations return DFL_ERR_UNSUPPORTED.
 */
typedef struct DflConv1dParams {
  const void* x;         /* [batch, seq_len, c_in] */
  const void* w;         /* [taps, c_out, c_in] */
  const void* bias;      /* [c_out] or NULL */
  const void* row_mask;  /* [batch, seq_len] or NULL */
  void*       out;       /* [batch, seq_len, c_out] */
  int32_t batch, seq_len, c_in, c_out, taps;
  int32_t mask_elem_size; /* 1, 4 or 8 */
  int32_t activation;    /* DFL_ACT_* */
  int32_t dtype;
  int32_t* status;       /* optional device int32, see dfl_check_status() */
} DflConv1dParams;
DFL_API int dfl_conv1d_supported(const DflConv1dParams* p);
DFL_API int dfl_conv1d(const DflConv1dParams* p, void* stream);

/*
 * Residual add + LayerNorm in one pass (the tail of a layer's two output blocks):
 *     out[r, :] = LayerNorm(x[r, :] + residual[r, :]) * gamma + beta
 * with the sum, the mean and the (biased) variance in fp32 and the result rounded to `dtype`.  Replaces, in the
 * encoder's layer loop (deberta.py:268-270), `self.LayerNorm(hidden_states + input_tensor)` of
 * DebertaV2SelfOutput.forward (_reference.py:108-112) and DebertaV2Output.forward (_reference.py:481-485), which
 * PyTorch runs as an elementwise add and a layer-norm kernel; the dense projection in front of it stays the
 * caller's GEMM.  x, residual and out are [rows, hidden] row-major (out may alias x or residual), gamma and beta
 * [hidden]; residual and beta may be NULL.  hidden * sizeof(dtype) must be a multiple of 16 bytes and hidden at most
 * 4096 (F16/BF16) or 2048 (F32): dfl_add_layernorm_supported() tells, other sizes return DFL_ERR_UNSUPPORTED.
 * Unlike PyTorch, which rounds the sum to `dtype` before normalising, the sum stays in fp32.
 */
typedef struct DflAddLayerNormParams {
  const void* x;         /* [rows, hidden] */
  const void* residual;  /* [rows, hidden] or NULL */
  const void* gamma;     /* [hidden] */
  const void* beta;      /* [hidden] or NULL */
  void*       out;       /* [rows, hidden] */
  int64_t rows;
  int32_t hidden;
  float   eps;
  int32_t dtype;
  const void* row_mask;    /* [rows] or NULL: output rows whose element is zero are written as zeros */
  int32_t mask_elem_size;  /* 1, 4 or 8 */
  void*       out2;        /* optional second copy of the result, row r written to row out2_rows[r] of out2 */
  const int32_t* out2_rows; /* device [rows], required with out2; a negative entry skips the row */
} DflAddLayerNormParams;
DFL_API int dfl_add_layernorm_supported(int dtype, int hidden);
/*
 * Row gather: dst[r, :] = src[rows[r], :] for r < n_rows (rows of row_bytes bytes, a multiple of 16; a negative
 * entry writes zeros).  Used to pack the valid positions of a padded batch into consecutive rows and back.
 */
DFL_API int dfl_copy_rows(const void* src, void* dst, const int32_t* rows_dev, int64_t n_rows, int32_t row_bytes,
                          void* stream);
DFL_API int dfl_add_layernorm(const DflAddLayerNormParams* p, void* stream);

/*
 * Embedding front-end in one pass: token-embedding gather, optional position-embedding add, LayerNorm, padding mask:
 *     out[r, :] = LayerNorm(table[ids[r], :] (+ pos_table[pos_ids[r], :])) * gamma + beta,   zeros where row_mask[r] == 0
 * What Hugging Face's DebertaV2Embeddings.forward computes in front of the encoder the reference replaces
 * (optimize_deberta keeps `model.embeddings` as it is, deberta.py:322-330) for a model without token types and
 * without an embedding projection, as an embedding gather, an add, a layer-norm kernel and a multiply; the
 * reference's benchmark builds its inputs the same way (`table[ids]`, benchmark_cuda.py:176-183).  Same kernel,
 * limits and fp32 arithmetic as dfl_add_layernorm.  An id outside [0, vocab) (or a position outside
 * [0, positions)) cannot fault: the row is read as zeros and code 98 is written to `status`, which
 * dfl_check_status() then reports as DFL_ERR_BAD_ARG.
 */
typedef struct DflEmbedLayerNormParams {
  const void* ids;        /* [rows] int32 or int64 token ids */
  const void* table;      /* [vocab, hidden] */
  const void* pos_ids;    /* [rows] or NULL (same integer type as ids) */
  const void* pos_table;  /* [positions, hidden] or NULL; goes with pos_ids */
  const void* gamma;      /* [hidden] */
  const void* beta;       /* [hidden] or NULL */
  const void* row_mask;   /* [rows] or NULL */
  void*       out;        /* [rows, hidden] */
  int64_t rows, vocab, positions;
  int32_t hidden;
  float   eps;
  int32_t dtype;
  int32_t id_elem_size;   /* 4 or 8 */
  int32_t mask_elem_size; /* 1, 4 or 8 */
  int32_t* status;        /* optional device int32, see dfl_check_status() */
} DflEmbedLayerNormParams;
DFL_API int dfl_embed_layernorm(const DflEmbedLayerNormParams* p, void* stream);

#ifdef __cplusplus
}
#endif
#endif  /* DFL_B200_H_ */
