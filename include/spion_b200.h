/*
 * spion_b200 - C ABI of the B200 (sm_100a) implementation of SPION's layer-wise
 * block-sparse attention path.
 *
 * Every pointer below is a DEVICE pointer unless its name starts with host_.  All
 * buffers (inputs, outputs, scratch) are allocated by the caller (PyTorch in the
 * reference); the library allocates only its own per-context workspace, at context
 * creation / spion_set_pattern time, never inside a forward or backward call.
 * Every call is asynchronous on the context's stream (spion_set_stream; default:
 * the legacy default stream, like the reference) unless stated otherwise.
 * Functions return 0 on success and a negative SPION_ERR_* code otherwise (the
 * reference's entry points return void and ignore every CUDA / cuSPARSE status).
 *
 * Citations name files of the reference project (mlsys-lab-sogang/SPION).
 */
#ifndef SPION_B200_H
#define SPION_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct spion_ctx spion_ctx;

enum {
  SPION_OK = 0,
  SPION_ERR_ARG = -1,          /* null pointer / bad enum / size mismatch            */
  SPION_ERR_SHAPE = -2,        /* unsupported shape (e.g. seq_len % block_size != 0)   */
  SPION_ERR_CUDA = -3,         /* a CUDA runtime call or kernel launch failed          */
  SPION_ERR_TIMEOUT = -4,      /* a bounded device-side wait gave up (status word)     */
  SPION_ERR_UNSUPPORTED = -5,  /* combination not built (dtype / head_dim / block)     */
  SPION_ERR_ALLOC = -6,        /* workspace allocation failed                          */
  SPION_ERR_STATE = -7         /* call order (e.g. native forward before set_pattern)  */
};

enum { SPION_F32 = 0, SPION_BF16 = 1 };
enum { SPION_CONV_DIAG = 0, SPION_CONV_BOX = 1 };
enum { SPION_SELECT_PATHS = 0, SPION_SELECT_TOPK = 1 };
enum { SPION_KIND_DENSE = 0, SPION_KIND_DENSE_KPM = 1, SPION_KIND_BLOCK = 2, SPION_KIND_BLOCK_KPM = 3 };
enum { SPION_ENGINE_AUTO = 0, SPION_ENGINE_SIMT = 1, SPION_ENGINE_TCGEN05 = 2, SPION_ENGINE_SIMT_STAGED = 3 };

const char* spion_status_string(int status);
int spion_version(void);

/* ------------------------------------------------------------------ contexts ---- */

/* Replaces `Attention* init(int emb_dim, int seq_len, int num_batches, int block_size)`
 * of models/block_attn.cu:547 and models/block_attn_mask.cu:655 (kind = BLOCK / BLOCK_KPM)
 * and `init(int emb_dim, int seq_len, int num_batches)` of models/attn.cu:265 and
 * models/attn_mask.cu:280 (kind = DENSE / DENSE_KPM, block_size ignored).
 * num_batches = heads * per-device batch.  dtype: SPION_F32 for the reference's layouts;
 * SPION_BF16 is accepted by the native (_ex) calls only.  device < 0: current device.
 * Returns NULL on failure. */
spion_ctx* spion_create(int kind, int head_dim, int seq_len, int num_batches, int block_size,
                        int dtype, int device);

/* Replaces `void destroy(Attention*)` (models/block_attn.cu:565, models/attn.cu:278). */
void spion_destroy(spion_ctx* ctx);

/* The reference runs everything on the legacy default stream (models/block_attn.cu:468);
 * here the caller chooses (pass torch.cuda.current_stream().cuda_stream). */
int spion_set_stream(spion_ctx* ctx, void* cuda_stream);

/* SPION_ENGINE_AUTO picks tcgen05 kernels where they exist (bf16, block 64/32, head_dim 64/32),
 * otherwise the SIMT kernels: for fp32 with block 32/64 and head_dim 32/64 the fused ones (one
 * forward and two backward launches, no score scratch), else one kernel per stage of the
 * reference's pipeline.  SPION_ENGINE_SIMT_STAGED forces the per-stage kernels.  Forcing an engine
 * that cannot run the shape gives UNSUPPORTED. */
int spion_set_engine(spion_ctx* ctx, int engine);

/* Reads the context's device status word (synchronises the stream).  Non-zero means a
 * bounded wait inside a kernel gave up; the word is cleared. */
int spion_check_device_status(spion_ctx* ctx);

/* Operand layout of the native (_ex / _fused) calls on the tcgen05 engine.
 *   heads == 0 (default): Q, K, V, O, dO, dQ, dK, dV are [BH, L, d], one matrix per (b,h) pair.
 *   heads == H > 0: they are [B, L, H, d] (B = num_batches / H), i.e. the [B, L, H*d] tensor a linear
 *   projection writes, read in place through a 2-D tensor map with a [64, d] box at column h*d.  This
 *   removes the head split / merge copies of models/attention.py:84-96,131-139 and the per-call
 *   flatten / permute copies of models/attention_blockcuda.py:47-49,78-80.  P, dS, lse and keypad keep
 *   their (b*H + h)-major layouts.  UNSUPPORTED on contexts the tcgen05 engine cannot run. */
int spion_set_head_layout(spion_ctx* ctx, int heads);

/* Masks of 32 x 32 blocks on the tcgen05 engine (bf16, head_dim 64) have two sets of kernels for the calls that
 * store no probabilities (spion_attn_forward_fused with P_optional == NULL, spion_attn_backward_fused):
 *   1: on the mask's own blocks (up to four selected blocks gathered into one 128-row operand; no unselected
 *      block is ever computed);
 *   2: on derived 64 x 64 super-blocks whose unselected quarters are masked (also what serves head_dim 32 and
 *      every call that stores P);
 *   0 (default): chosen when the mask is set -- 1 when the gathered operands are at least 70 % full on
 *      average (masks with three or more blocks per block row), else 2.
 * Takes effect when the next pattern is set.  No counterpart in the reference. */
int spion_set_block32_path(spion_ctx* ctx, int path);
/* Which of the two serves the current pattern: 1 or 2; 0 when the context is not a 32-wide mask on the tcgen05
 * engine (or no pattern is set). */
int spion_block32_path_in_use(const spion_ctx* ctx);

/* Failure-path self-test that faults nothing: launches one CTA that waits, with the given limit
 * in clock cycles (at most 2e9), on a barrier nobody arrives on.  The kernel gives up, records the
 * time-out in the status word and exits normally; the call then returns what
 * spion_check_device_status returns, i.e. SPION_ERR_TIMEOUT when the machinery works, and the
 * context stays usable. */
int spion_selftest_bounded_wait(spion_ctx* ctx, long long limit_cycles);

/* Number of kernels this context has launched since creation (bench bookkeeping). */
long long spion_launch_count(const spion_ctx* ctx);

/* Per-kernel timing of the pipelines (the reference has cudaEvent pairs around every stage,
 * all commented out: models/block_attn.cu:456-486).  enable != 0: CUDA events are recorded on the
 * context's stream between the kernels of every forward / backward call.  spion_profile_get
 * synchronises, folds the pending events in, and returns the total milliseconds and the number
 * of launches of one stage (SPION_STAGE_*); spion_profile_reset clears the totals. */
enum {
  SPION_STAGE_STRUCTURE = 0,   /* block CSR/CSC (re)build                         */
  SPION_STAGE_SDDMM_S = 1,     /* S = Q K^T on the mask                            */
  SPION_STAGE_SOFTMAX_FWD = 2, /* sparse row softmax                               */
  SPION_STAGE_SPMM_O = 3,      /* O = P V                                          */
  SPION_STAGE_SDDMM_DP = 4,    /* dP = dO V^T on the mask                          */
  SPION_STAGE_SOFTMAX_BWD = 5, /* dS from dP, P                                    */
  SPION_STAGE_SPMM_DQ = 6,     /* dQ = dS K                                        */
  SPION_STAGE_SPMM_DK = 7,     /* dK = dS^T Q                                      */
  SPION_STAGE_SPMM_DV = 8,     /* dV = P^T dO                                      */
  SPION_STAGE_FUSED_DP_DS = 9, /* (unused; kept so that the stage numbers stay stable)      */
  SPION_STAGE_SPMM_DKDV = 10,  /* fused kernels: dK and dV in one kernel           */
  SPION_STAGE_FUSED_FWD = 11,  /* fused kernels: S, softmax, P V in one kernel     */
  SPION_STAGE_BWD_ROW = 12,    /* fused kernels: dP, dS and dQ per block row (P read, dS written) */
  SPION_STAGE_BWD_ROW_RC = 13, /* recompute backward, row side: S, dP, dS on chip, dQ and delta written */
  SPION_STAGE_BWD_COL_RC = 14, /* recompute backward, column side: S, dP, P, dS on chip, dK and dV written */
  SPION_STAGE_COUNT = 15
};
int spion_profile(spion_ctx* ctx, int enable);
int spion_profile_get(spion_ctx* ctx, int stage, double* total_ms, long long* launches);
int spion_profile_reset(spion_ctx* ctx);
const char* spion_stage_name(int stage);

/* ------------------------------------------ reference-layout sparse attention ---- */

/* Replaces `attn_forward` of models/block_attn.cu:552-556 (keypad == NULL) and of
 * models/block_attn_mask.cu:660-663 (keypad = the `mask` argument, already multiplied
 * by 1e6: models/attention_blockcuda_mask.py:42-43; flat index bh*L + column).
 *   Q [BH,L,d]  Kt [BH,d,L]  V [BH,L,d]  attn [BH*nnz] (out: P in element-CSR order)
 *   out [BH,L,d]  offsets [L+1]  columns [>= nnz]  sum_mat [L]   (all int32)
 * nnz = selected elements per (b,h) matrix = Offsets[L]. */
int spion_block_attn_forward(spion_ctx* ctx, const float* Q, const float* Kt, const float* V,
                             const float* keypad, float* attn, float* out,
                             const int* offsets, const int* columns, const int* sum_mat, int nnz);

/* Replaces `attn_backward` of models/block_attn.cu:558-563 / models/block_attn_mask.cu:665-670.
 *   Q [BH,L,d]  K [BH,L,d]  Vt [BH,d,L]  P [BH*nnz]  dO [BH,L,d]
 *   dP_scratch, dS_scratch [BH*nnz] (caller-allocated, contents destroyed)
 *   dQ, dK, dV [BH,L,d] (out). */
int spion_block_attn_backward(spion_ctx* ctx, const float* Q, const float* K, const float* Vt,
                              const float* P, const float* dO, float* dP_scratch, float* dS_scratch,
                              float* dQ, float* dK, float* dV,
                              const int* offsets, const int* columns, const int* sum_mat, int nnz);

/* No counterpart in the reference.  stable != 0: the caller promises that the (offsets, columns,
 * sum_mat) arrays it passes to the two calls above stay allocated and unchanged for as long as it
 * passes them (a cache per mask, as spion_b200/attention_blockcuda.py keeps).  The block structure is
 * then rebuilt only when one of the three pointers or nnz changes, instead of on every forward and
 * every backward.  Default 0: the reference's own Python builds fresh arrays per call, whose
 * addresses are recycled and identify nothing. */
int spion_csr_arrays_are_stable(spion_ctx* ctx, int stable);

/* ------------------------------------------- reference-layout dense attention ---- */

/* Replaces `attn_forward` of models/attn.cu:269 (keypad == NULL) and models/attn_mask.cu:284.
 * Layouts as the reference's Python passes them (models/attention_cuda.py:18-36):
 *   Qt [BH,d,L]  K [BH,L,d]  Vt [BH,d,L]  attn [BH,L,L] stored transposed (attn[bh,j,i] = P[i,j])
 *   out [BH,d,L]. */
int spion_dense_attn_forward(spion_ctx* ctx, const float* Qt, const float* K, const float* Vt,
                             const float* keypad, float* attn, float* out);

/* Replaces `attn_backward` of models/attn.cu:273 / models/attn_mask.cu:288
 * (models/attention_cuda.py:39-74):
 *   Qt [BH,d,L]  Kt [BH,d,L]  V [BH,L,d]  attn [BH,L,L] (as written by forward)  dOt [BH,d,L]
 *   s1, s2, s3 [BH*L*L] caller scratch (s1 receives dP, s3 receives dS; s2 is not touched)
 *   dQt, dKt, dVt [BH,d,L] (out). */
int spion_dense_attn_backward(spion_ctx* ctx, const float* Qt, const float* Kt, const float* V,
                              const float* attn, const float* dOt, float* s1, float* s2, float* s3,
                              float* dQt, float* dKt, float* dVt);

/* Head/batch mean of the dense attention tensor (models/model_transformer.py:137):
 * A[i,j] = mean_h mean_b P[b,h,i,j].  `attn` is [B*H, L, L]; transposed != 0 means it is
 * stored as spion_dense_attn_forward writes it. */
int spion_mean_attention_map(const float* attn, int batch, int heads, int L, int transposed,
                             float* A, void* cuda_stream);

/* The same mean taken from block-tile probabilities ([BH, nnzb, bs, bs], what the native forward
 * returns): with the full mask this is the warm-up phase without a [B,H,L,L] tensor in the
 * reference's layout.  Cells of unselected blocks are 0.  blk_row / col_idx: block CSR (device). */
int spion_mean_map_tiles(const void* P, int dtype, const int32_t* blk_row, const int32_t* col_idx,
                         int block_size, int nnzb, int num_batches, int L, float* A, void* cuda_stream);

/* ------------------------------------------------------------ pattern discovery ---- */

/* Replaces the inline driver block main_conv_ff.py:255-279 (and its flood_fill, :35-62):
 *   pooled = avg_pool(conv(A)) ; thresh = quantile(pooled, param) ; 2*nb greedy walkers ;
 *   binarise ; force the diagonal ; block CSR + CSC.
 * select = SPION_SELECT_TOPK replaces main_conv.py:246-251 (param = density).
 * F = 1 skips the convolution (main_ff.py:255).
 *   A [L,L] fp32            mat [nb*nb] uint8 (out)       pooled [nb*nb] fp32 (out)
 *   thresh [1] fp32 (out)   nnzb [1] int32 (out)
 *   row_ptr [nb+1], col_idx [nb*nb], blk_row [nb*nb]      block CSR (out; first nnzb entries valid)
 *   col_ptr [nb+1], row_idx [nb*nb], csc_pos [nb*nb]      block CSC (out; csc_pos = CSR block id)
 *   work [nb*nb] int32 scratch
 * host_nnzb: if not NULL the call synchronises the stream and stores the block count. */
int spion_discover_pattern(const float* A, int L, int block_size, int conv_kind, int F,
                           int select, double param,
                           uint8_t* mat, float* pooled, float* thresh, int32_t* nnzb,
                           int32_t* row_ptr, int32_t* col_idx, int32_t* blk_row,
                           int32_t* col_ptr, int32_t* row_idx, int32_t* csc_pos,
                           int32_t* work, int32_t* host_nnzb, void* cuda_stream);

/* Block CSR + CSC of a given 0/1 mask (e.g. one loaded from the reference's pickle,
 * main_inference.py:164-166).  Same outputs as above. */
int spion_build_structure(const uint8_t* mat, int nb, int32_t* nnzb,
                          int32_t* row_ptr, int32_t* col_idx, int32_t* blk_row,
                          int32_t* col_ptr, int32_t* row_idx, int32_t* csc_pos,
                          int32_t* work, int32_t* host_nnzb, void* cuda_stream);

/* Replaces the per-call CSR construction of models/attention_blockcuda.py:31-43:
 *   sum_mat [L], offsets [L+1], columns [repeat * nnz]  (int32), nnz = nnzb * bs^2. */
int spion_expand_csr(const int32_t* row_ptr, const int32_t* col_idx, int nb, int block_size,
                     int nnzb, int repeat, int32_t* sum_mat, int32_t* offsets, int32_t* columns,
                     void* cuda_stream);

/* ------------------------------------------------------- native (block-tile) API ---- */

/* Fix the layer's block mask for the native calls (done once per layer at discovery,
 * where the reference calls reconstruct_for_blocksparse, models/attention.py:105).
 * mat [nb*nb] uint8 device.  Synchronises once to learn the block count. */
int spion_set_pattern(spion_ctx* ctx, const uint8_t* mat);
int spion_pattern_nnzb(const spion_ctx* ctx);

/* Native forward.  dtype = the context's (fp32 or bf16 elements).
 *   Q, K, V, O  [BH,L,d] row-major (no transposed copies: compare attention_blockcuda.py:48)
 *   P           [BH, nnzb, bs, bs] block tiles in CSR block order (out; needed by backward)
 *   keypad      [BH*L] fp32 penalty (1e6 on padded keys) or NULL
 *   S_scratch   [BH*nnzb*bs*bs] fp32, used by the per-stage SIMT kernels only (NULL allowed when
 *               spion_needs_scratch() is 0).
 * On the tcgen05 engine and with the fused fp32 kernels this is one forward kernel with the
 * probabilities stored. */
int spion_attn_forward_ex(spion_ctx* ctx, const void* Q, const void* K, const void* V,
                          const float* keypad, void* P, void* O, float* S_scratch);

/* Native backward.
 *   dS          [BH, nnzb, bs, bs] elements of the context dtype (scratch, written)
 *   O           the forward output: required on the tcgen05 engine; the fused fp32 kernels use it
 *               when given (one pass over a block row instead of two), NULL allowed there
 *   dP_scratch  [BH*nnzb*bs*bs] fp32, used by the per-stage SIMT kernels only
 *   delta       unused (may be NULL)
 *   dQ, dK, dV  [BH,L,d] (out). */
int spion_attn_backward_ex(spion_ctx* ctx, const void* Q, const void* K, const void* V,
                           const void* P, const void* O, const void* dO,
                           void* dS, float* dP_scratch, float* delta,
                           void* dQ, void* dK, void* dV);

/* 1 when spion_attn_forward_ex / spion_attn_backward_ex of this context need their fp32 scratch
 * arguments (the per-stage SIMT kernels run), 0 when they may be NULL.  No reference counterpart
 * (the reference allocates its backward scratch on every call, models/attention_blockcuda.py:84-85). */
int spion_needs_scratch(const spion_ctx* ctx);

/* Fused native forward (tcgen05 engine only; UNSUPPORTED otherwise).  S never reaches HBM: one
 * kernel computes the scores of a block row in tensor memory, the sparse row softmax in registers and
 * O = P V from shared memory.  It writes O and one fp32 log-sum-exp value per row (lse [BH*L], log2
 * domain, including the reference's non-selected-key term of models/block_attn.cu:71).
 * P_optional: if not NULL the [BH, nnzb, bs, bs] probabilities are stored as well (what the reference
 * returns as `attn`, and what spion_attn_backward_ex reads). */
int spion_supports_fused(const spion_ctx* ctx);   /* 1 if the fused call can run this context */
int spion_attn_forward_fused(spion_ctx* ctx, const void* Q, const void* K, const void* V,
                             const float* keypad, void* O, float* lse, void* P_optional);

/* Fused native backward (tcgen05 engine only; UNSUPPORTED otherwise): the counterpart of
 * spion_attn_forward_fused called with P_optional == NULL.  Neither P nor dS exists in global memory:
 * both kernels rebuild their tiles from Q, K, V, dO and the forward's log-sum-exp (replaces
 * models/block_attn.cu:489-545 and the two nnz-sized scratch arrays of models/attention_blockcuda.py:84-85).
 *   O, dO [as Q]   lse [BH*L] as written by spion_attn_forward_fused   keypad as passed to the forward
 *   dQ, dK, dV (out).  The context keeps one [BH*L] fp32 array (delta) between its two kernels. */
int spion_attn_backward_fused(spion_ctx* ctx, const void* Q, const void* K, const void* V,
                              const void* O, const void* dO, const float* lse, const float* keypad,
                              void* dQ, void* dK, void* dV);

/* Head / batch mean of the probabilities of the current pattern (models/model_transformer.py:137) from
 * Q, K and the forward's log-sum-exp, without a stored P (tcgen05 engine only): A [L, L] fp32, zero
 * outside the selected blocks.  With the full mask this is the warm-up phase's attention map. */
int spion_mean_map_recompute(spion_ctx* ctx, const void* Q, const void* K, const float* lse,
                             const float* keypad, float* A);

/* Stand-alone sparse row softmax on block tiles (the kernels of models/block_attn.cu:33-130):
 * forward S (fp32 tiles) -> P (context dtype), backward (dP fp32, P) -> dS (context dtype). */
int spion_softmax_forward_ex(spion_ctx* ctx, const float* S, const float* keypad, void* P);
int spion_softmax_backward_ex(spion_ctx* ctx, const float* dP, const void* P, void* dS);

/* ---------------------------------------------------------- no-allocation forward ---- */

/* No counterpart in the reference.  Native forward (same math and layouts as
 * spion_attn_forward_ex on the SIMT engine) for callers that must not allocate device memory
 * -- a plugin inside a process whose GPU memory is fully budgeted, a real-time loop, code that
 * runs where cudaMalloc is off limits: no context, no caller scratch.  The fp32 score scratch
 * lives in a fixed array inside the library (spion_static_scratch_capacity() floats, 64 MiB,
 * held by every GPU that loads the library).  num_batches*nnzb*block_size^2 beyond that is
 * refused with SPION_ERR_SHAPE.  The array is shared by all calls on a device: calls that overlap
 * on the GPU race.  The first call on each device looks up the array's address; make it outside
 * stream capture (the address is kept per device and does not survive a device reset).
 * row_ptr [nb+1], col_idx [nnzb], blk_row [nnzb]: block CSR (device); nnzb must be that CSR's own
 * block count (row_ptr[nb] == nnzb; nnzb > nb*nb is refused), because the capacity check uses it. */
size_t spion_static_scratch_capacity(void);
int spion_attn_forward_static(const void* Q, const void* K, const void* V, const float* keypad,
                              void* P, void* O, const int32_t* row_ptr, const int32_t* col_idx,
                              const int32_t* blk_row, int head_dim, int seq_len, int num_batches,
                              int block_size, int nnzb, int dtype, void* cuda_stream);

/* ------------------------------------------------------------------------------------------
 * Layer normalisation of the encoder layers around the attention call (the reference uses
 * torch.nn.LayerNorm: models/model_transformer.py).  [M, N] fp32 rows, N in {64, 128, 256, 512};
 * biased variance, eps inside the square root.  y / dy are fp32 (is_bf16 == 0) or bf16.  mean, rstd: [M]
 * (written by the forward, read by the backward).  The backward also returns the weight and bias
 * gradients [N], summed in a fixed order (deterministic); workspace: spion_layernorm_workspace_floats(N)
 * floats.  No context: the calls run on the stream given. */
int spion_layernorm_forward(const float* x, const float* gamma, const float* beta, void* y, int y_is_bf16,
                            float* mean, float* rstd, long long M, int N, float eps, void* cuda_stream);
long long spion_layernorm_workspace_floats(int N);
int spion_layernorm_backward(const float* x, const void* dy, int dy_is_bf16, const float* gamma, const float* mean,
                             const float* rstd, float* dx, float* dgamma, float* dbeta, float* workspace,
                             long long M, int N, void* cuda_stream);

/* Residual connection + normalisation in one pass (X = branch + X; norm(X) in the reference's encoder layer,
 * models/model_transformer.py): sum_out = x + res (x fp32; res fp32, or bf16 with res_is_bf16 != 0),
 * y = LayerNorm(sum_out); mean / rstd as spion_layernorm_forward.  sum_out must not alias x or res. */
int spion_add_layernorm_forward(const float* x, const void* res, int res_is_bf16, float* sum_out, const float* gamma,
                                const float* beta, void* y, int y_is_bf16, float* mean, float* rstd, long long M, int N,
                                float eps, void* cuda_stream);
/* Its backward: x is the saved sum; dx = (gradient through the normalisation) + dskip, where dskip (may be NULL) is
 * the gradient the sum receives from its other consumers; dx is the gradient of both addends, dx_bf16 (may be NULL)
 * receives a bf16 copy of it.  dgamma, dbeta, workspace as spion_layernorm_backward. */
int spion_add_layernorm_backward(const float* x, const void* dy, int dy_is_bf16, const float* gamma, const float* mean,
                                 const float* rstd, const float* dskip, float* dx, void* dx_bf16, float* dgamma,
                                 float* dbeta, float* workspace, long long M, int N, void* cuda_stream);

/* Sum of the rows of an [M, N] matrix (fp32, or bf16 with dy_is_bf16 != 0), N in {64, 128, 256, 512}: out [N] fp32.
 * The bias gradient of a linear layer (torch.nn.Linear in the reference's encoder) as one streaming pass plus a
 * fixed-order reduction.  workspace: spion_layernorm_workspace_floats(N) floats. */
int spion_column_sums(const void* dy, int dy_is_bf16, float* out, float* workspace, long long M, int N,
                      void* cuda_stream);

/* Weight gradient of a token embedding with a small table (torch.nn.Embedding(vocab_size, embedding_dim) in the
 * reference's encoder, models/model_transformer.py; vocab_size 256 - 512 in its tasks):
 *   dW[v, :] = sum over tokens t with ids[t] == v of g[t, :]
 * ids [T] int64, g [T, N] fp32 (or bf16 with g_is_bf16 != 0), both 16-byte aligned; dW [V, N] fp32 is overwritten;
 * ids outside [0, V) are skipped.  N in {32, 64, 128, 256}, V * N <= 24576 (the table is kept in shared memory).
 * workspace: spion_embedding_workspace_floats(T, V, N) floats.  Fixed summation order: same bits on every run. */
long long spion_embedding_workspace_floats(long long T, int V, int N);
/* Token + position embedding of the encoder input in one pass (models/model_transformer.py, Embeddings):
 * out[t, :] = tok[ids[t], :] + pos[t % L, :] for t in [0, T), T = batch * L; tok [V, N], pos [>= L, N], out [T, N] fp32,
 * 16-byte aligned, N a multiple of 4; an id outside [0, V) gives the position row alone. */
int spion_embedding_forward(const long long* ids, const float* tok, const float* pos, float* out, long long T, int L,
                            int V, int N, void* cuda_stream);
int spion_embedding_backward(const long long* ids, const void* g, int g_is_bf16, long long T, int V, int N,
                             float* dW, float* workspace, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* SPION_B200_H */
