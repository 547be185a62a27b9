// C ABI of spion_b200: contexts, the reference-layout entry points and the native ones.
// Orchestration only; kernels live in simt_fused.cu, simt_attn.cu, structure.cu, pattern.cu, tc_fused.cu, tc_engine.cu.
//
// Pipelines (reference: Attention::attn_forward / attn_backward, models/block_attn.cu:453-545):
//   forward   S = Q K^T on the mask  ->  P = sparse row softmax(S)  ->  O = P V
//   backward  dP = dO V^T on the mask -> dS = softmax'(dP, P) -> dQ = dS K ; dK = dS^T Q ; dV = P^T dO
#include <new>

#include "common.cuh"

namespace {

struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
    // Always, not only when the device differs: cudaSetDevice also binds the device's primary context to the
    // calling thread, which the driver entry point that encodes tensor maps needs (a thread of the autograd
    // engine that has not launched anything yet has no context bound, cudaGetDevice does not bind one).
    if (dev >= 0) ok = cudaSetDevice(dev) == cudaSuccess;
  }
  ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

template <typename T>
bool dev_alloc(T** p, size_t n) { return cudaMalloc((void**)p, n * sizeof(T)) == cudaSuccess; }

int rebuild_structure(spion_ctx* c) {
  c->launches += 1;
  return spion_launch_build_structure(c->mat, c->nb, c->nnzb_dev, c->row_ptr, c->col_idx, c->blk_row, c->col_ptr,
                                      c->row_idx, c->csc_pos, c->work, c->stream);
}

bool is_dense(const spion_ctx* c) { return c->kind == SPION_KIND_DENSE || c->kind == SPION_KIND_DENSE_KPM; }
bool is_kpm(const spion_ctx* c) { return c->kind == SPION_KIND_DENSE_KPM || c->kind == SPION_KIND_BLOCK_KPM; }

}  // namespace

extern "C" const char* spion_status_string(int s) {
  switch (s) {
    case SPION_OK: return "ok";
    case SPION_ERR_ARG: return "bad argument";
    case SPION_ERR_SHAPE: return "unsupported shape";
    case SPION_ERR_CUDA: return "CUDA error";
    case SPION_ERR_TIMEOUT: return "device-side wait timed out";
    case SPION_ERR_UNSUPPORTED: return "combination not supported";
    case SPION_ERR_ALLOC: return "allocation failed";
    case SPION_ERR_STATE: return "call order";
    default: return "unknown status";
  }
}

extern "C" int spion_version(void) { return 100; }

extern "C" spion_ctx* spion_create(int kind, int head_dim, int seq_len, int num_batches, int block_size, int dtype,
                                   int device) {
  if (kind < SPION_KIND_DENSE || kind > SPION_KIND_BLOCK_KPM) return nullptr;
  if (head_dim < 1 || seq_len < 1 || num_batches < 1) return nullptr;
  if (dtype != SPION_F32 && dtype != SPION_BF16) return nullptr;
  const bool dense = kind == SPION_KIND_DENSE || kind == SPION_KIND_DENSE_KPM;
  int bs = block_size;
  if (dense) bs = (seq_len % 64 == 0) ? 64 : 32;          // internal tiling of the dense surface
  if (bs < 1 || seq_len % bs != 0) return nullptr;         // the reference truncates silently: int(L/bs)
  const int nb = seq_len / bs;
  if (nb > SPION_MAX_NB) return nullptr;

  DeviceGuard guard(device);
  if (!guard.ok) return nullptr;
  spion_ctx* c = new (std::nothrow) spion_ctx();
  if (!c) return nullptr;
  c->kind = kind; c->d = head_dim; c->L = seq_len; c->BH = num_batches; c->bs = bs; c->nb = nb;
  c->dtype = dtype; c->engine = SPION_ENGINE_AUTO;
  cudaGetDevice(&c->device);
  c->scale = 1.0f / sqrtf((float)head_dim);               // models/block_attn.cu:419
  c->stream = 0;
  c->nnzb = -1;
  c->launches = 0;
  c->tc = nullptr;
  c->heads = 0;
  c->block32_path = 0;
  c->csr_stable = 0; c->csr_key[0] = c->csr_key[1] = c->csr_key[2] = nullptr; c->csr_nnz = -1;
  c->prof_on = 0; c->prof_n = 0;
  for (int i = 0; i < SPION_PROF_MAX_MARKS; ++i) { c->prof_ev[i] = nullptr; c->prof_stage[i] = -1; }
  for (int i = 0; i < SPION_STAGE_COUNT; ++i) { c->prof_ms[i] = 0; c->prof_cnt[i] = 0; }
  const size_t cap = (size_t)nb * nb;
  bool ok = dev_alloc(&c->mat, cap) && dev_alloc(&c->row_ptr, (size_t)nb + 1) && dev_alloc(&c->col_idx, cap) &&
            dev_alloc(&c->blk_row, cap) && dev_alloc(&c->col_ptr, (size_t)nb + 1) && dev_alloc(&c->row_idx, cap) &&
            dev_alloc(&c->csc_pos, cap) && dev_alloc(&c->work, cap) && dev_alloc(&c->nnzb_dev, 1) &&
            dev_alloc(&c->status_dev, 1);
  if (ok) ok = cudaMemset(c->status_dev, 0, sizeof(int)) == cudaSuccess;
  if (ok && dense) {
    ok = spion_launch_fill_mat(c->mat, (int)cap, 1, 0) == SPION_OK && rebuild_structure(c) == SPION_OK &&
         cudaStreamSynchronize(0) == cudaSuccess;
    c->nnzb = (int)cap;
  }
  if (!ok) { spion_destroy(c); return nullptr; }
  return c;
}

extern "C" void spion_destroy(spion_ctx* c) {
  if (!c) return;
  DeviceGuard guard(c->device);
  tc_engine_release(c);
  for (int i = 0; i < SPION_PROF_MAX_MARKS; ++i) if (c->prof_ev[i]) cudaEventDestroy(c->prof_ev[i]);
  cudaFree(c->mat); cudaFree(c->row_ptr); cudaFree(c->col_idx); cudaFree(c->blk_row); cudaFree(c->col_ptr);
  cudaFree(c->row_idx); cudaFree(c->csc_pos); cudaFree(c->work); cudaFree(c->nnzb_dev); cudaFree(c->status_dev);
  delete c;
}

extern "C" int spion_set_stream(spion_ctx* c, void* cuda_stream) {
  if (!c) return SPION_ERR_ARG;
  c->stream = (cudaStream_t)cuda_stream;
  return SPION_OK;
}

extern "C" int spion_set_engine(spion_ctx* c, int engine) {
  if (!c || engine < SPION_ENGINE_AUTO || engine > SPION_ENGINE_SIMT_STAGED) return SPION_ERR_ARG;
  if (engine == SPION_ENGINE_TCGEN05 && !tc_engine_supports(c)) return SPION_ERR_UNSUPPORTED;
  if ((engine == SPION_ENGINE_SIMT || engine == SPION_ENGINE_SIMT_STAGED) && c->heads != 0) return SPION_ERR_UNSUPPORTED;
  c->engine = engine;
  return SPION_OK;
}

extern "C" int spion_check_device_status(spion_ctx* c) {
  if (!c) return SPION_ERR_ARG;
  int word = 0;
  SPION_CUDA_TRY(cudaMemcpyAsync(&word, c->status_dev, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  SPION_CUDA_TRY(cudaStreamSynchronize(c->stream));
  if (word != 0) {
    SPION_CUDA_TRY(cudaMemsetAsync(c->status_dev, 0, sizeof(int), c->stream));
    fprintf(stderr, "spion_b200: device status word = 0x%x (a bounded wait gave up)\n", word);
    return SPION_ERR_TIMEOUT;
  }
  return SPION_OK;
}

extern "C" int spion_csr_arrays_are_stable(spion_ctx* c, int stable) {
  if (!c) return SPION_ERR_ARG;
  c->csr_stable = stable != 0;
  c->csr_key[0] = c->csr_key[1] = c->csr_key[2] = nullptr;
  c->csr_nnz = -1;
  return SPION_OK;
}

extern "C" int spion_set_head_layout(spion_ctx* c, int heads) {
  if (!c || heads < 0) return SPION_ERR_ARG;
  if (heads > 0) {
    if (is_dense(c) || !tc_engine_supports(c)) return SPION_ERR_UNSUPPORTED;   // the SIMT kernels address [BH, L, d] only
    if (c->BH % heads != 0) return SPION_ERR_SHAPE;
  }
  c->heads = heads;
  return SPION_OK;
}

extern "C" int spion_set_block32_path(spion_ctx* c, int path) {
  if (!c || path < 0 || path > 2) return SPION_ERR_ARG;
  c->block32_path = path;
  return SPION_OK;
}

extern "C" int spion_selftest_bounded_wait(spion_ctx* c, long long limit_cycles) {
  if (!c || limit_cycles < 1 || limit_cycles > 2000000000LL) return SPION_ERR_ARG;
  DeviceGuard guard(c->device);
  int rc = tc_engine_wait_selftest(c, limit_cycles);
  if (rc) return rc;
  return spion_check_device_status(c);      // expected: SPION_ERR_TIMEOUT, and the word is cleared again
}

extern "C" long long spion_launch_count(const spion_ctx* c) { return c ? c->launches : 0; }

// ------------------------------------------------------------ per-stage timing
int prof_drain(spion_ctx* c) {
  if (c->prof_n == 0) return SPION_OK;
  SPION_CUDA_TRY(cudaEventSynchronize(c->prof_ev[c->prof_n - 1]));
  for (int i = 1; i < c->prof_n; ++i) {
    const int st = c->prof_stage[i];
    if (st < 0) continue;
    float ms = 0.f;
    SPION_CUDA_TRY(cudaEventElapsedTime(&ms, c->prof_ev[i - 1], c->prof_ev[i]));
    c->prof_ms[st] += ms;
    c->prof_cnt[st] += 1;
  }
  c->prof_n = 0;
  return SPION_OK;
}

int prof_mark(spion_ctx* c, int stage) {
  if (!c->prof_on) return SPION_OK;
  if (stage < 0 && c->prof_n > SPION_PROF_MAX_MARKS - 16) {
    int rc = prof_drain(c);
    if (rc) return rc;
  }
  if (c->prof_n >= SPION_PROF_MAX_MARKS) return SPION_OK;
  if (!c->prof_ev[c->prof_n]) SPION_CUDA_TRY(cudaEventCreate(&c->prof_ev[c->prof_n]));
  SPION_CUDA_TRY(cudaEventRecord(c->prof_ev[c->prof_n], c->stream));
  c->prof_stage[c->prof_n] = stage;
  c->prof_n += 1;
  return SPION_OK;
}

extern "C" int spion_profile(spion_ctx* c, int enable) {
  if (!c) return SPION_ERR_ARG;
  DeviceGuard guard(c->device);
  if (!enable && c->prof_on) { int rc = prof_drain(c); if (rc) return rc; }
  c->prof_on = enable != 0;
  return SPION_OK;
}

extern "C" int spion_profile_get(spion_ctx* c, int stage, double* total_ms, long long* launches) {
  if (!c || stage < 0 || stage >= SPION_STAGE_COUNT) return SPION_ERR_ARG;
  DeviceGuard guard(c->device);
  int rc = prof_drain(c);
  if (rc) return rc;
  if (total_ms) *total_ms = c->prof_ms[stage];
  if (launches) *launches = c->prof_cnt[stage];
  return SPION_OK;
}

extern "C" int spion_profile_reset(spion_ctx* c) {
  if (!c) return SPION_ERR_ARG;
  DeviceGuard guard(c->device);
  int rc = prof_drain(c);
  for (int i = 0; i < SPION_STAGE_COUNT; ++i) { c->prof_ms[i] = 0; c->prof_cnt[i] = 0; }
  return rc;
}

extern "C" const char* spion_stage_name(int stage) {
  static const char* names[SPION_STAGE_COUNT] = {
      "structure", "sddmm_s", "softmax_fwd", "spmm_o", "sddmm_dp", "softmax_bwd", "spmm_dq", "spmm_dk", "spmm_dv",
      "fused_dp_ds", "spmm_dkdv", "fused_fwd", "bwd_row", "bwd_row_rc", "bwd_col_rc"};
  return (stage >= 0 && stage < SPION_STAGE_COUNT) ? names[stage] : "?";
}

// fp32 contexts run the fused SIMT kernels unless the per-stage ones are forced
static bool use_simt_fused(const spion_ctx* c, int value_mode) {
  return c->dtype == SPION_F32 && c->engine != SPION_ENGINE_SIMT_STAGED &&
         simt_fused_supports(c->bs, c->d, c->BH, value_mode);
}

// ============================================================ reference-layout sparse
// The block structure is derived from the caller's element CSR on every call: the reference's Python
// rebuilds those arrays for each forward (models/attention_blockcuda.py:26-43), usually into recycled
// allocations, so their addresses say nothing about their contents.  A caller that keeps the arrays
// alive and unchanged for as long as it passes them (spion_csr_arrays_are_stable) skips the rebuild
// when the same three pointers and nnz come back.
static int legacy_structure(spion_ctx* c, const int* offsets, const int* columns, const int* sum_mat, int nnz) {
  if (nnz < 0 || nnz % (c->bs * c->bs) != 0) return SPION_ERR_SHAPE;
  const int nnzb = nnz / (c->bs * c->bs);
  if (nnzb > c->nb * c->nb) return SPION_ERR_SHAPE;
  if (c->csr_stable && c->csr_key[0] == offsets && c->csr_key[1] == columns && c->csr_key[2] == sum_mat &&
      c->csr_nnz == nnz && c->nnzb == nnzb) {
    prof_mark(c, -1);
    return SPION_OK;
  }
  c->csr_key[0] = offsets; c->csr_key[1] = columns; c->csr_key[2] = sum_mat; c->csr_nnz = nnz;
  prof_mark(c, -1);
  int rc = spion_launch_mat_from_elemcsr(offsets, columns, sum_mat, c->nb, c->bs, c->mat, c->stream);
  if (rc) return rc;
  c->launches += 1;
  rc = rebuild_structure(c);
  if (rc) return rc;
  prof_mark(c, SPION_STAGE_STRUCTURE);
  c->nnzb = nnzb;
  return SPION_OK;
}

extern "C" int spion_block_attn_forward(spion_ctx* c, const float* Q, const float* Kt, const float* V,
                                        const float* keypad, float* attn, float* out, const int* offsets,
                                        const int* columns, const int* sum_mat, int nnz) {
  if (!c || !Q || !Kt || !V || !attn || !out || !offsets || !columns || !sum_mat) return SPION_ERR_ARG;
  if (is_dense(c) || c->dtype != SPION_F32) return SPION_ERR_STATE;
  if (is_kpm(c) && !keypad) return SPION_ERR_ARG;
  DeviceGuard guard(c->device);
  int rc = legacy_structure(c, offsets, columns, sum_mat, nnz);
  if (rc) return rc;
  const Pattern p = ctx_pattern(c);
  const ValueLayout vl{VAL_ELEMCSR, c->L, (long long)nnz};
  const OperandLayout rm = row_major_operand(c->L, c->d), tr = transposed_operand(c->L, c->d);
  // floor of the running maximum: -100 (models/block_attn.cu:48) or 0 (models/block_attn_mask.cu:105)
  if (use_simt_fused(c, VAL_ELEMCSR)) {
    rc = simt_fused_forward(Q, rm, Kt, tr, V, rm, is_kpm(c) ? keypad : nullptr, is_kpm(c) ? 0.0f : -100.0f, attn, vl, out,
                            rm, p, c->BH, c->L, c->d, c->scale, c->stream);
    if (!rc) prof_mark(c, SPION_STAGE_FUSED_FWD);
    c->launches += 1;
    return rc;
  }
  rc = simt_sddmm(SPION_F32, SPION_F32, Q, rm, Kt, tr, attn, vl, p, c->nnzb, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SDDMM_S);
  if (rc) return rc;
  rc = softmax_fwd_rows(SPION_F32, attn, vl, attn, vl, p, c->BH, c->L, c->scale, is_kpm(c) ? keypad : nullptr,
                        is_kpm(c) ? 0.0f : -100.0f, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SOFTMAX_FWD);
  if (rc) return rc;
  rc = simt_spmm(SPION_F32, SPION_F32, false, attn, vl, V, rm, out, rm, p, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SPMM_O);
  c->launches += 3;
  return rc;
}

extern "C" int spion_block_attn_backward(spion_ctx* c, const float* Q, const float* K, const float* Vt, const float* P,
                                         const float* dO, float* dP_scratch, float* dS_scratch, float* dQ, float* dK,
                                         float* dV, const int* offsets, const int* columns, const int* sum_mat,
                                         int nnz) {
  if (!c || !Q || !K || !Vt || !P || !dO || !dP_scratch || !dS_scratch || !dQ || !dK || !dV || !offsets || !columns ||
      !sum_mat)
    return SPION_ERR_ARG;
  if (is_dense(c) || c->dtype != SPION_F32) return SPION_ERR_STATE;
  DeviceGuard guard(c->device);
  int rc = legacy_structure(c, offsets, columns, sum_mat, nnz);
  if (rc) return rc;
  const Pattern p = ctx_pattern(c);
  const ValueLayout vl{VAL_ELEMCSR, c->L, (long long)nnz};
  const OperandLayout rm = row_major_operand(c->L, c->d), tr = transposed_operand(c->L, c->d);
  if (use_simt_fused(c, VAL_ELEMCSR)) {
    c->launches += 2;
    return simt_fused_backward(Q, rm, K, rm, Vt, tr, P, vl, nullptr, rm, dO, rm, dS_scratch, vl, dQ, rm, dK, rm, dV, rm, p, c->BH, c->d,
                               c->scale, c->stream, c);
  }
  rc = simt_sddmm(SPION_F32, SPION_F32, dO, rm, Vt, tr, dP_scratch, vl, p, c->nnzb, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SDDMM_DP);
  if (rc) return rc;
  rc = softmax_bwd_rows(SPION_F32, dP_scratch, vl, P, vl, dS_scratch, vl, p, c->BH, c->L, c->scale, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SOFTMAX_BWD);
  if (rc) return rc;
  rc = simt_spmm(SPION_F32, SPION_F32, false, dS_scratch, vl, K, rm, dQ, rm, p, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SPMM_DQ);
  if (rc) return rc;
  rc = simt_spmm(SPION_F32, SPION_F32, true, dS_scratch, vl, Q, rm, dK, rm, p, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SPMM_DK);
  if (rc) return rc;
  rc = simt_spmm(SPION_F32, SPION_F32, true, P, vl, dO, rm, dV, rm, p, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SPMM_DV);
  c->launches += 5;
  return rc;
}

// ============================================================ reference-layout dense
extern "C" int spion_dense_attn_forward(spion_ctx* c, const float* Qt, const float* K, const float* Vt,
                                        const float* keypad, float* attn, float* out) {
  if (!c || !Qt || !K || !Vt || !attn || !out) return SPION_ERR_ARG;
  if (!is_dense(c) || c->dtype != SPION_F32) return SPION_ERR_STATE;
  if (is_kpm(c) && !keypad) return SPION_ERR_ARG;
  DeviceGuard guard(c->device);
  const Pattern p = ctx_pattern(c);
  const ValueLayout vl{VAL_DENSE_T, c->L, (long long)c->L * c->L};
  const OperandLayout rm = row_major_operand(c->L, c->d), tr = transposed_operand(c->L, c->d);
  prof_mark(c, -1);
  int rc = simt_sddmm(SPION_F32, SPION_F32, Qt, tr, K, rm, attn, vl, p, c->nnzb, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SDDMM_S);
  if (rc) return rc;
  // running-maximum floor -10 (models/attn.cu:21); key padding as models/attn_mask.cu:20
  rc = softmax_fwd_dense_t(attn, c->BH, c->L, c->scale, is_kpm(c) ? keypad : nullptr, -10.0f, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SOFTMAX_FWD);
  if (rc) return rc;
  rc = simt_spmm(SPION_F32, SPION_F32, false, attn, vl, Vt, tr, out, tr, p, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SPMM_O);
  c->launches += 3;
  return rc;
}

extern "C" int spion_dense_attn_backward(spion_ctx* c, const float* Qt, const float* Kt, const float* V,
                                         const float* attn, const float* dOt, float* s1, float* s2, float* s3,
                                         float* dQt, float* dKt, float* dVt) {
  (void)s2;
  if (!c || !Qt || !Kt || !V || !attn || !dOt || !s1 || !s3 || !dQt || !dKt || !dVt) return SPION_ERR_ARG;
  if (!is_dense(c) || c->dtype != SPION_F32) return SPION_ERR_STATE;
  DeviceGuard guard(c->device);
  const Pattern p = ctx_pattern(c);
  const ValueLayout vl{VAL_DENSE_T, c->L, (long long)c->L * c->L};
  const OperandLayout rm = row_major_operand(c->L, c->d), tr = transposed_operand(c->L, c->d);
  prof_mark(c, -1);
  int rc = simt_sddmm(SPION_F32, SPION_F32, dOt, tr, V, rm, s1, vl, p, c->nnzb, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SDDMM_DP);
  if (rc) return rc;
  rc = softmax_bwd_dense_t(s1, attn, s3, c->BH, c->L, c->scale, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SOFTMAX_BWD);
  if (rc) return rc;
  rc = simt_spmm(SPION_F32, SPION_F32, false, s3, vl, Kt, tr, dQt, tr, p, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SPMM_DQ);
  if (rc) return rc;
  rc = simt_spmm(SPION_F32, SPION_F32, true, s3, vl, Qt, tr, dKt, tr, p, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SPMM_DK);
  if (rc) return rc;
  rc = simt_spmm(SPION_F32, SPION_F32, true, attn, vl, dOt, tr, dVt, tr, p, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SPMM_DV);
  c->launches += 5;
  return rc;
}

// ============================================================ native (block-tile) API
extern "C" int spion_set_pattern(spion_ctx* c, const uint8_t* mat) {
  if (!c || !mat) return SPION_ERR_ARG;
  if (is_dense(c)) return SPION_ERR_STATE;
  DeviceGuard guard(c->device);
  SPION_CUDA_TRY(cudaMemcpyAsync(c->mat, mat, (size_t)c->nb * c->nb, cudaMemcpyDeviceToDevice, c->stream));
  int rc = rebuild_structure(c);
  if (rc) return rc;
  int32_t n = 0;
  SPION_CUDA_TRY(cudaMemcpyAsync(&n, c->nnzb_dev, sizeof(int32_t), cudaMemcpyDeviceToHost, c->stream));
  SPION_CUDA_TRY(cudaStreamSynchronize(c->stream));
  c->nnzb = n;
  if (tc_engine_supports(c)) {
    rc = tc_engine_prepare(c);
    if (rc) return rc;
  }
  return SPION_OK;
}

extern "C" int spion_pattern_nnzb(const spion_ctx* c) { return c ? c->nnzb : SPION_ERR_ARG; }

static bool use_tc(const spion_ctx* c) {
  if (c->engine == SPION_ENGINE_SIMT || c->engine == SPION_ENGINE_SIMT_STAGED) return false;
  return tc_engine_supports(c);
}

extern "C" int spion_attn_forward_ex(spion_ctx* c, const void* Q, const void* K, const void* V, const float* keypad,
                                     void* P, void* O, float* S_scratch) {
  if (!c || !Q || !K || !V || !P || !O) return SPION_ERR_ARG;
  if (is_dense(c) || c->nnzb < 0) return SPION_ERR_STATE;
  DeviceGuard guard(c->device);
  if (use_tc(c)) return tc_engine_forward(c, Q, K, V, keypad, P, O, S_scratch);
  if (c->heads != 0) return SPION_ERR_UNSUPPORTED;
  const Pattern p = ctx_pattern(c);
  const long long nnz = (long long)c->nnzb * c->bs * c->bs;
  const ValueLayout vl{VAL_BLOCKTILE, c->L, nnz};
  const OperandLayout rm = row_major_operand(c->L, c->d);
  prof_mark(c, -1);
  if (use_simt_fused(c, VAL_BLOCKTILE)) {
    int rc = simt_fused_forward((const float*)Q, rm, (const float*)K, rm, (const float*)V, rm, keypad,
                                keypad ? 0.0f : -100.0f, (float*)P, vl, (float*)O, rm, p, c->BH, c->L, c->d, c->scale,
                                c->stream);
    if (!rc) prof_mark(c, SPION_STAGE_FUSED_FWD);
    c->launches += 1;
    return rc;
  }
  if (!S_scratch) return SPION_ERR_ARG;
  int rc = simt_sddmm(c->dtype, SPION_F32, Q, rm, K, rm, S_scratch, vl, p, c->nnzb, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SDDMM_S);
  if (rc) return rc;
  rc = softmax_fwd_rows(c->dtype, S_scratch, vl, P, vl, p, c->BH, c->L, c->scale, keypad, keypad ? 0.0f : -100.0f,
                        c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SOFTMAX_FWD);
  if (rc) return rc;
  rc = simt_spmm(c->dtype, c->dtype, false, P, vl, V, rm, O, rm, p, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SPMM_O);
  c->launches += 3;
  return rc;
}

extern "C" int spion_attn_backward_ex(spion_ctx* c, const void* Q, const void* K, const void* V, const void* P,
                                      const void* O, const void* dO, void* dS, float* dP_scratch, float* delta,
                                      void* dQ, void* dK, void* dV) {
  if (!c || !Q || !K || !V || !P || !dO || !dS || !dQ || !dK || !dV) return SPION_ERR_ARG;
  if (is_dense(c) || c->nnzb < 0) return SPION_ERR_STATE;
  DeviceGuard guard(c->device);
  if (use_tc(c)) {
    if (!O) return SPION_ERR_ARG;
    (void)delta;
    return tc_engine_backward(c, Q, K, V, P, O, dO, dS, dP_scratch, dQ, dK, dV);
  }
  if (c->heads != 0) return SPION_ERR_UNSUPPORTED;
  const Pattern p = ctx_pattern(c);
  const long long nnz = (long long)c->nnzb * c->bs * c->bs;
  const ValueLayout vl{VAL_BLOCKTILE, c->L, nnz};
  const OperandLayout rm = row_major_operand(c->L, c->d);
  prof_mark(c, -1);
  if (use_simt_fused(c, VAL_BLOCKTILE)) {
    c->launches += 2;
    return simt_fused_backward((const float*)Q, rm, (const float*)K, rm, (const float*)V, rm, (const float*)P, vl,
                               (const float*)O, rm, (const float*)dO, rm, (float*)dS, vl, (float*)dQ, rm, (float*)dK, rm, (float*)dV, rm, p,
                               c->BH, c->d, c->scale, c->stream, c);
  }
  if (!dP_scratch) return SPION_ERR_ARG;
  int rc = simt_sddmm(c->dtype, SPION_F32, dO, rm, V, rm, dP_scratch, vl, p, c->nnzb, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SDDMM_DP);
  if (rc) return rc;
  rc = softmax_bwd_rows(c->dtype, dP_scratch, vl, P, vl, dS, vl, p, c->BH, c->L, c->scale, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SOFTMAX_BWD);
  if (rc) return rc;
  rc = simt_spmm(c->dtype, c->dtype, false, dS, vl, K, rm, dQ, rm, p, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SPMM_DQ);
  if (rc) return rc;
  rc = simt_spmm(c->dtype, c->dtype, true, dS, vl, Q, rm, dK, rm, p, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SPMM_DK);
  if (rc) return rc;
  rc = simt_spmm(c->dtype, c->dtype, true, P, vl, dO, rm, dV, rm, p, c->BH, c->d, c->stream);
  if (!rc) prof_mark(c, SPION_STAGE_SPMM_DV);
  c->launches += 5;
  return rc;
}

extern "C" int spion_needs_scratch(const spion_ctx* c) {
  if (!c || is_dense(c)) return 0;
  return (use_tc(c) || use_simt_fused(c, VAL_BLOCKTILE)) ? 0 : 1;
}

extern "C" int spion_supports_fused(const spion_ctx* c) {
  return (c && !is_dense(c) && use_tc(c)) ? 1 : 0;
}

extern "C" int spion_attn_forward_fused(spion_ctx* c, const void* Q, const void* K, const void* V, const float* keypad,
                                        void* O, float* lse, void* P_optional) {
  if (!c || !Q || !K || !V || !O || !lse) return SPION_ERR_ARG;
  if (is_dense(c) || c->nnzb < 0) return SPION_ERR_STATE;
  if (!use_tc(c)) return SPION_ERR_UNSUPPORTED;
  DeviceGuard guard(c->device);
  return tc_engine_forward_fused(c, Q, K, V, keypad, O, lse, P_optional);
}

extern "C" int spion_attn_backward_fused(spion_ctx* c, const void* Q, const void* K, const void* V, const void* O,
                                         const void* dO, const float* lse, const float* keypad, void* dQ, void* dK,
                                         void* dV) {
  if (!c || !Q || !K || !V || !O || !dO || !lse || !dQ || !dK || !dV) return SPION_ERR_ARG;
  if (is_dense(c) || c->nnzb < 0) return SPION_ERR_STATE;
  if (!use_tc(c)) return SPION_ERR_UNSUPPORTED;
  DeviceGuard guard(c->device);
  return tc_engine_backward_fused(c, Q, K, V, O, dO, lse, keypad, dQ, dK, dV);
}

extern "C" int spion_block32_path_in_use(const spion_ctx* c) {
  if (!c) return SPION_ERR_ARG;
  return use_tc(c) ? tc_engine_block32_path(c) : 0;
}

extern "C" int spion_mean_map_recompute(spion_ctx* c, const void* Q, const void* K, const float* lse,
                                        const float* keypad, float* A) {
  if (!c || !Q || !K || !lse || !A) return SPION_ERR_ARG;
  if (is_dense(c) || c->nnzb < 0) return SPION_ERR_STATE;
  if (!use_tc(c)) return SPION_ERR_UNSUPPORTED;
  DeviceGuard guard(c->device);
  return tc_engine_mean_map(c, Q, K, lse, keypad, A);
}

extern "C" int spion_softmax_forward_ex(spion_ctx* c, const float* S, const float* keypad, void* P) {
  if (!c || !S || !P) return SPION_ERR_ARG;
  if (is_dense(c) || c->nnzb < 0) return SPION_ERR_STATE;
  DeviceGuard guard(c->device);
  const ValueLayout vl{VAL_BLOCKTILE, c->L, (long long)c->nnzb * c->bs * c->bs};
  c->launches += 1;
  return softmax_fwd_rows(c->dtype, S, vl, P, vl, ctx_pattern(c), c->BH, c->L, c->scale, keypad,
                          keypad ? 0.0f : -100.0f, c->stream);
}

extern "C" int spion_softmax_backward_ex(spion_ctx* c, const float* dP, const void* P, void* dS) {
  if (!c || !dP || !P || !dS) return SPION_ERR_ARG;
  if (is_dense(c) || c->nnzb < 0) return SPION_ERR_STATE;
  DeviceGuard guard(c->device);
  const ValueLayout vl{VAL_BLOCKTILE, c->L, (long long)c->nnzb * c->bs * c->bs};
  c->launches += 1;
  return softmax_bwd_rows(c->dtype, dP, vl, P, vl, dS, vl, ctx_pattern(c), c->BH, c->L, c->scale, c->stream);
}
