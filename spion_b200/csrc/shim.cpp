// Drop-in shims: four tiny shared objects that export exactly the symbols the reference's
// ctypes loaders bind (models/attention.py:141-191) -- init / attn_forward / attn_backward /
// destroy -- with the reference's argument order, and forward to libspion_b200.so.
//
//   SPION_SHIM_KIND 0  attn.so             models/attn.cu:265-280
//   SPION_SHIM_KIND 1  attn_mask.so        models/attn_mask.cu:280-298
//   SPION_SHIM_KIND 2  block_attn.so       models/block_attn.cu:547-568
//   SPION_SHIM_KIND 3  block_attn_mask.so  models/block_attn_mask.cu:655-674
//
// The reference's functions return void and swallow every error.  The shims return the int
// status instead (a caller bound to the void prototype simply ignores the register; ctypes'
// default restype is c_int) and print it to stderr when a call fails, so that a failure is loud.
#include <stdio.h>

#include "../../include/spion_b200.h"

#ifndef SPION_SHIM_KIND
#error "define SPION_SHIM_KIND"
#endif

static int report(const char* what, int rc) {
  if (rc != SPION_OK) fprintf(stderr, "spion_b200 shim: %s failed: %s (%d)\n", what, spion_status_string(rc), rc);
  return rc;
}

extern "C" {

#if SPION_SHIM_KIND == 0 || SPION_SHIM_KIND == 1
spion_ctx* init(int emb_dim, int seq_len, int num_batches) {
  return spion_create(SPION_SHIM_KIND == 0 ? SPION_KIND_DENSE : SPION_KIND_DENSE_KPM, emb_dim, seq_len, num_batches, 0,
                      SPION_F32, -1);
}
#if SPION_SHIM_KIND == 0
int attn_forward(spion_ctx* a, float* hQuery, float* hKey, float* hValue, float* hAttn, float* hOut) {
  return report("attn_forward", spion_dense_attn_forward(a, hQuery, hKey, hValue, nullptr, hAttn, hOut));
}
#else
int attn_forward(spion_ctx* a, float* hQuery, float* hKey, float* hValue, float* hMask, float* hAttn, float* hOut) {
  return report("attn_forward", spion_dense_attn_forward(a, hQuery, hKey, hValue, hMask, hAttn, hOut));
}
#endif
int attn_backward(spion_ctx* a, float* hQuery, float* hKey, float* hValue, float* hAttnScore, float* hGradOutput,
                   float* hGradAttnScore, float* hGradAttnScale, float* hGradAttn, float* hGradQuery, float* hGradKey,
                   float* hGradValue) {
  return report("attn_backward", spion_dense_attn_backward(a, hQuery, hKey, hValue, hAttnScore, hGradOutput, hGradAttnScore,
                                                    hGradAttnScale, hGradAttn, hGradQuery, hGradKey, hGradValue));
}
#else
spion_ctx* init(int emb_dim, int seq_len, int num_batches, int block_size) {
  return spion_create(SPION_SHIM_KIND == 2 ? SPION_KIND_BLOCK : SPION_KIND_BLOCK_KPM, emb_dim, seq_len, num_batches,
                      block_size, SPION_F32, -1);
}
#if SPION_SHIM_KIND == 2
int attn_forward(spion_ctx* a, float* hQuery, float* hKey, float* hValue, float* hAttn, float* hOut, int* hOffsets,
                  int* hColumns, int* hSum_mat, int nnz) {
  return report("attn_forward",
         spion_block_attn_forward(a, hQuery, hKey, hValue, nullptr, hAttn, hOut, hOffsets, hColumns, hSum_mat, nnz));
}
#else
int attn_forward(spion_ctx* a, float* hQuery, float* hKey, float* hValue, float* hMask, float* hAttn, float* hOut,
                  int* hOffsets, int* hColumns, int* hSum_mat, int nnz) {
  return report("attn_forward",
         spion_block_attn_forward(a, hQuery, hKey, hValue, hMask, hAttn, hOut, hOffsets, hColumns, hSum_mat, nnz));
}
#endif
int attn_backward(spion_ctx* a, float* hQuery, float* hKey, float* hValue, float* hAttnScore, float* hGradOutput,
                   float* hGradAttnScore, float* hGradAttn, float* hGradQuery, float* hGradKey, float* hGradValue,
                   int* hOffsets, int* hColumns, int* hSum_mat, int nnz) {
  return report("attn_backward",
         spion_block_attn_backward(a, hQuery, hKey, hValue, hAttnScore, hGradOutput, hGradAttnScore, hGradAttn,
                                   hGradQuery, hGradKey, hGradValue, hOffsets, hColumns, hSum_mat, nnz));
}
#endif

void destroy(spion_ctx* a) { spion_destroy(a); }

}  // extern "C"
