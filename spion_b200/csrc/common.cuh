// Shared declarations of the spion_b200 library (host + device).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/spion_b200.h"

#define SPION_MAX_NB 512            // largest number of blocks per side (L=16384, block 32)
#define SPION_PROF_MAX_MARKS 64

// -------------------------------------------------------------------------------------
// Block-sparse structure of one layer's mask, all device pointers.
struct Pattern {
  const int32_t* row_ptr;   // [nb+1]
  const int32_t* col_idx;   // [nnzb]  block column of CSR block id
  const int32_t* blk_row;   // [nnzb]  block row of CSR block id
  const int32_t* col_ptr;   // [nb+1]
  const int32_t* row_idx;   // [nnzb]  block row of CSC entry
  const int32_t* csc_pos;   // [nnzb]  CSR block id of CSC entry
  int nb;
  int bs;
};

// Where the values of the sparse matrices (S, P, dP, dS) live.
enum ValueMode {
  VAL_ELEMCSR = 0,    // reference layout: element rows, selected columns ascending  [BH][nnz]
  VAL_BLOCKTILE = 1,  // native layout: [BH][nnzb][bs][bs], CSR block order
  VAL_DENSE_T = 2     // reference dense layout: [BH][L(j)][L(i)]  (value(i,j) at j*L + i)
};

struct ValueLayout {
  int mode;
  int L;
  long long bh_stride;   // elements between consecutive (b,h) matrices
};

// Dense operand (Q, K, V, dO, O, dQ, dK, dV): element (bh, l, n) at bh*bh_stride + l*sl + n*sd.
struct OperandLayout {
  long long bh_stride;
  long long sl;
  long long sd;
};

static inline OperandLayout row_major_operand(int L, int d) { return OperandLayout{(long long)L * d, d, 1}; }
static inline OperandLayout transposed_operand(int L, int d) { return OperandLayout{(long long)L * d, 1, L}; }

// Address of value tile (block row r, block column c, CSR block id blk):
// element (i, j) of the tile sits at base + i*si + j*sj (in elements, inside one (b,h) matrix).
__device__ __forceinline__ void tile_address(const ValueLayout& vl, const Pattern& p, int r, int c, int blk,
                                             long long& base, long long& si, long long& sj) {
  const int bs = p.bs;
  if (vl.mode == VAL_ELEMCSR) {
    const int rp = p.row_ptr[r];
    const int nblk = p.row_ptr[r + 1] - rp;
    base = (long long)rp * bs * bs + (long long)(blk - rp) * bs;
    si = (long long)nblk * bs;
    sj = 1;
  } else if (vl.mode == VAL_BLOCKTILE) {
    base = (long long)blk * bs * bs;
    si = bs;
    sj = 1;
  } else {
    base = (long long)c * bs * vl.L + (long long)r * bs;
    si = 1;
    sj = vl.L;
  }
}

// -------------------------------------------------------------------------------------
// Context (host side).
struct spion_ctx {
  int kind, d, L, BH, bs, nb, dtype, device, engine;
  int heads;                // 0: operands [BH, L, d]; H > 0: operands [B, L, H, d] (tensor-core engine only)
  int block32_path;         // 32-wide masks on the tensor-core engine: 0 chosen per mask, 1 the mask's own blocks, 2 super-blocks
  float scale;
  cudaStream_t stream;
  // structure workspace (device), capacity nb*nb blocks
  uint8_t* mat;
  int32_t *row_ptr, *col_idx, *blk_row, *col_ptr, *row_idx, *csc_pos, *work, *nnzb_dev;
  int nnzb;                 // block count of the current pattern (host copy), -1 if none
  int csr_stable;           // reference-layout calls: the caller keeps its element-CSR arrays alive and unchanged
  const void* csr_key[3];   // ... and these are the arrays the current structure was built from
  int csr_nnz;
  int* status_dev;          // device status word written by bounded waits
  long long launches;
  void* tc;                 // tensor-core engine state (tensor maps, ...), owned by tc_engine.cu
  // per-stage timing (off by default): events recorded between the kernels of a pipeline
  int prof_on;
  int prof_n;                               // marks recorded since the last drain
  cudaEvent_t prof_ev[SPION_PROF_MAX_MARKS];
  int prof_stage[SPION_PROF_MAX_MARKS];     // stage that ENDS at this mark (-1: start of a pipeline)
  double prof_ms[SPION_STAGE_COUNT];
  long long prof_cnt[SPION_STAGE_COUNT];
};

// record "stage finished" on the context's stream; stage = -1 opens a pipeline
int prof_mark(spion_ctx* c, int stage);
int prof_drain(spion_ctx* c);

static inline Pattern ctx_pattern(const spion_ctx* c) {
  return Pattern{c->row_ptr, c->col_idx, c->blk_row, c->col_ptr, c->row_idx, c->csc_pos, c->nb, c->bs};
}

#define SPION_CUDA_TRY(expr)                                                          \
  do {                                                                                \
    cudaError_t _e = (expr);                                                          \
    if (_e != cudaSuccess) {                                                          \
      fprintf(stderr, "spion_b200: %s failed: %s (%s:%d)\n", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return SPION_ERR_CUDA;                                                          \
    }                                                                                 \
  } while (0)

#define SPION_LAUNCH_CHECK()                                                          \
  do {                                                                                \
    cudaError_t _e = cudaGetLastError();                                              \
    if (_e != cudaSuccess) {                                                          \
      fprintf(stderr, "spion_b200: kernel launch failed: %s (%s:%d)\n", cudaGetErrorString(_e), __FILE__, __LINE__); \
      return SPION_ERR_CUDA;                                                          \
    }                                                                                 \
  } while (0)

// ------------------------------------------------------------------ element conversions
__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// ------------------------------------------------------------------ launchers across files
// structure.cu
int spion_launch_build_structure(const uint8_t* mat, int nb, int32_t* nnzb, int32_t* row_ptr, int32_t* col_idx,
                                 int32_t* blk_row, int32_t* col_ptr, int32_t* row_idx, int32_t* csc_pos,
                                 int32_t* work, cudaStream_t st);
int spion_launch_mat_from_elemcsr(const int* offsets, const int* columns, const int* sum_mat, int nb, int bs,
                                  uint8_t* mat, cudaStream_t st);
int spion_launch_fill_mat(uint8_t* mat, int n, int value, cudaStream_t st);

// simt_attn.cu
int simt_sddmm(int dtype_in, int dtype_val, const void* A, OperandLayout la, const void* B, OperandLayout lb,
               void* vals, ValueLayout vl, Pattern p, int nnzb, int BH, int d, cudaStream_t st);
int simt_spmm(int dtype_val, int dtype_op, bool trans, const void* vals, ValueLayout vl, const void* Bop,
              OperandLayout lb, void* out, OperandLayout lo, Pattern p, int BH, int d, cudaStream_t st);
int softmax_fwd_rows(int dtype_out, const float* S, ValueLayout vin, void* P, ValueLayout vout, Pattern p, int BH,
                     int L, float scale, const float* keypad, float floor, cudaStream_t st);
int softmax_bwd_rows(int dtype_p, const float* dP, ValueLayout vdp, const void* P, ValueLayout vp, void* dS,
                     ValueLayout vds, Pattern p, int BH, int L, float scale, cudaStream_t st);
int softmax_fwd_dense_t(float* S, int BH, int L, float scale, const float* keypad, float floor, cudaStream_t st);
int softmax_bwd_dense_t(const float* dP, const float* P, float* dS, int BH, int L, float scale, cudaStream_t st);

// simt_fused.cu: fused fp32 kernels (value layouts with contiguous tile rows)
bool simt_fused_supports(int bs, int d, int BH, int value_mode);
int simt_fused_forward(const float* Q, OperandLayout lq, const float* K, OperandLayout lk, const float* V,
                       OperandLayout lv, const float* keypad, float floor_v, float* P, ValueLayout vl, float* O,
                       OperandLayout lo, Pattern p, int BH, int L, int d, float scale, cudaStream_t st);
int simt_fused_backward(const float* Q, OperandLayout lq, const float* K, OperandLayout lk, const float* V,
                        OperandLayout lv, const float* P, ValueLayout vp, const float* O_or_null, OperandLayout lo,
                        const float* dO, OperandLayout ldo, float* dS, ValueLayout vds, float* dQ, OperandLayout ldq,
                        float* dK, OperandLayout ldk, float* dV, OperandLayout ldv, Pattern p, int BH, int d,
                        float scale, cudaStream_t st, struct spion_ctx* prof);

// tc_engine.cu: tcgen05 / TMA engine (bf16, block-tile layout)
bool tc_engine_supports(const spion_ctx* c);
int tc_engine_prepare(spion_ctx* c);       // after the pattern is set
void tc_engine_release(spion_ctx* c);
int tc_engine_forward(spion_ctx* c, const void* Q, const void* K, const void* V, const float* keypad, void* P, void* O,
                      float* S_scratch);
int tc_engine_backward(spion_ctx* c, const void* Q, const void* K, const void* V, const void* P, const void* O,
                       const void* dO, void* dS, float* dP_scratch, void* dQ, void* dK, void* dV);
int tc_engine_forward_fused(spion_ctx* c, const void* Q, const void* K, const void* V, const float* keypad, void* O,
                            float* lse, void* P_optional);
int tc_engine_backward_fused(spion_ctx* c, const void* Q, const void* K, const void* V, const void* O, const void* dO,
                             const float* lse, const float* keypad, void* dQ, void* dK, void* dV);
int tc_engine_mean_map(spion_ctx* c, const void* Q, const void* K, const float* lse, const float* keypad, float* A);
int tc_engine_wait_selftest(spion_ctx* c, long long limit_cycles);
int tc_engine_block32_path(const spion_ctx* c);   // 1 own blocks, 2 super-blocks, 0: not a 32-wide mask on this engine
