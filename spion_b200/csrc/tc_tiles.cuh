// Tile and descriptor helpers shared by the tensor-core kernels (tc_engine.cu, tc_fused.cu).
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace tc {

constexpr int BS = 64;                  // block size of the engine
constexpr int VT_BYTES = BS * BS * 2;   // one bf16 value tile (P or dS)
constexpr float LOG2E = 1.4426950408889634f;

enum : int { ERR_LOAD_WAIT = 1, ERR_MMA_WAIT = 2, ERR_MMA2_WAIT = 4 };

__device__ __forceinline__ void report(int* status, int code) { atomicOr(status, code); }

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Packed bf16 arithmetic (two values per register, one rounding per operation).
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// A descriptor's start-address field counts 16-byte units in its low 14 bits: stepping an operand by
// `bytes` inside one tile is an add on the low word (the tiles are 1024-byte aligned and at most 8 KB, so
// the field never carries).
__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) { return desc + (uint64_t)(bytes >> 4); }

template <int D> struct OpTile {
  static constexpr int ROW_BYTES = D * 2;                        // 128 (D=64) or 64 (D=32)
  static constexpr int BYTES = BS * ROW_BYTES;
  static constexpr uint32_t LAYOUT = (D == 64) ? LAYOUT_SW128 : LAYOUT_SW64;
  static constexpr uint32_t SBO = 8 * ROW_BYTES;                 // 8-row swizzle atom
  // K-major use (contraction over the head dimension): 16 elements = 32 bytes per K step
  __device__ static uint64_t kmajor(uint32_t saddr, int kk) { return make_smem_desc(saddr + kk * 32, 16, SBO, LAYOUT); }
  // MN-major use (contraction over the 64 rows of the tile): 16 rows per K step
  __device__ static uint64_t mnmajor(uint32_t saddr, int kk) {
    return make_smem_desc(saddr + kk * 16 * ROW_BYTES, BYTES, SBO, LAYOUT);
  }
  static constexpr uint32_t K_STEP = 32, MN_STEP = 16 * ROW_BYTES;   // bytes per K step of the two uses
};
// bf16 value tile [64 x 64], 128-byte rows, SWIZZLE_128B
struct ValTile {
  __device__ static uint64_t kmajor(uint32_t saddr, int kk) { return make_smem_desc(saddr + kk * 32, 16, 1024, LAYOUT_SW128); }
  __device__ static uint64_t mnmajor(uint32_t saddr, int kk) {
    return make_smem_desc(saddr + kk * 2048, VT_BYTES, 1024, LAYOUT_SW128);
  }
  static constexpr uint32_t K_STEP = 32, MN_STEP = 2048;
};


#ifdef SPION_TRACE
// Developer build only: nanosecond stamps (%globaltimer) of thread 0 at phase boundaries, 16 per unit,
// for the first units of every CTA.
static __device__ unsigned long long* g_spion_trace;     // one copy per translation unit (no relocatable device code)
static __device__ int g_spion_trace_units;
#define SPION_TRACE_SETTER(name)                                                              \
  extern "C" int name(void* device_buffer, int units_per_cta) {                               \
    SPION_CUDA_TRY(cudaMemcpyToSymbol(g_spion_trace, &device_buffer, sizeof(void*)));         \
    SPION_CUDA_TRY(cudaMemcpyToSymbol(g_spion_trace_units, &units_per_cta, sizeof(int)));     \
    return SPION_OK;                                                                          \
  }
__device__ __forceinline__ void trace_stamp(int unit_ordinal, int k) {
  if (threadIdx.x == 0 && g_spion_trace && unit_ordinal < g_spion_trace_units) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");
    g_spion_trace[((size_t)blockIdx.x * g_spion_trace_units + unit_ordinal) * 16 + k] = t;
  }
}
__device__ __forceinline__ void trace_stamp_t(int thread, int unit_ordinal, int k) {
  if ((int)threadIdx.x == thread && g_spion_trace && unit_ordinal < g_spion_trace_units) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");
    g_spion_trace[((size_t)blockIdx.x * g_spion_trace_units + unit_ordinal) * 16 + k] = t;
  }
}
#define SPION_STAMP(u, k) trace_stamp(u, k)
#define SPION_STAMP_T(t, u, k) trace_stamp_t(t, u, k)
#else
#define SPION_STAMP(u, k)
#define SPION_STAMP_T(t, u, k)
#endif

// Where the [L x D] operand matrix of (b,h) pair `bh` starts inside the 2-D tensor the maps describe.
//   heads == 0: operands are [BH, L, D]      -> rows bh*L ..,      columns 0 .. D,        row pitch D
//   heads == H: operands are [B, L, H, D]    -> rows (bh/H)*L ..,  columns (bh%H)*D ..,   row pitch H*D
// (the second form is what a linear projection writes before any head split; models/attention.py:131-139)
struct OpPos { int row0, x0, ld; };
__device__ __forceinline__ OpPos op_pos(int bh, int L, int heads, int D) {
  if (heads == 0) return OpPos{bh * L, 0, D};
  const int b = bh / heads;
  return OpPos{b * L, (bh - b * heads) * D, heads * D};
}

constexpr int ROW_NCH = 4;              // tiles of a block row that the row kernels handle as one chunk

// One record of the sorted row list: {row_ptr, blocks | row << 16, col0 | col1 << 16, col2 | col3 << 16}.
struct RowRec {
  int rp, nblk, r, c01, c23;
  __device__ RowRec() : rp(0), nblk(0), r(0), c01(0), c23(0) {}
  __device__ explicit RowRec(int4 ri) : rp(ri.x), nblk(ri.y & 0xffff), r(ri.y >> 16), c01(ri.z), c23(ri.w) {}
  __device__ int col(int t, const int* __restrict__ col_idx) const {          // block column of the row's t-th block
    return t < 4 ? (((t & 2) ? c23 : c01) >> ((t & 1) * 16)) & 0xffff : col_idx[rp + t];
  }
  __device__ bool single() const { return nblk <= ROW_NCH; }
  __device__ int chunk() const { return single() ? ROW_NCH : 2; }             // tiles per chunk
  __device__ int nchunks() const { return (nblk + chunk() - 1) / chunk(); }
  // Load jobs.  A short row has one (Q, K and V tiles of the row).  A long row has 2*nchunks: the K pairs of
  // pass A, then the K and V pairs of pass B; job g uses buffers [2*(g&1), 2*(g&1)+1] and the barriers of
  // that half, so job g+2 is requested as soon as job g has released its half and two jobs are in flight.
  __device__ int njobs() const { return nblk == 0 ? 0 : (single() ? 1 : 2 * nchunks()); }
};

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct TcState {
  EncodeTiledFn encode = nullptr;
  int sms = 0;                  // multiprocessors of the context's device
  int fwd_ctas = 0, row_ctas = 0, col_ctas = 0;   // resident CTAs per SM of the persistent kernels
  int rc_row_ctas = 0;                            // ... of the recompute row kernel (the column kernel: one per SM)
  int pipe_ctas = 0;                              // ... of the pipelined forward for short rows
  int n_long = 0;               // block rows with more than ROW_NCH blocks: the first n_long records of row_info
  int* n_long_dev = nullptr;
  float* delta_ws = nullptr;    // [BH*L] delta_i = sum_n dO_in O_in, written by the row kernel, read by the column kernel
  float* lse_ws = nullptr;      // [BH*L] log-sum-exp workspace for the calls that do not expose it
  int* col_order = nullptr;     // block columns from the longest to the shortest
  // the same columns as records for the streaming column kernel: one load per column / per pair of entries
  int4* col_rec = nullptr;      // [nb] in col_order: {block column, first pair, pairs, entries}
  int4* col_pair = nullptr;     // [sum of pairs] {block row of entry 0, of entry 1 (-1: none), CSR block id 0, 1}
  size_t col_pair_cap = 0;
  int4* row_info = nullptr;     // per block row: {row_ptr, blocks, col0 | col1 << 16, col2 | col3 << 16}: one load instead of two dependent ones
  // 32-wide masks run on 64-wide super-blocks: derived structure + which 32x32 quarters are selected
  bool super = false;
  int nb64 = 0, nnzb64 = 0;
  uint8_t* mat64 = nullptr; uint8_t* submask = nullptr;
  int32_t *row_ptr64 = nullptr, *col_idx64 = nullptr, *blk_row64 = nullptr, *col_ptr64 = nullptr, *row_idx64 = nullptr,
          *csc_pos64 = nullptr, *work64 = nullptr, *nnzb64_dev = nullptr;
  void* p64_ws = nullptr; void* ds64_ws = nullptr;     // [BH, nnzb64, 64, 64] bf16 each
  size_t ws_elems = 0;
  // 32-wide masks with head_dim 64: kernels on the mask's own blocks (tc_b32.cu) for the calls without stored P
  bool b32 = false;             // the context's shape has these kernels
  bool b32_use = false;         // ... and the current mask runs on them (spion_set_block32_path, else chosen per mask)
  float b32_fill = 0.f;         // selected blocks per gathered job of the current mask (at most 4)
  int* b32_jobs_dev = nullptr;
  int b32_ctas[3] = {0, 0, 0};  // resident CTAs per SM of the forward / row / column kernel
  int4* b32_row_rec = nullptr;  // [nb] block rows, longest first: {row_ptr, blocks, block row, 0}
  int4* b32_col_rec = nullptr;  // [nb] block columns likewise: {col_ptr, entries, block column, 0}
};

// What the kernels see: the 64-block structure (the mask's own, or the derived super-block one).
struct TcView {
  const int32_t *row_ptr, *col_idx, *col_ptr, *row_idx, *csc_pos;
  const uint8_t* submask;       // nullptr: every block is fully selected
  const int4* row_info;
  int nb, nnzb;
};
inline TcView tc_view(const spion_ctx* c, const TcState* s) {
  if (s->super)
    return TcView{s->row_ptr64, s->col_idx64, s->col_ptr64, s->row_idx64, s->csc_pos64, s->submask, s->row_info, s->nb64, s->nnzb64};
  return TcView{c->row_ptr, c->col_idx, c->col_ptr, c->row_idx, c->csc_pos, nullptr, s->row_info, c->nb, c->nnzb};
}

// 2-D bf16 tensor of `rows` x `cols` (row-major, contiguous rows) read or written in boxes of
// box_rows x box_cols; box_cols * 2 bytes is 128 (SWIZZLE_128B) or 64 (SWIZZLE_64B).
inline int make_map(TcState* s, CUtensorMap* m, const void* base, uint64_t rows, uint32_t cols, uint32_t box_cols,
                    uint32_t box_rows) {
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = (box_cols * 2 == 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  CUresult r = s->encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "spion_b200: cuTensorMapEncodeTiled failed (%d) rows=%llu cols=%u\n", (int)r,
            (unsigned long long)rows, cols);
    return SPION_ERR_CUDA;
  }
  return SPION_OK;
}


// How many CTAs of a persistent kernel one SM holds at once: the limits are shared memory (dynamic +
// static + the per-CTA reservation), registers (allocated per warp in units of 256) and tensor memory
// (512 columns).  Computed from the device's limits and the kernel's own attributes.
template <typename K>
inline int resident_ctas(K kernel, int device, int threads, size_t dyn_smem, int tmem_cols, int* out) {
  cudaFuncAttributes fa;
  if (cudaFuncGetAttributes(&fa, kernel) != cudaSuccess) return SPION_ERR_CUDA;
  int smem_sm = 0, smem_resv = 0, regs_sm = 0;
  if (cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, device) != cudaSuccess ||
      cudaDeviceGetAttribute(&smem_resv, cudaDevAttrReservedSharedMemoryPerBlock, device) != cudaSuccess ||
      cudaDeviceGetAttribute(&regs_sm, cudaDevAttrMaxRegistersPerMultiprocessor, device) != cudaSuccess)
    return SPION_ERR_CUDA;
  const size_t per_cta = dyn_smem + fa.sharedSizeBytes + (size_t)smem_resv;
  const int warps = (threads + 31) / 32;
  const int regs_warp = ((fa.numRegs * 32 + 255) / 256) * 256;
  int n = (int)((size_t)smem_sm / per_cta);
  if (regs_warp > 0 && regs_sm / (regs_warp * warps) < n) n = regs_sm / (regs_warp * warps);
  if (tmem_cols > 0 && 512 / tmem_cols < n) n = 512 / tmem_cols;
  if (n < 1) return SPION_ERR_CUDA;
  *out = n;
  return SPION_OK;
}

// Map over one dense operand (Q, K, V, dO): [BH*L, D] rows, or [B*L, H*D] rows with a [64 x D] box at
// column h*D when the context's operands are in the merged-head form.
inline int make_operand_map(const spion_ctx* c, TcState* s, CUtensorMap* m, const void* base, int D) {
  if (c->heads == 0) return make_map(s, m, base, (uint64_t)c->BH * c->L, (uint32_t)D, (uint32_t)D, BS);
  return make_map(s, m, base, (uint64_t)(c->BH / c->heads) * c->L, (uint32_t)(c->heads * D), (uint32_t)D, BS);
}

// tc_recompute_col.cu: streaming column kernel of the recompute backward (reads the context's delta array)
int col_stream_set_attrs(int d);
int col_stream_backward(spion_ctx* c, TcState* s, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                        const CUtensorMap& mdo, const float* lse, const float* keypad, void* dK, void* dV);

// tc_recompute.cu
int recompute_set_attrs(TcState* s, int d, int device);
int recompute_backward(spion_ctx* c, TcState* s, const void* Q, const void* K, const void* V, const void* O,
                       const void* dO, const float* lse, const float* keypad, void* dQ, void* dK, void* dV);
int recompute_mean_map(spion_ctx* c, TcState* s, const void* Q, const void* K, const float* lse, const float* keypad,
                       float* A);

// tc_fwd_pipe.cu: forward of the records [rank0, nb) of row_info (rows of at most ROW_NCH blocks)
int pipe_set_attrs(TcState* s, int d, int device);
int pipe_forward(spion_ctx* c, TcState* s, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                 const CUtensorMap& mp, bool store_p, const float* keypad, void* O, float* lse, int rank0);

// tc_b32.cu: masks of 32-wide blocks on the blocks themselves (bf16, head_dim 64; no stored P)
bool b32_applies(const spion_ctx* c);
int b32_set_attrs(TcState* s, int device);
int b32_prepare(spion_ctx* c, TcState* s);
void b32_release(TcState* s);
int b32_forward(spion_ctx* c, TcState* s, const void* Q, const void* K, const void* V, const float* keypad, void* O,
                float* lse);
int b32_backward(spion_ctx* c, TcState* s, const void* Q, const void* K, const void* V, const void* O, const void* dO,
                 const float* lse, const float* keypad, void* dQ, void* dK, void* dV);

// tc_fused.cu
int fused_set_attrs(TcState* s, int d, int device);
int fused_forward(spion_ctx* c, TcState* s, const void* Q, const void* K, const void* V, const float* keypad, void* O,
                  float* lse, void* P64_optional);

}  // namespace tc
