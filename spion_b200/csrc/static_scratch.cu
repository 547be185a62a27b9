// Sparse attention forward for callers that cannot allocate device memory.
//
// Some hosts of this library are not allowed to call cudaMalloc at the point where they need
// attention: code running inside a memory pool it does not own, a plugin loaded into a serving
// process whose device memory is fully budgeted by the framework, or a real-time loop in which
// an allocation (which may synchronise the device) is forbidden.  The ordinary forward call needs
// one fp32 scratch value per selected score (the raw S = Q K^T tiles between the SDDMM kernel and
// the softmax kernel), which the caller normally allocates.  Here that scratch is a fixed
// array inside the library image instead, so the caller passes only inputs and outputs.
//
// Limits and rules:
//   * the array holds SPION_STATIC_SCRATCH_FLOATS values (64 MiB); every GPU that loads the
//     library carries it until the process exits;
//   * a call whose num_batches * nnzb * block^2 exceeds that is refused with SPION_ERR_SHAPE;
//   * all calls share the one array per device and it keeps the previous call's contents.  The
//     SDDMM kernel overwrites every value the softmax kernel later reads, so nothing has to be
//     cleared; but two calls that overlap on the GPU (different streams, or different host threads)
//     race on it -- serialise them;
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress);
//     make that first call outside any stream capture.  The address is remembered per device
//     ordinal for the life of the process (concurrent first calls from several host threads store
//     the same value); it does not survive a cudaDeviceReset of that device;
//   * nnzb must be the block count of the CSR that is passed (row_ptr[nb] == nnzb, nnzb <= nb^2): the
//     capacity check is made on nnzb, the kernels index the array by the block ids row_ptr yields.
// The entry point calls no cudaMalloc / cudaFree / allocating library routine.
#include "common.cuh"

#define SPION_STATIC_SCRATCH_FLOATS (16u * 1024u * 1024u)
#define SPION_MAX_DEVICES 64

static __device__ __align__(256) float g_static_scratch[SPION_STATIC_SCRATCH_FLOATS];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address:
// the address each device uses is asked for once, with that device current.
static float* g_scratch_addr[SPION_MAX_DEVICES] = {nullptr};

static int static_scratch_for_current_device(float** out) {
  int dev = -1;
  SPION_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= SPION_MAX_DEVICES) return SPION_ERR_UNSUPPORTED;
  if (!g_scratch_addr[dev]) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
    if (e != cudaSuccess || !p) {
      fprintf(stderr, "spion_b200: cudaGetSymbolAddress(static scratch) failed on device %d: %s\n", dev,
              cudaGetErrorString(e));
      return SPION_ERR_CUDA;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return SPION_OK;
}

extern "C" size_t spion_static_scratch_capacity(void) { return (size_t)SPION_STATIC_SCRATCH_FLOATS; }

extern "C" int spion_attn_forward_static(const void* Q, const void* K, const void* V, const float* keypad, void* P,
                                         void* O, const int32_t* row_ptr, const int32_t* col_idx,
                                         const int32_t* blk_row, int head_dim, int seq_len, int num_batches,
                                         int block_size, int nnzb, int dtype, void* cuda_stream) {
  if (!Q || !K || !V || !P || !O || !row_ptr || !col_idx || !blk_row) return SPION_ERR_ARG;
  if (dtype != SPION_F32 && dtype != SPION_BF16) return SPION_ERR_ARG;
  if (head_dim < 1 || seq_len < 1 || num_batches < 1 || block_size < 1 || nnzb < 0) return SPION_ERR_ARG;
  if (seq_len % block_size != 0 || seq_len / block_size > SPION_MAX_NB) return SPION_ERR_SHAPE;
  // The kernels walk the device row_ptr and index the scratch by block id, so the count the capacity
  // check uses must be the CSR's own: row_ptr[nb] == nnzb is the caller's contract, nnzb <= nb^2 is checked.
  if ((long long)nnzb > (long long)(seq_len / block_size) * (seq_len / block_size)) return SPION_ERR_SHAPE;
  const unsigned long long need = (unsigned long long)num_batches * (unsigned long long)nnzb * block_size * block_size;
  if (need > (unsigned long long)SPION_STATIC_SCRATCH_FLOATS) {
    fprintf(stderr,
            "spion_b200: spion_attn_forward_static needs %llu scratch values (num_batches*nnzb*block^2) but the "
            "built-in array holds %u; use spion_attn_forward_ex with caller-allocated scratch\n",
            need, SPION_STATIC_SCRATCH_FLOATS);
    return SPION_ERR_SHAPE;
  }
  float* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  const int nb = seq_len / block_size;
  // forward only walks rows: the column-major arrays are not needed
  const Pattern p{row_ptr, col_idx, blk_row, nullptr, nullptr, nullptr, nb, block_size};
  const long long nnz = (long long)nnzb * block_size * block_size;
  const ValueLayout vl{VAL_BLOCKTILE, seq_len, nnz};
  const OperandLayout rm = row_major_operand(seq_len, head_dim);
  const float scale = 1.0f / sqrtf((float)head_dim);
  rc = simt_sddmm(dtype, SPION_F32, Q, rm, K, rm, scratch, vl, p, nnzb, num_batches, head_dim, st);
  if (rc) return rc;
  rc = softmax_fwd_rows(dtype, scratch, vl, P, vl, p, num_batches, seq_len, scale, keypad, keypad ? 0.0f : -100.0f, st);
  if (rc) return rc;
  return simt_spmm(dtype, dtype, false, P, vl, V, rm, O, rm, p, num_batches, head_dim, st);
}
