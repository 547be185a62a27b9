// Block CSR / CSC construction and the reference's element-level CSR expansion.
//
// Integer work, bit-exact against oracle/csr.py.  Replaces the torch op chain of
// models/attention_blockcuda.py:31-43 (sum / repeat / cumsum / Upsample / nonzero /
// repeat(BH)), which the reference re-runs on every forward call of every layer.
#include "common.cuh"

namespace {

// One CTA.  mat [nb*nb] uint8 -> CSR (row_ptr, col_idx, blk_row), CSC (col_ptr, row_idx,
// csc_pos) and the block count.  work [nb*nb] receives the CSR block id of every set cell.
__global__ void __launch_bounds__(1024) build_structure_kernel(
    const uint8_t* __restrict__ mat, int nb, int32_t* __restrict__ nnzb, int32_t* __restrict__ row_ptr,
    int32_t* __restrict__ col_idx, int32_t* __restrict__ blk_row, int32_t* __restrict__ col_ptr,
    int32_t* __restrict__ row_idx, int32_t* __restrict__ csc_pos, int32_t* __restrict__ work) {
  __shared__ int s_cnt[SPION_MAX_NB + 1];
  __shared__ int s_ptr[SPION_MAX_NB + 1];
  const int tid = threadIdx.x;
  // ---- rows
  for (int r = tid; r < nb; r += blockDim.x) {
    int n = 0;
    for (int c = 0; c < nb; ++c) n += mat[(size_t)r * nb + c] != 0;
    s_cnt[r] = n;
  }
  __syncthreads();
  if (tid == 0) {
    int acc = 0;
    for (int r = 0; r < nb; ++r) { s_ptr[r] = acc; acc += s_cnt[r]; }
    s_ptr[nb] = acc;
    *nnzb = acc;
  }
  __syncthreads();
  for (int r = tid; r <= nb; r += blockDim.x) row_ptr[r] = s_ptr[r];
  for (int r = tid; r < nb; r += blockDim.x) {
    int pos = s_ptr[r];
    for (int c = 0; c < nb; ++c) {
      if (mat[(size_t)r * nb + c]) {
        col_idx[pos] = c;
        blk_row[pos] = r;
        work[(size_t)r * nb + c] = pos;
        ++pos;
      }
    }
  }
  __syncthreads();
  // ---- columns
  for (int c = tid; c < nb; c += blockDim.x) {
    int n = 0;
    for (int r = 0; r < nb; ++r) n += mat[(size_t)r * nb + c] != 0;
    s_cnt[c] = n;
  }
  __syncthreads();
  if (tid == 0) {
    int acc = 0;
    for (int c = 0; c < nb; ++c) { s_ptr[c] = acc; acc += s_cnt[c]; }
    s_ptr[nb] = acc;
  }
  __syncthreads();
  for (int c = tid; c <= nb; c += blockDim.x) col_ptr[c] = s_ptr[c];
  for (int c = tid; c < nb; c += blockDim.x) {
    int pos = s_ptr[c];
    for (int r = 0; r < nb; ++r) {
      if (mat[(size_t)r * nb + c]) {
        row_idx[pos] = r;
        csc_pos[pos] = work[(size_t)r * nb + c];
        ++pos;
      }
    }
  }
}

// Recover the block mask from the reference's element-level CSR (one CTA per block row).
__global__ void mat_from_elemcsr_kernel(const int* __restrict__ offsets, const int* __restrict__ columns,
                                        const int* __restrict__ sum_mat, int nb, int bs, uint8_t* __restrict__ mat) {
  const int r = blockIdx.x;
  const int n = sum_mat[(size_t)r * bs];
  const int base = offsets[(size_t)r * bs];
  for (int k = threadIdx.x; k * bs < n; k += blockDim.x) {
    const int c = columns[(size_t)base + (size_t)k * bs] / bs;
    if (c >= 0 && c < nb) mat[(size_t)r * nb + c] = 1;
  }
}

__global__ void fill_u8_kernel(uint8_t* p, int n, int v) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) p[i] = (uint8_t)v;
}

// One CTA per element row (x) and per repeat (y).
__global__ void expand_csr_kernel(const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ col_idx, int nb,
                                  int bs, int nnzb, int32_t* __restrict__ sum_mat, int32_t* __restrict__ offsets,
                                  int32_t* __restrict__ columns) {
  const int i = blockIdx.x;
  const int L = nb * bs;
  const size_t nnz = (size_t)nnzb * bs * bs;
  if (i == L) {                                         // the closing offset
    if (blockIdx.y == 0 && threadIdx.x == 0) offsets[L] = (int32_t)nnz;
    return;
  }
  const int r = i / bs, ii = i % bs;
  const int rp = row_ptr[r];
  const int n_r = (row_ptr[r + 1] - rp) * bs;
  const size_t off = (size_t)rp * bs * bs + (size_t)ii * n_r;
  if (blockIdx.y == 0 && threadIdx.x == 0) {
    sum_mat[i] = n_r;
    offsets[i] = (int32_t)off;
  }
  int32_t* out = columns + (size_t)blockIdx.y * nnz + off;
  for (int t = threadIdx.x; t < n_r; t += blockDim.x) out[t] = col_idx[rp + t / bs] * bs + (t % bs);
}

}  // namespace

int spion_launch_build_structure(const uint8_t* mat, int nb, int32_t* nnzb, int32_t* row_ptr, int32_t* col_idx,
                                 int32_t* blk_row, int32_t* col_ptr, int32_t* row_idx, int32_t* csc_pos,
                                 int32_t* work, cudaStream_t st) {
  build_structure_kernel<<<1, 1024, 0, st>>>(mat, nb, nnzb, row_ptr, col_idx, blk_row, col_ptr, row_idx, csc_pos, work);
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}

int spion_launch_mat_from_elemcsr(const int* offsets, const int* columns, const int* sum_mat, int nb, int bs,
                                  uint8_t* mat, cudaStream_t st) {
  SPION_CUDA_TRY(cudaMemsetAsync(mat, 0, (size_t)nb * nb, st));
  mat_from_elemcsr_kernel<<<nb, 128, 0, st>>>(offsets, columns, sum_mat, nb, bs, mat);
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}

int spion_launch_fill_mat(uint8_t* mat, int n, int value, cudaStream_t st) {
  fill_u8_kernel<<<(n + 255) / 256 > 1024 ? 1024 : (n + 255) / 256, 256, 0, st>>>(mat, n, value);
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}

extern "C" int spion_build_structure(const uint8_t* mat, int nb, int32_t* nnzb, int32_t* row_ptr, int32_t* col_idx,
                                     int32_t* blk_row, int32_t* col_ptr, int32_t* row_idx, int32_t* csc_pos,
                                     int32_t* work, int32_t* host_nnzb, void* cuda_stream) {
  if (!mat || !nnzb || !row_ptr || !col_idx || !blk_row || !col_ptr || !row_idx || !csc_pos || !work) return SPION_ERR_ARG;
  if (nb < 1 || nb > SPION_MAX_NB) return SPION_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  int rc = spion_launch_build_structure(mat, nb, nnzb, row_ptr, col_idx, blk_row, col_ptr, row_idx, csc_pos, work, st);
  if (rc) return rc;
  if (host_nnzb) {
    SPION_CUDA_TRY(cudaMemcpyAsync(host_nnzb, nnzb, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    SPION_CUDA_TRY(cudaStreamSynchronize(st));
  }
  return SPION_OK;
}

extern "C" int spion_expand_csr(const int32_t* row_ptr, const int32_t* col_idx, int nb, int block_size, int nnzb,
                                int repeat, int32_t* sum_mat, int32_t* offsets, int32_t* columns, void* cuda_stream) {
  if (!row_ptr || !col_idx || !sum_mat || !offsets || !columns) return SPION_ERR_ARG;
  if (nb < 1 || nb > SPION_MAX_NB || block_size < 1 || repeat < 1 || nnzb < 0) return SPION_ERR_SHAPE;
  if ((size_t)nnzb * block_size * block_size > 0x7fffffffULL) return SPION_ERR_SHAPE;   // Offsets are int32
  dim3 grid(nb * block_size + 1, repeat);
  expand_csr_kernel<<<grid, 128, 0, (cudaStream_t)cuda_stream>>>(row_ptr, col_idx, nb, block_size, nnzb, sum_mat,
                                                                 offsets, columns);
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}
