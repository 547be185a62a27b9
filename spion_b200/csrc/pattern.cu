// Pattern discovery on the GPU: convolution + block average pooling of the mean attention
// map, quantile threshold, the reference's greedy walkers, forced diagonal, block CSR/CSC.
//
// Replaces the CPU/Python block of the reference driver, main_conv_ff.py:255-279, and its
// recursive flood_fill (main_conv_ff.py:35-62); the top-k selection of main_conv.py:246-251;
// F == 1 gives main_ff.py:255 (no convolution).
//
// Integer outputs are bit-exact against oracle/pattern.py because the float stages use the
// same fixed order of fp64 additions (documented at each loop) and the same fused lerp.
#include "common.cuh"

namespace {

// ---------------------------------------------------------------- conv + pool (one CTA per cell)
// smem: tile[(bs+F-1)^2] fp32 (zero padded halo) | c[bs*bs] fp64 | rsum[bs] fp64
__global__ void __launch_bounds__(256) conv_pool_kernel(const float* __restrict__ A, int L, int bs, int kind, int F,
                                                        float* __restrict__ pooled) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int h = F / 2;
  const int T = bs + 2 * h;
  float* tile = reinterpret_cast<float*>(smem_raw);
  size_t off = ((size_t)T * T * sizeof(float) + 15) & ~(size_t)15;
  double* cval = reinterpret_cast<double*>(smem_raw + off);
  double* rsum = cval + (size_t)bs * bs;
  const int bi = blockIdx.y, bj = blockIdx.x, nb = gridDim.x;
  const int i0 = bi * bs - h, j0 = bj * bs - h;
  for (int t = threadIdx.x; t < T * T; t += blockDim.x) {
    const int ti = t / T, tj = t % T;
    const int gi = i0 + ti, gj = j0 + tj;
    tile[t] = (gi >= 0 && gi < L && gj >= 0 && gj < L) ? A[(size_t)gi * L + gj] : 0.0f;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < bs * bs; e += blockDim.x) {
    const int i = e / bs, j = e % bs;
    double c = 0.0;
    if (kind == SPION_CONV_DIAG) {
      // c = sum_{t=-h..h} A[i+t, j+t], added for t ascending (oracle: conv_fixed_order)
      for (int t = 0; t < F; ++t) c = c + (double)tile[(i + t) * T + (j + t)];
    } else {
      // box mean: u outer, v inner, ascending; one fp64 division
      for (int u = 0; u < F; ++u)
        for (int v = 0; v < F; ++v) c = c + (double)tile[(i + u) * T + (j + v)];
      c = c / (double)(F * F);
    }
    cval[e] = c;
  }
  __syncthreads();
  // r[i] = sum_jj c[i, jj]  (jj ascending), then p = sum_ii r[ii] (ii ascending): pool_fixed_order
  for (int i = threadIdx.x; i < bs; i += blockDim.x) {
    double r = 0.0;
    for (int jj = 0; jj < bs; ++jj) r = r + cval[i * bs + jj];
    rsum[i] = r;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double p = 0.0;
    for (int ii = 0; ii < bs; ++ii) p = p + rsum[ii];
    pooled[(size_t)bi * nb + bj] = (float)(p / (double)(bs * bs));
  }
}

// Diagonal filter, block 32 or 64 (the reference's settings: F = 31, main_conv_ff.py:258): the same sums in the
// same order as conv_pool_kernel, organised so that the filter taps are read once per eight outputs instead of
// once per output.  A thread computes a run of eight outputs (i0 + k, j0 + k), k = 0..7, along a diagonal of the
// block: they need the tile diagonal d_m = tile[i0 + m][j0 + m], m = 0 .. F + 6, and output k is
// ((d_k + d_k+1) + d_k+2) + ... in ascending order -- eight independent fp64 chains.  Runs start at
// i0 = 0, 8, .., j0 = -7 .. BS - 1 (outputs left of the block are skipped).  The pooled rows are padded by one
// double so that the row sums (one thread per row) do not collide in shared memory.
template <int BS, int F>
__global__ void __launch_bounds__(256) conv_pool_diag_kernel(const float* __restrict__ A, int L, float* __restrict__ pooled) {
  constexpr int H = F / 2, T = BS + 2 * H, RUN = 8, CS = BS + 1;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* tile = reinterpret_cast<float*>(smem_raw);
  double* cval = reinterpret_cast<double*>(smem_raw + (((size_t)T * T * sizeof(float) + 15) & ~(size_t)15));
  double* rsum = cval + (size_t)BS * CS;
  const int bi = blockIdx.y, bj = blockIdx.x, nb = gridDim.x;
  const int i0g = bi * BS - H, j0g = bj * BS - H;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // all of a thread's loads are issued before the first store (the tile is read with the latency of one load,
  // not of one load per row)
  constexpr int NR = (T + 7) / 8, NCOL = (T + 31) / 32;
  float v[NR][NCOL];
#pragma unroll
  for (int a = 0; a < NR; ++a) {
    const int ti = warp + 8 * a, gi = i0g + ti;
#pragma unroll
    for (int b = 0; b < NCOL; ++b) {
      const int tj = lane + 32 * b, gj = j0g + tj;
      v[a][b] = (ti < T && tj < T && gi >= 0 && gi < L && gj >= 0 && gj < L) ? A[(size_t)gi * L + gj] : 0.0f;
    }
  }
#pragma unroll
  for (int a = 0; a < NR; ++a) {
    const int ti = warp + 8 * a;
#pragma unroll
    for (int b = 0; b < NCOL; ++b) {
      const int tj = lane + 32 * b;
      if (ti < T && tj < T) tile[ti * T + tj] = v[a][b];
    }
  }
  __syncthreads();
  constexpr int RUNS = (BS / RUN) * (BS + RUN - 1);
  for (int r = threadIdx.x; r < RUNS; r += blockDim.x) {
    const int i0 = (r / (BS + RUN - 1)) * RUN, j0 = r % (BS + RUN - 1) - (RUN - 1);
    float d[F + RUN - 1];
#pragma unroll
    for (int m = 0; m < F + RUN - 1; ++m)          // taps left or right of the tile belong to skipped outputs only
      d[m] = (j0 + m >= 0 && j0 + m < T) ? tile[(i0 + m) * T + (j0 + m)] : 0.0f;
    double c[RUN];
#pragma unroll
    for (int k = 0; k < RUN; ++k) c[k] = 0.0;
    // c[k] = sum_{t = 0 .. F-1} d[k + t], t ascending (oracle: conv_fixed_order); the eight chains interleave
#pragma unroll
    for (int t = 0; t < F; ++t) {
#pragma unroll
      for (int k = 0; k < RUN; ++k) c[k] = c[k] + (double)d[k + t];
    }
#pragma unroll
    for (int k = 0; k < RUN; ++k) {
      const int j = j0 + k;
      if (j >= 0 && j < BS) cval[(i0 + k) * CS + j] = c[k];
    }
  }
  __syncthreads();
  // r[i] = sum_jj c[i, jj]  (jj ascending), then p = sum_ii r[ii] (ii ascending): pool_fixed_order
  for (int i = threadIdx.x; i < BS; i += blockDim.x) {
    double rr = 0.0;
#pragma unroll 8
    for (int jj = 0; jj < BS; ++jj) rr = rr + cval[i * CS + jj];
    rsum[i] = rr;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double p = 0.0;
#pragma unroll 8
    for (int ii = 0; ii < BS; ++ii) p = p + rsum[ii];
    pooled[(size_t)bi * nb + bj] = (float)(p / (double)(BS * BS));
  }
}

template <int BS, int F>
int launch_conv_pool_diag(const float* A, int L, int nb, float* pooled, cudaStream_t st) {
  constexpr int T = BS + F - 1;
  const size_t smem = (((size_t)T * T * sizeof(float) + 15) & ~(size_t)15) + ((size_t)BS * (BS + 1) + BS) * sizeof(double);
  if (smem > 48 * 1024)
    SPION_CUDA_TRY(cudaFuncSetAttribute(conv_pool_diag_kernel<BS, F>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  conv_pool_diag_kernel<BS, F><<<dim3(nb, nb), 256, smem, st>>>(A, L, pooled);
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}

// ---------------------------------------------------------------- order statistics (one CTA)
__device__ __forceinline__ uint32_t order_key(float x) {
  uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

// k-th smallest (0-based) of vals[0..n) by 4 passes of 8-bit radix select.  All threads call it.
__device__ float select_kth(const float* __restrict__ vals, int n, int k, int* hist, int* s_sel) {
  uint32_t prefix = 0, mask = 0;
  for (int pass = 3; pass >= 0; --pass) {
    const int shift = pass * 8;
    for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const uint32_t key = order_key(vals[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int acc = 0, digit = 255, kk = k;
      for (int b = 0; b < 256; ++b) {
        if (kk < acc + hist[b]) { digit = b; kk -= acc; break; }
        acc += hist[b];
      }
      s_sel[0] = digit;
      s_sel[1] = kk;
    }
    __syncthreads();
    prefix |= (uint32_t)s_sel[0] << shift;
    mask |= 255u << shift;
    k = s_sel[1];
    __syncthreads();
  }
  return key_to_float(prefix);
}

// ---------------------------------------------------------------- selection (one CTA)
// select == PATHS: thresh = torch.quantile(pooled, q) (linear), then 2*nb greedy walkers.
// select == TOPK : the kcount largest cells (ties: lower flat index first).
__global__ void __launch_bounds__(1024) select_kernel(const float* __restrict__ pooled, int nb, int select, float q,
                                                      int kcount, uint8_t* __restrict__ mat,
                                                      float* __restrict__ thresh_out) {
  __shared__ int hist[256];
  __shared__ int s_sel[2];
  __shared__ float s_thresh;
  __shared__ int s_warp[32];
  __shared__ int s_running;
  const int n = nb * nb;
  for (int i = threadIdx.x; i < n; i += blockDim.x) mat[i] = 0;
  __syncthreads();

  if (select == SPION_SELECT_PATHS) {
    // torch.quantile: rank = fp32(q) * fp32(n-1); lerp(lo, hi, w) as torch's fused CPU kernel
    const float rank = __fmul_rn(q, (float)(n - 1));
    const float fl = floorf(rank);
    const int lo_i = (int)fl;
    const int hi_i = (int)ceilf(rank);
    const float w = __fsub_rn(rank, fl);
    const float lo = select_kth(pooled, n, lo_i, hist, s_sel);
    const float hi = (hi_i == lo_i) ? lo : select_kth(pooled, n, hi_i, hist, s_sel);
    if (threadIdx.x == 0) {
      const float d = __fsub_rn(hi, lo);
      float t;
      if (fabsf(w) < 0.5f) t = __fmaf_rn(w, d, lo);
      else t = __fmaf_rn(-d, __fsub_rn(1.0f, w), hi);
      s_thresh = t;
      if (thresh_out) *thresh_out = t;
    }
    __syncthreads();
    const float thresh = s_thresh;
    // walkers: seeds (0,k) then (k,0); main_conv_ff.py:271-274.  Order-free: marks are idempotent.
    for (int s = threadIdx.x; s < 2 * nb; s += blockDim.x) {
      int x = (s < nb) ? 0 : s - nb;
      int y = (s < nb) ? s : 0;
      while (x < nb && y < nb) {                       // stops on the zero guard row / column (:37)
        const float D = (x + 1 < nb) ? pooled[(size_t)(x + 1) * nb + y] : 0.0f;
        const float R = (y + 1 < nb) ? pooled[(size_t)x * nb + y + 1] : 0.0f;
        const float G = (x + 1 < nb && y + 1 < nb) ? pooled[(size_t)(x + 1) * nb + y + 1] : 0.0f;
        float v;
        if (D > R) {
          if (D > G) { x += 1; v = D; } else { x += 1; y += 1; v = G; }
        } else {
          if (R > G) { y += 1; v = R; } else { x += 1; y += 1; v = G; }
        }
        if (v > thresh && v > 0.0f && x < nb && y < nb) mat[(size_t)x * nb + y] = 1;
      }
    }
  } else {
    if (thresh_out && threadIdx.x == 0) *thresh_out = 0.0f;
    if (kcount > 0) {
      const int kk = kcount > n ? n : kcount;
      const float v = select_kth(pooled, n, n - kk, hist, s_sel);   // kk-th largest
      // count strictly greater
      if (threadIdx.x == 0) s_running = 0;
      __syncthreads();
      int local = 0;
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        if (pooled[i] > v) { mat[i] = 1; ++local; }
      }
      atomicAdd(&s_running, local);
      __syncthreads();
      const int need = kk - s_running;                 // how many cells equal to v to take
      __syncthreads();
      if (threadIdx.x == 0) s_running = 0;
      __syncthreads();
      const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
      for (int base = 0; base < n; base += blockDim.x) {
        const int i = base + threadIdx.x;
        const int flag = (i < n && pooled[i] == v) ? 1 : 0;
        const unsigned bal = __ballot_sync(0xffffffffu, flag);
        const int in_warp = __popc(bal & ((1u << lane) - 1u));
        if (lane == 0) s_warp[wid] = __popc(bal);
        __syncthreads();
        int before = s_running;
        for (int w2 = 0; w2 < wid; ++w2) before += s_warp[w2];
        if (flag && before + in_warp < need) mat[i] = 1;
        __syncthreads();
        if (threadIdx.x == 0) {
          int tot = 0;
          for (int w2 = 0; w2 < nwarps; ++w2) tot += s_warp[w2];
          s_running += tot;
        }
        __syncthreads();
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nb; i += blockDim.x) mat[(size_t)i * nb + i] = 1;   // main_conv_ff.py:277-278
}

// ---------------------------------------------------------------- mean over (b,h) of the dense map
// out[i*L + j] = (1/H) sum_h ( (1/B) sum_b in[b*H + h][...] ), b and h ascending.
// A thread owns four consecutive memory columns of one row (16-byte loads, 512 contiguous bytes per warp and
// matrix) and keeps eight matrices' loads in flight; the additions stay in the order above.  L % 128 == 0.
__global__ void __launch_bounds__(256) mean_map_kernel(const float* __restrict__ attn, int B, int H, int L, int transposed,
                                                       float* __restrict__ A) {
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  const size_t LL = (size_t)L * L;
  const int row = blockIdx.y * 8 + ty, col = blockIdx.x * 128 + 4 * tx;        // memory coordinates
  const size_t m = (size_t)row * L + col;
  float4 acc_h = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int hh = 0; hh < H; ++hh) {
    float4 acc_b = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int b = 0; b < B; ++b) {
      const float4 v = *reinterpret_cast<const float4*>(attn + (size_t)(b * H + hh) * LL + m);
      acc_b.x += v.x; acc_b.y += v.y; acc_b.z += v.z; acc_b.w += v.w;
    }
    acc_h.x += acc_b.x / (float)B; acc_h.y += acc_b.y / (float)B;
    acc_h.z += acc_b.z / (float)B; acc_h.w += acc_b.w / (float)B;
  }
  const float4 r = make_float4(acc_h.x / (float)H, acc_h.y / (float)H, acc_h.z / (float)H, acc_h.w / (float)H);
  if (transposed) {                                          // memory (row = j, col = i) -> A[i][j]
    A[(size_t)(col + 0) * L + row] = r.x;
    A[(size_t)(col + 1) * L + row] = r.y;
    A[(size_t)(col + 2) * L + row] = r.z;
    A[(size_t)(col + 3) * L + row] = r.w;
  } else {
    *reinterpret_cast<float4*>(A + m) = r;
  }
}

// The same for any L that is a multiple of 32 (one value per thread, 32 x 32 tiles through shared memory).
__global__ void mean_map_kernel32(const float* __restrict__ attn, int B, int H, int L, int transposed,
                                  float* __restrict__ A) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x, ty = threadIdx.y;             // 32 x 8
  const size_t LL = (size_t)L * L;
  for (int rr = ty; rr < 32; rr += 8) {
    // memory coordinates: row = blockIdx.y*32 + rr, col = blockIdx.x*32 + tx
    const size_t m = (size_t)(blockIdx.y * 32 + rr) * L + blockIdx.x * 32 + tx;
    float acc_h = 0.0f;
    for (int hh = 0; hh < H; ++hh) {
      float acc_b = 0.0f;
#pragma unroll 8
      for (int b = 0; b < B; ++b) acc_b += attn[(size_t)(b * H + hh) * LL + m];   // loads of eight matrices in flight; sum in order
      acc_h += acc_b / (float)B;
    }
    tile[rr][tx] = acc_h / (float)H;
  }
  __syncthreads();
  for (int rr = ty; rr < 32; rr += 8) {
    if (transposed) {
      // memory (row=j, col=i) -> A[i][j]
      const int i = blockIdx.x * 32 + rr, j = blockIdx.y * 32 + tx;
      A[(size_t)i * L + j] = tile[tx][rr];
    } else {
      const int i = blockIdx.y * 32 + rr, j = blockIdx.x * 32 + tx;
      A[(size_t)i * L + j] = tile[rr][tx];
    }
  }
}

// Mean over the (b,h) matrices of block-tile probabilities: one CTA per selected block.
// A[i, j] = (1 / BH) * sum_bh P[bh][blk][i % bs][j % bs]; cells of unselected blocks stay 0.
template <typename T>
__global__ void __launch_bounds__(256) mean_map_tiles_kernel(const T* __restrict__ P, const int32_t* __restrict__ blk_row,
                                                             const int32_t* __restrict__ col_idx, int bs, int nnzb,
                                                             int BH, int L, float* __restrict__ A) {
  const int blk = blockIdx.x;
  const int r = blk_row[blk], c = col_idx[blk];
  const int n = bs * bs;
  const float inv = 1.0f / (float)BH;
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    float acc = 0.f;
    const T* src = P + (size_t)blk * n + e;
#pragma unroll 8
    for (int bh = 0; bh < BH; ++bh) acc += to_f32(src[(size_t)bh * nnzb * n]);   // eight loads in flight; sum in order
    A[(size_t)(r * bs + e / bs) * L + c * bs + e % bs] = acc * inv;
  }
}

}  // namespace

extern "C" int spion_mean_map_tiles(const void* P, int dtype, const int32_t* blk_row, const int32_t* col_idx,
                                    int block_size, int nnzb, int num_batches, int L, float* A, void* cuda_stream) {
  if (!P || !blk_row || !col_idx || !A) return SPION_ERR_ARG;
  if (block_size < 1 || nnzb < 0 || num_batches < 1 || L < 1 || L % block_size != 0) return SPION_ERR_SHAPE;
  if (dtype != SPION_F32 && dtype != SPION_BF16) return SPION_ERR_ARG;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  SPION_CUDA_TRY(cudaMemsetAsync(A, 0, (size_t)L * L * sizeof(float), st));
  if (nnzb == 0) return SPION_OK;
  if (dtype == SPION_F32)
    mean_map_tiles_kernel<float><<<nnzb, 256, 0, st>>>((const float*)P, blk_row, col_idx, block_size, nnzb,
                                                       num_batches, L, A);
  else
    mean_map_tiles_kernel<__nv_bfloat16><<<nnzb, 256, 0, st>>>((const __nv_bfloat16*)P, blk_row, col_idx, block_size,
                                                               nnzb, num_batches, L, A);
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}

extern "C" int spion_discover_pattern(const float* A, int L, int block_size, int conv_kind, int F, int select,
                                      double param, uint8_t* mat, float* pooled, float* thresh, int32_t* nnzb,
                                      int32_t* row_ptr, int32_t* col_idx, int32_t* blk_row, int32_t* col_ptr,
                                      int32_t* row_idx, int32_t* csc_pos, int32_t* work, int32_t* host_nnzb,
                                      void* cuda_stream) {
  if (!A || !mat || !pooled || !nnzb || !row_ptr || !col_idx || !blk_row || !col_ptr || !row_idx || !csc_pos || !work)
    return SPION_ERR_ARG;
  if (L < 1 || block_size < 1 || L % block_size != 0) return SPION_ERR_SHAPE;
  const int bs = block_size, nb = L / bs;
  if (nb > SPION_MAX_NB || bs > 128) return SPION_ERR_SHAPE;
  if (F < 1 || F % 2 == 0 || F > 65) return SPION_ERR_ARG;
  if (conv_kind != SPION_CONV_DIAG && conv_kind != SPION_CONV_BOX) return SPION_ERR_ARG;
  if (select != SPION_SELECT_PATHS && select != SPION_SELECT_TOPK) return SPION_ERR_ARG;
  if (select == SPION_SELECT_PATHS && !(param >= 0.0 && param <= 1.0)) return SPION_ERR_ARG;
  cudaStream_t st = (cudaStream_t)cuda_stream;

  const int T = bs + F - 1;
  size_t smem = (((size_t)T * T * sizeof(float) + 15) & ~(size_t)15) + ((size_t)bs * bs + bs) * sizeof(double);
  // The opt-in above 48 KB belongs to the current device only (a process may drive several), and the
  // call is cheap: make it on every launch that needs it instead of remembering one process-wide size.
  if (conv_kind == SPION_CONV_DIAG && F == 31 && (bs == 64 || bs == 32)) {      // the reference's filter: the faster kernel
    int rc = bs == 64 ? launch_conv_pool_diag<64, 31>(A, L, nb, pooled, st) : launch_conv_pool_diag<32, 31>(A, L, nb, pooled, st);
    if (rc) return rc;
  } else {
    if (smem > 48 * 1024)
      SPION_CUDA_TRY(cudaFuncSetAttribute(conv_pool_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    conv_pool_kernel<<<dim3(nb, nb), 256, smem, st>>>(A, L, bs, conv_kind, F, pooled);
    SPION_LAUNCH_CHECK();
  }

  int kcount = 0;
  if (select == SPION_SELECT_TOPK) kcount = (int)((double)(nb * nb) * param - (double)nb);   // main_conv.py:247
  select_kernel<<<1, 1024, 0, st>>>(pooled, nb, select, (float)param, kcount, mat, thresh);
  SPION_LAUNCH_CHECK();
  int rc = spion_launch_build_structure(mat, nb, nnzb, row_ptr, col_idx, blk_row, col_ptr, row_idx, csc_pos, work, st);
  if (rc) return rc;
  if (host_nnzb) {
    SPION_CUDA_TRY(cudaMemcpyAsync(host_nnzb, nnzb, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    SPION_CUDA_TRY(cudaStreamSynchronize(st));
  }
  return SPION_OK;
}

extern "C" int spion_mean_attention_map(const float* attn, int batch, int heads, int L, int transposed, float* A,
                                        void* cuda_stream) {
  if (!attn || !A) return SPION_ERR_ARG;
  if (batch < 1 || heads < 1 || L < 32 || L % 32 != 0) return SPION_ERR_SHAPE;
  const bool aligned = (((uintptr_t)attn | (uintptr_t)A) & 15u) == 0;          // 16-byte loads and stores
  if (L % 128 == 0 && aligned)
    mean_map_kernel<<<dim3(L / 128, L / 8), 256, 0, (cudaStream_t)cuda_stream>>>(attn, batch, heads, L, transposed, A);
  else
    mean_map_kernel32<<<dim3(L / 32, L / 32), dim3(32, 8), 0, (cudaStream_t)cuda_stream>>>(attn, batch, heads, L,
                                                                                            transposed, A);
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}
