// Layer normalisation over the last dimension of an [M, N] fp32 matrix, forward and backward, for the
// encoder layers around the attention call (the reference uses torch.nn.LayerNorm:
// models/model_transformer.py, `self.norm1 / self.norm2 / self.norm`).
//
// Why a kernel of its own: the rows are short (N = transformer_dim = 64 in the LRA configurations,
// config.py) and there are B * L of them (32 768 .. 524 288 per call).  The backward of the framework's
// operator computes the weight / bias gradients as a column reduction over all rows with a handful of
// CTAs (it is the largest single kernel of the small-batch training step); here the same pass that forms
// dX keeps per-lane partial sums of dgamma and dbeta in registers, one partial row per CTA goes to a
// workspace, and a second small kernel adds the partial rows in a fixed order (deterministic results).
//
// HBM-bound by design: forward reads X and writes Y (+ two floats per row); backward reads X and dY and
// writes dX.  One warp per row, lanes own the columns {2 l, 2 l + 1} + 64 k, rows are taken with stride
// (warps in the grid).  Y and dY may be bf16 (what the following linear layers consume / produce under
// mixed precision) or fp32.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace {

constexpr int LN_WARPS = 8;                 // warps per CTA
constexpr int LN_MAX_CTAS = 2048;           // partial rows of the weight / bias gradients

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <bool BF16> __device__ __forceinline__ float2 load2(const void* p, size_t i);
template <> __device__ __forceinline__ float2 load2<false>(const void* p, size_t i) {
  return *reinterpret_cast<const float2*>(static_cast<const float*>(p) + i);
}
template <> __device__ __forceinline__ float2 load2<true>(const void* p, size_t i) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(static_cast<const __nv_bfloat16*>(p) + i));
}
template <bool BF16> __device__ __forceinline__ void store2(void* p, size_t i, float2 v);
template <> __device__ __forceinline__ void store2<false>(void* p, size_t i, float2 v) {
  *reinterpret_cast<float2*>(static_cast<float*>(p) + i) = v;
}
template <> __device__ __forceinline__ void store2<true>(void* p, size_t i, float2 v) {
  *reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(p) + i) = __float22bfloat162_rn(v);
}

// K = N / 64: pairs of columns per lane
template <int K, bool Y_BF16>
__global__ void __launch_bounds__(LN_WARPS * 32) ln_fwd_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                               const float* __restrict__ beta, void* __restrict__ y,
                                                               float* __restrict__ mean, float* __restrict__ rstd,
                                                               long long M, float eps, const void* __restrict__ res,
                                                               int res_is_bf16, float* __restrict__ sum_out) {
  // res != nullptr: the row that is normalised is x + res (a residual connection: x the fp32 stream, res the
  // branch output, fp32 or bf16), and it is also written to sum_out
  constexpr int N = 64 * K;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * LN_WARPS + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * LN_WARPS;
  float2 g[K], b[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    g[k] = *reinterpret_cast<const float2*>(gamma + 64 * k + 2 * lane);
    b[k] = *reinterpret_cast<const float2*>(beta + 64 * k + 2 * lane);
  }
#pragma unroll 2   // the loads of a second row are issued before the first row's reductions
  for (long long r = warp0; r < M; r += nwarps) {
    float2 v[K];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const size_t i = (size_t)r * N + 64 * k + 2 * lane;
      v[k] = *reinterpret_cast<const float2*>(x + i);
      if (res) {
        const float2 a = res_is_bf16 ? load2<true>(res, i) : load2<false>(res, i);
        v[k].x += a.x; v[k].y += a.y;
        *reinterpret_cast<float2*>(sum_out + i) = v[k];
      }
      s += v[k].x + v[k].y;
    }
    const float mu = warp_sum(s) * (1.0f / N);
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const float dx = v[k].x - mu, dy = v[k].y - mu;
      q += dx * dx + dy * dy;
    }
    const float rs = rsqrtf(warp_sum(q) * (1.0f / N) + eps);      // biased variance, as torch.nn.LayerNorm
#pragma unroll
    for (int k = 0; k < K; ++k)
      store2<Y_BF16>(y, (size_t)r * N + 64 * k + 2 * lane,
                     make_float2((v[k].x - mu) * rs * g[k].x + b[k].x, (v[k].y - mu) * rs * g[k].y + b[k].y));
    if (lane == 0) { mean[r] = mu; rstd[r] = rs; }
  }
}

template <int K, bool DY_BF16>
__global__ void __launch_bounds__(LN_WARPS * 32) ln_bwd_kernel(const float* __restrict__ x, const void* __restrict__ dy,
                                                               const float* __restrict__ gamma, const float* __restrict__ mean,
                                                               const float* __restrict__ rstd, float* __restrict__ dx,
                                                               float* __restrict__ partial, long long M,
                                                               const float* __restrict__ dskip,
                                                               __nv_bfloat16* __restrict__ dx_bf16) {
  // dskip != nullptr: dx = (gradient through the normalisation) + dskip, the gradient that reaches the same row
  // through the residual connection; dx_bf16 != nullptr: a bf16 copy of dx (the gradient of a bf16 branch output)
  constexpr int N = 64 * K;
  __shared__ float s_g[LN_WARPS][N], s_b[LN_WARPS][N];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long warp0 = (long long)blockIdx.x * LN_WARPS + warp, nwarps = (long long)gridDim.x * LN_WARPS;
  float2 g[K], ag[K], ab[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    g[k] = *reinterpret_cast<const float2*>(gamma + 64 * k + 2 * lane);
    ag[k] = make_float2(0.f, 0.f);
    ab[k] = make_float2(0.f, 0.f);
  }
#pragma unroll 2
  for (long long r = warp0; r < M; r += nwarps) {
    const float mu = mean[r], rs = rstd[r];
    float2 xh[K], gy[K];
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const size_t i = (size_t)r * N + 64 * k + 2 * lane;
      const float2 xv = *reinterpret_cast<const float2*>(x + i);
      const float2 d = load2<DY_BF16>(dy, i);
      xh[k] = make_float2((xv.x - mu) * rs, (xv.y - mu) * rs);
      gy[k] = make_float2(d.x * g[k].x, d.y * g[k].y);
      c1 += gy[k].x + gy[k].y;
      c2 += gy[k].x * xh[k].x + gy[k].y * xh[k].y;
      ag[k].x += d.x * xh[k].x; ag[k].y += d.y * xh[k].y;
      ab[k].x += d.x; ab[k].y += d.y;
    }
    c1 = warp_sum(c1) * (1.0f / N);
    c2 = warp_sum(c2) * (1.0f / N);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const size_t i = (size_t)r * N + 64 * k + 2 * lane;
      float2 o = make_float2((gy[k].x - c1 - xh[k].x * c2) * rs, (gy[k].y - c1 - xh[k].y * c2) * rs);
      if (dskip) {
        const float2 a = *reinterpret_cast<const float2*>(dskip + i);
        o.x += a.x; o.y += a.y;
      }
      *reinterpret_cast<float2*>(dx + i) = o;
      if (dx_bf16) store2<true>(dx_bf16, i, o);
    }
  }
  // the CTA's partial row: the warps' sums added in warp order
#pragma unroll
  for (int k = 0; k < K; ++k) {
    *reinterpret_cast<float2*>(&s_g[warp][64 * k + 2 * lane]) = ag[k];
    *reinterpret_cast<float2*>(&s_b[warp][64 * k + 2 * lane]) = ab[k];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < N; c += blockDim.x) {
    float sg = 0.f, sb = 0.f;
#pragma unroll
    for (int w = 0; w < LN_WARPS; ++w) { sg += s_g[w][c]; sb += s_b[w][c]; }
    partial[(size_t)blockIdx.x * 2 * N + c] = sg;
    partial[(size_t)blockIdx.x * 2 * N + N + c] = sb;
  }
}

// dgamma[c] = sum over the partial rows; likewise dbeta.  One CTA of 32 warps per 32 columns: warp w adds the
// rows w, w + 32, ... of its columns (coalesced), then the 32 per-warp sums are added in warp order: the order
// of the additions is fixed, so the result does not depend on the run.
__global__ void __launch_bounds__(1024) ln_bwd_reduce_kernel(const float* __restrict__ partial, int rows, int N,
                                                              float* __restrict__ dgamma, float* __restrict__ dbeta) {
  __shared__ float s_p[32][33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;                      // column of the [rows, 2 N] partial matrix
  float s = 0.f;
  for (int r = warp; r < rows; r += 32) s += partial[(size_t)r * 2 * N + c];
  s_p[warp][lane] = s;
  __syncthreads();
  if (warp == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 32; ++w) t += s_p[w][lane];
    if (c < N) dgamma[c] = t; else dbeta[c - N] = t;
  }
}

// Column sums of an [M, N] matrix (the bias gradient of a linear layer: sum of dY over all rows), first stage:
// one partial row per CTA, same lane / column mapping and the same fixed-order second stage as above.
template <int K, bool BF16>
__global__ void __launch_bounds__(LN_WARPS * 32) colsum_kernel(const void* __restrict__ dy, float* __restrict__ partial,
                                                                long long M) {
  constexpr int N = 64 * K;
  __shared__ float s_b[LN_WARPS][N];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long warp0 = (long long)blockIdx.x * LN_WARPS + warp, nwarps = (long long)gridDim.x * LN_WARPS;
  float2 ab[K];
#pragma unroll
  for (int k = 0; k < K; ++k) ab[k] = make_float2(0.f, 0.f);
#pragma unroll 4
  for (long long r = warp0; r < M; r += nwarps) {
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const float2 d = load2<BF16>(dy, (size_t)r * N + 64 * k + 2 * lane);
      ab[k].x += d.x; ab[k].y += d.y;
    }
  }
#pragma unroll
  for (int k = 0; k < K; ++k) *reinterpret_cast<float2*>(&s_b[warp][64 * k + 2 * lane]) = ab[k];
  __syncthreads();
  for (int c = threadIdx.x; c < N; c += blockDim.x) {
    float sb = 0.f;
#pragma unroll
    for (int w = 0; w < LN_WARPS; ++w) sb += s_b[w][c];
    partial[(size_t)blockIdx.x * N + c] = sb;
  }
}

// out[c] = sum over the partial rows of an [rows, N] matrix, fixed order (see ln_bwd_reduce_kernel)
__global__ void __launch_bounds__(1024) colsum_reduce_kernel(const float* __restrict__ partial, int rows, int N,
                                                              float* __restrict__ out) {
  __shared__ float s_p[32][33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s = 0.f;
  for (int r = warp; r < rows; r += 32) s += partial[(size_t)r * N + c];
  s_p[warp][lane] = s;
  __syncthreads();
  if (warp == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 32; ++w) t += s_p[w][lane];
    out[c] = t;
  }
}

// ---- backward and column sums of widths 64 and 128 with 16-byte loads: N / 4 lanes per row, so a warp works on
// 32 / (N / 4) rows at once (twice the bytes in flight per warp of the kernels above at N = 64).  Lane j of a row owns
// columns 4 j .. 4 j + 3.  Same formulas; the per-row sums are formed in another order, the weight / bias gradients go
// through the same fixed-order second stage.  (The forward measured slower in this form and keeps one warp per row.)
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
  const uint2 w = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 w;
  w.x = *reinterpret_cast<const unsigned*>(&lo);
  w.y = *reinterpret_cast<const unsigned*>(&hi);
  *reinterpret_cast<uint2*>(p) = w;
}
template <int LPR>
__device__ __forceinline__ float row_sum(float v) {   // over the LPR lanes of a row (all 32 lanes take part)
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int N, typename TD>
__global__ void __launch_bounds__(LN_WARPS * 32) ln_bwd4_kernel(const float* __restrict__ x, const TD* __restrict__ dy,
                                                                const float* __restrict__ gamma, const float* __restrict__ mean,
                                                                const float* __restrict__ rstd, float* __restrict__ dx,
                                                                float* __restrict__ partial, long long M,
                                                                const float* __restrict__ dskip,
                                                                __nv_bfloat16* __restrict__ dx_bf16) {
  constexpr int LPR = N / 4, RPW = 32 / LPR;
  __shared__ float s_g[LN_WARPS * RPW][N], s_b[LN_WARPS * RPW][N];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, j = lane % LPR, sub = lane / LPR;
  const long long warp0 = (long long)blockIdx.x * LN_WARPS + warp, nwarps = (long long)gridDim.x * LN_WARPS;
  const float4 g = ld4(gamma + 4 * j);
  float4 ag = make_float4(0.f, 0.f, 0.f, 0.f), ab = ag;
#pragma unroll 2
  for (long long r0 = warp0 * RPW; r0 < M; r0 += nwarps * RPW) {
    const long long r = r0 + sub;
    const bool live = r < M;
    const long long rr = live ? r : 0;
    const size_t i = (size_t)rr * N + 4 * j;
    const float mu = mean[rr], rs = rstd[rr];
    const float4 xv = ld4(x + i);
    float4 d = ld4(dy + i);
    if (!live) d = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 xh = make_float4((xv.x - mu) * rs, (xv.y - mu) * rs, (xv.z - mu) * rs, (xv.w - mu) * rs);
    const float4 gy = make_float4(d.x * g.x, d.y * g.y, d.z * g.z, d.w * g.w);
    ag.x += d.x * xh.x, ag.y += d.y * xh.y, ag.z += d.z * xh.z, ag.w += d.w * xh.w;
    ab.x += d.x, ab.y += d.y, ab.z += d.z, ab.w += d.w;
    const float c1 = row_sum<LPR>((gy.x + gy.y) + (gy.z + gy.w)) * (1.0f / N);
    const float c2 = row_sum<LPR>((gy.x * xh.x + gy.y * xh.y) + (gy.z * xh.z + gy.w * xh.w)) * (1.0f / N);
    if (live) {
      float4 o = make_float4((gy.x - c1 - xh.x * c2) * rs, (gy.y - c1 - xh.y * c2) * rs, (gy.z - c1 - xh.z * c2) * rs,
                             (gy.w - c1 - xh.w * c2) * rs);
      if (dskip) {
        const float4 a = ld4(dskip + i);
        o.x += a.x, o.y += a.y, o.z += a.z, o.w += a.w;
      }
      st4(dx + i, o);
      if (dx_bf16) st4(dx_bf16 + i, o);
    }
  }
  // the CTA's partial row: the sums of its (warp, sub-row) groups added in that order
  st4(&s_g[warp * RPW + sub][4 * j], ag);
  st4(&s_b[warp * RPW + sub][4 * j], ab);
  __syncthreads();
  for (int c = threadIdx.x; c < N; c += blockDim.x) {
    float sg = 0.f, sb = 0.f;
#pragma unroll
    for (int w = 0; w < LN_WARPS * RPW; ++w) { sg += s_g[w][c]; sb += s_b[w][c]; }
    partial[(size_t)blockIdx.x * 2 * N + c] = sg;
    partial[(size_t)blockIdx.x * 2 * N + N + c] = sb;
  }
}

// Column sums with 16-byte loads: a row of N values takes LPR = N * sizeof(T) / 16 lanes (8 or 16 for N = 64, 16 or 32
// for N = 128), a warp reads 32 / LPR rows per step, four steps in flight.
template <int N, typename T>
__global__ void __launch_bounds__(LN_WARPS * 32) colsum4_kernel(const T* __restrict__ dy, float* __restrict__ partial,
                                                                long long M) {
  constexpr int PER = 16 / (int)sizeof(T), LPR = N / PER, RPW = 32 / LPR;
  __shared__ float s_b[LN_WARPS * RPW][N];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, j = lane % LPR, sub = lane / LPR;
  const long long warp0 = (long long)blockIdx.x * LN_WARPS + warp, nwarps = (long long)gridDim.x * LN_WARPS;
  float acc[PER];
#pragma unroll
  for (int k = 0; k < PER; ++k) acc[k] = 0.f;
#pragma unroll 4
  for (long long r = warp0 * RPW + sub; r < M; r += nwarps * RPW) {
    const T* src = dy + (size_t)r * N + PER * j;
    if constexpr (PER == 8) {
      const uint4 w = *reinterpret_cast<const uint4*>(src);
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w.y));
      const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w.z));
      const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w.w));
      acc[0] += a.x, acc[1] += a.y, acc[2] += b.x, acc[3] += b.y;
      acc[4] += c.x, acc[5] += c.y, acc[6] += d.x, acc[7] += d.y;
    } else {
      const float4 a = ld4(src);
      acc[0] += a.x, acc[1] += a.y, acc[2] += a.z, acc[3] += a.w;
    }
  }
#pragma unroll
  for (int k = 0; k < PER; ++k) s_b[warp * RPW + sub][PER * j + k] = acc[k];
  __syncthreads();
  for (int c = threadIdx.x; c < N; c += blockDim.x) {
    float sb = 0.f;
#pragma unroll
    for (int w = 0; w < LN_WARPS * RPW; ++w) sb += s_b[w][c];
    partial[(size_t)blockIdx.x * N + c] = sb;
  }
}

int ln_grid(long long M) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return -1;
  // at least eight rows per warp (fewer CTAs mean fewer partial rows of the weight / bias gradients to add up);
  // at most 8 CTAs of 8 warps per SM: all warp slots
  long long want = (M + LN_WARPS * 8 - 1) / (LN_WARPS * 8), cap = (long long)sms * 8;
  if (cap > LN_MAX_CTAS) cap = LN_MAX_CTAS;
  return (int)(want < cap ? want : cap);
}

}  // namespace

namespace {

// every pointer given (null ones aside) on a 16-byte boundary: what the kernels with 16-byte loads need
template <typename... P>
bool aligned16(const P*... p) { return ((... | (uintptr_t)p) & 15) == 0; }

int ln_forward(const float* x, const void* res, int res_is_bf16, float* sum_out, const float* gamma, const float* beta,
               void* y, int y_is_bf16, float* mean, float* rstd, long long M, int N, float eps, cudaStream_t stream) {
  const int grid = ln_grid(M);
  if (grid < 1) return SPION_ERR_CUDA;
#define SPION_LN_FWD(K)                                                                                               \
  if (y_is_bf16)                                                                                                      \
    ln_fwd_kernel<K, true><<<grid, LN_WARPS * 32, 0, stream>>>(x, gamma, beta, y, mean, rstd, M, eps, res, res_is_bf16, \
                                                               sum_out);                                              \
  else                                                                                                                \
    ln_fwd_kernel<K, false><<<grid, LN_WARPS * 32, 0, stream>>>(x, gamma, beta, y, mean, rstd, M, eps, res,            \
                                                                res_is_bf16, sum_out);
  switch (N) {
    case 64: SPION_LN_FWD(1) break;
    case 128: SPION_LN_FWD(2) break;
    case 256: SPION_LN_FWD(4) break;
    case 512: SPION_LN_FWD(8) break;
    default: return SPION_ERR_SHAPE;
  }
#undef SPION_LN_FWD
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}

int ln_backward(const float* x, const void* dy, int dy_is_bf16, const float* gamma, const float* mean, const float* rstd,
                const float* dskip, float* dx, __nv_bfloat16* dx_bf16, float* dgamma, float* dbeta, float* workspace,
                long long M, int N, cudaStream_t stream) {
  const int grid = ln_grid(M);
  if (grid < 1) return SPION_ERR_CUDA;
  if ((N == 64 || N == 128) && aligned16(x, dy, dx, dskip, dx_bf16, gamma)) {
    if (N == 64 && dy_is_bf16)
      ln_bwd4_kernel<64, __nv_bfloat16><<<grid, LN_WARPS * 32, 0, stream>>>(x, (const __nv_bfloat16*)dy, gamma, mean, rstd, dx,
                                                                            workspace, M, dskip, dx_bf16);
    else if (N == 64)
      ln_bwd4_kernel<64, float><<<grid, LN_WARPS * 32, 0, stream>>>(x, (const float*)dy, gamma, mean, rstd, dx, workspace, M,
                                                                    dskip, dx_bf16);
    else if (dy_is_bf16)
      ln_bwd4_kernel<128, __nv_bfloat16><<<grid, LN_WARPS * 32, 0, stream>>>(x, (const __nv_bfloat16*)dy, gamma, mean, rstd,
                                                                             dx, workspace, M, dskip, dx_bf16);
    else
      ln_bwd4_kernel<128, float><<<grid, LN_WARPS * 32, 0, stream>>>(x, (const float*)dy, gamma, mean, rstd, dx, workspace, M,
                                                                     dskip, dx_bf16);
    SPION_LAUNCH_CHECK();
    ln_bwd_reduce_kernel<<<2 * N / 32, 1024, 0, stream>>>(workspace, grid, N, dgamma, dbeta);
    SPION_LAUNCH_CHECK();
    return SPION_OK;
  }
#define SPION_LN_BWD(K)                                                                                              \
  if (dy_is_bf16)                                                                                                    \
    ln_bwd_kernel<K, true><<<grid, LN_WARPS * 32, 0, stream>>>(x, dy, gamma, mean, rstd, dx, workspace, M, dskip,    \
                                                               dx_bf16);                                             \
  else                                                                                                               \
    ln_bwd_kernel<K, false><<<grid, LN_WARPS * 32, 0, stream>>>(x, dy, gamma, mean, rstd, dx, workspace, M, dskip,   \
                                                                dx_bf16);
  switch (N) {
    case 64: SPION_LN_BWD(1) break;
    case 128: SPION_LN_BWD(2) break;
    case 256: SPION_LN_BWD(4) break;
    case 512: SPION_LN_BWD(8) break;
    default: return SPION_ERR_SHAPE;
  }
#undef SPION_LN_BWD
  SPION_LAUNCH_CHECK();
  ln_bwd_reduce_kernel<<<2 * N / 32, 1024, 0, stream>>>(workspace, grid, N, dgamma, dbeta);
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}

}  // namespace

// N must be 64, 128, 256 or 512; rows are contiguous.  Returns SPION_ERR_SHAPE otherwise.
extern "C" int spion_layernorm_forward(const float* x, const float* gamma, const float* beta, void* y, int y_is_bf16,
                                       float* mean, float* rstd, long long M, int N, float eps, void* cuda_stream) {
  if (!x || !gamma || !beta || !y || !mean || !rstd || M < 1) return SPION_ERR_ARG;
  return ln_forward(x, nullptr, 0, nullptr, gamma, beta, y, y_is_bf16, mean, rstd, M, N, eps, (cudaStream_t)cuda_stream);
}

// Residual connection and normalisation in one pass: sum_out = x + res (res fp32 or bf16), y = LayerNorm(sum_out).
extern "C" int spion_add_layernorm_forward(const float* x, const void* res, int res_is_bf16, float* sum_out,
                                           const float* gamma, const float* beta, void* y, int y_is_bf16, float* mean,
                                           float* rstd, long long M, int N, float eps, void* cuda_stream) {
  if (!x || !res || !sum_out || !gamma || !beta || !y || !mean || !rstd || M < 1) return SPION_ERR_ARG;
  return ln_forward(x, res, res_is_bf16, sum_out, gamma, beta, y, y_is_bf16, mean, rstd, M, N, eps,
                    (cudaStream_t)cuda_stream);
}

// Floats the backward needs as workspace for a width of N.
extern "C" long long spion_layernorm_workspace_floats(int N) { return (long long)LN_MAX_CTAS * 2 * N; }

extern "C" int spion_layernorm_backward(const float* x, const void* dy, int dy_is_bf16, const float* gamma,
                                        const float* mean, const float* rstd, float* dx, float* dgamma, float* dbeta,
                                        float* workspace, long long M, int N, void* cuda_stream) {
  if (!x || !dy || !gamma || !mean || !rstd || !dx || !dgamma || !dbeta || !workspace || M < 1) return SPION_ERR_ARG;
  return ln_backward(x, dy, dy_is_bf16, gamma, mean, rstd, nullptr, dx, nullptr, dgamma, dbeta, workspace, M, N,
                     (cudaStream_t)cuda_stream);
}

// Backward of spion_add_layernorm_forward: x is the saved sum; dx = (gradient through the normalisation) + dskip, where
// dskip (may be NULL) is the gradient the sum receives from its other consumers (the next residual connection).
// dx is the gradient of both addends; dx_bf16 (may be NULL) receives a bf16 copy for a bf16 addend.
extern "C" int spion_add_layernorm_backward(const float* x, const void* dy, int dy_is_bf16, const float* gamma,
                                            const float* mean, const float* rstd, const float* dskip, float* dx,
                                            void* dx_bf16, float* dgamma, float* dbeta, float* workspace, long long M,
                                            int N, void* cuda_stream) {
  if (!x || !dy || !gamma || !mean || !rstd || !dx || !dgamma || !dbeta || !workspace || M < 1) return SPION_ERR_ARG;
  return ln_backward(x, dy, dy_is_bf16, gamma, mean, rstd, dskip, dx, (__nv_bfloat16*)dx_bf16, dgamma, dbeta, workspace, M,
                     N, (cudaStream_t)cuda_stream);
}

// Sum of the rows of an [M, N] matrix (fp32 or bf16), N in {64, 128, 256, 512}: out[N] fp32.  The bias gradient of a
// linear layer.  workspace: spion_layernorm_workspace_floats(N) floats.  Fixed summation order.
extern "C" int spion_column_sums(const void* dy, int dy_is_bf16, float* out, float* workspace, long long M, int N,
                                 void* cuda_stream) {
  cudaStream_t stream = (cudaStream_t)cuda_stream;
  if (!dy || !out || !workspace || M < 1) return SPION_ERR_ARG;
  const int grid = ln_grid(M);
  if (grid < 1) return SPION_ERR_CUDA;
  if ((N == 64 || N == 128) && ((uintptr_t)dy & 15) == 0) {
    if (N == 64 && dy_is_bf16) colsum4_kernel<64, __nv_bfloat16><<<grid, LN_WARPS * 32, 0, stream>>>((const __nv_bfloat16*)dy, workspace, M);
    else if (N == 64) colsum4_kernel<64, float><<<grid, LN_WARPS * 32, 0, stream>>>((const float*)dy, workspace, M);
    else if (dy_is_bf16) colsum4_kernel<128, __nv_bfloat16><<<grid, LN_WARPS * 32, 0, stream>>>((const __nv_bfloat16*)dy, workspace, M);
    else colsum4_kernel<128, float><<<grid, LN_WARPS * 32, 0, stream>>>((const float*)dy, workspace, M);
    SPION_LAUNCH_CHECK();
    colsum_reduce_kernel<<<N / 32, 1024, 0, stream>>>(workspace, grid, N, out);
    SPION_LAUNCH_CHECK();
    return SPION_OK;
  }
#define SPION_COLSUM(K)                                                                                   \
  if (dy_is_bf16) colsum_kernel<K, true><<<grid, LN_WARPS * 32, 0, stream>>>(dy, workspace, M);            \
  else colsum_kernel<K, false><<<grid, LN_WARPS * 32, 0, stream>>>(dy, workspace, M);
  switch (N) {
    case 64: SPION_COLSUM(1) break;
    case 128: SPION_COLSUM(2) break;
    case 256: SPION_COLSUM(4) break;
    case 512: SPION_COLSUM(8) break;
    default: return SPION_ERR_SHAPE;
  }
#undef SPION_COLSUM
  SPION_LAUNCH_CHECK();
  colsum_reduce_kernel<<<N / 32, 1024, 0, stream>>>(workspace, grid, N, out);
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}
