// SIMT (CUDA-core, fp32 accumulate) kernels of the block-sparse attention path.
//
// They serve (1) the reference's fp32 layouts behind the drop-in entry points, where the
// 1e-4 max-abs parity bound rules out TF32/BF16 tensor-core inputs, and (2) every shape the
// tcgen05 engine does not cover.  Each kernel works on whole bs x bs blocks of the layer's
// mask; value tiles and dense operands are addressed through strides so that the reference's
// element-CSR layout, its transposed operands (models/attention_blockcuda.py:48,80), its
// S^T-stored dense attention (models/attention_cuda.py:36) and the native block-tile layout
// all go through the same code.
//
//   simt_sddmm        replaces cusparseSDDMM      (models/block_attn.cu:145-224, calls :459,:498)
//   simt_spmm         replaces cusparseSpMM N / T (models/block_attn.cu:236-393, calls :478,:516,:526,:536)
//   softmax_fwd_rows  replaces scale_softmax_kernel            (models/block_attn.cu:33-88, _mask.cu:88-140)
//   softmax_bwd_rows  replaces softmax_scale_backward_kernel   (models/block_attn.cu:90-130)
//   softmax_*_dense_t replace max_sum_exp_kernel[_large] / softmax_scale_backward_kernel[_large]
//                     (models/attn.cu:9-112, models/attn_mask.cu:8-122)
#include "common.cuh"

namespace {

constexpr int KC = 32;   // contraction chunk held in shared memory

template <typename T>
__device__ __forceinline__ float load_op(const T* base, long long idx) { return to_f32(base[idx]); }

// ------------------------------------------------------------------------------ SDDMM
// One CTA per (block, bh): vals(i,j) = sum_n A[r*bs+i, n] * B[c*bs+j, n].
template <typename TI, typename TV, int TM>
__global__ void __launch_bounds__(256) sddmm_kernel(const TI* __restrict__ A, OperandLayout la, const TI* __restrict__ B,
                                                    OperandLayout lb, TV* __restrict__ vals, ValueLayout vl, Pattern p,
                                                    int d) {
  constexpr int BS = TM * 16;
  __shared__ float As[KC][BS + 1];
  __shared__ float Bs[KC][BS + 1];
  const int blk = blockIdx.x, bh = blockIdx.y;
  const int r = p.blk_row[blk], c = p.col_idx[blk];
  const TI* Ab = A + (long long)bh * la.bh_stride + (long long)r * BS * la.sl;
  const TI* Bb = B + (long long)bh * lb.bh_stride + (long long)c * BS * lb.sl;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  float acc[TM][TM];
#pragma unroll
  for (int a = 0; a < TM; ++a)
#pragma unroll
    for (int b = 0; b < TM; ++b) acc[a][b] = 0.f;

  for (int n0 = 0; n0 < d; n0 += KC) {
    for (int idx = tid; idx < BS * KC; idx += 256) {
      int i, n;
      if (la.sd == 1) { n = idx % KC; i = idx / KC; } else { i = idx % BS; n = idx / BS; }
      As[n][i] = load_op(Ab, (long long)i * la.sl + (long long)(n0 + n) * la.sd);
      if (lb.sd == 1) { n = idx % KC; i = idx / KC; } else { i = idx % BS; n = idx / BS; }
      Bs[n][i] = load_op(Bb, (long long)i * lb.sl + (long long)(n0 + n) * lb.sd);
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < KC; ++k) {
      float a[TM], b[TM];
#pragma unroll
      for (int m = 0; m < TM; ++m) a[m] = As[k][ty * TM + m];
#pragma unroll
      for (int m = 0; m < TM; ++m) b[m] = Bs[k][tx * TM + m];
#pragma unroll
      for (int x = 0; x < TM; ++x)
#pragma unroll
        for (int y = 0; y < TM; ++y) acc[x][y] = fmaf(a[x], b[y], acc[x][y]);
    }
    __syncthreads();
  }
  long long base, si, sj;
  tile_address(vl, p, r, c, blk, base, si, sj);
  TV* out = vals + (long long)bh * vl.bh_stride + base;
#pragma unroll
  for (int x = 0; x < TM; ++x)
#pragma unroll
    for (int y = 0; y < TM; ++y) out[(long long)(ty * TM + x) * si + (long long)(tx * TM + y) * sj] = from_f32<TV>(acc[x][y]);
}

// ------------------------------------------------------------------------------ SpMM
// TRANS == false: one CTA per (block row r, bh):  out[r*bs+i, :] = sum_{c in row r} vals_{r,c}(i,j) * Bop[c*bs+j, :]
// TRANS == true : one CTA per (block col c, bh):  out[c*bs+j, :] = sum_{r in col c} vals_{r,c}(i,j) * Bop[r*bs+i, :]
// Output columns are produced 32 at a time (grid.z chunks of the head dimension).
template <typename TV, typename TO, int TM, bool TRANS>
__global__ void __launch_bounds__(256) spmm_kernel(const TV* __restrict__ vals, ValueLayout vl, const TO* __restrict__ Bop,
                                                   OperandLayout lb, TO* __restrict__ out, OperandLayout lo, Pattern p) {
  constexpr int BS = TM * 16;
  constexpr int TN = 2;                 // 16 thread columns x 2 = 32 output columns per chunk
  __shared__ float As[BS][BS + 1];      // As[k][m]
  __shared__ float Bs[BS][32 + 1];      // Bs[k][n]
  const int line = blockIdx.x, bh = blockIdx.y, n0 = blockIdx.z * 32;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int beg = TRANS ? p.col_ptr[line] : p.row_ptr[line];
  const int end = TRANS ? p.col_ptr[line + 1] : p.row_ptr[line + 1];
  const TV* vb = vals + (long long)bh * vl.bh_stride;
  const TO* Bb = Bop + (long long)bh * lb.bh_stride;
  float acc[TM][TN];
#pragma unroll
  for (int a = 0; a < TM; ++a)
#pragma unroll
    for (int b = 0; b < TN; ++b) acc[a][b] = 0.f;

  for (int e = beg; e < end; ++e) {
    int r, c, blk;
    if (TRANS) { c = line; r = p.row_idx[e]; blk = p.csc_pos[e]; } else { r = line; blk = e; c = p.col_idx[e]; }
    long long base, si, sj;
    tile_address(vl, p, r, c, blk, base, si, sj);
    const TV* tile = vb + base;
    for (int idx = tid; idx < BS * BS; idx += 256) {
      int i, j;
      if (sj == 1) { j = idx % BS; i = idx / BS; } else { i = idx % BS; j = idx / BS; }
      const float v = to_f32(tile[(long long)i * si + (long long)j * sj]);
      if (TRANS) As[i][j] = v; else As[j][i] = v;
    }
    const int krow0 = (TRANS ? r : c) * BS;
    for (int idx = tid; idx < BS * 32; idx += 256) {
      int k, n;
      if (lb.sd == 1) { n = idx % 32; k = idx / 32; } else { k = idx % BS; n = idx / BS; }
      Bs[k][n] = to_f32(Bb[(long long)(krow0 + k) * lb.sl + (long long)(n0 + n) * lb.sd]);
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < BS; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int m = 0; m < TM; ++m) a[m] = As[k][ty * TM + m];
#pragma unroll
      for (int n = 0; n < TN; ++n) b[n] = Bs[k][tx * TN + n];
#pragma unroll
      for (int x = 0; x < TM; ++x)
#pragma unroll
        for (int y = 0; y < TN; ++y) acc[x][y] = fmaf(a[x], b[y], acc[x][y]);
    }
    __syncthreads();
  }
  TO* ob = out + (long long)bh * lo.bh_stride + (long long)line * BS * lo.sl;
#pragma unroll
  for (int x = 0; x < TM; ++x)
#pragma unroll
    for (int y = 0; y < TN; ++y)
      ob[(long long)(ty * TM + x) * lo.sl + (long long)(n0 + tx * TN + y) * lo.sd] = from_f32<TO>(acc[x][y]);
}

// ------------------------------------------------------------------------------ row softmax
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per element row.  Values of a row: for each block k of block row r, bs consecutive
// elements at tile base + ii*si (sj == 1 layouts only).
//   v = S*scale - keypad[col];  m = max(floor, max v);  Z = sum exp(v-m) + (L-n_i) exp(-m);  P = exp(v-m)/Z
template <typename TP>
__global__ void __launch_bounds__(256) softmax_fwd_rows_kernel(const float* S, ValueLayout vin,   // S may alias P
                                                               TP* P, ValueLayout vout, Pattern p, int BH,
                                                               int L, float scale, const float* __restrict__ keypad,
                                                               float floor_v) {
  const long long row_g = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row_g >= (long long)BH * L) return;
  const int lane = threadIdx.x & 31;
  const int bh = (int)(row_g / L), row = (int)(row_g % L);
  const int bs = p.bs, r = row / bs, ii = row % bs;
  const int rp = p.row_ptr[r], nblk = p.row_ptr[r + 1] - rp;
  const float* Sb = S + (long long)bh * vin.bh_stride;
  TP* Pb = P + (long long)bh * vout.bh_stride;
  const float* kp = keypad ? keypad + (long long)bh * L : nullptr;

  float m = floor_v;
  for (int k = 0; k < nblk; ++k) {
    const int blk = rp + k, c = p.col_idx[blk];
    long long base, si, sj;
    tile_address(vin, p, r, c, blk, base, si, sj);
    const float* src = Sb + base + (long long)ii * si;
    for (int j = lane; j < bs; j += 32) {
      float v = src[j] * scale;
      if (kp) v -= kp[c * bs + j];
      m = fmaxf(m, v);
    }
  }
  m = warp_max(m);
  float sum = 0.f;
  for (int k = 0; k < nblk; ++k) {
    const int blk = rp + k, c = p.col_idx[blk];
    long long base, si, sj;
    tile_address(vin, p, r, c, blk, base, si, sj);
    const float* src = Sb + base + (long long)ii * si;
    for (int j = lane; j < bs; j += 32) {
      float v = src[j] * scale;
      if (kp) v -= kp[c * bs + j];
      sum += expf(v - m);
    }
  }
  sum = warp_sum(sum);
  sum += (float)(L - nblk * bs) * expf(-m);
  const float inv = 1.0f / sum;
  for (int k = 0; k < nblk; ++k) {
    const int blk = rp + k, c = p.col_idx[blk];
    long long base, si, sj, obase, osi, osj;
    tile_address(vin, p, r, c, blk, base, si, sj);
    tile_address(vout, p, r, c, blk, obase, osi, osj);
    const float* src = Sb + base + (long long)ii * si;
    TP* dst = Pb + obase + (long long)ii * osi;
    for (int j = lane; j < bs; j += 32) {
      float v = src[j] * scale;
      if (kp) v -= kp[c * bs + j];
      const float pv = (inv == 0.f) ? 0.f : expf(v - m) * inv;
      dst[j] = from_f32<TP>(pv);
    }
  }
}

//   t = dP*P ; s = sum_row t ; dS = (t - P*s) * scale
template <typename TP>
__global__ void __launch_bounds__(256) softmax_bwd_rows_kernel(const float* __restrict__ dP, ValueLayout vdp,
                                                               const TP* __restrict__ P, ValueLayout vp,
                                                               TP* __restrict__ dS, ValueLayout vds, Pattern p, int BH,
                                                               int L, float scale) {
  const long long row_g = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row_g >= (long long)BH * L) return;
  const int lane = threadIdx.x & 31;
  const int bh = (int)(row_g / L), row = (int)(row_g % L);
  const int bs = p.bs, r = row / bs, ii = row % bs;
  const int rp = p.row_ptr[r], nblk = p.row_ptr[r + 1] - rp;
  const float* dPb = dP + (long long)bh * vdp.bh_stride;
  const TP* Pb = P + (long long)bh * vp.bh_stride;
  TP* dSb = dS + (long long)bh * vds.bh_stride;
  float s = 0.f;
  for (int k = 0; k < nblk; ++k) {
    const int blk = rp + k, c = p.col_idx[blk];
    long long b1, s1, t1, b2, s2, t2;
    tile_address(vdp, p, r, c, blk, b1, s1, t1);
    tile_address(vp, p, r, c, blk, b2, s2, t2);
    const float* a = dPb + b1 + (long long)ii * s1;
    const TP* q = Pb + b2 + (long long)ii * s2;
    for (int j = lane; j < bs; j += 32) s += a[j] * to_f32(q[j]);
  }
  s = warp_sum(s);
  for (int k = 0; k < nblk; ++k) {
    const int blk = rp + k, c = p.col_idx[blk];
    long long b1, s1, t1, b2, s2, t2, b3, s3, t3;
    tile_address(vdp, p, r, c, blk, b1, s1, t1);
    tile_address(vp, p, r, c, blk, b2, s2, t2);
    tile_address(vds, p, r, c, blk, b3, s3, t3);
    const float* a = dPb + b1 + (long long)ii * s1;
    const TP* q = Pb + b2 + (long long)ii * s2;
    TP* o = dSb + b3 + (long long)ii * s3;
    for (int j = lane; j < bs; j += 32) {
      const float pv = to_f32(q[j]);
      o[j] = from_f32<TP>((a[j] * pv - pv * s) * scale);
    }
  }
}

// ---- rows of 32- or 64-wide blocks in 16-byte pieces: sixteen lanes per element row
// Lane hl of a row's sixteen owns four consecutive values of one block per step: step `it` covers block it (64-wide)
// or blocks 2 it and 2 it + 1 (32-wide).  Rows of at most 16 * 4 * ROW_STEPS_* values are read once into registers, all
// loads of a lane issued before the first use, and written once; longer rows make two passes.  Needs 16-byte
// aligned value arrays (8 bytes for bf16), which the launchers check; same formulas as the kernels above, other
// summation order.
constexpr int ROW_STEPS_FWD = 8, ROW_STEPS_BWD = 4;   // measured: deeper caches cost occupancy in the backward

template <int BS>
struct RowPiece {
  const int nblk, hl;
  __device__ __forceinline__ RowPiece(int nblk_, int hl_) : nblk(nblk_), hl(hl_) {}
  __device__ __forceinline__ int steps() const { return BS == 64 ? nblk : (nblk + 1) >> 1; }
  __device__ __forceinline__ int block(int it) const { return BS == 64 ? it : 2 * it + (hl >> 3); }
  __device__ __forceinline__ bool valid(int it) const { return block(it) < nblk; }
  __device__ __forceinline__ int col() const { return BS == 64 ? hl * 4 : (hl & 7) * 4; }
};

// Start of element row ii's values inside one (b,h) matrix and the distance between its slices of consecutive blocks.
__device__ __forceinline__ void row_base(const ValueLayout& vl, int bs, int rp, int nblk, int ii, long long& base,
                                         int& kstride) {
  if (vl.mode == VAL_ELEMCSR) {
    base = (long long)rp * bs * bs + (long long)ii * nblk * bs;
    kstride = bs;
  } else {
    base = (long long)rp * bs * bs + (long long)ii * bs;
    kstride = bs * bs;
  }
}

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 w = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&w.x);
  const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&w.y);
  const float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 w;
  w.x = *reinterpret_cast<const unsigned*>(&lo);
  w.y = *reinterpret_cast<const unsigned*>(&hi);
  *reinterpret_cast<uint2*>(p) = w;
}
__device__ __forceinline__ float half_max(unsigned mask, float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(mask, v, o));
  return v;
}
__device__ __forceinline__ float half_sum(unsigned mask, float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(mask, v, o);
  return v;
}
// The forward works in base-2 units (one multiply and one ex2 per value instead of a full-range expf; the issue
// slots were the kernel's second limit after the bytes in flight): v2 = S * (scale * log2 e) - keypad * log2 e.
constexpr float ROW_LOG2E = 1.4426950408889634f;
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float4 scaled(float4 v, float scale2, const float* kp) {
  v.x *= scale2, v.y *= scale2, v.z *= scale2, v.w *= scale2;
  if (kp) {
    const float4 k = load4(kp);
    v.x = fmaf(-k.x, ROW_LOG2E, v.x), v.y = fmaf(-k.y, ROW_LOG2E, v.y);
    v.z = fmaf(-k.z, ROW_LOG2E, v.z), v.w = fmaf(-k.w, ROW_LOG2E, v.w);
  }
  return v;
}
__device__ __forceinline__ float max4(float m, float4 v) { return fmaxf(fmaxf(m, fmaxf(v.x, v.y)), fmaxf(v.z, v.w)); }
__device__ __forceinline__ float4 exp4(float4 v, float m) {
  return make_float4(ex2f(v.x - m), ex2f(v.y - m), ex2f(v.z - m), ex2f(v.w - m));
}

template <typename TP, int BS>
__global__ void __launch_bounds__(256, 4) softmax_fwd_rows16_kernel(const float* S, ValueLayout vin,   // S may alias P
                                                                    TP* P, ValueLayout vout, Pattern p, int BH, int L,
                                                                    float scale, const float* __restrict__ keypad,
                                                                    float floor_v) {
  const unsigned ctas_per_bh = (unsigned)L >> 4;   // L is a multiple of the block size
  const int bh = (int)(blockIdx.x / ctas_per_bh), row = (int)(blockIdx.x % ctas_per_bh) * 16 + (threadIdx.x >> 4);
  const unsigned hmask = 0xffffu << (threadIdx.x & 16);
  const int r = row / BS, ii = row % BS;
  const int rp = p.row_ptr[r], nblk = p.row_ptr[r + 1] - rp;
  const RowPiece<BS> pc(nblk, threadIdx.x & 15);
  long long ibase, obase;
  int iks, oks;
  row_base(vin, BS, rp, nblk, ii, ibase, iks);
  row_base(vout, BS, rp, nblk, ii, obase, oks);
  const float* src = S + (long long)bh * vin.bh_stride + ibase + pc.col();
  TP* dst = P + (long long)bh * vout.bh_stride + obase + pc.col();
  const float* kp = keypad ? keypad + (long long)bh * L + pc.col() : nullptr;
  const int nsteps = pc.steps(), nvals = nblk * BS;
  const float scale2 = scale * ROW_LOG2E, floor2 = floor_v * ROW_LOG2E;

  if (nsteps <= ROW_STEPS_FWD) {
    float4 v[ROW_STEPS_FWD];
#pragma unroll
    for (int it = 0; it < ROW_STEPS_FWD; ++it) {
      if (it >= nsteps) break;
      if (pc.valid(it)) v[it] = load4(src + pc.block(it) * iks);
    }
    float m = floor2;
#pragma unroll
    for (int it = 0; it < ROW_STEPS_FWD; ++it) {
      if (it >= nsteps) break;
      if (pc.valid(it)) {
        v[it] = scaled(v[it], scale2, kp ? kp + p.col_idx[rp + pc.block(it)] * BS : nullptr);
        m = max4(m, v[it]);
      }
    }
    m = half_max(hmask, m);
    float sum = 0.f;
#pragma unroll
    for (int it = 0; it < ROW_STEPS_FWD; ++it) {
      if (it >= nsteps) break;
      if (pc.valid(it)) {
        v[it] = exp4(v[it], m);
        sum += (v[it].x + v[it].y) + (v[it].z + v[it].w);
      }
    }
    sum = half_sum(hmask, sum) + (float)(L - nvals) * ex2f(-m);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int it = 0; it < ROW_STEPS_FWD; ++it) {
      if (it >= nsteps) break;
      if (pc.valid(it)) {
        const float4 o = (inv == 0.f) ? make_float4(0.f, 0.f, 0.f, 0.f)
                                      : make_float4(v[it].x * inv, v[it].y * inv, v[it].z * inv, v[it].w * inv);
        store4(dst + pc.block(it) * oks, o);
      }
    }
    return;
  }

  // Longer rows, two passes with the loads of four steps in flight: (1) per lane the running maximum and the sum of
  // exponentials relative to it (rescaled when the maximum rises), joined over the sixteen lanes; (2) P.
  auto value = [&](int it) {
    return scaled(load4(src + pc.block(it) * iks), scale2, kp ? kp + p.col_idx[rp + pc.block(it)] * BS : nullptr);
  };
  float m = floor2, sum = 0.f;
  for (int it0 = 0; it0 < nsteps; it0 += 4) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (it0 + u < nsteps && pc.valid(it0 + u)) v[u] = value(it0 + u);
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (it0 + u < nsteps && pc.valid(it0 + u)) {
        const float vm = max4(m, v[u]);
        if (vm > m) {
          sum *= ex2f(m - vm);
          m = vm;
        }
        const float4 e = exp4(v[u], m);
        sum += (e.x + e.y) + (e.z + e.w);
      }
  }
  const float mrow = half_max(hmask, m);
  sum = half_sum(hmask, sum * ex2f(m - mrow)) + (float)(L - nvals) * ex2f(-mrow);
  const float inv = 1.0f / sum;
  for (int it0 = 0; it0 < nsteps; it0 += 4) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (it0 + u < nsteps && pc.valid(it0 + u)) v[u] = value(it0 + u);
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (it0 + u < nsteps && pc.valid(it0 + u)) {
        const float4 e = exp4(v[u], mrow);
        store4(dst + pc.block(it0 + u) * oks, (inv == 0.f) ? make_float4(0.f, 0.f, 0.f, 0.f)
                                                             : make_float4(e.x * inv, e.y * inv, e.z * inv, e.w * inv));
      }
  }
}

template <typename TP, int BS>
__global__ void __launch_bounds__(256, 4) softmax_bwd_rows16_kernel(const float* __restrict__ dP, ValueLayout vdp,
                                                                    const TP* __restrict__ P, ValueLayout vp,
                                                                    TP* __restrict__ dS, ValueLayout vds, Pattern p,
                                                                    int BH, int L, float scale) {
  const unsigned ctas_per_bh = (unsigned)L >> 4;   // L is a multiple of the block size
  const int bh = (int)(blockIdx.x / ctas_per_bh), row = (int)(blockIdx.x % ctas_per_bh) * 16 + (threadIdx.x >> 4);
  const unsigned hmask = 0xffffu << (threadIdx.x & 16);
  const int r = row / BS, ii = row % BS;
  const int rp = p.row_ptr[r], nblk = p.row_ptr[r + 1] - rp;
  const RowPiece<BS> pc(nblk, threadIdx.x & 15);
  long long b1, b2, b3;
  int k1, k2, k3;
  row_base(vdp, BS, rp, nblk, ii, b1, k1);
  row_base(vp, BS, rp, nblk, ii, b2, k2);
  row_base(vds, BS, rp, nblk, ii, b3, k3);
  const float* pa = dP + (long long)bh * vdp.bh_stride + b1 + pc.col();
  const TP* pq = P + (long long)bh * vp.bh_stride + b2 + pc.col();
  TP* po = dS + (long long)bh * vds.bh_stride + b3 + pc.col();
  const int nsteps = pc.steps();

  if (nsteps <= ROW_STEPS_BWD) {
    float4 a[ROW_STEPS_BWD], q[ROW_STEPS_BWD];
#pragma unroll
    for (int it = 0; it < ROW_STEPS_BWD; ++it) {
      if (it >= nsteps) break;
      if (pc.valid(it)) {
        a[it] = load4(pa + pc.block(it) * k1);
        q[it] = load4(pq + pc.block(it) * k2);
      }
    }
    float s = 0.f;
#pragma unroll
    for (int it = 0; it < ROW_STEPS_BWD; ++it) {
      if (it >= nsteps) break;
      if (pc.valid(it)) {
        a[it].x *= q[it].x, a[it].y *= q[it].y, a[it].z *= q[it].z, a[it].w *= q[it].w;
        s += (a[it].x + a[it].y) + (a[it].z + a[it].w);
      }
    }
    s = half_sum(hmask, s);
#pragma unroll
    for (int it = 0; it < ROW_STEPS_BWD; ++it) {
      if (it >= nsteps) break;
      if (pc.valid(it))
        store4(po + pc.block(it) * k3,
               make_float4((a[it].x - q[it].x * s) * scale, (a[it].y - q[it].y * s) * scale,
                           (a[it].z - q[it].z * s) * scale, (a[it].w - q[it].w * s) * scale));
    }
    return;
  }

  float s = 0.f;
  for (int it = 0; it < nsteps; ++it)
    if (pc.valid(it)) {
      const float4 a = load4(pa + pc.block(it) * k1), q = load4(pq + pc.block(it) * k2);
      s += (a.x * q.x + a.y * q.y) + (a.z * q.z + a.w * q.w);
    }
  s = half_sum(hmask, s);
  for (int it = 0; it < nsteps; ++it)
    if (pc.valid(it)) {
      const float4 a = load4(pa + pc.block(it) * k1), q = load4(pq + pc.block(it) * k2);
      store4(po + pc.block(it) * k3,
             make_float4((a.x * q.x - q.x * s) * scale, (a.y * q.y - q.y * s) * scale, (a.z * q.z - q.z * s) * scale,
                         (a.w * q.w - q.w * s) * scale));
    }
}

// Dense attention stored transposed (value(i,j) at j*L + i).  A CTA owns 32 consecutive query rows (lane = row, so
// that a warp touches 128 consecutive bytes per key) and its DENSE_WARPS warps split the keys; the row statistics
// of the slices meet in shared memory.  Three passes over the CTA's [L x 32] strip (maximum, sum, write), which
// stays in L2 between them.  Semantics as softmax_fwd_rows_kernel at full density (models/attn.cu:9-36).
constexpr int DENSE_WARPS = 8;

__global__ void __launch_bounds__(DENSE_WARPS * 32) softmax_fwd_dense_t_kernel(float* __restrict__ S, int L, float scale,
                                                                               const float* __restrict__ keypad,
                                                                               float floor_v) {
  __shared__ float s_red[DENSE_WARPS][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int i = blockIdx.x * 32 + lane;
  const int bh = blockIdx.y;
  const bool live = i < L;
  float* Sb = S + (long long)bh * L * L + (live ? i : 0);
  const float* kp = keypad ? keypad + (long long)bh * L : nullptr;
  const int per = (L + DENSE_WARPS - 1) / DENSE_WARPS, j0 = w * per, j1 = min(L, j0 + per);
  float m = floor_v;
  if (live) {
#pragma unroll 4
    for (int j = j0; j < j1; ++j) {
      float v = Sb[(long long)j * L] * scale;
      if (kp) v -= kp[j];
      m = fmaxf(m, v);
    }
  }
  s_red[w][lane] = m;
  __syncthreads();
#pragma unroll
  for (int k = 0; k < DENSE_WARPS; ++k) m = fmaxf(m, s_red[k][lane]);
  __syncthreads();
  float sum = 0.f;
  if (live) {
#pragma unroll 4
    for (int j = j0; j < j1; ++j) {
      float v = Sb[(long long)j * L] * scale;
      if (kp) v -= kp[j];
      sum += expf(v - m);
    }
  }
  s_red[w][lane] = sum;
  __syncthreads();
  sum = 0.f;
#pragma unroll
  for (int k = 0; k < DENSE_WARPS; ++k) sum += s_red[k][lane];      // slices added in slice order
  const float inv = 1.0f / sum;
  if (live) {
#pragma unroll 4
    for (int j = j0; j < j1; ++j) {
      float v = Sb[(long long)j * L] * scale;
      if (kp) v -= kp[j];
      Sb[(long long)j * L] = expf(v - m) * inv;
    }
  }
}

// dS = (dP . P - P rowsum(dP . P)) scale (models/attn.cu:67-87), same decomposition.
__global__ void __launch_bounds__(DENSE_WARPS * 32) softmax_bwd_dense_t_kernel(const float* __restrict__ dP,
                                                                               const float* __restrict__ P,
                                                                               float* __restrict__ dS, int L, float scale) {
  __shared__ float s_red[DENSE_WARPS][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int i = blockIdx.x * 32 + lane;
  const int bh = blockIdx.y;
  const bool live = i < L;
  const long long o = (long long)bh * L * L + (live ? i : 0);
  const int per = (L + DENSE_WARPS - 1) / DENSE_WARPS, j0 = w * per, j1 = min(L, j0 + per);
  float s = 0.f;
  if (live) {
#pragma unroll 4
    for (int j = j0; j < j1; ++j) s += dP[o + (long long)j * L] * P[o + (long long)j * L];
  }
  s_red[w][lane] = s;
  __syncthreads();
  s = 0.f;
#pragma unroll
  for (int k = 0; k < DENSE_WARPS; ++k) s += s_red[k][lane];
  if (live) {
#pragma unroll 4
    for (int j = j0; j < j1; ++j) {
      const float pv = P[o + (long long)j * L];
      dS[o + (long long)j * L] = (dP[o + (long long)j * L] * pv - pv * s) * scale;
    }
  }
}

}  // namespace

// ================================================================================ launchers
template <typename TI, typename TV>
static int sddmm_dispatch(const void* A, OperandLayout la, const void* B, OperandLayout lb, void* vals, ValueLayout vl,
                          Pattern p, int nnzb, int BH, int d, cudaStream_t st) {
  dim3 grid(nnzb, BH);
  if (p.bs == 64)
    sddmm_kernel<TI, TV, 4><<<grid, 256, 0, st>>>((const TI*)A, la, (const TI*)B, lb, (TV*)vals, vl, p, d);
  else if (p.bs == 32)
    sddmm_kernel<TI, TV, 2><<<grid, 256, 0, st>>>((const TI*)A, la, (const TI*)B, lb, (TV*)vals, vl, p, d);
  else
    return SPION_ERR_UNSUPPORTED;
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}

int simt_sddmm(int dtype_in, int dtype_val, const void* A, OperandLayout la, const void* B, OperandLayout lb, void* vals,
               ValueLayout vl, Pattern p, int nnzb, int BH, int d, cudaStream_t st) {
  if (d % KC != 0 || BH > 65535) return SPION_ERR_UNSUPPORTED;
  if (nnzb == 0) return SPION_OK;
  if (dtype_in == SPION_F32 && dtype_val == SPION_F32)
    return sddmm_dispatch<float, float>(A, la, B, lb, vals, vl, p, nnzb, BH, d, st);
  if (dtype_in == SPION_BF16 && dtype_val == SPION_F32)
    return sddmm_dispatch<__nv_bfloat16, float>(A, la, B, lb, vals, vl, p, nnzb, BH, d, st);
  return SPION_ERR_UNSUPPORTED;
}

template <typename TV, typename TO>
static int spmm_dispatch(bool trans, const void* vals, ValueLayout vl, const void* Bop, OperandLayout lb, void* out,
                         OperandLayout lo, Pattern p, int BH, int d, cudaStream_t st) {
  dim3 grid(p.nb, BH, d / 32);
#define SPION_SPMM(TMv, TR) \
  spmm_kernel<TV, TO, TMv, TR><<<grid, 256, 0, st>>>((const TV*)vals, vl, (const TO*)Bop, lb, (TO*)out, lo, p)
  if (p.bs == 64) { if (trans) SPION_SPMM(4, true); else SPION_SPMM(4, false); }
  else if (p.bs == 32) { if (trans) SPION_SPMM(2, true); else SPION_SPMM(2, false); }
  else return SPION_ERR_UNSUPPORTED;
#undef SPION_SPMM
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}

int simt_spmm(int dtype_val, int dtype_op, bool trans, const void* vals, ValueLayout vl, const void* Bop,
              OperandLayout lb, void* out, OperandLayout lo, Pattern p, int BH, int d, cudaStream_t st) {
  if (d % 32 != 0 || BH > 65535) return SPION_ERR_UNSUPPORTED;
  if (dtype_val == SPION_F32 && dtype_op == SPION_F32)
    return spmm_dispatch<float, float>(trans, vals, vl, Bop, lb, out, lo, p, BH, d, st);
  if (dtype_val == SPION_BF16 && dtype_op == SPION_BF16)
    return spmm_dispatch<__nv_bfloat16, __nv_bfloat16>(trans, vals, vl, Bop, lb, out, lo, p, BH, d, st);
  return SPION_ERR_UNSUPPORTED;
}

static bool aligned_to(const void* ptr, size_t n) { return ((uintptr_t)ptr & (n - 1)) == 0; }
static bool piece_layout(const ValueLayout& vl) { return vl.mode != VAL_DENSE_T && vl.bh_stride % 4 == 0; }

template <int BS>
static void softmax_fwd_rows16_launch(int dtype_out, const float* S, ValueLayout vin, void* P, ValueLayout vout, Pattern p,
                                      int BH, int L, float scale, const float* keypad, float floor_v, cudaStream_t st) {
  const unsigned grid = (unsigned)BH * (unsigned)(L / 16);
  if (dtype_out == SPION_F32)
    softmax_fwd_rows16_kernel<float, BS><<<grid, 256, 0, st>>>(S, vin, (float*)P, vout, p, BH, L, scale, keypad,
                                                               floor_v);
  else
    softmax_fwd_rows16_kernel<__nv_bfloat16, BS><<<grid, 256, 0, st>>>(S, vin, (__nv_bfloat16*)P, vout, p, BH, L,
                                                                       scale, keypad, floor_v);
}

int softmax_fwd_rows(int dtype_out, const float* S, ValueLayout vin, void* P, ValueLayout vout, Pattern p, int BH, int L,
                     float scale, const float* keypad, float floor_v, cudaStream_t st) {
  const long long rows = (long long)BH * L;
  const bool pieces = (p.bs == 32 || p.bs == 64) && piece_layout(vin) && piece_layout(vout) && aligned_to(S, 16) &&
                      aligned_to(P, dtype_out == SPION_F32 ? 16 : 8) && (!keypad || aligned_to(keypad, 16));
  if (pieces && p.bs == 64) {
    softmax_fwd_rows16_launch<64>(dtype_out, S, vin, P, vout, p, BH, L, scale, keypad, floor_v, st);
  } else if (pieces) {
    softmax_fwd_rows16_launch<32>(dtype_out, S, vin, P, vout, p, BH, L, scale, keypad, floor_v, st);
  } else {
    const unsigned grid = (unsigned)((rows + 7) / 8);
    if (dtype_out == SPION_F32)
      softmax_fwd_rows_kernel<float><<<grid, 256, 0, st>>>(S, vin, (float*)P, vout, p, BH, L, scale, keypad, floor_v);
    else
      softmax_fwd_rows_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(S, vin, (__nv_bfloat16*)P, vout, p, BH, L, scale,
                                                                   keypad, floor_v);
  }
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}

template <int BS>
static void softmax_bwd_rows16_launch(int dtype_p, const float* dP, ValueLayout vdp, const void* P, ValueLayout vp,
                                      void* dS, ValueLayout vds, Pattern p, int BH, int L, float scale, cudaStream_t st) {
  const unsigned grid = (unsigned)BH * (unsigned)(L / 16);
  if (dtype_p == SPION_F32)
    softmax_bwd_rows16_kernel<float, BS><<<grid, 256, 0, st>>>(dP, vdp, (const float*)P, vp, (float*)dS, vds, p, BH, L,
                                                               scale);
  else
    softmax_bwd_rows16_kernel<__nv_bfloat16, BS><<<grid, 256, 0, st>>>(dP, vdp, (const __nv_bfloat16*)P, vp,
                                                                       (__nv_bfloat16*)dS, vds, p, BH, L, scale);
}

int softmax_bwd_rows(int dtype_p, const float* dP, ValueLayout vdp, const void* P, ValueLayout vp, void* dS,
                     ValueLayout vds, Pattern p, int BH, int L, float scale, cudaStream_t st) {
  const long long rows = (long long)BH * L;
  const size_t pal = dtype_p == SPION_F32 ? 16 : 8;
  const bool pieces = (p.bs == 32 || p.bs == 64) && piece_layout(vdp) && piece_layout(vp) && piece_layout(vds) &&
                      aligned_to(dP, 16) && aligned_to(P, pal) && aligned_to(dS, pal);
  if (pieces && p.bs == 64) {
    softmax_bwd_rows16_launch<64>(dtype_p, dP, vdp, P, vp, dS, vds, p, BH, L, scale, st);
  } else if (pieces) {
    softmax_bwd_rows16_launch<32>(dtype_p, dP, vdp, P, vp, dS, vds, p, BH, L, scale, st);
  } else {
    const unsigned grid = (unsigned)((rows + 7) / 8);
    if (dtype_p == SPION_F32)
      softmax_bwd_rows_kernel<float><<<grid, 256, 0, st>>>(dP, vdp, (const float*)P, vp, (float*)dS, vds, p, BH, L,
                                                           scale);
    else
      softmax_bwd_rows_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(dP, vdp, (const __nv_bfloat16*)P, vp,
                                                                   (__nv_bfloat16*)dS, vds, p, BH, L, scale);
  }
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}

int softmax_fwd_dense_t(float* S, int BH, int L, float scale, const float* keypad, float floor_v, cudaStream_t st) {
  if (BH > 65535) return SPION_ERR_UNSUPPORTED;
  softmax_fwd_dense_t_kernel<<<dim3((L + 31) / 32, BH), DENSE_WARPS * 32, 0, st>>>(S, L, scale, keypad, floor_v);
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}

int softmax_bwd_dense_t(const float* dP, const float* P, float* dS, int BH, int L, float scale, cudaStream_t st) {
  if (BH > 65535) return SPION_ERR_UNSUPPORTED;
  softmax_bwd_dense_t_kernel<<<dim3((L + 31) / 32, BH), DENSE_WARPS * 32, 0, st>>>(dP, P, dS, L, scale);
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}
