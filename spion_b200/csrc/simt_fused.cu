// Fused fp32 (CUDA-core) kernels of the block-sparse attention path: the fp32 entry points keep the
// 1e-4 max-abs parity bound, which rules out TF32 / BF16 tensor-core inputs, so these run on the FMA
// pipes; fusing removes the S / dP round trips through memory that the staged kernels of
// simt_attn.cu make.
//
//   fused_fwd_kernel   per block row:  S = Q K^T -> sparse row softmax -> P (written once) -> O = P V
//                      replaces models/block_attn.cu:453-487 (cusparseSDDMM, scale_softmax_kernel, cusparseSpMM)
//   fused_bwd_row      per block row:  dP = dO V^T -> dS = (dP.P - P rowsum(dP.P)) scale -> dQ = dS K
//                      replaces models/block_attn.cu:498-516
//   fused_bwd_col      per block col:  dK = dS^T Q, dV = P^T dO      (models/block_attn.cu:526-536)
//
// A row of blocks can be arbitrarily long, so nothing but one tile is ever held on chip: pass 1 of the
// forward kernel leaves the scaled scores in the P tiles themselves (global memory, normally still in
// L2 when they are read back) while it accumulates the row maximum and denominator on line; pass 2
// reads them back, writes the probabilities over them and feeds the second product.  The backward
// row kernel does the same with dP in the dS tiles.
//
// Thread layout: a bs x bs tile is computed by (bs/4)^2 threads with 4x4 micro-tiles (rows
// contiguous, columns interleaved by bs/4 so that shared-memory reads of the second operand are
// conflict-free); a CTA of 256 threads therefore works on 256/(bs/4)^2 consecutive (b,h) matrices of
// the same block row: they share the mask, so the CTA runs in lock step.
//
// Layouts: operands through (row, column) strides, value tiles through tile_address(); only
// layouts whose tile rows are contiguous (element CSR, block tiles) are accepted.
#include "common.cuh"

namespace {

template <int BS, int D>
struct Cfg {
  static constexpr int TX = BS / 4;            // threads along a tile row
  static constexpr int NT = TX * TX;           // threads per (b,h) problem
  static constexpr int G = 256 / NT;           // problems per CTA
  static constexpr int TN = D / TX;            // output columns per thread in the bs x d products
  static constexpr int SA = D + 4;             // shared-memory row stride of a [bs x d] operand tile
  static constexpr int SP = BS + 4;            // ... of a [bs x bs] value tile
  static_assert(TN == 2 || TN == 4 || TN == 8, "unsupported shape");
};

// column of the thread's y-th output in a bs x d product: groups of 4 (or 2) contiguous columns
template <int BS, int D>
__device__ __forceinline__ int out_col(int tx, int y) {
  using C = Cfg<BS, D>;
  if (C::TN == 2) return tx * 2 + y;
  return (y >> 2) * (C::TX * 4) + tx * 4 + (y & 3);
}

template <int TN>
__device__ __forceinline__ void load_vec(const float* row, int tx, int TX, float (&b)[TN]) {
  if (TN == 2) {
    const float2 v = *reinterpret_cast<const float2*>(row + tx * 2);
    b[0] = v.x; b[1] = v.y;
  } else {
#pragma unroll
    for (int g4 = 0; g4 < TN / 4; ++g4) {
      const float4 v = *reinterpret_cast<const float4*>(row + g4 * TX * 4 + tx * 4);
      b[4 * g4] = v.x; b[4 * g4 + 1] = v.y; b[4 * g4 + 2] = v.z; b[4 * g4 + 3] = v.w;
    }
  }
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Start the asynchronous copy of a [ROWS x COLS] tile (element (i, n) at src + i*s_row + n*s_col) into
// shared memory, row-major with the given stride, by the NT threads of one problem.  The caller
// commits the group, waits for it and synchronises before the tile is read.
template <int ROWS, int COLS, int NT>
__device__ __forceinline__ void load_tile(float* dst, int stride, const float* __restrict__ src, long long s_row,
                                          long long s_col, int t) {
  if (s_col == 1 && (s_row & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
#pragma unroll
    for (int idx = t; idx < ROWS * COLS / 4; idx += NT) {
      const int row = idx / (COLS / 4), c4 = idx % (COLS / 4);
      cp_async16(dst + row * stride + c4 * 4, src + (long long)row * s_row + c4 * 4);
    }
  } else if (s_col == 1) {
    for (int idx = t; idx < ROWS * COLS; idx += NT) {
      const int row = idx / COLS, col = idx % COLS;
      cp_async4(dst + row * stride + col, src + (long long)row * s_row + col);
    }
  } else {
    for (int idx = t; idx < ROWS * COLS; idx += NT) {
      const int row = idx % ROWS, col = idx / ROWS;
      cp_async4(dst + row * stride + col, src + (long long)row * s_row + (long long)col * s_col);
    }
  }
}

// acc[x][y] += sum_n A[ty*4+x][n] * B[tx + y*TX][n]   (both tiles [bs x d] in shared memory)
template <int BS, int D>
__device__ __forceinline__ void tile_abt(const float* As, const float* Bs, int ty, int tx, float (&acc)[4][4]) {
  using C = Cfg<BS, D>;
#pragma unroll 2
  for (int n = 0; n < D; n += 4) {
    float4 a[4], b[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) a[x] = *reinterpret_cast<const float4*>(As + (ty * 4 + x) * C::SA + n);
#pragma unroll
    for (int y = 0; y < 4; ++y) b[y] = *reinterpret_cast<const float4*>(Bs + (tx + y * C::TX) * C::SA + n);
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) {
        acc[x][y] = fmaf(a[x].x, b[y].x, acc[x][y]);
        acc[x][y] = fmaf(a[x].y, b[y].y, acc[x][y]);
        acc[x][y] = fmaf(a[x].z, b[y].z, acc[x][y]);
        acc[x][y] = fmaf(a[x].w, b[y].w, acc[x][y]);
      }
  }
}

// acc[x][y] += sum_j Vt[ty*4+x][j] * B[j][out_col(y)]   (Vt: [bs x bs] value tile, B: [bs x d])
template <int BS, int D>
__device__ __forceinline__ void tile_ab(const float* Vt, const float* Bs, int ty, int tx,
                                        float (&acc)[4][Cfg<BS, D>::TN]) {
  using C = Cfg<BS, D>;
#pragma unroll 2
  for (int j = 0; j < BS; j += 4) {
    float a[4][4];
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const float4 v = *reinterpret_cast<const float4*>(Vt + (ty * 4 + x) * C::SP + j);
      a[x][0] = v.x; a[x][1] = v.y; a[x][2] = v.z; a[x][3] = v.w;
    }
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      float b[C::TN];
      load_vec<C::TN>(Bs + (j + jj) * C::SA, tx, C::TX, b);
#pragma unroll
      for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < C::TN; ++y) acc[x][y] = fmaf(a[x][jj], b[y], acc[x][y]);
    }
  }
}

// acc[x][y] += sum_i Vt[i][ty*4+x] * B[i][out_col(y)]   (transposed use of the value tile)
template <int BS, int D>
__device__ __forceinline__ void tile_atb(const float* Vt, const float* Bs, int ty, int tx,
                                         float (&acc)[4][Cfg<BS, D>::TN]) {
  using C = Cfg<BS, D>;
#pragma unroll 4
  for (int i = 0; i < BS; ++i) {
    const float4 v = *reinterpret_cast<const float4*>(Vt + i * C::SP + ty * 4);
    const float a[4] = {v.x, v.y, v.z, v.w};
    float b[C::TN];
    load_vec<C::TN>(Bs + i * C::SA, tx, C::TX, b);
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < C::TN; ++y) acc[x][y] = fmaf(a[x], b[y], acc[x][y]);
  }
}

template <int TX>
__device__ __forceinline__ float group_max(float v) {
#pragma unroll
  for (int o = TX / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int TX>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = TX / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// store the thread's 4 x TN outputs of a bs x d product
template <int BS, int D>
__device__ __forceinline__ void store_out(float* __restrict__ out, OperandLayout lo, int row0, int ty, int tx,
                                          const float (&acc)[4][Cfg<BS, D>::TN]) {
  using C = Cfg<BS, D>;
#pragma unroll
  for (int x = 0; x < 4; ++x) {
    float* o = out + (long long)(row0 + ty * 4 + x) * lo.sl;
    if (lo.sd == 1 && C::TN >= 4 && (lo.sl & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
#pragma unroll
      for (int g4 = 0; g4 < C::TN / 4; ++g4)
        *reinterpret_cast<float4*>(o + out_col<BS, D>(tx, 4 * g4)) =
            make_float4(acc[x][4 * g4], acc[x][4 * g4 + 1], acc[x][4 * g4 + 2], acc[x][4 * g4 + 3]);
    } else {
#pragma unroll
      for (int y = 0; y < C::TN; ++y) o[(long long)out_col<BS, D>(tx, y) * lo.sd] = acc[x][y];
    }
  }
}

// ------------------------------------------------------------------------------ forward
//   v = S*scale - keypad[col];  m = max(floor, max v);  Z = sum exp(v-m) + (L-n_i) exp(-m);  P = exp(v-m)/Z
// The K (pass 1) and V (pass 2) tiles are double-buffered: the copy of tile k+1 is in flight while
// tile k is used.
template <int BS, int D>
__global__ void __launch_bounds__(256, 3) fused_fwd_kernel(const float* __restrict__ Q, OperandLayout lq,
                                                           const float* __restrict__ K, OperandLayout lk,
                                                           const float* __restrict__ V, OperandLayout lv,
                                                           const float* __restrict__ keypad, float floor_v, float* P,
                                                           ValueLayout vl, float* __restrict__ O, OperandLayout lo,
                                                           Pattern p, int BH, int L, float scale) {
  using C = Cfg<BS, D>;
  constexpr int TILE = BS * C::SA;
  extern __shared__ __align__(16) float smem[];
  const int g = threadIdx.x / C::NT, t = threadIdx.x % C::NT;
  const int ty = t / C::TX, tx = t % C::TX;
  const int r = blockIdx.x;
  const int bh_raw = blockIdx.y * C::G + g;
  const bool active = bh_raw < BH;
  const int bh = active ? bh_raw : BH - 1;                       // idle problems shadow the last one, store nothing
  float* Qs = smem + g * (3 * TILE + BS * C::SP);
  float* Bs = Qs + TILE;                                        // two buffers: K tiles, then V tiles
  float* Ps = Qs + 3 * TILE;

  const int rp = p.row_ptr[r], nblk = p.row_ptr[r + 1] - rp;
  const int* cols = p.col_idx + rp;
  const float* Qb = Q + (long long)bh * lq.bh_stride + (long long)r * BS * lq.sl;
  const float* Kb = K + (long long)bh * lk.bh_stride;
  const float* Vb = V + (long long)bh * lv.bh_stride;
  float* Pb = P + (long long)bh * vl.bh_stride;
  const float* kp = keypad ? keypad + (long long)bh * L : nullptr;

  int c_cur = nblk > 0 ? cols[0] : 0, c_nxt = nblk > 1 ? cols[1] : 0;
  load_tile<BS, D, C::NT>(Qs, C::SA, Qb, lq.sl, lq.sd, t);
  if (nblk > 0) load_tile<BS, D, C::NT>(Bs, C::SA, Kb + (long long)c_cur * BS * lk.sl, lk.sl, lk.sd, t);
  cp_async_commit();

  // ---- pass 1: scores into the P tiles, running maximum and denominator per row
  float m[4], l[4];
#pragma unroll
  for (int x = 0; x < 4; ++x) { m[x] = floor_v; l[x] = 0.f; }
  for (int k = 0; k < nblk; ++k) {
    const int c = c_cur;
    if (k + 1 < nblk)
      load_tile<BS, D, C::NT>(Bs + ((k + 1) & 1) * TILE, C::SA, Kb + (long long)c_nxt * BS * lk.sl, lk.sl, lk.sd, t);
    cp_async_commit();
    c_cur = c_nxt;
    c_nxt = k + 2 < nblk ? cols[k + 2] : 0;
    cp_async_wait<1>();
    __syncthreads();                                             // tile k (and Q) have landed
    float acc[4][4];
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) acc[x][y] = 0.f;
    tile_abt<BS, D>(Qs, Bs + (k & 1) * TILE, ty, tx, acc);
    long long base, si, sj;
    tile_address(vl, p, r, c, rp + k, base, si, sj);
    float* tile = Pb + base;
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      float mx = -INFINITY;
#pragma unroll
      for (int y = 0; y < 4; ++y) {
        const int j = tx + y * C::TX;
        float v = acc[x][y] * scale;
        if (kp) v -= kp[c * BS + j];
        acc[x][y] = v;
        mx = fmaxf(mx, v);
        if (active) tile[(long long)(ty * 4 + x) * si + j] = v;
      }
      mx = group_max<C::TX>(mx);
      const float m_new = fmaxf(m[x], mx);
      float s = 0.f;
#pragma unroll
      for (int y = 0; y < 4; ++y) s += __expf(acc[x][y] - m_new);
      s = group_sum<C::TX>(s);
      l[x] = l[x] * __expf(m[x] - m_new) + s;
      m[x] = m_new;
    }
    __syncthreads();                                             // buffer k&1 may be refilled
  }
  float inv[4];
#pragma unroll
  for (int x = 0; x < 4; ++x) {
    const float z = l[x] + (float)(L - nblk * BS) * __expf(-m[x]);
    inv[x] = 1.0f / z;
  }

  // ---- pass 2: probabilities over the scores, O = P V
  float o[4][C::TN];
#pragma unroll
  for (int x = 0; x < 4; ++x)
#pragma unroll
    for (int y = 0; y < C::TN; ++y) o[x][y] = 0.f;
  c_cur = nblk > 0 ? cols[0] : 0;
  c_nxt = nblk > 1 ? cols[1] : 0;
  if (nblk > 0) load_tile<BS, D, C::NT>(Bs, C::SA, Vb + (long long)c_cur * BS * lv.sl, lv.sl, lv.sd, t);
  cp_async_commit();
  float sc[4][4];                                                // scores of the tile about to be used
  auto fetch_scores = [&](int k, int c) {
    long long base, si, sj;
    tile_address(vl, p, r, c, rp + k, base, si, sj);
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) sc[x][y] = Pb[base + (long long)(ty * 4 + x) * si + tx + y * C::TX];
  };
  if (nblk > 0) fetch_scores(0, c_cur);
  for (int k = 0; k < nblk; ++k) {
    const int c = c_cur;
    if (k + 1 < nblk)
      load_tile<BS, D, C::NT>(Bs + ((k + 1) & 1) * TILE, C::SA, Vb + (long long)c_nxt * BS * lv.sl, lv.sl, lv.sd, t);
    cp_async_commit();
    long long base, si, sj;
    tile_address(vl, p, r, c, rp + k, base, si, sj);
    float* tile = Pb + base;
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) {
        const int j = tx + y * C::TX;
        const float pv = (inv[x] == 0.f) ? 0.f : __expf(sc[x][y] - m[x]) * inv[x];
        if (active) tile[(long long)(ty * 4 + x) * si + j] = pv;
        Ps[(ty * 4 + x) * C::SP + j] = pv;
      }
    if (k + 1 < nblk) fetch_scores(k + 1, c_nxt);                // in flight during the product below
    c_cur = c_nxt;
    c_nxt = k + 2 < nblk ? cols[k + 2] : 0;
    cp_async_wait<1>();
    __syncthreads();                                             // V tile k has landed, Ps is complete
    tile_ab<BS, D>(Ps, Bs + (k & 1) * TILE, ty, tx, o);
    __syncthreads();                                             // Ps and buffer k&1 may be overwritten
  }
  cp_async_wait<0>();
  if (active) store_out<BS, D>(O + (long long)bh * lo.bh_stride, lo, r * BS, ty, tx, o);
}

// ------------------------------------------------------------------------------ backward, row side
//   t = dP.P ; s = rowsum(t) ; dS = (t - P s) scale ; dQ = dS K     (models/block_attn.cu:90-130, :498-516)
template <int BS, int D>
__global__ void __launch_bounds__(256, 3) fused_bwd_row_kernel(const float* __restrict__ dO, OperandLayout ldo,
                                                               const float* __restrict__ V, OperandLayout lv,
                                                               const float* __restrict__ K, OperandLayout lk,
                                                               const float* __restrict__ P, ValueLayout vp, float* dS,
                                                               ValueLayout vds, float* __restrict__ dQ,
                                                               OperandLayout ldq, Pattern p, int BH, float scale) {
  using C = Cfg<BS, D>;
  constexpr int TILE = BS * C::SA;
  extern __shared__ __align__(16) float smem[];
  const int g = threadIdx.x / C::NT, t = threadIdx.x % C::NT;
  const int ty = t / C::TX, tx = t % C::TX;
  const int r = blockIdx.x;
  const int bh_raw = blockIdx.y * C::G + g;
  const bool active = bh_raw < BH;
  const int bh = active ? bh_raw : BH - 1;
  float* As = smem + g * (3 * TILE + BS * C::SP);               // dO tile
  float* Bs = As + TILE;                                        // two buffers: V tiles, then K tiles
  float* Ss = As + 3 * TILE;                                    // dS tile

  const int rp = p.row_ptr[r], nblk = p.row_ptr[r + 1] - rp;
  const int* cols = p.col_idx + rp;
  const float* Vb = V + (long long)bh * lv.bh_stride;
  const float* Kb = K + (long long)bh * lk.bh_stride;
  const float* Pb = P + (long long)bh * vp.bh_stride;
  float* dSb = dS + (long long)bh * vds.bh_stride;

  int c_cur = nblk > 0 ? cols[0] : 0, c_nxt = nblk > 1 ? cols[1] : 0;
  load_tile<BS, D, C::NT>(As, C::SA, dO + (long long)bh * ldo.bh_stride + (long long)r * BS * ldo.sl, ldo.sl, ldo.sd, t);
  if (nblk > 0) load_tile<BS, D, C::NT>(Bs, C::SA, Vb + (long long)c_cur * BS * lv.sl, lv.sl, lv.sd, t);
  cp_async_commit();

  // ---- pass 1: dP into the dS tiles, row sums of dP.P
  float s[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k = 0; k < nblk; ++k) {
    const int c = c_cur;
    if (k + 1 < nblk)
      load_tile<BS, D, C::NT>(Bs + ((k + 1) & 1) * TILE, C::SA, Vb + (long long)c_nxt * BS * lv.sl, lv.sl, lv.sd, t);
    cp_async_commit();
    c_cur = c_nxt;
    c_nxt = k + 2 < nblk ? cols[k + 2] : 0;
    long long b1, s1, t1, b2, s2, t2;
    tile_address(vp, p, r, c, rp + k, b1, s1, t1);
    tile_address(vds, p, r, c, rp + k, b2, s2, t2);
    float pv[4][4];                                              // requested before the wait: both latencies overlap
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) pv[x][y] = Pb[b1 + (long long)(ty * 4 + x) * s1 + tx + y * C::TX];
    cp_async_wait<1>();
    __syncthreads();
    float acc[4][4];
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) acc[x][y] = 0.f;
    tile_abt<BS, D>(As, Bs + (k & 1) * TILE, ty, tx, acc);
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) {
        s[x] = fmaf(acc[x][y], pv[x][y], s[x]);
        if (active) dSb[b2 + (long long)(ty * 4 + x) * s2 + tx + y * C::TX] = acc[x][y];
      }
    __syncthreads();
  }
#pragma unroll
  for (int x = 0; x < 4; ++x) s[x] = group_sum<C::TX>(s[x]);

  // ---- pass 2: dS over dP, dQ = dS K
  float o[4][C::TN];
#pragma unroll
  for (int x = 0; x < 4; ++x)
#pragma unroll
    for (int y = 0; y < C::TN; ++y) o[x][y] = 0.f;
  c_cur = nblk > 0 ? cols[0] : 0;
  c_nxt = nblk > 1 ? cols[1] : 0;
  if (nblk > 0) load_tile<BS, D, C::NT>(Bs, C::SA, Kb + (long long)c_cur * BS * lk.sl, lk.sl, lk.sd, t);
  cp_async_commit();
  for (int k = 0; k < nblk; ++k) {
    const int c = c_cur;
    if (k + 1 < nblk)
      load_tile<BS, D, C::NT>(Bs + ((k + 1) & 1) * TILE, C::SA, Kb + (long long)c_nxt * BS * lk.sl, lk.sl, lk.sd, t);
    cp_async_commit();
    c_cur = c_nxt;
    c_nxt = k + 2 < nblk ? cols[k + 2] : 0;
    long long b1, s1, t1, b2, s2, t2;
    tile_address(vp, p, r, c, rp + k, b1, s1, t1);
    tile_address(vds, p, r, c, rp + k, b2, s2, t2);
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) {
        const int j = tx + y * C::TX;
        float* e = dSb + b2 + (long long)(ty * 4 + x) * s2 + j;
        const float pv = Pb[b1 + (long long)(ty * 4 + x) * s1 + j];
        const float ds = (*e * pv - pv * s[x]) * scale;
        if (active) *e = ds;
        Ss[(ty * 4 + x) * C::SP + j] = ds;
      }
    cp_async_wait<1>();
    __syncthreads();
    tile_ab<BS, D>(Ss, Bs + (k & 1) * TILE, ty, tx, o);
    __syncthreads();
  }
  cp_async_wait<0>();
  if (active) store_out<BS, D>(dQ + (long long)bh * ldq.bh_stride, ldq, r * BS, ty, tx, o);
}

// Row backward when O is at hand: rowsum(dP.P) = rowsum(dO.O) (delta), so dS of a tile needs nothing
// from the other tiles of its row and one pass suffices.  Two stages per block, V tile (for dP) and
// K tile (for dQ); the copy of one is in flight while the other is used.
template <int BS, int D>
__global__ void __launch_bounds__(256, 3) fused_bwd_row_delta_kernel(const float* __restrict__ dO, OperandLayout ldo,
                                                                     const float* __restrict__ O, OperandLayout lo,
                                                                     const float* __restrict__ V, OperandLayout lv,
                                                                     const float* __restrict__ K, OperandLayout lk,
                                                                     const float* __restrict__ P, ValueLayout vp,
                                                                     float* __restrict__ dS, ValueLayout vds,
                                                                     float* __restrict__ dQ, OperandLayout ldq,
                                                                     Pattern p, int BH, float scale) {
  using C = Cfg<BS, D>;
  constexpr int TILE = BS * C::SA;
  extern __shared__ __align__(16) float smem[];
  const int g = threadIdx.x / C::NT, t = threadIdx.x % C::NT;
  const int ty = t / C::TX, tx = t % C::TX;
  const int r = blockIdx.x;
  const int bh_raw = blockIdx.y * C::G + g;
  const bool active = bh_raw < BH;
  const int bh = active ? bh_raw : BH - 1;
  float* As = smem + g * (3 * TILE + BS * C::SP);               // dO tile
  float* Vs = As + TILE;
  float* Ks = As + 2 * TILE;
  float* Ss = As + 3 * TILE;                                    // dS tile

  const int rp = p.row_ptr[r], nblk = p.row_ptr[r + 1] - rp;
  const int* cols = p.col_idx + rp;
  const float* Vb = V + (long long)bh * lv.bh_stride;
  const float* Kb = K + (long long)bh * lk.bh_stride;
  const float* Pb = P + (long long)bh * vp.bh_stride;
  float* dSb = dS + (long long)bh * vds.bh_stride;

  int c_cur = nblk > 0 ? cols[0] : 0, c_nxt = nblk > 1 ? cols[1] : 0;
  load_tile<BS, D, C::NT>(As, C::SA, dO + (long long)bh * ldo.bh_stride + (long long)r * BS * ldo.sl, ldo.sl, ldo.sd, t);
  if (nblk > 0) load_tile<BS, D, C::NT>(Vs, C::SA, Vb + (long long)c_cur * BS * lv.sl, lv.sl, lv.sd, t);
  cp_async_commit();
  if (nblk > 0) load_tile<BS, D, C::NT>(Ks, C::SA, Kb + (long long)c_cur * BS * lk.sl, lk.sl, lk.sd, t);
  cp_async_commit();

  float delta[4] = {0.f, 0.f, 0.f, 0.f};
  float o[4][C::TN];
#pragma unroll
  for (int x = 0; x < 4; ++x)
#pragma unroll
    for (int y = 0; y < C::TN; ++y) o[x][y] = 0.f;

  for (int k = 0; k < nblk; ++k) {
    const int c = c_cur;
    long long b1, s1, t1, b2, s2, t2;
    tile_address(vp, p, r, c, rp + k, b1, s1, t1);
    tile_address(vds, p, r, c, rp + k, b2, s2, t2);
    float pv[4][4];                                              // requested before the wait: the latencies overlap
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) pv[x][y] = Pb[b1 + (long long)(ty * 4 + x) * s1 + tx + y * C::TX];
    cp_async_wait<1>();
    __syncthreads();                                             // V tile k (and dO) have landed
    if (k == 0) {
      const float* Ob = O + (long long)bh * lo.bh_stride + (long long)(r * BS + ty * 4) * lo.sl;
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        float a = 0.f;
#pragma unroll
        for (int y = 0; y < C::TN; ++y) {
          const int n = out_col<BS, D>(tx, y);
          a = fmaf(As[(ty * 4 + x) * C::SA + n], Ob[(long long)x * lo.sl + (long long)n * lo.sd], a);
        }
        delta[x] = group_sum<C::TX>(a);
      }
    }
    float acc[4][4];
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) acc[x][y] = 0.f;
    tile_abt<BS, D>(As, Vs, ty, tx, acc);
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) {
        const int j = tx + y * C::TX;
        const float ds = pv[x][y] * (acc[x][y] - delta[x]) * scale;
        if (active) dSb[b2 + (long long)(ty * 4 + x) * s2 + j] = ds;
        Ss[(ty * 4 + x) * C::SP + j] = ds;
      }
    __syncthreads();                                             // Ss complete, V buffer free
    if (k + 1 < nblk) load_tile<BS, D, C::NT>(Vs, C::SA, Vb + (long long)c_nxt * BS * lv.sl, lv.sl, lv.sd, t);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();                                             // K tile k has landed
    tile_ab<BS, D>(Ss, Ks, ty, tx, o);
    __syncthreads();                                             // Ss and the K buffer are free
    if (k + 1 < nblk) load_tile<BS, D, C::NT>(Ks, C::SA, Kb + (long long)c_nxt * BS * lk.sl, lk.sl, lk.sd, t);
    cp_async_commit();
    c_cur = c_nxt;
    c_nxt = k + 2 < nblk ? cols[k + 2] : 0;
  }
  cp_async_wait<0>();
  if (active) store_out<BS, D>(dQ + (long long)bh * ldq.bh_stride, ldq, r * BS, ty, tx, o);
}

// ------------------------------------------------------------------------------ backward, column side
//   dK[c] = sum_r dS(r,c)^T Q[r],  dV[c] = sum_r P(r,c)^T dO[r]     (models/block_attn.cu:526-536)
// Two stages per entry of the column: (dS, Q) for dK and (P, dO) for dV; the copy of one stage is in
// flight while the other is used.
template <int BS, int D>
__global__ void __launch_bounds__(256, 3) fused_bwd_col_kernel(const float* __restrict__ dS, ValueLayout vds,
                                                               const float* __restrict__ P, ValueLayout vp,
                                                               const float* __restrict__ Q, OperandLayout lq,
                                                               const float* __restrict__ dO, OperandLayout ldo,
                                                               float* __restrict__ dK, OperandLayout ldk,
                                                               float* __restrict__ dV, OperandLayout ldv, Pattern p,
                                                               int BH) {
  using C = Cfg<BS, D>;
  extern __shared__ __align__(16) float smem[];
  const int g = threadIdx.x / C::NT, t = threadIdx.x % C::NT;
  const int ty = t / C::TX, tx = t % C::TX;
  const int c = blockIdx.x;
  const int bh_raw = blockIdx.y * C::G + g;
  const bool active = bh_raw < BH;
  const int bh = active ? bh_raw : BH - 1;
  float* dSs = smem + g * (2 * BS * C::SA + 2 * BS * C::SP);
  float* Qs = dSs + BS * C::SP;
  float* Ps = Qs + BS * C::SA;
  float* Os = Ps + BS * C::SP;

  const float* dSb = dS + (long long)bh * vds.bh_stride;
  const float* Pb = P + (long long)bh * vp.bh_stride;
  const float* Qb = Q + (long long)bh * lq.bh_stride;
  const float* dOb = dO + (long long)bh * ldo.bh_stride;

  float ak[4][C::TN], av[4][C::TN];
#pragma unroll
  for (int x = 0; x < 4; ++x)
#pragma unroll
    for (int y = 0; y < C::TN; ++y) { ak[x][y] = 0.f; av[x][y] = 0.f; }

  const int e0 = p.col_ptr[c], e1 = p.col_ptr[c + 1];
  auto fetch_k = [&](int r, int blk) {                          // stage A: dS tile and Q rows of entry (r, blk)
    long long b1, s1, t1;
    tile_address(vds, p, r, c, blk, b1, s1, t1);
    load_tile<BS, BS, C::NT>(dSs, C::SP, dSb + b1, s1, t1, t);
    load_tile<BS, D, C::NT>(Qs, C::SA, Qb + (long long)r * BS * lq.sl, lq.sl, lq.sd, t);
  };
  auto fetch_v = [&](int r, int blk) {                          // stage B: P tile and dO rows
    long long b2, s2, t2;
    tile_address(vp, p, r, c, blk, b2, s2, t2);
    load_tile<BS, BS, C::NT>(Ps, C::SP, Pb + b2, s2, t2, t);
    load_tile<BS, D, C::NT>(Os, C::SA, dOb + (long long)r * BS * ldo.sl, ldo.sl, ldo.sd, t);
  };
  int r_cur = e0 < e1 ? p.row_idx[e0] : 0, b_cur = e0 < e1 ? p.csc_pos[e0] : 0;
  if (e0 < e1) fetch_k(r_cur, b_cur);
  cp_async_commit();
  for (int e = e0; e < e1; ++e) {
    const int r_nxt = e + 1 < e1 ? p.row_idx[e + 1] : 0, b_nxt = e + 1 < e1 ? p.csc_pos[e + 1] : 0;
    fetch_v(r_cur, b_cur);                                       // stage B was released at the end of the last iteration
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();                                             // stage A has landed
    tile_atb<BS, D>(dSs, Qs, ty, tx, ak);
    __syncthreads();                                             // stage A may be refilled
    if (e + 1 < e1) fetch_k(r_nxt, b_nxt);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();                                             // stage B has landed
    tile_atb<BS, D>(Ps, Os, ty, tx, av);
    __syncthreads();
    r_cur = r_nxt;
    b_cur = b_nxt;
  }
  cp_async_wait<0>();
  if (active) {
    store_out<BS, D>(dK + (long long)bh * ldk.bh_stride, ldk, c * BS, ty, tx, ak);
    store_out<BS, D>(dV + (long long)bh * ldv.bh_stride, ldv, c * BS, ty, tx, av);
  }
}

template <int BS, int D> constexpr size_t smem_row() { return sizeof(float) * Cfg<BS, D>::G * (3 * BS * Cfg<BS, D>::SA + BS * Cfg<BS, D>::SP); }
template <int BS, int D> constexpr size_t smem_col() { return sizeof(float) * Cfg<BS, D>::G * (2 * BS * Cfg<BS, D>::SA + 2 * BS * Cfg<BS, D>::SP); }

template <int BS, int D>
int set_attrs() {
  static bool done[64] = {};
  int dev = 0;
  SPION_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 64 && done[dev]) return SPION_OK;
  SPION_CUDA_TRY(cudaFuncSetAttribute(fused_fwd_kernel<BS, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_row<BS, D>()));
  SPION_CUDA_TRY(cudaFuncSetAttribute(fused_bwd_row_kernel<BS, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_row<BS, D>()));
  SPION_CUDA_TRY(cudaFuncSetAttribute(fused_bwd_row_delta_kernel<BS, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_row<BS, D>()));
  SPION_CUDA_TRY(cudaFuncSetAttribute(fused_bwd_col_kernel<BS, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_col<BS, D>()));
  if (dev < 64) done[dev] = true;
  return SPION_OK;
}

template <int BS, int D>
int fwd_launch(const float* Q, OperandLayout lq, const float* K, OperandLayout lk, const float* V, OperandLayout lv,
               const float* keypad, float floor_v, float* P, ValueLayout vl, float* O, OperandLayout lo, Pattern p,
               int BH, int L, float scale, cudaStream_t st) {
  int rc = set_attrs<BS, D>();
  if (rc) return rc;
  const dim3 grid(p.nb, (BH + Cfg<BS, D>::G - 1) / Cfg<BS, D>::G);
  fused_fwd_kernel<BS, D><<<grid, 256, smem_row<BS, D>(), st>>>(Q, lq, K, lk, V, lv, keypad, floor_v, P, vl, O, lo, p, BH,
                                                               L, scale);
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}

template <int BS, int D>
int bwd_launch(const float* Q, OperandLayout lq, const float* K, OperandLayout lk, const float* V, OperandLayout lv,
               const float* P, ValueLayout vp, const float* O, OperandLayout lo, const float* dO, OperandLayout ldo,
               float* dS, ValueLayout vds, float* dQ, OperandLayout ldq, float* dK, OperandLayout ldk, float* dV,
               OperandLayout ldv, Pattern p, int BH, float scale, cudaStream_t st, spion_ctx* prof) {
  int rc = set_attrs<BS, D>();
  if (rc) return rc;
  const dim3 grid(p.nb, (BH + Cfg<BS, D>::G - 1) / Cfg<BS, D>::G);
  if (O)
    fused_bwd_row_delta_kernel<BS, D><<<grid, 256, smem_row<BS, D>(), st>>>(dO, ldo, O, lo, V, lv, K, lk, P, vp, dS, vds,
                                                                           dQ, ldq, p, BH, scale);
  else
    fused_bwd_row_kernel<BS, D><<<grid, 256, smem_row<BS, D>(), st>>>(dO, ldo, V, lv, K, lk, P, vp, dS, vds, dQ, ldq, p,
                                                                     BH, scale);
  SPION_LAUNCH_CHECK();
  if (prof) prof_mark(prof, SPION_STAGE_BWD_ROW);
  fused_bwd_col_kernel<BS, D><<<grid, 256, smem_col<BS, D>(), st>>>(dS, vds, P, vp, Q, lq, dO, ldo, dK, ldk, dV, ldv, p,
                                                                   BH);
  SPION_LAUNCH_CHECK();
  if (prof) prof_mark(prof, SPION_STAGE_SPMM_DKDV);
  return SPION_OK;
}

}  // namespace

bool simt_fused_supports(int bs, int d, int BH, int value_mode) {
  return (bs == 32 || bs == 64) && (d == 32 || d == 64) && BH >= 1 && (BH + 3) / 4 <= 65535 &&
         (value_mode == VAL_ELEMCSR || value_mode == VAL_BLOCKTILE);
}

#define SPION_FUSED_DISPATCH(FN, ...)                                   \
  do {                                                                  \
    if (p.bs == 32 && d == 32) return FN<32, 32>(__VA_ARGS__);          \
    if (p.bs == 32 && d == 64) return FN<32, 64>(__VA_ARGS__);          \
    if (p.bs == 64 && d == 32) return FN<64, 32>(__VA_ARGS__);          \
    if (p.bs == 64 && d == 64) return FN<64, 64>(__VA_ARGS__);          \
    return SPION_ERR_UNSUPPORTED;                                       \
  } while (0)

int simt_fused_forward(const float* Q, OperandLayout lq, const float* K, OperandLayout lk, const float* V,
                       OperandLayout lv, const float* keypad, float floor_v, float* P, ValueLayout vl, float* O,
                       OperandLayout lo, Pattern p, int BH, int L, int d, float scale, cudaStream_t st) {
  if (!simt_fused_supports(p.bs, d, BH, vl.mode)) return SPION_ERR_UNSUPPORTED;
  SPION_FUSED_DISPATCH(fwd_launch, Q, lq, K, lk, V, lv, keypad, floor_v, P, vl, O, lo, p, BH, L, scale, st);
}

int simt_fused_backward(const float* Q, OperandLayout lq, const float* K, OperandLayout lk, const float* V,
                        OperandLayout lv, const float* P, ValueLayout vp, const float* O, OperandLayout lo,
                        const float* dO, OperandLayout ldo, float* dS, ValueLayout vds, float* dQ, OperandLayout ldq,
                        float* dK, OperandLayout ldk, float* dV, OperandLayout ldv, Pattern p, int BH, int d,
                        float scale, cudaStream_t st, spion_ctx* prof) {
  if (!simt_fused_supports(p.bs, d, BH, vp.mode) || vds.mode != vp.mode) return SPION_ERR_UNSUPPORTED;
  SPION_FUSED_DISPATCH(bwd_launch, Q, lq, K, lk, V, lv, P, vp, O, lo, dO, ldo, dS, vds, dQ, ldq, dK, ldk, dV, ldv, p, BH,
                       scale, st, prof);
}
