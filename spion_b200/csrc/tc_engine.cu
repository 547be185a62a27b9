// Tensor-core engine (sm_100a): block-sparse attention on bf16 block tiles with TMA-fed
// tcgen05.mma, accumulators in tensor memory (TMEM), fp32 softmax math in the epilogues.
//
// Replaces, for the native (block-tile) API, the reference's cuSPARSE calls and SIMT softmax
// kernels (models/block_attn.cu:453-545):
//   k_sddmm_fused<MODE 0>   S = Q K^T on the mask  + sparse row softmax  -> P      (:459, :468)
//   k_spmm<false>           O = P V ; dQ = dS K                                      (:478, :516)
//   k_sddmm_fused<MODE 1>   dP = dO V^T on the mask + softmax backward   -> dS      (:498, :507)
//   k_spmm<true>            dK = dS^T Q and dV = P^T dO in one pass over a block column (:526, :536)
//
// Every 64x64 block of the mask is one dense contraction: M = 64 rows (MMA M = 64, accumulator
// row m lives in TMEM lane (m % 16) + 32 * (m / 16)), N = 64 keys or the head dimension, K in
// steps of 16.  Operands are staged by TMA with the hardware swizzle (128 B rows: SWIZZLE_128B,
// 64 B rows: SWIZZLE_64B) and described to the MMA by shared-memory matrix descriptors; transposed
// products need no transposed copies: P/dS tiles and Q/K/V/dO tiles are read as MN-major operands.
// The softmax backward uses  sum_j dP_ij P_ij = sum_n dO_in O_in  (delta), so every dS tile is
// independent of the others and no second pass over the row is needed.
//
// All waits on mbarriers are bounded; on a time-out the CTA records a code in the context's
// status word, frees its TMEM and returns.
#include <cuda.h>

#include "common.cuh"
#include "tc_tiles.cuh"

using namespace tc;

namespace {

// =====================================================================================
// S (or dP) tiles of one block row + fused epilogue.  One CTA per (block row, bh), 128 threads.
//   MODE 0: P  = softmax row-wise over the selected blocks (reference semantics: the L - n_i
//                non-selected keys add exp(0 - m) each to the denominator)
//   MODE 1: dS = P * (dP - delta) * scale,  delta_i = sum_n dO_in O_in
// NCH tiles (64 TMEM columns each) are produced per chunk.
template <int D, int MODE, int NCH>
__global__ void __launch_bounds__(128) k_sddmm_fused(const __grid_constant__ CUtensorMap tmA,
                                                     const __grid_constant__ CUtensorMap tmB,
                                                     __nv_bfloat16* __restrict__ out,
                                                     const __nv_bfloat16* __restrict__ Pin,
                                                     const __nv_bfloat16* __restrict__ dOg,
                                                     const __nv_bfloat16* __restrict__ Og,
                                                     const float* __restrict__ keypad,
                                                     const int* __restrict__ row_ptr, const int* __restrict__ col_idx,
                                                     int L, int nnzb, float scale, float floor_v, int* status) {
  using T = OpTile<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA = sbase;
  const uint32_t sB = sbase + T::BYTES;
  const uint32_t bar_load = sB + NCH * T::BYTES;
  const uint32_t bar_mma = bar_load + 8;
  const uint32_t slot = bar_mma + 8;
  uint32_t* slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (slot - smem_u32(smem_raw)));

  const int r = blockIdx.x, bh = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr uint32_t TMEM_COLS = NCH * 64 < 32 ? 32 : NCH * 64;
  __shared__ int s_abort;                                         // an earlier CTA gave up: do not pile on
  if (tid == 0) s_abort = *reinterpret_cast<volatile int*>(status);
  __syncthreads();
  if (s_abort != 0) return;

  if (warp == 0) {
    tmem_alloc(slot, TMEM_COLS);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    fence_barrier_init();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot_ptr;

  const int rp = row_ptr[r];
  const int nblk = row_ptr[r + 1] - rp;
  const int nchunks = (nblk + NCH - 1) / NCH;
  const bool active = lane < 16;
  const int row = warp * 16 + (lane & 15);                       // accumulator row held by this thread
  const uint32_t tlane = tmem + ((uint32_t)(warp * 32) << 16);
  constexpr uint32_t IDESC = make_idesc_bf16(64, 64, 0, 0);
  uint32_t ph_load = 0, ph_mma = 0;
  bool ok = true;
  bool a_loaded = false;

  // produce the S tiles of chunk ch into TMEM
  auto produce = [&](int ch) -> bool {
    const int t0 = ch * NCH;
    const int nt = min(NCH, nblk - t0);
    if (tid == 0) {
      mbar_expect_tx(bar_load, (a_loaded ? 0 : T::BYTES) + nt * T::BYTES);
      if (!a_loaded) tma_load_2d(sA, &tmA, bar_load, 0, bh * L + r * BS);
      for (int t = 0; t < nt; ++t) tma_load_2d(sB + t * T::BYTES, &tmB, bar_load, 0, bh * L + col_idx[rp + t0 + t] * BS);
    }
    a_loaded = true;
    if (!__syncthreads_and(mbar_wait(bar_load, ph_load))) { if (tid == 0) report(status, ERR_LOAD_WAIT); return false; }
    ph_load ^= 1;
    if (tid == 0) {
      tc_fence_after();
      for (int t = 0; t < nt; ++t) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_bf16(tmem + t * 64, T::kmajor(sA, kk), T::kmajor(sB + t * T::BYTES, kk), IDESC, kk > 0);
      }
      mma_commit(bar_mma);
    }
    if (!__syncthreads_and(mbar_wait(bar_mma, ph_mma))) { if (tid == 0) report(status, ERR_MMA_WAIT); return false; }
    ph_mma ^= 1;
    tc_fence_after();
    return true;
  };
  // all threads are done reading TMEM / smem of the current chunk
  auto release = [&]() {
    tc_fence_before();
    __syncthreads();
  };

  if (MODE == 0) {
    const float sc2 = scale * LOG2E;
    const float* kp = keypad ? keypad + (size_t)bh * L : nullptr;
    float m2 = floor_v * LOG2E, l = 0.f;
    // ---- pass 1: row maximum and denominator
    for (int ch = 0; ch < nchunks && ok; ++ch) {
      ok = produce(ch);
      if (!ok) break;
      const int t0 = ch * NCH, nt = min(NCH, nblk - t0);
      float cm = m2;
      for (int t = 0; t < nt; ++t) {
        const int c = col_idx[rp + t0 + t];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t v[32];
          tmem_ld32(tlane + t * 64 + half * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float x = __uint_as_float(v[j]) * sc2;
            if (kp) x -= kp[c * BS + half * 32 + j] * LOG2E;
            cm = fmaxf(cm, x);
          }
        }
      }
      l *= exp2f(m2 - cm);
      m2 = cm;
      for (int t = 0; t < nt; ++t) {
        const int c = col_idx[rp + t0 + t];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t v[32];
          tmem_ld32(tlane + t * 64 + half * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float x = __uint_as_float(v[j]) * sc2;
            if (kp) x -= kp[c * BS + half * 32 + j] * LOG2E;
            l += exp2f(x - m2);
          }
        }
      }
      if (nchunks > 1) release();
    }
    l += (float)(L - nblk * BS) * exp2f(-m2);
    const float inv = 1.0f / l;
    // ---- pass 2: write P (TMEM still holds the tiles when the row fits in one chunk)
    for (int ch = 0; ch < nchunks && ok; ++ch) {
      if (nchunks > 1) { ok = produce(ch); if (!ok) break; }
      const int t0 = ch * NCH, nt = min(NCH, nblk - t0);
      for (int t = 0; t < nt; ++t) {
        const int blk = rp + t0 + t, c = col_idx[blk];
        __nv_bfloat16* dst = out + (((size_t)bh * nnzb + blk) * BS + row) * BS;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t v[32];
          tmem_ld32(tlane + t * 64 + half * 32, v);
          tmem_ld_wait();
          uint32_t w[16];
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float x0 = __uint_as_float(v[j]) * sc2, x1 = __uint_as_float(v[j + 1]) * sc2;
            if (kp) { x0 -= kp[c * BS + half * 32 + j] * LOG2E; x1 -= kp[c * BS + half * 32 + j + 1] * LOG2E; }
            w[j >> 1] = pack_bf16(exp2f(x0 - m2) * inv, exp2f(x1 - m2) * inv);
          }
          if (active) {
            uint4* d4 = reinterpret_cast<uint4*>(dst + half * 32);
#pragma unroll
            for (int q = 0; q < 4; ++q) d4[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
          }
        }
      }
      if (nchunks > 1) release();
    }
  } else {
    // delta of this thread's row
    float delta = 0.f;
    if (active) {
      const uint4* a4 = reinterpret_cast<const uint4*>(dOg + ((size_t)bh * L + r * BS + row) * D);
      const uint4* b4 = reinterpret_cast<const uint4*>(Og + ((size_t)bh * L + r * BS + row) * D);
#pragma unroll
      for (int q = 0; q < D / 8; ++q) {
        const uint4 a = a4[q], b = b4[q];
        delta += bf16_lo(a.x) * bf16_lo(b.x) + bf16_hi(a.x) * bf16_hi(b.x) + bf16_lo(a.y) * bf16_lo(b.y) +
                 bf16_hi(a.y) * bf16_hi(b.y) + bf16_lo(a.z) * bf16_lo(b.z) + bf16_hi(a.z) * bf16_hi(b.z) +
                 bf16_lo(a.w) * bf16_lo(b.w) + bf16_hi(a.w) * bf16_hi(b.w);
      }
    }
    for (int ch = 0; ch < nchunks && ok; ++ch) {
      ok = produce(ch);
      if (!ok) break;
      const int t0 = ch * NCH, nt = min(NCH, nblk - t0);
      for (int t = 0; t < nt; ++t) {
        const int blk = rp + t0 + t;
        const size_t off = (((size_t)bh * nnzb + blk) * BS + row) * BS;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t v[32];
          tmem_ld32(tlane + t * 64 + half * 32, v);
          tmem_ld_wait();
          if (active) {
            const uint4* p4 = reinterpret_cast<const uint4*>(Pin + off + half * 32);
            uint4* d4 = reinterpret_cast<uint4*>(out + off + half * 32);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 pw = p4[q];
              const uint32_t pws[4] = {pw.x, pw.y, pw.z, pw.w};
              uint32_t o[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const float p0 = bf16_lo(pws[u]), p1 = bf16_hi(pws[u]);
                const float g0 = __uint_as_float(v[q * 8 + 2 * u]), g1 = __uint_as_float(v[q * 8 + 2 * u + 1]);
                o[u] = pack_bf16(p0 * (g0 - delta) * scale, p1 * (g1 - delta) * scale);
              }
              d4[q] = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
        }
      }
      release();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

// =====================================================================================
// dP tiles of one block row + softmax backward -> dS, second generation of MODE 1 above:
// 4 warps (one per TMEM quadrant), two tiles per 64 columns (lane halves 0-15 / 16-31) so every
// lane owns a row, operands requested before TMEM is set up, P tiles brought in by TMA and the
// dS tiles written over them in shared memory and sent out by TMA stores (full-line writes).
template <int D>
__global__ void __launch_bounds__(128) k_dp_ds(const __grid_constant__ CUtensorMap tmdO,
                                               const __grid_constant__ CUtensorMap tmV,
                                               const __grid_constant__ CUtensorMap tmP,
                                               const __grid_constant__ CUtensorMap tmdS,
                                               const __nv_bfloat16* __restrict__ dOg,
                                               const __nv_bfloat16* __restrict__ Og,
                                               const int* __restrict__ row_ptr, const int* __restrict__ col_idx,
                                               int L, int nnzb, float scale, int* status) {
  using T = OpTile<D>;
  constexpr int NCH = 4;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  const uint32_t sA = sbase;                                   // dO tile
  const uint32_t sB = sA + T::BYTES;                           // V tiles
  const uint32_t sP = sB + NCH * T::BYTES;                     // P tiles in, dS tiles out
  const uint32_t bars = sP + NCH * VT_BYTES;
  const uint32_t bar_k = bars, bar_p = bars + 8, bar_s = bars + 16, slot = bars + 24;
  uint32_t* slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (slot - raw));
  __shared__ int s_abort;

  const int r = blockIdx.x, bh = blockIdx.y;
  const int tid = threadIdx.x, q = tid >> 5, lane = tid & 31;
  const int hf = lane >> 4;
  const int row = q * 16 + (lane & 15);
  const int rp = row_ptr[r];
  const int nblk = row_ptr[r + 1] - rp;
  const int nchunks = (nblk + NCH - 1) / NCH;
  bool a_loaded = false;

  auto issue_loads = [&](int ch) {                             // thread 0 only
    const int t0 = ch * NCH, nt = min(NCH, nblk - t0);
    mbar_expect_tx(bar_k, (a_loaded ? 0 : T::BYTES) + nt * T::BYTES);
    if (!a_loaded) tma_load_2d(sA, &tmdO, bar_k, 0, bh * L + r * BS);
    for (int t = 0; t < nt; ++t) tma_load_2d(sB + t * T::BYTES, &tmV, bar_k, 0, bh * L + col_idx[rp + t0 + t] * BS);
    mbar_expect_tx(bar_p, nt * VT_BYTES);
    for (int t = 0; t < nt; ++t)
      tma_load_2d(sP + t * VT_BYTES, &tmP, bar_p, 0, (int)(((size_t)bh * nnzb + rp + t0 + t) * BS));
  };

  if (tid == 0) {
    s_abort = *reinterpret_cast<volatile int*>(status);
    mbar_init(bar_k, 1);
    mbar_init(bar_p, 1);
    mbar_init(bar_s, 1);
    fence_barrier_init();
    if (s_abort == 0 && nblk > 0) issue_loads(0);
  }
  a_loaded = true;
  __syncthreads();
  if (s_abort != 0) return;
  if (q == 0) {
    tmem_alloc(slot, 128);
    tmem_relinquish();
  }
  // delta_i = sum_n dO_in O_in: the two owners of a row take one half of the head dimension each
  float delta;
  {
    const size_t off = ((size_t)bh * L + r * BS + row) * D + hf * (D / 2);
    const uint4* a4 = reinterpret_cast<const uint4*>(dOg + off);
    const uint4* b4 = reinterpret_cast<const uint4*>(Og + off);
    float acc = 0.f;
#pragma unroll
    for (int u = 0; u < D / 16; ++u) {
      const uint4 a = a4[u], b = b4[u];
      acc += bf16_lo(a.x) * bf16_lo(b.x) + bf16_hi(a.x) * bf16_hi(b.x) + bf16_lo(a.y) * bf16_lo(b.y) +
             bf16_hi(a.y) * bf16_hi(b.y) + bf16_lo(a.z) * bf16_lo(b.z) + bf16_hi(a.z) * bf16_hi(b.z) +
             bf16_lo(a.w) * bf16_lo(b.w) + bf16_hi(a.w) * bf16_hi(b.w);
    }
    delta = acc + __shfl_xor_sync(0xffffffffu, acc, 16);
  }
  const float nds = -delta * scale;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot_ptr;
  const uint32_t t_lane = tmem + ((uint32_t)(q * 32) << 16);
  constexpr uint32_t IDESC = make_idesc_bf16(64, 64, 0, 0);
  uint32_t ph_k = 0, ph_p = 0, ph_s = 0;
  bool ok = true;

  for (int ch = 0; ch < nchunks && ok; ++ch) {
    const int t0 = ch * NCH, nt = min(NCH, nblk - t0);
    if (ch > 0 && tid == 0) {
      bulk_wait_read_all();                                    // the previous dS tiles have left shared memory
      issue_loads(ch);
    }
    if (!__syncthreads_and(mbar_wait(bar_k, ph_k))) { if (tid == 0) report(status, ERR_LOAD_WAIT); ok = false; break; }
    ph_k ^= 1;
    if (tid == 0) {
      tc_fence_after();
      for (int t = 0; t < nt; ++t) {
        const uint32_t d_addr = tmem + ((uint32_t)((t & 1) * 16) << 16) + (t >> 1) * 64;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_bf16(d_addr, T::kmajor(sA, kk), T::kmajor(sB + t * T::BYTES, kk), IDESC, kk > 0);
      }
      mma_commit(bar_s);
    }
    const bool w1 = mbar_wait(bar_s, ph_s);
    const bool w2 = mbar_wait(bar_p, ph_p);
    if (!__syncthreads_and(w1 && w2)) { if (tid == 0) report(status, ERR_MMA_WAIT); ok = false; break; }
    ph_s ^= 1; ph_p ^= 1;
    tc_fence_after();
    for (int p = 0; p < 2; ++p) {
      const int t = 2 * p + hf;
      const bool mine = t < nt;
      const uint32_t tile = sP + t * VT_BYTES;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t v[32];
        tmem_ld32(t_lane + p * 64 + half * 32, v);
        tmem_ld_wait();
        if (mine) {
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            const int c = half * 4 + cc;
            const uint32_t addr = tile + row * 128 + ((c ^ (row & 7)) << 4);
            uint32_t w[4];
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr) : "memory");
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float p0 = bf16_lo(w[u]), p1 = bf16_hi(w[u]);
              const float g0 = __uint_as_float(v[cc * 8 + 2 * u]), g1 = __uint_as_float(v[cc * 8 + 2 * u + 1]);
              w[u] = pack_bf16(p0 * fmaf(g0, scale, nds), p1 * fmaf(g1, scale, nds));
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
          }
        }
      }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      for (int t = 0; t < nt; ++t)
        tma_store_2d(&tmdS, sP + t * VT_BYTES, 0, (int)(((size_t)bh * nnzb + rp + t0 + t) * BS));
      bulk_commit();
    }
  }
  if (tid == 0) bulk_wait_read_all();
  tc_fence_before();
  __syncthreads();
  if (q == 0) tmem_dealloc(tmem, 128);
}

// =====================================================================================
// Backward, row side: k_dp_ds plus dQ = dS K in the same CTA.  The K tiles are fetched into the
// V buffers as soon as the dP MMAs have consumed them (that load overlaps the dS arithmetic),
// the dS tiles in shared memory feed both the second product and the TMA stores, and for rows of
// at most 4 blocks the dQ accumulator reuses the TMEM columns of the first dP pair.
template <int D>
__global__ void __launch_bounds__(128) k_bwd_row(const __grid_constant__ CUtensorMap tmdO,
                                                 const __grid_constant__ CUtensorMap tmV,
                                                 const __grid_constant__ CUtensorMap tmK,
                                                 const __grid_constant__ CUtensorMap tmP,
                                                 const __grid_constant__ CUtensorMap tmdS,
                                                 const __nv_bfloat16* __restrict__ dOg,
                                                 const __nv_bfloat16* __restrict__ Og, __nv_bfloat16* __restrict__ dQ,
                                                 const int* __restrict__ row_ptr, const int* __restrict__ col_idx,
                                                 int L, int nnzb, float scale, int* status) {
  using T = OpTile<D>;
  constexpr int NCH = 4;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  const uint32_t sA = sbase;                                   // dO tile
  const uint32_t sB = sA + T::BYTES;                           // V tiles, then K tiles
  const uint32_t sP = sB + NCH * T::BYTES;                     // P tiles in, dS tiles out
  const uint32_t bars = sP + NCH * VT_BYTES;
  const uint32_t bar_v = bars, bar_p = bars + 8, bar_s = bars + 16, bar_k = bars + 24, bar_o = bars + 32, slot = bars + 40;
  uint32_t* slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (slot - raw));
  __shared__ int s_abort;

  const int r = blockIdx.x, bh = blockIdx.y;
  const int tid = threadIdx.x, q = tid >> 5, lane = tid & 31;
  const int hf = lane >> 4;
  const int row = q * 16 + (lane & 15);
  const int rp = row_ptr[r];
  const int nblk = row_ptr[r + 1] - rp;
  const int nchunks = (nblk + NCH - 1) / NCH;
  const bool single = nblk <= NCH;
  const uint32_t ncols = single ? 128u : 256u;
  const uint32_t dq_col = single ? 0u : 128u;
  bool a_loaded = false;

  auto issue_loads = [&](int ch) {                             // thread 0 only
    const int t0 = ch * NCH, nt = min(NCH, nblk - t0);
    mbar_expect_tx(bar_v, (a_loaded ? 0 : T::BYTES) + nt * T::BYTES);
    if (!a_loaded) tma_load_2d(sA, &tmdO, bar_v, 0, bh * L + r * BS);
    for (int t = 0; t < nt; ++t) tma_load_2d(sB + t * T::BYTES, &tmV, bar_v, 0, bh * L + col_idx[rp + t0 + t] * BS);
    mbar_expect_tx(bar_p, nt * VT_BYTES);
    for (int t = 0; t < nt; ++t)
      tma_load_2d(sP + t * VT_BYTES, &tmP, bar_p, 0, (int)(((size_t)bh * nnzb + rp + t0 + t) * BS));
  };

  if (tid == 0) {
    s_abort = *reinterpret_cast<volatile int*>(status);
    mbar_init(bar_v, 1);
    mbar_init(bar_p, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_k, 1);
    mbar_init(bar_o, 1);
    fence_barrier_init();
    if (s_abort == 0 && nblk > 0) issue_loads(0);
  }
  a_loaded = true;
  __syncthreads();
  if (s_abort != 0) return;
  if (q == 0) {
    tmem_alloc(slot, ncols);
    tmem_relinquish();
  }
  float delta;
  {
    const size_t off = ((size_t)bh * L + r * BS + row) * D + hf * (D / 2);
    const uint4* a4 = reinterpret_cast<const uint4*>(dOg + off);
    const uint4* b4 = reinterpret_cast<const uint4*>(Og + off);
    float acc = 0.f;
#pragma unroll
    for (int u = 0; u < D / 16; ++u) {
      const uint4 a = a4[u], b = b4[u];
      acc += bf16_lo(a.x) * bf16_lo(b.x) + bf16_hi(a.x) * bf16_hi(b.x) + bf16_lo(a.y) * bf16_lo(b.y) +
             bf16_hi(a.y) * bf16_hi(b.y) + bf16_lo(a.z) * bf16_lo(b.z) + bf16_hi(a.z) * bf16_hi(b.z) +
             bf16_lo(a.w) * bf16_lo(b.w) + bf16_hi(a.w) * bf16_hi(b.w);
    }
    delta = acc + __shfl_xor_sync(0xffffffffu, acc, 16);
  }
  const float nds = -delta * scale;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot_ptr;
  const uint32_t t_lane = tmem + ((uint32_t)(q * 32) << 16);
  constexpr uint32_t IDESC_P = make_idesc_bf16(64, 64, 0, 0);
  constexpr uint32_t IDESC_Q = make_idesc_bf16(64, D, 0, 1);
  uint32_t ph_v = 0, ph_p = 0, ph_s = 0, ph_k = 0, ph_o = 0;
  bool ok = true;

  for (int ch = 0; ch < nchunks && ok; ++ch) {
    const int t0 = ch * NCH, nt = min(NCH, nblk - t0);
    if (ch > 0 && tid == 0) {
      bulk_wait_read_all();                                    // previous dS tiles have left shared memory
      issue_loads(ch);
    }
    if (!__syncthreads_and(mbar_wait(bar_v, ph_v))) { if (tid == 0) report(status, ERR_LOAD_WAIT); ok = false; break; }
    ph_v ^= 1;
    if (tid == 0) {
      tc_fence_after();
      for (int t = 0; t < nt; ++t) {
        const uint32_t d_addr = tmem + ((uint32_t)((t & 1) * 16) << 16) + (t >> 1) * 64;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_bf16(d_addr, T::kmajor(sA, kk), T::kmajor(sB + t * T::BYTES, kk), IDESC_P, kk > 0);
      }
      mma_commit(bar_s);
    }
    const bool w1 = mbar_wait(bar_s, ph_s);
    if (tid == 0 && w1) {                                      // V consumed: bring K into the same buffers
      mbar_expect_tx(bar_k, nt * T::BYTES);
      for (int t = 0; t < nt; ++t) tma_load_2d(sB + t * T::BYTES, &tmK, bar_k, 0, bh * L + col_idx[rp + t0 + t] * BS);
    }
    const bool w2 = mbar_wait(bar_p, ph_p);
    if (!__syncthreads_and(w1 && w2)) { if (tid == 0) report(status, ERR_MMA_WAIT); ok = false; break; }
    ph_s ^= 1; ph_p ^= 1;
    tc_fence_after();
    for (int p = 0; p < 2; ++p) {
      const int t = 2 * p + hf;
      const bool mine = t < nt;
      const uint32_t tile = sP + t * VT_BYTES;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t v[32];
        tmem_ld32(t_lane + p * 64 + half * 32, v);
        tmem_ld_wait();
        if (mine) {
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            const int c = half * 4 + cc;
            const uint32_t addr = tile + row * 128 + ((c ^ (row & 7)) << 4);
            uint32_t w[4];
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr) : "memory");
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float p0 = bf16_lo(w[u]), p1 = bf16_hi(w[u]);
              const float g0 = __uint_as_float(v[cc * 8 + 2 * u]), g1 = __uint_as_float(v[cc * 8 + 2 * u + 1]);
              w[u] = pack_bf16(p0 * fmaf(g0, scale, nds), p1 * fmaf(g1, scale, nds));
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
          }
        }
      }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      for (int t = 0; t < nt; ++t)
        tma_store_2d(&tmdS, sP + t * VT_BYTES, 0, (int)(((size_t)bh * nnzb + rp + t0 + t) * BS));
      bulk_commit();
      if (mbar_wait(bar_k, ph_k)) {
        tc_fence_after();
        for (int t = 0; t < nt; ++t) {
          const uint32_t d_addr = tmem + ((uint32_t)((t & 1) * 16) << 16) + dq_col;
          const uint32_t first = (ch == 0 && t < 2) ? 0u : 1u;
#pragma unroll
          for (int kk = 0; kk < BS / 16; ++kk)
            mma_bf16(d_addr, ValTile::kmajor(sP + t * VT_BYTES, kk), T::mnmajor(sB + t * T::BYTES, kk), IDESC_Q,
                     (kk > 0) ? 1u : first);
        }
        mma_commit(bar_o);
      } else {
        report(status, ERR_LOAD_WAIT);
      }
    }
    ph_k ^= 1;
    if (!__syncthreads_and(mbar_wait(bar_o, ph_o))) { if (tid == 0) report(status, ERR_MMA2_WAIT); ok = false; break; }
    ph_o ^= 1;
    tc_fence_after();
  }

  if (ok) {
    const bool odd_valid = nblk >= 2;
    __nv_bfloat16* dst = dQ + ((size_t)bh * L + r * BS + row) * D + hf * (D / 2);
#pragma unroll
    for (int h = 0; h < D / 32; ++h) {
      uint32_t v[32];
      if (nblk > 0) {
        tmem_ld32(t_lane + dq_col + h * 32, v);
        tmem_ld_wait();
      }
      float acc[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float mine_v = (nblk > 0 && (hf == 0 || odd_valid)) ? __uint_as_float(v[j]) : 0.f;
        acc[j] = mine_v + __shfl_xor_sync(0xffffffffu, mine_v, 16);
      }
      if (D == 64) {
        if (hf == h) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 pk;
            pk.x = pack_bf16(acc[j], acc[j + 1]); pk.y = pack_bf16(acc[j + 2], acc[j + 3]);
            pk.z = pack_bf16(acc[j + 4], acc[j + 5]); pk.w = pack_bf16(acc[j + 6], acc[j + 7]);
            *reinterpret_cast<uint4*>(dst + j) = pk;
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; j += 8) {
          float val[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) val[u] = hf ? acc[16 + j + u] : acc[j + u];
          uint4 pk;
          pk.x = pack_bf16(val[0], val[1]); pk.y = pack_bf16(val[2], val[3]);
          pk.z = pack_bf16(val[4], val[5]); pk.w = pack_bf16(val[6], val[7]);
          *reinterpret_cast<uint4*>(dst + j) = pk;
        }
      }
    }
  }
  if (tid == 0) bulk_wait_read_all();
  tc_fence_before();
  __syncthreads();
  if (q == 0) tmem_dealloc(tmem, ncols);
}

// =====================================================================================
// Block SpMM.  128 threads, one CTA per (line, bh); NST value/operand tile pairs per chunk.
//   DUAL == false: line = block row r.   out0[r*64.., :] = sum_k  vals0(r, c_k)   * B0[c_k*64.., :]
//   DUAL == true : line = block column c.
//                  out0[c*64.., :] = sum_r vals0(r, c)^T * B0[r*64.., :]      (dK = dS^T Q)
//                  out1[c*64.., :] = sum_r vals1(r, c)^T * B1[r*64.., :]      (dV = P^T dO)
template <int D, bool DUAL, int NST>
__global__ void __launch_bounds__(128) k_spmm(const __grid_constant__ CUtensorMap tmV0,
                                              const __grid_constant__ CUtensorMap tmV1,
                                              const __grid_constant__ CUtensorMap tmB0,
                                              const __grid_constant__ CUtensorMap tmB1,
                                              __nv_bfloat16* __restrict__ out0, __nv_bfloat16* __restrict__ out1,
                                              const int* __restrict__ line_ptr, const int* __restrict__ idx,
                                              const int* __restrict__ pos, int L, int nnzb, int* status) {
  using T = OpTile<D>;
  constexpr int NP = DUAL ? 2 : 1;                                // products per entry
  constexpr int STAGE_BYTES = NP * (VT_BYTES + T::BYTES);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_load = sbase + NST * STAGE_BYTES;
  const uint32_t bar_mma = bar_load + 8;
  const uint32_t slot = bar_mma + 8;
  uint32_t* slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (slot - smem_u32(smem_raw)));

  const int line = blockIdx.x, bh = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr uint32_t TMEM_COLS = (NP * D) < 32 ? 32 : (NP * D);   // 32, 64 or 128: powers of two
  __shared__ int s_abort;                                         // an earlier CTA gave up: do not pile on
  if (tid == 0) s_abort = *reinterpret_cast<volatile int*>(status);
  __syncthreads();
  if (s_abort != 0) return;

  if (warp == 0) {
    tmem_alloc(slot, TMEM_COLS);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    fence_barrier_init();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot_ptr;

  const int beg = line_ptr[line], end = line_ptr[line + 1];
  constexpr uint32_t IDESC = make_idesc_bf16(64, D, DUAL ? 1 : 0, 1);
  uint32_t ph_load = 0, ph_mma = 0;
  bool ok = true;

  for (int e0 = beg; e0 < end && ok; e0 += NST) {
    const int nt = min(NST, end - e0);
    if (tid == 0) {
      mbar_expect_tx(bar_load, nt * STAGE_BYTES);
      for (int t = 0; t < nt; ++t) {
        const int e = e0 + t;
        const int other = idx[e];                                  // block column (CSR) or block row (CSC)
        const int blk = DUAL ? pos[e] : e;                         // CSR block id of the value tile
        const uint32_t st = sbase + t * STAGE_BYTES;
        const int vrow = (int)(((size_t)bh * nnzb + blk) * BS);
        tma_load_2d(st, &tmV0, bar_load, 0, vrow);
        tma_load_2d(st + VT_BYTES, &tmB0, bar_load, 0, bh * L + other * BS);
        if (DUAL) {
          tma_load_2d(st + VT_BYTES + T::BYTES, &tmV1, bar_load, 0, vrow);
          tma_load_2d(st + 2 * VT_BYTES + T::BYTES, &tmB1, bar_load, 0, bh * L + other * BS);
        }
      }
    }
    if (!__syncthreads_and(mbar_wait(bar_load, ph_load))) { if (tid == 0) report(status, ERR_LOAD_WAIT); ok = false; break; }
    ph_load ^= 1;
    if (tid == 0) {
      tc_fence_after();
      for (int t = 0; t < nt; ++t) {
        const uint32_t st = sbase + t * STAGE_BYTES;
        const uint32_t first = (e0 == beg && t == 0) ? 0u : 1u;
#pragma unroll
        for (int kk = 0; kk < BS / 16; ++kk) {
          const uint64_t a0 = DUAL ? ValTile::mnmajor(st, kk) : ValTile::kmajor(st, kk);
          mma_bf16(tmem, a0, T::mnmajor(st + VT_BYTES, kk), IDESC, (kk > 0) ? 1u : first);
        }
        if (DUAL) {
#pragma unroll
          for (int kk = 0; kk < BS / 16; ++kk)
            mma_bf16(tmem + D, ValTile::mnmajor(st + VT_BYTES + T::BYTES, kk),
                     T::mnmajor(st + 2 * VT_BYTES + T::BYTES, kk), IDESC, (kk > 0) ? 1u : first);
        }
      }
      mma_commit(bar_mma);
    }
    if (!__syncthreads_and(mbar_wait(bar_mma, ph_mma))) { if (tid == 0) report(status, ERR_MMA_WAIT); ok = false; break; }
    ph_mma ^= 1;
    tc_fence_after();
  }

  // epilogue: TMEM -> bf16 rows of the output(s)
  const bool active = lane < 16;
  const int row = warp * 16 + (lane & 15);
  const uint32_t tlane = tmem + ((uint32_t)(warp * 32) << 16);
  if (ok) {
#pragma unroll
    for (int pi = 0; pi < NP; ++pi) {
      __nv_bfloat16* dst = (pi == 0 ? out0 : out1) + ((size_t)bh * L + (size_t)line * BS + row) * D;
#pragma unroll
      for (int h = 0; h < D / 32; ++h) {
        uint32_t v[32];
        if (end > beg) {
          tmem_ld32(tlane + pi * D + h * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
        }
        if (active) {
          uint4* d4 = reinterpret_cast<uint4*>(dst + h * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            d4[q] = make_uint4(pack_bf16(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1])),
                               pack_bf16(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3])),
                               pack_bf16(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5])),
                               pack_bf16(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7])));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

// =====================================================================================
// host side
constexpr int NCH_FWD = 4, NCH_BWD = 4, NST_N = 4, NST_T = 2;

template <int D> constexpr size_t smem_sddmm(int nch) { return 1024 + (size_t)(1 + nch) * OpTile<D>::BYTES + 64; }
template <int D> constexpr size_t smem_dp_ds() { return 1024 + (size_t)5 * OpTile<D>::BYTES + 4 * VT_BYTES + 64; }
template <int D> constexpr size_t smem_spmm(int nst, int np) { return 1024 + (size_t)nst * np * (VT_BYTES + OpTile<D>::BYTES) + 64; }

template <int D>
int set_attrs() {
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_sddmm_fused<D, 0, NCH_FWD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem_sddmm<D>(NCH_FWD)));
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_sddmm_fused<D, 1, NCH_BWD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem_sddmm<D>(NCH_BWD)));
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_dp_ds<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dp_ds<D>()));
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_bwd_row<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dp_ds<D>()));
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_spmm<D, false, NST_N>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem_spmm<D>(NST_N, 1)));
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_spmm<D, true, NST_T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem_spmm<D>(NST_T, 2)));
  return SPION_OK;
}

template <int D>
int run_forward(spion_ctx* c, TcState* s, const void* Q, const void* K, const void* V, const float* keypad, void* P,
                void* O, float* S_scratch) {
  const Pattern p = ctx_pattern(c);
  const uint64_t rows = (uint64_t)c->BH * c->L, vrows = (uint64_t)c->BH * c->nnzb * BS;
  const long long nnz = (long long)c->nnzb * BS * BS;
  const ValueLayout vl{VAL_BLOCKTILE, c->L, nnz};
  const OperandLayout rm = row_major_operand(c->L, c->d);
  const dim3 grid(c->nb, c->BH);
  int rc;
  prof_mark(c, -1);
  if (s->stages & 1) {
    CUtensorMap mq, mk;
    if ((rc = make_map(s, &mq, Q, rows, D, BS)) || (rc = make_map(s, &mk, K, rows, D, BS))) return rc;
    k_sddmm_fused<D, 0, NCH_FWD><<<grid, 128, smem_sddmm<D>(NCH_FWD), c->stream>>>(
        mq, mk, (__nv_bfloat16*)P, nullptr, nullptr, nullptr, keypad, c->row_ptr, c->col_idx, c->L, c->nnzb, c->scale,
        keypad ? 0.0f : -100.0f, c->status_dev);
    SPION_LAUNCH_CHECK();
    c->launches += 1;
    prof_mark(c, SPION_STAGE_FUSED_S_P);
  } else {
    if (!S_scratch) return SPION_ERR_ARG;
    if ((rc = simt_sddmm(SPION_BF16, SPION_F32, Q, rm, K, rm, S_scratch, vl, p, c->nnzb, c->BH, c->d, c->stream))) return rc;
    prof_mark(c, SPION_STAGE_SDDMM_S);
    if ((rc = softmax_fwd_rows(SPION_BF16, S_scratch, vl, P, vl, p, c->BH, c->L, c->scale, keypad,
                               keypad ? 0.0f : -100.0f, c->stream))) return rc;
    prof_mark(c, SPION_STAGE_SOFTMAX_FWD);
    c->launches += 2;
  }
  if (s->stages & 2) {
    CUtensorMap mp, mv;
    if ((rc = make_map(s, &mp, P, vrows, BS, BS)) || (rc = make_map(s, &mv, V, rows, D, BS))) return rc;
    k_spmm<D, false, NST_N><<<grid, 128, smem_spmm<D>(NST_N, 1), c->stream>>>(
        mp, mp, mv, mv, (__nv_bfloat16*)O, nullptr, c->row_ptr, c->col_idx, nullptr, c->L, c->nnzb, c->status_dev);
    SPION_LAUNCH_CHECK();
  } else {
    if ((rc = simt_spmm(SPION_BF16, SPION_BF16, false, P, vl, V, rm, O, rm, p, c->BH, c->d, c->stream))) return rc;
  }
  c->launches += 1;
  prof_mark(c, SPION_STAGE_SPMM_O);
  return SPION_OK;
}

template <int D>
int run_backward(spion_ctx* c, TcState* s, const void* Q, const void* K, const void* V, const void* P, const void* O,
                 const void* dO, void* dS, float* dP_scratch, void* dQ, void* dK, void* dV) {
  const Pattern p = ctx_pattern(c);
  const uint64_t rows = (uint64_t)c->BH * c->L, vrows = (uint64_t)c->BH * c->nnzb * BS;
  const long long nnz = (long long)c->nnzb * BS * BS;
  const ValueLayout vl{VAL_BLOCKTILE, c->L, nnz};
  const OperandLayout rm = row_major_operand(c->L, c->d);
  const dim3 grid(c->nb, c->BH);
  int rc;
  prof_mark(c, -1);
  CUtensorMap mds, mp, mq, mk, mdo, mv;
  if ((rc = make_map(s, &mds, dS, vrows, BS, BS)) || (rc = make_map(s, &mp, P, vrows, BS, BS)) ||
      (rc = make_map(s, &mq, Q, rows, D, BS)) || (rc = make_map(s, &mk, K, rows, D, BS)) ||
      (rc = make_map(s, &mdo, dO, rows, D, BS)) || (rc = make_map(s, &mv, V, rows, D, BS)))
    return rc;
  const bool row_fused = (s->stages & 4) && (s->stages & 8) && !(s->stages & 64);
  if (row_fused) {
    k_bwd_row<D><<<grid, 128, smem_dp_ds<D>(), c->stream>>>(mdo, mv, mk, mp, mds, (const __nv_bfloat16*)dO,
                                                            (const __nv_bfloat16*)O, (__nv_bfloat16*)dQ, c->row_ptr,
                                                            c->col_idx, c->L, c->nnzb, c->scale, c->status_dev);
    SPION_LAUNCH_CHECK();
    c->launches += 1;
    prof_mark(c, SPION_STAGE_BWD_ROW);
  } else {
    if (s->stages & 4) {
      if (s->stages & 32)     // first-generation kernel, kept for comparison
        k_sddmm_fused<D, 1, NCH_BWD><<<grid, 128, smem_sddmm<D>(NCH_BWD), c->stream>>>(
            mdo, mv, (__nv_bfloat16*)dS, (const __nv_bfloat16*)P, (const __nv_bfloat16*)dO, (const __nv_bfloat16*)O,
            nullptr, c->row_ptr, c->col_idx, c->L, c->nnzb, c->scale, 0.f, c->status_dev);
      else
        k_dp_ds<D><<<grid, 128, smem_dp_ds<D>(), c->stream>>>(mdo, mv, mp, mds, (const __nv_bfloat16*)dO,
                                                              (const __nv_bfloat16*)O, c->row_ptr, c->col_idx, c->L,
                                                              c->nnzb, c->scale, c->status_dev);
      SPION_LAUNCH_CHECK();
      c->launches += 1;
      prof_mark(c, SPION_STAGE_FUSED_DP_DS);
    } else {
      if (!dP_scratch) return SPION_ERR_ARG;
      if ((rc = simt_sddmm(SPION_BF16, SPION_F32, dO, rm, V, rm, dP_scratch, vl, p, c->nnzb, c->BH, c->d, c->stream))) return rc;
      prof_mark(c, SPION_STAGE_SDDMM_DP);
      if ((rc = softmax_bwd_rows(SPION_BF16, dP_scratch, vl, P, vl, dS, vl, p, c->BH, c->L, c->scale, c->stream))) return rc;
      prof_mark(c, SPION_STAGE_SOFTMAX_BWD);
      c->launches += 2;
    }
    if (s->stages & 8) {
      k_spmm<D, false, NST_N><<<grid, 128, smem_spmm<D>(NST_N, 1), c->stream>>>(
          mds, mds, mk, mk, (__nv_bfloat16*)dQ, nullptr, c->row_ptr, c->col_idx, nullptr, c->L, c->nnzb, c->status_dev);
      SPION_LAUNCH_CHECK();
    } else {
      if ((rc = simt_spmm(SPION_BF16, SPION_BF16, false, dS, vl, K, rm, dQ, rm, p, c->BH, c->d, c->stream))) return rc;
    }
    c->launches += 1;
    prof_mark(c, SPION_STAGE_SPMM_DQ);
  }
  if (s->stages & 16) {
    k_spmm<D, true, NST_T><<<grid, 128, smem_spmm<D>(NST_T, 2), c->stream>>>(
        mds, mp, mq, mdo, (__nv_bfloat16*)dK, (__nv_bfloat16*)dV, c->col_ptr, c->row_idx, c->csc_pos, c->L, c->nnzb,
        c->status_dev);
    SPION_LAUNCH_CHECK();
    c->launches += 1;
    prof_mark(c, SPION_STAGE_SPMM_DKDV);
  } else {
    if ((rc = simt_spmm(SPION_BF16, SPION_BF16, true, dS, vl, Q, rm, dK, rm, p, c->BH, c->d, c->stream))) return rc;
    prof_mark(c, SPION_STAGE_SPMM_DK);
    if ((rc = simt_spmm(SPION_BF16, SPION_BF16, true, P, vl, dO, rm, dV, rm, p, c->BH, c->d, c->stream))) return rc;
    prof_mark(c, SPION_STAGE_SPMM_DV);
    c->launches += 2;
  }
  return SPION_OK;
}

}  // namespace

bool tc_engine_supports(const spion_ctx* c) {
  return c->dtype == SPION_BF16 && c->bs == BS && (c->d == 64 || c->d == 32) &&
         (c->kind == SPION_KIND_BLOCK || c->kind == SPION_KIND_BLOCK_KPM) && c->BH <= 65535 &&
         (unsigned long long)c->BH * c->L < 0x7fffffffULL;
}

int tc_engine_prepare(spion_ctx* c) {
  if (c->tc) return SPION_OK;
  TcState* s = new TcState();
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
    fprintf(stderr, "spion_b200: cuTensorMapEncodeTiled is not available from this driver\n");
    delete s;
    return SPION_ERR_CUDA;
  }
  s->encode = (EncodeTiledFn)fn;
  const char* env = getenv("SPION_TC_STAGES");
  if (env) s->stages = atoi(env) & 0x7f;
  int rc = (c->d == 64) ? set_attrs<64>() : set_attrs<32>();
  if (!rc) rc = fused_set_attrs(c->d);
  if (rc) { delete s; return rc; }
  c->tc = s;
  return SPION_OK;
}

void tc_engine_release(spion_ctx* c) {
  if (c->tc) { delete (TcState*)c->tc; c->tc = nullptr; }
}

int tc_engine_forward(spion_ctx* c, const void* Q, const void* K, const void* V, const float* keypad, void* P, void* O,
                      float* S_scratch) {
  if (!c->tc) return SPION_ERR_STATE;
  TcState* s = (TcState*)c->tc;
  if (c->nnzb == 0) return SPION_ERR_SHAPE;
  return c->d == 64 ? run_forward<64>(c, s, Q, K, V, keypad, P, O, S_scratch)
                    : run_forward<32>(c, s, Q, K, V, keypad, P, O, S_scratch);
}

int tc_engine_backward(spion_ctx* c, const void* Q, const void* K, const void* V, const void* P, const void* O,
                       const void* dO, void* dS, float* dP_scratch, void* dQ, void* dK, void* dV) {
  if (!c->tc) return SPION_ERR_STATE;
  TcState* s = (TcState*)c->tc;
  if (c->nnzb == 0) return SPION_ERR_SHAPE;
  return c->d == 64 ? run_backward<64>(c, s, Q, K, V, P, O, dO, dS, dP_scratch, dQ, dK, dV)
                    : run_backward<32>(c, s, Q, K, V, P, O, dO, dS, dP_scratch, dQ, dK, dV);
}

namespace tc {
int tc_engine_probabilities(spion_ctx* c, const void* Q, const void* K, const float* keypad, void* P) {
  TcState* s = (TcState*)c->tc;
  const uint64_t rows = (uint64_t)c->BH * c->L;
  CUtensorMap mq, mk;
  int rc;
  if ((rc = make_map(s, &mq, Q, rows, (uint32_t)c->d, BS)) || (rc = make_map(s, &mk, K, rows, (uint32_t)c->d, BS))) return rc;
  const dim3 grid(c->nb, c->BH);
  if (c->d == 64)
    k_sddmm_fused<64, 0, NCH_FWD><<<grid, 128, smem_sddmm<64>(NCH_FWD), c->stream>>>(
        mq, mk, (__nv_bfloat16*)P, nullptr, nullptr, nullptr, keypad, c->row_ptr, c->col_idx, c->L, c->nnzb, c->scale,
        keypad ? 0.0f : -100.0f, c->status_dev);
  else
    k_sddmm_fused<32, 0, NCH_FWD><<<grid, 128, smem_sddmm<32>(NCH_FWD), c->stream>>>(
        mq, mk, (__nv_bfloat16*)P, nullptr, nullptr, nullptr, keypad, c->row_ptr, c->col_idx, c->L, c->nnzb, c->scale,
        keypad ? 0.0f : -100.0f, c->status_dev);
  SPION_LAUNCH_CHECK();
  c->launches += 1;
  prof_mark(c, SPION_STAGE_FUSED_S_P);
  return SPION_OK;
}
}  // namespace tc

int tc_engine_forward_fused(spion_ctx* c, const void* Q, const void* K, const void* V, const float* keypad, void* O,
                            float* lse, void* P_optional) {
  if (!c->tc) return SPION_ERR_STATE;
  if (c->nnzb == 0) return SPION_ERR_SHAPE;
  return fused_forward(c, (TcState*)c->tc, Q, K, V, keypad, O, lse, P_optional);
}

int tc_engine_backward_fused(spion_ctx* c, const void* Q, const void* K, const void* V, const float* keypad,
                             const void* O, const float* lse, const void* dO, float* delta, void* dQ, void* dK,
                             void* dV) {
  if (!c->tc) return SPION_ERR_STATE;
  if (c->nnzb == 0) return SPION_ERR_SHAPE;
  return fused_backward(c, (TcState*)c->tc, Q, K, V, keypad, O, lse, dO, delta, dQ, dK, dV);
}
