// Tensor-core engine (sm_100a): block-sparse attention on bf16 block tiles with TMA-fed
// tcgen05.mma, accumulators in tensor memory (TMEM), fp32 softmax math in the epilogues.
//
// Replaces, for the native (block-tile) API, the reference's cuSPARSE calls and SIMT softmax
// kernels (models/block_attn.cu:453-545):
//   k_fwd_fused (tc_fused.cu)  S = Q K^T on the mask, sparse row softmax, O = P V        (:459-478)
//   k_bwd_row                  dP = dO V^T on the mask, softmax backward -> dS, dQ = dS K  (:498-516)
//   k_dp_ds + k_spmm<false>    the same two steps as separate kernels (debugging switch)
//   k_spmm<true>               dK = dS^T Q and dV = P^T dO in one pass over a block column (:526, :536)
// Masks with 32-wide blocks run on derived 64-wide super-blocks whose unselected quarters are
// masked inside the forward softmax (P = 0 there, so the backward needs no special handling).
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
// dP tiles of one block row + softmax backward -> dS (used when the row kernel below is split):
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
                                               const int4* __restrict__ row_info, const int* __restrict__ col_idx,
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

  const int bh = blockIdx.y;
  const int tid = threadIdx.x, q = tid >> 5, lane = tid & 31;
  const int hf = lane >> 4;
  const int row = q * 16 + (lane & 15);
  const int4 ri = row_info[blockIdx.x];                        // records are sorted, longest row first
  const int rp = ri.x, nblk = ri.y & 0xffff, r = ri.y >> 16;
  auto col_of = [&](int t) -> int {                            // block column of the row's t-th block
    return t < 4 ? ((t & 2 ? ri.w : ri.z) >> ((t & 1) * 16)) & 0xffff : col_idx[rp + t];
  };
  const int nchunks = (nblk + NCH - 1) / NCH;
  bool a_loaded = false;

  auto issue_loads = [&](int ch) {                             // all lanes of warp 0: one copy per lane
    const int t0 = ch * NCH, nt = min(NCH, nblk - t0);
    if (lane == 0) {
      mbar_expect_tx(bar_k, (a_loaded ? 0 : T::BYTES) + nt * T::BYTES);
      mbar_expect_tx(bar_p, nt * VT_BYTES);
    }
    __syncwarp();
    if (lane == 0 && !a_loaded) tma_load_2d(sA, &tmdO, bar_k, 0, bh * L + r * BS);
    if (lane >= 1 && lane <= nt) tma_load_2d(sB + (lane - 1) * T::BYTES, &tmV, bar_k, 0, bh * L + col_of(t0 + lane - 1) * BS);
    if (lane >= 9 && lane < 9 + nt)
      tma_load_2d(sP + (lane - 9) * VT_BYTES, &tmP, bar_p, 0, (int)(((size_t)bh * nnzb + rp + t0 + lane - 9) * BS));
  };

  if (q == 0) {
    if (lane == 0) {
      s_abort = *reinterpret_cast<volatile int*>(status);
      mbar_init(bar_k, 1);
      mbar_init(bar_p, 1);
      mbar_init(bar_s, 1);
      fence_barrier_init();
    }
    __syncwarp();
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
    if (ch > 0 && q == 0) {
      if (lane == 0) bulk_wait_read_all();                     // the previous dS tiles have left shared memory
      __syncwarp();
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
                                                 const int4* __restrict__ row_info, const int* __restrict__ col_idx,
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

  // (b,h) matrices are walked in descending order: the forward pass wrote P in ascending order, so the
  // most recently written tiles (still in L2) are read first, and the dS tiles this kernel writes
  // last are the ones the column kernel, which ascends, reads first.
  const int bh = gridDim.y - 1 - blockIdx.y;
  const int tid = threadIdx.x, q = tid >> 5, lane = tid & 31;
  const int hf = lane >> 4;
  const int row = q * 16 + (lane & 15);
  const int4 ri = row_info[blockIdx.x];                        // records are sorted, longest row first
  const int rp = ri.x, nblk = ri.y & 0xffff, r = ri.y >> 16;
  auto col_of = [&](int t) -> int {                            // block column of the row's t-th block
    return t < 4 ? ((t & 2 ? ri.w : ri.z) >> ((t & 1) * 16)) & 0xffff : col_idx[rp + t];
  };
  const int nchunks = (nblk + NCH - 1) / NCH;
  const bool single = nblk <= NCH;
  const uint32_t ncols = single ? 128u : 256u;
  const uint32_t dq_col = single ? 0u : 128u;
  bool a_loaded = false;

  auto issue_loads = [&](int ch) {                             // all lanes of warp 0: one copy per lane
    const int t0 = ch * NCH, nt = min(NCH, nblk - t0);
    if (lane == 0) {
      mbar_expect_tx(bar_v, (a_loaded ? 0 : T::BYTES) + nt * T::BYTES);
      mbar_expect_tx(bar_p, nt * VT_BYTES);
    }
    __syncwarp();
    if (lane == 0 && !a_loaded) tma_load_2d(sA, &tmdO, bar_v, 0, bh * L + r * BS);
    if (lane >= 1 && lane <= nt) tma_load_2d(sB + (lane - 1) * T::BYTES, &tmV, bar_v, 0, bh * L + col_of(t0 + lane - 1) * BS);
    if (lane >= 9 && lane < 9 + nt)
      tma_load_2d(sP + (lane - 9) * VT_BYTES, &tmP, bar_p, 0, (int)(((size_t)bh * nnzb + rp + t0 + lane - 9) * BS));
  };

  if (q == 0) {
    if (lane == 0) {
      s_abort = *reinterpret_cast<volatile int*>(status);
      mbar_init(bar_v, 1);
      mbar_init(bar_p, 1);
      mbar_init(bar_s, 1);
      mbar_init(bar_k, 1);
      mbar_init(bar_o, 1);
      fence_barrier_init();
    }
    __syncwarp();
    // long rows ask for their first tiles before the (larger) TMEM allocation, short rows after it:
    // each order measured faster for its case
    if (s_abort == 0 && nblk > 0 && !single) issue_loads(0);
  }
  __syncthreads();
  if (s_abort != 0) return;
  if (q == 0) {
    tmem_alloc(slot, ncols);
    tmem_relinquish();
    if (nblk > 0 && single) issue_loads(0);
  }
  a_loaded = true;
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
    if (ch > 0 && q == 0) {
      if (lane == 0) bulk_wait_read_all();                     // previous dS tiles have left shared memory
      __syncwarp();
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
    if (q == 0) {                                              // V consumed: bring K into the same buffers
      const bool all_ok = __all_sync(0xffffffffu, w1);
      if (all_ok) {
        if (lane == 0) mbar_expect_tx(bar_k, nt * T::BYTES);
        __syncwarp();
        if (lane < nt) tma_load_2d(sB + lane * T::BYTES, &tmK, bar_k, 0, bh * L + col_of(t0 + lane) * BS);
      }
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
                                              const int* __restrict__ pos, const int* __restrict__ order, int L,
                                              int nnzb, int* status) {
  using T = OpTile<D>;
  constexpr int NP = DUAL ? 2 : 1;                                // products per entry
  constexpr int STAGE_BYTES = NP * (VT_BYTES + T::BYTES);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // ring of NST stages, one entry of the line each: full[s] (tiles landed), empty[s] (MMAs that read them done)
  const uint32_t bar_full = sbase + NST * STAGE_BYTES;
  const uint32_t bar_empty = bar_full + 8 * NST;
  const uint32_t bar_done = bar_empty + 8 * NST;
  const uint32_t slot = bar_done + 8;
  uint32_t* slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (slot - smem_u32(smem_raw)));

  // One (b,h) matrix after the other (the value tiles of a matrix were written together, and a grid that
  // interleaves the matrices measured slower); inside a matrix the longest lines first when an order is given.
  const int bh = blockIdx.y, line = order ? order[blockIdx.x] : (int)blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr uint32_t TMEM_COLS = (NP * D) < 32 ? 32 : (NP * D);   // 32, 64 or 128: powers of two
  __shared__ int s_abort;                                         // an earlier CTA gave up: do not pile on
  const int beg = line_ptr[line], end = line_ptr[line + 1];
  const int n = end - beg;

  // warp 0, all lanes: request entry e into stage st (one copy per lane)
  auto fill = [&](int st, int e) {
    const uint32_t sa = sbase + st * STAGE_BYTES;
    if (lane == 0) mbar_expect_tx(bar_full + 8 * st, STAGE_BYTES);
    __syncwarp();
    if (lane < 2 * NP) {
      const int other = idx[e];                                    // block column (CSR) or block row (CSC)
      const int blk = DUAL ? pos[e] : e;                           // CSR block id of the value tile
      const int vrow = (int)(((size_t)bh * nnzb + blk) * BS);
      const int orow = bh * L + other * BS;
      if (lane == 0) tma_load_2d(sa, &tmV0, bar_full + 8 * st, 0, vrow);
      if (lane == 1) tma_load_2d(sa + VT_BYTES, &tmB0, bar_full + 8 * st, 0, orow);
      if (DUAL && lane == 2) tma_load_2d(sa + VT_BYTES + T::BYTES, &tmV1, bar_full + 8 * st, 0, vrow);
      if (DUAL && lane == 3) tma_load_2d(sa + 2 * VT_BYTES + T::BYTES, &tmB1, bar_full + 8 * st, 0, orow);
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      s_abort = *reinterpret_cast<volatile int*>(status);
      for (int st = 0; st < NST; ++st) { mbar_init(bar_full + 8 * st, 1); mbar_init(bar_empty + 8 * st, 1); }
      mbar_init(bar_done, 1);
      fence_barrier_init();
    }
  }
  __syncthreads();
  if (s_abort != 0) return;
  if (warp == 0) {
    tmem_alloc(slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot_ptr;
  constexpr uint32_t IDESC = make_idesc_bf16(64, D, DUAL ? 1 : 0, 1);
  bool ok = true;

  if (warp == 0) {
    // (requesting the first tiles before the TMEM allocation measured slower for this kernel)
    for (int t = 0; t < NST && t < n; ++t) fill(t, beg + t);
    for (int i = 0; i < n; ++i) {
      const int st = i % NST;
      const uint32_t ph = (uint32_t)(i / NST) & 1u;
      if (!__all_sync(0xffffffffu, mbar_wait(bar_full + 8 * st, ph))) { if (lane == 0) report(status, ERR_LOAD_WAIT); ok = false; break; }
      if (lane == 0) {
        tc_fence_after();
        const uint32_t sa = sbase + st * STAGE_BYTES;
        const uint32_t first = i == 0 ? 0u : 1u;
#pragma unroll
        for (int kk = 0; kk < BS / 16; ++kk) {
          const uint64_t a0 = DUAL ? ValTile::mnmajor(sa, kk) : ValTile::kmajor(sa, kk);
          mma_bf16(tmem, a0, T::mnmajor(sa + VT_BYTES, kk), IDESC, (kk > 0) ? 1u : first);
        }
        if (DUAL) {
#pragma unroll
          for (int kk = 0; kk < BS / 16; ++kk)
            mma_bf16(tmem + D, ValTile::mnmajor(sa + VT_BYTES + T::BYTES, kk),
                     T::mnmajor(sa + 2 * VT_BYTES + T::BYTES, kk), IDESC, (kk > 0) ? 1u : first);
        }
        if (i + 1 == n) mma_commit(bar_done);
        else mma_commit(bar_empty + 8 * st);
      }
      __syncwarp();
      if (i + NST < n) {                                           // this stage takes entry i + NST once its MMAs are done
        if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * st, ph))) { if (lane == 0) report(status, ERR_MMA_WAIT); ok = false; break; }
        fill(st, beg + i + NST);
      }
    }
  }
  {
    // only warp 0 polls the barrier of the last MMAs; the other warps sleep in the CTA barrier
    bool w = true;
    if (warp == 0) {
      w = (n > 0 && ok) ? mbar_wait(bar_done, 0) : (n == 0);
      tc_fence_before();
    }
    if (!__syncthreads_and(w)) { if (tid == 0 && ok) report(status, ERR_MMA_WAIT); ok = false; } else ok = true;
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
// ---------------------------------------------------------------- 32-wide masks on 64-wide super-blocks
__global__ void k_mat64_from_mat32(const uint8_t* __restrict__ mat32, int nb32, uint8_t* __restrict__ mat64) {
  const int nb64 = nb32 / 2;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < nb64 * nb64; i += gridDim.x * blockDim.x) {
    const int R = i / nb64, C = i % nb64;
    const uint8_t* m = mat32 + (size_t)(2 * R) * nb32 + 2 * C;
    mat64[i] = (m[0] | m[1] | m[nb32] | m[nb32 + 1]) ? 1 : 0;
  }
}
__global__ void k_submask(const uint8_t* __restrict__ mat32, int nb32, const int32_t* __restrict__ blk_row64,
                          const int32_t* __restrict__ col_idx64, const int32_t* __restrict__ nnzb64,
                          uint8_t* __restrict__ submask) {
  const int n = *nnzb64;
  for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < n; b += gridDim.x * blockDim.x) {
    const uint8_t* m = mat32 + (size_t)(2 * blk_row64[b]) * nb32 + 2 * col_idx64[b];
    submask[b] = (uint8_t)((m[0] ? 1 : 0) | (m[1] ? 2 : 0) | (m[nb32] ? 4 : 0) | (m[nb32 + 1] ? 8 : 0));
  }
}
// value tiles: [BH, nnzb64, 64, 64] super-tiles <-> [BH, nnzb32, 32, 32] tiles of the mask's own blocks.
// One CTA per (super-block, bh); id32 maps a cell of the 32-wide mask to its CSR block id.
template <bool TO64>
__global__ void __launch_bounds__(256) k_convert_tiles(__nv_bfloat16* __restrict__ v64, __nv_bfloat16* __restrict__ v32,
                                                       const int32_t* __restrict__ blk_row64,
                                                       const int32_t* __restrict__ col_idx64,
                                                       const uint8_t* __restrict__ submask,
                                                       const int32_t* __restrict__ id32, int nb32, int nnzb64,
                                                       int nnzb32) {
  const int b64 = blockIdx.x, bh = blockIdx.y;
  const int R = blk_row64[b64], C = col_idx64[b64];
  const uint8_t sm = submask[b64];
  __nv_bfloat16* t64 = v64 + ((size_t)bh * nnzb64 + b64) * 4096;
  for (int e = threadIdx.x; e < 4096 / 8; e += blockDim.x) {           // 8 elements (16 bytes) per step
    const int i = e / 8, j8 = (e % 8) * 8;
    const int a = i / 32, bq = j8 / 32;
    const bool on = (sm >> (a * 2 + bq)) & 1;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (on) {
      const int b32 = id32[(size_t)(2 * R + a) * nb32 + 2 * C + bq];
      __nv_bfloat16* t32 = v32 + ((size_t)bh * nnzb32 + b32) * 1024 + (i % 32) * 32 + (j8 % 32);
      if (TO64) val = *reinterpret_cast<const uint4*>(t32);
      else *reinterpret_cast<uint4*>(t32) = *reinterpret_cast<const uint4*>(t64 + i * 64 + j8);
    }
    if (TO64) *reinterpret_cast<uint4*>(t64 + i * 64 + j8) = val;
  }
}

// One record per block row, sorted by descending number of blocks (ties: ascending row), so that a
// grid walking the records starts its longest rows first.  One CTA; nb <= SPION_MAX_NB.
//   {row_ptr, blocks | row << 16, col0 | col1 << 16, col2 | col3 << 16}
__global__ void k_row_info(const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ col_idx, int nb,
                           int4* __restrict__ info) {
  __shared__ int s_n[SPION_MAX_NB];
  for (int r = threadIdx.x; r < nb; r += blockDim.x) s_n[r] = row_ptr[r + 1] - row_ptr[r];
  __syncthreads();
  for (int r = threadIdx.x; r < nb; r += blockDim.x) {
    const int rp = row_ptr[r], n = s_n[r];
    int rank = 0;
    for (int o = 0; o < nb; ++o) rank += (s_n[o] > n) || (s_n[o] == n && o < r);
    int c[4] = {0, 0, 0, 0};
    for (int t = 0; t < 4 && t < n; ++t) c[t] = col_idx[rp + t];
    info[rank] = make_int4(rp, n | (r << 16), c[0] | (c[1] << 16), c[2] | (c[3] << 16));
  }
}

// Lines (block columns) sorted by descending number of entries (ties: ascending index).  One CTA.
__global__ void k_line_order(const int32_t* __restrict__ line_ptr, int nb, int* __restrict__ order) {
  __shared__ int s_n[SPION_MAX_NB];
  for (int c = threadIdx.x; c < nb; c += blockDim.x) s_n[c] = line_ptr[c + 1] - line_ptr[c];
  __syncthreads();
  for (int c = threadIdx.x; c < nb; c += blockDim.x) {
    const int n = s_n[c];
    int rank = 0;
    for (int o = 0; o < nb; ++o) rank += (s_n[o] > n) || (s_n[o] == n && o < c);
    order[rank] = c;
  }
}

// Self-test of the bounded wait: one CTA waits on an mbarrier that nothing ever arrives on, with a
// short limit; it must give up, record ERR_LOAD_WAIT in the status word and return normally.
__global__ void k_wait_selftest(int* status, long long limit_cycles) {
  __shared__ __align__(8) unsigned long long bar_storage;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    fence_barrier_init();
  }
  __syncthreads();
  const bool ok = __syncthreads_and(mbar_wait_limit(bar, 0, limit_cycles));
  if (!ok && threadIdx.x == 0) report(status, ERR_LOAD_WAIT);
}

constexpr int NST_N = 4, NST_T = 2;

template <int D> constexpr size_t smem_dp_ds() { return 1024 + (size_t)5 * OpTile<D>::BYTES + 4 * VT_BYTES + 64; }
template <int D> constexpr size_t smem_spmm(int nst, int np) { return 1024 + (size_t)nst * np * (VT_BYTES + OpTile<D>::BYTES) + 128; }

template <int D>
int set_attrs() {
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_dp_ds<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dp_ds<D>()));
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_bwd_row<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dp_ds<D>()));
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_spmm<D, false, NST_N>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem_spmm<D>(NST_N, 1)));
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_spmm<D, true, NST_T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem_spmm<D>(NST_T, 2)));
  return SPION_OK;
}

int convert_tiles(spion_ctx* c, TcState* s, bool to64, void* v64, void* v32) {
  const dim3 grid(s->nnzb64, c->BH);
  if (to64)
    k_convert_tiles<true><<<grid, 256, 0, c->stream>>>((__nv_bfloat16*)v64, (__nv_bfloat16*)v32, s->blk_row64,
                                                       s->col_idx64, s->submask, c->work, c->nb, s->nnzb64, c->nnzb);
  else
    k_convert_tiles<false><<<grid, 256, 0, c->stream>>>((__nv_bfloat16*)v64, (__nv_bfloat16*)v32, s->blk_row64,
                                                        s->col_idx64, s->submask, c->work, c->nb, s->nnzb64, c->nnzb);
  SPION_LAUNCH_CHECK();
  c->launches += 1;
  return SPION_OK;
}

template <int D>
int run_backward(spion_ctx* c, TcState* s, const void* Q, const void* K, const void* V, const void* P_user,
                 const void* O, const void* dO, void* dS_user, void* dQ, void* dK, void* dV) {
  const TcView vw = tc_view(c, s);
  const void* P = P_user;
  void* dS = dS_user;
  int rc;
  if (s->super) {                    // bring the caller's 32-wide tiles into super-tile form
    if ((rc = convert_tiles(c, s, true, s->p64_ws, const_cast<void*>(P_user)))) return rc;
    P = s->p64_ws;
    dS = s->ds64_ws;
  }
  const uint64_t rows = (uint64_t)c->BH * c->L, vrows = (uint64_t)c->BH * vw.nnzb * BS;
  const dim3 grid(vw.nb, c->BH);
  prof_mark(c, -1);
  CUtensorMap mds, mp, mq, mk, mdo, mv;
  if ((rc = make_map(s, &mds, dS, vrows, BS, BS)) || (rc = make_map(s, &mp, P, vrows, BS, BS)) ||
      (rc = make_map(s, &mq, Q, rows, D, BS)) || (rc = make_map(s, &mk, K, rows, D, BS)) ||
      (rc = make_map(s, &mdo, dO, rows, D, BS)) || (rc = make_map(s, &mv, V, rows, D, BS)))
    return rc;
  if (!(s->stages & 64)) {
    k_bwd_row<D><<<grid, 128, smem_dp_ds<D>(), c->stream>>>(mdo, mv, mk, mp, mds, (const __nv_bfloat16*)dO,
                                                            (const __nv_bfloat16*)O, (__nv_bfloat16*)dQ, vw.row_info,
                                                            vw.col_idx, c->L, vw.nnzb, c->scale, c->status_dev);
    SPION_LAUNCH_CHECK();
    c->launches += 1;
    prof_mark(c, SPION_STAGE_BWD_ROW);
  } else {
    k_dp_ds<D><<<grid, 128, smem_dp_ds<D>(), c->stream>>>(mdo, mv, mp, mds, (const __nv_bfloat16*)dO,
                                                          (const __nv_bfloat16*)O, vw.row_info, vw.col_idx, c->L,
                                                          vw.nnzb, c->scale, c->status_dev);
    SPION_LAUNCH_CHECK();
    prof_mark(c, SPION_STAGE_FUSED_DP_DS);
    k_spmm<D, false, NST_N><<<dim3(vw.nb, c->BH), 128, smem_spmm<D>(NST_N, 1), c->stream>>>(
        mds, mds, mk, mk, (__nv_bfloat16*)dQ, nullptr, vw.row_ptr, vw.col_idx, nullptr, nullptr, c->L, vw.nnzb,
        c->status_dev);
    SPION_LAUNCH_CHECK();
    c->launches += 2;
    prof_mark(c, SPION_STAGE_SPMM_DQ);
  }
  k_spmm<D, true, NST_T><<<dim3(vw.nb, c->BH), 128, smem_spmm<D>(NST_T, 2), c->stream>>>(
      mds, mp, mq, mdo, (__nv_bfloat16*)dK, (__nv_bfloat16*)dV, vw.col_ptr, vw.row_idx, vw.csc_pos,
      s->col_order, c->L, vw.nnzb, c->status_dev);
  SPION_LAUNCH_CHECK();
  c->launches += 1;
  prof_mark(c, SPION_STAGE_SPMM_DKDV);
  return SPION_OK;
}

void free_super(TcState* s) {
  cudaFree(s->mat64); cudaFree(s->submask); cudaFree(s->row_ptr64); cudaFree(s->col_idx64); cudaFree(s->blk_row64);
  cudaFree(s->col_ptr64); cudaFree(s->row_idx64); cudaFree(s->csc_pos64); cudaFree(s->work64); cudaFree(s->nnzb64_dev);
  cudaFree(s->p64_ws); cudaFree(s->ds64_ws);
  s->mat64 = s->submask = nullptr;
  s->row_ptr64 = s->col_idx64 = s->blk_row64 = s->col_ptr64 = s->row_idx64 = s->csc_pos64 = s->work64 = s->nnzb64_dev = nullptr;
  s->p64_ws = s->ds64_ws = nullptr;
  s->ws_elems = 0;
}

// derive the super-block structure of a 32-wide mask (set_pattern time; synchronises once)
int build_super(spion_ctx* c, TcState* s) {
  const int nb64 = c->nb / 2;
  const size_t cap = (size_t)nb64 * nb64;
  if (!s->mat64) {
    bool ok = cudaMalloc(&s->mat64, cap) == cudaSuccess && cudaMalloc(&s->submask, cap) == cudaSuccess &&
              cudaMalloc(&s->row_ptr64, (nb64 + 1) * 4) == cudaSuccess && cudaMalloc(&s->col_idx64, cap * 4) == cudaSuccess &&
              cudaMalloc(&s->blk_row64, cap * 4) == cudaSuccess && cudaMalloc(&s->col_ptr64, (nb64 + 1) * 4) == cudaSuccess &&
              cudaMalloc(&s->row_idx64, cap * 4) == cudaSuccess && cudaMalloc(&s->csc_pos64, cap * 4) == cudaSuccess &&
              cudaMalloc(&s->work64, cap * 4) == cudaSuccess && cudaMalloc(&s->nnzb64_dev, 4) == cudaSuccess;
    if (!ok) return SPION_ERR_ALLOC;
  }
  s->nb64 = nb64;
  k_mat64_from_mat32<<<64, 256, 0, c->stream>>>(c->mat, c->nb, s->mat64);
  SPION_LAUNCH_CHECK();
  int rc = spion_launch_build_structure(s->mat64, nb64, s->nnzb64_dev, s->row_ptr64, s->col_idx64, s->blk_row64,
                                        s->col_ptr64, s->row_idx64, s->csc_pos64, s->work64, c->stream);
  if (rc) return rc;
  k_submask<<<64, 256, 0, c->stream>>>(c->mat, c->nb, s->blk_row64, s->col_idx64, s->nnzb64_dev, s->submask);
  SPION_LAUNCH_CHECK();
  int32_t n = 0;
  SPION_CUDA_TRY(cudaMemcpyAsync(&n, s->nnzb64_dev, 4, cudaMemcpyDeviceToHost, c->stream));
  SPION_CUDA_TRY(cudaStreamSynchronize(c->stream));
  s->nnzb64 = n;
  const size_t need = (size_t)c->BH * n * 4096;
  if (need > s->ws_elems) {
    cudaFree(s->p64_ws); cudaFree(s->ds64_ws);
    s->p64_ws = s->ds64_ws = nullptr;
    if (cudaMalloc(&s->p64_ws, need * 2) != cudaSuccess || cudaMalloc(&s->ds64_ws, need * 2) != cudaSuccess)
      return SPION_ERR_ALLOC;
    s->ws_elems = need;
  }
  c->launches += 3;
  return SPION_OK;
}

}  // namespace

bool tc_engine_supports(const spion_ctx* c) {
  const bool blocks = c->bs == BS || (c->bs == 32 && c->L % 64 == 0);
  return c->dtype == SPION_BF16 && blocks && (c->d == 64 || c->d == 32) &&
         (c->kind == SPION_KIND_BLOCK || c->kind == SPION_KIND_BLOCK_KPM) && c->BH <= 65535 &&
         (unsigned long long)c->BH * c->L < 0x7fffffffULL;
}

int tc_engine_prepare(spion_ctx* c) {
  TcState* s = (TcState*)c->tc;
  if (!s) {
    s = new TcState();
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
    if (env) s->stages = atoi(env);
    int rc = (c->d == 64) ? set_attrs<64>() : set_attrs<32>();
    if (!rc) rc = fused_set_attrs(c->d);
    if (!rc && cudaMalloc(&s->lse_ws, (size_t)c->BH * c->L * sizeof(float)) != cudaSuccess) rc = SPION_ERR_ALLOC;
    if (rc) { delete s; return rc; }
    s->super = c->bs == 32;
    c->tc = s;
  }
  if (s->super) {
    int rc = build_super(c, s);
    if (rc) return rc;
  }
  const TcView vw = tc_view(c, s);
  if (!s->row_info && cudaMalloc(&s->row_info, (size_t)SPION_MAX_NB * sizeof(int4)) != cudaSuccess) return SPION_ERR_ALLOC;
  k_row_info<<<1, 512, 0, c->stream>>>(vw.row_ptr, vw.col_idx, vw.nb, s->row_info);
  SPION_LAUNCH_CHECK();
  if (!s->col_order && cudaMalloc(&s->col_order, (size_t)SPION_MAX_NB * sizeof(int)) != cudaSuccess) return SPION_ERR_ALLOC;
  k_line_order<<<1, 512, 0, c->stream>>>(vw.col_ptr, vw.nb, s->col_order);
  SPION_LAUNCH_CHECK();
  c->launches += 2;
  return SPION_OK;
}

void tc_engine_release(spion_ctx* c) {
  if (!c->tc) return;
  TcState* s = (TcState*)c->tc;
  free_super(s);
  cudaFree(s->lse_ws);
  cudaFree(s->row_info);
  cudaFree(s->col_order);
  delete s;
  c->tc = nullptr;
}

// forward with the probabilities in the caller's tile layout (P_user may be NULL)
static int forward_any(spion_ctx* c, const void* Q, const void* K, const void* V, const float* keypad, void* O,
                       float* lse, void* P_user) {
  TcState* s = (TcState*)c->tc;
  if (!s) return SPION_ERR_STATE;
  if (c->nnzb == 0) return SPION_ERR_SHAPE;
  void* P64 = P_user ? (s->super ? s->p64_ws : P_user) : nullptr;
  int rc = fused_forward(c, s, Q, K, V, keypad, O, lse ? lse : s->lse_ws, P64);
  if (rc || !P_user || !s->super) return rc;
  return convert_tiles(c, s, false, s->p64_ws, P_user);
}

int tc_engine_forward(spion_ctx* c, const void* Q, const void* K, const void* V, const float* keypad, void* P, void* O,
                      float* S_scratch) {
  (void)S_scratch;
  return forward_any(c, Q, K, V, keypad, O, nullptr, P);
}

int tc_engine_backward(spion_ctx* c, const void* Q, const void* K, const void* V, const void* P, const void* O,
                       const void* dO, void* dS, float* dP_scratch, void* dQ, void* dK, void* dV) {
  (void)dP_scratch;
  if (!c->tc) return SPION_ERR_STATE;
  TcState* s = (TcState*)c->tc;
  if (c->nnzb == 0) return SPION_ERR_SHAPE;
  return c->d == 64 ? run_backward<64>(c, s, Q, K, V, P, O, dO, dS, dQ, dK, dV)
                    : run_backward<32>(c, s, Q, K, V, P, O, dO, dS, dQ, dK, dV);
}

int tc_engine_forward_fused(spion_ctx* c, const void* Q, const void* K, const void* V, const float* keypad, void* O,
                            float* lse, void* P_optional) {
  return forward_any(c, Q, K, V, keypad, O, lse, P_optional);
}


int tc_engine_wait_selftest(spion_ctx* c, long long limit_cycles) {
  k_wait_selftest<<<1, 128, 0, c->stream>>>(c->status_dev, limit_cycles);
  SPION_LAUNCH_CHECK();
  c->launches += 1;
  return SPION_OK;
}
