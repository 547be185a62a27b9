// Backward of the block-sparse attention without P or dS in global memory (sm_100a, bf16, 64x64 blocks).
//
// The forward kernel (tc_fused.cu) leaves one fp32 log-sum-exp per row, lse2_i = m_i log2(e) + log2(Z_i),
// where Z_i includes the reference's term for the non-selected keys (models/block_attn.cu:65-71).  With it
//     P_ij  = exp2(s_ij scale log2(e) - pad_j log2(e) - lse2_i)                      (:72-87)
//     dS_ij = P_ij (dP_ij - delta_i) scale,   delta_i = sum_n dO_in O_in             (:107-129)
// are functions of Q, K, V, dO, O alone, so both backward kernels rebuild the tiles they need in tensor
// memory / shared memory instead of reading what the forward pass and the row kernel would have stored:
//     k_bwd_row_rc   per block row:     S = Q K^T, dP = dO V^T  ->  dS  ->  dQ = dS K;   writes delta
//     k_bwd_col_stream (tc_recompute_col.cu)
//                    per block column:  S, dP of every entry    ->  P, dS  ->  dV += P^T dO, dK += dS^T Q
// This replaces models/block_attn.cu:489-545 (two cuSPARSE SDDMMs' worth of stored values, the softmax
// backward kernel and three SpMMs) with 16 L d e bytes of traffic per (b,h) matrix and step instead of
// 16 L d e + 5 nnz p.
//
// The kernels are persistent (grid = CTAs the device holds at once, units taken with stride grid) and
// use 8 math warps: warps w and w + 4 share TMEM quadrant w & 3 and split the 64 columns of a tile in
// two halves, which the backward allows without any exchange (lse and delta are per-row inputs).
// Thread 0 issues the TMA loads' MMAs; every wait on an mbarrier is bounded.
#include <cuda.h>

#include "common.cuh"
#include "tc_tiles.cuh"

using namespace tc;

#ifdef SPION_TRACE
SPION_TRACE_SETTER(spion_debug_trace_rc)
#endif

namespace {

constexpr int RC_THREADS = 256;

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 32 consecutive bf16 values (16 packed words) of row i, columns [32 g, 32 g + 32), into a [64 x 64]
// K-major SWIZZLE_128B tile (16-byte chunk c of row i sits at chunk c ^ (i & 7)).
__device__ __forceinline__ void store_half_row_swizzled(uint32_t tile, int i, int g, const uint32_t (&w)[16]) {
#pragma unroll
  for (int cc = 0; cc < 4; ++cc) {
    const int c = g * 4 + cc;
    const uint32_t addr = tile + i * 128 + ((c ^ (i & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * cc]), "r"(w[4 * cc + 1]),
                 "r"(w[4 * cc + 2]), "r"(w[4 * cc + 3])
                 : "memory");
  }
}

// P and dS of 32 scores: s, g = raw S and dP values of one row (TMEM), lse = the row's log-sum-exp
// (log2 domain, key-padding penalty already folded in per column through kp), nds = -delta scale.
template <bool WANT_P>
__device__ __forceinline__ void p_ds_32(const uint32_t (&s)[32], const uint32_t (&g)[32], float sc2, float scale,
                                        float lse, float nds, const float* kp32, bool live, uint32_t (&wp)[16],
                                        uint32_t (&wds)[16]) {
  if (live) {
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      float h0 = lse, h1 = lse;
      if (kp32) { h0 = fmaf(kp32[j], LOG2E, lse); h1 = fmaf(kp32[j + 1], LOG2E, lse); }
      const float p0 = ex2f(fmaf(__uint_as_float(s[j]), sc2, -h0)), p1 = ex2f(fmaf(__uint_as_float(s[j + 1]), sc2, -h1));
      if (WANT_P) wp[j >> 1] = pack_bf16(p0, p1);
      wds[j >> 1] = pack_bf16(p0 * fmaf(__uint_as_float(g[j]), scale, nds), p1 * fmaf(__uint_as_float(g[j + 1]), scale, nds));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) { if (WANT_P) wp[j] = 0u; wds[j] = 0u; }
  }
}

template <int D> constexpr size_t rc_row_smem() {
  // Q | dO | K x4 | V x4 (dS tiles reuse the V buffers when a V tile is as large as a dS tile) | barriers
  return 1024 + (size_t)(2 + 2 * ROW_NCH) * OpTile<D>::BYTES + (D == 64 ? 0 : (size_t)ROW_NCH * VT_BYTES) + 128;
}

// =====================================================================================
// Row side.  Unit = (sorted block row, bh).  Rows of at most 4 blocks are one chunk: S tiles in TMEM
// columns [0,128), dP tiles in [128,256), the dQ accumulator then reuses [0,D).  Longer rows stream pairs
// of tiles over the two halves of the K / V buffers: S of a pair in [64,128), dP in [128,192), dQ
// accumulating in [0,D); the S / dP MMAs of pair c+1 are issued right after the dQ MMAs of pair c, and
// because the tensor pipe retires in issue order their arrival also tells that dQ(c) is done and its
// half of the buffers can be refilled.
template <int D, bool SUB>
__global__ void __launch_bounds__(RC_THREADS, 2) k_bwd_row_rc(const __grid_constant__ CUtensorMap tmQ,
                                                              const __grid_constant__ CUtensorMap tmK,
                                                              const __grid_constant__ CUtensorMap tmV,
                                                              const __grid_constant__ CUtensorMap tmdO,
                                                              const __nv_bfloat16* __restrict__ dOg,
                                                              const __nv_bfloat16* __restrict__ Og,
                                                              const float* __restrict__ lse_in,
                                                              const float* __restrict__ keypad,
                                                              float* __restrict__ delta_out,
                                                              __nv_bfloat16* __restrict__ dQ,
                                                              const int4* __restrict__ row_info,
                                                              const int* __restrict__ col_idx,
                                                              const uint8_t* __restrict__ submask, int L, int BH,
                                                              int nrows, int heads, float scale, int* status) {
  using T = OpTile<D>;
  constexpr int NCH = ROW_NCH;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  const uint32_t sQ = sbase;
  const uint32_t sdO = sQ + T::BYTES;
  const uint32_t sK = sdO + T::BYTES;
  const uint32_t sV = sK + NCH * T::BYTES;
  const uint32_t sDS = (D == 64) ? sV : sV + NCH * T::BYTES;          // dS tiles (the V tiles are consumed first)
  const uint32_t bars = sV + NCH * T::BYTES + (D == 64 ? 0 : NCH * VT_BYTES);
  // per half of the buffers: bar_qk (Q + K tiles), bar_ov (dO + V tiles); bar_s: S and dP MMAs, bar_o: last dQ MMA
  const uint32_t bar_qk = bars, bar_ov = bars + 16, bar_s = bars + 32, bar_o = bars + 40, slot = bars + 48;
  uint32_t* slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (slot - raw));
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q = warp & 3, g = warp >> 2;                       // TMEM quadrant, column half of the tiles
  const int hf = lane >> 4;                                    // 0: even tiles of a pair, 1: odd tiles
  const int row = q * 16 + (lane & 15);
  const int total = nrows * BH;
  constexpr uint32_t ncols = 256u;

  // Warp 0, all lanes: request chunk ch of a unit into half hb (Q and dO with the first chunk).
  auto issue_loads = [&](const RowRec& R, int bh, int ch) {
    const int CH = R.chunk();
    const int t0 = ch * CH, nt = min(CH, R.nblk - t0);
    const int hb = R.single() ? 0 : (ch & 1), b0 = 2 * hb;
    const OpPos pos = op_pos(bh, L, heads, D);
    if (lane == 0) {
      mbar_expect_tx(bar_qk + 8 * hb, (ch == 0 ? T::BYTES : 0) + nt * T::BYTES);
      mbar_expect_tx(bar_ov + 8 * hb, (ch == 0 ? T::BYTES : 0) + nt * T::BYTES);
    }
    __syncwarp();
    if (lane == 0 && ch == 0) tma_load_2d(sQ, &tmQ, bar_qk + 8 * hb, pos.x0, pos.row0 + R.r * BS);
    if (lane == 16 && ch == 0) tma_load_2d(sdO, &tmdO, bar_ov + 8 * hb, pos.x0, pos.row0 + R.r * BS);
    if (lane >= 1 && lane <= nt)
      tma_load_2d(sK + (b0 + lane - 1) * T::BYTES, &tmK, bar_qk + 8 * hb, pos.x0, pos.row0 + R.col(t0 + lane - 1, col_idx) * BS);
    if (lane >= 9 && lane < 9 + nt)
      tma_load_2d(sV + (b0 + lane - 9) * T::BYTES, &tmV, bar_ov + 8 * hb, pos.x0, pos.row0 + R.col(t0 + lane - 9, col_idx) * BS);
  };
  auto first_loads = [&](const RowRec& R, int bh) {
    if (R.nblk > 0) issue_loads(R, bh, 0);
    if (!R.single() && R.nchunks() > 1) issue_loads(R, bh, 1);
  };

  int u = blockIdx.x;
  RowRec R;
  int bh = 0;
  if (u < total) { const int rank = u / BH; R = RowRec(row_info[rank]); bh = u - rank * BH; }

  if (warp == 0) {
    if (lane == 0) {
      s_abort = *reinterpret_cast<volatile int*>(status);
      for (int i = 0; i < 4; ++i) mbar_init(bar_qk + 8 * i, 1);      // bar_qk[2], bar_ov[2]
      mbar_init(bar_s, 1);
      mbar_init(bar_o, 1);
      fence_barrier_init();
    }
    __syncwarp();
    if (s_abort == 0 && u < total) first_loads(R, bh);
  }
  __syncthreads();
  if (s_abort != 0) return;
  if (warp == 0) {
    tmem_alloc(slot, ncols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot_ptr;
  const uint32_t t_lane = tmem + ((uint32_t)(q * 32) << 16);
  constexpr uint32_t IDESC_S = make_idesc_bf16(64, 64, 0, 0);
  constexpr uint32_t IDESC_Q = make_idesc_bf16(64, D, 0, 1);
  const float sc2 = scale * LOG2E;
  uint32_t pqk = 0, pov = 0, ps = 0, po = 0;                    // pqk / pov: one bit per half, thread 0 only
  bool ok = true;

  for (; u < total && ok; u += gridDim.x) {
    const int un = u + (int)gridDim.x;
    const bool has_next = un < total;
    RowRec Rn;
    int bhn = 0;
    if (has_next) { const int rank = un / BH; Rn = RowRec(row_info[rank]); bhn = un - rank * BH; }

    const int rp = R.rp, nblk = R.nblk, r = R.r;
    const bool single = R.single();
    const OpPos pos = op_pos(bh, L, heads, D);
    const float* kp = keypad ? keypad + (size_t)bh * L : nullptr;
    // 32-wide masks: bit (2*(row/32) + col/32) of submask[block] tells whether that quarter is selected
    auto quarter_ok = [&](int blk) -> bool { return !SUB || ((submask[blk] >> ((q >> 1) * 2 + g)) & 1); };

    // tid 0: S and dP MMAs of chunk ch; pair p of the chunk goes to columns colS + 64 p and colP + 64 p
    auto issue_sdp = [&](int ch, uint32_t colS, uint32_t colP) -> bool {
      const int CH = single ? NCH : 2;
      const int t0 = ch * CH, nt = min(CH, nblk - t0);
      const int hb = single ? 0 : (ch & 1), b0 = 2 * hb;
      if (!mbar_wait(bar_qk + 8 * hb, (pqk >> hb) & 1)) { report(status, ERR_LOAD_WAIT); return false; }
      pqk ^= 1u << hb;
      tc_fence_after();
      for (int t = 0; t < nt; ++t) {
        const uint32_t d_addr = tmem + ((uint32_t)((t & 1) * 16) << 16) + colS + (uint32_t)(t >> 1) * 64u;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_bf16(d_addr, T::kmajor(sQ, kk), T::kmajor(sK + (b0 + t) * T::BYTES, kk), IDESC_S, kk > 0);
      }
      if (!mbar_wait(bar_ov + 8 * hb, (pov >> hb) & 1)) { report(status, ERR_LOAD_WAIT); return false; }
      pov ^= 1u << hb;
      tc_fence_after();
      for (int t = 0; t < nt; ++t) {
        const uint32_t d_addr = tmem + ((uint32_t)((t & 1) * 16) << 16) + colP + (uint32_t)(t >> 1) * 64u;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_bf16(d_addr, T::kmajor(sdO, kk), T::kmajor(sV + (b0 + t) * T::BYTES, kk), IDESC_S, kk > 0);
      }
      mma_commit(bar_s);
      return true;
    };
    // tid 0: dQ += dS K for the tiles of a chunk (every tile into the one accumulator at lane offset 0)
    auto issue_dq = [&](int hb, int nt, bool first_chunk) {
      const int b0 = 2 * hb;
      for (int t = 0; t < nt; ++t) {
        const uint32_t first = (first_chunk && t == 0) ? 0u : 1u;
#pragma unroll
        for (int kk = 0; kk < BS / 16; ++kk)
          mma_bf16(tmem, ValTile::kmajor(sDS + (b0 + t) * VT_BYTES, kk), T::mnmajor(sK + (b0 + t) * T::BYTES, kk), IDESC_Q,
                   (kk > 0) ? 1u : first);
      }
    };

    float delta = 0.f;
    if (nblk > 0) {
      if (tid == 0) issue_sdp(0, single ? 0u : 64u, 128u);
      // delta_i = sum_n dO_in O_in: the two owners of a row take one half of the head dimension each
      {
        const size_t off = (size_t)(pos.row0 + r * BS + row) * pos.ld + pos.x0 + hf * (D / 2);
        const uint4* a4 = reinterpret_cast<const uint4*>(dOg + off);
        const uint4* b4 = reinterpret_cast<const uint4*>(Og + off);
        float acc = 0.f;
#pragma unroll
        for (int e = 0; e < D / 16; ++e) {
          const uint4 a = a4[e], b = b4[e];
          acc += bf16_lo(a.x) * bf16_lo(b.x) + bf16_hi(a.x) * bf16_hi(b.x) + bf16_lo(a.y) * bf16_lo(b.y) +
                 bf16_hi(a.y) * bf16_hi(b.y) + bf16_lo(a.z) * bf16_lo(b.z) + bf16_hi(a.z) * bf16_hi(b.z) +
                 bf16_lo(a.w) * bf16_lo(b.w) + bf16_hi(a.w) * bf16_hi(b.w);
        }
        delta = acc + __shfl_xor_sync(0xffffffffu, acc, 16);
      }
      const float lse = lse_in[(size_t)bh * L + r * BS + row];
      const float nds = -delta * scale;
      const int n = single ? 1 : R.nchunks();
      for (int c = 0; c < n && ok; ++c) {
        const int CH = single ? NCH : 2;
        const int hb = single ? 0 : (c & 1), t0 = c * CH, nt = min(CH, nblk - t0);
        // S(c) and dP(c) have arrived; in a long row that also means dQ(c-1) is complete
        if (!__syncthreads_and(mbar_wait(bar_s, ps))) { if (tid == 0) report(status, ERR_MMA_WAIT); ok = false; break; }
        ps ^= 1u;
        tc_fence_after();
        if (warp == 0 && c >= 1 && c + 1 < n) issue_loads(R, bh, c + 1);      // the other half is free again
        const uint32_t colS = single ? 0u : 64u;
        const int npairs = single ? 2 : 1;
        for (int p = 0; p < npairs; ++p) {
          const int t = 2 * p + hf;
          const bool mine = t < nt;
          const int cblk = mine ? R.col(t0 + t, col_idx) : 0;
          uint32_t sv[32], gv[32], wp[16], wds[16];
          tmem_ld32(t_lane + colS + p * 64 + g * 32, sv);
          tmem_ld32(t_lane + 128u + p * 64 + g * 32, gv);
          tmem_ld_wait();
          if (mine) {
            p_ds_32<false>(sv, gv, sc2, scale, lse, nds, kp ? kp + cblk * BS + g * 32 : nullptr, quarter_ok(rp + t0 + t), wp, wds);
            store_half_row_swizzled(sDS + (2 * hb + t) * VT_BYTES, row, g, wds);
          }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
          tc_fence_after();
          issue_dq(hb, nt, c == 0);
          if (c + 1 < n) issue_sdp(c + 1, 64u, 128u);
          else mma_commit(bar_o);
        }
      }
      if (ok) {
        if (!__syncthreads_and(mbar_wait(bar_o, po))) { if (tid == 0) report(status, ERR_MMA2_WAIT); ok = false; }
        po ^= 1u;
      }
      tc_fence_after();
    }
    if (ok && warp == 0 && has_next) first_loads(Rn, bhn);         // every buffer of this unit is free
    if (ok) {
      if (g == 0 && hf == 0) delta_out[(size_t)bh * L + r * BS + row] = delta;
      // accumulator rows sit in lanes 0-15 of every quadrant; the two warps of a quadrant take half the columns each
      __nv_bfloat16* dst = dQ + (size_t)(pos.row0 + r * BS + row) * pos.ld + pos.x0 + g * (D / 2);
      if (D == 64) {
        uint32_t v[32];
        if (nblk > 0) { tmem_ld32(t_lane + g * 32, v); tmem_ld_wait(); }
        else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
        }
        if (hf == 0) {
#pragma unroll
          for (int j = 0; j < 32; j += 8)
            *reinterpret_cast<uint4*>(dst + j) =
                make_uint4(pack_bf16(__uint_as_float(v[j]), __uint_as_float(v[j + 1])),
                           pack_bf16(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])),
                           pack_bf16(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5])),
                           pack_bf16(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7])));
        }
      } else {
        uint32_t v[16];
        if (nblk > 0) { tmem_ld16(t_lane + g * 16, v); tmem_ld_wait(); }
        else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0u;
        }
        if (hf == 0) {
#pragma unroll
          for (int j = 0; j < 16; j += 8)
            *reinterpret_cast<uint4*>(dst + j) =
                make_uint4(pack_bf16(__uint_as_float(v[j]), __uint_as_float(v[j + 1])),
                           pack_bf16(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])),
                           pack_bf16(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5])),
                           pack_bf16(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7])));
        }
      }
    }
    tc_fence_before();
    __syncthreads();                                               // the next unit's MMAs overwrite these columns
    tc_fence_after();
    R = Rn;
    bh = bhn;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, ncols);
}

constexpr size_t MM_SMEM(int tile_bytes) { return 1024 + (size_t)2 * 2 * 2 * tile_bytes + 128; }

// =====================================================================================
// Head / batch mean of the attention probabilities without a stored P (models/model_transformer.py:137):
//     A[i, j] = (1 / BH) sum_bh exp2(s_ij(bh) scale log2(e) - pad_j log2(e) - lse2_i(bh))   on the selected blocks.
// One CTA per selected block (r, c); the (b,h) matrices are taken two at a time (first in lanes 0-15 of
// every TMEM quadrant, second in lanes 16-31) through two stages: while the probabilities of one pair are
// summed in registers, the S tiles of the next pair are already being computed and the tiles of the pair
// after that are on their way.  Every thread keeps the 64 running sums of its row.
template <int D, bool SUB>
__global__ void __launch_bounds__(128) k_mean_map_rc(const __grid_constant__ CUtensorMap tmQ,
                                                     const __grid_constant__ CUtensorMap tmK,
                                                     const float* __restrict__ lse_in, const float* __restrict__ keypad,
                                                     float* __restrict__ A, const int* __restrict__ blk_row,
                                                     const int* __restrict__ col_idx, const uint8_t* __restrict__ submask,
                                                     int L, int BH, int heads, float scale, int* status) {
  using T = OpTile<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  // stage st: Q tiles of the pair at sbase + st*4*T + {0, T}, K tiles at + {2T, 3T}
  const uint32_t bars = sbase + 8 * T::BYTES;
  const uint32_t bar_full = bars, bar_s = bars + 16, slot = bars + 32;
  uint32_t* slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (slot - raw));
  __shared__ int s_abort;

  const int tid = threadIdx.x, q = tid >> 5, lane = tid & 31;
  const int hf = lane >> 4, row = q * 16 + (lane & 15);
  const int blk = blockIdx.x;
  const int r = blk_row[blk], c = col_idx[blk];
  const int npair = (BH + 1) >> 1;

  auto issue = [&](int it) {                                     // warp 0, all lanes
    const int st = it & 1;
    const int cnt = min(2, BH - 2 * it);
    const uint32_t base = sbase + st * 4 * T::BYTES;
    if (lane == 0) mbar_expect_tx(bar_full + 8 * st, cnt * 2 * T::BYTES);
    __syncwarp();
    if (lane < 2 * cnt) {
      const int hb = lane >> 1;
      const OpPos pos = op_pos(2 * it + hb, L, heads, D);
      if (lane & 1) tma_load_2d(base + (2 + hb) * T::BYTES, &tmK, bar_full + 8 * st, pos.x0, pos.row0 + c * BS);
      else tma_load_2d(base + hb * T::BYTES, &tmQ, bar_full + 8 * st, pos.x0, pos.row0 + r * BS);
    }
  };

  if (q == 0) {
    if (lane == 0) {
      s_abort = *reinterpret_cast<volatile int*>(status);
      for (int i = 0; i < 4; ++i) mbar_init(bar_full + 8 * i, 1);     // bar_full[2], bar_s[2]
      fence_barrier_init();
    }
    __syncwarp();
    if (s_abort == 0) {
      issue(0);
      if (npair > 1) issue(1);
    }
  }
  __syncthreads();
  if (s_abort != 0) return;
  if (q == 0) {
    tmem_alloc(slot, 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot_ptr;
  const uint32_t t_lane = tmem + ((uint32_t)(q * 32) << 16);
  constexpr uint32_t IDESC_S = make_idesc_bf16(64, 64, 0, 0);
  const float sc2 = scale * LOG2E;
  bool ok = true;

  // tid 0: S tiles of pair `it` into columns 64 (it & 1)
  auto issue_s = [&](int it) -> bool {
    const int st = it & 1;
    const int cnt = min(2, BH - 2 * it);
    if (!mbar_wait(bar_full + 8 * st, (uint32_t)(it >> 1) & 1u)) { report(status, ERR_LOAD_WAIT); return false; }
    tc_fence_after();
    const uint32_t base = sbase + st * 4 * T::BYTES;
    for (int hb = 0; hb < cnt; ++hb) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk)
        mma_bf16(tmem + ((uint32_t)(hb * 16) << 16) + (uint32_t)st * 64u, T::kmajor(base + hb * T::BYTES, kk),
                 T::kmajor(base + (2 + hb) * T::BYTES, kk), IDESC_S, kk > 0);
    }
    mma_commit(bar_s + 8 * st);
    return true;
  };

  float acc[64];
#pragma unroll
  for (int j = 0; j < 64; ++j) acc[j] = 0.f;
  const bool live0 = !SUB || ((submask[blk] >> ((q >> 1) * 2 + 0)) & 1);
  const bool live1 = !SUB || ((submask[blk] >> ((q >> 1) * 2 + 1)) & 1);

  if (tid == 0) issue_s(0);
  for (int it = 0; it < npair && ok; ++it) {
    const int st = it & 1;
    if (tid == 0 && it + 1 < npair) issue_s(it + 1);
    if (!__syncthreads_and(mbar_wait(bar_s + 8 * st, (uint32_t)(it >> 1) & 1u))) {
      if (tid == 0) report(status, ERR_MMA_WAIT);
      ok = false;
      break;
    }
    tc_fence_after();
    if (q == 0 && it + 2 < npair) issue(it + 2);                  // the MMAs have consumed this stage's tiles
    const int bh = 2 * it + hf;
    const bool mine = bh < BH;
    const float lse = mine ? lse_in[(size_t)bh * L + r * BS + row] : 0.f;
    const float* kp = (keypad && mine) ? keypad + (size_t)bh * L + c * BS : nullptr;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t v[32];
      tmem_ld32(t_lane + (uint32_t)st * 64u + half * 32, v);
      tmem_ld_wait();
      if (mine && (half ? live1 : live0)) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float h = kp ? fmaf(kp[half * 32 + j], LOG2E, lse) : lse;
          acc[half * 32 + j] += ex2f(fmaf(__uint_as_float(v[j]), sc2, -h));
        }
      }
    }
    tc_fence_before();
    __syncthreads();                                               // pair it + 2 overwrites these columns
    tc_fence_after();
  }
  if (ok) {
    const float inv = 1.0f / (float)BH;
    float* dst = A + (size_t)(r * BS + row) * L + c * BS;
#pragma unroll
    for (int j = 0; j < 64; j += 4) {
      float4 o;
      o.x = (acc[j] + __shfl_xor_sync(0xffffffffu, acc[j], 16)) * inv;
      o.y = (acc[j + 1] + __shfl_xor_sync(0xffffffffu, acc[j + 1], 16)) * inv;
      o.z = (acc[j + 2] + __shfl_xor_sync(0xffffffffu, acc[j + 2], 16)) * inv;
      o.w = (acc[j + 3] + __shfl_xor_sync(0xffffffffu, acc[j + 3], 16)) * inv;
      if (hf == 0) *reinterpret_cast<float4*>(dst + j) = o;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (q == 0) tmem_dealloc(tmem, 128);
}

}  // namespace

namespace tc {

// Shared-memory opt-in of the recompute kernels and how many CTAs of each one SM holds (256 of the 512
// tensor-memory columns each: at most two).
template <int D>
static int rc_attrs(TcState* s, int device) {
  int n = 0, rc;
  s->rc_row_ctas = 1 << 30;
#define SPION_RC_ATTR(SB)                                                                                                   \
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_bwd_row_rc<D, SB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)rc_row_smem<D>())); \
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_mean_map_rc<D, SB>, cudaFuncAttributeMaxDynamicSharedMemorySize,                    \
                                      (int)MM_SMEM(OpTile<D>::BYTES)));                                                     \
  if ((rc = resident_ctas(k_bwd_row_rc<D, SB>, device, RC_THREADS, rc_row_smem<D>(), 256, &n))) return rc;                  \
  s->rc_row_ctas = n < s->rc_row_ctas ? n : s->rc_row_ctas;                                                                 \

  SPION_RC_ATTR(false)
  SPION_RC_ATTR(true)
#undef SPION_RC_ATTR
  return SPION_OK;
}

int recompute_set_attrs(TcState* s, int d, int device) {
  int rc = d == 64 ? rc_attrs<64>(s, device) : rc_attrs<32>(s, device);
  return rc ? rc : col_stream_set_attrs(d);
}

template <int D>
static int rc_backward(spion_ctx* c, TcState* s, const void* Q, const void* K, const void* V, const void* O, const void* dO,
                       const float* lse, const float* keypad, void* dQ, void* dK, void* dV) {
  const TcView vw = tc_view(c, s);
  CUtensorMap mq, mk, mv, mdo;
  int rc;
  if ((rc = make_operand_map(c, s, &mq, Q, D)) || (rc = make_operand_map(c, s, &mk, K, D)) ||
      (rc = make_operand_map(c, s, &mv, V, D)) || (rc = make_operand_map(c, s, &mdo, dO, D)))
    return rc;
  prof_mark(c, -1);
  const long long total = (long long)c->BH * vw.nb;
  const long long row_cap = (long long)s->sms * s->rc_row_ctas;
  const int grid_row = (int)(total < row_cap ? total : row_cap);
#define SPION_RC_LAUNCH(SB)                                                                                              \
  k_bwd_row_rc<D, SB><<<grid_row, RC_THREADS, rc_row_smem<D>(), c->stream>>>(                                             \
      mq, mk, mv, mdo, (const __nv_bfloat16*)dO, (const __nv_bfloat16*)O, lse, keypad, s->delta_ws, (__nv_bfloat16*)dQ,   \
      vw.row_info, vw.col_idx, vw.submask, c->L, c->BH, vw.nb, c->heads, c->scale, c->status_dev);                        \
  SPION_LAUNCH_CHECK();                                                                                                  \
  prof_mark(c, SPION_STAGE_BWD_ROW_RC);
  if (vw.submask) { SPION_RC_LAUNCH(true) } else { SPION_RC_LAUNCH(false) }
#undef SPION_RC_LAUNCH
  if ((rc = col_stream_backward(c, s, mq, mk, mv, mdo, lse, keypad, dK, dV))) return rc;
  prof_mark(c, SPION_STAGE_BWD_COL_RC);
  c->launches += 2;
  return SPION_OK;
}

int recompute_backward(spion_ctx* c, TcState* s, const void* Q, const void* K, const void* V, const void* O,
                       const void* dO, const float* lse, const float* keypad, void* dQ, void* dK, void* dV) {
  return c->d == 64 ? rc_backward<64>(c, s, Q, K, V, O, dO, lse, keypad, dQ, dK, dV)
                    : rc_backward<32>(c, s, Q, K, V, O, dO, lse, keypad, dQ, dK, dV);
}

template <int D>
static int rc_mean_map(spion_ctx* c, TcState* s, const void* Q, const void* K, const float* lse, const float* keypad,
                       float* A) {
  const TcView vw = tc_view(c, s);
  CUtensorMap mq, mk;
  int rc;
  if ((rc = make_operand_map(c, s, &mq, Q, D)) || (rc = make_operand_map(c, s, &mk, K, D))) return rc;
  SPION_CUDA_TRY(cudaMemsetAsync(A, 0, (size_t)c->L * c->L * sizeof(float), c->stream));
  const int32_t* blk_row = s->super ? s->blk_row64 : c->blk_row;
  if (vw.submask)
    k_mean_map_rc<D, true><<<vw.nnzb, 128, MM_SMEM(OpTile<D>::BYTES), c->stream>>>(
        mq, mk, lse, keypad, A, blk_row, vw.col_idx, vw.submask, c->L, c->BH, c->heads, c->scale, c->status_dev);
  else
    k_mean_map_rc<D, false><<<vw.nnzb, 128, MM_SMEM(OpTile<D>::BYTES), c->stream>>>(
        mq, mk, lse, keypad, A, blk_row, vw.col_idx, vw.submask, c->L, c->BH, c->heads, c->scale, c->status_dev);
  SPION_LAUNCH_CHECK();
  c->launches += 1;
  return SPION_OK;
}

int recompute_mean_map(spion_ctx* c, TcState* s, const void* Q, const void* K, const float* lse, const float* keypad,
                       float* A) {
  return c->d == 64 ? rc_mean_map<64>(c, s, Q, K, lse, keypad, A) : rc_mean_map<32>(c, s, Q, K, lse, keypad, A);
}

}  // namespace tc
