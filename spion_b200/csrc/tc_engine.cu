// Tensor-core engine (sm_100a): block-sparse attention on bf16 block tiles with TMA-fed
// tcgen05.mma, accumulators in tensor memory (TMEM), fp32 softmax math in the epilogues.
//
// Replaces, for the native (block-tile) API, the reference's cuSPARSE calls and SIMT softmax
// kernels (models/block_attn.cu:453-545):
//   k_fwd_fused (tc_fused.cu)  S = Q K^T on the mask, sparse row softmax, O = P V        (:459-478)
//   k_bwd_row                  dP = dO V^T on the mask, softmax backward -> dS, dQ = dS K  (:498-516)
//   k_bwd_col                  dK = dS^T Q and dV = P^T dO in one pass over a block column (:526, :536)
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
// All three kernels are persistent: the grid is the number of CTAs the device holds at once, every
// CTA initialises its barriers and allocates its tensor memory once and then walks its share of the
// work units, asking for the next unit's tiles while the current unit's results are written.
//
// All waits on mbarriers are bounded; on a time-out the CTA records a code in the context's
// status word, frees its TMEM and returns.
#include <cuda.h>

#include "common.cuh"
#include "tc_tiles.cuh"

using namespace tc;

#ifdef SPION_TRACE
SPION_TRACE_SETTER(spion_debug_trace_engine)
#endif

namespace {

constexpr int ROW_THREADS = 128;
constexpr int COL_THREADS = 160;          // warp 0: loads + MMA issue; warps 1-4: one TMEM quadrant each
constexpr int COL_NST = 2;                // ring stages of the column kernel (one entry of a column each)

// =====================================================================================
// Backward, row side.  Unit = (sorted block row, bh).  Per unit: dP tiles (dO V^T) in TMEM, P tiles by
// TMA, dS = P (dP - delta) scale written over P in shared memory, stored by TMA and used in place for
// dQ = dS K; the K tiles arrive in the V buffers as soon as the dP MMAs have consumed V.
// Rows of at most 4 blocks are one chunk (dP in all 128 columns, the dQ accumulator then reuses the
// first 64).  Longer rows stream pairs of tiles over the two halves of the buffers: dP of a pair in
// columns [64,128), dQ accumulating in [0,64); the dP MMAs of pair c+1 are issued right after the dQ
// MMAs of pair c, and because the tensor pipe retires in issue order the arrival of dP(c+1) also
// tells that dQ(c) is done and its half of the buffers can be refilled.
template <int D>
__global__ void __launch_bounds__(ROW_THREADS, 3) k_bwd_row(const __grid_constant__ CUtensorMap tmdO,
                                                            const __grid_constant__ CUtensorMap tmV,
                                                            const __grid_constant__ CUtensorMap tmK,
                                                            const __grid_constant__ CUtensorMap tmP,
                                                            const __grid_constant__ CUtensorMap tmdS,
                                                            const __nv_bfloat16* __restrict__ dOg,
                                                            const __nv_bfloat16* __restrict__ Og,
                                                            __nv_bfloat16* __restrict__ dQ,
                                                            const int4* __restrict__ row_info,
                                                            const int* __restrict__ col_idx, int L, int nnzb, int BH,
                                                            int nrows, int heads, float scale, int* status) {
  using T = OpTile<D>;
  constexpr int NCH = ROW_NCH;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  const uint32_t sA = sbase;                                   // dO tile
  const uint32_t sB = sA + T::BYTES;                           // V tiles, then K tiles
  const uint32_t sP = sB + NCH * T::BYTES;                     // P tiles in, dS tiles out
  const uint32_t bars = sP + NCH * VT_BYTES;
  // per half of the buffers: bar_v (dO + V tiles), bar_p (P tiles), bar_k (K tiles); bar_s: dP MMAs, bar_o: last dQ MMA
  const uint32_t bar_v = bars, bar_p = bars + 16, bar_k = bars + 32, bar_s = bars + 48, bar_o = bars + 56, slot = bars + 64;
  uint32_t* slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (slot - raw));
  __shared__ int s_abort;

  const int tid = threadIdx.x, q = tid >> 5, lane = tid & 31;
  const int hf = lane >> 4;
  const int row = q * 16 + (lane & 15);
  const int total = nrows * BH;
  constexpr uint32_t ncols = 128u;

  // Warp 0, all lanes: request chunk ch of a unit (dO with the first chunk; V and P tiles) into half hb.
  auto issue_loads = [&](const RowRec& R, int bh, int ch) {
    const int CH = R.chunk();
    const int t0 = ch * CH, nt = min(CH, R.nblk - t0);
    const int hb = R.single() ? 0 : (ch & 1), b0 = 2 * hb;
    const OpPos pos = op_pos(bh, L, heads, D);
    if (lane == 0) {
      mbar_expect_tx(bar_v + 8 * hb, (ch == 0 ? T::BYTES : 0) + nt * T::BYTES);
      mbar_expect_tx(bar_p + 8 * hb, nt * VT_BYTES);
    }
    __syncwarp();
    if (lane == 0 && ch == 0) tma_load_2d(sA, &tmdO, bar_v + 8 * hb, pos.x0, pos.row0 + R.r * BS);
    if (lane >= 1 && lane <= nt)
      tma_load_2d(sB + (b0 + lane - 1) * T::BYTES, &tmV, bar_v + 8 * hb, pos.x0, pos.row0 + R.col(t0 + lane - 1, col_idx) * BS);
    if (lane >= 9 && lane < 9 + nt)
      tma_load_2d(sP + (b0 + lane - 9) * VT_BYTES, &tmP, bar_p + 8 * hb, 0, (int)(((size_t)bh * nnzb + R.rp + t0 + lane - 9) * BS));
  };
  auto first_loads = [&](const RowRec& R, int bh) {
    if (R.nblk > 0) issue_loads(R, bh, 0);
    if (!R.single() && R.nchunks() > 1) issue_loads(R, bh, 1);
  };

  int u = blockIdx.x;
  RowRec R;
  int bh = 0;
  if (u < total) { const int rank = u / BH; R = RowRec(row_info[rank]); bh = u - rank * BH; }

  if (q == 0) {
    if (lane == 0) {
      s_abort = *reinterpret_cast<volatile int*>(status);
      for (int i = 0; i < 6; ++i) mbar_init(bar_v + 8 * i, 1);      // bar_v[2], bar_p[2], bar_k[2]
      mbar_init(bar_s, 1);
      mbar_init(bar_o, 1);
      fence_barrier_init();
    }
    __syncwarp();
    if (s_abort == 0 && u < total) first_loads(R, bh);
  }
  __syncthreads();
  if (s_abort != 0) return;
  if (q == 0) {
    tmem_alloc(slot, ncols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot_ptr;
  const uint32_t t_lane = tmem + ((uint32_t)(q * 32) << 16);
  constexpr uint32_t IDESC_P = make_idesc_bf16(64, 64, 0, 0);
  constexpr uint32_t IDESC_Q = make_idesc_bf16(64, D, 0, 1);
  // parities run on across units.  pv, pk: one bit per half, thread 0 only; pp (one bit per half), ps, po: every thread
  uint32_t pv = 0, pk = 0, pp = 0, ps = 0, po = 0;
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

    // tid 0: dP MMAs of chunk ch (its dO / V tiles were requested earlier), pair p of the chunk in columns col0 + 64 p
    auto issue_dp = [&](int ch, uint32_t col0) -> bool {
      const int CH = single ? NCH : 2;
      const int t0 = ch * CH, nt = min(CH, nblk - t0);
      const int hb = single ? 0 : (ch & 1), b0 = 2 * hb;
      if (!mbar_wait(bar_v + 8 * hb, (pv >> hb) & 1)) { report(status, ERR_LOAD_WAIT); return false; }
      pv ^= 1u << hb;
      tc_fence_after();
      for (int t = 0; t < nt; ++t) {
        const uint32_t d_addr = tmem + ((uint32_t)((t & 1) * 16) << 16) + col0 + (uint32_t)(t >> 1) * 64u;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_bf16(d_addr, T::kmajor(sA, kk), T::kmajor(sB + (b0 + t) * T::BYTES, kk), IDESC_P, kk > 0);
      }
      mma_commit(bar_s);
      return true;
    };
    // warp 0, all lanes: the dP MMAs have consumed the V tiles of this chunk: bring K into the same buffers
    auto issue_k = [&](int hb, int t0, int nt) {
      if (lane == 0) mbar_expect_tx(bar_k + 8 * hb, nt * T::BYTES);
      __syncwarp();
      if (lane < nt)
        tma_load_2d(sB + (2 * hb + lane) * T::BYTES, &tmK, bar_k + 8 * hb, pos.x0, pos.row0 + R.col(t0 + lane, col_idx) * BS);
    };
    // dS = P (dP scale - delta scale), in place over the P tiles b0 + t; pair p of the chunk sits in columns colbase + 64 p
    auto ds_math = [&](uint32_t colbase, int b0, int nt, int npairs, float nds) {
      for (int p = 0; p < npairs; ++p) {
        const int t = 2 * p + hf;
        const bool mine = t < nt;
        const uint32_t tile = sP + (b0 + t) * VT_BYTES;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t v[32];
          tmem_ld32(t_lane + colbase + p * 64 + half * 32, v);
          tmem_ld_wait();
          if (mine) {
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
              const int c = half * 4 + cc;
              const uint32_t addr = tile + row * 128 + ((c ^ (row & 7)) << 4);
              uint32_t w[4];
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr) : "memory");
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float p0 = bf16_lo(w[e]), p1 = bf16_hi(w[e]);
                const float g0 = __uint_as_float(v[cc * 8 + 2 * e]), g1 = __uint_as_float(v[cc * 8 + 2 * e + 1]);
                w[e] = pack_bf16(p0 * fmaf(g0, scale, nds), p1 * fmaf(g1, scale, nds));
              }
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
            }
          }
        }
      }
    };
    // tid 0: store the dS tiles of a chunk and issue dQ += dS K (every tile into the one accumulator at lane offset 0)
    auto issue_dq = [&](int hb, int t0, int nt, bool first_chunk) -> bool {
      const int b0 = 2 * hb;
      for (int t = 0; t < nt; ++t)
        tma_store_2d(&tmdS, sP + (b0 + t) * VT_BYTES, 0, (int)(((size_t)bh * nnzb + rp + t0 + t) * BS));
      bulk_commit();
      if (!mbar_wait(bar_k + 8 * hb, (pk >> hb) & 1)) { report(status, ERR_LOAD_WAIT); return false; }
      pk ^= 1u << hb;
      tc_fence_after();
      for (int t = 0; t < nt; ++t) {
        const uint32_t first = (first_chunk && t == 0) ? 0u : 1u;
#pragma unroll
        for (int kk = 0; kk < BS / 16; ++kk)
          mma_bf16(tmem, ValTile::kmajor(sP + (b0 + t) * VT_BYTES, kk), T::mnmajor(sB + (b0 + t) * T::BYTES, kk), IDESC_Q,
                   (kk > 0) ? 1u : first);
      }
      return true;
    };

    if (nblk > 0) {
      if (tid == 0) issue_dp(0, single ? 0u : 64u);
      // delta_i = sum_n dO_in O_in: the two owners of a row take one half of the head dimension each
      float delta;
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
      const float nds = -delta * scale;
      const int n = single ? 1 : R.nchunks();
      for (int c = 0; c < n && ok; ++c) {
        const int CH = single ? NCH : 2;
        const int hb = single ? 0 : (c & 1), t0 = c * CH, nt = min(CH, nblk - t0);
        // dP(c) has arrived; in a long row that also means dQ(c-1) is complete
        if (!__syncthreads_and(mbar_wait(bar_s, ps))) { if (tid == 0) report(status, ERR_MMA_WAIT); ok = false; break; }
        ps ^= 1u;
        tc_fence_after();
        if (q == 0) {
          issue_k(hb, t0, nt);
          if (c >= 1 && c + 1 < n) {                               // the other half is free: it takes chunk c+1
            if (lane == 0) bulk_wait_read_all();                   // once the dS stores of chunk c-1 have read it
            __syncwarp();
            issue_loads(R, bh, c + 1);
          }
        }
        if (!__syncthreads_and(mbar_wait(bar_p + 8 * hb, (pp >> hb) & 1))) { if (tid == 0) report(status, ERR_LOAD_WAIT); ok = false; break; }
        pp ^= 1u << hb;
        ds_math(single ? 0u : 64u, 2 * hb, nt, single ? 2 : 1, nds);
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (tid == 0 && issue_dq(hb, t0, nt, c == 0)) {
          if (c + 1 < n) issue_dp(c + 1, 64u);
          else mma_commit(bar_o);
        }
      }
      if (ok) {
        if (!__syncthreads_and(mbar_wait(bar_o, po))) { if (tid == 0) report(status, ERR_MMA2_WAIT); ok = false; }
        po ^= 1u;
      }
      tc_fence_after();
    }
    if (ok && q == 0 && has_next) {                                // every buffer of this unit is free
      if (lane == 0) bulk_wait_read_all();
      __syncwarp();
      first_loads(Rn, bhn);
    }
    if (ok) {
      // the accumulator rows sit in lanes 0-15 of every quadrant: those lanes write the whole row
      __nv_bfloat16* dst = dQ + (size_t)(pos.row0 + r * BS + row) * pos.ld + pos.x0;
#pragma unroll
      for (int h = 0; h < D / 32; ++h) {
        uint32_t v[32];
        if (nblk > 0) {
          tmem_ld32(t_lane + h * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
        }
        if (hf == 0) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 pk4;
            pk4.x = pack_bf16(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
            pk4.y = pack_bf16(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
            pk4.z = pack_bf16(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
            pk4.w = pack_bf16(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
            *reinterpret_cast<uint4*>(dst + h * 32 + j) = pk4;
          }
        }
      }
    }
    tc_fence_before();
    __syncthreads();                                               // the next unit's dP MMAs overwrite these columns
    tc_fence_after();
    R = Rn;
    bh = bhn;
  }
  if (tid == 0) bulk_wait_read_all();
  tc_fence_before();
  __syncthreads();
  if (q == 0) tmem_dealloc(tmem, ncols);
}

// =====================================================================================
// Backward, column side.  Unit = (block column c, bh):
//     dK[c*64.., :] = sum_r dS(r, c)^T Q[r*64.., :]        dV[c*64.., :] = sum_r P(r, c)^T dO[r*64.., :]
// The value tiles are read as MN-major A operands, so no transposed copies exist anywhere.
// Warp 0 feeds a ring of COL_NST stages (one entry of a column each: dS, Q, P, dO tiles) and issues the
// MMAs; the ring runs on across the units of the CTA, so the first tiles of the next column load while
// the current one finishes.  The two accumulators of a unit share 64 TMEM columns (dK in lanes 0-15 of
// every quadrant, dV in lanes 16-31) and units alternate between two such buffers: warps 1-4 (TMEM
// quadrant = warp & 3) turn buffer j & 1 into output rows while warp 0 already accumulates the next unit
// into the other one.
template <int D>
__global__ void __launch_bounds__(COL_THREADS) k_bwd_col(const __grid_constant__ CUtensorMap tmdS,
                                                         const __grid_constant__ CUtensorMap tmP,
                                                         const __grid_constant__ CUtensorMap tmQ,
                                                         const __grid_constant__ CUtensorMap tmdO,
                                                         __nv_bfloat16* __restrict__ dK, __nv_bfloat16* __restrict__ dV,
                                                         const int* __restrict__ col_ptr, const int* __restrict__ row_idx,
                                                         const int* __restrict__ csc_pos, const int* __restrict__ order,
                                                         int L, int nnzb, int BH, int nb, int heads, int* status) {
  using T = OpTile<D>;
  constexpr int NST = COL_NST;
  constexpr int STAGE_BYTES = 2 * (VT_BYTES + T::BYTES);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  // full[s]: tiles of stage s landed; empty[s]: the MMAs that read stage s are done;
  // done[b]: accumulator buffer b holds a finished unit; free[b]: its rows have been read out (4 warps arrive)
  const uint32_t bar_full = sbase + NST * STAGE_BYTES;
  const uint32_t bar_empty = bar_full + 8 * NST;
  const uint32_t bar_done = bar_empty + 8 * NST;
  const uint32_t bar_free = bar_done + 16;
  const uint32_t slot = bar_free + 16;
  uint32_t* slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (slot - raw));
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int total = nb * BH, G = (int)gridDim.x;
  constexpr uint32_t TMEM_COLS = 128u;                              // two buffers of 64 columns

  if (warp == 0 && lane == 0) {
    s_abort = *reinterpret_cast<volatile int*>(status);
    for (int st = 0; st < NST; ++st) { mbar_init(bar_full + 8 * st, 1); mbar_init(bar_empty + 8 * st, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(bar_done + 8 * b, 1); mbar_init(bar_free + 8 * b, 4); }
    fence_barrier_init();
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
  constexpr uint32_t IDESC = make_idesc_bf16(64, D, 1, 1);

  // unit u -> (bh, block column); columns of one (b,h) matrix together, the longest first
  auto unit_line = [&](int uu, int& bh, int& line, int& beg, int& end) {
    bh = uu / nb;
    line = order[uu - bh * nb];
    beg = col_ptr[line];
    end = col_ptr[line + 1];
  };

  if (warp == 0) {
    // ------------------------------------------------------------ loads + MMA issue
    // fill cursor: the next entry to request (runs ahead of the MMAs, across units)
    int fu = blockIdx.x, fbh = 0, fline = 0, fe = 0, fend = 0;
    auto fill_seek = [&]() {                                         // move to the next unit that has entries
      while (fu < total) {
        unit_line(fu, fbh, fline, fe, fend);
        if (fe < fend) return;
        fu += G;
      }
    };
    fill_seek();
    int nfill = 0, nuse = 0;                                         // entries requested / consumed by this CTA
    auto fill_one = [&]() -> bool {                                  // all lanes; false on a time-out
      const int st = nfill % NST;
      if (nfill >= NST) {                                            // the MMAs of the entry NST back must be done
        if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * st, (uint32_t)(nfill / NST - 1) & 1u))) return false;
      }
      const uint32_t sa = sbase + st * STAGE_BYTES;
      if (lane == 0) mbar_expect_tx(bar_full + 8 * st, STAGE_BYTES);
      __syncwarp();
      if (lane < 4) {
        const OpPos pos = op_pos(fbh, L, heads, D);
        const int vrow = (int)(((size_t)fbh * nnzb + csc_pos[fe]) * BS);     // CSR block id of the value tile
        const int orow = pos.row0 + row_idx[fe] * BS;
        if (lane == 0) tma_load_2d(sa, &tmdS, bar_full + 8 * st, 0, vrow);
        if (lane == 1) tma_load_2d(sa + VT_BYTES, &tmQ, bar_full + 8 * st, pos.x0, orow);
        if (lane == 2) tma_load_2d(sa + VT_BYTES + T::BYTES, &tmP, bar_full + 8 * st, 0, vrow);
        if (lane == 3) tma_load_2d(sa + 2 * VT_BYTES + T::BYTES, &tmdO, bar_full + 8 * st, pos.x0, orow);
      }
      ++nfill;
      if (++fe >= fend) { fu += G; fill_seek(); }
      return true;
    };
    bool ok = true;
    int uses0 = 0, uses1 = 0;                                        // units with entries that went to buffer 0 / 1
    int j = 0;
    for (int uu = blockIdx.x; uu < total && ok; uu += G, ++j) {
      int bh, line, beg, end;
      unit_line(uu, bh, line, beg, end);
      const int n = end - beg;
      if (n == 0) continue;
      const int buf = j & 1;
      const int uses = buf ? uses1 : uses0;
      if (uses >= 1) {                                               // the rows of the unit before last have been read out
        if (!__all_sync(0xffffffffu, mbar_wait(bar_free + 8 * buf, (uint32_t)(uses - 1) & 1u))) { ok = false; break; }
        tc_fence_after();
      }
      const uint32_t acc = tmem + (uint32_t)buf * 64u;
      for (int i = 0; i < n && ok; ++i) {
        while (ok && nfill < nuse + NST && fu < total) ok = fill_one();
        if (!ok) break;
        const int st = nuse % NST;
        if (!__all_sync(0xffffffffu, mbar_wait(bar_full + 8 * st, (uint32_t)(nuse / NST) & 1u))) { ok = false; break; }
        if (lane == 0) {
          tc_fence_after();
          const uint32_t sa = sbase + st * STAGE_BYTES;
          const uint32_t first = i == 0 ? 0u : 1u;
#pragma unroll
          for (int kk = 0; kk < BS / 16; ++kk)                       // dK += dS^T Q  (lanes 0-15 of every quadrant)
            mma_bf16(acc, ValTile::mnmajor(sa, kk), T::mnmajor(sa + VT_BYTES, kk), IDESC, (kk > 0) ? 1u : first);
#pragma unroll
          for (int kk = 0; kk < BS / 16; ++kk)                       // dV += P^T dO  (lanes 16-31)
            mma_bf16(acc + (16u << 16), ValTile::mnmajor(sa + VT_BYTES + T::BYTES, kk),
                     T::mnmajor(sa + 2 * VT_BYTES + T::BYTES, kk), IDESC, (kk > 0) ? 1u : first);
          mma_commit(bar_empty + 8 * st);
          if (i + 1 == n) mma_commit(bar_done + 8 * buf);
        }
        __syncwarp();
        ++nuse;
      }
      if (buf) ++uses1; else ++uses0;
    }
    if (!ok && lane == 0) report(status, ERR_LOAD_WAIT);
  } else {
    // ------------------------------------------------------------ output rows: TMEM -> bf16 -> global
    const int qd = warp & 3;                                         // TMEM quadrant of this warp
    const int row = qd * 16 + (lane & 15);
    __nv_bfloat16* out = lane < 16 ? dK : dV;
    bool ok = true;
    int uses0 = 0, uses1 = 0;
    int j = 0;
    for (int uu = blockIdx.x; uu < total && ok; uu += G, ++j) {
      int bh, line, beg, end;
      unit_line(uu, bh, line, beg, end);
      const int n = end - beg;
      const int buf = j & 1;
      const OpPos pos = op_pos(bh, L, heads, D);
      __nv_bfloat16* dst = out + (size_t)(pos.row0 + line * BS + row) * pos.ld + pos.x0;
      if (n > 0) {
        const int uses = buf ? uses1 : uses0;
        if (!__all_sync(0xffffffffu, mbar_wait(bar_done + 8 * buf, (uint32_t)uses & 1u))) { ok = false; break; }
        tc_fence_after();
      }
      const uint32_t tl = tmem + ((uint32_t)(qd * 32) << 16) + (uint32_t)buf * 64u;
#pragma unroll
      for (int h = 0; h < D / 32; ++h) {
        uint32_t v[32];
        if (n > 0) {
          tmem_ld32(tl + h * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = 0u;
        }
        uint4* d4 = reinterpret_cast<uint4*>(dst + h * 32);
#pragma unroll
        for (int e = 0; e < 4; ++e)
          d4[e] = make_uint4(pack_bf16(__uint_as_float(v[8 * e]), __uint_as_float(v[8 * e + 1])),
                             pack_bf16(__uint_as_float(v[8 * e + 2]), __uint_as_float(v[8 * e + 3])),
                             pack_bf16(__uint_as_float(v[8 * e + 4]), __uint_as_float(v[8 * e + 5])),
                             pack_bf16(__uint_as_float(v[8 * e + 6]), __uint_as_float(v[8 * e + 7])));
      }
      if (n > 0) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_free + 8 * buf);
        if (buf) ++uses1; else ++uses0;
      }
    }
    if (!ok && lane == 0) report(status, ERR_MMA_WAIT);
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
                           int4* __restrict__ info, int* __restrict__ n_long) {
  __shared__ int s_n[SPION_MAX_NB];
  if (threadIdx.x == 0) *n_long = 0;
  for (int r = threadIdx.x; r < nb; r += blockDim.x) s_n[r] = row_ptr[r + 1] - row_ptr[r];
  __syncthreads();
  for (int r = threadIdx.x; r < nb; r += blockDim.x)
    if (s_n[r] > ROW_NCH) atomicAdd(n_long, 1);                     // rows that need the streamed schedule
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

// Column records for the streaming column kernel, in col_order: one CTA.
//   rec[x]  = {block column, index of its first pair, pairs, entries}
//   pair[p] = {block row of the pair's first entry, of its second (-1: none), CSR block ids of the two}
__global__ void k_col_recs(const int32_t* __restrict__ col_ptr, const int32_t* __restrict__ row_idx,
                           const int32_t* __restrict__ csc_pos, const int* __restrict__ order, int nb,
                           int4* __restrict__ rec, int4* __restrict__ pair) {
  __shared__ int s_first[SPION_MAX_NB + 1];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int x = 0; x < nb; ++x) {
      const int c = order[x];
      s_first[x] = acc;
      acc += (col_ptr[c + 1] - col_ptr[c] + 1) >> 1;
    }
    s_first[nb] = acc;
  }
  __syncthreads();
  for (int x = threadIdx.x; x < nb; x += blockDim.x) {
    const int c = order[x], beg = col_ptr[c], n = col_ptr[c + 1] - beg, np = (n + 1) >> 1;
    rec[x] = make_int4(c, s_first[x], np, n);
    for (int k = 0; k < np; ++k) {
      const int e0 = beg + 2 * k;
      const bool two = e0 + 1 < beg + n;
      pair[s_first[x] + k] = make_int4(row_idx[e0], two ? row_idx[e0 + 1] : -1, csc_pos[e0], two ? csc_pos[e0 + 1] : 0);
    }
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

template <int D> constexpr size_t smem_row() { return 1024 + (size_t)5 * OpTile<D>::BYTES + 4 * VT_BYTES + 128; }
template <int D> constexpr size_t smem_col() { return 1024 + (size_t)COL_NST * 2 * (VT_BYTES + OpTile<D>::BYTES) + 128; }

// Shared-memory opt-in of the two backward kernels, and how many CTAs of each one SM holds at once
// (the persistent grids; both kernels take 128 of the 512 tensor-memory columns).
template <int D>
int set_attrs(TcState* s, int device) {
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_bwd_row<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_row<D>()));
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_bwd_col<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_col<D>()));
  int rc;
  if ((rc = resident_ctas(k_bwd_row<D>, device, ROW_THREADS, smem_row<D>(), 128, &s->row_ctas))) return rc;
  if ((rc = resident_ctas(k_bwd_col<D>, device, COL_THREADS, smem_col<D>(), 128, &s->col_ctas))) return rc;
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

int ensure_super_ws(spion_ctx* c, TcState* s);

template <int D>
int run_backward(spion_ctx* c, TcState* s, const void* Q, const void* K, const void* V, const void* P_user,
                 const void* O, const void* dO, void* dS_user, void* dQ, void* dK, void* dV) {
  const TcView vw = tc_view(c, s);
  const void* P = P_user;
  void* dS = dS_user;
  int rc;
  if (s->super) {                    // bring the caller's 32-wide tiles into super-tile form
    if ((rc = ensure_super_ws(c, s))) return rc;
    if ((rc = convert_tiles(c, s, true, s->p64_ws, const_cast<void*>(P_user)))) return rc;
    P = s->p64_ws;
    dS = s->ds64_ws;
  }
  const uint64_t vrows = (uint64_t)c->BH * vw.nnzb * BS;
  prof_mark(c, -1);
  CUtensorMap mds, mp, mq, mk, mdo, mv;
  if ((rc = make_map(s, &mds, dS, vrows, BS, BS, BS)) || (rc = make_map(s, &mp, P, vrows, BS, BS, BS)) ||
      (rc = make_operand_map(c, s, &mq, Q, D)) || (rc = make_operand_map(c, s, &mk, K, D)) ||
      (rc = make_operand_map(c, s, &mdo, dO, D)) || (rc = make_operand_map(c, s, &mv, V, D)))
    return rc;
  const long long total = (long long)c->BH * vw.nb;
  const long long row_cap = (long long)s->sms * s->row_ctas, col_cap = (long long)s->sms * s->col_ctas;
  k_bwd_row<D><<<(int)(total < row_cap ? total : row_cap), ROW_THREADS, smem_row<D>(), c->stream>>>(
      mdo, mv, mk, mp, mds, (const __nv_bfloat16*)dO, (const __nv_bfloat16*)O, (__nv_bfloat16*)dQ, vw.row_info,
      vw.col_idx, c->L, vw.nnzb, c->BH, vw.nb, c->heads, c->scale, c->status_dev);
  SPION_LAUNCH_CHECK();
  c->launches += 1;
  prof_mark(c, SPION_STAGE_BWD_ROW);
  k_bwd_col<D><<<(int)(total < col_cap ? total : col_cap), COL_THREADS, smem_col<D>(), c->stream>>>(
      mds, mp, mq, mdo, (__nv_bfloat16*)dK, (__nv_bfloat16*)dV, vw.col_ptr, vw.row_idx, vw.csc_pos, s->col_order, c->L,
      vw.nnzb, c->BH, vw.nb, c->heads, c->status_dev);
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

// [BH, nnzb64, 64, 64] bf16 workspaces for P and dS in super-tile form
int ensure_super_ws(spion_ctx* c, TcState* s) {
  const size_t need = (size_t)c->BH * s->nnzb64 * 4096;
  if (need <= s->ws_elems) return SPION_OK;
  cudaFree(s->p64_ws); cudaFree(s->ds64_ws);
  s->p64_ws = s->ds64_ws = nullptr;
  s->ws_elems = 0;
  if (cudaMalloc(&s->p64_ws, need * 2) != cudaSuccess || cudaMalloc(&s->ds64_ws, need * 2) != cudaSuccess)
    return SPION_ERR_ALLOC;
  s->ws_elems = need;
  return SPION_OK;
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
  // The two super-tile workspaces serve the calls that store P (and the stored-path backward).  When the mask runs
  // on its own blocks they are allocated only if such a call arrives (ensure_super_ws), not here.
  if (!(s->b32 && s->b32_use)) {
    int rc = ensure_super_ws(c, s);
    if (rc) return rc;
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
    if (cudaDeviceGetAttribute(&s->sms, cudaDevAttrMultiProcessorCount, c->device) != cudaSuccess || s->sms < 1) {
      delete s;
      return SPION_ERR_CUDA;
    }
    int rc = (c->d == 64) ? set_attrs<64>(s, c->device) : set_attrs<32>(s, c->device);
    if (!rc) rc = fused_set_attrs(s, c->d, c->device);
    if (!rc) rc = recompute_set_attrs(s, c->d, c->device);
    if (!rc) rc = pipe_set_attrs(s, c->d, c->device);
    if (!rc && b32_applies(c)) { rc = b32_set_attrs(s, c->device); s->b32 = rc == SPION_OK; }
    if (!rc && cudaMalloc(&s->delta_ws, (size_t)c->BH * c->L * sizeof(float)) != cudaSuccess) rc = SPION_ERR_ALLOC;
    if (!rc && cudaMalloc(&s->lse_ws, (size_t)c->BH * c->L * sizeof(float)) != cudaSuccess) rc = SPION_ERR_ALLOC;
    if (rc) { delete s; return rc; }
    s->super = c->bs == 32;
    c->tc = s;
  }
  if (s->b32) {                      // decides whether the mask runs on its own blocks (before the super-block set-up)
    int rc = b32_prepare(c, s);
    if (rc) return rc;
  }
  if (s->super) {
    int rc = build_super(c, s);
    if (rc) return rc;
  }
  const TcView vw = tc_view(c, s);
  // value-tile rows are 32-bit TMA coordinates: (bh * nnzb + block) * 64 must stay below 2^31
  if ((unsigned long long)c->BH * (unsigned long long)vw.nnzb * BS >= 0x7fffffffULL) return SPION_ERR_SHAPE;
  if (!s->row_info && cudaMalloc(&s->row_info, (size_t)SPION_MAX_NB * sizeof(int4)) != cudaSuccess) return SPION_ERR_ALLOC;
  if (!s->n_long_dev && cudaMalloc(&s->n_long_dev, sizeof(int)) != cudaSuccess) return SPION_ERR_ALLOC;
  k_row_info<<<1, 512, 0, c->stream>>>(vw.row_ptr, vw.col_idx, vw.nb, s->row_info, s->n_long_dev);
  SPION_LAUNCH_CHECK();
  SPION_CUDA_TRY(cudaMemcpyAsync(&s->n_long, s->n_long_dev, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  SPION_CUDA_TRY(cudaStreamSynchronize(c->stream));                // set_pattern time: once per mask
  if (!s->col_order && cudaMalloc(&s->col_order, (size_t)SPION_MAX_NB * sizeof(int)) != cudaSuccess) return SPION_ERR_ALLOC;
  k_line_order<<<1, 512, 0, c->stream>>>(vw.col_ptr, vw.nb, s->col_order);
  SPION_LAUNCH_CHECK();
  if (!s->col_rec && cudaMalloc(&s->col_rec, (size_t)SPION_MAX_NB * sizeof(int4)) != cudaSuccess) return SPION_ERR_ALLOC;
  if ((size_t)vw.nnzb > s->col_pair_cap) {                         // at most one pair per entry
    cudaFree(s->col_pair);
    s->col_pair = nullptr;
    s->col_pair_cap = 0;
    if (cudaMalloc(&s->col_pair, (size_t)vw.nnzb * sizeof(int4)) != cudaSuccess) return SPION_ERR_ALLOC;
    s->col_pair_cap = (size_t)vw.nnzb;
  }
  k_col_recs<<<1, 512, 0, c->stream>>>(vw.col_ptr, vw.row_idx, vw.csc_pos, s->col_order, vw.nb, s->col_rec, s->col_pair);
  SPION_LAUNCH_CHECK();
  c->launches += 2;
  return SPION_OK;
}

void tc_engine_release(spion_ctx* c) {
  if (!c->tc) return;
  TcState* s = (TcState*)c->tc;
  free_super(s);
  b32_release(s);
  cudaFree(s->lse_ws);
  cudaFree(s->delta_ws);
  cudaFree(s->n_long_dev);
  cudaFree(s->row_info);
  cudaFree(s->col_order);
  cudaFree(s->col_rec);
  cudaFree(s->col_pair);
  delete s;
  c->tc = nullptr;
}

// forward with the probabilities in the caller's tile layout (P_user may be NULL)
static int forward_any(spion_ctx* c, const void* Q, const void* K, const void* V, const float* keypad, void* O,
                       float* lse, void* P_user) {
  TcState* s = (TcState*)c->tc;
  if (!s) return SPION_ERR_STATE;
  if (c->nnzb == 0) return SPION_ERR_SHAPE;
  if (s->b32 && s->b32_use && !P_user) return b32_forward(c, s, Q, K, V, keypad, O, lse ? lse : s->lse_ws);
  if (P_user && s->super) {
    int rc = ensure_super_ws(c, s);
    if (rc) return rc;
  }
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


int tc_engine_backward_fused(spion_ctx* c, const void* Q, const void* K, const void* V, const void* O, const void* dO,
                             const float* lse, const float* keypad, void* dQ, void* dK, void* dV) {
  if (!c->tc) return SPION_ERR_STATE;
  if (c->nnzb == 0) return SPION_ERR_SHAPE;
  TcState* s = (TcState*)c->tc;
  if (s->b32 && s->b32_use) return b32_backward(c, s, Q, K, V, O, dO, lse, keypad, dQ, dK, dV);
  return recompute_backward(c, s, Q, K, V, O, dO, lse, keypad, dQ, dK, dV);
}

int tc_engine_mean_map(spion_ctx* c, const void* Q, const void* K, const float* lse, const float* keypad, float* A) {
  if (!c->tc) return SPION_ERR_STATE;
  if (c->nnzb == 0) return SPION_ERR_SHAPE;
  return recompute_mean_map(c, (TcState*)c->tc, Q, K, lse, keypad, A);
}

int tc_engine_block32_path(const spion_ctx* c) {
  const TcState* s = (const TcState*)c->tc;
  if (!s || !s->super) return 0;
  return (s->b32 && s->b32_use) ? 1 : 2;
}

int tc_engine_wait_selftest(spion_ctx* c, long long limit_cycles) {
  k_wait_selftest<<<1, 128, 0, c->stream>>>(c->status_dev, limit_cycles);
  SPION_LAUNCH_CHECK();
  c->launches += 1;
  return SPION_OK;
}
