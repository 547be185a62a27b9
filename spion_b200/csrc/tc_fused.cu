// Fused block-sparse attention forward (sm_100a, bf16, 64x64 blocks): S and the sparse row softmax
// stay on chip; Q, K, V are read once per use, O and one fp32 log-sum-exp per row are written
// (the P tiles only when the caller asks for them, e.g. for the backward pass).
//
//   k_fwd_fused   per block row:   S = Q K^T (tcgen05, TMEM) -> row softmax (fp32, registers)
//                                  -> P (bf16, swizzled shared memory) -> O = P V (tcgen05)
//                 replaces the three forward stages of models/block_attn.cu:453-487.
//
// Softmax semantics are the reference's (models/block_attn.cu:48-87): every non-selected key of a
// row adds exp(0 - m) to the denominator.  lse2_i = m_i*log2(e) + log2(Z_i) is stored so that
// P_ij = exp2(s_ij*scale*log2(e) - lse2_i) can be recomputed from Q and K.
//
// Accumulator placement: an MMA with M = 64 fills TMEM lanes (m%16) + 32*(m/16); a second tile is
// placed in the same columns at lane offset 16, so that all 32 lanes of every warp hold a row
// (lanes 0-15: even tile of a pair, lanes 16-31: odd tile).
#include "tc_tiles.cuh"

using namespace tc;

#ifdef SPION_TRACE
SPION_TRACE_SETTER(spion_debug_trace_fused)
#endif

namespace {

constexpr int FWD_THREADS = 160;           // warps 0-3: one TMEM quadrant each (math); warp 4: TMA loads, MMA issue, tile stores
constexpr int FWD_NCH = ROW_NCH;           // tiles of a row that fits in one chunk
// TMEM (128 columns): S pairs at [0,64) and [64,128); O overwrites [0,64) once P has been extracted.

template <int D> constexpr size_t fwd_smem_bytes() {
  // Q | K x4 | V x4 | (P x4 only when a K tile is smaller than a P tile) | barriers
  return 1024 + (size_t)(1 + 2 * FWD_NCH) * OpTile<D>::BYTES + (D == 64 ? 0 : (size_t)FWD_NCH * VT_BYTES) + 64;
}

// Store one 64-value bf16 row into a [64 x 64] K-major SWIZZLE_128B tile (16-byte chunk c of row i
// sits at chunk c ^ (i & 7)): the image TMA would have produced, readable by tcgen05.mma.
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 32 consecutive values (16 packed words) of row i, columns [32 g, 32 g + 32), into the same image.
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

__device__ __forceinline__ void store_row_swizzled(uint32_t tile, int i, const uint32_t (&w)[32]) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint32_t addr = tile + i * 128 + ((c ^ (i & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * c]), "r"(w[4 * c + 1]),
                 "r"(w[4 * c + 2]), "r"(w[4 * c + 3])
                 : "memory");
  }
}

// Persistent CTAs (the grid is the number of CTAs the device holds at once): CTA i works on units i,
// i + grid, i + 2 grid, ... of the list (sorted block row, bh), bh fastest.  Four math warps (one per TMEM
// quadrant) do the softmax arithmetic and write the output rows; a fifth, the control warp, issues every
// TMA load, MMA and tile store, so the math warps never spend issue slots or wait on a copy engine.
// Barriers are initialised and tensor memory is allocated once per CTA; the operand tiles of the next
// unit are requested as soon as the last MMA of the current one has retired, so they arrive while the
// current unit's output rows are written.
// A row of the block is owned by two threads of one warp (lane l: even tiles, lane l+16: odd tiles), so
// the row statistics need only one warp shuffle.  Rows with at most 4 blocks are done in one chunk (S in
// all 128 columns, O then overwrites the first 64); longer rows stream chunks of 2 tiles through columns
// [64,128) in two passes (row maximum, then exp / P / O).  P is kept unnormalised (exp2(x - m) <= 1) and
// the output row is divided by the denominator at the end.
// STORE_P: also write the normalised probabilities as [64 x 64] bf16 tiles (TMA store from the shared
// memory tiles the second product reads): rows of one chunk are rescaled in place once the
// denominator is known; longer rows accumulate the denominator on line in pass A instead.
// heads: 0 = operands [BH, L, D]; H = operands [B, L, H, D] (see op_pos).
template <int D, bool STORE_P, bool SUB>
__global__ void __launch_bounds__(FWD_THREADS, 3) k_fwd_fused(const __grid_constant__ CUtensorMap tmQ,
                                                              const __grid_constant__ CUtensorMap tmK,
                                                              const __grid_constant__ CUtensorMap tmV,
                                                              const __grid_constant__ CUtensorMap tmP,
                                                              __nv_bfloat16* __restrict__ O, float* __restrict__ lse_out,
                                                              const float* __restrict__ keypad,
                                                              const int4* __restrict__ row_info,
                                                              const int* __restrict__ col_idx,
                                                              const uint8_t* __restrict__ submask, int L, int nnzb,
                                                              int BH, int nrows, int heads, float scale, float floor_v,
                                                              int* status) {
  using T = OpTile<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  const uint32_t sQ = sbase;
  const uint32_t sK = sQ + T::BYTES;
  const uint32_t sV = sK + FWD_NCH * T::BYTES;
  const uint32_t sP = (D == 64) ? sK : sV + FWD_NCH * T::BYTES;            // P tiles reuse the K buffers
  const uint32_t bars = sV + FWD_NCH * T::BYTES + (D == 64 ? 0 : FWD_NCH * VT_BYTES);
  const uint32_t bar_k0 = bars, bar_v0 = bars + 8, bar_s = bars + 16, bar_o = bars + 24, slot = bars + 32;
  const uint32_t bar_k1 = bars + 40, bar_v1 = bars + 48;          // second half of the buffers (long rows)
  uint32_t* slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (slot - raw));
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool ctl = warp == 4;                                  // control warp: no arithmetic, no TMEM reads
  const int q = warp & 3;                                      // TMEM quadrant of a math warp
  const int hf = lane >> 4;                                    // 0: even tiles, 1: odd tiles
  const int row = q * 16 + (lane & 15);                        // row of the block this thread owns
  const int total = nrows * BH;
  constexpr uint32_t ncols = 128u;
  constexpr uint32_t o_col = 0u;

  // Called by all lanes of the control warp: lane 0 announces the bytes, then one lane per tile issues its copy
  // (a single thread needs about 0.1 us per copy; a row has up to nine).
  auto issue_job = [&](const RowRec& R, int bh, int g) {
    const bool single = R.single();
    const int CH = R.chunk(), nchunks = R.nchunks();
    const bool with_v = single || g >= nchunks;
    const int ch = (single || g < nchunks) ? g : g - nchunks;
    const int t0 = ch * CH, nt = min(CH, R.nblk - t0);
    const int hb = single ? 0 : (g & 1), b0 = 2 * hb;
    const uint32_t bk = hb ? bar_k1 : bar_k0, bv = hb ? bar_v1 : bar_v0;
    const OpPos pos = op_pos(bh, L, heads, D);
    if (lane == 0) {
      mbar_expect_tx(bk, (g == 0 ? T::BYTES : 0) + nt * T::BYTES);
      if (with_v) mbar_expect_tx(bv, nt * T::BYTES);
    }
    __syncwarp();
    if (lane == 0 && g == 0) tma_load_2d(sQ, &tmQ, bk, pos.x0, pos.row0 + R.r * BS);
    if (lane >= 1 && lane <= nt)
      tma_load_2d(sK + (b0 + lane - 1) * T::BYTES, &tmK, bk, pos.x0, pos.row0 + R.col(t0 + lane - 1, col_idx) * BS);
    if (with_v && lane >= 9 && lane < 9 + nt)
      tma_load_2d(sV + (b0 + lane - 9) * T::BYTES, &tmV, bv, pos.x0, pos.row0 + R.col(t0 + lane - 9, col_idx) * BS);
  };

  int u = blockIdx.x;
  RowRec R;
  int bh = 0;
  if (u < total) { const int rank = u / BH; R = RowRec(row_info[rank]); bh = u - rank * BH; }

  if (ctl) {
    if (lane == 0) {
      s_abort = *reinterpret_cast<volatile int*>(status);
      mbar_init(bar_k0, 1);
      mbar_init(bar_v0, 1);
      mbar_init(bar_k1, 1);
      mbar_init(bar_v1, 1);
      mbar_init(bar_s, 1);
      mbar_init(bar_o, 1);
      fence_barrier_init();
    }
    __syncwarp();
    if (s_abort == 0 && u < total) {                           // operands are on their way before TMEM is set up
      if (R.njobs() > 0) issue_job(R, bh, 0);
      if (R.njobs() > 1) issue_job(R, bh, 1);
    }
  }
  __syncthreads();
  if (s_abort != 0) return;
  if (ctl) {
    tmem_alloc(slot, ncols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot_ptr;

  const uint32_t t_lane = tmem + ((uint32_t)(q * 32) << 16);
  constexpr uint32_t IDESC_S = make_idesc_bf16(64, 64, 0, 0);
  constexpr uint32_t IDESC_O = make_idesc_bf16(64, D, 0, 1);
  const float sc2 = scale * LOG2E;
  // Barrier parities run on across the units of this CTA.  pk / pv: one bit per half of the buffers
  // (only thread 0 waits on the load barriers); ps / po: bar_s / bar_o (every thread waits on each phase).
  uint32_t pk = 0, pv = 0, ps = 0, po = 0;
  bool ok = true;

  int ord = 0;
  for (; u < total && ok; u += gridDim.x, ++ord) {
    SPION_STAMP(ord, 0);
    // the unit after this one (its operands are requested before this unit's output is written)
    const int un = u + (int)gridDim.x;
    const bool has_next = un < total;
    RowRec Rn;
    int bhn = 0;
    if (has_next) { const int rank = un / BH; Rn = RowRec(row_info[rank]); bhn = un - rank * BH; }

    const int rp = R.rp, nblk = R.nblk, r = R.r;
    auto col_of = [&](int t) -> int { return R.col(t, col_idx); };
    // 32-wide masks: bit (2*(row/32) + col/32) of submask[block] tells whether that quarter is selected
    const int rh2 = (q >> 1) * 2;
    auto quarter_ok = [&](int blk, int half) -> bool { return !SUB || ((submask[blk] >> (rh2 + half)) & 1); };
    int n_sel = nblk * BS;                                       // selected keys of this thread's row
    if (SUB) {
      n_sel = 0;
      for (int t = 0; t < nblk; ++t) n_sel += 32 * __popc((submask[rp + t] >> rh2) & 3);
    }
    const bool single = R.single();
    const int CH = R.chunk();
    const int nchunks = R.nchunks();
    const int njobs = R.njobs();
    const float* kp = keypad ? keypad + (size_t)bh * L : nullptr;
    const OpPos pos = op_pos(bh, L, heads, D);

    // All buffers of this unit are free (its last MMA has retired): ask for the next unit's first tiles.
    auto prefetch_next = [&]() {
      if (ctl && has_next) {
        if (STORE_P) {                                           // the tile stores must have read their tiles
          if (lane == 0) bulk_wait_read_all();
          __syncwarp();
        }
        if (Rn.njobs() > 0) issue_job(Rn, bhn, 0);
        if (Rn.njobs() > 1) issue_job(Rn, bhn, 1);
      }
    };

    // control lane: wait for the K tiles of job g (already requested) and issue the S MMAs of its chunk into
    // accumulator columns col(t); the commit arrives on bar
    auto issue_s = [&](int g, uint32_t pair_stride, uint32_t col0, uint32_t bar) -> bool {
      const int ch = (single || g < nchunks) ? g : g - nchunks;
      const int t0 = ch * CH, nt = min(CH, nblk - t0);
      const int hb = single ? 0 : (g & 1), b0 = 2 * hb;
      if (!mbar_wait(hb ? bar_k1 : bar_k0, (pk >> hb) & 1)) { report(status, ERR_LOAD_WAIT); return false; }
      pk ^= 1u << hb;
      tc_fence_after();
      const uint64_t dq0 = T::kmajor(sQ, 0);
      uint64_t dk0 = T::kmajor(sK + b0 * T::BYTES, 0);
      for (int t = 0; t < nt; ++t, dk0 = desc_advance(dk0, T::BYTES)) {
        const uint32_t d_addr = tmem + ((uint32_t)((t & 1) * 16) << 16) + col0 + (uint32_t)(t >> 1) * pair_stride;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_bf16(d_addr, desc_advance(dq0, kk * T::K_STEP), desc_advance(dk0, kk * T::K_STEP), IDESC_S, kk > 0);
      }
      mma_commit(bar);
      return true;
    };

    float m2 = floor_v * LOG2E;
    float mraw = -INFINITY;
    float l_part = 0.f;
    const bool online = STORE_P && !single;                        // denominator needed before P is written

    // Row statistics of one chunk whose pair p sits in columns colbase + 64 p: the maximum, and for
    // `online` also the running sum of exponentials.
    auto stats_math = [&](uint32_t colbase, int t0, int nt, int npairs) {
      if (!online) {
        for (int p = 0; p < npairs; ++p) {
          const int t = 2 * p + hf;
          const bool mine = t < nt;
          const int c = mine ? col_of(t0 + t) : 0;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t v[32];
            tmem_ld32(t_lane + colbase + p * 64 + half * 32, v);
            tmem_ld_wait();
            if (mine && quarter_ok(rp + t0 + t, half)) {
              if (!kp) {                                            // the scale is positive: compare raw scores
                float ma = mraw, mb = -INFINITY, mc = -INFINITY, md = -INFINITY;   // four chains instead of one
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  ma = fmaxf(ma, fmaxf(__uint_as_float(v[j]), __uint_as_float(v[j + 1])));
                  mb = fmaxf(mb, fmaxf(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])));
                  mc = fmaxf(mc, fmaxf(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5])));
                  md = fmaxf(md, fmaxf(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7])));
                }
                mraw = fmaxf(fmaxf(ma, mb), fmaxf(mc, md));
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  m2 = fmaxf(m2, fmaf(__uint_as_float(v[j]), sc2, -kp[c * BS + half * 32 + j] * LOG2E));
              }
            }
          }
        }
      } else {
        for (int p = 0; p < npairs; ++p) {
          const int t = 2 * p + hf;
          const bool mine = t < nt;
          const int c = mine ? col_of(t0 + t) : 0;
          uint32_t v0[32], v1[32];
          tmem_ld32(t_lane + colbase + p * 64, v0);
          tmem_ld32(t_lane + colbase + p * 64 + 32, v1);
          tmem_ld_wait();
          float cm = -INFINITY;
          if (mine) {
            const bool ok0 = quarter_ok(rp + t0 + t, 0), ok1 = quarter_ok(rp + t0 + t, 1);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float x0 = __uint_as_float(v0[j]) * sc2, x1 = __uint_as_float(v1[j]) * sc2;
              if (kp) { x0 -= kp[c * BS + j] * LOG2E; x1 -= kp[c * BS + 32 + j] * LOG2E; }
              if (!ok0) x0 = -INFINITY;
              if (!ok1) x1 = -INFINITY;
              v0[j] = __float_as_uint(x0); v1[j] = __float_as_uint(x1);
              cm = fmaxf(cm, fmaxf(x0, x1));
            }
          }
          cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, 16));
          const float m_new = fmaxf(m2, cm);
          float sum = 0.f;
          if (mine) {
#pragma unroll
            for (int j = 0; j < 32; ++j) sum += ex2(__uint_as_float(v0[j]) - m_new) + ex2(__uint_as_float(v1[j]) - m_new);
          }
          l_part = l_part * exp2f(m2 - m_new) + sum;
          m2 = m_new;
        }
      }
    };

    // Exponentials of one chunk against the fixed m2 (the row maximum, or the log-sum-exp when the
    // denominator is already known), packed to bf16 and stored as the K-major P tiles b0 + t.
    auto prob_math = [&](uint32_t colbase, int b0, int t0, int nt, int npairs) {
      for (int p = 0; p < npairs; ++p) {
        const int t = 2 * p + hf;
        const bool mine = t < nt;
        const int c = mine ? col_of(t0 + t) : 0;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t v[32], w[16];
          tmem_ld32(t_lane + colbase + p * 64 + half * 32, v);
          tmem_ld_wait();
          if (mine && quarter_ok(rp + t0 + t, half)) {
            float la = 0.f, lb = 0.f, lc = 0.f, ld = 0.f;               // four independent running sums
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float h0 = m2, h1 = m2;
              if (kp) { h0 = fmaf(kp[c * BS + half * 32 + j], LOG2E, m2); h1 = fmaf(kp[c * BS + half * 32 + j + 1], LOG2E, m2); }
              const float e0 = ex2(fmaf(__uint_as_float(v[j]), sc2, -h0)), e1 = ex2(fmaf(__uint_as_float(v[j + 1]), sc2, -h1));
              if ((j & 6) == 0) la += e0 + e1;
              else if ((j & 6) == 2) lb += e0 + e1;
              else if ((j & 6) == 4) lc += e0 + e1;
              else ld += e0 + e1;
              w[j >> 1] = pack_bf16(e0, e1);
            }
            l_part += (la + lb) + (lc + ld);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) w[j] = 0u;
          }
          if (mine) store_half_row_swizzled(sP + (b0 + t) * VT_BYTES, row, half, w);
        }
      }
    };

    // control lane: O += P V for the tiles of one chunk (after its V tiles have arrived), then the P tile stores.
    // Every tile of the row accumulates into the one [64 x D] accumulator at lane offset 0.
    auto issue_pv = [&](int hb, int t0, int nt, bool first_chunk) -> bool {
      const int b0 = 2 * hb;
      if (!mbar_wait(hb ? bar_v1 : bar_v0, (pv >> hb) & 1)) { report(status, ERR_LOAD_WAIT); return false; }
      pv ^= 1u << hb;
      tc_fence_after();
      uint64_t dp0 = ValTile::kmajor(sP + b0 * VT_BYTES, 0), dv0 = T::mnmajor(sV + b0 * T::BYTES, 0);
      for (int t = 0; t < nt; ++t, dp0 = desc_advance(dp0, VT_BYTES), dv0 = desc_advance(dv0, T::BYTES)) {
        const uint32_t first = (first_chunk && t == 0) ? 0u : 1u;
#pragma unroll
        for (int kk = 0; kk < BS / 16; ++kk)
          mma_bf16(tmem + o_col, desc_advance(dp0, kk * ValTile::K_STEP), desc_advance(dv0, kk * T::MN_STEP), IDESC_O,
                   (kk > 0) ? 1u : first);
      }
      if (STORE_P) {                                                // these tiles are final: store them now
        for (int t = 0; t < nt; ++t)
          tma_store_2d(&tmP, sP + (b0 + t) * VT_BYTES, 0, (int)(((size_t)bh * nnzb + rp + t0 + t) * BS));
        bulk_commit();
      }
      return true;
    };
    float lse_fixed = 0.f;
    auto finish_stats = [&]() {
      m2 = fmaxf(m2, mraw * sc2);
      m2 = fmaxf(m2, __shfl_xor_sync(0xffffffffu, m2, 16));        // both owners of a row agree
      if (online) {
        const float l = l_part + __shfl_xor_sync(0xffffffffu, l_part, 16) + (float)(L - n_sel) * exp2f(-m2);
        lse_fixed = m2 + log2f(l);
        m2 = lse_fixed;                                             // pass B then produces normalised P directly
        l_part = 0.f;
      }
    };

    if (single && nblk > 0) {
      // ---------------------------------------------------------------- rows of at most 4 blocks
      if (ctl && lane == 0) issue_s(0, 64u, 0u, bar_s);
      if (!__syncthreads_and(mbar_wait(bar_s, ps))) { if (tid == 0) report(status, ERR_MMA_WAIT); ok = false; }
      ps ^= 1u;
      tc_fence_after();
      SPION_STAMP(ord, 1);
      if (ok) {
        if (!ctl) {
          stats_math(0u, 0, nblk, 2);
          finish_stats();
        }
        SPION_STAMP(ord, 2);
        if (ctl) {
        } else if (STORE_P) {
          // keep both tiles' exponentials packed in registers, normalise once the denominator is known
          uint32_t wp[2][32];
#pragma unroll
          for (int p = 0; p < 2; ++p) {
            const int t = 2 * p + hf;
            const bool mine = t < nblk;
            const int c = mine ? col_of(t) : 0;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t v[32];
              tmem_ld32(t_lane + p * 64 + half * 32, v);
              tmem_ld_wait();
              if (mine && quarter_ok(rp + t, half)) {
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                  float h0 = m2, h1 = m2;
                  if (kp) { h0 = fmaf(kp[c * BS + half * 32 + j], LOG2E, m2); h1 = fmaf(kp[c * BS + half * 32 + j + 1], LOG2E, m2); }
                  const float e0 = ex2(fmaf(__uint_as_float(v[j]), sc2, -h0)), e1 = ex2(fmaf(__uint_as_float(v[j + 1]), sc2, -h1));
                  l_part += e0 + e1;
                  wp[p][half * 16 + (j >> 1)] = pack_bf16(e0, e1);
                }
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) wp[p][half * 16 + j] = 0u;
              }
            }
          }
          const float l = l_part + __shfl_xor_sync(0xffffffffu, l_part, 16) + (float)(L - n_sel) * exp2f(-m2);
          // 1/l as a sum of two bf16 values: the packed product then carries one rounding of the result only
          const float inv = 1.0f / l;
          const float inv_h = bf16_hi(pack_bf16(0.f, inv));
          const uint32_t inv_hi = pack_bf16(inv_h, inv_h), inv_lo = pack_bf16(inv - inv_h, inv - inv_h);
          lse_fixed = m2 + log2f(l);
#pragma unroll
          for (int p = 0; p < 2; ++p) {
            const int t = 2 * p + hf;
            if (t < nblk) {
#pragma unroll
              for (int j = 0; j < 32; ++j) wp[p][j] = fma_bf16x2(wp[p][j], inv_hi, mul_bf16x2(wp[p][j], inv_lo));
              store_row_swizzled(sP + t * VT_BYTES, row, wp[p]);
            }
          }
        } else {
          prob_math(0u, 0, 0, nblk, 2);
        }
        SPION_STAMP(ord, 3);
        fence_proxy_async();                                        // P rows -> visible to the MMA proxy
        tc_fence_before();
        __syncthreads();
        SPION_STAMP(ord, 4);
        if (ctl && lane == 0 && issue_pv(0, 0, nblk, true)) mma_commit(bar_o);
        if (!__syncthreads_and(mbar_wait(bar_o, po))) { if (tid == 0) report(status, ERR_MMA2_WAIT); ok = false; }
        po ^= 1u;
        tc_fence_after();
      }
    } else if (nblk > 0) {
      // ---------------------------------------------------------------- longer rows: pairs of tiles, two passes
      // Pass A (statistics): the pair of chunk c sits in columns 64 (c & 1); the MMAs of chunk c+1 are
      // issued before the arithmetic on chunk c.  bar_s serves the even chunks, bar_o the odd ones.
      const int n = nchunks;
      if (ctl && lane == 0) issue_s(0, 0u, 0u, bar_s);
      for (int c = 0; c < n && ok; ++c) {
        const int b = c & 1;
        if (ctl && lane == 0 && c + 1 < n) issue_s(c + 1, 0u, (uint32_t)(b ^ 1) * 64u, b ? bar_s : bar_o);
        if (!__syncthreads_and(mbar_wait(b ? bar_o : bar_s, b ? po : ps))) {
          if (tid == 0) report(status, ERR_MMA_WAIT);
          ok = false;
          break;
        }
        if (b) po ^= 1u; else ps ^= 1u;
        tc_fence_after();
        if (ctl && c + 2 < njobs) issue_job(R, bh, c + 2);         // the S MMAs have consumed this half's K tiles
        if (!ctl) stats_math((uint32_t)b * 64u, 2 * c, min(2, nblk - 2 * c), 1);
        tc_fence_before();
        __syncthreads();                                            // chunk c+2 overwrites these columns
      }
      if (!ctl) finish_stats();
      // Pass B: S of a chunk in columns [64,128), O accumulates in [0,64).  The tensor pipe completes in
      // issue order: once S(c+1) has arrived, O += P V of chunk c is complete too, and its half of the
      // buffers is requested again.
      if (ok && ctl && lane == 0) issue_s(n, 0u, 64u, bar_s);
      for (int c = 0; c < n && ok; ++c) {
        const int g = n + c, hb = g & 1, t0 = 2 * c, nt = min(2, nblk - t0);
        if (!__syncthreads_and(mbar_wait(bar_s, ps))) { if (tid == 0) report(status, ERR_MMA_WAIT); ok = false; break; }
        ps ^= 1u;
        tc_fence_after();
        if (c > 0 && ctl && g + 1 < njobs) {                        // chunk c-1 is finished: its half takes job g+1
          if (STORE_P && lane == 0) bulk_wait_read_all();           // once the tile stores have read it
          __syncwarp();
          issue_job(R, bh, g + 1);
        }
        if (!ctl) prob_math(64u, 2 * hb, t0, nt, 1);
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (ctl && lane == 0 && issue_pv(hb, t0, nt, c == 0)) {
          if (c + 1 < n) issue_s(g + 1, 0u, 64u, bar_s);
          else mma_commit(bar_o);
        }
      }
      if (ok) {
        if (!__syncthreads_and(mbar_wait(bar_o, po))) { if (tid == 0) report(status, ERR_MMA2_WAIT); ok = false; }
        po ^= 1u;
      }
      tc_fence_after();
    } else if (!ctl) {
      finish_stats();
    }
    SPION_STAMP(ord, 5);
    if (ok) prefetch_next();
    SPION_STAMP(ord, 6);
    // ------------------------------------------------------------------ output rows of this unit
    if (ok && !ctl) {
      float inv = 1.0f, lse2 = lse_fixed;
      if (!STORE_P) {
        const float l = l_part + __shfl_xor_sync(0xffffffffu, l_part, 16) + (float)(L - n_sel) * exp2f(-m2);
        inv = 1.0f / l;
        lse2 = m2 + log2f(l);
      } else if (nblk == 0) {
        lse2 = m2 + log2f((float)L * exp2f(-m2));
      }
      if (hf == 0) lse_out[(size_t)bh * L + r * BS + row] = lse2;
      // the accumulator rows sit in lanes 0-15 of every quadrant: those lanes write the whole row
      __nv_bfloat16* dst = O + (size_t)(pos.row0 + r * BS + row) * pos.ld + pos.x0;
#pragma unroll
      for (int h = 0; h < D / 32; ++h) {
        uint32_t v[32];
        if (nblk > 0) {
          tmem_ld32(t_lane + o_col + h * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
        }
        if (hf == 0) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 pk4;
            pk4.x = pack_bf16(__uint_as_float(v[j]) * inv, __uint_as_float(v[j + 1]) * inv);
            pk4.y = pack_bf16(__uint_as_float(v[j + 2]) * inv, __uint_as_float(v[j + 3]) * inv);
            pk4.z = pack_bf16(__uint_as_float(v[j + 4]) * inv, __uint_as_float(v[j + 5]) * inv);
            pk4.w = pack_bf16(__uint_as_float(v[j + 6]) * inv, __uint_as_float(v[j + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + h * 32 + j) = pk4;
          }
        }
      }
    }
    SPION_STAMP(ord, 7);
    // the next unit's S MMAs overwrite the accumulator columns read above
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    SPION_STAMP(ord, 8);
    if (threadIdx.x == 0) SPION_STAMP(ord, 9 + 0 * nblk);
#ifdef SPION_TRACE
    if (threadIdx.x == 0 && g_spion_trace && ord < g_spion_trace_units)
      g_spion_trace[((size_t)blockIdx.x * g_spion_trace_units + ord) * 16 + 15] = (unsigned long long)nblk;
#endif
    R = Rn;
    bh = bhn;
  }
  if (STORE_P && ctl && lane == 0) bulk_wait_read_all();          // shared memory must outlive the tile stores
  tc_fence_before();
  __syncthreads();
  if (ctl) tmem_dealloc(tmem, ncols);
}

}  // namespace

namespace tc {

// Opt in to the shared memory the kernels need and learn how many CTAs of them one SM holds (the
// persistent grid is that many per SM).
template <int D>
static int fwd_attrs(TcState* s, int device) {
  const int bytes = (int)fwd_smem_bytes<D>();
  int occ = 1 << 30, n = 0, rc;
#define SPION_FWD_ATTR(SP, SB)                                                                                      \
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_fwd_fused<D, SP, SB>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes)); \
  if ((rc = resident_ctas(k_fwd_fused<D, SP, SB>, device, FWD_THREADS, (size_t)bytes, 128, &n))) return rc;         \
  occ = n < occ ? n : occ;
  SPION_FWD_ATTR(false, false)
  SPION_FWD_ATTR(true, false)
  SPION_FWD_ATTR(false, true)
  SPION_FWD_ATTR(true, true)
#undef SPION_FWD_ATTR
  s->fwd_ctas = occ;
  return SPION_OK;
}

int fused_set_attrs(TcState* s, int d, int device) { return d == 64 ? fwd_attrs<64>(s, device) : fwd_attrs<32>(s, device); }

template <int D>
static int fwd_launch(spion_ctx* c, TcState* s, const void* Q, const void* K, const void* V, const float* keypad,
                      void* O, float* lse, void* P64) {
  const TcView vw = tc_view(c, s);
  const uint64_t vrows = (uint64_t)c->BH * vw.nnzb * BS;
  CUtensorMap mq, mk, mv, mp;
  int rc;
  if ((rc = make_operand_map(c, s, &mq, Q, D)) || (rc = make_operand_map(c, s, &mk, K, D)) ||
      (rc = make_operand_map(c, s, &mv, V, D)))
    return rc;
  if (P64) { if ((rc = make_map(s, &mp, P64, vrows, BS, BS, BS))) return rc; } else mp = mq;
  prof_mark(c, -1);
  // Masks whose rows all have at most four blocks run on the pipelined kernel for short rows
  // (tc_fwd_pipe.cu: about 1.7x less time per row, two CTAs per SM).  As soon as some rows are longer,
  // everything goes through this file's kernel: a second launch for a handful of long rows costs more
  // than the pipelining gains (measured at 5 % density, L = 4096: 79 us split against 70 us in one launch).
  const bool all_short = s->n_long == 0;
  const int rows_here = all_short ? 0 : vw.nb;
  const long long total = (long long)c->BH * rows_here;
  const float floor_v = keypad ? 0.0f : -100.0f;
  if (total > 0) {
    const int grid = (int)(total < (long long)s->sms * s->fwd_ctas ? total : (long long)s->sms * s->fwd_ctas);
#define SPION_FWD_LAUNCH(SP, SB)                                                                                  \
  k_fwd_fused<D, SP, SB><<<grid, FWD_THREADS, fwd_smem_bytes<D>(), c->stream>>>(                                   \
      mq, mk, mv, mp, (__nv_bfloat16*)O, lse, keypad, vw.row_info, vw.col_idx, vw.submask, c->L, vw.nnzb, c->BH,   \
      rows_here, c->heads, c->scale, floor_v, c->status_dev)
    if (P64) { if (vw.submask) SPION_FWD_LAUNCH(true, true); else SPION_FWD_LAUNCH(true, false); }
    else { if (vw.submask) SPION_FWD_LAUNCH(false, true); else SPION_FWD_LAUNCH(false, false); }
#undef SPION_FWD_LAUNCH
    SPION_LAUNCH_CHECK();
    c->launches += 1;
  }
  if (all_short && (rc = pipe_forward(c, s, mq, mk, mv, mp, P64 != nullptr, keypad, O, lse, 0))) return rc;
  prof_mark(c, SPION_STAGE_FUSED_FWD);
  return SPION_OK;
}

int fused_forward(spion_ctx* c, TcState* s, const void* Q, const void* K, const void* V, const float* keypad, void* O,
                  float* lse, void* P64_optional) {
  return c->d == 64 ? fwd_launch<64>(c, s, Q, K, V, keypad, O, lse, P64_optional)
                    : fwd_launch<32>(c, s, Q, K, V, keypad, O, lse, P64_optional);
}

}  // namespace tc
