// Column side of the recompute backward as a streaming pipeline (sm_100a, bf16, 64x64 blocks):
//     dK[c] = sum_r dS(r,c)^T Q[r],   dV[c] = sum_r P(r,c)^T dO[r]        (models/block_attn.cu:526, :536)
// with P and dS rebuilt on chip from Q, K, V, dO, the forward's log-sum-exp and the row kernel's delta
// (see tc_recompute.cu for the formulas).  One persistent CTA per SM:
//
//   warp 0 (loads)     streams the entries of its block columns, two at a time ("pairs"), through a ring of pair
//                      slots in shared memory (each slot: Q[r], dO[r] of both entries, by TMA; K[c], V[c] once per
//                      column into one of two sets).  The ring runs on across columns; column and pair records come
//                      from two small per-pattern tables and are requested a column ahead.
//   warp 9 (S / dP)    as soon as a pair has landed: S = [Q0; Q1] K^T and dP = [dO0; dO1] V^T, one M = 128 product
//                      each, into one of three tensor-memory sets, up to two pairs ahead of the math warps.
//   warps 1-8 (math)   wait for S / dP of a pair (normally long complete), form P and dS for their 32 columns of
//                      their row, write them as bf16 tiles [query x key] into one of two tile sets and signal with
//                      one mbarrier arrival per warp; no CTA-wide barrier exists in the steady state.  A column's
//                      rows are written out after the first pair of the next column, when its last MMAs have retired.
//   warp 10 (dK / dV)  when the tiles of a pair are written: dV += P^T dO and dK += dS^T Q into the column's
//                      accumulators (dK in lanes 0-15 of every quadrant, dV in lanes 16-31; two column sets).
// Two issuing warps because the products of one pair are 24 instructions and one thread issues a small
// tcgen05.mma at best every 25-30 ns: with a single issuer the MMA stream, not the arithmetic, set the pace.
//
// Every wait is bounded; on a time-out the waiting warp records a code in the status word and the CTA winds down.
#include "tc_tiles.cuh"

using namespace tc;

#ifdef SPION_TRACE
SPION_TRACE_SETTER(spion_debug_trace_col)
#endif

namespace {

constexpr int CS_THREADS = 352;                      // warp 0: loads; warps 1-8: math; warp 9: S / dP MMAs; warp 10: dK / dV MMAs

template <int D> struct ColStream {
  using T = OpTile<D>;
  static constexpr int NP = (D == 64) ? 4 : 8;       // pair slots in the ring
  static constexpr uint32_t SLOT = 4 * T::BYTES;     // Q0, Q1, dO0, dO1 (the two Q tiles and the two dO tiles are each one 128-row operand)
  static constexpr uint32_t KV_SET = 2 * T::BYTES;   // K[c], V[c] of a column; two sets, columns alternate
  static constexpr uint32_t PD_SET = 4 * VT_BYTES;   // P0, dS0, P1, dS1
  static constexpr size_t SMEM = (size_t)NP * SLOT + 2 * KV_SET + 2 * PD_SET + 512;
};

__device__ __forceinline__ float ex2c(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void store_half_row_c(uint32_t tile, int i, int g, const uint32_t (&w)[16]) {
#pragma unroll
  for (int cc = 0; cc < 4; ++cc) {
    const int c = g * 4 + cc;
    const uint32_t addr = tile + i * 128 + ((c ^ (i & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * cc]), "r"(w[4 * cc + 1]),
                 "r"(w[4 * cc + 2]), "r"(w[4 * cc + 3])
                 : "memory");
  }
}

// position in the stream of pairs of this CTA: unit ordinal i, pair k of that unit
// The record of the column after the current one is requested a whole column early, so that crossing a column
// boundary never waits for a load.
struct PairCur {
  int i, k;
  int4 cur, nxt;                                      // column records {block column, first pair, pairs, entries} of units i, i+1
  __device__ int line() const { return cur.x; }
  __device__ int pbeg() const { return cur.y; }
  __device__ int npairs() const { return cur.z; }
  __device__ int n() const { return cur.w; }
  __device__ int cnt() const { return min(2, cur.w - 2 * k); }   // entries of pair k
};

template <int D, bool SUB>
__global__ void __launch_bounds__(CS_THREADS, 1) k_bwd_col_stream(const __grid_constant__ CUtensorMap tmQ,
                                                                  const __grid_constant__ CUtensorMap tmK,
                                                                  const __grid_constant__ CUtensorMap tmV,
                                                                  const __grid_constant__ CUtensorMap tmdO,
                                                                  const float* __restrict__ lse_in,
                                                                  const float* __restrict__ delta_in,
                                                                  const float* __restrict__ keypad,
                                                                  __nv_bfloat16* __restrict__ dK,
                                                                  __nv_bfloat16* __restrict__ dV,
                                                                  const int4* __restrict__ col_rec,
                                                                  const int4* __restrict__ col_pair,
                                                                  const uint8_t* __restrict__ submask, int L, int BH,
                                                                  int nb, int heads, float scale, int* status) {
  using C = ColStream<D>;
  using T = OpTile<D>;
  constexpr int NP = C::NP;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t sbase = smem_u32(smem_raw);                   // must be 1024-aligned (checked below)
  const uint32_t sKV = sbase + NP * C::SLOT;
  const uint32_t sPD = sKV + 2 * C::KV_SET;
  const uint32_t bars = sPD + 2 * C::PD_SET;
  // pfull[ps]: tiles of a pair slot landed; pdone[ps]: the MMAs that read the slot retired;
  // s_ready[set]: S / dP of a pair are in tensor memory; p_ready[set]: its P / dS tiles are written (8 arrivals, one per math warp);
  // acc_done[par]: a column's accumulators are complete; acc_free[par]: they have been read out (8 arrivals, one per math warp)
  const uint32_t pfull = bars, pdone = bars + 64, s_ready = bars + 128, p_ready = bars + 152, acc_done = bars + 168,
                 acc_free = bars + 184, kv_full = bars + 200, slot = bars + 216, abort_w = bars + 220, kv_free = bars + 224,
                 t_free = bars + 240;                           // t_free[3]: S / dP set read out by the math warps (8 arrivals, one per math warp)
  uint32_t* slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (slot - sbase));
  volatile int* abort_ptr = reinterpret_cast<volatile int*>(smem_raw + (abort_w - sbase));
  auto sK = [&](int par) { return sKV + par * C::KV_SET; };
  auto sV = [&](int par) { return sKV + par * C::KV_SET + T::BYTES; };
  auto sQ = [&](int ps, int e) { return sbase + ps * C::SLOT + e * T::BYTES; };
  auto sdO = [&](int ps, int e) { return sbase + ps * C::SLOT + (2 + e) * T::BYTES; };
  auto sP = [&](int set, int e) { return sPD + set * C::PD_SET + (2 * e) * VT_BYTES; };
  auto sDS = [&](int set, int e) { return sPD + set * C::PD_SET + (2 * e + 1) * VT_BYTES; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = (int)gridDim.x;
  const int total = nb * BH;
  const int n_my = total > (int)blockIdx.x ? (total - (int)blockIdx.x + G - 1) / G : 0;
  constexpr uint32_t ncols = 512u;
  constexpr uint32_t ACC = 384u;                                 // three S / dP sets of 128 columns, then two accumulator sets of 64

  // columns of one (b,h) matrix together, the longest first: unit ordinal i of this CTA -> (bh, record)
  auto bh_of = [&](int i) -> int { return ((int)blockIdx.x + i * G) / nb; };
  auto rec_of = [&](int i) -> int4 {
    if (i >= n_my) return make_int4(0, 0, 0, 0);
    const int uu = (int)blockIdx.x + i * G;
    return col_rec[uu - (uu / nb) * nb];
  };
  auto shift = [&](PairCur& c) { ++c.i; c.k = 0; c.cur = c.nxt; c.nxt = rec_of(c.i + 1); };
  auto skip = [&](PairCur& c) { while (c.i < n_my && c.cur.w == 0) shift(c); };    // columns without entries
  auto start = [&](PairCur& c) { c.i = 0; c.k = 0; c.cur = rec_of(0); c.nxt = rec_of(1); skip(c); };
  auto next = [&](PairCur& c) {
    if (++c.k >= c.npairs()) { shift(c); skip(c); }
  };

  if (warp == 0 && lane == 0) {
    int a = *reinterpret_cast<volatile int*>(status);
    if ((sbase & 1023u) != 0u) { report(status, ERR_LOAD_WAIT); a = 1; }
    *abort_ptr = a;
    for (int i = 0; i < NP; ++i) { mbar_init(pfull + 8 * i, 1); mbar_init(pdone + 8 * i, 1); }
    mbar_init(s_ready + 16, 1);
    for (int i = 0; i < 3; ++i) mbar_init(t_free + 8 * i, 8);       // one arrival per math warp
    for (int i = 0; i < 2; ++i) {
      mbar_init(s_ready + 8 * i, 1);
      mbar_init(p_ready + 8 * i, 8);
      mbar_init(acc_done + 8 * i, 1);
      mbar_init(acc_free + 8 * i, 8);
      mbar_init(kv_full + 8 * i, 1);
      mbar_init(kv_free + 8 * i, 1);
    }
    fence_barrier_init();
  }
  __syncthreads();
  if (*abort_ptr != 0) return;
  if (warp == 0) {
    tmem_alloc(slot, ncols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot_ptr;
  constexpr uint32_t IDESC_S = make_idesc_bf16(64, 64, 0, 0);
  constexpr uint32_t IDESC_T = make_idesc_bf16(64, D, 1, 1);

  auto wait_all = [&](uint32_t bar, uint32_t parity, int code) -> bool {     // whole warp
    const bool w = __all_sync(0xffffffffu, mbar_wait(bar, parity));
    if (!w && lane == 0) report(status, code);
    return w;
  };
  constexpr uint32_t IDESC_S2 = make_idesc_bf16(128, 64, 0, 0);       // both entries of a pair as one 128-row operand
  const uint64_t KM_BASE = T::kmajor(sbase, 0), MN_BASE = T::mnmajor(sbase, 0), VMN_BASE = ValTile::mnmajor(sbase, 0);

  if (warp == 0) {
    // ================================================================== loader warp
    // Pairs in stream order into the ring: a slot is refilled when the MMAs of the pair it held have retired,
    // K[c] / V[c] of a column when the S / dP products of the column before last (same set) have retired.  Both conditions are produced by
    // the MMA warp from pairs that are already loaded, so these waits cannot deadlock.
    bool ok = true;
    int kv_loads0 = 0, kv_loads1 = 0;                             // columns whose K / V went to set 0 / 1
    PairCur c;
    start(c);
    // pair records (block rows of the two entries): lane l keeps the record of pair l of the current column and of the
    // next one, both requested a column early
    int4 prs = make_int4(0, -1, 0, 0), prs_n = prs;
    int cached_i = -1;
    for (int jl = 0; ok && c.i < n_my; ++jl, next(c)) {
      const int ps = jl % NP;
      if (c.i != cached_i) {                                     // first pair of a column
        prs = (cached_i >= 0 && c.i == cached_i + 1) ? prs_n : (lane < c.npairs() ? col_pair[c.pbeg() + lane] : prs);
        cached_i = c.i;
        if (c.i + 1 < n_my && lane < c.nxt.z) prs_n = col_pair[c.nxt.y + lane];
      }
      int4 pr;
      if (c.k < 32) {
        pr.x = __shfl_sync(0xffffffffu, prs.x, c.k);
        pr.y = __shfl_sync(0xffffffffu, prs.y, c.k);
      } else {
        pr = col_pair[c.pbeg() + c.k];
      }
      if (jl >= NP && !wait_all(pdone + 8 * ps, (uint32_t)(jl / NP - 1) & 1u, ERR_MMA2_WAIT)) { ok = false; break; }
      const int par = c.i & 1;
      if (c.k == 0) {
        const int loads = par ? kv_loads1 : kv_loads0;
        if (loads >= 1 && !wait_all(kv_free + 8 * par, (uint32_t)(loads - 1) & 1u, ERR_MMA2_WAIT)) { ok = false; break; }
      }
      const int cnt = c.cnt();
      const OpPos pos = op_pos(bh_of(c.i), L, heads, D);
      if (lane == 0) {
        mbar_expect_tx(pfull + 8 * ps, 2 * cnt * T::BYTES);
        if (c.k == 0) mbar_expect_tx(kv_full + 8 * par, 2 * T::BYTES);
      }
      __syncwarp();
      if (c.k == 0) {
        if (lane == 4) tma_load_2d(sK(par), &tmK, kv_full + 8 * par, pos.x0, pos.row0 + c.line() * BS);
        if (lane == 5) tma_load_2d(sV(par), &tmV, kv_full + 8 * par, pos.x0, pos.row0 + c.line() * BS);
        if (par) ++kv_loads1; else ++kv_loads0;
      }
      if (lane < 2 * cnt) {
        const int e = lane >> 1;
        const int orow = pos.row0 + (e ? pr.y : pr.x) * BS;
        if (lane & 1) tma_load_2d(sdO(ps, e), &tmdO, pfull + 8 * ps, pos.x0, orow);
        else tma_load_2d(sQ(ps, e), &tmQ, pfull + 8 * ps, pos.x0, orow);
      }
    }
  } else if (warp == 9) {
    // ================================================================== S / dP warp
    bool ok = true;
    int kv_waits0 = 0, kv_waits1 = 0;
    // S = [Q0; Q1] K^T and dP = [dO0; dO1] V^T of pair j into tensor-memory set j & 1: one M = 128 chain each (rows
    // 0-63: first entry, 64-127: second; with a single entry the upper half is computed from stale tiles and ignored)
    auto issue_sdp = [&](const PairCur& c, int j) -> bool {
      const int ps = j % NP, set = j % 3, par = c.i & 1;
      if (j >= 3 && !wait_all(t_free + 8 * set, (uint32_t)(j / 3 - 1) & 1u, ERR_MMA_WAIT)) return false;   // pair j - 3 read out
      if (c.k == 0) {
        const int w = par ? kv_waits1 : kv_waits0;
        if (!wait_all(kv_full + 8 * par, (uint32_t)w & 1u, ERR_LOAD_WAIT)) return false;
        if (par) ++kv_waits1; else ++kv_waits0;
      }
      if (!wait_all(pfull + 8 * ps, (uint32_t)(j / NP) & 1u, ERR_LOAD_WAIT)) return false;
      if (lane == 0) {
        tc_fence_after();
        // every operand descriptor is one add on a descriptor of the buffer base (built once, outside the loop)
        const uint64_t dq0 = desc_advance(KM_BASE, ps * C::SLOT), do0 = desc_advance(dq0, 2 * T::BYTES);
        const uint64_t dk0 = desc_advance(KM_BASE, NP * C::SLOT + par * C::KV_SET), dv0 = desc_advance(dk0, T::BYTES);
        const uint32_t d0 = tmem + (uint32_t)set * 128u;
        // the two products are independent accumulation chains: alternate them, so that an MMA never has to wait
        // for the one issued just before it
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          mma_bf16(d0, desc_advance(dq0, kk * T::K_STEP), desc_advance(dk0, kk * T::K_STEP), IDESC_S2, kk > 0);
          mma_bf16(d0 + 64u, desc_advance(do0, kk * T::K_STEP), desc_advance(dv0, kk * T::K_STEP), IDESC_S2, kk > 0);
        }
        mma_commit(s_ready + 8 * set);
        if (c.k + 1 == c.npairs()) mma_commit(kv_free + 8 * par);   // K[c], V[c] are read by these products only
      }
      __syncwarp();
      return true;
    };
    PairCur SC;
    start(SC);
    for (int js = 0; ok && SC.i < n_my; ++js, next(SC)) ok = issue_sdp(SC, js);
  } else if (warp == 10) {
    // ================================================================== dK / dV warp
    bool ok = true;
    int acc_uses0 = 0, acc_uses1 = 0;                             // columns that have gone to accumulator set 0 / 1
    // dV += P^T dO, dK += dS^T Q of pair j into the accumulators of its column
    auto issue_dkdv = [&](const PairCur& c, int j) -> bool {
      const int ps = j % NP, set = j & 1, par = c.i & 1;
      if (c.k == 0) {                                            // the accumulator set's previous column must be read out
        const int uses = par ? acc_uses1 : acc_uses0;
        if (uses >= 1 && !wait_all(acc_free + 8 * par, (uint32_t)(uses - 1) & 1u, ERR_MMA2_WAIT)) return false;
      }
      if (!wait_all(p_ready + 8 * set, (uint32_t)(j >> 1) & 1u, ERR_MMA_WAIT)) return false;
      SPION_STAMP_T(320, j, 5);
      if (lane == 0) {
        tc_fence_after();
        const int cnt = c.cnt();
        const uint32_t acc = tmem + ACC + (uint32_t)par * 64u;
        for (int e = 0; e < cnt; ++e) {
          const uint32_t first = (c.k == 0 && e == 0) ? 0u : 1u;
          const uint64_t dp0 = desc_advance(VMN_BASE, NP * C::SLOT + 2 * C::KV_SET + set * C::PD_SET + 2 * e * VT_BYTES);
          const uint64_t dds0 = desc_advance(dp0, VT_BYTES);
          const uint64_t bq0 = desc_advance(MN_BASE, ps * C::SLOT + e * T::BYTES), bo0 = desc_advance(bq0, 2 * T::BYTES);
#pragma unroll
          for (int kk = 0; kk < BS / 16; ++kk) {                 // the two accumulators alternate (independent chains)
            mma_bf16(acc + (16u << 16), desc_advance(dp0, kk * ValTile::MN_STEP), desc_advance(bo0, kk * T::MN_STEP), IDESC_T,
                     (kk > 0) ? 1u : first);                     // dV += P^T dO   (lanes 16-31)
            mma_bf16(acc, desc_advance(dds0, kk * ValTile::MN_STEP), desc_advance(bq0, kk * T::MN_STEP), IDESC_T,
                     (kk > 0) ? 1u : first);                     // dK += dS^T Q   (lanes 0-15)
          }
        }
        mma_commit(pdone + 8 * ps);
        if (c.k + 1 == c.npairs()) mma_commit(acc_done + 8 * par);
      }
      __syncwarp();
      if (c.k + 1 == c.npairs()) { if (par) ++acc_uses1; else ++acc_uses0; }
      return true;
    };

    PairCur DC;
    start(DC);
    for (int jd = 0; ok && DC.i < n_my; ++jd, next(DC)) {
      SPION_STAMP_T(320, jd, 0);
      ok = issue_dkdv(DC, jd);
      SPION_STAMP_T(320, jd, 3);
    }
  } else {
    // ================================================================== math warps
    const int q = warp & 3, g = (warp - 1) >> 2;                 // TMEM quadrant, column half of the tiles
    // S / dP of a pair are one 128-row accumulator: quadrants 0-1 hold the first entry's rows, 2-3 the second's
    const int es = q >> 1;                                       // entry of the pair this warp works on
    const int row = (q & 1) * 32 + lane;                         // its query row inside the entry's block
    const int orow = q * 16 + (lane & 15);                       // output row (the column accumulators are 64-row ones)
    const uint32_t t_lane = tmem + ((uint32_t)(q * 32) << 16);
    const float sc2 = scale * LOG2E;
    bool ok = true;
    int j = 0;                                                   // pairs seen so far
    int reads0 = 0, reads1 = 0;                                  // columns read out of accumulator set 0 / 1
    bool prev_valid = false;
    int prev_par = 0;
    __nv_bfloat16* prev_dst = nullptr;

    auto write_rows = [&](__nv_bfloat16* dst, uint32_t taddr, bool have) {
      if (D == 64) {
        uint32_t v[32];
        if (have) { tmem_ld32(taddr + g * 32, v); tmem_ld_wait(); }
        else {
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = 0u;
        }
#pragma unroll
        for (int e = 0; e < 32; e += 8)
          *reinterpret_cast<uint4*>(dst + e) =
              make_uint4(pack_bf16(__uint_as_float(v[e]), __uint_as_float(v[e + 1])),
                         pack_bf16(__uint_as_float(v[e + 2]), __uint_as_float(v[e + 3])),
                         pack_bf16(__uint_as_float(v[e + 4]), __uint_as_float(v[e + 5])),
                         pack_bf16(__uint_as_float(v[e + 6]), __uint_as_float(v[e + 7])));
      } else {
        uint32_t v[16];
        if (have) { tmem_ld16(taddr + g * 16, v); tmem_ld_wait(); }
        else {
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = 0u;
        }
#pragma unroll
        for (int e = 0; e < 16; e += 8)
          *reinterpret_cast<uint4*>(dst + e) =
              make_uint4(pack_bf16(__uint_as_float(v[e]), __uint_as_float(v[e + 1])),
                         pack_bf16(__uint_as_float(v[e + 2]), __uint_as_float(v[e + 3])),
                         pack_bf16(__uint_as_float(v[e + 4]), __uint_as_float(v[e + 5])),
                         pack_bf16(__uint_as_float(v[e + 6]), __uint_as_float(v[e + 7])));
      }
    };
    // rows of the column whose accumulators are still in tensor memory (lanes 0-15: dK, lanes 16-31: dV)
    auto write_prev = [&]() -> bool {
      const int reads = prev_par ? reads1 : reads0;
      if (!mbar_wait(acc_done + 8 * prev_par, (uint32_t)reads & 1u)) { report(status, ERR_MMA2_WAIT); return false; }
      tc_fence_after();
      write_rows(prev_dst, t_lane + ACC + (uint32_t)prev_par * 64u, true);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_free + 8 * prev_par);
      if (prev_par) ++reads1; else ++reads0;
      prev_valid = false;
      return true;
    };

    // Per-row inputs of this lane's entry of a pair come from two dependent loads (pair record, then lse / delta).
    // Both run ahead of the pair stream, across column boundaries: the record of pair j + 2 and the lse / delta of
    // pair j + 1 are requested while pair j is worked on, so neither load is ever waited for.
    float lse_n = 0.f, nds_n = 0.f;                               // pair j + 1
    bool mine_n = false;
    uint8_t sub_n = 0;
    int4 prB = make_int4(-1, -1, 0, 0);                           // pair j + 2: its record, its (b,h) matrix
    int bhB = 0;
    PairCur P2;                                                   // position of the next record to request
    start(P2);
    auto request_record = [&]() {
      if (P2.i < n_my) { prB = col_pair[P2.pbeg() + P2.k]; bhB = bh_of(P2.i); next(P2); }
      else prB = make_int4(-1, -1, 0, 0);
    };
    auto request_inputs = [&]() {                                 // stage B -> stage A
      const int r = es ? prB.y : prB.x;
      mine_n = r >= 0;
      lse_n = 0.f; nds_n = 0.f; sub_n = 0;
      if (mine_n) {
        const size_t ri = (size_t)bhB * L + (size_t)r * BS + row;
        lse_n = lse_in[ri];
        nds_n = delta_in[ri];                                     // raw: any arithmetic here would wait for the load
        sub_n = SUB ? submask[es ? prB.w : prB.z] : (uint8_t)0xff;
      }
    };
    request_record();                                             // pair 0
    request_inputs();
    request_record();                                             // pair 1
    PairCur U;
    U.i = 0; U.k = 0; U.cur = rec_of(0); U.nxt = rec_of(1);
    for (; U.i < n_my && ok; shift(U)) {
      const int i = U.i;
      const int bh = bh_of(i);
      const int n = U.n();
      const OpPos pos = op_pos(bh, L, heads, D);
      __nv_bfloat16* dst = (lane < 16 ? dK : dV) + (size_t)(pos.row0 + U.line() * BS + orow) * pos.ld + pos.x0 + g * (D / 2);
      if (n == 0) {                                              // a column without entries: zero rows, no tensor memory
        write_rows(dst, 0u, false);
        continue;
      }
      const int par = i & 1;
      const float* kp = keypad ? keypad + (size_t)bh * L + U.line() * BS + g * 32 : nullptr;
      const int npairs = U.npairs();
      for (int k = 0; k < npairs && ok; ++k, ++j) {
        const int set = j & 1;
        const float lse = lse_n, nds = -nds_n * scale;
        const bool mine = mine_n, live = mine_n && ((sub_n >> ((q & 1) * 2 + g)) & 1);
        SPION_STAMP_T(32, j, 8);
        request_inputs();                                         // pair j + 1, from the record requested a pair ago
        request_record();                                         // pair j + 2
        // the tile set of pair j - 2 must have been consumed (its MMAs were issued two pairs ago)
        if (j >= 2 && !mbar_wait(pdone + 8 * ((j - 2) % NP), (uint32_t)((j - 2) / NP) & 1u)) { report(status, ERR_MMA2_WAIT); ok = false; break; }
        SPION_STAMP_T(32, j, 12);
        if (!mbar_wait(s_ready + 8 * (j % 3), (uint32_t)(j / 3) & 1u)) { report(status, ERR_MMA_WAIT); ok = false; break; }
        tc_fence_after();
        SPION_STAMP_T(32, j, 9);
        uint32_t sv[32], gv[32];
        tmem_ld32(t_lane + (uint32_t)(j % 3) * 128u + g * 32, sv);
        tmem_ld32(t_lane + (uint32_t)(j % 3) * 128u + 64u + g * 32, gv);
        tmem_ld_wait();
        if (mine) {
          uint32_t wp[16], wds[16];
          if (live) {
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
              float h0 = lse, h1 = lse;
              if (kp) { h0 = fmaf(kp[c], LOG2E, lse); h1 = fmaf(kp[c + 1], LOG2E, lse); }
              const float p0 = ex2c(fmaf(__uint_as_float(sv[c]), sc2, -h0)), p1 = ex2c(fmaf(__uint_as_float(sv[c + 1]), sc2, -h1));
              wp[c >> 1] = pack_bf16(p0, p1);
              wds[c >> 1] = pack_bf16(p0 * fmaf(__uint_as_float(gv[c]), scale, nds), p1 * fmaf(__uint_as_float(gv[c + 1]), scale, nds));
            }
          } else {
#pragma unroll
            for (int c = 0; c < 16; ++c) { wp[c] = 0u; wds[c] = 0u; }
          }
          store_half_row_c(sP(set, es), row, g, wp);
          store_half_row_c(sDS(set, es), row, g, wds);
        }
        fence_proxy_async();                                      // tiles -> visible to the MMAs
        tc_fence_before();
        __syncwarp();                                             // one arrival per warp: hundreds of arrivals on one
        if (lane == 0) {                                          // barrier word would serialise in shared memory
          mbar_arrive(t_free + 8 * (j % 3));                      // S / dP of this pair are in registers: the set is free
          mbar_arrive(p_ready + 8 * set);
        }
        SPION_STAMP_T(32, j, 10);
        if (k == 0 && prev_valid) ok = write_prev();
        SPION_STAMP_T(32, j, 11);              // the previous column's last MMAs have long retired
      }
      if (!ok) break;
      if (prev_valid) ok = write_prev();                          // (only when the loop above did not run its k == 0 branch)
      prev_valid = true;
      prev_par = par;
      prev_dst = dst;
    }
    if (ok && prev_valid) write_prev();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, ncols);
}

}  // namespace

namespace tc {

template <int D>
static int cs_attrs() {
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_bwd_col_stream<D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ColStream<D>::SMEM));
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_bwd_col_stream<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ColStream<D>::SMEM));
  return SPION_OK;
}

int col_stream_set_attrs(int d) { return d == 64 ? cs_attrs<64>() : cs_attrs<32>(); }

template <int D>
static int cs_launch(spion_ctx* c, TcState* s, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                     const CUtensorMap& mdo, const float* lse, const float* keypad, void* dK, void* dV) {
  const TcView vw = tc_view(c, s);
  const long long total = (long long)c->BH * vw.nb;
  const int grid = (int)(total < (long long)s->sms ? total : (long long)s->sms);       // one CTA per SM (all 512 TMEM columns)
  if (vw.submask)
    k_bwd_col_stream<D, true><<<grid, CS_THREADS, ColStream<D>::SMEM, c->stream>>>(
        mq, mk, mv, mdo, lse, s->delta_ws, keypad, (__nv_bfloat16*)dK, (__nv_bfloat16*)dV, s->col_rec, s->col_pair,
        vw.submask, c->L, c->BH, vw.nb, c->heads, c->scale, c->status_dev);
  else
    k_bwd_col_stream<D, false><<<grid, CS_THREADS, ColStream<D>::SMEM, c->stream>>>(
        mq, mk, mv, mdo, lse, s->delta_ws, keypad, (__nv_bfloat16*)dK, (__nv_bfloat16*)dV, s->col_rec, s->col_pair,
        vw.submask, c->L, c->BH, vw.nb, c->heads, c->scale, c->status_dev);
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}

int col_stream_backward(spion_ctx* c, TcState* s, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                        const CUtensorMap& mdo, const float* lse, const float* keypad, void* dK, void* dV) {
  return c->d == 64 ? cs_launch<64>(c, s, mq, mk, mv, mdo, lse, keypad, dK, dV)
                    : cs_launch<32>(c, s, mq, mk, mv, mdo, lse, keypad, dK, dV);
}

}  // namespace tc
