// Fused forward for block rows of at most four blocks, software-pipelined across work units
// (sm_100a, bf16, 64x64 blocks).  Same arithmetic, semantics and outputs as k_fwd_fused (tc_fused.cu;
// replaces models/block_attn.cu:453-487), which keeps the rows of more than four blocks.
//
// Why a second kernel: a short row is a chain  loads -> S MMAs -> row softmax -> P V MMAs -> output rows
// in which the two MMA steps and the loads are pure latency (about a microsecond each) for the four math
// warps.  Here nothing of that chain is waited for in line:
//   * a control warp issues every TMA load, MMA and tile store and is the only one that waits on copies;
//   * tensor memory holds two accumulator sets and shared memory two Q / K sets, so the S tiles of unit
//     i+1 are computed while the math warps are still on unit i;
//   * the output rows of unit i are read out after the row statistics of unit i+1, when its P V product
//     has long retired;
//   * hand-offs are mbarrier arrivals (P written, accumulator set read out), never a CTA-wide barrier.
// Per unit i (set s = i & 1), math warps:   wait S(i) | statistics | output rows of unit i-1 | exp, P tiles
//                   control warp:            S(i+1) as soon as set s^1 is read out | P V(i) when P(i) is
//                                            written | then the loads of V(i+1) and Q, K(i+2)
//
// Two CTAs per SM (112 KB of tiles and 256 tensor-memory columns each).  Every wait is bounded.
#include "tc_tiles.cuh"

using namespace tc;

#ifdef SPION_TRACE
SPION_TRACE_SETTER(spion_debug_trace_pipe)
#endif

namespace {

constexpr int PIPE_THREADS = 160;          // warps 0-3: math (one TMEM quadrant each); warp 4: control
constexpr int NCH = ROW_NCH;

template <int D> constexpr size_t pipe_smem_bytes() {
  // Q x2 | K x4 x2 (P tiles reuse the K set when a K tile is as large as a P tile) | V x4 | [P x4] | barriers
  return (size_t)(2 + 2 * NCH + NCH) * OpTile<D>::BYTES + (D == 64 ? 0 : (size_t)NCH * VT_BYTES) + 128;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 32 consecutive values (16 packed words) of row i, columns [32 g, 32 g + 32), into a [64 x 64] K-major
// SWIZZLE_128B tile (16-byte chunk c of row i sits at chunk c ^ (i & 7)).
__device__ __forceinline__ void store_half_row(uint32_t tile, int i, int g, const uint32_t (&w)[16]) {
#pragma unroll
  for (int cc = 0; cc < 4; ++cc) {
    const int c = g * 4 + cc;
    const uint32_t addr = tile + i * 128 + ((c ^ (i & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * cc]), "r"(w[4 * cc + 1]),
                 "r"(w[4 * cc + 2]), "r"(w[4 * cc + 3])
                 : "memory");
  }
}

template <int D, bool STORE_P, bool SUB>
__global__ void __launch_bounds__(PIPE_THREADS, 2) k_fwd_pipe(const __grid_constant__ CUtensorMap tmQ,
                                                              const __grid_constant__ CUtensorMap tmK,
                                                              const __grid_constant__ CUtensorMap tmV,
                                                              const __grid_constant__ CUtensorMap tmP,
                                                              __nv_bfloat16* __restrict__ O, float* __restrict__ lse_out,
                                                              const float* __restrict__ keypad,
                                                              const int4* __restrict__ row_info,
                                                              const int* __restrict__ col_idx,
                                                              const uint8_t* __restrict__ submask, int L, int nnzb, int BH,
                                                              int rank0, int nrows, int heads, float scale, float floor_v,
                                                              int* status) {
  using T = OpTile<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t sbase = smem_u32(smem_raw);                   // must be 1024-aligned (checked below): no slack is reserved
  const uint32_t sQ = sbase;                                   // [2]
  const uint32_t sK = sQ + 2 * T::BYTES;                       // [2][4]
  const uint32_t sV = sK + 2 * NCH * T::BYTES;                 // [4]
  const uint32_t sPsep = sV + NCH * T::BYTES;                  // [4], D == 32 only
  const uint32_t bars = sPsep + (D == 64 ? 0 : NCH * VT_BYTES);
  const uint32_t bar_qk = bars, bar_v = bars + 16, bar_s = bars + 24, bar_o = bars + 40, bar_p = bars + 56,
                 bar_t = bars + 72, slot = bars + 88, abort_w = bars + 92, bar_x = bars + 96;
  uint32_t* slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (slot - sbase));
  volatile int* abort_ptr = reinterpret_cast<volatile int*>(smem_raw + (abort_w - sbase));
  auto sP = [&](int s, int t) -> uint32_t { return D == 64 ? sK + (s * NCH + t) * T::BYTES : sPsep + t * VT_BYTES; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool ctl = warp == 4;
  const int q = warp & 3;
  const int hf = lane >> 4;
  const int row = q * 16 + (lane & 15);
  const int G = (int)gridDim.x;
  const int total = (nrows - rank0) * BH;
  const int n_my = total > (int)blockIdx.x ? (total - (int)blockIdx.x + G - 1) / G : 0;
  constexpr uint32_t ncols = 256u;

  auto unit = [&](int i, RowRec& R, int& bh) {
    const int u = (int)blockIdx.x + i * G;
    const int rk = u / BH;
    bh = u - rk * BH;
    R = RowRec(row_info[rank0 + rk]);
  };

  if (ctl) {
    if (lane == 0) {
      int a = *reinterpret_cast<volatile int*>(status);
      if ((sbase & 1023u) != 0u) { report(status, ERR_LOAD_WAIT); a = 1; }      // the tiles need 1024-byte alignment
      *abort_ptr = a;
      for (int i = 0; i < 2; ++i) {
        mbar_init(bar_qk + 8 * i, 1);
        mbar_init(bar_s + 8 * i, 1);
        mbar_init(bar_o + 8 * i, 1);
        mbar_init(bar_p + 8 * i, 128);
        mbar_init(bar_t + 8 * i, 128);
      }
      mbar_init(bar_v, 1);
      mbar_init(bar_x, 1);
      fence_barrier_init();
    }
  }
  __syncthreads();
  if (*abort_ptr != 0) return;
  if (ctl) {
    tmem_alloc(slot, ncols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot_ptr;
  constexpr uint32_t IDESC_S = make_idesc_bf16(64, 64, 0, 0);
  constexpr uint32_t IDESC_O = make_idesc_bf16(64, D, 0, 1);

  if (ctl) {
    // ================================================================== control warp
    uint32_t ph_qk = 0, ph_v = 0, ph_p = 0, ph_o = 0, ph_t = 0, ph_x = 0;   // one bit per set (ph_v, ph_x: one bit)
    bool busy0 = false, busy1 = false;                            // accumulator set holds a unit that has not been read out
    bool ok = true;

    auto issue_qk = [&](int i) {                                  // all lanes
      RowRec R; int bh;
      unit(i, R, bh);
      if (R.nblk == 0) return;
      const int s = i & 1;
      const OpPos pos = op_pos(bh, L, heads, D);
      if (lane == 0) mbar_expect_tx(bar_qk + 8 * s, (1 + R.nblk) * T::BYTES);
      __syncwarp();
      if (lane == 0) tma_load_2d(sQ + s * T::BYTES, &tmQ, bar_qk + 8 * s, pos.x0, pos.row0 + R.r * BS);
      if (lane >= 1 && lane <= R.nblk)
        tma_load_2d(sK + (s * NCH + lane - 1) * T::BYTES, &tmK, bar_qk + 8 * s, pos.x0,
                    pos.row0 + R.col(lane - 1, col_idx) * BS);
    };
    auto issue_v = [&](int i) {                                   // all lanes
      RowRec R; int bh;
      unit(i, R, bh);
      if (R.nblk == 0) return;
      const OpPos pos = op_pos(bh, L, heads, D);
      if (lane == 0) mbar_expect_tx(bar_v, R.nblk * T::BYTES);
      __syncwarp();
      if (lane < R.nblk)
        tma_load_2d(sV + lane * T::BYTES, &tmV, bar_v, pos.x0, pos.row0 + R.col(lane, col_idx) * BS);
    };
    auto wait_all = [&](uint32_t bar, uint32_t parity, int code) -> bool {
      const bool w = __all_sync(0xffffffffu, mbar_wait(bar, parity));
      if (!w && lane == 0) report(status, code);
      return w;
    };
    auto issue_s = [&](int i) -> bool {                           // S tiles of unit i into set i & 1
      RowRec R; int bh;
      unit(i, R, bh);
      if (R.nblk == 0) return true;
      const int s = i & 1;
      if (s ? busy1 : busy0) {                                    // the set's previous unit must have been read out
        if (!wait_all(bar_t + 8 * s, (ph_t >> s) & 1, ERR_MMA2_WAIT)) return false;
        ph_t ^= 1u << s;
      }
      if (!wait_all(bar_qk + 8 * s, (ph_qk >> s) & 1, ERR_LOAD_WAIT)) return false;
      ph_qk ^= 1u << s;
      if (lane == 0) {
        tc_fence_after();
        const uint64_t dq0 = T::kmajor(sQ + s * T::BYTES, 0);
        uint64_t dk0 = T::kmajor(sK + s * NCH * T::BYTES, 0);
        for (int t = 0; t < R.nblk; ++t, dk0 = desc_advance(dk0, T::BYTES)) {
          const uint32_t d_addr = tmem + (uint32_t)s * 128u + ((uint32_t)((t & 1) * 16) << 16) + (uint32_t)(t >> 1) * 64u;
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            mma_bf16(d_addr, desc_advance(dq0, kk * T::K_STEP), desc_advance(dk0, kk * T::K_STEP), IDESC_S, kk > 0);
        }
        mma_commit(bar_s + 8 * s);
      }
      __syncwarp();
      if (s) busy1 = true; else busy0 = true;
      return true;
    };
    auto issue_pv = [&](int i) -> bool {                          // O = P V of unit i, then its tile stores
      RowRec R; int bh;
      unit(i, R, bh);
      if (R.nblk == 0) return true;
      const int s = i & 1;
      if (!wait_all(bar_p + 8 * s, (ph_p >> s) & 1, ERR_MMA_WAIT)) return false;
      ph_p ^= 1u << s;
      if (!wait_all(bar_v, ph_v & 1, ERR_LOAD_WAIT)) return false;
      ph_v ^= 1u;
      if (lane == 0) {
        tc_fence_after();
        uint64_t dp0 = ValTile::kmajor(sP(s, 0), 0), dv0 = T::mnmajor(sV, 0);
        for (int t = 0; t < R.nblk; ++t, dp0 = desc_advance(dp0, VT_BYTES), dv0 = desc_advance(dv0, T::BYTES)) {
#pragma unroll
          for (int kk = 0; kk < BS / 16; ++kk)
            mma_bf16(tmem + (uint32_t)s * 128u, desc_advance(dp0, kk * ValTile::K_STEP), desc_advance(dv0, kk * T::MN_STEP),
                     IDESC_O, (kk > 0 || t > 0) ? 1u : 0u);
        }
        // With a separate P buffer (D == 32) the math warps overwrite it as soon as they see bar_o: when the tiles
        // are also stored, bar_o must then wait for the stores' reads as well (see below).
        mma_commit((STORE_P && D != 64) ? bar_x : bar_o + 8 * s);
        if (STORE_P) {
          for (int t = 0; t < R.nblk; ++t)
            tma_store_2d(&tmP, sP(s, t), 0, (int)(((size_t)bh * nnzb + R.rp + t) * BS));
          bulk_commit();
        }
      }
      __syncwarp();
      if (STORE_P && D != 64) {
        if (!wait_all(bar_x, ph_x & 1, ERR_MMA2_WAIT)) return false;
        ph_x ^= 1u;
        if (lane == 0) { bulk_wait_read_all(); mbar_arrive(bar_o + 8 * s); }
        __syncwarp();
      }
      // the V buffers, this set's K (= P) buffers and Q are free once the product has retired
      if (!wait_all(bar_o + 8 * s, (ph_o >> s) & 1, ERR_MMA2_WAIT)) return false;
      ph_o ^= 1u << s;
      if (STORE_P && D == 64) {
        if (lane == 0) bulk_wait_read_all();
        __syncwarp();
      }
      return true;
    };

    if (n_my > 0) {
      issue_qk(0);
      issue_v(0);
      if (n_my > 1) issue_qk(1);
      ok = issue_s(0);
    }
    for (int i = 0; i < n_my && ok; ++i) {
      if (i + 1 < n_my) ok = issue_s(i + 1);
      if (ok) ok = issue_pv(i);
      if (!ok) break;
      if (i + 1 < n_my) issue_v(i + 1);
      if (i + 2 < n_my) issue_qk(i + 2);
    }
  } else {
    // ================================================================== math warps
    const uint32_t t_lane = tmem + ((uint32_t)(q * 32) << 16);
    const float sc2 = scale * LOG2E;
    uint32_t ph_s = 0, ph_o = 0;                                  // one bit per set
    bool ok = true;
    // the unit whose output rows are still in tensor memory
    bool prev_valid = false;
    int prev_s = 0, prev_nblk = 0;
    float prev_inv = 0.f, prev_lse = 0.f;
    __nv_bfloat16* prev_dst = nullptr;
    float* prev_lse_dst = nullptr;

    auto write_out = [&]() -> bool {                              // output rows of the previous unit
      if (prev_nblk > 0) {
        if (!mbar_wait(bar_o + 8 * prev_s, (ph_o >> prev_s) & 1)) { report(status, ERR_MMA2_WAIT); return false; }
        ph_o ^= 1u << prev_s;
        tc_fence_after();
      }
      if (hf == 0) *prev_lse_dst = prev_lse;
      // the accumulator rows sit in lanes 0-15 of every quadrant: those lanes write the whole row
#pragma unroll
      for (int h = 0; h < D / 32; ++h) {
        uint32_t v[32];
        if (prev_nblk > 0) {
          tmem_ld32(t_lane + (uint32_t)prev_s * 128u + h * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
        }
        if (hf == 0) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 o4;
            o4.x = pack_bf16(__uint_as_float(v[j]) * prev_inv, __uint_as_float(v[j + 1]) * prev_inv);
            o4.y = pack_bf16(__uint_as_float(v[j + 2]) * prev_inv, __uint_as_float(v[j + 3]) * prev_inv);
            o4.z = pack_bf16(__uint_as_float(v[j + 4]) * prev_inv, __uint_as_float(v[j + 5]) * prev_inv);
            o4.w = pack_bf16(__uint_as_float(v[j + 6]) * prev_inv, __uint_as_float(v[j + 7]) * prev_inv);
            *reinterpret_cast<uint4*>(prev_dst + h * 32 + j) = o4;
          }
        }
      }
      if (prev_nblk > 0) {                                        // the set may take the S tiles of the unit after next
        tc_fence_before();
        mbar_arrive(bar_t + 8 * prev_s);
      }
      return true;
    };

    for (int i = 0; i < n_my && ok; ++i) {
      RowRec R; int bh;
      unit(i, R, bh);
      const int s = i & 1;
      const int rp = R.rp, nblk = R.nblk;
      const uint32_t t_set = t_lane + (uint32_t)s * 128u;
      const float* kp = keypad ? keypad + (size_t)bh * L : nullptr;
      const OpPos pos = op_pos(bh, L, heads, D);
      const int rh2 = (q >> 1) * 2;
      auto quarter_ok = [&](int blk, int half) -> bool { return !SUB || ((submask[blk] >> (rh2 + half)) & 1); };
      int n_sel = nblk * BS;
      if (SUB) {
        n_sel = 0;
        for (int t = 0; t < nblk; ++t) n_sel += 32 * __popc((submask[rp + t] >> rh2) & 3);
      }
      float m2 = floor_v * LOG2E, mraw = -INFINITY, l_part = 0.f;
      SPION_STAMP(i, 0);
      if (nblk > 0) {
        if (!mbar_wait(bar_s + 8 * s, (ph_s >> s) & 1)) { report(status, ERR_MMA_WAIT); ok = false; break; }
        ph_s ^= 1u << s;
        tc_fence_after();
        SPION_STAMP(i, 1);
        // ---- row maximum over the selected keys
        for (int p = 0; p < 2; ++p) {
          const int t = 2 * p + hf;
          const bool mine = t < nblk;
          const int c = mine ? R.col(t, col_idx) : 0;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t v[32];
            tmem_ld32(t_set + p * 64 + half * 32, v);
            tmem_ld_wait();
            if (mine && quarter_ok(rp + t, half)) {
              if (!kp) {                                          // the scale is positive: compare raw scores
                float ma = mraw, mb = -INFINITY, mc = -INFINITY, md = -INFINITY;
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
      }
      m2 = fmaxf(m2, mraw * sc2);
      m2 = fmaxf(m2, __shfl_xor_sync(0xffffffffu, m2, 16));        // both owners of a row agree
      SPION_STAMP(i, 2);
      if (prev_valid) {
        if (!write_out()) { ok = false; break; }
      }
      SPION_STAMP(i, 3);
      float inv = 1.0f, lse2;
      if (nblk > 0) {
        // ---- exponentials against the row maximum, P tiles (normalised when they are also stored)
        uint32_t wp[2][32];
#pragma unroll
        for (int p = 0; p < 2; ++p) {
          const int t = 2 * p + hf;
          const bool mine = t < nblk;
          const int c = mine ? R.col(t, col_idx) : 0;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t v[32];
            tmem_ld32(t_set + p * 64 + half * 32, v);
            tmem_ld_wait();
            if (mine && quarter_ok(rp + t, half)) {
              float la = 0.f, lb = 0.f;
#pragma unroll
              for (int j = 0; j < 32; j += 2) {
                float h0 = m2, h1 = m2;
                if (kp) { h0 = fmaf(kp[c * BS + half * 32 + j], LOG2E, m2); h1 = fmaf(kp[c * BS + half * 32 + j + 1], LOG2E, m2); }
                const float e0 = ex2(fmaf(__uint_as_float(v[j]), sc2, -h0)), e1 = ex2(fmaf(__uint_as_float(v[j + 1]), sc2, -h1));
                if (j & 2) lb += e0 + e1; else la += e0 + e1;
                wp[p][half * 16 + (j >> 1)] = pack_bf16(e0, e1);
              }
              l_part += la + lb;
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) wp[p][half * 16 + j] = 0u;
            }
            if (!STORE_P && mine) {
              uint32_t w16[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) w16[j] = wp[p][half * 16 + j];
              store_half_row(sP(s, t), row, half, w16);
            }
          }
        }
        const float l = l_part + __shfl_xor_sync(0xffffffffu, l_part, 16) + (float)(L - n_sel) * exp2f(-m2);
        lse2 = m2 + log2f(l);
        if (STORE_P) {
          // 1/l as a sum of two bf16 values: the packed product then carries one rounding of the result only
          const float il = 1.0f / l;
          const float il_h = bf16_hi(pack_bf16(0.f, il));
          const uint32_t inv_hi = pack_bf16(il_h, il_h), inv_lo = pack_bf16(il - il_h, il - il_h);
#pragma unroll
          for (int p = 0; p < 2; ++p) {
            const int t = 2 * p + hf;
            if (t < nblk) {
#pragma unroll
              for (int half = 0; half < 2; ++half) {
                uint32_t w16[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const uint32_t x = wp[p][half * 16 + j];
                  w16[j] = fma_bf16x2(x, inv_hi, mul_bf16x2(x, inv_lo));
                }
                store_half_row(sP(s, t), row, half, w16);
              }
            }
          }
        } else {
          inv = 1.0f / l;
        }
        fence_proxy_async();                                      // P rows -> visible to the MMA and the tile stores
        tc_fence_before();
        mbar_arrive(bar_p + 8 * s);
      } else {
        lse2 = m2 + log2f((float)L * exp2f(-m2));
      }
      SPION_STAMP(i, 4);
#ifdef SPION_TRACE
      if (threadIdx.x == 0 && g_spion_trace && i < g_spion_trace_units)
        g_spion_trace[((size_t)blockIdx.x * g_spion_trace_units + i) * 16 + 15] = (unsigned long long)nblk;
#endif
      prev_valid = true;
      prev_s = s;
      prev_nblk = nblk;
      prev_inv = inv;
      prev_lse = lse2;
      prev_dst = O + (size_t)(pos.row0 + R.r * BS + row) * pos.ld + pos.x0;
      prev_lse_dst = lse_out + (size_t)bh * L + R.r * BS + row;
    }
    if (ok && prev_valid) write_out();
  }
  tc_fence_before();
  __syncthreads();
  if (ctl) tmem_dealloc(tmem, ncols);
}

}  // namespace

namespace tc {

template <int D>
static int pipe_attrs(TcState* s, int device) {
  const int bytes = (int)pipe_smem_bytes<D>();
  int occ = 1 << 30, n = 0, rc;
#define SPION_PIPE_ATTR(SP, SB)                                                                                    \
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_fwd_pipe<D, SP, SB>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes)); \
  if ((rc = resident_ctas(k_fwd_pipe<D, SP, SB>, device, PIPE_THREADS, (size_t)bytes, 256, &n))) return rc;        \
  occ = n < occ ? n : occ;
  SPION_PIPE_ATTR(false, false)
  SPION_PIPE_ATTR(true, false)
  SPION_PIPE_ATTR(false, true)
  SPION_PIPE_ATTR(true, true)
#undef SPION_PIPE_ATTR
  s->pipe_ctas = occ;
  return SPION_OK;
}

int pipe_set_attrs(TcState* s, int d, int device) { return d == 64 ? pipe_attrs<64>(s, device) : pipe_attrs<32>(s, device); }

template <int D>
static int pipe_launch(spion_ctx* c, TcState* s, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                       const CUtensorMap& mp, bool store_p, const float* keypad, void* O, float* lse, int rank0) {
  const TcView vw = tc_view(c, s);
  const long long total = (long long)c->BH * (vw.nb - rank0);
  if (total <= 0) return SPION_OK;
  const long long cap = (long long)s->sms * s->pipe_ctas;
  const int grid = (int)(total < cap ? total : cap);
  const float floor_v = keypad ? 0.0f : -100.0f;
#define SPION_PIPE_LAUNCH(SP, SB)                                                                                    \
  k_fwd_pipe<D, SP, SB><<<grid, PIPE_THREADS, pipe_smem_bytes<D>(), c->stream>>>(                                     \
      mq, mk, mv, mp, (__nv_bfloat16*)O, lse, keypad, vw.row_info, vw.col_idx, vw.submask, c->L, vw.nnzb, c->BH, rank0, \
      vw.nb, c->heads, c->scale, floor_v, c->status_dev)
  if (store_p) { if (vw.submask) SPION_PIPE_LAUNCH(true, true); else SPION_PIPE_LAUNCH(true, false); }
  else { if (vw.submask) SPION_PIPE_LAUNCH(false, true); else SPION_PIPE_LAUNCH(false, false); }
#undef SPION_PIPE_LAUNCH
  SPION_LAUNCH_CHECK();
  c->launches += 1;
  return SPION_OK;
}

int pipe_forward(spion_ctx* c, TcState* s, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                 const CUtensorMap& mp, bool store_p, const float* keypad, void* O, float* lse, int rank0) {
  return c->d == 64 ? pipe_launch<64>(c, s, mq, mk, mv, mp, store_p, keypad, O, lse, rank0)
                    : pipe_launch<32>(c, s, mq, mk, mv, mp, store_p, keypad, O, lse, rank0);
}

}  // namespace tc
