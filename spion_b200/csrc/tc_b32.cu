// Block-sparse attention on masks of 32 x 32 blocks, on the blocks themselves (sm_100a, bf16, head_dim 64):
// forward and the recompute backward without ever forming an unselected block.
//
// tcgen05.mma needs M = 64 or 128 rows, a 32-wide block row has 32.  The kernels therefore gather up to
// four selected 32-row tiles of the OTHER operand into one 128-row operand and, where the 32 rows of the
// unit's own block have to be the output rows, compute the transposed product:
//
//   k_b32<FWD>  unit = block row r (32 queries) of one (b,h) matrix
//               S^T[128 keys x 32 q] = K_g Q_r^T           (K_g: four selected key blocks, K-major A, M = 128)
//               row statistics across the keys, P^T = exp2(.) as bf16 rows of 32 queries
//               O^T[64 d x 32 q]   += V_g^T P^T            (V_g as MN-major A, P^T as MN-major B)
//               two passes over the row's blocks (maximum, then exponentials); replaces
//               models/block_attn.cu:453-487 for 32-wide masks
//   k_b32<ROW>  unit = block row r:   S^T, dP^T = V_g dO_r^T  ->  dS^T  ->  dQ^T += K_g^T dS^T;  writes delta
//   k_b32<COL>  unit = block column c (32 keys): four selected query blocks gathered,
//               S[128 q x 32 keys] = Q_g K_c^T, dP = dO_g V_c^T  ->  P, dS rows of 32 keys
//               dV^T[64 d x 32 keys] += dO_g^T P,  dK^T += Q_g^T dS          (models/block_attn.cu:489-545)
//
// In the transposed kernels a thread owns one KEY (a tensor-memory lane) and 32 queries (columns): the
// log-sum-exp and delta of the backward are per column and come from shared memory, the forward reduces
// its maxima and sums across lanes once per unit with a halving shuffle tree.  Neither P nor dS is written
// to global memory.  All three kernels are the same pipeline: a control warp (TMA loads, MMA issue) and
// four math warps (one per tensor-memory quadrant = one gathered block each), two stages of operand
// buffers, S / dP double-buffered in tensor memory, the unit's accumulator double-buffered so that the
// output rows of unit u are written while unit u+1 is computed.  Every mbarrier wait is bounded.
#include <cuda.h>

#include "common.cuh"
#include "tc_tiles.cuh"

using namespace tc;

#ifdef SPION_TRACE
SPION_TRACE_SETTER(spion_debug_trace_b32)
#endif

namespace {

enum : int { B32_FWD = 0, B32_ROW = 1, B32_COL = 2 };

constexpr int B32 = 32;                    // block size these kernels serve
constexpr int HD = 64;                     // head dimension
constexpr int GN = 4;                      // gathered blocks per job (128 rows)
constexpr int B32_THREADS = 224;           // warps 0-3: math; warp 4: loads; warp 5: first products; warp 6: second products
constexpr uint32_t TB = B32 * HD * 2;      // one [32 x 64] bf16 operand tile: 4096 bytes
constexpr uint32_t GB = GN * TB;           // gathered operand: [128 x 64], 16 KB
constexpr uint32_t VB = 128 * B32 * 2;     // P^T / dS^T / P / dS: [128 x 32] bf16, 64-byte rows, 8 KB

template <int MODE> struct Cfg {
  static constexpr bool FWD = MODE == B32_FWD, ROW = MODE == B32_ROW, COL = MODE == B32_COL;
  // Rings of gathered operands.  G0 = K_g (FWD, ROW) or Q_g (COL); G1 = V_g or dO_g.  A slot of K_g is free as
  // soon as S has been computed in the forward (three slots: the loads run two jobs ahead); in the row kernel
  // K_g is read again by the dQ product, three slots keep one job of distance there too.
  static constexpr int D0 = COL ? 2 : 3, D1 = 2;
  static constexpr int NVAL = COL ? 2 : 1;             // value buffers per stage (COL: P and dS)
  static constexpr int NUNIT = FWD ? 1 : 2;            // small operands of a unit (Q | Q, dO | K, V)
  static constexpr int UBUF = FWD ? 2 : 1;             // buffers for them
  static constexpr uint32_t OFF_G1 = D0 * GB, OFF_V = OFF_G1 + D1 * GB, OFF_U = OFF_V + 2 * NVAL * VB;
  static constexpr uint32_t TILES = OFF_U + UBUF * NUNIT * TB;
  static constexpr uint32_t SMEM = 1024 + TILES;       // + alignment slack
  static constexpr uint32_t TMEM_COLS = FWD ? 128 : 256;
  // tensor-memory columns: S (two stages), dP (two stages), accumulators
  static constexpr uint32_t S_COL = 0, DP_COL = 64, ACC_COL = FWD ? 64 : 128;
};

__device__ __forceinline__ float ex2a(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 32 bf16 values (16 packed words) as row i of a [128 x 32] tile with 64-byte rows in the SWIZZLE_64B image
// (16-byte chunk c of row i sits at chunk c ^ ((i >> 1) & 3)): the MN-major B operand of the second products.
__device__ __forceinline__ void store_row64(uint32_t tile, int i, const uint32_t (&w)[16]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t addr = tile + i * 64 + ((c ^ ((i >> 1) & 3)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * c]), "r"(w[4 * c + 1]),
                 "r"(w[4 * c + 2]), "r"(w[4 * c + 3])
                 : "memory");
  }
}

// Reduce a[n] over the 32 lanes of the warp for every n: afterwards lane n holds the result for index n
// (returned).  Halving tree: 16 + 8 + 4 + 2 + 1 shuffles.
template <bool MAX>
__device__ __forceinline__ float lanes_reduce32(float (&a)[32], int lane) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    const bool up = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < off; ++i) {
      const float keep = up ? a[i + off] : a[i];
      const float send = up ? a[i] : a[i + off];
      const float got = __shfl_xor_sync(0xffffffffu, send, off);
      a[i] = MAX ? fmaxf(keep, got) : keep + got;
    }
  }
  return a[0];
}

// Where a warp is in the CTA's sequence of units and jobs.  The control warp runs three of these (loads,
// first products, second products), every math warp one; all of them walk the same sequence.
// A line record is {start in the index array, blocks | line << 16, id0 | id1 << 16, id2 | id3 << 16}: the ids of
// the first four blocks come with the record, and the record of the following unit is requested when
// the cursor enters a unit, so that no dependent global load sits between two jobs.
template <int MODE> struct Cursor {
  const int4* rec;
  int total, BH, stride;
  int u, uc, jg, jb;           // unit index in the launch; units with work, jobs, jobs with second products seen so far
  int rp, n, line, bh;         // the unit: start in the index array, blocks, block row / column, (b,h) matrix
  int id01, id23;              // its first four block ids
  int nch, njobs, jl;
  bool valid;
  int4 nrec;                   // record of unit u + stride (valid if nvalid)
  bool nvalid;
  __device__ static int rec_id(const int4& r, int t) { return (((t & 2) ? r.w : r.z) >> ((t & 1) * 16)) & 0xffff; }
  __device__ static int rec_n(const int4& r) { return r.y & 0xffff; }
  __device__ void set(const int4& r) {
    rp = r.x; n = r.y & 0xffff; line = r.y >> 16; id01 = r.z; id23 = r.w;
    bh = u - (u / BH) * BH;
    nch = (n + GN - 1) / GN;
    njobs = Cfg<MODE>::FWD ? 2 * nch : nch;
  }
  __device__ void request_next() {
    const int un = u + stride;
    nvalid = un < total;
    if (nvalid) nrec = rec[un / BH];
  }
  __device__ void init(const int4* rec_, int total_, int BH_) {
    rec = rec_; total = total_; BH = BH_; stride = gridDim.x;
    u = blockIdx.x; uc = 0; jg = 0; jb = 0; jl = 0;
    valid = u < total;
    if (valid) set(rec[u / BH]);
    request_next();
  }
  __device__ void next_unit() {
    u += stride; jl = 0;
    valid = nvalid;
    if (valid) set(nrec);
    request_next();
  }
  __device__ int next_bh() const { const int un = u + stride; return un - (un / BH) * BH; }
  __device__ bool empty() const { return valid && n == 0; }
  __device__ int first_id(int t) const { return (((t & 2) ? id23 : id01) >> ((t & 1) * 16)) & 0xffff; }
  // the job at the cursor
  __device__ bool is_b() const { return !Cfg<MODE>::FWD || jl >= nch; }       // has second products
  __device__ int chunk() const { return (Cfg<MODE>::FWD && jl >= nch) ? jl - nch : jl; }
  __device__ int t0() const { return chunk() * GN; }
  __device__ int nt() const { return min(GN, n - t0()); }
  __device__ bool first_b() const { return Cfg<MODE>::FWD ? jl == nch : jl == 0; }
  __device__ bool last() const { return jl == njobs - 1; }
  // step to the next job (callers skip empty units themselves)
  __device__ void advance() {
    ++jg;
    if (is_b()) ++jb;
    if (++jl == njobs) { ++uc; next_unit(); }
  }
};

// Barrier slots (8 bytes each) in shared memory.  A parity wait only tells two consecutive phases of a barrier
// apart, so every waiter waits for every phase of the barriers it uses: the barriers of K_g / Q_g, S and dP
// get one phase per job (index j), those of V_g / dO_g, the value buffers and the second products one phase
// per job that has second products (index jb; in the backward kernels every job has them, jb = j).
enum : int {
  BAR_FULL0 = 0,    // [3] gathered operand 0 (+ the unit's small operands with the unit's first job) has landed
  BAR_FULL1 = 3,    // [2] gathered operand 1 has landed
  BAR_FREE0 = 5,    // [3] the products that read slot j % D0 of ring 0 have retired
  BAR_FREE1 = 8,    // [2] ... slot j & 1 of ring 1
  BAR_SREADY = 10,  // [2] first products of the job retired: S (and dP) are in tensor memory
  BAR_MDONE = 12,   // [2] the four math warps have read S / dP out of tensor memory
  BAR_ODONE = 14,   // [2] second products of the job retired: its value buffers are free
  BAR_OFULL = 16,   // [2] the unit's accumulator is complete
  BAR_OFREE = 18,   // [2] ... and has been read out
  BAR_UFREE = 20,   // [2] the first products of a unit no longer need its small operands
  BAR_PREADY = 22,  // [2] the four math warps have written the value rows of a job with second products
  BAR_COUNT = 24
};

template <int MODE>
__global__ void __launch_bounds__(B32_THREADS, 2)
k_b32(const __grid_constant__ CUtensorMap tmG0, const __grid_constant__ CUtensorMap tmG1,
      const __grid_constant__ CUtensorMap tmU0, const __grid_constant__ CUtensorMap tmU1,
      const __nv_bfloat16* __restrict__ in0,      // ROW: dO
      const __nv_bfloat16* __restrict__ in1,      // ROW: O
      const float* __restrict__ lse_in,           // ROW / COL
      const float* __restrict__ delta_in,         // COL
      const float* __restrict__ keypad,
      __nv_bfloat16* __restrict__ out0,           // FWD: O, ROW: dQ, COL: dK
      __nv_bfloat16* __restrict__ out1,           // COL: dV
      float* __restrict__ fout,                   // FWD: lse, ROW: delta
      const int4* __restrict__ recs, const int* __restrict__ idx, int L, int BH, int nlines, int heads, float scale,
      float floor_v, int* status) {
  using C = Cfg<MODE>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) unsigned long long s_bars[BAR_COUNT];
  __shared__ __align__(8) unsigned long long s_math_bar;
  __shared__ uint32_t s_slot;
  __shared__ int s_abort;
  __shared__ __align__(16) float s_red0[4][32];   // FWD: per-warp maxima; ROW: lse; COL: key padding (two units each)
  __shared__ __align__(16) float s_red1[4][32];   // FWD: per-warp sums;   ROW: -delta scale (two units)
  __shared__ __align__(16) float s_mw[4][32];     // FWD: the unit's maxima, one copy per math warp
  __shared__ __align__(16) float s_inv[32];       // FWD: 1 / denominator

  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  auto sG0 = [&](int k) -> uint32_t { return sbase + k * GB; };
  auto sG1 = [&](int k) -> uint32_t { return sbase + C::OFF_G1 + k * GB; };
  auto sVA = [&](int st) -> uint32_t { return sbase + C::OFF_V + st * C::NVAL * VB; };
  auto sVB = [&](int st) -> uint32_t { return sbase + C::OFF_V + st * C::NVAL * VB + VB; };
  auto sU = [&](int ub, int k) -> uint32_t { return sbase + C::OFF_U + (ub * C::NUNIT + k) * TB; };
  const uint32_t bars = smem_u32(s_bars);
  auto bar = [&](int which, int i) -> uint32_t { return bars + (which + i) * 8; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int total = nlines * BH;
  const float sc2 = scale * LOG2E;

  if (tid == 0) {
    s_abort = *reinterpret_cast<volatile int*>(status);
    for (int i = 0; i < BAR_COUNT; ++i) {
      const bool by_math = (i >= BAR_MDONE && i < BAR_MDONE + 2) || (i >= BAR_OFREE && i < BAR_OFREE + 2) || i >= BAR_PREADY;
      mbar_init(bar(i, 0), by_math ? 4 : 1);
    }
    mbar_init(smem_u32(&s_math_bar), 4);
    fence_barrier_init();
  }
  __syncthreads();
  if (s_abort != 0) return;
  if (warp == 4) {
    tmem_alloc(smem_u32(&s_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_slot;

  // bounded wait of one thread; a failure is recorded in the status word: the low three bits say what kind of wait
  // gave up (as in the other tensor-core kernels), bits 4-20 which one of this kernel's waits, bits 24-26 which kernel
  auto wait1 = [&](uint32_t b, uint32_t parity, int code) -> bool {
    if (mbar_wait(b, parity)) return true;
    report(status, code | (0x1000000 << MODE));
    return false;
  };

  if (warp == 4) {
    // =================================================================== loader warp
    Cursor<MODE> cl;
    cl.init(recs, total, BH);
    while (cl.empty()) cl.next_unit();
    // Block id of this lane's gathered tile (lanes 0-3 and 8-11: tiles 0-3 of G0 / G1): from the record for
    // the first chunk, otherwise loaded when the previous job's copies were issued.
    const int li = lane & 7;
    int pblk = 0;
    bool ok = true;
    while (ok && cl.valid) {
      const int j = cl.jg, jb = cl.jb, s0 = j % C::D0, s1 = jb & 1;
      const int ub = C::UBUF == 2 ? (cl.uc & 1) : 0;
      const bool two = !C::FWD || cl.is_b();                               // G1 as well
      if (lane == 0) {
        if (j >= C::D0) ok = wait1(bar(BAR_FREE0, s0), ((uint32_t)(j / C::D0) & 1u) ^ 1u, ERR_MMA2_WAIT | 0x10);
        if (ok && two && jb >= 2) ok = wait1(bar(BAR_FREE1, s1), ((uint32_t)(jb >> 1) & 1u) ^ 1u, ERR_MMA2_WAIT | 0x20);
        if (ok && cl.jl == 0 && cl.uc >= C::UBUF)          // the unit that used this set of small operands before
          ok = wait1(bar(BAR_UFREE, ub), (C::UBUF == 2 ? ((uint32_t)(cl.uc >> 1) & 1u) : ((uint32_t)cl.uc & 1u)) ^ 1u, ERR_MMA_WAIT | 0x40);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      SPION_STAMP_T(128, j, 0);
      const int t0 = cl.t0(), nt = cl.nt();
      const OpPos pos = op_pos(cl.bh, L, heads, HD);
      const int blk = t0 == 0 ? cl.first_id(li & 3) : pblk;
      if (lane == 0) {
        mbar_expect_tx(bar(BAR_FULL0, s0), (uint32_t)nt * TB + (cl.jl == 0 ? C::NUNIT * TB : 0u));
        if (two) mbar_expect_tx(bar(BAR_FULL1, s1), (uint32_t)nt * TB);
      }
      __syncwarp();
      if (lane < nt) tma_load_2d(sG0(s0) + lane * TB, &tmG0, bar(BAR_FULL0, s0), pos.x0, pos.row0 + blk * B32);
      if (two && lane >= 8 && lane < 8 + nt)
        tma_load_2d(sG1(s1) + (lane - 8) * TB, &tmG1, bar(BAR_FULL1, s1), pos.x0, pos.row0 + blk * B32);
      if (cl.jl == 0) {
        if (lane == 16) tma_load_2d(sU(ub, 0), &tmU0, bar(BAR_FULL0, s0), pos.x0, pos.row0 + cl.line * B32);
        if (C::NUNIT == 2 && lane == 17)
          tma_load_2d(sU(ub, 1), &tmU1, bar(BAR_FULL0, s0), pos.x0, pos.row0 + cl.line * B32);
      }
      cl.advance();
      while (cl.empty()) cl.next_unit();
      if (cl.valid && cl.t0() > 0 && li < cl.nt()) pblk = idx[cl.rp + cl.t0() + li];
      SPION_STAMP_T(128, j, 1);
    }
  } else if (warp == 5) {
    // =================================================================== first products (one thread)
    if (lane == 0) {
      constexpr uint32_t IDESC_1 = make_idesc_bf16(128, B32, 0, 0);      // [128 x 64] . [32 x 64]^T
      Cursor<MODE> cm;
      cm.init(recs, total, BH);
      while (cm.empty()) cm.next_unit();
      bool ok = true;
      while (ok && cm.valid) {
        const int j = cm.jg, s0 = j % C::D0, s1 = cm.jb & 1, st = j & 1;      // backward kernels: jb = j
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        const int ub = C::UBUF == 2 ? (cm.uc & 1) : 0;
        SPION_STAMP_T(160, j, 2);
        ok = wait1(bar(BAR_FULL0, s0), (uint32_t)(j / C::D0) & 1u, ERR_LOAD_WAIT | 0x100);
        if (ok && !C::FWD) ok = wait1(bar(BAR_FULL1, s1), ph, ERR_LOAD_WAIT | 0x200);
        if (ok && j >= 2) ok = wait1(bar(BAR_MDONE, st), ph ^ 1u, ERR_MMA_WAIT | 0x400);      // S / dP columns read out
        if (!ok) break;
        SPION_STAMP_T(160, j, 3);
        tc_fence_after();
        const uint64_t a0 = OpTile<HD>::kmajor(sG0(s0), 0), b0 = OpTile<HD>::kmajor(sU(ub, 0), 0);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          mma_bf16(tmem + C::S_COL + st * 32, desc_advance(a0, kk * 32), desc_advance(b0, kk * 32), IDESC_1, kk > 0);
        if (!C::FWD) {
          const uint64_t a1 = OpTile<HD>::kmajor(sG1(s1), 0), b1 = OpTile<HD>::kmajor(sU(ub, 1), 0);
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk)
            mma_bf16(tmem + C::DP_COL + st * 32, desc_advance(a1, kk * 32), desc_advance(b1, kk * 32), IDESC_1, kk > 0);
        }
        mma_commit(bar(BAR_SREADY, st));
        if (C::FWD) mma_commit(bar(BAR_FREE0, s0));                      // K_g is not read again
        if (C::ROW) mma_commit(bar(BAR_FREE1, s1));                      // V_g is not read again
        if (cm.last()) mma_commit(bar(BAR_UFREE, ub));
        SPION_STAMP_T(160, j, 4);
        cm.advance();
        while (cm.empty()) cm.next_unit();
      }
    }
    __syncwarp();                     // the idle lanes wait here for the issuing lane: the CTA barrier below is warp-aligned
  } else if (warp == 6) {
    // =================================================================== second products (one thread)
    if (lane == 0) {
      constexpr uint32_t IDESC_2 = make_idesc_bf16(64, B32, 1, 1);       // [128 x 64]^T . [128 x 32]
      Cursor<MODE> co;
      co.init(recs, total, BH);
      while (co.empty()) co.next_unit();
      bool ok = true;
      while (ok && co.valid) {
        if (co.is_b()) {
          const int j = co.jg, jb = co.jb, s0 = j % C::D0, s1 = jb & 1, ob = co.uc & 1;
          const int st = s1;                                                  // value buffers of the job
          const uint32_t ph = (uint32_t)(jb >> 1) & 1u;
          SPION_STAMP_T(192, j, 5);
          ok = wait1(bar(BAR_PREADY, s1), ph, ERR_MMA_WAIT | 0x1000);
          if (ok && C::FWD) ok = wait1(bar(BAR_FULL1, s1), ph, ERR_LOAD_WAIT | 0x2000);       // V_g
          // (already complete: the first products waited for them; this thread observes the copies itself)
          if (ok && !C::FWD) ok = wait1(bar(BAR_FULL0, s0), (uint32_t)(j / C::D0) & 1u, ERR_LOAD_WAIT | 0x4000);
          if (ok && C::COL) ok = wait1(bar(BAR_FULL1, s1), ph, ERR_LOAD_WAIT | 0x8000);
          // the accumulator of the unit before the previous one must have been read out
          if (ok && co.first_b() && co.uc >= 2) ok = wait1(bar(BAR_OFREE, ob), ((uint32_t)(co.uc >> 1) & 1u) ^ 1u, ERR_MMA2_WAIT | 0x10000);
          if (!ok) break;
          SPION_STAMP_T(192, j, 6);
          tc_fence_after();
          const int ksteps = 2 * co.nt();                                   // 16 gathered rows per step
          const bool fresh = co.first_b();
          const uint32_t acc = tmem + C::ACC_COL + (C::COL ? (uint32_t)ob * 32u : ((uint32_t)(ob * 16) << 16));
          if (C::COL) {
            const uint64_t aq = OpTile<HD>::mnmajor(sG0(s0), 0), ao = OpTile<HD>::mnmajor(sG1(s1), 0);
            const uint64_t bp = make_smem_desc(sVA(st), VB, 512, LAYOUT_SW64), bd = make_smem_desc(sVB(st), VB, 512, LAYOUT_SW64);
            for (int kk = 0; kk < ksteps; ++kk) {
              const uint32_t accum = (kk > 0 || !fresh) ? 1u : 0u;
              mma_bf16(acc + (16u << 16), desc_advance(ao, kk * 2048), desc_advance(bp, kk * 1024), IDESC_2, accum);   // dV^T
              mma_bf16(acc, desc_advance(aq, kk * 2048), desc_advance(bd, kk * 1024), IDESC_2, accum);                 // dK^T
            }
          } else {
            const uint64_t a = OpTile<HD>::mnmajor(C::FWD ? sG1(s1) : sG0(s0), 0);     // V_g (forward) or K_g (dQ)
            const uint64_t b = make_smem_desc(sVA(st), VB, 512, LAYOUT_SW64);
            for (int kk = 0; kk < ksteps; ++kk)
              mma_bf16(acc, desc_advance(a, kk * 2048), desc_advance(b, kk * 1024), IDESC_2, (kk > 0 || !fresh) ? 1u : 0u);
          }
          mma_commit(bar(BAR_ODONE, st));
          if (C::FWD || C::COL) mma_commit(bar(BAR_FREE1, s1));
          if (C::ROW || C::COL) mma_commit(bar(BAR_FREE0, s0));
          if (co.last()) mma_commit(bar(BAR_OFULL, ob));
          SPION_STAMP_T(192, j, 7);
        }
        co.advance();
        while (co.empty()) co.next_unit();
      }
    }
    __syncwarp();
  } else {
    // =================================================================== math warps
    Cursor<MODE> c;
    c.init(recs, total, BH);
    const uint32_t t_lane = tmem + ((uint32_t)(warp * 32) << 16);
    const int grow = warp * 32 + lane;                    // this thread's row of the gathered operand and of the value tiles
    const float floor2 = floor_v * LOG2E;
    const uint32_t bar_math = smem_u32(&s_math_bar);
    uint32_t pmath = 0;
    bool ok = true;
    // all 128 math threads meet here; bounded like every other wait (a warp that gave up never arrives)
    auto math_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_math);
      const bool good = mbar_wait(bar_math, pmath);
      pmath ^= 1u;
      return good;
    };
    // this warp has read the S / dP columns st and, for a job with second products, written its rows of value buffer sv
    auto job_done = [&](int st, int sv) {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar(BAR_MDONE, st));
        if (sv >= 0) mbar_arrive(bar(BAR_PREADY, sv));
      }
    };
    // before the value rows of a job with second products are written: the products that read the buffer two such
    // jobs ago have retired (every warp waits, also one without a block in this job: see the note at the barrier list)
    auto values_free = [&](int jb) -> bool {
      if (jb < 2 || mbar_wait(bar(BAR_ODONE, jb & 1), ((uint32_t)(jb >> 1) & 1u) ^ 1u)) return true;
      report(status, ERR_MMA2_WAIT | 0x40000);
      return false;
    };

    // ROW: the dO and O words of this thread's quarter row and the row's lse, for the unit after the current one
    uint4 pa0 = make_uint4(0, 0, 0, 0), pa1 = pa0, pb0 = pa0, pb1 = pa0;
    float plse = 0.f;
    bool pre_unit = false;
    auto row_fetch = [&](size_t vec, size_t off0, int ld) {
      const size_t off = off0 + (size_t)(tid >> 2) * ld + (tid & 3) * 16;
      pa0 = *reinterpret_cast<const uint4*>(in0 + off); pa1 = *reinterpret_cast<const uint4*>(in0 + off + 8);
      pb0 = *reinterpret_cast<const uint4*>(in1 + off); pb1 = *reinterpret_cast<const uint4*>(in1 + off + 8);
      if (tid < 32) plse = lse_in[vec + tid];
    };
    // COL: lse and -delta scale of this thread's row in the next job; block id of its row in the job after
    float nx0 = 0.f, nx1 = 0.f;
    int pblk = 0;
    bool pre_job = false;

    while (ok && c.valid) {
      const OpPos pos = op_pos(c.bh, L, heads, HD);
      const int line = c.line, bh = c.bh, n = c.n, rp = c.rp, nch = c.nch;
      const size_t vec0 = (size_t)bh * L + (size_t)line * B32;             // first row / key of the unit in [BH, L] arrays
      const size_t out_off = (size_t)(pos.row0 + line * B32) * pos.ld + pos.x0;
      if (n == 0) {
        // a line without selected blocks: zero output rows (FWD: the denominator is L exp(-floor))
        const int row = tid >> 2, part = tid & 3;
        const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
        uint4* d0 = reinterpret_cast<uint4*>(out0 + out_off + (size_t)row * pos.ld + part * 16);
        d0[0] = zero4; d0[1] = zero4;
        if (C::COL) {
          uint4* d1 = reinterpret_cast<uint4*>(out1 + out_off + (size_t)row * pos.ld + part * 16);
          d1[0] = zero4; d1[1] = zero4;
        }
        if (C::FWD && tid < 32) fout[vec0 + tid] = floor2 + log2f((float)L * exp2f(-floor2));
        if (C::ROW && tid < 32) fout[vec0 + tid] = 0.f;
        c.next_unit();
        continue;
      }
      const int ub = c.uc & 1, ob = c.uc & 1;
      const uint32_t pfull = (uint32_t)(c.uc >> 1) & 1u;
      const float* kp = keypad ? keypad + (size_t)bh * L : nullptr;

      if (C::FWD) {
        // ------------------------------------------------ pass A: maxima per query, kept per lane (= per key slot)
        float mx[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) mx[i] = -INFINITY;
        for (int jl = 0; jl < nch && ok; ++jl) {
          const int st = c.jg & 1, t0 = jl * GN, nt = min(GN, n - t0);
          float pad = 0.f;
          if (kp && warp < nt) pad = kp[(t0 == 0 ? c.first_id(warp) : idx[rp + t0 + warp]) * B32 + lane] * LOG2E;
          SPION_STAMP_T(0, c.jg, 8);
          if (!mbar_wait(bar(BAR_SREADY, st), (uint32_t)(c.jg >> 1) & 1u)) { report(status, ERR_MMA_WAIT | 0x20000); ok = false; break; }
          SPION_STAMP_T(0, c.jg, 9);
          tc_fence_after();
          if (warp < nt) {
            uint32_t v[32];
            tmem_ld32(t_lane + C::S_COL + st * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) mx[i] = fmaxf(mx[i], fmaf(__uint_as_float(v[i]), sc2, -pad));
          }
          SPION_STAMP_T(0, c.jg, 10);
          job_done(st, -1);
          c.advance();
        }
        if (!ok) break;
        s_red0[warp][lane] = lanes_reduce32<true>(mx, lane);
        if (!math_sync()) { report(status, ERR_MMA_WAIT | 0x100000); ok = false; break; }
        // every warp keeps its own copy of the 32 maxima (no second CTA-wide meeting)
        s_mw[warp][lane] = fmaxf(fmaxf(floor2, s_red0[0][lane]), fmaxf(fmaxf(s_red0[1][lane], s_red0[2][lane]), s_red0[3][lane]));
        __syncwarp();
        // ------------------------------------------------ pass B: exponentials, P^T rows, sums per query
        float z[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) z[i] = 0.f;
        for (int jl = 0; jl < nch && ok; ++jl) {
          const int st = c.jg & 1, t0 = jl * GN, nt = min(GN, n - t0);
          float pad = 0.f;
          if (kp && warp < nt) pad = kp[(t0 == 0 ? c.first_id(warp) : idx[rp + t0 + warp]) * B32 + lane] * LOG2E;
          SPION_STAMP_T(0, c.jg, 8);
          if (!mbar_wait(bar(BAR_SREADY, st), (uint32_t)(c.jg >> 1) & 1u)) { report(status, ERR_MMA_WAIT | 0x20000); ok = false; break; }
          SPION_STAMP_T(0, c.jg, 9);
          tc_fence_after();
          const int sv = c.jb & 1;
          if (!values_free(c.jb)) { ok = false; break; }
          if (warp < nt) {
            uint32_t v[32], w[16];
            tmem_ld32(t_lane + C::S_COL + st * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float e0 = ex2a(fmaf(__uint_as_float(v[i]), sc2, -(pad + s_mw[warp][i])));
              const float e1 = ex2a(fmaf(__uint_as_float(v[i + 1]), sc2, -(pad + s_mw[warp][i + 1])));
              z[i] += e0; z[i + 1] += e1;
              w[i >> 1] = pack_bf16(e0, e1);
            }
            store_row64(sVA(sv), grow, w);
            fence_proxy_async();
          }
          SPION_STAMP_T(0, c.jg, 10);
          job_done(st, sv);
          c.advance();
        }
        if (!ok) break;
        s_red1[warp][lane] = lanes_reduce32<false>(z, lane);
        if (!math_sync()) { report(status, ERR_MMA_WAIT | 0x100000); ok = false; break; }
        if (warp == 0) {
          const float m = s_mw[0][lane];
          const float l = (s_red1[0][lane] + s_red1[1][lane]) + (s_red1[2][lane] + s_red1[3][lane]) +
                          (float)(L - n * B32) * exp2f(-m);
          s_inv[lane] = 1.0f / l;
          fout[vec0 + lane] = m + log2f(l);
        }
        if (!math_sync()) { report(status, ERR_MMA_WAIT | 0x100000); ok = false; break; }
      } else {
        // ------------------------------------------------ backward: per-unit vectors into shared memory
        if (C::ROW) {
          // delta_i = sum_n dO_in O_in of the unit's 32 rows (four threads per row) and the lse of the same rows.
          // The operands were requested while the previous unit was computed (row_fetch at its start).
          if (!pre_unit) row_fetch(vec0, out_off, pos.ld);
          const uint32_t aw[8] = {pa0.x, pa0.y, pa0.z, pa0.w, pa1.x, pa1.y, pa1.z, pa1.w};
          const uint32_t bw[8] = {pb0.x, pb0.y, pb0.z, pb0.w, pb1.x, pb1.y, pb1.z, pb1.w};
          float acc = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) acc += bf16_lo(aw[i]) * bf16_lo(bw[i]) + bf16_hi(aw[i]) * bf16_hi(bw[i]);
          acc += __shfl_xor_sync(0xffffffffu, acc, 1);
          acc += __shfl_xor_sync(0xffffffffu, acc, 2);
          const int row = tid >> 2;
          if ((tid & 3) == 0) { fout[vec0 + row] = acc; s_red1[ub][row] = -acc * scale; }
          if (tid < 32) s_red0[ub][tid] = plse;
          pre_unit = c.nvalid && Cursor<MODE>::rec_n(c.nrec) > 0;
          if (pre_unit) {
            const int bhn = c.next_bh(), linen = c.nrec.y >> 16;
            const OpPos pn = op_pos(bhn, L, heads, HD);
            row_fetch((size_t)bhn * L + (size_t)linen * B32, (size_t)(pn.row0 + linen * B32) * pn.ld + pn.x0, pn.ld);
          }
        } else {
          if (tid < 32) s_red0[ub][tid] = kp ? kp[line * B32 + tid] * LOG2E : 0.f;     // penalty of the unit's 32 keys
        }
        if (!math_sync()) { report(status, ERR_MMA_WAIT | 0x100000); ok = false; break; }
        for (int jl = 0; jl < nch && ok; ++jl) {
          const int st = c.jg & 1, t0 = jl * GN, nt = min(GN, n - t0);
          // ROW: this thread is a key of gathered block `warp` (its padding penalty); COL: a query row (its lse and
          // delta, requested while the previous job was computed)
          float mine0 = 0.f, mine1 = 0.f;
          if (C::ROW) {
            if (kp && warp < nt) mine0 = kp[(t0 == 0 ? c.first_id(warp) : idx[rp + t0 + warp]) * B32 + lane] * LOG2E;
          } else if (pre_job) {
            mine0 = nx0; mine1 = nx1;
          } else if (warp < nt) {
            const int blk = t0 == 0 ? c.first_id(warp) : idx[rp + t0 + warp];
            mine0 = lse_in[(size_t)bh * L + blk * B32 + lane];
            mine1 = -delta_in[(size_t)bh * L + blk * B32 + lane] * scale;
          }
          const bool more = jl + 1 < nch;
          const int ntn = more ? min(GN, n - t0 - GN) : 0;
          if (C::COL && more && warp < ntn) pblk = idx[rp + t0 + GN + warp];          // used after this job's arithmetic
          SPION_STAMP_T(0, c.jg, 8);
          if (!mbar_wait(bar(BAR_SREADY, st), (uint32_t)(c.jg >> 1) & 1u)) { report(status, ERR_MMA_WAIT | 0x20000); ok = false; break; }
          SPION_STAMP_T(0, c.jg, 9);
          tc_fence_after();
          const int sv = c.jb & 1;
          if (!values_free(c.jb)) { ok = false; break; }
          if (warp < nt) {
            uint32_t v[32], g[32], wp[16], wd[16];
            tmem_ld32(t_lane + C::S_COL + st * 32, v);
            tmem_ld32(t_lane + C::DP_COL + st * 32, g);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              // ROW: column i is a query (lse, delta from shared memory); COL: column i is a key (penalty from shared memory)
              const float h0 = s_red0[ub][i] + mine0, h1 = s_red0[ub][i + 1] + mine0;
              const float p0 = ex2a(fmaf(__uint_as_float(v[i]), sc2, -h0)), p1 = ex2a(fmaf(__uint_as_float(v[i + 1]), sc2, -h1));
              const float n0 = C::ROW ? s_red1[ub][i] : mine1, n1 = C::ROW ? s_red1[ub][i + 1] : mine1;
              if (C::COL) wp[i >> 1] = pack_bf16(p0, p1);
              wd[i >> 1] = pack_bf16(p0 * fmaf(__uint_as_float(g[i]), scale, n0), p1 * fmaf(__uint_as_float(g[i + 1]), scale, n1));
            }
            if (C::COL) { store_row64(sVA(sv), grow, wp); store_row64(sVB(sv), grow, wd); }
            else store_row64(sVA(sv), grow, wd);
            fence_proxy_async();
          }
          if (C::COL) {
            // lse and delta of the row this thread owns in the NEXT job: a later chunk of this column, or the
            // first chunk of the next unit (its ids come with the prefetched record)
            pre_job = false;
            int blkn = -1, bhn = bh;
            if (more) {
              pre_job = true;
              if (warp < ntn) blkn = pblk;
            } else if (c.nvalid && Cursor<MODE>::rec_n(c.nrec) > 0) {
              pre_job = true;
              bhn = c.next_bh();
              if (warp < min(GN, Cursor<MODE>::rec_n(c.nrec))) blkn = Cursor<MODE>::rec_id(c.nrec, warp);
            }
            if (blkn >= 0) {
              nx0 = lse_in[(size_t)bhn * L + blkn * B32 + lane];
              nx1 = -delta_in[(size_t)bhn * L + blkn * B32 + lane] * scale;
            }
          }
          SPION_STAMP_T(0, c.jg, 10);
          job_done(st, sv);
          c.advance();
        }
        if (!ok) break;
      }

      // ------------------------------------------------ output rows of the unit (transposed accumulators)
      SPION_STAMP_T(0, c.jg - 1, 12);
      if (!mbar_wait(bar(BAR_OFULL, ob), pfull)) { report(status, ERR_MMA2_WAIT | 0x80000); ok = false; break; }
      SPION_STAMP_T(0, c.jg - 1, 13);
      tc_fence_after();
      {
        uint32_t v[32];
        tmem_ld32(t_lane + C::ACC_COL + (C::COL ? ob * 32 : 0), v);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BAR_OFREE, ob));
        // lanes 0-15 / 16-31 of every quadrant hold rows 16 warp + (lane & 15) of two accumulators:
        // FWD / ROW: the units of even / odd ordinal; COL: dK^T / dV^T of this unit
        const int jd = warp * 16 + (lane & 15);
        if (C::COL) {
          __nv_bfloat16* dst = (lane < 16 ? out0 : out1) + out_off + jd;
#pragma unroll
          for (int i = 0; i < 32; ++i) dst[(size_t)i * pos.ld] = __float2bfloat16(__uint_as_float(v[i]));
        } else if ((lane >> 4) == ob) {
          __nv_bfloat16* dst = out0 + out_off + jd;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            dst[(size_t)i * pos.ld] = __float2bfloat16(__uint_as_float(v[i]) * (C::FWD ? s_inv[i] : 1.0f));
        }
      }
      SPION_STAMP_T(0, c.jg - 1, 14);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, C::TMEM_COLS);
}

}  // namespace

namespace {

// Lines (block rows or block columns) of the mask as records {start in the index array, blocks | line << 16,
// id0 | id1 << 16, id2 | id3 << 16} (the ids of the line's first four blocks), from the longest to the shortest
// line (ties: ascending index).  One CTA.
__global__ void k_b32_recs(const int32_t* __restrict__ line_ptr, const int32_t* __restrict__ ids, int nb,
                           int4* __restrict__ rec, int* __restrict__ jobs_out) {
  __shared__ int s_n[SPION_MAX_NB];
  if (jobs_out && threadIdx.x == 0) *jobs_out = 0;
  for (int i = threadIdx.x; i < nb; i += blockDim.x) s_n[i] = line_ptr[i + 1] - line_ptr[i];
  __syncthreads();
  for (int i = threadIdx.x; i < nb; i += blockDim.x) {
    const int n = s_n[i], p = line_ptr[i];
    int rank = 0;
    for (int o = 0; o < nb; ++o) rank += (s_n[o] > n) || (s_n[o] == n && o < i);
    int c[4] = {0, 0, 0, 0};
    for (int t = 0; t < 4 && t < n; ++t) c[t] = ids[p + t];
    rec[rank] = make_int4(p, n | (i << 16), c[0] | (c[1] << 16), c[2] | (c[3] << 16));
  }
  if (jobs_out) {                                  // gathered jobs of all lines: sum of ceil(blocks / 4)
    __syncthreads();
    int mine = 0;
    for (int i = threadIdx.x; i < nb; i += blockDim.x) mine += (s_n[i] + GN - 1) / GN;
    atomicAdd(jobs_out, mine);
  }
}

// [32 x 64] boxes over one dense operand ([BH*L, 64] rows, or [B*L, H*64] rows in the merged-head form)
int make_map32(const spion_ctx* c, TcState* s, CUtensorMap* m, const void* base) {
  if (c->heads == 0) return make_map(s, m, base, (uint64_t)c->BH * c->L, HD, HD, B32);
  return make_map(s, m, base, (uint64_t)(c->BH / c->heads) * c->L, (uint32_t)(c->heads * HD), HD, B32);
}

template <int MODE>
int b32_attr(TcState* s, int device) {
  SPION_CUDA_TRY(cudaFuncSetAttribute(k_b32<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<MODE>::SMEM));
  return resident_ctas(k_b32<MODE>, device, B32_THREADS, Cfg<MODE>::SMEM, (int)Cfg<MODE>::TMEM_COLS, &s->b32_ctas[MODE]);
}

template <int MODE>
int b32_grid(const spion_ctx* c, const TcState* s) {
  const long long total = (long long)c->BH * c->nb, cap = (long long)s->sms * s->b32_ctas[MODE];
  return (int)(total < cap ? total : cap);
}

}  // namespace

namespace tc {

bool b32_applies(const spion_ctx* c) { return c->bs == B32 && c->d == HD; }

int b32_set_attrs(TcState* s, int device) {
  int rc;
  if ((rc = b32_attr<B32_FWD>(s, device)) || (rc = b32_attr<B32_ROW>(s, device)) || (rc = b32_attr<B32_COL>(s, device)))
    return rc;
  return SPION_OK;
}

// Once per mask: the sorted row and column records of the mask's own 32-wide structure, and whether these
// kernels or the super-block kernels serve the mask.  A job works on a 128-row operand gathered from up to
// four blocks; with fewer than about three blocks per job (masks that are little more than their diagonal
// band) the unused rows and the per-unit overhead cost more than the quarters the super-blocks waste
// (measured on the L x density grid of the kernel sweep: the paths break even at 2.8 - 3.0 blocks per job).
int b32_prepare(spion_ctx* c, TcState* s) {
  if (!s->b32_row_rec && cudaMalloc(&s->b32_row_rec, (size_t)SPION_MAX_NB * sizeof(int4)) != cudaSuccess) return SPION_ERR_ALLOC;
  if (!s->b32_col_rec && cudaMalloc(&s->b32_col_rec, (size_t)SPION_MAX_NB * sizeof(int4)) != cudaSuccess) return SPION_ERR_ALLOC;
  if (!s->b32_jobs_dev && cudaMalloc(&s->b32_jobs_dev, sizeof(int)) != cudaSuccess) return SPION_ERR_ALLOC;
  k_b32_recs<<<1, 512, 0, c->stream>>>(c->row_ptr, c->col_idx, c->nb, s->b32_row_rec, s->b32_jobs_dev);
  SPION_LAUNCH_CHECK();
  k_b32_recs<<<1, 512, 0, c->stream>>>(c->col_ptr, c->row_idx, c->nb, s->b32_col_rec, nullptr);
  SPION_LAUNCH_CHECK();
  c->launches += 2;
  int jobs = 0;
  SPION_CUDA_TRY(cudaMemcpyAsync(&jobs, s->b32_jobs_dev, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  SPION_CUDA_TRY(cudaStreamSynchronize(c->stream));                // pattern time: once per mask
  s->b32_fill = jobs > 0 ? (float)c->nnzb / (float)jobs : 0.0f;
  s->b32_use = c->block32_path == 1 || (c->block32_path == 0 && s->b32_fill >= 2.8f);
  return SPION_OK;
}

void b32_release(TcState* s) {
  cudaFree(s->b32_row_rec);
  cudaFree(s->b32_col_rec);
  cudaFree(s->b32_jobs_dev);
  s->b32_row_rec = s->b32_col_rec = nullptr;
  s->b32_jobs_dev = nullptr;
}

int b32_forward(spion_ctx* c, TcState* s, const void* Q, const void* K, const void* V, const float* keypad, void* O,
                float* lse) {
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = make_map32(c, s, &mq, Q)) || (rc = make_map32(c, s, &mk, K)) || (rc = make_map32(c, s, &mv, V))) return rc;
  prof_mark(c, -1);
  k_b32<B32_FWD><<<b32_grid<B32_FWD>(c, s), B32_THREADS, Cfg<B32_FWD>::SMEM, c->stream>>>(
      mk, mv, mq, mq, nullptr, nullptr, nullptr, nullptr, keypad, (__nv_bfloat16*)O, nullptr, lse, s->b32_row_rec,
      c->col_idx, c->L, c->BH, c->nb, c->heads, c->scale, keypad ? 0.0f : -100.0f, c->status_dev);
  SPION_LAUNCH_CHECK();
  c->launches += 1;
  prof_mark(c, SPION_STAGE_FUSED_FWD);
  return SPION_OK;
}

int b32_backward(spion_ctx* c, TcState* s, const void* Q, const void* K, const void* V, const void* O, const void* dO,
                 const float* lse, const float* keypad, void* dQ, void* dK, void* dV) {
  CUtensorMap mq, mk, mv, mdo;
  int rc;
  if ((rc = make_map32(c, s, &mq, Q)) || (rc = make_map32(c, s, &mk, K)) || (rc = make_map32(c, s, &mv, V)) ||
      (rc = make_map32(c, s, &mdo, dO)))
    return rc;
  prof_mark(c, -1);
  k_b32<B32_ROW><<<b32_grid<B32_ROW>(c, s), B32_THREADS, Cfg<B32_ROW>::SMEM, c->stream>>>(
      mk, mv, mq, mdo, (const __nv_bfloat16*)dO, (const __nv_bfloat16*)O, lse, nullptr, keypad, (__nv_bfloat16*)dQ, nullptr,
      s->delta_ws, s->b32_row_rec, c->col_idx, c->L, c->BH, c->nb, c->heads, c->scale, 0.0f, c->status_dev);
  SPION_LAUNCH_CHECK();
  prof_mark(c, SPION_STAGE_BWD_ROW_RC);
  k_b32<B32_COL><<<b32_grid<B32_COL>(c, s), B32_THREADS, Cfg<B32_COL>::SMEM, c->stream>>>(
      mq, mdo, mk, mv, nullptr, nullptr, lse, s->delta_ws, keypad, (__nv_bfloat16*)dK, (__nv_bfloat16*)dV, nullptr,
      s->b32_col_rec, c->row_idx, c->L, c->BH, c->nb, c->heads, c->scale, 0.0f, c->status_dev);
  SPION_LAUNCH_CHECK();
  prof_mark(c, SPION_STAGE_BWD_COL_RC);
  c->launches += 2;
  return SPION_OK;
}

}  // namespace tc
