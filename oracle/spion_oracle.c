/* Plain-C restatement of the SPION hot path (test infrastructure, CPU only).
 *
 * A second, independent restatement next to the numpy one (oracle/pattern.py, oracle/csr.py,
 * oracle/attention.py): the tests require both to agree bit for bit on every integer result and on
 * the pooled map / threshold, and within fp32 rounding on the attention step.  bench.py times the
 * attention step of this file as its CPU baseline.  Nothing in the product links against it.
 *
 *   pattern   main_conv_ff.py:255-279 (conv, pool, guard, quantile, seeds, binarise, diagonal),
 *             main_conv_ff.py:35-62   (flood_fill walker), main_conv.py:246-251 (top-k variant),
 *             main_ff.py:255          (no convolution)
 *   CSR       models/attention_blockcuda.py:31-43
 *   attention models/block_attn.cu:33-130 (sparse softmax forward / backward), :453-545 (pipeline)
 *
 * Float stages of the pattern use the fixed order of fp64 additions documented in oracle/pattern.py.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define CONV_DIAG 0
#define CONV_BOX 1

int oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------ pattern: float stages */
/* pooled[nb*nb] (fp32) from A[L*L] (fp32).  F = 1: average pool only. */
int oracle_pooled(const float* A, int L, int bs, int F, int kind, float* pooled) {
  if (L < 1 || bs < 1 || L % bs != 0 || F < 1 || F % 2 == 0) return -1;
  const int nb = L / bs, h = F / 2;
  double* c = (double*)malloc((size_t)L * L * sizeof(double));
  if (!c) return -2;
#pragma omp parallel for schedule(static)
  for (int i = 0; i < L; ++i) {
    for (int j = 0; j < L; ++j) {
      double acc = 0.0;
      if (F == 1) {
        acc = (double)A[(size_t)i * L + j];
      } else if (kind == CONV_DIAG) {
        for (int t = -h; t <= h; ++t) {                /* t ascending; out-of-range taps add +0.0 */
          const int ii = i + t, jj = j + t;
          acc = acc + ((ii >= 0 && ii < L && jj >= 0 && jj < L) ? (double)A[(size_t)ii * L + jj] : 0.0);
        }
      } else {
        for (int u = -h; u <= h; ++u)                  /* u outer, v inner, both ascending */
          for (int v = -h; v <= h; ++v) {
            const int ii = i + u, jj = j + v;
            acc = acc + ((ii >= 0 && ii < L && jj >= 0 && jj < L) ? (double)A[(size_t)ii * L + jj] : 0.0);
          }
        acc = acc / (double)(F * F);
      }
      c[(size_t)i * L + j] = acc;
    }
  }
  /* r[i, bj] = sum_jj c[i, bj*bs+jj] (jj ascending); p[bi, bj] = sum_ii r[bi*bs+ii, bj] (ii ascending) */
  double* r = (double*)malloc((size_t)L * nb * sizeof(double));
  if (!r) { free(c); return -2; }
#pragma omp parallel for schedule(static)
  for (int i = 0; i < L; ++i)
    for (int bj = 0; bj < nb; ++bj) {
      double acc = 0.0;
      for (int jj = 0; jj < bs; ++jj) acc = acc + c[(size_t)i * L + bj * bs + jj];
      r[(size_t)i * nb + bj] = acc;
    }
  for (int bi = 0; bi < nb; ++bi)
    for (int bj = 0; bj < nb; ++bj) {
      double acc = 0.0;
      for (int ii = 0; ii < bs; ++ii) acc = acc + r[(size_t)(bi * bs + ii) * nb + bj];
      pooled[bi * nb + bj] = (float)(acc / (double)(bs * bs));
    }
  free(r);
  free(c);
  return 0;
}

static int cmp_float(const void* a, const void* b) {
  const float x = *(const float*)a, y = *(const float*)b;
  return (x > y) - (x < y);
}

/* fp32 multiply-add the way oracle/pattern.py's _fma32 forms it: exact product in fp64, one fp64 add */
static float fma32(float a, float b, float c) { return (float)((double)a * (double)b + (double)c); }

/* torch.quantile(pooled, q), linear interpolation (main_conv_ff.py:268) */
int oracle_quantile(const float* pooled, int n, float q, float* out) {
  if (n < 1) return -1;
  float* s = (float*)malloc((size_t)n * sizeof(float));
  if (!s) return -2;
  memcpy(s, pooled, (size_t)n * sizeof(float));
  qsort(s, (size_t)n, sizeof(float), cmp_float);
  const float rank = q * (float)(n - 1);
  const int lo_i = (int)floorf(rank), hi_i = (int)ceilf(rank);
  const float w = rank - (float)lo_i;
  const float lo = s[lo_i], hi = s[hi_i];
  const float d = hi - lo;
  *out = (fabsf(w) < 0.5f) ? fma32(w, d, lo) : fma32(-d, 1.0f - w, hi);
  free(s);
  return 0;
}

/* ------------------------------------------------------------------ pattern: integer stages */
/* 2*nb walkers from the first row, then the first column, on the zero-guarded grid; mat is the mask
 * BEFORE the diagonal is forced. */
int oracle_greedy_paths(const float* pooled, int nb, float thresh, uint8_t* mat) {
  const int g1 = nb + 1;
  float* g = (float*)calloc((size_t)g1 * g1, sizeof(float));
  if (!g) return -2;
  for (int i = 0; i < nb; ++i) memcpy(g + (size_t)i * g1, pooled + (size_t)i * nb, (size_t)nb * sizeof(float));
  memset(mat, 0, (size_t)nb * nb);
  for (int s = 0; s < 2 * nb; ++s) {
    int x = s < nb ? 0 : s - nb, y = s < nb ? s : 0;
    while (!(x + 1 == g1 || y + 1 == g1)) {
      const float D = g[(size_t)(x + 1) * g1 + y], R = g[(size_t)x * g1 + y + 1], G = g[(size_t)(x + 1) * g1 + y + 1];
      float v;
      if (D > R) {
        if (D > G) { x += 1; v = D; } else { x += 1; y += 1; v = G; }
      } else {
        if (R > G) { y += 1; v = R; } else { x += 1; y += 1; v = G; }
      }
      if (v > thresh && v > 0.0f) mat[x * nb + y] = 1;   /* x, y < nb here: the guard cells hold 0 */
    }
  }
  free(g);
  return 0;
}

typedef struct { double neg; int idx; } topk_item;
static int cmp_topk(const void* a, const void* b) {
  const topk_item* x = (const topk_item*)a; const topk_item* y = (const topk_item*)b;
  if (x->neg != y->neg) return (x->neg > y->neg) - (x->neg < y->neg);
  return (x->idx > y->idx) - (x->idx < y->idx);
}

/* SPION-C: the k = int(nb^2 * density - nb) largest pooled cells, ties towards the lower flat index */
int oracle_topk_mask(const float* pooled, int nb, double density, uint8_t* mat) {
  const int n = nb * nb;
  const int k = (int)((double)nb * (double)nb * density - (double)nb);
  memset(mat, 0, (size_t)n);
  if (k <= 0) return 0;
  topk_item* it = (topk_item*)malloc((size_t)n * sizeof(topk_item));
  if (!it) return -2;
  for (int i = 0; i < n; ++i) { it[i].neg = -(double)pooled[i]; it[i].idx = i; }
  qsort(it, (size_t)n, sizeof(topk_item), cmp_topk);
  for (int i = 0; i < k && i < n; ++i) mat[it[i].idx] = 1;
  free(it);
  return 0;
}

void oracle_force_diagonal(uint8_t* mat, int nb) {
  for (int i = 0; i < nb; ++i) mat[i * nb + i] = 1;
}

/* Full SPION-CF step (select = 0: quantile + walkers with parameter q; 1: top-k with parameter density). */
int oracle_discover(const float* A, int L, int bs, int F, int kind, int select, double param, uint8_t* mat,
                    float* pooled_out, float* thresh_out) {
  const int nb = L / bs;
  float* pooled = pooled_out ? pooled_out : (float*)malloc((size_t)nb * nb * sizeof(float));
  if (!pooled) return -2;
  int rc = oracle_pooled(A, L, bs, F, kind, pooled);
  float thresh = 0.0f;
  if (!rc) {
    if (select == 0) {
      rc = oracle_quantile(pooled, nb * nb, (float)param, &thresh);
      if (!rc) rc = oracle_greedy_paths(pooled, nb, thresh, mat);
    } else {
      rc = oracle_topk_mask(pooled, nb, param, mat);
    }
  }
  if (!rc) oracle_force_diagonal(mat, nb);
  if (thresh_out) *thresh_out = thresh;
  if (!pooled_out) free(pooled);
  return rc;
}

/* ------------------------------------------------------------------ CSR */
/* Block CSR and CSC of mat[nb*nb]; arrays sized nb+1 / nb*nb by the caller.  Returns the block count. */
int oracle_block_csr(const uint8_t* mat, int nb, int32_t* row_ptr, int32_t* col_idx, int32_t* blk_row,
                     int32_t* col_ptr, int32_t* row_idx, int32_t* csc_pos) {
  int n = 0;
  for (int r = 0; r < nb; ++r) {
    row_ptr[r] = n;
    for (int c = 0; c < nb; ++c)
      if (mat[r * nb + c]) { col_idx[n] = c; blk_row[n] = r; ++n; }
  }
  row_ptr[nb] = n;
  int m = 0;
  for (int c = 0; c < nb; ++c) {
    col_ptr[c] = m;
    for (int r = 0; r < nb; ++r)
      if (mat[r * nb + c]) {
        int pos = row_ptr[r];
        while (col_idx[pos] != c) ++pos;
        row_idx[m] = r; csc_pos[m] = pos; ++m;
      }
  }
  col_ptr[nb] = m;
  return n;
}

/* The reference's per-call element CSR (models/attention_blockcuda.py:31-43):
 * sum_mat[L], offsets[L+1], columns[repeat*nnz]; returns nnz. */
long long oracle_element_csr(const uint8_t* mat, int nb, int bs, int repeat, int32_t* sum_mat, int32_t* offsets,
                             int32_t* columns) {
  const int L = nb * bs;
  long long nnz = 0;
  for (int i = 0; i < L; ++i) {
    const int r = i / bs;
    int cnt = 0;
    offsets[i] = (int32_t)nnz;
    for (int c = 0; c < nb; ++c)
      if (mat[r * nb + c]) {
        for (int jj = 0; jj < bs; ++jj) columns[nnz + cnt * bs + jj] = c * bs + jj;
        ++cnt;
      }
    sum_mat[i] = cnt * bs;
    nnz += (long long)cnt * bs;
  }
  offsets[L] = (int32_t)nnz;
  for (int k = 1; k < repeat; ++k) memcpy(columns + (size_t)k * nnz, columns, (size_t)nnz * sizeof(int32_t));
  return nnz;
}

/* ------------------------------------------------------------------ attention step */
/* One forward (+ backward when dO != NULL) of the layer-wise sparse attention, fp32, statement by
 * statement as the reference kernels compute it (models/block_attn.cu:33-130):
 *   v_j = (q_i . k_j) * scale - pen_j            over the selected keys j of row i only
 *   m   = max(floor, max_j v_j)
 *   Z   = sum_j exp(v_j - m) + (L - n_i) * exp(-m)        every non-selected key counts as score 0
 *   p_j = exp(v_j - m) / Z        (all zero when 1/Z == 0)
 *   O_i = sum_j p_j v_j^T ...     dP_j = dO_i . V_j ; t = dP.p ; dS = (t - p sum t) scale
 *   dQ_i = sum_j dS_j K_j ; dK_j += dS_j Q_i ; dV_j += p_j dO_i
 * Q, K, V, dO, O, dQ, dK, dV: [BH, L, d] row-major.  pen: [BH*L] penalty (1e6 on padded keys) or NULL.
 * P (out) and dS (scratch, may be NULL without dO): [BH, nnz] in the reference's element-CSR order.
 * Work is split over (b,h) x block rows, then (b,h) x block columns, so no two threads write one row. */
int oracle_attention_step(const float* Q, const float* K, const float* V, const float* dO, const float* pen,
                          float floor_v, const uint8_t* mat, int BH, int L, int d, int bs, float* O, float* P,
                          float* dS, float* dQ, float* dK, float* dV) {
  if (L % bs != 0 || BH < 1 || d < 1) return -1;
  const int nb = L / bs;
  int32_t* row_ptr = (int32_t*)malloc((size_t)(nb + 1) * sizeof(int32_t));
  int32_t* col_ptr = (int32_t*)malloc((size_t)(nb + 1) * sizeof(int32_t));
  int32_t* col_idx = (int32_t*)malloc((size_t)nb * nb * sizeof(int32_t));
  int32_t* blk_row = (int32_t*)malloc((size_t)nb * nb * sizeof(int32_t));
  int32_t* row_idx = (int32_t*)malloc((size_t)nb * nb * sizeof(int32_t));
  int32_t* csc_pos = (int32_t*)malloc((size_t)nb * nb * sizeof(int32_t));
  if (!row_ptr || !col_ptr || !col_idx || !blk_row || !row_idx || !csc_pos) return -2;
  const int nnzb = oracle_block_csr(mat, nb, row_ptr, col_idx, blk_row, col_ptr, row_idx, csc_pos);
  const long long nnz = (long long)nnzb * bs * bs;
  const float scale = 1.0f / sqrtf((float)d);
  const int backward = dO != NULL;
  if (backward && !dS) return -1;

#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int bh = 0; bh < BH; ++bh)
    for (int r = 0; r < nb; ++r) {
      const int rp = row_ptr[r], nblk = row_ptr[r + 1] - rp, n_i = nblk * bs;
      float* v = (float*)malloc((size_t)(n_i > 0 ? n_i : 1) * sizeof(float));
      const float* Kb = K + (size_t)bh * L * d;
      const float* Vb = V + (size_t)bh * L * d;
      for (int ii = 0; ii < bs; ++ii) {
        const int i = r * bs + ii;
        const float* q = Q + ((size_t)bh * L + i) * d;
        /* element-CSR offset of row i: all rows of earlier block rows, then ii rows of this one */
        const size_t off = (size_t)bh * nnz + (size_t)rp * bs * bs + (size_t)ii * n_i;
        float m = floor_v;
        for (int k = 0; k < nblk; ++k) {
          const int c = col_idx[rp + k];
          for (int jj = 0; jj < bs; ++jj) {
            const int j = c * bs + jj;
            const float* kr = Kb + (size_t)j * d;
            float s = 0.0f;
            for (int n = 0; n < d; ++n) s += q[n] * kr[n];
            s *= scale;
            if (pen) s -= pen[(size_t)bh * L + j];
            v[k * bs + jj] = s;
            if (s > m) m = s;
          }
        }
        float z = 0.0f;
        for (int t = 0; t < n_i; ++t) { v[t] = expf(v[t] - m); z += v[t]; }
        z += (float)(L - n_i) * expf(-m);
        const float inv = 1.0f / z;
        float* o = O + ((size_t)bh * L + i) * d;
        for (int n = 0; n < d; ++n) o[n] = 0.0f;
        for (int k = 0; k < nblk; ++k) {
          const int c = col_idx[rp + k];
          for (int jj = 0; jj < bs; ++jj) {
            const float p = (inv == 0.0f) ? 0.0f : v[k * bs + jj] * inv;
            v[k * bs + jj] = p;
            P[off + k * bs + jj] = p;
            const float* vr = Vb + (size_t)(c * bs + jj) * d;
            for (int n = 0; n < d; ++n) o[n] += p * vr[n];
          }
        }
        if (!backward) continue;
        const float* g = dO + ((size_t)bh * L + i) * d;
        float tsum = 0.0f;
        for (int k = 0; k < nblk; ++k) {
          const int c = col_idx[rp + k];
          for (int jj = 0; jj < bs; ++jj) {
            const float* vr = Vb + (size_t)(c * bs + jj) * d;
            float dp = 0.0f;
            for (int n = 0; n < d; ++n) dp += g[n] * vr[n];
            const float t = dp * v[k * bs + jj];
            dS[off + k * bs + jj] = t;
            tsum += t;
          }
        }
        float* dq = dQ + ((size_t)bh * L + i) * d;
        for (int n = 0; n < d; ++n) dq[n] = 0.0f;
        for (int k = 0; k < nblk; ++k) {
          const int c = col_idx[rp + k];
          for (int jj = 0; jj < bs; ++jj) {
            const float ds = (dS[off + k * bs + jj] - v[k * bs + jj] * tsum) * scale;
            dS[off + k * bs + jj] = ds;
            const float* kr = Kb + (size_t)(c * bs + jj) * d;
            for (int n = 0; n < d; ++n) dq[n] += ds * kr[n];
          }
        }
      }
      free(v);
    }

  if (backward) {
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int bh = 0; bh < BH; ++bh)
      for (int c = 0; c < nb; ++c) {
        for (int jj = 0; jj < bs; ++jj) {
          float* dk = dK + ((size_t)bh * L + c * bs + jj) * d;
          float* dv = dV + ((size_t)bh * L + c * bs + jj) * d;
          for (int n = 0; n < d; ++n) { dk[n] = 0.0f; dv[n] = 0.0f; }
        }
        for (int e = col_ptr[c]; e < col_ptr[c + 1]; ++e) {
          const int r = row_idx[e], rp = row_ptr[r], n_i = (row_ptr[r + 1] - rp) * bs;
          const int k = csc_pos[e] - rp;                          /* position of block c inside row r */
          for (int ii = 0; ii < bs; ++ii) {
            const int i = r * bs + ii;
            const size_t off = (size_t)bh * nnz + (size_t)rp * bs * bs + (size_t)ii * n_i + (size_t)k * bs;
            const float* q = Q + ((size_t)bh * L + i) * d;
            const float* g = dO + ((size_t)bh * L + i) * d;
            for (int jj = 0; jj < bs; ++jj) {
              const float ds = dS[off + jj], p = P[off + jj];
              float* dk = dK + ((size_t)bh * L + c * bs + jj) * d;
              float* dv = dV + ((size_t)bh * L + c * bs + jj) * d;
              for (int n = 0; n < d; ++n) { dk[n] += ds * q[n]; dv[n] += p * g[n]; }
            }
          }
        }
      }
  }
  free(row_ptr); free(col_ptr); free(col_idx); free(blk_row); free(row_idx); free(csc_pos);
  return 0;
}
