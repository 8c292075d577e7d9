/*
 * CPU oracle for neighborhood attention forward (test infrastructure, NOT product code).
 *
 * Only the test suite, the smoke check and the benchmark's CPU-baseline leg may call this.
 * The GPU product path never links, imports or falls back to anything in this file.
 *
 * It restates, as plain windowed C loops, the algorithm the reference defines in
 *   csrc/include/natten/cuda/reference/mask.hpp:47-89    (window left/right, window start/end)
 *   csrc/include/natten/cuda/reference/mask.hpp:220-225  (per-dilation-group extent)
 *   csrc/include/natten/cuda/reference/mask.hpp:258-269  (coord -> (coord / d, coord % d))
 *   csrc/include/natten/cuda/reference/mask.hpp:306-343  (neighbour predicate, extra-KV rule)
 *   csrc/include/natten/cuda/reference/fna_reference_forward.hpp:63-211
 *        (scaled logits, running max, exp, sum, O = sum(p v) / sum(p), LSE = log(sum) + max)
 *   csrc/include/natten/cuda/reference/fna_reference_forward.hpp:246-288 (heads-last strides, GQA)
 *
 * Instead of scanning every key and masking, each query enumerates only the keys inside its
 * window box (O(N * prod(kernel)) work), which is the same set the reference's mask lets through.
 *
 * Parity pin: tests/golden/ holds outputs of the reference package itself (its CPU-capable
 * flex path, fp32) on seeded inputs; tests/test_oracle.py checks this file against them.
 *
 * Layout: Q [B, *shape, Hq, D], K [B, *shape, Hkv, D], V [B, *shape, Hkv, Dv] contiguous fp32;
 * extra K/V [B, n_extra, Hkv, D|Dv]; output [B, n_tok, Hq, Dv], LSE [B, n_tok, Hq], where
 * n_tok = number of tokens when tok_idx == NULL, else the length of the tok_idx sample
 * (flat row-major token indices), so that full-size problems can be checked on a row sample.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* Threads the following calls may use (the benchmark's CPU-baseline leg bounds them by the
 * cores this process may really run on); returns the value in effect. */
int na_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

#define NA_MAX_DIM 3

/* mask.hpp:47-57 */
static inline int win_left(int k) { return k / 2; }
static inline int win_right(int k) { return k / 2 + (k % 2 - 1); }

/* mask.hpp:59-80 */
static inline int win_start(int i, int k, int s, int L, int causal) {
  int wl = win_left(k), wr = win_right(k);
  if (causal) {
    int lead = (i / s) * s + s - 1;
    if (lead > L - 1) lead = L - 1;
    int st = lead - wl - wr;
    return st > 0 ? st : 0;
  }
  int lead = (i / s) * s + s / 2;
  if (lead > L - 1) lead = L - 1;
  int st = lead - wl;
  if (st < 0) st = 0;
  if (lead + wr >= L) st += L - wr - lead - 1;
  return st;
}

/* mask.hpp:82-89 */
static inline int win_end(int i, int start, int k, int L, int causal) {
  if (causal) return (i + 1 < L) ? i + 1 : L;
  return start + k;
}

/* mask.hpp:220-225: number of coordinates x in [0, X) with x % d == g */
static inline int group_extent(int X, int d, int g) {
  int padding = 1 - ((g + (d - (X % d))) / d);
  return X / d + padding;
}

typedef struct {
  int ndim;
  int shape[NA_MAX_DIM];
  int kernel[NA_MAX_DIM], stride[NA_MAX_DIM], dilation[NA_MAX_DIM], causal[NA_MAX_DIM];
} na_params;

/* Window box of one query: per axis [start, end) in dilation-group coordinates + its group. */
static void query_window(const na_params* p, const int* qc, int* g, int* st, int* en) {
  for (int a = 0; a < p->ndim; ++a) {
    int d = p->dilation[a];
    g[a] = qc[a] % d;
    int i = qc[a] / d;
    int L = group_extent(p->shape[a], d, g[a]);
    st[a] = win_start(i, p->kernel[a], p->stride[a], L, p->causal[a]);
    en[a] = win_end(i, st[a], p->kernel[a], L, p->causal[a]);
  }
}

#define ACC double
#define FN(name) name##_acc64
#include "na_oracle_body.inc"
#undef ACC
#undef FN

#define ACC float
#define FN(name) name##_acc32
#include "na_oracle_body.inc"
#undef ACC
#undef FN

/*
 * acc64 != 0: logits, softmax and the PV sum are accumulated in double (the parity checker);
 * acc64 == 0: fp32 accumulation as fna_reference_forward.hpp does (the timed CPU baseline).
 * Returns 0 on success, non-zero on an invalid argument.
 */
int na_oracle_forward(const float* q, const float* k, const float* v, float* out, float* lse,
                      int ndim, const int* shape, int B, int Hq, int Hkv, int D, int Dv,
                      const int* kernel, const int* stride, const int* dilation, const int* causal,
                      float scale, const float* add_k, const float* add_v, int n_extra,
                      const int64_t* tok_idx, int64_t n_tok, int acc64) {
  if (ndim < 1 || ndim > NA_MAX_DIM || Hkv <= 0 || Hq % Hkv != 0) return 1;
  na_params p;
  memset(&p, 0, sizeof(p));
  p.ndim = ndim;
  for (int a = 0; a < ndim; ++a) {
    p.shape[a] = shape[a];
    p.kernel[a] = kernel[a];
    p.stride[a] = stride ? stride[a] : 1;
    p.dilation[a] = dilation ? dilation[a] : 1;
    p.causal[a] = causal ? causal[a] : 0;
    /* utils/checks.py:486-508: k*d <= X, s <= k; utils/checks.py:400-407: k >= 2 */
    if (p.kernel[a] < 2 || p.stride[a] < 1 || p.dilation[a] < 1) return 2;
    if (p.kernel[a] * p.dilation[a] > p.shape[a] || p.stride[a] > p.kernel[a]) return 3;
  }
  if (n_extra > 0 && (!add_k || !add_v)) return 4;
  if (acc64)
    return na_forward_acc64(q, k, v, out, lse, &p, B, Hq, Hkv, D, Dv, scale, add_k, add_v,
                            n_extra, tok_idx, n_tok);
  return na_forward_acc32(q, k, v, out, lse, &p, B, Hq, Hkv, D, Dv, scale, add_k, add_v, n_extra,
                          tok_idx, n_tok);
}

/*
 * Dense attention (the reference's `attention()` used for the extra-KV tokens,
 * src/natten/functional.py:532-540): Q [B, Nq, Hq, D], K [B, Nk, Hkv, D], V [B, Nk, Hkv, Dv];
 * causal != 0 requires Nq == Nk and lets query i see keys 0..i.
 */
int na_oracle_dense(const float* q, const float* k, const float* v, float* out, float* lse, int B,
                    int Nq, int Nk, int Hq, int Hkv, int D, int Dv, float scale, int causal) {
  if (Hkv <= 0 || Hq % Hkv != 0 || (causal && Nq != Nk)) return 1;
  int rep = Hq / Hkv;
#pragma omp parallel
  {
    double* s = (double*)malloc(sizeof(double) * (size_t)Nk);
    double* acc = (double*)malloc(sizeof(double) * (size_t)Dv);
#pragma omp for collapse(2) schedule(dynamic, 16)
    for (int b = 0; b < B; ++b)
      for (int i = 0; i < Nq; ++i)
        for (int h = 0; h < Hq; ++h) {
          const float* qr = q + (((size_t)b * Nq + i) * Hq + h) * D;
          int hk = h / rep;
          int n = causal ? i + 1 : Nk;
          double m = -INFINITY;
          for (int j = 0; j < n; ++j) {
            const float* kr = k + (((size_t)b * Nk + j) * Hkv + hk) * D;
            double d = 0;
            for (int c = 0; c < D; ++c) d += (double)qr[c] * kr[c];
            s[j] = d * scale;
            if (s[j] > m) m = s[j];
          }
          double sum = 0;
          for (int c = 0; c < Dv; ++c) acc[c] = 0;
          for (int j = 0; j < n; ++j) {
            double pj = exp(s[j] - m);
            sum += pj;
            const float* vr = v + (((size_t)b * Nk + j) * Hkv + hk) * Dv;
            for (int c = 0; c < Dv; ++c) acc[c] += pj * vr[c];
          }
          float* o = out + (((size_t)b * Nq + i) * Hq + h) * Dv;
          for (int c = 0; c < Dv; ++c) o[c] = (float)(acc[c] / sum);
          if (lse) lse[((size_t)b * Nq + i) * Hq + h] = (float)(log(sum) + m);
        }
    free(s);
    free(acc);
  }
  return 0;
}

/*
 * Two-way LSE merge (src/natten/attn_merge.py:75-98), fp32 arithmetic:
 *   o = o0 - sigmoid(l1 - l0) * (o0 - o1);   l = l0 - logsigmoid(l0 - l1)
 * rows = B * N * H; o* are [rows, D] fp32, l* are [rows].
 */
int na_oracle_merge(const float* o0, const float* l0, const float* o1, const float* l1, float* o,
                    float* l, int64_t rows, int D) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    float d = l1[r] - l0[r];
    float sg = 1.0f / (1.0f + expf(-d));
    for (int c = 0; c < D; ++c) {
      float a = o0[r * D + c], b = o1[r * D + c];
      o[r * D + c] = a - sg * (a - b);
    }
    /* logsigmoid(x) = min(x, 0) - log1p(exp(-|x|)) */
    float x = l0[r] - l1[r];
    float ls = (x < 0 ? x : 0.0f) - log1pf(expf(-fabsf(x)));
    l[r] = l0[r] - ls;
  }
  return 0;
}

/*
 * Backward of neighborhood attention, double accumulation (checker only). Restates
 * csrc/include/natten/cuda/reference/fna_reference_backward.hpp:62-160 (dQ), :177-275 (dK),
 * :293-385 (dV): with s_ij = scale q_i.k_j, P_ij = exp(s_ij - LSE_i), dP_ij = dO_i.v_j,
 * delta_i = dO_i.O_i:
 *   dS_ij = scale P_ij (dP_ij - delta_i);  dQ_i = sum_j dS_ij k_j;  dK_j = sum_i dS_ij q_i;
 *   dV_j = sum_i P_ij dO_i,
 * j running over the query's window and the extra tokens (which get d_add_k / d_add_v). The
 * forward quantities are recomputed here in double from q, k, v, so the result does not depend on
 * anybody's rounded O or LSE (delta_i = sum_j P_ij dP_ij). GQA: the gradients of a key/value head
 * sum over the query heads that share it. All arrays fp32, layouts as in na_oracle_forward; the
 * gradient buffers are overwritten.
 */
int na_oracle_backward(const float* q, const float* k, const float* v, const float* d_out,
                       float* dq, float* dk, float* dv, int ndim, const int* shape, int B, int Hq,
                       int Hkv, int D, int Dv, const int* kernel, const int* stride,
                       const int* dilation, const int* causal, float scale, const float* add_k,
                       const float* add_v, float* d_add_k, float* d_add_v, int n_extra) {
  if (ndim < 1 || ndim > NA_MAX_DIM || Hkv <= 0 || Hq % Hkv != 0) return 1;
  na_params p;
  memset(&p, 0, sizeof(p));
  p.ndim = ndim;
  int64_t N = 1, win = 1;
  for (int a = 0; a < ndim; ++a) {
    p.shape[a] = shape[a];
    p.kernel[a] = kernel[a];
    p.stride[a] = stride ? stride[a] : 1;
    p.dilation[a] = dilation ? dilation[a] : 1;
    p.causal[a] = causal ? causal[a] : 0;
    if (p.kernel[a] < 2 || p.stride[a] < 1 || p.dilation[a] < 1) return 2;
    if (p.kernel[a] * p.dilation[a] > p.shape[a] || p.stride[a] > p.kernel[a]) return 3;
    N *= shape[a];
    win *= kernel[a];
  }
  if (n_extra > 0 && (!add_k || !add_v || !d_add_k || !d_add_v)) return 4;
  win += n_extra;
  const int rep = Hq / Hkv;
  const int nd = ndim;

  /* one (batch, key/value head) pair per task: it owns its slices of dK, dV and the extras */
#pragma omp parallel
  {
    double* s = (double*)malloc(sizeof(double) * (size_t)win);
    double* dp = (double*)malloc(sizeof(double) * (size_t)win);
    int64_t* kidx = (int64_t*)malloc(sizeof(int64_t) * (size_t)win);
    double* gk = (double*)malloc(sizeof(double) * (size_t)(N + n_extra) * D);
    double* gv = (double*)malloc(sizeof(double) * (size_t)(N + n_extra) * Dv);
    double* gq = (double*)malloc(sizeof(double) * (size_t)D);
#pragma omp for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < B; ++b)
      for (int hk = 0; hk < Hkv; ++hk) {
        memset(gk, 0, sizeof(double) * (size_t)(N + n_extra) * D);
        memset(gv, 0, sizeof(double) * (size_t)(N + n_extra) * Dv);
        for (int64_t tok = 0; tok < N; ++tok) {
          int qc[NA_MAX_DIM] = {0, 0, 0}, g[NA_MAX_DIM], st[NA_MAX_DIM], en[NA_MAX_DIM];
          int64_t r = tok;
          for (int a = nd - 1; a >= 0; --a) {
            qc[a] = (int)(r % p.shape[a]);
            r /= p.shape[a];
          }
          query_window(&p, qc, g, st, en);
          int64_t nk = 0;
          int c[NA_MAX_DIM];
          int lo[NA_MAX_DIM] = {0, 0, 0}, hi[NA_MAX_DIM] = {1, 1, 1};
          for (int a = 0; a < nd; ++a) {
            lo[a] = st[a];
            hi[a] = en[a];
          }
          for (c[0] = lo[0]; c[0] < hi[0]; ++c[0])
            for (c[1] = lo[1]; c[1] < hi[1]; ++c[1])
              for (c[2] = lo[2]; c[2] < hi[2]; ++c[2]) {
                int64_t lin = 0;
                for (int a = 0; a < nd; ++a)
                  lin = lin * p.shape[a] + ((int64_t)c[a] * p.dilation[a] + g[a]);
                kidx[nk++] = lin;
              }
          const int64_t nall = nk + n_extra;
          for (int h = hk * rep; h < (hk + 1) * rep; ++h) {
            const float* qr = q + (((size_t)b * N + tok) * Hq + h) * D;
            const float* gor = d_out + (((size_t)b * N + tok) * Hq + h) * Dv;
            double m = -INFINITY;
            for (int64_t j = 0; j < nall; ++j) {
              const float* kr = (j < nk) ? k + (((size_t)b * N + kidx[j]) * Hkv + hk) * D
                                         : add_k + (((size_t)b * n_extra + (j - nk)) * Hkv + hk) * D;
              const float* vr = (j < nk) ? v + (((size_t)b * N + kidx[j]) * Hkv + hk) * Dv
                                         : add_v + (((size_t)b * n_extra + (j - nk)) * Hkv + hk) * Dv;
              double d = 0, e = 0;
              for (int x = 0; x < D; ++x) d += (double)qr[x] * kr[x];
              for (int x = 0; x < Dv; ++x) e += (double)gor[x] * vr[x];
              s[j] = d * scale;
              dp[j] = e;
              if (s[j] > m) m = s[j];
            }
            double sum = 0, delta = 0;
            for (int64_t j = 0; j < nall; ++j) {
              s[j] = exp(s[j] - m);
              sum += s[j];
            }
            for (int64_t j = 0; j < nall; ++j) {
              s[j] /= sum; /* P_ij */
              delta += s[j] * dp[j];
            }
            for (int x = 0; x < D; ++x) gq[x] = 0;
            for (int64_t j = 0; j < nall; ++j) {
              const int64_t row = (j < nk) ? kidx[j] : N + (j - nk);
              const float* kr = (j < nk) ? k + (((size_t)b * N + kidx[j]) * Hkv + hk) * D
                                         : add_k + (((size_t)b * n_extra + (j - nk)) * Hkv + hk) * D;
              const double ds = (double)scale * s[j] * (dp[j] - delta);
              for (int x = 0; x < D; ++x) {
                gq[x] += ds * kr[x];
                gk[row * D + x] += ds * qr[x];
              }
              for (int x = 0; x < Dv; ++x) gv[row * Dv + x] += s[j] * gor[x];
            }
            float* dqr = dq + (((size_t)b * N + tok) * Hq + h) * D;
            for (int x = 0; x < D; ++x) dqr[x] = (float)gq[x];
          }
        }
        for (int64_t t = 0; t < N; ++t) {
          float* o1 = dk + (((size_t)b * N + t) * Hkv + hk) * D;
          float* o2 = dv + (((size_t)b * N + t) * Hkv + hk) * Dv;
          for (int x = 0; x < D; ++x) o1[x] = (float)gk[t * D + x];
          for (int x = 0; x < Dv; ++x) o2[x] = (float)gv[t * Dv + x];
        }
        for (int64_t t = 0; t < n_extra; ++t) {
          float* o1 = d_add_k + (((size_t)b * n_extra + t) * Hkv + hk) * D;
          float* o2 = d_add_v + (((size_t)b * n_extra + t) * Hkv + hk) * Dv;
          for (int x = 0; x < D; ++x) o1[x] = (float)gk[(N + t) * D + x];
          for (int x = 0; x < Dv; ++x) o2[x] = (float)gv[(N + t) * Dv + x];
        }
      }
    free(s);
    free(dp);
    free(kidx);
    free(gk);
    free(gv);
    free(gq);
  }
  return 0;
}
