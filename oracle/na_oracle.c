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
