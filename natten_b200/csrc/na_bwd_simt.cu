// Neighborhood attention BACKWARD on the original token layout with CUDA-core fp32 arithmetic
// (sm_100a): dQ, dK, dV (and the gradients of extra key/value tokens) for fp32 / fp16 / bf16
// operands and any head dim up to 256. Companion of na_simt.cu (same layout, same window walk).
//
// Semantics follow the reference's naive backward kernels
// (csrc/include/natten/cuda/reference/fna_reference_backward.hpp:62-160 dQ, 177-275 dK, 293-385 dV)
// and its delta pre-pass (csrc/src/compute_delta.cu): with s_ij = scale q_i.k_j,
// P_ij = exp(s_ij - LSE_i), dP_ij = dO_i.v_j, delta_i = dO_i.O_i,
//   dS_ij = scale P_ij (dP_ij - delta_i),  dQ_i = sum_j dS_ij k_j,
//   dK_j = sum_i dS_ij q_i,  dV_j = sum_i P_ij dO_i.
// Three kernels, no atomics, deterministic:
//   * delta: one warp per (batch, token, head) row.
//   * dQ: one warp per query; walks the query's window box 32 keys at a time.
//   * dK/dV: one warp per (batch, key token, kv head); the queries that attend a key form a box too
//     (window start and end are monotone in the query coordinate), found per axis by two binary
//     searches. Extra tokens are attended by every query: the same kernel with the whole layout as
//     the box.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include "common.cuh"
#include "fna_host.cuh"

namespace b200na {
namespace {

constexpr int kMaxD = 256;
constexpr int kWarps = 4;

template <class T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <class T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__half>(__half* p, float v) { *p = __float2half_rn(v); }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct BwdParams {
  NaAxes ax;
  int64_t N;  // tokens per batch
  int B, Hq, Hkv, D;
  int n_extra;
  float scale;
};

// delta[b, tok, h] = sum_d dO * O
template <class T>
__global__ void __launch_bounds__(kWarps * 32) delta_kernel(const T* __restrict__ o,
                                                            const T* __restrict__ d_out,
                                                            float* __restrict__ delta, int64_t rows,
                                                            int D) {
  const int lane = threadIdx.x & 31;
  const int64_t n_warps = (int64_t)gridDim.x * kWarps;
  for (int64_t r = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); r < rows; r += n_warps) {
    float acc = 0.f;
    for (int c = lane; c < D; c += 32) acc = fmaf(ldf(o + r * D + c), ldf(d_out + r * D + c), acc);
    acc = wsum(acc);
    if (lane == 0) delta[r] = acc;
  }
}

// Coordinates of a flat row-major token index.
__device__ __forceinline__ void token_coords(const NaAxes& ax, int64_t tok, int (&c)[B200NA_MAX_DIM]) {
#pragma unroll
  for (int a = B200NA_MAX_DIM - 1; a >= 0; --a) {
    if (a < ax.ndim) {
      c[a] = (int)(tok % ax.shape[a]);
      tok /= ax.shape[a];
    } else {
      c[a] = 0;
    }
  }
}

template <class T>
__global__ void __launch_bounds__(kWarps * 32) na_bwd_dq_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
    const T* __restrict__ d_out, const float* __restrict__ lse, const float* __restrict__ delta,
    const T* __restrict__ add_k, const T* __restrict__ add_v, T* __restrict__ dq,
    const BwdParams p) {
  __shared__ float q_sm[kWarps][kMaxD];
  __shared__ float do_sm[kWarps][kMaxD];
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int64_t total = (int64_t)p.B * p.N * p.Hq;
  const int64_t n_warps = (int64_t)gridDim.x * kWarps;
  const int rep = p.Hq / p.Hkv;
  const int D = p.D;
  const int nd = p.ax.ndim;

  for (int64_t w = (int64_t)blockIdx.x * kWarps + wib; w < total; w += n_warps) {
    const int h = (int)(w % p.Hq);
    const int64_t bt = w / p.Hq;
    const int64_t tok = bt % p.N;
    const int64_t b = bt / p.N;
    const int hk = h / rep;
    int qc[B200NA_MAX_DIM];
    token_coords(p.ax, tok, qc);
    int g[B200NA_MAX_DIM] = {0, 0, 0}, st[B200NA_MAX_DIM] = {0, 0, 0}, len[B200NA_MAX_DIM] = {1, 1, 1};
#pragma unroll
    for (int a = 0; a < B200NA_MAX_DIM; ++a) {
      if (a < nd) {
        const int d = p.ax.dilation[a];
        g[a] = qc[a] % d;
        const int i = qc[a] / d;
        const int L = group_extent(p.ax.shape[a], d, g[a]);
        st[a] = win_start(i, p.ax.kernel[a], p.ax.stride[a], L, p.ax.causal[a]);
        len[a] = win_end(i, st[a], p.ax.kernel[a], L, p.ax.causal[a]) - st[a];
      }
    }
    const int nk = len[0] * len[1] * len[2];
    const int n_all = nk + p.n_extra;

    __syncwarp();
    const int64_t row = (b * p.N + tok) * p.Hq + h;
    for (int c = lane; c < D; c += 32) {
      q_sm[wib][c] = ldf(q + row * D + c);
      do_sm[wib][c] = ldf(d_out + row * D + c);
    }
    __syncwarp();
    const float row_lse = lse[row], row_delta = delta[row];

    float acc[kMaxD / 32];
#pragma unroll
    for (int t = 0; t < kMaxD / 32; ++t) acc[t] = 0.f;

    for (int j0 = 0; j0 < n_all; j0 += 32) {
      const int j = j0 + lane;
      const T* krow = nullptr;
      const T* vrow = nullptr;
      if (j < nk) {
        int r = j;
        const int c2 = r % len[2]; r /= len[2];
        const int c1 = r % len[1]; r /= len[1];
        const int cc[B200NA_MAX_DIM] = {r, c1, c2};
        int64_t lin = 0;
#pragma unroll
        for (int a = 0; a < B200NA_MAX_DIM; ++a)
          if (a < nd) lin = lin * p.ax.shape[a] + ((int64_t)(st[a] + cc[a]) * p.ax.dilation[a] + g[a]);
        krow = k + ((b * p.N + lin) * p.Hkv + hk) * D;
        vrow = v + ((b * p.N + lin) * p.Hkv + hk) * D;
      } else if (j < n_all) {
        const int64_t e = j - nk;
        krow = add_k + ((b * p.n_extra + e) * p.Hkv + hk) * D;
        vrow = add_v + ((b * p.n_extra + e) * p.Hkv + hk) * D;
      }
      float ds = 0.f;
      if (krow) {
        float s = 0.f, dp = 0.f;
        for (int c = 0; c < D; ++c) {
          s = fmaf(q_sm[wib][c], ldf(krow + c), s);
          dp = fmaf(do_sm[wib][c], ldf(vrow + c), dp);
        }
        ds = p.scale * expf(s * p.scale - row_lse) * (dp - row_delta);
      }
      const int n_here = min(32, n_all - j0);
      for (int jj = 0; jj < n_here; ++jj) {
        const float dsb = __shfl_sync(0xffffffffu, ds, jj);
        const T* kr = reinterpret_cast<const T*>(
            __shfl_sync(0xffffffffu, (unsigned long long)krow, jj));
#pragma unroll
        for (int t = 0; t < kMaxD / 32; ++t) {
          const int c = lane + 32 * t;
          if (c < D) acc[t] = fmaf(dsb, ldf(kr + c), acc[t]);
        }
      }
    }
    T* out = dq + row * D;
#pragma unroll
    for (int t = 0; t < kMaxD / 32; ++t) {
      const int c = lane + 32 * t;
      if (c < D) stf(out + c, acc[t]);
    }
  }
}

// Queries of one axis (dilation-group coordinates, extent L) whose window holds key coordinate j:
// [lo, hi). Window start and end never decrease with the query coordinate, so both bounds are
// found by bisection.
__device__ __forceinline__ void attending_queries(int j, int k, int s, int L, int causal, int& lo,
                                                  int& hi) {
  int a = 0, b = L;
  while (a < b) {  // first query whose window end is beyond j
    const int mid = (a + b) >> 1;
    const int st = win_start(mid, k, s, L, causal);
    if (win_end(mid, st, k, L, causal) > j) b = mid; else a = mid + 1;
  }
  lo = a;
  b = L;
  while (a < b) {  // first query whose window start is beyond j
    const int mid = (a + b) >> 1;
    if (win_start(mid, k, s, L, causal) > j) b = mid; else a = mid + 1;
  }
  hi = a;
}

// extra == 0: one warp per (batch, key token, kv head) -> dk, dv rows of the token layout.
// extra == 1: one warp per (batch, extra token, kv head) -> d_add_k, d_add_v rows; every query
//             attends an extra token.
template <class T>
__global__ void __launch_bounds__(kWarps * 32) na_bwd_dkdv_kernel(
    const T* __restrict__ q, const T* __restrict__ k_src, const T* __restrict__ v_src,
    const T* __restrict__ d_out, const float* __restrict__ lse, const float* __restrict__ delta,
    T* __restrict__ dk, T* __restrict__ dv, const BwdParams p, const int extra) {
  __shared__ float k_sm[kWarps][kMaxD];
  __shared__ float v_sm[kWarps][kMaxD];
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int64_t n_keys = extra ? p.n_extra : p.N;
  const int64_t total = (int64_t)p.B * n_keys * p.Hkv;
  const int64_t n_warps = (int64_t)gridDim.x * kWarps;
  const int rep = p.Hq / p.Hkv;
  const int D = p.D;
  const int nd = p.ax.ndim;

  for (int64_t w = (int64_t)blockIdx.x * kWarps + wib; w < total; w += n_warps) {
    const int hk = (int)(w % p.Hkv);
    const int64_t bt = w / p.Hkv;
    const int64_t tok = bt % n_keys;
    const int64_t b = bt / n_keys;

    // box of attending queries: per axis first coordinate, count and step in layout coordinates
    int first[B200NA_MAX_DIM] = {0, 0, 0}, len[B200NA_MAX_DIM] = {1, 1, 1}, step[B200NA_MAX_DIM] = {1, 1, 1};
    if (extra) {
#pragma unroll
      for (int a = 0; a < B200NA_MAX_DIM; ++a)
        if (a < nd) len[a] = p.ax.shape[a];
    } else {
      int kc[B200NA_MAX_DIM];
      token_coords(p.ax, tok, kc);
#pragma unroll
      for (int a = 0; a < B200NA_MAX_DIM; ++a) {
        if (a < nd) {
          const int d = p.ax.dilation[a];
          const int g = kc[a] % d;
          const int L = group_extent(p.ax.shape[a], d, g);
          int lo, hi;
          attending_queries(kc[a] / d, p.ax.kernel[a], p.ax.stride[a], L, p.ax.causal[a], lo, hi);
          first[a] = lo * d + g;
          len[a] = hi - lo;
          step[a] = d;
        }
      }
    }
    const int64_t nq = (int64_t)len[0] * len[1] * len[2];
    const int64_t n_all = nq * rep;  // (query, head of the group) pairs

    __syncwarp();
    const int64_t krow = (b * n_keys + tok) * p.Hkv + hk;
    for (int c = lane; c < D; c += 32) {
      k_sm[wib][c] = ldf(k_src + krow * D + c);
      v_sm[wib][c] = ldf(v_src + krow * D + c);
    }
    __syncwarp();

    float acc_k[kMaxD / 32], acc_v[kMaxD / 32];
#pragma unroll
    for (int t = 0; t < kMaxD / 32; ++t) acc_k[t] = acc_v[t] = 0.f;

    for (int64_t j0 = 0; j0 < n_all; j0 += 32) {
      const int64_t j = j0 + lane;
      int64_t qrow = -1;
      float pj = 0.f, ds = 0.f;
      if (j < n_all) {
        const int hh = (int)(j % rep);
        int64_t r = j / rep;
        const int c2 = (int)(r % len[2]); r /= len[2];
        const int c1 = (int)(r % len[1]); r /= len[1];
        const int cc[B200NA_MAX_DIM] = {(int)r, c1, c2};
        int64_t lin = 0;
#pragma unroll
        for (int a = 0; a < B200NA_MAX_DIM; ++a)
          if (a < nd) lin = lin * p.ax.shape[a] + (first[a] + (int64_t)cc[a] * step[a]);
        qrow = (b * p.N + lin) * p.Hq + (hk * rep + hh);
        float s = 0.f, dp = 0.f;
        for (int c = 0; c < D; ++c) {
          s = fmaf(k_sm[wib][c], ldf(q + qrow * D + c), s);
          dp = fmaf(v_sm[wib][c], ldf(d_out + qrow * D + c), dp);
        }
        pj = expf(s * p.scale - lse[qrow]);
        ds = p.scale * pj * (dp - delta[qrow]);
      }
      const int n_here = (int)min((int64_t)32, n_all - j0);
      for (int jj = 0; jj < n_here; ++jj) {
        const float pb = __shfl_sync(0xffffffffu, pj, jj);
        const float dsb = __shfl_sync(0xffffffffu, ds, jj);
        const int64_t qr = __shfl_sync(0xffffffffu, qrow, jj);
#pragma unroll
        for (int t = 0; t < kMaxD / 32; ++t) {
          const int c = lane + 32 * t;
          if (c < D) {
            acc_k[t] = fmaf(dsb, ldf(q + qr * D + c), acc_k[t]);
            acc_v[t] = fmaf(pb, ldf(d_out + qr * D + c), acc_v[t]);
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < kMaxD / 32; ++t) {
      const int c = lane + 32 * t;
      if (c < D) {
        stf(dk + krow * D + c, acc_k[t]);
        stf(dv + krow * D + c, acc_v[t]);
      }
    }
  }
}

int grid_for(int64_t warps, int* blocks) {
  int sms = 0;
  int rc = sm_count_of_current_device(&sms);
  if (rc != B200NA_OK) return rc;
  int64_t n = (warps + kWarps - 1) / kWarps;
  const int64_t cap = (int64_t)sms * 32;
  *blocks = (int)(n < 1 ? 1 : (n > cap ? cap : n));
  return B200NA_OK;
}

template <class T>
int launch_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_out,
               const float* lse, const void* add_k, const void* add_v, void* dq, void* dk, void* dv,
               void* d_add_k, void* d_add_v, float* delta, const BwdParams& p,
               cudaStream_t stream) {
  const int64_t rows = (int64_t)p.B * p.N * p.Hq;
  int blocks = 0, rc;
  if ((rc = grid_for(rows, &blocks)) != B200NA_OK) return rc;
  delta_kernel<T><<<blocks, kWarps * 32, 0, stream>>>((const T*)o, (const T*)d_out, delta, rows, p.D);
  B200NA_CUDA_TRY(cudaGetLastError());
  na_bwd_dq_kernel<T><<<blocks, kWarps * 32, 0, stream>>>(
      (const T*)q, (const T*)k, (const T*)v, (const T*)d_out, lse, delta, (const T*)add_k,
      (const T*)add_v, (T*)dq, p);
  B200NA_CUDA_TRY(cudaGetLastError());
  if ((rc = grid_for((int64_t)p.B * p.N * p.Hkv, &blocks)) != B200NA_OK) return rc;
  na_bwd_dkdv_kernel<T><<<blocks, kWarps * 32, 0, stream>>>(
      (const T*)q, (const T*)k, (const T*)v, (const T*)d_out, lse, delta, (T*)dk, (T*)dv, p, 0);
  B200NA_CUDA_TRY(cudaGetLastError());
  if (p.n_extra > 0) {
    if ((rc = grid_for((int64_t)p.B * p.n_extra * p.Hkv, &blocks)) != B200NA_OK) return rc;
    na_bwd_dkdv_kernel<T><<<blocks, kWarps * 32, 0, stream>>>(
        (const T*)q, (const T*)add_k, (const T*)add_v, (const T*)d_out, lse, delta, (T*)d_add_k,
        (T*)d_add_v, p, 1);
    B200NA_CUDA_TRY(cudaGetLastError());
  }
  return B200NA_OK;
}

}  // namespace
}  // namespace b200na

namespace b200na {
int launch_delta(const void* o, const void* d_out, float* delta, int64_t rows, int D, int dtype,
                 cudaStream_t stream) {
  int blocks = 0;
  const int rc = grid_for(rows, &blocks);
  if (rc != B200NA_OK) return rc;
  if (dtype == B200NA_F32)
    delta_kernel<float><<<blocks, kWarps * 32, 0, stream>>>((const float*)o, (const float*)d_out,
                                                            delta, rows, D);
  else if (dtype == B200NA_F16)
    delta_kernel<__half><<<blocks, kWarps * 32, 0, stream>>>((const __half*)o, (const __half*)d_out,
                                                             delta, rows, D);
  else if (dtype == B200NA_BF16)
    delta_kernel<__nv_bfloat16><<<blocks, kWarps * 32, 0, stream>>>(
        (const __nv_bfloat16*)o, (const __nv_bfloat16*)d_out, delta, rows, D);
  else
    return B200NA_ERR_INVALID_ARGUMENT;
  B200NA_CUDA_TRY(cudaGetLastError());
  return B200NA_OK;
}
}  // namespace b200na

extern "C" B200NA_API int b200na_na_backward_simt(
    const void* q, const void* k, const void* v, const void* o, const void* d_out, const float* lse,
    const void* add_k, const void* add_v, int n_extra, void* dq, void* dk, void* dv, void* d_add_k,
    void* d_add_v, float* delta_scratch, int ndim, const int* shape, const int* kernel,
    const int* stride, const int* dilation, const int* causal, int B, int Hq, int Hkv, int D,
    int dtype, float scale, b200na_stream_t stream) {
  using namespace b200na;
  if (!q || !k || !v || !o || !d_out || !lse || !dq || !dk || !dv || !delta_scratch)
    return B200NA_ERR_INVALID_ARGUMENT;
  if (n_extra < 0 || (n_extra > 0 && (!add_k || !add_v || !d_add_k || !d_add_v)))
    return B200NA_ERR_INVALID_ARGUMENT;
  if (B < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv != 0 || D < 1 || !(scale > 0.f))
    return B200NA_ERR_INVALID_ARGUMENT;
  if (D > kMaxD) return B200NA_ERR_UNSUPPORTED;
  BwdParams p;
  memset(&p, 0, sizeof(p));
  int rc = fill_axes(p.ax, ndim, shape, kernel, stride, dilation, causal);
  if (rc != B200NA_OK) return rc;
  p.N = 1;
  for (int a = 0; a < ndim; ++a) p.N *= p.ax.shape[a];
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.D = D;
  p.n_extra = n_extra;
  p.scale = scale;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case B200NA_F32:
      return launch_bwd<float>(q, k, v, o, d_out, lse, add_k, add_v, dq, dk, dv, d_add_k, d_add_v,
                               delta_scratch, p, s);
    case B200NA_F16:
      return launch_bwd<__half>(q, k, v, o, d_out, lse, add_k, add_v, dq, dk, dv, d_add_k, d_add_v,
                                delta_scratch, p, s);
    case B200NA_BF16:
      return launch_bwd<__nv_bfloat16>(q, k, v, o, d_out, lse, add_k, add_v, dq, dk, dv, d_add_k,
                                       d_add_v, delta_scratch, p, s);
    default:
      return B200NA_ERR_INVALID_ARGUMENT;
  }
}
