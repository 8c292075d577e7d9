// Neighborhood attention forward on the ORIGINAL token layout with CUDA-core fp32 arithmetic
// (sm_100a). This is the path for fp32 operands and for head dims the tensor-core kernel does not
// take; it also accepts fp16/bf16 operands (converted to fp32 on load).
//
// Semantics follow the reference's naive kernel and mask
// (csrc/include/natten/cuda/reference/fna_reference_forward.hpp:63-211, mask.hpp:47-89, 220-225,
// 306-343): scaled logits, running max, exp, O = sum(p v) / sum(p), LSE = log(sum) + max, extra KV
// tokens attended by every query. Instead of scanning all keys and masking, each query walks only
// the keys inside its window box.
//
// One warp owns one (batch, token, head) query. Keys are processed 32 at a time: lane l computes
// the full q.k dot product of key l, the warp reduces max and sum with shuffles, and for P.V every
// lane owns head-dim columns l, l+32, ... so value rows are read coalesced.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include "common.cuh"

namespace b200na {
namespace {

constexpr int kMaxD = 256;
constexpr int kWarpsPerBlock = 4;

template <class T> __device__ __forceinline__ float ld_f(const T* p);
template <> __device__ __forceinline__ float ld_f<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_f<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <class T> __device__ __forceinline__ void st_f(T* p, float v);
template <> __device__ __forceinline__ void st_f<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st_f<__half>(__half* p, float v) { *p = __float2half_rn(v); }
template <> __device__ __forceinline__ void st_f<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

struct SimtParams {
  NaAxes ax;
  int64_t N;   // key/value tokens per batch
  int64_t Nq;  // query tokens per batch (== N except for dense cross attention)
  int dense;   // dense attention: every query sees keys [0, N) (causal: [0, i + 1))
  int B, Hq, Hkv, D;
  int n_extra;
  float scale;
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <class T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) na_simt_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ o,
    float* __restrict__ lse, const T* __restrict__ add_k, const T* __restrict__ add_v,
    const SimtParams p) {
  __shared__ float q_sm[kWarpsPerBlock][kMaxD];
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int64_t total = (int64_t)p.B * p.Nq * p.Hq;
  const int64_t n_warps = (int64_t)gridDim.x * kWarpsPerBlock;
  const int rep = p.Hq / p.Hkv;
  const int D = p.D;
  const int nd = p.ax.ndim;

  for (int64_t w = (int64_t)blockIdx.x * kWarpsPerBlock + wib; w < total; w += n_warps) {
    const int h = (int)(w % p.Hq);
    const int64_t bt = w / p.Hq;
    const int64_t tok = bt % p.Nq;
    const int64_t b = bt / p.Nq;
    const int hk = h / rep;

    // window box of this query, in dilation-group coordinates
    int g[B200NA_MAX_DIM] = {0, 0, 0}, st[B200NA_MAX_DIM] = {0, 0, 0}, len[B200NA_MAX_DIM] = {1, 1, 1};
    if (p.dense) {
      len[0] = p.ax.causal[0] ? (int)min((int64_t)tok + 1, p.N) : (int)p.N;
    } else {
      int64_t r = tok;
#pragma unroll
      for (int a = B200NA_MAX_DIM - 1; a >= 0; --a) {
        if (a < nd) {
          const int c = (int)(r % p.ax.shape[a]);
          r /= p.ax.shape[a];
          const int d = p.ax.dilation[a];
          g[a] = c % d;
          const int i = c / d;
          const int L = group_extent(p.ax.shape[a], d, g[a]);
          st[a] = win_start(i, p.ax.kernel[a], p.ax.stride[a], L, p.ax.causal[a]);
          len[a] = win_end(i, st[a], p.ax.kernel[a], L, p.ax.causal[a]) - st[a];
        }
      }
    }
    const int nk = len[0] * len[1] * len[2];
    const int n_all = nk + p.n_extra;

    __syncwarp();
    const T* qr = q + ((b * p.Nq + tok) * p.Hq + h) * D;
    for (int c = lane; c < D; c += 32) q_sm[wib][c] = ld_f(qr + c);
    __syncwarp();

    float m = -INFINITY, sum = 0.f;
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
        const int c0 = r;
        const int cc[B200NA_MAX_DIM] = {c0, c1, c2};
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
      float s = -INFINITY;
      if (krow) {
        float d = 0.f;
        for (int c = 0; c < D; ++c) d = fmaf(q_sm[wib][c], ld_f(krow + c), d);
        s = d * p.scale;
      }
      const float m_new = fmaxf(m, warp_max(s));  // finite: every chunk holds at least one key
      const float corr = expf(m - m_new);         // exp(-inf) = 0 on the first chunk
      const float pj = krow ? expf(s - m_new) : 0.f;
      sum = sum * corr + warp_sum(pj);
#pragma unroll
      for (int t = 0; t < kMaxD / 32; ++t) acc[t] *= corr;
      m = m_new;
      const int n_here = min(32, n_all - j0);
      for (int jj = 0; jj < n_here; ++jj) {
        const float pb = __shfl_sync(0xffffffffu, pj, jj);
        const T* vr = reinterpret_cast<const T*>(
            __shfl_sync(0xffffffffu, (unsigned long long)vrow, jj));
#pragma unroll
        for (int t = 0; t < kMaxD / 32; ++t) {
          const int c = lane + 32 * t;
          if (c < D) acc[t] = fmaf(pb, ld_f(vr + c), acc[t]);
        }
      }
    }
    const float inv = 1.f / sum;
    T* orow = o + ((b * p.Nq + tok) * p.Hq + h) * D;
#pragma unroll
    for (int t = 0; t < kMaxD / 32; ++t) {
      const int c = lane + 32 * t;
      if (c < D) st_f(orow + c, acc[t] * inv);
    }
    if (lse && lane == 0) lse[(b * p.Nq + tok) * p.Hq + h] = logf(sum) + m;
  }
}

template <class T>
int launch_simt(const void* q, const void* k, const void* v, void* o, float* lse, const void* ak,
                const void* av, const SimtParams& p, cudaStream_t stream) {
  int sms = 0;
  int rc = sm_count_of_current_device(&sms);
  if (rc != B200NA_OK) return rc;
  const int64_t total = (int64_t)p.B * p.Nq * p.Hq;
  int64_t blocks = (total + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const int64_t cap = (int64_t)sms * 32;
  if (blocks > cap) blocks = cap;
  na_simt_kernel<T><<<(int)blocks, kWarpsPerBlock * 32, 0, stream>>>(
      (const T*)q, (const T*)k, (const T*)v, (T*)o, lse, (const T*)ak, (const T*)av, p);
  B200NA_CUDA_TRY(cudaGetLastError());
  return B200NA_OK;
}

}  // namespace

// Dense attention on CUDA cores (fp32 operands, or head dims the tensor-core kernel does not
// take); called by b200na_fmha_forward.
int simt_dense_forward(const void* q, const void* k, const void* v, void* o, float* lse, int B,
                       int Nq, int Nk, int Hq, int Hkv, int D, int dtype, float scale, int causal,
                       cudaStream_t stream) {
  if (D > kMaxD) return B200NA_ERR_UNSUPPORTED;
  SimtParams p;
  memset(&p, 0, sizeof(p));
  p.ax.ndim = 1;
  for (int a = 0; a < B200NA_MAX_DIM; ++a) {
    p.ax.shape[a] = 1; p.ax.kernel[a] = 1; p.ax.stride[a] = 1; p.ax.dilation[a] = 1;
  }
  p.ax.shape[0] = Nk;
  p.ax.causal[0] = causal ? 1 : 0;
  p.N = Nk; p.Nq = Nq; p.dense = 1;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.n_extra = 0; p.scale = scale;
  switch (dtype) {
    case B200NA_F32: return launch_simt<float>(q, k, v, o, lse, nullptr, nullptr, p, stream);
    case B200NA_F16: return launch_simt<__half>(q, k, v, o, lse, nullptr, nullptr, p, stream);
    case B200NA_BF16: return launch_simt<__nv_bfloat16>(q, k, v, o, lse, nullptr, nullptr, p, stream);
    default: return B200NA_ERR_INVALID_ARGUMENT;
  }
}

}  // namespace b200na

extern "C" B200NA_API int b200na_na_forward_simt(const void* q, const void* k, const void* v, void* o,
                                      float* lse, int ndim, const int* shape, const int* kernel,
                                      const int* stride, const int* dilation, const int* causal,
                                      int B, int Hq, int Hkv, int D, int dtype, float scale,
                                      const void* add_k, const void* add_v, int n_extra,
                                      b200na_stream_t stream) {
  using namespace b200na;
  if (!q || !k || !v || !o) return B200NA_ERR_INVALID_ARGUMENT;
  if (B < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv != 0 || D < 1) return B200NA_ERR_INVALID_ARGUMENT;
  if (D > kMaxD) return B200NA_ERR_UNSUPPORTED;
  if (n_extra < 0 || (n_extra > 0 && (!add_k || !add_v))) return B200NA_ERR_INVALID_ARGUMENT;
  SimtParams p;
  int rc = fill_axes(p.ax, ndim, shape, kernel, stride, dilation, causal);
  if (rc != B200NA_OK) return rc;
  p.N = 1;
  for (int a = 0; a < ndim; ++a) p.N *= shape[a];
  p.Nq = p.N;
  p.dense = 0;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.n_extra = n_extra; p.scale = scale;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case B200NA_F32: return launch_simt<float>(q, k, v, o, lse, add_k, add_v, p, s);
    case B200NA_F16: return launch_simt<__half>(q, k, v, o, lse, add_k, add_v, p, s);
    case B200NA_BF16: return launch_simt<__nv_bfloat16>(q, k, v, o, lse, add_k, add_v, p, s);
    default: return B200NA_ERR_INVALID_ARGUMENT;
  }
}
