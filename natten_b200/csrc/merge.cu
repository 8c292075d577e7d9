// Two-way LSE merge of attention outputs for sm_100a: one pass over HBM with 16-byte vectors,
// fp32 arithmetic. Behavioural twin of the reference's elementwise chain in
// src/natten/attn_merge.py:75-98:
//   o = o0 - sigmoid(l1 - l0) * (o0 - o1);   l = l0 - logsigmoid(l0 - l1)
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace b200na {
namespace {

template <class T> struct Cvt;
template <> struct Cvt<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct Cvt<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// One thread owns kElems consecutive elements (16 bytes) of one row.
template <class T, int kElems, bool kVec>
__global__ void __launch_bounds__(256) merge_kernel(const T* o0,   // o may alias o0 or o1:
                                                    const float* __restrict__ l0,
                                                    const T* o1,   // no __restrict__ on these
                                                    const float* __restrict__ l1, T* o, float* l,
                                                    int64_t rows, int D, int chunks) {
  const int64_t total = rows * chunks;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += step) {
    const int64_t row = idx / chunks;
    const int chunk = (int)(idx - row * chunks);
    const float a = l0[row], b = l1[row];
    // sigmoid(b - a), written so that neither branch overflows
    const float dlt = b - a;
    const float e = expf(-fabsf(dlt));
    const float sg = dlt >= 0.f ? 1.f / (1.f + e) : e / (1.f + e);
    const int64_t base = row * D + (int64_t)chunk * kElems;
    if (kVec) {
      struct alignas(16) Pack { T v[kElems]; };
      const Pack x0 = *reinterpret_cast<const Pack*>(o0 + base);
      const Pack x1 = *reinterpret_cast<const Pack*>(o1 + base);
      Pack y;
#pragma unroll
      for (int i = 0; i < kElems; ++i) {
        const float f0 = Cvt<T>::to_f(x0.v[i]), f1 = Cvt<T>::to_f(x1.v[i]);
        y.v[i] = Cvt<T>::from_f(f0 - sg * (f0 - f1));
      }
      *reinterpret_cast<Pack*>(o + base) = y;
    } else {
      const int n = (D - chunk * kElems) < kElems ? (D - chunk * kElems) : kElems;
      for (int i = 0; i < n; ++i) {
        const float f0 = Cvt<T>::to_f(o0[base + i]), f1 = Cvt<T>::to_f(o1[base + i]);
        o[base + i] = Cvt<T>::from_f(f0 - sg * (f0 - f1));
      }
    }
    if (chunk == 0) {
      // l0 - logsigmoid(l0 - l1) = max(l0, l1) + log1p(exp(-|l0 - l1|)); written from the larger
      // one so that an empty partial result (LSE = -inf, what a clipped slab call returns for a
      // query none of whose keys it holds) merges to the other input instead of NaN
      const float mx = fmaxf(a, b);
      l[row] = mx == -INFINITY ? -INFINITY : mx + log1pf(expf(-fabsf(a - b)));
    }
  }
}

template <class T>
int merge_typed(const void* o0, const float* l0, const void* o1, const float* l1, void* o,
                float* l, int64_t rows, int D, cudaStream_t stream) {
  constexpr int kElems = 16 / (int)sizeof(T);
  const uintptr_t al = reinterpret_cast<uintptr_t>(o0) | reinterpret_cast<uintptr_t>(o1) |
                       reinterpret_cast<uintptr_t>(o);
  const bool vec = (D % kElems == 0) && (al % 16 == 0);
  const int chunks = (D + kElems - 1) / kElems;
  int sms = 0;
  int rc = sm_count_of_current_device(&sms);
  if (rc != B200NA_OK) return rc;
  const int64_t total = rows * chunks;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)sms * 32;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (vec)
    merge_kernel<T, kElems, true><<<(int)blocks, 256, 0, stream>>>(
        (const T*)o0, l0, (const T*)o1, l1, (T*)o, l, rows, D, chunks);
  else
    merge_kernel<T, kElems, false><<<(int)blocks, 256, 0, stream>>>(
        (const T*)o0, l0, (const T*)o1, l1, (T*)o, l, rows, D, chunks);
  B200NA_CUDA_TRY(cudaGetLastError());
  return B200NA_OK;
}

}  // namespace
}  // namespace b200na

extern "C" B200NA_API int b200na_merge(const void* o0, const float* l0, const void* o1, const float* l1,
                            void* o, float* l, int64_t rows, int D, int dtype,
                            b200na_stream_t stream) {
  if (!o0 || !l0 || !o1 || !l1 || !o || !l || rows < 0 || D < 1)
    return B200NA_ERR_INVALID_ARGUMENT;
  // every thread of a row reads l0[row] and l1[row], one of them writes l[row]: the output LSE
  // must be a buffer of its own
  if (l == l0 || l == l1) return B200NA_ERR_INVALID_ARGUMENT;
  if (rows == 0) return B200NA_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case B200NA_F32: return b200na::merge_typed<float>(o0, l0, o1, l1, o, l, rows, D, s);
    case B200NA_F16: return b200na::merge_typed<__half>(o0, l0, o1, l1, o, l, rows, D, s);
    case B200NA_BF16: return b200na::merge_typed<__nv_bfloat16>(o0, l0, o1, l1, o, l, rows, D, s);
    default: return B200NA_ERR_INVALID_ARGUMENT;
  }
}
