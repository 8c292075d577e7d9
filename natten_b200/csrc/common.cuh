// Shared host/device definitions for the natten_b200 kernels: error codes, neighborhood
// window arithmetic and small index helpers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/natten_b200.h"

#define B200NA_MAX_DIM 3

#define B200NA_HD __host__ __device__ __forceinline__

namespace b200na {

// Records the last CUDA error text for b200na_strerror(B200NA_ERR_CUDA).
void set_last_cuda_error(cudaError_t e, const char* where);

#define B200NA_CUDA_TRY(expr)                                   \
  do {                                                          \
    cudaError_t _e = (expr);                                    \
    if (_e != cudaSuccess) {                                    \
      ::b200na::set_last_cuda_error(_e, #expr);                 \
      return B200NA_ERR_CUDA;                                   \
    }                                                           \
  } while (0)

// ---- neighborhood window arithmetic --------------------------------------------------------
// Same integer semantics as the reference's csrc/include/natten/cuda/reference/mask.hpp:47-89
// (window left/right, start, end) and :220-225 (extent of one dilation group).

B200NA_HD int imin(int a, int b) { return a < b ? a : b; }
B200NA_HD int imax(int a, int b) { return a > b ? a : b; }

// Number of coordinates x in [0, X) with x % d == g.
B200NA_HD int group_extent(int X, int d, int g) {
  return X / d + (1 - ((g + (d - (X % d))) / d));
}

// First key index (inclusive) attended by query index i of a group with extent L.
B200NA_HD int win_start(int i, int k, int s, int L, int causal) {
  const int wl = k / 2;
  const int wr = k / 2 + (k % 2 - 1);
  if (causal) {
    const int lead = imin((i / s) * s + s - 1, L - 1);
    return imax(lead - wl - wr, 0);
  }
  const int lead = imin((i / s) * s + s / 2, L - 1);
  return imax(lead - wl, 0) + ((lead + wr >= L) ? (L - wr - lead - 1) : 0);
}

// One past the last key index attended by query index i.
B200NA_HD int win_end(int i, int start, int k, int L, int causal) {
  return causal ? imin(i + 1, L) : start + k;
}

// Per-axis problem description shared by the attention kernels.
struct NaAxes {
  int ndim;
  int shape[B200NA_MAX_DIM];     // original token layout X_a
  int kernel[B200NA_MAX_DIM];
  int stride[B200NA_MAX_DIM];
  int dilation[B200NA_MAX_DIM];
  int causal[B200NA_MAX_DIM];
};

// Validates kernel/stride/dilation against the token layout with the reference's rules
// (src/natten/utils/checks.py:400-407 k >= 2; :486-508 k*d <= X, s <= k).
inline int validate_axes(const NaAxes& ax) {
  if (ax.ndim < 1 || ax.ndim > B200NA_MAX_DIM) return B200NA_ERR_INVALID_ARGUMENT;
  for (int a = 0; a < ax.ndim; ++a) {
    if (ax.shape[a] < 1 || ax.kernel[a] < 2 || ax.stride[a] < 1 || ax.dilation[a] < 1)
      return B200NA_ERR_INVALID_ARGUMENT;
    if ((int64_t)ax.kernel[a] * ax.dilation[a] > ax.shape[a]) return B200NA_ERR_INVALID_ARGUMENT;
    if (ax.stride[a] > ax.kernel[a]) return B200NA_ERR_INVALID_ARGUMENT;
  }
  return B200NA_OK;
}

inline int fill_axes(NaAxes& ax, int ndim, const int* shape, const int* kernel, const int* stride,
                     const int* dilation, const int* causal) {
  if (ndim < 1 || ndim > B200NA_MAX_DIM || !shape || !kernel) return B200NA_ERR_INVALID_ARGUMENT;
  ax.ndim = ndim;
  for (int a = 0; a < B200NA_MAX_DIM; ++a) {
    const bool on = a < ndim;
    ax.shape[a] = on ? shape[a] : 1;
    ax.kernel[a] = on ? kernel[a] : 1;
    ax.stride[a] = on && stride ? stride[a] : 1;
    ax.dilation[a] = on && dilation ? dilation[a] : 1;
    ax.causal[a] = on && causal ? (causal[a] != 0) : 0;
  }
  return validate_axes(ax);
}

// CUDA-core dense attention (na_simt.cu), used by b200na_fmha_forward for fp32 operands and
// head dims outside the tensor-core kernel's set.
int simt_dense_forward(const void* q, const void* k, const void* v, void* o, float* lse, int B,
                       int Nq, int Nk, int Hq, int Hkv, int D, int dtype, float scale, int causal,
                       cudaStream_t stream);

inline int sm_count_of_current_device(int* sms) {
  int dev = 0;
  B200NA_CUDA_TRY(cudaGetDevice(&dev));
  B200NA_CUDA_TRY(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev));
  return B200NA_OK;
}

}  // namespace b200na
