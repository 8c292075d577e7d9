// Token permute / unpermute for sm_100a: a bandwidth-bound gather that re-tiles a 1/2/3-D token
// layout (with dilation folded into the batch) so that every multi-dimensional attention tile is
// a contiguous run of rows. Behavioural twin of the reference's
// csrc/include/natten/cuda/tokperm/token_permute_kernel.cuh:159-378 and of
// src/natten/token_permute/torch_impl.py:99-187 (permute) / :190-267 (unpermute).
//
// Both directions are written as gathers over DESTINATION tokens: a group of lanes owns one
// destination token row (H*D contiguous elements), computes its source row once, and moves the
// row with 16-byte vector loads/stores (narrower vectors when the row pitch is not a multiple of
// 16 bytes). Rows are contiguous on both sides, so every access is a full 32-byte sector.
#include "common.cuh"

namespace b200na {
namespace {

struct TokPermParams {
  int ndim;
  int X[B200NA_MAX_DIM];   // token layout
  int T[B200NA_MAX_DIM];   // tile
  int d[B200NA_MAX_DIM];   // dilation
  int R[B200NA_MAX_DIM];   // tiles per dilation group
  int ord[B200NA_MAX_DIM]; // ord[0] = fastest axis of the tiled modes
  int G;                   // prod(d)
  int tile_size;           // prod(T)
  int64_t S;               // permuted rows per (batch, group) = prod(R*T)
  int64_t N;               // tokens per batch = prod(X)
  int64_t B;               // batch
  int64_t row_vecs;        // vectors per token row
};

template <int VEC>
struct VecT;
template <> struct VecT<16> { using type = uint4; };
template <> struct VecT<8> { using type = uint2; };
template <> struct VecT<4> { using type = uint32_t; };
template <> struct VecT<2> { using type = uint16_t; };
template <> struct VecT<1> { using type = uint8_t; };

template <class V>
__device__ __forceinline__ V zero_vec() {
  V v;
  memset(&v, 0, sizeof(V));
  return v;
}

// Streaming load: every input byte is read exactly once.
template <class V>
__device__ __forceinline__ V load_stream(const V* p) { return *p; }
template <>
__device__ __forceinline__ uint4 load_stream<uint4>(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Row index of the permuted tensor [B*G, S] <-> token coordinate of the original layout.
// Returns the source row (in rows of the *other* tensor) for destination row `dst`,
// or -1 when the destination is padding (permute only).
template <bool kUnpermute>
__device__ __forceinline__ int64_t source_row(const TokPermParams& p, int64_t dst) {
  if (!kUnpermute) {
    // dst = bp * S + s in the permuted tensor; source in the original layout.
    const int64_t bp = dst / p.S;
    int64_t s = dst - bp * p.S;
    const int64_t b = bp / p.G;
    int gl = (int)(bp - b * p.G);
    int tl = (int)(s % p.tile_size);
    int64_t rl = s / p.tile_size;
    int c[B200NA_MAX_DIM] = {0, 0, 0};
#pragma unroll
    for (int j = 0; j < B200NA_MAX_DIM; ++j) {
      if (j < p.ndim) {
        const int a = p.ord[j];
        const int g = gl % p.d[a]; gl /= p.d[a];
        const int t = tl % p.T[a]; tl /= p.T[a];
        const int r = (int)(rl % p.R[a]); rl /= p.R[a];
        c[a] = (r * p.T[a] + t) * p.d[a] + g;
      }
    }
    int64_t n = 0;
    bool ok = true;
#pragma unroll
    for (int a = 0; a < B200NA_MAX_DIM; ++a) {
      if (a < p.ndim) {
        ok = ok && (c[a] < p.X[a]);
        n = n * p.X[a] + c[a];
      }
    }
    return ok ? b * p.N + n : -1;
  } else {
    // dst = b * N + n in the original layout; source in the permuted tensor (always valid).
    const int64_t b = dst / p.N;
    int64_t n = dst - b * p.N;
    int g[B200NA_MAX_DIM], r[B200NA_MAX_DIM], t[B200NA_MAX_DIM];
#pragma unroll
    for (int a = B200NA_MAX_DIM - 1; a >= 0; --a) {
      if (a < p.ndim) {
        const int c = (int)(n % p.X[a]); n /= p.X[a];
        g[a] = c % p.d[a];
        const int i = c / p.d[a];
        r[a] = i / p.T[a];
        t[a] = i - r[a] * p.T[a];
      }
    }
    int gl = 0, tl = 0;
    int64_t rl = 0;
#pragma unroll
    for (int j = B200NA_MAX_DIM - 1; j >= 0; --j) {
      if (j < p.ndim) {
        const int a = p.ord[j];
        gl = gl * p.d[a] + g[a];
        tl = tl * p.T[a] + t[a];
        rl = rl * p.R[a] + r[a];
      }
    }
    return (b * p.G + gl) * p.S + rl * p.tile_size + tl;
  }
}

// kLanes lanes cooperate on one destination row; a warp moves 32 / kLanes rows at a time.
template <bool kUnpermute, int VEC, int kLanes>
__global__ void __launch_bounds__(256) tokperm_kernel(const void* __restrict__ in,
                                                      void* __restrict__ out,
                                                      const TokPermParams p, int64_t dst_rows) {
  using V = typename VecT<VEC>::type;
  constexpr int kRowsPerWarp = 32 / kLanes;
  constexpr int kUnroll = 8;
  const int lane = threadIdx.x & 31;
  const int sub = lane % kLanes;
  const int slot = lane / kLanes;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const V* src_base = reinterpret_cast<const V*>(in);
  V* dst_base = reinterpret_cast<V*>(out);

  for (int64_t row0 = warp * kRowsPerWarp; row0 < dst_rows; row0 += n_warps * kRowsPerWarp) {
    const int64_t dst = row0 + slot;
    if (dst >= dst_rows) continue;
    const int64_t src = source_row<kUnpermute>(p, dst);
    V* d = dst_base + dst * p.row_vecs;
    if (src < 0) {
      for (int64_t v = sub; v < p.row_vecs; v += kLanes) d[v] = zero_vec<V>();
      continue;
    }
    const V* s = src_base + src * p.row_vecs;
    int64_t v = sub;
    // Batches of kUnroll independent loads per lane keep enough bytes in flight per SM.
    for (; v + (int64_t)(kUnroll - 1) * kLanes < p.row_vecs; v += (int64_t)kUnroll * kLanes) {
      V tmp[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) tmp[u] = load_stream(s + v + (int64_t)u * kLanes);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) d[v + (int64_t)u * kLanes] = tmp[u];
    }
    for (; v < p.row_vecs; v += kLanes) d[v] = load_stream(s + v);
  }
}

template <bool kUnpermute, int VEC>
int launch_lanes(const void* in, void* out, const TokPermParams& p, int64_t dst_rows,
                 cudaStream_t stream) {
  int sms = 0;
  int rc = sm_count_of_current_device(&sms);
  if (rc != B200NA_OK) return rc;
  // lanes per row: smallest power of two covering the row, capped at a full warp
  int lanes = 1;
  while (lanes < 32 && lanes < p.row_vecs) lanes <<= 1;
  const int rows_per_warp = 32 / lanes;
  const int64_t warps_needed = (dst_rows + rows_per_warp - 1) / rows_per_warp;
  const int64_t blocks_needed = (warps_needed + 7) / 8;
  const int64_t cap = (int64_t)sms * 16;  // 8 resident CTAs of 256 threads per SM, two waves
  const int grid = (int)(blocks_needed < cap ? (blocks_needed > 0 ? blocks_needed : 1) : cap);
#define B200NA_TP_LAUNCH(L)                                                                  \
  tokperm_kernel<kUnpermute, VEC, L><<<grid, 256, 0, stream>>>(in, out, p, dst_rows)
  switch (lanes) {
    case 1: B200NA_TP_LAUNCH(1); break;
    case 2: B200NA_TP_LAUNCH(2); break;
    case 4: B200NA_TP_LAUNCH(4); break;
    case 8: B200NA_TP_LAUNCH(8); break;
    case 16: B200NA_TP_LAUNCH(16); break;
    default: B200NA_TP_LAUNCH(32); break;
  }
#undef B200NA_TP_LAUNCH
  B200NA_CUDA_TRY(cudaGetLastError());
  return B200NA_OK;
}

template <bool kUnpermute>
int tokperm_generic(const void* in, void* out, int ndim, const int* shape, const int* tile,
                    const int* dilation, int B, int H, int D, int elem_bytes, int flip,
                    cudaStream_t stream) {
  if (!in || !out || !shape || !tile) return B200NA_ERR_INVALID_ARGUMENT;
  if (ndim < 1 || ndim > B200NA_MAX_DIM || B < 1 || H < 1 || D < 1)
    return B200NA_ERR_INVALID_ARGUMENT;
  if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8)
    return B200NA_ERR_INVALID_ARGUMENT;
  TokPermParams p;
  memset(&p, 0, sizeof(p));
  p.ndim = ndim;
  p.G = 1;
  p.tile_size = 1;
  p.S = 1;
  p.N = 1;
  p.B = B;
  for (int a = 0; a < B200NA_MAX_DIM; ++a) {
    const bool on = a < ndim;
    p.X[a] = on ? shape[a] : 1;
    p.T[a] = on ? tile[a] : 1;
    p.d[a] = on && dilation ? dilation[a] : 1;
    if (p.X[a] < 1 || p.T[a] < 1 || p.d[a] < 1) return B200NA_ERR_INVALID_ARGUMENT;
    const int tiles = (p.X[a] + p.T[a] - 1) / p.T[a];
    p.R[a] = (tiles + p.d[a] - 1) / p.d[a];
    p.G *= p.d[a];
    p.tile_size *= p.T[a];
    p.S *= (int64_t)p.R[a] * p.T[a];
    p.N *= p.X[a];
  }
  for (int j = 0; j < ndim; ++j) p.ord[j] = flip ? j : ndim - 1 - j;
  const int64_t row_bytes = (int64_t)H * D * elem_bytes;
  const int64_t dst_rows = kUnpermute ? (int64_t)B * p.N : (int64_t)B * p.G * p.S;
  if (dst_rows == 0) return B200NA_OK;
  const uintptr_t align = reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) |
                          (uintptr_t)row_bytes;
  int vec = 16;
  while (vec > 1 && (align % vec) != 0) vec >>= 1;
  if (vec < elem_bytes) return B200NA_ERR_ALIGNMENT;  // pointers must be element-aligned
  p.row_vecs = row_bytes / vec;
  switch (vec) {
    case 16: return launch_lanes<kUnpermute, 16>(in, out, p, dst_rows, stream);
    case 8: return launch_lanes<kUnpermute, 8>(in, out, p, dst_rows, stream);
    case 4: return launch_lanes<kUnpermute, 4>(in, out, p, dst_rows, stream);
    case 2: return launch_lanes<kUnpermute, 2>(in, out, p, dst_rows, stream);
    default: return launch_lanes<kUnpermute, 1>(in, out, p, dst_rows, stream);
  }
}

}  // namespace
}  // namespace b200na

extern "C" B200NA_API int b200na_token_permute(const void* in, void* out, int ndim, const int* shape,
                                    const int* tile, const int* dilation, int B, int H, int D,
                                    int elem_bytes, int flip, b200na_stream_t stream) {
  return b200na::tokperm_generic<false>(in, out, ndim, shape, tile, dilation, B, H, D, elem_bytes,
                                        flip, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" B200NA_API int b200na_token_unpermute(const void* in, void* out, int ndim, const int* shape,
                                      const int* tile, const int* dilation, int B, int H, int D,
                                      int elem_bytes, int flip, b200na_stream_t stream) {
  return b200na::tokperm_generic<true>(in, out, ndim, shape, tile, dilation, B, H, D, elem_bytes,
                                       flip, reinterpret_cast<cudaStream_t>(stream));
}
