// Whole-operator entry points: token permute -> fused neighborhood attention -> token unpermute
// behind ONE C call, for hosts that bind the C ABI directly (the reference runs the same three
// stages from Python: src/natten/backends/blackwell_fna.py:91-181). The permuted copies of Q, K,
// V, O and LSE live in a workspace the caller provides.
#include <mutex>

#include "common.cuh"

namespace b200na {
namespace {

constexpr int64_t kAlign = 256;
inline int64_t align_up(int64_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

struct FusedPlan {
  bool identity;            // 1-D, undilated, tile multiples: no permutation at all
  int G;                    // prod(dilation)
  int q_shape[B200NA_MAX_DIM], kv_shape[B200NA_MAX_DIM];  // padded per-group extents
  int64_t sq, skv;          // permuted rows per (batch, group)
  int64_t off_q, off_k, off_v, off_o, off_lse, total;
};

int make_plan(FusedPlan& pl, int ndim, const int* shape, const int* dilation, const int* q_tile,
              const int* kv_tile, int B, int Hq, int Hkv, int D, int elem_bytes, bool want_lse) {
  if (ndim < 1 || ndim > B200NA_MAX_DIM || !shape || !q_tile || !kv_tile || B < 1 || Hq < 1 ||
      Hkv < 1 || D < 1)
    return B200NA_ERR_INVALID_ARGUMENT;
  pl.G = 1;
  pl.sq = pl.skv = 1;
  bool ident = ndim == 1;
  for (int a = 0; a < ndim; ++a) {
    const int d = dilation ? dilation[a] : 1;
    if (shape[a] < 1 || d < 1 || q_tile[a] < 1 || kv_tile[a] < 1) return B200NA_ERR_INVALID_ARGUMENT;
    const int rq = ((shape[a] + q_tile[a] - 1) / q_tile[a] + d - 1) / d;
    const int rk = ((shape[a] + kv_tile[a] - 1) / kv_tile[a] + d - 1) / d;
    pl.q_shape[a] = rq * q_tile[a];
    pl.kv_shape[a] = rk * kv_tile[a];
    if ((int64_t)pl.G * d > (1 << 20) || pl.sq > ((int64_t)1 << 40) / pl.q_shape[a] ||
        pl.skv > ((int64_t)1 << 40) / pl.kv_shape[a])
      return B200NA_ERR_UNSUPPORTED;
    pl.G *= d;
    pl.sq *= pl.q_shape[a];
    pl.skv *= pl.kv_shape[a];
    ident = ident && d == 1 && pl.q_shape[a] == shape[a] && pl.kv_shape[a] == shape[a];
  }
  pl.identity = ident;
  // sizes far beyond any device's memory are refused before the byte sums below could wrap
  const int64_t kMaxElems = (int64_t)1 << 46;
  if ((int64_t)B * pl.G > kMaxElems / pl.sq || (int64_t)B * pl.G > kMaxElems / pl.skv ||
      (int64_t)B * pl.G * pl.sq > kMaxElems / ((int64_t)Hq * D) ||
      (int64_t)B * pl.G * pl.skv > kMaxElems / ((int64_t)Hkv * D))
    return B200NA_ERR_UNSUPPORTED;
  const int64_t bp = (int64_t)B * pl.G;
  int64_t off = 0;
  pl.off_q = off; off += ident ? 0 : align_up(bp * pl.sq * Hq * D * elem_bytes);
  pl.off_k = off; off += ident ? 0 : align_up(bp * pl.skv * Hkv * D * elem_bytes);
  pl.off_v = off; off += ident ? 0 : align_up(bp * pl.skv * Hkv * D * elem_bytes);
  pl.off_o = off; off += ident ? 0 : align_up(bp * pl.sq * Hq * D * elem_bytes);
  pl.off_lse = off; off += (ident || !want_lse) ? 0 : align_up(bp * pl.sq * Hq * 4);
  pl.total = off;
  return B200NA_OK;
}

}  // namespace

// Shared by b200na_na_forward and its static-workspace variant.
int na_forward_with_workspace(const void* q, const void* k, const void* v, void* o, float* lse,
                              int ndim, const int* shape, const int* kernel, const int* stride,
                              const int* dilation, const int* causal, const int* q_tile,
                              const int* kv_tile, int B, int Hq, int Hkv, int D, int dtype,
                              float scale, void* workspace, int64_t workspace_bytes,
                              b200na_stream_t stream) {
  if (!q || !k || !v || !o) return B200NA_ERR_INVALID_ARGUMENT;
  if (dtype != B200NA_F16 && dtype != B200NA_BF16) return B200NA_ERR_UNSUPPORTED;
  FusedPlan pl;
  int rc = make_plan(pl, ndim, shape, dilation, q_tile, kv_tile, B, Hq, Hkv, D, 2, lse != nullptr);
  if (rc != B200NA_OK) return rc;
  int ones[B200NA_MAX_DIM] = {1, 1, 1};
  const int* dil = dilation ? dilation : ones;
  if (pl.identity) {
    return b200na_fna_forward(q, k, v, o, lse, ndim, shape, pl.q_shape, pl.kv_shape, kernel, stride,
                              dil, causal, q_tile, kv_tile, B, Hq, Hkv, D, dtype, scale, stream);
  }
  if (!workspace || workspace_bytes < pl.total) return B200NA_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(workspace) % kAlign != 0) return B200NA_ERR_ALIGNMENT;
  char* ws = static_cast<char*>(workspace);
  void* qp = ws + pl.off_q; void* kp = ws + pl.off_k; void* vp = ws + pl.off_v;
  void* op = ws + pl.off_o;
  float* lp = lse ? reinterpret_cast<float*>(ws + pl.off_lse) : nullptr;
  if ((rc = b200na_token_permute(q, qp, ndim, shape, q_tile, dil, B, Hq, D, 2, 1, stream))) return rc;
  if ((rc = b200na_token_permute(k, kp, ndim, shape, kv_tile, dil, B, Hkv, D, 2, 1, stream))) return rc;
  if ((rc = b200na_token_permute(v, vp, ndim, shape, kv_tile, dil, B, Hkv, D, 2, 1, stream))) return rc;
  if ((rc = b200na_fna_forward(qp, kp, vp, op, lp, ndim, shape, pl.q_shape, pl.kv_shape, kernel,
                               stride, dil, causal, q_tile, kv_tile, B * pl.G, Hq, Hkv, D, dtype,
                               scale, stream)))
    return rc;
  if ((rc = b200na_token_unpermute(op, o, ndim, shape, q_tile, dil, B, Hq, D, 2, 1, stream))) return rc;
  if (lse) rc = b200na_token_unpermute(lp, lse, ndim, shape, q_tile, dil, B, Hq, 1, 4, 1, stream);
  return rc;
}

}  // namespace b200na

namespace b200na {
namespace {

// Scratch of b200na_na_forward_static. It is part of the loaded module: every device that loads
// this library holds these bytes from module load until the process exits.
static __device__ __align__(256) unsigned char g_static_workspace[B200NA_STATIC_WORKSPACE_BYTES];

// In host code `g_static_workspace` is only a handle for the runtime, not a device address; the
// address a kernel can use comes from cudaGetSymbolAddress, looked up once per device while that
// device is current.
int static_workspace_address(void** out) {
  static std::mutex mu;
  static void* cached[64] = {nullptr};
  int dev = 0;
  B200NA_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return B200NA_ERR_DEVICE;
  std::lock_guard<std::mutex> lk(mu);
  if (!cached[dev]) {
    void* ptr = nullptr;
    B200NA_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_workspace));
    if (!ptr) return B200NA_ERR_CUDA;
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return B200NA_OK;
}

}  // namespace
}  // namespace b200na

extern "C" B200NA_API int b200na_na_forward_static(const void* q, const void* k, const void* v,
                                                   void* o, float* lse, int ndim, const int* shape,
                                                   const int* kernel, const int* stride,
                                                   const int* dilation, const int* causal,
                                                   const int* q_tile, const int* kv_tile, int B,
                                                   int Hq, int Hkv, int D, int dtype, float scale,
                                                   b200na_stream_t stream) {
  using namespace b200na;
  FusedPlan pl;
  int rc = make_plan(pl, ndim, shape, dilation, q_tile, kv_tile, B, Hq, Hkv, D, 2, lse != nullptr);
  if (rc != B200NA_OK) return rc;
  if (pl.total > (int64_t)B200NA_STATIC_WORKSPACE_BYTES) return B200NA_ERR_WORKSPACE_LIMIT;
  void* ws = nullptr;
  if ((rc = static_workspace_address(&ws)) != B200NA_OK) return rc;
  // Nothing in the workspace has to start at zero: the permute kernels overwrite every row they
  // own (padding rows with zeros) and the unpermute kernels never read rows the attention kernel
  // skipped, so whatever an earlier call left behind is never observed.
  return na_forward_with_workspace(q, k, v, o, lse, ndim, shape, kernel, stride, dilation, causal,
                                   q_tile, kv_tile, B, Hq, Hkv, D, dtype, scale, ws,
                                   (int64_t)B200NA_STATIC_WORKSPACE_BYTES, stream);
}

extern "C" B200NA_API int64_t b200na_na_forward_workspace_bytes(int ndim, const int* shape,
                                                                const int* dilation,
                                                                const int* q_tile,
                                                                const int* kv_tile, int B, int Hq,
                                                                int Hkv, int D, int want_lse) {
  b200na::FusedPlan pl;
  const int rc = b200na::make_plan(pl, ndim, shape, dilation, q_tile, kv_tile, B, Hq, Hkv, D, 2,
                                   want_lse != 0);
  return rc == B200NA_OK ? pl.total : (int64_t)rc;
}

extern "C" B200NA_API int b200na_na_forward(const void* q, const void* k, const void* v, void* o,
                                            float* lse, int ndim, const int* shape,
                                            const int* kernel, const int* stride,
                                            const int* dilation, const int* causal,
                                            const int* q_tile, const int* kv_tile, int B, int Hq,
                                            int Hkv, int D, int dtype, float scale,
                                            void* workspace, int64_t workspace_bytes,
                                            b200na_stream_t stream) {
  return b200na::na_forward_with_workspace(q, k, v, o, lse, ndim, shape, kernel, stride, dilation,
                                           causal, q_tile, kv_tile, B, Hq, Hkv, D, dtype, scale,
                                           workspace, workspace_bytes, stream);
}
