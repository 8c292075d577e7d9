// Device-side pieces shared by the tensor-core attention kernels (forward: fna_sm100.cu,
// backward: fna_bwd_sm100.cu): bounded mbarrier waits, operand-type packing, and the element
// mask of a 128-column tile built from per-axis prefix bit tables.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "common.cuh"
#include "ptx.cuh"

namespace b200na {

#ifdef B200NA_TEST_HOOKS
// test-hook build: waits give up after about a millisecond, so that a test can make one expire
constexpr long long kWaitLimitCycles = 2000000ll;
#else
constexpr long long kWaitLimitCycles = 4000000000ll;  // ~2 s at 2 GHz
#endif

// Operand element types of the kernel templates.
enum : int { kTyF16 = 0, kTyBf16 = 1, kTyE4m3 = 2, kTyE5m2 = 3 };

// Bounded mbarrier wait. Returns false when the CTA is draining (this or another wait expired):
// the first expiry records `code` in the device status word and raises the CTA's abort flag.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                         int* status, int code) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!ptx::mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitLimitCycles) {
      *abort_flag = 1;
      atomicCAS(status, 0, code);
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Two fp32 values -> two 16-bit floats in one word, `lo` in the low half.
template <int kType>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if (kType == kTyBf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// 16 bytes of output elements from fp32 values scaled by `mul`: 8 (16-bit) or 16 (8-bit) values.
template <int kType>
__device__ __forceinline__ uint4 pack_out16(const uint32_t* f, float mul) {
  uint4 o;
  if (kType >= kTyE4m3) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = __uint_as_float(f[4 * i]) * mul, b = __uint_as_float(f[4 * i + 1]) * mul,
                  c = __uint_as_float(f[4 * i + 2]) * mul, d = __uint_as_float(f[4 * i + 3]) * mul;
      w[i] = kType == kTyE4m3 ? ptx::pack4_e4m3(a, b, c, d) : ptx::pack4_e5m2(a, b, c, d);
    }
    o = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
    o.x = pack2<kType>(__uint_as_float(f[0]) * mul, __uint_as_float(f[1]) * mul);
    o.y = pack2<kType>(__uint_as_float(f[2]) * mul, __uint_as_float(f[3]) * mul);
    o.z = pack2<kType>(__uint_as_float(f[4]) * mul, __uint_as_float(f[5]) * mul);
    o.w = pack2<kType>(__uint_as_float(f[6]) * mul, __uint_as_float(f[7]) * mul);
  }
  return o;
}

// Per-axis prefix bit tables over a 128-token tile of shape T (tokens ordered axis 0 fastest):
// pref[off_a + x], off_a = sum_{b<a} (T[b] + 1), has bit j set iff the in-tile coordinate of
// token j along axis a is < x. Filled cooperatively by `n_threads` threads; 136 entries suffice.
__device__ __forceinline__ void build_prefix_tables(uint4* pref, int ndim,
                                                    const int (&T)[B200NA_MAX_DIM], int tid,
                                                    int n_threads) {
  int off = 0;
  for (int a = 0; a < ndim; ++a) {
    int below = 1;
    for (int b = 0; b < a; ++b) below *= T[b];
    for (int x = tid; x <= T[a]; x += n_threads) {
      uint32_t wds[4];
#pragma unroll
      for (int wd = 0; wd < 4; ++wd) {
        uint32_t bits = 0;
#pragma unroll 1
        for (int j = 0; j < 32; ++j) {
          const int t = ((wd * 32 + j) / below) % T[a];
          if (t < x) bits |= 1u << j;
        }
        wds[wd] = bits;
      }
      pref[off + x] = make_uint4(wds[0], wds[1], wds[2], wds[3]);
    }
    off += T[a] + 1;
  }
}

// Mask of the 128 tokens of the tile whose first token has coordinates `base`: bit j is set iff
// token j lies in [lo[a], hi[a]) on every axis. Six shared-memory loads and a few logic
// operations per axis, for any (also non power-of-two) tile shape.
template <int NDIM>
__device__ __forceinline__ uint4 tile_mask(const uint4* pref, const int (&T)[B200NA_MAX_DIM],
                                           const int (&lo)[B200NA_MAX_DIM],
                                           const int (&hi)[B200NA_MAX_DIM],
                                           const int (&base)[B200NA_MAX_DIM]) {
  uint4 mk = make_uint4(~0u, ~0u, ~0u, ~0u);
  int off = 0;
#pragma unroll
  for (int a = 0; a < B200NA_MAX_DIM; ++a) {
    if (a < NDIM) {
      const int l = imin(imax(lo[a] - base[a], 0), T[a]);
      const int h = imin(imax(hi[a] - base[a], 0), T[a]);
      const uint4 ph = pref[off + h];
      const uint4 pl = pref[off + l];
      const bool none = h <= l;
      mk.x &= none ? 0u : (ph.x & ~pl.x);
      mk.y &= none ? 0u : (ph.y & ~pl.y);
      mk.z &= none ? 0u : (ph.z & ~pl.z);
      mk.w &= none ? 0u : (ph.w & ~pl.w);
      off += T[a] + 1;
    }
  }
  return mk;
}

}  // namespace b200na
