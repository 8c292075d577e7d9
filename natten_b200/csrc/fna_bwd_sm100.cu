// Fused neighborhood attention BACKWARD for sm_100a (B200) on tensor cores: TMA-fed tiles,
// tcgen05 MMAs with TMEM accumulators, operands read straight from the caller's [B, *X, H, D]
// layout through rank-5 tensor maps (same boxes as the forward kernel in fna_sm100.cu).
//
// Functional contract = the reference's Blackwell FNA backward
// (natten::blackwell_na{1,2,3}d_backward, csrc/include/natten/blackwell_fna.h:92-152; arithmetic
// csrc/include/natten/cuda/reference/fna_reference_backward.hpp:62-385): with
// P = exp(scale q.k - LSE), dP = dO.v, delta = dO.O:  dS = P (dP - delta),
//   dQ = scale dS K,   dK = scale dS^T Q,   dV = P^T dO,
// P and dS rounded to the operand type before the second products. The design is this library's:
// ONE kernel template serves both passes, because they are mirror images of each other.
//   * A CTA owns a stationary 128-token ROW tile and streams 128-token COLUMN tiles past it:
//       pass dQ   : rows = queries (R1 = Q, R2 = dO), columns = keys    (C1 = K, C2 = V)
//       pass dKdV : rows = keys    (R1 = K, R2 = V),  columns = queries (C1 = Q, C2 = dO)
//     In both, S = R1 C1^T and dP = R2 C2^T; then dQ += dS C1, resp. dK += dS C1 and dV += P C2.
//     No atomics, no partial sums in memory: every gradient row is owned by exactly one CTA.
//   * The columns a row tile needs form a box of tiles in both passes: a query's keys are its
//     window, and a key's queries are the inverse window - an interval per axis, because window
//     start and end never decrease with the query coordinate (found by bisection).
//   * TMEM: S [0,128) dP [128,256) acc0 [256,256+D) acc1 [384,384+D). Pass dKdV: P and dS (16-bit)
//     overwrite S and dP in place, privately per thread, and feed the second MMAs from TMEM; the
//     four regions fill TMEM, so a column tile's products and its P / dS arithmetic alternate.
//   * Pass dQ has one accumulator, so it is software-pipelined: dS goes to two 64-column buffers
//     in [384,512), S / dP are handed back to the tensor pipe as soon as the softmax threads hold
//     them in registers, and the next tile's S and dP are computed while this tile's dS is. The
//     C1 (K) and C2 (V) column tiles have rings of their own there: a C2 stage is free after dP,
//     a C1 stage only after the dQ product.
//   * Row statistics (LSE, delta) are per thread in pass dQ; in pass dKdV they belong to the
//     columns and are staged through shared memory per column tile.
//   * Warp roles: 16 softmax warps (four threads per row, 32 columns each: the P / dS arithmetic
//     is latency-bound, more warps per sub-partition hide it), 1 MMA-issue warp (pass dQ: a
//     second one for the dQ products, in another sub-partition), 1 load warp that also decodes
//     work items and classifies tiles (descriptor / record rings as in the forward kernel). Every mbarrier wait is bounded; on expiry the CTA records a status word
//     (shared with the forward kernel) and drains.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "fna_device.cuh"
#include "fna_host.cuh"
#include "ptx.cuh"

namespace b200na {
namespace {

constexpr int kTile = 128;          // tokens per row tile and per column tile
constexpr int kParts = 4;           // threads per row: each owns 32 of a column tile's 128 columns
constexpr int kSoftmaxWarps = 16;   // 4 column parts x 4 warps (one thread per row and part)
constexpr int kSoftmaxThreads = 512;
constexpr int kMmaWarp = 16;
constexpr int kLoadWarp = 17;
constexpr int kMma2Warp = 18;       // pass dQ: issues the dQ products (kMmaWarp issues S and dP)
constexpr int kThreads = 608;
// Registers are allocated to warps in groups of four, so 19 warps cost as much as 20: 96 per
// thread; the 16-column chunks of the P / dS loop keep the live set well below that.
constexpr int kTmemCols = 512;
constexpr int kDescSlots = 3;
constexpr int kDescBytes = 128;
#ifndef B200NA_BWD_RING1
#define B200NA_BWD_RING1 3
#endif
constexpr int kTileRecs = 8;

// status word: (role << 8) | barrier id; roles 5 = softmax, 6 = mma, 7 = load, 9 = second mma
// issuer of pass dQ (backward kernel)
enum : int { kStRFull = 1, kStREmpty, kStCFull, kStCEmpty, kStSdpFull, kStDsFull, kStAccFull,
             kStAccEmpty, kStDescFull, kStDescEmpty, kStRecFull, kStRecEmpty, kStSmemAlign,
             kStSdpFree, kStDsFree, kStVFull, kStVEmpty, kStDpFull, kStPFull };

struct BwdTcParams {
  int ndim;
  int X[B200NA_MAX_DIM];
  int kernel[B200NA_MAX_DIM];
  int stride[B200NA_MAX_DIM];
  int dil[B200NA_MAX_DIM];
  int causal[B200NA_MAX_DIM];
  int Tr[B200NA_MAX_DIM];   // row tile shape
  int Tc[B200NA_MAX_DIM];   // column tile shape
  int Rr[B200NA_MAX_DIM];   // row tiles per axis per dilation group
  int G;                    // prod(dil)
  int B, Hq, Hkv, rep;
  int n_extra;              // pass dQ: extra key/value tokens appended to every query's columns
  int extra_tiles;          // ceil(n_extra / 128)
  int dense_rows;           // pass over the extra tokens: rows = the n_extra tokens of a batch
                            // entry (one axis), columns = all its queries, every valid row
                            // interacts with every column; X[0] is then the COLUMN extent
  int row_extent;           // dense_rows: number of rows (n_extra)
  int n_rtiles;             // row tiles per (batch, group, head)
  int row_heads;            // heads the row tiles carry: Hq (pass dQ) or Hkv (pass dKdV)
  long long total_work;     // n_rtiles * row_heads * B * G
  float scale;              // applied to dQ / dK in the epilogue
  float scale_log2;         // scale * log2(e)
  const float* lse;         // [B, *X, Hq]
  const float* delta;       // [B, *X, Hq]
  void* out0;               // dQ (pass dQ) or dK (pass dKdV)
  void* out1;               // dV (pass dKdV)
  int* status;
  unsigned long long* work;  // [0] next work item, [1] CTAs done (dynamic item scheduler)
  long long* trace;          // instrumented builds only: [5 roles][1024] event stamps of CTA 0
};

// Event trace of CTA 0 in pass dQ (-DB200NA_BWD_TRACE=1): (clock << 8) | code per event.
#if defined(B200NA_BWD_TRACE) && B200NA_BWD_TRACE
#define BTRACE_DECL(skip) int btrace_n_ = -(skip);
#define BTRACE(role, code)                                                              \
  {                                                                                     \
    if (p.trace != nullptr && blockIdx.x == 0 && btrace_n_ < 1024) {                 \
      if (btrace_n_ >= 0) p.trace[(role) * 1024 + btrace_n_] = (clock64() << 8) | (code); \
      ++btrace_n_;                                                                      \
    }                                                                                   \
  }
#else
#define BTRACE_DECL(skip)
#define BTRACE(role, code) {}
#endif

struct Item {
  int b, h;                   // batch entry; head of the row tile (query head or kv head)
  int g[B200NA_MAX_DIM];      // dilation group offset per axis
  int L[B200NA_MAX_DIM];      // extent of this dilation group
  int r_lo[B200NA_MAX_DIM];   // first row coordinate of the tile (group coordinates)
  int c_org[B200NA_MAX_DIM];  // first column coordinate of the first column tile per axis: the
                              // tiles start where the rows' columns start, not on a grid from 0
  int c_n[B200NA_MAX_DIM];    // column tiles per axis
  // column tiles [int_lo, int_hi) of an axis, counted from c_org, lie inside the (inverse)
  // window of every row
  int int_lo[B200NA_MAX_DIM];
  int int_hi[B200NA_MAX_DIM];
  int n_tiles;                // column tiles to visit (times the heads of the group in pass dKdV),
                              // extra-token tiles included
  int n_na;                   // neighborhood column tiles (without the extra-token tiles)
  int n_per_head;             // column tiles per head
  int skip;
};
static_assert(sizeof(Item) <= kDescBytes, "descriptor slot too small");

// Window of a query along one axis, group coordinates: [st, en).
__device__ __forceinline__ void fwd_window(const BwdTcParams& p, int a, int i, int L, int& st,
                                           int& en) {
  st = win_start(i, p.kernel[a], p.stride[a], L, p.causal[a]);
  en = win_end(i, st, p.kernel[a], L, p.causal[a]);
}
// Queries whose window holds key j (the inverse window): [lo, hi); empty for j outside [0, L).
__device__ __forceinline__ void inv_window(const BwdTcParams& p, int a, int j, int L, int& lo,
                                           int& hi) {
  if (j >= L) {
    lo = hi = L;
    return;
  }
  int x = 0, y = L;
  while (x < y) {  // first query whose window end is beyond j
    const int mid = (x + y) >> 1;
    int st, en;
    fwd_window(p, a, mid, L, st, en);
    if (en > j) y = mid; else x = mid + 1;
  }
  lo = x;
  y = L;
  while (x < y) {  // first query whose window start is beyond j
    const int mid = (x + y) >> 1;
    if (win_start(mid, p.kernel[a], p.stride[a], L, p.causal[a]) > j) y = mid; else x = mid + 1;
  }
  hi = x;
}
// Columns that interact with row coordinate i: the window (rows = queries) or the inverse window
// (rows = keys).
template <bool kKeyRows>
__device__ __forceinline__ void row_span(const BwdTcParams& p, int a, int i, int L, int& lo,
                                         int& hi) {
  if (kKeyRows && p.dense_rows) {  // an extra token: every query attends it
    lo = 0;
    hi = i < p.row_extent ? L : 0;
  } else if (kKeyRows) {
    inv_window(p, a, i, L, lo, hi);
  } else {
    fwd_window(p, a, i < L ? i : L - 1, L, lo, hi);
  }
}

struct WorkCursor {
  long long w;
  int rt, h, bp;
  __device__ __forceinline__ void init(const BwdTcParams& p, long long w0) {
    w = w0;
    rt = (int)(w0 % p.n_rtiles);
    const long long rest = w0 / p.n_rtiles;
    h = (int)(rest % p.row_heads);
    bp = (int)(rest / p.row_heads);
  }
};

template <int NDIM, bool kKeyRows>
__device__ __forceinline__ void decode_item(const BwdTcParams& p, const WorkCursor& cur, Item& it) {
  it.h = cur.h;
  it.b = (p.G > 1) ? cur.bp / p.G : cur.bp;
  int gl = (p.G > 1) ? cur.bp - it.b * p.G : 0;
  int rl = cur.rt;
  it.n_per_head = 1;
  it.skip = 0;
#pragma unroll
  for (int a = 0; a < B200NA_MAX_DIM; ++a) {
    if (a < NDIM) {
      int g = 0;
      if (p.G > 1) {
        g = gl % p.dil[a];
        gl /= p.dil[a];
      }
      it.g[a] = g;
      const int L = p.dil[a] == 1 ? p.X[a] : group_extent(p.X[a], p.dil[a], g);
      it.L[a] = L;
      int r = rl;
      if (a + 1 < NDIM) {
        const int rn = rl / p.Rr[a];
        r = rl - rn * p.Rr[a];
        rl = rn;
      }
      const int Lr = (kKeyRows && p.dense_rows) ? p.row_extent : L;  // extent of the rows
      const int lo = r * p.Tr[a];
      if (lo >= Lr) it.skip = 1;  // the tile lies beyond this dilation group
      it.r_lo[a] = lo;
      const int last = (lo + p.Tr[a] - 1 < Lr) ? lo + p.Tr[a] - 1 : Lr - 1;  // last real row
      int s_lo, e_lo, s_hi, e_hi;
      row_span<kKeyRows>(p, a, lo, L, s_lo, e_lo);
      row_span<kKeyRows>(p, a, last, L, s_hi, e_hi);
      const int Tc = p.Tc[a];
      int n = (e_hi - s_lo + Tc - 1) / Tc;
      if (n < 1) n = 1;  // a key nobody attends: visit one (fully masked) tile
      it.c_org[a] = s_lo;
      it.c_n[a] = n;
      it.int_lo[a] = (s_hi - s_lo + Tc - 1) / Tc;
      it.int_hi[a] = e_lo > s_lo ? (e_lo - s_lo) / Tc : 0;
      // rows past the extent (padding) interact with nothing: no tile is mask-free then
      if (lo + p.Tr[a] > Lr) it.int_hi[a] = it.int_lo[a];
      it.n_per_head *= it.c_n[a];
    } else {
      it.g[a] = 0; it.L[a] = 1; it.r_lo[a] = 0; it.c_org[a] = 0; it.c_n[a] = 1;
      it.int_lo[a] = 0; it.int_hi[a] = 1;
    }
  }
  it.n_na = it.n_per_head * (kKeyRows ? p.rep : 1);
  it.n_tiles = it.n_na + (kKeyRows ? 0 : p.extra_tiles);
}

// kPipe (pass dQ): the C1 and C2 column tiles live in rings of their own, because C2 (V) is free
// again right after the dP product while C1 (K) is needed until the dQ product of its tile.
template <int D, bool kPipe>
struct Smem {
  static constexpr int kTileBytes = kTile * D * 2;          // one 128-token operand tile
  static constexpr int kStages = (D == 128) ? 2 : 3;        // (C1, C2) pairs, or C2 tiles, in flight
  static constexpr int kRing1 = kPipe ? (D == 128 ? B200NA_BWD_RING1 : 4) : kStages;  // C1 ring
  static constexpr int kStage1Bytes = kPipe ? kTileBytes : 2 * kTileBytes;
  static constexpr int kRowOff = 0;                         // R1, R2
  static constexpr int kColOff = 2 * kTileBytes;
  static constexpr int kCol2Off = kColOff + kRing1 * kStage1Bytes;   // C2 ring (kPipe only)
  static constexpr int kPrefOff = kCol2Off + (kPipe ? kStages * kTileBytes : 0);
  static constexpr int kPrefEntries = 136;
  static constexpr int kStatOff = kPrefOff + kPrefEntries * 16;   // column stats [2][2][128] fp32
  static constexpr int kDescOff = kStatOff + (kPipe ? 0 : 2 * 2 * kTile * 4);
  static constexpr int kRecOff = kDescOff + kDescSlots * kDescBytes;
  static constexpr int kBarOff = kRecOff + kTileRecs * 16;
  // r_full, r_empty, sdp_full, sdp_free, acc_full, acc_empty, ds_full[2], ds_free[2],
  // desc_full[], desc_empty[], rec_full[8], rec_empty[8], c_full[R1], c_empty[R1], v_full[S],
  // v_empty[S]
  static constexpr int kNumBars = 10 + 2 * kDescSlots + 2 * kTileRecs + 2 * kRing1 + 2 * kStages;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kBytes = kMiscOff + 16;
  static_assert(kBytes <= 227 * 1024, "shared memory budget of one CTA");
};

struct Bars {
  uint64_t *r_full, *r_empty, *sdp_full, *sdp_free, *acc_full, *acc_empty, *ds_full, *ds_free;
  // pass dKdV only: these share the slots of ds_free[0] and ds_full[1], which pass dQ alone uses
  uint64_t *dp_full, *p_full;
  uint64_t *desc_full, *desc_empty, *rec_full, *rec_empty, *c_full, *c_empty, *v_full, *v_empty;
};

constexpr int kTileInterior = 1, kTileBoundary = 2, kTileRagged = 3;

// Per-item constants of the column-tile walk and classification, held in registers by the load
// thread (all its instructions are dependent, so shared-memory reads per tile would add latency).
struct TileWalk {
  int org[B200NA_MAX_DIM], end[B200NA_MAX_DIM], int_lo[B200NA_MAX_DIM], int_hi[B200NA_MAX_DIM];
  __device__ __forceinline__ void load(const Item& it) {
#pragma unroll
    for (int a = 0; a < B200NA_MAX_DIM; ++a) {
      org[a] = it.c_org[a];
      end[a] = it.c_n[a];
      int_lo[a] = it.int_lo[a];
      int_hi[a] = it.int_hi[a];
    }
  }
  template <int NDIM>
  __device__ __forceinline__ bool interior(const int (&c)[B200NA_MAX_DIM]) const {
    bool in = true;
#pragma unroll
    for (int a = 0; a < B200NA_MAX_DIM; ++a)
      if (a < NDIM) in = in && c[a] >= int_lo[a] && c[a] < int_hi[a];
    return in;
  }
  // colexicographic walk, axis 0 fastest; wraps to the first tile after the last one
  template <int NDIM>
  __device__ __forceinline__ void next(int (&c)[B200NA_MAX_DIM]) const {
    if (++c[0] < end[0]) return;
    c[0] = 0;
    if (NDIM == 1) return;
    if (++c[1] < end[1]) return;
    c[1] = 0;
    if (NDIM == 2) return;
    if (++c[2] < end[2]) return;
    c[2] = 0;
  }
};

template <int D, int kType, int NDIM, bool kKeyRows>
__global__ void __launch_bounds__(kThreads, 1)
fna_bwd_kernel(const __grid_constant__ CUtensorMap tm_r1, const __grid_constant__ CUtensorMap tm_r2,
               const __grid_constant__ CUtensorMap tm_c1, const __grid_constant__ CUtensorMap tm_c2,
               const __grid_constant__ CUtensorMap tm_e1, const __grid_constant__ CUtensorMap tm_e2,
               const BwdTcParams p) {
  constexpr bool kPipe = !kKeyRows;
  using SM = Smem<D, kPipe>;
  constexpr int kStages = SM::kStages;
  constexpr int kRing1 = SM::kRing1;
  constexpr int kTileBytes = SM::kTileBytes;
  constexpr int kDBlocks = D / 64;
  constexpr int kBlockBytes = kTile * 128;
  typedef typename std::conditional<kType == kTyBf16, __nv_bfloat16, __half>::type T;

  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* row_sm = smem + SM::kRowOff;
  uint8_t* col_sm = smem + SM::kColOff;
  uint8_t* col2_sm = smem + SM::kCol2Off;
  uint4* pref = reinterpret_cast<uint4*>(smem + SM::kPrefOff);
  float* colstat = reinterpret_cast<float*>(smem + SM::kStatOff);  // [2 buf][lse | delta][128]
  uint8_t* desc_sm = smem + SM::kDescOff;
  int4* tile_rec = reinterpret_cast<int4*>(smem + SM::kRecOff);
  uint64_t* bar_base = reinterpret_cast<uint64_t*>(smem + SM::kBarOff);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::kMiscOff + 4);

  Bars bars;
  bars.r_full = bar_base + 0;
  bars.r_empty = bar_base + 1;
  bars.sdp_full = bar_base + 2;
  bars.sdp_free = bar_base + 3;
  bars.acc_full = bar_base + 4;
  bars.acc_empty = bar_base + 5;
  bars.ds_full = bar_base + 6;   // [2]
  bars.ds_free = bar_base + 8;   // [2]
  bars.dp_full = bar_base + 8;
  bars.p_full = bar_base + 7;
  bars.desc_full = bar_base + 10;
  bars.desc_empty = bars.desc_full + kDescSlots;
  bars.rec_full = bars.desc_empty + kDescSlots;
  bars.rec_empty = bars.rec_full + kTileRecs;
  bars.c_full = bars.rec_empty + kTileRecs;
  bars.c_empty = bars.c_full + kRing1;
  bars.v_full = bars.c_empty + kRing1;
  bars.v_empty = bars.v_full + kStages;

  // read through a shuffle so that the compiler knows the value is warp-uniform: role branches
  // are then uniform, and address arithmetic inside them can use the uniform datapath
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;

  if ((ptx::smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, (8 << 8) | kStSmemAlign);
    return;
  }
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    ptx::mbar_init(bars.r_full, 1);
    ptx::mbar_init(bars.r_empty, 1);
    ptx::mbar_init(bars.sdp_full, 1);
    ptx::mbar_init(bars.sdp_free, kSoftmaxWarps);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(bars.ds_full + s, kSoftmaxWarps);
      ptx::mbar_init(bars.ds_free + s, 1);
    }
    ptx::mbar_init(bars.acc_full, 1);
    ptx::mbar_init(bars.acc_empty, kSoftmaxWarps);
    for (int s = 0; s < kDescSlots; ++s) {
      ptx::mbar_init(bars.desc_full + s, 1);
      // softmax warps + the MMA-issuing threads
      ptx::mbar_init(bars.desc_empty + s, kSoftmaxWarps + (kPipe ? 2 : 1));
    }
    for (int s = 0; s < kTileRecs; ++s) {
      ptx::mbar_init(bars.rec_full + s, 1);
      ptx::mbar_init(bars.rec_empty + s, kSoftmaxWarps);
    }
    for (int s = 0; s < kRing1; ++s) {
      ptx::mbar_init(bars.c_full + s, 1);
      ptx::mbar_init(bars.c_empty + s, 1);
    }
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(bars.v_full + s, 1);
      ptx::mbar_init(bars.v_empty + s, 1);
    }
    ptx::fence_barrier_init();
  }
  // per-axis prefix bit tables over the COLUMN tile, for the masks of boundary tiles
  build_prefix_tables(pref, p.ndim, p.Tc, threadIdx.x, kThreads);
  if (warp == kMmaWarp) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  if (warp == kLoadWarp && lane == 0) {
    ptx::prefetch_tensormap(&tm_r1);
    ptx::prefetch_tensormap(&tm_r2);
    ptx::prefetch_tensormap(&tm_c1);
    ptx::prefetch_tensormap(&tm_c2);
    if (p.extra_tiles) {
      ptx::prefetch_tensormap(&tm_e1);
      ptx::prefetch_tensormap(&tm_e2);
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);
  constexpr uint32_t kSCol = 0, kDpCol = 128, kAcc0Col = 256, kAcc1Col = 384;
  // Pass dQ keeps one accumulator, so columns [384, 512) are free: they hold two buffers of packed
  // dS (64 columns each). With dS written there instead of over dP, the logit / dP columns are
  // free again as soon as the softmax threads have read them, and the MMA thread computes the next
  // column tile's S and dP while the threads turn this tile's values into dS.
  constexpr uint32_t kDsCol = 384, kDsBufCols = 64;

  if (warp < kSoftmaxWarps) {
    // ============ P / dS computation and the epilogue (four threads per row) ====================
    const int part = warp >> 2;  // 0..3: columns [32 part, 32 part + 32) of every column tile
    const int row = ((warp & 3) << 5) | lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) << 5) << 16);
    const uint32_t my_s = lane_addr + kSCol + part * 32;
    const uint32_t my_dp = lane_addr + kDpCol + part * 32;
    const float c = p.scale_log2;
    constexpr float kLog2e = 1.4426950408889634f;
    uint32_t ph_sdp = 0, ph_dp = 0, ph_acc = 0, tseq = 0, dseq = 0;
    BTRACE_DECL(4 * 40)
    // in-tile coordinates of this thread's row, and of the column whose statistics it fetches
    int tr[B200NA_MAX_DIM], tcol[B200NA_MAX_DIM];
    {
      int rl = row, cl = row;
#pragma unroll
      for (int a = 0; a < B200NA_MAX_DIM; ++a) {
        tr[a] = (a < NDIM) ? rl % p.Tr[a] : 0;
        rl /= (a < NDIM) ? p.Tr[a] : 1;
        tcol[a] = (a < NDIM) ? cl % p.Tc[a] : 0;
        cl /= (a < NDIM) ? p.Tc[a] : 1;
      }
    }
    for (uint32_t seq = 0;; ++seq) {
      const uint32_t dslot = seq % kDescSlots;
      if (!__all_sync(0xffffffffu, wait_bar(bars.desc_full + dslot, (seq / kDescSlots) & 1,
                                            abort_flag, p.status, (5 << 8) | kStDescFull)))
        break;
      const Item& it = *reinterpret_cast<const Item*>(desc_sm + dslot * kDescBytes);
      const int n_tiles = it.n_tiles;
      if (n_tiles < 0) break;
      const int n_per_head = it.n_per_head;
      // span of columns this thread's row interacts with, per axis; token index of the row
      int lo_a[B200NA_MAX_DIM], hi_a[B200NA_MAX_DIM];
      bool row_valid = true;
      long long row_tok = it.b;
#pragma unroll
      for (int a = 0; a < B200NA_MAX_DIM; ++a) {
        if (a < NDIM) {
          const int i = it.r_lo[a] + tr[a];
          const bool dense = kKeyRows && p.dense_rows;
          row_valid = row_valid && i < (dense ? p.row_extent : it.L[a]);
          row_span<kKeyRows>(p, a, i, it.L[a], lo_a[a], hi_a[a]);
          row_tok = row_tok * (dense ? p.row_extent : p.X[a]) + (i * p.dil[a] + it.g[a]);
        } else {
          lo_a[a] = 0; hi_a[a] = 1;
        }
      }
      // pass dQ: the statistics belong to this thread's row
      float row_l = INFINITY, row_d = 0.f;
      if (!kKeyRows && row_valid) {
        row_l = p.lse[row_tok * p.Hq + it.h] * kLog2e;
        row_d = p.delta[row_tok * p.Hq + it.h];
      }
      const uint64_t c2 = ptx::f32x2(c, c), nl2 = ptx::f32x2(-row_l, -row_l),
                     nd2 = ptx::f32x2(-row_d, -row_d);
      bool alive = true;
      for (int iter = 0; iter < n_tiles; ++iter) {
        if (!__all_sync(0xffffffffu,
                        wait_bar(bars.rec_full + tseq % kTileRecs, (tseq / kTileRecs) & 1,
                                 abort_flag, p.status, (5 << 8) | kStRecFull))) {
          alive = false;
          break;
        }
        const int4 rec = tile_rec[tseq % kTileRecs];  // x = code, y/z/w = first column coordinate
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bars.rec_empty + tseq % kTileRecs);
        ++tseq;
        const bool interior = rec.x == kTileInterior;
        const int base3[B200NA_MAX_DIM] = {rec.y, rec.z, rec.w};
        // double-buffered by a count that runs across items, so that the buffer a thread fills
        // is never one a slower thread may still be reading
        float* stat = colstat + (tseq & 1) * 2 * kTile;
        if (kKeyRows) {
          // the statistics belong to the columns (queries): 128 threads fetch one column each
          if (part == 0) {
            const int hq = it.h * p.rep + iter / n_per_head;
            bool ok = true;
            long long tok = it.b;
#pragma unroll
            for (int a = 0; a < B200NA_MAX_DIM; ++a) {
              if (a < NDIM) {
                const int i = base3[a] + tcol[a];
                ok = ok && i < it.L[a];
                tok = tok * p.X[a] + (i * p.dil[a] + it.g[a]);
              }
            }
            // a column past the extent gets -LSE = -inf, i.e. P = 0
            // stored negated, so that the packed additions below take them as they are
            stat[row] = ok ? -p.lse[tok * p.Hq + hq] * kLog2e : -INFINITY;
            stat[kTile + row] = ok ? -p.delta[tok * p.Hq + hq] : 0.f;
          }
          named_bar_sync(1, kSoftmaxThreads);
        }
        uint32_t mw = ~0u;  // mask bits of this thread's 32 columns (boundary tiles only)
        if (rec.x == kTileRagged) {
          // last tile of the extra tokens: rec.y of its columns exist
          const int vcols = imin(imax(rec.y - part * 32, 0), 32);
          mw = vcols >= 32 ? ~0u : ((1u << vcols) - 1u);
        } else if (!interior) {
          const uint4 mk = tile_mask<NDIM>(pref, p.Tc, lo_a, hi_a, base3);
          mw = part == 0 ? mk.x : (part == 1 ? mk.y : (part == 2 ? mk.z : mk.w));
        }
        if (!__all_sync(0xffffffffu, wait_bar(bars.sdp_full, ph_sdp, abort_flag, p.status,
                                              (5 << 8) | kStSdpFull))) {
          alive = false;
          break;
        }
        ph_sdp ^= 1;
        ptx::tc_fence_after_sync();
        if (lane == 0 && (warp == 0 || warp == 15)) BTRACE(warp == 0 ? 2 : 3, 8);
        if constexpr (kPipe) {
          // all 32 logits and dP values of this thread into registers, then hand the columns
          // back to the MMA thread before doing the arithmetic
          uint32_t sr[32], dr[32];
          ptx::tmem_ld32(my_s, sr);
          ptx::tmem_ld32(my_dp, dr);
          ptx::tmem_ld_wait();
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bars.sdp_free);
          if (lane == 0 && (warp == 0 || warp == 15)) BTRACE(warp == 0 ? 2 : 3, 9);
          // packed (two-wide) arithmetic: half the instructions of the scalar forms
          uint32_t dk[16];
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float x0, x1, d0, d1;
            ptx::f32x2_split(ptx::fma_f32x2(ptx::f32x2(sr[j], sr[j + 1]), c2, nl2), x0, x1);
            float p0 = ptx::ex2(x0), p1 = ptx::ex2(x1);
            if (!interior) {
              p0 = ((mw >> j) & 1u) ? p0 : 0.f;
              p1 = ((mw >> (j + 1)) & 1u) ? p1 : 0.f;
            }
            ptx::f32x2_split(ptx::mul_f32x2(ptx::f32x2(p0, p1),
                                            ptx::add_f32x2(ptx::f32x2(dr[j], dr[j + 1]), nd2)),
                             d0, d1);
            dk[j >> 1] = pack2<kType>(d0, d1);
          }
          if (lane == 0 && (warp == 0 || warp == 15)) BTRACE(warp == 0 ? 2 : 3, 10);
          // the dS buffer of two tiles ago must have been consumed by its dQ product
          const uint32_t buf = dseq & 1;
          if (!__all_sync(0xffffffffu, wait_bar(bars.ds_free + buf, ((dseq >> 1) & 1) ^ 1,
                                                abort_flag, p.status, (5 << 8) | kStDsFree))) {
            alive = false;
            break;
          }
          ++dseq;
          ptx::tc_fence_after_sync();
          ptx::tmem_st16(lane_addr + kDsCol + buf * kDsBufCols + part * 16, dk);
          ptx::tmem_st_wait();
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bars.ds_full + buf);
          if (lane == 0 && (warp == 0 || warp == 15)) BTRACE(warp == 0 ? 2 : 3, 11);
        } else {
          // Pass dKdV. The two 128-column regions swap roles with every tile: S arrives in
          // region `reg`, dP in the other one. P = 2^(s c - lse) needs S only, so it is computed
          // (and stored, 16-bit, over the first half of this thread's consumed logits) while the
          // dP product still runs; dS = P (dP - delta) follows once dP is there and goes over
          // the second half. As soon as dP is in registers its region is handed back, and the
          // next tile's S is computed there during this tile's dS arithmetic and products.
          const uint32_t reg = dseq & 1;
          ++dseq;
          const uint32_t my_r = lane_addr + (reg ? kDpCol : kSCol) + part * 32;
          const uint32_t my_o = lane_addr + (reg ? kSCol : kDpCol) + part * 32;
          float pf[32];
          {
            uint32_t sr[32];
            ptx::tmem_ld32(my_r, sr);
            ptx::tmem_ld_wait();
            if (lane == 0 && (warp == 0 || warp == 15)) BTRACE(warp == 0 ? 2 : 3, 9);
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const uint64_t nl = *reinterpret_cast<const uint64_t*>(stat + part * 32 + j);
              float x0, x1;
              ptx::f32x2_split(ptx::fma_f32x2(ptx::f32x2(sr[j], sr[j + 1]), c2, nl), x0, x1);
              float p0 = ptx::ex2(x0), p1 = ptx::ex2(x1);
              if (!interior) {
                p0 = ((mw >> j) & 1u) ? p0 : 0.f;
                p1 = ((mw >> (j + 1)) & 1u) ? p1 : 0.f;
              }
              pf[j] = p0;
              pf[j + 1] = p1;
              pk[j >> 1] = pack2<kType>(p0, p1);
            }
            ptx::tmem_st16(my_r, pk);
          }
          if (lane == 0 && (warp == 0 || warp == 15)) BTRACE(warp == 0 ? 2 : 3, 10);
          // P is complete: its product with C2 can start while dS is still being computed
          ptx::tmem_st_wait();
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bars.p_full);
          if (lane == 0 && (warp == 0 || warp == 15)) BTRACE(warp == 0 ? 2 : 3, 11);
          if (!__all_sync(0xffffffffu, wait_bar(bars.dp_full, ph_dp, abort_flag, p.status,
                                                (5 << 8) | kStDpFull))) {
            alive = false;
            break;
          }
          ph_dp ^= 1;
          ptx::tc_fence_after_sync();
          if (lane == 0 && (warp == 0 || warp == 15)) BTRACE(warp == 0 ? 2 : 3, 12);
          {
            uint32_t dr[32];
            ptx::tmem_ld32(my_o, dr);
            ptx::tmem_ld_wait();
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bars.sdp_free);
            if (lane == 0 && (warp == 0 || warp == 15)) BTRACE(warp == 0 ? 2 : 3, 13);
            uint32_t dk[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const uint64_t nd = *reinterpret_cast<const uint64_t*>(stat + kTile + part * 32 + j);
              float d0, d1;
              ptx::f32x2_split(ptx::mul_f32x2(ptx::f32x2(pf[j], pf[j + 1]),
                                              ptx::add_f32x2(ptx::f32x2(dr[j], dr[j + 1]), nd)),
                               d0, d1);
              dk[j >> 1] = pack2<kType>(d0, d1);
            }
            ptx::tmem_st16(my_r + 16, dk);
          }
          ptx::tmem_st_wait();
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bars.ds_full);
          if (lane == 0 && (warp == 0 || warp == 15)) BTRACE(warp == 0 ? 2 : 3, 14);
        }
      }
      if (!alive) break;
      // ---- epilogue: accumulators -> gradient rows ----
      if (!__all_sync(0xffffffffu, wait_bar(bars.acc_full, ph_acc, abort_flag, p.status,
                                            (5 << 8) | kStAccFull)))
        break;
      ph_acc ^= 1;
      ptx::tc_fence_after_sync();
      const long long out_row = row_tok * p.row_heads + it.h;
#pragma unroll
      for (int acc = 0; acc < (kKeyRows ? 2 : 1); ++acc) {
        constexpr int kCols = D / kParts;  // output columns per thread: 32 or 16
        T* orow = reinterpret_cast<T*>(acc ? p.out1 : p.out0) + out_row * D + part * kCols;
        const float mul = acc ? 1.f : p.scale;
        const uint32_t src = lane_addr + (acc ? kAcc1Col : kAcc0Col) + part * kCols;
        uint32_t orr[kCols];
        if (kCols == 32) ptx::tmem_ld32(src, reinterpret_cast<uint32_t(&)[32]>(orr));
        else ptx::tmem_ld16(src, reinterpret_cast<uint32_t(&)[16]>(orr));
        ptx::tmem_ld_wait();
        if (row_valid) {
#pragma unroll
          for (int v4 = 0; v4 < kCols / 8; ++v4) {
            uint4 o;
            o.x = pack2<kType>(__uint_as_float(orr[v4 * 8 + 0]) * mul, __uint_as_float(orr[v4 * 8 + 1]) * mul);
            o.y = pack2<kType>(__uint_as_float(orr[v4 * 8 + 2]) * mul, __uint_as_float(orr[v4 * 8 + 3]) * mul);
            o.z = pack2<kType>(__uint_as_float(orr[v4 * 8 + 4]) * mul, __uint_as_float(orr[v4 * 8 + 5]) * mul);
            o.w = pack2<kType>(__uint_as_float(orr[v4 * 8 + 6]) * mul, __uint_as_float(orr[v4 * 8 + 7]) * mul);
            *reinterpret_cast<uint4*>(orow + v4 * 8) = o;
          }
        }
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        ptx::mbar_arrive(bars.acc_empty);
        ptx::mbar_arrive(bars.desc_empty + dslot);
      }
    }
  } else if (warp == kMmaWarp || (kPipe && warp == kMma2Warp)) {
    // =============================== MMA issue ==============================================
    // Pass dKdV: one thread issues everything. Pass dQ: the S / dP products and the dQ products
    // are issued by two threads in warps of different sub-partitions - an issuing thread shares
    // its scheduler with four busy softmax warps, and one thread alone cannot feed the tensor
    // pipe at its rate then. The two streams touch disjoint TMEM columns and are ordered against
    // each other through the softmax threads' barriers only.
    {
      // the whole warp runs this role; lane 0 performs the MMAs, commits and arrives
      const uint32_t issue = lane == 0;
      constexpr uint32_t idesc_s = ptx::make_idesc(kType == kTyBf16 ? 1 : 0, 0, 0, kTile, kTile);
      constexpr uint32_t idesc_acc = ptx::make_idesc(kType == kTyBf16 ? 1 : 0, 0, 1, kTile, D);
      constexpr uint32_t desc_hi = ptx::smem_desc_hi_sw128();
      const uint32_t row_base = ptx::smem_u32(row_sm);
      const uint32_t col_base = ptx::smem_u32(col_sm);
      const uint32_t col2_base = ptx::smem_u32(col2_sm);
      const uint32_t r1_lo = ptx::smem_desc_lo(row_base, 16);
      const uint32_t r2_lo = ptx::smem_desc_lo(row_base + kTileBytes, 16);
      const uint32_t s_tm = tmem_base + kSCol, dp_tm = tmem_base + kDpCol;
      const uint32_t acc0_tm = tmem_base + kAcc0Col, acc1_tm = tmem_base + kAcc1Col;
      const bool second = kPipe && warp == kMma2Warp;
      const int role = second ? 9 : 6;  // status word role
      auto wait_all = [&](uint64_t* bar, uint32_t parity, volatile int* af, int* st, int code) {
        return __all_sync(0xffffffffu, wait_bar(bar, parity, af, st, code)) != 0;
      };
      BTRACE_DECL(second ? 2 * 40 : 3 * 40)
      // S = R1 C1^T and dP = R2 C2^T: both operands K-major, contraction over the head dim
      auto issue_rc = [&](uint32_t d_tm, uint32_t r_lo, uint32_t ctile) {
        const uint32_t bd = ptx::smem_desc_lo(ctile, 16);
#pragma unroll
        for (int kb = 0; kb < D / 16; ++kb) {
          const uint32_t koff = ((kb >> 2) * kBlockBytes + (kb & 3) * 32) >> 4;
          ptx::mma_ss_lohi_if(issue, d_tm, r_lo + koff, desc_hi, bd + koff, desc_hi, idesc_s,
                           kb > 0 ? 1u : 0u);
        }
      };
      // acc += A C: A = 16-bit values in TMEM, 8 columns per 16-column step starting at `a_tm`
      // with `a_pair_stride` columns between pairs of steps; B = the column tile read MN-major,
      // contraction over the 128 columns
      auto issue_acc = [&](uint32_t acc_tm, uint32_t a_tm, uint32_t a_pair_stride, uint32_t ctile,
                           bool first) {
        const uint32_t bd = ptx::smem_desc_lo(ctile, kBlockBytes);
#pragma unroll
        for (int ks = 0; ks < kTile / 16; ++ks)
          ptx::mma_ts_lohi_if(issue, acc_tm, a_tm + (ks >> 1) * a_pair_stride + (ks & 1) * 8,
                           bd + ks * (2048 >> 4), desc_hi, idesc_acc, (first && ks == 0) ? 0u : 1u);
      };
      uint32_t ph_r = 0, ph_ae = 1;
      uint32_t slot = 0, ph_c = 0;    // ring position in the C1 (or combined) stages
      uint32_t slot2 = 0, ph_v = 0;   // pass dQ: ring position in the C2 stages
      uint32_t gt = 0;                // column tiles handled so far, over all items
      uint32_t slot_d = 0;            // pass dKdV: stage of the tile whose accumulations come next
      bool alive = true;
      for (uint32_t seq = 0; alive; ++seq) {
        const uint32_t dslot = seq % kDescSlots;
        if (!wait_all(bars.desc_full + dslot, (seq / kDescSlots) & 1, abort_flag, p.status,
                      (role << 8) | kStDescFull)) break;
        const int n = __shfl_sync(
            0xffffffffu, reinterpret_cast<const Item*>(desc_sm + dslot * kDescBytes)->n_tiles, 0);
        ptx::mbar_arrive_if(issue, bars.desc_empty + dslot);
        if (n < 0) break;
        if (kPipe && !second) {
          // ---- pass dQ, first issuer: dP and S of each column tile as soon as the softmax
          // threads have read the previous tile's. dP goes first: its C2 tile arrives early (a
          // C2 stage is released right after the product).
          if (!wait_all(bars.r_full, ph_r, abort_flag, p.status, (role << 8) | kStRFull)) break;
          ph_r ^= 1;
          for (int t = 0; t < n; ++t) {
            if (!wait_all(bars.sdp_free, (gt & 1) ^ 1, abort_flag, p.status,
                          (role << 8) | kStSdpFree) ||
                !wait_all(bars.v_full + slot2, ph_v, abort_flag, p.status,
                          (role << 8) | kStVFull)) {
              alive = false; break;
            }
            ++gt;
            if (lane == 0) BTRACE(0, 1);
            ptx::tc_fence_after_sync();
            issue_rc(dp_tm, r2_lo, col2_base + slot2 * kTileBytes);
            ptx::tc_commit_if(issue, bars.v_empty + slot2);
            if (++slot2 == kStages) {
              slot2 = 0;
              ph_v ^= 1;
            }
            if (!wait_all(bars.c_full + slot, ph_c, abort_flag, p.status,
                          (role << 8) | kStCFull)) {
              alive = false; break;
            }
            if (lane == 0) BTRACE(0, 2);
            ptx::tc_fence_after_sync();
            issue_rc(s_tm, r1_lo, col_base + slot * kTileBytes);
            ptx::tc_commit_if(issue, bars.sdp_full);
            // the row tiles are read by these products only
            if (t == n - 1) ptx::tc_commit_if(issue, bars.r_empty);
            if (lane == 0) BTRACE(0, 3);
            if (++slot == kRing1) {
              slot = 0;
              ph_c ^= 1;
            }
          }
        } else if (kPipe) {
          // ---- pass dQ, second issuer: dQ += dS C1 of each column tile when its dS is stored
          for (int t = 0; t < n; ++t) {
            const uint32_t buf = gt & 1;
            // the C1 wait cannot block (S of this tile was computed from the same stage); it
            // orders this thread's reads after the tile's arrival
            if (!wait_all(bars.ds_full + buf, (gt >> 1) & 1, abort_flag, p.status,
                          (role << 8) | kStDsFull) ||
                !wait_all(bars.c_full + slot, ph_c, abort_flag, p.status,
                          (role << 8) | kStCFull)) {
              alive = false; break;
            }
            ++gt;
            if (t == 0) {
              // the previous item's epilogue must have drained the accumulator
              if (!wait_all(bars.acc_empty, ph_ae, abort_flag, p.status,
                            (role << 8) | kStAccEmpty)) {
                alive = false; break;
              }
              ph_ae ^= 1;
            }
            if (lane == 0) BTRACE(4, 4);
            ptx::tc_fence_after_sync();
            issue_acc(acc0_tm, tmem_base + kDsCol + buf * kDsBufCols, 16,
                      col_base + slot * kTileBytes, t == 0);
            ptx::tc_commit_if(issue, bars.c_empty + slot);
            ptx::tc_commit_if(issue, bars.ds_free + buf);
            if (t == n - 1) ptx::tc_commit_if(issue, bars.acc_full);
            if (lane == 0) BTRACE(4, 5);
            if (++slot == kRing1) {
              slot = 0;
              ph_c ^= 1;
            }
          }
        } else {
          // ---- pass dKdV, per tile t: dV += P C2 when P is stored; S of tile t + 1 as soon as
          // the softmax threads have taken dP of tile t out of the region it goes to; dK += dS C1
          // when dS is stored; then dP of tile t + 1 (it overwrites tile t's P / dS operands,
          // behind their readers in issue order).
          if (!wait_all(bars.r_full, ph_r, abort_flag, p.status, (role << 8) | kStRFull)) break;
          ph_r ^= 1;
          const uint32_t reg_tm[2] = {s_tm, dp_tm};
          // first tile of the item: S, then dP (the other region's last readers, the previous
          // item's accumulations, were issued before)
          if (!wait_all(bars.c_full + slot, ph_c, abort_flag, p.status, (role << 8) | kStCFull) ||
              !wait_all(bars.sdp_free, (gt & 1) ^ 1, abort_flag, p.status,
                        (role << 8) | kStSdpFree))
            break;
          uint32_t c_cur = col_base + slot * 2 * kTileBytes, c_next = 0;
          ptx::tc_fence_after_sync();
          issue_rc(reg_tm[gt & 1], r1_lo, c_cur);
          ptx::tc_commit_if(issue, bars.sdp_full);
          issue_rc(reg_tm[(gt & 1) ^ 1], r2_lo, c_cur + kTileBytes);
          ptx::tc_commit_if(issue, bars.dp_full);
          if (n == 1) ptx::tc_commit_if(issue, bars.r_empty);
          ++gt;
          if (++slot == kStages) {
            slot = 0;
            ph_c ^= 1;
          }
          for (int t = 0; t < n; ++t) {
            const uint32_t k = gt - 1;  // global index of tile t (its S was the last one issued)
            if (t == 0) {
              // the previous item's epilogue must have drained the accumulators
              if (!wait_all(bars.acc_empty, ph_ae, abort_flag, p.status,
                            (role << 8) | kStAccEmpty)) {
                alive = false; break;
              }
              ph_ae ^= 1;
            }
            // Of a thread's columns [32 q, 32 q + 32) of the tile's region, [32 q, 32 q + 16)
            // hold its packed P and [32 q + 16, 32 q + 32) its dS.
            // acc1 += P C2 as soon as P is stored, while the threads still work on dS
            if (!wait_all(bars.p_full, k & 1, abort_flag, p.status, (role << 8) | kStPFull)) {
              alive = false; break;
            }
            if (lane == 0) BTRACE(0, 1);
            ptx::tc_fence_after_sync();
            issue_acc(acc1_tm, reg_tm[k & 1], 32, c_cur + kTileBytes, t == 0);
            if (lane == 0) BTRACE(0, 2);
            if (t + 1 < n) {
              // S of the next tile, into the region dP of this tile has been taken out of
              if (!wait_all(bars.c_full + slot, ph_c, abort_flag, p.status,
                            (role << 8) | kStCFull) ||
                  !wait_all(bars.sdp_free, (gt & 1) ^ 1, abort_flag, p.status,
                            (role << 8) | kStSdpFree)) {
                alive = false; break;
              }
              c_next = col_base + slot * 2 * kTileBytes;
              if (lane == 0) BTRACE(0, 3);
              ptx::tc_fence_after_sync();
              issue_rc(reg_tm[gt & 1], r1_lo, c_next);
              ptx::tc_commit_if(issue, bars.sdp_full);
              if (lane == 0) BTRACE(0, 4);
              ++gt;
              if (++slot == kStages) {
                slot = 0;
                ph_c ^= 1;
              }
            }
            // acc0 += dS C1
            if (!wait_all(bars.ds_full, k & 1, abort_flag, p.status, (role << 8) | kStDsFull)) {
              alive = false; break;
            }
            if (lane == 0) BTRACE(0, 5);
            ptx::tc_fence_after_sync();
            issue_acc(acc0_tm, reg_tm[k & 1] + 16, 32, c_cur, t == 0);
            ptx::tc_commit_if(issue, bars.c_empty + slot_d);
            if (lane == 0) BTRACE(0, 6);
            if (t == n - 1) ptx::tc_commit_if(issue, bars.acc_full);
            if (++slot_d == kStages) slot_d = 0;
            if (t + 1 < n) {
              // dP of the next tile over this tile's P / dS, behind their readers in issue order
              issue_rc(reg_tm[k & 1], r2_lo, c_next + kTileBytes);
              ptx::tc_commit_if(issue, bars.dp_full);
              if (lane == 0) BTRACE(0, 7);
              // the row tiles are read by the S / dP products only
              if (t + 1 == n - 1) ptx::tc_commit_if(issue, bars.r_empty);
            }
            c_cur = c_next;
          }
        }
      }
    }
  } else if (warp == kLoadWarp) {
    // ============ TMA loads, work-item decode, tile classification ==========================
    if (lane == 0) {
      uint32_t ph_re = 1, slot = 0, ph_ce = 1, slot2 = 0, ph_ve = 1, published = 0, tseq = 0;
      BTRACE_DECL(2 * 40)
      bool alive = true;
      // items are drawn in order from an atomic counter (row tiles differ a lot in how many
      // column tiles they need: borders, the first rows of a causal axis)
      WorkCursor cur;
      auto publish_next = [&]() -> const Item* {
        const uint32_t ds = published % kDescSlots;
        if (!wait_bar(bars.desc_empty + ds, ((published / kDescSlots) & 1) ^ 1, abort_flag,
                      p.status, (7 << 8) | kStDescEmpty)) {
          alive = false;
          return nullptr;
        }
        Item* out = reinterpret_cast<Item*>(desc_sm + ds * kDescBytes);
        bool found = false;
        while (true) {
          const long long w = (long long)atomicAdd(p.work, 1ull);
          if (w >= p.total_work) break;
          cur.init(p, w);
          decode_item<NDIM, kKeyRows>(p, cur, *out);
          if (!out->skip) { found = true; break; }
        }
        if (!found) out->n_tiles = -1;
        ptx::mbar_arrive(bars.desc_full + ds);
        ++published;
        return out;
      };
      const Item* itp = publish_next();
      while (alive && itp != nullptr && itp->n_tiles >= 0) {
        const Item& it = *itp;
        const int n_tiles = it.n_tiles, n_per_head = it.n_per_head, b = it.b;
        const int g0 = it.g[0], g1 = it.g[1], g2 = it.g[2];
        // the stationary row tiles: R1, R2 of head it.h
        if (!wait_bar(bars.r_empty, ph_re, abort_flag, p.status, (7 << 8) | kStREmpty)) break;
        ph_re ^= 1;
        ptx::mbar_arrive_expect_tx(bars.r_full, 2 * kTileBytes);
        {
          const int x0 = it.r_lo[0] * p.dil[0] + g0, x1 = it.r_lo[1] * p.dil[1] + g1,
                    x2 = it.r_lo[2] * p.dil[2] + g2;
          for (int db = 0; db < kDBlocks; ++db) {
            ptx::tma_load_5d(row_sm + db * kBlockBytes, &tm_r1, bars.r_full, it.h * D + db * 64,
                             x0, x1, x2, b);
            ptx::tma_load_5d(row_sm + kTileBytes + db * kBlockBytes, &tm_r2, bars.r_full,
                             it.h * D + db * 64, x0, x1, x2, b);
          }
        }
        TileWalk tw;
        tw.load(it);
        int tc[B200NA_MAX_DIM] = {0, 0, 0};
        // head of the column tiles: the kv head of a query head, or the query heads of a kv head
        int col_head = kKeyRows ? it.h * p.rep : it.h / p.rep;
        int in_head = 0;
        const Item* next = nullptr;
        const int publish_at = imin(kStages - 1, n_tiles - 1);
        const int n_na = it.n_na;
        for (int iter = 0; iter < n_tiles && alive; ++iter) {
          // pass dQ: the extra tokens follow the neighborhood tiles; every query attends them
          const bool is_extra = iter >= n_na;
          int4 rec;
          int x0, x1, x2;
          if (is_extra) {
            const int e0 = (iter - n_na) * kTile, valid = p.n_extra - e0;
            rec = make_int4(valid >= kTile ? kTileInterior : kTileRagged, valid, 0, 0);
            x0 = e0; x1 = 0; x2 = 0;
          } else {
            const int k0 = tw.org[0] + tc[0] * p.Tc[0],
                      k1 = NDIM > 1 ? tw.org[1] + tc[1] * p.Tc[1] : 0,
                      k2 = NDIM > 2 ? tw.org[2] + tc[2] * p.Tc[2] : 0;
            rec = make_int4(tw.template interior<NDIM>(tc) ? kTileInterior : kTileBoundary, k0, k1,
                            k2);
            x0 = k0 * p.dil[0] + g0; x1 = k1 * p.dil[1] + g1; x2 = k2 * p.dil[2] + g2;
            tw.template next<NDIM>(tc);
          }
          if (!wait_bar(bars.rec_empty + tseq % kTileRecs, ((tseq / kTileRecs) & 1) ^ 1, abort_flag,
                        p.status, (7 << 8) | kStRecEmpty)) { alive = false; break; }
          tile_rec[tseq % kTileRecs] = rec;
          ptx::mbar_arrive(bars.rec_full + tseq % kTileRecs);
          ++tseq;
          if constexpr (kPipe) {
            // C2 first: its stage is free long before the C1 stage of the same age
            if (!wait_bar(bars.v_empty + slot2, ph_ve, abort_flag, p.status,
                          (7 << 8) | kStVEmpty)) {
              alive = false; break;
            }
            BTRACE(1, 6);
            ptx::mbar_arrive_expect_tx(bars.v_full + slot2, kTileBytes);
            for (int db = 0; db < kDBlocks; ++db)
              ptx::tma_load_5d(col2_sm + slot2 * kTileBytes + db * kBlockBytes,
                               is_extra ? &tm_e2 : &tm_c2, bars.v_full + slot2,
                               col_head * D + db * 64, x0, x1, x2, b);
            if (++slot2 == kStages) {
              slot2 = 0;
              ph_ve ^= 1;
            }
            if (!wait_bar(bars.c_empty + slot, ph_ce, abort_flag, p.status,
                          (7 << 8) | kStCEmpty)) {
              alive = false; break;
            }
            BTRACE(1, 7);
            ptx::mbar_arrive_expect_tx(bars.c_full + slot, kTileBytes);
            for (int db = 0; db < kDBlocks; ++db)
              ptx::tma_load_5d(col_sm + slot * kTileBytes + db * kBlockBytes,
                               is_extra ? &tm_e1 : &tm_c1, bars.c_full + slot,
                               col_head * D + db * 64, x0, x1, x2, b);
          } else {
            if (!wait_bar(bars.c_empty + slot, ph_ce, abort_flag, p.status,
                          (7 << 8) | kStCEmpty)) {
              alive = false; break;
            }
            ptx::mbar_arrive_expect_tx(bars.c_full + slot, 2 * kTileBytes);
            uint8_t* dst = col_sm + slot * 2 * kTileBytes;
            for (int db = 0; db < kDBlocks; ++db) {
              ptx::tma_load_5d(dst + db * kBlockBytes, is_extra ? &tm_e1 : &tm_c1,
                               bars.c_full + slot, col_head * D + db * 64, x0, x1, x2, b);
              ptx::tma_load_5d(dst + kTileBytes + db * kBlockBytes, is_extra ? &tm_e2 : &tm_c2,
                               bars.c_full + slot, col_head * D + db * 64, x0, x1, x2, b);
            }
          }
          if (++slot == kRing1) {
            slot = 0;
            ph_ce ^= 1;
          }
          if (kKeyRows && ++in_head == n_per_head) {  // next query head of the group
            in_head = 0;
            ++col_head;
          }
          if (alive && iter == publish_at) next = publish_next();
        }
        itp = next;
      }
    }
  }

  // ---- teardown ----------------------------------------------------------------------------
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) {
    // the last CTA to get here re-arms the work counters for the next launch that uses them
    __threadfence();
    if (atomicAdd(p.work + 1, 1ull) == (unsigned long long)gridDim.x - 1) {
      p.work[0] = 0;
      p.work[1] = 0;
      __threadfence();
    }
  }
  if (*abort_flag) {
    // draining after an expired wait: let loads in flight land before shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
    __syncthreads();
  }
  if (warp == kMmaWarp) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host side -------------------------------------------------------------------------------

long long* g_bwd_trace = nullptr;
int g_bwd_trace_pass = 0;

template <int D, bool kBf16, bool kKeyRows>
const void* bwd_kernel_for_ndim(int ndim) {
  constexpr int kType = kBf16 ? kTyBf16 : kTyF16;
  if (ndim == 1) return (const void*)fna_bwd_kernel<D, kType, 1, kKeyRows>;
  if (ndim == 2) return (const void*)fna_bwd_kernel<D, kType, 2, kKeyRows>;
  return (const void*)fna_bwd_kernel<D, kType, 3, kKeyRows>;
}
const void* bwd_kernel_variant(int D, bool bf16, int ndim, bool key_rows) {
  if (D == 128) {
    if (bf16) return key_rows ? bwd_kernel_for_ndim<128, true, true>(ndim)
                              : bwd_kernel_for_ndim<128, true, false>(ndim);
    return key_rows ? bwd_kernel_for_ndim<128, false, true>(ndim)
                    : bwd_kernel_for_ndim<128, false, false>(ndim);
  }
  if (bf16) return key_rows ? bwd_kernel_for_ndim<64, true, true>(ndim)
                            : bwd_kernel_for_ndim<64, true, false>(ndim);
  return key_rows ? bwd_kernel_for_ndim<64, false, true>(ndim)
                  : bwd_kernel_for_ndim<64, false, false>(ndim);
}

// Opt-in shared memory per kernel variant and device, set once.
int ensure_smem_attribute(const void* fn, int smem_bytes) {
  static std::mutex mu;
  static const void* done[64][24];
  int dev = 0;
  B200NA_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return B200NA_ERR_DEVICE;
  std::lock_guard<std::mutex> lk(mu);
  for (int i = 0; i < 24; ++i) {
    if (done[dev][i] == fn) return B200NA_OK;
    if (done[dev][i] == nullptr) {
      B200NA_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           smem_bytes));
      done[dev][i] = fn;
      return B200NA_OK;
    }
  }
  return B200NA_ERR_UNSUPPORTED;
}

}  // namespace
}  // namespace b200na

extern "C" B200NA_API int b200na_na_backward_direct(
    const void* q, const void* k, const void* v, const void* o, const void* d_out, const float* lse,
    const void* add_k, const void* add_v, int n_extra, void* dq, void* dk, void* dv, void* d_add_k,
    void* d_add_v, float* delta_scratch, int ndim, const int* shape, const int* kernel,
    const int* stride, const int* dilation, const int* causal, const int* q_tile,
    const int* kv_tile, int B, int Hq, int Hkv, int D, int dtype, float scale,
    b200na_stream_t stream_) {
  using namespace b200na;
  if (!q || !k || !v || !o || !d_out || !lse || !dq || !dk || !dv || !delta_scratch || !shape ||
      !kernel || !q_tile || !kv_tile)
    return B200NA_ERR_INVALID_ARGUMENT;
  if (n_extra < 0 || (n_extra > 0 && (!add_k || !add_v || !d_add_k || !d_add_v)))
    return B200NA_ERR_INVALID_ARGUMENT;
  if (B < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv != 0) return B200NA_ERR_INVALID_ARGUMENT;
  if (dtype != B200NA_F16 && dtype != B200NA_BF16) return B200NA_ERR_UNSUPPORTED;
  if (D != 64 && D != 128) return B200NA_ERR_UNSUPPORTED;
  if (!(scale > 0.f)) return B200NA_ERR_INVALID_ARGUMENT;
  uintptr_t al = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                 reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(d_out) |
                 reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) |
                 reinterpret_cast<uintptr_t>(dv);
  if (n_extra > 0)
    al |= reinterpret_cast<uintptr_t>(add_k) | reinterpret_cast<uintptr_t>(add_v) |
          reinterpret_cast<uintptr_t>(d_add_k) | reinterpret_cast<uintptr_t>(d_add_v);
  if (al % 16 != 0) return B200NA_ERR_ALIGNMENT;
  NaAxes ax;
  int rc = fill_axes(ax, ndim, shape, kernel, stride, dilation, causal);
  if (rc != B200NA_OK) return rc;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int sms = 0;
  int* status_ptr = nullptr;
  if ((rc = fna_device_info(&sms, &status_ptr)) != B200NA_OK) return rc;

  BwdTcParams base;
  memset(&base, 0, sizeof(base));
  base.ndim = ndim;
  base.G = 1;
  int tq[B200NA_MAX_DIM], tkv[B200NA_MAX_DIM];
  long long tokens = 1, nq = 1, nkv = 1;
  for (int a = 0; a < B200NA_MAX_DIM; ++a) {
    const bool on = a < ndim;
    base.X[a] = ax.shape[a]; base.kernel[a] = ax.kernel[a]; base.stride[a] = ax.stride[a];
    base.dil[a] = ax.dilation[a]; base.causal[a] = ax.causal[a];
    tq[a] = on ? q_tile[a] : 1;
    tkv[a] = on ? kv_tile[a] : 1;
    if (tq[a] < 1 || tkv[a] < 1) return B200NA_ERR_INVALID_ARGUMENT;
    base.G *= base.dil[a];
    tokens *= base.X[a];
    nq *= tq[a];
    nkv *= tkv[a];
  }
  if (nq != kTile || nkv != kTile) return B200NA_ERR_INVALID_ARGUMENT;
  if (tokens * B > 0x7fffffffLL || (long long)Hq * D > 0x7fffffffLL) return B200NA_ERR_UNSUPPORTED;
  base.B = B; base.Hq = Hq; base.Hkv = Hkv; base.rep = Hq / Hkv;
  base.scale = scale;
  base.scale_log2 = scale * 1.4426950408889634f;
  base.lse = lse;
  base.delta = delta_scratch;
  base.status = status_ptr;

  CUtensorMap mq, mdo, mk, mv;
  if ((rc = fna_make_tensor_map_direct(&mq, q, dtype, B, base.X, Hq, D, tq, base.dil)) != B200NA_OK) return rc;
  if ((rc = fna_make_tensor_map_direct(&mdo, d_out, dtype, B, base.X, Hq, D, tq, base.dil)) != B200NA_OK) return rc;
  if ((rc = fna_make_tensor_map_direct(&mk, k, dtype, B, base.X, Hkv, D, tkv, base.dil)) != B200NA_OK) return rc;
  if ((rc = fna_make_tensor_map_direct(&mv, v, dtype, B, base.X, Hkv, D, tkv, base.dil)) != B200NA_OK) return rc;
  // extra tokens [B, n_extra, Hkv, D] are a one-axis layout of their own; flat views of Q / dO
  // ([B, N, Hq, D]) serve the pass that computes their gradients
  const int flat_tile[B200NA_MAX_DIM] = {kTile, 1, 1}, ones[B200NA_MAX_DIM] = {1, 1, 1};
  const int x_extra[B200NA_MAX_DIM] = {n_extra > 0 ? n_extra : 1, 1, 1};
  const int x_flat[B200NA_MAX_DIM] = {(int)tokens, 1, 1};
  CUtensorMap mek = mk, mev = mv, mqf = mq, mdof = mdo;
  if (n_extra > 0) {
    if ((rc = fna_make_tensor_map_direct(&mek, add_k, dtype, B, x_extra, Hkv, D, flat_tile, ones)) != B200NA_OK) return rc;
    if ((rc = fna_make_tensor_map_direct(&mev, add_v, dtype, B, x_extra, Hkv, D, flat_tile, ones)) != B200NA_OK) return rc;
    if ((rc = fna_make_tensor_map_direct(&mqf, q, dtype, B, x_flat, Hq, D, flat_tile, ones)) != B200NA_OK) return rc;
    if ((rc = fna_make_tensor_map_direct(&mdof, d_out, dtype, B, x_flat, Hq, D, flat_tile, ones)) != B200NA_OK) return rc;
  }

  if ((rc = launch_delta(o, d_out, delta_scratch, tokens * B * Hq, D, dtype, stream)) != B200NA_OK)
    return rc;

  // pass 0: dQ (rows Q, dO; columns K, V, then the extra tokens); pass 1: dK, dV (rows K, V;
  // columns Q, dO); pass 2, with extra tokens only: their gradients (rows = the extra tokens,
  // columns = all queries of the batch entry, flat)
  for (int pass = 0; pass < (n_extra > 0 ? 3 : 2); ++pass) {
    const bool key_rows = pass >= 1;
    const bool dense = pass == 2;
    BwdTcParams p = base;
    int kernel_ndim = ndim;
    if (dense) {
      kernel_ndim = 1;
      p.ndim = 1;
      p.G = 1;
      p.dense_rows = 1;
      p.row_extent = n_extra;
      for (int a = 0; a < B200NA_MAX_DIM; ++a) {
        p.X[a] = a == 0 ? (int)tokens : 1;
        p.kernel[a] = 1; p.stride[a] = 1; p.dil[a] = 1; p.causal[a] = 0;
      }
    }
    if (pass == 0) {
      p.n_extra = n_extra;
      p.extra_tiles = (n_extra + kTile - 1) / kTile;
    }
    long long n_rtiles = 1;
    for (int a = 0; a < B200NA_MAX_DIM; ++a) {
      p.Tr[a] = dense ? flat_tile[a] : (key_rows ? tkv[a] : tq[a]);
      p.Tc[a] = dense ? flat_tile[a] : (key_rows ? tq[a] : tkv[a]);
      // rows per axis: the largest dilation group, or the extra tokens
      const int need = dense ? (a == 0 ? n_extra : 1) : (p.X[a] + p.dil[a] - 1) / p.dil[a];
      p.Rr[a] = (need + p.Tr[a] - 1) / p.Tr[a];
      n_rtiles *= p.Rr[a];
    }
    if (n_rtiles > 0x7fffffffLL) return B200NA_ERR_UNSUPPORTED;
    p.n_rtiles = (int)n_rtiles;
    p.row_heads = key_rows ? Hkv : Hq;
    p.total_work = n_rtiles * p.row_heads * B * p.G;
    p.out0 = dense ? d_add_k : (key_rows ? dk : dq);
    p.out1 = dense ? d_add_v : (key_rows ? dv : nullptr);
    if ((rc = fna_work_counters(&p.work, stream)) != B200NA_OK) return rc;
    p.trace = pass == g_bwd_trace_pass ? g_bwd_trace : nullptr;
    const void* fn = bwd_kernel_variant(D, dtype == B200NA_BF16, kernel_ndim, key_rows);
    const int smem_bytes = key_rows ? (D == 128 ? Smem<128, false>::kBytes : Smem<64, false>::kBytes)
                                    : (D == 128 ? Smem<128, true>::kBytes : Smem<64, true>::kBytes);
    if ((rc = ensure_smem_attribute(fn, smem_bytes)) != B200NA_OK) return rc;
    const int grid = (int)(p.total_work < sms ? p.total_work : sms);
    void* args_q[] = {(void*)&mq, (void*)&mdo, (void*)&mk, (void*)&mv, (void*)&mek, (void*)&mev, (void*)&p};
    void* args_k[] = {(void*)&mk, (void*)&mv, (void*)&mq, (void*)&mdo, (void*)&mek, (void*)&mev, (void*)&p};
    void* args_e[] = {(void*)&mek, (void*)&mev, (void*)&mqf, (void*)&mdof, (void*)&mek, (void*)&mev, (void*)&p};
    B200NA_CUDA_TRY(cudaLaunchKernel(fn, dim3(grid), dim3(kThreads),
                                     dense ? args_e : (key_rows ? args_k : args_q), smem_bytes,
                                     stream));
  }
  return B200NA_OK;
}

#if defined(B200NA_BWD_TRACE) && B200NA_BWD_TRACE
extern "C" B200NA_API void b200na_debug_set_bwd_trace(void* buf, int pass) {
  b200na::g_bwd_trace = reinterpret_cast<long long*>(buf);
  b200na::g_bwd_trace_pass = pass;
}
#endif
