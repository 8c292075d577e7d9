// Fused neighborhood attention forward for sm_100a (B200): TMA-fed shared-memory tiles,
// tcgen05 (UMMA) matrix multiplies accumulating in tensor memory, online softmax in registers.
//
// Functional contract = the reference's Blackwell FNA forward
// (csrc/src/blackwell_fna_forward.cu:57-267 host contract; mask geometry
// csrc/include/natten/cuda/fna_blackwell/collective/fna_fusion.hpp:88-124, 284-489): a CTA owns
// a 256-row query tile and walks the bounding box of key/value tiles (128 rows each) its
// queries' windows touch. Operands are either the caller's [B, *X, H, D] tensors, gathered tile
// by tile through rank-5 tensor maps (direct mode), or token-permuted [B', S, H, D] tensors.
// The design is this library's own:
//   * warp roles: 16 softmax warps (a 128-row half per 8 warps, two threads per row),
//     1 MMA-issue warp (run converged, lane 0 performs the MMAs), 1 TMA-load warp that also
//     decodes work items; persistent CTAs draw (q-tile, head, batch') items from a counter.
//     A second shape of the same template owns ONE 128-row half per CTA (10 warps, half the
//     shared and tensor memory) and runs two CTAs per SM: for small windows, where 128 queries
//     share far fewer keys than 256 do.
//   * key/value tiles gathered from the caller's layout start at the first attended key instead
//     of on a grid; head dims below the kernel's 64 / 128 channels are read through tensor maps
//     with the head as an axis of its own (the missing channels come back as zeros).
//   * TMEM: S0 S1 O0 O1 (128 fp32 columns each at D = 128); P (16-bit) overwrites S in place and
//     feeds P.V straight from TMEM; the O rescale is lazy (only when a row maximum grows by more
//     than 2^8) and is done by the softmax threads between the two MMAs of their half.
//   * every KV tile is classified against the whole query tile in closed form; only boundary
//     tiles pay for the element mask, built from per-axis prefix bit tables in shared memory.
//   * the same kernel runs dense attention (extra KV tokens, self-attention fast path).
//   * every mbarrier wait is bounded: on expiry the CTA records a status word and drains.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <mutex>
#include <unordered_map>
#include <type_traits>

#include "common.cuh"
#include "fna_device.cuh"
#include "fna_host.cuh"
#include "fna_instrument.cuh"
#include "ptx.cuh"

namespace b200na {
namespace {

constexpr int kQTile = 256;      // query rows of a two-half work item (a one-half item has kHalf)
constexpr int kHalf = 128;       // rows per softmax warpgroup / per MMA (M)
constexpr int kKVTile = 128;     // key/value rows per tile (N of QK^T, K of P.V)
constexpr int kSoftmaxThreadsPerHalf = 256;   // 2 column parts x 4 warps, one thread per row and part
// A CTA has 8 softmax warps per half, an MMA-issuing warp and a load warp: 18 warps with two
// halves (registers are allocated to warps in groups of four, so they cost as much as 20: the
// per-thread ceiling is 65536 / 640 = 102 -> 96, which the streaming softmax loop fits into), 10
// warps with one half, two such CTAs per SM (the same 640 thread slots).
constexpr int kDescSlots = 4;     // work-item descriptors the load warp may run ahead by
constexpr int kDescBytes = 128;
constexpr int kTileRecs = 8;      // per-tile records in flight (more than the K/V ring holds tiles)
constexpr float kRescaleThreshold = 8.0f;              // log2 units

// status word: (role << 8) | barrier id, role 1 = softmax, 2 = mma, 3 = load, 4 = setup
enum : int { kStSQFull = 1, kStSFull, kStPFull, kStOFull, kStOEmpty, kStKVFull, kStKVEmpty,
             kStQEmpty, kStSmemAlign, kStDescFull, kStDescEmpty, kStRecFull };

__device__ int g_status_word;
// Work counters of the dynamic item scheduler: [slot][0] = next item, [slot][1] = CTAs finished;
// the last CTA of a launch to finish zeroes its pair again. Two kernels in flight must never
// share a pair, so pairs belong to streams: launches on one stream run one after the other and
// reuse that stream's pair ([0, kStreamSlots)). A launch that is being captured into a CUDA graph
// may later be replayed on any stream, next to anything: it takes a pair of its own from a
// separate pool that is handed out in turn ([kStreamSlots, kCounterSlots)).
constexpr int kStreamSlots = 1024;
constexpr int kCounterSlots = 4096;
__device__ unsigned long long g_work_counters[kCounterSlots][2];

struct FnaParams {
  int ndim;
  int X[B200NA_MAX_DIM];
  int kernel[B200NA_MAX_DIM];
  int stride[B200NA_MAX_DIM];
  int dil[B200NA_MAX_DIM];
  int causal[B200NA_MAX_DIM];
  int Tq[B200NA_MAX_DIM];
  int Tkv[B200NA_MAX_DIM];
  int tkv_shift[B200NA_MAX_DIM];  // log2(Tkv) when Tkv is a power of two, else -1
  int Rq[B200NA_MAX_DIM];   // query tiles per axis per dilation group
  int Rkv[B200NA_MAX_DIM];  // kv tiles per axis per dilation group
  int G;                    // prod(dil)
  int q_org[B200NA_MAX_DIM];   // layout coordinate of local query index 0 (spatial sharding; else 0)
  int kv_org[B200NA_MAX_DIM];  // layout coordinate of local key/value index 0
  int q_len[B200NA_MAX_DIM];   // number of real (non-padding) local query coordinates per axis
  int o_ext[B200NA_MAX_DIM];   // direct: extents of the Q / O / LSE tensors (rows are written there)
  int kv_ext[B200NA_MAX_DIM];  // direct: extents of the K / V tensors
  int clip;                    // windows are cut to the keys [clip_lo, clip_hi) that are present
  int clip_lo[B200NA_MAX_DIM];
  int clip_hi[B200NA_MAX_DIM];
  int dense;                // dense attention: one axis, window = all keys (or causal prefix)
  int direct;               // Q/K/V/O/LSE are in the caller's [B, *X, H, D] layout (no permutation)
  long long tok_stride[3];  // direct: elements between consecutive tokens of q, k, v (0 = H * D)
  int half_axis;            // direct: axis along which the query tile splits into its two halves
  int n_extra;              // extra key/value tokens every query attends (0 = none)
  int extra_tiles;          // ceil(n_extra / 128): KV tiles appended to every item's walk
  int Bp, Hq, Hkv;
  int halves;               // 128-row halves of a query tile: 2 (256-token tile) or 1 (128)
  int d_real;               // head dim of the tensors (<= the kernel's D; the rest reads as zeros)
  int sep_heads;            // direct: tensor maps list the head as an axis of its own (d_real < D)
  int Sq, Skv;              // rows per batch' in the q / kv tensors
  int n_qtiles;             // ceil(Sq / 256)
  long long total_work;     // n_qtiles * Hq * Bp
  float scale;
  float scale_log2;
  void* o;
  float* lse;
  int* status;
  unsigned long long* work;  // [0] next work item, [1] CTAs done (see g_work_counters)
#ifdef B200NA_PROFILE
  long long* prof;  // [grid][4 roles][8] cycle counters (instrumented builds only)
#endif
#ifdef B200NA_TEST_HOOKS
  int test_withhold;  // test-hook build: every CTA keeps back the record of its n-th tile (0 = off)
#endif
};

struct Item {
  int bp, h, hk, qt;
  int b;                      // batch entry (bp / G)
  int g[B200NA_MAX_DIM];      // dilation group offset per axis
  int L[B200NA_MAX_DIM];      // extent of this dilation group (dense: number of keys)
  int q_lo[B200NA_MAX_DIM];   // first query coordinate of the tile
  int kv_lo[B200NA_MAX_DIM];  // first key coordinate of the first kv tile per axis
  int kv_t0[B200NA_MAX_DIM];  // the same in tile units (permuted operands: tiles lie on a grid)
  int kv_n[B200NA_MAX_DIM];   // kv tiles per axis
  int ws_hi[B200NA_MAX_DIM];  // window start of the tile's last query
  int we_lo[B200NA_MAX_DIM];  // window end of the tile's first query
  int n_tiles;   // neighborhood tiles + extra-KV tiles
  int n_na;      // neighborhood tiles only
  int skip;
};
static_assert(sizeof(Item) <= kDescBytes, "descriptor slot too small");

__device__ __forceinline__ void axis_window(const FnaParams& p, int a, int i, int L, int& st,
                                            int& en) {
  if (p.dense) {
    st = 0;
    en = p.causal[0] ? imin(i + 1, L) : L;
  } else if (p.stride[a] == 1) {
    // unit stride: the stride-group leader is the query itself, no division needed
    const int k = p.kernel[a];
    const int wl = k >> 1, wr = (k >> 1) + ((k & 1) - 1);
    const int lead = imin(i, L - 1);
    if (p.causal[a]) {
      st = imax(lead - wl - wr, 0);
      en = imin(i + 1, L);
    } else {
      st = imax(lead - wl, 0) + ((lead + wr >= L) ? (L - wr - lead - 1) : 0);
      en = st + k;
    }
  } else {
    st = win_start(i, p.kernel[a], p.stride[a], L, p.causal[a]);
    en = win_end(i, st, p.kernel[a], L, p.causal[a]);
  }
  if (p.clip) {
    // partial attention over the keys that are present: the rest of the window belongs to
    // another call, whose result is merged with this one. Start and end stay monotone in i;
    // an empty window is [st, st).
    st = imin(imax(st, p.clip_lo[a]), p.clip_hi[a]);
    en = imax(imin(en, p.clip_hi[a]), st);
  }
}

// Coordinates of work item w = ((bp * Hq) + h) * n_qtiles + qt (decode_item turns qt into tile
// coordinates and walks causal axes from the far end, see there).
struct WorkCursor {
  long long w;
  int qt, h, bp;
  __device__ __forceinline__ void init(const FnaParams& p, long long w0) {
    w = w0;
    qt = (int)(w0 % p.n_qtiles);
    const long long rest = w0 / p.n_qtiles;
    h = (int)(rest % p.Hq);
    bp = (int)(rest / p.Hq);
  }
};

// x / d and x % d with a shift when d is a power of two (sh >= 0), else a real division.
__device__ __forceinline__ int div_fast(int x, int d, int sh) { return sh >= 0 ? (x >> sh) : x / d; }

// Geometry of one work item. Runs on the load warp's single thread, so integer divisions are
// avoided wherever the launch parameters allow (no dilation, unit stride, power-of-two tiles).
template <int NDIM>
__device__ __forceinline__ void decode_item(const FnaParams& p, const WorkCursor& cur, Item& it) {
  it.h = cur.h;
  it.bp = cur.bp;
  it.hk = (p.Hq == p.Hkv) ? cur.h : cur.h / (p.Hq / p.Hkv);
  it.b = (p.G > 1) ? cur.bp / p.G : cur.bp;
  int gl = (p.G > 1) ? cur.bp - it.b * p.G : 0;
  int ql = cur.qt;
  int qt = 0, qt_mul = 1;
  it.n_tiles = 1;
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
      it.L[a] = p.dense ? p.Skv : (p.dil[a] == 1 ? p.X[a] : group_extent(p.X[a], p.dil[a], g));
      int r = ql;
      if (a + 1 < NDIM) {  // the last axis takes what is left
        const int qn = ql / p.Rq[a];
        r = ql - qn * p.Rq[a];
        ql = qn;
      }
      // Longest items first: along a causal axis the number of kv tiles grows with the query
      // coordinate, so that axis is walked from its far end and the items a CTA draws last -
      // the ones that decide how long the other CTAs idle at the end - are the short ones.
      if (p.causal[a]) r = p.Rq[a] - 1 - r;
      qt += r * qt_mul;
      qt_mul *= p.Rq[a];
      if (!p.dense && r * p.Tq[a] >= p.q_len[a]) it.skip = 1;  // tile holds padding rows only
      if (p.direct && p.q_org[a] + r * p.Tq[a] >= it.L[a]) it.skip = 1;  // beyond this dilation group
      it.q_lo[a] = p.q_org[a] + r * p.Tq[a];
      const int q_hi = it.q_lo[a] + p.Tq[a] - 1;
      int s_lo, e_lo, s_hi, e_hi;
      axis_window(p, a, it.q_lo[a], it.L[a], s_lo, e_lo);
      axis_window(p, a, q_hi, it.L[a], s_hi, e_hi);
      it.ws_hi[a] = s_hi;
      it.we_lo[a] = e_lo;
      if (p.direct) {
        // Tiles gathered from the caller's layout may start at any coordinate: the walk begins
        // at the first key any query of the item attends, so a window that is a whole number of
        // tiles wide costs exactly that many tiles, wherever it starts.
        it.kv_lo[a] = s_lo;
        it.kv_t0[a] = 0;
        it.kv_n[a] = div_fast(e_hi - s_lo + p.Tkv[a] - 1, p.Tkv[a], p.tkv_shift[a]);
        if (p.clip && e_hi <= s_lo) {
          // none of the item's keys are present along this axis: one tile, masked for every row,
          // so that the rows still get O = 0 and LSE = -inf for the merge
          it.kv_lo[a] = imin(s_lo, p.clip_hi[a] - 1);
          it.kv_n[a] = 1;
        }
      } else {
        // windows are in layout coordinates, the key/value buffer starts at kv_org and is tiled
        // from there
        it.kv_t0[a] = div_fast(s_lo - p.kv_org[a], p.Tkv[a], p.tkv_shift[a]);
        it.kv_n[a] = div_fast(e_hi - p.kv_org[a] + p.Tkv[a] - 1, p.Tkv[a], p.tkv_shift[a]) - it.kv_t0[a];
        it.kv_lo[a] = p.kv_org[a] + it.kv_t0[a] * p.Tkv[a];
      }
      it.n_tiles *= it.kv_n[a];
    } else {
      it.L[a] = 1; it.q_lo[a] = 0; it.kv_lo[a] = 0; it.kv_t0[a] = 0; it.kv_n[a] = 1;
      it.ws_hi[a] = 0; it.we_lo[a] = 1; it.g[a] = 0;
    }
  }
  it.qt = qt;
  if (p.dense && it.qt * kQTile >= p.Sq) it.skip = 1;
  it.n_na = it.n_tiles;
  it.n_tiles += p.extra_tiles;
}
// Position of the kv-tile walk of one item: tile counters per axis (from 0) and the layout
// coordinate of the tile's first key per axis.
struct KvWalk {
  int c[B200NA_MAX_DIM];
  int lo[B200NA_MAX_DIM];
};
// First row of the tile in a token-permuted key/value operand.
template <int NDIM>
__device__ __forceinline__ int kv_tile_row(const FnaParams& p, const Item& it, const KvWalk& w) {
  if (NDIM == 1) return (it.kv_t0[0] + w.c[0]) * kKVTile;
  if (NDIM == 2) return (it.kv_t0[0] + w.c[0] + p.Rkv[0] * (it.kv_t0[1] + w.c[1])) * kKVTile;
  return (it.kv_t0[0] + w.c[0] +
          p.Rkv[0] * (it.kv_t0[1] + w.c[1] + p.Rkv[1] * (it.kv_t0[2] + w.c[2]))) * kKVTile;
}
// True when every key of the tile lies inside the window of every query of the item.
template <int NDIM>
__device__ __forceinline__ bool kv_tile_interior(const FnaParams& p, const Item& it,
                                                 const KvWalk& w) {
  bool in = true;
#pragma unroll
  for (int a = 0; a < B200NA_MAX_DIM; ++a) {
    if (a < NDIM) in = in && (w.lo[a] >= it.ws_hi[a]) && (w.lo[a] + p.Tkv[a] <= it.we_lo[a]);
  }
  return in;
}

// ES = bytes per operand element (2: fp16 / bf16, 1: 8-bit floats); kH = 128-row halves of the
// query tile a CTA owns: 2 (one CTA per SM) or 1 (two CTAs per SM, each with half the shared
// memory and half the tensor memory)
template <int D, int ES, int kH>
struct Smem {
  static constexpr int kTileBytes = kKVTile * D * ES;       // one K or V tile / one Q half
  // ring slots shared by K and V
  static constexpr int kStages = kH == 2 ? ((kTileBytes >= 32768) ? 4 : 6)
                                         : ((kTileBytes >= 32768) ? 2 : 4);
  static constexpr int kQOff = 0;
  static constexpr int kKVOff = kH * kTileBytes;
  static constexpr int kPrefOff = kKVOff + kStages * kTileBytes;
  static constexpr int kPrefEntries = 136;                  // sum(T_a + 1) <= 128 + 1 + 2 + 2
  static constexpr int kXchgOff = kPrefOff + kPrefEntries * 16;   // row max / row sum exchange
  static constexpr int kXchgBytes = (2 * 2 * 2 + 2 * 2) * kHalf * 4;
  static constexpr int kDescOff = kXchgOff + kXchgBytes;          // work-item descriptor ring
  static constexpr int kRecOff = kDescOff + kDescSlots * kDescBytes;  // per-tile records
  static constexpr int kBarOff = kRecOff + kTileRecs * 16;
  // barriers: q_full, q_empty, s_full[2], p_full[2], o_full[2], o_empty[2], desc_full[4],
  // desc_empty[4], rec_full[8], kv_full[S], kv_empty[S]
  static constexpr int kNumBars = 10 + 2 * kDescSlots + kTileRecs + 2 * kStages;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  // 1 KB per softmax warp: output rows are regrouped there so that stores cover whole rows
  static constexpr int kStageOff = (kMiscOff + 16 + 127) / 128 * 128;
  static constexpr int kStageBytes = 1024;
  static constexpr int kBytes = kStageOff + 8 * kH * kStageBytes;
  // two CTAs of the one-half variant share an SM: 228 KB minus 1 KB the system keeps per CTA
  static_assert(kBytes <= (kH == 2 ? 227 * 1024 : 113 * 1024), "shared memory budget");
  // a record is overwritten kTileRecs tiles later; its readers lag the load warp by at most
  // the tiles the K/V ring holds plus one
  static_assert(kTileRecs >= kStages / 2 + 3, "per-tile record ring too short");
};

// Position in the K/V ring: slot index and the phase parity of that slot's barriers.
template <int kStages>
struct RingPos {
  uint32_t slot = 0, phase = 0;
  __device__ __forceinline__ void advance() {
    if (++slot == kStages) {
      slot = 0;
      phase ^= 1;
    }
  }
};

struct Bars {
  uint64_t* q_full;
  uint64_t* q_empty;
  uint64_t* s_full;   // [2]
  uint64_t* p_full;   // [2]
  uint64_t* o_full;   // [2]
  uint64_t* o_empty;  // [2]
  uint64_t* desc_full;   // [kDescSlots] descriptor published by the load warp
  uint64_t* desc_empty;  // [kDescSlots] every consumer has copied the descriptor
  uint64_t* rec_full;    // [kTileRecs] per-tile record written by the load warp
  uint64_t* kv_full;  // [stages]
  uint64_t* kv_empty; // [stages]
};

// Consumer side of the work-item descriptor ring: waits for descriptor number `seq` and returns
// it in place (nullptr when the CTA is draining). The slot stays valid until every consumer has
// called release_item for it; the ring is deeper than the number of items in flight, so holding
// a slot for a whole item costs nothing. The end of the work list is a descriptor with
// n_tiles < 0.
__device__ __forceinline__ const Item* fetch_item(const uint8_t* desc_sm, const Bars& bars,
                                                  uint32_t seq, volatile int* abort_flag,
                                                  int* status, int role) {
  const uint32_t slot = seq % kDescSlots;
  if (!wait_bar(bars.desc_full + slot, (seq / kDescSlots) & 1, abort_flag, status,
                (role << 8) | kStDescFull))
    return nullptr;
  return reinterpret_cast<const Item*>(desc_sm + slot * kDescBytes);
}
__device__ __forceinline__ void release_item(const Bars& bars, uint32_t seq) {
  ptx::mbar_arrive(bars.desc_empty + seq % kDescSlots);
}

// Advances the colexicographic kv-tile walk by one tile (no divisions on the per-tile path).
template <int NDIM>
__device__ __forceinline__ void kv_tile_next(const FnaParams& p, const Item& it, KvWalk& w) {
  ++w.c[0];
  w.lo[0] += p.Tkv[0];
  if (NDIM == 1 || w.c[0] < it.kv_n[0]) return;
  w.c[0] = 0;
  w.lo[0] = it.kv_lo[0];
  ++w.c[1];
  w.lo[1] += p.Tkv[1];
  if (NDIM == 2 || w.c[1] < it.kv_n[1]) return;
  w.c[1] = 0;
  w.lo[1] = it.kv_lo[1];
  ++w.c[2];
  w.lo[2] += p.Tkv[2];
}

// kH = 2: the CTA owns a 256-row query tile as two halves that alternate on the tensor pipe, one
// CTA per SM. kH = 1: a 128-row query tile per CTA and two CTAs per SM - the two tiles then walk
// key/value boxes of their own (the union of the windows of 128 queries is much smaller than
// that of 256 when windows are small) and their item boundaries are staggered, so one CTA's
// pipeline fill and drain overlaps the other's steady state. Chosen per problem by the host
// (query tile of 128 or 256 tokens).
template <int D, int kType, int NDIM, int kH>
__global__ void __launch_bounds__((8 * kH + 2) * 32, kH == 1 ? 2 : 1)
fna_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_ek,
               const __grid_constant__ CUtensorMap tm_ev, const FnaParams p) {
  constexpr int kES = kType >= kTyE4m3 ? 1 : 2;   // bytes per operand element
  constexpr bool kF8 = kES == 1;
  // the CTA-shape constants of this variant (the file-level ones are the two-half values)
  constexpr int kQTile = kHalf * kH;
  constexpr int kSoftmaxWarps = 8 * kH;
  constexpr int kMmaWarp = kSoftmaxWarps;
  constexpr int kLoadWarp = kSoftmaxWarps + 1;
  constexpr int kThreads = (kSoftmaxWarps + 2) * 32;
  constexpr int kTmemCols = 256 * kH;
  using SM = Smem<D, kES, kH>;
  constexpr int kStages = SM::kStages;
  constexpr int kTileBytes = SM::kTileBytes;
  constexpr int kBlockElems = 128 / kES;           // elements of one 128-byte column block
  constexpr int kDBlocks = D / kBlockElems;        // 128-byte column blocks per row
  constexpr int kBlockBytes = kKVTile * 128;       // one column block of a 128-row tile

  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* q_sm = smem + SM::kQOff;
  uint8_t* kv_sm = smem + SM::kKVOff;
  uint4* pref = reinterpret_cast<uint4*>(smem + SM::kPrefOff);
  float* xmax = reinterpret_cast<float*>(smem + SM::kXchgOff);        // [2 parity][2 half][2 part][128]
  float* xsum = xmax + 2 * 2 * 2 * kHalf;                             // [2 half][2 part][128]
  uint8_t* desc_sm = smem + SM::kDescOff;
  int4* tile_rec = reinterpret_cast<int4*>(smem + SM::kRecOff);
  uint64_t* bar_base = reinterpret_cast<uint64_t*>(smem + SM::kBarOff);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::kMiscOff + 4);

  Bars bars;
  bars.q_full = bar_base + 0;
  bars.q_empty = bar_base + 1;
  bars.s_full = bar_base + 2;
  bars.p_full = bar_base + 4;
  bars.o_full = bar_base + 6;
  bars.o_empty = bar_base + 8;
  bars.desc_full = bar_base + 10;
  bars.desc_empty = bar_base + 10 + kDescSlots;
  bars.rec_full = bar_base + 10 + 2 * kDescSlots;
  bars.kv_full = bar_base + 10 + 2 * kDescSlots + kTileRecs;
  bars.kv_empty = bar_base + 10 + 2 * kDescSlots + kTileRecs + kStages;

  // read through a shuffle so that the compiler knows the value is warp-uniform: role branches
  // are then uniform, and address arithmetic inside them can use the uniform datapath
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;

  // ---- setup -------------------------------------------------------------------------------
  if ((ptx::smem_u32(smem) & 1023u) != 0) {  // swizzled tiles need 1024-byte aligned bases
    if (threadIdx.x == 0) atomicCAS(p.status, 0, (4 << 8) | kStSmemAlign);
    return;
  }
#if defined(B200NA_PROFILE) && B200NA_PROFILE >= 2
  for (int i = threadIdx.x; i < 2048; i += kThreads) reinterpret_cast<uint32_t*>(smem + SM::kBytes)[i] = 0;
#endif
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    ptx::mbar_init(bars.q_full, 1);
    ptx::mbar_init(bars.q_empty, 1);
    for (int h = 0; h < 2; ++h) {
      ptx::mbar_init(bars.s_full + h, 1);
      ptx::mbar_init(bars.p_full + h, kSoftmaxThreadsPerHalf);
      ptx::mbar_init(bars.o_full + h, 1);
      ptx::mbar_init(bars.o_empty + h, kSoftmaxThreadsPerHalf);
    }
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(bars.kv_full + s, 1);
      ptx::mbar_init(bars.kv_empty + s, 1);
    }
    for (int s = 0; s < kTileRecs; ++s) ptx::mbar_init(bars.rec_full + s, 1);
    for (int s = 0; s < kDescSlots; ++s) {
      ptx::mbar_init(bars.desc_full + s, 1);
      ptx::mbar_init(bars.desc_empty + s, kSoftmaxWarps * 32 + 1);  // softmax threads + MMA thread
    }
    ptx::fence_barrier_init();
  }
  // per-axis prefix bit tables over the key/value tile, for the masks of boundary tiles
  build_prefix_tables(pref, p.ndim, p.Tkv, threadIdx.x, kThreads);
  if (warp == kMmaWarp) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  if (warp == kLoadWarp && lane == 0) {
    ptx::prefetch_tensormap(&tm_q);
    ptx::prefetch_tensormap(&tm_k);
    ptx::prefetch_tensormap(&tm_v);
    if (p.extra_tiles) {
      ptx::prefetch_tensormap(&tm_ek);
      ptx::prefetch_tensormap(&tm_ev);
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);
  // TMEM columns (kH = 2): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [384,384+D); (kH = 1):
  // S0 [0,128) O0 [128,128+D); P aliases S.
  auto s_col = [](int half) -> uint32_t { return (uint32_t)half * 128u; };
  auto o_col = [](int half) -> uint32_t { return (uint32_t)kH * 128u + (uint32_t)half * 128u; };

  if (warp < kSoftmaxWarps) {
    // ======================= softmax + correction + epilogue ===============================
    // Two threads share a query row: `part` 0 owns key columns [0, 64) of every tile and output
    // columns [0, D/2), `part` 1 the other halves. A lone warp cannot keep a sub-partition's
    // issue slots busy, so halving the per-thread work halves the softmax latency that sits
    // between the two MMAs of a half.
    const int half = warp >> 3;
    const int part = (warp >> 2) & 1;
    const int row = ((warp & 3) << 5) | lane;          // row inside the half = TMEM lane
    const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) << 5) << 16);
    const uint32_t s_addr = lane_addr + s_col(half);
    const uint32_t my_s = s_addr + part * 64;                 // my 64 fp32 logit columns
    const uint32_t my_p = s_addr + part * 64;                 // my 32 packed P columns (in place)
    const uint32_t my_o = lane_addr + o_col(half) + part * (D / 2);
    const int bar_id = 1 + half;
    const float c = p.scale_log2;
    uint32_t ph_s = 0, ph_o = 0;
    uint32_t tseq = 0;  // tiles consumed so far, indexes the per-tile record ring
    uint8_t* o_ptr = reinterpret_cast<uint8_t*>(p.o);
    // in-tile coordinates of this thread's query row (fixed for the whole kernel)
    int tq[B200NA_MAX_DIM];
    {
      int rl = half * kHalf + row;
#pragma unroll
      for (int a = 0; a < B200NA_MAX_DIM; ++a) {
        tq[a] = (a < NDIM) ? rl % p.Tq[a] : 0;
        rl /= (a < NDIM) ? p.Tq[a] : 1;
      }
    }

    PROF_DECL
    // window of this thread's query row
    // Kept as start | end << 16 per axis in the 3-D kernel (the host admits 3-D extents below
    // 2^16 only): six live registers less across the tile loop, which is what keeps the
    // compiler from spilling inside it.
    constexpr bool kPackWindow = NDIM == 3;
    int ws[B200NA_MAX_DIM], we[B200NA_MAX_DIM];
    uint32_t wse[B200NA_MAX_DIM];
    auto row_window = [&](const Item& item, int (&s_)[B200NA_MAX_DIM], int (&e_)[B200NA_MAX_DIM]) {
#pragma unroll
      for (int a = 0; a < B200NA_MAX_DIM; ++a) {
        if (a < NDIM) {
          axis_window(p, a, item.q_lo[a] + tq[a], item.L[a], s_[a], e_[a]);
        } else {
          s_[a] = 0; e_[a] = 1;
        }
      }
    };
    const Item* itp = fetch_item(desc_sm, bars, 0, abort_flag, p.status, 1);
    if (__all_sync(0xffffffffu, itp != nullptr) && itp->n_tiles >= 0) row_window(*itp, ws, we);
    for (uint32_t seq = 0;; ++seq) {
      if (!__all_sync(0xffffffffu, itp != nullptr)) break;
      const Item& it = *itp;  // read in place: the fields do not occupy registers across a tile
      const int n_tiles = it.n_tiles;
      if (n_tiles < 0) break;  // end of this CTA's work list
#pragma unroll
      for (int a = 0; a < B200NA_MAX_DIM; ++a) wse[a] = (uint32_t)ws[a] | ((uint32_t)we[a] << 16);
      float m = -INFINITY, sum = 0.f;   // sum covers this thread's columns only
      bool alive = true;
      for (int iter = 0; iter < n_tiles; ++iter) {
        // The load warp classified the tile when it fetched it: x = 0 nothing to mask, 1 window
        // boundary (y, z, w = first key coordinate of the tile per axis), 2 ragged last tile of
        // the extra tokens (y = valid columns). The record is there long before the logits are,
        // so the masks are ready when the wait for the logits ends.
        if (!__all_sync(0xffffffffu,
                        wait_bar(bars.rec_full + tseq % kTileRecs, (tseq / kTileRecs) & 1,
                                 abort_flag, p.status, (1 << 8) | kStRecFull))) {
          alive = false;
          break;
        }
        const int4 rec = tile_rec[tseq % kTileRecs];
        ++tseq;
        const bool interior = rec.x == 0;
        // Mask words of this thread's two 32-column chunks (boundary tiles only).
        uint32_t mw0 = ~0u, mw1 = ~0u;
        if (rec.x == 2) {
          const int v0 = imin(imax(rec.y - (part * 64), 0), 32);
          const int v1 = imin(imax(rec.y - (part * 64 + 32), 0), 32);
          mw0 = v0 >= 32 ? ~0u : ((1u << v0) - 1u);
          mw1 = v1 >= 32 ? ~0u : ((1u << v1) - 1u);
        } else if (!interior) {
          const int base3[B200NA_MAX_DIM] = {rec.y, rec.z, rec.w};
          if constexpr (kPackWindow) {
#pragma unroll
            for (int a = 0; a < B200NA_MAX_DIM; ++a) {
              ws[a] = (int)(wse[a] & 0xffffu);
              we[a] = (int)(wse[a] >> 16);
            }
          }
          const uint4 mk = tile_mask<NDIM>(pref, p.Tkv, ws, we, base3);
          mw0 = part ? mk.z : mk.x;
          mw1 = part ? mk.w : mk.y;
        }
        // warp-uniform outcome: the TMEM accesses below are warp-collective
        if (!__all_sync(0xffffffffu, wait_bar(bars.s_full + half, ph_s, abort_flag, p.status,
                                              (1 << 8) | kStSFull))) {
          alive = false;
          break;
        }
        ph_s ^= 1;
        PROF_MARK(0)
        if (row == 0 && part == 0) TRACE(half, 1)
        ptx::tc_fence_after_sync();
        // Pass 1: row maximum of the raw logits over this thread's 64 columns. Chunk 1 is read
        // first and dropped, chunk 0 stays in registers for pass 2.
        uint32_t sr[32];
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
        ptx::tmem_ld32(my_s + 32, sr);
        ptx::tmem_ld_wait();
        if (!interior) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (!((mw1 >> j) & 1u)) sr[j] = 0xff800000u;  // -inf
        }
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          mx0 = ptx::max3(mx0, __uint_as_float(sr[j]), __uint_as_float(sr[j + 1]));
          mx1 = ptx::max3(mx1, __uint_as_float(sr[j + 2]), __uint_as_float(sr[j + 3]));
        }
        ptx::tmem_ld32(my_s, sr);
        ptx::tmem_ld_wait();
        PROF_MARK(1)
        if (!interior) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (!((mw0 >> j) & 1u)) sr[j] = 0xff800000u;
        }
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          mx2 = ptx::max3(mx2, __uint_as_float(sr[j]), __uint_as_float(sr[j + 1]));
          mx3 = ptx::max3(mx3, __uint_as_float(sr[j + 2]), __uint_as_float(sr[j + 3]));
        }
        const float my_max = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        float* xm = xmax + (((iter & 1) * 2 + half) * 2) * kHalf;
        xm[part * kHalf + row] = my_max;
        named_bar_sync(bar_id, kSoftmaxThreadsPerHalf);
        const float m_new = ptx::max3(m, my_max, xm[(part ^ 1) * kHalf + row]);
        // Lazy rescale: keep the stale maximum while the true one is at most 2^8 larger.
        const bool grow = (m_new - m) * c > kRescaleThreshold;  // NaN (-inf - -inf) -> false
        if (__any_sync(0xffffffffu, grow)) {
          const float f = grow ? ptx::ex2((m - m_new) * c) : 1.f;
          if (grow) {
            sum *= f;
            m = m_new;
          }
          if (iter > 0) {
            // O_half is quiescent here: P.V of the previous tile completed before s_full fired.
#pragma unroll
            for (int ch = 0; ch < D / 32; ++ch) {
              uint32_t orr[16];
              ptx::tmem_ld16(my_o + ch * 16, orr);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) orr[j] = __float_as_uint(__uint_as_float(orr[j]) * f);
              ptx::tmem_st16(my_o + ch * 16, orr);
            }
          }
        }
        const float neg_mc = (m == -INFINITY) ? 0.f : -m * c;
        // Pass 2: p = 2^(s*c - m*c), 32 columns at a time; each packed chunk of P overwrites
        // logit columns this same thread has already consumed, so no other thread is involved.
        // x = s c - m c and the row sums in packed (two-wide) arithmetic: half the instructions
        // of the scalar forms for these two steps
        const uint64_t c2 = ptx::f32x2(c, c), nmc2 = ptx::f32x2(neg_mc, neg_mc);
        uint64_t acc0 = ptx::f32x2(0.f, 0.f), acc1 = acc0;
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          if (ch == 1) {
            ptx::tmem_ld32(my_s + 32, sr);
            ptx::tmem_ld_wait();
            if (!interior) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (!((mw1 >> j) & 1u)) sr[j] = 0xff800000u;
            }
          }
          if (kF8) {
            // 8-bit operands: P is rounded to e4m3, four probabilities per TMEM column
            uint32_t pk[8];
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float x0, x1, x2, x3;
              ptx::f32x2_split(ptx::fma_f32x2(ptx::f32x2(sr[j], sr[j + 1]), c2, nmc2), x0, x1);
              ptx::f32x2_split(ptx::fma_f32x2(ptx::f32x2(sr[j + 2], sr[j + 3]), c2, nmc2), x2, x3);
              const float p0 = ptx::ex2(x0), p1 = ptx::ex2(x1), p2 = ptx::ex2(x2), p3 = ptx::ex2(x3);
              acc0 = ptx::add_f32x2(acc0, ptx::f32x2(p0, p1));
              acc1 = ptx::add_f32x2(acc1, ptx::f32x2(p2, p3));
              pk[j >> 2] = ptx::pack4_e4m3(p0, p1, p2, p3);
            }
            ptx::tmem_st8(my_p + ch * 8, pk);
          } else {
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float x0, x1, x2, x3;
              ptx::f32x2_split(ptx::fma_f32x2(ptx::f32x2(sr[j], sr[j + 1]), c2, nmc2), x0, x1);
              ptx::f32x2_split(ptx::fma_f32x2(ptx::f32x2(sr[j + 2], sr[j + 3]), c2, nmc2), x2, x3);
              const float p0 = ptx::ex2(x0), p1 = ptx::ex2(x1), p2 = ptx::ex2(x2), p3 = ptx::ex2(x3);
              acc0 = ptx::add_f32x2(acc0, ptx::f32x2(p0, p1));
              acc1 = ptx::add_f32x2(acc1, ptx::f32x2(p2, p3));
              pk[j >> 1] = pack2<kType>(p0, p1);
              pk[(j >> 1) + 1] = pack2<kType>(p2, p3);
            }
            ptx::tmem_st16(my_p + ch * 16, pk);
          }
        }
        {
          float s0, s1, s2, s3;
          ptx::f32x2_split(acc0, s0, s1);
          ptx::f32x2_split(acc1, s2, s3);
          sum += (s0 + s1) + (s2 + s3);
        }
        PROF_MARK(2)
        ptx::tmem_st_wait();
        ptx::tc_fence_before_sync();
        ptx::mbar_arrive(bars.p_full + half);
        PROF_MARK(3)
        if (row == 0 && part == 0) TRACE(half, 2)
      }
      if (!alive) break;
      // The next item's descriptor was published while this item's second tile was loaded: its
      // window arithmetic is done here, in the time this thread would otherwise wait for the
      // last P.V.
      const Item* nxt = fetch_item(desc_sm, bars, seq + 1, abort_flag, p.status, 1);
      int nws[B200NA_MAX_DIM] = {0, 0, 0}, nwe[B200NA_MAX_DIM] = {1, 1, 1};
      if (__all_sync(0xffffffffu, nxt != nullptr) && nxt->n_tiles >= 0) row_window(*nxt, nws, nwe);
      // ---- epilogue: O / sum -> global, LSE ----
      // Everything that does not need the accumulator comes before the wait for the last P.V:
      // the row sums are final once the last tile's exponentials are.
      float* xs = xsum + half * 2 * kHalf;
      xs[part * kHalf + row] = sum;
      named_bar_sync(bar_id, kSoftmaxThreadsPerHalf);
      const float total = sum + xs[(part ^ 1) * kHalf + row];
      // Row of O / LSE this thread writes: a row of the permuted [B', S, H, D] operand, or - in
      // direct mode - the token of the caller's [B, *X, H, D] layout the query row stands for.
      long long out_row;
      bool valid;
      if (p.direct) {
        long long tok = it.b;
        valid = true;
#pragma unroll
        for (int a = 0; a < B200NA_MAX_DIM; ++a) {
          if (a < NDIM) {
            const int qa = it.q_lo[a] + tq[a];
            valid = valid && qa < it.L[a] && qa - p.q_org[a] < p.q_len[a];
            tok = tok * p.o_ext[a] + ((qa - p.q_org[a]) * p.dil[a] + it.g[a]);
          }
        }
        out_row = tok * p.Hq + it.h;
      } else {
        const int q_row = it.qt * kQTile + half * kHalf + row;
        valid = q_row < p.Sq;
        out_row = ((long long)it.bp * p.Sq + q_row) * p.Hq + it.h;
      }
      const float inv = total > 0.f ? 1.f / total : 0.f;
      if (!__all_sync(0xffffffffu, wait_bar(bars.o_full + half, ph_o, abort_flag, p.status,
                                            (1 << 8) | kStOFull)))
        break;
      ph_o ^= 1;
      PROF_MARK(4)
      ptx::tc_fence_after_sync();
      // This thread's share of its output row: D/2 elements = kChunks 16-byte chunks. A store of
      // one chunk per lane would touch 32 rows (32 separate lines) per instruction, and the
      // load/store unit would spend more time on the epilogue than the arithmetic does. The
      // chunks go through a 1 KB warp-private staging buffer instead, kRowsPerRound rows at a
      // time, and come back out with consecutive lanes holding consecutive chunks of one row:
      // every store instruction then writes whole rows.
      constexpr int kChunks = (D / 2) * kES / 16;       // 8 (128 bytes) or 4 (64 bytes)
      constexpr int kRowsPerRound = 64 / kChunks;       // rows whose chunks fill the 1 KB buffer
      constexpr int kPer = 16 / kES;                    // output elements per chunk
      uint4 pk[kChunks];
#pragma unroll
      for (int ch = 0; ch < D / 64; ++ch) {
        uint32_t orr[32];
        ptx::tmem_ld32(my_o + ch * 32, orr);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int v4 = 0; v4 < 32 / kPer; ++v4)
          pk[ch * (32 / kPer) + v4] = pack_out16<kType>(orr + v4 * kPer, inv);
      }
      // rows of the output tensor are d_real elements wide; chunks past that are not stored
      uint8_t* const orow = valid ? o_ptr + (out_row * p.d_real + part * (D / 2)) * kES : nullptr;
      const int my_chunks = imin(imax((p.d_real - part * (D / 2)) / kPer, 0), kChunks);
      uint4* const stage = reinterpret_cast<uint4*>(smem + SM::kStageOff + warp * SM::kStageBytes);
#pragma unroll
      for (int rd = 0; rd < 32 / kRowsPerRound; ++rd) {
        __syncwarp();
        if (lane / kRowsPerRound == rd) {
          const int lr = lane % kRowsPerRound;
#pragma unroll
          for (int cidx = 0; cidx < kChunks; ++cidx)  // XOR placement: conflict-free both ways
            stage[lr * kChunks + (cidx ^ (lr % kChunks))] = pk[cidx];
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int idx = i * 32 + lane;
          const int lr = idx / kChunks, cidx = (idx % kChunks) ^ (lr % kChunks);
          const uint4 val = stage[idx];
          // the row's address lives in the lane that owns the row (null: padding row)
          const unsigned long long rp = __shfl_sync(
              0xffffffffu, (unsigned long long)(uintptr_t)orow, rd * kRowsPerRound + lr);
          if (rp != 0ull && cidx < my_chunks)
            *reinterpret_cast<uint4*>((uint8_t*)(uintptr_t)rp + cidx * 16) = val;
        }
      }
      if (p.lse != nullptr && valid && part == 0)
        p.lse[out_row] = logf(total) + m * p.scale;
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(bars.o_empty + half);
      release_item(bars, seq);
      PROF_MARK(5)
      itp = nxt;
#pragma unroll
      for (int a = 0; a < B200NA_MAX_DIM; ++a) { ws[a] = nws[a]; we[a] = nwe[a]; }
    }
    if (row == 0 && part == 0) { PROF_FLUSH(half) }
  } else if (warp == kMmaWarp) {
    // =============================== MMA issue ==============================================
    {
      // the whole warp runs this role, converged, so that descriptor arithmetic stays in uniform
      // registers; lane 0 performs the MMAs, commits and arrives
      const uint32_t issue = lane == 0;
      auto wait_all = [&](uint64_t* bar, uint32_t parity, volatile int* af, int* st, int code) {
        return __all_sync(0xffffffffu, wait_bar(bar, parity, af, st, code)) != 0;
      };
      // element format codes of the instruction descriptor: kind::f16 0 = fp16, 1 = bf16;
      // kind::f8f6f4 0 = e4m3, 1 = e5m2 (P is always e4m3)
      constexpr int kFmt = kF8 ? (kType == kTyE5m2 ? 1 : 0) : (kType == kTyBf16 ? 1 : 0);
      constexpr uint32_t idesc_qk = ptx::make_idesc_ab(kFmt, kFmt, 0, 0, kHalf, kKVTile);
      constexpr uint32_t idesc_pv = ptx::make_idesc_ab(kF8 ? 0 : kFmt, kFmt, 0, 1, kHalf, D);
      uint32_t ph_q = 0, ph_p[2] = {0, 0}, ph_oe[2] = {1, 1};
      RingPos<kStages> ring;  // K and V tiles in load order
      const uint32_t q_base = ptx::smem_u32(q_sm);
      const uint32_t kv_base = ptx::smem_u32(kv_sm);
      bool alive = true;

      // Descriptors are kept as (low, high) words: the high word is one constant, the low word
      // of a tile is computed once and each K step adds a compile-time offset to it. Every
      // instruction of this role is on the critical path: the stream is warp-uniform so that
      // this arithmetic is done in uniform registers, where the MMA instruction takes it from.
      constexpr uint32_t desc_hi = ptx::smem_desc_hi_sw128();
      const uint32_t q_lo[2] = {ptx::smem_desc_lo(q_base, 16),
                                ptx::smem_desc_lo(q_base + kTileBytes, 16)};
      const uint32_t s_tm[2] = {tmem_base + s_col(0), tmem_base + s_col(1)};
      const uint32_t o_tm[2] = {tmem_base + o_col(0), tmem_base + o_col(1)};

      auto issue_qk = [&](int half, uint32_t k_addr) {
        const uint32_t a_lo = half ? q_lo[1] : q_lo[0];
        const uint32_t b_lo = ptx::smem_desc_lo(k_addr, 16);
        const uint32_t d = half ? s_tm[1] : s_tm[0];
        // one MMA consumes 32 bytes of the head dim per row: K = 16 (16-bit) or 32 (8-bit)
#pragma unroll
        for (int kb = 0; kb < D * kES / 32; ++kb) {
          const uint32_t koff = ((kb >> 2) * kBlockBytes + (kb & 3) * 32) >> 4;
          if (kF8)
            ptx::mma_ss_lohi_f8_if(issue, d, a_lo + koff, desc_hi, b_lo + koff, desc_hi,
                                   idesc_qk, kb > 0 ? 1u : 0u);
          else
            ptx::mma_ss_lohi_if(issue, d, a_lo + koff, desc_hi, b_lo + koff, desc_hi, idesc_qk,
                                kb > 0 ? 1u : 0u);
        }
      };
      // P for keys [0,64) sits in S columns [0,32), for keys [64,128) in columns [64,96): each
      // softmax thread writes its packed probabilities over its own logits.
      auto issue_pv = [&](int half, uint32_t v_addr, bool first) {
        const uint32_t b_lo = ptx::smem_desc_lo(v_addr, kBlockBytes);
        const uint32_t d = half ? o_tm[1] : o_tm[0];
        const uint32_t a = half ? s_tm[1] : s_tm[0];
        if (kF8) {
          // 8-bit: K = 32 keys per MMA = 8 packed columns; a thread's 64 probabilities take 16
          // columns at [0,16) resp. [64,80); V rows are 128 bytes, 32 rows per step
#pragma unroll
          for (int ks = 0; ks < kKVTile / 32; ++ks)
            ptx::mma_ts_lohi_f8_if(issue, d, a + (ks >> 1) * 64 + (ks & 1) * 8,
                                   b_lo + ks * (4096 >> 4), desc_hi, idesc_pv,
                                   (first && ks == 0) ? 0u : 1u);
        } else {
#pragma unroll
          for (int ks = 0; ks < kKVTile / 16; ++ks)
            ptx::mma_ts_lohi_if(issue, d, a + (ks >> 2) * 64 + (ks & 3) * 8,
                                b_lo + ks * (2048 >> 4), desc_hi, idesc_pv,
                                (first && ks == 0) ? 0u : 1u);
        }
      };

      PROF2_DECL
      for (uint32_t seq = 0; alive; ++seq) {
        const Item* itp = fetch_item(desc_sm, bars, seq, abort_flag, p.status, 2);
        if (!__all_sync(0xffffffffu, itp != nullptr)) break;
        const int n = __shfl_sync(0xffffffffu, itp->n_tiles, 0);  // all this role needs
        ptx::mbar_arrive_if(issue, bars.desc_empty + seq % kDescSlots);
        if (n < 0) break;
        PROF2_MARK(6)
        if (!wait_all(bars.q_full, ph_q, abort_flag, p.status, (2 << 8) | kStSQFull)) break;
        ph_q ^= 1;
        PROF2_MARK(0)
        TRACE2(2, 10)
        // tile 0: S_h = Q_h K0^T for both halves
        const uint32_t slot_k = ring.slot;
        if (!wait_all(bars.kv_full + slot_k, ring.phase, abort_flag, p.status,
                      (2 << 8) | kStKVFull)) break;
        ring.advance();
        PROF2_MARK(1)
        ptx::tc_fence_after_sync();
#pragma unroll
        for (int h = 0; h < kH; ++h) {
          issue_qk(h, kv_base + slot_k * kTileBytes);
          ptx::tc_commit_if(issue, bars.s_full + h);
        }
        ptx::tc_commit_if(issue, bars.kv_empty + slot_k);
        if (n == 1) ptx::tc_commit_if(issue, bars.q_empty);
        for (int iter = 0; iter < n && alive; ++iter) {
          // Both operands of this iteration (V of this tile, K of the next) are waited for up
          // front, so that nothing but the softmax hand-off separates the MMA bursts below.
          const uint32_t slot_v = ring.slot;
          if (!wait_all(bars.kv_full + slot_v, ring.phase, abort_flag, p.status,
                        (2 << 8) | kStKVFull)) { alive = false; break; }
          ring.advance();
          TRACE2(2, 11)
          const bool more = iter + 1 < n;
          uint32_t slot_kn = 0;
          if (more) {
            slot_kn = ring.slot;
            if (!wait_all(bars.kv_full + slot_kn, ring.phase, abort_flag, p.status,
                          (2 << 8) | kStKVFull)) { alive = false; break; }
            ring.advance();
            TRACE2(2, 16)
          }
          const uint32_t v_addr = kv_base + slot_v * kTileBytes;
          const uint32_t k_addr = kv_base + slot_kn * kTileBytes;
#pragma unroll
          for (int h = 0; h < kH; ++h) {
            if (!wait_all(bars.p_full + h, ph_p[h], abort_flag, p.status, (2 << 8) | kStPFull)) {
              alive = false; break;
            }
            ph_p[h] ^= 1;
            TRACE2(2, 12 + h)
            if (iter == 0) {
              // the previous item's epilogue must have drained O_h before it is overwritten
              if (!wait_all(bars.o_empty + h, ph_oe[h], abort_flag, p.status,
                            (2 << 8) | kStOEmpty)) { alive = false; break; }
              ph_oe[h] ^= 1;
            }
            ptx::tc_fence_after_sync();
            issue_pv(h, v_addr, iter == 0);
            TRACE2(2, 14 + h)
            if (more) {
              issue_qk(h, k_addr);
              ptx::tc_commit_if(issue, bars.s_full + h);
              TRACE2(2, 17 + h)
            } else {
              ptx::tc_commit_if(issue, bars.o_full + h);
            }
          }
          if (!alive) break;
          ptx::tc_commit_if(issue, bars.kv_empty + slot_v);
          if (more) {
            ptx::tc_commit_if(issue, bars.kv_empty + slot_kn);
            if (iter + 2 == n) ptx::tc_commit_if(issue, bars.q_empty);  // last Q.K^T has been issued
          }
        }
      }
      PROF2_FLUSH(2)
    }
  } else if (warp == kLoadWarp) {
    // =============================== TMA loads + item decode ================================
    if (lane == 0) {
      uint32_t ph_qe = 1;
      RingPos<kStages> ring;
      bool alive = true;
      PROF2_DECL
      // The load warp decodes every work item once (integer divisions, window arithmetic) and
      // publishes it through a small descriptor ring; it runs one item ahead of its own loads,
      // so the other roles find the next item's geometry - and its Q tile - waiting for them.
      // Descriptors are built in place in the ring and this thread reads its own copy back from
      // there: only it ever writes a slot, and not before kDescSlots further items.
      // Items are handed out by an atomic counter, in order: a CTA that drew short items (the
      // first query tiles of a causal axis, tiles at the borders) simply draws more of them.
      WorkCursor cur;
      uint32_t published = 0;
      uint32_t tseq = 0;  // tiles fetched so far, indexes the per-tile record ring
      // Decodes the next item that is not all padding and publishes it; publishes the end marker
      // (n_tiles < 0) when the list is exhausted. Returns the published descriptor (nullptr when
      // the CTA is draining).
      auto publish_next = [&]() -> const Item* {
        const uint32_t slot = published % kDescSlots;
        if (!wait_bar(bars.desc_empty + slot, ((published / kDescSlots) & 1) ^ 1, abort_flag,
                      p.status, (3 << 8) | kStDescEmpty)) {
          alive = false;
          return nullptr;
        }
        Item* out = reinterpret_cast<Item*>(desc_sm + slot * kDescBytes);
        bool found = false;
        while (true) {
          const long long w = (long long)atomicAdd(p.work, 1ull);
          if (w >= p.total_work) break;
          cur.init(p, w);
          decode_item<NDIM>(p, cur, *out);
          if (!out->skip) { found = true; break; }
        }
        if (!found) out->n_tiles = -1;
        ptx::mbar_arrive(bars.desc_full + slot);  // release: the descriptor is visible to waiters
        ++published;
        return out;
      };
      const Item* itp = publish_next();
      while (alive && itp != nullptr && itp->n_tiles >= 0) {
        const Item& it = *itp;
        const int n_tiles = it.n_tiles, n_na = it.n_na, bp = it.bp, hk = it.hk;
        if (!wait_bar(bars.q_empty, ph_qe, abort_flag, p.status, (3 << 8) | kStQEmpty)) break;
        ph_qe ^= 1;
        ptx::mbar_arrive_expect_tx(bars.q_full, kH * kTileBytes);
        for (int h = 0; h < kH; ++h)
          for (int db = 0; db < kDBlocks; ++db) {
            if (p.direct) {
              // box = half a query tile in the caller's layout; dilation is the box's element
              // stride, rows past the extent come back as zeros
              int x[B200NA_MAX_DIM];
#pragma unroll
              for (int a = 0; a < B200NA_MAX_DIM; ++a)
                x[a] = (it.q_lo[a] - p.q_org[a] +
                        ((h && a == p.half_axis) ? (p.Tq[a] >> 1) : 0)) * p.dil[a] + it.g[a];
              if (p.sep_heads) {
                // (channel, head, then the layout axes and the batch entry): channels past the
                // tensor's head dim come back as zeros
                if (NDIM < 3) x[NDIM] = it.b;
                ptx::tma_load_5d(q_sm + h * kTileBytes + db * kBlockBytes, &tm_q, bars.q_full,
                                 db * kBlockElems, it.h, x[0], x[1], x[2]);
              } else {
                ptx::tma_load_5d(q_sm + h * kTileBytes + db * kBlockBytes, &tm_q, bars.q_full,
                                 it.h * D + db * kBlockElems, x[0], x[1], x[2], it.b);
              }
            } else {
              ptx::tma_load_4d(q_sm + h * kTileBytes + db * kBlockBytes, &tm_q, bars.q_full,
                               db * kBlockElems, it.h, it.qt * kQTile + h * kHalf, bp);
            }
          }
        KvWalk walk = {{0, 0, 0}, {it.kv_lo[0], it.kv_lo[1], it.kv_lo[2]}};
        const Item* next = nullptr;
        const int publish_at = imin(kStages / 2 - 1, n_tiles - 1);
        for (int iter = 0; iter < n_tiles && alive; ++iter) {
          const bool is_extra = iter >= n_na;
          const int row0 = is_extra ? (iter - n_na) * kKVTile
                                    : (p.direct ? 0 : kv_tile_row<NDIM>(p, it, walk));
          int4 rec;
          if (is_extra) {
            const int valid = p.n_extra - (iter - n_na) * kKVTile;
            rec = make_int4(valid >= kKVTile ? 0 : 2, valid, 0, 0);
          } else {
            rec = make_int4(kv_tile_interior<NDIM>(p, it, walk) ? 0 : 1, walk.lo[0],
                            NDIM > 1 ? walk.lo[1] : 0, NDIM > 2 ? walk.lo[2] : 0);
          }
          // direct mode: coordinates of the tile's first key in the caller's layout
          int xk[B200NA_MAX_DIM] = {0, 0, 0};
          if (p.direct && !is_extra) {
#pragma unroll
            for (int a = 0; a < B200NA_MAX_DIM; ++a)
              xk[a] = (a < NDIM) ? (walk.lo[a] - p.kv_org[a]) * p.dil[a] + it.g[a] : 0;
          }
          if (!is_extra) kv_tile_next<NDIM>(p, it, walk);
          // extra tokens are shared by the dilation groups of a batch entry
          const int b_src = is_extra ? it.b : bp;
          for (int kv = 0; kv < 2; ++kv) {
            const uint32_t slot = ring.slot;
            if (!wait_bar(bars.kv_empty + slot, ring.phase ^ 1, abort_flag, p.status,
                          (3 << 8) | kStKVEmpty)) { alive = false; break; }
            ring.advance();
            TRACE2(3, 20 + kv)
            // The record goes out with its K tile. The K/V ring holds fewer tiles than
            // kTileRecs, so the entry it replaces is long consumed.
            if (kv == 0) {
              tile_rec[tseq % kTileRecs] = rec;
#ifdef B200NA_TEST_HOOKS
              if (!(p.test_withhold != 0 && (int)tseq + 1 == p.test_withhold))
#endif
              ptx::mbar_arrive(bars.rec_full + tseq % kTileRecs);
              ++tseq;
            }
            ptx::mbar_arrive_expect_tx(bars.kv_full + slot, kTileBytes);
            for (int db = 0; db < kDBlocks; ++db) {
              if (p.direct && !is_extra && p.sep_heads)
                ptx::tma_load_5d(kv_sm + slot * kTileBytes + db * kBlockBytes,
                                 kv == 0 ? &tm_k : &tm_v, bars.kv_full + slot, db * kBlockElems, hk,
                                 xk[0], NDIM < 2 ? it.b : xk[1], NDIM < 3 ? (NDIM < 2 ? 0 : it.b) : xk[2]);
              else if (p.direct && !is_extra)
                ptx::tma_load_5d(kv_sm + slot * kTileBytes + db * kBlockBytes,
                                 kv == 0 ? &tm_k : &tm_v, bars.kv_full + slot, hk * D + db * kBlockElems,
                                 xk[0], xk[1], xk[2], it.b);
              else
                ptx::tma_load_4d(kv_sm + slot * kTileBytes + db * kBlockBytes,
                                 is_extra ? (kv == 0 ? &tm_ek : &tm_ev) : (kv == 0 ? &tm_k : &tm_v),
                                 bars.kv_full + slot, db * kBlockElems, hk, row0, b_src);
            }
          }
          // Once this item's first tiles fill the ring the load thread would only wait for free
          // slots: that is when it decodes and publishes the next item.
          if (alive && iter == publish_at) next = publish_next();
        }
        itp = next;
      }
      PROF2_FLUSH(3)
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
#if defined(B200NA_PROFILE) && B200NA_PROFILE >= 2
  if (blockIdx.x == 0) {
    const uint32_t* tb = reinterpret_cast<const uint32_t*>(smem + SM::kBytes);
    for (int i = threadIdx.x; i < 2048; i += kThreads) p.prof[296 * 32 + 4096 + i] = tb[i];
  }
#endif
  if (*abort_flag) {
    // Draining after an expired wait: give loads that are still in flight time to land in this
    // CTA's shared memory before it is released.
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encode_fn(EncodeTiledFn* fn) {
  static std::mutex mu;
  static EncodeTiledFn cached = nullptr;
  std::lock_guard<std::mutex> lk(mu);
  if (!cached) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    B200NA_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres));
    if (!sym || qres != cudaDriverEntryPointSuccess) {
      set_last_cuda_error(cudaErrorUnknown, "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
      return B200NA_ERR_CUDA;
    }
    cached = reinterpret_cast<EncodeTiledFn>(sym);
  }
  *fn = cached;
  return B200NA_OK;
}

// Bytes per element and tensor-map data type of an operand dtype code (0 = not a tensor-core type).
int elem_bytes_of(int dtype) {
  return (dtype == B200NA_F16 || dtype == B200NA_BF16) ? 2
         : (dtype == B200NA_E4M3 || dtype == B200NA_E5M2) ? 1 : 0;
}
CUtensorMapDataType tma_type_of(int dtype) {
  return dtype == B200NA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
         : dtype == B200NA_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
}

// Tensor map over a heads-last [Bp, S, H, D] tensor; box = 128 bytes of the head dim (64 16-bit or
// 128 8-bit elements) x 1 (h) x 128 (s) x 1.
int make_tensor_map(CUtensorMap* tm, const void* ptr, int dtype, int Bp, int S, int H, int D) {
  EncodeTiledFn enc = nullptr;
  int rc = get_encode_fn(&enc);
  if (rc != B200NA_OK) return rc;
  const cuuint64_t es = (cuuint64_t)elem_bytes_of(dtype);
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)Bp};
  const cuuint64_t strides[3] = {(cuuint64_t)D * es, (cuuint64_t)H * D * es,
                                 (cuuint64_t)S * H * D * es};
  const cuuint32_t box[4] = {(cuuint32_t)(128 / es), 1, (cuuint32_t)kKVTile, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = enc(tm, tma_type_of(dtype), 4, const_cast<void*>(ptr), dims, strides, box,
                         estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
    return B200NA_ERR_CUDA;
  }
  return B200NA_OK;
}

// Tensor map over the caller's heads-last [B, X0, X1, X2, H, D] tensor, seen as the 5-D array
// (H*D, X0, X1, X2, B) - axis 0 right after the channel dimension, so that a box lands in
// shared memory in the tile's own row order (axis 0 fastest). The box spans 128 bytes of one
// head's channels and tile[a] * dil[a] positions per axis, traversed with element stride dil[a]:
// it picks the tile's tokens of one dilation group; positions past an extent read as zeros.
int make_tensor_map_direct(CUtensorMap* tm, const void* ptr, int dtype, int B, const int* X,
                           int H, int D, const int* tile, const int* dil,
                           long long token_stride = 0, int ndim_sep = 0) {
  EncodeTiledFn enc = nullptr;
  int rc = get_encode_fn(&enc);
  if (rc != B200NA_OK) return rc;
  const cuuint64_t es = (cuuint64_t)elem_bytes_of(dtype);
  if (ndim_sep > 0) {
    // Head dim below the kernel's: the head becomes an axis of its own, (D, H, then the ndim_sep
    // layout axes, then the batch entry), so that a 128-byte box of channels reads zeros past
    // the head dim instead of the next head. Five axes in all: three layout axes leave no room
    // for the batch axis, so that case needs B == 1.
    if (ndim_sep == 3 && B != 1) return B200NA_ERR_UNSUPPORTED;
    const cuuint64_t row = (cuuint64_t)(token_stride > 0 ? token_stride : (long long)H * D) * es;
    if (row % 16 != 0 || (D * es) % 16 != 0 || row < (cuuint64_t)H * D * es) return B200NA_ERR_ALIGNMENT;
    cuuint64_t dims[5] = {(cuuint64_t)D, (cuuint64_t)H, 1, 1, 1};
    cuuint64_t strides[4] = {(cuuint64_t)D * es, row, row, row};
    cuuint32_t box[5] = {(cuuint32_t)(128 / es), 1, 1, 1, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    // byte stride of layout axis a: row * prod(X[a+1 .. ndim_sep-1])
    cuuint64_t tokens = 1;
    for (int a = 0; a < ndim_sep; ++a) tokens *= (cuuint64_t)X[a];
    cuuint64_t below = tokens;
    for (int a = 0; a < ndim_sep; ++a) {
      below /= (cuuint64_t)X[a];
      dims[2 + a] = (cuuint64_t)X[a];
      strides[1 + a] = row * below;
      box[2 + a] = (cuuint32_t)(tile[a] * dil[a]);
      estr[2 + a] = (cuuint32_t)dil[a];
      if (box[2 + a] > 256 || estr[2 + a] > 8) return B200NA_ERR_UNSUPPORTED;
    }
    if (ndim_sep < 3) {
      dims[2 + ndim_sep] = (cuuint64_t)B;
      strides[1 + ndim_sep] = row * tokens;
    }
    for (int a = ndim_sep + 1; a < 3; ++a) strides[1 + a] = row * tokens * (cuuint64_t)B;  // extent 1
    const CUresult r = enc(tm, tma_type_of(dtype), 5, const_cast<void*>(ptr), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_last_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
      return B200NA_ERR_CUDA;
    }
    return B200NA_OK;
  }
  // bytes from one token to the next: H * D elements when the tensor is contiguous, more when it
  // is a view into a wider row (q, k or v inside a fused [.., 3, H, D] projection output)
  const cuuint64_t row = (cuuint64_t)(token_stride > 0 ? token_stride : (long long)H * D) * es;
  if (row % 16 != 0 || row < (cuuint64_t)H * D * es) return B200NA_ERR_ALIGNMENT;
  const cuuint64_t dims[5] = {(cuuint64_t)H * D, (cuuint64_t)X[0], (cuuint64_t)X[1],
                              (cuuint64_t)X[2], (cuuint64_t)B};
  const cuuint64_t strides[4] = {row * X[1] * X[2], row * X[2], row, row * X[0] * X[1] * X[2]};
  cuuint32_t box[5] = {(cuuint32_t)(128 / es), 1, 1, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  for (int a = 0; a < B200NA_MAX_DIM; ++a) {
    box[1 + a] = (cuuint32_t)(tile[a] * dil[a]);
    estr[1 + a] = (cuuint32_t)dil[a];
    if (box[1 + a] > 256 || estr[1 + a] > 8) return B200NA_ERR_UNSUPPORTED;
  }
  const CUresult r = enc(tm, tma_type_of(dtype), 5, const_cast<void*>(ptr), dims, strides, box,
                         estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
    return B200NA_ERR_CUDA;
  }
  return B200NA_OK;
}

template <int D, int kType>
const void* kernel_for_ndim(int ndim, int halves) {
  if (halves == 1) {
    if (ndim == 1) return (const void*)fna_fwd_kernel<D, kType, 1, 1>;
    if (ndim == 2) return (const void*)fna_fwd_kernel<D, kType, 2, 1>;
    return (const void*)fna_fwd_kernel<D, kType, 3, 1>;
  }
  if (ndim == 1) return (const void*)fna_fwd_kernel<D, kType, 1, 2>;
  if (ndim == 2) return (const void*)fna_fwd_kernel<D, kType, 2, 2>;
  return (const void*)fna_fwd_kernel<D, kType, 3, 2>;
}
// Built (head dim, dtype) pairs: 16-bit floats with 64 / 128, 8-bit floats with 128.
bool variant_supported(int D, int dtype) {
  if (dtype == B200NA_F16 || dtype == B200NA_BF16) return D == 64 || D == 128;
  if (dtype == B200NA_E4M3 || dtype == B200NA_E5M2) return D == 128;
  return false;
}
// Head dim of the kernel variant that takes tensors of head dim D (0: none). The reference's
// Blackwell kernels accept every multiple of 8, 16 for 8-bit floats
// (csrc/src/blackwell_fna_forward.cu:123-138, 178-191); here the missing channels of a smaller
// head dim are zeros the tensor-map boxes fill in, and the output rows keep the tensors' width.
int kernel_head_dim(int D, int dtype) {
  if (D < 8 || D > 128) return 0;
  if (dtype == B200NA_F16 || dtype == B200NA_BF16) return D % 8 != 0 ? 0 : (D <= 64 ? 64 : 128);
  if (dtype == B200NA_E4M3 || dtype == B200NA_E5M2) return D % 16 != 0 ? 0 : 128;
  return 0;
}
const void* kernel_variant(int D, int dtype, int ndim, int halves) {
  switch (dtype) {
    case B200NA_F16:
      return D == 128 ? kernel_for_ndim<128, kTyF16>(ndim, halves)
                      : kernel_for_ndim<64, kTyF16>(ndim, halves);
    case B200NA_BF16:
      return D == 128 ? kernel_for_ndim<128, kTyBf16>(ndim, halves)
                      : kernel_for_ndim<64, kTyBf16>(ndim, halves);
    case B200NA_E4M3:
      return kernel_for_ndim<128, kTyE4m3>(ndim, halves);
    default:
      return kernel_for_ndim<128, kTyE5m2>(ndim, halves);
  }
}
int smem_bytes_of(int D, int dtype, int halves) {
  if (halves == 1) {
    if (elem_bytes_of(dtype) == 1) return Smem<128, 1, 1>::kBytes;
    return D == 128 ? Smem<128, 2, 1>::kBytes : Smem<64, 2, 1>::kBytes;
  }
  if (elem_bytes_of(dtype) == 1) return Smem<128, 1, 2>::kBytes;
  return D == 128 ? Smem<128, 2, 2>::kBytes : Smem<64, 2, 2>::kBytes;
}
// threads of a CTA and CTAs per SM of the one- and two-half variants
inline int threads_of(int halves) { return (8 * halves + 2) * 32; }
inline int ctas_per_sm(int halves) { return halves == 1 ? 2 : 1; }

// shared memory of the event trace of instrumented builds (none in the product build)
#if defined(B200NA_PROFILE) && B200NA_PROFILE >= 2
constexpr int kTraceSmem = 8192;
#else
constexpr int kTraceSmem = 0;
#endif

struct DeviceState {
  bool ready = false;
  int sms = 0;
  int* status_ptr = nullptr;
  unsigned long long* counters = nullptr;  // g_work_counters on this device
  std::mutex slot_mu;
  std::unordered_map<cudaStream_t, int> stream_slot;   // counter pair of each stream seen so far
  unsigned next_graph_slot = 0;                        // captured launches take theirs in turn
};

// Per-device one-time setup: capability check, opt-in shared memory, status word address.
int device_state(DeviceState** out) {
  static std::mutex mu;
  static DeviceState states[64];
  int dev = 0;
  B200NA_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return B200NA_ERR_DEVICE;
  std::lock_guard<std::mutex> lk(mu);
  DeviceState& st = states[dev];
  if (!st.ready) {
    int major = 0;
    B200NA_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) return B200NA_ERR_DEVICE;
    B200NA_CUDA_TRY(cudaDeviceGetAttribute(&st.sms, cudaDevAttrMultiProcessorCount, dev));
    const int dtypes[4] = {B200NA_F16, B200NA_BF16, B200NA_E4M3, B200NA_E5M2};
    for (int t = 0; t < 4; ++t)
      for (int D = 64; D <= 128; D += 64)
        for (int nd = 1; nd <= B200NA_MAX_DIM; ++nd)
          for (int halves = 1; halves <= 2; ++halves) {
            if (!variant_supported(D, dtypes[t])) continue;
            const void* fn = kernel_variant(D, dtypes[t], nd, halves);
            B200NA_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 smem_bytes_of(D, dtypes[t], halves) + kTraceSmem));
            cudaFuncAttributes fa;
            B200NA_CUDA_TRY(cudaFuncGetAttributes(&fa, fn));
            // the CTAs of an SM must fit the register file
            if (fa.numRegs * threads_of(halves) * ctas_per_sm(halves) > 65536)
              return B200NA_ERR_UNSUPPORTED;
          }
    void* sp = nullptr;
    B200NA_CUDA_TRY(cudaGetSymbolAddress(&sp, g_status_word));
    st.status_ptr = reinterpret_cast<int*>(sp);
    B200NA_CUDA_TRY(cudaMemset(st.status_ptr, 0, sizeof(int)));
    B200NA_CUDA_TRY(cudaGetSymbolAddress(&sp, g_work_counters));
    st.counters = reinterpret_cast<unsigned long long*>(sp);
    B200NA_CUDA_TRY(cudaMemset(st.counters, 0, sizeof(unsigned long long) * kCounterSlots * 2));
    st.ready = true;
  }
  *out = &st;
  return B200NA_OK;
}

#ifdef B200NA_PROFILE
long long* g_prof_buffer = nullptr;
#endif
#ifdef B200NA_TEST_HOOKS
int g_test_withhold = 0;
#endif

int launch_fna(const void* q, const void* k, const void* v, FnaParams& p, int D, int dtype,
               cudaStream_t stream, const void* add_k = nullptr, const void* add_v = nullptr) {
  DeviceState* st = nullptr;
  int rc = device_state(&st);
  if (rc != B200NA_OK) return rc;
  const uintptr_t al = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                       reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(p.o);
  if (al % 16 != 0) return B200NA_ERR_ALIGNMENT;
  const int Dk = kernel_head_dim(D, dtype);   // D is the tensors' head dim, Dk the kernel's
  if (Dk == 0) return B200NA_ERR_UNSUPPORTED;
  // the 3-D kernel keeps a row's window bounds as 16-bit halves of one register per axis
  if (p.ndim == 3)
    for (int a = 0; a < 3; ++a)
      if (p.X[a] >= 65536) return B200NA_ERR_UNSUPPORTED;
  p.d_real = D;
  p.sep_heads = (p.direct && D != Dk) ? 1 : 0;
  CUtensorMap tq, tk, tv;
  if (p.direct) {
    int half_tile[B200NA_MAX_DIM];
    for (int a = 0; a < B200NA_MAX_DIM; ++a)
      half_tile[a] = (a == p.half_axis && p.halves == 2) ? p.Tq[a] / 2 : p.Tq[a];
    const int B = p.Bp / p.G;
    const int sep = p.sep_heads ? p.ndim : 0;
    if ((rc = make_tensor_map_direct(&tq, q, dtype, B, p.o_ext, p.Hq, D, half_tile, p.dil, p.tok_stride[0], sep)) != B200NA_OK) return rc;
    if ((rc = make_tensor_map_direct(&tk, k, dtype, B, p.kv_ext, p.Hkv, D, p.Tkv, p.dil, p.tok_stride[1], sep)) != B200NA_OK) return rc;
    if ((rc = make_tensor_map_direct(&tv, v, dtype, B, p.kv_ext, p.Hkv, D, p.Tkv, p.dil, p.tok_stride[2], sep)) != B200NA_OK) return rc;
  } else {
    if ((rc = make_tensor_map(&tq, q, dtype, p.Bp, p.Sq, p.Hq, D)) != B200NA_OK) return rc;
    if ((rc = make_tensor_map(&tk, k, dtype, p.Bp, p.Skv, p.Hkv, D)) != B200NA_OK) return rc;
    if ((rc = make_tensor_map(&tv, v, dtype, p.Bp, p.Skv, p.Hkv, D)) != B200NA_OK) return rc;
  }
  // extra key/value tokens [B, n_extra, Hkv, D]; without them the maps alias K/V and are unused
  CUtensorMap tek = tk, tev = tv;
  if (p.n_extra > 0) {
    if (!add_k || !add_v) return B200NA_ERR_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(add_k) | reinterpret_cast<uintptr_t>(add_v)) % 16 != 0)
      return B200NA_ERR_ALIGNMENT;
    if ((rc = make_tensor_map(&tek, add_k, dtype, p.Bp / p.G, p.n_extra, p.Hkv, D)) != B200NA_OK) return rc;
    if ((rc = make_tensor_map(&tev, add_v, dtype, p.Bp / p.G, p.n_extra, p.Hkv, D)) != B200NA_OK) return rc;
  }
  p.extra_tiles = (p.n_extra + kKVTile - 1) / kKVTile;
  p.status = st->status_ptr;
  if ((rc = fna_work_counters(&p.work, stream)) != B200NA_OK) return rc;
#ifdef B200NA_PROFILE
  p.prof = g_prof_buffer;
#endif
#ifdef B200NA_TEST_HOOKS
  p.test_withhold = g_test_withhold;
#endif
  p.total_work = (long long)p.n_qtiles * p.Hq * p.Bp;
  if (p.total_work == 0) return B200NA_OK;
  const long long slots = (long long)st->sms * ctas_per_sm(p.halves);
  const int grid = (int)(p.total_work < slots ? p.total_work : slots);
  const void* fn = kernel_variant(Dk, dtype, p.ndim, p.halves);
  void* args[] = {(void*)&tq, (void*)&tk, (void*)&tv, (void*)&tek, (void*)&tev, (void*)&p};
  constexpr int kExtraSmem = kTraceSmem;
  B200NA_CUDA_TRY(cudaLaunchKernel(fn, dim3(grid), dim3(threads_of(p.halves)), args,
                                   smem_bytes_of(Dk, dtype, p.halves) + kExtraSmem,
                                   stream));
  return B200NA_OK;
}

}  // namespace
}  // namespace b200na

namespace b200na {
int fna_make_tensor_map_direct(CUtensorMap* tm, const void* ptr, int dtype, int B, const int* X,
                               int H, int D, const int* tile, const int* dil) {
  return make_tensor_map_direct(tm, ptr, dtype, B, X, H, D, tile, dil);
}
int fna_work_counters(unsigned long long** pair, cudaStream_t stream) {
  DeviceState* st = nullptr;
  const int rc = device_state(&st);
  if (rc != B200NA_OK) return rc;
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  B200NA_CUDA_TRY(cudaStreamIsCapturing(stream, &capturing));
  std::lock_guard<std::mutex> lk(st->slot_mu);
  int slot;
  if (capturing != cudaStreamCaptureStatusNone) {
    // a graph node keeps its pair for every replay; nodes get distinct pairs until the pool of
    // kCounterSlots - kStreamSlots has gone round once
    slot = kStreamSlots + (int)(st->next_graph_slot++ % (unsigned)(kCounterSlots - kStreamSlots));
  } else {
    auto it = st->stream_slot.find(stream);
    if (it == st->stream_slot.end()) {
      // more streams than pairs: later streams share by position (not expected in practice)
      const int fresh = (int)(st->stream_slot.size() % (size_t)kStreamSlots);
      it = st->stream_slot.emplace(stream, fresh).first;
    }
    slot = it->second;
  }
  *pair = st->counters + 2 * slot;
  return B200NA_OK;
}
int fna_device_info(int* sms, int** status_ptr) {
  DeviceState* st = nullptr;
  const int rc = device_state(&st);
  if (rc != B200NA_OK) return rc;
  *sms = st->sms;
  *status_ptr = st->status_ptr;
  return B200NA_OK;
}
}  // namespace b200na

namespace b200na {
namespace {
int fna_forward_impl(
    const void* q, const void* k, const void* v, void* o, float* lse, int ndim,
    const int* qkv_shape, const int* q_shape, const int* kv_shape, const int* kernel,
    const int* stride, const int* dilation, const int* causal, const int* q_tile,
    const int* kv_tile, int Bp, int Hq, int Hkv, int D, int dtype, float scale,
    const int* q_origin, const int* q_extent, const int* kv_origin, const void* add_k,
    const void* add_v, int n_extra, b200na_stream_t stream) {
  if (n_extra < 0) return B200NA_ERR_INVALID_ARGUMENT;
  if (!q || !k || !v || !o || !qkv_shape || !q_shape || !kv_shape || !kernel || !q_tile || !kv_tile)
    return B200NA_ERR_INVALID_ARGUMENT;
  if (Bp < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv != 0) return B200NA_ERR_INVALID_ARGUMENT;
  if (kernel_head_dim(D, dtype) == 0) return B200NA_ERR_UNSUPPORTED;
  if (!(scale > 0.f)) return B200NA_ERR_INVALID_ARGUMENT;
  const bool sharded = q_origin != nullptr || kv_origin != nullptr || q_extent != nullptr;
  if (sharded && !(q_origin && kv_origin && q_extent)) return B200NA_ERR_INVALID_ARGUMENT;
  NaAxes ax;
  int rc = fill_axes(ax, ndim, qkv_shape, kernel, stride, dilation, causal);
  if (rc != B200NA_OK) return rc;
  FnaParams p;
  memset(&p, 0, sizeof(p));
  p.ndim = ndim;
  p.G = 1;
  long long sq = 1, skv = 1, tq = 1, tkv = 1;
  for (int a = 0; a < B200NA_MAX_DIM; ++a) {
    const bool on = a < ndim;
    p.X[a] = ax.shape[a]; p.kernel[a] = ax.kernel[a]; p.stride[a] = ax.stride[a];
    p.dil[a] = ax.dilation[a]; p.causal[a] = ax.causal[a];
    p.Tq[a] = on ? q_tile[a] : 1;
    p.Tkv[a] = on ? kv_tile[a] : 1;
    p.tkv_shift[a] = -1;
    for (int sh = 0; sh < 8; ++sh)
      if (p.Tkv[a] == (1 << sh)) p.tkv_shift[a] = sh;
    const int qs = on ? q_shape[a] : 1, ks = on ? kv_shape[a] : 1;
    if (p.Tq[a] < 1 || p.Tkv[a] < 1 || qs < 1 || ks < 1) return B200NA_ERR_INVALID_ARGUMENT;
    if (qs % p.Tq[a] != 0 || ks % p.Tkv[a] != 0) return B200NA_ERR_INVALID_ARGUMENT;
    const int need = (p.X[a] + p.dil[a] - 1) / p.dil[a];  // largest dilation group
    if (sharded) {
      // a local slab of an undilated layout: [origin, origin + extent) must lie inside it
      if (p.dil[a] != 1) return B200NA_ERR_UNSUPPORTED;
      p.q_org[a] = on ? q_origin[a] : 0;
      p.kv_org[a] = on ? kv_origin[a] : 0;
      p.q_len[a] = on ? q_extent[a] : 1;
      if (p.q_org[a] < 0 || p.kv_org[a] < 0 || p.q_len[a] < 1 || p.q_len[a] > qs ||
          p.q_org[a] + p.q_len[a] > p.X[a] || p.kv_org[a] >= p.X[a])
        return B200NA_ERR_INVALID_ARGUMENT;
      // the key/value slab must hold every key the local queries' windows reach
      const int first = p.q_org[a], last = p.q_org[a] + p.q_len[a] - 1;
      const int lo = win_start(first, p.kernel[a], p.stride[a], p.X[a], p.causal[a]);
      const int st_last = win_start(last, p.kernel[a], p.stride[a], p.X[a], p.causal[a]);
      const int hi = win_end(last, st_last, p.kernel[a], p.X[a], p.causal[a]);
      if (lo < p.kv_org[a] || hi > p.kv_org[a] + ks) return B200NA_ERR_INVALID_ARGUMENT;
    } else {
      // padded per-group extents must cover the largest dilation group
      if (qs < need || ks < need) return B200NA_ERR_INVALID_ARGUMENT;
      p.q_org[a] = 0;
      p.kv_org[a] = 0;
      p.q_len[a] = need;
    }
    p.Rq[a] = qs / p.Tq[a];
    p.Rkv[a] = ks / p.Tkv[a];
    p.G *= p.dil[a];
    sq *= qs; skv *= ks; tq *= p.Tq[a]; tkv *= p.Tkv[a];
  }
  if ((tq != kQTile && tq != kHalf) || tkv != kKVTile) return B200NA_ERR_INVALID_ARGUMENT;
  p.halves = (int)(tq / kHalf);
  if (Bp % p.G != 0) return B200NA_ERR_INVALID_ARGUMENT;
  if (sq > 0x7fffffffLL || skv > 0x7fffffffLL) return B200NA_ERR_UNSUPPORTED;
  p.dense = 0;
  p.Bp = Bp; p.Hq = Hq; p.Hkv = Hkv;
  p.Sq = (int)sq; p.Skv = (int)skv;
  p.n_qtiles = (int)(sq / tq);
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.o = o;
  p.lse = lse;
  p.n_extra = n_extra;
  return launch_fna(q, k, v, p, D, dtype, reinterpret_cast<cudaStream_t>(stream), add_k, add_v);
}
}  // namespace
}  // namespace b200na

namespace b200na {
namespace {
// Neighborhood attention straight on the caller's [B, *X, H, D] tensors: the tile gathers that
// the token permutation would do are done by the tensor maps, and O / LSE rows are written to
// their final place.
int fna_direct_impl(const void* q, const void* k, const void* v, void* o, float* lse, int ndim,
                    const int* shape, const int* kernel, const int* stride, const int* dilation,
                    const int* causal, const int* q_tile, const int* kv_tile, int B, int Hq,
                    int Hkv, int D, int dtype, float scale, const void* add_k, const void* add_v,
                    int n_extra, const long long* token_strides, b200na_stream_t stream,
                    const int* q_origin = nullptr, const int* q_extent = nullptr,
                    const int* kv_origin = nullptr, const int* kv_extent = nullptr, int clip = 0) {
  if (!q || !k || !v || !o || !shape || !kernel || !q_tile || !kv_tile)
    return B200NA_ERR_INVALID_ARGUMENT;
  // slabs: q / o / lse hold layout coordinates [q_origin, q_origin + q_extent), k / v hold
  // [kv_origin, kv_origin + kv_extent); window arithmetic stays in layout coordinates
  const bool sharded = q_origin || q_extent || kv_origin || kv_extent;
  if (sharded && !(q_origin && q_extent && kv_origin && kv_extent)) return B200NA_ERR_INVALID_ARGUMENT;
  if (clip && !sharded) return B200NA_ERR_INVALID_ARGUMENT;
  if (n_extra < 0 || (n_extra > 0 && (!add_k || !add_v))) return B200NA_ERR_INVALID_ARGUMENT;
  if (B < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv != 0) return B200NA_ERR_INVALID_ARGUMENT;
  if (kernel_head_dim(D, dtype) == 0) return B200NA_ERR_UNSUPPORTED;
  if (!(scale > 0.f)) return B200NA_ERR_INVALID_ARGUMENT;
  NaAxes ax;
  int rc = fill_axes(ax, ndim, shape, kernel, stride, dilation, causal);
  if (rc != B200NA_OK) return rc;
  FnaParams p;
  memset(&p, 0, sizeof(p));
  p.ndim = ndim;
  p.G = 1;
  p.direct = 1;
  p.half_axis = 0;
  for (int i = 0; i < 3; ++i) p.tok_stride[i] = token_strides ? token_strides[i] : 0;
  long long sq = 1, skv = 1, tq = 1, tkv = 1, tokens = 1;
  for (int a = 0; a < B200NA_MAX_DIM; ++a) {
    const bool on = a < ndim;
    p.X[a] = ax.shape[a]; p.kernel[a] = ax.kernel[a]; p.stride[a] = ax.stride[a];
    p.dil[a] = ax.dilation[a]; p.causal[a] = ax.causal[a];
    p.Tq[a] = on ? q_tile[a] : 1;
    p.Tkv[a] = on ? kv_tile[a] : 1;
    if (p.Tq[a] < 1 || p.Tkv[a] < 1) return B200NA_ERR_INVALID_ARGUMENT;
    if (p.Tq[a] > 1) p.half_axis = a;  // the slowest-varying axis of the tile's row order
    p.tkv_shift[a] = -1;
    for (int sh = 0; sh < 8; ++sh)
      if (p.Tkv[a] == (1 << sh)) p.tkv_shift[a] = sh;
    int need = (p.X[a] + p.dil[a] - 1) / p.dil[a];  // largest dilation group
    p.q_org[a] = 0;
    p.kv_org[a] = 0;
    p.o_ext[a] = p.X[a];
    p.kv_ext[a] = p.X[a];
    p.clip_lo[a] = 0;
    p.clip_hi[a] = p.X[a];
    if (sharded) {
      if (p.dil[a] != 1) return B200NA_ERR_UNSUPPORTED;
      p.q_org[a] = on ? q_origin[a] : 0;
      p.kv_org[a] = on ? kv_origin[a] : 0;
      p.o_ext[a] = on ? q_extent[a] : 1;
      p.kv_ext[a] = on ? kv_extent[a] : 1;
      if (p.q_org[a] < 0 || p.kv_org[a] < 0 || p.o_ext[a] < 1 || p.kv_ext[a] < 1 ||
          p.q_org[a] + p.o_ext[a] > p.X[a] || p.kv_org[a] + p.kv_ext[a] > p.X[a])
        return B200NA_ERR_INVALID_ARGUMENT;
      need = p.o_ext[a];
      const int first = p.q_org[a], last = p.q_org[a] + p.o_ext[a] - 1;
      const int lo = win_start(first, p.kernel[a], p.stride[a], p.X[a], p.causal[a]);
      const int st_last = win_start(last, p.kernel[a], p.stride[a], p.X[a], p.causal[a]);
      const int hi = win_end(last, st_last, p.kernel[a], p.X[a], p.causal[a]);
      if (clip) {
        p.clip_lo[a] = p.kv_org[a];
        p.clip_hi[a] = p.kv_org[a] + p.kv_ext[a];
      } else if (lo < p.kv_org[a] || hi > p.kv_org[a] + p.kv_ext[a]) {
        // the key/value slab must hold every key the local queries' windows reach
        return B200NA_ERR_INVALID_ARGUMENT;
      }
    }
    p.q_len[a] = need;
    p.Rq[a] = (need + p.Tq[a] - 1) / p.Tq[a];
    p.Rkv[a] = (need + p.Tkv[a] - 1) / p.Tkv[a];
    p.G *= p.dil[a];
    sq *= (long long)p.Rq[a] * p.Tq[a];
    skv *= (long long)p.Rkv[a] * p.Tkv[a];
    tq *= p.Tq[a]; tkv *= p.Tkv[a];
    tokens *= p.X[a];
  }
  if ((tq != kQTile && tq != kHalf) || tkv != kKVTile) return B200NA_ERR_INVALID_ARGUMENT;
  p.halves = (int)(tq / kHalf);
  // a 256-token query tile is fetched as two boxes, split along its last non-unit axis
  if (p.halves == 2 && p.Tq[p.half_axis] % 2 != 0) return B200NA_ERR_UNSUPPORTED;
  if (sq > 0x7fffffffLL || skv > 0x7fffffffLL || tokens * B > 0x7fffffffLL ||
      (long long)Hq * D > 0x7fffffffLL)
    return B200NA_ERR_UNSUPPORTED;
  p.dense = 0;
  p.clip = clip ? 1 : 0;
  p.Bp = B * p.G; p.Hq = Hq; p.Hkv = Hkv;
  p.Sq = (int)sq; p.Skv = (int)skv;
  p.n_qtiles = (int)(sq / tq);
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.o = o;
  p.lse = lse;
  p.n_extra = n_extra;
  return launch_fna(q, k, v, p, D, dtype, reinterpret_cast<cudaStream_t>(stream), add_k, add_v);
}
}  // namespace
}  // namespace b200na

extern "C" B200NA_API int b200na_na_forward_direct(
    const void* q, const void* k, const void* v, const void* add_k, const void* add_v,
    int n_extra, void* o, float* lse, int ndim, const int* shape, const int* kernel,
    const int* stride, const int* dilation, const int* causal, const int* q_tile,
    const int* kv_tile, int B, int Hq, int Hkv, int D, int dtype, float scale,
    b200na_stream_t stream) {
  return b200na::fna_direct_impl(q, k, v, o, lse, ndim, shape, kernel, stride, dilation, causal,
                                 q_tile, kv_tile, B, Hq, Hkv, D, dtype, scale, add_k, add_v,
                                 n_extra, nullptr, stream);
}

extern "C" B200NA_API int b200na_na_forward_direct_strided(
    const void* q, const void* k, const void* v, const void* add_k, const void* add_v,
    int n_extra, void* o, float* lse, int ndim, const int* shape, const int* kernel,
    const int* stride, const int* dilation, const int* causal, const int* q_tile,
    const int* kv_tile, int B, int Hq, int Hkv, int D, int dtype, float scale,
    long long q_token_stride, long long k_token_stride, long long v_token_stride,
    b200na_stream_t stream) {
  const long long ts[3] = {q_token_stride, k_token_stride, v_token_stride};
  return b200na::fna_direct_impl(q, k, v, o, lse, ndim, shape, kernel, stride, dilation, causal,
                                 q_tile, kv_tile, B, Hq, Hkv, D, dtype, scale, add_k, add_v,
                                 n_extra, ts, stream);
}

extern "C" B200NA_API int b200na_na_forward_direct_sharded(
    const void* q, const void* k, const void* v, const void* add_k, const void* add_v,
    int n_extra, void* o, float* lse, int ndim, const int* global_shape, const int* kernel,
    const int* stride, const int* causal, const int* q_tile, const int* kv_tile,
    const int* q_origin, const int* q_extent, const int* kv_origin, const int* kv_extent,
    int clip_to_kv, int B, int Hq, int Hkv, int D, int dtype, float scale,
    b200na_stream_t stream) {
  if (!q_origin || !q_extent || !kv_origin || !kv_extent) return B200NA_ERR_INVALID_ARGUMENT;
  return b200na::fna_direct_impl(q, k, v, o, lse, ndim, global_shape, kernel, stride, nullptr,
                                 causal, q_tile, kv_tile, B, Hq, Hkv, D, dtype, scale, add_k,
                                 add_v, n_extra, nullptr, stream, q_origin, q_extent, kv_origin,
                                 kv_extent, clip_to_kv);
}

extern "C" B200NA_API int b200na_fna_forward_sharded(
    const void* q, const void* k, const void* v, void* o, float* lse, int ndim,
    const int* qkv_shape, const int* q_shape, const int* kv_shape, const int* kernel,
    const int* stride, const int* dilation, const int* causal, const int* q_tile,
    const int* kv_tile, int Bp, int Hq, int Hkv, int D, int dtype, float scale,
    const int* q_origin, const int* q_extent, const int* kv_origin, b200na_stream_t stream) {
  return b200na::fna_forward_impl(q, k, v, o, lse, ndim, qkv_shape, q_shape, kv_shape, kernel,
                                  stride, dilation, causal, q_tile, kv_tile, Bp, Hq, Hkv, D, dtype,
                                  scale, q_origin, q_extent, kv_origin, nullptr, nullptr, 0, stream);
}

extern "C" B200NA_API int b200na_fna_forward_extra_kv(
    const void* q, const void* k, const void* v, const void* add_k, const void* add_v,
    int n_extra, void* o, float* lse, int ndim, const int* qkv_shape, const int* q_shape,
    const int* kv_shape, const int* kernel, const int* stride, const int* dilation,
    const int* causal, const int* q_tile, const int* kv_tile, int Bp, int Hq, int Hkv, int D,
    int dtype, float scale, b200na_stream_t stream) {
  if (n_extra > 0 && (!add_k || !add_v)) return B200NA_ERR_INVALID_ARGUMENT;
  return b200na::fna_forward_impl(q, k, v, o, lse, ndim, qkv_shape, q_shape, kv_shape, kernel,
                                  stride, dilation, causal, q_tile, kv_tile, Bp, Hq, Hkv, D, dtype,
                                  scale, nullptr, nullptr, nullptr, add_k, add_v, n_extra, stream);
}

extern "C" B200NA_API int b200na_fna_forward(const void* q, const void* k, const void* v, void* o,
                                             float* lse, int ndim, const int* qkv_shape,
                                             const int* q_shape, const int* kv_shape,
                                             const int* kernel, const int* stride,
                                             const int* dilation, const int* causal,
                                             const int* q_tile, const int* kv_tile, int Bp, int Hq,
                                             int Hkv, int D, int dtype, float scale,
                                             b200na_stream_t stream) {
  return b200na::fna_forward_impl(q, k, v, o, lse, ndim, qkv_shape, q_shape, kv_shape, kernel,
                                  stride, dilation, causal, q_tile, kv_tile, Bp, Hq, Hkv, D, dtype,
                                  scale, nullptr, nullptr, nullptr, nullptr, nullptr, 0, stream);
}

extern "C" B200NA_API int b200na_fmha_forward(const void* q, const void* k, const void* v, void* o, float* lse,
                                   int B, int Nq, int Nk, int Hq, int Hkv, int D, int dtype,
                                   float scale, int causal, b200na_stream_t stream) {
  using namespace b200na;
  if (!q || !k || !v || !o) return B200NA_ERR_INVALID_ARGUMENT;
  if (B < 1 || Nq < 1 || Nk < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv != 0)
    return B200NA_ERR_INVALID_ARGUMENT;
  if (causal && Nq != Nk) return B200NA_ERR_INVALID_ARGUMENT;
  if (dtype != B200NA_F32 && dtype != B200NA_F16 && dtype != B200NA_BF16 &&
      dtype != B200NA_E4M3 && dtype != B200NA_E5M2)
    return B200NA_ERR_INVALID_ARGUMENT;
  if (elem_bytes_of(dtype) == 1 && kernel_head_dim(D, dtype) == 0) return B200NA_ERR_UNSUPPORTED;
  if (kernel_head_dim(D, dtype) == 0 || !(scale > 0.f))
    return simt_dense_forward(q, k, v, o, lse, B, Nq, Nk, Hq, Hkv, D, dtype, scale, causal,
                              reinterpret_cast<cudaStream_t>(stream));
  FnaParams p;
  memset(&p, 0, sizeof(p));
  p.ndim = 1;
  p.G = 1;
  for (int a = 0; a < B200NA_MAX_DIM; ++a) {
    p.X[a] = 1; p.kernel[a] = 1; p.stride[a] = 1; p.dil[a] = 1; p.causal[a] = 0;
    p.Tq[a] = 1; p.Tkv[a] = 1; p.Rq[a] = 1; p.Rkv[a] = 1; p.q_len[a] = 1; p.tkv_shift[a] = 0;
  }
  p.X[0] = Nk;
  p.q_len[0] = Nq;
  p.causal[0] = causal ? 1 : 0;
  p.Tq[0] = kQTile;
  p.Tkv[0] = kKVTile;
  p.tkv_shift[0] = 7;
  p.n_qtiles = (Nq + kQTile - 1) / kQTile;
  p.Rq[0] = p.n_qtiles;
  p.Rkv[0] = (Nk + kKVTile - 1) / kKVTile;
  p.dense = 1;
  p.halves = 2;
  p.Bp = B; p.Hq = Hq; p.Hkv = Hkv;
  p.Sq = Nq; p.Skv = Nk;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.o = o;
  p.lse = lse;
  return launch_fna(q, k, v, p, D, dtype, reinterpret_cast<cudaStream_t>(stream));
}

#ifdef B200NA_PROFILE
// Instrumented builds only: device buffer of [grid][4][8] int64 cycle counters.
extern "C" B200NA_API void b200na_debug_set_prof(void* buf) {
  b200na::g_prof_buffer = reinterpret_cast<long long*>(buf);
}
#endif

#ifdef B200NA_TEST_HOOKS
// Test-hook build only (never the product library): from now on the load warp of every CTA keeps
// back the record of its n-th key/value tile, so that the wait for it expires; 0 switches it off.
extern "C" B200NA_API int b200na_test_withhold_record(int n) {
  b200na::g_test_withhold = n;
  return B200NA_OK;
}
#endif

extern "C" B200NA_API int b200na_device_status(int* status) {
  using namespace b200na;
  if (!status) return B200NA_ERR_INVALID_ARGUMENT;
  DeviceState* st = nullptr;
  int rc = device_state(&st);
  if (rc != B200NA_OK) return rc;
  B200NA_CUDA_TRY(cudaDeviceSynchronize());
  B200NA_CUDA_TRY(cudaMemcpy(status, st->status_ptr, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status != 0) {
    B200NA_CUDA_TRY(cudaMemset(st->status_ptr, 0, sizeof(int)));
    return B200NA_ERR_KERNEL_TIMEOUT;
  }
  return B200NA_OK;
}
