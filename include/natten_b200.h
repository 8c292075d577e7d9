/*
 * natten_b200 — C ABI of the B200 (sm_100a) neighborhood-attention forward path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle, launches its
 * kernels asynchronously on that stream and returns B200NA_OK or a negative error code (text via
 * b200na_strerror). The caller owns every buffer, including scratch. After the first attention
 * call on a device the library neither allocates nor frees device memory and never synchronises
 * a stream; that first call does a one-time set-up of the device (kernel attributes, two small
 * synchronising cudaMemset calls on the library's own status word and work counters) and should
 * be made before any stream capture.
 *
 * Streams and CUDA graphs: the attention kernels hand out their work items through a pair of
 * device counters. Launches on one stream share that stream's pair (they run one after the
 * other); a launch recorded under stream capture gets a pair of its own, from a pool of 3072
 * handed out in turn, and keeps it for every replay. Any number of streams and graph replays may
 * therefore run next to each other; the limits are 1024 distinct eager streams per device and
 * 3072 captured attention launches alive at the same time (beyond them pairs are shared again,
 * and two kernels that share a pair while both are in flight compute wrong results).
 *
 * Tensor layouts are the reference's: heads-last and contiguous.
 *   token layout tensors   [B, X0(, X1(, X2)), H, D]
 *   permuted ("tiled")     [B * prod(dilation), S, H, D],  S = prod(R_a * T_a),
 *                          R_a = ceil(ceil(X_a / T_a) / d_a)
 *   logsumexp              same without the trailing D, always fp32
 * Axis arrays (shape, tile, kernel, ...) have `ndim` entries, axis 0 first, exactly as the
 * reference's Python tuples.
 */
#ifndef NATTEN_B200_H_
#define NATTEN_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200NA_OK 0
#define B200NA_ERR_INVALID_ARGUMENT (-1) /* a shape / size / flag violates the documented contract */
#define B200NA_ERR_UNSUPPORTED (-2)      /* valid in the reference, not implemented here          */
#define B200NA_ERR_ALIGNMENT (-3)        /* a pointer or row pitch is not aligned as required     */
#define B200NA_ERR_CUDA (-4)             /* a CUDA runtime / driver call failed (see last error)  */
#define B200NA_ERR_DEVICE (-5)           /* current device is not compute capability 10.x         */
#define B200NA_ERR_KERNEL_TIMEOUT (-6)   /* a bounded device-side wait expired (see device_status) */
#define B200NA_ERR_WORKSPACE_LIMIT (-7)  /* problem needs more scratch than the built-in array holds */

/* Element types of Q/K/V/O. */
#define B200NA_F32 0
#define B200NA_F16 1
#define B200NA_BF16 2
#define B200NA_E4M3 3 /* 8-bit float, 4 exponent bits (torch.float8_e4m3fn) */
#define B200NA_E5M2 4 /* 8-bit float, 5 exponent bits (torch.float8_e5m2) */

/* Exported-symbol marker (the library is built with hidden visibility by default). */
#if defined(__GNUC__)
#define B200NA_API __attribute__((visibility("default")))
#else
#define B200NA_API
#endif

/* Opaque CUDA stream handle (a cudaStream_t / CUstream passed as a pointer; NULL = default). */
typedef void* b200na_stream_t;

/* Human-readable text for an error code returned by this library. Never NULL. */
B200NA_API const char* b200na_strerror(int code);

/* Library version (major * 10000 + minor * 100 + patch). */
B200NA_API int b200na_version(void);

/*
 * Token permute: replaces natten::token_permute_{1,2,3}d
 * (reference: csrc/include/natten/token_permute.h:34-52, csrc/src/token_permute.cu:61-266,
 * kernel csrc/include/natten/cuda/tokperm/token_permute_kernel.cuh:159-378).
 *   out[b*G + lin(g), lin(r)*|T| + lin(t), h, :] = in[b, (r_a*T_a + t_a)*d_a + g_a ..., h, :]
 * and zero where a source coordinate is outside `shape` (padding). lin() is colexicographic
 * (axis 0 fastest) when flip != 0 — what the attention kernels expect — else last axis fastest.
 * in:  [B, *shape, H, D]; out: [B*prod(dilation), prod(R_a*tile_a), H, D]; bit copy of
 * elem_bytes-wide elements (1, 2, 4 or 8). `in` and `out` must not overlap.
 */
B200NA_API int b200na_token_permute(const void* in, void* out, int ndim, const int* shape, const int* tile,
                         const int* dilation, int B, int H, int D, int elem_bytes, int flip,
                         b200na_stream_t stream);

/*
 * Token unpermute: replaces natten::token_unpermute_{1,2,3}d
 * (reference: csrc/include/natten/token_permute.h:54-74, csrc/src/token_unpermute.cu).
 * Exact inverse of b200na_token_permute restricted to valid coordinates (padding dropped).
 * in: [B*prod(dilation), prod(R_a*tile_a), H, D]; out: [B, *shape, H, D].
 */
B200NA_API int b200na_token_unpermute(const void* in, void* out, int ndim, const int* shape, const int* tile,
                           const int* dilation, int B, int H, int D, int elem_bytes, int flip,
                           b200na_stream_t stream);

/*
 * Fused neighborhood attention forward on token-permuted operands: replaces
 * natten::blackwell_na{1,2,3}d_forward (reference: csrc/include/natten/blackwell_fna.h:36-88,
 * csrc/src/blackwell_fna_forward.cu:57-267).
 *   q:   [Bp, Sq, Hq, D]   permuted with q_tile;  k, v: [Bp, Skv, Hkv, D] permuted with kv_tile
 *   o:   [Bp, Sq, Hq, D]   same element type as q
 *   lse: [Bp, Sq, Hq] fp32 natural-log logsumexp of the scaled logits; may be NULL
 *   Bp = batch * prod(dilation); dilation group of a slice = Bp index mod prod(dilation),
 *   decoded colexicographically (axis 0 fastest).
 *   qkv_shape: original token layout X; q_shape / kv_shape: padded per-group extents R_a*T_a
 *   (prod = Sq / Skv). prod(q_tile) must be 256 or 128 and prod(kv_tile) 128; tiles divide the
 *   shapes. A 256-token query tile runs one CTA per SM with two 128-row halves that share every
 *   key/value tile; a 128-token one runs two CTAs per SM, each walking the key/value box of its
 *   own queries - fewer tile products when windows are small, twice the tile loads per row.
 *   kernel/stride/dilation/causal: the reference's kernel_size / stride / dilation / is_causal.
 *   dtype: B200NA_F16 or B200NA_BF16 with D a multiple of 8, or B200NA_E4M3 / B200NA_E5M2 with D
 *   a multiple of 16 (the reference's rules, csrc/src/blackwell_fna_forward.cu:123-138, 178-191;
 *   8-bit: fp32 accumulation and softmax, P rounded to e4m3 before P.V, O in the operand type),
 *   8 <= D <= 128. The kernels are built for 64 and 128 channels (8-bit: 128); the channels a
 *   smaller head dim lacks are zeros the tensor-map boxes fill in, and O rows are D wide.
 *   Hq % Hkv == 0. scale multiplies q.k. With ndim = 3 every axis of qkv_shape must be
 *   shorter than 65536 tokens (B200NA_ERR_UNSUPPORTED otherwise; b200na_na_forward_simt has no
 *   such limit).
 * Rows of o/lse that correspond to padding tokens are left unspecified.
 */
B200NA_API int b200na_fna_forward(const void* q, const void* k, const void* v, void* o, float* lse, int ndim,
                       const int* qkv_shape, const int* q_shape, const int* kv_shape,
                       const int* kernel, const int* stride, const int* dilation,
                       const int* causal, const int* q_tile, const int* kv_tile, int Bp, int Hq,
                       int Hkv, int D, int dtype, float scale, b200na_stream_t stream);

/*
 * b200na_fna_forward with extra key/value tokens that EVERY query attends in addition to its
 * neighborhood (cross-attention context), fused into the same kernel and the same softmax. The
 * reference runs a second attention over the extra tokens and merges the two results
 * (src/natten/functional.py:524-559); the semantics are those of its reference mask
 * (csrc/include/natten/cuda/reference/mask.hpp:314-318). The extra tiles ride the same K/V ring
 * as the neighborhood tiles, so the dense-attention pass, the merge pass and their traffic vanish.
 *   add_k, add_v: [Bp / prod(dilation), n_extra, Hkv, D] in the ORIGINAL batch order (not
 *   permuted, shared by the dilation groups of a batch entry); n_extra need not be a tile multiple.
 */
B200NA_API int b200na_fna_forward_extra_kv(
    const void* q, const void* k, const void* v, const void* add_k, const void* add_v,
    int n_extra, void* o, float* lse, int ndim, const int* qkv_shape, const int* q_shape,
    const int* kv_shape, const int* kernel, const int* stride, const int* dilation,
    const int* causal, const int* q_tile, const int* kv_tile, int Bp, int Hq, int Hkv, int D,
    int dtype, float scale, b200na_stream_t stream);

/*
 * Neighborhood attention forward on the caller's own tensors - q/o [B, *shape, Hq, D], k/v
 * [B, *shape, Hkv, D], lse [B, *shape, Hq] fp32 (nullable), heads last, contiguous - in ONE
 * kernel and with no scratch memory. It replaces the whole flow of the reference's backend
 * (src/natten/backends/blackwell_fna.py:111-165: token_permute of Q, K, V -> FNA kernel ->
 * token_unpermute of O and LSE): the tile gathers of the permutation
 * (csrc/include/natten/cuda/tokperm/token_permute_kernel.cuh:159-378), dilation included, are
 * done by the kernel's tensor-map loads, and every O / LSE row is stored at its final address.
 * Results are those of b200na_token_permute + b200na_fna_forward_extra_kv +
 * b200na_token_unpermute with the same tile shapes.
 *   q_tile / kv_tile: prod = 256 (or 128) / 128; tile[a] * dilation[a] <= 256 and dilation[a] <= 8 on
 *   every axis, otherwise B200NA_ERR_UNSUPPORTED (use the permuted path then). Also
 *   B200NA_ERR_UNSUPPORTED: a head dim other than 64 / 128 (8-bit: 128) on a 3-D layout with
 *   B > 1 (the tensor map then has no axis left for the batch entry; call per batch entry, or
 *   use the permuted path).
 *   add_k / add_v [B, n_extra, Hkv, D]: optional extra tokens every query attends (n_extra = 0
 *   and NULL for none).
 */
B200NA_API int b200na_na_forward_direct(
    const void* q, const void* k, const void* v, const void* add_k, const void* add_v,
    int n_extra, void* o, float* lse, int ndim, const int* shape, const int* kernel,
    const int* stride, const int* dilation, const int* causal, const int* q_tile,
    const int* kv_tile, int B, int Hq, int Hkv, int D, int dtype, float scale,
    b200na_stream_t stream);

/*
 * b200na_na_forward_direct for q, k, v that are VIEWS into wider token rows - typically the three
 * slices of a fused projection output [B, *shape, 3, H, D], which the reference's layers separate
 * with a permute + copy (src/natten/modules.py:104-113). `*_token_stride` is the distance between
 * consecutive tokens in elements (>= H * D, a multiple of 16 bytes; 0 = contiguous); batch entries
 * are prod(shape) tokens apart. The tensor maps absorb the stride, nothing is copied. o and lse
 * are contiguous as always.
 */
B200NA_API int b200na_na_forward_direct_strided(
    const void* q, const void* k, const void* v, const void* add_k, const void* add_v,
    int n_extra, void* o, float* lse, int ndim, const int* shape, const int* kernel,
    const int* stride, const int* dilation, const int* causal, const int* q_tile,
    const int* kv_tile, int B, int Hq, int Hkv, int D, int dtype, float scale,
    long long q_token_stride, long long k_token_stride, long long v_token_stride,
    b200na_stream_t stream);

/*
 * The same kernel on one rank's SLAB of a spatially sharded, undilated token layout. The
 * reference has no counterpart (it has no multi-GPU code); window arithmetic follows
 * csrc/include/natten/cuda/reference/mask.hpp:59-89 in layout ("global") coordinates.
 *   qkv_shape: the WHOLE token layout; q holds query coordinates [q_origin, q_origin + q_extent)
 *   per axis, padded to q_shape (tile multiples); k, v hold key coordinates
 *   [kv_origin, kv_origin + kv_shape) (padding beyond the layout is never attended).
 *   The key/value slab must contain every key the local queries' windows reach (own slab plus the
 *   halo received from neighbouring ranks); otherwise B200NA_ERR_INVALID_ARGUMENT.
 *   All dilations must be 1. Passing NULL for the three arrays is b200na_fna_forward.
 */
B200NA_API int b200na_fna_forward_sharded(
    const void* q, const void* k, const void* v, void* o, float* lse, int ndim,
    const int* qkv_shape, const int* q_shape, const int* kv_shape, const int* kernel,
    const int* stride, const int* dilation, const int* causal, const int* q_tile,
    const int* kv_tile, int Bp, int Hq, int Hkv, int D, int dtype, float scale,
    const int* q_origin, const int* q_extent, const int* kv_origin, b200na_stream_t stream);

/*
 * One rank's slab on the caller's layout, no permuted copies: q, o, lse are contiguous
 * [B, *q_extent, H, D] tensors holding layout coordinates [q_origin, q_origin + q_extent) of an
 * undilated token layout global_shape, k and v hold [kv_origin, kv_origin + kv_extent). Window
 * arithmetic stays in layout coordinates (mask.hpp:59-89); the reference has no counterpart.
 *   clip_to_kv == 0: the key/value slab must hold every key the local queries' windows reach,
 *     otherwise B200NA_ERR_INVALID_ARGUMENT.
 *   clip_to_kv != 0: partial attention over the keys that are present - every window is cut to
 *     the slab; a query none of whose keys are present gets O = 0 and LSE = -inf. Partial
 *     results over disjoint key slabs combine with b200na_merge to the full result, which lets
 *     a rank attend its own frames while the frames of other ranks are still in flight
 *     (the use the reference's merge_attentions hints at, src/natten/attn_merge.py:199-204).
 * add_k / add_v: n_extra extra key/value tokens [B, n_extra, Hkv, D] every query attends (NULL and
 * 0 for none); when partial results are merged, pass them to exactly one of the calls.
 * Also the building block for streaming a host-resident problem through the GPU along axis 0.
 */
B200NA_API int b200na_na_forward_direct_sharded(
    const void* q, const void* k, const void* v, const void* add_k, const void* add_v,
    int n_extra, void* o, float* lse, int ndim, const int* global_shape, const int* kernel,
    const int* stride, const int* causal, const int* q_tile, const int* kv_tile,
    const int* q_origin, const int* q_extent, const int* kv_origin, const int* kv_extent,
    int clip_to_kv, int B, int Hq, int Hkv, int D, int dtype, float scale,
    b200na_stream_t stream);

/*
 * Whole operator in one call: token permute of Q, K, V -> fused attention -> unpermute of O and
 * LSE, i.e. the forward of the reference's Python backend adapter
 * (src/natten/backends/blackwell_fna.py:91-181) for hosts that bind this C ABI directly.
 *   q: [B, *shape, Hq, D]; k, v: [B, *shape, Hkv, D]; o: [B, *shape, Hq, D]; lse: [B, *shape, Hq]
 *   fp32 or NULL. dtype F16/BF16, D in {64, 128}, prod(q_tile) = 256 or 128, prod(kv_tile) = 128.
 *   workspace: device scratch for the permuted copies, 256-byte aligned, at least
 *   b200na_na_forward_workspace_bytes(...) bytes (0 for 1-D undilated tile-multiple layouts,
 *   which need no permutation). Contents are unspecified afterwards; calls that share a
 *   workspace must be ordered on one stream.
 * b200na_na_forward_workspace_bytes returns the size, or a negative error code.
 */
B200NA_API int64_t b200na_na_forward_workspace_bytes(int ndim, const int* shape,
                                                     const int* dilation, const int* q_tile,
                                                     const int* kv_tile, int B, int Hq, int Hkv,
                                                     int D, int want_lse);
B200NA_API int b200na_na_forward(const void* q, const void* k, const void* v, void* o, float* lse,
                                 int ndim, const int* shape, const int* kernel, const int* stride,
                                 const int* dilation, const int* causal, const int* q_tile,
                                 const int* kv_tile, int B, int Hq, int Hkv, int D, int dtype,
                                 float scale, void* workspace, int64_t workspace_bytes,
                                 b200na_stream_t stream);

/*
 * b200na_na_forward without a workspace argument and without any allocation. This entry has no
 * counterpart in the reference.
 *
 * Who it is for: code that needs the operator at a point where it is not allowed to obtain device
 * memory — a plug-in inside a host application that owns the whole device-memory budget and hands
 * none out after start-up, a serving loop that must not hit the allocator (a cudaMalloc can stall
 * the device and has unbounded latency), or a process that gave all of its memory to a pool when it
 * started. Such callers still pass their own inputs and outputs; only the scratch for the permuted
 * copies comes from the library: a fixed array of B200NA_STATIC_WORKSPACE_BYTES that is part of the
 * loaded module (every GPU that loads the library holds it until the process exits).
 *
 * Same arguments, results and kernels as b200na_na_forward. Differences:
 *   - returns B200NA_ERR_WORKSPACE_LIMIT when b200na_na_forward_workspace_bytes(...) for the
 *     problem exceeds B200NA_STATIC_WORKSPACE_BYTES (use b200na_na_forward then);
 *   - calls no cudaMalloc / cudaFree and no allocating library routine;
 *   - the first call on each device looks up the array's device address (and does the library's
 *     usual one-time per-device set-up); make that first call outside any stream capture. With
 *     CUDA's lazy module loading that first call is also the moment the driver brings the
 *     module holding the array (and each kernel's code, on its first launch) onto the device: a
 *     caller about to hand its memory budget away should make one small call per device and
 *     dtype at start-up, before it does - later calls then change nothing in device memory;
 *   - all calls on a device share the one array, which keeps whatever the previous call left in
 *     it (nothing in it needs clearing between calls); two calls that can overlap on the GPU —
 *     different streams, or the same stream from unsynchronised threads — race on it and corrupt
 *     each other's results. Order them on one stream.
 */
#define B200NA_STATIC_WORKSPACE_BYTES (32u * 1024u * 1024u)
B200NA_API int b200na_na_forward_static(const void* q, const void* k, const void* v, void* o,
                                        float* lse, int ndim, const int* shape, const int* kernel,
                                        const int* stride, const int* dilation, const int* causal,
                                        const int* q_tile, const int* kv_tile, int B, int Hq,
                                        int Hkv, int D, int dtype, float scale,
                                        b200na_stream_t stream);

/*
 * Dense attention forward: replaces natten::blackwell_fmha_forward for the non-varlen case
 * (reference: csrc/src/blackwell_fmha.cu:55-260; Python caller src/natten/functional.py:74-348),
 * used for the extra (cross-attention) KV tokens and the self-attention fast path.
 *   q: [B, Nq, Hq, D]; k, v: [B, Nk, Hkv, D]; o: [B, Nq, Hq, D]; lse: [B, Nq, Hq] or NULL.
 *   causal != 0 requires Nq == Nk (query i sees keys 0..i). Nq, Nk need not be tile multiples.
 *   fp16/bf16 with D a multiple of 8 up to 128 (8-bit floats: of 16) run on the tensor cores;
 *   fp32 operands and other head dims (D <= 256) run on CUDA cores with fp32 arithmetic.
 */
B200NA_API int b200na_fmha_forward(const void* q, const void* k, const void* v, void* o, float* lse, int B,
                        int Nq, int Nk, int Hq, int Hkv, int D, int dtype, float scale, int causal,
                        b200na_stream_t stream);

/*
 * Neighborhood attention forward on the ORIGINAL token layout with CUDA-core fp32 arithmetic.
 * This is the path for fp32 operands (the reference serves fp32 through its CUTLASS 2.x / Flex
 * backends: src/natten/backends/fna.py, flex.py; semantics csrc/include/natten/cuda/reference/
 * mask.hpp:47-89, fna_reference_forward.hpp:63-211) and for head dims the tensor-core kernel
 * does not take. Extra KV tokens are attended by every query (mask.hpp:314-318).
 *   q: [B, *shape, Hq, D]; k, v: [B, *shape, Hkv, D]; add_k/add_v: [B, n_extra, Hkv, D] or NULL;
 *   o: [B, *shape, Hq, D]; lse: [B, *shape, Hq] or NULL. dtype: F32, F16 or BF16. D <= 256.
 */
B200NA_API int b200na_na_forward_simt(const void* q, const void* k, const void* v, void* o, float* lse,
                           int ndim, const int* shape, const int* kernel, const int* stride,
                           const int* dilation, const int* causal, int B, int Hq, int Hkv, int D,
                           int dtype, float scale, const void* add_k, const void* add_v,
                           int n_extra, b200na_stream_t stream);

/*
 * Neighborhood attention BACKWARD on the original token layout with CUDA-core fp32 arithmetic:
 * the gradients the reference's backward ops return (natten::blackwell_na{1,2,3}d_backward,
 * csrc/include/natten/blackwell_fna.h:92-152, after natten::compute_delta,
 * csrc/include/natten/compute_delta.h:35; arithmetic as in csrc/include/natten/cuda/reference/
 * fna_reference_backward.hpp:62-385), on the caller's layout, any of F32 / F16 / BF16, D <= 256,
 * extra key/value tokens included (their gradients go to d_add_k / d_add_v).
 *   q, dq, o, d_out: [B, *shape, Hq, D]; k, v, dk, dv: [B, *shape, Hkv, D]; lse: [B, *shape, Hq]
 *   fp32 as returned by the forward; add_k, add_v, d_add_k, d_add_v: [B, n_extra, Hkv, D] or NULL;
 *   delta_scratch: B * prod(shape) * Hq floats of caller-owned scratch (overwritten).
 * Three to four launches (delta, dQ, dK/dV, extra tokens), no atomics: results are deterministic.
 */
B200NA_API int b200na_na_backward_simt(
    const void* q, const void* k, const void* v, const void* o, const void* d_out, const float* lse,
    const void* add_k, const void* add_v, int n_extra, void* dq, void* dk, void* dv, void* d_add_k,
    void* d_add_v, float* delta_scratch, int ndim, const int* shape, const int* kernel,
    const int* stride, const int* dilation, const int* causal, int B, int Hq, int Hkv, int D,
    int dtype, float scale, b200na_stream_t stream);

/*
 * Neighborhood attention BACKWARD on tensor cores, on the caller's layout: replaces
 * natten::blackwell_na{1,2,3}d_backward (csrc/include/natten/blackwell_fna.h:92-152) together with
 * the token permutes / unpermutes around it (src/natten/backends/blackwell_fna.py:217-300) and
 * natten::compute_delta (csrc/include/natten/compute_delta.h:35). Three launches: delta, one pass
 * of the tcgen05 kernel for dQ (a CTA per 128-query tile streams key/value tiles), one pass of the
 * same kernel for dK and dV (a CTA per 128-key tile streams the query tiles that attend it). No
 * atomics: results are deterministic (the reference's Blackwell backward has no deterministic mode,
 * src/natten/backends/blackwell_fna.py:209-215).
 *   Tensors as in b200na_na_backward_simt (extra tokens and their gradients included: they are
 *   appended to every query's columns in the dQ pass and get a third pass of the same kernel,
 *   rows = the extra tokens, columns = all queries); dtype F16 or BF16; D in {64, 128}.
 *   q_tile / kv_tile: prod = 128 each; tile[a] * dilation[a] <= 256 and dilation[a] <= 8,
 *   otherwise B200NA_ERR_UNSUPPORTED (use b200na_na_backward_simt then).
 */
B200NA_API int b200na_na_backward_direct(
    const void* q, const void* k, const void* v, const void* o, const void* d_out, const float* lse,
    const void* add_k, const void* add_v, int n_extra, void* dq, void* dk, void* dv, void* d_add_k,
    void* d_add_v, float* delta_scratch, int ndim, const int* shape, const int* kernel,
    const int* stride, const int* dilation, const int* causal, const int* q_tile,
    const int* kv_tile, int B, int Hq, int Hkv, int D, int dtype, float scale,
    b200na_stream_t stream);

/*
 * Two-way LSE merge: replaces the elementwise chain of natten.merge_attentions
 * (reference: src/natten/attn_merge.py:48-105; call site src/natten/functional.py:548-554).
 *   o = o0 - sigmoid(l1 - l0) * (o0 - o1);  l = l0 - logsigmoid(l0 - l1)   (fp32 arithmetic)
 *   o0, o1, o: [rows, D] of `dtype`; l0, l1, l: [rows] fp32; rows = B * N * H.
 * An input whose LSE is -inf (no keys) leaves the other input unchanged.
 * o may alias o0 or o1 (each element is read before it is written, by the same thread); l must
 * not alias l0 or l1 (B200NA_ERR_INVALID_ARGUMENT): every thread of a row reads both.
 */
B200NA_API int b200na_merge(const void* o0, const float* l0, const void* o1, const float* l1, void* o,
                 float* l, int64_t rows, int D, int dtype, b200na_stream_t stream);

/*
 * Device-side status of the tensor-core kernels on the current device. Returns B200NA_OK with
 * *status == 0 if no bounded wait has expired since the last call; otherwise returns
 * B200NA_ERR_KERNEL_TIMEOUT and stores a non-zero diagnostic word (role << 8 | barrier that gave
 * up): the results of the launches since the last call are not to be used. Synchronises the
 * device (so it is a check for tests and debugging, not for every step) and resets the word; the
 * context stays usable. The reference has no counterpart: its kernels spin
 * without a bound (csrc/include/natten/cuda/fna_blackwell/kernel/
 * sm100_fna_fwd_kernel_tma_warpspecialized.hpp).
 */
B200NA_API int b200na_device_status(int* status);

#ifdef __cplusplus
}
#endif
#endif /* NATTEN_B200_H_ */
