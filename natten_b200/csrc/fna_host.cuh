// Host-side helpers shared by the tensor-core kernels (defined in fna_sm100.cu / na_bwd_simt.cu).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200na {

// Tensor map over a heads-last [B, X0, X1, X2, H, D] 16-bit tensor seen as (H*D, X0, X1, X2, B):
// a box of 64 channels x tile[a] * dil[a] positions per axis, traversed with element stride
// dil[a]. B200NA_ERR_UNSUPPORTED when a box exceeds 256 positions or a stride exceeds 8.
int fna_make_tensor_map_direct(CUtensorMap* tm, const void* ptr, int dtype, int B, const int* X,
                               int H, int D, const int* tile, const int* dil);

// One-time per-device setup of the attention kernels; returns the SM count and the address of the
// device status word that bounded waits report into.
int fna_device_info(int* sms, int** status_ptr);

// A zeroed pair of device counters {next work item, CTAs finished} for one launch on `stream` of a
// persistent kernel that hands out its items dynamically; the kernel's last CTA must zero the
// pair again. Launches on one stream share that stream's pair (they cannot overlap); a launch
// under stream capture gets a pair of its own from a pool of 3072 that is handed out in turn.
int fna_work_counters(unsigned long long** pair, cudaStream_t stream);

// delta[row] = sum_d o[row, d] * d_out[row, d] (fp32), rows of D elements of `dtype`.
int launch_delta(const void* o, const void* d_out, float* delta, int64_t rows, int D, int dtype,
                 cudaStream_t stream);

}  // namespace b200na
