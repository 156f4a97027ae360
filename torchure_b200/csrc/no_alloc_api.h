// Allocation-free attention backward.  This entry point has no counterpart in the reference.
//
// Some callers must not allocate device memory at the moment they need the attention gradient: code that runs
// inside a region where cudaMalloc is forbidden or would serialise the device (a CUDA graph being replayed by an
// embedding runtime, a real-time serving loop with a fixed memory plan, a plugin whose host owns the allocator and
// hands out no scratch).  The regular path (`attn_bwd` in the Python extension) asks PyTorch's allocator for two
// rows of per-query statistics; this variant keeps them in a fixed array that is part of the library image.
#pragma once
#include <cuda_runtime.h>

extern "C" {

// Largest problem the built-in scratch covers: B * Hq * S query rows.
#define TB_ATTN_BWD_NOALLOC_MAX_ROWS (512 * 1024)

// Causal GQA attention backward for head_dim 128 (same math and layouts as the regular entry point):
//   d_o  [B*S, Hq*128] bf16     gradient of the attention output
//   qk   [B*S, (Hq+Hkv)*128]    bf16 queries | keys (normalised, rotated)
//   qkv  [B*S, (Hq+2Hkv)*128]   bf16 raw projection; only the V columns are read
//   o    [B*S, Hq*128] bf16, lse [B, Hq, S] fp32   saved by the forward pass
//   dqkv [B*S, (Hq+2Hkv)*128]   bf16 OUT: dq | dk | dv
//   status                      device int, OUT: set non-zero if a bounded wait inside a kernel expired (zero it first)
// Shapes as for the forward pass: S a multiple of 128, Hq a multiple of Hkv with an even ratio.
// Returns 0 on success, a negative code on a bad argument, -30 if B*Hq*S exceeds TB_ATTN_BWD_NOALLOC_MAX_ROWS and
// -31 if the scratch symbol could not be resolved on the current device.
//
// No device memory is allocated or freed, here or in anything it calls.  The per-row statistics live in one
// static device array of 2 * TB_ATTN_BWD_NOALLOC_MAX_ROWS floats (4 MiB) that every GPU loading this library holds
// until the process exits.  The FIRST call on each device resolves the array's address (cudaGetSymbolAddress)
// and sets that device's kernel attributes (both are kept per device, so several GPUs may be driven from one
// process), so make that first call outside any stream capture.  All calls share the array and it keeps
// whatever the previous call left there; nothing in it needs clearing because each call rewrites the rows it
// reads.  Two calls that overlap on the GPU (different streams) would race on it: order them.
int tb_attn_bwd_noalloc(const void* d_o, const void* qk, const void* qkv, const void* o, const float* lse, void* dqkv,
                        int B, int S, int Hq, int Hkv, int* status, cudaStream_t stream);
}
