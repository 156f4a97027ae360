// Host-callable launchers of the tcgen05 flash-attention kernels (attention_fwd_sm100.cu, attention_bwd_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {

// qk  [B*S, (Hq+Hkv)*128] bf16 (queries then keys, normalised and rotated), qkv [B*S, (Hq+2Hkv)*128] bf16 (V columns
// are read), o [B*S, Hq*128] bf16, lse [B, Hq, S] fp32.  Causal.  Needs S % 128 == 0 and an even Hq/Hkv.
int attn_fwd(const void* qk, const void* qkv, void* o, float* lse, int B, int S, int Hq, int Hkv, int* err,
             cudaStream_t stream);

// Backward.  `delta` and `lse2` are scratch rows of B*Hq*S floats each, filled by attn_bwd_prep and read by the two
// gradient kernels.  dqkv [B*S, (Hq+2Hkv)*128] bf16 receives dq | dk | dv (gradients w.r.t. the rotated q and k).
void attn_bwd_prep(const void* d_o, const void* o, const float* lse, float* delta, float* lse2, int B, int S, int Hq,
                   cudaStream_t stream);
int attn_bwd_dq(const void* qk, const void* qkv, const void* d_o, void* dqkv, const float* delta, const float* lse2,
                int B, int S, int Hq, int Hkv, int* err, cudaStream_t stream);
int attn_bwd_dkv(const void* qk, const void* qkv, const void* d_o, void* dqkv, const float* delta, const float* lse2,
                 int B, int S, int Hq, int Hkv, int* err, cudaStream_t stream);

}  // namespace tb
