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
int attn_bwd_prep(const void* d_o, const void* o, const float* lse, float* delta, float* lse2, int B, int S, int Hq,
                  cudaStream_t stream);
int attn_bwd_dq(const void* qk, const void* qkv, const void* d_o, void* dqkv, const float* delta, const float* lse2,
                int B, int S, int Hq, int Hkv, int* err, cudaStream_t stream);
int attn_bwd_dkv(const void* qk, const void* qkv, const void* d_o, void* dqkv, const float* delta, const float* lse2,
                 int B, int S, int Hq, int Hkv, int* err, cudaStream_t stream);

// One operand of the fused backward: bf16 matrix [rows, ld] (row stride ld elements, 16-byte aligned base and rows);
// head h occupies columns [col0 + 128 h, col0 + 128 h + 128).
struct AttnOperand {
  const void* ptr;
  int64_t ld;
  int64_t col0;
};

// Block-pair forward: queries of one tensor against keys / values of another (the unit of ring attention), written
// into a compact o [B*Sq, Hq*128] / lse [B, Hq, Sq].  Rows of batch b: queries at b * q_bstride + q_row0 of the
// q tensor (q_rows rows in all), keys / values at b * kv_bstride + kv_row0 (kv_rows rows).  causal as in attn_fwd
// (Sq == Skv), else every query sees every key.  Even Hq / Hkv, Sq and Skv multiples of 128.
int attn_fwd_pair(const AttnOperand& q, const AttnOperand& k, const AttnOperand& v, void* o, float* lse, int B, int Sq,
                  int Skv, int Hq, int Hkv, int64_t q_rows, int q_bstride, int q_row0, int64_t kv_rows, int kv_bstride,
                  int kv_row0, bool causal, int* err, cudaStream_t stream);

// Merge a block pair's (o_p bf16 [B*Sq, Hq*128], lse_p [B, Hq, Sq]) into running fp32 results that cover the whole
// local sequence: out_acc [B*acc_stride, Hq*128], lse_acc [B, Hq, acc_stride] (initialise to 0 and -inf); the pair's
// queries start at row acc_row0 of every batch element.
int attn_merge(float* out_acc, float* lse_acc, const void* o_p, const float* lse_p, int B, int Sq, int Hq, int acc_stride,
               int acc_row0, cudaStream_t stream);

// Where a block pair sits inside larger tensors (nullptr = the tensors are exactly [B*Sq] / [B*Skv] rows): q and dO
// rows of batch b at b * q_bstride + q_row0, k / v rows at b * kv_bstride + kv_row0; statistics and the dQ accumulator
// are [B, Hq, stat_stride(, 128)] with this call's queries starting at stat_row0.  dK / dV outputs stay compact.
struct AttnPairLayout {
  int64_t q_rows;
  int q_bstride, q_row0;
  int64_t kv_rows;
  int kv_bstride, kv_row0;
  int stat_stride, stat_row0;
};

// Single-pass backward (attention_bwd_fused_sm100.cu): five tile products per block pair instead of seven.
//   q [B*Sq rows], k / v [B*Skv rows], d_o [B*Sq, Hq*128] bf16
//   nds / nlse2  [B, Hq, Sq] fp32 from attn_bwd_stats: -rowsum(dO*O)/sqrt(d) and -lse*log2(e)
//   dq_acc  fp32 [B, Hq, Sq, 128] (head-major): every CTA ADDS its partial dQ tiles, so it must hold zeros (which
//           attn_bwd_stats writes) or a running sum to extend on entry; attn_dq_convert turns it into bf16 columns
//   dk, dv  bf16 destinations of the first row of KV head 0 (row stride ld_dkv elements, 16-byte aligned)
//   causal  query block qb sees key blocks <= qb (needs Sq == Skv); false = every query sees every key
// Needs Sq % 128 == 0, Skv % 128 == 0 and Hq % Hkv == 0.
int attn_bwd_stats(const void* d_o, const void* o, const float* lse, float* nds, float* nlse2, float* dq_acc, int B,
                   int S, int Hq, cudaStream_t stream);
int attn_bwd_fused(const AttnOperand& q, const AttnOperand& k, const AttnOperand& v, const void* d_o, float* dq_acc,
                   void* dk, void* dv, int64_t ld_dkv, const float* nds, const float* nlse2, int B, int Sq, int Skv,
                   int Hq, int Hkv, bool causal, int* err, cudaStream_t stream, const AttnPairLayout* lay = nullptr);
// dst[(b S + s), 128 h + d] (bf16, row stride ld_dst elements) = dq_acc[b, h, s, d]
int attn_dq_convert(const float* dq_acc, void* dst, int64_t ld_dst, int B, int S, int Hq, cudaStream_t stream);

}  // namespace tb
