// Host-callable launchers of the sm_100a kernels.  Plain C++ signatures (raw device pointers, sizes, a
// stream) so the kernels compile without the PyTorch headers; bindings.cpp adapts tensors to them.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {

// ---- tcgen05 GEMM --------------------------------------------------------------------------
// C[M,N] = A * B^T over bf16 operands with fp32 accumulation in TMEM.
//   a_mn == false: A is stored [M, K] (K contiguous), lda = row stride in elements
//   a_mn == true : A is stored [K, M] (M contiguous), lda = row stride in elements
//   b_mn == false: B is stored [N, K] (K contiguous)
//   b_mn == true : B is stored [K, N] (N contiguous)
// out_mode 0: C bf16 store, 1: C fp32 store, 2: C fp32 += (TMA reduce-add)
// Returns 0 or a negative code for an argument error.  `err` is a device int that a kernel sets when
// one of its bounded waits expires.
int gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
              bool a_mn, bool b_mn, int out_mode, int* err, int num_sms, cudaStream_t stream, int force_splits = 0);
// CTA pairs the device holds at once (0 before the first pair launch of this process).
int gemm_pair_capacity();
// The CTA-pair kernel behind gemm_bf16 (tiles of 256 x 256 on two SMs); `splits` as chosen by gemm_bf16.
int gemm2_bf16(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
               bool a_mn, bool b_mn, int out_mode, int splits, int* err, int num_sms, cudaStream_t stream);

// ---- elementwise / normalisation -------------------------------------------------------------
// h = rmsnorm(x_new) * w with x_new = x (+ y); optional gather x = table[ids].  Writes x_new when y or ids
// is given.  x/x_out fp32 [M,D], y bf16 [M,D], h bf16 [M,D], rstd fp32 [M].  With ids, rows come from `table` (fp32)
// or, when table_bf16 is given, from that bf16 copy (an x_out is required then: the row is re-read from it).
void add_rmsnorm_fwd(const float* x, const __nv_bfloat16* y, const int64_t* ids, const float* table,
                     const __nv_bfloat16* table_bf16, const float* w, float* x_out, __nv_bfloat16* h, float* rstd, int M,
                     int D, float eps, cudaStream_t stream);
// dx = dx_in + d rmsnorm; dw += sum_rows(dh * xhat).  dx_bf16 (optional) receives a bf16 copy of dx.
// variant 0: rows staged through shared memory when the shape allows (D <= 1024); 1: the register-resident kernels
void rmsnorm_bwd(const __nv_bfloat16* dh, const float* x, const float* w, const float* rstd, const float* dx_in,
                 float* dx, __nv_bfloat16* dx_bf16, float* dw, int M, int D, int num_sms, int* err, cudaStream_t stream,
                 int variant = 0);
// per-head RMSNorm + RoPE on the q and k column ranges of qkv [M, (Hq+2Hkv)*hd]; out [M, (Hq+Hkv)*hd]
void qknorm_rope_fwd(const __nv_bfloat16* qkv, const float* qw, const float* kw, const float* cos, const float* sin,
                     __nv_bfloat16* out, int M, int S, int Hq, int Hkv, int hd, float eps, int use_norm,
                     cudaStream_t stream);
// in place on the q/k column ranges of dqkv [M, (Hq+2Hkv)*hd]; dqw/dkw fp32 [hd] accumulate.  dq_acc (optional):
// head-major fp32 [B, Hq, S, hd] holding dq instead of the q columns of dqkv (they are only written then).
// Returns 0, or a negative code when the row buffers do not fit / the launch failed.  `err`: device error word, set
// when a staged row never arrives.
int qknorm_rope_bwd(__nv_bfloat16* dqkv, const __nv_bfloat16* qkv, const float* qw, const float* kw, const float* cos,
                    const float* sin, float* dqw, float* dkw, const float* dq_acc, int M, int S, int Hq, int Hkv, int hd,
                    float eps, int use_norm, int num_sms, int* err, cudaStream_t stream, int force_stages = 0,
                    int force_warps = 0);
void swiglu_fwd(const __nv_bfloat16* gu, __nv_bfloat16* act, int M, int F, cudaStream_t stream);
void swiglu_bwd(const __nv_bfloat16* dact, const __nv_bfloat16* gu, __nv_bfloat16* dgu, int M, int F,
                cudaStream_t stream);
// dtable[ids[r]] += dx[r]
void embedding_bwd(const float* dx, const int64_t* ids, float* dtable, int M, int D, cudaStream_t stream);
// Deterministic multi-source variant: dtable[id] += scale * sum_p sum_{r: ids_p[r] == id} rows_p[r] with a fixed
// order of additions and no atomics (sources may be peer GPUs' buffers).  sq_delta (optional, `blocks` floats) receives
// per-CTA sum(new^2 - old^2) of the touched elements.
int embedding_scatter(int n_sources, const int64_t* const* ids, const float* const* rows, float* dtable, int M, int D,
                      float scale, float* sq_delta, int blocks, cudaStream_t stream, int64_t* ids_scratch = nullptr);
// logits [C, V] bf16 (row stride ldl) -> per-row loss (0 for ignored rows) and, in place, dlogits scaled by
// *inv_n_valid.
void ce_softmax_grad(__nv_bfloat16* logits, int64_t ldl, const int64_t* labels, float* row_loss,
                     const float* inv_n_valid, int C, int V, int ignore_index, cudaStream_t stream);
// The same for a vocabulary sharded over ranks (this rank's logits hold columns [vocab_lo, vocab_lo + V)):
// ce_row_stats writes each row's maximum, sum of exponentials relative to it and target logit (0 when the target is
// another rank's) to stats[0 / 1 / 2][C]; ce_grad_from_lse, given the log-sum-exp over ALL ranks' columns, overwrites
// the logits with (softmax - onehot) * *inv_n_valid (zeros for ignored rows).
void ce_row_stats(const __nv_bfloat16* logits, int64_t ldl, const int64_t* labels, float* stats, int C, int V,
                  int64_t vocab_lo, int ignore_index, cudaStream_t stream);
void ce_grad_from_lse(__nv_bfloat16* logits, int64_t ldl, const int64_t* labels, const float* lse,
                      const float* inv_n_valid, int C, int V, int64_t vocab_lo, int ignore_index, cudaStream_t stream);
void cast_f32_to_bf16(const float* src, __nv_bfloat16* dst, int64_t n, cudaStream_t stream);
// x *= *scale unless *scale == 1
void scale_inplace_f32(float* x, const float* scale, int64_t n, cudaStream_t stream);
void scale_inplace_bf16(__nv_bfloat16* x, const float* scale, int64_t n, cudaStream_t stream);

// ---- multi-tensor ------------------------------------------------------------------------------
struct TensorList {           // device-resident table (built once per parameter set)
  const int64_t* ptrs_a;      // meaning depends on the op
  const int64_t* ptrs_b;
  const int64_t* ptrs_c;
  const int64_t* ptrs_d;
  const int64_t* ptrs_e;
  const int64_t* numel;       // elements per tensor
  const int32_t* flags;       // per-tensor flags
  const int32_t* block_tensor;   // per thread block: tensor index
  const int32_t* block_chunk;    // per thread block: chunk index inside the tensor
  int n_blocks;
};
constexpr int kChunkElems = 16384;
// fp32 master p, fp32/bf16 grad g (flag bit0 = grad is bf16), m, v fp32, optional bf16 shadow (ptr 0 = none).
// `hyper` (optional, device): {lr, bias1, bias2} overriding the scalar arguments at run time.
void adamw_multi(const TensorList& t, float lr, float beta1, float beta2, float eps, float weight_decay,
                 float bias1, float bias2, const float* grad_scale, int maximize, const float* hyper,
                 cudaStream_t stream);
// out[0] = sqrt(sum(partials[0..n))), out[1] = min(1, max_norm / (out[0] + eps)) (1 when max_norm <= 0); one launch,
// fixed summation order
void finalize_norm(const float* partials, int n, float max_norm, float eps, float* out, cudaStream_t stream);
// out[0] += sum over all tensors of x^2 (flag bit0 = bf16)
void sqnorm_multi(const TensorList& t, float* out, cudaStream_t stream);
void scale_multi(const TensorList& t, const float* scale, cudaStream_t stream);
void zero_multi(const TensorList& t, cudaStream_t stream);
// bucket[off_i ...] (=|+=) cast(grad_i); sq (optional) receives the sum of squares of the result
void bucket_pack_multi(const TensorList& t, int accumulate, float post_scale, float* sq, cudaStream_t stream);

}  // namespace tb
