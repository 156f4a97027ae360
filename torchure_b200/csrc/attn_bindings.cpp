// Python bindings of the attention kernels.
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include <cuda_bf16.h>

#include "attn_api.h"

torch::Tensor attn_err_word();

void register_attn(pybind11::module_& m) {
  m.def("attn_fwd", [](const torch::Tensor& qk, const torch::Tensor& qkv, torch::Tensor& o, torch::Tensor& lse,
                       int64_t B, int64_t S, int64_t Hq, int64_t Hkv) {
    TORCH_CHECK(qk.is_contiguous() && qkv.is_contiguous() && o.is_contiguous() && lse.is_contiguous());
    TORCH_CHECK(qk.size(1) == (Hq + Hkv) * 128 && qkv.size(1) == (Hq + 2 * Hkv) * 128, "attention: head_dim 128 layout");
    const int rc = tb::attn_fwd(qk.data_ptr(), qkv.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), (int)B, (int)S,
                                (int)Hq, (int)Hkv, attn_err_word().data_ptr<int>(),
                                at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(rc == 0, "attn_fwd failed with code ", rc);
  });
  m.def("attn_bwd", [](const torch::Tensor& d_o, const torch::Tensor& qk, const torch::Tensor& qkv,
                       const torch::Tensor& o, const torch::Tensor& lse, torch::Tensor& dqkv, int64_t B, int64_t S,
                       int64_t Hq, int64_t Hkv) {
    TORCH_CHECK(d_o.is_contiguous() && qk.is_contiguous() && qkv.is_contiguous() && o.is_contiguous() &&
                lse.is_contiguous() && dqkv.is_contiguous());
    auto stream = at::cuda::getCurrentCUDAStream().stream();
    // scratch: per-row statistics shared by the dQ and dK/dV kernels
    torch::Tensor scratch = torch::empty({2, B * Hq * S}, lse.options());
    float* delta = scratch.data_ptr<float>();
    float* lse2 = delta + B * Hq * S;
    int* err = attn_err_word().data_ptr<int>();
    tb::attn_bwd_prep(d_o.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), delta, lse2, (int)B, (int)S, (int)Hq, stream);
    int rc = tb::attn_bwd_dq(qk.data_ptr(), qkv.data_ptr(), d_o.data_ptr(), dqkv.data_ptr(), delta, lse2, (int)B, (int)S,
                             (int)Hq, (int)Hkv, err, stream);
    TORCH_CHECK(rc == 0, "attn_bwd_dq failed with code ", rc);
    rc = tb::attn_bwd_dkv(qk.data_ptr(), qkv.data_ptr(), d_o.data_ptr(), dqkv.data_ptr(), delta, lse2, (int)B, (int)S,
                          (int)Hq, (int)Hkv, err, stream);
    TORCH_CHECK(rc == 0, "attn_bwd_dkv failed with code ", rc);
  });
  // single-pass backward: statistics (+ accumulator clear), fused kernel, conversion of dQ to bf16
  m.def("attn_bwd_fused", [](const torch::Tensor& d_o, const torch::Tensor& qk, const torch::Tensor& qkv,
                             const torch::Tensor& o, const torch::Tensor& lse, torch::Tensor& dqkv, int64_t B, int64_t S,
                             int64_t Hq, int64_t Hkv, bool convert_dq) {
    TORCH_CHECK(d_o.is_contiguous() && qk.is_contiguous() && qkv.is_contiguous() && o.is_contiguous() &&
                lse.is_contiguous() && dqkv.is_contiguous());
    auto stream = at::cuda::getCurrentCUDAStream().stream();
    torch::Tensor scratch = torch::empty({2, B * Hq * S}, lse.options());
    torch::Tensor dq_acc = torch::empty({B, Hq, S, 128}, lse.options());
    float* nds = scratch.data_ptr<float>();
    float* nlse2 = nds + B * Hq * S;
    int* err = attn_err_word().data_ptr<int>();
    const int64_t wqk = (Hq + Hkv) * 128, wqkv = (Hq + 2 * Hkv) * 128;
    int rc = tb::attn_bwd_stats(d_o.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), nds, nlse2, dq_acc.data_ptr<float>(),
                                (int)B, (int)S, (int)Hq, stream);
    TORCH_CHECK(rc == 0, "attn_bwd_stats failed with code ", rc);
    auto* out = reinterpret_cast<__nv_bfloat16*>(dqkv.data_ptr());
    rc = tb::attn_bwd_fused({qk.data_ptr(), wqk, 0}, {qk.data_ptr(), wqk, Hq * 128}, {qkv.data_ptr(), wqkv, (Hq + Hkv) * 128},
                            d_o.data_ptr(), dq_acc.data_ptr<float>(), out + Hq * 128, out + (Hq + Hkv) * 128, wqkv, nds,
                            nlse2, (int)B, (int)S, (int)S, (int)Hq, (int)Hkv, true, err, stream);
    TORCH_CHECK(rc == 0, "attn_bwd_fused failed with code ", rc);
    // convert_dq = false leaves dq in the returned head-major fp32 accumulator for a consumer that reads it there
    // (the QK-norm / RoPE backward); the q columns of dqkv are not written then
    if (convert_dq) {
      rc = tb::attn_dq_convert(dq_acc.data_ptr<float>(), out, wqkv, (int)B, (int)S, (int)Hq, stream);
      TORCH_CHECK(rc == 0, "dq conversion failed with code ", rc);
    }
    return dq_acc;
  }, pybind11::arg("d_o"), pybind11::arg("qk"), pybind11::arg("qkv"), pybind11::arg("o"), pybind11::arg("lse"),
     pybind11::arg("dqkv"), pybind11::arg("B"), pybind11::arg("S"), pybind11::arg("Hq"), pybind11::arg("Hkv"),
     pybind11::arg("convert_dq") = true);
  // ---- block-pair entry points (ring attention, Ulysses, any caller with its own q / k / v tensors) --------------
  // q, k, v: bf16 [rows, ld] with innermost stride 1; head h at columns [col0 + 128 h, ...)
  m.def("attn_fwd_pair", [](const torch::Tensor& q, int64_t q_col0, const torch::Tensor& k, int64_t k_col0,
                            const torch::Tensor& v, int64_t v_col0, torch::Tensor& o, torch::Tensor& lse, int64_t B,
                            int64_t Sq, int64_t Skv, int64_t Hq, int64_t Hkv, int64_t q_bstride, int64_t q_row0,
                            int64_t kv_bstride, int64_t kv_row0, bool causal) {
    TORCH_CHECK(q.dim() == 2 && k.dim() == 2 && v.dim() == 2 && q.stride(1) == 1 && k.stride(1) == 1 && v.stride(1) == 1);
    TORCH_CHECK(q.scalar_type() == torch::kBFloat16 && k.scalar_type() == torch::kBFloat16 &&
                v.scalar_type() == torch::kBFloat16 && o.scalar_type() == torch::kBFloat16);
    TORCH_CHECK(o.is_contiguous() && lse.is_contiguous() && o.numel() == B * Sq * Hq * 128 && lse.numel() == B * Hq * Sq);
    TORCH_CHECK((B - 1) * q_bstride + q_row0 + Sq <= q.size(0) && (B - 1) * kv_bstride + kv_row0 + Skv <= k.size(0) &&
                k.size(0) == v.size(0), "attn_fwd_pair: rows out of range");
    const int rc = tb::attn_fwd_pair({q.data_ptr(), q.stride(0), q_col0}, {k.data_ptr(), k.stride(0), k_col0},
                                     {v.data_ptr(), v.stride(0), v_col0}, o.data_ptr(), lse.data_ptr<float>(), (int)B,
                                     (int)Sq, (int)Skv, (int)Hq, (int)Hkv, q.size(0), (int)q_bstride, (int)q_row0, k.size(0),
                                     (int)kv_bstride, (int)kv_row0, causal, attn_err_word().data_ptr<int>(),
                                     at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(rc == 0, "attn_fwd_pair failed with code ", rc);
  });
  m.def("attn_merge", [](torch::Tensor& out_acc, torch::Tensor& lse_acc, const torch::Tensor& o_p,
                         const torch::Tensor& lse_p, int64_t B, int64_t Sq, int64_t Hq, int64_t acc_stride,
                         int64_t acc_row0) {
    TORCH_CHECK(out_acc.is_contiguous() && lse_acc.is_contiguous() && o_p.is_contiguous() && lse_p.is_contiguous());
    TORCH_CHECK(out_acc.scalar_type() == torch::kFloat32 && o_p.scalar_type() == torch::kBFloat16);
    TORCH_CHECK(out_acc.numel() == B * acc_stride * Hq * 128 && lse_acc.numel() == B * Hq * acc_stride &&
                acc_row0 + Sq <= acc_stride);
    const int rc = tb::attn_merge(out_acc.data_ptr<float>(), lse_acc.data_ptr<float>(), o_p.data_ptr(),
                                  lse_p.data_ptr<float>(), (int)B, (int)Sq, (int)Hq, (int)acc_stride, (int)acc_row0,
                                  at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(rc == 0, "attn_merge failed with code ", rc);
  });
  // -rowsum(dO*O)/sqrt(d), -lse*log2(e) and a cleared head-major dQ accumulator
  m.def("attn_bwd_stats", [](const torch::Tensor& d_o, const torch::Tensor& o, const torch::Tensor& lse,
                             torch::Tensor& nds, torch::Tensor& nlse2, torch::Tensor& dq_acc, int64_t B, int64_t S,
                             int64_t Hq) {
    TORCH_CHECK(d_o.is_contiguous() && o.is_contiguous() && lse.is_contiguous() && nds.is_contiguous() &&
                nlse2.is_contiguous() && dq_acc.is_contiguous() && dq_acc.numel() == B * Hq * S * 128);
    const int rc = tb::attn_bwd_stats(d_o.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), nds.data_ptr<float>(),
                                      nlse2.data_ptr<float>(), dq_acc.data_ptr<float>(), (int)B, (int)S, (int)Hq,
                                      at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(rc == 0, "attn_bwd_stats failed with code ", rc);
  });
  // one block pair of the single-pass backward: ADDS into dq_acc, WRITES compact dk / dv [B*Skv, Hkv*128]
  m.def("attn_bwd_pair", [](const torch::Tensor& q, int64_t q_col0, const torch::Tensor& k, int64_t k_col0,
                            const torch::Tensor& v, int64_t v_col0, const torch::Tensor& d_o, torch::Tensor& dq_acc,
                            torch::Tensor& dk, torch::Tensor& dv, const torch::Tensor& nds, const torch::Tensor& nlse2,
                            int64_t B, int64_t Sq, int64_t Skv, int64_t Hq, int64_t Hkv, int64_t q_bstride, int64_t q_row0,
                            int64_t kv_bstride, int64_t kv_row0, int64_t stat_stride, int64_t stat_row0, bool causal) {
    TORCH_CHECK(q.dim() == 2 && k.dim() == 2 && v.dim() == 2 && q.stride(1) == 1 && k.stride(1) == 1 && v.stride(1) == 1);
    TORCH_CHECK(d_o.is_contiguous() && d_o.size(0) == q.size(0) && d_o.size(1) == Hq * 128, "attn_bwd_pair: dO layout");
    TORCH_CHECK(dk.is_contiguous() && dv.is_contiguous() && dk.numel() == B * Skv * Hkv * 128 && dv.numel() == dk.numel());
    TORCH_CHECK(dq_acc.numel() == B * Hq * stat_stride * 128 && nds.numel() == B * Hq * stat_stride &&
                nlse2.numel() == nds.numel() && stat_row0 + Sq <= stat_stride);
    TORCH_CHECK((B - 1) * q_bstride + q_row0 + Sq <= q.size(0) && (B - 1) * kv_bstride + kv_row0 + Skv <= k.size(0) &&
                k.size(0) == v.size(0), "attn_bwd_pair: rows out of range");
    tb::AttnPairLayout lay{q.size(0), (int)q_bstride, (int)q_row0, k.size(0), (int)kv_bstride, (int)kv_row0,
                           (int)stat_stride, (int)stat_row0};
    const int rc = tb::attn_bwd_fused({q.data_ptr(), q.stride(0), q_col0}, {k.data_ptr(), k.stride(0), k_col0},
                                      {v.data_ptr(), v.stride(0), v_col0}, d_o.data_ptr(), dq_acc.data_ptr<float>(),
                                      dk.data_ptr(), dv.data_ptr(), Hkv * 128, nds.data_ptr<float>(),
                                      nlse2.data_ptr<float>(), (int)B, (int)Sq, (int)Skv, (int)Hq, (int)Hkv, causal,
                                      attn_err_word().data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream(), &lay);
    TORCH_CHECK(rc == 0, "attn_bwd_pair failed with code ", rc);
  });
  m.def("attn_dq_convert", [](const torch::Tensor& dq_acc, torch::Tensor& dst, int64_t B, int64_t S, int64_t Hq) {
    TORCH_CHECK(dq_acc.is_contiguous() && dst.dim() == 2 && dst.stride(1) == 1 && dst.size(0) == B * S);
    const int rc = tb::attn_dq_convert(dq_acc.data_ptr<float>(), dst.data_ptr(), dst.stride(0), (int)B, (int)S, (int)Hq,
                                       at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(rc == 0, "attn_dq_convert failed with code ", rc);
  });
  // the statistics pass alone (profiling and tests)
  m.def("attn_bwd_prep", [](const torch::Tensor& d_o, const torch::Tensor& o, const torch::Tensor& lse,
                            torch::Tensor& delta, torch::Tensor& lse2, int64_t B, int64_t S, int64_t Hq) {
    TORCH_CHECK(d_o.is_contiguous() && o.is_contiguous() && lse.is_contiguous() && delta.is_contiguous() &&
                lse2.is_contiguous());
    tb::attn_bwd_prep(d_o.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), delta.data_ptr<float>(),
                      lse2.data_ptr<float>(), (int)B, (int)S, (int)Hq, at::cuda::getCurrentCUDAStream().stream());
  });
}
