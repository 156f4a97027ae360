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
  // the statistics pass alone (profiling and tests)
  m.def("attn_bwd_prep", [](const torch::Tensor& d_o, const torch::Tensor& o, const torch::Tensor& lse,
                            torch::Tensor& delta, torch::Tensor& lse2, int64_t B, int64_t S, int64_t Hq) {
    TORCH_CHECK(d_o.is_contiguous() && o.is_contiguous() && lse.is_contiguous() && delta.is_contiguous() &&
                lse2.is_contiguous());
    tb::attn_bwd_prep(d_o.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), delta.data_ptr<float>(),
                      lse2.data_ptr<float>(), (int)B, (int)S, (int)Hq, at::cuda::getCurrentCUDAStream().stream());
  });
}
