// Python bindings: adapt torch tensors to the raw-pointer launchers of api.h.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "api.h"
#include "comm_api.h"
#include "attn_api.h"

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int g_sm_reserve = 0;  // SMs the persistent kernels leave free for communication kernels

int num_sms() {
  static int n = 0;
  if (n == 0) n = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int usable = n - g_sm_reserve;
  return usable > 8 ? usable : 8;
}

// one error word per process (one process drives one GPU)
torch::Tensor& err_word() {
  static torch::Tensor t;
  if (!t.defined()) t = torch::zeros({4}, torch::dtype(torch::kInt32).device(torch::kCUDA));
  return t;
}

const __nv_bfloat16* bf(const torch::Tensor& t) { return reinterpret_cast<const __nv_bfloat16*>(t.data_ptr()); }
__nv_bfloat16* bfm(torch::Tensor& t) { return reinterpret_cast<__nv_bfloat16*>(t.data_ptr()); }
template <class T>
const T* opt_ptr(const c10::optional<torch::Tensor>& t) {
  return t.has_value() && t->defined() ? reinterpret_cast<const T*>(t->data_ptr()) : nullptr;
}
template <class T>
T* opt_mptr(c10::optional<torch::Tensor>& t) {
  return t.has_value() && t->defined() ? reinterpret_cast<T*>(t->data_ptr()) : nullptr;
}

void gemm(const torch::Tensor& a, const torch::Tensor& b, torch::Tensor& out, bool a_mn, bool b_mn, int64_t out_mode,
          int64_t splits) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && out.is_cuda(), "gemm: CUDA tensors required");
  TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16, "gemm: bf16 operands");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2, "gemm: 2-D tensors");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1, "gemm: innermost stride must be 1");
  const int64_t M = a_mn ? a.size(1) : a.size(0), K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0), Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm: reduction sizes differ: ", K, " vs ", Kb);
  TORCH_CHECK(out.size(0) == M && out.size(1) == N, "gemm: output shape");
  TORCH_CHECK(out_mode == 0 ? out.scalar_type() == torch::kBFloat16 : out.scalar_type() == torch::kFloat32,
              "gemm: output dtype does not match out_mode");
  c10::cuda::CUDAGuard guard(a.device());
  const int rc = tb::gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), (int)M, (int)N, (int)K, a.stride(0),
                               b.stride(0), out.stride(0), a_mn, b_mn, (int)out_mode, err_word().data_ptr<int>(),
                               num_sms(), cur_stream(), (int)splits);
  TORCH_CHECK(rc == 0, "gemm_bf16 failed with code ", rc);
}

void add_rmsnorm_fwd(c10::optional<torch::Tensor> x, c10::optional<torch::Tensor> y, c10::optional<torch::Tensor> ids,
                     c10::optional<torch::Tensor> table, const torch::Tensor& w, c10::optional<torch::Tensor> x_out,
                     torch::Tensor& h, torch::Tensor& rstd, double eps) {
  const int M = (int)h.size(0), D = (int)h.size(1);
  TORCH_CHECK(D % 4 == 0, "rmsnorm: D must be a multiple of 4");
  const bool bf16_table = table.has_value() && table->defined() && table->scalar_type() == torch::kBFloat16;
  TORCH_CHECK(!bf16_table || (x_out.has_value() && x_out->defined()), "a bf16 table needs x_out");
  tb::add_rmsnorm_fwd(opt_ptr<float>(x), opt_ptr<__nv_bfloat16>(y), opt_ptr<int64_t>(ids),
                      bf16_table ? nullptr : opt_ptr<float>(table), bf16_table ? opt_ptr<__nv_bfloat16>(table) : nullptr,
                      w.data_ptr<float>(), opt_mptr<float>(x_out), bfm(h), rstd.data_ptr<float>(), M, D, (float)eps,
                      cur_stream());
}

void rmsnorm_bwd(const torch::Tensor& dh, const torch::Tensor& x, const torch::Tensor& w, const torch::Tensor& rstd,
                 c10::optional<torch::Tensor> dx_in, torch::Tensor& dx, c10::optional<torch::Tensor> dx_bf16,
                 torch::Tensor& dw, int64_t variant) {
  const int M = (int)x.size(0), D = (int)x.size(1);
  TORCH_CHECK(dh.is_contiguous() && x.is_contiguous() && dx.is_contiguous(), "rmsnorm_bwd: operands must be contiguous");
  tb::rmsnorm_bwd(bf(dh), x.data_ptr<float>(), w.data_ptr<float>(), rstd.data_ptr<float>(), opt_ptr<float>(dx_in),
                  dx.data_ptr<float>(), opt_mptr<__nv_bfloat16>(dx_bf16), dw.data_ptr<float>(), M, D, num_sms(),
                  err_word().data_ptr<int>(), cur_stream(), (int)variant);
}

void qknorm_rope_fwd(const torch::Tensor& qkv, const torch::Tensor& qw, const torch::Tensor& kw,
                     const torch::Tensor& cos, const torch::Tensor& sin, torch::Tensor& out, int64_t S, int64_t Hq,
                     int64_t Hkv, double eps, bool use_norm) {
  TORCH_CHECK(qkv.size(1) == (Hq + 2 * Hkv) * 128, "qknorm_rope: head_dim must be 128");
  tb::qknorm_rope_fwd(bf(qkv), qw.data_ptr<float>(), kw.data_ptr<float>(), cos.data_ptr<float>(),
                      sin.data_ptr<float>(), bfm(out), (int)qkv.size(0), (int)S, (int)Hq, (int)Hkv, 128, (float)eps,
                      use_norm ? 1 : 0, cur_stream());
}

void qknorm_rope_bwd(torch::Tensor& dqkv, const torch::Tensor& qkv, const torch::Tensor& qw, const torch::Tensor& kw,
                     const torch::Tensor& cos, const torch::Tensor& sin, torch::Tensor& dqw, torch::Tensor& dkw,
                     int64_t S, int64_t Hq, int64_t Hkv, double eps, bool use_norm,
                     c10::optional<torch::Tensor> dq_acc, int64_t stages, int64_t warps) {
  TORCH_CHECK(qkv.size(1) == (Hq + 2 * Hkv) * 128, "qknorm_rope: head_dim must be 128");
  if (dq_acc.has_value() && dq_acc->defined())
    TORCH_CHECK(dq_acc->scalar_type() == torch::kFloat32 && dq_acc->is_contiguous() &&
                    dq_acc->numel() == qkv.size(0) * Hq * 128,
                "qknorm_rope_bwd: dq_acc must be fp32 [B, Hq, S, 128]");
  TORCH_CHECK(cos.stride(0) == 128 && sin.stride(0) == 128 && cos.is_contiguous() && sin.is_contiguous(),
              "qknorm_rope_bwd: cos / sin tables must be contiguous [S, 128]");
  // rows are staged by bulk copies: 16-byte aligned bases (row and head offsets are multiples of 256 bytes)
  TORCH_CHECK(dqkv.is_contiguous() && qkv.is_contiguous() && (reinterpret_cast<uintptr_t>(dqkv.data_ptr()) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(qkv.data_ptr()) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(cos.data_ptr()) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(sin.data_ptr()) & 15) == 0,
              "qknorm_rope_bwd: operands must be contiguous and 16-byte aligned");
  const int rc = tb::qknorm_rope_bwd(bfm(dqkv), bf(qkv), qw.data_ptr<float>(), kw.data_ptr<float>(),
                                     cos.data_ptr<float>(), sin.data_ptr<float>(), dqw.data_ptr<float>(),
                                     dkw.data_ptr<float>(), opt_ptr<float>(dq_acc), (int)qkv.size(0), (int)S, (int)Hq,
                                     (int)Hkv, 128, (float)eps, use_norm ? 1 : 0, num_sms(), err_word().data_ptr<int>(),
                                     cur_stream(), (int)stages, (int)warps);
  TORCH_CHECK(rc == 0, "qknorm_rope_bwd failed with code ", rc);
}

void swiglu_fwd(const torch::Tensor& gu, torch::Tensor& act) {
  TORCH_CHECK(act.size(1) % 8 == 0, "swiglu: F must be a multiple of 8");
  tb::swiglu_fwd(bf(gu), bfm(act), (int)act.size(0), (int)act.size(1), cur_stream());
}
void swiglu_bwd(const torch::Tensor& dact, const torch::Tensor& gu, torch::Tensor& dgu) {
  tb::swiglu_bwd(bf(dact), bf(gu), bfm(dgu), (int)dact.size(0), (int)dact.size(1), cur_stream());
}
void embedding_bwd(const torch::Tensor& dx, const torch::Tensor& ids, torch::Tensor& dtable) {
  tb::embedding_bwd(dx.data_ptr<float>(), ids.data_ptr<int64_t>(), dtable.data_ptr<float>(), (int)dx.size(0),
                    (int)dx.size(1), cur_stream());
}
void ce_softmax_grad(torch::Tensor& logits, const torch::Tensor& labels, torch::Tensor& row_loss,
                     const torch::Tensor& inv_n_valid, int64_t ignore_index) {
  TORCH_CHECK(logits.stride(1) == 1 && logits.stride(0) % 8 == 0, "ce: logits rows must be 16-byte aligned");
  tb::ce_softmax_grad(bfm(logits), logits.stride(0), labels.data_ptr<int64_t>(), row_loss.data_ptr<float>(),
                      inv_n_valid.data_ptr<float>(), (int)logits.size(0), (int)logits.size(1), (int)ignore_index,
                      cur_stream());
}
void ce_row_stats(const torch::Tensor& logits, const torch::Tensor& labels, torch::Tensor& stats, int64_t vocab_lo,
                  int64_t ignore_index) {
  TORCH_CHECK(logits.stride(1) == 1 && logits.stride(0) % 8 == 0, "ce: logits rows must be 16-byte aligned");
  TORCH_CHECK(stats.is_contiguous() && stats.scalar_type() == torch::kFloat32 && stats.numel() == 3 * logits.size(0) &&
              labels.numel() == logits.size(0), "ce_row_stats: stats must be fp32 [3, rows]");
  tb::ce_row_stats(bf(logits), logits.stride(0), labels.data_ptr<int64_t>(),
                   stats.data_ptr<float>(), (int)logits.size(0), (int)logits.size(1), vocab_lo, (int)ignore_index,
                   cur_stream());
}
void ce_grad_from_lse(torch::Tensor& logits, const torch::Tensor& labels, const torch::Tensor& lse,
                      const torch::Tensor& inv_n_valid, int64_t vocab_lo, int64_t ignore_index) {
  TORCH_CHECK(logits.stride(1) == 1 && logits.stride(0) % 8 == 0, "ce: logits rows must be 16-byte aligned");
  TORCH_CHECK(lse.is_contiguous() && lse.scalar_type() == torch::kFloat32 && lse.numel() == logits.size(0) &&
              labels.numel() == logits.size(0), "ce_grad_from_lse: lse must be fp32 [rows]");
  tb::ce_grad_from_lse(bfm(logits), logits.stride(0), labels.data_ptr<int64_t>(), lse.data_ptr<float>(),
                       inv_n_valid.data_ptr<float>(), (int)logits.size(0), (int)logits.size(1), vocab_lo,
                       (int)ignore_index, cur_stream());
}
void cast_to_bf16(const torch::Tensor& src, torch::Tensor& dst) {
  tb::cast_f32_to_bf16(src.data_ptr<float>(), bfm(dst), src.numel(), cur_stream());
}
void scale_inplace(torch::Tensor& x, const torch::Tensor& scale) {
  if (x.scalar_type() == torch::kFloat32) tb::scale_inplace_f32(x.data_ptr<float>(), scale.data_ptr<float>(), x.numel(), cur_stream());
  else tb::scale_inplace_bf16(bfm(x), scale.data_ptr<float>(), x.numel(), cur_stream());
}

tb::TensorList as_list(const torch::Tensor& ptrs, const torch::Tensor& numel, const torch::Tensor& flags,
                       const torch::Tensor& block_tensor, const torch::Tensor& block_chunk) {
  tb::TensorList t;
  const int64_t n = numel.numel();
  const int64_t* base = ptrs.data_ptr<int64_t>();
  t.ptrs_a = base; t.ptrs_b = base + n; t.ptrs_c = base + 2 * n; t.ptrs_d = base + 3 * n; t.ptrs_e = base + 4 * n;
  t.numel = numel.data_ptr<int64_t>();
  t.flags = flags.data_ptr<int32_t>();
  t.block_tensor = block_tensor.data_ptr<int32_t>();
  t.block_chunk = block_chunk.data_ptr<int32_t>();
  t.n_blocks = (int)block_tensor.numel();
  return t;
}

void adamw_multi(const torch::Tensor& ptrs, const torch::Tensor& numel, const torch::Tensor& flags,
                 const torch::Tensor& bt, const torch::Tensor& bc, double lr, double b1, double b2, double eps,
                 double wd, double bias1, double bias2, c10::optional<torch::Tensor> grad_scale, bool maximize,
                 c10::optional<torch::Tensor> hyper) {
  tb::adamw_multi(as_list(ptrs, numel, flags, bt, bc), (float)lr, (float)b1, (float)b2, (float)eps, (float)wd,
                  (float)bias1, (float)bias2, opt_ptr<float>(grad_scale), maximize ? 1 : 0, opt_ptr<float>(hyper),
                  cur_stream());
}
void sqnorm_multi(const torch::Tensor& ptrs, const torch::Tensor& numel, const torch::Tensor& flags,
                  const torch::Tensor& bt, const torch::Tensor& bc, torch::Tensor& out) {
  tb::sqnorm_multi(as_list(ptrs, numel, flags, bt, bc), out.data_ptr<float>(), cur_stream());
}
void scale_multi(const torch::Tensor& ptrs, const torch::Tensor& numel, const torch::Tensor& flags,
                 const torch::Tensor& bt, const torch::Tensor& bc, const torch::Tensor& scale) {
  tb::scale_multi(as_list(ptrs, numel, flags, bt, bc), scale.data_ptr<float>(), cur_stream());
}
void zero_multi(const torch::Tensor& ptrs, const torch::Tensor& numel, const torch::Tensor& flags,
                const torch::Tensor& bt, const torch::Tensor& bc) {
  tb::zero_multi(as_list(ptrs, numel, flags, bt, bc), cur_stream());
}
void bucket_pack_multi(const torch::Tensor& ptrs, const torch::Tensor& numel, const torch::Tensor& flags,
                       const torch::Tensor& bt, const torch::Tensor& bc, bool accumulate, double post_scale,
                       c10::optional<torch::Tensor> sq) {
  tb::bucket_pack_multi(as_list(ptrs, numel, flags, bt, bc), accumulate ? 1 : 0, (float)post_scale,
                        opt_mptr<float>(sq), cur_stream());
}

torch::Tensor error_word() { return err_word(); }

}  // namespace

torch::Tensor attn_err_word() { return err_word(); }

void register_comm(pybind11::module_& m);
void register_attn(pybind11::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm, "bf16 tcgen05 GEMM: out = A * B^T (operand majors selectable)", pybind11::arg("a"),
        pybind11::arg("b"), pybind11::arg("out"), pybind11::arg("a_mn"), pybind11::arg("b_mn"), pybind11::arg("out_mode"),
        pybind11::arg("splits") = 0);
  m.def("set_sm_reserve", [](int64_t n) { g_sm_reserve = (int)n; }, "persistent kernels use (SM count - n) CTAs");
  m.def("gemm_pair_capacity", &tb::gemm_pair_capacity, "CTA pairs (2-SM clusters) resident at once; 0 before the first launch");
  m.def("error_word", &error_word, "device int32[4]; [0] is set when a bounded wait of a kernel expired");
  m.def("add_rmsnorm_fwd", &add_rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd, pybind11::arg("dh"), pybind11::arg("x"), pybind11::arg("w"), pybind11::arg("rstd"),
        pybind11::arg("dx_in"), pybind11::arg("dx"), pybind11::arg("dx_bf16"), pybind11::arg("dw"),
        pybind11::arg("variant") = 0);
  m.def("qknorm_rope_fwd", &qknorm_rope_fwd);
  m.def("qknorm_rope_bwd", &qknorm_rope_bwd, pybind11::arg("dqkv"), pybind11::arg("qkv"), pybind11::arg("qw"),
        pybind11::arg("kw"), pybind11::arg("cos"), pybind11::arg("sin"), pybind11::arg("dqw"), pybind11::arg("dkw"),
        pybind11::arg("S"), pybind11::arg("Hq"), pybind11::arg("Hkv"), pybind11::arg("eps"), pybind11::arg("use_norm"),
        pybind11::arg("dq_acc") = c10::nullopt, pybind11::arg("stages") = 0, pybind11::arg("warps") = 0);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("embedding_bwd", &embedding_bwd);
  // ids_ptrs / rows_ptrs: device-visible addresses (ints) of int64 [M] ids and fp32 [M, D] rows, one pair per source
  m.def("embedding_scatter", [](std::vector<int64_t> ids_ptrs, std::vector<int64_t> rows_ptrs, torch::Tensor& dtable,
                                int64_t M, double scale, c10::optional<torch::Tensor> sq_delta, int64_t blocks,
                                c10::optional<torch::Tensor> ids_scratch) {
    TORCH_CHECK(ids_ptrs.size() == rows_ptrs.size() && !ids_ptrs.empty() && ids_ptrs.size() <= 8, "1..8 sources");
    TORCH_CHECK(dtable.scalar_type() == torch::kFloat32 && dtable.dim() == 2 && dtable.stride(1) == 1 &&
                dtable.stride(0) == dtable.size(1), "embedding_scatter: dtable must be contiguous fp32 [V, D]");
    const int64_t* ids[8];
    const float* rows[8];
    for (size_t p = 0; p < ids_ptrs.size(); ++p) {
      TORCH_CHECK(ids_ptrs[p] % 8 == 0 && rows_ptrs[p] % 16 == 0, "embedding_scatter: unaligned source");
      ids[p] = reinterpret_cast<const int64_t*>(ids_ptrs[p]);
      rows[p] = reinterpret_cast<const float*>(rows_ptrs[p]);
    }
    if (sq_delta.has_value() && sq_delta->defined())
      TORCH_CHECK(sq_delta->scalar_type() == torch::kFloat32 && sq_delta->numel() >= blocks);
    int64_t* scratch = nullptr;
    if (ids_scratch.has_value() && ids_scratch->defined()) {
      TORCH_CHECK(ids_scratch->scalar_type() == torch::kInt64 && ids_scratch->is_contiguous() &&
                      ids_scratch->numel() >= (int64_t)ids_ptrs.size() * M,
                  "embedding_scatter: ids_scratch must be int64 with room for every source's ids");
      scratch = ids_scratch->data_ptr<int64_t>();
    }
    const int rc = tb::embedding_scatter((int)ids_ptrs.size(), ids, rows, dtable.data_ptr<float>(), (int)M,
                                         (int)dtable.size(1), (float)scale, opt_mptr<float>(sq_delta), (int)blocks,
                                         cur_stream(), scratch);
    TORCH_CHECK(rc == 0, "embedding_scatter failed with code ", rc);
  }, pybind11::arg("ids_ptrs"), pybind11::arg("rows_ptrs"), pybind11::arg("dtable"), pybind11::arg("M"),
     pybind11::arg("scale"), pybind11::arg("sq_delta"), pybind11::arg("blocks"),
     pybind11::arg("ids_scratch") = c10::nullopt);
  m.def("ce_softmax_grad", &ce_softmax_grad);
  m.def("ce_row_stats", &ce_row_stats);
  m.def("ce_grad_from_lse", &ce_grad_from_lse);
  m.def("cast_to_bf16", &cast_to_bf16);
  m.def("scale_inplace", &scale_inplace);
  m.def("adamw_multi", &adamw_multi);
  m.def("sqnorm_multi", &sqnorm_multi);
  m.def("finalize_norm", [](const torch::Tensor& partials, double max_norm, double eps, torch::Tensor& out) {
    TORCH_CHECK(partials.scalar_type() == torch::kFloat32 && partials.is_contiguous() && out.numel() >= 2 &&
                out.scalar_type() == torch::kFloat32);
    tb::finalize_norm(partials.data_ptr<float>(), (int)partials.numel(), (float)max_norm, (float)eps,
                      out.data_ptr<float>(), cur_stream());
  });
  m.def("scale_multi", &scale_multi);
  m.def("zero_multi", &zero_multi);
  m.def("bucket_pack_multi", &bucket_pack_multi);
  register_comm(m);
  register_attn(m);
}
