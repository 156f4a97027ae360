// Python bindings of the NVLink collective kernels.
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include "comm_api.h"

namespace {

torch::Tensor& comm_err_word() {
  static torch::Tensor t;
  if (!t.defined()) t = torch::zeros({4}, torch::dtype(torch::kInt32).device(torch::kCUDA));
  return t;
}

tb::CommCtx make_ctx(const std::vector<int64_t>& peers, int64_t mc, int64_t rank, int64_t world, int64_t limit_ns) {
  TORCH_CHECK((int)peers.size() <= tb::kCommMaxRanks && world <= tb::kCommMaxRanks, "at most 8 ranks per communicator");
  tb::CommCtx c{};
  for (size_t i = 0; i < peers.size(); ++i) c.peer_bufs[i] = (uint64_t)peers[i];
  c.mc_buf = (uint64_t)mc;
  c.rank = (int)rank;
  c.world = (int)world;
  c.err = comm_err_word().data_ptr<int>();
  c.wait_limit_ns = (uint64_t)limit_ns;
  c.grid_counter = nullptr;
  return c;
}

cudaStream_t cs() { return at::cuda::getCurrentCUDAStream().stream(); }

int dt_of(int64_t code) { return code == 0 ? tb::kF32 : tb::kBF16; }

}  // namespace

void register_comm(pybind11::module_& m) {
  m.attr("COMM_FLAG_BYTES") = tb::kFlagBytes;
  m.attr("COMM_PARTIAL_BYTES") = tb::kPartialBytes;
  m.attr("COMM_MAX_BLOCKS") = tb::kCommMaxBlocks;
  m.attr("COMM_MAX_RANKS") = tb::kCommMaxRanks;
  m.attr("COMM_MAX_SEGMENTS") = tb::kCommMaxSegments;
  m.def("comm_error_word", [] { return comm_err_word(); });
  m.def("comm_all_reduce", [](std::vector<int64_t> peers, int64_t mc, int64_t rank, int64_t world, int64_t limit,
                              int64_t off, int64_t n, int64_t dtype, int64_t op, bool use_mc, int64_t sq_slot,
                              int64_t blocks) {
    tb::comm_all_reduce(make_ctx(peers, mc, rank, world, limit), off, n, dt_of(dtype), (int)op, use_mc, (int)sq_slot, 0,
                        (int)blocks, cs());
  });
  m.def("comm_all_reduce_fused", [](std::vector<int64_t> peers, int64_t mc, int64_t rank, int64_t world, int64_t limit,
                                    int64_t off, torch::Tensor in, torch::Tensor out, int64_t n, int64_t dtype,
                                    int64_t op, bool use_mc, bool oneshot, int64_t blocks) {
    tb::comm_all_reduce_fused(make_ctx(peers, mc, rank, world, limit), off, in.data_ptr(), out.data_ptr(), n,
                              dt_of(dtype), (int)op, use_mc, oneshot, (int)blocks, cs());
  });
  m.def("comm_all_gather", [](std::vector<int64_t> peers, int64_t mc, int64_t rank, int64_t world, int64_t limit,
                              int64_t dst_off, torch::Tensor in, torch::Tensor out, int64_t n, int64_t dtype,
                              bool use_mc, int64_t blocks) {
    tb::comm_all_gather(make_ctx(peers, mc, rank, world, limit), dst_off, in.data_ptr(), out.data_ptr(), n, dt_of(dtype),
                        use_mc, (int)blocks, cs());
  });
  m.def("comm_reduce_scatter", [](std::vector<int64_t> peers, int64_t mc, int64_t rank, int64_t world, int64_t limit,
                                  int64_t off, torch::Tensor in, torch::Tensor out, int64_t n, int64_t dtype, int64_t op,
                                  bool use_mc, int64_t blocks) {
    tb::comm_reduce_scatter(make_ctx(peers, mc, rank, world, limit), off, in.data_ptr(), out.data_ptr(), n, dt_of(dtype),
                            (int)op, use_mc, (int)blocks, cs());
  });
  m.def("comm_all_to_all", [](std::vector<int64_t> peers, int64_t mc, int64_t rank, int64_t world, int64_t limit,
                              int64_t dst_off, torch::Tensor in, torch::Tensor out, int64_t n, int64_t dtype,
                              int64_t blocks) {
    tb::comm_all_to_all(make_ctx(peers, mc, rank, world, limit), dst_off, in.data_ptr(), out.data_ptr(), n, dt_of(dtype),
                        (int)blocks, cs());
  });
  m.def("comm_broadcast", [](std::vector<int64_t> peers, int64_t mc, int64_t rank, int64_t world, int64_t limit,
                             int64_t off, torch::Tensor buf, int64_t n, int64_t dtype, int64_t src, bool use_mc,
                             int64_t blocks) {
    tb::comm_broadcast(make_ctx(peers, mc, rank, world, limit), off, buf.data_ptr(), n, dt_of(dtype), (int)src, use_mc,
                       (int)blocks, cs());
  });
  // segments: (byte offset in the symmetric allocation, elements per chunk); element size from dtype
  m.def("comm_all_gather_inplace", [](std::vector<int64_t> peers, int64_t mc, int64_t rank, int64_t world, int64_t limit,
                                      std::vector<int64_t> offs, std::vector<int64_t> chunk_bytes, bool use_mc,
                                      int64_t blocks) {
    TORCH_CHECK(offs.size() == chunk_bytes.size() && offs.size() <= (size_t)tb::kCommMaxSegments, "too many segments");
    tb::CommSegments sg{};
    sg.n = (int)offs.size();
    for (int i = 0; i < sg.n; ++i) {
      TORCH_CHECK(offs[i] % 16 == 0 && chunk_bytes[i] % 16 == 0, "segments must be 16-byte aligned");
      sg.off[i] = (uint64_t)offs[i];
      sg.nvec[i] = chunk_bytes[i] / 16;
    }
    tb::comm_all_gather_inplace(make_ctx(peers, mc, rank, world, limit), sg, use_mc, (int)blocks, cs());
  });
  m.def("comm_reduce_scatter_symm", [](std::vector<int64_t> peers, int64_t mc, int64_t rank, int64_t world, int64_t limit,
                                       std::vector<int64_t> offs, std::vector<torch::Tensor> outs, int64_t op,
                                       bool use_mc, int64_t sq_slot, int64_t blocks) {
    TORCH_CHECK(offs.size() == outs.size() && offs.size() <= (size_t)tb::kCommMaxSegments, "too many segments");
    tb::CommSegments sg{};
    sg.n = (int)offs.size();
    for (int i = 0; i < sg.n; ++i) {
      TORCH_CHECK(outs[i].scalar_type() == torch::kFloat32 && outs[i].is_contiguous(), "fp32 contiguous shards");
      const int64_t bytes = outs[i].numel() * 4;
      TORCH_CHECK(offs[i] % 16 == 0 && bytes % 16 == 0 && ((uintptr_t)outs[i].data_ptr() & 15) == 0, "16-byte alignment");
      sg.off[i] = (uint64_t)offs[i];
      sg.nvec[i] = bytes / 16;
      sg.out[i] = outs[i].data_ptr();
    }
    tb::comm_reduce_scatter_symm(make_ctx(peers, mc, rank, world, limit), sg, (int)op, use_mc, (int)sq_slot, (int)blocks,
                                 cs());
  });
  m.def("ag_gemm", [](std::vector<int64_t> peers, int64_t mc, int64_t rank, int64_t world, int64_t limit, int64_t a_off,
                      int64_t g_off, int64_t epoch, torch::Tensor b, torch::Tensor c, int64_t M, int64_t K, bool b_mn) {
    const int64_t N = b_mn ? b.size(1) : b.size(0);
    TORCH_CHECK(b.stride(1) == 1 && c.stride(1) == 1 && (b_mn ? b.size(0) : b.size(1)) == K && c.size(0) == M && c.size(1) == N);
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    const int rc = tb::ag_gemm_bf16(make_ctx(peers, mc, rank, world, limit), a_off, g_off, (uint32_t)epoch, b.data_ptr(),
                                    c.data_ptr(), (int)M, (int)N, (int)K, b.stride(0), c.stride(0), b_mn, sms, cs());
    TORCH_CHECK(rc == 0, "ag_gemm failed with code ", rc);
  });
  m.def("gemm_rs", [](std::vector<int64_t> peers, int64_t mc, int64_t rank, int64_t world, int64_t limit,
                      torch::Tensor a, torch::Tensor b, int64_t c_off, bool b_mn) {
    const int64_t N = b_mn ? b.size(1) : b.size(0);
    TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && a.size(1) == (b_mn ? b.size(0) : b.size(1)));
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    const int rc = tb::gemm_rs_bf16(make_ctx(peers, mc, rank, world, limit), a.data_ptr(), b.data_ptr(), c_off,
                                    (int)a.size(0), (int)N, (int)a.size(1), a.stride(0), b.stride(0), b_mn, sms, cs());
    TORCH_CHECK(rc == 0, "gemm_rs failed with code ", rc);
  });
  m.def("comm_barrier", [](std::vector<int64_t> peers, int64_t mc, int64_t rank, int64_t world, int64_t limit,
                           int64_t pretend_world, int64_t phase) {
    TORCH_CHECK(phase >= 0 && phase < 8, "barrier phase 0..7");
    tb::comm_barrier(make_ctx(peers, mc, rank, world, limit), (int)phase, (int)pretend_world, cs());
  }, pybind11::arg("peers"), pybind11::arg("mc"), pybind11::arg("rank"), pybind11::arg("world"), pybind11::arg("limit"),
     pybind11::arg("pretend_world"), pybind11::arg("phase") = 0);
}
