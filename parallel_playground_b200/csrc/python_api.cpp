// pybind11 module `moe_cuda_b200_ext`: the compiled twin of the reference's
// torch extension (csrc/python_api.cpp:170-532) for the ops on the MoE hot
// path, the All2All class and naive_moe_forward_dispatch included. Same function names, positional order and keyword names; every op runs
// on the current CUDA stream (python_api.cpp:26-28) and returns None. The
// bodies only forward to include/moe_cuda_b200_torch.hpp, i.e. to the C ABI.
//
// The ctypes module parallel_playground_b200/moe_cuda.py offers the same names
// without a C++ compile step; this module exists for callers that link the
// reference's C++ API (at::Tensor signatures).
#include <ATen/cuda/CUDAContext.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "moe_cuda_b200_torch.hpp"

namespace {

cudaStream_t current_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_layout(const at::Tensor &grouped_layout, const at::Tensor &D, const at::Tensor &scale_d) {
  if (grouped_layout.scalar_type() != at::ScalarType::Int)
    throw std::invalid_argument("invalid grouped layout type");  // python_api.cpp:257
  if (D.size(-1) / 128 != scale_d.size(-2))
    throw std::invalid_argument("incorrect output scale d layout");  // python_api.cpp:259
}

void swiglu(at::Tensor &A, at::Tensor &scale_a, at::Tensor &gate_weight, at::Tensor &gate_scale,
            at::Tensor &up_weight, at::Tensor &up_scale, at::Tensor &D, at::Tensor &scale_d,
            GemmType gemm_type, at::Tensor &grouped_layout) {
  check_layout(grouped_layout, D, scale_d);
  auto stream = current_stream();
  moe_cuda::kernels::fp8_grouped_gemm_swiglu(A, gate_weight, up_weight, scale_a, gate_scale,
                                             up_scale, scale_d, D, gemm_type,
                                             grouped_layout.data_ptr<int>(), stream);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "MoE CUDA kernels for B200 (sm_100a): compiled twin of the reference's moe_cuda module";
  namespace py = pybind11;

  py::enum_<GemmType>(m, "GemmType")
      .value("Normal", GemmType::Normal)
      .value("MGroupedContiguous", GemmType::MGroupedContiguous)
      .value("MGroupedMasked", GemmType::MGroupedMasked)
      .value("Batched", GemmType::Batched)
      .export_values();

  m.def("init", [](const std::string &, const std::string &) { (void)moeb_abi_version(); },
        py::arg("library_root"), py::arg("cuda_home"),
        "Kept for compatibility; this build has no JIT paths to set.");

  m.def(
      "fp8_grouped_gemm_nt",
      [](at::Tensor &act, at::Tensor &act_scale, at::Tensor &weight, at::Tensor &weight_scale,
         at::Tensor &output, GemmType gemm_type, at::Tensor grouped_layout) {
        auto stream = current_stream();
        moe_cuda::kernels::fp8_grouped_gemm_nt(act, act_scale, weight, weight_scale, output,
                                               gemm_type, grouped_layout.data_ptr<int>(), stream);
      },
      py::arg("act"), py::arg("act_scale"), py::arg("weight"), py::arg("weight_scale"),
      py::arg("output"), py::arg("gemm_type"), py::arg("grouped_layout"));

  // python_api.cpp:192-211 of the reference
  m.def(
      "bf16_gemm",
      [](at::Tensor &a, at::Tensor &b, at::Tensor &d, std::optional<at::Tensor> c,
         GemmType gemm_type, const std::string &compiled_dims,
         std::optional<at::Tensor> grouped_layout) {
        auto stream = current_stream();
        int *layout_ptr = grouped_layout.has_value() ? grouped_layout->data_ptr<int>() : nullptr;
        moe_cuda::kernels::bf16_gemm(a, b, c, d, gemm_type, compiled_dims, layout_ptr, stream);
      },
      py::arg("a"), py::arg("b"), py::arg("d"), py::arg("c") = py::none(),
      py::arg("gemm_type") = GemmType::Normal, py::arg("compiled_dims") = "",
      py::arg("grouped_layout") = py::none());

  // python_api.cpp:213-231 of the reference
  m.def(
      "fp8_gemm_nt",
      [](at::Tensor &act, at::Tensor &act_scale, at::Tensor &weight, at::Tensor &weight_scale,
         at::Tensor &output, GemmType gemm_type, const std::string &compiled_dims,
         std::optional<at::Tensor> grouped_layout) {
        auto stream = current_stream();
        int *layout_ptr = grouped_layout.has_value() ? grouped_layout->data_ptr<int>() : nullptr;
        moe_cuda::kernels::fp8_gemm_nt(act, act_scale, weight, weight_scale, output, gemm_type,
                                       compiled_dims, layout_ptr, stream);
      },
      py::arg("act"), py::arg("act_scale"), py::arg("weight"), py::arg("weight_scale"),
      py::arg("output"), py::arg("gemm_type") = GemmType::Normal, py::arg("compiled_dims") = "",
      py::arg("grouped_layout") = py::none());

  const char *names_typed[] = {"fp8_grouped_gemm_swiglu", "fp8_grouped_gemm_swiglu_sub",
                               "fp8_grouped_gemm_swiglu_pp"};
  for (const char *name : names_typed)
    m.def(name, &swiglu, py::arg("A"), py::arg("scale_a"), py::arg("gate_weight"),
          py::arg("gate_scale"), py::arg("up_weight"), py::arg("up_scale"), py::arg("D"),
          py::arg("scale_d"), py::arg("gemm_type"), py::arg("grouped_layout"));

  struct Fixed {
    const char *name;
    GemmType type;
  };
  const Fixed fixed[] = {
      {"fp8_grouped_gemm_swiglu_contiguous", GemmType::MGroupedContiguous},
      {"fp8_grouped_gemm_swiglu_masked", GemmType::MGroupedMasked},
      {"fp8_grouped_gemm_swiglu_sub_contiguous", GemmType::MGroupedContiguous},
      {"fp8_grouped_gemm_swiglu_sub_masked", GemmType::MGroupedMasked},
      {"fp8_grouped_gemm_swiglu_contiguous_pp", GemmType::MGroupedContiguous},
      {"fp8_grouped_gemm_swiglu_masked_pp", GemmType::MGroupedMasked},
  };
  for (const Fixed &f : fixed) {
    const GemmType type = f.type;
    m.def(
        f.name,
        [type](at::Tensor &A, at::Tensor &scale_a, at::Tensor &gate_weight, at::Tensor &gate_scale,
               at::Tensor &up_weight, at::Tensor &up_scale, at::Tensor &D, at::Tensor &scale_d,
               at::Tensor &grouped_layout) {
          swiglu(A, scale_a, gate_weight, gate_scale, up_weight, up_scale, D, scale_d, type,
                 grouped_layout);
        },
        py::arg("A"), py::arg("scale_a"), py::arg("gate_weight"), py::arg("gate_scale"),
        py::arg("up_weight"), py::arg("up_scale"), py::arg("D"), py::arg("scale_d"),
        py::arg("grouped_layout"));
  }

  m.def(
      "cast",
      [](at::Tensor &inp, at::Tensor &out, std::optional<at::Tensor> &scale) {
        moe_cuda::kernels::cast(inp, out, scale, current_stream());
      },
      py::arg("inp"), py::arg("out"), py::arg("scale") = py::none());

  m.def(
      "fused_silu_mul_quant",
      [](at::Tensor &gemm_out, at::Tensor &swiglu_out, at::Tensor &scale) {
        moe_cuda::kernels::fused_silu_mul_quant(gemm_out, swiglu_out, scale, current_stream());
      },
      py::arg("gemm_out"), py::arg("swiglu_out"), py::arg("scale"));

  // python_api.cpp:85-166, 477-514 of the reference: class All2All. The reference
  // takes its peer mappings from ThunderKittens; here the caller passes them
  // (`peer_base`: address of every rank's symmetric buffer of `symmetric_bytes`
  // bytes in this process, `rank`, `world_size`).
  m.def("all2all_symmetric_bytes",
        [](int max_num_tokens, int num_experts, int experts_per_token, int expert_padding,
           int hidden_dim, int world_size) {
          moeb_ep_config cfg{max_num_tokens, hidden_dim,  num_experts, experts_per_token,
                             expert_padding, world_size,  0,           0,
                             0};
          return moeb_ep_symmetric_bytes(&cfg);
        });
  py::class_<moe_cuda::All2AllBase, std::shared_ptr<moe_cuda::All2AllBase>>(m, "All2All")
      .def(py::init([](uint32_t max_num_tokens, uint32_t num_experts, uint32_t experts_per_token,
                       uint32_t expert_padding, uint32_t hidden_dim,
                       std::optional<uint32_t> hidden_dim_scale, at::ScalarType in_dtype,
                       at::ScalarType out_dtype, std::optional<at::ScalarType> scale_dtype,
                       std::optional<uint32_t> max_private_tokens,
                       std::optional<uint32_t> dp_group_size,
                       std::optional<uint32_t> node_group_size,
                       std::optional<uint32_t> ep_group_size, int device,
                       const std::vector<uint64_t> &peer_base, int rank) {
             (void)node_group_size;
             (void)ep_group_size;
             if (dp_group_size.has_value() && *dp_group_size != 1)
               throw std::invalid_argument("dp_group_size must divide world size; only 1 is supported");
             const uint32_t world = (uint32_t)peer_base.size();
             moe_cuda::ParallelConfig pc{1, 1, world, world, world};
             if (device < 0) cudaGetDevice(&device);
             (void)rank;
             moe_cuda::ParallelConfig cfg = pc;
             return moe_cuda::make_all2all_ranked(max_num_tokens, num_experts, experts_per_token,
                                                  expert_padding, hidden_dim, hidden_dim_scale,
                                                  in_dtype, out_dtype, scale_dtype,
                                                  max_private_tokens, device, rank, cfg, peer_base,
                                                  current_stream());
           }),
           py::arg("max_num_tokens"), py::arg("num_experts"), py::arg("experts_per_token"),
           py::arg("expert_padding"), py::arg("hidden_dim"),
           py::arg("hidden_dim_scale") = py::none(), py::arg("in_dtype"), py::arg("out_dtype"),
           py::arg("scale_dtype") = py::none(), py::arg("max_private_tokens") = py::none(),
           py::arg("dp_group_size") = py::none(), py::arg("node_group_size") = py::none(),
           py::arg("ep_group_size") = py::none(), py::arg("device") = -1, py::arg("peer_base"),
           py::arg("rank") = 0)
      .def(
          "dispatch",
          [](moe_cuda::All2AllBase &self, at::Tensor &out_expert_num_tokens, at::Tensor &out_expert_x,
             std::optional<at::Tensor> out_expert_x_scale, at::Tensor &dp_x,
             std::optional<at::Tensor> dp_x_scale, at::Tensor &indices, at::Tensor &weights,
             std::optional<at::Tensor> bound_m, bool do_send, bool do_recv) {
            self.dispatch(out_expert_num_tokens, out_expert_x, out_expert_x_scale, dp_x, dp_x_scale,
                          indices, weights, bound_m, do_send, do_recv, current_stream());
          },
          py::arg("out_expert_num_tokens"), py::arg("out_expert_x"),
          py::arg("out_expert_x_scale") = py::none(), py::arg("dp_x"),
          py::arg("dp_x_scale") = py::none(), py::arg("indices"), py::arg("weights"),
          py::arg("bound_m") = py::none(), py::arg("do_send") = true, py::arg("do_recv") = true)
      .def(
          "combine",
          [](moe_cuda::All2AllBase &self, at::Tensor &out_tokens, at::Tensor &indices,
             at::Tensor &weights, at::Tensor &expert_y, std::optional<at::Tensor> bound_m,
             bool do_send, bool do_recv, bool accumulate) {
            self.combine(out_tokens, indices, weights, expert_y, bound_m, do_send, do_recv,
                         accumulate, current_stream());
          },
          py::arg("out_tokens"), py::arg("indices"), py::arg("weights"), py::arg("expert_y"),
          py::arg("bound_m") = py::none(), py::arg("do_send") = true, py::arg("do_recv") = true,
          py::arg("accumulate") = false)
      .def_property_readonly("max_recv_tokens", &moe_cuda::All2AllBase::max_recv_tokens);

  // python_api.cpp:516-532 of the reference, same 21 positional arguments
  m.def("naive_moe_forward_dispatch",
        [](moe_cuda::All2AllBase &all2all, uint32_t num_experts, uint32_t experts_per_token,
           uint32_t hidden_dim, GemmType gemm_type, at::Tensor &input, at::Tensor &input_scales,
           at::Tensor &gate, at::Tensor &gate_scales, at::Tensor &up, at::Tensor &up_scales,
           at::Tensor &down, at::Tensor &down_scales, at::Tensor &indices, at::Tensor &weights,
           at::Tensor &out_tokens, at::Tensor &expert_x, at::Tensor &expert_x_scales,
           at::Tensor &inter_y, at::Tensor &inter_y_scales, at::Tensor &expert_y) {
          moe_cuda::naive_moe_forward_dispatch(all2all, num_experts, experts_per_token, hidden_dim,
                                               gemm_type, input, input_scales, gate, gate_scales, up,
                                               up_scales, down, down_scales, indices, weights,
                                               out_tokens, expert_x, expert_x_scales, inter_y,
                                               inter_y_scales, expert_y, current_stream());
        });
}
