// C++ op API with the reference's signatures, on top of the C ABI.
//
// Header-only mirror of moe_cuda::kernels::* (csrc/kernels/internal_api.hpp:20-87)
// and moe_cuda::api::* (csrc/apis/moe.hpp:19-153) of the reference: the same
// function names, argument order and at::Tensor& types, so that callers of
// the reference's C++ API (its pybind module csrc/python_api.cpp, its tests
// test/test_cpp/test_kernel{2,3}.cpp) compile against this header unchanged.
// Every function forwards to libmoe_cuda_b200.so (include/moe_cuda_b200.h) and
// throws std::runtime_error where the reference prints and exits
// (moe_cuda/include/moe_cuda/error.hpp:11-22).
//
// Expert parallel: All2AllBase / make_all2all / naive_moe_forward_dispatch
// (csrc/all2all/all2all_base.hpp:11-52) over the C-ABI context moeb_ep_*; the
// caller hands make_all2all the peer-mapped symmetric buffers, which the
// reference obtains from ThunderKittens' TKParallelTensor.
//
// Not provided: GemmType::Batched, and the at::Tensor forms of
// fused_dispatch_grouped_gemm_swiglu / fused_grouped_gemm_combine with
// TKParallelTensor arguments (internal_api.hpp:63-85): moeb_ep_fused_dispatch_swiglu
// / moeb_ep_fused_gemm_combine take the context instead, and the Python module
// offers the reference's 31- / 21-argument forms.
#pragma once

#include <cuda_runtime_api.h>
#include <torch/types.h>

#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#include "moe_cuda_b200.h"

// moe_cuda/include/moe_cuda/types.h:2-10; values match MOEB_GEMM_*.
#ifndef MOE_CUDA_B200_HAVE_GEMMTYPE
#define MOE_CUDA_B200_HAVE_GEMMTYPE
enum class GemmType {
  Normal = 0,
  MGroupedContiguous,
  MGroupedMasked,
  Batched,
};
#endif

namespace moe_cuda {

namespace detail {
inline void check(int rc, const char *who) {
  if (rc != 0)
    throw std::runtime_error(std::string(who) + ": " + moeb_status_string(rc) + " (" +
                             moeb_last_error() + ")");
}
inline void need(bool ok, const char *msg) {
  if (!ok) throw std::invalid_argument(msg);
}
inline int64_t rows_of(const at::Tensor &t) { return t.numel() / t.size(-1); }
// activation scales as [K/128, rows] fp32; a [rows, K/128] tensor is transposed
// the way api::fp8_gemm_nt does (csrc/apis/moe.hpp:30)
inline at::Tensor mn_major_scale(const at::Tensor &s, int64_t rows, int64_t n_kb) {
  need(s.scalar_type() == at::kFloat && s.numel() == rows * n_kb, "activation scale shape/dtype");
  if (s.dim() >= 2 && s.size(-2) == n_kb) return s.contiguous();
  return s.reshape({rows, n_kb}).t().contiguous();
}
struct GemmDims {
  int m_total, N, K, G, max_m;
};
inline GemmDims gemm_dims(const at::Tensor &A, const at::Tensor &W, GemmType type) {
  need(W.dim() == 3, "weights must be [G, N, K]");
  GemmDims d{};
  d.G = (int)W.size(0);
  d.N = (int)W.size(1);
  d.K = (int)W.size(2);
  if (type == GemmType::MGroupedMasked) {
    need(A.dim() == 3 && A.size(0) == d.G && A.size(2) == d.K,
         "masked layout takes A of shape [G, max_m, K]");
    d.max_m = (int)A.size(1);
    d.m_total = d.G * d.max_m;
  } else {
    need(A.dim() == 2 && A.size(1) == d.K, "contiguous layout takes A of shape [M, K]");
    d.m_total = (int)A.size(0);
  }
  return d;
}
}  // namespace detail

namespace kernels {

// internal_api.hpp:20-23 / csrc/kernels/cast.cuh:283-347 (bf16 -> e4m3, 1x128 scales,
// row-major [rows, H/128] like the reference kernel writes them)
inline void cast(at::Tensor &inp, at::Tensor &out, std::optional<at::Tensor> &scale,
                 cudaStream_t stream) {
  detail::need(inp.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kFloat8_e4m3fn &&
                   scale.has_value(),
               "cast: only bfloat16 -> float8_e4m3fn with a scale tensor is on the MoE path");
  const int H = (int)inp.size(-1);
  const int rows = (int)detail::rows_of(inp);
  const bool mn_major = scale->dim() >= 2 && scale->size(-2) == H / 128 &&
                        scale->size(-1) == rows && !(scale->size(-1) == H / 128);
  detail::check(moeb_cast_bf16_to_e4m3(inp.data_ptr(), out.data_ptr(), scale->data_ptr<float>(),
                                       rows, H, mn_major ? 1 : 0, stream),
                "cast");
}
inline void cast(at::Tensor &inp, at::Tensor &out, cudaStream_t stream) {
  std::optional<at::Tensor> none;
  cast(inp, out, none, stream);
}

// internal_api.hpp:25-26 / src/moe_ops.cu:38-50
inline void fused_silu_mul_quant(at::Tensor &gemm_out, at::Tensor &swiglu_out, at::Tensor &scale,
                                 cudaStream_t stream) {
  const int I = (int)gemm_out.size(-1) / 2;
  const int rows = (int)detail::rows_of(gemm_out);
  detail::check(moeb_fused_silu_mul_quant(gemm_out.data_ptr(), swiglu_out.data_ptr(),
                                          scale.data_ptr<float>(), rows, I, 0, stream),
                "fused_silu_mul_quant");
}

// internal_api.hpp:33-38 -> api::fp8_grouped_gemm_swiglu (moe.hpp:100-118) -> kernel3
inline void fp8_grouped_gemm_swiglu(at::Tensor &A, at::Tensor &gate_weight, at::Tensor &up_weight,
                                    at::Tensor &scale_a, at::Tensor &scale_gate,
                                    at::Tensor &scale_up, at::Tensor &scale_d, at::Tensor &D,
                                    GemmType gemm_type, int *grouped_layout,
                                    cudaStream_t &stream) {
  detail::need(grouped_layout != nullptr,
               "grouped_layout cannot be null for grouped FP8 swiglu GEMM");
  detail::need(gemm_type == GemmType::MGroupedContiguous || gemm_type == GemmType::MGroupedMasked,
               "fp8_grouped_gemm_swiglu supports MGroupedContiguous and MGroupedMasked");
  const detail::GemmDims d = detail::gemm_dims(A, gate_weight, gemm_type);
  at::Tensor sa = detail::mn_major_scale(scale_a, d.m_total, d.K / 128);
  detail::check(moeb_fp8_grouped_gemm_swiglu(
                    A.data_ptr(), sa.data_ptr<float>(), gate_weight.data_ptr(),
                    scale_gate.data_ptr<float>(), up_weight.data_ptr(), scale_up.data_ptr<float>(),
                    D.data_ptr(), scale_d.data_ptr<float>(), d.m_total, d.N, d.K, d.G,
                    static_cast<int>(gemm_type), grouped_layout, d.max_m, nullptr, stream),
                "fp8_grouped_gemm_swiglu");
}
// kernel3_sub and kernel4 (ping-pong) are other schedules of the same computation
// (internal_api.hpp:40-51); here they are the same kernel.
inline void fp8_grouped_gemm_swiglu_sub(at::Tensor &A, at::Tensor &gate_weight,
                                        at::Tensor &up_weight, at::Tensor &scale_a,
                                        at::Tensor &scale_gate, at::Tensor &scale_up,
                                        at::Tensor &scale_d, at::Tensor &D, GemmType gemm_type,
                                        int *grouped_layout, cudaStream_t &stream) {
  fp8_grouped_gemm_swiglu(A, gate_weight, up_weight, scale_a, scale_gate, scale_up, scale_d, D,
                          gemm_type, grouped_layout, stream);
}
inline void fp8_grouped_gemm_swiglu_consumer_pp(at::Tensor &A, at::Tensor &gate_weight,
                                                at::Tensor &up_weight, at::Tensor &scale_a,
                                                at::Tensor &scale_gate, at::Tensor &scale_up,
                                                at::Tensor &scale_d, at::Tensor &D,
                                                GemmType gemm_type, int *grouped_layout,
                                                cudaStream_t &stream) {
  fp8_grouped_gemm_swiglu(A, gate_weight, up_weight, scale_a, scale_gate, scale_up, scale_d, D,
                          gemm_type, grouped_layout, stream);
}

// internal_api.hpp:53-56 -> api::fp8_grouped_gemm (moe.hpp:51-70) -> kernel2
inline void fp8_grouped_gemm_nt(at::Tensor &act, at::Tensor &act_scale, at::Tensor &weight,
                                at::Tensor &weight_scale, at::Tensor &output, GemmType gemm_type,
                                int *grouped_layout, cudaStream_t &stream) {
  detail::need(grouped_layout != nullptr, "grouped_layout cannot be null for grouped FP8 GEMM");
  detail::need(gemm_type == GemmType::MGroupedContiguous || gemm_type == GemmType::MGroupedMasked,
               "fp8_grouped_gemm only supports MGroupedContiguous and MGroupedMasked");
  const detail::GemmDims d = detail::gemm_dims(act, weight, gemm_type);
  const bool f32 = output.scalar_type() == at::kFloat;
  detail::need(f32 || output.scalar_type() == at::kBFloat16, "output must be bf16 or fp32");
  at::Tensor sa = detail::mn_major_scale(act_scale, d.m_total, d.K / 128);
  detail::check(moeb_fp8_grouped_gemm_nt(act.data_ptr(), sa.data_ptr<float>(), weight.data_ptr(),
                                         weight_scale.data_ptr<float>(), output.data_ptr(),
                                         f32 ? MOEB_OUT_F32 : MOEB_OUT_BF16, d.m_total, d.N, d.K,
                                         d.G, static_cast<int>(gemm_type), grouped_layout, d.max_m,
                                         nullptr, stream),
                "fp8_grouped_gemm_nt");
}

// internal_api.hpp:58-61 -> api::fp8_gemm_nt (moe.hpp:19-49). GemmType::Normal runs
// as a grouped GEMM with one group (weight [N,K] or [1,N,K]); the grouped types
// forward to fp8_grouped_gemm_nt; Batched is not built.
inline void fp8_gemm_nt(at::Tensor &act, at::Tensor &act_scale, at::Tensor &weight,
                        at::Tensor &weight_scale, at::Tensor &output, GemmType gemm_type,
                        const std::string & /*compiled_dims*/, int *grouped_layout,
                        cudaStream_t &stream) {
  if (gemm_type == GemmType::MGroupedContiguous || gemm_type == GemmType::MGroupedMasked) {
    fp8_grouped_gemm_nt(act, act_scale, weight, weight_scale, output, gemm_type, grouped_layout,
                        stream);
    return;
  }
  detail::need(gemm_type == GemmType::Normal, "fp8_gemm_nt: GemmType::Batched is not built");
  detail::need(act.dim() == 2 && (weight.dim() == 2 || (weight.dim() == 3 && weight.size(0) == 1)),
               "fp8_gemm_nt takes act [M,K] and weight [N,K]");
  const int M = (int)act.size(0), K = (int)act.size(1), N = (int)weight.size(-2);
  detail::need(weight.size(-1) == K && output.numel() == (int64_t)M * N, "shape mismatch");
  const bool f32 = output.scalar_type() == at::kFloat;
  detail::need(f32 || output.scalar_type() == at::kBFloat16, "output must be bf16 or fp32");
  at::Tensor sa = detail::mn_major_scale(act_scale, M, K / 128);
  at::Tensor layout = at::zeros({M > 0 ? M : 1}, act.options().dtype(at::kInt));
  detail::check(moeb_fp8_grouped_gemm_nt(act.data_ptr(), sa.data_ptr<float>(), weight.data_ptr(),
                                         weight_scale.data_ptr<float>(), output.data_ptr(),
                                         f32 ? MOEB_OUT_F32 : MOEB_OUT_BF16, M, N, K, 1,
                                         MOEB_GEMM_M_GROUPED_CONTIGUOUS, layout.data_ptr<int>(), 0,
                                         nullptr, stream),
                "fp8_gemm_nt");
}
// internal_api.hpp:58-61 -> api::bf16_gemm (moe.hpp:72-98). C is accepted and
// ignored, as in the reference; Batched is not built.
inline void bf16_gemm(at::Tensor &A, at::Tensor &B, std::optional<at::Tensor> & /*C*/, at::Tensor &D,
                      GemmType gemm_type, const std::string & /*compiled_dims*/, int *grouped_layout,
                      cudaStream_t &stream) {
  detail::need(gemm_type != GemmType::Batched, "bf16_gemm: GemmType::Batched is not built");
  detail::need(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16,
               "bf16_gemm takes bfloat16 operands");
  const bool f32 = D.scalar_type() == at::kFloat;
  detail::need(f32 || D.scalar_type() == at::kBFloat16, "D must be bf16 or fp32");
  int m_total, N, K, G = 1, max_m = 0;
  if (gemm_type == GemmType::Normal) {
    detail::need(A.dim() == 2 && (B.dim() == 2 || (B.dim() == 3 && B.size(0) == 1)),
                 "bf16_gemm takes A [M,K] and B [N,K]");
    m_total = (int)A.size(0);
    K = (int)A.size(1);
    N = (int)B.size(-2);
    detail::need(B.size(-1) == K, "A and B disagree on K");
  } else {
    detail::need(grouped_layout != nullptr, "grouped_layout cannot be null for grouped BF16 GEMM");
    const detail::GemmDims d = detail::gemm_dims(A, B, gemm_type);
    m_total = d.m_total, N = d.N, K = d.K, G = d.G, max_m = d.max_m;
  }
  detail::need(D.numel() == (int64_t)m_total * N, "D has the wrong number of elements");
  detail::check(moeb_bf16_gemm(A.data_ptr(), B.data_ptr(), D.data_ptr(),
                               f32 ? MOEB_OUT_F32 : MOEB_OUT_BF16, m_total, N, K, G,
                               static_cast<int>(gemm_type), grouped_layout, max_m, nullptr, stream),
                "bf16_gemm");
}

}  // namespace kernels

namespace api {
// csrc/apis/moe.hpp: thin dispatchers by GemmType; same behaviour as kernels::*
using kernels::fp8_grouped_gemm_swiglu;
using kernels::fp8_grouped_gemm_swiglu_consumer_pp;
using kernels::fp8_grouped_gemm_swiglu_sub;
inline void fp8_grouped_gemm(at::Tensor &act, at::Tensor &act_scale, at::Tensor &weight,
                             at::Tensor &weight_scale, at::Tensor &output, GemmType gemm_type,
                             int *grouped_layout, cudaStream_t &stream) {
  kernels::fp8_grouped_gemm_nt(act, act_scale, weight, weight_scale, output, gemm_type,
                               grouped_layout, stream);
}
}  // namespace api

// One-GPU whole layer (the W = 1 form of naive_moe_forward, src/moe_ops.cu:153-191,
// with the router in front). `workspace` is a uint8 CUDA tensor of at least
// moeb_moe_forward_workspace_bytes(cfg) bytes.
inline void moe_forward(const moeb_layer_config &cfg, at::Tensor &x, at::Tensor &w_router,
                        std::optional<at::Tensor> router_bias, at::Tensor &gate,
                        at::Tensor &gate_scale, at::Tensor &up, at::Tensor &up_scale,
                        at::Tensor &down, at::Tensor &down_scale, at::Tensor &out,
                        at::Tensor &workspace, cudaStream_t stream) {
  detail::check(
      moeb_moe_forward(&cfg, x.data_ptr(), w_router.data_ptr(),
                       router_bias.has_value() ? router_bias->data_ptr<float>() : nullptr,
                       gate.data_ptr(), gate_scale.data_ptr<float>(), up.data_ptr(),
                       up_scale.data_ptr<float>(), down.data_ptr(), down_scale.data_ptr<float>(),
                       out.data_ptr(), nullptr, nullptr, workspace.data_ptr(),
                       (size_t)workspace.numel(), nullptr, stream),
      "moe_forward");
}

// ---- expert parallel ---------------------------------------------------------
// csrc/runtime/parallel.h:3-9
struct ParallelConfig {
  uint32_t tp_size;
  uint32_t dp_size;
  uint32_t ep_size;
  uint32_t node_size;
  uint32_t world_size;
};

// csrc/all2all/all2all_base.hpp:11-31
class All2AllBase {
 public:
  All2AllBase() = default;
  virtual ~All2AllBase() = default;
  virtual void dispatch(at::Tensor &out_expert_num_tokens, at::Tensor &out_expert_x,
                        std::optional<at::Tensor> &out_expert_x_scale, at::Tensor &dp_x,
                        std::optional<at::Tensor> &dp_x_scale, at::Tensor &indices,
                        at::Tensor &weights, std::optional<at::Tensor> &bound_m,
                        bool do_send = true, bool do_recv = true,
                        cudaStream_t stream = nullptr) = 0;
  virtual void combine(at::Tensor &out_tokens, at::Tensor &indices, at::Tensor &weights,
                       at::Tensor &expert_y, std::optional<at::Tensor> &bound_m,
                       bool do_send = true, bool do_recv = true, bool accumulate = false,
                       cudaStream_t stream = nullptr) = 0;
  virtual uint32_t max_recv_tokens() const = 0;
  // per-row expert id (-1 padding) of the rows the last dispatch delivered: the
  // grouped layout of the MGroupedContiguous GEMMs
  virtual int *grouped_layout() const = 0;
};

// All2AllBase over the C-ABI context. The symmetric buffers (one per rank, each
// moeb_ep_symmetric_bytes(cfg) bytes, mapped into this process) and the local
// workspace are the caller's; `local_workspace` is kept alive by this object.
class All2AllContext final : public All2AllBase {
 public:
  All2AllContext(const moeb_ep_config &cfg, const std::vector<uint64_t> &peer_base,
                 at::Tensor local_workspace, cudaStream_t stream)
      : cfg_(cfg), local_(std::move(local_workspace)) {
    detail::need((int)peer_base.size() == cfg.world, "one symmetric buffer address per rank");
    detail::check(moeb_ep_create(&cfg_, peer_base.data(), local_.data_ptr(),
                                 (size_t)local_.numel() * local_.element_size(), stream, &ctx_),
                  "All2All");
    detail::check(moeb_ep_get_view(ctx_, &view_), "All2All");
  }
  ~All2AllContext() override { moeb_ep_destroy(ctx_); }
  All2AllContext(const All2AllContext &) = delete;
  All2AllContext &operator=(const All2AllContext &) = delete;

  void dispatch(at::Tensor &out_expert_num_tokens, at::Tensor &out_expert_x,
                std::optional<at::Tensor> &out_expert_x_scale, at::Tensor &dp_x,
                std::optional<at::Tensor> &dp_x_scale, at::Tensor &indices, at::Tensor &weights,
                std::optional<at::Tensor> &bound_m, bool do_send = true, bool do_recv = true,
                cudaStream_t stream = nullptr) override {
    (void)weights;
    (void)bound_m;   // validated and unused by the reference as well (all2all_tk.hpp:284-290)
    if (do_send) {
      // all2all_tk.hpp:298,327: both scale tensors are dereferenced unconditionally
      detail::need(dp_x_scale.has_value() && out_expert_x_scale.has_value(),
                   "dp_x_scale and out_expert_x_scale are required");
      detail::need(indices.scalar_type() == at::kInt, "indices must be int32 [T, k]");
    }
    detail::check(
        moeb_ep_dispatch(ctx_, nullptr, do_send ? dp_x.data_ptr() : nullptr,
                         do_send ? dp_x_scale->data_ptr<float>() : nullptr,
                         do_send ? indices.data_ptr<int>() : nullptr,
                         do_send ? (int)dp_x.size(0) : 0, do_send ? out_expert_x.data_ptr() : nullptr,
                         do_send ? out_expert_x_scale->data_ptr<float>() : nullptr,
                         do_send ? (int)out_expert_x.size(0) : 0, do_send, do_recv, nullptr, stream),
        "All2All::dispatch");
    if (do_send)   // unpadded rows per local expert (all2all_tk.hpp:216-219,317-320)
      cudaMemcpyAsync(out_expert_num_tokens.data_ptr(), view_.tokens_per_expert,
                      sizeof(int32_t) * view_.local_experts, cudaMemcpyDeviceToDevice, stream);
  }
  void combine(at::Tensor &out_tokens, at::Tensor &indices, at::Tensor &weights,
               at::Tensor &expert_y, std::optional<at::Tensor> &bound_m, bool do_send = true,
               bool do_recv = true, bool accumulate = false,
               cudaStream_t stream = nullptr) override {
    (void)indices;
    (void)bound_m;
    detail::need(expert_y.scalar_type() == at::kBFloat16 && out_tokens.scalar_type() == at::kBFloat16,
                 "combine only supports bfloat16");   // a2a_context_tk.hpp:181-182
    detail::check(moeb_ep_combine(ctx_, expert_y.data_ptr(), weights.data_ptr<float>(),
                                  out_tokens.data_ptr(), accumulate, do_send, do_recv, nullptr,
                                  stream),
                  "All2All::combine");
  }
  uint32_t max_recv_tokens() const override { return (uint32_t)view_.max_recv_rows; }
  int *grouped_layout() const override { return view_.grouped_layout; }
  moeb_ep_ctx *handle() const { return ctx_; }

 private:
  moeb_ep_config cfg_;
  at::Tensor local_;
  moeb_ep_ctx *ctx_ = nullptr;
  moeb_ep_view view_{};
};

// csrc/all2all/all2all_base.hpp:33-41. The reference's version allocates its
// parallel tensors itself; this one is given them: `peer_base` holds the address
// of every rank's symmetric buffer (moeb_ep_symmetric_bytes bytes each) in this
// process. in/out/scale dtypes are e4m3 / bf16 / fp32 (the only ones the
// reference's transport supports, a2a_context_tk.hpp:181-195); dp_size must be 1.
// (make_all2all_ranked: CUDA device and rank given separately; make_all2all below
// takes local_rank for both, as the reference does.)
inline std::shared_ptr<All2AllBase> make_all2all_ranked(
    uint32_t max_num_tokens, uint32_t num_experts, uint32_t experts_per_token,
    uint32_t expert_padding, uint32_t hidden_dim, std::optional<uint32_t> hidden_dim_scale,
    c10::ScalarType in_dtype, c10::ScalarType out_dtype, std::optional<c10::ScalarType> scale_dtype,
    std::optional<uint32_t> max_private_tokens_opt, int device, int rank,
    ParallelConfig parallel_config, const std::vector<uint64_t> &peer_base, cudaStream_t stream) {
  (void)hidden_dim_scale;
  (void)max_private_tokens_opt;   // no private / overflow split in this transport
  detail::need(in_dtype == at::kFloat8_e4m3fn && out_dtype == at::kBFloat16 &&
                   (!scale_dtype.has_value() || *scale_dtype == at::kFloat),
               "All2All moves e4m3 tokens with fp32 scales out and bf16 rows back");
  detail::need(parallel_config.dp_size <= 1, "dp_size must be 1");
  moeb_ep_config cfg{(int)max_num_tokens, (int)hidden_dim,        (int)num_experts,
                     (int)experts_per_token, (int)expert_padding, (int)parallel_config.world_size,
                     rank,                0,                   0};
  const size_t bytes = moeb_ep_local_bytes(&cfg);
  detail::need(bytes > 0, "bad expert-parallel configuration");
  at::Tensor ws = at::empty({(int64_t)bytes},
                            at::TensorOptions().dtype(at::kByte).device(at::kCUDA, device));
  return std::make_shared<All2AllContext>(cfg, peer_base, ws, stream);
}

inline std::shared_ptr<All2AllBase> make_all2all(
    uint32_t max_num_tokens, uint32_t num_experts, uint32_t experts_per_token,
    uint32_t expert_padding, uint32_t hidden_dim, std::optional<uint32_t> hidden_dim_scale,
    c10::ScalarType in_dtype, c10::ScalarType out_dtype, std::optional<c10::ScalarType> scale_dtype,
    std::optional<uint32_t> max_private_tokens_opt, int local_rank, ParallelConfig parallel_config,
    const std::vector<uint64_t> &peer_base, cudaStream_t stream) {
  return make_all2all_ranked(max_num_tokens, num_experts, experts_per_token, expert_padding,
                             hidden_dim, hidden_dim_scale, in_dtype, out_dtype, scale_dtype,
                             max_private_tokens_opt, local_rank, local_rank, parallel_config,
                             peer_base, stream);
}

// csrc/all2all/all2all_base.hpp:43-52 -> src/moe_ops.cu:153-239: dispatch -> gate/up
// SwiGLU grouped GEMM -> down grouped GEMM -> combine on the caller's buffers.
// The GEMMs get the per-row expert ids of the dispatch as their layout.
inline void naive_moe_forward_dispatch(All2AllBase &a2a, uint32_t num_experts,
                                       uint32_t experts_per_token, uint32_t hidden_dim,
                                       GemmType gemm_type, at::Tensor &input,
                                       at::Tensor &input_scales, at::Tensor &gate,
                                       at::Tensor &gate_scales, at::Tensor &up,
                                       at::Tensor &up_scales, at::Tensor &down,
                                       at::Tensor &down_scales, at::Tensor &indices,
                                       at::Tensor &weights, at::Tensor &out_tokens,
                                       at::Tensor &expert_x, at::Tensor &expert_x_scales,
                                       at::Tensor &inter_y, at::Tensor &inter_y_scales,
                                       at::Tensor &expert_y, cudaStream_t stream) {
  (void)num_experts;
  (void)experts_per_token;
  (void)hidden_dim;
  detail::need(gemm_type == GemmType::MGroupedContiguous,
               "the dispatch delivers the contiguous layout");
  at::Tensor counts = at::empty({(int64_t)gate.size(0)}, indices.options());
  std::optional<at::Tensor> xs(expert_x_scales), is(input_scales), none;
  a2a.dispatch(counts, expert_x, xs, input, is, indices, weights, none, true, true, stream);
  kernels::fp8_grouped_gemm_swiglu(expert_x, gate, up, expert_x_scales, gate_scales, up_scales,
                                   inter_y_scales, inter_y, gemm_type, a2a.grouped_layout(), stream);
  kernels::fp8_grouped_gemm_nt(inter_y, inter_y_scales, down, down_scales, expert_y, gemm_type,
                               a2a.grouped_layout(), stream);
  a2a.combine(out_tokens, indices, weights, expert_y, none, true, true, false, stream);
}

}  // namespace moe_cuda
