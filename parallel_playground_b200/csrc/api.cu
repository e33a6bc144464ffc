// Error reporting and the one-GPU whole-layer entry points of the C ABI.
//
// moeb_moe_forward is the W=1 form of the reference's naive_moe_forward
// (src/moe_ops.cu:153-191: dispatch -> gate/up SwiGLU GEMM -> down GEMM ->
// combine) with the router in front; with one rank the all-to-all dispatch and
// combine degenerate to a local permute and un-permute.
#include "common.cuh"
#include "moe_cuda_b200.h"

#include <cstdio>
#include <cstring>

namespace moeb {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* what, cudaError_t e) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", what, cudaGetErrorName(e),
           cudaGetErrorString(e));
}
thread_local int tl_status_scopes = 0;

void set_last_error_msg(const char* msg) {
  snprintf(g_last_error, sizeof(g_last_error), "%s", msg);
}

// Workspace carving for moeb_moe_forward; every region is 256-byte aligned.
struct LayerWorkspace {
  size_t logits, router_ws, indices, weights, counts, offsets, dst_row, src_token, src_slot, layout,
      plan_ws, expert_x, expert_x_scale, inter, inter_scale, expert_y, total;
  int m_cap;
  size_t plan_ws_bytes, router_ws_bytes;
};

static size_t align256(size_t x) { return (x + 255) / 256 * 256; }

static bool carve(const moeb_layer_config& c, LayerWorkspace* w) {
  if (c.T < 0 || c.H <= 0 || c.I <= 0 || c.E <= 0 || c.k <= 0 || c.k > c.E || c.H % 128 != 0 ||
      c.I % 128 != 0)
    return false;
  const int m_cap = moeb_route_plan_rows(c.T, c.k, c.E, 128);
  if (m_cap < 0) return false;
  w->m_cap = m_cap;
  w->plan_ws_bytes = moeb_route_plan_workspace_bytes(c.T, c.k, c.E);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off += align256(bytes);
    return at;
  };
  const size_t n_pairs = (size_t)c.T * c.k;
  w->logits = take((size_t)c.T * c.E * 4);
  w->router_ws_bytes = moeb_router_logits_workspace_bytes(c.T, c.H, c.E);
  w->router_ws = take(w->router_ws_bytes);
  w->indices = take(n_pairs * 4);
  w->weights = take(n_pairs * 4);
  w->counts = take((size_t)c.E * 4);
  w->offsets = take((size_t)(c.E + 1) * 4);
  w->dst_row = take(n_pairs * 4);
  w->src_token = take((size_t)m_cap * 4);
  w->src_slot = take((size_t)m_cap * 4);
  w->layout = take((size_t)m_cap * 4);
  w->plan_ws = take(w->plan_ws_bytes);
  w->expert_x = take((size_t)m_cap * c.H);
  w->expert_x_scale = take((size_t)m_cap * (c.H / 128) * 4);
  w->inter = take((size_t)m_cap * c.I);
  w->inter_scale = take((size_t)m_cap * (c.I / 128) * 4);
  w->expert_y = take((size_t)m_cap * c.H * 2);
  w->total = off;
  return true;
}

}  // namespace moeb

using namespace moeb;

extern "C" int moeb_abi_version(void) { return 1; }

extern "C" const char* moeb_status_string(int status) {
  switch (status) {
    case kOk: return "ok";
    case kInvalidArgument: return "invalid argument";
    case kCudaError: return "CUDA error";
    case kNotImplemented: return "not implemented";
    case kDeviceTimeout: return "a bounded device-side wait expired";
    case kUnsupportedShape: return "unsupported shape";
    case kNoDriverEntry: return "driver entry point unavailable";
    case kTooLarge: return "size exceeds a fixed limit";
    default: return "unknown status";
  }
}

extern "C" const char* moeb_last_error(void) { return g_last_error; }

extern "C" size_t moeb_moe_forward_workspace_bytes(const moeb_layer_config* cfg) {
  LayerWorkspace w;
  if (!cfg || !carve(*cfg, &w)) return 0;
  return w.total;
}

extern "C" int moeb_moe_forward(const moeb_layer_config* cfg, const void* x_bf16,
                                const void* w_router_bf16, const float* router_bias,
                                const void* gate_q,
                                const float* gate_scale, const void* up_q, const float* up_scale,
                                const void* down_q, const float* down_scale, void* out_bf16,
                                int32_t* indices_out, float* weights_out, void* workspace,
                                size_t workspace_bytes, int32_t* status_dev, void* stream) {
  LayerWorkspace w;
  if (!cfg || !carve(*cfg, &w)) {
    set_last_error_msg("moeb_moe_forward: bad layer configuration (H, I multiples of 128; k <= E)");
    return kInvalidArgument;
  }
  if (!x_bf16 || !w_router_bf16 || !gate_q || !gate_scale || !up_q || !up_scale || !down_q ||
      !down_scale || !out_bf16 || !workspace) {
    set_last_error_msg("moeb_moe_forward: null pointer");
    return kInvalidArgument;
  }
  if (workspace_bytes < w.total || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) {
    set_last_error_msg("moeb_moe_forward: workspace too small or not 256-byte aligned");
    return kInvalidArgument;
  }
  const moeb_layer_config& c = *cfg;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  float* logits = reinterpret_cast<float*>(ws + w.logits);
  int32_t* indices = reinterpret_cast<int32_t*>(ws + w.indices);
  float* weights = reinterpret_cast<float*>(ws + w.weights);
  int32_t* counts = reinterpret_cast<int32_t*>(ws + w.counts);
  int32_t* offsets = reinterpret_cast<int32_t*>(ws + w.offsets);
  int32_t* dst_row = reinterpret_cast<int32_t*>(ws + w.dst_row);
  int32_t* src_token = reinterpret_cast<int32_t*>(ws + w.src_token);
  int32_t* src_slot = reinterpret_cast<int32_t*>(ws + w.src_slot);
  int32_t* layout = reinterpret_cast<int32_t*>(ws + w.layout);
  void* expert_x = ws + w.expert_x;
  float* expert_x_scale = reinterpret_cast<float*>(ws + w.expert_x_scale);
  void* inter = ws + w.inter;
  float* inter_scale = reinterpret_cast<float*>(ws + w.inter_scale);
  void* expert_y = ws + w.expert_y;

  int rc;
  // status words: [0,4) router GEMM (when it runs on the tensor cores) and gate/up GEMM,
  // [4,8) down GEMM
  StatusScope status_scope(status_dev, 8, (cudaStream_t)stream);
  if ((rc = moeb_router_logits_ws(x_bf16, w_router_bf16, router_bias, logits, c.T, c.H, c.E,
                                  ws + w.router_ws, w.router_ws_bytes, status_dev, stream)))
    return rc;
  if ((rc = moeb_router_select(logits, c.T, c.E, c.k, c.router_mode, c.n_group, c.topk_group,
                               c.renorm, c.route_scale, indices, weights, stream)))
    return rc;
  if ((rc = moeb_route_plan(indices, c.T, c.k, c.E, 128, w.m_cap, counts, offsets, dst_row,
                            src_token, src_slot, layout, ws + w.plan_ws, w.plan_ws_bytes, stream)))
    return rc;
  if ((rc = moeb_permute_quant(x_bf16, dst_row, c.T, c.k, c.H, w.m_cap, expert_x, expert_x_scale,
                               stream)))
    return rc;
  if ((rc = moeb_fp8_grouped_gemm_swiglu(expert_x, expert_x_scale, gate_q, gate_scale, up_q,
                                         up_scale, inter, inter_scale, w.m_cap, c.I, c.H, c.E,
                                         MOEB_GEMM_M_GROUPED_CONTIGUOUS, layout, 0, status_dev,
                                         stream)))
    return rc;
  // the second GEMM must not clear a timeout recorded by the first one
  if ((rc = moeb_fp8_grouped_gemm_nt(inter, inter_scale, down_q, down_scale, expert_y,
                                     MOEB_OUT_BF16, w.m_cap, c.H, c.I, c.E,
                                     MOEB_GEMM_M_GROUPED_CONTIGUOUS, layout, 0,
                                     status_dev ? status_dev + 4 : nullptr, stream)))
    return rc;
  if ((rc = moeb_unpermute_combine(expert_y, dst_row, weights, c.T, c.k, c.H, out_bf16, 0, stream)))
    return rc;
  cudaStream_t s = (cudaStream_t)stream;
  if (indices_out)
    MOEB_CUDA_TRY(cudaMemcpyAsync(indices_out, indices, (size_t)c.T * c.k * 4,
                                  cudaMemcpyDeviceToDevice, s));
  if (weights_out)
    MOEB_CUDA_TRY(cudaMemcpyAsync(weights_out, weights, (size_t)c.T * c.k * 4,
                                  cudaMemcpyDeviceToDevice, s));
  return kOk;
}

extern "C" int moeb_moe_forward_host(const moeb_layer_config* cfg, const void* x_bf16_host,
                                     void* out_bf16_host, void* dev_x, void* dev_out,
                                     const void* w_router_bf16, const float* router_bias,
                                     const void* gate_q,
                                     const float* gate_scale, const void* up_q,
                                     const float* up_scale, const void* down_q,
                                     const float* down_scale, void* workspace,
                                     size_t workspace_bytes, int32_t* status_dev, void* stream) {
  if (!cfg || !x_bf16_host || !out_bf16_host || !dev_x || !dev_out) {
    set_last_error_msg("moeb_moe_forward_host: null pointer");
    return kInvalidArgument;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const size_t bytes = (size_t)cfg->T * cfg->H * 2;
  MOEB_CUDA_TRY(cudaMemcpyAsync(dev_x, x_bf16_host, bytes, cudaMemcpyHostToDevice, s));
  const int rc = moeb_moe_forward(cfg, dev_x, w_router_bf16, router_bias, gate_q, gate_scale, up_q,
                                  up_scale,
                                  down_q, down_scale, dev_out, nullptr, nullptr, workspace,
                                  workspace_bytes, status_dev, stream);
  if (rc) return rc;
  MOEB_CUDA_TRY(cudaMemcpyAsync(out_bf16_host, dev_out, bytes, cudaMemcpyDeviceToHost, s));
  return kOk;
}
