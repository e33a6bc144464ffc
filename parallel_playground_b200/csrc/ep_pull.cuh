// Receiver side of the pull-style expert-parallel dispatch.
//
// The reference's fused kernel lets a few "comm" CTAs fetch every token row this
// rank's experts need from the GPU that holds it and count the rows per 128-row
// block, while the other CTAs run the grouped GEMM and wait on those counters
// (moe_cuda/include/moe_cuda/kernels/kernel5_1.cuh:698-758 comm_path, :274-285
// the wait, :751-755 the red.release.gpu that publishes a row). pull_rows() below
// is that comm path for this library's buffers; it is used twice:
//   * as the role of the trailing CTAs of the fused gate/up kernel
//     (grouped_gemm.cu, kOptFused), and
//   * as a kernel of its own (ep_ctx.cu: the receive half of a dispatch that is
//     not fused with the GEMM).
//
// What a row needs. Every rank keeps its tokens, quantised once (e4m3 + one
// fp32 scale per 128 columns), in its symmetric buffer. The sender tells the
// owner of expert row r where the row comes from with ONE 8-byte word,
// pos[r] = (tag << 32) | (token * k + slot), stored into the owner's memory; the
// owner knows the source rank of r from the all-gathered counts. A worker warp
//   1. polls pos[r] until it carries this step's tag (bounded),
//   2. loads the H e4m3 bytes and the H/128 scales of that token from the source
//      rank with 16-byte / 4-byte peer loads (plain loads, no TMA multicast),
//   3. stores them to expert_x[r,:] and, MN-major, to scale[kb*m_cap + r],
//   4. publishes the row: fence, then one gpu-scope add on arrived[r/128].
// A warp fetches several rows per pass so that more loads are in flight over
// NVLink. Every wait is bounded; on expiry the status word gets
// {4, 7 (role: pull), row, tag} and the worker stops.
#pragma once

#include "common.cuh"

namespace moeb {

struct PullParams {
  const uint64_t* peer_base;    // [W] base address of every rank's symmetric buffer
  size_t xq_off, xs_off;        // byte offsets of this step's quantised tokens / scales in it
  const unsigned long long* pos;  // [m_cap] (tag << 32) | (token*k + slot), written by the senders
  const int32_t* source_rank;   // [m_cap] source rank of row r, -1 for padding rows
  const int32_t* m_valid;       // rows in use on this rank
  uint8_t* x_out;               // [m_cap, H] e4m3
  float* scale_out;             // [H/128, m_cap] fp32, MN-major
  int32_t* arrived;             // [m_cap/128] rows published per block
  int32_t* status;              // optional int32[4]
  int m_cap, H, k;
  uint32_t tag;
};

// grouped_gemm.cu: gate/up + SwiGLU grouped GEMM whose last n_comm CTAs run
// pull_rows(pull) while the others compute and wait on arrive_cnt >= arrive_need.
int fp8_swiglu_fused_dispatch(const void* A, const float* scale_a, const void* gate,
                              const float* scale_gate, const void* up, const float* scale_up,
                              void* D, float* scale_d, int m_total, const int32_t* m_valid_dev,
                              int N, int K, int G, const int32_t* grouped_layout,
                              int32_t* status_dev, const PullParams& pull,
                              const int32_t* arrive_cnt, const int32_t* arrive_need, int n_comm,
                              cudaStream_t stream);

// grouped_gemm.cu: down projection whose store warps send row r to
// peer_base[row_rank[r]] + home_off, row row_pos[r] (bf16 [*, N]).
int fp8_gemm_nt_scatter_off(const void* A, const float* scale_a, const void* W,
                            const float* scale_w, const uint64_t* peer_base, size_t home_off,
                            const int32_t* row_rank, const int32_t* row_pos, int m_total,
                            const int32_t* m_valid_dev, int N, int K, int G,
                            const int32_t* grouped_layout, int32_t* status_dev,
                            cudaStream_t stream);
// grouped_gemm.cu: the MLP in row chunks, gate/up of a chunk beside the down projection
// of the chunk before it.
int fp8_mlp_chunked(const void* A, const float* scale_a, const void* gate, const float* scale_gate,
                    const void* up, const float* scale_up, void* D, float* scale_d,
                    const void* down, const float* scale_down, const uint64_t* peer_out,
                    size_t home_off, const int32_t* row_rank, const int32_t* row_pos, int m_total,
                    const int32_t* m_valid_dev, int I, int H, int G, const int32_t* grouped_layout,
                    int32_t* plan, int chunks, int n_down_ctas, int32_t* status_swiglu,
                    int32_t* status_down, cudaStream_t main, cudaStream_t aux, cudaEvent_t ev_fork,
                    cudaEvent_t ev_join, const cudaEvent_t* ev_chunk, cudaEvent_t ev_gate_up_done);
// ep_p2p.cu: moeb_ep_dispatch_once that also fills the home-row map (-1: dropped).
int ep_dispatch_once_home(const void* x_bf16, const int32_t* indices, const int32_t* send_row,
                          const int32_t* send_offsets, const int32_t* dest_base, int T, int t_max,
                          int k, int H, int E, int W, int rank, int m_cap,
                          const uint64_t* peer_stash_x, const uint64_t* peer_stash_scale,
                          const uint64_t* peer_pos, int32_t* dst_rank, int32_t* dst_row,
                          int32_t* home_row, int32_t* overflow, cudaStream_t stream);
// ep_p2p.cu: rank barrier over flag words at peer_base[p] + flags_off.
int ep_barrier_off(const uint64_t* peer_base, size_t flags_off, int rank, int W, int channel,
                   uint32_t epoch, int32_t* status_dev, cudaStream_t stream);

#if defined(__CUDACC__)

constexpr int kRolePull = 7;
constexpr uint64_t kPullLimitNs = 2000ull * 1000 * 1000;  // 2 s per row word

__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int32_t* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu_s32(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// The sender's word for row r, once it carries `tag`; -1 if the wait ran out.
__device__ __forceinline__ int pull_wait_pos(const PullParams& q, int r) {
  unsigned long long w = ld_relaxed_sys_u64(q.pos + r);
  if ((uint32_t)(w >> 32) == q.tag) return (int)(uint32_t)w;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    w = ld_relaxed_sys_u64(q.pos + r);
    if ((uint32_t)(w >> 32) == q.tag) return (int)(uint32_t)w;
    if ((++spins & 63u) == 0u && global_timer_ns() - t0 > kPullLimitNs) {
      if (q.status != nullptr && atomicCAS(&q.status[0], 0, (int)kDeviceTimeout) == 0) {
        q.status[1] = kRolePull;
        q.status[2] = r;
        q.status[3] = (int)q.tag;
      }
      return -1;
    }
    __nanosleep(200);
  }
}

// One pass of a worker warp: kRows consecutive rows (all in one 128-row block),
// each up to kVec * 512 bytes wide. Lanes 0..kRows-1 poll the rows' words at the
// same time; every load of the pass (rows and scales, local or over NVLink) is in
// flight before the first store; one fence and one counter update per pass.
template <int kRows, int kVec>
__device__ __forceinline__ bool pull_pass(const PullParams& q, int r0, int rows, int n_kb,
                                          int vec_per_row, int lane) {
  int my_src = -1, my_pos = -1;
  if (lane < kRows && r0 + lane < rows) {
    my_src = q.source_rank[r0 + lane];
    if (my_src >= 0) {
      my_pos = pull_wait_pos(q, r0 + lane);
      if (my_pos < 0) my_src = -2;  // the wait ran out
    }
  }
  if (__any_sync(0xffffffffu, my_src == -2)) return false;
  const uint4* from[kRows];
  const float* sfrom[kRows];
  bool live[kRows];
  int n_done = 0;
#pragma unroll
  for (int j = 0; j < kRows; ++j) {
    const int src = __shfl_sync(0xffffffffu, my_src, j);
    const int pos = __shfl_sync(0xffffffffu, my_pos, j);
    live[j] = src >= 0;
    n_done += live[j] ? 1 : 0;
    const int tok = live[j] ? pos / q.k : 0;
    const uint64_t base = q.peer_base[live[j] ? src : 0];
    from[j] = reinterpret_cast<const uint4*>(base + q.xq_off + (size_t)tok * q.H);
    sfrom[j] = reinterpret_cast<const float*>(base + q.xs_off) + (size_t)tok * n_kb;
  }
  uint4 v[kRows][kVec];
  float sc[kRows][2];
#pragma unroll
  for (int j = 0; j < kRows; ++j) {
#pragma unroll
    for (int u = 0; u < kVec; ++u) {
      const int i = u * 32 + lane;
      if (live[j] && i < vec_per_row) v[j][u] = from[j][i];
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int kb = u * 32 + lane;
      if (live[j] && kb < n_kb) sc[j][u] = sfrom[j][kb];
    }
  }
#pragma unroll
  for (int j = 0; j < kRows; ++j) {
#pragma unroll
    for (int u = 0; u < kVec; ++u) {
      const int i = u * 32 + lane;
      if (live[j] && i < vec_per_row)
        reinterpret_cast<uint4*>(q.x_out + (size_t)(r0 + j) * q.H)[i] = v[j][u];
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int kb = u * 32 + lane;
      if (live[j] && kb < n_kb) q.scale_out[(size_t)kb * q.m_cap + r0 + j] = sc[j][u];
    }
  }
  // publish: every lane's stores of these rows are ordered before the add
  __syncwarp();
  if (lane == 0 && n_done > 0) {
    __threadfence();
    red_release_gpu_add(q.arrived + r0 / 128, n_done);  // 128-row blocks of the GEMM
  }
  return true;
}

// `worker` of `n_workers` warps; all 32 lanes call it together. Rows are taken
// in ascending order, so row blocks complete in the order the GEMM walks them.
// H <= 4096: four rows per pass; H <= 8192: two (the rows wait in registers).
__device__ __forceinline__ void pull_rows(const PullParams& q, int worker, int n_workers) {
  const int lane = threadIdx.x & 31;
  const int rows = min(max(*q.m_valid, 0), q.m_cap);
  const int n_kb = q.H / kQuantBlock;
  const int vec_per_row = q.H / 16;  // 16-byte pieces
  if (q.H <= 4096) {
    for (int r0 = 4 * worker; r0 < rows; r0 += 4 * n_workers)
      if (!pull_pass<4, 8>(q, r0, rows, n_kb, vec_per_row, lane)) return;
  } else {
    for (int r0 = 2 * worker; r0 < rows; r0 += 2 * n_workers)
      if (!pull_pass<2, 16>(q, r0, rows, n_kb, vec_per_row, lane)) return;
  }
}

#endif  // __CUDACC__

}  // namespace moeb
