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
// Rows of one warp are fetched two at a time so that more loads are in flight
// over NVLink. Every wait is bounded; on expiry the status word gets
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

// `worker` of `n_workers` warps; all 32 lanes call it together.
__device__ __forceinline__ void pull_rows(const PullParams& q, int worker, int n_workers) {
  const int lane = threadIdx.x & 31;
  const int rows = min(max(*q.m_valid, 0), q.m_cap);
  const int n_kb = q.H / kQuantBlock;
  const int vec_per_row = q.H / 16;  // 16-byte pieces
  for (int r0 = 2 * worker; r0 < rows; r0 += 2 * n_workers) {
    // two rows per pass: r0 and r0 + 1 (same 128-row block)
    int src[2], tok[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int r = r0 + j;
      src[j] = r < rows ? q.source_rank[r] : -1;
      tok[j] = -1;
      if (src[j] >= 0) {
        int pos = 0;
        if (lane == 0) pos = pull_wait_pos(q, r);
        pos = __shfl_sync(0xffffffffu, pos, 0);
        if (pos < 0) return;  // the wait ran out: reported, stop
        tok[j] = pos / q.k;
      }
    }
    const uint4* from[2];
    const float* sfrom[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint64_t base = src[j] >= 0 ? q.peer_base[src[j]] : 0;
      from[j] = reinterpret_cast<const uint4*>(base + q.xq_off + (size_t)max(tok[j], 0) * q.H);
      sfrom[j] = reinterpret_cast<const float*>(base + q.xs_off) + (size_t)max(tok[j], 0) * n_kb;
    }
    // H <= 8192: at most 16 pieces per lane per row; both rows' loads are issued
    // before the first store
    for (int i0 = 0; i0 < vec_per_row; i0 += 32 * 4) {
      uint4 v[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * 32 + lane;
          if (tok[j] >= 0 && i < vec_per_row) v[j][u] = from[j][i];
        }
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * 32 + lane;
          if (tok[j] >= 0 && i < vec_per_row)
            reinterpret_cast<uint4*>(q.x_out + (size_t)(r0 + j) * q.H)[i] = v[j][u];
        }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      if (tok[j] < 0) continue;
      for (int kb = lane; kb < n_kb; kb += 32)
        q.scale_out[(size_t)kb * q.m_cap + r0 + j] = sfrom[j][kb];
    }
    // publish: every lane's stores of these rows are ordered before the add
    __syncwarp();
    const int n_done = (tok[0] >= 0 ? 1 : 0) + (tok[1] >= 0 ? 1 : 0);
    if (lane == 0 && n_done > 0) {
      __threadfence();
      red_release_gpu_add(q.arrived + r0 / 128, n_done);  // 128-row blocks of the GEMM
    }
  }
}

#endif  // __CUDACC__

}  // namespace moeb
