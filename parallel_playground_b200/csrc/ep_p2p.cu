// Expert-parallel dispatch and combine over peer memory (NVLink / NVSwitch).
//
// The reference moves tokens between GPUs with plain loads/stores into peer
// mappings of symmetric buffers (csrc/kernels/all2all/a2a_dispatch_send_tk.cuh:260-274,
// a2a_combine_send_tk.cuh:144-149) and needs a host round trip for the routing
// plan (csrc/all2all/all2all_tk.hpp:309-320). Here the whole exchange is two
// kernels with no host involvement:
//   dispatch  every token row is quantised once (1x128 FP8) and its k copies are
//             stored straight into the owning ranks' expert-sorted activation
//             buffers (16-byte peer stores) — packing, transport and un-packing
//             of the staged variant collapse into one pass;
//   combine   every token pulls its k expert outputs from the owners' output
//             buffers (16-byte peer loads) and reduces them with its weights.
// Destination rows follow from the all-gathered per-expert counts, so the row
// order is the same deterministic one as everywhere else: (expert, source rank,
// token, slot). Ranks meet between the phases in ep_barrier_kernel (flag words in
// peer memory, bounded wait); the data kernels themselves never wait on a peer.
// Peer buffers are addressed through a device array of W base addresses.
#include "common.cuh"
#include "ep_pull.cuh"
#include "moe_cuda_b200.h"

namespace moeb {

constexpr int kEpMaxTopK = 32;
constexpr int kEpMaxScaleBlocks = 512;  // H <= 65536
constexpr int kEpMaxWorld = 64;

// One CTA. For every global expert e (owner d = e / E_local):
//   dest_base[e] = first row of e in d's padded layout + rows of e sent by lower ranks
// and for this rank: m_valid = padded row total, plus the receiver-side layout.
__global__ void __launch_bounds__(1024)
ep_dest_base_kernel(const int32_t* __restrict__ counts_all, int W, int E, int rank, int pad,
                    int32_t* __restrict__ dest_base, int32_t* __restrict__ m_valid) {
  extern __shared__ int ep_smem[];
  int* tot = ep_smem;        // [E] rows of expert e over all ranks
  int* poff = tot + E;       // [E] padded offset of e inside its owner's layout
  const int e_local = E / W;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0;
    for (int s = 0; s < W; ++s) t += counts_all[(size_t)s * E + e];
    tot[e] = t;
  }
  __syncthreads();
  // one thread per owner rank walks its E_local experts
  for (int d = threadIdx.x; d < W; d += blockDim.x) {
    int off = 0;
    for (int le = 0; le < e_local; ++le) {
      poff[d * e_local + le] = off;
      off += round_up(tot[d * e_local + le], pad);
    }
    if (d == rank) *m_valid = off;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int lower = 0;
    for (int s = 0; s < rank; ++s) lower += counts_all[(size_t)s * E + e];
    dest_base[e] = poff[e] + lower;
  }
}

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  f[0] = bf16_bits_to_float(v.x & 0xffffu); f[1] = bf16_bits_to_float(v.x >> 16);
  f[2] = bf16_bits_to_float(v.y & 0xffffu); f[3] = bf16_bits_to_float(v.y >> 16);
  f[4] = bf16_bits_to_float(v.z & 0xffffu); f[5] = bf16_bits_to_float(v.z >> 16);
  f[6] = bf16_bits_to_float(v.w & 0xffffu); f[7] = bf16_bits_to_float(v.w >> 16);
}

// One CTA per token (grid-stride). The row is read and quantised once; copy j
// goes to rank dst_rank[j], row dst_row[j]: H e4m3 bytes into peer_x, H/128 fp32
// scales into the peer's row-major scale staging [m_cap, H/128] (one contiguous
// run per row; the owner transposes it locally).
__global__ void __launch_bounds__(512)
ep_dispatch_p2p_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ indices,
                       const int32_t* __restrict__ send_row,
                       const int32_t* __restrict__ send_offsets,
                       const int32_t* __restrict__ dest_base, int T, int k, int H, int E, int W,
                       int m_cap, const uint64_t* __restrict__ peer_x,
                       const uint64_t* __restrict__ peer_scale,
                       const uint64_t* __restrict__ peer_pos, int32_t* __restrict__ dst_rank,
                       int32_t* __restrict__ dst_row, int32_t* __restrict__ overflow,
                       const uint64_t* __restrict__ stash_x,
                       const uint64_t* __restrict__ stash_scale, int rank, int t_max,
                       int32_t* __restrict__ home_row) {
  __shared__ int rows_s[kEpMaxTopK];
  __shared__ int ranks_s[kEpMaxTopK];
  __shared__ float scales_s[kEpMaxScaleBlocks];
  // once-per-rank form: the distinct destination ranks of the token
  __shared__ int dests_s[kEpMaxTopK];
  __shared__ int ndest_s;
  const bool dedup = stash_x != nullptr;
  const int e_local = E / W;
  const int n_kb = H / kQuantBlock;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    __syncthreads();
    if (threadIdx.x < k) {
      const int e = indices[(size_t)t * k + threadIdx.x];
      int d = -1, r = -1;
      if (e >= 0 && e < E) {
        const int within = send_row[(size_t)t * k + threadIdx.x] - send_offsets[e];
        d = e / e_local;
        r = dest_base[e] + within;
        if (r >= m_cap) {  // the owner's buffer is too small for this routing
          atomicAdd(overflow, 1);
          d = -1;
          r = -1;
        }
      }
      rows_s[threadIdx.x] = r;
      ranks_s[threadIdx.x] = d;
      dst_rank[(size_t)t * k + threadIdx.x] = d;
      dst_row[(size_t)t * k + threadIdx.x] = r;
      // row of this copy's result in the home buffer; a dropped copy has none
      if (home_row != nullptr) home_row[(size_t)t * k + threadIdx.x] = r >= 0 ? t * k + (int)threadIdx.x : -1;
      // tell the owner where this row came from (used when its output is sent home)
      if (r >= 0 && peer_pos != nullptr)
        reinterpret_cast<int32_t*>(peer_pos[d])[r] = t * k + (int)threadIdx.x;
    }
    __syncthreads();
    if (dedup && threadIdx.x == 0) {
      int n = 0;
      for (int j = 0; j < k; ++j) {
        const int d = ranks_s[j];
        bool seen = d < 0;
        for (int i = 0; i < n && !seen; ++i) seen = dests_s[i] == d;
        if (!seen) dests_s[n++] = d;
      }
      ndest_s = n;
    }
    if (dedup) __syncthreads();
    // row of this token in a destination's stash [W * t_max rows]
    const size_t stash_row = (size_t)rank * t_max + t;
    for (int c0 = 0; c0 < H; c0 += blockDim.x * 16) {
      const int col = c0 + threadIdx.x * 16;
      const bool active = col < H;
      float f[16];
      float amax = 0.0f;
      if (active) {
        unpack8(ld_nc_v4(x + (size_t)t * H + col), f);
        unpack8(ld_nc_v4(x + (size_t)t * H + col + 8), f + 8);
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
      const float s = quant_scale_from_amax(amax);
      if (!active) continue;
      uint4 q;
      q.x = f32x4_to_e4m3x4(quant_value(f[0], s), quant_value(f[1], s), quant_value(f[2], s), quant_value(f[3], s));
      q.y = f32x4_to_e4m3x4(quant_value(f[4], s), quant_value(f[5], s), quant_value(f[6], s), quant_value(f[7], s));
      q.z = f32x4_to_e4m3x4(quant_value(f[8], s), quant_value(f[9], s), quant_value(f[10], s), quant_value(f[11], s));
      q.w = f32x4_to_e4m3x4(quant_value(f[12], s), quant_value(f[13], s), quant_value(f[14], s), quant_value(f[15], s));
      // the block's scale is kept for one coalesced store per copy below
      if ((threadIdx.x & 7) == 0) scales_s[col / kQuantBlock] = s;
      if (dedup) {
        // one copy per destination rank, into that rank's stash; the owner fans it
        // out to the token's experts locally (ep_unstash_kernel)
        const int nd = ndest_s;
        for (int i = 0; i < nd; ++i) {
          uint8_t* px = reinterpret_cast<uint8_t*>(stash_x[dests_s[i]]);
          *reinterpret_cast<uint4*>(px + stash_row * H + col) = q;
        }
      } else {
        for (int j = 0; j < k; ++j) {
          const int r = rows_s[j];
          if (r < 0) continue;
          uint8_t* px = reinterpret_cast<uint8_t*>(peer_x[ranks_s[j]]);
          *reinterpret_cast<uint4*>(px + (size_t)r * H + col) = q;
        }
      }
    }
    __syncthreads();
    // the row's H/128 scales: one contiguous run per copy (consecutive lanes,
    // consecutive words) instead of single words from 32 different threads
    if (dedup) {
      const int nd = ndest_s;
      for (int i = threadIdx.x; i < n_kb * nd; i += blockDim.x) {
        const int j = i / n_kb, kb = i - j * n_kb;
        reinterpret_cast<float*>(stash_scale[dests_s[j]])[stash_row * n_kb + kb] = scales_s[kb];
      }
    } else {
      for (int i = threadIdx.x; i < n_kb * k; i += blockDim.x) {
        const int j = i / n_kb, kb = i - j * n_kb;
        const int r = rows_s[j];
        if (r >= 0)
          reinterpret_cast<float*>(peer_scale[ranks_s[j]])[(size_t)r * n_kb + kb] = scales_s[kb];
      }
    }
  }
}

// Owner side of the once-per-rank dispatch: row r of the expert-sorted buffer is
// the stash row of (its source rank, its token): copy the H e4m3 bytes and the
// H/128 scales (into the row-major staging that ep_scale_transpose_kernel reads).
// One warp per row; padding rows (no source) are skipped.
__global__ void __launch_bounds__(256)
ep_unstash_kernel(const uint8_t* __restrict__ stash_x, const float* __restrict__ stash_scale,
                  const int32_t* __restrict__ source_rank, const int32_t* __restrict__ pos,
                  const int32_t* __restrict__ m_valid, int m_cap, int k, int t_max, int H,
                  uint8_t* __restrict__ x_out, float* __restrict__ scale_out) {
  const int rows = min(*m_valid, m_cap);
  const int n_kb = H / kQuantBlock;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const int src = source_rank[r];
    if (src < 0) continue;
    const size_t srow = (size_t)src * t_max + pos[r] / k;
    const uint4* from = reinterpret_cast<const uint4*>(stash_x + srow * H);
    uint4* to = reinterpret_cast<uint4*>(x_out + (size_t)r * H);
    for (int i = lane; i < H / 16; i += 32) to[i] = from[i];
    for (int i = lane; i < n_kb; i += 32) scale_out[(size_t)r * n_kb + i] = stash_scale[srow * n_kb + i];
  }
}

// Owner side: scale staging [rows, n_kb] (row-major, as received) -> [n_kb, m_cap]
// (MN-major, what the GEMM reads). Only rows < *m_valid are touched.
__global__ void __launch_bounds__(256)
ep_scale_transpose_kernel(const float* __restrict__ staging, const int32_t* __restrict__ m_valid,
                          int m_cap, int n_kb, float* __restrict__ scale_mn) {
  __shared__ float tile[32][33];
  const int rows = min(*m_valid, m_cap);
  const int r0 = blockIdx.x * 32;
  if (r0 >= rows) return;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int kb0 = 0; kb0 < n_kb; kb0 += 32) {
    for (int i = ty; i < 32; i += 8) {
      const int r = r0 + i, kb = kb0 + tx;
      tile[i][tx] = (r < rows && kb < n_kb) ? staging[(size_t)r * n_kb + kb] : 0.0f;
    }
    __syncthreads();
    for (int i = ty; i < 32; i += 8) {
      const int kb = kb0 + i, r = r0 + tx;
      if (kb < n_kb && r < rows) scale_mn[(size_t)kb * m_cap + r] = tile[tx][i];
    }
    __syncthreads();
  }
}

// out[t,:] = (accumulate ? out[t,:] : 0) + sum_j w[t,j] * Y_{dst_rank[t,j]}[dst_row[t,j], :]
// with Y read from peer memory; same fp32 fma order as the local un-permute.
__global__ void __launch_bounds__(512)
ep_combine_pull_kernel(const uint64_t* __restrict__ peer_y, const int32_t* __restrict__ dst_rank,
                       const int32_t* __restrict__ dst_row, const float* __restrict__ weights,
                       int T, int k, int H, __nv_bfloat16* __restrict__ out, int accumulate) {
  __shared__ int rows_s[kEpMaxTopK];
  __shared__ int ranks_s[kEpMaxTopK];
  __shared__ float w_s[kEpMaxTopK];
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    __syncthreads();
    if (threadIdx.x < k) {
      rows_s[threadIdx.x] = dst_row[(size_t)t * k + threadIdx.x];
      ranks_s[threadIdx.x] = dst_rank[(size_t)t * k + threadIdx.x];
      w_s[threadIdx.x] = weights[(size_t)t * k + threadIdx.x];
    }
    __syncthreads();
    for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
      float acc[8];
      if (accumulate) {
        unpack8(*reinterpret_cast<const uint4*>(out + (size_t)t * H + c), acc);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
      }
      // issue the k remote loads first, then reduce in slot order
      uint4 v[8];
      for (int j0 = 0; j0 < k; j0 += 8) {
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const int j = j0 + jj;
          v[jj] = make_uint4(0, 0, 0, 0);
          if (j < k && rows_s[j] >= 0) {
            const __nv_bfloat16* py = reinterpret_cast<const __nv_bfloat16*>(peer_y[ranks_s[j]]);
            v[jj] = *reinterpret_cast<const uint4*>(py + (size_t)rows_s[j] * H + c);
          }
        }
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const int j = j0 + jj;
          if (j < k && rows_s[j] >= 0) {
            float f[8];
            unpack8(v[jj], f);
            const float w = w_s[j];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = __fmaf_rn(w, f[i], acc[i]);
          }
        }
      }
      uint4 o;
      __nv_bfloat162 p2;
      p2 = __floats2bfloat162_rn(acc[0], acc[1]); o.x = *reinterpret_cast<uint32_t*>(&p2);
      p2 = __floats2bfloat162_rn(acc[2], acc[3]); o.y = *reinterpret_cast<uint32_t*>(&p2);
      p2 = __floats2bfloat162_rn(acc[4], acc[5]); o.z = *reinterpret_cast<uint32_t*>(&p2);
      p2 = __floats2bfloat162_rn(acc[6], acc[7]); o.w = *reinterpret_cast<uint32_t*>(&p2);
      *reinterpret_cast<uint4*>(out + (size_t)t * H + c) = o;
    }
  }
}

}  // namespace moeb

using namespace moeb;

// ----------------------------------------------------- rank barrier / counts --
// Barrier between the ranks' streams through flag words in peer memory, with an
// optional payload (this rank's per-expert counts, written into row `rank` of
// every peer's counts array before the flag). One CTA per rank:
//   1. payload stores to every peer, then a system-scope fence;
//   2. thread p stores `epoch` into peer p's flags[rank] (release);
//   3. thread p waits until this rank's flags[p] has reached `epoch` (acquire).
// Kernels launched earlier on the stream have completed before this one starts,
// so a peer that sees the flag also sees their stores. Epochs only grow; the
// comparison is wrap-safe. The wait is bounded: after kBarrierLimitNs the
// kernel records kDeviceTimeout in `status` and returns, it never spins forever.
constexpr uint64_t kBarrierLimitNs = 2000ull * 1000 * 1000;
constexpr int kBarrierThreads = 256;

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kBarrierThreads)
ep_barrier_kernel(const uint64_t* __restrict__ peer_flags, size_t flags_off,
                  const uint64_t* __restrict__ peer_counts,
                  const int32_t* __restrict__ my_counts, int n_counts, int rank, int W,
                  int channel, uint32_t epoch, int32_t* __restrict__ status) {
  if (peer_counts != nullptr) {
    for (int p = 0; p < W; ++p) {
      int32_t* dst = reinterpret_cast<int32_t*>(peer_counts[p]) + (size_t)rank * n_counts;
      for (int i = threadIdx.x; i < n_counts; i += kBarrierThreads) dst[i] = my_counts[i];
    }
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < W) {
    const int p = threadIdx.x;
    uint32_t* theirs =
        reinterpret_cast<uint32_t*>(peer_flags[p] + flags_off) + (size_t)channel * W + rank;
    st_release_sys_u32(theirs, epoch);
    const uint32_t* mine =
        reinterpret_cast<const uint32_t*>(peer_flags[rank] + flags_off) + (size_t)channel * W + p;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys_u32(mine) - epoch) < 0) {
      if ((++spins & 255u) == 0u && global_timer_ns() - t0 > kBarrierLimitNs) {
        if (status != nullptr && atomicCAS(&status[0], 0, (int)kDeviceTimeout) == 0) {
          status[1] = 4;      // role: rank barrier
          status[2] = p;      // the peer that did not arrive
          status[3] = (int)epoch;
        }
        break;
      }
    }
  }
  __syncthreads();
  __threadfence_system();
}

extern "C" int moeb_ep_dest_base(const int32_t* counts_all, int W, int E, int rank, int pad,
                                 int32_t* dest_base, int32_t* m_valid, void* stream) {
  if (!counts_all || !dest_base || !m_valid || W <= 0 || W > kEpMaxWorld || E <= 0 || E > 1024 ||
      E % W != 0 || rank < 0 || rank >= W || pad <= 0) {
    set_last_error_msg("moeb_ep_dest_base: bad argument (E <= 1024, W <= 64, E % W == 0)");
    return kInvalidArgument;
  }
  ep_dest_base_kernel<<<1, 1024, 2 * E * sizeof(int), (cudaStream_t)stream>>>(
      counts_all, W, E, rank, pad, dest_base, m_valid);
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}

extern "C" int moeb_ep_dispatch_p2p(const void* x_bf16, const int32_t* indices,
                                    const int32_t* send_row, const int32_t* send_offsets,
                                    const int32_t* dest_base, int T, int k, int H, int E, int W,
                                    int m_cap, const uint64_t* peer_x, const uint64_t* peer_scale,
                                    const uint64_t* peer_pos, int32_t* dst_rank, int32_t* dst_row,
                                    int32_t* overflow, void* stream) {
  if ((T > 0 && (!x_bf16 || !indices || !send_row || !dst_rank || !dst_row)) || !send_offsets ||
      !dest_base || !peer_x || !peer_scale || !overflow || T < 0 || k <= 0 || k > kEpMaxTopK ||
      H <= 0 || H % kQuantBlock != 0 || H / kQuantBlock > kEpMaxScaleBlocks || E <= 0 || W <= 0 ||
      E % W != 0 || m_cap <= 0) {
    set_last_error_msg("moeb_ep_dispatch_p2p: bad argument");
    return kInvalidArgument;
  }
  if (T == 0) return kOk;
  int threads = round_up(ceil_div(H, 16), 32);
  if (threads > 512) threads = 512;
  const int cap = 148 * 16;
  ep_dispatch_p2p_kernel<<<T < cap ? T : cap, threads, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x_bf16, indices, send_row, send_offsets, dest_base, T, k, H, E, W,
      m_cap, peer_x, peer_scale, peer_pos, dst_rank, dst_row, overflow, nullptr, nullptr, 0, 0,
      nullptr);
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}

extern "C" int moeb_ep_dispatch_once(const void* x_bf16, const int32_t* indices,
                                     const int32_t* send_row, const int32_t* send_offsets,
                                     const int32_t* dest_base, int T, int t_max, int k, int H,
                                     int E, int W, int rank, int m_cap,
                                     const uint64_t* peer_stash_x,
                                     const uint64_t* peer_stash_scale, const uint64_t* peer_pos,
                                     int32_t* dst_rank, int32_t* dst_row, int32_t* overflow,
                                     void* stream) {
  return moeb::ep_dispatch_once_home(x_bf16, indices, send_row, send_offsets, dest_base, T, t_max, k,
                                     H, E, W, rank, m_cap, peer_stash_x, peer_stash_scale, peer_pos,
                                     dst_rank, dst_row, nullptr, overflow, (cudaStream_t)stream);
}

// moeb_ep_dispatch_once that also fills the home-row map of the push combine
// (home_row[t*k+slot] = t*k+slot, or -1 for a dropped copy); used by ep_ctx.cu.
int moeb::ep_dispatch_once_home(const void* x_bf16, const int32_t* indices, const int32_t* send_row,
                                const int32_t* send_offsets, const int32_t* dest_base, int T,
                                int t_max, int k, int H, int E, int W, int rank, int m_cap,
                                const uint64_t* peer_stash_x, const uint64_t* peer_stash_scale,
                                const uint64_t* peer_pos, int32_t* dst_rank, int32_t* dst_row,
                                int32_t* home_row, int32_t* overflow, cudaStream_t stream) {
  if ((T > 0 && (!x_bf16 || !indices || !send_row || !dst_rank || !dst_row)) || !send_offsets ||
      !dest_base || !peer_stash_x || !peer_stash_scale || !peer_pos || !overflow || T < 0 ||
      T > t_max || k <= 0 || k > kEpMaxTopK || H <= 0 || H % kQuantBlock != 0 ||
      H / kQuantBlock > kEpMaxScaleBlocks || E <= 0 || W <= 0 || E % W != 0 || rank < 0 ||
      rank >= W || m_cap <= 0) {
    set_last_error_msg("moeb_ep_dispatch_once: bad argument");
    return kInvalidArgument;
  }
  if (T == 0) return kOk;
  int threads = round_up(ceil_div(H, 16), 32);
  if (threads > 512) threads = 512;
  const int cap = 148 * 16;
  ep_dispatch_p2p_kernel<<<T < cap ? T : cap, threads, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x_bf16, indices, send_row, send_offsets, dest_base, T, k, H, E, W,
      m_cap, nullptr, nullptr, peer_pos, dst_rank, dst_row, overflow, peer_stash_x,
      peer_stash_scale, rank, t_max, home_row);
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}

extern "C" int moeb_ep_unstash(const void* stash_x, const float* stash_scale,
                               const int32_t* source_rank, const int32_t* pos,
                               const int32_t* m_valid, int m_cap, int k, int t_max, int H,
                               void* expert_x, float* scale_staging, void* stream) {
  if (!stash_x || !stash_scale || !source_rank || !pos || !m_valid || !expert_x ||
      !scale_staging || m_cap <= 0 || k <= 0 || t_max <= 0 || H <= 0 || H % kQuantBlock != 0) {
    set_last_error_msg("moeb_ep_unstash: bad argument");
    return kInvalidArgument;
  }
  const int blocks = ceil_div(m_cap, 8) < 148 * 8 ? ceil_div(m_cap, 8) : 148 * 8;
  ep_unstash_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)stash_x, stash_scale, source_rank, pos, m_valid, m_cap, k, t_max, H,
      (uint8_t*)expert_x, scale_staging);
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}

extern "C" int moeb_ep_scale_transpose(const float* staging, const int32_t* m_valid, int m_cap,
                                       int n_kb, float* scale_mn, void* stream) {
  if (!staging || !m_valid || !scale_mn || m_cap <= 0 || n_kb <= 0) {
    set_last_error_msg("moeb_ep_scale_transpose: bad argument");
    return kInvalidArgument;
  }
  ep_scale_transpose_kernel<<<ceil_div(m_cap, 32), 256, 0, (cudaStream_t)stream>>>(
      staging, m_valid, m_cap, n_kb, scale_mn);
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}

extern "C" int moeb_ep_combine_pull(const uint64_t* peer_y, const int32_t* dst_rank,
                                    const int32_t* dst_row, const float* weights, int T, int k,
                                    int H, void* out_bf16, int accumulate, void* stream) {
  if (!peer_y || (T > 0 && (!dst_rank || !dst_row || !weights || !out_bf16)) || T < 0 || k <= 0 ||
      k > kEpMaxTopK || H <= 0 || H % 8 != 0) {
    set_last_error_msg("moeb_ep_combine_pull: bad argument");
    return kInvalidArgument;
  }
  if (T == 0) return kOk;
  int threads = round_up(ceil_div(H, 8), 32);
  if (threads > 512) threads = 512;
  const int cap = 148 * 8;
  ep_combine_pull_kernel<<<T < cap ? T : cap, threads, 0, (cudaStream_t)stream>>>(
      peer_y, dst_rank, dst_row, weights, T, k, H, (__nv_bfloat16*)out_bf16, accumulate);
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}

extern "C" int moeb_ep_barrier(const uint64_t* peer_flags, const uint64_t* peer_counts,
                               const int32_t* my_counts, int n_counts, int rank, int W,
                               int channel, uint32_t epoch, int32_t* status_dev, void* stream) {
  using namespace moeb;
  if (!peer_flags || W <= 0 || W > kBarrierThreads || rank < 0 || rank >= W || channel < 0 ||
      (peer_counts != nullptr && (!my_counts || n_counts <= 0))) {
    set_last_error_msg("moeb_ep_barrier: bad argument");
    return kInvalidArgument;
  }
  ep_barrier_kernel<<<1, kBarrierThreads, 0, (cudaStream_t)stream>>>(
      peer_flags, 0, peer_counts, my_counts, n_counts, rank, W, channel, epoch, status_dev);
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}

// The same barrier over flag words that lie `flags_off` bytes into every rank's
// symmetric buffer (peer_base: the W buffer base addresses); no payload.
int moeb::ep_barrier_off(const uint64_t* peer_base, size_t flags_off, int rank, int W, int channel,
                         uint32_t epoch, int32_t* status_dev, cudaStream_t stream) {
  ep_barrier_kernel<<<1, kBarrierThreads, 0, stream>>>(peer_base, flags_off, nullptr, nullptr, 0,
                                                       rank, W, channel, epoch, status_dev);
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}
