// Routing plan: a deterministic, device-only counting sort of the (token, slot)
// pairs by expert, with every expert's row range padded to `pad` rows.
//
// It replaces three pieces of the reference: the single-CTA atomicAdd
// histogram/scan at the head of dispatch_send
// (csrc/kernels/all2all/a2a_dispatch_send_tk.cuh:128-210), the same logic in
// compute_routing_info (moe_cuda/include/moe_cuda/kernels/kernel5_1.cuh:448-696)
// and the host loop WorkerState::process_routing_info
// (csrc/all2all/a2a_worker_tk.hpp:163-384), which needs a device->host->device
// round trip. The reference's slot order inside an expert depends on atomicAdd
// arrival order (test/test_cpp/test_all2all.cpp:646-651); here it is fixed:
// rows of an expert are ordered by (token, slot), so the maps are reproducible.
//
// Three launches over chunks of 256 pairs:
//   1. plan_count   : per-chunk expert histogram (+ fills the row maps with -1)
//   2. plan_scan    : per-expert exclusive prefix over chunks, expert totals
//   3. plan_scatter : padded expert offsets, stable rank of every pair inside
//                     its chunk -> dst_row and the inverse maps
#include "common.cuh"
#include "moe_cuda_b200.h"

#include <cstdio>
#include <mutex>

namespace moeb {

constexpr int kPlanChunk = 256;  // pairs per CTA == threads per CTA
constexpr int kPlanMaxExperts = 1024;

__global__ void __launch_bounds__(kPlanChunk)
plan_count_kernel(const int32_t* __restrict__ indices, int n_pairs, int E, int m_cap,
                  int32_t* __restrict__ chunk_counts,  // [n_chunks, E]
                  int32_t* __restrict__ src_token, int32_t* __restrict__ src_slot,
                  int32_t* __restrict__ grouped_layout, int32_t* __restrict__ bad_index) {
  extern __shared__ int hist[];
  for (int e = threadIdx.x; e < E; e += kPlanChunk) hist[e] = 0;
  __syncthreads();
  const int i = blockIdx.x * kPlanChunk + threadIdx.x;
  if (i < n_pairs) {
    const int e = indices[i];
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);  // a count: order does not matter
    else atomicAdd(bad_index, 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kPlanChunk)
    chunk_counts[(size_t)blockIdx.x * E + e] = hist[e];
  // clear the row maps (padding rows keep -1)
  for (int r = blockIdx.x * kPlanChunk + threadIdx.x; r < m_cap; r += gridDim.x * kPlanChunk) {
    src_token[r] = -1;
    src_slot[r] = -1;
    grouped_layout[r] = -1;
  }
}

// One CTA per expert: exclusive prefix of that expert's counts over the chunks
// (each thread owns a run of consecutive chunks, then a block-wide scan).
__global__ void __launch_bounds__(kPlanChunk)
plan_scan_kernel(int32_t* __restrict__ chunk_counts, int n_chunks, int E,
                 int32_t* __restrict__ expert_counts) {
  __shared__ int part[kPlanChunk];
  const int e = blockIdx.x;
  const int per = ceil_div(n_chunks, kPlanChunk);
  const int c0 = threadIdx.x * per;
  const int c1 = min(n_chunks, c0 + per);
  int sum = 0;
  for (int c = c0; c < c1; ++c) sum += chunk_counts[(size_t)c * E + e];
  part[threadIdx.x] = sum;
  __syncthreads();
  // Hillis-Steele inclusive scan over 256 partial sums
  for (int off = 1; off < kPlanChunk; off <<= 1) {
    const int v = threadIdx.x >= off ? part[threadIdx.x - off] : 0;
    __syncthreads();
    part[threadIdx.x] += v;
    __syncthreads();
  }
  int run = part[threadIdx.x] - sum;  // exclusive base of this thread's run
  for (int c = c0; c < c1; ++c) {
    const int v = chunk_counts[(size_t)c * E + e];
    chunk_counts[(size_t)c * E + e] = run;
    run += v;
  }
  if (threadIdx.x == kPlanChunk - 1) expert_counts[e] = part[kPlanChunk - 1];
}

__global__ void __launch_bounds__(kPlanChunk)
plan_scatter_kernel(const int32_t* __restrict__ indices, int n_pairs, int k, int E, int m_cap,
                    int pad,
                    const int32_t* __restrict__ chunk_base,  // [n_chunks, E] exclusive bases
                    const int32_t* __restrict__ expert_counts,
                    int32_t* __restrict__ padded_offsets,  // [E+1], written by CTA 0
                    int32_t* __restrict__ dst_row,
                    int32_t* __restrict__ src_token, int32_t* __restrict__ src_slot,
                    int32_t* __restrict__ grouped_layout) {
  extern __shared__ int wcount[];  // [8 warps][E], then poff[E+1]
  constexpr int kWarps = kPlanChunk / 32;
  int* poff = wcount + kWarps * E;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int j = threadIdx.x; j < kWarps * E; j += kPlanChunk) wcount[j] = 0;
  // every CTA rebuilds the padded expert offsets (E <= 1024 values)
  for (int j = threadIdx.x; j < E; j += kPlanChunk) poff[j] = round_up(expert_counts[j], pad);
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int j = 0; j < E; ++j) {
      const int n = poff[j];
      poff[j] = off;
      off += n;
    }
    poff[E] = off;
  }
  __syncthreads();
  if (blockIdx.x == 0)
    for (int j = threadIdx.x; j <= E; j += kPlanChunk) padded_offsets[j] = poff[j];

  const int i = blockIdx.x * kPlanChunk + threadIdx.x;
  int e = -1;
  if (i < n_pairs) {
    e = indices[i];
    if (e < 0 || e >= E) e = -1;
  }
  // lanes of this warp routed to the same expert
  const unsigned peers = __match_any_sync(0xffffffffu, e);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (e >= 0 && rank_in_warp == 0) wcount[warp * E + e] = __popc(peers);
  __syncthreads();
  // exclusive prefix over the 8 warps, per expert
  for (int x = threadIdx.x; x < E; x += kPlanChunk) {
    int run = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const int v = wcount[w * E + x];
      wcount[w * E + x] = run;
      run += v;
    }
  }
  __syncthreads();
  if (e >= 0) {
    const int r = poff[e] + chunk_base[(size_t)blockIdx.x * E + e] +
                  wcount[warp * E + e] + rank_in_warp;
    dst_row[i] = r;
    if (r < m_cap) {
      src_token[r] = i / k;
      src_slot[r] = i % k;
      grouped_layout[r] = e;
    }
  } else if (i < n_pairs) {
    dst_row[i] = -1;
  }
}

// Receiver-side plan for EP > 1 (one CTA; E_local*W <= a few thousand segments).
// Segment (s, e) of the receive buffer holds the rows source rank s sent for
// local expert e, ordered (s, e); its rows go to the padded expert-major layout
// ordered (e, s).
__global__ void __launch_bounds__(1024)
recv_plan_kernel(const int32_t* __restrict__ counts_all, int W, int E, int first_expert,
                 int E_local, int pad, int recv_cap, int m_cap,
                 int32_t* __restrict__ tokens_per_expert, int32_t* __restrict__ padded_offsets,
                 int32_t* __restrict__ recv_to_row, int32_t* __restrict__ grouped_layout,
                 int32_t* __restrict__ source_rank) {
  extern __shared__ int rp_smem[];
  int* seg_src = rp_smem;                   // [W*E_local] first recv-buffer row of segment (s,e)
  int* seg_dst = seg_src + W * E_local;     // [W*E_local] first layout row of segment (s,e)
  int* poff = seg_dst + W * E_local;        // [E_local+1]
  for (int r = threadIdx.x; r < m_cap; r += blockDim.x) {
    grouped_layout[r] = -1;
    source_rank[r] = -1;
  }
  for (int r = threadIdx.x; r < recv_cap; r += blockDim.x) recv_to_row[r] = -1;
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < E_local; ++e) {
      int tot = 0;
      for (int s = 0; s < W; ++s) tot += counts_all[(size_t)s * E + first_expert + e];
      tokens_per_expert[e] = tot;
      poff[e] = off;
      padded_offsets[e] = off;
      off += round_up(tot, pad);
    }
    poff[E_local] = off;
    padded_offsets[E_local] = off;
    int src = 0;
    for (int s = 0; s < W; ++s)
      for (int e = 0; e < E_local; ++e) {
        seg_src[s * E_local + e] = src;
        src += counts_all[(size_t)s * E + first_expert + e];
      }
    for (int e = 0; e < E_local; ++e) {
      int dst = poff[e];
      for (int s = 0; s < W; ++s) {
        seg_dst[s * E_local + e] = dst;
        dst += counts_all[(size_t)s * E + first_expert + e];
      }
    }
  }
  __syncthreads();
  // one warp per segment writes its rows
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int seg = warp; seg < W * E_local; seg += nwarps) {
    const int s = seg / E_local, e = seg % E_local;
    const int n = counts_all[(size_t)s * E + first_expert + e];
    const int src = seg_src[seg], dst = seg_dst[seg];
    for (int j = lane; j < n; j += 32) {
      if (src + j < recv_cap) recv_to_row[src + j] = dst + j;
      if (dst + j < m_cap) {
        grouped_layout[dst + j] = e;
        source_rank[dst + j] = s;
      }
    }
  }
}

}  // namespace moeb

extern "C" int moeb_route_plan_rows(int T, int k, int E, int pad) {
  if (T < 0 || k <= 0 || E <= 0 || pad <= 0) return -1;
  const long long worst = (long long)T * k + (long long)E * (pad - 1);
  const long long rows = (worst + pad - 1) / pad * pad;
  return rows > 0x7fffffffLL ? -1 : (int)rows;
}

extern "C" size_t moeb_route_plan_workspace_bytes(int T, int k, int E) {
  if (T < 0 || k <= 0 || E <= 0) return 0;
  size_t n_chunks = ((size_t)T * k + moeb::kPlanChunk - 1) / moeb::kPlanChunk;
  // With T == 0 one CTA still runs (it clears the row maps) and stores one
  // histogram row of E words, so the table never has fewer than one row.
  if (n_chunks == 0) n_chunks = 1;
  // chunk bases + one int32 counter of out-of-range indices, rounded to 256 B
  return ((n_chunks * E + 1) * sizeof(int32_t) + 255) / 256 * 256;
}

extern "C" int moeb_route_plan(const int32_t* indices, int T, int k, int E, int pad, int m_cap,
                               int32_t* expert_counts, int32_t* padded_offsets, int32_t* dst_row,
                               int32_t* src_token, int32_t* src_slot, int32_t* grouped_layout,
                               void* workspace, size_t workspace_bytes, void* stream) {
  using namespace moeb;
  // with T == 0 the per-pair arrays are empty and may be null
  if ((T > 0 && (!indices || !dst_row)) || !expert_counts || !padded_offsets || !src_token ||
      !src_slot || !grouped_layout || !workspace || T < 0 || k <= 0 || E <= 0 ||
      E > kPlanMaxExperts || pad <= 0) {
    set_last_error_msg("moeb_route_plan: bad argument (need 0 < E <= 1024, k > 0, pad > 0)");
    return kInvalidArgument;
  }
  const int rows_needed = moeb_route_plan_rows(T, k, E, pad);
  if (rows_needed < 0 || (long long)T * k > 0x7fffffffLL) {
    set_last_error_msg("moeb_route_plan: T * k (plus padding) does not fit in 32 bits");
    return kTooLarge;
  }
  if (m_cap < rows_needed || workspace_bytes < moeb_route_plan_workspace_bytes(T, k, E)) {
    set_last_error_msg("moeb_route_plan: m_cap or workspace too small");
    return kInvalidArgument;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const int n_pairs = T * k;
  const int n_chunks = ceil_div(n_pairs, kPlanChunk);
  int32_t* chunk_counts = (int32_t*)workspace;
  // behind the table, which has at least one row (the CTA that runs for T == 0)
  int32_t* bad_index = chunk_counts + (size_t)(n_chunks > 0 ? n_chunks : 1) * E;
  MOEB_CUDA_TRY(cudaMemsetAsync(bad_index, 0, sizeof(int32_t), s));
  // at least one CTA so that the row maps are cleared even when T == 0
  const int grid = n_chunks > 0 ? n_chunks : 1;
  plan_count_kernel<<<grid, kPlanChunk, E * sizeof(int), s>>>(
      indices, n_pairs, E, m_cap, chunk_counts, src_token, src_slot, grouped_layout, bad_index);
  plan_scan_kernel<<<E, kPlanChunk, 0, s>>>(chunk_counts, n_chunks, E, expert_counts);
  plan_scatter_kernel<<<grid, kPlanChunk, ((kPlanChunk / 32) * E + E + 1) * sizeof(int), s>>>(
      indices, n_pairs, k, E, m_cap, pad, chunk_counts, expert_counts, padded_offsets, dst_row,
      src_token, src_slot, grouped_layout);
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}

extern "C" int moeb_recv_plan(const int32_t* counts_all, int W, int E, int first_expert,
                              int E_local, int pad, int recv_cap, int m_cap,
                              int32_t* tokens_per_expert, int32_t* padded_offsets,
                              int32_t* recv_to_row, int32_t* grouped_layout, int32_t* source_rank,
                              void* stream) {
  using namespace moeb;
  if (!counts_all || !tokens_per_expert || !padded_offsets || !recv_to_row || !grouped_layout ||
      !source_rank || W <= 0 || E <= 0 || E_local <= 0 || first_expert < 0 ||
      first_expert + E_local > E || pad <= 0 || recv_cap < 0 || m_cap < 0) {
    set_last_error_msg("moeb_recv_plan: bad argument");
    return kInvalidArgument;
  }
  const size_t smem = ((size_t)2 * W * E_local + E_local + 1) * sizeof(int);
  if (smem > 48 * 1024) {
    set_last_error_msg("moeb_recv_plan: W * E_local too large");
    return kUnsupportedShape;
  }
  recv_plan_kernel<<<1, 1024, smem, (cudaStream_t)stream>>>(
      counts_all, W, E, first_expert, E_local, pad, recv_cap, m_cap, tokens_per_expert,
      padded_offsets, recv_to_row, grouped_layout, source_rank);
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}

// ---------------------------------------------------------------------------
// Routing plan without caller-provided scratch memory.
//
// Some hosts of this library cannot hand it a workspace: an inference server
// whose memory pool claimed the whole GPU at start-up (a later cudaMalloc
// fails), or a plugin host whose rules forbid allocation calls once serving has
// begun because cudaMalloc synchronises the device. For them the per-chunk
// histogram lives in the fixed array below. It is part of the library image, so
// every GPU that loads the library holds these 513 KiB until the process exits.
namespace moeb {

constexpr int kStaticPlanScratchInts = 128 * 1024;  // chunk bases: ceil(T*k/256) * E <= 131072
static __device__ __align__(256) int32_t g_plan_scratch[kStaticPlanScratchInts + 64];

// In host code `g_plan_scratch` is only a handle for the runtime, not a device
// address. The address on the current device comes from cudaGetSymbolAddress;
// it is looked up once per device and remembered.
static int static_plan_scratch(int32_t** out) {
  static std::mutex mu;
  static int32_t* per_device[64] = {nullptr};
  int dev = -1;
  MOEB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    set_last_error_msg("moeb_route_plan_static: device ordinal out of range");
    return kInvalidArgument;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (per_device[dev] == nullptr) {
    int32_t* ptr = nullptr;
    MOEB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_plan_scratch));
    per_device[dev] = ptr;
  }
  *out = per_device[dev];
  return kOk;
}

}  // namespace moeb

extern "C" int moeb_route_plan_static_max_ints(void) { return moeb::kStaticPlanScratchInts; }

extern "C" int moeb_route_plan_static(const int32_t* indices, int T, int k, int E, int pad,
                                      int m_cap, int32_t* expert_counts, int32_t* padded_offsets,
                                      int32_t* dst_row, int32_t* src_token, int32_t* src_slot,
                                      int32_t* grouped_layout, void* stream) {
  using namespace moeb;
  if ((T > 0 && (!indices || !dst_row)) || !expert_counts || !padded_offsets || !src_token ||
      !src_slot || !grouped_layout || T < 0 || k <= 0 || E <= 0 || E > kPlanMaxExperts ||
      pad <= 0) {
    set_last_error_msg("moeb_route_plan_static: bad argument (need 0 < E <= 1024, k > 0, pad > 0)");
    return kInvalidArgument;
  }
  const int rows_needed = moeb_route_plan_rows(T, k, E, pad);
  if (rows_needed < 0 || m_cap < rows_needed) {
    set_last_error_msg("moeb_route_plan_static: m_cap too small (or T * k beyond 32 bits)");
    return rows_needed < 0 ? kTooLarge : kInvalidArgument;
  }
  const long long n_pairs_ll = (long long)T * k;
  const long long n_chunks_ll = (n_pairs_ll + kPlanChunk - 1) / kPlanChunk;
  if (n_chunks_ll * E > kStaticPlanScratchInts) {
    char msg[200];
    snprintf(msg, sizeof(msg),
             "moeb_route_plan_static: ceil(T*k/256)*E = %lld exceeds the built-in scratch of %d "
             "entries; use moeb_route_plan with a caller workspace",
             n_chunks_ll * E, kStaticPlanScratchInts);
    set_last_error_msg(msg);
    return kTooLarge;
  }
  int32_t* scratch = nullptr;
  const int rc = static_plan_scratch(&scratch);
  if (rc != kOk) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const int n_pairs = (int)n_pairs_ll;
  const int n_chunks = (int)n_chunks_ll;
  int32_t* chunk_counts = scratch;
  // the counter of out-of-range indices sits behind the largest possible table
  // and is the only word that has to start at zero; the table itself is fully
  // rewritten by plan_count_kernel before it is read
  int32_t* bad_index = scratch + kStaticPlanScratchInts;
  MOEB_CUDA_TRY(cudaMemsetAsync(bad_index, 0, sizeof(int32_t), s));
  const int grid = n_chunks > 0 ? n_chunks : 1;
  plan_count_kernel<<<grid, kPlanChunk, E * sizeof(int), s>>>(
      indices, n_pairs, E, m_cap, chunk_counts, src_token, src_slot, grouped_layout, bad_index);
  plan_scan_kernel<<<E, kPlanChunk, 0, s>>>(chunk_counts, n_chunks, E, expert_counts);
  plan_scatter_kernel<<<grid, kPlanChunk, ((kPlanChunk / 32) * E + E + 1) * sizeof(int), s>>>(
      indices, n_pairs, k, E, m_cap, pad, chunk_counts, expert_counts, padded_offsets, dst_row,
      src_token, src_slot, grouped_layout);
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}
