// Expert-parallel context behind the C ABI: dispatch, combine and the whole EP
// layer as single calls, for hosts that are not Python.
//
// It stands where the reference has All2All / All2AllContext / WorkerState
// (csrc/all2all/all2all_tk.hpp:201-394, a2a_context_tk.hpp:66-178,
// a2a_worker_tk.hpp:163-384) and, for the fused form, kernel5_1's dispatch inside
// the gate/up GEMM (moe_cuda/include/moe_cuda/kernels/kernel5_1.cuh:448-758).
// Differences that the hardware and the transport suggest:
//   * no host round trip: the per-expert counts travel with a rank barrier kernel
//     and the routing plan of both sides is computed on the device;
//   * pull transport: a rank quantises its tokens once into its symmetric buffer;
//     the senders only push one 8-byte word per expert copy (where the row comes
//     from), the owners load the rows over NVLink — either in a kernel of their
//     own, or inside the gate/up GEMM by a few comm CTAs while the other CTAs
//     compute on the row blocks that have already landed;
//   * the results travel home inside the down GEMM's store warps
//     (moeb_fp8_grouped_gemm_nt_scatter), followed by one rank barrier and a
//     local weighted reduction.
// Peer memory is supplied by the caller: one symmetric buffer per rank of
// moeb_ep_symmetric_bytes() bytes, mapped into every rank's address space (CUDA
// VMM / IPC, torch symmetric memory, ...), and the table of the W base addresses
// as this process sees them. The library allocates no device memory.
#include "common.cuh"
#include "ep_pull.cuh"
#include "moe_cuda_b200.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

namespace moeb {

constexpr int kEpCtxMaxWorld = 64;
constexpr int kEpCtxMaxExperts = 1024;
constexpr int kTimingSlots = 64;   // steps whose stage events are kept
constexpr int kTimingStages = 7;   // start, router, dispatch send, dispatch receive, gate/up, down, combine

static size_t al256(size_t x) { return (x + 255) / 256 * 256; }

struct SymLayout {
  size_t flags, counts, xq, xs, pos, home, stash_x, stash_scale, pos32p, total;
  size_t counts_stride, xq_stride, xs_stride;  // per parity
};
struct LocalLayout {
  size_t peer_tab, send_counts, send_offs, send_row, send_token, send_slot, send_layout, plan_ws,
      dest_base, m_valid, overflow, dst_rank, dst_row, home_row, tokens_per_expert, padded_offsets,
      grouped_layout, source_rank, pos32, arrive_need, arrived, inter_done, expert_x, scale_mn,
      scale_stage,
      tab_stash_x, tab_stash_scale, tab_pos32p, total;
  size_t plan_ws_bytes;
};

static bool ep_config_ok(const moeb_ep_config* c) {
  return c && c->max_tokens > 0 && c->hidden > 0 && c->hidden % 128 == 0 && c->hidden <= 8192 &&
         c->num_experts > 0 &&
         c->num_experts <= kEpCtxMaxExperts && c->top_k > 0 && c->top_k <= 32 &&
         c->expert_padding > 0 && c->expert_padding % 128 == 0 && c->world > 0 &&
         c->world <= kEpCtxMaxWorld && c->rank >= 0 && c->rank < c->world &&
         c->num_experts % c->world == 0 && c->capacity_rows >= 0 && c->transport >= 0 &&
         c->transport <= 2;
}

static int ep_m_cap(const moeb_ep_config& c) {
  const int e_local = c.num_experts / c.world;
  if ((long long)c.max_tokens * c.world > 0x7fffffffLL) return -1;
  const int worst = moeb_route_plan_rows(c.max_tokens * c.world, c.top_k, e_local, c.expert_padding);
  if (worst < 0) return -1;
  if (c.capacity_rows == 0) return worst;
  const long long cap = ((long long)c.capacity_rows + c.expert_padding - 1) / c.expert_padding *
                        c.expert_padding;
  return cap < worst ? (int)cap : worst;
}

static bool sym_layout(const moeb_ep_config& c, SymLayout* s) {
  const int m_cap = ep_m_cap(c);
  if (m_cap <= 0) return false;
  const size_t n_kb = c.hidden / 128;
  size_t off = 0;
  auto take = [&](size_t b) {
    const size_t at = off;
    off += al256(b);
    return at;
  };
  s->flags = take((size_t)2 * c.world * 4);
  s->counts_stride = al256((size_t)c.world * c.num_experts * 4);
  s->counts = take(2 * s->counts_stride);
  s->xq_stride = al256((size_t)c.max_tokens * c.hidden);
  s->xq = take(2 * s->xq_stride);
  s->xs_stride = al256((size_t)c.max_tokens * n_kb * 4);
  s->xs = take(2 * s->xs_stride);
  s->pos = take((size_t)m_cap * 8);
  s->home = take((size_t)c.max_tokens * c.top_k * c.hidden * 2);
  // push transport: one row per (source rank, token) and the senders' position words
  s->stash_x = take((size_t)c.world * c.max_tokens * c.hidden);
  s->stash_scale = take((size_t)c.world * c.max_tokens * n_kb * 4);
  s->pos32p = take((size_t)m_cap * 4);
  s->total = off;
  return true;
}

static bool local_layout(const moeb_ep_config& c, LocalLayout* l) {
  const int m_cap = ep_m_cap(c);
  if (m_cap <= 0) return false;
  const size_t pairs = (size_t)c.max_tokens * c.top_k;
  const size_t n_kb = c.hidden / 128;
  const size_t e_local = c.num_experts / c.world;
  const size_t nb = (size_t)m_cap / 128 + 1;
  size_t off = 0;
  auto take = [&](size_t b) {
    const size_t at = off;
    off += al256(b);
    return at;
  };
  l->peer_tab = take((size_t)c.world * 8);
  l->send_counts = take((size_t)c.num_experts * 4);
  l->send_offs = take((size_t)(c.num_experts + 1) * 4);
  l->send_row = take(pairs * 4);
  l->send_token = take(pairs * 4);
  l->send_slot = take(pairs * 4);
  l->send_layout = take(pairs * 4);
  l->plan_ws_bytes = moeb_route_plan_workspace_bytes(c.max_tokens, c.top_k, c.num_experts);
  l->plan_ws = take(l->plan_ws_bytes);
  l->dest_base = take((size_t)c.num_experts * 4);
  l->m_valid = take(4);
  l->overflow = take(4);
  l->dst_rank = take(pairs * 4);
  l->dst_row = take(pairs * 4);
  l->home_row = take(pairs * 4);
  l->tokens_per_expert = take(e_local * 4);
  l->padded_offsets = take((e_local + 1) * 4);
  l->grouped_layout = take((size_t)m_cap * 4);
  l->source_rank = take((size_t)m_cap * 4);
  l->pos32 = take((size_t)m_cap * 4);
  l->arrive_need = take(nb * 4);
  l->arrived = take(nb * 4);
  l->inter_done = take((nb > 16 ? nb : 16) * 4);   // (also the chunk plan of the chunked MLP: 2 x 8 words)
  l->expert_x = take((size_t)m_cap * c.hidden);
  l->scale_mn = take((size_t)m_cap * n_kb * 4);
  l->scale_stage = take((size_t)m_cap * n_kb * 4);
  l->tab_stash_x = take((size_t)c.world * 8);
  l->tab_stash_scale = take((size_t)c.world * 8);
  l->tab_pos32p = take((size_t)c.world * 8);
  l->total = off;
  return true;
}

// Workspace of the whole-layer call (depends on the expert width I).
struct LayerWs {
  size_t logits, router_ws, router_ws_bytes, indices, weights, inter, inter_scale, total;
};
static void layer_ws(const moeb_ep_config& c, int m_cap, int I, LayerWs* w) {
  const size_t pairs = (size_t)c.max_tokens * c.top_k;
  size_t off = 0;
  auto take = [&](size_t b) {
    const size_t at = off;
    off += al256(b);
    return at;
  };
  w->logits = take((size_t)c.max_tokens * c.num_experts * 4);
  w->router_ws_bytes = moeb_router_logits_workspace_bytes(c.max_tokens, c.hidden, c.num_experts);
  w->router_ws = take(w->router_ws_bytes);
  w->indices = take(pairs * 4);
  w->weights = take(pairs * 4);
  w->inter = take((size_t)m_cap * I);
  w->inter_scale = take((size_t)m_cap * (I / 128) * 4);
  w->total = off;
}

}  // namespace moeb

struct moeb_ep_ctx {
  moeb_ep_config cfg;
  moeb::SymLayout sym;
  moeb::LocalLayout loc;
  int m_cap, e_local, n_comm;
  uint64_t peer_host[moeb::kEpCtxMaxWorld];
  uint8_t* sym_mine;   // this rank's symmetric buffer
  uint8_t* local;      // local workspace
  uint32_t step;       // dispatches so far (the tag of the current one)
  uint32_t fence_epoch;
  int n_tokens;        // tokens of the dispatch in flight
  bool sent, received;
  // where the received rows go (the caller's tensors or the context's own) and
  // how many rows that buffer has; peer_rows: rows every rank can receive
  uint8_t* out_x;
  float* out_scale;
  int out_rows, peer_rows;
  int transport;       // configured: 0 = by call (push for bf16 tokens, else pull), 1 = pull, 2 = push
  bool auto_push;      // set by the whole-layer call around its dispatch
  bool push_cur;       // transport of the dispatch in flight
  int32_t* pos32_cur;  // source position of every received row (local copy or the senders' words)
  // second stream and events for the overlapped MLP (host-side objects)
  cudaStream_t aux;
  cudaEvent_t ev_fork, ev_join, ev_chunk[8];
  int mlp_mode;        // whole-layer call: 0 = GEMMs one after the other, 1 = in row chunks
  int mlp_chunks;      // row chunks of mode 1
  int down_ctas;       // SMs of a chunk's down launch while the next chunk's gate/up launch runs
  // optional stage timing (host-side events, no device memory)
  bool timing;
  int timing_n;
  cudaEvent_t ev[moeb::kTimingSlots][moeb::kTimingStages];
};

namespace moeb {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Pre-quantised tokens (e4m3 [T,H] + fp32 scales, MN-major [H/128, T], the layout
// of the reference's dispatch input, csrc/all2all/all2all_tk.hpp:292-300) into the
// symmetric buffer: rows as they are, scales row-major [T, H/128].
__global__ void __launch_bounds__(256)
ep_stage_q_kernel(const uint8_t* __restrict__ xq, const float* __restrict__ xs_mn, int T, int H,
                  uint8_t* __restrict__ out_q, float* __restrict__ out_s) {
  const int n_kb = H / 128;
  const size_t n_vec = (size_t)T * H / 16;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec;
       i += (size_t)gridDim.x * blockDim.x)
    reinterpret_cast<uint4*>(out_q)[i] = ld_nc_v4(reinterpret_cast<const uint4*>(xq) + i);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)T * n_kb;
       i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / n_kb), kb = (int)(i % n_kb);
    out_s[i] = xs_mn[(size_t)kb * T + t];
  }
}

// One CTA: (a) this rank's per-expert send counts into row `rank` of every rank's
// counts table, rank barrier over flag channel 0 (bounded wait); (b) from the
// gathered counts: destination row of every expert's first copy from this rank,
// and the whole receiver-side plan of this rank (rows per local expert, padded
// offsets, expert id and source rank of every row, rows per 128-row block); the
// arrival counters are cleared. Row order: (expert, source rank, token, slot).
__global__ void __launch_bounds__(1024)
ep_exchange_plan_kernel(const uint64_t* __restrict__ peer_base, size_t flags_off, size_t counts_off,
                        const int32_t* __restrict__ my_counts, int W, int E, int rank, int pad,
                        uint32_t epoch, int m_cap, int32_t* __restrict__ dest_base,
                        int32_t* __restrict__ m_valid, int32_t* __restrict__ tokens_per_expert,
                        int32_t* __restrict__ padded_offsets, int32_t* __restrict__ grouped_layout,
                        int32_t* __restrict__ source_rank, int32_t* __restrict__ arrive_need,
                        int32_t* __restrict__ arrived, int32_t* __restrict__ inter_done,
                        int32_t* __restrict__ overflow, int32_t* __restrict__ status) {
  extern __shared__ int xp_smem[];
  int* tot = xp_smem;      // [E]
  int* poff = tot + E;     // [E] padded offset inside the owner's layout
  const int e_local = E / W;
  // (a) counts to every peer, then the flags
  for (int p = 0; p < W; ++p) {
    int32_t* dst = reinterpret_cast<int32_t*>(peer_base[p] + counts_off) + (size_t)rank * E;
    for (int i = threadIdx.x; i < E; i += blockDim.x) dst[i] = my_counts[i];
  }
  if (threadIdx.x == 0) *overflow = 0;
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < W) {
    const int p = threadIdx.x;
    st_release_sys(reinterpret_cast<uint32_t*>(peer_base[p] + flags_off) + rank, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(peer_base[rank] + flags_off) + p;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++spins & 255u) == 0u && global_timer_ns() - t0 > kPullLimitNs) {
        if (status != nullptr && atomicCAS(&status[0], 0, (int)kDeviceTimeout) == 0) {
          status[1] = 4;  // role: rank barrier
          status[2] = p;
          status[3] = (int)epoch;
        }
        break;
      }
    }
  }
  __syncthreads();
  __threadfence_system();
  // (b) plans
  __shared__ int rows_now, rows_before;
  const int32_t* counts_all = reinterpret_cast<const int32_t*>(peer_base[rank] + counts_off);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0;
    for (int s = 0; s < W; ++s) t += counts_all[(size_t)s * E + e];
    tot[e] = t;
  }
  if (threadIdx.x == 0) rows_before = min(max(*m_valid, 0), m_cap);  // the previous step's rows
  __syncthreads();
  for (int d = threadIdx.x; d < W; d += blockDim.x) {
    int off = 0;
    for (int le = 0; le < e_local; ++le) {
      poff[d * e_local + le] = off;
      if (d == rank) {
        tokens_per_expert[le] = tot[d * e_local + le];
        padded_offsets[le] = off;
      }
      off += round_up(tot[d * e_local + le], pad);
    }
    if (d == rank) {
      padded_offsets[e_local] = off;
      rows_now = min(off, m_cap);
      *m_valid = rows_now;
    }
  }
  __syncthreads();
  // rows of this and of the previous step start as padding (rows beyond both
  // already are: the buffers are cleared when the context is created)
  const int clear_to = max(rows_now, rows_before);
  for (int r = threadIdx.x; r < clear_to; r += blockDim.x) {
    grouped_layout[r] = -1;
    source_rank[r] = -1;
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int lower = 0;
    for (int s = 0; s < rank; ++s) lower += counts_all[(size_t)s * E + e];
    dest_base[e] = poff[e] + lower;
  }
  __syncthreads();
  // this rank's rows: one warp per (local expert, source rank) segment
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int seg = warp; seg < W * e_local; seg += nwarps) {
    const int le = seg / W, s = seg % W;
    const int e = rank * e_local + le;
    int dst = poff[e];
    for (int s2 = 0; s2 < s; ++s2) dst += counts_all[(size_t)s2 * E + e];
    const int n = counts_all[(size_t)s * E + e];
    for (int j = lane; j < n; j += 32)
      if (dst + j < m_cap) {
        grouped_layout[dst + j] = le;
        source_rank[dst + j] = s;
      }
  }
  __syncthreads();
  // rows per 128-row block (what the fused GEMM waits for), counters cleared
  const int n_blocks = ceil_div(rows_now, 128);
  for (int b = warp; b < n_blocks; b += nwarps) {
    int c = 0;
    for (int j = lane; j < 128; j += 32) c += grouped_layout[b * 128 + j] >= 0 ? 1 : 0;
    c += __shfl_xor_sync(0xffffffffu, c, 16);
    c += __shfl_xor_sync(0xffffffffu, c, 8);
    c += __shfl_xor_sync(0xffffffffu, c, 4);
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    if (lane == 0) {
      arrive_need[b] = c;
      arrived[b] = 0;
      inter_done[b] = 0;   // (scratch words of the chunked MLP)
    }
  }
}

// Sender: one word per expert copy, in the order of the send plan (sorted by
// expert), so that consecutive threads store consecutive words of an owner's pos
// array. Also records where each (token, slot) went.
__global__ void __launch_bounds__(256)
ep_pos_push_kernel(const uint64_t* __restrict__ peer_base, size_t pos_off,
                   const int32_t* __restrict__ send_layout, const int32_t* __restrict__ send_token,
                   const int32_t* __restrict__ send_slot, const int32_t* __restrict__ send_offs,
                   const int32_t* __restrict__ dest_base, int n_pairs, int k, int E, int W,
                   int m_cap, uint32_t tag, int32_t* __restrict__ dst_rank,
                   int32_t* __restrict__ dst_row, int32_t* __restrict__ home_row,
                   int32_t* __restrict__ overflow) {
  const int e_local = E / W;
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < n_pairs; j += gridDim.x * blockDim.x) {
    const int e = send_layout[j];
    if (e < 0 || e >= E) continue;   // (pairs with an invalid expert id are not in the plan)
    const int i = send_token[j] * k + send_slot[j];
    const int d = e / e_local;
    const int r = dest_base[e] + (j - send_offs[e]);
    if (r >= m_cap) {                // the owner's buffer is too small for this routing
      atomicAdd(overflow, 1);
      dst_rank[i] = -1;
      dst_row[i] = -1;
      home_row[i] = -1;
      continue;
    }
    unsigned long long* pos = reinterpret_cast<unsigned long long*>(peer_base[d] + pos_off);
    pos[r] = ((unsigned long long)tag << 32) | (uint32_t)i;
    dst_rank[i] = d;
    dst_row[i] = r;
    home_row[i] = i;
  }
}

// (token, slot) pairs whose expert id is out of range never enter the send plan:
// mark them as dropped before ep_pos_push_kernel fills in the others.
__global__ void __launch_bounds__(256)
ep_mark_invalid_kernel(const int32_t* __restrict__ indices, int n_pairs, int E,
                       int32_t* __restrict__ dst_rank, int32_t* __restrict__ dst_row,
                       int32_t* __restrict__ home_row) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_pairs; i += gridDim.x * blockDim.x) {
    const int e = indices[i];
    if (e < 0 || e >= E) {
      dst_rank[i] = -1;
      dst_row[i] = -1;
      home_row[i] = -1;
    }
  }
}

// Receive half of a dispatch that is not fused with the GEMM: every warp of the
// grid is a pull worker (ep_pull.cuh); pos32 keeps the plain source position of
// every row for the way home.
__global__ void __launch_bounds__(384)
ep_pull_kernel(const PullParams q) {
  pull_rows(q, (int)blockIdx.x * (int)(blockDim.x >> 5) + (int)(threadIdx.x >> 5),
            (int)gridDim.x * (int)(blockDim.x >> 5));
}

// pos32[r] = low word of pos[r] for rows that hold a token (after the pull, when
// every word carries the step's tag).
__global__ void __launch_bounds__(256)
ep_pos32_kernel(const unsigned long long* __restrict__ pos, const int32_t* __restrict__ source_rank,
                const int32_t* __restrict__ m_valid, int m_cap, uint32_t tag,
                int32_t* __restrict__ pos32) {
  const int rows = min(max(*m_valid, 0), m_cap);
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x) {
    const unsigned long long w = pos[r];
    pos32[r] = (source_rank[r] >= 0 && (uint32_t)(w >> 32) == tag) ? (int)(uint32_t)w : -1;
  }
}

// Combine, send half, for callers that ran their own down projection: row r of
// expert_y goes to its source rank's home buffer at row pos32[r] (one warp per
// row, 16-byte peer stores).
__global__ void __launch_bounds__(256)
ep_send_home_kernel(const __nv_bfloat16* __restrict__ y, const int32_t* __restrict__ source_rank,
                    const int32_t* __restrict__ pos32, const int32_t* __restrict__ m_valid,
                    int m_cap, int H, const uint64_t* __restrict__ peer_base, size_t home_off) {
  const int rows = min(max(*m_valid, 0), m_cap);
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const int src = source_rank[r], pos = pos32[r];
    if (src < 0 || pos < 0) continue;
    const uint4* from = reinterpret_cast<const uint4*>(y + (size_t)r * H);
    uint4* to = reinterpret_cast<uint4*>(peer_base[src] + home_off + (size_t)pos * H * 2);
    for (int i = lane; i < H / 8; i += 32) to[i] = from[i];
  }
}

static int sm_count_ctx() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
    n = 148;
  return n;
}

template <typename T>
static T* at(uint8_t* base, size_t off) {
  return reinterpret_cast<T*>(base + off);
}

static void record_stage(moeb_ep_ctx* c, int stage, cudaStream_t s) {
  if (c->timing && c->timing_n < kTimingSlots) cudaEventRecord(c->ev[c->timing_n][stage], s);
}

static PullParams make_pull(moeb_ep_ctx* c, int32_t* status) {
  PullParams q{};
  const int par = (int)(c->step & 1u);
  q.peer_base = at<const uint64_t>(c->local, c->loc.peer_tab);
  q.xq_off = c->sym.xq + par * c->sym.xq_stride;
  q.xs_off = c->sym.xs + par * c->sym.xs_stride;
  q.pos = at<const unsigned long long>(c->sym_mine, c->sym.pos);
  q.source_rank = at<const int32_t>(c->local, c->loc.source_rank);
  q.m_valid = at<const int32_t>(c->local, c->loc.m_valid);
  q.x_out = c->out_x;
  q.scale_out = c->out_scale;
  q.arrived = at<int32_t>(c->local, c->loc.arrived);
  q.status = status;
  q.m_cap = c->out_rows;
  q.H = c->cfg.hidden;
  q.k = c->cfg.top_k;
  q.tag = c->step;
  return q;
}

// Where the received rows go: the caller's tensors (the reference's out_expert_x /
// out_expert_x_scale) or the context's own buffers.
static int set_output(moeb_ep_ctx* c, void* out_x, float* out_scale, int out_rows) {
  if (out_x == nullptr && out_scale == nullptr) {
    c->out_x = c->local + c->loc.expert_x;
    c->out_scale = at<float>(c->local, c->loc.scale_mn);
    c->out_rows = c->m_cap;
    return kOk;
  }
  // (every rank's senders bound their rows by max_recv_rows, so the caller's
  // tensors must have exactly that many rows, as the reference's do)
  if (!out_x || !out_scale || out_rows != c->m_cap ||
      (reinterpret_cast<uintptr_t>(out_x) & 15u) != 0) {
    set_last_error_msg(
        "moeb_ep_dispatch: out_expert_x [max_recv_rows, H] and out_expert_x_scale "
        "[H/128, max_recv_rows] come together, 16-byte aligned");
    return kInvalidArgument;
  }
  c->out_x = static_cast<uint8_t*>(out_x);
  c->out_scale = out_scale;
  c->out_rows = out_rows;
  return kOk;
}

// Send half: quantise (or stage) the tokens, plan, exchange the counts, push the
// per-copy words. Afterwards the layout of this rank's rows is known; the rows
// themselves are fetched by the receive half or by the fused GEMM.
static int dispatch_send(moeb_ep_ctx* c, const void* x_bf16, const void* x_q, const float* x_scale_mn,
                         const int32_t* indices, int T, bool push, int32_t* status,
                         cudaStream_t s) {
  const moeb_ep_config& g = c->cfg;
  // `push`: transport of this dispatch, chosen by the caller from the entry point
  // and the configuration only (never from this rank's token count or pointers:
  // every rank must take the same branch, ranks without tokens included).
  if (push && T > 0 && !x_bf16) {
    set_last_error_msg("moeb_ep_dispatch: the push transport takes bf16 tokens");
    return kInvalidArgument;
  }
  if (T < 0 || T > g.max_tokens) {
    set_last_error_msg("moeb_ep_dispatch: num_tokens exceeds max_tokens");
    return kInvalidArgument;
  }
  if (T > 0 && (!indices || (!x_bf16 && !(x_q && x_scale_mn)))) {
    set_last_error_msg("moeb_ep_dispatch: null tokens or indices");
    return kInvalidArgument;
  }
  c->step += 1;
  if (c->step == 0) c->step = 1;   // tag 0 is what a fresh buffer holds
  const int par = (int)(c->step & 1u);
  uint8_t* xq = c->sym_mine + c->sym.xq + par * c->sym.xq_stride;
  float* xs = reinterpret_cast<float*>(c->sym_mine + c->sym.xs + par * c->sym.xs_stride);
  int rc;
  if (T > 0 && !push) {
    if (x_bf16) {
      if ((rc = moeb_cast_bf16_to_e4m3(x_bf16, xq, xs, T, g.hidden, 0, s))) return rc;
    } else {
      ep_stage_q_kernel<<<148 * 4, 256, 0, s>>>((const uint8_t*)x_q, x_scale_mn, T, g.hidden, xq, xs);
    }
  }
  uint8_t* L = c->local;
  const int pairs_cap = moeb_route_plan_rows(T, g.top_k, g.num_experts, 1);
  if ((rc = moeb_route_plan(indices, T, g.top_k, g.num_experts, 1, pairs_cap,
                            at<int32_t>(L, c->loc.send_counts), at<int32_t>(L, c->loc.send_offs),
                            at<int32_t>(L, c->loc.send_row), at<int32_t>(L, c->loc.send_token),
                            at<int32_t>(L, c->loc.send_slot), at<int32_t>(L, c->loc.send_layout),
                            L + c->loc.plan_ws, c->loc.plan_ws_bytes, s)))
    return rc;
  const size_t counts_off = c->sym.counts + par * c->sym.counts_stride;
  ep_exchange_plan_kernel<<<1, 1024, 2 * g.num_experts * sizeof(int), s>>>(
      at<const uint64_t>(L, c->loc.peer_tab), c->sym.flags, counts_off,
      at<const int32_t>(L, c->loc.send_counts), g.world, g.num_experts, g.rank, g.expert_padding,
      c->step, c->out_rows, at<int32_t>(L, c->loc.dest_base), at<int32_t>(L, c->loc.m_valid),
      at<int32_t>(L, c->loc.tokens_per_expert), at<int32_t>(L, c->loc.padded_offsets),
      at<int32_t>(L, c->loc.grouped_layout), at<int32_t>(L, c->loc.source_rank),
      at<int32_t>(L, c->loc.arrive_need), at<int32_t>(L, c->loc.arrived),
      at<int32_t>(L, c->loc.inter_done), at<int32_t>(L, c->loc.overflow), status);
  if (push) {
    // quantise + one peer store per destination rank + one word per copy
    if ((rc = ep_dispatch_once_home(
             x_bf16, indices, at<const int32_t>(L, c->loc.send_row),
             at<const int32_t>(L, c->loc.send_offs), at<const int32_t>(L, c->loc.dest_base), T,
             g.max_tokens, g.top_k, g.hidden, g.num_experts, g.world, g.rank, c->peer_rows,
             at<const uint64_t>(L, c->loc.tab_stash_x), at<const uint64_t>(L, c->loc.tab_stash_scale),
             at<const uint64_t>(L, c->loc.tab_pos32p), at<int32_t>(L, c->loc.dst_rank),
             at<int32_t>(L, c->loc.dst_row), at<int32_t>(L, c->loc.home_row),
             at<int32_t>(L, c->loc.overflow), s)))
      return rc;
  } else if (T > 0) {
    const int n_pairs = T * g.top_k;
    const int blocks = ceil_div(n_pairs, 256) < 148 * 8 ? ceil_div(n_pairs, 256) : 148 * 8;
    ep_mark_invalid_kernel<<<blocks, 256, 0, s>>>(indices, n_pairs, g.num_experts,
                                                  at<int32_t>(L, c->loc.dst_rank),
                                                  at<int32_t>(L, c->loc.dst_row),
                                                  at<int32_t>(L, c->loc.home_row));
    // the send plan lists the pairs with a valid expert id, sorted by expert
    ep_pos_push_kernel<<<blocks, 256, 0, s>>>(
        at<const uint64_t>(L, c->loc.peer_tab), c->sym.pos, at<const int32_t>(L, c->loc.send_layout),
        at<const int32_t>(L, c->loc.send_token), at<const int32_t>(L, c->loc.send_slot),
        at<const int32_t>(L, c->loc.send_offs), at<const int32_t>(L, c->loc.dest_base), n_pairs,
        g.top_k, g.num_experts, g.world, c->peer_rows, c->step, at<int32_t>(L, c->loc.dst_rank),
        at<int32_t>(L, c->loc.dst_row), at<int32_t>(L, c->loc.home_row),
        at<int32_t>(L, c->loc.overflow));
  }
  MOEB_CUDA_TRY(cudaGetLastError());
  c->n_tokens = T;
  c->sent = true;
  c->received = false;
  c->push_cur = push;
  c->pos32_cur = push ? at<int32_t>(c->sym_mine, c->sym.pos32p) : at<int32_t>(L, c->loc.pos32);
  return kOk;
}

static int fence(moeb_ep_ctx* c, int32_t* status, cudaStream_t s);

static int pos32_launch(moeb_ep_ctx* c, cudaStream_t s) {
  uint8_t* L = c->local;
  ep_pos32_kernel<<<148, 256, 0, s>>>(at<const unsigned long long>(c->sym_mine, c->sym.pos),
                                      at<const int32_t>(L, c->loc.source_rank),
                                      at<const int32_t>(L, c->loc.m_valid), c->out_rows, c->step,
                                      at<int32_t>(L, c->loc.pos32));
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}

static int dispatch_recv(moeb_ep_ctx* c, int32_t* status, cudaStream_t s) {
  if (!c->sent) {
    set_last_error_msg("moeb_ep_dispatch: the receive half needs a preceding send half");
    return kInvalidArgument;
  }
  if (c->push_cur) {
    // every rank's stores have landed (rank barrier), then the owner-side fan-out
    // of the stash rows and the scales' way to MN-major
    uint8_t* L = c->local;
    int rc = fence(c, status, s);
    if (rc) return rc;
    const int32_t* m_valid = at<const int32_t>(L, c->loc.m_valid);
    if ((rc = moeb_ep_unstash(c->sym_mine + c->sym.stash_x,
                              at<const float>(c->sym_mine, c->sym.stash_scale),
                              at<const int32_t>(L, c->loc.source_rank), c->pos32_cur, m_valid,
                              c->out_rows, c->cfg.top_k, c->cfg.max_tokens, c->cfg.hidden, c->out_x,
                              at<float>(L, c->loc.scale_stage), s)))
      return rc;
    if ((rc = moeb_ep_scale_transpose(at<const float>(L, c->loc.scale_stage), m_valid, c->out_rows,
                                      c->cfg.hidden / 128, c->out_scale, s)))
      return rc;
    c->received = true;
    return kOk;
  }
  const PullParams q = make_pull(c, status);
  ep_pull_kernel<<<sm_count_ctx() * 2, 384, 0, s>>>(q);
  MOEB_CUDA_TRY(cudaGetLastError());
  const int rc = pos32_launch(c, s);
  if (rc) return rc;
  c->received = true;
  return kOk;
}

static int fence(moeb_ep_ctx* c, int32_t* status, cudaStream_t s) {
  c->fence_epoch += 1;
  // flag channel 1 of the same flag words
  return ep_barrier_off(at<const uint64_t>(c->local, c->loc.peer_tab), c->sym.flags, c->cfg.rank,
                        c->cfg.world, 1, c->fence_epoch, status, s);
}

static int combine_recv(moeb_ep_ctx* c, const float* weights, void* out_bf16, int accumulate,
                        int32_t* status, cudaStream_t s) {
  if (c->n_tokens > 0 && (!weights || !out_bf16)) {
    set_last_error_msg("moeb_ep_combine: null weights or output");
    return kInvalidArgument;
  }
  int rc = fence(c, status, s);   // every rank's rows have come home
  if (rc) return rc;
  return moeb_unpermute_combine(c->sym_mine + c->sym.home,
                                at<const int32_t>(c->local, c->loc.home_row), weights, c->n_tokens,
                                c->cfg.top_k, c->cfg.hidden, out_bf16, accumulate, s);
}

}  // namespace moeb

using namespace moeb;

extern "C" int moeb_ep_max_recv_rows(const moeb_ep_config* cfg) {
  if (!ep_config_ok(cfg)) return -1;
  return ep_m_cap(*cfg);
}

extern "C" size_t moeb_ep_symmetric_bytes(const moeb_ep_config* cfg) {
  SymLayout s;
  if (!ep_config_ok(cfg) || !sym_layout(*cfg, &s)) return 0;
  return s.total;
}

extern "C" size_t moeb_ep_local_bytes(const moeb_ep_config* cfg) {
  LocalLayout l;
  if (!ep_config_ok(cfg) || !local_layout(*cfg, &l)) return 0;
  return l.total;
}

extern "C" int moeb_ep_create(const moeb_ep_config* cfg, const uint64_t* peer_base_host,
                              void* local_workspace, size_t local_bytes, void* stream,
                              moeb_ep_ctx** out) {
  if (!out) return kInvalidArgument;
  *out = nullptr;
  SymLayout sl;
  LocalLayout ll;
  if (!ep_config_ok(cfg) || !sym_layout(*cfg, &sl) || !local_layout(*cfg, &ll)) {
    set_last_error_msg(
        "moeb_ep_create: bad configuration (hidden % 128, hidden <= 8192, num_experts % world, "
        "top_k <= 32, expert_padding % 128, world <= 64)");
    return kInvalidArgument;
  }
  if (!peer_base_host || !local_workspace || local_bytes < ll.total ||
      (reinterpret_cast<uintptr_t>(local_workspace) & 255u) != 0) {
    set_last_error_msg("moeb_ep_create: null pointer, or local workspace too small / not 256-byte aligned");
    return kInvalidArgument;
  }
  for (int p = 0; p < cfg->world; ++p)
    if (peer_base_host[p] == 0 || (peer_base_host[p] & 255u) != 0) {
      set_last_error_msg("moeb_ep_create: every peer base must be a non-null 256-byte aligned address");
      return kInvalidArgument;
    }
  moeb_ep_ctx* c = new (std::nothrow) moeb_ep_ctx();
  if (!c) return kCudaError;
  c->cfg = *cfg;
  c->sym = sl;
  c->loc = ll;
  c->m_cap = ep_m_cap(*cfg);
  c->peer_rows = c->m_cap;
  c->e_local = cfg->num_experts / cfg->world;
  const char* e = getenv("MOEB_EP_COMM_SMS");
  c->n_comm = e ? atoi(e) : 12;
  if (c->n_comm < 1) c->n_comm = 1;
  if (c->n_comm > 64) c->n_comm = 64;
  memcpy(c->peer_host, peer_base_host, sizeof(uint64_t) * cfg->world);
  c->sym_mine = reinterpret_cast<uint8_t*>(peer_base_host[cfg->rank]);
  c->local = static_cast<uint8_t*>(local_workspace);
  c->step = 0;
  c->fence_epoch = 0;
  c->n_tokens = 0;
  c->sent = c->received = false;
  c->timing = false;
  c->timing_n = 0;
  set_output(c, nullptr, nullptr, 0);
  c->aux = nullptr;
  c->ev_fork = c->ev_join = nullptr;
  // How the whole-layer call runs the two expert GEMMs (MOEB_EP_MLP = seq | chunks).
  // With more than one rank the down projection is bound by NVLink (most of its rows
  // go to other ranks) and the link idles during gate/up. "chunks" splits the rows into
  // MOEB_EP_MLP_CHUNKS ranges and runs the down projection of a range, on
  // MOEB_EP_DOWN_SMS SMs, beside the gate/up GEMM of the next one. Measured at 4 ranks
  // (both GEMMs, ms): default workload seq 1.59, chunks 1.53 (4 ranges, 52 SMs; 6 ranges
  // 1.59, 44 SMs 1.70); DeepSeek-V3 shape seq 1.86, chunks 1.89. What the overlap wins
  // (the SM time the down kernel spends waiting for the link, at most 0.2 ms) goes into
  // eight launches' ramps and tails, so the default stays "seq".
  c->mlp_mode = 0;
  if (const char* o = getenv("MOEB_EP_MLP")) {
    if (!strcmp(o, "seq") || !strcmp(o, "0")) c->mlp_mode = 0;
    else if (!strcmp(o, "chunks")) c->mlp_mode = 1;
  }
  c->mlp_chunks = 4;
  if (const char* o = getenv("MOEB_EP_MLP_CHUNKS")) c->mlp_chunks = atoi(o);
  if (c->mlp_chunks < 2 || c->mlp_chunks > 8) c->mlp_chunks = 4;
  c->down_ctas = 52;
  if (const char* o = getenv("MOEB_EP_DOWN_SMS")) c->down_ctas = atoi(o);
  if (c->down_ctas <= 0 || c->down_ctas > 120) c->down_ctas = 52;
  for (int i = 0; i < 8; ++i) c->ev_chunk[i] = nullptr;
  if (c->mlp_mode != 0) {
    bool ok = cudaStreamCreateWithFlags(&c->aux, cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming) == cudaSuccess &&
              cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; ok && i < 8; ++i)
      ok = cudaEventCreateWithFlags(&c->ev_chunk[i], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) {
      set_last_error_msg("moeb_ep_create: could not create the second stream");
      delete c;
      return kCudaError;
    }
  }
  c->transport = cfg->transport;
  if (const char* t = getenv("MOEB_EP_TRANSPORT")) c->transport = atoi(t);
  c->push_cur = false;
  c->auto_push = false;
  c->pos32_cur = at<int32_t>(c->local, ll.pos32);
  uint64_t tabs[3][kEpCtxMaxWorld];
  for (int p = 0; p < cfg->world; ++p) {
    tabs[0][p] = peer_base_host[p] + sl.stash_x;
    tabs[1][p] = peer_base_host[p] + sl.stash_scale;
    tabs[2][p] = peer_base_host[p] + sl.pos32p;
  }
  cudaStream_t s = (cudaStream_t)stream;
  // flags, counts and the per-row words start at zero (tag 0 = nothing yet); the
  // caller lets every rank finish this call before the first dispatch anywhere
  cudaError_t err = cudaMemsetAsync(c->sym_mine + sl.flags, 0, sl.xq - sl.flags, s);
  if (err == cudaSuccess) err = cudaMemsetAsync(c->sym_mine + sl.pos, 0, sl.home - sl.pos, s);
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(c->local + ll.peer_tab, c->peer_host, sizeof(uint64_t) * cfg->world,
                          cudaMemcpyHostToDevice, s);
  const size_t tab_off[3] = {ll.tab_stash_x, ll.tab_stash_scale, ll.tab_pos32p};
  for (int i = 0; i < 3 && err == cudaSuccess; ++i)
    err = cudaMemcpyAsync(c->local + tab_off[i], tabs[i], sizeof(uint64_t) * cfg->world,
                          cudaMemcpyHostToDevice, s);
  if (err == cudaSuccess) err = cudaMemsetAsync(c->local + ll.m_valid, 0, 4, s);
  if (err == cudaSuccess)   // every row starts as padding (-1)
    err = cudaMemsetAsync(c->local + ll.grouped_layout, 0xff, ll.pos32 - ll.grouped_layout, s);
  if (err == cudaSuccess) err = cudaMemsetAsync(c->local + ll.overflow, 0, 4, s);
  if (err == cudaSuccess) err = cudaStreamSynchronize(s);
  if (err != cudaSuccess) {
    set_last_error("moeb_ep_create", err);
    delete c;
    return kCudaError;
  }
  *out = c;
  return kOk;
}

extern "C" int moeb_ep_destroy(moeb_ep_ctx* ctx) {
  if (!ctx) return kOk;
  if (ctx->aux) cudaStreamDestroy(ctx->aux);
  if (ctx->ev_fork) cudaEventDestroy(ctx->ev_fork);
  if (ctx->ev_join) cudaEventDestroy(ctx->ev_join);
  for (int i = 0; i < 8; ++i)
    if (ctx->ev_chunk[i]) cudaEventDestroy(ctx->ev_chunk[i]);
  if (ctx->timing)
    for (int i = 0; i < kTimingSlots; ++i)
      for (int j = 0; j < kTimingStages; ++j) cudaEventDestroy(ctx->ev[i][j]);
  delete ctx;
  return kOk;
}

extern "C" int moeb_ep_get_view(moeb_ep_ctx* c, moeb_ep_view* v) {
  if (!c || !v) return kInvalidArgument;
  uint8_t* L = c->local;
  v->expert_x = c->out_x;
  v->expert_x_scale = c->out_scale;
  v->grouped_layout = at<int32_t>(L, c->loc.grouped_layout);
  v->m_valid = at<int32_t>(L, c->loc.m_valid);
  v->tokens_per_expert = at<int32_t>(L, c->loc.tokens_per_expert);
  v->padded_offsets = at<int32_t>(L, c->loc.padded_offsets);
  v->source_rank = at<int32_t>(L, c->loc.source_rank);
  v->source_pos = c->pos32_cur;
  v->dst_rank = at<int32_t>(L, c->loc.dst_rank);
  v->dst_row = at<int32_t>(L, c->loc.dst_row);
  v->overflow = at<int32_t>(L, c->loc.overflow);
  v->home = c->sym_mine + c->sym.home;
  v->max_recv_rows = c->m_cap;
  v->local_experts = c->e_local;
  v->rows = c->out_rows;
  return kOk;
}

extern "C" int moeb_ep_dispatch(moeb_ep_ctx* c, const void* x_bf16, const void* x_q,
                                const float* x_scale_mn, const int32_t* indices, int num_tokens,
                                void* out_expert_x, float* out_expert_x_scale, int out_rows,
                                int do_send, int do_recv, int32_t* status_dev, void* stream) {
  if (!c) return kInvalidArgument;
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
  if (do_send) {
    if ((rc = set_output(c, out_expert_x, out_expert_x_scale, out_rows))) return rc;
    // transport: pull unless the context is configured for push
    if ((rc = dispatch_send(c, x_bf16, x_q, x_scale_mn, indices, num_tokens, c->transport == 2,
                            status_dev, s)))
      return rc;
  }
  if (do_recv && (rc = dispatch_recv(c, status_dev, s))) return rc;
  return kOk;
}

extern "C" int moeb_ep_combine(moeb_ep_ctx* c, const void* expert_y_bf16, const float* weights,
                               void* out_bf16, int accumulate, int do_send, int do_recv,
                               int32_t* status_dev, void* stream) {
  if (!c) return kInvalidArgument;
  if (!c->received) {
    set_last_error_msg("moeb_ep_combine: needs a completed dispatch");
    return kInvalidArgument;
  }
  cudaStream_t s = (cudaStream_t)stream;
  uint8_t* L = c->local;
  if (do_send) {
    if (!expert_y_bf16) {
      set_last_error_msg("moeb_ep_combine: null expert_y");
      return kInvalidArgument;
    }
    ep_send_home_kernel<<<sm_count_ctx() * 8, 256, 0, s>>>(
        (const __nv_bfloat16*)expert_y_bf16, at<const int32_t>(L, c->loc.source_rank),
        c->pos32_cur, at<const int32_t>(L, c->loc.m_valid), c->out_rows, c->cfg.hidden,
        at<const uint64_t>(L, c->loc.peer_tab), c->sym.home);
    MOEB_CUDA_TRY(cudaGetLastError());
  }
  if (do_recv) return combine_recv(c, weights, out_bf16, accumulate, status_dev, s);
  return kOk;
}

extern "C" int moeb_ep_fused_dispatch_swiglu(moeb_ep_ctx* c, const void* x_bf16, const void* x_q,
                                             const float* x_scale_mn, const int32_t* indices,
                                             int num_tokens, void* out_expert_x,
                                             float* out_expert_x_scale, int out_rows,
                                             const void* gate_q, const float* gate_scale,
                                             const void* up_q, const float* up_scale, void* D,
                                             float* scale_d, int intermediate, int fused,
                                             int32_t* status_dev, void* stream) {
  if (!c) return kInvalidArgument;
  if (!gate_q || !gate_scale || !up_q || !up_scale || !D || !scale_d || intermediate <= 0 ||
      intermediate % 128 != 0) {
    set_last_error_msg("moeb_ep_fused_dispatch_swiglu: null pointer or bad intermediate size");
    return kInvalidArgument;
  }
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
  StatusScope status_scope(status_dev, 4, s);
  if ((rc = set_output(c, out_expert_x, out_expert_x_scale, out_rows))) return rc;
  if (fused && c->transport == 2) {
    set_last_error_msg("moeb_ep_fused_dispatch_swiglu: the fused form uses the pull transport");
    return kInvalidArgument;
  }
  // transport: pull when fused or configured so; push when configured so, or when
  // the whole-layer call asks for it (its tokens are always bf16)
  const bool push = !fused && (c->transport == 2 || (c->transport == 0 && c->auto_push));
  if ((rc = dispatch_send(c, x_bf16, x_q, x_scale_mn, indices, num_tokens, push, status_dev, s)))
    return rc;
  record_stage(c, 2, s);
  uint8_t* L = c->local;
  const int32_t* layout = at<const int32_t>(L, c->loc.grouped_layout);
  const int32_t* m_valid = at<const int32_t>(L, c->loc.m_valid);
  if (fused) {
    record_stage(c, 3, s);   // (the receive half runs inside the GEMM)
    const PullParams q = make_pull(c, status_dev);
    if ((rc = fp8_swiglu_fused_dispatch(c->out_x, c->out_scale, gate_q, gate_scale, up_q, up_scale,
                                        D, scale_d, c->out_rows, m_valid, intermediate,
                                        c->cfg.hidden, c->e_local, layout, status_dev, q,
                                        at<const int32_t>(L, c->loc.arrived),
                                        at<const int32_t>(L, c->loc.arrive_need), c->n_comm, s)))
      return rc;
    if ((rc = pos32_launch(c, s))) return rc;
    c->received = true;
  } else {
    if ((rc = dispatch_recv(c, status_dev, s))) return rc;
    record_stage(c, 3, s);
    if ((rc = moeb_fp8_grouped_gemm_swiglu_dyn(c->out_x, c->out_scale, gate_q, gate_scale, up_q,
                                               up_scale, D, scale_d, c->out_rows, m_valid,
                                               intermediate, c->cfg.hidden, c->e_local,
                                               MOEB_GEMM_M_GROUPED_CONTIGUOUS, layout, 0,
                                               status_dev, s)))
      return rc;
  }
  record_stage(c, 4, s);
  return kOk;
}

extern "C" int moeb_ep_fused_gemm_combine(moeb_ep_ctx* c, const void* A, const float* scale_a,
                                          const void* down_q, const float* down_scale,
                                          int intermediate, const float* weights, void* out_bf16,
                                          int accumulate, int32_t* status_dev, void* stream) {
  if (!c) return kInvalidArgument;
  if (!c->received) {
    set_last_error_msg("moeb_ep_fused_gemm_combine: needs a completed dispatch");
    return kInvalidArgument;
  }
  cudaStream_t s = (cudaStream_t)stream;
  uint8_t* L = c->local;
  int rc;
  StatusScope status_scope(status_dev, 4, s);   // (the barrier's words [4,8) stick)
  // down projection; its store warps send every row home over NVLink
  if ((rc = fp8_gemm_nt_scatter_off(A, scale_a, down_q, down_scale,
                                    at<const uint64_t>(L, c->loc.peer_tab), c->sym.home,
                                    at<const int32_t>(L, c->loc.source_rank), c->pos32_cur,
                                    c->out_rows,
                                    at<const int32_t>(L, c->loc.m_valid), c->cfg.hidden,
                                    intermediate, c->e_local,
                                    at<const int32_t>(L, c->loc.grouped_layout), status_dev, s)))
    return rc;
  record_stage(c, 5, s);
  return combine_recv(c, weights, out_bf16, accumulate, status_dev ? status_dev + 4 : nullptr, s);
}

extern "C" size_t moeb_ep_moe_forward_workspace_bytes(const moeb_ep_ctx* c, int intermediate) {
  if (!c || intermediate <= 0 || intermediate % 128 != 0) return 0;
  LayerWs w;
  layer_ws(c->cfg, c->m_cap, intermediate, &w);
  return w.total;
}

extern "C" int moeb_ep_moe_forward(moeb_ep_ctx* c, const moeb_layer_config* cfg, const void* x_bf16,
                                   const void* w_router_bf16, const float* router_bias,
                                   const void* gate_q, const float* gate_scale, const void* up_q,
                                   const float* up_scale, const void* down_q,
                                   const float* down_scale, void* out_bf16, int32_t* indices_out,
                                   float* weights_out, void* workspace, size_t workspace_bytes,
                                   int fused, int32_t* status_dev, void* stream) {
  if (!c || !cfg) return kInvalidArgument;
  const moeb_ep_config& g = c->cfg;
  if (cfg->H != g.hidden || cfg->E != g.num_experts || cfg->k != g.top_k || cfg->T < 0 ||
      cfg->T > g.max_tokens || cfg->I <= 0 || cfg->I % 128 != 0) {
    set_last_error_msg("moeb_ep_moe_forward: layer configuration does not match the context");
    return kInvalidArgument;
  }
  LayerWs w;
  layer_ws(g, c->m_cap, cfg->I, &w);
  if (!workspace || workspace_bytes < w.total || (reinterpret_cast<uintptr_t>(workspace) & 255u)) {
    set_last_error_msg("moeb_ep_moe_forward: workspace too small or not 256-byte aligned");
    return kInvalidArgument;
  }
  if ((cfg->T > 0 && (!x_bf16 || !out_bf16)) || !w_router_bf16 || !gate_q || !gate_scale || !up_q ||
      !up_scale || !down_q || !down_scale) {
    set_last_error_msg("moeb_ep_moe_forward: null pointer");
    return kInvalidArgument;
  }
  cudaStream_t s = (cudaStream_t)stream;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  float* logits = at<float>(ws, w.logits);
  int32_t* indices = at<int32_t>(ws, w.indices);
  float* weights = at<float>(ws, w.weights);
  void* inter = ws + w.inter;
  float* inter_scale = at<float>(ws, w.inter_scale);
  const int T = cfg->T, H = cfg->H;
  int rc;
  // (the rank barrier's words [8,12) are never cleared here: its first report sticks)
  StatusScope status_scope(status_dev, 8, s);
  record_stage(c, 0, s);
  if (T > 0) {
    if ((rc = moeb_router_logits_ws(x_bf16, w_router_bf16, router_bias, logits, T, H,
                                    g.num_experts, ws + w.router_ws, w.router_ws_bytes, status_dev,
                                    s)))
      return rc;
    if ((rc = moeb_router_select(logits, T, g.num_experts, g.top_k, cfg->router_mode, cfg->n_group,
                                 cfg->topk_group, cfg->renorm, cfg->route_scale, indices, weights,
                                 s)))
      return rc;
  }
  record_stage(c, 1, s);
  // status words: [0,4) gate/up GEMM and the rows it waits for, [4,8) down GEMM,
  // [8,12) rank barrier of the combine
  if (!fused && c->mlp_mode != 0) {
    // dispatch, then the two GEMMs in row chunks: the down projection of a chunk, whose
    // rows go home over NVLink, beside the gate/up GEMM of the next one
    uint8_t* L = c->local;
    if ((rc = set_output(c, nullptr, nullptr, 0))) return rc;
    if ((rc = dispatch_send(c, x_bf16, nullptr, nullptr, indices, T, c->transport != 1, status_dev,
                            s)))
      return rc;
    record_stage(c, 2, s);
    if ((rc = dispatch_recv(c, status_dev, s))) return rc;
    record_stage(c, 3, s);
    cudaEvent_t mid = (c->timing && c->timing_n < kTimingSlots) ? c->ev[c->timing_n][4] : nullptr;
    // (the chunk plan lives in the per-block counter array, unused on this path)
    rc = fp8_mlp_chunked(c->out_x, c->out_scale, gate_q, gate_scale, up_q, up_scale, inter,
                         inter_scale, down_q, down_scale, at<const uint64_t>(L, c->loc.peer_tab),
                         c->sym.home, at<const int32_t>(L, c->loc.source_rank), c->pos32_cur,
                         c->out_rows, at<const int32_t>(L, c->loc.m_valid), cfg->I, H, c->e_local,
                         at<const int32_t>(L, c->loc.grouped_layout),
                         at<int32_t>(L, c->loc.inter_done), c->mlp_chunks, c->down_ctas, status_dev,
                         status_dev ? status_dev + 4 : nullptr, s, c->aux, c->ev_fork, c->ev_join,
                         c->ev_chunk, mid);
    if (rc) return rc;
    record_stage(c, 5, s);
    if ((rc = combine_recv(c, weights, out_bf16, 0, status_dev ? status_dev + 8 : nullptr, s)))
      return rc;
  } else {
    c->auto_push = true;   // bf16 tokens on every rank: the push transport unless configured otherwise
    rc = moeb_ep_fused_dispatch_swiglu(c, x_bf16, nullptr, nullptr, indices, T, nullptr, nullptr, 0,
                                       gate_q, gate_scale, up_q, up_scale, inter, inter_scale,
                                       cfg->I, fused, status_dev, stream);
    c->auto_push = false;
    if (rc) return rc;
    if ((rc = moeb_ep_fused_gemm_combine(c, inter, inter_scale, down_q, down_scale, cfg->I, weights,
                                         out_bf16, 0, status_dev ? status_dev + 4 : nullptr,
                                         stream)))
      return rc;
  }
  record_stage(c, 6, s);
  if (c->timing && c->timing_n < kTimingSlots) c->timing_n += 1;
  if (indices_out && T > 0)
    MOEB_CUDA_TRY(cudaMemcpyAsync(indices_out, indices, (size_t)T * g.top_k * 4,
                                  cudaMemcpyDeviceToDevice, s));
  if (weights_out && T > 0)
    MOEB_CUDA_TRY(cudaMemcpyAsync(weights_out, weights, (size_t)T * g.top_k * 4,
                                  cudaMemcpyDeviceToDevice, s));
  return kOk;
}

extern "C" int moeb_ep_mlp_mode(const moeb_ep_ctx* c) { return c ? c->mlp_mode : -1; }

extern "C" int moeb_ep_set_timing(moeb_ep_ctx* c, int enable) {
  if (!c) return kInvalidArgument;
  if (enable && !c->timing) {
    for (int i = 0; i < kTimingSlots; ++i)
      for (int j = 0; j < kTimingStages; ++j)
        if (cudaEventCreate(&c->ev[i][j]) != cudaSuccess) return kCudaError;
    c->timing = true;
  }
  if (!enable && c->timing) {
    for (int i = 0; i < kTimingSlots; ++i)
      for (int j = 0; j < kTimingStages; ++j) cudaEventDestroy(c->ev[i][j]);
    c->timing = false;
  }
  c->timing_n = 0;
  return kOk;
}

extern "C" int moeb_ep_read_timing(moeb_ep_ctx* c, float* stage_ms, int* steps) {
  if (!c || !stage_ms || !steps) return kInvalidArgument;
  *steps = c->timing ? c->timing_n : 0;
  for (int j = 0; j < kTimingStages - 1; ++j) stage_ms[j] = 0.0f;
  if (*steps == 0) return kOk;
  for (int i = 0; i < c->timing_n; ++i)
    for (int j = 0; j < kTimingStages - 1; ++j) {
      float ms = 0.0f;
      const cudaError_t e = cudaEventElapsedTime(&ms, c->ev[i][j], c->ev[i][j + 1]);
      if (e != cudaSuccess) {
        set_last_error("moeb_ep_read_timing (synchronise the stream first)", e);
        return kCudaError;
      }
      stage_ms[j] += ms / (float)c->timing_n;
    }
  c->timing_n = 0;
  return kOk;
}
