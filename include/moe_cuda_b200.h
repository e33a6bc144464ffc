/*
 * C ABI of libmoe_cuda_b200.so — the sm_100a (B200) implementation of the
 * expert-parallel MoE layer hot path of moe_cuda (kingsleykimm/parallel_playground):
 *
 *   router top-k -> token permutation + FP8 (e4m3, 1x128) quantisation ->
 *   [all-to-all dispatch] -> FP8 SwiGLU grouped GEMM (gate/up, then down) ->
 *   [all-to-all combine] -> weighted un-permute.
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer unless its name ends in `_host`.
 *  - Every function returns 0 on success or a moeb status code (see
 *    moeb_status_string); it never exits the process and never allocates
 *    device memory: the caller owns inputs, outputs and workspaces.
 *  - `stream` is a cudaStream_t passed as void*; work is enqueued, not awaited.
 *  - FP8 means e4m3fn (max 448). Activation scales are fp32, one per 128
 *    consecutive K elements of a row, stored MN-major: scale[kb * rows + row].
 *    Weight scales are fp32, one per 128x128 block: scale[(g*N/128 + nb)*K/128 + kb].
 *  - `status_dev` (optional, may be NULL) is an int32[4] device word a kernel
 *    fills when one of its bounded waits expires: {code, role, tile, k-block}.
 *    The entry point zeroes it before launching.
 *
 * Each declaration cites the reference interface it replaces as
 * path-in-reference:line.
 */
#ifndef MOE_CUDA_B200_H_
#define MOE_CUDA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* moe_cuda/include/moe_cuda/types.h:2-10 (GemmType) */
enum {
  MOEB_GEMM_NORMAL = 0,
  MOEB_GEMM_M_GROUPED_CONTIGUOUS = 1,
  MOEB_GEMM_M_GROUPED_MASKED = 2,
  MOEB_GEMM_BATCHED = 3
};

/* Router scoring modes (no counterpart: the reference has no router, README.md:50). */
enum {
  MOEB_ROUTER_SOFTMAX = 0,       /* softmax -> top-k -> optional renormalise */
  MOEB_ROUTER_SIGMOID_GROUPED = 1 /* sigmoid -> group-limited top-k -> renormalise */
};

enum {
  MOEB_OUT_BF16 = 0,
  MOEB_OUT_F32 = 1
};

int moeb_abi_version(void);
/* Human-readable text for a status code. */
const char *moeb_status_string(int status);
/* Text of the last failure on the calling thread ("" if none). */
const char *moeb_last_error(void);

/* ---- a1: router ---------------------------------------------------------
 * No reference implementation exists (roadmap item, README.md:50); callers of
 * the reference fabricate `indices`/`weights` (test/test_cpp/test_all2all.cpp:132-140,
 * python/benchmark_fused_moe.py:624-628). Output types follow what dispatch
 * consumes: indices int32 [T,k], weights fp32 [T,k]
 * (csrc/all2all/all2all_tk.hpp:271-279). */

/* logits[T,E] (fp32) = x[T,H] (bf16) * w_gate[H,E] (bf16) + logit_bias[E], fp32
 * accumulation; logit_bias (fp32) may be NULL. */
int moeb_router_logits(const void *x_bf16, const void *w_gate_bf16, const float *logit_bias,
                       float *logits, int T, int H, int E, void *stream);

/* The same product with a caller-provided scratch buffer. With many tokens and more than
 * 64 experts (E % 8 == 0) the contraction bounds the kernels behind moeb_router_logits;
 * with a workspace of moeb_router_logits_workspace_bytes(T, H, E) bytes (256-byte aligned)
 * the logits are computed on the tcgen05 tensor cores instead: w_gate transposed to
 * K-major, a bf16 GEMM with its K range split over the SMs, and the slices' fp32 partial
 * sums added in a fixed order (bit-reproducible; the sums differ from moeb_router_logits'
 * in the last bits, as any two accumulation orders do). The size query returns 0 where
 * that path does not apply; with no or too small a workspace the call is
 * moeb_router_logits. x and logits must be 16-byte aligned. status_dev: optional int32[4]
 * of the GEMM's bounded waits. */
size_t moeb_router_logits_workspace_bytes(int T, int H, int E);
int moeb_router_logits_ws(const void *x_bf16, const void *w_gate_bf16, const float *logit_bias,
                          float *logits, int T, int H, int E, void *workspace,
                          size_t workspace_bytes, int32_t *status_dev, void *stream);

/* Select on given fp32 logits. Ties go to the lower expert id.
 * SOFTMAX:  top-k by logit, w_j = exp(l_j - max) / sum over the selected
 *           (renorm != 0) or over all experts (renorm == 0), times route_scale.
 * SIGMOID_GROUPED: s = sigmoid(l); experts form n_group consecutive groups;
 *           group score = sum of its two largest s; keep the topk_group best
 *           groups; top-k by s among them; w_j = s_j / sum(selected) * route_scale.
 * The arithmetic is defined operation by operation (see oracle/moe_oracle.c)
 * so indices and weights are bit-reproducible. */
int moeb_router_select(const float *logits, int T, int E, int k, int mode, int n_group,
                       int topk_group, int renorm, float route_scale, int32_t *indices,
                       float *weights, void *stream);

/* ---- a2: routing plan ---------------------------------------------------
 * Replaces the block-0 phase of dispatch_send
 * (csrc/kernels/all2all/a2a_dispatch_send_tk.cuh:128-210), compute_routing_info
 * (moe_cuda/include/moe_cuda/kernels/kernel5_1.cuh:448-696) and the host loop
 * WorkerState::process_routing_info (csrc/all2all/a2a_worker_tk.hpp:163-384),
 * entirely on the device and in a deterministic order: rows of an expert are
 * sorted by (token, slot).
 *
 *   expert_counts  [E]      unpadded rows per expert
 *   padded_offsets [E+1]    first row of each expert when every expert's range
 *                           is rounded up to `pad` rows; [E] = total padded rows
 *   dst_row        [T*k]    row of (token, slot) in the expert-sorted layout
 *   src_token/src_slot [m_cap]  inverse map, -1 on padding rows
 *   grouped_layout [m_cap]  expert id of each row, -1 on padding rows (the
 *                           MGroupedContiguous layout, kernel3.hpp:155)
 * m_cap must be >= T*k + E*(pad-1) rounded up to pad (see moeb_route_plan_rows). */
int moeb_route_plan_rows(int T, int k, int E, int pad);
size_t moeb_route_plan_workspace_bytes(int T, int k, int E);
int moeb_route_plan(const int32_t *indices, int T, int k, int E, int pad, int m_cap,
                    int32_t *expert_counts, int32_t *padded_offsets, int32_t *dst_row,
                    int32_t *src_token, int32_t *src_slot, int32_t *grouped_layout,
                    void *workspace, size_t workspace_bytes, void *stream);

/* The same routing plan for callers that cannot give the library a workspace.
 * It has no counterpart in the reference. Typical callers: an inference server
 * whose memory pool took the whole GPU at start-up, so that any later
 * cudaMalloc fails, or a host that bans allocation calls while serving because
 * cudaMalloc synchronises the device. The scratch (per-chunk expert histogram)
 * is a fixed array inside the library image: 513 KiB of device memory on every
 * GPU that loads the library, held until the process exits.
 *  - Limit: ceil(T*k/256) * E <= moeb_route_plan_static_max_ints() (131072);
 *    larger problems return status 7 (moeb_status_string: "size exceeds a fixed
 *    limit") and must use moeb_route_plan.
 *  - The function calls no cudaMalloc / cudaFree and no allocating library.
 *  - The first call on each device looks up the array's device address (with
 *    that device current); make that first call before any stream capture.
 *  - All calls on a device share the one array: two calls whose kernels overlap
 *    on the GPU (different streams, no ordering) race on it. Calls on one stream
 *    are safe; nothing of a previous call's contents is relied on.
 * Outputs are identical to moeb_route_plan's. */
int moeb_route_plan_static_max_ints(void);
int moeb_route_plan_static(const int32_t *indices, int T, int k, int E, int pad, int m_cap,
                           int32_t *expert_counts, int32_t *padded_offsets, int32_t *dst_row,
                           int32_t *src_token, int32_t *src_slot, int32_t *grouped_layout,
                           void *stream);

/* ---- a3: 1x128 FP8 quantisation -----------------------------------------
 * csrc/kernels/cast.cuh:45-109 (cast_bf16_to_e4m3_blkscaled_128_kernel) behind
 * moe_cuda::kernels::cast (csrc/kernels/internal_api.hpp:20-23).
 * S = amax/448 (1 if the block is all zero), q = e4m3(clamp(x / S, +-448)).
 * scale_mn_major == 0: scale[row*H/128 + kb] (what the reference kernel writes);
 * != 0: scale[kb*rows + row] (what the GEMMs read). */
int moeb_cast_bf16_to_e4m3(const void *x_bf16, void *q_e4m3, float *scale, int rows, int H,
                           int scale_mn_major, void *stream);

/* csrc/kernels/cast.cuh:113-196 (fused_silu_mul_quant_kernel) behind
 * moe_cuda::kernels::fused_silu_mul_quant (internal_api.hpp:25-26).
 * gemm_out [rows, 2*I] bf16 (gate | up) -> y = g/(1+exp(-g)) * u -> 1x128 quant. */
int moeb_fused_silu_mul_quant(const void *gemm_out_bf16, void *q_e4m3, float *scale, int rows,
                              int I, int scale_mn_major, void *stream);

/* ---- a3+a4 (one rank): fused quantise + permute --------------------------
 * Replaces cast + dispatch_send scatter + dispatch_recv compaction
 * (a2a_dispatch_send_tk.cuh:224-293, a2a_dispatch_recv_tk.cuh:111-161) when the
 * source and destination are the same GPU: each token row is read once,
 * quantised once and written to its k rows of expert_x [m_cap,H] (e4m3) and
 * expert_x_scale [H/128, m_cap] (fp32, MN-major). */
int moeb_permute_quant(const void *x_bf16, const int32_t *dst_row, int T, int k, int H, int m_cap,
                       void *expert_x, float *expert_x_scale, void *stream);

/* EP>1 sender side: quantise each token once and write its k copies into a
 * packed send buffer of `row_bytes`-byte rows (H e4m3 bytes followed by H/128
 * fp32 scales, rounded up to 16 B) at row send_row[t*k+j]. */
int moeb_dispatch_pack(const void *x_bf16, const int32_t *send_row, int T, int k, int H,
                       void *send_buf, int row_bytes, void *stream);
/* The same packing for tokens that are already quantised — the form the
 * reference's All2All::dispatch takes (csrc/all2all/all2all_tk.hpp:201-334:
 * dp_x e4m3 [T,H], dp_x_scale fp32 MN-major [H/128,T]). */
int moeb_dispatch_pack_q(const void *x_e4m3, const float *x_scale_mn, const int32_t *send_row,
                         int T, int k, int H, void *send_buf, int row_bytes, void *stream);
/* EP>1 receiver side: recv_buf rows (same row format) -> expert_x / expert_x_scale
 * at row recv_to_row[r] (rows with recv_to_row < 0 are skipped). */
int moeb_dispatch_unpack(const void *recv_buf, const int32_t *recv_to_row, int n_recv, int H,
                         int row_bytes, int m_cap, void *expert_x, float *expert_x_scale,
                         void *stream);
/* EP>1 receiver-side map: from the all-gathered unpadded counts
 * counts_all[W,E] build, for this rank's experts [first_expert, first_expert+E_local):
 * tokens_per_expert[E_local], padded_offsets[E_local+1], recv_to_row[recv_cap]
 * (position in the (source rank, expert, token, slot)-ordered receive buffer ->
 * row of the (expert, source rank, token, slot)-ordered padded layout),
 * grouped_layout[m_cap] and source_rank[m_cap] (-1 on padding). Mirrors
 * a2a_worker_tk.hpp:163-384 with ascending source rank order
 * (kernel5_1.cuh:552-563, python/benchmark_fused_moe.py:198-236). */
int moeb_recv_plan(const int32_t *counts_all, int W, int E, int first_expert, int E_local,
                   int pad, int recv_cap, int m_cap, int32_t *tokens_per_expert,
                   int32_t *padded_offsets, int32_t *recv_to_row, int32_t *grouped_layout,
                   int32_t *source_rank, void *stream);
/* Gather bf16 rows: out[r,:] = y[row_of[r],:] for r < n (row_of < 0 -> zeros);
 * the combine-send packing (a2a_combine_send_tk.cuh:61-185). */
int moeb_gather_rows_bf16(const void *y_bf16, const int32_t *row_of, int n, int H, void *out_bf16,
                          void *stream);

/* ---- a4/a7 over peer memory (EP > 1, no host round trip) ---------------------
 * The reference's transport: loads/stores into peer mappings of symmetric
 * buffers (csrc/kernels/all2all/a2a_dispatch_send_tk.cuh:260-274,
 * a2a_combine_recv_tk.cuh:117-178) around a host-side routing plan
 * (csrc/all2all/all2all_tk.hpp:309-320). Here: counts are all-gathered on the
 * device, moeb_ep_dest_base turns them into destination rows, moeb_ep_dispatch_p2p
 * quantises every token once and stores its k copies directly into the owners'
 * buffers, moeb_ep_combine_pull reads the k expert outputs back from the owners
 * and reduces them. peer_* are device arrays of W buffer base addresses (this
 * rank's own buffer included); the caller lets the ranks meet between the phases
 * with moeb_ep_barrier (stream-ordered, no host wait).
 *   counts_all [W,E] int32; dest_base [E]; m_valid [1] = this rank's padded rows;
 *   send_row / send_offsets: moeb_route_plan(pad = 1) outputs dst_row / padded_offsets;
 *   peer_x[d]: e4m3 [m_cap,H]; peer_scale[d]: fp32 [m_cap, H/128] (row-major staging,
 *   transposed by the owner with moeb_ep_scale_transpose); peer_y[d]: bf16 [m_cap,H];
 *   dst_rank/dst_row [T,k]: where each copy went (-1 if dropped); overflow [1] counts
 *   copies that did not fit in m_cap rows; peer_pos[d] (optional): int32 [m_cap], receives
 *   t*k+slot of every stored copy so that the owner can send the result home. */
int moeb_ep_dest_base(const int32_t *counts_all, int W, int E, int rank, int pad,
                      int32_t *dest_base, int32_t *m_valid, void *stream);
/* Stream-ordered barrier between the W ranks through flag words in peer memory,
 * optionally carrying this rank's counts (the reference exchanges its counts and
 * synchronises its ranks through ThunderKittens barriers in peer memory,
 * csrc/all2all/a2a_context_tk.hpp:66-71, a2a_dispatch_send_tk.cuh:260-274).
 *   peer_flags[d]: uint32 [channels, W] in rank d's symmetric memory, zero before the
 *   first call; epoch: the same on every rank and larger (mod 2^32) on every call per
 *   channel; peer_counts[d] (optional): int32 [W, n_counts], row `rank` of every peer
 *   receives my_counts before the flag. The wait is bounded (2 s): on expiry
 *   status_dev[0..3] = {4 (device timeout), 4 (role: rank barrier), missing peer, epoch} and the kernel
 *   returns. Kernels queued earlier on `stream` are complete on every rank before
 *   any kernel queued after the barrier starts. */
int moeb_ep_barrier(const uint64_t *peer_flags, const uint64_t *peer_counts,
                    const int32_t *my_counts, int n_counts, int rank, int W, int channel,
                    uint32_t epoch, int32_t *status_dev, void *stream);
int moeb_ep_dispatch_p2p(const void *x_bf16, const int32_t *indices, const int32_t *send_row,
                         const int32_t *send_offsets, const int32_t *dest_base, int T, int k, int H,
                         int E, int W, int m_cap, const uint64_t *peer_x,
                         const uint64_t *peer_scale, const uint64_t *peer_pos, int32_t *dst_rank,
                         int32_t *dst_row, int32_t *overflow, void *stream);
int moeb_ep_scale_transpose(const float *staging, const int32_t *m_valid, int m_cap, int n_kb,
                            float *scale_mn, void *stream);
/* Once-per-rank dispatch (the reference sends a token once per expert copy,
 * a2a_dispatch_send_tk.cuh:224-293; this form sends it once per destination rank):
 * moeb_ep_dispatch_once stores the quantised row of token t into the stash of every
 * rank that owns at least one of its k experts, at stash row rank*t_max + t
 * (peer_stash_x[d]: e4m3 [W*t_max, H]; peer_stash_scale[d]: fp32 [W*t_max, H/128]),
 * and the per-copy words dst_rank / dst_row / peer_pos as moeb_ep_dispatch_p2p does.
 * After the ranks have met and moeb_recv_plan has run, moeb_ep_unstash fans the rows
 * out on the owner: row r of expert_x and of the row-major scale staging comes from
 * stash row source_rank[r]*t_max + pos[r]/k. Same bytes in expert_x as the direct form. */
int moeb_ep_dispatch_once(const void *x_bf16, const int32_t *indices, const int32_t *send_row,
                          const int32_t *send_offsets, const int32_t *dest_base, int T, int t_max,
                          int k, int H, int E, int W, int rank, int m_cap,
                          const uint64_t *peer_stash_x, const uint64_t *peer_stash_scale,
                          const uint64_t *peer_pos, int32_t *dst_rank, int32_t *dst_row,
                          int32_t *overflow, void *stream);
int moeb_ep_unstash(const void *stash_x, const float *stash_scale, const int32_t *source_rank,
                    const int32_t *pos, const int32_t *m_valid, int m_cap, int k, int t_max, int H,
                    void *expert_x, float *scale_staging, void *stream);
int moeb_ep_combine_pull(const uint64_t *peer_y, const int32_t *dst_rank, const int32_t *dst_row,
                         const float *weights, int T, int k, int H, void *out_bf16, int accumulate,
                         void *stream);

/* ---- a5: gate/up grouped GEMM + SwiGLU + 1x128 re-quantisation ------------
 * moe_cuda::kernels::fp8_grouped_gemm_swiglu (internal_api.hpp:33-38) ->
 * api::fp8_grouped_gemm_swiglu (csrc/apis/moe.hpp:100-118) -> kernel3
 * (moe_cuda/include/moe_cuda/kernels/kernel3.cuh:101-447; variants kernel3_sub,
 * kernel4 compute the same result).
 *   A [m_total,K] e4m3, scale_a [K/128, m_total];
 *   gate, up [G,N,K] e4m3 (K-major), scale_gate/up [G*N/128, K/128];
 *   D [m_total,N] e4m3, scale_d [N/128, m_total].
 * CONTIGUOUS: grouped_layout[m_total] = expert id per row, -1 padding; every
 * expert's rows start on a multiple of 128. MASKED: A is [G,max_m,K] (m_total =
 * G*max_m, max_m % 128 == 0) and grouped_layout[G] = valid rows per expert.
 * Padding rows of D are written as zeros with scale 1. */
int moeb_fp8_grouped_gemm_swiglu(const void *A, const float *scale_a, const void *gate,
                                 const float *scale_gate, const void *up, const float *scale_up,
                                 void *D, float *scale_d, int m_total, int N, int K, int G,
                                 int gemm_type, const int32_t *grouped_layout, int max_m,
                                 int32_t *status_dev, void *stream);

/* Same, with the number of rows in use read from device memory: row blocks at or
 * beyond *m_valid_dev are not visited. For buffers sized for the worst case when
 * the real row count exists only on the device (expert-parallel dispatch without
 * a host round trip); m_total stays the allocation size and the stride of the
 * MN-major scale tensors. m_valid_dev may be NULL. */
int moeb_fp8_grouped_gemm_swiglu_dyn(const void *A, const float *scale_a, const void *gate,
                                     const float *scale_gate, const void *up,
                                     const float *scale_up, void *D, float *scale_d, int m_total,
                                     const int32_t *m_valid_dev, int N, int K, int G, int gemm_type,
                                     const int32_t *grouped_layout, int max_m, int32_t *status_dev,
                                     void *stream);

/* ---- a6: down-projection grouped GEMM -----------------------------------
 * moe_cuda::kernels::fp8_grouped_gemm_nt (internal_api.hpp:53-56) ->
 * api::fp8_grouped_gemm (moe.hpp:51-70) -> kernel2
 * (moe_cuda/include/moe_cuda/kernels/kernel2.cuh:82-362).
 *   out[m,:] = sum_kb (A_q[m,kb] . W_q[g][:,kb]^T) * scale_a[kb,m] * scale_w[g][n/128,kb]
 * out is bf16 or fp32 [m_total,N]. Layout arguments as above. */
int moeb_fp8_grouped_gemm_nt(const void *A, const float *scale_a, const void *W,
                             const float *scale_w, void *out, int out_dtype, int m_total, int N,
                             int K, int G, int gemm_type, const int32_t *grouped_layout, int max_m,
                             int32_t *status_dev, void *stream);

int moeb_fp8_grouped_gemm_nt_dyn(const void *A, const float *scale_a, const void *W,
                                 const float *scale_w, void *out, int out_dtype, int m_total,
                                 const int32_t *m_valid_dev, int N, int K, int G, int gemm_type,
                                 const int32_t *grouped_layout, int max_m, int32_t *status_dev,
                                 void *stream);

/* Down projection whose epilogue sends every output row home (EP combine fused
 * into the GEMM): row r goes to peer_out[row_rank[r]] (bf16 [*, N]) at row
 * row_pos[r] with 16-byte peer stores while the tensor core works on the next
 * tile; padding rows are not stored. This is the fused_grouped_gemm_combine of
 * the reference, which exists there as a launcher only
 * (csrc/jit_kernels/impls/kernel5_2.hpp:125-220, its kernel5_2.cuh is empty);
 * the weighting stays with the source rank (moeb_unpermute_combine over its
 * [T*k, N] buffer) so that the reduction order is unchanged. Contiguous layout. */
int moeb_fp8_grouped_gemm_nt_scatter(const void *A, const float *scale_a, const void *W,
                                     const float *scale_w, const uint64_t *peer_out,
                                     const int32_t *row_rank, const int32_t *row_pos, int m_total,
                                     const int32_t *m_valid_dev, int N, int K, int G,
                                     const int32_t *grouped_layout, int32_t *status_dev,
                                     void *stream);

/* BF16 GEMM D[M,N] = A[M,K] * B[g][N,K]^T with fp32 accumulation
 * (csrc/kernels/internal_api.hpp:58-61 -> csrc/apis/moe.hpp:72-98: sm90_bf16_gemm,
 * sm90_bf16_grouped_gemm_contiguous / _masked; the reference ignores its optional
 * C operand, which therefore has no parameter here). Not on the FP8 MoE path;
 * provided so that every op of the module has a live entry point. A bf16 [m_total,K],
 * B bf16 [G,N,K], D bf16 or fp32 [m_total,N]; gemm_type MOEB_GEMM_NORMAL (G = 1, no
 * layout) or one of the grouped types with the layouts of the FP8 GEMMs above.
 * N, K multiples of 8 (16-byte rows); grouped with G > 1: N % 128 == 0. */
int moeb_bf16_gemm(const void *A, const void *B, void *D, int out_dtype, int m_total, int N, int K,
                   int G, int gemm_type, const int32_t *grouped_layout, int max_m,
                   int32_t *status_dev, void *stream);

/* ---- a7: weighted un-permute (combine) ------------------------------------
 * a2a_combine_recv_tk.cuh:61-200: out[t,:] = (accumulate ? out[t,:] : 0) +
 * sum_j w[t,j] * y[row[t,j],:], fp32 fused multiply-adds in slot order, stored
 * as bf16. y is bf16 [*,H]. */
int moeb_unpermute_combine(const void *y_bf16, const int32_t *row_of_slot, const float *weights,
                           int T, int k, int H, void *out_bf16, int accumulate, void *stream);

/* ---- whole layer on one GPU ------------------------------------------------
 * The W=1 form of naive_moe_forward (src/moe_ops.cu:153-191): router -> plan ->
 * permute+quant -> gate/up+SwiGLU GEMM -> down GEMM -> weighted un-permute.
 * Weights are pre-quantised (e4m3 + 128x128 scales). `workspace` must hold
 * moeb_moe_forward_workspace_bytes(...) bytes, 256-byte aligned. indices_out /
 * weights_out (optional) receive the routing decision. status_dev (optional) is
 * int32[8] here: one 4-word record per GEMM. router_bias (optional) is fp32 [E]. */
typedef struct {
  int T, H, I, E, k;
  int router_mode, n_group, topk_group, renorm;
  float route_scale;
} moeb_layer_config;

size_t moeb_moe_forward_workspace_bytes(const moeb_layer_config *cfg);
int moeb_moe_forward(const moeb_layer_config *cfg, const void *x_bf16, const void *w_router_bf16,
                     const float *router_bias, const void *gate_q, const float *gate_scale, const void *up_q,
                     const float *up_scale, const void *down_q, const float *down_scale,
                     void *out_bf16, int32_t *indices_out, float *weights_out, void *workspace,
                     size_t workspace_bytes, int32_t *status_dev, void *stream);

/* Host-buffer form of the same call: copies x from (pinned) host memory,
 * runs the layer and copies out back, all on `stream`. dev_x / dev_out are
 * caller-provided device staging buffers of T*H bf16 each. */
int moeb_moe_forward_host(const moeb_layer_config *cfg, const void *x_bf16_host,
                          void *out_bf16_host, void *dev_x, void *dev_out,
                          const void *w_router_bf16, const float *router_bias, const void *gate_q,
                          const float *gate_scale,
                          const void *up_q, const float *up_scale, const void *down_q,
                          const float *down_scale, void *workspace, size_t workspace_bytes,
                          int32_t *status_dev, void *stream);

/* ---- expert-parallel context: dispatch, combine and the EP layer as single calls ----
 * Replaces, for W > 1 ranks, All2All / All2AllBase and their context and worker
 * (csrc/all2all/all2all_base.hpp:11-52, all2all_tk.hpp:201-394, a2a_context_tk.hpp:66-178,
 * a2a_worker_tk.hpp:163-384), naive_moe_forward (src/moe_ops.cu:153-191) and the fused
 * dispatch + gate/up GEMM of kernel5_1 (csrc/tk_bindings.cu:17-60,
 * moe_cuda/include/moe_cuda/kernels/kernel5_1.cuh:448-778). One process per GPU.
 *
 * Memory comes from the caller:
 *   - one SYMMETRIC buffer per rank of moeb_ep_symmetric_bytes(cfg) bytes, 256-byte
 *     aligned, mapped into every rank's address space (CUDA VMM handles, IPC, torch
 *     symmetric memory: what the reference gets from TKParallelTensor); peer_base_host[p]
 *     is the address of rank p's buffer as THIS process sees it (host array of W words);
 *   - a LOCAL workspace of moeb_ep_local_bytes(cfg) bytes, 256-byte aligned.
 * moeb_ep_create clears the flag words of this rank's symmetric buffer and returns after
 * its stream work is done; the caller must let EVERY rank finish moeb_ep_create before any
 * rank dispatches (one host-side barrier at set-up; none afterwards).
 *
 * Transport. The per-expert counts travel with a rank-barrier kernel, which also plans both
 * sides. Then either PUSH (default for bf16 tokens): the sender quantises every token once
 * (e4m3, 1x128 scales) and stores it once per destination RANK into that rank's stash, plus
 * one word per expert copy; after a rank barrier the owners fan the stash rows out to their
 * experts' rows locally. Or PULL (pre-quantised tokens, and the fused form): the rank's
 * quantised tokens sit in its symmetric buffer, every expert copy costs its sender one
 * 8-byte word stored into the owner's buffer, and the owners load the rows over NVLink (plain
 * peer loads, no TMA multicast) -- in a kernel of their own or, fused, by a few comm CTAs of
 * the gate/up GEMM while its other CTAs already compute on the 128-row blocks that have
 * landed. Expert outputs go home inside the down GEMM's store warps, then one rank barrier
 * and a local weighted reduction. All forms deliver the same bytes in the same rows. Rows of an expert are
 * ordered (source rank, token, slot). Every device-side wait is bounded (2 s), after which
 * status_dev gets {4, role, index, tag} and the kernels run to their end.
 * One dispatch/combine pair in flight per context (all2all_tk.hpp:31-32). */
typedef struct {
  int max_tokens;      /* tokens a rank brings to one dispatch, at most */
  int hidden;          /* H, multiple of 128 */
  int num_experts;     /* E over all ranks, multiple of world; rank r owns experts [r*E/W, (r+1)*E/W) */
  int top_k;           /* experts per token, <= 32 */
  int expert_padding;  /* every local expert's rows start on a multiple of this (128) */
  int world, rank;
  int capacity_rows;   /* rows a rank can receive; 0 = worst case (all2all_tk.hpp:101-106) */
  int transport;       /* 0 = push in moeb_ep_moe_forward(fused = 0), pull elsewhere; 1 = always
                          pull; 2 = always push (bf16 tokens, not fused). Every rank must use the
                          same value: the choice never depends on a rank's own tokens */
} moeb_ep_config;

typedef struct moeb_ep_ctx moeb_ep_ctx;

/* What a rank holds after a dispatch (device pointers into the local workspace / this
 * rank's symmetric buffer; valid until moeb_ep_destroy). */
typedef struct {
  void *expert_x;              /* e4m3 [max_recv_rows, H] */
  float *expert_x_scale;       /* fp32 [H/128, max_recv_rows], MN-major */
  int32_t *grouped_layout;     /* [max_recv_rows] local expert id per row, -1 padding */
  int32_t *m_valid;            /* [1] padded rows in use */
  int32_t *tokens_per_expert;  /* [E/W] unpadded rows per local expert */
  int32_t *padded_offsets;     /* [E/W + 1] */
  int32_t *source_rank;        /* [max_recv_rows] rank a row came from, -1 padding */
  int32_t *source_pos;         /* [max_recv_rows] token*k + slot on that rank (after the receive half) */
  int32_t *dst_rank, *dst_row; /* [T, k] where this rank's copies went, -1 if dropped */
  int32_t *overflow;           /* [1] copies dropped because the owner's capacity_rows was too small */
  void *home;                  /* bf16 [max_tokens*k, H]: expert outputs of this rank's tokens */
  int max_recv_rows, local_experts;
  int rows;                    /* rows of expert_x (= max_recv_rows) */
} moeb_ep_view;

int moeb_ep_max_recv_rows(const moeb_ep_config *cfg);
size_t moeb_ep_symmetric_bytes(const moeb_ep_config *cfg);
size_t moeb_ep_local_bytes(const moeb_ep_config *cfg);
int moeb_ep_create(const moeb_ep_config *cfg, const uint64_t *peer_base_host,
                   void *local_workspace, size_t local_bytes, void *stream, moeb_ep_ctx **out);
int moeb_ep_destroy(moeb_ep_ctx *ctx);
int moeb_ep_get_view(moeb_ep_ctx *ctx, moeb_ep_view *view);

/* All2All::dispatch (all2all_tk.hpp:201-334). Tokens are either bf16 [T,H] (x_bf16; they
 * are quantised here) or already quantised as the reference passes them (x_q e4m3 [T,H] +
 * x_scale_mn fp32 [H/128, T]); indices int32 [T,k]. do_send / do_recv are the two halves of
 * the reference (:292-334): the send half quantises, plans, exchanges the counts and
 * announces the copies; the receive half fetches the rows. After the send half the layout
 * fields of the view are valid, after the receive half expert_x / expert_x_scale /
 * source_pos as well. The rows land in out_expert_x (e4m3 [out_rows, H]) /
 * out_expert_x_scale (fp32 [H/128, out_rows]) with out_rows == max_recv_rows, or, when both
 * are NULL, in buffers of the context (see the view). status_dev: optional int32[4]. */
int moeb_ep_dispatch(moeb_ep_ctx *ctx, const void *x_bf16, const void *x_q,
                     const float *x_scale_mn, const int32_t *indices, int num_tokens,
                     void *out_expert_x, float *out_expert_x_scale, int out_rows, int do_send,
                     int do_recv, int32_t *status_dev, void *stream);

/* All2All::combine (all2all_tk.hpp:336-394): send half: every row of expert_y (bf16
 * [max_recv_rows, H]) goes to its source rank's home buffer; receive half: rank barrier,
 * then out[t] = (accumulate ? out[t] : 0) + sum_j weights[t,j] * home[t*k+j] in slot order. */
int moeb_ep_combine(moeb_ep_ctx *ctx, const void *expert_y_bf16, const float *weights,
                    void *out_bf16, int accumulate, int do_send, int do_recv,
                    int32_t *status_dev, void *stream);

/* fused_dispatch_grouped_gemm_swiglu (csrc/tk_bindings.cu:17-60): dispatch and the
 * gate/up + SwiGLU + re-quantisation GEMM over what arrives, in one call. Token and output
 * arguments as moeb_ep_dispatch; gate/up e4m3 [E/W, I, H] with 128x128 scales; D e4m3
 * [max_recv_rows, I], scale_d fp32 [I/128, max_recv_rows]. fused != 0: a few comm CTAs of
 * the GEMM kernel fetch the rows while the others compute on the 128-row blocks that have
 * arrived (kernel5_1.cuh:274-285, 698-758); fused == 0: the rows are fetched by a kernel of
 * their own first. Same bits either way. */
int moeb_ep_fused_dispatch_swiglu(moeb_ep_ctx *ctx, const void *x_bf16, const void *x_q,
                                  const float *x_scale_mn, const int32_t *indices,
                                  int num_tokens, void *out_expert_x, float *out_expert_x_scale,
                                  int out_rows, const void *gate_q, const float *gate_scale,
                                  const void *up_q, const float *up_scale, void *D, float *scale_d,
                                  int intermediate, int fused, int32_t *status_dev, void *stream);

/* fused_grouped_gemm_combine (csrc/tk_bindings.cu:62-94; the reference ships the launcher
 * only, csrc/jit_kernels/impls/kernel5_2.hpp:125-220): the down projection of A (e4m3
 * [max_recv_rows, I], scale_a fp32 [I/128, max_recv_rows]) whose store warps send every row
 * to its source rank, then the rank barrier and the weighted reduction into out_bf16 [T, H].
 * status_dev: optional int32[8] (GEMM, barrier). */
int moeb_ep_fused_gemm_combine(moeb_ep_ctx *ctx, const void *A, const float *scale_a,
                               const void *down_q, const float *down_scale, int intermediate,
                               const float *weights, void *out_bf16, int accumulate,
                               int32_t *status_dev, void *stream);

/* The whole layer on W ranks in one call: router -> dispatch -> gate/up + SwiGLU GEMM ->
 * down GEMM (rows sent home by its store warps) -> barrier -> weighted reduction
 * (naive_moe_forward_dispatch, csrc/python_api.cpp:516-532, with the router in front).
 * cfg->H/E/k must match the context, cfg->T <= max_tokens; gate/up [E/W,I,H], down
 * [E/W,H,I] hold this rank's experts. fused != 0: the dispatch's receive half runs inside
 * the gate/up GEMM (kernel5_1 semantics), else as a kernel of its own before it; both give
 * the same bits. workspace: moeb_ep_moe_forward_workspace_bytes(ctx, I) bytes, 256-byte
 * aligned. status_dev: optional int32[12] (gate/up GEMM, down GEMM, rank barrier / pull). */
size_t moeb_ep_moe_forward_workspace_bytes(const moeb_ep_ctx *ctx, int intermediate);
int moeb_ep_moe_forward(moeb_ep_ctx *ctx, const moeb_layer_config *cfg, const void *x_bf16,
                        const void *w_router_bf16, const float *router_bias, const void *gate_q,
                        const float *gate_scale, const void *up_q, const float *up_scale,
                        const void *down_q, const float *down_scale, void *out_bf16,
                        int32_t *indices_out, float *weights_out, void *workspace,
                        size_t workspace_bytes, int fused, int32_t *status_dev, void *stream);

/* Optional stage timing of moeb_ep_moe_forward with CUDA events owned by the context (the
 * reference brackets its launches with NVTX ranges, csrc/runtime/utils.h:7-15): after
 * moeb_ep_set_timing(ctx, 1) up to 64 calls are recorded; moeb_ep_read_timing (after the
 * stream has been synchronised) returns the mean milliseconds of {router, dispatch send
 * half, dispatch receive half (0 when it is fused into the GEMM), gate/up GEMM, down GEMM,
 * barrier + reduction} and the number of calls, and starts a new series. */
int moeb_ep_set_timing(moeb_ep_ctx *ctx, int enable);
int moeb_ep_read_timing(moeb_ep_ctx *ctx, float *stage_ms6, int *steps);

/* How moeb_ep_moe_forward (fused = 0) runs the two expert GEMMs on this context:
 * 0 = one after the other; 1 = in row chunks, the down projection of a chunk (whose rows
 * go home over NVLink) on a part of the SMs beside the gate/up GEMM of the next chunk
 * (launches ordered by events on two streams; no kernel waits on another). Both give the
 * same bits. Chosen when the context is made: 0 unless the environment variable
 * MOEB_EP_MLP (seq | chunks) says otherwise (measured at 4 ranks the chunked form wins
 * nothing); MOEB_EP_MLP_CHUNKS (2..8, default 4) and MOEB_EP_DOWN_SMS (default 52) size
 * mode 1. With mode 1 the stage times read "gate/up GEMM" up to the end of the last
 * gate/up launch and "down GEMM" for what is left of the down projection after it.
 * Returns the mode, or -1 without a context. */
int moeb_ep_mlp_mode(const moeb_ep_ctx *ctx);

#ifdef __cplusplus
}
#endif
#endif /* MOE_CUDA_B200_H_ */
