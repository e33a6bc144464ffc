// FP8 (e4m3) grouped GEMMs for the MoE experts on sm_100a:
//   * gate/up projection + SwiGLU + 1x128 re-quantisation  (kSwiglu = true)
//   * down projection, bf16/fp32 output                     (kSwiglu = false)
//
// Math contract (reference: moe_cuda/include/moe_cuda/kernels/kernel3.cuh:292-446
// for gate/up, kernel2.cuh:263-360 for down): activations carry one fp32 scale
// per row per 128 K-elements (MN-major, scale_a[kb*m_total + row]), weights one
// fp32 scale per 128x128 block. For every 128-wide K block the FP8 product is
// accumulated in fp32 by the tensor core, multiplied by scale_a*scale_b and added
// to an fp32 accumulator ("promotion"), exactly the reference's scheme; the
// SwiGLU epilogue is y = up*gate/(1+exp(-gate)), s = rowmax_128(|y|)/448,
// D = e4m3(y/s), scale_d[n/128, row] = s.
//
// Blackwell mapping. One persistent CTA per SM, 384 threads:
//   warp 0      TMA producer: A tile [128 x 128 B] and B tile [256 x 128 B]
//               (gate rows | up rows, or 256 weight rows) per K block into a
//               4-stage shared-memory ring (3 stages for the bf16 row-store
//               form of the down projection), 128-byte swizzle, no multicast.
//   warp 1      issues tcgen05.mma (kind::f8f6f4, M=128, N=256, K=32) x4 per K
//               block into one of two 256-column TMEM buffers; a fresh buffer
//               per K block because the fp32 block scales must be applied
//               between K blocks.
//   warp 2      owns the TMEM allocation (512 columns).
//   warps 4-11  two warpgroups; thread r of each reads TMEM lane r (= tile row
//               r) with tcgen05.ld and folds the scaled partial sums into 128
//               fp32 registers; warpgroup h owns column half h. At the end of a
//               tile they run the epilogue while the tensor core already works
//               on the next tile; output rows are staged in shared memory and
//               leave the SM as whole 128- / 256-byte runs (to local memory, or
//               for the down projection also to peer GPUs: the EP combine).
// Ragged M: a tile is (128-row block, N block); the expert of a row block comes
// from grouped_layout, so no host-side knowledge of the per-expert counts is
// needed and padding-only blocks are skipped.
#include "common.cuh"
#include "ep_pull.cuh"
#include "moe_cuda_b200.h"

#include <cstdio>
#include <cstdlib>
#include <mutex>

namespace moeb {

constexpr int kBM = 128;
constexpr int kBK = 128;
constexpr int kUmmaN = 256;
constexpr int kUmmaK = 32;
constexpr int kStages = 4;
constexpr int kTileABytes = kBM * kBK;       // 16 KiB
constexpr int kTileBBytes = kUmmaN * kBK;    // 32 KiB
constexpr int kStageBytes = kTileABytes + kTileBBytes;
constexpr int kGemmThreads = 384;
constexpr int kEpiThreads = 256;
constexpr int kEpiWarps = kEpiThreads / 32;
constexpr int kTmemCols = 512;
// Register split after launch (168 x 384 threads are allocated): the producer /
// MMA warpgroup gives registers to the two promotion warpgroups. The totals must
// match exactly: 128 * 40 + 256 * 232 == 384 * 168.
constexpr int kRegsProducerWg = 40;
constexpr int kRegsEpilogueWg = 232;
static_assert(128 * kRegsProducerWg + 256 * kRegsEpilogueWg == kGemmThreads * 168, "register pool");
constexpr int kSmemAux = 4096;  // barriers, TMEM slot, abort flag, amax exchange
constexpr int kGemmSmemBytes = kStages * kStageBytes + kSmemAux + 1024 /* alignment slack */;
// Row-store epilogue of the down projection (bf16 rows written locally, or
// stored to peer GPUs for the EP combine): per promotion warpgroup a staging
// area of 128 rows x 128 bf16 columns (row pitch 272 B, conflict-free for
// 16-byte accesses) and 128 destination row pointers, so that every row leaves
// the SM as one 256-byte run (two rows per warp store) instead of 16-byte pieces
// of 32 different rows. The staging takes the place of one pipeline stage: this
// kernel runs on three (measured: no loss against four for the down projection).
constexpr int kStagesScatter = 3;
constexpr int kScatterRowPitch = 272;
constexpr int kScatterWgBytes = 128 * kScatterRowPitch + 128 * 8;
constexpr int kGemmSmemBytesScatter =
    kStagesScatter * kStageBytes + kSmemAux + 1024 + 2 * kScatterWgBytes;
static_assert(kGemmSmemBytesScatter <= 232448, "shared memory per CTA");

// gate/up kernel: the tile's 128 x 128 e4m3 bytes are staged (row pitch 144 B) so
// that each output row leaves the SM as one 128-byte run
constexpr int kSwigluRowPitch = 144;
constexpr int kGemmSmemBytesSwiglu = kGemmSmemBytes + 128 * kSwigluRowPitch;

enum Role { kRoleProducer = 1, kRoleMma = 2, kRoleEpilogue = 3, kRoleStore = 5 };

struct GemmParams {
  const float* scale_a;   // [K/128, m_total]
  const float* scale_b0;  // gate (swiglu) or weight scales [G*N/128, K/128]
  const float* scale_b1;  // up scales (swiglu); unused otherwise
  void* out;              // swiglu: e4m3 [m_total, N]; else bf16 / f32 [m_total, N]
  float* scale_d;         // swiglu: [N/128, m_total]
  const int32_t* layout;  // contiguous: expert per row; masked: rows per expert
  int32_t* status;        // optional int32[4]
  int m_total, N, K, G;
  int masked, max_m, out_f32;
  int num_m_blocks, num_n_blocks;
  int group_m;             // row blocks walked together (tile order), see tile_mn
  const int32_t* m_valid;  // optional device word: rows in use (<= m_total); blocks beyond it are not visited
  // optional scatter epilogue of the down projection (EP combine fused into the
  // GEMM): row r is stored to peer buffer scatter_out[scatter_rank[r]] at row
  // scatter_pos[r] instead of out[r]
  const uint64_t* scatter_out;
  size_t scatter_off;  // byte offset of the destination buffer behind every base address
  const int32_t* scatter_rank;
  const int32_t* scatter_pos;
  uint32_t wait_hint_ns;  // suspend-time hint of the mbarrier waits (0 = plain polling)
  // Fused dispatch (kOptFused): the last n_comm CTAs pull this rank's rows from
  // their source ranks (ep_pull.cuh) and count them per 128-row block; the other
  // CTAs run the GEMM and wait for a block's rows before they load it.
  const int32_t* arrive_cnt;   // [num_m_blocks] rows landed so far
  const int32_t* arrive_need;  // [num_m_blocks] rows the block holds
  int n_comm;
  PullParams pull;
  // max_ctas > 0 bounds the grid (chunked MLP: a gate/up and a down launch share the SMs).
  int max_ctas;
  // Chunked MLP: optional device word, first row of this launch's range (a multiple of
  // 128 * group_m); the range ends at *m_valid. Row blocks before it are not visited.
  const int32_t* m_begin;
  // bf16 kernel, dense fp32 output only: the K range is cut into k_splits slices of
  // kb_per_split 64-element blocks; slice s of a tile is an item of its own and writes
  // its partial sums to out + s * m_total * N (summed by the caller). 0 / 1: no split.
  int k_splits, kb_per_split;
};

struct TileInfo {
  int m_block, n_block, g, rows_valid;
  bool valid;
};

// Tile index -> (row block, N block). group_m <= 1: N fastest, so the CTAs of a
// wave share few row blocks and cover every N block of them. With many N blocks
// (wide experts) a wave would then touch every weight tile of an expert once and
// never again before it has left L2; group_m > 1 walks group_m row blocks together,
// row block fastest, so that a wave re-uses each weight tile group_m times.
__device__ __forceinline__ void tile_mn(const GemmParams& p, int tile, int& m_block, int& n_block) {
  if (p.group_m <= 1) {
    m_block = tile / p.num_n_blocks;
    n_block = tile - m_block * p.num_n_blocks;
    return;
  }
  const int per_group = p.group_m * p.num_n_blocks;
  const int grp = tile / per_group;
  const int w = tile - grp * per_group;
  const int m0 = grp * p.group_m;
  const int gm = min(p.group_m, p.num_m_blocks - m0);
  n_block = w / gm;
  m_block = m0 + (w - n_block * gm);
}

// The one layout word that decides a tile: the expert id of the block's first
// row (contiguous) or the expert's row count (masked).
__device__ __forceinline__ size_t tile_key_index(const GemmParams& p, int tile) {
  int m_block, n_block;
  tile_mn(p, tile, m_block, n_block);
  return p.masked ? (size_t)(m_block / (p.max_m / kBM)) : (size_t)m_block * kBM;
}

__device__ __forceinline__ TileInfo make_tile(const GemmParams& p, int tile, int key) {
  TileInfo t;
  tile_mn(p, tile, t.m_block, t.n_block);
  if (!p.masked) {
    // every expert's rows start on a multiple of 128, so the first row decides
    t.g = key;
    t.valid = t.g >= 0 && t.g < p.G;
    t.rows_valid = kBM;
  } else {
    const int blocks_per_expert = p.max_m / kBM;
    t.g = t.m_block / blocks_per_expert;
    const int m_in = (t.m_block - t.g * blocks_per_expert) * kBM;
    t.valid = m_in < key;
    t.rows_valid = min(kBM, key - m_in);
  }
  return t;
}

// First tile of this CTA: a launch over a row range starts at the range's first row
// block. Evaluated where a role's tile loop starts (nothing stays live in the loops).
__device__ __forceinline__ int first_tile_of(const GemmParams& p) {
  int t = blockIdx.x;
  if (p.m_begin != nullptr) t += (max(__ldg(p.m_begin), 0) / kBM) * p.num_n_blocks;
  return t;
}

// Self-contained form used by the producer and MMA warps, which run on 40
// registers: kept as lean as possible (a spill in their loops sits on the
// critical path of every K block).
__device__ __forceinline__ TileInfo get_tile(const GemmParams& p, int tile) {
  TileInfo t;
  tile_mn(p, tile, t.m_block, t.n_block);
  if (!p.masked) {
    t.g = __ldg(p.layout + (size_t)t.m_block * kBM);
    t.valid = t.g >= 0 && t.g < p.G;
    t.rows_valid = kBM;
  } else {
    const int blocks_per_expert = p.max_m / kBM;
    t.g = t.m_block / blocks_per_expert;
    const int m_in = (t.m_block - t.g * blocks_per_expert) * kBM;
    const int cnt = __ldg(p.layout + t.g);
    t.valid = m_in < cnt;
    t.rows_valid = min(kBM, cnt - m_in);
  }
  return t;
}

// Walks the tiles of this CTA in order. The layout word of the NEXT candidate
// tile is requested while the current tile is processed, so that the global
// load latency is not paid at every tile boundary.
struct TileWalker {
  int tile, cand, cand_key, stride;
  TileInfo ti;
  __device__ __forceinline__ void prefetch(const GemmParams& p, int num_tiles) {
    cand = tile + stride;
    cand_key = cand < num_tiles ? __ldg(p.layout + tile_key_index(p, cand)) : 0;
  }
  // first valid tile at or after `start`
  __device__ __forceinline__ void seek(const GemmParams& p, int start, int num_tiles) {
    tile = start;
    ti.valid = false;
    while (tile < num_tiles) {
      ti = make_tile(p, tile, __ldg(p.layout + tile_key_index(p, tile)));
      if (ti.valid) break;
      tile += stride;
    }
  }
  // move to the next valid tile, using the prefetched word when it applies
  __device__ __forceinline__ void advance(const GemmParams& p, int num_tiles) {
    if (cand < num_tiles) {
      const TileInfo c = make_tile(p, cand, cand_key);
      if (c.valid) {
        tile = cand;
        ti = c;
        return;
      }
      seek(p, cand + stride, num_tiles);
    } else {
      tile = num_tiles;
      ti.valid = false;
    }
  }
};

// wait for every tcgen05.ld issued so far; the registers are listed as in/out
// operands so that no use of them can be scheduled above the wait
__device__ __forceinline__ void tmem_wait_ld_fence(uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]),
        "+r"(v[7]), "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]),
        "+r"(v[14]), "+r"(v[15]), "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]),
        "+r"(v[21]), "+r"(v[22]), "+r"(v[23]), "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]),
        "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
      :
      : "memory");
}

// Bulk asynchronous copy shared -> global (local or peer memory): both addresses
// 16-byte aligned, size a multiple of 16 bytes. Completion is tracked per thread
// through bulk groups.
__device__ __forceinline__ void bulk_store_s2g(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
               "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_group_read0() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_group0() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// acc[kOffset/2 .. kOffset/2+16) += v[0..32) * m, accumulators kept as float2 pairs
template <int kOffset>
__device__ __forceinline__ void fma_chunk(float2 (&acc)[64], const uint32_t (&v)[32], float m) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    acc[kOffset / 2 + i].x = fmaf(__uint_as_float(v[2 * i]), m, acc[kOffset / 2 + i].x);
    acc[kOffset / 2 + i].y = fmaf(__uint_as_float(v[2 * i + 1]), m, acc[kOffset / 2 + i].y);
  }
}

// kOffload: the finished tile leaves the SM through a store warp. The promotion
// warps only stage it in shared memory and signal an mbarrier; warp 2 (gate/up;
// warps 2 and 3, one per column half, for the down projection) then issues one
// bulk asynchronous copy (cp.async.bulk shared -> global) per row, to local
// memory or straight to a peer GPU, while the promotion warps are already in the
// next tile's K loop. Without it the promotion warps copy the tile out themselves.
// kOpt bits: kOptOffload (above); kOptEarly: open the next tile (first scales,
// layout word) before the epilogue instead of after it; kOptTanh: SiLU through one
// tanh.approx instead of ex2 + rcp (half the special-function work of the SwiGLU
// epilogue).
// kOptFused: dispatch fused into the GEMM (see GemmParams::arrive_cnt).
constexpr int kOptOffload = 1, kOptEarly = 2, kOptTanh = 4, kOptFused = 8;
// Fused dispatch: wait (bounded) until all rows of a 128-row block have been
// published by the comm CTAs. Every lane of the warp polls the same word.
__device__ __forceinline__ bool wait_rows_arrived(const GemmParams& p, int m_block,
                                                  volatile int* abort_flag) {
  const int need = __ldg(p.arrive_need + m_block);
  if (ld_acquire_gpu_s32(p.arrive_cnt + m_block) >= need) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (ld_acquire_gpu_s32(p.arrive_cnt + m_block) < need) {
    if ((++spins & 15u) == 0u) {
      if (*abort_flag != 0) return false;
      if (global_timer_ns() - t0 > kPullLimitNs) {
        *abort_flag = 1;
        return false;
      }
    }
    __nanosleep(100);
  }
  return true;
}

template <bool kSwiglu, bool kScatter = false, int kOpt = 0>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tm_a,
                        const __grid_constant__ CUtensorMap tm_b0,
                        const __grid_constant__ CUtensorMap tm_b1, const GemmParams p) {
  constexpr int kSt = kScatter ? kStagesScatter : kStages;  // pipeline stages
  constexpr bool kOffload = (kOpt & kOptOffload) != 0;
  constexpr bool kEarly = (kOpt & kOptEarly) != 0;
  constexpr bool kTanh = (kOpt & kOptTanh) != 0;
  constexpr bool kFused = (kOpt & kOptFused) != 0;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte alignment
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t smem_base = smem_u32(smem);
  uint8_t* aux = smem + kSt * kStageBytes;
  const uint32_t bar_base = smem_u32(aux);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kSt + s); };
  auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * kSt + b); };
  auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * kSt + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux + 8 * (2 * kSt + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* amax_x = reinterpret_cast<float*>(aux + 256);  // [2 tile parities][2 halves][128 rows]
  // hand-off of the staged output tile to the store warp(s) (kOffload)
  auto staged_bar = [&](int h) { return bar_base + 3072u + 8u * h; };
  auto stage_free_bar = [&](int h) { return bar_base + 3072u + 16u + 8u * h; };
  // output staging: row-store epilogue of the down projection (kScatter), or the
  // 128 x 128-byte tile of the gate/up kernel
  uint8_t* scatter_smem = aux + kSmemAux;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSt; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tmem_full_bar(b), 1);
      mbar_init(tmem_empty_bar(b), kEpiWarps);
    }
    if constexpr (kOffload) {
      // gate/up: all eight promotion warps stage one tile; down: four per column half
      mbar_init(staged_bar(0), kSwiglu ? kEpiWarps : kEpiWarps / 2);
      mbar_init(staged_bar(1), kEpiWarps / 2);
      mbar_init(stage_free_bar(0), 1);
      mbar_init(stage_free_bar(1), 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b0);
    tma_prefetch_desc(&tm_b1);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // with a device-side row count (EP: known only after the count exchange) the
  // tile range shrinks to the rows in use
  int num_m_blocks = p.num_m_blocks;
  if (p.m_valid != nullptr) {
    num_m_blocks = min(num_m_blocks, ceil_div(max(__ldg(p.m_valid), 0), kBM));
    // whole groups of row blocks (blocks past the rows in use hold padding only)
    if (p.group_m > 1) num_m_blocks = min(p.num_m_blocks, round_up(num_m_blocks, p.group_m));
  }
  const int num_tiles = num_m_blocks * p.num_n_blocks;
  const int num_kb = p.K / kBK;
  // tiles are dealt round-robin to the CTAs that run the GEMM
  const int tile_stride = (int)gridDim.x - (kFused ? p.n_comm : 0);

  if (kFused && (int)blockIdx.x >= tile_stride) {
    // ------------------------------------------------ comm CTA: pull rows --
    pull_rows(p.pull, ((int)blockIdx.x - tile_stride) * (kGemmThreads / 32) + warp,
              p.n_comm * (kGemmThreads / 32));
  } else if (warp < 4) {
    setmaxnreg_dec<kRegsProducerWg>();
    if (warp == 0) {
      // ------------------------------------------------------ TMA producer --
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // (the producer and MMA warps run on 40 registers: they use the plain tile
      // loop; only the promotion warps prefetch the next tile's layout word)
      for (int tile = first_tile_of(p); tile < num_tiles && ok; tile += tile_stride) {
        const TileInfo ti = get_tile(p, tile);
        if (!ti.valid) continue;
        const int a_row = ti.m_block * kBM;
        const int b_row0 = ti.g * p.N + (kSwiglu ? ti.n_block * 128 : ti.n_block * 256);
        const int b_row1 = kSwiglu ? b_row0 : b_row0 + 128;
        if constexpr (kFused) {
          // the block's rows must have landed before the TMA unit reads them
          if (!wait_rows_arrived(p, ti.m_block, abort_flag)) {
            if (lane == 0) report_timeout(p.status, kRoleProducer, tile, -4);
            break;
          }
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, p.wait_hint_ns)) {
            if (lane == 0) report_timeout(p.status, kRoleProducer, tile, kb);
            ok = false;
            break;
          }
          if (lane == 0) {
            const uint32_t sa = smem_base + stage * kStageBytes;
            const uint32_t sb = sa + kTileABytes;
            mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
            tma_load_2d(sa, &tm_a, kb * kBK, a_row, full_bar(stage));
            tma_load_2d(sb, &tm_b0, kb * kBK, b_row0, full_bar(stage));
            tma_load_2d(sb + kTileBBytes / 2, &tm_b1, kb * kBK, b_row1, full_bar(stage));
          }
          __syncwarp();
          if (++stage == kSt) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    } else if (warp == 1) {
      // -------------------------------------------------------- MMA issuer --
      constexpr uint32_t idesc = make_idesc_e4m3_f32(kBM, kUmmaN);
      int stage = 0, buf = 0;
      uint32_t phase = 0, bphase = 0;
      bool ok = true;
      for (int tile = first_tile_of(p); tile < num_tiles && ok; tile += tile_stride) {
        const TileInfo ti = get_tile(p, tile);
        if (!ti.valid) continue;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(tmem_empty_bar(buf), bphase ^ 1u, abort_flag, p.wait_hint_ns) ||
              !mbar_wait_bounded(full_bar(stage), phase, abort_flag, p.wait_hint_ns)) {
            if (lane == 0) report_timeout(p.status, kRoleMma, tile, kb);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (lane == 0) {
            const uint32_t sa = smem_base + stage * kStageBytes;
            const uint64_t a_desc = make_sw128_kmajor_desc(sa);
            const uint64_t b_desc = make_sw128_kmajor_desc(sa + kTileABytes);
            const uint32_t d_tmem = tmem_base + (uint32_t)buf * kUmmaN;
#pragma unroll
            for (int k4 = 0; k4 < kBK / kUmmaK; ++k4) {
              // advance 32 bytes along K inside the 128-byte swizzle atom
              const uint64_t koff = (uint64_t)((k4 * kUmmaK) >> 4);
              tc_mma_f8f6f4(d_tmem, a_desc + koff, b_desc + koff, idesc, k4 > 0 ? 1u : 0u);
            }
            tc_commit(empty_bar(stage));     // smem stage reusable once the MMAs are done
            tc_commit(tmem_full_bar(buf));   // partial sums ready for the epilogue warps
          }
          __syncwarp();
          if (++stage == kSt) {
            stage = 0;
            phase ^= 1u;
          }
          buf ^= 1;
          if (buf == 0) bphase ^= 1u;
        }
      }
    } else if (kOffload && (warp == 2 || (!kSwiglu && warp == 3))) {
      // ------------------------------------------------------- store warp --
      // Takes every staged tile (gate/up) or column half (down) out of shared
      // memory: one bulk asynchronous copy per row, lane l owns rows l, l+32,
      // l+64, l+96. Down projection: one warp per column half (warps 2 and 3).
      const int h = warp - 2;
      uint32_t sphase = 0;
      for (int tile = first_tile_of(p); tile < num_tiles; tile += tile_stride) {
        const TileInfo ti = get_tile(p, tile);
        if (!ti.valid) continue;
        if (!mbar_wait_bounded(staged_bar(h), sphase, abort_flag, p.wait_hint_ns)) {
          if (lane == 0) report_timeout(p.status, kRoleStore, tile, -1);
          break;
        }
        if constexpr (kSwiglu) {
          uint8_t* out_tile = reinterpret_cast<uint8_t*>(p.out) + (size_t)ti.n_block * 128;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int r = lane + 32 * i;
            const int grow = ti.m_block * kBM + r;
            if (grow < p.m_total)
              bulk_store_s2g(out_tile + (size_t)grow * p.N,
                             smem_u32(scatter_smem + r * kSwigluRowPitch), 128);
          }
        } else {
          const uint8_t* stage = scatter_smem + h * kScatterWgBytes;
          const uint64_t* row_dst =
              reinterpret_cast<const uint64_t*>(stage + 128 * kScatterRowPitch);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int r = lane + 32 * i;
            const uint64_t d = row_dst[r];
            if (d != 0)
              bulk_store_s2g(reinterpret_cast<void*>(d), smem_u32(stage + r * kScatterRowPitch),
                             256);
          }
        }
        bulk_commit_group();
        bulk_wait_group_read0();   // the staging area has been read: it may be rewritten
        __syncwarp();
        if (lane == 0) mbar_arrive(stage_free_bar(h));
        sphase ^= 1u;
      }
      bulk_wait_group0();          // every row has reached global memory
    }
  } else {
    // ------------------------------------------- promotion + epilogue warps --
    setmaxnreg_inc<kRegsEpilogueWg>();
    const int h = (warp - 4) >> 2;  // column half owned by this warpgroup
    const int quarter = warp & 3;   // TMEM lane quarter this warp may access
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    int buf = 0;
    uint32_t bphase = 0;
    int tile_parity = 0;
    uint32_t sphase = 0;  // phase of the staging hand-off (kOffload)
    bool ok = true;
    const int n_scale_blocks = p.N / 128;
    // Measured on B200: asking for the next tile's layout word one tile early
    // pays off for the gate/up kernel (long K loop, -16 %), not for the down
    // kernel (short K loop), which keeps the plain tile loop.
    constexpr bool kTileLookAhead = kSwiglu || kOffload;
    // Per-tile addresses of this thread's scales, and the values a tile needs
    // first (scales of K block 0, layout word of the row).
    struct EpiTile {
      const float *sa_ptr, *sb0_ptr, *sb1_ptr;
      float sa0, sb00, sb10;
      int row, lay;
    };
    auto open_tile = [&](const TileInfo& t) {
      EpiTile e;
      if constexpr (kFused) {
        // the scales of the block are written by the comm CTAs: wait for them too
        if (!wait_rows_arrived(p, t.m_block, abort_flag)) ok = false;
      }
      e.row = t.m_block * kBM + row_in_tile;
      const int row_ld = e.row < p.m_total ? e.row : p.m_total - 1;
      int nb0;  // weight scale block for the first multiplier
      if (kSwiglu) {
        nb0 = t.n_block;
      } else {
        nb0 = t.n_block * 2 + h;
        if (nb0 >= n_scale_blocks) nb0 = n_scale_blocks - 1;  // half tile past N: unused
      }
      e.sa_ptr = p.scale_a + row_ld;
      e.sb0_ptr = p.scale_b0 + ((size_t)t.g * n_scale_blocks + nb0) * num_kb;
      e.sb1_ptr = kSwiglu ? p.scale_b1 + ((size_t)t.g * n_scale_blocks + nb0) * num_kb : e.sb0_ptr;
      e.sa0 = __ldg(e.sa_ptr);
      e.sb00 = __ldg(e.sb0_ptr);
      e.sb10 = __ldg(e.sb1_ptr);
      // the row's layout word is needed only in the tile epilogue; the look-ahead
      // path asks for it here, the plain path when it gets there
      e.lay = (kTileLookAhead && !p.masked) ? __ldg(p.layout + row_ld) : 0;
      return e;
    };
    TileWalker w;
    w.stride = tile_stride;
    EpiTile et{};
    int tile = kTileLookAhead ? 0 : first_tile_of(p);
    if constexpr (kTileLookAhead) {
      w.seek(p, first_tile_of(p), num_tiles);
      if (w.tile < num_tiles) et = open_tile(w.ti);
      tile = w.tile;
    }
    while (tile < num_tiles && ok) {
      TileInfo ti;
      if constexpr (kTileLookAhead) {
        ti = w.ti;
        w.prefetch(p, num_tiles);
      } else {
        ti = get_tile(p, tile);
        if (!ti.valid) {
          tile += tile_stride;
          continue;
        }
        et = open_tile(ti);
      }
      const int row = et.row;
      const float* sa_ptr = et.sa_ptr;
      const float* sb0_ptr = et.sb0_ptr;
      const float* sb1_ptr = et.sb1_ptr;
      const int lay_row = et.lay;

      float2 acc2[64];  // 128 fp32 accumulators; ACC(i) names element i
#define ACC(i) (((i)&1) ? acc2[(i) >> 1].y : acc2[(i) >> 1].x)
#pragma unroll
      for (int i = 0; i < 64; ++i) acc2[i] = make_float2(0.0f, 0.0f);

      // scales of the next K block are fetched while the current one is promoted
      // (deeper look-ahead was measured slower: it costs registers in this loop)
      float sa_next = et.sa0, sb0_next = et.sb00, sb1_next = et.sb10;
      // running pointers (one 64-bit value each instead of base + index: the
      // loop is register-critical, and this form measured 2 % faster)
      const float* sa_run = sa_ptr + p.m_total;
      const float* sb_run = sb0_ptr + 1;
      const ptrdiff_t sb_delta = sb1_ptr - sb0_ptr;
      // kept rolled: unrolled by two the loop was measured 17 % slower on B200
#pragma unroll 1
      for (int kb = 0; kb < num_kb; ++kb) {
        const float m0 = sa_next * sb0_next;
        const float m1 = sa_next * sb1_next;
        if (kb + 1 < num_kb) {
          sa_next = __ldg(sa_run);
          sb0_next = __ldg(sb_run);
          sb1_next = __ldg(sb_run + sb_delta);
          sa_run += p.m_total;
          ++sb_run;
        }
        if (!mbar_wait_bounded(tmem_full_bar(buf), bphase, abort_flag, p.wait_hint_ns)) {
          if (lane == 0) report_timeout(p.status, kRoleEpilogue, tile, kb);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t t0 = tmem_base + lane_addr + (uint32_t)buf * kUmmaN;
        // column offsets of this thread's four 32-column chunks
        const uint32_t c0 = kSwiglu ? h * 64 : h * 128;
        const uint32_t c1 = c0 + 32;
        const uint32_t c2 = kSwiglu ? 128 + h * 64 : c0 + 64;
        const uint32_t c3 = c2 + 32;
        const float mhi = kSwiglu ? m1 : m0;
        // two 32-register staging buffers: the next TMEM load is in flight while
        // the previous chunk is folded in (one buffer, two loads per wait, packed
        // f32x2 FMAs and a plain tcgen05.wait::ld were all measured slower)
        uint32_t va[32], vb[32];
        tmem_ld_32x32b_x32(t0 + c0, va);
        tmem_wait_ld_fence(va);
        tmem_ld_32x32b_x32(t0 + c1, vb);
        fma_chunk<0>(acc2, va, m0);
        tmem_wait_ld_fence(vb);
        tmem_ld_32x32b_x32(t0 + c2, va);
        fma_chunk<32>(acc2, vb, m0);
        tmem_wait_ld_fence(va);
        tmem_ld_32x32b_x32(t0 + c3, vb);
        fma_chunk<64>(acc2, va, mhi);
        tmem_wait_ld_fence(vb);
        // all TMEM reads of this warp are done: hand the buffer back
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(tmem_empty_bar(buf));
        fma_chunk<96>(acc2, vb, mhi);
        buf ^= 1;
        if (buf == 0) bphase ^= 1u;
      }
      if (!ok) break;

      // With the store warp (kOffload) the next tile is opened before the epilogue:
      // its layout word was requested a tile ago, and the first scales it needs are
      // in flight while this tile's epilogue runs.
      // Down projection: the next tile is opened before the epilogue, so that the
      // first scales it needs are in flight while this tile is converted and staged.
      // Gate/up: the same, but only after the SwiGLU loop, when the registers of the
      // `up` accumulators are free (opened earlier, the extra live values spill).
      EpiTile et_next{};
      if constexpr (kTileLookAhead && kEarly && !kSwiglu) {
        w.advance(p, num_tiles);
        if (w.tile < num_tiles) et_next = open_tile(w.ti);
      }

      // ------------------------------------------------------- tile epilogue --
      bool row_ok = row < p.m_total;
      if (row_ok) {
        if (p.masked) row_ok = row_in_tile < ti.rows_valid;
        else row_ok = (kTileLookAhead ? lay_row : __ldg(p.layout + row)) >= 0;
      }
      if (kSwiglu) {
        // acc[0..63] = gate, acc[64..127] = up for columns n_block*128 + h*64 + [0,64)
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float g = ACC(i);
          float y;
          if constexpr (kTanh) {
            // g * sigmoid(g) = hg * (tanh(hg) + 1) with hg = g / 2
            const float hg = 0.5f * g;
            y = ACC(64 + i) * fmaf(hg, tanh_approx(hg), hg);
          } else {
            y = __fdividef(ACC(64 + i) * g, 1.0f + __expf(-g));
          }
          ACC(i) = y;
          amax = fmaxf(amax, fabsf(y));
        }
        if constexpr (kTileLookAhead && kEarly) {
          w.advance(p, num_tiles);
          if (w.tile < num_tiles) et_next = open_tile(w.ti);
        }
        float* xchg = amax_x + tile_parity * 256;
        xchg[h * 128 + row_in_tile] = amax;
        named_barrier_sync(1, kEpiThreads);
        amax = fmaxf(amax, xchg[(h ^ 1) * 128 + row_in_tile]);
        float s = quant_scale_from_amax(amax);
        if (!row_ok) s = 1.0f;
        // one reciprocal per row instead of 64 IEEE divisions; the conversion
        // saturates to +-448, which is the clamp
        const float inv = amax > 0.0f ? __fdiv_rn(kFp8Max, amax) : 1.0f;
        if constexpr (kOffload) {
          // the store warp has taken the previous tile out of the staging area
          if (!mbar_wait_bounded(stage_free_bar(0), sphase ^ 1u, abort_flag, p.wait_hint_ns)) {
            if (lane == 0) report_timeout(p.status, kRoleEpilogue, tile, -2);
            break;
          }
        }
        if (row < p.m_total) {
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            packed[i] = row_ok ? f32x4_to_e4m3x4(ACC(4 * i) * inv, ACC(4 * i + 1) * inv,
                                                 ACC(4 * i + 2) * inv, ACC(4 * i + 3) * inv)
                               : 0u;
          }
          // this thread's 64 bytes of the row into the tile's staging area
          uint8_t* st_row = scatter_smem + row_in_tile * kSwigluRowPitch + h * 64;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            reinterpret_cast<uint4*>(st_row)[i] =
                make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
          if (h == 0) p.scale_d[(size_t)ti.n_block * p.m_total + row] = s;
        }
        if constexpr (kOffload) {
          // hand the staged tile to the store warp and go on with the next tile
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(staged_bar(0));
          sphase ^= 1u;
        } else {
        // both warpgroups have staged their halves: every row (128 bytes) goes out
        // as one run, eight lanes per row
        named_barrier_sync(3, kEpiThreads);
        {
          const int tid = threadIdx.x - 128;
          uint8_t* out_tile = reinterpret_cast<uint8_t*>(p.out) + (size_t)ti.n_block * 128;
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int u = it * kEpiThreads + tid;
            const int r = u >> 3, part = u & 7;
            const int grow = ti.m_block * kBM + r;
            if (grow < p.m_total)
              *reinterpret_cast<uint4*>(out_tile + (size_t)grow * p.N + part * 16) =
                  *reinterpret_cast<const uint4*>(scatter_smem + r * kSwigluRowPitch + part * 16);
          }
        }
        }
        tile_parity ^= 1;
      } else {
        const int col0 = ti.n_block * 256 + h * 128;
        if constexpr (kScatter) {
          // Send every row home: to the rank it came from, at its (token, slot)
          // position. Thread r owns row r of the tile: it writes its 128 columns
          // (256 B) to the warpgroup's staging area; then 16 lanes per row store the
          // row as one contiguous 256-byte run to the peer.
          uint8_t* stage = scatter_smem + h * kScatterWgBytes;
          uint64_t* row_dst = reinterpret_cast<uint64_t*>(stage + 128 * kScatterRowPitch);
          const int wg_tid = threadIdx.x - (4 + 4 * h) * 32;  // 0..127 inside the warpgroup
          uint64_t my_dst = 0;
          if (row_ok && col0 < p.N) {
            if (p.scatter_out != nullptr) {
              const int src = __ldg(p.scatter_rank + row);
              const int pos = __ldg(p.scatter_pos + row);
              if (src >= 0 && pos >= 0)
                my_dst = __ldg(p.scatter_out + src) + p.scatter_off + ((size_t)pos * p.N + col0) * 2;
            }
          }
          // local output: every row of the tile is written, rows that hold no
          // token (padding, beyond a masked expert's count) as zeros
          const bool local = p.scatter_out == nullptr;
          if (local && row < p.m_total && col0 < p.N)
            my_dst = reinterpret_cast<uint64_t>(p.out) + ((size_t)row * p.N + col0) * 2;
          if constexpr (kOffload) {
            // the store warp has taken the previous tile out of this half's staging area
            if (!mbar_wait_bounded(stage_free_bar(h), sphase ^ 1u, abort_flag, p.wait_hint_ns)) {
              if (lane == 0) report_timeout(p.status, kRoleEpilogue, tile, -2);
              break;
            }
          }
          row_dst[row_in_tile] = my_dst;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            uint32_t wv[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __nv_bfloat162 b = __floats2bfloat162_rn(ACC(8 * i + 2 * j), ACC(8 * i + 2 * j + 1));
              wv[j] = row_ok ? *reinterpret_cast<uint32_t*>(&b) : 0u;
            }
            *reinterpret_cast<uint4*>(stage + row_in_tile * kScatterRowPitch + 16 * i) =
                make_uint4(wv[0], wv[1], wv[2], wv[3]);
          }
          if constexpr (kOffload) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(staged_bar(h));
            sphase ^= 1u;
          } else {
          named_barrier_sync(2 + h, 128);
          // 128 rows x 16 sixteen-byte pieces; consecutive lanes take consecutive pieces
#pragma unroll 4
          for (int it = 0; it < 16; ++it) {
            const int u = it * 128 + wg_tid;
            const int r = u >> 4, part = u & 15;
            const uint64_t d = row_dst[r];
            if (d != 0) {
              const uint4 v =
                  *reinterpret_cast<const uint4*>(stage + r * kScatterRowPitch + 16 * part);
              *reinterpret_cast<uint4*>(d + (size_t)(part * 16)) = v;
            }
          }
          // the staging area is reused by this warpgroup's next tile
          named_barrier_sync(2 + h, 128);
          }
        } else
        if (row < p.m_total && col0 < p.N) {
          if (p.out_f32) {
            float* dst = reinterpret_cast<float*>(p.out) + (size_t)row * p.N + col0;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float4 v = row_ok ? make_float4(ACC(4 * i), ACC(4 * i + 1), ACC(4 * i + 2),
                                              ACC(4 * i + 3))
                                : make_float4(0.f, 0.f, 0.f, 0.f);
              reinterpret_cast<float4*>(dst)[i] = v;
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)row * p.N + col0;
            constexpr bool store = true;
            if (store) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                uint32_t wv[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  __nv_bfloat162 b =
                      __floats2bfloat162_rn(ACC(8 * i + 2 * j), ACC(8 * i + 2 * j + 1));
                  wv[j] = row_ok ? *reinterpret_cast<uint32_t*>(&b) : 0u;
                }
                reinterpret_cast<uint4*>(dst)[i] = make_uint4(wv[0], wv[1], wv[2], wv[3]);
              }
            }
          }
        }
      }
      if constexpr (kTileLookAhead && kEarly) {
        et = et_next;
        tile = w.tile;
      } else if constexpr (kTileLookAhead) {
        // next tile (its layout word was requested at the start of this one)
        w.advance(p, num_tiles);
        if (w.tile < num_tiles) et = open_tile(w.ti);
        tile = w.tile;
      } else {
        tile += tile_stride;
      }
    }
  }

#undef ACC
  // ---------------------------------------------------------------- teardown --
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------- BF16 GEMM --
// D[M,N] = A[M,K] * B[g][N,K]^T in bf16 with fp32 accumulation, dense (one
// group) or grouped like the FP8 kernels (reference: csrc/apis/moe.hpp:72-98 ->
// sm90_bf16_gemm / sm90_bf16_grouped_gemm_*). Same warp roles, TMA ring and tile
// walk as above; without block scales the whole K range of a tile accumulates in
// one TMEM buffer (tcgen05.mma kind::f16), so the eight epilogue warps only run
// once per tile: read the 128 x 256 fp32 tile, convert, and store whole rows
// through the staging area while the tensor core fills the other buffer.
constexpr int kB16K = 64;                 // bf16 K elements per stage = 128 bytes per row
constexpr int kStagesB16 = 3;
constexpr int kGemmSmemBytesB16 =
    kStagesB16 * kStageBytes + kSmemAux + 1024 + 2 * kScatterWgBytes;
static_assert(kGemmSmemBytesB16 <= 232448, "shared memory per CTA");

// kind::f16 instruction descriptor: bf16 x bf16 -> f32, both operands K-major
__host__ __device__ constexpr uint32_t make_idesc_bf16_f32(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_bf16_kernel(const __grid_constant__ CUtensorMap tm_a,
                         const __grid_constant__ CUtensorMap tm_b, const GemmParams p) {
  constexpr int kSt = kStagesB16;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t smem_base = smem_u32(smem);
  uint8_t* aux = smem + kSt * kStageBytes;
  const uint32_t bar_base = smem_u32(aux);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kSt + s); };
  auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * kSt + b); };
  auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * kSt + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux + 8 * (2 * kSt + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* stage_smem = aux + kSmemAux;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kSt; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tmem_full_bar(b), 1);
      mbar_init(tmem_empty_bar(b), kEpiWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  int num_m_blocks = p.num_m_blocks;
  if (p.m_valid != nullptr) num_m_blocks = min(num_m_blocks, ceil_div(max(__ldg(p.m_valid), 0), kBM));
  const int num_tiles = num_m_blocks * p.num_n_blocks;
  const int num_kb = ceil_div(p.K, kB16K);  // a ragged last block is zero-filled by TMA
  // work items: (tile, K slice), the slices of a tile on neighbouring CTAs
  const int splits = p.k_splits > 1 ? p.k_splits : 1;
  const int kb_per = p.k_splits > 1 ? p.kb_per_split : num_kb;
  const int num_items = num_tiles * splits;
  // dense form: no layout, every tile belongs to group 0
  auto tile_of = [&](int tile) {
    if (p.layout != nullptr) return get_tile(p, tile);
    TileInfo t;
    t.m_block = tile / p.num_n_blocks;
    t.n_block = tile - t.m_block * p.num_n_blocks;
    t.g = 0;
    t.rows_valid = kBM;
    t.valid = true;
    return t;
  };

  if (warp == 0) {
    // -------------------------------------------------------- TMA producer --
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      const int tile = item / splits;
      const int kb0 = (item - tile * splits) * kb_per, kb1 = min(kb0 + kb_per, num_kb);
      const TileInfo ti = tile_of(tile);
      if (!ti.valid) continue;
      const int a_row = ti.m_block * kBM;
      const int b_row = ti.g * p.N + ti.n_block * 256;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, p.wait_hint_ns)) {
          if (lane == 0) report_timeout(p.status, kRoleProducer, tile, kb);
          ok = false;
          break;
        }
        if (lane == 0) {
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb = sa + kTileABytes;
          mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
          tma_load_2d(sa, &tm_a, kb * kB16K, a_row, full_bar(stage));
          tma_load_2d(sb, &tm_b, kb * kB16K, b_row, full_bar(stage));
          tma_load_2d(sb + kTileBBytes / 2, &tm_b, kb * kB16K, b_row + 128, full_bar(stage));
        }
        __syncwarp();
        if (++stage == kSt) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer --
    constexpr uint32_t idesc = make_idesc_bf16_f32(kBM, kUmmaN);
    int stage = 0, buf = 0;
    uint32_t phase = 0, bphase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      const int tile = item / splits;
      const int kb0 = (item - tile * splits) * kb_per, kb1 = min(kb0 + kb_per, num_kb);
      const TileInfo ti = tile_of(tile);
      if (!ti.valid) continue;
      if (!mbar_wait_bounded(tmem_empty_bar(buf), bphase ^ 1u, abort_flag, p.wait_hint_ns)) {
        if (lane == 0) report_timeout(p.status, kRoleMma, tile, -1);
        break;
      }
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait_bounded(full_bar(stage), phase, abort_flag, p.wait_hint_ns)) {
          if (lane == 0) report_timeout(p.status, kRoleMma, tile, kb);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint64_t a_desc = make_sw128_kmajor_desc(sa);
          const uint64_t b_desc = make_sw128_kmajor_desc(sa + kTileABytes);
          const uint32_t d_tmem = tmem_base + (uint32_t)buf * kUmmaN;
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            // 16 bf16 = 32 bytes along K inside the 128-byte swizzle atom
            const uint64_t koff = (uint64_t)((k4 * 32) >> 4);
            tc_mma_f16(d_tmem, a_desc + koff, b_desc + koff, idesc, (kb > kb0 || k4 > 0) ? 1u : 0u);
          }
          tc_commit(empty_bar(stage));
          if (kb == kb1 - 1) tc_commit(tmem_full_bar(buf));  // the tile (or its K slice) is complete
        }
        __syncwarp();
        if (++stage == kSt) {
          stage = 0;
          phase ^= 1u;
        }
      }
      buf ^= 1;
      if (buf == 0) bphase ^= 1u;
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------ epilogue warps --
    const int h = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int wg_tid = threadIdx.x - (4 + 4 * h) * 32;
    uint8_t* stage = stage_smem + h * kScatterWgBytes;
    int buf = 0;
    uint32_t bphase = 0;
    for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
      const int tile = item / splits;
      const int slice = item - tile * splits;
      const TileInfo ti = tile_of(tile);
      if (!ti.valid) continue;
      if (!mbar_wait_bounded(tmem_full_bar(buf), bphase, abort_flag, p.wait_hint_ns)) {
        if (lane == 0) report_timeout(p.status, kRoleEpilogue, tile, -1);
        break;
      }
      tc_fence_after_sync();
      const int row = ti.m_block * kBM + row_in_tile;
      const int col0 = ti.n_block * 256 + h * 128;
      bool row_ok = row < p.m_total;
      if (row_ok && p.layout != nullptr) {
        if (p.masked) row_ok = row_in_tile < ti.rows_valid;
        else row_ok = __ldg(p.layout + row) >= 0;
      }
      const uint32_t t0 = tmem_base + lane_addr + (uint32_t)buf * kUmmaN + (uint32_t)h * 128;
      float* out_f32 = reinterpret_cast<float*>(p.out) +
                       ((size_t)slice * p.m_total + row) * p.N + col0;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(t0 + 32 * c, v);
        tmem_wait_ld_fence(v);
        if (p.out_f32) {
          if (row < p.m_total) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (col0 + 32 * c + 4 * i < p.N)
                reinterpret_cast<float4*>(out_f32 + 32 * c)[i] =
                    row_ok ? make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                         __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]))
                           : make_float4(0.f, 0.f, 0.f, 0.f);
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t wv[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2 * j]),
                                                       __uint_as_float(v[8 * i + 2 * j + 1]));
              wv[j] = row_ok ? *reinterpret_cast<uint32_t*>(&b) : 0u;
            }
            *reinterpret_cast<uint4*>(stage + row_in_tile * kScatterRowPitch + 64 * c + 16 * i) =
                make_uint4(wv[0], wv[1], wv[2], wv[3]);
          }
        }
      }
      // all TMEM reads of this warp are done: hand the buffer back
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar(buf));
      if (!p.out_f32) {
        named_barrier_sync(2 + h, 128);
        // whole rows: 16 lanes x 16 bytes per row, two rows per warp store; the last
        // N block may cover fewer than 256 columns
        const int cols_here = min(128, p.N - col0);  // <= 0: this half lies past N
#pragma unroll 4
        for (int it = 0; it < 16; ++it) {
          const int u = it * 128 + wg_tid;
          const int r = u >> 4, part = u & 15;
          const int grow = ti.m_block * kBM + r;
          if (grow < p.m_total && part * 8 < cols_here)
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) +
                                      (size_t)grow * p.N + col0 + part * 8) =
                *reinterpret_cast<const uint4*>(stage + r * kScatterRowPitch + 16 * part);
        }
        named_barrier_sync(2 + h, 128);
      }
      buf ^= 1;
      if (buf == 0) bphase ^= 1u;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// --------------------------------------------------------------------- host --
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// [rows, K] matrix, row-major; box = 128 rows x 128 bytes, 128-byte swizzle.
// elem_bytes = 1 (e4m3 as bytes) or 2 (bf16).
static int make_tile_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K,
                         int elem_bytes = 1) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_last_error_msg("cuTensorMapEncodeTiled is not available from this driver");
    return kNoDriverEntry;
  }
  const cuuint64_t dims[2] = {K, rows};
  const cuuint64_t strides[1] = {K * (uint64_t)elem_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), 128};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r =
      fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8,
         2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error_msg("cuTensorMapEncodeTiled failed");
    return kCudaError;
  }
  return kOk;
}

static int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Suspend-time hint of the kernels' mbarrier waits; MOEB_WAIT_HINT_NS overrides it
// for tuning runs (0 = plain polling).
static uint32_t gemm_wait_hint_ns() {
  static long v = -1;
  if (v < 0) {
    const char* e = getenv("MOEB_WAIT_HINT_NS");
    v = e ? atol(e) : (long)kWaitHintNs;
    if (v < 0) v = kWaitHintNs;
  }
  return (uint32_t)v;
}

// Tile-order tactic by the number of N blocks (sweep in launch_grouped_gemm).
static int default_group_m(int num_n_blocks) {
  return num_n_blocks >= 32 ? 16 : num_n_blocks >= 14 ? 8 : 1;
}

// keep_status: the status words are not cleared (a later launch of a chunked run must
// not wipe what an earlier one reported).
template <bool kSwiglu>
static int launch_grouped_gemm(const void* A, const void* B0, const void* B1, GemmParams p,
                               cudaStream_t stream, bool keep_status = false) {
  if (p.m_total == 0) return kOk;
  CUtensorMap tm_a, tm_b0, tm_b1;
  int rc;
  if ((rc = make_tile_map(&tm_a, A, (uint64_t)p.m_total, (uint64_t)p.K)) != kOk) return rc;
  if ((rc = make_tile_map(&tm_b0, B0, (uint64_t)p.G * p.N, (uint64_t)p.K)) != kOk) return rc;
  if ((rc = make_tile_map(&tm_b1, B1, (uint64_t)p.G * p.N, (uint64_t)p.K)) != kOk) return rc;
  p.wait_hint_ns = gemm_wait_hint_ns();
  p.num_m_blocks = ceil_div(p.m_total, kBM);
  p.num_n_blocks = kSwiglu ? p.N / 128 : ceil_div(p.N, 256);
  // Tactic: tile order by the number of N blocks (the reference picks block sizes
  // by waves and last-wave use, csrc/jit_kernels/heuristics/heuristics.hpp:136-281;
  // here the tile is fixed at 128 x 256 and the walk is what the shapes differ in).
  // CUDA-event sweep on B200, one launch each, gate/up | down in ms:
  //   N blocks (shape)            group_m = 1      4        8        16
  //   112 | 16 (H4096 I14336)     4.86 | 2.20  4.51|2.12  4.35|2.10  4.27|2.10
  //    16 | 28 (H7168 I2048)      0.989| 0.548 .979|.519  .972|.521  .974|.532
  //    12 | 16 (H4096 I1536)      0.834| 0.464 .841|.452  .841|.460  .839|.447
  //     6 |  8 (H2048 I768)       0.243| 0.177 .242|.177  .242|.177  .242|.177
  // MOEB_GEMM_GROUP_M overrides the choice (sweeps).
  static const int group_env = [] {
    const char* e = getenv("MOEB_GEMM_GROUP_M");
    return e ? atoi(e) : 0;
  }();
  p.group_m = group_env > 0 ? group_env : default_group_m(p.num_n_blocks);
  if (p.masked) p.group_m = 1;
  using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap,
                            const GemmParams);
  // Measured on B200 (one launch each, default workload): gate/up with the tanh
  // form of SiLU 0.842 ms against 0.852; the store warp or an earlier opening of
  // the next tile make gate/up slower (0.87 / 1.02 ms) and are not used there; down
  // projection with store warps and the early opening 0.456 ms against 0.508.
  // MOEB_GEMM_PLAIN=1 selects the forms without these options (comparison runs).
  static const bool plain = [] {
    const char* e = getenv("MOEB_GEMM_PLAIN");
    return e && e[0] == '1';
  }();
  KernelFn kernel = grouped_gemm_fp8_kernel<kSwiglu>;
  int smem_bytes = kSwiglu ? kGemmSmemBytesSwiglu : kGemmSmemBytes;
  int n_comm = 0;
  if constexpr (kSwiglu) {
    if (!plain) kernel = grouped_gemm_fp8_kernel<true, false, kOptTanh>;
    if (p.arrive_cnt != nullptr) {
      // dispatch fused into this launch: n_comm CTAs pull rows, the rest compute
      kernel = grouped_gemm_fp8_kernel<true, false, kOptTanh | kOptFused>;
      n_comm = p.n_comm;
    }
  } else {
    // bf16 output, local or to peers: rows are staged in shared memory and leave
    // the SM whole; f32 output keeps the plain epilogue
    if (p.scatter_out != nullptr || !p.out_f32) {
      kernel = plain ? grouped_gemm_fp8_kernel<false, true, 0>
                     : grouped_gemm_fp8_kernel<false, true, kOptOffload | kOptEarly>;
      smem_bytes = kGemmSmemBytesScatter;
    }
  }
  // per device and cheap, so it is simply repeated on every launch
  MOEB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     smem_bytes));
  if (p.status && !keep_status && !status_scope_open())
    MOEB_CUDA_TRY(cudaMemsetAsync(p.status, 0, 4 * sizeof(int32_t), stream));
  const long long tiles = (long long)p.num_m_blocks * p.num_n_blocks;
  // every CTA must be resident at once in the fused form (compute CTAs wait for
  // comm CTAs): one CTA per SM, never more CTAs than SMs
  int compute_sms = sm_count() - n_comm;
  if (p.max_ctas > 0 && p.max_ctas < compute_sms) compute_sms = p.max_ctas;
  const int grid = (int)(tiles < compute_sms ? tiles : compute_sms) + n_comm;
  kernel<<<grid, kGemmThreads, smem_bytes, stream>>>(tm_a, tm_b0, tm_b1, p);
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}

static int check_common(const char* who, const void* A, const float* scale_a, const void* B,
                        const float* scale_b, const void* out, int m_total, int N, int K, int G,
                        int gemm_type, const int32_t* layout, int max_m) {
  char msg[256];
  const char* why = nullptr;
  if (!A || !scale_a || !B || !scale_b || !out || !layout) why = "null pointer";
  else if (m_total < 0 || N <= 0 || K <= 0 || G <= 0) why = "non-positive dimension";
  else if (K % 128 != 0 || N % 128 != 0) why = "N and K must be multiples of 128";
  else if (!aligned16(A) || !aligned16(B) || !aligned16(out)) why = "A, weights and output must be 16-byte aligned";
  else if (gemm_type != MOEB_GEMM_M_GROUPED_CONTIGUOUS && gemm_type != MOEB_GEMM_M_GROUPED_MASKED)
    why = "only MGroupedContiguous and MGroupedMasked are supported";
  else if (gemm_type == MOEB_GEMM_M_GROUPED_MASKED &&
           (max_m <= 0 || max_m % 128 != 0 || (long long)max_m * G != m_total))
    why = "masked layout needs max_m % 128 == 0 and m_total == G * max_m";
  else if ((long long)G * N > 0x7fffffffLL || (long long)m_total * (long long)N > (1LL << 40))
    why = "problem too large";
  if (why) {
    snprintf(msg, sizeof(msg), "%s: %s", who, why);
    set_last_error_msg(msg);
    return kInvalidArgument;
  }
  return kOk;
}

}  // namespace moeb

using namespace moeb;

extern "C" int moeb_fp8_grouped_gemm_swiglu(const void* A, const float* scale_a, const void* gate,
                                            const float* scale_gate, const void* up,
                                            const float* scale_up, void* D, float* scale_d,
                                            int m_total, int N, int K, int G, int gemm_type,
                                            const int32_t* grouped_layout, int max_m,
                                            int32_t* status_dev, void* stream) {
  return moeb_fp8_grouped_gemm_swiglu_dyn(A, scale_a, gate, scale_gate, up, scale_up, D, scale_d,
                                          m_total, nullptr, N, K, G, gemm_type, grouped_layout,
                                          max_m, status_dev, stream);
}

extern "C" int moeb_fp8_grouped_gemm_swiglu_dyn(const void* A, const float* scale_a,
                                                const void* gate, const float* scale_gate,
                                                const void* up, const float* scale_up, void* D,
                                                float* scale_d, int m_total,
                                                const int32_t* m_valid_dev, int N, int K, int G,
                                                int gemm_type, const int32_t* grouped_layout,
                                                int max_m, int32_t* status_dev, void* stream) {
  int rc = check_common("moeb_fp8_grouped_gemm_swiglu", A, scale_a, gate, scale_gate, D, m_total,
                        N, K, G, gemm_type, grouped_layout, max_m);
  if (rc != kOk) return rc;
  if (!up || !scale_up || !scale_d || !aligned16(up)) {
    set_last_error_msg("moeb_fp8_grouped_gemm_swiglu: null or unaligned up / scale_d");
    return kInvalidArgument;
  }
  GemmParams p{};
  p.scale_a = scale_a;
  p.scale_b0 = scale_gate;
  p.scale_b1 = scale_up;
  p.out = D;
  p.scale_d = scale_d;
  p.layout = grouped_layout;
  p.status = status_dev;
  p.m_total = m_total;
  p.N = N;
  p.K = K;
  p.G = G;
  p.masked = gemm_type == MOEB_GEMM_M_GROUPED_MASKED;
  p.max_m = max_m;
  p.m_valid = m_valid_dev;
  return launch_grouped_gemm<true>(A, gate, up, p, (cudaStream_t)stream);
}

// Gate/up GEMM with the dispatch fused in (used by the expert-parallel context,
// ep_ctx.cu): contiguous layout, rows in use read from *m_valid_dev.
int moeb::fp8_swiglu_fused_dispatch(const void* A, const float* scale_a, const void* gate,
                                    const float* scale_gate, const void* up,
                                    const float* scale_up, void* D, float* scale_d, int m_total,
                                    const int32_t* m_valid_dev, int N, int K, int G,
                                    const int32_t* grouped_layout, int32_t* status_dev,
                                    const PullParams& pull, const int32_t* arrive_cnt,
                                    const int32_t* arrive_need, int n_comm, cudaStream_t stream) {
  int rc = check_common("fp8_swiglu_fused_dispatch", A, scale_a, gate, scale_gate, D, m_total, N, K,
                        G, MOEB_GEMM_M_GROUPED_CONTIGUOUS, grouped_layout, 0);
  if (rc != kOk) return rc;
  if (!up || !scale_up || !scale_d || !aligned16(up) || !arrive_cnt || !arrive_need ||
      !m_valid_dev || n_comm <= 0 || n_comm >= sm_count()) {
    set_last_error_msg("fp8_swiglu_fused_dispatch: bad argument");
    return kInvalidArgument;
  }
  GemmParams p{};
  p.scale_a = scale_a;
  p.scale_b0 = scale_gate;
  p.scale_b1 = scale_up;
  p.out = D;
  p.scale_d = scale_d;
  p.layout = grouped_layout;
  p.status = status_dev;
  p.m_total = m_total;
  p.N = N;
  p.K = K;
  p.G = G;
  p.m_valid = m_valid_dev;
  p.arrive_cnt = arrive_cnt;
  p.arrive_need = arrive_need;
  p.n_comm = n_comm;
  p.pull = pull;
  p.pull.status = status_dev;
  return launch_grouped_gemm<true>(A, gate, up, p, stream);
}

// Row ranges of a chunked MLP: plan[2c] = first row, plan[2c+1] = end row of chunk c.
// The rows in use are split evenly into `chunks` ranges of whole groups of row blocks.
__global__ void mlp_chunk_plan_kernel(const int32_t* __restrict__ m_valid, int chunks,
                                      int align_rows, int32_t* __restrict__ plan) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int valid = max(m_valid[0], 0);
  const int per = round_up(max(ceil_div(valid, chunks), 1), align_rows);
  // (an empty chunk starts on the group boundary behind every row in use, so that its
  // launch finds no tile at all)
  const int valid_up = round_up(valid, align_rows);
  for (int c = 0; c < chunks; ++c) {
    plan[2 * c] = min(c * per, valid_up);
    plan[2 * c + 1] = c + 1 == chunks ? valid : min((c + 1) * per, valid);
  }
}

// Expert MLP of a rank in row chunks, for the expert-parallel layer: gate/up of chunk
// c+1 (stream `main`, all SMs but n_down_ctas) runs beside the down projection of chunk
// c (stream `aux`, n_down_ctas SMs), whose store warps send the rows home over NVLink.
// The link, which bounds the down projection when most rows are remote, is then busy
// from the end of the first gate/up chunk on instead of after the whole gate/up GEMM.
// No kernel waits on another: a chunk's down launch follows its gate/up launch through
// an event, and both kernels are the plain launches' (two launches that poll one
// another's progress must not share a GPU: nothing guarantees that both are resident). The first gate/up chunk and the last down chunk have the GPU
// to themselves. `plan` holds 2 * chunks int32 (written here); ev_chunk: one event per
// chunk. The result is that of the two plain launches, bit for bit.
int moeb::fp8_mlp_chunked(const void* A, const float* scale_a, const void* gate,
                          const float* scale_gate, const void* up, const float* scale_up, void* D,
                          float* scale_d, const void* down, const float* scale_down,
                          const uint64_t* peer_out, size_t home_off, const int32_t* row_rank,
                          const int32_t* row_pos, int m_total, const int32_t* m_valid_dev, int I,
                          int H, int G, const int32_t* grouped_layout, int32_t* plan, int chunks,
                          int n_down_ctas, int32_t* status_swiglu, int32_t* status_down,
                          cudaStream_t main, cudaStream_t aux, cudaEvent_t ev_fork,
                          cudaEvent_t ev_join, const cudaEvent_t* ev_chunk,
                          cudaEvent_t ev_gate_up_done) {
  int rc = check_common("fp8_mlp_chunked", A, scale_a, gate, scale_gate, D, m_total, I, H, G,
                        MOEB_GEMM_M_GROUPED_CONTIGUOUS, grouped_layout, 0);
  if (rc != kOk) return rc;
  if (!up || !scale_up || !scale_d || !down || !scale_down || !peer_out || !row_rank || !row_pos ||
      !plan || !m_valid_dev || !ev_chunk || chunks < 2 || chunks > 8 || n_down_ctas <= 0 ||
      n_down_ctas >= sm_count() || !aligned16(up) || !aligned16(down)) {
    set_last_error_msg("fp8_mlp_chunked: bad argument");
    return kInvalidArgument;
  }
  if (m_total == 0) return kOk;
  GemmParams g{};
  g.scale_a = scale_a;
  g.scale_b0 = scale_gate;
  g.scale_b1 = scale_up;
  g.out = D;
  g.scale_d = scale_d;
  g.layout = grouped_layout;
  g.status = status_swiglu;
  g.m_total = m_total;
  g.N = I;
  g.K = H;
  g.G = G;
  GemmParams d{};
  d.scale_a = scale_d;
  d.scale_b0 = scale_down;
  d.scale_b1 = scale_down;
  d.layout = grouped_layout;
  d.status = status_down;
  d.m_total = m_total;
  d.N = H;
  d.K = I;
  d.G = G;
  d.scatter_out = peer_out;
  d.scatter_off = home_off;
  d.scatter_rank = row_rank;
  d.scatter_pos = row_pos;
  // chunk boundaries on whole groups of row blocks of both kernels' tile orders
  static const int group_env = [] {
    const char* e = getenv("MOEB_GEMM_GROUP_M");
    return e ? atoi(e) : 0;
  }();
  const int gm_a = group_env > 0 ? group_env : default_group_m(I / 128);
  const int gm_b = group_env > 0 ? group_env : default_group_m(ceil_div(H, 256));
  const int align_rows = kBM * (gm_a > gm_b ? gm_a : gm_b);
  mlp_chunk_plan_kernel<<<1, 32, 0, main>>>(m_valid_dev, chunks, align_rows, plan);
  MOEB_CUDA_TRY(cudaGetLastError());
  MOEB_CUDA_TRY(cudaEventRecord(ev_fork, main));
  MOEB_CUDA_TRY(cudaStreamWaitEvent(aux, ev_fork, 0));
  const int all = sm_count();
  for (int c = 0; c < chunks; ++c) {
    g.m_begin = plan + 2 * c;
    g.m_valid = plan + 2 * c + 1;
    g.max_ctas = c == 0 ? 0 : all - n_down_ctas;
    if ((rc = launch_grouped_gemm<true>(A, gate, up, g, main, c > 0)) != kOk) return rc;
    MOEB_CUDA_TRY(cudaEventRecord(ev_chunk[c], main));
    MOEB_CUDA_TRY(cudaStreamWaitEvent(aux, ev_chunk[c], 0));
    d.m_begin = plan + 2 * c;
    d.m_valid = plan + 2 * c + 1;
    d.max_ctas = c + 1 == chunks ? 0 : n_down_ctas;
    if ((rc = launch_grouped_gemm<false>(D, down, down, d, aux, c > 0)) != kOk) return rc;
  }
  if (ev_gate_up_done != nullptr) MOEB_CUDA_TRY(cudaEventRecord(ev_gate_up_done, main));
  MOEB_CUDA_TRY(cudaEventRecord(ev_join, aux));
  MOEB_CUDA_TRY(cudaStreamWaitEvent(main, ev_join, 0));
  return kOk;
}

extern "C" int moeb_fp8_grouped_gemm_nt(const void* A, const float* scale_a, const void* W,
                                        const float* scale_w, void* out, int out_dtype,
                                        int m_total, int N, int K, int G, int gemm_type,
                                        const int32_t* grouped_layout, int max_m,
                                        int32_t* status_dev, void* stream) {
  return moeb_fp8_grouped_gemm_nt_dyn(A, scale_a, W, scale_w, out, out_dtype, m_total, nullptr, N,
                                      K, G, gemm_type, grouped_layout, max_m, status_dev, stream);
}

extern "C" int moeb_fp8_grouped_gemm_nt_dyn(const void* A, const float* scale_a, const void* W,
                                            const float* scale_w, void* out, int out_dtype,
                                            int m_total, const int32_t* m_valid_dev, int N, int K,
                                            int G, int gemm_type, const int32_t* grouped_layout,
                                            int max_m, int32_t* status_dev, void* stream) {
  int rc = check_common("moeb_fp8_grouped_gemm_nt", A, scale_a, W, scale_w, out, m_total, N, K, G,
                        gemm_type, grouped_layout, max_m);
  if (rc != kOk) return rc;
  if (out_dtype != MOEB_OUT_BF16 && out_dtype != MOEB_OUT_F32) {
    set_last_error_msg("moeb_fp8_grouped_gemm_nt: out_dtype must be bf16 or f32");
    return kInvalidArgument;
  }
  GemmParams p{};
  p.scale_a = scale_a;
  p.scale_b0 = scale_w;
  p.scale_b1 = scale_w;
  p.out = out;
  p.scale_d = nullptr;
  p.layout = grouped_layout;
  p.status = status_dev;
  p.m_total = m_total;
  p.N = N;
  p.K = K;
  p.G = G;
  p.masked = gemm_type == MOEB_GEMM_M_GROUPED_MASKED;
  p.max_m = max_m;
  p.out_f32 = out_dtype == MOEB_OUT_F32;
  p.m_valid = m_valid_dev;
  return launch_grouped_gemm<false>(A, W, W, p, (cudaStream_t)stream);
}

extern "C" int moeb_fp8_grouped_gemm_nt_scatter(const void* A, const float* scale_a, const void* W,
                                                const float* scale_w, const uint64_t* peer_out,
                                                const int32_t* row_rank, const int32_t* row_pos,
                                                int m_total, const int32_t* m_valid_dev, int N,
                                                int K, int G, const int32_t* grouped_layout,
                                                int32_t* status_dev, void* stream) {
  return moeb::fp8_gemm_nt_scatter_off(A, scale_a, W, scale_w, peer_out, 0, row_rank, row_pos,
                                       m_total, m_valid_dev, N, K, G, grouped_layout, status_dev,
                                       (cudaStream_t)stream);
}

int moeb::fp8_gemm_nt_scatter_off(const void* A, const float* scale_a, const void* W,
                                  const float* scale_w, const uint64_t* peer_out, size_t home_off,
                                  const int32_t* row_rank, const int32_t* row_pos, int m_total,
                                  const int32_t* m_valid_dev, int N, int K, int G,
                                  const int32_t* grouped_layout, int32_t* status_dev,
                                  cudaStream_t stream) {
  if (!peer_out || !row_rank || !row_pos) {
    set_last_error_msg("moeb_fp8_grouped_gemm_nt_scatter: null scatter argument");
    return kInvalidArgument;
  }
  // `out` is never written in scatter mode; any aligned non-null pointer passes the checks
  int rc = check_common("moeb_fp8_grouped_gemm_nt_scatter", A, scale_a, W, scale_w, A, m_total, N,
                        K, G, MOEB_GEMM_M_GROUPED_CONTIGUOUS, grouped_layout, 0);
  if (rc != kOk) return rc;
  GemmParams p{};
  p.scale_a = scale_a;
  p.scale_b0 = scale_w;
  p.scale_b1 = scale_w;
  p.out = nullptr;
  p.layout = grouped_layout;
  p.status = status_dev;
  p.m_total = m_total;
  p.N = N;
  p.K = K;
  p.G = G;
  p.m_valid = m_valid_dev;
  p.scatter_out = peer_out;
  p.scatter_off = home_off;
  p.scatter_rank = row_rank;
  p.scatter_pos = row_pos;
  return launch_grouped_gemm<false>(A, W, W, p, stream);
}

// Dense D[s] = A[:, slice s of K] * B[:, slice s of K]^T, fp32 partial sums of k_splits K
// slices at D + s * m_total * N (router.cu sums them). A [m_total, K], B [N, K] bf16.
int moeb::bf16_gemm_splitk_f32(const void* A, const void* B, float* D, int m_total, int N, int K,
                               int k_splits, int32_t* status_dev, cudaStream_t s) {
  if (!A || !B || !D || m_total <= 0 || N <= 0 || K <= 0 || K % 8 != 0 || N % 4 != 0 ||
      !aligned16(A) || !aligned16(B) || !aligned16(D) || k_splits < 1) {
    set_last_error_msg("bf16_gemm_splitk_f32: bad argument");
    return kInvalidArgument;
  }
  CUtensorMap tm_a, tm_b;
  int rc;
  if ((rc = make_tile_map(&tm_a, A, (uint64_t)m_total, (uint64_t)K, 2)) != kOk) return rc;
  if ((rc = make_tile_map(&tm_b, B, (uint64_t)N, (uint64_t)K, 2)) != kOk) return rc;
  GemmParams p{};
  p.out = D;
  p.status = status_dev;
  p.m_total = m_total;
  p.N = N;
  p.K = K;
  p.G = 1;
  p.out_f32 = 1;
  p.wait_hint_ns = gemm_wait_hint_ns();
  p.num_m_blocks = ceil_div(m_total, kBM);
  p.num_n_blocks = ceil_div(N, 256);
  const int num_kb = ceil_div(K, kB16K);
  p.k_splits = bf16_splitk_slices(K, k_splits);
  p.kb_per_split = ceil_div(num_kb, k_splits < num_kb ? k_splits : num_kb);
  MOEB_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_bf16_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kGemmSmemBytesB16));
  if (status_dev && !status_scope_open())
    MOEB_CUDA_TRY(cudaMemsetAsync(status_dev, 0, 4 * sizeof(int32_t), s));
  const long long items = (long long)p.num_m_blocks * p.num_n_blocks * p.k_splits;
  const int grid = (int)(items < sm_count() ? items : sm_count());
  grouped_gemm_bf16_kernel<<<grid, kGemmThreads, kGemmSmemBytesB16, s>>>(tm_a, tm_b, p);
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}

// Slices a split into `want` parts really has: every slice holds at least one 64-element
// K block.
int moeb::bf16_splitk_slices(int K, int want) {
  const int num_kb = ceil_div(K, kB16K);
  if (want < 1) want = 1;
  if (want > num_kb) want = num_kb;
  return ceil_div(num_kb, ceil_div(num_kb, want));
}

extern "C" int moeb_bf16_gemm(const void* A, const void* B, void* D, int out_dtype, int m_total,
                              int N, int K, int G, int gemm_type, const int32_t* grouped_layout,
                              int max_m, int32_t* status_dev, void* stream) {
  using namespace moeb;
  const bool grouped =
      gemm_type == MOEB_GEMM_M_GROUPED_CONTIGUOUS || gemm_type == MOEB_GEMM_M_GROUPED_MASKED;
  const char* why = nullptr;
  if (!A || !B || !D) why = "null pointer";
  else if (m_total < 0 || N <= 0 || K <= 0 || G <= 0) why = "non-positive dimension";
  else if (K % 8 != 0 || N % 8 != 0) why = "N and K must be multiples of 8";
  else if (!aligned16(A) || !aligned16(B) || !aligned16(D)) why = "A, B and D must be 16-byte aligned";
  else if (gemm_type != MOEB_GEMM_NORMAL && !grouped) why = "GemmType Batched is not built";
  else if (gemm_type == MOEB_GEMM_NORMAL && G != 1) why = "a dense GEMM has one group";
  else if (grouped && !grouped_layout) why = "grouped GEMM needs grouped_layout";
  else if (grouped && G > 1 && N % 128 != 0) why = "grouped GEMM needs N % 128 == 0";
  else if (gemm_type == MOEB_GEMM_M_GROUPED_MASKED &&
           (max_m <= 0 || max_m % 128 != 0 || (long long)max_m * G != m_total))
    why = "masked layout needs max_m % 128 == 0 and m_total == G * max_m";
  else if (out_dtype != MOEB_OUT_BF16 && out_dtype != MOEB_OUT_F32) why = "out_dtype must be bf16 or f32";
  else if ((long long)G * N > 0x7fffffffLL) why = "G * N too large";
  if (why) {
    char msg[200];
    snprintf(msg, sizeof(msg), "moeb_bf16_gemm: %s", why);
    set_last_error_msg(msg);
    return kInvalidArgument;
  }
  if (m_total == 0) return kOk;
  CUtensorMap tm_a, tm_b;
  int rc;
  if ((rc = make_tile_map(&tm_a, A, (uint64_t)m_total, (uint64_t)K, 2)) != kOk) return rc;
  if ((rc = make_tile_map(&tm_b, B, (uint64_t)G * N, (uint64_t)K, 2)) != kOk) return rc;
  GemmParams p{};
  p.out = D;
  p.layout = grouped ? grouped_layout : nullptr;
  p.status = status_dev;
  p.m_total = m_total;
  p.N = N;
  p.K = K;
  p.G = G;
  p.masked = gemm_type == MOEB_GEMM_M_GROUPED_MASKED;
  p.max_m = max_m;
  p.out_f32 = out_dtype == MOEB_OUT_F32;
  p.wait_hint_ns = gemm_wait_hint_ns();
  p.num_m_blocks = ceil_div(m_total, kBM);
  p.num_n_blocks = ceil_div(N, 256);
  cudaStream_t s = (cudaStream_t)stream;
  MOEB_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_bf16_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kGemmSmemBytesB16));
  if (status_dev && !status_scope_open())
    MOEB_CUDA_TRY(cudaMemsetAsync(status_dev, 0, 4 * sizeof(int32_t), s));
  const long long tiles = (long long)p.num_m_blocks * p.num_n_blocks;
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  grouped_gemm_bf16_kernel<<<grid, kGemmThreads, kGemmSmemBytesB16, s>>>(tm_a, tm_b, p);
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}
