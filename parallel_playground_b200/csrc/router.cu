// Router: logits = x * W_gate (bf16 in, fp32 accumulate), then a bit-reproducible
// scoring + top-k selection on the fp32 logits.
//
// The reference library has no router (its README lists "fuse gate matmul +
// grouped topk kernels" as future work, README.md:50); its tests fabricate the
// routing (test/test_cpp/test_all2all.cpp:132-140). The outputs here have the
// types its dispatch consumes: int32 indices [T,k], fp32 weights [T,k]
// (csrc/all2all/all2all_tk.hpp:271-279).
#include "common.cuh"
#include "det_math.h"
#include "moe_cuda_b200.h"

namespace moeb {

// ------------------------------------------------------------------ logits --
// logits[T,E] = x[T,H] * W[H,E] (+ bias). <= 0.2 % of the layer's FLOPs, so it
// must only not get in the way: the kernel streams x once from HBM (its bound)
// and takes the small weight matrix from L2. Up to 64 experts bf16 mma.sync tiles
// (m16n8k16, fp32 accumulate) keep up with the stream; beyond that the contraction
// itself becomes the limit of the mma.sync path and the logits go through the
// tcgen05 bf16 GEMM when the caller brings a workspace (further down).
//
// CTA = 8 warps = TM token tiles (16 tokens each) x KS slices of the K range;
// the slices are summed in slice order at the end (deterministic).
//  * x goes from global memory straight into mma A fragments, no shared-memory
//    staging: a thread owns 8 consecutive K elements (one 16-byte load) of rows
//    r and r+8. The K order inside a 32-element group is permuted to make that
//    possible (a dot product does not care), and the W rows are staged in the
//    same permuted order. A whole chunk of
//    kKR K elements (kKR/32 x 2 loads of 16 bytes per thread) is requested one
//    chunk ahead, which keeps ~64 KiB per SM in flight.
//  * W chunks [KS x kKR rows][EP experts] arrive through cp.async into a double
//    buffer, stored [k][e] as in global memory and read with ldmatrix.trans.
constexpr int kRtThreads = 256;
constexpr int kKR = 256;             // K elements per slice and chunk
constexpr int kRtSteps = kKR / 32;   // 32-element groups per chunk

__host__ __device__ constexpr int rt_ws(int nt8) { return 8 * nt8 + 8; }  // padded W row (bf16)
__host__ __device__ constexpr int rt_smem_bytes(int nt8, int ks) {
  const int wbuf = 2 * ks * kKR * rt_ws(nt8) * 2;        // two W buffers
  const int red = 8 * 16 * 8 * nt8 * 4;                  // partial sums of the 8 warps
  return wbuf > red ? wbuf : red;
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
               : "=r"(r[0]), "=r"(r[1])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1,
                                               uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 16-byte cp.async; src_bytes = 0 writes zeros
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src),
               "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit_group() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <int NT8, int KS>  // the CTA covers experts [e_base, e_base + 8*NT8) and 16*(8/KS) tokens
__global__ void __launch_bounds__(kRtThreads, 1)
router_logits_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wg,
                     const float* __restrict__ bias, float* __restrict__ logits, int T, int H,
                     int E) {
  constexpr int TM = 8 / KS;
  constexpr int EP = 8 * NT8;
  constexpr int WS = rt_ws(NT8);
  constexpr int kBufElems = KS * kKR * WS;
  extern __shared__ __align__(16) uint8_t rt_smem[];
  __nv_bfloat16* wsm = reinterpret_cast<__nv_bfloat16*>(rt_smem);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tm = warp % TM, ks = warp / TM;
  const int e_base = blockIdx.y * EP;
  const int t_tile = (blockIdx.x * TM + tm) * 16;
  // K range of slice ks: whole 32-element groups
  const int groups = ceil_div(H, 32);
  const int slice_len = ceil_div(groups, KS) * 32;
  const int num_chunks = ceil_div(slice_len, kKR);
  const int k_slice = ks * slice_len;
  const bool vec_w = (E % 8) == 0;  // 16-byte aligned W rows

  // rows of x this thread loads (A fragment rows g and g+8), clamped; rows past
  // T are computed and dropped
  const int q = lane & 3;
  const int ra = min(t_tile + (lane >> 2), T - 1);
  const int rb = min(t_tile + (lane >> 2) + 8, T - 1);
  const __nv_bfloat16* xa = x + (size_t)ra * H + q * 8;
  const __nv_bfloat16* xb = x + (size_t)rb * H + q * 8;

  auto load_a = [&](uint4 (&fa)[kRtSteps], uint4 (&fb)[kRtSteps], int chunk) {
    const int k0 = k_slice + chunk * kKR;
#pragma unroll
    for (int s = 0; s < kRtSteps; ++s) {
      const int k = k0 + s * 32;
      // inside the slice and inside H (H % 8 == 0, so a vector is all in or all out)
      const bool in = (chunk * kKR + s * 32 < slice_len) && (k + q * 8 < H);
      fa[s] = in ? ld_nc_v4(xa + k) : make_uint4(0, 0, 0, 0);
      fb[s] = in ? ld_nc_v4(xb + k) : make_uint4(0, 0, 0, 0);
    }
  };
  // W rows of every slice for one chunk -> buffer `buf`
  auto stage_w = [&](int chunk, int buf) {
    __nv_bfloat16* dst = wsm + buf * kBufElems;
    for (int v = threadIdx.x; v < KS * kKR * NT8; v += kRtThreads) {
      const int row = v / NT8, nv = v % NT8;       // row = slice * kKR + r
      const int sl = row / kKR, r = row % kKR;
      const int h = sl * slice_len + chunk * kKR + r;
      const int e = e_base + nv * 8;
      const bool row_in = (chunk * kKR + r < slice_len) && h < H;
      // rows are stored in the order the mma consumes them (see lm_row below):
      // physical element p = 8q + i of a 32-element group goes to position
      // 16*(i/4) + 8*((i/2)%2) + 2q + i%2, which keeps the rows one ldmatrix reads
      // consecutive (and free of bank conflicts)
      const int p = r & 31;
      const int pos = 16 * ((p >> 2) & 1) + 8 * ((p >> 1) & 1) + 2 * (p >> 3) + (p & 1);
      __nv_bfloat16* d = dst + (row - p + pos) * WS + nv * 8;
      if (vec_w) {
        const bool in = row_in && e < E;  // E % 8 == 0: the vector is all in or all out
        cp_async_16(smem_u32(d), in ? (const void*)(wg + (size_t)h * E + e) : (const void*)wg,
                    in ? 16 : 0);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          d[i] = (row_in && e + i < E) ? wg[(size_t)h * E + e + i] : __float2bfloat16(0.0f);
      }
    }
    cp_async_commit_group();
  };

  float acc[NT8][4];
#pragma unroll
  for (int i = 0; i < NT8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  // ldmatrix row addresses: matrix m = lane/8 holds k rows 0..7 (m even) or 8..15
  // (m odd) of a k16 step, in the consumption order the staging wrote
  const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8;
  const int lm_col = (lane >> 4) * 8;

  uint4 fa0[kRtSteps], fb0[kRtSteps], fa1[kRtSteps], fb1[kRtSteps];
  stage_w(0, 0);
  load_a(fa0, fb0, 0);

  auto compute = [&](const uint4 (&fa)[kRtSteps], const uint4 (&fb)[kRtSteps], int buf) {
    const uint32_t wbase = smem_u32(wsm + buf * kBufElems + (ks * kKR) * WS);
#pragma unroll
    for (int s = 0; s < kRtSteps; ++s) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint32_t a0 = half ? fa[s].z : fa[s].x, a2 = half ? fa[s].w : fa[s].y;
        const uint32_t a1 = half ? fb[s].z : fb[s].x, a3 = half ? fb[s].w : fb[s].y;
        const uint32_t row_addr = wbase + (uint32_t)((s * 32 + half * 16 + lm_row) * WS) * 2u;
        if constexpr (NT8 == 1) {
          uint32_t b[2];
          ldmatrix_x2_trans(b, row_addr);
          mma_bf16_16816(acc[0], a0, a1, a2, a3, b[0], b[1]);
        } else {
#pragma unroll
          for (int j = 0; j < NT8 / 2; ++j) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, row_addr + (uint32_t)(j * 16 + lm_col) * 2u);
            mma_bf16_16816(acc[2 * j], a0, a1, a2, a3, b[0], b[1]);
            mma_bf16_16816(acc[2 * j + 1], a0, a1, a2, a3, b[2], b[3]);
          }
        }
      }
    }
  };

  // two chunks per round so that the register buffers alternate without copies
  for (int c = 0; c < num_chunks; c += 2) {
    cp_async_wait_all();
    __syncthreads();                       // W chunk c is in buffer 0; buffer 1 is free
    if (c + 1 < num_chunks) {
      stage_w(c + 1, 1);
      load_a(fa1, fb1, c + 1);
    }
    compute(fa0, fb0, 0);
    if (c + 1 >= num_chunks) break;
    cp_async_wait_all();
    __syncthreads();                       // W chunk c+1 is in buffer 1; buffer 0 is free
    if (c + 2 < num_chunks) {
      stage_w(c + 2, 0);
      load_a(fa0, fb0, c + 2);
    }
    compute(fa1, fb1, 1);
  }
  __syncthreads();  // all warps are done with the W buffers: reuse them for the partial sums

  // partial sums -> shared memory [ks][tm][16 rows][EP], then summed in slice order
  float* red = reinterpret_cast<float*>(rt_smem);
  {
    float* mine = red + (size_t)(ks * TM + tm) * 16 * EP;
    const int r = lane >> 2, cpair = (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < NT8; ++i) {
      mine[r * EP + i * 8 + cpair] = acc[i][0];
      mine[r * EP + i * 8 + cpair + 1] = acc[i][1];
      mine[(r + 8) * EP + i * 8 + cpair] = acc[i][2];
      mine[(r + 8) * EP + i * 8 + cpair + 1] = acc[i][3];
    }
  }
  __syncthreads();
  for (int o = threadIdx.x; o < TM * 16 * EP; o += kRtThreads) {
    const int e_in = o % EP, row = (o / EP) % 16, m = o / (EP * 16);
    const int t = (blockIdx.x * TM + m) * 16 + row, e = e_base + e_in;
    if (t >= T || e >= E) continue;
    float v = red[(size_t)m * 16 * EP + row * EP + e_in];
#pragma unroll
    for (int sl = 1; sl < KS; ++sl) v += red[(size_t)(sl * TM + m) * 16 * EP + row * EP + e_in];
    logits[(size_t)t * E + e] = v + (bias != nullptr ? bias[e] : 0.0f);
  }
}

// ------------------------------------------------------- logits, many experts --
// More than 64 experts and many tokens: the kernel above would read x once per
// 64-expert block. Here a warp owns 32 tokens x 128 experts of one K slice (two
// m16 tiles that share every B fragment, 128 fp32 partial sums per thread), so a
// CTA of 8 warps = (8 / KS) token tiles x KS slices covers 128 experts and x is
// read once per 128-expert block: once from HBM and, with 256 experts, once more
// from L2 by the CTA of the other block, which runs in the same wave. x goes from
// global memory straight into the A fragments as above, one 64-element chunk per
// slice ahead (32 KiB in flight per SM); W chunks [KS x 64 rows][128 experts] are
// double-buffered in shared memory.
constexpr int kKRW = 64;              // K elements per slice and chunk
constexpr int kRtStepsW = kKRW / 32;
constexpr int kWideNT8 = 16;          // 8-expert mma tiles per warp
constexpr int kWideEP = 8 * kWideNT8; // experts per CTA

__host__ __device__ constexpr int rt_wide_smem_bytes(int ks) {
  const int wbuf = 2 * ks * kKRW * rt_ws(kWideNT8) * 2;
  const int red = 8 * 32 * kWideEP * 4;
  return wbuf > red ? wbuf : red;
}

template <int KS>
__global__ void __launch_bounds__(kRtThreads, 1)
router_logits_wide_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wg,
                          const float* __restrict__ bias, float* __restrict__ logits, int T, int H,
                          int E) {
  constexpr int TT = 8 / KS;
  constexpr int EP = kWideEP;
  constexpr int WS = rt_ws(kWideNT8);
  constexpr int kBufElems = KS * kKRW * WS;
  extern __shared__ __align__(16) uint8_t rt_smem[];
  __nv_bfloat16* wsm = reinterpret_cast<__nv_bfloat16*>(rt_smem);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tm = warp % TT, ks = warp / TT;
  const int e_base = blockIdx.y * EP;
  const int t_tile = (blockIdx.x * TT + tm) * 32;
  const int groups = ceil_div(H, 32);
  const int slice_len = ceil_div(groups, KS) * 32;
  const int num_chunks = ceil_div(slice_len, kKRW);
  const int k_slice = ks * slice_len;
  const bool vec_w = (E % 8) == 0;

  // x rows of this thread: rows g and g+8 of both m16 tiles, clamped (rows past
  // T are computed and dropped)
  const int q = lane & 3;
  const __nv_bfloat16* xr[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    xr[j] = x + (size_t)min(t_tile + (lane >> 2) + 8 * j, T - 1) * H + q * 8;

  auto load_a = [&](uint4 (&f)[kRtStepsW][4], int chunk) {
    const int k0 = k_slice + chunk * kKRW;
#pragma unroll
    for (int s = 0; s < kRtStepsW; ++s) {
      const int k = k0 + s * 32;
      const bool in = (chunk * kKRW + s * 32 < slice_len) && (k + q * 8 < H);
#pragma unroll
      for (int j = 0; j < 4; ++j) f[s][j] = in ? ld_nc_v4(xr[j] + k) : make_uint4(0, 0, 0, 0);
    }
  };
  // W rows of every slice for one chunk -> buffer `buf`, each 32-row group in the
  // order the mma consumes it (the permutation of the kernel above)
  auto stage_w = [&](int chunk, int buf) {
    __nv_bfloat16* dst = wsm + buf * kBufElems;
    for (int v = threadIdx.x; v < KS * kKRW * kWideNT8; v += kRtThreads) {
      const int row = v / kWideNT8, nv = v % kWideNT8;
      const int sl = row / kKRW, r = row % kKRW;
      const int h = sl * slice_len + chunk * kKRW + r;
      const int e = e_base + nv * 8;
      const bool row_in = (chunk * kKRW + r < slice_len) && h < H;
      const int p = r & 31;
      const int pos = 16 * ((p >> 2) & 1) + 8 * ((p >> 1) & 1) + 2 * (p >> 3) + (p & 1);
      __nv_bfloat16* d = dst + (row - p + pos) * WS + nv * 8;
      if (vec_w) {
        const bool in = row_in && e < E;
        cp_async_16(smem_u32(d), in ? (const void*)(wg + (size_t)h * E + e) : (const void*)wg,
                    in ? 16 : 0);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          d[i] = (row_in && e + i < E) ? wg[(size_t)h * E + e + i] : __float2bfloat16(0.0f);
      }
    }
    cp_async_commit_group();
  };

  float acc[2][kWideNT8][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int i = 0; i < kWideNT8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[m][i][j] = 0.0f;

  const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8;
  const int lm_col = (lane >> 4) * 8;

  uint4 f0[kRtStepsW][4], f1[kRtStepsW][4];
  stage_w(0, 0);
  load_a(f0, 0);

  auto compute = [&](const uint4 (&f)[kRtStepsW][4], int buf) {
    const uint32_t wbase = smem_u32(wsm + buf * kBufElems + (ks * kKRW) * WS);
#pragma unroll
    for (int s = 0; s < kRtStepsW; ++s) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t a[2][4];
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          const uint4 fa = f[s][2 * m], fb = f[s][2 * m + 1];
          a[m][0] = half ? fa.z : fa.x;
          a[m][2] = half ? fa.w : fa.y;
          a[m][1] = half ? fb.z : fb.x;
          a[m][3] = half ? fb.w : fb.y;
        }
        const uint32_t row_addr = wbase + (uint32_t)((s * 32 + half * 16 + lm_row) * WS) * 2u;
#pragma unroll
        for (int j = 0; j < kWideNT8 / 2; ++j) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, row_addr + (uint32_t)(j * 16 + lm_col) * 2u);
#pragma unroll
          for (int m = 0; m < 2; ++m) {
            mma_bf16_16816(acc[m][2 * j], a[m][0], a[m][1], a[m][2], a[m][3], b[0], b[1]);
            mma_bf16_16816(acc[m][2 * j + 1], a[m][0], a[m][1], a[m][2], a[m][3], b[2], b[3]);
          }
        }
      }
    }
  };

  for (int c = 0; c < num_chunks; c += 2) {
    cp_async_wait_all();
    __syncthreads();
    if (c + 1 < num_chunks) {
      stage_w(c + 1, 1);
      load_a(f1, c + 1);
    }
    compute(f0, 0);
    if (c + 1 >= num_chunks) break;
    cp_async_wait_all();
    __syncthreads();
    if (c + 2 < num_chunks) {
      stage_w(c + 2, 0);
      load_a(f0, c + 2);
    }
    compute(f1, 1);
  }
  __syncthreads();  // the W buffers become the partial sums [ks][tm][32 rows][EP]

  float* red = reinterpret_cast<float*>(rt_smem);
  {
    float* mine = red + (size_t)(ks * TT + tm) * 32 * EP;
    const int r = lane >> 2, cpair = (lane & 3) * 2;
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int i = 0; i < kWideNT8; ++i) {
        float* o = mine + (16 * m + r) * EP + i * 8 + cpair;
        o[0] = acc[m][i][0];
        o[1] = acc[m][i][1];
        o[8 * EP] = acc[m][i][2];
        o[8 * EP + 1] = acc[m][i][3];
      }
  }
  __syncthreads();
  for (int o = threadIdx.x; o < TT * 32 * EP; o += kRtThreads) {
    const int e_in = o % EP, row = (o / EP) % 32, m = o / (EP * 32);
    const int t = (blockIdx.x * TT + m) * 32 + row, e = e_base + e_in;
    if (t >= T || e >= E) continue;
    float v = red[(size_t)m * 32 * EP + row * EP + e_in];
#pragma unroll
    for (int sl = 1; sl < KS; ++sl) v += red[(size_t)(sl * TT + m) * 32 * EP + row * EP + e_in];
    logits[(size_t)t * E + e] = v + (bias != nullptr ? bias[e] : 0.0f);
  }
}

// ------------------------------------------- logits on the tcgen05 tensor cores --
// With more than 64 experts the contraction itself bounds the mma.sync kernels above
// (measured on B200, 8192 tokens x 4096 x 256 experts: 104 us, ~165 TFLOP/s, against
// 12 us for reading x once). Given a workspace the logits go through the tcgen05 bf16
// GEMM instead: W [H,E] is transposed to K-major [E,H] (a few MB), the GEMM runs with
// the K range split over enough CTAs to fill the GPU, and the slices' fp32 partial sums
// are added in slice order (+ bias) - the same result on every run.
__global__ void __launch_bounds__(256)
router_transpose_w_kernel(const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ wt,
                          int H, int E) {
  __shared__ __nv_bfloat16 tile[32][33];
  const int h0 = blockIdx.x * 32, e0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int h = h0 + ty + 8 * i, e = e0 + tx;
    tile[ty + 8 * i][tx] = (h < H && e < E) ? w[(size_t)h * E + e] : __float2bfloat16(0.0f);
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int e = e0 + ty + 8 * i, h = h0 + tx;
    if (e < E && h < H) wt[(size_t)e * H + h] = tile[tx][ty + 8 * i];
  }
}

__global__ void __launch_bounds__(256)
router_sum_slices_kernel(const float* __restrict__ partial, const float* __restrict__ bias,
                         float* __restrict__ logits, size_t n, int E, int slices) {
  // n = T * E, a multiple of 4 (E % 8 == 0)
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n;
       i += (size_t)gridDim.x * blockDim.x * 4) {
    float4 v = *reinterpret_cast<const float4*>(partial + i);
    for (int s = 1; s < slices; ++s) {
      const float4 o = *reinterpret_cast<const float4*>(partial + (size_t)s * n + i);
      v.x += o.x;
      v.y += o.y;
      v.z += o.z;
      v.w += o.w;
    }
    if (bias != nullptr) {
      const int e = (int)(i % (size_t)E);
      v.x += bias[e];
      v.y += bias[e + 1];
      v.z += bias[e + 2];
      v.w += bias[e + 3];
    }
    *reinterpret_cast<float4*>(logits + i) = v;
  }
}

// K slices of the tensor-core path, 0 = the path does not apply to this shape.
static int tc_router_slices(int T, int H, int E) {
  if (E <= 64 || E % 8 != 0 || T < 1024) return 0;
  const long long tiles = (long long)ceil_div(T, 128) * ceil_div(E, 256);
  int want = (int)(148 / tiles);
  if (want < 1) want = 1;
  if (want > 8) want = 8;
  // at least 8 K blocks of 64 per slice
  while (want > 1 && ceil_div(H, 64) / want < 8) --want;
  return bf16_splitk_slices(H, want);
}
static size_t tc_router_wt_bytes(int H, int E) {
  return ((size_t)E * H * 2 + 255) / 256 * 256;
}

// ------------------------------------------------------------------ select --
// One warp per token; the token's scores live in shared memory. All arithmetic
// that decides an index or a weight goes through det_math.h so that the CPU
// oracle reproduces it bit for bit.
constexpr int kSelWarps = 4;
constexpr int kMaxExperts = 1024;
constexpr int kMaxTopK = 32;

struct ArgBest {
  float v;
  int i;
};
// a is better than b: larger value, ties to the lower index; i < 0 marks "none".
__device__ __forceinline__ bool better(float av, int ai, float bv, int bi) {
  if (bi < 0) return ai >= 0;
  if (ai < 0) return false;
  return (av > bv) || (av == bv && ai < bi);
}
__device__ __forceinline__ ArgBest warp_argbest(float v, int i) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, off);
    const int oi = __shfl_xor_sync(0xffffffffu, i, off);
    if (better(ov, oi, v, i)) {
      v = ov;
      i = oi;
    }
  }
  return {v, i};
}

__global__ void __launch_bounds__(kSelWarps * 32)
router_select_kernel(const float* __restrict__ logits, int T, int E, int k, int mode, int n_group,
                     int topk_group, int renorm, float route_scale, int32_t* __restrict__ indices,
                     float* __restrict__ weights) {
  extern __shared__ float sel_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kSelWarps + warp;
  float* score = sel_smem + (size_t)warp * (2 * E + 64);  // selection key per expert
  float* prob = score + E;                                // weight numerator per expert
  float* gscore = prob + E;                               // per-group score (<= 32)
  int* gkeep = reinterpret_cast<int*>(gscore + 32);
  if (t >= T) return;  // whole warp leaves together
  const float* lrow = logits + (size_t)t * E;

  float denom_all = 0.0f;
  if (mode == MOEB_ROUTER_SOFTMAX) {
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, lrow[e]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    float part = 0.0f;
    for (int e = lane; e < E; e += 32) {
      const float l = lrow[e];
      const float p = moeb_det_expf(moeb_add(l, -m));
      score[e] = l;  // selection on the logit itself (monotone in p, no exp ties)
      prob[e] = p;
      part = moeb_add(part, p);
    }
    // butterfly sum: every lane ends with the same bits (a+b == b+a)
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
      part = moeb_add(part, __shfl_xor_sync(0xffffffffu, part, off));
    denom_all = part;
  } else {
    for (int e = lane; e < E; e += 32) {
      const float s = moeb_det_sigmoidf(lrow[e]);
      score[e] = s;
      prob[e] = s;
    }
  }
  __syncwarp();

  if (mode == MOEB_ROUTER_SIGMOID_GROUPED && n_group > 1) {
    const int gsize = E / n_group;
    if (lane < n_group) {
      float b1 = -INFINITY, b2 = -INFINITY;  // two largest scores of the group
      for (int j = 0; j < gsize; ++j) {
        const float s = score[lane * gsize + j];
        if (s > b1) {
          b2 = b1;
          b1 = s;
        } else if (s > b2) {
          b2 = s;
        }
      }
      gscore[lane] = gsize > 1 ? moeb_add(b1, b2) : b1;
      gkeep[lane] = 0;
    }
    __syncwarp();
    for (int r = 0; r < topk_group; ++r) {
      float v = 0.0f;
      int i = -1;
      if (lane < n_group && gkeep[lane] == 0) {
        v = gscore[lane];
        i = lane;
      }
      const ArgBest b = warp_argbest(v, i);
      if (lane == 0 && b.i >= 0) gkeep[b.i] = 1;
      __syncwarp();
    }
    // experts of dropped groups can no longer be selected
    for (int e = lane; e < E; e += 32)
      if (gkeep[e / gsize] == 0) score[e] = -INFINITY;
    __syncwarp();
  }

  // top-k by (score desc, index asc); -inf entries of dropped groups lose to any kept one
  float sel_p = 0.0f;  // lane j holds the numerator of pick j
  int sel_i = -1;
  for (int j = 0; j < k; ++j) {
    float v = 0.0f;
    int i = -1;
    for (int e = lane; e < E; e += 32) {
      const float s = score[e];
      if (s != s) continue;                 // NaN logits are never selected
      if (__float_as_uint(prob[e]) == 0xffffffffu) continue;  // already taken
      if (better(s, e, v, i)) {
        v = s;
        i = e;
      }
    }
    const ArgBest b = warp_argbest(v, i);
    if (lane == j) {
      sel_i = b.i;
      sel_p = b.i >= 0 ? prob[b.i] : 0.0f;
    }
    __syncwarp();
    if (lane == 0 && b.i >= 0) prob[b.i] = __uint_as_float(0xffffffffu);  // mark as taken
    __syncwarp();
  }

  // denominator: sequential sum over the picks in pick order (lane 0 .. k-1)
  float denom = 0.0f;
  for (int j = 0; j < k; ++j) denom = moeb_add(denom, __shfl_sync(0xffffffffu, sel_p, j));
  if (mode == MOEB_ROUTER_SOFTMAX && !renorm) denom = denom_all;
  if (lane < k) {
    float w = moeb_div(sel_p, denom);
    w = moeb_mul(w, route_scale);
    indices[(size_t)t * k + lane] = sel_i;
    weights[(size_t)t * k + lane] = w;
  }
}

template <int NT8, int KS>
static cudaError_t launch_logits(const void* x, const void* wg, const float* bias, float* logits,
                                 int T, int H, int E, cudaStream_t s) {
  constexpr int TM = 8 / KS;
  constexpr int smem = rt_smem_bytes(NT8, KS);
  auto kernel = router_logits_kernel<NT8, KS>;
  cudaError_t err =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (err != cudaSuccess) return err;
  const dim3 grid(ceil_div(T, 16 * TM), ceil_div(E, 8 * NT8));
  kernel<<<grid, kRtThreads, smem, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)wg, bias,
                                        logits, T, H, E);
  return cudaGetLastError();
}

template <int KS>
static cudaError_t launch_logits_wide(const void* x, const void* wg, const float* bias,
                                      float* logits, int T, int H, int E, cudaStream_t s) {
  constexpr int smem = rt_wide_smem_bytes(KS);
  auto kernel = router_logits_wide_kernel<KS>;
  cudaError_t err =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (err != cudaSuccess) return err;
  const dim3 grid(ceil_div(T, 32 * (8 / KS)), ceil_div(E, kWideEP));
  kernel<<<grid, kRtThreads, smem, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)wg, bias,
                                        logits, T, H, E);
  return cudaGetLastError();
}

// K slices of the many-expert kernel, 0 = use the kernel with 64-expert blocks:
// the most tokens per CTA (fewest passes over W) that still fills most of the SMs.
static int pick_wide_slices(int T, int E) {
  if (E <= 64) return 0;
  const long long blocks = ceil_div(E, kWideEP);
  if ((long long)ceil_div(T, 128) * blocks >= 96) return 2;
  if ((long long)ceil_div(T, 64) * blocks >= 96) return 4;
  return 0;
}

// Tile shape. Many tokens: 64 tokens x 2 K slices per CTA with up to 64 experts,
// so that x is read once (or once per 64-expert block, from L2). Few tokens
// (decode): 16 tokens x 8 K slices per CTA and expert blocks narrow enough to
// give the GPU a full wave of CTAs (x is small then; W is what gets streamed).
struct RouterTile {
  int nt8, ks;
};
static RouterTile pick_router_tile(int T, int E) {
  int nt8_max = 1;
  while (nt8_max < 8 && 8 * nt8_max < E) nt8_max *= 2;
  if ((long long)ceil_div(T, 64) * ceil_div(E, 8 * nt8_max) >= 96) return {nt8_max, 2};
  // (the 8-slice form keeps its W buffers within shared memory up to 16 experts)
  for (int nt8 = nt8_max < 2 ? nt8_max : 2; nt8 >= 1; nt8 /= 2)
    if ((long long)ceil_div(T, 16) * ceil_div(E, 8 * nt8) >= 148 || nt8 == 1) return {nt8, 8};
  return {1, 8};
}

}  // namespace moeb

extern "C" int moeb_router_logits(const void* x_bf16, const void* w_gate_bf16,
                                  const float* logit_bias, float* logits, int T, int H, int E,
                                  void* stream) {
  using namespace moeb;
  // (with T == 0 the per-token arrays are empty and may be null)
  if ((T > 0 && (!x_bf16 || !logits)) || !w_gate_bf16 || T < 0 || H <= 0 || E <= 0 || H % 8 != 0) {
    set_last_error_msg("moeb_router_logits: bad argument (H must be a multiple of 8)");
    return kInvalidArgument;
  }
  if (T == 0) return kOk;
  cudaStream_t s = (cudaStream_t)stream;
  const RouterTile tile = pick_router_tile(T, E);
  const int wide = pick_wide_slices(T, E);
  cudaError_t err = cudaSuccess;
  if (wide == 2) {
    err = launch_logits_wide<2>(x_bf16, w_gate_bf16, logit_bias, logits, T, H, E, s);
  } else if (wide == 4) {
    err = launch_logits_wide<4>(x_bf16, w_gate_bf16, logit_bias, logits, T, H, E, s);
  } else if (tile.ks == 2) {
    switch (tile.nt8) {
      case 8: err = launch_logits<8, 2>(x_bf16, w_gate_bf16, logit_bias, logits, T, H, E, s); break;
      case 4: err = launch_logits<4, 2>(x_bf16, w_gate_bf16, logit_bias, logits, T, H, E, s); break;
      case 2: err = launch_logits<2, 2>(x_bf16, w_gate_bf16, logit_bias, logits, T, H, E, s); break;
      default: err = launch_logits<1, 2>(x_bf16, w_gate_bf16, logit_bias, logits, T, H, E, s); break;
    }
  } else {
    if (tile.nt8 == 2) err = launch_logits<2, 8>(x_bf16, w_gate_bf16, logit_bias, logits, T, H, E, s);
    else err = launch_logits<1, 8>(x_bf16, w_gate_bf16, logit_bias, logits, T, H, E, s);
  }
  MOEB_CUDA_TRY(err);
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}

extern "C" size_t moeb_router_logits_workspace_bytes(int T, int H, int E) {
  using namespace moeb;
  if (T <= 0 || H <= 0 || E <= 0 || H % 8 != 0) return 0;
  if (tc_router_slices(T, H, E) == 0) return 0;
  // slices * T <= max(T, 148 * 128) (a split never makes more items than SMs), so this
  // size also serves every smaller token count: a workspace sized for the most tokens
  // a caller will ever pass is enough for all its calls
  const size_t rows = T > 148 * 128 ? (size_t)T : (size_t)148 * 128;
  return tc_router_wt_bytes(H, E) + rows * E * 4;
}

extern "C" int moeb_router_logits_ws(const void* x_bf16, const void* w_gate_bf16,
                                     const float* logit_bias, float* logits, int T, int H, int E,
                                     void* workspace, size_t workspace_bytes, int32_t* status_dev,
                                     void* stream) {
  using namespace moeb;
  const size_t need = moeb_router_logits_workspace_bytes(T, H, E);
  if (need == 0 || !workspace || workspace_bytes < need ||
      (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return moeb_router_logits(x_bf16, w_gate_bf16, logit_bias, logits, T, H, E, stream);
  if (!x_bf16 || !w_gate_bf16 || !logits ||
      ((reinterpret_cast<uintptr_t>(x_bf16) | reinterpret_cast<uintptr_t>(logits)) & 15u) != 0) {
    set_last_error_msg("moeb_router_logits_ws: null or unaligned pointer (x, logits: 16 bytes)");
    return kInvalidArgument;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const int slices = tc_router_slices(T, H, E);
  __nv_bfloat16* wt = static_cast<__nv_bfloat16*>(workspace);
  float* partial = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + tc_router_wt_bytes(H, E));
  router_transpose_w_kernel<<<dim3(ceil_div(H, 32), ceil_div(E, 32)), 256, 0, s>>>(
      (const __nv_bfloat16*)w_gate_bf16, wt, H, E);
  MOEB_CUDA_TRY(cudaGetLastError());
  const bool direct = slices == 1 && logit_bias == nullptr;
  int rc = bf16_gemm_splitk_f32(x_bf16, wt, direct ? logits : partial, T, E, H, slices, status_dev, s);
  if (rc != kOk) return rc;
  if (!direct) {
    const size_t n = (size_t)T * E;
    const int blocks = (int)((n / 4 + 255) / 256 < 148 * 8 ? (n / 4 + 255) / 256 : 148 * 8);
    router_sum_slices_kernel<<<blocks, 256, 0, s>>>(partial, logit_bias, logits, n, E, slices);
    MOEB_CUDA_TRY(cudaGetLastError());
  }
  return kOk;
}

extern "C" int moeb_router_select(const float* logits, int T, int E, int k, int mode, int n_group,
                                  int topk_group, int renorm, float route_scale, int32_t* indices,
                                  float* weights, void* stream) {
  using namespace moeb;
  if ((T > 0 && (!logits || !indices || !weights)) || T < 0 || E <= 0 || k <= 0 || k > E ||
      k > kMaxTopK || E > kMaxExperts) {
    set_last_error_msg("moeb_router_select: bad argument (need 0 < k <= min(E,32), E <= 1024)");
    return kInvalidArgument;
  }
  if (mode != MOEB_ROUTER_SOFTMAX && mode != MOEB_ROUTER_SIGMOID_GROUPED) {
    set_last_error_msg("moeb_router_select: unknown router mode");
    return kInvalidArgument;
  }
  if (mode == MOEB_ROUTER_SIGMOID_GROUPED) {
    if (n_group < 1 || n_group > 32 || E % n_group != 0 || topk_group < 1 ||
        topk_group > n_group || (long long)topk_group * (E / n_group) < k) {
      set_last_error_msg("moeb_router_select: bad group configuration");
      return kInvalidArgument;
    }
  }
  if (T == 0) return kOk;
  const size_t smem = (size_t)kSelWarps * (2 * E + 64) * sizeof(float);
  router_select_kernel<<<ceil_div(T, kSelWarps), kSelWarps * 32, smem, (cudaStream_t)stream>>>(
      logits, T, E, k, mode, n_group, topk_group, renorm, route_scale, indices, weights);
  MOEB_CUDA_TRY(cudaGetLastError());
  return kOk;
}
