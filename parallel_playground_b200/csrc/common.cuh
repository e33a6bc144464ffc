// Shared device/host helpers for the sm_100a MoE kernels: status codes, bounded
// mbarrier waits, TMA / tcgen05 PTX wrappers, small vector utilities.
//
// Every device-side wait in this library is bounded: it polls for a limited
// wall-clock time, then records a status code in global memory and lets the
// kernel run to its normal teardown, so a logic error shows up as an error
// code on the host instead of a hung GPU.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace moeb {

// Status codes returned by every C-ABI entry point (0 = success).
enum Status : int {
  kOk = 0,
  kInvalidArgument = 1,
  kCudaError = 2,
  kNotImplemented = 3,
  kDeviceTimeout = 4,   // a bounded device-side wait expired
  kUnsupportedShape = 5,
  kNoDriverEntry = 6,   // cuTensorMapEncodeTiled could not be resolved
  kTooLarge = 7,
};

// Device status word layout (int32[4], zeroed by the host before a launch):
//   [0] status code (first writer wins), [1] role id that gave up,
//   [2] tile index, [3] k-block index.
struct DeviceStatus {
  int code;
  int role;
  int tile;
  int kblock;
};

#define MOEB_CUDA_TRY(expr)                                  \
  do {                                                       \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) {                                 \
      moeb::set_last_error(#expr, _e);                       \
      return moeb::kCudaError;                               \
    }                                                        \
  } while (0)

void set_last_error(const char* what, cudaError_t e);
void set_last_error_msg(const char* msg);

// Device status words (first report wins, see report_timeout). A kernel launcher called on
// its own clears its four words before the launch. A call that strings several launches
// together (a whole layer, a dispatch + GEMM) opens a StatusScope instead: the outermost
// scope clears all the caller's words once, and no launcher inside it clears anything, so
// that a report of an early launch (a rank barrier that ran out, the router's GEMM) is not
// wiped by a later one that shares its words.
extern thread_local int tl_status_scopes;
inline bool status_scope_open() { return tl_status_scopes > 0; }
struct StatusScope {
  StatusScope(int32_t* status, int words, cudaStream_t s) {
    if (tl_status_scopes == 0 && status != nullptr) cudaMemsetAsync(status, 0, sizeof(int32_t) * words, s);
    ++tl_status_scopes;
  }
  ~StatusScope() { --tl_status_scopes; }
  StatusScope(const StatusScope&) = delete;
  StatusScope& operator=(const StatusScope&) = delete;
};

// grouped_gemm.cu: dense bf16 GEMM (tcgen05) with the K range split into slices, fp32
// partial sums per slice at D + s * m_total * N; bf16_splitk_slices: the slices a request
// for `want` really gets (every slice holds at least one 64-element K block).
int bf16_gemm_splitk_f32(const void* A, const void* B, float* D, int m_total, int N, int K,
                         int k_splits, int32_t* status_dev, cudaStream_t s);
int bf16_splitk_slices(int K, int want);

constexpr int kQuantBlock = 128;       // activation scale granularity (1 x 128)
constexpr float kFp8Max = 448.0f;      // e4m3fn finite maximum

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ inline int round_up(int a, int b) { return ceil_div(a, b) * b; }

#if defined(__CUDACC__)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---------------------------------------------------------------- mbarrier --
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// try_wait with a suspend-time hint: the hardware parks the warp until the
// phase completes or `hint_ns` elapse, so a waiting warp does not burn issue
// slots of its scheduler (a hot polling loop in the producer / MMA warps slows
// down the promotion warps that share their schedulers).
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity,
                                                   uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}

// Wait on an mbarrier phase for at most `limit_ns`. `abort_flag` is a shared
// memory word that any role of the CTA sets when it gives up; the others then
// stop waiting as well. Returns false if the wait was abandoned.
constexpr uint64_t kWaitLimitNs = 400ull * 1000 * 1000;  // 0.4 s per wait
constexpr uint32_t kWaitHintNs = 1000 * 1000;            // park up to 1 ms per try
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  volatile int* abort_flag,
                                                  uint32_t hint_ns = kWaitHintNs) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (hint_ns != 0) {
      if (mbar_try_wait_hint(bar, parity, hint_ns)) return true;
    } else {
      // plain polling: look at the clock only every 64 tries
      if (mbar_try_wait(bar, parity)) return true;
      if ((++spins & 63u) != 0u) continue;
    }
    if (*abort_flag != 0) return false;
    if (global_timer_ns() - t0 > kWaitLimitNs) {
      *abort_flag = 1;
      return false;
    }
  }
}

__device__ __forceinline__ void report_timeout(int* status, int role, int tile, int kb) {
  if (status != nullptr && atomicCAS(&status[0], 0, (int)kDeviceTimeout) == 0) {
    status[1] = role;
    status[2] = tile;
    status[3] = kb;
  }
}

// --------------------------------------------------------------------- TMA --
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load, global -> this CTA's shared memory, completion on an mbarrier.
// x (innermost coordinate) times the element size must be a multiple of 16 B.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ----------------------------------------------------------------- tcgen05 --
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result_addr, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_result_addr),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier once every previously issued tcgen05.mma of this thread
// has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]^T, FP8 (e4m3/e5m2...) operands, FP32
// accumulate, one CTA. `accumulate == 0` overwrites D.
__device__ __forceinline__ void tc_mma_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of
// 128 bytes with the 128-byte swizzle (what a TMA load with
// CU_TENSOR_MAP_SWIZZLE_128B writes): 8-row groups are 1024 B apart.
__device__ __forceinline__ uint64_t make_sw128_kmajor_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                        // descriptor version for sm_100
  d |= (uint64_t)2 << 61;                        // layout type: SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f8f6f4: e4m3 x e4m3 -> f32, both operands
// K-major, tile M x N.
__host__ __device__ constexpr uint32_t make_idesc_e4m3_f32(int m, int n) {
  return (1u << 4)                       // D format f32
         | (0u << 7) | (0u << 10)        // A, B format e4m3
         | ((uint32_t)(n >> 3) << 17)    // N / 8
         | ((uint32_t)(m >> 4) << 24);   // M / 16
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives the
// 32 columns of TMEM lane (lane_base + i).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ------------------------------------------------------------- conversions --
__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}
// Two floats -> two e4m3 bytes (round to nearest even, saturate to +-448).
// Byte 0 of the result holds `lo`.
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi) {
  return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ uint32_t f32x4_to_e4m3x4(float a, float b, float c, float d) {
  return f32x2_to_e4m3x2(a, b) | (f32x2_to_e4m3x2(c, d) << 16);
}
// amax/448 with the zero-block guard of the reference cast kernel.
__device__ __forceinline__ float quant_scale_from_amax(float amax) {
  return amax > 0.0f ? __fdiv_rn(amax, kFp8Max) : 1.0f;
}
__device__ __forceinline__ float quant_value(float x, float scale) {
  return fmaxf(-kFp8Max, fminf(kFp8Max, __fdiv_rn(x, scale)));
}

__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

#endif  // __CUDACC__

}  // namespace moeb
