// Shared device helpers for the sm_100a kernels: PTX wrappers (mbarrier, bulk copies, tcgen05/TMEM, acquire/release
// flags), bounded waits that record an error status instead of spinning forever, warp reductions.
//
// Every device-side wait in this tree goes through a *_bounded helper: it gives up after a fixed number of polls,
// writes a code into the launch's status word and lets the kernel drain and return, so a lost signal can never hang
// the GPU. (The upstream kernels poll without a limit: pear/models/qwen3_5/rollout/blackwell/csrc/ar_norm.cu:155-165,
// deploy/blackwell/nvfp4/csrc/megakernel.cu:1169.)
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define PEAR_API extern "C" __attribute__((visibility("default")))

// status codes written to the per-launch status word (0 = ok)
enum PearStatus : int {
  PEAR_OK = 0,
  PEAR_ERR_MBAR_TIMEOUT = 1,     // an mbarrier phase did not complete within the poll budget
  PEAR_ERR_GRID_BARRIER = 2,     // a grid-wide barrier was not reached by every CTA within the poll budget
  PEAR_ERR_FLAG_TIMEOUT = 3,     // a peer/flag word never took the awaited value
  PEAR_ERR_BAD_INSTR = 4,        // the instruction interpreter met an unknown opcode
  PEAR_ERR_TMEM = 5,             // tensor-memory allocation did not return
  PEAR_ERR_SMEM_ALIGN = 6,       // the dynamic shared memory base was not aligned as the kernel's layout needs
};

#define PEAR_CUDA_CHECK(expr)                                                                  \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess) return (int)_e;                                                     \
  } while (0)

#define PEAR_LAUNCH_CHECK()                                                                    \
  do {                                                                                         \
    cudaError_t _e = cudaGetLastError();                                                       \
    if (_e != cudaSuccess) return (int)_e;                                                     \
  } while (0)

namespace pear {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint32_t lane_id() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(r));
  return r;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------------------------------------ warp reductions
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// block reduce through shared scratch of >= 32 floats; every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) scratch[w] = v;
  __syncthreads();
  float r = (l < nw) ? scratch[l] : 0.f;
  r = warp_sum(r);
  return r;
}

// ------------------------------------------------------------------------------------------------ status word
__device__ __forceinline__ void set_status(int* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

// ------------------------------------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Poll budget: try_wait itself blocks for a hardware-defined slice, so 1<<22 polls is several seconds at most.
constexpr uint32_t kMbarPolls = 1u << 22;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int* status) {
  for (uint32_t i = 0; i < kMbarPolls; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (status && (i & 1023u) == 1023u && *(volatile int*)status != 0) return false;  // someone else gave up
  }
  set_status(status, PEAR_ERR_MBAR_TIMEOUT);
  return false;
}

// Non-suspending variant for the single threads on a pipeline's critical path (weight producer, MMA issuer): test_wait
// returns at once, so the thread reacts to a completed phase within a few cycles instead of after try_wait's
// suspension slice.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_spin_bounded(uint64_t* bar, uint32_t parity, int* status) {
  for (uint32_t i = 0; i < (1u << 26); ++i) {
    if (mbar_test_wait(bar, parity)) return true;
    if (status && (i & 65535u) == 65535u && *(volatile int*)status != 0) return false;  // someone else gave up
  }
  set_status(status, PEAR_ERR_MBAR_TIMEOUT);
  return false;
}

// Same wait with a sleep between polls: for threads whose wake-up latency does not matter but whose polling would
// compete with the tensor core's and the copy engine's own shared-memory traffic.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, int* status, unsigned ns = 100) {
  for (uint32_t i = 0; i < kMbarPolls; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(ns);
    if (status && (i & 1023u) == 1023u && *(volatile int*)status != 0) return false;
  }
  set_status(status, PEAR_ERR_MBAR_TIMEOUT);
  return false;
}

// ------------------------------------------------------------------------------------------------ bulk copies (TMA)
// 1-D bulk copy global -> shared, completion counted on an mbarrier. Both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// 2-D tiled TMA load (no multicast). x is the innermost coordinate: x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tensor_map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(smem_dst)),
      "l"(tensor_map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const void* tensor_map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tensor_map) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ------------------------------------------------------------------------------------------------ acquire / release
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_f32(float* p, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}

// Wait until *flag >= target (system scope), at most `polls` polls. Returns false (and records) on expiry.
__device__ __forceinline__ bool wait_flag_ge_sys_bounded(const uint32_t* flag, uint32_t target, uint32_t polls, int* status) {
  for (uint32_t i = 0; i < polls; ++i) {
    if ((int32_t)(ld_acquire_sys(flag) - target) >= 0) return true;
    if (i > 64) __nanosleep(64);
  }
  set_status(status, PEAR_ERR_FLAG_TIMEOUT);
  return false;
}

// ------------------------------------------------------------------------------------------------ tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tcgen05_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc], bf16/f16 inputs, fp32 accumulate; one thread issues.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= (A * SFA)[smem desc] * (B * SFB)[smem desc]: e2m1 operands with one ue4m3 scale per 16 K elements (NVFP4),
// scale factors read from tensor memory; M = 128, K = 64 per instruction, fp32 accumulate. One thread issues.
__device__ __forceinline__ void umma_nvfp4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate,
                                           uint32_t tmem_sfa, uint32_t tmem_sfb) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}
// Instruction descriptor of the block-scaled NVFP4 MMA: e2m1 x e2m1, ue4m3 scales, K-major operands, K = 64.
__host__ __device__ constexpr uint32_t umma_idesc_nvfp4(int m, int n) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | (0u << 23) | ((uint32_t)(m >> 4) << 24);
}
// Copy 32 rows x 16 bytes from shared memory into 4 tensor-memory columns of all four 32-lane quarters (scale factors).
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// Shared-memory matrix descriptor, no swizzle, K-major: 8-row x 16-byte core matrices of 128 contiguous bytes;
// `lbo` = bytes between the two 16-byte K chunks an instruction reads, `sbo` = bytes between 8-row groups.
__device__ __forceinline__ uint64_t umma_desc_interleaved(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes with the 128-byte swizzle
// (what a TMA box of 64 x 16-bit elements with CU_TENSOR_MAP_SWIZZLE_128B writes): 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);        // start address, 16-byte units
  d |= (uint64_t)1 << 16;                              // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024u >> 4) << 32;                   // stride byte offset: 8 rows * 128 B
  d |= (uint64_t)1 << 46;                              // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                              // SWIZZLE_128B
  return d;
}
// Instruction descriptor for kind::f16: A, B bf16 (format 1) or f16 (format 0), both K-major, fp32 accumulator.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int m, int n, int ab_format) {
  return (1u << 4) | ((uint32_t)ab_format << 7) | ((uint32_t)ab_format << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

// 32 lanes x 32 columns of fp32 from TMEM: thread i of the warp gets lane (warp%4)*32+i, columns c..c+31.
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// ------------------------------------------------------------------------------------------------ small math
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// ------------------------------------------------------------------------------------------------ dependent launches
// A kernel launched through launch_dependent() may start while the kernel before it in the stream is still running
// (programmatic dependent launch): its blocks become resident as the earlier kernel's blocks retire, run whatever does
// not depend on earlier kernels (barrier and TMEM set-up, loads of weights), and call grid_dependency_wait() before the
// first access to memory that an earlier kernel writes or reads. grid_dependency_wait() returns once every kernel
// before this one in the stream has completed and its writes are visible; without the launch attribute it returns at
// once. grid_dependency_trigger() lets the NEXT kernel's blocks be scheduled as soon as every block of this grid has
// called it or exited; that kernel still waits for this one's completion in its own grid_dependency_wait().
// (The upstream GEMM launches the same way: pear/models/qwen3_5/rollout/blackwell/csrc/stream_gemm.cu:3-4.)
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#ifdef __CUDACC__
inline bool dependent_launch_enabled() {
  static const bool on = [] {
    const char* e = getenv("PEAR_DEPENDENT_LAUNCH");
    return !(e && e[0] == '0');
  }();
  return on;
}

// Launch `kernel` as a programmatic dependent of the work before it in `stream`. Every kernel launched this way calls
// grid_dependency_wait() before it touches anything but constants (weights, its own parameters).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(bool dependent, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = dependent && dependent_launch_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(static_cast<Args&&>(args))...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  return launch_kernel(true, kernel, grid, block, smem, stream, static_cast<Args&&>(args)...);
}
// An ordinary launch (the kernel starts after everything before it in the stream has completed) of a kernel that calls
// grid_dependency_trigger(): the kernel AFTER it, if launched as a dependent, may still start early. The step's small
// kernels are launched this way: as dependents they measured slower (a chain of row-norm kernels: 6.5 us per launch
// against 5.2 us), while the GEMM after each of them gains from filling its weight ring during their run.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_ordinary(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  return launch_kernel(false, kernel, grid, block, smem, stream, static_cast<Args&&>(args)...);
}
#endif

}  // namespace pear
