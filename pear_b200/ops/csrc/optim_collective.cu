// Gradient reduce-scatter fused with the cast / scale, the global-norm clip and the sharded AdamW update, and the
// parameter all-gather fused into the update's store, over NVLink / NVSwitch peer memory (upstream: NCCL reduce-scatter by
// FSDP2, then `_multi_tensor_adam` on the shards, then the next step's NCCL all-gather: pear/trainer/engine.py:155-236).
//
// Every rank holds a full flat gradient bucket (bf16 or fp32) and a full flat bf16 parameter bucket in symmetric memory
// and owns elements [lo, lo + n) of both, for which it also keeps the fp32 master weights and the two moments.
//   1. rs_sumsq:  pull the own range of every rank's gradient bucket (16-byte peer loads), sum in rank order in fp32,
//                 scale, store the reduced fp32 shard, and add this rank's sum of squares into slot `rank` of EVERY rank's
//                 norm buffer (one P2P store per peer: the all-reduce of the norm costs no extra collective).
//   2. adamw_bcast: total norm from the `world` partial sums, clip coefficient, AdamW on the shard in fp32, and the new
//                 bf16 parameters stored into the own range of EVERY rank's parameter bucket (the all-gather).
// The caller orders the steps with the flag kernels of comm_kernels.cu (signal + bounded wait) on the same stream:
// barrier, 1, barrier, 2, barrier. No step waits on a peer inside these two kernels.
#include "common.cuh"

#include <cuda_bf16.h>

namespace pear {

constexpr int kOptMaxRanks = 8;
struct OptPeers {
  void* p[kOptMaxRanks];
};

__device__ __forceinline__ uint4 opt_ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// 8 consecutive gradient elements of one rank starting at element `e` (a multiple of 8) as fp32
template <bool BF16>
__device__ __forceinline__ void load8(const void* base, size_t e, float (&g)[8]) {
  if (BF16) {
    const uint4 v = opt_ld_volatile_v4((const __nv_bfloat16*)base + e);
    const __nv_bfloat162* h = (const __nv_bfloat162*)&v;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      g[2 * i] = f.x;
      g[2 * i + 1] = f.y;
    }
  } else {
    const uint4 a = opt_ld_volatile_v4((const float*)base + e), b = opt_ld_volatile_v4((const float*)base + e + 4);
    g[0] = __uint_as_float(a.x); g[1] = __uint_as_float(a.y); g[2] = __uint_as_float(a.z); g[3] = __uint_as_float(a.w);
    g[4] = __uint_as_float(b.x); g[5] = __uint_as_float(b.y); g[6] = __uint_as_float(b.z); g[7] = __uint_as_float(b.w);
  }
}

template <bool BF16>
__global__ void __launch_bounds__(256) rs_sumsq_kernel(OptPeers grads, int rank, int world, size_t lo, size_t n, float scale,
                                                       float* __restrict__ reduced, float* __restrict__ block_sums) {
  __shared__ float red[8];
  float sq = 0.f;
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += (size_t)gridDim.x * blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, g[8];
    for (int r = 0; r < world; ++r) {  // rank order: every shard owner sums in the same order as a reference would
      load8<BF16>(grads.p[r], lo + i, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += g[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      acc[j] *= scale;
      sq += acc[j] * acc[j];
    }
    *(float4*)(reduced + i) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *(float4*)(reduced + i + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < 8; ++w) s += red[w];
    block_sums[blockIdx.x] = s;  // summed in block order by the publishing kernel: the norm is run-to-run identical
  }
}

// one warp: add the block sums in order and store the total into slot `rank` of every rank's norm buffer
__global__ void publish_sumsq_kernel(const float* __restrict__ block_sums, int nblocks, OptPeers norm_bufs, int rank, int world) {
  float s = 0.f;
  for (int i = threadIdx.x; i < nblocks; i += 32) s += block_sums[i];
  s = warp_sum(s);
  if (threadIdx.x < world) {
    ((volatile float*)norm_bufs.p[threadIdx.x])[rank] = s;
    __threadfence_system();
  }
}

__global__ void __launch_bounds__(256) adamw_bcast_kernel(const float* __restrict__ reduced, float* __restrict__ master,
                                                          float* __restrict__ m, float* __restrict__ v, const float* my_norm_buf,
                                                          OptPeers params, int world, size_t lo, size_t n, float lr, float beta1,
                                                          float beta2, float eps, float weight_decay, float bias1, float bias2,
                                                          float max_norm, float* __restrict__ norm_out) {
  float total = 0.f;
  for (int r = 0; r < world; ++r) total += ((const volatile float*)my_norm_buf)[r];
  const float norm = sqrtf(total);
  const float clip = max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
  if (blockIdx.x == 0 && threadIdx.x == 0 && norm_out) *norm_out = norm;
  const float step = lr / bias1, inv_sqrt_b2 = rsqrtf(bias2), decay = 1.f - lr * weight_decay;
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += (size_t)gridDim.x * blockDim.x * 8) {
    float g[8], p[8], mm[8], vv[8];
    *(float4*)&g[0] = *(const float4*)(reduced + i); *(float4*)&g[4] = *(const float4*)(reduced + i + 4);
    *(float4*)&p[0] = *(const float4*)(master + i);  *(float4*)&p[4] = *(const float4*)(master + i + 4);
    *(float4*)&mm[0] = *(const float4*)(m + i);      *(float4*)&mm[4] = *(const float4*)(m + i + 4);
    *(float4*)&vv[0] = *(const float4*)(v + i);      *(float4*)&vv[4] = *(const float4*)(v + i + 4);
    __nv_bfloat162 out[4];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * clip;
      mm[j] = beta1 * mm[j] + (1.f - beta1) * gj;
      vv[j] = beta2 * vv[j] + (1.f - beta2) * gj * gj;
      p[j] = p[j] * decay - step * mm[j] / (sqrtf(vv[j]) * inv_sqrt_b2 + eps);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) out[j] = __floats2bfloat162_rn(p[2 * j], p[2 * j + 1]);
    *(float4*)(master + i) = *(float4*)&p[0]; *(float4*)(master + i + 4) = *(float4*)&p[4];
    *(float4*)(m + i) = *(float4*)&mm[0];     *(float4*)(m + i + 4) = *(float4*)&mm[4];
    *(float4*)(v + i) = *(float4*)&vv[0];     *(float4*)(v + i + 4) = *(float4*)&vv[4];
    const uint4 packed = *(const uint4*)out;
    for (int r = 0; r < world; ++r) *(uint4*)((__nv_bfloat16*)params.p[r] + lo + i) = packed;  // the all-gather
  }
  __threadfence_system();
}

static OptPeers opt_ptrs(const void* const* a, int world) {
  OptPeers p{};
  for (int i = 0; i < world; ++i) p.p[i] = const_cast<void*>(a[i]);
  return p;
}
constexpr int kOptBlocks = 592;  // 4 per SM

}  // namespace pear

// grads[r]: rank r's flat gradient bucket (bf16 when grads_bf16, else fp32). This rank owns elements [lo, lo + n), both
// multiples of 8. reduced: fp32 [n]; block_sums: fp32 [592] scratch; norm_bufs[r]: rank r's fp32 [8] norm buffer.
PEAR_API int pear_rs_sumsq(const void* const* grads, int grads_bf16, int rank, int world, size_t lo, size_t n, float scale,
                           float* reduced, float* block_sums, const void* const* norm_bufs, void* stream) {
  using namespace pear;
  if (world < 1 || world > kOptMaxRanks || (lo % 8) || (n % 8)) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  if (grads_bf16) rs_sumsq_kernel<true><<<kOptBlocks, 256, 0, s>>>(opt_ptrs(grads, world), rank, world, lo, n, scale, reduced, block_sums);
  else rs_sumsq_kernel<false><<<kOptBlocks, 256, 0, s>>>(opt_ptrs(grads, world), rank, world, lo, n, scale, reduced, block_sums);
  PEAR_LAUNCH_CHECK();
  publish_sumsq_kernel<<<1, 32, 0, s>>>(block_sums, kOptBlocks, opt_ptrs(norm_bufs, world), rank, world);
  PEAR_LAUNCH_CHECK();
  return 0;
}

// AdamW (decoupled weight decay) on the shard; bias1 = 1 - beta1^t, bias2 = 1 - beta2^t; max_norm <= 0 disables the clip.
// params[r]: rank r's flat bf16 parameter bucket; norm_out (may be null): the global gradient norm before the clip.
PEAR_API int pear_adamw_bcast(const float* reduced, float* master, float* m, float* v, const float* my_norm_buf,
                              const void* const* params, int world, size_t lo, size_t n, float lr, float beta1, float beta2,
                              float eps, float weight_decay, float bias1, float bias2, float max_norm, float* norm_out,
                              void* stream) {
  using namespace pear;
  if (world < 1 || world > kOptMaxRanks || (lo % 8) || (n % 8)) return (int)cudaErrorInvalidValue;
  adamw_bcast_kernel<<<kOptBlocks, 256, 0, (cudaStream_t)stream>>>(reduced, master, m, v, my_norm_buf, opt_ptrs(params, world), world,
                                                                  lo, n, lr, beta1, beta2, eps, weight_decay, bias1, bias2,
                                                                  max_norm, norm_out);
  PEAR_LAUNCH_CHECK();
  return 0;
}

// ------------------------------------------------------------------------------------------------ local fused AdamW
// One pass over a parameter tensor: p, m, v read and written once, the gradient read once (torch's AdamW statements make
// about a dozen passes). The gradient may be fp32 or bf16; `grad_scale` carries the clip coefficient.
namespace pear {
template <bool G_BF16>
__global__ void __launch_bounds__(256) adamw_local_kernel(float* __restrict__ p, const void* __restrict__ g, float* __restrict__ m,
                                                          float* __restrict__ v, size_t n, float lr, float beta1, float beta2, float eps,
                                                          float weight_decay, float bias1, float bias2, float grad_scale) {
  const float step = lr / bias1, inv_sqrt_b2 = rsqrtf(bias2), decay = 1.f - lr * weight_decay;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float gi = (G_BF16 ? __bfloat162float(((const __nv_bfloat16*)g)[i]) : ((const float*)g)[i]) * grad_scale;
    const float mi = beta1 * m[i] + (1.f - beta1) * gi;
    const float vi = beta2 * v[i] + (1.f - beta2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    p[i] = p[i] * decay - step * mi / (sqrtf(vi) * inv_sqrt_b2 + eps);
  }
}
}  // namespace pear

PEAR_API int pear_adamw_local(float* p, const void* g, int grad_bf16, float* m, float* v, size_t n, float lr, float beta1, float beta2,
                              float eps, float weight_decay, float bias1, float bias2, float grad_scale, void* stream) {
  using namespace pear;
  if (n == 0) return 0;
  const size_t want = (n + 255) / 256;
  const int grid = (int)(want < 148 * 16 ? want : 148 * 16);
  if (grad_bf16) adamw_local_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(p, g, m, v, n, lr, beta1, beta2, eps, weight_decay, bias1, bias2, grad_scale);
  else adamw_local_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(p, g, m, v, n, lr, beta1, beta2, eps, weight_decay, bias1, bias2, grad_scale);
  PEAR_LAUNCH_CHECK();
  return 0;
}
