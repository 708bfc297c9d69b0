// Kernels that talk to peer GPUs directly over NVLink / NVSwitch through symmetric memory (every rank allocates the
// same buffers and exchanges their addresses once; a kernel then reads or writes a peer's buffer with plain loads and
// stores). Nothing here uses cluster multicast or TMA on peer memory.
//
// Synchronisation is by 32-bit flags in each rank's signal region, laid out [slot][source rank]. A flag carries an
// epoch that only grows; a waiter polls its OWN copy (`ld.acquire.sys`) until the epoch is reached. EVERY wait has a
// poll budget: on expiry the kernel writes an error code to its status word and returns, so a peer that never arrives
// costs a bounded delay, not a hung GPU (upstream's waits are unbounded polls: rollout/blackwell/csrc/ar_norm.cu:155-165,
// logits_gather.cu:68).
#include "common.cuh"

#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace pear {

constexpr int kMaxRanks = 8;
constexpr int kFlagSlotStride = kMaxRanks;  // uint32 per slot

struct PeerPtrs {
  void* p[kMaxRanks];
};

// 16-byte load that always goes to memory (peer data must never come from a stale cache line)
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// true once flag >= epoch (wrap-safe); false after `budget` polls
__device__ __forceinline__ bool wait_flag_sys(const uint32_t* flag, uint32_t epoch, uint32_t budget) {
  for (uint32_t i = 0; i < budget; ++i) {
    if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
    if (i > 32) __nanosleep(100);
  }
  return false;
}

// ------------------------------------------------------------------------------------------------ signal / wait
// Tell every rank "my slot reached `epoch`": one release store per peer, ordered after everything this stream wrote.
__global__ void symm_signal_kernel(PeerPtrs flags, int rank, int world, int slot, uint32_t epoch) {
  const int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();
    st_release_sys((uint32_t*)flags.p[r] + slot * kFlagSlotStride + rank, epoch);
  }
}

// Wait until every rank's flag of `slot` in MY signal region reached `epoch`.
__global__ void symm_wait_kernel(const uint32_t* my_flags, int world, int slot, uint32_t epoch, uint32_t budget, int* status) {
  const int r = threadIdx.x;
  if (r < world && !wait_flag_sys(my_flags + slot * kFlagSlotStride + r, epoch, budget)) set_status(status, PEAR_ERR_FLAG_TIMEOUT);
}

// ------------------------------------------------------------------------------------------------ all-reduce + add + norm
// One-shot all-reduce fused with the fp32 residual add and the (1 + w) RMSNorm (the op after every row-parallel
// projection of a tensor-parallel decode step; upstream ar_norm.cu:61-208 at TP2 with a sentinel protocol).
// Each rank has written its partial rows [T, H] (bf16) into buffer `epoch & 1` of its symmetric region. The kernel
// signals that, waits for all ranks' signals, then every rank reads all partials straight from the peers' memory, sums
// them in rank order in fp32 (all ranks get bit-identical sums), adds the residual, writes it back and writes the
// normalised rows. Two buffers by epoch parity are enough: a rank overwrites buffer b again at epoch e + 2, which it
// only reaches after every rank signalled e + 1, i.e. after they finished reading e.
template <int VEC>
__global__ void __launch_bounds__(256) ar_add_rmsnorm_kernel(PeerPtrs partials, PeerPtrs flags, int rank, int world, int slot,
                                                             uint32_t epoch, float* __restrict__ residual,
                                                             const float* __restrict__ weight, __nv_bfloat16* __restrict__ out,
                                                             int T, int H, size_t buf_elems, float eps, uint32_t budget, int* status) {
  __shared__ float red[8];
  __shared__ int ok_flag;
  const int tid = threadIdx.x;
  if (blockIdx.x == 0 && tid < world) {
    __threadfence_system();
    st_release_sys((uint32_t*)flags.p[tid] + slot * kFlagSlotStride + rank, epoch);
  }
  if (tid == 0) ok_flag = 1;
  __syncthreads();
  if (tid < world && !wait_flag_sys((const uint32_t*)flags.p[rank] + slot * kFlagSlotStride + tid, epoch, budget)) {
    set_status(status, PEAR_ERR_FLAG_TIMEOUT);
    ok_flag = 0;
  }
  __syncthreads();
  if (!ok_flag) return;
  const size_t boff = (size_t)(epoch & 1u) * buf_elems;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    float ssq = 0.f;
    for (int i = tid * VEC; i < H; i += blockDim.x * VEC) {
      float acc[VEC];
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
      for (int r = 0; r < world; ++r) {
        const __nv_bfloat16* src = (const __nv_bfloat16*)partials.p[r] + boff + (size_t)t * H + i;
        const uint4 v = ld_volatile_v4(src);
        const __nv_bfloat162* h2 = (const __nv_bfloat162*)&v;
#pragma unroll
        for (int j = 0; j < VEC / 2; ++j) {
          const float2 f = __bfloat1622float2(h2[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      float* res = residual + (size_t)t * H + i;
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        acc[j] += res[j];
        res[j] = acc[j];
        ssq += acc[j] * acc[j];
      }
    }
    ssq = warp_sum(ssq);
    if ((tid & 31) == 0) red[tid >> 5] = ssq;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
    const float rstd = rsqrtf(tot / (float)H + eps);
    __syncthreads();
    for (int i = tid * VEC; i < H; i += blockDim.x * VEC) {
      const float* res = residual + (size_t)t * H + i;
      __nv_bfloat16* o = out + (size_t)t * H + i;
#pragma unroll
      for (int j = 0; j < VEC; ++j) o[j] = __float2bfloat16_rn(res[j] * rstd * (1.f + weight[i + j]));
    }
  }
}

// ------------------------------------------------------------------------------------------------ weight sync: bf16 -> NVFP4
// amax of a bf16 matrix that may live on a peer (the trainer's staging buffer): float bits through atomicMax.
__global__ void amax_bf16_kernel(const __nv_bfloat16* __restrict__ src, size_t n, unsigned int* __restrict__ out_bits) {
  float m = 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i * 8 < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 v = ld_volatile_v4(src + i * 8);
    const __nv_bfloat162* h2 = (const __nv_bfloat162*)&v;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h2[j]);
      m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) atomicMax(out_bits, __float_as_uint(m));
}

__device__ __forceinline__ uint32_t e2m1_code(float x) {
  const float a = fabsf(x);
  // nearest e2m1 magnitude; a tie goes to the code with an even index
  uint32_t c = a > 0.25f ? 1u : 0u;
  c = a >= 0.75f ? 2u : c;
  c = a > 1.25f ? 3u : c;
  c = a >= 1.75f ? 4u : c;
  c = a > 2.5f ? 5u : c;
  c = a >= 3.5f ? 6u : c;
  c = a > 5.0f ? 7u : c;
  return c | ((x < 0.f && c != 0u) ? 8u : 0u);
}

// Weight broadcast fused with requantisation: every receiving rank pulls the bf16 rows from the sender's staging buffer
// over NVLink and writes NVFP4 (e2m1 codes, e4m3 block scales, power-of-two tensor scale) directly in the decode
// megakernel's streaming layout, so the bf16 copy never lands in the receiver's HBM. One thread per 16-element block.
//   codes : (tile * ks + kstage) * 18432 + (chunk * 16 + row/8) * 128 + (row%8) * 16 + byte      chunk = (k % 256) / 32
//   scales: ... + 16384 + j * 512 + (row%32) * 16 + (row/32) * 4 + block                          j = (k % 256) / 64
__global__ void bcast_quant_nvfp4_kernel(const __nv_bfloat16* __restrict__ src, int rows, int K, int ld, float gscale,
                                         uint8_t* __restrict__ packed) {
  const int blocks_per_row = K >> 4;
  const int ks = K >> 8;
  const size_t total = (size_t)rows * blocks_per_row;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int row = (int)(idx / blocks_per_row), blk = (int)(idx % blocks_per_row);
    const __nv_bfloat16* s = src + (size_t)row * ld + blk * 16;
    const uint4 v0 = ld_volatile_v4(s), v1 = ld_volatile_v4(s + 8);
    float x[16];
    const __nv_bfloat162* a = (const __nv_bfloat162*)&v0;
    const __nv_bfloat162* b = (const __nv_bfloat162*)&v1;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(a[j]);
      x[2 * j] = f.x; x[2 * j + 1] = f.y;
      f = __bfloat1622float2(b[j]);
      x[8 + 2 * j] = f.x; x[8 + 2 * j + 1] = f.y;
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(x[j]));
    const float target = fminf(amax / 6.0f * gscale, 448.f);
    const __nv_fp8_storage_t sc = __nv_cvt_float_to_fp8(target, __NV_SATFINITE, __NV_E4M3);
    const float sf = __half2float(__half(__nv_cvt_fp8_to_halfraw(sc, __NV_E4M3)));
    const float inv = sf > 0.f ? gscale / sf : 0.f;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      lo |= e2m1_code(x[j] * inv) << (4 * j);
      hi |= e2m1_code(x[8 + j] * inv) << (4 * j);
    }
    const int tile = row >> 7, r = row & 127;
    const int k = blk * 16, kst = k >> 8, kin = k & 255;
    uint8_t* stage = packed + ((size_t)tile * ks + kst) * 18432;
    uint8_t* dst = stage + ((kin >> 5) * 16 + (r >> 3)) * 128 + (r & 7) * 16 + ((kin >> 4) & 1) * 8;
    *(uint2*)dst = make_uint2(lo, hi);
    stage[16384 + (kin >> 6) * 512 + (r & 31) * 16 + (r >> 5) * 4 + ((kin >> 4) & 3)] = (uint8_t)sc;
  }
}

// ------------------------------------------------------------------------------------------------ logits all-gather
// Vocab-parallel lm_head: every rank holds fp32 logits [T, Vs] of its vocabulary shard and writes them into the full
// [T, V] buffer of EVERY rank at column offset rank * Vs with 16-byte stores over NVLink (upstream sg_logits / lg_gather,
// rollout/blackwell/csrc/logits_gather.cu:32-68, for two ranks). Grid-stride over (peer, row, 4-float vector), peers
// visited starting after the own rank so the ranks write to different targets at any moment. Completion is published by
// pear_symm_signal after the kernel; readers wait with pear_symm_wait.
__global__ void __launch_bounds__(256) logits_allgather_kernel(const float4* __restrict__ shard, PeerPtrs full, int rank, int world, int T, int Vs4,
                                                                int ld4) {
  const size_t per_peer = (size_t)T * Vs4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < per_peer * world; i += (size_t)gridDim.x * blockDim.x) {
    const int p = (rank + 1 + (int)(i / per_peer)) % world;
    const size_t e = i % per_peer;
    const int t = (int)(e / Vs4), c = (int)(e % Vs4);
    ((float4*)full.p[p])[(size_t)t * ld4 + (size_t)rank * Vs4 + c] = shard[e];
  }
  __threadfence_system();
}

// ------------------------------------------------------------------------------------------------ sharded argmax exchange
// The drafter's greedy token under vocabulary parallelism (upstream draft_argmax.cu: one tagged 64-bit word per row
// swapped with the peer): every rank reduces its logits shard [rows, Vs] to (max value, global token id) per row, packs
// them as an ORDERED 64-bit key (monotone float bits << 32 | ~token, so ties go to the lower id) and stores the key into
// slot `rank` of EVERY rank's exchange buffer [rows][world]. After signal / wait, arg_finish takes the maximum key per row.
__global__ void __launch_bounds__(256) argmax_shard_kernel(const float* __restrict__ logits, int Vs, int ld, int v0, PeerPtrs xbuf, int rank, int world) {
  __shared__ unsigned long long red[8];
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* x = logits + (size_t)row * ld;
  unsigned long long best = 0ull;
  for (int i = tid; i < Vs; i += blockDim.x) {
    uint32_t b = __float_as_uint(x[i]);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);  // monotone map of IEEE floats to unsigned
    const unsigned long long key = ((unsigned long long)b << 32) | (uint32_t)~(uint32_t)(v0 + i);
    best = key > best ? key : best;
  }
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((tid & 31) == 0) red[tid >> 5] = best;
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < 8; ++w) best = red[w] > best ? red[w] : best;
    for (int p = 0; p < world; ++p) {
      const int peer = (rank + p) % world;
      ((volatile unsigned long long*)xbuf.p[peer])[(size_t)row * kMaxRanks + rank] = best;
    }
    __threadfence_system();
  }
}

__global__ void argmax_finish_kernel(const unsigned long long* __restrict__ my_xbuf, int rows, int world, int* __restrict__ token, float* __restrict__ value) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  unsigned long long best = 0ull;
  for (int r = 0; r < world; ++r) {
    const unsigned long long k = ((const volatile unsigned long long*)my_xbuf)[(size_t)row * kMaxRanks + r];
    best = k > best ? k : best;
  }
  uint32_t b = (uint32_t)(best >> 32);
  b = (b & 0x80000000u) ? (b & 0x7FFFFFFFu) : ~b;
  token[row] = (int)~(uint32_t)best;
  value[row] = __uint_as_float(b);
}

}  // namespace pear

using namespace pear;

// ------------------------------------------------------------------------------------------------ strided block pull
// Copy a [rows, row_bytes] block out of a peer's (or the local) memory into local memory, both sides strided: the weight-sync
// receiver takes only its own tensor-parallel shard of each tensor out of the sender's staging buffer (a column-parallel
// matrix is a row range, a row-parallel one a column range). 16-byte loads when both sides allow it. One CTA per group of rows.
__global__ void __launch_bounds__(256) pull_block_kernel(const uint8_t* __restrict__ src, long long src_ld, uint8_t* __restrict__ dst, long long dst_ld,
                                                         int rows, long long row_bytes, int vec) {
  constexpr long long kChunk = 32768;  // bytes of a row one CTA copies
  const long long c0 = (long long)blockIdx.y * kChunk;
  const long long c1 = c0 + kChunk < row_bytes ? c0 + kChunk : row_bytes;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint8_t* s = src + (long long)r * src_ld;
    uint8_t* d = dst + (long long)r * dst_ld;
    if (vec) {
      for (long long i = (c0 >> 4) + threadIdx.x; i < (c1 >> 4); i += blockDim.x) ((uint4*)d)[i] = ((const uint4*)s)[i];
    } else {
      for (long long i = c0 + threadIdx.x; i < c1; i += blockDim.x) d[i] = s[i];
    }
  }
}

static PeerPtrs to_ptrs(const void* const* host_ptrs, int world) {
  PeerPtrs p;
  for (int i = 0; i < kMaxRanks; ++i) p.p[i] = i < world ? const_cast<void*>(host_ptrs[i]) : nullptr;
  return p;
}

// flags: host array of `world` device pointers (each rank's signal region). Slots are 8 uint32 apart.
PEAR_API int pear_symm_signal(const void* const* flags, int rank, int world, int slot, unsigned epoch, void* stream) {
  if (world < 1 || world > kMaxRanks) return (int)cudaErrorInvalidValue;
  symm_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(to_ptrs(flags, world), rank, world, slot, epoch);
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_symm_wait(const void* my_flags, int world, int slot, unsigned epoch, unsigned budget, int* status, void* stream) {
  if (world < 1 || world > kMaxRanks) return (int)cudaErrorInvalidValue;
  symm_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((const uint32_t*)my_flags, world, slot, epoch, budget, status);
  PEAR_LAUNCH_CHECK();
  return 0;
}

// partials[r]: rank r's symmetric region of 2 x buf_elems bf16 (buffers by epoch parity), each buffer holding [T, H].
PEAR_API int pear_ar_add_rmsnorm(const void* const* partials, const void* const* flags, int rank, int world, int slot,
                                 unsigned epoch, float* residual, const float* weight, void* out_bf16, int T, int H,
                                 size_t buf_elems, float eps, unsigned budget, int* status, int num_ctas, void* stream) {
  if (world < 1 || world > kMaxRanks || (H % 8) != 0) return (int)cudaErrorInvalidValue;
  const int grid = T < num_ctas ? (T > 0 ? T : 1) : num_ctas;
  ar_add_rmsnorm_kernel<8><<<grid, 256, 0, (cudaStream_t)stream>>>(to_ptrs(partials, world), to_ptrs(flags, world), rank, world,
                                                                   slot, epoch, residual, weight, (__nv_bfloat16*)out_bf16, T, H,
                                                                   buf_elems, eps, budget, status);
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_amax_bf16(const void* src, size_t n, void* out_bits, void* stream) {
  if (n % 8) return (int)cudaErrorInvalidValue;
  amax_bf16_kernel<<<296, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)src, n, (unsigned int*)out_bits);
  PEAR_LAUNCH_CHECK();
  return 0;
}

// src: bf16 [rows, K] with leading dimension ld (local or a peer's memory); packed: tiles x (K/256) stages of 18432 bytes,
// zero-initialised by the caller when rows is not a multiple of 128.
PEAR_API int pear_bcast_quant_nvfp4(const void* src, int rows, int K, int ld, float gscale, void* packed, void* stream) {
  if ((K % 256) != 0 || (ld % 8) != 0) return (int)cudaErrorInvalidValue;
  bcast_quant_nvfp4_kernel<<<592, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)src, rows, K, ld, gscale, (uint8_t*)packed);
  PEAR_LAUNCH_CHECK();
  return 0;
}

// shard: fp32 [T, Vs] contiguous; full[r]: rank r's fp32 [T, ld] buffer (ld >= world * Vs); Vs and ld multiples of 4.
PEAR_API int pear_logits_allgather(const void* shard, const void* const* full, int rank, int world, int T, int Vs, int ld, void* stream) {
  if (world < 1 || world > kMaxRanks || (Vs % 4) || (ld % 4)) return (int)cudaErrorInvalidValue;
  logits_allgather_kernel<<<296, 256, 0, (cudaStream_t)stream>>>((const float4*)shard, to_ptrs(full, world), rank, world, T, Vs / 4, ld / 4);
  PEAR_LAUNCH_CHECK();
  return 0;
}

// logits: this rank's fp32 shard [rows, Vs] (columns v0 .. v0 + Vs of the vocabulary); xbuf[r]: rank r's exchange buffer
// of rows * 8 uint64. Order with pear_symm_signal / pear_symm_wait, then pear_argmax_finish.
PEAR_API int pear_argmax_shard(const float* logits, int rows, int Vs, int ld, int v0, const void* const* xbuf, int rank, int world, void* stream) {
  if (world < 1 || world > kMaxRanks) return (int)cudaErrorInvalidValue;
  argmax_shard_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>(logits, Vs, ld, v0, to_ptrs(xbuf, world), rank, world);
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_argmax_finish(const void* my_xbuf, int rows, int world, int* token, float* value, void* stream) {
  argmax_finish_kernel<<<(rows + 127) / 128, 128, 0, (cudaStream_t)stream>>>((const unsigned long long*)my_xbuf, rows, world, token, value);
  PEAR_LAUNCH_CHECK();
  return 0;
}

// src: a device pointer into a peer's symmetric buffer (or local memory); strides and sizes in bytes.
PEAR_API int pear_pull_block(const void* src, long long src_ld, void* dst, long long dst_ld, int rows, long long row_bytes, void* stream) {
  if (rows <= 0 || row_bytes <= 0) return 0;
  const int vec = ((uintptr_t)src % 16 == 0) && ((uintptr_t)dst % 16 == 0) && (src_ld % 16 == 0) && (dst_ld % 16 == 0) && (row_bytes % 16 == 0);
  const long long chunks = (row_bytes + 32767) / 32768;
  if (chunks > 65535) return (int)cudaErrorInvalidValue;  // a single row of more than 2 GB: cut it on the caller's side
  const long long want = 1184 / chunks > 0 ? 1184 / chunks : 1;
  const dim3 grid((unsigned)(rows < want ? rows : want), (unsigned)chunks);
  pull_block_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)src, src_ld, (uint8_t*)dst, dst_ld, rows, row_bytes, vec);
  PEAR_LAUNCH_CHECK();
  return 0;
}
