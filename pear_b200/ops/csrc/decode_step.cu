// Kernels of the batched, GPU-resident rollout step (decode and speculative-verify rows of many sequences at once).
// Every per-sequence quantity a step needs lives in device arrays that the step's own kernels update (context length,
// replay count, record parity, next input tokens), so a step is a fixed sequence of launches with fixed arguments and
// can be replayed as a CUDA graph without the host in the loop (upstream gets there through vLLM's runner buffers and
// per-size graphs: rollout/blackwell/cudagraph.py:4-34, rollout/hopper/gdn.py:58-171).
//
// Row layout of a step: B sequences x T rows (row = b * T + t); t = 0 is the last committed token, t >= 1 the drafts.
// A sequence with ctx[b] < 0 is an empty batch slot: every kernel skips it.
//
//   ds_add_rmsnorm        residual (+)= sum of split-K planes; (1 + w) RMSNorm -> bf16 activations for the next GEMM
//   ds_reduce_parts_bf16  sum of split-K planes -> bf16 rows in the tensor-parallel all-reduce workspace
//   ds_attn_prep          per-head q/k RMSNorm + RoPE + gate split + K/V written into the paged cache (one kernel;
//                         upstream rollout/attention.py:5-71 `_qk_norm_rope_gate_kernel` + the cache write)
//   ds_paged_attn_simt    reference / small-shape paged verify attention with the sigmoid gate fused
//   ds_gdn_verify         Gated-DeltaNet core of a verify step under the replay scheme (upstream gdn_verify.cu:643-1395):
//                         replay the rows committed by the previous step, write the state once, then the block's outputs
//   ds_verify_chunks / ds_verify_finish   vocabulary-sharded rejection sampler of greedy drafts with in-kernel Philox
//   ds_mtp_input          drafter input rows [norm_e(embed(token)) | norm_h(hidden)] (upstream rollout/blackwell/mtp.py:16)
//   ds_argmax_chunks / ds_argmax_finish   drafter's greedy token over a vocabulary shard
#include "common.cuh"

#include <cudaTypedefs.h>
#include <cuda_bf16.h>
#include <cfloat>

namespace pear {

constexpr int kDsMaxRanks = 8;
struct DsPeers {
  void* p[kDsMaxRanks];
};

// ------------------------------------------------------------------------------------------------ Philox noise
__device__ __forceinline__ uint4 ds_philox4x32_10(uint4 ctr, uint2 key) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0; key.y += W1;
  }
  return ctr;
}
// 23 random bits + 1/2: every value is exact in fp32 and lies strictly inside (0, 1). (With 24 bits the largest one,
// 2^24 - 1/2, rounds to 2^24: a uniform of exactly 1 makes the exponential-race key infinite, and at 248 320 draws per row
// that happened in about 1.5 percent of the rows: found by the goodness-of-fit test.)
__device__ __forceinline__ float ds_u01(uint32_t x) { return ((float)(x >> 9) + 0.5f) * (1.0f / 8388608.0f); }
// uniforms of vocabulary ids 4*q .. 4*q+3 of (row, step): the same numbers whatever the sharding or the chunking
__device__ __forceinline__ uint4 ds_noise4(uint32_t seed, uint32_t step, uint32_t row, uint32_t quad) {
  return ds_philox4x32_10(make_uint4(quad, row, step, 0u), make_uint2(seed, 0x5eedu));
}
__device__ __forceinline__ float ds_accept_u(uint32_t seed, uint32_t step, uint32_t row) {
  return ds_u01(ds_philox4x32_10(make_uint4(0xffffffffu, row, step, 1u), make_uint2(seed, 0x5eedu)).x);
}

__global__ void ds_philox_uniform_kernel(float* out, int rows, int V, uint32_t seed, uint32_t step) {
  const int row = blockIdx.y;
  for (int q = blockIdx.x * blockDim.x + threadIdx.x; q * 4 < V; q += gridDim.x * blockDim.x) {
    const uint4 r = ds_noise4(seed, step, row, q);
    const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
    for (int e = 0; e < 4; ++e)
      if (q * 4 + e < V) out[(size_t)row * V + q * 4 + e] = ds_u01(rr[e]);
  }
}
__global__ void ds_accept_uniform_kernel(float* out, int rows, uint32_t seed, uint32_t step) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < rows) out[r] = ds_accept_u(seed, step, r);
}

// ------------------------------------------------------------------------------------------------ add + RMSNorm
// mode 0: residual += sum(planes); mode 1: residual = sum(planes); then out = bf16(residual * rstd * (1 + w)).
__global__ void __launch_bounds__(256) ds_add_rmsnorm_kernel(const float* __restrict__ parts, int nsplit, long long split_stride, int ldp,
                                                             float* __restrict__ residual, int mode, const float* __restrict__ w,
                                                             __nv_bfloat16* __restrict__ out, int H, float eps, int one_plus) {
  grid_dependency_trigger();
  grid_dependency_wait();
  __shared__ float red[8];
  const int row = blockIdx.x, tid = threadIdx.x;
  float* res = residual + (size_t)row * H;
  // a row of up to 8192 elements stays in registers between the two passes (8 x 4 per thread); every load of the kernel
  // (residual, planes, norm weight) is issued before the first use
  constexpr int kMaxIt = 8;
  float4 v[kMaxIt], g[kMaxIt];
  const bool in_regs = H <= kMaxIt * 1024;
  float ssq = 0.f;
  if (in_regs) {
#pragma unroll
    for (int k = 0; k < kMaxIt; ++k) {
      const int i = tid * 4 + k * 1024;
      v[k] = (i < H && mode == 0) ? *(const float4*)(res + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      g[k] = i < H ? *(const float4*)(w + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int s = 0; s < nsplit; ++s) {
      const float* ps = parts + (size_t)s * split_stride + (size_t)row * ldp;
#pragma unroll
      for (int k = 0; k < kMaxIt; ++k) {
        const int i = tid * 4 + k * 1024;
        if (i < H) {
          const float4 p = *(const float4*)(ps + i);
          v[k].x += p.x; v[k].y += p.y; v[k].z += p.z; v[k].w += p.w;
        }
      }
    }
#pragma unroll
    for (int k = 0; k < kMaxIt; ++k) {
      const int i = tid * 4 + k * 1024;
      if (i < H) {
        if (nsplit > 0 || mode == 1) *(float4*)(res + i) = v[k];
        ssq += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
      }
    }
  } else {
    for (int i = tid * 4; i < H; i += 1024) {
      float4 t = mode == 0 ? *(const float4*)(res + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < nsplit; ++s) {
        const float4 p = *(const float4*)(parts + (size_t)s * split_stride + (size_t)row * ldp + i);
        t.x += p.x; t.y += p.y; t.z += p.z; t.w += p.w;
      }
      if (nsplit > 0 || mode == 1) *(float4*)(res + i) = t;
      ssq += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
    }
  }
  ssq = warp_sum(ssq);
  if ((tid & 31) == 0) red[tid >> 5] = ssq;
  __syncthreads();
  float tot = 0.f;
  for (int k = 0; k < 8; ++k) tot += red[k];
  const float rstd = rsqrtf(tot / (float)H + eps);
  const float a = one_plus ? 1.f : 0.f;
  auto emit = [&](int i, const float4& x, const float4& gg) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(x.x * rstd * (a + gg.x), x.y * rstd * (a + gg.y));
    __nv_bfloat162 hi = __floats2bfloat162_rn(x.z * rstd * (a + gg.z), x.w * rstd * (a + gg.w));
    uint2 pk;
    pk.x = *(uint32_t*)&lo; pk.y = *(uint32_t*)&hi;
    *(uint2*)(out + (size_t)row * H + i) = pk;
  };
  if (in_regs) {
#pragma unroll
    for (int k = 0; k < kMaxIt; ++k) {
      const int i = tid * 4 + k * 1024;
      if (i < H) emit(i, v[k], g[k]);
    }
  } else {
    for (int i = tid * 4; i < H; i += 1024) emit(i, *(const float4*)(res + i), *(const float4*)(w + i));
  }
}

// sum of split-K planes -> bf16 rows (the rank's partial of a row-parallel projection, staged for the all-reduce).
// `epoch_ctr` (may be null): the workspace has two [rows, H] buffers; the one of epoch *epoch_ctr + 1 is written.
__global__ void __launch_bounds__(256) ds_reduce_parts_bf16_kernel(const float* __restrict__ parts, int nsplit, long long split_stride, int ldp,
                                                                   __nv_bfloat16* __restrict__ out, size_t buf_elems,
                                                                   const uint32_t* __restrict__ epoch_ctr, int H) {
  grid_dependency_trigger();
  grid_dependency_wait();
  const int row = blockIdx.x;
  __nv_bfloat16* o = out + (epoch_ctr ? (size_t)((*epoch_ctr + 1u) & 1u) * buf_elems : 0) + (size_t)row * H;
  for (int i = threadIdx.x * 4; i < H; i += 1024) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < nsplit; ++s) {
      const float4 p = *(const float4*)(parts + (size_t)s * split_stride + (size_t)row * ldp + i);
      v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 pk;
    pk.x = *(uint32_t*)&lo; pk.y = *(uint32_t*)&hi;
    *(uint2*)(o + i) = pk;
  }
}

// ------------------------------------------------------------------------------------------------ attention prep
// qkv fp32 row: Hq x [q(D) | gate(D)] (or Hq x q(D) when ungated), then Hkv x k(D), then Hkv x v(D).
// One CTA per row, a warp per head: (1 + w) RMSNorm over the head, RoPE on the first `rot` channels pairing channel i
// with i + rot/2 (all three M-RoPE axes carry the same position for generated text), q -> bf16 [row][Hq][D],
// k and v -> bf16 into the paged cache at position ctx[b] + t. The gate stays in the projection output.
template <int D>
__global__ void __launch_bounds__(256) ds_attn_prep_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ qn_w,
                                                           const float* __restrict__ kn_w, const double* __restrict__ inv_freq, int rot,
                                                           const int* __restrict__ ctx, const int* __restrict__ rope_off,
                                                           const int* __restrict__ block_table, int max_blocks, int T, int Hq, int Hkv, int gated,
                                                           float eps, __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ kc,
                                                           __nv_bfloat16* __restrict__ vc) {
  grid_dependency_trigger();
  grid_dependency_wait();
  __shared__ float cs[64], sn[64];
  __shared__ float head[8][D];
  const int row = blockIdx.x, b = row / T, t = row % T;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = ctx[b];
  if (c < 0) return;
  const int pos = c + t;
  const int half = rot >> 1;
  if (threadIdx.x < half) {
    const double ang = (double)(pos + rope_off[b]) * inv_freq[threadIdx.x];
    double sv, cv;
    sincos(ang, &sv, &cv);
    cs[threadIdx.x] = (float)cv; sn[threadIdx.x] = (float)sv;
  }
  __syncthreads();
  const float* x = qkv + (size_t)row * ld;
  const int qstride = gated ? 2 * D : D;
  const size_t cache_row = ((size_t)block_table[(size_t)b * max_blocks + (pos >> 4)] * 16 + (pos & 15)) * Hkv;
  for (int h = warp; h < Hq + 2 * Hkv; h += 8) {
    const float* src;
    const float* nw = nullptr;
    __nv_bfloat16* dst;
    if (h < Hq) { src = x + (size_t)h * qstride; nw = qn_w; dst = q_out + ((size_t)row * Hq + h) * D; }
    else if (h < Hq + Hkv) { src = x + (size_t)Hq * qstride + (size_t)(h - Hq) * D; nw = kn_w; dst = kc + (cache_row + (h - Hq)) * D; }
    else { src = x + (size_t)Hq * qstride + (size_t)Hkv * D + (size_t)(h - Hq - Hkv) * D; dst = vc + (cache_row + (h - Hq - Hkv)) * D; }
    float v[D / 32];
    float ssq = 0.f;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) { v[i] = src[lane + 32 * i]; ssq += v[i] * v[i]; }
    if (nw) {
      ssq = warp_sum(ssq);
      const float rstd = rsqrtf(ssq / (float)D + eps);
#pragma unroll
      for (int i = 0; i < D / 32; ++i) head[warp][lane + 32 * i] = v[i] * rstd * (1.f + nw[lane + 32 * i]);
      __syncwarp();
#pragma unroll
      for (int i = 0; i < D / 32; ++i) {
        const int ch = lane + 32 * i;
        float y = head[warp][ch];
        if (ch < half) y = y * cs[ch] - head[warp][ch + half] * sn[ch];
        else if (ch < rot) y = y * cs[ch - half] + head[warp][ch - half] * sn[ch - half];
        v[i] = y;
      }
      __syncwarp();
    }
#pragma unroll
    for (int i = 0; i < D / 32; ++i) dst[lane + 32 * i] = __float2bfloat16_rn(v[i]);
  }
}

// ------------------------------------------------------------------------------------------------ paged attention (SIMT)
// Row (b, t) attends to keys 0 .. ctx[b] + t of its sequence. Grid (rows, kv heads); a warp per query head of the group.
// out bf16 [row][Hq * D] = softmax(q k^T * scale) v * sigmoid(gate). The plain statement of the op: the tensor-core
// kernel (paged_attn_tc.cu) is checked against it, and it serves head sizes that kernel is not built for.
template <int D>
__global__ void __launch_bounds__(256) ds_paged_attn_simt_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                                                                 const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_table,
                                                                 int max_blocks, const int* __restrict__ ctx, int T, int Hq, int Hkv, float scale,
                                                                 const float* __restrict__ gate_src, int gate_ld, int gated,
                                                                 __nv_bfloat16* __restrict__ out) {
  const int row = blockIdx.x, kvh = blockIdx.y, b = row / T, t = row % T;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = Hq / Hkv;
  const int c = ctx[b];
  if (warp >= group || c < 0) return;
  const int h = kvh * group + warp;
  const int len = c + t + 1;
  constexpr int PER = D / 32;
  float qv[PER], acc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) { qv[i] = __bfloat162float(q[((size_t)row * Hq + h) * D + lane + 32 * i]) * scale; acc[i] = 0.f; }
  float m = -FLT_MAX, l = 0.f;
  for (int k = 0; k < len; ++k) {
    const int blk = block_table[(size_t)b * max_blocks + (k >> 4)];
    const size_t base = (((size_t)blk * 16 + (k & 15)) * Hkv + kvh) * D;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) s += qv[i] * __bfloat162float(kc[base + lane + 32 * i]);
    s = warp_sum(s);
    const float mn = fmaxf(m, s), corr = __expf(m - mn), p = __expf(s - mn);
    l = l * corr + p;
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = acc[i] * corr + p * __bfloat162float(vc[base + lane + 32 * i]);
    m = mn;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    float o = acc[i] * inv;
    if (gated) {
      const float g = gate_src[(size_t)row * gate_ld + (size_t)h * 2 * D + D + lane + 32 * i];
      o *= 1.f / (1.f + __expf(-g));
    }
    out[(size_t)row * Hq * D + (size_t)h * D + lane + 32 * i] = __float2bfloat16_rn(o);
  }
}

// ------------------------------------------------------------------------------------------------ GDN verify core
// proj fp32 row: [q (Hk*128) | k (Hk*128) | v (Hv*128) | z (Hv*128) | b (Hv) | a (Hv)].
// Per sequence and GDN layer the cache holds the recurrent state at the START of the sequence's last block (fp32
// [Hv][128][128], one slot) and a two-copy record of that block: conv_rec [slot][2][3 + Tmax][C] = the three conv inputs
// before the block followed by the block's conv inputs, ab_rec [slot][2][Tmax][2 * Hv] = its (a, b) rows. A step reads copy
// `parity[b]`, replays the first ncommit[b] rows of the old block into the state (those were accepted), stores the state,
// then runs this step's T rows to produce their outputs and writes the new block into the other copy. Nothing of the
// rejected rows ever reaches the stored state. T = 0 only replays (flush before a snapshot or when the sequence leaves
// the batch). (Upstream: rollout/blackwell/csrc/gdn_verify.cu:643 verify, :737 prep — effective vectors, 3xTF32.)
//
// The rows' recurrence  S <- g_t S;  u_t = beta_t (v_t - S k_t);  S <- S + u_t k_t^T;  o_t = S q_t  is independent per
// state row i and linear in the start state S0, so with G_t = g_0 .. g_t
//     a_t[i] = G_t (S0 k_t)[i] + sum_{tau < t}  (G_t / G_tau) u_tau[i] (k_tau . k_t),      u_t[i] = beta_t (v_t[i] - a_t[i])
//     o_t[i] = G_t (S0 q_t)[i] + sum_{tau <= t} (G_t / G_tau) u_tau[i] (k_tau . q_t)
//     S_nc   = G_{nc-1} S0 + sum_{tau < nc} (G_{nc-1} / G_tau) u_tau k_tau^T                (the state that is stored)
// Two kernels. ds_gdn_prep_kernel (a CTA per key head and one per value head, per sequence) runs the conv + SiLU + L2 norm
// front end of every row once per KEY head (three value heads share it), the gates, the k.k / k.q table, writes the new
// record, and leaves the vectors already laid out as tensor-core operands. ds_gdn_state_kernel (CTA per value head and sequence, two per SM)
// makes the two passes over the 64 KB state as tcgen05 products: P = S0 [k_0..k_7 | q_0..q_7] (M = 128 state rows, N = 16
// vectors, K = 128) and the rank-nc update D = U' K^T (M = 128, N = 128, K = 8); between them each of 128 threads walks
// its row's <= 8 steps on scalars. kind::tf32 with every fp32 operand split into a tf32 head and a remainder (x = hi + lo;
// hi.hi + hi.lo + lo.hi products, fp32 accumulation): the state keeps fp32 accuracy (2e-7 of its scale per step against
// float64). The state arrives as four TMA boxes [128 rows x 32 columns] with the 128-byte swizzle, which IS the K-major
// operand layout; its remainder lives in tensor memory (the A operand of the lo.hi product); the vectors are one 32-row
// K-major swizzled tile, U' and K^T 128 x 8 K-major tiles without swizzle. (An MN-major view of the vector tile as the
// update's B operand gave wrong products with 32-bit elements: K^T is stored explicitly instead.)
constexpr int kGdnD = 128;
constexpr int kGdnRows = 8;    // most rows one CTA walks: replayed (<= Tmax) + new (<= Tmax), Tmax <= 4
constexpr int kGdnThreads = 256;
// what the prep kernel leaves per (sequence, key head) and per (sequence, value head), in the state kernel's smem layout
constexpr uint32_t kGdnXBytes = 16384;   // vectors: 4 panels of [32 rows][128 bytes]: rows 0-7 k, 8-15 q, 16-31 remainders
constexpr uint32_t kGdnKtBytes = 8192;   // K^T head | remainder: [16 groups of 8 rows j][2 K chunks][8 rows][16 bytes] each
constexpr uint32_t kGdnGramBytes = 512;  // kk [8][8], kq [8][8] (no decays)
constexpr uint32_t kGdnKeyBlock = kGdnXBytes + kGdnKtBytes + kGdnGramBytes;
constexpr uint32_t kGdnValBlock = 4096 + 64;  // v [8][128] fp32 (conv outputs), decay [8], beta [8]
// shared memory of the state kernel
constexpr uint32_t kGdnS = 0;                             // state: 4 boxes of [128 rows][128 bytes], swizzled; head part in place
constexpr uint32_t kGdnKey = 65536;                       // the key block as the prep kernel wrote it
constexpr uint32_t kGdnVal = kGdnKey + kGdnKeyBlock;      // the value block; v rows turn into the rows' outputs
constexpr uint32_t kGdnU = kGdnVal + kGdnValBlock + 64;   // U' head | remainder, same layout as K^T (1024-byte aligned not needed)
constexpr uint32_t kGdnRed = kGdnU + 8192;                // [8][8 warps] sum o^2
constexpr uint32_t kGdnTab = kGdnRed + 256;               // gcum [8], urat [8], wkk [8][8], wkq [8][8]
constexpr uint32_t kGdnBar = kGdnTab + 1024;
constexpr uint32_t kGdnSmem = kGdnBar + 64 + 1024;        // + alignment slack
constexpr uint32_t kGdnTmemCols = 256;                    // [0, 128): the state's remainder; [128, 256): P (32 columns), then D
static_assert(kGdnU % 16 == 0 && kGdnVal % 16 == 0 && kGdnKeyBlock % 16 == 0 && kGdnValBlock % 16 == 0, "bulk copy alignment");

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// A operand in tensor memory: lanes = the 128 rows, one 32-bit column per K element
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void gdn_tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void gdn_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// x = hi + lo with hi a tf32 value (10 mantissa bits, rounded to nearest) and lo the exact remainder
__device__ __forceinline__ void tf32_split(float x, float& hi, float& lo) {
  hi = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
  lo = x - hi;
}
__device__ __forceinline__ void tf32_split4(const float4& v, float4& h, float4& l) {
  tf32_split(v.x, h.x, l.x); tf32_split(v.y, h.y, l.y); tf32_split(v.z, h.z, l.z); tf32_split(v.w, h.w, l.w);
}

// CTAs (x, sequence b) of 128 threads. x < Hk: key head x — thread c runs channel c of q and of k through the conv, then the
// norms, the table and the operand images. x >= Hk: value head x - Hk — thread c runs channel c of v; the gates.
// The heavier key-head CTAs have the lower block indices and start first.
constexpr int kGdnPrepThreads = 128;
__global__ void __launch_bounds__(kGdnPrepThreads, 4) ds_gdn_prep_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ conv_w,
                                                                         const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                                                         float* __restrict__ conv_rec, float* __restrict__ ab_rec,
                                                                         const int* __restrict__ slots, const int* __restrict__ ctx,
                                                                         const int* __restrict__ parity, const int* __restrict__ ncommit, int T, int Tmax,
                                                                         int Hk, int Hv, float l2_eps, uint8_t* __restrict__ key_blocks,
                                                                         uint8_t* __restrict__ val_blocks) {
  constexpr int D = kGdnD, RM = kGdnRows;
  __shared__ __align__(16) float qk[2][RM][D];  // normalised q, k
  __shared__ float red[2][RM][4];
  __shared__ float nrm[2][RM];
  grid_dependency_trigger();
  grid_dependency_wait();
  const int b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (ctx[b] < 0) return;
  const int slot = slots[b], par = parity[b] & 1, nc = min(ncommit[b], Tmax);
  const int C = 2 * Hk * D + Hv * D;
  const size_t rec_rows = 3 + Tmax;
  const float* rin = conv_rec + ((size_t)slot * 2 + par) * rec_rows * C;
  float* rout = conv_rec + ((size_t)slot * 2 + (par ^ 1)) * rec_rows * C;
  const int total = min(nc + T, RM);

  // the raw inputs of a channel: the window and every row; stores the new block's record ([the three conv inputs before it |
  // its own conv inputs] = inputs nc .. nc + 2 + T) as the values arrive
  auto load_channel = [&](int ch, float (&in)[3 + RM]) {
#pragma unroll
    for (int j = 0; j < 3 + RM; ++j) {
      const int r = j - 3;
      float a = 0.f;
      if (j < 3 + total) a = r < nc ? rin[(size_t)j * C + ch] : proj[(size_t)(b * T + (r - nc)) * ld + ch];
      in[j] = a;
    }
  };
  // (a loop of its own: a store between two loads would order them, the record being one array, and the 11 loads of a
  // channel would become 11 round trips to memory)
  auto store_record = [&](int ch, const float (&in)[3 + RM]) {
#pragma unroll
    for (int j = 0; j < 3 + RM; ++j)
      if (j < 3 + total && j >= nc) rout[(size_t)(j - nc) * C + ch] = in[j];
  };
  auto conv_silu = [&](int ch, const float (&in)[3 + RM], float (&y)[RM]) {
    const float4 w = *(const float4*)(conv_w + (size_t)ch * 4);
#pragma unroll
    for (int r = 0; r < RM; ++r) {
      const float c = in[r] * w.x + in[r + 1] * w.y + in[r + 2] * w.z + in[r + 3] * w.w;
      y[r] = c / (1.f + __expf(-c));
    }
  };

  if ((int)blockIdx.x >= Hk) {  // ---- a value head: conv outputs of v, the gates
    const int hv = blockIdx.x - Hk;
    const int ch = 2 * Hk * D + hv * D + tid;
    float gate_a = 0.f, gate_b = 0.f;
    if (tid < total) {
      if (tid < nc) {
        const float* abin = ab_rec + ((size_t)slot * 2 + par) * Tmax * 2 * Hv;
        gate_a = abin[(size_t)tid * 2 * Hv + hv]; gate_b = abin[(size_t)tid * 2 * Hv + Hv + hv];
      } else {
        const float* x = proj + (size_t)(b * T + (tid - nc)) * ld;
        gate_b = x[C + Hv * D + hv]; gate_a = x[C + Hv * D + Hv + hv];
      }
    }
    float in[3 + RM], y[RM];
    load_channel(ch, in);
    store_record(ch, in);
    conv_silu(ch, in, y);
    float* vb = (float*)(val_blocks + ((size_t)b * Hv + hv) * kGdnValBlock);
#pragma unroll
    for (int r = 0; r < RM; ++r) vb[r * D + tid] = y[r];
    if (tid < RM) {
      float decay = 1.f, beta = 0.f;
      if (tid < total) {
        if (tid >= nc) {
          float* about = ab_rec + ((size_t)slot * 2 + (par ^ 1)) * Tmax * 2 * Hv;
          about[(size_t)(tid - nc) * 2 * Hv + hv] = gate_a; about[(size_t)(tid - nc) * 2 * Hv + Hv + hv] = gate_b;
        }
        const float ax = gate_a + dt_bias[hv];
        const float sp = ax > 20.f ? ax : log1pf(__expf(ax));
        decay = __expf(-__expf(A_log[hv]) * sp);
        beta = 1.f / (1.f + __expf(-gate_b));
      }
      vb[RM * D + tid] = decay;
      vb[RM * D + RM + tid] = beta;
    }
    return;
  }

  // ---- a key head
  const int hk = blockIdx.x;
  uint8_t* kb = key_blocks + ((size_t)b * Hk + hk) * kGdnKeyBlock;
  {
    const int ch_q = hk * D + tid, ch_k = Hk * D + hk * D + tid;
    float inq[3 + RM], ink[3 + RM], yq[RM], yk[RM];
    load_channel(ch_q, inq);
    load_channel(ch_k, ink);
    store_record(ch_q, inq);
    store_record(ch_k, ink);
    conv_silu(ch_q, inq, yq);
    conv_silu(ch_k, ink, yk);
#pragma unroll
    for (int r = 0; r < RM; ++r) {
      const float sq = warp_sum(yq[r] * yq[r]), sk = warp_sum(yk[r] * yk[r]);
      if (lane == 0) { red[0][r][warp] = sq; red[1][r][warp] = sk; }
    }
    __syncthreads();
    if (tid < 2 * RM) {
      const int wh = tid >> 3, r = tid & 7;
      const float s = red[wh][r][0] + red[wh][r][1] + red[wh][r][2] + red[wh][r][3];
      nrm[wh][r] = wh == 0 ? rsqrtf(s + l2_eps) * rsqrtf((float)D) : rsqrtf(s + l2_eps);
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < RM; ++r) {
      qk[0][r][tid] = r < total ? yq[r] * nrm[0][r] : 0.f;
      qk[1][r][tid] = r < total ? yk[r] * nrm[1][r] : 0.f;
    }
  }
  __syncthreads();
  // the table (no decays: those belong to the value head)
  float* gram = (float*)(kb + kGdnXBytes + kGdnKtBytes);
  for (int e = warp; e < 2 * RM * RM; e += kGdnPrepThreads / 32) {
    const int tau = (e & 63) >> 3, t = e & 7;
    const bool isq = e >= 64;
    const bool valid = tau < total && t < total && (isq ? (tau <= t && t >= nc) : (tau < t));  // the same in the whole warp
    float d = 0.f;
    if (valid) {
      const float4 a = ((const float4*)qk[1][tau])[lane];
      const float4 c = ((const float4*)qk[isq ? 0 : 1][t])[lane];
      d = warp_sum(a.x * c.x + a.y * c.y + a.z * c.z + a.w * c.w);
    }
    if (lane == 0) gram[e] = d;
  }
  // the vectors as the K-major operand tile (heads in rows 0-15, remainders in rows 16-31)
  for (int task = tid; task < 16 * 32; task += kGdnPrepThreads) {
    const int n = task >> 5, c = task & 31;  // vector n (0-7: k of row n, 8-15: q of row n - 8), 16-byte chunk c of its 32
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (n < RM) v = ((const float4*)qk[1][n])[c];
    else if (n - RM >= nc) v = ((const float4*)qk[0][n - RM])[c];
    float4 h, l;
    tf32_split4(v, h, l);
    uint8_t* dst = kb + (c >> 3) * 4096 + n * 128 + (((c & 7) ^ (n & 7)) << 4);
    *(float4*)dst = h;
    *(float4*)(dst + 2048) = l;  // rows 16 + n
  }
  // K^T of the committed rows: thread j, four rows tau at a time -> one 16-byte chunk of the head and of the remainder
#pragma unroll
  for (int kc = 0; kc < 2; ++kc) {
    const int j = tid;
    float4 v = make_float4(qk[1][4 * kc][j], qk[1][4 * kc + 1][j], qk[1][4 * kc + 2][j], qk[1][4 * kc + 3][j]);
    if (4 * kc >= nc) v.x = 0.f;
    if (4 * kc + 1 >= nc) v.y = 0.f;
    if (4 * kc + 2 >= nc) v.z = 0.f;
    if (4 * kc + 3 >= nc) v.w = 0.f;
    float4 h, l;
    tf32_split4(v, h, l);
    uint8_t* kt = kb + kGdnXBytes + (j >> 3) * 256 + kc * 128 + (j & 7) * 16;
    *(float4*)kt = h;
    *(float4*)(kt + 4096) = l;
  }
}

// CTA (value head hv, sequence b), 256 threads, two CTAs per SM.
__global__ void __launch_bounds__(kGdnThreads, 2) ds_gdn_state_kernel(const __grid_constant__ CUtensorMap map_s, const float* __restrict__ proj, int ld,
                                                                      const float* __restrict__ norm_w, const int* __restrict__ slots,
                                                                      const int* __restrict__ ctx, const int* __restrict__ ncommit, int T, int Tmax, int Hk,
                                                                      int Hv, float rms_eps, const uint8_t* __restrict__ key_blocks,
                                                                      const uint8_t* __restrict__ val_blocks, __nv_bfloat16* __restrict__ out, int* status) {
  constexpr int D = kGdnD, RM = kGdnRows, NW = kGdnThreads / 32;
  extern __shared__ __align__(1024) uint8_t gdn_smem_raw[];
  uint8_t* sm = (uint8_t*)(((uintptr_t)gdn_smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* Ssm = sm + kGdnS;
  uint8_t* Xsm = sm + kGdnKey;
  uint8_t* Ktsm = Xsm + kGdnXBytes;
  const float* gram = (const float*)(Ktsm + kGdnKtBytes);
  float* cvs = (float*)(sm + kGdnVal);      // [8][128]: v, then the rows' outputs
  const float* dec = cvs + RM * D;          // [8] decays, [8] betas
  uint8_t* Usm = sm + kGdnU;
  float* red = (float*)(sm + kGdnRed);
  float* gcum = (float*)(sm + kGdnTab);     // [RM]: g_0 .. g_t
  float* urat = gcum + RM;                  // [RM]: g_{tau+1} .. g_{nc-1}
  float* wkk = urat + RM;                   // [RM][RM]: (G_t / G_tau) k_tau . k_t, tau < t
  float* wkq = wkk + RM * RM;               // [RM][RM]: (G_t / G_tau) k_tau . q_t, tau <= t, t >= nc
  uint64_t* bar = (uint64_t*)(sm + kGdnBar);  // [0]: state loaded; [1]: MMAs done (two phases); [2]: the prep kernel's blocks loaded
  uint32_t* tmem_slot = (uint32_t*)(bar + 3);
  const int hv = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qd = warp & 3, hh = warp >> 2;  // row 32 qd + lane (the TMEM lanes this warp may touch), columns 64 hh .. + 63
  const int srow = qd * 32 + lane;
  if (ctx[b] < 0) {
    grid_dependency_wait();  // every block waits before it leaves: the grid must not complete ahead of the kernels before it
    return;
  }
  const int slot = slots[b], nc = min(ncommit[b], Tmax);
  const int hk = hv / (Hv / Hk);
  const int total = min(nc + T, RM);
  const int srow0 = (slot * Hv + hv) * D;  // first row of this head in the [slots * Hv * 128, 128] view of the state
  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    mbar_init(&bar[2], 1);
    mbar_fence_init();
    mbar_expect_tx(&bar[0], D * D * 4);
    for (int p = 0; p < 4; ++p) tma_load_2d(Ssm + p * 16384, &map_s, p * 32, srow0, &bar[0]);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kGdnTmemCols);
    tmem_relinquish();
  }
  // Up to here the kernel read only what no kernel of this step writes before it (the sequence's slot and context, this
  // layer's state): the state streams in while the kernels ahead in the stream (projection GEMM, prep) run.
  grid_dependency_trigger();
  grid_dependency_wait();
  if (tid == 0) {
    mbar_expect_tx(&bar[2], kGdnKeyBlock + kGdnValBlock);
    bulk_load_1d(Xsm, key_blocks + ((size_t)b * Hk + hk) * kGdnKeyBlock, kGdnKeyBlock, &bar[2]);
    bulk_load_1d(cvs, val_blocks + ((size_t)b * Hv + hv) * kGdnValBlock, kGdnValBlock, &bar[2]);
  }
  // the output gate of the new rows and the norm weight: the kernel's only other global loads, issued before any wait
  const int row = tid >> 1, half = tid & 1;  // the output norm: a pair of threads per channel (one publishes)
  float zz[4] = {0.f, 0.f, 0.f, 0.f};
  {
    const int C = 2 * Hk * D + Hv * D;
#pragma unroll
    for (int t = 0; t < 4; ++t)
      if (t < T && half == 0) zz[t] = proj[(size_t)(b * T + t) * ld + C + hv * D + row];
  }
  const float nw = norm_w[row];
  __syncthreads();  // the mbarriers' initialisation and the TMEM address are visible to every thread
  const uint32_t tmem = *tmem_slot;
  bool ok = mbar_wait_bounded(&bar[2], 0, status);

  // ---- (1) the table with the decays between the two rows folded in
  if (ok && tid < 2 * RM * RM) {
    const int tau = (tid & 63) >> 3, t = tid & 7;
    float d = gram[tid];
    for (int s = tau + 1; s <= t; ++s) d *= dec[s];
    (tid >= 64 ? wkq : wkk)[tau * RM + t] = d;
  } else if (ok && tid < 2 * RM * RM + RM) {
    const int r = tid - 2 * RM * RM;
    float g = 1.f, u = 1.f;
    for (int s = 0; s <= r && s < total; ++s) g *= dec[s];
    for (int s = r + 1; s < nc; ++s) u *= dec[s];
    gcum[r] = g;
    urat[r] = r < nc ? u : 0.f;
  }

  // ---- (2) the state: head part in place (the A operand in shared memory), remainder into tensor memory
  if (ok) ok = mbar_wait_bounded(&bar[0], 0, status);
  ok = __syncthreads_and(ok ? 1 : 0) != 0;
  if (!ok) {  // the whole CTA leaves together
    if (warp == 1) tmem_dealloc(tmem, kGdnTmemCols);
    return;
  }
  const uint32_t lane_base = tmem + ((uint32_t)(qd * 32) << 16);
  const int sx = srow & 7;
#pragma unroll 1
  for (int pp = 0; pp < 2; ++pp) {
    const int p = 2 * hh + pp;
    uint8_t* base = Ssm + p * 16384 + srow * 128;
    uint32_t lo[32];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float4* ptr = (float4*)(base + ((c ^ sx) << 4));
      float4 h, l;
      tf32_split4(*ptr, h, l);
      *ptr = h;
      lo[4 * c] = __float_as_uint(l.x); lo[4 * c + 1] = __float_as_uint(l.y); lo[4 * c + 2] = __float_as_uint(l.z); lo[4 * c + 3] = __float_as_uint(l.w);
    }
    gdn_tmem_st_x32(lane_base + p * 32, lo);
  }
  gdn_wait_st();
  fence_proxy_async();
  tcgen05_fence_before();
  __syncthreads();
  if (tid == 0) {
    tcgen05_fence_after();
    constexpr uint32_t idesc_p = umma_idesc_f16(128, 32, 2), idesc_l = umma_idesc_f16(128, 16, 2);
    const uint32_t s_addr = smem_u32(Ssm), x_addr = smem_u32(Xsm);
#pragma unroll
    for (int kk = 0; kk < 16; ++kk)  // hi . [vector heads | vector remainders]: 32 columns
      umma_tf32(tmem + 128, umma_desc_sw128(s_addr + (kk >> 2) * 16384) + (uint64_t)((kk & 3) * 2),
                umma_desc_sw128(x_addr + (kk >> 2) * 4096) + (uint64_t)((kk & 3) * 2), idesc_p, kk != 0 ? 1u : 0u);
#pragma unroll
    for (int kk = 0; kk < 16; ++kk)  // lo . vector heads, onto the first 16 columns
      umma_tf32_ts(tmem + 128, tmem + kk * 8, umma_desc_sw128(x_addr + (kk >> 2) * 4096) + (uint64_t)((kk & 3) * 2), idesc_l, 1u);
    tcgen05_commit(&bar[1]);
  }
  ok = mbar_wait_bounded(&bar[1], 0, status);
  ok = __syncthreads_and(ok ? 1 : 0) != 0;
  if (!ok) {
    if (warp == 1) tmem_dealloc(tmem, kGdnTmemCols);
    return;
  }
  tcgen05_fence_after();

  // ---- (3) a thread per state row walks the rows on scalars
  if (hh == 0) {
    uint32_t pr[32];
    tmem_ld_32x32b_x32(lane_base + 128, pr);
    tcgen05_wait_ld();
    float u[RM];
#pragma unroll
    for (int t = 0; t < RM; ++t) {
      u[t] = 0.f;
      if (t < total) {
        float a = gcum[t] * (__uint_as_float(pr[t]) + __uint_as_float(pr[16 + t]));
#pragma unroll
        for (int tau = 0; tau < t; ++tau) a += u[tau] * wkk[tau * RM + t];
        u[t] = dec[RM + t] * (cvs[t * D + srow] - a);
        if (t >= nc) {
          float o = gcum[t] * (__uint_as_float(pr[8 + t]) + __uint_as_float(pr[24 + t]));
#pragma unroll
          for (int tau = 0; tau <= t; ++tau) o += u[tau] * wkq[tau * RM + t];
          cvs[t * D + srow] = o;  // the row's output
        }
      }
    }
    float4 h0, h1, l0, l1;
    tf32_split4(make_float4(u[0] * urat[0], u[1] * urat[1], u[2] * urat[2], u[3] * urat[3]), h0, l0);
    tf32_split4(make_float4(u[4] * urat[4], u[5] * urat[5], u[6] * urat[6], u[7] * urat[7]), h1, l1);
    uint8_t* ub = Usm + (srow >> 3) * 256 + (srow & 7) * 16;
    *(float4*)ub = h0; *(float4*)(ub + 128) = h1;
    *(float4*)(ub + 4096) = l0; *(float4*)(ub + 4096 + 128) = l1;
    fence_proxy_async();
  }
  tcgen05_fence_before();
  __syncthreads();
  if (nc > 0) {  // the same in the whole CTA
    if (tid == 0) {
      tcgen05_fence_after();
      constexpr uint32_t idesc_u = umma_idesc_f16(128, 128, 2);
      const uint64_t ua = umma_desc_interleaved(smem_u32(Usm), 128, 256), ul = umma_desc_interleaved(smem_u32(Usm + 4096), 128, 256);
      const uint64_t kh = umma_desc_interleaved(smem_u32(Ktsm), 128, 256), kl = umma_desc_interleaved(smem_u32(Ktsm + 4096), 128, 256);
      umma_tf32(tmem + 128, ua, kh, idesc_u, 0u);
      umma_tf32(tmem + 128, ul, kh, idesc_u, 1u);
      umma_tf32(tmem + 128, ua, kl, idesc_u, 1u);
      tcgen05_commit(&bar[1]);
    }
    ok = mbar_wait_bounded(&bar[1], 1, status);
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    if (!ok) {
      if (warp == 1) tmem_dealloc(tmem, kGdnTmemCols);
      return;
    }
    tcgen05_fence_after();
    // the stored state: G (hi + lo) + D, written over the head part and sent back by TMA (the only state write of the step)
    const float G = gcum[nc - 1];
#pragma unroll 1
    for (int pp = 0; pp < 2; ++pp) {
      const int p = 2 * hh + pp;
      uint8_t* base = Ssm + p * 16384 + srow * 128;
      uint32_t dd[32], lo[32];
      tmem_ld_32x32b_x32(lane_base + 128 + p * 32, dd);
      tmem_ld_32x32b_x32(lane_base + p * 32, lo);
      tcgen05_wait_ld();
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float4* ptr = (float4*)(base + ((c ^ sx) << 4));
        float4 v = *ptr;
        v.x = G * (v.x + __uint_as_float(lo[4 * c])) + __uint_as_float(dd[4 * c]);
        v.y = G * (v.y + __uint_as_float(lo[4 * c + 1])) + __uint_as_float(dd[4 * c + 1]);
        v.z = G * (v.z + __uint_as_float(lo[4 * c + 2])) + __uint_as_float(dd[4 * c + 2]);
        v.w = G * (v.w + __uint_as_float(lo[4 * c + 3])) + __uint_as_float(dd[4 * c + 3]);
        *ptr = v;
      }
    }
    fence_proxy_async();
    tcgen05_fence_before();
    __syncthreads();
    if (tid == 0) {
      for (int p = 0; p < 4; ++p)
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&map_s), "r"(p * 32), "r"(srow0),
                     "r"(smem_u32(Ssm + p * 16384))
                     : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
  }
  if (warp == 1) {  // every tensor-memory access of the CTA lies before the last barrier passed
    tcgen05_fence_after();
    tmem_dealloc(tmem, kGdnTmemCols);
  }

  // ---- (4) gated RMSNorm of the new rows' outputs
  const float mine = half == 0 ? 1.f : 0.f;  // a pair holds the same channel: only one of the two enters the sums
  for (int r = nc; r < total; ++r) {
    const float o = cvs[r * D + row] * mine;
    const float so = warp_sum(o * o);
    if (lane == 0) red[r * NW + warp] = so;
  }
  __syncthreads();
  if (half == 0) {
    for (int r = nc; r < total; ++r) {
      const int t = r - nc;
      float so = 0.f;
      for (int w8 = 0; w8 < NW; ++w8) so += red[r * NW + w8];
      const float z = t == 0 ? zz[0] : (t == 1 ? zz[1] : (t == 2 ? zz[2] : zz[3]));
      out[(size_t)(b * T + t) * Hv * D + hv * D + row] =
          __float2bfloat16_rn(cvs[r * D + row] * rsqrtf(so / (float)D + rms_eps) * nw * (z / (1.f + __expf(-z))));
    }
  }
  // the stores read shared memory asynchronously: they must have finished reading before the CTA's memory goes away
  if (tid == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// ------------------------------------------------------------------------------------------------ sharded verify sampler
// Rejection sampling of greedy drafts over a vocabulary that may be sharded over ranks (upstream verify_sampler.cu runs
// on gathered logits; here every rank reduces its own shard to small records and only the records travel).
// Row (b, t) holds the logits after input token t; its draft is the step's input token t + 1 (none for the last row).
// Per (row, chunk of the local shard): max, sum exp, the best exponential-race key with the draft excluded, the draft's
// own logit if it lives in the chunk, NaN / +inf count. The records are stored into slot [rank] of every rank's record
// buffer (plain peer stores); after the flag barrier one CTA per sequence merges ranks x chunks in a fixed order, walks
// the rows (accept while log p(draft) > log u), takes the first rejected row's winner (or the bonus row's) and writes the
// step's results AND the next step's inputs.
struct DsRec {
  float max, sumexp, best_key, best_z;
  int best_id, nonfinite;
  float draft_z;
  int pad;
};

__global__ void __launch_bounds__(256) ds_verify_chunks_kernel(const float* __restrict__ logits, int ld, int Vs, int v0, float inv_temp,
                                                               const int* __restrict__ tok_in, const int* __restrict__ ctx, int T, int chunks,
                                                               uint32_t seed, const uint32_t* __restrict__ step_ctr, DsPeers recs, int rank, int world,
                                                               const uint32_t* __restrict__ epoch_ctr, size_t rec_buf_elems) {
  grid_dependency_trigger();
  grid_dependency_wait();
  __shared__ float red[8 * 5];
  __shared__ int redi[8 * 2];
  const int chunk = blockIdx.x, row = blockIdx.y, b = row / T, t = row % T, tid = threadIdx.x;
  if (ctx[b] < 0) return;
  const int per = (((Vs + chunks - 1) / chunks) + 3) & ~3;
  const int lo = chunk * per, hi = min(Vs, lo + per);
  const int draft = (t + 1 < T) ? tok_in[b * T + t + 1] : -1;
  const uint32_t step = *step_ctr;
  const float* x = logits + (size_t)row * ld;
  float m = -FLT_MAX, bk = -FLT_MAX, bz = 0.f, dz = -FLT_MAX;
  int bid = -1, nf = 0;
  for (int i = lo + tid * 4; i < hi; i += 1024) {
    const uint4 rnd = ds_noise4(seed, step, (uint32_t)row, (uint32_t)((v0 + i) >> 2));
    const uint32_t rr[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (i + e < hi) {
        const float z = x[i + e] * inv_temp;
        if (isnan(z) || z == INFINITY) ++nf;
        m = fmaxf(m, z);
        const int id = v0 + i + e;
        if (id == draft) { dz = z; continue; }
        const float key = z - __logf(-__logf(ds_u01(rr[e])));
        if (key > bk) { bk = key; bid = id; bz = z; }
      }
    }
  }
  float wm = warp_max(m);
  if ((tid & 31) == 0) red[tid >> 5] = wm;
  __syncthreads();
  float cmax = -FLT_MAX;
  for (int k = 0; k < 8; ++k) cmax = fmaxf(cmax, red[k]);
  __syncthreads();
  float s = 0.f;
  for (int i = lo + tid; i < hi; i += 256) s += __expf(x[i] * inv_temp - cmax);
  s = warp_sum(s);
  nf = (int)warp_sum((float)nf);
  dz = warp_max(dz);
  for (int o = 16; o > 0; o >>= 1) {
    const float ok = __shfl_xor_sync(0xffffffffu, bk, o), oz = __shfl_xor_sync(0xffffffffu, bz, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bid, o);
    if (ok > bk || (ok == bk && oi >= 0 && (bid < 0 || oi < bid))) { bk = ok; bid = oi; bz = oz; }
  }
  if ((tid & 31) == 0) {
    const int w8 = tid >> 5;
    red[w8] = s; red[8 + w8] = bk; red[16 + w8] = bz; red[24 + w8] = (float)nf; red[32 + w8] = dz; redi[w8] = bid;
  }
  __syncthreads();
  if (tid == 0) {
    DsRec r;
    float ts = 0.f, k = -FLT_MAX, z = 0.f, d = -FLT_MAX;
    int id = -1, tn = 0;
    for (int w8 = 0; w8 < 8; ++w8) {
      ts += red[w8]; tn += (int)red[24 + w8]; d = fmaxf(d, red[32 + w8]);
      if (red[8 + w8] > k || (red[8 + w8] == k && redi[w8] >= 0 && (id < 0 || redi[w8] < id))) { k = red[8 + w8]; id = redi[w8]; z = red[16 + w8]; }
    }
    r.max = cmax; r.sumexp = ts; r.best_key = k; r.best_z = z; r.best_id = id; r.nonfinite = tn; r.draft_z = d; r.pad = 0;
    const size_t buf = epoch_ctr ? (size_t)((*epoch_ctr + 1u) & 1u) * rec_buf_elems : 0;
    const size_t idx = buf + ((size_t)rank * gridDim.y + row) * chunks + chunk;
    for (int p = 0; p < world; ++p) {
      const int peer = (rank + p) % world;
      uint4* dst = (uint4*)((DsRec*)recs.p[peer] + idx);
      const uint4* srcv = (const uint4*)&r;
      dst[0] = srcv[0]; dst[1] = srcv[1];
    }
    if (world > 1) __threadfence_system();
  }
}

// One CTA (32 threads) per sequence. Outputs of the step: out_tok [B][T] (-1 after the last emitted token), out_lp,
// n_accept [B], nonfinite [B]. Next step's inputs: tok_in[b][0] = the emitted token that follows the accepted drafts
// (the drafter fills tok_in[b][1..]), ctx += accepted + 1, ncommit = accepted + 1, parity ^= 1, sel_row[b] = the row
// whose hidden state feeds the drafter, mtp_tok [B][T] = the token after each row (drafter input of its first pass),
// mtp_ctx [T][B] = the context length of drafter pass k (pass 0 runs over the step's rows, pass k >= 1 over one new row).
// ------------------------------------------------------------------------------------------------ top-k log-probs
// The 32 largest scaled logits of every row with their token ids (what score centering reads from the sampler), over a
// vocabulary that may be sharded: a CTA per (row, chunk of the local shard) selects its chunk's top 32 and stores the list to
// every rank like the sampler's records; after the flag barrier one CTA per row merges ranks x chunks lists and turns them
// into log-probs with the row's log-sum-exp from the sampler's own records. Selection: a histogram of (chunk max - z) in
// 2048 bins of 1/32 finds the bin where the count reaches 32, the elements up to that bin are collected (at most 1024: when
// more than that lie within 1/32 of the 32nd value the surplus of that bin is cut in arrival order) and sorted in shared
// memory. (Upstream: rollout/blackwell/csrc/sampler.cu — top-32 log-probs beside the sampled token.)
constexpr int kTopK = 32, kTopBins = 2048, kTopCand = 1024;
struct DsTop {
  float z[kTopK];
  int id[kTopK];
};
__device__ __forceinline__ unsigned long long ds_top_key(float z, int id) {
  const uint32_t b = __float_as_uint(z);
  const uint32_t u = (b & 0x80000000u) ? ~b : (b | 0x80000000u);  // order-preserving
  return ((unsigned long long)u << 32) | (uint32_t)(0x7fffffff - id);  // equal values: the lower id first
}
__device__ __forceinline__ void ds_top_unkey(unsigned long long k, float& z, int& id) {
  const uint32_t u = (uint32_t)(k >> 32);
  z = __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
  id = 0x7fffffff - (int)(uint32_t)k;
}
// descending bitonic sort of n (a power of two, <= 1024) keys in shared memory by 256 threads
__device__ __forceinline__ void ds_sort_desc(unsigned long long* a, int n) {
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int l = i ^ j;
        if (l > i) {
          const unsigned long long x = a[i], y = a[l];
          const bool up = (i & k) != 0;  // ascending block of the bitonic network
          if (up ? (x > y) : (x < y)) { a[i] = y; a[l] = x; }
        }
      }
      __syncthreads();
    }
  }
}
__global__ void __launch_bounds__(256) ds_topk_chunks_kernel(const float* __restrict__ logits, int ld, int Vs, int v0, float inv_temp,
                                                             const int* __restrict__ ctx, int T, int chunks, DsPeers tops, int rank, int world,
                                                             const uint32_t* __restrict__ epoch_ctr, size_t buf_elems) {
  grid_dependency_trigger();
  grid_dependency_wait();
  __shared__ int hist[kTopBins];
  __shared__ unsigned long long cand[kTopCand];
  __shared__ int part[256];
  __shared__ float red[8];
  __shared__ int s_bin, s_count;
  const int chunk = blockIdx.x, row = blockIdx.y, b = row / T, tid = threadIdx.x;
  if (ctx[b] < 0) return;
  const int per = (((Vs + chunks - 1) / chunks) + 3) & ~3;
  const int lo = chunk * per, hi = min(Vs, lo + per);
  const float* x = logits + (size_t)row * ld;
  float m = -FLT_MAX;
  for (int i = lo + tid; i < hi; i += 256) {
    const float z = x[i] * inv_temp;
    if (z == z) m = fmaxf(m, z);
  }
  m = warp_max(m);
  if ((tid & 31) == 0) red[tid >> 5] = m;
  for (int i = tid; i < kTopBins; i += 256) hist[i] = 0;
  if (tid == 0) { s_count = 0; s_bin = kTopBins - 1; }
  __syncthreads();
  float cmax = -FLT_MAX;
  for (int k = 0; k < 8; ++k) cmax = fmaxf(cmax, red[k]);
  auto bin_of = [&](float z) {  // (a NaN or infinite distance lands in the last bin)
    const float d = (cmax - z) * 32.f;
    return d < (float)(kTopBins - 1) ? max(0, (int)d) : kTopBins - 1;
  };
  for (int i = lo + tid; i < hi; i += 256) {
    const float z = x[i] * inv_temp;
    if (z == z) atomicAdd(&hist[bin_of(z)], 1);
  }
  __syncthreads();
  int local = 0;
#pragma unroll
  for (int k = 0; k < kTopBins / 256; ++k) local += hist[tid * (kTopBins / 256) + k];
  part[tid] = local;
  __syncthreads();
  for (int o = 1; o < 256; o <<= 1) {  // inclusive scan
    const int v = tid >= o ? part[tid - o] : 0;
    __syncthreads();
    part[tid] += v;
    __syncthreads();
  }
  const int need = min(kTopK, part[255]);
  const int excl = part[tid] - local;
  if (need > 0 && excl < need && part[tid] >= need) {  // exactly one thread
    int c = excl;
    for (int k = 0; k < kTopBins / 256; ++k) {
      c += hist[tid * (kTopBins / 256) + k];
      if (c >= need) { s_bin = tid * (kTopBins / 256) + k; break; }
    }
  }
  __syncthreads();
  const int tb = s_bin;
  // first everything strictly above the threshold bin (fewer than 32 elements), then the threshold bin itself up to the cap
  for (int pass = 0; pass < 2; ++pass) {
    for (int i = lo + tid; i < hi; i += 256) {
      const float z = x[i] * inv_temp;
      if (!(z == z)) continue;
      const int bn = bin_of(z);
      if (pass == 0 ? bn < tb : bn == tb) {
        const int pos = atomicAdd(&s_count, 1);
        if (pos < kTopCand) cand[pos] = ds_top_key(z, v0 + i);
      }
    }
    __syncthreads();
  }
  const int n = min(s_count, kTopCand);
  int n2 = 64;
  while (n2 < n) n2 <<= 1;
  for (int i = n + tid; i < n2; i += 256) cand[i] = 0ull;  // below every real key
  __syncthreads();
  ds_sort_desc(cand, n2);
  if (tid < kTopK) {
    float z = -INFINITY;
    int id = -1;
    if (tid < n) ds_top_unkey(cand[tid], z, id);
    const size_t buf = epoch_ctr ? (size_t)((*epoch_ctr + 1u) & 1u) * buf_elems : 0;
    const size_t idx = buf + ((size_t)rank * gridDim.y + row) * chunks + chunk;
    for (int p = 0; p < world; ++p) {
      DsTop* dst = (DsTop*)tops.p[(rank + p) % world] + idx;
      dst->z[tid] = z;
      dst->id[tid] = id;
    }
    if (world > 1) __threadfence_system();
  }
}

// One CTA per row: merge world x chunks sorted lists, log-probs against the row's log-sum-exp (from the sampler's records).
__global__ void __launch_bounds__(256) ds_topk_finish_kernel(const DsTop* __restrict__ tops, size_t top_buf_elems, const DsRec* __restrict__ recs,
                                                             size_t rec_buf_elems, const uint32_t* __restrict__ epoch_ctr, int world, int chunks,
                                                             int rows, const int* __restrict__ ctx, int T, int* __restrict__ out_id,
                                                             float* __restrict__ out_lp) {
  grid_dependency_trigger();
  grid_dependency_wait();
  __shared__ unsigned long long keys[kTopCand];
  __shared__ float s_lse;
  const int row = blockIdx.x, tid = threadIdx.x;
  if (ctx[row / T] < 0) return;
  // (launched after the flag barrier, which has advanced the epoch: the lists and records of this step sit in buffer epoch & 1;
  // the chunk kernels, launched before it, wrote buffer (epoch + 1) & 1 of the value they saw)
  const size_t tbuf = epoch_ctr ? (size_t)((*epoch_ctr) & 1u) * top_buf_elems : 0;
  const size_t rbuf = epoch_ctr ? (size_t)((*epoch_ctr) & 1u) * rec_buf_elems : 0;
  const int lists = world * chunks, total = lists * kTopK;
  int n2 = 64;
  while (n2 < total) n2 <<= 1;
  for (int i = tid; i < n2; i += 256) {
    unsigned long long k = 0ull;
    if (i < total) {
      const int l = i / kTopK, e = i % kTopK, r = l / chunks, c = l % chunks;
      const DsTop* t = tops + tbuf + ((size_t)r * rows + row) * chunks + c;
      if (t->id[e] >= 0) k = ds_top_key(t->z[e], t->id[e]);
    }
    keys[i] = k;
  }
  if (tid == 0) {
    float gm = -FLT_MAX;
    for (int l = 0; l < lists; ++l) gm = fmaxf(gm, recs[rbuf + ((size_t)(l / chunks) * rows + row) * chunks + (l % chunks)].max);
    float sum = 0.f;
    for (int l = 0; l < lists; ++l) {
      const DsRec& r = recs[rbuf + ((size_t)(l / chunks) * rows + row) * chunks + (l % chunks)];
      sum += r.sumexp * __expf(r.max - gm);
    }
    s_lse = gm + __logf(sum);
  }
  __syncthreads();
  ds_sort_desc(keys, n2);
  if (tid < kTopK) {
    float z = -INFINITY;
    int id = -1;
    if (keys[tid] != 0ull) ds_top_unkey(keys[tid], z, id);
    out_id[(size_t)row * kTopK + tid] = id;
    out_lp[(size_t)row * kTopK + tid] = id >= 0 ? z - s_lse : -INFINITY;
  }
}

__global__ void ds_verify_finish_kernel(const DsRec* __restrict__ recs, size_t rec_buf_elems, const uint32_t* __restrict__ epoch_ctr, int world,
                                        int chunks, int rows_total, int T, uint32_t seed, uint32_t* __restrict__ step_ctr, int* __restrict__ tok_in,
                                        int* __restrict__ ctx, int* __restrict__ ncommit, int* __restrict__ parity, int* __restrict__ out_tok,
                                        float* __restrict__ out_lp, int* __restrict__ n_accept, int* __restrict__ nonfinite,
                                        int* __restrict__ sel_row, int* __restrict__ mtp_tok, int* __restrict__ mtp_ctx, int B) {
  grid_dependency_trigger();
  grid_dependency_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t step = *step_ctr;
  if (b < B && ctx[b] >= 0) {
    const DsRec* base = recs + (epoch_ctr ? (size_t)((*epoch_ctr) & 1u) * rec_buf_elems : 0);
    int acc = 0, nf = 0;
    bool stopped = false;
    for (int t = 0; t < T; ++t) {
      const int row = b * T + t;
      float m = -FLT_MAX;
      for (int r = 0; r < world; ++r)
        for (int c = 0; c < chunks; ++c) m = fmaxf(m, base[((size_t)r * rows_total + row) * chunks + c].max);
      float s = 0.f, bk = -FLT_MAX, bz = 0.f, dz = -FLT_MAX;
      int bid = -1;
      for (int r = 0; r < world; ++r)
        for (int c = 0; c < chunks; ++c) {
          const DsRec& e = base[((size_t)r * rows_total + row) * chunks + c];
          s += e.sumexp * __expf(e.max - m);
          nf += e.nonfinite;
          dz = fmaxf(dz, e.draft_z);
          if (e.best_key > bk || (e.best_key == bk && e.best_id >= 0 && (bid < 0 || e.best_id < bid))) { bk = e.best_key; bid = e.best_id; bz = e.best_z; }
        }
      const float lse = m + __logf(s);
      if (stopped) { out_tok[row] = -1; out_lp[row] = 0.f; mtp_tok[row] = 0; continue; }
      const int draft = (t + 1 < T) ? tok_in[row + 1] : -1;
      bool accept = false;
      if (draft >= 0) {
        const float lp = dz - lse;
        accept = lp > __logf(fmaxf(ds_accept_u(seed, step, (uint32_t)row), 1e-30f));
        if (accept) { out_tok[row] = draft; out_lp[row] = lp; mtp_tok[row] = draft; ++acc; }
      }
      if (!accept) {
        out_tok[row] = bid; out_lp[row] = bz - lse; mtp_tok[row] = bid;
        stopped = true;
      }
    }
    const int c0 = ctx[b];
    mtp_ctx[b] = c0;
    for (int k = 1; k < T; ++k) mtp_ctx[(size_t)k * B + b] = c0 + acc + k;
    n_accept[b] = acc; nonfinite[b] = nf;
    sel_row[b] = b * T + acc;
    tok_in[b * T] = out_tok[b * T + acc];
    ctx[b] = c0 + acc + 1;
    ncommit[b] = acc + 1;
    parity[b] ^= 1;
  } else if (b < B) {
    n_accept[b] = 0; nonfinite[b] = 0; sel_row[b] = b * T;
    for (int k = 0; k < T; ++k) mtp_ctx[(size_t)k * B + b] = -1;
    for (int t = 0; t < T; ++t) { out_tok[b * T + t] = -1; out_lp[b * T + t] = 0.f; mtp_tok[b * T + t] = 0; }
  }
}

// the step counter moves in a launch of its own: every CTA of the finish kernel has read it by then
__global__ void ds_bump_kernel(uint32_t* ctr) {
  grid_dependency_trigger();
  grid_dependency_wait();
  if (threadIdx.x == 0 && blockIdx.x == 0) *ctr += 1u;
}

// ------------------------------------------------------------------------------------------------ drafter input rows
// out bf16 [row][2H] = [ rmsnorm_e(embed[token[row]]) | rmsnorm_h(hidden[src_row(row)]) ], both (1 + w).
// src_row: sel (may be null -> identity) maps the output row to the row of `hidden`.
__global__ void __launch_bounds__(256) ds_mtp_input_kernel(const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ table, int V,
                                                           const float* __restrict__ hidden, const int* __restrict__ sel,
                                                           const float* __restrict__ we, const float* __restrict__ wh, int H, float eps,
                                                           __nv_bfloat16* __restrict__ out) {
  grid_dependency_trigger();
  grid_dependency_wait();
  __shared__ float red[16];
  const int row = blockIdx.x, tid = threadIdx.x;
  const int id = min(max(tokens[row], 0), V - 1);
  const __nv_bfloat16* e = table + (size_t)id * H;
  const float* h = hidden + (size_t)(sel ? sel[row] : row) * H;
  float se = 0.f, sh = 0.f;
  for (int i = tid; i < H; i += 256) {
    const float a = __bfloat162float(e[i]), c = h[i];
    se += a * a; sh += c * c;
  }
  se = warp_sum(se); sh = warp_sum(sh);
  if ((tid & 31) == 0) { red[tid >> 5] = se; red[8 + (tid >> 5)] = sh; }
  __syncthreads();
  se = 0.f; sh = 0.f;
  for (int k = 0; k < 8; ++k) { se += red[k]; sh += red[8 + k]; }
  const float re = rsqrtf(se / (float)H + eps), rh = rsqrtf(sh / (float)H + eps);
  __nv_bfloat16* o = out + (size_t)row * 2 * H;
  for (int i = tid; i < H; i += 256) {
    o[i] = __float2bfloat16_rn(__bfloat162float(e[i]) * re * (1.f + we[i]));
    o[H + i] = __float2bfloat16_rn(h[i] * rh * (1.f + wh[i]));
  }
}

// rows of fp32 [*, H] gathered through `sel` (the drafter's hidden state of the accepted row)
__global__ void ds_gather_rows_kernel(const float* __restrict__ src, const int* __restrict__ sel, float* __restrict__ dst, int H) {
  grid_dependency_trigger();
  grid_dependency_wait();
  const int row = blockIdx.x;
  const float4* s = (const float4*)(src + (size_t)sel[row] * H);
  float4* d = (float4*)(dst + (size_t)row * H);
  for (int i = threadIdx.x; i < H / 4; i += blockDim.x) d[i] = s[i];
}

// ------------------------------------------------------------------------------------------------ draft argmax
// Greedy token of the drafter over a vocabulary shard: chunk records (ordered 64-bit key: monotone float bits << 32 |
// ~token id, so ties go to the lower id) stored into every rank's buffer, then a per-row maximum over ranks x chunks.
__global__ void __launch_bounds__(256) ds_argmax_chunks_kernel(const float* __restrict__ logits, int ld, int Vs, int v0, int chunks, DsPeers keys,
                                                               int rank, int world, const uint32_t* __restrict__ epoch_ctr, size_t buf_elems) {
  grid_dependency_trigger();
  grid_dependency_wait();
  __shared__ unsigned long long red[8];
  const int chunk = blockIdx.x, row = blockIdx.y, tid = threadIdx.x;
  const int per = (Vs + chunks - 1) / chunks, lo = chunk * per, hi = min(Vs, lo + per);
  const float* x = logits + (size_t)row * ld;
  unsigned long long best = 0ull;
  for (int i = lo + tid; i < hi; i += 256) {
    uint32_t bits = __float_as_uint(x[i]);
    bits = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
    const unsigned long long key = ((unsigned long long)bits << 32) | (uint32_t)~(uint32_t)(v0 + i);
    best = key > best ? key : best;
  }
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((tid & 31) == 0) red[tid >> 5] = best;
  __syncthreads();
  if (tid == 0) {
    for (int k = 1; k < 8; ++k) best = red[k] > best ? red[k] : best;
    const size_t buf = epoch_ctr ? (size_t)((*epoch_ctr + 1u) & 1u) * buf_elems : 0;
    const size_t idx = buf + ((size_t)rank * gridDim.y + row) * chunks + chunk;
    for (int p = 0; p < world; ++p) ((unsigned long long*)keys.p[(rank + p) % world])[idx] = best;
    if (world > 1) __threadfence_system();
  }
}

// token of each row -> dst[row * dst_stride + dst_off] (the next draft slot of the step's input tokens) and `tok_out`
__global__ void ds_argmax_finish_kernel(const unsigned long long* __restrict__ keys, size_t buf_elems, const uint32_t* __restrict__ epoch_ctr,
                                        int world, int chunks, int rows, int* __restrict__ dst, int dst_stride, int dst_off,
                                        int* __restrict__ tok_out) {
  grid_dependency_trigger();
  grid_dependency_wait();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  const unsigned long long* base = keys + (epoch_ctr ? (size_t)((*epoch_ctr) & 1u) * buf_elems : 0);
  unsigned long long best = 0ull;
  for (int r = 0; r < world; ++r)
    for (int c = 0; c < chunks; ++c) {
      const unsigned long long k = base[((size_t)r * rows + row) * chunks + c];
      best = k > best ? k : best;
    }
  const int tok = (int)~(uint32_t)best;
  dst[(size_t)row * dst_stride + dst_off] = tok;
  if (tok_out) tok_out[row] = tok;
}

// ------------------------------------------------------------------------------------------------ device-epoch barrier
// All ranks' streams meet. The epoch lives in a device counter (so a captured graph can replay it): flag value
// *ctr + 1 is released to every peer, every peer's flag is awaited with a bounded poll, then the counter takes the
// new value. One CTA. Buffers exchanged under this barrier alternate by the epoch's parity.
__global__ void ds_symm_barrier_kernel(DsPeers flags, int rank, int world, int slot, uint32_t* ctr, uint32_t budget, int* status) {
  grid_dependency_trigger();
  grid_dependency_wait();
  const int r = threadIdx.x;
  const uint32_t e = *ctr + 1u;
  if (r < world) {
    __threadfence_system();
    st_release_sys((uint32_t*)flags.p[r] + slot * 8 + rank, e);
    bool ok = false;
    for (uint32_t i = 0; i < budget; ++i) {
      if ((int32_t)(ld_acquire_sys((const uint32_t*)flags.p[rank] + slot * 8 + r) - e) >= 0) { ok = true; break; }
      if (i > 32) __nanosleep(100);
    }
    if (!ok) set_status(status, PEAR_ERR_FLAG_TIMEOUT);
  }
  __syncthreads();
  if (r == 0) *ctr = e;
}

// ------------------------------------------------------------------------------------------------ all-reduce + add + norm
// The tensor-parallel reduction of a row-parallel projection fused with the fp32 residual add and the (1 + w) RMSNorm,
// with the epoch in a device counter (graph replay). Every rank has staged its bf16 partial rows in buffer
// (*ctr + 1) & 1 of its workspace; the kernel releases that epoch to the peers, waits for theirs, sums all partials in
// rank order in fp32 straight from peer memory, adds the residual and normalises. The last CTA to finish stores the new
// epoch. (Upstream ar_norm.cu:61-208 at two ranks.)
// Sum of every rank's 8 bf16 partial values at one position, in rank order, fp32. All peers' loads are issued before
// the first one is consumed (one NVLink round trip per position instead of one per rank): the loop bounds are compile-time
// constants, the ranks beyond `world` are predicated off.
__device__ __forceinline__ void ds_sum_partials(const DsPeers& partials, int world, size_t off, float (&acc)[8]) {
  uint4 v[kDsMaxRanks];
#pragma unroll
  for (int r = 0; r < kDsMaxRanks; ++r) {
    if (r < world) {
      const __nv_bfloat16* src = (const __nv_bfloat16*)partials.p[r] + off;
      asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v[r].x), "=r"(v[r].y), "=r"(v[r].z), "=r"(v[r].w) : "l"(src) : "memory");
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
  for (int r = 0; r < kDsMaxRanks; ++r) {
    if (r < world) {
      const __nv_bfloat162* h2 = (const __nv_bfloat162*)&v[r];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h2[j]);
        acc[2 * j] += f.x; acc[2 * j + 1] += f.y;
      }
    }
  }
}

// block-wide sum of one float per thread (up to 32 warps), result to every thread
__device__ __forceinline__ float ds_block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float tot = 0.f;
  const int nw = (blockDim.x + 31) >> 5;
  for (int k = 0; k < nw; ++k) tot += red[k];
  return tot;
}

__global__ void __launch_bounds__(1024) ds_ar_add_rmsnorm_kernel(DsPeers partials, DsPeers flags, int rank, int world, int slot, uint32_t* ctr,
                                                                uint32_t* ticket, float* __restrict__ residual, int mode,
                                                                const float* __restrict__ weight, __nv_bfloat16* __restrict__ out, int T, int H,
                                                                size_t buf_elems, float eps, uint32_t budget, int* status) {
  grid_dependency_trigger();
  grid_dependency_wait();
  __shared__ float red[32];
  __shared__ int ok_flag;
  const int tid = threadIdx.x, nt = blockDim.x;
  const uint32_t epoch = *ctr + 1u;
  if (blockIdx.x == 0 && tid < world) {
    __threadfence_system();
    st_release_sys((uint32_t*)flags.p[tid] + slot * 8 + rank, epoch);
  }
  if (tid == 0) ok_flag = 1;
  __syncthreads();
  if (tid < world) {
    bool ok = false;
    for (uint32_t i = 0; i < budget; ++i) {
      if ((int32_t)(ld_acquire_sys((const uint32_t*)flags.p[rank] + slot * 8 + tid) - epoch) >= 0) { ok = true; break; }
      if (i > 32) __nanosleep(100);
    }
    if (!ok) { set_status(status, PEAR_ERR_FLAG_TIMEOUT); ok_flag = 0; }
  }
  __syncthreads();
  if (ok_flag) {
    const size_t boff = (size_t)(epoch & 1u) * buf_elems;
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
      float ssq = 0.f;
      for (int i = tid * 8; i < H; i += nt * 8) {
        float acc[8];
        ds_sum_partials(partials, world, boff + (size_t)t * H + i, acc);
        float* res = residual + (size_t)t * H + i;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (mode == 0) acc[j] += res[j];
          res[j] = acc[j];
          ssq += acc[j] * acc[j];
        }
      }
      const float rstd = rsqrtf(ds_block_sum(ssq, red) / (float)H + eps);
      for (int i = tid * 8; i < H; i += nt * 8) {
        const float* res = residual + (size_t)t * H + i;
        __nv_bfloat16* o = out + (size_t)t * H + i;
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(res[j] * rstd * (1.f + weight[i + j]));
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(ticket, 1u) == gridDim.x - 1) { *ticket = 0u; *ctr = epoch; }
  }
}

// Two-shot form for many rows (the one-shot kernel moves (W - 1) x T rows into every rank; this one moves (W - 1) / W x T
// rows in and as many out): row t belongs to rank t % W. After every rank has staged its partial rows, the owner sums the
// W partials of its rows from peer memory in rank order, adds ITS copy of the fp32 residual (a row's residual is only kept
// current on its owner), normalises, and stores the bf16 row into the `out` buffer of EVERY rank with 16-byte peer stores
// (with `bcast_residual` also the fp32 residual row, for the consumers that read the residual itself). The last CTA of a
// rank to finish releases a second flag to every peer and waits for theirs, so the kernel ends only when every rank's rows
// have landed here. `out` (and `residual` when broadcast) are symmetric buffers. (Upstream's four-rank form: rollout/hopper/
// csrc/ar_norm.cu:138-227, with the multicast store replaced by unicast peer stores.)
// With multicast addresses of the three symmetric buffers (NVLS: the same offset of every rank's buffer behind one address)
// the owner of a row gets the sum of all ranks' partial rows from ONE `multimem.ld_reduce` per 16 bytes (the switch adds,
// fp32 accumulation, bf16 result) instead of one peer load per rank, and sends the normalised row (and the residual) to all
// ranks with ONE `multimem.st` instead of one peer store per rank. Null addresses: plain peer loads and stores.
__device__ __forceinline__ void ds_mc_sum_bf16x8(const __nv_bfloat16* mc, float (&acc)[8]) {
  uint32_t r0, r1, r2, r3;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "l"(mc)
               : "memory");
  const uint32_t r[4] = {r0, r1, r2, r3};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(*(const __nv_bfloat162*)&r[j]);
    acc[2 * j] = f.x; acc[2 * j + 1] = f.y;
  }
}
__device__ __forceinline__ void ds_mc_store16(void* mc, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(__uint_as_float(a)), "f"(__uint_as_float(b)),
               "f"(__uint_as_float(c)), "f"(__uint_as_float(d))
               : "memory");
}

__global__ void __launch_bounds__(1024) ds_ar2_add_rmsnorm_kernel(DsPeers partials, DsPeers flags, DsPeers outs, DsPeers residuals, int rank, int world,
                                                                 int slot, uint32_t* ctr, uint32_t* ticket, int mode, int bcast_residual,
                                                                 const float* __restrict__ weight, int T, int H, size_t buf_elems, int fixed_buf, float eps,
                                                                 uint32_t budget, int* status, const __nv_bfloat16* mc_partials, __nv_bfloat16* mc_outs,
                                                                 float* mc_residuals) {
  grid_dependency_trigger();
  grid_dependency_wait();
  __shared__ float red[32];
  __shared__ int ok_flag;
  const int tid = threadIdx.x, nt = blockDim.x;
  const uint32_t epoch = *ctr + 1u;
  if (blockIdx.x == 0 && tid < world) {
    __threadfence_system();
    st_release_sys((uint32_t*)flags.p[tid] + slot * 8 + rank, epoch);
  }
  if (tid == 0) ok_flag = 1;
  __syncthreads();
  if (tid < world) {
    bool ok = false;
    for (uint32_t i = 0; i < budget; ++i) {
      if ((int32_t)(ld_acquire_sys((const uint32_t*)flags.p[rank] + slot * 8 + tid) - epoch) >= 0) { ok = true; break; }
      if (i > 32) __nanosleep(100);
    }
    if (!ok) { set_status(status, PEAR_ERR_FLAG_TIMEOUT); ok_flag = 0; }
  }
  __syncthreads();
  float* residual = (float*)residuals.p[rank];
  if (ok_flag) {
    // fixed_buf >= 0: the partial rows were written straight into that buffer of the workspace by the producing GEMM
    const size_t boff = (size_t)(fixed_buf >= 0 ? (uint32_t)fixed_buf : (epoch & 1u)) * buf_elems;
    for (int t = rank + world * (int)blockIdx.x; t < T; t += world * (int)gridDim.x) {
      float ssq = 0.f;
      for (int i = tid * 8; i < H; i += nt * 8) {
        float acc[8];
        if (mc_partials) ds_mc_sum_bf16x8(mc_partials + boff + (size_t)t * H + i, acc);
        else ds_sum_partials(partials, world, boff + (size_t)t * H + i, acc);
        float* res = residual + (size_t)t * H + i;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (mode == 0) acc[j] += res[j];
          res[j] = acc[j];
          ssq += acc[j] * acc[j];
        }
      }
      const float rstd = rsqrtf(ds_block_sum(ssq, red) / (float)H + eps);
      for (int i = tid * 8; i < H; i += nt * 8) {
        const float* res = residual + (size_t)t * H + i;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = res[j];
        uint4 pk;
        __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0] * rstd * (1.f + weight[i]), v[1] * rstd * (1.f + weight[i + 1]));
        __nv_bfloat162 p1 = __floats2bfloat162_rn(v[2] * rstd * (1.f + weight[i + 2]), v[3] * rstd * (1.f + weight[i + 3]));
        __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4] * rstd * (1.f + weight[i + 4]), v[5] * rstd * (1.f + weight[i + 5]));
        __nv_bfloat162 p3 = __floats2bfloat162_rn(v[6] * rstd * (1.f + weight[i + 6]), v[7] * rstd * (1.f + weight[i + 7]));
        pk.x = *(uint32_t*)&p0; pk.y = *(uint32_t*)&p1; pk.z = *(uint32_t*)&p2; pk.w = *(uint32_t*)&p3;
        if (mc_outs) {
          ds_mc_store16(mc_outs + (size_t)t * H + i, pk.x, pk.y, pk.z, pk.w);
          if (bcast_residual) {  // (also rewrites this rank's own copy with the value it already holds)
            float* rd = mc_residuals + (size_t)t * H + i;
            ds_mc_store16(rd, __float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
            ds_mc_store16(rd + 4, __float_as_uint(v[4]), __float_as_uint(v[5]), __float_as_uint(v[6]), __float_as_uint(v[7]));
          }
        } else {
          for (int p = 0; p < world; ++p) {
            const int peer = (rank + p) % world;
            *(uint4*)((__nv_bfloat16*)outs.p[peer] + (size_t)t * H + i) = pk;
            if (bcast_residual && peer != rank) {
              float4* rd = (float4*)((float*)residuals.p[peer] + (size_t)t * H + i);
              rd[0] = make_float4(v[0], v[1], v[2], v[3]);
              rd[1] = make_float4(v[4], v[5], v[6], v[7]);
            }
          }
        }
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int last;
  if (tid == 0) {
    __threadfence();
    last = atomicAdd(ticket, 1u) == gridDim.x - 1 ? 1 : 0;
  }
  __syncthreads();
  if (last) {  // every CTA of this rank has stored its rows: tell the peers, wait for theirs, then move the epoch
    if (tid < world) {
      __threadfence_system();
      st_release_sys((uint32_t*)flags.p[tid] + (slot + 1) * 8 + rank, epoch);
      bool ok = false;
      for (uint32_t i = 0; i < budget; ++i) {
        if ((int32_t)(ld_acquire_sys((const uint32_t*)flags.p[rank] + (slot + 1) * 8 + tid) - epoch) >= 0) { ok = true; break; }
        if (i > 32) __nanosleep(100);
      }
      if (!ok) set_status(status, PEAR_ERR_FLAG_TIMEOUT);
    }
    __syncthreads();
    if (tid == 0) { *ticket = 0u; *ctr = epoch; }
  }
}

}  // namespace pear

using namespace pear;

static DsPeers ds_ptrs(const void* const* host_ptrs, int world) {
  DsPeers p;
  for (int i = 0; i < kDsMaxRanks; ++i) p.p[i] = (host_ptrs && i < world) ? const_cast<void*>(host_ptrs[i]) : nullptr;
  return p;
}

PEAR_API int pear_ds_philox_uniform(float* out, int rows, int V, unsigned seed, unsigned step, void* stream) {
  ds_philox_uniform_kernel<<<dim3(64, rows), 256, 0, (cudaStream_t)stream>>>(out, rows, V, seed, step);
  PEAR_LAUNCH_CHECK();
  return 0;
}
PEAR_API int pear_ds_accept_uniform(float* out, int rows, unsigned seed, unsigned step, void* stream) {
  ds_accept_uniform_kernel<<<(rows + 127) / 128, 128, 0, (cudaStream_t)stream>>>(out, rows, seed, step);
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_ds_add_rmsnorm(const float* parts, int nsplit, long long split_stride, int ldp, float* residual, int mode, const float* w,
                                 void* out_bf16, int rows, int H, float eps, int one_plus, void* stream) {
  if (H % 4 || (nsplit > 0 && ldp % 4)) return (int)cudaErrorInvalidValue;
  if (rows <= 0) return 0;
  PEAR_CUDA_CHECK(launch_ordinary(ds_add_rmsnorm_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream, parts, nsplit, split_stride, ldp, residual, mode, w, (__nv_bfloat16*)out_bf16, H, eps,
                                                                one_plus));
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_ds_reduce_parts_bf16(const float* parts, int nsplit, long long split_stride, int ldp, void* out_bf16, size_t buf_elems,
                                       const unsigned* epoch_ctr, int rows, int H, void* stream) {
  if (H % 4 || ldp % 4) return (int)cudaErrorInvalidValue;
  if (rows <= 0) return 0;
  PEAR_CUDA_CHECK(launch_ordinary(ds_reduce_parts_bf16_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream, parts, nsplit, split_stride, ldp, (__nv_bfloat16*)out_bf16, buf_elems, epoch_ctr, H));
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_ds_attn_prep(const float* qkv, int ld, const float* qn_w, const float* kn_w, const double* inv_freq, int rot, const int* ctx,
                               const int* rope_off, const int* block_table, int max_blocks, int rows, int T, int Hq, int Hkv, int D, int gated,
                               float eps, void* q_out, void* kc, void* vc, void* stream) {
  if (rot > 128 || rot > D || (rot & 1)) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
#define PEAR_PREP(DD)                                                                                                                       \
  PEAR_CUDA_CHECK(launch_ordinary(ds_attn_prep_kernel<DD>, dim3(rows), dim3(256), 0, s, qkv, ld, qn_w, kn_w, inv_freq, rot, ctx, rope_off, block_table, \
                                   max_blocks, T, Hq, Hkv, gated, eps, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc))
  if (D == 256) PEAR_PREP(256);
  else if (D == 128) PEAR_PREP(128);
  else if (D == 64) PEAR_PREP(64);
  else return (int)cudaErrorInvalidValue;
#undef PEAR_PREP
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_ds_paged_attn_simt(const void* q, const void* kc, const void* vc, const int* block_table, int max_blocks, const int* ctx, int rows,
                                     int T, int Hq, int Hkv, int D, float scale, const float* gate_src, int gate_ld, int gated, void* out,
                                     void* stream) {
  if (Hq % Hkv || Hq / Hkv > 8) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 grid(rows, Hkv);
#define PEAR_PA(DD)                                                                                                                          \
  ds_paged_attn_simt_kernel<DD><<<grid, 256, 0, s>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, block_table, \
                                                     max_blocks, ctx, T, Hq, Hkv, scale, gate_src, gate_ld, gated, (__nv_bfloat16*)out)
  if (D == 256) PEAR_PA(256);
  else if (D == 128) PEAR_PA(128);
  else if (D == 64) PEAR_PA(64);
  else return (int)cudaErrorInvalidValue;
#undef PEAR_PA
  PEAR_LAUNCH_CHECK();
  return 0;
}

// Bytes of scratch pear_ds_gdn_verify needs for a batch of B sequences (the prep kernel's blocks).
PEAR_API long long pear_ds_gdn_scratch_bytes(int B, int Hk, int Hv) {
  return (long long)B * Hk * pear::kGdnKeyBlock + (long long)B * Hv * pear::kGdnValBlock;
}

PEAR_API int pear_ds_gdn_verify(const float* proj, int ld, const float* conv_w, const float* A_log, const float* dt_bias, const float* norm_w,
                                float* state, int num_slots, float* conv_rec, float* ab_rec, const int* slots, const int* ctx, const int* parity,
                                const int* ncommit, int B, int T, int Tmax, int Hk, int Hv, float l2_eps, float rms_eps, void* out, void* scratch,
                                int* status, void* stream) {
  if (Hv % Hk || Hv / Hk > 8 || T > Tmax || Tmax > 4 || B <= 0 || 2 * Tmax > kGdnRows || num_slots <= 0 || ((uintptr_t)state % 16) || ((uintptr_t)scratch % 16))
    return (int)cudaErrorInvalidValue;
  constexpr int smem = (int)kGdnSmem;
  static PFN_cuTensorMapEncodeTiled_v12000 enc = nullptr;
  if (!enc) {
    cudaDriverEntryPointQueryResult q;
    void* p = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return (int)cudaErrorNotSupported;
    enc = (PFN_cuTensorMapEncodeTiled_v12000)p;
  }
  CUtensorMap map_s;  // the state as a matrix [slots * Hv * 128 rows, 128 fp32]: boxes of 128 rows x 32 columns, 128-byte swizzle
  {
    cuuint64_t dims[2] = {128u, (cuuint64_t)num_slots * Hv * 128u};
    cuuint64_t strides[1] = {512u};
    cuuint32_t box[2] = {32u, 128u};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&map_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, state, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 1000 + (int)r;
  }
  static bool configured = false;
  if (!configured) {
    PEAR_CUDA_CHECK(cudaFuncSetAttribute(ds_gdn_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  uint8_t* key_blocks = (uint8_t*)scratch;
  uint8_t* val_blocks = key_blocks + (size_t)B * Hk * kGdnKeyBlock;
  cudaStream_t s = (cudaStream_t)stream;
  PEAR_CUDA_CHECK(launch_ordinary(ds_gdn_prep_kernel, dim3(Hk + Hv, B), dim3(kGdnPrepThreads), 0, s, proj, ld, conv_w, A_log, dt_bias, conv_rec, ab_rec, slots, ctx,
                                  parity, ncommit, T, Tmax, Hk, Hv, l2_eps, key_blocks, val_blocks));
  PEAR_CUDA_CHECK(launch_dependent(ds_gdn_state_kernel, dim3(Hv, B), dim3(kGdnThreads), smem, s, map_s, proj, ld, norm_w, slots, ctx, ncommit, T, Tmax, Hk,
                                   Hv, rms_eps, (const uint8_t*)key_blocks, (const uint8_t*)val_blocks, (__nv_bfloat16*)out, status));
  return 0;
}

PEAR_API int pear_ds_top_bytes() { return (int)sizeof(DsTop); }

// tops: host array of `world` device pointers (each rank's list buffer: 2 x world x rows x chunks lists); null for one rank
// together with a single local buffer in slot 0.
PEAR_API int pear_ds_topk_chunks(const float* logits, int ld, int Vs, int v0, float temperature, const int* ctx, int B, int T, int chunks,
                                 const void* const* tops, int rank, int world, const unsigned* epoch_ctr, size_t buf_elems, void* stream) {
  if (temperature <= 0.f || chunks < 1 || world < 1 || world > kDsMaxRanks) return (int)cudaErrorInvalidValue;
  PEAR_CUDA_CHECK(launch_ordinary(ds_topk_chunks_kernel, dim3(chunks, B * T), dim3(256), 0, (cudaStream_t)stream, logits, ld, Vs, v0, 1.f / temperature, ctx,
                                  T, chunks, ds_ptrs(tops, world), rank, world, epoch_ctr, buf_elems));
  return 0;
}

PEAR_API int pear_ds_topk_finish(const void* my_tops, size_t top_buf_elems, const void* my_recs, size_t rec_buf_elems, const unsigned* epoch_ctr,
                                 int world, int chunks, int B, int T, const int* ctx, int* out_id, float* out_lp, void* stream) {
  if (world * chunks * kTopK > kTopCand) return (int)cudaErrorInvalidValue;
  PEAR_CUDA_CHECK(launch_ordinary(ds_topk_finish_kernel, dim3(B * T), dim3(256), 0, (cudaStream_t)stream, (const DsTop*)my_tops, top_buf_elems,
                                  (const DsRec*)my_recs, rec_buf_elems, epoch_ctr, world, chunks, B * T, ctx, T, out_id, out_lp));
  return 0;
}

PEAR_API int pear_ds_rec_bytes() { return (int)sizeof(DsRec); }

// recs: host array of `world` device pointers (each rank's record buffer: 2 x world x rows x chunks records); null for one rank
// together with `local_recs`.
PEAR_API int pear_ds_verify_chunks(const float* logits, int ld, int Vs, int v0, float temperature, const int* tok_in, const int* ctx, int B, int T,
                                   int chunks, unsigned seed, const unsigned* step_ctr, const void* const* recs, int rank, int world,
                                   const unsigned* epoch_ctr, size_t rec_buf_elems, void* stream) {
  if (temperature <= 0.f || chunks < 1 || world < 1 || world > kDsMaxRanks) return (int)cudaErrorInvalidValue;
  PEAR_CUDA_CHECK(launch_ordinary(ds_verify_chunks_kernel, dim3(dim3(chunks, B * T)), dim3(256), 0, (cudaStream_t)stream, logits, ld, Vs, v0, 1.f / temperature, tok_in, ctx, T, chunks, seed,
                                                                                 step_ctr, ds_ptrs(recs, world), rank, world, epoch_ctr, rec_buf_elems));
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_ds_verify_finish(const void* my_recs, size_t rec_buf_elems, const unsigned* epoch_ctr, int world, int chunks, int B, int T,
                                   unsigned seed, unsigned* step_ctr, int* tok_in, int* ctx, int* ncommit, int* parity, int* out_tok, float* out_lp,
                                   int* n_accept, int* nonfinite, int* sel_row, int* mtp_tok, int* mtp_ctx, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  PEAR_CUDA_CHECK(launch_ordinary(ds_verify_finish_kernel, dim3((B + 31) / 32), dim3(32), 0, s, (const DsRec*)my_recs, rec_buf_elems, epoch_ctr, world, chunks, B * T, T, seed, step_ctr, tok_in,
                                                       ctx, ncommit, parity, out_tok, out_lp, n_accept, nonfinite, sel_row, mtp_tok, mtp_ctx, B));
  PEAR_LAUNCH_CHECK();
  PEAR_CUDA_CHECK(launch_ordinary(ds_bump_kernel, dim3(1), dim3(32), 0, s, step_ctr));
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_ds_mtp_input(const int* tokens, const void* table, int V, const float* hidden, const int* sel, const float* we, const float* wh,
                               int rows, int H, float eps, void* out, void* stream) {
  if (rows <= 0) return 0;
  PEAR_CUDA_CHECK(launch_ordinary(ds_mtp_input_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream, tokens, (const __nv_bfloat16*)table, V, hidden, sel, we, wh, H, eps, (__nv_bfloat16*)out));
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_ds_gather_rows(const float* src, const int* sel, float* dst, int rows, int H, void* stream) {
  if (H % 4) return (int)cudaErrorInvalidValue;
  PEAR_CUDA_CHECK(launch_ordinary(ds_gather_rows_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream, src, sel, dst, H));
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_ds_argmax_chunks(const float* logits, int ld, int Vs, int v0, int rows, int chunks, const void* const* keys, int rank, int world,
                                   const unsigned* epoch_ctr, size_t buf_elems, void* stream) {
  if (chunks < 1 || world < 1 || world > kDsMaxRanks) return (int)cudaErrorInvalidValue;
  PEAR_CUDA_CHECK(launch_ordinary(ds_argmax_chunks_kernel, dim3(dim3(chunks, rows)), dim3(256), 0, (cudaStream_t)stream, logits, ld, Vs, v0, chunks, ds_ptrs(keys, world), rank, world, epoch_ctr,
                                                                                buf_elems));
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_ds_argmax_finish(const void* my_keys, size_t buf_elems, const unsigned* epoch_ctr, int world, int chunks, int rows, int* dst,
                                   int dst_stride, int dst_off, int* tok_out, void* stream) {
  PEAR_CUDA_CHECK(launch_ordinary(ds_argmax_finish_kernel, dim3((rows + 127) / 128), dim3(128), 0, (cudaStream_t)stream, (const unsigned long long*)my_keys, buf_elems, epoch_ctr, world, chunks,
                                                                                rows, dst, dst_stride, dst_off, tok_out));
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_ds_symm_barrier(const void* const* flags, int rank, int world, int slot, unsigned* ctr, unsigned budget, int* status, void* stream) {
  if (world < 1 || world > kDsMaxRanks) return (int)cudaErrorInvalidValue;
  PEAR_CUDA_CHECK(launch_ordinary(ds_symm_barrier_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, ds_ptrs(flags, world), rank, world, slot, ctr, budget, status));
  PEAR_LAUNCH_CHECK();
  return 0;
}

// partials[r]: rank r's workspace of 2 x buf_elems bf16; ctr / ticket: device words of this rank (ticket zero-initialised).
PEAR_API int pear_ds_ar_add_rmsnorm(const void* const* partials, const void* const* flags, int rank, int world, int slot, unsigned* ctr,
                                    unsigned* ticket, float* residual, int mode, const float* weight, void* out_bf16, int T, int H, size_t buf_elems,
                                    float eps, unsigned budget, int* status, int num_ctas, void* stream) {
  if (world < 1 || world > kDsMaxRanks || (H % 8) != 0 || T <= 0) return (int)cudaErrorInvalidValue;
  const int grid = T < num_ctas ? T : num_ctas;
  const int threads = ((H / 8 + 31) / 32 * 32) < 1024 ? ((H / 8 + 31) / 32 * 32) : 1024;  // one 16-byte position per thread when the row fits
  PEAR_CUDA_CHECK(launch_ordinary(ds_ar_add_rmsnorm_kernel, dim3(grid), dim3(threads), 0, (cudaStream_t)stream, ds_ptrs(partials, world), ds_ptrs(flags, world), rank, world, slot, ctr, ticket,
                                                                   residual, mode, weight, (__nv_bfloat16*)out_bf16, T, H, buf_elems, eps, budget, status));
  PEAR_LAUNCH_CHECK();
  return 0;
}

// Two-shot form: outs[r] / residuals[r] are rank r's symmetric `out` (bf16 [T, H]) and residual (fp32 [T, H]) buffers; uses flag
// slots `slot` and `slot + 1`.
PEAR_API int pear_ds_ar2_add_rmsnorm(const void* const* partials, const void* const* flags, const void* const* outs, const void* const* residuals,
                                     int rank, int world, int slot, unsigned* ctr, unsigned* ticket, int mode, int bcast_residual, const float* weight,
                                     int T, int H, size_t buf_elems, int fixed_buf, float eps, unsigned budget, int* status, int num_ctas,
                                     const void* mc_partials, void* mc_outs, void* mc_residuals, void* stream) {
  if (world < 1 || world > kDsMaxRanks || (H % 8) != 0 || T <= 0) return (int)cudaErrorInvalidValue;
  if ((mc_partials != nullptr) != (mc_outs != nullptr) || (mc_outs && bcast_residual && !mc_residuals)) return (int)cudaErrorInvalidValue;
  const int mine = (T - rank + world - 1) / world;  // rows this rank owns
  int grid = mine < num_ctas ? mine : num_ctas;
  if (grid < 1) grid = 1;
  const int threads = ((H / 8 + 31) / 32 * 32) < 1024 ? ((H / 8 + 31) / 32 * 32) : 1024;
  PEAR_CUDA_CHECK(launch_ordinary(ds_ar2_add_rmsnorm_kernel, dim3(grid), dim3(threads), 0, (cudaStream_t)stream, ds_ptrs(partials, world), ds_ptrs(flags, world), ds_ptrs(outs, world),
                                                                    ds_ptrs(residuals, world), rank, world, slot, ctr, ticket, mode, bcast_residual, weight,
                                                                    T, H, buf_elems, fixed_buf, eps, budget, status, (const __nv_bfloat16*)mc_partials,
                                                                    (__nv_bfloat16*)mc_outs, (float*)mc_residuals));
  PEAR_LAUNCH_CHECK();
  return 0;
}
