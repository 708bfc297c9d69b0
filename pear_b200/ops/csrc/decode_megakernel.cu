// Persistent decode megakernel for sm_100a: one launch = one decode/verify step (T <= 8 rows) of one sequence over
// the whole NVFP4-quantised hybrid model. One CTA per SM walks its own instruction list (megakernel.cuh).
//
// Design (re-derived for B200; the counterpart of upstream deploy/blackwell/nvfp4/csrc/megakernel.cu):
//  * Weights are pre-packed into 18 KB "stages" (128 rows x 256 K): the e2m1 codes as the tensor core's K-major
//    shared-memory image (8-row x 16-byte core matrices) and the e4m3 block scales as the 32 x 16-byte atoms that
//    tcgen05.cp spreads over tensor memory. A producer warp streams stages with 1-D bulk copies (TMA engine, mbarrier
//    completion) into a shared-memory ring, following the same instruction list as the consumers but never waiting on
//    activations: weights of the NEXT op keep streaming while the consumers sit in a grid barrier.
//  * GEMV ops are stream-K: the (row tile, k-stage) space of an op is cut into contiguous per-CTA ranges; one thread
//    issues tcgen05.mma.kind::mxf4nvf4.block_scale (M 128 x N 16|32 x K 64, hardware dequantisation, fp32 accumulators
//    in tensor memory); four warps drain the accumulator with tcgen05.ld and add the partial sums to the fp32 output
//    with red.global.add (the residual add comes for free). Two accumulators alternate between segments.
//  * The weights stay exactly NVFP4. Activations are expanded on the fly into a sum of FP4 terms, each the NVFP4
//    quantisation of the previous term's residual (scale rounded up, x4 gain per term), laid out as extra rows of the
//    B operand: 4 terms for T <= 4 reach ~10 bits, so activations are better than bf16 although the MMA is 4-bit.
//  * Prologues build that operand straight from the fp32 buffers in L2: plain, (1+w) RMSNorm, SwiGLU, or the GDN gated
//    RMSNorm; a per-row power-of-two pre-scale keeps every block scale inside e4m3's range.
//  * All waits are bounded (common.cuh); on expiry the CTA records a status, drains and frees its tensor memory.
#include "common.cuh"
#include "megakernel.cuh"

#include <cooperative_groups.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

namespace mk {
using namespace pear;

constexpr int kTmemCols = 512;
constexpr int kAccCol = 0;        // 2 accumulators x 32 columns
constexpr int kSfaCol = 64;       // ring slots x 16 columns
constexpr int kSfbCol = 64 + 16 * 8;  // 320 columns: a 4-column group per K-64 block of a 5120-wide activation row
constexpr int kMaxMmas = kMaxSegStages * 4;
// shared-memory image of the activation scales: per K-64 block nb rows x 16 bytes (bytes 0..3 = the 4 block scales);
// tcgen05.cp always reads 32 rows, so with nb = 16 it also reads the next image (lanes the MMA never looks at)
__host__ __device__ constexpr int sfb_bytes(int nb) { return kMaxMmas * nb * 16 + 512; }
constexpr int kStatBytes = 3072;

struct Smem {
  uint64_t full[16];
  uint64_t empty[16];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  float red[64];
  float gscale[8];   // 1 / g_t: the epilogue's undo of the row pre-scale
};

struct Ctx {
  const Params* p;
  uint8_t* ring;       // ns * kStageBytes
  uint8_t* xs;         // scratch: B operand image | activation scale image | statistics (other ops use it freely)
  Smem* sm;
  const StepRec* rec;  // current step record
  StepRec* rec_next;
  int ns;              // ring stages
  int nb;              // rows of the B operand (16 or 32)
  int stage, phase;    // ring cursor (meaningful in the issuing thread)
  int seg;             // GEMV segments executed so far (accumulator alternation)
  uint32_t tmem;
  uint32_t barrier_target;
};

__device__ __forceinline__ int step_rows(const Ctx& c, const Desc& d) {
  return (d.i7 & 8) ? *(volatile const int*)&c.rec_next->rows_draft : c.rec->T;
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory"); }

// ---------------------------------------------------------------------------------------------------------------------
// grid barrier for the consumer warps: release-add by one thread per CTA, acquire-poll with a budget
// ---------------------------------------------------------------------------------------------------------------------
constexpr uint32_t kGridPolls = 1u << 22;
__device__ __forceinline__ void grid_barrier(Ctx& c) {
  consumer_sync();
  c.barrier_target += gridDim.x;
  if (threadIdx.x == 0) {
    red_release_gpu_add(c.p->barrier, 1u);
    bool ok = false;
    for (uint32_t i = 0; i < kGridPolls; ++i) {
      if ((int32_t)(ld_acquire_gpu(c.p->barrier) - c.barrier_target) >= 0) { ok = true; break; }
      if (i > 256) __nanosleep(20);
      if ((i & 16383u) == 16383u && *(volatile int*)c.p->status != 0) break;
    }
    if (!ok) { set_status(c.p->status, PEAR_ERR_GRID_BARRIER); c.sm->abort_flag = 1; }
  }
  consumer_sync();
}

// ---------------------------------------------------------------------------------------------------------------------
// GEMV
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float e4m3_to_f32(uint32_t code) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)code, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// Quantise 16 pre-scaled values into `terms` NVFP4 blocks (term i encodes the residual of terms < i, with a gain of
// 4^i folded into its scale) and store codes + scales into the B operand image.
//   codes : B + (chunk * (nb/8) + n/8) * 128 + (n%8) * 16 + half * 8     (chunk = block/2, half = block%2, 8 bytes)
//   scales: SFB + (block/4) * nb * 16 + n * 16 + block%4                    (n = term * tpad + row)
__device__ __forceinline__ void quantize_block(float (&r)[16], int terms, int tpad, int row, int blk, int nb, uint8_t* B,
                                               uint8_t* SFB) {
  float gain = 1.f;
  for (int term = 0; term < terms; ++term) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(r[i]));
    const float target = amax * (1.f / 6.f) * gain;
    uint32_t code = (uint32_t)__nv_cvt_float_to_fp8(target, __NV_SATFINITE, __NV_E4M3);
    float sv = e4m3_to_f32(code);
    if (sv < target && code < 0x7Eu) { ++code; sv = e4m3_to_f32(code); }  // round the scale up: no code saturates
    const float inv = sv > 0.f ? gain / sv : 0.f;
    const float back = sv / gain;
    uint32_t words[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t byte = (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(r[2 * i] * inv, r[2 * i + 1] * inv), __NV_E2M1,
                                                               cudaRoundNearest) & 0xffu;
      words[i >> 2] |= byte << (8 * (i & 3));
      __half2_raw hr = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)byte, __NV_E2M1);
      const float2 dq = __half22float2(*reinterpret_cast<__half2*>(&hr));
      r[2 * i] -= dq.x * back;
      r[2 * i + 1] -= dq.y * back;
    }
    const int n = term * tpad + row;
    *(uint2*)(B + ((size_t)(blk >> 1) * (nb >> 3) + (n >> 3)) * 128 + (n & 7) * 16 + (blk & 1) * 8) = make_uint2(words[0], words[1]);
    SFB[(blk >> 2) * nb * 16 + n * 16 + (blk & 3)] = (uint8_t)code;
    gain *= 4.f;
  }
}

// Build the B operand (FP4 terms of the activation rows) for K range [k0, k0 + kn) of the op's input.
//
// Register-resident rounds over PAIRS of rows (no stack, no spills: the L1 left beside 227 KB of shared memory is too
// small to absorb any): thread `tid` owns K block `tid` (16 elements) of both rows and, for tid < 128, one block of
// the left-over columns 256.. (block 256 + tid/2 of row tid%2), i.e. 3 blocks = 48 values. All global loads of a round
// are issued before the first use; the row statistics (RMS, maximum) are reduced with shuffles and one shared-memory
// exchange; the blocks are quantised straight from registers. PRO_NORM always covers the whole row.
template <int PRO>
__device__ __forceinline__ void gemv_prologue_t(Ctx& c, const Desc& d, int k0, int kn, int T, int tpad, int terms) {
  const StepRec* rec = c.rec;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const float* in = (const float*)d.p1;
  if ((d.i7 & 1) && PRO != PRO_GDN_NORM) in += (size_t)rec->parity * d.i8;
  const int istride = d.i3, nb = c.nb;
  uint8_t* B = c.xs;
  uint8_t* SFB = c.xs + (size_t)(kMaxSegStages * kStageK / 32) * (nb >> 3) * 128;
  float* stat = (float*)(SFB + sfb_bytes(nb));  // [warp][row of the pair][2]: partial (sum of squares, maximum)
  const float* zbase = (const float*)d.p2;
  if (PRO == PRO_GDN_NORM && (d.i7 & 1)) zbase += (size_t)rec->parity * d.i8;
  const int nblk = kn >> 4;
  const float* wp = PRO == PRO_NORM ? (const float*)d.p2 : (const float*)d.p3;

  for (int t0 = 0; t0 < tpad; t0 += 2) {
    // ---- items: e = 0, 1: (block tid, row t0 + e); e = 2: (block 256 + tid/2, row t0 + tid%2) for tid < 128
    const int b2 = 256 + (tid >> 1), r2 = tid & 1;
    float4 x[3][4];
    // ---- loads (all issued before use)
#pragma unroll
    for (int e = 0; e < 3; ++e) {
      const int b = e < 2 ? tid : b2, t = t0 + (e < 2 ? e : r2);
      const bool valid = b < nblk && t < T && (e < 2 || tid < 128);
      const int k = k0 + b * 16;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        x[e][i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (valid) {
          if (PRO == PRO_GDN_NORM) x[e][i] = __ldcg((const float4*)((const float*)d.p1 + (size_t)t * istride + k) + i);
          else x[e][i] = __ldcg((const float4*)(in + (size_t)t * istride + k) + i);
        }
      }
    }
    if (PRO == PRO_SWIGLU || PRO == PRO_GDN_NORM) {
      // second operand: loaded while the first is in flight, folded in as it arrives
#pragma unroll
      for (int e = 0; e < 3; ++e) {
        const int b = e < 2 ? tid : b2, t = t0 + (e < 2 ? e : r2);
        const bool valid = b < nblk && t < T && (e < 2 || tid < 128);
        const int k = k0 + b * 16;
        float4 y[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          y[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (valid) {
            if (PRO == PRO_GDN_NORM) y[i] = __ldcg((const float4*)(zbase + (size_t)t * d.i9 + k) + i);
            else y[i] = __ldcg((const float4*)(in + (size_t)t * istride + k + d.i0) + i);
          }
        }
        if (PRO == PRO_SWIGLU) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            x[e][i].x = silu_f(x[e][i].x) * y[i].x; x[e][i].y = silu_f(x[e][i].y) * y[i].y;
            x[e][i].z = silu_f(x[e][i].z) * y[i].z; x[e][i].w = silu_f(x[e][i].w) * y[i].w;
          }
        } else {
          // the head statistic needs the raw o: keep sum(o^2) in .. a scalar, fold silu(z) now
          float ssq = 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            ssq += x[e][i].x * x[e][i].x + x[e][i].y * x[e][i].y + x[e][i].z * x[e][i].z + x[e][i].w * x[e][i].w;
            x[e][i].x *= silu_f(y[i].x); x[e][i].y *= silu_f(y[i].y); x[e][i].z *= silu_f(y[i].z); x[e][i].w *= silu_f(y[i].w);
          }
          // a head is 8 consecutive blocks: lanes 8h..8h+7 (items 0, 1); lanes of equal row, stride 2 (item 2)
          if (e < 2) {
            ssq += __shfl_xor_sync(0xffffffffu, ssq, 1); ssq += __shfl_xor_sync(0xffffffffu, ssq, 2);
            ssq += __shfl_xor_sync(0xffffffffu, ssq, 4);
          } else {
            ssq += __shfl_xor_sync(0xffffffffu, ssq, 2); ssq += __shfl_xor_sync(0xffffffffu, ssq, 4);
            ssq += __shfl_xor_sync(0xffffffffu, ssq, 8);
          }
          const float rs = rsqrtf(ssq * (1.f / 128.f) + d.f1);
#pragma unroll
          for (int i = 0; i < 4; ++i) { x[e][i].x *= rs; x[e][i].y *= rs; x[e][i].z *= rs; x[e][i].w *= rs; }
        }
      }
    }
    // ---- weights and per-item statistics
    float ss[3], mx[3];
#pragma unroll
    for (int e = 0; e < 3; ++e) {
      ss[e] = 0.f; mx[e] = 0.f;
      if (e == 1) continue;  // item 1 shares item 0's weight block: handled together below
    }
    if (PRO == PRO_NORM || PRO == PRO_GDN_NORM) {
#pragma unroll
      for (int wsel = 0; wsel < 2; ++wsel) {
        const int b = wsel == 0 ? tid : b2;
        const int kw = PRO == PRO_NORM ? (k0 + b * 16) : ((k0 + b * 16) & 127);
        float4 w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = b < nblk ? __ldg((const float4*)(wp + kw) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int e = (wsel == 0 ? 0 : 2); e < (wsel == 0 ? 2 : 3); ++e) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float4 v = x[e][i];
            if (PRO == PRO_NORM) {
              ss[e] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
              v.x *= 1.f + w[i].x; v.y *= 1.f + w[i].y; v.z *= 1.f + w[i].z; v.w *= 1.f + w[i].w;
            } else {
              v.x *= w[i].x; v.y *= w[i].y; v.z *= w[i].z; v.w *= w[i].w;
            }
            x[e][i] = v;
          }
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 3; ++e)
#pragma unroll
      for (int i = 0; i < 4; ++i)
        mx[e] = fmaxf(mx[e], fmaxf(fmaxf(fabsf(x[e][i].x), fabsf(x[e][i].y)), fmaxf(fabsf(x[e][i].z), fabsf(x[e][i].w))));
    // ---- per-row reduction over the CTA
    float rss[2], rmx[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rss[r] = warp_sum(ss[r] + (r2 == r ? ss[2] : 0.f));
      rmx[r] = warp_max(fmaxf(mx[r], r2 == r ? mx[2] : 0.f));
    }
    consumer_sync();  // the previous round's partials have been consumed
    if (lane == 0) {
      stat[warp * 4 + 0] = rss[0]; stat[warp * 4 + 1] = rmx[0]; stat[warp * 4 + 2] = rss[1]; stat[warp * 4 + 3] = rmx[1];
    }
    consumer_sync();
    float f[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float s2 = 0.f, m = 0.f;
#pragma unroll
      for (int wq = 0; wq < kConsumerWarps; ++wq) { s2 += stat[wq * 4 + 2 * r]; m = fmaxf(m, stat[wq * 4 + 2 * r + 1]); }
      float rstd = 1.f;
      if (PRO == PRO_NORM) { rstd = rsqrtf(s2 / (float)d.i0 + d.f1); m *= rstd; }
      // power-of-two row gain: the largest block scale lands at or below 2048 / 6
      float g = 1.f;
      if (m > 0.f && m < 3.0e38f) g = exp2f(floorf(log2f(2048.f / m)));
      g = fminf(fmaxf(g, 1.0e-30f), 1.0e30f);
      if (tid == 0 && t0 + r < 8) c.sm->gscale[t0 + r] = 1.f / g;
      f[r] = g * rstd;
    }
    // ---- quantise from registers
#pragma unroll
    for (int e = 0; e < 3; ++e) {
      const int b = e < 2 ? tid : b2, row = e < 2 ? e : r2;
      if (b < nblk && (e < 2 || tid < 128)) {
        float r16[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          r16[4 * i] = x[e][i].x * f[row]; r16[4 * i + 1] = x[e][i].y * f[row];
          r16[4 * i + 2] = x[e][i].z * f[row]; r16[4 * i + 3] = x[e][i].w * f[row];
        }
        quantize_block(r16, terms, tpad, t0 + row, b, nb, B, SFB);
      }
    }
  }
}

__device__ __noinline__ void gemv_prologue(Ctx& c, const Desc& d, int k0, int kn, int T, int tpad, int terms) {
  switch (d.i5) {
    case PRO_NORM: gemv_prologue_t<PRO_NORM>(c, d, k0, kn, T, tpad, terms); break;
    case PRO_SWIGLU: gemv_prologue_t<PRO_SWIGLU>(c, d, k0, kn, T, tpad, terms); break;
    case PRO_GDN_NORM: gemv_prologue_t<PRO_GDN_NORM>(c, d, k0, kn, T, tpad, terms); break;
    default: gemv_prologue_t<PRO_PLAIN>(c, d, k0, kn, T, tpad, terms); break;
  }
}

__device__ __noinline__ void op_gemv(Ctx& c, const Instr& ins) {
  const Desc& d = c.p->descs[ins.desc];
  const int tile = ins.a, ks0 = ins.b, nks = ins.c;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = step_rows(c, d);
  const int tpad = T <= 4 ? 4 : 8, nb = c.nb, terms = min(4, nb / tpad);
  // flags: bit0 build the B operand; bit1 the whole row sits in smem (K <= 5120) and k-stages index it absolutely
  const bool whole = ins.d & 2;
  const int ab = c.seg & 1;
  const uint32_t use = (uint32_t)(c.seg >> 1) & 1u;  // parity of this use of accumulator `ab`
  uint8_t* B = c.xs;
  uint8_t* SFB = c.xs + (size_t)(kMaxSegStages * kStageK / 32) * (nb >> 3) * 128;
  const bool issuer = tid == 4 * 32;  // lane 0 of warp 4: warps 0-3 own the four tensor-memory lane quarters
  const int dbg = c.p->pad;  // timing experiments only: 1 skip the prologue, 2 skip UTCCP/MMA issue, 4 skip the epilogue math
  if (ins.d & 1) {
    // every MMA that reads the old B operand has completed once the previous segment's accumulator is full
    if (c.seg > 0) mbar_wait_bounded(&c.sm->acc_full[(c.seg - 1) & 1], (uint32_t)((c.seg - 1) >> 1) & 1u, c.p->status);
    consumer_sync();
    if (!(dbg & 1)) {
      if (whole) gemv_prologue(c, d, 0, d.i0, T, tpad, terms);
      else gemv_prologue(c, d, ks0 * kStageK, nks * kStageK, T, tpad, terms);
    }
    fence_proxy_async();  // generic-proxy stores to the operand images -> visible to the tensor core / tcgen05.cp
    consumer_sync();
    if (issuer && !(dbg & 2)) {
      const int nmma = (whole ? d.i1 : nks) * 4;
      tcgen05_fence_after();
      for (int m = 0; m < nmma; ++m)
        tmem_cp_32x128b_warpx4(c.tmem + kSfbCol + m * 4, umma_desc_interleaved(smem_u32(SFB + m * nb * 16), 128, 128));
    }
  }
  if (issuer) {
    bool ok = mbar_wait_bounded(&c.sm->acc_empty[ab], use ^ 1u, c.p->status);
    tcgen05_fence_after();
    const uint32_t idesc = umma_idesc_nvfp4(128, nb);
    const uint32_t chunk_b = (uint32_t)(nb >> 3) * 128u;
    const uint32_t b_addr = smem_u32(B);
    for (int s = 0; s < nks; ++s) {
      if (ok) ok = mbar_wait_bounded(&c.sm->full[c.stage], c.phase, c.p->status);
      if (ok && !(dbg & 2)) {
        tcgen05_fence_after();
        const uint32_t a_addr = smem_u32(c.ring + (size_t)c.stage * kStageBytes);
        const int kst = whole ? ks0 + s : s;  // stage index inside the B operand
#pragma unroll
        for (int j = 0; j < 4; ++j)
          tmem_cp_32x128b_warpx4(c.tmem + kSfaCol + c.stage * 16 + j * 4,
                                 umma_desc_interleaved(a_addr + kStageCodeBytes + j * 512, 128, 128));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint64_t da = umma_desc_interleaved(a_addr + j * 4096, 2048, 128);
          const uint64_t db = umma_desc_interleaved(b_addr + (uint32_t)(kst * 4 + j) * 2u * chunk_b, chunk_b, 128);
          umma_nvfp4(c.tmem + kAccCol + ab * 32, da, db, idesc, (s | j) != 0 ? 1u : 0u, c.tmem + kSfaCol + c.stage * 16 + j * 4,
                     c.tmem + kSfbCol + (kst * 4 + j) * 4);
        }
      }
      tcgen05_commit(&c.sm->empty[c.stage]);  // frees the ring slot once these MMAs (and copies) have read it
      if (++c.stage == c.ns) { c.stage = 0; c.phase ^= 1; }
    }
    tcgen05_commit(&c.sm->acc_full[ab]);
  }
  if (warp < 4) {
    // ---- epilogue: lane quarter `warp`; row = tile * 128 + warp * 32 + lane; column n = term * tpad + token
    const bool ok = mbar_wait_bounded(&c.sm->acc_full[ab], use, c.p->status);
    tcgen05_fence_after();
    float v[8];  // per token: sum over terms of D[term * tpad + token] * 4^-term
#pragma unroll
    for (int t = 0; t < 8; ++t) v[t] = 0.f;
    if (ok && !(dbg & 4)) {
      if (nb == 16) {
        uint32_t q[16];
        tmem_ld_32x32b_x16(c.tmem + ((uint32_t)(warp * 32) << 16) + kAccCol + ab * 32, q);
        tcgen05_wait_ld();
        if (tpad == 4) {
#pragma unroll
          for (int t = 0; t < 4; ++t)
            v[t] = __uint_as_float(q[t]) + 0.25f * __uint_as_float(q[4 + t]) + 0.0625f * __uint_as_float(q[8 + t]) +
                   0.015625f * __uint_as_float(q[12 + t]);
        } else {
#pragma unroll
          for (int t = 0; t < 8; ++t) v[t] = __uint_as_float(q[t]) + 0.25f * __uint_as_float(q[8 + t]);
        }
      } else {
        uint32_t q[32];
        tmem_ld_32x32b_x32(c.tmem + ((uint32_t)(warp * 32) << 16) + kAccCol + ab * 32, q);
        tcgen05_wait_ld();
        if (tpad == 4) {
#pragma unroll
          for (int t = 0; t < 4; ++t)
            v[t] = __uint_as_float(q[t]) + 0.25f * __uint_as_float(q[4 + t]) + 0.0625f * __uint_as_float(q[8 + t]) +
                   0.015625f * __uint_as_float(q[12 + t]);
        } else {
#pragma unroll
          for (int t = 0; t < 8; ++t)
            v[t] = __uint_as_float(q[t]) + 0.25f * __uint_as_float(q[8 + t]) + 0.0625f * __uint_as_float(q[16 + t]) +
                   0.015625f * __uint_as_float(q[24 + t]);
        }
      }
    }
    tcgen05_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&c.sm->acc_empty[ab]);
    if (ok && !(dbg & 4)) {
      float* out = (float*)d.p4;
      if (d.i7 & 2) out += (size_t)c.rec->parity * d.i8;
      const int row = tile * kTileRows + warp * 32 + lane;
      if (row < d.i2) {
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          if (t < T) {
            const float val = v[t] * c.sm->gscale[t] * d.f0;
            if (d.i6 == EPI_RED) red_add_f32(out + (size_t)t * d.i4 + row, val);
            else out[(size_t)t * d.i4 + row] = val;
          }
        }
      }
    }
  }
  ++c.seg;
}

// ---------------------------------------------------------------------------------------------------------------------
// small ops
// ---------------------------------------------------------------------------------------------------------------------
// EMBED: out[t][a .. a+b) = bf16 table[token[t]][...] ; desc p0 = table (bf16 [V][H]), p4 = out (fp32), i0 = H, i4 = out stride
__device__ void op_embed(Ctx& c, const Instr& ins) {
  const Desc& d = c.p->descs[ins.desc];
  const __nv_bfloat16* table = (const __nv_bfloat16*)d.p0;
  float* out = (float*)d.p4;
  const int T = c.rec->T;
  for (int t = 0; t < T; ++t) {
    const int tok = min(max(c.rec->tokens[t], 0), c.p->vocab - 1);  // a corrupted record must never turn into a wild read
    const __nv_bfloat16* src = table + (size_t)tok * d.i0 + ins.a;
    float* dst = out + (size_t)t * d.i4 + ins.a;
    for (int i = threadIdx.x; i < ins.b; i += kConsumerThreads) dst[i] = __bfloat162float(src[i]);
  }
}

// ZERO: p4[a .. a+b) = 0 (parity handling: i7 & 2 -> current parity, i7 & 4 -> the other parity)
__device__ void op_zero(Ctx& c, const Instr& ins) {
  const Desc& d = c.p->descs[ins.desc];
  float* out = (float*)d.p4;
  if (d.i7 & 2) out += (size_t)c.rec->parity * d.i8;
  if (d.i7 & 4) out += (size_t)(c.rec->parity ^ 1) * d.i8;
  float4* o4 = (float4*)(out + ins.a);
  for (int i = threadIdx.x; i < ins.b / 4; i += kConsumerThreads) o4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
}

// COPY: p4[a .. a+b) = p1[a .. a+b)
__device__ void op_copy(Ctx& c, const Instr& ins) {
  const Desc& d = c.p->descs[ins.desc];
  const float4* src = (const float4*)((const float*)d.p1 + ins.a);
  float4* dst = (float4*)((float*)d.p4 + ins.a);
  for (int i = threadIdx.x; i < ins.b / 4; i += kConsumerThreads) dst[i] = src[i];
}

}  // namespace mk

#include "mk_gdn.cuh"
#include "mk_attn.cuh"
#include "mk_sample.cuh"

namespace mk {

// ---------------------------------------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1) mk_main(const __grid_constant__ Params p, int ns, int nb) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  Smem* sm = (Smem*)smem_raw;
  uint8_t* ring = smem_raw + 1024;
  uint8_t* xs = ring + (size_t)ns * kStageBytes;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    for (int i = 0; i < ns; ++i) { mbar_init(&sm->full[i], 1); mbar_init(&sm->empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sm->acc_full[i], 1); mbar_init(&sm->acc_empty[i], 4); }
    sm->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {  // the whole tensor memory of the SM: this kernel is the only resident CTA (one per SM)
    tmem_alloc(&sm->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const Instr* list = p.instrs + (size_t)blockIdx.x * p.max_instrs;

  if (tid >= kConsumerThreads) {
    // ------------------------------------------------------------------------------------------ producer warp
    if (tid == kConsumerThreads) {
      int stage = 0, phase = 0;
      bool ok = true;
      Instr next = list[0];
      for (int ip = 0; ip < p.max_instrs && ok; ++ip) {
        const Instr ins = next;
        if (ins.op == OP_END) break;
        if (ip + 1 < p.max_instrs) next = list[ip + 1];  // in flight while this instruction's stages are issued
        if (ins.op != OP_GEMV) continue;
        const Desc& d = p.descs[ins.desc];
        const uint8_t* src = (const uint8_t*)d.p0 + ((size_t)ins.a * d.i1 + ins.b) * kStageBytes;
        for (int s = 0; s < ins.c; ++s) {
          ok = mbar_wait_bounded(&sm->empty[stage], phase ^ 1, p.status);
          if (!ok) break;
          mbar_expect_tx(&sm->full[stage], kStageBytes);
          bulk_load_1d(ring + (size_t)stage * kStageBytes, src + (size_t)s * kStageBytes, kStageBytes, &sm->full[stage]);
          if (++stage == ns) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------------------------------ consumer warps
    Ctx c;
    c.p = &p; c.ring = ring; c.xs = xs; c.sm = sm;
    c.rec = p.rec + p.step_parity; c.rec_next = p.rec + (p.step_parity ^ 1);
    c.ns = ns; c.nb = nb; c.stage = 0; c.phase = 0; c.seg = 0; c.tmem = sm->tmem_base; c.barrier_target = p.barrier_base;
    // instruction fetch is software-pipelined: the next instruction (and its descriptor's cache line) is requested
    // while the current one executes, so no op starts with a dependent chain of L2 round trips
    Instr next = list[0];
    for (int ip = 0; ip < p.max_instrs; ++ip) {
      const Instr ins = next;
      if (ins.op == OP_END) break;
      if (ip + 1 < p.max_instrs) next = list[ip + 1];
      if (*(volatile int*)&sm->abort_flag) {
        // drain: keep the ring protocol alive so the producer is never left waiting on a full ring
        if (ins.op == OP_GEMV && tid == 4 * 32) {
          for (int s = 0; s < ins.c; ++s) {
            mbar_wait_bounded(&sm->full[c.stage], c.phase, p.status);
            mbar_arrive(&sm->empty[c.stage]);
            if (++c.stage == c.ns) { c.stage = 0; c.phase ^= 1; }
          }
        }
        continue;
      }
      switch (ins.op) {
        case OP_GEMV: op_gemv(c, ins); break;
        case OP_BARRIER: grid_barrier(c); break;
        case OP_EMBED: op_embed(c, ins); break;
        case OP_ZERO: op_zero(c, ins); break;
        case OP_COPY: op_copy(c, ins); break;
        case OP_GDN: if (!(p.pad & 16)) op_gdn(c, ins); break;
        case OP_ATTN: if (!(p.pad & 32)) op_attn(c, ins); break;
        case OP_ATTN_COMBINE: if (!(p.pad & 32)) op_attn_combine(c, ins); break;
        case OP_SAMPLE_PART: op_sample_part(c, ins); break;
        case OP_SAMPLE_FIN: op_sample_fin(c, ins); break;
        case OP_DRAFT_IN: op_draft_in(c, ins); break;
        case OP_ARGMAX_PART: op_argmax_part(c, ins); break;
        case OP_ARGMAX_FIN: op_argmax_fin(c, ins); break;
        default: set_status(p.status, PEAR_ERR_BAD_INSTR); break;
      }
      if (next.op != OP_END && next.op != OP_BARRIER)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p.descs + next.desc));
    }
    // every issued MMA has completed before tensor memory is released
    if (c.seg > 0) mbar_wait_bounded(&sm->acc_full[(c.seg - 1) & 1], (uint32_t)((c.seg - 1) >> 1) & 1u, p.status);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) {
    tcgen05_fence_after();
    tmem_dealloc(sm->tmem_base, kTmemCols);
  }
}

}  // namespace mk

// ---------------------------------------------------------------------------------------------------------------------
// host entry points
// ---------------------------------------------------------------------------------------------------------------------
static int mk_scratch_bytes(int nb) {
  const int need = (mk::kMaxSegStages * mk::kStageK / 32) * (nb / 8) * 128 + mk::sfb_bytes(nb) + mk::kStatBytes;
  return need > 82176 ? need : 82176;  // the attention op's tiles need 80.4 KB of the same region
}
PEAR_API int pear_mk_smem_bytes(int ns, int nb) { return 1024 + ns * mk::kStageBytes + mk_scratch_bytes(nb); }

// Launch one step. `params` is a host copy of mk::Params; `nb` = rows of the activation operand (16: up to 4 rows x 4
// terms or 8 rows x 2 terms; 32: 8 rows x 4 terms). Cooperative launch: all CTAs are co-resident or the launch fails
// (never a deadlocked grid barrier).
PEAR_API int pear_mk_launch(const void* params, int num_ctas, int ns, int nb, void* stream) {
  static int configured_smem = -1;
  if ((nb != 16 && nb != 32) || ns < 2 || ns > 8) return (int)cudaErrorInvalidValue;
  const int smem = pear_mk_smem_bytes(ns, nb);
  if (smem > 232448) return (int)cudaErrorInvalidValue;
  if (configured_smem < smem) {
    PEAR_CUDA_CHECK(cudaFuncSetAttribute(mk::mk_main, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured_smem = smem;
  }
  mk::Params p = *(const mk::Params*)params;
  void* args[] = {(void*)&p, (void*)&ns, (void*)&nb};
  PEAR_CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)mk::mk_main, dim3(num_ctas), dim3(mk::kThreads), args,
                                              (size_t)smem, (cudaStream_t)stream));
  return 0;
}

PEAR_API int pear_mk_sizes(int* out) {
  out[0] = sizeof(mk::Instr); out[1] = sizeof(mk::Desc); out[2] = sizeof(mk::StepRec); out[3] = sizeof(mk::StepOut);
  out[4] = sizeof(mk::Params); out[5] = mk::kStageBytes; out[6] = mk::kXStride; out[7] = mk::kThreads;
  return 0;
}
