// Persistent decode megakernel for sm_100a: one launch = one decode/verify step (T <= 8 rows) of one sequence over
// the whole NVFP4-quantised hybrid model. One CTA per SM walks its own instruction list (megakernel.cuh).
//
// Design (re-derived for B200; the counterpart of upstream deploy/blackwell/nvfp4/csrc/megakernel.cu):
//  * Weights are pre-packed into 18 KB "stages" (128 rows x 256 K: e2m1 codes in mma-fragment order + e4m3 block
//    scales). A producer warp streams stages with 1-D bulk copies (TMA engine, mbarrier completion) into a shared
//    memory ring, following the same instruction list as the consumers but never waiting on activations: weights of
//    the NEXT op keep streaming while the consumers sit in a grid barrier, so HBM never idles across op boundaries.
//  * GEMV ops are stream-K: the (row tile, k-stage) space of an op is cut into contiguous per-CTA ranges; partial sums
//    are added to the fp32 output with red.global.add (the residual add comes for free).
//  * Prologues build the f16 activation rows in shared memory straight from the fp32 buffers in L2: plain, (1+w)
//    RMSNorm, SwiGLU, or the GDN gated RMSNorm.
//  * Dequantisation is exact: e2m1 -> f16 (cvt), times the e4m3 block scale in f16 (<= 6 significant bits), then
//    mma.sync m16n8k16 with fp32 accumulation; activations stay f16 (not re-quantised to 4 bits).
//  * All waits are bounded (common.cuh); on expiry the CTA records a status and drains.
#include "common.cuh"
#include "megakernel.cuh"

#include <cooperative_groups.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

namespace mk {
using namespace pear;

struct Smem {
  uint64_t full[16];
  uint64_t empty[16];
  float red[64];
  float rstd[8];
  int rstd_tag;
  int abort_flag;
};

struct Ctx {
  const Params* p;
  uint8_t* ring;       // NS * kStageBytes
  __half* xs;          // activation rows [MAXT][kXStride] (also scratch of the non-GEMV ops)
  Smem* sm;
  const StepRec* rec;  // current step record
  StepRec* rec_next;
  int ns;              // ring stages
  int maxt;            // activation rows kept in smem (power of two)
  int stage, phase;    // consumer ring cursor
  uint32_t barrier_target;
};

__device__ __forceinline__ int step_rows(const Ctx& c, const Desc& d) {
  return (d.i7 & 8) ? *(volatile const int*)&c.rec_next->rows_draft : c.rec->T;
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory"); }

// ---------------------------------------------------------------------------------------------------------------------
// grid barrier for the consumer warps: release-add by one thread per CTA, acquire-poll with a budget
// ---------------------------------------------------------------------------------------------------------------------
constexpr uint32_t kGridPolls = 1u << 21;
__device__ __forceinline__ void grid_barrier(Ctx& c) {
  consumer_sync();
  c.barrier_target += gridDim.x;
  if (threadIdx.x == 0) {
    __threadfence();
    red_release_gpu_add(c.p->barrier, 1u);
    bool ok = false;
    for (uint32_t i = 0; i < kGridPolls; ++i) {
      if ((int32_t)(ld_acquire_gpu(c.p->barrier) - c.barrier_target) >= 0) { ok = true; break; }
      if (i > 32) __nanosleep(32);
      if ((i & 4095u) == 4095u && *(volatile int*)c.p->status != 0) break;
    }
    if (!ok) { set_status(c.p->status, PEAR_ERR_GRID_BARRIER); c.sm->abort_flag = 1; }
  }
  consumer_sync();
}

// ---------------------------------------------------------------------------------------------------------------------
// GEMV
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

__device__ __forceinline__ __half2 e2m1x2_to_h2(uint32_t byte) {
  __half2_raw r = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)byte, __NV_E2M1);
  return *reinterpret_cast<__half2*>(&r);
}
__device__ __forceinline__ __half2 e4m3x2_to_h2(uint32_t two_bytes) {
  __half2_raw r = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)two_bytes, __NV_E4M3);
  return *reinterpret_cast<__half2*>(&r);
}

__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float clamp_h(float v) { return fminf(fmaxf(v, -65504.f), 65504.f); }

// Build the f16 activation rows for K range [k0, k0 + kn) of the op's input into c.xs.
__device__ void gemv_prologue(Ctx& c, const Desc& d, int k0, int kn) {
  const StepRec* rec = c.rec;
  const int T = step_rows(c, d);
  const int tid = threadIdx.x;
  const float* in = (const float*)d.p1;
  if ((d.i7 & 1) && d.i5 != PRO_GDN_NORM) in += (size_t)rec->parity * d.i8;
  const int istride = d.i3;
  const int pro = d.i5;
  if (pro == PRO_NORM) {
    // rstd per row over the whole K; cached per descriptor
    if (c.sm->rstd_tag != (int)(&d - c.p->descs)) {
      for (int t = 0; t < T; ++t) {
        float s = 0.f;
        const float4* row = (const float4*)(in + (size_t)t * istride);
        for (int i = tid; i < d.i0 / 4; i += kConsumerThreads) {
          float4 v = __ldcg(row + i);
          s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        s = warp_sum(s);
        consumer_sync();
        if ((tid & 31) == 0) c.sm->red[tid >> 5] = s;
        consumer_sync();
        if (tid == 0) {
          float tot = 0.f;
          for (int w = 0; w < kConsumerWarps; ++w) tot += c.sm->red[w];
          c.sm->rstd[t] = rsqrtf(tot / (float)d.i0 + d.f1);
        }
      }
      if (tid == 0) c.sm->rstd_tag = (int)(&d - c.p->descs);
      consumer_sync();
    }
    const float* w = (const float*)d.p2;
    for (int t = 0; t < T; ++t) {
      const float rs = c.sm->rstd[t];
      const float* row = in + (size_t)t * istride + k0;
      __half* xr = c.xs + (size_t)(t & (c.maxt - 1)) * kXStride;
      for (int i = tid * 4; i < kn; i += kConsumerThreads * 4) {
        float4 v = __ldcg((const float4*)(row + i));
        float4 g = *(const float4*)(w + k0 + i);
        __half2 a = __floats2half2_rn(clamp_h(v.x * rs * (1.f + g.x)), clamp_h(v.y * rs * (1.f + g.y)));
        __half2 b = __floats2half2_rn(clamp_h(v.z * rs * (1.f + g.z)), clamp_h(v.w * rs * (1.f + g.w)));
        *(uint2*)(xr + i) = make_uint2(h2_as_u32(a), h2_as_u32(b));
      }
    }
  } else if (pro == PRO_PLAIN) {
    for (int t = 0; t < T; ++t) {
      const float* row = in + (size_t)t * istride + k0;
      __half* xr = c.xs + (size_t)(t & (c.maxt - 1)) * kXStride;
      for (int i = tid * 4; i < kn; i += kConsumerThreads * 4) {
        float4 v = __ldcg((const float4*)(row + i));
        __half2 a = __floats2half2_rn(clamp_h(v.x), clamp_h(v.y));
        __half2 b = __floats2half2_rn(clamp_h(v.z), clamp_h(v.w));
        *(uint2*)(xr + i) = make_uint2(h2_as_u32(a), h2_as_u32(b));
      }
    }
  } else if (pro == PRO_SWIGLU) {
    // input rows hold [gate (K) | up (K)]
    for (int t = 0; t < T; ++t) {
      const float* row = in + (size_t)t * istride + k0;
      const float* up = row + d.i0;
      __half* xr = c.xs + (size_t)(t & (c.maxt - 1)) * kXStride;
      for (int i = tid * 4; i < kn; i += kConsumerThreads * 4) {
        float4 g = __ldcg((const float4*)(row + i));
        float4 u = __ldcg((const float4*)(up + i));
        __half2 a = __floats2half2_rn(clamp_h(silu_f(g.x) * u.x), clamp_h(silu_f(g.y) * u.y));
        __half2 b = __floats2half2_rn(clamp_h(silu_f(g.z) * u.z), clamp_h(silu_f(g.w) * u.w));
        *(uint2*)(xr + i) = make_uint2(h2_as_u32(a), h2_as_u32(b));
      }
    }
  } else {  // PRO_GDN_NORM: per (row, head of 128): o * rsqrt(mean(o^2) + eps) * w * silu(z); k0, kn multiples of 128
    const float* zbase = (const float*)d.p2;  // z rows: same row stride as the record (d.i8 reused as z stride)
    if (d.i7 & 1) zbase += (size_t)rec->parity * d.i8;
    const int zstride = d.i9;
    const float* nw = (const float*)d.p3;
    const int warp = tid >> 5, lane = tid & 31;
    const int heads = kn / 128;
    for (int item = warp; item < T * heads; item += kConsumerWarps) {
      const int t = item / heads, h = item % heads;
      const float* o = (const float*)d.p1 + (size_t)t * istride + k0 + h * 128;
      const float* z = zbase + (size_t)t * zstride + k0 + h * 128;
      float4 v = __ldcg((const float4*)(o + lane * 4));
      float s = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
      const float rs = rsqrtf(s * (1.f / 128.f) + d.f1);
      float4 zz = __ldcg((const float4*)(z + lane * 4));
      float4 ww = *(const float4*)(nw + lane * 4);
      __half* xr = c.xs + (size_t)(t & (c.maxt - 1)) * kXStride + h * 128 + lane * 4;
      __half2 a = __floats2half2_rn(clamp_h(v.x * rs * ww.x * silu_f(zz.x)), clamp_h(v.y * rs * ww.y * silu_f(zz.y)));
      __half2 b = __floats2half2_rn(clamp_h(v.z * rs * ww.z * silu_f(zz.z)), clamp_h(v.w * rs * ww.w * silu_f(zz.w)));
      *(uint2*)xr = make_uint2(h2_as_u32(a), h2_as_u32(b));
    }
  }
}

// One stage for one warp: 16 rows x 256 K. Packed layout (see pear_b200/models/nvfp4.py: pack_stages):
//   codes : ((warp*4 + quad)*32 + lane)*16 + j*4 + byte ; byte0 (row g, k 4t,4t+1) byte1 (row g+8, same k)
//           byte2 (row g, k 4t+2,4t+3) byte3 (row g+8, same k), k relative to block quad*64 + j*16
//   scales: 16384 + (warp*4 + quad)*64 + g*8 + j*2 + half   (half 0: row g, 1: row g+8)
__device__ __forceinline__ void gemv_stage(const uint8_t* stage, const __half* xrow, int warp, int lane, float (&acc)[4]) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint4 codes = *(const uint4*)(stage + ((warp * 4 + q) * 32 + lane) * 16);
    const uint2 sc = *(const uint2*)(stage + kStageCodeBytes + (warp * 4 + q) * 64 + g * 8);
    const uint32_t cw[4] = {codes.x, codes.y, codes.z, codes.w};
    const uint32_t sw[4] = {sc.x & 0xffffu, sc.x >> 16, sc.y & 0xffffu, sc.y >> 16};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half2 s2 = e4m3x2_to_h2(sw[j]);
      const __half2 s_lo = __low2half2(s2), s_hi = __high2half2(s2);
      uint32_t a[4];
      a[0] = h2_as_u32(__hmul2(e2m1x2_to_h2(cw[j] & 0xffu), s_lo));
      a[1] = h2_as_u32(__hmul2(e2m1x2_to_h2((cw[j] >> 8) & 0xffu), s_hi));
      a[2] = h2_as_u32(__hmul2(e2m1x2_to_h2((cw[j] >> 16) & 0xffu), s_lo));
      a[3] = h2_as_u32(__hmul2(e2m1x2_to_h2(cw[j] >> 24), s_hi));
      const uint2 b = *(const uint2*)(xrow + q * 64 + j * 16 + t * 4);
      mma_f16(acc, a, b.x, b.y);
    }
  }
}

__device__ void op_gemv(Ctx& c, const Instr& ins) {
  const Desc& d = c.p->descs[ins.desc];
  const int tile = ins.a, ks0 = ins.b, nks = ins.c;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (ins.d & 1) {
    consumer_sync();  // previous users of xs are done
    gemv_prologue(c, d, ks0 * kStageK, nks * kStageK);
    consumer_sync();
  }
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const int g = lane >> 2, t = lane & 3;
  const __half* xrow = c.xs + (size_t)(g & (c.maxt - 1)) * kXStride;
  bool ok = true;
  for (int s = 0; s < nks; ++s) {
    if (ok) ok = mbar_wait_bounded(&c.sm->full[c.stage], c.phase, c.p->status);
    if (ok) gemv_stage(c.ring + (size_t)c.stage * kStageBytes, xrow + s * kStageK, warp, lane, acc);
    __syncwarp();
    if (lane == 0) mbar_arrive(&c.sm->empty[c.stage]);
    if (++c.stage == c.ns) { c.stage = 0; c.phase ^= 1; }
  }
  // epilogue: c0 (row g, token 2t) c1 (row g, token 2t+1) c2 (row g+8, token 2t) c3 (row g+8, token 2t+1)
  const int T = step_rows(c, d);
  float* out = (float*)d.p4;
  if (d.i7 & 2) out += (size_t)c.rec->parity * d.i8;
  const int ostride = d.i4;
  const int r0 = tile * kTileRows + warp * 16 + g;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = r0 + (i >> 1) * 8, tok = 2 * t + (i & 1);
    if (tok < T && row < d.i2) {
      float v = acc[i] * d.f0;
      if (d.i6 == EPI_RED) red_add_f32(out + (size_t)tok * ostride + row, v);
      else out[(size_t)tok * ostride + row] = v;
    }
  }
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
    const int tok = c.rec->tokens[t];
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
__global__ void __launch_bounds__(kThreads, 1) mk_main(const __grid_constant__ Params p, int ns, int maxt) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  Smem* sm = (Smem*)smem_raw;
  uint8_t* ring = smem_raw + 1024;
  __half* xs = (__half*)(ring + (size_t)ns * kStageBytes);
  const int tid = threadIdx.x;
  if (tid == 0) {
    for (int i = 0; i < ns; ++i) { mbar_init(&sm->full[i], 1); mbar_init(&sm->empty[i], kConsumerWarps); }
    sm->rstd_tag = -1;
    sm->abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  const Instr* list = p.instrs + (size_t)blockIdx.x * p.max_instrs;

  if (tid >= kConsumerThreads) {
    // ------------------------------------------------------------------------------------------ producer warp
    if (tid == kConsumerThreads) {
      int stage = 0, phase = 0;
      bool ok = true;
      for (int ip = 0; ip < p.max_instrs && ok; ++ip) {
        const Instr ins = list[ip];
        if (ins.op == OP_END) break;
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
    c.ns = ns; c.maxt = maxt; c.stage = 0; c.phase = 0; c.barrier_target = p.barrier_base;
    for (int ip = 0; ip < p.max_instrs; ++ip) {
      const Instr ins = list[ip];
      if (ins.op == OP_END) break;
      if (*(volatile int*)&sm->abort_flag) {
        // drain: keep the ring protocol alive so the producer is never left waiting on a full ring
        if (ins.op == OP_GEMV) {
          for (int s = 0; s < ins.c; ++s) {
            mbar_wait_bounded(&sm->full[c.stage], c.phase, p.status);
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive(&sm->empty[c.stage]);
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
        case OP_GDN: op_gdn(c, ins); break;
        case OP_ATTN: op_attn(c, ins); break;
        case OP_ATTN_COMBINE: op_attn_combine(c, ins); break;
        case OP_SAMPLE_PART: op_sample_part(c, ins); break;
        case OP_SAMPLE_FIN: op_sample_fin(c, ins); break;
        case OP_DRAFT_IN: op_draft_in(c, ins); break;
        case OP_ARGMAX_PART: op_argmax_part(c, ins); break;
        case OP_ARGMAX_FIN: op_argmax_fin(c, ins); break;
        default: set_status(p.status, PEAR_ERR_BAD_INSTR); break;
      }
    }
  }
}

}  // namespace mk

// ---------------------------------------------------------------------------------------------------------------------
// host entry points
// ---------------------------------------------------------------------------------------------------------------------
PEAR_API int pear_mk_smem_bytes(int ns, int maxt) {
  return 1024 + ns * mk::kStageBytes + maxt * mk::kXStride * 2;
}

// Launch one step. `params` is a host copy of mk::Params. Cooperative launch: all CTAs are co-resident or the launch
// fails (never a deadlocked grid barrier).
PEAR_API int pear_mk_launch(const void* params, int num_ctas, int ns, int maxt, void* stream) {
  static int configured_smem = -1;
  const int smem = pear_mk_smem_bytes(ns, maxt);
  if (configured_smem < smem) {
    PEAR_CUDA_CHECK(cudaFuncSetAttribute(mk::mk_main, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured_smem = smem;
  }
  mk::Params p = *(const mk::Params*)params;
  void* args[] = {(void*)&p, (void*)&ns, (void*)&maxt};
  PEAR_CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)mk::mk_main, dim3(num_ctas), dim3(mk::kThreads), args,
                                              (size_t)smem, (cudaStream_t)stream));
  return 0;
}

PEAR_API int pear_mk_sizes(int* out) {
  out[0] = sizeof(mk::Instr); out[1] = sizeof(mk::Desc); out[2] = sizeof(mk::StepRec); out[3] = sizeof(mk::StepOut);
  out[4] = sizeof(mk::Params); out[5] = mk::kStageBytes; out[6] = mk::kXStride; out[7] = mk::kThreads;
  return 0;
}
