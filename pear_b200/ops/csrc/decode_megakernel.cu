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
  uint64_t bload;      // completion of the activation-operand bulk copies
  uint32_t tmem_base;
  int abort_flag;
  float red[64];
  float gscale[8];   // 1 / g_t: the epilogue's undo of the row pre-scale
  int fin_unit;      // unit of the next GEMV's operand this CTA's epilogue warps build (-1: none)
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
  int nload;           // operand loads so far (parity of the bload barrier)
  uint32_t tmem;
  uint32_t barrier_target;
  int ip;              // index of the instruction being executed (tracing)
};

__device__ __forceinline__ int step_rows(const Ctx& c, const Desc& d) {
  return (d.i7 & 8) ? *(volatile const int*)&c.rec_next->rows_draft : c.rec->T;
}

// Timeline record (thread 0 of the traced CTAs only): mark ids are small integers documented beside their call sites.
__device__ __forceinline__ void trace_mark(const Ctx& c, int id) {
  // three timelines per traced CTA: thread 0, the MMA-issuing thread, the weight producer thread
  const int who = threadIdx.x == 0 ? 0 : (threadIdx.x == 4 * 32 ? 1 : (threadIdx.x == kConsumerThreads ? 2 : -1));
  if (c.p->trace == nullptr || who < 0 || (int)blockIdx.x >= c.p->trace_ctas) return;
  unsigned long long* base = c.p->trace + ((size_t)blockIdx.x * 3 + who) * c.p->trace_cap * 2;
  const unsigned long long n = base[0];
  if ((int)n + 1 >= c.p->trace_cap) return;
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  base[2 * (n + 1)] = ((unsigned long long)id << 32) | (unsigned)c.ip;
  base[2 * (n + 1) + 1] = t;
  base[0] = n + 1;
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
}  // namespace mk

#include "mk_quant.cuh"

namespace mk {

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
  trace_mark(c, 10);  // gemv: entered
  if (ins.d & 1) {
    // every MMA that reads the old B operand has completed once the previous segment's accumulator is full
    // (one polling thread per wait: hundreds of threads polling an mbarrier slow the tensor core's own operand reads)
    if (c.seg > 0 && tid == 0) mbar_wait_bounded(&c.sm->acc_full[(c.seg - 1) & 1], (uint32_t)((c.seg - 1) >> 1) & 1u, c.p->status);
    consumer_sync();
    trace_mark(c, 11);  // gemv: previous MMAs drained, operand load starts
    // the operand images of this op were built by OP_QUANT in the previous phase: pull this segment's K range
    const int k0 = whole ? 0 : ks0 * kStageK, kn = whole ? d.i0 : nks * kStageK;
    const uint32_t chunk_bytes = (uint32_t)(nb >> 3) * 128u;
    const uint32_t b_bytes = (uint32_t)(kn >> 5) * chunk_bytes;
    const uint32_t sf_bytes = (uint32_t)(kn >> 6) * nb * 16u + (nb == 16 ? 256u : 0u);  // tcgen05.cp reads 32 rows
    if (tid == 0 && !(dbg & 1)) {
      asm volatile("fence.proxy.async;" ::: "memory");
      mbar_expect_tx(&c.sm->bload, b_bytes + sf_bytes);
      bulk_load_1d(B, (const uint8_t*)d.p5 + (size_t)(k0 >> 5) * chunk_bytes, b_bytes, &c.sm->bload);
      bulk_load_1d(SFB, (const uint8_t*)d.p6 + (size_t)(k0 >> 6) * nb * 16, sf_bytes, &c.sm->bload);
    }
    if (tid == 0 && !(dbg & 1)) mbar_wait_bounded(&c.sm->bload, (uint32_t)c.nload & 1u, c.p->status);
    ++c.nload;
    if (tid < 8) {
      // epilogue factor per row: undo the pre-gain, apply the deferred RMS of PRO_NORM
      float f = 1.f / kPreGain;
      if (d.i5 == PRO_NORM) f *= rsqrtf(__ldcg((const float*)d.p7 + tid) / (float)d.i0 + d.f1);
      c.sm->gscale[tid] = f;
    }
    consumer_sync();
    trace_mark(c, 12);  // gemv: operand in shared memory
  }
  if (issuer) {
    bool ok = mbar_spin_bounded(&c.sm->acc_empty[ab], use ^ 1u, c.p->status);
    trace_mark(c, 21);  // issuer: accumulator free
    tcgen05_fence_after();
    const uint32_t idesc = umma_idesc_nvfp4(128, nb);
    const uint32_t chunk_b = (uint32_t)(nb >> 3) * 128u;
    const uint64_t a_desc0 = umma_desc_interleaved(smem_u32(c.ring), 2048, 128);
    const uint64_t sfa_desc0 = umma_desc_interleaved(smem_u32(c.ring) + kStageCodeBytes, 128, 128);
    const uint64_t b_desc0 = umma_desc_interleaved(smem_u32(B), chunk_b, 128);
    const uint32_t a_hi = (uint32_t)(a_desc0 >> 32), sfa_hi = (uint32_t)(sfa_desc0 >> 32), b_hi = (uint32_t)(b_desc0 >> 32);
    const uint32_t b_mma = (2u * chunk_b) >> 4;  // address-field step of the B operand per MMA (64 K elements)
    const uint32_t acc_addr = c.tmem + kAccCol + ab * 32;
    const int kst0 = whole ? ks0 : 0;            // stage index inside the B operand
    uint32_t b_lo = (uint32_t)b_desc0 + (uint32_t)kst0 * 4u * b_mma;
    // the operand's scale factors (one 4-column group per MMA) are copied into tensor memory right before the MMA that
    // reads them, like the weights' own: the tensor pipe overlaps such a copy with the previous MMA, whereas copying
    // the whole row's groups up front would sit on the critical path of every GEMV op
    const uint64_t sfb_desc0 = umma_desc_interleaved(smem_u32(SFB), 128, 128);
    const uint32_t sfb_hi = (uint32_t)(sfb_desc0 >> 32), sfb_mma = (uint32_t)(nb * 16) >> 4;
    uint32_t sfb_lo = (uint32_t)sfb_desc0 + (uint32_t)kst0 * 4u * sfb_mma;
    uint32_t accumulate = 0;
    // Two stages per iteration: what bounds this loop is the issuing thread's own chain of latencies (barrier poll,
    // issue, commit), so both polls go out back to back and eight MMAs follow; each scale-factor copy sits directly
    // in front of its MMA, where the tensor pipe overlaps it with the previous MMA.
    constexpr int kGroup = 4;
    for (int s = 0; s < nks; s += kGroup) {
      const int n = min(kGroup, nks - s);
      int st[kGroup];
      uint32_t ph[kGroup];
      bool ready[kGroup];
#pragma unroll
      for (int g = 0; g < kGroup; ++g) {
        int x = c.stage + g;
        ph[g] = c.phase;
        if (x >= c.ns) { x -= c.ns; ph[g] ^= 1u; }
        st[g] = x;
        ready[g] = g >= n || mbar_test_wait(&c.sm->full[x], ph[g]);
      }
#pragma unroll
      for (int g = 0; g < kGroup; ++g)
        if (ok && !ready[g]) ok = mbar_spin_bounded(&c.sm->full[st[g]], ph[g], c.p->status);
      tcgen05_fence_after();
#pragma unroll
      for (int g = 0; g < kGroup; ++g) {
        if (g < n) {
          if (ok && !(dbg & 2)) {
            const uint32_t a_lo = (uint32_t)a_desc0 + (uint32_t)st[g] * (kStageBytes >> 4);
            const uint32_t sfa_lo = (uint32_t)sfa_desc0 + (uint32_t)st[g] * (kStageBytes >> 4);
            const uint32_t sfa_addr = c.tmem + kSfaCol + st[g] * 16, sfb_addr = c.tmem + kSfbCol + st[g] * 16;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              tmem_cp_32x128b_warpx4(sfa_addr + j * 4, ((uint64_t)sfa_hi << 32) | (sfa_lo + j * 32));
              tmem_cp_32x128b_warpx4(sfb_addr + j * 4, ((uint64_t)sfb_hi << 32) | (sfb_lo + j * sfb_mma));
              umma_nvfp4(acc_addr, ((uint64_t)a_hi << 32) | (a_lo + j * 256), ((uint64_t)b_hi << 32) | (b_lo + j * b_mma), idesc,
                         accumulate, sfa_addr + j * 4, sfb_addr + j * 4);
              accumulate = 1;
            }
          }
          b_lo += 4u * b_mma;
          sfb_lo += 4u * sfb_mma;
          tcgen05_commit(&c.sm->empty[st[g]]);  // frees the ring slot once these MMAs (and copies) have read it
        }
      }
      c.stage += n;
      if (c.stage >= c.ns) { c.stage -= c.ns; c.phase ^= 1; }
    }
    tcgen05_commit(&c.sm->acc_full[ab]);
    trace_mark(c, 22);  // issuer: segment issued
  }
  if (warp < 4) {
    // ---- epilogue: lane quarter `warp`; row = tile * 128 + warp * 32 + lane; column n = term * tpad + token
    bool ok = true;
    if (lane == 0) ok = mbar_wait_relaxed(&c.sm->acc_full[ab], use, c.p->status);
    ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
    trace_mark(c, 13);  // gemv: accumulator full
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
    if (d.pad[0] > 0) {
      // This GEMV feeds another one: count this contribution to the row tile; the warps that delivered the last one
      // ("finishers") turn the now complete 128 outputs into one unit of the next GEMV's operand.
      const Desc& cd = c.p->descs[d.pad[0] - 1];
      __threadfence();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (tid == 0) {
        const int slot = d.pad[1] + tile % (cd.i0 >> 7);
        const int expect = __ldg(c.p->tile_expect + slot);  // 0: this program does not run the consumer
        const bool last = expect > 0 && atomicAdd(c.p->tile_cnt + slot, 1) + 1 == expect;
        if (last) c.p->tile_cnt[slot] = 0;  // nobody touches the counter again before the next step
        c.sm->fin_unit = last ? tile % (cd.i0 >> 7) : -1;
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
      const int unit = *(volatile int*)&c.sm->fin_unit;
      if (unit >= 0) {
        __threadfence();
        quant_units(c, cd, unit, 1, 128);
      }
    }
  }
  trace_mark(c, 14);  // gemv: epilogue issued
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
    mbar_init(&sm->bload, 1);
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
      // L2 look-ahead: a second cursor walks the same instruction list `l2_ahead` stages in front of the ring and asks
      // the TMA engine to pull those stages into L2, so HBM keeps streaming through phases in which the ring is full
      // (grid barriers, recurrent/attention ops); the ring then refills from L2 faster than HBM could deliver.
      // (requested in chunks of up to 8 stages per bulk-prefetch instruction: every bulk instruction costs this
      // thread a few hundred cycles whatever its size.)
      int pf_ip = 0, pf_s = 0, pf_left = 0, pf_issued = 0, main_issued = 0;
      const uint8_t* pf_src = nullptr;
      bool pf_end = p.l2_ahead <= 0;
      auto pf_step = [&]() {
        while (!pf_end && pf_issued < main_issued + p.l2_ahead) {
          while (!pf_end && pf_s >= pf_left) {
            if (pf_ip >= p.max_instrs) { pf_end = true; break; }
            const Instr pi = list[pf_ip++];
            if (pi.op == OP_END) { pf_end = true; break; }
            if (pi.op != OP_GEMV) continue;
            const Desc& pd = p.descs[pi.desc];
            pf_src = (const uint8_t*)pd.p0 + ((size_t)pi.a * pd.i1 + pi.b) * kStageBytes;
            pf_s = 0; pf_left = pi.c;
          }
          if (pf_end) return;
          const int n = min(8, pf_left - pf_s);
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(pf_src + (size_t)pf_s * kStageBytes), "r"(n * kStageBytes) : "memory");
          pf_s += n; pf_issued += n;
        }
      };
      pf_step();
      Instr next = list[0];
      for (int ip = 0; ip < p.max_instrs && ok; ++ip) {
        const Instr ins = next;
        if (ins.op == OP_END) break;
        if (ip + 1 < p.max_instrs) next = list[ip + 1];  // in flight while this instruction's stages are issued
        if (ins.op != OP_GEMV) continue;
        const Desc& d = p.descs[ins.desc];
        const uint8_t* src = (const uint8_t*)d.p0 + ((size_t)ins.a * d.i1 + ins.b) * kStageBytes;
        Ctx tc; tc.p = &p; tc.ip = ip;
        trace_mark(tc, 40);  // producer: first stage of this instruction about to be requested
        for (int s = 0; s < ins.c; ++s) {
          if (s == 8) trace_mark(tc, 41);  // producer: 8 stages requested
          ok = mbar_spin_bounded(&sm->empty[stage], phase ^ 1, p.status);
          if (!ok) break;
          mbar_expect_tx(&sm->full[stage], kStageBytes);
          bulk_load_1d(ring + (size_t)stage * kStageBytes, src + (size_t)s * kStageBytes, kStageBytes, &sm->full[stage]);
          if (++stage == ns) { stage = 0; phase ^= 1; }
          ++main_issued;
          if ((main_issued & 3) == 0) pf_step();
        }
        trace_mark(tc, 42);  // producer: all stages of this instruction requested
      }
    }
  } else {
    // ------------------------------------------------------------------------------------------ consumer warps
    Ctx c;
    c.p = &p; c.ring = ring; c.xs = xs; c.sm = sm;
    c.rec = p.rec + p.step_parity; c.rec_next = p.rec + (p.step_parity ^ 1);
    c.ns = ns; c.nb = nb; c.stage = 0; c.phase = 0; c.seg = 0; c.nload = 0; c.tmem = sm->tmem_base; c.barrier_target = p.barrier_base; c.ip = 0;
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
      c.ip = ip;
      trace_mark(c, 1);  // instruction start (op code = instrs[ip].op)
      switch (ins.op) {
        case OP_GEMV: op_gemv(c, ins); break;
        case OP_BARRIER: grid_barrier(c); break;
        case OP_EMBED: op_embed(c, ins); break;
        case OP_ZERO: op_zero(c, ins); break;
        case OP_COPY: op_copy(c, ins); break;
        case OP_QUANT: op_quant(c, ins); break;
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
    c.ip = p.max_instrs;
    trace_mark(c, 2);  // list finished
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
