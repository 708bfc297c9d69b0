// Megakernel op: OP_QUANT builds the activation operand of the NEXT GEMV op, once for the whole grid.
//
// The block-scaled MMA takes 4-bit operands on both sides. The weights stay exactly NVFP4; the activations are expanded
// into a sum of FP4 terms (term i = NVFP4 quantisation of the residual of terms < i with a gain of 4^i folded into its
// block scale), laid out as extra rows of the B operand, so 4 terms give ~12 bits. Quantising inside every GEMV CTA
// would repeat the same work 148 times (and is latency bound at 8 warps per SM), so it is a phase of its own: unit u =
// K elements [128 u, 128 u + 128) of every row; one warp-row of 8 lanes per (row, unit) handles its 8 blocks of 16. The
// images land in global memory (they stay in L2) in exactly the shared-memory layout the tensor core reads; the GEMV
// CTAs pull their K range with one bulk copy each.
//
//   B image   : (chunk * (nb/8) + n/8) * 128 + (n%8) * 16 + half * 8   chunk = k/32, half = (k/16)%2, n = term * tpad + row
//   SFB image : (k/64) * nb * 16 + n * 16 + (k/16)%4                     one e4m3 scale per 16 elements
//   stats     : float[8] per GEMV descriptor: sum of squares per row (PRO_NORM; rstd is applied by the GEMV epilogue)
//
// Prologue kinds (Desc.i5 of the GEMV descriptor): PLAIN x; NORM x (1 + w) with the RMS deferred; SWIGLU silu(g) u;
// GDN_NORM o rstd_head w silu(z) (a unit is exactly one head, so the head RMS is an 8-lane shuffle reduction).
// A fixed pre-gain of 1/4 centres typical activations in e4m3's scale range: block maxima from 2^-3 to 3584 get normal
// scales, smaller blocks subnormal ones (multiples of 2^-9), larger ones clip.
#pragma once

namespace mk {
using namespace pear;

constexpr float kPreGain = 0.25f;

__device__ __forceinline__ uint32_t h2u(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u2h(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// FP4 term expansion in packed-half arithmetic with no conversion instructions (f32 <-> fp8/fp4 `cvt` runs on the
// low-rate XU pipe). A thread holds 4 consecutive activations (2 half2); the 4 lanes of a quad hold one block of 16.
// Every term uses the UNIFORM part of the e2m1 grid, {0, +-0.5, .. +-2} (codes 0..4 are linear in the magnitude):
// scale s = ceil_e4m3(max|r| / 2 * 4^term), q = rint(2 r 4^term / s) in [-4, 4], residual r -= q s / (2 * 4^term): a
// term removes exactly 3 bits. Rounding uses the 1536.0 magic constant of f16.
//
// Work layout: one WARP per (unit of 128 K elements, row): lane l holds elements [4 l, 4 l + 4) of the unit, so global
// loads are one coalesced 512-byte row segment per warp, the head / row sum of squares is a warp reduction, and the code
// is short (it runs cold at every phase: the megakernel is far larger than the instruction caches).
__device__ __forceinline__ void quantize_quad(__half2 x0, __half2 x1, int terms, int tpad, int row, int blk, int qd, int nb, uint8_t* B,
                                              uint8_t* SFB) {
  const __half2 magic = __float2half2_rn(1536.f);
  float gain = 1.f, inv_gain = 1.f;  // 4^term and its inverse
#pragma unroll 1
  for (int term = 0; term < terms; ++term) {
    __half2 m2 = __hmax2(__habs2(x0), __habs2(x1));
    float amax = fmaxf(__low2float(m2), __high2float(m2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    // scale: amax / 2 * gain rounded UP to an e4m3 value (3 mantissa bits; subnormals are multiples of 2^-9)
    const float target = fminf(amax * 0.5f * gain, 448.f);
    uint32_t code;
    float sv;
    if (target >= 0.015625f) {
      const uint32_t sbits = (__float_as_uint(target) + 0x000FFFFFu) & 0xFFF00000u;
      sv = __uint_as_float(sbits);
      code = (sbits >> 20) - 960u;  // (exponent - 120) << 3 | mantissa
    } else {
      code = max(1u, (uint32_t)ceilf(target * 512.f));
      sv = (float)code * 0.001953125f;
    }
    // clamped to the f16 range: a block of zeros with the smallest scale would otherwise give 0 * inf = NaN
    const __half2 inv2 = __float2half2_rn(fminf(__fdividef(2.f * gain, sv), 60000.f));
    const __half2 nhb = __float2half2_rn(-0.5f * sv * inv_gain);  // minus one grid step
    uint32_t nib[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      __half2& x = i == 0 ? x0 : x1;
      const __half2 p = __hmul2(x, inv2);
      const __half2 ta = __hadd2(__habs2(p), magic);  // low mantissa bits = rint(|p|) in 0..4
      const uint32_t pb = h2u(p), tb = h2u(ta);
      nib[i] = (tb & 0x00070007u) | ((pb >> 12) & 0x00080008u);          // sign-magnitude code per half
      const uint32_t qs = h2u(__hsub2(ta, magic)) | (pb & 0x80008000u);  // signed q as half2
      x = __hfma2(u2h(qs), nhb, x);
    }
    // this lane's 4 nibbles, elements in K order: two bytes of the block's eight
    const uint32_t w = (nib[0] & 0xFu) | ((nib[0] >> 12) & 0xF0u) | ((nib[1] & 0xFu) << 8) | ((nib[1] >> 4) & 0xF000u);
    const int n = term * tpad + row;
    *(uint16_t*)(B + ((size_t)(blk >> 1) * (nb >> 3) + (n >> 3)) * 128 + (n & 7) * 16 + (blk & 1) * 8 + qd * 2) = (uint16_t)w;
    if (qd == 0) SFB[(size_t)(blk >> 2) * nb * 16 + n * 16 + (blk & 3)] = (uint8_t)code;
    gain *= 4.f;
    inv_gain *= 0.25f;
  }
}

// Two callers: the OP_QUANT phase (inputs produced by a non-GEMV op), and the epilogue warps of a GEMV whose row tile
// just received its last stream-K contribution ("finishers": a row tile of 128 outputs is exactly one unit of the next
// GEMV's K, so that GEMV needs no phase of its own for its operand).
// Instr: a = first unit (128 K elements each), b = unit count; desc = the GEMV descriptor whose operand is built.
// Desc fields used: p1 input rows, p2 norm weight | z rows, p3 gated-norm weight, p5 B image, p6 SFB image, p7 stats,
//                   i0 K, i3 input row stride, i5 prologue, i7 flags, i8 parity stride, i9 z row stride, f1 eps.
// `nthreads` threads (whole warps, numbered from threadIdx 0) build units [first, first + count) of descriptor d's operand.
__device__ __noinline__ void quant_units(Ctx& c, const Desc& d, int first, int count, int nthreads) {
  const StepRec* rec = c.rec;
  const int T = step_rows(c, d);
  const int tpad = T <= 4 ? 4 : 8, nb = c.nb, terms = min(4, nb / tpad);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = nthreads >> 5;
  const int pro = d.i5;
  const float* in = (const float*)d.p1;
  if ((d.i7 & 1) && pro != PRO_GDN_NORM) in += (size_t)rec->parity * d.i8;
  const float* zbase = (const float*)d.p2;
  if (pro == PRO_GDN_NORM && (d.i7 & 1)) zbase += (size_t)rec->parity * d.i8;
  uint8_t* B = (uint8_t*)d.p5;
  uint8_t* SFB = (uint8_t*)d.p6;
  float* stats = (float*)d.p7;
#pragma unroll 1
  for (int item = warp; item < count * tpad; item += nwarps) {  // one warp per (unit, row)
    const int unit = first + item / tpad, row = item % tpad;
    const int k = unit * 128 + lane * 4;
    const bool valid = row < T;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    float ssq = 0.f;
    if (valid) {
      x = __ldcg((const float4*)(in + (size_t)row * d.i3 + k));
      if (pro == PRO_NORM) {
        const float4 w = __ldg((const float4*)((const float*)d.p2 + k));
        ssq = x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
        x.x *= 1.f + w.x; x.y *= 1.f + w.y; x.z *= 1.f + w.z; x.w *= 1.f + w.w;
      } else if (pro == PRO_SWIGLU) {
        const float4 u = __ldcg((const float4*)(in + (size_t)row * d.i3 + k + d.i0));
        x.x = silu_f(x.x) * u.x; x.y = silu_f(x.y) * u.y; x.z = silu_f(x.z) * u.z; x.w = silu_f(x.w) * u.w;
      } else if (pro == PRO_GDN_NORM) {
        const float4 z = __ldcg((const float4*)(zbase + (size_t)row * d.i9 + k));
        const float4 w = __ldg((const float4*)((const float*)d.p3 + (k & 127)));
        ssq = x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
        x.x *= w.x * silu_f(z.x); x.y *= w.y * silu_f(z.y); x.z *= w.z * silu_f(z.z); x.w *= w.w * silu_f(z.w);
      }
    }
    ssq = warp_sum(ssq);  // over the unit's 128 elements (a GDN head is exactly one unit)
    float f = kPreGain;
    if (pro == PRO_GDN_NORM) f *= rsqrtf(ssq * (1.f / 128.f) + d.f1);
    if (pro == PRO_NORM && valid && lane == 0) atomicAdd(stats + row, ssq);
    quantize_quad(__floats2half2_rn(x.x * f, x.y * f), __floats2half2_rn(x.z * f, x.w * f), terms, tpad, row, unit * 8 + (lane >> 2), lane & 3,
                  nb, B, SFB);
  }
  // the images are read by bulk copies (async proxy) of other CTAs after the next grid barrier
  asm volatile("fence.proxy.async;" ::: "memory");
  __threadfence();
}

__device__ __forceinline__ void op_quant(Ctx& c, const Instr& ins) {
  quant_units(c, c.p->descs[ins.desc], ins.a, ins.b, kConsumerThreads);
}

}  // namespace mk
