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

// FP4 term expansion of 16 activations in packed-half arithmetic with no conversion instructions (f32 <-> fp8/fp4 `cvt`
// runs on the low-rate XU pipe). The 16 values arrive as 8 half2 with the pairing (k, k + 4) inside each group of 8.
// Every term uses the UNIFORM part of the e2m1 grid, {0, +-0.5, .. +-2} (codes 0..4 are linear in the magnitude):
// scale s = ceil_e4m3(max|r| / 2 * 4^term), q = rint(2 r 4^term / s) in [-4, 4], residual r -= q s / (2 * 4^term): a
// term removes exactly 3 bits. Rounding uses the 1536.0 magic constant of f16.
__device__ __forceinline__ void quantize_block_h2(__half2 (&x)[8], int terms, int tpad, int row, int blk, int nb, uint8_t* B,
                                                  uint8_t* SFB) {
  const __half2 magic = __float2half2_rn(1536.f);
  float gain = 1.f, inv_gain = 1.f;  // 4^term and its inverse
  for (int term = 0; term < terms; ++term) {
    __half2 m2 = __habs2(x[0]);
#pragma unroll
    for (int i = 1; i < 8; ++i) m2 = __hmax2(m2, __habs2(x[i]));
    const float amax = fmaxf(__low2float(m2), __high2float(m2));
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
    uint32_t nib[4][2];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __half2 p = __hmul2(x[i], inv2);
      const __half2 ta = __hadd2(__habs2(p), magic);  // low mantissa bits = rint(|p|) in 0..4
      const uint32_t pb = h2u(p), tb = h2u(ta);
      const uint32_t n2 = (tb & 0x00070007u) | ((pb >> 12) & 0x00080008u);  // sign-magnitude code per half
      const uint32_t qs = h2u(__hsub2(ta, magic)) | (pb & 0x80008000u);     // signed q as half2
      x[i] = __hfma2(u2h(qs), nhb, x[i]);
      nib[i & 3][i >> 2] = n2;
    }
    // word of a group of 8 values: low 16 bits = nibbles of k 0..3, high 16 bits = nibbles of k 4..7
    const uint32_t w0 = nib[0][0] + 16u * nib[1][0] + 256u * nib[2][0] + 4096u * nib[3][0];
    const uint32_t w1 = nib[0][1] + 16u * nib[1][1] + 256u * nib[2][1] + 4096u * nib[3][1];
    const int n = term * tpad + row;
    *(uint2*)(B + ((size_t)(blk >> 1) * (nb >> 3) + (n >> 3)) * 128 + (n & 7) * 16 + (blk & 1) * 8) = make_uint2(w0, w1);
    SFB[(size_t)(blk >> 2) * nb * 16 + n * 16 + (blk & 3)] = (uint8_t)code;
    gain *= 4.f;
    inv_gain *= 0.25f;
  }
}

// 16 consecutive floats (already scaled) -> 8 half2 with the (k, k + 4) pairing inside each group of 8
__device__ __forceinline__ void pack_pairs(const float4 (&v)[4], float f, __half2 (&h)[8]) {
  h[0] = __floats2half2_rn(v[0].x * f, v[1].x * f); h[1] = __floats2half2_rn(v[0].y * f, v[1].y * f);
  h[2] = __floats2half2_rn(v[0].z * f, v[1].z * f); h[3] = __floats2half2_rn(v[0].w * f, v[1].w * f);
  h[4] = __floats2half2_rn(v[2].x * f, v[3].x * f); h[5] = __floats2half2_rn(v[2].y * f, v[3].y * f);
  h[6] = __floats2half2_rn(v[2].z * f, v[3].z * f); h[7] = __floats2half2_rn(v[2].w * f, v[3].w * f);
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
  const int tid = threadIdx.x;
  const int pro = d.i5;
  const float* in = (const float*)d.p1;
  if ((d.i7 & 1) && pro != PRO_GDN_NORM) in += (size_t)rec->parity * d.i8;
  const float* zbase = (const float*)d.p2;
  if (pro == PRO_GDN_NORM && (d.i7 & 1)) zbase += (size_t)rec->parity * d.i8;
  uint8_t* B = (uint8_t*)d.p5;
  uint8_t* SFB = (uint8_t*)d.p6;
  float* stats = (float*)d.p7;
  const int items = count * tpad * 8;  // (unit, row, block of the unit): 8 consecutive lanes share (unit, row)
  for (int idx = tid; idx < ((items + 31) & ~31); idx += nthreads) {
    const bool live = idx < items;
    const int unit = first + idx / (tpad * 8), row = (idx >> 3) % tpad, blk = unit * 8 + (idx & 7);
    const int k = blk * 16;
    const bool valid = live && row < T;
    float4 x[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    float ssq = 0.f;
    if (valid) {
      const float* src = (pro == PRO_GDN_NORM ? (const float*)d.p1 : in) + (size_t)row * d.i3 + k;
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = __ldcg((const float4*)src + i);
      if (pro == PRO_NORM) {
        const float4* w4 = (const float4*)((const float*)d.p2 + k);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 w = __ldg(w4 + i);
          ssq += x[i].x * x[i].x + x[i].y * x[i].y + x[i].z * x[i].z + x[i].w * x[i].w;
          x[i].x *= 1.f + w.x; x[i].y *= 1.f + w.y; x[i].z *= 1.f + w.z; x[i].w *= 1.f + w.w;
        }
      } else if (pro == PRO_SWIGLU) {
        const float4* u4 = (const float4*)(in + (size_t)row * d.i3 + k + d.i0);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 u = __ldcg(u4 + i);
          x[i].x = silu_f(x[i].x) * u.x; x[i].y = silu_f(x[i].y) * u.y; x[i].z = silu_f(x[i].z) * u.z; x[i].w = silu_f(x[i].w) * u.w;
        }
      } else if (pro == PRO_GDN_NORM) {
        const float4* z4 = (const float4*)(zbase + (size_t)row * d.i9 + k);
        const float4* w4 = (const float4*)((const float*)d.p3 + (k & 127));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 z = __ldcg(z4 + i), w = __ldg(w4 + i);
          ssq += x[i].x * x[i].x + x[i].y * x[i].y + x[i].z * x[i].z + x[i].w * x[i].w;
          x[i].x *= w.x * silu_f(z.x); x[i].y *= w.y * silu_f(z.y); x[i].z *= w.z * silu_f(z.z); x[i].w *= w.w * silu_f(z.w);
        }
      }
    }
    // reduce the sum of squares over the 8 lanes of this (unit, row)
    ssq += __shfl_xor_sync(0xffffffffu, ssq, 1);
    ssq += __shfl_xor_sync(0xffffffffu, ssq, 2);
    ssq += __shfl_xor_sync(0xffffffffu, ssq, 4);
    float f = kPreGain;
    if (pro == PRO_GDN_NORM) f *= rsqrtf(ssq * (1.f / 128.f) + d.f1);
    if (pro == PRO_NORM && valid && (idx & 7) == 0) atomicAdd(stats + row, ssq);
    if (live) {
      __half2 h[8];
      pack_pairs(x, f, h);
      quantize_block_h2(h, terms, tpad, row, blk, nb, B, SFB);
    }
  }
  // the images are read by bulk copies (async proxy) of other CTAs after the next grid barrier
  asm volatile("fence.proxy.async;" ::: "memory");
  __threadfence();
}

__device__ __forceinline__ void op_quant(Ctx& c, const Instr& ins) {
  quant_units(c, c.p->descs[ins.desc], ins.a, ins.b, kConsumerThreads);
}

}  // namespace mk
