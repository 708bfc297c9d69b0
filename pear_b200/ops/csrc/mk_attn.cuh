// Megakernel ops: split-KV paged attention of a decode/verify block (T <= 8 query rows per sequence) and the combine.
//
// OP_ATTN item = (kv head h, split s of n): all G*T query rows of the kv head's group against keys
// [s*chunk, (s+1)*chunk) of the cache; the LAST split also takes the block's own T keys (causal), which it first
// normalises, rotates and writes into the cache. Per 64-key tile: S = Q K^T on mma.sync (K fragments straight from
// global/L2, 8 keys per warp), online softmax per row through shared memory, O += P V on mma.sync with V staged by
// cp.async and read with ldmatrix.trans; every warp owns D/8 output dims for all rows. Partials (o, m, l) go to
// global; OP_ATTN_COMBINE merges the splits and applies the sigmoid output gate.
// (Counterpart of upstream deploy/blackwell/nvfp4/csrc/attention.cuh and rollout/blackwell/csrc/verify_attn.cu.)
//
// Desc: p0 qkv rows fp32 [T][i0]: per q head [q(D) | gate(D)] x Hq, then k (Hkv x D), then v (Hkv x D)
//       p1 k cache bf16, p2 v cache bf16: [blocks][i6 tokens][Hkv][D]     p7 block table int32 (null: identity)
//       p3 fp32 q_norm w[D] | k_norm w[D]    p4 partials fp32 [T*Hq][i4][D+2]   p5 fp32 inv_freq[i5/2]
//       p6 gated output fp32 [T][Hq*D] (combine)
//       i0 row stride, i1 Hkv, i2 Hq, i3 D, i4 max splits, i5 rotary dim (64), i6 block size in tokens,
//       i7 & 8: rows come from the drafter's row count, i9 gate present (1) or not (0: q heads are [q(D)] only)
//       f0 softmax scale, f1 norm eps
#pragma once

namespace mk {
using namespace pear;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(smem_u32(p)));
}


__device__ __forceinline__ size_t kv_offset(const Desc& d, int pos, int h) {
  const int bs = d.i6;
  int blk = pos / bs, off = pos % bs;
  if (d.p7) blk = ((const int*)d.p7)[blk];
  return (((size_t)blk * bs + off) * d.i1 + h) * d.i3;
}

// (1+w) RMSNorm + rotary embedding of one head vector by one warp; lane holds elements lane + 32 i.
template <int D>
__device__ __forceinline__ void norm_rope_warp(const float* src, const float* w, const float* inv_freq, int pos, float eps,
                                               float (&x)[D / 32], int lane) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < D / 32; ++i) { x[i] = __ldcg(src + lane + 32 * i); s += x[i] * x[i]; }
  s = warp_sum(s);
  const float rs = rsqrtf(s / (float)D + eps);
#pragma unroll
  for (int i = 0; i < D / 32; ++i) x[i] = x[i] * rs * (1.f + w[lane + 32 * i]);
  // rotary_dim 64: pair (lane, lane + 32) lives in x[0], x[1]
  // the angle is reduced modulo 2 pi in double so that sincosf stays on its fast, stack-free path at long contexts
  double ang = (double)pos * (double)inv_freq[lane];
  ang -= 6.283185307179586 * rint(ang * 0.15915494309189535);
  float sn, cs;
  sincosf((float)ang, &sn, &cs);
  const float a = x[0], b = x[1];
  x[0] = a * cs - b * sn;
  x[1] = b * cs + a * sn;
}

template <int D>
__device__ __noinline__ void attn_item(Ctx& c, const Desc& d, int h, int split, int nsplit) {
  constexpr int QS = D + 16;     // Q row stride (halves): bytes = D*2 + 32
  constexpr int VS = D + 8;      // V row stride (halves)
  constexpr int SS = 68;         // S row stride (floats)
  constexpr int PS = 72;         // P row stride (halves)
  constexpr int NT = D / 64;     // output n-tiles (8 dims) per warp
  const int T = step_rows(c, d), pos0 = c.rec->pos0;
  const int Hkv = d.i1, Hq = d.i2, G = Hq / Hkv;
  const int M = G * T, Mt = (M + 15) >> 4;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int qw = d.i9 ? 2 * D : D;  // width of one q head in the row
  const float* rows = (const float*)d.p0;
  const __nv_bfloat16* kc = (const __nv_bfloat16*)d.p1;
  const __nv_bfloat16* vc = (const __nv_bfloat16*)d.p2;
  const float* qn = (const float*)d.p3;
  const float* kn = qn + D;
  const float* inv_freq = (const float*)d.p5;

  consumer_sync();
  __nv_bfloat16* Qs = (__nv_bfloat16*)c.xs;                 // [48][QS]
  __nv_bfloat16* Vs = Qs + 48 * QS;                          // [64][VS]
  float* Ss = (float*)(Vs + 64 * VS);                        // [48][SS]
  __nv_bfloat16* Ps = (__nv_bfloat16*)(Ss + 48 * SS);        // [48][PS]
  float* m_s = (float*)(Ps + 48 * PS);                       // [48]
  float* l_s = m_s + 48;
  float* al_s = l_s + 48;

  // ---- key range
  const int kv_len = pos0;
  int chunk = (kv_len + nsplit - 1) / nsplit;
  chunk = (chunk + 15) & ~15;
  int k_begin = min(split * chunk, kv_len), k_end = min(kv_len, k_begin + chunk);
  const bool last = (split == nsplit - 1);
  if (last) k_end = kv_len + T;  // the block's own keys

  // ---- Q rows: norm + rope -> bf16; row = tq * G + jq
  for (int row = warp; row < Mt * 16; row += kConsumerWarps) {
    float x[D / 32];
    if (row < M) {
      const int tq = row / G, jq = row % G;
      norm_rope_warp<D>(rows + (size_t)tq * d.i0 + (size_t)(h * G + jq) * qw, qn, inv_freq, pos0 + tq, d.f1, x, lane);
    } else {
#pragma unroll
      for (int i = 0; i < D / 32; ++i) x[i] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < D / 32; ++i) Qs[row * QS + lane + 32 * i] = __float2bfloat16_rn(x[i]);
  }
  // ---- the block's own K/V rows into the cache (last split only)
  if (last) {
    const float* kbase = rows + (size_t)Hq * qw;
    for (int tq = warp; tq < T; tq += kConsumerWarps) {
      float x[D / 32];
      norm_rope_warp<D>(kbase + (size_t)tq * d.i0 + h * D, kn, inv_freq, pos0 + tq, d.f1, x, lane);
      __nv_bfloat16* kd = (__nv_bfloat16*)kc + kv_offset(d, pos0 + tq, h);
      __nv_bfloat16* vd = (__nv_bfloat16*)vc + kv_offset(d, pos0 + tq, h);
      const float* vsrc = kbase + (size_t)tq * d.i0 + (size_t)Hkv * D + h * D;
#pragma unroll
      for (int i = 0; i < D / 32; ++i) {
        kd[lane + 32 * i] = __float2bfloat16_rn(x[i]);
        vd[lane + 32 * i] = __float2bfloat16_rn(__ldcg(vsrc + lane + 32 * i));
      }
    }
    __threadfence_block();
  }
  if (tid < 48) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; al_s[tid] = 1.f; }
  float O[3][NT][4];
#pragma unroll
  for (int a = 0; a < 3; ++a)
#pragma unroll
    for (int b = 0; b < NT; ++b)
#pragma unroll
      for (int e = 0; e < 4; ++e) O[a][b][e] = 0.f;
  consumer_sync();

  // K fragments of this warp's 8 keys of a tile, straight from global; the next tile's are prefetched
  uint2 kb[D / 16], kb_next[D / 16];
  if (k_begin < k_end) {
    const __nv_bfloat16* krow = kc + kv_offset(d, min(k_begin + warp * 8 + g, k_end - 1), h);
#pragma unroll
    for (int j = 0; j < D / 16; ++j) kb[j] = __ldcg((const uint2*)(krow + 16 * j + 4 * t4));
  }
  for (int kt = k_begin; kt < k_end; kt += 64) {
    // ---- V tile (64 keys) by cp.async
    for (int idx = tid; idx < 64 * (D / 8); idx += kConsumerThreads) {
      const int key = idx / (D / 8), part = idx % (D / 8);
      const int kp = min(kt + key, k_end - 1);
      cp_async16(Vs + key * VS + part * 8, vc + kv_offset(d, kp, h) + part * 8);
    }
    // ---- S = Q K^T for this warp's 8 keys; K fragments straight from global
    {
      if (kt + 64 < k_end) {
        const __nv_bfloat16* krow = kc + kv_offset(d, min(kt + 64 + warp * 8 + g, k_end - 1), h);
#pragma unroll
        for (int j = 0; j < D / 16; ++j) kb_next[j] = __ldcg((const uint2*)(krow + 16 * j + 4 * t4));
      }
#pragma unroll
      for (int mi = 0; mi < 3; ++mi) {
        if (mi < Mt) {
          float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int j = 0; j < D / 16; ++j) {
            const uint2 qa = *(const uint2*)(Qs + (mi * 16 + g) * QS + 16 * j + 4 * t4);
            const uint2 qb = *(const uint2*)(Qs + (mi * 16 + g + 8) * QS + 16 * j + 4 * t4);
            mma_bf16(s, qa.x, qb.x, qa.y, qb.y, kb[j].x, kb[j].y);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int row = mi * 16 + g + (e >> 1) * 8;
            const int kk = kt + warp * 8 + 2 * t4 + (e & 1);
            const int tq = row / G;
            const bool vis = kk < k_end && kk <= pos0 + tq && row < M;
            Ss[row * SS + warp * 8 + 2 * t4 + (e & 1)] = vis ? s[e] * d.f0 : -INFINITY;
          }
        }
      }
#pragma unroll
      for (int j = 0; j < D / 16; ++j) kb[j] = kb_next[j];
    }
    consumer_sync();
    // ---- online softmax: one warp per row, two keys per lane
    for (int row = warp; row < Mt * 16; row += kConsumerWarps) {
      const float s0 = Ss[row * SS + lane], s1 = Ss[row * SS + lane + 32];
      const float mx = warp_max(fmaxf(s0, s1));
      const float mo = m_s[row];
      const float mn = fmaxf(mo, mx);
      float p0 = 0.f, p1 = 0.f, al = 1.f;
      if (mn != -INFINITY) {
        p0 = __expf(s0 - mn); p1 = __expf(s1 - mn);
        al = (mo == -INFINITY) ? 0.f : __expf(mo - mn);
      }
      Ps[row * PS + lane] = __float2bfloat16_rn(p0);
      Ps[row * PS + lane + 32] = __float2bfloat16_rn(p1);
      const float ps = warp_sum(p0 + p1);
      if (lane == 0) { m_s[row] = mn; l_s[row] = l_s[row] * al + ps; al_s[row] = al; }
    }
    cp_async_wait_all();
    consumer_sync();
    // ---- O = O * alpha + P V ; this warp's dims [warp * D/8, + D/8)
#pragma unroll
    for (int mi = 0; mi < 3; ++mi) {
      if (mi < Mt) {
        const float a0 = al_s[mi * 16 + g], a1 = al_s[mi * 16 + g + 8];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { O[mi][nt][0] *= a0; O[mi][nt][1] *= a0; O[mi][nt][2] *= a1; O[mi][nt][3] *= a1; }
      }
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {  // 4 k16 steps over the 64 keys
      uint32_t vb[NT][2];
#pragma unroll
      for (int np = 0; np < NT; np += 2) {
        // lanes 0-15: keys kk*16 + (lane & 15) of n-tile np; lanes 16-31: same keys of n-tile np + 1
        const __nv_bfloat16* p = Vs + (kk * 16 + (lane & 15)) * VS + warp * (D / 8) + (np + (lane >> 4)) * 8;
        ldmatrix_x4_trans(vb[np][0], vb[np][1], vb[np + 1][0], vb[np + 1][1], p);
      }
#pragma unroll
      for (int mi = 0; mi < 3; ++mi) {
        if (mi < Mt) {
          const uint32_t pa0 = *(const uint32_t*)(Ps + (mi * 16 + g) * PS + kk * 16 + 2 * t4);
          const uint32_t pa1 = *(const uint32_t*)(Ps + (mi * 16 + g + 8) * PS + kk * 16 + 2 * t4);
          const uint32_t pa2 = *(const uint32_t*)(Ps + (mi * 16 + g) * PS + kk * 16 + 2 * t4 + 8);
          const uint32_t pa3 = *(const uint32_t*)(Ps + (mi * 16 + g + 8) * PS + kk * 16 + 2 * t4 + 8);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) mma_bf16(O[mi][nt], pa0, pa1, pa2, pa3, vb[nt][0], vb[nt][1]);
        }
      }
    }
    consumer_sync();
  }
  // ---- partials
  float* part = (float*)d.p4;
  const int nsmax = d.i4;
#pragma unroll
  for (int mi = 0; mi < 3; ++mi) {
    if (mi < Mt) {
#pragma unroll
      for (int e2 = 0; e2 < 2; ++e2) {
        const int row = mi * 16 + g + e2 * 8;
        if (row < M) {
          const int tq = row / G, jq = row % G;
          float* dst = part + ((size_t)(tq * Hq + h * G + jq) * nsmax + split) * (D + 2);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
            *(float2*)(dst + warp * (D / 8) + nt * 8 + 2 * t4) = make_float2(O[mi][nt][e2 * 2], O[mi][nt][e2 * 2 + 1]);
        }
      }
    }
  }
  if (tid < M) {
    const int tq = tid / G, jq = tid % G;
    float* dst = part + ((size_t)(tq * Hq + h * G + jq) * nsmax + split) * (D + 2);
    dst[D] = m_s[tid];
    dst[D + 1] = l_s[tid];
  }
}

__device__ void op_attn(Ctx& c, const Instr& ins) {
  const Desc& d = c.p->descs[ins.desc];
  if (d.i3 == 256) attn_item<256>(c, d, ins.a, ins.b, ins.c);
  else attn_item<128>(c, d, ins.a, ins.b, ins.c);
}

// Combine: item = (row tq, q head) pair; one warp per pair. Output = softmax-merged o, times sigmoid(gate) if gated.
__device__ __noinline__ void op_attn_combine(Ctx& c, const Instr& ins) {
  const Desc& d = c.p->descs[ins.desc];
  const int T = step_rows(c, d);
  const int Hq = d.i2, D = d.i3, nsmax = d.i4, nsplit = ins.c;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* part = (const float*)d.p4;
  const float* rows = (const float*)d.p0;
  float* out = (float*)d.p6;
  const int qw = d.i9 ? 2 * D : D;
  for (int pair = ins.a + warp; pair < ins.a + ins.b && pair < T * Hq; pair += kConsumerWarps) {
    const int tq = pair / Hq, hq = pair % Hq;
    const float* base = part + (size_t)pair * nsmax * (D + 2);
    float mx = -INFINITY;
    for (int s = lane; s < nsplit; s += 32) mx = fmaxf(mx, __ldcg(base + (size_t)s * (D + 2) + D));
    mx = warp_max(mx);
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    float l = 0.f;
    const int per = D / 32;  // dims per lane (8 or 4), contiguous
    // Lanes first take one split each (its max and sum), then the partial outputs are accumulated split by split with the
    // weight broadcast by shuffle: no load depends on a loaded flag, so the unrolled loop keeps eight splits in flight
    // (the split-by-split version with an early `continue` paid one L2 round trip per split: ~20 us at 37 splits).
    for (int s0 = 0; s0 < nsplit; s0 += 32) {
      const int sl = s0 + lane;
      const float ms = sl < nsplit ? __ldcg(base + (size_t)sl * (D + 2) + D) : -INFINITY;
      const float ls = sl < nsplit ? __ldcg(base + (size_t)sl * (D + 2) + D + 1) : 0.f;
      const float w = ms == -INFINITY ? 0.f : __expf(ms - mx);
      l += w * ls;
      const int cnt = min(32, nsplit - s0);
#pragma unroll 8
      for (int j = 0; j < cnt; ++j) {
        const float wj = __shfl_sync(0xffffffffu, w, j);
        const float2* p = (const float2*)(base + (size_t)(s0 + j) * (D + 2) + lane * per);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (2 * i < per) {
            const float2 v = __ldcg(p + i);
            acc[2 * i] += wj > 0.f ? wj * v.x : 0.f;       // an empty split's slot may hold anything
            acc[2 * i + 1] += wj > 0.f ? wj * v.y : 0.f;
          }
        }
      }
    }
    l = warp_sum(l);
    const float inv = l > 0.f ? 1.f / l : 0.f;
    for (int i = 0; i < per; ++i) {
      float v = acc[i] * inv;
      if (d.i9) v *= sigmoid_f(__ldcg(rows + (size_t)tq * d.i0 + (size_t)hq * qw + D + lane * per + i));
      out[(size_t)tq * Hq * D + hq * D + lane * per + i] = v;
    }
  }
}

}  // namespace mk
