// Megakernel op: Gated-DeltaNet core of one (value head, row range) item for a decode/verify block, under the
// "replay" scheme for speculative decoding (upstream rollout/blackwell/gdn/replay.py:15-35, csrc/gdn_verify.cu):
// the state slot holds the state at the START of the previous block; this step first replays the rows of the previous
// block that were committed (from that block's record of conv inputs and b/a rows), stores the state and the conv
// window at the start of the current block, then computes the current block's outputs without committing them.
//
// Desc: p0 record rows, fp32 [2 parities][T][i0]: columns [0,C) conv inputs (q | k | v), [C, C+Hv*128) z,
//          then Hv b values, then Hv a values          (i8 = floats between the two parities)
//       p2 conv weight fp32 [C][4]      p3 fp32 A_log[Hv] | dt_bias[Hv]
//       p4 state slot fp32 [Hv][128][128]   p5 conv slots fp32 [2 parities][3][C]   p6 output fp32 [T][i4]
//       i0 record row stride, i1 Hv, i2 Hk, i3 C, i4 output stride, f1 L2-norm eps
// Instr: a value head, b first row of the head, c rows (<= 64)
#pragma once

namespace mk {
using namespace pear;

constexpr int kGdnD = 128;          // key dim == value dim per head
constexpr int kGdnMaxRows = 19;     // 3 window rows + up to 8 replayed + up to 8 current
constexpr int kGdnCh = 2 * kGdnD + 64;  // q, k and up to 64 v channels staged per item

__device__ __noinline__ void op_gdn(Ctx& c, const Instr& ins) {
  const Desc& d = c.p->descs[ins.desc];
  const StepRec* rec = c.rec;
  const int T = rec->T, R = rec->n_replay, par = rec->parity;
  const int hv = ins.a, row0 = ins.b, nrows = ins.c;
  const int Hv = d.i1, Hk = d.i2, C = d.i3, rstride = d.i0;
  const int hk = hv / (Hv / Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const float* rec_cur = (const float*)d.p0 + (size_t)par * d.i8;
  const float* rec_prev = (const float*)d.p0 + (size_t)(par ^ 1) * d.i8;
  const float* conv_w = (const float*)d.p2;
  const float* conv_rd = (const float*)d.p5 + (size_t)(par ^ 1) * 3 * C;
  float* conv_wr = (float*)d.p5 + (size_t)par * 3 * C;
  const int nseq = R + T;  // rows of the extended sequence that get a conv output

  consumer_sync();
  trace_mark(c, 55);  // gdn: op entered, scratch free
  float* xin = (float*)c.xs;                       // [3 + nseq][kGdnCh]
  float* u = xin + kGdnMaxRows * kGdnCh;           // [nseq][kGdnCh]
  float* dec = u + 16 * kGdnCh;                    // [16] exp(g)
  float* beta = dec + 16;                          // [16]

  // ---- stage the conv inputs of this item's channels, q(128) k(128) v(nrows), the conv weights and the gates:
  // every global load is issued before the first use (one L2 round trip for the whole staging)
  const int nch = 2 * kGdnD + nrows;
  auto gch_of = [&](int ch) {
    return ch < kGdnD ? hk * kGdnD + ch
         : ch < 2 * kGdnD ? Hk * kGdnD + hk * kGdnD + (ch - kGdnD)
                          : 2 * Hk * kGdnD + hv * kGdnD + row0 + (ch - 2 * kGdnD);
  };
  // Compact code on purpose: the megakernel's code is far larger than the instruction caches, so every op starts cold
  // and its cost is the number of instruction-cache lines it touches, not its arithmetic. All loops over rows are rolled;
  // the input columns go global -> shared with 4-byte asynchronous copies (all in flight at once without unrolling),
  // and no index is divided: a thread owns up to two channels of the item.
  {
    int gchs[2];
    bool okc[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int ch = tid + e * kConsumerThreads;
      okc[e] = ch < nch;
      gchs[e] = okc[e] ? gch_of(ch) : 0;
    }
#pragma unroll 1
    for (int r = 0; r < 3 + nseq; ++r) {
      const float* row = r < 3 ? conv_rd + (size_t)r * C : r < 3 + R ? rec_prev + (size_t)(r - 3) * rstride : rec_cur + (size_t)(r - 3 - R) * rstride;
#pragma unroll
      for (int e = 0; e < 2; ++e)
        if (okc[e])
          asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(xin + r * kGdnCh + tid + e * kConsumerThreads)), "l"(row + gchs[e]) : "memory");
    }
    float4 wv[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) wv[e] = okc[e] ? __ldg((const float4*)(conv_w + (size_t)gchs[e] * 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
    float gb = 0.f, ga = 0.f, A_log = 0.f, dt_bias = 0.f;
    if (tid < nseq) {
      const float* row = tid < R ? rec_prev + (size_t)tid * rstride : rec_cur + (size_t)(tid - R) * rstride;
      gb = __ldcg(row + C + Hv * kGdnD + hv);
      ga = __ldcg(row + C + Hv * kGdnD + Hv + hv);
      A_log = __ldg((const float*)d.p3 + hv);
      dt_bias = __ldg((const float*)d.p3 + Hv + hv);
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    trace_mark(c, 56);  // gdn: input columns in shared memory (this thread's)
    const bool qk_writer = (hv % (Hv / Hk) == 0) && row0 == 0;
    // a thread reads back only what it copied itself: no barrier needed before the convolution
#pragma unroll 1
    for (int r = 0; r < nseq; ++r) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        if (!okc[e]) continue;
        const float* x = xin + r * kGdnCh + tid + e * kConsumerThreads;
        const float acc = wv[e].x * x[0] + wv[e].y * x[kGdnCh] + wv[e].z * x[2 * kGdnCh] + wv[e].w * x[3 * kGdnCh];
        u[r * kGdnCh + tid + e * kConsumerThreads] = silu_f(acc);
      }
    }
    // conv window for the next step: rows [R, R + 3) of the extended sequence
#pragma unroll 1
    for (int w = 0; w < 3; ++w) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int ch = tid + e * kConsumerThreads;
        if (okc[e] && (ch >= 2 * kGdnD || qk_writer)) conv_wr[(size_t)w * C + gchs[e]] = xin[(R + w) * kGdnCh + ch];
      }
    }
    if (tid < nseq) {
      dec[tid] = __expf(-__expf(A_log) * softplus_f(ga + dt_bias));
      beta[tid] = sigmoid_f(gb);
    }
  }
  consumer_sync();
  trace_mark(c, 51);  // gdn: conv done
  // ---- L2 norm of q (scaled by D^-0.5) and k per row: one warp per (row, q|k)
#pragma unroll 1
  for (int item = warp; item < 2 * nseq; item += kConsumerWarps) {
    float* v = u + (item >> 1) * kGdnCh + (item & 1) * kGdnD;
    float4 x = *(float4*)(v + lane * 4);
    float s = warp_sum(x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w);
    float r = rsqrtf(s + d.f1) * ((item & 1) ? 1.f : 0.08838834764831845f);
    x.x *= r; x.y *= r; x.z *= r; x.w *= r;
    *(float4*)(v + lane * 4) = x;
  }
  consumer_sync();
  trace_mark(c, 52);  // gdn: q, k normalised

  // ---- recurrence: thread (row = tid / 4, kq = tid % 4) owns columns {16 i + 4 kq .. + 3 : i = 0..7} of its row
  const int r = tid >> 2, kq = tid & 3;
  const bool active = r < nrows;
  float S[32];
  float* srow = (float*)d.p4 + ((size_t)hv * kGdnD + row0 + (active ? r : 0)) * kGdnD;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float4 v = active ? __ldcg((const float4*)(srow + 16 * i + 4 * kq)) : make_float4(0.f, 0.f, 0.f, 0.f);
    S[4 * i] = v.x; S[4 * i + 1] = v.y; S[4 * i + 2] = v.z; S[4 * i + 3] = v.w;
  }
  float* out = (float*)d.p6;
  trace_mark(c, 53);  // gdn: state rows loaded (issued)
#pragma unroll 1
  for (int s = 0; s < nseq; ++s) {
    if (s == R && active) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        *(float4*)(srow + 16 * i + 4 * kq) = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
    }
    const float* qs = u + s * kGdnCh;
    const float* ks = qs + kGdnD;
    const float vv = active ? qs[2 * kGdnD + r] : 0.f;
    const float de = dec[s], be = beta[s];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 k4 = *(const float4*)(ks + 16 * i + 4 * kq);
      S[4 * i] *= de; S[4 * i + 1] *= de; S[4 * i + 2] *= de; S[4 * i + 3] *= de;
      dot += S[4 * i] * k4.x + S[4 * i + 1] * k4.y + S[4 * i + 2] * k4.z + S[4 * i + 3] * k4.w;
    }
    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    dot += __shfl_xor_sync(0xffffffffu, dot, 2);
    const float uu = (vv - dot) * be;
    float o = 0.f;
    const bool want_out = s >= R;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 k4 = *(const float4*)(ks + 16 * i + 4 * kq);
      S[4 * i] += uu * k4.x; S[4 * i + 1] += uu * k4.y; S[4 * i + 2] += uu * k4.z; S[4 * i + 3] += uu * k4.w;
      if (want_out) {
        const float4 q4 = *(const float4*)(qs + 16 * i + 4 * kq);
        o += S[4 * i] * q4.x + S[4 * i + 1] * q4.y + S[4 * i + 2] * q4.z + S[4 * i + 3] * q4.w;
      }
    }
    if (want_out) {
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (active && kq == 0) out[(size_t)(s - R) * d.i4 + hv * kGdnD + row0 + r] = o;
    }
  }
  trace_mark(c, 54);  // gdn: recurrence done
  if (R == nseq && active) {  // T == 0 never happens; kept for completeness when a block is replay-only
#pragma unroll
    for (int i = 0; i < 8; ++i)
      *(float4*)(srow + 16 * i + 4 * kq) = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
  }
  if (d.pad[0] > 0) {
    // The head's outputs feed the output projection: the item that completes the head (its last row part) builds that
    // GEMV's operand unit (one head of 128 values = one unit) instead of a quantisation phase of its own.
    const Desc& cd = c.p->descs[d.pad[0] - 1];
    __threadfence();
    consumer_sync();
    if (tid == 0) {
      const int slot = d.pad[1] + hv;
      const int expect = __ldg(c.p->tile_expect + slot);
      const bool last = expect > 0 && atomicAdd(c.p->tile_cnt + slot, 1) + 1 == expect;
      if (last) c.p->tile_cnt[slot] = 0;
      c.sm->fin_unit = last ? hv : -1;
    }
    consumer_sync();
    const int unit = *(volatile int*)&c.sm->fin_unit;
    if (unit >= 0) {
      __threadfence();
      quant_units(c, cd, unit, 1, kConsumerThreads);
    }
    consumer_sync();  // fin_unit is rewritten by the next item
  }
}

}  // namespace mk
