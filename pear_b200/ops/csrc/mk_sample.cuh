// Megakernel ops: speculative verify sampling, bookkeeping, drafter inputs and draft argmax.
//
// Sampling is temperature-only with the exponential race (argmax of logit/T + Gumbel noise, Philox4x32-10 noise keyed
// by seed/step/row/vocab index). Drafts are greedy, so the lossless acceptance rule is `u < p_target(draft)` and a
// rejected position resamples from the target distribution with the draft token removed (upstream
// rollout/blackwell/csrc/verify_sampler.cu; rollout/sampler.py:105-125). Each row's race is run with its draft
// excluded up front, so acceptance only has to pick which row's winner is emitted.
//
// SAMPLE desc: p0 logits fp32 [T][i0], p1 prompt tokens int32 (prefill bookkeeping), p4 partials fp32 [8][i3][4]
//              i0 logits stride, i1 vocab, i2 chunk (multiple of 1024), i3 chunks, i4 draft tokens per step,
//              i5 prompt length, i6 mode (0 decode, 1 prefill bookkeeping), i9 mask token id
// DRAFT_IN desc: p0 embedding table bf16 [V][H], p1 target residual rows fp32 [T][i3], p2 fp32 norm_e w[H] | norm_h w[H],
//              p4 out fp32 [8][2H], p5 prompt tokens, i0 H, i3 residual row stride, i5 mask token id, i6 mode, f1 eps
// ARGMAX desc: p0 drafter logits fp32 [8][i0], p4 partials fp32 [8][i3][2], i0 stride, i1 vocab, i2 chunk, i3 chunks,
//              i4 draft tokens per step
#pragma once

namespace mk {
using namespace pear;

__device__ __forceinline__ float step_temperature(const Ctx& c) { return c.p->ctrl ? c.p->ctrl->temperature : c.p->temperature; }
__device__ __forceinline__ uint32_t step_seed(const Ctx& c) { return c.p->ctrl ? c.p->ctrl->seed : c.p->seed; }

__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
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
__device__ __forceinline__ float u01(uint32_t x) { return ((float)(x >> 9) + 0.5f) * (1.0f / 8388608.0f); }
__device__ __forceinline__ float gumbel(uint32_t x) { return -__logf(-__logf(u01(x))); }

// merge (max, sum of exp relative to max)
__device__ __forceinline__ void ms_merge(float& m, float& s, float m2, float s2) {
  const float mn = fmaxf(m, m2);
  if (mn == -INFINITY) { m = mn; s = 0.f; return; }
  s = s * __expf(m - mn) + s2 * __expf(m2 - mn);
  m = mn;
}

__device__ __noinline__ void op_sample_part(Ctx& c, const Instr& ins) {
  const Desc& d = c.p->descs[ins.desc];
  const StepRec* rec = c.rec;
  const int T = rec->T, V = d.i1, chunk = d.i2, nchunks = d.i3;
  const float inv_t = 1.f / step_temperature(c);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float* part = (float*)d.p4;
  for (int ch = ins.a; ch < ins.a + ins.b; ++ch) {
    for (int r = 0; r < T; ++r) {
      const float* row = (const float*)d.p0 + (size_t)r * d.i0;
      const int excl = (r < T - 1) ? rec->tokens[r + 1] : -1;
      float m = -INFINITY, s = 0.f, best = -INFINITY;
      int bidx = 0x7fffffff;
      for (int i = ch * chunk + tid * 4; i < min(V, (ch + 1) * chunk); i += kConsumerThreads * 4) {
        const float4 z4 = __ldcg((const float4*)(row + i));
        const uint4 rnd = philox4x32_10(make_uint4((uint32_t)(i >> 2), (uint32_t)r, (uint32_t)rec->step, 0u),
                                        make_uint2(step_seed(c), 0x5eedu));
        const float z[4] = {z4.x * inv_t, z4.y * inv_t, z4.z * inv_t, z4.w * inv_t};
        const uint32_t rr[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (i + e < V) {
            ms_merge(m, s, z[e], 1.f);
            const float key = z[e] + gumbel(rr[e]);
            if (i + e != excl && (key > best || (key == best && i + e < bidx))) { best = key; bidx = i + e; }
          }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
        const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, bidx, o);
        ms_merge(m, s, m2, s2);
        if (b2 > best || (b2 == best && i2 < bidx)) { best = b2; bidx = i2; }
      }
      consumer_sync();
      if (lane == 0) {
        c.sm->red[warp * 4 + 0] = m; c.sm->red[warp * 4 + 1] = s; c.sm->red[warp * 4 + 2] = best;
        c.sm->red[warp * 4 + 3] = __int_as_float(bidx);
      }
      consumer_sync();
      if (tid == 0) {
        for (int w = 1; w < kConsumerWarps; ++w) {
          ms_merge(m, s, c.sm->red[w * 4], c.sm->red[w * 4 + 1]);
          const float b2 = c.sm->red[w * 4 + 2];
          const int i2 = __float_as_int(c.sm->red[w * 4 + 3]);
          if (b2 > best || (b2 == best && i2 < bidx)) { best = b2; bidx = i2; }
        }
        float* p = part + ((size_t)r * nchunks + ch) * 4;
        p[0] = m; p[1] = s; p[2] = best; p[3] = __int_as_float(bidx);
      }
    }
  }
}

// Record of the next step for a prefill block: the prompt supplies the tokens.
__device__ __forceinline__ void book_prefill(Ctx& c, const Desc& d) {
  const StepRec* rec = c.rec;
  StepRec* nx = c.rec_next;
  const int* prompt = (const int*)d.p1;
  const int P = d.i5;
  const int pos = rec->pos0 + rec->T;
  nx->pos0 = pos; nx->n_replay = rec->T; nx->parity = rec->parity ^ 1; nx->step = rec->step + 1;
  nx->n_out_total = rec->n_out_total; nx->rows_draft = rec->T; nx->n_acc = rec->T - 1;
  const int left = (P - 1) - pos;  // prompt tokens still to prefill (the last prompt token opens the first decode step)
  if (left > 0) {
    nx->mode = 1; nx->T = min(8, left);
    for (int i = 0; i < nx->T; ++i) nx->tokens[i] = prompt[pos + i];
  } else {
    nx->mode = 0; nx->T = 1;
    nx->tokens[0] = prompt[P - 1];
  }
}

__device__ __noinline__ void op_sample_fin(Ctx& c, const Instr& ins) {
  const Desc& d = c.p->descs[ins.desc];
  const StepRec* rec = c.rec;
  StepRec* nx = c.rec_next;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (d.i6 == 1) {
    if (tid == 0) book_prefill(c, d);
    return;
  }
  const int T = rec->T, nchunks = d.i3;
  const float inv_t = 1.f / step_temperature(c);
  const float* part = (const float*)d.p4;
  float* lse_s = c.sm->red;        // [8]
  float* best_s = c.sm->red + 8;   // [8] (int bits)
  consumer_sync();
  if (warp < T) {
    float m = -INFINITY, s = 0.f, best = -INFINITY;
    int bidx = 0x7fffffff;
    for (int ch = lane; ch < nchunks; ch += 32) {
      const float4 p = __ldcg((const float4*)(part + ((size_t)warp * nchunks + ch) * 4));
      ms_merge(m, s, p.x, p.y);
      const int i2 = __float_as_int(p.w);
      if (p.z > best || (p.z == best && i2 < bidx)) { best = p.z; bidx = i2; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
      const int i2 = __shfl_xor_sync(0xffffffffu, bidx, o);
      ms_merge(m, s, m2, s2);
      if (b2 > best || (b2 == best && i2 < bidx)) { best = b2; bidx = i2; }
    }
    if (lane == 0) { lse_s[warp] = m + __logf(s); best_s[warp] = __int_as_float(bidx); }
  }
  consumer_sync();
  if (tid == 0) {
    const float* logits = (const float*)d.p0;
    int n_acc = 0;
    for (int r = 0; r < T - 1; ++r) {
      const int dtok = min(max(rec->tokens[r + 1], 0), c.p->vocab - 1);
      const float lp = __ldcg(logits + (size_t)r * d.i0 + dtok) * inv_t - lse_s[r];
      const uint4 rnd = philox4x32_10(make_uint4(0xffffffffu, (uint32_t)r, (uint32_t)rec->step, 1u),
                                      make_uint2(step_seed(c), 0x5eedu));
      if (__logf(u01(rnd.x)) < lp) ++n_acc; else break;
    }
    const int y = __float_as_int(best_s[n_acc]);
    StepOut* o = c.p->out_ring + (rec->step % c.p->ring);
    o->step = rec->step; o->n_out = n_acc + 1; o->n_accept = n_acc; o->pos0 = rec->pos0;
    for (int i = 0; i < n_acc; ++i) o->tokens[i] = rec->tokens[i + 1];
    o->tokens[n_acc] = y;
    o->logprobs[0] = __ldcg(logits + (size_t)n_acc * d.i0 + y) * inv_t - lse_s[n_acc];
    const int nd = d.i4;
    nx->T = 1 + nd; nx->pos0 = rec->pos0 + n_acc + 1; nx->n_replay = n_acc + 1; nx->parity = rec->parity ^ 1;
    nx->step = rec->step + 1; nx->mode = 0; nx->n_out_total = rec->n_out_total + n_acc + 1;
    nx->rows_draft = n_acc + 1 + (nd > 0 ? nd - 1 : 0); nx->n_acc = n_acc;
    nx->tokens[0] = y;
    for (int i = 1; i < 8; ++i) nx->tokens[i] = d.i9;
  }
}

// Drafter input row `a`: [norm_e(embed(next token)) | norm_h(target residual row)]
__device__ __noinline__ void op_draft_in(Ctx& c, const Instr& ins) {
  const Desc& d = c.p->descs[ins.desc];
  const StepRec* rec = c.rec;
  const StepRec* nx = c.rec_next;
  const int row = ins.a, H = d.i0, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (row >= nx->rows_draft) return;
  int tok, src;
  if (d.i6 == 1) {
    const int* prompt = (const int*)d.p5;
    tok = prompt[rec->pos0 + row + 1]; src = row;
  } else {
    const int n_acc = nx->n_acc;
    if (row <= n_acc) { tok = row < n_acc ? rec->tokens[row + 1] : nx->tokens[0]; src = row; }
    else { tok = d.i5; src = n_acc; }
  }
  tok = min(max(tok, 0), c.p->vocab - 1);
  const __nv_bfloat16* e = (const __nv_bfloat16*)d.p0 + (size_t)tok * H;
  const float* hrow = (const float*)d.p1 + (size_t)src * d.i3;
  const float* w = (const float*)d.p2;
  float* out = (float*)d.p4 + (size_t)row * 2 * H;
  float se = 0.f, sh = 0.f;
  for (int i = tid; i < H; i += kConsumerThreads) {
    const float a = __bfloat162float(e[i]), b = __ldcg(hrow + i);
    se += a * a; sh += b * b;
  }
  se = warp_sum(se); sh = warp_sum(sh);
  consumer_sync();
  if (lane == 0) { c.sm->red[warp] = se; c.sm->red[16 + warp] = sh; }
  consumer_sync();
  float te = 0.f, th = 0.f;
  for (int i = 0; i < kConsumerWarps; ++i) { te += c.sm->red[i]; th += c.sm->red[16 + i]; }
  const float re = rsqrtf(te / (float)H + d.f1), rh = rsqrtf(th / (float)H + d.f1);
  for (int i = tid; i < H; i += kConsumerThreads) {
    out[i] = __bfloat162float(e[i]) * re * (1.f + w[i]);
    out[H + i] = __ldcg(hrow + i) * rh * (1.f + w[H + i]);
  }
  consumer_sync();
}

__device__ __noinline__ void op_argmax_part(Ctx& c, const Instr& ins) {
  const Desc& d = c.p->descs[ins.desc];
  const StepRec* nx = c.rec_next;
  const int V = d.i1, chunk = d.i2, nchunks = d.i3, nd = d.i4;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float* part = (float*)d.p4;
  for (int ch = ins.a; ch < ins.a + ins.b; ++ch) {
    for (int k = 0; k < nd; ++k) {
      const float* row = (const float*)d.p0 + (size_t)(nx->n_acc + k) * d.i0;
      float best = -INFINITY;
      int bidx = 0x7fffffff;
      for (int i = ch * chunk + tid * 4; i < min(V, (ch + 1) * chunk); i += kConsumerThreads * 4) {
        const float4 z4 = __ldcg((const float4*)(row + i));
        const float z[4] = {z4.x, z4.y, z4.z, z4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (i + e < V && (z[e] > best || (z[e] == best && i + e < bidx))) { best = z[e]; bidx = i + e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, bidx, o);
        if (b2 > best || (b2 == best && i2 < bidx)) { best = b2; bidx = i2; }
      }
      consumer_sync();
      if (lane == 0) { c.sm->red[warp * 2] = best; c.sm->red[warp * 2 + 1] = __int_as_float(bidx); }
      consumer_sync();
      if (tid == 0) {
        for (int w = 1; w < kConsumerWarps; ++w) {
          const float b2 = c.sm->red[w * 2];
          const int i2 = __float_as_int(c.sm->red[w * 2 + 1]);
          if (b2 > best || (b2 == best && i2 < bidx)) { best = b2; bidx = i2; }
        }
        float* p = part + ((size_t)k * nchunks + ch) * 2;
        p[0] = best; p[1] = __int_as_float(bidx);
      }
    }
  }
}

__device__ __noinline__ void op_argmax_fin(Ctx& c, const Instr& ins) {
  const Desc& d = c.p->descs[ins.desc];
  StepRec* nx = c.rec_next;
  const int nchunks = d.i3, nd = d.i4;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* part = (const float*)d.p4;
  if (warp < nd) {
    float best = -INFINITY;
    int bidx = 0x7fffffff;
    for (int ch = lane; ch < nchunks; ch += 32) {
      const float b2 = __ldcg(part + ((size_t)warp * nchunks + ch) * 2);
      const int i2 = __float_as_int(__ldcg(part + ((size_t)warp * nchunks + ch) * 2 + 1));
      if (b2 > best || (b2 == best && i2 < bidx)) { best = b2; bidx = i2; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
      const int i2 = __shfl_xor_sync(0xffffffffu, bidx, o);
      if (b2 > best || (b2 == best && i2 < bidx)) { best = b2; bidx = i2; }
    }
    if (lane == 0) nx->tokens[1 + warp] = bidx;
  }
}

}  // namespace mk
