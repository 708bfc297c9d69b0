// Stand-alone kernels of the batched rollout path (the decode megakernel has its own fused versions of these for one
// session): fused sampler, rejection sampler for greedy drafts, Gated-DeltaNet recurrent decode step, split-KV paged
// decode/verify attention, embedding lookup with vision-placeholder merge, paged-KV block gather/scatter for the host
// tier. All fp32 arithmetic; every kernel is bandwidth- or latency-bound SIMT work, laid out for coalesced 16-byte
// accesses and grids that cover 148 SMs.
#include "common.cuh"

#include <cuda_bf16.h>
#include <cfloat>

namespace pear {

// ------------------------------------------------------------------------------------------------ fused sampler
// Upstream rollout/blackwell/csrc/sampler.cu (k1_chunks / k2_rows / k3_rank): temperature-only sampling by the
// exponential race argmax(z - log(-log u)), log-softmax, top-K log-probs, the sampled token's rank and the count of
// NaN / +inf logits. Pass 1: `chunks` CTAs per row, each reduces its slice to (max, sum exp, best race key, its top-K).
// Pass 2: one CTA per row merges the chunk records. Pass 3 (same kernel as 2, after the merge): rank = number of
// logits >= the sampled one, counted by the row's CTA over the whole row.
constexpr int kSampK = 32;
struct ChunkRec {
  float max, sumexp, best_key, best_z;
  int best_id, nonfinite, pad0, pad1;
  float top_v[kSampK];
  int top_i[kSampK];
};

__device__ __forceinline__ float race_key(float z, float u) {
  u = fminf(fmaxf(u, 1e-20f), 1.f - 1e-7f);
  return z - logf(-logf(u));
}

// block-wide top-K of per-thread candidates by repeated arg-max (K <= 32, small): values in smem
__device__ void block_topk(float* vals, int* ids, int n, float* out_v, int* out_i, int k, float* red_v, int* red_i) {
  const int tid = threadIdx.x, nt = blockDim.x;
  for (int round = 0; round < k; ++round) {
    float bv = -FLT_MAX;
    int bi = -1, bpos = -1;
    for (int i = tid; i < n; i += nt)
      if (vals[i] > bv || (vals[i] == bv && bi >= 0 && ids[i] < bi)) { bv = vals[i]; bi = ids[i]; bpos = i; }
    // warp argmax
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o), op = __shfl_xor_sync(0xffffffffu, bpos, o);
      if (ov > bv || (ov == bv && oi >= 0 && (bi < 0 || oi < bi))) { bv = ov; bi = oi; bpos = op; }
    }
    if ((tid & 31) == 0) { red_v[tid >> 5] = bv; red_i[2 * (tid >> 5)] = bi; red_i[2 * (tid >> 5) + 1] = bpos; }
    __syncthreads();
    if (tid == 0) {
      float v = -FLT_MAX; int id = -1, pos = -1;
      for (int w = 0; w < (nt >> 5); ++w)
        if (red_v[w] > v || (red_v[w] == v && red_i[2 * w] >= 0 && (id < 0 || red_i[2 * w] < id))) { v = red_v[w]; id = red_i[2 * w]; pos = red_i[2 * w + 1]; }
      out_v[round] = v; out_i[round] = id;
      if (pos >= 0) vals[pos] = -FLT_MAX;
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(256) sample_chunks_kernel(const float* __restrict__ logits, int V, int ld, float inv_temp,
                                                            const float* __restrict__ noise, int chunks, int topk, ChunkRec* __restrict__ recs) {
  extern __shared__ float sh[];  // top-K pass: candidate values [2048 + K] | ids [2048 + K] | running best values [K] | ids [K]
  const int row = blockIdx.y, chunk = blockIdx.x, tid = threadIdx.x;
  const int per = (V + chunks - 1) / chunks, lo = chunk * per, hi = min(V, lo + per);
  const float* x = logits + (size_t)row * ld;
  const float* u = noise + (size_t)row * V;
  float m = -FLT_MAX, bk = -FLT_MAX, bz = 0.f;
  int bid = -1, nf = 0;
  for (int i = lo + tid; i < hi; i += blockDim.x) {
    const float z = x[i] * inv_temp;
    if (isnan(z) || z == INFINITY) ++nf;
    m = fmaxf(m, z);
    const float key = race_key(z, u[i]);
    if (key > bk) { bk = key; bid = i; bz = z; }
  }
  __shared__ float red[8 * 4];
  __shared__ int redi[8 * 2];
  float wm = warp_max(m);
  if ((tid & 31) == 0) red[tid >> 5] = wm;
  __syncthreads();
  float cmax = -FLT_MAX;
  for (int w = 0; w < 8; ++w) cmax = fmaxf(cmax, red[w]);
  __syncthreads();
  float s = 0.f;
  for (int i = lo + tid; i < hi; i += blockDim.x) s += __expf(x[i] * inv_temp - cmax);
  s = warp_sum(s);
  nf = (int)warp_sum((float)nf);
  // best race key of the chunk
  for (int o = 16; o > 0; o >>= 1) {
    const float ok = __shfl_xor_sync(0xffffffffu, bk, o), oz = __shfl_xor_sync(0xffffffffu, bz, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bid, o);
    if (ok > bk || (ok == bk && oi >= 0 && (bid < 0 || oi < bid))) { bk = ok; bid = oi; bz = oz; }
  }
  if ((tid & 31) == 0) { red[tid >> 5] = s; red[8 + (tid >> 5)] = bk; red[16 + (tid >> 5)] = bz; red[24 + (tid >> 5)] = (float)nf; redi[tid >> 5] = bid; }
  __syncthreads();
  ChunkRec* rec = recs + (size_t)row * chunks + chunk;
  if (tid == 0) {
    float ts = 0.f, k = -FLT_MAX, z = 0.f; int id = -1, tn = 0;
    for (int w = 0; w < 8; ++w) {
      ts += red[w]; tn += (int)red[24 + w];
      if (red[8 + w] > k || (red[8 + w] == k && redi[w] >= 0 && (id < 0 || redi[w] < id))) { k = red[8 + w]; id = redi[w]; z = red[16 + w]; }
    }
    rec->max = cmax; rec->sumexp = ts; rec->best_key = k; rec->best_id = id; rec->best_z = z; rec->nonfinite = tn;
  }
  __syncthreads();
  // exact top-K of the chunk: the slice goes through shared memory in pieces, keeping the running best K
  float* cv = sh;                       // [cap + K]
  int* ci = (int*)(sh + 2048 + kSampK);  // [cap + K]
  float* tv = (float*)(ci + 2048 + kSampK);
  int* ti = (int*)(tv + kSampK);
  if (tid < kSampK) { tv[tid] = -FLT_MAX; ti[tid] = -1; }
  __syncthreads();
  for (int base = lo; base < hi; base += 2048) {
    const int n = min(2048, hi - base);
    for (int i = tid; i < n; i += blockDim.x) { cv[i] = x[base + i] * inv_temp; ci[i] = base + i; }
    if (tid < topk) { cv[n + tid] = tv[tid]; ci[n + tid] = ti[tid]; }
    __syncthreads();
    block_topk(cv, ci, n + topk, tv, ti, topk, red, redi);
  }
  if (tid < kSampK) { rec->top_v[tid] = tid < topk ? tv[tid] : -FLT_MAX; rec->top_i[tid] = tid < topk ? ti[tid] : -1; }
}

__global__ void __launch_bounds__(256) sample_rows_kernel(const float* __restrict__ logits, int V, int ld, float inv_temp, int chunks, int topk,
                                                          const ChunkRec* __restrict__ recs, int* __restrict__ tok, float* __restrict__ tok_lp,
                                                          int* __restrict__ top_id, float* __restrict__ top_lp, int* __restrict__ rank,
                                                          int* __restrict__ nonfinite) {
  extern __shared__ float sh[];
  __shared__ float s_lse, s_z;
  __shared__ int s_tok;
  __shared__ float red[8];
  __shared__ int redi[16];
  const int row = blockIdx.x, tid = threadIdx.x;
  const ChunkRec* r = recs + (size_t)row * chunks;
  float* cv = sh;
  int* ci = (int*)(sh + chunks * kSampK);
  float* tv = (float*)(ci + chunks * kSampK);
  int* ti = (int*)(tv + kSampK);
  if (tid == 0) {
    float m = -FLT_MAX;
    for (int c = 0; c < chunks; ++c) m = fmaxf(m, r[c].max);
    float s = 0.f, bk = -FLT_MAX, bz = 0.f; int bid = -1, nf = 0;
    for (int c = 0; c < chunks; ++c) {
      s += r[c].sumexp * __expf(r[c].max - m);
      nf += r[c].nonfinite;
      if (r[c].best_key > bk || (r[c].best_key == bk && r[c].best_id >= 0 && (bid < 0 || r[c].best_id < bid))) { bk = r[c].best_key; bid = r[c].best_id; bz = r[c].best_z; }
    }
    s_lse = m + __logf(s); s_tok = bid; s_z = bz;
    tok[row] = bid; tok_lp[row] = bz - s_lse; nonfinite[row] = nf;
  }
  for (int i = tid; i < chunks * kSampK; i += blockDim.x) { cv[i] = r[i / kSampK].top_v[i % kSampK]; ci[i] = r[i / kSampK].top_i[i % kSampK]; }
  __syncthreads();
  block_topk(cv, ci, chunks * kSampK, tv, ti, topk, red, redi);
  if (tid < topk) { top_id[(size_t)row * topk + tid] = ti[tid]; top_lp[(size_t)row * topk + tid] = tv[tid] - s_lse; }
  // rank of the sampled token: logits >= its logit
  const float* x = logits + (size_t)row * ld;
  const float z = s_z;
  int cnt = 0;
  for (int i = tid; i < V; i += blockDim.x) cnt += (x[i] * inv_temp >= z) ? 1 : 0;
  cnt = (int)warp_sum((float)cnt);
  __syncthreads();
  if ((tid & 31) == 0) red[tid >> 5] = (float)cnt;
  __syncthreads();
  if (tid == 0) { int t = 0; for (int w = 0; w < 8; ++w) t += (int)red[w]; rank[row] = t; }
}

// ------------------------------------------------------------------------------------------------ verify sampler
// Rejection sampling of greedy drafts (upstream verify_sampler.cu): row j of a request holds the logits after draft
// j - 1; draft d_j is accepted while log p(d_j) > log u_j (lossless for a deterministic drafter); at the first
// rejection the token is resampled from the residual distribution, which for a point-mass proposal is p with d_j
// removed: exponential race over the row with the draft's key set to -inf. If every draft is accepted the bonus token is
// a plain sample of the last row. One CTA per request; rows are processed in order until the first rejection.
__global__ void __launch_bounds__(256) verify_greedy_kernel(const float* __restrict__ logits, int V, int ld, float inv_temp, const int* __restrict__ drafts,
                                                            int n_draft, const float* __restrict__ accept_u, const float* __restrict__ noise,
                                                            int* __restrict__ out_tokens, int* __restrict__ n_accept, float* __restrict__ out_lp) {
  __shared__ float red[8], redk[8];
  __shared__ int redi[8];
  __shared__ float s_lse;
  __shared__ int s_stop;
  const int req = blockIdx.x, tid = threadIdx.x;
  const int rows = n_draft + 1;
  int accepted = 0;
  for (int j = 0; j < rows; ++j) {
    const float* x = logits + ((size_t)req * rows + j) * ld;
    const float* u = noise + ((size_t)req * rows + j) * V;
    float m = -FLT_MAX;
    for (int i = tid; i < V; i += blockDim.x) m = fmaxf(m, x[i] * inv_temp);
    m = warp_max(m);
    if ((tid & 31) == 0) red[tid >> 5] = m;
    __syncthreads();
    m = -FLT_MAX;
    for (int w = 0; w < 8; ++w) m = fmaxf(m, red[w]);
    __syncthreads();
    float s = 0.f;
    for (int i = tid; i < V; i += blockDim.x) s += __expf(x[i] * inv_temp - m);
    s = warp_sum(s);
    if ((tid & 31) == 0) red[tid >> 5] = s;
    __syncthreads();
    if (tid == 0) {
      float t = 0.f;
      for (int w = 0; w < 8; ++w) t += red[w];
      s_lse = m + __logf(t);
      s_stop = 1;
      if (j < n_draft) {
        const int d = drafts[req * n_draft + j];
        const float lp = x[d] * inv_temp - s_lse;
        if (lp > __logf(fmaxf(accept_u[req * n_draft + j], 1e-30f))) {
          out_tokens[req * rows + j] = d; out_lp[req * rows + j] = lp; s_stop = 0;
        }
      }
    }
    __syncthreads();
    if (!s_stop) { ++accepted; continue; }
    // resample this row (excluding the rejected draft) or sample the bonus token
    const int banned = j < n_draft ? drafts[req * n_draft + j] : -1;
    float bk = -FLT_MAX, bz = 0.f; int bid = -1;
    for (int i = tid; i < V; i += blockDim.x) {
      if (i == banned) continue;
      const float z = x[i] * inv_temp, key = race_key(z, u[i]);
      if (key > bk) { bk = key; bid = i; bz = z; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ok = __shfl_xor_sync(0xffffffffu, bk, o), oz = __shfl_xor_sync(0xffffffffu, bz, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bid, o);
      if (ok > bk || (ok == bk && oi >= 0 && (bid < 0 || oi < bid))) { bk = ok; bid = oi; bz = oz; }
    }
    if ((tid & 31) == 0) { redk[tid >> 5] = bk; red[tid >> 5] = bz; redi[tid >> 5] = bid; }
    __syncthreads();
    if (tid == 0) {
      float k = -FLT_MAX, z = 0.f; int id = -1;
      for (int w = 0; w < 8; ++w)
        if (redk[w] > k || (redk[w] == k && redi[w] >= 0 && (id < 0 || redi[w] < id))) { k = redk[w]; id = redi[w]; z = red[w]; }
      out_tokens[req * rows + j] = id; out_lp[req * rows + j] = z - s_lse;
      for (int r = j + 1; r < rows; ++r) { out_tokens[req * rows + r] = -1; out_lp[req * rows + r] = 0.f; }
    }
    break;
  }
  if (tid == 0) n_accept[req] = accepted;
}

// ------------------------------------------------------------------------------------------------ GDN decode step
// One token of the gated delta rule for a batch of sequences (upstream Triton `_conv_decode/_decode/_norm`,
// rollout/blackwell/gdn/kernels.py:93-282; hopper gdn_decode.cu): causal conv(4) update + SiLU, gates, L2 norm of q/k,
// S <- S exp(g); u = (v - S k) beta; S <- S + u k^T; o = S q, then the gated RMSNorm o * rstd * w * silu(z).
// CTA per (value head, sequence), 128 threads = one state row (v index) each; K = V = 128.
//   x [B][C] conv inputs (q | k | v), z [B][Hv*128], a,b [B][Hv]; conv_state [slot][3][C]; state [slot][Hv][128][128]
__global__ void __launch_bounds__(128) gdn_decode_kernel(const float* __restrict__ x, const float* __restrict__ z, const float* __restrict__ a,
                                                         const float* __restrict__ b, const float* __restrict__ conv_w, const float* __restrict__ A_log,
                                                         const float* __restrict__ dt_bias, const float* __restrict__ norm_w,
                                                         float* __restrict__ conv_state, float* __restrict__ state, const int* __restrict__ slots,
                                                         float* __restrict__ out, int Hk, int Hv, float l2_eps, float rms_eps) {
  constexpr int D = 128;
  __shared__ float q[D], k[D], red[8];
  const int hv = blockIdx.x, seq = blockIdx.y, tid = threadIdx.x;
  const int hk = hv / (Hv / Hk), C = 2 * Hk * D + Hv * D, slot = slots[seq];
  const float* xs = x + (size_t)seq * C;
  float* cs = conv_state + (size_t)slot * 3 * C;
  auto conv = [&](int ch) {
    const float* w = conv_w + (size_t)ch * 4;
    const float y = cs[ch] * w[0] + cs[C + ch] * w[1] + cs[2 * C + ch] * w[2] + xs[ch] * w[3];
    return y / (1.f + __expf(-y));
  };
  const float qv = conv(hk * D + tid), kv = conv(Hk * D + hk * D + tid), vv = conv(2 * Hk * D + hv * D + tid);
  // L2 norms over the head
  float sq = warp_sum(qv * qv), sk = warp_sum(kv * kv);
  if ((tid & 31) == 0) { red[tid >> 5] = sq; red[4 + (tid >> 5)] = sk; }
  __syncthreads();
  sq = red[0] + red[1] + red[2] + red[3];
  sk = red[4] + red[5] + red[6] + red[7];
  q[tid] = qv * rsqrtf(sq + l2_eps) * rsqrtf((float)D);
  k[tid] = kv * rsqrtf(sk + l2_eps);
  __syncthreads();
  const float av = a[(size_t)seq * Hv + hv] + dt_bias[hv];
  const float sp = av > 20.f ? av : log1pf(__expf(av));
  const float decay = __expf(-__expf(A_log[hv]) * sp);
  const float beta = 1.f / (1.f + __expf(-b[(size_t)seq * Hv + hv]));
  // this thread owns state row `tid` (value index): S[v][:]
  float4* S = (float4*)(state + (((size_t)slot * Hv + hv) * D + tid) * D);
  float dot = 0.f;
#pragma unroll 8
  for (int i = 0; i < D / 4; ++i) {
    float4 s = S[i];
    s.x *= decay; s.y *= decay; s.z *= decay; s.w *= decay;
    dot += s.x * k[4 * i] + s.y * k[4 * i + 1] + s.z * k[4 * i + 2] + s.w * k[4 * i + 3];
    S[i] = s;
  }
  const float uu = (vv - dot) * beta;
  float o = 0.f;
#pragma unroll 8
  for (int i = 0; i < D / 4; ++i) {
    float4 s = S[i];
    s.x += uu * k[4 * i]; s.y += uu * k[4 * i + 1]; s.z += uu * k[4 * i + 2]; s.w += uu * k[4 * i + 3];
    o += s.x * q[4 * i] + s.y * q[4 * i + 1] + s.z * q[4 * i + 2] + s.w * q[4 * i + 3];
    S[i] = s;
  }
  // gated RMSNorm over the head's 128 outputs
  float so = warp_sum(o * o);
  __syncthreads();
  if ((tid & 31) == 0) red[tid >> 5] = so;
  __syncthreads();
  so = red[0] + red[1] + red[2] + red[3];
  const float zz = z[(size_t)seq * Hv * D + hv * D + tid];
  out[(size_t)seq * Hv * D + hv * D + tid] = o * rsqrtf(so / D + rms_eps) * norm_w[tid] * (zz / (1.f + __expf(-zz)));
}

// Conv window shift after the step (a launch of its own: the step's CTAs all read the old window).
__global__ void gdn_conv_shift_kernel(const float* __restrict__ x, float* __restrict__ conv_state, const int* __restrict__ slots, int C) {
  const int seq = blockIdx.y, ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= C) return;
  float* cs = conv_state + (size_t)slots[seq] * 3 * C;
  cs[ch] = cs[C + ch];
  cs[C + ch] = cs[2 * C + ch];
  cs[2 * C + ch] = x[(size_t)seq * C + ch];
}

// ------------------------------------------------------------------------------------------------ paged decode attention
// Split-KV paged attention for decode / verify rows (upstream verify_attn.cu, split_attn.cu): q [R][Hq][D] (already
// normed and rotated), KV cache in 16-token blocks [block][16][Hkv][D] bf16, per-row context length (causal inside a
// verify block comes from giving row j the length ctx + j + 1). Grid (split, kv head, row); a warp per q head of the
// group; online softmax over this split's tokens; partial (o, m, l) merged by the combine kernel.
template <int D>
__global__ void __launch_bounds__(256) paged_attn_split_kernel(const float* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                                                               const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_table, int max_blocks,
                                                               const int* __restrict__ ctx_len, int Hq, int Hkv, float scale, int nsplit,
                                                               float* __restrict__ part_o, float* __restrict__ part_ml) {
  const int split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = Hq / Hkv;
  if (warp >= group) return;
  const int h = kvh * group + warp;
  const int len = ctx_len[row];
  const int per = (((len + nsplit - 1) / nsplit) + 15) & ~15;
  const int lo = split * per, hi = min(len, lo + per);
  constexpr int PER = D / 32;
  float qv[PER], acc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) { qv[i] = q[((size_t)row * Hq + h) * D + lane + 32 * i] * scale; acc[i] = 0.f; }
  float m = -FLT_MAX, l = 0.f;
  for (int t = lo; t < hi; ++t) {
    const int blk = block_table[(size_t)row * max_blocks + (t >> 4)];
    const size_t base = (((size_t)blk * 16 + (t & 15)) * Hkv + kvh) * D;
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
  const size_t o = (((size_t)row * Hq + h) * nsplit + split);
#pragma unroll
  for (int i = 0; i < PER; ++i) part_o[o * D + lane + 32 * i] = acc[i];
  if (lane == 0) { part_ml[o * 2] = m; part_ml[o * 2 + 1] = l; }
}

template <int D>
__global__ void paged_attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int nsplit, float* __restrict__ out) {
  const size_t rh = blockIdx.x;
  const int tid = threadIdx.x;
  float m = -FLT_MAX;
  for (int s = 0; s < nsplit; ++s) m = fmaxf(m, part_ml[(rh * nsplit + s) * 2]);
  float l = 0.f, acc = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = part_ml[(rh * nsplit + s) * 2], ls = part_ml[(rh * nsplit + s) * 2 + 1];
    if (ls <= 0.f) continue;
    const float w = __expf(ms - m);
    l += ls * w;
    acc += part_o[(rh * nsplit + s) * D + tid] * w;
  }
  out[rh * D + tid] = l > 0.f ? acc / l : 0.f;
}

// ------------------------------------------------------------------------------------------------ embedding + KV blocks
// out[t] = mask[t] ? embeds[t] : table[ids[t]]  (vision-embedding placeholder rows replace the image-pad tokens)
__global__ void embed_merge_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table, const float* __restrict__ embeds,
                                   const unsigned char* __restrict__ mask, float* __restrict__ out, int H, int V) {
  const int t = blockIdx.x;
  const bool use = mask != nullptr && mask[t];
  const int id = min(max(ids[t], 0), V - 1);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[(size_t)t * H + i] = use ? embeds[(size_t)t * H + i] : __bfloat162float(table[(size_t)id * H + i]);
}

// Gather `n` cache blocks (block_bytes each, 16-byte multiples) into a contiguous staging buffer, or scatter them back:
// the device side of the host-DRAM KV tier (one pinned copy per staging buffer instead of one per block).
__global__ void kv_blocks_copy_kernel(uint4* __restrict__ cache, uint4* __restrict__ staging, const int* __restrict__ block_ids, int vec_per_block,
                                      int to_staging) {
  const int b = blockIdx.x;
  uint4* c = cache + (size_t)block_ids[b] * vec_per_block;
  uint4* s = staging + (size_t)b * vec_per_block;
  for (int i = threadIdx.x; i < vec_per_block; i += blockDim.x) {
    if (to_staging) s[i] = c[i];
    else c[i] = s[i];
  }
}

}  // namespace pear

using namespace pear;

PEAR_API int pear_sample_workspace_bytes(int rows, int chunks) { return (int)(sizeof(ChunkRec) * (size_t)rows * chunks); }

PEAR_API int pear_fused_sample(const float* logits, int rows, int V, int ld, float temperature, const float* noise, int chunks, int topk,
                               void* workspace, int* tok, float* tok_lp, int* top_id, float* top_lp, int* rank, int* nonfinite, void* stream) {
  if (topk < 1 || topk > kSampK || chunks < 1 || chunks > 64 || temperature <= 0.f) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t sh1 = (size_t)(2048 + kSampK) * 8 + kSampK * 8;
  sample_chunks_kernel<<<dim3(chunks, rows), 256, sh1, s>>>(logits, V, ld, 1.f / temperature, noise, chunks, topk, (ChunkRec*)workspace);
  PEAR_LAUNCH_CHECK();
  const size_t sh2 = (size_t)chunks * kSampK * 8 + kSampK * 8;
  sample_rows_kernel<<<rows, 256, sh2, s>>>(logits, V, ld, 1.f / temperature, chunks, topk, (const ChunkRec*)workspace, tok, tok_lp, top_id, top_lp,
                                            rank, nonfinite);
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_verify_greedy(const float* logits, int requests, int n_draft, int V, int ld, float temperature, const int* drafts,
                                const float* accept_u, const float* noise, int* out_tokens, int* n_accept, float* out_lp, void* stream) {
  if (temperature <= 0.f) return (int)cudaErrorInvalidValue;
  verify_greedy_kernel<<<requests, 256, 0, (cudaStream_t)stream>>>(logits, V, ld, 1.f / temperature, drafts, n_draft, accept_u, noise, out_tokens,
                                                                   n_accept, out_lp);
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_gdn_decode(const float* x, const float* z, const float* a, const float* b, const float* conv_w, const float* A_log,
                             const float* dt_bias, const float* norm_w, float* conv_state, float* state, const int* slots, float* out, int batch,
                             int Hk, int Hv, float l2_eps, float rms_eps, void* stream) {
  if (Hv % Hk) return (int)cudaErrorInvalidValue;
  gdn_decode_kernel<<<dim3(Hv, batch), 128, 0, (cudaStream_t)stream>>>(x, z, a, b, conv_w, A_log, dt_bias, norm_w, conv_state, state, slots, out, Hk,
                                                                       Hv, l2_eps, rms_eps);
  PEAR_LAUNCH_CHECK();
  const int C = 2 * Hk * 128 + Hv * 128;
  gdn_conv_shift_kernel<<<dim3((C + 255) / 256, batch), 256, 0, (cudaStream_t)stream>>>(x, conv_state, slots, C);
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_paged_attention(const float* q, const void* kc, const void* vc, const int* block_table, int max_blocks, const int* ctx_len,
                                  int rows, int Hq, int Hkv, int D, float scale, int nsplit, float* part_o, float* part_ml, float* out, void* stream) {
  if (Hq % Hkv || Hq / Hkv > 8 || (D != 128 && D != 256)) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 grid(nsplit, Hkv, rows);
  if (D == 256) {
    paged_attn_split_kernel<256><<<grid, 256, 0, s>>>(q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, block_table, max_blocks, ctx_len, Hq, Hkv, scale, nsplit, part_o, part_ml);
    PEAR_LAUNCH_CHECK();
    paged_attn_combine_kernel<256><<<rows * Hq, 256, 0, s>>>(part_o, part_ml, nsplit, out);
  } else {
    paged_attn_split_kernel<128><<<grid, 256, 0, s>>>(q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, block_table, max_blocks, ctx_len, Hq, Hkv, scale, nsplit, part_o, part_ml);
    PEAR_LAUNCH_CHECK();
    paged_attn_combine_kernel<128><<<rows * Hq, 128, 0, s>>>(part_o, part_ml, nsplit, out);
  }
  PEAR_LAUNCH_CHECK();
  return 0;
}

// ------------------------------------------------------------------------------------------------ exact-max top-p
// Nucleus mask of one row per CTA: softmax of logits * inv_temp shifted by the row's EXACT maximum, then bisection on the
// probability threshold (the smallest kept probability): `iters` passes over the row, no sort, tokens tied with the pivot
// all kept; tokens outside the nucleus are set to -inf in place. The row (1 MB at 248 320 tokens) stays in L2 between
// the passes. (Upstream: pear/rollout/top_p.py:11-268 — vLLM's pivot search with the shift changed to the exact maximum.)
constexpr int kTopPThreads = 1024;
__device__ __forceinline__ float topp_block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();  // `red` of the previous reduction has been read
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < kTopPThreads / 32; ++i) t += red[i];
  return t;
}
__global__ void __launch_bounds__(kTopPThreads) top_p_mask_kernel(float* __restrict__ logits, long long ld, int V, float inv_temp,
                                                                  const float* __restrict__ top_p, int iters) {
  __shared__ float red[kTopPThreads / 32];
  float* x = logits + (long long)blockIdx.x * ld;
  const float p = top_p[blockIdx.x];
  if (!(p < 1.f)) return;  // the whole CTA
  float m = -INFINITY;
  for (int i = threadIdx.x; i < V; i += kTopPThreads) m = fmaxf(m, x[i]);
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = red[0];
#pragma unroll
  for (int i = 1; i < kTopPThreads / 32; ++i) m = fmaxf(m, red[i]);
  float s = 0.f;
  for (int i = threadIdx.x; i < V; i += kTopPThreads) s += __expf((x[i] - m) * inv_temp);
  s = topp_block_sum(s, red);
  const float inv_s = 1.f / s;
  float lo = 0.f, hi = inv_s;  // the largest probability is exp(0) / s
  for (int it = 0; it < iters; ++it) {
    const float mid = 0.5f * (lo + hi);
    float mass = 0.f;
    for (int i = threadIdx.x; i < V; i += kTopPThreads) {
      const float q = __expf((x[i] - m) * inv_temp) * inv_s;
      mass += q >= mid ? q : 0.f;
    }
    mass = topp_block_sum(mass, red);
    if (mass >= p) lo = mid;  // the threshold can still rise
    else hi = mid;
  }
  for (int i = threadIdx.x; i < V; i += kTopPThreads)
    if (!(__expf((x[i] - m) * inv_temp) * inv_s >= lo)) x[i] = -INFINITY;
}

// logits fp32 [rows, ld] (modified in place), top_p fp32 [rows]; rows with top_p >= 1 are left alone.
PEAR_API int pear_top_p_mask(float* logits, long long ld, int rows, int V, float temperature, const float* top_p, int iters, void* stream) {
  if (rows <= 0) return 0;
  if (V <= 0 || temperature <= 0.f || iters < 1) return (int)cudaErrorInvalidValue;
  top_p_mask_kernel<<<rows, kTopPThreads, 0, (cudaStream_t)stream>>>(logits, ld, V, 1.f / temperature, top_p, iters);
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_embed_merge(const int* ids, const void* table, const float* embeds, const unsigned char* mask, float* out, int T, int H, int V,
                              void* stream) {
  embed_merge_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(ids, (const __nv_bfloat16*)table, embeds, mask, out, H, V);
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_kv_blocks_copy(void* cache, void* staging, const int* block_ids, int n, int block_bytes, int to_staging, void* stream) {
  if (block_bytes % 16) return (int)cudaErrorInvalidValue;
  kv_blocks_copy_kernel<<<n, 256, 0, (cudaStream_t)stream>>>((uint4*)cache, (uint4*)staging, block_ids, block_bytes / 16, to_staging);
  PEAR_LAUNCH_CHECK();
  return 0;
}

// ------------------------------------------------------------------------------------------------ no-allocation variant
// pear_fused_sample with its workspace inside the library's own device image (declaration and contract:
// pear_no_alloc.h). The array exists once per device; its address is looked up on the first call on each device.
#include "pear_no_alloc.h"

static __device__ __align__(256) unsigned char g_sample_scratch[PEAR_SAMPLE_STATIC_MAX_RECORDS * sizeof(pear::ChunkRec)];

extern "C" __attribute__((visibility("default"))) int pear_fused_sample_static(
    const float* logits, int rows, int V, int ld, float temperature, const float* noise, int chunks, int topk, int* tok, float* tok_lp,
    int* top_id, float* top_lp, int* rank, int* nonfinite, void* stream) {
  static void* scratch_of_device[64] = {nullptr};
  if (topk < 1 || topk > kSampK || chunks < 1 || chunks > 64 || temperature <= 0.f || rows < 1 || V < 1) return PEAR_NOALLOC_BAD_ARGUMENT;
  if (rows > PEAR_SAMPLE_STATIC_MAX_ROWS || (long long)rows * chunks > PEAR_SAMPLE_STATIC_MAX_RECORDS) return PEAR_NOALLOC_TOO_LARGE;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
  if (scratch_of_device[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_sample_scratch);
    if (e != cudaSuccess) return (int)e;
    scratch_of_device[dev] = p;
  }
  ChunkRec* ws = (ChunkRec*)scratch_of_device[dev];
  cudaStream_t s = (cudaStream_t)stream;
  const size_t sh1 = (size_t)(2048 + kSampK) * 8 + kSampK * 8;
  sample_chunks_kernel<<<dim3(chunks, rows), 256, sh1, s>>>(logits, V, ld, 1.f / temperature, noise, chunks, topk, ws);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  const size_t sh2 = (size_t)chunks * kSampK * 8 + kSampK * 8;
  sample_rows_kernel<<<rows, 256, sh2, s>>>(logits, V, ld, 1.f / temperature, chunks, topk, ws, tok, tok_lp, top_id, top_lp, rank, nonfinite);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}
