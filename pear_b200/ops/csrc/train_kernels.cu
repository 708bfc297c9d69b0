// Trainer-side kernels beyond the element-wise set: running softmax statistics of the fused log-prob / entropy head
// (logits are produced chunk by chunk by the tcgen05 GEMM and never stored whole; upstream trainer/head.py:10-344), and
// the Gated-DeltaNet front end (causal conv(4) + SiLU + q/k L2 norm over packed sequences; upstream trainer/gdn.py:40-95).
#include "common.cuh"

#include <cfloat>

namespace pear {

// One CTA per row. Folds a chunk of logits z = x * inv_temp (columns [v0, v0 + Vc)) into the row's running
//   m = max z,  s1 = sum exp(z - m),  s2 = sum exp(z - m) * z
// and records z at the requested ids that fall inside the chunk. After the last chunk:
//   lse = m + log s1,  log p(id) = z_id - lse,  entropy = lse - s2 / s1.
__global__ void __launch_bounds__(256) head_stats_update_kernel(const float* __restrict__ x, int ld, int Vc, int v0, float inv_temp,
                                                                float* __restrict__ run, const int* __restrict__ ids, int J,
                                                                float* __restrict__ id_z) {
  __shared__ float red[8], red2[8];
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* xr = x + (size_t)row * ld;
  float m = -FLT_MAX;
  for (int i = tid; i < Vc; i += blockDim.x) m = fmaxf(m, xr[i] * inv_temp);
  m = warp_max(m);
  if ((tid & 31) == 0) red[tid >> 5] = m;
  __syncthreads();
  m = -FLT_MAX;
  for (int w = 0; w < 8; ++w) m = fmaxf(m, red[w]);
  float* r = run + (size_t)row * 4;
  const float m_old = r[0];
  const float m_new = fmaxf(m_old, m);
  __syncthreads();
  float s1 = 0.f, s2 = 0.f;
  for (int i = tid; i < Vc; i += blockDim.x) {
    const float z = xr[i] * inv_temp, e = __expf(z - m_new);
    s1 += e;
    s2 += e * z;
  }
  s1 = warp_sum(s1);
  s2 = warp_sum(s2);
  if ((tid & 31) == 0) { red[tid >> 5] = s1; red2[tid >> 5] = s2; }
  __syncthreads();
  if (tid == 0) {
    float t1 = 0.f, t2 = 0.f;
    for (int w = 0; w < 8; ++w) { t1 += red[w]; t2 += red2[w]; }
    const float c = m_old == -FLT_MAX ? 0.f : __expf(m_old - m_new);
    r[0] = m_new;
    r[1] = r[1] * c + t1;
    r[2] = r[2] * c + t2;
  }
  for (int j = tid; j < J; j += blockDim.x) {
    const int id = ids[(size_t)row * J + j];
    if (id >= v0 && id < v0 + Vc) id_z[(size_t)row * J + j] = xr[id - v0] * inv_temp;
  }
}

__global__ void head_stats_finish_kernel(const float* __restrict__ run, const float* __restrict__ id_z, int J, float* __restrict__ lp,
                                         float* __restrict__ ent, int rows) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  const float* r = run + (size_t)row * 4;
  const float lse = r[0] + logf(r[1]);
  ent[row] = lse - r[2] / r[1];
  for (int j = 0; j < J; ++j) lp[(size_t)row * J + j] = id_z[(size_t)row * J + j] - lse;
}

// GDN front end over packed sequences: y[t, c] = silu(sum_j w[c, j] * x[t - 3 + j, c]) with rows before the sequence
// start read as zero; the q and k heads (128 channels each) are then L2-normalised, q also scaled by 128^-0.5.
// Grid (head-sized channel group, token); 128 threads. seq_start[t] = first row of the sequence token t belongs to.
__global__ void __launch_bounds__(128) gdn_front_kernel(const float* __restrict__ x, const float* __restrict__ w, const int* __restrict__ seq_start,
                                                        float* __restrict__ y, int C, int qk_channels, float eps) {
  __shared__ float red[4];
  const int t = blockIdx.y, ch = blockIdx.x * 128 + threadIdx.x;
  const int s0 = seq_start[t];
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int tt = t - 3 + j;
    if (tt >= s0) acc += w[(size_t)ch * 4 + j] * x[(size_t)tt * C + ch];
  }
  float v = acc / (1.f + __expf(-acc));
  if (blockIdx.x * 128 < qk_channels) {  // a q or k head: normalise over its 128 channels
    float ss = warp_sum(v * v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = red[0] + red[1] + red[2] + red[3];
    v *= rsqrtf(ss + eps);
    if (blockIdx.x * 128 < qk_channels / 2) v *= 0.08838834764831845f;  // q heads: 128^-0.5
  }
  y[(size_t)t * C + ch] = v;
}

// Backward of the front end, step 1: gradient at the convolution output. Same grid as the forward; the convolution and
// SiLU are recomputed (4 loads), the L2 norm's Jacobian needs one more block reduction (y_hat . dy).
__global__ void __launch_bounds__(128) gdn_front_bwd_act_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                                const int* __restrict__ seq_start, const float* __restrict__ dy,
                                                                float* __restrict__ dacc, int C, int qk_channels, float eps) {
  __shared__ float red[8];
  const int t = blockIdx.y, ch = blockIdx.x * 128 + threadIdx.x;
  const int s0 = seq_start[t];
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int tt = t - 3 + j;
    if (tt >= s0) acc += w[(size_t)ch * 4 + j] * x[(size_t)tt * C + ch];
  }
  const float sig = 1.f / (1.f + __expf(-acc));
  const float v = acc * sig;
  float dv = dy[(size_t)t * C + ch];
  if (blockIdx.x * 128 < qk_channels) {
    float ss = warp_sum(v * v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = red[0] + red[1] + red[2] + red[3];
    const float n = rsqrtf(ss + eps), yhat = v * n;
    float dot = warp_sum(yhat * dv);
    if ((threadIdx.x & 31) == 0) red[4 + (threadIdx.x >> 5)] = dot;
    __syncthreads();
    dot = red[4] + red[5] + red[6] + red[7];
    const float scale = blockIdx.x * 128 < qk_channels / 2 ? 0.08838834764831845f : 1.f;
    dv = scale * n * (dv - yhat * dot);
  }
  dacc[(size_t)t * C + ch] = dv * (sig + acc * sig * (1.f - sig));
}

// Step 2: dx[t] = sum_j w[j] dacc[t + 3 - j] over the rows of the same sequence, and dw[c, j] += sum_t dacc[t] x[t - 3 + j].
// Grid (channel group of 128, chunk of 64 tokens); one thread per channel, coalesced over channels.
__global__ void __launch_bounds__(128) gdn_front_bwd_conv_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                                 const int* __restrict__ seq_start, const float* __restrict__ dacc,
                                                                 float* __restrict__ dx, float* __restrict__ dw, int T, int C) {
  const int ch = blockIdx.x * 128 + threadIdx.x, t0 = blockIdx.y * 64, t1 = min(T, t0 + 64);
  float wj[4], dwj[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 4; ++j) wj[j] = w[(size_t)ch * 4 + j];
  for (int t = t0; t < t1; ++t) {
    const int s0 = seq_start[t];
    const float d = dacc[(size_t)t * C + ch];
    float g = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int tu = t + 3 - j;  // the output row that read x[t] through tap j
      if (tu < T && seq_start[tu] <= t) g += wj[j] * dacc[(size_t)tu * C + ch];
      const int ti = t - 3 + j;  // the input row that output row t read through tap j
      if (ti >= s0) dwj[j] += d * x[(size_t)ti * C + ch];
    }
    dx[(size_t)t * C + ch] = g;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) atomicAdd(dw + (size_t)ch * 4 + j, dwj[j]);
}

}  // namespace pear

using namespace pear;

// dy [T, C] -> dx [T, C] and dw [C, 4] (ZERO at launch; accumulated with atomics). dacc: fp32 [T, C] scratch.
PEAR_API int pear_gdn_front_bwd(const float* x, const float* w, const int* seq_start, const float* dy, float* dacc, float* dx, float* dw,
                                int T, int C, int qk_channels, float eps, void* stream) {
  if (C % 128 || qk_channels % 256) return (int)cudaErrorInvalidValue;
  gdn_front_bwd_act_kernel<<<dim3(C / 128, T), 128, 0, (cudaStream_t)stream>>>(x, w, seq_start, dy, dacc, C, qk_channels, eps);
  PEAR_LAUNCH_CHECK();
  gdn_front_bwd_conv_kernel<<<dim3(C / 128, (T + 63) / 64), 128, 0, (cudaStream_t)stream>>>(x, w, seq_start, dacc, dx, dw, T, C);
  PEAR_LAUNCH_CHECK();
  return 0;
}

// run: float[rows][4] = (m, s1, s2, unused); the caller initialises it to (-FLT_MAX, 0, 0, 0) before the first chunk.
PEAR_API int pear_head_stats_update(const float* logits, int rows, int ld, int Vc, int v0, float temperature, float* run, const int* ids, int J,
                                    float* id_z, void* stream) {
  head_stats_update_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>(logits, ld, Vc, v0, 1.f / temperature, run, ids, J, id_z);
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_head_stats_finish(const float* run, const float* id_z, int J, float* lp, float* ent, int rows, void* stream) {
  head_stats_finish_kernel<<<(rows + 127) / 128, 128, 0, (cudaStream_t)stream>>>(run, id_z, J, lp, ent, rows);
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_gdn_front(const float* x, const float* w, const int* seq_start, float* y, int T, int C, int qk_channels, float eps, void* stream) {
  if (C % 128 || qk_channels % 256) return (int)cudaErrorInvalidValue;
  gdn_front_kernel<<<dim3(C / 128, T), 128, 0, (cudaStream_t)stream>>>(x, w, seq_start, y, C, qk_channels, eps);
  PEAR_LAUNCH_CHECK();
  return 0;
}

// ------------------------------------------------------------------------------------------------ delta-rule chunk loop
// The sequential part of the chunked (WY) Gated-DeltaNet scan for one sequence: per value head and chunk c of 64 tokens,
// with the chunk-local operands prepared in parallel beforehand (W = T (beta k e^G), U = T (beta v), Qe = q e^G,
// A = tril(q k^T * decay), Kt = k e^(G_C - G), gamma = e^(G_C)):
//     v' = U - W S^T;   o = Qe S^T + A v';   S <- gamma S + v'^T Kt (+ E)
// The backward of this loop is the SAME linear recurrence run over the chunks in reverse with the roles of W and Kt
// swapped (dS_c = gamma dS_{c+1} + (U' - Kt dS_{c+1}^T)^T W + dO^T Qe with U' = -A^T dO), so one kernel serves both:
// the optional additive term E, the optional v' output and the optional state history exist for that use.
// Grid (value head, 32-wide slice of the value dimension), 512 threads: the rows of S (one per value channel) are
// independent, so four CTAs share a head without talking. fp32 SIMT throughout; S lives in shared memory as St[k][v]. Operands are
// staged transposed with padded rows so that a warp reads consecutive words (upstream: cuDNN / FlashInfer sm100 GDN
// kernels, pear/models/qwen3_5/trainer/blackwell/delta_rule.py:91-161).
namespace pear {
constexpr int kScC = 64, kScK = 128, kScVs = 32, kScPad = 65;

constexpr int kScT = 512;                       // threads: 16 warps, four per scheduler, to cover the shared-memory latency
constexpr int kScV1 = kScVs / (kScT / kScC);    // value channels per thread in steps 1-2 (4)
constexpr int kScV3 = kScVs / (kScT / kScK);    // value channels per thread in step 3 (8)

__global__ void __launch_bounds__(kScT, 1)
gdn_chunk_loop_kernel(const float* __restrict__ W, const float* __restrict__ U, const float* __restrict__ Qe, const float* __restrict__ A,
                      const float* __restrict__ Kt, const float* __restrict__ gamma, const float* __restrict__ S0, const float* __restrict__ E,
                      float* __restrict__ O, float* __restrict__ S_out, float* __restrict__ S_hist, float* __restrict__ VP, int n_chunks, int V) {
  extern __shared__ float sh[];
  float* Wt = sh;                        // [128 k][65]  (i < 64)
  float* Qt = Wt + kScK * kScPad;        // [128 k][65]
  float* Ks = Qt + kScK * kScPad;        // [64 i][128 k]
  float* At = Ks + kScC * kScK;          // [64 j][65]   At[j][i] = A[i][j]
  float* St = At + kScC * kScPad;        // [128 k][32 v]
  float* vps = St + kScK * kScVs;        // [64 j][32 v]
  const int h = blockIdx.x, vs = blockIdx.y * kScVs, tid = threadIdx.x;
  // state slice: S[h][vs + v][k] -> St[k][v]
  for (int e = tid; e < kScVs * kScK; e += kScT) {
    const int v = e / kScK, k = e % kScK;
    St[k * kScVs + v] = S0 ? S0[((size_t)h * V + vs + v) * kScK + k] : 0.f;
  }
  __syncthreads();
  const int i = tid & 63, vq = tid >> 6;      // steps 1-2: row i of the chunk, value channels vq * kScV1 ..
  const int kk = tid & 127, vh = tid >> 7;    // step 3: key channel kk, value channels vh * kScV3 ..
  for (int c = 0; c < n_chunks; ++c) {
    const size_t hc = (size_t)h * n_chunks + c;
    const float* Wc = W + hc * kScC * kScK;
    const float* Qc = Qe + hc * kScC * kScK;
    const float* Kc = Kt + hc * kScC * kScK;
    const float* Ac = A + hc * kScC * kScC;
    // small operands of the later steps are requested now, and the next chunk's operands are pulled into L2, so that
    // their latency hides under this chunk's staging and arithmetic
    const float4 u0 = *(const float4*)(U + (hc * kScC + i) * V + vs + vq * kScV1);
    const float gm = gamma[hc];
    float e8[kScV3];
#pragma unroll
    for (int j = 0; j < kScV3; ++j) e8[j] = E ? E[(hc * V + vs + vh * kScV3 + j) * kScK + kk] : 0.f;
    if (c + 1 < n_chunks) {
      const size_t nx = hc + 1;
      if (tid < 256) {  // 3 x 32 KB in 128-byte lines
        asm volatile("prefetch.global.L2 [%0];" ::"l"(W + nx * kScC * kScK + tid * 32));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(Qe + nx * kScC * kScK + tid * 32));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(Kt + nx * kScC * kScK + tid * 32));
      } else if (tid < 384) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(A + nx * kScC * kScC + (tid - 256) * 32));
      } else if (tid < 448) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(U + (nx * kScC + (tid - 384)) * V + vs));
      }
    }
    // coalesced along k, transposed into padded rows; 8 loads of each operand in flight per thread (a dependent
    // load-store loop would expose the global latency once per iteration)
#pragma unroll 1
    for (int e0 = tid; e0 < kScC * kScK; e0 += kScT * 8) {
      float w8[8], q8[8], k8[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) { w8[u] = Wc[e0 + u * kScT]; q8[u] = Qc[e0 + u * kScT]; k8[u] = Kc[e0 + u * kScT]; }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int e = e0 + u * kScT, r = e / kScK, k = e % kScK;
        Wt[k * kScPad + r] = w8[u];
        Qt[k * kScPad + r] = q8[u];
        Ks[e] = k8[u];
      }
    }
    {
      float a8[kScC * kScC / kScT];
#pragma unroll
      for (int u = 0; u < kScC * kScC / kScT; ++u) a8[u] = Ac[tid + u * kScT];
#pragma unroll
      for (int u = 0; u < kScC * kScC / kScT; ++u) { const int e = tid + u * kScT; At[(e % kScC) * kScPad + e / kScC] = a8[u]; }
    }
    if (S_hist) {  // the state BEFORE this chunk, for a backward pass
      float* dst = S_hist + (hc * V + vs) * kScK;
#pragma unroll 8
      for (int e = tid; e < kScVs * kScK; e += kScT) dst[e] = St[(e % kScK) * kScVs + e / kScK];
    }
    __syncthreads();
    // 1. v' = U - W S^T and the state part of the output, Qe S^T
    float wv[kScV1], ov[kScV1];
#pragma unroll
    for (int j = 0; j < kScV1; ++j) wv[j] = ov[j] = 0.f;
#pragma unroll 8
    for (int k = 0; k < kScK; ++k) {
      const float w = Wt[k * kScPad + i], q = Qt[k * kScPad + i];
      const float4 s0 = *(const float4*)(St + k * kScVs + vq * kScV1);
      wv[0] += w * s0.x; wv[1] += w * s0.y; wv[2] += w * s0.z; wv[3] += w * s0.w;
      ov[0] += q * s0.x; ov[1] += q * s0.y; ov[2] += q * s0.z; ov[3] += q * s0.w;
    }
    const float4 vp4 = make_float4(u0.x - wv[0], u0.y - wv[1], u0.z - wv[2], u0.w - wv[3]);
    *(float4*)(vps + i * kScVs + vq * kScV1) = vp4;
    if (VP) *(float4*)(VP + (hc * kScC + i) * V + vs + vq * kScV1) = vp4;
    __syncthreads();
    // 2. o = Qe S^T + A v' (skipped when the caller wants the states only)
    if (O) {
#pragma unroll 8
      for (int j = 0; j < kScC; ++j) {
        const float a = At[j * kScPad + i];
        const float4 p0 = *(const float4*)(vps + j * kScVs + vq * kScV1);
        ov[0] += a * p0.x; ov[1] += a * p0.y; ov[2] += a * p0.z; ov[3] += a * p0.w;
      }
      *(float4*)(O + (hc * kScC + i) * V + vs + vq * kScV1) = make_float4(ov[0], ov[1], ov[2], ov[3]);
    }
    // 3. S <- gamma S + v'^T Kt (every thread owns St[kk][vh * 8 .. + 7]; nobody reads St before the next barrier pair)
    float acc[kScV3];
#pragma unroll
    for (int j = 0; j < kScV3; ++j) acc[j] = 0.f;
#pragma unroll 4
    for (int r = 0; r < kScC; ++r) {
      const float kt = Ks[r * kScK + kk];
      const float4 p = *(const float4*)(vps + r * kScVs + vh * kScV3), p2 = *(const float4*)(vps + r * kScVs + vh * kScV3 + 4);
      acc[0] += kt * p.x; acc[1] += kt * p.y; acc[2] += kt * p.z; acc[3] += kt * p.w;
      acc[4] += kt * p2.x; acc[5] += kt * p2.y; acc[6] += kt * p2.z; acc[7] += kt * p2.w;
    }
#pragma unroll
    for (int j = 0; j < kScV3; ++j) acc[j] += e8[j];  // additive term of the state update (reversed scan of the backward: dO^T Qe)
    __syncthreads();  // every thread has finished reading St (step 1) and vps before they change
#pragma unroll
    for (int j = 0; j < kScV3; ++j) St[kk * kScVs + vh * kScV3 + j] = gm * St[kk * kScVs + vh * kScV3 + j] + acc[j];
    __syncthreads();
  }
  for (int e = tid; e < kScVs * kScK; e += kScT) {
    const int v = e / kScK, k = e % kScK;
    S_out[((size_t)h * V + vs + v) * kScK + k] = St[k * kScVs + v];
  }
}
static_assert(kScV1 == 4 && kScV3 == 8, "the unrolled accumulators above are written for 512 threads");
}  // namespace pear

// W, Qe, Kt: fp32 [H, n, 64, 128]; U, O, VP: fp32 [H, n, 64, V]; A: fp32 [H, n, 64, 64]; gamma: fp32 [H, n]; S0 (may be
// null), S_out: fp32 [H, V, 128]; E (may be null), S_hist (may be null): fp32 [H, n, V, 128]; O and VP may be null.
// V a multiple of 32.
PEAR_API int pear_gdn_chunk_loop(const float* W, const float* U, const float* Qe, const float* A, const float* Kt, const float* gamma,
                                 const float* S0, const float* E, float* O, float* S_out, float* S_hist, float* VP, int H, int n_chunks,
                                 int V, void* stream) {
  using namespace pear;
  if (V % kScVs || H <= 0 || n_chunks <= 0) return (int)cudaErrorInvalidValue;
  constexpr int smem = (2 * kScK * kScPad + kScC * kScK + kScC * kScPad + kScK * kScVs + kScC * kScVs) * 4;
  static bool configured = false;
  if (!configured) {
    PEAR_CUDA_CHECK(cudaFuncSetAttribute(gdn_chunk_loop_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  gdn_chunk_loop_kernel<<<dim3(H, V / kScVs), kScT, smem, (cudaStream_t)stream>>>(W, U, Qe, A, Kt, gamma, S0, E, O, S_out, S_hist, VP, n_chunks, V);
  PEAR_LAUNCH_CHECK();
  return 0;
}
