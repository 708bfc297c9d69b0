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
