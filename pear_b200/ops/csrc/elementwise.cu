// Memory-bound trainer/rollout ops for sm_100a: (1+w) RMSNorm and residual-add RMSNorm fwd/bwd, gated RMSNorm fwd/bwd,
// SwiGLU fwd/bwd, sigmoid output gate fwd/bwd, rotary embedding. Each is one pass over its operands with 16-byte
// accesses and fp32 math; outputs are rounded once. (Counterparts of the upstream Triton kernels
// pear/models/qwen3_5/trainer/rms_norm.py:111-160, trainer/gdn.py:206-275, trainer/mlp.py:9-60, trainer/attention.py:24-67.)
#include "common.cuh"

namespace pear {

enum DType : int { DT_F32 = 0, DT_BF16 = 1 };

__device__ __forceinline__ float ld_as_f32(const void* p, size_t i, int dt) {
  return dt == DT_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ void st_from_f32(void* p, size_t i, int dt, float v) {
  if (dt == DT_F32) ((float*)p)[i] = v; else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}

// 4 consecutive elements
__device__ __forceinline__ float4 ld4(const void* p, size_t i, int dt) {
  if (dt == DT_F32) return *(const float4*)((const float*)p + i);
  const uint2 u = *(const uint2*)((const __nv_bfloat16*)p + i);
  const __nv_bfloat162 a = *(const __nv_bfloat162*)&u.x, b = *(const __nv_bfloat162*)&u.y;
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void st4(void* p, size_t i, int dt, float4 v) {
  if (dt == DT_F32) { *(float4*)((float*)p + i) = v; return; }
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u; u.x = *(uint32_t*)&a; u.y = *(uint32_t*)&b;
  *(uint2*)((__nv_bfloat16*)p + i) = u;
}

// ---------------------------------------------------------------------------------------------------------------------
// RMSNorm forward: optional residual add (res_in + x -> res_out), y = r * rstd * (w + one_plus). One row per group of
// `tpr` threads (tpr = 32 for short rows: one warp per row; = blockDim for long rows).
// ---------------------------------------------------------------------------------------------------------------------
template <bool WARP_ROWS>
__global__ void rms_norm_fwd_kernel(const void* __restrict__ x, int x_dt, const float* __restrict__ res_in,
                                    const float* __restrict__ w, void* __restrict__ y, int y_dt,
                                    float* __restrict__ res_out, float* __restrict__ rstd_out, int rows, int dim,
                                    float eps, float w_offset) {
  __shared__ float scratch[32];
  const int lane = threadIdx.x & 31;
  const int row = WARP_ROWS ? blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5) : blockIdx.x;
  if (WARP_ROWS && row >= rows) return;
  const int tpr = WARP_ROWS ? 32 : blockDim.x;
  const int tin = WARP_ROWS ? lane : threadIdx.x;
  const size_t base = (size_t)row * dim;
  float ss = 0.f;
  for (int i = tin * 4; i < dim; i += tpr * 4) {
    float4 v = ld4(x, base + i, x_dt);
    if (res_in) {
      const float4 r = *(const float4*)(res_in + base + i);
      v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
    }
    if (res_out) *(float4*)(res_out + base + i) = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = WARP_ROWS ? warp_sum(ss) : block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)dim + eps);
  if (rstd_out && tin == 0) rstd_out[row] = rstd;
  for (int i = tin * 4; i < dim; i += tpr * 4) {
    float4 v;
    if (res_out) v = *(const float4*)(res_out + base + i);
    else {
      v = ld4(x, base + i, x_dt);
      if (res_in) { const float4 r = *(const float4*)(res_in + base + i); v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w; }
    }
    const float4 g = *(const float4*)(w + i);
    v.x *= rstd * (g.x + w_offset); v.y *= rstd * (g.y + w_offset);
    v.z *= rstd * (g.z + w_offset); v.w *= rstd * (g.w + w_offset);
    st4(y, base + i, y_dt, v);
  }
}

// RMSNorm backward: r = normalised input (fp32 [rows, dim]); dx = rstd * (g - r * rstd^2 * mean(g * r)) (+ dres),
// g = dy * (w + off); dw[i] += sum_rows dy * r * rstd (fp32 atomics onto a zeroed buffer).
template <bool WARP_ROWS>
__global__ void rms_norm_bwd_kernel(const float* __restrict__ dy, const float* __restrict__ r, const float* __restrict__ w,
                                    const float* __restrict__ rstd_in, const float* __restrict__ dres,
                                    float* __restrict__ dx, float* __restrict__ dw, int rows, int dim, float w_offset) {
  __shared__ float scratch[32];
  const int lane = threadIdx.x & 31;
  const int row = WARP_ROWS ? blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5) : blockIdx.x;
  if (WARP_ROWS && row >= rows) return;
  const int tpr = WARP_ROWS ? 32 : blockDim.x;
  const int tin = WARP_ROWS ? lane : threadIdx.x;
  const size_t base = (size_t)row * dim;
  const float rstd = rstd_in[row];
  float dot = 0.f;
  for (int i = tin * 4; i < dim; i += tpr * 4) {
    const float4 g = *(const float4*)(dy + base + i), v = *(const float4*)(r + base + i), ww = *(const float4*)(w + i);
    dot += g.x * (ww.x + w_offset) * v.x + g.y * (ww.y + w_offset) * v.y + g.z * (ww.z + w_offset) * v.z +
           g.w * (ww.w + w_offset) * v.w;
  }
  dot = WARP_ROWS ? warp_sum(dot) : block_sum(dot, scratch);
  const float c = dot * rstd * rstd / (float)dim;
  for (int i = tin * 4; i < dim; i += tpr * 4) {
    const float4 g = *(const float4*)(dy + base + i), v = *(const float4*)(r + base + i), ww = *(const float4*)(w + i);
    float4 o;
    o.x = rstd * (g.x * (ww.x + w_offset) - v.x * c); o.y = rstd * (g.y * (ww.y + w_offset) - v.y * c);
    o.z = rstd * (g.z * (ww.z + w_offset) - v.z * c); o.w = rstd * (g.w * (ww.w + w_offset) - v.w * c);
    if (dres) { const float4 e = *(const float4*)(dres + base + i); o.x += e.x; o.y += e.y; o.z += e.z; o.w += e.w; }
    *(float4*)(dx + base + i) = o;
    if (dw) {
      atomicAdd(dw + i, g.x * v.x * rstd); atomicAdd(dw + i + 1, g.y * v.y * rstd);
      atomicAdd(dw + i + 2, g.z * v.z * rstd); atomicAdd(dw + i + 3, g.w * v.w * rstd);
    }
  }
}

// Short rows (dim <= 1024: per-head q / k norms): one warp per row, rows strided over a grid of a few CTAs per SM. The
// weight gradient is summed per CTA in shared memory and flushed with one global atomic per element and CTA (per-row
// global atomics onto the same few hundred addresses serialise: 2.2 ms for 115 k rows of 256 against ~0.1 ms of traffic).
__global__ void __launch_bounds__(256) rms_norm_bwd_rows_kernel(const float* __restrict__ dy, const float* __restrict__ r,
                                                                const float* __restrict__ w, const float* __restrict__ rstd_in,
                                                                const float* __restrict__ dres, float* __restrict__ dx,
                                                                float* __restrict__ dw, int rows, int dim, float w_offset) {
  __shared__ float sdw[1024];
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) sdw[i] = 0.f;
  __syncthreads();
  for (int row = blockIdx.x * wpb + (threadIdx.x >> 5); row < rows; row += gridDim.x * wpb) {
    const size_t base = (size_t)row * dim;
    const float rstd = rstd_in[row];
    float dot = 0.f;
    for (int i = lane * 4; i < dim; i += 128) {
      const float4 g = *(const float4*)(dy + base + i), v = *(const float4*)(r + base + i), ww = *(const float4*)(w + i);
      dot += g.x * (ww.x + w_offset) * v.x + g.y * (ww.y + w_offset) * v.y + g.z * (ww.z + w_offset) * v.z +
             g.w * (ww.w + w_offset) * v.w;
    }
    dot = warp_sum(dot);
    const float c = dot * rstd * rstd / (float)dim;
    for (int i = lane * 4; i < dim; i += 128) {
      const float4 g = *(const float4*)(dy + base + i), v = *(const float4*)(r + base + i), ww = *(const float4*)(w + i);
      float4 o;
      o.x = rstd * (g.x * (ww.x + w_offset) - v.x * c); o.y = rstd * (g.y * (ww.y + w_offset) - v.y * c);
      o.z = rstd * (g.z * (ww.z + w_offset) - v.z * c); o.w = rstd * (g.w * (ww.w + w_offset) - v.w * c);
      if (dres) { const float4 e = *(const float4*)(dres + base + i); o.x += e.x; o.y += e.y; o.z += e.z; o.w += e.w; }
      *(float4*)(dx + base + i) = o;
      if (dw) {
        atomicAdd(sdw + i, g.x * v.x * rstd); atomicAdd(sdw + i + 1, g.y * v.y * rstd);
        atomicAdd(sdw + i + 2, g.z * v.z * rstd); atomicAdd(sdw + i + 3, g.w * v.w * rstd);
      }
    }
  }
  __syncthreads();
  if (dw)
    for (int i = threadIdx.x; i < dim; i += blockDim.x) atomicAdd(dw + i, sdw[i]);
}

// ---------------------------------------------------------------------------------------------------------------------
// Gated RMSNorm over head vectors (dim 128 typical): y = o * rstd * w * silu(z); one warp per row.
// ---------------------------------------------------------------------------------------------------------------------
__global__ void gated_rms_norm_fwd_kernel(const float* __restrict__ o, const float* __restrict__ z,
                                          const float* __restrict__ w, void* __restrict__ y, int y_dt,
                                          float* __restrict__ rstd_out, int rows, int dim, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const size_t base = (size_t)row * dim;
  float ss = 0.f;
  for (int i = lane * 4; i < dim; i += 128) {
    const float4 v = *(const float4*)(o + base + i);
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)dim + eps);
  if (rstd_out && lane == 0) rstd_out[row] = rstd;
  for (int i = lane * 4; i < dim; i += 128) {
    const float4 v = *(const float4*)(o + base + i), zz = *(const float4*)(z + base + i), ww = *(const float4*)(w + i);
    st4(y, base + i, y_dt, make_float4(v.x * rstd * ww.x * silu_f(zz.x), v.y * rstd * ww.y * silu_f(zz.y),
                                       v.z * rstd * ww.z * silu_f(zz.z), v.w * rstd * ww.w * silu_f(zz.w)));
  }
}

__device__ __forceinline__ float dsilu_f(float x) {
  const float s = sigmoid_f(x);
  return s * (1.f + x * (1.f - s));
}

__global__ void gated_rms_norm_bwd_kernel(const float* __restrict__ dy, const float* __restrict__ o,
                                          const float* __restrict__ z, const float* __restrict__ w,
                                          const float* __restrict__ rstd_in, float* __restrict__ d_o,
                                          float* __restrict__ d_z, float* __restrict__ dw, int rows, int dim) {
  // rows strided over the grid; the weight gradient is summed per CTA in shared memory first (dim <= 1024)
  __shared__ float sdw[1024];
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) sdw[i] = 0.f;
  __syncthreads();
  for (int row = blockIdx.x * wpb + (threadIdx.x >> 5); row < rows; row += gridDim.x * wpb) {
    const size_t base = (size_t)row * dim;
    const float rstd = rstd_in[row];
    float dot = 0.f;
    for (int i = lane; i < dim; i += 32) dot += dy[base + i] * w[i] * silu_f(z[base + i]) * o[base + i];
    dot = warp_sum(dot);
    const float c = dot * rstd * rstd / (float)dim;
    for (int i = lane; i < dim; i += 32) {
      const float g = dy[base + i], ov = o[base + i], zv = z[base + i], sz = silu_f(zv);
      d_o[base + i] = rstd * (g * w[i] * sz - ov * c);
      d_z[base + i] = g * ov * rstd * w[i] * dsilu_f(zv);
      atomicAdd(sdw + i, g * ov * rstd * sz);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < dim; i += blockDim.x) atomicAdd(dw + i, sdw[i]);
}

// ---------------------------------------------------------------------------------------------------------------------
// SwiGLU, sigmoid gate
// ---------------------------------------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const float* __restrict__ gate, const float* __restrict__ up, void* __restrict__ y,
                                  int y_dt, size_t n) {
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (size_t)gridDim.x * blockDim.x * 4) {
    const float4 g = *(const float4*)(gate + i), u = *(const float4*)(up + i);
    st4(y, i, y_dt, make_float4(silu_f(g.x) * u.x, silu_f(g.y) * u.y, silu_f(g.z) * u.z, silu_f(g.w) * u.w));
  }
}
__global__ void swiglu_bwd_kernel(const float* __restrict__ dy, const float* __restrict__ gate,
                                  const float* __restrict__ up, float* __restrict__ dgate, float* __restrict__ dup, size_t n) {
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (size_t)gridDim.x * blockDim.x * 4) {
    const float4 d = *(const float4*)(dy + i), g = *(const float4*)(gate + i), u = *(const float4*)(up + i);
    *(float4*)(dgate + i) = make_float4(d.x * u.x * dsilu_f(g.x), d.y * u.y * dsilu_f(g.y), d.z * u.z * dsilu_f(g.z),
                                        d.w * u.w * dsilu_f(g.w));
    *(float4*)(dup + i) = make_float4(d.x * silu_f(g.x), d.y * silu_f(g.y), d.z * silu_f(g.z), d.w * silu_f(g.w));
  }
}
__global__ void sigmoid_gate_fwd_kernel(const float* __restrict__ x, const float* __restrict__ gate, void* __restrict__ y,
                                        int y_dt, size_t n) {
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (size_t)gridDim.x * blockDim.x * 4) {
    const float4 a = *(const float4*)(x + i), g = *(const float4*)(gate + i);
    st4(y, i, y_dt, make_float4(a.x * sigmoid_f(g.x), a.y * sigmoid_f(g.y), a.z * sigmoid_f(g.z), a.w * sigmoid_f(g.w)));
  }
}
__global__ void sigmoid_gate_bwd_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                        const float* __restrict__ gate, float* __restrict__ dx, float* __restrict__ dgate, size_t n) {
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (size_t)gridDim.x * blockDim.x * 4) {
    const float4 d = *(const float4*)(dy + i), a = *(const float4*)(x + i), g = *(const float4*)(gate + i);
    const float s0 = sigmoid_f(g.x), s1 = sigmoid_f(g.y), s2 = sigmoid_f(g.z), s3 = sigmoid_f(g.w);
    *(float4*)(dx + i) = make_float4(d.x * s0, d.y * s1, d.z * s2, d.w * s3);
    *(float4*)(dgate + i) = make_float4(d.x * a.x * s0 * (1.f - s0), d.y * a.y * s1 * (1.f - s1),
                                        d.z * a.z * s2 * (1.f - s2), d.w * a.w * s3 * (1.f - s3));
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Rotary embedding on the first 2*half channels of x [T, H, D], pairing channel i with i + half. `sign` = -1 gives the
// transpose (backward). cos/sin: fp32 [T, half].
// ---------------------------------------------------------------------------------------------------------------------
__global__ void rope_kernel(const float* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn,
                            float* __restrict__ y, int T, int H, int D, int half, float sign) {
  const size_t n = (size_t)T * H * D;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int d = (int)(i % D);
    const size_t th = i / D;
    const int t = (int)(th / H);
    float v = x[i];
    if (d < half) {
      v = v * cs[(size_t)t * half + d] - sign * x[i + half] * sn[(size_t)t * half + d];
    } else if (d < 2 * half) {
      v = v * cs[(size_t)t * half + d - half] + sign * x[i - half] * sn[(size_t)t * half + d - half];
    }
    y[i] = v;
  }
}

}  // namespace pear

using namespace pear;

static inline int grid_for(size_t n, int block, int per_thread) {
  size_t g = (n + (size_t)block * per_thread - 1) / ((size_t)block * per_thread);
  return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

PEAR_API int pear_rms_norm_fwd(const void* x, int x_dt, const float* res_in, const float* w, void* y, int y_dt,
                               float* res_out, float* rstd, int rows, int dim, float eps, int one_plus, void* stream) {
  if (dim % 4) return (int)cudaErrorInvalidValue;
  const float off = one_plus ? 1.f : 0.f;
  if (dim <= 1024) {
    const int wpb = 8;
    rms_norm_fwd_kernel<true><<<(rows + wpb - 1) / wpb, wpb * 32, 0, (cudaStream_t)stream>>>(x, x_dt, res_in, w, y, y_dt, res_out,
                                                                                         rstd, rows, dim, eps, off);
  } else {
    rms_norm_fwd_kernel<false><<<rows, 256, 0, (cudaStream_t)stream>>>(x, x_dt, res_in, w, y, y_dt, res_out, rstd, rows, dim, eps, off);
  }
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_rms_norm_bwd(const float* dy, const float* r, const float* w, const float* rstd, const float* dres, float* dx,
                               float* dw, int rows, int dim, int one_plus, void* stream) {
  if (dim % 4) return (int)cudaErrorInvalidValue;
  const float off = one_plus ? 1.f : 0.f;
  if (dim <= 1024) {
    const int wpb = 8, want = (rows + wpb - 1) / wpb, cap = 148 * 8;
    rms_norm_bwd_rows_kernel<<<want < cap ? want : cap, wpb * 32, 0, (cudaStream_t)stream>>>(dy, r, w, rstd, dres, dx, dw, rows, dim, off);
  } else {
    rms_norm_bwd_kernel<false><<<rows, 256, 0, (cudaStream_t)stream>>>(dy, r, w, rstd, dres, dx, dw, rows, dim, off);
  }
  PEAR_LAUNCH_CHECK();
  return 0;
}

PEAR_API int pear_gated_rms_norm_fwd(const float* o, const float* z, const float* w, void* y, int y_dt, float* rstd, int rows,
                                     int dim, float eps, void* stream) {
  if (dim % 4) return (int)cudaErrorInvalidValue;
  gated_rms_norm_fwd_kernel<<<(rows + 7) / 8, 256, 0, (cudaStream_t)stream>>>(o, z, w, y, y_dt, rstd, rows, dim, eps);
  PEAR_LAUNCH_CHECK();
  return 0;
}
PEAR_API int pear_gated_rms_norm_bwd(const float* dy, const float* o, const float* z, const float* w, const float* rstd,
                                     float* d_o, float* d_z, float* dw, int rows, int dim, void* stream) {
  if (dim > 1024) return (int)cudaErrorInvalidValue;
  const int want = (rows + 7) / 8, cap = 148 * 8;
  gated_rms_norm_bwd_kernel<<<want < cap ? want : cap, 256, 0, (cudaStream_t)stream>>>(dy, o, z, w, rstd, d_o, d_z, dw, rows, dim);
  PEAR_LAUNCH_CHECK();
  return 0;
}
PEAR_API int pear_swiglu_fwd(const float* gate, const float* up, void* y, int y_dt, long long n, void* stream) {
  if (n % 4) return (int)cudaErrorInvalidValue;
  swiglu_fwd_kernel<<<grid_for(n, 256, 4), 256, 0, (cudaStream_t)stream>>>(gate, up, y, y_dt, (size_t)n);
  PEAR_LAUNCH_CHECK();
  return 0;
}
PEAR_API int pear_swiglu_bwd(const float* dy, const float* gate, const float* up, float* dgate, float* dup, long long n, void* stream) {
  if (n % 4) return (int)cudaErrorInvalidValue;
  swiglu_bwd_kernel<<<grid_for(n, 256, 4), 256, 0, (cudaStream_t)stream>>>(dy, gate, up, dgate, dup, (size_t)n);
  PEAR_LAUNCH_CHECK();
  return 0;
}
PEAR_API int pear_sigmoid_gate_fwd(const float* x, const float* gate, void* y, int y_dt, long long n, void* stream) {
  if (n % 4) return (int)cudaErrorInvalidValue;
  sigmoid_gate_fwd_kernel<<<grid_for(n, 256, 4), 256, 0, (cudaStream_t)stream>>>(x, gate, y, y_dt, (size_t)n);
  PEAR_LAUNCH_CHECK();
  return 0;
}
PEAR_API int pear_sigmoid_gate_bwd(const float* dy, const float* x, const float* gate, float* dx, float* dgate, long long n, void* stream) {
  if (n % 4) return (int)cudaErrorInvalidValue;
  sigmoid_gate_bwd_kernel<<<grid_for(n, 256, 4), 256, 0, (cudaStream_t)stream>>>(dy, x, gate, dx, dgate, (size_t)n);
  PEAR_LAUNCH_CHECK();
  return 0;
}
PEAR_API int pear_rope(const float* x, const float* cs, const float* sn, float* y, int T, int H, int D, int half, float sign, void* stream) {
  const size_t n = (size_t)T * H * D;
  rope_kernel<<<grid_for(n, 256, 1), 256, 0, (cudaStream_t)stream>>>(x, cs, sn, y, T, H, D, half, sign);
  PEAR_LAUNCH_CHECK();
  return 0;
}
