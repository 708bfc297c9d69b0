// Causal variable-length attention forward for head dimension 256 with grouped KV heads on the sm_100a tensor cores
// (training forward without gradients, rollout prefill; upstream calls FlashAttention-4 / TensorRT-LLM context FMHA
// here: pear/models/qwen3_5/trainer/blackwell/ulysses_attention.py:144, rollout/blackwell/attention.py).
//
// One CTA per (sequence, 128 query rows, query head), 11 warps. S = Q K^T (128 x 128 per KV tile, 16 tcgen05.mma of
// K = 16) and O += P V (128 x 256, 8 MMAs with V read MN-major straight from its row-major tile) accumulate in tensor
// memory (S: two buffers in columns 0..255, O: columns 256..511). Warps 0..7 = softmax, two per TMEM lane quarter
// (same 32 query rows, each half of the tile's keys and half of O's columns); 8 = TMA producer of Q and K; 9 = MMA
// issuer; 10 = TMA producer of V. The softmax warps read S with tcgen05.ld, keep the running maximum and sum, rescale O
// in tensor memory only when a row maximum grew by more than 2^8, and write P as bf16 into shared memory in the
// 128-byte-swizzled K-major layout the MMA reads. The tensor pipe runs S0, S1, PV0, S2, PV1, ...: the scores of tile
// j+1 are ready before the softmax warps finish tile j. All waits are bounded and report through `status`.
#include "common.cuh"

#include <cudaTypedefs.h>
#include <cuda_bf16.h>
#include <cfloat>

namespace pear {

constexpr int kHd = 256, kQT = 128, kKT = 128;
constexpr int kAttnThreads = 352;
constexpr uint32_t kPanel = 128 * 128;  // bytes of one [128 rows x 64 bf16] swizzled panel
constexpr uint32_t kQOff = 0, kKOff = 4 * kPanel, kVOff = 8 * kPanel, kPOff = 12 * kPanel, kBarOff = 14 * kPanel, kXchOff = kBarOff + 256;
constexpr uint32_t kAlignSlack = 768;  // what is left of 227 KB for rounding the dynamic shared memory base up to 1024 bytes
constexpr uint32_t kTmemCols = 512, kTmemS = 0, kTmemO = 256;  // S: two buffers of 128 columns, O: 256 columns

struct AttnBars {
  uint64_t q_full, k_full, k_empty, v_full, v_empty, s_full[2], p_full, o_done;
  uint32_t tmem_base;
};

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tcgen05_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// MN-major operand tile with the 128-byte swizzle: rows of 128 bytes along MN (64 bf16), 8 K rows per 1024-byte atom;
// `lbo` = bytes between 64-element MN groups, 8-row K groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// One thread polls, the rest of the warp follows once the phase has completed (many pollers slow the tensor core's
// shared-memory reads).
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, int lane, int* status) {
  bool ok = true;
  if (lane == 0) ok = mbar_wait_bounded(bar, parity, status);
  ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  if (ok && lane != 0) ok = mbar_wait_bounded(bar, parity, status);
  return __all_sync(0xffffffffu, ok);
}

__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, float* __restrict__ lse,
                const int* __restrict__ cu_q, const int* __restrict__ cu_k, int batch, int heads_q, int heads_kv, int ldo,
                int total_q, float scale, int causal, int* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  if ((uint32_t)(smem - smem_raw) > kAlignSlack) {  // never seen: the base of dynamic shared memory is 1024-byte aligned
    if (threadIdx.x == 0) set_status(status, PEAR_ERR_SMEM_ALIGN);
    return;
  }
  AttnBars* bars = (AttnBars*)(smem + kBarOff);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // which (sequence, query tile) this CTA owns; the last tiles (most keys under the causal mask) start first
  int slot = gridDim.x - 1 - blockIdx.x, b = 0, q0 = -1;
  for (; b < batch; ++b) {
    const int nt = (cu_q[b + 1] - cu_q[b] + kQT - 1) / kQT;
    if (slot < nt) { q0 = slot * kQT; break; }
    slot -= nt;
  }
  if (q0 < 0) return;
  const int h = blockIdx.y, hk = h / (heads_q / heads_kv);
  const int q_row0 = cu_q[b] + q0, lq = cu_q[b + 1] - cu_q[b];
  const int k_row0 = cu_k[b], lk = cu_k[b + 1] - cu_k[b];
  const int off = lk - lq;  // query i sees keys 0 .. i + off
  const int kv_end = causal ? max(0, min(lk, q0 + kQT + off)) : lk;
  const int ntiles = (kv_end + kKT - 1) / kKT;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    mbar_init(&bars->k_full, 1); mbar_init(&bars->k_empty, 1);
    mbar_init(&bars->v_full, 1); mbar_init(&bars->v_empty, 1);
    mbar_init(&bars->s_full[0], 1); mbar_init(&bars->s_full[1], 1);
    mbar_init(&bars->p_full, 8); mbar_init(&bars->o_done, 1);
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 8) {
    // ---------------------------------------------------------------------------------------- Q and K producer
    if (lane == 0 && ntiles > 0) {
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_k);
      mbar_expect_tx(&bars->q_full, 4 * kPanel);
      for (int p = 0; p < 4; ++p) tma_load_2d(smem + kQOff + p * kPanel, &map_q, h * kHd + p * 64, q_row0, &bars->q_full);
      for (int j = 0; j < ntiles; ++j) {
        if (j > 0 && !mbar_wait_bounded(&bars->k_empty, (j - 1) & 1, status)) break;
        mbar_expect_tx(&bars->k_full, 4 * kPanel);
        for (int p = 0; p < 4; ++p)
          tma_load_2d(smem + kKOff + p * kPanel, &map_k, hk * kHd + p * 64, k_row0 + j * kKT, &bars->k_full);
      }
    }
  } else if (warp == 10) {
    // ---------------------------------------------------------------------------------------- V producer
    if (lane == 0) {
      prefetch_tensormap(&map_v);
      for (int j = 0; j < ntiles; ++j) {
        if (j > 0 && !mbar_wait_bounded(&bars->v_empty, (j - 1) & 1, status)) break;
        mbar_expect_tx(&bars->v_full, 4 * kPanel);
        for (int p = 0; p < 4; ++p)
          tma_load_2d(smem + kVOff + p * kPanel, &map_v, hk * kHd + p * 64, k_row0 + j * kKT, &bars->v_full);
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------------------------------- MMA issuer
    if (lane == 0 && ntiles > 0) {
      constexpr uint32_t idesc_s = umma_idesc_f16(kQT, kKT, 1);
      constexpr uint32_t idesc_o = umma_idesc_f16(kQT, kHd, 1) | (1u << 16);  // B (= V) MN-major
      const uint32_t q_addr = smem_u32(smem + kQOff), k_addr = smem_u32(smem + kKOff), v_addr = smem_u32(smem + kVOff),
                     p_addr = smem_u32(smem + kPOff);
      auto issue_s = [&](int j) -> bool {
        if (!mbar_wait_bounded(&bars->k_full, j & 1, status)) return false;
        tcgen05_fence_after();
#pragma unroll
        for (int kk = 0; kk < kHd / 16; ++kk) {
          const uint64_t da = umma_desc_sw128(q_addr + (kk >> 2) * kPanel) + (uint64_t)((kk & 3) * 2);
          const uint64_t db = umma_desc_sw128(k_addr + (kk >> 2) * kPanel) + (uint64_t)((kk & 3) * 2);
          umma_f16(tmem + kTmemS + (j & 1) * kKT, da, db, idesc_s, kk != 0 ? 1u : 0u);
        }
        tcgen05_commit(&bars->k_empty);
        tcgen05_commit(&bars->s_full[j & 1]);
        return true;
      };
      // order on the tensor pipe: S0, S1, PV0, S2, PV1, S3, ... so that the softmax of tile j+1 always finds its S ready
      bool ok = mbar_wait_bounded(&bars->q_full, 0, status);
      if (ok) { tcgen05_fence_after(); ok = issue_s(0); }
      if (ok && ntiles > 1) ok = issue_s(1);
      for (int j = 0; j < ntiles && ok; ++j) {
        ok = mbar_wait_bounded(&bars->p_full, j & 1, status) && mbar_wait_bounded(&bars->v_full, j & 1, status);
        if (!ok) break;
        tcgen05_fence_after();
#pragma unroll
        for (int kk = 0; kk < kKT / 16; ++kk) {
          const uint64_t da = umma_desc_sw128(p_addr + (kk >> 2) * kPanel) + (uint64_t)((kk & 3) * 2);
          const uint64_t db = umma_desc_mn_sw128(v_addr + kk * 2048, kPanel);
          umma_f16(tmem + kTmemO, da, db, idesc_o, (j | kk) != 0 ? 1u : 0u);
        }
        tcgen05_commit(&bars->v_empty);
        tcgen05_commit(&bars->o_done);
        // P of tile j has arrived, so the softmax warps have finished reading S buffer j & 1
        if (j + 2 < ntiles) ok = issue_s(j + 2);
      }
    }
  } else {
    // ---------------------------------------------------------------------------------------- softmax + epilogue
    // Two warps per TMEM lane quarter: both own the same 32 query rows, `half` 0 takes keys 0..63 of the tile and O
    // columns 0..127, `half` 1 the rest. They exchange the tile's row maximum through shared memory (one 64-thread
    // named barrier per tile), keep separate partial sums, and take identical rescale decisions.
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;     // query row of the tile = TMEM lane
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const uint32_t s_base = lane_base + kTmemS + half * 64, o_cols = lane_base + kTmemO + half * 128;
    const float sl2 = scale * 1.4426950408889634f;
    const int qi = q0 + row;                 // position inside the sequence
    const int last_key = causal ? min(lk - 1, qi + off) : lk - 1;
    float m_ref = -INFINITY, l_run = 0.f;    // m_ref: the (possibly stale) maximum the exponents refer to
    uint8_t* p_row = smem + kPOff + half * kPanel + row * 128;
    float* xch = (float*)(smem + kXchOff);   // [2 tiles][2 halves][128 rows]
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      ok = warp_wait(&bars->s_full[j & 1], (j >> 1) & 1, lane, status);
      if (!ok) break;
      tcgen05_fence_after();
      const int k0 = j * kKT + half * 64;
      // rows of this tile whose last visible key lies before the tile's end need the mask (the diagonal and the tail)
      const bool masked = j * kKT + kKT - 1 > (causal ? min(lk - 1, q0 + off) : lk - 1);
      const uint32_t s_cols = s_base + (j & 1) * kKT;
      uint32_t ra[32], rb[32];  // this thread's 64 scores stay in registers for both passes
      tmem_ld_32x32b_x32(s_cols, ra);
      tmem_ld_32x32b_x32(s_cols + 32, rb);
      tcgen05_wait_ld();
      float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
      if (masked) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (k0 + i <= last_key) m0 = fmaxf(m0, __uint_as_float(ra[i]));
          if (k0 + 32 + i <= last_key) m1 = fmaxf(m1, __uint_as_float(rb[i]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          m0 = fmaxf(m0, __uint_as_float(ra[i])); m1 = fmaxf(m1, __uint_as_float(ra[i + 1]));
          m2 = fmaxf(m2, __uint_as_float(rb[i])); m3 = fmaxf(m3, __uint_as_float(rb[i + 1]));
        }
      }
      float m_tile = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      float* x = xch + (j & 1) * 256;
      x[half * 128 + row] = m_tile;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
      m_tile = fmaxf(m_tile, x[(half ^ 1) * 128 + row]);
      const float m_new = fmaxf(m_ref, m_tile);
      // lazy rescale: the reference moves only when some row's maximum grew by more than 2^8 (exponents stay small)
      const bool grow = (m_new - m_ref) * sl2 > 8.f;
      const bool any = __any_sync(0xffffffffu, grow);
      const float m_use = any ? m_new : m_ref;
      const float e_ref = m_use == -INFINITY ? 0.f : m_use * sl2;
      uint32_t pk[32];
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint32_t(&r)[32] = c == 0 ? ra : rb;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = ex2_approx(fmaf(__uint_as_float(r[i]), sl2, -e_ref));
          float p1 = ex2_approx(fmaf(__uint_as_float(r[i + 1]), sl2, -e_ref));
          if (masked) {
            if (k0 + c * 32 + i > last_key) p0 = 0.f;
            if (k0 + c * 32 + i + 1 > last_key) p1 = 0.f;
          }
          sum0 += p0;
          sum1 += p1;
          const __nv_bfloat162 pp = __floats2bfloat162_rn(p0, p1);
          pk[c * 16 + (i >> 1)] = *(const uint32_t*)&pp;
        }
      }
      const float alpha = !any ? 1.f : (m_ref == -INFINITY ? 0.f : ex2_approx(m_ref * sl2 - e_ref));
      l_run = l_run * alpha + (sum0 + sum1);
      if (j > 0) {
        ok = warp_wait(&bars->o_done, (j - 1) & 1, lane, status);
        if (!ok) break;
        tcgen05_fence_after();
        if (any) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            tmem_ld_32x32b_x32(o_cols + c * 32, ra);
            tcgen05_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) ra[i] = __float_as_uint(__uint_as_float(ra[i]) * alpha);
            tmem_st_32x32b_x32(o_cols + c * 32, ra);
          }
          tcgen05_wait_st();
        }
      }
      m_ref = m_use;
      // P row: this half's 64 keys = one panel, 8 chunks of 16 bytes, chunk index xor (row % 8) inside the 128-byte line
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const uint4 v = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
        *(uint4*)(p_row + ((ch ^ (row & 7)) << 4)) = v;
      }
      fence_proxy_async();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full);
    }
    // epilogue: O / l as bf16, log-sum-exp in natural units; the two halves add their partial sums first
    const bool valid = qi < lq;
    if (ntiles > 0 && ok) ok = warp_wait(&bars->o_done, (ntiles - 1) & 1, lane, status);
    float* xl = xch + (ntiles & 1) * 256;  // the slot the last tile did not use
    xl[half * 128 + row] = l_run;
    asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
    l_run += xl[(half ^ 1) * 128 + row];
    if (ok) {
      tcgen05_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* dst = out + (size_t)(q_row0 + row) * ldo + h * kHd + half * 128;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        if (ntiles > 0) {
          tmem_ld_32x32b_x32(o_cols + c * 32, r);
          tcgen05_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 v;
            __nv_bfloat162 a0 = __floats2bfloat162_rn(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
            __nv_bfloat162 a1 = __floats2bfloat162_rn(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
            __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
            __nv_bfloat162 a3 = __floats2bfloat162_rn(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
            v.x = *(uint32_t*)&a0; v.y = *(uint32_t*)&a1; v.z = *(uint32_t*)&a2; v.w = *(uint32_t*)&a3;
            *(uint4*)(dst + c * 32 + i) = v;
          }
        }
      }
      if (valid && lse && half == 0) lse[(size_t)h * total_q + q_row0 + row] = l_run > 0.f ? m_ref * scale + logf(l_run) : -INFINITY;
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 9) {
    tcgen05_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------ host side
static PFN_cuTensorMapEncodeTiled_v12000 attn_get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    cudaDriverEntryPointQueryResult q;
    void* p = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
  }
  return fn;
}

// [rows, cols] bf16 with row stride ld (elements): boxes of 128 rows x 64 columns, 128-byte swizzle, zero fill outside.
static int attn_make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld) {
  auto enc = attn_get_encode();
  if (!enc) return (int)cudaErrorNotSupported;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, 128u};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

}  // namespace pear

// Packed variable-length attention forward, head dimension 256. q [total_q, heads_q, 256], k and v [total_k, heads_kv,
// 256] bf16 with row strides ldq / ldk / ldv (elements, multiples of 8; heads are 256 elements apart); cu_q, cu_k:
// device int32 [batch + 1] row offsets of the sequences; every sequence needs keys >= queries, the queries are its last
// positions (chunked prefill). out [total_q, heads_q, 256] bf16 with row stride ldo; lse (may be null) [heads_q, total_q]
// fp32. `status` is a device int that a bounded wait sets on expiry.
PEAR_API int pear_attn_varlen_fwd_hd256(const void* q, const void* k, const void* v, void* out, float* lse, const int* cu_q,
                                        const int* cu_k, int batch, int total_q, int total_k, int heads_q, int heads_kv,
                                        int ldq, int ldk, int ldv, int ldo, float scale, int causal, int* status,
                                        void* stream) {
  using namespace pear;
  if (batch <= 0 || total_q <= 0) return 0;
  if (heads_kv <= 0 || heads_q % heads_kv) return (int)cudaErrorInvalidValue;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8) || ((uintptr_t)q % 16) || ((uintptr_t)k % 16) || ((uintptr_t)v % 16) ||
      ((uintptr_t)out % 16))
    return (int)cudaErrorInvalidValue;
  CUtensorMap mq, mk, mv;
  int r = attn_make_map(&mq, q, total_q, heads_q * kHd, ldq);
  if (r) return r;
  r = attn_make_map(&mk, k, total_k, heads_kv * kHd, ldk);
  if (r) return r;
  r = attn_make_map(&mv, v, total_k, heads_kv * kHd, ldv);
  if (r) return r;
  constexpr int smem = (int)kXchOff + 2048 + (int)kAlignSlack;  // = 227 KB, the most one CTA can have
  static bool configured = false;
  if (!configured) {
    PEAR_CUDA_CHECK(cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  const dim3 grid((total_q + kQT - 1) / kQT + batch, heads_q);
  attn_fwd_kernel<<<grid, kAttnThreads, smem, (cudaStream_t)stream>>>(mq, mk, mv, (__nv_bfloat16*)out, lse, cu_q, cu_k, batch,
                                                                      heads_q, heads_kv, ldo, total_q, scale, causal, status);
  PEAR_LAUNCH_CHECK();
  return 0;
}
