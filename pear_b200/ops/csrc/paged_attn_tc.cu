// Paged decode / verify attention for head dimension 256 on the sm_100a tensor cores, sigmoid output gate fused.
// (Upstream: rollout/blackwell/csrc/verify_attn.cu:479-587 — tcgen05 paged attention of verify rows; FlashInfer's
// TensorRT-LLM decode kernel for single rows: rollout/blackwell/attention.py:395.)
//
// One CTA per (sequence, KV head). All query rows that share the KV head form the M dimension of the score MMA:
// row r = g * T + t for query head g of the group and step row t (R = group * T <= 128 rows, the rest of the 128 TMEM
// lanes idle), so every K / V page is read from HBM once per KV head whatever the group size. KV pages are 16 tokens
// of [page][16][Hkv][256] bf16; a tile of 128 keys = 8 pages, each fetched as 4 TMA boxes of 16 rows x 64 columns
// (128-byte swizzle) into the K-major tile layout the MMA reads; V is used MN-major straight from the same layout.
// Pipeline and warp roles are those of the training forward kernel (attn_tcgen05.cu): S = Q K^T and O += P V accumulate
// in tensor memory, eight softmax warps (two per TMEM lane quarter) keep running maxima and sums with the lazy rescale,
// P goes back to shared memory as bf16. Row (g, t) sees keys 0 .. ctx + t. The epilogue divides by the row sum,
// multiplies by sigmoid(gate) read from the projection output and writes bf16 [row][Hq * 256].
//
// Shared prefixes (the samples of one prompt group share their prompt's KV pages; a 6k-token prefix of an 8k context is
// 3/4 of all page reads): with an item table, a CTA can serve SEVERAL sequences at once over a key range whose pages
// they share - their query rows stack in the M dimension (5 sequences x 24 rows fill the 128 lanes that one sequence
// leaves mostly idle), so the shared pages cross L2 -> shared memory once per group instead of once per sequence. Such
// items, and the per-sequence items over the rest of the context, write un-normalised partial outputs with their running
// maximum and sum; a small kernel merges a row's partials, applies the gate and writes bf16.
// Every wait is bounded; no cluster multicast.
#include "common.cuh"

#include <cudaTypedefs.h>
#include <cuda_bf16.h>
#include <cfloat>

namespace pear {

constexpr int kPaHd = 256, kPaQT = 128, kPaKT = 128;
constexpr int kPaThreads = 352;
constexpr uint32_t kPaPanel = 128 * 128;
constexpr uint32_t kPaQOff = 0, kPaKOff = 4 * kPaPanel, kPaVOff = 8 * kPaPanel, kPaPOff = 12 * kPaPanel, kPaBarOff = 14 * kPaPanel,
                   kPaXchOff = kPaBarOff + 256;
constexpr uint32_t kPaAlignSlack = 768;
constexpr uint32_t kPaTmemCols = 512, kPaTmemS = 0, kPaTmemO = 256;

struct PaBars {
  uint64_t k_full, k_empty, v_full, v_empty, s_full[2], p_full, o_done;
  uint32_t tmem_base;
};

__device__ __forceinline__ void pa_tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
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
__device__ __forceinline__ float pa_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void pa_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ uint64_t pa_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// A wait gives up only on its OWN poll budget (never because another CTA reported a problem): the two softmax warps of
// a lane quarter meet at a named barrier every tile, so they must reach the same decision from the same mbarrier.
__device__ __forceinline__ bool pa_wait(uint64_t* bar, uint32_t parity, int* status) {
  if (mbar_wait_bounded(bar, parity, nullptr)) return true;
  set_status(status, PEAR_ERR_MBAR_TIMEOUT);
  return false;
}
__device__ __forceinline__ bool pa_warp_wait(uint64_t* bar, uint32_t parity, int lane, int* status) {
  bool ok = true;
  if (lane == 0) ok = pa_wait(bar, parity, status);
  ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  if (ok && lane != 0) ok = pa_wait(bar, parity, status);
  return __all_sync(0xffffffffu, ok);
}

// An item of the work table: `nseq` sequences of the batch (seq[0 .. nseq), at most 16; their pages agree on the item's
// key range), keys [key_begin, key_end) (key_begin a multiple of 128; key_end < 0: up to every sequence's own context end,
// causal inside the step's rows), partial slot `slot`; the item also marks slots clear_from .. clear_to - 1 of its rows empty.
constexpr int kPaItemSeqs = 16;
struct PaItem {
  int nseq, key_begin, key_end, slot, clear_from, clear_to, pad1, pad2;
  int seq[kPaItemSeqs];
};

__global__ void __launch_bounds__(kPaThreads, 1)
paged_attn_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const __nv_bfloat16* __restrict__ q,
                     const int* __restrict__ block_table, int max_blocks, const int* __restrict__ ctx, int T, int Hq, int Hkv, float scale,
                     const float* __restrict__ gate_src, int gate_ld, int gated, __nv_bfloat16* __restrict__ out, int* status,
                     const PaItem* __restrict__ items, float* __restrict__ part_o, float* __restrict__ part_ml, int rows_total) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  grid_dependency_trigger();
  if ((uint32_t)(smem - smem_raw) > kPaAlignSlack) {
    grid_dependency_wait();
    if (threadIdx.x == 0) set_status(status, PEAR_ERR_SMEM_ALIGN);
    return;
  }
  // zero Q, K, V tiles (rows beyond R and pages beyond the context must hold finite values) while the kernel ahead in the
  // stream drains; every global access follows the wait
  for (uint32_t i = threadIdx.x; i < (12 * kPaPanel) / 16; i += kPaThreads) ((uint4*)smem)[i] = make_uint4(0u, 0u, 0u, 0u);
  grid_dependency_wait();
  PaBars* bars = (PaBars*)(smem + kPaBarOff);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.y;
  PaItem it;
  if (items) it = items[blockIdx.x];
  else { it.nseq = 1; it.key_begin = 0; it.key_end = -1; it.slot = 0; it.clear_from = it.clear_to = 0; it.seq[0] = blockIdx.x; }
  if (it.nseq <= 0) return;
  const int b = it.seq[0];
  const int group = Hq / Hkv, RS = group * T, R = it.nseq * RS;  // rows per sequence, rows of the item
  int c_max = -1;
  for (int s2 = 0; s2 < it.nseq; ++s2) c_max = max(c_max, ctx[it.seq[s2]]);
  if (c_max < 0) return;
  const int kv_end = it.key_end >= 0 ? it.key_end : c_max + T;  // keys key_begin .. kv_end - 1 are visited
  const int jt0 = it.key_begin / kPaKT;
  const int ntiles = max(0, (kv_end + kPaKT - 1) / kPaKT - jt0);
  const int* table = block_table + (size_t)b * max_blocks;

  __syncthreads();  // the tiles are zero: stage the query rows
  for (int i = threadIdx.x; i < R * 32; i += kPaThreads) {
    const int r = i >> 5, ch = i & 31;  // 32 chunks of 16 bytes per row
    const int sq = r / RS, g = (r % RS) / T, t = r % T;
    const uint4 v = *(const uint4*)(q + ((size_t)(it.seq[sq] * T + t) * Hq + kvh * group + g) * kPaHd + ch * 8);
    *(uint4*)(smem + kPaQOff + (ch >> 3) * kPaPanel + r * 128 + (((ch & 7) ^ (r & 7)) << 4)) = v;
  }
  fence_proxy_async();
  if (threadIdx.x == 0) {
    mbar_init(&bars->k_full, 1); mbar_init(&bars->k_empty, 1);
    mbar_init(&bars->v_full, 1); mbar_init(&bars->v_empty, 1);
    mbar_init(&bars->s_full[0], 1); mbar_init(&bars->s_full[1], 1);
    mbar_init(&bars->p_full, 8); mbar_init(&bars->o_done, 1);
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(&bars->tmem_base, kPaTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 8 || warp == 10) {
    // ---------------------------------------------------------------------------------------- K (warp 8) / V (warp 10) pages
    // lane l fetches box (page l / 4, 64-column panel l % 4) of the tile: the 32 boxes of a tile are issued at once
    const bool is_k = warp == 8;
    const CUtensorMap* map = is_k ? &map_k : &map_v;
    uint64_t* full = is_k ? &bars->k_full : &bars->v_full;
    uint64_t* empty = is_k ? &bars->k_empty : &bars->v_empty;
    uint8_t* dst = smem + (is_k ? kPaKOff : kPaVOff);
    const int pg = lane >> 2, p = lane & 3;
    if (lane == 0) prefetch_tensormap(map);
    for (int j = 0; j < ntiles; ++j) {
      bool ok = true;
      if (j > 0 && lane == 0) ok = pa_wait(empty, (j - 1) & 1, status);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      const int npages = min(8, (kv_end - (jt0 + j) * kPaKT + 15) >> 4);
      if (lane == 0) mbar_expect_tx(full, (uint32_t)npages * 4u * 2048u);
      __syncwarp();
      if (pg < npages) tma_load_2d(dst + p * kPaPanel + pg * 2048, map, kvh * kPaHd + p * 64, table[(jt0 + j) * 8 + pg] * 16, full);
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------------------------------- MMA issuer
    if (lane == 0 && ntiles > 0) {
      constexpr uint32_t idesc_s = umma_idesc_f16(kPaQT, kPaKT, 1);
      constexpr uint32_t idesc_o = umma_idesc_f16(kPaQT, kPaHd, 1) | (1u << 16);  // B (= V) MN-major
      const uint32_t q_addr = smem_u32(smem + kPaQOff), k_addr = smem_u32(smem + kPaKOff), v_addr = smem_u32(smem + kPaVOff),
                     p_addr = smem_u32(smem + kPaPOff);
      auto issue_s = [&](int j) -> bool {
        if (!pa_wait(&bars->k_full, j & 1, status)) return false;
        tcgen05_fence_after();
#pragma unroll
        for (int kk = 0; kk < kPaHd / 16; ++kk) {
          const uint64_t da = umma_desc_sw128(q_addr + (kk >> 2) * kPaPanel) + (uint64_t)((kk & 3) * 2);
          const uint64_t db = umma_desc_sw128(k_addr + (kk >> 2) * kPaPanel) + (uint64_t)((kk & 3) * 2);
          umma_f16(tmem + kPaTmemS + (j & 1) * kPaKT, da, db, idesc_s, kk != 0 ? 1u : 0u);
        }
        tcgen05_commit(&bars->k_empty);
        tcgen05_commit(&bars->s_full[j & 1]);
        return true;
      };
      bool ok = issue_s(0);
      if (ok && ntiles > 1) ok = issue_s(1);
      for (int j = 0; j < ntiles && ok; ++j) {
        ok = pa_wait(&bars->p_full, j & 1, status) && pa_wait(&bars->v_full, j & 1, status);
        if (!ok) break;
        tcgen05_fence_after();
#pragma unroll
        for (int kk = 0; kk < kPaKT / 16; ++kk) {
          const uint64_t da = umma_desc_sw128(p_addr + (kk >> 2) * kPaPanel) + (uint64_t)((kk & 3) * 2);
          const uint64_t db = pa_desc_mn_sw128(v_addr + kk * 2048, kPaPanel);
          umma_f16(tmem + kPaTmemO, da, db, idesc_o, (j | kk) != 0 ? 1u : 0u);
        }
        tcgen05_commit(&bars->v_empty);
        tcgen05_commit(&bars->o_done);
        if (j + 2 < ntiles) ok = issue_s(j + 2);
      }
    }
  } else {
    // ---------------------------------------------------------------------------------------- softmax + epilogue
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const uint32_t s_base = lane_base + kPaTmemS + half * 64, o_cols = lane_base + kPaTmemO + half * 128;
    const float sl2 = scale * 1.4426950408889634f;
    const int sq = row < R ? row / RS : 0;
    const int bs = it.seq[sq];  // this row's sequence
    const int c = ctx[bs];
    const bool valid = row < R && c >= 0;
    const int g = valid ? (row % RS) / T : 0, t = valid ? row % T : 0;
    const int last_key = valid ? min(kv_end - 1, c + t) : -1;
    float m_ref = -INFINITY, l_run = 0.f;
    uint8_t* p_row = smem + kPaPOff + half * kPaPanel + row * 128;
    float* xch = (float*)(smem + kPaXchOff);
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      ok = pa_warp_wait(&bars->s_full[j & 1], (j >> 1) & 1, lane, status);
      if (!ok) break;
      tcgen05_fence_after();
      const int k0 = (jt0 + j) * kPaKT + half * 64;
      const uint32_t s_cols = s_base + (j & 1) * kPaKT;
      uint32_t ra[32], rb[32];
      tmem_ld_32x32b_x32(s_cols, ra);
      tmem_ld_32x32b_x32(s_cols + 32, rb);
      tcgen05_wait_ld();
      // rows beyond R and keys beyond a row's horizon are masked in every tile (the tail tile always needs it and the
      // idle lanes must stay at zero weight)
      float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (k0 + i <= last_key) m0 = fmaxf(m0, __uint_as_float(ra[i]));
        if (k0 + 32 + i <= last_key) m1 = fmaxf(m1, __uint_as_float(rb[i]));
      }
      float m_tile = fmaxf(m0, m1);
      float* x = xch + (j & 1) * 256;
      x[half * 128 + row] = m_tile;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
      m_tile = fmaxf(m_tile, x[(half ^ 1) * 128 + row]);
      const float m_new = fmaxf(m_ref, m_tile);
      const bool grow = (m_new - m_ref) * sl2 > 8.f;
      const bool any = __any_sync(0xffffffffu, grow);
      const float m_use = any ? m_new : m_ref;
      const float e_ref = m_use == -INFINITY ? 0.f : m_use * sl2;
      uint32_t pk[32];
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const uint32_t(&r)[32] = cc == 0 ? ra : rb;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = pa_ex2(fmaf(__uint_as_float(r[i]), sl2, -e_ref));
          float p1 = pa_ex2(fmaf(__uint_as_float(r[i + 1]), sl2, -e_ref));
          if (k0 + cc * 32 + i > last_key) p0 = 0.f;
          if (k0 + cc * 32 + i + 1 > last_key) p1 = 0.f;
          sum0 += p0;
          sum1 += p1;
          const __nv_bfloat162 pp = __floats2bfloat162_rn(p0, p1);
          pk[cc * 16 + (i >> 1)] = *(const uint32_t*)&pp;
        }
      }
      const float alpha = !any ? 1.f : (m_ref == -INFINITY ? 0.f : pa_ex2(m_ref * sl2 - e_ref));
      l_run = l_run * alpha + (sum0 + sum1);
      if (j > 0) {
        ok = pa_warp_wait(&bars->o_done, (j - 1) & 1, lane, status);
        if (!ok) break;
        tcgen05_fence_after();
        if (any) {
#pragma unroll 1
          for (int cc = 0; cc < 4; ++cc) {
            tmem_ld_32x32b_x32(o_cols + cc * 32, ra);
            tcgen05_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) ra[i] = __float_as_uint(__uint_as_float(ra[i]) * alpha);
            pa_tmem_st_32x32b_x32(o_cols + cc * 32, ra);
          }
          pa_wait_st();
        }
      }
      m_ref = m_use;
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
    if (ntiles > 0 && ok) ok = pa_warp_wait(&bars->o_done, (ntiles - 1) & 1, lane, status);
    float* xl = xch + (ntiles & 1) * 256;
    xl[half * 128 + row] = l_run;
    asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
    l_run += xl[(half ^ 1) * 128 + row];
    if (items) {
      // partial result of this item: un-normalised O (fp32), the reference maximum in log2 units and the row sum.
      // (The TMEM loads are warp-wide instructions: every lane runs them, the stores are per valid row.)
      const bool have = ok && ntiles > 0;  // uniform over the warp
      const int h = kvh * group + g;
      const size_t prow = (size_t)(bs * T + t) * Hq + h;
      if (have) tcgen05_fence_after();
      float* po = part_o + ((size_t)it.slot * rows_total * Hq + prow) * kPaHd + half * 128;
#pragma unroll 1
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t r[32];
        if (have) {
          tmem_ld_32x32b_x32(o_cols + cc * 32, r);
          tcgen05_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) *(uint4*)(po + cc * 32 + i) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
        }
      }
      if (valid && half == 0) {
        float* pm = part_ml + ((size_t)it.slot * rows_total * Hq + prow) * 2;
        pm[0] = (have && l_run > 0.f) ? m_ref * sl2 : -INFINITY;
        pm[1] = have ? l_run : 0.f;
        for (int e = it.clear_from; e < it.clear_to; ++e) {
          float* pe = part_ml + ((size_t)e * rows_total * Hq + prow) * 2;
          pe[0] = -INFINITY; pe[1] = 0.f;
        }
      }
    } else if (!items && ok && ntiles > 0) {
      tcgen05_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const int h = kvh * group + g;
      const size_t grow_ = (size_t)(bs * T + t);
      __nv_bfloat16* dst = out + grow_ * Hq * kPaHd + (size_t)h * kPaHd + half * 128;
      const float* gsrc = gate_src + grow_ * gate_ld + (size_t)h * 2 * kPaHd + kPaHd + half * 128;
#pragma unroll 1
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(o_cols + cc * 32, r);
        tcgen05_wait_ld();
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            float o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(r[i + e]) * inv;
            if (gated) {
              const float4 g0 = *(const float4*)(gsrc + cc * 32 + i), g1 = *(const float4*)(gsrc + cc * 32 + i + 4);
              const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
              for (int e = 0; e < 8; ++e) o[e] *= 1.f / (1.f + __expf(-gg[e]));
            }
            uint4 v;
            __nv_bfloat162 a0 = __floats2bfloat162_rn(o[0], o[1]), a1 = __floats2bfloat162_rn(o[2], o[3]);
            __nv_bfloat162 a2 = __floats2bfloat162_rn(o[4], o[5]), a3 = __floats2bfloat162_rn(o[6], o[7]);
            v.x = *(uint32_t*)&a0; v.y = *(uint32_t*)&a1; v.z = *(uint32_t*)&a2; v.w = *(uint32_t*)&a3;
            *(uint4*)(dst + cc * 32 + i) = v;
          }
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 9) {
    tcgen05_fence_after();
    tmem_dealloc(tmem, kPaTmemCols);
  }
}

// Merge a row's partial results: out = (sum_p 2^(m_p - m) O_p) / (sum_p 2^(m_p - m) l_p) * sigmoid(gate), bf16.
// Grid (rows, Hq), 64 threads x 4 columns. Rows of empty batch slots (ctx < 0) are written as zeros.
__global__ void __launch_bounds__(64) paged_attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int nparts,
                                                                int rows_total, int T, int Hq, const int* __restrict__ ctx,
                                                                const float* __restrict__ gate_src, int gate_ld, int gated,
                                                                __nv_bfloat16* __restrict__ out) {
  grid_dependency_trigger();
  grid_dependency_wait();
  const int row = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const size_t prow = (size_t)row * Hq + h;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float l = 0.f;
  if (ctx[row / T] >= 0) {
    float m = -INFINITY;
    for (int p = 0; p < nparts; ++p) m = fmaxf(m, part_ml[((size_t)p * rows_total * Hq + prow) * 2]);
    for (int p = 0; p < nparts; ++p) {
      const float mp = part_ml[((size_t)p * rows_total * Hq + prow) * 2], lp = part_ml[((size_t)p * rows_total * Hq + prow) * 2 + 1];
      if (!(lp > 0.f) || mp == -INFINITY) continue;
      const float w = pa_ex2(mp - m);
      const float4 o = *(const float4*)(part_o + ((size_t)p * rows_total * Hq + prow) * kPaHd + tid * 4);
      acc.x += w * o.x; acc.y += w * o.y; acc.z += w * o.z; acc.w += w * o.w;
      l += w * lp;
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  float o[4] = {acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv};
  if (gated) {
    const float4 g = *(const float4*)(gate_src + (size_t)row * gate_ld + (size_t)h * 2 * kPaHd + kPaHd + tid * 4);
    o[0] *= 1.f / (1.f + __expf(-g.x)); o[1] *= 1.f / (1.f + __expf(-g.y));
    o[2] *= 1.f / (1.f + __expf(-g.z)); o[3] *= 1.f / (1.f + __expf(-g.w));
  }
  __nv_bfloat162 a0 = __floats2bfloat162_rn(o[0], o[1]), a1 = __floats2bfloat162_rn(o[2], o[3]);
  uint2 v;
  v.x = *(uint32_t*)&a0; v.y = *(uint32_t*)&a1;
  *(uint2*)(out + (size_t)row * Hq * kPaHd + (size_t)h * kPaHd + tid * 4) = v;
}

static PFN_cuTensorMapEncodeTiled_v12000 pa_get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    cudaDriverEntryPointQueryResult q;
    void* p = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
  }
  return fn;
}

// the paged cache seen as a matrix [pages * 16 token rows, Hkv * 256 columns]; boxes of one page x 64 columns
static int pa_make_map(CUtensorMap* map, const void* base, long long rows, int cols) {
  auto enc = pa_get_encode();
  if (!enc) return (int)cudaErrorNotSupported;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64u, 16u};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

}  // namespace pear

// q bf16 [B * T, Hq, 256] (normed, rotated); kc / vc bf16 [num_pages, 16, Hkv, 256] with this step's rows already written;
// block_table int32 [B, max_blocks]; ctx int32 [B] = tokens cached before the step (< 0: empty slot); gate_src fp32 rows of
// the q projection output ([Hq x (q | gate)] per row, leading dimension gate_ld) when `gated`. out bf16 [B * T, Hq * 256].
// Needs group * T <= 128. `status` is a device int that a bounded wait sets on expiry.
// With an item table (`items` = device array of `n_items` 24-int records {sequences, key begin, key end or -1, partial slot,
// first slot to clear, end of the slots to clear, 0, 0, sequence indices x 16}; every active row must be covered by items whose key ranges partition its context):
// the items write partial results into part_o [nparts, B * T, Hq, 256] / part_ml [nparts, B * T, Hq, 2] (fp32) and a second
// kernel merges them. A group item needs sequences * (Hq / Hkv) * T <= 128 rows. `items` null: one CTA per sequence.
PEAR_API int pear_paged_attn_tc_hd256(const void* q, const void* kc, const void* vc, long long num_pages, const int* block_table, int max_blocks,
                                      const int* ctx, int B, int T, int Hq, int Hkv, float scale, const float* gate_src, int gate_ld, int gated,
                                      void* out, int* status, const int* items, int n_items, int nparts, float* part_o, float* part_ml,
                                      void* stream) {
  using namespace pear;
  if (B <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv || (Hq / Hkv) * T > 128 || T < 1) return (int)cudaErrorInvalidValue;
  if (items && (n_items <= 0 || nparts <= 0 || !part_o || !part_ml)) return (int)cudaErrorInvalidValue;
  if (((uintptr_t)q % 16) || ((uintptr_t)kc % 16) || ((uintptr_t)vc % 16) || ((uintptr_t)out % 16) || (gated && (gate_ld % 4))) return (int)cudaErrorInvalidValue;
  CUtensorMap mk, mv;
  int r = pa_make_map(&mk, kc, num_pages * 16, Hkv * kPaHd);
  if (r) return r;
  r = pa_make_map(&mv, vc, num_pages * 16, Hkv * kPaHd);
  if (r) return r;
  constexpr int smem = (int)kPaXchOff + 2048 + (int)kPaAlignSlack;
  static bool configured = false;
  if (!configured) {
    PEAR_CUDA_CHECK(cudaFuncSetAttribute(paged_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  PEAR_CUDA_CHECK(launch_dependent(paged_attn_tc_kernel, dim3(items ? n_items : B, Hkv), dim3(kPaThreads), smem, (cudaStream_t)stream, mk, mv,
                                   (const __nv_bfloat16*)q, block_table, max_blocks, ctx, T, Hq, Hkv, scale, (const float*)gate_src, gate_ld, gated,
                                   (__nv_bfloat16*)out, status, (const PaItem*)items, part_o, part_ml, B * T));
  if (items) {
    PEAR_CUDA_CHECK(launch_ordinary(paged_attn_combine_kernel, dim3(B * T, Hq), dim3(64), 0, (cudaStream_t)stream, part_o, part_ml, nparts, B * T, T, Hq,
                                     ctx, (const float*)gate_src, gate_ld, gated, (__nv_bfloat16*)out));
  }
  return 0;
}
