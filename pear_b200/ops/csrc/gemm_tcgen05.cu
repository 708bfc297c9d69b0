// bf16 GEMM for sm_100a on the 5th-generation tensor cores: C[M,N] = A[M,K] * B[N,K]^T, fp32 accumulation in tensor
// memory. Persistent, warp-specialised: warp 0 feeds a 4-stage shared-memory ring with 2-D TMA loads (128-byte swizzle),
// warp 1 issues tcgen05.mma (128 x BN x 16 per instruction) into one of two TMEM accumulators, warps 2-5 drain the
// other accumulator with tcgen05.ld and write C, so the epilogue of tile i overlaps the main loop of tile i+1.
// (The building block of the fused paths; upstream calls cuBLAS/cuBLASLt here: pear/models/qwen3_5/trainer/operands.py:204,
// rollout/blackwell/csrc/gemm_lt.cpp.) No cluster multicast anywhere: operands come through plain per-CTA TMA loads.
// Operand forms: each operand is either K-major (a row-major [rows, K] matrix: the forward's X and W) or MN-major (a
// row-major [K, rows] matrix, the reduction running over its ROWS: what the backward products dX = dY W and dW = dY^T X
// read). A K-major tile is [rows][64 k] (128-byte rows); an MN-major tile is one panel of [64 k][64 rows] per 64 output
// rows (the same 128-byte-swizzled TMA box, the tensor core told through its descriptors to read it transposed).
#include "common.cuh"

#include <cudaTypedefs.h>

namespace pear {

constexpr int kBM = 128, kBK = 64, kStages = 4;
constexpr int kGemmThreads = 192;

struct GemmSmem {
  uint64_t full[kStages], empty[kStages];
  uint64_t tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
};

// MN-major operand tile with the 128-byte swizzle: rows of 128 bytes along MN (64 bf16), 8 K rows per 1024-byte atom;
// `lbo` = bytes between 64-element MN groups, 8-row K groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t gemm_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

template <int BN, bool OUT_BF16, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, void* __restrict__ c,
                 int M, int N, int K, int ldc, int* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr uint32_t kABytes = kBM * kBK * 2, kBBytes = BN * kBK * 2, kStageBytes = kABytes + kBBytes;
  uint8_t* tiles = smem;  // [stage][A | B], 1024-byte aligned
  GemmSmem* sm = (GemmSmem*)(smem + kStages * kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + kBM - 1) / kBM, tiles_n = (N + BN - 1) / BN, ntiles = tiles_m * tiles_n;
  const int kblocks = (K + kBK - 1) / kBK;
  // Tile order: bands of kBand row tiles; inside a band the row tile varies fastest, so the ~148 tiles in flight at any time cover about kBand x (148 / kBand) tiles: kBand A panels and ~9 B panels
  // (~70 MB at K = 8192) stay in the 126 MB L2 instead of 148 different A panels streaming from HBM for every wave.
  constexpr int kBand = 16;
  auto tile_origin = [&](int t, int& m0, int& n0) {
    const int band = t / (kBand * tiles_n), in_band = t % (kBand * tiles_n);
    const int rows_here = min(kBand, tiles_m - band * kBand);
    m0 = (band * kBand + in_band % rows_here) * kBM;
    n0 = (in_band / rows_here) * BN;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) { mbar_init(&sm->full[i], 1); mbar_init(&sm->empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sm->tmem_full[i], 1); mbar_init(&sm->tmem_empty[i], 4); }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&sm->tmem_base, 2 * BN);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = sm->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      int st = 0, ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
        int m0, n0;
        tile_origin(tile, m0, n0);
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = mbar_wait_bounded(&sm->empty[st], ph ^ 1, status);
          if (!ok) break;
          uint8_t* a = tiles + st * kStageBytes;
          mbar_expect_tx(&sm->full[st], kStageBytes);
          if (A_MN) {
#pragma unroll
            for (int p = 0; p < kBM / 64; ++p) tma_load_2d(a + p * 8192, &map_a, m0 + p * 64, kb * kBK, &sm->full[st]);
          } else {
            tma_load_2d(a, &map_a, kb * kBK, m0, &sm->full[st]);
          }
          if (B_MN) {
#pragma unroll
            for (int p = 0; p < BN / 64; ++p) tma_load_2d(a + kABytes + p * 8192, &map_b, n0 + p * 64, kb * kBK, &sm->full[st]);
          } else {
            tma_load_2d(a + kABytes, &map_b, kb * kBK, n0, &sm->full[st]);
          }
          if (++st == kStages) { st = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(kBM, BN, 1) | (A_MN ? (1u << 15) : 0u) | (B_MN ? (1u << 16) : 0u);
      int st = 0, ph = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++it) {
        const int ab = it & 1;
        ok = mbar_wait_bounded(&sm->tmem_empty[ab], ((it >> 1) & 1) ^ 1, status);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + ab * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = mbar_wait_bounded(&sm->full[st], ph, status);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(tiles + st * kStageBytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // a K step of 16: 32 bytes along a K-major row, 16 rows (2048 bytes) down an MN-major panel
            const uint64_t da = A_MN ? gemm_desc_mn_sw128(a_addr + k * 2048, 8192) : umma_desc_sw128(a_addr) + (uint64_t)(k * 2);
            const uint64_t db = B_MN ? gemm_desc_mn_sw128(a_addr + kABytes + k * 2048, 8192) : umma_desc_sw128(a_addr + kABytes) + (uint64_t)(k * 2);
            umma_f16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tcgen05_commit(&sm->empty[st]);  // the stage is free once these MMAs have read it
          if (++st == kStages) { st = 0; ph ^= 1; }
        }
        tcgen05_commit(&sm->tmem_full[ab]);
      }
    }
  } else {
    // ------------------------------------------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
      const int ab = it & 1;
      int m0, n0;
      tile_origin(tile, m0, n0);
      if (ok) ok = mbar_wait_bounded(&sm->tmem_full[ab], (it >> 1) & 1, status);
      if (!ok) break;
      tcgen05_fence_after();
      const int row = m0 + q * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + ab * BN + c0, r);
        tcgen05_wait_ld();
        if (row < M) {
          const int col = n0 + c0;
          if (OUT_BF16) {
            __nv_bfloat16* dst = (__nv_bfloat16*)c + (size_t)row * ldc + col;
            if (col + 32 <= N && (ldc % 8) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 v;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                v.x = *(uint32_t*)&p0; v.y = *(uint32_t*)&p1; v.z = *(uint32_t*)&p2; v.w = *(uint32_t*)&p3;
                *(uint4*)(dst + j) = v;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col + j < N) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
            }
          } else {
            float* dst = (float*)c + (size_t)row * ldc + col;
            if (col + 32 <= N && (ldc % 4) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *(float4*)(dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                                  __uint_as_float(r[j + 3]));
            } else {
              for (int j = 0; j < 32; ++j)
                if (col + j < N) dst[j] = __uint_as_float(r[j]);
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm->tmem_empty[ab]);
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ------------------------------------------------------------------------------------------------ host side
static PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
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

// Row-major [rows, cols] bf16 matrix with leading dimension ld (elements); box = [box_rows, 64 cols], 128-byte swizzle.
static int make_map_bf16(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  auto enc = get_encode();
  if (!enc) return (int)cudaErrorNotSupported;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

// The same matrix read MN-major: a row-major [k_rows, mn_cols] matrix, box = [64 k rows, 64 mn columns].
static int make_map_bf16_mn(CUtensorMap* map, const void* base, int k_rows, int mn_cols, int ld) {
  auto enc = get_encode();
  if (!enc) return (int)cudaErrorNotSupported;
  cuuint64_t dims[2] = {(cuuint64_t)mn_cols, (cuuint64_t)k_rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)kBK};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

template <int BN, bool OUT_BF16, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, void* c, int M, int N, int K, int ldc, int* status,
                       int num_sms, cudaStream_t stream) {
  constexpr int smem = kStages * (kBM * kBK * 2 + BN * kBK * 2) + 1024;
  static bool configured = false;
  if (!configured) {
    PEAR_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_kernel<BN, OUT_BF16, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  const int ntiles = ((M + kBM - 1) / kBM) * ((N + BN - 1) / BN);
  const int grid = ntiles < num_sms ? ntiles : num_sms;
  gemm_bf16_kernel<BN, OUT_BF16, A_MN, B_MN><<<grid, kGemmThreads, smem, stream>>>(ma, mb, c, M, N, K, ldc, status);
  PEAR_LAUNCH_CHECK();
  return 0;
}

}  // namespace pear

// C[M,N] (fp32 or bf16, leading dimension ldc) = A[M,K] (bf16, lda) * B[N,K]^T (bf16, ldb).
// Requirements: A, B 16-byte aligned, lda and ldb multiples of 8. `status` is a device int (0 = ok) that a bounded wait
// sets on expiry.
PEAR_API int pear_gemm_bf16_nt(const void* a, const void* b, void* c, int M, int N, int K, int lda, int ldb, int ldc,
                               int out_bf16, int* status, int num_sms, void* stream) {
  using namespace pear;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)a % 16) || ((uintptr_t)b % 16)) return (int)cudaErrorInvalidValue;
  const bool wide = N > 128;
  CUtensorMap ma, mb;
  int r = make_map_bf16(&ma, a, M, K, lda, kBM);
  if (r) return r;
  r = make_map_bf16(&mb, b, N, K, ldb, wide ? 256 : 128);
  if (r) return r;
  cudaStream_t s = (cudaStream_t)stream;
  if (wide) return out_bf16 ? launch_gemm<256, true, false, false>(ma, mb, c, M, N, K, ldc, status, num_sms, s)
                            : launch_gemm<256, false, false, false>(ma, mb, c, M, N, K, ldc, status, num_sms, s);
  return out_bf16 ? launch_gemm<128, true, false, false>(ma, mb, c, M, N, K, ldc, status, num_sms, s)
                  : launch_gemm<128, false, false, false>(ma, mb, c, M, N, K, ldc, status, num_sms, s);
}

// The backward products of a linear layer Y = X W^T on the same kernel (upstream leaves them to cuBLAS):
//   a_mn = 0, b_mn = 1:  C[M,N] = A[M,K] * B[K,N]      (dX = dY W: a = dY [M, K], b = W stored row-major [K, N])
//   a_mn = 1, b_mn = 1:  C[M,N] = A[K,M]^T * B[K,N]    (dW = dY^T X: a = dY stored [K, M], b = X stored [K, N])
// lda / ldb are the row strides of the matrices as stored. Same alignment rules as pear_gemm_bf16_nt.
PEAR_API int pear_gemm_bf16_form(const void* a, const void* b, void* c, int M, int N, int K, int lda, int ldb, int ldc, int a_mn, int b_mn,
                                 int out_bf16, int* status, int num_sms, void* stream) {
  using namespace pear;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)a % 16) || ((uintptr_t)b % 16) || !b_mn) return (int)cudaErrorInvalidValue;
  const bool wide = N > 128;
  CUtensorMap ma, mb;
  int r = a_mn ? make_map_bf16_mn(&ma, a, K, M, lda) : make_map_bf16(&ma, a, M, K, lda, kBM);
  if (r) return r;
  r = make_map_bf16_mn(&mb, b, K, N, ldb);
  if (r) return r;
  cudaStream_t s = (cudaStream_t)stream;
#define PEAR_FORM(BN_, OUT_)                                                                                              \
  (a_mn ? launch_gemm<BN_, OUT_, true, true>(ma, mb, c, M, N, K, ldc, status, num_sms, s)                                 \
        : launch_gemm<BN_, OUT_, false, true>(ma, mb, c, M, N, K, ldc, status, num_sms, s))
  if (wide) return out_bf16 ? PEAR_FORM(256, true) : PEAR_FORM(256, false);
  return out_bf16 ? PEAR_FORM(128, true) : PEAR_FORM(128, false);
#undef PEAR_FORM
}
