// Weight-streaming bf16 GEMM for the rollout step (decode / verify rows): Y[m, n] = sum_k X[m, k] * W[n, k] where the
// step has few token rows (M up to a few hundred) and the weight matrix is what has to come from HBM. The roles of the
// operands are swapped relative to the training GEMM: the WEIGHTS are the tensor core's A operand (128 output features
// per CTA = the 128 TMEM lanes), the TOKENS are the B operand (N = a block of BT tokens), so every CTA streams its own
// 16 KB weight panels through a deep TMA ring and the accumulator is Y^T in tensor memory. Work items are
// (128-row weight tile, K split, token block); K is split when there are fewer weight tiles than SMs so that all 148 SMs
// stream (the partial sums go to separate fp32 planes that the consumer adds: no atomics, fixed summation order).
// (Upstream: rollout/blackwell/csrc/stream_gemm.cu:105-316 — weights as A, tokens as N, split-K partials.)
// Warp roles as in the training GEMM: warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 epilogue over the four TMEM
// lane quarters; two accumulators so that the epilogue of one item overlaps the main loop of the next.
// The epilogue writes Y un-transposed: a thread holds one output feature and 32 tokens; a warp stages its 32 features x 32
// tokens in shared memory and sends the box with one TMA store (scalar global stores, 128 per thread, took 4.7 us per
// 128 x 128 tile, the largest fixed cost of a 20-40 us launch). No cluster multicast; every wait is bounded.
#include "common.cuh"

#include <cudaTypedefs.h>

namespace pear {

constexpr int kSgBM = 128, kSgBK = 64;
constexpr int kSgThreads = 192;

// Ring depth: as many [weights | tokens] stages as 224 KB hold. The weight bytes a CTA keeps in flight set its share of the
// HBM bandwidth (the loaded latency is microseconds). A separate, shallow ring for the token panels (they come from L2) was
// measured and is slower: 46 us against 36 us on 16480 x 5120 at 128 tokens, because the token loads queue behind the
// weight loads in the same TMA unit and see the same latency.
template <int BT, int EPI>
struct SgCfg {
  static constexpr int kDual = EPI == 2 ? 2 : 1;
  static constexpr int kStageBytes = kDual * kSgBM * kSgBK * 2 + BT * kSgBK * 2;
  // the epilogue's staging: per epilogue warp two boxes of 32 tokens x 32 features (fp32 or bf16) that TMA stores read
  static constexpr int kBoxBytes = 32 * 32 * (EPI == 0 ? 4 : 2);
  static constexpr int kStagingBytes = 4 * 2 * kBoxBytes;
  static constexpr int kStagesRaw = (224 * 1024 - kStagingBytes) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 12 ? 12 : kStagesRaw;
  static constexpr int kSmem = kStages * kStageBytes + kStagingBytes + 1024;
};

struct SgSmem {
  uint64_t full[12], empty[12];
  uint64_t tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
};

// EPI 0: fp32 planes out[split][m][n]; EPI 1: bf16 out[m][n] (one split); EPI 2: SwiGLU — the item multiplies TWO weight
// tiles (gate rows n0.. and up rows up_row0 + n0..) into two accumulators and writes silu(gate) * up as bf16.
// Launched as a programmatic dependent: see the producer.
template <int BT, int EPI>
__global__ void __launch_bounds__(kSgThreads, 1)
stream_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_o,
                   int M, int N, int K, int nsplit, int up_row0, int* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr int kDual = EPI == 2 ? 2 : 1;
  constexpr uint32_t kABytes = kSgBM * kSgBK * 2, kXBytes = BT * kSgBK * 2;
  constexpr uint32_t kStageBytes = kDual * kABytes + kXBytes;
  constexpr int kStages = SgCfg<BT, EPI>::kStages;
  constexpr int kAccBufs = (kDual * 2 * BT <= 512) ? 2 : 1;
  constexpr uint32_t kTmemCols = kDual * kAccBufs * BT < 32 ? 32 : kDual * kAccBufs * BT;
  uint8_t* tiles = smem;
  uint8_t* staging = smem + kStages * kStageBytes;
  SgSmem* sm = (SgSmem*)(staging + SgCfg<BT, EPI>::kStagingBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (N + kSgBM - 1) / kSgBM, tblocks = (M + BT - 1) / BT;
  const int nitems = tiles_n * nsplit * tblocks;
  const int kblocks = (K + kSgBK - 1) / kSgBK;
  auto item = [&](int it, int& n0, int& m0, int& s, int& kb0, int& kb1) {
    const int tb = it % tblocks, rest = it / tblocks;
    s = rest % nsplit;
    n0 = (rest / nsplit) * kSgBM;
    m0 = tb * BT;
    kb0 = (int)((long long)kblocks * s / nsplit);
    kb1 = (int)((long long)kblocks * (s + 1) / nsplit);
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) { mbar_init(&sm->full[i], 1); mbar_init(&sm->empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sm->tmem_full[i], 1); mbar_init(&sm->tmem_empty[i], 4); }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&sm->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = sm->tmem_base;

  grid_dependency_trigger();  // the next kernel's blocks may take the SMs this grid's blocks leave
  if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&map_w);
      prefetch_tensormap(&map_x);
      // The weight halves of the first ring round go out BEFORE the wait for the kernels ahead in the stream (weights are
      // constants of the step): they stream in while the previous kernel drains. The token halves, which that kernel may
      // still be writing, follow the wait.
      int pre = 0;
      for (int it = blockIdx.x; it < nitems && pre < kStages; it += gridDim.x) {
        int n0, m0, s, kb0, kb1;
        item(it, n0, m0, s, kb0, kb1);
        for (int kb = kb0; kb < kb1 && pre < kStages; ++kb, ++pre) {
          uint8_t* a = tiles + pre * kStageBytes;
          mbar_expect_tx(&sm->full[pre], kStageBytes);
          tma_load_2d(a, &map_w, kb * kSgBK, n0, &sm->full[pre]);
          if (kDual == 2) tma_load_2d(a + kABytes, &map_w, kb * kSgBK, up_row0 + n0, &sm->full[pre]);
        }
      }
      grid_dependency_wait();
      int st = 0, ph = 0, cnt = 0;
      bool ok = true;
      for (int it = blockIdx.x; it < nitems && ok; it += gridDim.x) {
        int n0, m0, s, kb0, kb1;
        item(it, n0, m0, s, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb, ++cnt) {
          uint8_t* a = tiles + st * kStageBytes;
          if (cnt >= pre) {
            ok = mbar_wait_bounded(&sm->empty[st], ph ^ 1, status);
            if (!ok) break;
            mbar_expect_tx(&sm->full[st], kStageBytes);
            tma_load_2d(a, &map_w, kb * kSgBK, n0, &sm->full[st]);
            if (kDual == 2) tma_load_2d(a + kABytes, &map_w, kb * kSgBK, up_row0 + n0, &sm->full[st]);
          }
          tma_load_2d(a + kDual * kABytes, &map_x, kb * kSgBK, m0, &sm->full[st]);
          if (++st == kStages) { st = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(kSgBM, BT, 1);
      int st = 0, ph = 0, n_it = 0;
      bool ok = true;
      grid_dependency_wait();  // the bounded waits below count from the completion of the kernel ahead, however long it runs
      for (int it = blockIdx.x; it < nitems && ok; it += gridDim.x, ++n_it) {
        int n0, m0, s, kb0, kb1;
        item(it, n0, m0, s, kb0, kb1);
        const int ab = kAccBufs == 2 ? (n_it & 1) : 0;
        const uint32_t par = kAccBufs == 2 ? ((n_it >> 1) & 1) : (n_it & 1);
        ok = mbar_wait_bounded(&sm->tmem_empty[ab], par ^ 1, status);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + ab * kDual * BT;
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait_bounded(&sm->full[st], ph, status);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(tiles + st * kStageBytes);
          const uint64_t da = umma_desc_sw128(a_addr), dx = umma_desc_sw128(a_addr + kDual * kABytes);
#pragma unroll
          for (int k = 0; k < kSgBK / 16; ++k)
            umma_f16(d_tmem, da + (uint64_t)(k * 2), dx + (uint64_t)(k * 2), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          if (kDual == 2) {
            const uint64_t du = umma_desc_sw128(a_addr + kABytes);
#pragma unroll
            for (int k = 0; k < kSgBK / 16; ++k)
              umma_f16(d_tmem + BT, du + (uint64_t)(k * 2), dx + (uint64_t)(k * 2), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tcgen05_commit(&sm->empty[st]);
          if (++st == kStages) { st = 0; ph ^= 1; }
        }
        tcgen05_commit(&sm->tmem_full[ab]);
      }
    }
  } else {
    const int q = warp & 3;
    int n_it = 0, box = 0;
    bool ok = true;
    constexpr int kBoxBytes = SgCfg<BT, EPI>::kBoxBytes;
    uint8_t* my_boxes = staging + (warp - 2) * 2 * kBoxBytes;
    prefetch_tensormap(&map_o);
    grid_dependency_wait();  // `out` may still be read by a kernel ahead in the stream
    for (int it = blockIdx.x; it < nitems; it += gridDim.x, ++n_it) {
      int n0, m0, s, kb0, kb1;
      item(it, n0, m0, s, kb0, kb1);
      const int ab = kAccBufs == 2 ? (n_it & 1) : 0;
      const uint32_t par = kAccBufs == 2 ? ((n_it >> 1) & 1) : (n_it & 1);
      if (ok) ok = mbar_wait_bounded(&sm->tmem_full[ab], par, status);
      ok = __all_sync(0xffffffffu, ok);  // the warp leaves together: the arrive below is per warp
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t acc = tmem_base + ((uint32_t)(q * 32) << 16) + ab * kDual * BT;
#pragma unroll 1
      for (int c0 = 0; c0 < BT; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(acc + c0, r);
        if (EPI == 2) {
          uint32_t u[32];
          tmem_ld_32x32b_x32(acc + BT + c0, u);
          tcgen05_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float g = __uint_as_float(r[j]);
            r[j] = __float_as_uint(g / (1.f + __expf(-g)) * __uint_as_float(u[j]));
          }
        } else {
          tcgen05_wait_ld();
        }
        if (n0 + q * 32 < N && m0 + c0 < M && kb1 > kb0) {  // the same in the whole warp; the store clips the box at N and M
          uint8_t* dst = my_boxes + (box & 1) * kBoxBytes;
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");  // the store before the last one has read its box
          __syncwarp();
          if (EPI == 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) *(uint32_t*)(dst + j * 128 + lane * 4) = r[j];
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) *(__nv_bfloat16*)(dst + j * 64 + lane * 2) = __float2bfloat16_rn(__uint_as_float(r[j]));
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(&map_o), "r"(n0 + q * 32),
                         "r"(m0 + c0), "r"(s), "r"(smem_u32(dst))
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          ++box;
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm->tmem_empty[ab]);
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // every store of this warp has been performed
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

static PFN_cuTensorMapEncodeTiled_v12000 sg_get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    cudaDriverEntryPointQueryResult q;
    void* p = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
  }
  return fn;
}

static int sg_make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  auto enc = sg_get_encode();
  if (!enc) return (int)cudaErrorNotSupported;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)kSgBK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

// The output as [nsplit planes][M rows][N features] (fp32 planes or one bf16 matrix): boxes of 32 features x 32 rows.
static int sg_make_out_map(CUtensorMap* map, void* base, int M, int N, int ldo, long long split_stride, int nsplit, bool fp32) {
  auto enc = sg_get_encode();
  if (!enc) return (int)cudaErrorNotSupported;
  const cuuint64_t es = fp32 ? 4 : 2;
  cuuint64_t dims[3] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)nsplit};
  cuuint64_t strides[2] = {(cuuint64_t)ldo * es, (cuuint64_t)(nsplit > 1 ? split_stride : (long long)M * ldo) * es};
  cuuint32_t box[3] = {32u, 32u, 1u};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

template <int BT, int EPI>
static int sg_launch(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mo, int M, int N, int K, int nsplit,
                     int up_row0, int* status, int num_sms, cudaStream_t stream) {
  constexpr int smem = SgCfg<BT, EPI>::kSmem;
  static bool configured = false;
  if (!configured) {
    PEAR_CUDA_CHECK(cudaFuncSetAttribute(stream_gemm_kernel<BT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  const int nitems = ((N + kSgBM - 1) / kSgBM) * nsplit * ((M + BT - 1) / BT);
  const int grid = nitems < num_sms ? nitems : num_sms;
  PEAR_CUDA_CHECK(launch_dependent(stream_gemm_kernel<BT, EPI>, dim3(grid), dim3(kSgThreads), smem, stream, mw, mx, mo, M, N, K, nsplit, up_row0,
                                   status));
  return 0;
}

template <int EPI>
static int sg_dispatch(int bt, const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mo, int M, int N, int K, int nsplit, int up_row0,
                       int* status, int num_sms, cudaStream_t s) {
  switch (bt) {
    case 32: return sg_launch<32, EPI>(mw, mx, mo, M, N, K, nsplit, up_row0, status, num_sms, s);
    case 64: return sg_launch<64, EPI>(mw, mx, mo, M, N, K, nsplit, up_row0, status, num_sms, s);
    case 128: return sg_launch<128, EPI>(mw, mx, mo, M, N, K, nsplit, up_row0, status, num_sms, s);
    default: return sg_launch<256, EPI>(mw, mx, mo, M, N, K, nsplit, up_row0, status, num_sms, s);
  }
}

}  // namespace pear

// Y = X W^T for a step of M token rows. x [M, K] bf16 (ldx), w [N, K] bf16 (ldw); both 16-byte aligned, ldx / ldw multiples of 8;
// out 16-byte aligned, ldo a multiple of 4 (fp32) or 8 (bf16).
//   epi 0: out fp32, `nsplit` planes of [M, ldo] that are `split_stride` elements apart (the consumer adds the planes);
//   epi 1: out bf16 [M, ldo] (nsplit must be 1);
//   epi 2: w holds [gate rows | up rows] with the up rows starting at row `up_row0`; N = number of gate rows; out bf16
//          [M, ldo] = silu(x gate^T) * (x up^T) (nsplit must be 1).
// Planes whose K range is empty are not written (cannot happen while nsplit <= ceil(K / 64)).
PEAR_API int pear_stream_gemm_bf16(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldw, int ldo, long long split_stride,
                                   int nsplit, int epi, int up_row0, int* status, int num_sms, void* stream) {
  using namespace pear;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((ldx % 8) || (ldw % 8) || ((uintptr_t)x % 16) || ((uintptr_t)w % 16) || nsplit < 1 || epi < 0 || epi > 2) return (int)cudaErrorInvalidValue;
  // the output goes out by TMA stores: 16-byte aligned base, row and plane strides multiples of 16 bytes
  if (((uintptr_t)out % 16) || (ldo % (epi == 0 ? 4 : 8)) || (nsplit > 1 && (split_stride % 4))) return (int)cudaErrorInvalidValue;
  if (epi != 0 && nsplit != 1) return (int)cudaErrorInvalidValue;
  if (nsplit > (K + kSgBK - 1) / kSgBK) return (int)cudaErrorInvalidValue;
  // token block: the whole step when it is small; for larger steps the block size that fills the SMs best (work items =
  // weight tiles x token blocks x K splits, executed in rounds of num_sms), the larger block on a near tie
  int bt = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  if (M > 128) {
    const int tiles_n = (N + kSgBM - 1) / kSgBM;
    double best = -1.0;
    for (int cand = 256; cand >= 64; cand >>= 1) {
      const long long items = (long long)tiles_n * ((M + cand - 1) / cand) * nsplit;
      const long long rounds = (items + num_sms - 1) / num_sms;
      const double eff = (double)items / (double)(rounds * num_sms) * (cand == 64 ? 0.9 : 1.0);  // 64-token blocks reuse a weight tile less
      if (eff > best + 0.05) { best = eff; bt = cand; }
    }
  }
  CUtensorMap mw, mx;
  const int w_rows = epi == 2 ? up_row0 + N : N;
  int r = sg_make_map(&mw, w, w_rows, K, ldw, kSgBM);
  if (r) return r;
  r = sg_make_map(&mx, x, M, K, ldx, bt);
  if (r) return r;
  CUtensorMap mo;
  r = sg_make_out_map(&mo, out, M, N, ldo, split_stride, nsplit, epi == 0);
  if (r) return r;
  cudaStream_t s = (cudaStream_t)stream;
  if (epi == 0) return sg_dispatch<0>(bt, mw, mx, mo, M, N, K, nsplit, up_row0, status, num_sms, s);
  if (epi == 1) return sg_dispatch<1>(bt, mw, mx, mo, M, N, K, nsplit, up_row0, status, num_sms, s);
  return sg_dispatch<2>(bt, mw, mx, mo, M, N, K, nsplit, up_row0, status, num_sms, s);
}
