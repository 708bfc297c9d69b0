// bf16 GEMMs on tcgen05 fused with the collective that precedes or follows them, over peer memory (NVLink / NVSwitch):
//
//   all-gather -> GEMM   C[M, N] = gather_r(A_r)[M, K] * B[N, K]^T,  A row-sharded: rank r holds rows [r M/W, (r+1) M/W)
//       There is no separate gather launch: two copier warps per CTA pull the remote shards over NVLink, 128-row block by
//       block in the order the tiles will need them, into a local full-A buffer and publish each block with a release
//       flag; the TMA producer computes the tiles of the local shard first and takes a remote block as soon as its flag
//       is up (bounded waits on both sides). Every remote byte crosses NVLink exactly once: reading remote tiles straight
//       from peer memory re-fetched each A block once per N tile (measured 3.7 ms against 0.8 ms for NCCL + cuBLAS at
//       M = N = K = 8192 on two GPUs).
//
//   GEMM -> reduce-scatter   C_r[M/W, N] = sum_s A_s[M, K_s] * B_s[N, K_s]^T restricted to the rows rank r owns
//       There is no reduce pass: tiles are visited owner by owner starting after the own rank (at any moment the ranks
//       write to different owners) and the own tiles come last. The epilogue of a tile owned by a peer PUSHES the fp32
//       partial into that peer's staging slot for this source with plain 16-byte stores over NVLink and raises a per-tile
//       flag; the epilogue of an own tile waits (bounded) for the flags of the other sources, adds their staged partials
//       (local reads) to its accumulator and writes the final rows. No atomics, no zeroing; a first version that used
//       `red.add` packets over NVLink ran at 0.90 ms against 0.51 ms for cuBLAS + NCCL at 8192^3 on two GPUs.
//
// Upstream runs these as separate steps (FSDP2 NCCL all-gather then cuBLAS, `operands.py:204`; split-K partials then
// `ar_norm.cu` at TP2). The main loop is the one of gemm_tcgen05.cu: 4-stage TMA ring, one MMA-issuing thread, two TMEM
// accumulators, four epilogue warps. No cluster multicast anywhere.
#include "common.cuh"

#include <cudaTypedefs.h>

namespace pear {

constexpr int kCBM = 128, kCBK = 64, kCStages = 4, kCThreads = 256, kCMaxRanks = 8;  // warps: TMA, MMA, 4 epilogue, 2 copier

struct CollSmem {
  uint64_t full[kCStages], empty[kCStages];
  uint64_t tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
};

struct MapSet {
  CUtensorMap a[kCMaxRanks];
};
struct OutPtrs {
  float* p[kCMaxRanks];
};
struct FlagPtrs {
  uint32_t* p[kCMaxRanks];
};

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool wait_epoch(const uint32_t* flag, uint32_t epoch, uint32_t budget) {
  for (uint32_t i = 0; i < budget; ++i) {
    if ((int32_t)(ld_acquire_sys_u32(flag) - epoch) >= 0) return true;
    if (i > 32) __nanosleep(100);
  }
  return false;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool wait_epoch_gpu(const uint32_t* flag, uint32_t epoch, uint32_t budget) {
  for (uint32_t i = 0; i < budget; ++i) {
    if ((int32_t)(ld_acquire_gpu_u32(flag) - epoch) >= 0) return true;
    if (i > 32) __nanosleep(100);
  }
  return false;
}
// MODE 0: all-gather -> GEMM (outs.p[r] = rank r's A shard; A tiles from the local shard or the local full buffer; C local)
// MODE 1: GEMM -> reduce-scatter (A, B local; outs.p[r] = rank r's staging buffer; c = this rank's result rows)
// MODE 2: GEMM -> all-to-all (A [M local tokens, K], B local; column group p of width N / world goes to rank p: outs.p[p] =
//         rank p's bf16 buffer [world * M, ldc], this rank's rows at rank * M)
// MODE 3: all-to-all -> GEMM (outs.p[p] = rank p's bf16 buffer [world * M, K / world]: all tokens, rank p's K columns; this
//         rank multiplies ITS M tokens over the whole K; copier warps stage the peers' column groups into a_full [M, K])
template <int BN, int MODE, bool OUT_BF16>
__global__ void __launch_bounds__(kCThreads, 1)
gemm_coll_kernel(const __grid_constant__ MapSet maps, const __grid_constant__ CUtensorMap map_b, void* __restrict__ c,
                 const __grid_constant__ OutPtrs outs, int M, int N, int K, int ldc, int rank, int world,
                 const uint32_t* __restrict__ my_flags, int slot, uint32_t epoch, uint32_t budget, int* status,
                 uint4* __restrict__ a_full, uint32_t* __restrict__ chunk_flags, const __grid_constant__ FlagPtrs rs_flags) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ int copier_ok;
  __shared__ int epi_ok;  // decision of the epilogue's elected waiter, read by all four epilogue warps after a barrier
  constexpr uint32_t kABytes = kCBM * kCBK * 2, kBBytes = BN * kCBK * 2, kStageBytes = kABytes + kBBytes;
  uint8_t* tiles = smem;
  CollSmem* sm = (CollSmem*)(smem + kCStages * kStageBytes);
  float* epi_tile = (float*)(smem + kCStages * kStageBytes + 1024);  // 4 warps x 32 x 33 floats (reduce-scatter push)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = M / kCBM, tiles_n = (N + BN - 1) / BN, ntiles = tiles_m * tiles_n;
  const int kblocks = (K + kCBK - 1) / kCBK;
  const int m_local = M / world, tiles_m_local = m_local / kCBM;
  // tile order: owner-major starting at the own rank (MODE 0) or at the next rank (MODE 1)
  auto tile_coords = [&](int t, int& owner, int& m0, int& n0) {
    constexpr int kBand = 16;
    if (MODE == 3) {
      owner = rank;
      const int band = t / (kBand * tiles_n), in_band = t % (kBand * tiles_n);
      const int rows_here = min(kBand, tiles_m - band * kBand);
      m0 = (band * kBand + in_band % rows_here) * kCBM;
      n0 = (in_band / rows_here) * BN;
      return;
    }
    if (MODE == 2) {
      // destination-major starting after the own rank (at any moment the ranks store to different peers), own columns last
      const int tiles_n_dest = tiles_n / world, per_dest = tiles_m * tiles_n_dest;
      const int o = t / per_dest, rest = t % per_dest;
      owner = (rank + 1 + o) % world;
      const int band = rest / (kBand * tiles_n_dest), in_band = rest % (kBand * tiles_n_dest);
      const int rows_here = min(kBand, tiles_m - band * kBand);
      m0 = (band * kBand + in_band % rows_here) * kCBM;
      n0 = (owner * tiles_n_dest + in_band / rows_here) * BN;
      return;
    }
    const int per_owner = tiles_m_local * tiles_n;
    const int o = t / per_owner, rest = t % per_owner;
    owner = (rank + (MODE == 1 ? 1 : 0) + o) % world;
    // inside an owner's rows: bands of 16 row tiles, the row tile varying fastest (a wave's A and B panels stay in L2)
    const int band = rest / (kBand * tiles_n), in_band = rest % (kBand * tiles_n);
    const int rows_here = min(kBand, tiles_m_local - band * kBand);
    m0 = (owner * tiles_m_local + band * kBand + in_band % rows_here) * kCBM;
    n0 = (in_band / rows_here) * BN;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < kCStages; ++i) { mbar_init(&sm->full[i], 1); mbar_init(&sm->empty[i], 1); }
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
    if (lane == 0) {
      prefetch_tensormap(&map_b);
      int st = 0, ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
        int owner, m0, n0;
        tile_coords(tile, owner, m0, n0);
        if (MODE == 0 && owner != rank) {
          // the copier warps publish every remote 128-row block of A in the local full buffer
          if (!wait_epoch_gpu(chunk_flags + m0 / kCBM, 8u, budget)) set_status(status, PEAR_ERR_FLAG_TIMEOUT);  // all 8 pieces of the block
        }
        // MODE 0: maps.a[0] = the local shard (rows relative to it), maps.a[1] = the local full-A buffer (global rows)
        const CUtensorMap* ma = MODE == 0 ? (owner == rank ? &maps.a[0] : &maps.a[1]) : &maps.a[0];
        const int am0 = (MODE == 0 && owner == rank) ? m0 - owner * m_local : m0;
        const int kbg = kblocks / world;  // MODE 3: K blocks per column group
        int group_ready = rank;
        for (int kb = 0; kb < kblocks; ++kb) {
          // MODE 3: the own column group first (local data), then the groups in the order the copier warps fetch them
          const int kb2 = MODE == 3 ? (kb + rank * kbg) % kblocks : kb;
          const int grp = MODE == 3 ? kb2 / kbg : 0;
          if (MODE == 3 && grp != rank && grp != group_ready) {
            if (!wait_epoch_gpu(chunk_flags + (m0 / kCBM) * world + grp, 8u, budget)) set_status(status, PEAR_ERR_FLAG_TIMEOUT);
            group_ready = grp;
          }
          ok = mbar_wait_bounded(&sm->empty[st], ph ^ 1, status);
          if (!ok) break;
          uint8_t* a = tiles + st * kStageBytes;
          mbar_expect_tx(&sm->full[st], kStageBytes);
          if (MODE == 3) tma_load_2d(a, grp == rank ? &maps.a[0] : &maps.a[1], grp == rank ? (kb2 - grp * kbg) * kCBK : kb2 * kCBK, m0, &sm->full[st]);
          else tma_load_2d(a, ma, kb * kCBK, am0, &sm->full[st]);
          tma_load_2d(a + kABytes, &map_b, kb2 * kCBK, n0, &sm->full[st]);
          if (++st == kCStages) { st = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(kCBM, BN, 1);
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
          const uint64_t da = umma_desc_sw128(a_addr), db = umma_desc_sw128(a_addr + kABytes);
#pragma unroll
          for (int k = 0; k < kCBK / 16; ++k)
            umma_f16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
          tcgen05_commit(&sm->empty[st]);
          if (++st == kCStages) { st = 0; ph ^= 1; }
        }
        tcgen05_commit(&sm->tmem_full[ab]);
      }
    }
  } else if (warp < 6) {
    const int q = warp & 3;
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
      const int ab = it & 1;
      int owner, m0, n0;
      tile_coords(tile, owner, m0, n0);
      // index of this tile among the owner's tiles: (m tile inside the owner's rows) * tiles_n + n tile
      const int tile_in_owner = ((m0 - owner * m_local) / kCBM) * tiles_n + n0 / BN;
      // The four epilogue warps meet at named barriers inside a tile, so they must take the SAME decision to go on or to
      // leave: one elected thread waits (it gives up only on its own poll budget, never because another CTA reported a
      // problem) and publishes the result; every warp reads it after a barrier that all of them always reach. A late
      // peer flag is recorded in the status word but does not end the tile: its rows are wrong, the kernel still returns.
      if (warp == 2 && lane == 0) {
        bool w = ok && mbar_wait_bounded(&sm->tmem_full[ab], (it >> 1) & 1, nullptr);
        if (ok && !w) set_status(status, PEAR_ERR_MBAR_TIMEOUT);
        if (w && MODE == 1 && owner == rank && world > 1) {
          for (int s2 = 1; s2 < world; ++s2) {
            const int src = (rank + s2) % world;
            if (!wait_epoch(rs_flags.p[rank] + (size_t)src * tiles_m_local * tiles_n + tile_in_owner, epoch, budget)) set_status(status, PEAR_ERR_FLAG_TIMEOUT);
          }
        }
        *(volatile int*)&epi_ok = w ? 1 : 0;
      }
      asm volatile("bar.sync 4, 128;" ::: "memory");
      ok = *(volatile int*)&epi_ok != 0;
      if (!ok) break;  // all 128 epilogue threads leave together
      tcgen05_fence_after();
      const int row = m0 + q * 32 + lane;
      asm volatile("bar.sync 4, 128;" ::: "memory");  // everyone has read the decision before the next tile overwrites it
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + ab * BN + c0, r);
        tcgen05_wait_ld();
        const int col = n0 + c0;
        if (MODE == 1) {
          const int lrow = row - owner * m_local;
          if (owner != rank) {
            // push the partial into the owner's staging slot of this source: stage[owner][rank][lrow][col]. The accumulator
            // arrives one ROW per lane; over NVLink a warp store should cover contiguous bytes, so the 32 x 32 block is
            // transposed through shared memory and written one 128-byte row segment per warp instruction.
            float* tb = epi_tile + (warp - 2) * (32 * 33);
#pragma unroll
            for (int j = 0; j < 32; ++j) tb[lane * 33 + j] = __uint_as_float(r[j]);
            __syncwarp();
            // the staged partials are bf16 (half the NVLink bytes and half the owner's re-read; the sum itself stays fp32)
            const int lrow0 = (m0 - owner * m_local) + q * 32;
            __nv_bfloat16* dst0 = (__nv_bfloat16*)outs.p[owner] + ((size_t)rank * m_local + lrow0) * ldc + col;
            const int hr = lane >> 4, cc = (lane & 15) * 2;
            if (col + cc + 1 < N) {
#pragma unroll 4
              for (int rr = 0; rr < 32; rr += 2)
                *(__nv_bfloat162*)(dst0 + (size_t)(rr + hr) * ldc + cc) = __floats2bfloat162_rn(tb[(rr + hr) * 33 + cc], tb[(rr + hr) * 33 + cc + 1]);
            }
            __syncwarp();
          } else {
            // own tile: add what the other sources pushed (their flags were awaited before this loop) and write the result
            float* dst = (float*)c + (size_t)lrow * ldc + col;
            for (int s2 = 1; s2 < world; ++s2) {
              const int src = (rank + s2) % world;
              const __nv_bfloat16* ps = (const __nv_bfloat16*)outs.p[rank] + ((size_t)src * m_local + lrow) * ldc + col;
              if (col + 32 <= N) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  const uint4 v = __ldcg((const uint4*)(ps + j));
                  const __nv_bfloat162* h2 = (const __nv_bfloat162*)&v;
#pragma unroll
                  for (int u = 0; u < 4; ++u) {
                    const float2 f = __bfloat1622float2(h2[u]);
                    r[j + 2 * u] = __float_as_uint(__uint_as_float(r[j + 2 * u]) + f.x);
                    r[j + 2 * u + 1] = __float_as_uint(__uint_as_float(r[j + 2 * u + 1]) + f.y);
                  }
                }
              } else {
                for (int j = 0; j < 32; ++j)
                  if (col + j < N) r[j] = __float_as_uint(__uint_as_float(r[j]) + __bfloat162float(ps[j]));
              }
            }
            if (col + 32 <= N) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *(float4*)(dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            } else {
              for (int j = 0; j < 32; ++j)
                if (col + j < N) dst[j] = __uint_as_float(r[j]);
            }
          }
        } else if (MODE == 2) {
          // the 32 x 32 block goes to the owner of its column group as bf16: transposed through shared memory so that one
          // warp store covers two 64-byte row segments instead of 32 scattered 4-byte words
          float* tb = epi_tile + (warp - 2) * (32 * 33);
#pragma unroll
          for (int j = 0; j < 32; ++j) tb[lane * 33 + j] = __uint_as_float(r[j]);
          __syncwarp();
          const int group = N / world;
          __nv_bfloat16* dst0 = (__nv_bfloat16*)outs.p[owner] + ((size_t)rank * M + m0 + q * 32) * ldc + (col - owner * group);
          const int hr = lane >> 4, cc = (lane & 15) * 2;
#pragma unroll 4
          for (int rr = 0; rr < 32; rr += 2) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(tb[(rr + hr) * 33 + cc], tb[(rr + hr) * 33 + cc + 1]);
            *(__nv_bfloat162*)(dst0 + (size_t)(rr + hr) * ldc + cc) = v;
          }
          __syncwarp();
        } else if (OUT_BF16) {
          __nv_bfloat16* dst = (__nv_bfloat16*)c + (size_t)row * ldc + col;
          if (col + 32 <= N) {
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
          if (col + 32 <= N) {
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
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm->tmem_empty[ab]);
      if (MODE == 1 && owner != rank) {
        // the whole tile is stored: publish it to the owner (release after every epilogue thread's stores)
        __threadfence_system();
        asm volatile("bar.sync 4, 128;" ::: "memory");
        if (warp == 2 && lane == 0)
          asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(rs_flags.p[owner] + (size_t)rank * tiles_m_local * tiles_n + tile_in_owner), "r"(epoch) : "memory");
      }
    }
    if (MODE != 0) __threadfence_system();  // the adds / peer stores are performed before the host-ordered "done" signal that follows the kernel
  }
  if (MODE == 0 && warp >= 6 && world > 1) {
    // ------------------------------------------------------------------------------------------------ copier warps
    const int ct = threadIdx.x - 192;  // 0..63
    // A 128-row block is copied as kSub pieces of 16 rows by (up to) kSub different CTAs, so that all SMs' copier warps
    // share the gather; the block's counter (zero at launch) counts its pieces, the consumer waits for kSub.
    constexpr int kSub = 8;
    const int remote_tiles = tiles_m - tiles_m_local;
    const size_t vec_per_piece = (size_t)(kCBM / kSub) * K / 8;  // 16-byte vectors of 16 rows (rows are contiguous: lda == K)
    for (int cidx = blockIdx.x; cidx < remote_tiles * kSub; cidx += gridDim.x) {
      const int t = cidx / kSub, piece = cidx % kSub;
      const int owner = (rank + 1 + t / tiles_m_local) % world, mt = t % tiles_m_local;
      if (ct == 0) {
        copier_ok = wait_epoch(my_flags + slot * kCMaxRanks + owner, epoch, budget) ? 1 : 0;
        if (!copier_ok) set_status(status, PEAR_ERR_FLAG_TIMEOUT);
      }
      asm volatile("bar.sync 3, 64;" ::: "memory");
      if (copier_ok) {
        const uint4* src = (const uint4*)outs.p[owner] + ((size_t)mt * kSub + piece) * vec_per_piece;
        uint4* dst = a_full + ((size_t)(owner * tiles_m_local + mt) * kSub + piece) * vec_per_piece;
        for (size_t i = ct; i < vec_per_piece; i += 64 * 8) {
          uint4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (i + (size_t)u * 64 < vec_per_piece)
              asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w) : "l"(src + i + (size_t)u * 64) : "memory");
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (i + (size_t)u * 64 < vec_per_piece) dst[i + (size_t)u * 64] = v[u];
        }
        // the block is read by TMA (async proxy) of other CTAs: make the generic-proxy stores visible to it
        asm volatile("fence.proxy.async;" ::: "memory");
        __threadfence();
      }
      asm volatile("bar.sync 3, 64;" ::: "memory");
      // counted also after a timeout (the status word already says so): nobody is left waiting for this block
      if (ct == 0) asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(chunk_flags + owner * tiles_m_local + mt), "r"(1u) : "memory");
    }
  }
  if (MODE == 3 && warp >= 6 && world > 1) {
    // ------------------------------------------------------------------------------------------------ copier warps (all-to-all)
    // Peer p holds [all tokens][its K / world columns]; this rank needs its own M tokens of every column group. A
    // (128-row block, group) is copied as 8 pieces of 16 rows (contiguous at the source, strided by K here), group by
    // group starting after the own rank, and counted in chunk_flags[block * world + group] (zero at launch).
    const int ct = threadIdx.x - 192;
    constexpr int kSub = 8;
    const int kg8 = K / world / 8;  // 16-byte vectors per source row
    const size_t vec_per_piece = (size_t)(kCBM / kSub) * kg8;
    for (int cidx = blockIdx.x; cidx < (world - 1) * tiles_m * kSub; cidx += gridDim.x) {
      const int t = cidx / kSub, piece = cidx % kSub;
      const int p = (rank + 1 + t / tiles_m) % world, mt = t % tiles_m;
      if (ct == 0) {
        copier_ok = wait_epoch(my_flags + slot * kCMaxRanks + p, epoch, budget) ? 1 : 0;
        if (!copier_ok) set_status(status, PEAR_ERR_FLAG_TIMEOUT);
      }
      asm volatile("bar.sync 3, 64;" ::: "memory");
      if (copier_ok) {
        const int row0 = mt * kCBM + piece * (kCBM / kSub);
        const uint4* src = (const uint4*)outs.p[p] + ((size_t)rank * M + row0) * kg8;
        uint4* dst = a_full + ((size_t)row0 * K + (size_t)p * (K / world)) / 8;
        for (size_t i = ct; i < vec_per_piece; i += 64 * 8) {
          uint4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (i + (size_t)u * 64 < vec_per_piece)
              asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w) : "l"(src + i + (size_t)u * 64) : "memory");
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const size_t e = i + (size_t)u * 64;
            if (e < vec_per_piece) dst[(e / kg8) * (size_t)(K / 8) + e % kg8] = v[u];
          }
        }
        asm volatile("fence.proxy.async;" ::: "memory");
        __threadfence();
      }
      asm volatile("bar.sync 3, 64;" ::: "memory");
      if (ct == 0) asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(chunk_flags + mt * world + p), "r"(1u) : "memory");
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

static PFN_cuTensorMapEncodeTiled_v12000 coll_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    cudaDriverEntryPointQueryResult q;
    void* p = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
  }
  return fn;
}

static int coll_map_bf16(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  auto enc = coll_encode();
  if (!enc) return (int)cudaErrorNotSupported;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)kCBK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

template <int BN, int MODE, bool OUT_BF16>
static int launch_coll(const MapSet& maps, const CUtensorMap& mb, void* c, const OutPtrs& outs, int M, int N, int K, int ldc, int rank,
                       int world, const uint32_t* flags, int slot, uint32_t epoch, uint32_t budget, int* status, int num_sms,
                       cudaStream_t stream, void* a_full = nullptr, void* chunk_flags = nullptr, const FlagPtrs* rs_flags = nullptr) {
  constexpr int smem = kCStages * (kCBM * kCBK * 2 + BN * kCBK * 2) + 1024 + 4 * 32 * 33 * 4;
  static bool configured = false;
  if (!configured) {
    PEAR_CUDA_CHECK(cudaFuncSetAttribute(gemm_coll_kernel<BN, MODE, OUT_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  const int ntiles = (M / kCBM) * ((N + BN - 1) / BN);
  const int grid = ntiles < num_sms ? ntiles : num_sms;
  gemm_coll_kernel<BN, MODE, OUT_BF16><<<grid, kCThreads, smem, stream>>>(maps, mb, c, outs, M, N, K, ldc, rank, world, flags, slot, epoch,
                                                                          budget, status, (uint4*)a_full, (uint32_t*)chunk_flags, rs_flags ? *rs_flags : FlagPtrs{});
  PEAR_LAUNCH_CHECK();
  return 0;
}

}  // namespace pear

using namespace pear;

// all-gather -> GEMM. a_shards[r]: rank r's [M / world, K] bf16 shard (symmetric memory, rows contiguous: lda == K);
// my_flags: this rank's signal region; the owner of shard r must have signalled `epoch` in `slot` (pear_symm_signal)
// after writing it. a_full: local [M, K] bf16 buffer the remote shards are copied into; chunk_flags: local uint32 per
// 128-row block of A, ZERO at launch (the 8 pieces of a block each add one). C [M, N] is local (fp32 or bf16). M / world must be a multiple of 128.
PEAR_API int pear_ag_gemm_bf16(const void* const* a_shards, const void* b, void* c, int M, int N, int K, int lda, int ldb, int ldc,
                               int out_bf16, int rank, int world, const void* my_flags, int slot, unsigned epoch, unsigned budget,
                               int* status, int num_sms, void* a_full, void* chunk_flags, void* stream) {
  if (world < 1 || world > kCMaxRanks || M % (world * kCBM) || lda != K || (K % 8) || (ldb % 8)) return (int)cudaErrorInvalidValue;
  MapSet maps;
  int e = coll_map_bf16(&maps.a[0], a_shards[rank], M / world, K, lda, kCBM);
  if (e) return e;
  e = coll_map_bf16(&maps.a[1], a_full, M, K, K, kCBM);
  if (e) return e;
  for (int r = 2; r < kCMaxRanks; ++r) maps.a[r] = maps.a[0];
  CUtensorMap mb;
  e = coll_map_bf16(&mb, b, N, K, ldb, 256);
  if (e) return e;
  OutPtrs shards{};
  for (int r = 0; r < world; ++r) shards.p[r] = (float*)const_cast<void*>(a_shards[r]);
  cudaStream_t s = (cudaStream_t)stream;
  return out_bf16 ? launch_coll<256, 0, true>(maps, mb, c, shards, M, N, K, ldc, rank, world, (const uint32_t*)my_flags, slot, epoch, budget, status, num_sms, s, a_full, chunk_flags)
                  : launch_coll<256, 0, false>(maps, mb, c, shards, M, N, K, ldc, rank, world, (const uint32_t*)my_flags, slot, epoch, budget, status, num_sms, s, a_full, chunk_flags);
}

// GEMM -> reduce-scatter. A [M, K_local], B [N, K_local] local bf16. stage[r]: rank r's staging buffer in symmetric memory,
// bf16 [world sources][M / world][ldc] (ldc a multiple of 8); flags[r]: rank r's uint32 [world sources][tiles of an owner] in symmetric memory
// (any values below `epoch`); out: local fp32 [M / world, ldc] result. Before the call every rank must have finished
// reading its staging buffer of the previous call (one pear_symm_signal / wait round). The result is complete when the
// kernel ends.
PEAR_API int pear_gemm_rs_bf16(const void* a, const void* b, void* const* stage, void* const* flags, void* out, int M, int N, int K, int lda,
                               int ldb, int ldc, int rank, int world, unsigned epoch, unsigned budget, int* status, int num_sms, void* stream) {
  if (world < 1 || world > kCMaxRanks || M % (world * kCBM) || (lda % 8) || (ldb % 8) || (ldc % 8) || N % 4) return (int)cudaErrorInvalidValue;
  MapSet maps;
  int e = coll_map_bf16(&maps.a[0], a, M, K, lda, kCBM);
  if (e) return e;
  for (int r = 1; r < kCMaxRanks; ++r) maps.a[r] = maps.a[0];
  CUtensorMap mb;
  e = coll_map_bf16(&mb, b, N, K, ldb, 256);
  if (e) return e;
  OutPtrs outs{};
  FlagPtrs fl{};
  for (int r = 0; r < world; ++r) { outs.p[r] = (float*)stage[r]; fl.p[r] = (uint32_t*)flags[r]; }
  return launch_coll<256, 1, false>(maps, mb, out, outs, M, N, K, ldc, rank, world, nullptr, 0, epoch, budget, status, num_sms, (cudaStream_t)stream,
                                    nullptr, nullptr, &fl);
}

// Projection GEMM -> all-to-all (Ulysses: tokens sharded before, heads sharded after). A [M, K] (this rank's tokens), B
// [N, K] local bf16; the columns are `world` groups of N / world (a multiple of 128) and group p is stored as bf16 into
// outs[p] (rank p's [world * M, ldo] buffer in symmetric memory) at rows [rank * M, (rank + 1) * M). M a multiple of 128.
// The stores are visible to the peers after a pear_symm_signal / pear_symm_wait round that follows the kernel.
PEAR_API int pear_gemm_a2a_bf16(const void* a, const void* b, void* const* outs_, int M, int N, int K, int lda, int ldb, int ldo, int rank,
                                int world, int* status, int num_sms, void* stream) {
  if (world < 1 || world > kCMaxRanks || M % kCBM || N % world || (N / world) % 128 || (lda % 8) || (ldb % 8) || (ldo % 2))
    return (int)cudaErrorInvalidValue;
  MapSet maps;
  int e = coll_map_bf16(&maps.a[0], a, M, K, lda, kCBM);
  if (e) return e;
  for (int r = 1; r < kCMaxRanks; ++r) maps.a[r] = maps.a[0];
  const bool wide = (N / world) % 256 == 0;
  CUtensorMap mb;
  e = coll_map_bf16(&mb, b, N, K, ldb, wide ? 256 : 128);
  if (e) return e;
  OutPtrs outs{};
  for (int r = 0; r < world; ++r) outs.p[r] = (float*)outs_[r];
  cudaStream_t s = (cudaStream_t)stream;
  return wide ? launch_coll<256, 2, true>(maps, mb, nullptr, outs, M, N, K, ldo, rank, world, nullptr, 0, 0, 1u << 22, status, num_sms, s)
              : launch_coll<128, 2, true>(maps, mb, nullptr, outs, M, N, K, ldo, rank, world, nullptr, 0, 0, 1u << 22, status, num_sms, s);
}

// All-to-all -> GEMM (Ulysses: head-sharded attention output in, token-sharded o_proj out). srcs[p]: rank p's bf16 buffer
// [world * M, K / world] in symmetric memory (all tokens, rank p's columns, rows contiguous), published by pear_symm_signal
// (`slot`, `epoch`) after it was written. b [N, K] local. C [M, N] = this rank's tokens (rows [rank * M, ...) of every
// source) times b^T. a_full: local bf16 [M, K] staging; chunk_flags: uint32 [M / 128 * world], ZERO at launch.
// M a multiple of 128, K / world a multiple of 64.
PEAR_API int pear_a2a_gemm_bf16(const void* const* srcs, const void* b, void* c, int M, int N, int K, int ldb, int ldc, int out_bf16,
                                int rank, int world, const void* my_flags, int slot, unsigned epoch, unsigned budget, int* status,
                                int num_sms, void* a_full, void* chunk_flags, void* stream) {
  if (world < 1 || world > kCMaxRanks || M % kCBM || K % world || (K / world) % kCBK || (ldb % 8)) return (int)cudaErrorInvalidValue;
  const int kg = K / world;
  MapSet maps;
  int e = coll_map_bf16(&maps.a[0], (const __nv_bfloat16*)srcs[rank] + (size_t)rank * M * kg, M, kg, kg, kCBM);
  if (e) return e;
  e = coll_map_bf16(&maps.a[1], a_full, M, K, K, kCBM);
  if (e) return e;
  for (int r = 2; r < kCMaxRanks; ++r) maps.a[r] = maps.a[0];
  CUtensorMap mb;
  e = coll_map_bf16(&mb, b, N, K, ldb, 256);
  if (e) return e;
  OutPtrs src{};
  for (int r = 0; r < world; ++r) src.p[r] = (float*)const_cast<void*>(srcs[r]);
  cudaStream_t s = (cudaStream_t)stream;
  return out_bf16 ? launch_coll<256, 3, true>(maps, mb, c, src, M, N, K, ldc, rank, world, (const uint32_t*)my_flags, slot, epoch, budget, status, num_sms, s, a_full, chunk_flags)
                  : launch_coll<256, 3, false>(maps, mb, c, src, M, N, K, ldc, rank, world, (const uint32_t*)my_flags, slot, epoch, budget, status, num_sms, s, a_full, chunk_flags);
}
