// bf16 GEMM on CTA pairs: C[M,N] (+)= alpha * A * B^T (+ bias) with `tcgen05.mma.cta_group::2`.
//
// Two CTAs of a cluster (two SMs) compute one 256 x 256 output tile.  Each CTA loads its own 128 rows of A and ONE
// HALF (128 columns) of the B tile; the leader CTA's single MMA thread issues 256 x 256 x 16 instructions that read A
// and the two B halves from both CTAs' shared memory and write each CTA's 128 x 256 accumulator into its own TMEM.
// Compared with one CTA per 128 x 256 tile this halves the B bytes every SM pulls from L2 and stores in shared
// memory per flop, so a stage is 32 KB instead of 48 KB and the ring is six stages deep instead of four: the
// single-CTA kernel is limited by exactly that (operand fetch, not tensor-core issue).
//
// Per CTA (192 threads): warp 0 TMA producer, warp 1 TMEM allocation (+ MMA issue in the leader), warps 2-5 epilogue.
//   full[s]       leader only: transaction bytes of BOTH CTAs' loads of stage s (the peer's TMA signals it remotely)
//   empty[s]      both CTAs: `tcgen05.commit` with a two-CTA mask when the MMAs that read stage s have completed
//   tmem_full[b]  both CTAs: the same commit form after the last k-block of a tile
//   tmem_empty[b] leader only, count 8: the four epilogue warps of each CTA arrive (the peer's remotely)
// Loads are plain 2-CTA TMA loads, one per CTA: no load is multicast.  Every wait is bounded; a timeout writes a code
// into the status word and the pair leaves through the common exit (cluster barrier, TMEM release).
// The reference has no GEMM kernel of its own (cuBLAS through torch); this is the dense-layer hot path of training.
#include "sm100_common.cuh"

namespace b200 {

constexpr int G2_BM = 128;        // rows per CTA (256 per pair)
constexpr int G2_BN = 256;        // columns per pair; each CTA stages 128 of them
constexpr int G2_BK = 64;
constexpr int G2_THREADS = 192;
constexpr int G2_STAGES = 6;
constexpr int G2_A_BYTES = G2_BM * G2_BK * 2;          // 16 KB
constexpr int G2_B_BYTES = (G2_BN / 2) * G2_BK * 2;    // 16 KB
constexpr int G2_STAGE_BYTES = G2_A_BYTES + G2_B_BYTES;
constexpr int G2_EPI_OFFSET = G2_STAGES * G2_STAGE_BYTES;
constexpr int G2_EPI_BUF = 32 * 128;
constexpr int G2_BAR_OFFSET = G2_EPI_OFFSET + 4 * 2 * G2_EPI_BUF;
constexpr int G2_SMEM_TOTAL = G2_BAR_OFFSET + 256 + 1024;

enum Gemm2Flags : int { G2_OUT_F32 = 1, G2_ACCUMULATE = 2, G2_BIAS = 4 };

struct Gemm2Args {
  const __nv_bfloat16* bias;
  int M, N, K;
  int a_mn, b_mn;
  int flags;
  float alpha;
  int tiles_m, tiles_n;   // in 256 x 256 pair tiles
  int* err;
};

struct Gemm2Maps {
  CUtensorMap a, b, c;
};

// ---- cluster / 2-CTA forms of the primitives
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local` (an address in this CTA's shared window) as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into THIS CTA's shared memory whose completion bytes are counted on an mbarrier of either CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at this offset in BOTH CTAs when all MMAs issued so far by this thread have completed
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask)
               : "memory");
}

__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int GROUP = 8;  // 8 pair tiles = 2048 rows share each 256-column B panel while it is L2-hot
  const int per_group = GROUP * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP;
  const int gsize = min(tiles_m - first_m, GROUP);
  const int r = tile - g * per_group;
  tm = first_m + (r % gsize);
  tn = r / gsize;
}

__global__ void __launch_bounds__(G2_THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ Gemm2Maps maps, void* Cptr, Gemm2Args p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + G2_BAR_OFFSET);
  uint64_t* empty_bar = full_bar + G2_STAGES;
  uint64_t* tmem_full = empty_bar + G2_STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  __shared__ int cta_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();        // 0 = leader (issues the MMAs), 1 = peer
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int nkb = (p.K + G2_BK - 1) / G2_BK;

  if (threadIdx.x == 0) {
    cta_abort = 0;
    for (int i = 0; i < G2_STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tmem_full[i], 1); mbar_init(&tmem_empty[i], 8); }
    fence_barrier_init();
    prefetch_tmap(&maps.a); prefetch_tmap(&maps.b); prefetch_tmap(&maps.c);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers exist before any remote signal can reach them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------ producer (both CTAs): own A rows, own half of B
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        int tm, tn;
        pair_tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * 256 + static_cast<int>(rank) * G2_BM;
        const int n0 = tn * G2_BN + static_cast<int>(rank) * (G2_BN / 2);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, p.err, ERR_WAIT_EMPTY, &cta_abort)) { ok = false; break; }
          uint8_t* sA = smem + s * G2_STAGE_BYTES;
          uint8_t* sB = sA + G2_A_BYTES;
          const uint32_t leader_full = map_to_cta(smem_u32(&full_bar[s]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * G2_STAGE_BYTES);
          const int k0 = kb * G2_BK;
          if (!p.a_mn) {
            tma_load_2d_pair(sA, &maps.a, leader_full, k0, m0);
          } else {
            tma_load_2d_pair(sA, &maps.a, leader_full, m0, k0);
            tma_load_2d_pair(sA + 8192, &maps.a, leader_full, m0 + 64, k0);
          }
          if (!p.b_mn) {
            tma_load_2d_pair(sB, &maps.b, leader_full, k0, n0);
          } else {
            tma_load_2d_pair(sB, &maps.b, leader_full, n0, k0);
            tma_load_2d_pair(sB + 8192, &maps.b, leader_full, n0 + 64, k0);
          }
          if (++s == G2_STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc_bf16(256, G2_BN, p.a_mn, p.b_mn);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, ++it) {
        const int buf = it & 1;
        if (!mbar_wait(&tmem_empty[buf], ((it >> 1) & 1) ^ 1, p.err, ERR_WAIT_TMEM_EMPTY, &cta_abort)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * G2_BN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, p.err, ERR_WAIT_FULL, &cta_abort)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(smem + s * G2_STAGE_BYTES);
          const uint32_t b_base = a_base + G2_A_BYTES;
#pragma unroll
          for (int k = 0; k < G2_BK / 16; ++k) {
            const uint64_t adesc = p.a_mn ? make_smem_desc_sw128(a_base + k * 2048, 8192, 1024)
                                          : make_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = p.b_mn ? make_smem_desc_sw128(b_base + k * 2048, 8192, 1024)
                                          : make_smem_desc_sw128(b_base + k * 32, 16, 1024);
            umma_bf16_ss_pair(d_tmem, adesc, bdesc, idesc, (kb | k) != 0);
          }
          umma_commit_pair(&empty_bar[s]);
          if (++s == G2_STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit_pair(&tmem_full[buf]);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------ epilogue (both CTAs): this CTA's 128 rows of the pair tile
    const int q = warp & 3;
    const bool out_f32 = p.flags & G2_OUT_F32;
    const bool accum = p.flags & G2_ACCUMULATE;
    const bool has_bias = p.flags & G2_BIAS;
    uint8_t* stage_base = smem + G2_EPI_OFFSET + (warp - 2) * 2 * G2_EPI_BUF;
    int sbuf = 0;
    int it = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, ++it) {
      int tm, tn;
      pair_tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      const int buf = it & 1;
      ok = mbar_wait(&tmem_full[buf], (it >> 1) & 1, p.err, ERR_WAIT_TMEM_FULL, &cta_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int row0 = tm * 256 + static_cast<int>(rank) * G2_BM + q * 32;
      const uint32_t t_row = tmem_base + buf * G2_BN + (static_cast<uint32_t>(q * 32) << 16);
      const int sw = lane & 7;
#pragma unroll 1
      for (int c = 0; c < G2_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = tn * G2_BN + c * 32;
        if (col0 >= p.N || row0 >= p.M) continue;  // warp-uniform: the whole chunk is outside C
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
        if (has_bias) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (col0 + i < p.N) v[i] += __bfloat162float(p.bias[col0 + i]);
        }
        uint8_t* sb = stage_base + sbuf * G2_EPI_BUF;
        if (out_f32) {
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(sb + lane * 128 + ((j ^ sw) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (accum) tma_reduce_add_2d(&maps.c, sb, col0, row0);
            else tma_store_2d(&maps.c, sb, col0, row0);
            tma_store_commit();
          }
          sbuf ^= 1;
        } else {
          const int half = c & 1;
          if (half == 0) {
            if (lane == 0) tma_store_wait_read<1>();
            __syncwarp();
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_bf16x2(v[8 * j], v[8 * j + 1]);
            o.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
            o.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
            o.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
            *reinterpret_cast<uint4*>(sb + lane * 128 + (((half * 4 + j) ^ sw) << 4)) = o;
          }
          const bool last_of_pair = half == 1 || col0 + 32 >= p.N;
          if (last_of_pair) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&maps.c, sb, col0 - half * 32, row0);
              tma_store_commit();
            }
            sbuf ^= 1;
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[buf]), 0));
    }
    if (lane == 0) tma_store_wait<0>();
  }

  // common exit: nobody leaves while its partner can still read its shared memory, write its TMEM or signal it
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

int make_tmap_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                 uint32_t box_outer, bool f32);

}  // namespace b200

using namespace b200;

// Returns 1 when the pair kernel serves this problem (the caller falls back to the single-CTA kernel otherwise).
extern "C" int b200_gemm2_supported(int M, int N, int K) { return M >= 512 && N >= 256 && K >= 64; }

// Same contract as b200_gemm_bf16 (plain operands, no split-K).
extern "C" int b200_gemm2_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda, long long ldb,
                               long long ldc, int a_mn, int b_mn, int flags, float alpha, int max_ctas, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (N % 8) || (ldc % 4) || (!(flags & G2_OUT_F32) && (ldc % 8))) return -10;
  if ((flags & G2_ACCUMULATE) && !(flags & G2_OUT_F32)) return -12;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -11;
  Gemm2Maps maps;
  int rc;
  if (!a_mn) rc = make_tmap_2d(&maps.a, A, K, M, lda, G2_BK, G2_BM, false);
  else rc = make_tmap_2d(&maps.a, A, M, K, lda, 64, G2_BK, false);
  if (rc) return rc;
  if (!b_mn) rc = make_tmap_2d(&maps.b, B, K, N, ldb, G2_BK, G2_BN / 2, false);
  else rc = make_tmap_2d(&maps.b, B, N, K, ldb, 64, G2_BK, false);
  if (rc) return rc;
  const bool f32 = flags & G2_OUT_F32;
  rc = make_tmap_2d(&maps.c, C, N, M, ldc, f32 ? 32 : 64, 32, f32);
  if (rc) return rc;
  Gemm2Args p;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.M = M; p.N = N; p.K = K;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.flags = flags;
  p.alpha = alpha;
  p.tiles_m = (M + 255) / 256;
  p.tiles_n = (N + G2_BN - 1) / G2_BN;
  p.err = err;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm2_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_TOTAL) != cudaSuccess) return -3;
    attr_set = true;
  }
  static int num_sms = 0;
  if (!num_sms) {
    int dev;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  int pairs = num_sms / 2;
  if (max_ctas > 1 && max_ctas / 2 < pairs) pairs = max_ctas / 2;
  const int tiles = p.tiles_m * p.tiles_n;
  if (tiles < pairs) pairs = tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(G2_THREADS);
  cfg.dynamicSmemBytes = G2_SMEM_TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm2_bf16_kernel, maps, C, p);
  return e == cudaSuccess ? 0 : -4;
}
