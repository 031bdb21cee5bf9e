// bf16 GEMM for sm_100a: tcgen05.mma with TMEM accumulators, TMA-fed operand
// pipeline, persistent warp-specialised CTAs.
//
//   C[M,N] (+)= alpha * A[M,K] * B[N,K]^T (+ bias[N])
//
// A and B may each be K-major (contraction dimension contiguous) or MN-major
// (the M/N dimension contiguous), which covers the three GEMMs of a linear
// layer without a transposed weight copy:
//   forward  Y  = X  * W^T      A = X  (K-major)   B = W  (K-major)
//   dgrad    dX = dY * W        A = dY (K-major)   B = W  (MN-major)
//   wgrad    dW += dY^T * X     A = dY (MN-major)  B = X  (MN-major), fp32 accumulate
//
// Roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and
// TMEM owner, warps 2-5 = epilogue (TMEM -> registers -> global).  Two TMEM
// accumulator buffers let the epilogue of tile i overlap the main loop of tile
// i+1.  The library GEMM this replaces is cuBLAS behind nn.Linear in the
// reference (opt_prime traced submodules call nn.Linear -> cuBLASLt).
#include "sm100_common.cuh"

namespace b200 {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 224;  // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue, warp 6 peer push (all-gather)
constexpr int GEMM_UMMA_K = 16;

enum GemmFlags : int {
  GEMM_OUT_F32 = 1,     // C is fp32 (else bf16)
  GEMM_ACCUMULATE = 2,  // C += result (C must be fp32 or bf16 as per GEMM_OUT_F32)
  GEMM_BIAS = 4,        // add bf16 bias[N]
};

constexpr int GEMM_MAX_PARTS = 8;

struct GemmArgs {
  void* C;
  const __nv_bfloat16* bias;
  int M, N, K;
  long long ldc;
  int a_mn, b_mn;
  int flags;
  float alpha;
  int tiles_m, tiles_n;
  int ksplit;  // >1: each output tile is computed by `ksplit` work items over disjoint K ranges (fp32 reduce-add epilogue)
  int* err;
  // ---- operands split by rows over several buffers, each possibly in ANOTHER GPU's memory (peer-mapped):
  // A row block m belongs to part m / a_part_rows and is loaded through maps.a[part] (all-gather -> GEMM);
  // C row block m goes to part m / c_part_rows through maps.c[part] (GEMM -> reduce-scatter: the epilogue's TMA
  // stores land in the owner's staging buffer).  Parts == 1 is the plain GEMM.
  int a_parts, a_part_rows;
  int c_parts, c_part_rows;
  int tile_rotate;                 // M-tile order starts here (local rows first for AG, remote rows first for RS)
  const uint32_t* ready_flags;     // [MAX_PARTS] epochs written by the owners of the A parts (may be null)
  uint32_t ready_epoch;
  const uint32_t* ready_epoch_ptr; // when set, the epoch is read from device memory (launches replayed from a CUDA graph)
  // ---- all-gather by push, inside this kernel: warp 6 of every CTA copies a slice of this rank's A shard into every
  // peer's gather buffer (plain stores over NVLink); the CTA that finishes last raises this rank's flag on all peers.
  const uint4* push_src;           // this rank's shard (null: no push)
  long long push_n16;              // its size in 16-byte units
  uint4* push_dst[GEMM_MAX_PARTS]; // where the shard goes in each peer's buffer (entry of this rank unused)
  uint32_t* push_flag[GEMM_MAX_PARTS];  // flag word of this rank on each peer
  unsigned int* push_counter;      // local counter of finished CTAs (zero before launch; reset by the last CTA)
  int push_rank, push_world;
};

struct GemmMaps {
  CUtensorMap a[GEMM_MAX_PARTS];
  CUtensorMap b;
  CUtensorMap c[GEMM_MAX_PARTS];
};

__device__ __forceinline__ bool wait_ready_flag(const uint32_t* flag, uint32_t epoch, int* err, volatile int* cta_abort) {
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int32_t>(v - epoch) >= 0) return true;
    if ((++spins & 0xff) == 0) {
      if (*cta_abort) return false;
      if (t0 == 0) t0 = globaltimer_ns();
      else if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
        *cta_abort = 1;
        atomicCAS(err, 0, ERR_WAIT_PEER);
        return false;
      }
    }
  }
}

template <int BN>
struct GemmSmem {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES;   // 1024-aligned
  static constexpr int EPI_BUF_BYTES = 32 * 128;            // 32 rows x 128 B
  static constexpr int BAR_OFFSET = EPI_OFFSET + 4 * 2 * EPI_BUF_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // barriers + alignment slack
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  // Grouped rasterisation: 8 M-tiles share each B panel while it is L2-hot.
  constexpr int GROUP = 8;
  int per_group = GROUP * tiles_n;
  int g = tile / per_group;
  int first_m = g * GROUP;
  int gsize = min(tiles_m - first_m, GROUP);
  int r = tile - g * per_group;
  tm = first_m + (r % gsize);
  tn = r / gsize;
}

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ GemmMaps maps, GemmArgs p) {
  using S = GemmSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + S::STAGES;
  uint64_t* tmem_full = empty_bar + S::STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  __shared__ int cta_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int mn_tiles = p.tiles_m * p.tiles_n;
  const int num_tiles = mn_tiles * p.ksplit;
  const int nkb_total = (p.K + GEMM_BK - 1) / GEMM_BK;
  const int nkb_per = (nkb_total + p.ksplit - 1) / p.ksplit;

  if (threadIdx.x == 0) {
    cta_abort = 0;
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);
    }
    fence_barrier_init();
    prefetch_tmap(&maps.a[0]);
    prefetch_tmap(&maps.b);
    prefetch_tmap(&maps.c[0]);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      uint32_t ready_mask = p.push_src ? (1u << p.push_rank) : 0u;  // the local shard needs no flag
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile % mn_tiles, p.tiles_m, p.tiles_n, tm, tn);
        tm = (tm + p.tile_rotate) % p.tiles_m;
        const int m0 = tm * GEMM_BM, n0 = tn * BN;
        int a_part = 0, a_y = m0;
        if (p.a_parts > 1) {
          a_part = m0 / p.a_part_rows;
          a_y = m0 - a_part * p.a_part_rows;
          if (p.ready_flags && !((ready_mask >> a_part) & 1u)) {
            const uint32_t want = p.ready_epoch_ptr ? *p.ready_epoch_ptr : p.ready_epoch;
            if (!wait_ready_flag(p.ready_flags + a_part, want, p.err, &cta_abort)) { ok = false; break; }
            asm volatile("fence.proxy.async;" ::: "memory");
            ready_mask |= 1u << a_part;
          }
        }
        const CUtensorMap* tmA = &maps.a[a_part];
        const int kb_lo = (tile / mn_tiles) * nkb_per;
        const int kb_hi = min(nkb_total, kb_lo + nkb_per);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, p.err, ERR_WAIT_EMPTY, &cta_abort)) { ok = false; break; }
          uint8_t* sA = smem + s * S::STAGE_BYTES;
          uint8_t* sB = sA + S::A_BYTES;
          mbar_expect_tx(&full_bar[s], S::STAGE_BYTES);
          const int k0 = kb * GEMM_BK;
          if (!p.a_mn) {
            tma_load_2d(sA, tmA, &full_bar[s], k0, a_y);
          } else {
#pragma unroll
            for (int j = 0; j < GEMM_BM / 64; ++j) tma_load_2d(sA + j * 8192, tmA, &full_bar[s], m0 + j * 64, k0);
          }
          if (!p.b_mn) {
            tma_load_2d(sB, &maps.b, &full_bar[s], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sB + j * 8192, &maps.b, &full_bar[s], n0 + j * 64, k0);
          }
          if (++s == S::STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) {
        // Error path: let copies already in flight land before the CTA exits.
        for (int i = 0; i < S::STAGES; ++i) {
          unsigned long long t0 = globaltimer_ns();
          while (!mbar_try_wait(&full_bar[i], 0) && !mbar_try_wait(&full_bar[i], 1) && globaltimer_ns() - t0 < 1000000ull) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(GEMM_BM, BN, p.a_mn, p.b_mn);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int buf = it & 1;
        if (!mbar_wait(&tmem_empty[buf], ((it >> 1) & 1) ^ 1, p.err, ERR_WAIT_TMEM_EMPTY, &cta_abort)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        const int kb_lo = (tile / mn_tiles) * nkb_per;
        const int kb_hi = min(nkb_total, kb_lo + nkb_per);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, p.err, ERR_WAIT_FULL, &cta_abort)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(smem + s * S::STAGE_BYTES);
          const uint32_t b_base = a_base + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < GEMM_BK / GEMM_UMMA_K; ++k) {
            const uint64_t adesc = p.a_mn ? make_smem_desc_sw128(a_base + k * 2048, 8192, 1024)
                                          : make_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = p.b_mn ? make_smem_desc_sw128(b_base + k * 2048, 8192, 1024)
                                          : make_smem_desc_sw128(b_base + k * 32, 16, 1024);
            umma_bf16_ss(d_tmem, adesc, bdesc, idesc, ((kb - kb_lo) | k) != 0);
          }
          umma_commit(&empty_bar[s]);
          if (++s == S::STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[buf]);
      }
    }
    __syncwarp();
  } else if (warp == 6) {
    // ------------------------------------------------ peer push (all-gather -> GEMM only)
    if (p.push_src) {
      const long long per_cta = (p.push_n16 + gridDim.x - 1) / gridDim.x;
      const long long lo = static_cast<long long>(blockIdx.x) * per_cta;
      long long hi = lo + per_cta;
      if (hi > p.push_n16) hi = p.push_n16;
      for (long long i = lo + lane; i < hi; i += 32) {
        const uint4 v = p.push_src[i];
        for (int r = 0; r < p.push_world; ++r)
          if (r != p.push_rank) p.push_dst[r][i] = v;
      }
      __threadfence_system();
      __syncwarp();
      if (lane == 0) {
        const unsigned int prev = atomicAdd(p.push_counter, 1u);
        if (prev == gridDim.x - 1) {  // every CTA's slice has been stored and fenced
          *p.push_counter = 0;
          __threadfence_system();
          for (int r = 0; r < p.push_world; ++r)
            if (r != p.push_rank)
              asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.push_flag[r]),
                           "r"(p.ready_epoch_ptr ? *p.ready_epoch_ptr : p.ready_epoch) : "memory");
        }
      }
    }
  } else {
    // ------------------------------------------------ epilogue (warps 2..5)
    // TMEM -> registers -> (alpha, bias, cast) -> 128B-swizzled smem staging -> TMA store, or TMA reduce-add for
    // fp32 accumulation (the add happens in the memory system: C is never read back into the SM).
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    const bool out_f32 = p.flags & GEMM_OUT_F32;
    const bool accum = p.flags & GEMM_ACCUMULATE;
    const bool has_bias = p.flags & GEMM_BIAS;
    uint8_t* stage_base = smem + S::EPI_OFFSET + (warp - 2) * 2 * S::EPI_BUF_BYTES;
    int sbuf = 0;
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
      int tm, tn;
      tile_coords(tile % mn_tiles, p.tiles_m, p.tiles_n, tm, tn);
      tm = (tm + p.tile_rotate) % p.tiles_m;
      const bool first_split = tile < mn_tiles;  // bias is added by exactly one of the K splits
      const int buf = it & 1;
      ok = mbar_wait(&tmem_full[buf], (it >> 1) & 1, p.err, ERR_WAIT_TMEM_FULL, &cta_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      int row0 = tm * GEMM_BM + q * 32;
      const CUtensorMap* tmC = &maps.c[0];
      if (p.c_parts > 1) {
        const int c_part = row0 / p.c_part_rows;
        row0 -= c_part * p.c_part_rows;
        tmC = &maps.c[c_part];
      }
      const uint32_t t_row = tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16);
      const int sw = lane & 7;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = tn * BN + c * 32;
        if (col0 >= p.N) continue;  // warp-uniform: the whole chunk is outside C
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
        if (has_bias && first_split) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (col0 + i < p.N) v[i] += __bfloat162float(p.bias[col0 + i]);
        }
        uint8_t* sb = stage_base + sbuf * S::EPI_BUF_BYTES;
        if (out_f32) {
          if (lane == 0) tma_store_wait_read<1>();  // the store issued from this buffer two chunks ago has read it
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(sb + lane * 128 + ((j ^ sw) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (accum) tma_reduce_add_2d(tmC, sb, col0, row0);
            else tma_store_2d(tmC, sb, col0, row0);
            tma_store_commit();
          }
          sbuf ^= 1;
        } else {
          const int half = c & 1;  // two 32-column chunks share one 64-column (128-byte) staging row
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
          const bool last_of_pair = half == 1 || col0 + 32 >= p.N || c == BN / 32 - 1;
          if (last_of_pair) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(tmC, sb, col0 - half * 32, row0);
              tma_store_commit();
            }
            sbuf ^= 1;
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
    }
    if (lane == 0) tma_store_wait<0>();  // all of this warp's stores have landed before the CTA may exit
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  // Tensor-map encoding is a driver call and needs a current context on the calling thread.  Threads that have
  // only ever used device 0 implicitly (autograd workers) have none until their first runtime call.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(0);
    ctx_bound = true;
  }
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || !ptr) return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2D tensor map (bf16 or fp32): `inner` contiguous elements per row, `outer` rows, row pitch `ld` elements.
int make_tmap_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                 uint32_t box_outer, bool f32) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * (f32 ? 4 : 2)};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2000 - static_cast<int>(r);
}

static int g_num_sms = 0;

template <int BN>
static int launch_gemm(const void* const* A_parts, const void* B, void* const* C_parts, GemmArgs& p, long long lda, long long ldb,
                       int max_ctas, cudaStream_t stream) {
  using S = GemmSmem<BN>;
  GemmMaps maps;
  int rc = 0;
  for (int i = 0; i < p.a_parts && !rc; ++i) {
    const int rows = p.a_parts > 1 ? p.a_part_rows : p.M;
    if (!p.a_mn) rc = make_tmap_2d(&maps.a[i], A_parts[i], p.K, rows, lda, GEMM_BK, GEMM_BM, false);
    else rc = make_tmap_2d(&maps.a[i], A_parts[i], p.M, p.K, lda, 64, GEMM_BK, false);
  }
  if (rc) return rc;
  for (int i = p.a_parts; i < GEMM_MAX_PARTS; ++i) maps.a[i] = maps.a[0];
  if (!p.b_mn) rc = make_tmap_2d(&maps.b, B, p.K, p.N, ldb, GEMM_BK, BN, false);
  else rc = make_tmap_2d(&maps.b, B, p.N, p.K, ldb, 64, GEMM_BK, false);
  if (rc) return rc;
  const bool f32 = p.flags & GEMM_OUT_F32;
  for (int i = 0; i < p.c_parts && !rc; ++i) {
    const int rows = p.c_parts > 1 ? p.c_part_rows : p.M;
    rc = make_tmap_2d(&maps.c[i], C_parts[i], p.N, rows, p.ldc, f32 ? 32 : 64, 32, f32);
  }
  if (rc) return rc;
  for (int i = p.c_parts; i < GEMM_MAX_PARTS; ++i) maps.c[i] = maps.c[0];
  p.tiles_m = (p.M + GEMM_BM - 1) / GEMM_BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return -3;
    attr_set = true;
  }
  if (!g_num_sms) {
    int dev;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  int ctas = g_num_sms;
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  int tiles = p.tiles_m * p.tiles_n * p.ksplit;
  if (tiles < ctas) ctas = tiles;
  gemm_bf16_tcgen05_kernel<BN><<<ctas, GEMM_THREADS, S::TOTAL, stream>>>(maps, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace b200

// Shared implementation of the entry points below.
static int gemm_dispatch(const void* const* A_parts, int a_parts, int a_part_rows, const void* B, void* const* C_parts, int c_parts,
                         int c_part_rows, const void* bias, int M, int N, int K, long long lda, long long ldb, long long ldc,
                         int a_mn, int b_mn, int flags, float alpha, int bn, int max_ctas, int ksplit, int tile_rotate,
                         const uint32_t* ready_flags, uint32_t ready_epoch, int* err, cudaStream_t stream,
                         const b200::GemmArgs* push_cfg = nullptr) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (N % 8) || (ldc % 4) || (!(flags & GEMM_OUT_F32) && (ldc % 8))) return -10;
  if ((flags & GEMM_ACCUMULATE) && !(flags & GEMM_OUT_F32)) return -12;  // accumulation is into fp32 only
  if (a_parts < 1 || a_parts > GEMM_MAX_PARTS || c_parts < 1 || c_parts > GEMM_MAX_PARTS) return -14;
  if (a_parts > 1 && (a_mn || a_part_rows % GEMM_BM || a_part_rows * a_parts < M)) return -15;
  if (c_parts > 1 && (c_part_rows % GEMM_BM || c_part_rows * c_parts < M)) return -15;
  for (int i = 0; i < a_parts; ++i)
    if (reinterpret_cast<uintptr_t>(A_parts[i]) & 15) return -11;
  for (int i = 0; i < c_parts; ++i)
    if (reinterpret_cast<uintptr_t>(C_parts[i]) & 15) return -11;
  if (reinterpret_cast<uintptr_t>(B) & 15) return -11;
  GemmArgs p;
  p.C = C_parts[0];
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.flags = flags;
  p.alpha = alpha;
  p.err = err;
  p.a_parts = a_parts; p.a_part_rows = a_part_rows;
  p.c_parts = c_parts; p.c_part_rows = c_part_rows;
  p.tile_rotate = tile_rotate;
  p.ready_flags = ready_flags;
  p.ready_epoch = ready_epoch;
  p.ready_epoch_ptr = push_cfg ? push_cfg->ready_epoch_ptr : nullptr;
  p.push_src = nullptr;
  p.push_n16 = 0;
  p.push_counter = nullptr;
  p.push_rank = p.push_world = 0;
  for (int i = 0; i < GEMM_MAX_PARTS; ++i) { p.push_dst[i] = nullptr; p.push_flag[i] = nullptr; }
  if (push_cfg) {
    p.push_src = push_cfg->push_src;
    p.push_n16 = push_cfg->push_n16;
    p.push_counter = push_cfg->push_counter;
    p.push_rank = push_cfg->push_rank;
    p.push_world = push_cfg->push_world;
    for (int i = 0; i < GEMM_MAX_PARTS; ++i) { p.push_dst[i] = push_cfg->push_dst[i]; p.push_flag[i] = push_cfg->push_flag[i]; }
  }
  // split-K: partial products are summed by the fp32 reduce-add epilogue, so C must be fp32 and pre-initialised
  const int nkb_total = (K + GEMM_BK - 1) / GEMM_BK;
  if (ksplit < 1) ksplit = 1;
  if (ksplit > nkb_total) ksplit = nkb_total;
  if (ksplit > 1) {
    if ((flags & (GEMM_OUT_F32 | GEMM_ACCUMULATE)) != (GEMM_OUT_F32 | GEMM_ACCUMULATE)) return -13;
    const int per = (nkb_total + ksplit - 1) / ksplit;
    ksplit = (nkb_total + per - 1) / per;  // no empty split
  }
  p.ksplit = ksplit;
  if (bn == 0) {
    // 256-wide tiles halve A re-reads; fall back to 128 when that fills the SMs better.
    long long t256 = static_cast<long long>((M + 127) / 128) * ((N + 255) / 256);
    bn = (t256 >= 148 * 2 || (N % 256 == 0 && t256 >= 148)) ? 256 : 128;
    if (N <= 128) bn = 128;
  }
  const int tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
  p.tile_rotate = ((tile_rotate % tiles_m) + tiles_m) % tiles_m;
  if (bn == 256) return launch_gemm<256>(A_parts, B, C_parts, p, lda, ldb, max_ctas, stream);
  return launch_gemm<128>(A_parts, B, C_parts, p, lda, ldb, max_ctas, stream);
}

// C[M,N] (+)= alpha * A * B^T (+ bias).  a_mn / b_mn: 0 = K-major ([rows][K], pitch ld), 1 = MN-major ([K][rows]).
// Requirements: all base pointers 16-byte aligned; lda, ldb multiples of 8 elements; N % 8 == 0; ldc % 8 == 0
// (bf16) or % 4 == 0 (fp32).  `err` is a device int that receives a nonzero code if a bounded wait ran out.
// bn: 0 = pick, else 128 or 256.  max_ctas limits the persistent grid (0 = all SMs).  ksplit > 1 needs fp32 accumulate.
extern "C" int b200_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                              long long lda, long long ldb, long long ldc, int a_mn, int b_mn, int flags, float alpha,
                              int bn, int max_ctas, int ksplit, int* err, cudaStream_t stream) {
  const void* a_parts[1] = {A};
  void* c_parts[1] = {C};
  return gemm_dispatch(a_parts, 1, 0, B, c_parts, 1, 0, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, flags, alpha, bn, max_ctas, ksplit, 0,
                       nullptr, 0, err, stream);
}

// Row-partitioned operands for the fused tensor-parallel kernels.
//   a_parts > 1 (all-gather -> GEMM): rows [i*a_part_rows, (i+1)*a_part_rows) of A are read from A_parts[i], which may
//     be another GPU's peer-mapped memory; before the first read of part i the kernel waits (bounded) until
//     ready_flags[i] >= ready_epoch.  A must be K-major.
//   c_parts > 1 (GEMM -> reduce-scatter): rows [i*c_part_rows, ...) of C are written to C_parts[i] with row index
//     relative to the part, i.e. straight into the owner rank's staging buffer over NVLink.
//   tile_rotate: first M tile in the processing order.
extern "C" int b200_gemm_bf16_parts(const void* const* A_parts, int a_parts, int a_part_rows, const void* B, void* const* C_parts,
                                    int c_parts, int c_part_rows, const void* bias, int M, int N, int K, long long lda,
                                    long long ldb, long long ldc, int a_mn, int b_mn, int flags, float alpha, int bn,
                                    int tile_rotate, const void* ready_flags, unsigned int ready_epoch, int* err,
                                    cudaStream_t stream) {
  return gemm_dispatch(A_parts, a_parts, a_part_rows, B, C_parts, c_parts, c_part_rows, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, flags,
                       alpha, bn, 0, 1, tile_rotate, static_cast<const uint32_t*>(ready_flags), ready_epoch, err, stream);
}

// All-gather -> GEMM in one kernel.  C[T, N] = gather_rows(X)[T, K] * B^T where every rank holds `x_local` [T/world, K].
//   x_local     this rank's shard (any device memory); its rows are read directly for the local tiles and pushed by the
//               kernel's copy warps into gather_ptrs[r] + rank * shard_bytes of every peer r (peer-mapped buffers);
//   gather_ptrs per-rank gather buffers [world][T/world, K] as mapped in this process; the local one is read by TMA
//               once the owner of each part has raised flag_ptrs[rank][slot][owner] to `epoch`;
//   counter     device uint32 (zero), used to find the last CTA.
// Tiles of the local rows are computed first, so the math starts while remote rows are still in flight.
static int ag_gemm_impl(const void* x_local, void* const* gather_ptrs, void* const* flag_ptrs, int rank, int world, int slot,
                        unsigned int epoch, const uint32_t* epoch_ptr, void* counter, const void* B, void* C, int T, int N, int K,
                        long long ldb, long long ldc, int b_mn, int* err, cudaStream_t stream) {
  using namespace b200;
  if (world < 1 || world > GEMM_MAX_PARTS || T % world) return -14;
  const int Tl = T / world;
  const long long shard_bytes = static_cast<long long>(Tl) * K * 2;
  if (shard_bytes % 16) return -10;
  GemmArgs cfg;
  cfg.ready_epoch_ptr = epoch_ptr;
  cfg.push_src = static_cast<const uint4*>(x_local);
  cfg.push_n16 = shard_bytes / 16;
  cfg.push_counter = static_cast<unsigned int*>(counter);
  cfg.push_rank = rank;
  cfg.push_world = world;
  const void* a_parts[GEMM_MAX_PARTS];
  for (int r = 0; r < GEMM_MAX_PARTS; ++r) { cfg.push_dst[r] = nullptr; cfg.push_flag[r] = nullptr; }
  for (int r = 0; r < world; ++r) {
    cfg.push_dst[r] = reinterpret_cast<uint4*>(static_cast<char*>(gather_ptrs[r]) + rank * shard_bytes);
    cfg.push_flag[r] = static_cast<uint32_t*>(flag_ptrs[r]) + slot * 8 + rank;
    // part r of A: own rows straight from x_local, other rows from the local gather buffer (filled by rank r's push)
    a_parts[r] = (r == rank) ? x_local : static_cast<const void*>(static_cast<char*>(gather_ptrs[rank]) + r * shard_bytes);
  }
  void* c_parts[1] = {C};
  const uint32_t* ready = static_cast<const uint32_t*>(flag_ptrs[rank]) + slot * 8;
  return gemm_dispatch(a_parts, world, Tl, B, c_parts, 1, 0, nullptr, T, N, K, K, ldb, ldc, 0, b_mn, 0, 1.0f, 0, 0, 1, rank * (Tl / GEMM_BM),
                       ready, epoch, err, stream, &cfg);
}
extern "C" int b200_ag_gemm_bf16(const void* x_local, void* const* gather_ptrs, void* const* flag_ptrs, int rank, int world, int slot,
                                 unsigned int epoch, void* counter, const void* B, void* C, int T, int N, int K, long long ldb,
                                 long long ldc, int b_mn, int* err, cudaStream_t stream) {
  return ag_gemm_impl(x_local, gather_ptrs, flag_ptrs, rank, world, slot, epoch, nullptr, counter, B, C, T, N, K, ldb, ldc, b_mn, err,
                      stream);
}
// Same, with the epoch read from device memory at run time (`epoch_ptr`, bumped by b200_epoch_bump earlier in the
// stream): the launch can be captured in a CUDA graph and replayed.
extern "C" int b200_ag_gemm_bf16_dev(const void* x_local, void* const* gather_ptrs, void* const* flag_ptrs, int rank, int world,
                                     int slot, const void* epoch_ptr, void* counter, const void* B, void* C, int T, int N, int K,
                                     long long ldb, long long ldc, int b_mn, int* err, cudaStream_t stream) {
  return ag_gemm_impl(x_local, gather_ptrs, flag_ptrs, rank, world, slot, 0, static_cast<const uint32_t*>(epoch_ptr), counter, B, C, T,
                      N, K, ldb, ldc, b_mn, err, stream);
}
