// Causal flash attention backward for sm_100a (bf16, head_dim 128, GQA native) on tcgen05 tensor cores.
//
// Inputs: the packed QKV projection [tokens, (Hq + 2 Hkv) * 128] the forward kernel read, its output O and
// log-sum-exp, and dO.  Output: the gradient of the packed projection in the same layout, so the QKV GEMM's
// backward consumes it without any concatenation.
//
// One CTA = one block of 128 keys of one (batch, query head); it walks the query blocks i >= j (causal) and runs
// five 128x128x128 products per step on the tensor core:
//     S  = Q K^T            -> TMEM X0        dP = dO V^T          -> TMEM X1
//     dV += P^T dO          -> TMEM (kept)    dK += dS^T Q         -> TMEM (kept)
//     dQ_i = dS K           -> TMEM X1, drained into an fp32 buffer with TMA reduce-add (other key blocks add theirs)
// with P = exp2(S * c - LSE) and dS = P (dP - Delta) computed by eight warps (thread = half a query row) and
// handed to the tensor core as bf16 through 128B-swizzled shared memory.  dK / dV of the query heads that share a KV head are
// summed the same way (fp32 reduce-add), and a last pass applies the softmax scale and rounds the buffer to bf16.
// Roles (320 threads): warp 0 TMA producer (K, V once; Q double-buffered, dO single), warp 1 MMA issuer, warps 2-9
// softmax / gradient warps (two per TMEM lane quadrant, each owning 64 of the 128 columns of its rows).  S_{t+1} is
// issued while dQ_t drains, and the P half of the softmax runs while dO_{t+1} is still in flight, so loads are off the
// critical path.
// Every mbarrier wait is bounded; a timeout sets the device status word and the CTA leaves through the common exit
// that frees its TMEM.
// Replaces the backward of torch SDPA / flash_attn_2_cuda used by the reference
// (gpt-neox/megatron/model/flash_attention.py:468-786).
#include "sm100_common.cuh"
#include <math_constants.h>

namespace b200 {

constexpr int FB_T = 128;                        // tile edge: query rows, keys and head_dim
constexpr int FB_THREADS = 320;                  // TMA warp, MMA warp, eight softmax / gradient warps
constexpr int FB_TILE_BYTES = FB_T * FB_T * 2;   // 32 KB bf16 tile = two 64-column halves
constexpr int FB_HALF_BYTES = FB_TILE_BYTES / 2;

struct FlashBwdArgs {
  const float* lse;     // [B, Hq, S] natural log
  const float* delta;   // [B, Hq, S] rowsum(dO * O)
  int B, S, Hq, Hkv;
  float scale, scale_log2;
  int causal;
  int* err;
};

struct FlashBwdSmem {
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = K_OFF + FB_TILE_BYTES;
  static constexpr int Q_OFF = V_OFF + FB_TILE_BYTES;        // two buffers
  static constexpr int DO_OFF = Q_OFF + 2 * FB_TILE_BYTES;
  static constexpr int P_OFF = DO_OFF + FB_TILE_BYTES;
  static constexpr int DS_OFF = P_OFF + FB_TILE_BYTES;       // also the fp32 staging of the reduce-add epilogues
  static constexpr int BAR_OFF = DS_OFF + FB_TILE_BYTES;     // 224 KB
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

// 32 rows x 32 fp32 columns of a TMEM accumulator -> swizzled 4 KB staging -> TMA reduce-add at (x, y).
// `stage` is the warp's own 4 KB; `n_issued` counts this warp's bulk groups.
__device__ __forceinline__ void drain_chunk_reduce(uint32_t taddr, uint8_t* stage, int lane, const CUtensorMap* tm, int x, int y,
                                                   int& n_issued) {
  uint32_t v[32];
  tmem_ld_32x32(taddr, v);
  tmem_ld_wait();
  if (n_issued > 0) {  // the previous reduce-add has read the staging buffer
    if (lane == 0) tma_store_wait_read<0>();
    __syncwarp();
  }
  const int sw = lane & 7;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    *reinterpret_cast<uint4*>(stage + lane * 128 + ((j ^ sw) << 4)) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    tma_reduce_add_2d(tm, stage, x, y);
    tma_store_commit();
  }
  ++n_issued;
}

__global__ void __launch_bounds__(FB_THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO,
                 const __grid_constant__ CUtensorMap tmAcc, FlashBwdArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FlashBwdSmem::BAR_OFF);
  uint64_t* kv_full = bars;          // 1
  uint64_t* q_full = bars + 1;       // 2
  uint64_t* q_empty = bars + 3;      // 2
  uint64_t* do_full = bars + 5;      // 1
  uint64_t* do_empty = bars + 6;     // 1
  uint64_t* s_full = bars + 7;       // 1
  uint64_t* dp_full = bars + 8;      // 1
  uint64_t* ds_done = bars + 9;      // 1 (count 8)
  uint64_t* dq_full = bars + 10;     // 1
  uint64_t* x1_free = bars + 11;     // 1 (count 8)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  __shared__ int cta_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_blk = (p.S + FB_T - 1) / FB_T;
  const int jblk = blockIdx.x;                  // key block; block 0 has the most query blocks and starts first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kvh = head / (p.Hq / p.Hkv);
  const int i_start = p.causal ? jblk : 0;
  const int T = n_blk - i_start;                // query blocks this CTA visits
  const int row_base = batch * p.S;
  const int kv0 = jblk * FB_T;
  const int xq = head * FB_T;
  const int xk = (p.Hq + kvh) * FB_T;
  const int xv = (p.Hq + p.Hkv + kvh) * FB_T;

  if (threadIdx.x == 0) {
    cta_abort = 0;
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); }
    mbar_init(do_full, 1); mbar_init(do_empty, 1);
    mbar_init(s_full, 1); mbar_init(dp_full, 1);
    mbar_init(ds_done, 8); mbar_init(dq_full, 1); mbar_init(x1_free, 8);
    fence_barrier_init();
    prefetch_tmap(&tmQKV); prefetch_tmap(&tmDO); prefetch_tmap(&tmAcc);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tX0 = tmem_base, tX1 = tmem_base + 128, tDK = tmem_base + 256, tDV = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      uint8_t* sK = smem + FlashBwdSmem::K_OFF;
      uint8_t* sV = smem + FlashBwdSmem::V_OFF;
      mbar_expect_tx(kv_full, 2 * FB_TILE_BYTES);
      tma_load_2d(sK, &tmQKV, kv_full, xk, row_base + kv0);
      tma_load_2d(sK + FB_HALF_BYTES, &tmQKV, kv_full, xk + 64, row_base + kv0);
      tma_load_2d(sV, &tmQKV, kv_full, xv, row_base + kv0);
      tma_load_2d(sV + FB_HALF_BYTES, &tmQKV, kv_full, xv + 64, row_base + kv0);
      for (int t = 0; t < T; ++t) {
        const int b = t & 1;
        const int qrow = row_base + (i_start + t) * FB_T;
        uint8_t* sQ = smem + FlashBwdSmem::Q_OFF + b * FB_TILE_BYTES;
        uint8_t* sDO = smem + FlashBwdSmem::DO_OFF;
        if (!mbar_wait(&q_empty[b], ((t >> 1) & 1) ^ 1, p.err, ERR_WAIT_EMPTY, &cta_abort)) break;
        mbar_expect_tx(&q_full[b], FB_TILE_BYTES);
        tma_load_2d(sQ, &tmQKV, &q_full[b], xq, qrow);
        tma_load_2d(sQ + FB_HALF_BYTES, &tmQKV, &q_full[b], xq + 64, qrow);
        if (!mbar_wait(do_empty, (t & 1) ^ 1, p.err, ERR_WAIT_EMPTY, &cta_abort)) break;
        mbar_expect_tx(do_full, FB_TILE_BYTES);
        tma_load_2d(sDO, &tmDO, do_full, xq, qrow);
        tma_load_2d(sDO + FB_HALF_BYTES, &tmDO, do_full, xq + 64, qrow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_kk = make_idesc_bf16(FB_T, FB_T, 0, 0);   // both operands K-major (S, dP)
      const uint32_t idesc_mm = make_idesc_bf16(FB_T, FB_T, 1, 1);   // both MN-major (dV, dK)
      const uint32_t idesc_km = make_idesc_bf16(FB_T, FB_T, 0, 1);   // A K-major, B MN-major (dQ)
      const uint32_t k_base = smem_u32(smem + FlashBwdSmem::K_OFF);
      const uint32_t v_base = smem_u32(smem + FlashBwdSmem::V_OFF);
      const uint32_t do_base = smem_u32(smem + FlashBwdSmem::DO_OFF);
      const uint32_t p_base = smem_u32(smem + FlashBwdSmem::P_OFF);
      const uint32_t ds_base = smem_u32(smem + FlashBwdSmem::DS_OFF);
      auto issue_s = [&](int t) -> bool {
        const int b = t & 1;
        if (!mbar_wait(&q_full[b], (t >> 1) & 1, p.err, ERR_WAIT_FULL, &cta_abort)) return false;
        tc_fence_after_sync();
        const uint32_t q_base = smem_u32(smem + FlashBwdSmem::Q_OFF + b * FB_TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < FB_T / 16; ++ks) {
          const uint32_t off = (ks >> 2) * FB_HALF_BYTES + (ks & 3) * 32;
          umma_bf16_ss(tX0, make_smem_desc_sw128(q_base + off, 16, 1024), make_smem_desc_sw128(k_base + off, 16, 1024), idesc_kk,
                       ks != 0);
        }
        umma_commit(s_full);
        return true;
      };
      bool ok = T > 0 && mbar_wait(kv_full, 0, p.err, ERR_WAIT_FULL, &cta_abort);
      if (ok) ok = issue_s(0);
      for (int t = 0; t < T && ok; ++t) {
        const int b = t & 1;
        const uint32_t ph = t & 1;
        const uint32_t q_base = smem_u32(smem + FlashBwdSmem::Q_OFF + b * FB_TILE_BYTES);
        if (!mbar_wait(do_full, ph, p.err, ERR_WAIT_FULL, &cta_abort)) { ok = false; break; }
        if (t > 0 && !mbar_wait(x1_free, (t - 1) & 1, p.err, ERR_WAIT_TMEM_EMPTY, &cta_abort)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < FB_T / 16; ++ks) {   // dP = dO V^T
          const uint32_t off = (ks >> 2) * FB_HALF_BYTES + (ks & 3) * 32;
          umma_bf16_ss(tX1, make_smem_desc_sw128(do_base + off, 16, 1024), make_smem_desc_sw128(v_base + off, 16, 1024), idesc_kk,
                       ks != 0);
        }
        umma_commit(dp_full);
        if (!mbar_wait(ds_done, ph, p.err, ERR_WAIT_TMEM_FULL, &cta_abort)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < FB_T / 16; ++ks) {   // dQ_t = dS K   (contraction over the 128 keys)
          umma_bf16_ss(tX1, make_smem_desc_sw128(ds_base + (ks >> 2) * FB_HALF_BYTES + (ks & 3) * 32, 16, 1024),
                       make_smem_desc_sw128(k_base + ks * 2048, FB_HALF_BYTES, 1024), idesc_km, ks != 0);
        }
#pragma unroll
        for (int ks = 0; ks < FB_T / 16; ++ks) {   // dK += dS^T Q   (contraction over the 128 query rows)
          umma_bf16_ss(tDK, make_smem_desc_sw128(ds_base + ks * 2048, FB_HALF_BYTES, 1024),
                       make_smem_desc_sw128(q_base + ks * 2048, FB_HALF_BYTES, 1024), idesc_mm, (t | ks) != 0);
        }
        umma_commit(dq_full);                      // dQ_t is in X1 and nothing reads the dS tile any more
#pragma unroll
        for (int ks = 0; ks < FB_T / 16; ++ks) {   // dV += P^T dO
          umma_bf16_ss(tDV, make_smem_desc_sw128(p_base + ks * 2048, FB_HALF_BYTES, 1024),
                       make_smem_desc_sw128(do_base + ks * 2048, FB_HALF_BYTES, 1024), idesc_mm, (t | ks) != 0);
        }
        umma_commit(&q_empty[b]);
        umma_commit(do_empty);
        if (t + 1 == T) umma_commit(s_full);       // phase T: every product of this CTA has completed
        if (t + 1 < T) ok = issue_s(t + 1);   // X0 is free (S_t was read before ds_done); its commit also covers dV_t
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------ softmax / gradient warps
    // Two warps per TMEM lane quadrant: the warp of group `wg` owns key columns [64 wg, 64 wg + 64) of its 32 query
    // rows in P / dS (and head-dim columns [64 wg, 64 wg + 64) of dQ, dK, dV), so the pair never has to talk.
    const int quad = warp & 3;
    const int wg = (warp - 2) >> 2;
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int sw = r & 7;
    const int colbase = wg * 64;
    uint8_t* prow = smem + FlashBwdSmem::P_OFF + wg * FB_HALF_BYTES + r * 128;
    uint8_t* dsrow = smem + FlashBwdSmem::DS_OFF + wg * FB_HALF_BYTES + r * 128;
    // this warp's 32 rows x 64 columns of the dS tile double as its 4 KB reduce-add staging buffer: dQ_t is drained
    // after the products that read dS_t (dQ_t, dK_t) have completed, while dV_t and S_{t+1} still run
    uint8_t* stage = smem + FlashBwdSmem::DS_OFF + wg * FB_HALF_BYTES + quad * 4096;
    int n_issued = 0;
    bool ok = true;
    const long long stat0 = (static_cast<long long>(batch) * p.Hq + head) * p.S;
    float lse_next = 0.f, delta_next = 0.f;
    if (i_start * FB_T + r < p.S) {
      lse_next = p.lse[stat0 + i_start * FB_T + r];
      delta_next = p.delta[stat0 + i_start * FB_T + r];
    }
    for (int t = 0; t < T; ++t) {
      const uint32_t ph = t & 1;
      const int q0 = (i_start + t) * FB_T;
      const int qi = q0 + r;
      const bool row_ok = qi < p.S;
      const float lse2 = lse_next * 1.4426950408889634f;
      const float delta = delta_next;
      if (t + 1 < T && qi + FB_T < p.S) {   // the next block's row statistics arrive while this block is processed
        lse_next = p.lse[stat0 + qi + FB_T];
        delta_next = p.delta[stat0 + qi + FB_T];
      }
      const bool need_mask = (p.causal && kv0 + FB_T > q0) || (kv0 + FB_T > p.S) || (q0 + FB_T > p.S);
      ok = mbar_wait(s_full, ph, p.err, ERR_WAIT_TMEM_FULL, &cta_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      // ---- P = exp2(S * c - LSE): kept in registers for dS, bf16 copy into the swizzled tile for dV
      uint32_t v0[32], v1[32];
      tmem_ld_32x32(tX0 + lane_addr + colbase, v0);
      tmem_ld_32x32(tX0 + lane_addr + colbase + 32, v1);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float s0 = fmaf(__uint_as_float(v0[i]), p.scale_log2, -lse2);
        float s1 = fmaf(__uint_as_float(v1[i]), p.scale_log2, -lse2);
        if (need_mask) {
          const int k0 = kv0 + colbase + i, k1 = k0 + 32;
          if (!row_ok || k0 >= p.S || (p.causal && k0 > qi)) s0 = -CUDART_INF_F;
          if (!row_ok || k1 >= p.S || (p.causal && k1 > qi)) s1 = -CUDART_INF_F;
        }
        v0[i] = __float_as_uint(exp2f(s0));
        v1[i] = __float_as_uint(exp2f(s1));
      }
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 o;
        o.x = pack_bf16x2(__uint_as_float(v0[8 * g]), __uint_as_float(v0[8 * g + 1]));
        o.y = pack_bf16x2(__uint_as_float(v0[8 * g + 2]), __uint_as_float(v0[8 * g + 3]));
        o.z = pack_bf16x2(__uint_as_float(v0[8 * g + 4]), __uint_as_float(v0[8 * g + 5]));
        o.w = pack_bf16x2(__uint_as_float(v0[8 * g + 6]), __uint_as_float(v0[8 * g + 7]));
        *reinterpret_cast<uint4*>(prow + ((g ^ sw) << 4)) = o;
        o.x = pack_bf16x2(__uint_as_float(v1[8 * g]), __uint_as_float(v1[8 * g + 1]));
        o.y = pack_bf16x2(__uint_as_float(v1[8 * g + 2]), __uint_as_float(v1[8 * g + 3]));
        o.z = pack_bf16x2(__uint_as_float(v1[8 * g + 4]), __uint_as_float(v1[8 * g + 5]));
        o.w = pack_bf16x2(__uint_as_float(v1[8 * g + 6]), __uint_as_float(v1[8 * g + 7]));
        *reinterpret_cast<uint4*>(prow + (((4 + g) ^ sw) << 4)) = o;
      }
      ok = mbar_wait(dp_full, ph, p.err, ERR_WAIT_TMEM_FULL, &cta_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      if (n_issued > 0) {   // my dS rows are the staging buffer my last reduce-add reads from
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
      }
      // ---- dS = P (dP - Delta); the softmax scale is applied when the fp32 sums are rounded
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t d[32];
        tmem_ld_32x32(tX1 + lane_addr + colbase + c * 32, d);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t ow[4];
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const int i = 8 * g + 2 * w;
            const float p0 = __uint_as_float(c ? v1[i] : v0[i]), p1 = __uint_as_float(c ? v1[i + 1] : v0[i + 1]);
            ow[w] = pack_bf16x2((__uint_as_float(d[i]) - delta) * p0, (__uint_as_float(d[i + 1]) - delta) * p1);
          }
          *reinterpret_cast<uint4*>(dsrow + (((c * 4 + g) ^ sw) << 4)) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_done);
      // ---- drain my half of dQ_t (the products that read dS_t have completed when dq_full flips)
      ok = mbar_wait(dq_full, ph, p.err, ERR_WAIT_TMEM_FULL, &cta_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
#pragma unroll 1
      for (int c = 0; c < 2; ++c)
        drain_chunk_reduce(tX1 + lane_addr + colbase + c * 32, stage, lane, &tmAcc, xq + colbase + c * 32, row_base + q0 + quad * 32,
                           n_issued);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(x1_free);
    }
    // ---- dK, dV of this (key block, query head): summed over the query heads of the group in the fp32 buffer
    if (ok && T > 0) {
      ok = mbar_wait(s_full, T & 1, p.err, ERR_WAIT_TMEM_FULL, &cta_abort);   // the last dV product has completed
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && T > 0) {
      tc_fence_after_sync();
#pragma unroll 1
      for (int c = 0; c < 2; ++c)
        drain_chunk_reduce(tDK + lane_addr + colbase + c * 32, stage, lane, &tmAcc, xk + colbase + c * 32, row_base + kv0 + quad * 32,
                           n_issued);
#pragma unroll 1
      for (int c = 0; c < 2; ++c)
        drain_chunk_reduce(tDV + lane_addr + colbase + c * 32, stage, lane, &tmAcc, xv + colbase + c * 32, row_base + kv0 + quad * 32,
                           n_issued);
    }
    if (lane == 0) tma_store_wait<0>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b, h, s] = sum_d dO * O ; one warp per (token, head)
__global__ void flash_bwd_delta_kernel(const __nv_bfloat16* __restrict__ o, long long o_stride, const __nv_bfloat16* __restrict__ dout,
                                       long long do_stride, float* __restrict__ delta, int B, int S, int Hq) {
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(B) * S * Hq;
  if (w >= total) return;
  const long long tok = w / Hq;
  const int h = static_cast<int>(w % Hq);
  const uint2 a = *reinterpret_cast<const uint2*>(o + tok * o_stride + h * FB_T + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(dout + tok * do_stride + h * FB_T + lane * 4);
  float acc = __uint_as_float(a.x << 16) * __uint_as_float(b.x << 16) + __uint_as_float(a.x & 0xffff0000u) * __uint_as_float(b.x & 0xffff0000u) +
              __uint_as_float(a.y << 16) * __uint_as_float(b.y << 16) + __uint_as_float(a.y & 0xffff0000u) * __uint_as_float(b.y & 0xffff0000u);
#pragma unroll
  for (int off = 16; off; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    const long long bi = tok / S, si = tok % S;
    delta[(bi * Hq + h) * S + si] = acc;
  }
}

// fp32 sums -> bf16; the q and k gradients (the first `scaled4` float4 of every row) take the softmax scale here
__global__ void flash_bwd_round_kernel(const float4* __restrict__ acc, uint2* __restrict__ out, long long n4, int row4, int scaled4,
                                       float scale) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = acc[i];
    const float f = static_cast<int>(i % row4) < scaled4 ? scale : 1.f;
    out[i] = make_uint2(pack_bf16x2(v.x * f, v.y * f), pack_bf16x2(v.z * f, v.w * f));
  }
}

int make_tmap_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                 uint32_t box_outer, bool f32);

}  // namespace b200

using namespace b200;

// qkv:  [B*S, row_stride] bf16 (q heads, k heads, v heads per row; head_dim 128)      out / dout: [B*S, *_stride] bf16
// lse:  [B, Hq, S] fp32 from the forward kernel                                       delta: [B, Hq, S] fp32 scratch
// acc:  [B*S, (Hq + 2 Hkv) * 128] fp32 scratch (zeroed here)                          dqkv:  same shape, bf16, contiguous
extern "C" int b200_flash_bwd(const void* qkv, long long row_stride, const void* out, long long out_stride, const void* dout,
                              long long dout_stride, const float* lse, float* delta, float* acc, void* dqkv, int B, int S, int Hq,
                              int Hkv, int head_dim, float scale, int causal, int* err, cudaStream_t stream) {
  if (head_dim != FB_T || Hq % Hkv || row_stride % 8 || out_stride % 8 || dout_stride % 8) return -10;
  if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(dout) |
       reinterpret_cast<uintptr_t>(acc) | reinterpret_cast<uintptr_t>(dqkv)) & 15)
    return -11;
  if (B <= 0 || S <= 0) return 0;
  const long long tokens = static_cast<long long>(B) * S;
  const long long width = static_cast<long long>(Hq + 2 * Hkv) * FB_T;
  CUtensorMap tmQKV, tmDO, tmAcc;
  int rc = make_tmap_2d(&tmQKV, qkv, static_cast<uint64_t>(width), static_cast<uint64_t>(tokens), row_stride, 64, FB_T, false);
  if (!rc) rc = make_tmap_2d(&tmDO, dout, static_cast<uint64_t>(Hq) * FB_T, static_cast<uint64_t>(tokens), dout_stride, 64, FB_T, false);
  if (!rc) rc = make_tmap_2d(&tmAcc, acc, static_cast<uint64_t>(width), static_cast<uint64_t>(tokens), width, 32, 32, true);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FlashBwdSmem::TOTAL) != cudaSuccess) return -3;
    attr_set = true;
  }
  if (cudaMemsetAsync(acc, 0, static_cast<size_t>(tokens * width) * sizeof(float), stream) != cudaSuccess) return -4;
  {
    const long long warps = tokens * Hq;
    const int threads = 256;
    const long long blocks = (warps * 32 + threads - 1) / threads;
    flash_bwd_delta_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(out), out_stride, static_cast<const __nv_bfloat16*>(dout), dout_stride, delta, B, S, Hq);
  }
  FlashBwdArgs a;
  a.lse = lse; a.delta = delta;
  a.B = B; a.S = S; a.Hq = Hq; a.Hkv = Hkv;
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = causal;
  a.err = err;
  dim3 grid((S + FB_T - 1) / FB_T, Hq, B);
  flash_bwd_kernel<<<grid, FB_THREADS, FlashBwdSmem::TOTAL, stream>>>(tmQKV, tmDO, tmAcc, a);
  const long long n4 = tokens * width / 4;
  long long blocks = (n4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  flash_bwd_round_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(reinterpret_cast<const float4*>(acc),
                                                                            reinterpret_cast<uint2*>(dqkv), n4, static_cast<int>(width / 4),
                                                                            (Hq + Hkv) * FB_T / 4, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
