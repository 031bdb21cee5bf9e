// Causal flash attention forward for sm_100a (bf16, head_dim 128, GQA native) on tcgen05 tensor cores.
//
// Reads q, k, v straight out of the packed QKV projection [tokens, (Hq + 2 Hkv) * 128] through ONE tiled TMA
// descriptor (box 64 x 128, 128-byte swizzle), so there is no transpose, no repeat_kv and no padding copy.
// One CTA = 128 query rows of one (batch, head).  Roles (320 threads):
//   warp 0      TMA producer: Q once, then K_j / V_j tiles of 128 keys into two-deep rings;
//   warp 1      MMA issuer:  S_j = Q K_j^T  (SS MMA, 128x128x16 x8)  into one of two TMEM score buffers,
//               then O += P_j V_j with P_j read from shared memory; S_{j+1} is issued before P_j V_j so the
//               tensor core works on the next scores while the softmax warps are busy;
//   warps 2-9   softmax: two warps per TMEM lane quadrant, each thread owns 64 of its query row's 128 scores
//               (tcgen05.ld into registers once), the pair exchanges row maxima through shared memory, online
//               softmax in the log2 domain, P_j is written as bf16 into a 128B-swizzled K-major tile (double
//               buffered), and the
//               accumulator O in TMEM is rescaled only when the running max moved by more than 2^8 (the stale
//               max keeps exp2 arguments small; the final 1/l normalisation makes it exact).
// Output: O [tokens, Hq * 128] bf16 and the log-sum-exp per (batch, head, row) for the backward pass.
// Replaces torch SDPA / flash_attn_2_cuda of the reference (opt_prime traced graphs call
// F.scaled_dot_product_attention; gpt-neox/megatron/model/flash_attention.py:468-786).
#include "sm100_common.cuh"
#include <math_constants.h>

namespace b200 {

constexpr int FA_BM = 128;   // query rows per CTA
constexpr int FA_BN = 128;   // keys per tile
constexpr int FA_D = 128;
constexpr int FA_THREADS = 320;         // TMA warp, MMA warp, eight softmax warps
constexpr int FA_TILE_BYTES = FA_BM * FA_D * 2;       // 32 KB: two 64-column halves of 16 KB
constexpr int FA_HALF_BYTES = FA_TILE_BYTES / 2;
constexpr float FA_RESCALE_THRESHOLD = 8.0f;          // log2 units

struct FlashArgs {
  __nv_bfloat16* out;     // [tokens, Hq*D]
  float* lse;             // [B, Hq, S] natural-log LSE (may be null)
  int B, S, Hq, Hkv;
  long long out_stride;
  float scale_log2;       // softmax scale * log2(e)
  int causal;
  int* err;
};

struct FlashSmem {
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + FA_TILE_BYTES;
  static constexpr int V_OFF = K_OFF + 2 * FA_TILE_BYTES;
  static constexpr int P_OFF = V_OFF + 2 * FA_TILE_BYTES;
  static constexpr int BAR_OFF = P_OFF + 2 * FA_TILE_BYTES;
  static constexpr int XCHG_OFF = BAR_OFF + 256;              // 4 x 128 floats: half-row maxima / sums [2 parities][2 groups]
  static constexpr int TOTAL = XCHG_OFF + 4 * FA_BM * 4;      // 231,680 B: the dynamic window itself is 1024-byte aligned
};

__global__ void __launch_bounds__(FA_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQKV, FlashArgs p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {  // the swizzled tiles need 1024-byte alignment; no static shared memory precedes the window
    if (threadIdx.x == 0) atomicCAS(p.err, 0, ERR_BAD_ALIGNMENT);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FlashSmem::BAR_OFF);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // 2
  uint64_t* k_empty = bars + 3;       // 2
  uint64_t* v_full = bars + 5;        // 2
  uint64_t* v_empty = bars + 7;       // 2
  uint64_t* s_full = bars + 9;        // 2
  uint64_t* s_empty = bars + 11;      // 2 (count 4: one arrive per softmax warp)
  uint64_t* p_full = bars + 13;       // 2 (count 4)
  uint64_t* p_empty = bars + 15;      // 2 (PV MMA that read P buffer b has completed)
  uint64_t* o_done = bars + 17;       // 1
  uint64_t* pair_bar = bars + 18;     // 4 (count 64: the two warps that share a TMEM lane quadrant)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 22);
  volatile int& cta_abort = *reinterpret_cast<volatile int*>(bars + 23);
  float* xchg = reinterpret_cast<float*>(smem + FlashSmem::XCHG_OFF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qblk = (p.S + FA_BM - 1) / FA_BM;
  const int qblk = n_qblk - 1 - blockIdx.x;  // heavy (late) blocks first under the causal mask
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kvh = head / (p.Hq / p.Hkv);
  const int q0 = qblk * FA_BM;
  const int kv_end = p.causal ? min(p.S, q0 + FA_BM) : p.S;
  const int n_kv = (kv_end + FA_BN - 1) / FA_BN;
  const int row_base = batch * p.S;  // token row of this batch in the packed matrix
  const int xq = head * FA_D;
  const int xk = (p.Hq + kvh) * FA_D;
  const int xv = (p.Hq + p.Hkv + kvh) * FA_D;

  if (threadIdx.x == 0) {
    cta_abort = 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 8);
      mbar_init(&p_full[i], 8); mbar_init(&p_empty[i], 1);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&pair_bar[i], 64);
    mbar_init(o_done, 1);
    fence_barrier_init();
    prefetch_tmap(&tmQKV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S0 = tmem_base;           // two score buffers: columns [0,128) and [128,256)
  const uint32_t tmem_O = tmem_base + 256;      // output accumulator: columns [256,384)

  if (warp == 0) {
    if (lane == 0) {
      uint8_t* sQ = smem + FlashSmem::Q_OFF;
      mbar_expect_tx(q_full, FA_TILE_BYTES);
      tma_load_2d(sQ, &tmQKV, q_full, xq, row_base + q0);
      tma_load_2d(sQ + FA_HALF_BYTES, &tmQKV, q_full, xq + 64, row_base + q0);
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int b = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        uint8_t* sK = smem + FlashSmem::K_OFF + b * FA_TILE_BYTES;
        uint8_t* sV = smem + FlashSmem::V_OFF + b * FA_TILE_BYTES;
        if (!mbar_wait(&k_empty[b], ph, p.err, ERR_WAIT_EMPTY, &cta_abort)) { ok = false; break; }
        mbar_expect_tx(&k_full[b], FA_TILE_BYTES);
        tma_load_2d(sK, &tmQKV, &k_full[b], xk, row_base + j * FA_BN);
        tma_load_2d(sK + FA_HALF_BYTES, &tmQKV, &k_full[b], xk + 64, row_base + j * FA_BN);
        if (!mbar_wait(&v_empty[b], ph, p.err, ERR_WAIT_EMPTY, &cta_abort)) { ok = false; break; }
        mbar_expect_tx(&v_full[b], FA_TILE_BYTES);
        tma_load_2d(sV, &tmQKV, &v_full[b], xv, row_base + j * FA_BN);
        tma_load_2d(sV + FA_HALF_BYTES, &tmQKV, &v_full[b], xv + 64, row_base + j * FA_BN);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc_bf16(FA_BM, FA_BN, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(FA_BM, FA_D, 0, 1);
      const uint32_t q_base = smem_u32(smem + FlashSmem::Q_OFF);
      bool ok = mbar_wait(q_full, 0, p.err, ERR_WAIT_FULL, &cta_abort);
      auto issue_pv = [&](int i) -> bool {
        const int b = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(&v_full[b], ph, p.err, ERR_WAIT_FULL, &cta_abort)) return false;
        if (!mbar_wait(&p_full[b], ph, p.err, ERR_WAIT_TMEM_FULL, &cta_abort)) return false;
        tc_fence_after_sync();
        const uint32_t p_base = smem_u32(smem + FlashSmem::P_OFF + b * FA_TILE_BYTES);
        const uint32_t v_base = smem_u32(smem + FlashSmem::V_OFF + b * FA_TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < FA_BN / 16; ++ks) {
          const uint64_t adesc = make_smem_desc_sw128(p_base + (ks >> 2) * FA_HALF_BYTES + (ks & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(v_base + ks * 2048, FA_HALF_BYTES, 1024);
          umma_bf16_ss(tmem_O, adesc, bdesc, idesc_pv, (i | ks) != 0);
        }
        umma_commit(&v_empty[b]);
        umma_commit(&p_empty[b]);
        return true;
      };
      for (int j = 0; j < n_kv && ok; ++j) {
        const int b = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[b], ph, p.err, ERR_WAIT_FULL, &cta_abort)) { ok = false; break; }
        if (!mbar_wait(&s_empty[b], ph ^ 1, p.err, ERR_WAIT_TMEM_EMPTY, &cta_abort)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t k_base = smem_u32(smem + FlashSmem::K_OFF + b * FA_TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < FA_D / 16; ++ks) {
          const uint32_t off = (ks >> 2) * FA_HALF_BYTES + (ks & 3) * 32;
          umma_bf16_ss(tmem_S0 + b * FA_BN, make_smem_desc_sw128(q_base + off, 16, 1024),
                       make_smem_desc_sw128(k_base + off, 16, 1024), idesc_qk, ks != 0);
        }
        umma_commit(&s_full[b]);
        umma_commit(&k_empty[b]);
        if (j > 0) ok = issue_pv(j - 1);
      }
      if (ok && n_kv > 0) ok = issue_pv(n_kv - 1);
      if (ok) umma_commit(o_done);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------ softmax / correction / epilogue
    // Two warps per TMEM lane quadrant (so every scheduler has two softmax warps to switch between): the warp of
    // group `wg` owns columns [64 wg, 64 wg + 64) of each of its 32 query rows.  The pair exchanges the row maximum
    // (and, at the end, the row sum) through shared memory, synchronised by a bounded mbarrier wait.
    const int quad = warp & 3;
    const int wg = (warp - 2) >> 2;
    const int r = quad * 32 + lane;          // row inside the tile
    const int qi = q0 + r;                   // query position inside the sequence
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int sw = r & 7;
    const int colbase = wg * 64;
    float m_used = -CUDART_INF_F;            // max used for the exponentials so far (log2 domain)
    float l = 0.f;                           // sum over this warp's columns only
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int b = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      ok = mbar_wait(&s_full[b], ph, p.err, ERR_WAIT_TMEM_FULL, &cta_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t tS = tmem_S0 + b * FA_BN + lane_addr + colbase;
      const int kv0 = j * FA_BN + colbase;
      const bool need_mask = (p.causal && j * FA_BN + FA_BN > q0) || (j * FA_BN + FA_BN > p.S);
      uint32_t v0[32], v1[32];
      tmem_ld_32x32(tS, v0);
      tmem_ld_32x32(tS + 32, v1);
      tmem_ld_wait();
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int k0 = kv0 + i, k1 = kv0 + 32 + i;
          if (k0 >= p.S || (p.causal && k0 > qi)) v0[i] = 0xff800000u;
          if (k1 >= p.S || (p.causal && k1 > qi)) v1[i] = 0xff800000u;
        }
      }
      float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
      for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], fmaxf(__uint_as_float(v0[i]), __uint_as_float(v1[i])));
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // exchange the half-row maxima
      xchg[(b * 2 + wg) * FA_BM + r] = mx;
      mbar_arrive(&pair_bar[quad]);
      ok = mbar_wait(&pair_bar[quad], j & 1, p.err, ERR_WAIT_FULL, &cta_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      mx = fmaxf(mx, xchg[(b * 2 + (wg ^ 1)) * FA_BM + r]);
      const float m_cand = mx * p.scale_log2;
      float m_new = m_used;
      bool rescale = false;
      if (m_cand > m_used + FA_RESCALE_THRESHOLD || m_used == -CUDART_INF_F) {
        m_new = fmaxf(m_cand, m_used);
        rescale = (m_used != -CUDART_INF_F);
      }
      // the P buffer of this parity was last read by PV_{j-2}
      if (j >= 2) {
        ok = mbar_wait(&p_empty[b], ((j - 2) >> 1) & 1, p.err, ERR_WAIT_TMEM_EMPTY, &cta_abort);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      if (__any_sync(0xffffffffu, rescale)) {
        // O is complete up to PV_{j-1} only after that MMA has finished
        ok = mbar_wait(&p_empty[(j - 1) & 1], ((j - 1) >> 1) & 1, p.err, ERR_WAIT_TMEM_EMPTY, &cta_abort);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        const float alpha = rescale ? exp2f(m_used - m_new) : 1.f;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_O + lane_addr + colbase + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x32(tmem_O + lane_addr + colbase + c * 32, v);
        }
        tmem_st_wait();
        l *= alpha;
      }
      m_used = m_new;
      const float msub = (m_used == -CUDART_INF_F) ? 0.f : m_used;
      // exponentials, row sum, bf16 P into this group's 64-column half of the swizzled K-major tile
      uint8_t* prow = smem + FlashSmem::P_OFF + b * FA_TILE_BYTES + wg * FA_HALF_BYTES + r * 128;
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float e0 = exp2f(fmaf(__uint_as_float(v0[i]), p.scale_log2, -msub));
        const float e1 = exp2f(fmaf(__uint_as_float(v1[i]), p.scale_log2, -msub));
        rs4[i & 3] += e0 + e1;
        v0[i] = __float_as_uint(e0);
        v1[i] = __float_as_uint(e1);
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
      l += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[b]);
        mbar_arrive(&p_full[b]);
      }
    }
    // ------------------------------------------------ epilogue
    if (ok && n_kv > 0) {
      ok = mbar_wait(o_done, 0, p.err, ERR_WAIT_TMEM_FULL, &cta_abort);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {   // total row sum = the pair's two partial sums
      const int fb = n_kv & 1;  // the maxima slots of this parity were last read two tiles ago
      xchg[(fb * 2 + wg) * FA_BM + r] = l;
      mbar_arrive(&pair_bar[quad]);
      ok = mbar_wait(&pair_bar[quad], n_kv & 1, p.err, ERR_WAIT_FULL, &cta_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) l += xchg[((n_kv & 1) * 2 + (wg ^ 1)) * FA_BM + r];
    }
    if (ok) {
      tc_fence_after_sync();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = qi < p.S;
      __nv_bfloat16* dst = p.out + static_cast<long long>(row_base + qi) * p.out_stride + head * FA_D + colbase;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        if (n_kv > 0) {
          tmem_ld_32x32(tmem_O + lane_addr + colbase + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[8 * g]) * inv_l, __uint_as_float(v[8 * g + 1]) * inv_l);
            o.y = pack_bf16x2(__uint_as_float(v[8 * g + 2]) * inv_l, __uint_as_float(v[8 * g + 3]) * inv_l);
            o.z = pack_bf16x2(__uint_as_float(v[8 * g + 4]) * inv_l, __uint_as_float(v[8 * g + 5]) * inv_l);
            o.w = pack_bf16x2(__uint_as_float(v[8 * g + 6]) * inv_l, __uint_as_float(v[8 * g + 7]) * inv_l);
            *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = o;
          }
        }
      }
      if (p.lse && row_ok && wg == 0)
        p.lse[(static_cast<long long>(batch) * p.Hq + head) * p.S + qi] = (l > 0.f) ? (m_used + log2f(l)) * 0.6931471805599453f : -CUDART_INF_F;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

int make_tmap_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                 uint32_t box_outer, bool f32);

}  // namespace b200

using namespace b200;

// qkv: [B*S, row_stride] bf16 with q heads, then k heads, then v heads in every row (head_dim 128).
// out: [B*S, out_stride] bf16 (Hq*128 columns used); lse: [B, Hq, S] fp32 or NULL.
extern "C" int b200_flash_fwd(const void* qkv, long long row_stride, void* out, long long out_stride, float* lse, int B, int S,
                              int Hq, int Hkv, int head_dim, float scale, int causal, int* err, cudaStream_t stream) {
  if (head_dim != FA_D || Hq % Hkv || row_stride % 8 || out_stride % 8) return -10;
  if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(out)) & 15) return -11;
  if (B <= 0 || S <= 0) return 0;
  CUtensorMap tm;
  int rc = make_tmap_2d(&tm, qkv, static_cast<uint64_t>(Hq + 2 * Hkv) * FA_D, static_cast<uint64_t>(B) * S, row_stride, 64, FA_BM, false);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FlashSmem::TOTAL) != cudaSuccess) return -3;
    attr_set = true;
  }
  FlashArgs a;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.lse = lse;
  a.B = B; a.S = S; a.Hq = Hq; a.Hkv = Hkv;
  a.out_stride = out_stride;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = causal;
  a.err = err;
  dim3 grid((S + FA_BM - 1) / FA_BM, Hq, B);
  flash_fwd_kernel<<<grid, FA_THREADS, FlashSmem::TOTAL, stream>>>(tm, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
