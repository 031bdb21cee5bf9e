// Paged-KV decode attention and KV page writes for continuous-batching inference (bf16, GQA native).
//
// Page pools (per layer):  K, V : [num_pages, PAGE (16 tokens), kv_heads, head_dim (128)]  bf16.
// A sequence owns a list of pages (its row of the block table) and a length.  Decode attention for one new
// token per sequence is memory-bound: every K/V element is read once and used by the `G = q_heads / kv_heads`
// query heads that share it.  One CTA handles (sequence, kv head, split of the sequence); per iteration it
// consumes exactly one page: 16 groups of 8 lanes take one token each, a lane holds 16 of the 128 dims.
// Scores are reduced inside the 8-lane group, softmax is kept online per group, and the 16 groups (and the
// splits, through a small fp32 scratch) are merged at the end.
//
// The reference has no paged cache: it keeps a dense [B, heads, max_seq, D] tensor per layer, copies the whole
// prefix every step and calls SDPA on it (opt_prime/opt_prime/kv_cache.py:391-403).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <math_constants.h>

namespace b200 {

constexpr int PA_PAGE = 16;
constexpr int PA_D = 128;
constexpr int PA_THREADS = 128;

__device__ __forceinline__ void bf16x8_to_f32(const uint4& u, float* f) {
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(b[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// partial layout (when splits > 1): [seq][q_head][split][D + 2] fp32 = (acc[0..D), m, l)
template <int G>
__global__ void __launch_bounds__(PA_THREADS)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride, const __nv_bfloat16* __restrict__ k_pool,
                    const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ block_table, int max_blocks,
                    const int* __restrict__ seq_lens, int kv_heads, int parts, float scale_log2, int splits,
                    __nv_bfloat16* __restrict__ out, long long out_stride, float* __restrict__ partial) {
  // `parts` CTAs share one kv head when it serves more than G query heads (G_total = G * parts)
  const int seq = blockIdx.x, kvh = blockIdx.y / parts, part = blockIdx.y % parts, split = blockIdx.z;
  const int len = seq_lens[seq];
  const int n_pages = (len + PA_PAGE - 1) / PA_PAGE;
  const int pages_per_split = (n_pages + splits - 1) / splits;
  const int p_lo = split * pages_per_split;
  const int p_hi = min(n_pages, p_lo + pages_per_split);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = warp * 4 + (lane >> 3);  // token slot inside the page, 0..15
  const int sub = lane & 7;                // which 16-dim slice of the head
  const int d0 = sub * 16;

  float qf[G][16];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    const __nv_bfloat16* qp = q + seq * q_stride + (static_cast<long long>(kvh) * G * parts + part * G + h) * PA_D + d0;
    bf16x8_to_f32(*reinterpret_cast<const uint4*>(qp), &qf[h][0]);
    bf16x8_to_f32(*reinterpret_cast<const uint4*>(qp + 8), &qf[h][8]);
  }
  float acc[G][16];
  float m[G], l[G];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    m[h] = -CUDART_INF_F;
    l[h] = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[h][i] = 0.f;
  }
  const long long tok_stride = static_cast<long long>(kv_heads) * PA_D;
  for (int p = p_lo; p < p_hi; ++p) {
    const int page = block_table[static_cast<long long>(seq) * max_blocks + p];
    const int tok = p * PA_PAGE + grp;
    const long long off = (static_cast<long long>(page) * PA_PAGE + grp) * tok_stride + static_cast<long long>(kvh) * PA_D + d0;
    float kf[16], vf[16];
    bf16x8_to_f32(__ldg(reinterpret_cast<const uint4*>(k_pool + off)), &kf[0]);
    bf16x8_to_f32(__ldg(reinterpret_cast<const uint4*>(k_pool + off + 8)), &kf[8]);
    bf16x8_to_f32(__ldg(reinterpret_cast<const uint4*>(v_pool + off)), &vf[0]);
    bf16x8_to_f32(__ldg(reinterpret_cast<const uint4*>(v_pool + off + 8)), &vf[8]);
    const bool valid = tok < len;
#pragma unroll
    for (int h = 0; h < G; ++h) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) s += qf[h][i] * kf[i];
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      s = valid ? s * scale_log2 : -CUDART_INF_F;
      const float mn = fmaxf(m[h], s);
      if (mn > -CUDART_INF_F) {
        const float corr = exp2f(m[h] - mn);
        const float pw = exp2f(s - mn);
        l[h] = l[h] * corr + pw;
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[h][i] = acc[h][i] * corr + pw * vf[i];
        m[h] = mn;
      }
    }
  }
  // ---- merge the 16 token groups of this CTA
  __shared__ float sm_acc[16][G][PA_D];
  __shared__ float sm_m[16][G], sm_l[16][G];
#pragma unroll
  for (int h = 0; h < G; ++h) {
#pragma unroll
    for (int i = 0; i < 16; ++i) sm_acc[grp][h][d0 + i] = acc[h][i];
    if (sub == 0) { sm_m[grp][h] = m[h]; sm_l[grp][h] = l[h]; }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * PA_D; idx += PA_THREADS) {
    const int h = idx / PA_D, d = idx % PA_D;
    float M = -CUDART_INF_F;
#pragma unroll
    for (int g = 0; g < 16; ++g) M = fmaxf(M, sm_m[g][h]);
    float L = 0.f, a = 0.f;
    if (M > -CUDART_INF_F) {
#pragma unroll
      for (int g = 0; g < 16; ++g) {
        const float w = exp2f(sm_m[g][h] - M);
        L += sm_l[g][h] * w;
        a += sm_acc[g][h][d] * w;
      }
    }
    const int qh = kvh * G * parts + part * G + h;
    if (splits == 1) {
      out[seq * out_stride + static_cast<long long>(qh) * PA_D + d] = __float2bfloat16(L > 0.f ? a / L : 0.f);
    } else {
      float* pp = partial + ((static_cast<long long>(seq) * (kv_heads * G * parts) + qh) * splits + split) * (PA_D + 2);
      pp[d] = a;
      if (d == 0) { pp[PA_D] = M; pp[PA_D + 1] = L; }
    }
  }
}

__global__ void __launch_bounds__(PA_D)
paged_decode_merge_kernel(const float* __restrict__ partial, int q_heads, int splits, __nv_bfloat16* __restrict__ out,
                          long long out_stride) {
  const int seq = blockIdx.x, qh = blockIdx.y, d = threadIdx.x;
  const float* base = partial + (static_cast<long long>(seq) * q_heads + qh) * splits * (PA_D + 2);
  float M = -CUDART_INF_F;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, base[s * (PA_D + 2) + PA_D]);
  float L = 0.f, a = 0.f;
  if (M > -CUDART_INF_F) {
    for (int s = 0; s < splits; ++s) {
      const float w = exp2f(base[s * (PA_D + 2) + PA_D] - M);
      L += base[s * (PA_D + 2) + PA_D + 1] * w;
      a += base[s * (PA_D + 2) + d] * w;
    }
  }
  out[seq * out_stride + static_cast<long long>(qh) * PA_D + d] = __float2bfloat16(L > 0.f ? a / L : 0.f);
}

// Scatter the K and V heads of new tokens (rows of a packed QKV projection, after RoPE) into their pages.
__global__ void paged_kv_write_kernel(const __nv_bfloat16* __restrict__ qkv, long long row_stride, int q_heads, int kv_heads,
                                      const int* __restrict__ seq_ids, const int* __restrict__ positions,
                                      const int* __restrict__ block_table, int max_blocks, __nv_bfloat16* __restrict__ k_pool,
                                      __nv_bfloat16* __restrict__ v_pool, long long tokens) {
  const int vec_per_tok = kv_heads * PA_D / 8;
  const long long total = tokens * vec_per_tok;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / vec_per_tok;
    const int c = static_cast<int>(i % vec_per_tok);
    const int pos = positions[t];
    const int page = block_table[static_cast<long long>(seq_ids[t]) * max_blocks + pos / PA_PAGE];
    const long long dst = (static_cast<long long>(page) * PA_PAGE + pos % PA_PAGE) * kv_heads * PA_D + c * 8;
    const __nv_bfloat16* src = qkv + t * row_stride + static_cast<long long>(q_heads) * PA_D + c * 8;
    *reinterpret_cast<uint4*>(k_pool + dst) = *reinterpret_cast<const uint4*>(src);
    *reinterpret_cast<uint4*>(v_pool + dst) = *reinterpret_cast<const uint4*>(src + static_cast<long long>(kv_heads) * PA_D);
  }
}

}  // namespace b200

using namespace b200;

// floats of scratch needed by b200_paged_decode for the given problem (0 when a single split is used)
extern "C" long long b200_paged_decode_scratch_floats(int n_seqs, int q_heads, int splits) {
  return splits <= 1 ? 0 : static_cast<long long>(n_seqs) * q_heads * splits * (PA_D + 2);
}

extern "C" int b200_paged_decode(const void* q, long long q_stride, const void* k_pool, const void* v_pool, const int* block_table,
                                 int max_blocks, const int* seq_lens, int n_seqs, int q_heads, int kv_heads, int head_dim,
                                 float scale, int splits, void* out, long long out_stride, float* scratch, cudaStream_t stream) {
  if (head_dim != PA_D || q_heads % kv_heads || q_stride % 8 || out_stride % 8) return -10;
  if (n_seqs <= 0) return 0;
  if (splits < 1) splits = 1;
  if (splits > 1 && !scratch) return -11;
  const int Gt = q_heads / kv_heads;
  const int G = Gt >= 4 ? 4 : Gt;  // query heads per CTA; larger groups are split over several CTAs
  if (Gt % G) return -12;
  const int parts = Gt / G;
  const float sl2 = scale * 1.4426950408889634f;
  dim3 grid(n_seqs, kv_heads * parts, splits);
  auto Q = static_cast<const __nv_bfloat16*>(q);
  auto K = static_cast<const __nv_bfloat16*>(k_pool);
  auto V = static_cast<const __nv_bfloat16*>(v_pool);
  auto O = static_cast<__nv_bfloat16*>(out);
#define LAUNCH(GG) paged_decode_kernel<GG><<<grid, PA_THREADS, 0, stream>>>(Q, q_stride, K, V, block_table, max_blocks, seq_lens, \
                                                                       kv_heads, parts, sl2, splits, O, out_stride, scratch)
  switch (G) {
    case 1: LAUNCH(1); break;
    case 2: LAUNCH(2); break;
    case 4: LAUNCH(4); break;
    default: return -12;
  }
#undef LAUNCH
  if (splits > 1) paged_decode_merge_kernel<<<dim3(n_seqs, q_heads), PA_D, 0, stream>>>(scratch, q_heads, splits, O, out_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int b200_paged_kv_write(const void* qkv, long long row_stride, int q_heads, int kv_heads, int head_dim, const int* seq_ids,
                                   const int* positions, const int* block_table, int max_blocks, void* k_pool, void* v_pool,
                                   long long tokens, cudaStream_t stream) {
  if (head_dim != PA_D || row_stride % 8) return -10;
  if (tokens <= 0) return 0;
  long long work = tokens * (kv_heads * PA_D / 8);
  int blocks = static_cast<int>((work + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  paged_kv_write_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(qkv), row_stride, q_heads, kv_heads, seq_ids,
                                                   positions, block_table, max_blocks, static_cast<__nv_bfloat16*>(k_pool),
                                                   static_cast<__nv_bfloat16*>(v_pool), tokens);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
