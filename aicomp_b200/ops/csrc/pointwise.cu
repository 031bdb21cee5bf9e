// Memory-bound fused ops for bf16 transformer training/inference on sm_100a:
// RoPE (in place, q and k of a packed QKV tensor), SwiGLU and tanh-GELU
// forward/backward, fused cross-entropy (loss + in-place dlogits), embedding
// gather / scatter-add, scaled masked / causal softmax forward/backward.
// All use 16-byte vector accesses and grid-stride loops sized to 148 SMs.
//
// Counterparts in the reference are eager / torch.jit ops: RoPE
// (gpt-neox/megatron/model/positional_embeddings.py:96-119), bias-GELU
// (gpt-neox/megatron/model/activations.py:64-99), CrossEntropyLoss on fp32
// logits (opt_prime/opt_prime/schedule.py:477-525) and the warp-softmax CUDA
// kernels (gpt-neox/megatron/fused_kernels/scaled_masked_softmax.h,
// scaled_upper_triang_masked_softmax.h) whose 2048-column limit does not apply here.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <math_constants.h>

namespace b200 {

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(b[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) b[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_add(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------ RoPE
// x: [tokens, heads_total, D] rows of a packed projection output with row
// pitch `row_stride` elements; the first `n_rot_heads` heads of every token are
// rotated (q heads then k heads of a packed QKV; v is left alone).
// HF "rotate_half" pairing: (x[i], x[i + D/2]).  cos/sin tables: [max_pos, D/2] fp32.
// sign = +1 forward, -1 backward (the transpose of a rotation).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ pos, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, long long tokens, int n_rot_heads, int D,
                            long long row_stride, float sign) {
  const int half = D / 2;
  const int vec_per_head = half / 8;
  const long long total = tokens * n_rot_heads * vec_per_head;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % vec_per_head);
    const long long th = i / vec_per_head;
    const int h = static_cast<int>(th % n_rot_heads);
    const long long t = th / n_rot_heads;
    const int p = pos[t];
    __nv_bfloat16* base = x + t * row_stride + static_cast<long long>(h) * D + v * 8;
    uint4 u1 = *reinterpret_cast<const uint4*>(base);
    uint4 u2 = *reinterpret_cast<const uint4*>(base + half);
    float a[8], b[8], c[8], s[8];
    unpack8(u1, a);
    unpack8(u2, b);
    const float4* cp = reinterpret_cast<const float4*>(cos_t + static_cast<long long>(p) * half + v * 8);
    const float4* sp = reinterpret_cast<const float4*>(sin_t + static_cast<long long>(p) * half + v * 8);
    float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
    s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w; s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
    float o1[8], o2[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sn = s[j] * sign;
      o1[j] = a[j] * c[j] - b[j] * sn;
      o2[j] = b[j] * c[j] + a[j] * sn;
    }
    *reinterpret_cast<uint4*>(base) = pack8(o1);
    *reinterpret_cast<uint4*>(base + half) = pack8(o2);
  }
}

// ------------------------------------------------------------------ SwiGLU
// gu: [rows, 2*I] (gate | up) -> out [rows, I] = silu(gate) * up
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, long long rows, int I) {
  const int vpr = I / 8;
  const long long total = rows * vpr;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vpr;
    const int c = static_cast<int>(i % vpr) * 8;
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(gu + r * 2 * I + c), g);
    unpack8(*reinterpret_cast<const uint4*>(gu + r * 2 * I + I + c), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    *reinterpret_cast<uint4*>(out + r * I + c) = pack8(o);
  }
}
// dgu: [rows, 2*I] receives (dgate | dup)
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ dgu, long long rows, int I) {
  const int vpr = I / 8;
  const long long total = rows * vpr;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vpr;
    const int c = static_cast<int>(i % vpr) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const uint4*>(gu + r * 2 * I + c), g);
    unpack8(*reinterpret_cast<const uint4*>(gu + r * 2 * I + I + c), u);
    unpack8(*reinterpret_cast<const uint4*>(dout + r * I + c), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sg;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (sg + silu * (1.f - sg));
    }
    *reinterpret_cast<uint4*>(dgu + r * 2 * I + c) = pack8(dg);
    *reinterpret_cast<uint4*>(dgu + r * 2 * I + I + c) = pack8(du);
  }
}

// ------------------------------------------------------------------ GELU (tanh form)
__device__ __forceinline__ float gelu_tanh(float x) {
  const float k = 0.7978845608028654f;
  return 0.5f * x * (1.f + tanhf(k * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float k = 0.7978845608028654f;
  const float t = tanhf(k * (x + 0.044715f * x * x * x));
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * (1.f + 3.f * 0.044715f * x * x);
}
__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n8) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float a[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], a);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = gelu_tanh(a[j]);
    reinterpret_cast<uint4*>(y)[i] = pack8(o);
  }
}
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                __nv_bfloat16* __restrict__ dx, long long n8) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float a[8], d[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], a);
    unpack8(reinterpret_cast<const uint4*>(dy)[i], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = d[j] * gelu_tanh_grad(a[j]);
    reinterpret_cast<uint4*>(dx)[i] = pack8(o);
  }
}

// ------------------------------------------------------------------ cross entropy
// One CTA per token row.  Pass 1: online max / sum-exp over V.  Pass 2 (row is
// L2-resident): overwrite logits with dlogits = (softmax - onehot) * grad_scale,
// or zero for ignore_index rows.  loss[row] = lse - logit[label] (0 if ignored).
constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS)
cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels, float* __restrict__ loss,
                     int V, long long ld, int ignore_index, float grad_scale, const float* __restrict__ grad_scale_dev,
                     int write_grad) {
  __shared__ float red_m[CE_THREADS / 32], red_s[CE_THREADS / 32];
  __shared__ float sh_lse;
  const long long row = blockIdx.x;
  __nv_bfloat16* x = logits + row * ld;
  const long long label = labels[row];
  const bool ignored = (label == ignore_index) || label < 0 || label >= V;
  const int nvec = V / 8;  // V % 8 == 0 required
  float m = -CUDART_INF_F, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float a[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], a);
    float lm = a[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, a[j]);
    const float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(a[j] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  // block reduce (max, sum)
  float wm = warp_max(m);
  s = (m == -CUDART_INF_F) ? 0.f : s * __expf(m - wm);  // idle threads hold (-inf, 0)
  s = warp_add(s);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { red_m[w] = wm; red_s[w] = s; }
  __syncthreads();
  if (w == 0) {
    float mm = (l < CE_THREADS / 32) ? red_m[l] : -CUDART_INF_F;
    float ssum = (l < CE_THREADS / 32) ? red_s[l] : 0.f;
    const float gm = warp_max(mm);
    ssum = (mm == -CUDART_INF_F) ? 0.f : ssum * __expf(mm - gm);
    ssum = warp_add(ssum);
    if (l == 0) sh_lse = gm + logf(ssum);
  }
  __syncthreads();
  const float lse = sh_lse;
  if (threadIdx.x == 0) loss[row] = ignored ? 0.f : lse - __bfloat162float(x[label]);
  if (!write_grad) return;
  __syncthreads();  // label logit read before it is overwritten
  const float gs = ignored ? 0.f : grad_scale * (grad_scale_dev ? *grad_scale_dev : 1.f);
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float a[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], a);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float pj = __expf(a[j] - lse);
      if (i * 8 + j == label) pj -= 1.f;
      o[j] = pj * gs;
    }
    reinterpret_cast<uint4*>(x)[i] = pack8(o);
  }
}

// ------------------------------------------------------------------ embedding
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, long long tokens, int H, int vocab) {
  const int vpr = H / 8;
  const long long total = tokens * vpr;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / vpr;
    const int c = static_cast<int>(i % vpr);
    long long id = ids[t];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (id >= 0 && id < vocab) v = reinterpret_cast<const uint4*>(table + id * H)[c];
    reinterpret_cast<uint4*>(out + t * H)[c] = v;
  }
}
// grad table is fp32 (the optimizer's main gradient); rows collide rarely, atomics are fine.
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dtable, long long tokens, int H, int vocab) {
  const int vpr = H / 8;
  const long long total = tokens * vpr;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / vpr;
    const int c = static_cast<int>(i % vpr);
    long long id = ids[t];
    if (id < 0 || id >= vocab) continue;
    float d[8];
    unpack8(reinterpret_cast<const uint4*>(dout + t * H)[c], d);
    float* dst = dtable + id * H + c * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + j, d[j]);
  }
}

// ------------------------------------------------------------------ scaled masked / causal softmax
// x: [batches, sq, sk] bf16.  mode 0: no mask, 1: uint8 mask [mask_batches, sq, sk] (1 = masked -> -10000, as
// the reference kernels), 2: causal (row i keeps columns 0..i + (sk - sq)), masked outputs are exactly 0.
// One warp per row, any sk (strided loop; three passes over an L1/L2-resident row).
__global__ void softmax_fwd_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ mask,
                                   __nv_bfloat16* __restrict__ y, long long rows, int sq, int sk, float scale, int mode,
                                   int heads, int mask_batches) {
  const int warps_per_block = blockDim.x >> 5;
  const int l = threadIdx.x & 31;
  for (long long row = blockIdx.x * static_cast<long long>(warps_per_block) + (threadIdx.x >> 5); row < rows;
       row += static_cast<long long>(gridDim.x) * warps_per_block) {
    const __nv_bfloat16* xr = x + row * sk;
    __nv_bfloat16* yr = y + row * sk;
    const int qi = static_cast<int>(row % sq);
    const int limit = (mode == 2) ? min(sk, qi + 1 + (sk - sq)) : sk;
    const long long mrow = (mask_batches > 1 ? (row / (static_cast<long long>(heads) * sq)) * sq : 0) + qi;
    const uint8_t* mr = (mode == 1) ? mask + mrow * sk : nullptr;
    float m = -CUDART_INF_F;
    for (int c = l; c < limit; c += 32) {
      float v = __bfloat162float(xr[c]) * scale;
      if (mr && mr[c]) v = -10000.f;
      m = fmaxf(m, v);
    }
    m = warp_max(m);
    float s = 0.f;
    for (int c = l; c < limit; c += 32) {
      float v = __bfloat162float(xr[c]) * scale;
      if (mr && mr[c]) v = -10000.f;
      s += __expf(v - m);
    }
    s = warp_add(s);
    const float inv = 1.f / s;
    for (int c = l; c < sk; c += 32) {
      float o = 0.f;
      if (c < limit) {
        float v = __bfloat162float(xr[c]) * scale;
        if (mr && mr[c]) v = -10000.f;
        o = __expf(v - m) * inv;
      }
      yr[c] = __float2bfloat16(o);
    }
  }
}
// dx = scale * (dy*y - y * sum(dy*y))
__global__ void softmax_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ dx, long long rows, int sk, float scale) {
  const int warps_per_block = blockDim.x >> 5;
  const int l = threadIdx.x & 31;
  for (long long row = blockIdx.x * static_cast<long long>(warps_per_block) + (threadIdx.x >> 5); row < rows;
       row += static_cast<long long>(gridDim.x) * warps_per_block) {
    const __nv_bfloat16* dr = dy + row * sk;
    const __nv_bfloat16* yr = y + row * sk;
    float s = 0.f;
    for (int c = l; c < sk; c += 32) s += __bfloat162float(dr[c]) * __bfloat162float(yr[c]);
    s = warp_add(s);
    for (int c = l; c < sk; c += 32) {
      const float yy = __bfloat162float(yr[c]);
      dx[row * sk + c] = __float2bfloat16(scale * (__bfloat162float(dr[c]) * yy - yy * s));
    }
  }
}

static inline int grid_for(long long work_items, int threads) {
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = 148LL * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace b200

using namespace b200;
#define CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? 0 : -4)

extern "C" int b200_rope(void* x, const int* pos, const float* cos_t, const float* sin_t, long long tokens,
                         int n_rot_heads, int D, long long row_stride, float sign, cudaStream_t stream) {
  if (D % 16 || row_stride % 8) return -10;
  if (tokens <= 0 || n_rot_heads <= 0) return 0;
  const long long work = tokens * n_rot_heads * (D / 16);
  rope_kernel<<<grid_for(work, 256), 256, 0, stream>>>(static_cast<__nv_bfloat16*>(x), pos, cos_t, sin_t, tokens,
                                                      n_rot_heads, D, row_stride, sign);
  return CHECK_LAUNCH();
}
extern "C" int b200_swiglu_fwd(const void* gu, void* out, long long rows, int I, cudaStream_t stream) {
  if (I % 8) return -10;
  if (rows <= 0) return 0;
  swiglu_fwd_kernel<<<grid_for(rows * (I / 8), 256), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(gu),
                                                                      static_cast<__nv_bfloat16*>(out), rows, I);
  return CHECK_LAUNCH();
}
extern "C" int b200_swiglu_bwd(const void* gu, const void* dout, void* dgu, long long rows, int I, cudaStream_t stream) {
  if (I % 8) return -10;
  if (rows <= 0) return 0;
  swiglu_bwd_kernel<<<grid_for(rows * (I / 8), 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dout), static_cast<__nv_bfloat16*>(dgu), rows, I);
  return CHECK_LAUNCH();
}
extern "C" int b200_gelu_fwd(const void* x, void* y, long long n, cudaStream_t stream) {
  if (n % 8) return -10;
  if (n <= 0) return 0;
  gelu_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n / 8);
  return CHECK_LAUNCH();
}
extern "C" int b200_gelu_bwd(const void* x, const void* dy, void* dx, long long n, cudaStream_t stream) {
  if (n % 8) return -10;
  if (n <= 0) return 0;
  gelu_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy),
                                                           static_cast<__nv_bfloat16*>(dx), n / 8);
  return CHECK_LAUNCH();
}
// logits [rows, V] bf16 with row pitch ld; overwritten with the gradient when write_grad != 0.
// The gradient is scaled by grad_scale * (*grad_scale_dev if given): e.g. 1 / (number of valid tokens) kept on the device.
extern "C" int b200_cross_entropy(void* logits, const long long* labels, float* loss, long long rows, int V, long long ld,
                                  int ignore_index, float grad_scale, const float* grad_scale_dev, int write_grad,
                                  cudaStream_t stream) {
  if (V % 8 || ld % 8) return -10;
  if (rows <= 0) return 0;
  cross_entropy_kernel<<<static_cast<unsigned>(rows), CE_THREADS, 0, stream>>>(static_cast<__nv_bfloat16*>(logits), labels, loss, V, ld,
                                                                             ignore_index, grad_scale, grad_scale_dev, write_grad);
  return CHECK_LAUNCH();
}
extern "C" int b200_embedding_fwd(const long long* ids, const void* table, void* out, long long tokens, int H, int vocab,
                                  cudaStream_t stream) {
  if (H % 8) return -10;
  if (tokens <= 0) return 0;
  embedding_fwd_kernel<<<grid_for(tokens * (H / 8), 256), 256, 0, stream>>>(ids, static_cast<const __nv_bfloat16*>(table),
                                                                           static_cast<__nv_bfloat16*>(out), tokens, H, vocab);
  return CHECK_LAUNCH();
}
extern "C" int b200_embedding_bwd(const long long* ids, const void* dout, float* dtable, long long tokens, int H, int vocab,
                                  cudaStream_t stream) {
  if (H % 8) return -10;
  if (tokens <= 0) return 0;
  embedding_bwd_kernel<<<grid_for(tokens * (H / 8), 256), 256, 0, stream>>>(ids, static_cast<const __nv_bfloat16*>(dout), dtable,
                                                                           tokens, H, vocab);
  return CHECK_LAUNCH();
}
// x: [batch, heads, sq, sk] (rows = batch*heads*sq).  mode: 0 none, 1 uint8 mask [mask_batches (1 or batch), 1, sq, sk]
// broadcast over heads, 2 causal.
extern "C" int b200_softmax_fwd(const void* x, const uint8_t* mask, void* y, long long rows, int sq, int sk, float scale,
                                int mode, int heads, int mask_batches, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (mode == 1 && (!mask || heads <= 0 || mask_batches <= 0)) return -10;
  softmax_fwd_kernel<<<grid_for(rows, 8), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), mask, static_cast<__nv_bfloat16*>(y),
                                                           rows, sq, sk, scale, mode, heads > 0 ? heads : 1, mask_batches);
  return CHECK_LAUNCH();
}
extern "C" int b200_softmax_bwd(const void* dy, const void* y, void* dx, long long rows, int sk, float scale, cudaStream_t stream) {
  if (rows <= 0) return 0;
  softmax_bwd_kernel<<<grid_for(rows, 8), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(y),
                                                           static_cast<__nv_bfloat16*>(dx), rows, sk, scale);
  return CHECK_LAUNCH();
}
