// RMSNorm / LayerNorm forward and backward for bf16 activations (fp32 math).
//
// One CTA per row in the forward; the backward is persistent (a fixed number
// of CTAs stride over the rows) so that each CTA can keep its partial weight
// (and bias) gradient in registers and spill it once to a [ctas, H] fp32
// scratch that a second small kernel folds into the gradient.
//
// The forward optionally fuses the residual add that precedes every norm in a
// pre-norm transformer block:  r = x + residual;  y = norm(r) * w.
// Replaces eager HF norms of the reference's traced graphs (LlamaRMSNorm /
// nn.LayerNorm, e.g. gpt-neox/megatron/model/norms.py:34-76).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace b200 {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_VEC = 4;  // 16-byte vectors per thread -> H <= 256*8*4 = 8192
constexpr int NORM_BWD_ROWS = 2; // rows a backward CTA processes per loop iteration

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < NORM_THREADS / 32) ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}

struct Vec8 {
  float f[8];
};
__device__ __forceinline__ Vec8 load8(const __nv_bfloat16* p) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
  Vec8 v;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(b[i]);
    v.f[2 * i] = f.x;
    v.f[2 * i + 1] = f.y;
  }
  return v;
}
__device__ __forceinline__ Vec8 unpack8(const uint4& u) {
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
  Vec8 v;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(b[i]);
    v.f[2 * i] = f.x;
    v.f[2 * i + 1] = f.y;
  }
  return v;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const Vec8& v) {
  uint4 u;
  __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) b[i] = __floats2bfloat162_rn(v.f[2 * i], v.f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

// ------------------------------------------------------------------ forward
// IS_LN: LayerNorm (mean subtraction, optional bias) else RMSNorm.
template <bool IS_LN>
__global__ void __launch_bounds__(NORM_THREADS)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ res_out,
                float* __restrict__ stat_rstd, float* __restrict__ stat_mean, int rows, int H, float eps) {
  __shared__ float red[NORM_THREADS / 32];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const long long base = static_cast<long long>(row) * H;
  const int nvec = H / 8;
  Vec8 v[NORM_MAX_VEC];
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_MAX_VEC; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      v[i] = load8(x + base + c * 8);
      if (residual) {
        Vec8 r = load8(residual + base + c * 8);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i].f[j] += r.f[j];
      }
      if (res_out) {
        store8(res_out + base + c * 8, v[i]);
        // norm the value that was stored (bf16-rounded), as the unfused graph would
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i].f[j] = __bfloat162float(__float2bfloat16(v[i].f[j]));
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { s += v[i].f[j]; ss += v[i].f[j] * v[i].f[j]; }
    }
  }
  float mean = 0.f;
  if (IS_LN) {
    mean = block_sum(s, red) / H;
    float var = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAX_VEC; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { float d = v[i].f[j] - mean; var += d * d; }
      }
    }
    ss = block_sum(var, red);
  } else {
    ss = block_sum(ss, red);
  }
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0) {
    if (stat_rstd) stat_rstd[row] = rstd;
    if (IS_LN && stat_mean) stat_mean[row] = mean;
  }
#pragma unroll
  for (int i = 0; i < NORM_MAX_VEC; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      Vec8 wv = load8(w + c * 8);
      Vec8 o;
#pragma unroll
      for (int j = 0; j < 8; ++j) o.f[j] = (v[i].f[j] - mean) * rstd * wv.f[j];
      if (IS_LN && b) {
        Vec8 bv = load8(b + c * 8);
#pragma unroll
        for (int j = 0; j < 8; ++j) o.f[j] += bv.f[j];
      }
      store8(y + base + c * 8, o);
    }
  }
}

// ------------------------------------------------------------------ backward
// dx = rstd * (g - xhat * mean(g * xhat) [- mean(g)])   with g = dy * w
// dw partial = sum_rows dy * xhat ; db partial = sum_rows dy
// `dres` (optional) is added to dx: the gradient arriving on the residual branch.
// Each loop iteration handles ROWS consecutive rows at once: their loads are all in flight together and one pair of
// block barriers serves all of them (a row at a time left the kernel bound by load and barrier latency).  The raw
// bf16 vectors stay in registers between the two phases; NV = 16-byte vectors per thread (H <= NV * 2048).
template <bool IS_LN, int NV, int ROWS>
__global__ void __launch_bounds__(NORM_THREADS, 2)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                const __nv_bfloat16* __restrict__ w, const float* __restrict__ stat_rstd,
                const float* __restrict__ stat_mean, const __nv_bfloat16* __restrict__ dres,
                __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, float* __restrict__ db_partial,
                int rows, int H) {
  constexpr int NRED = ROWS * (IS_LN ? 2 : 1);
  __shared__ float red[NORM_THREADS / 32][NRED];
  const int nvec = H / 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float dw_acc[NV][8];
  float db_acc[IS_LN ? NV : 1][8];
  Vec8 wv[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dw_acc[i][j] = 0.f;
      wv[i].f[j] = 0.f;
      if (IS_LN) db_acc[i][j] = 0.f;
    }
    if (c < nvec) wv[i] = load8(w + c * 8);
  }
  for (long long rb = static_cast<long long>(blockIdx.x) * ROWS; rb < rows; rb += static_cast<long long>(gridDim.x) * ROWS) {
    uint4 dyr[ROWS][NV], xr[ROWS][NV];
    float rstd[ROWS], mean[ROWS], sums[NRED];
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
      const bool live = rb + k < rows;
      rstd[k] = live ? stat_rstd[rb + k] : 0.f;
      mean[k] = (IS_LN && live) ? stat_mean[rb + k] : 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * NORM_THREADS;
        if (live && c < nvec) {
          dyr[k][i] = *reinterpret_cast<const uint4*>(dy + (rb + k) * H + c * 8);
          xr[k][i] = *reinterpret_cast<const uint4*>(x + (rb + k) * H + c * 8);
        } else {
          dyr[k][i] = make_uint4(0, 0, 0, 0);
          xr[k][i] = make_uint4(0, 0, 0, 0);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const Vec8 d = unpack8(dyr[k][i]), xv = unpack8(xr[k][i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv.f[j] - mean[k]) * rstd[k];
          const float g = d.f[j] * wv[i].f[j];
          dw_acc[i][j] += d.f[j] * xh;
          if (IS_LN) db_acc[i][j] += d.f[j];
          s1 += g * xh;
          s2 += g;
        }
      }
      sums[k] = warp_sum(s1);
      if (IS_LN) sums[ROWS + k] = warp_sum(s2);
    }
    __syncthreads();   // the previous iteration's readers of `red` are done
    if (lane == 0) {
#pragma unroll
      for (int k = 0; k < NRED; ++k) red[warp][k] = sums[k];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < NRED; ++k) {
      float t = 0.f;
#pragma unroll
      for (int ww = 0; ww < NORM_THREADS / 32; ++ww) t += red[ww][k];
      sums[k] = t / H;
    }
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
      if (rb + k >= rows) break;
      const float s1 = sums[k], s2 = IS_LN ? sums[ROWS + k] : 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * NORM_THREADS;
        if (c < nvec) {
          const Vec8 d = unpack8(dyr[k][i]), xv = unpack8(xr[k][i]);
          Vec8 o;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float xh = (xv.f[j] - mean[k]) * rstd[k];
            o.f[j] = rstd[k] * (d.f[j] * wv[i].f[j] - xh * s1 - s2);
          }
          if (dres) {
            const Vec8 r = load8(dres + (rb + k) * H + c * 8);
#pragma unroll
            for (int j = 0; j < 8; ++j) o.f[j] += r.f[j];
          }
          store8(dx + (rb + k) * H + c * 8, o);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      float4* dst = reinterpret_cast<float4*>(dw_partial + static_cast<long long>(blockIdx.x) * H + c * 8);
      dst[0] = make_float4(dw_acc[i][0], dw_acc[i][1], dw_acc[i][2], dw_acc[i][3]);
      dst[1] = make_float4(dw_acc[i][4], dw_acc[i][5], dw_acc[i][6], dw_acc[i][7]);
      if (IS_LN && db_partial) {
        float4* dstb = reinterpret_cast<float4*>(db_partial + static_cast<long long>(blockIdx.x) * H + c * 8);
        dstb[0] = make_float4(db_acc[i][0], db_acc[i][1], db_acc[i][2], db_acc[i][3]);
        dstb[1] = make_float4(db_acc[i][4], db_acc[i][5], db_acc[i][6], db_acc[i][7]);
      }
    }
  }
}

template <bool IS_LN>
static void launch_norm_bwd(int ctas, cudaStream_t stream, const __nv_bfloat16* dy, const __nv_bfloat16* x, const __nv_bfloat16* w,
                            const float* rstd, const float* mean, const __nv_bfloat16* dres, __nv_bfloat16* dx, float* dwp, float* dbp,
                            int rows, int H) {
  if (H <= NORM_THREADS * 8 * 2)
    norm_bwd_kernel<IS_LN, 2, NORM_BWD_ROWS><<<ctas, NORM_THREADS, 0, stream>>>(dy, x, w, rstd, mean, dres, dx, dwp, dbp, rows, H);
  else
    norm_bwd_kernel<IS_LN, 4, NORM_BWD_ROWS / 2><<<ctas, NORM_THREADS, 0, stream>>>(dy, x, w, rstd, mean, dres, dx, dwp, dbp, rows, H);
}

// Number of CTAs for `rows` rows: every CTA gets the same number of row groups (no ragged last wave).
static int norm_bwd_grid(int rows, int H, int max_ctas) {
  const int per = H <= NORM_THREADS * 8 * 2 ? NORM_BWD_ROWS : NORM_BWD_ROWS / 2;
  const int groups = (rows + per - 1) / per;
  const int waves = (groups + max_ctas - 1) / max_ctas;
  return (groups + waves - 1) / waves;
}

// Fold [parts, H] partials into grad (fp32, accumulate) or grad_bf16 (overwrite or accumulate).
// One CTA = 32 columns; its 8 warps take every 8th partial row, then combine through shared memory.
__global__ void __launch_bounds__(256)
norm_fold_partials_kernel(const float* __restrict__ partial, int parts, int H, float* __restrict__ grad_f32,
                          __nv_bfloat16* __restrict__ grad_bf16, int accumulate) {
  __shared__ float red[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (c < H)
    for (int p = warp; p < parts; p += 8) s += partial[static_cast<long long>(p) * H + c];
  red[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && c < H) {
#pragma unroll
    for (int ww = 1; ww < 8; ++ww) s += red[ww][lane];
    if (grad_f32) grad_f32[c] = accumulate ? grad_f32[c] + s : s;
    if (grad_bf16) grad_bf16[c] = __float2bfloat16(accumulate ? __bfloat162float(grad_bf16[c]) + s : s);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_norm_bwd_ctas() { return 296; }

// y = norm(x [+ residual]) * w [+ b]; res_out (optional) receives x + residual.  H % 8 == 0, H <= 8192.
extern "C" int b200_norm_fwd(const void* x, const void* residual, const void* w, const void* b, void* y, void* res_out,
                             float* rstd, float* mean, int rows, int H, float eps, int is_layernorm,
                             cudaStream_t stream) {
  if (H % 8 || H > NORM_THREADS * 8 * NORM_MAX_VEC) return -10;
  if (rows <= 0) return 0;
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto R = static_cast<const __nv_bfloat16*>(residual);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto B = static_cast<const __nv_bfloat16*>(b);
  auto Y = static_cast<__nv_bfloat16*>(y);
  auto RO = static_cast<__nv_bfloat16*>(res_out);
  if (is_layernorm) norm_fwd_kernel<true><<<rows, NORM_THREADS, 0, stream>>>(X, R, W, B, Y, RO, rstd, mean, rows, H, eps);
  else norm_fwd_kernel<false><<<rows, NORM_THREADS, 0, stream>>>(X, R, W, B, Y, RO, rstd, mean, rows, H, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Backward.  `scratch` holds 2 * ctas * H floats (ctas = b200_norm_bwd_ctas()).
// dw/db go to fp32 (dw_f32/db_f32, accumulate flag) and/or bf16 buffers.
extern "C" int b200_norm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const float* mean,
                             const void* dres, void* dx, float* scratch, float* dw_f32, void* dw_bf16, float* db_f32,
                             void* db_bf16, int accumulate, int rows, int H, int is_layernorm, cudaStream_t stream) {
  if (H % 8 || H > NORM_THREADS * 8 * NORM_MAX_VEC) return -10;
  if (rows <= 0) return 0;
  const int ctas = norm_bwd_grid(rows, H, b200_norm_bwd_ctas());
  float* dwp = scratch;
  float* dbp = scratch + static_cast<long long>(b200_norm_bwd_ctas()) * H;
  auto DY = static_cast<const __nv_bfloat16*>(dy);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto DR = static_cast<const __nv_bfloat16*>(dres);
  auto DX = static_cast<__nv_bfloat16*>(dx);
  if (is_layernorm) launch_norm_bwd<true>(ctas, stream, DY, X, W, rstd, mean, DR, DX, dwp, dbp, rows, H);
  else launch_norm_bwd<false>(ctas, stream, DY, X, W, rstd, mean, DR, DX, dwp, nullptr, rows, H);
  norm_fold_partials_kernel<<<(H + 31) / 32, 256, 0, stream>>>(dwp, ctas, H, dw_f32, static_cast<__nv_bfloat16*>(dw_bf16), accumulate);
  if (is_layernorm && (db_f32 || db_bf16))
    norm_fold_partials_kernel<<<(H + 31) / 32, 256, 0, stream>>>(dbp, ctas, H, db_f32, static_cast<__nv_bfloat16*>(db_bf16), accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ---------------------------------------------------------------- allocation-free RMSNorm backward
#include "b200_noalloc.h"
#include <mutex>

// Partial weight gradients of b200_rmsnorm_bwd_noalloc: one row of H floats per CTA.  In host code this name is only
// a handle for cudaGetSymbolAddress; kernels receive the looked-up device address.
static __device__ __align__(256) float g_rmsnorm_noalloc_partials[B200_NOALLOC_CTAS * B200_NOALLOC_MAX_H];

static int noalloc_scratch_for_current_device(float** out) {
  constexpr int kMaxDevices = 64;
  static float* cached[kMaxDevices] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200_NOALLOC_ERR_SYMBOL;
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    void* p = nullptr;  // once per device, with that device current: the array has one instance per GPU
    if (cudaGetSymbolAddress(&p, g_rmsnorm_noalloc_partials) != cudaSuccess || !p) return B200_NOALLOC_ERR_SYMBOL;
    cached[dev] = static_cast<float*>(p);
  }
  *out = cached[dev];
  return 0;
}

extern "C" int b200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                                        void* dx, float* dw_f32, void* dw_bf16, int accumulate, int rows, int H,
                                        cudaStream_t stream) {
  if (H > B200_NOALLOC_MAX_H) return B200_NOALLOC_ERR_TOO_LARGE;
  if (H % 8 || H <= 0) return -10;
  if (rows <= 0) return 0;
  float* partials = nullptr;
  int rc = noalloc_scratch_for_current_device(&partials);
  if (rc) return rc;
  const int ctas = norm_bwd_grid(rows, H, B200_NOALLOC_CTAS);
  // every CTA writes all H entries of its own row of `partials`, and the fold below reads exactly `ctas` rows:
  // nothing left over from an earlier call is ever read, so no clearing is needed.
  launch_norm_bwd<false>(ctas, stream, static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
                         static_cast<const __nv_bfloat16*>(w), rstd, nullptr, static_cast<const __nv_bfloat16*>(dres),
                         static_cast<__nv_bfloat16*>(dx), partials, nullptr, rows, H);
  if (dw_f32 || dw_bf16)
    norm_fold_partials_kernel<<<(H + 31) / 32, 256, 0, stream>>>(partials, ctas, H, dw_f32, static_cast<__nv_bfloat16*>(dw_bf16),
                                                                 accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
