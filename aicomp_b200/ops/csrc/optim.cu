// Fused AdamW over a flat parameter arena: bf16 working weights, fp32 master
// weights and moments, fp32 main gradients.  One launch updates a whole
// pipeline stage; the gradient is optionally zeroed in the same pass so the
// next step's wgrad GEMMs can accumulate into it without a separate memset.
// Global-norm clipping reads a device scalar (sum of squares) so no host sync
// sits between the norm reduction and the update.
// The reference leaves the optimizer to the user (torch.optim.Adam/AdamW on
// fp32 parameters, opt_prime/examples/pp_train_llama5.py:134).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace b200 {

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay;
  float bias_corr1, bias_corr2;  // 1 - beta^t
  float grad_scale;              // multiplies every gradient (e.g. 1/num_microbatches)
  float max_norm;                // <= 0: no clipping
};

// 4 elements per thread, 16-byte accesses on the fp32 streams.
__global__ void __launch_bounds__(256)
adamw_kernel(__nv_bfloat16* __restrict__ p16, float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
             float* __restrict__ g, const __nv_bfloat16* __restrict__ g16, const float* __restrict__ norm_sq, long long n4,
             AdamArgs a, int zero_grad) {
  float clip = 1.f;
  if (a.max_norm > 0.f && norm_sq) {
    const float nrm = sqrtf(*norm_sq) * a.grad_scale;
    clip = fminf(1.f, a.max_norm / (nrm + 1e-6f));
  }
  const float gs = a.grad_scale * clip;
  const float step = a.lr / a.bias_corr1;
  const float inv_bc2 = rsqrtf(a.bias_corr2);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 gg;
    if (g) {
      gg = reinterpret_cast<float4*>(g)[i];
    } else {
      uint2 u = reinterpret_cast<const uint2*>(g16)[i];
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
      float2 lo = __bfloat1622float2(b[0]), hi = __bfloat1622float2(b[1]);
      gg = make_float4(lo.x, lo.y, hi.x, hi.y);
    }
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float4 ww = reinterpret_cast<float4*>(master)[i];
    float gx[4] = {gg.x * gs, gg.y * gs, gg.z * gs, gg.w * gs};
    float mx[4] = {mm.x, mm.y, mm.z, mm.w};
    float vx[4] = {vv.x, vv.y, vv.z, vv.w};
    float wx[4] = {ww.x, ww.y, ww.z, ww.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      mx[j] = a.beta1 * mx[j] + (1.f - a.beta1) * gx[j];
      vx[j] = a.beta2 * vx[j] + (1.f - a.beta2) * gx[j] * gx[j];
      const float denom = sqrtf(vx[j]) * inv_bc2 + a.eps;
      wx[j] = wx[j] * (1.f - a.lr * a.weight_decay) - step * mx[j] / denom;
    }
    reinterpret_cast<float4*>(m)[i] = make_float4(mx[0], mx[1], mx[2], mx[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vx[0], vx[1], vx[2], vx[3]);
    reinterpret_cast<float4*>(master)[i] = make_float4(wx[0], wx[1], wx[2], wx[3]);
    if (p16) {
      uint2 o;
      __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
      ob[0] = __floats2bfloat162_rn(wx[0], wx[1]);
      ob[1] = __floats2bfloat162_rn(wx[2], wx[3]);
      reinterpret_cast<uint2*>(p16)[i] = o;
    }
    if (zero_grad && g) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// out[0] += sum(g^2) over n4*4 floats (out must be zeroed by the caller).
__global__ void __launch_bounds__(256) sumsq_kernel(const float* __restrict__ g, long long n4, float* __restrict__ out) {
  float s = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 x = reinterpret_cast<const float4*>(g)[i];
    s += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  __shared__ float red[8];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 8) {
    s = red[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) s += __shfl_xor_sync(0xffu, s, o);
    if (threadIdx.x == 0) atomicAdd(out, s);
  }
}

// dst (bf16 or fp32) = cast(src fp32 * scale): used to refresh bf16 weights from masters.
__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n4, float scale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 x = reinterpret_cast<const float4*>(src)[i];
    uint2 o;
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
    ob[0] = __floats2bfloat162_rn(x.x * scale, x.y * scale);
    ob[1] = __floats2bfloat162_rn(x.z * scale, x.w * scale);
    reinterpret_cast<uint2*>(dst)[i] = o;
  }
}
// acc (fp32) += src (bf16)
__global__ void accum_bf16_into_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ acc, long long n4) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint2 u = reinterpret_cast<const uint2*>(src)[i];
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
    float2 lo = __bfloat1622float2(b[0]), hi = __bfloat1622float2(b[1]);
    float4 a = reinterpret_cast<float4*>(acc)[i];
    a.x += lo.x; a.y += lo.y; a.z += hi.x; a.w += hi.y;
    reinterpret_cast<float4*>(acc)[i] = a;
  }
}

static inline int ew_grid(long long items) {
  long long b = (items + 255) / 256;
  const long long cap = 148LL * 8;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace b200

using namespace b200;

// n must be a multiple of 4 and all pointers 16-byte aligned (8 for bf16).  Exactly one of g (fp32) / g16 (bf16).
extern "C" int b200_adamw(void* p16, float* master, float* m, float* v, float* g, const void* g16, const float* norm_sq,
                          long long n, float lr, float beta1, float beta2, float eps, float weight_decay, int step,
                          float grad_scale, float max_norm, int zero_grad, cudaStream_t stream) {
  if (n % 4 || (!g && !g16)) return -10;
  if (n <= 0) return 0;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  double b1 = 1.0, b2 = 1.0;
  for (int i = 0; i < step; ++i) { b1 *= beta1; b2 *= beta2; if (b1 < 1e-30 && b2 < 1e-30) break; }
  a.bias_corr1 = static_cast<float>(1.0 - b1);
  a.bias_corr2 = static_cast<float>(1.0 - b2);
  a.grad_scale = grad_scale;
  a.max_norm = max_norm;
  adamw_kernel<<<ew_grid(n / 4), 256, 0, stream>>>(static_cast<__nv_bfloat16*>(p16), master, m, v, g,
                                                   static_cast<const __nv_bfloat16*>(g16), norm_sq, n / 4, a, zero_grad);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
extern "C" int b200_sumsq(const float* g, long long n, float* out, cudaStream_t stream) {
  if (n % 4) return -10;
  if (n <= 0) return 0;
  sumsq_kernel<<<ew_grid(n / 4), 256, 0, stream>>>(g, n / 4, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
extern "C" int b200_cast_f32_bf16(const float* src, void* dst, long long n, float scale, cudaStream_t stream) {
  if (n % 4) return -10;
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<ew_grid(n / 4), 256, 0, stream>>>(src, static_cast<__nv_bfloat16*>(dst), n / 4, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
extern "C" int b200_accum_bf16_f32(const void* src, float* acc, long long n, cudaStream_t stream) {
  if (n % 4) return -10;
  if (n <= 0) return 0;
  accum_bf16_into_f32_kernel<<<ew_grid(n / 4), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), acc, n / 4);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
