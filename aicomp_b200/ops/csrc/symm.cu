// Peer-memory ("symmetric") buffers and the collectives built directly on them.
//
// Buffers are cudaMalloc'd, exported with CUDA IPC and opened by every other
// rank of a process group on the same NVSwitch domain, so kernels address a
// peer's HBM with ordinary loads and stores over NVLink 5.  On top of that:
//
//   * signal / wait   monotonically increasing 32-bit epochs in a flag pad,
//                     written to peers with release-at-system-scope stores and
//                     polled with acquire loads under a time limit;
//   * all_reduce_mean two-shot gradient all-reduce fused with the 1/dp scaling:
//                     every rank sums its slice from all peers' buffers in fp32
//                     (reduce-scatter), then pulls the other slices (all-gather);
//   * page push       prefill -> decode KV-cache page transfer: one CTA per page
//                     copies K and V of all layers into the peer's page pool and
//                     raises the request's ready flag only after the data.
//
// The reference moves gradients with NCCL all-reduce inside torch DDP
// (opt_prime/opt_prime/opti_pri.py:852) and has no KV transfer at all.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <string.h>

namespace b200 {

constexpr unsigned long long PEER_WAIT_LIMIT_NS = 2000000000ull;  // 2 s
constexpr int MAX_PEERS = 8;
constexpr int ERR_WAIT_PEER_CODE = 5;

struct PeerPtrs {
  void* p[MAX_PEERS];
};

__device__ __forceinline__ unsigned long long gtime_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Wait until *flag >= epoch (wrap-safe), at most PEER_WAIT_LIMIT_NS.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, int* err) {
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  while (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) < 0) {
    if ((++spins & 0xff) == 0) {
      if (t0 == 0) t0 = gtime_ns();
      else if (gtime_ns() - t0 > PEER_WAIT_LIMIT_NS) {
        atomicCAS(err, 0, ERR_WAIT_PEER_CODE);
        return false;
      }
      __nanosleep(64);
    }
  }
  return true;
}

// flags layout on every rank: [slot][MAX_PEERS] uint32; rank r's arrival is written at [slot][r] on each peer.
__global__ void signal_kernel(PeerPtrs flags, int rank, int world, int slot, uint32_t epoch) {
  __threadfence_system();
  const int t = threadIdx.x;
  if (t < world) st_release_sys(static_cast<uint32_t*>(flags.p[t]) + slot * MAX_PEERS + rank, epoch);
}
__global__ void wait_kernel(const uint32_t* my_flags, int world, int slot, uint32_t epoch, int* err) {
  const int t = threadIdx.x;
  if (t < world) wait_flag(my_flags + slot * MAX_PEERS + t, epoch, err);
}

// Epochs kept in device memory: a launch sequence that bumps, signals and waits through these entry points contains no
// host-side counter and can be captured in a CUDA graph and replayed (every rank replays the same sequence).
__global__ void bump_epoch_kernel(uint32_t* e) { *e += 1u; }
__global__ void signal_dev_kernel(PeerPtrs flags, int rank, int world, int slot, const uint32_t* epoch) {
  __threadfence_system();
  const int t = threadIdx.x;
  if (t < world) st_release_sys(static_cast<uint32_t*>(flags.p[t]) + slot * MAX_PEERS + rank, *epoch);
}
__global__ void wait_dev_kernel(const uint32_t* my_flags, int world, int slot, const uint32_t* epoch, int* err) {
  const int t = threadIdx.x;
  if (t < world) wait_flag(my_flags + slot * MAX_PEERS + t, *epoch, err);
}

// ---------------------------------------------------------------- gradient all-reduce (mean)
// Phase 1: rank r owns elements [r*chunk, (r+1)*chunk) and writes the scaled sum of all peers' values there.
// Every CTA first waits (bounded) until all peers have signalled that their gradients are final.
__global__ void __launch_bounds__(512)
reduce_scatter_mean_kernel(PeerPtrs bufs, const uint32_t* my_flags, int rank, int world, int slot, uint32_t epoch,
                           long long chunk4, long long n4, float scale, int* err) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < world && !wait_flag(my_flags + slot * MAX_PEERS + threadIdx.x, epoch, err)) ok = 0;
  __syncthreads();
  if (!ok) return;
  const long long lo = static_cast<long long>(rank) * chunk4;
  long long hi = lo + chunk4;
  if (hi > n4) hi = n4;
  for (long long i = lo + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < hi;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int p = 0; p < MAX_PEERS; ++p) {
      if (p < world) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(bufs.p[(rank + p) % world]) + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    reinterpret_cast<float4*>(bufs.p[rank])[i] = acc;
  }
}
// Phase 2: copy every other rank's reduced slice into the local buffer.
__global__ void __launch_bounds__(512)
all_gather_slices_kernel(PeerPtrs bufs, const uint32_t* my_flags, int rank, int world, int slot, uint32_t epoch,
                         long long chunk4, long long n4, int* err) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < world && !wait_flag(my_flags + slot * MAX_PEERS + threadIdx.x, epoch, err)) ok = 0;
  __syncthreads();
  if (!ok) return;
  float4* mine = reinterpret_cast<float4*>(bufs.p[rank]);
  for (int pp = 1; pp < world; ++pp) {
    const int src = (rank + pp) % world;
    const long long lo = static_cast<long long>(src) * chunk4;
    long long hi = lo + chunk4;
    if (hi > n4) hi = n4;
    const float4* theirs = reinterpret_cast<const float4*>(bufs.p[src]);
    for (long long i = lo + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < hi;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
      mine[i] = __ldcg(theirs + i);
  }
}

// ---------------------------------------------------------------- generic peer copy (pull) of 16-byte units
__global__ void __launch_bounds__(512)
peer_pull_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long long n16) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n16;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = __ldcg(src + i);
}

// ---------------------------------------------------------------- KV page push (prefill GPU -> decode GPU)
// Pools are [layers][2 (K,V)][pages][page_bytes].  CTA b copies page src_pages[b] of every layer to page
// dst_pages[b] of the peer pool.  The last CTA to finish publishes `ready_value` in the peer's ready word, after a
// system-scope fence, so the decode side never sees the flag before the pages.
__global__ void __launch_bounds__(256)
kv_push_kernel(const uint4* __restrict__ src_pool, uint4* __restrict__ dst_pool, const int* __restrict__ src_pages,
               const int* __restrict__ dst_pages, int n_pages, int layers, long long src_pool_pages,
               long long dst_pool_pages, int page16, uint32_t* dst_ready, uint32_t ready_value,
               unsigned int* done_counter) {
  const int b = blockIdx.x;
  if (b < n_pages) {
    const long long sp = src_pages[b], dp = dst_pages[b];
    for (int l = 0; l < layers * 2; ++l) {
      const uint4* s = src_pool + (static_cast<long long>(l) * src_pool_pages + sp) * page16;
      uint4* d = dst_pool + (static_cast<long long>(l) * dst_pool_pages + dp) * page16;
      for (int i = threadIdx.x; i < page16; i += blockDim.x) d[i] = s[i];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *done_counter = 0;
      if (dst_ready) st_release_sys(dst_ready, ready_value);
    }
  }
}

}  // namespace b200

using namespace b200;

// ---------------------------------------------------------------- host API
extern "C" int b200_symm_alloc(long long bytes, void** out_ptr, void* out_handle64) {
  void* p = nullptr;
  if (cudaMalloc(&p, static_cast<size_t>(bytes)) != cudaSuccess) return -1;
  if (cudaMemset(p, 0, static_cast<size_t>(bytes)) != cudaSuccess) return -2;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return -3;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(out_handle64, &h, 64);
  *out_ptr = p;
  return cudaDeviceSynchronize() == cudaSuccess ? 0 : -4;
}
extern "C" int b200_symm_open(const void* handle64, void** out_ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return -100 - static_cast<int>(e);
  *out_ptr = p;
  return 0;
}
extern "C" int b200_symm_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : -1; }
extern "C" int b200_symm_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : -1; }

static PeerPtrs to_peers(void* const* ptrs, int world) {
  PeerPtrs pp;
  for (int i = 0; i < MAX_PEERS; ++i) pp.p[i] = i < world ? ptrs[i] : nullptr;
  return pp;
}

extern "C" int b200_epoch_bump(void* epoch, cudaStream_t stream) {
  bump_epoch_kernel<<<1, 1, 0, stream>>>(static_cast<uint32_t*>(epoch));
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
extern "C" int b200_signal_dev(void* const* flag_ptrs, int rank, int world, int slot, const void* epoch, cudaStream_t stream) {
  if (world > MAX_PEERS) return -10;
  signal_dev_kernel<<<1, 32, 0, stream>>>(to_peers(flag_ptrs, world), rank, world, slot, static_cast<const uint32_t*>(epoch));
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
extern "C" int b200_wait_dev(const void* my_flags, int world, int slot, const void* epoch, int* err, cudaStream_t stream) {
  if (world > MAX_PEERS) return -10;
  wait_dev_kernel<<<1, 32, 0, stream>>>(static_cast<const uint32_t*>(my_flags), world, slot, static_cast<const uint32_t*>(epoch), err);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
extern "C" int b200_signal(void* const* flag_ptrs, int rank, int world, int slot, unsigned int epoch, cudaStream_t stream) {
  if (world > MAX_PEERS) return -10;
  signal_kernel<<<1, 32, 0, stream>>>(to_peers(flag_ptrs, world), rank, world, slot, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
extern "C" int b200_wait(const void* my_flags, int world, int slot, unsigned int epoch, int* err, cudaStream_t stream) {
  if (world > MAX_PEERS) return -10;
  wait_kernel<<<1, 32, 0, stream>>>(static_cast<const uint32_t*>(my_flags), world, slot, epoch, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// In-place mean all-reduce of n fp32 elements that live at the same offset of every rank's symmetric buffer.
// buf_ptrs[r] / flag_ptrs[r]: rank r's buffer (already offset to the region) / flag pad as mapped in THIS process.
// Uses flag slots slot..slot+2 with the caller-incremented epoch.  ctas: grid size (0 = 4 per SM... capped).
extern "C" int b200_allreduce_mean_f32(void* const* buf_ptrs, void* const* flag_ptrs, int rank, int world, long long n,
                                       int slot, unsigned int epoch, int ctas, int* err, cudaStream_t stream) {
  if (world > MAX_PEERS || n % 4) return -10;
  if (n <= 0) return 0;
  const long long n4 = n / 4;
  const long long chunk4 = (n4 + world - 1) / world;
  if (ctas <= 0) ctas = 148 * 2;
  long long need = (chunk4 + 511) / 512;
  if (need < ctas) ctas = static_cast<int>(need < 1 ? 1 : need);
  PeerPtrs bufs = to_peers(buf_ptrs, world), flags = to_peers(flag_ptrs, world);
  const uint32_t* mine = static_cast<const uint32_t*>(flag_ptrs[rank]);
  signal_kernel<<<1, 32, 0, stream>>>(flags, rank, world, slot, epoch);                    // my gradients are final
  reduce_scatter_mean_kernel<<<ctas, 512, 0, stream>>>(bufs, mine, rank, world, slot, epoch, chunk4, n4, 1.0f / world, err);
  signal_kernel<<<1, 32, 0, stream>>>(flags, rank, world, slot + 1, epoch);                // my slice is reduced
  all_gather_slices_kernel<<<ctas, 512, 0, stream>>>(bufs, mine, rank, world, slot + 1, epoch, chunk4, n4, err);
  signal_kernel<<<1, 32, 0, stream>>>(flags, rank, world, slot + 2, epoch);                // I no longer read peers
  wait_kernel<<<1, 32, 0, stream>>>(mine, world, slot + 2, epoch, err);                    // nobody reads me any more
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Reduce-scatter only (sharded optimizer): afterwards rank r holds the mean over all ranks in its own slice
// [r*chunk, (r+1)*chunk), chunk = ceil(n/4/world)*4 elements; the rest of its buffer still holds its local values.
// Returns after every peer has finished reading this rank's buffer, so the caller may overwrite it.
extern "C" int b200_reduce_scatter_mean_f32(void* const* buf_ptrs, void* const* flag_ptrs, int rank, int world, long long n,
                                            int slot, unsigned int epoch, int ctas, int* err, cudaStream_t stream) {
  if (world > MAX_PEERS || n % 4) return -10;
  if (n <= 0) return 0;
  const long long n4 = n / 4;
  const long long chunk4 = (n4 + world - 1) / world;
  if (ctas <= 0) ctas = 148 * 2;
  long long need = (chunk4 + 511) / 512;
  if (need < ctas) ctas = static_cast<int>(need < 1 ? 1 : need);
  PeerPtrs bufs = to_peers(buf_ptrs, world), flags = to_peers(flag_ptrs, world);
  const uint32_t* mine = static_cast<const uint32_t*>(flag_ptrs[rank]);
  signal_kernel<<<1, 32, 0, stream>>>(flags, rank, world, slot, epoch);                    // my gradients are final
  reduce_scatter_mean_kernel<<<ctas, 512, 0, stream>>>(bufs, mine, rank, world, slot, epoch, chunk4, n4, 1.0f / world, err);
  signal_kernel<<<1, 32, 0, stream>>>(flags, rank, world, slot + 2, epoch);                // I no longer read peers
  wait_kernel<<<1, 32, 0, stream>>>(mine, world, slot + 2, epoch, err);                    // nobody reads me any more
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int b200_peer_pull(void* dst, const void* src, long long bytes, int ctas, cudaStream_t stream) {
  if (bytes % 16) return -10;
  if (bytes <= 0) return 0;
  if (ctas <= 0) ctas = 148;
  peer_pull_kernel<<<ctas, 512, 0, stream>>>(static_cast<uint4*>(dst), static_cast<const uint4*>(src), bytes / 16);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int b200_kv_push(const void* src_pool, void* dst_pool, const int* src_pages, const int* dst_pages, int n_pages,
                            int layers, long long src_pool_pages, long long dst_pool_pages, int page_bytes, void* dst_ready,
                            unsigned int ready_value, void* done_counter, cudaStream_t stream) {
  if (page_bytes % 16) return -10;
  if (n_pages <= 0) return 0;
  kv_push_kernel<<<n_pages, 256, 0, stream>>>(static_cast<const uint4*>(src_pool), static_cast<uint4*>(dst_pool), src_pages,
                                             dst_pages, n_pages, layers, src_pool_pages, dst_pool_pages, page_bytes / 16,
                                             static_cast<uint32_t*>(dst_ready), ready_value,
                                             static_cast<unsigned int*>(done_counter));
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ---------------------------------------------------------------- reduce staged partial results
// out[i] = sum_p in[p * part_stride + i]  (bf16 in, fp32 add, bf16 out): the local half of GEMM -> reduce-scatter,
// after every tensor-parallel peer's GEMM epilogue has stored its partial tile rows into this rank's staging buffer.
namespace b200 {
__global__ void __launch_bounds__(256)
sum_parts_bf16_kernel(const uint4* __restrict__ in, int parts, long long part_stride16, uint4* __restrict__ out, long long n16) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n16;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int p = 0; p < parts; ++p) {
      const uint4 u = in[p * part_stride16 + i];
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(b[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) ob[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    out[i] = o;
  }
}
}  // namespace b200

extern "C" int b200_sum_parts_bf16(const void* in, int parts, long long part_stride_elems, void* out, long long n, cudaStream_t stream) {
  if (n % 8 || part_stride_elems % 8) return -10;
  if (n <= 0) return 0;
  long long n16 = n / 8;
  long long blocks = (n16 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  b200::sum_parts_bf16_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<const uint4*>(in), parts, part_stride_elems / 8,
                                                                          static_cast<uint4*>(out), n16);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ---------------------------------------------------------------- stream-ordered mailbox primitives (pipeline P2P)
// A pipeline stage hands a micro-batch to its neighbour by copying it into a ring slot in the neighbour's memory
// (copy engine, no SMs) and then storing the message number into a flag beside the slot; the neighbour's stream waits
// for the flag with a stream memory operation, which holds no SM either.  A receive that is posted early therefore
// takes no resources away from the persistent GEMM kernels that run while it is pending, unlike a receive kernel.
__global__ void store_flag_kernel(uint32_t* flag, uint32_t value) {
  __threadfence_system();
  st_release_sys(flag, value);
}
// *flag = value (flag may live in a peer's memory), ordered after all earlier work of the stream.
extern "C" int b200_stream_store_flag(void* flag, unsigned int value, cudaStream_t stream) {
  store_flag_kernel<<<1, 1, 0, stream>>>(static_cast<uint32_t*>(flag), value);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

typedef CUresult (*StreamWaitValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
static StreamWaitValue32Fn get_wait_value_fn() {
  static StreamWaitValue32Fn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWaitValue32", &ptr, cudaEnableDefault, &q) != cudaSuccess || !ptr) return nullptr;
    fn = reinterpret_cast<StreamWaitValue32Fn>(ptr);
  }
  return fn;
}
// Later work of `stream` runs once (int32)(*flag - value) >= 0.  `flag` is in THIS device's memory (a peer stores
// into it).  The wait occupies no SM; it ends when the flag arrives or the owning process exits.
extern "C" int b200_stream_wait_flag_geq(void* flag, unsigned int value, cudaStream_t stream) {
  StreamWaitValue32Fn fn = get_wait_value_fn();
  if (!fn) return -1;
  CUresult r = fn(reinterpret_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(flag), value, CU_STREAM_WAIT_VALUE_GEQ);
  return r == CUDA_SUCCESS ? 0 : -2000 - static_cast<int>(r);
}
// Device-to-device copy by the copy engines; either side may be a peer mapping.
extern "C" int b200_copy_async(void* dst, const void* src, long long bytes, cudaStream_t stream) {
  if (bytes <= 0) return 0;
  return cudaMemcpyAsync(dst, src, static_cast<size_t>(bytes), cudaMemcpyDeviceToDevice, stream) == cudaSuccess ? 0 : -4;
}
