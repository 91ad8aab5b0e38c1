// Shared helpers for the sm_100a kernels of enginekernel_b200.
//
// Every launcher is an extern "C" function that takes raw device pointers, sizes
// and a cudaStream_t, launches on that stream and returns 0 or a CUDA error code
// (negative values are argument errors found before any launch).  Nothing here
// allocates memory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_set>

#define EK_PAGE 64          // tokens per cache page (must match cache/pages.py)
#define EK_MAX_HEAD_DIM 256

#define EK_ERR_ARG (-2)      // a size the kernel does not take
#define EK_EXPORT extern "C" __attribute__((visibility("default")))

namespace ek {

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

// Four neighbouring values as floats: one 16-byte (float) or 8-byte (bfloat16) access.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<bf16> {
  static __device__ __forceinline__ float4 load(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void store(bf16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block whose size is a multiple of 32 (at most 1024 threads).
// `scratch` holds 33 floats of shared memory; every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();                       // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    float t = lane < nw ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    float t = lane < nw ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Where the keys and values of one cache entry live.  A page holds EK_PAGE
// consecutive positions of one sequence for all KV heads:
//   base[((page * heads + head) * EK_PAGE + pos % EK_PAGE) * head_dim + d]
// `block_table[slot * table_stride + pos / EK_PAGE]` gives the page of a position.
struct PagedKV {
  void* k;                  // this entry's key pages
  void* v;                  // this entry's value pages
  const int* block_table;   // [slots, table_stride]
  int table_stride;
  int heads;                // KV heads
  int head_dim;
};

__device__ __forceinline__ size_t page_offset(const PagedKV& c, int page, int head, int pos) {
  return (((size_t)page * c.heads + head) * EK_PAGE + (pos & (EK_PAGE - 1))) * (size_t)c.head_dim;
}

// Programmatic dependent launch: a kernel launched with `launch_pdl` may start while the
// kernel before it on the stream is still draining.  It must call `pdl_wait()` before it
// reads anything that kernel wrote or writes anything that kernel reads (only constants -
// weights, tables - may be touched earlier), and calls `pdl_launch_dependents()` at its top
// so that its own successor can be set up early.  Both are no-ops in a plain launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Split of an SM's 256 KB between L1 and shared memory that a kernel wants, in percent of
// shared memory (set once per kernel and device).  A kernel without a preference inherits what
// the kernel before it left: the decode attention kernel, which streams through L1, ran 1.5x
// slower behind the GEMM's all-shared split until it asked for its own.
inline void prefer_carveout(const void* fn, int percent_shared) {
  static std::mutex mu;
  static std::unordered_set<unsigned long long> seen;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return;
  const unsigned long long key = (unsigned long long)(uintptr_t)fn * 64ull + (unsigned)device;
  std::lock_guard<std::mutex> lock(mu);
  if (seen.insert(key).second)
    cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, percent_shared);
}

// Streaming multiprocessors of the current device (asked once per device; 0 if it cannot be asked).
inline int sm_count() {
  static int cached[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  if (cached[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    cached[device] = n;
  }
  return cached[device];
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same with the blocks along grid.y grouped into thread-block clusters of `cluster_y`
// (which must divide grid.y): they run at the same time and can read one another's shared memory.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, int cluster_y, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 1;
  attr[1].val.clusterDim.y = (unsigned)cluster_y;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same with the blocks along grid.x grouped into clusters of `cluster_x`.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster_x(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                        cudaStream_t stream, int cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = (unsigned)cluster_x;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Cluster-wide barrier (every thread of every block of the cluster) that also orders shared
// memory writes before it against reads of them after it.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A 32-bit float to the same shared-memory offset in block `rank` of this cluster (seen there
// after the next cluster barrier).
__device__ __forceinline__ void st_cluster_f32(float* own, unsigned rank, float v) {
  unsigned a = (unsigned)__cvta_generic_to_shared(own), r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(r), "f"(v) : "memory");
}
// Four floats (16-byte aligned) to the same shared-memory offset in block `rank` of this cluster.
__device__ __forceinline__ void st_cluster_f32x4(float* own, unsigned rank, float4 v) {
  unsigned a = (unsigned)__cvta_generic_to_shared(own), r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"r"(r), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// Four floats (16-byte aligned) to the same shared-memory offset in block `rank` of this cluster, as
// an asynchronous store that counts its 16 bytes on the mbarrier at `own_bar`'s offset in that block:
// a thread there that has seen the barrier's phase complete sees the data.
__device__ __forceinline__ void st_async_f32x4(float* own, unsigned rank, float4 v, unsigned own_bar) {
  unsigned a = (unsigned)__cvta_generic_to_shared(own), r, b;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(b) : "r"(own_bar), "r"(rank));
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
               ::"r"(r), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "r"(b) : "memory");
}
// Four floats (16-byte aligned) at the same shared-memory offset in block `rank` of this cluster.
__device__ __forceinline__ float4 ld_cluster_f32x4(const float* own, unsigned rank) {
  unsigned a = (unsigned)__cvta_generic_to_shared(own), r;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(r) : "memory");
  return v;
}
// A 32-bit float at the same shared-memory offset in block `rank` of this cluster.
__device__ __forceinline__ float ld_cluster_f32(const float* own, unsigned rank) {
  unsigned a = (unsigned)__cvta_generic_to_shared(own), r;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(r) : "memory");
  return v;
}

}  // namespace ek

#define EK_RETURN_LAUNCH_STATUS() return (int)cudaGetLastError()
