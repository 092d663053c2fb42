// Shared helpers of the sm_100a kernels: element types, conversions, warp and
// block reductions, the C calling convention of the library.
//
// Every exported function is `extern "C"`, takes raw device pointers, sizes
// and a stream, launches on that stream and returns the cudaError_t of the
// launch as an int (0 = success).  Element types are passed as codes:
// 0 = float32, 1 = bfloat16.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <math.h>

#define IFX_API extern "C" __attribute__((visibility("default")))

enum IfxDtype : int { IFX_F32 = 0, IFX_BF16 = 1 };

// Error codes above the CUDA range, returned for arguments a kernel refuses.
enum IfxError : int {
  IFX_ERR_UNSUPPORTED = 100001,   // a size or type the kernel does not take
  IFX_ERR_ALIGNMENT = 100002,     // a pointer or stride that breaks an alignment rule
};
// What a kernel writes into the device error word that its caller passes: 1 = a bounded wait ran out,
// 2 = the decode attention kernel met a context longer than the bound it was launched with.
constexpr int IFX_DEVICE_ERR_WAIT = 1, IFX_DEVICE_ERR_DECODE_PIECES = 2;


typedef __nv_bfloat16 bf16;

template <typename T> struct Num;
template <> struct Num<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct Num<bf16> {
  static __device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ bf16 from_f(float v) { return __float2bfloat16_rn(v); }
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

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of additions depends only on blockDim, so a row's result does not
// depend on what else is in the batch.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : 0.0f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

// Description of one layer's slice of a paged key/value pool laid out as
// [page][layer][k|v][kv_head][slot_in_page][head_dim].
struct PagedKV {
  void* k;                 // this layer's keys of page 0
  void* v;                 // this layer's values of page 0
  long long page_stride;   // elements between consecutive pages
  int head_stride;         // elements between kv heads = page_size * head_dim
  int page_size;           // tokens per page (a power of two)
  int page_shift;          // log2(page_size)
};

#define IFX_LAUNCH_CHECK() ((int)cudaGetLastError())

// Programmatic dependent launch.  Every kernel of the library starts with pdl_enter(): it lets the kernel
// after it in the stream be launched at once (that kernel's launch latency and set-up then overlap this
// kernel's work; it waits at its own pdl_wait), and waits until the kernel before it has finished and
// its writes are visible.  A kernel may do work that does not depend on the kernels before it (reading
// parameters or a step's metadata) between pdl_launch_dependents() and pdl_wait(); it must not write
// anything there.  Kernels are launched with launch_pdl(), which sets the attribute that allows this;
// after a kernel that never signals (a library kernel) the launch behaves like a plain one.
#ifdef IFX_TIMELINE
// Optional instrumentation (a build of its own, never the serving one): the first thread of a kernel's
// first block notes the global timer once the kernel before it is complete, so that the gaps between
// kernels can be read in place, inside a replayed graph.  One list per translation unit; the host reader
// that IFX_STAMP_READER defines copies it out, and the lists are merged by time.
static __device__ unsigned long long ifx_stamps[4096];
static __device__ unsigned int ifx_stamp_count;
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    const unsigned i = atomicAdd(&ifx_stamp_count, 1u);
    if (i < 4096) ifx_stamps[i] = t;
  }
}
#define IFX_STAMP_READER(name) \
  IFX_API int name(unsigned long long* host, int reset) { \
    unsigned int n = 0; cudaDeviceSynchronize(); cudaMemcpyFromSymbol(&n, ifx_stamp_count, sizeof(n)); \
    if (n > 4096) n = 4096; \
    if (n) cudaMemcpyFromSymbol(host, ifx_stamps, n * sizeof(unsigned long long)); \
    if (reset) { unsigned int z = 0; cudaMemcpyToSymbol(ifx_stamp_count, &z, sizeof(z)); } \
    return (int)n; }
#else
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
#define IFX_STAMP_READER(name)
#endif
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() {
  pdl_launch_dependents();
  pdl_wait();
}
template <typename Kern, typename... Args>
inline int launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
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
  return (int)cudaLaunchKernelEx(&cfg, kern, args...);
}

// The same with the blocks grouped into thread-block clusters of `cluster` blocks (grid dimensions are
// multiples of it).
template <typename Kern, typename... Args>
inline int launch_pdl_cluster(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, dim3 cluster, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster.x;
  attr[1].val.clusterDim.y = cluster.y;
  attr[1].val.clusterDim.z = cluster.z;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return (int)cudaLaunchKernelEx(&cfg, kern, args...);
}
