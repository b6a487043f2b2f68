// Shared device helpers for the sm_100a kernels of this library.
//
// Every kernel here is launched through an extern "C" function that takes raw
// device pointers, sizes and a CUDA stream; the Python side (csrc/ops.py) checks
// shapes, types and contiguity before it calls.  Element types are passed as an
// integer code so that one entry point serves the bfloat16 and the float32 path.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define BN_F32 0
#define BN_BF16 1

// Tokens per cache page.  A sequence holds whole pages; position p of a sequence
// lies in page_table[slot][p / BN_PAGE] at row p % BN_PAGE.
#define BN_PAGE 64

// Launch status: 0 ok, otherwise a code that csrc/ops.py turns into an exception.
#define BN_OK 0
#define BN_ERR_BAD_ARG 1
#define BN_ERR_LAUNCH 2

// ---- programmatic dependent launch -----------------------------------------------------------
// Every kernel of this library is launched with programmatic stream serialization: it may start
// while the kernel before it in the stream is still running, and calls pdl_wait() before its
// first access to global memory that another kernel may write (or, for writes, read).  Kernels
// call pdl_launch_dependents() early so that their successor's prologue overlaps them.  What a
// kernel does before pdl_wait() touches only read-only weights, shared and tensor memory.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <utility>
// Compile with -DBN_NO_PDL to serialise kernels completely (for comparisons; csrc/build.py's
// EXTRA_FLAGS); nothing at run time switches it.
#ifdef BN_NO_PDL
static inline bool bn_pdl_enabled() { return false; }
#else
static inline bool bn_pdl_enabled() { return true; }
#endif

// Timestamp probes inside the TMA-fed kernels (where a block's time goes) exist only in builds
// made with -DBN_TRACE; the default build has neither the stores nor the entry points.
#ifdef BN_TRACE
#define BN_TRACE_ONLY(...) __VA_ARGS__
#else
#define BN_TRACE_ONLY(...)
#endif
template <typename... KArgs, typename... Args>
static inline cudaError_t bn_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = bn_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
// The same for a grid of thread-block clusters.
template <typename... KArgs, typename... Args>
static inline cudaError_t bn_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                            cudaStream_t stream, dim3 cluster, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster.x;
  attr[0].val.clusterDim.y = cluster.y;
  attr[0].val.clusterDim.z = cluster.z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = bn_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#define BN_LAUNCH(kernel, grid, block, smem, stream, ...)                                  \
  do {                                                                                     \
    cudaError_t e__ = bn_launch(kernel, grid, block, smem, stream, __VA_ARGS__);           \
    if (e__ != cudaSuccess) return BN_ERR_LAUNCH + (int)e__;                               \
  } while (0)

#define BN_CHECK_LAUNCH()                                    \
  do {                                                       \
    cudaError_t e__ = cudaGetLastError();                    \
    if (e__ != cudaSuccess) return BN_ERR_LAUNCH + (int)e__; \
  } while (0)

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Load/store of one element of a buffer whose type is only known by code.
__device__ __forceinline__ float load_as_f32(const void* p, int dtype, size_t i) {
  return dtype == BN_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ void store_from_f32(void* p, int dtype, size_t i, float v) {
  if (dtype == BN_F32) ((float*)p)[i] = v;
  else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}

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

// Block-wide sum for blocks of up to 1024 threads; `scratch` holds 32 floats.
// Every thread gets the result.  The order of additions depends only on the
// block size, never on what else runs, so a row's result does not change with
// the batch around it.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (threadIdx.x < nwarp) ? scratch[threadIdx.x] : 0.f;
  if (warp == 0) {
    r = warp_sum(r);
    if (lane == 0) scratch[0] = r;
  }
  __syncthreads();
  return scratch[0];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (threadIdx.x < nwarp) ? scratch[threadIdx.x] : -INFINITY;
  if (warp == 0) {
    r = warp_max(r);
    if (lane == 0) scratch[0] = r;
  }
  __syncthreads();
  return scratch[0];
}

// Address of row (p % BN_PAGE) of key/value head `kvh` in the page that holds position p.
// Cache layout per schedule entry: [n_pages][n_kv_heads][BN_PAGE][head_dim].
__device__ __forceinline__ size_t cache_row_offset(const int* page_table_row, int p,
                                                   int n_kv_heads, int kvh, int head_dim) {
  int page = page_table_row[p / BN_PAGE];
  return (((size_t)page * n_kv_heads + kvh) * BN_PAGE + (p % BN_PAGE)) * (size_t)head_dim;
}
