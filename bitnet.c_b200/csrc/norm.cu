// Residual add fused with RMSNorm.
//
//   v = x[row] (+ delta[row]);  x[row] = v (when write_x);  out[r] = v * rsqrt(mean(v^2) + eps) * w
//
// x is the float32 residual stream; delta is the output of the part that ran
// before (any element type), possibly as n_parts partial sums [n_parts, rows, width] left by
// a product that split its inner dimension (linear_mma.cu); they are added in order of the
// part index.  The sum and the statistics are float32.  With a
// row index the kernel reads only the listed rows and writes them densely: this
// serves the final norm, which is needed at the wanted positions only.
// Reference: eps is added to the mean inside the root, out = x * scale * w
// (src/transformer/rmsnorm_scalar.c:4-13); the residual add fused in front is the
// reference's residual_rmsnorm kernel (src/gpu_cuda.cu:5077).
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

// Few rows (decode): one row per block would leave most SMs idle and each block with a long
// chain of loads, so a row is spread over a thread-block cluster of NORM_CLUSTER blocks.  Each
// block holds its columns in registers, the sums of squares meet through distributed shared
// memory, and every block adds them in rank order, so all see the same scale.
#define NORM_CLUSTER 8
#define NORM_CL_THREADS 128
#define NORM_CL_VEC 4  // float4 groups per thread: up to 128 * 4 * 4 = 2048 columns per block

__device__ __forceinline__ float4 load4_as_f32(const void* p, int dtype, size_t i) {
  if (dtype == BN_F32) return *reinterpret_cast<const float4*>((const float*)p + i);
  uint2 raw = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)p + i);
  float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4_from_f32(void* p, int dtype, size_t i, float4 v) {
  if (dtype == BN_F32) {
    *reinterpret_cast<float4*>((float*)p + i) = v;
  } else {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<unsigned*>(&a);
    raw.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>((__nv_bfloat16*)p + i) = raw;
  }
}

__global__ void __cluster_dims__(1, NORM_CLUSTER, 1) __launch_bounds__(NORM_CL_THREADS)
add_rmsnorm_cluster_kernel(float* __restrict__ x, const void* __restrict__ delta, int delta_dtype, int n_parts,
                           size_t part_stride, const void* __restrict__ w, int w_dtype, void* __restrict__ out,
                           int out_dtype, const int* __restrict__ rows, int width, int cols_per_block, float eps,
                           int write_x) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  __shared__ float scratch[32];
  __shared__ float block_ss;
  cg::cluster_group cluster = cg::this_cluster();
  const int r = blockIdx.x, rank = blockIdx.y;  // the cluster spans gridDim.y == NORM_CLUSTER
  const size_t row = rows ? (size_t)rows[r] : (size_t)r;
  const int c0 = rank * cols_per_block, c1 = min(width, c0 + cols_per_block);
  float4 v[NORM_CL_VEC];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < NORM_CL_VEC; ++u) {
    int c = c0 + (u * NORM_CL_THREADS + threadIdx.x) * 4;
    v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < c1) {
      float4 a = *reinterpret_cast<const float4*>(x + row * width + c);
      if (delta) {
        for (int p = 0; p < n_parts; ++p) {
          float4 d = load4_as_f32(delta, delta_dtype, p * part_stride + row * width + c);
          a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
        }
      }
      v[u] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) block_ss = ss;
  cluster.sync();
  float total = 0.f;
  for (int k = 0; k < NORM_CLUSTER; ++k) total += *cluster.map_shared_rank(&block_ss, k);
  float scale = 1.0f / sqrtf(total / (float)width + eps);
#pragma unroll
  for (int u = 0; u < NORM_CL_VEC; ++u) {
    int c = c0 + (u * NORM_CL_THREADS + threadIdx.x) * 4;
    if (c < c1) {
      float4 a = v[u];
      if (write_x) *reinterpret_cast<float4*>(x + row * width + c) = a;
      float4 g = load4_as_f32(w, w_dtype, c);
      store4_from_f32(out, out_dtype, (size_t)r * width + c,
                      make_float4(a.x * scale * g.x, a.y * scale * g.y, a.z * scale * g.z, a.w * scale * g.w));
    }
  }
  cluster.sync();  // no block may leave while another still reads its sum
}

__global__ void add_rmsnorm_kernel(float* __restrict__ x, const void* __restrict__ delta, int delta_dtype,
                                   int n_parts, size_t part_stride, const void* __restrict__ w, int w_dtype, void* __restrict__ out,
                                   int out_dtype, const int* __restrict__ rows, int width, float eps,
                                   int write_x, int vec4) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  extern __shared__ __align__(16) float v[];  // width floats, then 32 for the reduction
  float* scratch = v + width;
  int r = blockIdx.x;
  size_t row = rows ? (size_t)rows[r] : (size_t)r;
  float* xr = x + row * width;
  float ss = 0.f;
  if (vec4) {
    // groups of four columns, whole 8- or 16-byte pieces (the launcher checked the alignment)
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
      float4 a = *reinterpret_cast<const float4*>(xr + i);
      if (delta) {
        for (int p = 0; p < n_parts; ++p) {
          float4 d = load4_as_f32(delta, delta_dtype, p * part_stride + row * width + i);
          a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
        }
      }
      *reinterpret_cast<float4*>(v + i) = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      float a = xr[i];
      if (delta) {
        for (int p = 0; p < n_parts; ++p) a += load_as_f32(delta, delta_dtype, p * part_stride + row * width + i);
      }
      v[i] = a;
      ss += a * a;
    }
  }
  ss = block_sum(ss, scratch);
  float scale = 1.0f / sqrtf(ss / (float)width + eps);
  if (vec4) {
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
      float4 a = *reinterpret_cast<const float4*>(v + i);
      if (write_x) *reinterpret_cast<float4*>(xr + i) = a;
      float4 g = load4_as_f32(w, w_dtype, i);
      store4_from_f32(out, out_dtype, (size_t)r * width + i,
                      make_float4(a.x * scale * g.x, a.y * scale * g.y, a.z * scale * g.z, a.w * scale * g.w));
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      float a = v[i];
      if (write_x) xr[i] = a;
      store_from_f32(out, out_dtype, (size_t)r * width + i, a * scale * load_as_f32(w, w_dtype, i));
    }
  }
}

extern "C" int bn_add_rmsnorm(float* x, const void* delta, int delta_dtype, int n_parts, long long part_stride,
                              const void* w, int w_dtype,
                              void* out, int out_dtype, const int* rows, int n_rows, int width, float eps,
                              int write_x, cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (width <= 0 || !(eps > 0.f) || (delta && n_parts < 1)) return BN_ERR_BAD_ARG;
  // few rows of a wide model: a cluster of blocks per row (columns in multiples of 4, all pointers
  // and row strides 16-byte aligned)
  int cols = ((width + NORM_CLUSTER - 1) / NORM_CLUSTER + 3) / 4 * 4;
  bool aligned = width % 8 == 0 && (((uintptr_t)x | (uintptr_t)out | (uintptr_t)w | (uintptr_t)delta) & 15) == 0 &&
                 (part_stride % 8) == 0;
  if (n_rows <= 256 && width >= 1024 && aligned && cols <= NORM_CL_THREADS * NORM_CL_VEC * 4) {
    BN_LAUNCH(add_rmsnorm_cluster_kernel, dim3(n_rows, NORM_CLUSTER), NORM_CL_THREADS, 0, stream, 
        x, delta, delta_dtype, n_parts, (size_t)part_stride, w, w_dtype, out, out_dtype, rows, width, cols, eps,
        write_x);
    BN_CHECK_LAUNCH();
    return BN_OK;
  }
  size_t smem = ((size_t)width + 32) * sizeof(float);
  if (smem > 200 * 1024) return BN_ERR_BAD_ARG;  // width beyond 51,168: refused
  if (smem > 48 * 1024) {
    static size_t granted = 0;
    if (smem > granted) {
      cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
      granted = smem;
    }
  }
  int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  BN_LAUNCH(add_rmsnorm_kernel, n_rows, threads, smem, stream, x, delta, delta_dtype, n_parts, (size_t)part_stride, w,
                                                       w_dtype, out, out_dtype,
                                                       rows, width, eps, write_x, aligned ? 1 : 0);
  BN_CHECK_LAUNCH();
  return BN_OK;
}
