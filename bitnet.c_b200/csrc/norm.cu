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

__global__ void add_rmsnorm_kernel(float* __restrict__ x, const void* __restrict__ delta, int delta_dtype,
                                   int n_parts, size_t part_stride, const void* __restrict__ w, int w_dtype, void* __restrict__ out,
                                   int out_dtype, const int* __restrict__ rows, int width, float eps,
                                   int write_x) {
  extern __shared__ float v[];  // width floats, then 32 for the reduction
  float* scratch = v + width;
  int r = blockIdx.x;
  size_t row = rows ? (size_t)rows[r] : (size_t)r;
  float* xr = x + row * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float a = xr[i];
    if (delta) {
      for (int p = 0; p < n_parts; ++p) a += load_as_f32(delta, delta_dtype, p * part_stride + row * width + i);
    }
    v[i] = a;
    ss += a * a;
  }
  ss = block_sum(ss, scratch);
  float scale = 1.0f / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float a = v[i];
    if (write_x) xr[i] = a;
    store_from_f32(out, out_dtype, (size_t)r * width + i, a * scale * load_as_f32(w, w_dtype, i));
  }
}

extern "C" int bn_add_rmsnorm(float* x, const void* delta, int delta_dtype, int n_parts, long long part_stride,
                              const void* w, int w_dtype,
                              void* out, int out_dtype, const int* rows, int n_rows, int width, float eps,
                              int write_x, cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (width <= 0 || !(eps > 0.f) || (delta && n_parts < 1)) return BN_ERR_BAD_ARG;
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
  add_rmsnorm_kernel<<<n_rows, threads, smem, stream>>>(x, delta, delta_dtype, n_parts, (size_t)part_stride, w,
                                                       w_dtype, out, out_dtype,
                                                       rows, width, eps, write_x);
  BN_CHECK_LAUNCH();
  return BN_OK;
}
