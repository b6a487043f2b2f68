// SwiGLU over rows of width 2 I that hold, alternating, 8 gate values and the 8 up values of the
// same indices: out[t, i] = silu(h[t, 16 (i / 8) + i % 8]) * h[t, 16 (i / 8) + 8 + i % 8].
// (The stacked gate/up weight is laid out that way so that the small-batch product can apply
// the activation in its epilogue, linear_mma.cu.)
// Reference: silu(z) = z / (1 + exp(-z)) with exact expf on the reference-activation
// path (src/transformer/cpu_backend.c:365-392, src/transformer/prefill_backend.c:25-49).
#include "common.cuh"

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ h, T* __restrict__ out, int inter, size_t total) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  size_t t = idx / inter;
  int i = (int)(idx - t * inter);
  size_t col = (size_t)(i >> 3) * 16 + (i & 7);
  float g = to_f32<T>(h[t * 2 * inter + col]);
  float u = to_f32<T>(h[t * 2 * inter + col + 8]);
  float s = g / (1.0f + expf(-g));
  out[idx] = from_f32<T>(s * u);
}

extern "C" int bn_silu_mul(const void* h, void* out, int dtype, int n_rows, int inter, cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (inter <= 0 || inter % 8) return BN_ERR_BAD_ARG;
  size_t total = (size_t)n_rows * inter;
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == BN_F32)
    BN_LAUNCH((silu_mul_kernel<float>), blocks, 256, 0, stream, (const float*)h, (float*)out, inter, total);
  else if (dtype == BN_BF16)
    BN_LAUNCH((silu_mul_kernel<__nv_bfloat16>), blocks, 256, 0, stream, (const __nv_bfloat16*)h, (__nv_bfloat16*)out, inter, total);
  else
    return BN_ERR_BAD_ARG;
  BN_CHECK_LAUNCH();
  return BN_OK;
}
