// SwiGLU over rows of width 2 I that hold, alternating, 8 gate values and the 8 up values of the
// same indices: out[t, i] = silu(h[t, 16 (i / 8) + i % 8]) * h[t, 16 (i / 8) + 8 + i % 8].
// (The stacked gate/up weight is laid out that way so that the small-batch product can apply
// the activation in its epilogue, linear_tc.cu.)  One thread takes a block of 8: it reads the 8
// gate and 8 up values as whole 16- or 32-byte pieces and writes 8 results.
// Reference: silu(z) = z / (1 + exp(-z)) with exact expf on the reference-activation
// path (src/transformer/cpu_backend.c:365-392, src/transformer/prefill_backend.c:25-49).
#include "common.cuh"

__device__ __forceinline__ float silu_mul_one(float g, float u) { return g / (1.0f + expf(-g)) * u; }

__global__ void silu_mul_bf16_kernel(const __nv_bfloat16* __restrict__ h, __nv_bfloat16* __restrict__ out,
                                     int blocks_per_row, size_t total_blocks) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_blocks) return;
  size_t t = idx / blocks_per_row;
  size_t j = idx - t * blocks_per_row;
  const uint4* src = reinterpret_cast<const uint4*>(h + (t * blocks_per_row + j) * 16);
  uint4 gr = src[0], ur = src[1];
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gr);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&ur);
  uint4 res;
  __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 g = __bfloat1622float2(g2[i]), u = __bfloat1622float2(u2[i]);
    r2[i] = __floats2bfloat162_rn(silu_mul_one(g.x, u.x), silu_mul_one(g.y, u.y));
  }
  *reinterpret_cast<uint4*>(out + (t * blocks_per_row + j) * 8) = res;
}

__global__ void silu_mul_f32_kernel(const float* __restrict__ h, float* __restrict__ out, int blocks_per_row,
                                    size_t total_blocks) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_blocks) return;
  size_t t = idx / blocks_per_row;
  size_t j = idx - t * blocks_per_row;
  const float4* src = reinterpret_cast<const float4*>(h + (t * blocks_per_row + j) * 16);
  float4 g0 = src[0], g1 = src[1], u0 = src[2], u1 = src[3];
  float4* dst = reinterpret_cast<float4*>(out + (t * blocks_per_row + j) * 8);
  dst[0] = make_float4(silu_mul_one(g0.x, u0.x), silu_mul_one(g0.y, u0.y), silu_mul_one(g0.z, u0.z), silu_mul_one(g0.w, u0.w));
  dst[1] = make_float4(silu_mul_one(g1.x, u1.x), silu_mul_one(g1.y, u1.y), silu_mul_one(g1.z, u1.z), silu_mul_one(g1.w, u1.w));
}

// h: [n_rows, 2 * inter], out: [n_rows, inter]; inter a multiple of 8, both 16-byte aligned.
extern "C" int bn_silu_mul(const void* h, void* out, int dtype, int n_rows, int inter, cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (inter <= 0 || inter % 8 || (((uintptr_t)h | (uintptr_t)out) & 15)) return BN_ERR_BAD_ARG;
  int bpr = inter / 8;
  size_t total = (size_t)n_rows * bpr;
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == BN_F32)
    BN_LAUNCH(silu_mul_f32_kernel, blocks, 256, 0, stream, (const float*)h, (float*)out, bpr, total);
  else if (dtype == BN_BF16)
    BN_LAUNCH(silu_mul_bf16_kernel, blocks, 256, 0, stream, (const __nv_bfloat16*)h, (__nv_bfloat16*)out, bpr, total);
  else
    return BN_ERR_BAD_ARG;
  return BN_OK;
}

// x = x * scale, then (cap != 0) x = tanhf(x / cap) * cap: an output head's logit scale and the
// reference's final soft-cap (src/transformer/logits.c:325-333), float32 in place.
__global__ void scale_softcap_kernel(float* __restrict__ x, size_t n, float scale, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = x[i] * scale;
  if (cap != 0.0f) v = tanhf(v * (1.0f / cap)) * cap;
  x[i] = v;
}

extern "C" int bn_scale_softcap(float* x, long long n, float scale, float cap, cudaStream_t stream) {
  if (n <= 0) return BN_OK;
  if (!x) return BN_ERR_BAD_ARG;
  unsigned blocks = (unsigned)(((size_t)n + 255) / 256);
  BN_LAUNCH(scale_softcap_kernel, blocks, 256, 0, stream, x, (size_t)n, scale, cap);
  return BN_OK;
}
