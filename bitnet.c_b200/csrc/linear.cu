// out[M, N] = x[M, K] . W[N, K]^T for few rows M: the weight matrix is streamed once
// per group of up to 8 rows of x, one warp per output column.  Weights are row-major
// [out_features, in_features], y = W x, as in the reference (src/quant/f32_scalar.c:10-31);
// its decode path uses a warp-per-row matvec as well (src/gpu_cuda.cu:3976-4012).
// Products are accumulated in float32 whatever the storage type.
#include "common.cuh"

template <typename T>
struct VecLd;
template <>
struct VecLd<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float* o) {
    float4 v = __ldg(reinterpret_cast<const float4*>(p));
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <>
struct VecLd<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float* o) {
    uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      o[2 * i] = f.x; o[2 * i + 1] = f.y;
    }
  }
};

#define SK_MT 8
#define SK_WARPS 8

template <typename T>
__global__ void linear_skinny_kernel(const T* __restrict__ x, const T* __restrict__ w, void* __restrict__ out,
                                     int out_dtype, int M, int N, int K, int ldo) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int n = blockIdx.x * SK_WARPS + warp;
  if (n >= N) return;
  constexpr int VN = VecLd<T>::N;
  const T* wrow = w + (size_t)n * K;
  for (int m0 = 0; m0 < M; m0 += SK_MT) {
    int mt = min(SK_MT, M - m0);
    float acc[SK_MT];
#pragma unroll
    for (int i = 0; i < SK_MT; ++i) acc[i] = 0.f;
    for (int k = lane * VN; k < K; k += 32 * VN) {
      float wv[VN];
      VecLd<T>::load(wrow + k, wv);
#pragma unroll
      for (int i = 0; i < SK_MT; ++i) {
        if (i < mt) {
          float xv[VN];
          VecLd<T>::load(x + (size_t)(m0 + i) * K + k, xv);
#pragma unroll
          for (int e = 0; e < VN; ++e) acc[i] = fmaf(wv[e], xv[e], acc[i]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < SK_MT; ++i) {
      if (i < mt) {
        float v = warp_sum(acc[i]);
        if (lane == 0) store_from_f32(out, out_dtype, (size_t)(m0 + i) * ldo + n, v);
      }
    }
  }
}

// x and w share the element type `dtype`; K must be a multiple of 8 (16-byte rows).
extern "C" int bn_linear_skinny(const void* x, const void* w, int dtype, void* out, int out_dtype, int M, int N,
                                int K, int ldo, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return BN_OK;
  if (K <= 0 || K % 8 || ldo < N) return BN_ERR_BAD_ARG;
  unsigned blocks = (unsigned)((N + SK_WARPS - 1) / SK_WARPS);
  if (dtype == BN_F32)
    BN_LAUNCH((linear_skinny_kernel<float>), blocks, SK_WARPS * 32, 0, stream, (const float*)x, (const float*)w, out,
                                                                    out_dtype, M, N, K, ldo);
  else if (dtype == BN_BF16)
    BN_LAUNCH((linear_skinny_kernel<__nv_bfloat16>), blocks, SK_WARPS * 32, 0, stream, 
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, out, out_dtype, M, N, K, ldo);
  else
    return BN_ERR_BAD_ARG;
  BN_CHECK_LAUNCH();
  return BN_OK;
}
