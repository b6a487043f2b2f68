// out[M, N] = x[M, K] . W[N, K]^T for few rows M: the weight matrix is streamed once per group
// of up to 8 rows of x.  A block stages a chunk of those rows of x in shared memory; a warp takes
// two output columns and two 16-byte pieces of each per step, so that four weight loads are in
// flight per lane and what it reads of x serves both columns.  Weights are row-major
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
  __device__ static void load_shared(const float* p, float* o) {
    float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <>
struct VecLd<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void unpack(uint4 v, float* o) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      o[2 * i] = f.x; o[2 * i + 1] = f.y;
    }
  }
  __device__ static void load(const __nv_bfloat16* p, float* o) { unpack(__ldg(reinterpret_cast<const uint4*>(p)), o); }
  __device__ static void load_shared(const __nv_bfloat16* p, float* o) { unpack(*reinterpret_cast<const uint4*>(p), o); }
};

#define SK_MT 8
#define SK_WARPS 8
#define SK_COLS 2   // output columns per warp
#define SK_KC 1024  // elements of a row of x staged at a time (SK_MT rows: 32 KB in float32)

template <typename T>
__global__ void __launch_bounds__(SK_WARPS * 32)
linear_skinny_kernel(const T* __restrict__ x, const T* __restrict__ w, void* __restrict__ out, int out_dtype, int M, int N,
                     int K, int ldo) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  __shared__ __align__(16) T xs[SK_MT][SK_KC];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int VN = VecLd<T>::N;
  const int n0 = (blockIdx.x * SK_WARPS + warp) * SK_COLS;
  const int nc = min(SK_COLS, N - n0);  // <= 0: this warp has no column, it only helps staging
  // columns past the matrix read the last one again (their sums are not stored)
  const T* wrow[SK_COLS];
#pragma unroll
  for (int c = 0; c < SK_COLS; ++c) wrow[c] = w + (size_t)min(n0 + c, N - 1) * K;
  for (int m0 = 0; m0 < M; m0 += SK_MT) {
    const int mt = min(SK_MT, M - m0);
    float acc[SK_MT][SK_COLS];
#pragma unroll
    for (int i = 0; i < SK_MT; ++i)
#pragma unroll
      for (int c = 0; c < SK_COLS; ++c) acc[i][c] = 0.f;
    for (int kc = 0; kc < K; kc += SK_KC) {
      const int kn = min(SK_KC, K - kc);  // a multiple of 8
      __syncthreads();  // the chunk before this one has been used by every warp
      for (int i = 0; i < mt; ++i)
        for (int kk = threadIdx.x * VN; kk < kn; kk += SK_WARPS * 32 * VN)
          *reinterpret_cast<uint4*>(&xs[i][kk]) = __ldg(reinterpret_cast<const uint4*>(x + (size_t)(m0 + i) * K + kc + kk));
      __syncthreads();
      if (nc <= 0) continue;
      // The order of the additions of one output depends on K alone: lane l adds the products of
      // elements l*VN.. of every piece of 32*VN elements in turn (two pieces per step), then the
      // lanes are summed by the same tree.
      for (int k = lane * VN; k < kn; k += 2 * 32 * VN) {
        const bool second = k + 32 * VN < kn;
        float wv[2][SK_COLS][VN];
#pragma unroll
        for (int c = 0; c < SK_COLS; ++c) {
          VecLd<T>::load(wrow[c] + kc + k, wv[0][c]);
          if (second) VecLd<T>::load(wrow[c] + kc + k + 32 * VN, wv[1][c]);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (u == 1 && !second) break;
#pragma unroll
          for (int i = 0; i < SK_MT; ++i) {
            if (i < mt) {
              float xv[VN];
              VecLd<T>::load_shared(&xs[i][k + u * 32 * VN], xv);
#pragma unroll
              for (int c = 0; c < SK_COLS; ++c)
#pragma unroll
                for (int e = 0; e < VN; ++e) acc[i][c] = fmaf(wv[u][c][e], xv[e], acc[i][c]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < SK_MT; ++i) {
      if (i < mt) {
#pragma unroll
        for (int c = 0; c < SK_COLS; ++c) {
          float v = warp_sum(acc[i][c]);
          if (lane == 0 && c < nc) store_from_f32(out, out_dtype, (size_t)(m0 + i) * ldo + n0 + c, v);
        }
      }
    }
  }
}

// x and w share the element type `dtype`; K must be a multiple of 8 (16-byte rows).
extern "C" int bn_linear_skinny(const void* x, const void* w, int dtype, void* out, int out_dtype, int M, int N,
                                int K, int ldo, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return BN_OK;
  if (K <= 0 || K % 8 || ldo < N) return BN_ERR_BAD_ARG;
  unsigned blocks = (unsigned)((N + SK_WARPS * SK_COLS - 1) / (SK_WARPS * SK_COLS));
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
