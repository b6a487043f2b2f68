// out[M, N] = x[M, K] . W[N, K]^T for few rows M: the weight matrix is streamed once per group
// of up to 8 rows of x.  A block stages a chunk of those rows of x in shared memory; a warp takes
// two output columns and two 16-byte pieces of each per step, so that four weight loads are in
// flight per lane and what it reads of x serves both columns.  Weights are row-major
// [out_features, in_features], y = W x, as in the reference (src/quant/f32_scalar.c:10-31);
// its decode path uses a warp-per-row matvec as well (src/gpu_cuda.cu:3976-4012).
// Products are accumulated in float32 whatever the storage type.
// A matrix with few rows has too few warps to keep the memory busy (4,096 rows are 256 blocks on 148
// SMs), so its inner dimension is shared out over blockIdx.y: split s takes the chunks s, s + splits,
// ... of x, leaves its float32 partial sums in a scratch buffer, and a second small kernel adds
// the splits in their order.  How many splits depends on the matrix alone (never on the rows of x),
// so the order of a result's additions does not depend on what else is in the batch.
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
                     int K, int ldo, float* __restrict__ partial) {
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
    for (int kc = blockIdx.y * SK_KC; kc < K; kc += gridDim.y * SK_KC) {
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
          if (lane == 0 && c < nc) {
            if (gridDim.y > 1) partial[((size_t)blockIdx.y * M + m0 + i) * N + n0 + c] = v;
            else store_from_f32(out, out_dtype, (size_t)(m0 + i) * ldo + n0 + c, v);
          }
        }
      }
    }
  }
}

// out[m, n] = partial[0][m, n] + partial[1][m, n] + ... in that order.
__global__ void __launch_bounds__(256)
linear_skinny_sum_kernel(const float* __restrict__ partial, int splits, void* __restrict__ out, int out_dtype, int M, int N, int ldo) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)M * N) return;
  const int m = (int)(i / N), n = (int)(i - (size_t)m * N);
  float v = 0.f;
  for (int s = 0; s < splits; ++s) v += partial[(size_t)s * M * N + i];
  store_from_f32(out, out_dtype, (size_t)m * ldo + n, v);
}

static int sk_sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}
// Over how many blocks the inner dimension of an [N, K] matrix is shared out: enough for about four
// blocks per SM, at most one per chunk of x, and among those counts the one whose longest share
// of chunks is shortest.
extern "C" int bn_linear_skinny_splits(int N, int K) {
  if (N <= 0 || K <= 0) return 1;
  const int blocks = (N + SK_WARPS * SK_COLS - 1) / (SK_WARPS * SK_COLS), chunks = (K + SK_KC - 1) / SK_KC;
  int want = (4 * sk_sm_count() + blocks - 1) / blocks;
  if (want > chunks) want = chunks;
  if (want <= 1) return 1;
  int best = want;
  for (int s = want; s <= chunks && s <= 2 * want; ++s)
    if ((chunks + s - 1) / s < (chunks + best - 1) / best) best = s;
  return best;
}

// x and w share the element type `dtype`; K must be a multiple of 8 (16-byte rows).  partial: float32
// scratch of bn_linear_skinny_splits(N, K) * M * N floats (not used when that is 1).
extern "C" int bn_linear_skinny(const void* x, const void* w, int dtype, void* out, int out_dtype, int M, int N,
                                int K, int ldo, float* partial, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return BN_OK;
  if (K <= 0 || K % 8 || ldo < N) return BN_ERR_BAD_ARG;
  const int splits = bn_linear_skinny_splits(N, K);
  if (splits > 1 && !partial) return BN_ERR_BAD_ARG;
  dim3 grid((unsigned)((N + SK_WARPS * SK_COLS - 1) / (SK_WARPS * SK_COLS)), (unsigned)splits);
  if (dtype == BN_F32)
    BN_LAUNCH((linear_skinny_kernel<float>), grid, SK_WARPS * 32, 0, stream, (const float*)x, (const float*)w, out,
              out_dtype, M, N, K, ldo, partial);
  else if (dtype == BN_BF16)
    BN_LAUNCH((linear_skinny_kernel<__nv_bfloat16>), grid, SK_WARPS * 32, 0, stream,
              (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, out, out_dtype, M, N, K, ldo, partial);
  else
    return BN_ERR_BAD_ARG;
  if (splits > 1) {
    const size_t total = (size_t)M * N;
    BN_LAUNCH(linear_skinny_sum_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, (const float*)partial, splits, out,
              out_dtype, M, N, ldo);
  }
  BN_CHECK_LAUNCH();
  return BN_OK;
}
