// out[M, N] = x[M, K] . W[N, K]^T in bfloat16 for M <= 64: the decode-time projections.
//
// The step is bound by reading W once from HBM, so the kernel is built around that stream:
// every thread pulls 16-byte pieces of two weight rows straight from global memory into
// registers, one chunk of K ahead of the arithmetic, with no shared-memory stage for W; the
// few rows of x are staged in shared memory (cp.async, double buffered) and shared by the
// four warps of a block.  The products run on the tensor cores as m16n8k16 with the roles
// swapped: 16 weight rows are the "M" side and 8 rows of x the "N" side, so a batch of 1 to 64
// costs 1 to 8 instructions per 16x16 piece of W.  Accumulation is float32.
//
// A 16-byte piece holds 8 consecutive k.  Thread (g, t) of a warp takes k = 8t..8t+7 of a
// 32-wide chunk for weight rows g and g+8 and for x row g, and feeds them to two MMAs; the
// same permutation of k on both operands leaves the dot products unchanged.
//
// Epilogues: (0) store; (1) float32 partial sums per K-split, summed by the kernel that adds
// them to the residual (norm.cu); (2) SwiGLU for a weight whose rows alternate 8 gate rows and
// 8 up rows, so that one thread holds gate_i and up_i of the same i.
//
// A weight with few rows gives too few blocks to keep enough loads in flight, so K may be split
// over gridDim.y for modes 0 and 2 as well: every block writes its float32 partial tile to
// scratch, and the block that arrives last at the tile's counter (an atomic ticket, no waiting)
// adds the partials up in split order and runs the epilogue.  The order of the additions is
// fixed, so the result does not depend on which block came last.
// Reference for the operation: y = W x with float32 accumulation (src/quant/bf16_scalar.c:4-21);
// its decode path is a warp-per-row matvec (src/gpu_cuda.cu:3995) and a fused gate/up + SiLU
// kernel (src/gpu_cuda.cu:4547).
#include "mma.cuh"

#define LM_KC 128                 // k per stage
#define LM_XS_STRIDE (LM_KC + 32) // bf16 elements per staged row of x: 320 bytes, conflict-free 16-byte reads
#define LM_ROWS 64                // weight rows per block (4 warps x 16)

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

struct LmArgs {
  const __nv_bfloat16* x;
  const __nv_bfloat16* w;
  void* out;
  int out_dtype;  // for mode 0 and 2
  int M, N, K;
  int k_per_split;  // multiple of LM_KC
  int mode;         // 0 store, 1 partial, 2 swiglu
  int ldo;
  float* scratch;   // modes 0/2 with gridDim.y > 1: [splits][row blocks][64 rows][8*NT] partial tiles
  int* counters;    // one ticket counter per row block, zero before and after the launch
};

template <int NT>
__global__ void __launch_bounds__(128) linear_mma_kernel(LmArgs a) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [2][NT*8][LM_XS_STRIDE]
  constexpr int MP = NT * 8;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * LM_ROWS + warp * 16;
  const int ks = blockIdx.y * a.k_per_split;
  const int ke = min(a.K, ks + a.k_per_split);
  const int n_chunks = (ke - ks + LM_KC - 1) / LM_KC;
  const int r_lo = min(row0 + g, a.N - 1), r_hi = min(row0 + g + 8, a.N - 1);
  const __nv_bfloat16* w_lo = a.w + (size_t)r_lo * a.K;
  const __nv_bfloat16* w_hi = a.w + (size_t)r_hi * a.K;

  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  auto stage_x = [&](int chunk, int buf) {
    // MP rows x 16 pieces of 16 bytes
    int k0 = ks + chunk * LM_KC;
    __nv_bfloat16* dst = xs + (size_t)buf * MP * LM_XS_STRIDE;
    for (int p = tid; p < MP * (LM_KC / 8); p += 128) {
      int r = p / (LM_KC / 8), c = (p % (LM_KC / 8)) * 8;
      bool ok = r < a.M && k0 + c < ke;
      const __nv_bfloat16* src = ok ? a.x + (size_t)r * a.K + k0 + c : a.x;
      cp_async16(dst + (size_t)r * LM_XS_STRIDE + c, src, ok);
    }
    cp_async_commit();
  };
  auto load_w = [&](int chunk, uint4 (&lo)[4], uint4 (&hi)[4]) {
    int k0 = ks + chunk * LM_KC + t * 8;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      int k = k0 + s * 32;
      if (k < ke) {
        lo[s] = ldg_stream(w_lo + k);
        hi[s] = ldg_stream(w_hi + k);
      } else {
        lo[s] = make_uint4(0, 0, 0, 0);
        hi[s] = make_uint4(0, 0, 0, 0);
      }
    }
  };

  uint4 wlo[2][4], whi[2][4];
  if (n_chunks > 0) {
    stage_x(0, 0);
    load_w(0, wlo[0], whi[0]);
  }
#pragma unroll 1
  for (int c = 0; c < n_chunks; c += 2) {
    // two chunks per trip so that the register buffers are indexed by constants
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int cc = c + h;
      if (cc >= n_chunks) break;
      if (cc + 1 < n_chunks) {
        stage_x(cc + 1, (h + 1) & 1);
        load_w(cc + 1, wlo[(h + 1) & 1], whi[(h + 1) & 1]);
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      const __nv_bfloat16* xb = xs + (size_t)h * MP * LM_XS_STRIDE;
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        uint4 lo = wlo[h][s], hi = whi[h][s];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          uint4 xv = *reinterpret_cast<const uint4*>(xb + (size_t)(nt * 8 + g) * LM_XS_STRIDE + s * 32 + t * 8);
          mma_bf16(acc[nt], lo.x, hi.x, lo.y, hi.y, xv.x, xv.y);
          mma_bf16(acc[nt], lo.z, hi.z, lo.w, hi.w, xv.z, xv.w);
        }
      }
      __syncthreads();
    }
  }

  // c0: (row g, m 2t)  c1: (row g, m 2t+1)  c2: (row g+8, m 2t)  c3: (row g+8, m 2t+1)
  const int n_lo = row0 + g, n_hi = row0 + g + 8;
  if (a.mode != 1 && gridDim.y > 1) {
    __shared__ int s_last;
    const size_t tile_floats = (size_t)LM_ROWS * MP;
    float* mine = a.scratch + ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * tile_floats;
    // element (row r of the block, column m) of this thread's fragment lives at r * MP + m
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      int m = nt * 8 + 2 * t;
      *reinterpret_cast<float2*>(mine + (size_t)(warp * 16 + g) * MP + m) = make_float2(acc[nt][0], acc[nt][1]);
      *reinterpret_cast<float2*>(mine + (size_t)(warp * 16 + g + 8) * MP + m) = make_float2(acc[nt][2], acc[nt][3]);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      int ticket = atomicAdd(a.counters + blockIdx.x, 1);
      s_last = (ticket == (int)gridDim.y - 1);
      if (s_last) a.counters[blockIdx.x] = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    for (int sp = 0; sp < (int)gridDim.y; ++sp) {
      const float* part = a.scratch + ((size_t)sp * gridDim.x + blockIdx.x) * tile_floats;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        int m = nt * 8 + 2 * t;
        float2 lo = __ldcg(reinterpret_cast<const float2*>(part + (size_t)(warp * 16 + g) * MP + m));
        float2 hi = __ldcg(reinterpret_cast<const float2*>(part + (size_t)(warp * 16 + g + 8) * MP + m));
        acc[nt][0] += lo.x; acc[nt][1] += lo.y; acc[nt][2] += hi.x; acc[nt][3] += hi.y;
      }
    }
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      int m = nt * 8 + 2 * t + j;
      if (m >= a.M) continue;
      float v_lo = acc[nt][j], v_hi = acc[nt][2 + j];
      if (a.mode == 0) {
        if (n_lo < a.N) store_from_f32(a.out, a.out_dtype, (size_t)m * a.ldo + n_lo, v_lo);
        if (n_hi < a.N) store_from_f32(a.out, a.out_dtype, (size_t)m * a.ldo + n_hi, v_hi);
      } else if (a.mode == 1) {
        float* part = (float*)a.out + ((size_t)blockIdx.y * a.M + m) * a.N;
        if (n_lo < a.N) part[n_lo] = v_lo;
        if (n_hi < a.N) part[n_hi] = v_hi;
      } else {
        // rows [16j, 16j+8) are gate rows 8j.., rows [16j+8, 16j+16) the matching up rows
        int i = (row0 >> 4) * 8 + g;
        if (n_hi < a.N) {
          float s = v_lo / (1.0f + expf(-v_lo));
          store_from_f32(a.out, a.out_dtype, (size_t)m * a.ldo + i, s * v_hi);
        }
      }
    }
  }
}

// x [M, K], w [N, K] bfloat16.  mode 0: out [M, ldo] of out_dtype.  mode 1: out is float32
// [n_splits, M, N] (every split writes its whole slice).  mode 2: w has N = 2 I rows in blocks
// of 8 gate / 8 up rows, out [M, ldo] holds silu(gate) * up for I columns.
// With n_splits > 1 in modes 0 and 2, scratch must hold n_splits * ceil(N/64) * 64 * Mp floats
// (Mp = M rounded up to 8, 16, 32 or 64) and counters ceil(N/64) zeroed ints; both may be
// shared by launches that do not overlap on the device.
extern "C" int bn_linear_mma(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K, int ldo,
                             int mode, int n_splits, float* scratch, long long scratch_floats, int* counters,
                             int n_counters, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return BN_OK;
  if (M > 64 || K <= 0 || K % 8 || n_splits < 1 || mode < 0 || mode > 2) return BN_ERR_BAD_ARG;
  if (mode == 2 && (N % 16)) return BN_ERR_BAD_ARG;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return BN_ERR_BAD_ARG;
  LmArgs a;
  a.x = (const __nv_bfloat16*)x; a.w = (const __nv_bfloat16*)w; a.out = out; a.out_dtype = out_dtype;
  a.M = M; a.N = N; a.K = K; a.mode = mode; a.ldo = ldo; a.scratch = scratch; a.counters = counters;
  int chunks = (K + LM_KC - 1) / LM_KC;
  if (n_splits > chunks) n_splits = chunks;
  a.k_per_split = ((chunks + n_splits - 1) / n_splits) * LM_KC;
  n_splits = (chunks * LM_KC + a.k_per_split - 1) / a.k_per_split;  // no empty split
  int nt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
  int row_blocks = (N + LM_ROWS - 1) / LM_ROWS;
  if (mode != 1 && n_splits > 1) {
    if (!scratch || !counters || n_counters < row_blocks ||
        scratch_floats < (long long)n_splits * row_blocks * LM_ROWS * nt * 8)
      return BN_ERR_BAD_ARG;
  }
  dim3 grid(row_blocks, n_splits);
  size_t smem = (size_t)2 * nt * 8 * LM_XS_STRIDE * sizeof(__nv_bfloat16);
  switch (nt) {
    case 1: linear_mma_kernel<1><<<grid, 128, smem, stream>>>(a); break;
    case 2: linear_mma_kernel<2><<<grid, 128, smem, stream>>>(a); break;
    case 4: linear_mma_kernel<4><<<grid, 128, smem, stream>>>(a); break;
    default: linear_mma_kernel<8><<<grid, 128, smem, stream>>>(a); break;
  }
  BN_CHECK_LAUNCH();
  return BN_OK;
}
