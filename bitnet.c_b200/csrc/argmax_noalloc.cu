// bn_argmax_noalloc: the two-stage argmax of sampling.cu with its scratch in a fixed array of
// this library instead of memory the caller allocates.  See argmax_noalloc.h for who needs
// this, the limits and the rules; nothing in the reference corresponds to it.
//
// The kernel is the same as the normal one: 64 blocks scan a row of logits, each leaves its
// (value, index) in the scratch, and the block that draws the row's last ticket reduces the 64
// and writes the result; lower index wins among equal values.
#include "argmax_noalloc.h"
#include <math.h>
#include <stdint.h>
#include <mutex>

#define NA_BLOCKS 64  // blocks per row
#define NA_MAX_DEVICES 64

struct NaScratch {
  float part_v[BN_ARGMAX_NOALLOC_MAX_ROWS * NA_BLOCKS];  // 64 KB
  int part_i[BN_ARGMAX_NOALLOC_MAX_ROWS * NA_BLOCKS];    // 64 KB
  int tickets[BN_ARGMAX_NOALLOC_MAX_ROWS];               // 1 KB, must be zero when a call starts
};

// One copy per GPU that loads the library, for the life of the process.  In host code this name
// is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) NaScratch g_scratch;

__device__ __forceinline__ bool na_better(float v, int i, float best, int bi) {
  return bi == 0x7fffffff || (i != 0x7fffffff && (v > best || (v == best && i < bi)));
}

__global__ void argmax_noalloc_kernel(const float* __restrict__ logits, int ld, int vocab, int* __restrict__ out,
                                      NaScratch* __restrict__ scratch) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ int s_last;
  const int r = blockIdx.x, nb = gridDim.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* l = logits + (size_t)r * ld;
  const int per = (vocab + nb - 1) / nb;
  const int lo = blockIdx.y * per, hi = min(vocab, lo + per);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    float v = l[i];
    if (na_better(v, i, best, bi)) { best = v; bi = i; }
  }
  auto block_reduce = [&]() {
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (na_better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
      int nw = blockDim.x >> 5;
      best = lane < nw ? sv[lane] : -INFINITY;
      bi = lane < nw ? si[lane] : 0x7fffffff;
      for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (na_better(ov, oi, best, bi)) { best = ov; bi = oi; }
      }
    }
    __syncthreads();
  };
  block_reduce();
  if (threadIdx.x == 0) {
    scratch->part_v[r * NA_BLOCKS + blockIdx.y] = best;
    scratch->part_i[r * NA_BLOCKS + blockIdx.y] = bi;
    __threadfence();
    int ticket = atomicAdd(&scratch->tickets[r], 1);
    s_last = (ticket == nb - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  best = -INFINITY;
  bi = 0x7fffffff;
  for (int i = threadIdx.x; i < nb; i += blockDim.x) {
    float v = __ldcg(&scratch->part_v[r * NA_BLOCKS + i]);
    int idx = __ldcg(&scratch->part_i[r * NA_BLOCKS + i]);
    if (na_better(v, idx, best, bi)) { best = v; bi = idx; }
  }
  block_reduce();
  if (threadIdx.x == 0) out[r] = bi == 0x7fffffff ? 0 : bi;
}

// Device address of g_scratch on each device, looked up on the first call there (under the lock:
// two host threads may make their first call at once).
static NaScratch* g_scratch_addr[NA_MAX_DEVICES];
static std::mutex g_setup_lock;

extern "C" int bn_argmax_noalloc(const float* logits, int ld, int n_rows, int vocab, int* out, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (!logits || !out || vocab <= 0 || ld < vocab) return 1;
  if (n_rows > BN_ARGMAX_NOALLOC_MAX_ROWS) return BN_ARGMAX_NOALLOC_TOO_MANY_ROWS;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NA_MAX_DEVICES) return BN_ARGMAX_NOALLOC_NO_DEVICE_ADDRESS;
  // the scratch used is the current device's copy: the logits must live there too (asking where a
  // pointer lives allocates nothing)
  cudaPointerAttributes where;
  if (cudaPointerGetAttributes(&where, logits) != cudaSuccess) { cudaGetLastError(); return 1; }
  if (where.type == cudaMemoryTypeDevice && where.device != dev) return BN_ARGMAX_NOALLOC_WRONG_DEVICE;
  NaScratch* scratch;
  {
    std::lock_guard<std::mutex> hold(g_setup_lock);
    scratch = g_scratch_addr[dev];
    if (!scratch) {
      // set-up, once per device, with that device current: the symbol's address on this device
      void* p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, g_scratch);
      if (e != cudaSuccess || !p) return BN_ARGMAX_NOALLOC_NO_DEVICE_ADDRESS;
      scratch = g_scratch_addr[dev] = (NaScratch*)p;
    }
  }
  // the array keeps the last call's contents; the tickets must start at zero
  cudaError_t e = cudaMemsetAsync(scratch->tickets, 0, sizeof(int) * n_rows, stream);
  if (e != cudaSuccess) return 100 + (int)e;
  int nb = vocab >= 8192 ? NA_BLOCKS : 1;
  argmax_noalloc_kernel<<<dim3(n_rows, nb), 256, 0, stream>>>(logits, ld, vocab, out, scratch);
  e = cudaGetLastError();
  if (e != cudaSuccess) return 100 + (int)e;
  return 0;
}
