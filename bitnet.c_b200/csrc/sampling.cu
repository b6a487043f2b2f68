// Choosing the next token on the device: argmax, temperature sampling, repeat penalty.
//
// Reference (src/sampler.c:137-173): (1) repeat penalty over the distinct recent ids,
// logit > 0 ? logit / p : logit * p; (2) temperature 0 -> argmax, first maximum wins
// (src/sampler_backend.c:129-135; lower index on ties in src/gpu_cuda.cu:9013-9018);
// (3) else logits / T, softmax with expf, r = rng_float(), first i with r < cdf_i,
// fallback n-1 (src/sampler.c:63-85).  The generator is xorshift64* with the upper 32
// bits of state * 0x2545F4914F6CDD1D, r = (u32 >> 8) / 2^24 (src/sampler.c:6-15).
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ float rng_next_float(unsigned long long* state) {
  unsigned long long s = *state;
  s ^= s >> 12;
  s ^= s << 25;
  s ^= s >> 27;
  *state = s;
  unsigned int u = (unsigned int)((s * 0x2545F4914F6CDD1DULL) >> 32);
  return (float)(u >> 8) / 16777216.0f;
}

__global__ void repeat_penalty_kernel(float* __restrict__ logits, int ld, int vocab,
                                      const int* __restrict__ recent, int recent_stride,
                                      const int* __restrict__ recent_len, float penalty) {
  int r = blockIdx.x;
  const int* ids = recent + (size_t)r * recent_stride;
  int n = min(recent_len[r], recent_stride);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    int tok = ids[i];
    if (tok < 0 || tok >= vocab) continue;
    bool seen = false;
    for (int j = 0; j < i; ++j)
      if (ids[j] == tok) { seen = true; break; }
    if (seen) continue;
    float* l = logits + (size_t)r * ld + tok;
    float v = *l;
    *l = v > 0.f ? v / penalty : v * penalty;
  }
}

extern "C" int bn_repeat_penalty(float* logits, int ld, int n_rows, int vocab, const int* recent,
                                 int recent_stride, const int* recent_len, float penalty, cudaStream_t stream) {
  if (n_rows <= 0 || recent_stride <= 0) return BN_OK;
  repeat_penalty_kernel<<<n_rows, 64, 0, stream>>>(logits, ld, vocab, recent, recent_stride, recent_len, penalty);
  BN_CHECK_LAUNCH();
  return BN_OK;
}

__global__ void argmax_kernel(const float* __restrict__ logits, int ld, int vocab, int* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  int r = blockIdx.x;
  const float* l = logits + (size_t)r * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    float v = l[i];
    if (v > best || (v == best && i < bi) || bi == 0x7fffffff) { best = v; bi = i; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
  }
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
    }
    if (lane == 0) out[r] = bi == 0x7fffffff ? 0 : bi;
  }
}

extern "C" int bn_argmax(const float* logits, int ld, int n_rows, int vocab, int* out, cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (vocab <= 0) return BN_ERR_BAD_ARG;
  argmax_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, ld, vocab, out);
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// One block per row.  Each thread owns a contiguous run of the vocabulary so that the
// cumulative distribution is walked in index order.
__global__ void sample_temperature_kernel(const float* __restrict__ logits, int ld, int vocab, float temperature,
                                          unsigned long long* __restrict__ rng, int* __restrict__ out) {
  __shared__ float scratch[32];
  __shared__ float tsum[SAMPLE_THREADS];
  __shared__ float r_shared;
  __shared__ int pick;
  int row = blockIdx.x;
  const float* l = logits + (size_t)row * ld;
  int per = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  int lo = threadIdx.x * per, hi = min(vocab, lo + per);
  float m = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) m = fmaxf(m, l[i] / temperature);
  m = block_max(m, scratch);
  float s = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) s += expf(l[i] / temperature - m);
  s = block_sum(s, scratch);
  float local = 0.f;
  for (int i = lo; i < hi; ++i) local += expf(l[i] / temperature - m) / s;
  tsum[threadIdx.x] = local;
  if (threadIdx.x == 0) {
    r_shared = rng_next_float(rng + row);
    pick = vocab - 1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // Serial walk over 1024 partial sums: first run whose inclusive sum exceeds r.
    float r = r_shared, cdf = 0.f;
    int owner = -1;
    for (int k = 0; k < SAMPLE_THREADS; ++k) {
      if (r < cdf + tsum[k]) { owner = k; break; }
      cdf += tsum[k];
    }
    if (owner >= 0) {
      int a = owner * per, b = min(vocab, a + per);
      for (int i = a; i < b; ++i) {
        cdf += expf(l[i] / temperature - m) / s;
        if (r < cdf) { pick = i; break; }
        if (i == b - 1) pick = min(vocab - 1, b);  // rounding pushed it past this run
      }
    }
    out[row] = pick;
  }
}

extern "C" int bn_sample_temperature(const float* logits, int ld, int n_rows, int vocab, float temperature,
                                     unsigned long long* rng, int* out, cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (vocab <= 0 || !(temperature > 0.f)) return BN_ERR_BAD_ARG;
  sample_temperature_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, ld, vocab, temperature, rng, out);
  BN_CHECK_LAUNCH();
  return BN_OK;
}
