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

// f(value, index) for every element of a row, the block's threads striding over it; 16-byte loads
// where the row allows them, so that a thread has several loads in flight (one block reads a whole
// row of the vocabulary, and what it waits for is the memory's latency).
template <class F>
__device__ __forceinline__ void row_for_each(const float* p, int n, F f) {  // (p may have been written by this kernel)
  const int nv = ((((uintptr_t)p) & 15) == 0) ? (n >> 2) : 0;
  const float4* p4 = reinterpret_cast<const float4*>(p);
#pragma unroll 4
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const float4 v = p4[i];
    f(v.x, 4 * i); f(v.y, 4 * i + 1); f(v.z, 4 * i + 2); f(v.w, 4 * i + 3);
  }
  for (int i = 4 * nv + threadIdx.x; i < n; i += blockDim.x) f(p[i], i);
}

// `index` (may be null) maps a row of logits to its row of sampler state: sequences leave a
// batch at different times, their state rows stay where they are.
__global__ void repeat_penalty_kernel(float* __restrict__ logits, int ld, int vocab,
                                      const int* __restrict__ recent, int recent_stride,
                                      const int* __restrict__ recent_len, const int* __restrict__ index,
                                      float penalty) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  int r = blockIdx.x;
  int sr = index ? index[r] : r;
  const int* ids = recent + (size_t)sr * recent_stride;
  int n = min(recent_len[sr], recent_stride);
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
                                 int recent_stride, const int* recent_len, const int* index, float penalty,
                                 cudaStream_t stream) {
  if (n_rows <= 0 || recent_stride <= 0) return BN_OK;
  BN_LAUNCH(repeat_penalty_kernel, n_rows, 64, 0, stream, logits, ld, vocab, recent, recent_stride, recent_len, index,
                                                  penalty);
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// The sampler's window of recent tokens is a ring (src/sampler.c:54-59): write at recent_pos,
// advance it, grow recent_len up to the window.
__global__ void accept_kernel(int* __restrict__ recent, int recent_stride, int* __restrict__ recent_len,
                              int* __restrict__ recent_pos, const int* __restrict__ index,
                              const int* __restrict__ tokens, int n_rows) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n_rows) return;
  int sr = index ? index[r] : r;
  int pos = recent_pos[sr];
  recent[(size_t)sr * recent_stride + pos] = tokens[r];
  recent_pos[sr] = (pos + 1) % recent_stride;
  if (recent_len[sr] < recent_stride) recent_len[sr] += 1;
}

extern "C" int bn_sampler_accept(int* recent, int recent_stride, int* recent_len, int* recent_pos,
                                 const int* index, const int* tokens, int n_rows, cudaStream_t stream) {
  if (n_rows <= 0 || recent_stride <= 0) return BN_OK;
  BN_LAUNCH(accept_kernel, (n_rows + 127) / 128, 128, 0, stream, recent, recent_stride, recent_len, recent_pos, index,
                                                         tokens, n_rows);
  BN_CHECK_LAUNCH();
  return BN_OK;
}

#define ARGMAX_BLOCKS 64  // blocks per row: a row of 128k logits is scanned by 64 SMs at once

__device__ __forceinline__ bool argmax_better(float v, int i, float best, int bi) {
  // larger value wins; on equal values the lower index (src/gpu_cuda.cu:9013-9018)
  return bi == 0x7fffffff || (i != 0x7fffffff && (v > best || (v == best && i < bi)));
}

// Each block reduces its slice of a row to (value, index) in part_v / part_i; the block that
// draws the last ticket of the row reduces the row's slices and writes the result.
__global__ void argmax_kernel(const float* __restrict__ logits, int ld, int vocab, int* __restrict__ out,
                              float* __restrict__ part_v, int* __restrict__ part_i, int* __restrict__ tickets) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ int s_last;
  const int r = blockIdx.x, nb = gridDim.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* l = logits + (size_t)r * ld;
  const int per = (((vocab + nb - 1) / nb) + 3) & ~3;  // a multiple of four: 16-byte loads where the row allows
  const int lo = min(vocab, (int)blockIdx.y * per), hi = min(vocab, lo + per);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  int i0 = lo;
  if ((((uintptr_t)(l + lo)) & 15) == 0) {
    const int nv = (hi - lo) >> 2;
    for (int q = threadIdx.x; q < nv; q += blockDim.x) {
      const float4 v = *reinterpret_cast<const float4*>(l + lo + 4 * q);
      const int i = lo + 4 * q;
      if (argmax_better(v.x, i, best, bi)) { best = v.x; bi = i; }
      if (argmax_better(v.y, i + 1, best, bi)) { best = v.y; bi = i + 1; }
      if (argmax_better(v.z, i + 2, best, bi)) { best = v.z; bi = i + 2; }
      if (argmax_better(v.w, i + 3, best, bi)) { best = v.w; bi = i + 3; }
    }
    i0 = lo + 4 * nv;
  }
  for (int i = i0 + threadIdx.x; i < hi; i += blockDim.x) {
    float v = l[i];
    if (argmax_better(v, i, best, bi)) { best = v; bi = i; }
  }
  auto block_reduce = [&]() {
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (argmax_better(ov, oi, best, bi)) { best = ov; bi = oi; }
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
        if (argmax_better(ov, oi, best, bi)) { best = ov; bi = oi; }
      }
    }
    __syncthreads();
  };
  block_reduce();
  if (threadIdx.x == 0) {
    part_v[(size_t)r * nb + blockIdx.y] = best;
    part_i[(size_t)r * nb + blockIdx.y] = bi;
    __threadfence();
    int ticket = atomicAdd(tickets + r, 1);
    s_last = (ticket == nb - 1);
    if (s_last) tickets[r] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  best = -INFINITY;
  bi = 0x7fffffff;
  for (int i = threadIdx.x; i < nb; i += blockDim.x) {
    float v = __ldcg(part_v + (size_t)r * nb + i);
    int idx = __ldcg(part_i + (size_t)r * nb + i);
    if (argmax_better(v, idx, best, bi)) { best = v; bi = idx; }
  }
  block_reduce();
  if (threadIdx.x == 0) out[r] = bi == 0x7fffffff ? 0 : bi;
}

// part_v / part_i: scratch of n_rows * 64 entries; tickets: n_rows ints, zero before and after.
extern "C" int bn_argmax(const float* logits, int ld, int n_rows, int vocab, int* out, float* part_v, int* part_i,
                         int* tickets, cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (vocab <= 0 || !part_v || !part_i || !tickets) return BN_ERR_BAD_ARG;
  int nb = vocab >= 8192 ? ARGMAX_BLOCKS : 1;
  BN_LAUNCH(argmax_kernel, dim3(n_rows, nb), 256, 0, stream, logits, ld, vocab, out, part_v, part_i, tickets);
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// One block per row.  Each thread owns a contiguous run of the vocabulary so that the
// cumulative distribution is walked in index order.
__global__ void __launch_bounds__(SAMPLE_THREADS) sample_temperature_kernel(const float* __restrict__ logits, int ld, int vocab, float temperature,
                                          unsigned long long* __restrict__ rng, const int* __restrict__ index,
                                          int* __restrict__ out) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  __shared__ float scratch[32];
  __shared__ float tsum[SAMPLE_THREADS];
  __shared__ float r_shared;
  __shared__ int pick;
  int row = blockIdx.x;
  const float* l = logits + (size_t)row * ld;
  const int per = (((vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS) + 3) & ~3;  // a multiple of four
  const int lo = min(vocab, (int)threadIdx.x * per), hi = min(vocab, lo + per);
  float m = -INFINITY;
  row_for_each(l, vocab, [&](float x, int) { m = fmaxf(m, x / temperature); });
  m = block_max(m, scratch);
  float s = 0.f;
  row_for_each(l, vocab, [&](float x, int) { s += expf(x / temperature - m); });
  s = block_sum(s, scratch);
  // the mass of this thread's run, then the mass before it (runs in index order)
  float local = 0.f;
  if ((((uintptr_t)l) & 15) == 0) {
    int i = lo;
    for (; i + 4 <= hi; i += 4) {
      const float4 v = *reinterpret_cast<const float4*>(l + i);
      local += expf(v.x / temperature - m) / s;
      local += expf(v.y / temperature - m) / s;
      local += expf(v.z / temperature - m) / s;
      local += expf(v.w / temperature - m) / s;
    }
    for (; i < hi; ++i) local += expf(l[i] / temperature - m) / s;
  } else {
    for (int i = lo; i < hi; ++i) local += expf(l[i] / temperature - m) / s;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    float t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) tsum[warp] = incl;
  if (threadIdx.x == 0) {
    r_shared = rng_next_float(rng + (index ? index[row] : row));
    pick = vocab - 1;  // if rounding leaves the whole sum below r
  }
  __syncthreads();
  // running sums at the borders of the runs: a run's start is, bit for bit, the end of the run before it
  float warp_off = 0.f;
  for (int w = 0; w < warp; ++w) warp_off += tsum[w];
  float prev = __shfl_up_sync(0xffffffffu, incl, 1);
  if (lane == 0) prev = 0.f;
  const float before = warp_off + prev, end = warp_off + incl;
  // the one thread whose run takes the running sum past r walks it
  const float r = r_shared;
  const bool last_run = hi >= vocab;
  if (lo < hi && !(r < before) && (r < end || last_run)) {
    float cdf = before;
    int got = -1;
    for (int i = lo; i < hi; ++i) {
      cdf += expf(l[i] / temperature - m) / s;
      if (r < cdf) { got = i; break; }
    }
    if (got < 0) got = min(vocab - 1, hi);  // rounding pushed it past this run
    pick = got;
  }
  __syncthreads();
  if (threadIdx.x == 0) out[row] = pick;
}

extern "C" int bn_sample_temperature(const float* logits, int ld, int n_rows, int vocab, float temperature,
                                     unsigned long long* rng, const int* index, int* out, cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (vocab <= 0 || !(temperature > 0.f)) return BN_ERR_BAD_ARG;
  BN_LAUNCH(sample_temperature_kernel, n_rows, SAMPLE_THREADS, 0, stream, logits, ld, vocab, temperature, rng, index, out);
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// ---- nucleus (top-p) sampling -----------------------------------------------------------------
// Reference (src/sampler.c:95-135): keep tokens with p >= (1 - topp) / (n - 1), sort them by
// falling probability, cut after the first whose running sum exceeds topp, draw
// r = rng_float() * that sum and take the first token whose running sum exceeds r.
// Both cuts are "the first token, in sorted order, whose running sum exceeds a threshold".
// Instead of sorting, the kernel bisects on the probability value: with
// F(x) = sum of candidates with p >= x, the wanted token has the largest p with F(p) > threshold;
// among tokens of exactly that probability the lower index comes first.  Sums are double.

__device__ __forceinline__ double block_sum_double(double v, double* scratch) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  double r = (threadIdx.x < nwarp) ? scratch[threadIdx.x] : 0.0;
  if (warp == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    if (lane == 0) scratch[0] = r;
  }
  __syncthreads();
  return scratch[0];
}

// Sum of p[i] over candidates (p >= cutoff) whose bit pattern is >= key.  Probabilities are
// non-negative floats, so their bit patterns order like their values.
__device__ double mass_at_least(const float* p, int n, unsigned cutoff_bits, unsigned key, double* scratch) {
  double s = 0.0;
  unsigned k = max(key, cutoff_bits);
  row_for_each(p, n, [&](float v, int) {
    if (__float_as_uint(v) >= k) s += (double)v;
  });
  return block_sum_double(s, scratch);
}

// Masses in fixed point: p * 2^62 as an integer is exact for every float p >= 2^-38 (the cut-off
// (1 - topp) / (n - 1) is far above that), the whole mass fits 64 bits, and integer sums do not
// depend on the order of the additions, so shared-memory atomics may do them.
#define NUC_ONE 4611686018427387904.0  // 2^62
__device__ __forceinline__ unsigned long long nuc_fixed(float v) { return (unsigned long long)((double)v * NUC_ONE); }

// For every thread the sum of v over the threads behind it (higher index); *total the sum over all.
__device__ unsigned long long block_suffix_exclusive(unsigned long long v, unsigned long long* warp_tot,
                                                     unsigned long long* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  unsigned long long s = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    unsigned long long t = __shfl_down_sync(0xffffffffu, s, o);
    if (lane + o < 32) s += t;
  }
  __syncthreads();
  if (lane == 0) warp_tot[warp] = s;
  __syncthreads();
  unsigned long long behind = 0, all = 0;
  for (int w = 0; w < nwarp; ++w) {
    unsigned long long t = warp_tot[w];
    all += t;
    if (w > warp) behind += t;
  }
  *total = all;
  return (s - v) + behind;
}

// One level of the search for the key: among the candidates whose bits agree with `prefix` under
// `mask`, the masses of the 2^nbits values of the next bits (from `shift` up) go into hist; the
// result is the largest such value whose mass, together with everything above it (`above` on
// entry: the mass above the prefix), exceeds thr, and the mass above that value.  *total is the
// mass of all candidates under the prefix plus `above`.
__device__ unsigned nucleus_level(const float* p, int n, unsigned cutoff_bits, unsigned mask, unsigned prefix, int shift,
                                  int nbits, unsigned long long above, unsigned long long thr, unsigned long long* hist,
                                  unsigned long long* warp_tot, unsigned long long* above_out, unsigned long long* total) {
  __shared__ unsigned s_bin;
  __shared__ unsigned long long s_above;
  const int bins = 1 << nbits;
  for (int i = threadIdx.x; i < bins; i += blockDim.x) hist[i] = 0ull;
  if (threadIdx.x == 0) { s_bin = 0u; s_above = above; }
  __syncthreads();
  row_for_each(p, n, [&](float v, int) {
    const unsigned b = __float_as_uint(v);
    if (b >= cutoff_bits && (b & mask) == prefix) atomicAdd(&hist[(b >> shift) & (unsigned)(bins - 1)], nuc_fixed(v));
  });
  __syncthreads();
  // each thread owns a run of bins; runs of higher bins belong to higher threads
  const int per = (bins + (int)blockDim.x - 1) / (int)blockDim.x;
  const int b0 = (int)threadIdx.x * per, b1 = min(bins, b0 + per);
  unsigned long long mine = 0;
  for (int b = b0; b < b1; ++b) mine += hist[b];
  unsigned long long all;
  const unsigned long long behind = above + block_suffix_exclusive(mine, warp_tot, &all);
  *total = above + all;
  if (behind <= thr && behind + mine > thr) {  // the crossing lies in this thread's run (at most one thread)
    unsigned long long run = behind;
    for (int b = b1 - 1; b >= b0; --b) {
      if (run + hist[b] > thr) { s_bin = (unsigned)b; s_above = run; break; }
      run += hist[b];
    }
  }
  __syncthreads();
  *above_out = s_above;
  return s_bin;
}

// First token in (falling p, rising index) order whose running sum exceeds thr; *cum_out is that
// running sum.  If none exceeds it, the last candidate in that order and the whole mass.  The key
// (the wanted token's probability as bits) is found 12, 12 and 8 bits at a time.
__device__ int nucleus_first_exceeding(const float* p, int n, unsigned cutoff_bits, unsigned max_bits, double thr,
                                       double* cum_out, double* dscratch, int* iscratch, unsigned long long* hist,
                                       unsigned long long* warp_tot) {
  (void)max_bits;
  const unsigned long long thr_fx = thr <= 0.0 ? 0ull : (thr >= 2.0 ? (unsigned long long)(2.0 * NUC_ONE) : (unsigned long long)(thr * NUC_ONE));
  unsigned long long above_fx = 0, total_fx = 0, dummy;
  unsigned lo = nucleus_level(p, n, cutoff_bits, 0u, 0u, 20, 12, 0ull, thr_fx, hist, warp_tot, &above_fx, &total_fx) << 20;
  const bool none = !(total_fx > thr_fx);
  const double total = (double)total_fx / NUC_ONE;
  if (!none) {
    lo |= nucleus_level(p, n, cutoff_bits, 0xFFF00000u, lo, 8, 12, above_fx, thr_fx, hist, warp_tot, &above_fx, &dummy) << 8;
    lo |= nucleus_level(p, n, cutoff_bits, 0xFFFFFF00u, lo, 0, 8, above_fx, thr_fx, hist, warp_tot, &above_fx, &dummy);
  }
  // `lo` is now the probability (as bits) of the wanted token, or, if none exceeds thr, the
  // cut-off: then the smallest candidate probability is looked up and its last index taken.
  __shared__ unsigned s_key;
  if (none) {
    unsigned best = 0xffffffffu;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      unsigned b = __float_as_uint(p[i]);
      if (b >= cutoff_bits) best = min(best, b);
    }
    for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) iscratch[threadIdx.x >> 5] = (int)best;
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned b = 0xffffffffu;
      for (int w = 0; w < (int)((blockDim.x + 31) >> 5); ++w) b = min(b, (unsigned)iscratch[w]);
      s_key = b;
    }
    __syncthreads();
    lo = s_key;
  }
  double above = none ? ((lo == 0xffffffffu) ? 0.0 : mass_at_least(p, n, cutoff_bits, lo + 1, dscratch))
                      : (double)above_fx / NUC_ONE;
  float pv = __uint_as_float(lo);
  // how many tokens of probability pv are needed: the k-th (1-based) in index order
  __shared__ int s_k;
  __shared__ double s_cum;
  __shared__ int s_pick;
  // count the ties: every thread owns a contiguous run of the vocabulary
  int mine = 0;
  const int per = (((n + blockDim.x - 1) / blockDim.x) + 3) & ~3;  // a multiple of four
  const int a = min(n, (int)threadIdx.x * per), b = min(n, a + per);
  if ((((uintptr_t)p) & 15) == 0) {
    int i = a;
    for (; i + 4 <= b; i += 4) {
      const float4 v = *reinterpret_cast<const float4*>(p + i);
      mine += (__float_as_uint(v.x) == lo) + (__float_as_uint(v.y) == lo) + (__float_as_uint(v.z) == lo) +
              (__float_as_uint(v.w) == lo);
    }
    for (; i < b; ++i) mine += (__float_as_uint(p[i]) == lo);
  } else {
    for (int i = a; i < b; ++i) mine += (__float_as_uint(p[i]) == lo);
  }
  // ties before this thread's run, and all of them
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  int incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  __syncthreads();
  if (lane == 31) iscratch[warp] = incl;
  __syncthreads();
  int before = incl - mine, ties = 0;
  for (int w = 0; w < nwarp; ++w) {
    int t = iscratch[w];
    ties += t;
    if (w < warp) before += t;
  }
  if (threadIdx.x == 0) {
    int k = ties;  // none exceeds: the last of them
    double cum = total;
    if (!none) {
      // the smallest j with above + j * pv > thr
      double j0 = floor((thr - above) / (double)pv);
      int j = (int)fmin(fmax(j0, 0.0), (double)ties);
      while (j > 1 && above + (double)(j - 1) * (double)pv > thr) --j;
      while (j < ties && !(above + (double)j * (double)pv > thr)) ++j;
      k = max(1, min(j, ties));
      cum = above + (double)k * (double)pv;
    }
    s_k = k;
    s_cum = cum;
    s_pick = max(0, n - 1);
  }
  __syncthreads();
  const int k = s_k;
  *cum_out = s_cum;
  // the thread whose run holds the k-th tie finds it
  if (before < k && k <= before + mine) {
    int seen = before;
    for (int i = a; i < b; ++i) {
      if (__float_as_uint(p[i]) == lo && ++seen == k) { s_pick = i; break; }
    }
  }
  __syncthreads();
  return s_pick;
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_topp_kernel(const float* __restrict__ logits, int ld, int vocab, float temperature,
                                   float topp, unsigned long long* __restrict__ rng, const int* __restrict__ index,
                                   float* __restrict__ probs, int* __restrict__ out) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  __shared__ float scratch[32];
  __shared__ double dscratch[32];
  __shared__ int iscratch[SAMPLE_THREADS];
  __shared__ float r_shared;
  __shared__ unsigned long long hist[4096];
  __shared__ unsigned long long warp_tot[32];
  int row = blockIdx.x;
  const float* l = logits + (size_t)row * ld;
  float* p = probs + (size_t)row * vocab;
  float m = -INFINITY;
  row_for_each(l, vocab, [&](float x, int) { m = fmaxf(m, x / temperature); });
  m = block_max(m, scratch);
  float s = 0.f;
  row_for_each(l, vocab, [&](float x, int) { s += expf(x / temperature - m); });
  s = block_sum(s, scratch);
  float pmax = 0.f;
  row_for_each(l, vocab, [&](float x, int i) {
    float v = expf(x / temperature - m) / s;
    p[i] = v;
    pmax = fmaxf(pmax, v);
  });
  pmax = block_max(pmax, scratch);  // also orders the writes of p before the reads below
  if (threadIdx.x == 0) r_shared = rng_next_float(rng + (index ? index[row] : row));
  __syncthreads();
  if (vocab == 1) {
    if (threadIdx.x == 0) out[row] = 0;
    return;
  }
  float cutoff = (1.0f - topp) / (float)(vocab - 1);
  unsigned cutoff_bits = __float_as_uint(fmaxf(cutoff, 0.f));
  unsigned max_bits = __float_as_uint(pmax);
  double cumulative, c2;
  int last = nucleus_first_exceeding(p, vocab, cutoff_bits, max_bits, (double)topp, &cumulative, dscratch, iscratch, hist,
                                     warp_tot);
  float r = r_shared * (float)cumulative;
  int pick = nucleus_first_exceeding(p, vocab, cutoff_bits, max_bits, (double)r, &c2, dscratch, iscratch, hist, warp_tot);
  if (threadIdx.x == 0) out[row] = (c2 > cumulative) ? last : pick;
}

// probs: scratch of n_rows * vocab floats.
extern "C" int bn_sample_topp(const float* logits, int ld, int n_rows, int vocab, float temperature, float topp,
                              unsigned long long* rng, const int* index, float* probs, int* out,
                              cudaStream_t stream) {
  if (n_rows <= 0) return BN_OK;
  if (vocab <= 0 || !(temperature > 0.f) || !(topp > 0.f && topp < 1.f) || !probs) return BN_ERR_BAD_ARG;
  BN_LAUNCH(sample_topp_kernel, n_rows, SAMPLE_THREADS, 0, stream, logits, ld, vocab, temperature, topp, rng, index, probs,
                                                           out);
  BN_CHECK_LAUNCH();
  return BN_OK;
}
