// Decode attention in bfloat16: one new token per sequence attends over its paged cache.
//
// With one query per sequence there is little work per (sequence, head), and at small batch
// too few (sequence, key/value head) pairs to fill 148 SMs, so the keys of a sequence are split
// into chunks of DEC_CHUNK positions: grid = (sequences, key/value heads x head groups, chunks).
// A block handles the up to 8 query heads that share its key/value head, so every key and
// value row is read once for all of them.  It writes an unnormalised partial result with its
// maximum and sum; a second kernel combines the chunks of a (sequence, head).  Chunk borders
// are multiples of DEC_CHUNK in position, so how a row is summed depends on its own position
// only, never on the batch around it.
//
// Reference: scores = q.k * scale over the causal range, softmax with the maximum subtracted,
// weighted sum of values, query head h uses key/value head h / (H / KV)
// (src/transformer/gqa_scalar.c:61-121); the running maximum/sum form is its flash variant
// (gqa_scalar.c:127-207).  Its CUDA decode kernel is one block per head without a split over
// the keys (src/gpu_cuda.cu:9718).
#include "common.cuh"

#define DEC_THREADS 128
#define DEC_CHUNK 128
#define DEC_GB 8  // query heads per block

__device__ __forceinline__ void bf16x8_to_f32(const uint4& v, float* o) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    o[2 * i] = f.x;
    o[2 * i + 1] = f.y;
  }
}

__global__ void __launch_bounds__(DEC_THREADS)
attention_decode_partial_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, int n_heads, int n_kv_heads,
                                int head_dim, float scale, int window, const int* __restrict__ tok_pos,
                                const int* __restrict__ slots, const int* __restrict__ page_table, int pt_stride,
                                const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                                float* __restrict__ part_o, float* __restrict__ part_ml, int n_splits) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  __shared__ float q_s[DEC_GB * 256];
  __shared__ float p_s[DEC_GB * DEC_CHUNK];
  __shared__ float red[DEC_THREADS * DEC_GB * 8];
  const int b = blockIdx.x, split = blockIdx.z, tid = threadIdx.x;
  const int group = n_heads / n_kv_heads;
  const int gblocks = (group + DEC_GB - 1) / DEC_GB;
  const int kvh = blockIdx.y / gblocks, gb = blockIdx.y % gblocks;
  const int h0 = kvh * group + gb * DEC_GB;
  const int G = min(DEC_GB, group - gb * DEC_GB);
  const int pos = tok_pos[b];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int c0 = split * DEC_CHUNK;
  if (c0 > pos || c0 + DEC_CHUNK <= lo) return;  // no key of this chunk is visible
  const int* pt = page_table + (size_t)slots[b] * pt_stride;
  // a chunk of 128 positions lies in two pages; their ids are fetched once
  const int page_a = pt[c0 / BN_PAGE];
  const int page_b = (c0 + BN_PAGE <= pos) ? pt[c0 / BN_PAGE + 1] : page_a;
  auto row_off = [&](int j) -> size_t {  // row of key/value j of this chunk (0 <= j < 128)
    int page = j < BN_PAGE ? page_a : page_b;
    return (((size_t)page * n_kv_heads + kvh) * BN_PAGE + (j & (BN_PAGE - 1))) * (size_t)head_dim;
  };

  for (int i = tid; i < G * head_dim; i += DEC_THREADS) {
    int g = i / head_dim, d = i - g * head_dim;
    q_s[g * 256 + d] = __bfloat162float(q[(size_t)b * q_stride + (size_t)(h0 + g) * head_dim + d]);
  }
  __syncthreads();

  // ---- scores: one key per thread, all G heads at once
  {
    int p = c0 + tid;
    bool valid = p >= lo && p <= pos;
    float dot[DEC_GB];
#pragma unroll
    for (int g = 0; g < DEC_GB; ++g) dot[g] = 0.f;
    if (valid) {
      const __nv_bfloat16* krow = k_cache + row_off(tid);
      // head_dim is a multiple of 16: two 16-byte loads are issued before either is used
      for (int d = 0; d < head_dim; d += 16) {
        uint4 raw0 = *reinterpret_cast<const uint4*>(krow + d);
        uint4 raw1 = *reinterpret_cast<const uint4*>(krow + d + 8);
        float kf[16];
        bf16x8_to_f32(raw0, kf);
        bf16x8_to_f32(raw1, kf + 8);
#pragma unroll
        for (int g = 0; g < DEC_GB; ++g) {
          if (g < G) {
            const float* qq = q_s + g * 256 + d;
#pragma unroll
            for (int e = 0; e < 16; ++e) dot[g] = fmaf(qq[e], kf[e], dot[g]);
          }
        }
      }
    }
#pragma unroll
    for (int g = 0; g < DEC_GB; ++g)
      if (g < G) p_s[g * DEC_CHUNK + tid] = valid ? dot[g] * scale : -INFINITY;
  }
  __syncthreads();

  // ---- per head: maximum, exponentials, sum (warp w takes heads w, w+4)
  {
    int warp = tid >> 5, lane = tid & 31;
    for (int g = warp; g < G; g += DEC_THREADS / 32) {
      float* ps = p_s + g * DEC_CHUNK;
      float m = -INFINITY;
      for (int j = lane; j < DEC_CHUNK; j += 32) m = fmaxf(m, ps[j]);
      m = warp_max(m);
      float l = 0.f;
      for (int j = lane; j < DEC_CHUNK; j += 32) {
        float e = expf(ps[j] - m);  // exp(-inf) = 0 for keys outside the range
        ps[j] = e;
        l += e;
      }
      l = warp_sum(l);
      if (lane == 0) {
        size_t o = (((size_t)b * n_heads + h0 + g) * n_splits + split) * 2;
        part_ml[o] = m;
        part_ml[o + 1] = l;
      }
    }
  }
  __syncthreads();

  // ---- weighted sum of values: head_dim/8 threads per key, several keys at a time
  const int tpk = head_dim / 8;           // threads per key
  const int kp = DEC_THREADS / tpk;       // keys in flight
  const int kg = tid / tpk, piece = tid - kg * tpk;
  float acc[DEC_GB][8];
#pragma unroll
  for (int g = 0; g < DEC_GB; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
  if (kg < kp) {
    int j_hi = min(DEC_CHUNK, pos - c0 + 1);
    int j_lo = max(0, lo - c0);
    // four value rows are requested before the first is used
    for (int j = j_lo + kg; j < j_hi; j += 4 * kp) {
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        int ju = j + u * kp;
        raw[u] = ju < j_hi ? *reinterpret_cast<const uint4*>(v_cache + row_off(ju) + piece * 8) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        int ju = j + u * kp;
        if (ju >= j_hi) break;
        float vf[8];
        bf16x8_to_f32(raw[u], vf);
#pragma unroll
        for (int g = 0; g < DEC_GB; ++g) {
          if (g < G) {
            float pj = p_s[g * DEC_CHUNK + ju];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(pj, vf[e], acc[g][e]);
          }
        }
      }
    }
    // red[kg][g][piece*8 + e]; one key group holds G*head_dim floats
#pragma unroll
    for (int g = 0; g < DEC_GB; ++g)
      if (g < G)
#pragma unroll
        for (int e = 0; e < 8; ++e) red[((size_t)kg * G + g) * head_dim + piece * 8 + e] = acc[g][e];
  }
  __syncthreads();
  for (int i = tid; i < G * head_dim; i += DEC_THREADS) {
    float s = 0.f;
    for (int k = 0; k < kp; ++k) s += red[(size_t)k * G * head_dim + i];
    int g = i / head_dim, d = i - g * head_dim;
    part_o[(((size_t)b * n_heads + h0 + g) * n_splits + split) * head_dim + d] = s;
  }
}

__global__ void attention_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                int n_splits, int head_dim, int window,
                                                const int* __restrict__ tok_pos, __nv_bfloat16* __restrict__ out,
                                                int out_stride, int n_heads) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  const int b = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const int pos = tok_pos[b];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int s0 = lo / DEC_CHUNK, s1 = pos / DEC_CHUNK;  // chunks that hold a visible key
  const float* ml = part_ml + ((size_t)b * n_heads + h) * n_splits * 2;
  const float* po = part_o + ((size_t)b * n_heads + h) * n_splits * head_dim;
  float m = -INFINITY;
  for (int s = s0; s <= s1; ++s) m = fmaxf(m, ml[2 * s]);
  float num = 0.f, den = 0.f;
  for (int s = s0; s <= s1; ++s) {
    float w = expf(ml[2 * s] - m);
    den += w * ml[2 * s + 1];
    if (d < head_dim) num += w * po[(size_t)s * head_dim + d];
  }
  if (d < head_dim) out[(size_t)b * out_stride + (size_t)h * head_dim + d] = __float2bfloat16_rn(num / den);
}

// q: [n_seqs, q_stride] bfloat16, one row per sequence; tok_pos[b] is the position of that
// token (its key and value are already in the cache); part_o / part_ml are scratch of
// n_seqs * n_heads * n_splits * head_dim and n_seqs * n_heads * n_splits * 2 floats, where
// n_splits * 128 must cover the longest sequence.
extern "C" int bn_attention_decode(const void* q, int q_stride, void* out, int out_stride, int n_seqs, int n_heads,
                                   int n_kv_heads, int head_dim, float scale, int window, const int* tok_pos,
                                   const int* slots, const int* page_table, int pt_stride, const void* k_cache,
                                   const void* v_cache, float* part_o, float* part_ml, int n_splits,
                                   cudaStream_t stream) {
  if (n_seqs <= 0) return BN_OK;
  if (head_dim <= 0 || head_dim % 16 || head_dim > 256 || n_kv_heads <= 0 || n_heads % n_kv_heads || n_splits <= 0 ||
      window < 0 || !part_o || !part_ml)
    return BN_ERR_BAD_ARG;
  int group = n_heads / n_kv_heads;
  int gblocks = (group + DEC_GB - 1) / DEC_GB;
  if ((long long)n_kv_heads * gblocks > 65535 || n_splits > 65535 || n_heads > 65535) return BN_ERR_BAD_ARG;
  dim3 grid(n_seqs, n_kv_heads * gblocks, n_splits);
  BN_LAUNCH(attention_decode_partial_kernel, grid, DEC_THREADS, 0, stream, 
      (const __nv_bfloat16*)q, q_stride, n_heads, n_kv_heads, head_dim, scale, window, tok_pos, slots, page_table,
      pt_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, part_o, part_ml, n_splits);
  BN_CHECK_LAUNCH();
  int threads = ((head_dim + 31) / 32) * 32;
  BN_LAUNCH(attention_decode_combine_kernel, dim3(n_seqs, n_heads), threads, 0, stream, 
      part_o, part_ml, n_splits, head_dim, window, tok_pos, (__nv_bfloat16*)out, out_stride, n_heads);
  BN_CHECK_LAUNCH();
  return BN_OK;
}
