// Decode attention in bfloat16: one new token per sequence attends over its paged cache.
//
// With one query per sequence there is little work per (sequence, head), and at small batch
// too few (sequence, key/value head) pairs to fill 148 SMs, so the keys of a sequence are split
// into chunks of DEC_CHUNK positions: grid = (sequences, key/value heads x head groups, chunks).
// A block handles the up to 8 query heads that share its key/value head, so every key and
// value row is read once for all of them.  It writes an unnormalised partial result with its
// maximum and sum.  Chunk borders are multiples of DEC_CHUNK in position, so how a row is summed
// depends on its own position only, never on the batch around it.
//
// Two forms:
//  * fused (the decode step): the kernel takes the raw q|k|v row of the new token, applies the
//    rotary encoding to the queries itself, and the block whose chunk holds the new position
//    rotates the new key and writes key and value into the cache before it reads them; the
//    block that draws the last ticket of a (sequence, head group) combines the chunks.  One
//    launch instead of three (rotary + append, partial, combine).
//  * plain: queries are given ready-made, keys and values are already cached, and a second
//    kernel combines the chunks.
//
// Reference: scores = q.k * scale over the causal range, softmax with the maximum subtracted,
// weighted sum of values, query head h uses key/value head h / (H / KV)
// (src/transformer/gqa_scalar.c:61-121); the running maximum/sum form is its flash variant
// (gqa_scalar.c:127-207); rotary pairs (i, i + half) with angle pos * theta^(-2i/dims) as a running
// float32 product (src/transformer/cpu_backend.c:283-296, src/model_arch.c:322-338).  Its CUDA
// decode kernels: one block per head without a split over the keys (src/gpu_cuda.cu:9718), and a
// variant with the rotary encoding of q fused in (src/gpu_cuda.cu:9989).
#include "mma.cuh"

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

struct DecArgs {
  const __nv_bfloat16* q;  // plain: queries; fused: the q|k|v rows, queries first
  int q_stride;
  int n_heads, n_kv_heads, head_dim;
  float scale;
  int window;
  const int* tok_pos;
  const int* slots;
  const int* page_table;
  int pt_stride;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  float* part_o;
  float* part_ml;
  int n_splits;
  // fused only
  int k_off, v_off;       // element offsets of the key and value heads in a row
  int rotary_dims;        // 0: no rotation
  float theta_scale;
  int* tickets;           // one per (sequence, blockIdx.y), zero before and after
  __nv_bfloat16* out;
  int out_stride;
};

template <bool FUSED>
__global__ void __launch_bounds__(DEC_THREADS) attention_decode_kernel(DecArgs a) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  __shared__ float q_s[DEC_GB * 256];
  __shared__ float p_s[DEC_GB * DEC_CHUNK];
  __shared__ float red[DEC_THREADS * DEC_GB * 8];
  __shared__ float ml_s[DEC_GB * 2];
  __shared__ int s_last;
  const int b = blockIdx.x, split = blockIdx.z, tid = threadIdx.x;
  const int head_dim = a.head_dim, n_kv_heads = a.n_kv_heads, n_heads = a.n_heads;
  const int group = n_heads / n_kv_heads;
  const int gblocks = (group + DEC_GB - 1) / DEC_GB;
  const int kvh = blockIdx.y / gblocks, gb = blockIdx.y % gblocks;
  const int h0 = kvh * group + gb * DEC_GB;
  const int G = min(DEC_GB, group - gb * DEC_GB);
  const int pos = a.tok_pos[b];
  const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int c0 = split * DEC_CHUNK;
  if (c0 > pos || c0 + DEC_CHUNK <= lo) return;  // no key of this chunk is visible
  const int* pt = a.page_table + (size_t)a.slots[b] * a.pt_stride;
  // a chunk of 128 positions lies in two pages; their ids are fetched once
  const int page_a = pt[c0 / BN_PAGE];
  const int page_b = (c0 + BN_PAGE <= pos) ? pt[c0 / BN_PAGE + 1] : page_a;
  auto row_off = [&](int j) -> size_t {  // row of key/value j of this chunk (0 <= j < 128)
    int page = j < BN_PAGE ? page_a : page_b;
    return (((size_t)page * n_kv_heads + kvh) * BN_PAGE + (j & (BN_PAGE - 1))) * (size_t)head_dim;
  };
  const __nv_bfloat16* qrow = a.q + (size_t)b * a.q_stride;

  if (FUSED) {
    const int half = a.rotary_dims >> 1;
    // queries: rotate the first rotary_dims of each head, pass the rest through
    for (int p = tid; p < G * half; p += DEC_THREADS) {
      int g = p / half, i = p - g * half;
      float s, c;
      sincosf(rope_angle(pos, i, a.theta_scale), &s, &c);
      const __nv_bfloat16* hd = qrow + (size_t)(h0 + g) * head_dim;
      float x = __bfloat162float(hd[i]), y = __bfloat162float(hd[i + half]);
      // the rotated query is rounded to bfloat16 as the unfused path stores it
      q_s[g * 256 + i] = __bfloat162float(__float2bfloat16_rn(x * c - y * s));
      q_s[g * 256 + i + half] = __bfloat162float(__float2bfloat16_rn(x * s + y * c));
    }
    const int rest = head_dim - a.rotary_dims;
    for (int p = tid; p < G * rest; p += DEC_THREADS) {
      int g = p / rest, d = a.rotary_dims + p - g * rest;
      q_s[g * 256 + d] = __bfloat162float(qrow[(size_t)(h0 + g) * head_dim + d]);
    }
    // the block whose chunk holds the new position stores the new key (rotated) and value
    if (pos / DEC_CHUNK == split) {
      const size_t off = row_off(pos - c0);
      const __nv_bfloat16* kraw = qrow + a.k_off + (size_t)kvh * head_dim;
      const __nv_bfloat16* vraw = qrow + a.v_off + (size_t)kvh * head_dim;
      for (int i = tid; i < half; i += DEC_THREADS) {
        float s, c;
        sincosf(rope_angle(pos, i, a.theta_scale), &s, &c);
        float x = __bfloat162float(kraw[i]), y = __bfloat162float(kraw[i + half]);
        a.k_cache[off + i] = __float2bfloat16_rn(x * c - y * s);
        a.k_cache[off + i + half] = __float2bfloat16_rn(x * s + y * c);
      }
      for (int d = a.rotary_dims + tid; d < head_dim; d += DEC_THREADS) a.k_cache[off + d] = kraw[d];
      for (int d = tid; d < head_dim; d += DEC_THREADS) a.v_cache[off + d] = vraw[d];
    }
  } else {
    for (int i = tid; i < G * head_dim; i += DEC_THREADS) {
      int g = i / head_dim, d = i - g * head_dim;
      q_s[g * 256 + d] = __bfloat162float(qrow[(size_t)(h0 + g) * head_dim + d]);
    }
  }
  __syncthreads();  // q_s is complete; the new key and value are visible to this block

  // ---- scores: one key per thread, all G heads at once
  {
    int p = c0 + tid;
    bool valid = p >= lo && p <= pos;
    float dot[DEC_GB];
#pragma unroll
    for (int g = 0; g < DEC_GB; ++g) dot[g] = 0.f;
    if (valid) {
      const __nv_bfloat16* krow = a.k_cache + row_off(tid);
      // 64 dimensions (eight 16-byte loads) are requested before the first is used
      for (int d0 = 0; d0 < head_dim; d0 += 64) {
        uint4 raw[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          raw[u] = (d0 + u * 8 < head_dim) ? *reinterpret_cast<const uint4*>(krow + d0 + u * 8) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (d0 + u * 8 >= head_dim) break;
          float kf[8];
          bf16x8_to_f32(raw[u], kf);
#pragma unroll
          for (int g = 0; g < DEC_GB; ++g) {
            if (g < G) {
              const float* qq = q_s + g * 256 + d0 + u * 8;
#pragma unroll
              for (int e = 0; e < 8; ++e) dot[g] = fmaf(qq[e], kf[e], dot[g]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int g = 0; g < DEC_GB; ++g)
      if (g < G) p_s[g * DEC_CHUNK + tid] = valid ? dot[g] * a.scale : -INFINITY;
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
        size_t o = (((size_t)b * n_heads + h0 + g) * a.n_splits + split) * 2;
        a.part_ml[o] = m;
        a.part_ml[o + 1] = l;
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
    // eight value rows are requested before the first is used
    for (int j = j_lo + kg; j < j_hi; j += 8 * kp) {
      uint4 raw[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        int ju = j + u * kp;
        raw[u] = ju < j_hi ? *reinterpret_cast<const uint4*>(a.v_cache + row_off(ju) + piece * 8) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
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
    a.part_o[(((size_t)b * n_heads + h0 + g) * a.n_splits + split) * head_dim + d] = s;
  }

  if (FUSED) {
    // ---- the block that draws the last ticket of this (sequence, head group) combines the chunks
    const int s0 = lo / DEC_CHUNK, s1 = pos / DEC_CHUNK;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      int* t = a.tickets + (size_t)b * gridDim.y + blockIdx.y;
      int ticket = atomicAdd(t, 1);
      s_last = (ticket == s1 - s0);
      if (s_last) *t = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid < G) {
      const float* ml = a.part_ml + ((size_t)b * n_heads + h0 + tid) * a.n_splits * 2;
      float m = -INFINITY;
      for (int s = s0; s <= s1; ++s) m = fmaxf(m, __ldcg(ml + 2 * s));
      float den = 0.f;
      for (int s = s0; s <= s1; ++s) den += expf(__ldcg(ml + 2 * s) - m) * __ldcg(ml + 2 * s + 1);
      ml_s[tid * 2] = m;
      ml_s[tid * 2 + 1] = den;
    }
    __syncthreads();
    for (int i = tid; i < G * head_dim; i += DEC_THREADS) {
      int g = i / head_dim, d = i - g * head_dim;
      const float* ml = a.part_ml + ((size_t)b * n_heads + h0 + g) * a.n_splits * 2;
      const float* po = a.part_o + ((size_t)b * n_heads + h0 + g) * a.n_splits * head_dim;
      float m = ml_s[g * 2], num = 0.f;
      for (int s = s0; s <= s1; ++s) num += expf(__ldcg(ml + 2 * s) - m) * __ldcg(po + (size_t)s * head_dim + d);
      a.out[(size_t)b * a.out_stride + (size_t)(h0 + g) * head_dim + d] = __float2bfloat16_rn(num / ml_s[g * 2 + 1]);
    }
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

static int check_dec(int n_heads, int n_kv_heads, int head_dim, int n_splits, int window, const float* part_o,
                     const float* part_ml) {
  if (head_dim <= 0 || head_dim % 16 || head_dim > 256 || n_kv_heads <= 0 || n_heads % n_kv_heads || n_splits <= 0 ||
      window < 0 || !part_o || !part_ml)
    return BN_ERR_BAD_ARG;
  int group = n_heads / n_kv_heads;
  int gblocks = (group + DEC_GB - 1) / DEC_GB;
  if ((long long)n_kv_heads * gblocks > 65535 || n_splits > 65535 || n_heads > 65535) return BN_ERR_BAD_ARG;
  return BN_OK;
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
  int st = check_dec(n_heads, n_kv_heads, head_dim, n_splits, window, part_o, part_ml);
  if (st) return st;
  int gblocks = (n_heads / n_kv_heads + DEC_GB - 1) / DEC_GB;
  DecArgs a = {};
  a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride; a.n_heads = n_heads; a.n_kv_heads = n_kv_heads;
  a.head_dim = head_dim; a.scale = scale; a.window = window; a.tok_pos = tok_pos; a.slots = slots;
  a.page_table = page_table; a.pt_stride = pt_stride; a.k_cache = (__nv_bfloat16*)k_cache;
  a.v_cache = (__nv_bfloat16*)v_cache; a.part_o = part_o; a.part_ml = part_ml; a.n_splits = n_splits;
  dim3 grid(n_seqs, n_kv_heads * gblocks, n_splits);
  BN_LAUNCH(attention_decode_kernel<false>, grid, DEC_THREADS, 0, stream, a);
  int threads = ((head_dim + 31) / 32) * 32;
  BN_LAUNCH(attention_decode_combine_kernel, dim3(n_seqs, n_heads), threads, 0, stream,
      part_o, part_ml, n_splits, head_dim, window, tok_pos, (__nv_bfloat16*)out, out_stride, n_heads);
  return BN_OK;
}

// The decode step in one launch.  qkv: [n_seqs, q_stride] bfloat16 rows holding the raw query
// heads first, the key heads at element k_off and the value heads at v_off.  The kernel rotates
// queries and the new key (rotary_dims = 0: no rotation), writes the new key and value into the
// cache at tok_pos[b], attends, and combines.  tickets: n_seqs * n_kv_heads * ceil(group / 8)
// ints, zero before and after.
extern "C" int bn_attention_decode_fused(const void* qkv, int q_stride, int k_off, int v_off, void* out, int out_stride,
                                         int n_seqs, int n_heads, int n_kv_heads, int head_dim, float scale,
                                         int window, int rotary_dims, float theta_scale, const int* tok_pos,
                                         const int* slots, const int* page_table, int pt_stride, void* k_cache,
                                         void* v_cache, float* part_o, float* part_ml, int n_splits, int* tickets,
                                         int n_tickets, cudaStream_t stream) {
  if (n_seqs <= 0) return BN_OK;
  int st = check_dec(n_heads, n_kv_heads, head_dim, n_splits, window, part_o, part_ml);
  if (st) return st;
  int gblocks = (n_heads / n_kv_heads + DEC_GB - 1) / DEC_GB;
  if (rotary_dims < 0 || rotary_dims > head_dim || (rotary_dims & 1) || !tickets ||
      (long long)n_seqs * n_kv_heads * gblocks > n_tickets)
    return BN_ERR_BAD_ARG;
  DecArgs a = {};
  a.q = (const __nv_bfloat16*)qkv; a.q_stride = q_stride; a.n_heads = n_heads; a.n_kv_heads = n_kv_heads;
  a.head_dim = head_dim; a.scale = scale; a.window = window; a.tok_pos = tok_pos; a.slots = slots;
  a.page_table = page_table; a.pt_stride = pt_stride; a.k_cache = (__nv_bfloat16*)k_cache;
  a.v_cache = (__nv_bfloat16*)v_cache; a.part_o = part_o; a.part_ml = part_ml; a.n_splits = n_splits;
  a.k_off = k_off; a.v_off = v_off; a.rotary_dims = rotary_dims; a.theta_scale = theta_scale; a.tickets = tickets;
  a.out = (__nv_bfloat16*)out; a.out_stride = out_stride;
  dim3 grid(n_seqs, n_kv_heads * gblocks, n_splits);
  BN_LAUNCH(attention_decode_kernel<true>, grid, DEC_THREADS, 0, stream, a);
  return BN_OK;
}
