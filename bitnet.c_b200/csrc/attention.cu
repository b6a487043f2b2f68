// Causal softmax attention over the paged cache, for any mix of new tokens: whole
// prompts, pieces of prompts, or one token per sequence.  One block per (token, head).
// This is the general kernel: it serves the float32 path and every shape; the
// bfloat16 path uses the specialised kernels in attention_prefill.cu and
// attention_decode.cu where they apply.
//
// Reference: for query head h the key/value head is h / (n_heads / n_kv_heads);
// s_i = (q . K[t_i]) * scale over the causal range only, p = softmax(s) with the
// maximum subtracted, out = sum_i p_i V[t_i]   (src/transformer/gqa_scalar.c:61-121,
// prefill: src/transformer/batched_attn_scalar.c:97-169).  The online form with a
// running maximum and sum is the reference's flash variant (gqa_scalar.c:127-207).
#include "common.cuh"

#define ATT_THREADS 128
#define ATT_CHUNK 128

template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float* o) {
    float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float* o) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      o[2 * i] = f.x; o[2 * i + 1] = f.y;
    }
  }
};

template <typename T>
__global__ void attention_general_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out,
                                         int out_stride, int n_heads, int n_kv_heads, int head_dim,
                                         float scale, int window, const int* __restrict__ tok_seq,
                                         const int* __restrict__ tok_pos, const int* __restrict__ slots,
                                         const int* __restrict__ page_table, int pt_stride,
                                         const T* __restrict__ k_cache, const T* __restrict__ v_cache) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  extern __shared__ float sm[];
  float* qs = sm;                    // head_dim
  float* ps = qs + head_dim;         // ATT_CHUNK scores, then probabilities
  float* scratch = ps + ATT_CHUNK;   // 32
  int t = blockIdx.x, h = blockIdx.y;
  int kvh = h / (n_heads / n_kv_heads);
  int pos = tok_pos[t];
  const int* pt = page_table + (size_t)slots[tok_seq[t]] * pt_stride;
  int lo = window > 0 ? max(0, pos - window + 1) : 0;

  const T* qrow = q + (size_t)t * q_stride + (size_t)h * head_dim;
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) qs[d] = to_f32<T>(qrow[d]);
  __syncthreads();

  constexpr int VN = Vec16<T>::N;
  constexpr int MAX_D = 2;  // output dims per thread: head_dim <= 256
  float acc[MAX_D] = {0.f, 0.f};
  float m_run = -INFINITY, l_run = 0.f;

  for (int base = lo; base <= pos; base += ATT_CHUNK) {
    int n = min(ATT_CHUNK, pos - base + 1);
    float s = -INFINITY;
    if ((int)threadIdx.x < n) {
      int p = base + threadIdx.x;
      const T* krow = k_cache + cache_row_offset(pt, p, n_kv_heads, kvh, head_dim);
      float dot = 0.f;
      for (int d = 0; d < head_dim; d += VN) {
        float kv[VN];
        Vec16<T>::load(krow + d, kv);
#pragma unroll
        for (int e = 0; e < VN; ++e) dot = fmaf(qs[d + e], kv[e], dot);
      }
      s = dot * scale;
    }
    float m_chunk = block_max(s, scratch);
    float m_new = fmaxf(m_run, m_chunk);
    float alpha = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
    float p_mine = ((int)threadIdx.x < n) ? expf(s - m_new) : 0.f;
    ps[threadIdx.x] = p_mine;
    float l_chunk = block_sum(p_mine, scratch);  // has the barrier that publishes ps[]
    l_run = l_run * alpha + l_chunk;
    m_run = m_new;
#pragma unroll
    for (int r = 0; r < MAX_D; ++r) {
      int d = threadIdx.x + r * ATT_THREADS;
      if (d < head_dim) {
        float a = acc[r] * alpha;
        for (int j = 0; j < n; ++j) {
          const T* vrow = v_cache + cache_row_offset(pt, base + j, n_kv_heads, kvh, head_dim);
          a = fmaf(ps[j], to_f32<T>(vrow[d]), a);
        }
        acc[r] = a;
      }
    }
    __syncthreads();  // ps[] is rewritten by the next chunk
  }
  float inv = 1.0f / l_run;
  T* orow = out + (size_t)t * out_stride + (size_t)h * head_dim;
#pragma unroll
  for (int r = 0; r < MAX_D; ++r) {
    int d = threadIdx.x + r * ATT_THREADS;
    if (d < head_dim) orow[d] = from_f32<T>(acc[r] * inv);
  }
}

// q: [n_tokens, q_stride] with head h at element h*head_dim; out likewise with out_stride.
// The keys and values of the new tokens must already be in the cache.
extern "C" int bn_attention_general(const void* q, int q_stride, void* out, int out_stride, int dtype,
                                    int n_tokens, int n_heads, int n_kv_heads, int head_dim, float scale,
                                    int window, const int* tok_seq, const int* tok_pos, const int* slots,
                                    const int* page_table, int pt_stride,
                                    const void* k_cache, const void* v_cache, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (head_dim <= 0 || head_dim % 16 || head_dim > 256 || n_kv_heads <= 0 || n_heads % n_kv_heads ||
      window < 0)
    return BN_ERR_BAD_ARG;
  if (n_heads > 65535) return BN_ERR_BAD_ARG;
  dim3 grid(n_tokens, n_heads);
  size_t smem = (head_dim + ATT_CHUNK + 32) * sizeof(float);
  if (dtype == BN_F32)
    BN_LAUNCH((attention_general_kernel<float>), grid, ATT_THREADS, smem, stream, 
        (const float*)q, q_stride, (float*)out, out_stride, n_heads, n_kv_heads, head_dim, scale, window,
        tok_seq, tok_pos, slots, page_table, pt_stride, (const float*)k_cache, (const float*)v_cache);
  else if (dtype == BN_BF16)
    BN_LAUNCH((attention_general_kernel<__nv_bfloat16>), grid, ATT_THREADS, smem, stream, 
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, n_heads, n_kv_heads, head_dim,
        scale, window, tok_seq, tok_pos, slots, page_table, pt_stride,
        (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache);
  else
    return BN_ERR_BAD_ARG;
  BN_CHECK_LAUNCH();
  return BN_OK;
}
