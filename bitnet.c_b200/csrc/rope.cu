// Rotary position encoding of the query and key heads of a packed row, fused with
// the write of the new keys and values into the paged cache.
//
// Reference: pairs (i, i + rotary_dims/2) are rotated,
//   x[i] = a cos - b sin,  x[i + half] = a sin + b cos   (src/transformer/cpu_backend.c:283-296)
// with angle_0 = pos and angle_{i+1} = angle_i * theta^(-2/rotary_dims) as a running
// float32 product (src/model_arch.c:322-338, src/transformer.c:143-162); keys are
// stored rotated and values as they are (src/transformer/cpu.c:859-898).
#include "common.cuh"

#define ROPE_THREADS 256

// One block per token.  The cosines and sines of the token's position are computed once into
// shared memory; then the block walks the token's work items:
//   [0, n_rot_heads * half)           one rotation pair (head, i); a pair of a key head also goes to the cache
//   [.., + n_kv_heads * head_dim)     one value element -> cache, and the key element at the same place if
//                                     no rotation touched it (dimensions past rotary_dims, or no rotation at all)
template <typename T>
__global__ void rope_append_kernel(T* __restrict__ x, int row_stride, int n_rot_heads, int head_dim,
                                   int rotary_dims, float theta_scale, const int* __restrict__ tok_pos,
                                   int k_off, int v_off, int n_kv_heads, const int* __restrict__ tok_seq,
                                   const int* __restrict__ slots, const int* __restrict__ page_table,
                                   int pt_stride, T* __restrict__ k_cache, T* __restrict__ v_cache) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  __shared__ float cs[128], sn[128];  // rotary_dims <= head_dim <= 256
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  T* row = x + (size_t)t * row_stride;
  const int half = rotary_dims >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float angle = (float)pos;
    for (int k = 0; k < i; ++k) angle *= theta_scale;
    sincosf(angle, &sn[i], &cs[i]);
  }
  __syncthreads();
  const int n_pairs = n_rot_heads * half;
  const int n_copy = k_cache ? n_kv_heads * head_dim : 0;
  const int* pt = k_cache ? page_table + (size_t)slots[tok_seq[t]] * pt_stride : nullptr;
  for (int item = threadIdx.x; item < n_pairs + n_copy; item += blockDim.x) {
    if (item < n_pairs) {
      int h = item / half, i = item - h * half;
      float s = sn[i], c = cs[i];
      T* hd = row + (size_t)h * head_dim;
      float a = to_f32<T>(hd[i]), b = to_f32<T>(hd[i + half]);
      T lo = from_f32<T>(a * c - b * s), hi = from_f32<T>(a * s + b * c);
      hd[i] = lo;
      hd[i + half] = hi;
      int e = h * head_dim - k_off;  // element offset of this head among the key heads
      if (k_cache && e >= 0 && e < n_kv_heads * head_dim) {
        size_t off = cache_row_offset(pt, pos, n_kv_heads, e / head_dim, head_dim);
        k_cache[off + i] = lo;
        k_cache[off + i + half] = hi;
      }
    } else {
      int e = item - n_pairs;
      int kvh = e / head_dim, d = e - kvh * head_dim;
      size_t off = cache_row_offset(pt, pos, n_kv_heads, kvh, head_dim) + d;
      v_cache[off] = row[v_off + e];
      bool rotated = d < rotary_dims && (k_off + kvh * head_dim) < n_rot_heads * head_dim;
      if (!rotated) k_cache[off] = row[k_off + e];
    }
  }
}

// x: [n_tokens, row_stride] with the heads to rotate first in each row.  When k_cache is
// not null the n_kv_heads key heads at element offset k_off (already rotated if they are
// among the first n_rot_heads) and the value heads at v_off are written to the cache.
extern "C" int bn_rope_append(void* x, int dtype, int n_tokens, int row_stride, int n_rot_heads, int head_dim,
                              int rotary_dims, float theta_scale, const int* tok_pos, int k_off, int v_off,
                              int n_kv_heads, const int* tok_seq, const int* slots, const int* page_table,
                              int pt_stride, void* k_cache, void* v_cache,
                              cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (head_dim <= 0 || rotary_dims < 0 || rotary_dims > head_dim || (rotary_dims & 1)) return BN_ERR_BAD_ARG;
  if (k_cache && (!v_cache || !tok_seq || !slots || !page_table)) return BN_ERR_BAD_ARG;
  if (k_cache && (k_off % head_dim)) return BN_ERR_BAD_ARG;  // key heads start at a head border
  int items = n_rot_heads * (rotary_dims / 2) + (k_cache ? n_kv_heads * head_dim : 0);
  if (items <= 0) return BN_OK;
  dim3 grid(n_tokens);
  const int threads = ROPE_THREADS;
  if (dtype == BN_F32)
    BN_LAUNCH((rope_append_kernel<float>), grid, threads, 0, stream, 
        (float*)x, row_stride, n_rot_heads, head_dim, rotary_dims, theta_scale, tok_pos, k_off, v_off,
        n_kv_heads, tok_seq, slots, page_table, pt_stride, (float*)k_cache, (float*)v_cache);
  else if (dtype == BN_BF16)
    BN_LAUNCH((rope_append_kernel<__nv_bfloat16>), grid, threads, 0, stream, 
        (__nv_bfloat16*)x, row_stride, n_rot_heads, head_dim, rotary_dims, theta_scale, tok_pos, k_off, v_off,
        n_kv_heads, tok_seq, slots, page_table, pt_stride, (__nv_bfloat16*)k_cache,
        (__nv_bfloat16*)v_cache);
  else
    return BN_ERR_BAD_ARG;
  BN_CHECK_LAUNCH();
  return BN_OK;
}
