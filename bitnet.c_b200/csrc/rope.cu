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

// The same for bfloat16 rows whose pieces are all multiples of 8 elements (rotary_dims a multiple
// of 16, head_dim, row_stride, k_off, v_off multiples of 8): every work item moves 16 bytes.
//   [0, n_rot_heads * hc)                        a pair of chunks (head, c) and (head, c + hc) of the rotary half
//   [.., + n_kv_heads * plain)                   a key chunk that no rotation touches -> cache
//   [.., + n_kv_heads * head_dim / 8)            a value chunk -> cache
__global__ void rope_append_bf16x8_kernel(__nv_bfloat16* __restrict__ x, int row_stride, int n_rot_heads, int head_dim,
                                          int rotary_dims, float theta_scale, const int* __restrict__ tok_pos,
                                          int k_off, int v_off, int n_kv_heads, const int* __restrict__ tok_seq,
                                          const int* __restrict__ slots, const int* __restrict__ page_table,
                                          int pt_stride, __nv_bfloat16* __restrict__ k_cache,
                                          __nv_bfloat16* __restrict__ v_cache) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float cs[128], sn[128];
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  __nv_bfloat16* row = x + (size_t)t * row_stride;
  const int half = rotary_dims >> 1, hc = half >> 3, hdc = head_dim >> 3;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float angle = (float)pos;
    for (int k = 0; k < i; ++k) angle *= theta_scale;
    sincosf(angle, &sn[i], &cs[i]);
  }
  __syncthreads();
  const int* pt = k_cache ? page_table + (size_t)slots[tok_seq[t]] * pt_stride : nullptr;
  const int first_key = k_off / head_dim;                   // index of the first key head among the row's heads
  const int rot_keys = k_cache ? max(0, min(n_kv_heads, n_rot_heads - first_key)) : 0;  // key heads that are rotated
  const int n_pairs = n_rot_heads * hc;
  // key chunks that no rotation writes: all chunks of unrotated key heads, chunks past rotary_dims of rotated ones
  const int plain_rot = hdc - 2 * hc;
  const int n_kplain = k_cache ? rot_keys * plain_rot + (n_kv_heads - rot_keys) * hdc : 0;
  const int n_v = k_cache ? n_kv_heads * hdc : 0;
  for (int item = threadIdx.x; item < n_pairs + n_kplain + n_v; item += blockDim.x) {
    if (item < n_pairs) {
      const int h = item / hc, c = item - h * hc;
      __nv_bfloat16* hd = row + (size_t)h * head_dim;
      uint4 xv = *reinterpret_cast<const uint4*>(hd + c * 8), yv = *reinterpret_cast<const uint4*>(hd + half + c * 8);
      const __nv_bfloat16* xs = reinterpret_cast<const __nv_bfloat16*>(&xv);
      const __nv_bfloat16* ys = reinterpret_cast<const __nv_bfloat16*>(&yv);
      uint4 lo4, hi4;
      __nv_bfloat16* los = reinterpret_cast<__nv_bfloat16*>(&lo4);
      __nv_bfloat16* his = reinterpret_cast<__nv_bfloat16*>(&hi4);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float c_ = cs[c * 8 + e], s_ = sn[c * 8 + e];
        const float a = __bfloat162float(xs[e]), b = __bfloat162float(ys[e]);
        los[e] = __float2bfloat16_rn(a * c_ - b * s_);
        his[e] = __float2bfloat16_rn(a * s_ + b * c_);
      }
      *reinterpret_cast<uint4*>(hd + c * 8) = lo4;
      *reinterpret_cast<uint4*>(hd + half + c * 8) = hi4;
      const int kh = h - first_key;
      if (k_cache && kh >= 0 && kh < n_kv_heads) {
        const size_t off = cache_row_offset(pt, pos, n_kv_heads, kh, head_dim);
        *reinterpret_cast<uint4*>(k_cache + off + c * 8) = lo4;
        *reinterpret_cast<uint4*>(k_cache + off + half + c * 8) = hi4;
      }
    } else if (item < n_pairs + n_kplain) {
      int e = item - n_pairs, kh, c;
      if (e < rot_keys * plain_rot) {
        kh = e / plain_rot;
        c = 2 * hc + (e - kh * plain_rot);
      } else {
        e -= rot_keys * plain_rot;
        kh = rot_keys + e / hdc;
        c = e - (kh - rot_keys) * hdc;
      }
      const size_t off = cache_row_offset(pt, pos, n_kv_heads, kh, head_dim);
      *reinterpret_cast<uint4*>(k_cache + off + c * 8) = *reinterpret_cast<const uint4*>(row + k_off + (size_t)kh * head_dim + c * 8);
    } else {
      const int e = item - n_pairs - n_kplain, kh = e / hdc, c = e - kh * hdc;
      const size_t off = cache_row_offset(pt, pos, n_kv_heads, kh, head_dim);
      *reinterpret_cast<uint4*>(v_cache + off + c * 8) = *reinterpret_cast<const uint4*>(row + v_off + (size_t)kh * head_dim + c * 8);
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
  else if (dtype == BN_BF16 && (rotary_dims % 16) == 0 && (head_dim % 8) == 0 && (row_stride % 8) == 0 && (k_off % 8) == 0 &&
           (v_off % 8) == 0 && (((uintptr_t)x | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0)
    BN_LAUNCH(rope_append_bf16x8_kernel, grid, threads, 0, stream, (__nv_bfloat16*)x, row_stride, n_rot_heads, head_dim,
              rotary_dims, theta_scale, tok_pos, k_off, v_off, n_kv_heads, tok_seq, slots, page_table, pt_stride,
              (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache);
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
