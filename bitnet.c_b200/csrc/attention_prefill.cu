// Causal attention of many new tokens per sequence in bfloat16 (prefill), over the paged cache.
//
// One block takes 64 consecutive new tokens of one sequence and one query head, and walks the
// sequence's cache pages from the first visible key to the last: a page holds 64 positions of
// one key/value head contiguously, so a page is exactly one key tile.  Scores and the weighted
// sum run on the tensor cores (m16n8k16, bfloat16 in, float32 accumulate); maxima, exponentials
// and sums stay in float32 registers (online softmax); keys and values are double-buffered in
// shared memory through cp.async, in a 16-byte XOR swizzle that keeps ldmatrix conflict-free.
// The new tokens' own keys and values must already be in the cache, so the same kernel serves
// whole prompts, pieces of prompts (earlier keys come from the cache) and ragged batches.
//
// Head sizes in steps of 16 run on the instantiation for 64, 128 or 256 with the missing
// dimensions zero in shared memory.
// Reference: per (head, token) scores over the cached keys 0..pos, scale 1/sqrt(head size),
// softmax, weighted sum of values; the key/value head of query head h is h / (H / KV)
// (src/transformer/batched_attn_scalar.c:97-169, flash variant :171-245).  The reference's CUDA
// prefill attention is one block per (head, token) on CUDA cores (src/gpu_cuda.cu:9772).
#include "mma.cuh"

#define PF_M 64       // query rows per block
#define PF_N 64       // keys per tile = BN_PAGE
#define PF_THREADS 128

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows hold HD bfloat16.
template <int HD>
__device__ __forceinline__ unsigned tile_off(int row, int chunk) {
  return (unsigned)(row * HD * 2 + ((chunk ^ (row & 7)) << 4));
}

template <int HD>
__global__ void __launch_bounds__(PF_THREADS)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                         int out_stride, int n_heads, int n_kv_heads, int head_dim, float scale_log2e, int window,
                         const int* __restrict__ tile_seq, const int* __restrict__ tile_row0,
                         const int* __restrict__ seq_start, const int* __restrict__ seq_pos0,
                         const int* __restrict__ slots, const int* __restrict__ page_table, int pt_stride,
                         const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int TILE_BYTES = PF_N * HD * 2;
  constexpr int CHUNKS = HD / 8;   // 16-byte chunks per row
  constexpr int KSTEPS = HD / 16;  // k-steps of the score product
  constexpr int NT_O = HD / 8;     // 8-wide column tiles of the output
  const unsigned s_q = (unsigned)__cvta_generic_to_shared(smem);
  const unsigned s_k = s_q + PF_M * HD * 2;      // two stages
  const unsigned s_v = s_k + 2 * TILE_BYTES;     // two stages

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  // blocks start in the order of their index, heads fastest: tiles are listed by rising work (the
  // keys they see), the last ones start first over all heads, and the query heads of one key/value
  // head run side by side
  const int blk = gridDim.y - 1 - blockIdx.y;
  const int seq = tile_seq[blk], row0 = tile_row0[blk], h = blockIdx.x;
  const int kvh = h / (n_heads / n_kv_heads);
  const int start = seq_start[seq], n_new = seq_start[seq + 1] - start, pos0 = seq_pos0[seq];
  const int* pt = page_table + (size_t)slots[seq] * pt_stride;
  const int real_chunks = head_dim / 8;
  const int rows_here = min(PF_M, n_new - row0);
  const int seq_last = pos0 + n_new - 1;  // the last position of this sequence that the cache holds

  // visible key range of this block
  const int q_first = pos0 + row0, q_last = pos0 + row0 + rows_here - 1;
  const int lo_first = window > 0 ? max(0, q_first - window + 1) : 0;
  const int tile_lo = lo_first / PF_N, tile_hi = q_last / PF_N;

  // ---- stage Q (rows beyond the sequence's tokens and dimensions beyond head_dim are zero)
  for (int p = tid; p < PF_M * CHUNKS; p += PF_THREADS) {
    int r = p / CHUNKS, c = p % CHUNKS;
    bool ok = r < rows_here && c < real_chunks;
    const __nv_bfloat16* src = ok ? q + (size_t)(start + row0 + r) * q_stride + (size_t)h * head_dim + c * 8 : q;
    cp_async16(s_q + tile_off<HD>(r, c), src, ok);
  }
  auto load_kv = [&](int tile, int stage) {
    int page = pt[tile];
    const __nv_bfloat16* kb = k_cache + ((size_t)page * n_kv_heads + kvh) * BN_PAGE * head_dim;
    const __nv_bfloat16* vb = v_cache + ((size_t)page * n_kv_heads + kvh) * BN_PAGE * head_dim;
    for (int p = tid; p < PF_N * CHUNKS; p += PF_THREADS) {
      int r = p / CHUNKS, c = p % CHUNKS;
      bool ok = c < real_chunks;
      // value rows behind the sequence's last position are zero here, whatever the cache holds:
      // their weights are zero, but zero times anything must be zero
      bool okv = ok && tile * PF_N + r <= seq_last;
      size_t off = (size_t)r * head_dim + c * 8;
      cp_async16(s_k + stage * TILE_BYTES + tile_off<HD>(r, c), ok ? kb + off : kb, ok);
      cp_async16(s_v + stage * TILE_BYTES + tile_off<HD>(r, c), okv ? vb + off : vb, okv);
    }
  };
  load_kv(tile_lo, 0);
  cp_async_commit();

  float o[NT_O][4];
#pragma unroll
  for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  // query positions of this thread's two rows; rows past the end look like the first row so
  // that they see at least one key (their result is not stored)
  int qpos[2], qlo[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    int r = warp * 16 + g + e * 8;
    qpos[e] = r < rows_here ? pos0 + row0 + r : q_first;
    qlo[e] = window > 0 ? max(0, qpos[e] - window + 1) : 0;
  }

  for (int tile = tile_lo; tile <= tile_hi; ++tile) {
    const int stage = (tile - tile_lo) & 1;
    if (tile + 1 <= tile_hi) {
      load_kv(tile + 1, stage ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    // ---- S = Q K^T for this warp's 16 rows and the tile's 64 keys
    float s[PF_N / 8][4];
#pragma unroll
    for (int j = 0; j < PF_N / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    const unsigned kb = s_k + stage * TILE_BYTES, vb = s_v + stage * TILE_BYTES;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      unsigned a0, a1, a2, a3;
      {
        int mi = lane >> 3, r = lane & 7;
        ldsm_x4(s_q + tile_off<HD>(warp * 16 + r + (mi & 1) * 8, ks * 2 + (mi >> 1)), a0, a1, a2, a3);
      }
#pragma unroll
      for (int j = 0; j < PF_N / 8; j += 2) {
        unsigned b0, b1, b2, b3;
        int mi = lane >> 3, r = lane & 7;
        ldsm_x4(kb + tile_off<HD>((j + (mi >> 1)) * 8 + r, ks * 2 + (mi & 1)), b0, b1, b2, b3);
        mma_bf16(s[j], a0, a1, a2, a3, b0, b1);
        mma_bf16(s[j + 1], a0, a1, a2, a3, b2, b3);
      }
    }

    // ---- mask, running maximum, exponentials
    const int kbase = tile * PF_N;
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int j = 0; j < PF_N / 8; ++j) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        int e = c >> 1;
        int kpos = kbase + j * 8 + 2 * t + (c & 1);
        bool ok = kpos <= qpos[e] && kpos >= qlo[e];
        float v = ok ? s[j][c] * scale_log2e : -INFINITY;
        s[j][c] = v;
        m_new[e] = fmaxf(m_new[e], v);
      }
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      m_new[e] = fmaxf(m_new[e], __shfl_xor_sync(0xffffffffu, m_new[e], 1));
      m_new[e] = fmaxf(m_new[e], __shfl_xor_sync(0xffffffffu, m_new[e], 2));
    }
    float alpha[2], l_add[2] = {0.f, 0.f};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      // a row can have no visible key in this tile (and none before): keep it at zero
      alpha[e] = (m_run[e] == -INFINITY) ? 0.f : exp2f(m_run[e] - m_new[e]);
    }
#pragma unroll
    for (int j = 0; j < PF_N / 8; ++j) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        int e = c >> 1;
        float p = (m_new[e] == -INFINITY) ? 0.f : exp2f(s[j][c] - m_new[e]);
        s[j][c] = p;
        l_add[e] += p;
      }
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      l_run[e] = l_run[e] * alpha[e] + l_add[e];  // per-thread partial sums; quads are combined at the end
      m_run[e] = m_new[e];
    }
#pragma unroll
    for (int j = 0; j < NT_O; ++j) {
      o[j][0] *= alpha[0]; o[j][1] *= alpha[0];
      o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
    }

    // ---- O += P V
#pragma unroll
    for (int ks = 0; ks < PF_N / 16; ++ks) {
      unsigned a0 = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
      unsigned a1 = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
      unsigned a2 = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
      unsigned a3 = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
      for (int j = 0; j < NT_O; j += 2) {
        unsigned b0, b1, b2, b3;
        int mi = lane >> 3, r = lane & 7;
        ldsm_x4_trans(vb + tile_off<HD>(ks * 16 + (mi & 1) * 8 + r, j + (mi >> 1)), b0, b1, b2, b3);
        mma_bf16(o[j], a0, a1, a2, a3, b0, b1);
        mma_bf16(o[j + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();  // the stage is overwritten by the load after next
  }

  // ---- normalise and store
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 1);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 2);
  }
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    int r = warp * 16 + g + e * 8;
    if (r >= rows_here) continue;
    float inv = 1.0f / l_run[e];
    __nv_bfloat16* orow = out + (size_t)(start + row0 + r) * out_stride + (size_t)h * head_dim;
#pragma unroll
    for (int j = 0; j < NT_O; ++j) {
      int d = j * 8 + 2 * t;
      if (d < head_dim) {
        __nv_bfloat162 v = __floats2bfloat162_rn(o[j][2 * e] * inv, o[j][2 * e + 1] * inv);
        *reinterpret_cast<__nv_bfloat162*>(orow + d) = v;
      }
    }
  }
}

template <int HD>
static int launch_prefill(const void* q, int q_stride, void* out, int out_stride, int n_tiles, int n_heads,
                          int n_kv_heads, int head_dim, float scale, int window, const int* tile_seq,
                          const int* tile_row0, const int* seq_start, const int* seq_pos0, const int* slots,
                          const int* page_table, int pt_stride, const void* k_cache, const void* v_cache,
                          cudaStream_t stream) {
  size_t smem = (size_t)PF_M * HD * 2 + 4 * (size_t)PF_N * HD * 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
    configured = true;
  }
  if (n_tiles > 65535) return BN_ERR_BAD_ARG;
  dim3 grid(n_heads, n_tiles);
  BN_LAUNCH((attention_prefill_kernel<HD>), grid, PF_THREADS, smem, stream, 
      (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, n_heads, n_kv_heads, head_dim,
      scale * 1.4426950408889634f, window, tile_seq, tile_row0, seq_start, seq_pos0, slots, page_table, pt_stride,
      (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache);
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// q: [tokens, q_stride] bfloat16 (head h at element h*head_dim), out [tokens, out_stride].
// tile_seq / tile_row0: for each block its sequence and the first of its 64 new-token rows;
// seq_start [n_seqs+1]: first packed row of each sequence; seq_pos0: its length before the step.
extern "C" int bn_attention_prefill(const void* q, int q_stride, void* out, int out_stride, int n_tiles, int n_heads,
                                    int n_kv_heads, int head_dim, float scale, int window, const int* tile_seq,
                                    const int* tile_row0, const int* seq_start, const int* seq_pos0,
                                    const int* slots, const int* page_table, int pt_stride, const void* k_cache,
                                    const void* v_cache, cudaStream_t stream) {
  if (n_tiles <= 0) return BN_OK;
  if (head_dim <= 0 || head_dim % 16 || head_dim > 256 || n_kv_heads <= 0 || n_heads % n_kv_heads || window < 0 ||
      n_heads > 65535 || (q_stride % 8) || (out_stride % 2) || (((uintptr_t)q) & 15))
    return BN_ERR_BAD_ARG;
  if (head_dim <= 64)
    return launch_prefill<64>(q, q_stride, out, out_stride, n_tiles, n_heads, n_kv_heads, head_dim, scale, window,
                              tile_seq, tile_row0, seq_start, seq_pos0, slots, page_table, pt_stride, k_cache, v_cache,
                              stream);
  if (head_dim <= 128)
    return launch_prefill<128>(q, q_stride, out, out_stride, n_tiles, n_heads, n_kv_heads, head_dim, scale, window,
                               tile_seq, tile_row0, seq_start, seq_pos0, slots, page_table, pt_stride, k_cache,
                               v_cache, stream);
  return launch_prefill<256>(q, q_stride, out, out_stride, n_tiles, n_heads, n_kv_heads, head_dim, scale, window,
                             tile_seq, tile_row0, seq_start, seq_pos0, slots, page_table, pt_stride, k_cache, v_cache,
                             stream);
}
