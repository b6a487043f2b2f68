// Decode attention in bfloat16 on tensor cores: one new token per sequence over its paged cache,
// position encoding, cache write, attention and the combination of the key chunks in one launch.
//
// grid = (sequences, key/value heads x groups of 16 query heads, chunks of 128 positions).
// A block first asks for its whole chunk of keys and values (two pages each, up to 64 KB) with
// cp.async, so a step that reads hundreds of megabytes of cache has them all in flight at once;
// while they travel it rotates the queries of its head group into a 16-row tile (the query heads
// that share the key/value head are the rows).  The block whose chunk holds the new position
// also rotates the new key, writes key and value to the cache and puts them into its tiles
// directly.  Each of the four warps then takes 32 keys: scores on m16n8k16 MMAs, float32 softmax
// statistics, the weighted value sum on MMAs again; the warps' results are merged in shared
// memory, written as an unnormalised partial with maximum and sum, and the block that draws the
// last ticket of its (sequence, head group) merges the chunks and writes the output.
// Chunk borders are multiples of 128 in position, so a row's arithmetic depends on its own
// position only.  Head sizes in steps of 16 run on the instantiation for 64, 128 or 256 with the
// missing dimensions zero in shared memory.
//
// Reference: scores = q.k * scale over the causal range, softmax with the maximum subtracted,
// weighted sum of values, query head h uses key/value head h / (H / KV)
// (src/transformer/gqa_scalar.c:61-121; online form gqa_scalar.c:127-207); rotary pairs
// (i, i + half), angle pos * theta^(-2i/dims) as a running float32 product
// (src/transformer/cpu_backend.c:283-296, src/model_arch.c:322-338).  The reference's CUDA decode
// attention is one block per head on CUDA cores without a split over the keys, with a variant
// that fuses the rotary encoding of q (src/gpu_cuda.cu:9718, 9989).
#include "common.cuh"

#define DT_THREADS 128
#define DT_CHUNK 128
#define DT_ROWS 16  // query heads per block (the MMA's 16 rows)

__device__ __forceinline__ void dt_cp_async16(unsigned smem, const void* gmem, bool valid) {
  int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void dt_ldsm_x4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void dt_ldsm_x4_trans(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void dt_mma(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned dt_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
// Byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows hold HD bfloat16 (XOR swizzle).
template <int HD>
__device__ __forceinline__ unsigned dt_off(int row, int chunk) {
  return (unsigned)(row * HD * 2 + ((chunk ^ (row & 7)) << 4));
}
__device__ __forceinline__ float dt_angle(int pos, int i, float theta_scale) {
  float angle = (float)pos;
  for (int k = 0; k < i; ++k) angle *= theta_scale;
  return angle;
}

struct DtArgs {
  const __nv_bfloat16* qkv;  // [n_seqs, q_stride]: raw query heads, key heads at k_off, value heads at v_off
  int q_stride, k_off, v_off;
  int n_heads, n_kv_heads, head_dim;
  float scale_log2e;
  int window;
  int rotary_dims;
  float theta_scale;
  const int* tok_pos;
  const int* slots;
  const int* page_table;
  int pt_stride;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  float* part_o;   // [n_seqs][n_heads][n_splits][head_dim]
  float* part_ml;  // [n_seqs][n_heads][n_splits][2]: maximum (in the scaled log2 domain) and sum
  int n_splits;
  int* tickets;    // [n_seqs][gridDim.y], zero before and after
  __nv_bfloat16* out;
  int out_stride;
};

template <int HD>
__global__ void __launch_bounds__(DT_THREADS) attention_decode_tc_kernel(DtArgs a) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  pdl_wait();               // the kernels before this one have completed and their writes are visible
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int CHUNKS = HD / 8, KSTEPS = HD / 16, NT_O = HD / 8;
  constexpr int TILE_BYTES = DT_CHUNK * HD * 2;
  const unsigned s_q = (unsigned)__cvta_generic_to_shared(smem);
  const unsigned s_k = s_q + DT_ROWS * HD * 2;
  const unsigned s_v = s_k + TILE_BYTES;
  unsigned char* q_tile = smem;
  unsigned char* k_tile = smem + DT_ROWS * HD * 2;
  unsigned char* v_tile = k_tile + TILE_BYTES;
  float* o_part = reinterpret_cast<float*>(k_tile);               // [4 warps][16][HD], after the scores
  float* ml_part = reinterpret_cast<float*>(v_tile + TILE_BYTES);  // [4 warps][16][2]
  float* ml_fin = ml_part + 4 * DT_ROWS * 2;                       // [16][2]
  __shared__ int s_last;

  const int b = blockIdx.x, split = blockIdx.z, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g4 = lane >> 2, t4 = lane & 3;
  const int head_dim = a.head_dim, n_kv_heads = a.n_kv_heads, n_heads = a.n_heads;
  const int group = n_heads / n_kv_heads;
  const int gblocks = (group + DT_ROWS - 1) / DT_ROWS;
  const int kvh = blockIdx.y / gblocks, gb = blockIdx.y % gblocks;
  const int h0 = kvh * group + gb * DT_ROWS;
  const int G = min(DT_ROWS, group - gb * DT_ROWS);
  const int pos = a.tok_pos[b];
  const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int c0 = split * DT_CHUNK;
  if (c0 > pos || c0 + DT_CHUNK <= lo) return;  // no key of this chunk is visible
  const int* pt = a.page_table + (size_t)a.slots[b] * a.pt_stride;
  const int page_a = pt[c0 / BN_PAGE];
  const int page_b = (c0 + BN_PAGE <= pos) ? pt[c0 / BN_PAGE + 1] : page_a;
  auto row_off = [&](int j) -> size_t {  // cache row of key/value j of this chunk (0 <= j < 128)
    int page = j < BN_PAGE ? page_a : page_b;
    return (((size_t)page * n_kv_heads + kvh) * BN_PAGE + (j & (BN_PAGE - 1))) * (size_t)head_dim;
  };
  const int real_chunks = head_dim / 8;
  const int new_row = (pos / DT_CHUNK == split) ? pos - c0 : -1;  // the new token's row, if it is in this chunk
  const int j_lo = max(0, lo - c0), j_hi = min(DT_CHUNK, pos - c0 + 1);  // visible rows [j_lo, j_hi)

  // ---- ask for the chunk's keys and values (rows outside the range and padding dimensions are zero)
  for (int p = tid; p < DT_CHUNK * CHUNKS; p += DT_THREADS) {
    int r = p / CHUNKS, c = p - r * CHUNKS;
    if (r == new_row) continue;  // written below from the new token's row
    bool ok = r >= j_lo && r < j_hi && c < real_chunks;
    size_t off = ok ? row_off(r) + (size_t)c * 8 : 0;
    dt_cp_async16(s_k + dt_off<HD>(r, c), a.k_cache + off, ok);
    dt_cp_async16(s_v + dt_off<HD>(r, c), a.v_cache + off, ok);
  }
  asm volatile("cp.async.commit_group;");

  // ---- queries of this head group: rotate, round to bfloat16, place as rows of the 16-row tile
  const __nv_bfloat16* qrow = a.qkv + (size_t)b * a.q_stride;
  const int half = a.rotary_dims >> 1;
  auto q_at = [&](int g, int d) -> __nv_bfloat16* {
    return reinterpret_cast<__nv_bfloat16*>(q_tile + dt_off<HD>(g, d >> 3)) + (d & 7);
  };
  for (int p = tid; p < DT_ROWS * HD; p += DT_THREADS) {  // zero rows past G and padding dimensions
    int g = p / HD, d = p - g * HD;
    if (g >= G || d >= head_dim) *q_at(g, d) = __float2bfloat16_rn(0.f);
  }
  for (int p = tid; p < G * half; p += DT_THREADS) {
    int g = p / half, i = p - g * half;
    float s, c;
    sincosf(dt_angle(pos, i, a.theta_scale), &s, &c);
    const __nv_bfloat16* hd = qrow + (size_t)(h0 + g) * head_dim;
    float x = __bfloat162float(hd[i]), y = __bfloat162float(hd[i + half]);
    *q_at(g, i) = __float2bfloat16_rn(x * c - y * s);
    *q_at(g, i + half) = __float2bfloat16_rn(x * s + y * c);
  }
  {
    const int rest = head_dim - a.rotary_dims;
    for (int p = tid; p < G * rest; p += DT_THREADS) {
      int g = p / rest, d = a.rotary_dims + p - g * rest;
      *q_at(g, d) = qrow[(size_t)(h0 + g) * head_dim + d];
    }
  }
  // ---- the new token's key (rotated) and value: to the cache and into this block's tiles
  if (new_row >= 0) {
    const size_t off = row_off(new_row);
    const __nv_bfloat16* kraw = qrow + a.k_off + (size_t)kvh * head_dim;
    const __nv_bfloat16* vraw = qrow + a.v_off + (size_t)kvh * head_dim;
    auto tile_at = [&](unsigned char* tile, int d) -> __nv_bfloat16* {
      return reinterpret_cast<__nv_bfloat16*>(tile + dt_off<HD>(new_row, d >> 3)) + (d & 7);
    };
    for (int i = tid; i < half; i += DT_THREADS) {
      float s, c;
      sincosf(dt_angle(pos, i, a.theta_scale), &s, &c);
      float x = __bfloat162float(kraw[i]), y = __bfloat162float(kraw[i + half]);
      __nv_bfloat16 k0 = __float2bfloat16_rn(x * c - y * s), k1 = __float2bfloat16_rn(x * s + y * c);
      a.k_cache[off + i] = k0;
      a.k_cache[off + i + half] = k1;
      *tile_at(k_tile, i) = k0;
      *tile_at(k_tile, i + half) = k1;
    }
    for (int d = a.rotary_dims + tid; d < head_dim; d += DT_THREADS) {
      a.k_cache[off + d] = kraw[d];
      *tile_at(k_tile, d) = kraw[d];
    }
    for (int d = tid; d < head_dim; d += DT_THREADS) {
      a.v_cache[off + d] = vraw[d];
      *tile_at(v_tile, d) = vraw[d];
    }
    for (int d = head_dim + tid; d < HD; d += DT_THREADS) {  // padding dimensions of the new row
      *tile_at(k_tile, d) = __float2bfloat16_rn(0.f);
      *tile_at(v_tile, d) = __float2bfloat16_rn(0.f);
    }
  }
  asm volatile("cp.async.wait_group 0;");
  __syncthreads();

  // ---- this warp's 32 keys: S = Q K^T
  float s[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
  const int krow0 = warp * 32;
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    unsigned a0, a1, a2, a3;
    const int mi = lane >> 3, r = lane & 7;
    dt_ldsm_x4(s_q + dt_off<HD>(r + (mi & 1) * 8, ks * 2 + (mi >> 1)), a0, a1, a2, a3);
#pragma unroll
    for (int j = 0; j < 4; j += 2) {
      unsigned b0, b1, b2, b3;
      dt_ldsm_x4(s_k + dt_off<HD>(krow0 + (j + (mi >> 1)) * 8 + r, ks * 2 + (mi & 1)), b0, b1, b2, b3);
      dt_mma(s[j], a0, a1, a2, a3, b0, b1);
      dt_mma(s[j + 1], a0, a1, a2, a3, b2, b3);
    }
  }
  // mask, maximum, exponentials, sum; rows g4 and g4 + 8 of the head tile
  float m_w[2] = {-INFINITY, -INFINITY}, l_w[2] = {0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      int jr = krow0 + j * 8 + 2 * t4 + (c & 1);
      bool ok = jr >= j_lo && jr < j_hi;
      float v = ok ? s[j][c] * a.scale_log2e : -INFINITY;
      s[j][c] = v;
      m_w[c >> 1] = fmaxf(m_w[c >> 1], v);
    }
  }
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    m_w[e] = fmaxf(m_w[e], __shfl_xor_sync(0xffffffffu, m_w[e], 1));
    m_w[e] = fmaxf(m_w[e], __shfl_xor_sync(0xffffffffu, m_w[e], 2));
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      int e = c >> 1;
      float p = (m_w[e] == -INFINITY) ? 0.f : exp2f(s[j][c] - m_w[e]);
      s[j][c] = p;
      l_w[e] += p;
    }
  }
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    l_w[e] += __shfl_xor_sync(0xffffffffu, l_w[e], 1);
    l_w[e] += __shfl_xor_sync(0xffffffffu, l_w[e], 2);
  }
  // ---- O = P V over this warp's 32 keys
  float o[NT_O][4];
#pragma unroll
  for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < 2; ++ks) {
    unsigned a0 = dt_pack(s[2 * ks][0], s[2 * ks][1]);
    unsigned a1 = dt_pack(s[2 * ks][2], s[2 * ks][3]);
    unsigned a2 = dt_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]);
    unsigned a3 = dt_pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
    const int mi = lane >> 3, r = lane & 7;
#pragma unroll
    for (int j = 0; j < NT_O; j += 2) {
      unsigned b0, b1, b2, b3;
      dt_ldsm_x4_trans(s_v + dt_off<HD>(krow0 + ks * 16 + (mi & 1) * 8 + r, j + (mi >> 1)), b0, b1, b2, b3);
      dt_mma(o[j], a0, a1, a2, a3, b0, b1);
      dt_mma(o[j + 1], a0, a1, a2, a3, b2, b3);
    }
  }
  __syncthreads();  // every warp has read the key tile: it now holds the warps' partial outputs
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    int row = g4 + e * 8;
    if (t4 == 0) {
      ml_part[(warp * DT_ROWS + row) * 2] = m_w[e];
      ml_part[(warp * DT_ROWS + row) * 2 + 1] = l_w[e];
    }
#pragma unroll
    for (int j = 0; j < NT_O; ++j) {
      float2 v = make_float2(o[j][2 * e], o[j][2 * e + 1]);
      *reinterpret_cast<float2*>(o_part + ((size_t)(warp * DT_ROWS + row)) * HD + j * 8 + 2 * t4) = v;
    }
  }
  __syncthreads();
  // ---- merge the four warps: this chunk's unnormalised partial, its maximum and its sum
  if (tid < G) {
    float m = -INFINITY;
    for (int w = 0; w < 4; ++w) m = fmaxf(m, ml_part[(w * DT_ROWS + tid) * 2]);
    float l = 0.f;
    for (int w = 0; w < 4; ++w) {
      float mw = ml_part[(w * DT_ROWS + tid) * 2];
      if (mw != -INFINITY) l += exp2f(mw - m) * ml_part[(w * DT_ROWS + tid) * 2 + 1];
    }
    ml_fin[tid * 2] = m;
    ml_fin[tid * 2 + 1] = l;
    size_t oo = (((size_t)b * n_heads + h0 + tid) * a.n_splits + split) * 2;
    a.part_ml[oo] = m;
    a.part_ml[oo + 1] = l;
  }
  __syncthreads();
  for (int i = tid; i < G * head_dim; i += DT_THREADS) {
    int g = i / head_dim, d = i - g * head_dim;
    float m = ml_fin[g * 2], acc = 0.f;
    for (int w = 0; w < 4; ++w) {
      float mw = ml_part[(w * DT_ROWS + g) * 2];
      if (mw != -INFINITY) acc += exp2f(mw - m) * o_part[(size_t)(w * DT_ROWS + g) * HD + d];
    }
    a.part_o[(((size_t)b * n_heads + h0 + g) * a.n_splits + split) * head_dim + d] = acc;
  }

  // ---- the block that draws the last ticket of this (sequence, head group) merges the chunks
  const int s0 = lo / DT_CHUNK, s1 = pos / DT_CHUNK;
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
    for (int s_ = s0; s_ <= s1; ++s_) m = fmaxf(m, __ldcg(ml + 2 * s_));
    float den = 0.f;
    for (int s_ = s0; s_ <= s1; ++s_) den += exp2f(__ldcg(ml + 2 * s_) - m) * __ldcg(ml + 2 * s_ + 1);
    ml_fin[tid * 2] = m;
    ml_fin[tid * 2 + 1] = den;
  }
  __syncthreads();
  for (int i = tid; i < G * head_dim; i += DT_THREADS) {
    int g = i / head_dim, d = i - g * head_dim;
    const float* ml = a.part_ml + ((size_t)b * n_heads + h0 + g) * a.n_splits * 2;
    const float* po = a.part_o + ((size_t)b * n_heads + h0 + g) * a.n_splits * head_dim;
    float m = ml_fin[g * 2], num = 0.f;
    for (int s_ = s0; s_ <= s1; ++s_) num += exp2f(__ldcg(ml + 2 * s_) - m) * __ldcg(po + (size_t)s_ * head_dim + d);
    a.out[(size_t)b * a.out_stride + (size_t)(h0 + g) * head_dim + d] = __float2bfloat16_rn(num / ml_fin[g * 2 + 1]);
  }
}

template <int HD>
static int launch_dt(const DtArgs& a, dim3 grid, cudaStream_t stream) {
  size_t smem = (size_t)DT_ROWS * HD * 2 + 2 * (size_t)DT_CHUNK * HD * 2 + (4 * DT_ROWS * 2 + DT_ROWS * 2) * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
    configured = true;
  }
  BN_LAUNCH(attention_decode_tc_kernel<HD>, grid, DT_THREADS, smem, stream, a);
  return BN_OK;
}

// qkv: [n_seqs, q_stride] bfloat16 rows with the raw query heads first, the key heads at element
// k_off and the value heads at v_off (all multiples of 8 elements).  The kernel rotates queries and
// the new key (rotary_dims = 0: none), writes the new key and value into the cache at tok_pos[b],
// attends and combines.  part_o / part_ml: scratch of n_seqs * n_heads * n_splits * head_dim and
// n_seqs * n_heads * n_splits * 2 floats, n_splits * 128 covering the longest sequence;
// tickets: n_seqs * n_kv_heads * ceil(group / 16) ints, zero before and after.
extern "C" int bn_attention_decode_tc(const void* qkv, int q_stride, int k_off, int v_off, void* out, int out_stride,
                                      int n_seqs, int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                      int rotary_dims, float theta_scale, const int* tok_pos, const int* slots,
                                      const int* page_table, int pt_stride, void* k_cache, void* v_cache,
                                      float* part_o, float* part_ml, int n_splits, int* tickets, int n_tickets,
                                      cudaStream_t stream) {
  if (n_seqs <= 0) return BN_OK;
  if (head_dim <= 0 || head_dim % 16 || head_dim > 256 || n_kv_heads <= 0 || n_heads % n_kv_heads || n_splits <= 0 ||
      window < 0 || !part_o || !part_ml || !tickets || rotary_dims < 0 || rotary_dims > head_dim || (rotary_dims & 1))
    return BN_ERR_BAD_ARG;
  int group = n_heads / n_kv_heads;
  int gblocks = (group + DT_ROWS - 1) / DT_ROWS;
  if ((long long)n_kv_heads * gblocks > 65535 || n_splits > 65535 ||
      (long long)n_seqs * n_kv_heads * gblocks > n_tickets)
    return BN_ERR_BAD_ARG;
  DtArgs a = {};
  a.qkv = (const __nv_bfloat16*)qkv; a.q_stride = q_stride; a.k_off = k_off; a.v_off = v_off;
  a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim;
  a.scale_log2e = scale * 1.4426950408889634f; a.window = window; a.rotary_dims = rotary_dims;
  a.theta_scale = theta_scale; a.tok_pos = tok_pos; a.slots = slots; a.page_table = page_table; a.pt_stride = pt_stride;
  a.k_cache = (__nv_bfloat16*)k_cache; a.v_cache = (__nv_bfloat16*)v_cache; a.part_o = part_o; a.part_ml = part_ml;
  a.n_splits = n_splits; a.tickets = tickets; a.out = (__nv_bfloat16*)out; a.out_stride = out_stride;
  dim3 grid(n_seqs, n_kv_heads * gblocks, n_splits);
  if (head_dim <= 64) return launch_dt<64>(a, grid, stream);
  if (head_dim <= 128) return launch_dt<128>(a, grid, stream);
  return launch_dt<256>(a, grid, stream);
}
