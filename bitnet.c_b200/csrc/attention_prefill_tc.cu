// Causal attention of many new tokens per sequence in bfloat16 (prefill) on the 5th-generation
// tensor cores: scores and the weighted value sum are tcgen05.mma instructions with their
// accumulators in tensor memory, operands arrive by TMA.
//
// One block takes 128 consecutive new tokens of one sequence and one query head and walks the
// sequence's cache pages (64 positions of one key/value head, contiguous: one key tile) from the
// first visible key to the last.  Per page j:
//     S_j = Q K_j^T          M=128, N=64,  K=head size   -> tensor memory, two buffers
//     P_j = exp2(S_j * scale * log2(e) - m)  in float32 by 128 threads, one query row each (the
//                             row of the accumulator is the thread's own TMEM lane: no shuffles),
//                             rounded to bfloat16 and written back into tensor memory, over the
//                             first half of the columns S_j came from
//     O  += P_j V_j          M=128, N=head size, K=64    -> tensor memory
// Roles of the 192 threads: warp 0 requests Q once and the pages through a ring of stages (TMA,
// 128-byte swizzle); one thread of warp 1 issues the MMAs, S_{j+1} ahead of P_j V_j so that the
// tensor pipe works on the next scores while the softmax warps handle the current ones; warps 2-5
// do the softmax and the epilogue.  The running maximum m of a row is only raised when the new
// maximum exceeds it by more than 8 (a factor 256, harmless in float32 and bfloat16); then the
// row's O is rescaled in tensor memory.  Sums and maxima are float32; the result is O / sum.
//
// P is the second product's A operand read from tensor memory (two bfloat16 per 32-bit column);
// the tensor pipe runs its instructions in order, so S_{j+2}, issued after P_j V_j, cannot
// overwrite P_j before it has been used.  V is that product's B operand with the head dimension
// contiguous (MN-major); K and Q are K-major.
// The new tokens' own keys and values must already be in the cache, so the same kernel serves
// whole prompts, pieces of prompts and ragged batches (a table gives each block its sequence and
// first row).  Head sizes in steps of 16 up to 128 run on the instantiation for 64 or 128: columns
// past the head size read as zero (TMA fills what lies outside the tensor).  Value rows behind a
// sequence's last position are cleared in shared memory, whatever the cache holds there.
//
// Every wait on an mbarrier is bounded in time; a wait that gives up sets a flag that ends all
// other waits of the block, records a code in *status, and the block drains, frees its tensor
// memory and returns without storing.
//
// Reference: per (head, token) scores over the cached keys 0..pos, scale 1/sqrt(head size),
// softmax, weighted sum of values; the key/value head of query head h is h / (H / KV)
// (src/transformer/batched_attn_scalar.c:97-169, flash variant :171-245).  The reference's CUDA
// prefill attention is one block per (head, token) on CUDA cores (src/gpu_cuda.cu:9772).
#include "tma.cuh"
#include "umma.cuh"

#define PT_ROWS 128      // query rows per block (UMMA M)
#define PT_KEYS 64       // keys per tile = BN_PAGE
#define PT_THREADS 192
#define PT_RESCALE 8.0f  // raise a row's reference maximum only beyond this (log2 domain)
#define PT_ERR_WAIT 5

struct PtArgs {
  __nv_bfloat16* out;
  int out_stride;
  int n_heads, n_kv_heads, head_dim;
  float scale_log2e;
  int window;
  const int* tile_seq;
  const int* tile_row0;
  const int* seq_start;
  const int* seq_pos0;
  const int* slots;
  const int* page_table;
  int pt_stride;
  int* status;
  BN_TRACE_ONLY(unsigned long long* trace;)  // debugging: timestamps of block (0, 0), or null
};
#define PT_TRACE_TILES 12  // per tile: 6 stamps of a softmax thread, 3 of the MMA thread

// Bounded wait that also ends when another thread of the block has given up.
__device__ __forceinline__ bool pt_wait(unsigned bar, unsigned parity, volatile int* failed, int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = global_timer();
  for (;;) {
    if (mbar_try_wait_for(bar, parity, TMA_SUSPEND_NS)) return true;
    if (*failed) return false;
    if (global_timer() - t0 > TMA_WAIT_NS) {
      *failed = 1;
      atomicExch(status, PT_ERR_WAIT);
      return false;
    }
  }
}

template <int HD, int KS, int VS>
__global__ void __launch_bounds__(PT_THREADS)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, PtArgs a) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr int BOXES = HD / 64;
  constexpr int Q_BOX = PT_ROWS * 128;             // 16 KB: 128 rows x 64 dimensions
  constexpr int KV_BOX = PT_KEYS * 128;            // 8 KB: 64 keys x 64 dimensions
  constexpr int Q_BYTES = BOXES * Q_BOX;
  constexpr int PAGE_BYTES = BOXES * KV_BOX;       // one page of keys (or values) of one head
  constexpr unsigned TMEM_COLS = 256;              // S0 at 0, S1 at 64, O at 128
  constexpr unsigned O_COL = 128;
  // D float32, A and B bfloat16, M = 128; scores: N = 64, both operands K-major; output: N = HD, B MN-major
  constexpr unsigned IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(PT_KEYS >> 3) << 17) | ((PT_ROWS >> 4) << 24);
  constexpr unsigned IDESC_O = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(HD >> 3) << 17) | ((PT_ROWS >> 4) << 24);

  // The block has no static shared memory, so the dynamic part starts at the (1024-byte aligned)
  // base of the block's window: the swizzle is a function of the address.
  unsigned char* q_smem = smem_raw;
  unsigned char* k_smem = q_smem + Q_BYTES;                   // KS pages of keys
  unsigned char* v_smem = k_smem + KS * PAGE_BYTES;           // VS pages of values
  unsigned long long* bars = (unsigned long long*)(v_smem + VS * PAGE_BYTES);
  // barriers: q_full, k_full[KS], k_empty[KS], v_full[VS], v_empty[VS], s_full[2], p_full[2], pv_done
  const unsigned bar0 = smem_u32(bars);
  const unsigned q_full = bar0, k_full0 = bar0 + 8, k_empty0 = k_full0 + 8 * KS, v_full0 = k_empty0 + 8 * KS,
                 v_empty0 = v_full0 + 8 * VS, s_full0 = v_empty0 + 8 * VS,
                 p_full0 = s_full0 + 16, pv_done = p_full0 + 16;
  unsigned* tmem_slot = (unsigned*)(bars + 2 * KS + 2 * VS + 6);
  volatile int* failed = (volatile int*)(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Blocks start in the order of their index, heads fastest: the last tiles of a sequence see the
  // most keys and start first, over all heads, so that the short tiles fill the tail; and the query
  // heads that share a key/value head run side by side and find its pages in the L2.
  const int blk = gridDim.y - 1 - blockIdx.y;
  const int seq = a.tile_seq[blk], row0 = a.tile_row0[blk], h = blockIdx.x;
  const int head_dim = a.head_dim;
  const int kvh = h / (a.n_heads / a.n_kv_heads);
  const int start = a.seq_start[seq], n_new = a.seq_start[seq + 1] - start, pos0 = a.seq_pos0[seq];
  const int* pt = a.page_table + (size_t)a.slots[seq] * a.pt_stride;
  const int rows_here = min(PT_ROWS, n_new - row0);
  // visible key range of this block
  const int q_first = pos0 + row0, q_last = q_first + rows_here - 1;
  const int lo_first = a.window > 0 ? max(0, q_first - a.window + 1) : 0;
  const int tile_lo = lo_first / PT_KEYS, tile_hi = q_last / PT_KEYS;
  const int n_tiles = tile_hi - tile_lo + 1;
  const int seq_last = pos0 + n_new - 1;  // the last position of this sequence that the cache holds

  if (tid == 0) {
    *failed = 0;
    if (smem_u32(smem_raw) & 1023u) {  // a misplaced window would make every tile wrong: give up at once
      *failed = 1;
      atomicExch(a.status, PT_ERR_WAIT);
    }
    tma_prefetch_map(&map_q);
    tma_prefetch_map(&map_k);
    tma_prefetch_map(&map_v);
    mbar_init(q_full, 1);
    for (int s = 0; s < KS; ++s) {
      mbar_init(k_full0 + 8 * s, 1);
      mbar_init(k_empty0 + 8 * s, 1);
    }
    for (int s = 0; s < VS; ++s) {
      mbar_init(v_full0 + 8 * s, 1);
      mbar_init(v_empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_full0 + 8 * b, 1);
      mbar_init(p_full0 + 8 * b, 4);  // one arrival per softmax warp
    }
    mbar_init(pv_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;
  pdl_wait();  // q and this step's cache rows come from the kernels before this one

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int bx = 0; bx < BOXES; ++bx)
        tma_load_2d(smem_u32(q_smem + bx * Q_BOX), &map_q, q_full, h * head_dim + bx * 64, start + row0);
      // Keys and values have rings of their own: a key stage is free as soon as the scores that
      // read it are done, a value stage only after the output product, one softmax later.  The
      // order of the requests is the order in which the stages come free: K(t + KS - 1), then V(t).
      auto request = [&](int j, bool values) -> bool {
        const int n = values ? VS : KS, s = j % n, round = j / n;
        const unsigned empty = (values ? v_empty0 : k_empty0) + 8 * s, bar = (values ? v_full0 : k_full0) + 8 * s;
        const int page = __ldg(pt + tile_lo + j);  // asked for before the wait, needed after it
        if (round > 0 && !pt_wait(empty, (unsigned)(round - 1) & 1u, failed, a.status)) return false;
        const unsigned dst = smem_u32((values ? v_smem : k_smem) + s * PAGE_BYTES);
        mbar_expect_tx(bar, PAGE_BYTES);
#pragma unroll
        for (int bx = 0; bx < BOXES; ++bx)
          tma_load_3d(dst + bx * KV_BOX, values ? &map_v : &map_k, bar, bx * 64, kvh * BN_PAGE, page);
        return true;
      };
      bool ok = true;
      for (int j = 0; ok && j < min(KS - 1, n_tiles); ++j) ok = request(j, false);
      for (int t = 0; ok && t < n_tiles; ++t) {
        if (t + KS - 1 < n_tiles) ok = request(t + KS - 1, false);
        if (ok) ok = request(t, true);
      }
    }
  } else if (warp == 1) {
    // The whole warp walks the loop, so that addresses and descriptors are warp-uniform values;
    // one elected lane issues the MMAs and commits.
    const bool issuer = elect_one();
    const unsigned tbase = __shfl_sync(0xffffffffu, tmem_base, 0);
    bool ok = __all_sync(0xffffffffu, pt_wait(q_full, 0, failed, a.status));
    const unsigned sq = smem_u32(q_smem);
    BN_TRACE_ONLY(const bool tracing = a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && issuer;)
    for (int j = 0; ok && j <= n_tiles; ++j) {
      if (j < n_tiles) {
        // S_j = Q K_j^T into score buffer j & 1
        const int s = j % KS, b = j & 1;
        BN_TRACE_ONLY(const bool trs = tracing && j < PT_TRACE_TILES;)
        ok = __all_sync(0xffffffffu, pt_wait(k_full0 + 8 * s, (unsigned)(j / KS) & 1u, failed, a.status));
        if (!ok) break;
        BN_TRACE_ONLY(if (trs) a.trace[j * 12 + 9] = global_timer();)
        // (S_j reuses the buffer of S_{j-2} and P_{j-2}: P_{j-2} V_{j-2} was issued before and the
        // tensor pipe keeps the order)
        BN_TRACE_ONLY(if (trs) a.trace[j * 12 + 10] = global_timer();)
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned sk = smem_u32(k_smem + s * PAGE_BYTES);
        if (issuer) {
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks)
            umma_mma(tbase + b * PT_KEYS, umma_desc_k(sq + (ks >> 2) * Q_BOX + (ks & 3) * 32),
                   umma_desc_k(sk + (ks >> 2) * KV_BOX + (ks & 3) * 32), IDESC_S, ks ? 1u : 0u);
          BN_TRACE_ONLY(if (trs) a.trace[j * 12 + 11] = global_timer();)
          umma_commit(k_empty0 + 8 * s);  // the key stage may be refilled
          umma_commit(s_full0 + 8 * b);
          BN_TRACE_ONLY(if (trs) a.trace[j * 12 + 6] = global_timer();)
        }
        __syncwarp();
      }
      if (j >= 1) {
        // O += P_{j-1} V_{j-1}
        const int i = j - 1, s = i % VS, b = i & 1;
        ok = __all_sync(0xffffffffu, pt_wait(p_full0 + 8 * b, (unsigned)(i >> 1) & 1u, failed, a.status) &&
                                         pt_wait(v_full0 + 8 * s, (unsigned)(i / VS) & 1u, failed, a.status));
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        BN_TRACE_ONLY(const bool tr = tracing && i < PT_TRACE_TILES;)
        BN_TRACE_ONLY(if (tr) a.trace[i * 12 + 7] = global_timer();)
        const unsigned sv = smem_u32(v_smem + s * PAGE_BYTES);
        if (issuer) {
#pragma unroll
          for (int kk = 0; kk < PT_KEYS / 16; ++kk)
            umma_mma_ts(tbase + O_COL, tbase + b * PT_KEYS + kk * 8, umma_desc_mn(sv + kk * 2048, KV_BOX), IDESC_O,
                      (i | kk) ? 1u : 0u);
          umma_commit(v_empty0 + 8 * s);    // the value stage may be refilled
          umma_commit(pv_done);             // O holds the pages up to i
          BN_TRACE_ONLY(if (tr) a.trace[i * 12 + 8] = global_timer();)
        }
        __syncwarp();
      }
    }
  } else {
    // ---- softmax and epilogue: thread <-> query row <-> TMEM lane
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const unsigned lane_addr = tmem_base + ((unsigned)(quad * 32) << 16);
    // rows past the sequence's tokens look like the first row so that they see at least one key
    const int qpos = r < rows_here ? q_first + r : q_first;
    const int qlo = a.window > 0 ? max(0, qpos - a.window + 1) : 0;
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int b = j & 1, tile = tile_lo + j;
      BN_TRACE_ONLY(const bool tr = a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && tid == 64 && j < PT_TRACE_TILES;)
      BN_TRACE_ONLY(if (tr) a.trace[j * 12 + 0] = global_timer();)
      if (!pt_wait(s_full0 + 8 * b, (unsigned)(j >> 1) & 1u, failed, a.status)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      BN_TRACE_ONLY(if (tr) a.trace[j * 12 + 1] = global_timer();)
      float s[PT_KEYS];
      tmem_ld64(lane_addr + b * PT_KEYS, s);
      BN_TRACE_ONLY(if (tr) a.trace[j * 12 + 2] = global_timer();)
      // mask, then the maximum of the raw scores (the scale is positive); four chains, not one
      const int k0 = tile * PT_KEYS;
      if (!(k0 >= qlo && k0 + PT_KEYS - 1 <= qpos)) {
#pragma unroll
        for (int k = 0; k < PT_KEYS; ++k) {
          const int kpos = k0 + k;
          if (!(kpos >= qlo && kpos <= qpos)) s[k] = -INFINITY;
        }
      }
      float mx[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
      for (int k = 4; k < PT_KEYS; ++k) mx[k & 3] = fmaxf(mx[k & 3], s[k]);
      const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * a.scale_log2e;
      bool need = false;
      if (m_ref == -INFINITY) m_ref = m_tile;  // nothing accumulated for this row yet: O and the sum are zero
      else need = m_tile > m_ref + PT_RESCALE;
      if (__any_sync(0xffffffffu, need)) {
        // O of the pages before this one must be complete before it is rescaled (j >= 1 here)
        if (!pt_wait(pv_done, (unsigned)(j - 1) & 1u, failed, a.status)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float alpha = need ? exp2f(m_ref - m_tile) : 1.0f;
        if (need) { m_ref = m_tile; l_run *= alpha; }
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          float o[32];
          tmem_ld32(lane_addr + O_COL + c, o);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= alpha;
          tmem_st32(lane_addr + O_COL + c, o);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      // exponentials 2^(s * scale - m) and the row's sum (a row that has seen no key yet has only
      // -inf scores, which give 0 whatever m is)
      const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int k = 0; k < PT_KEYS; ++k) {
        s[k] = ex2_approx(fmaf(s[k], a.scale_log2e, neg_m));
        ls[k & 3] += s[k];
      }
      l_run += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      BN_TRACE_ONLY(if (tr) a.trace[j * 12 + 3] = global_timer();)
      // P as bfloat16 into tensor memory, two keys per column, over the columns S came from
      BN_TRACE_ONLY(if (tr) a.trace[j * 12 + 4] = global_timer();)
      {
        float pk[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) pk[c] = __uint_as_float(pack_bf16x2(s[2 * c], s[2 * c + 1]));
        tmem_st32(lane_addr + b * PT_KEYS, pk);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      if (tile * PT_KEYS + PT_KEYS - 1 > seq_last) {
        // the page holds rows behind the sequence's last position: their weights are zero, but zero
        // times anything must be zero, so clear those value rows (warp w takes every fourth row)
        unsigned char* sv = v_smem + (j % VS) * PAGE_BYTES;
        const int first = max(0, seq_last + 1 - tile * PT_KEYS);
        for (int e = (warp - 2) * 32 + lane; e < (PT_KEYS - first) * (HD / 8); e += 128) {
          int row = first + e / (HD / 8), c = e % (HD / 8);
          *reinterpret_cast<uint4*>(sv + (c >> 3) * KV_BOX + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // before the MMA reads the cleared rows
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full0 + 8 * b);
      BN_TRACE_ONLY(if (tr) a.trace[j * 12 + 5] = global_timer();)
    }
    // ---- epilogue: O / sum -> out
    if (ok && pt_wait(pv_done, (unsigned)(n_tiles - 1) & 1u, failed, a.status)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv = 1.0f / l_run;
      __nv_bfloat16* orow = a.out + (size_t)(start + row0 + r) * a.out_stride + (size_t)h * head_dim;
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        float o[32];
        tmem_ld32(lane_addr + O_COL + c, o);
        if (r < rows_here) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            if (c + g * 8 < head_dim) {  // head sizes are multiples of 16: groups of 8 are whole
              uint4 w = make_uint4(pack_bf16x2(o[g * 8] * inv, o[g * 8 + 1] * inv), pack_bf16x2(o[g * 8 + 2] * inv, o[g * 8 + 3] * inv),
                                   pack_bf16x2(o[g * 8 + 4] * inv, o[g * 8 + 5] * inv), pack_bf16x2(o[g * 8 + 6] * inv, o[g * 8 + 7] * inv));
              *reinterpret_cast<uint4*>(orow + c + g * 8) = w;
            }
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*failed) {
    // a wait gave up: loads that were requested may still be landing in this block's shared memory
    unsigned long long t0 = global_timer();
    while (global_timer() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

#ifdef BN_TRACE
// Debugging aid: bn_attention_prefill_tc_trace(1) makes the next launch record timestamps of block
// (0, 0) (device buffer allocated here; not used on the product path).
static unsigned long long* g_pt_trace = nullptr;
static bool g_pt_trace_armed = false;
extern "C" int bn_attention_prefill_tc_trace(int on) {
  if (g_pt_trace) cudaFree(g_pt_trace);
  g_pt_trace = nullptr; g_pt_trace_armed = false;
  if (!on) return 0;
  if (cudaMalloc(&g_pt_trace, PT_TRACE_TILES * 12 * 8) != cudaSuccess) return 1;
  cudaMemset(g_pt_trace, 0, PT_TRACE_TILES * 12 * 8);
  g_pt_trace_armed = true;
  return 0;
}
extern "C" int bn_attention_prefill_tc_trace_read(unsigned long long* host) {
  if (!g_pt_trace) return 1;
  return cudaMemcpy(host, g_pt_trace, PT_TRACE_TILES * 12 * 8, cudaMemcpyDeviceToHost) != cudaSuccess;
}
#endif

template <int HD, int KS, int VS>
static int launch_pt(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const PtArgs& a, int n_tiles,
                     cudaStream_t stream) {
  size_t smem = (size_t)PT_ROWS * HD * 2 + (size_t)(KS + VS) * PT_KEYS * HD * 2 + (2 * KS + 2 * VS + 6) * 8 + 16;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<HD, KS, VS>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
    configured = true;
  }
  if (n_tiles > 65535) return BN_ERR_BAD_ARG;
  dim3 grid(a.n_heads, n_tiles);
  BN_LAUNCH((attention_prefill_tc_kernel<HD, KS, VS>), grid, PT_THREADS, smem, stream, mq, mk, mv, a);
  return BN_OK;
}

// q: [n_tokens, q_stride] bfloat16 (head h at element h*head_dim; 16-byte aligned, q_stride a
// multiple of 8), out [n_tokens, out_stride] (out_stride a multiple of 8, 16-byte aligned).
// tile_seq / tile_row0: for each block its sequence and the first of its 128 new-token rows;
// seq_start [n_seqs+1]: first packed row of each sequence; seq_pos0: its length before the step.
// The caches are [n_cache_pages, n_kv_heads, 64, head_dim], contiguous and 16-byte aligned, and
// already hold the new tokens.  head_dim: a multiple of 16 up to 128.  status: one int on the
// device, left as it is unless a wait inside the kernel gave up (then 5; nothing is stored by
// that block).
extern "C" int bn_attention_prefill_tc(const void* q, int q_stride, int n_tokens, void* out, int out_stride, int n_tiles,
                                       int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                       const int* tile_seq, const int* tile_row0, const int* seq_start,
                                       const int* seq_pos0, const int* slots, const int* page_table, int pt_stride,
                                       const void* k_cache, const void* v_cache, int n_cache_pages, int* status,
                                       cudaStream_t stream) {
  if (n_tiles <= 0) return BN_OK;
  if (head_dim <= 0 || head_dim % 16 || head_dim > 128 || n_kv_heads <= 0 || n_heads % n_kv_heads || window < 0 ||
      n_heads > 65535 || (q_stride % 8) || (out_stride % 8) || n_tokens <= 0 || n_cache_pages <= 0 || !status ||
      (((uintptr_t)q | (uintptr_t)out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15))
    return BN_ERR_BAD_ARG;
  CUtensorMap mq, mk, mv;
  if (!tma_map_bf16_strided(&mq, q, (unsigned long long)n_tokens, (unsigned long long)n_heads * head_dim,
                            (unsigned long long)q_stride, PT_ROWS) ||
      !tma_map_bf16_pages(&mk, k_cache, n_cache_pages, (unsigned long long)n_kv_heads * BN_PAGE, head_dim, BN_PAGE) ||
      !tma_map_bf16_pages(&mv, v_cache, n_cache_pages, (unsigned long long)n_kv_heads * BN_PAGE, head_dim, BN_PAGE))
    return BN_ERR_BAD_ARG;
  PtArgs a = {};
  a.out = (__nv_bfloat16*)out; a.out_stride = out_stride; a.n_heads = n_heads; a.n_kv_heads = n_kv_heads;
  a.head_dim = head_dim; a.scale_log2e = scale * 1.4426950408889634f; a.window = window; a.tile_seq = tile_seq;
  a.tile_row0 = tile_row0; a.seq_start = seq_start; a.seq_pos0 = seq_pos0; a.slots = slots; a.page_table = page_table;
  a.pt_stride = pt_stride; a.status = status;
  BN_TRACE_ONLY(a.trace = nullptr;)
  BN_TRACE_ONLY(if (g_pt_trace_armed) { a.trace = g_pt_trace; g_pt_trace_armed = false; })
  // shared memory per block: 64 KB and 96 KB, so that two blocks share an SM (tensor memory
  // allows no more: 256 columns each) and one block's softmax overlaps the other's products
  // (a third key stage at head size 128 was measured and changes nothing: the softmax is the pace)
  if (head_dim <= 64) return launch_pt<64, 3, 3>(mq, mk, mv, a, n_tiles, stream);
  return launch_pt<128, 2, 2>(mq, mk, mv, a, n_tiles, stream);
}
