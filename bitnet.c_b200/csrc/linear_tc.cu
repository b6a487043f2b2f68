// out[M, N] = x[M, K] . W[N, K]^T in bfloat16 on the 5th-generation tensor cores (tcgen05),
// for M <= 64: weights stream HBM -> shared memory by TMA, products accumulate in tensor memory.
//
// The roles are swapped so that the weight is the 128-row operand: D[128 weight rows, Mp batch
// columns] += W_tile[128, 64] . x_tile[Mp, 64]^T, one tcgen05.mma of shape M=128, N=Mp, K=16 per 16
// columns of k, issued by one thread.
//
// A tile is 128 weight rows.  Weights with few rows have fewer tiles than the GPU has SMs, so the
// inner dimension of a tile is split over a thread-block cluster of C blocks (C x tiles is about
// one and a half times the number of SMs): block r of the cluster multiplies k-blocks
// [r KB/C, (r+1) KB/C).  Each block leaves its float32 partial tile in its own shared memory; after a cluster barrier every block
// sends each other block the slice of rows that block owns, as one bulk copy from shared memory to
// the owner's shared memory that completes on an mbarrier there (distributed shared memory; a
// copy is posted and needs no round trip, where loads from another block's shared memory took 1
// to 4 us per tile).  The owner adds up its C copies of the slice in rank order and runs the
// epilogue on it.  Nothing goes through global memory, all blocks of a tile finish together, and
// the order of the additions is fixed.
//
// A block of 192 threads (320 with the wider accumulators):
//   warp 0     one thread issues the TMA loads of W and x tiles into a ring of stages and arms each
//              stage's "full" mbarrier with the bytes to expect;
//   warp 1     allocates tensor memory; one thread waits for "full", issues four MMAs per stage,
//              commits them to the stage's "empty" mbarrier and at the end to "accumulator full";
//   warps 2-5  wait for the accumulator, move it from tensor memory to shared memory
//              (tcgen05.ld, one weight row per thread), send and receive the slices, add them up
//              and store with consecutive threads on consecutive output columns.
// Tiles are 128-byte swizzled both by TMA and in the MMA's shared-memory descriptors.  No register
// ever holds a weight, so the bytes in flight per SM are the ring's size (about 100 KB); a block
// uses less than half of an SM's shared memory so that a block of the next kernel fits beside it.
//
// The kernel is launched with programmatic stream serialization: the loads of its first weight
// tiles are issued before griddepcontrol.wait, i.e. while the kernel before it in the stream is
// still draining; everything that reads x or writes memory comes after the wait.
//
// Epilogues: (0) store, (2) SwiGLU over weight rows that alternate 8 gate and 8 up rows, (3) add
// to a float32 residual in place and prepare the RMSNorm that follows it: the residual's new
// values times the norm's gain go out in bfloat16, and each block leaves the sum of squares of its
// slice of every row; the product that consumes those rows (any epilogue) multiplies its result
// rows by 1 / sqrt(sum of the parts / width + eps), which is the same as normalising its input
// rows (W (s x) = s (W x)).  The parts are added in a fixed order, statistics stay in float32.
//
// Every wait on an mbarrier is bounded in time; when a wait gives up the block records a code
// in *status, still takes part in the cluster barriers, lets its loads drain for a bounded time,
// frees its tensor memory and returns (tma.cuh).
//
// Reference for the operation: y = W x with float32 accumulation (src/quant/bf16_scalar.c:4-21);
// the reference's CUDA backend reaches tensor cores only through cuBLAS (src/gpu_cuda.cu:11850-11879).
#include "tma.cuh"
#include "umma.cuh"

#define TC_BM 128      // weight rows per tile (UMMA M)
#define TC_BK 64       // k per stage: 128 bytes of bfloat16, one swizzle row
// Ring depth by accumulator width: at most ~110 KB of shared memory per block, so that a block of
// the next kernel in the stream fits on the same SM and fetches its first weight tiles while this
// kernel's blocks are finishing (programmatic dependent launch).
#define TC_STAGES_FOR(MP) ((MP) == 16 ? 6 : ((MP) == 32 ? 5 : 4))
// Threads of a block: producer warp, MMA warp, and four epilogue warps (one per TMEM lane
// quadrant), eight for the two wider accumulators (two warps share a quadrant, half the columns each;
// sixteen would need more registers than two blocks per SM have).
// (An accumulator of 128 columns with a ring of three stages was tried for 65 to 128 rows: the library
// product is faster there, 3.1 against 3.7 ms for the products of 32 layers of width 4096.)
#define TC_EPI_FOR(MP) ((MP) >= 32 ? 256 : 128)
#define TC_THREADS_FOR(MP) (64 + TC_EPI_FOR(MP))

#define TC_ERR_FULL_WAIT 1
#define TC_ERR_EMPTY_WAIT 2
#define TC_ERR_ACC_WAIT 3
#define TC_ERR_SLICE_WAIT 6

struct TcArgs {
  void* out;
  int out_dtype;
  int M, N, K;
  int ldo;
  int mode;        // 0 store, 2 swiglu, 3 residual add + gain + sums of squares
  int k_blocks;    // ceil(K / 64)
  const float* row_ss;   // [ss_parts][ss_stride]: sums of squares of the input rows, or null (rows are plain)
  int ss_parts, ss_stride;
  float inv_width, eps;  // of the norm whose scale the input rows still lack
  const void* gain;      // mode 3: the next norm's weight [N]
  int gain_dtype;
  __nv_bfloat16* xg;     // mode 3: [M, N] residual * gain
  float* ss_out;         // mode 3: [tiles * cluster][ss_out_stride] sums of squares of this block's slice of each row
  int ss_out_stride;
  int* status;     // 0, or the code of a wait that gave up
  BN_TRACE_ONLY(unsigned long long* trace;)  // debugging: 8 timestamps of block 0 per launch, or null
};

// First row (of 128) of the slice that cluster rank r reduces and stores.  SwiGLU: multiples of 16,
// so that a gate row and its up row (8 apart) stay in one slice; else multiples of 4.
__device__ __host__ __forceinline__ int slice_start(int r, int c, int mode) {
  return mode == 2 ? 16 * ((8 * r) / c) : 4 * ((32 * r) / c);
}
// The most rows any rank's slice has.
__device__ __host__ __forceinline__ int slice_rows_max(int c, int mode) {
  return mode == 2 ? 16 * ((8 + c - 1) / c) : 4 * ((32 + c - 1) / c);
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address in block `rank`'s shared memory of what lies at `local_addr` here.
__device__ __forceinline__ unsigned map_to_rank(unsigned local_addr, unsigned rank) {
  unsigned remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
// `bytes` (a multiple of 16, both ends 16-byte aligned) from this block's shared memory into
// another block's, completing on an mbarrier of that block.
__device__ __forceinline__ void push_to_rank(unsigned remote_dst, unsigned local_src, unsigned bytes, unsigned remote_bar) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(remote_dst), "r"(local_src), "r"(bytes), "r"(remote_bar) : "memory");
}
template <int MP>  // batch columns of the accumulator: 16, 32 or 64
__global__ void __launch_bounds__(TC_THREADS_FOR(MP))
linear_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TcArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr int A_BYTES = TC_BM * TC_BK * 2;   // 16 KB
  constexpr int B_BYTES = MP * TC_BK * 2;      // 2, 4 or 8 KB
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TC_STAGES = TC_STAGES_FOR(MP);
  constexpr int EPI = TC_EPI_FOR(MP);          // epilogue threads
  constexpr int MPS = MP + 4;  // floats per weight row of the partial tile in shared memory (padded: no bank conflicts)
  // the partial tile, the slices received from the other blocks (at most 192 rows) and, in mode 3,
  // the squares of this block's slice reuse the ring
  static_assert((TC_BM + 192) * MPS * 4 <= TC_STAGES * STAGE_BYTES, "partial tile and received slices reuse the ring");
  constexpr unsigned TMEM_COLS = MP < 32 ? 32 : MP;
  // instruction descriptor: D float32 (bits 4-5 = 1), A and B bfloat16 (bits 7-9, 10-12 = 1), both
  // K-major, N >> 3 at bit 17, M >> 4 at bit 24
  constexpr unsigned IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(MP >> 3) << 17) | ((TC_BM >> 4) << 24);

  // the same offset in every block of the cluster (dynamic shared memory starts at the same address)
  unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned long long* bars = (unsigned long long*)(base + TC_STAGES * STAGE_BYTES);
  unsigned* tmem_slot = (unsigned*)(bars + 2 * TC_STAGES + 2);
  float* row_scale = (float*)(tmem_slot + 2);  // [64]: 1 / rms of the input rows (when row_ss is given)
  float* ss_chunk = row_scale + 64;            // [EPI / MP][MP]: partial sums on the way there
  // (Storing the partial sums straight from registers into a buffer of the owning block outside
  // its ring saves the cluster barrier before the copies and the copy engine's latency (1.5
  // against 2.3 us from the complete accumulator to the last store at 8 rows and 7 blocks), but
  // the buffer costs the narrow accumulator a stage of its ring, and the decode step was 2 %
  // slower with it; at 64 rows the stores of a whole tile take longer than the copies.)
  float* partial = (float*)base;  // [128][MPS]: partial[row][m], valid once all MMAs have read the ring
  float* recv = partial + TC_BM * MPS;  // [C - 1][slot_rows][MPS]: this block's slice as the other blocks computed it
  __shared__ int s_failed;
  __shared__ int s_acc_ok;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int C = gridDim.x, rank = blockIdx.x, tile = blockIdx.y;  // the cluster spans gridDim.x
  const int kb0 = (int)((long long)rank * a.k_blocks / C), kb1 = (int)((long long)(rank + 1) * a.k_blocks / C);
  const int n_kb = kb1 - kb0;
  const unsigned full0 = smem_u32(bars), empty0 = smem_u32(bars + TC_STAGES), acc_bar = smem_u32(bars + 2 * TC_STAGES);
  const unsigned slice_bar = acc_bar + 8;  // completes when the other blocks' copies of this block's slice have landed
  const int r0 = slice_start(rank, C, a.mode), rows = slice_start(rank + 1, C, a.mode) - r0;
  const int slot_rows = slice_rows_max(C, a.mode);
  float* item_sq = recv + (C - 1) * slot_rows * MPS;  // mode 3: [M][rows] squares of the new residual values
  constexpr int W = MP == 16 ? 1 : 4;  // batch rows per epilogue item (see part two)
  // mode 3: the residual values and the gains of a thread's first items, fetched while the products run
  constexpr int PRE = 2;  // so many items per thread (few threads have more)
  float pre_old[PRE][W], pre_gain[PRE];
#pragma unroll
  for (int k = 0; k < PRE; ++k) {
    pre_gain[k] = 0.f;
#pragma unroll
    for (int i = 0; i < W; ++i) pre_old[k][i] = 0.f;
  }

  if (tid == 0) {
    s_failed = 0;
    s_acc_ok = 0;
    tma_prefetch_map(&map_w);
    tma_prefetch_map(&map_x);
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(acc_bar, 1);
    mbar_init(slice_bar, 1);
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
  BN_TRACE_ONLY(const bool tracing = a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0;)
  BN_TRACE_ONLY(if (tracing && tid == 0) a.trace[0] = global_timer();)
  // the kernel that follows in the stream may start its own prologue now
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      // Weights do not depend on the kernel before this one: the first ring of W tiles is
      // requested before the dependency wait, the matching x tiles after it.
      const int pre = min(n_kb, TC_STAGES);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(full0 + 8 * i, STAGE_BYTES);
        tma_load_2d(smem_u32(base + i * STAGE_BYTES), &map_w, full0 + 8 * i, (kb0 + i) * TC_BK, tile * TC_BM);
      }
      BN_TRACE_ONLY(if (tracing) a.trace[1] = global_timer();)
      asm volatile("griddepcontrol.wait;" ::: "memory");
      BN_TRACE_ONLY(if (tracing) a.trace[2] = global_timer();)
      bool failed = false;
      for (int i = 0; i < n_kb; ++i) {
        int s = i % TC_STAGES, round = i / TC_STAGES;
        unsigned dst = smem_u32(base + s * STAGE_BYTES);
        if (round > 0) {
          if (!mbar_wait(empty0 + 8 * s, (round & 1) ^ 1, a.status, TC_ERR_EMPTY_WAIT)) { failed = true; break; }
          mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
          tma_load_2d(dst, &map_w, full0 + 8 * s, (kb0 + i) * TC_BK, tile * TC_BM);
        }
        tma_load_2d(dst + A_BYTES, &map_x, full0 + 8 * s, (kb0 + i) * TC_BK, 0);
      }
      BN_TRACE_ONLY(if (tracing) a.trace[3] = global_timer();)  // all loads issued
      if (failed) s_failed = 1;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool failed = false;
      for (int i = 0; i < n_kb; ++i) {
        int s = i % TC_STAGES, round = i / TC_STAGES;
        if (!mbar_wait(full0 + 8 * s, round & 1, a.status, TC_ERR_FULL_WAIT)) { failed = true; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        unsigned sa = smem_u32(base + s * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
        for (int kk = 0; kk < TC_BK / 16; ++kk)
          umma_mma(tmem_base, umma_desc_k(sa + kk * 32), umma_desc_k(sb + kk * 32), IDESC, (i | kk) ? 1u : 0u);
        umma_commit(empty0 + 8 * s);  // arrives when these MMAs have read the stage
      }
      if (!failed) umma_commit(acc_bar);  // arrives when every MMA above is done
      if (failed) s_failed = 1;
      BN_TRACE_ONLY(if (tracing) a.trace[4] = global_timer();)  // all MMAs issued
    }
  } else {
    // ---- epilogue warps, part one: accumulator -> shared memory (TMEM lane quadrant warp % 4)
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    if (a.row_ss != nullptr) {
      // the scale each input row still lacks, from the parts its producer left: the epilogue threads
      // share a row's parts in EPI / MP chunks, then one thread per row adds the chunks in order
      pdl_wait();
      constexpr int CH = EPI / MP;
      const int t = tid - 64, m = t % MP, c = t / MP;
      const int per = (a.ss_parts + CH - 1) / CH;
      float ss = 0.f;
      if (m < a.M)
        for (int p = c * per; p < min(a.ss_parts, (c + 1) * per); ++p) ss += a.row_ss[(size_t)p * a.ss_stride + m];
      ss_chunk[c * MP + m] = ss;
      asm volatile("bar.sync 1, %0;" ::"n"(EPI) : "memory");
      if (t < a.M) {
        float tot = 0.f;
#pragma unroll
        for (int q = 0; q < CH; ++q) tot += ss_chunk[q * MP + t];
        row_scale[t] = 1.0f / sqrtf(tot * a.inv_width + a.eps);
      }
    }
    if (a.mode == 3) {
      pdl_wait();
      const int t = tid - 64;
      const int dm = EPI / rows, dn = EPI - dm * rows;
      int mg = t / rows, nl = t - mg * rows;
#pragma unroll
      for (int k = 0; k < PRE; ++k) {
        const int n = tile * TC_BM + r0 + nl;
        if (mg * W < a.M && n < a.N) {
          pre_gain[k] = load_as_f32(a.gain, a.gain_dtype, (size_t)n);
#pragma unroll
          for (int i = 0; i < W; ++i)
            if (mg * W + i < a.M) pre_old[k][i] = ((const float*)a.out)[(size_t)(mg * W + i) * a.ldo + n];
        }
        mg += dm; nl += dn;
        if (nl >= rows) { nl -= rows; ++mg; }
      }
    }
    if (warp == 2 && lane == 0) {
      int ok = mbar_wait(acc_bar, 0, a.status, TC_ERR_ACC_WAIT) ? 1 : 0;
      if (!ok) s_failed = 1;
      s_acc_ok = ok;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(EPI) : "memory");
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    BN_TRACE_ONLY(if (tracing && tid == 64) a.trace[7] = global_timer();)  // accumulator complete
    // with eight epilogue warps, warps 2-5 take the first half of the columns and 6-9 the second
    constexpr int COLS = MP * 128 / EPI;
    const int c0 = ((warp - 2) >> 2) * COLS;
    float v[COLS];
    if (s_acc_ok) {
#pragma unroll
      for (int c = 0; c < COLS; c += 16) tmem_ld16(tmem_base + ((unsigned)(quad * 32) << 16) + c0 + c, v + c);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    } else {
#pragma unroll
      for (int c = 0; c < COLS; ++c) v[c] = 0.f;
    }
    // every MMA has completed, so nothing reads the ring any more: it now holds the partial tile,
    // weight row by weight row (a thread writes its row's columns as groups of four)
#pragma unroll
    for (int c = 0; c < COLS; c += 4)
      *reinterpret_cast<float4*>(partial + row * MPS + c0 + c) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
    // the bulk copies below read these values through the asynchronous proxy
    if (C > 1) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    // what this block is about to receive: its slice from each other block
    if (tid == 64 && C > 1) mbar_expect_tx(slice_bar, (unsigned)((C - 1) * rows * MPS * 4));
  }

  // ---- every block of the cluster has its partial tile in shared memory and reads its ring no more
  __syncwarp();
  if (C > 1) {
    cluster_sync_all();
    if (tid == 64) {
      // each other block gets the rows it owns, as this block computed them; slot: this block's
      // rank among the others.  Start with the next rank so that the copies spread over the blocks.
      for (int i = 1; i < C; ++i) {
        const int d = (rank + i) % C;
        const int d0 = slice_start(d, C, a.mode), drows = slice_start(d + 1, C, a.mode) - d0;
        const int slot = rank < d ? rank : rank - 1;
        push_to_rank(map_to_rank(smem_u32(recv + slot * slot_rows * MPS), d), smem_u32(partial + d0 * MPS),
                     (unsigned)(drows * MPS * 4), map_to_rank(slice_bar, d));
      }
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
  }

  if (warp >= 2) {
    // part two: this block's slice of the rows, summed over the cluster in rank order, then stored.
    // Consecutive threads take consecutive rows (output columns), so global accesses coalesce.
    pdl_wait();  // before the first global write of this thread
    const int t = tid - 64;
    if (C > 1 && t == 0 && !mbar_wait(slice_bar, 0, a.status, TC_ERR_SLICE_WAIT)) s_failed = 1;
    // the slices have landed, and (also in a cluster of one) every warp has written its part of the partial tile
    asm volatile("bar.sync 1, %0;" ::"n"(EPI) : "memory");
    // One item is a row of the slice and W batch rows: (nl, mg) with batch rows W mg .. W mg + W - 1;
    // items are numbered mg * rows + nl and a thread takes every EPI-th of them (the division once,
    // then steps).  With many batch rows the epilogue is bound by the instructions it issues: four
    // values per load.  With few there are fewer such items than threads and the longest chain of
    // dependent instructions counts: one value per item.  The blocks' copies of the slice start at
    // these shared-memory addresses, in rank order:
    unsigned copy[8];
#pragma unroll
    for (int q = 0; q < 8; ++q)
      copy[q] = smem_u32(q == rank ? partial + r0 * MPS : recv + (q < rank ? q : q - 1) * slot_rows * MPS);
    auto load_copy = [&](unsigned addr, float* v) {
      if constexpr (W == 4)
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "r"(addr));
      else
        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v[0]) : "r"(addr));
    };
    auto slice_values = [&](int nl, int mg, float* v) {
      const unsigned off = (unsigned)(nl * MPS + mg * W) * 4u;
      if (C == 1) {  // predicated-off loads and additions would still take issue slots
        load_copy(copy[0] + off, v);
        return;
      }
      float p[8][W];
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (q < C) load_copy(copy[q] + off, p[q]);
#pragma unroll
      for (int i = 0; i < W; ++i) v[i] = p[0][i];
#pragma unroll
      for (int q = 1; q < 8; ++q)
        if (q < C) {
#pragma unroll
          for (int i = 0; i < W; ++i) v[i] += p[q][i];
        }
    };
    const int mgroups = (a.M + W - 1) / W;
    if (a.mode == 0) {
      const int dm = EPI / rows, dn = EPI - dm * rows;
      int mg = t / rows, nl = t - mg * rows;
      while (mg < mgroups) {
        const int n = tile * TC_BM + r0 + nl;
        if (n < a.N) {
          float v[W];
          slice_values(nl, mg, v);
#pragma unroll
          for (int i = 0; i < W; ++i) {
            const int m = mg * W + i;
            if (m < a.M) store_from_f32(a.out, a.out_dtype, (size_t)m * a.ldo + n, a.row_ss != nullptr ? v[i] * row_scale[m] : v[i]);
          }
        }
        mg += dm; nl += dn;
        if (nl >= rows) { nl -= rows; ++mg; }
      }
    } else if (a.mode == 3) {
      // out is the float32 residual [M, ldo]: add, write back, hand on residual * gain, and leave
      // this slice's sum of squares per row (the squares in a fixed place each, then one thread
      // per batch row adds them in order)
      float* res = (float*)a.out;
      const int dm = EPI / rows, dn = EPI - dm * rows;
      int mg = t / rows, nl = t - mg * rows;
      // one item; old and gain: its residual values and gain if they were fetched ahead
      auto residual_item = [&](int mg, int nl, const float* old, float gain_ahead) {
        const int n = tile * TC_BM + r0 + nl;
        float sq[W];
#pragma unroll
        for (int i = 0; i < W; ++i) sq[i] = 0.f;
        if (n < a.N) {
          float v[W];
          slice_values(nl, mg, v);
          const float gain = old != nullptr ? gain_ahead : load_as_f32(a.gain, a.gain_dtype, (size_t)n);
#pragma unroll
          for (int i = 0; i < W; ++i) {
            const int m = mg * W + i;
            if (m < a.M) {
              float* rp = res + (size_t)m * a.ldo + n;
              const float nv = (old != nullptr ? old[i] : *rp) + (a.row_ss != nullptr ? v[i] * row_scale[m] : v[i]);
              *rp = nv;
              a.xg[(size_t)m * a.N + n] = __float2bfloat16_rn(nv * gain);
              sq[i] = nv * nv;
            }
          }
        }
#pragma unroll
        for (int i = 0; i < W; ++i) item_sq[(mg * W + i) * rows + nl] = sq[i];
      };
#pragma unroll
      for (int k = 0; k < PRE; ++k) {
        if (mg < mgroups) residual_item(mg, nl, pre_old[k], pre_gain[k]);
        mg += dm; nl += dn;
        if (nl >= rows) { nl -= rows; ++mg; }
      }
      while (mg < mgroups) {
        residual_item(mg, nl, nullptr, 0.f);
        mg += dm; nl += dn;
        if (nl >= rows) { nl -= rows; ++mg; }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(EPI) : "memory");
      for (int m = t; m < a.M; m += EPI) {
        float ss = 0.f;
        for (int i = 0; i < rows; i += 4) {  // slices are multiples of four rows
          const float4 q4 = *reinterpret_cast<const float4*>(item_sq + m * rows + i);
          ss += q4.x; ss += q4.y; ss += q4.z; ss += q4.w;
        }
        a.ss_out[(size_t)(tile * C + rank) * a.ss_out_stride + m] = ss;
      }
    } else {
      // rows 16j..16j+7 of a tile are gate rows, rows 16j+8..16j+15 the up rows of the same indices;
      // item = (gate row, W batch rows); consecutive gate rows are consecutive activations.  The
      // exponential and the division are the fast ones (relative error about 2^-21, far below the
      // bfloat16 the activations are stored in).
      const int gates = rows / 2;
      const int dm = EPI / gates, dj = EPI - dm * gates;
      int mg = t / gates, j = t - mg * gates;
      while (mg < mgroups) {
        const int nl = (j >> 3) * 16 + (j & 7);  // the gate row within the slice
        const int n = tile * TC_BM + r0 + nl;
        if (n < a.N) {
          float g[W], u[W];
          slice_values(nl, mg, g);
          slice_values(nl + 8, mg, u);
          const int col = (n >> 4) * 8 + (n & 7);
#pragma unroll
          for (int i = 0; i < W; ++i) {
            const int m = mg * W + i;
            if (m < a.M) {
              const float rs = a.row_ss != nullptr ? row_scale[m] : 1.0f;
              const float gv = g[i] * rs, uv = u[i] * rs;
              store_from_f32(a.out, a.out_dtype, (size_t)m * a.ldo + col, __fdividef(gv, 1.0f + __expf(-gv)) * uv);
            }
          }
        }
        mg += dm; j += dj;
        if (j >= gates) { j -= gates; ++mg; }
      }
    }
    BN_TRACE_ONLY(if (tracing && warp == 2 && lane == 0) a.trace[5] = global_timer();)  // epilogue done
  }

  // No block reads another's shared memory, and every copy into this block has landed (the wait on
  // slice_bar above); what is left before leaving is that this block's own copies have read their source.
  if (tid == 64 && C > 1) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (s_failed) {
    // a wait gave up: loads and copies that were issued may still be landing in this block's shared memory
    unsigned long long t0 = global_timer();
    while (global_timer() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
  BN_TRACE_ONLY(if (tracing && tid == 32) a.trace[6] = global_timer();)
}

#ifdef BN_TRACE
// Debugging aid: bn_linear_tc_trace(n) makes the next n launches record timestamps of block 0
// (device buffer allocated here; not used on the product path).
static unsigned long long* g_trace = nullptr;
static int g_trace_n = 0, g_trace_cap = 0;
extern "C" int bn_linear_tc_trace(int n) {
  if (g_trace) cudaFree(g_trace);
  g_trace = nullptr; g_trace_n = 0; g_trace_cap = 0;
  if (n <= 0) return 0;
  if (cudaMalloc(&g_trace, (size_t)n * 64) != cudaSuccess) return 1;
  cudaMemset(g_trace, 0, (size_t)n * 64);
  g_trace_cap = n;
  return 0;
}
extern "C" int bn_linear_tc_trace_read(unsigned long long* host, int n) {
  if (!g_trace || n > g_trace_cap) return 1;
  return cudaMemcpy(host, g_trace, (size_t)n * 64, cudaMemcpyDeviceToHost) != cudaSuccess;
}
#endif

static int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

template <int MP>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const TcArgs& a, int cluster, int tiles,
                     cudaStream_t stream) {
  constexpr int TC_STAGES = TC_STAGES_FOR(MP);
  size_t smem = (size_t)TC_STAGES * (TC_BM * TC_BK * 2 + MP * TC_BK * 2) + (2 * TC_STAGES + 2) * 8 + 16 + (64 + 256) * 4 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(linear_tc_kernel<MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cluster, tiles);
  cfg.blockDim = dim3(TC_THREADS_FOR(MP));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = bn_pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, linear_tc_kernel<MP>, mw, mx, a);
  if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
  return BN_OK;
}

// Blocks per tile when the caller leaves the choice to the kernel: about 1.5 blocks per SM in all.
// With one block per SM the bytes in flight (one ring each) do not cover the memory's latency, and
// while a block runs its epilogue its SM fetches nothing; with more than some 250 blocks clusters no
// longer fit in one wave.  Measured on the four products of a layer of width 4096 (32 layers, one
// CUDA graph, 8 rows): 3/4/1/4 blocks per tile 2.79 ms, 5/7/1/7 2.58 ms, 6/8/1/8 2.76 ms.
static int auto_cluster(int tiles, int k_blocks) {
  int cluster = (sm_count() * 157 / 100 + tiles / 2) / tiles;
  int by_k = k_blocks / 4;  // at least four k-blocks per block
  if (cluster > by_k) cluster = by_k;
  if (cluster > 8) cluster = 8;
  if (cluster < 1) cluster = 1;
  return cluster;
}
// How many blocks share a tile's inner dimension when the caller leaves the choice to the kernel
// (mode 3 writes tiles x this many parts of sums of squares).
extern "C" int bn_linear_tc_auto_cluster(int N, int K) {
  if (N <= 0 || K <= 0) return 1;
  return auto_cluster((N + TC_BM - 1) / TC_BM, (K + TC_BK - 1) / TC_BK);
}

// x [M, K], w [N, K] bfloat16, both 16-byte aligned with K a multiple of 8.  mode 0: out [M, ldo]
// of out_dtype; mode 2: N = 2 I weight rows in blocks of 8 gate / 8 up rows, out holds
// silu(gate) * up in I columns; mode 3: out is a float32 residual [M, ldo] that the product is
// added to in place, xg [M, N] bfloat16 receives residual * gain (gain [N] of gain_dtype) and
// ss_out [tiles * cluster][ss_out_stride] the sums of squares of each block's slice of every row
// (tiles = ceil(N / 128); cluster must be given).  row_ss (or null): [ss_parts][ss_stride] sums of
// squares of the rows of x as a mode-3 product left them; the result rows are then multiplied by
// 1 / sqrt(sum / width + eps) with inv_width = 1 / width.  cluster: blocks that share a tile's
// inner dimension, 1 to 8 (0: chosen so that cluster x tiles is about one and a half times the number of SMs).  status:
// one int on the device, left 0 unless a wait inside the kernel gave up.
extern "C" int bn_linear_tc_ex(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K, int ldo,
                               int mode, int cluster, const float* row_ss, int ss_parts, int ss_stride, float inv_width,
                               float eps, const void* gain, int gain_dtype, void* xg, float* ss_out, int ss_out_stride,
                               int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return BN_OK;
  if (M > 64 || K <= 0 || K % 8 || cluster < 0 || cluster > 8 || (mode != 0 && mode != 2 && mode != 3) || !status)
    return BN_ERR_BAD_ARG;
  if (mode == 2 && (N % 16)) return BN_ERR_BAD_ARG;
  if (mode == 3 && (!gain || !xg || !ss_out || ss_out_stride < M || cluster == 0 || out_dtype != BN_F32 ||
                    (gain_dtype != BN_F32 && gain_dtype != BN_BF16)))
    return BN_ERR_BAD_ARG;
  if (row_ss && (ss_parts <= 0 || ss_stride < M)) return BN_ERR_BAD_ARG;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return BN_ERR_BAD_ARG;
  int mp = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  int tiles = (N + TC_BM - 1) / TC_BM;
  int k_blocks = (K + TC_BK - 1) / TC_BK;
  if (tiles > 65535) return BN_ERR_BAD_ARG;
  if (cluster == 0) cluster = auto_cluster(tiles, k_blocks);
  if (cluster > k_blocks) {
    if (mode == 3) return BN_ERR_BAD_ARG;  // the caller sized ss_out for the cluster it named
    cluster = k_blocks;
  }
  {
    // the partial tile, the received slices and (mode 3) the squares must fit in the ring they reuse
    const int stages = TC_STAGES_FOR(mp == 16 ? 16 : (mp == 32 ? 32 : 64));
    const long long ring = (long long)stages * (TC_BM * TC_BK * 2 + mp * TC_BK * 2);
    const int max_rows = slice_rows_max(cluster, mode);
    long long need = (long long)(TC_BM + (cluster - 1) * max_rows) * (mp + 4) * 4;
    if (mode == 3) need += (long long)(M + 3) * max_rows * 4;
    if (need > ring) return BN_ERR_BAD_ARG;
  }
  CUtensorMap mw, mx;
  if (!tma_map_bf16_rows(&mw, w, N, K, TC_BM) || !tma_map_bf16_rows(&mx, x, M, K, mp)) return BN_ERR_BAD_ARG;
  TcArgs a;
  a.out = out; a.out_dtype = out_dtype; a.M = M; a.N = N; a.K = K; a.ldo = ldo; a.mode = mode;
  a.k_blocks = k_blocks; a.status = status;
  a.row_ss = row_ss; a.ss_parts = ss_parts; a.ss_stride = ss_stride; a.inv_width = inv_width; a.eps = eps;
  a.gain = gain; a.gain_dtype = gain_dtype; a.xg = (__nv_bfloat16*)xg; a.ss_out = ss_out; a.ss_out_stride = ss_out_stride;
  BN_TRACE_ONLY(a.trace = nullptr;)
  BN_TRACE_ONLY(if (g_trace && g_trace_n < g_trace_cap) a.trace = g_trace + 8 * (g_trace_n++);)
  if (mp == 16) return launch_tc<16>(mw, mx, a, cluster, tiles, stream);
  if (mp == 32) return launch_tc<32>(mw, mx, a, cluster, tiles, stream);
  return launch_tc<64>(mw, mx, a, cluster, tiles, stream);
}

// The plain forms (modes 0 and 2, plain input rows).
extern "C" int bn_linear_tc(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K, int ldo,
                            int mode, int cluster, int* status, cudaStream_t stream) {
  if (mode == 3) return BN_ERR_BAD_ARG;
  return bn_linear_tc_ex(x, w, out, out_dtype, M, N, K, ldo, mode, cluster, nullptr, 0, 0, 0.f, 0.f, nullptr, 0, nullptr,
                         nullptr, 0, status, stream);
}
