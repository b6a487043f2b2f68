// out[M, N] = x[M, K] . W[N, K]^T for many rows (prefill) in bfloat16 on the 5th-generation tensor
// cores, with the work that follows a projection done in its epilogue.
//
// A persistent kernel, one block per SM.  A block takes output tiles of 128 rows x 256 columns in
// turn (tile t = block index + i x blocks; tiles of one column of W run side by side on
// neighbouring blocks, so that a slice of W is read from memory once and then found in the L2).
// Operands arrive by TMA (boxes of 128 x 64 and 256 x 64 elements, 128-byte swizzle) through a
// ring of four stages of 48 KB; one thread issues tcgen05.mma (M 128, N 256, K 16, four per
// stage) into one of two accumulators of 256 columns in tensor memory; while it works on the next
// tile's accumulator, four epilogue warps read the finished one (a thread owns a row: its TMEM
// lane) and finish it:
//   mode 0  store (bfloat16 or float32);
//   mode 2  SwiGLU: columns hold gate and up values in alternating blocks of 8 (the layout of the
//           stacked weight), out[m, i] = silu(gate_i) * up_i, [M, N / 2];
//   mode 3  residual[m, n] += result (float32, in place); xg[m, n] = residual * gain[n] (the next
//           norm's weight) in bfloat16; ss_out[tile column][m] = sum of squares of the new
//           residual values of these 256 columns: the rows of xg still lack the norm's scale
//           1 / sqrt(sum of the parts / N + eps), which the product that consumes them applies
//           to its own result rows, W (s x) = s (W x): modes 0 and 2 take such rows (row_ss).
// This removes the separate passes over the activations that a library product leaves to other
// kernels: the SwiGLU pass over [M, 2 I] and both residual + norm passes of a layer.
//
// Every wait on an mbarrier is bounded in time; a wait that gives up records code 7 in *status,
// and every role leaves its loops; the block frees its tensor memory and returns.
//
// Reference: y = W x with float32 accumulation (src/quant/f32_scalar.c:4-32); the reference's
// prefill runs these products through cublasGemmEx and separate kernels for the activation and
// the residual + norm (src/gpu_cuda.cu:11850-11879, 10320, 5108).
#include "tma.cuh"
#include "umma.cuh"
#include <math.h>

#define GM_BM 128
#define GM_BN 256
#define GM_BK 64
#define GM_STAGES 4
#define GM_THREADS 192
#define GM_ERR_WAIT 7

struct GmArgs {
  void* out;        // modes 0, 2: [M, ldo]
  int out_dtype;
  int M, N, K, ldo, mode;
  int k_blocks, m_tiles, n_tiles;
  const float* row_ss;  // [ss_parts][ss_stride]: sums of squares of the input rows, or null (rows are plain)
  int ss_parts, ss_stride;
  float inv_width, eps;
  float* residual;      // mode 3: [M, N] float32
  const void* gain;     // mode 3: [N]
  int gain_dtype;
  __nv_bfloat16* xg;    // mode 3: [M, N]
  float* ss_out;        // mode 3: [n_tiles][ss_out_stride]
  int ss_out_stride;
  int* status;
};

__device__ __forceinline__ float gm_silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }

// The epilogue of one tile for one thread in modes 0 and 2: row m of the output, the 256 columns
// from n0 on, read from the thread's TMEM lane at acc_addr (see the modes at the top of this file).
__device__ __forceinline__ void gm_finish_tile(const GmArgs& a, unsigned acc_addr, int m, int n0, float scale) {
  const bool live = m < a.M;
#pragma unroll 1
  for (int c = 0; c < GM_BN; c += 32) {
    float v[32];
    tmem_ld32(acc_addr + c, v);
    if (!live || n0 + c >= a.N) continue;
    if (a.mode == 0) {
      if (a.out_dtype == BN_BF16) {
        __nv_bfloat16* o = (__nv_bfloat16*)a.out + (size_t)m * a.ldo + n0 + c;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          if (n0 + c + g * 8 < a.N)  // N is a multiple of 8
            *reinterpret_cast<uint4*>(o + g * 8) =
                make_uint4(pack_bf16x2(v[g * 8] * scale, v[g * 8 + 1] * scale), pack_bf16x2(v[g * 8 + 2] * scale, v[g * 8 + 3] * scale),
                           pack_bf16x2(v[g * 8 + 4] * scale, v[g * 8 + 5] * scale), pack_bf16x2(v[g * 8 + 6] * scale, v[g * 8 + 7] * scale));
        }
      } else {
        float* o = (float*)a.out + (size_t)m * a.ldo + n0 + c;
#pragma unroll
        for (int g = 0; g < 8; ++g)
          if (n0 + c + g * 4 < a.N)
            *reinterpret_cast<float4*>(o + g * 4) = make_float4(v[g * 4] * scale, v[g * 4 + 1] * scale, v[g * 4 + 2] * scale, v[g * 4 + 3] * scale);
      }
    } else {
      // two blocks of 8 gate + 8 up values -> 16 outputs at column (n0 + c) / 2
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        if (n0 + c + g * 16 >= a.N) continue;  // N is a multiple of 16 here
        float r[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) r[e] = gm_silu_mul(v[g * 16 + e] * scale, v[g * 16 + 8 + e] * scale);
        const size_t oc = (size_t)m * a.ldo + (size_t)((n0 + c) >> 1) + g * 8;
        if (a.out_dtype == BN_BF16) {
          *reinterpret_cast<uint4*>((__nv_bfloat16*)a.out + oc) =
              make_uint4(pack_bf16x2(r[0], r[1]), pack_bf16x2(r[2], r[3]), pack_bf16x2(r[4], r[5]), pack_bf16x2(r[6], r[7]));
        } else {
          *reinterpret_cast<float4*>((float*)a.out + oc) = make_float4(r[0], r[1], r[2], r[3]);
          *reinterpret_cast<float4*>((float*)a.out + oc + 4) = make_float4(r[4], r[5], r[6], r[7]);
        }
      }
    }
  }
}

// The epilogue of one tile for one warp in mode 3: rows m0 .. m0 + 31 (the warp's TMEM lanes).  A
// thread that walks its own row touches 32 cache lines with every load or store of the warp, and
// the residual is read and written in float32: that kept the load/store unit busy for longer than
// the tile's products took.  So the accumulator goes through shared memory 32 columns at a time
// (stage: [32 rows][33] floats of this warp), and comes back with eight lanes on the 32 columns of a
// row, four rows per instruction: whole 128-byte lines of the residual, 64 bytes of the rows for
// the next product.  The squares of a row are summed per lane over the tile's columns in a fixed
// order, then over the row's eight lanes.
#define GM_STG 33
__device__ __forceinline__ void gm_finish_tile_rows(const GmArgs& a, unsigned acc_addr, int m0, int n0, int nt, const float* gains,
                                                    float* stage, int lane) {
  const int sub = lane >> 3, q4 = (lane & 7) * 4;
  float ssl[8];
#pragma unroll
  for (int it = 0; it < 8; ++it) ssl[it] = 0.f;
#pragma unroll 1
  for (int c = 0; c < GM_BN; c += 32) {
    float v[32];
    tmem_ld32(acc_addr + c, v);
    __syncwarp();  // the chunk before this one has been read
#pragma unroll
    for (int j = 0; j < 32; ++j) stage[lane * GM_STG + j] = v[j];
    __syncwarp();
    const int col = n0 + c + q4;
    if (col < a.N) {  // the same for a whole group of four columns: N is a multiple of 8
      const float4 g4 = *reinterpret_cast<const float4*>(gains + c + q4);
      float4 old[8];
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int m = m0 + it * 4 + sub;
        old[it] = m < a.M ? *reinterpret_cast<const float4*>(a.residual + (size_t)m * a.N + col) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int r = it * 4 + sub, m = m0 + r;
        if (m >= a.M) continue;
        const float* sv = stage + r * GM_STG + q4;
        const float x0 = old[it].x + sv[0], x1 = old[it].y + sv[1], x2 = old[it].z + sv[2], x3 = old[it].w + sv[3];
        *reinterpret_cast<float4*>(a.residual + (size_t)m * a.N + col) = make_float4(x0, x1, x2, x3);
        *reinterpret_cast<uint2*>(a.xg + (size_t)m * a.N + col) = make_uint2(pack_bf16x2(x0 * g4.x, x1 * g4.y), pack_bf16x2(x2 * g4.z, x3 * g4.w));
        ssl[it] = fmaf(x3, x3, fmaf(x2, x2, fmaf(x1, x1, fmaf(x0, x0, ssl[it]))));
      }
    }
  }
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    float t = ssl[it];
    t += __shfl_xor_sync(0xffffffffu, t, 1);
    t += __shfl_xor_sync(0xffffffffu, t, 2);
    t += __shfl_xor_sync(0xffffffffu, t, 4);
    const int m = m0 + it * 4 + sub;
    if ((lane & 7) == 0 && m < a.M) a.ss_out[(size_t)nt * a.ss_out_stride + m] = t;
  }
}

__global__ void __launch_bounds__(GM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, GmArgs a) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr int A_BYTES = GM_BM * GM_BK * 2;  // 16 KB
  constexpr int B_BYTES = GM_BN * GM_BK * 2;  // 32 KB
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr unsigned TMEM_COLS = 512;         // two accumulators of 256 columns
  // D float32, A and B bfloat16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
  constexpr unsigned IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(GM_BN >> 3) << 17) | ((GM_BM >> 4) << 24);

  unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned long long* bars = (unsigned long long*)(base + GM_STAGES * STAGE_BYTES);
  // full[S], empty[S], acc_full[2], acc_empty[2]
  const unsigned full0 = smem_u32(bars), empty0 = full0 + 8 * GM_STAGES, acc_full0 = empty0 + 8 * GM_STAGES,
                 acc_empty0 = acc_full0 + 16;
  unsigned* tmem_slot = (unsigned*)(bars + 2 * GM_STAGES + 4);
  volatile int* failed = (volatile int*)(tmem_slot + 1);
  float* gain_s = (float*)(tmem_slot + 4);  // [2][256]: the gains of the tile's columns, per accumulator
  float* stage_s = gain_s + 2 * GM_BN;      // [4 warps][32][GM_STG]: mode 3, an accumulator chunk on its way to whole rows

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_tiles_total = a.m_tiles * a.n_tiles;

  if (tid == 0) {
    *failed = 0;
    tma_prefetch_map(&map_x);
    tma_prefetch_map(&map_w);
    for (int s = 0; s < GM_STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 4);  // one arrival per epilogue warp
    }
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
  pdl_wait();  // the rows of x (and the residual) come from the kernels before this one

  if (warp == 0) {
    // ---- producer: one thread requests the stages of all this block's tiles in turn
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < n_tiles_total; t += gridDim.x) {
        const int mt = t % a.m_tiles, nt = t / a.m_tiles;
        for (int kb = 0; kb < a.k_blocks; ++kb, ++it) {
          const int s = it % GM_STAGES, round = it / GM_STAGES;
          if (round > 0 && (!mbar_wait(empty0 + 8 * s, (unsigned)(round - 1) & 1u, a.status, GM_ERR_WAIT) || *failed)) {
            *failed = 1;
            ok = false;
            break;
          }
          const unsigned dst = smem_u32(base + s * STAGE_BYTES);
          mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
          tma_load_2d(dst, &map_x, full0 + 8 * s, kb * GM_BK, mt * GM_BM);
          tma_load_2d(dst + A_BYTES, &map_w, full0 + 8 * s, kb * GM_BK, nt * GM_BN);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue: one thread, accumulator tile_i & 1
    if (lane == 0) {
      int it = 0, tile_i = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < n_tiles_total; t += gridDim.x, ++tile_i) {
        const int buf = tile_i & 1, use = tile_i >> 1;
        if (use > 0 && (!mbar_wait(acc_empty0 + 8 * buf, (unsigned)(use - 1) & 1u, a.status, GM_ERR_WAIT) || *failed)) {
          *failed = 1;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned acc = tmem_base + buf * GM_BN;
        for (int kb = 0; kb < a.k_blocks; ++kb, ++it) {
          const int s = it % GM_STAGES, round = it / GM_STAGES;
          if (!mbar_wait(full0 + 8 * s, (unsigned)round & 1u, a.status, GM_ERR_WAIT) || *failed) {
            *failed = 1;
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned sa = smem_u32(base + s * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < GM_BK / 16; ++kk)
            umma_mma(acc, umma_desc_k(sa + kk * 32), umma_desc_k(sb + kk * 32), IDESC, (kb | kk) ? 1u : 0u);
          umma_commit(empty0 + 8 * s);  // arrives when these MMAs have read the stage
        }
        if (ok) umma_commit(acc_full0 + 8 * buf);  // arrives when the tile's last MMA is done
      }
    }
  } else {
    // ---- epilogue: thread <-> row of the tile <-> TMEM lane (a warp reaches the lanes of its index modulo 4)
    const int quad = warp & 3, et = tid - 64;
    const int row = quad * 32 + lane;
    const unsigned lane_addr = tmem_base + ((unsigned)(quad * 32) << 16);
    int tile_i = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < n_tiles_total; t += gridDim.x, ++tile_i) {
      const int mt = t % a.m_tiles, nt = t / a.m_tiles, buf = tile_i & 1;
      const int m = mt * GM_BM + row, n0 = nt * GM_BN;
      const bool live = m < a.M;
      // what does not depend on the accumulator: the scale the input rows still lack, the gains
      float scale = 1.0f;
      if (a.row_ss != nullptr && live) {
        float ss = 0.f;
        for (int p = 0; p < a.ss_parts; ++p) ss += a.row_ss[(size_t)p * a.ss_stride + m];
        scale = 1.0f / sqrtf(ss * a.inv_width + a.eps);
      }
      if (a.mode == 3) {
        for (int c = et; c < GM_BN; c += 128) gain_s[buf * GM_BN + c] = n0 + c < a.N ? load_as_f32(a.gain, a.gain_dtype, (size_t)(n0 + c)) : 0.f;
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      if (ok && (!mbar_wait(acc_full0 + 8 * buf, (unsigned)(tile_i >> 1) & 1u, a.status, GM_ERR_WAIT) || *failed)) {
        *failed = 1;
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) continue;  // walk the remaining tiles without work (their barrier above is still kept)
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (a.mode == 3)
        gm_finish_tile_rows(a, lane_addr + buf * GM_BN, mt * GM_BM + quad * 32, n0, nt, gain_s + buf * GM_BN,
                            stage_s + (warp - 2) * 32 * GM_STG, lane);
      else
        gm_finish_tile(a, lane_addr + buf * GM_BN, m, n0, scale);
      // the accumulator may be written again
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
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

// ---- the same product with pairs of blocks working as one (tcgen05 cta_group::2) ----------------
// Two blocks of a cluster, on neighbouring SMs, take a tile of 256 rows x 256 columns together:
// each loads its 128 rows of x and its 128 of the tile's 256 rows of W, one MMA instruction of
// the pair's leader (M 256, N 256, K 16) reads both blocks' shared memories and writes each
// block's 128 rows of the accumulator into that block's tensor memory.  Per flop a block moves two
// thirds of the operand bytes through its shared memory that it moves alone (32 KB instead of
// 48 KB per stage, six stages instead of four), which is what limits the single-block form.
// Signals: both blocks' TMA loads complete on the leader's barrier of the stage (the leader has
// announced the bytes of both); the leader's commits arrive on both blocks' "stage is free" and
// "accumulator is complete" barriers; both blocks' epilogue warps arrive on the leader's
// "accumulator is free" barrier.
#define GM2_STAGES 6

__device__ __forceinline__ unsigned gm_cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ unsigned gm_map_to_rank(unsigned local_addr, unsigned rank) {
  unsigned remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ void gm_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A box into this block's shared memory whose bytes are counted on a barrier of the pair's leader.
__device__ __forceinline__ void gm_tma_load_2d_pair(unsigned dst, const CUtensorMap* map, unsigned leader_bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(leader_bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void gm_mma_pair(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc,
                                            unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// Arrives, when the MMAs issued so far are done, on the barrier at this address in both blocks of the pair.
__device__ __forceinline__ void gm_commit_pair(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void gm_arrive_remote(unsigned cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__global__ void __launch_bounds__(GM_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, GmArgs a) {
  pdl_launch_dependents();
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr int A_BYTES = GM_BM * GM_BK * 2;        // 16 KB: this block's 128 rows of x
  constexpr int B_BYTES = (GM_BN / 2) * GM_BK * 2;  // 16 KB: this block's 128 rows of W
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr unsigned TMEM_COLS = 512;
  // M = 256 over the pair
  constexpr unsigned IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(GM_BN >> 3) << 17) | (((2 * GM_BM) >> 4) << 24);

  unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned long long* bars = (unsigned long long*)(base + GM2_STAGES * STAGE_BYTES);
  const unsigned full0 = smem_u32(bars), empty0 = full0 + 8 * GM2_STAGES, acc_full0 = empty0 + 8 * GM2_STAGES,
                 acc_empty0 = acc_full0 + 16;
  unsigned* tmem_slot = (unsigned*)(bars + 2 * GM2_STAGES + 4);
  volatile int* failed = (volatile int*)(tmem_slot + 1);
  float* gain_s = (float*)(tmem_slot + 4);
  float* stage_s = gain_s + 2 * GM_BN;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const unsigned rank = gm_cluster_rank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int m_pairs = (a.m_tiles + 1) / 2;
  const int n_tiles_total = m_pairs * a.n_tiles;

  if (tid == 0) {
    *failed = 0;
    tma_prefetch_map(&map_x);
    tma_prefetch_map(&map_w);
    for (int s = 0; s < GM2_STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);   // used in the leader: its own announcement; the bytes of both blocks
      mbar_init(empty0 + 8 * s, 1);  // the leader's commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);   // the leader's commit
      mbar_init(acc_empty0 + 8 * b, 8);  // used in the leader: four epilogue warps of each block
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  gm_cluster_sync();  // both blocks' barriers exist before either signals the other
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    // ---- producer: this block's halves of the operands; the bytes count on the leader's barrier
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int t = pair; ok && t < n_tiles_total; t += n_pairs) {
        const int mp = t % m_pairs, nt = t / m_pairs;
        for (int kb = 0; kb < a.k_blocks; ++kb, ++it) {
          const int s = it % GM2_STAGES, round = it / GM2_STAGES;
          if (round > 0 && (!mbar_wait(empty0 + 8 * s, (unsigned)(round - 1) & 1u, a.status, GM_ERR_WAIT) || *failed)) {
            *failed = 1;
            ok = false;
            break;
          }
          const unsigned dst = smem_u32(base + s * STAGE_BYTES);
          if (leader) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
          const unsigned bar = gm_map_to_rank(full0 + 8 * s, 0);
          gm_tma_load_2d_pair(dst, &map_x, bar, kb * GM_BK, mp * 2 * GM_BM + (int)rank * GM_BM);
          gm_tma_load_2d_pair(dst + A_BYTES, &map_w, bar, kb * GM_BK, nt * GM_BN + (int)rank * (GM_BN / 2));
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue: the leader's thread, for both blocks
    if (lane == 0 && leader) {
      int it = 0, tile_i = 0;
      bool ok = true;
      for (int t = pair; ok && t < n_tiles_total; t += n_pairs, ++tile_i) {
        const int buf = tile_i & 1, use = tile_i >> 1;
        if (use > 0 && (!mbar_wait(acc_empty0 + 8 * buf, (unsigned)(use - 1) & 1u, a.status, GM_ERR_WAIT) || *failed)) {
          *failed = 1;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned acc = tmem_base + buf * GM_BN;
        for (int kb = 0; kb < a.k_blocks; ++kb, ++it) {
          const int s = it % GM2_STAGES, round = it / GM2_STAGES;
          if (!mbar_wait(full0 + 8 * s, (unsigned)round & 1u, a.status, GM_ERR_WAIT) || *failed) {
            *failed = 1;
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned sa = smem_u32(base + s * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < GM_BK / 16; ++kk)
            gm_mma_pair(acc, umma_desc_k(sa + kk * 32), umma_desc_k(sb + kk * 32), IDESC, (kb | kk) ? 1u : 0u);
          gm_commit_pair(empty0 + 8 * s);  // both blocks' stage is free when these MMAs have read it
        }
        if (ok) gm_commit_pair(acc_full0 + 8 * buf);  // both blocks' accumulator is complete
      }
    }
  } else {
    // ---- epilogue: this block's 128 rows of the pair's tile
    const int quad = warp & 3, et = tid - 64;
    const int row = quad * 32 + lane;
    const unsigned lane_addr = tmem_base + ((unsigned)(quad * 32) << 16);
    int tile_i = 0;
    bool ok = true;
    for (int t = pair; t < n_tiles_total; t += n_pairs, ++tile_i) {
      const int mp = t % m_pairs, nt = t / m_pairs, buf = tile_i & 1;
      const int m = mp * 2 * GM_BM + (int)rank * GM_BM + row, n0 = nt * GM_BN;
      float scale = 1.0f;
      if (a.row_ss != nullptr && m < a.M) {
        float ss = 0.f;
        for (int p = 0; p < a.ss_parts; ++p) ss += a.row_ss[(size_t)p * a.ss_stride + m];
        scale = 1.0f / sqrtf(ss * a.inv_width + a.eps);
      }
      if (a.mode == 3) {
        for (int c = et; c < GM_BN; c += 128) gain_s[buf * GM_BN + c] = n0 + c < a.N ? load_as_f32(a.gain, a.gain_dtype, (size_t)(n0 + c)) : 0.f;
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      if (ok && (!mbar_wait(acc_full0 + 8 * buf, (unsigned)(tile_i >> 1) & 1u, a.status, GM_ERR_WAIT) || *failed)) {
        *failed = 1;
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) continue;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (a.mode == 3)
        gm_finish_tile_rows(a, lane_addr + buf * GM_BN, mp * 2 * GM_BM + (int)rank * GM_BM + quad * 32, n0, nt,
                            gain_s + buf * GM_BN, stage_s + (warp - 2) * 32 * GM_STG, lane);
      else
        gm_finish_tile(a, lane_addr + buf * GM_BN, m, n0, scale);
      // the pair's accumulator may be written again once all eight epilogue warps have said so
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) gm_arrive_remote(gm_map_to_rank(acc_empty0 + 8 * buf, 0));
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*failed) {
    unsigned long long t0 = global_timer();
    while (global_timer() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  gm_cluster_sync();  // neither block leaves, or frees its tensor memory, while the other may still use it
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

static int g_gemm_pairs = 1;

static int gm_sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

// How many parts of sums of squares a mode-3 product of N columns writes (rows of ss_out).
extern "C" int bn_gemm_tc_parts(int N) { return N <= 0 ? 0 : (N + GM_BN - 1) / GM_BN; }

// x: [M, K] bfloat16 rows (K a multiple of 8, 16-byte aligned), w: [N, K] bfloat16.
// mode 0: out [M, ldo] of out_dtype (N a multiple of 8).  mode 2: out [M, ldo], ldo >= N / 2 (N a
// multiple of 16).  mode 3: residual [M, N] float32 (in place), gain [N], xg [M, N] bfloat16, ss_out
// [bn_gemm_tc_parts(N)][ss_out_stride >= M] (N a multiple of 8).  row_ss (or null): [ss_parts][ss_stride]
// sums of squares of the rows of x over a width of 1 / inv_width, eps of that norm.  status: one
// int on the device, left as it is unless a wait inside the kernel gave up (then 7).
extern "C" int bn_gemm_tc(const void* x, const void* w, int M, int N, int K, void* out, int out_dtype, int ldo, int mode,
                          const float* row_ss, int ss_parts, int ss_stride, float inv_width, float eps, float* residual,
                          const void* gain, int gain_dtype, void* xg, float* ss_out, int ss_out_stride, int* status,
                          cudaStream_t stream) {
  if (M <= 0 || N <= 0) return BN_OK;
  if (K <= 0 || K % 8 || N % 8 || !status || (((uintptr_t)x | (uintptr_t)w) & 15)) return BN_ERR_BAD_ARG;
  if (mode == 0 || mode == 2) {
    if (!out || (out_dtype != BN_BF16 && out_dtype != BN_F32) || ((uintptr_t)out & 15)) return BN_ERR_BAD_ARG;
    if (mode == 2 && (N % 16 || ldo < N / 2 || ldo % 8)) return BN_ERR_BAD_ARG;
    if (mode == 0 && (ldo < N || ldo % 8)) return BN_ERR_BAD_ARG;
  } else if (mode == 3) {
    if (!residual || !gain || !xg || !ss_out || ss_out_stride < M || row_ss != nullptr ||
        (((uintptr_t)residual | (uintptr_t)xg) & 15))
      return BN_ERR_BAD_ARG;
  } else {
    return BN_ERR_BAD_ARG;
  }
  if (row_ss != nullptr && (ss_parts <= 0 || ss_stride < M)) return BN_ERR_BAD_ARG;
  const bool pairs = g_gemm_pairs != 0;
  CUtensorMap mx, mw;
  if (!tma_map_bf16_rows(&mx, x, (unsigned long long)M, (unsigned long long)K, GM_BM) ||
      !tma_map_bf16_rows(&mw, w, (unsigned long long)N, (unsigned long long)K, pairs ? GM_BN / 2 : GM_BN))
    return BN_ERR_BAD_ARG;
  GmArgs a = {};
  a.out = out; a.out_dtype = out_dtype; a.M = M; a.N = N; a.K = K; a.ldo = ldo; a.mode = mode;
  a.k_blocks = (K + GM_BK - 1) / GM_BK; a.m_tiles = (M + GM_BM - 1) / GM_BM; a.n_tiles = (N + GM_BN - 1) / GM_BN;
  a.row_ss = row_ss; a.ss_parts = ss_parts; a.ss_stride = ss_stride; a.inv_width = inv_width; a.eps = eps;
  a.residual = residual; a.gain = gain; a.gain_dtype = gain_dtype; a.xg = (__nv_bfloat16*)xg; a.ss_out = ss_out;
  a.ss_out_stride = ss_out_stride; a.status = status;
  if (pairs) {
    size_t smem = (size_t)GM2_STAGES * (GM_BM + GM_BN / 2) * GM_BK * 2 + (2 * GM2_STAGES + 4) * 8 + 16 + 2 * GM_BN * 4 + 4 * 32 * GM_STG * 4 + 1024;
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
      configured = true;
    }
    long long tiles = (long long)((a.m_tiles + 1) / 2) * a.n_tiles;
    long long want = tiles < gm_sm_count() / 2 ? tiles : gm_sm_count() / 2;
    cudaError_t e = bn_launch_cluster(gemm_tc_pair_kernel, dim3((unsigned)(2 * want)), dim3(GM_THREADS), smem, stream, dim3(2, 1, 1),
                                      mx, mw, a);
    if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
    return BN_OK;
  }
  size_t smem = (size_t)GM_STAGES * (GM_BM + GM_BN) * GM_BK * 2 + (2 * GM_STAGES + 4) * 8 + 16 + 2 * GM_BN * 4 + 4 * 32 * GM_STG * 4 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
    configured = true;
  }
  long long tiles = (long long)a.m_tiles * a.n_tiles;
  unsigned blocks = (unsigned)(tiles < gm_sm_count() ? tiles : gm_sm_count());
  BN_LAUNCH(gemm_tc_kernel, blocks, GM_THREADS, smem, stream, mx, mw, a);
  return BN_OK;
}

// 1: pairs of blocks work as one (cta_group::2, the default); 0: every block alone.
extern "C" int bn_gemm_tc_pairs(int on) {
  int was = g_gemm_pairs;
  if (on == 0 || on == 1) g_gemm_pairs = on;
  return was;
}
