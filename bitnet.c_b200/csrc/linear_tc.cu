// out[M, N] = x[M, K] . W[N, K]^T in bfloat16 on the 5th-generation tensor cores (tcgen05),
// for M <= 64: weights stream HBM -> shared memory by TMA, products accumulate in tensor memory.
//
// The roles are swapped so that the weight is the 128-row operand: D[128 weight rows, Mp batch
// columns] += W_tile[128, 64] . x_tile[Mp, 64]^T, one tcgen05.mma of shape M=128, N=Mp, K=16 per 16
// columns of k, issued by one thread.
//
// Work is cut stream-K fashion: the tiles x k-blocks space (tile = 128 weight rows, k-block = 64
// columns) is one line of units, and each of the (at most one per SM) persistent blocks takes a
// contiguous stretch of it, so every block streams the same number of bytes whatever N and K
// are.  A stretch crosses tile borders: each (block, tile) piece is a *segment* with its own
// accumulator.  A segment that covers a whole tile runs the epilogue directly.  A tile that is
// shared between blocks is finished through scratch: every block writes its float32 partial tile
// and draws a ticket of the tile's counter; the one that draws the last ticket adds the partials
// in block order and runs the epilogue.  No block ever waits for another.
//
// A block of 192 threads:
//   warp 0     one thread issues the TMA loads of W and x tiles into a ring of TC_STAGES stages and
//              arms each stage's "full" mbarrier with the bytes to expect;
//   warp 1     allocates tensor memory (two accumulators); one thread waits for "full", issues four
//              MMAs per stage, commits them to the stage's "empty" mbarrier and, at the end of a
//              segment, to that accumulator's "full" mbarrier;
//   warps 2-5  wait for an accumulator, read it from tensor memory (tcgen05.ld, one weight row per
//              thread), release it, and run the partial-tile protocol and the epilogue, while the
//              MMA thread already fills the other accumulator.
// Tiles are 128-byte swizzled both by TMA and in the MMA's shared-memory descriptors.  No
// register ever holds a weight, so the bytes in flight per SM are the ring's size (about 100 KB).
//
// The kernel is launched with programmatic stream serialization: the loads of its first weight
// tiles are issued before griddepcontrol.wait, i.e. while the kernel before it in the stream is
// still draining; everything that reads x or writes memory comes after the wait.
//
// Epilogues: (0) store, (2) SwiGLU over weight rows that alternate 8 gate and 8 up rows.
//
// Every wait on an mbarrier is bounded in time; when a wait gives up the block records a code
// in *status, lets its loads drain for a bounded time, frees its tensor memory and returns.
//
// Reference for the operation: y = W x with float32 accumulation (src/quant/bf16_scalar.c:4-21);
// the reference's CUDA backend reaches tensor cores only through cuBLAS (src/gpu_cuda.cu:11850-11879).
#include "common.cuh"
#include <cuda.h>
#include <cudaTypedefs.h>

#define TC_BM 128      // weight rows per tile (UMMA M)
#define TC_BK 64       // k per stage: 128 bytes of bfloat16, one swizzle row
// Ring depth by accumulator width: at most ~110 KB of shared memory per block, so that a block of
// the next kernel in the stream fits on the same SM and fetches its first weight tiles while this
// kernel's blocks are finishing (programmatic dependent launch).
#define TC_STAGES_FOR(MP) ((MP) == 16 ? 6 : ((MP) == 32 ? 5 : 4))
#define TC_THREADS 192
#define TC_WAIT_NS 2000000000ull  // two seconds

#define TC_ERR_FULL_WAIT 1
#define TC_ERR_EMPTY_WAIT 2
#define TC_ERR_ACC_WAIT 3
#define TC_ERR_ACC_FREE_WAIT 4

struct TcArgs {
  void* out;
  int out_dtype;
  int M, N, K;
  int ldo;
  int mode;        // 0 store, 2 swiglu
  int k_blocks;    // ceil(K / 64)
  int tiles;       // ceil(N / 128)
  float* scratch;  // [blocks][2][128][Mp] partial tiles of the first and last segment of a block
  int* counters;   // one ticket per tile, zero before and after
  int* status;     // 0, or the code of a wait that gave up
  int l2_prefetch; // k-blocks of W, beyond the ring, that a block asks into L2 before the dependency wait
  unsigned long long* trace;  // debugging: 8 timestamps of block 0 per launch, or null
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: false (and *status set) when the phase did not complete within TC_WAIT_NS.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = global_timer();
  while (!mbar_try_wait(bar, parity)) {
    if (global_timer() - t0 > TC_WAIT_NS) {
      atomicExch(status, code);
      return false;
    }
  }
  return true;
}
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* map, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, unsigned bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzled:
// start address >> 4; leading byte offset 1 (unused for swizzled K-major); stride byte offset
// 1024 >> 4 between groups of 8 rows; descriptor version 1; layout type 2 = SWIZZLE_128B.
__device__ __forceinline__ unsigned long long umma_desc(unsigned addr) {
  return (unsigned long long)((addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc,
                                          unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(unsigned addr, float* v) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(addr));
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// The stretch of units of block c: [unit_start(c), unit_start(c + 1)).
__device__ __forceinline__ long long unit_start(long long c, long long total, int blocks) { return c * total / blocks; }
// The block whose stretch holds unit u.
__device__ __forceinline__ int block_of(long long u, long long total, int blocks) {
  int c = (int)(u * blocks / total);
  while (c + 1 < blocks && unit_start(c + 1, total, blocks) <= u) ++c;
  while (c > 0 && unit_start(c, total, blocks) > u) --c;
  return c;
}

// Walks the segments of a block's stretch: (tile, first k-block, one past the last k-block).
struct Segments {
  long long u, u_end;
  int kb;
  __device__ Segments(long long u0, long long u1, int k_blocks) : u(u0), u_end(u1), kb(k_blocks) {}
  __device__ bool next(int& tile, int& kb_lo, int& kb_hi) {
    if (u >= u_end) return false;
    tile = (int)(u / kb);
    kb_lo = (int)(u - (long long)tile * kb);
    long long left = u_end - u;
    kb_hi = (int)min((long long)kb, kb_lo + left);
    u += kb_hi - kb_lo;
    return true;
  }
};

template <int MP>  // batch columns of an accumulator: 16, 32 or 64
__global__ void __launch_bounds__(TC_THREADS)
linear_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TcArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr int A_BYTES = TC_BM * TC_BK * 2;   // 16 KB
  constexpr int B_BYTES = MP * TC_BK * 2;      // 2, 4 or 8 KB
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TC_STAGES = TC_STAGES_FOR(MP);
  constexpr unsigned TMEM_COLS = 2 * MP < 32 ? 32 : 2 * MP;  // two accumulators; a power of two >= 32
  // instruction descriptor: D float32 (bits 4-5 = 1), A and B bfloat16 (bits 7-9, 10-12 = 1), both
  // K-major, N >> 3 at bit 17, M >> 4 at bit 24
  constexpr unsigned IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(MP >> 3) << 17) | ((TC_BM >> 4) << 24);

  unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned long long* bars = (unsigned long long*)(base + TC_STAGES * STAGE_BYTES);
  unsigned* tmem_slot = (unsigned*)(bars + 2 * TC_STAGES + 4);
  __shared__ int s_last;
  __shared__ int s_failed;
  __shared__ int s_acc_ok;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int blocks = gridDim.x;
  const long long total = (long long)a.tiles * a.k_blocks;
  const long long u0 = unit_start(blockIdx.x, total, blocks), u1 = unit_start(blockIdx.x + 1, total, blocks);
  const unsigned full0 = smem_u32(bars), empty0 = smem_u32(bars + TC_STAGES);
  const unsigned acc_full0 = smem_u32(bars + 2 * TC_STAGES), acc_free0 = smem_u32(bars + 2 * TC_STAGES + 2);

  if (tid == 0) {
    s_failed = 0;
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_free0 + 8 * b, 128);  // every epilogue thread arrives
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
  const bool tracing = a.trace != nullptr && blockIdx.x == 0;
  if (tracing && tid == 0) a.trace[0] = global_timer();
  // the kernel that follows in the stream may start its own prologue now
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      // Weights do not depend on the kernel before this one: the first ring of W tiles is
      // requested before the dependency wait, the matching x tiles after it.
      // Further W tiles of the stretch are only asked into L2: the requests are served while this
      // block sits in the wait, so that the kernel before this one ends with HBM still busy.
      int tile, kb_lo, kb_hi, it = 0;
      {
        Segments seg(u0, u1, a.k_blocks);
        const int ahead = TC_STAGES + a.l2_prefetch;
        while (it < ahead && seg.next(tile, kb_lo, kb_hi)) {
          for (int kb = kb_lo; kb < kb_hi && it < ahead; ++kb, ++it) {
            if (it < TC_STAGES) {
              mbar_expect_tx(full0 + 8 * it, STAGE_BYTES);
              tma_load_2d(smem_u32(base + it * STAGE_BYTES), &map_w, full0 + 8 * it, kb * TC_BK, tile * TC_BM);
            } else {
              tma_prefetch_l2_2d(&map_w, kb * TC_BK, tile * TC_BM);
            }
          }
        }
      }
      if (tracing) a.trace[1] = global_timer();
      asm volatile("griddepcontrol.wait;" ::: "memory");
      if (tracing) a.trace[2] = global_timer();
      Segments seg(u0, u1, a.k_blocks);
      it = 0;
      bool failed = false;
      while (!failed && seg.next(tile, kb_lo, kb_hi)) {
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          int s = it % TC_STAGES, round = it / TC_STAGES;
          unsigned dst = smem_u32(base + s * STAGE_BYTES);
          if (round > 0) {
            if (!mbar_wait(empty0 + 8 * s, (round & 1) ^ 1, a.status, TC_ERR_EMPTY_WAIT)) { failed = true; break; }
            mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
            tma_load_2d(dst, &map_w, full0 + 8 * s, kb * TC_BK, tile * TC_BM);
          }
          tma_load_2d(dst + A_BYTES, &map_x, full0 + 8 * s, kb * TC_BK, 0);
        }
      }
      if (failed) s_failed = 1;
      if (tracing) a.trace[3] = global_timer();  // all loads issued
    }
  } else if (warp == 1) {
    if (lane == 0) {
      Segments seg(u0, u1, a.k_blocks);
      int tile, kb_lo, kb_hi, it = 0, j = 0;
      bool failed = false;
      while (!failed && seg.next(tile, kb_lo, kb_hi)) {
        const int buf = j & 1;
        // the epilogue must have emptied this accumulator (first use of each: passes at once)
        if (!mbar_wait(acc_free0 + 8 * buf, ((j >> 1) & 1) ^ 1, a.status, TC_ERR_ACC_FREE_WAIT)) { failed = true; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned tmem_d = tmem_base + buf * MP;
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          int s = it % TC_STAGES, round = it / TC_STAGES;
          if (!mbar_wait(full0 + 8 * s, round & 1, a.status, TC_ERR_FULL_WAIT)) { failed = true; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          unsigned sa = smem_u32(base + s * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < TC_BK / 16; ++kk)
            umma_bf16(tmem_d, umma_desc(sa + kk * 32), umma_desc(sb + kk * 32), IDESC, (kb > kb_lo || kk) ? 1u : 0u);
          umma_commit(empty0 + 8 * s);  // arrives when these MMAs have read the stage
        }
        if (!failed) umma_commit(acc_full0 + 8 * buf);  // arrives when the segment's MMAs are done
        ++j;
      }
      if (failed) s_failed = 1;
      if (tracing) a.trace[4] = global_timer();  // all MMAs issued
    }
  } else {
    // ---- epilogue warps: TMEM lane quadrant warp % 4, one weight row per thread
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const size_t tile_floats = (size_t)TC_BM * MP;
    asm volatile("griddepcontrol.wait;" ::: "memory");  // before any global write of this kernel
    Segments seg(u0, u1, a.k_blocks);
    int tile, kb_lo, kb_hi, j = 0;
    float v[MP];
    while (seg.next(tile, kb_lo, kb_hi)) {
      const int buf = j & 1;
      // one thread waits (bounded) for the accumulator; the four warps then agree on the outcome
      if (warp == 2 && lane == 0) {
        s_acc_ok = mbar_wait(acc_full0 + 8 * buf, (j >> 1) & 1, a.status, TC_ERR_ACC_WAIT) ? 1 : 0;
        if (!s_acc_ok) s_failed = 1;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (!s_acc_ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int c = 0; c < MP; c += 16) tmem_ld16(tmem_base + ((unsigned)(quad * 32) << 16) + buf * MP + c, v + c);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(acc_free0 + 8 * buf);  // the MMA thread may overwrite this accumulator

      const int n = tile * TC_BM + row_in_tile;
      bool run_epilogue = true;
      if (kb_lo != 0 || kb_hi != a.k_blocks) {
        // a tile shared with other blocks: slot 0 holds a block's first segment, slot 1 its last
        const long long t0 = (long long)tile * a.k_blocks;
        const int c_first = block_of(t0, total, blocks), c_last = block_of(t0 + a.k_blocks - 1, total, blocks);
        const int my_slot = (j == 0) ? 0 : 1;
        float* mine = a.scratch + ((size_t)blockIdx.x * 2 + my_slot) * tile_floats + (size_t)row_in_tile * MP;
#pragma unroll
        for (int c = 0; c < MP; c += 4) *reinterpret_cast<float4*>(mine + c) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          int ticket = atomicAdd(a.counters + tile, 1);
          s_last = (ticket == c_last - c_first);
          if (s_last) a.counters[tile] = 0;  // ready for the next launch
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        run_epilogue = s_last != 0;
        if (run_epilogue) {
          __threadfence();
#pragma unroll
          for (int c = 0; c < MP; ++c) v[c] = 0.f;
          for (int cb = c_first; cb <= c_last; ++cb) {
            // block cb's piece of this tile is its first segment iff its stretch starts inside the tile
            long long cs = unit_start(cb, total, blocks);
            int slot = (cs >= t0) ? 0 : 1;
            // a block whose stretch starts exactly at the tile start also uses slot 0 (j == 0)
            const float* part = a.scratch + ((size_t)cb * 2 + slot) * tile_floats + (size_t)row_in_tile * MP;
#pragma unroll
            for (int c = 0; c < MP; c += 4) {
              float4 p = __ldcg(reinterpret_cast<const float4*>(part + c));
              v[c] += p.x; v[c + 1] += p.y; v[c + 2] += p.z; v[c + 3] += p.w;
            }
          }
        }
      }
      if (run_epilogue) {
        if (a.mode == 0) {
          if (n < a.N) {
#pragma unroll
            for (int m = 0; m < MP; ++m)
              if (m < a.M) store_from_f32(a.out, a.out_dtype, (size_t)m * a.ldo + n, v[m]);
          }
        } else {
          // rows 16j..16j+7 are gate rows 8j.., rows 16j+8..16j+15 the up rows of the same indices:
          // lane L (L % 16 < 8) holds a gate value and lane L + 8 the matching up value
          const int i = (n >> 4) * 8 + (n & 7);
#pragma unroll
          for (int m = 0; m < MP; ++m) {
            float other = __shfl_xor_sync(0xffffffffu, v[m], 8);
            if ((lane & 8) == 0 && m < a.M && n < a.N) {
              float g = v[m];
              store_from_f32(a.out, a.out_dtype, (size_t)m * a.ldo + i, g / (1.0f + expf(-g)) * other);
            }
          }
        }
      }
      ++j;
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the four warps take the segments in lockstep
    }
    if (tracing && warp == 2 && lane == 0) a.trace[5] = global_timer();  // epilogues done
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (s_failed) {
    // a wait gave up: loads that were issued may still be landing in this block's shared memory
    unsigned long long t0 = global_timer();
    while (global_timer() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
  if (tracing && tid == 32) a.trace[6] = global_timer();
}

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

static PFN_cuTensorMapEncodeTiled get_encode() {
  static PFN_cuTensorMapEncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (PFN_cuTensorMapEncodeTiled)p;
  }
  return fn;
}

// A [rows, K] bfloat16 row-major matrix, loaded in boxes of box_rows x 64 with 128-byte swizzle;
// rows and columns outside the matrix read as zero.
static bool make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
  PFN_cuTensorMapEncodeTiled enc = get_encode();
  if (!enc) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

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
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const TcArgs& a, int blocks, cudaStream_t stream) {
  constexpr int TC_STAGES = TC_STAGES_FOR(MP);
  size_t smem = (size_t)TC_STAGES * (TC_BM * TC_BK * 2 + MP * TC_BK * 2) + (2 * TC_STAGES + 4) * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(linear_tc_kernel<MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(TC_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, linear_tc_kernel<MP>, mw, mx, a);
  if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
  return BN_OK;
}

// x [M, K], w [N, K] bfloat16, both 16-byte aligned with K a multiple of 8.  mode 0: out [M, ldo]
// of out_dtype; mode 2: N = 2 I weight rows in blocks of 8 gate / 8 up rows, out holds
// silu(gate) * up in I columns.  max_blocks caps the number of persistent blocks (0: one per SM).
// scratch: blocks * 2 * 128 * Mp floats (Mp = 16, 32 or 64 >= M); counters: ceil(N/128) zeroed
// ints; both may be shared by launches that do not overlap.  status: one int on the device, left 0
// unless a wait inside the kernel gave up.
extern "C" int bn_linear_tc(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K, int ldo,
                            int mode, int max_blocks, float* scratch, long long scratch_floats, int* counters,
                            int n_counters, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return BN_OK;
  if (M > 64 || K <= 0 || K % 8 || max_blocks < 0 || (mode != 0 && mode != 2) || !status) return BN_ERR_BAD_ARG;
  if (mode == 2 && (N % 16)) return BN_ERR_BAD_ARG;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return BN_ERR_BAD_ARG;
  int mp = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  int tiles = (N + TC_BM - 1) / TC_BM;
  int k_blocks = (K + TC_BK - 1) / TC_BK;
  long long total = (long long)tiles * k_blocks;
  int blocks = max_blocks > 0 ? max_blocks : sm_count();
  if (blocks > total) blocks = (int)total;
  if (!scratch || !counters || n_counters < tiles || scratch_floats < (long long)blocks * 2 * TC_BM * mp)
    return BN_ERR_BAD_ARG;
  CUtensorMap mw, mx;
  if (!make_map(&mw, w, N, K, TC_BM) || !make_map(&mx, x, M, K, mp)) return BN_ERR_BAD_ARG;
  TcArgs a;
  a.out = out; a.out_dtype = out_dtype; a.M = M; a.N = N; a.K = K; a.ldo = ldo; a.mode = mode;
  a.k_blocks = k_blocks; a.tiles = tiles; a.scratch = scratch; a.counters = counters; a.status = status;
  static int l2_prefetch = -1;
  if (l2_prefetch < 0) {
    const char* e = getenv("BN_TC_L2_PREFETCH");  // tuning knob: k-blocks per block, 0 = off
    l2_prefetch = e ? atoi(e) : 16;
    if (l2_prefetch < 0) l2_prefetch = 0;
  }
  a.l2_prefetch = l2_prefetch;
  a.trace = nullptr;
  if (g_trace && g_trace_n < g_trace_cap) a.trace = g_trace + 8 * (g_trace_n++);
  if (mp == 16) return launch_tc<16>(mw, mx, a, blocks, stream);
  if (mp == 32) return launch_tc<32>(mw, mx, a, blocks, stream);
  return launch_tc<64>(mw, mx, a, blocks, stream);
}
