// Decode attention in bfloat16 on tensor cores: one new token per sequence over its paged cache,
// position encoding, cache write, attention and the combination of the key chunks in one launch.
//
// grid = (sequences, key/value heads x groups of 16 query heads, splits).  A block walks a run of
// the sequence's cache pages (64 positions each) through a ring of two or three shared-memory
// stages.  One thread requests whole pages by TMA (a page of one head's keys is HD/64 boxes of
// 64 rows x 128 bytes, 128-byte swizzled, completing on the stage's mbarrier); the ring is filled
// at the start, before the dependency wait of the programmatic launch: page table, positions and
// the cached rows of earlier positions were written by kernels that completed before the kernel in
// front of this one, which only produces the new token's q|k|v row.  The query heads that share
// the key/value head are the 16 rows of an MMA tile; the block rotates them itself.  The block
// whose run holds the new position also rotates the new key, writes key and value to the cache
// and puts them into its stage directly (rows of that page behind the new position are cleared
// in shared memory, whatever the cache holds there).  Each of the four warps owns 16 of a page's 64
// keys and keeps its own running maximum, sum and output (scores and the weighted value sum on
// m16n8k16 MMAs, statistics in float32), so the loop needs no exchange between warps; at the end
// the four are merged in shared memory.  With more than one split per sequence the merged result
// is written as an unnormalised partial with maximum and sum, and the block that draws the last
// ticket of its (sequence, head group) merges the splits and writes the output; with at most eight
// splits these are one thread-block cluster instead, every block keeps its result in its own
// shared memory and, after the cluster's barrier, adds up a slice of the output read from all of
// them through distributed shared memory (no global round trip, no ticket).  How many pages a
// block walks is chosen by the host from the batch (few sequences: many splits; many sequences:
// one block per sequence and head group, no partials at all).
// Page borders are fixed in position, so a row's arithmetic depends on its own position and the
// split size only.  Head sizes in steps of 16 run on the instantiation for 64, 128 or 256 with the
// missing dimensions zero in shared memory.
//
// Reference: scores = q.k * scale over the causal range, softmax with the maximum subtracted,
// weighted sum of values, query head h uses key/value head h / (H / KV)
// (src/transformer/gqa_scalar.c:61-121; online form gqa_scalar.c:127-207); rotary pairs
// (i, i + half), angle pos * theta^(-2i/dims) as a running float32 product
// (src/transformer/cpu_backend.c:283-296, src/model_arch.c:322-338).  The reference's CUDA decode
// attention is one block per head on CUDA cores without a split over the keys, with a variant
// that fuses the rotary encoding of q (src/gpu_cuda.cu:9718, 9989).
#include "tma.cuh"
#include "mma.cuh"

#define DT_THREADS 128
#define DT_SPLIT_MIN_PAGES 8  // a sequence with fewer visible pages is not split (the merge would cost more than the walk)
#define DT_ROWS 16  // query heads per block (the MMA's 16 rows)

// Byte offset of 16-byte chunk `chunk` of row `row` in the query tile, whose rows hold HD bfloat16 (XOR swizzle).
template <int HD>
__device__ __forceinline__ unsigned dt_off(int row, int chunk) {
  return (unsigned)(row * HD * 2 + ((chunk ^ (row & 7)) << 4));
}
// The same for a page of keys or values as TMA leaves it: boxes of 64 rows x 128 bytes (64
// dimensions), box after box, the chunk index within a row XORed with the row's low three bits.
#define DT_BOX_BYTES (BN_PAGE * 128)
__device__ __forceinline__ unsigned dt_koff(int row, int chunk) {
  return (unsigned)((chunk >> 3) * DT_BOX_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}
#define DT_ERR_PAGE_WAIT 4
__device__ __forceinline__ void dt_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// One float of block `rank`'s shared memory, at the address that `local_addr` has here.
__device__ __forceinline__ float dt_ld_dsmem(unsigned local_addr, unsigned rank) {
  unsigned remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
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
  int* status;     // 0, or DT_ERR_PAGE_WAIT when a page never arrived
  BN_TRACE_ONLY(unsigned long long* trace;)  // debugging: timestamps of blocks (0, 0, z), 16 per block, or null
  float* part_o;   // [n_seqs][n_heads][splits][head_dim]
  float* part_ml;  // [n_seqs][n_heads][splits][2]: maximum (in the scaled log2 domain) and sum
  int pages_per_block;
  int cluster;     // 1: the splits of a sequence are one thread-block cluster and merge through distributed shared memory
  const int* items;  // null, or for each blockIdx.x what it works on: sequence | split << 16 | splits << 24, or -1 for
                     // nothing.  The grid then has no z; clusters of `group` blocks run along x, and a cluster
                     // holds either the splits of one sequence or `group` sequences that are not split.
  int* tickets;    // [n_seqs][gridDim.y], zero before and after
  __nv_bfloat16* out;
  int out_stride;
};

template <int HD, int DT_STAGES>
__global__ void __launch_bounds__(DT_THREADS)
attention_decode_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, DtArgs a) {
  pdl_launch_dependents();  // the next kernel in the stream may begin its prologue
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  BN_TRACE_ONLY(unsigned long long* tr = (a.trace && a.items == nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) ? a.trace + 16 * blockIdx.z : nullptr;)
  BN_TRACE_ONLY(if (tr) tr[0] = global_timer();)
  constexpr int CHUNKS = HD / 8, KSTEPS = HD / 16, NT_O = HD / 8, BOXES = HD / 64;
  constexpr int PAGE_BYTES = BN_PAGE * HD * 2;       // one page of keys (or values) of one head
  constexpr int STAGE_BYTES = 2 * PAGE_BYTES;
  constexpr int OSTRIDE = HD + 8;                    // floats per row of a warp's output (padded against bank conflicts)
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* stages = smem;                      // 1024-byte aligned: the swizzle is a function of the address
  unsigned char* q_tile = stages + DT_STAGES * STAGE_BYTES;
  __nv_bfloat16* new_kv = reinterpret_cast<__nv_bfloat16*>(q_tile + DT_ROWS * HD * 2);  // [2][HD]
  float* ml_part = reinterpret_cast<float*>(new_kv + 2 * HD);  // [4 warps][16][2]
  float* ml_fin = ml_part + 4 * DT_ROWS * 2;                   // [16][2]
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(ml_fin + DT_ROWS * 2);  // [DT_STAGES]
  float* cs_tab = reinterpret_cast<float*>(bars + DT_STAGES);  // [rotary_dims / 2][2]: cosine, sine of this position's angles
  float* wsc = cs_tab + HD;                                    // [4 warps][16]: each warp's weight in the block's result
  float* o_part = reinterpret_cast<float*>(stages);            // [4 warps][16][OSTRIDE], after the loop
  float* o_fin = o_part + 4 * DT_ROWS * OSTRIDE;               // [16][HD]: the block's unnormalised result
  static_assert((4 * DT_ROWS * OSTRIDE + DT_ROWS * HD) * 4 <= DT_STAGES * STAGE_BYTES, "the warps' outputs and the block's result reuse the stages");
  const unsigned s_q = smem_u32(q_tile), s_st = smem_u32(stages), full0 = smem_u32(bars);
  __shared__ int s_last;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // which sequence, which of its splits, of how many
  int b = blockIdx.x, zi = blockIdx.z, nz = gridDim.z;
  if (a.items != nullptr) {
    const int item = a.items[blockIdx.x];
    if (item < 0) {  // padding: the whole cluster is, or its other blocks work alone
      pdl_wait();
      return;
    }
    b = item & 0xFFFF; zi = (item >> 16) & 0xFF; nz = (item >> 24) & 0x7F;
  }
  const int g4 = lane >> 2, t4 = lane & 3;
  const int head_dim = a.head_dim, n_kv_heads = a.n_kv_heads, n_heads = a.n_heads;
  const int group = n_heads / n_kv_heads;
  const int gblocks = (group + DT_ROWS - 1) / DT_ROWS;
  const int kvh = blockIdx.y / gblocks, gb = blockIdx.y % gblocks;
  const int h0 = kvh * group + gb * DT_ROWS;
  const int G = min(DT_ROWS, group - gb * DT_ROWS);
  const int pos = a.tok_pos[b];
  const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  // pages that hold a visible key, and this block's run of them
  const int p_lo = lo / BN_PAGE, p_hi = pos / BN_PAGE;
  // The blocks of a sequence share its visible pages evenly (as many as the launch gives each
  // sequence, whatever the bound it was sized for); a sequence too short for a split to pay is the
  // first block's alone.
  const int vis = p_hi - p_lo + 1;
  const int ppb = vis < DT_SPLIT_MIN_PAGES ? vis : min(a.pages_per_block, (vis + nz - 1) / nz);
  const int my_lo = p_lo + zi * ppb;
  const int my_hi = min(p_hi, my_lo + ppb - 1);
  const int z_lo = 0, z_hi = (vis - 1) / ppb;  // splits with a visible page
  const bool alone = (z_lo == z_hi);
  const bool clustered = a.cluster != 0 && !alone;  // the same for every block of the cluster
  if (my_lo > my_hi) {
    pdl_wait();  // no block of this grid ends before the grids in front of it have
    if (clustered) {  // nothing to add, but the cluster's barriers need every block
      dt_cluster_sync();
      dt_cluster_sync();
    }
    return;
  }
  const int n_pages = my_hi - my_lo + 1;
  const int n_splits = nz;
  const int* pt = a.page_table + (size_t)a.slots[b] * a.pt_stride;
  const bool has_new = (p_hi >= my_lo && p_hi <= my_hi);  // the new token's page is in this run
  const int new_row = pos - p_hi * BN_PAGE;

  auto request_page = [&](int page_idx, int stage) {  // one thread: the whole page of this head, keys and values
    const int page = pt[page_idx];
    const unsigned bar = full0 + 8 * stage, sk = s_st + stage * STAGE_BYTES, sv = sk + PAGE_BYTES;
    mbar_expect_tx(bar, STAGE_BYTES);
#pragma unroll
    for (int bx = 0; bx < BOXES; ++bx) {
      tma_load_3d(sk + bx * DT_BOX_BYTES, &map_k, bar, bx * 64, kvh * BN_PAGE, page);
      tma_load_3d(sv + bx * DT_BOX_BYTES, &map_v, bar, bx * 64, kvh * BN_PAGE, page);
    }
  };
  if (tid == 0) {
    tma_prefetch_map(&map_k);
    tma_prefetch_map(&map_v);
    for (int st = 0; st < DT_STAGES; ++st) mbar_init(full0 + 8 * st, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int st = 0; st < DT_STAGES; ++st)  // the whole ring is requested at once
      if (st < n_pages) request_page(my_lo + st, st);
  }
  BN_TRACE_ONLY(if (tr) tr[1] = global_timer();)
  // the rotation of this position, also before the wait: it depends on the position only
  const int half = a.rotary_dims >> 1;
  for (int i = tid; i < half; i += DT_THREADS) {
    float sn, cs;
    sincosf(rope_angle(pos, i, a.theta_scale), &sn, &cs);
    cs_tab[2 * i] = cs;
    cs_tab[2 * i + 1] = sn;
  }
  // rows past the head group and dimensions past the head size are zero in the query tile and in
  // the new token's row (also before the wait)
  for (int p = tid; p < DT_ROWS * HD / 8; p += DT_THREADS) reinterpret_cast<uint4*>(q_tile)[p] = make_uint4(0u, 0u, 0u, 0u);
  for (int p = tid; p < 2 * HD / 8; p += DT_THREADS) reinterpret_cast<uint4*>(new_kv)[p] = make_uint4(0u, 0u, 0u, 0u);
  BN_TRACE_ONLY(if (tr) tr[2] = global_timer();)
  pdl_wait();  // the kernel before this one has completed: the q|k|v rows are there
  BN_TRACE_ONLY(if (tr) tr[3] = global_timer();)
  __syncthreads();

  // ---- queries of this head group (rotated, rounded to bfloat16, rows of the 16-row tile) and the
  // new token's key (rotated) and value (to the cache, and kept for this block's stage).  The
  // work is a list of 16-byte items, one per thread, so that all loads are in flight together.
  const __nv_bfloat16* qrow = a.qkv + (size_t)b * a.q_stride;
  const __nv_bfloat16* kraw = qrow + a.k_off + (size_t)kvh * head_dim;
  const __nv_bfloat16* vraw = qrow + a.v_off + (size_t)kvh * head_dim;
  const size_t new_off = has_new ? (((size_t)pt[p_hi] * n_kv_heads + kvh) * BN_PAGE + new_row) * (size_t)head_dim : 0;
  if ((a.rotary_dims & 15) == 0) {
    const int hc = half >> 3;                           // chunks of 8 in half the rotary dimensions
    const int rc = (head_dim - a.rotary_dims) >> 3;     // chunks that are not rotated
    const int per_head = hc + rc;                       // items of one head: rotary pairs, then plain chunks
    const int n_q = G * per_head, n_k = has_new ? per_head : 0, n_v = has_new ? (head_dim >> 3) : 0;
    for (int item = tid; item < n_q + n_k + n_v; item += DT_THREADS) {
      if (item >= n_q + n_k) {  // a chunk of the new value
        const int c = item - n_q - n_k;
        const uint4 v = *reinterpret_cast<const uint4*>(vraw + c * 8);
        *reinterpret_cast<uint4*>(a.v_cache + new_off + c * 8) = v;
        *reinterpret_cast<uint4*>(new_kv + HD + c * 8) = v;
        continue;
      }
      const bool is_k = item >= n_q;
      const int g = is_k ? 0 : item / per_head, c = is_k ? item - n_q : item - g * per_head;
      const __nv_bfloat16* src = is_k ? kraw : qrow + (size_t)(h0 + g) * head_dim;
      if (c >= hc) {  // a plain chunk behind the rotary dimensions
        const int d = a.rotary_dims + (c - hc) * 8;
        const uint4 v = *reinterpret_cast<const uint4*>(src + d);
        if (is_k) {
          *reinterpret_cast<uint4*>(a.k_cache + new_off + d) = v;
          *reinterpret_cast<uint4*>(new_kv + d) = v;
        } else {
          *reinterpret_cast<uint4*>(q_tile + dt_off<HD>(g, d >> 3)) = v;
        }
        continue;
      }
      uint4 xv = *reinterpret_cast<const uint4*>(src + c * 8), yv = *reinterpret_cast<const uint4*>(src + half + c * 8);
      const __nv_bfloat16* xs = reinterpret_cast<const __nv_bfloat16*>(&xv);
      const __nv_bfloat16* ys = reinterpret_cast<const __nv_bfloat16*>(&yv);
      uint4 lo4, hi4;
      __nv_bfloat16* los = reinterpret_cast<__nv_bfloat16*>(&lo4);
      __nv_bfloat16* his = reinterpret_cast<__nv_bfloat16*>(&hi4);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float cs = cs_tab[2 * (c * 8 + e)], sn = cs_tab[2 * (c * 8 + e) + 1];
        const float x = __bfloat162float(xs[e]), y = __bfloat162float(ys[e]);
        los[e] = __float2bfloat16_rn(x * cs - y * sn);
        his[e] = __float2bfloat16_rn(x * sn + y * cs);
      }
      if (is_k) {
        *reinterpret_cast<uint4*>(a.k_cache + new_off + c * 8) = lo4;
        *reinterpret_cast<uint4*>(a.k_cache + new_off + half + c * 8) = hi4;
        *reinterpret_cast<uint4*>(new_kv + c * 8) = lo4;
        *reinterpret_cast<uint4*>(new_kv + half + c * 8) = hi4;
      } else {
        *reinterpret_cast<uint4*>(q_tile + dt_off<HD>(g, c)) = lo4;
        *reinterpret_cast<uint4*>(q_tile + dt_off<HD>(g, c + hc)) = hi4;
      }
    }
  } else {
    // rotary dimensions that are no multiple of 16: element by element
    auto q_at = [&](int g, int d) -> __nv_bfloat16* {
      return reinterpret_cast<__nv_bfloat16*>(q_tile + dt_off<HD>(g, d >> 3)) + (d & 7);
    };
    for (int p = tid; p < G * half; p += DT_THREADS) {
      int g = p / half, i = p - g * half;
      const float cs = cs_tab[2 * i], sn = cs_tab[2 * i + 1];
      const __nv_bfloat16* hd = qrow + (size_t)(h0 + g) * head_dim;
      float x = __bfloat162float(hd[i]), y = __bfloat162float(hd[i + half]);
      *q_at(g, i) = __float2bfloat16_rn(x * cs - y * sn);
      *q_at(g, i + half) = __float2bfloat16_rn(x * sn + y * cs);
    }
    const int rest = head_dim - a.rotary_dims;
    for (int p = tid; p < G * rest; p += DT_THREADS) {
      int g = p / rest, d = a.rotary_dims + p - g * rest;
      *q_at(g, d) = qrow[(size_t)(h0 + g) * head_dim + d];
    }
    if (has_new) {
      for (int i = tid; i < half; i += DT_THREADS) {
        const float cs = cs_tab[2 * i], sn = cs_tab[2 * i + 1];
        float x = __bfloat162float(kraw[i]), y = __bfloat162float(kraw[i + half]);
        __nv_bfloat16 k0 = __float2bfloat16_rn(x * cs - y * sn), k1 = __float2bfloat16_rn(x * sn + y * cs);
        a.k_cache[new_off + i] = k0;
        a.k_cache[new_off + i + half] = k1;
        new_kv[i] = k0;
        new_kv[i + half] = k1;
      }
      for (int d = a.rotary_dims + tid; d < head_dim; d += DT_THREADS) {
        a.k_cache[new_off + d] = kraw[d];
        new_kv[d] = kraw[d];
      }
      for (int d = tid; d < head_dim; d += DT_THREADS) {
        a.v_cache[new_off + d] = vraw[d];
        new_kv[HD + d] = vraw[d];
      }
    }
  }

  // ---- the loop over this block's pages; warp w owns keys 16w..16w+15 of every page
  float o[NT_O][4];
#pragma unroll
  for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int mi = lane >> 3, r8 = lane & 7;
  // Q as MMA operand fragments, kept in registers when the head is small enough
  constexpr bool Q_IN_REGS = HD <= 128;
  unsigned qf[Q_IN_REGS ? KSTEPS : 1][4];
  bool failed = false;
  BN_TRACE_ONLY(if (tr) tr[4] = global_timer();)
  for (int i = 0; i < n_pages; ++i) {
    const int stage = i % DT_STAGES;
    // one thread watches the stage's mbarrier, the others sleep at the block's barrier
    bool arrived = true;
    if (tid == 0) arrived = mbar_wait(full0 + 8 * stage, (unsigned)(i / DT_STAGES) & 1u, a.status, DT_ERR_PAGE_WAIT);
    // page i has landed for everyone; the stage of page i-1 is free; q and new_kv are written
    if (__syncthreads_or(arrived ? 0 : 1)) { failed = true; break; }
    BN_TRACE_ONLY(if (tr && i < 2) tr[5 + i] = global_timer();)
    if (tid == 0 && i >= 1 && i - 1 + DT_STAGES < n_pages) request_page(my_lo + i - 1 + DT_STAGES, (i - 1) % DT_STAGES);
    if (Q_IN_REGS && i == 0) {
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks)
        ldsm_x4(s_q + dt_off<HD>(r8 + (mi & 1) * 8, ks * 2 + (mi >> 1)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }
    const int page_idx = my_lo + i;
    const unsigned sk = s_st + stage * STAGE_BYTES, sv = sk + PAGE_BYTES;
    if (has_new && page_idx == p_hi) {
      // put the new token's row into the stage (the page came with what the cache held there) and
      // clear the value rows behind it: their weights are zero, but zero times anything must be zero
      unsigned char* kt = stages + stage * STAGE_BYTES;
      for (int c = tid; c < 2 * CHUNKS; c += DT_THREADS) {
        int which = c / CHUNKS, cc = c - which * CHUNKS;
        *reinterpret_cast<uint4*>(kt + which * PAGE_BYTES + dt_koff(new_row, cc)) =
            *reinterpret_cast<const uint4*>(new_kv + which * HD + cc * 8);
      }
      for (int c = tid; c < (BN_PAGE - 1 - new_row) * CHUNKS; c += DT_THREADS) {
        int r = new_row + 1 + c / CHUNKS, cc = c % CHUNKS;
        *reinterpret_cast<uint4*>(kt + PAGE_BYTES + dt_koff(r, cc)) = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncthreads();
    }
    // S = Q K^T for this warp's 16 keys
    float s[2][4];
    s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
    const int krow0 = warp * 16;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      unsigned a0, a1, a2, a3, b0, b1, b2, b3;
      if (Q_IN_REGS) {
        a0 = qf[ks][0]; a1 = qf[ks][1]; a2 = qf[ks][2]; a3 = qf[ks][3];
      } else {
        ldsm_x4(s_q + dt_off<HD>(r8 + (mi & 1) * 8, ks * 2 + (mi >> 1)), a0, a1, a2, a3);
      }
      ldsm_x4(sk + dt_koff(krow0 + (mi >> 1) * 8 + r8, ks * 2 + (mi & 1)), b0, b1, b2, b3);
      mma_bf16(s[0], a0, a1, a2, a3, b0, b1);
      mma_bf16(s[1], a0, a1, a2, a3, b2, b3);
    }
    // mask, running maximum, exponentials; rows g4 and g4 + 8 of the head tile
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        int kpos = page_idx * BN_PAGE + krow0 + j * 8 + 2 * t4 + (c & 1);
        bool ok = kpos >= lo && kpos <= pos;
        float v = ok ? s[j][c] * a.scale_log2e : -INFINITY;
        s[j][c] = v;
        m_new[c >> 1] = fmaxf(m_new[c >> 1], v);
      }
    }
    float alpha[2], l_add[2] = {0.f, 0.f};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      m_new[e] = fmaxf(m_new[e], __shfl_xor_sync(0xffffffffu, m_new[e], 1));
      m_new[e] = fmaxf(m_new[e], __shfl_xor_sync(0xffffffffu, m_new[e], 2));
      alpha[e] = (m_run[e] == -INFINITY) ? 0.f : exp2f(m_run[e] - m_new[e]);
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
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
    // O += P V over the 16 keys
    {
      unsigned a0 = pack_bf16(s[0][0], s[0][1]), a1 = pack_bf16(s[0][2], s[0][3]);
      unsigned a2 = pack_bf16(s[1][0], s[1][1]), a3 = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
      for (int j = 0; j < NT_O; j += 2) {
        unsigned b0, b1, b2, b3;
        ldsm_x4_trans(sv + dt_koff(krow0 + (mi & 1) * 8 + r8, j + (mi >> 1)), b0, b1, b2, b3);
        mma_bf16(o[j], a0, a1, a2, a3, b0, b1);
        mma_bf16(o[j + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }
  if (failed) {
    // a page never arrived: loads that were requested may still be landing in this block's shared
    // memory, so give them a bounded time and leave without a result (the status word says so)
    unsigned long long t0 = global_timer();
    while (global_timer() - t0 < 200000ull) __nanosleep(1000);
    if (clustered) {
      dt_cluster_sync();
      dt_cluster_sync();
    }
    return;
  }
  BN_TRACE_ONLY(if (tr) tr[7] = global_timer();)
  __syncthreads();  // every warp is done with the stages: they now hold the warps' outputs
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 1);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 2);
    int row = g4 + e * 8;
    if (t4 == 0) {
      ml_part[(warp * DT_ROWS + row) * 2] = m_run[e];
      ml_part[(warp * DT_ROWS + row) * 2 + 1] = l_run[e];
    }
#pragma unroll
    for (int j = 0; j < NT_O; ++j) {
      float2 v = make_float2(o[j][2 * e], o[j][2 * e + 1]);
      *reinterpret_cast<float2*>(o_part + ((size_t)(warp * DT_ROWS + row)) * OSTRIDE + j * 8 + 2 * t4) = v;
    }
  }
  __syncthreads();
  // ---- merge the four warps: weights first (one thread per warp and row), then the rows
  if (tid < 4 * DT_ROWS) {
    const int w = tid >> 4, g = tid & 15;
    float m = -INFINITY;
    for (int x = 0; x < 4; ++x) m = fmaxf(m, ml_part[(x * DT_ROWS + g) * 2]);
    const float mw = ml_part[(w * DT_ROWS + g) * 2];
    wsc[tid] = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
    if (w == 0) ml_fin[g * 2] = m;
  }
  __syncthreads();
  if (tid < DT_ROWS) {
    float l = 0.f;
    for (int w = 0; w < 4; ++w) l += wsc[w * DT_ROWS + tid] * ml_part[(w * DT_ROWS + tid) * 2 + 1];
    ml_fin[tid * 2 + 1] = l;  // rows past G hold zeros: maximum -inf, sum 0
  }
  __syncthreads();
  for (int i = tid; i < G * head_dim; i += DT_THREADS) {
    int g = i / head_dim, d = i - g * head_dim;
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) acc += wsc[w * DT_ROWS + g] * o_part[(size_t)(w * DT_ROWS + g) * OSTRIDE + d];
    if (alone)  // the only split of this sequence: normalise and store
      a.out[(size_t)b * a.out_stride + (size_t)(h0 + g) * head_dim + d] = __float2bfloat16_rn(acc / ml_fin[g * 2 + 1]);
    else if (clustered) o_fin[g * HD + d] = acc;
    else a.part_o[(((size_t)b * n_heads + h0 + g) * n_splits + zi) * head_dim + d] = acc;
  }
  if (alone) {
    BN_TRACE_ONLY(if (tr) tr[8] = global_timer();)
    return;
  }
  if (clustered) {
    // ---- every block's result is in its own shared memory: after the cluster's barrier each
    // active block adds up, in split order, a slice of the rows' dimensions read from all of them
    dt_cluster_sync();
    BN_TRACE_ONLY(if (tr) tr[8] = global_timer();)
    const unsigned a_ml = smem_u32(ml_fin), a_o = smem_u32(o_fin);
    const int n_act = z_hi - z_lo + 1, mine = zi - z_lo;
    const int total = G * head_dim, per = (total + n_act - 1) / n_act;
    for (int i = mine * per + tid; i < min(total, (mine + 1) * per); i += DT_THREADS) {
      int g = i / head_dim, d = i - g * head_dim;
      // every split's maximum, sum and value of this element in one round of remote loads (a thread
      // works out the weights of its row itself: a second round would cost more than the arithmetic)
      float mz[8], lz[8], v[8], m = -INFINITY;
#pragma unroll
      for (int z = 0; z < 8; ++z) {
        const bool on = z >= z_lo && z <= z_hi;
        mz[z] = on ? dt_ld_dsmem(a_ml + (unsigned)(g * 2) * 4, (unsigned)z) : -INFINITY;
        lz[z] = on ? dt_ld_dsmem(a_ml + (unsigned)(g * 2 + 1) * 4, (unsigned)z) : 0.f;
        v[z] = on ? dt_ld_dsmem(a_o + (unsigned)(g * HD + d) * 4, (unsigned)z) : 0.f;
      }
#pragma unroll
      for (int z = 0; z < 8; ++z) m = fmaxf(m, mz[z]);
      float den = 0.f, num = 0.f;
#pragma unroll
      for (int z = 0; z < 8; ++z) {
        const float w = (mz[z] == -INFINITY) ? 0.f : exp2f(mz[z] - m);
        den += w * lz[z];
        num += w * v[z];
      }
      a.out[(size_t)b * a.out_stride + (size_t)(h0 + g) * head_dim + d] = __float2bfloat16_rn(num / den);
    }
    BN_TRACE_ONLY(if (tr) tr[10] = global_timer();)
    dt_cluster_sync();  // no block leaves while another still reads its result
    return;
  }
  if (tid < G) {
    size_t oo = (((size_t)b * n_heads + h0 + tid) * n_splits + zi) * 2;
    a.part_ml[oo] = ml_fin[tid * 2];
    a.part_ml[oo + 1] = ml_fin[tid * 2 + 1];
  }

  // ---- the block that draws the last ticket of this (sequence, head group) merges the splits
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int* t = a.tickets + (size_t)b * gridDim.y + blockIdx.y;
    int ticket = atomicAdd(t, 1);
    s_last = (ticket == z_hi - z_lo);
    if (s_last) *t = 0;
  }
  __syncthreads();
  BN_TRACE_ONLY(if (tr) tr[9] = global_timer();)
  if (!s_last) return;
  __threadfence();
  if (tid < G) {
    const float* ml = a.part_ml + ((size_t)b * n_heads + h0 + tid) * n_splits * 2;
    float m = -INFINITY;
    for (int z = z_lo; z <= z_hi; ++z) m = fmaxf(m, __ldcg(ml + 2 * z));
    float den = 0.f;
    for (int z = z_lo; z <= z_hi; ++z) den += exp2f(__ldcg(ml + 2 * z) - m) * __ldcg(ml + 2 * z + 1);
    ml_fin[tid * 2] = m;
    ml_fin[tid * 2 + 1] = den;
  }
  __syncthreads();
  for (int i = tid; i < G * head_dim; i += DT_THREADS) {
    int g = i / head_dim, d = i - g * head_dim;
    const float* ml = a.part_ml + ((size_t)b * n_heads + h0 + g) * n_splits * 2;
    const float* po = a.part_o + ((size_t)b * n_heads + h0 + g) * n_splits * head_dim;
    float m = ml_fin[g * 2], num = 0.f;
    for (int z = z_lo; z <= z_hi; ++z) num += exp2f(__ldcg(ml + 2 * z) - m) * __ldcg(po + (size_t)z * head_dim + d);
    a.out[(size_t)b * a.out_stride + (size_t)(h0 + g) * head_dim + d] = __float2bfloat16_rn(num / ml_fin[g * 2 + 1]);
  }
  BN_TRACE_ONLY(if (tr) tr[10] = global_timer();)
}

#ifdef BN_TRACE
// Debugging aid: bn_attention_decode_tc_trace(n) makes the next n launches record timestamps of
// their blocks (0, 0, z < 8) (device buffer allocated here; not used on the product path).
static unsigned long long* g_dt_trace = nullptr;
static int g_dt_trace_n = 0, g_dt_trace_cap = 0;
extern "C" int bn_attention_decode_tc_trace(int n) {
  if (g_dt_trace) cudaFree(g_dt_trace);
  g_dt_trace = nullptr; g_dt_trace_n = 0; g_dt_trace_cap = 0;
  if (n <= 0) return 0;
  if (cudaMalloc(&g_dt_trace, (size_t)n * 8 * 16 * 8) != cudaSuccess) return 1;
  cudaMemset(g_dt_trace, 0, (size_t)n * 8 * 16 * 8);
  g_dt_trace_cap = n;
  return 0;
}
extern "C" int bn_attention_decode_tc_trace_read(unsigned long long* host, int n) {
  if (!g_dt_trace || n > g_dt_trace_cap) return 1;
  return cudaMemcpy(host, g_dt_trace, (size_t)n * 8 * 16 * 8, cudaMemcpyDeviceToHost) != cudaSuccess;
}
#endif

// Dynamic shared memory of a block: alignment slack, the ring of key and value pages, the query
// tile, the new key and value, the warps' and the block's maxima and sums, the ring's mbarriers,
// the rotation table and the warps' weights.
template <int HD, int DT_STAGES>
static constexpr size_t dt_smem_bytes() {
  return 1024 + (size_t)DT_STAGES * 2 * BN_PAGE * HD * 2 + (size_t)DT_ROWS * HD * 2 + 2 * HD * 2 +
         (4 * DT_ROWS * 2 + DT_ROWS * 2) * sizeof(float) + DT_STAGES * 8 + HD * sizeof(float) + 4 * DT_ROWS * sizeof(float);
}
template <int HD, int DT_STAGES>
static int launch_dt2(const CUtensorMap& mk, const CUtensorMap& mv, const DtArgs& a, dim3 grid, dim3 cluster, cudaStream_t stream) {
  size_t smem = dt_smem_bytes<HD, DT_STAGES>();
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_tc_kernel<HD, DT_STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
    configured = true;
  }
  if (a.cluster) {
    cudaError_t e = bn_launch_cluster(attention_decode_tc_kernel<HD, DT_STAGES>, grid, dim3(DT_THREADS), smem, stream,
                                      cluster, mk, mv, a);
    if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
    return BN_OK;
  }
  BN_LAUNCH((attention_decode_tc_kernel<HD, DT_STAGES>), grid, DT_THREADS, smem, stream, mk, mv, a);
  return BN_OK;
}
// How many blocks of a ring depth fit on the device at once (asked of the runtime once per kernel).
template <int HD, int DT_STAGES>
static long long dt_slots() {
  static long long slots = 0;
  if (!slots) {
    size_t smem = dt_smem_bytes<HD, DT_STAGES>();
    int per_sm = 0, dev = 0, sms = 0;
    cudaFuncSetAttribute(attention_decode_tc_kernel<HD, DT_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_tc_kernel<HD, DT_STAGES>, DT_THREADS, smem) != cudaSuccess ||
        cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || per_sm <= 0 || sms <= 0)
      slots = 2 * 148;
    else
      slots = (long long)per_sm * sms;
  }
  return slots;
}
// Ring depth.  Short runs (at most two pages per block) take two stages: both pages are requested
// at once anyway.  Otherwise three stages keep a block's pages coming, but two let a third block
// share the SM (shared memory is the limit at head size 128): when that saves a wave of blocks it
// wins although each block runs about an eighth slower (40 heads of 128, 2,000 positions, 8
// sequences = 320 blocks: 77 us with three stages in two waves, 53 us with two stages in one).
template <int HD>
static int launch_dt(const CUtensorMap& mk, const CUtensorMap& mv, const DtArgs& a, dim3 grid, dim3 cluster, cudaStream_t stream) {
  if (a.pages_per_block <= 2) return launch_dt2<HD, 2>(mk, mv, a, grid, cluster, stream);
  const long long blocks = (long long)grid.x * grid.y * grid.z;
  const long long s3 = dt_slots<HD, 3>(), s2 = dt_slots<HD, 2>();
  const long long w3 = (blocks + s3 - 1) / s3, w2 = (blocks + s2 - 1) / s2;
  if (w2 * 115 < w3 * 100) return launch_dt2<HD, 2>(mk, mv, a, grid, cluster, stream);
  return launch_dt2<HD, 3>(mk, mv, a, grid, cluster, stream);
}

// qkv: [n_seqs, q_stride] bfloat16 rows with the raw query heads first, the key heads at element
// k_off and the value heads at v_off (all multiples of 8 elements).  The kernel rotates queries and
// the new key (rotary_dims = 0: none), writes the new key and value into the cache at tok_pos[b],
// attends and combines.  A block walks pages_per_block pages of 64 positions; n_splits blocks cover
// a sequence, so n_splits * pages_per_block * 64 must cover the longest sequence.  part_o / part_ml:
// scratch of n_seqs * n_heads * n_splits * head_dim and n_seqs * n_heads * n_splits * 2 floats (unused
// when n_splits is 1); tickets: n_seqs * n_kv_heads * ceil(group / 16) ints, zero before and after.
// The caches are [n_cache_pages, n_kv_heads, 64, head_dim], contiguous and 16-byte aligned.  status:
// one int on the device, left as it is unless a page load never completed (then 4, and the output
// of that launch is not valid).
//
// With items (n_items ints on the device, a multiple of group; group 1 to 8): block x of the grid
// works on what items[x] names, sequence | split << 16 | splits << 24, or on nothing (-1).  Clusters
// of `group` blocks run along x; a cluster must hold either the `group` splits of one sequence, in
// order, or sequences that are not split (splits = 1) and padding.  n_splits and pages_per_block
// are not used then.  This is how a batch of unequal lengths gets more blocks for its long
// sequences than for its short ones, and its long ones started first.
static int dt_run(const void* qkv, int q_stride, int k_off, int v_off, void* out, int out_stride,
                  int n_seqs, int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                  int rotary_dims, float theta_scale, const int* tok_pos, const int* slots,
                  const int* page_table, int pt_stride, void* k_cache, void* v_cache,
                  int n_cache_pages, int* status, float* part_o, float* part_ml, int n_splits, int pages_per_block, int* tickets,
                  int n_tickets, const int* items, int n_items, int item_group, cudaStream_t stream) {
  if (n_seqs <= 0) return BN_OK;
  if (items != nullptr) {
    if (n_items <= 0 || item_group < 1 || item_group > 8 || n_items % item_group || n_seqs > 65535) return BN_ERR_BAD_ARG;
    n_splits = item_group;
    pages_per_block = 1 << 20;
  }
  if (head_dim <= 0 || head_dim % 16 || head_dim > 256 || n_kv_heads <= 0 || n_heads % n_kv_heads || n_splits <= 0 ||
      pages_per_block <= 0 || window < 0 || !part_o || !part_ml || !tickets || !status || n_cache_pages <= 0 ||
      (((uintptr_t)k_cache | (uintptr_t)v_cache) & 15) || rotary_dims < 0 ||
      rotary_dims > head_dim || (rotary_dims & 1))
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
  a.status = status;
  BN_TRACE_ONLY(a.trace = nullptr;)
  BN_TRACE_ONLY(if (g_dt_trace && g_dt_trace_n < g_dt_trace_cap && n_splits <= 8) a.trace = g_dt_trace + (size_t)8 * 16 * (g_dt_trace_n++);)
  a.cluster = (n_splits > 1 && n_splits <= 8) ? 1 : 0;  // few splits: one cluster per (sequence, head group)
  a.pages_per_block = pages_per_block; a.tickets = tickets; a.out = (__nv_bfloat16*)out; a.out_stride = out_stride;
  a.items = items;
  dim3 grid(n_seqs, n_kv_heads * gblocks, n_splits), cluster(1, 1, n_splits);
  if (items != nullptr) {
    BN_TRACE_ONLY(a.trace = nullptr;)
    grid = dim3(n_items, n_kv_heads * gblocks, 1);
    cluster = dim3(item_group, 1, 1);
  }
  CUtensorMap mk, mv;
  if (!tma_map_bf16_pages(&mk, k_cache, n_cache_pages, (unsigned long long)n_kv_heads * BN_PAGE, head_dim, BN_PAGE) ||
      !tma_map_bf16_pages(&mv, v_cache, n_cache_pages, (unsigned long long)n_kv_heads * BN_PAGE, head_dim, BN_PAGE))
    return BN_ERR_BAD_ARG;
  if (head_dim <= 64) return launch_dt<64>(mk, mv, a, grid, cluster, stream);
  if (head_dim <= 128) return launch_dt<128>(mk, mv, a, grid, cluster, stream);
  return launch_dt<256>(mk, mv, a, grid, cluster, stream);
}
extern "C" int bn_attention_decode_tc(const void* qkv, int q_stride, int k_off, int v_off, void* out, int out_stride,
                                      int n_seqs, int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                      int rotary_dims, float theta_scale, const int* tok_pos, const int* slots,
                                      const int* page_table, int pt_stride, void* k_cache, void* v_cache,
                                      int n_cache_pages, int* status, float* part_o, float* part_ml, int n_splits, int pages_per_block, int* tickets,
                                      int n_tickets, cudaStream_t stream) {
  return dt_run(qkv, q_stride, k_off, v_off, out, out_stride, n_seqs, n_heads, n_kv_heads, head_dim, scale, window, rotary_dims,
                theta_scale, tok_pos, slots, page_table, pt_stride, k_cache, v_cache, n_cache_pages, status, part_o, part_ml,
                n_splits, pages_per_block, tickets, n_tickets, nullptr, 0, 0, stream);
}
extern "C" int bn_attention_decode_tc_items(const void* qkv, int q_stride, int k_off, int v_off, void* out, int out_stride,
                                            int n_seqs, int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                            int rotary_dims, float theta_scale, const int* tok_pos, const int* slots,
                                            const int* page_table, int pt_stride, void* k_cache, void* v_cache,
                                            int n_cache_pages, int* status, float* part_o, float* part_ml, int* tickets,
                                            int n_tickets, const int* items, int n_items, int item_group, cudaStream_t stream) {
  if (!items) return BN_ERR_BAD_ARG;
  return dt_run(qkv, q_stride, k_off, v_off, out, out_stride, n_seqs, n_heads, n_kv_heads, head_dim, scale, window, rotary_dims,
                theta_scale, tok_pos, slots, page_table, pt_stride, k_cache, v_cache, n_cache_pages, status, part_o, part_ml,
                1, 1, tickets, n_tickets, items, n_items, item_group, stream);
}
