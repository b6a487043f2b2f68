// Tensor-memory-accelerator loads and the mbarriers they complete on, shared by the kernels that
// stream tiles from global memory (linear_tc.cu, attention_decode_tc.cu).
//
// Every wait is bounded in time: a wait that gives up records a code in a status word of the
// caller and returns false, so that the kernel can drain and return instead of spinning.
#pragma once
#include "common.cuh"
#include <cuda.h>
#include <cudaTypedefs.h>
#include <mutex>

#define TMA_WAIT_NS 2000000000ull  // two seconds

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
// The same, but the thread may stay suspended up to `ns` nanoseconds while the phase is incomplete
// (it is woken when the phase completes): a waiting thread then takes no issue slots from the
// warps that compute.
__device__ __forceinline__ bool mbar_try_wait_for(unsigned bar, unsigned parity, unsigned ns) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
  return ok != 0;
}
#define TMA_SUSPEND_NS 20000u
// Bounded wait: false (and *status set to code) when the phase did not complete within TMA_WAIT_NS.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = global_timer();
  for (;;) {
    if (mbar_try_wait_for(bar, parity, TMA_SUSPEND_NS)) return true;
    if (global_timer() - t0 > TMA_WAIT_NS) {
      atomicExch(status, code);
      return false;
    }
  }
}
// One box of a two-dimensional tensor map into shared memory; c0 is the coordinate along the
// contiguous dimension (c0 x element size must be a multiple of 16 bytes), c1 the row.
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, unsigned bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

static PFN_cuTensorMapEncodeTiled tma_encoder() {
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

// A [rows, cols] bfloat16 row-major matrix (row stride `cols` elements, a multiple of 8; base
// 16-byte aligned), loaded in boxes of box_rows x 64 elements with 128-byte swizzle: in shared
// memory a box is box_rows rows of 128 bytes, and the 16-byte chunk c of row r lies at chunk
// c ^ (r & 7) (the box must start on a 1024-byte boundary).  Rows and columns outside the matrix
// read as zero.
// The same with rows `row_stride` elements apart (a multiple of 8, at least cols).
static bool tma_map_bf16_strided(CUtensorMap* map, const void* ptr, unsigned long long rows, unsigned long long cols,
                                 unsigned long long row_stride, int box_rows);
static bool tma_map_bf16_rows(CUtensorMap* map, const void* ptr, unsigned long long rows, unsigned long long cols,
                              int box_rows) {
  return tma_map_bf16_strided(map, ptr, rows, cols, cols, box_rows);
}
// Encoded maps are kept: a map is a pure function of its arguments, weights and caches are
// described again at every launch, and the driver call that encodes one costs a microsecond or two
// of a launch that is otherwise ten.  A small direct-mapped table per library; a slot that holds
// another key is overwritten.
struct TmaMapSlot {
  bool used;
  int kind, box_rows;
  const void* ptr;
  unsigned long long a, b, c;
  CUtensorMap map;
};
#define TMA_MAP_SLOTS 1024
static TmaMapSlot g_tma_maps[TMA_MAP_SLOTS];
static std::mutex g_tma_maps_lock;
static unsigned tma_map_slot(int kind, const void* ptr, unsigned long long a, unsigned long long b, unsigned long long c,
                             int box_rows) {
  unsigned long long h = (unsigned long long)(uintptr_t)ptr * 0x9E3779B97F4A7C15ull;
  h ^= (a + 0x7F4A7C15ull) * 0xBF58476D1CE4E5B9ull;
  h ^= (b * 31 + c * 131 + (unsigned long long)box_rows * 7 + (unsigned long long)kind) * 0x94D049BB133111EBull;
  return (unsigned)(h >> 40) % TMA_MAP_SLOTS;
}
static bool tma_map_lookup(int kind, const void* ptr, unsigned long long a, unsigned long long b, unsigned long long c,
                           int box_rows, CUtensorMap* out) {
  std::lock_guard<std::mutex> hold(g_tma_maps_lock);
  const TmaMapSlot& s = g_tma_maps[tma_map_slot(kind, ptr, a, b, c, box_rows)];
  if (!s.used || s.kind != kind || s.ptr != ptr || s.a != a || s.b != b || s.c != c || s.box_rows != box_rows) return false;
  *out = s.map;
  return true;
}
static void tma_map_keep(int kind, const void* ptr, unsigned long long a, unsigned long long b, unsigned long long c,
                         int box_rows, const CUtensorMap* map) {
  std::lock_guard<std::mutex> hold(g_tma_maps_lock);
  TmaMapSlot& s = g_tma_maps[tma_map_slot(kind, ptr, a, b, c, box_rows)];
  s.used = true; s.kind = kind; s.ptr = ptr; s.a = a; s.b = b; s.c = c; s.box_rows = box_rows; s.map = *map;
}

static bool tma_map_bf16_strided(CUtensorMap* map, const void* ptr, unsigned long long rows, unsigned long long cols,
                                 unsigned long long row_stride, int box_rows) {
  if (tma_map_lookup(0, ptr, rows, cols, row_stride, box_rows, map)) return true;
  PFN_cuTensorMapEncodeTiled enc = tma_encoder();
  if (!enc) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  if (enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  tma_map_keep(0, ptr, rows, cols, row_stride, box_rows, map);
  return true;
}

__device__ __forceinline__ void tma_load_3d(unsigned dst, const CUtensorMap* map, unsigned bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

// A paged bfloat16 tensor [pages, rows_per_page, cols] (contiguous; cols a multiple of 8; base
// 16-byte aligned), loaded in boxes of box_rows x 64 elements of one page with 128-byte swizzle
// (layout in shared memory as for tma_map_bf16_rows).  Coordinates: (column, row in page, page).
static bool tma_map_bf16_pages(CUtensorMap* map, const void* ptr, unsigned long long pages,
                               unsigned long long rows_per_page, unsigned long long cols, int box_rows) {
  if (tma_map_lookup(1, ptr, pages, rows_per_page, cols, box_rows, map)) return true;
  PFN_cuTensorMapEncodeTiled enc = tma_encoder();
  if (!enc) return false;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows_per_page, (cuuint64_t)pages};
  cuuint64_t strides[2] = {(cuuint64_t)cols * 2, (cuuint64_t)rows_per_page * cols * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  if (enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  tma_map_keep(1, ptr, pages, rows_per_page, cols, box_rows, map);
  return true;
}
