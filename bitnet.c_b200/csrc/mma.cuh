// Warp-level tensor-core pieces shared by the kernels that use mma.sync (prefill attention with
// large heads, decode attention, the second small-batch product): the m16n8k16 bfloat16 MMA,
// ldmatrix, cp.async with zero fill, bfloat16 packing, and the rotary angle.
#pragma once
#include "common.cuh"

// D (16x8, float32) += A (16x16, bfloat16, row-major fragments a0..a3) . B (16x8, fragments b0, b1)
__device__ __forceinline__ void mma_bf16(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Four 8x8 matrices of 16-bit elements from shared memory (lane l gives the address of row l % 8 of
// matrix l / 8), as they are or transposed.
__device__ __forceinline__ void ldsm_x4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
// 16 bytes global -> shared, asynchronously; with valid == false the 16 bytes are zero-filled and
// nothing is read.
__device__ __forceinline__ void cp_async16(unsigned smem, const void* gmem, bool valid) {
  int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  cp_async16((unsigned)__cvta_generic_to_shared(smem), gmem, valid);
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

// The rotary angle of pair i at position pos: pos * theta_scale^i as a running float32 product
// (src/transformer.c:143-162).
__device__ __forceinline__ float rope_angle(int pos, int i, float theta_scale) {
  float angle = (float)pos;
  for (int k = 0; k < i; ++k) angle *= theta_scale;
  return angle;
}
