// Warp-level tiles for mma.sync.m16n8k16 (bfloat16 in, float32 out) read from shared memory with plain
// 4-byte loads: both operands lie row-major with the summed index innermost (A[m][k]; B transposed, Bt[n][k]).
// With rows padded by MMA_PAD elements (a row stride of 4 words modulo 32) a fragment load meets no bank twice.
#pragma once
#include "common.cuh"

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const bf16* row) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// rows r0..r0+15, columns k0..k0+15 of a row-major matrix in shared memory, as the A operand: one ldmatrix of
// four 8 x 8 pieces (rows 0-7 / 8-15 times columns 0-7 / 8-15; lane l names row l % 8 of piece l / 8).  Rows
// must start on 16-byte boundaries (ld and k0 multiples of 8).
__device__ __forceinline__ void load_a(uint32_t (&a)[4], const bf16* A, int ld, int r0, int k0, int lane) {
  const int piece = lane >> 3, r = lane & 7;
  ldmatrix_x4(a, A + (r0 + r + (piece & 1) * 8) * ld + k0 + (piece >> 1) * 8);
}
// the B operands of two neighbouring tiles of output columns, n0..n0+7 (b[0], b[1]) and n0+8..n0+15 (b[2], b[3]),
// from Bt[n][k] (the operand transposed, row-major), by one ldmatrix
__device__ __forceinline__ void load_b_pair(uint32_t (&b)[4], const bf16* Bt, int ld, int n0, int k0, int lane) {
  const int piece = lane >> 3, r = lane & 7;
  ldmatrix_x4(b, Bt + (n0 + r + (piece >> 1) * 8) * ld + k0 + (piece & 1) * 8);
}
// the B operand for output columns n0..n0+7 from Bt[n][k] (the operand transposed, row-major)
__device__ __forceinline__ void load_b(uint32_t& b0, uint32_t& b1, const bf16* Bt, int ld, int n0, int k0, int lane) {
  const bf16* p = Bt + (n0 + (lane >> 2)) * ld + k0 + 2 * (lane & 3);
  b0 = *reinterpret_cast<const uint32_t*>(p);
  b1 = *reinterpret_cast<const uint32_t*>(p + 8);
}
__device__ __forceinline__ void split_bf16(float x, bf16* hi, bf16* lo) {
  *hi = __float2bfloat16_rn(x);
  *lo = __float2bfloat16_rn(x - __bfloat162float(*hi));
}

