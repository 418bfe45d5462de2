// Warp-level m16n8k16 tensor-core step (legacy mma.sync path) for f16 / bf16 operands with fp32 accumulation, and the
// helpers around it.  Fragment layout (g = lane / 4, t = lane % 4): A rows g, g+8, k = 2t, 2t+1, 2t+8, 2t+9;
// B (k x n) k = 2t, 2t+1, 2t+8, 2t+9, n = g; C rows g, g+8, columns 2t, 2t+1.
#pragma once
#include "psa_common.cuh"

namespace psa {

template <typename T> struct MmaOp;
template <> struct MmaOp<__half> {
  static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};
template <> struct MmaOp<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

// B fragment (16 k x 8 n) of a matrix stored [k][n] row-major in shared memory: `row_ptr` = this lane's row
// &M[k0 + (lane & 15)][n0] (16-byte aligned).
__device__ __forceinline__ void ldsm_x2_trans(uint32_t (&b)[2], const void* row_ptr) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(row_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b[0]), "=r"(b[1]) : "r"(a));
}

}  // namespace psa
