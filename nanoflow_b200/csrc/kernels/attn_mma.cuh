// Warp-level building blocks shared by the mma.sync attention kernels (attention.cu, attention_dec.cu):
// cp.async, ldmatrix, the bf16 m16n8k16 MMA, quad reductions of the softmax state and the Q fragment
// loader.
#pragma once
#include "common.cuh"

namespace nf {

constexpr int kPage = 16;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                              uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Q fragment loader: rows of the 16-row tile come from `row_ptr(r)` (nullptr => zero row).
template <int HD, class RowPtr>
__device__ __forceinline__ void load_q_frags(uint32_t (&qa)[HD / 16][4], RowPtr row_ptr) {
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* r0 = row_ptr(lane >> 2);
  const __nv_bfloat16* r1 = row_ptr((lane >> 2) + 8);
  const int c = (lane & 3) * 2;
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    qa[ks][0] = r0 ? *reinterpret_cast<const uint32_t*>(r0 + ks * 16 + c) : 0u;
    qa[ks][1] = r1 ? *reinterpret_cast<const uint32_t*>(r1 + ks * 16 + c) : 0u;
    qa[ks][2] = r0 ? *reinterpret_cast<const uint32_t*>(r0 + ks * 16 + c + 8) : 0u;
    qa[ks][3] = r1 ? *reinterpret_cast<const uint32_t*>(r1 + ks * 16 + c + 8) : 0u;
  }
}

}  // namespace nf
