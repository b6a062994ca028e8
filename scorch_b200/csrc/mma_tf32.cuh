// TF32 tensor-core helpers shared by the dense-block kernels: mma.sync m16n8k8 with the 3xTF32
// split (x = hi + lo; hi*hi + hi*lo + lo*hi, fp32 accumulate), which keeps fp32-level accuracy.
// Fragment layout of mma.m16n8k8 (g = lane/4, t = lane%4): A rows g, g+8 / k columns t, t+4;
// B k rows t, t+4 / column g; C rows g, g+8 / columns 2t, 2t+1.
#pragma once

namespace sb {

__device__ __forceinline__ void split_tf32(float x, unsigned& hi, unsigned& lo) {
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
  const float r = x - __uint_as_float(hi);
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(r));
}

__device__ __forceinline__ void mma_tf32(float (&c)[4], const unsigned (&a)[4], unsigned b0,
                                         unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// c += a * b with fp32-level accuracy: small cross terms first, then the main term.
__device__ __forceinline__ void mma_3xtf32(float (&c)[4], const unsigned (&ahi)[4],
                                           const unsigned (&alo)[4], unsigned bhi0, unsigned bhi1,
                                           unsigned blo0, unsigned blo1) {
  mma_tf32(c, alo, bhi0, bhi1);
  mma_tf32(c, ahi, blo0, blo1);
  mma_tf32(c, ahi, bhi0, bhi1);
}

}  // namespace sb
