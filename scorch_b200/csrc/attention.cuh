// Shared by the sparse-attention kernels (attention.cu: 16x16 blocks on mma.sync; attention_band.cu:
// 128-row tiles of a band on tcgen05): the argument block, the TF32 split, and the launch of the
// scattered-entry kernel that both paths run first.
#pragma once

#include <math.h>

#include "common.cuh"

namespace sb {

struct AttnArgs {
  int m;
  int RB;
  const int* rb_ptr;
  const int* blk_col;
  const int* blk_ent;
  const int* blk_mask;
  const int* rem_pos;
  const float* mask_val;  // may be null
  const int* mask_is_ones; // device flag: every mask value is 1.0f (the mask values are then not read)
  const float* Q;
  const float* K;
  const float* V;
  float* O;
  float2* stats;          // [batch][m]: (running maximum in log2 units, sum) of each row's scattered entries
  int has_rem;            // the scattered-entry kernel ran: O and stats hold its results
  const int* rem_ent;     // entry index in the mask of each scattered entry (for its mask value)
  const int* rem_crd;     // its column
  unsigned ldq, ldk, ldv;
  long long ldo;
  long long stride_q, stride_k, stride_v, stride_o;
  float scale;
};

// x = hi + lo with both parts valid TF32 values (low 13 mantissa bits zero): hi is x truncated,
// lo the truncated remainder, so hi*hi + hi*lo + lo*hi misses the product by ~2^-20 relative.
// (Two logic operations and one subtraction; rounding instead of truncating measured slower
// and no more accurate at the fp32 level.)
__device__ __forceinline__ void attn_split(float x, unsigned& hi, unsigned& lo) {
  hi = __float_as_uint(x) & 0xffffe000u;
  lo = __float_as_uint(x - __uint_as_float(hi)) & 0xffffe000u;
}
// 2^x on the special-function unit (ex2.approx: 2 ulp; 2^-inf = 0)
__device__ __forceinline__ float attn_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 256-bit read-only load (32-byte aligned): one instruction covers whole 128-byte lines of the
// K / V rows, half the L1 wavefronts of 128-bit loads
struct Float8 { float v[8]; };
__device__ __forceinline__ Float8 ldg8(const float* p) {
  Float8 r;
  asm volatile("ld.global.nc.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]),
                 "=f"(r.v[6]), "=f"(r.v[7])
               : "l"(p));
  return r;
}


// Launches attn_scattered_kernel (attention.cu) over the plan's remaining entries and, when mask
// values are given, the kernels that set the "every mask value is 1" flag first.
int attn_launch_scattered(const AttnArgs& a, int64_t d, int64_t nnz, int64_t rem_nnz, int64_t batch,
                          int* flags, cudaStream_t st);

}  // namespace sb
