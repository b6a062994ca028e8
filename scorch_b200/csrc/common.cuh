// Shared helpers of the sm_100a sparse kernels: status/error plumbing, cache-hinted loads,
// warp-level primitives.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "scorch_b200.h"

namespace sb {

// ---- error plumbing -----------------------------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int status, const char* fmt, ...);

#define SB_CHECK_ARG(cond, ...)                                   \
  do {                                                            \
    if (!(cond)) return ::sb::fail(SB_ERR_INVALID_ARG, __VA_ARGS__); \
  } while (0)

#define SB_CUDA(call)                                                                   \
  do {                                                                                  \
    cudaError_t e__ = (call);                                                           \
    if (e__ != cudaSuccess)                                                             \
      return ::sb::fail(SB_ERR_CUDA, "%s failed: %s (%s:%d)", #call,                    \
                        cudaGetErrorString(e__), __FILE__, __LINE__);                   \
  } while (0)

#define SB_LAUNCH_CHECK(name)                                                           \
  do {                                                                                  \
    cudaError_t e__ = cudaGetLastError();                                               \
    if (e__ != cudaSuccess)                                                             \
      return ::sb::fail(SB_ERR_CUDA, "launch of %s failed: %s", name,                   \
                        cudaGetErrorString(e__));                                       \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Number of SMs of the current device (148 on B200), cached per process.
int sm_count();

// ---- row plan layout (see include/scorch_b200.h) --------------------------------------------
// int32 words:  [0] heavy rows  [1] segments  [2] capacity heavy  [3] capacity segments
//               [4..7] reserved
//   heavy_row[cap_heavy]      row id of each heavy row
//   heavy_seg0[cap_heavy]     first segment slot of the row
//   heavy_nseg[cap_heavy]     segments of the row
//   seg_heavy[cap_seg]        heavy-row slot a segment belongs to
struct PlanView {
  const int* hdr;
  const int* heavy_row;
  const int* heavy_seg0;
  const int* heavy_nseg;
  const int* seg_heavy;
  int cap_heavy;
  int cap_seg;
};
int64_t plan_cap_heavy(int64_t nnz);
int64_t plan_cap_seg(int64_t nnz);
PlanView plan_view(const void* plan, int64_t nnz);

// Exclusive scan of n int counts into out[0..n]; total (int64) at *total_dev; block_sum holds
// ceil(n / 4096) + 1 int64 temporaries.  Defined in spgemm.cu.
int exclusive_scan_i32(int n, const int* cnt, int* out, long long* block_sum, long long* total_dev,
                       cudaStream_t st);

// Gather kernels over the entries that a block plan leaves outside its blocks (sddmm.cu /
// spmm.cu): entries are taken through the list `rem_ent`, rows described by `rem_pos`.
// out_compact: `crd` and the results are indexed by position in the list (the list then only
// locates the mask values); val_compact: so are the values.  `rem_ent` may be null when the
// arrays it would index are compact or absent.
int sddmm_remainder(int64_t m, int64_t d, int64_t rem_nnz, const int* rem_pos, const int* rem_ent,
                    const int* crd, const float* mask_val, const float* Q, int64_t ldq,
                    const float* K, int64_t ldk, float* out, int64_t batch, int64_t stride_q,
                    int64_t stride_k, int64_t stride_out, int out_compact, cudaStream_t st);
int spmm_remainder(int64_t m, int64_t k, const int* rem_pos, const int* rem_ent, const int* crd,
                   const float* val, const float* B, int64_t ldb, const float* bias, int relu,
                   float* C, int64_t ldc, int64_t batch, int64_t stride_val, int64_t stride_b,
                   int64_t stride_c, int val_compact, cudaStream_t st);

// SpMM over wide dense operands with the operand rows staged through shared memory by bulk
// copies (spmm_wide.cu); `spmm_wide_wanted` tells whether that kernel is selected.
bool spmm_wide_wanted();
int spmm_wide_launch(int64_t m, int64_t k, const int* pos, const int* crd, const float* val, const float* B,
                     int64_t ldb, const float* bias, int relu, float* C, int64_t ldc, cudaStream_t st);

// ---- device helpers ------------------------------------------------------------------------
#ifdef __CUDACC__

constexpr unsigned FULL = 0xffffffffu;

// Read-only, L1-allocating 128-bit gather of a dense operand row (B / Q / K / V).
__device__ __forceinline__ float4 ldg4(const float* p) {
  return __ldg(reinterpret_cast<const float4*>(p));
}
// Streaming loads of the CSR arrays: read once, do not keep in L1.
__device__ __forceinline__ int ld_stream(const int* p) {
  int v;
  asm volatile("ld.global.nc.L1::no_allocate.s32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_stream(const float* p) {
  float v;
  asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
// Streaming (evict-first) 128-bit store of an output row: written once, never re-read here.
__device__ __forceinline__ void st_stream4(float* p, float4 v) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

__device__ __forceinline__ void fma4(float4& acc, float a, const float4& b) {
  acc.x = fmaf(a, b.x, acc.x);
  acc.y = fmaf(a, b.y, acc.y);
  acc.z = fmaf(a, b.z, acc.z);
  acc.w = fmaf(a, b.w, acc.w);
}
__device__ __forceinline__ float dot4(const float4& a, const float4& b, float acc) {
  acc = fmaf(a.x, b.x, acc);
  acc = fmaf(a.y, b.y, acc);
  acc = fmaf(a.z, b.z, acc);
  acc = fmaf(a.w, b.w, acc);
  return acc;
}

template <int WIDTH>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = WIDTH / 2; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
  return v;
}
template <int WIDTH>
__device__ __forceinline__ float group_max(float v) {
#pragma unroll
  for (int o = WIDTH / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL, v, o));
  return v;
}

// Row containing entry p: largest r in [lo, hi) with pos[r] <= p  (pos ascending, pos[hi] > p).
__device__ __forceinline__ int row_of_entry(const int* __restrict__ pos, int lo, int hi, int p) {
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(pos + mid) <= p) lo = mid; else hi = mid;
  }
  return lo;
}

#endif  // __CUDACC__

}  // namespace sb
