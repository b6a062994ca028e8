// CSR SpMV for sm_100a.
//
// Rows up to SB_HEAVY_ROW_NNZ entries: G lanes per row (G chosen from the mean row length, so a
// warp covers 32/G rows and its loads of crd/val stay contiguous), shuffle-tree sum.
// Heavier rows: one CTA per plan segment, block-wide fixed-order sum, then a fixed-order add of
// the segment sums.  x is gathered through the read-only path (it is L2 resident: 8 MB for 2M
// columns); the CSR streams are read once with no-allocate loads.
#include "common.cuh"

namespace sb {

template <typename T>
__device__ __forceinline__ T shfl_xor_t(T v, int o) { return __shfl_xor_sync(FULL, v, o); }

template <typename T, int G>
__global__ void __launch_bounds__(256)
spmv_rows_kernel(int m, const int* __restrict__ pos, const int* __restrict__ crd,
                 const T* __restrict__ val, const T* __restrict__ x, T* __restrict__ y,
                 int skip_heavy) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = t / G;
  const int l = (int)(t % G);
  T acc = T(0);
  bool write = false;
  if (row < m) {
    const int b = __ldg(pos + row), e = __ldg(pos + row + 1);
    if (!(skip_heavy && e - b > SB_HEAVY_ROW_NNZ)) {
      write = true;
      for (int p = b + l; p < e; p += G) acc += val[p] * __ldg(x + crd[p]);
    }
  }
#pragma unroll
  for (int o = G / 2; o > 0; o >>= 1) acc += shfl_xor_t(acc, o);
  if (write && l == 0) y[row] = acc;
}

struct SpmvHeavy {
  const int* hdr;
  const int* heavy_row;
  const int* heavy_seg0;
  const int* heavy_nseg;
  const int* seg_heavy;
  float* scratch;
};

__global__ void __launch_bounds__(256)
spmv_heavy_kernel(const int* __restrict__ pos, const int* __restrict__ crd,
                  const float* __restrict__ val, const float* __restrict__ x,
                  float* __restrict__ y, SpmvHeavy h) {
  __shared__ float part[8];
  const int seg = blockIdx.x;
  if (seg >= __ldg(h.hdr + 1)) return;
  const int slot = __ldg(h.seg_heavy + seg);
  const int row = __ldg(h.heavy_row + slot);
  const int seg0 = __ldg(h.heavy_seg0 + slot);
  const int nseg = __ldg(h.heavy_nseg + slot);
  const int rb = __ldg(pos + row), re = __ldg(pos + row + 1);
  const int b = rb + (seg - seg0) * SB_HEAVY_ROW_NNZ;
  const int e = min(re, b + SB_HEAVY_ROW_NNZ);
  float acc = 0.f;
  for (int p = b + threadIdx.x; p < e; p += 256)
    acc = fmaf(ld_stream(val + p), __ldg(x + ld_stream(crd + p)), acc);
  acc = group_sum<32>(acc);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = part[0];
#pragma unroll
    for (int w = 1; w < 8; w++) s += part[w];
    if (nseg == 1) y[row] = s; else h.scratch[seg] = s;
  }
}

__global__ void spmv_heavy_finalize_kernel(float* __restrict__ y, SpmvHeavy h, int bound) {
  const int slot = blockIdx.x * blockDim.x + threadIdx.x;
  if (slot >= bound || slot >= __ldg(h.hdr)) return;
  const int nseg = __ldg(h.heavy_nseg + slot);
  if (nseg == 1) return;
  const int seg0 = __ldg(h.heavy_seg0 + slot);
  float s = 0.f;
  for (int t = 0; t < nseg; t++) s += h.scratch[seg0 + t];
  y[__ldg(h.heavy_row + slot)] = s;
}

template <typename T>
static int launch_rows(int64_t m, int64_t nnz, const int32_t* pos, const int32_t* crd,
                       const T* val, const T* x, T* y, int skip_heavy, cudaStream_t st) {
  const double mean = m > 0 ? (double)nnz / (double)m : 0.0;
  const int threads = 256;
#define SB_SPMV_LAUNCH(G)                                                                    \
  spmv_rows_kernel<T, G><<<(unsigned)ceil_div(m * (int64_t)G, threads), threads, 0, st>>>(   \
      (int)m, pos, crd, val, x, y, skip_heavy)
  if (mean <= 3.0) SB_SPMV_LAUNCH(2);
  else if (mean <= 6.0) SB_SPMV_LAUNCH(4);
  else if (mean <= 12.0) SB_SPMV_LAUNCH(8);
  else if (mean <= 48.0) SB_SPMV_LAUNCH(16);
  else SB_SPMV_LAUNCH(32);
#undef SB_SPMV_LAUNCH
  SB_LAUNCH_CHECK("spmv_rows_kernel");
  return SB_OK;
}

static int check_spmv(int64_t m, int64_t n, int64_t nnz, const void* pos, const void* crd,
                      const void* val, const void* x, const void* y) {
  SB_CHECK_ARG(m >= 0 && n >= 0 && nnz >= 0, "spmv: negative size");
  SB_CHECK_ARG(m < INT32_MAX / 32 * 32 && n < INT32_MAX, "spmv: dimension exceeds int32");
  if (nnz > INT32_MAX) return fail(SB_ERR_OVERFLOW, "spmv: nnz does not fit int32 row pointers");
  SB_CHECK_ARG(pos, "spmv: pos is null");
  SB_CHECK_ARG(nnz == 0 || (crd && val && x), "spmv: null crd/val/x");
  SB_CHECK_ARG(m == 0 || y, "spmv: y is null");
  return SB_OK;
}

}  // namespace sb

using namespace sb;

extern "C" {

size_t sb_spmv_csr_scratch_bytes(int64_t segments) {
  return segments > 0 ? (size_t)segments * sizeof(float) : 0;
}

int sb_spmv_csr_f32(int64_t m, int64_t n, int64_t nnz, const int32_t* pos, const int32_t* crd,
                    const float* val, const float* x, float* y, const void* plan,
                    int64_t plan_segments, void* scratch, size_t scratch_bytes, void* stream) {
  int rc = check_spmv(m, n, nnz, pos, crd, val, x, y);
  if (rc != SB_OK) return rc;
  if (m == 0) return SB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool heavy = plan && plan_segments != 0;
  if (heavy) {
    SB_CHECK_ARG(aligned16(plan), "spmv: plan must be 16-byte aligned");
    const int64_t segs = plan_segments < 0 ? plan_cap_seg(nnz) : plan_segments;
    SB_CHECK_ARG(scratch, "spmv: scratch is null");
    if (scratch_bytes < sb_spmv_csr_scratch_bytes(segs))
      return fail(SB_ERR_WORKSPACE, "spmv: scratch has %zu bytes, needs %zu", scratch_bytes,
                  sb_spmv_csr_scratch_bytes(segs));
  }
  rc = launch_rows<float>(m, nnz, pos, crd, val, x, y, heavy ? 1 : 0, st);
  if (rc != SB_OK) return rc;
  if (heavy) {
    PlanView pv = plan_view(plan, nnz);
    const int64_t segs = plan_segments < 0 ? pv.cap_seg : plan_segments;
    SpmvHeavy h{pv.hdr, pv.heavy_row, pv.heavy_seg0, pv.heavy_nseg, pv.seg_heavy,
                static_cast<float*>(scratch)};
    spmv_heavy_kernel<<<(unsigned)segs, 256, 0, st>>>(pos, crd, val, x, y, h);
    SB_LAUNCH_CHECK("spmv_heavy_kernel");
    const int bound = (int)(segs < pv.cap_heavy ? segs : pv.cap_heavy);
    spmv_heavy_finalize_kernel<<<(unsigned)ceil_div(bound, 128), 128, 0, st>>>(y, h, bound);
    SB_LAUNCH_CHECK("spmv_heavy_finalize_kernel");
  }
  return SB_OK;
}

int sb_spmv_csr_typed(int dtype, int64_t m, int64_t n, int64_t nnz, const int32_t* pos,
                      const int32_t* crd, const void* val, const void* x, void* y, void* stream) {
  int rc = check_spmv(m, n, nnz, pos, crd, val, x, y);
  if (rc != SB_OK) return rc;
  if (m == 0) return SB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case SB_F32:
      return launch_rows<float>(m, nnz, pos, crd, (const float*)val, (const float*)x, (float*)y, 0, st);
    case SB_F64:
      return launch_rows<double>(m, nnz, pos, crd, (const double*)val, (const double*)x, (double*)y, 0, st);
    case SB_I32:  // unsigned arithmetic: same bits as the reference's wrapping int32 math
      return launch_rows<unsigned int>(m, nnz, pos, crd, (const unsigned int*)val,
                                       (const unsigned int*)x, (unsigned int*)y, 0, st);
    case SB_I64:
      return launch_rows<unsigned long long>(m, nnz, pos, crd, (const unsigned long long*)val,
                                             (const unsigned long long*)x, (unsigned long long*)y, 0, st);
    default:
      return fail(SB_ERR_UNSUPPORTED, "spmv_typed: unknown dtype %d", dtype);
  }
}

}  // extern "C"
