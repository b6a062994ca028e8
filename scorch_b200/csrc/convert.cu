// Device-side data-format plumbing either side of the sparse kernels, so that whole pipelines
// stay on the GPU:
//   * dense matrix -> CSR (what the reference's callers do with torch's to_sparse_csr(), e.g. the
//     pruned weight matrices of bench/bench_sparse_autoencoder.py:233,261): two phases because
//     the output size is data dependent — count (row pointers + total), then fill;
//   * symmetric normalisation of an adjacency pattern, val[p] = d_i^-1/2 d_j^-1/2 with d = stored
//     entries per row of A + I (bench/bench_gcn.py:233-267, there with torch scatter ops).
#include "common.cuh"

namespace sb {

constexpr int kConvWarps = 8;

// One warp per row: stored (non-zero) entries of the row.  -0.0 compares equal to zero and is
// dropped, NaN is kept: the semantics of torch.Tensor.to_sparse_csr().
__global__ void __launch_bounds__(kConvWarps * 32)
dense_count_kernel(int m, int n, const float* __restrict__ A, long long lda, int* __restrict__ cnt) {
  const int row = blockIdx.x * kConvWarps + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= m) return;
  const float* a = A + (long long)row * lda;
  int c = 0;
  for (int j = lane; j < n; j += 32) c += (ld_stream(a + j) != 0.f);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(FULL, c, o);
  if (lane == 0) cnt[row] = c;
}

// One warp per row: columns and values of the stored entries in ascending column order.
__global__ void __launch_bounds__(kConvWarps * 32)
dense_fill_kernel(int m, int n, const float* __restrict__ A, long long lda,
                  const int* __restrict__ pos, int* __restrict__ crd, float* __restrict__ val) {
  const int row = blockIdx.x * kConvWarps + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= m) return;
  const float* a = A + (long long)row * lda;
  int out = __ldg(pos + row);
  for (int j0 = 0; j0 < n; j0 += 32) {
    const int j = j0 + lane;
    const float v = j < n ? ld_stream(a + j) : 0.f;
    const bool keep = j < n && v != 0.f;
    const unsigned mask = __ballot_sync(FULL, keep);
    if (keep) {
      const int p = out + __popc(mask & ((1u << lane) - 1u));
      crd[p] = j;
      val[p] = v;
    }
    out += __popc(mask);
  }
}

// One warp per row of the pattern.
__global__ void __launch_bounds__(kConvWarps * 32)
sym_normalize_kernel(int m, const int* __restrict__ pos, const int* __restrict__ crd,
                     float* __restrict__ val) {
  const int row = blockIdx.x * kConvWarps + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= m) return;
  const int b = __ldg(pos + row), e = __ldg(pos + row + 1);
  const float di = e > b ? 1.0f / sqrtf((float)(e - b)) : 0.f;
  for (int p = b + lane; p < e; p += 32) {
    const int j = ld_stream(crd + p);
    const int dj = __ldg(pos + j + 1) - __ldg(pos + j);
    val[p] = di * (dj > 0 ? 1.0f / sqrtf((float)dj) : 0.f);
  }
}

}  // namespace sb

using namespace sb;

extern "C" {

size_t sb_dense_to_csr_workspace_bytes(int64_t m) {
  if (m < 0) m = 0;
  // row counts + scan temporaries (one int64 per 4096 rows + 1) + total
  return (size_t)(((m + 1) * 4 + 255) / 256 * 256) + (size_t)((ceil_div(m + 1, 4096) + 1) * 8 + 255) / 256 * 256 + 256;
}

int sb_dense_to_csr_count(int64_t m, int64_t n, const float* A, int64_t lda, int32_t* pos,
                          int64_t* nnz_host, void* ws, size_t ws_bytes, void* stream) {
  SB_CHECK_ARG(m >= 0 && n >= 0 && m < INT32_MAX && n < INT32_MAX, "dense_to_csr: bad size");
  SB_CHECK_ARG(pos && nnz_host, "dense_to_csr: null pos / nnz_host");
  SB_CHECK_ARG(m == 0 || n == 0 || A, "dense_to_csr: A is null");
  SB_CHECK_ARG(lda >= n, "dense_to_csr: leading dimension smaller than n");
  cudaStream_t st = (cudaStream_t)stream;
  *nnz_host = 0;
  if (m == 0) {
    SB_CUDA(cudaMemsetAsync(pos, 0, 4, st));
    SB_CUDA(cudaStreamSynchronize(st));
    return SB_OK;
  }
  const size_t need = sb_dense_to_csr_workspace_bytes(m);
  SB_CHECK_ARG(ws && aligned16(ws), "dense_to_csr: workspace is null or misaligned");
  if (ws_bytes < need)
    return fail(SB_ERR_WORKSPACE, "dense_to_csr: workspace has %zu bytes, needs %zu", ws_bytes, need);
  char* base = static_cast<char*>(ws);
  int* cnt = reinterpret_cast<int*>(base);
  const size_t off1 = (size_t)(((m + 1) * 4 + 255) / 256 * 256);
  long long* block_sum = reinterpret_cast<long long*>(base + off1);
  long long* total = reinterpret_cast<long long*>(base + need - 256);
  dense_count_kernel<<<(unsigned)ceil_div(m, kConvWarps), kConvWarps * 32, 0, st>>>((int)m, (int)n, A, lda, cnt);
  SB_LAUNCH_CHECK("dense_count_kernel");
  int rc = exclusive_scan_i32((int)m, cnt, pos, block_sum, total, st);
  if (rc != SB_OK) return rc;
  long long t = 0;
  SB_CUDA(cudaMemcpyAsync(&t, total, 8, cudaMemcpyDeviceToHost, st));
  SB_CUDA(cudaStreamSynchronize(st));
  if (t > INT32_MAX) return fail(SB_ERR_OVERFLOW, "dense_to_csr: %lld stored entries do not fit int32", t);
  *nnz_host = t;
  return SB_OK;
}

int sb_dense_to_csr_fill(int64_t m, int64_t n, const float* A, int64_t lda, const int32_t* pos,
                         int32_t* crd, float* val, void* stream) {
  SB_CHECK_ARG(m >= 0 && n >= 0 && m < INT32_MAX && n < INT32_MAX, "dense_to_csr: bad size");
  SB_CHECK_ARG(lda >= n, "dense_to_csr: leading dimension smaller than n");
  if (m == 0 || n == 0) return SB_OK;
  SB_CHECK_ARG(A && pos, "dense_to_csr: null A / pos");
  // (crd / val may be null only when the matrix has no stored entry: nothing is written then)
  dense_fill_kernel<<<(unsigned)ceil_div(m, kConvWarps), kConvWarps * 32, 0, (cudaStream_t)stream>>>(
      (int)m, (int)n, A, lda, pos, crd, val);
  SB_LAUNCH_CHECK("dense_fill_kernel");
  return SB_OK;
}

int sb_csr_sym_normalize_f32(int64_t m, int64_t nnz, const int32_t* pos, const int32_t* crd,
                             float* val, void* stream) {
  SB_CHECK_ARG(m >= 0 && nnz >= 0 && m < INT32_MAX, "sym_normalize: bad size");
  if (nnz > INT32_MAX) return fail(SB_ERR_OVERFLOW, "sym_normalize: nnz does not fit int32");
  if (m == 0 || nnz == 0) return SB_OK;
  SB_CHECK_ARG(pos && crd && val, "sym_normalize: null pointer");
  sym_normalize_kernel<<<(unsigned)ceil_div(m, kConvWarps), kConvWarps * 32, 0, (cudaStream_t)stream>>>(
      (int)m, pos, crd, val);
  SB_LAUNCH_CHECK("sym_normalize_kernel");
  return SB_OK;
}

}  // extern "C"
