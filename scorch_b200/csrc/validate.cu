// CSR input validation on the device: the checks a bounds-checking tool would make on the
// kernels' index arithmetic, done once on the inputs instead of inside the hot loops.  The
// kernels of this library trust their inputs (like the reference's loops, csrc/spmm.h:2035-2077:
// no check of crd against the operand's height); a row pointer that runs backwards or a column
// index out of range makes them read or write outside their arrays.  sb_csr_validate finds the
// first such entry without touching anything outside pos[0..m] and crd[0..nnz): row pointers
// first (every later read is bounded by them), then the columns of every row.
#include "common.cuh"

namespace sb {

// Every violation proposes the key (row << 32 | entry); the smallest key wins (atomicMin), so the
// entry that is reported does not depend on scheduling.  The host reads the arrays at that
// place again to name the violation.
__global__ void validate_pos_kernel(int m, long long nnz, const int* __restrict__ pos, unsigned long long* key) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i > m) return;
  const int p = pos[i];
  const bool bad = (i == 0 && p != 0) || (i == m && (long long)p != nnz) || p < 0 || (long long)p > nnz ||
                   (i < m && pos[i + 1] < p);
  if (bad) atomicMin(key, (unsigned long long)(unsigned)i << 32);
}

// one warp per row (row pointers are known to be valid here)
__global__ void validate_crd_kernel(int m, int n, const int* __restrict__ pos, const int* __restrict__ crd,
                                    int sorted_unique, unsigned long long* key) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= m) return;
  const int b = pos[row], e = pos[row + 1];
  for (int p = b + lane; p < e; p += 32) {
    const int c = crd[p];
    if (c < 0 || c >= n || (sorted_unique && p > b && crd[p - 1] >= c))
      atomicMin(key, ((unsigned long long)(unsigned)row << 32) | (unsigned)p);
  }
}

}  // namespace sb

using namespace sb;

extern "C" {

size_t sb_csr_validate_workspace_bytes(void) { return 32; }

int sb_csr_validate(int64_t m, int64_t n, int64_t nnz, const int32_t* pos, const int32_t* crd,
                    int sorted_unique, int32_t* report_host, void* ws, size_t ws_bytes, void* stream) {
  SB_CHECK_ARG(m >= 0 && n >= 0 && nnz >= 0 && m < INT32_MAX && n <= INT32_MAX && nnz <= INT32_MAX,
               "csr_validate: bad size");
  SB_CHECK_ARG(pos && report_host && (crd || nnz == 0), "csr_validate: null pointer");
  SB_CHECK_ARG(ws && aligned16(ws) && ws_bytes >= sb_csr_validate_workspace_bytes(),
               "csr_validate: workspace is null, misaligned or smaller than 32 bytes");
  cudaStream_t st = (cudaStream_t)stream;
  unsigned long long* key = static_cast<unsigned long long*>(ws);
  unsigned long long k = 0;
  report_host[0] = report_host[1] = report_host[2] = report_host[3] = 0;
  SB_CUDA(cudaMemsetAsync(key, 0xff, 8, st));
  validate_pos_kernel<<<(unsigned)ceil_div(m + 1, 256), 256, 0, st>>>((int)m, nnz, pos, key);
  SB_LAUNCH_CHECK("validate_pos_kernel");
  SB_CUDA(cudaMemcpyAsync(&k, key, 8, cudaMemcpyDeviceToHost, st));
  SB_CUDA(cudaStreamSynchronize(st));
  if (k != ~0ull) {
    const int64_t i = (int64_t)(k >> 32);
    int32_t pair[2] = {0, 0};
    SB_CUDA(cudaMemcpyAsync(pair, pos + i, i < m ? 8 : 4, cudaMemcpyDeviceToHost, st));
    SB_CUDA(cudaStreamSynchronize(st));
    const int32_t p = pair[0];
    report_host[1] = (int32_t)i;
    report_host[3] = p;
    if (i == 0 && p != 0) report_host[0] = SB_CSR_BAD_FIRST_POS;
    else if (p < 0 || (int64_t)p > nnz) report_host[0] = SB_CSR_POS_OUT_OF_RANGE;
    else if (i == m) report_host[0] = SB_CSR_BAD_LAST_POS;
    else { report_host[0] = SB_CSR_POS_DECREASES; report_host[3] = pair[1]; }
    return SB_OK;
  }
  if (m == 0 || nnz == 0) return SB_OK;
  validate_crd_kernel<<<(unsigned)ceil_div(m, 8), 256, 0, st>>>((int)m, (int)n, pos, crd, sorted_unique, key);
  SB_LAUNCH_CHECK("validate_crd_kernel");
  SB_CUDA(cudaMemcpyAsync(&k, key, 8, cudaMemcpyDeviceToHost, st));
  SB_CUDA(cudaStreamSynchronize(st));
  if (k != ~0ull) {
    const int64_t row = (int64_t)(k >> 32), p = (int64_t)(k & 0xffffffffull);
    int32_t c = 0;
    SB_CUDA(cudaMemcpyAsync(&c, crd + p, 4, cudaMemcpyDeviceToHost, st));
    SB_CUDA(cudaStreamSynchronize(st));
    report_host[0] = (c < 0 || (int64_t)c >= n) ? SB_CSR_COLUMN_OUT_OF_RANGE : SB_CSR_COLUMNS_NOT_ASCENDING;
    report_host[1] = (int32_t)row;
    report_host[2] = (int32_t)p;
    report_host[3] = c;
  }
  return SB_OK;
}

}  // extern "C"
