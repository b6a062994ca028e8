// Status plumbing, the heavy-row plan, nnz-balanced row partition and CSR<->COO row plumbing.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace sb {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return status;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// A row is heavy when it holds more than SB_HEAVY_ROW_NNZ entries, so there are fewer than
// nnz / SB_HEAVY_ROW_NNZ heavy rows, and at most nnz / SB_HEAVY_ROW_NNZ + (heavy rows) segments.
int64_t plan_cap_heavy(int64_t nnz) { return nnz / SB_HEAVY_ROW_NNZ + 1; }
int64_t plan_cap_seg(int64_t nnz) { return nnz / SB_HEAVY_ROW_NNZ + plan_cap_heavy(nnz); }

PlanView plan_view(const void* plan, int64_t nnz) {
  PlanView v;
  const int* w = static_cast<const int*>(plan);
  v.cap_heavy = (int)plan_cap_heavy(nnz);
  v.cap_seg = (int)plan_cap_seg(nnz);
  v.hdr = w;
  v.heavy_row = w + 8;
  v.heavy_seg0 = v.heavy_row + v.cap_heavy;
  v.heavy_nseg = v.heavy_seg0 + v.cap_heavy;
  v.seg_heavy = v.heavy_nseg + v.cap_heavy;
  return v;
}

__global__ void plan_build_kernel(int m, const int* __restrict__ pos, int* hdr, int* heavy_row,
                                  int* heavy_seg0, int* heavy_nseg, int* seg_heavy, int cap_heavy,
                                  int cap_seg) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= m) return;
  const int len = pos[i + 1] - pos[i];
  if (len <= SB_HEAVY_ROW_NNZ) return;
  const int nseg = (len + SB_HEAVY_ROW_NNZ - 1) / SB_HEAVY_ROW_NNZ;
  const int slot = atomicAdd(&hdr[0], 1);
  const int seg0 = atomicAdd(&hdr[1], nseg);
  if (slot >= cap_heavy || seg0 + nseg > cap_seg) return;  // cannot happen for a valid pos[]
  heavy_row[slot] = i;
  heavy_seg0[slot] = seg0;
  heavy_nseg[slot] = nseg;
  for (int s = 0; s < nseg; s++) seg_heavy[seg0 + s] = slot;
}

__global__ void partition_kernel(int m, const int* __restrict__ pos, int parts, long long* out) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g > parts) return;
  if (g == parts) { out[g] = m; return; }
  const long long nnz = pos[m];
  const long long target = (nnz * g) / parts;
  // first row r with pos[r] >= target
  int lo = 0, hi = m;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if ((long long)pos[mid] < target) lo = mid + 1; else hi = mid;
  }
  out[g] = lo;
}

// pos[r] = first entry p with row[p] >= r  (row sorted ascending)
__global__ void coo_to_pos_kernel(int m, long long nnz, const int* __restrict__ row, int* pos) {
  const long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (p > nnz) return;
  const int prev = (p == 0) ? -1 : row[p - 1];
  const int cur = (p == nnz) ? m : row[p];
  for (int r = prev + 1; r <= cur; r++) pos[r] = (int)p;
}

__global__ void pos_to_rows_kernel(int m, const int* __restrict__ pos, int* row) {
  // one warp per CSR row
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= m) return;
  const int b = pos[w], e = pos[w + 1];
  for (int p = b + lane; p < e; p += 32) row[p] = w;
}

}  // namespace sb

using namespace sb;

extern "C" {

int sb_abi_version(void) { return 1; }

const char* sb_status_string(int s) {
  switch (s) {
    case SB_OK: return "ok";
    case SB_ERR_INVALID_ARG: return "invalid argument";
    case SB_ERR_CUDA: return "CUDA error";
    case SB_ERR_OVERFLOW: return "int32 overflow";
    case SB_ERR_WORKSPACE: return "workspace too small";
    case SB_ERR_UNSUPPORTED: return "unsupported";
    default: return "unknown status";
  }
}

const char* sb_last_error(void) { return sb::g_err; }

size_t sb_csr_plan_bytes(int64_t m, int64_t nnz) {
  (void)m;
  if (nnz < 0) nnz = 0;
  const int64_t words = 8 + 3 * plan_cap_heavy(nnz) + plan_cap_seg(nnz);
  return (size_t)((words * 4 + 255) / 256 * 256);
}

int64_t sb_csr_plan_max_segments(int64_t nnz) { return plan_cap_seg(nnz < 0 ? 0 : nnz); }

int sb_csr_plan_build(int64_t m, int64_t nnz, const int32_t* pos, void* plan, size_t plan_bytes,
                      void* stream) {
  SB_CHECK_ARG(m >= 0 && nnz >= 0, "plan_build: negative size");
  SB_CHECK_ARG(m < INT32_MAX && nnz <= INT32_MAX, "plan_build: m or nnz exceeds int32");
  SB_CHECK_ARG(pos && plan, "plan_build: null pointer");
  SB_CHECK_ARG(aligned16(plan), "plan_build: plan must be 16-byte aligned");
  if (plan_bytes < sb_csr_plan_bytes(m, nnz))
    return fail(SB_ERR_WORKSPACE, "plan_build: plan buffer has %zu bytes, needs %zu", plan_bytes,
                sb_csr_plan_bytes(m, nnz));
  cudaStream_t st = (cudaStream_t)stream;
  PlanView v = plan_view(plan, nnz);
  int* w = static_cast<int*>(plan);
  SB_CUDA(cudaMemsetAsync(w, 0, 32, st));
  if (m > 0) {
    const int threads = 256;
    plan_build_kernel<<<(unsigned)ceil_div(m, threads), threads, 0, st>>>(
        (int)m, pos, w, const_cast<int*>(v.heavy_row), const_cast<int*>(v.heavy_seg0),
        const_cast<int*>(v.heavy_nseg), const_cast<int*>(v.seg_heavy), v.cap_heavy, v.cap_seg);
    SB_LAUNCH_CHECK("plan_build_kernel");
  }
  return SB_OK;
}

int sb_csr_plan_counts(const void* plan, int64_t* heavy_rows_host, int64_t* segments_host,
                       void* stream) {
  SB_CHECK_ARG(plan, "plan_counts: null plan");
  int h[2] = {0, 0};
  cudaStream_t st = (cudaStream_t)stream;
  SB_CUDA(cudaMemcpyAsync(h, plan, sizeof(h), cudaMemcpyDeviceToHost, st));
  SB_CUDA(cudaStreamSynchronize(st));
  if (heavy_rows_host) *heavy_rows_host = h[0];
  if (segments_host) *segments_host = h[1];
  return SB_OK;
}

int sb_partition_rows_by_nnz(int64_t m, const int32_t* pos, int parts, int64_t* bounds,
                             void* stream) {
  SB_CHECK_ARG(m >= 0 && m < INT32_MAX, "partition: bad m");
  SB_CHECK_ARG(parts >= 1 && parts <= 4096, "partition: parts must be in [1, 4096]");
  SB_CHECK_ARG(pos && bounds, "partition: null pointer");
  partition_kernel<<<(unsigned)ceil_div(parts + 1, 128), 128, 0, (cudaStream_t)stream>>>(
      (int)m, pos, parts, reinterpret_cast<long long*>(bounds));
  SB_LAUNCH_CHECK("partition_kernel");
  return SB_OK;
}

int sb_coo_rows_to_csr_pos(int64_t m, int64_t nnz, const int32_t* row_sorted, int32_t* pos,
                           void* stream) {
  SB_CHECK_ARG(m >= 0 && m < INT32_MAX && nnz >= 0 && nnz <= INT32_MAX, "coo_to_pos: bad size");
  SB_CHECK_ARG(pos && (row_sorted || nnz == 0), "coo_to_pos: null pointer");
  const int threads = 256;
  coo_to_pos_kernel<<<(unsigned)ceil_div(nnz + 1, threads), threads, 0, (cudaStream_t)stream>>>(
      (int)m, (long long)nnz, row_sorted, pos);
  SB_LAUNCH_CHECK("coo_to_pos_kernel");
  return SB_OK;
}

int sb_csr_pos_to_coo_rows(int64_t m, int64_t nnz, const int32_t* pos, int32_t* row,
                           void* stream) {
  SB_CHECK_ARG(m >= 0 && m < INT32_MAX && nnz >= 0, "pos_to_rows: bad size");
  SB_CHECK_ARG(pos && (row || nnz == 0), "pos_to_rows: null pointer");
  if (m == 0 || nnz == 0) return SB_OK;
  const int threads = 256;
  pos_to_rows_kernel<<<(unsigned)ceil_div(m * 32, threads), threads, 0, (cudaStream_t)stream>>>(
      (int)m, pos, row);
  SB_LAUNCH_CHECK("pos_to_rows_kernel");
  return SB_OK;
}

}  // extern "C"
