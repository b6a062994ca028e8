// Device-side data-format plumbing either side of the sparse kernels, so that whole pipelines
// stay on the GPU:
//   * dense matrix -> CSR (what the reference's callers do with torch's to_sparse_csr(), e.g. the
//     pruned weight matrices of bench/bench_sparse_autoencoder.py:233,261): two phases because
//     the output size is data dependent — count (row pointers + total), then fill;
//   * symmetric normalisation of an adjacency pattern, val[p] = d_i^-1/2 d_j^-1/2 with d = stored
//     entries per row of A + I (bench/bench_gcn.py:233-267, there with torch scatter ops);
//   * CSR transpose (CSR -> CSC of the same matrix = CSR of its transpose), the re-layout the
//     reference's front end does with torch ops before every prebuilt dispatch when an operand
//     is stored in the other mode order (src/scorch/stensor.py:785-896, ops.py:299-303,333-346):
//     count per column, scan, scatter, then each output row sorted by its (unique) source rows,
//     so the result does not depend on the order the scatter's atomics were served in;
//   * per-row top-k of a dense matrix straight to CSR (the k largest pre-activations of a
//     sparse-autoencoder layer, columns ascending, optional ReLU on the kept values): radix
//     select of the k-th largest key per row, then an ordered compaction.
#include <algorithm>

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

// ---- CSR transpose ---------------------------------------------------------------------------
__global__ void transpose_count_kernel(long long nnz, const int* __restrict__ crd, int* cnt) {
  for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < nnz;
       p += (long long)gridDim.x * blockDim.x)
    atomicAdd(cnt + ld_stream(crd + p), 1);
}

// One warp per source row: entry p = (row, j) takes the next free slot of output row j.
__global__ void __launch_bounds__(kConvWarps * 32)
transpose_scatter_kernel(int m, const int* __restrict__ pos, const int* __restrict__ crd, int* cursor,
                         int* __restrict__ trow, int* __restrict__ perm) {
  const int row = blockIdx.x * kConvWarps + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= m) return;
  const int b = __ldg(pos + row), e = __ldg(pos + row + 1);
  for (int p = b + lane; p < e; p += 32) {
    const int q = atomicAdd(cursor + ld_stream(crd + p), 1);
    trow[q] = row;
    perm[q] = p;
  }
}

// Ascending sort of n (key, payload) pairs by key with compare-exchanges that always move the
// smaller key to the lower index (the first step of every merge pairs i with its mirror image in
// the block), so positions >= n behave like +infinity without being stored.  `sync` separates
// the steps (a warp or a CTA barrier).
template <typename Sync>
__device__ __forceinline__ void sort_pairs(int* key, int* pay, int n, int tid, int nthreads, Sync sync) {
  for (int k = 2; (k >> 1) < n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int t = tid; t < n; t += nthreads) {
        const int partner = (j == (k >> 1)) ? (t ^ (k - 1)) : (t ^ j);
        if (partner > t && partner < n) {
          const int a = key[t], b = key[partner];
          if (a > b) {
            key[t] = b; key[partner] = a;
            const int pa = pay[t]; pay[t] = pay[partner]; pay[partner] = pa;
          }
        }
      }
      sync();
    }
  }
}

constexpr int kSortWarpRow = 64;     // rows up to this length: one warp, in shared memory
constexpr int kSortCtaRow = 2048;    // up to this length: the CTA, in shared memory; longer: in place

// Each CTA sorts kConvWarps consecutive output rows of (trow, perm) by trow.
__global__ void __launch_bounds__(kConvWarps * 32)
transpose_sort_rows_kernel(int n_rows, const int* __restrict__ tpos, int* trow, int* perm) {
  __shared__ int s_key[kSortCtaRow];
  __shared__ int s_pay[kSortCtaRow];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int base = blockIdx.x * kConvWarps;
  {
    const int row = base + warp;
    if (row < n_rows) {
      const int b = __ldg(tpos + row), len = __ldg(tpos + row + 1) - b;
      if (len > 1 && len <= kSortWarpRow) {
        int* k = s_key + warp * kSortWarpRow;
        int* v = s_pay + warp * kSortWarpRow;
        for (int t = lane; t < len; t += 32) { k[t] = trow[b + t]; v[t] = perm[b + t]; }
        __syncwarp();
        sort_pairs(k, v, len, lane, 32, [] { __syncwarp(); });
        for (int t = lane; t < len; t += 32) { trow[b + t] = k[t]; perm[b + t] = v[t]; }
      }
    }
  }
  for (int r = 0; r < kConvWarps; r++) {
    const int row = base + r;
    if (row >= n_rows) break;
    const int b = __ldg(tpos + row), len = __ldg(tpos + row + 1) - b;
    if (len <= kSortWarpRow) continue;            // uniform over the CTA
    __syncthreads();
    if (len <= kSortCtaRow) {
      for (int t = threadIdx.x; t < len; t += blockDim.x) { s_key[t] = trow[b + t]; s_pay[t] = perm[b + t]; }
      __syncthreads();
      sort_pairs(s_key, s_pay, len, (int)threadIdx.x, (int)blockDim.x, [] { __syncthreads(); });
      for (int t = threadIdx.x; t < len; t += blockDim.x) { trow[b + t] = s_key[t]; perm[b + t] = s_pay[t]; }
    } else {
      sort_pairs(trow + b, perm + b, len, (int)threadIdx.x, (int)blockDim.x, [] { __syncthreads(); });
    }
  }
}

template <typename T>
__global__ void transpose_gather_kernel(long long nnz, const int* __restrict__ perm,
                                        const T* __restrict__ val, T* __restrict__ tval) {
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < nnz;
       q += (long long)gridDim.x * blockDim.x)
    tval[q] = val[perm[q]];
}

// ---- per-row top-k -> CSR ----------------------------------------------------------------------
// Keys order like the floats: larger float <-> larger unsigned key (NaN above +inf, as torch.topk).
__device__ __forceinline__ unsigned topk_key(float x) {
  const unsigned u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int kTopkThreads = 256;

// One CTA per row.  Four 8-bit radix passes find the key T of the k-th largest element and how
// many elements equal to T are still needed; a last pass keeps, in column order, every element
// above T and the first `need` elements equal to T (ties go to the lower column).
__global__ void __launch_bounds__(kTopkThreads)
topk_rows_kernel(int n, int k, const float* __restrict__ X, long long ldx, int relu,
                 int* __restrict__ crd, float* __restrict__ val) {
  __shared__ int hist[256];
  __shared__ unsigned s_prefix;
  __shared__ int s_need;
  __shared__ int s_warp_gt[kTopkThreads / 32], s_warp_eq[kTopkThreads / 32];
  __shared__ int s_out, s_eq_seen;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* x = X + (long long)blockIdx.x * ldx;
  unsigned prefix = 0, mask = 0;
  int need = k;
  for (int shift = 24; shift >= 0; shift -= 8) {
    hist[tid] = 0;
    __syncthreads();
    for (int j = tid; j < n; j += kTopkThreads) {
      const unsigned key = topk_key(ld_stream(x + j));
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int above = 0, b = 255;
      for (; b > 0; b--) {
        if (above + hist[b] >= need) break;
        above += hist[b];
      }
      s_prefix = prefix | ((unsigned)b << shift);
      s_need = need - above;
    }
    __syncthreads();
    prefix = s_prefix;
    need = s_need;
    mask |= 255u << shift;
    __syncthreads();
  }
  // prefix = key of the k-th largest element; `need` of the elements equal to it are kept
  if (tid == 0) { s_out = 0; s_eq_seen = 0; }
  __syncthreads();
  const long long out0 = (long long)blockIdx.x * k;
  for (int j0 = 0; j0 < n; j0 += kTopkThreads) {
    const int j = j0 + tid;
    float v = 0.f;
    bool gt = false, eq = false;
    if (j < n) {
      v = ld_stream(x + j);
      const unsigned key = topk_key(v);
      gt = key > prefix;
      eq = key == prefix;
    }
    const unsigned m_gt = __ballot_sync(FULL, gt), m_eq = __ballot_sync(FULL, eq);
    if (lane == 0) { s_warp_gt[warp] = __popc(m_gt); s_warp_eq[warp] = __popc(m_eq); }
    __syncthreads();
    int eq_before = s_eq_seen, gt_before = 0;
    for (int w = 0; w < warp; w++) { eq_before += s_warp_eq[w]; gt_before += s_warp_gt[w]; }
    const unsigned below = (1u << lane) - 1u;
    const int my_eq_rank = eq_before + __popc(m_eq & below);     // equals before this element
    const bool keep = gt || (eq && my_eq_rank < need);
    // kept elements before this one in the chunk: all greater ones + equals still within `need`
    int eq_kept_before = min(need, my_eq_rank) - min(need, s_eq_seen);
    const int slot = s_out + gt_before + __popc(m_gt & below) + eq_kept_before;
    if (keep) {
      crd[out0 + slot] = j;
      val[out0 + slot] = (relu && !(v > 0.f)) ? 0.f : v;
    }
    __syncthreads();
    if (tid == 0) {
      int tg = 0, te = 0;
      for (int w = 0; w < kTopkThreads / 32; w++) { tg += s_warp_gt[w]; te += s_warp_eq[w]; }
      const int seen = s_eq_seen;
      s_out += tg + (min(need, seen + te) - min(need, seen));
      s_eq_seen = seen + te;
    }
    __syncthreads();
  }
}

__global__ void topk_pos_kernel(int m, int k, int* pos) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i <= m) pos[i] = i * k;
}

}  // namespace sb

using namespace sb;

extern "C" {

size_t sb_csr_transpose_workspace_bytes(int64_t n, int64_t nnz) {
  if (n < 0) n = 0;
  if (nnz < 0) nnz = 0;
  // column counts / cursors (n + 1 ints), scan temporaries, total, source-entry permutation
  return (size_t)(((n + 1) * 4 + 255) / 256 * 256) +
         (size_t)((ceil_div(n + 1, 4096) + 1) * 8 + 255) / 256 * 256 + 256 +
         (size_t)((nnz * 4 + 255) / 256 * 256);
}

int sb_csr_transpose(int dtype, int64_t m, int64_t n, int64_t nnz, const int32_t* pos,
                     const int32_t* crd, const void* val, int32_t* tpos, int32_t* tcrd, void* tval,
                     void* ws, size_t ws_bytes, void* stream) {
  SB_CHECK_ARG(m >= 0 && n >= 0 && nnz >= 0 && m < INT32_MAX && n < INT32_MAX, "csr_transpose: bad size");
  if (nnz > INT32_MAX) return fail(SB_ERR_OVERFLOW, "csr_transpose: nnz does not fit int32");
  SB_CHECK_ARG(dtype >= SB_F32 && dtype <= SB_I64, "csr_transpose: unknown dtype");
  SB_CHECK_ARG(pos && tpos, "csr_transpose: null row pointers");
  SB_CHECK_ARG(nnz == 0 || (crd && tcrd), "csr_transpose: null crd / tcrd");
  SB_CHECK_ARG((val == nullptr) == (tval == nullptr), "csr_transpose: val and tval must both be given or both be null");
  const size_t need = sb_csr_transpose_workspace_bytes(n, nnz);
  SB_CHECK_ARG(ws && aligned16(ws), "csr_transpose: workspace is null or misaligned");
  if (ws_bytes < need)
    return fail(SB_ERR_WORKSPACE, "csr_transpose: workspace has %zu bytes, needs %zu", ws_bytes, need);
  cudaStream_t st = (cudaStream_t)stream;
  char* base = static_cast<char*>(ws);
  int* cnt = reinterpret_cast<int*>(base);
  const size_t off1 = (size_t)(((n + 1) * 4 + 255) / 256 * 256);
  const size_t off2 = off1 + (size_t)((ceil_div(n + 1, 4096) + 1) * 8 + 255) / 256 * 256;
  long long* block_sum = reinterpret_cast<long long*>(base + off1);
  long long* total = reinterpret_cast<long long*>(base + off2);
  int* perm = reinterpret_cast<int*>(base + off2 + 256);
  SB_CUDA(cudaMemsetAsync(cnt, 0, (size_t)(n + 1) * 4, st));
  if (nnz > 0) {
    const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(nnz, 256), 32 * sm_count());
    transpose_count_kernel<<<blocks, 256, 0, st>>>(nnz, crd, cnt);
    SB_LAUNCH_CHECK("transpose_count_kernel");
  }
  if (n == 0) {
    SB_CUDA(cudaMemsetAsync(tpos, 0, 4, st));
    return SB_OK;
  }
  int rc = exclusive_scan_i32((int)n, cnt, tpos, block_sum, total, st);
  if (rc != SB_OK) return rc;
  if (nnz == 0 || m == 0) return SB_OK;
  SB_CUDA(cudaMemcpyAsync(cnt, tpos, (size_t)n * 4, cudaMemcpyDeviceToDevice, st));  // cursors
  transpose_scatter_kernel<<<(unsigned)ceil_div(m, kConvWarps), kConvWarps * 32, 0, st>>>(
      (int)m, pos, crd, cnt, tcrd, perm);
  SB_LAUNCH_CHECK("transpose_scatter_kernel");
  transpose_sort_rows_kernel<<<(unsigned)ceil_div(n, kConvWarps), kConvWarps * 32, 0, st>>>(
      (int)n, tpos, tcrd, perm);
  SB_LAUNCH_CHECK("transpose_sort_rows_kernel");
  if (val) {
    const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(nnz, 256), 32 * sm_count());
    if (dtype == SB_F32 || dtype == SB_I32)
      transpose_gather_kernel<unsigned><<<blocks, 256, 0, st>>>(nnz, perm, (const unsigned*)val, (unsigned*)tval);
    else
      transpose_gather_kernel<unsigned long long><<<blocks, 256, 0, st>>>(
          nnz, perm, (const unsigned long long*)val, (unsigned long long*)tval);
    SB_LAUNCH_CHECK("transpose_gather_kernel");
  }
  return SB_OK;
}

int sb_topk_rows_to_csr_f32(int64_t m, int64_t n, int64_t k, const float* X, int64_t ldx, int relu,
                            int32_t* pos, int32_t* crd, float* val, void* stream) {
  SB_CHECK_ARG(m >= 0 && n >= 0 && k >= 0 && m < INT32_MAX && n < INT32_MAX, "topk_rows: bad size");
  SB_CHECK_ARG(k <= n, "topk_rows: k exceeds the row length");
  if (m * k > INT32_MAX) return fail(SB_ERR_OVERFLOW, "topk_rows: m*k does not fit int32 row pointers");
  SB_CHECK_ARG(pos, "topk_rows: pos is null");
  SB_CHECK_ARG(ldx >= n, "topk_rows: leading dimension smaller than n");
  cudaStream_t st = (cudaStream_t)stream;
  topk_pos_kernel<<<(unsigned)ceil_div(m + 1, 256), 256, 0, st>>>((int)m, (int)k, pos);
  SB_LAUNCH_CHECK("topk_pos_kernel");
  if (m == 0 || k == 0) return SB_OK;
  SB_CHECK_ARG(X && crd && val, "topk_rows: null pointer");
  topk_rows_kernel<<<(unsigned)m, kTopkThreads, 0, st>>>((int)n, (int)k, X, ldx, relu, crd, val);
  SB_LAUNCH_CHECK("topk_rows_kernel");
  return SB_OK;
}

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
