// Element-wise products and sums of two CSR matrices of the same shape:
//   multiply  C[i,j] = A[i,j] * B[i,j]   stored where BOTH operands store an entry (intersection)
//   add       C[i,j] = A[i,j] + B[i,j]   stored where EITHER operand stores an entry (union)
// with ascending columns per row and the symbolic structure kept (a sum or product that happens
// to be zero stays stored) — the output the reference's compiler emits for
// einsum("ij,ij->ij", A, B) and A + B over compressed operands
// (src/scorch/ops.py:375-819, exercised by tests/test_scorch/test_kernels_comprehensive.py:119-200).
// Two phases like SpGEMM, because the output size depends on the data: the symbolic phase counts
// the common columns of every row pair and scans the counts into row pointers; the numeric phase
// writes columns and values.  One warp per row: lanes take entries of one operand's row and
// binary-search the other operand's row, so hub rows cost O(len log len) and no sequential merge.
#include "common.cuh"

namespace sb {

constexpr int kEwWarps = 8;

// Number of entries of crd[b, e) smaller than c, and whether c is among them (found).
__device__ __forceinline__ int rank_in_row(const int* __restrict__ crd, int b, int e, int c, bool& found) {
  int lo = b, hi = e;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(crd + mid) < c) lo = mid + 1; else hi = mid;
  }
  found = lo < e && __ldg(crd + lo) == c;
  return lo - b;
}

__global__ void __launch_bounds__(kEwWarps * 32)
ewise_count_kernel(int op, int m, const int* __restrict__ Apos, const int* __restrict__ Acrd,
                   const int* __restrict__ Bpos, const int* __restrict__ Bcrd, int* __restrict__ cnt) {
  const int row = blockIdx.x * kEwWarps + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= m) return;
  const int ab = __ldg(Apos + row), ae = __ldg(Apos + row + 1);
  const int bb = __ldg(Bpos + row), be = __ldg(Bpos + row + 1);
  int common = 0;
  for (int p = ab + lane; p < ae; p += 32) {
    bool found;
    rank_in_row(Bcrd, bb, be, ld_stream(Acrd + p), found);
    common += found;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) common += __shfl_xor_sync(FULL, common, o);
  if (lane == 0) cnt[row] = op == 0 ? common : (ae - ab) + (be - bb) - common;
}

template <typename T>
__global__ void __launch_bounds__(kEwWarps * 32)
ewise_fill_kernel(int op, int m, const int* __restrict__ Apos, const int* __restrict__ Acrd,
                  const T* __restrict__ Aval, const int* __restrict__ Bpos, const int* __restrict__ Bcrd,
                  const T* __restrict__ Bval, const int* __restrict__ Cpos, int* __restrict__ Ccrd,
                  T* __restrict__ Cval) {
  const int row = blockIdx.x * kEwWarps + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= m) return;
  const int ab = __ldg(Apos + row), ae = __ldg(Apos + row + 1);
  const int bb = __ldg(Bpos + row), be = __ldg(Bpos + row + 1);
  const int out = __ldg(Cpos + row);
  const unsigned below = (1u << lane) - 1u;
  // entries of A: a common column goes to (common columns before it) for a product; for a sum every
  // A entry goes to (its index in A) + (entries of B before its column that A does not store)
  int common_before = 0;
  for (int p0 = ab; p0 < ae; p0 += 32) {
    const int p = p0 + lane;
    bool found = false;
    int rank_b = 0, c = 0;
    if (p < ae) {
      c = ld_stream(Acrd + p);
      rank_b = rank_in_row(Bcrd, bb, be, c, found);
    }
    const unsigned hits = __ballot_sync(FULL, found);
    const int mine = common_before + __popc(hits & below);   // common columns before this entry
    if (p < ae) {
      if (op == 0) {
        if (found) {
          Ccrd[out + mine] = c;
          Cval[out + mine] = Aval[p] * Bval[bb + rank_b];
        }
      } else {
        const int dst = out + (p - ab) + rank_b - mine;
        Ccrd[dst] = c;
        Cval[dst] = found ? Aval[p] + Bval[bb + rank_b] : Aval[p];
      }
    }
    common_before += __popc(hits);
  }
  if (op == 0) return;
  // entries only B stores: (entries of A before the column) + (B-only entries before it)
  common_before = 0;
  for (int p0 = bb; p0 < be; p0 += 32) {
    const int p = p0 + lane;
    bool found = false;
    int rank_a = 0, c = 0;
    if (p < be) {
      c = ld_stream(Bcrd + p);
      rank_a = rank_in_row(Acrd, ab, ae, c, found);
    }
    const unsigned hits = __ballot_sync(FULL, found);
    const int mine = common_before + __popc(hits & below);
    if (p < be && !found) {
      const int dst = out + rank_a + (p - bb) - mine;
      Ccrd[dst] = c;
      Cval[dst] = Bval[p];
    }
    common_before += __popc(hits);
  }
}

}  // namespace sb

using namespace sb;

extern "C" {

size_t sb_csr_ewise_workspace_bytes(int64_t m) {
  if (m < 0) m = 0;
  // row counts + scan temporaries + total
  return (size_t)(((m + 1) * 4 + 255) / 256 * 256) + (size_t)((ceil_div(m + 1, 4096) + 1) * 8 + 255) / 256 * 256 + 256;
}

static int check_ewise(int op, int64_t m, const void* Apos, const void* Bpos) {
  SB_CHECK_ARG(op == SB_EWISE_MUL || op == SB_EWISE_ADD, "csr_ewise: unknown operation");
  SB_CHECK_ARG(m >= 0 && m < INT32_MAX, "csr_ewise: bad row count");
  SB_CHECK_ARG(Apos && Bpos, "csr_ewise: null row pointers");
  return SB_OK;
}

int sb_csr_ewise_symbolic(int op, int64_t m, const int32_t* Apos, const int32_t* Acrd, const int32_t* Bpos,
                          const int32_t* Bcrd, int32_t* Cpos, int64_t* nnz_host, void* ws, size_t ws_bytes,
                          void* stream) {
  int rc = check_ewise(op, m, Apos, Bpos);
  if (rc != SB_OK) return rc;
  SB_CHECK_ARG(Cpos && nnz_host, "csr_ewise: null Cpos / nnz_host");
  cudaStream_t st = (cudaStream_t)stream;
  *nnz_host = 0;
  if (m == 0) {
    SB_CUDA(cudaMemsetAsync(Cpos, 0, 4, st));
    SB_CUDA(cudaStreamSynchronize(st));
    return SB_OK;
  }
  const size_t need = sb_csr_ewise_workspace_bytes(m);
  SB_CHECK_ARG(ws && aligned16(ws), "csr_ewise: workspace is null or misaligned");
  if (ws_bytes < need)
    return fail(SB_ERR_WORKSPACE, "csr_ewise: workspace has %zu bytes, needs %zu", ws_bytes, need);
  char* base = static_cast<char*>(ws);
  int* cnt = reinterpret_cast<int*>(base);
  const size_t off1 = (size_t)(((m + 1) * 4 + 255) / 256 * 256);
  long long* block_sum = reinterpret_cast<long long*>(base + off1);
  long long* total = reinterpret_cast<long long*>(base + need - 256);
  ewise_count_kernel<<<(unsigned)ceil_div(m, kEwWarps), kEwWarps * 32, 0, st>>>(op, (int)m, Apos, Acrd, Bpos,
                                                                              Bcrd, cnt);
  SB_LAUNCH_CHECK("ewise_count_kernel");
  rc = exclusive_scan_i32((int)m, cnt, Cpos, block_sum, total, st);
  if (rc != SB_OK) return rc;
  long long t = 0;
  SB_CUDA(cudaMemcpyAsync(&t, total, 8, cudaMemcpyDeviceToHost, st));
  SB_CUDA(cudaStreamSynchronize(st));
  if (t > INT32_MAX) return fail(SB_ERR_OVERFLOW, "csr_ewise: %lld stored entries do not fit int32", t);
  *nnz_host = t;
  return SB_OK;
}

int sb_csr_ewise_numeric(int op, int dtype, int64_t m, const int32_t* Apos, const int32_t* Acrd,
                         const void* Aval, const int32_t* Bpos, const int32_t* Bcrd, const void* Bval,
                         const int32_t* Cpos, int32_t* Ccrd, void* Cval, void* stream) {
  int rc = check_ewise(op, m, Apos, Bpos);
  if (rc != SB_OK) return rc;
  if (m == 0) return SB_OK;
  SB_CHECK_ARG(Cpos, "csr_ewise: Cpos is null");
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = (unsigned)ceil_div(m, kEwWarps);
#define SB_EW(T)                                                                                          \
  ewise_fill_kernel<T><<<grid, kEwWarps * 32, 0, st>>>(op, (int)m, Apos, Acrd, (const T*)Aval, Bpos, Bcrd, \
                                                        (const T*)Bval, Cpos, Ccrd, (T*)Cval)
  switch (dtype) {
    case SB_F32: SB_EW(float); break;
    case SB_F64: SB_EW(double); break;
    case SB_I32: SB_EW(unsigned int); break;        // unsigned: the reference's wrapping arithmetic
    case SB_I64: SB_EW(unsigned long long); break;
    default: return fail(SB_ERR_UNSUPPORTED, "csr_ewise: unknown dtype %d", dtype);
  }
#undef SB_EW
  SB_LAUNCH_CHECK("ewise_fill_kernel");
  return SB_OK;
}

}  // extern "C"
