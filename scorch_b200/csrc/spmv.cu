// CSR SpMV for sm_100a.
//
// fp32: entry-tiled kernel (below), balanced by stored entries.  x is gathered through the
// read-only path (it is L2 resident: 8 MB for 2M columns); the CSR streams are read once with
// no-allocate loads.  The other registry dtypes (f64 / i32 / i64) use a plain G-lanes-per-row
// kernel (G chosen from the mean row length).
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

// ---- fp32: entry-tiled kernel ------------------------------------------------------------------
// The entry arrays are cut into tiles of kTile consecutive entries, one CTA per tile, whatever
// the row lengths are (power-law rows included: a hub row simply spans many tiles).  A tile
//   1. finds its first and last row with a 256-ary search over pos[] (3 rounds for 2M rows),
//   2. streams its crd/val slices with 8 independent loads per thread, gathers x and leaves the
//      products in shared memory,
//   3. sums each row's segment (one thread per row for short rows, one warp per row for long
//      ones) and writes y for rows that lie completely inside the tile.
// A row cut by a tile border leaves partial sums in the scratch arrays; a second, tiny kernel
// adds them in tile order, so the result does not depend on scheduling.
constexpr int kTile = 2048;
constexpr int kTileThreads = 256;

struct TileScratch {
  float* carry_first;  // partial sum of the tile's first row when that row began in an earlier tile
  float* carry_last;   // partial sum of the tile's last row when it began here and continues
  int* last_row;       // that last row, or -1
};

// Largest r in [lo, hi) with pos[r] <= p, given pos[lo] <= p < pos[hi]; all threads of the CTA
// call it together and get the same answer.
__device__ __forceinline__ int find_row_cta(const int* __restrict__ pos, int lo, int hi, int p) {
  const int tid = threadIdx.x;
  while (true) {
    const int span = hi - lo;
    if (span <= kTileThreads) {
      const int r = lo + tid;
      const int c = __syncthreads_count(r < hi && __ldg(pos + r) <= p);
      return lo + c - 1;
    }
    const int step = (span + kTileThreads - 1) / kTileThreads;
    const long long r = (long long)lo + (long long)tid * step;
    const int c = __syncthreads_count(r < hi && __ldg(pos + r) <= p);
    lo = lo + (c - 1) * step;
    hi = min(hi, lo + step);
  }
}

__global__ void __launch_bounds__(kTileThreads)
spmv_tile_kernel(int m, int nnz, const int* __restrict__ pos, const int* __restrict__ crd,
                 const float* __restrict__ val, const float* __restrict__ x, float* __restrict__ y,
                 TileScratch sc) {
  __shared__ float prod[kTile];
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int e0 = t * kTile, e1 = min(nnz, e0 + kTile);
  // products first: the loads are independent of the row search below
  {
    int j[kTile / kTileThreads];
    float a[kTile / kTileThreads];
#pragma unroll
    for (int q = 0; q < kTile / kTileThreads; q++) {
      const int e = e0 + tid + q * kTileThreads;
      j[q] = 0;
      a[q] = 0.f;
      if (e < e1) {
        j[q] = ld_stream(crd + e);
        a[q] = ld_stream(val + e);
      }
    }
#pragma unroll
    for (int q = 0; q < kTile / kTileThreads; q++) {
      const int e = e0 + tid + q * kTileThreads;
      prod[tid + q * kTileThreads] = (e < e1) ? a[q] * __ldg(x + j[q]) : 0.f;
    }
  }
  const int r_lo = find_row_cta(pos, 0, m, e0);
  const int r_hi = find_row_cta(pos, r_lo, m, e1 - 1);
  __syncthreads();
  const int nr = r_hi - r_lo + 1;
  const bool thread_per_row = nr >= 128;
  const int first = thread_per_row ? tid : warp;
  const int stride = thread_per_row ? kTileThreads : kTileThreads / 32;
  for (int r = r_lo + first; r <= r_hi; r += stride) {
    const int rb = __ldg(pos + r), re = __ldg(pos + r + 1);
    const int b = max(rb, e0) - e0, e = min(re, e1) - e0;
    float s = 0.f;
    if (thread_per_row) {
      for (int i = b; i < e; i++) s += prod[i];
    } else {
      for (int i = b + lane; i < e; i += 32) s += prod[i];
      s = group_sum<32>(s);
      if (lane != 0) continue;
    }
    if (rb >= e0 && re <= e1) {
      y[r] = s;
    } else if (rb < e0) {
      sc.carry_first[t] = s;             // continues a row that began in an earlier tile
    } else {
      sc.carry_last[t] = s;              // begins here, continues in the next tile
    }
  }
  if (tid == 0) {
    const int rb = __ldg(pos + r_hi), re = __ldg(pos + r_hi + 1);
    sc.last_row[t] = (re > e1 && rb >= e0) ? r_hi : -1;
  }
}

// Adds the pieces of every row that was cut by tile borders, in tile order.
__global__ void spmv_tile_fixup_kernel(int ntiles, const int* __restrict__ pos, float* __restrict__ y,
                                       TileScratch sc) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= ntiles) return;
  const int r = sc.last_row[t];
  if (r < 0) return;
  const long long row_end = pos[r + 1];
  float s = sc.carry_last[t];
  for (int u = t + 1; u < ntiles; u++) {
    s += sc.carry_first[u];
    if (row_end <= (long long)(u + 1) * kTile) break;
  }
  y[r] = s;
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
  // (the tile kernels add up to one tile, 2048 entries, to an entry index held in an int)
  if (nnz > INT32_MAX - 4096)
    return fail(SB_ERR_OVERFLOW, "spmv: nnz=%lld does not fit int32 row pointers", (long long)nnz);
  SB_CHECK_ARG(pos, "spmv: pos is null");
  SB_CHECK_ARG(nnz == 0 || (crd && val && x), "spmv: null crd/val/x");
  SB_CHECK_ARG(m == 0 || y, "spmv: y is null");
  return SB_OK;
}

}  // namespace sb

using namespace sb;

extern "C" {

size_t sb_spmv_csr_scratch_bytes(int64_t nnz) {
  if (nnz <= 0) return 0;
  const size_t tiles = (size_t)ceil_div(nnz, kTile);
  return ((tiles * 4 + 255) / 256 * 256) * 3;
}

int sb_spmv_csr_f32(int64_t m, int64_t n, int64_t nnz, const int32_t* pos, const int32_t* crd,
                    const float* val, const float* x, float* y, void* scratch, size_t scratch_bytes,
                    void* stream) {
  int rc = check_spmv(m, n, nnz, pos, crd, val, x, y);
  if (rc != SB_OK) return rc;
  if (m == 0) return SB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  // rows without entries are not visited by any tile
  SB_CUDA(cudaMemsetAsync(y, 0, (size_t)m * sizeof(float), st));
  if (nnz == 0) return SB_OK;
  const size_t need = sb_spmv_csr_scratch_bytes(nnz);
  SB_CHECK_ARG(scratch && aligned16(scratch), "spmv: scratch is null or misaligned");
  if (scratch_bytes < need)
    return fail(SB_ERR_WORKSPACE, "spmv: scratch has %zu bytes, needs %zu", scratch_bytes, need);
  const int tiles = (int)ceil_div(nnz, kTile);
  const size_t stride = need / 3;
  char* base = static_cast<char*>(scratch);
  TileScratch sc{reinterpret_cast<float*>(base), reinterpret_cast<float*>(base + stride),
                 reinterpret_cast<int*>(base + 2 * stride)};
  spmv_tile_kernel<<<tiles, kTileThreads, 0, st>>>((int)m, (int)nnz, pos, crd, val, x, y, sc);
  SB_LAUNCH_CHECK("spmv_tile_kernel");
  spmv_tile_fixup_kernel<<<(unsigned)ceil_div(tiles, 128), 128, 0, st>>>(tiles, pos, y, sc);
  SB_LAUNCH_CHECK("spmv_tile_fixup_kernel");
  return SB_OK;
}

int sb_spmv_csr_typed(int dtype, int64_t m, int64_t n, int64_t nnz, const int32_t* pos,
                      const int32_t* crd, const void* val, const void* x, void* y, void* stream) {
  int rc = check_spmv(m, n, nnz, pos, crd, val, x, y);
  if (rc != SB_OK) return rc;
  if (m == 0) return SB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case SB_F32:  // without scratch: the lanes-per-row kernel
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
