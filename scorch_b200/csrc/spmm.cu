// CSR x dense SpMM for sm_100a.
//
// Work split (nnz-balanced):
//   * rows with at most SB_HEAVY_ROW_NNZ entries: one warp per row.  L lanes span a column tile
//     with 128-bit loads of the dense operand, the 32/L lane groups take alternate entries of the
//     row, and a fixed-order shuffle tree adds the groups;
//   * heavier rows (hubs of power-law graphs): cut into segments of SB_HEAVY_ROW_NNZ entries by
//     the row plan; one CTA per segment, one partial sum per warp in shared memory, added in warp
//     order; rows with several segments go through a scratch buffer and a fixed-order finalise.
// The CSR column/value streams are read with coalesced no-allocate loads, one 32-entry chunk per
// warp at a time, and handed to the lanes by shuffles; C is written once with streaming stores.
// Large k is cut into column panels on grid.y, so that one panel of the dense operand stays in
// L2 while all rows pass over it.
#include "common.cuh"

namespace sb {

constexpr int kWarpsPerCta = 8;

struct SpmmArgs {
  int m;
  int k;
  const int* pos;
  const int* crd;
  const float* val;
  const float* B;
  long long ldb;
  const float* bias;
  int relu;
  float* C;
  long long ldc;
  long long stride_val, stride_b, stride_c;
  int skip_heavy;  // rows longer than SB_HEAVY_ROW_NNZ are left to the heavy kernels
};

// Accumulate entries [b, e) of one row into acc[] for this lane's columns.
// L lanes per group, G = 32/L groups; group g takes entries b+g, b+g+G, ...
template <int L, int VEC>
__device__ __forceinline__ void accumulate_range(float4 (&acc)[VEC], const int* __restrict__ crd,
                                                 const float* __restrict__ val,
                                                 const float* __restrict__ Bcol, long long ldb,
                                                 int b, int e, int lane, bool col_ok[VEC]) {
  constexpr int G = 32 / L;
  const int g = lane / L;
  // software pipeline: the next chunk's indices/values are in flight while this chunk's rows of
  // the dense operand are gathered
  int next_j = 0;
  float next_a = 0.f;
  if (b + lane < e) {
    next_j = ld_stream(crd + b + lane);
    next_a = ld_stream(val + b + lane);
  }
  for (int p0 = b; p0 < e; p0 += 32) {
    const int cnt = min(32, e - p0);
    const int my_j = next_j;
    const float my_a = next_a;
    if (p0 + 32 + lane < e) {
      next_j = ld_stream(crd + p0 + 32 + lane);
      next_a = ld_stream(val + p0 + 32 + lane);
    }
    if (cnt == 32) {
      constexpr int STEPS = 32 / G;
      constexpr int U = (STEPS >= 8) ? 8 : STEPS;
#pragma unroll 1
      for (int s0 = 0; s0 < STEPS; s0 += U) {
        int j[U];
        float a[U];
        float4 bv[U][VEC];
#pragma unroll
        for (int u = 0; u < U; u++) {
          const int t = (s0 + u) * G + g;
          j[u] = __shfl_sync(FULL, my_j, t);
          a[u] = __shfl_sync(FULL, my_a, t);
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
          const float* brow = Bcol + (long long)j[u] * ldb;
#pragma unroll
          for (int v = 0; v < VEC; v++)
            bv[u][v] = col_ok[v] ? ldg4(brow + v * L * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
#pragma unroll
          for (int v = 0; v < VEC; v++) fma4(acc[v], a[u], bv[u][v]);
        }
      }
    } else {
      for (int t0 = 0; t0 < cnt; t0 += G) {
        const int t = t0 + g;
        const int j = __shfl_sync(FULL, my_j, t & 31);
        const float a = __shfl_sync(FULL, my_a, t & 31);
        if (t < cnt) {
          const float* brow = Bcol + (long long)j * ldb;
#pragma unroll
          for (int v = 0; v < VEC; v++)
            if (col_ok[v]) fma4(acc[v], a, ldg4(brow + v * L * 4));
        }
      }
    }
  }
}

template <int L, int VEC>
__device__ __forceinline__ void reduce_groups(float4 (&acc)[VEC]) {
#pragma unroll
  for (int o = L; o < 32; o <<= 1) {
#pragma unroll
    for (int v = 0; v < VEC; v++) {
      acc[v].x += __shfl_xor_sync(FULL, acc[v].x, o);
      acc[v].y += __shfl_xor_sync(FULL, acc[v].y, o);
      acc[v].z += __shfl_xor_sync(FULL, acc[v].z, o);
      acc[v].w += __shfl_xor_sync(FULL, acc[v].w, o);
    }
  }
}

__device__ __forceinline__ float4 epilogue(float4 s, const float* bias, int col, int relu) {
  if (bias) {
    const float4 bb = ldg4(bias + col);
    s.x += bb.x; s.y += bb.y; s.z += bb.z; s.w += bb.w;
  }
  if (relu) {
    s.x = s.x > 0.f ? s.x : 0.f;
    s.y = s.y > 0.f ? s.y : 0.f;
    s.z = s.z > 0.f ? s.z : 0.f;
    s.w = s.w > 0.f ? s.w : 0.f;
  }
  return s;
}

// One warp per row; grid = (row blocks, column tiles, batch).
template <int L, int VEC>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
spmm_rows_kernel(SpmmArgs a) {
  constexpr int TILE = L * 4 * VEC;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerCta + warp;
  if (row >= a.m) return;
  const int b = __ldg(a.pos + row), e = __ldg(a.pos + row + 1);
  if (a.skip_heavy && e - b > SB_HEAVY_ROW_NNZ) return;
  const long long bz = blockIdx.z;
  const int l = lane % L;
  const int col0 = blockIdx.y * TILE + l * 4;
  bool col_ok[VEC];
  float4 acc[VEC];
#pragma unroll
  for (int v = 0; v < VEC; v++) {
    col_ok[v] = (col0 + v * L * 4) < a.k;
    acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  accumulate_range<L, VEC>(acc, a.crd, a.val + bz * a.stride_val, a.B + bz * a.stride_b + col0,
                           a.ldb, b, e, lane, col_ok);
  reduce_groups<L, VEC>(acc);
  if (lane < L) {
    float* crow = a.C + bz * a.stride_c + (long long)row * a.ldc;
#pragma unroll
    for (int v = 0; v < VEC; v++) {
      const int col = col0 + v * L * 4;
      if (col_ok[v]) st_stream4(crow + col, epilogue(acc[v], a.bias, col, a.relu));
    }
  }
}

struct HeavyArgs {
  const int* hdr;
  const int* heavy_row;
  const int* heavy_seg0;
  const int* heavy_nseg;
  const int* seg_heavy;
  float* scratch;            // [batch][segments_cap][k]
  long long scratch_batch;   // elements between batch items
};

// One CTA per heavy-row segment; grid = (segments, column tiles, batch).
template <int L, int VEC>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
spmm_heavy_kernel(SpmmArgs a, HeavyArgs h) {
  constexpr int TILE = L * 4 * VEC;
  __shared__ float4 part[kWarpsPerCta][VEC][L];
  const int seg = blockIdx.x;
  if (seg >= __ldg(h.hdr + 1)) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = __ldg(h.seg_heavy + seg);
  const int row = __ldg(h.heavy_row + slot);
  const int seg0 = __ldg(h.heavy_seg0 + slot);
  const int nseg = __ldg(h.heavy_nseg + slot);
  const int rb = __ldg(a.pos + row), re = __ldg(a.pos + row + 1);
  const int sb_ = rb + (seg - seg0) * SB_HEAVY_ROW_NNZ;
  const int se = min(re, sb_ + SB_HEAVY_ROW_NNZ);
  const long long bz = blockIdx.z;
  const int l = lane % L;
  const int col0 = blockIdx.y * TILE + l * 4;
  bool col_ok[VEC];
  float4 acc[VEC];
#pragma unroll
  for (int v = 0; v < VEC; v++) {
    col_ok[v] = (col0 + v * L * 4) < a.k;
    acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // each warp owns a contiguous slice of the segment (a multiple of 32 entries)
  constexpr int SLICE = SB_HEAVY_ROW_NNZ / kWarpsPerCta;
  const int wb = min(se, sb_ + warp * SLICE), we = min(se, wb + SLICE);
  accumulate_range<L, VEC>(acc, a.crd, a.val + bz * a.stride_val, a.B + bz * a.stride_b + col0,
                           a.ldb, wb, we, lane, col_ok);
  reduce_groups<L, VEC>(acc);
  if (lane < L) {
#pragma unroll
    for (int v = 0; v < VEC; v++) part[warp][v][l] = acc[v];
  }
  __syncthreads();
  if (warp == 0 && lane < L) {
#pragma unroll
    for (int v = 0; v < VEC; v++) {
      float4 s = part[0][v][l];
#pragma unroll
      for (int w = 1; w < kWarpsPerCta; w++) {
        const float4 t = part[w][v][l];
        s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
      }
      const int col = col0 + v * L * 4;
      if (!col_ok[v]) continue;
      if (nseg == 1) {
        st_stream4(a.C + bz * a.stride_c + (long long)row * a.ldc + col,
                   epilogue(s, a.bias, col, a.relu));
      } else {
        float* dst = h.scratch + bz * h.scratch_batch + (long long)seg * a.k + col;
        *reinterpret_cast<float4*>(dst) = s;
      }
    }
  }
}

// Adds the segment sums of every multi-segment heavy row in segment order.
// grid = (heavy rows bound, 1, batch); threads span the columns in float4 units.
__global__ void spmm_heavy_finalize_kernel(SpmmArgs a, HeavyArgs h) {
  const int slot = blockIdx.x;
  if (slot >= __ldg(h.hdr)) return;
  const int nseg = __ldg(h.heavy_nseg + slot);
  if (nseg == 1) return;
  const int row = __ldg(h.heavy_row + slot);
  const int seg0 = __ldg(h.heavy_seg0 + slot);
  const long long bz = blockIdx.z;
  const float* src = h.scratch + bz * h.scratch_batch + (long long)seg0 * a.k;
  float* crow = a.C + bz * a.stride_c + (long long)row * a.ldc;
  for (int col = threadIdx.x * 4; col < a.k; col += blockDim.x * 4) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int t = 0; t < nseg; t++) {
      const float4 v = *reinterpret_cast<const float4*>(src + (long long)t * a.k + col);
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    st_stream4(crow + col, epilogue(s, a.bias, col, a.relu));
  }
}

// Scalar path for any dtype / any layout: one warp per row, lanes span 32 columns per grid.y
// step.  Used for f64/i32/i64 (registry parity) and for fp32 operands that are not 16-byte
// aligned or whose k is not a multiple of 4.
template <typename T>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
spmm_generic_kernel(int m, int k, const int* __restrict__ pos, const int* __restrict__ crd,
                    const T* __restrict__ val, const T* __restrict__ B, long long ldb,
                    const T* __restrict__ bias, int relu, T* __restrict__ C, long long ldc,
                    long long stride_val, long long stride_b, long long stride_c) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerCta + warp;
  if (row >= m) return;
  const long long bz = blockIdx.z;
  val += bz * stride_val;
  B += bz * stride_b;
  C += bz * stride_c;
  const int col = blockIdx.y * 32 + lane;
  if (col >= k) return;
  T acc = bias ? bias[col] : T(0);
  const int b = pos[row], e = pos[row + 1];
  for (int p = b; p < e; p++) acc += val[p] * B[(long long)crd[p] * ldb + col];
  if (relu) acc = acc > T(0) ? acc : T(0);
  C[(long long)row * ldc + col] = acc;
}

template <int L, int VEC>
static int launch_vec(const SpmmArgs& a, int64_t batch, const void* plan, int64_t nnz,
                      int64_t plan_segments, void* scratch, cudaStream_t st) {
  constexpr int TILE = L * 4 * VEC;
  const unsigned tiles = (unsigned)ceil_div(a.k, TILE);
  dim3 grid((unsigned)ceil_div(a.m, kWarpsPerCta), tiles, (unsigned)batch);
  spmm_rows_kernel<L, VEC><<<grid, kWarpsPerCta * 32, 0, st>>>(a);
  SB_LAUNCH_CHECK("spmm_rows_kernel");
  if (plan && plan_segments != 0) {
    PlanView pv = plan_view(plan, nnz);
    const int64_t segs = plan_segments < 0 ? pv.cap_seg : plan_segments;
    HeavyArgs h{pv.hdr, pv.heavy_row, pv.heavy_seg0, pv.heavy_nseg, pv.seg_heavy,
                static_cast<float*>(scratch), (long long)segs * a.k};
    dim3 hg((unsigned)segs, tiles, (unsigned)batch);
    spmm_heavy_kernel<L, VEC><<<hg, kWarpsPerCta * 32, 0, st>>>(a, h);
    SB_LAUNCH_CHECK("spmm_heavy_kernel");
    const int64_t heavy_bound = segs < pv.cap_heavy ? segs : pv.cap_heavy;
    dim3 fg((unsigned)heavy_bound, 1, (unsigned)batch);
    const int threads = a.k >= 1024 ? 256 : (a.k >= 512 ? 128 : 64);
    spmm_heavy_finalize_kernel<<<fg, threads, 0, st>>>(a, h);
    SB_LAUNCH_CHECK("spmm_heavy_finalize_kernel");
  }
  return SB_OK;
}

template <typename T>
static int launch_generic(int64_t m, int64_t k, const int32_t* pos, const int32_t* crd,
                          const T* val, const T* B, int64_t ldb, const T* bias, int relu, T* C,
                          int64_t ldc, int64_t batch, int64_t sv, int64_t sbb, int64_t sc,
                          cudaStream_t st) {
  dim3 grid((unsigned)ceil_div(m, kWarpsPerCta), (unsigned)ceil_div(k, 32), (unsigned)batch);
  spmm_generic_kernel<T><<<grid, kWarpsPerCta * 32, 0, st>>>(
      (int)m, (int)k, pos, crd, val, B, ldb, bias, relu, C, ldc, sv, sbb, sc);
  SB_LAUNCH_CHECK("spmm_generic_kernel");
  return SB_OK;
}

static int check_common(int64_t m, int64_t n, int64_t k, int64_t nnz, const void* pos,
                        const void* crd, const void* val, const void* B, int64_t ldb,
                        const void* C, int64_t ldc) {
  SB_CHECK_ARG(m >= 0 && n >= 0 && k >= 0 && nnz >= 0, "spmm: negative size");
  SB_CHECK_ARG(m < INT32_MAX && n < INT32_MAX && k < INT32_MAX, "spmm: dimension exceeds int32");
  if (nnz > INT32_MAX)
    return fail(SB_ERR_OVERFLOW, "spmm: nnz=%lld does not fit the int32 row pointers",
                (long long)nnz);
  SB_CHECK_ARG(pos, "spmm: pos is null");
  SB_CHECK_ARG(nnz == 0 || (crd && val), "spmm: crd/val is null");
  SB_CHECK_ARG(m == 0 || k == 0 || C, "spmm: C is null");
  SB_CHECK_ARG(nnz == 0 || k == 0 || B, "spmm: B is null");
  SB_CHECK_ARG(ldb >= k && ldc >= k, "spmm: leading dimension smaller than k");
  return SB_OK;
}

}  // namespace sb

using namespace sb;

extern "C" {

size_t sb_spmm_csr_scratch_bytes(int64_t segments, int64_t k, int64_t batch) {
  if (segments <= 0 || k <= 0 || batch <= 0) return 0;
  return (size_t)segments * (size_t)k * (size_t)batch * sizeof(float);
}

int sb_spmm_csr_f32(int64_t m, int64_t n, int64_t k, int64_t nnz, const int32_t* pos,
                    const int32_t* crd, const float* val, const float* B, int64_t ldb,
                    const float* bias, int relu, float* C, int64_t ldc, int64_t batch,
                    int64_t stride_val, int64_t stride_b, int64_t stride_c, const void* plan,
                    int64_t plan_segments, void* scratch, size_t scratch_bytes, void* stream) {
  int rc = check_common(m, n, k, nnz, pos, crd, val, B, ldb, C, ldc);
  if (rc != SB_OK) return rc;
  SB_CHECK_ARG(batch >= 1 && batch <= 65535, "spmm: batch must be in [1, 65535]");
  SB_CHECK_ARG(stride_val >= 0 && stride_b >= 0 && stride_c >= 0, "spmm: negative batch stride");
  if (m == 0 || k == 0) return SB_OK;
  cudaStream_t st = (cudaStream_t)stream;

  const bool vec_ok = (k % 4 == 0) && (ldb % 4 == 0) && (ldc % 4 == 0) && aligned16(B) &&
                      aligned16(C) && (!bias || aligned16(bias)) && (stride_b % 4 == 0) &&
                      (stride_c % 4 == 0);
  if (!vec_ok) {
    return launch_generic<float>(m, k, pos, crd, val, B, ldb, bias, relu, C, ldc, batch,
                                 stride_val, stride_b, stride_c, st);
  }
  if (plan) {
    SB_CHECK_ARG(aligned16(plan), "spmm: plan must be 16-byte aligned");
    const int64_t segs = plan_segments < 0 ? plan_cap_seg(nnz) : plan_segments;
    if (segs > 0) {
      SB_CHECK_ARG(scratch && aligned16(scratch), "spmm: scratch is null or misaligned");
      const size_t need = sb_spmm_csr_scratch_bytes(segs, k, batch);
      if (scratch_bytes < need)
        return fail(SB_ERR_WORKSPACE, "spmm: scratch has %zu bytes, needs %zu", scratch_bytes, need);
    }
  }
  SpmmArgs a;
  a.m = (int)m; a.k = (int)k; a.pos = pos; a.crd = crd; a.val = val; a.B = B; a.ldb = ldb;
  a.bias = bias; a.relu = relu; a.C = C; a.ldc = ldc;
  a.stride_val = stride_val; a.stride_b = stride_b; a.stride_c = stride_c;
  a.skip_heavy = (plan && plan_segments != 0) ? 1 : 0;
  if (k <= 16) return launch_vec<4, 1>(a, batch, plan, nnz, plan_segments, scratch, st);
  if (k <= 32) return launch_vec<8, 1>(a, batch, plan, nnz, plan_segments, scratch, st);
  if (k <= 64) return launch_vec<16, 1>(a, batch, plan, nnz, plan_segments, scratch, st);
  if (k <= 128) return launch_vec<32, 1>(a, batch, plan, nnz, plan_segments, scratch, st);
  if (k <= 256) return launch_vec<32, 2>(a, batch, plan, nnz, plan_segments, scratch, st);
  return launch_vec<32, 4>(a, batch, plan, nnz, plan_segments, scratch, st);
}

int sb_spmm_csr_typed(int dtype, int64_t m, int64_t n, int64_t k, int64_t nnz, const int32_t* pos,
                      const int32_t* crd, const void* val, const void* B, int64_t ldb, void* C,
                      int64_t ldc, void* stream) {
  int rc = check_common(m, n, k, nnz, pos, crd, val, B, ldb, C, ldc);
  if (rc != SB_OK) return rc;
  if (m == 0 || k == 0) return SB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case SB_F32:
      return sb_spmm_csr_f32(m, n, k, nnz, pos, crd, (const float*)val, (const float*)B, ldb,
                             nullptr, 0, (float*)C, ldc, 1, 0, 0, 0, nullptr, 0, nullptr, 0, stream);
    case SB_F64:
      return launch_generic<double>(m, k, pos, crd, (const double*)val, (const double*)B, ldb,
                                    nullptr, 0, (double*)C, ldc, 1, 0, 0, 0, st);
    case SB_I32:  // unsigned arithmetic: same bits as the reference's wrapping int32 math
      return launch_generic<unsigned int>(m, k, pos, crd, (const unsigned int*)val,
                                          (const unsigned int*)B, ldb, nullptr, 0,
                                          (unsigned int*)C, ldc, 1, 0, 0, 0, st);
    case SB_I64:
      return launch_generic<unsigned long long>(m, k, pos, crd, (const unsigned long long*)val,
                                                (const unsigned long long*)B, ldb, nullptr, 0,
                                                (unsigned long long*)C, ldc, 1, 0, 0, 0, st);
    default:
      return fail(SB_ERR_UNSUPPORTED, "spmm_typed: unknown dtype %d", dtype);
  }
}

}  // extern "C"
