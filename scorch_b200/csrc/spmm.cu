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

// floats of the dense operand in flight per lane (32 = 128 bytes measured best on B200: 64 loses
// 25 % on the GCN layers to register pressure, 16 loses 4 % there)
#ifndef SB_SPMM_INFLIGHT
#define SB_SPMM_INFLIGHT 32
#endif

// mean stored entries per row below which a launch takes several rows per warp: 64 where the
// whole warp spans one column tile that covers the operand (128 < k <= 256: four rows per warp
// one after the other), 24 otherwise (narrow tiles, a row per lane group: a 4096-row, 41-per-row,
// 64-column product measured 16 us that way against 10 us with a warp per row; and wide operands
// taken in column panels)
#ifndef SB_SPMM_SHORT_ROW_MEAN
#define SB_SPMM_SHORT_ROW_MEAN 24
#endif
#ifndef SB_SPMM_SHORT_ROW_MEAN_FULL_WARP
#define SB_SPMM_SHORT_ROW_MEAN_FULL_WARP 64
#endif

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
  const int* ent;  // optional entry list: entry p of pos[] is entry ent[p] of crd / val
  int val_compact; // with ent: the value of listed entry p is val[p], not val[ent[p]]
  int accumulate;  // add to the existing contents of C (before bias / ReLU)
  int short_rows;  // many rows of a few dozen entries: several rows per warp
};

// W floats (4 = 128-bit, 8 = 256-bit) moved by one load/store instruction.
template <int W>
struct Pack {
  float v[W];
};

// Gather of a dense-operand row slice through the read-only path.  (An L2 evict-last policy on
// these loads was measured on the 4096-column configuration and lost 25 %: left out.)
template <int W>
__device__ __forceinline__ Pack<W> ld_dense(const float* p) {
  Pack<W> r;
  if constexpr (W == 8) {
    asm volatile("ld.global.nc.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]),
                   "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7])
                 : "l"(p));
  } else {
    asm volatile("ld.global.nc.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3])
                 : "l"(p));
  }
  return r;
}

// Streaming (evict-first) store of an output slice: written once, never re-read here.
template <int W>
__device__ __forceinline__ void st_stream(float* p, const Pack<W>& r) {
  if constexpr (W == 8)
    asm volatile("st.global.cs.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(r.v[0]),
                 "f"(r.v[1]), "f"(r.v[2]), "f"(r.v[3]), "f"(r.v[4]), "f"(r.v[5]), "f"(r.v[6]),
                 "f"(r.v[7])
                 : "memory");
  else
    asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(r.v[0]), "f"(r.v[1]),
                 "f"(r.v[2]), "f"(r.v[3])
                 : "memory");
}

// Accumulate entries [b, e) of one row into acc[] for this lane's columns.
// L lanes per group (each lane VEC packs of W floats, pack v at column (l + v*L)*W of the tile),
// G = 32/L groups; group g takes entries b+g, b+g+G, ...  EXACT: the tile has no ragged edge.
template <int L, int VEC, int W, bool EXACT>
__device__ __forceinline__ void accumulate_range(Pack<W> (&acc)[VEC], const int* __restrict__ crd,
                                                 const float* __restrict__ val,
                                                 const float* __restrict__ Bcol, unsigned ldb,
                                                 int b, int e, int lane, const bool (&col_ok)[VEC],
                                                 const int* __restrict__ ent = nullptr,
                                                 bool val_compact = false, bool have_first = false,
                                                 int first_j = 0, float first_a = 0.f) {
  constexpr int G = 32 / L;
  const int g = lane / L;
  // software pipeline: the next chunk's indices/values are in flight while this chunk's rows of
  // the dense operand are gathered (the caller may have fetched the first chunk already)
  int next_j = first_j;
  float next_a = first_a;
  if (!have_first && b + lane < e) {
    const int x = ent ? ld_stream(ent + b + lane) : b + lane;
    next_j = ld_stream(crd + x);
    next_a = ld_stream(val + (val_compact ? b + lane : x));
  }
  for (int p0 = b; p0 < e; p0 += 32) {
    const int cnt = min(32, e - p0);
    const int my_j = next_j;
    const float my_a = next_a;
    if (p0 + 32 + lane < e) {
      const int x = ent ? ld_stream(ent + p0 + 32 + lane) : p0 + 32 + lane;
      next_j = ld_stream(crd + x);
      next_a = ld_stream(val + (val_compact ? p0 + 32 + lane : x));
    }
    if (cnt == 32) {
      constexpr int STEPS = 32 / G;
      constexpr int UMAX = SB_SPMM_INFLIGHT / (VEC * W);  // floats in flight per lane
      constexpr int U = (STEPS < UMAX) ? STEPS : UMAX;
#pragma unroll 1
      for (int s0 = 0; s0 < STEPS; s0 += U) {
        float a[U];
        Pack<W> bv[U][VEC];
#pragma unroll
        for (int u = 0; u < U; u++) {
          const int t = (s0 + u) * G + g;
          const unsigned j = (unsigned)__shfl_sync(FULL, my_j, t);
          a[u] = __shfl_sync(FULL, my_a, t);
          const float* brow = Bcol + (size_t)((unsigned long long)j * ldb);
#pragma unroll
          for (int v = 0; v < VEC; v++) {
            if (EXACT || col_ok[v]) {
              bv[u][v] = ld_dense<W>(brow + v * L * W);
            } else {
#pragma unroll
              for (int w = 0; w < W; w++) bv[u][v].v[w] = 0.f;
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
#pragma unroll
          for (int v = 0; v < VEC; v++) {
#pragma unroll
            for (int w = 0; w < W; w++) acc[v].v[w] = fmaf(a[u], bv[u][v].v[w], acc[v].v[w]);
          }
        }
      }
    } else {
      // (batching these loads like the full chunk's, predicated on the count, measured slower)
      for (int t0 = 0; t0 < cnt; t0 += G) {
        const int t = t0 + g;
        const unsigned j = (unsigned)__shfl_sync(FULL, my_j, t & 31);
        const float a = __shfl_sync(FULL, my_a, t & 31);
        if (t < cnt) {
          const float* brow = Bcol + (size_t)((unsigned long long)j * ldb);
#pragma unroll
          for (int v = 0; v < VEC; v++) {
            if (EXACT || col_ok[v]) {
              const Pack<W> x = ld_dense<W>(brow + v * L * W);
#pragma unroll
              for (int w = 0; w < W; w++) acc[v].v[w] = fmaf(a, x.v[w], acc[v].v[w]);
            }
          }
        }
      }
    }
  }
}

template <int L, int VEC, int W>
__device__ __forceinline__ void reduce_groups(Pack<W> (&acc)[VEC]) {
#pragma unroll
  for (int o = L; o < 32; o <<= 1) {
#pragma unroll
    for (int v = 0; v < VEC; v++) {
#pragma unroll
      for (int w = 0; w < W; w++) acc[v].v[w] += __shfl_xor_sync(FULL, acc[v].v[w], o);
    }
  }
}

template <int W>
__device__ __forceinline__ Pack<W> epilogue(Pack<W> s, const float* bias, int col, int relu) {
  if (bias) {
#pragma unroll
    for (int w = 0; w < W; w += 4) {
      const float4 bb = ldg4(bias + col + w);
      s.v[w] += bb.x; s.v[w + 1] += bb.y; s.v[w + 2] += bb.z; s.v[w + 3] += bb.w;
    }
  }
  if (relu) {
#pragma unroll
    for (int w = 0; w < W; w++) s.v[w] = s.v[w] > 0.f ? s.v[w] : 0.f;
  }
  return s;
}

// One warp per R consecutive rows; grid = (row blocks, column tiles, batch).  R = 1 in general;
// launches over many short rows (the entries a block plan leaves outside its blocks) use R = 4:
// the rows' bounds and first index chunks are fetched together, so the rows share one start-up
// latency instead of paying it each.
constexpr int kShortRowsPerWarp = 4;  // (2 and 8 measured slower)
// (four CTAs per SM for the short-row form: 64 registers; five and three measured slower)
template <int L, int VEC, int W, bool EXACT, int R>
__device__ __forceinline__ void rows_body(const SpmmArgs& a, int block_x) {
  constexpr int TILE = L * W * VEC;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_base = (block_x * kWarpsPerCta + warp) * R;
  if (row_base >= a.m) return;
  const long long bz = blockIdx.z;
  const int l = lane % L;
  const int col0 = blockIdx.y * TILE + l * W;
  const float* val = a.val + bz * a.stride_val;
  bool col_ok[VEC];
#pragma unroll
  for (int v = 0; v < VEC; v++) col_ok[v] = EXACT || (col0 + v * L * W) < a.k;
  int pb = 0;  // lane r <= R: pos[row_base + r] (rows past the end read pos[m]: empty)
  if (lane <= R) pb = __ldg(a.pos + min(row_base + lane, a.m));
  int first_j[R];
  float first_a[R];
  if (R > 1) {
#pragma unroll
    for (int r = 0; r < R; r++) {
      const int b = __shfl_sync(FULL, pb, r), e = __shfl_sync(FULL, pb, r + 1);
      first_j[r] = 0;
      first_a[r] = 0.f;
      if (b + lane < e) {
        const int x = a.ent ? ld_stream(a.ent + b + lane) : b + lane;
        first_j[r] = ld_stream(a.crd + x);
        first_a[r] = ld_stream(val + (a.val_compact ? b + lane : x));
      }
    }
  }
#pragma unroll 1
  for (int rr = 0; rr < R; rr++) {
    const int row = row_base + rr;
    if (row >= a.m) break;
    const int b = __shfl_sync(FULL, pb, rr), e = __shfl_sync(FULL, pb, rr + 1);
    if (a.skip_heavy && e - b > SB_HEAVY_ROW_NNZ) continue;
    Pack<W> acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; v++) {
#pragma unroll
      for (int w = 0; w < W; w++) acc[v].v[w] = 0.f;
    }
    float* crow = a.C + bz * a.stride_c + (long long)row * a.ldc;
    if (a.accumulate && lane < L) {
      // the row's present contents start the first lane group's sums: the load overlaps the
      // index loads and gathers instead of sitting between the reduction and the store
#pragma unroll
      for (int v = 0; v < VEC; v++) {
        if (!col_ok[v]) continue;
#pragma unroll
        for (int w = 0; w < W; w += 4) {
          const float4 old = *reinterpret_cast<const float4*>(crow + col0 + v * L * W + w);
          acc[v].v[w] = old.x; acc[v].v[w + 1] = old.y; acc[v].v[w + 2] = old.z; acc[v].v[w + 3] = old.w;
        }
      }
    }
    int fj = 0;
    float fa = 0.f;
    if (R > 1) {
#pragma unroll
      for (int r = 0; r < R; r++) {
        if (r == rr) { fj = first_j[r]; fa = first_a[r]; }
      }
    }
    accumulate_range<L, VEC, W, EXACT>(acc, a.crd, val, a.B + bz * a.stride_b + col0, (unsigned)a.ldb,
                                             b, e, lane, col_ok, a.ent, a.val_compact != 0, R > 1, fj, fa);
    reduce_groups<L, VEC, W>(acc);
    if (lane < L) {
#pragma unroll
      for (int v = 0; v < VEC; v++) {
        const int col = col0 + v * L * W;
        if (!col_ok[v]) continue;
        st_stream<W>(crow + col, epilogue<W>(acc[v], a.bias, col, a.relu));
      }
    }
  }
}

template <int L, int VEC, int W, bool EXACT, int R>
__global__ void __launch_bounds__(kWarpsPerCta * 32, R > 1 ? 4 : 1)
spmm_rows_kernel(SpmmArgs a) {
  rows_body<L, VEC, W, EXACT, R>(a, (int)blockIdx.x);
}

// Short rows, narrow tiles (L <= 16 lanes span the tile): each of the 32/L lane groups of a warp
// takes a row of its own, so a warp works on 32/L rows at once and no sums cross lanes.  A group
// reads its row's indices/values L at a time and keeps SB_SPMM_INFLIGHT floats of gathered
// operand rows in flight per lane.  Rows longer than kGroupedMaxRow (but not heavy) are done by
// the whole warp afterwards, like the general kernel does.
#ifndef SB_SPMM_GROUPED_MAX_ROW
#define SB_SPMM_GROUPED_MAX_ROW 64
#endif
constexpr int kGroupedMaxRow = SB_SPMM_GROUPED_MAX_ROW;

template <int L, int W, bool EXACT>
__device__ __forceinline__ void rows_grouped_body(const SpmmArgs& a, int block_x) {
  constexpr int G = 32 / L;
  constexpr int TILE = L * W;
  constexpr int UMAX = SB_SPMM_INFLIGHT / W;
  constexpr int U = (L < UMAX) ? L : UMAX;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_base = (block_x * kWarpsPerCta + warp) * G;
  if (row_base >= a.m) return;
  const int g = lane / L, l = lane % L;
  const int row = row_base + g;
  const long long bz = blockIdx.z;
  const float* val = a.val + bz * a.stride_val;
  const int col0 = blockIdx.y * TILE + l * W;
  const bool col_ok = EXACT || col0 < a.k;
  const float* Bcol = a.B + bz * a.stride_b + col0;
  const unsigned ldb = (unsigned)a.ldb;
  int b = 0, e = 0;
  if (row < a.m) {
    b = __ldg(a.pos + row);
    e = __ldg(a.pos + row + 1);
  }
  const bool heavy = a.skip_heavy && (e - b) > SB_HEAVY_ROW_NNZ;
  const bool by_warp = !heavy && (e - b) > kGroupedMaxRow;
  const bool mine = row < a.m && !heavy && !by_warp;
  const int ge = mine ? e : b;
  float* crow = a.C + bz * a.stride_c + (long long)row * a.ldc;
  Pack<W> acc;
#pragma unroll
  for (int w = 0; w < W; w++) acc.v[w] = 0.f;
  if (a.accumulate && mine && col_ok) {
#pragma unroll
    for (int w = 0; w < W; w += 4) {
      const float4 old = *reinterpret_cast<const float4*>(crow + col0 + w);
      acc.v[w] = old.x; acc.v[w + 1] = old.y; acc.v[w + 2] = old.z; acc.v[w + 3] = old.w;
    }
  }
  const int longest = __reduce_max_sync(FULL, ge - b);
  int next_j = 0;
  float next_a = 0.f;
  if (b + l < ge) {
    const int x = a.ent ? ld_stream(a.ent + b + l) : b + l;
    next_j = ld_stream(a.crd + x);
    next_a = ld_stream(val + (a.val_compact ? b + l : x));
  }
#pragma unroll 1
  for (int q0 = 0; q0 < longest; q0 += L) {
    const int p0 = b + q0;
    const int my_j = next_j;
    const float my_a = next_a;
    if (p0 + L + l < ge) {
      const int x = a.ent ? ld_stream(a.ent + p0 + L + l) : p0 + L + l;
      next_j = ld_stream(a.crd + x);
      next_a = ld_stream(val + (a.val_compact ? p0 + L + l : x));
    }
    const int cnt = ge - p0;                    // entries this group still has (may be <= 0)
    const int most = min(L, longest - q0);      // warp-uniform
#pragma unroll 1
    for (int t0 = 0; t0 < most; t0 += U) {
      float av[U];
      Pack<W> bv[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int t = t0 + u;
        const unsigned j = (unsigned)__shfl_sync(FULL, my_j, t, L);
        av[u] = __shfl_sync(FULL, my_a, t, L);
        if (t < cnt && col_ok) {
          bv[u] = ld_dense<W>(Bcol + (size_t)((unsigned long long)j * ldb));
        } else {
          av[u] = 0.f;
#pragma unroll
          for (int w = 0; w < W; w++) bv[u].v[w] = 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
#pragma unroll
        for (int w = 0; w < W; w++) acc.v[w] = fmaf(av[u], bv[u].v[w], acc.v[w]);
      }
    }
  }
  if (mine && col_ok) st_stream<W>(crow + col0, epilogue<W>(acc, a.bias, col0, a.relu));
  // rows too long for one lane group: the whole warp, one row after the other
  if (__any_sync(FULL, by_warp)) {
#pragma unroll 1
    for (int gg = 0; gg < G; gg++) {
      if (!__shfl_sync(FULL, (int)by_warp, gg * L)) continue;
      const int rb = __shfl_sync(FULL, b, gg * L), re = __shfl_sync(FULL, e, gg * L);
      Pack<W> acc2[1];
      bool ok2[1] = {col_ok};
#pragma unroll
      for (int w = 0; w < W; w++) acc2[0].v[w] = 0.f;
      float* crow2 = a.C + bz * a.stride_c + (long long)(row_base + gg) * a.ldc;
      if (a.accumulate && lane < L && col_ok) {
#pragma unroll
        for (int w = 0; w < W; w += 4) {
          const float4 old = *reinterpret_cast<const float4*>(crow2 + col0 + w);
          acc2[0].v[w] = old.x; acc2[0].v[w + 1] = old.y; acc2[0].v[w + 2] = old.z; acc2[0].v[w + 3] = old.w;
        }
      }
      accumulate_range<L, 1, W, EXACT>(acc2, a.crd, val, Bcol, ldb, rb, re, lane, ok2, a.ent,
                                       a.val_compact != 0);
      reduce_groups<L, 1, W>(acc2);
      if (lane < L && col_ok) st_stream<W>(crow2 + col0, epilogue<W>(acc2[0], a.bias, col0, a.relu));
    }
  }
}

template <int L, int W, bool EXACT>
__global__ void __launch_bounds__(kWarpsPerCta * 32, 4)
spmm_rows_grouped_kernel(SpmmArgs a) {
  rows_grouped_body<L, W, EXACT>(a, (int)blockIdx.x);
}

struct HeavyArgs {
  const int* hdr;
  const int* heavy_row;
  const int* heavy_seg0;
  const int* heavy_nseg;
  const int* seg_heavy;
  float* scratch;            // [batch][segments][k] segment sums of multi-segment rows
  long long scratch_batch;   // elements between batch items
  int* arrived;              // [batch][column tiles][segments] segments done per heavy row (zeroed)
  int segments;              // heavy CTAs in grid.x (>= the plan's segment count)
  int first_heavy;           // blockIdx.x of the first heavy CTA; the row CTAs take the other indices
};

// One CTA per heavy-row segment.  The CTA that finishes a row's last outstanding segment adds
// the row's segment sums in segment order and writes the row (fixed order, whichever CTA does it).
template <int L, int VEC, int W, bool EXACT>
__device__ __forceinline__ void heavy_body(const SpmmArgs& a, const HeavyArgs& h, int seg) {
  constexpr int TILE = L * W * VEC;
  __shared__ Pack<W> part[kWarpsPerCta][VEC][L];
  __shared__ int s_last;
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
  const int col0 = blockIdx.y * TILE + l * W;
  bool col_ok[VEC];
  Pack<W> acc[VEC];
#pragma unroll
  for (int v = 0; v < VEC; v++) {
    col_ok[v] = EXACT || (col0 + v * L * W) < a.k;
#pragma unroll
    for (int w = 0; w < W; w++) acc[v].v[w] = 0.f;
  }
  // each warp owns a contiguous slice of the segment (a multiple of 32 entries)
  constexpr int SLICE = SB_HEAVY_ROW_NNZ / kWarpsPerCta;
  const int wb = min(se, sb_ + warp * SLICE), we = min(se, wb + SLICE);
  accumulate_range<L, VEC, W, EXACT>(acc, a.crd, a.val + bz * a.stride_val,
                                           a.B + bz * a.stride_b + col0, (unsigned)a.ldb, wb, we,
                                           lane, col_ok);
  reduce_groups<L, VEC, W>(acc);
  if (lane < L) {
#pragma unroll
    for (int v = 0; v < VEC; v++) part[warp][v][l] = acc[v];
  }
  __syncthreads();
  if (warp == 0 && lane < L) {
#pragma unroll
    for (int v = 0; v < VEC; v++) {
      Pack<W> s = part[0][v][l];
#pragma unroll
      for (int w2 = 1; w2 < kWarpsPerCta; w2++) {
        const Pack<W> t = part[w2][v][l];
#pragma unroll
        for (int w = 0; w < W; w++) s.v[w] += t.v[w];
      }
      const int col = col0 + v * L * W;
      if (!col_ok[v]) continue;
      if (nseg == 1) {
        float* dst = a.C + bz * a.stride_c + (long long)row * a.ldc + col;
        if (a.accumulate) {
#pragma unroll
          for (int w = 0; w < W; w += 4) {
            const float4 old = *reinterpret_cast<const float4*>(dst + w);
            s.v[w] += old.x; s.v[w + 1] += old.y; s.v[w + 2] += old.z; s.v[w + 3] += old.w;
          }
        }
        st_stream<W>(dst, epilogue<W>(s, a.bias, col, a.relu));
      } else {
        float* dst = h.scratch + bz * h.scratch_batch + (long long)seg * a.k + col;
#pragma unroll
        for (int w = 0; w < W; w += 4)
          *reinterpret_cast<float4*>(dst + w) = make_float4(s.v[w], s.v[w + 1], s.v[w + 2], s.v[w + 3]);
        __threadfence();  // the segment sum is visible before this CTA counts itself done
      }
    }
  }
  if (nseg == 1) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    int* cnt = h.arrived + ((long long)bz * gridDim.y + blockIdx.y) * h.segments + seg0;
    s_last = (atomicAdd(cnt, 1) == nseg - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* src = h.scratch + bz * h.scratch_batch + (long long)seg0 * a.k;
  float* crow = a.C + bz * a.stride_c + (long long)row * a.ldc;
  const int tile0 = blockIdx.y * TILE;
  for (int c = threadIdx.x * 4; c < TILE; c += blockDim.x * 4) {
    const int col = tile0 + c;
    if (col >= a.k) break;
    Pack<4> s;
    s.v[0] = s.v[1] = s.v[2] = s.v[3] = 0.f;
    if (a.accumulate) {
      const float4 old = *reinterpret_cast<const float4*>(crow + col);
      s.v[0] = old.x; s.v[1] = old.y; s.v[2] = old.z; s.v[3] = old.w;
    }
    for (int t = 0; t < nseg; t++) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (long long)t * a.k + col));
      s.v[0] += v.x; s.v[1] += v.y; s.v[2] += v.z; s.v[3] += v.w;
    }
    st_stream<4>(crow + col, epilogue<4>(s, a.bias, col, a.relu));
  }
}

// Rows and heavy-row segments in one launch; grid = (row blocks + segments, column tiles, batch):
// the segment CTAs [first_heavy, first_heavy + segments) run beside the row CTAs instead of
// waiting for a launch of their own.
// (Both bodies inlined want 76-96 registers; three CTAs per SM, like the rows kernel alone gets,
// caps that at 85.)
template <int L, int VEC, int W, bool EXACT, int R>
__global__ void __launch_bounds__(kWarpsPerCta * 32, R > 1 ? 4 : 3)
spmm_rows_heavy_kernel(SpmmArgs a, HeavyArgs h) {
  const int hb = (int)blockIdx.x - h.first_heavy;
  if (hb >= 0 && hb < h.segments)
    heavy_body<L, VEC, W, EXACT>(a, h, hb);
  else
    rows_body<L, VEC, W, EXACT, R>(a, hb < 0 ? (int)blockIdx.x : hb - h.segments + h.first_heavy);
}

template <int L, int W, bool EXACT>
__global__ void __launch_bounds__(kWarpsPerCta * 32, 4)
spmm_grouped_heavy_kernel(SpmmArgs a, HeavyArgs h) {
  const int hb = (int)blockIdx.x - h.first_heavy;
  if (hb >= 0 && hb < h.segments)
    heavy_body<L, 1, W, EXACT>(a, h, hb);
  else
    rows_grouped_body<L, W, EXACT>(a, hb < 0 ? (int)blockIdx.x : hb - h.segments + h.first_heavy);
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

template <int L, int VEC, int W, bool EXACT>
static int launch_vec2(const SpmmArgs& a, int64_t batch, const void* plan, int64_t nnz,
                       int64_t plan_segments, void* scratch, cudaStream_t st) {
  constexpr int TILE = L * W * VEC;
  const unsigned tiles = (unsigned)ceil_div(a.k, TILE);
  // short rows: a row per lane group where the tile is narrow, else several rows per warp
  constexpr bool kGrouped = (L <= 16 && VEC == 1);
  const int rows_per_warp = !a.short_rows ? 1 : (kGrouped ? 32 / L : kShortRowsPerWarp);
  const int64_t row_ctas = ceil_div(ceil_div(a.m, rows_per_warp), kWarpsPerCta);
  if (plan && plan_segments != 0) {
    PlanView pv = plan_view(plan, nnz);
    const int64_t segs = plan_segments < 0 ? pv.cap_seg : plan_segments;
    float* sums = static_cast<float*>(scratch);
    int* arrived = reinterpret_cast<int*>(sums + (size_t)segs * a.k * batch);
    HeavyArgs h{pv.hdr, pv.heavy_row, pv.heavy_seg0, pv.heavy_nseg, pv.seg_heavy,
                sums, (long long)segs * a.k, arrived, (int)segs, 0};
    SB_CUDA(cudaMemsetAsync(arrived, 0, (size_t)segs * tiles * batch * sizeof(int), st));
    // Long rows: the rows in a launch of their own, then the segments (one launch with both
    // bodies needs 10-20 more registers per thread and measured 3 % / 20 % slower at 256 / 64
    // columns on a 2 M-row power-law graph).  Short-row passes (a row chunk's share of a
    // matrix: few segments, a launch of their own would leave most SMs idle): one launch, the
    // segment CTAs behind the row CTAs (4 % faster than in front at 256 columns).
    int64_t fused_rows = row_ctas;
    if (!a.short_rows) {
      dim3 rgrid((unsigned)row_ctas, tiles, (unsigned)batch);
      spmm_rows_kernel<L, VEC, W, EXACT, 1><<<rgrid, kWarpsPerCta * 32, 0, st>>>(a);
      SB_LAUNCH_CHECK("spmm_rows_kernel");
      fused_rows = 0;
    }
    h.first_heavy = (int)fused_rows;
    dim3 grid((unsigned)(segs + fused_rows), tiles, (unsigned)batch);
    if (a.short_rows) {
      if constexpr (kGrouped)
        spmm_grouped_heavy_kernel<L, W, EXACT><<<grid, kWarpsPerCta * 32, 0, st>>>(a, h);
      else
        spmm_rows_heavy_kernel<L, VEC, W, EXACT, kShortRowsPerWarp><<<grid, kWarpsPerCta * 32, 0, st>>>(a, h);
    } else
      spmm_rows_heavy_kernel<L, VEC, W, EXACT, 1><<<grid, kWarpsPerCta * 32, 0, st>>>(a, h);
    SB_LAUNCH_CHECK("spmm_rows_heavy_kernel");
    return SB_OK;
  }
  dim3 grid((unsigned)row_ctas, tiles, (unsigned)batch);
  if (a.short_rows) {
    if constexpr (kGrouped)
      spmm_rows_grouped_kernel<L, W, EXACT><<<grid, kWarpsPerCta * 32, 0, st>>>(a);
    else
      spmm_rows_kernel<L, VEC, W, EXACT, kShortRowsPerWarp><<<grid, kWarpsPerCta * 32, 0, st>>>(a);
  } else
    spmm_rows_kernel<L, VEC, W, EXACT, 1><<<grid, kWarpsPerCta * 32, 0, st>>>(a);
  SB_LAUNCH_CHECK("spmm_rows_kernel");
  return SB_OK;
}

template <int L, int VEC, int W>
static int launch_vec(const SpmmArgs& a, int64_t batch, const void* plan, int64_t nnz,
                      int64_t plan_segments, void* scratch, cudaStream_t st) {
  if (a.k % (L * W * VEC) == 0)
    return launch_vec2<L, VEC, W, true>(a, batch, plan, nnz, plan_segments, scratch, st);
  return launch_vec2<L, VEC, W, false>(a, batch, plan, nnz, plan_segments, scratch, st);
}

template <typename T>
static int launch_generic(int64_t m, int64_t k, const int32_t* pos, const int32_t* crd,
                          const T* val, const T* B, int64_t ldb, const T* bias, int relu, T* C,
                          int64_t ldc, int64_t batch, int64_t sv, int64_t sbb, int64_t sc,
                          cudaStream_t st) {
  if (ceil_div(k, 32) > 65535)
    return fail(SB_ERR_UNSUPPORTED,
                "spmm: the scalar path (dtype other than f32, or unaligned operands) takes at most "
                "%d columns, got %lld", 65535 * 32, (long long)k);
  dim3 grid((unsigned)ceil_div(m, kWarpsPerCta), (unsigned)ceil_div(k, 32), (unsigned)batch);
  spmm_generic_kernel<T><<<grid, kWarpsPerCta * 32, 0, st>>>(
      (int)m, (int)k, pos, crd, val, B, ldb, bias, relu, C, ldc, sv, sbb, sc);
  SB_LAUNCH_CHECK("spmm_generic_kernel");
  return SB_OK;
}

// Picks the vector kernel for k and the operands' alignment (the caller has checked the 128-bit
// requirements).
static int spmm_vec_dispatch(const SpmmArgs& a, int64_t k, int64_t ldb, int64_t ldc, int64_t stride_b,
                             int64_t stride_c, const float* B, const float* C, int64_t batch,
                             const void* plan, int64_t nnz, int64_t plan_segments, void* scratch,
                             cudaStream_t st) {
  // 256-bit loads (8 floats per lane) when every row slice is 32-byte aligned, else 128-bit.
  const bool wide_ok = (k % 8 == 0) && (ldb % 8 == 0) && (ldc % 8 == 0) && (stride_b % 8 == 0) &&
                       (stride_c % 8 == 0) && ((reinterpret_cast<uintptr_t>(B) & 31u) == 0) &&
                       ((reinterpret_cast<uintptr_t>(C) & 31u) == 0);
#define SB_GO(L, VEC, W) \
  return launch_vec<L, VEC, W>(a, batch, plan, nnz, plan_segments, scratch, st)
  if (wide_ok) {
    if (k <= 32) SB_GO(4, 1, 8);
    if (k <= 64) SB_GO(8, 1, 8);
    if (k <= 128) SB_GO(16, 1, 8);
    // wider operands: 256-column panels on grid.y (a 32768-row panel = 32 MB stays in L2 while
    // all row blocks pass over it; 128- and 512-column panels measured slower)
    SB_GO(32, 1, 8);
  }
  if (k <= 16) SB_GO(4, 1, 4);
  if (k <= 32) SB_GO(8, 1, 4);
  if (k <= 64) SB_GO(16, 1, 4);
  if (k <= 128) SB_GO(32, 1, 4);
  SB_GO(32, 2, 4);
#undef SB_GO
}

// Rows of the entries outside the dense blocks of a block plan (blocked.cu): C += A_rem B, then
// bias / ReLU.  Entries are taken through the list `rem_ent`; no heavy-row split (the blocked
// path is only offered for matrices without heavy rows).
int spmm_remainder(int64_t m, int64_t k, const int* rem_pos, const int* rem_ent, const int* crd,
                   const float* val, const float* B, int64_t ldb, const float* bias, int relu,
                   float* C, int64_t ldc, int64_t batch, int64_t stride_val, int64_t stride_b,
                   int64_t stride_c, int val_compact, cudaStream_t st) {
  SpmmArgs a;
  a.m = (int)m; a.k = (int)k; a.pos = rem_pos; a.crd = crd; a.val = val; a.B = B; a.ldb = ldb;
  a.bias = bias; a.relu = relu; a.C = C; a.ldc = ldc;
  a.stride_val = stride_val; a.stride_b = stride_b; a.stride_c = stride_c;
  a.skip_heavy = 0; a.ent = rem_ent; a.val_compact = val_compact; a.accumulate = 1; a.short_rows = 1;
  return spmm_vec_dispatch(a, k, ldb, ldc, stride_b, stride_c, B, C, batch, nullptr, 0, 0, nullptr, st);
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
  // segment sums + one arrival counter per (segment, column tile of at most 256 columns)
  const size_t tiles = (size_t)ceil_div(k, 16);
  return (size_t)segments * (size_t)batch * ((size_t)k * sizeof(float) + tiles * sizeof(int));
}

static int spmm_csr_f32_impl(int64_t m, int64_t n, int64_t k, int64_t nnz, const int32_t* pos,
                             const int32_t* crd, const float* val, const float* B, int64_t ldb,
                             const float* bias, int relu, float* C, int64_t ldc, int64_t batch,
                             int64_t stride_val, int64_t stride_b, int64_t stride_c,
                             const void* plan, int64_t plan_segments, void* scratch,
                             size_t scratch_bytes, int accumulate, void* stream) {
  int rc = check_common(m, n, k, nnz, pos, crd, val, B, ldb, C, ldc);
  if (rc != SB_OK) return rc;
  SB_CHECK_ARG(batch >= 1 && batch <= 65535, "spmm: batch must be in [1, 65535]");
  SB_CHECK_ARG(stride_val >= 0 && stride_b >= 0 && stride_c >= 0, "spmm: negative batch stride");
  if (m == 0 || k == 0) return SB_OK;
  cudaStream_t st = (cudaStream_t)stream;

  const bool vec_ok = (k % 4 == 0) && (ldb % 4 == 0) && (ldc % 4 == 0) && aligned16(B) &&
                      aligned16(C) && (!bias || aligned16(bias)) && (stride_b % 4 == 0) &&
                      (stride_c % 4 == 0) && ldb < (1ll << 32);
  if (!vec_ok) {
    if (accumulate)
      return fail(SB_ERR_UNSUPPORTED,
                  "spmm: accumulation needs the vector layout (k, ldb, ldc multiples of 4; B, C "
                  "16-byte aligned)");
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
  // wide operands, no heavy rows: optionally the bulk-copy kernel of spmm_wide.cu
  if (k >= 512 && batch == 1 && !accumulate && !(plan && plan_segments != 0) && spmm_wide_wanted())
    return spmm_wide_launch(m, k, pos, crd, val, B, ldb, bias, relu, C, ldc, st);
  SpmmArgs a;
  a.m = (int)m; a.k = (int)k; a.pos = pos; a.crd = crd; a.val = val; a.B = B; a.ldb = ldb;
  a.bias = bias; a.relu = relu; a.C = C; a.ldc = ldc;
  a.stride_val = stride_val; a.stride_b = stride_b; a.stride_c = stride_c;
  a.skip_heavy = (plan && plan_segments != 0) ? 1 : 0;
  a.ent = nullptr;
  a.val_compact = 0;
  a.accumulate = accumulate ? 1 : 0;
  // many short rows (e.g. one row chunk's share of a matrix): several rows per warp
  a.short_rows = (nnz < (int64_t)((k > 128 && k <= 256) ? SB_SPMM_SHORT_ROW_MEAN_FULL_WARP
                                                        : SB_SPMM_SHORT_ROW_MEAN) * m) ? 1 : 0;
  return spmm_vec_dispatch(a, k, ldb, ldc, stride_b, stride_c, B, C, batch, plan, nnz, plan_segments, scratch, st);
}

int sb_spmm_csr_f32(int64_t m, int64_t n, int64_t k, int64_t nnz, const int32_t* pos,
                    const int32_t* crd, const float* val, const float* B, int64_t ldb,
                    const float* bias, int relu, float* C, int64_t ldc, int64_t batch,
                    int64_t stride_val, int64_t stride_b, int64_t stride_c, const void* plan,
                    int64_t plan_segments, void* scratch, size_t scratch_bytes, void* stream) {
  return spmm_csr_f32_impl(m, n, k, nnz, pos, crd, val, B, ldb, bias, relu, C, ldc, batch,
                           stride_val, stride_b, stride_c, plan, plan_segments, scratch,
                           scratch_bytes, 0, stream);
}

int sb_spmm_csr_acc_f32(int64_t m, int64_t n, int64_t k, int64_t nnz, const int32_t* pos,
                        const int32_t* crd, const float* val, const float* B, int64_t ldb,
                        const float* bias, int relu, float* C, int64_t ldc, int64_t batch,
                        int64_t stride_val, int64_t stride_b, int64_t stride_c, const void* plan,
                        int64_t plan_segments, void* scratch, size_t scratch_bytes, void* stream) {
  return spmm_csr_f32_impl(m, n, k, nnz, pos, crd, val, B, ldb, bias, relu, C, ldc, batch,
                           stride_val, stride_b, stride_c, plan, plan_segments, scratch,
                           scratch_bytes, 1, stream);
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
