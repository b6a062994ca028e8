// SDDMM (sampled dense-dense product) over the stored entries of a CSR or COO mask, and the row
// softmax over CSR values that sits between SDDMM and SpMM in sparse attention.
//
// SDDMM work split: the entry list is cut into spans of 8 x 32 consecutive entries, one warp per
// span, so the split is balanced by nnz whatever the row lengths are.  Per 32-entry chunk the
// warp reads the column ids / mask values with one coalesced load and finds each entry's row
// (one binary search per span, a short forward walk per chunk, a per-lane refinement only when
// a chunk crosses rows); then G lanes share each dot product: 128-bit loads of whole K-row lines,
// the Q row kept in registers while consecutive entries share it, and a transpose-reduce that
// costs about one shuffle per entry and leaves entry t of the chunk on lane t, so results are
// written back as one coalesced line per chunk.
#include <math.h>

#include "common.cuh"

// 128-bit K-row loads gathered together per lane (4 measured best on B200: 8 costs occupancy)
#ifndef SB_SDDMM_INFLIGHT
#define SB_SDDMM_INFLIGHT 4
#endif

namespace sb {

constexpr int kSddmmWarps = 8;

struct SddmmArgs {
  int m;
  int d;
  long long nnz;
  const int* pos;   // CSR mask (null for COO)
  const int* row;   // COO mask (null for CSR)
  const int* crd;
  int rowwise;            // one warp per row of pos[] (short rows) instead of one per entry span
  const int* ent;         // optional entry list: entry q of this launch is entry ent[q] of crd /
                          // mask_val / out_val (pos then describes the listed entries per row)
  int out_compact;        // the launch works on a compact list: crd and out_val are indexed by the
                          // list position q; ent (if given) only locates mask_val[ent[q]]
  const float* mask_val;  // may be null
  const float* Q;
  long long ldq;
  const float* K;
  long long ldk;
  float* out_val;
  int* out_row;  // optional fresh coordinates (CSR variant)
  int* out_col;
  long long stride_q, stride_k, stride_out;
};

// Row of entry p, searching forward from row r (pos[r] <= p): a few steps of linear walk (the
// common case: the next chunk starts in the same or the next row), then a bounded binary search.
__device__ __forceinline__ int advance_row(const int* __restrict__ pos, int m, int r, int p) {
#pragma unroll 1
  for (int t = 0; t < 4; t++) {
    if (__ldg(pos + r + 1) > p) return r;
    r++;
  }
  return row_of_entry(pos, r, m, p);
}

constexpr int kChunksPerWarp = 8;  // a warp owns 8 consecutive 32-entry chunks: one row search
constexpr int kRowsPerWarp = 4;   // row-wise launches: consecutive rows per warp (2, 8 measured slower)

// Sums G per-lane partial values for G entries across the G lanes of a group with G-1 shuffles
// (a butterfly that halves the number of live values per lane at every step).  On return lane l
// of the group holds, in v[0], the complete sum for entry l.
template <int G>
__device__ __forceinline__ void transpose_reduce(float (&v)[G], int lane) {
#pragma unroll
  for (int o = G / 2; o >= 1; o >>= 1) {
    const bool upper = (lane & o) != 0;
#pragma unroll
    for (int i = 0; i < o; i++) {
      const float send = upper ? v[i] : v[i + o];
      const float keep = upper ? v[i + o] : v[i];
      v[i] = keep + __shfl_xor_sync(FULL, send, o);
    }
  }
}

// Partial dot products of one full chunk whose 32 entries all share the Q row held in q[]: group
// entry t of this lane's group goes to part[t].
template <int G, int VEC, int HALF>
__device__ __forceinline__ void chunk_dots(float (&part)[G], const float4 (&q)[VEC], int my_j,
                                           const float* __restrict__ K, unsigned ldk, int g0,
                                           const bool (&col_ok)[VEC]) {
#pragma unroll
  for (int t0 = 0; t0 < G; t0 += HALF) {
    float4 kv[HALF][VEC];
#pragma unroll
    for (int u = 0; u < HALF; u++) {
      const int idx = g0 + t0 + u;
      const int j = __shfl_sync(FULL, my_j, idx);
      const float* krow = K + (size_t)((unsigned long long)(unsigned)j * ldk);
#pragma unroll
      for (int v = 0; v < VEC; v++)
        kv[u][v] = col_ok[v] ? ldg4(krow + v * G * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < HALF; u++) {
      float acc = 0.f;
#pragma unroll
      for (int v = 0; v < VEC; v++) acc = dot4(q[v], kv[u][v], acc);
      part[t0 + u] = acc;
    }
  }
}

// The last, partly filled chunk of a row (ROWWISE): its cnt < 32 entries are dealt round-robin to
// the 32/G groups (entry e -> group e % (32/G), slot e / (32/G)), so every group has work and the
// chunk costs ceil(cnt / (32/G)) slots instead of G.  After transpose_reduce lane l of group k
// owns entry l * (32/G) + k.
template <int G, int VEC, int HALF>
__device__ __forceinline__ void chunk_dots_tail(float (&part)[G], const float4 (&q)[VEC], int my_j,
                                                const float* __restrict__ K, unsigned ldk, int lane,
                                                int cnt, const bool (&col_ok)[VEC]) {
  constexpr int NG = 32 / G;
  const int grp = lane / G;
  const int nslots = (cnt + NG - 1) / NG;  // warp-uniform
#pragma unroll
  for (int t0 = 0; t0 < G; t0 += HALF) {
    if (t0 < nslots) {
      float4 kv[HALF][VEC];
#pragma unroll
      for (int u = 0; u < HALF; u++) {
        const int idx = (t0 + u) * NG + grp;  // <= 31
        const int j = __shfl_sync(FULL, my_j, idx);
        const float* krow = K + (size_t)((unsigned long long)(unsigned)j * ldk);
#pragma unroll
        for (int v = 0; v < VEC; v++)
          kv[u][v] = (idx < cnt && col_ok[v]) ? ldg4(krow + v * G * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < HALF; u++) {
        float acc = 0.f;
#pragma unroll
        for (int v = 0; v < VEC; v++) acc = dot4(q[v], kv[u][v], acc);
        part[t0 + u] = acc;
      }
    } else {
#pragma unroll
      for (int u = 0; u < HALF; u++) part[t0 + u] = 0.f;
    }
  }
}

// G lanes per dot product, VEC float4 of the Q/K row per lane (G*VEC*4 >= d; EXACT: == d, no
// column predicates).  A 32-entry chunk is handled as 32/G groups of G consecutive entries: a
// group gathers its G K rows (each row read by G adjacent lanes: whole 128-byte lines), forms G
// partial dots per lane and transpose-reduces them, after which lane t of the warp owns entry t
// of the chunk.  Full chunks that lie inside one mask row take a path without per-entry row
// bookkeeping or predicates.
// ROWWISE: one warp per kRowsPerWarp mask rows, row by row, instead of one per entry span (used
// for the short rows of a block plan's remainder list, where spans would cross a row boundary in
// almost every chunk).
// (row-wise launches: four CTAs per SM, 64 registers, measured 4 % faster than three)
template <int G, int VEC, bool EXACT, bool ROWWISE>
__global__ void __launch_bounds__(kSddmmWarps * 32, (VEC >= 4 || G >= 32) ? 2 : (ROWWISE ? 4 : 3))
sddmm_kernel(SddmmArgs a) {
  // K rows gathered together (8 and 16 loads in flight per lane were measured on the row-wise
  // launches too and lost to the occupancy they cost)
  constexpr int HALF = (SB_SDDMM_INFLIGHT / VEC < G) ? (SB_SDDMM_INFLIGHT / VEC) : G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long span = (long long)blockIdx.x * kSddmmWarps + warp;
  long long p0 = 0, p_end = 0;
  // row-wise: the warp takes kRowsPerWarp consecutive rows; their bounds and first index chunks
  // are fetched together, so the rows share one start-up latency instead of paying it each
  constexpr int R = ROWWISE ? kRowsPerWarp : 1;
  int pb = 0;                 // lane r <= R: pos[first row + r]
  int first_j[R];
  long long first_p[R];
  float first_s[R];
  if (ROWWISE) {
    const long long row_base = span * R;
    if (row_base >= a.m) return;
    if (lane <= R) pb = __ldg(a.pos + min(row_base + lane, (long long)a.m));
#pragma unroll
    for (int r = 0; r < R; r++) {
      const int b = __shfl_sync(FULL, pb, r), e = __shfl_sync(FULL, pb, r + 1);
      first_j[r] = 0; first_p[r] = 0; first_s[r] = 1.f;
      if (b + lane < e) {
        first_p[r] = a.ent ? (long long)ld_stream(a.ent + b + lane) : b + lane;
        first_j[r] = ld_stream(a.crd + (a.out_compact ? b + lane : first_p[r]));
        if (a.mask_val) first_s[r] = ld_stream(a.mask_val + first_p[r]);
      }
    }
  } else {
    p0 = span * (32 * kChunksPerWarp);
    if (p0 >= a.nnz) return;
    p_end = min(a.nnz, p0 + 32 * kChunksPerWarp);
  }
  const long long bz = blockIdx.y;
  const int g0 = (lane / G) * G, l = lane % G;  // first lane of my group, my slice of the row
  const float* Q = a.Q + bz * a.stride_q + l * 4;
  const float* K = a.K + bz * a.stride_k + l * 4;
  float* out = a.out_val + bz * a.stride_out;
  const unsigned ldq = (unsigned)a.ldq, ldk = (unsigned)a.ldk;  // row pitches fit 32 bits

  bool col_ok[VEC];
#pragma unroll
  for (int v = 0; v < VEC; v++) col_ok[v] = EXACT || (l + v * G) * 4 < a.d;
  float4 q[VEC];
#pragma unroll
  for (int v = 0; v < VEC; v++) q[v] = make_float4(0.f, 0.f, 0.f, 0.f);
  int q_row = -1;
  int r0 = ROWWISE ? 0 : (a.pos ? row_of_entry(a.pos, 0, a.m, (int)p0) : 0);

  auto load_q = [&](int row) {
    q_row = row;
    const float* qrow = Q + (size_t)((unsigned long long)(unsigned)row * ldq);
#pragma unroll
    for (int v = 0; v < VEC; v++)
      if (col_ok[v]) q[v] = ldg4(qrow + v * G * 4);
  };

  // software pipeline: the next chunk's entries are in flight while this chunk's K rows are
  // gathered
  int next_j = 0, next_i = 0;
  long long next_p = 0;
  float next_s = 1.f;
  if (!ROWWISE && p0 + lane < p_end) {
    next_p = a.ent ? (long long)ld_stream(a.ent + p0 + lane) : p0 + lane;
    next_j = ld_stream(a.crd + (a.out_compact ? p0 + lane : next_p));
    if (a.mask_val) next_s = ld_stream(a.mask_val + next_p);
    if (a.row) next_i = ld_stream(a.row + next_p);
  }
#pragma unroll 1
  for (int rr = 0; rr < R; rr++) {
  if (ROWWISE) {
    // this row's bounds and first chunk (select chains: the arrays stay in registers)
    p0 = __shfl_sync(FULL, pb, rr);
    p_end = __shfl_sync(FULL, pb, rr + 1);
    r0 = (int)(span * R) + rr;
#pragma unroll
    for (int r = 0; r < R; r++) {
      if (r == rr) { next_j = first_j[r]; next_p = first_p[r]; next_s = first_s[r]; }
    }
  }
#pragma unroll 1
  for (; p0 < p_end; p0 += 32) {
    const int cnt = (int)min((long long)32, p_end - p0);
    const int my_j = next_j;
    int my_i = next_i;
    const float my_s = next_s;
    const long long my_p = next_p;
    if (p0 + 32 + lane < p_end) {
      next_p = a.ent ? (long long)ld_stream(a.ent + p0 + 32 + lane) : p0 + 32 + lane;
      next_j = ld_stream(a.crd + (a.out_compact ? p0 + 32 + lane : next_p));
      if (a.mask_val) next_s = ld_stream(a.mask_val + next_p);
      if (a.row) next_i = ld_stream(a.row + next_p);
    }
    bool one_row = ROWWISE;  // warp-uniform: every entry of the chunk lies in row r0
    if (ROWWISE) {
      my_i = r0;
    } else if (a.pos) {
      r0 = advance_row(a.pos, a.m, r0, (int)p0);
      my_i = r0;
      one_row = __ldg(a.pos + r0 + 1) > (int)p0 + cnt - 1;
      if (!one_row) my_i = row_of_entry(a.pos, r0, a.m, (int)p0 + min(lane, cnt - 1));
    }
    if (bz == 0 && lane < cnt) {
      if (a.out_row) a.out_row[my_p] = my_i;
      if (a.out_col) a.out_col[my_p] = my_j;
    }

    float part[G];
    bool dealt = false;  // warp-uniform: the chunk's entries were dealt round-robin to the groups
    if (one_row && (ROWWISE || cnt == 32)) {
      // every entry of the chunk shares Q row r0
      if (r0 != q_row) load_q(r0);
      if (!ROWWISE || cnt == 32) {
        chunk_dots<G, VEC, HALF>(part, q, my_j, K, ldk, g0, col_ok);
      } else {
        if constexpr (ROWWISE) {
          chunk_dots_tail<G, VEC, HALF>(part, q, my_j, K, ldk, lane, cnt, col_ok);
          dealt = true;
        }
      }
    } else {
#pragma unroll 1
      for (int t = 0; t < G; t++) {
        const int idx = g0 + t;
        const unsigned j = (unsigned)__shfl_sync(FULL, my_j, idx);
        const int i = __shfl_sync(FULL, my_i, idx);
        float acc = 0.f;
        if (idx < cnt) {
          if (i != q_row) load_q(i);
          const float* krow = K + (size_t)((unsigned long long)j * ldk);
#pragma unroll
          for (int v = 0; v < VEC; v++)
            if (col_ok[v]) acc = dot4(q[v], ldg4(krow + v * G * 4), acc);
        }
        // part[] is indexed with compile-time constants only: scatter through a select chain
#pragma unroll
        for (int x = 0; x < G; x++) part[x] = (x == t) ? acc : part[x];
      }
    }
    transpose_reduce<G>(part, lane);
    if (ROWWISE && dealt) {
      const int e = l * (32 / G) + lane / G;  // the entry this lane owns
      const float s_e = __shfl_sync(FULL, my_s, e);
      const int p_e = __shfl_sync(FULL, (int)my_p, e);
      if (e < cnt) out[a.out_compact ? p0 + e : (long long)p_e] = s_e * part[0];
    } else if (lane < cnt) {
      out[a.out_compact ? p0 + lane : my_p] = my_s * part[0];
    }
  }
  }
}

// Any d / any alignment: one lane per entry, scalar loop over d.
__global__ void sddmm_generic_kernel(SddmmArgs a) {
  const long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= a.nnz) return;
  const long long bz = blockIdx.y;
  const int j = a.crd[p];
  const int i = a.row ? a.row[p] : row_of_entry(a.pos, 0, a.m, (int)p);
  const float* q = a.Q + bz * a.stride_q + (long long)i * a.ldq;
  const float* k = a.K + bz * a.stride_k + (long long)j * a.ldk;
  float acc = 0.f;
  for (int c = 0; c < a.d; c++) acc = fmaf(q[c], k[c], acc);
  a.out_val[bz * a.stride_out + p] = (a.mask_val ? a.mask_val[p] : 1.f) * acc;
  if (bz == 0) {
    if (a.out_row) a.out_row[p] = i;
    if (a.out_col) a.out_col[p] = j;
  }
}

template <int G, int VEC>
static int launch_sddmm(const SddmmArgs& a, int64_t batch, cudaStream_t st) {
  const bool exact = a.d == G * VEC * 4;
  if (a.rowwise && a.pos) {
    dim3 grid((unsigned)ceil_div(ceil_div(a.m, kRowsPerWarp), kSddmmWarps), (unsigned)batch);
    if (exact) sddmm_kernel<G, VEC, true, true><<<grid, kSddmmWarps * 32, 0, st>>>(a);
    else sddmm_kernel<G, VEC, false, true><<<grid, kSddmmWarps * 32, 0, st>>>(a);
  } else {
    const long long spans = ceil_div(a.nnz, 32 * kChunksPerWarp);
    dim3 grid((unsigned)ceil_div(spans, kSddmmWarps), (unsigned)batch);
    if (exact) sddmm_kernel<G, VEC, true, false><<<grid, kSddmmWarps * 32, 0, st>>>(a);
    else sddmm_kernel<G, VEC, false, false><<<grid, kSddmmWarps * 32, 0, st>>>(a);
  }
  SB_LAUNCH_CHECK("sddmm_kernel");
  return SB_OK;
}

static int sddmm_dispatch(SddmmArgs a, int64_t batch, cudaStream_t st) {
  if (a.nnz == 0) return SB_OK;
  const bool vec_ok = (a.d % 4 == 0) && (a.ldq % 4 == 0) && (a.ldk % 4 == 0) && aligned16(a.Q) &&
                      aligned16(a.K) && (a.stride_q % 4 == 0) && (a.stride_k % 4 == 0) &&
                      a.d <= 512 && a.ldq < (1ll << 32) && a.ldk < (1ll << 32);
  if (!vec_ok) {
    dim3 grid((unsigned)ceil_div(a.nnz, 256), (unsigned)batch);
    sddmm_generic_kernel<<<grid, 256, 0, st>>>(a);
    SB_LAUNCH_CHECK("sddmm_generic_kernel");
    return SB_OK;
  }
  // G lanes share one dot product, each holding VEC float4 of the Q row (G*VEC*4 >= d); G
  // adjacent lanes read G*16 contiguous bytes of a K row, i.e. whole 128-byte lines for d >= 32.
  if (a.d <= 16) return launch_sddmm<4, 1>(a, batch, st);
  if (a.d <= 32) return launch_sddmm<8, 1>(a, batch, st);
  if (a.d <= 64) return launch_sddmm<8, 2>(a, batch, st);
  if (a.d <= 128) return launch_sddmm<8, 4>(a, batch, st);
  if (a.d <= 256) return launch_sddmm<16, 4>(a, batch, st);
  return launch_sddmm<32, 4>(a, batch, st);
}

// ---- CSR row softmax ------------------------------------------------------------------------
constexpr int kSoftmaxRegs = 12;  // rows up to 32*12 = 384 entries stay in registers

__global__ void __launch_bounds__(256)
csr_row_softmax_kernel(int m, const int* __restrict__ pos, const float* in, float* out, float scale,
                       long long stride) {  // in == out is allowed: no __restrict__ on the pair
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  if (row >= m) return;
  const int b = __ldg(pos + row), e = __ldg(pos + row + 1);
  if (b == e) return;
  in += (long long)blockIdx.y * stride;
  out += (long long)blockIdx.y * stride;
  float v[kSoftmaxRegs];
  float mx = -INFINITY;
#pragma unroll
  for (int r = 0; r < kSoftmaxRegs; r++) {
    const int p = b + lane + 32 * r;
    v[r] = (p < e) ? in[p] * scale : -INFINITY;
    mx = fmaxf(mx, v[r]);
  }
  for (int p = b + lane + 32 * kSoftmaxRegs; p < e; p += 32) mx = fmaxf(mx, in[p] * scale);
  mx = group_max<32>(mx);
  float sum = 0.f;
#pragma unroll
  for (int r = 0; r < kSoftmaxRegs; r++) {
    const int p = b + lane + 32 * r;
    v[r] = (p < e) ? expf(v[r] - mx) : 0.f;
    sum += v[r];
  }
  for (int p = b + lane + 32 * kSoftmaxRegs; p < e; p += 32) sum += expf(in[p] * scale - mx);
  sum = group_sum<32>(sum);
  // tail first: it still needs the untouched input when in == out
  for (int p = b + lane + 32 * kSoftmaxRegs; p < e; p += 32)
    out[p] = expf(in[p] * scale - mx) / sum;
#pragma unroll
  for (int r = 0; r < kSoftmaxRegs; r++) {
    const int p = b + lane + 32 * r;
    if (p < e) out[p] = v[r] / sum;
  }
}

static int check_sddmm(int64_t m, int64_t n, int64_t d, int64_t nnz, const void* crd,
                       const void* Q, int64_t ldq, const void* K, int64_t ldk, const void* out,
                       int64_t batch) {
  SB_CHECK_ARG(m >= 0 && n >= 0 && d >= 0 && nnz >= 0, "sddmm: negative size");
  SB_CHECK_ARG(m < INT32_MAX && n < INT32_MAX && d < INT32_MAX, "sddmm: dimension exceeds int32");
  // (the kernels add up to one span, 256 entries, to an entry index held in an int)
  if (nnz > INT32_MAX - 4096)
    return fail(SB_ERR_OVERFLOW, "sddmm: nnz=%lld does not fit int32", (long long)nnz);
  SB_CHECK_ARG(nnz == 0 || (crd && out), "sddmm: null crd/out");
  SB_CHECK_ARG(nnz == 0 || d == 0 || (Q && K), "sddmm: null Q/K");
  SB_CHECK_ARG(ldq >= d && ldk >= d, "sddmm: leading dimension smaller than d");
  SB_CHECK_ARG(batch >= 1 && batch <= 65535, "sddmm: batch must be in [1, 65535]");
  return SB_OK;
}

// The entries of a mask that lie outside its dense blocks (blocked.cu): same kernel, entries
// taken through the list `rem_ent`, rows described by `rem_pos`.  The caller has checked that the
// operands qualify for the vector path.
int sddmm_remainder(int64_t m, int64_t d, int64_t rem_nnz, const int* rem_pos, const int* rem_ent,
                    const int* crd, const float* mask_val, const float* Q, int64_t ldq,
                    const float* K, int64_t ldk, float* out, int64_t batch, int64_t stride_q,
                    int64_t stride_k, int64_t stride_out, int out_compact, cudaStream_t st) {
  SddmmArgs a{(int)m, (int)d, rem_nnz, rem_pos, nullptr, crd, 1, rem_ent, out_compact, mask_val, Q, ldq, K, ldk, out,
              nullptr, nullptr, stride_q, stride_k, stride_out};
  return sddmm_dispatch(a, batch, st);
}

}  // namespace sb

using namespace sb;

extern "C" {

int sb_sddmm_csr_f32(int64_t m, int64_t n, int64_t d, int64_t nnz, const int32_t* pos,
                     const int32_t* crd, const float* mask_val, const float* Q, int64_t ldq,
                     const float* K, int64_t ldk, float* out_val, int32_t* out_row,
                     int32_t* out_col, int64_t batch, int64_t stride_q, int64_t stride_k,
                     int64_t stride_out, void* stream) {
  int rc = check_sddmm(m, n, d, nnz, crd, Q, ldq, K, ldk, out_val, batch);
  if (rc != SB_OK) return rc;
  SB_CHECK_ARG(pos, "sddmm_csr: pos is null");
  SddmmArgs a{(int)m, (int)d, nnz, pos, nullptr, crd, 0, nullptr, 0, mask_val, Q, ldq, K, ldk, out_val,
              out_row, out_col, stride_q, stride_k, stride_out};
  return sddmm_dispatch(a, batch, (cudaStream_t)stream);
}

int sb_sddmm_coo_f32(int64_t m, int64_t n, int64_t d, int64_t nnz, const int32_t* row,
                     const int32_t* col, const float* mask_val, const float* Q, int64_t ldq,
                     const float* K, int64_t ldk, float* out_val, int64_t batch, int64_t stride_q,
                     int64_t stride_k, int64_t stride_out, void* stream) {
  int rc = check_sddmm(m, n, d, nnz, col, Q, ldq, K, ldk, out_val, batch);
  if (rc != SB_OK) return rc;
  SB_CHECK_ARG(nnz == 0 || row, "sddmm_coo: row is null");
  SddmmArgs a{(int)m, (int)d, nnz, nullptr, row, col, 0, nullptr, 0, mask_val, Q, ldq, K, ldk, out_val,
              nullptr, nullptr, stride_q, stride_k, stride_out};
  return sddmm_dispatch(a, batch, (cudaStream_t)stream);
}

int sb_csr_row_softmax_f32(int64_t m, int64_t nnz, const int32_t* pos, const float* in, float* out,
                           float scale, int64_t batch, int64_t stride, void* stream) {
  SB_CHECK_ARG(m >= 0 && m < INT32_MAX && nnz >= 0, "softmax: bad size");
  if (nnz > INT32_MAX) return fail(SB_ERR_OVERFLOW, "softmax: nnz does not fit int32");
  SB_CHECK_ARG(batch >= 1 && batch <= 65535, "softmax: batch must be in [1, 65535]");
  if (m == 0 || nnz == 0) return SB_OK;
  SB_CHECK_ARG(pos && in && out, "softmax: null pointer");
  dim3 grid((unsigned)ceil_div(m, 8), (unsigned)batch);
  csr_row_softmax_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((int)m, pos, in, out, scale,
                                                                 stride);
  SB_LAUNCH_CHECK("csr_row_softmax_kernel");
  return SB_OK;
}

}  // extern "C"
