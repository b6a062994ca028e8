// Sparse attention over a CSR mask in one pass over the mask's blocks:
//   O = softmax_rows(scale * mask_val .* (Q K^T) on the stored entries) V
// which the reference's caller runs as three operators with the scores in memory in between
// (bench/bench_sparse_transformer.py:304-382: SDDMM, row softmax, SpMM per head).
//
// An attention plan splits the mask, once, into
//   * the aligned 16x16 blocks that hold at least kMinBlockEntries stored entries (the fully
//     stored blocks of a band and the half-filled ones along its edges), each with a 16-bit mask
//     of the stored columns per row, and
//   * a CSR list of the remaining entries (the scattered ones).
// A call then runs two kernels:
//   1. attn_scattered_kernel over the remaining entries, a lane group per row: gather the K row,
//      dot product with the row's Q (held in registers), running row maximum / sum, gather the V
//      row and accumulate exp(score - max) V.  Per row it leaves the unnormalised sum in O and
//      (max, sum) in a small scratch array; no score is written anywhere;
//   2. attn_block_kernel, one warp per 16 mask rows, which starts its running maximum / sum and
//      its O accumulators from what kernel 1 left for the same rows and continues over the
//      blocks of the row block: S = Q K^T on the tensor cores, entries that are not stored masked
//      to -inf, P = exp(S - max), O += P V on the tensor cores; at the end O / sum is written.
//      The scores of the blocks never leave the registers.
// Arithmetic of the blocks: mma.sync m16n8k8 TF32 with the 3xTF32 split (fp32-level accuracy).
#include <math.h>

#include <algorithm>

#include "attention.cuh"
#include "common.cuh"
#include "mma_tf32.cuh"

namespace sb {

constexpr int kMinBlockEntries = SB_ATTN_MIN_BLOCK_ENTRIES;
constexpr int kDetectSlots = 1024;  // per-warp hash slots for counting entries per column block

// ---- plan layout -----------------------------------------------------------------------------------
// int32 words: hdr[16] ([0] blocks, [1] remainder entries), then
//   rb_ptr[RB+1]      blocks of row block b are [rb_ptr[b], rb_ptr[b+1])
//   blk_col[capB]     column block of each block
//   blk_ent[capB*16]  entry index of the first stored entry of (row r of the block)
//   blk_mask[capB*16] stored columns of (row r of the block), bit c = column 16*blk_col + c
//   rem_pos[m+1], rem_ent[nnz], rem_crd[nnz]   CSR of the entries outside the blocks: entry index
//                     in the mask and column (a copy, so the gather kernels need not go through
//                     rem_ent to find it)
//   cnt[max(RB, m)+1] scratch for the counts, block_sum scan temporaries, total (int64)
struct AttnPlan {
  int* hdr;
  int* rb_ptr;
  int* blk_col;
  int* blk_ent;
  int* blk_mask;
  int* rem_pos;
  int* rem_ent;
  int* rem_crd;
  int* cnt;
  long long* block_sum;
  long long* total;
  int RB;
  long long capB;
  size_t bytes;
};

static size_t al256(size_t x) { return (x + 255) & ~(size_t)255; }

static AttnPlan attn_plan_view(void* base, int64_t m, int64_t nnz) {
  AttnPlan p;
  char* c = static_cast<char*>(base);
  size_t off = 0;
  p.RB = (int)ceil_div(m, 16);
  p.capB = nnz / kMinBlockEntries + 1;
  p.hdr = reinterpret_cast<int*>(c + off); off += al256(16 * 4);
  p.rb_ptr = reinterpret_cast<int*>(c + off); off += al256((size_t)(p.RB + 1) * 4);
  p.blk_col = reinterpret_cast<int*>(c + off); off += al256((size_t)p.capB * 4);
  p.blk_ent = reinterpret_cast<int*>(c + off); off += al256((size_t)p.capB * 16 * 4);
  p.blk_mask = reinterpret_cast<int*>(c + off); off += al256((size_t)p.capB * 16 * 4);
  p.rem_pos = reinterpret_cast<int*>(c + off); off += al256((size_t)(m + 1) * 4);
  p.rem_ent = reinterpret_cast<int*>(c + off); off += al256((size_t)(nnz + 1) * 4);
  p.rem_crd = reinterpret_cast<int*>(c + off); off += al256((size_t)(nnz + 1) * 4);
  const int64_t cn = (m > p.RB ? m : p.RB) + 1;
  p.cnt = reinterpret_cast<int*>(c + off); off += al256((size_t)cn * 4);
  p.block_sum = reinterpret_cast<long long*>(c + off); off += al256((size_t)(ceil_div(cn, 4096) + 1) * 8);
  p.total = reinterpret_cast<long long*>(c + off); off += al256(16);
  p.bytes = off;
  return p;
}

// ---- plan construction --------------------------------------------------------------------------------
// lower bound of column c in row [b, e)
__device__ __forceinline__ int attn_find_col(const int* __restrict__ crd, int b, int e, int c) {
  while (b < e) {
    const int mid = (b + e) >> 1;
    if (__ldg(crd + mid) < c) b = mid + 1; else e = mid;
  }
  return b;
}

// One warp per row block.  The stored entries of the 16 rows are counted per column block in a
// per-warp shared-memory hash table; column blocks with at least kMinBlockEntries entries are
// selected and ranked ascending; lanes 0..15 then find, each in its own row, the first stored
// entry and the 16-bit column mask of every selected block.  A row block that touches more than
// kDetectSlots/2 distinct column blocks keeps no blocks (all its entries stay in the remainder).
template <bool WRITE>
__global__ void __launch_bounds__(128)
attn_detect_kernel(int m, int n, int RB, const int* __restrict__ pos, const int* __restrict__ crd,
                   int* __restrict__ cnt, const int* __restrict__ rb_ptr, int* __restrict__ blk_col,
                   int* __restrict__ blk_ent, int* __restrict__ blk_mask) {
  __shared__ int s_key[4][kDetectSlots];
  __shared__ int s_cnt[4][kDetectSlots];
  __shared__ int s_sel[4][kDetectSlots / 2 + 32];
  __shared__ int s_n[4][2];  // [0] distinct column blocks, [1] selected
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rb = blockIdx.x * 4 + warp;
  if (rb >= RB) return;
  const int i0 = rb * 16;
  int nsel = 0;
  if (i0 + 16 <= m) {
    int* key = s_key[warp];
    int* num = s_cnt[warp];
    int* sel = s_sel[warp];
    for (int t = lane; t < kDetectSlots; t += 32) { key[t] = -1; num[t] = 0; }
    if (lane == 0) { s_n[warp][0] = 0; s_n[warp][1] = 0; }
    __syncwarp();
    const int b0 = __ldg(pos + i0), e0 = __ldg(pos + i0 + 16);  // the 16 rows are contiguous
    bool overflow = false;
    for (int p = b0 + lane; p < e0 && !overflow; p += 32) {
      const int cb = __ldg(crd + p) >> 4;
      int h = (int)(((unsigned)cb * 0x9E3779B1u) >> 22) & (kDetectSlots - 1);
      // the table never fills (insertion stops at kDetectSlots/2 + 32 keys), so the probe ends
      while (true) {
        const int old = atomicCAS(&key[h], -1, cb);
        if (old == -1) {
          if (atomicAdd(&s_n[warp][0], 1) >= kDetectSlots / 2) overflow = true;
        }
        if (old == -1 || old == cb) { atomicAdd(&num[h], 1); break; }
        h = (h + 1) & (kDetectSlots - 1);
      }
    }
    __syncwarp();
    if (s_n[warp][0] <= kDetectSlots / 2) {
      for (int t = lane; t < kDetectSlots; t += 32) {
        // (a column block that sticks out over the last column is never selected: the block
        // kernel reads 16 whole rows of K and V)
        if (key[t] >= 0 && num[t] >= kMinBlockEntries && (key[t] + 1) * 16 <= n)
          sel[atomicAdd(&s_n[warp][1], 1)] = key[t];
      }
      __syncwarp();
      nsel = s_n[warp][1];
    }
    if (WRITE && nsel > 0) {
      const int base = __ldg(rb_ptr + rb);
      const int my_row = i0 + (lane & 15);
      const int rb_ = __ldg(pos + my_row), re_ = __ldg(pos + my_row + 1);
      // rank of each selected column block = number of smaller ones (ascending, deterministic)
      for (int x = 0; x < nsel; x++) {
        const int cb = sel[x];
        int smaller = 0;
        for (int y = lane; y < nsel; y += 32) smaller += sel[y] < cb;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) smaller += __shfl_xor_sync(FULL, smaller, o);
        const long long b = base + smaller;
        if (lane == 0) blk_col[b] = cb;
        if (lane < 16) {
          const int c0 = cb << 4;
          const int q = attn_find_col(crd, rb_, re_, c0);
          int mask = 0;
          for (int e = q; e < re_; e++) {
            const int c = __ldg(crd + e) - c0;
            if (c >= 16) break;
            mask |= 1 << c;
          }
          blk_ent[b * 16 + lane] = q;
          blk_mask[b * 16 + lane] = mask;
        }
      }
    }
  }
  if (!WRITE && lane == 0) cnt[rb] = nsel;
}

// One warp per row: the entries whose column block is not a block of the row block.  FILL writes
// their entry indices, otherwise only the count per row is produced.
template <bool FILL>
__global__ void __launch_bounds__(256)
attn_rem_kernel(int m, const int* __restrict__ pos, const int* __restrict__ crd,
                const int* __restrict__ rb_ptr, const int* __restrict__ blk_col, int* __restrict__ cnt,
                const int* __restrict__ rem_pos, int* __restrict__ rem_ent, int* __restrict__ rem_crd) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= m) return;
  const int b = __ldg(pos + row), e = __ldg(pos + row + 1);
  const int kb = __ldg(rb_ptr + (row >> 4)), ke = __ldg(rb_ptr + (row >> 4) + 1);
  int outp = FILL ? __ldg(rem_pos + row) : 0;
  for (int p0 = b; p0 < e; p0 += 32) {
    const int p = p0 + lane;
    bool keep = false;
    int col = 0;
    if (p < e) {
      col = __ldg(crd + p);
      const int cb = col >> 4;
      int lo = kb, hi = ke;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(blk_col + mid) < cb) lo = mid + 1; else hi = mid;
      }
      keep = !(lo < ke && __ldg(blk_col + lo) == cb);
    }
    const unsigned mask = __ballot_sync(FULL, keep);
    if (FILL && keep) {
      const int q = outp + __popc(mask & ((1u << lane) - 1));
      rem_ent[q] = p;
      rem_crd[q] = col;
    }
    outp += __popc(mask);
  }
  if (!FILL && lane == 0) cnt[row] = outp;
}

// flag[0] = 1 on entry; cleared if any mask value differs from 1.0f (a pure pattern mask, the
// common case, then costs the block kernel no mask-value loads)
__global__ void attn_mask_ones_kernel(const float* __restrict__ mask_val, long long nnz, int* flag) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  bool ones = true;
  for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < nnz; p += stride)
    ones = ones && (ld_stream(mask_val + p) == 1.0f);
  if (!__all_sync(FULL, ones) && (threadIdx.x & 31) == 0) *flag = 0;
}
__global__ void attn_flag_init_kernel(int* flag) { *flag = 1; }

// ---- the scattered entries -----------------------------------------------------------------------
// L = d / 8 lanes per mask row (a lane holds 8 features of the row's Q and 8 columns of its
// output), 32 / L rows per warp.  A group walks its row's scattered entries two at a time: K and
// V rows of both entries are gathered together (four 256-bit loads in flight per lane), the
// partial dot products are summed across the group's lanes, and the row's running maximum, sum
// and unnormalised output are updated once per pair.  Scores are in log2 units like the block
// kernel's.  The trip count is the longest row of the warp; finished groups idle.
constexpr int kScatWarps = 8;
template <int L>
__global__ void __launch_bounds__(kScatWarps * 32, 4)
attn_scattered_kernel(AttnArgs a) {
  constexpr int G = 32 / L;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane / L, l = lane % L;
  const int row = (blockIdx.x * kScatWarps + warp) * G + g;
  if ((blockIdx.x * kScatWarps + warp) * G >= a.m) return;
  const long long bz = blockIdx.y;
  const float* K = a.K + bz * a.stride_k + 8 * l;
  const float* V = a.V + bz * a.stride_v + 8 * l;
  const float scale = a.scale * 1.4426950408889634f;
  const float* mask_val = (a.mask_val && !__ldg(a.mask_is_ones)) ? a.mask_val : nullptr;
  const bool live = row < a.m;
  int b = 0, e = 0;
  Float8 q;
#pragma unroll
  for (int i = 0; i < 8; i++) q.v[i] = 0.f;
  if (live) {
    b = __ldg(a.rem_pos + row);
    e = __ldg(a.rem_pos + row + 1);
    q = ldg8(a.Q + bz * a.stride_q + (size_t)((unsigned long long)(unsigned)row * a.ldq) + 8 * l);
  }
  const int longest = __reduce_max_sync(FULL, e - b);
  float M = -INFINITY, Ls = 0.f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; i++) acc[i] = 0.f;
  // the group's next L entries: column and mask value, one per lane, a chunk ahead
  int next_j = 0;
  float next_w = 1.f;
  if (b + l < e) {
    next_j = ld_stream(a.rem_crd + b + l);
    if (mask_val) next_w = __ldg(mask_val + ld_stream(a.rem_ent + b + l));
  }
#pragma unroll 1
  for (int q0 = 0; q0 < longest; q0 += L) {
    const int p0 = b + q0;
    const int my_j = next_j;
    const float my_w = next_w;
    if (p0 + L + l < e) {
      next_j = ld_stream(a.rem_crd + p0 + L + l);
      if (mask_val) next_w = __ldg(mask_val + ld_stream(a.rem_ent + p0 + L + l));
    }
    const int cnt = e - p0;                       // entries this group still has (may be <= 0)
    const int most = min(L, longest - q0);        // warp-uniform
#pragma unroll 1
    for (int t0 = 0; t0 < most; t0 += 2) {
      Float8 kv[2], vv[2];
      float w[2];
      bool ok[2];
#pragma unroll
      for (int u = 0; u < 2; u++) {
        const int t = t0 + u;
        const unsigned j = (unsigned)__shfl_sync(FULL, my_j, t & (L - 1), L);
        w[u] = __shfl_sync(FULL, my_w, t & (L - 1), L);
        ok[u] = t < cnt && t < L;
        if (ok[u]) {
          kv[u] = ldg8(K + (size_t)((unsigned long long)j * a.ldk));
          vv[u] = ldg8(V + (size_t)((unsigned long long)j * a.ldv));
        } else {
#pragma unroll
          for (int i = 0; i < 8; i++) kv[u].v[i] = vv[u].v[i] = 0.f;
        }
      }
      float sc[2];
#pragma unroll
      for (int u = 0; u < 2; u++) {
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) d = fmaf(q.v[i], kv[u].v[i], d);
#pragma unroll
        for (int o = L / 2; o > 0; o >>= 1) d += __shfl_xor_sync(FULL, d, o);
        sc[u] = ok[u] ? d * scale * w[u] : -INFINITY;
      }
      const float nm = fmaxf(M, fmaxf(sc[0], sc[1]));
      const float ms = (nm == -INFINITY) ? 0.f : nm;
      const float alpha = attn_exp2(M - ms);      // 0 while the row has seen no entry
      const float p0e = attn_exp2(sc[0] - ms), p1e = attn_exp2(sc[1] - ms);
      M = nm;
      Ls = Ls * alpha + p0e + p1e;
#pragma unroll
      for (int i = 0; i < 8; i++) acc[i] = fmaf(p1e, vv[1].v[i], fmaf(p0e, vv[0].v[i], acc[i] * alpha));
    }
  }
  if (live) {
    float* orow = a.O + bz * a.stride_o + (long long)row * a.ldo + 8 * l;
    *reinterpret_cast<float4*>(orow) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(orow + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if (l == 0) a.stats[bz * a.m + row] = make_float2(M, Ls);
  }
}

// One warp per row block.  Thread (g, t) = (lane / 4, lane % 4) owns rows g and g+8 of the row
// block in every fragment.  Layouts (see mma_tf32.cuh):
//   S = Q K^T : A = Q rows, B column g of n-tile n = K row 8n+g; the feature index is permuted so
//               that k-step (4q+h) uses features 32q + 8t + 2h (+1): 256-bit loads of Q and K.
//               c[n][0..1] = S[g][8n+2t, +1], c[n][2..3] = S[g+8][8n+2t, +1].
//   O += P V  : k-step n covers block columns 8n..8n+7 with k-slot t = column 8n+2t and k-slot
//               t+4 = column 8n+2t+1, which is exactly where S left P: no data movement between
//               the two products.  B of column tile u is V[8n+2t (+1)][g*KT + u] (logical column
//               (u, g) = actual column g*KT + u), so a thread reads KT contiguous floats per V
//               row and writes KT contiguous floats per output row.
// Three CTAs per SM (168 registers; four spill, two leave the tensor pipe idle more often).
constexpr int kAttnWarps = 4;  // row blocks per CTA (1 and 2 measured the same)
template <int D16>  // head dimension d = 16 * D16 (of Q, K and V)
__global__ void __launch_bounds__(kAttnWarps * 32, 12 / kAttnWarps)
attn_block_kernel(AttnArgs a) {
  constexpr int KT = 2 * D16;
  // the warp's Q rows as pre-split TF32 A fragments, one 128-bit word per lane and k-step
  __shared__ uint4 sq_hi[kAttnWarps][2 * D16][32], sq_lo[kAttnWarps][2 * D16][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rb = blockIdx.x * kAttnWarps + warp;
  if (rb >= a.RB) return;
  const int g = lane >> 2, t = lane & 3;
  const long long bz = blockIdx.y;
  const float* Q = a.Q + bz * a.stride_q;
  const float* K = a.K + bz * a.stride_k;
  const float* V = a.V + bz * a.stride_v;
  float* O = a.O + bz * a.stride_o;
  const int i0 = rb * 16;
  const int kb = __ldg(a.rb_ptr + rb), ke = __ldg(a.rb_ptr + rb + 1);
  const float scale = a.scale * 1.4426950408889634f;  // scores are kept in log2 units: exp2 below
  const float* mask_val = (a.mask_val && !__ldg(a.mask_is_ones)) ? a.mask_val : nullptr;

  // running maximum M, (per-thread partial) sum L and output accumulators of both rows continue
  // from what the scattered-entry kernel left for them (the row's sum lives on lane t = 0)
  float M[2] = {-INFINITY, -INFINITY}, L[2] = {0.f, 0.f};
  float o[KT][4];
#pragma unroll
  for (int u = 0; u < KT; u++) o[u][0] = o[u][1] = o[u][2] = o[u][3] = 0.f;
  if (a.has_rem) {
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const int row = i0 + g + 8 * r;
      if (row >= a.m) continue;
      const float2 st = __ldg(a.stats + bz * a.m + row);
      M[r] = st.x;
      L[r] = (t == 0) ? st.y : 0.f;
      const float* orow = O + (long long)row * a.ldo;
#pragma unroll
      for (int e = 0; e < 2; e++) {
#pragma unroll
        for (int u = 0; u < KT; u += 4) {
          const float4 x = *reinterpret_cast<const float4*>(orow + (2 * t + e) * KT + u);
          o[u][2 * r + e] = x.x; o[u + 1][2 * r + e] = x.y; o[u + 2][2 * r + e] = x.z; o[u + 3][2 * r + e] = x.w;
        }
      }
    }
  }

  if (kb < ke) {  // (row blocks with blocks are complete: all 16 rows exist)
    {
      const float* qrow0 = Q + (size_t)((unsigned long long)(unsigned)(i0 + g) * a.ldq) + 8 * t;
      const float* qrow1 = Q + (size_t)((unsigned long long)(unsigned)(i0 + g + 8) * a.ldq) + 8 * t;
#pragma unroll
      for (int q = 0; q < D16 / 2; q++) {
        const Float8 v0 = ldg8(qrow0 + 32 * q), v1 = ldg8(qrow1 + 32 * q);
#pragma unroll
        for (int h = 0; h < 4; h++) {
          uint4 hi, lo;
          attn_split(v0.v[2 * h], hi.x, lo.x); attn_split(v1.v[2 * h], hi.y, lo.y);
          attn_split(v0.v[2 * h + 1], hi.z, lo.z); attn_split(v1.v[2 * h + 1], hi.w, lo.w);
          sq_hi[warp][4 * q + h][lane] = hi; sq_lo[warp][4 * q + h][lane] = lo;
        }
      }
    }
    Float8 kf[2][D16 / 2];
    auto load_k = [&](int j0) {
#pragma unroll
      for (int n = 0; n < 2; n++) {
        const float* krow = K + (size_t)((unsigned long long)(unsigned)(j0 + 8 * n + g) * a.ldk) + 8 * t;
#pragma unroll
        for (int q = 0; q < D16 / 2; q++) kf[n][q] = ldg8(krow + 32 * q);
      }
    };
    // descriptor of a block as this thread needs it: first column, stored-column masks and first
    // entries of rows g and g+8; read one block ahead
    struct Desc { int j0; unsigned m0, m1; int p0, p1; };
    auto load_desc = [&](int b) {
      Desc x;
      x.j0 = __ldg(a.blk_col + b) * 16;
      x.m0 = (unsigned)__ldg(a.blk_mask + (long long)b * 16 + g);
      x.m1 = (unsigned)__ldg(a.blk_mask + (long long)b * 16 + g + 8);
      x.p0 = x.p1 = 0;
      if (mask_val) {
        x.p0 = __ldg(a.blk_ent + (long long)b * 16 + g);
        x.p1 = __ldg(a.blk_ent + (long long)b * 16 + g + 8);
      }
      return x;
    };
    Desc d1 = load_desc(kb);                              // block b at the top of iteration b
    Desc d2 = (kb + 1 < ke) ? load_desc(kb + 1) : d1;     // block b+1
    load_k(d1.j0);
#pragma unroll 1
    for (int b = kb; b < ke; b++) {
      const Desc cur = d1;
      const unsigned m0 = cur.m0, m1 = cur.m1;
      // warp-uniform: every entry of the block is stored (the blocks inside a band)
      const bool full = __all_sync(FULL, (m0 & m1) == 0xffffu);
      // mask values of this thread's 8 entries: in flight while S is computed
      float w[2][4];
#pragma unroll
      for (int n = 0; n < 2; n++) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
          w[n][e] = w[n][2 + e] = 1.f;
          if (mask_val) {
            const int col = 8 * n + 2 * t + e;
            if (full) {
              w[n][e] = __ldg(mask_val + cur.p0 + col);
              w[n][2 + e] = __ldg(mask_val + cur.p1 + col);
            } else {
              if ((m0 >> col) & 1u) w[n][e] = __ldg(mask_val + cur.p0 + __popc(m0 & ((1u << col) - 1u)));
              if ((m1 >> col) & 1u) w[n][2 + e] = __ldg(mask_val + cur.p1 + __popc(m1 & ((1u << col) - 1u)));
            }
          }
        }
      }
      float vb[2][2][KT];
      auto load_v = [&]() {
#pragma unroll
        for (int n = 0; n < 2; n++) {
#pragma unroll
          for (int e = 0; e < 2; e++) {
            const float* vrow =
                V + (size_t)((unsigned long long)(unsigned)(cur.j0 + 8 * n + 2 * t + e) * a.ldv) + g * KT;
            if constexpr (KT == 8) {
              const Float8 x = ldg8(vrow);
#pragma unroll
              for (int u = 0; u < 8; u++) vb[n][e][u] = x.v[u];
            } else {
              const float4 x = ldg4(vrow);
              vb[n][e][0] = x.x; vb[n][e][1] = x.y; vb[n][e][2] = x.z; vb[n][e][3] = x.w;
            }
          }
        }
      };
      // S = Q K^T; main and cross terms accumulate separately, the two column tiles alternate
      float c[2][4], x[2][4];
#pragma unroll
      for (int n = 0; n < 2; n++) {
        c[n][0] = c[n][1] = c[n][2] = c[n][3] = 0.f;
        x[n][0] = x[n][1] = x[n][2] = x[n][3] = 0.f;
      }
#pragma unroll
      for (int q = 0; q < D16 / 2; q++) {
#pragma unroll
        for (int h = 0; h < 4; h++) {
          const uint4 qh = sq_hi[warp][4 * q + h][lane], ql = sq_lo[warp][4 * q + h][lane];
          const unsigned ahi[4] = {qh.x, qh.y, qh.z, qh.w};
          const unsigned alo[4] = {ql.x, ql.y, ql.z, ql.w};
          unsigned bh[2][2], bl[2][2];
#pragma unroll
          for (int n = 0; n < 2; n++) {
            attn_split(kf[n][q].v[2 * h], bh[n][0], bl[n][0]);
            attn_split(kf[n][q].v[2 * h + 1], bh[n][1], bl[n][1]);
          }
          mma_tf32(x[0], alo, bh[0][0], bh[0][1]);
          mma_tf32(x[1], alo, bh[1][0], bh[1][1]);
          mma_tf32(x[0], ahi, bl[0][0], bl[0][1]);
          mma_tf32(x[1], ahi, bl[1][0], bl[1][1]);
          mma_tf32(c[0], ahi, bh[0][0], bh[0][1]);
          mma_tf32(c[1], ahi, bh[1][0], bh[1][1]);
        }
      }
      // K rows of the next block (its descriptor was read an iteration ago) and the descriptor
      // of the block after it: in flight during the softmax update and P V
      d1 = d2;
      if (b + 1 < ke) load_k(d1.j0);
      if (b + 2 < ke) d2 = load_desc(b + 2);
      // the V rows of this block: in flight during the softmax update (issuing them before S
      // keeps 32 more registers live through it and measured 3 % slower)
      load_v();
      // scaled scores of the stored entries, -inf elsewhere
      float s[2][4];
#pragma unroll
      for (int n = 0; n < 2; n++) {
#pragma unroll
        for (int e = 0; e < 4; e++) s[n][e] = (c[n][e] + x[n][e]) * scale;
      }
      if (mask_val) {
#pragma unroll
        for (int n = 0; n < 2; n++) {
#pragma unroll
          for (int e = 0; e < 4; e++) s[n][e] *= w[n][e];
        }
      }
      if (!full) {
#pragma unroll
        for (int n = 0; n < 2; n++) {
#pragma unroll
          for (int e = 0; e < 2; e++) {
            const int col = 8 * n + 2 * t + e;
            if (!((m0 >> col) & 1u)) s[n][e] = -INFINITY;
            if (!((m1 >> col) & 1u)) s[n][2 + e] = -INFINITY;
          }
        }
      }
      // running softmax of rows g (r = 0) and g+8 (r = 1)
      float alpha[2];
#pragma unroll
      for (int r = 0; r < 2; r++) {
        float bm = fmaxf(fmaxf(s[0][2 * r], s[0][2 * r + 1]), fmaxf(s[1][2 * r], s[1][2 * r + 1]));
        bm = fmaxf(bm, __shfl_xor_sync(FULL, bm, 1));
        bm = fmaxf(bm, __shfl_xor_sync(FULL, bm, 2));
        const float nm = fmaxf(M[r], bm);
        const float ms = (nm == -INFINITY) ? 0.f : nm;
        alpha[r] = attn_exp2(M[r] - ms);  // 0 while the row has seen no entry
        M[r] = nm;
        float sum = 0.f;
#pragma unroll
        for (int n = 0; n < 2; n++) {
#pragma unroll
          for (int e = 0; e < 2; e++) {
            const float p = attn_exp2(s[n][2 * r + e] - ms);
            s[n][2 * r + e] = p;
            sum += p;
          }
        }
        L[r] = L[r] * alpha[r] + sum;
      }
      // (the maxima rarely move after the first blocks of a row block: no rescale then)
      if (!__all_sync(FULL, alpha[0] == 1.f && alpha[1] == 1.f)) {
#pragma unroll
        for (int u = 0; u < KT; u++) {
          o[u][0] *= alpha[0];
          o[u][1] *= alpha[0];
          o[u][2] *= alpha[1];
          o[u][3] *= alpha[1];
        }
      }
      // O += P V
#pragma unroll
      for (int n = 0; n < 2; n++) {
        unsigned ahi[4], alo[4];
        attn_split(s[n][0], ahi[0], alo[0]);  // row g,   column 8n+2t   (k-slot t)
        attn_split(s[n][2], ahi[1], alo[1]);  // row g+8, column 8n+2t
        attn_split(s[n][1], ahi[2], alo[2]);  // row g,   column 8n+2t+1 (k-slot t+4)
        attn_split(s[n][3], ahi[3], alo[3]);  // row g+8, column 8n+2t+1
        // four column tiles at a time, term by term: no mma waits on the one before it
#pragma unroll
        for (int u0 = 0; u0 < KT; u0 += 4) {
          unsigned bh[4][2], bl[4][2];
#pragma unroll
          for (int u = 0; u < 4; u++) {
            attn_split(vb[n][0][u0 + u], bh[u][0], bl[u][0]);
            attn_split(vb[n][1][u0 + u], bh[u][1], bl[u][1]);
          }
#pragma unroll
          for (int u = 0; u < 4; u++) mma_tf32(o[u0 + u], alo, bh[u][0], bh[u][1]);
#pragma unroll
          for (int u = 0; u < 4; u++) mma_tf32(o[u0 + u], ahi, bl[u][0], bl[u][1]);
#pragma unroll
          for (int u = 0; u < 4; u++) mma_tf32(o[u0 + u], ahi, bh[u][0], bh[u][1]);
        }
      }
    }
  }

  // O / sum
#pragma unroll
  for (int r = 0; r < 2; r++) {
    float sum = L[r];
    sum += __shfl_xor_sync(FULL, sum, 1);
    sum += __shfl_xor_sync(FULL, sum, 2);
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    const int row = i0 + g + 8 * r;
    if (row < a.m) {
      float* orow = O + (long long)row * a.ldo;
#pragma unroll
      for (int e = 0; e < 2; e++) {
#pragma unroll
        for (int u = 0; u < KT; u += 4) {
          const float4 x = make_float4(o[u][2 * r + e] * inv, o[u + 1][2 * r + e] * inv,
                                       o[u + 2][2 * r + e] * inv, o[u + 3][2 * r + e] * inv);
          *reinterpret_cast<float4*>(orow + (2 * t + e) * KT + u) = x;
        }
      }
    }
  }
}

}  // namespace sb

namespace sb {

int attn_launch_scattered(const AttnArgs& a, int64_t d, int64_t nnz, int64_t rem_nnz, int64_t batch,
                          int* flags, cudaStream_t st) {
  const int64_t m = a.m;
  if (a.mask_val && nnz > 0) {  // (without mask values no kernel reads the flag)
    attn_flag_init_kernel<<<1, 1, 0, st>>>(flags);
    const unsigned blocks_ones = (unsigned)std::min<int64_t>(ceil_div(nnz, 256 * 8), 4 * sm_count());
    attn_mask_ones_kernel<<<blocks_ones, 256, 0, st>>>(a.mask_val, nnz, flags);
    SB_LAUNCH_CHECK("attn_mask_ones_kernel");
  }
  if (rem_nnz > 0) {
    if (d == 32) {
      dim3 grid((unsigned)ceil_div(ceil_div(m, 8), kScatWarps), (unsigned)batch);
      attn_scattered_kernel<4><<<grid, kScatWarps * 32, 0, st>>>(a);
    } else {
      dim3 grid((unsigned)ceil_div(ceil_div(m, 4), kScatWarps), (unsigned)batch);
      attn_scattered_kernel<8><<<grid, kScatWarps * 32, 0, st>>>(a);
    }
    SB_LAUNCH_CHECK("attn_scattered_kernel");
  }
  return SB_OK;
}

}  // namespace sb

using namespace sb;

extern "C" {

size_t sb_attn_plan_bytes(int64_t m, int64_t nnz) {
  if (m < 0) m = 0;
  if (nnz < 0) nnz = 0;
  return attn_plan_view(nullptr, m, nnz).bytes;
}

int sb_attn_plan_build(int64_t m, int64_t n, int64_t nnz, const int32_t* pos, const int32_t* crd,
                       void* plan, size_t plan_bytes, int64_t* blocks_host, int64_t* rem_nnz_host,
                       void* stream) {
  SB_CHECK_ARG(m >= 0 && n >= 0 && nnz >= 0 && m < INT32_MAX - 16 && n < INT32_MAX - 16 && nnz < INT32_MAX,
               "attn_plan: bad size");
  SB_CHECK_ARG(pos && plan && (crd || nnz == 0), "attn_plan: null pointer");
  SB_CHECK_ARG(aligned16(plan), "attn_plan: plan must be 16-byte aligned");
  AttnPlan p = attn_plan_view(plan, m, nnz);
  if (plan_bytes < p.bytes)
    return fail(SB_ERR_WORKSPACE, "attn_plan: buffer has %zu bytes, needs %zu", plan_bytes, p.bytes);
  cudaStream_t st = (cudaStream_t)stream;
  SB_CUDA(cudaMemsetAsync(p.hdr, 0, 64, st));
  long long nblk = 0, nrem = 0;
  if (m > 0) {
    const unsigned wg = (unsigned)ceil_div(p.RB, 4);
    attn_detect_kernel<false><<<wg, 128, 0, st>>>((int)m, (int)n, p.RB, pos, crd, p.cnt, nullptr, nullptr,
                                                   nullptr, nullptr);
    SB_LAUNCH_CHECK("attn_detect_kernel<count>");
    int rc = exclusive_scan_i32(p.RB, p.cnt, p.rb_ptr, p.block_sum, p.total, st);
    if (rc != SB_OK) return rc;
    SB_CUDA(cudaMemcpyAsync(&nblk, p.total, 8, cudaMemcpyDeviceToHost, st));
    attn_detect_kernel<true><<<wg, 128, 0, st>>>((int)m, (int)n, p.RB, pos, crd, p.cnt, p.rb_ptr, p.blk_col,
                                                  p.blk_ent, p.blk_mask);
    SB_LAUNCH_CHECK("attn_detect_kernel<fill>");
    attn_rem_kernel<false><<<(unsigned)ceil_div(m * 32, 256), 256, 0, st>>>((int)m, pos, crd, p.rb_ptr,
                                                                           p.blk_col, p.cnt, nullptr, nullptr, nullptr);
    SB_LAUNCH_CHECK("attn_rem_kernel<count>");
    rc = exclusive_scan_i32((int)m, p.cnt, p.rem_pos, p.block_sum, p.total, st);
    if (rc != SB_OK) return rc;
    SB_CUDA(cudaMemcpyAsync(&nrem, p.total, 8, cudaMemcpyDeviceToHost, st));
    attn_rem_kernel<true><<<(unsigned)ceil_div(m * 32, 256), 256, 0, st>>>((int)m, pos, crd, p.rb_ptr,
                                                                          p.blk_col, nullptr, p.rem_pos, p.rem_ent, p.rem_crd);
    SB_LAUNCH_CHECK("attn_rem_kernel<fill>");
    SB_CUDA(cudaStreamSynchronize(st));
    int h[2] = {(int)nblk, (int)nrem};
    SB_CUDA(cudaMemcpyAsync(p.hdr, h, 8, cudaMemcpyHostToDevice, st));
    SB_CUDA(cudaStreamSynchronize(st));
  } else {
    SB_CUDA(cudaMemsetAsync(p.rb_ptr, 0, 4, st));
    SB_CUDA(cudaMemsetAsync(p.rem_pos, 0, 4, st));
    SB_CUDA(cudaStreamSynchronize(st));
  }
  if (blocks_host) *blocks_host = nblk;
  if (rem_nnz_host) *rem_nnz_host = nrem;
  return SB_OK;
}

// scratch: 256 bytes of flags, then [batch][m] (maximum, sum) pairs of the rows' scattered entries
size_t sb_sparse_attention_scratch_bytes(int64_t m, int64_t rem_nnz, int64_t batch) {
  if (m < 0) m = 0;
  if (batch < 0) batch = 0;
  return 256 + (rem_nnz > 0 ? (size_t)m * (size_t)batch * sizeof(float2) : 0);
}

int sb_sparse_attention_csr_f32(int64_t m, int64_t n, int64_t d, int64_t nnz, const int32_t* pos,
                                const int32_t* crd, const float* mask_val, const float* Q, int64_t ldq,
                                const float* K, int64_t ldk, const float* V, int64_t ldv, float scale,
                                float* O, int64_t ldo, int64_t batch, int64_t stride_q, int64_t stride_k,
                                int64_t stride_v, int64_t stride_o, const void* attn_plan, int64_t blocks,
                                int64_t rem_nnz, void* scratch, size_t scratch_bytes, int stages,
                                void* stream) {
  (void)pos;
  SB_CHECK_ARG(stages > 0 && stages <= SB_ATTN_ALL_STAGES, "sparse_attention: bad stage set");
  SB_CHECK_ARG(m >= 0 && n >= 0 && nnz >= 0 && m < INT32_MAX - 16 && n < INT32_MAX - 16 && nnz < INT32_MAX,
               "sparse_attention: bad size");
  SB_CHECK_ARG(batch >= 1 && batch <= 65535, "sparse_attention: batch must be in [1, 65535]");
  SB_CHECK_ARG(d == 32 || d == 64, "sparse_attention: head dimension must be 32 or 64");
  if (m == 0) return SB_OK;
  SB_CHECK_ARG(attn_plan && Q && K && V && O && (crd || nnz == 0), "sparse_attention: null pointer");
  SB_CHECK_ARG(ldq >= d && ldk >= d && ldv >= d && ldo >= d, "sparse_attention: row pitch smaller than d");
  auto aligned32 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; };
  SB_CHECK_ARG(ldq % 8 == 0 && ldk % 8 == 0 && ldv % 8 == 0 && stride_q % 8 == 0 && stride_k % 8 == 0 &&
               stride_v % 8 == 0 && aligned32(Q) && aligned32(K) && aligned32(V) && ldq < (1ll << 32) &&
               ldk < (1ll << 32) && ldv < (1ll << 32),
               "sparse_attention: Q/K/V must be 32-byte aligned with row pitches and batch strides that are "
               "multiples of 8");
  SB_CHECK_ARG(ldo % 4 == 0 && stride_o % 4 == 0 && aligned16(O),
               "sparse_attention: O must be 16-byte aligned with a row pitch that is a multiple of 4");
  SB_CHECK_ARG(blocks >= 0 && rem_nnz >= 0 && rem_nnz <= nnz && blocks * 256 + rem_nnz >= nnz &&
               blocks * kMinBlockEntries + rem_nnz <= nnz,
               "sparse_attention: block/remainder counts do not fit nnz");
  const size_t need = sb_sparse_attention_scratch_bytes(m, rem_nnz, batch);
  SB_CHECK_ARG(scratch && aligned16(scratch), "sparse_attention: scratch is null or misaligned");
  if (scratch_bytes < need)
    return fail(SB_ERR_WORKSPACE, "sparse_attention: scratch has %zu bytes, needs %zu", scratch_bytes, need);
  cudaStream_t st = (cudaStream_t)stream;
  AttnPlan p = attn_plan_view(const_cast<void*>(attn_plan), m, nnz);
  int* flags = static_cast<int*>(scratch);
  AttnArgs a;
  a.m = (int)m; a.RB = p.RB; a.rb_ptr = p.rb_ptr; a.blk_col = p.blk_col; a.blk_ent = p.blk_ent;
  a.blk_mask = p.blk_mask; a.rem_pos = p.rem_pos; a.rem_ent = p.rem_ent; a.rem_crd = p.rem_crd;
  a.mask_val = mask_val; a.mask_is_ones = flags;
  a.Q = Q; a.K = K; a.V = V; a.O = O;
  a.stats = reinterpret_cast<float2*>(static_cast<char*>(scratch) + 256);
  a.has_rem = rem_nnz > 0 ? 1 : 0;
  a.ldq = (unsigned)ldq; a.ldk = (unsigned)ldk; a.ldv = (unsigned)ldv; a.ldo = ldo;
  a.stride_q = stride_q; a.stride_k = stride_k; a.stride_v = stride_v; a.stride_o = stride_o;
  a.scale = scale;
  if (stages & SB_ATTN_STAGE_SCATTERED) {
    const int rc = attn_launch_scattered(a, d, nnz, rem_nnz, batch, flags, st);
    if (rc != SB_OK) return rc;
  }
  if (stages & SB_ATTN_STAGE_BLOCKS) {
    dim3 grid((unsigned)ceil_div(p.RB, kAttnWarps), (unsigned)batch);
    if (d == 32) attn_block_kernel<2><<<grid, kAttnWarps * 32, 0, st>>>(a);
    else attn_block_kernel<4><<<grid, kAttnWarps * 32, 0, st>>>(a);
    SB_LAUNCH_CHECK("attn_block_kernel");
  }
  return SB_OK;
}

}  // extern "C"
