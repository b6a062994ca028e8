// Dense 16x16 block path for CSR patterns that contain dense blocks (banded attention masks,
// block-structured weights): the only place this library uses the tensor cores.
//
// A block plan splits the pattern, once per matrix, into
//   * the aligned 16x16 blocks in which all 256 entries are stored (per row block: ascending
//     column blocks; per block: for each of its 16 rows the entry index of the block's first
//     column, so results land in the pattern's own entry order), and
//   * a CSR list of the remaining entries (indices into the original entry arrays).
// SDDMM and SpMM then run one tensor-core kernel over the dense blocks and the ordinary gather
// kernel over the remainder.  A gathered K / V row is used by 16 mask rows at once instead of
// one, which is what lifts these kernels off the L1 gather bound.
//
// Arithmetic: mma.sync m16n8k8 TF32 with the 3xTF32 split (x = hi + lo; hi*hi + hi*lo + lo*hi,
// fp32 accumulate), which keeps fp32-level accuracy (a single TF32 pass would miss the
// rtol 1e-4 contract).  Tiles are 16x16, far below the 64/128-row minimum of the tcgen05 path,
// so the warp-level mma is the fitting instruction here.
#include "common.cuh"
#include "mma_tf32.cuh"

namespace sb {

// ---- plan layout ---------------------------------------------------------------------------------
// int32 words: hdr[16] ([0] blocks, [1] remainder entries), then
//   rb_ptr[RB+1]   blocks of row block b are [rb_ptr[b], rb_ptr[b+1])
//   blk_col[capB]  column block of each dense block
//   blk_ent[capB*16] entry index of (row r of the block, first column of the block)
//   rem_pos[m+1], rem_ent[nnz]   CSR of the entries outside dense blocks
//   cnt[max(RB, m)] scratch for the counts, block_sum scan temporaries, total (int64)
struct BlockPlan {
  int* hdr;
  int* rb_ptr;
  int* blk_col;
  int* blk_ent;
  int* rem_pos;
  int* rem_ent;
  int* cnt;
  long long* block_sum;
  long long* total;
  int RB;
  long long capB;
  size_t bytes;
};

static size_t al(size_t x) { return (x + 255) & ~(size_t)255; }

static BlockPlan block_plan_view(void* base, int64_t m, int64_t nnz) {
  BlockPlan p;
  char* c = static_cast<char*>(base);
  size_t off = 0;
  p.RB = (int)ceil_div(m, 16);
  p.capB = nnz / 256 + 1;
  p.hdr = reinterpret_cast<int*>(c + off); off += al(16 * 4);
  p.rb_ptr = reinterpret_cast<int*>(c + off); off += al((size_t)(p.RB + 1) * 4);
  p.blk_col = reinterpret_cast<int*>(c + off); off += al((size_t)p.capB * 4);
  p.blk_ent = reinterpret_cast<int*>(c + off); off += al((size_t)p.capB * 16 * 4);
  p.rem_pos = reinterpret_cast<int*>(c + off); off += al((size_t)(m + 1) * 4);
  p.rem_ent = reinterpret_cast<int*>(c + off); off += al((size_t)(nnz + 1) * 4);
  const int64_t cn = (m > p.RB ? m : p.RB) + 1;
  p.cnt = reinterpret_cast<int*>(c + off); off += al((size_t)cn * 4);
  p.block_sum = reinterpret_cast<long long*>(c + off); off += al((size_t)(ceil_div(cn, 4096) + 1) * 8);
  p.total = reinterpret_cast<long long*>(c + off); off += al(16);
  p.bytes = off;
  return p;
}

// ---- plan construction ------------------------------------------------------------------------------
// lower bound of column c in row [b, e)
__device__ __forceinline__ int find_col(const int* __restrict__ crd, int b, int e, int c) {
  while (b < e) {
    const int mid = (b + e) >> 1;
    if (__ldg(crd + mid) < c) b = mid + 1; else e = mid;
  }
  return b;
}

// One warp per row block.  Candidate blocks come from the aligned 16-column runs of the block's
// first row; lanes 0..15 then check the same run in "their" row with a binary search.
template <bool WRITE>
__global__ void __launch_bounds__(128)
block_detect_kernel(int m, int RB, const int* __restrict__ pos, const int* __restrict__ crd,
                    int* __restrict__ cnt, const int* __restrict__ rb_ptr, int* __restrict__ blk_col,
                    int* __restrict__ blk_ent) {
  const int rb = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (rb >= RB) return;
  const int i0 = rb * 16;
  int found = 0;
  if (i0 + 16 <= m) {
    const int my_row = i0 + (lane & 15);
    const int rb_ = __ldg(pos + my_row), re_ = __ldg(pos + my_row + 1);
    const int b0 = __ldg(pos + i0), e0 = __ldg(pos + i0 + 1);
    const int base = WRITE ? __ldg(rb_ptr + rb) : 0;
    for (int p0 = b0; p0 < e0; p0 += 32) {
      const int p = p0 + lane;
      int c = -1;
      bool cand = false;
      if (p < e0) {
        c = __ldg(crd + p);
        cand = ((c & 15) == 0) && (p + 15 < e0) && (__ldg(crd + p + 15) == c + 15);
      }
      unsigned todo = __ballot_sync(FULL, cand);
      while (todo) {
        const int src = __ffs(todo) - 1;
        todo &= todo - 1;
        const int c0 = __shfl_sync(FULL, c, src);
        bool ok = true;
        int q = 0;
        if (lane < 16) {
          q = find_col(crd, rb_, re_, c0);
          ok = (q + 15 < re_) && (__ldg(crd + q) == c0) && (__ldg(crd + q + 15) == c0 + 15);
        }
        if (__all_sync(FULL, ok)) {
          if (WRITE) {
            if (lane == 0) blk_col[base + found] = c0 >> 4;
            if (lane < 16) blk_ent[(long long)(base + found) * 16 + lane] = q;
          }
          found++;
        }
      }
    }
  }
  if (!WRITE && lane == 0) cnt[rb] = found;
}

__global__ void rem_count_kernel(int m, const int* __restrict__ pos, const int* __restrict__ rb_ptr,
                                 int* __restrict__ cnt) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= m) return;
  const int rb = i >> 4;
  cnt[i] = (pos[i + 1] - pos[i]) - 16 * (rb_ptr[rb + 1] - rb_ptr[rb]);
}

// One warp per row: keeps the entries whose column block is not a dense block of the row block.
__global__ void __launch_bounds__(256)
rem_fill_kernel(int m, const int* __restrict__ pos, const int* __restrict__ crd,
                const int* __restrict__ rb_ptr, const int* __restrict__ blk_col,
                const int* __restrict__ rem_pos, int* __restrict__ rem_ent) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= m) return;
  const int b = __ldg(pos + row), e = __ldg(pos + row + 1);
  const int kb = __ldg(rb_ptr + (row >> 4)), ke = __ldg(rb_ptr + (row >> 4) + 1);
  int outp = __ldg(rem_pos + row);
  for (int p0 = b; p0 < e; p0 += 32) {
    const int p = p0 + lane;
    bool keep = false;
    if (p < e) {
      const int cb = __ldg(crd + p) >> 4;
      int lo = kb, hi = ke;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(blk_col + mid) < cb) lo = mid + 1; else hi = mid;
      }
      keep = !(lo < ke && __ldg(blk_col + lo) == cb);
    }
    const unsigned mask = __ballot_sync(FULL, keep);
    if (keep) rem_ent[outp + __popc(mask & ((1u << lane) - 1))] = p;
    outp += __popc(mask);
  }
}

struct BlockArgs {
  int m;
  const int* rb_ptr;
  const int* blk_col;
  const int* blk_ent;
  int RB;
};

// ---- SDDMM over the dense blocks -----------------------------------------------------------------------
// One warp per row block (16 mask rows); its Q rows stay in registers as pre-split TF32 pairs.
// Fragment layout of mma.m16n8k8 (g = lane/4, t = lane%4): A rows g, g+8 / k columns t, t+4;
// B k rows t, t+4 / column g; C rows g, g+8 / columns 2t, 2t+1.  The k index is a free
// permutation as long as A and B agree: k-step (2q+h) uses elements 16q + 4t + 2h (+1) of the
// feature dimension, so every thread reads its Q and K operands with 128-bit loads.
template <int D16>  // d = 16 * D16
__global__ void __launch_bounds__(128)
sddmm_block_kernel(BlockArgs a, const float* __restrict__ Q, unsigned ldq,
                   const float* __restrict__ K, unsigned ldk, const float* __restrict__ mask_val,
                   float* __restrict__ out, long long stride_q, long long stride_k,
                   long long stride_out) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rb = blockIdx.x * 4 + warp;
  if (rb >= a.RB) return;
  const int kb = __ldg(a.rb_ptr + rb), ke = __ldg(a.rb_ptr + rb + 1);
  if (kb == ke) return;
  const int g = lane >> 2, t = lane & 3;
  const long long bz = blockIdx.y;
  Q += bz * stride_q;
  K += bz * stride_k;
  out += bz * stride_out;
  const int i0 = rb * 16;

  unsigned qhi[2][D16][4], qlo[2][D16][4];
#pragma unroll
  for (int r = 0; r < 2; r++) {
    const float* qrow = Q + (size_t)((unsigned long long)(unsigned)(i0 + g + 8 * r) * ldq) + 4 * t;
#pragma unroll
    for (int q = 0; q < D16; q++) {
      const float4 v = ldg4(qrow + 16 * q);
      split_tf32(v.x, qhi[r][q][0], qlo[r][q][0]);
      split_tf32(v.y, qhi[r][q][1], qlo[r][q][1]);
      split_tf32(v.z, qhi[r][q][2], qlo[r][q][2]);
      split_tf32(v.w, qhi[r][q][3], qlo[r][q][3]);
    }
  }

  // software pipeline over the row block's dense blocks: the K rows of block b+1 are in flight
  // while block b is multiplied
  float4 kf[2][D16], kn[2][D16];
  auto load_k = [&](int b, float4 (&dst)[2][D16]) {
    const int j0 = __ldg(a.blk_col + b) * 16;
#pragma unroll
    for (int n = 0; n < 2; n++) {
      const float* krow = K + (size_t)((unsigned long long)(unsigned)(j0 + 8 * n + g) * ldk) + 4 * t;
#pragma unroll
      for (int q = 0; q < D16; q++) dst[n][q] = ldg4(krow + 16 * q);
    }
  };
  load_k(kb, kn);
  for (int b = kb; b < ke; b++) {
#pragma unroll
    for (int n = 0; n < 2; n++) {
#pragma unroll
      for (int q = 0; q < D16; q++) kf[n][q] = kn[n][q];
    }
    const int p0 = __ldg(a.blk_ent + (long long)b * 16 + g);
    const int p1 = __ldg(a.blk_ent + (long long)b * 16 + g + 8);
    if (b + 1 < ke) load_k(b + 1, kn);
    // main and cross terms accumulate separately: shorter dependent mma chains
    float c[2][4], x[2][4];
#pragma unroll
    for (int n = 0; n < 2; n++) {
      c[n][0] = c[n][1] = c[n][2] = c[n][3] = 0.f;
      x[n][0] = x[n][1] = x[n][2] = x[n][3] = 0.f;
    }
#pragma unroll
    for (int q = 0; q < D16; q++) {
#pragma unroll
      for (int h = 0; h < 2; h++) {
        const unsigned ahi[4] = {qhi[0][q][2 * h], qhi[1][q][2 * h], qhi[0][q][2 * h + 1],
                                 qhi[1][q][2 * h + 1]};
        const unsigned alo[4] = {qlo[0][q][2 * h], qlo[1][q][2 * h], qlo[0][q][2 * h + 1],
                                 qlo[1][q][2 * h + 1]};
#pragma unroll
        for (int n = 0; n < 2; n++) {
          const float k0 = h ? kf[n][q].z : kf[n][q].x;
          const float k1 = h ? kf[n][q].w : kf[n][q].y;
          unsigned bh0, bl0, bh1, bl1;
          split_tf32(k0, bh0, bl0);
          split_tf32(k1, bh1, bl1);
          mma_tf32(x[n], alo, bh0, bh1);
          mma_tf32(x[n], ahi, bl0, bl1);
          mma_tf32(c[n], ahi, bh0, bh1);
        }
      }
    }
#pragma unroll
    for (int n = 0; n < 2; n++) {
      const int col = 8 * n + 2 * t;
      float s00 = 1.f, s01 = 1.f, s10 = 1.f, s11 = 1.f;
      if (mask_val) {
        s00 = __ldg(mask_val + p0 + col); s01 = __ldg(mask_val + p0 + col + 1);
        s10 = __ldg(mask_val + p1 + col); s11 = __ldg(mask_val + p1 + col + 1);
      }
      out[p0 + col] = s00 * (c[n][0] + x[n][0]);
      out[p0 + col + 1] = s01 * (c[n][1] + x[n][1]);
      out[p1 + col] = s10 * (c[n][2] + x[n][2]);
      out[p1 + col + 1] = s11 * (c[n][3] + x[n][3]);
    }
  }
}

// ---- SpMM over the dense blocks ------------------------------------------------------------------------
// One warp per row block: C (16 x k) accumulates in registers over the row block's dense blocks
// and is written once (rows of row blocks without dense blocks are written as zeros, so that the
// remainder kernel can add to every row).  Column permutation: logical column (tile u, n) is
// actual column n*KT + u, so thread g reads KT contiguous floats of each V row and writes KT
// contiguous floats of each output row.
template <int KT>  // k = 8 * KT
__global__ void __launch_bounds__(128)
spmm_block_kernel(BlockArgs a, const float* __restrict__ val, const float* __restrict__ B,
                  unsigned ldb, float* __restrict__ C, long long ldc, long long stride_val,
                  long long stride_b, long long stride_c) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rb = blockIdx.x * 4 + warp;
  if (rb >= a.RB) return;
  const int g = lane >> 2, t = lane & 3;
  const long long bz = blockIdx.y;
  val += bz * stride_val;
  B += bz * stride_b;
  C += bz * stride_c;
  const int kb = __ldg(a.rb_ptr + rb), ke = __ldg(a.rb_ptr + rb + 1);
  const int i0 = rb * 16;

  float c[KT][4];
#pragma unroll
  for (int u = 0; u < KT; u++) c[u][0] = c[u][1] = c[u][2] = c[u][3] = 0.f;

  // (prefetching the next block's operands was measured here and lost: 147 registers)
  for (int b = kb; b < ke; b++) {
    const int j0 = __ldg(a.blk_col + b) * 16;
    const int p0 = __ldg(a.blk_ent + (long long)b * 16 + g);
    const int p1 = __ldg(a.blk_ent + (long long)b * 16 + g + 8);
    float pa[2][4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
      pa[0][e] = __ldg(val + p0 + 4 * t + e);
      pa[1][e] = __ldg(val + p1 + 4 * t + e);
    }
    // V rows j0 + 4t + {0..3}, KT contiguous floats at column g*KT
    float vb[4][KT];
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const float* vrow = B + (size_t)((unsigned long long)(unsigned)(j0 + 4 * t + e) * ldb) + g * KT;
#pragma unroll
      for (int u = 0; u < KT; u += 4) {
        const float4 x = ldg4(vrow + u);
        vb[e][u] = x.x; vb[e][u + 1] = x.y; vb[e][u + 2] = x.z; vb[e][u + 3] = x.w;
      }
    }
#pragma unroll
    for (int s = 0; s < 2; s++) {
      unsigned ahi[4], alo[4];
      split_tf32(pa[0][2 * s], ahi[0], alo[0]);
      split_tf32(pa[1][2 * s], ahi[1], alo[1]);
      split_tf32(pa[0][2 * s + 1], ahi[2], alo[2]);
      split_tf32(pa[1][2 * s + 1], ahi[3], alo[3]);
#pragma unroll
      for (int u = 0; u < KT; u++) {
        unsigned bh0, bl0, bh1, bl1;
        split_tf32(vb[2 * s][u], bh0, bl0);
        split_tf32(vb[2 * s + 1][u], bh1, bl1);
        mma_3xtf32(c[u], ahi, alo, bh0, bh1, bl0, bl1);
      }
    }
  }
  // C rows g, g+8; logical columns (u, 2t+e) -> actual (2t+e)*KT + u
#pragma unroll
  for (int r = 0; r < 2; r++) {
    const int row = i0 + g + 8 * r;
    if (row >= a.m) continue;
    float* crow = C + (long long)row * ldc;
#pragma unroll
    for (int e = 0; e < 2; e++) {
#pragma unroll
      for (int u = 0; u < KT; u += 4) {
        const float4 x = make_float4(c[u][2 * r + e], c[u + 1][2 * r + e], c[u + 2][2 * r + e],
                                     c[u + 3][2 * r + e]);
        *reinterpret_cast<float4*>(crow + (2 * t + e) * KT + u) = x;
      }
    }
  }
}

}  // namespace sb

using namespace sb;

extern "C" {

size_t sb_block_plan_bytes(int64_t m, int64_t nnz) {
  if (m < 0) m = 0;
  if (nnz < 0) nnz = 0;
  return block_plan_view(nullptr, m, nnz).bytes;
}

int sb_block_plan_build(int64_t m, int64_t n, int64_t nnz, const int32_t* pos, const int32_t* crd,
                        void* plan, size_t plan_bytes, int64_t* blocks_host, int64_t* rem_nnz_host,
                        void* stream) {
  (void)n;
  SB_CHECK_ARG(m >= 0 && nnz >= 0 && m < INT32_MAX - 16 && nnz < INT32_MAX, "block_plan: bad size");
  SB_CHECK_ARG(pos && plan && (crd || nnz == 0), "block_plan: null pointer");
  SB_CHECK_ARG(aligned16(plan), "block_plan: plan must be 16-byte aligned");
  BlockPlan p = block_plan_view(plan, m, nnz);
  if (plan_bytes < p.bytes)
    return fail(SB_ERR_WORKSPACE, "block_plan: buffer has %zu bytes, needs %zu", plan_bytes, p.bytes);
  cudaStream_t st = (cudaStream_t)stream;
  SB_CUDA(cudaMemsetAsync(p.hdr, 0, 64, st));
  long long nblk = 0, nrem = 0;
  if (m > 0) {
    const unsigned wg = (unsigned)ceil_div((int64_t)p.RB * 32, 128);
    block_detect_kernel<false><<<wg, 128, 0, st>>>((int)m, p.RB, pos, crd, p.cnt, nullptr, nullptr, nullptr);
    SB_LAUNCH_CHECK("block_detect_kernel<count>");
    int rc = exclusive_scan_i32(p.RB, p.cnt, p.rb_ptr, p.block_sum, p.total, st);
    if (rc != SB_OK) return rc;
    SB_CUDA(cudaMemcpyAsync(&nblk, p.total, 8, cudaMemcpyDeviceToHost, st));
    block_detect_kernel<true><<<wg, 128, 0, st>>>((int)m, p.RB, pos, crd, p.cnt, p.rb_ptr, p.blk_col, p.blk_ent);
    SB_LAUNCH_CHECK("block_detect_kernel<fill>");
    rem_count_kernel<<<(unsigned)ceil_div(m, 256), 256, 0, st>>>((int)m, pos, p.rb_ptr, p.cnt);
    SB_LAUNCH_CHECK("rem_count_kernel");
    rc = exclusive_scan_i32((int)m, p.cnt, p.rem_pos, p.block_sum, p.total, st);
    if (rc != SB_OK) return rc;
    SB_CUDA(cudaMemcpyAsync(&nrem, p.total, 8, cudaMemcpyDeviceToHost, st));
    rem_fill_kernel<<<(unsigned)ceil_div(m * 32, 256), 256, 0, st>>>((int)m, pos, crd, p.rb_ptr, p.blk_col,
                                                                   p.rem_pos, p.rem_ent);
    SB_LAUNCH_CHECK("rem_fill_kernel");
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

int sb_sddmm_csr_blocked_f32(int64_t m, int64_t n, int64_t d, int64_t nnz, const int32_t* pos,
                             const int32_t* crd, const float* mask_val, const float* Q, int64_t ldq,
                             const float* K, int64_t ldk, float* out_val, int64_t batch,
                             int64_t stride_q, int64_t stride_k, int64_t stride_out,
                             const void* block_plan, int64_t blocks, int64_t rem_nnz, void* stream) {
  (void)n; (void)pos;
  SB_CHECK_ARG(m >= 0 && nnz >= 0 && m < INT32_MAX - 16 && nnz < INT32_MAX, "sddmm_blocked: bad size");
  SB_CHECK_ARG(block_plan && crd && Q && K && out_val, "sddmm_blocked: null pointer");
  SB_CHECK_ARG(batch >= 1 && batch <= 65535, "sddmm_blocked: batch must be in [1, 65535]");
  SB_CHECK_ARG(d == 16 || d == 32 || d == 64 || d == 128, "sddmm_blocked: d must be 16, 32, 64 or 128");
  SB_CHECK_ARG(ldq % 4 == 0 && ldk % 4 == 0 && aligned16(Q) && aligned16(K) && stride_q % 4 == 0 &&
               stride_k % 4 == 0 && ldq < (1ll << 32) && ldk < (1ll << 32),
               "sddmm_blocked: Q/K must be 16-byte aligned with row pitches that are multiples of 4");
  SB_CHECK_ARG(blocks >= 0 && rem_nnz >= 0 && blocks * 256 + rem_nnz == nnz,
               "sddmm_blocked: block/remainder counts do not add up to nnz");
  cudaStream_t st = (cudaStream_t)stream;
  BlockPlan p = block_plan_view(const_cast<void*>(block_plan), m, nnz);
  if (blocks > 0) {
    BlockArgs a{(int)m, p.rb_ptr, p.blk_col, p.blk_ent, p.RB};
    dim3 grid((unsigned)ceil_div(p.RB, 4), (unsigned)batch);
#define SB_SDDMM_BLK(D16)                                                                        \
  sddmm_block_kernel<D16><<<grid, 128, 0, st>>>(a, Q, (unsigned)ldq, K, (unsigned)ldk, mask_val,  \
                                                out_val, stride_q, stride_k, stride_out)
    if (d == 16) SB_SDDMM_BLK(1);
    else if (d == 32) SB_SDDMM_BLK(2);
    else if (d == 64) SB_SDDMM_BLK(4);
    else SB_SDDMM_BLK(8);
#undef SB_SDDMM_BLK
    SB_LAUNCH_CHECK("sddmm_block_kernel");
  }
  if (rem_nnz > 0)
    return sddmm_remainder(m, d, rem_nnz, p.rem_pos, p.rem_ent, crd, mask_val, Q, ldq, K, ldk, out_val,
                           batch, stride_q, stride_k, stride_out, 0, st);
  return SB_OK;
}

int sb_spmm_csr_blocked_f32(int64_t m, int64_t n, int64_t k, int64_t nnz, const int32_t* pos,
                            const int32_t* crd, const float* val, const float* B, int64_t ldb,
                            const float* bias, int relu, float* C, int64_t ldc, int64_t batch,
                            int64_t stride_val, int64_t stride_b, int64_t stride_c,
                            const void* block_plan, int64_t blocks, int64_t rem_nnz, void* stream) {
  (void)n; (void)pos;
  SB_CHECK_ARG(m >= 0 && nnz >= 0 && m < INT32_MAX - 16 && nnz < INT32_MAX, "spmm_blocked: bad size");
  SB_CHECK_ARG(block_plan && crd && val && B && C, "spmm_blocked: null pointer");
  SB_CHECK_ARG(batch >= 1 && batch <= 65535, "spmm_blocked: batch must be in [1, 65535]");
  SB_CHECK_ARG(k == 32 || k == 64 || k == 128, "spmm_blocked: k must be 32, 64 or 128");
  SB_CHECK_ARG(ldb % 4 == 0 && ldc % 4 == 0 && aligned16(B) && aligned16(C) && stride_b % 4 == 0 &&
               stride_c % 4 == 0 && ldb < (1ll << 32) && (!bias || aligned16(bias)),
               "spmm_blocked: B/C must be 16-byte aligned with row pitches that are multiples of 4");
  SB_CHECK_ARG(blocks >= 0 && rem_nnz >= 0 && blocks * 256 + rem_nnz == nnz,
               "spmm_blocked: block/remainder counts do not add up to nnz");
  if (m == 0) return SB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  BlockPlan p = block_plan_view(const_cast<void*>(block_plan), m, nnz);
  BlockArgs a{(int)m, p.rb_ptr, p.blk_col, p.blk_ent, p.RB};
  dim3 grid((unsigned)ceil_div(p.RB, 4), (unsigned)batch);
#define SB_SPMM_BLK(KT)                                                                       \
  spmm_block_kernel<KT><<<grid, 128, 0, st>>>(a, val, B, (unsigned)ldb, C, ldc, stride_val,    \
                                              stride_b, stride_c)
  if (k == 32) SB_SPMM_BLK(4);
  else if (k == 64) SB_SPMM_BLK(8);
  else SB_SPMM_BLK(16);
#undef SB_SPMM_BLK
  SB_LAUNCH_CHECK("spmm_block_kernel");
  // the remainder kernel adds its rows to C and applies bias / ReLU (also when rem_nnz == 0)
  return spmm_remainder(m, k, p.rem_pos, p.rem_ent, crd, val, B, ldb, bias, relu, C, ldc, batch,
                        stride_val, stride_b, stride_c, 0, st);
}

}  // extern "C"
