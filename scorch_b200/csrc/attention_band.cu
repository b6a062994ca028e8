// Sparse attention over a banded CSR mask on the 5th-generation tensor cores (tcgen05 + TMEM):
//   O = softmax_rows(scale * mask_val .* (Q K^T) on the stored entries) V
// (reference caller: bench/bench_sparse_transformer.py:304-382, three operators per head).
//
// A band plan cuts the mask rows into tiles of 128 and gives every tile a window of 384
// consecutive columns around the diagonal.  The stored entries inside the window are described by
// a 384-bit mask per row (+ the index of the row's first entry in the window, for the mask
// values); the entries outside go to a CSR remainder list, which the scattered-entry kernel of
// attention.cu handles first, leaving per row an unnormalised output and (maximum, sum).
//
// attn_band_kernel, one CTA of nine warps per (tile, head): eight warps stage operands and own the
// rows, lane 0 of the ninth issues the tensor-core work (so that issuing overlaps the others' work):
//   1. Q tile and K window rows are read with plain loads (into registers ahead of the point where
//      their shared-memory buffer is free), split into TF32 hi / lo parts and stored to shared
//      memory in the tensor core's canonical K-major layout without swizzle (core matrix = 8 rows
//      x 16 bytes, the cores of one 8-row group side by side);
//   2. S = Q K^T  is issued as tcgen05.mma kind::tf32 (M 128, N 128, K 8) in three passes
//      (lo*hi, hi*lo, hi*hi: the 3xTF32 split, fp32-level accuracy) into 384 TMEM columns, one K
//      piece of 128 window columns at a time through two buffers;
//   3. every thread of the eight warps owns one row and half of the columns: it reads its scores
//      with tcgen05.ld, masks the entries that are not stored (without branches), applies scale
//      and mask values, takes the row maxima piece by piece while the next piece's products run,
//      and then writes P = exp2(S - max) back as hi (in place) and lo (64 spare columns);
//   4. O += P V  is issued with P read from TMEM as the A operand and V^T (transposed while it is
//      staged, so that it is K-major like K) as the B operand, 64 window columns at a time;
//   5. the epilogue reads O from TMEM, merges the scattered entries' (max, sum, O) and writes O / sum.
// TMEM: columns [0,384) S / P_hi, [384,448) O, [448,512) P_lo.  Every mbarrier wait is bounded by
// a clock limit; a wait that runs out sets a status word (sb_attn_band_status), the CTA frees its
// TMEM and returns.  No TMA, no multicast, no cluster: every operand goes through registers for
// the hi / lo split anyway.
#include <algorithm>

#include "attention.cuh"
#include "common.cuh"

namespace sb {

constexpr int kBandRows = SB_ATTN_BAND_ROWS;    // mask rows per tile
constexpr int kBandCols = SB_ATTN_BAND_COLS;    // columns of a tile's window
constexpr int kBandWords = kBandCols / 32;      // 32-bit words of a row's stored-column mask
constexpr int kBandWorkWarps = 8;              // warps that stage operands and do the softmax
constexpr int kBandThreads = (kBandWorkWarps + 1) * 32;   // + one warp whose lane 0 issues the tensor-core work
constexpr int kTmemCols = 512;
constexpr int kTmemO = 384;                     // first TMEM column of the output accumulator
constexpr int kTmemPlo = 448;                   // first TMEM column of the lo parts of P
constexpr long long kWaitClocks = 2000000000ll; // about a second: bound of every mbarrier wait

__device__ int g_band_status = 0;  // 0 ok; 1 a wait for the tensor cores ran out

// first column of tile t's window
__host__ __device__ inline int band_window_start(int tile, int n) {
  int c = tile * kBandRows - (kBandCols - kBandRows) / 2;
  if (c > n - kBandCols) c = n - kBandCols;
  return c < 0 ? 0 : c;
}

// ---- plan layout ---------------------------------------------------------------------------------
// int32 words: hdr[16] ([0] entries inside the windows, [1] remainder entries), then
//   ent0[m]            index of the row's first stored entry inside its tile's window
//   bits[m*12]         stored columns of the row inside the window, bit c = column window_start + c
//   rem_pos[m+1], rem_ent[nnz], rem_crd[nnz]   CSR of the entries outside the windows
//   cnt[m+1], block_sum, total                 scan temporaries
struct BandPlan {
  int* hdr;
  int* ent0;
  unsigned* bits;
  int* rem_pos;
  int* rem_ent;
  int* rem_crd;
  int* cnt;
  long long* block_sum;
  long long* total;
  size_t bytes;
};

static size_t band_al256(size_t x) { return (x + 255) & ~(size_t)255; }

static BandPlan band_plan_view(void* base, int64_t m, int64_t nnz) {
  BandPlan p;
  char* c = static_cast<char*>(base);
  size_t off = 0;
  p.hdr = reinterpret_cast<int*>(c + off); off += band_al256(16 * 4);
  p.ent0 = reinterpret_cast<int*>(c + off); off += band_al256((size_t)(m + 1) * 4);
  p.bits = reinterpret_cast<unsigned*>(c + off); off += band_al256((size_t)(m + 1) * kBandWords * 4);
  p.rem_pos = reinterpret_cast<int*>(c + off); off += band_al256((size_t)(m + 1) * 4);
  p.rem_ent = reinterpret_cast<int*>(c + off); off += band_al256((size_t)(nnz + 1) * 4);
  p.rem_crd = reinterpret_cast<int*>(c + off); off += band_al256((size_t)(nnz + 1) * 4);
  p.cnt = reinterpret_cast<int*>(c + off); off += band_al256((size_t)(m + 1) * 4);
  p.block_sum = reinterpret_cast<long long*>(c + off); off += band_al256((size_t)(ceil_div(m + 1, 4096) + 1) * 8);
  p.total = reinterpret_cast<long long*>(c + off); off += band_al256(16);
  p.bytes = off;
  return p;
}

__device__ __forceinline__ int band_lower_bound(const int* __restrict__ crd, int b, int e, int c) {
  while (b < e) {
    const int mid = (b + e) >> 1;
    if (__ldg(crd + mid) < c) b = mid + 1; else e = mid;
  }
  return b;
}

// One warp per mask row: the row's entries inside the window become bits; the others are counted.
__global__ void __launch_bounds__(256)
band_rows_kernel(int m, int n, const int* __restrict__ pos, const int* __restrict__ crd,
                 int* __restrict__ ent0, unsigned* __restrict__ bits, int* __restrict__ cnt,
                 unsigned long long* __restrict__ inside) {
  __shared__ unsigned s_bits[8][kBandWords];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  if (row >= m) return;
  const int b = __ldg(pos + row), e = __ldg(pos + row + 1);
  const int c0 = band_window_start(row / kBandRows, n);
  const int e0 = band_lower_bound(crd, b, e, c0);
  const int e1 = band_lower_bound(crd, e0, e, c0 + kBandCols);
  if (lane < kBandWords) s_bits[warp][lane] = 0u;
  __syncwarp();
  for (int p = e0 + lane; p < e1; p += 32) {
    const int c = __ldg(crd + p) - c0;
    atomicOr(&s_bits[warp][c >> 5], 1u << (c & 31));
  }
  __syncwarp();
  if (lane < kBandWords) bits[(size_t)row * kBandWords + lane] = s_bits[warp][lane];
  if (lane == 0) {
    ent0[row] = e0;
    cnt[row] = (e - b) - (e1 - e0);
    if (e1 > e0) atomicAdd(inside, (unsigned long long)(e1 - e0));
  }
}

// One warp per mask row: entry index and column of the entries outside the window, in row order.
__global__ void __launch_bounds__(256)
band_rem_kernel(int m, int n, const int* __restrict__ pos, const int* __restrict__ crd,
                const int* __restrict__ ent0, const int* __restrict__ rem_pos, int* __restrict__ rem_ent,
                int* __restrict__ rem_crd) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  if (row >= m) return;
  const int b = __ldg(pos + row), e = __ldg(pos + row + 1);
  const int c0 = band_window_start(row / kBandRows, n);
  const int e0 = __ldg(ent0 + row);
  const int e1 = band_lower_bound(crd, e0, e, c0 + kBandCols);
  const int dst = __ldg(rem_pos + row);
  for (int p = b + lane; p < e0; p += 32) {
    rem_ent[dst + (p - b)] = p;
    rem_crd[dst + (p - b)] = __ldg(crd + p);
  }
  for (int p = e1 + lane; p < e; p += 32) {
    rem_ent[dst + (e0 - b) + (p - e1)] = p;
    rem_crd[dst + (e0 - b) + (p - e1)] = __ldg(crd + p);
  }
}

// ---- tcgen05 / mbarrier wrappers ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Shared-memory matrix descriptor, no swizzle: start address, leading-dimension and stride byte
// offsets in 16-byte units, descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((saddr >> 4) & 0x3fffu) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46);
}
// Instruction descriptor of kind::tf32 with fp32 accumulation: D format F32 (bits 4-5 = 1), A and B
// format TF32 (bits 7-9, 10-12 = 2), B major (bit 16: 1 = MN-major), N / 8 (bits 17-22), M / 16 (24-28).
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int M, int N, int b_mn_major) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// the mbarrier receives one arrival when every tcgen05.mma issued so far by this thread is done
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void async_proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 32 consecutive TMEM columns of this thread's lane (= matrix row)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
      "%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),
        "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Waits for the given phase of the mbarrier, at most kWaitClocks; false when the wait ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  const long long t0 = clock64();
  for (;;) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if (clock64() - t0 > kWaitClocks) return false;
  }
}

struct BandArgs {
  int n;
  const int* ent0;
  const unsigned* bits;
  float* raw_scores;   // probe only: the tile's 128 x 384 products Q K^T, unscaled and unmasked
  float* tmem_image;   // probe only: the tile's 128 x 512 tensor-memory cells after the last O += P V
  int probe_tile;
  long long* clocks;   // probe only: clock64() of thread 0 at the kernel's phase boundaries
  int last_entry;      // nnz - 1 (bound of the mask-value reads)
};

// Rows [row0, row0 + ROWS) of a row-major matrix (row pitch ld floats, rows outside [0, limit)
// read as zeros) -> hi / lo parts in the canonical layout: 8-row groups of 8 * D floats; inside a
// group the 16-byte pieces (4 features) of the 8 rows are contiguous (128 bytes per core matrix),
// the D / 4 cores of the group side by side.  Lanes: 8 rows x 4 neighbouring cores = 512
// contiguous bytes of shared memory per warp store, 64 contiguous bytes of each row per load.
// Two halves, so that a piece can be loaded into registers while the buffer it goes to is still
// being read by the tensor cores.
template <int D, int ROWS>
struct BandPiece {
  static constexpr int QG = D / 16;                       // groups of 4 cores per row group
  static constexpr int TASKS = (ROWS / 8) * QG;           // (row group, core group) pairs, one per warp pass
  static constexpr int PASSES = TASKS / kBandWorkWarps;
  static_assert(TASKS % kBandWorkWarps == 0, "staging tasks must divide over the warps");
  float4 v[PASSES];

  __device__ __forceinline__ void load(const float* __restrict__ src, unsigned ld, int row0, int limit) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r8 = lane & 7, q4 = lane >> 3;
#pragma unroll
    for (int i = 0; i < PASSES; i++) {
      const int task = i * kBandWorkWarps + warp;
      const int rg = task / QG, core = (task % QG) * 4 + q4;
      const int row = row0 + rg * 8 + r8;
      v[i] = (row >= 0 && row < limit)
                 ? __ldg(reinterpret_cast<const float4*>(src + (size_t)((unsigned long long)(unsigned)row * ld) + core * 4))
                 : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  __device__ __forceinline__ void store(float* __restrict__ hi, float* __restrict__ lo) const {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r8 = lane & 7, q4 = lane >> 3;
#pragma unroll
    for (int i = 0; i < PASSES; i++) {
      const int task = i * kBandWorkWarps + warp;
      const int rg = task / QG, core = (task % QG) * 4 + q4;
      const int off = rg * 8 * D + core * 32 + r8 * 4;
      uint4 h, l;
      attn_split(v[i].x, h.x, l.x); attn_split(v[i].y, h.y, l.y);
      attn_split(v[i].z, h.z, l.z); attn_split(v[i].w, h.w, l.w);
      *reinterpret_cast<uint4*>(hi + off) = h;
      *reinterpret_cast<uint4*>(lo + off) = l;
    }
  }
};

// 64 rows [row0, row0 + 64) of V (row pitch ld floats, rows outside [0, limit) read as zeros) ->
// hi / lo parts of their transpose in the same canonical layout: "rows" are now the D features,
// the 64 window columns are the contiguous (K) direction, so an 8-feature group holds 16 cores of
// 128 bytes.  (The B operand of O += P V has to be K-major: with the descriptor's B-major bit set
// the tf32 instruction left the accumulator untouched on this hardware.)  A thread gathers four
// consecutive window columns of one feature with scalar loads (a warp reads 128 contiguous bytes
// per load) and stores them as one 16-byte piece; the 8 lanes of a feature group fill one core
// matrix, so the stores are free of bank conflicts.
template <int D>
struct BandPieceT {
  static constexpr int HALVES = D / 32;
  static constexpr int ITEMS = HALVES * 2;   // (32-feature half, 4-column block) pairs per thread: 16 blocks over 8 warps
  float v[ITEMS][4];

  __device__ __forceinline__ void load(const float* __restrict__ src, unsigned ld, int row0, int limit) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int it = 0; it < ITEMS; it++) {
      const int f = (it % HALVES) * 32 + lane, jb = warp * 2 + it / HALVES;
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {
        const int row = row0 + jb * 4 + jj;
        v[it][jj] = (row >= 0 && row < limit) ? __ldg(src + (size_t)((unsigned long long)(unsigned)row * ld) + f) : 0.f;
      }
    }
  }
  __device__ __forceinline__ void store(float* __restrict__ hi, float* __restrict__ lo) const {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int it = 0; it < ITEMS; it++) {
      const int f = (it % HALVES) * 32 + lane, jb = warp * 2 + it / HALVES;
      const int off = (f >> 3) * (16 * 32) + jb * 32 + (f & 7) * 4;   // floats
      uint4 h, l;
      attn_split(v[it][0], h.x, l.x); attn_split(v[it][1], h.y, l.y);
      attn_split(v[it][2], h.z, l.z); attn_split(v[it][3], h.w, l.w);
      *reinterpret_cast<uint4*>(hi + off) = h;
      *reinterpret_cast<uint4*>(lo + off) = l;
    }
  }
};

template <int D>
__global__ void __launch_bounds__(kBandThreads, 1)
attn_band_kernel(AttnArgs a, BandArgs b) {
  extern __shared__ __align__(128) unsigned char band_smem[];
  constexpr int TILE_FLOATS = kBandRows * D;           // one 128 x D operand part (hi or lo)
  constexpr int VT_FLOATS = 64 * D;                    // one part of a transposed 64-row piece of V
  constexpr uint32_t GROUP_BYTES = 8 * D * 4;          // an 8-row group: stride between row groups
  constexpr uint32_t VT_GROUP_BYTES = (64 / 4) * 128;  // 8 features x 64 window columns of V^T
  constexpr uint32_t CORE_BYTES = 128;                 // a core matrix: stride between neighbouring cores
  constexpr int KSTEPS = D / 8;                        // tcgen05.mma steps over the head dimension
  constexpr int ROUNDS = kBandCols / 64;               // O += P V, 64 window columns per round
  float* q_hi = reinterpret_cast<float*>(band_smem);
  float* q_lo = q_hi + TILE_FLOATS;
  float* kbuf = q_lo + TILE_FLOATS;                    // two K pieces (hi, lo each) = four V^T pieces
  float* s_red = kbuf + 4 * TILE_FLOATS;               // [2][128] row maxima, then row sums
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(s_red + 2 * kBandRows);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
  auto k_hi = [&](int i) { return kbuf + i * 2 * TILE_FLOATS; };
  auto k_lo = [&](int i) { return kbuf + i * 2 * TILE_FLOATS + TILE_FLOATS; };
  auto v_hi = [&](int i) { return kbuf + i * 2 * VT_FLOATS; };
  auto v_lo = [&](int i) { return kbuf + i * 2 * VT_FLOATS + VT_FLOATS; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = b.raw_scores ? b.probe_tile : (int)blockIdx.x;
  const long long bz = blockIdx.y;
  const int i0 = tile * kBandRows;
  const int c0 = band_window_start(tile, b.n);
  const float* Q = a.Q + bz * a.stride_q;
  const float* K = a.K + bz * a.stride_k;
  const float* V = a.V + bz * a.stride_v;
  float* O = a.O + bz * a.stride_o;
  // mbarriers: [0], [1] = the tensor cores are done with K piece buffer 0 / 1; [2] = with a round of O += P V
  const uint32_t bar_k0 = smem_u32(bars), bar_k1 = smem_u32(bars + 1), bar_pv = smem_u32(bars + 2);

  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_k0) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_k1) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_pv) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  int mark_i = 0;
  auto mark = [&]() {
    if (b.clocks && threadIdx.x == 0) b.clocks[mark_i] = clock64();
    mark_i++;
  };
  mark();   // 0

  constexpr uint32_t IDESC_S = umma_idesc_tf32(kBandRows, 128, 0);
  constexpr uint32_t IDESC_O = umma_idesc_tf32(kBandRows, D, 0);

  // Descriptors of the operand parts, built once; a k-step moves the start address by two cores
  // (2 * 128 bytes = 16 units of 16 bytes), which is a plain addition on the descriptor.
  const uint64_t dq_hi = umma_desc(smem_u32(q_hi), CORE_BYTES, GROUP_BYTES);
  const uint64_t dq_lo = umma_desc(smem_u32(q_lo), CORE_BYTES, GROUP_BYTES);
  constexpr uint64_t KSTEP = (2 * CORE_BYTES) >> 4;
  // S[:, 128 c .. 128 c + 127] = Q K_c^T from K piece buffer `buf` (one thread; three passes of the split)
  auto issue_scores = [&](int c, int buf, uint32_t bar) {
    tc_fence_after();
    const uint64_t dk_hi = umma_desc(smem_u32(k_hi(buf)), CORE_BYTES, GROUP_BYTES);
    const uint64_t dk_lo = umma_desc(smem_u32(k_lo(buf)), CORE_BYTES, GROUP_BYTES);
    const uint32_t d_tmem = tmem + (uint32_t)(c * 128);
#pragma unroll
    for (int pass = 0; pass < 3; pass++) {
      const uint64_t aa = pass == 0 ? dq_lo : dq_hi, bb = pass == 1 ? dk_lo : dk_hi;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ks++)
        umma_ss(d_tmem, aa + ks * KSTEP, bb + ks * KSTEP, IDESC_S, (pass | ks) != 0 ? 1u : 0u);
    }
    umma_commit(bar);
  };
  // every thread waits; the outcome is made uniform over the CTA
  auto wait_all = [&](uint32_t bar, uint32_t parity) {
    const bool ok = mbar_wait(bar, parity);
    const bool bad = __syncthreads_or(!ok) != 0;
    tc_fence_after();
    return bad;
  };

  // roles: warps 0..7 stage operands and own the rows (row = TMEM lane; columns 64 g + 32 h + [0, 32)
  // for g = 0..5); lane 0 of warp 8 issues the tensor-core work, so that issuing overlaps the others' work
  const bool worker = warp < kBandWorkWarps;
  const bool issuer = threadIdx.x == kBandWorkWarps * 32;
  const int lane_base = 32 * (warp & 3);
  const int r = lane_base + lane, h = (warp >> 2) & 1;
  const int row = i0 + r;
  const bool live = worker && row < a.m;
  const uint32_t t_row = tmem + ((uint32_t)lane_base << 16);
  const float scale = a.scale * 1.4426950408889634f;   // scores in log2 units
  float M_s = -INFINITY, L_s = 0.f, ms = 0.f, sum = 0.f;
  bool failed = false;

  do {
    // ---- S = Q K^T: K pieces of 128 window columns through two buffers; pieces are loaded into
    // registers ahead of the point where their buffer is free ------------------------------------------------
    BandPiece<D, kBandRows> pq;
    BandPiece<D, 128> pk0, pk1;
    if (worker) {
      pq.load(Q, a.ldq, i0, a.m);
      pk0.load(K, a.ldk, c0, b.n);
      pk1.load(K, a.ldk, c0 + 128, b.n);
      pq.store(q_hi, q_lo);
      pk0.store(k_hi(0), k_lo(0));
    }
    async_proxy_fence();
    __syncthreads();
    mark();   // 1: Q and K piece 0 staged
    if (issuer) issue_scores(0, 0, bar_k0);
    if (worker) {
      pk0.load(K, a.ldk, c0 + 256, b.n);                // piece 2, for buffer 0 once piece 0 is consumed
      pk1.store(k_hi(1), k_lo(1));
    }
    async_proxy_fence();
    __syncthreads();
    mark();   // 2: K piece 1 staged
    if (issuer) issue_scores(1, 1, bar_k1);
    // ---- what the row maxima and the probabilities need: stored-column bits, mask values ---------------------
    unsigned words[kBandWords];
#pragma unroll
    for (int w = 0; w < kBandWords; w++)
      words[w] = !live ? 0u : b.bits ? __ldg(b.bits + (size_t)row * kBandWords + w) : 0xffffffffu;  // (probe: all stored)
    const float* mask_val = (a.mask_val && !__ldg(a.mask_is_ones)) ? a.mask_val : nullptr;
    const int ent0 = (live && b.ent0) ? __ldg(b.ent0 + row) : 0;
    // scores of a 32-column chunk: scaled, times the mask value, -inf where nothing is stored.
    // Without branches: lanes differ in which columns are stored.  `ep` walks the row's entries
    // (their mask values); it is only dereferenced for stored columns' positions, clamped to `last`.
    const int last = b.last_entry;
    auto masked = [&](const float (&v)[32], unsigned word, int& ep, float (&sc)[32]) {
      if (mask_val) {
#pragma unroll
        for (int j = 0; j < 32; j++) {
          const bool on = (word >> j) & 1u;
          const float w = __ldg(mask_val + min(ep, last));
          sc[j] = on ? v[j] * scale * w : -INFINITY;
          ep += on;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; j++) sc[j] = ((word >> j) & 1u) ? v[j] * scale : -INFINITY;
      }
    };
    float mx = -INFINITY;
    int ep_max = ent0;
    // maxima of the scores of K piece c (rounds 2 c and 2 c + 1), once that piece's products are done
    auto row_max_piece = [&](int c) {
      if (!worker) return;
#pragma unroll
      for (int gg = 0; gg < 2; gg++) {
        const int g = 2 * c + gg;
        const unsigned w0 = g == 0 ? words[0] : g == 1 ? words[2] : g == 2 ? words[4] : g == 3 ? words[6]
                                              : g == 4 ? words[8] : words[10];
        const unsigned w1 = g == 0 ? words[1] : g == 1 ? words[3] : g == 2 ? words[5] : g == 3 ? words[7]
                                              : g == 4 ? words[9] : words[11];
        if (h == 1) ep_max += __popc(w0);
        const int cb = g * 64 + h * 32;
        float v[32], sc[32];
        tmem_ld32(t_row + (uint32_t)cb, v);
        if (b.raw_scores && !b.clocks) {
#pragma unroll
          for (int j = 0; j < 32; j++) b.raw_scores[(size_t)r * kBandCols + cb + j] = v[j];
        }
        masked(v, h ? w1 : w0, ep_max, sc);
#pragma unroll
        for (int j = 0; j < 32; j++) mx = fmaxf(mx, sc[j]);
        if (h == 0) ep_max += __popc(w1);
      }
    };
    BandPieceT<D> pv0, pv1;
    if (worker) {
      pv0.load(V, a.ldv, c0, b.n);
      pv1.load(V, a.ldv, c0 + 64, b.n);
    }
    if ((failed = wait_all(bar_k0, 0u))) break;          // piece 0 consumed
    mark();   // 3
    if (worker) pk0.store(k_hi(0), k_lo(0));
    async_proxy_fence();
    __syncthreads();
    mark();   // 4: K piece 2 staged
    if (issuer) issue_scores(2, 0, bar_k0);
    row_max_piece(0);
    if ((failed = wait_all(bar_k1, 0u))) break;          // piece 1 consumed: V^T buffers 2 and 3 are free
    mark();   // 5
    if (worker) {
      pv0.store(v_hi(2), v_lo(2));
      pv1.store(v_hi(3), v_lo(3));
      pv0.load(V, a.ldv, c0 + 128, b.n);
      pv1.load(V, a.ldv, c0 + 192, b.n);
    }
    row_max_piece(1);
    mark();   // 6: V^T pieces 0, 1 staged, maxima of pieces 0 and 1
    if ((failed = wait_all(bar_k0, 1u))) break;          // all scores are in tensor memory; buffers 0 and 1 free
    mark();   // 7
    if (worker) {
      pv0.store(v_hi(0), v_lo(0));
      pv1.store(v_hi(1), v_lo(1));
    }
    row_max_piece(2);
    mark();   // 8: V^T pieces 2, 3 staged, all maxima

    if (worker) s_red[h * kBandRows + r] = mx;
    __syncthreads();
    if (a.has_rem && live) {
      const float2 st = __ldg(a.stats + bz * a.m + row);
      M_s = st.x;
      L_s = st.y;
    }
    if (worker) {
      const float mt = fmaxf(fmaxf(s_red[r], s_red[kBandRows + r]), M_s);
      ms = (mt == -INFINITY) ? 0.f : mt;
    }
    mark();   // 9: row maxima

    // ---- O += P V, 64 window columns per round; V^T piece g sits in buffer (g + 2) % 4 -------------------
    int ep = ent0;
#pragma unroll 1
    for (int g = 0; g < ROUNDS; g++) {
      const int cb = g * 64 + h * 32;
      uint32_t ph[32], pl[32];
      if (worker) {
        const unsigned w0 = g == 0 ? words[0] : g == 1 ? words[2] : g == 2 ? words[4] : g == 3 ? words[6]
                                              : g == 4 ? words[8] : words[10];
        const unsigned w1 = g == 0 ? words[1] : g == 1 ? words[3] : g == 2 ? words[5] : g == 3 ? words[7]
                                              : g == 4 ? words[9] : words[11];
        if (h == 1) ep += __popc(w0);
        float v[32], sc[32];
        tmem_ld32(t_row + (uint32_t)cb, v);
        masked(v, h ? w1 : w0, ep, sc);
#pragma unroll
        for (int j = 0; j < 32; j++) {
          const float p = attn_exp2(sc[j] - ms);
          sum += p;
          attn_split(p, ph[j], pl[j]);
        }
        if (h == 0) ep += __popc(w1);
        // piece g + 3 goes to the buffer that round g - 1 releases below
        if (g >= 1 && g + 3 < ROUNDS) pv0.load(V, a.ldv, c0 + (g + 3) * 64, b.n);
      }
      mark();   // 10 + 4 g: probabilities of the round in registers
      // the round before must be done with the lo columns and with the V^T buffer that is refilled
      if (g > 0 && (failed = wait_all(bar_pv, (uint32_t)((g - 1) & 1)))) break;
      mark();   // 11 + 4 g: the round before is done
      if (worker) {
        tmem_st32(t_row + (uint32_t)cb, ph);
        tmem_st32(t_row + (uint32_t)(kTmemPlo + h * 32), pl);
        if (g >= 1 && g + 3 < ROUNDS) pv0.store(v_hi((g + 1) & 3), v_lo((g + 1) & 3));
        tmem_st_wait();
      }
      async_proxy_fence();
      tc_fence_before();
      __syncthreads();
      mark();   // 12 + 4 g: probabilities in tensor memory
      if (issuer) {
        tc_fence_after();
        const int vb = (g + 2) & 3;
        const uint64_t dv_hi = umma_desc(smem_u32(v_hi(vb)), CORE_BYTES, VT_GROUP_BYTES);
        const uint64_t dv_lo = umma_desc(smem_u32(v_lo(vb)), CORE_BYTES, VT_GROUP_BYTES);
        const uint32_t d_tmem = tmem + (uint32_t)kTmemO;
        const uint32_t p_hi = tmem + (uint32_t)(g * 64), p_lo = tmem + (uint32_t)kTmemPlo;
        const uint32_t later = g != 0 ? 1u : 0u;
#pragma unroll
        for (int pass = 0; pass < 3; pass++) {
          const uint32_t a_tmem = pass == 0 ? p_lo : p_hi;
          const uint64_t bb = pass == 1 ? dv_lo : dv_hi;
#pragma unroll
          for (int ks = 0; ks < 8; ks++)
            umma_ts(d_tmem, a_tmem + (uint32_t)(ks * 8), bb + ks * KSTEP, IDESC_O, (pass | ks) != 0 ? 1u : later);
        }
        umma_commit(bar_pv);
      }
      mark();   // 13 + 4 g
    }
    if (failed) break;
    if ((failed = wait_all(bar_pv, (uint32_t)((ROUNDS - 1) & 1)))) break;
    mark();   // 34
  } while (false);

  // ---- epilogue: merge the scattered entries' (max, sum, O), normalise, write --------------------------
  __syncthreads();
  if (worker) s_red[h * kBandRows + r] = sum;
  __syncthreads();
  if (!failed && !b.raw_scores && worker) {
    constexpr int HALF = D / 2;
    const float alpha = attn_exp2(M_s - ms);             // 0 for a row without scattered entries
    const float den = s_red[r] + s_red[kBandRows + r] + alpha * L_s;
    const float inv = den > 0.f ? 1.f / den : 0.f;
    float v[32];
    tmem_ld32(t_row + (uint32_t)(kTmemO + h * HALF), v);   // (reads 32 columns; HALF of them are used)
    if (live) {
      float* orow = O + (long long)row * a.ldo + h * HALF;
#pragma unroll
      for (int j = 0; j < HALF; j += 4) {
        float4 x = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        if (a.has_rem) {
          const float4 s = *reinterpret_cast<const float4*>(orow + j);
          x.x = fmaf(alpha, s.x, x.x); x.y = fmaf(alpha, s.y, x.y);
          x.z = fmaf(alpha, s.z, x.z); x.w = fmaf(alpha, s.w, x.w);
        }
        x.x *= inv; x.y *= inv; x.z *= inv; x.w *= inv;
        *reinterpret_cast<float4*>(orow + j) = x;
      }
    }
  }
  mark_i = 35;
  mark();     // 35: output written
  if (!failed && b.tmem_image && worker) {
#pragma unroll 1
    for (int c = 0; c < kTmemCols / 64; c++) {
      float v[32];
      tmem_ld32(t_row + (uint32_t)(c * 64 + h * 32), v);
#pragma unroll
      for (int j = 0; j < 32; j++) b.tmem_image[(size_t)r * kTmemCols + c * 64 + h * 32 + j] = v[j];
    }
  }
  if (failed && threadIdx.x == 0) atomicExch(&g_band_status, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
}

template <int D>
static size_t band_smem_bytes() {
  return (size_t)6 * kBandRows * D * 4 + 2 * kBandRows * 4 + 64;
}

template <int D>
static int band_launch(const AttnArgs& a, const BandArgs& b, unsigned tiles, unsigned batch, cudaStream_t st) {
  const size_t smem = band_smem_bytes<D>();
  // (set on every call: the attribute belongs to the current device's copy of the function, and a
  // process may drive more than one device)
  SB_CUDA(cudaFuncSetAttribute(attn_band_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  attn_band_kernel<D><<<dim3(tiles, batch), kBandThreads, smem, st>>>(a, b);
  SB_LAUNCH_CHECK("attn_band_kernel");
  return SB_OK;
}

}  // namespace sb

using namespace sb;

extern "C" {

size_t sb_attn_band_plan_bytes(int64_t m, int64_t nnz) {
  if (m < 0) m = 0;
  if (nnz < 0) nnz = 0;
  return band_plan_view(nullptr, m, nnz).bytes;
}

int sb_attn_band_plan_build(int64_t m, int64_t n, int64_t nnz, const int32_t* pos, const int32_t* crd,
                            void* plan, size_t plan_bytes, int64_t* inside_host, int64_t* rem_nnz_host,
                            void* stream) {
  SB_CHECK_ARG(m >= 0 && n >= 0 && nnz >= 0 && m < INT32_MAX - 1024 && n < INT32_MAX - 1024 && nnz < INT32_MAX,
               "attn_band_plan: bad size");
  SB_CHECK_ARG(pos && plan && (crd || nnz == 0), "attn_band_plan: null pointer");
  SB_CHECK_ARG(aligned16(plan), "attn_band_plan: plan must be 16-byte aligned");
  BandPlan p = band_plan_view(plan, m, nnz);
  if (plan_bytes < p.bytes)
    return fail(SB_ERR_WORKSPACE, "attn_band_plan: buffer has %zu bytes, needs %zu", plan_bytes, p.bytes);
  cudaStream_t st = (cudaStream_t)stream;
  SB_CUDA(cudaMemsetAsync(p.hdr, 0, 64, st));
  SB_CUDA(cudaMemsetAsync(p.total, 0, 16, st));
  long long nrem = 0;
  unsigned long long inside = 0;
  if (m > 0) {
    unsigned long long* inside_dev = reinterpret_cast<unsigned long long*>(p.total) + 1;
    const unsigned grid = (unsigned)ceil_div(m, 8);
    band_rows_kernel<<<grid, 256, 0, st>>>((int)m, (int)n, pos, crd, p.ent0, p.bits, p.cnt, inside_dev);
    SB_LAUNCH_CHECK("band_rows_kernel");
    SB_CUDA(cudaMemcpyAsync(&inside, inside_dev, 8, cudaMemcpyDeviceToHost, st));
    SB_CUDA(cudaStreamSynchronize(st));
    const int rc = exclusive_scan_i32((int)m, p.cnt, p.rem_pos, p.block_sum, p.total, st);
    if (rc != SB_OK) return rc;
    SB_CUDA(cudaMemcpyAsync(&nrem, p.total, 8, cudaMemcpyDeviceToHost, st));
    band_rem_kernel<<<grid, 256, 0, st>>>((int)m, (int)n, pos, crd, p.ent0, p.rem_pos, p.rem_ent, p.rem_crd);
    SB_LAUNCH_CHECK("band_rem_kernel");
    SB_CUDA(cudaStreamSynchronize(st));
    int h[2] = {(int)inside, (int)nrem};
    SB_CUDA(cudaMemcpyAsync(p.hdr, h, 8, cudaMemcpyHostToDevice, st));
    SB_CUDA(cudaStreamSynchronize(st));
  } else {
    SB_CUDA(cudaMemsetAsync(p.rem_pos, 0, 4, st));
    SB_CUDA(cudaStreamSynchronize(st));
  }
  if (inside_host) *inside_host = (int64_t)inside;
  if (rem_nnz_host) *rem_nnz_host = nrem;
  return SB_OK;
}

static int band_check(int64_t m, int64_t n, int64_t d, int64_t nnz, const float* Q, int64_t ldq, const float* K,
                      int64_t ldk, const float* V, int64_t ldv, const float* O, int64_t ldo, int64_t batch,
                      int64_t stride_q, int64_t stride_k, int64_t stride_v, int64_t stride_o) {
  SB_CHECK_ARG(m >= 0 && n >= 0 && nnz >= 0 && m < INT32_MAX - 1024 && n < INT32_MAX - 1024 && nnz < INT32_MAX,
               "sparse_attention_band: bad size");
  SB_CHECK_ARG(batch >= 1 && batch <= 65535, "sparse_attention_band: batch must be in [1, 65535]");
  SB_CHECK_ARG(d == 64, "sparse_attention_band: head dimension must be 64");
  if (m == 0) return SB_OK;   // (nothing to do: the callers return before any pointer is used)
  SB_CHECK_ARG(Q && K && V && O, "sparse_attention_band: null pointer");
  SB_CHECK_ARG(ldq >= d && ldk >= d && ldv >= d && ldo >= d, "sparse_attention_band: row pitch smaller than d");
  auto aligned32 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; };
  SB_CHECK_ARG(ldq % 8 == 0 && ldk % 8 == 0 && ldv % 8 == 0 && stride_q % 8 == 0 && stride_k % 8 == 0 &&
               stride_v % 8 == 0 && aligned32(Q) && aligned32(K) && aligned32(V) && ldq < (1ll << 32) &&
               ldk < (1ll << 32) && ldv < (1ll << 32),
               "sparse_attention_band: Q/K/V must be 32-byte aligned with row pitches and batch strides that "
               "are multiples of 8");
  SB_CHECK_ARG(ldo % 4 == 0 && stride_o % 4 == 0 && aligned16(O),
               "sparse_attention_band: O must be 16-byte aligned with a row pitch that is a multiple of 4");
  return SB_OK;
}

int sb_sparse_attention_band_f32(int64_t m, int64_t n, int64_t d, int64_t nnz, const int32_t* pos,
                                 const int32_t* crd, const float* mask_val, const float* Q, int64_t ldq,
                                 const float* K, int64_t ldk, const float* V, int64_t ldv, float scale,
                                 float* O, int64_t ldo, int64_t batch, int64_t stride_q, int64_t stride_k,
                                 int64_t stride_v, int64_t stride_o, const void* band_plan, int64_t rem_nnz,
                                 void* scratch, size_t scratch_bytes, int stages, void* stream) {
  (void)pos;
  (void)crd;
  SB_CHECK_ARG(stages > 0 && stages <= SB_ATTN_ALL_STAGES, "sparse_attention_band: bad stage set");
  int rc = band_check(m, n, d, nnz, Q, ldq, K, ldk, V, ldv, O, ldo, batch, stride_q, stride_k, stride_v, stride_o);
  if (rc != SB_OK) return rc;
  if (m == 0) return SB_OK;
  SB_CHECK_ARG(band_plan, "sparse_attention_band: null plan");
  SB_CHECK_ARG(rem_nnz >= 0 && rem_nnz <= nnz, "sparse_attention_band: remainder count does not fit nnz");
  const size_t need = sb_sparse_attention_scratch_bytes(m, rem_nnz, batch);
  SB_CHECK_ARG(scratch && aligned16(scratch), "sparse_attention_band: scratch is null or misaligned");
  if (scratch_bytes < need)
    return fail(SB_ERR_WORKSPACE, "sparse_attention_band: scratch has %zu bytes, needs %zu", scratch_bytes, need);
  cudaStream_t st = (cudaStream_t)stream;
  BandPlan p = band_plan_view(const_cast<void*>(band_plan), m, nnz);
  int* flags = static_cast<int*>(scratch);
  AttnArgs a = {};
  a.m = (int)m;
  a.rem_pos = p.rem_pos; a.rem_ent = p.rem_ent; a.rem_crd = p.rem_crd;
  a.mask_val = mask_val; a.mask_is_ones = flags;
  a.Q = Q; a.K = K; a.V = V; a.O = O;
  a.stats = reinterpret_cast<float2*>(static_cast<char*>(scratch) + 256);
  a.has_rem = rem_nnz > 0 ? 1 : 0;
  a.ldq = (unsigned)ldq; a.ldk = (unsigned)ldk; a.ldv = (unsigned)ldv; a.ldo = ldo;
  a.stride_q = stride_q; a.stride_k = stride_k; a.stride_v = stride_v; a.stride_o = stride_o;
  a.scale = scale;
  if (stages & SB_ATTN_STAGE_SCATTERED) {
    rc = attn_launch_scattered(a, d, nnz, rem_nnz, batch, flags, st);
    if (rc != SB_OK) return rc;
  }
  if (stages & SB_ATTN_STAGE_BLOCKS) {
    BandArgs b = {(int)n, p.ent0, p.bits, nullptr, nullptr, 0, nullptr, (int)std::max<int64_t>(nnz - 1, 0)};
    rc = band_launch<64>(a, b, (unsigned)ceil_div(m, kBandRows), (unsigned)batch, st);
    if (rc != SB_OK) return rc;
  }
  return SB_OK;
}

int sb_attn_band_probe(int64_t m, int64_t n, int64_t d, int64_t tile, const float* Q, int64_t ldq,
                       const float* K, int64_t ldk, const float* V, int64_t ldv, float* raw_scores,
                       float* tmem_image, long long* phase_clocks, void* stream) {
  int rc = band_check(m, n, d, 0, Q, ldq, K, ldk, V, ldv, raw_scores, d, 1, 0, 0, 0, 0);
  if (rc != SB_OK) return rc;
  SB_CHECK_ARG(tile >= 0 && tile < ceil_div(m, kBandRows), "attn_band_probe: tile out of range");
  AttnArgs a = {};
  a.m = (int)m;
  a.Q = Q; a.K = K; a.V = V; a.O = raw_scores;
  a.ldq = (unsigned)ldq; a.ldk = (unsigned)ldk; a.ldv = (unsigned)ldv; a.ldo = d;
  a.scale = 1.f;
  // (no plan: every window column counts as stored; O is not written)
  BandArgs b = {(int)n, nullptr, nullptr, raw_scores, tmem_image, (int)tile, phase_clocks, 0};
  return band_launch<64>(a, b, 1u, 1u, (cudaStream_t)stream);
}

int sb_attn_band_status(void) {
  int v = -1;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_band_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

}  // extern "C"
