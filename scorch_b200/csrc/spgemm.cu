// CSR x CSR SpGEMM (Gustavson) for sm_100a, two phases (symbolic / numeric) like the reference.
//
// Rows of A are binned by their product upper bound U_i = sum over the row's entries of the
// length of the matching B row:
//   bin 0  U <= 32      one warp per row, 64-slot hash set/accumulator in shared memory
//   bin 1  U <= 128     one warp per row, 256 slots
//   bin 2  U <= 512     one 128-thread CTA per row, 1024 slots
//   bin 3  U <= 2048    one 256-thread CTA per row, 4096 slots
//   bin 4  U <= 8192    one 512-thread CTA per row, 16384 slots
//   bin 5  U  > 8192    dense bitmap (+ dense accumulator) of n columns in the workspace; the
//                       rows' entries are spread over the GPU as (row, chunk) tasks
// Hash bins: open addressing with atomicCAS on the column key (+ atomicAdd on the value), load
// factor <= 0.5 by construction.  The numeric phase compacts each row's table in place and sorts
// the occupied part in shared memory (bitonic) so columns come out ascending like the
// reference's per-row sort; the dense bin emits columns in bitmap order, which is already
// ascending.  The structure is the symbolic union: a slot whose value cancels to 0 is kept.
// Row pointers come from a three-kernel exclusive scan in int64, stored as int32 with an
// overflow check.
//
// Values are reproducible bit for bit from run to run.  Several products may land on one output
// entry and the hardware serves their atomic additions in any order, so floating-point sums are
// not added as floats: every product is computed exactly in double, scaled by a power of two
// chosen per output row so that no partial sum can overflow (2^61 / (sum |a| of the row * max |b|)),
// rounded to a 64-bit integer and added with integer atomics, whose result does not depend on
// the order.  The total is converted back once per entry.  The rounding step is 2^-61 of the
// row's bound, far below fp32 (and fp64) resolution of the sum itself.  Rows whose bound is not
// finite (Inf / NaN operands) are added as floats like before, so those values propagate.
// Integer dtypes wrap like the reference's and need none of this.
#include <limits.h>
#include <string.h>

#include <algorithm>

#include "common.cuh"

namespace sb {

constexpr int kBins = 6;
constexpr int kEmpty = INT_MAX;
constexpr int kDenseWorkersMax = 296;  // 2 CTAs per SM on a 148-SM part
constexpr size_t kDenseBudget = (size_t)4 << 30;

// Workspace header (int64 words): [0..5] rows per bin, [8] total nnz of C.
struct WsLayout {
  long long* hdr;       // 16 int64
  int* bin_cursor;      // kBins ints (+ padding)
  int* upper;           // m ints: product upper bound per row (saturating)
  int* bin_rows;        // kBins * m ints
  int* row_cnt;         // m ints
  double* row_scale;    // m doubles: fixed-point scale of each output row (numeric phase)
  unsigned long long* max_b;  // bit pattern of max |b| over the right operand
  long long* block_sum; // scan temporaries
  int* dense_ctl;       // task prefix, per-row done counters and queue of the dense bin
  unsigned* bitmap;     // workers * words
  void* dense_acc;      // workers * n * sizeof(T)
  int workers;
  long long words;      // bitmap words per worker
  size_t total;
};

static size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }
// every accumulator slot is 8 bytes: 64-bit fixed point for the float types, the type itself
// (in the low bytes) for the integer ones
static size_t dtype_size(int) { return 8; }

static WsLayout ws_layout(void* base, int64_t m, int64_t n, int dtype) {
  WsLayout w;
  char* p = static_cast<char*>(base);
  size_t off = 0;
  w.hdr = reinterpret_cast<long long*>(p + off); off += align_up(16 * 8);
  w.bin_cursor = reinterpret_cast<int*>(p + off); off += align_up(16 * 4);
  w.upper = reinterpret_cast<int*>(p + off); off += align_up((size_t)m * 4);
  w.bin_rows = reinterpret_cast<int*>(p + off); off += align_up((size_t)m * 4 * kBins);
  w.row_cnt = reinterpret_cast<int*>(p + off); off += align_up((size_t)m * 4);
  w.row_scale = reinterpret_cast<double*>(p + off); off += align_up((size_t)m * 8);
  w.max_b = reinterpret_cast<unsigned long long*>(p + off); off += align_up(8);
  w.block_sum = reinterpret_cast<long long*>(p + off);
  off += align_up((size_t)(ceil_div(m > 0 ? m : 1, 4096) + 1) * 8);
  w.dense_ctl = reinterpret_cast<int*>(p + off); off += align_up((size_t)(2 * kDenseWorkersMax + 8) * 4);
  w.words = (n + 31) / 32;
  const size_t per_worker = (size_t)w.words * 4 + (size_t)n * dtype_size(dtype);
  long long workers = per_worker ? (long long)(kDenseBudget / per_worker) : kDenseWorkersMax;
  if (workers < 1) workers = 1;
  if (workers > kDenseWorkersMax) workers = kDenseWorkersMax;
  w.workers = (int)workers;
  w.bitmap = reinterpret_cast<unsigned*>(p + off); off += align_up((size_t)w.workers * w.words * 4);
  w.dense_acc = p + off; off += align_up((size_t)w.workers * (size_t)n * dtype_size(dtype));
  w.total = off;
  return w;
}

// ---- binning ---------------------------------------------------------------------------------
__device__ __forceinline__ int bin_of(int u) {
  if (u <= 32) return 0;
  if (u <= 128) return 1;
  if (u <= 512) return 2;
  if (u <= 2048) return 3;
  if (u <= 8192) return 4;
  return 5;
}

// 8 lanes per row of A: U_i and the row's bin; rows are appended to their bin's list with one
// atomic per (warp, bin).  Rows with U = 0 get row_cnt = 0 and join no bin.
__global__ void __launch_bounds__(256)
spgemm_bin_kernel(int m, const int* __restrict__ Apos, const int* __restrict__ Acrd,
                  const int* __restrict__ Bpos, int* __restrict__ upper, int* __restrict__ bin_rows,
                  int* __restrict__ bin_cursor, int* __restrict__ row_cnt) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = t >> 3;
  const int l = (int)(t & 7), lane = threadIdx.x & 31;
  long long u = 0;
  if (row < m) {
    const int b = __ldg(Apos + row), e = __ldg(Apos + row + 1);
    for (int p = b + l; p < e; p += 8) {
      const int j = ld_stream(Acrd + p);
      u += __ldg(Bpos + j + 1) - __ldg(Bpos + j);
    }
  }
  u += __shfl_xor_sync(FULL, u, 4);
  u += __shfl_xor_sync(FULL, u, 2);
  u += __shfl_xor_sync(FULL, u, 1);
  const int ui = u > INT_MAX ? INT_MAX : (int)u;
  const bool owner = (l == 0) && (row < m);
  int bin = -1;
  if (owner) {
    upper[row] = ui;
    if (ui == 0) row_cnt[row] = 0; else bin = bin_of(ui);
  }
#pragma unroll
  for (int b = 0; b < kBins; b++) {
    const unsigned mask = __ballot_sync(FULL, bin == b);
    if (mask == 0) continue;
    const int leader = __ffs(mask) - 1;
    int base = 0;
    if (lane == leader) base = atomicAdd(&bin_cursor[b], __popc(mask));
    base = __shfl_sync(FULL, base, leader);
    if (bin == b) bin_rows[(long long)b * m + base + __popc(mask & ((1u << lane) - 1))] = (int)row;
  }
}

// ---- hash + sort primitives ------------------------------------------------------------------
template <int S>
__device__ __forceinline__ int hash_slot(int c) {
  return (int)(((unsigned)c * 0x9E3779B1u) >> (32 - __builtin_ctz(S)));
}

// Slot of column c in the table, inserting it when absent (`fresh` = it was).
template <int S>
__device__ __forceinline__ int hash_find_or_insert(int* keys, int c, int& fresh) {
  int h = hash_slot<S>(c);
  while (true) {
    const int old = atomicCAS(&keys[h], kEmpty, c);
    if (old == kEmpty || old == c) {
      fresh += (old == kEmpty);
      return h;
    }
    h = (h + 1) & (S - 1);
  }
}

// ---- order-independent accumulation ------------------------------------------------------------
// An accumulator slot is 8 bytes.  Float types: a 64-bit fixed-point sum of the exactly computed,
// scaled products (integer atomics: the same bits whatever the order); with `fixed` false (the
// row's bound is not finite) the slot's low bytes hold a plain T added with float atomics.
// Integer types: the slot's low bytes hold T, added with wrapping integer atomics.
typedef unsigned long long Slot;

template <typename T> struct IsFloat { static constexpr bool value = false; };
template <> struct IsFloat<float> { static constexpr bool value = true; };
template <> struct IsFloat<double> { static constexpr bool value = true; };

template <typename T>
__device__ __forceinline__ void acc_add(Slot* slot, T a, T b, double scale, bool fixed) {
  if constexpr (IsFloat<T>::value) {
    if (fixed) {
      const long long q = __double2ll_rn((double)a * (double)b * scale);
      atomicAdd(slot, (Slot)q);
    } else {
      atomicAdd(reinterpret_cast<T*>(slot), a * b);
    }
  } else {
    atomicAdd(reinterpret_cast<T*>(slot), a * b);
  }
}

template <typename T>
__device__ __forceinline__ T acc_value(Slot v, double inv_scale, bool fixed) {
  if constexpr (IsFloat<T>::value) {
    if (fixed) return (T)((double)(long long)v * inv_scale);
  }
  T out;
  memcpy(&out, &v, sizeof(T));
  return out;
}

// scale = 2^(61 - exponent of bound); NaN marks "not fixed point"
__device__ __forceinline__ double scale_for_bound(double bound) {
  if (!(bound < 1.0e300)) return __longlong_as_double(0x7ff8000000000000LL);  // Inf / NaN
  if (bound <= 0.0) return 1.0;
  int e;
  frexp(bound, &e);                 // bound = f * 2^e, f in [0.5, 1)
  return ldexp(1.0, 61 - e);        // bound * scale < 2^61
}

// Bitonic sort of the first P slots (P a power of two <= S) by key, values carried along.
template <typename T, int NT, bool WARP_SCOPE>
__device__ __forceinline__ void bitonic_sort(int* keys, T* vals, int P, int tid) {
  for (int k = 2; k <= P; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int t = tid; t < P / 2; t += NT) {
        const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
        const int x = i | j;
        const bool up = (i & k) == 0;
        const int a = keys[i], b = keys[x];
        if ((a > b) == up) {
          keys[i] = b; keys[x] = a;
          const T va = vals[i]; vals[i] = vals[x]; vals[x] = va;
        }
      }
      if (WARP_SCOPE) __syncwarp(); else __syncthreads();
    }
  }
}

// Moves the occupied slots of a hash table to the front, in place, NT slots per round: a round
// reads its slots into registers, scans the occupancy, and writes them at the running offset,
// which never runs ahead of the slots already read.  Then pads up to the next power of two with
// empty keys and returns that size (what the sort has to cover).  One warp (WARP_SCOPE) or one
// CTA of NT threads; `s_scan` is NT/32 + 1 ints of shared memory (unused for a warp).
template <typename T, int S, int NT, bool WARP_SCOPE>
__device__ __forceinline__ int compact_table(int* keys, T* vals, int tid, int* s_scan) {
  const int lane = tid & 31, warp = tid >> 5;
  int run = 0;
  for (int r0 = 0; r0 < S; r0 += NT) {
    const int key = keys[r0 + tid];
    const T val = vals[r0 + tid];
    const bool occ = key != kEmpty;
    const unsigned ball = __ballot_sync(FULL, occ);
    int off = __popc(ball & ((1u << lane) - 1));
    int total = __popc(ball);
    if (!WARP_SCOPE) {
      if (lane == 0) s_scan[warp] = total;
      __syncthreads();  // also: every slot of this round has been read
      int before = 0;
      total = 0;
#pragma unroll
      for (int w = 0; w < NT / 32; w++) {
        const int c = s_scan[w];
        if (w < warp) before += c;
        total += c;
      }
      off += before;
      __syncthreads();  // s_scan is rewritten next round
    } else {
      __syncwarp();
    }
    if (occ) {
      keys[run + off] = key;
      vals[run + off] = val;
    }
    run += total;
    if (WARP_SCOPE) __syncwarp(); else __syncthreads();
  }
  int P = 1;
  while (P < run) P <<= 1;
  for (int t = run + tid; t < P; t += NT) keys[t] = kEmpty;
  if (WARP_SCOPE) __syncwarp(); else __syncthreads();
  return P;
}

struct CsrIn {
  const int* Apos; const int* Acrd; const void* Aval;
  const int* Bpos; const int* Bcrd; const void* Bval;
  const double* row_scale;   // numeric phase, float types: fixed-point scale per output row
};

// The products of A entries [pa0, pa1) (at most 32, one per lane) spread evenly over the lanes
// of a warp: lane l looks up the B row of entry pa0 + l, a warp scan of the row lengths numbers
// the products, and every lane then takes products lane, lane + 32, ... — a 5-step search over
// the scanned lengths tells which entry a product belongs to.  No lane idles on a short B row and
// the index loads of 32 entries are in flight together, instead of one dependent chain
// (A entry -> B row pointers -> B entries) per entry.  `emit(a_value, pb)` is called once per
// product with the value of its A entry (T(0) in the symbolic phase) and its position in B.
// `defer(pa, len)` may take an entry out of the warp's share (it returns true and deals with the
// entry's products itself): the dense rows hand B rows of hub length to the whole CTA that way.
template <typename T, bool NUMERIC, typename F, typename D>
__device__ __forceinline__ void expand_products(const CsrIn& in, int pa0, int pa1, int lane, F&& emit,
                                                D&& defer) {
  const int pa = pa0 + lane;
  int bb = 0, len = 0;
  T a = T(0);
  if (pa < pa1) {
    const int j = __ldg(in.Acrd + pa);
    bb = __ldg(in.Bpos + j);
    len = __ldg(in.Bpos + j + 1) - bb;
    if (defer(pa, len)) len = 0;
    if (NUMERIC) a = static_cast<const T*>(in.Aval)[pa];
  }
  int incl = len;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_up_sync(FULL, incl, o);
    if (lane >= o) incl += y;
  }
  const int total = __shfl_sync(FULL, incl, 31);
  const int excl = incl - len;
  for (int q0 = 0; q0 < total; q0 += 32) {
    const int q = q0 + lane;
    // largest e with excl[e] <= q (lanes past the end search too: shuffles need the whole warp)
    int e = 0;
#pragma unroll
    for (int step = 16; step > 0; step >>= 1) {
      const int v = __shfl_sync(FULL, excl, e + step);
      if (v <= q) e += step;
    }
    const int e_excl = __shfl_sync(FULL, excl, e);
    const int e_bb = __shfl_sync(FULL, bb, e);
    T e_a;
    if constexpr (sizeof(T) == 8) {
      const long long bits = __shfl_sync(FULL, *reinterpret_cast<const long long*>(&a), e);
      memcpy(&e_a, &bits, 8);
    } else {
      const int bits = __shfl_sync(FULL, *reinterpret_cast<const int*>(&a), e);
      memcpy(&e_a, &bits, 4);
    }
    if (q < total) emit(e_a, e_bb + (q - e_excl));
  }
}

// One warp per row (bins 0, 1): 32 A entries at a time, their products spread over the lanes.
template <typename T, int S, bool NUMERIC>
__global__ void __launch_bounds__(128)
spgemm_warp_kernel(const int* __restrict__ rows, int nrows, CsrIn in, int* __restrict__ row_cnt,
                   const int* __restrict__ Cpos, int* __restrict__ Ccrd, T* __restrict__ Cval) {
  __shared__ int s_keys[4][S];
  __shared__ Slot s_vals[4][NUMERIC ? S : 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * 4 + warp;
  if (r >= nrows) return;
  const int i = __ldg(rows + r);
  int* keys = s_keys[warp];
  Slot* vals = s_vals[warp];
  for (int t = lane; t < S; t += 32) {
    keys[t] = kEmpty;
    if (NUMERIC) vals[t] = 0;
  }
  __syncwarp();
  double scale = 1.0;
  if (NUMERIC && IsFloat<T>::value) scale = in.row_scale[i];
  const bool fixed = scale == scale;
  const T* Bval = static_cast<const T*>(in.Bval);
  const int ab = __ldg(in.Apos + i), ae = __ldg(in.Apos + i + 1);
  int fresh = 0;
  for (int pa0 = ab; pa0 < ae; pa0 += 32) {
    expand_products<T, NUMERIC>(in, pa0, min(ae, pa0 + 32), lane, [&](T a, int pb) {
      const int c = __ldg(in.Bcrd + pb);
      const int h = hash_find_or_insert<S>(keys, c, fresh);
      if (NUMERIC) acc_add<T>(vals + h, a, Bval[pb], scale, fixed);
    }, [](int, int) { return false; });
  }
  __syncwarp();
  if (!NUMERIC) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) fresh += __shfl_xor_sync(FULL, fresh, o);
    if (lane == 0) row_cnt[i] = fresh;
  } else {
    const int P = compact_table<Slot, S, 32, true>(keys, vals, lane, nullptr);
    bitonic_sort<Slot, 32, true>(keys, vals, P, lane);
    const int base = __ldg(Cpos + i), cnt = __ldg(Cpos + i + 1) - base;
    const double inv = 1.0 / scale;
    for (int t = lane; t < cnt; t += 32) {
      Ccrd[base + t] = keys[t];
      Cval[base + t] = acc_value<T>(vals[t], inv, fixed);
    }
  }
}

// One CTA per row (bins 2-4): warps take alternate slabs of 32 entries of the A row.
template <typename T, int S, int NT, bool NUMERIC>
__global__ void __launch_bounds__(NT)
spgemm_cta_kernel(const int* __restrict__ rows, int nrows, CsrIn in, int* __restrict__ row_cnt,
                  const int* __restrict__ Cpos, int* __restrict__ Ccrd, T* __restrict__ Cval) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Slot* vals = reinterpret_cast<Slot*>(smem_raw);                 // S accumulators (numeric only)
  int* keys = reinterpret_cast<int*>(smem_raw + (NUMERIC ? sizeof(Slot) * S : 0));
  __shared__ int s_fresh;
  __shared__ int s_scan[NT / 32 + 1];
  const int r = blockIdx.x;
  if (r >= nrows) return;
  const int i = __ldg(rows + r);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int t = tid; t < S; t += NT) {
    keys[t] = kEmpty;
    if (NUMERIC) vals[t] = 0;
  }
  if (tid == 0) s_fresh = 0;
  __syncthreads();
  double scale = 1.0;
  if (NUMERIC && IsFloat<T>::value) scale = in.row_scale[i];
  const bool fixed = scale == scale;
  const T* Bval = static_cast<const T*>(in.Bval);
  const int ab = __ldg(in.Apos + i), ae = __ldg(in.Apos + i + 1);
  int fresh = 0;
  // warps take slabs of 32 A entries; a slab's products are spread over the warp's lanes
  for (int pa0 = ab + 32 * warp; pa0 < ae; pa0 += NT) {
    expand_products<T, NUMERIC>(in, pa0, min(ae, pa0 + 32), lane, [&](T a, int pb) {
      const int c = __ldg(in.Bcrd + pb);
      const int h = hash_find_or_insert<S>(keys, c, fresh);
      if (NUMERIC) acc_add<T>(vals + h, a, Bval[pb], scale, fixed);
    }, [](int, int) { return false; });
  }
  if (!NUMERIC) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) fresh += __shfl_xor_sync(FULL, fresh, o);
    if (lane == 0 && fresh) atomicAdd(&s_fresh, fresh);
    __syncthreads();
    if (tid == 0) row_cnt[i] = s_fresh;
  } else {
    __syncthreads();
    const int P = compact_table<Slot, S, NT, false>(keys, vals, tid, s_scan);
    bitonic_sort<Slot, NT, false>(keys, vals, P, tid);
    const int base = __ldg(Cpos + i), cnt = __ldg(Cpos + i + 1) - base;
    const double inv = 1.0 / scale;
    for (int t = tid; t < cnt; t += NT) {
      Ccrd[base + t] = keys[t];
      Cval[base + t] = acc_value<T>(vals[t], inv, fixed);
    }
  }
}

// Bin 5 (rows whose products do not fit a shared-memory table): dense bitmap (+ accumulator) of
// n columns per row in the workspace.  Rows are handled in batches of up to `slots` rows, one
// slot each; a row's A entries are cut into chunks of kDenseChunk entries and the (row, chunk)
// tasks of a batch are handed out through an atomic queue, so a hub row with hundreds of
// thousands of entries is spread over the whole GPU.  The CTA that finishes a row's last chunk
// (a counter per row, no spinning) walks the row's bitmap in ascending column order, emits the
// row and leaves bitmap and accumulator all-zero for the next batch.
constexpr int kDenseChunk = 2048;     // A entries per task
constexpr int kLongBRow = 2048;       // B rows at least this long are walked by the whole CTA
constexpr int kDeferCap = 64;

struct DenseCtl {
  int* task_pref;  // [slots + 1]
  int* done;       // [slots]
  int* queue;      // [1]
};

__global__ void dense_batch_setup_kernel(const int* __restrict__ rows, int r0, int nb,
                                         const int* __restrict__ Apos, DenseCtl ctl) {
  if (threadIdx.x == 0) {
    int run = 0;
    for (int k = 0; k < nb; k++) {
      ctl.task_pref[k] = run;
      const int i = rows[r0 + k];
      const int len = Apos[i + 1] - Apos[i];
      run += max(1, (len + kDenseChunk - 1) / kDenseChunk);
      ctl.done[k] = 0;
    }
    ctl.task_pref[nb] = run;
    *ctl.queue = 0;
  }
}

template <typename T, bool NUMERIC>
__global__ void __launch_bounds__(256)
spgemm_dense_kernel(const int* __restrict__ rows, int r0, int nb, CsrIn in, long long words,
                    unsigned* __restrict__ bitmap_all, Slot* __restrict__ acc_all, long long n,
                    DenseCtl ctl, int* __restrict__ row_cnt, const int* __restrict__ Cpos,
                    int* __restrict__ Ccrd, T* __restrict__ Cval) {
  __shared__ int s_warp[8];
  __shared__ int s_base;
  __shared__ int s_task;
  __shared__ int s_last;
  __shared__ int s_ndefer;
  __shared__ int s_defer[kDeferCap];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int total = __ldg(ctl.task_pref + nb);
  while (true) {
    if (tid == 0) {
      s_task = atomicAdd(ctl.queue, 1);
      s_ndefer = 0;
    }
    __syncthreads();
    const int task = s_task;
    if (task >= total) return;
    // slot k with task_pref[k] <= task < task_pref[k+1]
    int lo = 0, hi = nb;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (__ldg(ctl.task_pref + mid) <= task) lo = mid; else hi = mid;
    }
    const int k = lo;
    const int chunk = task - __ldg(ctl.task_pref + k);
    const int nchunks = __ldg(ctl.task_pref + k + 1) - __ldg(ctl.task_pref + k);
    const int i = __ldg(rows + r0 + k);
    unsigned* bitmap = bitmap_all + (long long)k * words;
    Slot* acc = NUMERIC ? acc_all + (long long)k * n : nullptr;
    double scale = 1.0;
    if (NUMERIC && IsFloat<T>::value) scale = in.row_scale[i];
    const bool fixed = scale == scale;
    const int ab = __ldg(in.Apos + i) + chunk * kDenseChunk;
    const int ae = min(__ldg(in.Apos + i + 1), ab + kDenseChunk);
    // warps take slabs of 32 A entries; a slab's products are spread over the warp's lanes.  B
    // rows of hub length are put aside and walked by the whole CTA afterwards.
    auto add = [&](T av, int pb) {
      const int c = __ldg(in.Bcrd + pb);
      if (NUMERIC) acc_add<T>(acc + c, av, static_cast<const T*>(in.Bval)[pb], scale, fixed);
      atomicOr(&bitmap[c >> 5], 1u << (c & 31));
    };
    for (int pa0 = ab + 32 * warp; pa0 < ae; pa0 += 256) {
      expand_products<T, NUMERIC>(in, pa0, min(ae, pa0 + 32), lane, add, [&](int pa, int len) {
        if (len < kLongBRow) return false;
        const int slot = atomicAdd(&s_ndefer, 1);
        if (slot >= kDeferCap) return false;
        s_defer[slot] = pa;
        return true;
      });
    }
    __syncthreads();
    const int nd = min(s_ndefer, kDeferCap);
    for (int q = 0; q < nd; q++) {
      const int pa = s_defer[q];
      const int j = __ldg(in.Acrd + pa);
      const T av = NUMERIC ? static_cast<const T*>(in.Aval)[pa] : T(0);
      const int bb = __ldg(in.Bpos + j), be = __ldg(in.Bpos + j + 1);
      for (int pb = bb + tid; pb < be; pb += 256) add(av, pb);
    }
    // publish this chunk, then find out whether it was the row's last one
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(ctl.done + k, 1) == nchunks - 1);
    __syncthreads();
    if (!s_last) continue;
    __threadfence();
    // walk the bitmap in ascending order, 256 words per step
    if (tid == 0) s_base = 0;
    __syncthreads();
    const int out0 = NUMERIC ? __ldg(Cpos + i) : 0;
    for (long long w0 = 0; w0 < words; w0 += 256) {
      const long long w = w0 + tid;
      unsigned bits = 0;
      if (w < words) {
        bits = __ldcg(bitmap + w);  // the bits were set by L2 atomics: do not trust L1
        if (bits) bitmap[w] = 0;
      }
      const int cnt = __popc(bits);
      // block-wide exclusive scan of cnt
      int incl = cnt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(FULL, incl, o);
        if (lane >= o) incl += y;
      }
      if (lane == 31) s_warp[warp] = incl;
      __syncthreads();
      int warp_off = 0, step_total = 0;
#pragma unroll
      for (int q = 0; q < 8; q++) {
        const int v = s_warp[q];
        if (q < warp) warp_off += v;
        step_total += v;
      }
      const int base = s_base;
      if (NUMERIC && bits) {
        int o = out0 + base + warp_off + incl - cnt;
        while (bits) {
          const int bit = __ffs(bits) - 1;
          bits &= bits - 1;
          const long long c = w * 32 + bit;
          Ccrd[o] = (int)c;
          Cval[o] = acc_value<T>(__ldcg(acc + c), 1.0 / scale, fixed);
          acc[c] = 0;
          o++;
        }
      }
      __syncthreads();
      if (tid == 0) s_base = base + step_total;
      __syncthreads();
    }
    if (!NUMERIC && tid == 0) row_cnt[i] = s_base;
    __syncthreads();
  }
}

// ---- exclusive scan of row counts (int64 accumulate, int32 store) ------------------------------
constexpr int kScanTile = 4096;

__global__ void __launch_bounds__(1024)
scan_reduce_kernel(int m, const int* __restrict__ cnt, long long* __restrict__ block_sum) {
  __shared__ long long s[32];
  const long long base = (long long)blockIdx.x * kScanTile;
  long long v = 0;
  for (int q = 0; q < 4; q++) {
    const long long i = base + q * 1024 + threadIdx.x;
    if (i < m) v += cnt[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    v = s[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
    if (threadIdx.x == 0) block_sum[blockIdx.x] = v;
  }
}

__global__ void scan_blocks_kernel(int nb, long long* block_sum, long long* hdr_total) {
  // single thread block, sequential over at most a few thousand tiles
  if (threadIdx.x == 0) {
    long long run = 0;
    for (int b = 0; b < nb; b++) {
      const long long v = block_sum[b];
      block_sum[b] = run;
      run += v;
    }
    *hdr_total = run;
  }
}

__global__ void __launch_bounds__(1024)
scan_write_kernel(int m, const int* __restrict__ cnt, const long long* __restrict__ block_sum,
                  int* __restrict__ Cpos) {
  __shared__ long long s[32];
  const long long base = (long long)blockIdx.x * kScanTile;
  // each thread owns 4 consecutive rows
  const long long i0 = base + (long long)threadIdx.x * 4;
  int c[4];
  long long mine = 0;
#pragma unroll
  for (int q = 0; q < 4; q++) {
    c[q] = (i0 + q < m) ? cnt[i0 + q] : 0;
    mine += c[q];
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  long long incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const long long y = __shfl_up_sync(FULL, incl, o);
    if (lane >= o) incl += y;
  }
  if (lane == 31) s[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    long long v = s[lane];
    long long iv = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const long long y = __shfl_up_sync(FULL, iv, o);
      if (lane >= o) iv += y;
    }
    s[lane] = iv - v;  // exclusive over warps
  }
  __syncthreads();
  long long run = block_sum[blockIdx.x] + s[warp] + incl - mine;
  if (blockIdx.x == 0 && threadIdx.x == 0) Cpos[0] = 0;
#pragma unroll
  for (int q = 0; q < 4; q++) {
    run += c[q];
    if (i0 + q < m) Cpos[i0 + q + 1] = (int)run;
  }
}

// Exclusive scan of n int counts into out[0..n] (int32), running total in int64 at *total_dev.
// `block_sum` needs ceil(n / 4096) + 1 int64 slots.
int exclusive_scan_i32(int n, const int* cnt, int* out, long long* block_sum, long long* total_dev,
                       cudaStream_t st) {
  if (n <= 0) {
    SB_CUDA(cudaMemsetAsync(out, 0, 4, st));
    SB_CUDA(cudaMemsetAsync(total_dev, 0, 8, st));
    return SB_OK;
  }
  const int nb = (int)ceil_div(n, kScanTile);
  scan_reduce_kernel<<<nb, 1024, 0, st>>>(n, cnt, block_sum);
  SB_LAUNCH_CHECK("scan_reduce_kernel");
  scan_blocks_kernel<<<1, 32, 0, st>>>(nb, block_sum, total_dev);
  SB_LAUNCH_CHECK("scan_blocks_kernel");
  scan_write_kernel<<<nb, 1024, 0, st>>>(n, cnt, block_sum, out);
  SB_LAUNCH_CHECK("scan_write_kernel");
  return SB_OK;
}

// ---- fixed-point scales of the numeric phase (float types) ---------------------------------------
template <typename T>
__global__ void spgemm_max_abs_kernel(long long nnz, const T* __restrict__ val, unsigned long long* out) {
  double mx = 0.0;
  bool bad = false;
  for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < nnz;
       p += (long long)gridDim.x * blockDim.x) {
    const double v = fabs((double)val[p]);
    if (!(v < 1.0e300)) bad = true; else mx = fmax(mx, v);
  }
  if (bad) mx = __longlong_as_double(0x7ff0000000000000LL);  // +inf: sorts above every finite bit pattern
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmax(mx, __shfl_xor_sync(FULL, mx, o));
  // non-negative doubles order like their bit patterns
  if ((threadIdx.x & 31) == 0) atomicMax(out, (unsigned long long)__double_as_longlong(mx));
}

// 8 lanes per row: scale of row i from sum |a| over the row and max |b|.
template <typename T>
__global__ void __launch_bounds__(256)
spgemm_row_scale_kernel(int m, const int* __restrict__ Apos, const T* __restrict__ Aval,
                        const unsigned long long* __restrict__ max_b, double* __restrict__ row_scale) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = t >> 3;
  const int l = (int)(t & 7);
  double s = 0.0;
  if (row < m) {
    const int b = __ldg(Apos + row), e = __ldg(Apos + row + 1);
    for (int p = b + l; p < e; p += 8) s += fabs((double)Aval[p]);
  }
  s += __shfl_xor_sync(FULL, s, 4);
  s += __shfl_xor_sync(FULL, s, 2);
  s += __shfl_xor_sync(FULL, s, 1);
  if (l == 0 && row < m) row_scale[row] = scale_for_bound(s * __longlong_as_double((long long)*max_b));
}

// ---- host side ---------------------------------------------------------------------------------
template <typename T, bool NUMERIC>
static int launch_bins(const WsLayout& w, const long long* counts, int64_t m, int64_t n,
                       const CsrIn& in, const int* Cpos, int* Ccrd, T* Cval, cudaStream_t st) {
  const int* rows0 = w.bin_rows;
  if (counts[0] > 0) {
    spgemm_warp_kernel<T, 64, NUMERIC><<<(unsigned)ceil_div(counts[0], 4), 128, 0, st>>>(
        rows0, (int)counts[0], in, w.row_cnt, Cpos, Ccrd, Cval);
    SB_LAUNCH_CHECK("spgemm_warp_kernel<64>");
  }
  if (counts[1] > 0) {
    spgemm_warp_kernel<T, 256, NUMERIC><<<(unsigned)ceil_div(counts[1], 4), 128, 0, st>>>(
        rows0 + m, (int)counts[1], in, w.row_cnt, Cpos, Ccrd, Cval);
    SB_LAUNCH_CHECK("spgemm_warp_kernel<256>");
  }
#define SB_CTA_BIN(IDX, SLOTS, THREADS)                                                        \
  if (counts[IDX] > 0) {                                                                      \
    constexpr int S = SLOTS;                                                                  \
    const size_t smem = (size_t)S * 4 + (NUMERIC ? (size_t)S * sizeof(Slot) : 0);             \
    auto k = spgemm_cta_kernel<T, S, THREADS, NUMERIC>;                                       \
    SB_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    k<<<(unsigned)counts[IDX], THREADS, smem, st>>>(rows0 + (long long)IDX * m, (int)counts[IDX], \
                                                    in, w.row_cnt, Cpos, Ccrd, Cval);         \
    SB_LAUNCH_CHECK("spgemm_cta_kernel");                                                     \
  }
  SB_CTA_BIN(2, 1024, 128)
  SB_CTA_BIN(3, 4096, 256)
  SB_CTA_BIN(4, 16384, 512)
#undef SB_CTA_BIN
  if (counts[5] > 0) {
    DenseCtl ctl{w.dense_ctl, w.dense_ctl + kDenseWorkersMax + 1, w.dense_ctl + 2 * kDenseWorkersMax + 2};
    const int grid = 4 * sm_count();
    for (long long r0 = 0; r0 < counts[5]; r0 += w.workers) {
      const int nb = (int)((counts[5] - r0) < w.workers ? (counts[5] - r0) : w.workers);
      dense_batch_setup_kernel<<<1, 32, 0, st>>>(rows0 + 5 * m, (int)r0, nb, in.Apos, ctl);
      SB_LAUNCH_CHECK("dense_batch_setup_kernel");
      spgemm_dense_kernel<T, NUMERIC><<<grid, 256, 0, st>>>(
          rows0 + 5 * m, (int)r0, nb, in, w.words, w.bitmap, static_cast<Slot*>(w.dense_acc),
          (long long)n, ctl, w.row_cnt, Cpos, Ccrd, Cval);
      SB_LAUNCH_CHECK("spgemm_dense_kernel");
    }
  }
  return SB_OK;
}

static int check_spgemm(int64_t m, int64_t kb, int64_t n, const void* Apos, const void* Bpos,
                        void* ws, size_t ws_bytes, int dtype) {
  SB_CHECK_ARG(m >= 0 && kb >= 0 && n >= 0, "spgemm: negative size");
  SB_CHECK_ARG(m < INT32_MAX / 8 && kb < INT32_MAX && n < INT32_MAX - 1,
               "spgemm: dimension exceeds the supported int32 range");
  SB_CHECK_ARG(Apos && Bpos, "spgemm: null row pointers");
  SB_CHECK_ARG(ws && aligned16(ws), "spgemm: workspace is null or misaligned");
  (void)dtype;
  const size_t need = sb_spgemm_workspace_bytes(m, n, SB_F32);  // the same for every dtype
  if (ws_bytes < need)
    return fail(SB_ERR_WORKSPACE, "spgemm: workspace has %zu bytes, needs %zu", ws_bytes, need);
  return SB_OK;
}

}  // namespace sb

using namespace sb;

extern "C" {

size_t sb_spgemm_workspace_bytes(int64_t m, int64_t n, int dtype) {
  if (m < 0) m = 0;
  if (n < 0) n = 0;
  // One size for all dtypes (the symbolic phase does not know the numeric dtype): the largest
  // of the per-dtype layouts.
  (void)dtype;
  const size_t a = ws_layout(nullptr, m, n, SB_F32).total;
  const size_t b = ws_layout(nullptr, m, n, SB_F64).total;
  return a > b ? a : b;
}

int sb_spgemm_symbolic(int64_t m, int64_t kb, int64_t n, const int32_t* Apos, const int32_t* Acrd,
                       const int32_t* Bpos, const int32_t* Bcrd, int32_t* Cpos,
                       int64_t* total_nnz_host, void* ws, size_t ws_bytes, void* stream) {
  int rc = check_spgemm(m, kb, n, Apos, Bpos, ws, ws_bytes, SB_F32);
  if (rc != SB_OK) return rc;
  SB_CHECK_ARG(Cpos && total_nnz_host, "spgemm_symbolic: null output");
  cudaStream_t st = (cudaStream_t)stream;
  // the symbolic phase only needs the bitmaps; lay the workspace out for the smallest dtype so
  // that any numeric dtype (whose layout is recomputed there) fits the caller's buffer
  WsLayout w = ws_layout(ws, m, n, SB_F32);
  *total_nnz_host = 0;
  SB_CUDA(cudaMemsetAsync(w.hdr, 0, 16 * 8, st));
  SB_CUDA(cudaMemsetAsync(w.bin_cursor, 0, 16 * 4, st));
  if (m == 0) {
    SB_CUDA(cudaMemsetAsync(Cpos, 0, 4, st));
    SB_CUDA(cudaStreamSynchronize(st));
    return SB_OK;
  }
  spgemm_bin_kernel<<<(unsigned)ceil_div(m * 8, 256), 256, 0, st>>>(
      (int)m, Apos, Acrd, Bpos, w.upper, w.bin_rows, w.bin_cursor, w.row_cnt);
  SB_LAUNCH_CHECK("spgemm_bin_kernel");
  int cursors[kBins];
  SB_CUDA(cudaMemcpyAsync(cursors, w.bin_cursor, sizeof(cursors), cudaMemcpyDeviceToHost, st));
  SB_CUDA(cudaStreamSynchronize(st));
  long long counts[kBins];
  for (int b = 0; b < kBins; b++) counts[b] = cursors[b];
  if (counts[kBins - 1] > 0) SB_CUDA(cudaMemsetAsync(w.bitmap, 0, (size_t)w.workers * w.words * 4, st));
  CsrIn in{Apos, Acrd, nullptr, Bpos, Bcrd, nullptr, nullptr};
  rc = launch_bins<float, false>(w, counts, m, n, in, nullptr, nullptr, nullptr, st);
  if (rc != SB_OK) return rc;
  rc = exclusive_scan_i32((int)m, w.row_cnt, Cpos, w.block_sum, w.hdr + 8, st);
  if (rc != SB_OK) return rc;
  // keep the bin sizes in the workspace header for the numeric phase
  SB_CUDA(cudaMemcpyAsync(w.hdr, counts, sizeof(counts), cudaMemcpyHostToDevice, st));
  long long total = 0;
  SB_CUDA(cudaMemcpyAsync(&total, w.hdr + 8, 8, cudaMemcpyDeviceToHost, st));
  SB_CUDA(cudaStreamSynchronize(st));
  *total_nnz_host = total;
  if (total > INT32_MAX)
    return fail(SB_ERR_OVERFLOW, "spgemm: the product has %lld stored entries, which does not fit "
                "the int32 row pointers", total);
  return SB_OK;
}

int sb_spgemm_numeric(int dtype, int64_t m, int64_t kb, int64_t n, const int32_t* Apos,
                      const int32_t* Acrd, const void* Aval, const int32_t* Bpos,
                      const int32_t* Bcrd, const void* Bval, const int32_t* Cpos, int32_t* Ccrd,
                      void* Cval, void* ws, size_t ws_bytes, void* stream) {
  SB_CHECK_ARG(dtype >= SB_F32 && dtype <= SB_I64, "spgemm_numeric: unknown dtype");
  int rc = check_spgemm(m, kb, n, Apos, Bpos, ws, ws_bytes, dtype);
  if (rc != SB_OK) return rc;
  SB_CHECK_ARG(Cpos, "spgemm_numeric: Cpos is null");
  if (m == 0) return SB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  // the row bins sit at dtype-independent offsets; the dense area is re-laid-out for `dtype`
  WsLayout w = ws_layout(ws, m, n, dtype);
  long long counts[kBins];
  SB_CUDA(cudaMemcpyAsync(counts, w.hdr, sizeof(counts), cudaMemcpyDeviceToHost, st));
  SB_CUDA(cudaStreamSynchronize(st));
  long long binned = 0;
  for (int b = 0; b < kBins; b++) {
    SB_CHECK_ARG(counts[b] >= 0 && counts[b] <= m, "spgemm_numeric: workspace does not hold the "
                 "bins of a symbolic call");
    binned += counts[b];
  }
  SB_CHECK_ARG(binned <= m, "spgemm_numeric: workspace does not hold the bins of a symbolic call");
  if (binned == 0) return SB_OK;
  SB_CHECK_ARG(Ccrd && Cval && Aval && Bval, "spgemm_numeric: null pointer");
  if (counts[kBins - 1] > 0) {
    SB_CUDA(cudaMemsetAsync(w.bitmap, 0, (size_t)w.workers * w.words * 4, st));
    SB_CUDA(cudaMemsetAsync(w.dense_acc, 0, (size_t)w.workers * (size_t)n * dtype_size(dtype), st));
  }
  CsrIn in{Apos, Acrd, Aval, Bpos, Bcrd, Bval, w.row_scale};
  if (dtype == SB_F32 || dtype == SB_F64) {
    long long bnnz = 0;   // stored entries of B = its last row pointer
    SB_CUDA(cudaMemcpyAsync(&bnnz, Bpos + kb, 4, cudaMemcpyDeviceToHost, st));
    SB_CUDA(cudaMemsetAsync(w.max_b, 0, 8, st));
    SB_CUDA(cudaStreamSynchronize(st));
    bnnz &= 0xffffffffLL;
    if (bnnz > 0) {
      const unsigned blocks = (unsigned)std::min<long long>(ceil_div(bnnz, 256), 8LL * sm_count());
      if (dtype == SB_F32) spgemm_max_abs_kernel<float><<<blocks, 256, 0, st>>>(bnnz, (const float*)Bval, w.max_b);
      else spgemm_max_abs_kernel<double><<<blocks, 256, 0, st>>>(bnnz, (const double*)Bval, w.max_b);
      SB_LAUNCH_CHECK("spgemm_max_abs_kernel");
    }
    const unsigned grid = (unsigned)ceil_div(m * 8, 256);
    if (dtype == SB_F32)
      spgemm_row_scale_kernel<float><<<grid, 256, 0, st>>>((int)m, Apos, (const float*)Aval, w.max_b, w.row_scale);
    else
      spgemm_row_scale_kernel<double><<<grid, 256, 0, st>>>((int)m, Apos, (const double*)Aval, w.max_b, w.row_scale);
    SB_LAUNCH_CHECK("spgemm_row_scale_kernel");
  }
  switch (dtype) {
    case SB_F32:
      return launch_bins<float, true>(w, counts, m, n, in, Cpos, Ccrd, (float*)Cval, st);
    case SB_F64:
      return launch_bins<double, true>(w, counts, m, n, in, Cpos, Ccrd, (double*)Cval, st);
    case SB_I32:
      return launch_bins<unsigned int, true>(w, counts, m, n, in, Cpos, Ccrd, (unsigned int*)Cval, st);
    default:
      return launch_bins<unsigned long long, true>(w, counts, m, n, in, Cpos, Ccrd,
                                                   (unsigned long long*)Cval, st);
  }
}

}  // extern "C"
