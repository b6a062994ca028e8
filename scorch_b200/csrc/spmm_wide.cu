// CSR x dense SpMM for wide dense operands (k >= 512) with the operand rows staged through shared
// memory by the bulk-copy engine, and the probe kernel that measures the L2 gather rate such a
// product is bound by.
//
// A product with a wide operand reads one k-wide row of B per stored entry.  Taken in 256-column
// panels (one 32768-row panel = 32 MB stays in L2 while all rows of A pass over it) DRAM traffic
// is already the compulsory one; what remains is L2 -> SM traffic: nnz * k * 4 bytes.  The rows
// kernel of spmm.cu gathers those slices through L1 into registers (ld.global.nc.v8).  Here a
// producer warp issues one 1-D bulk copy (cp.async.bulk, global -> shared, completion counted on
// an mbarrier; no multicast) per stored entry and panel into a ring of shared-memory stages, and
// 256 consumer threads — one per column of the panel — add the weighted slices.  L1 and the
// register file are off the data path; what is measured against the rows kernel is whether the
// L2 delivers more that way.
//
// Every wait on an mbarrier is bounded: after kSpinLimit failed polls the thread records the
// failure in a status word (sb_spmm_wide_status) and leaves its loops.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

#ifndef SB_SPMM_TMA_STAGES
#define SB_SPMM_TMA_STAGES 4
#endif

namespace sb {

constexpr int kTmaStages = SB_SPMM_TMA_STAGES;
constexpr int kTmaChunk = 32;                 // stored entries (operand-row slices) per stage
constexpr int kTmaPanel = 256;                // columns per panel = consumer threads
constexpr int kTmaThreads = kTmaPanel + 32;   // + the producer warp
constexpr unsigned kSpinLimit = 1u << 24;

__device__ int g_wide_status = 0;  // 0 ok; 1 a producer wait gave up; 2 a consumer wait gave up

struct WideArgs {
  int m, k;
  const int* pos;
  const int* crd;
  const float* val;
  const float* B;
  long long ldb;
  const float* bias;
  int relu;
  float* C;
  long long ldc;
  int panels;
};

struct __align__(128) WideStage {
  float slice[kTmaChunk][kTmaPanel];   // 32 KB
};

constexpr int kTmaBatch = 32;  // tasks whose first index chunks the producer stages at a time

struct WideShared {
  WideStage stage[kTmaStages];
  float a[kTmaStages][kTmaChunk];
  // first chunk (column indices, values) of the next tasks, staged by asynchronous copies one
  // batch ahead of their use: [buffer][task in batch][entry]
  int pre_j[2][kTmaBatch][kTmaChunk];
  float pre_a[2][kTmaBatch][kTmaChunk];
  unsigned long long full[kTmaStages];
  unsigned long long empty[kTmaStages];
};

__device__ __forceinline__ unsigned smem_addr(const void* p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_addr(bar))
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(
                   smem_addr(bar)),
               "r"(bytes)
               : "memory");
}
// Bounded wait for the phase with the given parity; false = gave up.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
  const unsigned addr = smem_addr(bar);
  for (unsigned spin = 0; spin < kSpinLimit; spin++) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
// 1-D bulk copy global -> shared of `bytes` (multiple of 16, both addresses 16-byte aligned);
// completion is counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}

// Persistent CTAs over (panel, row) tasks, panel-major, so that all CTAs work on one panel of B
// at a time.  Warp 8 produces, warps 0-7 consume (thread c = column c of the panel).
__global__ void __launch_bounds__(kTmaThreads, 1)
spmm_wide_kernel(WideArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  WideShared& s = *reinterpret_cast<WideShared*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int i = 0; i < kTmaStages; i++) {
      mbar_init(&s.full[i], 1);                // the producer's elected lane (+ the bytes it announces)
      mbar_init(&s.empty[i], kTmaPanel / 32);  // one arrival per consumer warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const long long tasks = (long long)a.m * a.panels;
  unsigned it = 0;  // chunks this CTA has gone through: stage = it % stages, phase = it / stages
  if (warp == kTmaPanel / 32) {
    // ---- producer ----
    // Tasks are taken in batches of 32 (lane l looks after task l of the batch).  Row bounds are
    // loaded two batches ahead and the first index chunk of every task one batch ahead (4-byte
    // asynchronous copies into shared memory), so the issue loop below finds them there and
    // waits for nothing but free stages.
    const long long stride = gridDim.x, batch_stride = stride * kTmaBatch;
    auto bounds = [&](long long base, int& b, int& e) {
      const long long t = base + lane * stride;
      b = e = 0;
      if (t < tasks) {
        const int row = (int)(t % a.m);
        b = __ldg(a.pos + row);
        e = __ldg(a.pos + row + 1);
      }
    };
    auto stage_indices = [&](int buf, int my_b, int my_e) {
      for (int i = 0; i < kTmaBatch; i++) {
        const int p = __shfl_sync(FULL, my_b, i) + lane;
        if (p < __shfl_sync(FULL, my_e, i)) {
          asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_addr(&s.pre_j[buf][i][lane])),
                       "l"(a.crd + p)
                       : "memory");
          asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_addr(&s.pre_a[buf][i][lane])),
                       "l"(a.val + p)
                       : "memory");
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    int cur_b, cur_e, nxt_b, nxt_e;
    bounds(blockIdx.x, cur_b, cur_e);
    bounds(blockIdx.x + batch_stride, nxt_b, nxt_e);
    stage_indices(0, cur_b, cur_e);
    int buf = 0;
    for (long long base = blockIdx.x; base < tasks; base += batch_stride, buf ^= 1) {
      stage_indices(buf ^ 1, nxt_b, nxt_e);            // next batch's first chunks
      int nn_b, nn_e;
      bounds(base + 2 * batch_stride, nn_b, nn_e);     // bounds of the batch after it
      asm volatile("cp.async.wait_group 1;" ::: "memory");   // this batch's chunks have landed
      __syncwarp();
      for (int i = 0; i < kTmaBatch; i++) {
        const long long t = base + i * stride;
        if (t >= tasks) break;
        const int panel = (int)(t / a.m);
        const int b = __shfl_sync(FULL, cur_b, i), e = __shfl_sync(FULL, cur_e, i);
        const unsigned bytes = (unsigned)min(kTmaPanel, a.k - panel * kTmaPanel) * 4u;
        const float* Bp = a.B + (long long)panel * kTmaPanel;
        for (int p0 = b; p0 < e; p0 += kTmaChunk, it++) {
          const unsigned st = it % kTmaStages, ph = (it / kTmaStages) & 1u;
          const int p = p0 + lane;
          const bool valid = p < e;
          int j = 0;
          float av = 0.f;
          if (valid) {
            if (p0 == b) {
              j = s.pre_j[buf][i][lane];
              av = s.pre_a[buf][i][lane];
            } else {  // rows longer than one chunk: the further chunks are read on demand
              j = ld_stream(a.crd + p);
              av = ld_stream(a.val + p);
            }
          }
          if (!mbar_wait(&s.empty[st], ph ^ 1u)) {   // (a fresh barrier passes the first round)
            atomicExch(&g_wide_status, 1);
            asm volatile("cp.async.wait_all;" ::: "memory");
            return;
          }
          s.a[st][lane] = av;
          __syncwarp();
          // one arrival announces the whole chunk's bytes (an arrival per lane would be 32
          // serialised updates of the barrier word), then every lane issues its copy
          if (lane == 0) mbar_arrive_expect_tx(&s.full[st], (unsigned)min(kTmaChunk, e - p0) * bytes);
          __syncwarp();
          if (valid) bulk_load(&s.stage[st].slice[lane][0], Bp + (long long)j * a.ldb, bytes, &s.full[st]);
        }
      }
      cur_b = nxt_b; cur_e = nxt_e;
      nxt_b = nn_b; nxt_e = nn_e;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    return;
  }
  // ---- consumers ----
  for (long long t = blockIdx.x; t < tasks; t += gridDim.x) {
    const int panel = (int)(t / a.m), row = (int)(t % a.m);
    const int b = __ldg(a.pos + row), e = __ldg(a.pos + row + 1);
    const int col = panel * kTmaPanel + tid;
    float acc = 0.f;
    for (int p0 = b; p0 < e; p0 += kTmaChunk, it++) {
      const unsigned st = it % kTmaStages, ph = (it / kTmaStages) & 1u;
      if (!mbar_wait(&s.full[st], ph)) {
        atomicExch(&g_wide_status, 2);
        return;
      }
      const int cnt = min(kTmaChunk, e - p0);
      if (col < a.k) {
#pragma unroll 8
        for (int l = 0; l < cnt; l++) acc = fmaf(s.a[st][l], s.stage[st].slice[l][tid], acc);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.empty[st]);
    }
    if (col < a.k) {
      if (a.bias) acc += __ldg(a.bias + col);
      if (a.relu) acc = acc > 0.f ? acc : 0.f;
      a.C[(long long)row * a.ldc + col] = acc;
    }
  }
}

// ---- L2 gather-rate probe ----------------------------------------------------------------------
// Every warp reads `gathers` pseudo-random 1 KB rows (256 floats, one 256-bit load per lane, four
// in flight) of a `rows`-row panel and keeps a checksum: the load pattern of a wide SpMM over an
// L2-resident panel with nothing else on the critical path.
__global__ void __launch_bounds__(256)
l2_gather_probe_kernel(const float* __restrict__ panel, unsigned rows, int gathers, float* out) {
  const unsigned warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  unsigned x = warp * 2654435761u + 12345u;
  float acc = 0.f;
  for (int g = 0; g < gathers; g += 4) {
    float v[4][8];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      x = x * 1664525u + 1013904223u;
      const float* p = panel + (size_t)(__umulhi(x, rows)) * 256 + lane * 8;
      asm volatile("ld.global.nc.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                   : "=f"(v[u][0]), "=f"(v[u][1]), "=f"(v[u][2]), "=f"(v[u][3]), "=f"(v[u][4]),
                     "=f"(v[u][5]), "=f"(v[u][6]), "=f"(v[u][7])
                   : "l"(p));
    }
#pragma unroll
    for (int u = 0; u < 4; u++) acc += v[u][0] + v[u][3] + v[u][5] + v[u][6];
  }
  if (acc == 123.456f) out[warp] = acc;  // keeps the loads alive; practically never true
}

// Which kernel sb_spmm_csr_f32 takes for wide operands: 1 = this file's bulk-copy kernel,
// 0 = the gather kernel of spmm.cu.  Set by sb_spmm_wide_select(), else by the environment
// variable SCORCH_B200_SPMM_WIDE = "tma" | "gather", else the default below.
constexpr int kWideDefault = 0;
static int g_wide_mode = -1;

static int wide_mode() {
  if (g_wide_mode < 0) {
    const char* e = std::getenv("SCORCH_B200_SPMM_WIDE");
    g_wide_mode = (e && !std::strcmp(e, "tma")) ? 1 : ((e && !std::strcmp(e, "gather")) ? 0 : kWideDefault);
  }
  return g_wide_mode;
}

bool spmm_wide_wanted() { return wide_mode() == 1; }

int spmm_wide_launch(int64_t m, int64_t k, const int* pos, const int* crd, const float* val, const float* B,
                     int64_t ldb, const float* bias, int relu, float* C, int64_t ldc, cudaStream_t st) {
  WideArgs a;
  a.m = (int)m; a.k = (int)k; a.pos = pos; a.crd = crd; a.val = val; a.B = B; a.ldb = ldb;
  a.bias = bias; a.relu = relu; a.C = C; a.ldc = ldc;
  a.panels = (int)ceil_div(k, kTmaPanel);
  const size_t smem = sizeof(WideShared) + 128;
  static bool configured[64] = {false};
  int dev = 0;
  SB_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    SB_CUDA(cudaFuncSetAttribute(spmm_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = true;
  }
  const long long tasks = (long long)m * a.panels;
  const unsigned grid = (unsigned)std::min<long long>(tasks, sm_count());
  spmm_wide_kernel<<<grid, kTmaThreads, smem, st>>>(a);
  SB_LAUNCH_CHECK("spmm_wide_kernel");
  return SB_OK;
}

}  // namespace sb

using namespace sb;

extern "C" {

int sb_spmm_wide_select(int mode) {
  const int before = wide_mode();
  if (mode == 0 || mode == 1) g_wide_mode = mode;
  return before;
}

int sb_spmm_wide_status(void) {
  int v = -1;
  if (cudaMemcpyFromSymbol(&v, g_wide_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

int sb_probe_l2_gather(const float* panel, int64_t rows, int64_t gathers_per_warp, int64_t warps,
                       float* out, void* stream) {
  SB_CHECK_ARG(panel && out && rows > 0 && rows < (1ll << 24) && gathers_per_warp > 0 && warps > 0,
               "probe_l2_gather: bad argument");
  SB_CHECK_ARG(gathers_per_warp % 4 == 0 && warps % 8 == 0, "probe_l2_gather: gathers must be a multiple of 4, warps of 8");
  l2_gather_probe_kernel<<<(unsigned)(warps / 8), 256, 0, (cudaStream_t)stream>>>(panel, (unsigned)rows,
                                                                                  (int)gathers_per_warp, out);
  SB_LAUNCH_CHECK("l2_gather_probe_kernel");
  return SB_OK;
}

}  // extern "C"
