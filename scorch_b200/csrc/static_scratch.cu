// SpMV for callers that cannot allocate device memory.
//
// Some hosts of this library never get to call cudaMalloc: a plugin that runs inside another
// runtime's memory budget (every byte on the device belongs to the host application's arena),
// or a real-time / pre-initialised service that must not touch the allocator after start-up.
// sb_spmv_csr_f32 needs two caller-provided buffers besides its inputs and outputs: the row plan
// and the heavy-segment scratch.  The entry point below keeps both in one array that is part of
// the library image, so the caller passes nothing but the matrix, x and y.
//
// Price: every GPU that loads the library holds SB_STATIC_SCRATCH_BYTES of device memory until
// the process exits, the supported nnz is capped, and because all calls share the one array,
// two calls that overlap on the same GPU (different streams or threads) race on it.
#include <mutex>

#include "common.cuh"

namespace sb {

// plan for the largest supported matrix + one float per heavy segment
constexpr long long kStaticMaxNnz = SB_STATIC_SPMV_MAX_NNZ;
constexpr long long kCapHeavy = kStaticMaxNnz / SB_HEAVY_ROW_NNZ + 1;
constexpr long long kCapSeg = kStaticMaxNnz / SB_HEAVY_ROW_NNZ + kCapHeavy;
constexpr long long kPlanBytes = ((8 + 3 * kCapHeavy + kCapSeg) * 4 + 255) / 256 * 256;
constexpr long long kSegBytes = (kCapSeg * 4 + 255) / 256 * 256;
static_assert(kPlanBytes + kSegBytes <= SB_STATIC_SCRATCH_BYTES, "static scratch too small");

// In host code this name is only a handle for the symbol, not a device address: the address a
// kernel can use comes from cudaGetSymbolAddress (below), once per device.
static __device__ __align__(256) unsigned char g_static_scratch[SB_STATIC_SCRATCH_BYTES];

static std::mutex g_mu;
static unsigned char* g_dev_ptr[64] = {nullptr};

// Device address of the array on the current device; resolved on the first call per device.
static int static_scratch_ptr(unsigned char** out) {
  int dev = 0;
  SB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(SB_ERR_UNSUPPORTED, "static scratch: device index %d", dev);
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_dev_ptr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(SB_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s",
                  cudaGetErrorString(e));
    g_dev_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_dev_ptr[dev];
  return SB_OK;
}

}  // namespace sb

using namespace sb;

extern "C" {

int sb_spmv_csr_f32_static(int64_t m, int64_t n, int64_t nnz, const int32_t* pos,
                           const int32_t* crd, const float* val, const float* x, float* y,
                           void* stream) {
  if (nnz > kStaticMaxNnz)
    return fail(SB_ERR_UNSUPPORTED,
                "spmv_static: nnz=%lld exceeds the %lld entries the built-in scratch covers; use "
                "sb_spmv_csr_f32 with caller-provided plan and scratch",
                (long long)nnz, (long long)kStaticMaxNnz);
  SB_CHECK_ARG(m >= 0 && nnz >= 0 && pos, "spmv_static: bad size or null pos");
  unsigned char* base = nullptr;
  int rc = static_scratch_ptr(&base);
  if (rc != SB_OK) return rc;
  void* plan = base;
  void* seg = base + kPlanBytes;
  // The array keeps whatever the previous call left.  plan_build zeroes the plan header it
  // counts into; every segment sum is written before the finalise kernel reads it.
  rc = sb_csr_plan_build(m, nnz, pos, plan, (size_t)kPlanBytes, stream);
  if (rc != SB_OK) return rc;
  // -1: launch for the worst-case segment count of this nnz, so no count has to come back to
  // the host (no synchronisation, no allocation); surplus CTAs exit at once.
  return sb_spmv_csr_f32(m, n, nnz, pos, crd, val, x, y, plan, -1, seg, (size_t)kSegBytes, stream);
}

}  // extern "C"
