// SpMV for callers that cannot allocate device memory.
//
// Some hosts of this library never get to call cudaMalloc: a plugin that runs inside another
// runtime's memory budget (every byte on the device belongs to the host application's arena),
// or a real-time / pre-initialised service that must not touch the allocator after start-up.
// sb_spmv_csr_f32 needs one caller-provided buffer besides its inputs and outputs: the scratch
// for the partial sums of rows cut by tile borders.  The entry point below keeps it in an array
// that is part of the library image, so the caller passes nothing but the matrix, x and y.
//
// Price: every GPU that loads the library holds SB_STATIC_SCRATCH_BYTES of device memory until
// the process exits, the supported nnz is capped, and because all calls share the one array,
// two calls that overlap on the same GPU (different streams or threads) race on it.
#include <mutex>

#include "common.cuh"

namespace sb {

// partial-sum arrays of the largest supported matrix: three 4-byte arrays with one slot per
// 2048-entry tile (the layout of sb_spmv_csr_scratch_bytes)
constexpr long long kStaticMaxNnz = SB_STATIC_SPMV_MAX_NNZ;
static_assert(((kStaticMaxNnz / 2048 + 1) * 4 + 255) / 256 * 256 * 3 <= SB_STATIC_SCRATCH_BYTES,
              "static scratch too small");

// In host code this name is only a handle for the symbol, not a device address: the address a
// kernel can use comes from cudaGetSymbolAddress (below), once per device.
static __device__ __align__(256) unsigned char g_static_scratch[SB_STATIC_SCRATCH_BYTES];

static std::mutex g_mu;
static unsigned char* g_dev_ptr[64] = {nullptr};

// Device address of the array on the current device; resolved on the first call per device and
// kept for the life of the process (a cudaDeviceReset would leave it stale: see the header).
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
  SB_CHECK_ARG(m >= 0 && n >= 0 && nnz >= 0, "spmv_static: negative size");
  SB_CHECK_ARG(pos, "spmv_static: pos is null");
  if (nnz > kStaticMaxNnz)
    return fail(SB_ERR_UNSUPPORTED,
                "spmv_static: nnz=%lld exceeds the %lld entries the built-in scratch covers; use "
                "sb_spmv_csr_f32 with a scratch buffer of your own",
                (long long)nnz, (long long)kStaticMaxNnz);
  unsigned char* base = nullptr;
  int rc = static_scratch_ptr(&base);
  if (rc != SB_OK) return rc;
  // The array keeps whatever the previous call left: every slot the fix-up kernel reads is
  // written by the tile kernel of the same call first.
  return sb_spmv_csr_f32(m, n, nnz, pos, crd, val, x, y, base, (size_t)SB_STATIC_SCRATCH_BYTES, stream);
}

}  // extern "C"
