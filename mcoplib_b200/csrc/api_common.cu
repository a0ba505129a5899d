// Error reporting and version of the mcop_b200 C ABI.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include <atomic>
#include <mutex>

#include "common.cuh"
#include "tma_pipe.cuh"

namespace mcop {
namespace {
thread_local char g_error[512] = "";
}

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

// Error word written by pipeline kernels whose bounded wait ran out (one per device that loads the library).
__device__ int g_pipe_error_word = 0;

namespace {
constexpr int kMaxDevices = 64;
std::atomic<int*> g_err_ptr[kMaxDevices];
std::atomic<int> g_sm_count[kMaxDevices];
}  // namespace

int* pipe_error_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  int* p = g_err_ptr[dev].load(std::memory_order_acquire);
  if (p) return p;
  void* sym = nullptr;
  if (cudaGetSymbolAddress(&sym, g_pipe_error_word) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  g_err_ptr[dev].store(static_cast<int*>(sym), std::memory_order_release);
  return static_cast<int*>(sym);
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("MCOP_DISABLE_PDL");
    return !(v && v[0] && v[0] != '0');
  }();
  return on;
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  int n = g_sm_count[dev].load(std::memory_order_relaxed);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
    (void)cudaGetLastError();
    return 148;
  }
  g_sm_count[dev].store(n, std::memory_order_relaxed);
  return n;
}

// The dynamic shared memory a kernel may use above 48 KB is a property of the kernel ON ONE DEVICE, so the sizes
// already granted are remembered per (device, kernel); a process that drives several GPUs sets it on each.
// (A fixed table, no heap: the library's entry points never allocate.  When the table is full the attribute is simply
// set again on every call, which is correct, only slower.)
cudaError_t ensure_dynamic_smem(const void* kernel, size_t bytes) {
  struct Granted { int dev; const void* kernel; size_t bytes; };
  constexpr int kSlots = 1024;
  static std::mutex mu;
  static Granted table[kSlots];
  static int used = 0;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  Granted* slot = nullptr;
  for (int i = 0; i < used; ++i)
    if (table[i].dev == dev && table[i].kernel == kernel) { slot = &table[i]; break; }
  if (slot && slot->bytes >= bytes) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) return e;
  if (!slot && used < kSlots) {
    slot = &table[used++];
    slot->dev = dev;
    slot->kernel = kernel;
  }
  if (slot) slot->bytes = bytes;
  return cudaSuccess;
}

// Self-test of the bounded wait: a stage is armed and no copy is ever issued for it, so the wait must run out.  The
// kernel then does what the pipeline kernels do: the CTA agrees that the wait failed, one thread runs the (bounded)
// drain, everybody returns.  Nothing is in flight at any time.
__global__ void selftest_wait_kernel(uint32_t limit, int* err) {
  __shared__ __align__(8) uint64_t bar[1];
  if (threadIdx.x == 0) {
    mbar_init(&bar[0], 1);
    mbar_init_fence();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_expect_tx(&bar[0], 256);
  __syncthreads();
  const bool ok = mbar_wait_bounded(&bar[0], 0, err, MCOP_DEVERR_SELFTEST, limit);
  if (!__syncthreads_and(ok) && threadIdx.x == 0) (void)mbar_wait_bounded(&bar[0], 0, err, MCOP_DEVERR_SELFTEST, limit);
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return MCOP_OK;
  return set_error(MCOP_ERR_CUDA, "%s: kernel launch failed: %s", what, cudaGetErrorString(e));
}
}  // namespace mcop

extern "C" int mcop_version(void) { return 100; }
extern "C" const char* mcop_last_error(void) { return mcop::g_error; }

extern "C" int mcop_device_error(void) {
  int* p = mcop::pipe_error_ptr();
  if (!p) return mcop::set_error(MCOP_ERR_CUDA, "device_error: the error word of the current device is not reachable");
  int v = 0;
  cudaError_t e = cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return mcop::set_error(MCOP_ERR_CUDA, "device_error: %s", cudaGetErrorString(e));
  if (v != 0) {
    const int zero = 0;
    (void)cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice);
  }
  return v;
}

extern "C" int mcop_selftest_wait_timeout(int spin_limit, mcop_stream_t stream) {
  MCOP_REQUIRE(spin_limit >= 1 && spin_limit <= (1 << 20), MCOP_ERR_ARGUMENT, "selftest_wait_timeout: spin_limit must be in [1, 2^20]");
  int* err = mcop::pipe_error_ptr();
  MCOP_REQUIRE(err != nullptr, MCOP_ERR_CUDA, "selftest_wait_timeout: the error word of the current device is not reachable");
  mcop::selftest_wait_kernel<<<1, 64, 0, (cudaStream_t)stream>>>((uint32_t)spin_limit, err);
  return mcop::check_launch("selftest_wait_timeout");
}
