// Row pipeline primitives for sm_100a: 1-D bulk asynchronous copies (TMA, cp.async.bulk, never multicast)
// from global into shared memory, completion tracked by an mbarrier per stage.
//
// Usage pattern of the row-streaming kernels (one elected thread produces, every thread consumes):
//   prologue : elected thread arms stage s (expect_tx with the byte count) and issues the copies of row s;
//   steady   : all threads wait on stage s (bounded spin), move the row to registers, pass a CTA barrier,
//              then the elected thread re-arms stage s for the row STAGES ahead.
// Every wait is bounded: when the limit is hit the kernel records an error code in the per-device error word
// (pipe_error_ptr()), stops issuing new copies, drains the copies already in flight (again bounded) and returns,
// so a lost completion can never turn into a hang.  The host reads (and clears) the code with mcop_device_error().
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mcop {

// Device address of the error word of the current device (0 = no error); set by a pipeline kernel whose bounded
// wait ran out.  Resolved once per device with cudaGetSymbolAddress; returns nullptr if that fails.
int* pipe_error_ptr();

constexpr uint32_t kPipeSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
// makes the barrier initialisation visible to the asynchronous proxy before the first copy uses it
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// orders earlier generic-proxy accesses of shared memory before later asynchronous-proxy writes to it
__device__ __forceinline__ void proxy_fence_before_reuse() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// global -> shared bulk copy; dst, src 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (after recording `code`) if the phase did not complete within `limit` tries.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int* err, int code, uint32_t limit = kPipeSpinLimit) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  if (err) atomicCAS(err, 0, code);
  return false;
}

// The same with a suspend-time hint: a thread whose phase is not complete yet may stay suspended in hardware for up to
// kPipeSleepNs before the instruction returns, instead of coming back at once and polling again.  For kernels whose
// warps mostly wait for data (the gather) this leaves the issue slots to the warps that have work: measured +3 % there,
// -1 % in the norm and scatter kernels, whose waits are short - so only the gather uses it.  Bounded like the plain
// form: kPipeSleepLimit tries of at most kPipeSleepNs each (about 1.3 s).
constexpr uint32_t kPipeSleepNs = 20000u;
constexpr uint32_t kPipeSleepLimit = 1u << 16;
__device__ __forceinline__ bool mbar_wait_bounded_sleepy(uint64_t* bar, uint32_t parity, int* err, int code) {
  for (uint32_t i = 0; i < kPipeSleepLimit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity), "r"(kPipeSleepNs)
        : "memory");
    if (ok) return true;
  }
  if (err) atomicCAS(err, 0, code);
  return false;
}

// Position in a ring of `stages` buffers: stage index and phase parity of its mbarrier, advanced without the
// integer division a running counter would need on every row.
struct RingPos {
  int s = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void advance(int stages) {
    if (++s == stages) { s = 0; phase ^= 1u; }
  }
};

__device__ __forceinline__ uint4 lds_u4(const void* p) {
  uint4 r;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(smem_addr(p)));
  return r;
}

// Programmatic dependent launch.  The kernels of the path are launched with the stream-serialisation attribute, which
// lets the NEXT kernel's CTAs be scheduled (and run their set-up: barrier initialisation, shared-memory carve-up) while
// the previous kernel is still finishing, instead of after its last CTA has retired and the launch latency has passed.
//   pdl_launch_dependents(): "the kernel after me may start being scheduled" - called first thing in every such kernel;
//   pdl_wait(): blocks until every kernel ahead in the stream has COMPLETED and its writes are visible - called before
//               the kernel's first access to global memory (so nothing is read early and nothing is overwritten early).
// A kernel launched without the attribute, before or after, is ordered as usual.  MCOP_DISABLE_PDL=1 in the environment
// (read once) launches everything without the attribute, for comparisons.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Number of SMs of the current device (cached per device; no allocation, no synchronisation).
int sm_count();

// Makes sure `kernel` may use `bytes` of dynamic shared memory on the CURRENT device (the attribute is per device;
// what has been granted is remembered per device and kernel).  Thread-safe.
cudaError_t ensure_dynamic_smem(const void* kernel, size_t bytes);

}  // namespace mcop
