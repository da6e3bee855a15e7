// mbarrier and TMA (cp.async.bulk.tensor) helpers shared by the kernels that
// stage tiles through shared memory with the tensor memory accelerator, and the
// host-side tensor-map builder.
//
// Every wait on an mbarrier is bounded: after about a second without progress
// the waiter stores a code in a host-visible status word and returns false, and
// the kernel runs to its normal end instead of spinning.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200attn {

// ---- host side (defined in attn_tc5.cu) --------------------------------------
// 4-D tiled map over a 16-bit tensor: dims (128, n1, n2, n3), strides s1..s3 in
// elements (a unit extent may carry stride 0), box 64 x box1 x box2 x 1 elements,
// 128-byte swizzle, out-of-range elements read as zero.  False if the geometry
// cannot be encoded (strides not multiples of 16 bytes, extents too large).
bool make_tensor_map_4d(CUtensorMap *map, bool bf16, const void *base, uint64_t n1, uint64_t n2, uint64_t n3, long s1,
                        long s2, long s3, uint32_t box1, uint32_t box2);

namespace tma {

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait.  Returns false (and raises the flags) when the phase has not
// completed within ~2e9 cycles, or at once when another waiter already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          int *error_flag, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3ff) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > 2000000000LL) {
        *abort_flag = 1;
        *reinterpret_cast<volatile int *>(error_flag) = code;
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Orders this thread's earlier generic-proxy accesses to shared memory before later
// accesses of the async proxy (a TMA write into a buffer the thread has just written).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// One box of a 4-D tiled map -> shared memory; completion counts bytes on `bar`.  No multicast.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

} // namespace tma
} // namespace b200attn
