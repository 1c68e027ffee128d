// Asynchronous-copy building blocks shared by the stage-1 kernels: mbarriers, tiled TMA loads, the proxy fence,
// and the kernel-parameter block that carries the TMA descriptors.
#pragma once

#include <cuda.h>

#include "ft_common.cuh"

namespace ft {

// Kernel parameters of the kernels that use TMA: the common ones plus the descriptors of the K and V buffers
// ([rows, kv heads, head_dim], box 64 x 1 x 64 elements, 128-byte swizzle).  has_tma == 0: gather only.
struct alignas(64) TcParams {
  CUtensorMap k_map;
  CUtensorMap v_map;
  CUtensorMap q_map;       // [batch, heads, head_dim], box 64 x q_box_rows x 1: one request
  CUtensorMap q_map_tile;  // same tensor, box 64 x G x 128 / G: a whole Q tile of consecutive requests
  Stage1Params p;
  int has_tma;
  int q_box_rows;     // 0: gather Q with cp.async (group size not a power of two <= 128, or no descriptor)
  unsigned int* sched;  // persistent kernel: {tasks claimed beyond the first per CTA, CTAs finished}, zero between launches
};

__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// announces transaction bytes without arriving
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// the barrier gets one arrival when all earlier cp.async copies of this thread have landed
__device__ __forceinline__ void mbar_arrive_on_cp_async(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::
          "r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}

// Bounded wait for the phase of `bar` with the given parity: false after `limit` probes.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int limit) {
  for (int it = 0; it < limit; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

}  // namespace ft
