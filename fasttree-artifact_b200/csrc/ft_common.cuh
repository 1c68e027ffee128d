// Shared device-side definitions of the tree-attention decode kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fasttree_b200.h"

namespace ft {

// One word per device; kernels OR error bits into it instead of faulting.
__device__ int g_device_status = 0;

__device__ __forceinline__ void flag_error(int bit) { atomicOr(&g_device_status, bit); }

// Developer builds with -DFT_TIMELINE record, per CTA of a stage-1 launch, {start ns, end ns, SM id, kind, twelve marks} so that
// the placement and overlap of the task families can be read back (ft_debug_timeline); normal builds compile none of it.
#ifdef FT_TIMELINE
constexpr int FT_TIMELINE_CTAS = 1 << 16;
__device__ unsigned long long g_timeline[16 * FT_TIMELINE_CTAS];
__device__ __forceinline__ unsigned long long timeline_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define FT_TL_BEGIN() const unsigned long long tl_begin = ft::timeline_now()
#define FT_TL_END(kind)                                                        \
  do {                                                                         \
    if (threadIdx.x == 0 && blockIdx.x < ft::FT_TIMELINE_CTAS) {               \
      unsigned sm_id;                                                          \
      asm volatile("mov.u32 %0, %%smid;" : "=r"(sm_id));                       \
      ft::g_timeline[16 * blockIdx.x + 0] = tl_begin;                           \
      ft::g_timeline[16 * blockIdx.x + 1] = ft::timeline_now();                 \
      ft::g_timeline[16 * blockIdx.x + 2] = sm_id;                              \
      ft::g_timeline[16 * blockIdx.x + 3] = (kind);                             \
    }                                                                          \
  } while (0)
#define FT_TL_MARK(i)                                                          \
  do {                                                                         \
    if (blockIdx.x < ft::FT_TIMELINE_CTAS) ft::g_timeline[16 * blockIdx.x + 4 + (i)] = ft::timeline_now(); \
  } while (0)
// -DFT_TL_TILE=n moves the per-tile marks of the tensor-core kernel to tile n and swaps the start-up marks 2, 5, 6, 7 for
// {tile n+1's scores seen, scores in registers, row maximum known, P stored}.
#ifdef FT_TL_TILE
#define FT_TL_DETAIL_MARK(i) FT_TL_MARK(i)
#define FT_TL_COARSE_MARK(i) do { } while (0)
#else
#define FT_TL_TILE 5
#define FT_TL_DETAIL_MARK(i) do { } while (0)
#define FT_TL_COARSE_MARK(i) FT_TL_MARK(i)
#endif
// -DFT_TL_LOADERS hands the per-tile mark slots of the softmax to the loaders and the MMA warp instead (tile n: K issue
// start / end = 5 / 6, V issue start / end = 7 / 11, K and V seen by the MMA warp = 1 / 4).
#ifdef FT_TL_LOADERS
#define FT_TL_SOFTMAX_MARK(i) do { } while (0)
#else
#define FT_TL_SOFTMAX_MARK(i) do { if ((i) == 5 || (i) == 6 || (i) == 7) { FT_TL_DETAIL_MARK(i); } else { FT_TL_MARK(i); } } while (0)
#endif
#else
#define FT_TL_MARK(i) do { } while (0)
#define FT_TL_SOFTMAX_MARK(i) do { } while (0)
#define FT_TL_DETAIL_MARK(i) do { } while (0)
#define FT_TL_COARSE_MARK(i) do { } while (0)
#define FT_TL_TILE 5
#define FT_TL_BEGIN() do { } while (0)
#define FT_TL_END(kind) do { } while (0)
#endif

// Everything a stage-1 kernel needs, passed by value.
struct Stage1Params {
  const void* q;
  const void* k;
  const void* v;
  const int32_t* kv_entries;
  const int32_t* kv_offs;
  const int32_t* kv_lens;
  const int32_t* q_entries;
  const int32_t* q_offs;
  const int32_t* q_lens;
  const int32_t* q_ranges;  // optional [num_partial_rows][2]: the chunk tokens [begin, end) a partial row attends to
  const int32_t* dev_phase; // optional device array {n0, n1, o0, o1}: the persistent kernel reads its vnode range here
  const int32_t* kv_entries_aux;  // optional second row-id table: vnodes whose kv_offs value has bit 30 set index it
  int64_t kv_entries_aux_len;
  float* mid_o;
  float* mid_lse;
  int64_t q_s0, q_s1, k_s0, k_s1, v_s0, v_s1, mo_s0, mo_s1, ml_s0;
  int64_t kv_rows;
  int64_t kv_entries_len;
  int64_t num_partial_rows;
  int32_t batch;
  int32_t group;        // query heads per KV head
  int32_t head_dim;
  int32_t node_offset;  // first vnode of this launch
  int32_t node_count;   // vnodes in this launch
  int32_t num_kv_heads;
  int32_t node_split;   // fused launch: vnodes [0, node_split) of the launch are many-row tasks
  int32_t lead_wide;    // fused launch: many-row CTAs placed before the few-row CTAs in block order
  int32_t workers;      // fused launch: persistent few-row workers (0: one CTA per few-row task)
  float sm_scale;
};

// Row ids of a vnode's KV chunk.  vnode_to_kv_offs normally indexes vnode_to_kv_entries; with bit 30 set (and an
// auxiliary table given) the low 30 bits index vnode_to_kv_entries_aux instead: the serving path addresses tree
// nodes straight through req_to_token and keeps the concatenated row ids of grouped private tails in a table of its own.
constexpr int FT_AUX_BIT = 1 << 30;
__device__ __forceinline__ const int32_t* kv_ids_base(const Stage1Params& p, int kv_off) {
  return (kv_off & FT_AUX_BIT) != 0 && p.kv_entries_aux != nullptr ? p.kv_entries_aux + (kv_off & (FT_AUX_BIT - 1))
                                                                   : p.kv_entries + kv_off;
}
// readable row ids of the chunk (a table that ends early is a plan error: the caller flags it, those tokens become padding)
__device__ __forceinline__ int kv_ids_limit(const Stage1Params& p, int kv_off, int kv_len) {
  if (kv_off < 0) return 0;
  const bool aux = (kv_off & FT_AUX_BIT) != 0 && p.kv_entries_aux != nullptr;
  const int64_t readable = aux ? p.kv_entries_aux_len - (int64_t)(kv_off & (FT_AUX_BIT - 1)) : p.kv_entries_len - (int64_t)kv_off;
  return (int)(readable < (int64_t)kv_len ? (readable < 0 ? 0 : readable) : kv_len);
}

struct Stage2Params {
  const int32_t* r2v_entries;
  const int32_t* r2v_offs;
  const int32_t* r2v_lens;
  const float* mid_o;
  const float* mid_lse;
  void* o;
  float* o_lse;
  int64_t mo_s0, mo_s1, ml_s0, o_s0, o_s1;
  int64_t num_partial_rows;
  int32_t batch;
  int32_t heads;
  int32_t head_dim;
  int32_t o_vec;  // 1: o rows are aligned for 4-element vector stores
};

// Programmatic dependent launch: stage 1 lets the next kernel of the stream be scheduled while its own CTAs are
// still running; stage 2 is launched with that permission and waits here until stage 1 has completed and its
// writes are visible, so only its launch latency and its reads of the plan tables overlap stage 1's tail.
__device__ __forceinline__ void allow_dependent_launch() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void wait_for_prior_grid() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// Tensor-core kernels use a 1-D grid with the kv head varying fastest, so that CTAs launched next to
// each other read the same tokens' rows (adjacent 2*D-byte slices of one pool row).
__device__ __forceinline__ void task_of_block(const Stage1Params& p, int block, int& vnode, int& kv_head) {
  vnode = p.node_offset + block / p.num_kv_heads;
  kv_head = block - (block / p.num_kv_heads) * p.num_kv_heads;
}

template <typename T>
__device__ __forceinline__ float to_float(T x);
template <>
__device__ __forceinline__ float to_float<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_float<__half>(__half x) { return __half2float(x); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_float(float x);
template <>
__device__ __forceinline__ float from_float<float>(float x) { return x; }
template <>
__device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

}  // namespace ft
