// Stage 2: per-(request, query head) log-sum-exp merge of the request's partial
// rows (kernel_bench/fasttree.py:482-546).
//
// One warp per (request, head); lanes span head_dim in float4 chunks, so a
// partial row of head_dim 128 is one 512-byte coalesced warp load.  The
// weights exp(lse_i - max) are computed lane-parallel (32 partial rows at a
// time) and broadcast by shuffle, which keeps the dependent chain per partial
// to one FMA.  Memory-bound on the partial buffers; those are written by stage
// 1 just before and are normally still in L2.
#pragma once

#include "ft_common.cuh"

namespace ft {

template <typename T>
__global__ void __launch_bounds__(128) stage2_merge_kernel(Stage2Params p) {
  constexpr int MAXC = 2;  // float4 chunks per lane: head_dim <= 256
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t pair = (int64_t)blockIdx.x * 4 + warp;
  if (pair >= (int64_t)p.batch * p.heads) return;
  const int req = (int)(pair / p.heads);
  const int head = (int)(pair - (int64_t)req * p.heads);
  const int off = p.r2v_offs[req];
  const int n = p.r2v_lens[req];
  const int chunks = p.head_dim >> 2;
  int first_rows = lane < n ? p.r2v_entries[off + lane] : -1;  // plan data: readable before stage 1 is done
  wait_for_prior_grid();                                       // the partial buffers are complete from here on

  // pass 1: maximum LSE over the request's partial rows
  float mx = -INFINITY;
  for (int i = lane; i < n; i += 32) {
    const int row = i < 32 ? first_rows : p.r2v_entries[off + i];
    if (row < 0 || row >= p.num_partial_rows) {
      flag_error(FT_DEV_BAD_ROW_INDEX);
      continue;
    }
    mx = fmaxf(mx, p.mid_lse[(int64_t)row * p.ml_s0 + head]);
  }
  mx = warp_max(mx);

  float4 acc[MAXC];
#pragma unroll
  for (int c = 0; c < MAXC; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
  float wsum = 0.f;
  if (mx > -INFINITY) {
    for (int base = 0; base < n; base += 32) {
      const int cnt = min(32, n - base);
      int my_row = -1;
      float my_w = 0.f;
      if (lane < cnt) {
        const int row = p.r2v_entries[off + base + lane];
        if (row >= 0 && row < p.num_partial_rows) {
          my_row = row;
          my_w = expf(p.mid_lse[(int64_t)row * p.ml_s0 + head] - mx);
        }
      }
      wsum += my_w;
#pragma unroll 4
      for (int i = 0; i < cnt; ++i) {
        const int row = __shfl_sync(0xffffffffu, my_row, i);
        const float w = __shfl_sync(0xffffffffu, my_w, i);
        if (row < 0 || w == 0.f) continue;  // -inf LSE marks an empty partial
        const float4* __restrict__ src =
            reinterpret_cast<const float4*>(p.mid_o + (int64_t)row * p.mo_s0 + (int64_t)head * p.mo_s1);
#pragma unroll
        for (int c = 0; c < MAXC; ++c) {
          const int ch = lane + 32 * c;
          if (ch < chunks) {
            const float4 x = __ldcg(src + ch);
            acc[c].x = fmaf(w, x.x, acc[c].x);
            acc[c].y = fmaf(w, x.y, acc[c].y);
            acc[c].z = fmaf(w, x.z, acc[c].z);
            acc[c].w = fmaf(w, x.w, acc[c].w);
          }
        }
      }
    }
  }
  wsum = warp_sum(wsum);
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  T* __restrict__ dst = reinterpret_cast<T*>(p.o) + (int64_t)req * p.o_s0 + (int64_t)head * p.o_s1;
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int ch = lane + 32 * c;
    if (ch < chunks) {
      dst[4 * ch + 0] = from_float<T>(acc[c].x * inv);
      dst[4 * ch + 1] = from_float<T>(acc[c].y * inv);
      dst[4 * ch + 2] = from_float<T>(acc[c].z * inv);
      dst[4 * ch + 3] = from_float<T>(acc[c].w * inv);
    }
  }
  if (p.o_lse != nullptr && lane == 0)
    p.o_lse[(int64_t)req * p.heads + head] = wsum > 0.f ? mx + logf(wsum) : -INFINITY;
}

}  // namespace ft
