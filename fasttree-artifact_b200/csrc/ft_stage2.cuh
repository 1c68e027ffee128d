// Stage 2: per-(request, query head) log-sum-exp merge of the request's partial
// rows (kernel_bench/fasttree.py:482-546).
//
// One warp per (request, head); lanes span head_dim in float4 chunks, so a
// partial row of head_dim 128 is one 512-byte coalesced warp load.  The
// weights exp(lse_i - max) are computed lane-parallel (32 partial rows at a
// time, running maximum across batches) and broadcast by shuffle, which keeps
// the dependent chain per partial to one FMA.  Memory-bound on the partial buffers; those are written by stage
// 1 just before and are normally still in L2.
#pragma once

#include "ft_common.cuh"

namespace ft {

// MAXC: float4 chunks per lane (1: head_dim <= 128, 2: head_dim <= 256).  RB: partial rows in flight per lane.  A
// request's merge is a chain of L2 round trips, one per batch of RB rows.  A launch that fits one round of CTAs is
// bound by that chain (a head-sharded plan - one KV head per GPU, 128-token chunks - hands a request 30 and more
// partial rows), so it runs with RB = 8 at six CTAs per SM - RB = 16 at four when it does not even fill two CTAs per
// SM, which is the sharded case; a launch of several rounds (cfg4: 65 536 request-head pairs) is bound by how many
// warps the SM holds and runs with RB = 4 at nine (head_dim <= 128).
template <typename T, int MAXC, int RB>
__global__ void __launch_bounds__(128, RB >= 16 ? 4 : ((MAXC == 1 && RB == 4) ? 9 : 6)) stage2_merge_kernel(Stage2Params p) {
  allow_dependent_launch();  // a following stage-1 launch may set itself up under this kernel's tail
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t pair = (int64_t)blockIdx.x * 4 + warp;
  if (pair >= (int64_t)p.batch * p.heads) return;
  const int req = (int)(pair / p.heads);
  const int head = (int)(pair - (int64_t)req * p.heads);
  const int off = p.r2v_offs[req];
  const int n = p.r2v_lens[req];
  const int chunks = p.head_dim >> 2;
  int batch_rows = lane < n ? p.r2v_entries[off + lane] : -1;  // plan data: readable before stage 1 is done
  wait_for_prior_grid();                                       // the partial buffers are complete from here on

  // One pass with a running maximum (as in the online softmax): per batch of up to 32 partial rows the lanes
  // fetch their row's LSE while the first rows of the batch are already being loaded - the row addresses depend
  // on the plan only - so a request with few partials costs one round trip to the partial buffers, not two.
  float mx = -INFINITY;
  float4 acc[MAXC];
#pragma unroll
  for (int c = 0; c < MAXC; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
  float wsum = 0.f;
  for (int base = 0; base < n; base += 32) {
    const int cnt = min(32, n - base);
    int my_row = -1;
    const int row = batch_rows;
    batch_rows = base + 32 + lane < n ? p.r2v_entries[off + base + 32 + lane] : -1;  // the next batch's ids travel under this batch's rows
    if (lane < cnt) {
      if (row >= 0 && row < p.num_partial_rows)
        my_row = row;
      else
        flag_error(FT_DEV_BAD_ROW_INDEX);
    }
    const float my_lse = my_row >= 0 ? __ldcg(p.mid_lse + (int64_t)my_row * p.ml_s0 + head) : -INFINITY;
    float my_w = 0.f;
    for (int i0 = 0; i0 < cnt; i0 += RB) {
      float4 x[RB][MAXC];
      int rows[RB];
#pragma unroll
      for (int r = 0; r < RB; ++r) {
        rows[r] = i0 + r < cnt ? __shfl_sync(0xffffffffu, my_row, (i0 + r) & 31) : -1;
        const float4* __restrict__ src =
            reinterpret_cast<const float4*>(p.mid_o + (int64_t)(rows[r] >= 0 ? rows[r] : 0) * p.mo_s0 + (int64_t)head * p.mo_s1);
#pragma unroll
        for (int c = 0; c < MAXC; ++c) {
          const int ch = lane + 32 * c;
          x[r][c] = rows[r] >= 0 && ch < chunks ? __ldcg(src + ch) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      if (i0 == 0) {  // the batch's LSEs are needed only now: rescale what has been summed so far to the new maximum
        const float bm = warp_max(my_lse);
        const float new_mx = fmaxf(mx, bm);
        const float corr = new_mx == -INFINITY ? 1.f : expf(mx - new_mx);  // 0 for the first batch
        wsum *= corr;
#pragma unroll
        for (int c = 0; c < MAXC; ++c) {
          acc[c].x *= corr;
          acc[c].y *= corr;
          acc[c].z *= corr;
          acc[c].w *= corr;
        }
        mx = new_mx;
        my_w = my_lse > -INFINITY ? expf(my_lse - mx) : 0.f;  // -inf LSE marks an empty partial
        wsum += my_w;
      }
#pragma unroll
      for (int r = 0; r < RB; ++r) {
        const float w = __shfl_sync(0xffffffffu, my_w, (i0 + r) & 31);
        if (rows[r] < 0 || w == 0.f) continue;
#pragma unroll
        for (int c = 0; c < MAXC; ++c) {
          acc[c].x = fmaf(w, x[r][c].x, acc[c].x);
          acc[c].y = fmaf(w, x[r][c].y, acc[c].y);
          acc[c].z = fmaf(w, x[r][c].z, acc[c].z);
          acc[c].w = fmaf(w, x[r][c].w, acc[c].w);
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
      alignas(16) T out[4] = {from_float<T>(acc[c].x * inv), from_float<T>(acc[c].y * inv), from_float<T>(acc[c].z * inv),
                  from_float<T>(acc[c].w * inv)};
      if (p.o_vec) {  // four elements in one store when the output rows allow it
        if constexpr (sizeof(T) == 2)
          *reinterpret_cast<uint2*>(dst + 4 * ch) = *reinterpret_cast<const uint2*>(out);
        else
          *reinterpret_cast<float4*>(dst + 4 * ch) = *reinterpret_cast<const float4*>(out);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) dst[4 * ch + e] = out[e];
      }
    }
  }
  if (p.o_lse != nullptr && lane == 0)
    p.o_lse[(int64_t)req * p.heads + head] = wsum > 0.f ? mx + logf(wsum) : -INFINITY;
}

}  // namespace ft
