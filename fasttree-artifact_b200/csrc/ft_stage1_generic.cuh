// Stage 1, scalar fp32 kernel: any storage type, any head_dim <= 256.
//
// One CTA per (vnode, kv head), as in the reference launch grid
// (kernel_bench/fasttree.py:448-451).  Each warp owns one packed query row
// (request slot x group member) at a time, lanes span the head dimension, and
// the KV chunk is walked four tokens per step (their row ids, then their K
// rows, are independent loads in flight together) with a warp-shuffle online
// softmax.  It is the correctness path for fp32 inputs and unusual head sizes;
// the 16-bit / head_dim 64,128 cases go to the tensor-core kernels.
#pragma once

#include "ft_common.cuh"

namespace ft {

template <typename T>
__global__ void __launch_bounds__(128) stage1_generic_kernel(Stage1Params p) {
  allow_dependent_launch();
  wait_for_prior_grid();  // nothing of the preceding kernel's is read or overwritten before this
  constexpr int MAXJ = 8;  // 8 x 32 lanes = head_dim up to 256
  constexpr int TB = 4;    // tokens per step (more in flight per step measured slower: register pressure)
  const int vn = blockIdx.x + p.node_offset;
  const int kvh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_off = p.q_offs[vn], q_len = p.q_lens[vn];
  const int kv_off = p.kv_offs[vn], kv_len = p.kv_lens[vn];
  const int G = p.group, D = p.head_dim;
  const int rows = q_len * G;
  const int32_t* ids = kv_ids_base(p, kv_off);
  const int id_lim = kv_ids_limit(p, kv_off, max(kv_len, 0));
  const T* __restrict__ kbase = reinterpret_cast<const T*>(p.k) + (int64_t)kvh * p.k_s1;
  const T* __restrict__ vbase = reinterpret_cast<const T*>(p.v) + (int64_t)kvh * p.v_s1;

  for (int row = warp; row < rows; row += 4) {
    const int slot = row / G, g = row - slot * G;
    const int64_t prow = (int64_t)q_off + slot;
    if (prow < 0 || prow >= p.num_partial_rows) {
      if (lane == 0) flag_error(FT_DEV_BAD_ROW_INDEX);
      continue;
    }
    const int req = p.q_entries[prow];
    if (req < 0 || req >= p.batch) {
      if (lane == 0) flag_error(FT_DEV_BAD_Q_INDEX);
      continue;
    }
    const int head = kvh * G + g;
    const T* __restrict__ qp = reinterpret_cast<const T*>(p.q) + (int64_t)req * p.q_s0 + (int64_t)head * p.q_s1;
    float qreg[MAXJ], acc[MAXJ];
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
      const int d = lane + 32 * j;
      qreg[j] = d < D ? to_float<T>(qp[d]) : 0.f;
      acc[j] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    // the chunk tokens [r_lo, r_hi) this row attends to: the whole chunk unless the plan narrows it
    int r_lo = 0, r_hi = kv_len;
    if (p.q_ranges != nullptr) {
      r_lo = max(p.q_ranges[2 * prow], 0);
      r_hi = min(p.q_ranges[2 * prow + 1], kv_len);
    }
    for (int t0 = r_lo; t0 < r_hi; t0 += TB) {
      int rowid[TB];
      float s[TB];
      bool bad = false;  // flagged once after the loads: an atomic between them would serialise them
#pragma unroll
      for (int u = 0; u < TB; ++u) {
        int64_t idx = -1;
        if (t0 + u < r_hi) {
          if (t0 + u < id_lim) idx = ids[t0 + u];
          if (idx < 0 || idx >= p.kv_rows) {
            bad = true;
            idx = -1;
          }
        }
        rowid[u] = (int)idx;
      }
      if (bad && lane == 0) flag_error(FT_DEV_BAD_KV_INDEX);
#pragma unroll
      for (int u = 0; u < TB; ++u) {
        float part = 0.f;
        if (rowid[u] >= 0) {
          const T* __restrict__ kp = kbase + (int64_t)rowid[u] * p.k_s0;
#pragma unroll
          for (int j = 0; j < MAXJ; ++j) {
            const int d = lane + 32 * j;
            if (d < D) part = fmaf(qreg[j], to_float<T>(kp[d]), part);
          }
        }
        s[u] = part;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int u = 0; u < TB; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
      }
      float m_new = m;
#pragma unroll
      for (int u = 0; u < TB; ++u) {
        s[u] = rowid[u] >= 0 ? s[u] * p.sm_scale : -INFINITY;  // scale after the dot, in fp32 (fasttree.py:376)
        m_new = fmaxf(m_new, s[u]);
      }
      if (m_new == -INFINITY) continue;  // nothing valid yet
      const float corr = expf(m - m_new);
      l *= corr;
#pragma unroll
      for (int j = 0; j < MAXJ; ++j) acc[j] *= corr;
#pragma unroll
      for (int u = 0; u < TB; ++u) {
        if (rowid[u] < 0) continue;
        const float pr = expf(s[u] - m_new);
        l += pr;
        // the reference casts the probabilities to V's type before P*V (fasttree.py:391)
        const float pv = to_float<T>(from_float<T>(pr));
        const T* __restrict__ vp = vbase + (int64_t)rowid[u] * p.v_s0;
#pragma unroll
        for (int j = 0; j < MAXJ; ++j) {
          const int d = lane + 32 * j;
          if (d < D) acc[j] = fmaf(pv, to_float<T>(vp[d]), acc[j]);
        }
      }
      m = m_new;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    float* __restrict__ op = p.mid_o + prow * p.mo_s0 + (int64_t)head * p.mo_s1;
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
      const int d = lane + 32 * j;
      if (d < D) op[d] = acc[j] * inv;
    }
    if (lane == 0) p.mid_lse[prow * p.ml_s0 + head] = l > 0.f ? logf(l) + m : -INFINITY;
  }
}

}  // namespace ft
