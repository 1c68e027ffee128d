// Stage 1 for fp32 storage (head_dim 64 or 128): exact fp32 arithmetic on the
// CUDA cores, tiled through shared memory.
//
// One CTA (8 warps) per (vnode, kv head, block of 16 packed query rows).  The KV
// chunk is walked 32 tokens at a time: the tile's K and V rows are gathered by
// row id with 16-byte loads, one tile ahead of the arithmetic (the loads of tile
// t+1 are in flight, in registers, while tile t is computed from shared memory).
//   S[16 x 32]   lane = token, warp w owns rows w and w+8: 2 dot products of length
//                head_dim per thread, Q broadcast from shared memory (two warps per
//                scheduler: the arithmetic of a tile is one dependent chain per warp,
//                and with four warps of four rows a tile took twice as long)
//   softmax      a row's 32 scores sit in the 32 lanes of one warp: shuffles
//   O[16 x D]    thread owns columns lane, lane+32, ... of its warp's 2 rows; the
//                probabilities are broadcast by shuffle, V read conflict-free
// Same conventions as the other stage-1 kernels (kernel_bench/fasttree.py:360-413):
// scores scaled after the dot product, normalised partial output, lse = log(sum) + max;
// optional per-row token ranges; bad indices are skipped and flagged.
#pragma once

#include "ft_common.cuh"

namespace ft {

template <int D>
struct F32Cfg {
  static constexpr int ROWS = 16, TILE = 32, THREADS = 256;
  static constexpr int WARPS = THREADS / 32, RPW = ROWS / WARPS;  // rows per warp
  static constexpr int KSTRIDE = D + 1;              // floats between K rows: lane = token reads are conflict-free
  static constexpr int Q_FLOATS = ROWS * D, K_FLOATS = TILE * KSTRIDE, V_FLOATS = TILE * D;
  static constexpr int K_OFF = ((Q_FLOATS + 3) / 4) * 4, V_OFF = ((K_OFF + K_FLOATS + 3) / 4) * 4;
  static constexpr int SMEM_BYTES = (V_OFF + V_FLOATS) * 4;
  static constexpr int C4 = D / 4;                   // float4 chunks per row
  static constexpr int LOADS = TILE * C4 / THREADS;  // float4 loads per thread per operand per tile
};

template <int D>
__global__ void __launch_bounds__(256) stage1_f32_kernel(Stage1Params p) {
  using C = F32Cfg<D>;
  allow_dependent_launch();
  wait_for_prior_grid();  // nothing of the preceding kernel's is read or overwritten before this
  extern __shared__ __align__(16) float smem_f32[];
  float* q_s = smem_f32;
  float* k_s = smem_f32 + C::K_OFF;
  float* v_s = smem_f32 + C::V_OFF;
  const int vn = blockIdx.x + p.node_offset, kvh = blockIdx.y, row0 = blockIdx.z * C::ROWS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q_off = p.q_offs[vn], q_len = p.q_lens[vn];
  const int kv_off = p.kv_offs[vn], kv_len = max(p.kv_lens[vn], 0);
  const int G = p.group;
  const int rows = min(q_len * G - row0, C::ROWS);
  if (rows <= 0) return;
  // the grid's row blocks come from the caller's request tile: a vnode with more rows than that is a plan error
  if (blockIdx.z == gridDim.z - 1 && q_len * G - row0 > C::ROWS && threadIdx.x == 0) flag_error(FT_DEV_BAD_ROW_INDEX);
  const int32_t* ids = kv_ids_base(p, kv_off);
  const int id_lim = kv_ids_limit(p, kv_off, kv_len);
  const float* kbase = reinterpret_cast<const float*>(p.k) + (int64_t)kvh * p.k_s1;
  const float* vbase = reinterpret_cast<const float*>(p.v) + (int64_t)kvh * p.v_s1;

  // ---- Q rows of this block -> shared memory (zeros for rows past the end or with a bad index)
  for (int i = tid; i < C::ROWS * C::C4; i += C::THREADS) {
    const int r = i / C::C4, c4 = i - r * C::C4;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < rows) {
      const int prow = row0 + r, slot = prow / G, gg = prow - slot * G;
      const int64_t part = (int64_t)q_off + slot;
      if (part >= 0 && part < p.num_partial_rows) {
        const int req = p.q_entries[part];
        if (req >= 0 && req < p.batch)
          x = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.q) + (int64_t)req * p.q_s0 +
                                               (int64_t)(kvh * G + gg) * p.q_s1 + 4 * c4);
        else if (c4 == 0)
          flag_error(FT_DEV_BAD_Q_INDEX);
      } else if (c4 == 0) {
        flag_error(FT_DEV_BAD_ROW_INDEX);
      }
    }
    *reinterpret_cast<float4*>(q_s + r * D + 4 * c4) = x;
  }

  // per-thread state: rows warp + WARPS * i
  constexpr int RPW = C::RPW, NW = C::WARPS;
  float m_run[RPW], l_run[RPW], acc[RPW][D / 32];
  int r_lo[RPW], r_hi[RPW];
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    m_run[i] = -INFINITY;
    l_run[i] = 0.f;
#pragma unroll
    for (int j = 0; j < D / 32; ++j) acc[i][j] = 0.f;
    r_lo[i] = 0;
    r_hi[i] = kv_len;
    const int r = warp + NW * i;
    if (p.q_ranges != nullptr && r < rows) {
      const int64_t part = (int64_t)q_off + (row0 + r) / G;
      if (part >= 0 && part < p.num_partial_rows) {
        r_lo[i] = max(p.q_ranges[2 * part], 0);
        r_hi[i] = min(p.q_ranges[2 * part + 1], kv_len);
      }
    }
  }

  const int ntiles = (kv_len + C::TILE - 1) / C::TILE;
  float4 kreg[C::LOADS], vreg[C::LOADS];
  // the tile's rows -> registers (zeros for padding and bad row ids)
  auto fetch = [&](int t) {
    bool bad = false;
#pragma unroll
    for (int u = 0; u < C::LOADS; ++u) {
      const int i = u * C::THREADS + tid, tok = i / C::C4, c4 = i - tok * C::C4;
      const int pos = t * C::TILE + tok;
      int64_t row = -1;
      if (pos < kv_len) {
        if (pos < id_lim) row = ids[pos];
        if (row < 0 || row >= p.kv_rows) {
          bad = true;
          row = -1;
        }
      }
      if (row >= 0) {
        kreg[u] = __ldg(reinterpret_cast<const float4*>(kbase + row * p.k_s0) + c4);
        vreg[u] = __ldg(reinterpret_cast<const float4*>(vbase + row * p.v_s0) + c4);
      } else {
        kreg[u] = vreg[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    if (bad) flag_error(FT_DEV_BAD_KV_INDEX);
  };
  auto stash = [&]() {
#pragma unroll
    for (int u = 0; u < C::LOADS; ++u) {
      const int i = u * C::THREADS + tid, tok = i / C::C4, c4 = i - tok * C::C4;
      float* kd = k_s + tok * C::KSTRIDE + 4 * c4;
      kd[0] = kreg[u].x;
      kd[1] = kreg[u].y;
      kd[2] = kreg[u].z;
      kd[3] = kreg[u].w;
      *reinterpret_cast<float4*>(v_s + tok * D + 4 * c4) = vreg[u];
    }
  };

  if (ntiles > 0) fetch(0);
  for (int t = 0; t < ntiles; ++t) {
    __syncthreads();  // the previous tile has been consumed (and, at t = 0, Q is in place)
    stash();
    __syncthreads();
    if (t + 1 < ntiles) fetch(t + 1);  // in flight during the arithmetic below

    // ---- S = Q K^T for this thread's rows and its token
    float s[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) s[i] = 0.f;
    const float* kr = k_s + lane * C::KSTRIDE;
#pragma unroll 4
    for (int d4 = 0; d4 < C::C4; ++d4) {
      const float k0 = kr[4 * d4], k1 = kr[4 * d4 + 1], k2 = kr[4 * d4 + 2], k3 = kr[4 * d4 + 3];
#pragma unroll
      for (int i = 0; i < RPW; ++i) {
        const float4 qv = *reinterpret_cast<const float4*>(q_s + (warp + NW * i) * D + 4 * d4);
        s[i] = fmaf(qv.x, k0, s[i]);
        s[i] = fmaf(qv.y, k1, s[i]);
        s[i] = fmaf(qv.z, k2, s[i]);
        s[i] = fmaf(qv.w, k3, s[i]);
      }
    }
    // ---- online softmax per row (32 tokens = 32 lanes)
    const int pos = t * C::TILE + lane;
    float pr[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      const bool seen = pos >= r_lo[i] && pos < r_hi[i];
      const float x = seen ? s[i] * p.sm_scale : -INFINITY;
      const float m_new = fmaxf(m_run[i], warp_max(x));
      if (m_new == -INFINITY) {  // nothing valid for this row yet
        pr[i] = 0.f;
        continue;
      }
      const float corr = expf(m_run[i] - m_new);  // 0 while m_run is -inf
      pr[i] = seen ? expf(x - m_new) : 0.f;
      l_run[i] = l_run[i] * corr + warp_sum(pr[i]);
#pragma unroll
      for (int j = 0; j < D / 32; ++j) acc[i][j] *= corr;
      m_run[i] = m_new;
    }
    // ---- O += P V
#pragma unroll 4
    for (int tok = 0; tok < C::TILE; ++tok) {
      float vv[D / 32];
#pragma unroll
      for (int j = 0; j < D / 32; ++j) vv[j] = v_s[tok * D + lane + 32 * j];
#pragma unroll
      for (int i = 0; i < RPW; ++i) {
        const float w = __shfl_sync(0xffffffffu, pr[i], tok);
#pragma unroll
        for (int j = 0; j < D / 32; ++j) acc[i][j] = fmaf(w, vv[j], acc[i][j]);
      }
    }
  }

  // ---- normalise and write the partial rows
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    const int r = warp + NW * i;
    if (r >= rows) continue;
    const int prow = row0 + r, slot = prow / G, gg = prow - slot * G;
    const int64_t part = (int64_t)q_off + slot;
    if (part < 0 || part >= p.num_partial_rows) continue;
    const int head = kvh * G + gg;
    const float inv = l_run[i] > 0.f ? 1.f / l_run[i] : 0.f;
    float* op = p.mid_o + part * p.mo_s0 + (int64_t)head * p.mo_s1;
#pragma unroll
    for (int j = 0; j < D / 32; ++j) op[lane + 32 * j] = acc[i][j] * inv;
    if (lane == 0) p.mid_lse[part * p.ml_s0 + head] = l_run[i] > 0.f ? logf(l_run[i]) + m_run[i] : -INFINITY;
  }
}

}  // namespace ft
