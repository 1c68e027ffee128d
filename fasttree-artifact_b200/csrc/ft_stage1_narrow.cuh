// Stage 1 for tasks with few query rows (leaves and low-fan-out nodes): the
// memory-bound shape.  Tensor cores are used "swapped": the 64-token KV tile is
// the M side of the MMA and the packed query rows (requests x GQA group, at
// most 8*NQ) are the N side,
//
//     S^T[tokens, rows] = K[tokens, d] . Q^T[d, rows]          (m16n8k16, A = K tile)
//     O^T[d, rows]     += V^T[d, tokens] . P^T[tokens, rows]   (A = V tile, transposing ldmatrix)
//
// so no MMA work is spent on padding query rows up to 16 and the per-thread
// softmax / rescale state is a quarter of the row-major formulation.  P^T
// reaches the second MMA's B operand with one movmatrix per 8x8 block.
//
// One CTA (4 warps) per (vnode, kv head); each warp owns 16 of every 64 tokens
// and the four (max, sum, O) partials are merged through shared memory.  K/V
// rows are gathered by row id with 16-byte cp.async copies into the same
// 3-stage, XOR-swizzled ring as the wide kernel (KvPipe).
#pragma once

#include "ft_common.cuh"
#include "ft_stage1_mma.cuh"

namespace ft {

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(v) : "r"(addr));
  return v;
}

template <int D, int NQ>
struct NarrowCfg {
  using M = MmaCfg<D>;
  static constexpr int ROWS = 8 * NQ;               // query rows per pass
  static constexpr int Q_BYTES = 16 * M::ROWB;      // room for 16 rows either way
  static constexpr int IDXB = 512;                  // tokens per row-id block (two blocks in shared memory)
  static constexpr int IDX_BYTES = 2 * IDXB * 4;
  static constexpr int OSTRIDE = D + 4;
  static constexpr int EPI_BYTES = 4 * ROWS * OSTRIDE * 4 + 2 * 4 * ROWS * 4;
  static constexpr int SMEM_BYTES = Q_BYTES + IDX_BYTES + (M::PIPE_BYTES > EPI_BYTES ? M::PIPE_BYTES : EPI_BYTES);
};

template <typename T, int D, int NQ>
__device__ __forceinline__ void narrow_body(const Stage1Params& p, uint8_t* smem, const int vn, const int kvh) {
  using C = MmaCfg<D>;
  using N = NarrowCfg<D, NQ>;
  const uint32_t q_sm = smem_u32(smem);
  const uint32_t idx_sm = q_sm + N::Q_BYTES;
  const uint32_t pipe_sm = idx_sm + N::IDX_BYTES;
  float* epi_o = reinterpret_cast<float*>(smem + N::Q_BYTES + N::IDX_BYTES);
  float* epi_m = epi_o + 4 * N::ROWS * N::OSTRIDE;
  float* epi_l = epi_m + 4 * N::ROWS;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int q_off = p.q_offs[vn], q_len = p.q_lens[vn];
  const int kv_off = p.kv_offs[vn], kv_len = max(p.kv_lens[vn], 0);
  const int G = p.group;
  const int rows = q_len * G;
  if (rows <= 0) return;
  if (tid == 0) FT_TL_MARK(0);
  const float scale2 = p.sm_scale * 1.4426950408889634f;
  const int ntiles = (kv_len + C::TILE - 1) / C::TILE;
  const int ld_c = tid % C::CPR, ld_r = tid / C::CPR;
  const int tok0 = warp * 16;  // this warp's 16 tokens of every tile

  KvPipe<T, D, N::IDXB> pipe(p, kvh, kv_off, kv_len, smem + N::Q_BYTES, idx_sm, pipe_sm);

  for (int row0 = 0; row0 < rows; row0 += N::ROWS) {
    pipe.issue_first_indices();  // the K/V row ids travel while the request ids below are fetched
    // ---- request ids first (independent loads), then the copies
    constexpr int QPASSES = (N::ROWS + C::TPP - 1) / C::TPP;
    int64_t q_src[QPASSES];
#pragma unroll
    for (int ps = 0; ps < QPASSES; ++ps) {
      q_src[ps] = -1;
      const int r = ps * C::TPP + ld_r;
      const int prow = row0 + r;
      if (r < N::ROWS && prow < rows) {
        const int slot = prow / G, gg = prow - slot * G;
        const int64_t part = (int64_t)q_off + slot;
        if (part >= 0 && part < p.num_partial_rows) {
          const int req = p.q_entries[part];
          if (req >= 0 && req < p.batch)
            q_src[ps] = (int64_t)req * p.q_s0 + (int64_t)(kvh * G + gg) * p.q_s1 + ld_c * 8;
          else
            flag_error(FT_DEV_BAD_Q_INDEX);
        } else {
          flag_error(FT_DEV_BAD_ROW_INDEX);
        }
      }
    }
#pragma unroll
    for (int ps = 0; ps < QPASSES; ++ps) {
      const int r = ps * C::TPP + ld_r;
      if (r < N::ROWS) {
        const bool ok = q_src[ps] >= 0;
        cp_async16(q_sm + C::swzq(r, ld_c), reinterpret_cast<const T*>(p.q) + (ok ? q_src[ps] : 0), ok);
      }
    }
    cp_async_commit();
    pipe.wait_indices();  // also lands Q
    if (tid == 0) FT_TL_MARK(1);
    pipe.prologue();

    float o_acc[D / 16][NQ][4];
#pragma unroll
    for (int mb = 0; mb < D / 16; ++mb)
#pragma unroll
      for (int nq = 0; nq < NQ; ++nq) o_acc[mb][nq][0] = o_acc[mb][nq][1] = o_acc[mb][nq][2] = o_acc[mb][nq][3] = 0.f;
    float m_run[NQ][2], l_run[NQ][2];
#pragma unroll
    for (int nq = 0; nq < NQ; ++nq) {
      m_run[nq][0] = m_run[nq][1] = -INFINITY;
      l_run[nq][0] = l_run[nq][1] = 0.f;
    }
    uint32_t qb[NQ][D / 16][2];  // Q^T as the "col" operand: row nq*8+g8, d = 16kk + 2*t4 (+8)

    for (int j = 0; j < ntiles; ++j) {
      pipe.advance(j);
      if (tid == 0 && j < 4) FT_TL_MARK(2 + j);
      if (j == 0) {
#pragma unroll
        for (int nq = 0; nq < NQ; ++nq)
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            qb[nq][kk][0] = lds32(q_sm + C::swzq(nq * 8 + g8, 2 * kk) + 4 * t4);
            qb[nq][kk][1] = lds32(q_sm + C::swzq(nq * 8 + g8, 2 * kk + 1) + 4 * t4);
          }
      }
      const uint32_t k_sm = pipe.k_stage(j), v_sm = pipe.v_stage(j);

      // S^T = K Q^T : two interleaved accumulator chains per row block
      float s[2][NQ][4];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int nq = 0; nq < NQ; ++nq) s[h][nq][0] = s[h][nq][1] = s[h][nq][2] = s[h][nq][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t ka[4];
        ldmatrix_x4(ka, k_sm + C::swz(tok0 + (lane & 7) + 8 * ((lane >> 3) & 1), 2 * kk + (lane >> 4)));
#pragma unroll
        for (int nq = 0; nq < NQ; ++nq) mma16816<T>(s[kk & 1][nq], ka, qb[nq][kk][0], qb[nq][kk][1]);
      }

      const int pos_lo = j * C::TILE + tok0 + g8;  // token of c0,c1; c2,c3 are 8 further
      const bool lo_ok = pos_lo < kv_len, hi_ok = pos_lo + 8 < kv_len;
      uint32_t pb[NQ][2];
      bool rescale = false;
      float corr[NQ][2];
#pragma unroll
      for (int nq = 0; nq < NQ; ++nq) {
        float x0 = (s[0][nq][0] + s[1][nq][0]) * scale2, x1 = (s[0][nq][1] + s[1][nq][1]) * scale2;
        float x2 = (s[0][nq][2] + s[1][nq][2]) * scale2, x3 = (s[0][nq][3] + s[1][nq][3]) * scale2;
        if (!lo_ok) x0 = x1 = -INFINITY;
        if (!hi_ok) x2 = x3 = -INFINITY;
        float ma = fmaxf(x0, x2), mb_ = fmaxf(x1, x3);  // rows 2*t4 and 2*t4+1 over this thread's two tokens
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, o));
          mb_ = fmaxf(mb_, __shfl_xor_sync(0xffffffffu, mb_, o));
        }
        const float na = fmaxf(m_run[nq][0], ma), nb = fmaxf(m_run[nq][1], mb_);
        const float sa = na == -INFINITY ? 0.f : na, sb = nb == -INFINITY ? 0.f : nb;
        corr[nq][0] = fast_exp2(m_run[nq][0] - sa);
        corr[nq][1] = fast_exp2(m_run[nq][1] - sb);
        rescale |= (na != m_run[nq][0]) | (nb != m_run[nq][1]);
        m_run[nq][0] = na;
        m_run[nq][1] = nb;
        const float p0 = fast_exp2(x0 - sa), p1 = fast_exp2(x1 - sb);
        const float p2 = fast_exp2(x2 - sa), p3 = fast_exp2(x3 - sb);
        l_run[nq][0] = l_run[nq][0] * corr[nq][0] + p0 + p2;
        l_run[nq][1] = l_run[nq][1] * corr[nq][1] + p1 + p3;
        // (token g8 | g8+8 ; rows 2t4,2t4+1) -> (row g8 ; tokens 2t4,2t4+1 | +8): the B operand of P^T
        pb[nq][0] = movmatrix_trans(pack2<T>(p0, p1));
        pb[nq][1] = movmatrix_trans(pack2<T>(p2, p3));
      }
      if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int mb = 0; mb < D / 16; ++mb)
#pragma unroll
          for (int nq = 0; nq < NQ; ++nq) {
            o_acc[mb][nq][0] *= corr[nq][0];
            o_acc[mb][nq][1] *= corr[nq][1];
            o_acc[mb][nq][2] *= corr[nq][0];
            o_acc[mb][nq][3] *= corr[nq][1];
          }
      }
      // O^T += V^T P^T
#pragma unroll
      for (int mb = 0; mb < D / 16; ++mb) {
        uint32_t va[4];
        ldmatrix_x4_trans(va, v_sm + C::swz(tok0 + (lane & 7) + 8 * (lane >> 4), 2 * mb + ((lane >> 3) & 1)));
#pragma unroll
        for (int nq = 0; nq < NQ; ++nq) mma16816<T>(o_acc[mb][nq], va, pb[nq][0], pb[nq][1]);
      }
    }
    pipe.drain();  // ring idle: reuse it as the staging area
    if (tid == 0) FT_TL_MARK(6);

    // ---- stage this warp's (max, sum, O^T) partial
#pragma unroll
    for (int nq = 0; nq < NQ; ++nq) {
      float la = l_run[nq][0], lb = l_run[nq][1];
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        la += __shfl_xor_sync(0xffffffffu, la, o);
        lb += __shfl_xor_sync(0xffffffffu, lb, o);
      }
      const int r = nq * 8 + 2 * t4;
      float* dst = epi_o + (warp * N::ROWS + r) * N::OSTRIDE + g8;
#pragma unroll
      for (int mb = 0; mb < D / 16; ++mb) {
        dst[mb * 16] = o_acc[mb][nq][0];
        dst[N::OSTRIDE + mb * 16] = o_acc[mb][nq][1];
        dst[mb * 16 + 8] = o_acc[mb][nq][2];
        dst[N::OSTRIDE + mb * 16 + 8] = o_acc[mb][nq][3];
      }
      if (g8 == 0) {
        epi_m[warp * N::ROWS + r] = m_run[nq][0];
        epi_m[warp * N::ROWS + r + 1] = m_run[nq][1];
        epi_l[warp * N::ROWS + r] = la;
        epi_l[warp * N::ROWS + r + 1] = lb;
      }
    }
    __syncthreads();

    // ---- merge the four warps, normalise, write the partial rows
    {
      const int r = tid >> 3, seg = tid & 7;
      const int prow = row0 + r;
      if (r < N::ROWS && prow < rows) {
        const int slot = prow / G, gg = prow - slot * G;
        const int64_t part = (int64_t)q_off + slot;
        if (part >= 0 && part < p.num_partial_rows) {
          float M = -INFINITY;
#pragma unroll
          for (int w = 0; w < 4; ++w) M = fmaxf(M, epi_m[w * N::ROWS + r]);
          float L = 0.f;
          float4 out[D / 32];
#pragma unroll
          for (int i = 0; i < D / 32; ++i) out[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const float mw = epi_m[w * N::ROWS + r];
            const float f = mw == -INFINITY ? 0.f : fast_exp2(mw - M);
            L = fmaf(epi_l[w * N::ROWS + r], f, L);
            const float4* src = reinterpret_cast<const float4*>(epi_o + (w * N::ROWS + r) * N::OSTRIDE);
#pragma unroll
            for (int i = 0; i < D / 32; ++i) {
              const float4 x = src[seg + 8 * i];
              out[i].x = fmaf(f, x.x, out[i].x);
              out[i].y = fmaf(f, x.y, out[i].y);
              out[i].z = fmaf(f, x.z, out[i].z);
              out[i].w = fmaf(f, x.w, out[i].w);
            }
          }
          const float inv = L > 0.f ? 1.f / L : 0.f;
          const int head = kvh * G + gg;
          float4* dst = reinterpret_cast<float4*>(p.mid_o + part * p.mo_s0 + (int64_t)head * p.mo_s1);
#pragma unroll
          for (int i = 0; i < D / 32; ++i)
            dst[seg + 8 * i] = make_float4(out[i].x * inv, out[i].y * inv, out[i].z * inv, out[i].w * inv);
          if (seg == 0)
            p.mid_lse[part * p.ml_s0 + head] = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
        }
      }
    }
    __syncthreads();
  }
}

// Tasks with at most 8 query rows run the one-block body, the others the
// two-block body (which also loops if a task has more than 16 rows).
template <typename T, int D>
__device__ __forceinline__ void narrow_dispatch(const Stage1Params& p, uint8_t* smem, const int vn, const int kvh) {
  const int rows = p.q_lens[vn] * p.group;
  if (rows <= 8)
    narrow_body<T, D, 1>(p, smem, vn, kvh);
  else
    narrow_body<T, D, 2>(p, smem, vn, kvh);
}

template <typename T, int D>
__global__ void __launch_bounds__(128, 2) stage1_narrow_kernel(Stage1Params p) {
  allow_dependent_launch();
  wait_for_prior_grid();  // nothing of the preceding kernel's is read or overwritten before this
  extern __shared__ __align__(1024) uint8_t smem[];
  int vn, kvh;
  task_of_block(p, blockIdx.x, vn, kvh);
  FT_TL_BEGIN();
  narrow_dispatch<T, D>(p, smem, vn, kvh);
  FT_TL_END(2);
}

}  // namespace ft
