// Stage 1 for few-row tasks as PERSISTENT workers: each CTA walks a list of
// (vnode, kv head) tasks and keeps ONE software pipeline running across task
// boundaries, so the start-up latency of a task (metadata -> row ids -> first
// K/V tile) is hidden behind the tiles of the tasks before it.  This
// is what short leaves need: a 64-token leaf is a single tile, and with one
// CTA per task its whole life is start-up latency.
//
// The per-tile arithmetic is that of the swapped-operand kernel
// (ft_stage1_narrow.cuh): S^T = K.Q^T and O^T += V^T.P^T with m16n8k16, four
// warps splitting every 64-token tile by tokens, merged through shared memory at
// the end of the task.
//
// Task list of worker w out of W: tasks w, w + W, w + 2W, ... of the launch's
// few-row tasks ((vnode, kv head) pairs in plan order, kv head fastest, so the
// planner's longest-first order is dealt round-robin and the workers that run
// side by side read adjacent slices of the same pool rows).  The assignment is
// static: all workers of a launch start together, and a shared counter would
// put an atomic's round trip on every worker's start-up path.
//
// Pipeline: every loop iteration is one slot.  A slot is a (task, tile) pair or
// a bubble, decided when it enters; the stages sit at fixed distances,
//   iteration s      row ids of the tile (and the task's request ids) -> rings
//   iteration s + 4  are the 64 row ids consecutive?  (one warp; the answer is
//                    read by everyone one iteration later)
//   iteration s + 5  K/V rows of the tile -> 3-stage ring: four tiled TMA copies
//                    (128-byte swizzle, no multicast) for a consecutive tile,
//                    16-byte cp.async copies row by row otherwise; the task's Q
//                    rows with cp.async
//   iteration s + 7  MMA + online softmax; at a task's last tile the epilogue,
//                    staged through the ring stage just freed
// Row ids, request ids and task metadata travel in cp.async groups, one per
// iteration with wait_group 3 at the top, so such a copy issued in iteration i
// is complete in iteration i + 4 whatever its latency.  The issue work of an
// iteration is spread over the warps (warp 0 task metadata, warp 1 request ids
// and the consecutive-ids test, warps 2-3 row ids, one lane of warp 3 the TMA
// copies), each reading only the metadata it needs.
// A K/V tile and the task's Q rows signal the mbarrier of the tile's ring stage
// (transaction bytes for TMA, one arrival per thread when its cp.async copies
// have landed), which the consumer waits on - bounded.  Task metadata enters a
// 16-entry ring at least four iterations before the task's first slot.  No stage
// waits on an earlier one: when an input is not there yet the slot is a bubble.
#pragma once

#include "ft_async.cuh"
#include "ft_common.cuh"
#include "ft_stage1_mma.cuh"
#include "ft_stage1_narrow.cuh"

namespace ft {

template <int D>
struct StreamCfg {
  using M = MmaCfg<D>;
  static constexpr int QBUFS = 3;
  static constexpr int Q_BYTES = QBUFS * 16 * M::ROWB;
  static constexpr int IDS_SLOTS = 8;
  static constexpr int IDS_OFF = Q_BYTES;
  static constexpr int IDS_BYTES = IDS_SLOTS * 64 * 4;
  static constexpr int QID_SLOTS = 8;
  static constexpr int QID_OFF = IDS_OFF + IDS_BYTES;
  static constexpr int QID_BYTES = QID_SLOTS * 16 * 4;
  static constexpr int TASK_RING = 16;
  static constexpr int META_OFF = QID_OFF + QID_BYTES;  // 8 ints per task: q_off, q_len, kv_off, kv_len, kv head
  static constexpr int META_BYTES = TASK_RING * 32;
  static constexpr int ML_OFF = META_OFF + META_BYTES;  // staged (max, sum) of the four warps
  static constexpr int ML_BYTES = 2 * 4 * 16 * 4;
  static constexpr int DENSE_OFF = ML_OFF + ML_BYTES;   // per ids-ring slot: first row of a consecutive tile, or -1
  static constexpr int BAR_OFF = DENSE_OFF + IDS_SLOTS * 4;  // one mbarrier per K/V ring stage
  static constexpr int PIPE_OFF = (BAR_OFF + 3 * 8 + 1023) / 1024 * 1024;  // swizzled tiles sit on 1024-byte boundaries
  static constexpr int WAIT_LIMIT = 1 << 16;
  static constexpr int SMEM_BYTES = PIPE_OFF + M::PIPE_BYTES;
};
static_assert(StreamCfg<128>::SMEM_BYTES <= 115712, "two CTAs must fit in one SM's shared memory");
static_assert(MmaCfg<128>::STAGES == 3, "one mbarrier per ring stage");

// one 64-token tile for one warp (its 16 tokens); NQ = 8-row blocks of the task (1 or 2)
template <typename T, int D, int NQ>
__device__ __forceinline__ void stream_tile(uint32_t k_sm, uint32_t v_sm, int tok0, int pos0, int kv_len, float scale2,
                                            const uint32_t (&qb)[2][D / 16][2], float (&o_acc)[D / 16][2][4],
                                            float (&m_run)[2][2], float (&l_run)[2][2], int lane) {
  using C = MmaCfg<D>;
  const int g8 = lane >> 2;
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
  const int pos_lo = pos0 + tok0 + g8;  // token of c0,c1; c2,c3 are 8 further
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
    float ma = fmaxf(x0, x2), mb_ = fmaxf(x1, x3);
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
#pragma unroll
  for (int mb = 0; mb < D / 16; ++mb) {
    uint32_t va[4];
    ldmatrix_x4_trans(va, v_sm + C::swz(tok0 + (lane & 7) + 8 * (lane >> 4), 2 * mb + ((lane >> 3) & 1)));
#pragma unroll
    for (int nq = 0; nq < NQ; ++nq) mma16816<T>(o_acc[mb][nq], va, pb[nq][0], pb[nq][1]);
  }
}

// Tasks are numbered first_task .. first_task + ntasks - 1 in the launch's (vnode, kv head) order; this CTA is
// worker `worker` of `nworkers`.
template <typename T, int D>
__device__ __forceinline__ void stream_worker(const TcParams& tp, uint8_t* smem, const int first_task,
                                              const int ntasks, const int worker, const int nworkers) {
  using C = MmaCfg<D>;
  using S = StreamCfg<D>;
  const Stage1Params& p = tp.p;
  const uint32_t sm = smem_u32(smem);
  const uint32_t bars = sm + S::BAR_OFF;
  int* dense_box = reinterpret_cast<int*>(smem + S::DENSE_OFF);
  if ((sm & 1023u) != 0u) {  // the swizzled tile layout needs a 1024-byte aligned window
    if (threadIdx.x == 0) flag_error(FT_DEV_WAIT_TIMEOUT);
    return;
  }
  if (threadIdx.x == 0) {
    for (int b = 0; b < C::STAGES; ++b) mbar_init(bars + 8 * b, 128);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    if (tp.has_tma) {
      asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tp.k_map)) : "memory");
      asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tp.v_map)) : "memory");
    }
  }
  __syncthreads();
  const uint32_t ids_sm = sm + S::IDS_OFF, qid_sm = sm + S::QID_OFF, meta_sm = sm + S::META_OFF, pipe_sm = sm + S::PIPE_OFF;
  const int* ids_ptr = reinterpret_cast<const int*>(smem + S::IDS_OFF);
  const int* qid_ptr = reinterpret_cast<const int*>(smem + S::QID_OFF);
  int* meta_ptr = reinterpret_cast<int*>(smem + S::META_OFF);
  float* epi_m = reinterpret_cast<float*>(smem + S::ML_OFF);
  float* epi_l = epi_m + 4 * 16;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int ld_c = tid % C::CPR, ld_r = tid / C::CPR;
  const int G = p.group, H = p.num_kv_heads;
  const float scale2 = p.sm_scale * 1.4426950408889634f;
  const uint32_t row_lim = (uint32_t)(p.kv_rows < 0x7fffffffLL ? p.kv_rows : 0x7fffffffLL);
  const int tok0 = warp * 16;

  // readable row ids of a task (a table that ends early is a plan error: flagged, the tokens become padding)
  auto id_limit = [&](int kv_off, int kv_len) {
    return kv_ids_limit(p, kv_off, kv_len);
  };
  // row ids of tile `t` of the task in metadata slot `m` -> ids ring slot `rs`; at t == 0 also the request ids
  auto issue_ids = [&](int m, int t, int rs, int qs) {
    if (warp >= 2) {  // warps 2-3: the tile's 64 row ids
      const int i = tid - 64;
      const int kv_off = meta_ptr[m * 8 + 2], kv_len = max(meta_ptr[m * 8 + 3], 0);
      const int lim = id_limit(kv_off, kv_len);
      const int pos = t * C::TILE + i;
      if (pos < lim) cp_async4(ids_sm + (rs * C::TILE + i) * 4, kv_ids_base(p, kv_off) + pos);
      if (i == 0 && t == 0 && lim < kv_len) flag_error(FT_DEV_BAD_KV_INDEX);
    } else if (warp == 1 && t == 0) {  // warp 1: request ids of the task's (at most 16) slots
      const int q_off = meta_ptr[m * 8 + 0], q_len = meta_ptr[m * 8 + 1];
      if (lane < min(q_len, 16)) {
        const int64_t part = (int64_t)q_off + lane;
        if (part >= 0 && part < p.num_partial_rows)
          cp_async4(qid_sm + (qs * 16 + lane) * 4, p.q_entries + part);
        else
          flag_error(FT_DEV_BAD_ROW_INDEX);
      }
    }
  };
  // K/V rows of the tile -> ring stage `st`; at t == 0 also the task's query rows -> Q buffer `qbuf`
  auto issue_kv = [&](int m, int t, int rs, int qs, int st, int qbuf) {
    const uint32_t k_sm = pipe_sm + st * 2 * C::STAGE_BYTES, v_sm = k_sm + C::STAGE_BYTES;
    const uint32_t full = bars + 8 * st;
    const int first_row = dense_box[rs];
    if (first_row >= 0) {  // 64 consecutive rows: the copy engine writes the tile, no load instructions
      if (tid == 96) {
        // The stage was last touched with ordinary loads and stores (tile reads, epilogue staging), all of them
        // before a CTA barrier of an earlier iteration, i.e. complete.  No proxy fence here: it would also wait
        // for this thread's copies in flight (the row ids just issued) - a full memory round trip per iteration.
        const int kvh = meta_ptr[m * 8 + 4];
        mbar_expect_tx(full, 2 * C::STAGE_BYTES);
#pragma unroll
        for (int h = 0; h < D / 64; ++h) {
          tma_load_3d(k_sm + h * C::BLOCK_BYTES, &tp.k_map, 64 * h, kvh, first_row, full);
          tma_load_3d(v_sm + h * C::BLOCK_BYTES, &tp.v_map, 64 * h, kvh, first_row, full);
        }
      }
    } else {
      const int kv_off = meta_ptr[m * 8 + 2], kv_len = max(meta_ptr[m * 8 + 3], 0);
      const int kvh = meta_ptr[m * 8 + 4];
      const int lim = id_limit(kv_off, kv_len);
      const T* kbase = reinterpret_cast<const T*>(p.k) + (int64_t)kvh * p.k_s1 + ld_c * 8;
      const T* vbase = reinterpret_cast<const T*>(p.v) + (int64_t)kvh * p.v_s1 + ld_c * 8;
      const int* ring = ids_ptr + rs * C::TILE + ld_r;
      const int pos0 = t * C::TILE + ld_r;
      // Only the 16-token blocks that hold tokens of the chunk are filled (zeros after the last token): a warp
      // whose block lies past the end of the chunk skips the tile altogether, so nothing reads the other rows.
      const int fill = min(C::TILE, (max(kv_len - t * C::TILE, 0) + 15) & ~15);
      uint32_t row[C::PASSES];
#pragma unroll
      for (int ps = 0; ps < C::PASSES; ++ps)
        row[ps] = pos0 + ps * C::TPP < lim ? (uint32_t)ring[ps * C::TPP] : 0xffffffffu;
      bool bad = false;
#pragma unroll
      for (int ps = 0; ps < C::PASSES; ++ps) {
        const int r = ps * C::TPP + ld_r;
        if (r < fill) {
          const bool ok = row[ps] < row_lim;
          bad |= !ok && pos0 + ps * C::TPP < lim;
          const int64_t off = (int64_t)(ok ? row[ps] : 0u);
          cp_async16(k_sm + C::swz(r, ld_c), kbase + off * p.k_s0, ok);
          cp_async16(v_sm + C::swz(r, ld_c), vbase + off * p.v_s0, ok);
        }
      }
      if (bad) flag_error(FT_DEV_BAD_KV_INDEX);
    }
    if (t == 0) {
      const int q_off = meta_ptr[m * 8 + 0], q_len = meta_ptr[m * 8 + 1];
      const int kvh = meta_ptr[m * 8 + 4];
      const int rows = min(q_len * G, 16);
      if (tid == 0 && q_len * G > 16) flag_error(FT_DEV_BAD_ROW_INDEX);  // not a few-row task: rows beyond 16 are dropped
      const uint32_t q_sm = sm + qbuf * 16 * C::ROWB;
      constexpr int QPASSES = (16 + C::TPP - 1) / C::TPP;
#pragma unroll
      for (int ps = 0; ps < QPASSES; ++ps) {
        const int r = ps * C::TPP + ld_r;
        if (r < 16) {
          int64_t src = -1;
          if (r < rows) {
            const int slot = r / G, gg = r - slot * G;
            const int req = qid_ptr[qs * 16 + slot];
            const int64_t part = (int64_t)q_off + slot;
            if (part >= 0 && part < p.num_partial_rows) {
              if (req >= 0 && req < p.batch)
                src = (int64_t)req * p.q_s0 + (int64_t)(kvh * G + gg) * p.q_s1 + ld_c * 8;
              else
                flag_error(FT_DEV_BAD_Q_INDEX);
            }
          }
          cp_async16(q_sm + C::swzq(r, ld_c), reinterpret_cast<const T*>(p.q) + (src >= 0 ? src : 0), src >= 0);
        }
      }
    }
    // one arrival per thread: at once when this thread copied nothing for the slot (a TMA tile that is not the
    // task's first: the transaction bytes alone gate the barrier), else once all its copies so far (gathered rows,
    // Q rows) have landed
    if (first_row >= 0 && t != 0)
      mbar_arrive(full);
    else
      mbar_arrive_on_cp_async(full);
  };

  // ---- pipeline state, identical in every thread
  int next_task = worker;  // next task of this worker's list whose metadata copy is still to issue
  int meta_issued = 0, meta_1 = 0, meta_2 = 0, meta_3 = 0, meta_4 = 0;  // tasks whose metadata copy was issued by now / 1..4 iterations ago
  int tasks_done = 0;
  uint32_t stage_phase = 0;  // bit b: phase of ring stage b's mbarrier that its next consumer waits for
  int front_task = -1, front_tile = 0, front_ntiles = 0;
  int dt0 = -1, dt1 = -1, dt2 = -1, dt3 = -1, dt4 = -1, dt5 = -1, dt6 = -1, dt7 = -1;  // task (sequence number) of the slot that entered k iterations ago
  int dl0 = 0, dl1 = 0, dl2 = 0, dl3 = 0, dl4 = 0, dl5 = 0, dl6 = 0, dl7 = 0;              // its tile

  float o_acc[D / 16][2][4];
  float m_run[2][2], l_run[2][2];
  uint32_t qb[2][D / 16][2];
  int c_rows = 0, c_qoff = 0, c_kvlen = 0, c_kvh = 0, c_tiles = 1;

#ifdef FT_TIMELINE
  unsigned long long tl_first = 0;
  int tl_bubbles = 0;
  long long tl_c0 = 0, tl_sum_top = 0, tl_sum_issue = 0, tl_sum_wait = 0, tl_sum_tile = 0, tl_sum_epi = 0;
  int tl_iters = 0, tl_tiles = 0;
#endif
  cp_async_commit();
  for (unsigned int it = 8;; ++it) {
#ifdef FT_TIMELINE
    tl_c0 = clock64();
#endif
    cp_async_wait<3>();
    __syncthreads();
#ifdef FT_TIMELINE
    { const long long c = clock64(); tl_sum_top += c - tl_c0; tl_c0 = c; ++tl_iters; }
#endif

    // ---- metadata of up to two more tasks -> task ring
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (next_task < ntasks && meta_issued - tasks_done < S::TASK_RING) {
        const int j = tid - 8 * u;
        if (j >= 0 && j < 5) {  // warp 0, five lanes per task
          const int b = first_task + next_task;
          const int vn = p.node_offset + b / H;
          const int m = meta_issued % S::TASK_RING;
          if (j < 4) {
            const int32_t* tab = j == 0 ? p.q_offs : j == 1 ? p.q_lens : j == 2 ? p.kv_offs : p.kv_lens;
            cp_async4(meta_sm + m * 32 + j * 4, tab + vn);
          } else {
            meta_ptr[m * 8 + 4] = b - (b / H) * H;
          }
        }
        next_task += nworkers;
        ++meta_issued;
      }
    }

    // ---- the slot entering the pipeline: next tile of the front task, else the next task whose metadata has landed
    dt7 = dt6, dt6 = dt5, dt5 = dt4, dt4 = dt3, dt3 = dt2, dt2 = dt1, dt1 = dt0;
    dl7 = dl6, dl6 = dl5, dl5 = dl4, dl4 = dl3, dl3 = dl2, dl2 = dl1, dl1 = dl0;
    if (front_tile + 1 < front_ntiles) {
      ++front_tile;
      dt0 = front_task;
      dl0 = front_tile;
    } else if (front_task + 1 < meta_4) {
      ++front_task;
      front_tile = 0;
      const int kv_len = max(meta_ptr[(front_task % S::TASK_RING) * 8 + 3], 0);
      front_ntiles = max(1, (kv_len + C::TILE - 1) / C::TILE);  // an empty chunk still gets one (fully masked) tile
      dt0 = front_task;
      dl0 = 0;
    } else {
      dt0 = -1;
    }

    if (dt0 >= 0) issue_ids(dt0 % S::TASK_RING, dl0, it % S::IDS_SLOTS, dt0 % S::QID_SLOTS);
    if (dt4 >= 0 && warp == 1) {  // the slot's row ids have landed: is it a full tile of consecutive rows?
      const int m = dt4 % S::TASK_RING, rs = (it - 4) % S::IDS_SLOTS;
      const int lim = id_limit(meta_ptr[m * 8 + 2], max(meta_ptr[m * 8 + 3], 0));
      int first_row = -1;
      if (tp.has_tma && (dl4 + 1) * C::TILE <= lim) {
        const int* ids = ids_ptr + rs * C::TILE;
        const int r0 = ids[0];
        const bool mine = ids[lane] == r0 + lane && ids[lane + 32] == r0 + lane + 32;
        if (__all_sync(0xffffffffu, mine) && r0 >= 0 && (uint32_t)(r0 + C::TILE) <= row_lim) first_row = r0;
      }
      if (lane == 0) dense_box[rs] = first_row;
    }
    if (dt5 >= 0)
      issue_kv(dt5 % S::TASK_RING, dl5, (it - 5) % S::IDS_SLOTS, dt5 % S::QID_SLOTS, (it - 5) % C::STAGES, dt5 % S::QBUFS);
    cp_async_commit();

    // ---- consume
#ifdef FT_TIMELINE
    { const long long c = clock64(); tl_sum_issue += c - tl_c0; tl_c0 = c; }
    if (dt7 < 0) ++tl_bubbles;
    if (dt7 >= 0 && tl_first == 0) tl_first = timeline_now();
#endif
    if (dt7 >= 0) {
      const int m = dt7 % S::TASK_RING;
      const int stage = (it - 7) % C::STAGES;
      const uint32_t parity = (stage_phase >> stage) & 1u;  // bubbles skip stages, so the phase is tracked per stage
      stage_phase ^= 1u << stage;
      if (!mbar_wait(bars + 8 * stage, parity, S::WAIT_LIMIT)) {
        flag_error(FT_DEV_WAIT_TIMEOUT);  // every thread of the CTA sees the same barrier: all leave together
        break;
      }
#ifdef FT_TIMELINE
      { const long long c = clock64(); tl_sum_wait += c - tl_c0; tl_c0 = c; ++tl_tiles; }
#endif
      if (dl7 == 0) {  // a new task: its Q rows arrived together with this tile
        c_qoff = meta_ptr[m * 8 + 0];
        c_rows = min(meta_ptr[m * 8 + 1] * G, 16);
        c_kvlen = max(meta_ptr[m * 8 + 3], 0);
        c_kvh = meta_ptr[m * 8 + 4];
        c_tiles = max(1, (c_kvlen + C::TILE - 1) / C::TILE);
        const uint32_t q_sm = sm + (dt7 % S::QBUFS) * 16 * C::ROWB;
#pragma unroll
        for (int nq = 0; nq < 2; ++nq) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            qb[nq][kk][0] = lds32(q_sm + C::swzq(nq * 8 + g8, 2 * kk) + 4 * t4);
            qb[nq][kk][1] = lds32(q_sm + C::swzq(nq * 8 + g8, 2 * kk + 1) + 4 * t4);
          }
          m_run[nq][0] = m_run[nq][1] = -INFINITY;
          l_run[nq][0] = l_run[nq][1] = 0.f;
#pragma unroll
          for (int mb = 0; mb < D / 16; ++mb) o_acc[mb][nq][0] = o_acc[mb][nq][1] = o_acc[mb][nq][2] = o_acc[mb][nq][3] = 0.f;
        }
      }
      const uint32_t k_sm = pipe_sm + stage * 2 * C::STAGE_BYTES, v_sm = k_sm + C::STAGE_BYTES;
      if (dl7 * C::TILE + tok0 < c_kvlen) {  // else: this warp's 16 tokens are all past the end of the chunk
        if (c_rows <= 8)
          stream_tile<T, D, 1>(k_sm, v_sm, tok0, dl7 * C::TILE, c_kvlen, scale2, qb, o_acc, m_run, l_run, lane);
        else
          stream_tile<T, D, 2>(k_sm, v_sm, tok0, dl7 * C::TILE, c_kvlen, scale2, qb, o_acc, m_run, l_run, lane);
      }

#ifdef FT_TIMELINE
      { const long long c = clock64(); tl_sum_tile += c - tl_c0; tl_c0 = c; }
#endif
      if (dl7 == c_tiles - 1) {
        // ---- end of the task: merge the four warps through the stage just consumed, write the partial rows
        __syncthreads();  // every warp is done reading this stage
        float* epi_o = reinterpret_cast<float*>(smem + S::PIPE_OFF + stage * 2 * C::STAGE_BYTES);
        const int nq_used = c_rows <= 8 ? 1 : 2;
#pragma unroll
        for (int nq = 0; nq < 2; ++nq) {
          if (nq < nq_used) {
            float la = l_run[nq][0], lb = l_run[nq][1];
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
              la += __shfl_xor_sync(0xffffffffu, la, o);
              lb += __shfl_xor_sync(0xffffffffu, lb, o);
            }
            const int r = nq * 8 + 2 * t4;
            float* dst = epi_o + (warp * 16 + r) * D;
            const int sw = t4 << 3;  // rows are D floats apart: rotate the columns by the row pair to spread the banks
            if (tok0 < c_kvlen || c_tiles > 1)  // a warp that saw no token stages no output (its maximum stays -inf)
#pragma unroll
            for (int mb = 0; mb < D / 16; ++mb) {
              dst[(mb * 16 + g8) ^ sw] = o_acc[mb][nq][0];
              dst[D + ((mb * 16 + g8) ^ sw)] = o_acc[mb][nq][1];
              dst[(mb * 16 + 8 + g8) ^ sw] = o_acc[mb][nq][2];
              dst[D + ((mb * 16 + 8 + g8) ^ sw)] = o_acc[mb][nq][3];
            }
            if (g8 == 0) {
              epi_m[warp * 16 + r] = m_run[nq][0];
              epi_m[warp * 16 + r + 1] = m_run[nq][1];
              epi_l[warp * 16 + r] = la;
              epi_l[warp * 16 + r + 1] = lb;
            }
          }
        }
        __syncthreads();
        {
          const int r = tid >> 3, seg = tid & 7;
          if (r < c_rows) {
            const int slot = r / G, gg = r - slot * G;
            const int64_t part = (int64_t)c_qoff + slot;
            if (part >= 0 && part < p.num_partial_rows) {
              float M = -INFINITY;
#pragma unroll
              for (int w = 0; w < 4; ++w) M = fmaxf(M, epi_m[w * 16 + r]);
              float L = 0.f;
              float4 out[D / 32];
#pragma unroll
              for (int i = 0; i < D / 32; ++i) out[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                const float mw = epi_m[w * 16 + r];
                if (mw == -INFINITY) continue;  // that warp saw no valid token for this row and staged nothing
                const float f = fast_exp2(mw - M);
                L = fmaf(epi_l[w * 16 + r], f, L);
                const float4* src = reinterpret_cast<const float4*>(epi_o + (w * 16 + r) * D);
#pragma unroll
                for (int i = 0; i < D / 32; ++i) {
                  const float4 x = src[(seg + 8 * i) ^ (((r >> 1) & 3) << 1)];
                  out[i].x = fmaf(f, x.x, out[i].x);
                  out[i].y = fmaf(f, x.y, out[i].y);
                  out[i].z = fmaf(f, x.z, out[i].z);
                  out[i].w = fmaf(f, x.w, out[i].w);
                }
              }
              const float inv = L > 0.f ? 1.f / L : 0.f;
              const int head = c_kvh * G + gg;
              float4* dst = reinterpret_cast<float4*>(p.mid_o + part * p.mo_s0 + (int64_t)head * p.mo_s1);
#pragma unroll
              for (int i = 0; i < D / 32; ++i)
                dst[seg + 8 * i] = make_float4(out[i].x * inv, out[i].y * inv, out[i].z * inv, out[i].w * inv);
              if (seg == 0)
                p.mid_lse[part * p.ml_s0 + head] = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
            }
          }
        }
        ++tasks_done;
#ifdef FT_TIMELINE
        { const long long c = clock64(); tl_sum_epi += c - tl_c0; tl_c0 = c; }
#endif
        // the stage is refilled only after the barrier at the top of a later iteration
      }
    }
    meta_4 = meta_3;
    meta_3 = meta_2;
    meta_2 = meta_1;
    meta_1 = meta_issued;

    // ---- leave when the list is exhausted and every slot in flight has been consumed
    if (next_task >= ntasks && tasks_done == meta_issued) break;
  }
#ifdef FT_TIMELINE
  if (tid == 0 && blockIdx.x < FT_TIMELINE_CTAS) {  // developer builds: where this worker's cycles went
    unsigned long long* rec = g_timeline + 16 * blockIdx.x;
    rec[4] = tl_first;
    rec[5] = tl_bubbles;
    rec[6] = tl_iters;
    rec[7] = tasks_done;
    rec[8] = tl_tiles;
    rec[9] = tl_sum_top;
    rec[10] = tl_sum_issue;
    rec[11] = tl_sum_wait;
    rec[12] = tl_sum_tile;
    rec[13] = tl_sum_epi;
  }
#endif
  cp_async_wait<0>();
  __syncthreads();
}

template <typename T, int D>
__global__ void __launch_bounds__(128, 2) stage1_stream_kernel(const __grid_constant__ TcParams tp) {
  allow_dependent_launch();
  wait_for_prior_grid();  // nothing of the preceding kernel's is read or overwritten before this
  extern __shared__ __align__(1024) uint8_t smem[];
  stream_worker<T, D>(tp, smem, 0, tp.p.node_count * tp.p.num_kv_heads, (int)blockIdx.x, (int)gridDim.x);
}

}  // namespace ft
