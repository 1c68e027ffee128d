// Stage 1 as ONE persistent kernel (head_dim 128, 16-bit types): two CTAs per SM
// walk the launch's task list and keep their K/V streams running across task
// boundaries, so that a task's start-up (claim -> metadata -> row ids -> first
// tile) and its epilogue hide behind the tiles of its neighbours, and the grid
// does not depend on the plan.
//
// A task is a (vnode, kv head) pair: the vnode's packed query rows (requests x
// GQA group), 128 per pass, against the vnode's KV chunk, 64 tokens per tile:
//
//   S[128 x 64]   = Q[128 x 128] . K_tile^T      tcgen05.mma, A and B operands K-major in shared memory
//   O[128 x 128] += P[128 x 64]  . V_tile        tcgen05.mma, A operand (P) in tensor memory, B MN-major
//
// Every task takes this path, also those with a handful of rows (leaves): the
// tensor core then multiplies padding, which costs nothing while the step is
// bound by HBM, and only the warps that own live rows do softmax work.
//
// Tensor memory (256 columns per CTA): two 64-column S buffers and 128 columns
// of O.  P_t is written by the softmax threads over the first 32 columns of the
// S buffer it was computed from (two 16-bit values per column) and read from
// there by P.V, so it never touches shared memory.
//
// Roles (8 warps; the register file is traded between the two warpgroups at start)
//   warps 0-3   softmax: thread r owns query row r (= TMEM lane r)
//   warp  4     MMA issue (one lane)
//   warp  5     scheduler + K loader: claims tasks (the first is the CTA's index, the rest come from a device
//               counter in list order - longest first as the planner sorts them), fetches their metadata one
//               task ahead, publishes them in a 4-entry ring for the other roles, and loads their K tiles
//   warp  6     V loader
//   warp  7     Q loader: TMA boxes (whole tile when the request ids are consecutive, else per request) or cp.async
// K and V tiles of 64 consecutive pool rows come by tiled TMA (128-byte swizzle, no multicast), any other tile is
// gathered row by row with 16-byte cp.async; row ids sit in registers, one tile ahead, reaching across the task
// boundary.  Hand-offs are mbarriers, each with one waiting role; every wait is bounded (wall time) and unwinds
// the CTA through an abort flag and the device status word.
//
// What overlaps what: the loaders run ahead of the tensor core by the depth of their rings (K 2 tiles, V 3),
// into the next task; the MMA warp issues the first S tiles of the next task while the softmax threads still
// write the partial rows of the previous one; the next task's Q tile is fetched as soon as the last S of the
// current task has been issued; S_t+1 is computed while the softmax of tile t runs, and the softmax of tile t+1
// may finish before P_t . V_t has (the P and P.V barriers alternate between two instances by tile parity, so
// a thread one tile ahead neither arrives twice in one phase nor loses count of the phases).
//
// Arithmetic conventions as in the other stage-1 kernels (kernel_bench/fasttree.py:360-413).
#pragma once

#include "ft_stage1_tc.cuh"

namespace ft {

struct PsCfg {
  static constexpr int THREADS = 256;
  static constexpr int TILE = 64;
  static constexpr int D = 128;
  static constexpr int NSK = 2, NSV = 3;               // K / V ring stages (a V tile is held until P.V, after the softmax)
  static constexpr int TR = 4;                         // task ring entries
  static constexpr int Q_OFF = 0;                      // 2 blocks x [128 rows][128 B]
  static constexpr int K_OFF = 32768;                  // NSK x (2 blocks x [64 tok][128 B])
  static constexpr int V_OFF = K_OFF + NSK * 16384;
  static constexpr int REQ_OFF = V_OFF + NSV * 16384;  // request ids of the task being loaded (128)
  static constexpr int TASK_OFF = REQ_OFF + 512;       // TR x 8 ints
  static constexpr int BAR_OFF = TASK_OFF + TR * 32;
  // barrier indices
  static constexpr int K_FULL = 0, K_EMPTY = K_FULL + NSK, V_FULL = K_EMPTY + NSK, V_EMPTY = V_FULL + NSV;
  static constexpr int Q_FULL = V_EMPTY + NSV, Q_EMPTY = Q_FULL + 1;
  static constexpr int TASK_FULL = Q_EMPTY + 1, TASK_EMPTY = TASK_FULL + TR;
  static constexpr int S_FULL = TASK_EMPTY + TR, P_FULL = S_FULL + 2, PV_DONE = P_FULL + 2;
  static constexpr int NBARS = PV_DONE + 2;
  static constexpr int ABORT_OFF = BAR_OFF + NBARS * 8;
  static constexpr int TMEM_SLOT_OFF = ABORT_OFF + 4;
  static constexpr int SMEM_BYTES = TMEM_SLOT_OFF + 4;
  static constexpr int TMEM_COLS = 256;                // S0 [0,64), S1 [64,128), O [128,256)
  static constexpr int O_COL = 128;
  static constexpr int REGS_SOFTMAX = 184, REGS_OTHER = 72;
};
static_assert(PsCfg::SMEM_BYTES <= 115712, "two CTAs must fit in one SM's shared memory");
static_assert((PsCfg::BAR_OFF & 7) == 0, "mbarriers are 8-byte aligned");


__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// First wait that gave up since the record was last read: {wait id (0 = none), block, warp, task sequence number,
// tile counter, 0...}.  Wait ids: 1 task ring, 2 S tile, 3 P.V before O is touched, 4 P.V before the epilogue, 5 Q tile,
// 6 V tile, 7 P, 8 K tile, 9 P.V before an S buffer is reused, 10 K/V stage free, 11 Q buffer free, 12 task slot free.
__device__ int g_wait_diag[8] = {0, 0, 0, 0, 0, 0, 0, 0};

__device__ __forceinline__ void note_wait(int id, int seq, int counter) {
  if (atomicCAS(&g_wait_diag[0], 0, id) == 0) {
    g_wait_diag[1] = (int)blockIdx.x;
    g_wait_diag[2] = (int)(threadIdx.x >> 5);
    g_wait_diag[3] = seq;
    g_wait_diag[4] = counter;
  }
}

// Bounded wait of the persistent kernel.  A role may legitimately wait for as long as another task runs, so the
// bound is wall time (about a quarter of a second on the global timer), not a probe count; it also ends as
// soon as another role has raised the CTA's abort flag.
__device__ __forceinline__ bool ps_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  unsigned long long t0 = 0;
  for (int it = 0;; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((it & 63) == 63) {
      if (*abort_flag != 0) return false;
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      if (now - t0 > 250000000ull) return false;
    }
  }
}

struct PsTask {
  int vn, kvh, q_off, q_len, kv_off, kv_len, row0;
};

template <typename T>
__global__ void __launch_bounds__(PsCfg::THREADS, 2) stage1_persist_kernel(const __grid_constant__ TcParams tp) {
  using C = PsCfg;
  allow_dependent_launch();
  FT_TL_BEGIN();
  extern __shared__ __align__(1024) uint8_t smem[];
  const Stage1Params& p = tp.p;
  const uint32_t sm = smem_u32(smem);
  const uint32_t bars = sm + C::BAR_OFF;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::ABORT_OFF);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::TMEM_SLOT_OFF);
  volatile int* task_ring = reinterpret_cast<volatile int*>(smem + C::TASK_OFF);
  auto bar = [&](int i) { return bars + 8u * i; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.group, H = p.num_kv_heads;
  const float scale2 = p.sm_scale * 1.4426950408889634f;
  const uint32_t row_lim = (uint32_t)(p.kv_rows < 0x7fffffffLL ? p.kv_rows : 0x7fffffffLL);

  const bool usable = (sm & 1023u) == 0u;  // the swizzled operand layout needs a 1024-byte aligned window
  if (!usable && tid == 0) flag_error(FT_DEV_WAIT_TIMEOUT);

  // ---- one-time set-up: barriers, tensor memory
  if (usable) {
    if (tid == 32 && tp.has_tma) {
      asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tp.k_map)) : "memory");
      asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tp.v_map)) : "memory");
      if (tp.q_box_rows > 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tp.q_map_tile)) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tp.q_map)) : "memory");
      }
    }
    if (tid == 0) {
      for (int s = 0; s < C::NSK; ++s) {
        mbar_init(bar(C::K_FULL + s), 32);   // the loader's lanes
        mbar_init(bar(C::K_EMPTY + s), 1);   // tcgen05.commit
      }
      for (int s = 0; s < C::NSV; ++s) {
        mbar_init(bar(C::V_FULL + s), 32);
        mbar_init(bar(C::V_EMPTY + s), 1);
      }
      mbar_init(bar(C::Q_FULL), 32);
      mbar_init(bar(C::Q_EMPTY), 1);
      for (int s = 0; s < C::TR; ++s) {
        mbar_init(bar(C::TASK_FULL + s), 1);
        mbar_init(bar(C::TASK_EMPTY + s), 128);  // every softmax thread, once it is past the task
      }
      for (int b = 0; b < 2; ++b) {
        mbar_init(bar(C::S_FULL + b), 1);
        mbar_init(bar(C::P_FULL + b), 128);
        mbar_init(bar(C::PV_DONE + b), 1);
      }
      *abort_flag = 0;
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(sm + C::TMEM_SLOT_OFF),
                   "r"(C::TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = usable ? *tmem_slot : 0u;
  wait_for_prior_grid();  // everything above is on-chip set-up; the preceding kernel's results are visible from here on
  // the launch's vnode range: host arguments, or read from the device so that the launch outlives the plan
  int node_offset = p.node_offset, node_count = p.node_count;
  if (p.dev_phase != nullptr) {
    const int n0 = max(__ldg(p.dev_phase + 0), 0), n1 = max(__ldg(p.dev_phase + 1), 0);
    node_offset = max(__ldg(p.dev_phase + 2), 0);
    node_count = n0 + n1;
    if (n0 > 0 && n1 > 0 && __ldg(p.dev_phase + 3) != node_offset + n0) {  // the phases must be adjacent
      if (threadIdx.x == 0) flag_error(FT_DEV_BAD_ROW_INDEX);
      node_count = n0;
    }
  }
  const int total_tasks = (int)min((long long)node_count * H, 0x7fffffffLL);
  if (tid == 0) FT_TL_MARK(0);
#ifdef FT_TIMELINE
  long long tl_s = 0, tl_epi = 0, tl_task = 0, tl_pv = 0, tl_c = 0;
  int tl_tasks = 0, tl_tiles = 0;
#define PS_TL_T0() tl_c = (long long)timeline_now()
#define PS_TL_ADD(acc) acc += (long long)timeline_now() - tl_c
#else
#define PS_TL_T0() do { } while (0)
#define PS_TL_ADD(acc) do { } while (0)
#endif

  bool dead = !usable;
  auto give_up = [&](int wait_id, int seq_, int counter) {
    if (*abort_flag == 0) note_wait(wait_id, seq_, counter);  // only the wait that gave up first is of interest
    *abort_flag = 1;
    flag_error(FT_DEV_WAIT_TIMEOUT);
    dead = true;
  };
  // A wait made by a whole warp: every lane leaves with the same answer, so that the warp stays converged for
  // the warp-collective tensor-memory instructions that follow (or gives up as one).
  auto warp_wait = [&](uint32_t b_, uint32_t parity) {
    const bool ok = ps_wait(b_, parity, abort_flag);
    return __all_sync(0xffffffffu, ok) != 0;
  };
  // entry `seq` of the task stream: false when the wait gave up; t.vn < 0 marks the end of the stream
  auto read_task = [&](int seq, PsTask& t, bool whole_warp) {
    const int slot = seq % C::TR;
    if (!(whole_warp ? warp_wait(bar(C::TASK_FULL + slot), (uint32_t)(seq / C::TR) & 1u)
                     : ps_wait(bar(C::TASK_FULL + slot), (uint32_t)(seq / C::TR) & 1u, abort_flag)))
      return false;
    const volatile int* e = task_ring + slot * 8;
    t.vn = e[0];
    t.kvh = e[1];
    t.q_off = e[2];
    t.q_len = e[3];
    t.kv_off = e[4];
    t.kv_len = e[5];
    t.row0 = e[6];
    return true;
  };
  auto id_limit = [&](int kv_off, int kv_len) {  // readable row ids of a chunk (a table that ends early is a plan error)
    return kv_ids_limit(p, kv_off, kv_len);
  };
  // one K or V tile into `buf`, signalling `full`: TMA when its 64 row ids (cur: two per lane) are consecutive
  auto load_tile = [&](const CUtensorMap* map, const T* base, int64_t s0, int kvh, int tt, int id_lim, const int (&cur)[2],
                       uint32_t buf, uint32_t full) {
    bool dense = false;
    int first_row = 0;
    if (tp.has_tma && (tt + 1) * C::TILE <= id_lim) {
      first_row = __shfl_sync(0xffffffffu, cur[0], 0);
      const bool mine = cur[0] == first_row + lane && cur[1] == first_row + lane + 32;
      dense = __all_sync(0xffffffffu, mine) && first_row >= 0 && (uint32_t)(first_row + C::TILE) <= row_lim;
    }
    if (dense) {
      if (lane == 0) {
        mbar_arrive_expect_tx(full, 16384);
        tma_load_3d(buf, map, 0, kvh, first_row, full);
        tma_load_3d(buf + 8192, map, 64, kvh, first_row, full);
      } else {
        mbar_arrive(full);
      }
      return;
    }
    const int c = lane & 15;
    bool bad = false, stored = false;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll 4
      for (int i = 0; i < 16; ++i) {
        const int rr = (lane >> 4) + 2 * i + 32 * h, pos = tt * C::TILE + rr;  // row rr: slot h of lane rr & 31
        const int id = __shfl_sync(0xffffffffu, cur[h], rr & 31);
        const uint32_t row = pos < id_lim ? (uint32_t)id : 0xffffffffu;
        const bool ok = row < row_lim;  // padding (0xffffffff), negative and too-large ids all fail this test
        bad |= !ok && pos < id_lim;
        stored |= !ok;
        cp_async16(buf + tc_swz(rr, c, 8192), base + (int64_t)(ok ? row : 0u) * s0 + c * 8, ok);
      }
    }
    if (bad) flag_error(FT_DEV_BAD_KV_INDEX);
    if (stored) proxy_fence();  // the zero rows were plain shared stores
    mbar_arrive_on_cp_async(full);
  };
  auto fetch_ids = [&](int kv_off, int lim, int tile, int (&dst)[2]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int pos = tile * C::TILE + lane + 32 * h;
      dst[h] = pos < lim ? __ldg(kv_ids_base(p, kv_off) + pos) : -1;
    }
  };

  if (warp < 4) {
    // ==================================================================== softmax (one query row per thread)
    reg_grow<C::REGS_SOFTMAX>();
    const int r = tid;  // row inside the pass = TMEM lane
    const uint32_t t_lane = tmem + ((uint32_t)(warp * 32) << 16);
    int gx = 0;  // tiles seen so far, over all tasks: S / P buffer and barrier instance gx & 1, phase gx >> 1
    // P.V of tile `tile` has completed (every thread observes every phase of both barrier instances in order)
    auto pv_done = [&](int tile) { return warp_wait(bar(C::PV_DONE + (tile & 1)), (uint32_t)(tile >> 1) & 1u); };
    for (int seq = 0; !dead; ++seq) {
      PsTask t;
      PS_TL_T0();
      if (!read_task(seq, t, true)) {
        give_up(1, seq, gx);
        break;
      }
      PS_TL_ADD(tl_task);
      if (t.vn < 0) break;
      const int rows = min(t.q_len * G - t.row0, 128);
      const int kv_len = t.kv_len;
      const int ntiles = (kv_len + C::TILE - 1) / C::TILE;
      const bool warp_live = warp * 32 < rows;  // a warp whose 32 rows are all past the end only keeps step
      const int prow = t.row0 + r;              // packed row of the task
      const bool live = r < rows;
      int slot = 0, gg = 0;
      if (live) {
        slot = prow / G;
        gg = prow - slot * G;
      }
      const int64_t part = (int64_t)t.q_off + slot;
      const bool store = live && part >= 0 && part < p.num_partial_rows;
      int r_lo = 0, r_hi = kv_len;  // the chunk tokens this row attends to: all of them unless the plan narrows it
      if (p.q_ranges != nullptr && store) {
        r_lo = max(p.q_ranges[2 * part], 0);
        r_hi = min(p.q_ranges[2 * part + 1], kv_len);
      }
      float m_used = -INFINITY, l_run = 0.f;
      for (int j = 0; j < ntiles && !dead; ++j, ++gx) {
        const int b = gx & 1;
        PS_TL_T0();
        if (!warp_wait(bar(C::S_FULL + b), (uint32_t)(gx >> 1) & 1u)) {
          give_up(2, seq, gx);
          break;
        }
        PS_TL_ADD(tl_s);
#ifdef FT_TIMELINE
        if (gx == 0 && tid == 0) FT_TL_MARK(3);
        ++tl_tiles;
#endif
        tc_fence_after();
        const uint32_t s_col = t_lane + b * C::TILE;
        float corr = 1.f;
        bool grow = false;
        uint32_t w[32];
        if (warp_live) {
          float s[64];
          tmem_ld32_nowait(s_col, *reinterpret_cast<float(*)[32]>(&s[0]));  // both halves in flight, one wait
          tmem_ld32_nowait(s_col + 32, *reinterpret_cast<float(*)[32]>(&s[32]));
          tmem_wait_ld();
          const int lo = r_lo - j * C::TILE, hi = r_hi - j * C::TILE;
          if (lo > 0 || hi < C::TILE) {
#pragma unroll
            for (int c = 0; c < 64; ++c)
              if (c < lo || c >= hi) s[c] = -INFINITY;
          }
          // four independent chains (one warp or two per scheduler cannot hide a 32-deep dependent chain)
          float mx4[4] = {fmaxf(s[0], s[1]), fmaxf(s[2], s[3]), fmaxf(s[4], s[5]), fmaxf(s[6], s[7])};
#pragma unroll
          for (int c = 8; c < 64; c += 8) {
#pragma unroll
            for (int k = 0; k < 4; ++k) asm("max.f32 %0, %0, %1, %2;" : "+f"(mx4[k]) : "f"(s[c + 2 * k]), "f"(s[c + 2 * k + 1]));
          }
          float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
          mx *= scale2;  // scale2 > 0
          if (mx > m_used + 8.f || m_used == -INFINITY) {  // the offset may lag the true maximum by up to 2^8
            grow = mx > -INFINITY;
            if (grow) {
              corr = fast_exp2(m_used - mx);  // 0 on the first tile
              m_used = mx;
            }
          }
          l_run *= corr;
          const float neg_off = m_used == -INFINITY ? 0.f : -m_used;
          const float2 sc2 = make_float2(scale2, scale2), no2 = make_float2(neg_off, neg_off);
          float2 sum4[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float2 e = __ffma2_rn(make_float2(s[2 * i], s[2 * i + 1]), sc2, no2);
            if (FT_EXP2_FMA_EVERY > 0 && (i % (FT_EXP2_FMA_EVERY > 0 ? FT_EXP2_FMA_EVERY : 1)) == (FT_EXP2_FMA_EVERY > 0 ? FT_EXP2_FMA_EVERY : 1) - 1) {
              e.x = exp2_fma(e.x);
              e.y = exp2_fma(e.y);
            } else {
              e.x = fast_exp2(e.x);
              e.y = fast_exp2(e.y);
            }
            sum4[i & 3] = __fadd2_rn(sum4[i & 3], e);
            w[i] = pack2<T>(e.x, e.y);
          }
          {
            const float2 sum2 = __fadd2_rn(__fadd2_rn(sum4[0], sum4[1]), __fadd2_rn(sum4[2], sum4[3]));
            l_run += sum2.x + sum2.y;
          }
        }
        // P_t goes to the S buffer just read, which the tensor core does not write again before it has consumed it
        // (the MMA warp waits for P.V of tile t before it issues S of tile t + 2).  Bookkeeping first: P.V of tile
        // t - 2 is long done, but every thread looks at every phase of the two P.V barriers in turn so that their
        // parities keep their meaning.  O is only touched when the running offset has to grow, and then P.V of
        // tile t - 1 must be done too.
        PS_TL_T0();
        if (gx >= 2 && !pv_done(gx - 2)) {
          give_up(3, seq, gx);
          break;
        }
        PS_TL_ADD(tl_pv);
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          if (!pv_done(gx - 1)) {
            give_up(3, seq, gx);
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int cb = 0; cb < 4; ++cb) {
            float o[32];
            tmem_ld32(t_lane + C::O_COL + cb * 32, o);
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] *= corr;
            tmem_st32(t_lane + C::O_COL + cb * 32, o);
          }
        }
        if (warp_live) tmem_st32(s_col, *reinterpret_cast<float(*)[32]>(&w[0]));
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar(C::P_FULL + b));
      }
      // ---- epilogue: wait for the last two P.V (in order), normalise, write this thread's partial row
      PS_TL_T0();
      if (!dead && gx >= 2 && !pv_done(gx - 2)) give_up(4, seq, gx);
      if (!dead && gx >= 1 && !pv_done(gx - 1)) give_up(4, seq, gx);
      if (!dead) {
        tc_fence_after();
        const int head = t.kvh * G + gg;
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        if (warp_live) {
          float4* dst = store ? reinterpret_cast<float4*>(p.mid_o + part * p.mo_s0 + (int64_t)head * p.mo_s1) : nullptr;
#pragma unroll
          for (int cb = 0; cb < 4; ++cb) {
            float o[32];
            tmem_ld32(t_lane + C::O_COL + cb * 32, o);  // warp-collective
            if (dst != nullptr) {
#pragma unroll
              for (int c = 0; c < 8; ++c)
                dst[cb * 8 + c] = make_float4(o[4 * c] * inv, o[4 * c + 1] * inv, o[4 * c + 2] * inv, o[4 * c + 3] * inv);
            }
          }
          if (store)
            p.mid_lse[part * p.ml_s0 + head] = l_run > 0.f ? (m_used + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
        }
        tc_fence_before();
        // the task's ring entry may be reused once every softmax thread is past it (the other roles are done with a
        // task before its last P.V completes)
        mbar_arrive(bar(C::TASK_EMPTY + seq % C::TR));
      }
      PS_TL_ADD(tl_epi);
#ifdef FT_TIMELINE
      if (tl_tasks == 0 && tid == 0) FT_TL_MARK(4);
      ++tl_tasks;
#endif
    }
#ifdef FT_TIMELINE
    if (tid == 0 && blockIdx.x < FT_TIMELINE_CTAS) {
      unsigned long long* rec = g_timeline + 16 * blockIdx.x;
      rec[9] = tl_tasks;
      rec[10] = tl_tiles;
      rec[11] = tl_s;
      rec[12] = tl_epi;
      rec[13] = tl_task;
      rec[14] = tl_pv;
      rec[15] = timeline_now();
    }
#endif
  } else {
    reg_shrink<C::REGS_OTHER>();
    if (warp == 4) {
      // ================================================================== MMA issue
      if (lane == 0 && !dead) {
        const uint32_t idesc_s = tc_idesc<T>(128, C::TILE, false);
        const uint32_t idesc_o = tc_idesc<T>(128, C::D, true);
        const uint64_t q_desc = tc_desc(sm + C::Q_OFF, 16, 1024);
        const uint32_t o_tmem = tmem + (uint32_t)C::O_COL;
        int gx = 0, qseq = 0;  // tiles / tasks issued so far
        for (int seq = 0; !dead; ++seq) {
          PsTask t;
          if (!read_task(seq, t, false)) {
            give_up(1, seq, gx);
            break;
          }
          if (t.vn < 0) break;
          const int ntiles = (t.kv_len + C::TILE - 1) / C::TILE;
          if (!ps_wait(bar(C::Q_FULL), (uint32_t)qseq & 1u, abort_flag)) {
            give_up(5, seq, qseq);
            break;
          }
          ++qseq;
          const int g0 = gx;
          // O += P(tile) . V(tile): four k-steps of 16 tokens, P from tensor memory
          auto pv = [&](int tile) {
            const int sv = tile % C::NSV, b = tile & 1;
            if (!ps_wait(bar(C::V_FULL + sv), (uint32_t)(tile / C::NSV) & 1u, abort_flag)) {
              give_up(6, seq, tile);
              return;
            }
            if (!ps_wait(bar(C::P_FULL + b), (uint32_t)(tile >> 1) & 1u, abort_flag)) {
              give_up(7, seq, tile);
              return;
            }
            proxy_fence();
            tc_fence_after();
            const uint64_t v_desc = tc_desc(sm + C::V_OFF + sv * 16384, 8192, 1024);
            const uint32_t p_tmem = tmem + (uint32_t)(b * C::TILE);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              tc_mma_ts(o_tmem, p_tmem + (uint32_t)(ks * 8), v_desc + (uint64_t)(ks * 128), idesc_o, (tile > g0 || ks > 0) ? 1u : 0u);
            tc_commit(bar(C::PV_DONE + b));
            tc_commit(bar(C::V_EMPTY + sv));
          };
          for (int tt = 0; tt < ntiles && !dead; ++tt, ++gx) {
            const int sk = gx % C::NSK, b = gx & 1;
            if (!ps_wait(bar(C::K_FULL + sk), (uint32_t)(gx / C::NSK) & 1u, abort_flag)) {
              give_up(8, seq, gx);
              break;
            }
#ifdef FT_TIMELINE
            if (gx == 0) FT_TL_MARK(2);
#endif
            // S buffer b still holds P of tile gx - 2 until that tile's P.V has COMPLETED: MMAs of different
            // shapes are not ordered against each other, so issue order alone does not protect it
            if (gx >= 2 && !ps_wait(bar(C::PV_DONE + b), (uint32_t)((gx - 2) >> 1) & 1u, abort_flag)) {
              give_up(9, seq, gx);
              break;
            }
            proxy_fence();
            tc_fence_after();
            const uint64_t k_desc = tc_desc(sm + C::K_OFF + sk * 16384, 16, 1024);
            const uint32_t s_tmem = tmem + (uint32_t)(b * C::TILE);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {  // 8 k-steps of 16 along head_dim: +32 B inside a block, +1 block after 4
              const uint64_t a = q_desc + (uint64_t)((ks >> 2) * (16384 >> 4) + (ks & 3) * 2);
              const uint64_t bb = k_desc + (uint64_t)((ks >> 2) * (8192 >> 4) + (ks & 3) * 2);
              tc_mma(s_tmem, a, bb, idesc_s, ks > 0);
            }
            tc_commit(bar(C::S_FULL + b));
            tc_commit(bar(C::K_EMPTY + sk));
            if (tt == ntiles - 1) tc_commit(bar(C::Q_EMPTY));  // the Q tile may be replaced
            if (tt > 0) pv(gx - 1);
          }
          if (!dead) pv(gx - 1);
        }
      }
      __syncwarp();
    } else if (warp == 5) {
      // ================================================================== scheduler + K loader
      unsigned int* counters = tp.sched;
      const T* kbase0 = reinterpret_cast<const T*>(p.k);
      auto meta_load = [&](int b_) {  // lanes 0-3: q_off, q_len, kv_off, kv_len of the task's vnode
        int v = 0;
        if (b_ < total_tasks && lane < 4) {
          const int vn = node_offset + b_ / H;
          const int32_t* tab = lane == 0 ? p.q_offs : lane == 1 ? p.q_lens : lane == 2 ? p.kv_offs : p.kv_lens;
          v = __ldg(tab + vn);
        }
        return v;
      };
      int g = 0, seq = 0;
      int b = (int)blockIdx.x;  // the first task needs no claim
      int meta = meta_load(b);
      int pre[2] = {-1, -1};
      int pre_b = -1;           // `pre` holds the row ids of tile 0 of task pre_b
      while (!dead) {
        const int slot0 = seq % C::TR;
        if (b >= total_tasks) {  // the end marker
          if (!warp_wait(bar(C::TASK_EMPTY + slot0), ((uint32_t)(seq / C::TR) & 1u) ^ 1u)) {
            give_up(12, seq, b);
            break;
          }
          if (lane == 0) {
            task_ring[slot0 * 8] = -1;
            mbar_arrive(bar(C::TASK_FULL + slot0));
          }
          break;
        }
        // claim the task after this one right away: the round trip overlaps this task's loads
        int b_next = total_tasks;
        if (lane == 0) b_next = (int)gridDim.x + (int)atomicAdd(counters, 1u);
        int meta_next = 0;
        bool next_known = false;
        PsTask t;
        t.vn = node_offset + b / H;
        t.kvh = b - (b / H) * H;
        t.q_off = __shfl_sync(0xffffffffu, meta, 0);
        t.q_len = __shfl_sync(0xffffffffu, meta, 1);
        t.kv_off = __shfl_sync(0xffffffffu, meta, 2);
        t.kv_len = max(__shfl_sync(0xffffffffu, meta, 3), 0);
        const int rows_total = t.q_len * G;
        if (rows_total > 0 && t.kv_len == 0) {
          // an empty chunk: nothing to stream; its partial rows are zero with an LSE of -inf
          for (int64_t i = lane; i < (int64_t)rows_total * 32; i += 32) {
            const int prow = (int)(i >> 5), c4 = (int)(i & 31);
            const int slot = prow / G, gg = prow - slot * G;
            const int64_t part = (int64_t)t.q_off + slot;
            if (part >= 0 && part < p.num_partial_rows) {
              const int head = t.kvh * G + gg;
              reinterpret_cast<float4*>(p.mid_o + part * p.mo_s0 + (int64_t)head * p.mo_s1)[c4] = make_float4(0.f, 0.f, 0.f, 0.f);
              if (c4 == 0) p.mid_lse[part * p.ml_s0 + head] = -INFINITY;
            }
          }
        } else if (rows_total > 0) {
          const int ntiles = (t.kv_len + C::TILE - 1) / C::TILE;
          const int id_lim = id_limit(t.kv_off, t.kv_len);
          if (id_lim < t.kv_len && lane == 0) flag_error(FT_DEV_BAD_KV_INDEX);
          const T* base = kbase0 + (int64_t)t.kvh * p.k_s1;
          for (int row0 = 0; row0 < rows_total && !dead; row0 += 128) {
            // publish this pass
            const int slot = seq % C::TR;
            if (!warp_wait(bar(C::TASK_EMPTY + slot), ((uint32_t)(seq / C::TR) & 1u) ^ 1u)) {
              give_up(12, seq, b);
              break;
            }
            if (lane == 0) {
              volatile int* e = task_ring + slot * 8;
              e[0] = t.vn;
              e[1] = t.kvh;
              e[2] = t.q_off;
              e[3] = t.q_len;
              e[4] = t.kv_off;
              e[5] = t.kv_len;
              e[6] = row0;
              mbar_arrive(bar(C::TASK_FULL + slot));
            }
            __syncwarp();
            ++seq;
            const bool last_pass = row0 + 128 >= rows_total;
            int cur[2], nxt[2] = {-1, -1};
            if (pre_b == b && row0 == 0) {
              cur[0] = pre[0];
              cur[1] = pre[1];
            } else {
              fetch_ids(t.kv_off, id_lim, 0, cur);
            }
            for (int tt = 0; tt < ntiles && !dead; ++tt, ++g) {
              if (tt + 1 < ntiles) fetch_ids(t.kv_off, id_lim, tt + 1, nxt);
              const int sk = g % C::NSK;
              if (!warp_wait(bar(C::K_EMPTY + sk), ((uint32_t)(g / C::NSK) & 1u) ^ 1u)) {
                give_up(10, seq, g);
                break;
              }
              load_tile(&tp.k_map, base, p.k_s0, t.kvh, tt, id_lim, cur, sm + C::K_OFF + sk * 16384, bar(C::K_FULL + sk));
#ifdef FT_TIMELINE
              if (g == 0 && lane == 0) FT_TL_MARK(1);
#endif
              if (last_pass && !next_known) {  // the claim has had a tile's time to come back: fetch that task's metadata
                b_next = __shfl_sync(0xffffffffu, b_next, 0);
                meta_next = meta_load(b_next);
                next_known = true;
              }
              if (last_pass && tt == ntiles - 1 && b_next < total_tasks) {
                // last tile of the task: the next task's first row ids, so that its first tile follows at once
                const int n_off = __shfl_sync(0xffffffffu, meta_next, 2), n_len = max(__shfl_sync(0xffffffffu, meta_next, 3), 0);
                if (n_len > 0) {
                  fetch_ids(n_off, id_limit(n_off, n_len), 0, pre);
                  pre_b = b_next;
                }
              }
              cur[0] = nxt[0];
              cur[1] = nxt[1];
            }
          }
        }
        if (!next_known) {
          b_next = __shfl_sync(0xffffffffu, b_next, 0);
          meta_next = meta_load(b_next);
        }
        b = b_next;
        meta = meta_next;
      }
      cp_async_wait<0>();
    } else if (warp == 6) {
      // ================================================================== V loader
      const T* vbase0 = reinterpret_cast<const T*>(p.v);
      int g = 0;
      int pre[2] = {-1, -1}, pre_seq = -1;  // row ids of tile 0 of entry `pre_seq`, fetched while the entry before it was loading
      for (int seq = 0; !dead; ++seq) {
        PsTask t;
        if (!read_task(seq, t, true)) {
          give_up(1, seq, g);
          break;
        }
        if (t.vn < 0) break;
        const int kv_len = t.kv_len, kv_off = t.kv_off;
        const int ntiles = (kv_len + C::TILE - 1) / C::TILE;
        const int id_lim = id_limit(kv_off, kv_len);
        const T* base = vbase0 + (int64_t)t.kvh * p.v_s1;
        int cur[2], nxt[2] = {-1, -1};
        if (pre_seq == seq) {
          cur[0] = pre[0];
          cur[1] = pre[1];
        } else {
          fetch_ids(kv_off, id_lim, 0, cur);
        }
        for (int tt = 0; tt < ntiles && !dead; ++tt, ++g) {
          if (tt + 1 < ntiles) {
            fetch_ids(kv_off, id_lim, tt + 1, nxt);
          } else {
            // last tile of the entry: if the next one is already published, fetch its first row ids now
            const int nseq = seq + 1, nslot = nseq % C::TR;
            if (mbar_test(bar(C::TASK_FULL + nslot), (uint32_t)(nseq / C::TR) & 1u)) {
              const volatile int* e = task_ring + nslot * 8;
              const int n_vn = e[0], n_off = e[4], n_len = e[5];
              if (n_vn >= 0 && n_len > 0) {
                fetch_ids(n_off, id_limit(n_off, n_len), 0, pre);
                pre_seq = nseq;
              }
            }
          }
          const int sv = g % C::NSV;
          if (!warp_wait(bar(C::V_EMPTY + sv), ((uint32_t)(g / C::NSV) & 1u) ^ 1u)) {
            give_up(10, seq, g);
            break;
          }
          load_tile(&tp.v_map, base, p.v_s0, t.kvh, tt, id_lim, cur, sm + C::V_OFF + sv * 16384, bar(C::V_FULL + sv));
          cur[0] = nxt[0];
          cur[1] = nxt[1];
        }
      }
      cp_async_wait<0>();
    } else {
      // ================================================================== Q loader (warp 7)
      const uint32_t req_sm = sm + C::REQ_OFF;
      const int* req_of = reinterpret_cast<const int*>(smem + C::REQ_OFF);
      const uint32_t q_sm = sm + C::Q_OFF;
      const uint32_t full = bar(C::Q_FULL);
      int qseq = 0;
      for (int seq = 0; !dead; ++seq) {
        PsTask t;
        if (!read_task(seq, t, true)) {
          give_up(1, seq, qseq);
          break;
        }
        if (t.vn < 0) break;
        const int rows = min(t.q_len * G - t.row0, 128);
        const int first_slot = t.row0 / G, nslots = (t.row0 + rows - 1) / G - first_slot + 1;  // <= 128
        // request ids of this pass's slots (the previous entry's ids are no longer needed: its copies were issued)
        for (int i = lane; i < nslots; i += 32) {
          const int64_t part = (int64_t)t.q_off + first_slot + i;
          if (part >= 0 && part < p.num_partial_rows) {
            cp_async4(req_sm + i * 4, p.q_entries + part);
          } else {
            flag_error(FT_DEV_BAD_ROW_INDEX);
            asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(req_sm + i * 4), "r"(-1) : "memory");
          }
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncwarp();
        bool in_order = false;
        if (tp.q_box_rows > 0 && rows >= 64) {  // small tasks fetch exactly their rows, request by request
          const int req0 = req_of[0];
          bool mine = true;
          for (int i = lane; i < nslots; i += 32) mine &= req_of[i] == req0 + i;
          in_order = __all_sync(0xffffffffu, mine) && req0 >= 0 && (int64_t)req0 + nslots <= p.batch;
        }
        if (!warp_wait(bar(C::Q_EMPTY), ((uint32_t)qseq & 1u) ^ 1u)) {
          give_up(11, seq, qseq);
          break;
        }
        ++qseq;
        if (in_order) {
          // consecutive requests: the tile is one strided block of the Q tensor, two boxes of [128 / G requests][G heads][64]
          if (lane == 0) {
            mbar_arrive_expect_tx(full, 32768u);  // full boxes: rows past the task's requests are dead rows
            tma_load_3d(q_sm, &tp.q_map_tile, 0, t.kvh * G, req_of[0], full);
            tma_load_3d(q_sm + 16384, &tp.q_map_tile, 64, t.kvh * G, req_of[0], full);
          } else {
            mbar_arrive(full);
          }
        } else if (tp.q_box_rows > 0) {
          // the G rows of a request are adjacent heads of one Q row: boxes of up to 8 rows x 64 elements per half.
          // G divides 128 here, so a pass starts on a request and a box never straddles an 8-row group.
          const int br = tp.q_box_rows;
          uint32_t bytes = 0;
          for (int i = lane; i < nslots; i += 32) {
            const int req = req_of[i];
            if (req >= 0 && req < p.batch)
              bytes += (uint32_t)G * 256u;
            else if ((int64_t)t.q_off + first_slot + i >= 0 && (int64_t)t.q_off + first_slot + i < p.num_partial_rows)
              flag_error(FT_DEV_BAD_Q_INDEX);
          }
          mbar_arrive_expect_tx(full, bytes);
          for (int i = lane; i < nslots; i += 32) {
            const int req = req_of[i];
            if (req >= 0 && req < p.batch) {
              for (int sub = 0; sub < G; sub += br) {
                const int rr = i * G + sub;
                const uint32_t dst = q_sm + (uint32_t)((rr >> 3) * 1024 + (rr & 7) * 128);
                tma_load_3d(dst, &tp.q_map, 0, t.kvh * G + sub, req, full);
                tma_load_3d(dst + 16384, &tp.q_map, 64, t.kvh * G + sub, req, full);
              }
            }
          }
        } else {
          const int ld_c = lane & 15, ld_r = lane >> 4;
          const int fill = (rows + 7) & ~7;  // whole 8-row groups; rows past the end are dead and may hold anything finite
          for (int ps = 0; ps < 64; ++ps) {
            const int rr = ps * 2 + ld_r;
            if (rr >= fill) break;
            const int prow = t.row0 + rr;
            int64_t src = -1;
            if (rr < rows) {
              const int slot = prow / G, gg = prow - slot * G;
              const int req = req_of[slot - first_slot];
              if (req >= 0 && req < p.batch)
                src = (int64_t)req * p.q_s0 + (int64_t)(t.kvh * G + gg) * p.q_s1 + ld_c * 8;
              else if ((int64_t)t.q_off + slot >= 0 && (int64_t)t.q_off + slot < p.num_partial_rows)
                flag_error(FT_DEV_BAD_Q_INDEX);
            }
            cp_async16(q_sm + tc_swz(rr, ld_c, 16384), reinterpret_cast<const T*>(p.q) + (src >= 0 ? src : 0), src >= 0);
          }
          proxy_fence();  // rows past the end were zero-filled with plain shared stores
          mbar_arrive_on_cp_async(full);
          cp_async_wait<0>();
        }
      }
    }
  }

  // ---- release tensor memory; the last CTA to get here re-arms the claim counter for the next launch
  tc_fence_before();
  __syncthreads();
  if (usable && warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(C::TMEM_COLS) : "memory");
  }
  FT_TL_END(3);
  if (tid == 0) {
    __threadfence();
    const unsigned int done = atomicAdd(tp.sched + 1, 1u);
    if (done == gridDim.x - 1) {
      tp.sched[0] = 0u;
      tp.sched[1] = 0u;
      __threadfence();
    }
  }
}

}  // namespace ft
