// Stage 1 for tasks with many query rows (shared prefixes): 5th-generation
// tensor cores (tcgen05.mma) with accumulators in tensor memory.
//
// One CTA (128 threads) per (vnode, kv head) handles up to 128 packed query
// rows (requests x GQA group) per pass against the vnode's KV chunk, 64 tokens
// per tile:
//
//   S[128 x 64]   = Q[128 x 128] . K_tile^T        tcgen05.mma, A and B K-major
//   O[128 x 128] += P[128 x 64]  . V_tile          tcgen05.mma, B MN-major
//
// Q, K, V and P sit in shared memory in the canonical 128-byte-swizzled
// operand layout (64-element blocks, 8-row groups of 1024 bytes); K/V rows are
// gathered by row id with 16-byte cp.async copies (the KV pool is token
// granular, so there is no dense box for a tiled TMA copy).  S and O live in
// TMEM (two 64-column S buffers and 128 columns of O in a 256-column allocation;
// two CTAs fit on an SM).  The scores of tile j+1 are issued before the softmax
// of tile j starts, so the tensor pipe works while the CUDA cores do the
// exponentials; P.V of tile j follows as soon as P is written.  Thread t owns query row t = TMEM lane t: it reads its row of S with
// tcgen05.ld, does the online softmax without any cross-lane traffic, writes
// its row of P, and rescales its row of O in TMEM only when the running
// maximum has grown by more than 2^8 (the exponent offset may lag the true
// maximum; sum and output use the same offset, so the result is unchanged).
// A fifth warp does nothing but issue the MMAs (one elected lane), so that the
// descriptor arithmetic and the issue latency stay off the softmax warps'
// critical path; completion comes back through mbarriers (tcgen05.commit)
// that every thread polls with a bounded wait.
//
// Arithmetic conventions as in the other stage-1 kernels
// (kernel_bench/fasttree.py:360-413): fp32 scores scaled after the dot product,
// probabilities rounded to the storage type before P.V, normalised partial
// output, lse = log(sum) + max.
#pragma once

#include <type_traits>

#include "ft_common.cuh"
#include "ft_stage1_mma.cuh"
#include "ft_stage1_narrow.cuh"

namespace ft {

struct TcCfg {
  static constexpr int THREADS = 160;  // warps 0-3: one query row per thread (loads, softmax); warp 4: issues the MMAs
  static constexpr int ROWS = 128;    // query rows per pass (UMMA M)
  static constexpr int TILE = 64;     // tokens per tile (UMMA N of S, K of P.V)
  static constexpr int D = 128;
  static constexpr int Q_OFF = 0;                     // 2 blocks x [128 rows][128 B]
  static constexpr int K_OFF = 32768;                 // 2 buffers x (2 blocks x [64 tok][128 B])
  static constexpr int V_OFF = K_OFF + 2 * 16384;
  static constexpr int P_OFF = V_OFF + 2 * 16384;     // [128 rows][128 B]
  static constexpr int IDX_OFF = P_OFF + 16384;       // 3 slots x 64 row ids
  static constexpr int BAR_OFF = IDX_OFF + 3 * 64 * 4;   // two mbarriers: scores ready, P.V done
  static constexpr int TMEM_SLOT_OFF = BAR_OFF + 16;
  static constexpr int SMEM_BYTES = TMEM_SLOT_OFF + 8;
  static constexpr int TMEM_COLS = 256;
  static constexpr int S_COL = 0, O_COL = 128;           // S is double-buffered: columns [0,64) and [64,128)
  static constexpr int WAIT_LIMIT = 1 << 16;   // probes of mbarrier.try_wait (each suspends for a while) before giving up
};

// canonical K-major / MN-major 128B-swizzled position of 16-byte chunk `c16` (0..15 over 256 B)
// of row `r` in an operand whose 64-element blocks are `block_bytes` apart
__device__ __forceinline__ uint32_t tc_swz(int r, int c16, int block_bytes) {
  return static_cast<uint32_t>((c16 >> 3) * block_bytes + (r >> 3) * 1024 + (r & 7) * 128 + (((c16 & 7) ^ (r & 7)) << 4));
}

__device__ __forceinline__ uint64_t tc_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) /* descriptor version */ |
         (2ull << 61) /* SWIZZLE_128B */;
}

// kind::f16 instruction descriptor: fp32 accumulate, A K-major, dense
template <typename T>
__device__ __forceinline__ uint32_t tc_idesc(int m, int n, bool b_mn_major) {
  const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// Polls the mbarrier; gives up after WAIT_LIMIT probes (the caller then flags the error and unwinds).
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity) {
  for (int it = 0; it < TcCfg::WAIT_LIMIT; ++it) {
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

template <typename T>
__device__ __forceinline__ void tc_body(const Stage1Params& p, uint8_t* smem, const int vn, const int kvh) {
  using C = TcCfg;
  const uint32_t sm = smem_u32(smem);
  const uint32_t q_sm = sm + C::Q_OFF, p_sm = sm + C::P_OFF, idx_sm = sm + C::IDX_OFF;
  const uint32_t bar_s = sm + C::BAR_OFF, bar_o = bar_s + 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::TMEM_SLOT_OFF);

  const int tid = threadIdx.x, warp = tid >> 5;
  const bool mma_warp = warp == 4;   // this warp only issues MMAs and takes part in the barriers
  const bool mma_lane = tid == 128;
  const int q_off = p.q_offs[vn], q_len = p.q_lens[vn];
  const int kv_off = p.kv_offs[vn], kv_len = max(p.kv_lens[vn], 0);
  const int G = p.group;
  const int rows = q_len * G;
  if (rows <= 0) return;
  if ((sm & 1023u) != 0u) {  // the swizzled operand layout needs a 1024-byte aligned window
    if (tid == 0) flag_error(FT_DEV_WAIT_TIMEOUT);
    return;
  }
  const float scale2 = p.sm_scale * 1.4426950408889634f;
  const int ntiles = (kv_len + C::TILE - 1) / C::TILE;
  const int ld_c = tid & 15, ld_r = tid >> 4;
  // row ids past the end of the table are a plan error: flag once, treat those tokens as padding
  const int64_t readable = p.kv_entries_len - (int64_t)kv_off;
  const int id_lim = kv_off < 0 ? 0 : (int)(readable < (int64_t)kv_len ? (readable < 0 ? 0 : readable) : kv_len);
  if (id_lim < kv_len && tid == 0) flag_error(FT_DEV_BAD_KV_INDEX);
  const uint32_t row_lim = (uint32_t)(p.kv_rows < 0x7fffffffLL ? p.kv_rows : 0x7fffffffLL);
  // this thread's 8 (row, chunk) positions inside a 64-token operand tile
  const uint32_t tile_pos = tc_swz(ld_r, ld_c, 8192);
  const T* __restrict__ kbase = reinterpret_cast<const T*>(p.k) + (int64_t)kvh * p.k_s1 + ld_c * 8;
  const T* __restrict__ vbase = reinterpret_cast<const T*>(p.v) + (int64_t)kvh * p.v_s1 + ld_c * 8;

  // ---- one-time set-up: barrier, tensor memory
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_s) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_o) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(sm + C::TMEM_SLOT_OFF),
                 "r"(C::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);  // this warp's 32-lane quadrant
  const uint32_t idesc_s = tc_idesc<T>(128, C::TILE, false);
  const uint32_t idesc_o = tc_idesc<T>(128, C::D, true);
  uint32_t waits_s = 0, waits_o = 0;  // phases consumed on each barrier (same value in every thread)
  bool dead = false;

  // row ids of tile t -> ring slot t % 3 (threads 0..63, one id each; joins the open cp.async group)
  auto issue_ids = [&](int t) {
    if (tid < C::TILE) {  // (warps 0 and 1)
      const int pos = t * C::TILE + tid;
      if (pos < id_lim) cp_async4(idx_sm + ((t % 3) * C::TILE + tid) * 4, p.kv_entries + kv_off + pos);
    }
  };
  // rows of tile t of K (or V) -> buffer `buf_sm`
  auto issue_rows = [&](int t, uint32_t buf_sm, const T* base, int64_t stride) {
    if (mma_warp) return;
    // all eight row ids first (independent shared-memory loads), then the copies
    const int* ring = reinterpret_cast<const int*>(smem + C::IDX_OFF) + (t % 3) * C::TILE + ld_r;
    const int pos0 = t * C::TILE + ld_r;
    uint32_t row[8];
#pragma unroll
    for (int ps = 0; ps < 8; ++ps) row[ps] = pos0 + ps * 8 < id_lim ? (uint32_t)ring[ps * 8] : 0xffffffffu;
    bool bad = false;
#pragma unroll
    for (int ps = 0; ps < 8; ++ps) {  // rows ld_r, ld_r + 8, ...: same swizzle phase, 1024 bytes apart
      const bool ok = row[ps] < row_lim;  // padding (0xffffffff), negative and too-large ids all fail this test
      bad |= !ok && pos0 + ps * 8 < id_lim;
      cp_async16(buf_sm + tile_pos + ps * 1024, base + (int64_t)(ok ? row[ps] : 0u) * stride, ok);
    }
    if (bad) flag_error(FT_DEV_BAD_KV_INDEX);
  };
  auto k_buf = [&](int t) { return sm + C::K_OFF + (t & 1) * 16384; };
  auto v_buf = [&](int t) { return sm + C::V_OFF + (t & 1) * 16384; };

  for (int row0 = 0; row0 < rows && !dead; row0 += C::ROWS) {
    // ---- Q tile (gathered by request id), row ids of the first tiles
#pragma unroll 4
    for (int ps = 0; ps < (mma_warp ? 0 : 16); ++ps) {
      const int r = ps * 8 + ld_r;
      const int prow = row0 + r;
      int64_t src = -1;
      if (prow < rows) {
        const int slot = prow / G, gg = prow - slot * G;
        const int64_t part = (int64_t)q_off + slot;
        if (part >= 0 && part < p.num_partial_rows) {
          const int req = p.q_entries[part];
          if (req >= 0 && req < p.batch)
            src = (int64_t)req * p.q_s0 + (int64_t)(kvh * G + gg) * p.q_s1 + ld_c * 8;
          else
            flag_error(FT_DEV_BAD_Q_INDEX);
        } else {
          flag_error(FT_DEV_BAD_ROW_INDEX);
        }
      }
      cp_async16(q_sm + tc_swz(r, ld_c, 16384), reinterpret_cast<const T*>(p.q) + (src >= 0 ? src : 0), src >= 0);
    }
    for (int t = 0; t < 3; ++t)
      if (t < ntiles) issue_ids(t);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    // K_0, V_0, K_1 and wait for them (start-up; steady state overlaps these with the MMAs)
    if (ntiles > 0) {
      issue_rows(0, k_buf(0), kbase, p.k_s0);
      issue_rows(0, v_buf(0), vbase, p.v_s0);
      if (ntiles > 1) issue_rows(1, k_buf(1), kbase, p.k_s0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    proxy_fence();
    tc_fence_before();
    __syncthreads();

    auto issue_s = [&](int t) {  // S[t & 1] = Q K_t^T : 8 k-steps of 16 along head_dim
      const uint32_t kb = k_buf(t);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t a = tc_desc(q_sm + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024);
        const uint64_t b = tc_desc(kb + (ks >> 2) * 8192 + (ks & 3) * 32, 16, 1024);
        tc_mma(tmem + C::S_COL + (t & 1) * C::TILE, a, b, idesc_s, ks > 0);
      }
    };
    auto issue_pv = [&](int t) {  // O += P V_t : 4 k-steps of 16 tokens
      const uint32_t vb = v_buf(t);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint64_t a = tc_desc(p_sm + ks * 32, 16, 1024);
        const uint64_t b = tc_desc(vb + ks * 2048, 8192, 1024);
        tc_mma(tmem + C::O_COL, a, b, idesc_o, (t > 0 || ks > 0) ? 1u : 0u);
      }
    };

    if (mma_lane && ntiles > 0) {
      tc_fence_after();
      issue_s(0);
      tc_commit(bar_s);
    }
    float m_used = -INFINITY, l_run = 0.f;

#ifdef FT_TC_PROFILE
    long long prof[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    long long t_prev = clock64();
#define FT_MARK(i) { const long long t_now = clock64(); prof[i] += t_now - t_prev; t_prev = t_now; }
#else
#define FT_MARK(i)
#endif
    for (int j = 0; j < ntiles; ++j) {
      // K_{j+1} (copied during the previous iteration) must be visible before S_{j+1} is issued
      cp_async_wait<1>();
      proxy_fence();
      FT_MARK(0)
      const bool ok_s = tc_wait(bar_s, waits_s & 1);  // S_j ready
      ++waits_s;
      FT_MARK(1)
      if (__syncthreads_or(!ok_s)) {
        if (tid == 0) flag_error(FT_DEV_WAIT_TIMEOUT);
        dead = true;
        break;
      }
      tc_fence_after();
      FT_MARK(8)
      if (mma_lane && j + 1 < ntiles) {  // the tensor pipe computes the next scores during this softmax
        issue_s(j + 1);
        tc_commit(bar_s);
      }
      bool ok_o = true;
      if (!mma_warp) {
      // K buffer of tile j is free again (S_j done)
      if (j + 2 < ntiles) issue_rows(j + 2, k_buf(j + 2), kbase, p.k_s0);
      FT_MARK(9)
      if (j + 3 < ntiles) issue_ids(j + 3);
      cp_async_commit();
      FT_MARK(2)

      // ---- softmax of this thread's row (scores stay unscaled until the exponent: one FMA per element)
      float s[64];
      const uint32_t s_col = t_lane + C::S_COL + (j & 1) * C::TILE;
      tmem_ld32(s_col, *reinterpret_cast<float(*)[32]>(&s[0]));
      tmem_ld32(s_col + 32, *reinterpret_cast<float(*)[32]>(&s[32]));
      const int valid = kv_len - j * C::TILE;  // columns >= valid are padding (last tile only)
      if (valid < C::TILE) {
#pragma unroll
        for (int c = 0; c < 64; ++c)
          if (c >= valid) s[c] = -INFINITY;
      }
      float mx = fmaxf(s[0], s[1]);
#pragma unroll
      for (int c = 2; c < 64; c += 2) asm("max.f32 %0, %0, %1, %2;" : "+f"(mx) : "f"(s[c]), "f"(s[c + 1]));
      mx *= scale2;  // scale2 > 0
      float corr = 1.f;
      bool grow = false;
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
      float2 sum2 = make_float2(0.f, 0.f);
      uint32_t w[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float2 x = __ffma2_rn(make_float2(s[2 * i], s[2 * i + 1]), sc2, no2);
        x.x = fast_exp2(x.x);
        x.y = fast_exp2(x.y);
        sum2 = __fadd2_rn(sum2, x);
        w[i] = pack2<T>(x.x, x.y);
      }
      l_run += sum2.x + sum2.y;
      FT_MARK(3)

      // P.V of the previous tile must be done before P and O are touched
      if (j > 0) {
        ok_o = tc_wait(bar_o, waits_o & 1);
        ++waits_o;
        tc_fence_after();
        if (__any_sync(0xffffffffu, grow)) {  // rescale this warp's rows of O in tensor memory
#pragma unroll
          for (int cb = 0; cb < 4; ++cb) {
            float o[32];
            tmem_ld32(t_lane + C::O_COL + cb * 32, o);
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] *= corr;
            tmem_st32(t_lane + C::O_COL + cb * 32, o);
          }
          tmem_wait_st();
        }
      }
      FT_MARK(4)
      // V buffer of tile j-1 is free (its P.V is done)
      if (j + 1 < ntiles) issue_rows(j + 1, v_buf(j + 1), vbase, p.v_s0);
      cp_async_commit();
      const uint32_t p_row = p_sm + (tid >> 3) * 1024 + (tid & 7) * 128;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(p_row + ((c8 ^ (tid & 7)) << 4)),
                     "r"(w[4 * c8]), "r"(w[4 * c8 + 1]), "r"(w[4 * c8 + 2]), "r"(w[4 * c8 + 3])
                     : "memory");
      FT_MARK(5)
      cp_async_wait<2>();  // V_j (copied during the previous iteration) has landed
      proxy_fence();       // P (generic stores) and V_j (cp.async) become visible to the tensor core
      tc_fence_before();   // orders this thread's tcgen05.ld/st before the barrier
      } else if (j > 0) {
        ++waits_o;  // the MMA warp does not wait for P.V here but must keep the phase count of the barrier
      }
      if (__syncthreads_or(!ok_o)) {
        if (tid == 0) flag_error(FT_DEV_WAIT_TIMEOUT);
        dead = true;
        break;
      }
      FT_MARK(6)
      if (mma_lane) {
        tc_fence_after();
        issue_pv(j);
        tc_commit(bar_o);
      }
      FT_MARK(7)
    }
#ifdef FT_TC_PROFILE
    if (blockIdx.x == 0 && (tid == 0 || tid == 37))
      printf("tc profile tid %d tiles %d: cpwait+top %lld | barS %lld | sync+issueS+loadK %lld | tmem ld+softmax %lld | "
             "barO+rescale %lld | loadV+Pstore %lld | wait2+fence+sync %lld | issuePV %lld | syncA %lld | issueK %lld (cycles per tile)\n",
             tid, ntiles, prof[0] / ntiles, prof[1] / ntiles, prof[2] / ntiles, prof[3] / ntiles, prof[4] / ntiles,
             prof[5] / ntiles, prof[6] / ntiles, prof[7] / ntiles, prof[8] / ntiles, prof[9] / ntiles);
#endif
    if (dead) break;

    // ---- epilogue: wait for the last P.V, normalise, write this thread's partial row
    bool ok = true;
    if (ntiles > 0) {
      ok = tc_wait(bar_o, waits_o & 1);  // the last P.V
      ++waits_o;
    }
    if (__syncthreads_or(!ok)) {
      if (tid == 0) flag_error(FT_DEV_WAIT_TIMEOUT);
      dead = true;
      break;
    }
    tc_fence_after();
    const int prow = row0 + tid;
    const bool live = !mma_warp && prow < rows;
    int slot = 0, gg = 0;
    if (live) {
      slot = prow / G;
      gg = prow - slot * G;
    }
    const int64_t part = (int64_t)q_off + slot;
    const bool store = live && part >= 0 && part < p.num_partial_rows;
    const int head = kvh * G + gg;
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    float4* dst = reinterpret_cast<float4*>(p.mid_o + part * p.mo_s0 + (int64_t)head * p.mo_s1);
#pragma unroll
    for (int cb = 0; cb < 4; ++cb) {
      float o[32];
      if (ntiles > 0 && !mma_warp) {
        tmem_ld32(t_lane + C::O_COL + cb * 32, o);  // warp-collective: every lane of the warp takes part
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) o[c] = 0.f;
      }
      if (store) {
#pragma unroll
        for (int c = 0; c < 8; ++c)
          dst[cb * 8 + c] = make_float4(o[4 * c] * inv, o[4 * c + 1] * inv, o[4 * c + 2] * inv, o[4 * c + 3] * inv);
      }
    }
    if (store) p.mid_lse[part * p.ml_s0 + head] = l_run > 0.f ? (m_used + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
    tc_fence_before();
    __syncthreads();  // S/O columns and the operand buffers are reused by the next pass
    tc_fence_after();
  }

  // ---- release tensor memory
  cp_async_wait<0>();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(C::TMEM_COLS) : "memory");
  }
}

template <typename T>
__global__ void __launch_bounds__(TcCfg::THREADS, 2) stage1_tc_kernel(Stage1Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  int vn, kvh;
  task_of_block(p, blockIdx.x, vn, kvh);
  tc_body<T>(p, smem, vn, kvh);
}

// Both task families in one grid (head_dim 128): the first `p.node_split` vnodes of the launch are
// many-row tasks for the tcgen05 body, the rest few-row tasks for the swapped-operand body.  The
// tensor-bound and the memory-bound CTAs then share the SMs instead of running back to back.
template <typename T>
__global__ void __launch_bounds__(TcCfg::THREADS, 2) stage1_fused_kernel(Stage1Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  int vn, kvh;
  task_of_block(p, blockIdx.x, vn, kvh);  // blocks [0, node_split * heads) are the many-row tasks: they start first
  if (vn - p.node_offset < p.node_split) {
    tc_body<T>(p, smem, vn, kvh);
  } else {
    if (threadIdx.x >= 128) return;  // the few-row body is written for four warps
    narrow_dispatch<T, 128>(p, smem, vn, kvh);
  }
}

}  // namespace ft
