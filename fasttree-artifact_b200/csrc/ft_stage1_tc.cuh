// Stage 1 for tasks with many query rows (shared prefixes): 5th-generation
// tensor cores (tcgen05.mma) with accumulators in tensor memory, K/V tiles
// staged by TMA, warp-specialised.
//
// One CTA (256 threads) per (vnode, kv head) handles up to 128 packed query
// rows (requests x GQA group) per pass against the vnode's KV chunk, 64 tokens
// per tile:
//
//   S[128 x 64]   = Q[128 x 128] . K_tile^T        tcgen05.mma, A and B K-major
//   O[128 x 128] += P[128 x 64]  . V_tile          tcgen05.mma, B MN-major
//
// Roles
//   warps 0-3  softmax: thread t owns query row t = TMEM lane t.  It reads its
//              row of S with tcgen05.ld, does the online softmax with no
//              cross-lane traffic, writes its row of P over the first half of
//              the S buffer it has just read (tcgen05.st; P.V takes its A
//              operand from tensor memory) and rescales its row of O in TMEM
//              only when the running maximum grew by more than 2^8 (the
//              exponent offset may lag the true maximum; sum and output use the
//              same offset, so the result is unchanged).  Only that rescale
//              waits for the previous tile's P.V.
//              At the end it stages its normalised row in shared memory and
//              each warp writes its 32 rows to the partial buffer with full-row
//              (512-byte) store instructions.
//   warp 4     MMA issue (one elected lane): S_t is issued before the softmax of
//              tile t-1 has finished (two S buffers in TMEM), P.V of tile t-1
//              as soon as its P is written.
//   warp 5     K loads.  A tile whose 64 row ids are consecutive is fetched
//              with two tiled TMA copies (cp.async.bulk.tensor, 128-byte
//              swizzle, no multicast) straight into the operand layout; any
//              other tile (scattered pool slots, the ragged last tile) is
//              gathered with 16-byte cp.async copies.  Row ids reach a small
//              shared ring with cp.async two tiles ahead.
//   warps 6-7  Q gather (by request id), concurrent with the first K loads:
//              when G is a power of two, two TMA boxes for the whole tile if the
//              request ids are consecutive, else one box per request (its G
//              adjacent heads); 16-byte cp.async copies otherwise.
//   warp 6     then loads the V tiles the same way as warp 5 loads K, with the
//              row ids in registers (two per lane, one tile ahead), so the two
//              loaders share nothing and a gathered tile costs each of them
//              half of the copies.
// The two warpgroups trade registers at start-up (setmaxnreg): the kernel
// launches at 128 registers per thread, so that a CTA takes exactly two
// equal-sized warps per scheduler partition and two CTAs always fit on an SM
// whatever mix of roles they run; the softmax warps then grow to 184 and the
// others shrink to 72.
// Hand-offs are mbarriers (full/empty per K, V and S buffer, P written, P.V
// done), each with exactly one waiting role; every wait is bounded and unwinds
// the CTA through an abort flag.
//
// Q, K and V use the canonical 128-byte-swizzled operand layout (64-element
// blocks, 8-row groups of 1024 bytes).  TMEM: two 64-column S buffers (P of a
// tile, 16-bit, takes the first 32 columns of its S buffer) and 128 columns of O
// in a 256-column allocation, so two CTAs share an SM.
// S buffer b is written again by S_{t+2} while it may still hold P_t.  Nothing
// but issue order protects it: every MMA of this kernel has the same shape
// (M 128, N 64, K 16 - P.V is issued as two 64-column halves of O for that
// reason), and same-shape MMAs of one CTA execute in the order they were issued.
//
// Arithmetic conventions as in the other stage-1 kernels
// (kernel_bench/fasttree.py:360-413): fp32 scores scaled after the dot product,
// probabilities rounded to the storage type before P.V, normalised partial
// output, lse = log(sum) + max.
#pragma once

#include <type_traits>

#include "ft_async.cuh"
#include "ft_common.cuh"
#include "ft_stage1_mma.cuh"
#include "ft_stage1_narrow.cuh"
#include "ft_stage1_stream.cuh"

namespace ft {

struct TcCfg {
  static constexpr int THREADS = 256;
  static constexpr int ROWS = 128;    // query rows per pass (UMMA M)
  static constexpr int TILE = 64;     // tokens per tile (UMMA N of S, K of P.V)
  static constexpr int D = 128;
  static constexpr int Q_OFF = 0;                     // 2 blocks x [128 rows][128 B]
  static constexpr int NSK = 3;                       // K ring: one stage more than V, K being needed a softmax earlier
  static constexpr int K_OFF = 32768;                 // NSK buffers x (2 blocks x [64 tok][128 B])
  static constexpr int V_OFF = K_OFF + NSK * 16384;   // 2 buffers, same shape
  static constexpr int IDX_SLOTS = 3;
  static constexpr int IDX_OFF = V_OFF + 2 * 16384;   // IDX_SLOTS x 64 row ids
  static constexpr int BAR_OFF = IDX_OFF + IDX_SLOTS * 64 * 4;
  static constexpr int NBARS = 18;
  static constexpr int ABORT_OFF = BAR_OFF + NBARS * 8;
  static constexpr int TMEM_SLOT_OFF = ABORT_OFF + 4;
  static constexpr int SMEM_BYTES = TMEM_SLOT_OFF + 4;
  static constexpr int TMEM_COLS = 256;
  static constexpr int S_COL = 0, O_COL = 128;        // S is double-buffered: columns [0,64) and [64,128)
  static constexpr int WAIT_LIMIT = 1 << 16;          // probes of mbarrier.try_wait before a wait gives up
  // barrier indices
  static constexpr int K_FULL = 0, K_EMPTY = 3, V_FULL = 6, V_EMPTY = 8, S_FULL = 10, P_FULL = 12, PV_DONE = 14,
                       Q_FULL = 16;
  static constexpr int OUT_STRIDE = 528;              // bytes between staged output rows (512 + 16: conflict-free 16-byte stores)
  static constexpr int REGS_SOFTMAX = 184, REGS_OTHER = 72;
  static constexpr int REGS_WORKER = 232;             // few-row workers of the fused kernel: four warps, the other four leave
};
static_assert(TcCfg::SMEM_BYTES <= 115712, "two CTAs must fit in one SM's shared memory");
static_assert(128 * TcCfg::OUT_STRIDE <= TcCfg::IDX_OFF, "the staged output rows reuse the Q, K and V buffers");
static_assert((TcCfg::REGS_SOFTMAX + TcCfg::REGS_OTHER) * 128 <= 2 * 128 * 128, "register trade must balance");

template <int N>
__device__ __forceinline__ void reg_grow() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_shrink() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(N)); }

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
// O += A . B with A in tensor memory (lane = row, two 16-bit elements per column, K-major) and B in shared memory
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
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
// 32 columns without the wait: for callers that issue several loads and wait once (tmem_wait_ld)
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, float (&v)[32]) {
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
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
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

// 2^x on the FMA / ALU pipes: floor(x) is peeled off with a round-down add of 1.5 * 2^23 (the integer lands in the
// low mantissa bits), a cubic gives 2^frac to 9e-5 relative (far below the rounding of P to its 16-bit type), and the
// integer is added back into the exponent field.  Exactly 0 for x <= -126 (masked scores are -inf).  Used for a
// share of the softmax's exponentials where the MUFU unit (ex2.approx: a quarter-rate pipe) is the limiter.
__device__ __forceinline__ float exp2_fma(float x) {
  const float xc = fmaxf(x, -126.f);
  float t;
  asm("add.rm.ftz.f32 %0, %1, %2;" : "=f"(t) : "f"(xc), "f"(12582912.f));
  const float f = xc - (t - 12582912.f);
  const float p = fmaf(f, fmaf(f, fmaf(f, 0.07706569f, 0.22764646f), 0.69511646f), 1.f);
  const float r = __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
  return x > -126.f ? r : 0.f;
}
#ifndef FT_EXP2_FMA_EVERY
#define FT_EXP2_FMA_EVERY 0  // n > 0: every n-th pair of a row's 32 score pairs takes exp2_fma instead of ex2.approx
#endif

// Bounded wait for the phase of `bar` with the given parity.  Gives up after WAIT_LIMIT probes or as soon as
// another role has raised the CTA's abort flag; the caller then raises the flag itself and unwinds.
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (int it = 0; it < TcCfg::WAIT_LIMIT; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((it & 15) == 15 && *abort_flag != 0) return false;
  }
  return false;
}

// Row-by-row gather of one 64-token operand tile (scattered pool slots, the ragged last tile): 16-byte copies that
// zero-fill invalid rows themselves, so the loop has no branch.  Kept out of line: tiles of consecutive rows - every
// tile of the benchmark shapes - never come here, and their loaders' code stays as small as it was.
// ids in shared memory (K loader); returns true when a row id inside the chunk was out of range
template <typename T>
__device__ __noinline__ bool tc_gather_tile_smem(uint32_t buf, const T* base, int64_t stride, const int* ids, int t, int id_lim,
                                                 uint32_t row_lim, int lane) {
  const int c = lane & 15;
  bool bad = false;
#pragma unroll 4
  for (int i = 0; i < 32; ++i) {
    const int r = (lane >> 4) + 2 * i, pos = t * TcCfg::TILE + r;
    const uint32_t row = pos < id_lim ? (uint32_t)ids[r] : 0xffffffffu;
    const bool ok = row < row_lim;  // padding (0xffffffff), negative and too-large ids all fail this test
    bad |= !ok && pos < id_lim;
    cp_async16_zfill(buf + tc_swz(r, c, 8192), base + (int64_t)(ok ? row : 0u) * stride + c * 8, ok);
  }
  return bad;
}
// ids in registers, two per lane: row r is slot r >> 5 of lane r & 31 (V loader)
template <typename T>
__device__ __noinline__ bool tc_gather_tile_regs(uint32_t buf, const T* base, int64_t stride, int id0, int id1, int t, int id_lim,
                                                 uint32_t row_lim, int lane) {
  const int c = lane & 15;
  bool bad = false;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#pragma unroll 4
    for (int i = 0; i < 16; ++i) {
      const int r = (lane >> 4) + 2 * i + 32 * h, pos = t * TcCfg::TILE + r;
      const int id = __shfl_sync(0xffffffffu, h == 0 ? id0 : id1, r & 31);
      const uint32_t row = pos < id_lim ? (uint32_t)id : 0xffffffffu;
      const bool ok = row < row_lim;
      bad |= !ok && pos < id_lim;
      cp_async16_zfill(buf + tc_swz(r, c, 8192), base + (int64_t)(ok ? row : 0u) * stride + c * 8, ok);
    }
  }
  return bad;
}

template <typename T>
__device__ __forceinline__ void tc_body(const TcParams& tp, uint8_t* smem, const int vn, const int kvh) {
  using C = TcCfg;
  const Stage1Params& p = tp.p;
  const uint32_t sm = smem_u32(smem);
  const uint32_t q_sm = sm + C::Q_OFF, idx_sm = sm + C::IDX_OFF, bars = sm + C::BAR_OFF;
  const uint32_t req_sm = sm + C::V_OFF;  // request ids of a pass's rows, staged before the pass's first V load
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::ABORT_OFF);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::TMEM_SLOT_OFF);
  auto bar = [&](int i) { return bars + 8u * i; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if ((sm & 1023u) != 0u) {  // the swizzled operand layout needs a 1024-byte aligned window
    if (tid == 0) flag_error(FT_DEV_WAIT_TIMEOUT);
    return;
  }
  // The kernel may have been scheduled while the preceding kernel of the stream is still running (programmatic
  // dependent launch).  CTAs of the first wave - the only ones that can be resident that early - do their on-chip
  // set-up first and wait for the preceding kernel after it, so launch and set-up hide under that kernel's tail;
  // later CTAs find the wait already satisfied and issue their task's table reads before the set-up instead, which
  // hides the reads' latency as well.
  uint32_t num_sms;
  asm("mov.u32 %0, %%nsmid;" : "=r"(num_sms));
  const bool first_wave = blockIdx.x < 2u * num_sms;
  int q_off = 0, q_len = 0, kv_off = 0, kv_len = 0;
  auto read_task = [&]() {
    wait_for_prior_grid();
    q_off = p.q_offs[vn];
    q_len = p.q_lens[vn];
    kv_off = p.kv_offs[vn];
    kv_len = max(p.kv_lens[vn], 0);
  };
  if (!first_wave) read_task();

  // ---- one-time set-up: barriers, tensor memory
  if (tid == 32 && tp.has_tma) {  // the first TMA copy would otherwise pay for fetching its descriptor
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tp.k_map)) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tp.v_map)) : "memory");
    if (tp.q_box_rows > 0) {
      asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tp.q_map_tile)) : "memory");
      asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tp.q_map)) : "memory");
    }
  }
  if (tid == 0) {
    for (int b = 0; b < C::NSK; ++b) {
      mbar_init(bar(C::K_FULL + b), 32);   // the loader's lanes
      mbar_init(bar(C::K_EMPTY + b), 1);   // tcgen05.commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar(C::V_FULL + b), 32);
      mbar_init(bar(C::V_EMPTY + b), 1);
      mbar_init(bar(C::S_FULL + b), 1);
      // P of tile g is announced on barrier g & 1: a thread that is a tile ahead of the slowest one arrives on the
      // other barrier, never twice in one phase
      mbar_init(bar(C::P_FULL + b), 128);  // the softmax threads
      mbar_init(bar(C::PV_DONE + b), 1);
    }
    mbar_init(bar(C::Q_FULL), 64);  // the Q-gather threads
    *abort_flag = 0;
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
  if (first_wave) read_task();
  if (tid == 0) FT_TL_MARK(0);
  const int G = p.group;
  const int rows = q_len * G;  // <= 0: nothing to do but to give the tensor memory back
  const float scale2 = p.sm_scale * 1.4426950408889634f;
  const int ntiles = (kv_len + C::TILE - 1) / C::TILE;
  // row ids past the end of the table are a plan error: flag once, treat those tokens as padding
  const int id_lim = kv_ids_limit(p, kv_off, kv_len);
  const int32_t* ids_of_chunk = kv_ids_base(p, kv_off);
  if (rows > 0 && id_lim < kv_len && tid == 0) flag_error(FT_DEV_BAD_KV_INDEX);
  const uint32_t row_lim = (uint32_t)(p.kv_rows < 0x7fffffffLL ? p.kv_rows : 0x7fffffffLL);
  auto k_buf = [&](int t) { return sm + C::K_OFF + (t % C::NSK) * 16384; };
  auto v_buf = [&](int t) { return sm + C::V_OFF + (t & 1) * 16384; };

  // Tiles are numbered g = 0, 1, 2, ... across passes; tile g uses V / S buffer g & 1 for the (g >> 1)-th time and K
  // buffer g % NSK for the (g / NSK)-th time, which gives every wait its barrier phase without per-barrier counters.
  int g0 = 0, pass = 0;
  bool dead = false;
  auto give_up = [&]() {
    *abort_flag = 1;
    flag_error(FT_DEV_WAIT_TIMEOUT);
    dead = true;
  };

  // end of a pass: every role is done with the buffers and the TMEM columns
  auto pass_end = [&]() {
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (*abort_flag != 0) return false;
    g0 += ntiles;  // buffers and barrier phases carry on from where this pass stopped
    ++pass;
    return true;
  };

  // Each warpgroup sets its register budget on entry to its own code, so that the budget holds for all of it.
  if (warp < 4) {
    reg_grow<C::REGS_SOFTMAX>();
    for (int row0 = 0; row0 < rows; row0 += C::ROWS) {
      {
        // ================================================================ softmax (one query row per thread)
        const uint32_t t_lane = tmem + ((uint32_t)(warp * 32) << 16);  // this warp's 32-lane quadrant
        float m_used = -INFINITY, l_run = 0.f;
        // the chunk tokens [r_lo, r_hi) this thread's row attends to: the whole chunk unless the plan narrows it
        // (a row past the end of the task attends to nothing: its results are never stored)
        int r_lo = 0, r_hi = row0 + tid < rows ? kv_len : 0;
        if (p.q_ranges != nullptr && row0 + tid < rows) {
          const int64_t part = (int64_t)q_off + (row0 + tid) / G;
          if (part >= 0 && part < p.num_partial_rows) {
            r_lo = max(p.q_ranges[2 * part], 0);
            r_hi = min(p.q_ranges[2 * part + 1], kv_len);
          }
        }
        const bool warp_has_rows = row0 + warp * 32 < rows;
        for (int j = 0; j < ntiles && !dead; ++j) {
          const int g = g0 + j, b = g & 1;
          if (!tc_wait(bar(C::S_FULL + b), (uint32_t)(g >> 1) & 1u, abort_flag)) {
            give_up();
            break;
          }
          tc_fence_after();
          if (j == 0 && tid == 0) FT_TL_COARSE_MARK(2);
          if (j == FT_TL_TILE && tid == 0) FT_TL_MARK(10);
          if (j == FT_TL_TILE + 1 && tid == 0) FT_TL_DETAIL_MARK(2);
          // A warp none of whose 32 rows attends to a token of this tile has no softmax to do: in a group of short
          // nodes (block-diagonal ranges) that is most warps in most tiles, and in a task of fewer than 128 rows the
          // warps past its end in every tile.  Its rows of P are zero (rows past the end of the task may hold
          // anything: no result of theirs is stored); the wait above still paces it, one arrival per tile.
          if (!__any_sync(0xffffffffu, r_lo < min(r_hi, (j + 1) * C::TILE) && r_hi > j * C::TILE)) {
            if (warp_has_rows) {
              float zero[32];
#pragma unroll
              for (int c = 0; c < 32; ++c) zero[c] = 0.f;
              tmem_st32(t_lane + C::S_COL + b * C::TILE, zero);
              tmem_wait_st();
            }
            tc_fence_before();
            mbar_arrive(bar(C::P_FULL + b));
            continue;
          }
          float s[64];
          const uint32_t s_col = t_lane + C::S_COL + b * C::TILE;
          tmem_ld32_nowait(s_col, *reinterpret_cast<float(*)[32]>(&s[0]));  // both halves in flight, one wait
          tmem_ld32_nowait(s_col + 32, *reinterpret_cast<float(*)[32]>(&s[32]));
          tmem_wait_ld();
          if (j == FT_TL_TILE && tid == 0) FT_TL_SOFTMAX_MARK(5);
          // columns outside [lo, hi) are padding (last tile) or tokens this row does not attend to
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
          if (j == FT_TL_TILE && tid == 0) FT_TL_SOFTMAX_MARK(6);
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
          float2 sum4[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
          uint32_t w[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {  // scores stay unscaled until the exponent: one packed FMA per pair
            float2 x = __ffma2_rn(make_float2(s[2 * i], s[2 * i + 1]), sc2, no2);
            if (FT_EXP2_FMA_EVERY > 0 && (i % (FT_EXP2_FMA_EVERY > 0 ? FT_EXP2_FMA_EVERY : 1)) == (FT_EXP2_FMA_EVERY > 0 ? FT_EXP2_FMA_EVERY : 1) - 1) {
              x.x = exp2_fma(x.x);
              x.y = exp2_fma(x.y);
            } else {
              x.x = fast_exp2(x.x);
              x.y = fast_exp2(x.y);
            }
            sum4[i & 3] = __fadd2_rn(sum4[i & 3], x);
            w[i] = pack2<T>(x.x, x.y);
          }
          {
            const float2 sum2 = __fadd2_rn(__fadd2_rn(sum4[0], sum4[1]), __fadd2_rn(sum4[2], sum4[3]));
            l_run += sum2.x + sum2.y;
          }
          // Only a rescale of O has to wait for P.V of the previous tile.  (That tile's barrier phase cannot be
          // confused with an older one: S_g was committed after P.V of tile g-2, so that phase is long complete.)
          if (j == FT_TL_TILE && tid == 0) FT_TL_SOFTMAX_MARK(11);
          if (j > 0 && __any_sync(0xffffffffu, grow)) {
            if (!tc_wait(bar(C::PV_DONE + ((g - 1) & 1)), (uint32_t)((g - 1) >> 1) & 1u, abort_flag)) {
              give_up();
              break;
            }
            tc_fence_after();
#pragma unroll
            for (int cb = 0; cb < 4; ++cb) {  // this warp's rows of O in tensor memory
              float o[32];
              tmem_ld32(t_lane + C::O_COL + cb * 32, o);
#pragma unroll
              for (int c = 0; c < 32; ++c) o[c] *= corr;
              tmem_st32(t_lane + C::O_COL + cb * 32, o);
            }
          }
          if (j == FT_TL_TILE && tid == 0) FT_TL_SOFTMAX_MARK(1);
          // P_g takes the place of the scores just read: 64 16-bit values = the first 32 columns of S buffer b
          tmem_st32(s_col, *reinterpret_cast<float(*)[32]>(&w[0]));
          tmem_wait_st();
          if (j == FT_TL_TILE && tid == 0) FT_TL_SOFTMAX_MARK(7);
          tc_fence_before();  // orders this thread's tcgen05.ld/st before the hand-off
          mbar_arrive(bar(C::P_FULL + b));
          if (j == FT_TL_TILE && tid == 0) FT_TL_SOFTMAX_MARK(4);
        }
        // ---- epilogue: wait for the last P.V, normalise, write this thread's partial row
        if (!dead && ntiles > 0 &&
            !tc_wait(bar(C::PV_DONE + ((g0 + ntiles - 1) & 1)), (uint32_t)((g0 + ntiles - 1) >> 1) & 1u, abort_flag))
          give_up();
        if (!dead) {
          tc_fence_after();
          if (tid == 0) FT_TL_MARK(3);
          const int prow = row0 + tid;
          const bool live = prow < rows;
          int slot = 0, gg = 0;
          if (live) {
            slot = prow / G;
            gg = prow - slot * G;
          }
          const int64_t part = (int64_t)q_off + slot;
          const bool store = live && part >= 0 && part < p.num_partial_rows;
          const int head = kvh * G + gg;
          const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
          // stage the normalised row in shared memory (every operand buffer is idle by now)
          const uint32_t out_row = sm + (uint32_t)tid * C::OUT_STRIDE;
#pragma unroll
          for (int cb = 0; cb < 4; ++cb) {
            float o[32];
            if (ntiles > 0) {
              tmem_ld32(t_lane + C::O_COL + cb * 32, o);  // warp-collective: every lane of the warp takes part
            } else {
#pragma unroll
              for (int c = 0; c < 32; ++c) o[c] = 0.f;
            }
#pragma unroll
            for (int c = 0; c < 8; ++c)
              asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"r"(out_row + (cb * 8 + c) * 16),
                           "f"(o[4 * c] * inv), "f"(o[4 * c + 1] * inv), "f"(o[4 * c + 2] * inv), "f"(o[4 * c + 3] * inv)
                           : "memory");
          }
          if (tid == 0) FT_TL_MARK(8);
          if (store)
            p.mid_lse[part * p.ml_s0 + head] = l_run > 0.f ? (m_used + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
          // each warp staged its own 32 rows: write them out one row per instruction (32 lanes x 16 bytes)
          __syncwarp();
          float* my_dst = store ? p.mid_o + part * p.mo_s0 + (int64_t)head * p.mo_s1 : nullptr;
          const uint32_t warp_rows = sm + (uint32_t)(warp * 32) * C::OUT_STRIDE + lane * 16;
#pragma unroll 16
          for (int i = 0; i < 32; ++i) {
            float* dst = reinterpret_cast<float*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_dst), i));
            float4 x;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];\n"
                         : "=f"(x.x), "=f"(x.y), "=f"(x.z), "=f"(x.w)
                         : "r"(warp_rows + i * C::OUT_STRIDE));
            if (dst != nullptr) reinterpret_cast<float4*>(dst)[lane] = x;
          }
          if (tid == 0) FT_TL_MARK(9);
        }
      }
      if (!pass_end()) break;
    }
  } else {
    reg_shrink<C::REGS_OTHER>();
    for (int row0 = 0; row0 < rows; row0 += C::ROWS) {
      if (warp >= 6) {
        // ================================================================ Q gather (64 threads)
        // request ids of this pass's slots -> the (still unused) V buffers, then the rows themselves
        const int qt = tid - 192, ld_c = qt & 15, ld_r = qt >> 4;
        const int row_end = min(rows, row0 + C::ROWS);
        const int first_slot = row0 / G, nslots = (row_end - 1) / G - first_slot + 1;  // <= 128
        for (int i = qt; i < nslots; i += 64) {
          const int64_t part = (int64_t)q_off + first_slot + i;
          if (part >= 0 && part < p.num_partial_rows) {
            cp_async4(req_sm + i * 4, p.q_entries + part);
          } else {
            flag_error(FT_DEV_BAD_ROW_INDEX);
            asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(req_sm + i * 4), "r"(-1) : "memory");
          }
        }
        cp_async_commit();
        cp_async_wait<0>();
        asm volatile("bar.sync 1, 64;\n" ::: "memory");
        const int* req_of = reinterpret_cast<const int*>(smem + C::V_OFF);
        // Requests with consecutive ids (the usual case: the leaves under a node are numbered in tree order) make
        // the whole Q tile one strided block of the Q tensor: two boxes of [128 / G requests][G heads][64].
        bool in_order = false;
        if (tp.q_box_rows > 0) {
          const int req0 = req_of[0];
          bool mine = true;
          for (int i = lane; i < nslots; i += 32) mine &= req_of[i] == req0 + i;
          in_order = __all_sync(0xffffffffu, mine) && req0 >= 0 && (int64_t)req0 + nslots <= p.batch;
        }
        if (in_order) {
          if (qt == 0) {
            mbar_arrive_expect_tx(bar(C::Q_FULL), 32768);  // full boxes: rows past the task's requests are dead rows
            tma_load_3d(q_sm, &tp.q_map_tile, 0, kvh * G, req_of[0], bar(C::Q_FULL));
            tma_load_3d(q_sm + 16384, &tp.q_map_tile, 64, kvh * G, req_of[0], bar(C::Q_FULL));
          } else {
            mbar_arrive(bar(C::Q_FULL));
          }
        } else if (tp.q_box_rows > 0) {
          // The G rows of a request are adjacent heads of one Q row: one box of up to 8 rows x 64 elements per
          // half.  G divides 128 here, so passes start on a request and a box never straddles an 8-row group.
          const int br = tp.q_box_rows;
          uint32_t bytes = 0;
          for (int i = qt; i < nslots; i += 64) {
            const int req = req_of[i];
            if (req >= 0 && req < p.batch)
              bytes += (uint32_t)G * 256u;
            else if ((int64_t)q_off + first_slot + i >= 0 && (int64_t)q_off + first_slot + i < p.num_partial_rows)
              flag_error(FT_DEV_BAD_Q_INDEX);
          }
          mbar_arrive_expect_tx(bar(C::Q_FULL), bytes);
          for (int i = qt; i < nslots; i += 64) {
            const int req = req_of[i];
            if (req >= 0 && req < p.batch) {
              for (int sub = 0; sub < G; sub += br) {
                const int r = i * G + sub;
                const uint32_t dst = q_sm + (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
                tma_load_3d(dst, &tp.q_map, 0, kvh * G + sub, req, bar(C::Q_FULL));
                tma_load_3d(dst + 16384, &tp.q_map, 64, kvh * G + sub, req, bar(C::Q_FULL));
              }
            }
          }
        } else {
#pragma unroll 4
          for (int ps = 0; ps < 32; ++ps) {
            const int r = ps * 4 + ld_r;
            const int prow = row0 + r;
            int64_t src = -1;
            if (prow < rows) {
              const int slot = prow / G, gg = prow - slot * G;
              const int req = req_of[slot - first_slot];
              if (req >= 0 && req < p.batch)
                src = (int64_t)req * p.q_s0 + (int64_t)(kvh * G + gg) * p.q_s1 + ld_c * 8;
              else if ((int64_t)q_off + slot >= 0 && (int64_t)q_off + slot < p.num_partial_rows)
                flag_error(FT_DEV_BAD_Q_INDEX);
            }
            cp_async16(q_sm + tc_swz(r, ld_c, 16384), reinterpret_cast<const T*>(p.q) + (src >= 0 ? src : 0), src >= 0);
          }
          proxy_fence();                            // rows past the end were zero-filled with plain shared stores
          mbar_arrive_on_cp_async(bar(C::Q_FULL));  // one arrival per thread once its copies have landed
          cp_async_wait<0>();
        }
        asm volatile("bar.sync 1, 64;\n" ::: "memory");  // both warps are done with the staged request ids: V may land there
        if (warp == 6) {
          // ============================================================== V loader (this warp, once Q is on its way)
          // Row ids live in registers, two per lane and one tile ahead, so this role shares nothing with the K
          // loader: same dense test (64 consecutive pool rows -> two TMA boxes), same gather otherwise.
          const T* vbase = reinterpret_cast<const T*>(p.v) + (int64_t)kvh * p.v_s1;
          auto fetch_ids = [&](int t, int (&dst)[2]) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int pos = t * C::TILE + lane + 32 * h;
              dst[h] = pos < id_lim ? __ldg(ids_of_chunk + pos) : -1;
            }
          };
          int cur[2] = {-1, -1}, nxt[2] = {-1, -1};
          if (ntiles > 0) fetch_ids(0, cur);
          for (int t = 0; t < ntiles && !dead; ++t) {
            if (t + 1 < ntiles) fetch_ids(t + 1, nxt);
            const int g = g0 + t, b = g & 1;
            bool dense = false;
            int first_row = 0;
            if (tp.has_tma && (t + 1) * C::TILE <= id_lim) {
              first_row = __shfl_sync(0xffffffffu, cur[0], 0);
              const bool mine = cur[0] == first_row + lane && cur[1] == first_row + lane + 32;
              dense = __all_sync(0xffffffffu, mine) && first_row >= 0 && (uint32_t)(first_row + C::TILE) <= row_lim;
            }
            if (!tc_wait(bar(C::V_EMPTY + b), ((uint32_t)(g >> 1) & 1u) ^ 1u, abort_flag)) {
              give_up();
              break;
            }
            const uint32_t buf = v_buf(g), full = bar(C::V_FULL + b);
#ifdef FT_TL_LOADERS
            if (t == FT_TL_TILE && lane == 0) FT_TL_MARK(7);
#endif
            if (dense) {
              if (lane == 0) {
                mbar_arrive_expect_tx(full, 16384);
                tma_load_3d(buf, &tp.v_map, 0, kvh, first_row, full);
                tma_load_3d(buf + 8192, &tp.v_map, 64, kvh, first_row, full);
              } else {
                mbar_arrive(full);
              }
            } else {
              const bool bad = tc_gather_tile_regs<T>(buf, vbase, p.v_s0, cur[0], cur[1], t, id_lim, row_lim, lane);
              if (bad) flag_error(FT_DEV_BAD_KV_INDEX);
              mbar_arrive_on_cp_async(full);
            }
#ifdef FT_TL_LOADERS
            if (t == FT_TL_TILE && lane == 0) FT_TL_MARK(11);
#endif
            cur[0] = nxt[0];
            cur[1] = nxt[1];
          }
          cp_async_wait<0>();
        }
      } else if (warp == 5) {
        // ================================================================ loader
        const int* ring = reinterpret_cast<const int*>(smem + C::IDX_OFF);
        auto issue_ids = [&](int t) {  // 64 row ids of tile t -> slot t % 3, two per lane
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int i = lane + 32 * h, pos = t * C::TILE + i;
            if (pos < id_lim) cp_async4(idx_sm + ((t % C::IDX_SLOTS) * C::TILE + i) * 4, ids_of_chunk + pos);
          }
        };
        // one operand tile (K or V of tile t) into `buf`, signalling `full`
        auto load_tile = [&](int t, uint32_t buf, uint32_t full, const CUtensorMap* map, const T* base, int64_t stride,
                             bool dense, int first_row) {
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
          const int* ids = ring + (t % C::IDX_SLOTS) * C::TILE;
          const bool bad = tc_gather_tile_smem<T>(buf, base, stride, ids, t, id_lim, row_lim, lane);
          if (bad) flag_error(FT_DEV_BAD_KV_INDEX);
          mbar_arrive_on_cp_async(full);
        };
        const T* kbase = reinterpret_cast<const T*>(p.k) + (int64_t)kvh * p.k_s1;
        if (ntiles > 0) issue_ids(0);
        cp_async_commit();
        if (ntiles > 1) issue_ids(1);
        cp_async_commit();
        // K only: the V tiles have a loader warp of their own (below), so a tile whose rows must be gathered one
        // by one costs each of the two warps half of the copies, and K never waits behind a V buffer.
        for (int s = 0; s < ntiles && !dead; ++s) {
          const int g = g0 + s, b = g % C::NSK;
          cp_async_wait<1>();  // ids of tile s have landed (this lane's copies)
          __syncwarp();
          if (s == 0 && lane == 0) FT_TL_COARSE_MARK(5);
          // dense tile: 64 valid, consecutive row ids inside the buffer -> TMA
          const int* ids = ring + (s % C::IDX_SLOTS) * C::TILE;
          bool dense = false;
          int first_row = 0;
          if (tp.has_tma && (s + 1) * C::TILE <= id_lim) {
            first_row = ids[0];
            const bool mine = ids[lane] == first_row + lane && ids[lane + 32] == first_row + lane + 32;
            dense = __all_sync(0xffffffffu, mine) && first_row >= 0 && (uint32_t)(first_row + C::TILE) <= row_lim;
          }
          if (!tc_wait(bar(C::K_EMPTY + b), ((uint32_t)(g / C::NSK) & 1u) ^ 1u, abort_flag)) {
            give_up();
            break;
          }
#ifdef FT_TL_LOADERS
          if (s == FT_TL_TILE && lane == 0) FT_TL_MARK(5);
#endif
          load_tile(s, k_buf(g), bar(C::K_FULL + b), &tp.k_map, kbase, p.k_s0, dense, first_row);
#ifdef FT_TL_LOADERS
          if (s == FT_TL_TILE && lane == 0) FT_TL_MARK(6);
#endif
          if (s + 2 < ntiles) issue_ids(s + 2);  // into the slot of tile s-1, whose ids were last used a step ago
          cp_async_commit();
        }
        cp_async_wait<0>();
      } else {
        // ================================================================ MMA issue
        if (lane == 0) {
          const uint32_t idesc_s = tc_idesc<T>(128, C::TILE, false);
          const uint32_t idesc_o = tc_idesc<T>(128, 64, true);  // P.V in two 64-column halves: the shape of S
          const uint64_t q_desc = tc_desc(q_sm, 16, 1024);
          auto issue_pv = [&](int t) {  // O += P_t V_t : per half of O, 4 k-steps of 16 tokens, A = P_t in tensor memory
            const int g = g0 + t, b = g & 1;
            const uint32_t use = (uint32_t)(g >> 1) & 1u;
            if (!tc_wait(bar(C::P_FULL + b), use, abort_flag)) return false;
            if (!tc_wait(bar(C::V_FULL + b), use, abort_flag)) return false;
#ifdef FT_TL_LOADERS
            if (t == FT_TL_TILE) FT_TL_MARK(4);
#endif
            proxy_fence();
            tc_fence_after();
            const uint32_t p_tmem = tmem + C::S_COL + b * C::TILE;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint64_t v_desc = tc_desc(v_buf(g) + h * 8192, 8192, 1024);
#pragma unroll
              for (int ks = 0; ks < 4; ++ks)
                tc_mma_ts(tmem + C::O_COL + h * 64, p_tmem + (uint32_t)(ks * 8), v_desc + (uint64_t)(ks * 128), idesc_o,
                          (t > 0 || ks > 0) ? 1u : 0u);
            }
            tc_commit(bar(C::V_EMPTY + b));
            tc_commit(bar(C::PV_DONE + b));
            return true;
          };
          if (ntiles > 0 && !tc_wait(bar(C::Q_FULL), (uint32_t)pass & 1u, abort_flag)) give_up();
          FT_TL_COARSE_MARK(7);
          for (int t = 0; t < ntiles && !dead; ++t) {
            const int g = g0 + t, b = g & 1, kb = g % C::NSK;
            // S_t = Q K_t^T into S buffer b.  The buffer's previous tenant, P of tile t-2, was consumed by a P.V issued
            // before this point, and same-shape MMAs execute in issue order.
            if (!tc_wait(bar(C::K_FULL + kb), (uint32_t)(g / C::NSK) & 1u, abort_flag)) {
              give_up();
              break;
            }
            if (t == 0) FT_TL_COARSE_MARK(6);
#ifdef FT_TL_LOADERS
            if (t == FT_TL_TILE) FT_TL_MARK(1);
#endif
            proxy_fence();
            tc_fence_after();
            const uint64_t k_desc = tc_desc(k_buf(g), 16, 1024);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {  // 8 k-steps of 16 along head_dim: +32 B inside a block, +1 block after 4
              const uint64_t a = q_desc + (uint64_t)((ks >> 2) * (16384 >> 4) + (ks & 3) * 2);
              const uint64_t bb = k_desc + (uint64_t)((ks >> 2) * (8192 >> 4) + (ks & 3) * 2);
              tc_mma(tmem + C::S_COL + b * C::TILE, a, bb, idesc_s, ks > 0);
            }
            tc_commit(bar(C::K_EMPTY + kb));
            tc_commit(bar(C::S_FULL + b));
            if (t > 0 && !issue_pv(t - 1)) {
              give_up();
              break;
            }
          }
          if (!dead && ntiles > 0 && !issue_pv(ntiles - 1)) give_up();
        }
        __syncwarp();
      }
      if (!pass_end()) break;
    }
  }

  // ---- release tensor memory
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(C::TMEM_COLS) : "memory");
  }
}

template <typename T>
__global__ void __launch_bounds__(TcCfg::THREADS, 2) stage1_tc_kernel(const __grid_constant__ TcParams tp) {
  allow_dependent_launch();
  extern __shared__ __align__(1024) uint8_t smem[];
  int vn, kvh;
  task_of_block(tp.p, blockIdx.x, vn, kvh);
  FT_TL_BEGIN();
  tc_body<T>(tp, smem, vn, kvh);
  FT_TL_END(1);
}

// Both task families in one grid (head_dim 128): the tensor-bound many-row CTAs (tcgen05 body, one task each)
// and the memory-bound few-row CTAs (swapped-operand body) share the SMs instead of running back to back.
// Block order, which is the order the hardware starts them in:
//   [0, lead)                 many-row tasks 0 .. lead-1
//   [lead, lead + few_ctas)   few-row CTAs: persistent workers that split the few-row tasks between them
//                             (p.workers > 0), or one CTA per few-row task (p.workers == 0)
//   the rest                  the remaining many-row tasks
// `lead` leaves room for the few-row CTAs to start at once beside the first many-row CTAs.
template <typename T>
__global__ void __launch_bounds__(TcCfg::THREADS, 2) stage1_fused_kernel(const __grid_constant__ TcParams tp) {
  allow_dependent_launch();
  extern __shared__ __align__(1024) uint8_t smem[];
  const Stage1Params& p = tp.p;
  const int H = p.num_kv_heads;
  const int wide_tasks = p.node_split * H, few_tasks = (p.node_count - p.node_split) * H;
  const int few_ctas = p.workers > 0 ? p.workers : few_tasks;
  const int b = (int)blockIdx.x;
  FT_TL_BEGIN();
  if (b < p.lead_wide || b >= p.lead_wide + few_ctas) {
    const int task = b < p.lead_wide ? b : b - few_ctas;
    tc_body<T>(tp, smem, p.node_offset + task / H, task % H);
    FT_TL_END(1);
  } else {
    // This CTA will not allocate tensor memory.  Saying so at once matters: the SM admits no second CTA of a
    // kernel that uses tensor memory while a resident one still holds the right to allocate.
    if (threadIdx.x < 32) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    if (threadIdx.x >= 128) {  // the few-row bodies are written for four warps: the others hand over their registers
      reg_shrink<24>();
      return;
    }
    reg_grow<TcCfg::REGS_WORKER>();
    wait_for_prior_grid();  // nothing of the preceding kernel's is read or overwritten before this
    const int w = b - p.lead_wide;
    if (p.workers > 0) {
      stream_worker<T, 128>(tp, smem, wide_tasks, few_tasks, w, p.workers);
    } else {
      const int task = wide_tasks + w;
      narrow_dispatch<T, 128>(p, smem, p.node_offset + task / H, task % H);
    }
    FT_TL_END(2);
  }
}

}  // namespace ft
