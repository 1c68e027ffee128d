// Stage 1, warp-level tensor-core kernel (mma.sync m16n8k16, fp16/bf16 inputs,
// fp32 accumulate), head_dim 64 or 128.
//
// One CTA (4 warps) per (vnode, kv head).  The vnode's query rows are the
// requests of the vnode x the GQA group, packed as row = slot * G + g.  Rows
// are processed 64 at a time, 16 per warp.  When a vnode has fewer than 64
// rows the spare warps do not idle: with <= 16 rows the four warps each take a
// quarter of every 64-token KV tile (two halves for <= 32 rows) and their
// running (max, sum, acc) are merged through shared memory at the end - the
// memory-bound shape of leaf and low-fan-out nodes.
//
// K/V rows are gathered by row id (vnode_to_kv_entries) with 16-byte cp.async
// copies into a 3-stage shared-memory ring (KvPipe); every 256-byte row is
// XOR-swizzled at 16-byte granularity so that ldmatrix reads are bank-conflict
// free.  Each KV byte is read from global memory once per (vnode, 64-row block).
//
// Arithmetic follows kernel_bench/fasttree.py:360-413: scores scaled after the
// dot product in fp32, online softmax, probabilities rounded to the storage
// type before P*V, outputs normalised, lse = log(sum) + max.
#pragma once

#include "ft_common.cuh"

namespace ft {

__device__ __forceinline__ uint32_t smem_u32(const void* ptr) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(ptr));
}

// 16-byte asynchronous copy; an invalid source becomes 16 zero bytes (plain shared store, made visible by the
// same barrier that publishes the copies)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  if (valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
  } else {
    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};\n" ::"r"(dst), "r"(0) : "memory");
  }
}
// the same without a branch: an invalid row reads nothing (source size 0) and the copy engine writes 16 zero bytes,
// so a gather loop stays one straight instruction stream and the zeros need no proxy fence
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(valid ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
struct MmaCfg {
  static constexpr int THREADS = 128;
  static constexpr int TILE = 64;               // tokens per pipeline stage
  static constexpr int STAGES = 3;
  static constexpr int ROWB = D * 2;            // bytes of one Q/K/V row (16-bit elements)
  static constexpr int CPR = D / 8;             // 16-byte chunks per row
  static constexpr int TPP = THREADS / CPR;     // rows one pass of the CTA covers
  static constexpr int PASSES = TILE / TPP;
  static constexpr int QROWS = 64;
  static constexpr int Q_BYTES = QROWS * ROWB;
  static constexpr int STAGE_BYTES = TILE * ROWB;  // one K or V tile
  static constexpr int PIPE_BYTES = STAGES * 2 * STAGE_BYTES;
  static constexpr int OSTRIDE = D + 4;         // floats per staged output row
  static constexpr int EPI_BYTES = 4 * 16 * OSTRIDE * 4 + 2 * 4 * 16 * 4;
  static constexpr int WIDE_IDXB = 128;         // row-id block of the wide kernel (2 x 512 B: all the room two CTAs/SM leave)
  static constexpr int WIDE_IDX_BYTES = 2 * WIDE_IDXB * 4;
  static constexpr int SMEM_BYTES = Q_BYTES + WIDE_IDX_BYTES + (PIPE_BYTES > EPI_BYTES ? PIPE_BYTES : EPI_BYTES);
  // Q rows: one row after the other, the 16-byte chunks of a row XOR-swizzled by the row
  __device__ static __forceinline__ uint32_t swzq(int row, int chunk) {
    return static_cast<uint32_t>(row * ROWB + ((chunk ^ (row & 7)) << 4));
  }
  // K/V tiles: 64-element (128-byte) column blocks one after the other, each [TILE rows][128 bytes] with the
  // chunks of a row XOR-swizzled by the row: the layout a tiled TMA copy with the 128-byte swizzle writes, and
  // conflict-free for ldmatrix and 16-byte cp.async alike
  static constexpr int BLOCK_BYTES = TILE * 128;
  __device__ static __forceinline__ uint32_t swz(int row, int chunk) {
    return static_cast<uint32_t>((chunk >> 3) * BLOCK_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
  }
};

__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ int lds_s32(uint32_t addr) {
  int v;
  asm volatile("ld.shared.s32 %0, [%1];\n" : "=r"(v) : "r"(addr));
  return v;
}

// Gathered K/V streaming for one (vnode chunk, kv head): a ring of STAGES K/V
// tiles filled with 16-byte cp.async copies, fed by a two-block ring of row
// ids in shared memory.  The row ids are themselves fetched with cp.async, a
// whole block (IDXB tokens) at a time and one block ahead of use: a plain
// global load issued next to ~100 KB of outstanding tile copies only returns
// after those have drained, which stalls the issue of the following tile.
template <typename T, int D, int IDXB>
struct KvPipe {
  using C = MmaCfg<D>;
  static constexpr int TPB = IDXB / C::TILE;     // tiles per row-id block
  static constexpr int IDX_BYTES = 2 * IDXB * 4;
  const Stage1Params& p;
  const T* kbase;
  const T* vbase;
  const int* idx_ptr;
  const int32_t* ids;  // the chunk's row ids in global memory
  uint32_t idx_sm, pipe_sm, row_lim;
  int kv_off, kv_len, id_lim, ntiles, tid, ld_c, ld_r;

  // idx_ptr_ / idx_sm_: generic pointer and shared-window address of the same row-id ring
  __device__ __forceinline__ KvPipe(const Stage1Params& p_, int kvh, int kv_off_, int kv_len_, const void* idx_ptr_,
                                    uint32_t idx_sm_, uint32_t pipe_sm_)
      : p(p_), idx_ptr(static_cast<const int*>(idx_ptr_)), idx_sm(idx_sm_), pipe_sm(pipe_sm_), kv_off(kv_off_),
        kv_len(kv_len_) {
    tid = threadIdx.x;
    // row ids past the end of the table are a plan error: flagged once, those tokens become padding
    id_lim = kv_ids_limit(p, kv_off, kv_len);
    ids = kv_ids_base(p, kv_off);
    if (id_lim < kv_len && tid == 0) flag_error(FT_DEV_BAD_KV_INDEX);
    row_lim = (uint32_t)(p.kv_rows < 0x7fffffffLL ? p.kv_rows : 0x7fffffffLL);
    ld_c = tid % C::CPR;
    ld_r = tid / C::CPR;
    ntiles = (kv_len + C::TILE - 1) / C::TILE;
    kbase = reinterpret_cast<const T*>(p.k) + (int64_t)kvh * p.k_s1 + ld_c * 8;
    vbase = reinterpret_cast<const T*>(p.v) + (int64_t)kvh * p.v_s1 + ld_c * 8;
  }
  // row ids of tokens [b*IDXB, (b+1)*IDXB) -> ring slot b&1 (joins the caller's open cp.async group)
  __device__ __forceinline__ void issue_idx_block(int b) {
    const uint32_t dst = idx_sm + (b & 1) * IDXB * 4;
#pragma unroll
    for (int i = 0; i < IDXB / C::THREADS; ++i) {
      const int t = i * C::THREADS + tid;
      const int pos = b * IDXB + t;
      if (pos < id_lim) cp_async4(dst + t * 4, ids + pos);
    }
  }
  // blocks 0 and 1: issue early (their round trip then overlaps the caller's own dependent loads), wait before
  // the first tile
  __device__ __forceinline__ void issue_first_indices() {
    issue_idx_block(0);
    if (IDXB < kv_len) issue_idx_block(1);
    cp_async_commit();
  }
  __device__ __forceinline__ void wait_indices() {
    cp_async_wait<0>();
    __syncthreads();
  }
  __device__ __forceinline__ void prime_indices() {
    issue_first_indices();
    wait_indices();
  }
  // K/V rows of tile `tile` -> stage tile % STAGES (joins the open group)
  __device__ __forceinline__ void issue_tile(int tile) {
    const uint32_t k_sm = pipe_sm + (tile % C::STAGES) * 2 * C::STAGE_BYTES;
    const uint32_t v_sm = k_sm + C::STAGE_BYTES;
    // all row ids of this thread first (independent shared-memory loads), then the copies
    const int* ring = idx_ptr + ((tile / TPB) & 1) * IDXB + (tile % TPB) * C::TILE + ld_r;
    const int pos0 = tile * C::TILE + ld_r;
    uint32_t row[C::PASSES];
#pragma unroll
    for (int ps = 0; ps < C::PASSES; ++ps) row[ps] = pos0 + ps * C::TPP < id_lim ? (uint32_t)ring[ps * C::TPP] : 0xffffffffu;
    bool bad = false;
#pragma unroll
    for (int ps = 0; ps < C::PASSES; ++ps) {
      const int r = ps * C::TPP + ld_r;
      const bool ok = row[ps] < row_lim;  // padding (0xffffffff), negative and too-large ids all fail this test
      bad |= !ok && pos0 + ps * C::TPP < id_lim;
      const int64_t off = (int64_t)(ok ? row[ps] : 0u);
      cp_async16(k_sm + C::swz(r, ld_c), kbase + off * p.k_s0, ok);
      cp_async16(v_sm + C::swz(r, ld_c), vbase + off * p.v_s0, ok);
    }
    if (bad) flag_error(FT_DEV_BAD_KV_INDEX);
  }
  // tiles 0 .. STAGES-2, one group each
  __device__ __forceinline__ void prologue() {
#pragma unroll
    for (int s = 0; s < C::STAGES - 1; ++s) {
      if (s < ntiles) issue_tile(s);
      cp_async_commit();
    }
  }
  // top of iteration j: tile j has landed; refill the stage freed by tile j-1
  __device__ __forceinline__ void advance(int j) {
    cp_async_wait<C::STAGES - 2>();
    __syncthreads();
    const int nt = j + C::STAGES - 1;
    if (nt < ntiles) {
      issue_tile(nt);
      // the first tile of a row-id block is going out: the block before it is dead, refill its slot
      if (nt % TPB == 0 && nt >= TPB && (nt / TPB + 1) * IDXB < kv_len) issue_idx_block(nt / TPB + 1);
    }
    cp_async_commit();
  }
  __device__ __forceinline__ uint32_t k_stage(int j) const { return pipe_sm + (j % C::STAGES) * 2 * C::STAGE_BYTES; }
  __device__ __forceinline__ uint32_t v_stage(int j) const { return k_stage(j) + C::STAGE_BYTES; }
  __device__ __forceinline__ void drain() {
    cp_async_wait<0>();
    __syncthreads();
  }
};

// One 64-token tile for one warp: NB = 8-token blocks this warp owns (2, 4 or 8).
template <typename T, int D, int NB>
__device__ __forceinline__ void mma_tile(const uint32_t k_sm, const uint32_t v_sm, const int tok0,
                                         const int first_pos, const int (&lo)[2], const int (&hi)[2],
                                         const float scale2, const uint32_t (&qf)[D / 16][4],
                                         float (&o_acc)[D / 8][4], float (&m_run)[2], float (&l_run)[2],
                                         const int lane) {
  using C = MmaCfg<D>;
  const int t4 = lane & 3;
  float s[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;

  // S = Q K^T.  K rows sit [token][d]; that is the "col" operand as stored.
#pragma unroll
  for (int kk2 = 0; kk2 < D / 32; ++kk2) {
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      uint32_t kb[4];
      ldmatrix_x4(kb, k_sm + C::swz(tok0 + nb * 8 + (lane & 7), 4 * kk2 + (lane >> 3)));
      mma16816<T>(s[nb], qf[2 * kk2], kb[0], kb[1]);
      mma16816<T>(s[nb], qf[2 * kk2 + 1], kb[2], kb[3]);
    }
  }

  // scale (log2 domain); mask the tokens outside [lo, hi) of this thread's two rows (row g8: elements 0-1,
  // row g8+8: elements 2-3) - the tail of the chunk, or what a row of a group of short nodes does not attend to
  const bool masked = first_pos < max(lo[0], lo[1]) || first_pos + NB * 8 > min(hi[0], hi[1]);
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float x = s[nb][e] * scale2;
      if (masked) {
        const int pos = first_pos + nb * 8 + 2 * t4 + (e & 1);
        if (pos < lo[e >> 1] || pos >= hi[e >> 1]) x = -INFINITY;
      }
      s[nb][e] = x;
    }
  }
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    mx0 = fmaxf(mx0, fmaxf(s[nb][0], s[nb][1]));
    mx1 = fmaxf(mx1, fmaxf(s[nb][2], s[nb][3]));
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
  const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
  const float c0 = fast_exp2(m_run[0] - ms0), c1 = fast_exp2(m_run[1] - ms1);
  m_run[0] = mn0;
  m_run[1] = mn1;
  l_run[0] *= c0;
  l_run[1] *= c1;
#pragma unroll
  for (int nd = 0; nd < D / 8; ++nd) {
    o_acc[nd][0] *= c0;
    o_acc[nd][1] *= c0;
    o_acc[nd][2] *= c1;
    o_acc[nd][3] *= c1;
  }

  // P = exp2(S - max); the sum uses the fp32 values, the MMA the rounded ones
  uint32_t pf[NB / 2][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    const float p0 = fast_exp2(s[nb][0] - ms0), p1 = fast_exp2(s[nb][1] - ms0);
    const float p2 = fast_exp2(s[nb][2] - ms1), p3 = fast_exp2(s[nb][3] - ms1);
    l_run[0] += p0 + p1;
    l_run[1] += p2 + p3;
    pf[nb >> 1][(nb & 1) * 2 + 0] = pack2<T>(p0, p1);
    pf[nb >> 1][(nb & 1) * 2 + 1] = pack2<T>(p2, p3);
  }

  // O += P V.  V rows sit [token][d]; the transposing ldmatrix yields the "col" operand.
#pragma unroll
  for (int kt = 0; kt < NB / 2; ++kt) {
#pragma unroll
    for (int nd2 = 0; nd2 < D / 16; ++nd2) {
      uint32_t vb[4];
      ldmatrix_x4_trans(vb, v_sm + C::swz(tok0 + kt * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), 2 * nd2 + (lane >> 4)));
      mma16816<T>(o_acc[2 * nd2], pf[kt], vb[0], vb[1]);
      mma16816<T>(o_acc[2 * nd2 + 1], pf[kt], vb[2], vb[3]);
    }
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(128, 2) stage1_mma_kernel(Stage1Params p) {
  allow_dependent_launch();
  wait_for_prior_grid();  // nothing of the preceding kernel's is read or overwritten before this
  using C = MmaCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t q_sm = smem_u32(smem);
  const uint32_t idx_sm = q_sm + C::Q_BYTES;
  const uint32_t pipe_sm = idx_sm + C::WIDE_IDX_BYTES;
  float* epi_o = reinterpret_cast<float*>(smem + C::Q_BYTES + C::WIDE_IDX_BYTES);
  float* epi_m = epi_o + 4 * 16 * C::OSTRIDE;
  float* epi_l = epi_m + 4 * 16;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int vn, kvh;
  task_of_block(p, blockIdx.x, vn, kvh);
  const int q_off = p.q_offs[vn], q_len = p.q_lens[vn];
  const int kv_off = p.kv_offs[vn], kv_len = max(p.kv_lens[vn], 0);
  const int G = p.group;
  const int rows = q_len * G;
  if (rows <= 0) return;
  const float scale2 = p.sm_scale * 1.4426950408889634f;
  const int ntiles = (kv_len + C::TILE - 1) / C::TILE;
  const int ld_c = tid % C::CPR, ld_r = tid / C::CPR;

  KvPipe<T, D, C::WIDE_IDXB> pipe(p, kvh, kv_off, kv_len, smem + C::Q_BYTES, idx_sm, pipe_sm);

  for (int row0 = 0; row0 < rows; row0 += C::QROWS) {
    const int rows_here = min(C::QROWS, rows - row0);
    const int n_rb = (rows_here + 15) >> 4;                 // 16-row blocks in use: 1..4
    const int rb_log = n_rb <= 1 ? 0 : (n_rb <= 2 ? 1 : 2);  // warps are dealt to 1, 2 or 4 row blocks
    const int ways = 4 >> rb_log;                           // warps sharing one row block split the tile
    const int my_rb = warp & ((1 << rb_log) - 1);
    const int my_way = warp >> rb_log;
    const bool active = my_rb < n_rb;

    // ---- gather the row ids first (independent loads), then start the copies
    constexpr int QPASSES = C::QROWS / C::TPP;
    int64_t q_src[QPASSES];
    const int q_passes = (n_rb * 16 + C::TPP - 1) / C::TPP;
#pragma unroll
    for (int ps = 0; ps < QPASSES; ++ps) {
      q_src[ps] = -1;
      const int prow = row0 + ps * C::TPP + ld_r;
      if (ps < q_passes && prow < rows) {
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
      if (ps < q_passes) {
        const bool ok = q_src[ps] >= 0;
        cp_async16(q_sm + C::swzq(ps * C::TPP + ld_r, ld_c),
                   reinterpret_cast<const T*>(p.q) + (ok ? q_src[ps] : 0), ok);
      }
    }
    pipe.prime_indices();  // also lands Q
    pipe.prologue();

    float o_acc[D / 8][4];
#pragma unroll
    for (int nd = 0; nd < D / 8; ++nd) o_acc[nd][0] = o_acc[nd][1] = o_acc[nd][2] = o_acc[nd][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    uint32_t qf[D / 16][4];
    // chunk tokens [lo, hi) this thread's two rows attend to: the whole chunk unless the plan narrows it
    int lo[2] = {0, 0}, hi[2] = {kv_len, kv_len};
    if (p.q_ranges != nullptr && active) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int prow = row0 + my_rb * 16 + (lane >> 2) + 8 * h;
        const int64_t part = (int64_t)q_off + prow / G;
        if (prow < rows && part >= 0 && part < p.num_partial_rows) {
          lo[h] = max(p.q_ranges[2 * part], 0);
          hi[h] = min(p.q_ranges[2 * part + 1], kv_len);
        }
      }
    }

    for (int j = 0; j < ntiles; ++j) {
      pipe.advance(j);  // tile j has landed for every thread; tile j-1's stage is being refilled
      if (j == 0 && active) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ldmatrix_x4(qf[kk], q_sm + C::swzq(my_rb * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), 2 * kk + (lane >> 4)));
      }
      if (active) {
        const uint32_t k_sm = pipe.k_stage(j), v_sm = pipe.v_stage(j);
        if (ways == 4) {
          const int tok0 = my_way * 16;
          mma_tile<T, D, 2>(k_sm, v_sm, tok0, j * C::TILE + tok0, lo, hi, scale2, qf, o_acc, m_run, l_run, lane);
        } else if (ways == 2) {
          const int tok0 = my_way * 32;
          mma_tile<T, D, 4>(k_sm, v_sm, tok0, j * C::TILE + tok0, lo, hi, scale2, qf, o_acc, m_run, l_run, lane);
        } else {
          mma_tile<T, D, 8>(k_sm, v_sm, 0, j * C::TILE, lo, hi, scale2, qf, o_acc, m_run, l_run, lane);
        }
      }
    }
    pipe.drain();  // the ring is idle: its memory becomes the output staging area

    if (active) {
      float l0 = l_run[0], l1 = l_run[1];
      l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
      l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
      l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
      l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
      const int g8 = lane >> 2, t4 = lane & 3;
      float* dst0 = epi_o + (warp * 16 + g8) * C::OSTRIDE + 2 * t4;
      float* dst1 = dst0 + 8 * C::OSTRIDE;
#pragma unroll
      for (int nd = 0; nd < D / 8; ++nd) {
        *reinterpret_cast<float2*>(dst0 + nd * 8) = make_float2(o_acc[nd][0], o_acc[nd][1]);
        *reinterpret_cast<float2*>(dst1 + nd * 8) = make_float2(o_acc[nd][2], o_acc[nd][3]);
      }
      if (t4 == 0) {
        epi_m[warp * 16 + g8] = m_run[0];
        epi_m[warp * 16 + g8 + 8] = m_run[1];
        epi_l[warp * 16 + g8] = l0;
        epi_l[warp * 16 + g8 + 8] = l1;
      }
    }
    __syncthreads();

    // ---- merge the warps that shared a row block, normalise, write the partial rows
    {
      const int r = tid >> 3, seg = tid & 7;
      for (int rb = 0; rb < n_rb; ++rb) {
        const int prow = row0 + rb * 16 + r;
        if (prow >= rows) continue;
        const int slot = prow / G, gg = prow - slot * G;
        const int64_t part = (int64_t)q_off + slot;
        if (part < 0 || part >= p.num_partial_rows) continue;  // flagged above
        float M = -INFINITY;
        for (int w = 0; w < ways; ++w) M = fmaxf(M, epi_m[(rb + (w << rb_log)) * 16 + r]);
        float L = 0.f;
        float4 out[D / 32];
#pragma unroll
        for (int i = 0; i < D / 32; ++i) out[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int w = 0; w < ways; ++w) {
          const int ww = rb + (w << rb_log);
          const float mw = epi_m[ww * 16 + r];
          const float f = mw == -INFINITY ? 0.f : fast_exp2(mw - M);
          L = fmaf(epi_l[ww * 16 + r], f, L);
          const float4* src = reinterpret_cast<const float4*>(epi_o + (ww * 16 + r) * C::OSTRIDE);
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
    __syncthreads();  // staging area and Q tile are reused by the next 64-row block
  }
}

}  // namespace ft
