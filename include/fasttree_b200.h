/*
 * fasttree_b200 - C ABI of the B200 (sm_100a) tree-attention decode engine.
 *
 * The library replaces the device half of the FastTree artifact's decode path.
 * Every entry point is `extern "C"`, takes plain device pointers, sizes and
 * element strides, returns an int status (0 = ok, negative = error, text via
 * ft_last_error()), never throws, never aborts and - unless its comment says
 * otherwise - never allocates device memory: the caller owns all tensors, the
 * plan tables and the partial-result scratch, exactly as in the reference
 * (kernel_bench/fasttree.py:265-280, fasttree_sglang_plugin_v0_2_13/metadata.py:40-58).
 *
 * Reference interfaces replaced (paths inside PanZaifeng/FastTree-Artifact):
 *   ft_decode   <- fasttree_decode            kernel_bench/fasttree.py:582-642
 *                                             (= fasttree_sglang_plugin_v0_2_13/attn_kernels.py:288-348)
 *   ft_stage1   <- _fasttree_decode_stage1    kernel_bench/fasttree.py:416-479 (kernel :299-413)
 *   ft_stage2   <- _fasttree_decode_stage2    kernel_bench/fasttree.py:549-579 (kernel :482-546)
 *   ft_bump_kv_lens <- prepare_for_fasttree_step
 *                                             fasttree_sglang_plugin_v0_2_13/schedule.py:278-283
 */
#ifndef FASTTREE_B200_H_
#define FASTTREE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Storage type of Q, K, V and O.  Accumulation and softmax are always fp32. */
enum ft_dtype { FT_F16 = 0, FT_BF16 = 1, FT_F32 = 2 };

/* Which stage-1 kernel family to use. */
enum ft_path {
  FT_PATH_AUTO = 0,    /* pick per launch from dtype / head_dim / rows per task */
  FT_PATH_GENERIC = 1, /* scalar fp32 kernel: any dtype, head_dim <= 256 */
  FT_PATH_MMA = 2,     /* mma.sync tensor-core kernels, 16-bit types, head_dim 64/128: per phase the
                          narrow (swapped-operand) kernel for <= 16 query rows per task, else the wide one */
  FT_PATH_TCGEN05 = 3, /* tcgen05/TMEM kernel for 128-row tasks, 16-bit types, head_dim 128 */
  FT_PATH_MMA_WIDE = 4, /* the wide mma.sync kernel for every task (ablation / cross-check) */
  FT_PATH_STREAM = 5,   /* like AUTO, but few-row phases run the persistent kernel that pipelines across tasks */
  FT_PATH_PERSIST = 6   /* one persistent tcgen05 kernel (a CTA per SM) for every task: 16-bit types, head_dim 128 */
};

/* Status codes. */
enum ft_status {
  FT_OK = 0,
  FT_ERR_INVALID_ARGUMENT = -1, /* null pointer, negative size, bad stride ... */
  FT_ERR_UNSUPPORTED = -2,      /* head_dim / dtype / alignment the chosen path cannot do */
  FT_ERR_CUDA = -3,             /* a CUDA runtime call failed; see ft_last_error() */
  FT_ERR_DEVICE_STATUS = -4,    /* a kernel flagged bad plan data (index out of range, wait ran out) */
  FT_ERR_TOO_LARGE = -5         /* problem exceeds a fixed capacity of the entry point */
};

/* Bits of the device status word (ft_read_device_status). */
enum ft_device_flag {
  FT_DEV_BAD_KV_INDEX = 1,  /* a gathered K/V row index was outside [0, kv_rows) */
  FT_DEV_BAD_Q_INDEX = 2,   /* a request id was outside [0, batch) */
  FT_DEV_BAD_ROW_INDEX = 4, /* a partial-row id was outside [0, num_partial_rows) */
  FT_DEV_WAIT_TIMEOUT = 8   /* a bounded barrier wait gave up */
};

/*
 * One decode step over one layer.  Field meanings follow the positional
 * arguments of the reference's fasttree_decode (kernel_bench/fasttree.py:582-604).
 * All pointers are device pointers; strides are in ELEMENTS of the respective
 * tensor; the innermost (head_dim) stride is 1.
 */
typedef struct ft_decode_args {
  /* tensors -------------------------------------------------------------- */
  const void* q;          /* [batch, num_qo_heads, head_dim]                    */
  const void* k_buffer;   /* [kv_rows, num_kv_heads, head_dim] (KV pool / tree) */
  const void* v_buffer;   /* same shape as k_buffer                            */
  void* o;                /* [batch, num_qo_heads, head_dim], written          */
  float* o_lse;           /* optional [batch, num_qo_heads] merged LSE, or NULL */
  int32_t dtype;          /* enum ft_dtype                                     */
  int32_t batch;
  int32_t num_qo_heads;
  int32_t num_kv_heads;
  int32_t head_dim;
  int32_t path;           /* enum ft_path                                      */
  int64_t kv_rows;
  int64_t q_stride0, q_stride1;
  int64_t k_stride0, k_stride1;
  int64_t v_stride0, v_stride1;
  int64_t o_stride0, o_stride1;
  /* plan tables (int32, device) ------------------------------------------ */
  const int32_t* vnode_to_kv_entries; /* K/V row ids; in the serving path this is the flat req_to_token table */
  int64_t kv_entries_len;             /* number of readable entries                       */
  const int32_t* vnode_to_kv_offs;    /* [num_vnodes] start of the vnode's row-id run     */
  const int32_t* vnode_to_kv_lens;    /* [num_vnodes]                                     */
  const int32_t* vnode_to_q_entries;  /* [num_partial_rows] request id of partial row r   */
  const int32_t* vnode_to_q_offs;     /* [num_vnodes] first partial row of the vnode      */
  const int32_t* vnode_to_q_lens;     /* [num_vnodes] requests (= partial rows) in it     */
  const int32_t* req_to_vnode_entries;/* partial-row ids grouped by request               */
  const int32_t* req_to_vnode_offs;   /* [batch]                                          */
  const int32_t* req_to_vnode_lens;   /* [batch]                                          */
  int64_t num_partial_rows;
  int32_t phase_node_nums[2];         /* vnodes per phase (reference: big / small request tiles) */
  int32_t phase_node_offsets[2];
  int32_t phase_q_tile_sizes[2];      /* requests per vnode of each phase AT MOST: tile x GQA group bounds the query rows
                                         of the phase's tasks and selects its kernel (> 16 rows: many-row kernels, else
                                         few-row kernels; fp32: row blocks of the tiled kernel).  The kernels read the
                                         actual counts from vnode_to_q_lens, but rows beyond the declared bound are
                                         dropped and flagged (FT_DEV_BAD_ROW_INDEX).  <= 0 = unknown (slow, safe choice). */
  int32_t phase_kv_tile_sizes[2];     /* accepted for signature compatibility; the kernels use 64-token tiles */
  /* scratch (caller-owned) ------------------------------------------------ */
  float* mid_o;                       /* [num_partial_rows, num_qo_heads, head_dim] */
  float* mid_lse;                     /* [num_partial_rows, num_qo_heads]           */
  int64_t mid_o_stride0, mid_o_stride1;
  int64_t mid_lse_stride0;
  /* scalars --------------------------------------------------------------- */
  float sm_scale;
  float logit_cap;                    /* accepted and ignored, as in the reference (fasttree.py:603) */
  void* stream;                       /* cudaStream_t                               */
  /* optional extension of the plan format (no counterpart in the reference) ---- */
  const int32_t* vnode_q_kv_ranges;   /* [num_partial_rows][2] or NULL: partial row r attends only to tokens
                                         [begin, end) of its vnode's KV chunk (positions relative to the chunk's
                                         start, clipped to the chunk).  This lets one vnode hold several short
                                         nodes with disjoint request sets (their KV concatenated, each request
                                         seeing only its own node's tokens).  NULL = every row sees the whole
                                         chunk, as in the reference.  Honoured by the many-row kernels (tcgen05,
                                         wide mma.sync) and by the generic kernel; the few-row kernels do not
                                         read it, so rows of vnodes with <= 16 query rows must cover their whole
                                         chunk (the planner of this library only narrows rows of many-row vnodes). */
  const int32_t* device_phase_info;   /* NULL, or a DEVICE array {phase_node_nums[0], phase_node_nums[1],
                                         phase_node_offsets[0], phase_node_offsets[1]} that stage 1 reads at run
                                         time instead of the host values above (the two phases must be adjacent:
                                         offset[1] = offset[0] + nums[0]).  The launch then does not depend on the
                                         plan: one persistent grid of 2 CTAs per SM (FT_PATH_PERSIST, which
                                         FT_PATH_AUTO selects here; 16-bit types, head_dim 128), so a decode step
                                         captured in a CUDA graph stays valid when the plan tables, which live in
                                         fixed-capacity device buffers, are rewritten for the next burst - what the
                                         reference cannot do (it sizes its grids on the host and switches CUDA graphs
                                         off, fasttree_sglang_plugin_v0_2_13/plugin.py:209-211).  batch, the table
                                         pointers and num_partial_rows (the capacity of mid_o / mid_lse) stay
                                         host-side arguments. */
  const int32_t* vnode_to_kv_entries_aux; /* NULL, or a second row-id table: a vnode whose vnode_to_kv_offs value has
                                         bit 30 set (FT_KV_OFFSET_AUX) takes its row ids from this table at the
                                         offset in the low 30 bits.  The serving path addresses tree nodes straight
                                         through req_to_token (one run of positions per vnode) and keeps here the
                                         concatenated row ids of private tails that run as one many-row vnode with
                                         vnode_q_kv_ranges (ft_gather_kv_entries builds it; ft_bump_tails and
                                         ft_refresh_tails extend it between the steps of a burst).  No counterpart in the reference, whose
                                         serving plan has one few-row task per request tail
                                         (fasttree_sglang_plugin_v0_2_13/schedule.py:212-232). */
  int64_t kv_entries_aux_len;         /* readable entries of vnode_to_kv_entries_aux */
} ft_decode_args;

/* Library version (major*10000 + minor*100 + patch). */
int ft_version(void);

/* sizeof(ft_decode_args) as compiled into the library, for bindings to check
 * their mirror of the struct against. */
int ft_decode_args_size(void);

/* Text of the last error raised on the calling thread ("" if none). */
const char* ft_last_error(void);

/* Stage 1 + stage 2 on args->stream; no host synchronisation.
 * Replaces fasttree_decode (kernel_bench/fasttree.py:582-642). */
int ft_decode(const ft_decode_args* args);

/* Partial attention of every vnode into mid_o / mid_lse (normalised partial
 * outputs and log(sum)+max, the reference's convention).
 * Replaces _fasttree_decode_stage1 (kernel_bench/fasttree.py:416-479). */
int ft_stage1(const ft_decode_args* args);

/* Log-sum-exp merge of each request's partial rows into o (and o_lse).
 * Replaces _fasttree_decode_stage2 (kernel_bench/fasttree.py:549-579).
 * Called on its own it is an ordinary launch, ordered after everything enqueued on the stream before it;
 * inside ft_decode it is launched as a programmatic dependent of stage 1. */
int ft_stage2(const ft_decode_args* args);

/* ft_decode fed from and drained to pinned host memory in one call, on args->stream; wait != 0 also synchronises
 * the stream before returning, so that o_host is valid.  q_host / o_host are packed [batch, heads, head_dim];
 * args->q is a packed device staging buffer that receives the query.  When the host buffers are mapped into the
 * device's address space (cudaHostAlloc / torch pinned memory) the query is fetched by a small copy kernel and
 * stage 2 writes the output rows straight into o_host over PCIe - no copy-engine transfer on the critical path;
 * args->o is then not written.  Otherwise: one cudaMemcpyAsync per buffer around the decode, through args->o.
 * This is the call pattern of a decode loop whose sampler runs on the host; the reference's harness keeps Q and
 * the output on the device (kernel_bench/benchmark.py:88-128). */
int ft_decode_host_io(const ft_decode_args* args, const void* q_host, void* o_host, int wait);

/* ft_decode for callers that cannot provide (or allocate) the mid_o / mid_lse scratch.  It has no counterpart
 * in the reference, whose planner and plugin always allocate those buffers with torch
 * (kernel_bench/fasttree.py:275-280, fasttree_sglang_plugin_v0_2_13/metadata.py:53-58).
 *
 * Who needs it: a serving worker that handed all free device memory to its KV pool at start-up cannot rely on a
 * later cudaMalloc succeeding, and a decode loop cannot afford the device-wide synchronisation cudaMalloc /
 * cudaFree imply.  Here the partial outputs and their LSE go to a fixed array of FT_STATIC_SCRATCH_BYTES (16 MiB)
 * compiled into the library; args->mid_o, args->mid_lse and their strides are ignored (they may be NULL),
 * everything else is as in ft_decode.  The call allocates nothing: no cudaMalloc, no cudaFree, no allocating
 * library routine.
 *
 * Limit: num_partial_rows * num_qo_heads * (head_dim + 1) * 4 bytes must fit in the array (e.g. 1016 partial
 * rows at 32 heads x 128); larger plans get FT_ERR_TOO_LARGE and must use ft_decode.
 * Set-up: the first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 * device current); make that first call before any stream capture begins.  The address is remembered per device
 * for the life of the process: after cudaDeviceReset the library must be reloaded.
 * Sharing: every call on a device uses the same array, which still holds the previous call's partials; stage 1
 * overwrites every row stage 2 reads, so nothing needs clearing, but two calls that overlap on the GPU
 * (different streams, or several threads) race on it - serialise them. */
#define FT_STATIC_SCRATCH_BYTES (16u << 20)
int ft_decode_static_scratch(const ft_decode_args* args);

/* vnode_to_kv_lens[last_vnodes[i]] += 1 for i < n, on the device: the token
 * just generated joins each request's last private KV chunk.
 * Replaces prepare_for_fasttree_step (fasttree_sglang_plugin_v0_2_13/schedule.py:278-283). */
int ft_bump_kv_lens(int32_t* vnode_to_kv_lens, const int32_t* last_vnodes, int32_t n, void* stream);

#define FT_KV_OFFSET_AUX (1 << 30)

/* Builds the auxiliary row-id table of a burst on the device: segment i copies seg_len[i] row ids from
 * src_table[seg_src[i] ...] (the flat req_to_token table) to aux_table[seg_dst[i] ...] and fills the next
 * seg_room[i] entries - room for the tokens the burst will generate - with the segment's first row id, a valid
 * row that no query row attends to.  Segments that reach outside either table are skipped and flagged
 * (FT_DEV_BAD_KV_INDEX).  All arrays are device arrays.  No counterpart in the reference. */
int ft_gather_kv_entries(const int32_t* src_table, int64_t src_len, const int32_t* seg_src, const int32_t* seg_len,
                         const int32_t* seg_dst, const int32_t* seg_room, int32_t n_segments, int32_t* aux_table,
                         int64_t aux_len, void* stream);

/* Between two steps of a burst, per request i < n, with tail_state[i] = {aux_pos, src_pos, index, room}:
 *   aux_pos >= 0 (the tail is a member of a grouped vnode; aux_pos / src_pos are one past its last row id in the
 *     auxiliary table / in req_to_token): the end of partial row `index` in vnode_q_kv_ranges moves up by one,
 *     aux_pos and src_pos advance, room shrinks (room exhausted: nothing changes, FT_DEV_BAD_KV_INDEX is flagged);
 *   aux_pos < 0 (the tail is a vnode of its own): vnode_to_kv_lens[index] += 1, as ft_bump_kv_lens does
 *     (index -1: unused entry).
 * Replaces prepare_for_fasttree_step (fasttree_sglang_plugin_v0_2_13/schedule.py:278-283) for plans with grouped tails. */
int ft_bump_tails(int32_t* tail_state, int32_t n, int32_t* vnode_q_kv_ranges, int64_t num_partial_rows,
                  int32_t* vnode_to_kv_lens, int32_t num_vnodes, void* stream);
/* aux_table[aux_pos - 1] = src_table[src_pos - 1] for every grouped tail: the newest token of a request gets its
 * KV-pool slot (and its req_to_token entry) only when the step's batch is prepared, after the plan or the bump, so
 * the copy of that one row id is made at the start of the step's first attention call.  Idempotent. */
int ft_refresh_tails(const int32_t* tail_state, int32_t n, const int32_t* src_table, int64_t src_len, int32_t* aux_table,
                     int64_t aux_len, void* stream);

/* Synchronises `stream`, copies the device status word of the current device
 * to *flags (bits of enum ft_device_flag) and clears it.  Kernels only ever
 * OR bits into the word when they meet bad plan data; they skip the access
 * instead of faulting. */
int ft_read_device_status(void* stream, int32_t* flags);

/* Runs one warp through the bounded mbarrier waits of the stage-1 kernels on a barrier nothing arrives at
 * (limit = probes before the plain wait gives up, 1 .. 2^20) and synchronises.  result_host[0] / [1] receive what
 * the plain wait and the abortable wait returned (0 = gave up, the expected answer); the kernel then raises
 * FT_DEV_WAIT_TIMEOUT in the device status word, as a stage-1 kernel whose wait ran out does.  No copy engine, tensor
 * core or tensor memory is used.  A health check for the failure-detection path; no counterpart in the reference. */
int ft_selftest_bounded_wait(int limit, int* result_host, void* stream);

/* Which bounded wait of the persistent stage-1 kernel gave up first since the last call (after
 * FT_DEV_WAIT_TIMEOUT): out8 = {wait id (0: none), block, warp, task sequence number, tile counter, 0, 0, 0};
 * the ids are listed next to the kernel (csrc/ft_stage1_persist.cuh).  Synchronises the device and clears the
 * record.  A diagnostic aid; no counterpart in the reference. */
int ft_read_wait_diagnostics(int32_t* out8);

/* Number of kernels this library has launched from the calling process. */
int64_t ft_launch_count(void);

/* Names of the kernels ft_stage1 would launch for these arguments, joined by '+' when there are two launches
 * (e.g. "stage1_fused_kernel", "stage1_tc_kernel+stage1_narrow_kernel"): the names a profiler shows.  Nothing is
 * launched.  NULL with ft_last_error() set when the arguments are rejected.  The text belongs to the calling
 * thread and is valid until its next call. */
const char* ft_stage1_path_name(const ft_decode_args* args);

/* ---- host-side planner -------------------------------------------------------------------------------------
 * Native counterpart of the tree splitter that produces the plan tables above (the tables the reference builds
 * in Python, kernel_bench/fasttree.py:99-296; this splitter uses a B200 cost model instead of the reference's
 * padding heuristic and is what ft_b200.planner.plan_b200 specifies).  Pure host code: no CUDA call, no device
 * memory.  ft_plan_b200_build creates a plan object, ft_plan_get_info reports the table sizes,
 * ft_plan_copy_tables copies the tables into caller-owned host arrays, ft_plan_free releases the object. */
typedef struct ft_plan ft_plan;

typedef struct ft_b200_model { /* machine constants of the cost model; NULL in ft_plan_b200_build = defaults */
  int32_t num_sms;             /* 148 */
  int32_t ctas_per_sm;         /* 2 */
  double waves;                /* rounds of resident CTAs to aim for: 1.0 */
  int32_t tile_tokens;         /* KV tile of the stage-1 kernels: 64 */
  int32_t rows_per_cta;        /* query rows one CTA holds: 64 (128 at head_dim 128) */
  int32_t min_chunk;           /* never cut a node's KV finer than this many tokens: 128 */
  int32_t nominal_split;       /* chunk length assumed while deciding the edges: 512 */
  double ridge_flop_per_byte;  /* flops that cost as much time as one streamed byte: 90 (360 at head_dim 128) */
  int32_t task_overhead_bytes; /* fixed cost of one more CTA in streamed-byte equivalents: 16384 */
  int32_t elem_bytes;          /* 2 */
  int32_t group_member_tokens; /* nodes up to this long, with few enough requests for the few-row kernels, may be
                                  packed into groups that run as one many-row task: 128; 0 = never */
  int32_t group_min_members;   /* smallest group worth forming: 6 */
} ft_b200_model;

typedef struct ft_plan_info {
  int64_t kv_entries;   /* length of vnode_to_kv_entries, including the 32 trailing -1 */
  int64_t vnodes;       /* length of the six per-vnode tables */
  int64_t partial_rows; /* length of vnode_to_q_entries = rows of mid_o / mid_lse; req_to_vnode_entries has 32 more */
  int64_t batch;        /* length of req_to_vnode_offs / lens */
  int64_t nodes;        /* length of node_assignments */
  int64_t virtual_nodes;
  int32_t phase_node_nums[2];
  int32_t phase_node_offsets[2];
  int32_t q_tile;       /* requests per task in phase 0 / 1: the tile sizes to pass as phase_q_tile_sizes */
  int32_t small_tile;
  int32_t tile_tokens;
  int32_t has_row_ranges; /* 1: the plan holds groups of short nodes and ft_plan_copy_row_ranges has a table to give */
  double target_bytes;  /* streamed bytes one task was sized for */
  int64_t aux_entries;  /* serving plans with groups: entries of the auxiliary row-id table the vnode offsets assume */
  int64_t aux_segments; /* ... and the number of segments ft_plan_copy_aux_segments reports */
} ft_plan_info;

/* Tree: n_nodes records in id order, node 0 the root, parents before children (parent[0] = -1); seqlen tokens per
 * node; the requests whose path contains node i are req_ids[req_offs[i] .. req_offs[i+1]); kv_ptrs[i] .. kv_ptrs[i+1]
 * are the node's rows in the K/V buffers.  num_kv_heads is the LOCAL head count of this GPU. */
int ft_plan_b200_build(const int32_t* parent, const int32_t* seqlen, int32_t n_nodes, const int64_t* req_offs,
                       const int32_t* req_ids, const int64_t* kv_ptrs, int32_t batch, int32_t num_qo_heads,
                       int32_t num_kv_heads, int32_t head_dim, const ft_b200_model* model, ft_plan** out);
/* The serving path's addressing (fasttree_sglang_plugin_v0_2_13/schedule.py:159-232 of the reference): a node's
 * KV, together with that of the ancestors it carries, is one run of positions in an existing row-id table (the
 * flattened req_to_token): [node_base[i] + node_offset[top carried ancestor], node_base[i] + node_offset[i] +
 * seqlen[i]).  n_extra further pairings of one request with one run (each request's private tail) take part in
 * the byte budget and are emitted last.  No vnode_to_kv_entries table is built (ft_plan_info.kv_entries = 0);
 * vnode_to_kv_offs are positions in the existing table; req_to_vnode_entries still gets its 32 trailing -1.
 * tail_room < 0: every vnode is one run, as above.  tail_room >= 0 (head_dim 128): short runs with few requests -
 * above all the private tails, thousands of one-tile tasks in a large burst - may be packed into groups that run as
 * ONE many-row vnode with per-row token ranges (ft_plan_copy_row_ranges; rows of plain vnodes get an open end there,
 * which the kernels clip to the chunk).  A group's row ids are the concatenation of its members' runs, each tail
 * followed by tail_room spare entries for the tokens the burst will add; they live in an auxiliary table
 * (ft_decode_args.vnode_to_kv_entries_aux) that the caller fills on the device with ft_gather_kv_entries from the
 * segment list of ft_plan_copy_aux_segments, and the group's vnode_to_kv_offs value is FT_KV_OFFSET_AUX + its
 * position in that table. */
int ft_plan_b200_build_direct(const int32_t* parent, const int32_t* seqlen, int32_t n_nodes, const int64_t* req_offs,
                              const int32_t* req_ids, const int64_t* node_base, const int64_t* node_offset,
                              int64_t n_extra, const int64_t* extra_begin, const int64_t* extra_end,
                              const int32_t* extra_req, int32_t tail_room, int32_t batch, int32_t num_qo_heads,
                              int32_t num_kv_heads, int32_t head_dim, const ft_b200_model* model, ft_plan** out);
/* segments: int32 [ft_plan_info.aux_segments][4] = {source position, length, position in the auxiliary table, room} */
int ft_plan_copy_aux_segments(const ft_plan* plan, int32_t* segments);
int ft_plan_get_info(const ft_plan* plan, ft_plan_info* info);
int ft_plan_copy_tables(const ft_plan* plan, int32_t* vnode_to_kv_entries, int32_t* vnode_to_kv_offs,
                        int32_t* vnode_to_kv_lens, int32_t* vnode_to_q_entries, int32_t* vnode_to_q_offs,
                        int32_t* vnode_to_q_lens, int32_t* req_to_vnode_entries, int32_t* req_to_vnode_offs,
                        int32_t* req_to_vnode_lens, int32_t* node_assignments);
/* The optional tenth table, vnode_q_kv_ranges of ft_decode_args ([partial_rows][2] int32): only when
 * ft_plan_info.has_row_ranges is 1 (ft_plan_b200_build at head_dim 128 with 16-bit elements, when short nodes were
 * packed into groups); FT_ERR_INVALID_ARGUMENT otherwise. */
int ft_plan_copy_row_ranges(const ft_plan* plan, int32_t* vnode_q_kv_ranges);
void ft_plan_free(ft_plan* plan);

#ifdef __cplusplus
}
#endif
#endif /* FASTTREE_B200_H_ */
