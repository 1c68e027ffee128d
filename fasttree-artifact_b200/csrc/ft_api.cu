// C ABI of the tree-attention decode engine: argument validation, kernel
// selection and launches.  Declarations and the mapping to the reference's
// Python entry points are in include/fasttree_b200.h.
#include <cuda.h>

#include <atomic>
#include <cstdarg>
#include <mutex>
#include <utility>
#include <cstdio>
#include <cstring>

#include "fasttree_b200.h"
#include "ft_common.cuh"
#include "ft_stage1_f32.cuh"
#include "ft_stage1_generic.cuh"
#include "ft_stage1_mma.cuh"
#include "ft_stage1_narrow.cuh"
#include "ft_stage1_stream.cuh"
#include "ft_stage1_tc.cuh"
#include "ft_stage1_persist.cuh"
#include "ft_stage2.cuh"

namespace {

thread_local char g_err[512] = "";
std::atomic<int64_t> g_launches{0};
thread_local int64_t t_launches = 0;  // launches issued by this host thread

void count_launch() {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  ++t_launches;
}

// ft_stage1_path_name walks the same selection code as ft_stage1 with launches switched off and collects the
// names of the kernels that would have been launched.
thread_local bool g_dry_run = false;
thread_local char g_kernel_names[160] = "";

bool dry_run(const char* kernel) {
  if (!g_dry_run) return false;
  const size_t used = strlen(g_kernel_names);
  snprintf(g_kernel_names + used, sizeof(g_kernel_names) - used, "%s%s", used ? "+" : "", kernel);
  return true;
}

// Largest dynamic shared memory of a kernel, raised once per device.  Several host threads may make their first
// call at the same time: the flag is atomic and setting the attribute twice is harmless.
struct OncePerDevice {
  std::atomic<bool> done[64];
  OncePerDevice() {
    for (auto& d : done) d.store(false, std::memory_order_relaxed);
  }
};

template <typename Kernel>
cudaError_t raise_smem_limit(OncePerDevice& once, Kernel kernel, int bytes, int* device_out = nullptr) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (device_out != nullptr) *device_out = dev;
  const bool tracked = dev >= 0 && dev < 64;
  if (tracked && once.done[dev].load(std::memory_order_acquire)) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && tracked) once.done[dev].store(true, std::memory_order_release);
  return e;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define FT_CUDA_OK(expr)                                                                      \
  do {                                                                                        \
    cudaError_t e_ = (expr);                                                                  \
    if (e_ != cudaSuccess) return fail(FT_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

int check_common(const ft_decode_args* a) {
  if (a == nullptr) return fail(FT_ERR_INVALID_ARGUMENT, "args is NULL");
  if (a->dtype != FT_F16 && a->dtype != FT_BF16 && a->dtype != FT_F32)
    return fail(FT_ERR_INVALID_ARGUMENT, "dtype %d is not one of FT_F16/FT_BF16/FT_F32", a->dtype);
  if (a->batch < 0 || a->num_qo_heads <= 0 || a->num_kv_heads <= 0 || a->head_dim <= 0)
    return fail(FT_ERR_INVALID_ARGUMENT, "batch/heads/head_dim must be positive (batch %d, hq %d, hkv %d, d %d)",
                a->batch, a->num_qo_heads, a->num_kv_heads, a->head_dim);
  if (a->num_qo_heads % a->num_kv_heads != 0)
    return fail(FT_ERR_INVALID_ARGUMENT, "num_qo_heads %d is not a multiple of num_kv_heads %d", a->num_qo_heads,
                a->num_kv_heads);
  // the reference asserts head_dim in {16,32,64,128,256} (kernel_bench/fasttree.py:439)
  const int d = a->head_dim;
  if (!(d == 16 || d == 32 || d == 64 || d == 128 || d == 256))
    return fail(FT_ERR_UNSUPPORTED, "head_dim %d is not one of 16, 32, 64, 128, 256", d);
  if (a->num_partial_rows < 0) return fail(FT_ERR_INVALID_ARGUMENT, "num_partial_rows is negative");
  if (a->mid_o == nullptr || a->mid_lse == nullptr)
    return fail(FT_ERR_INVALID_ARGUMENT, "mid_o / mid_lse scratch is NULL");
  if (!aligned16(a->mid_o) || a->mid_o_stride0 % 4 != 0 || a->mid_o_stride1 % 4 != 0)
    return fail(FT_ERR_UNSUPPORTED, "mid_o must be 16-byte aligned with strides that are multiples of 4 floats");
  return FT_OK;
}

int check_stage1(const ft_decode_args* a) {
  if (a->q == nullptr || a->k_buffer == nullptr || a->v_buffer == nullptr)
    return fail(FT_ERR_INVALID_ARGUMENT, "q / k_buffer / v_buffer is NULL");
  if (a->kv_rows <= 0) return fail(FT_ERR_INVALID_ARGUMENT, "kv_rows must be positive");
  for (int ph = 0; ph < 2; ++ph)
    if (a->phase_node_nums[ph] < 0 || a->phase_node_offsets[ph] < 0)
      return fail(FT_ERR_INVALID_ARGUMENT, "phase %d: negative vnode count or offset", ph);
  if (a->phase_node_nums[0] + a->phase_node_nums[1] > 0 || a->device_phase_info != nullptr) {
    if (!a->vnode_to_kv_entries || !a->vnode_to_kv_offs || !a->vnode_to_kv_lens || !a->vnode_to_q_entries ||
        !a->vnode_to_q_offs || !a->vnode_to_q_lens)
      return fail(FT_ERR_INVALID_ARGUMENT, "a vnode table pointer is NULL");
    if (a->kv_entries_len <= 0) return fail(FT_ERR_INVALID_ARGUMENT, "kv_entries_len must be positive");
  }
  if (a->num_kv_heads > 65535) return fail(FT_ERR_UNSUPPORTED, "more than 65535 kv heads");
  if (((int64_t)a->phase_node_nums[0] + a->phase_node_nums[1]) * a->num_kv_heads > 0x7fffffffLL)
    return fail(FT_ERR_TOO_LARGE, "vnodes x kv heads exceeds the grid limit");
  return FT_OK;
}

// Can the warp-MMA kernel take these arguments?  Returns a reason or NULL.
const char* mma_obstacle(const ft_decode_args* a) {
  if (a->dtype == FT_F32) return "fp32 inputs";
  if (a->head_dim != 64 && a->head_dim != 128) return "head_dim not 64 or 128";
  if (!aligned16(a->q) || !aligned16(a->k_buffer) || !aligned16(a->v_buffer)) return "q/k/v not 16-byte aligned";
  if (a->q_stride0 % 8 || a->q_stride1 % 8 || a->k_stride0 % 8 || a->k_stride1 % 8 || a->v_stride0 % 8 ||
      a->v_stride1 % 8)
    return "a q/k/v stride is not a multiple of 8 elements";
  // partial rows are written 16 bytes at a time
  if (!aligned16(a->mid_o) || a->mid_o_stride0 % 4 || a->mid_o_stride1 % 4) return "mid_o rows not 16-byte aligned";
  return nullptr;
}

int pick_path(const ft_decode_args* a) {
  const char* why = mma_obstacle(a);
  if (a->device_phase_info != nullptr) {  // only the persistent kernel has a grid that does not depend on the plan
    if (a->path != FT_PATH_AUTO && a->path != FT_PATH_PERSIST)
      return fail(FT_ERR_UNSUPPORTED, "device_phase_info needs path AUTO or PERSIST, got %d", a->path);
    if (why != nullptr || a->head_dim != 128)
      return fail(FT_ERR_UNSUPPORTED, "device_phase_info needs the persistent kernel: 16-bit types, head_dim 128, aligned buffers%s%s",
                  why ? "; " : "", why ? why : "");
    return FT_PATH_PERSIST;
  }
  if (a->path == FT_PATH_GENERIC) return FT_PATH_GENERIC;
  if (a->path == FT_PATH_MMA || a->path == FT_PATH_TCGEN05 || a->path == FT_PATH_MMA_WIDE || a->path == FT_PATH_STREAM ||
      a->path == FT_PATH_PERSIST) {
    if (why != nullptr) return fail(FT_ERR_UNSUPPORTED, "tensor-core path unavailable: %s", why);
    if ((a->path == FT_PATH_TCGEN05 || a->path == FT_PATH_PERSIST) && a->head_dim != 128)
      return fail(FT_ERR_UNSUPPORTED, "the tcgen05 kernels need head_dim 128, got %d", a->head_dim);
    return a->path;
  }
  if (a->path != FT_PATH_AUTO) return fail(FT_ERR_INVALID_ARGUMENT, "unknown path %d", a->path);
  return why == nullptr ? FT_PATH_AUTO : FT_PATH_GENERIC;
}

ft::Stage1Params stage1_params(const ft_decode_args* a) {
  ft::Stage1Params p;
  p.q = a->q;
  p.k = a->k_buffer;
  p.v = a->v_buffer;
  p.kv_entries = a->vnode_to_kv_entries;
  p.kv_offs = a->vnode_to_kv_offs;
  p.kv_lens = a->vnode_to_kv_lens;
  p.q_entries = a->vnode_to_q_entries;
  p.q_offs = a->vnode_to_q_offs;
  p.q_lens = a->vnode_to_q_lens;
  p.q_ranges = a->vnode_q_kv_ranges;
  p.dev_phase = a->device_phase_info;
  p.kv_entries_aux = a->vnode_to_kv_entries_aux;
  p.kv_entries_aux_len = a->vnode_to_kv_entries_aux != nullptr ? a->kv_entries_aux_len : 0;
  p.mid_o = a->mid_o;
  p.mid_lse = a->mid_lse;
  p.q_s0 = a->q_stride0;
  p.q_s1 = a->q_stride1;
  p.k_s0 = a->k_stride0;
  p.k_s1 = a->k_stride1;
  p.v_s0 = a->v_stride0;
  p.v_s1 = a->v_stride1;
  p.mo_s0 = a->mid_o_stride0;
  p.mo_s1 = a->mid_o_stride1;
  p.ml_s0 = a->mid_lse_stride0;
  p.kv_rows = a->kv_rows;
  p.kv_entries_len = a->kv_entries_len;
  p.num_partial_rows = a->num_partial_rows;
  p.batch = a->batch;
  p.group = a->num_qo_heads / a->num_kv_heads;
  p.head_dim = a->head_dim;
  p.node_offset = 0;
  p.node_count = 0;
  p.node_split = 0;
  p.lead_wide = 0;
  p.workers = 0;
  p.num_kv_heads = a->num_kv_heads;
  p.sm_scale = a->sm_scale;
  return p;
}

// Every stage-1 kernel is launched with permission to be scheduled before the preceding kernel of the stream has
// drained (programmatic dependent launch).  The kernels do nothing but on-chip set-up before their
// griddepcontrol.wait, which returns once the preceding kernel has completed and its writes are visible, so the
// permission is safe after any kernel; it pays after kernels that release their dependents early, as both stages of
// this library do: back-to-back decode calls overlap each launch and set-up with the previous kernel's tail.
template <typename... KArgs, typename... Args>
cudaError_t launch_early(void (*kernel)(KArgs...), dim3 grid, unsigned block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <typename T, int D>
int launch_mma(const ft::Stage1Params& p, int hkv, cudaStream_t st) {
  using C = ft::MmaCfg<D>;
  if (dry_run("stage1_mma_kernel")) return FT_OK;
  static OncePerDevice once;
  FT_CUDA_OK(raise_smem_limit(once, ft::stage1_mma_kernel<T, D>, C::SMEM_BYTES));
  const unsigned grid = (unsigned)p.node_count * (unsigned)hkv;
  FT_CUDA_OK(launch_early(ft::stage1_mma_kernel<T, D>, grid, C::THREADS, C::SMEM_BYTES, st, p));
  count_launch();
  return FT_OK;
}

template <typename T, int D>
int launch_narrow(const ft::Stage1Params& p, int hkv, cudaStream_t st) {
  using C = ft::NarrowCfg<D, 2>;
  if (dry_run("stage1_narrow_kernel")) return FT_OK;
  static OncePerDevice once;
  FT_CUDA_OK(raise_smem_limit(once, ft::stage1_narrow_kernel<T, D>, C::SMEM_BYTES));
  const unsigned grid = (unsigned)p.node_count * (unsigned)hkv;
  FT_CUDA_OK(launch_early(ft::stage1_narrow_kernel<T, D>, grid, 128, C::SMEM_BYTES, st, p));
  count_launch();
  return FT_OK;
}

int sm_count(int dev) {
  static std::atomic<int> sms[64];
  if (dev < 0 || dev >= 64) return 148;
  int n = sms[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    sms[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// Persistent few-row kernel: two CTAs per SM, each walking its share of the tasks.
template <typename T, int D>
int launch_stream(const ft::TcParams& tp, int hkv, cudaStream_t st) {
  using C = ft::StreamCfg<D>;
  if (dry_run("stage1_stream_kernel")) return FT_OK;
  static OncePerDevice once;
  int dev = 0;
  FT_CUDA_OK(raise_smem_limit(once, ft::stage1_stream_kernel<T, D>, C::SMEM_BYTES, &dev));
  const int64_t tasks = (int64_t)tp.p.node_count * hkv;
  const int64_t slots = 2LL * sm_count(dev);
  const unsigned grid = (unsigned)(tasks < slots ? tasks : slots);
  FT_CUDA_OK(launch_early(ft::stage1_stream_kernel<T, D>, grid, 128, C::SMEM_BYTES, st, tp));
  count_launch();
  return FT_OK;
}

// ---- TMA descriptors of the K / V buffers for the tcgen05 kernel -------------------------------------------
// The driver entry point is looked up through the runtime, so the library has no link-time dependency on libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

struct MapKey {
  const void* base;
  int64_t rows, s0, s1;
  int heads, dtype, box_heads, device;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && s0 == o.s0 && s1 == o.s1 && heads == o.heads && dtype == o.dtype &&
           box_heads == o.box_heads && device == o.device;
  }
};

// Descriptor of a [rows, heads, head_dim] 16-bit tensor (element strides s0, s1), box 64 (head_dim) x box_heads x
// box_rows, 128-byte swizzle.  Descriptors are cached by buffer identity (encoding one costs about a microsecond)
// in a hash table of 1024 slots, probed linearly over 8 slots; a full neighbourhood evicts its first slot.  A
// serving process holds two descriptors per layer's K/V buffer plus two per query shape - a few hundred at most.
bool tensor_map_3d(CUtensorMap* out, const void* base, int dtype, int head_dim, int64_t rows, int heads, int64_t s0,
                   int64_t s1, int box_heads, int box_rows) {
  constexpr int SLOTS = 1024, PROBES = 8;
  static std::mutex mu;
  static MapKey keys[SLOTS];
  static CUtensorMap maps[SLOTS];
  static bool used[SLOTS] = {};
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess) return false;  // the same address can name different memory on two devices
  const MapKey key{base, rows, s0, s1, heads, dtype + 16 * head_dim, box_heads * 1024 + box_rows, device};
  uint64_t h = reinterpret_cast<uintptr_t>(base) >> 8;
  h = (h ^ (uint64_t)key.box_heads * 0x9E3779B97F4A7C15ull ^ (uint64_t)(device + 1) * 0xC2B2AE3D27D4EB4Full ^
       (uint64_t)rows * 0x165667B19E3779F9ull) * 0xFF51AFD7ED558CCDull;
  const int home = (int)(h >> 40) & (SLOTS - 1);
  std::lock_guard<std::mutex> lock(mu);
  int slot = -1;
  for (int i = 0; i < PROBES; ++i) {
    const int j = (home + i) & (SLOTS - 1);
    if (used[j] && keys[j] == key) {
      *out = maps[j];
      return true;
    }
    if (!used[j] && slot < 0) slot = j;
  }
  if (slot < 0) slot = home;
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr || rows <= 0 || rows > 0x7fffffffLL || heads <= 0) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)head_dim, (cuuint64_t)heads, (cuuint64_t)rows};
  const cuuint64_t strides[2] = {(cuuint64_t)s1 * 2, (cuuint64_t)s0 * 2};  // bytes, for dimensions 1 and 2
  const cuuint32_t box[3] = {64, (cuuint32_t)box_heads, (cuuint32_t)box_rows};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMap m;
  const CUresult rc = enc(&m, dtype == FT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                          const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return false;
  keys[slot] = key;
  maps[slot] = m;
  used[slot] = true;
  *out = m;
  return true;
}

ft::TcParams tc_params(const ft::Stage1Params& p, const ft_decode_args* a) {
  ft::TcParams tp;
  memset(&tp, 0, sizeof(tp));
  tp.p = p;
  const int d = a->head_dim;
  tp.has_tma = tensor_map_3d(&tp.k_map, a->k_buffer, a->dtype, d, a->kv_rows, a->num_kv_heads, a->k_stride0,
                             a->k_stride1, 1, 64) &&
               tensor_map_3d(&tp.v_map, a->v_buffer, a->dtype, d, a->kv_rows, a->num_kv_heads, a->v_stride0,
                             a->v_stride1, 1, 64);
  // Q by TMA (tcgen05 kernel, head_dim 128): one box per request covering its G heads (at most 8 per box), or one
  // box for a whole tile of consecutive requests, when G is a power of two up to 128
  const int g = p.group;
  if (tp.has_tma && d == 128 && g >= 1 && g <= 128 && (g & (g - 1)) == 0) {
    const int box_heads = g < 8 ? g : 8;
    if (tensor_map_3d(&tp.q_map, a->q, a->dtype, d, a->batch, a->num_qo_heads, a->q_stride0, a->q_stride1, box_heads, 1) &&
        tensor_map_3d(&tp.q_map_tile, a->q, a->dtype, d, a->batch, a->num_qo_heads, a->q_stride0, a->q_stride1, g, 128 / g))
      tp.q_box_rows = box_heads;
  }
  return tp;
}

template <typename T>
int launch_tc(const ft::TcParams& p, int hkv, cudaStream_t st) {
  using C = ft::TcCfg;
  if (dry_run("stage1_tc_kernel")) return FT_OK;
  static OncePerDevice once;
  FT_CUDA_OK(raise_smem_limit(once, ft::stage1_tc_kernel<T>, C::SMEM_BYTES));
  const unsigned grid = (unsigned)p.p.node_count * (unsigned)hkv;
  FT_CUDA_OK(launch_early(ft::stage1_tc_kernel<T>, grid, C::THREADS, C::SMEM_BYTES, st, p));
  count_launch();
  return FT_OK;
}

// Claim counters of the persistent kernel: 64 pairs used round-robin by successive launches (each launch leaves
// its pair at zero when its last CTA finishes, so a pair is reusable as soon as that launch is over; launches
// 64 apart do not overlap in practice).
static __device__ unsigned int g_sched_counters[64][2];

template <typename T>
int launch_persist(ft::TcParams p, int hkv, cudaStream_t st) {
  using C = ft::PsCfg;
  if (dry_run("stage1_persist_kernel")) return FT_OK;
  static OncePerDevice once;
  int dev = 0;
  FT_CUDA_OK(raise_smem_limit(once, ft::stage1_persist_kernel<T>, C::SMEM_BYTES, &dev));
  if (dev < 0 || dev >= 64) return fail(FT_ERR_UNSUPPORTED, "device ordinal %d outside 0..63", dev);
  static std::atomic<unsigned int*> counters_of_device[64];
  unsigned int* base = counters_of_device[dev].load(std::memory_order_acquire);
  if (base == nullptr) {
    FT_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&base), g_sched_counters));
    counters_of_device[dev].store(base, std::memory_order_release);
  }
  static std::atomic<unsigned int> next_pair{0};
  p.sched = base + 2 * (next_pair.fetch_add(1, std::memory_order_relaxed) % 64u);
  const int64_t slots = 2LL * sm_count(dev);  // two resident CTAs per SM
  int64_t tasks = (int64_t)p.p.node_count * hkv;
  if (p.p.dev_phase != nullptr) tasks = slots;  // the task count is only known on the device: a full grid
  if (tasks <= 0) return FT_OK;
  if (tasks > 0x7fffffffLL) return fail(FT_ERR_TOO_LARGE, "vnodes x kv heads exceeds the task limit");
  const unsigned grid = (unsigned)(tasks < slots ? tasks : slots);
  FT_CUDA_OK(launch_early(ft::stage1_persist_kernel<T>, grid, C::THREADS, C::SMEM_BYTES, st, p));
  count_launch();
  return FT_OK;
}

template <typename T>
int launch_fused(ft::TcParams p, int hkv, cudaStream_t st) {
  constexpr int smem_a = ft::TcCfg::SMEM_BYTES > ft::StreamCfg<128>::SMEM_BYTES ? ft::TcCfg::SMEM_BYTES
                                                                                : ft::StreamCfg<128>::SMEM_BYTES;
  constexpr int smem = smem_a > ft::NarrowCfg<128, 2>::SMEM_BYTES ? smem_a : ft::NarrowCfg<128, 2>::SMEM_BYTES;
  static_assert(smem <= 115712, "two CTAs must fit in one SM's shared memory");
  if (dry_run("stage1_fused_kernel")) return FT_OK;
  static OncePerDevice once;
  int dev = 0;
  FT_CUDA_OK(raise_smem_limit(once, ft::stage1_fused_kernel<T>, smem, &dev));
  // Few-row tasks: a full set of persistent workers when each would get several tasks and the many-row CTAs
  // do not fill the device more than once (the task pipeline then hides the per-task start-up; the workers
  // take the slots the many-row CTAs leave and, as those finish, theirs too); one CTA per task otherwise (the
  // hardware then slots the small CTAs in wherever a many-row CTA finishes).  Many-row CTAs go first.
  const int64_t wide = (int64_t)p.p.node_split * hkv;
  const int64_t few = (int64_t)(p.p.node_count - p.p.node_split) * hkv;
  const int64_t slots = 2LL * sm_count(dev);
#ifdef FT_FORCE_WORKERS  // developer builds: persistent workers in every free slot, whatever the task count
  const int64_t workers = few < slots - wide ? few : (slots - wide > slots / 4 ? slots - wide : slots);
#else
  const int64_t workers = few >= 4 * slots && wide <= slots ? slots : 0;
#endif
  const int64_t few_ctas = workers > 0 ? workers : few;
  const int64_t lead = wide;
  if (wide + few_ctas > 0x7fffffffLL) return fail(FT_ERR_TOO_LARGE, "vnodes x kv heads exceeds the grid limit");
  p.p.workers = (int)workers;
  p.p.lead_wide = (int)lead;
  FT_CUDA_OK(launch_early(ft::stage1_fused_kernel<T>, (unsigned)(wide + few_ctas), ft::TcCfg::THREADS, smem, st, p));
  count_launch();
  return FT_OK;
}

// path: AUTO (<= 16 rows: persistent workers or narrow; above: tcgen05 when head_dim is 128, else wide),
// STREAM (like AUTO, always the persistent workers), MMA (narrow / wide), MMA_WIDE (wide for everything),
// TCGEN05 (tcgen05 for everything)
template <typename T, int D>
int launch_tensor(const ft::Stage1Params& p, const ft_decode_args* a, int hkv, cudaStream_t st, int max_rows, int path) {
  if constexpr (D == 128) {
    if (path == FT_PATH_TCGEN05 || ((path == FT_PATH_AUTO || path == FT_PATH_STREAM) && max_rows > 16))
      return launch_tc<T>(tc_params(p, a), hkv, st);
  }
  if (max_rows <= 16) {
    // few-row tasks only: persistent workers when there are several tasks per CTA slot, else one CTA per task
    int dev = 0;
    FT_CUDA_OK(cudaGetDevice(&dev));
    const bool many = (int64_t)p.node_count * hkv >= 8LL * sm_count(dev);
    if (path == FT_PATH_STREAM || (path == FT_PATH_AUTO && many)) return launch_stream<T, D>(tc_params(p, a), hkv, st);
  }
  if (path != FT_PATH_MMA_WIDE && max_rows <= 16) return launch_narrow<T, D>(p, hkv, st);
  return launch_mma<T, D>(p, hkv, st);
}

// fp32 storage at head_dim 64 / 128 with 16-byte aligned rows: the tiled CUDA-core kernel
bool f32_tiled_ok(const ft_decode_args* a) {
  if (a->dtype != FT_F32 || (a->head_dim != 64 && a->head_dim != 128)) return false;
  if (!aligned16(a->q) || !aligned16(a->k_buffer) || !aligned16(a->v_buffer)) return false;
  return a->q_stride0 % 4 == 0 && a->q_stride1 % 4 == 0 && a->k_stride0 % 4 == 0 && a->k_stride1 % 4 == 0 &&
         a->v_stride0 % 4 == 0 && a->v_stride1 % 4 == 0;
}

template <int D>
int launch_f32(const ft::Stage1Params& p, int hkv, cudaStream_t st, int max_rows) {
  using C = ft::F32Cfg<D>;
  if (dry_run("stage1_f32_kernel")) return FT_OK;
  static OncePerDevice once;
  FT_CUDA_OK(raise_smem_limit(once, ft::stage1_f32_kernel<D>, C::SMEM_BYTES));
  const int blocks_z = (max_rows + C::ROWS - 1) / C::ROWS;
  if (blocks_z > 65535) return fail(FT_ERR_TOO_LARGE, "too many query rows per vnode for the fp32 kernel");
  dim3 grid(p.node_count, hkv, blocks_z);
  FT_CUDA_OK(launch_early(ft::stage1_f32_kernel<D>, grid, C::THREADS, C::SMEM_BYTES, st, p));
  count_launch();
  return FT_OK;
}

template <typename T>
int launch_generic(const ft::Stage1Params& p, int hkv, cudaStream_t st) {
  if (dry_run("stage1_generic_kernel")) return FT_OK;
  dim3 grid(p.node_count, hkv);
  FT_CUDA_OK(launch_early(ft::stage1_generic_kernel<T>, grid, 128, 0, st, p));
  count_launch();
  return FT_OK;
}

// max_rows: upper bound on query rows (requests x group) of the tasks in the range
int launch_stage1_range(const ft_decode_args* a, int path, int offset, int count, int max_rows) {
  if (count <= 0) return FT_OK;
  ft::Stage1Params p = stage1_params(a);
  p.node_offset = offset;
  p.node_count = count;
  cudaStream_t st = static_cast<cudaStream_t>(a->stream);
  const int hkv = a->num_kv_heads;
  if (path != FT_PATH_GENERIC) {
    if (a->dtype == FT_F16)
      return a->head_dim == 128 ? launch_tensor<__half, 128>(p, a, hkv, st, max_rows, path)
                                : launch_tensor<__half, 64>(p, a, hkv, st, max_rows, path);
    return a->head_dim == 128 ? launch_tensor<__nv_bfloat16, 128>(p, a, hkv, st, max_rows, path)
                              : launch_tensor<__nv_bfloat16, 64>(p, a, hkv, st, max_rows, path);
  }
  // fp32 storage: the tiled kernel when the caller named no path (FT_PATH_GENERIC stays the scalar kernel) and the
  // phase's request tile bounds its rows
  if (a->path == FT_PATH_AUTO && f32_tiled_ok(a) && max_rows > 0 && max_rows < (1 << 20))
    return a->head_dim == 128 ? launch_f32<128>(p, hkv, st, max_rows) : launch_f32<64>(p, hkv, st, max_rows);
  switch (a->dtype) {
    case FT_F16: return launch_generic<__half>(p, hkv, st);
    case FT_BF16: return launch_generic<__nv_bfloat16>(p, hkv, st);
    default: return launch_generic<float>(p, hkv, st);
  }
}

// after_stage1: this launch directly follows a stage-1 launch of the same call on the same stream.  Only then may
// the kernel be scheduled early (programmatic dependent launch): it reads the request tables before it waits for
// the preceding kernel, which is safe after stage 1 (that kernel never writes them) but not after an arbitrary
// kernel of the caller's that may still be building those tables.
template <typename T>
int launch_stage2(const ft::Stage2Params& p, cudaStream_t st, bool after_stage1) {
  const int64_t pairs = (int64_t)p.batch * p.heads;
  if (pairs == 0) return FT_OK;
  const int64_t blocks = (pairs + 3) / 4;
  if (blocks > 0x7fffffffLL) return fail(FT_ERR_TOO_LARGE, "batch x heads too large for one launch");
  // launched with permission to be scheduled before the preceding kernel (stage 1) has drained; the kernel itself
  // waits for that kernel's completion before it touches the partial buffers
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = after_stage1 ? 1 : 0;
  int dev = 0;
  FT_CUDA_OK(cudaGetDevice(&dev));
  const bool one_round = blocks <= 6LL * sm_count(dev);  // latency-bound: more rows in flight per lane
  if (p.head_dim > 128)
    FT_CUDA_OK(cudaLaunchKernelEx(&cfg, ft::stage2_merge_kernel<T, 2, 4>, p));
  else if (blocks <= 2LL * sm_count(dev))
    FT_CUDA_OK(cudaLaunchKernelEx(&cfg, ft::stage2_merge_kernel<T, 1, 16>, p));
  else if (one_round)
    FT_CUDA_OK(cudaLaunchKernelEx(&cfg, ft::stage2_merge_kernel<T, 1, 8>, p));
  else
    FT_CUDA_OK(cudaLaunchKernelEx(&cfg, ft::stage2_merge_kernel<T, 1, 4>, p));
  count_launch();
  return FT_OK;
}

__global__ void bump_kv_lens_kernel(int32_t* kv_lens, const int32_t* last, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const int v = last[i];
    if (v >= 0) atomicAdd(kv_lens + v, 1);
  }
}

}  // namespace

extern "C" {

int ft_version(void) { return 100; }

int ft_decode_args_size(void) { return static_cast<int>(sizeof(ft_decode_args)); }

const char* ft_last_error(void) { return g_err; }

int64_t ft_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* ft_stage1_path_name(const ft_decode_args* args) {
  g_kernel_names[0] = '\0';
  g_dry_run = true;
  const int rc = ft_stage1(args);
  g_dry_run = false;
  if (rc != FT_OK) return nullptr;
  return g_kernel_names;
}

int ft_stage1(const ft_decode_args* a) {
  int rc = check_common(a);
  if (rc != FT_OK) return rc;
  rc = check_stage1(a);
  if (rc != FT_OK) return rc;
  const int path = pick_path(a);
  if (path < 0) return path;
  const int n0 = a->phase_node_nums[0], n1 = a->phase_node_nums[1];
  const int o0 = a->phase_node_offsets[0], o1 = a->phase_node_offsets[1];
  const int group = a->num_qo_heads / a->num_kv_heads;
  // A phase's request tile bounds the query rows of its tasks; a non-positive tile size means "unknown".
  const int64_t r0 = a->phase_q_tile_sizes[0] > 0 ? (int64_t)a->phase_q_tile_sizes[0] * group : 1 << 30;
  const int64_t r1 = a->phase_q_tile_sizes[1] > 0 ? (int64_t)a->phase_q_tile_sizes[1] * group : 1 << 30;
  const int rows0 = (int)(r0 < (1 << 30) ? r0 : (1 << 30)), rows1 = (int)(r1 < (1 << 30) ? r1 : (1 << 30));
  const bool same_kernel = path == FT_PATH_GENERIC || path == FT_PATH_MMA_WIDE || path == FT_PATH_TCGEN05 ||
                           ((rows0 > 16) == (rows1 > 16));
  // the persistent kernel takes every task of the launch, whatever its row count
  if (path == FT_PATH_PERSIST && a->device_phase_info != nullptr) {
    ft::Stage1Params p = stage1_params(a);  // node_offset / node_count come from the device array
    const ft::TcParams tp = tc_params(p, a);
    cudaStream_t st = static_cast<cudaStream_t>(a->stream);
    return a->dtype == FT_F16 ? launch_persist<__half>(tp, a->num_kv_heads, st)
                              : launch_persist<__nv_bfloat16>(tp, a->num_kv_heads, st);
  }
  if (path == FT_PATH_PERSIST) {
    cudaStream_t st = static_cast<cudaStream_t>(a->stream);
    const bool joined = n0 > 0 && n1 > 0 && o1 == o0 + n0;
    for (int ph = 0; ph < (joined ? 1 : 2); ++ph) {
      ft::Stage1Params p = stage1_params(a);
      p.node_offset = ph == 0 ? o0 : o1;
      p.node_count = joined ? n0 + n1 : (ph == 0 ? n0 : n1);
      if (p.node_count <= 0) continue;
      const ft::TcParams tp = tc_params(p, a);
      rc = a->dtype == FT_F16 ? launch_persist<__half>(tp, a->num_kv_heads, st)
                              : launch_persist<__nv_bfloat16>(tp, a->num_kv_heads, st);
      if (rc != FT_OK) return rc;
    }
    return FT_OK;
  }
  // head_dim 128, many-row phase followed directly by the few-row phase: one grid with both kernel bodies
  if (path == FT_PATH_AUTO && a->head_dim == 128 && n0 > 0 && n1 > 0 && o1 == o0 + n0 && rows0 > 16 && rows1 <= 16) {
    ft::Stage1Params p = stage1_params(a);
    p.node_offset = o0;
    p.node_count = n0 + n1;
    p.node_split = n0;
    cudaStream_t st = static_cast<cudaStream_t>(a->stream);
    const ft::TcParams tp = tc_params(p, a);
    return a->dtype == FT_F16 ? launch_fused<__half>(tp, a->num_kv_heads, st)
                              : launch_fused<__nv_bfloat16>(tp, a->num_kv_heads, st);
  }
  // Adjacent phases that want the same kernel go out as one grid.
  if (n0 > 0 && n1 > 0 && o1 == o0 + n0 && same_kernel)
    return launch_stage1_range(a, path, o0, n0 + n1, rows0 > rows1 ? rows0 : rows1);
  rc = launch_stage1_range(a, path, o0, n0, rows0);
  if (rc != FT_OK) return rc;
  return launch_stage1_range(a, path, o1, n1, rows1);
}

namespace {
int stage2_impl(const ft_decode_args* a, bool after_stage1) {
  int rc = check_common(a);
  if (rc != FT_OK) return rc;
  if (a->o == nullptr) return fail(FT_ERR_INVALID_ARGUMENT, "o is NULL");
  if (a->batch > 0 && (!a->req_to_vnode_entries || !a->req_to_vnode_offs || !a->req_to_vnode_lens))
    return fail(FT_ERR_INVALID_ARGUMENT, "a request table pointer is NULL");
  ft::Stage2Params p;
  p.r2v_entries = a->req_to_vnode_entries;
  p.r2v_offs = a->req_to_vnode_offs;
  p.r2v_lens = a->req_to_vnode_lens;
  p.mid_o = a->mid_o;
  p.mid_lse = a->mid_lse;
  p.o = a->o;
  p.o_lse = a->o_lse;
  p.mo_s0 = a->mid_o_stride0;
  p.mo_s1 = a->mid_o_stride1;
  p.ml_s0 = a->mid_lse_stride0;
  p.o_s0 = a->o_stride0;
  p.o_s1 = a->o_stride1;
  p.num_partial_rows = a->num_partial_rows;
  p.batch = a->batch;
  p.heads = a->num_qo_heads;
  p.head_dim = a->head_dim;
  {
    const int64_t esz = a->dtype == FT_F32 ? 4 : 2, vec = 4 * esz;  // bytes of one 4-element store
    p.o_vec = (reinterpret_cast<uintptr_t>(a->o) % vec == 0 && (a->o_stride0 * esz) % vec == 0 &&
               (a->o_stride1 * esz) % vec == 0)
                  ? 1
                  : 0;
  }
  cudaStream_t st = static_cast<cudaStream_t>(a->stream);
  switch (a->dtype) {
    case FT_F16: return launch_stage2<__half>(p, st, after_stage1);
    case FT_BF16: return launch_stage2<__nv_bfloat16>(p, st, after_stage1);
    default: return launch_stage2<float>(p, st, after_stage1);
  }
}
}  // namespace

int ft_stage2(const ft_decode_args* a) { return stage2_impl(a, false); }

int ft_decode(const ft_decode_args* a) {
  const int64_t before = t_launches;
  int rc = ft_stage1(a);
  if (rc != FT_OK) return rc;
  // a plan without vnodes launches no stage 1: stage 2 then follows whatever the caller enqueued before
  const bool launched = t_launches != before;
  return stage2_impl(a, launched);
}

namespace {
// Host-to-device copy done by the SMs: 16 bytes per thread from mapped pinned host memory.  For the few hundred
// KiB of a decode step's query this is several microseconds quicker than a copy-engine transfer, whose set-up
// and completion hand-shake dominate at that size.
__global__ void __launch_bounds__(256) host_to_device_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, size_t n16,
                                                             unsigned char* dst_tail, const unsigned char* src_tail, int tail) {
  // stage 1 may set itself up (barriers, tensor memory) while the query crosses PCIe; it waits for this kernel's
  // completion before it reads anything
  ft::allow_dependent_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n16) dst[i] = src[i];
  if (i < (size_t)tail) dst_tail[i] = src_tail[i];
}
}  // namespace

int ft_decode_host_io(const ft_decode_args* a, const void* q_host, void* o_host, int wait) {
  if (a == nullptr) return fail(FT_ERR_INVALID_ARGUMENT, "args is NULL");
  if (q_host == nullptr || o_host == nullptr) return fail(FT_ERR_INVALID_ARGUMENT, "q_host / o_host is NULL");
  if (a->q == nullptr || a->o == nullptr) return fail(FT_ERR_INVALID_ARGUMENT, "q / o (device staging buffers) is NULL");
  if (a->batch < 0 || a->num_qo_heads <= 0 || a->head_dim <= 0)
    return fail(FT_ERR_INVALID_ARGUMENT, "batch / num_qo_heads / head_dim must be positive");
  const int64_t row = (int64_t)a->num_qo_heads * a->head_dim;
  if (a->q_stride1 != a->head_dim || a->q_stride0 != row || a->o_stride1 != a->head_dim || a->o_stride0 != row)
    return fail(FT_ERR_UNSUPPORTED, "ft_decode_host_io needs packed [batch, heads, head_dim] device q and o");
  const size_t esz = a->dtype == FT_F32 ? 4 : 2;
  const size_t bytes = (size_t)a->batch * (size_t)row * esz;
  cudaStream_t st = static_cast<cudaStream_t>(a->stream);
  if (bytes == 0) return ft_decode(a);
  // Pinned host memory is mapped into the device's address space: the query is then fetched by a small kernel and
  // stage 2 writes the output rows straight into o_host over PCIe, so no copy-engine transfer sits on the step's
  // critical path.  Memory that is not mapped (pageable, or registered without the mapped flag) takes the copy
  // engine, one cudaMemcpyAsync per buffer.
  void *q_map = nullptr, *o_map = nullptr;
  const bool mapped = cudaHostGetDevicePointer(&q_map, const_cast<void*>(q_host), 0) == cudaSuccess &&
                      cudaHostGetDevicePointer(&o_map, o_host, 0) == cudaSuccess && aligned16(q_map) && aligned16(a->q) &&
                      aligned16(o_map);
  if (!mapped) {
    (void)cudaGetLastError();  // the failed query left an error behind
    FT_CUDA_OK(cudaMemcpyAsync(const_cast<void*>(a->q), q_host, bytes, cudaMemcpyHostToDevice, st));
    const int rc = ft_decode(a);
    if (rc != FT_OK) return rc;
    FT_CUDA_OK(cudaMemcpyAsync(o_host, a->o, bytes, cudaMemcpyDeviceToHost, st));
    if (wait) FT_CUDA_OK(cudaStreamSynchronize(st));
    return FT_OK;
  }
  const size_t n16 = bytes / 16;
  const int tail = (int)(bytes % 16);
  const unsigned blocks = (unsigned)((n16 + (tail ? 1 : 0) + 255) / 256);
  host_to_device_kernel<<<blocks, 256, 0, st>>>(static_cast<uint4*>(const_cast<void*>(a->q)), static_cast<const uint4*>(q_map), n16,
                                                static_cast<unsigned char*>(const_cast<void*>(a->q)) + 16 * n16,
                                                static_cast<const unsigned char*>(q_map) + 16 * n16, tail);
  FT_CUDA_OK(cudaGetLastError());
  count_launch();
  ft_decode_args b = *a;
  b.o = o_map;  // stage 2 writes the merged rows into host memory; the device staging buffer args->o is not used
  const int rc = ft_decode(&b);
  if (rc != FT_OK) return rc;
  if (wait) FT_CUDA_OK(cudaStreamSynchronize(st));
  return FT_OK;
}

// ---- ft_decode_static_scratch: partial-result scratch in a fixed device array owned by the library ----------
//
// The array lives in every CUDA context that loads this library, from load until exit.  In host code its name is
// only a stand-in for the device symbol, so the device address is looked up once per device with
// cudaGetSymbolAddress (that device being current) and that address is what the kernels receive.
#define FT_STATIC_SCRATCH_FLOATS (FT_STATIC_SCRATCH_BYTES / 4u)
static __device__ __align__(256) float g_static_scratch[FT_STATIC_SCRATCH_FLOATS];

int ft_decode_static_scratch(const ft_decode_args* a) {
  if (a == nullptr) return fail(FT_ERR_INVALID_ARGUMENT, "args is NULL");
  if (a->num_partial_rows < 0 || a->num_qo_heads <= 0 || a->head_dim <= 0)
    return fail(FT_ERR_INVALID_ARGUMENT, "num_partial_rows / num_qo_heads / head_dim must be positive");
  const int64_t per_row = (int64_t)a->num_qo_heads * (a->head_dim + 1);
  if (a->num_partial_rows > (int64_t)FT_STATIC_SCRATCH_FLOATS / per_row)
    return fail(FT_ERR_TOO_LARGE,
                "plan needs %lld partial rows x %d heads x (%d+1) floats = %lld bytes of scratch; the built-in array "
                "holds %u bytes - use ft_decode with caller-owned mid_o / mid_lse",
                (long long)a->num_partial_rows, a->num_qo_heads, a->head_dim,
                (long long)(a->num_partial_rows * per_row * 4), (unsigned)(4u * FT_STATIC_SCRATCH_FLOATS));
  static float* scratch_of_device[64] = {};
  int dev = 0;
  FT_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(FT_ERR_UNSUPPORTED, "device ordinal %d outside 0..63", dev);
  if (scratch_of_device[dev] == nullptr) {  // set-up: first call on this device
    float* ptr = nullptr;
    FT_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch));
    if (ptr == nullptr) return fail(FT_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    scratch_of_device[dev] = ptr;
  }
  ft_decode_args b = *a;
  b.mid_o = scratch_of_device[dev];
  b.mid_o_stride0 = (int64_t)a->num_qo_heads * a->head_dim;
  b.mid_o_stride1 = a->head_dim;
  b.mid_lse = b.mid_o + a->num_partial_rows * b.mid_o_stride0;
  b.mid_lse_stride0 = a->num_qo_heads;
  return ft_decode(&b);
}

int ft_bump_kv_lens(int32_t* vnode_to_kv_lens, const int32_t* last_vnodes, int32_t n, void* stream) {
  if (n < 0) return fail(FT_ERR_INVALID_ARGUMENT, "n is negative");
  if (n == 0) return FT_OK;
  if (vnode_to_kv_lens == nullptr || last_vnodes == nullptr)
    return fail(FT_ERR_INVALID_ARGUMENT, "vnode_to_kv_lens / last_vnodes is NULL");
  bump_kv_lens_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(vnode_to_kv_lens, last_vnodes, n);
  FT_CUDA_OK(cudaGetLastError());
  count_launch();
  return FT_OK;
}

namespace {
// one warp per segment of the auxiliary row-id table
__global__ void gather_kv_entries_kernel(const int32_t* __restrict__ src, int64_t src_len, const int32_t* __restrict__ seg_src,
                                         const int32_t* __restrict__ seg_len, const int32_t* __restrict__ seg_dst,
                                         const int32_t* __restrict__ seg_room, int n, int32_t* __restrict__ aux, int64_t aux_len) {
  const int seg = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (seg >= n) return;
  const int64_t from = seg_src[seg], len = seg_len[seg], to = seg_dst[seg], room = seg_room[seg];
  if (len <= 0 || room < 0 || from < 0 || from + len > src_len || to < 0 || to + len + room > aux_len) {
    if (lane == 0 && (len != 0 || room != 0)) ft::flag_error(FT_DEV_BAD_KV_INDEX);
    return;
  }
  for (int64_t i = lane; i < len; i += 32) aux[to + i] = src[from + i];
  const int32_t filler = src[from];
  for (int64_t i = lane; i < room; i += 32) aux[to + len + i] = filler;
}

__global__ void bump_tails_kernel(int32_t* __restrict__ state, int n, int32_t* __restrict__ ranges, int64_t rows,
                                  int32_t* __restrict__ kv_lens, int n_vnodes) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int32_t* st = state + 4 * (int64_t)i;
  const int aux_pos = st[0], index = st[2], room = st[3];
  if (aux_pos < 0) {
    if (index >= 0 && index < n_vnodes) kv_lens[index] += 1;
    else if (index != -1) ft::flag_error(FT_DEV_BAD_ROW_INDEX);  // {-1, x, -1, x}: an unused entry
    return;
  }
  if (room <= 0 || ranges == nullptr || index < 0 || index >= rows) {
    ft::flag_error(FT_DEV_BAD_KV_INDEX);
    return;
  }
  ranges[2 * (int64_t)index + 1] += 1;
  st[0] = aux_pos + 1;
  st[1] += 1;
  st[3] = room - 1;
}

__global__ void refresh_tails_kernel(const int32_t* __restrict__ state, int n, const int32_t* __restrict__ src, int64_t src_len,
                                     int32_t* __restrict__ aux, int64_t aux_len) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int32_t* st = state + 4 * (int64_t)i;
  const int64_t aux_pos = st[0], src_pos = st[1];
  if (aux_pos < 0) return;
  if (aux_pos < 1 || aux_pos > aux_len || src_pos < 1 || src_pos > src_len) {
    ft::flag_error(FT_DEV_BAD_KV_INDEX);
    return;
  }
  aux[aux_pos - 1] = src[src_pos - 1];
}
}  // namespace

int ft_gather_kv_entries(const int32_t* src_table, int64_t src_len, const int32_t* seg_src, const int32_t* seg_len,
                         const int32_t* seg_dst, const int32_t* seg_room, int32_t n_segments, int32_t* aux_table,
                         int64_t aux_len, void* stream) {
  if (n_segments < 0 || src_len < 0 || aux_len < 0) return fail(FT_ERR_INVALID_ARGUMENT, "negative size");
  if (n_segments == 0) return FT_OK;
  if (src_table == nullptr || seg_src == nullptr || seg_len == nullptr || seg_dst == nullptr || seg_room == nullptr ||
      aux_table == nullptr)
    return fail(FT_ERR_INVALID_ARGUMENT, "a table of ft_gather_kv_entries is NULL");
  gather_kv_entries_kernel<<<(n_segments + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src_table, src_len, seg_src, seg_len, seg_dst, seg_room, n_segments, aux_table, aux_len);
  FT_CUDA_OK(cudaGetLastError());
  count_launch();
  return FT_OK;
}

int ft_bump_tails(int32_t* tail_state, int32_t n, int32_t* vnode_q_kv_ranges, int64_t num_partial_rows,
                  int32_t* vnode_to_kv_lens, int32_t num_vnodes, void* stream) {
  if (n < 0 || num_partial_rows < 0 || num_vnodes < 0) return fail(FT_ERR_INVALID_ARGUMENT, "negative size");
  if (n == 0) return FT_OK;
  if (tail_state == nullptr || vnode_to_kv_lens == nullptr)
    return fail(FT_ERR_INVALID_ARGUMENT, "tail_state / vnode_to_kv_lens is NULL");
  bump_tails_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      tail_state, n, vnode_q_kv_ranges, num_partial_rows, vnode_to_kv_lens, num_vnodes);
  FT_CUDA_OK(cudaGetLastError());
  count_launch();
  return FT_OK;
}

int ft_refresh_tails(const int32_t* tail_state, int32_t n, const int32_t* src_table, int64_t src_len, int32_t* aux_table,
                     int64_t aux_len, void* stream) {
  if (n < 0 || src_len < 0 || aux_len < 0) return fail(FT_ERR_INVALID_ARGUMENT, "negative size");
  if (n == 0) return FT_OK;
  if (tail_state == nullptr || src_table == nullptr || aux_table == nullptr)
    return fail(FT_ERR_INVALID_ARGUMENT, "tail_state / src_table / aux_table is NULL");
  refresh_tails_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(tail_state, n, src_table, src_len,
                                                                                        aux_table, aux_len);
  FT_CUDA_OK(cudaGetLastError());
  count_launch();
  return FT_OK;
}

namespace {
// One warp waits on an mbarrier that nothing ever arrives at, through the same bounded waits the stage-1 kernels
// use.  No copy, no MMA and no tensor memory is involved, so a wait that runs out leaves nothing in flight.
__global__ void bounded_wait_selftest_kernel(int limit, int* result) {
  __shared__ __align__(8) unsigned long long barrier_word;
  __shared__ int abort_word;
  const uint32_t bar = ft::smem_u32(&barrier_word);
  if (threadIdx.x == 0) {
    ft::mbar_init(bar, 1);
    abort_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  // (1) the plain bounded wait of the persistent workers: gives up after `limit` probes
  const bool plain = ft::mbar_wait(bar, 0, limit);
  // (2) the tcgen05 kernel's wait: same limit semantics (its own constant), and it leaves early once a sibling
  // role has raised the CTA's abort flag - raised here by lane 0 before the call
  if (threadIdx.x == 0) abort_word = 1;
  __syncthreads();
  const bool aborted = ft::tc_wait(bar, 0, &abort_word);
  if (threadIdx.x == 0) {
    if (!plain || !aborted) ft::flag_error(FT_DEV_WAIT_TIMEOUT);  // what the kernels do when a wait runs out
    result[0] = plain ? 1 : 0;
    result[1] = aborted ? 1 : 0;
  }
}
}  // namespace

int ft_selftest_bounded_wait(int limit, int* result_host, void* stream) {
  if (result_host == nullptr) return fail(FT_ERR_INVALID_ARGUMENT, "result_host is NULL");
  if (limit < 1 || limit > (1 << 20)) return fail(FT_ERR_INVALID_ARGUMENT, "limit must be in [1, 2^20] probes");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int* dev = nullptr;
  FT_CUDA_OK(cudaMalloc(&dev, 2 * sizeof(int)));
  bounded_wait_selftest_kernel<<<1, 32, 0, st>>>(limit, dev);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaMemcpyAsync(result_host, dev, 2 * sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  cudaFree(dev);
  if (e != cudaSuccess) return fail(FT_ERR_CUDA, "bounded-wait self-test failed: %s", cudaGetErrorString(e));
  count_launch();
  return FT_OK;
}

#ifdef FT_TIMELINE
// Developer builds only: copies the first n per-CTA records {start ns, end ns, SM id, kind, 12 marks} of the last stage-1 launch.
int ft_debug_timeline(unsigned long long* out, int n) {
  if (out == nullptr || n < 0 || n > ft::FT_TIMELINE_CTAS) return fail(FT_ERR_INVALID_ARGUMENT, "bad timeline request");
  FT_CUDA_OK(cudaDeviceSynchronize());
  FT_CUDA_OK(cudaMemcpyFromSymbol(out, ft::g_timeline, sizeof(unsigned long long) * 16 * (size_t)n));
  return FT_OK;
}
#endif

int ft_read_wait_diagnostics(int32_t* out8) {
  if (out8 == nullptr) return fail(FT_ERR_INVALID_ARGUMENT, "out8 is NULL");
  FT_CUDA_OK(cudaDeviceSynchronize());
  FT_CUDA_OK(cudaMemcpyFromSymbol(out8, ft::g_wait_diag, 8 * sizeof(int)));
  if (out8[0] != 0) {
    const int zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    FT_CUDA_OK(cudaMemcpyToSymbol(ft::g_wait_diag, zero, sizeof(zero)));
  }
  return FT_OK;
}

int ft_read_device_status(void* stream, int32_t* flags) {
  if (flags == nullptr) return fail(FT_ERR_INVALID_ARGUMENT, "flags is NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  FT_CUDA_OK(cudaStreamSynchronize(st));
  int host = 0;
  FT_CUDA_OK(cudaMemcpyFromSymbol(&host, ft::g_device_status, sizeof(int)));
  if (host != 0) {
    const int zero = 0;
    FT_CUDA_OK(cudaMemcpyToSymbol(ft::g_device_status, &zero, sizeof(int)));
  }
  *flags = host;
  return FT_OK;
}

}  // extern "C"
