"""ctypes binding of libfasttree_b200.so (declarations: include/fasttree_b200.h).

The library is the only compute path.  If it cannot be loaded (not built and
no nvcc to build it with) every entry point raises :class:`FastTreeError`;
there is no PyTorch or CPU fallback.
"""
import ctypes
import os
import threading

from . import build as _build

FT_F16, FT_BF16, FT_F32 = 0, 1, 2
FT_PATH_AUTO, FT_PATH_GENERIC, FT_PATH_MMA, FT_PATH_TCGEN05, FT_PATH_MMA_WIDE, FT_PATH_STREAM, FT_PATH_PERSIST = 0, 1, 2, 3, 4, 5, 6
PATHS = {"auto": FT_PATH_AUTO, "generic": FT_PATH_GENERIC, "mma": FT_PATH_MMA, "tcgen05": FT_PATH_TCGEN05,
         "mma_wide": FT_PATH_MMA_WIDE, "stream": FT_PATH_STREAM, "persist": FT_PATH_PERSIST}

FT_STATIC_SCRATCH_BYTES = 16 << 20      # capacity of the array behind ft_decode_static_scratch

FT_DEV_BAD_KV_INDEX, FT_DEV_BAD_Q_INDEX, FT_DEV_BAD_ROW_INDEX, FT_DEV_WAIT_TIMEOUT = 1, 2, 4, 8

EXPORTS = ["ft_version", "ft_decode_args_size", "ft_last_error", "ft_decode", "ft_stage1", "ft_stage2",
           "ft_decode_static_scratch", "ft_decode_host_io", "ft_selftest_bounded_wait", "ft_read_wait_diagnostics", "ft_bump_kv_lens",
           "ft_gather_kv_entries", "ft_bump_tails", "ft_refresh_tails",
           "ft_read_device_status", "ft_launch_count", "ft_stage1_path_name",
           "ft_plan_b200_build", "ft_plan_b200_build_direct", "ft_plan_get_info", "ft_plan_copy_tables", "ft_plan_copy_row_ranges",
           "ft_plan_copy_aux_segments",
           "ft_plan_free"]


class FastTreeError(RuntimeError):
    """A C-ABI call returned a negative status; ``code`` holds it."""

    def __init__(self, code, message):
        super().__init__(f"fasttree_b200 error {code}: {message}")
        self.code = code


class B200ModelStruct(ctypes.Structure):
    """Mirror of ``struct ft_b200_model``."""
    _fields_ = [("num_sms", ctypes.c_int32), ("ctas_per_sm", ctypes.c_int32), ("waves", ctypes.c_double),
                ("tile_tokens", ctypes.c_int32), ("rows_per_cta", ctypes.c_int32), ("min_chunk", ctypes.c_int32),
                ("nominal_split", ctypes.c_int32), ("ridge_flop_per_byte", ctypes.c_double),
                ("task_overhead_bytes", ctypes.c_int32), ("elem_bytes", ctypes.c_int32),
                ("group_member_tokens", ctypes.c_int32), ("group_min_members", ctypes.c_int32)]


class PlanInfo(ctypes.Structure):
    """Mirror of ``struct ft_plan_info``."""
    _fields_ = [("kv_entries", ctypes.c_int64), ("vnodes", ctypes.c_int64), ("partial_rows", ctypes.c_int64),
                ("batch", ctypes.c_int64), ("nodes", ctypes.c_int64), ("virtual_nodes", ctypes.c_int64),
                ("phase_node_nums", ctypes.c_int32 * 2), ("phase_node_offsets", ctypes.c_int32 * 2),
                ("q_tile", ctypes.c_int32), ("small_tile", ctypes.c_int32), ("tile_tokens", ctypes.c_int32),
                ("has_row_ranges", ctypes.c_int32), ("target_bytes", ctypes.c_double),
                ("aux_entries", ctypes.c_int64), ("aux_segments", ctypes.c_int64)]


class DecodeArgs(ctypes.Structure):
    """Mirror of ``struct ft_decode_args``."""
    _fields_ = [
        ("q", ctypes.c_void_p), ("k_buffer", ctypes.c_void_p), ("v_buffer", ctypes.c_void_p),
        ("o", ctypes.c_void_p), ("o_lse", ctypes.c_void_p),
        ("dtype", ctypes.c_int32), ("batch", ctypes.c_int32), ("num_qo_heads", ctypes.c_int32),
        ("num_kv_heads", ctypes.c_int32), ("head_dim", ctypes.c_int32), ("path", ctypes.c_int32),
        ("kv_rows", ctypes.c_int64),
        ("q_stride0", ctypes.c_int64), ("q_stride1", ctypes.c_int64),
        ("k_stride0", ctypes.c_int64), ("k_stride1", ctypes.c_int64),
        ("v_stride0", ctypes.c_int64), ("v_stride1", ctypes.c_int64),
        ("o_stride0", ctypes.c_int64), ("o_stride1", ctypes.c_int64),
        ("vnode_to_kv_entries", ctypes.c_void_p), ("kv_entries_len", ctypes.c_int64),
        ("vnode_to_kv_offs", ctypes.c_void_p), ("vnode_to_kv_lens", ctypes.c_void_p),
        ("vnode_to_q_entries", ctypes.c_void_p), ("vnode_to_q_offs", ctypes.c_void_p),
        ("vnode_to_q_lens", ctypes.c_void_p),
        ("req_to_vnode_entries", ctypes.c_void_p), ("req_to_vnode_offs", ctypes.c_void_p),
        ("req_to_vnode_lens", ctypes.c_void_p),
        ("num_partial_rows", ctypes.c_int64),
        ("phase_node_nums", ctypes.c_int32 * 2), ("phase_node_offsets", ctypes.c_int32 * 2),
        ("phase_q_tile_sizes", ctypes.c_int32 * 2), ("phase_kv_tile_sizes", ctypes.c_int32 * 2),
        ("mid_o", ctypes.c_void_p), ("mid_lse", ctypes.c_void_p),
        ("mid_o_stride0", ctypes.c_int64), ("mid_o_stride1", ctypes.c_int64),
        ("mid_lse_stride0", ctypes.c_int64),
        ("sm_scale", ctypes.c_float), ("logit_cap", ctypes.c_float),
        ("stream", ctypes.c_void_p),
        ("vnode_q_kv_ranges", ctypes.c_void_p),
        ("device_phase_info", ctypes.c_void_p),
        ("vnode_to_kv_entries_aux", ctypes.c_void_p),
        ("kv_entries_aux_len", ctypes.c_int64),
    ]


_lock = threading.Lock()
_lib = None


def library_path():
    return _build.LIB_PATH


def load():
    """Load the library and declare the C ABI.  It is built first when it is missing or older than any of its
    sources (and nvcc is there to build it); a stale library that cannot be rebuilt is an error, not a silent
    run of old kernels."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = os.environ.get("FT_B200_LIBRARY") or _build.LIB_PATH      # a prebuilt library elsewhere, if named
        if path == _build.LIB_PATH and (_build._stale() or os.environ.get("FT_B200_REBUILD") == "1"):
            try:
                _build.build_library(force=True)
            except Exception as exc:  # no nvcc, or the compile failed
                state = "missing" if not os.path.exists(path) else "older than its sources"
                raise FastTreeError(-3, f"libfasttree_b200.so is {state} and could not be built: {exc}") from exc
        try:
            lib = ctypes.CDLL(path)
        except OSError as exc:
            raise FastTreeError(-3, f"cannot load {path}: {exc}") from exc
        argp = ctypes.POINTER(DecodeArgs)
        lib.ft_version.restype = ctypes.c_int
        lib.ft_decode_args_size.restype = ctypes.c_int
        if lib.ft_decode_args_size() != ctypes.sizeof(DecodeArgs):
            raise FastTreeError(-1, "struct ft_decode_args of the library (%d bytes) differs from the binding (%d)"
                                % (lib.ft_decode_args_size(), ctypes.sizeof(DecodeArgs)))
        lib.ft_last_error.restype = ctypes.c_char_p
        for name in ("ft_decode", "ft_stage1", "ft_stage2", "ft_decode_static_scratch"):
            fn = getattr(lib, name)
            fn.argtypes = [argp]
            fn.restype = ctypes.c_int
        lib.ft_decode_host_io.argtypes = [argp, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        lib.ft_decode_host_io.restype = ctypes.c_int
        lib.ft_selftest_bounded_wait.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_void_p]
        lib.ft_selftest_bounded_wait.restype = ctypes.c_int
        lib.ft_bump_kv_lens.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p]
        lib.ft_bump_kv_lens.restype = ctypes.c_int
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
        lib.ft_gather_kv_entries.argtypes = [vp, i64, vp, vp, vp, vp, i32, vp, i64, vp]
        lib.ft_gather_kv_entries.restype = ctypes.c_int
        lib.ft_bump_tails.argtypes = [vp, i32, vp, i64, vp, i32, vp]
        lib.ft_bump_tails.restype = ctypes.c_int
        lib.ft_refresh_tails.argtypes = [vp, i32, vp, i64, vp, i64, vp]
        lib.ft_refresh_tails.restype = ctypes.c_int
        lib.ft_read_device_status.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)]
        lib.ft_read_device_status.restype = ctypes.c_int
        lib.ft_launch_count.restype = ctypes.c_int64
        lib.ft_stage1_path_name.argtypes = [argp]
        lib.ft_stage1_path_name.restype = ctypes.c_char_p
        i32p, i64p = ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int64)
        lib.ft_plan_b200_build.argtypes = [i32p, i32p, ctypes.c_int32, i64p, i32p, i64p, ctypes.c_int32, ctypes.c_int32,
                                           ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(B200ModelStruct),
                                           ctypes.POINTER(ctypes.c_void_p)]
        lib.ft_plan_b200_build.restype = ctypes.c_int
        lib.ft_plan_b200_build_direct.argtypes = [i32p, i32p, ctypes.c_int32, i64p, i32p, i64p, i64p, ctypes.c_int64, i64p,
                                                  i64p, i32p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                                  ctypes.c_int32, ctypes.POINTER(B200ModelStruct),
                                                  ctypes.POINTER(ctypes.c_void_p)]
        lib.ft_plan_b200_build_direct.restype = ctypes.c_int
        lib.ft_plan_get_info.argtypes = [ctypes.c_void_p, ctypes.POINTER(PlanInfo)]
        lib.ft_plan_get_info.restype = ctypes.c_int
        lib.ft_plan_copy_tables.argtypes = [ctypes.c_void_p] + [i32p] * 10
        lib.ft_plan_copy_tables.restype = ctypes.c_int
        lib.ft_plan_copy_row_ranges.argtypes = [ctypes.c_void_p, i32p]
        lib.ft_plan_copy_row_ranges.restype = ctypes.c_int
        lib.ft_plan_copy_aux_segments.argtypes = [ctypes.c_void_p, i32p]
        lib.ft_plan_copy_aux_segments.restype = ctypes.c_int
        lib.ft_plan_free.argtypes = [ctypes.c_void_p]
        lib.ft_plan_free.restype = None
        _lib = lib
    return _lib


def check(rc):
    if rc != 0:
        raise FastTreeError(rc, load().ft_last_error().decode("utf-8", "replace"))


def read_wait_diagnostics():
    out = (ctypes.c_int32 * 8)()
    check(load().ft_read_wait_diagnostics(out))
    return list(out)


def launch_count():
    return int(load().ft_launch_count())


def read_device_status(stream=0):
    flags = ctypes.c_int32(0)
    check(load().ft_read_device_status(ctypes.c_void_p(stream), ctypes.byref(flags)))
    return flags.value
