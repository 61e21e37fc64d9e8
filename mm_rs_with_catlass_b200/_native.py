"""ctypes bindings of ``libcatcoc_b200.so`` (see ``csrc/include/catcoc/capi.h``).

The library is built in-tree by :mod:`._build`. On a machine with a GPU a missing or stale
library is an error (no silent PyTorch fallback); on a CPU-only machine the host-side parts
(scheduler replay, oracle, workspace geometry) still work.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

from . import _build

MAX_WORLD = 8

# enums mirrored from capi.h
IN_F16, IN_BF16, IN_S8, IN_E4M3, IN_E5M2, IN_MXE4M3, IN_MXE5M2 = range(7)
FMT_F16, FMT_BF16, FMT_F32, FMT_S32 = range(4)
MODE_LOCAL, MODE_RS, MODE_AR, MODE_AG = range(4)

E_BAD_ARG, E_ALIGNMENT, E_DRIVER, E_UNSUPPORTED, E_NOMEM, E_IO, E_TOO_LARGE = -1, -2, -3, -4, -5, -6, -7

STATUS_NAMES = {
    0: "ok",
    1: "pipeline wait timed out",
    2: "a peer's partial tile never arrived",
    3: "an owner's reduced tile never arrived",
    4: "a peer's A chunk never arrived",
    5: "barrier / wait_until timed out",
    6: "bad argument",
    7: "an offset left its buffer (bounds-checked build: what = site, expected = limit, seen = offset)",
}
LIM_STAGE, LIM_ARRIVE, LIM_DONE, LIM_AR_OUT, LIM_GATHERED, LIM_GFLAGS, LIM_PART, LIM_OUT = range(8)


class Tiling(C.Structure):
    _fields_ = [("bn", C.c_int), ("swizzle", C.c_int), ("num_ctas", C.c_int), ("seg_dim", C.c_int),
                ("use_multicast", C.c_int), ("rounds", C.c_int), ("cta_pair", C.c_int), ("pull", C.c_int),
                ("comm_warps", C.c_int), ("push_tma", C.c_int)]


class OpArgs(C.Structure):
    _fields_ = [
        ("mode", C.c_int), ("in_fmt", C.c_int),
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
        ("trans_a", C.c_int), ("trans_b", C.c_int),
        ("a", C.c_void_p), ("lda", C.c_int64),
        ("b", C.c_void_p), ("ldb", C.c_int64),
        ("out", C.c_void_p), ("ldc", C.c_int64), ("out_fmt", C.c_int),
        ("tiling", Tiling),
        ("rank", C.c_int), ("W", C.c_int),
        ("partial_fmt", C.c_int),
        ("stage", C.c_void_p * MAX_WORLD),
        ("stage_parity_bytes", C.c_int64),
        ("arrive", C.c_void_p * MAX_WORLD),
        ("ar_out", C.c_void_p * MAX_WORLD),
        ("ar_out_parity_bytes", C.c_int64),
        ("ar_out_mc", C.c_void_p),
        ("done", C.c_void_p * MAX_WORLD),
        ("done_mc", C.c_void_p),
        ("part", C.c_void_p), ("part_mc", C.c_void_p), ("part_parity_bytes", C.c_int64),
        ("gathered_mc", C.c_void_p), ("gflags_mc", C.c_void_p),
        ("gathered", C.c_void_p * MAX_WORLD),
        ("gathered_parity_bytes", C.c_int64),
        ("gflags", C.c_void_p * MAX_WORLD),
        ("ag_m", C.c_int), ("ag_ld", C.c_int), ("ag_raw", C.c_int),
        ("sfa", C.c_void_p), ("sfb", C.c_void_p), ("sf_k_blocks", C.c_int),
        ("scale_m", C.c_void_p), ("scale_n", C.c_void_p), ("bias", C.c_void_p),
        ("affine", C.c_int), ("alpha", C.c_float), ("beta", C.c_float),
        ("c_src", C.c_void_p), ("ldc_src", C.c_int64), ("bias_f", C.c_void_p),
        ("act", C.c_int),
        ("num_groups", C.c_int), ("group_ends", C.c_void_p), ("group_rows", C.c_int),
        ("a_rows_total", C.c_int), ("a_k_total", C.c_int), ("b_n_total", C.c_int), ("b_k_total", C.c_int),
        ("g_a_row_back", C.c_int), ("g_a_k", C.c_int), ("g_b_row", C.c_int), ("g_b_k", C.c_int),
        ("g_nvec", C.c_int),
        ("limit", C.c_int64 * 8),
        ("epoch_ptr", C.c_void_p), ("cta_counter", C.c_void_p), ("status", C.c_void_p),
        ("timeout_ns", C.c_uint64),
        ("withhold_signals", C.c_int),
        ("trace", C.c_void_p),
        ("events", C.c_void_p), ("events_cap", C.c_uint32),
    ]


class Tile(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("seg", "tile_in_seg", "mi", "ni", "m0", "n0", "rows", "cols")]


class ShmemCtx(C.Structure):
    _fields_ = [("rank", C.c_int), ("W", C.c_int), ("base", C.c_void_p * MAX_WORLD), ("mc_base", C.c_void_p),
                ("signal_off", C.c_void_p), ("barrier_off", C.c_int64), ("scratch_off", C.c_int64)]


class NativeError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__("catcoc native error %d: %s" % (code, message))
        self.code = code


_lib = None
_lock = threading.Lock()


def _declare(lib) -> None:
    vp, i32, i64, u32, u64 = C.c_void_p, C.c_int, C.c_int64, C.c_uint32, C.c_uint64
    P = C.POINTER
    sigs = {
        "catcoc_last_error": (C.c_char_p, []),
        "catcoc_version": (i32, []),
        "catcoc_is_checked_build": (i32, []),
        "catcoc_num_sms": (i32, [i32]),
        "catcoc_fused_launch": (i32, [P(OpArgs), vp]),
        "catcoc_stage_bytes": (i64, [i32, i32, i32, i32, i32, i32, i32]),
        "catcoc_arrive_words": (i64, [i32, i32, i32, i32, i32, i32]),
        "catcoc_done_words": (i64, [i32, i32, i32, i32, i32, i32]),
        "catcoc_gather_flag_words": (i64, [i32, i32, i32, i32]),
        "catcoc_sched_total_tiles": (i32, [i32] * 6),
        "catcoc_sched_get_tile": (i32, [i32] * 9 + [P(Tile)]),
        "catcoc_sched_get_tile_rounds": (i32, [i32] * 10 + [P(Tile)]),
        "catcoc_sched_get_tile_order": (i32, [i32] * 10 + [P(Tile)]),
        "catcoc_group_walk_replay": (i32, [i32, i32, i32, i32, i32, vp, i32, i32, P(Tile)]),
        "catcoc_oracle_matmul_f32": (i32, [vp, vp, vp, i32, i32, i32, i32, i32]),
        "catcoc_oracle_quant_matmul": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32]),
        "catcoc_oracle_dequant": (i32, [vp, vp, vp, vp, i32, i32]),
        "catcoc_oracle_compare": (i64, [vp, vp, i64, C.c_float, P(C.c_double)]),
        "catcoc_oracle_gemm": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, C.c_float, C.c_float]),
        "catcoc_oracle_gemv": (i32, [vp, vp, vp, vp, i32, i32, i32, C.c_float, C.c_float]),
        "catcoc_oracle_batched_matmul": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, i32]),
        "catcoc_oracle_grouped_matmul": (i32, [vp, vp, vp, i32, vp, i32, i32, i32, i32]),
        "catcoc_oracle_grouped_matmul_slice_k": (i32, [vp, vp, vp, i32, vp, i32, i32, i32]),
        "catcoc_oracle_grouped_quant_matmul": (i32, [vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32]),
        "catcoc_oracle_grouped_quant_matmul_slice_k": (i32, [vp, vp, vp, i32, vp, vp, vp, i32, i32, i32]),
        "catcoc_oracle_group_gemm": (i32, [i32, vp, vp, vp, vp, vp, vp, vp]),
        "catcoc_heap_create": (i32, [i32, i32, i32, i64, P(vp)]),
        "catcoc_heap_bytes": (i64, [vp]),
        "catcoc_heap_export_fd": (i32, [vp]),
        "catcoc_heap_import_peer": (i32, [vp, i32, i32]),
        "catcoc_heap_base": (vp, [vp, i32]),
        "catcoc_heap_multicast_supported": (i32, [i32]),
        "catcoc_heap_mc_create": (i32, [vp]),
        "catcoc_heap_mc_join": (i32, [vp, i32]),
        "catcoc_heap_mc_bind": (i32, [vp]),
        "catcoc_heap_mc_base": (vp, [vp]),
        "catcoc_heap_destroy": (i32, [vp]),
        "catcoc_fd_send": (i32, [C.c_char_p, i32, i32, i32]),
        "catcoc_fd_recv_open": (i32, [C.c_char_p]),
        "catcoc_fd_recv": (i32, [i32, i32, P(i32)]),
        "catcoc_fd_close": (i32, [i32]),
        "catcoc_shmem_barrier_all": (i32, [P(ShmemCtx), u32, u64, vp, vp]),
        "catcoc_shmem_put": (i32, [P(ShmemCtx), i32, i64, vp, i64, i64, u32, vp]),
        "catcoc_shmem_get": (i32, [P(ShmemCtx), i32, vp, i64, i64, vp]),
        "catcoc_shmem_wait_until": (i32, [P(ShmemCtx), i64, u32, u64, vp, vp]),
        "catcoc_shmem_mc_broadcast": (i32, [P(ShmemCtx), i64, vp, i64, vp]),
        "catcoc_shmem_mc_reduce_bf16": (i32, [P(ShmemCtx), vp, i64, i64, vp]),
        "catcoc_shmem_put_blocks": (i32, []),
        "catcoc_pad2d": (i32, [vp, i64, vp, i64, i64, i64, vp]),
        "catcoc_splitk_reduce": (i32, [vp, i32, i64, i32, i32, vp, i64, i32, C.c_float, C.c_float, vp, i64, vp, vp]),
        "catcoc_splitk_allreduce_flag_words": (i64, [i32, i32, i32]),
        "catcoc_splitk_allreduce": (i32, [P(ShmemCtx), vp, i32, i64, i32, i32, i32, i32, vp, i64, i32, i64, i64, i32, vp, vp, vp, u64, vp]),
        "catcoc_small_allgather_flag_words": (i64, [i32, i64, i32]),
        "catcoc_small_allgather": (i32, [P(ShmemCtx), vp, i64, i32, i64, i64, i64, i64, i32, vp, vp, vp, u64, vp]),
        "catcoc_gemv_workspace_floats": (i64, [i32, i32, i32]),
        "catcoc_gemv": (i32, [vp, i64, i32, i32, i32, i32, vp, vp, vp, C.c_float, C.c_float, vp, vp]),
        "catcoc_flash_attention": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, C.c_float, vp, u64, vp]),
        "catcoc_mla_workspace_bytes": (i64, [i32, i32, i32, i32]),
        "catcoc_mla_decode": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, C.c_float, i32, vp, u64, vp]),
        "catcoc_matmul_noalloc": (i32, [vp, i64, vp, i64, vp, i64, i32, i32, i32, i32, i32, i32, i32, vp]),
        "catcoc_matmul_noalloc_status": (i32, [P(u32)]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


def lib():
    """Returns the loaded library, building it first if the sources changed."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                # CATCOC_CHECKED=1 loads the build whose kernels bounds-check every workspace offset
                checked = os.environ.get("CATCOC_CHECKED", "0") == "1"
                target = _build.lib_path(checked)
                if os.environ.get("CATCOC_NO_BUILD") and target.exists():
                    path = target
                else:
                    path = _build.build(checked=checked)
                loaded = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
                _declare(loaded)
                _lib = loaded
    return _lib


def last_error() -> str:
    return (lib().catcoc_last_error() or b"").decode(errors="replace")


def check(code: int) -> int:
    """Raises :class:`NativeError` for a negative return code; passes other values through."""
    if code < 0:
        raise NativeError(code, last_error())
    return code
