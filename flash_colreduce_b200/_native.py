"""ctypes binding of the C ABI declared in ``include/flash_colreduce_b200.h``.

The shared library is the only implementation: if it has not been built
(``python flash_colreduce_b200/build.py``) importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

from .build import LIB_PATH  # path only; nothing is compiled at import time

FCR_OK = 0
FCR_ERR_BAD_ARG = 1
FCR_ERR_UNSUPPORTED = 2
FCR_ERR_WORKSPACE = 3
FCR_ERR_DEVICE_TIMEOUT = 4
FCR_ERR_CUDA = 5
FCR_ERR_NCCL = 6
FCR_NCCL_ID_BYTES = 128

FCR_F16, FCR_BF16, FCR_F32 = 0, 1, 2
FCR_SUM, FCR_MEAN, FCR_MAX = 0, 1, 2
REDUCTION_CODES = {"sum": FCR_SUM, "mean": FCR_MEAN, "max": FCR_MAX}

EXPORTS = (
    "fcr_version",
    "fcr_last_error",
    "fcr_plan_problem",
    "fcr_plan_item",
    "fcr_workspace_bytes",
    "fcr_colreduce",
    "fcr_colreduce_static",
    "fcr_finalize",
    "fcr_topk",
    "fcr_select_above",
    "fcr_read_device_status",
    "fcr_trace_enable",
    "fcr_trace_count",
    "fcr_trace_read",
    "fcr_read_device_status_static",
    "fcr_poll_device_status",
    "fcr_launch_count",
    "fcr_self_test_hooks",
    "fcr_plan_shards",
    "fcr_comm_unique_id",
    "fcr_comm_init",
    "fcr_comm_destroy",
    "fcr_sharded_workspace_bytes",
    "fcr_colreduce_sharded",
)


class Problem(C.Structure):
    """Mirror of ``fcr_problem``."""

    _fields_ = [
        ("B", C.c_int32), ("H", C.c_int32), ("M", C.c_int32), ("N", C.c_int32), ("D", C.c_int32),
        ("q_strides", C.c_int64 * 4),
        ("k_strides", C.c_int64 * 4),
        ("in_dtype", C.c_int32),
        ("reduction", C.c_int32),
        ("is_causal", C.c_int32),
        ("scale", C.c_float),
        ("causal_offset", C.c_int64),
        ("mean_M", C.c_int32), ("mean_N", C.c_int32),
    ]


class Plan(C.Structure):
    """Mirror of ``fcr_plan``."""

    _fields_ = [
        ("d_pad", C.c_int32), ("rows_per_block", C.c_int32),
        ("m_pad", C.c_int32), ("n_pad", C.c_int32),
        ("row_blocks", C.c_int32), ("col_blocks", C.c_int32),
        ("row_splits", C.c_int32), ("col_splits", C.c_int32),
        ("row_items", C.c_int32), ("col_items", C.c_int32),
        ("row_ctas", C.c_int32), ("col_ctas", C.c_int32),
        ("head_group", C.c_int32), ("short_items", C.c_int32),
        ("causal_offset", C.c_int64),
        ("valid_scores", C.c_int64),
        ("off_status", C.c_int64), ("off_neg_lse", C.c_int64),
        ("off_part_m", C.c_int64), ("off_part_l", C.c_int64), ("off_part_out", C.c_int64),
        ("workspace_bytes", C.c_int64),
        ("key_stream", C.c_int32), ("key_chunks", C.c_int32),
        ("off_scores", C.c_int64), ("score_cache", C.c_int32), ("static_schedule", C.c_int32),
    ]


class Shard(C.Structure):
    """Mirror of ``fcr_shard``."""

    _fields_ = [
        ("rank", C.c_int32), ("world", C.c_int32),
        ("head_lo", C.c_int32), ("head_hi", C.c_int32),
        ("n_ranges", C.c_int32),
        ("row_lo", C.c_int32 * 2), ("row_hi", C.c_int32 * 2),
        ("needs_reduce", C.c_int32),
    ]


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python flash_colreduce_b200/build.py` "
            "(there is no fallback implementation)"
        )
    lib = C.CDLL(LIB_PATH)
    lib.fcr_version.restype = C.c_char_p
    lib.fcr_last_error.restype = C.c_char_p
    lib.fcr_plan_problem.argtypes = [C.POINTER(Problem), C.c_int32, C.POINTER(Plan)]
    lib.fcr_plan_problem.restype = C.c_int
    lib.fcr_plan_item.argtypes = [C.POINTER(Problem), C.POINTER(Plan), C.c_int32, C.c_int32,
                                  C.POINTER(C.c_int32)]
    lib.fcr_plan_item.restype = C.c_int
    lib.fcr_workspace_bytes.argtypes = [C.POINTER(Problem), C.c_int32]
    lib.fcr_workspace_bytes.restype = C.c_size_t
    lib.fcr_colreduce.argtypes = [C.POINTER(Problem), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                  C.c_void_p, C.c_size_t, C.c_void_p]
    lib.fcr_colreduce.restype = C.c_int
    lib.fcr_colreduce_static.argtypes = [C.POINTER(Problem), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                         C.c_void_p]
    lib.fcr_colreduce_static.restype = C.c_int
    lib.fcr_finalize.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                 C.c_int32, C.c_int32, C.c_int32, C.c_void_p]
    lib.fcr_finalize.restype = C.c_int
    lib.fcr_topk.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_int32,
                             C.c_void_p, C.c_void_p]
    lib.fcr_topk.restype = C.c_int
    lib.fcr_select_above.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_float, C.c_void_p, C.c_int32,
                                     C.c_void_p, C.c_void_p]
    lib.fcr_select_above.restype = C.c_int
    lib.fcr_read_device_status.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]
    lib.fcr_read_device_status.restype = C.c_int
    lib.fcr_trace_enable.argtypes = [C.c_int32]
    lib.fcr_trace_enable.restype = C.c_int
    lib.fcr_trace_count.argtypes = []
    lib.fcr_trace_count.restype = C.c_int32
    lib.fcr_trace_read.argtypes = [C.c_int32, C.POINTER(C.c_float), C.POINTER(C.c_float)]
    lib.fcr_trace_read.restype = C.c_int
    lib.fcr_read_device_status_static.argtypes = [C.c_void_p, C.POINTER(C.c_int32)]
    lib.fcr_read_device_status_static.restype = C.c_int
    lib.fcr_poll_device_status.argtypes = [C.POINTER(C.c_int32)]
    lib.fcr_poll_device_status.restype = C.c_int
    lib.fcr_launch_count.argtypes = []
    lib.fcr_launch_count.restype = C.c_int64
    lib.fcr_self_test_hooks.argtypes = [C.c_int64, C.c_int32]
    lib.fcr_self_test_hooks.restype = C.c_int
    lib.fcr_plan_shards.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(Shard)]
    lib.fcr_plan_shards.restype = C.c_int
    lib.fcr_comm_unique_id.argtypes = [C.c_void_p]
    lib.fcr_comm_unique_id.restype = C.c_int
    lib.fcr_comm_init.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]
    lib.fcr_comm_init.restype = C.c_int
    lib.fcr_comm_destroy.argtypes = [C.c_void_p]
    lib.fcr_comm_destroy.restype = C.c_int
    lib.fcr_sharded_workspace_bytes.argtypes = [C.POINTER(Problem), C.POINTER(Shard)]
    lib.fcr_sharded_workspace_bytes.restype = C.c_size_t
    lib.fcr_colreduce_sharded.argtypes = [C.POINTER(Problem), C.POINTER(Shard), C.c_int32, C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_size_t, C.c_void_p,
                                          C.c_void_p]
    lib.fcr_colreduce_sharded.restype = C.c_int
    return lib


lib = _load()


def last_error() -> str:
    return lib.fcr_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    """Raises RuntimeError for a non-zero status from the library."""
    if rc != FCR_OK:
        raise RuntimeError(f"{what} failed with status {rc}: {last_error()}")


def make_problem(B, H, M, N, D, q_strides, k_strides, in_dtype, reduction, is_causal, scale,
                 causal_offset=-1, mean_M=0, mean_N=0) -> Problem:
    p = Problem()
    p.B, p.H, p.M, p.N, p.D = int(B), int(H), int(M), int(N), int(D)
    p.q_strides = (C.c_int64 * 4)(*[int(s) for s in q_strides])
    p.k_strides = (C.c_int64 * 4)(*[int(s) for s in k_strides])
    p.in_dtype = int(in_dtype)
    p.reduction = int(reduction)
    p.is_causal = 1 if is_causal else 0
    p.scale = float(scale)
    p.causal_offset = int(causal_offset)
    p.mean_M, p.mean_N = int(mean_M), int(mean_N)
    return p


def plan(problem: Problem, num_sms: int = 0) -> Plan:
    pl = Plan()
    check(lib.fcr_plan_problem(C.byref(problem), int(num_sms), C.byref(pl)), "fcr_plan_problem")
    return pl


def plan_item(problem: Problem, pl: Plan, which_pass: int, item: int) -> dict:
    """Decoded work item: head, split, streamed chunk and per-sub-tile tile ranges."""
    buf = (C.c_int32 * 10)()
    check(lib.fcr_plan_item(C.byref(problem), C.byref(pl), which_pass, item, buf), "fcr_plan_item")
    v = list(buf)
    return {"head": v[0], "split": v[1], "chunk": (v[2], v[3]),
            "sub": [(v[4], v[5], v[6]), (v[7], v[8], v[9])]}


def trace_times() -> list:
    """(rows_ms, cols_ms) of every call traced since ``fcr_trace_enable(1)``; synchronises."""
    out = []
    for i in range(lib.fcr_trace_count()):
        a, b = C.c_float(0), C.c_float(0)
        check(lib.fcr_trace_read(i, C.byref(a), C.byref(b)), "fcr_trace_read")
        out.append((a.value, b.value))
    return out
