"""ctypes bindings of libnano_nccl.so (C ABI v2 plus extensions).

The library is built in-tree by :mod:`nano_nccl_b200._build`; importing this module never falls
back to a Python implementation: a missing library raises.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

LIB_DIR = Path(__file__).resolve().parent / "lib"
LIB_PATH = LIB_DIR / "libnano_nccl.so"

STATUS_SUCCESS, STATUS_INVALID_ARGUMENT, STATUS_UNSUPPORTED, STATUS_ERROR = 0, 1, 2, 3
DTYPES = {"float": 0, "fp16": 1, "bf16": 2}
REDOPS = {"sum": 0, "avg": 1, "max": 2, "min": 3}
TRANSPORTS = {"auto": 0, "shm": 1, "p2p": 2, "socket": 3, "rdma": 4, "mixed": 5}
ALGOS = {"auto": 0, "oneshot": 1, "twoshot": 2, "nvls": 3, "ring": 4}
TRANSPORT_NAMES = {v: k for k, v in TRANSPORTS.items()}
ALGO_NAMES = {v: k for k, v in ALGOS.items()}


class AllReduceArgs(C.Structure):
    _fields_ = [("send_buffer", C.c_void_p), ("recv_buffer", C.c_void_p), ("stream", C.c_void_p),
                ("count", C.c_size_t), ("dtype", C.c_int32), ("redop", C.c_int32)]


class ReduceScatterArgs(C.Structure):
    _fields_ = [("send_buffer", C.c_void_p), ("recv_buffer", C.c_void_p), ("stream", C.c_void_p),
                ("recv_count", C.c_size_t), ("dtype", C.c_int32), ("redop", C.c_int32)]


class AllGatherArgs(C.Structure):
    _fields_ = [("send_buffer", C.c_void_p), ("recv_buffer", C.c_void_p), ("stream", C.c_void_p),
                ("send_count", C.c_size_t), ("dtype", C.c_int32)]


class ExtConfig(C.Structure):
    _fields_ = [("device", C.c_int), ("transport", C.c_int32), ("algo", C.c_int32),
                ("enable_multicast", C.c_int), ("wait_timeout_us", C.c_int64),
                ("relaxed_validation", C.c_int)]


class Stats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in
                ("launches", "oneshot", "twoshot", "nvls", "ring", "zero_copy", "local_only", "pipelined")]


class MpiSubgroupConfig(C.Structure):
    _fields_ = [("color", C.c_int), ("key", C.c_int), ("device", C.c_int), ("transport", C.c_int32)]


ALLGATHER_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t)

_lib = None


def load_library() -> C.CDLL:
    """Loads (once) and returns the native library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(f"{LIB_PATH} is missing: run `python -m nano_nccl_b200._build`")
    lib = C.CDLL(str(LIB_PATH), mode=C.RTLD_GLOBAL)
    P, I, S = C.c_void_p, C.c_int, C.c_int32
    sig = {
        "nano_nccl_abi_version": (C.c_uint32, []),
        "nano_nccl_status_string": (C.c_char_p, [S]),
        "nano_nccl_get_last_error": (C.c_char_p, []),
        "nano_nccl_destroy_communicator": (S, [P]),
        "nano_nccl_all_reduce": (S, [P, C.POINTER(AllReduceArgs)]),
        "nano_nccl_reduce_scatter": (S, [P, C.POINTER(ReduceScatterArgs)]),
        "nano_nccl_all_gather": (S, [P, C.POINTER(AllGatherArgs)]),
        "nano_nccl_check_async_error": (S, [P]),
        "nano_nccl_local_rank_count": (S, [P, C.POINTER(I)]),
        "nano_nccl_global_rank_count": (S, [P, C.POINTER(I)]),
        "nano_nccl_transport": (S, [P, C.POINTER(S)]),
        "nano_nccl_edge_transport": (S, [P, I, C.POINTER(S)]),
        "nano_nccl_edge_uses_gdr": (S, [P, I, C.POINTER(I)]),
        "nano_nccl_create_tcp_communicator": (S, [C.c_char_p, I, I, I, C.POINTER(ExtConfig), C.POINTER(P)]),
        "nano_nccl_create_callback_communicator": (S, [ALLGATHER_FN, P, I, I, C.POINTER(ExtConfig), C.POINTER(P)]),
        "nano_nccl_bootstrap_selftest": (I, [ALLGATHER_FN, P, I, I]),
        "nano_nccl_rank": (S, [P, C.POINTER(I)]),
        "nano_nccl_multicast_available": (S, [P, C.POINTER(I)]),
        "nano_nccl_set_algo": (S, [P, S]),
        "nano_nccl_set_grid_override": (S, [P, I]),
        "nano_nccl_last_algo": (S, [P, C.POINTER(S)]),
        "nano_nccl_symmetric_alloc": (S, [P, C.c_size_t, C.POINTER(P)]),
        "nano_nccl_symmetric_free": (S, [P, P]),
        "nano_nccl_register_buffer": (S, [P, P, C.c_size_t]),
        "nano_nccl_deregister_buffer": (S, [P, P]),
        "nano_nccl_peer_pointer": (S, [P, P, I, C.POINTER(P)]),
        "nano_nccl_multicast_pointer": (S, [P, P, C.POINTER(P)]),
        "nano_nccl_barrier": (S, [P, P]),
        "nano_nccl_get_stats": (S, [P, C.POINTER(Stats)]),
        "nano_nccl_emu_create": (S, [I, I, C.c_int64, C.POINTER(P)]),
        "nano_nccl_emu_destroy": (S, [P]),
        "nano_nccl_emu_all_reduce": (S, [P, C.POINTER(P), C.POINTER(P), C.c_size_t, S, S, S, I, P]),
        "nano_nccl_emu_reduce_scatter": (S, [P, C.POINTER(P), C.POINTER(P), C.c_size_t, S, S, I, P]),
        "nano_nccl_emu_all_gather": (S, [P, C.POINTER(P), C.POINTER(P), C.c_size_t, S, I, P]),
        "nano_nccl_emu_lonely_barrier": (S, [P, I, P]),
        "nano_nccl_emu_status": (S, [P, I, C.POINTER(C.c_uint32)]),
        "nano_nccl_emu_clear_status": (S, [P]),
        "nano_nccl_emu_set_abort": (S, [P, I]),
        "nano_nccl_gemm_bf16": (S, [P, P, P, P, I, I, I, P, I]),
        "nano_nccl_gemm_last_error": (I, [I]),
        "nano_nccl_gemm_clear_error": (None, [I]),
        "nano_nccl_fused_gemm_create": (S, [P, C.c_size_t, C.c_size_t, C.POINTER(P)]),
        "nano_nccl_fused_gemm_destroy": (S, [P]),
        "nano_nccl_gemm_rs": (S, [P, P, P, P, I, I, I, P]),
        "nano_nccl_ag_gemm": (S, [P, P, P, P, I, I, I, P, I]),
        "nano_nccl_fused_gemm_read_trace": (S, [P, C.POINTER(C.c_ulonglong), C.c_size_t, C.POINTER(C.c_size_t)]),
        "nano_nccl_push_copy": (S, [I, P, C.POINTER(P), I, C.c_size_t, I, I, I, P, P]),
        "nano_nccl_allocator_bind": (S, [P]),
        "nano_nccl_torch_alloc": (P, [C.c_size_t, I, P]),
        "nano_nccl_torch_free": (None, [P, C.c_size_t, I, P]),
        "nano_nccl_allocator_stats": (S, [C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class NanoNcclError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"nano_nccl status {status}: {message}")
        self.status = status
        self.message = message


def check(status: int) -> None:
    if status != STATUS_SUCCESS:
        msg = load_library().nano_nccl_get_last_error()
        err = NanoNcclError(status, msg.decode(errors="replace") if msg else "")
        if status == STATUS_INVALID_ARGUMENT:
            raise ValueError(str(err)) from err
        raise err


def library_loaded_path() -> str | None:
    """Path of the native library as the dynamic loader sees it (evidence that it is in use)."""
    try:
        with open("/proc/self/maps") as f:
            for line in f:
                if "libnano_nccl.so" in line:
                    return line.split()[-1]
    except OSError:
        pass
    return None
