"""ctypes binding of the C-ABI library (include/ssd_b200.h).

There is no CPU fallback: if the library is missing, loading raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

ABI_VERSION = 3
F32, BF16 = 0, 1
PASS_FWD, PASS_BWD = 0, 1
PATH_AUTO, PATH_SIMT, PATH_TC = 0, 1, 2
OK, EINVAL, EUNSUPPORTED, EWORKSPACE, ECUDA, EDEVICE = 0, -1, -2, -3, -4, -5
FWD_STATES_ONLY = 1
FWD_AUX_VALID = 2
BWD_DINIT_ONLY = 1

EXPORTS = (
    "ssd_b200_abi_version", "ssd_b200_last_error", "ssd_b200_workspace_bytes", "ssd_b200_states_bytes",
    "ssd_b200_resolve_path",
    "ssd_b200_fwd", "ssd_b200_bwd", "ssd_b200_materialize_cache", "ssd_b200_state_prefix_all", "ssd_b200_ipc_export", "ssd_b200_ipc_import", "ssd_b200_ipc_close", "ssd_b200_enable_peer_access", "ssd_b200_exchange_push", "ssd_b200_exchange_arrive",
    "ssd_b200_m3_prologue_fwd", "ssd_b200_m3_skip_fwd", "ssd_b200_m3_prologue_bwd", "ssd_b200_m3_chain_ws_floats", "ssd_b200_m3_chain_bwd", "ssd_b200_rope_fwd", "ssd_b200_rope_bwd",
    "ssd_b200_trapezoid_ws_floats", "ssd_b200_trapezoid_fwd", "ssd_b200_trapezoid_bwd",
    "ssd_b200_rmsnorm_ws_floats", "ssd_b200_rmsnorm_fwd", "ssd_b200_rmsnorm_fwd_presummed", "ssd_b200_rmsnorm_bwd", "ssd_b200_fwd_static_scratch", "ssd_b200_static_scratch_bytes", "ssd_b200_device_status", "ssd_b200_selftest_bounded_wait",
    "ssd_b200_launch_count", "ssd_b200_profile_enable", "ssd_b200_profile_kernels", "ssd_b200_profile_kernel_name",
    "ssd_b200_profile_read",
)


class Shape(C.Structure):
    _fields_ = [("abi_version", C.c_int32), ("dtype", C.c_int32), ("a_dtype", C.c_int32), ("path", C.c_int32),
                ("batch", C.c_int64), ("seqlen", C.c_int64), ("nheads", C.c_int64), ("headdim", C.c_int64),
                ("dstate", C.c_int64), ("ngroups", C.c_int64), ("chunk", C.c_int64)]


class FwdArgs(C.Structure):
    _fields_ = [("shape", Shape), ("x", C.c_void_p), ("a", C.c_void_p), ("dt", C.c_void_p), ("A_head", C.c_void_p),
                ("D", C.c_void_p), ("B", C.c_void_p), ("C", C.c_void_p), ("init", C.c_void_p), ("y", C.c_void_p),
                ("final_state", C.c_void_p), ("a_cumsum", C.c_void_p), ("cumsum_is_input", C.c_int32),
                ("flags", C.c_int32), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
                ("states", C.c_void_p), ("logdecay_total", C.c_void_p), ("ysq", C.c_void_p), ("skip", C.c_void_p)]


class BwdArgs(C.Structure):
    _fields_ = [("shape", Shape), ("x", C.c_void_p), ("a", C.c_void_p), ("dt", C.c_void_p), ("A_head", C.c_void_p),
                ("D", C.c_void_p), ("B", C.c_void_p), ("C", C.c_void_p), ("init", C.c_void_p),
                ("a_cumsum", C.c_void_p), ("dy", C.c_void_p), ("dfinal", C.c_void_p), ("dx", C.c_void_p),
                ("dB", C.c_void_p), ("dC", C.c_void_p), ("da", C.c_void_p), ("ddt", C.c_void_p),
                ("dA_head", C.c_void_p), ("dD", C.c_void_p), ("dinit", C.c_void_p),
                ("cumsum_is_input", C.c_int32), ("flags", C.c_int32), ("workspace", C.c_void_p),
                ("workspace_bytes", C.c_size_t), ("states", C.c_void_p), ("skip", C.c_void_p), ("dskip", C.c_void_p)]


_lib = None


def library_path() -> Path:
    return Path(__file__).resolve().parent / "csrc" / "libssd_b200.so"


def load() -> C.CDLL:
    """Load libssd_b200.so (once).  Raises ImportError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        raise ImportError(f"{path} is missing: build it first (python {path.parent.parent / 'build.py'}); "
                          "there is no fallback implementation")
    lib = C.CDLL(str(path))
    lib.ssd_b200_abi_version.restype = C.c_int
    lib.ssd_b200_last_error.restype = C.c_char_p
    lib.ssd_b200_workspace_bytes.restype = C.c_size_t
    lib.ssd_b200_workspace_bytes.argtypes = [C.POINTER(Shape), C.c_int]
    lib.ssd_b200_states_bytes.restype = C.c_size_t
    lib.ssd_b200_states_bytes.argtypes = [C.POINTER(Shape)]
    lib.ssd_b200_resolve_path.restype = C.c_int
    lib.ssd_b200_resolve_path.argtypes = [C.POINTER(Shape)]
    lib.ssd_b200_fwd.restype = C.c_int
    lib.ssd_b200_fwd.argtypes = [C.POINTER(FwdArgs), C.c_void_p]
    lib.ssd_b200_bwd.restype = C.c_int
    lib.ssd_b200_bwd.argtypes = [C.POINTER(BwdArgs), C.c_void_p]
    lib.ssd_b200_materialize_cache.restype = C.c_int
    lib.ssd_b200_materialize_cache.argtypes = [C.POINTER(Shape), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                               C.c_void_p]
    lib.ssd_b200_state_prefix_all.restype = C.c_int
    lib.ssd_b200_state_prefix_all.argtypes = ([C.c_void_p] * 6 + [C.c_int64] * 8 + [C.c_int32] + [C.c_void_p] * 2 + [C.c_int64] * 4
                                              + [C.c_void_p])
    lib.ssd_b200_ipc_export.restype = C.c_int
    lib.ssd_b200_ipc_export.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)]
    lib.ssd_b200_ipc_import.restype = C.c_int
    lib.ssd_b200_ipc_import.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    lib.ssd_b200_ipc_close.restype = C.c_int
    lib.ssd_b200_ipc_close.argtypes = [C.c_void_p]
    lib.ssd_b200_enable_peer_access.restype = C.c_int
    lib.ssd_b200_enable_peer_access.argtypes = [C.c_int32]
    lib.ssd_b200_exchange_push.restype = C.c_int
    lib.ssd_b200_exchange_push.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
    lib.ssd_b200_exchange_arrive.restype = C.c_int
    lib.ssd_b200_exchange_arrive.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p]
    lib.ssd_b200_m3_prologue_fwd.restype = C.c_int
    lib.ssd_b200_m3_prologue_fwd.argtypes = [C.POINTER(Shape)] + [C.c_void_p] * 7 + [C.c_int32] + [C.c_void_p] * 11
    lib.ssd_b200_rope_fwd.restype = C.c_int
    lib.ssd_b200_rope_fwd.argtypes = [C.c_int32] + [C.c_int64] * 4 + [C.c_int32] + [C.c_void_p] * 4
    lib.ssd_b200_rope_bwd.restype = C.c_int
    lib.ssd_b200_rope_bwd.argtypes = [C.c_int32] + [C.c_int64] * 4 + [C.c_int32] + [C.c_void_p] * 6
    lib.ssd_b200_trapezoid_ws_floats.restype = C.c_size_t
    lib.ssd_b200_trapezoid_ws_floats.argtypes = [C.c_int64, C.c_int64]
    lib.ssd_b200_trapezoid_fwd.restype = C.c_int
    lib.ssd_b200_trapezoid_fwd.argtypes = [C.c_int32, C.c_int64, C.c_int64] + [C.c_void_p] * 9
    lib.ssd_b200_trapezoid_bwd.restype = C.c_int
    lib.ssd_b200_trapezoid_bwd.argtypes = [C.c_int32, C.c_int64, C.c_int64] + [C.c_void_p] * 14
    lib.ssd_b200_rmsnorm_ws_floats.restype = C.c_size_t
    lib.ssd_b200_rmsnorm_ws_floats.argtypes = [C.c_int64, C.c_int64]
    lib.ssd_b200_rmsnorm_fwd.restype = C.c_int
    lib.ssd_b200_rmsnorm_fwd.argtypes = [C.c_int32, C.c_int64, C.c_int64, C.c_float] + [C.c_void_p] * 6
    lib.ssd_b200_rmsnorm_fwd_presummed.restype = C.c_int
    lib.ssd_b200_rmsnorm_fwd_presummed.argtypes = [C.c_int32, C.c_int64, C.c_int64, C.c_float] + [C.c_void_p] * 4 + [C.c_int64] + [C.c_void_p] * 3
    lib.ssd_b200_rmsnorm_bwd.restype = C.c_int
    lib.ssd_b200_rmsnorm_bwd.argtypes = [C.c_int32, C.c_int64, C.c_int64] + [C.c_void_p] * 10
    lib.ssd_b200_m3_skip_fwd.restype = C.c_int
    lib.ssd_b200_m3_skip_fwd.argtypes = [C.POINTER(Shape)] + [C.c_void_p] * 8
    lib.ssd_b200_m3_prologue_bwd.restype = C.c_int
    lib.ssd_b200_m3_prologue_bwd.argtypes = [C.POINTER(Shape)] + [C.c_void_p] * 18 + [C.c_int32] + [C.c_void_p] * 3
    lib.ssd_b200_m3_chain_ws_floats.restype = C.c_size_t
    lib.ssd_b200_m3_chain_ws_floats.argtypes = [C.POINTER(Shape)]
    lib.ssd_b200_m3_chain_bwd.restype = C.c_int
    lib.ssd_b200_m3_chain_bwd.argtypes = [C.POINTER(Shape)] + [C.c_void_p] * 13
    lib.ssd_b200_fwd_static_scratch.restype = C.c_int
    lib.ssd_b200_fwd_static_scratch.argtypes = [C.POINTER(FwdArgs), C.c_void_p]
    lib.ssd_b200_static_scratch_bytes.restype = C.c_size_t
    lib.ssd_b200_device_status.restype = C.c_int
    lib.ssd_b200_device_status.argtypes = [C.POINTER(Shape), C.c_void_p, C.c_void_p]
    lib.ssd_b200_selftest_bounded_wait.restype = C.c_int
    lib.ssd_b200_selftest_bounded_wait.argtypes = [C.c_void_p, C.c_int32, C.c_void_p]
    lib.ssd_b200_launch_count.restype = C.c_longlong
    lib.ssd_b200_profile_enable.argtypes = [C.c_int]
    lib.ssd_b200_profile_kernel_name.restype = C.c_char_p
    lib.ssd_b200_profile_kernel_name.argtypes = [C.c_int]
    lib.ssd_b200_profile_read.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_longlong), C.c_int]
    if lib.ssd_b200_abi_version() != ABI_VERSION:
        raise ImportError(f"{path}: ABI version {lib.ssd_b200_abi_version()} != {ABI_VERSION}; rebuild")
    _lib = lib
    return lib


def last_error() -> str:
    return load().ssd_b200_last_error().decode()


def check(rc: int) -> None:
    """Turn a negative return code into the exception type the reference operator raises."""
    if rc >= 0:
        return
    msg = last_error()
    if rc == EINVAL and "not divisible by chunk_size" in msg:
        raise AssertionError(msg)            # reference: src/kernels/ssd_scan.py:348-350
    if rc == EINVAL:
        raise ValueError(msg)
    if rc == EUNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(f"ssd_b200 error {rc}: {msg}")


def launch_count() -> int:
    return int(load().ssd_b200_launch_count())


def profile_enable(on: bool) -> None:
    load().ssd_b200_profile_enable(1 if on else 0)


def profile_read() -> dict[str, tuple[float, int]]:
    """Per-kernel (total ms, launches) since the last read; waits for the recorded events."""
    lib = load()
    n = lib.ssd_b200_profile_kernels()
    ms = (C.c_float * n)()
    cnt = (C.c_longlong * n)()
    check(lib.ssd_b200_profile_read(ms, cnt, n))
    return {lib.ssd_b200_profile_kernel_name(i).decode(): (float(ms[i]), int(cnt[i])) for i in range(n) if cnt[i]}
