"""ctypes binding of ``libfqla_sm100.so`` (declared in ``include/fqla.h``).

There is no fallback: if the library has not been built the first kernel call raises.
"""

from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libfqla_sm100.so")

P, I, LL, F = C.c_void_p, C.c_int, C.c_longlong, C.c_float

# name -> argument types, in the order of include/fqla.h
SIGNATURES = {
    "fqla_chunk_local_cumsum": [P, P, I, I, I, P, I, I, P, LL, I, P],
    "fqla_kkt_solve": [P, P, I, P, P, P, I, I, I, I, I, P, I, P, LL, P],
    "fqla_fwd_seq": [P] * 6 + [I] + [P] * 11 + [I] * 6 + [F, P, P, I, I, I, P],
    "fqla_bwd_dh": [P, P, P, P, P, I, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, P, P, I, I, I,
                    P],
    "fqla_bwd_main": [P] * 7 + [I] + [P] * 9 + [I, I, I, I, I, F, P, P, P, I, LL, I, P],
    "fqla_group_reduce": [P, P, LL, I, I, I, P],
    "fqla_warmup_scan": [P, I, I, P, I, I, F, I, P, P, P, P],
    "fqla_merge_states": [P, P, P, P, P, P, P, I, I, I, I, LL, P],
    "fqla_l2norm_fwd": [P, P, P, LL, I, I, F, P],
    "fqla_l2norm_bwd": [P, P, P, P, LL, I, I, I, P],
    "fqla_segment_scan": [P, I, I, P, I, P, I, F, I, P, P, P, P, P, P],
    "fqla_device_status": [P, I],
    "fqla_selftest_wait_timeout": [I, P],
    "fqla_fwd_noalloc": [P, P, P, P, P, I, P, P, P, I, I, I, I, I, F, P, P, P, I, I, LL, P],
}

_lib = None


class FqlaError(RuntimeError):
    pass


def load():
    """Load the shared library once and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FqlaError(
            f"{LIB_PATH} is missing: build the CUDA kernels first "
            "(python -m flashqla_b200.build). There is no CPU or PyTorch fallback."
        )
    lib = C.CDLL(LIB_PATH)
    lib.fqla_version.restype = I
    lib.fqla_version.argtypes = []
    lib.fqla_status_string.restype = C.c_char_p
    lib.fqla_status_string.argtypes = [I]
    lib.fqla_fwd_noalloc_max_pairs.restype = LL
    lib.fqla_fwd_noalloc_max_pairs.argtypes = []
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = I
        fn.argtypes = argtypes
    _lib = lib
    return lib


launch_count = 0  # kernels enqueued through this binding (one per successful entry-point call)


def check(status: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if status != 0:
        msg = load().fqla_status_string(status).decode()
        raise FqlaError(f"{what} failed with status {status}: {msg}")
