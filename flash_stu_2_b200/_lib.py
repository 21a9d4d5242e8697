"""ctypes binding of libstu_b200.so (the C-ABI declared in include/stu_b200.h).

The library is looked up next to this file.  There is no CPU implementation behind these calls:
when the library is missing the import of the ops raises, and every op refuses non-CUDA tensors.
"""
import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libstu_b200.so")

ERRORS = {
    -1: "unsupported dtype (only float32 and bfloat16)",
    -2: "bad shape argument",
    -3: "pointer or stride not 16-byte aligned",
    -4: "configuration not supported by the CUDA kernels",
    -5: "null pointer",
    -6: "device status word set",
    -7: "the call needs more scratch than the library's built-in 32 MiB array",
}

_lib = None

_P = c_void_p
_LL = c_longlong
_SIGNATURES = {
    "stu_b200_version": ([], c_int),
    "stu_set_status_word": ([_P], c_int),
    "stu_test_inject_wait_expiry": ([c_int], c_int),
    "stu_rmsnorm": ([_P, _P, _P, c_int, c_int, _LL, _LL, c_float, c_int, _P], c_int),
    "stu_bias_act": ([_P, _P, _LL, c_int, _LL, c_int, c_int, _P], c_int),
    "stu_embed": ([_P, _P, _P, c_int, c_int, c_int, _P, c_int, _P], c_int),
    "stu_linear": ([_P, _LL, _P, _LL, _LL, _P, _P, _LL, _P, _LL, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                    _P, c_float, c_int, c_int, _P], c_int),
    "stu_linear_can_fuse_norm": ([c_int, c_int, c_int, c_int, c_int], c_int),
    "stu_taps_even": ([_P, _P, c_int, c_int, c_int, c_int, _P], c_int),
    "stu_conv_prefill_approx": ([_P, _P, _P, _P, _LL, _LL, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 _P], c_int),
    "stu_conv_prefill_approx_tc5": ([_P, _P, _P, _P, _LL, _LL, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_int,
                                     _P], c_int),
    "stu_conv_prefill_set_timeline": ([_P], c_int),
    "stu_set_programmatic_launch": ([c_int], c_int),
    "stu_conv_prefill_approx_static": ([_P, _P, _P, _LL, _LL, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P],
                                       c_int),
    "stu_taps_rev8": ([_P, _P, c_int, c_int, c_int, _P], c_int),
    "stu_decode_approx": ([_P, _LL, _P, _P, _P, _P, _P, _P, _P, _LL, c_int, c_int, c_int, c_float, _P, c_int, _P],
                          c_int),
    "stu_decode_approx_shard": ([_P, _LL, _P, _P, _P, _P, _P, _P, _LL, c_int, c_int, c_int, c_int, c_float, c_int, _P,
                                 c_int, _P], c_int),
    "stu_decode_approx_pipelined": ([_P, _LL, _P, _P, _P, _P, _P, _P, _LL, c_int, c_int, c_int, c_int, c_float, c_int,
                                     _P, c_int, _P], c_int),
    "stu_block_step_workspace_bytes": ([c_int, c_int], c_longlong),
    "stu_block_decode_step": ([_P, _LL, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _LL, c_int, c_int, c_int, c_int, c_float,
                               c_float, _P, _LL, c_int, _P, c_int, _P], c_int),
    "stu_to_history": ([_P, _LL, _LL, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P], c_int),
    "stu_toeplitz": ([_P, _LL, c_int, _P, c_int, _LL, c_int, _P], c_int),
    "stu_full_combine": ([_P, _P, _LL, _P, _LL, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P], c_int),
    "stu_full_decode_prepare": ([_P, _LL, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P, c_int, _P], c_int),
    "stu_full_decode_combine": ([_P, _LL, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P], c_int),
    "stu_lds_final_state": ([_P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P], c_int),
    "stu_lds_chunk_scan": ([_P, _LL, _LL, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P], c_int),
    "stu_lds_decode_features": ([_P, _LL, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P], c_int),
    "stu_swa_forward": ([_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                         _P], c_int),
    "stu_decode_approx_projected": ([_P, _LL, _P, _LL, _P, _P, _P, _P, _LL, c_int, c_int, c_int, c_int, _P, c_int, _P],
                                    c_int),
    "stu_peer_dest_bytes": ([], c_int),
    "stu_peer_alloc": ([_P, _LL], c_int),
    "stu_peer_free": ([_P], c_int),
    "stu_peer_export": ([_P, _P], c_int),
    "stu_peer_open": ([_P, _P], c_int),
    "stu_peer_close": ([_P], c_int),
    "stu_peer_write": ([_P, _P, _LL], c_int),
    "stu_peer_read": ([_P, _P, _LL], c_int),
    "stu_linear_push": ([_P, _LL, _P, _LL, c_int, c_int, c_int, _P, _LL, c_int, _P], c_int),
    "stu_decode_approx_push": ([_P, _LL, _P, _P, _P, _P, _P, _P, _LL, c_int, c_int, c_int, c_int, c_float, _P, c_int,
                                _P], c_int),
    "stu_peer_combine": ([_P, _LL, _P, _LL, _LL, c_int, _P, c_int, _P, _P, _P, _LL, c_float, c_int, c_int, _P, c_int,
                          c_int, _P], c_int),
    "stu_peer_xchg_bytes": ([], c_int),
    "stu_peer_exchange": ([_P, _P, _LL, _P, _LL, c_int, c_int, _LL, _P, _P, _LL, c_float, c_int, c_int, _P, c_int,
                           c_int, _P], c_int),
    "stu_swa_prefill_scratch_elems": ([c_int, c_int, c_int, c_int], c_longlong),
    "stu_swa_prefill_tc5": ([_P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, _P,
                             c_int, _P], c_int),
    "stu_sample": ([_P, _LL, c_int, c_int, c_float, c_int, c_float, c_int, _P, _P, _LL, _P, c_int, _P], c_int),
}


def exported_symbols():
    """Names of every entry point this binding expects the library to export."""
    return sorted(_SIGNATURES)


def load(build_if_missing: bool = True):
    global _lib
    if _lib is not None:
        return _lib
    if build_if_missing:
        from . import _build
        if _build.stale():
            if os.path.exists(os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")):
                _build.build_library()
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing and could not be built: the flash_stu_2_b200 ops have no CPU fallback; "
            "run `python -c 'import __graft_entry__ as g; g.build()'` on a machine with nvcc")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (argtypes, restype) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
    _lib = lib
    return lib


def check(rc: int, what: str):
    if rc == 0:
        return
    if rc < 0:
        raise RuntimeError(f"{what}: {ERRORS.get(rc, 'error')} (code {rc})")
    raise RuntimeError(f"{what}: CUDA error {rc}")
