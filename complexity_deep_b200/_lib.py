"""ctypes binding of libcdeep.so (include/cdeep.h).

There is no fallback: if the library is missing the import of any accelerated module
raises, and every non-zero status code becomes a Python exception.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_longlong, c_size_t, c_void_p

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libcdeep.so")
CHECKS_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libcdeep_checks.so")

ABI_VERSION = 3

# name -> (restype, argtypes); mirrors include/cdeep.h one to one
SIGNATURES = {
    "cd_version": (c_int, []),
    "cd_error_string": (c_char_p, [c_int]),
    "cd_last_cuda_error": (c_char_p, []),
    "cd_max_groups": (c_int, []),
    "cd_checks_enabled": (c_int, []),
    "cd_splitk_workspace_bytes": (c_size_t, []),
    "cd_splitk_workspace_set": (c_int, [c_void_p, c_size_t, c_void_p]),
    "cd_splitk_ranges": (c_int, [c_int, c_int, c_int]),
    "cd_splitk_config": (c_int, [c_int]),
    "cd_status_fetch": (c_int, [ctypes.POINTER(c_int)]),
    "cd_selftest_wait_timeout": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "cd_route_workspace_bytes": (c_size_t, [c_int, c_int]),
    "cd_route": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                         c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "cd_route_static_max_tokens": (c_int, [c_int]),
    "cd_route_static": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_void_p]),
    "cd_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
                           c_int, c_int, c_void_p]),
    "cd_rmsnorm_split": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int,
                                 c_int, c_void_p]),
    "cd_gather_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "cd_qk_norm_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int,
                                c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "cd_decode_rope_append": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                                      c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_longlong,
                                      c_longlong, c_longlong, c_int, c_void_p, c_void_p]),
    "cd_decode_attention_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "cd_decode_attention": (c_int, [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong,
                                    c_longlong, c_longlong, c_void_p, c_longlong, c_float, c_int,
                                    c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                    c_size_t, c_void_p]),
    "cd_attention_prefill_supported": (c_int, [c_int, c_int, c_int, c_int, c_int]),
    "cd_attention_prefill": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                     c_void_p]),
    "cd_gate_up_packed_rows": (c_int, [c_int, c_int]),
    "cd_moe_up": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                          c_int, c_void_p]),
    "cd_moe_up_pair": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p,
                               c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "cd_pack_gate_up": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                c_void_p]),
    "cd_pack_down": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "cd_moe_down": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                            c_void_p]),
    "cd_peer_put_i32": (c_int, [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p]),
    "cd_ep_plan": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_longlong, c_int, c_void_p,
                           c_void_p, c_void_p, c_void_p]),
    "cd_push_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int,
                             c_int, c_void_p]),
    "cd_peer_barrier": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "cd_moe_down_push": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                 c_int, c_void_p]),
    "cd_moe_combine": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "cd_mu_qkv": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                          c_void_p]),
    "cd_mu_qkv_rope_supported": (c_int, [c_int, c_int, c_int, c_int, c_int]),
    "cd_mu_qkv_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int,
                               c_int, c_int, c_int, c_void_p]),
    "cd_mu_proj": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_float, c_int, c_float, c_float,
                           c_void_p, c_int, c_int, c_void_p]),
    "cd_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                          c_int, c_int, c_void_p]),
}

_lib = None


class CdeepError(RuntimeError):
    """A libcdeep entry point returned a non-zero status."""


def open_library(path: str) -> ctypes.CDLL:
    """Opens one build of the library and binds every declared entry point."""
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -m complexity_deep_b200.build` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback for these kernels.")
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if a declared symbol is not exported
        fn.restype = res
        fn.argtypes = args
    if lib.cd_version() != ABI_VERSION:
        raise ImportError(f"libcdeep ABI {lib.cd_version()} != expected {ABI_VERSION}; rebuild")
    return lib


def load() -> ctypes.CDLL:
    """Loads the library once; raises when it is missing or its ABI version differs.
    CDEEP_CHECKS=1 in the environment selects the checking build (libcdeep_checks.so)."""
    global _lib
    if _lib is None:
        _lib = open_library(CHECKS_LIB_PATH if os.environ.get("CDEEP_CHECKS") == "1" else LIB_PATH)
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        lib = load()
        msg = lib.cd_error_string(status).decode()
        detail = lib.cd_last_cuda_error().decode() if status in (2, 3) else ""
        raise CdeepError(f"{what}: {msg}" + (f" ({detail})" if detail else ""))
