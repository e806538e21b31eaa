"""ctypes binding of ``libdf11.so`` -- the place where the reference loads its PTX with
cupy (``cp.RawModule(path=ptx_path).get_function('decode')``, dfloat11/dfloat11.py:38-40).

There is no fallback: if the library cannot be loaded, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int32, c_int64, c_uint32, c_void_p

from .build import LIB_PATH, _stale, build_lib

DF11_OK = 0
DF11_ERR_BADARG = -1
DF11_ERR_CUDA = -2
DF11_ERR_CORRUPT = -3
DF11_ERR_NOSPACE = -4

STATUS_BAD_TABLE = 1
STATUS_BAD_POSITIONS = 2
STATUS_TRUNCATED = 4
STATUS_TIMEOUT = 8

# every symbol declared in include/df11.h: name -> (restype, argtypes)
SIGNATURES = {
    "df11_version": (c_int32, []),
    "df11_last_error": (c_char_p, []),
    "df11_decode": (c_int32, [c_void_p] * 6 + [c_int32, c_int64, c_int64, c_int32, c_void_p, c_int32, c_void_p]),
    "df11_selftest_wait_timeout": (c_int32, [c_void_p] * 6 + [c_int32, c_int64, c_int64, c_int32, c_int64, c_void_p,
                                             c_int32, c_void_p]),
    "df11_aux_bytes": (c_int64, [c_int64, c_int64]),
    "df11_seek_interval": (c_int32, [c_int32]),
    "df11_decode_range_prepared": (c_int32, [c_void_p] * 4 + [c_int64, c_int64, c_void_p, c_int32, c_int64, c_int64,
                                             c_void_p, c_int32, c_void_p]),
    "df11_decode_range_prepared_shared": (c_int32, [c_void_p] * 4 + [c_int64, c_int64, c_void_p, c_int32, c_int64,
                                                    c_int64, c_int32, c_void_p, c_int32, c_void_p]),
    "df11_prepare": (c_int32, [c_void_p] * 5 + [c_int64, c_int32, c_int64, c_int64, c_void_p, c_int32, c_void_p]),
    "df11_decode_prepared": (c_int32, [c_void_p] * 7 + [c_int32, c_int64, c_int64, c_int32, c_void_p, c_int32, c_void_p]),
    "df11_decode_prepared_shared": (c_int32, [c_void_p] * 7 + [c_int32, c_int64, c_int64, c_int32, c_void_p, c_int32,
                                              c_void_p]),
    "df11_gemv_partials_bytes": (c_int64, [c_int64, c_int64, c_int32]),
    "df11_gemv_prepared": (c_int32, [c_void_p] * 8 + [c_int64, c_int64, c_int64, c_int32, c_int32, c_int64, c_int64,
                                     c_void_p, c_int32, c_void_p]),
    "df11_decode_rows_prepared": (c_int32, [c_void_p] * 5 + [c_int64, c_int64, c_void_p, c_int32, c_int64, c_int64,
                                            c_void_p, c_int32, c_void_p]),
    "df11_decode_static": (c_int32, [c_void_p] * 6 + [c_int32, c_int64, c_int64, c_void_p, c_int32, c_void_p]),
    "df11_allreduce_flag_bytes": (c_int64, []),
    "df11_allreduce_counter_bytes": (c_int64, []),
    "df11_allreduce_bf16": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_int64, c_int64,
                                      c_int64, c_void_p, c_int32, c_void_p]),
    "df11_selftest_allreduce_one_gpu": (c_int32, [c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                                  c_int64, c_void_p, c_int32, c_void_p]),
    "df11_validate_host": (c_int32, [c_void_p, c_int32, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p]),
    "df11_encode_size": (c_int64, [c_void_p, c_int64, c_void_p]),
    "df11_encode_device_workspace_bytes": (c_int64, [c_int64]),
    "df11_encode_device_count": (c_int32, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                           c_int32, c_void_p]),
    "df11_encode_device_pack": (c_int32, [c_void_p, c_int64, c_void_p, c_void_p, c_int32, c_uint32, c_void_p, c_void_p,
                                          c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int32, c_void_p]),
    "df11_encode_host": (c_int32, [c_void_p, c_int64, c_void_p, c_void_p, c_int32, c_uint32, c_void_p, c_int64,
                                   c_void_p, c_int64, c_void_p, c_int64, c_int32]),
}


class DF11Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libdf11 error {code}: {message}")
        self.code = code


def _load() -> ctypes.CDLL:
    # A library older than its sources is rebuilt first (needs nvcc); a missing one that
    # cannot be built, or one that lacks a declared symbol, is an ImportError.
    if _stale():
        try:
            build_lib(force=True)
        except Exception as exc:  # noqa: BLE001
            if not os.path.exists(LIB_PATH):
                raise ImportError(
                    f"{LIB_PATH} is missing and could not be built ({exc}); build it with "
                    "`python dfloat11_b200/build.py` (needs nvcc; there is no non-CUDA fallback)") from exc
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise ImportError(f"{LIB_PATH} does not export {name}; rebuild it with "
                              "`python dfloat11_b200/build.py --force`") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


def check(rc: int) -> int:
    if rc < 0:
        raise DF11Error(int(rc), lib.df11_last_error().decode("utf-8", "replace"))
    return int(rc)
