"""The C ABI: every function declared in include/df11.h is exported by libdf11.so, host-only
entry points work without a GPU, and argument errors come back as codes with a message."""
import ctypes
import os
import re

import numpy as np

from dfloat11_b200 import _lib
from dfloat11_b200.build import LIB_PATH

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "df11.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(df11_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_functions()
    assert {"df11_decode", "df11_prepare", "df11_decode_prepared", "df11_aux_bytes", "df11_decode_static",
            "df11_validate_host", "df11_encode_size", "df11_encode_host", "df11_version",
            "df11_last_error"} <= set(names)
    lib = ctypes.CDLL(LIB_PATH)
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in df11.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature in _lib.py"


def test_version_and_sizes():
    assert _lib.lib.df11_version() >= 100
    small = _lib.lib.df11_aux_bytes(1000, 4000)
    big = _lib.lib.df11_aux_bytes(10 ** 8, 4 * 10 ** 8)
    assert 0 < small < big
    interval = _lib.lib.df11_seek_interval(0)
    assert interval in (16, 32)
    assert abs(big - 4 * 10 ** 8 * 68 / (32 * interval)) < 10 ** 6   # 0.133 bytes per element at 16, 0.066 at 32
    assert _lib.lib.df11_seek_interval(16) == 16
    at16 = _lib.lib.df11_aux_bytes(10 ** 8, 4 * 10 ** 8)
    assert _lib.lib.df11_seek_interval(32) == 32
    at32 = _lib.lib.df11_aux_bytes(10 ** 8, 4 * 10 ** 8)
    assert at32 < 0.51 * at16                                   # half the seek points (the table stays)
    assert _lib.lib.df11_seek_interval(24) == _lib.DF11_ERR_BADARG
    _lib.lib.df11_seek_interval(interval)
    assert _lib.lib.df11_aux_bytes(-1, 0) == _lib.DF11_ERR_BADARG


def test_argument_errors_do_not_need_a_gpu():
    L = _lib.lib
    buf = np.zeros(1024, np.uint8)
    p = buf.ctypes.data
    assert L.df11_decode(None, p, p, p, p, p, 4, 10, 10, 0, None, 0, None) == _lib.DF11_ERR_BADARG
    assert b"null" in L.df11_last_error()
    assert L.df11_decode(p, p, p, p, p, p, 1, 10, 10, 0, None, 0, None) == _lib.DF11_ERR_BADARG
    assert b"n_luts" in L.df11_last_error()
    assert L.df11_decode(p, p, p, p, p, p, 4, -1, 10, 0, None, 0, None) == _lib.DF11_ERR_BADARG
    assert L.df11_decode(p, p, p, p, p, p, 4, 0, 0, 0, None, 0, None) == _lib.DF11_OK     # nothing to do
    assert L.df11_prepare(p, p, p, p, p + 1, 1 << 20, 4, 10, 10, None, 0, None) == _lib.DF11_ERR_BADARG
    assert L.df11_prepare(p, p, p, p, p, 16, 4, 10, 10, None, 0, None) == _lib.DF11_ERR_NOSPACE
    assert L.df11_decode_static(p, p, p, p, p, p, 4, 10, (1 << 25) + 1, None, 0, None) == _lib.DF11_ERR_NOSPACE
    assert L.df11_encode_size(None, 0, None) == _lib.DF11_ERR_BADARG
    # the all-reduce entry points check their arguments before they touch the device
    eight = (ctypes.c_uint64 * 8)(*([p] * 8))
    assert L.df11_allreduce_flag_bytes() > 2 << 20 and L.df11_allreduce_counter_bytes() == 256
    assert L.df11_allreduce_bf16(None, eight, p, 0, 2, p, p, 8, 1 << 20, 0, None, 0, None) == _lib.DF11_ERR_BADARG
    assert L.df11_allreduce_bf16(eight, eight, p, 0, 9, p, p, 8, 1 << 20, 0, None, 0, None) == _lib.DF11_ERR_BADARG
    assert b"ranks" in L.df11_last_error()
    assert L.df11_allreduce_bf16(eight, eight, p, 2, 2, p, p, 8, 1 << 20, 0, None, 0, None) == _lib.DF11_ERR_BADARG
    assert L.df11_allreduce_bf16(eight, eight, p, 0, 2, p, p, 12, 1 << 20, 0, None, 0, None) == _lib.DF11_ERR_BADARG
    assert L.df11_allreduce_bf16(eight, eight, p, 0, 2, p, p, 1 << 20, 1 << 20, 0, None, 0, None) == _lib.DF11_ERR_NOSPACE
    assert L.df11_allreduce_bf16(eight, eight, p, 0, 2, p, p, 0, 1 << 20, 0, None, 0, None) == _lib.DF11_OK   # nothing to sum
    assert L.df11_selftest_allreduce_one_gpu(5, p, p, p, p, p, 8, 1 << 20, 0, None, 0, None) == _lib.DF11_ERR_BADARG
    assert L.df11_selftest_allreduce_one_gpu(2, p, p, p, p, p, 12, 1 << 20, 0, None, 0, None) == _lib.DF11_ERR_BADARG
    assert L.df11_decode_range_prepared_shared(p, p, p, p, 0, -1, p, 4, 10, 10, 1, None, 0, None) == _lib.DF11_ERR_BADARG
    assert L.df11_decode_range_prepared_shared(p, p, p, p, 0, 512, p, 4, 10, 10, -1, None, 0, None) == _lib.DF11_ERR_BADARG


def test_header_is_plain_c():
    """include/df11.h is what a foreign-function binding reads: it must compile as C99 and as C++."""
    import shutil
    import subprocess
    header = os.path.join(ROOT, "include", "df11.h")
    for compiler, language in (("gcc", ["-std=c99", "-x", "c"]), ("g++", ["-x", "c++"])):
        if shutil.which(compiler) is None:
            continue
        done = subprocess.run([compiler, "-fsyntax-only", "-Wall"] + language + [header], capture_output=True, text=True)
        assert done.returncode == 0, done.stderr
