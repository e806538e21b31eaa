"""Launches the REFERENCE's own decode kernel on the GPU.  TEST / BENCH INFRASTRUCTURE ONLY.

``oracle/Makefile`` (target ``ref``) compiles the reference's ``dfloat11/decode.cu`` where it
lies into ``oracle/_ref/`` and places its shipped ``decode.ptx`` beside it; this module loads
one of those files through the CUDA driver API (cupy, which the reference uses at
dfloat11/dfloat11.py:38-40, is not installed) and launches it exactly as the reference
does at dfloat11/dfloat11.py:139-151: grid ``ceil(n_bytes / 4096)``, block 512, dynamic
shared memory ``512*4 + 4 + 2*max_block_elems`` (dfloat11.py:305), nine arguments.

Used for two things only: bit-comparing the new kernel with the reference's on identical
inputs, and timing the reference kernel beside it.  The shipped package never imports this.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(_HERE, "_ref")
VARIANTS = {
    "shipped_ptx": "decode_shipped.ptx",      # the file a reference user runs (JIT from .target sm_52)
    "recompiled_sm100a": "decode_ref_sm100a.cubin",  # same source, nvcc -O3 for sm_100a
}

_functions = {}


def available(variant: str = "shipped_ptx") -> bool:
    return os.path.exists(os.path.join(REF_DIR, VARIANTS[variant]))


def _check(res):
    err = res[0]
    if int(err) != 0:
        raise RuntimeError(f"CUDA driver error {err}")
    return res[1:] if len(res) > 2 else (res[1] if len(res) == 2 else None)


def _function(variant: str, device: int):
    key = (variant, device)
    if key not in _functions:
        from cuda.bindings import driver
        torch.cuda.init()
        with torch.cuda.device(device):
            torch.zeros(1, device="cuda")          # make torch's primary context current
            path = os.path.join(REF_DIR, VARIANTS[variant])
            with open(path, "rb") as f:
                image = f.read() + b"\0"
            module = _check(driver.cuModuleLoadData(image))
            fn = _check(driver.cuModuleGetFunction(module, b"decode"))
            _check(driver.cuFuncSetAttribute(
                fn, driver.CUfunction_attribute.CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, 200 * 1024))
        _functions[key] = (module, fn)
    return _functions[key][1]


def shared_mem_size(output_positions_u32: np.ndarray) -> int:
    """dfloat11.py:299-306."""
    d = np.diff(output_positions_u32.astype(np.int64))
    return 512 * 4 + 4 + int(d.max()) * 2


def decode(luts, encoded_exponent, sign_mantissa, output_positions, gaps, out, shared_mem: int,
           variant: str = "shipped_ptx"):
    """Launch the reference kernel on torch's current stream.  All tensors on one CUDA device."""
    from cuda.bindings import driver
    device = luts.device.index
    fn = _function(variant, device)
    n_luts, n_bytes, n_elements = luts.shape[0], encoded_exponent.numel(), sign_mantissa.numel()
    if n_bytes >= 2 ** 31 or n_elements >= 2 ** 31:
        raise ValueError("the reference kernel takes 32-bit sizes (decode.cu:33)")
    grid = -(-n_bytes // 4096)
    args = [ctypes.c_void_p(t.data_ptr()) for t in
            (luts, encoded_exponent, sign_mantissa, output_positions, gaps, out)]
    args += [ctypes.c_int(n_luts), ctypes.c_int(n_bytes), ctypes.c_int(n_elements)]
    arg_ptrs = (ctypes.c_void_p * len(args))(*[ctypes.addressof(a) for a in args])
    stream = torch.cuda.current_stream(device).cuda_stream
    with torch.cuda.device(device):
        _check(driver.cuLaunchKernel(fn, grid, 1, 1, 512, 1, 1, int(shared_mem), stream,
                                     ctypes.addressof(arg_ptrs), 0))
    return out
