"""Torch-facing launchers of the libdf11 decode entry points.

These stand where the reference calls its cupy kernel object
(``_decode(grid=..., block=..., shared_mem=..., args=[...])``, dfloat11/dfloat11.py:142-151
and :576-585): same tensors, same meaning, but the launch goes through the C ABI of
``libdf11.so`` onto torch's current CUDA stream of the tensors' device.  There is no
CPU or pure-PyTorch fallback: tensors that are not on a CUDA device raise.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib


def _require_cuda(_pinned_ok=(), **tensors: torch.Tensor) -> torch.device:
    """The CUDA device all the tensors are on.  Names listed in ``_pinned_ok`` may instead be pinned
    host tensors: page-locked memory has the same address on the device (unified addressing), so a
    kernel can read the few bytes it needs of them over PCIe without a staging copy."""
    device = None
    for name, t in tensors.items():
        if t is None:
            continue
        if not t.is_cuda and name in _pinned_ok and t.is_pinned():
            if not t.is_contiguous():
                raise RuntimeError(f"`{name}` must be contiguous")
            continue
        if not t.is_cuda:
            raise RuntimeError(f"df11 decode needs CUDA tensors; `{name}` is on {t.device}")
        if not t.is_contiguous():
            raise RuntimeError(f"`{name}` must be contiguous")
        if device is None:
            device = t.device
        elif t.device != device:
            raise RuntimeError(f"`{name}` is on {t.device}, expected {device}")
    return device


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def decode(luts: torch.Tensor, encoded_exponent: torch.Tensor, sign_mantissa: torch.Tensor,
           output_positions: torch.Tensor, gaps: torch.Tensor, out: Optional[torch.Tensor] = None,
           max_block_elems: int = 0, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Decompress one DF11 unit into ``out`` (BF16, ``sign_mantissa.numel()`` elements).

    ``output_positions`` may be the uint8 byte view stored on disk or a uint32/int32 tensor.
    ``status`` is an optional int32 tensor of one element that receives DF11_STATUS_* bits.
    Asynchronous: returns right after the launch on the current stream.
    """
    device = _require_cuda(luts=luts, encoded_exponent=encoded_exponent, sign_mantissa=sign_mantissa,
                           output_positions=output_positions, gaps=gaps, out=out, status=status)
    n_elements = sign_mantissa.numel()
    if out is None:
        out = torch.empty(n_elements, dtype=torch.bfloat16, device=device)
    if out.dtype != torch.bfloat16 or out.numel() < n_elements:
        raise RuntimeError("`out` must be a bfloat16 tensor with at least n_elements elements")
    _lib.check(_lib.lib.df11_decode(
        luts.data_ptr(), encoded_exponent.data_ptr(), sign_mantissa.data_ptr(),
        output_positions.data_ptr(), gaps.data_ptr(), out.data_ptr(),
        luts.shape[0], encoded_exponent.numel(), n_elements, int(max_block_elems),
        status.data_ptr() if status is not None else None, device.index, _stream(device)))
    return out


def aux_bytes(n_bytes: int, n_elements: int) -> int:
    """Size in bytes of the auxiliary buffer `prepare` fills for a unit of these sizes."""
    return _lib.check(_lib.lib.df11_aux_bytes(int(n_bytes), int(n_elements)))


def prepare(luts: torch.Tensor, encoded_exponent: torch.Tensor, output_positions: torch.Tensor,
            gaps: torch.Tensor, n_elements: int, aux: Optional[torch.Tensor] = None,
            status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Fill (allocating if needed) the auxiliary buffer that ``decode_prepared`` reads."""
    device = _require_cuda(("encoded_exponent",), luts=luts, encoded_exponent=encoded_exponent,
                           output_positions=output_positions, gaps=gaps, aux=aux, status=status)
    need = aux_bytes(encoded_exponent.numel(), n_elements)
    if aux is None:
        aux = torch.empty(need, dtype=torch.uint8, device=device)
    _lib.check(_lib.lib.df11_prepare(
        luts.data_ptr(), encoded_exponent.data_ptr(), output_positions.data_ptr(), gaps.data_ptr(),
        aux.data_ptr(), aux.numel() * aux.element_size(), luts.shape[0], encoded_exponent.numel(),
        int(n_elements), status.data_ptr() if status is not None else None, device.index, _stream(device)))
    return aux


def decode_prepared(luts: torch.Tensor, encoded_exponent: torch.Tensor, sign_mantissa: torch.Tensor,
                    output_positions: torch.Tensor, gaps: torch.Tensor, aux: torch.Tensor,
                    out: Optional[torch.Tensor] = None, max_block_elems: int = 0,
                    status: Optional[torch.Tensor] = None, ctas_per_sm: int = 0) -> torch.Tensor:
    """Single-pass decode using the buffer made by ``prepare`` for the same unit.

    ``ctas_per_sm`` > 0 caps the CTAs the persistent kernel places on an SM, for a launch that
    should leave room for kernels of other streams (``df11_decode_prepared_shared``)."""
    device = _require_cuda(luts=luts, encoded_exponent=encoded_exponent, sign_mantissa=sign_mantissa,
                           output_positions=output_positions, gaps=gaps, aux=aux, out=out, status=status)
    n_elements = sign_mantissa.numel()
    if out is None:
        out = torch.empty(n_elements, dtype=torch.bfloat16, device=device)
    if out.dtype != torch.bfloat16 or out.numel() < n_elements:
        raise RuntimeError("`out` must be a bfloat16 tensor with at least n_elements elements")
    if ctas_per_sm:
        _lib.check(_lib.lib.df11_decode_prepared_shared(
            luts.data_ptr(), encoded_exponent.data_ptr(), sign_mantissa.data_ptr(),
            output_positions.data_ptr(), gaps.data_ptr(), aux.data_ptr(), out.data_ptr(),
            luts.shape[0], encoded_exponent.numel(), n_elements, int(ctas_per_sm),
            status.data_ptr() if status is not None else None, device.index, _stream(device)))
        return out
    _lib.check(_lib.lib.df11_decode_prepared(
        luts.data_ptr(), encoded_exponent.data_ptr(), sign_mantissa.data_ptr(),
        output_positions.data_ptr(), gaps.data_ptr(), aux.data_ptr(), out.data_ptr(),
        luts.shape[0], encoded_exponent.numel(), n_elements, int(max_block_elems),
        status.data_ptr() if status is not None else None, device.index, _stream(device)))
    return out


def seek_interval(elements: int = 0) -> int:
    """Elements per seek point of the prepared form (16 or 32), process-wide; a non-zero argument
    sets it.  Buffers made by ``prepare`` are only valid under the setting they were made under."""
    return _lib.check(_lib.lib.df11_seek_interval(int(elements)))


def chunk_elements() -> int:
    """Elements per independently decodable chunk of the prepared form (32 seek intervals)."""
    return 32 * seek_interval()


def decode_range_prepared(luts: torch.Tensor, encoded_exponent: torch.Tensor, sign_mantissa: torch.Tensor,
                          aux: torch.Tensor, first_element: int, range_elements: int, out: torch.Tensor,
                          status: Optional[torch.Tensor] = None, ctas_per_sm: int = 0) -> torch.Tensor:
    """Decompress elements ``[first_element, first_element + range_elements)`` of a prepared unit into
    ``out[:range_elements]``.  The range starts on a multiple of ``chunk_elements()`` and ends on one
    or at the end of the unit.  ``ctas_per_sm`` > 0 caps the CTAs per SM, as in ``decode_prepared``."""
    device = _require_cuda(luts=luts, encoded_exponent=encoded_exponent, sign_mantissa=sign_mantissa,
                           aux=aux, out=out, status=status)
    if out.dtype != torch.bfloat16 or out.numel() < range_elements:
        raise RuntimeError("`out` must be a bfloat16 tensor with at least range_elements elements")
    if ctas_per_sm:
        _lib.check(_lib.lib.df11_decode_range_prepared_shared(
            luts.data_ptr(), encoded_exponent.data_ptr(), sign_mantissa.data_ptr(), aux.data_ptr(),
            int(first_element), int(range_elements), out.data_ptr(), luts.shape[0], encoded_exponent.numel(),
            sign_mantissa.numel(), int(ctas_per_sm), status.data_ptr() if status is not None else None,
            device.index, _stream(device)))
        return out[:range_elements]
    _lib.check(_lib.lib.df11_decode_range_prepared(
        luts.data_ptr(), encoded_exponent.data_ptr(), sign_mantissa.data_ptr(), aux.data_ptr(),
        int(first_element), int(range_elements), out.data_ptr(), luts.shape[0], encoded_exponent.numel(),
        sign_mantissa.numel(), status.data_ptr() if status is not None else None, device.index, _stream(device)))
    return out[:range_elements]


def decode_rows_prepared(luts: torch.Tensor, encoded_exponent: torch.Tensor, sign_mantissa: torch.Tensor,
                         aux: torch.Tensor, rows: torch.Tensor, row_elements: int,
                         out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Decompress only the given rows of a unit viewed as ``[n_elements / row_elements, row_elements]``.

    ``rows`` is an int64 CUDA tensor; the result has one row per entry, in that order.  Needs the
    buffer made by ``prepare`` and a row length that is a multiple of ``chunk_elements()``.
    ``encoded_exponent`` and ``sign_mantissa`` may be pinned host tensors (the kernel then reads
    just those rows' bytes over PCIe), as may ``encoded_exponent`` in ``prepare``."""
    device = _require_cuda(("encoded_exponent", "sign_mantissa"), luts=luts, encoded_exponent=encoded_exponent,
                           sign_mantissa=sign_mantissa, aux=aux, rows=rows, out=out, status=status)
    if rows.dtype != torch.int64:
        raise RuntimeError("`rows` must be an int64 tensor")
    n_rows = rows.numel()
    if out is None:
        out = torch.empty(n_rows * row_elements, dtype=torch.bfloat16, device=device)
    if out.dtype != torch.bfloat16 or out.numel() < n_rows * row_elements:
        raise RuntimeError("`out` must be a bfloat16 tensor with at least n_rows * row_elements elements")
    _lib.check(_lib.lib.df11_decode_rows_prepared(
        luts.data_ptr(), encoded_exponent.data_ptr(), sign_mantissa.data_ptr(), aux.data_ptr(),
        rows.data_ptr(), n_rows, int(row_elements), out.data_ptr(), luts.shape[0], encoded_exponent.numel(),
        sign_mantissa.numel(), status.data_ptr() if status is not None else None, device.index, _stream(device)))
    return out[:n_rows * row_elements].view(n_rows, row_elements)


_gemv_scratch = {}          # device -> float32 tensor for the partial sums


def _gemv_workspace(device: torch.device, n_rows: int, in_features: int, m: int) -> torch.Tensor:
    need = _lib.check(_lib.lib.df11_gemv_partials_bytes(n_rows, in_features, m)) // 4
    buf = _gemv_scratch.get(device)
    if buf is None or buf.numel() < need:
        buf = _gemv_scratch[device] = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=device)
    return buf


def gemv_prepared(luts: torch.Tensor, encoded_exponent: torch.Tensor, sign_mantissa: torch.Tensor,
                  aux: torch.Tensor, x: torch.Tensor, first_element: int, n_rows: int, in_features: int,
                  bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                  status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ W.T (+ bias)`` for the ``[n_rows, in_features]`` matrix that starts at element
    ``first_element`` of a prepared unit, decoding the weights on the fly (never written).

    ``x`` is a contiguous BF16 tensor of 1..4 rows of ``in_features``; the result is
    ``[rows, n_rows]`` BF16.  Launches on one device share a scratch area, so they must be
    queued on one stream (or otherwise kept from overlapping)."""
    device = _require_cuda(luts=luts, encoded_exponent=encoded_exponent, sign_mantissa=sign_mantissa, aux=aux,
                           x=x, bias=bias, out=out, status=status)
    if x.dtype != torch.bfloat16 or (bias is not None and bias.dtype != torch.bfloat16):
        raise RuntimeError("`x` and `bias` must be bfloat16")
    if x.numel() % in_features:
        raise RuntimeError("`x` does not hold whole rows of in_features elements")
    m = x.numel() // in_features
    if out is None:
        out = torch.empty(m, n_rows, dtype=torch.bfloat16, device=device)
    if out.dtype != torch.bfloat16 or out.numel() < m * n_rows:
        raise RuntimeError("`out` must be a bfloat16 tensor of m * n_rows elements")
    partials = _gemv_workspace(device, n_rows, in_features, m)
    _lib.check(_lib.lib.df11_gemv_prepared(
        luts.data_ptr(), encoded_exponent.data_ptr(), sign_mantissa.data_ptr(), aux.data_ptr(), x.data_ptr(),
        out.data_ptr(), bias.data_ptr() if bias is not None else None, partials.data_ptr(),
        int(first_element), int(n_rows), int(in_features), int(m), luts.shape[0], encoded_exponent.numel(),
        sign_mantissa.numel(), status.data_ptr() if status is not None else None, device.index, _stream(device)))
    return out
