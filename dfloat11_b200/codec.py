"""Host side of the DF11 format: code construction, LUT layout and tensor packing.

Mirrors the roles of the reference's ``dfloat11/dfloat11_utils.py`` (``get_codec`` :24,
``get_32bit_codec`` :37, ``get_luts`` :68, ``encode_weights`` :173) and produces tensors
with the same layout and meaning, so that files written here load in the reference
and vice versa.  Differences, all inside what the format allows:

* the prefix code is built here (Huffman lengths, package-merge when the 32-bit limit
  binds, canonical assignment) instead of by the third-party ``dahuffman`` package, and
  carries no end-of-stream symbol: the last byte is padded with zero bits, which the
  decoder discards through ``n_elements`` exactly as it discards the reference's padding;
* LUT rows are filled explicitly for every index (the reference relies on forward fill,
  dfloat11_utils.py:103-106, and fails when index 0 of a row is unmapped);
* exponent values >= 240 cannot be represented (they collide with the row pointers,
  decode.cu:106) and are rejected with an error instead of being silently corrupted;
* bit packing is done by ``df11_encode_host`` in libdf11 (threads, linear time).
"""
from __future__ import annotations

import heapq
import os
from typing import Dict, Sequence, Tuple

import numpy as np
import torch

from . import _lib

BYTES_PER_THREAD = 8          # dfloat11.py:45
THREADS_PER_BLOCK = 512       # dfloat11.py:46
BLOCK_BYTES = BYTES_PER_THREAD * THREADS_PER_BLOCK
MAX_CODE_LEN = 32             # dfloat11_utils.py:49
MAX_SYMBOL = 239              # entries >= 240 are row pointers (decode.cu:106)
MAX_SUB_ROWS = 16             # pointers 240..255 address rows 16..1


class UnrepresentableError(ValueError):
    """The weights cannot be stored in the DF11 format (e.g. exponents >= 240)."""


def split_bf16(weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """BF16 tensor -> (exponent uint8, sign_mantissa uint8); dfloat11_utils.py:176-178."""
    assert weight.dtype == torch.bfloat16, weight.dtype
    w = weight.contiguous().view(torch.int16).flatten()
    exponent = ((w >> 7) & 0xFF).to(torch.uint8)
    sign_mantissa = (((w >> 8) & 0x80) | (w & 0x7F)).to(torch.uint8)
    return exponent, sign_mantissa


def exponent_histogram(exponent: torch.Tensor) -> np.ndarray:
    """256-bin histogram of a uint8 tensor (any device)."""
    flat = exponent.flatten()
    hist = torch.zeros(256, dtype=torch.int64, device=flat.device)
    step = 1 << 28                                   # bounded temporaries on very large units
    for s in range(0, flat.numel(), step):
        hist += torch.bincount(flat[s:s + step].to(torch.int32), minlength=256)
    return hist.cpu().numpy().astype(np.int64)


def _huffman_lengths(freq: np.ndarray) -> np.ndarray:
    syms = np.nonzero(freq)[0]
    lens = np.zeros(256, dtype=np.int64)
    if syms.size == 1:
        lens[syms[0]] = 1
        return lens
    heap = [(int(freq[s]), int(s), (int(s),)) for s in syms]
    heapq.heapify(heap)
    tick = 256
    while len(heap) > 1:
        fa, _, a = heapq.heappop(heap)
        fb, _, b = heapq.heappop(heap)
        for s in a + b:
            lens[s] += 1
        heapq.heappush(heap, (fa + fb, tick, a + b))
        tick += 1
    return lens


def _package_merge(freq: np.ndarray, limit: int) -> np.ndarray:
    """Optimal code lengths under a maximum length (used only when plain Huffman exceeds it)."""
    syms = sorted((int(s) for s in np.nonzero(freq)[0]), key=lambda s: (int(freq[s]), s))
    n = len(syms)
    assert n <= (1 << limit)
    leaves = [(int(freq[s]), (s,)) for s in syms]
    packages = list(leaves)
    for _ in range(limit - 1):
        merged = [(packages[i][0] + packages[i + 1][0], packages[i][1] + packages[i + 1][1])
                  for i in range(0, len(packages) - 1, 2)]
        packages = sorted(leaves + merged, key=lambda p: p[0])
    lens = np.zeros(256, dtype=np.int64)
    for _, members in packages[:2 * n - 2]:
        for s in members:
            lens[s] += 1
    return lens


def code_lengths(freq: np.ndarray, limit: int = MAX_CODE_LEN) -> np.ndarray:
    """Prefix-code length of every exponent value (0 = does not occur)."""
    freq = np.asarray(freq, dtype=np.int64)
    if freq.shape != (256,):
        raise ValueError("need a 256-bin histogram")
    if freq.sum() == 0:
        raise ValueError("empty histogram")
    if freq[MAX_SYMBOL + 1:].any():
        raise UnrepresentableError(
            "exponent values >= 240 (|w| >= 2^113, inf, nan) cannot be represented in DF11")
    lens = _huffman_lengths(freq)
    if lens.max() > limit:
        lens = _package_merge(freq, limit)
    return lens


def canonical_codes(lens: np.ndarray) -> np.ndarray:
    """Canonical assignment: shorter codes first, numerically increasing, MSB-first values."""
    vals = np.zeros(256, dtype=np.uint32)
    order = sorted((int(l), int(s)) for s, l in enumerate(lens) if l > 0)
    code, prev = 0, order[0][0]
    for l, s in order:
        code <<= (l - prev)
        vals[s] = code
        code += 1
        prev = l
    return vals


def build_luts(lens: np.ndarray, vals: np.ndarray) -> np.ndarray:
    """The ``luts`` tensor of the format (layout of dfloat11_utils.py:68-115).

    Row 0 is indexed by the first stream byte; an entry < 240 is the decoded exponent,
    an entry >= 240 points to row ``256 - entry`` which is indexed by the next byte; the
    last row gives the code length of every exponent value.
    """
    codes = [(int(lens[s]), int(vals[s]), s) for s in range(256) if lens[s] > 0]
    strs = {s: format(v, "b").rjust(l, "0") for l, v, s in codes}
    prefixes = {""}
    for s, c in strs.items():
        for cut in range(8, ((len(c) - 1) // 8) * 8 + 1, 8):
            prefixes.add(c[:cut])
    rows = sorted(prefixes, key=lambda p: (len(p), p))
    if len(rows) - 1 > MAX_SUB_ROWS:
        raise UnrepresentableError(
            f"the code needs {len(rows) - 1} second-level tables; the format can address {MAX_SUB_ROWS}")
    index = {p: i for i, p in enumerate(rows)}
    luts = np.zeros((len(rows) + 1, 256), dtype=np.uint8)
    filled = np.zeros((len(rows), 256), dtype=bool)
    for s, c in strs.items():
        for level in range((len(c) - 1) // 8 + 1):
            row = index[c[:8 * level]]
            rest = c[8 * level:]
            if len(rest) <= 8:                       # the code ends in this row
                first = int(rest.ljust(8, "0"), 2)
                luts[row, first:first + (1 << (8 - len(rest)))] = s
                filled[row, first:first + (1 << (8 - len(rest)))] = True
            else:                                    # pointer to the row of the longer prefix
                key = int(rest[:8], 2)
                luts[row, key] = 256 - index[c[:8 * level + 8]]
                filled[row, key] = True
    # indices no code reaches (only when the code is incomplete, e.g. a single symbol)
    # inherit the previous entry, as the reference's fill does
    for r in range(len(rows)):
        for i in range(256):
            if not filled[r, i]:
                luts[r, i] = luts[r, i - 1] if i > 0 else luts[r, np.argmax(filled[r])]
    for s in strs:
        luts[-1, s] = lens[s]
    return luts


def get_codec(weight: torch.Tensor):
    """Code table for the exponents of ``weight``: (lens[256], vals[256], histogram)."""
    exponent, _ = split_bf16(weight)
    hist = exponent_histogram(exponent)
    lens = code_lengths(hist)
    return lens, canonical_codes(lens), hist


def get_luts(lens: np.ndarray, vals: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(build_luts(lens, vals))


def pack_exponents(exponent: np.ndarray, lens: np.ndarray, vals: np.ndarray, n_threads: int | None = None,
                   pad: Tuple[int, int] = (0, 0)):
    """Exponent bytes -> (encoded, gaps, output_positions) through ``df11_encode_host``."""
    exponent = np.ascontiguousarray(exponent, dtype=np.uint8)
    code_len = np.ascontiguousarray(lens, dtype=np.uint8)
    code_val = np.ascontiguousarray(vals, dtype=np.uint32)
    n_bytes = _lib.check(_lib.lib.df11_encode_size(exponent.ctypes.data, exponent.size, code_len.ctypes.data))
    n_blocks = -(-n_bytes // BLOCK_BYTES)
    encoded = np.empty(n_bytes, dtype=np.uint8)
    gaps = np.empty(n_blocks * THREADS_PER_BLOCK * 5 // 8, dtype=np.uint8)
    positions = np.empty(n_blocks + 1, dtype=np.uint32)
    if n_threads is None:
        n_threads = max(1, min(32, os.cpu_count() or 1))
    _lib.check(_lib.lib.df11_encode_host(
        exponent.ctypes.data, exponent.size, code_len.ctypes.data, code_val.ctypes.data,
        int(pad[0]), int(pad[1]), encoded.ctypes.data, n_bytes, gaps.ctypes.data, gaps.size,
        positions.ctypes.data, positions.size, int(n_threads)))
    return encoded, gaps, positions


def pack_exponents_gpu(exponent: torch.Tensor, lens: np.ndarray, vals: np.ndarray, pad: Tuple[int, int] = (0, 0)):
    """The same packing on the GPU, for exponent bytes that live in device memory
    (``df11_encode_device_count`` / ``df11_encode_device_pack``): CUDA tensors
    ``(encoded uint8, gaps uint8, output_positions int32 holding uint32 bits)``, byte for byte
    what ``pack_exponents`` returns."""
    if not exponent.is_cuda or exponent.dtype != torch.uint8:
        raise RuntimeError("pack_exponents_gpu needs a uint8 CUDA tensor")
    exponent = exponent.contiguous()
    device = exponent.device
    n = exponent.numel()
    code_len = np.ascontiguousarray(lens, dtype=np.uint8)
    code_val = np.ascontiguousarray(vals, dtype=np.uint32)
    stream = torch.cuda.current_stream(device)
    workspace = torch.empty(_lib.check(_lib.lib.df11_encode_device_workspace_bytes(n)) // 8 + 1, dtype=torch.int64,
                            device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    total = np.zeros(1, dtype=np.int64)
    _lib.check(_lib.lib.df11_encode_device_count(
        exponent.data_ptr(), n, code_len.ctypes.data, code_val.ctypes.data, workspace.data_ptr(),
        workspace.numel() * 8, total.ctypes.data, status.data_ptr(), device.index, stream.cuda_stream))
    stream.synchronize()
    if status.item() != 0:
        raise UnrepresentableError("an exponent value that occurs has no code")
    n_bytes = (int(total[0]) + 7) // 8
    n_blocks = -(-n_bytes // BLOCK_BYTES)
    encoded = torch.empty((n_bytes + 3) // 4 * 4, dtype=torch.uint8, device=device)
    gaps = torch.empty(n_blocks * THREADS_PER_BLOCK * 5 // 8, dtype=torch.uint8, device=device)
    positions = torch.empty(n_blocks + 1, dtype=torch.int32, device=device)
    _lib.check(_lib.lib.df11_encode_device_pack(
        exponent.data_ptr(), n, code_len.ctypes.data, code_val.ctypes.data, int(pad[0]), int(pad[1]),
        workspace.data_ptr(), encoded.data_ptr(), n_bytes, gaps.data_ptr(), gaps.numel(), positions.data_ptr(),
        positions.numel(), device.index, stream.cuda_stream))
    return encoded[:n_bytes], gaps, positions


def encode_weights(weights: Sequence[torch.Tensor], n_threads: int | None = None) -> Dict[str, torch.Tensor]:
    """Compress the BF16 tensors of one unit (concatenated in order) into the six DF11 tensors.

    Same roles and dtypes as the buffers the reference registers (dfloat11.py:593-598):
    ``luts`` uint8 [n_luts,256], ``encoded_exponent`` uint8, ``sign_mantissa`` uint8,
    ``output_positions`` uint8 (a byte view of uint32), ``gaps`` uint8, ``split_positions`` int64.
    """
    flat = [w.detach().reshape(-1) for w in weights]
    sizes = torch.tensor([w.numel() for w in flat], dtype=torch.int64)
    split_positions = torch.cumsum(sizes, dim=0)[:-1]
    combined = torch.cat(flat) if len(flat) > 1 else flat[0]
    if combined.numel() == 0:
        raise ValueError("cannot compress an empty unit")
    exponent, sign_mantissa = split_bf16(combined)
    hist = exponent_histogram(exponent)
    lens = code_lengths(hist)
    vals = canonical_codes(lens)
    luts = build_luts(lens, vals)
    if exponent.is_cuda and os.environ.get("DF11_HOST_ENCODER", "0") != "1":
        # weights already on a GPU: pack there (same bytes as the host packer) and bring the
        # compressed tensors back, a third of the size of what would otherwise cross PCIe
        enc_d, gaps_d, pos_d = pack_exponents_gpu(exponent, lens, vals)
        encoded_t, gaps_t = enc_d.cpu(), gaps_d.cpu()
        positions_t = pos_d.cpu().view(torch.uint8)
    else:
        encoded, gaps, positions = pack_exponents(exponent.cpu().numpy(), lens, vals, n_threads)
        encoded_t, gaps_t = torch.from_numpy(encoded), torch.from_numpy(gaps)
        positions_t = torch.from_numpy(positions.view(np.uint8).copy())
    return {
        "luts": torch.from_numpy(luts),
        "encoded_exponent": encoded_t,
        "sign_mantissa": sign_mantissa.cpu(),
        "output_positions": positions_t,
        "gaps": gaps_t,
        "split_positions": split_positions,
    }


def validate_unit(luts, encoded_exponent, sign_mantissa, output_positions, gaps) -> int:
    """Host-side consistency check of one unit; returns ``max_block_elems``.  Raises DF11Error."""
    import ctypes
    luts_np = np.ascontiguousarray(luts.cpu().numpy() if isinstance(luts, torch.Tensor) else luts)
    pos_np = output_positions.cpu().numpy() if isinstance(output_positions, torch.Tensor) else output_positions
    pos_np = np.ascontiguousarray(pos_np)
    if pos_np.dtype == np.uint8:
        pos_np = pos_np.view(np.uint32)
    widest = ctypes.c_int32(0)
    _lib.check(_lib.lib.df11_validate_host(
        luts_np.ctypes.data, luts_np.shape[0], int(encoded_exponent.numel()), int(sign_mantissa.numel()),
        pos_np.ctypes.data, pos_np.size, int(gaps.numel()), ctypes.byref(widest)))
    return int(widest.value)
