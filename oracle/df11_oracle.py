"""CPU oracle for the DFloat11 decode path.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import this module; the shipped package never does.

Contents
--------
* ``decode_c``      -- ctypes front end of ``df11_oracle.c`` (scalar C, optional threads).
* ``decode_py``     -- the same rule as a pure-Python loop, for tiny cases; it
  shares no code with the C file, so the two check each other.
* ``split_bf16`` / ``merge_bf16`` -- exponent / sign-mantissa split
  (reference ``dfloat11/dfloat11_utils.py:177-178``) and its inverse
  (``dfloat11/decode.cu:207-209``).
* ``encode_py``     -- restatement of the reference bit packer
  (``dfloat11/dfloat11_utils.py:118-170``) for a given code table.
* ``luts_py``       -- restatement of the reference LUT builder
  (``dfloat11/dfloat11_utils.py:68-115``) for a given code table.

Parity status: pinned.  ``tests/golden/*.npz`` hold inputs and outputs of the
reference's own ``get_luts`` / ``encode`` (imported unmodified by
``tests/golden/make_golden.py``); ``tests/test_oracle.py`` checks every function
here against them.  The reference repository itself ships no test vectors.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None

WINDOW_BYTES = 8            # dfloat11.py:45
WINDOWS_PER_BLOCK = 512     # dfloat11.py:46
BLOCK_BYTES = WINDOW_BYTES * WINDOWS_PER_BLOCK


def build(force: bool = False) -> str:
    """Compile ``df11_oracle.c`` into ``liboracle.so`` next to it (gcc, seconds)."""
    src = os.path.join(_HERE, "df11_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B", "liboracle.so"])
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        lib = ctypes.CDLL(_LIB_PATH)
        lib.df11_oracle_decode.restype = ctypes.c_int
        lib.df11_oracle_decode.argtypes = [
            ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int64,
            ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p,
            ctypes.c_int64, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
        ]
        lib.df11_oracle_max_threads.restype = ctypes.c_int
        _lib = lib
    return _lib


def max_threads() -> int:
    return int(_load().df11_oracle_max_threads())


def _u8(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint8, a.dtype
    return a


def decode_c(luts, codes, sign_mantissa, output_positions, gaps, n_threads: int = 1,
             strict: bool = True, out: np.ndarray | None = None) -> np.ndarray:
    """Decode one DF11 unit on the CPU.  Returns the BF16 bit patterns as uint16 (written into
    ``out`` when given, which keeps page faults of a fresh buffer out of a timing)."""
    luts = _u8(luts).reshape(-1, 256)
    codes = _u8(codes)
    sm = _u8(sign_mantissa)
    gaps = _u8(gaps)
    pos = np.ascontiguousarray(output_positions)
    if pos.dtype == np.uint8:       # stored as a byte view on disk (dfloat11.py:596)
        pos = pos.view(np.uint32)
    assert pos.dtype == np.uint32
    if out is None:
        out = np.zeros(sm.size, dtype=np.uint16)
    assert out.dtype == np.uint16 and out.size >= sm.size and out.flags.c_contiguous
    rc = _load().df11_oracle_decode(
        luts.ctypes.data, luts.shape[0], codes.ctypes.data, codes.size,
        sm.ctypes.data, sm.size, pos.ctypes.data, gaps.ctypes.data, gaps.size,
        out.ctypes.data, int(n_threads), int(bool(strict)))
    if rc != 0:
        raise RuntimeError(f"df11_oracle_decode failed with code {rc}")
    return out


def decode_py(luts, codes, sign_mantissa, output_positions, gaps) -> np.ndarray:
    """Pure-Python statement of the decode rule (decode.cu:85-144,181,207-209)."""
    luts = np.asarray(luts, dtype=np.uint8).reshape(-1, 256)
    lens = luts[-1]
    codes = bytes(np.asarray(codes, dtype=np.uint8))
    sm = np.asarray(sign_mantissa, dtype=np.uint8)
    gaps = np.asarray(gaps, dtype=np.uint8)
    pos = np.asarray(output_positions)
    if pos.dtype == np.uint8:
        pos = pos.view(np.uint32)
    n_bytes, n_elements = len(codes), sm.size
    out = np.zeros(n_elements, dtype=np.uint16)
    n_blocks = -(-n_bytes // BLOCK_BYTES)
    gap_bits = np.unpackbits(gaps) if gaps.size else np.zeros(0, np.uint8)
    for b in range(n_blocks):
        o = int(pos[b])
        for t in range(b * WINDOWS_PER_BLOCK, (b + 1) * WINDOWS_PER_BLOCK):
            if t * WINDOW_BYTES >= n_bytes:
                break
            g = gap_bits[5 * t:5 * t + 5]
            p = int(g[0]) * 16 + int(g[1]) * 8 + int(g[2]) * 4 + int(g[3]) * 2 + int(g[4])
            chunk = codes[t * 8:t * 8 + 12].ljust(12, b"\0")
            bits = int.from_bytes(chunk, "big")          # 96 bits, MSB first
            while p < 64:
                x = (bits >> (96 - 32 - p)) & 0xFFFFFFFF
                e = int(luts[0][x >> 24])
                shift = 16
                while e >= 240 and shift >= 0:
                    e = int(luts[256 - e][(x >> shift) & 255])
                    shift -= 8
                if o < n_elements:
                    m = int(sm[o])
                    out[o] = ((m & 0x80) << 8) | (e << 7) | (m & 0x7F)
                o += 1
                ln = int(lens[e])
                if ln == 0:
                    raise RuntimeError("zero code length reached")
                p += ln
        if b + 1 < n_blocks and o != int(pos[b + 1]):
            raise RuntimeError(f"block {b} ended at {o}, expected {int(pos[b + 1])}")
    return out


def split_bf16(w_u16):
    """BF16 bit patterns -> (exponent uint8, sign_mantissa uint8); dfloat11_utils.py:177-178."""
    w = np.asarray(w_u16).view(np.uint16).astype(np.uint32)
    exponent = ((w >> 7) & 0xFF).astype(np.uint8)
    sign_mantissa = (((w >> 8) & 0x80) | (w & 0x7F)).astype(np.uint8)
    return exponent, sign_mantissa


def merge_bf16(exponent, sign_mantissa):
    """Inverse of ``split_bf16``; decode.cu:207-209."""
    e = np.asarray(exponent, dtype=np.uint32)
    m = np.asarray(sign_mantissa, dtype=np.uint32)
    return (((m & 0x80) << 8) | (e << 7) | (m & 0x7F)).astype(np.uint16)


def encode_py(symbols, code_len, code_val, eof_len, eof_val):
    """Bit packer of dfloat11_utils.py:118-170 for an explicit code table.

    ``code_len[s]`` / ``code_val[s]`` give the code of exponent value ``s``.
    Returns (encoded uint8, gaps uint8 (5-bit packed), output_positions uint32).
    """
    window_bits = 8 * WINDOW_BYTES
    block_bits = window_bits * WINDOWS_PER_BLOCK
    big, total = 0, 0
    gaps, positions = [], []
    for i, s in enumerate(symbols):
        if total // window_bits + 1 > len(gaps):
            gaps.append(total % window_bits)
        if total // block_bits + 1 > len(positions):
            positions.append(i)
        big = (big << int(code_len[s])) | int(code_val[s])
        total += int(code_len[s])
    n = len(symbols)
    rem = total % 8
    if rem:
        # the tail byte is completed with the leading bits of the end-of-stream code
        if total // window_bits + 1 > len(gaps):
            gaps.append(total % window_bits)
        if total // block_bits + 1 > len(positions):
            positions.append(n)
        room = 8 - rem
        if eof_len >= room:
            pad = eof_val >> (eof_len - room)
        else:
            pad = eof_val << (room - eof_len)
        big = (big << room) | pad
        total += room
    encoded = np.frombuffer(big.to_bytes(total // 8, "big"), dtype=np.uint8) if total else np.zeros(0, np.uint8)
    positions.append(n)
    n_blocks = -(-encoded.size // BLOCK_BYTES)
    gaps = gaps + [0] * (WINDOWS_PER_BLOCK * n_blocks - len(gaps))
    gap_bits = np.zeros((len(gaps), 5), dtype=np.uint8)
    for k, g in enumerate(gaps):
        for j in range(5):
            gap_bits[k, j] = (g >> (4 - j)) & 1
    return encoded.copy(), np.packbits(gap_bits.reshape(-1)), np.asarray(positions, dtype=np.uint32)


def encode_stream_py(symbols, code_len, code_val, eof_len, eof_val):
    """The same bit packer written the way the reference runs it (dfloat11_utils.py:118-170): one
    Python-level step per symbol, a small bit buffer from which whole bytes are taken as they
    fill up, so the cost is linear in the number of symbols.  ``encode_py`` above keeps the whole
    stream in one integer, which is simple to check but quadratic; this form is what the
    benchmark times as the reference's CPU compression rate.  Same arguments and results."""
    lens = [int(x) for x in code_len]
    vals = [int(x) for x in code_val]
    out = bytearray()
    gaps, positions = [], []
    window_bits = 8 * WINDOW_BYTES
    block_bits = window_bits * WINDOWS_PER_BLOCK
    held, n_held, total = 0, 0, 0
    next_window, next_block = 0, 0            # stream bit at which the next window / block starts
    for i, s in enumerate(symbols):
        if total >= next_window:              # first code that starts in a new window (windows are
            gaps.append(total - next_window)  # never skipped: a code is at most 32 bits, a window 64)
            next_window += window_bits
        if total >= next_block:
            positions.append(i)
            next_block += block_bits
        n = lens[s]
        held = (held << n) | vals[s]
        n_held += n
        total += n
        while n_held >= 8:
            n_held -= 8
            out.append(held >> n_held)
            held &= (1 << n_held) - 1
    n_symbols = len(symbols)
    if n_held:
        if total >= next_window:
            gaps.append(total - next_window)
        if total >= next_block:
            positions.append(n_symbols)
        room = 8 - n_held
        pad = (eof_val >> (eof_len - room)) if eof_len >= room else (eof_val << (room - eof_len))
        out.append(((held << room) | pad) & 0xFF)
    positions.append(n_symbols)
    encoded = np.frombuffer(bytes(out), dtype=np.uint8).copy()
    n_blocks = -(-encoded.size // BLOCK_BYTES)
    g = np.zeros(WINDOWS_PER_BLOCK * n_blocks, dtype=np.uint8)
    g[:len(gaps)] = gaps
    gap_bits = ((g[:, None] >> np.arange(4, -1, -1, dtype=np.uint8)) & 1).astype(np.uint8)
    return encoded, np.packbits(gap_bits.reshape(-1)), np.asarray(positions, dtype=np.uint32)


def luts_py(table):
    """LUT builder of dfloat11_utils.py:68-115 for an explicit code table.

    ``table`` is a sequence of ``(symbol, n_bits, value)`` in the iteration order
    of the reference's code-table dict (that order fixes the numbering of rows of
    equal prefix length, dfloat11_utils.py:71-77); the end-of-stream entry is left
    out, as the reference skips non-int keys (dfloat11_utils.py:72,85,110).

    Row 0 is the root; a row exists for every byte-aligned proper prefix of a
    code; entries < 240 are symbols, entries >= 240 point to row ``256-entry``;
    only the first index of a code's range is set explicitly and later indices
    inherit the previous value (dfloat11_utils.py:103-106); the final row holds
    code lengths.
    """
    table = [(int(s), int(b), int(v)) for s, b, v in table]
    strs = [(s, bin(v)[2:].rjust(b, "0")) for s, b, v in table]
    prefixes = [""]
    for _, c in strs:
        p = c[:((len(c) - 1) // 8) * 8]
        if p not in prefixes:
            prefixes.append(p)
    prefixes.sort(key=len)
    rows = np.zeros((len(prefixes) + 1, 256), dtype=np.uint8)
    for pi, p in enumerate(prefixes):
        level = len(p) // 8
        firsts = {}
        for s, c in strs:
            if not c.startswith(p):
                continue
            if (len(c) - 1) // 8 == level:
                key, val = int(c[level * 8:].ljust(8, "0"), 2), s
            else:
                key, val = int(c[level * 8:level * 8 + 8], 2), 256 - prefixes.index(c[:level * 8 + 8])
            if key in firsts and firsts[key] != val:
                raise ValueError("conflicting LUT entries")
            firsts[key] = val
        cur = None
        for i in range(256):
            if i in firsts:
                cur = firsts[i]
            if cur is None:
                raise ValueError("index 0 of a LUT row is unmapped")
            rows[pi, i] = cur
    for s, b, _ in table:
        rows[-1, s] = b
    return rows
