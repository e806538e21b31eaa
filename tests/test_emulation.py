"""The kernels' algorithm, run on the CPU.

``tests/emul/df11_emul.cpp`` (test-only, never part of libdf11) drives the very same
table builder, window routines and merge arithmetic the CUDA kernels use
(``dfloat11_b200/csrc/df11_common.h``) over plain host arrays, restating only the
block-level flow.  This checks the multi-symbol tables, the ownership rule at window
ends, escapes to the full LUT walk, clamps and the 8-element merge groups against the
reference-made golden vectors on a machine without a GPU.
"""
import ctypes
import os
import subprocess

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "emul", "df11_emul.cpp")
LIB = os.path.join(HERE, "emul", "libdf11_emul.so")


@pytest.fixture(scope="module")
def emul():
    deps = [SRC, os.path.join(HERE, "..", "dfloat11_b200", "csrc", "df11_common.h")]
    if not os.path.exists(LIB) or any(os.path.getmtime(d) > os.path.getmtime(LIB) for d in deps):
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-o", LIB, SRC])
    return ctypes.CDLL(LIB)


def _run(lib, g, K, prepared, cap):
    arrs = [np.ascontiguousarray(g[k]) for k in ("luts", "encoded", "sign_mantissa", "output_positions", "gaps")]
    luts, enc, sm, pos, gaps = arrs
    out = np.full(g["w"].size, 0xABCD, np.uint16)
    status = ctypes.c_int(0)
    vp = lambda a: a.ctypes.data_as(ctypes.c_void_p)  # noqa: E731
    rc = lib.df11_emul_decode(vp(luts), luts.shape[0], vp(enc), ctypes.c_int64(enc.size), vp(sm),
                              ctypes.c_int64(sm.size), vp(pos), vp(gaps), vp(out), K, prepared, cap,
                              ctypes.byref(status))
    return rc, status.value, out


@pytest.mark.parametrize("K", [9, 11, 12, 14])
@pytest.mark.parametrize("prepared", [0, 16, 32])
def test_kernel_algorithm_matches_golden(emul, golden, K, prepared):
    widest = int(np.diff(golden["output_positions"].astype(np.int64)).max())
    for reverse in ((0, 1) if prepared == 0 else (0,)):
        # the windows of a block write their staged exponents word by word next to each other: run the
        # decode pass front to back and back to front, a window that touches a neighbour's bytes shows
        emul.df11_emul_window_order(reverse)
        for cap in (0, widest):
            rc, status, out = _run(emul, golden, K, prepared, cap)
            assert rc == 0 and status == 0
            assert np.array_equal(out, golden["w"]), (reverse, cap)
    emul.df11_emul_window_order(0)


def test_small_staging_is_flagged_not_overrun(emul, golden):
    widest = int(np.diff(golden["output_positions"].astype(np.int64)).max())
    if widest < 64:
        pytest.skip("tiny case")
    rc, status, _ = _run(emul, golden, 11, 0, widest // 2)
    assert rc == 0 and status & 4          # DF11_STATUS_TRUNCATED


def test_table_entries_are_consistent(emul, golden):
    luts = np.ascontiguousarray(golden["luts"])
    lens = luts[-1].astype(np.int64)
    K = 11
    meta = np.zeros(1 << K, np.uint32)
    syms = np.zeros(1 << K, np.uint32)
    cnt = np.zeros(1 << K, np.uint32)
    vp = lambda a: a.ctypes.data_as(ctypes.c_void_p)  # noqa: E731
    assert emul.df11_emul_table(vp(luts), luts.shape[0], K, vp(meta), vp(syms), vp(cnt)) == 0
    for v in range(1 << K):
        m, s, c = int(meta[v]), int(syms[v]), int(cnt[v])
        if m == 1 << 24:                                    # escape
            assert c == 0xFFFF0080
            continue
        n, bits = (m >> 8) & 7, m & 0xFF
        assert 1 <= n <= 4 and (c & 0xFFFF) == (m & 0xFFFF)
        total = 0
        for j in range(n):
            assert ((c >> (16 + 4 * j)) & 15) == total      # start offsets
            assert total < K                                 # every symbol starts inside the index
            total += int(lens[(s >> (8 * j)) & 255])
        assert total == bits
        for j in range(n, 4):
            assert ((c >> (16 + 4 * j)) & 15) == 15


@pytest.mark.parametrize("n", [1, 15, 4097, 100_003])
@pytest.mark.parametrize("case", ["gaussian", "one_bit_codes", "eight_bit_codes", "deep_codes"])
def test_gpu_packer_rules_match_the_host_packer(emul, n, case):
    """The per-element rules of the GPU bit packer (shared arithmetic in df11_common.h, run here
    one element after the other) give the bytes of df11_encode_host, which the golden vectors
    pin to the reference's `encode`."""
    from dfloat11_b200 import codec
    rng = np.random.default_rng(n + len(case))
    if case == "gaussian":
        e = np.clip(np.rint(rng.normal(120, 2.5, size=n)), 1, 239).astype(np.uint8)
    elif case == "one_bit_codes":
        e = ((rng.random(n) < 0.9).astype(np.uint8) * 3 + 100).astype(np.uint8)
    elif case == "eight_bit_codes":
        e = rng.integers(0, 240, size=n).astype(np.uint8)
    else:
        p = 0.5 ** np.arange(1, 41)
        e = rng.choice(np.arange(60, 100), size=n, p=p / p.sum()).astype(np.uint8)
    hist = np.bincount(e, minlength=256)
    if (hist > 0).sum() < 2:
        hist[(int(e[0]) + 1) % 240] += 1
    lens = np.ascontiguousarray(codec.code_lengths(hist), dtype=np.uint8)
    vals = np.ascontiguousarray(codec.canonical_codes(lens), dtype=np.uint32)
    vp = lambda a: a.ctypes.data_as(ctypes.c_void_p)  # noqa: E731
    for pad in ((0, 0), (5, 0b10110), (32, 0xDEADBEEF)):
        enc_h, gaps_h, pos_h = codec.pack_exponents(e, lens, vals, n_threads=2, pad=pad)
        enc = np.full((enc_h.size + 3) // 4 * 4, 0xEE, np.uint8)
        gaps = np.full(gaps_h.size, 0xEE, np.uint8)
        pos = np.full(pos_h.size, 0xEEEEEEEE, np.uint32)
        rc = emul.df11_emul_pack(vp(e), ctypes.c_int64(n), vp(lens), vp(vals), ctypes.c_uint32(pad[0]),
                                 ctypes.c_uint32(pad[1]), vp(enc), ctypes.c_int64(enc_h.size), vp(gaps),
                                 ctypes.c_int64(gaps.size), vp(pos), ctypes.c_int64(pos.size))
        assert rc == 0
        assert np.array_equal(enc[:enc_h.size], enc_h)
        assert np.array_equal(gaps, gaps_h)
        assert np.array_equal(pos, pos_h)
