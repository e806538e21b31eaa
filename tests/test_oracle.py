"""Pins the CPU oracle against tensors produced by the reference's own codec.

Every golden file holds the original BF16 bit patterns and the six DF11 tensors
that the reference's ``get_luts`` / ``encode_weights`` (dfloat11_utils.py) made of
them; the oracle must reproduce the original exactly from those tensors, and
its restated encoder / LUT builder must reproduce the tensors byte for byte.
"""
import numpy as np
import pytest

from oracle import df11_oracle as oracle


def test_decode_c_matches_original(golden):
    out = oracle.decode_c(golden["luts"], golden["encoded"], golden["sign_mantissa"],
                          golden["output_positions"], golden["gaps"])
    assert out.dtype == np.uint16
    assert np.array_equal(out, golden["w"])


def test_decode_c_threads_and_byte_view(golden):
    pos_bytes = golden["output_positions"].view(np.uint8)   # on-disk form, dfloat11.py:596
    out = oracle.decode_c(golden["luts"], golden["encoded"], golden["sign_mantissa"],
                          pos_bytes, golden["gaps"], n_threads=4)
    assert np.array_equal(out, golden["w"])


def test_decode_py_matches_original(golden):
    if golden["w"].size > 32000:
        pytest.skip("pure-Python loop is kept to small cases")
    out = oracle.decode_py(golden["luts"], golden["encoded"], golden["sign_mantissa"],
                           golden["output_positions"], golden["gaps"])
    assert np.array_equal(out, golden["w"])


def test_split_merge(golden):
    e, m = oracle.split_bf16(golden["w"])
    assert np.array_equal(m, golden["sign_mantissa"])
    assert np.array_equal(oracle.merge_bf16(e, m), golden["w"])


def _tables(g):
    code_len = np.zeros(256, np.int64)
    code_val = np.zeros(256, np.uint64)
    code_len[g["table_syms"]] = g["table_bits"]
    code_val[g["table_syms"]] = g["table_vals"]
    return code_len, code_val


def test_encode_py_matches_reference(golden):
    e, _ = oracle.split_bf16(golden["w"])
    code_len, code_val = _tables(golden)
    enc, gaps, pos = oracle.encode_py(e.tolist(), code_len, code_val,
                                      int(golden["eof_bits"]), int(golden["eof_val"]))
    assert np.array_equal(enc, golden["encoded"])
    assert np.array_equal(gaps, golden["gaps"])
    assert np.array_equal(pos, golden["output_positions"])


def test_encode_stream_py_matches_reference(golden):
    """The linear-time restatement (what the benchmark times as the CPU compression rate)."""
    e, _ = oracle.split_bf16(golden["w"])
    code_len, code_val = _tables(golden)
    enc, gaps, pos = oracle.encode_stream_py(e.tolist(), code_len, code_val,
                                             int(golden["eof_bits"]), int(golden["eof_val"]))
    assert np.array_equal(enc, golden["encoded"])
    assert np.array_equal(gaps, golden["gaps"])
    assert np.array_equal(pos, golden["output_positions"])


def test_luts_py_matches_reference(golden):
    table = list(zip(golden["table_syms"].tolist(), golden["table_bits"].tolist(),
                     golden["table_vals"].tolist()))
    assert np.array_equal(oracle.luts_py(table), golden["luts"])


def test_oracle_reports_zero_length():
    g = __import__("tests.conftest", fromlist=["load_golden"]).load_golden("gauss_n3")
    luts = g["luts"].copy()
    luts[-1, :] = 0          # the reference kernel would spin forever here (decode.cu:116-118)
    with pytest.raises(RuntimeError):
        oracle.decode_c(luts, g["encoded"], g["sign_mantissa"], g["output_positions"], g["gaps"])
    with pytest.raises(RuntimeError):
        oracle.decode_py(luts, g["encoded"], g["sign_mantissa"], g["output_positions"], g["gaps"])


def test_golden_set_is_complete():
    from tests.conftest import golden_names
    names = set(golden_names())
    for want in ("gauss_multi", "gauss_n1", "gauss_n3", "gauss_wide", "two_exponents", "uniform_240",
                 "long_codes", "deep_codes", "byte_aligned_end", "block_aligned_end",
                 "window_aligned_plus2", "all_zero", "single_exponent"):
        assert want in names
