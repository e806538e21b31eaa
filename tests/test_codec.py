"""Host-side codec: code construction, LUT layout, native bit packer (no GPU needed)."""
import numpy as np
import pytest
import torch

from dfloat11_b200 import _lib, codec
from oracle import df11_oracle as oracle


def _code_arrays(g):
    code_len = np.zeros(256, np.uint8)
    code_val = np.zeros(256, np.uint32)
    code_len[g["table_syms"]] = g["table_bits"]
    code_val[g["table_syms"]] = g["table_vals"].astype(np.uint32)
    return code_len, code_val


@pytest.mark.parametrize("n_threads", [1, 3])
def test_native_packer_is_byte_identical_to_reference(golden, n_threads):
    e, _ = oracle.split_bf16(golden["w"])
    code_len, code_val = _code_arrays(golden)
    enc, gaps, pos = codec.pack_exponents(e, code_len, code_val, n_threads=n_threads,
                                          pad=(int(golden["eof_bits"]), int(golden["eof_val"])))
    assert np.array_equal(enc, golden["encoded"])
    assert np.array_equal(gaps, golden["gaps"])
    assert np.array_equal(pos, golden["output_positions"])


def test_native_packer_threads_agree_on_a_large_unit():
    rng = np.random.default_rng(5)
    w = (torch.randn(1_500_000, generator=torch.Generator().manual_seed(5)) * 0.02).to(torch.bfloat16)
    lens, vals, _ = codec.get_codec(w)
    e, _ = codec.split_bf16(w)
    one = codec.pack_exponents(e.numpy(), lens, vals, n_threads=1)
    many = codec.pack_exponents(e.numpy(), lens, vals, n_threads=7)
    for a, b in zip(one, many):
        assert np.array_equal(a, b)
    # and the single-thread result equals the restated reference packer on a prefix
    small = e.numpy()[:20000]
    ref = oracle.encode_py(small.tolist(), lens, vals, 0, 0)
    got = codec.pack_exponents(small, lens, vals, n_threads=1)
    for a, b in zip(ref, got):
        assert np.array_equal(a, b)
    del rng


def test_luts_match_reference_layout(golden):
    """Same code table -> same LUT rows as the reference builder (via its restatement)."""
    code_len, code_val = _code_arrays(golden)
    mine = codec.build_luts(code_len, code_val)
    ref = golden["luts"]
    # row numbering of equal-length prefixes follows dict order in the reference; compare
    # through decoding instead when the numbering differs
    if mine.shape == ref.shape and np.array_equal(mine, ref):
        return
    e, m = oracle.split_bf16(golden["w"])
    out = oracle.decode_c(mine, golden["encoded"], golden["sign_mantissa"], golden["output_positions"],
                          golden["gaps"])
    assert np.array_equal(out, golden["w"])


def _cases():
    g = torch.Generator().manual_seed(11)
    yield "gauss", [(torch.randn(70000, generator=g) * 0.02).to(torch.bfloat16)]
    yield "three_parts", [(torch.randn(n, generator=g) * 0.02).to(torch.bfloat16) for n in (4096, 1, 30000)]
    yield "one", [(torch.randn(1, generator=g)).to(torch.bfloat16)]
    yield "zeros", [torch.zeros(5000, dtype=torch.bfloat16)]
    yield "wide", [(torch.randn(50000, generator=g) * 7.0).to(torch.bfloat16)]
    rng = np.random.default_rng(3)
    e = rng.integers(0, 240, size=40000).astype(np.uint16)
    sm = rng.integers(0, 256, size=e.size).astype(np.uint16)
    w = (((sm & 0x80) << 8) | (e << 7) | (sm & 0x7F)).astype(np.uint16)
    yield "uniform240", [torch.from_numpy(w.view(np.int16)).view(torch.bfloat16)]
    # geometric exponent frequencies: deep code, several LUT levels, package-merge limit
    p = 0.5 ** np.arange(1, 41)
    e = rng.choice(np.arange(60, 100), size=60000, p=p / p.sum()).astype(np.uint16)
    sm = rng.integers(0, 256, size=e.size).astype(np.uint16)
    w = (((sm & 0x80) << 8) | (e << 7) | (sm & 0x7F)).astype(np.uint16)
    yield "geometric", [torch.from_numpy(w.view(np.int16)).view(torch.bfloat16)]


@pytest.mark.parametrize("name,weights", list(_cases()), ids=[c[0] for c in _cases()])
def test_round_trip_through_oracle(name, weights):
    t = codec.encode_weights(weights, n_threads=2)
    assert t["output_positions"].dtype == torch.uint8 and t["luts"].dtype == torch.uint8
    widest = codec.validate_unit(t["luts"], t["encoded_exponent"], t["sign_mantissa"],
                                 t["output_positions"], t["gaps"])
    assert 0 < widest <= 32768
    out = oracle.decode_c(t["luts"].numpy(), t["encoded_exponent"].numpy(), t["sign_mantissa"].numpy(),
                          t["output_positions"].numpy(), t["gaps"].numpy())
    want = torch.cat([w.reshape(-1) for w in weights]).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(out, want)
    sizes = [w.numel() for w in weights]
    assert t["split_positions"].tolist() == np.cumsum(sizes)[:-1].tolist()


def test_length_limit_binds():
    freq = np.zeros(256, np.int64)
    freq[10:50] = 2 ** np.arange(40)
    lens = codec.code_lengths(freq)
    assert lens.max() == 32 and lens[10:50].min() >= 1
    assert sum(2.0 ** -int(l) for l in lens if l) <= 1.0 + 1e-12
    vals = codec.canonical_codes(lens)
    luts = codec.build_luts(lens, vals)
    assert luts.shape[0] <= 18


def test_exponents_240_and_up_are_rejected():
    w = torch.tensor([float("inf"), 1.0], dtype=torch.bfloat16)
    with pytest.raises(codec.UnrepresentableError):
        codec.encode_weights([w])


def test_validate_rejects_corrupt_units(golden):
    if golden["encoded"].size < 8:
        pytest.skip("too small to corrupt meaningfully")
    luts = torch.from_numpy(golden["luts"].copy())
    enc = torch.from_numpy(golden["encoded"])
    sm = torch.from_numpy(golden["sign_mantissa"])
    pos = torch.from_numpy(golden["output_positions"].view(np.uint8).copy())
    gaps = torch.from_numpy(golden["gaps"])
    assert codec.validate_unit(luts, enc, sm, pos, gaps) == int(np.diff(golden["output_positions"].astype(np.int64)).max())
    bad = luts.clone()
    bad[-1, :] = 0                                   # zero code lengths: the reference kernel never returns
    with pytest.raises(_lib.DF11Error):
        codec.validate_unit(bad, enc, sm, pos, gaps)
    with pytest.raises(_lib.DF11Error):
        codec.validate_unit(luts, enc, sm[:-1], pos, gaps)      # element count disagrees
    with pytest.raises(_lib.DF11Error):
        codec.validate_unit(luts, enc, sm, pos, gaps[:-1])      # gaps truncated
