"""df11_decode_static: the decode entry point that allocates nothing.

Some callers of libdf11 cannot allocate device memory and cannot ask anyone else to: code
inside a CUDA-graph capture or a stream callback, or a plug-in in a serving process whose
memory was handed out at start-up.  For them the library carries its own fixed auxiliary
buffer.  This test calls that entry point through the C ABI, twice in a row on different
units (the second call finds the first call's contents in the shared buffer), and compares
every result bit for bit with the ordinary entry point's.  It also checks that a unit over
the stated size limit is refused.  It sits in a file of its own, collected last.
"""
import numpy as np
import pytest
import torch

from dfloat11_b200 import _lib, codec, ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _unit(n, seed, std=0.02):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(n, generator=g) * std).to(torch.bfloat16)
    t = codec.encode_weights([w])
    d = {k: v.to(DEV) for k, v in t.items() if k != "split_positions"}
    return w, d


def _decode_static(d, n, status):
    out = torch.full((n,), -1.0, dtype=torch.bfloat16, device=DEV)
    stream = torch.cuda.current_stream(torch.device(DEV)).cuda_stream
    rc = _lib.lib.df11_decode_static(
        d["luts"].data_ptr(), d["encoded_exponent"].data_ptr(), d["sign_mantissa"].data_ptr(),
        d["output_positions"].data_ptr(), d["gaps"].data_ptr(), out.data_ptr(),
        d["luts"].shape[0], d["encoded_exponent"].numel(), n, status.data_ptr(), 0, stream)
    _lib.check(rc)
    return out


def test_static_entry_point_matches_the_ordinary_one_twice_in_a_row():
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # two different units, the larger first: the second call meets stale seek points beyond its own
    for n, seed, std in ((3_000_017, 21, 0.02), (1_234_567, 22, 1.0)):
        w, d = _unit(n, seed, std)
        want = ops.decode(d["luts"], d["encoded_exponent"], d["sign_mantissa"], d["output_positions"], d["gaps"],
                          status=status)
        got = _decode_static(d, n, status)
        torch.cuda.synchronize()
        assert status.item() == 0
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))          # tolerance: none, bit-exact
        assert torch.equal(got.cpu().view(torch.int16), w.view(torch.int16))
    # and once more on the first size, back to back on the same stream without a sync in between
    w, d = _unit(3_000_017, 23)
    a = _decode_static(d, w.numel(), status)
    b = _decode_static(d, w.numel(), status)
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert torch.equal(a.cpu().view(torch.int16), w.view(torch.int16))


def test_static_entry_point_refuses_units_over_its_limit():
    w, d = _unit(4096, 24)
    out = torch.empty(8, dtype=torch.bfloat16, device=DEV)
    rc = _lib.lib.df11_decode_static(
        d["luts"].data_ptr(), d["encoded_exponent"].data_ptr(), d["sign_mantissa"].data_ptr(),
        d["output_positions"].data_ptr(), d["gaps"].data_ptr(), out.data_ptr(),
        d["luts"].shape[0], d["encoded_exponent"].numel(), (1 << 25) + 1, None, 0, None)
    assert rc == _lib.DF11_ERR_NOSPACE
    assert b"up to" in _lib.lib.df11_last_error()
