"""GPU parity tests of the decode kernels, called through the C ABI of libdf11.so.

Bar: bit-exact.  Checked against (1) the original BF16 tensors, (2) the CPU oracle,
(3) tensors produced by the reference's own encoder (tests/golden), and (4) the reference's
own kernel run on the same GPU on identical inputs.
"""
import numpy as np
import pytest
import torch

from dfloat11_b200 import _lib, codec, ops
from oracle import df11_oracle as oracle
from oracle import ref_kernel

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _to_dev(g):
    return dict(
        luts=torch.from_numpy(np.ascontiguousarray(g["luts"])).to(DEV),
        enc=torch.from_numpy(np.ascontiguousarray(g["encoded"])).to(DEV),
        sm=torch.from_numpy(np.ascontiguousarray(g["sign_mantissa"])).to(DEV),
        pos=torch.from_numpy(np.ascontiguousarray(g["output_positions"]).view(np.uint8).copy()).to(DEV),
        gaps=torch.from_numpy(np.ascontiguousarray(g["gaps"])).to(DEV),
    )


def _bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def _status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def _widest(pos_u32):
    return int(np.diff(np.asarray(pos_u32).astype(np.int64)).max())


@pytest.fixture(params=[16, 32])
def seek(request):
    """Runs a test of the prepared form once per seek interval (a process-wide setting)."""
    before = ops.seek_interval()
    ops.seek_interval(request.param)
    yield request.param
    ops.seek_interval(before)


def _unit_from_weights(weights, n_threads=None):
    t = codec.encode_weights(weights, n_threads=n_threads)
    d = dict(luts=t["luts"].to(DEV), enc=t["encoded_exponent"].to(DEV), sm=t["sign_mantissa"].to(DEV),
             pos=t["output_positions"].to(DEV), gaps=t["gaps"].to(DEV))
    widest = _widest(t["output_positions"].numpy().view(np.uint32))
    return t, d, widest


@pytest.mark.parametrize("exact_cap", [False, True])
def test_golden_two_pass(golden, exact_cap):
    d = _to_dev(golden)
    st = _status()
    cap = _widest(golden["output_positions"]) if exact_cap else 0
    out = torch.full((golden["w"].size,), -1.0, dtype=torch.bfloat16, device=DEV)
    ops.decode(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"], out=out, max_block_elems=cap, status=st)
    torch.cuda.synchronize()
    assert st.item() == 0
    assert np.array_equal(_bits(out), golden["w"])
    want = oracle.decode_c(golden["luts"], golden["encoded"], golden["sign_mantissa"],
                           golden["output_positions"], golden["gaps"])
    assert np.array_equal(_bits(out), want)


def test_golden_prepared(golden, seek):
    d = _to_dev(golden)
    st = _status()
    aux = ops.prepare(d["luts"], d["enc"], d["pos"], d["gaps"], golden["w"].size, status=st)
    assert aux.numel() == ops.aux_bytes(d["enc"].numel(), golden["w"].size)
    for _ in range(2):   # the auxiliary buffer is reusable
        out = torch.full((golden["w"].size,), -1.0, dtype=torch.bfloat16, device=DEV)
        ops.decode_prepared(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"], aux, out=out,
                            max_block_elems=_widest(golden["output_positions"]), status=st)
        torch.cuda.synchronize()
        assert st.item() == 0
        assert np.array_equal(_bits(out), golden["w"])


@pytest.mark.parametrize("variant", ["shipped_ptx", "recompiled_sm100a"])
def test_same_bits_as_reference_kernel(golden, variant):
    if not ref_kernel.available(variant):
        pytest.skip("reference kernel artefact not built (make -C oracle ref)")
    d = _to_dev(golden)
    smem = ref_kernel.shared_mem_size(golden["output_positions"])
    ref_out = torch.zeros(golden["w"].size, dtype=torch.bfloat16, device=DEV)
    ref_kernel.decode(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"], ref_out, smem, variant=variant)
    out = ops.decode(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"])
    torch.cuda.synchronize()
    assert np.array_equal(_bits(ref_out), golden["w"])
    assert torch.equal(out.view(torch.int16), ref_out.view(torch.int16))


def _scaled_llama_block(hidden, inter, kv, seed):
    g = torch.Generator().manual_seed(seed)
    shapes = [(hidden, hidden), (kv, hidden), (kv, hidden), (hidden, hidden),
              (inter, hidden), (inter, hidden), (hidden, inter)]
    return [(torch.randn(s, generator=g) * 0.02).to(torch.bfloat16) for s in shapes]


def test_llama_block_small_vs_oracle_and_reference():
    weights = _scaled_llama_block(512, 1792, 128, seed=0)       # 3.8 M elements, ~300 format blocks
    t, d, widest = _unit_from_weights(weights)
    want = torch.cat([w.reshape(-1) for w in weights])
    st = _status()
    out = ops.decode(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"], max_block_elems=widest, status=st)
    aux = ops.prepare(d["luts"], d["enc"], d["pos"], d["gaps"], want.numel(), status=st)
    out2 = ops.decode_prepared(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"], aux,
                               max_block_elems=widest, status=st)
    torch.cuda.synchronize()
    assert st.item() == 0
    assert torch.equal(out.cpu().view(torch.int16), want.view(torch.int16))
    assert torch.equal(out2.cpu().view(torch.int16), want.view(torch.int16))
    cpu = oracle.decode_c(t["luts"].numpy(), t["encoded_exponent"].numpy(), t["sign_mantissa"].numpy(),
                          t["output_positions"].numpy(), t["gaps"].numpy(), n_threads=4)
    assert np.array_equal(_bits(out), cpu)
    if ref_kernel.available():
        ref_out = torch.zeros_like(out)
        ref_kernel.decode(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"], ref_out,
                          512 * 4 + 4 + 2 * widest)
        torch.cuda.synchronize()
        assert torch.equal(ref_out.view(torch.int16), out.view(torch.int16))


def test_llama_block_full_size_round_trip():
    """One whole Llama-3.1-8B block (the seven matrices of hidden 4096 / 8 kv heads / intermediate 14336
    as one unit: 218 103 808 elements, N(0, 0.02), seed 0)."""
    weights = _scaled_llama_block(4096, 14336, 1024, seed=0)
    t, d, widest = _unit_from_weights(weights)
    want = torch.cat([w.reshape(-1) for w in weights]).to(DEV)
    assert want.numel() == 218_103_808
    st = _status()
    out = ops.decode(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"], max_block_elems=widest, status=st)
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    out.zero_()
    aux = ops.prepare(d["luts"], d["enc"], d["pos"], d["gaps"], want.numel(), status=st)
    ops.decode_prepared(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"], aux, out=out,
                        max_block_elems=widest, status=st)
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    assert st.item() == 0
    # the views the hook hands to the Linear layers are plain slices of the decoded buffer
    parts = torch.tensor_split(out, t["split_positions"].tolist())
    for p, w in zip(parts, weights):
        assert p.numel() == w.numel()
    # checksum-of-checksums against the original (size-independent property)
    assert int(out.view(torch.int16).to(torch.int64).sum().item()) == \
        int(want.view(torch.int16).to(torch.int64).sum().item())


def test_misaligned_pointers_take_the_slow_paths(golden):
    if golden["w"].size < 64:
        pytest.skip("tiny case")
    d = _to_dev(golden)

    def shifted(t, k):
        buf = torch.empty(t.numel() + 32, dtype=torch.uint8, device=DEV)
        view = buf[k:k + t.numel()]
        view.copy_(t)
        return view

    enc = shifted(d["enc"], 3)
    sm = shifted(d["sm"], 5)
    out_buf = torch.zeros(golden["w"].size + 8, dtype=torch.bfloat16, device=DEV)
    out = out_buf[1:1 + golden["w"].size]          # 2-byte aligned only
    st = _status()
    ops.decode(d["luts"], enc, sm, d["pos"], d["gaps"], out=out, status=st)
    torch.cuda.synchronize()
    assert st.item() == 0
    assert np.array_equal(_bits(out.contiguous()), golden["w"])
    assert out_buf[0].item() == 0 and out_buf[1 + golden["w"].size].item() == 0
    # the prepared form on the same misaligned tensors
    out_buf.zero_()
    aux = ops.prepare(d["luts"], enc, d["pos"], d["gaps"], golden["w"].size, status=st)
    ops.decode_prepared(d["luts"], enc, sm, d["pos"], d["gaps"], aux, out=out, status=st)
    torch.cuda.synchronize()
    assert st.item() == 0
    assert np.array_equal(_bits(out.contiguous()), golden["w"])
    assert out_buf[0].item() == 0 and out_buf[1 + golden["w"].size].item() == 0


def test_output_is_written_only_inside_the_unit(golden):
    d = _to_dev(golden)
    n = golden["w"].size
    buf = torch.full((n + 64,), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.decode(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"], out=buf[:n])
    torch.cuda.synchronize()
    assert torch.all(buf[n:] == 7.0)
    assert np.array_equal(_bits(buf[:n].contiguous()), golden["w"])


def test_runs_on_a_side_stream(golden):
    d = _to_dev(golden)
    s = torch.cuda.Stream(device=DEV)
    torch.cuda.synchronize()
    with torch.cuda.stream(s):
        out = ops.decode(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"])
    s.synchronize()
    assert np.array_equal(_bits(out), golden["w"])


def test_corrupt_units_set_status_and_return():
    from tests.conftest import load_golden
    g = load_golden("gauss_multi")
    d = _to_dev(g)
    n = g["w"].size
    # 1. zero code lengths: the reference kernel would never terminate (decode.cu:116-118)
    luts = d["luts"].clone()
    luts[-1, :] = 0
    st = _status()
    ops.decode(luts, d["enc"], d["sm"], d["pos"], d["gaps"], status=st)
    torch.cuda.synchronize()
    assert st.item() & _lib.STATUS_BAD_TABLE
    # 2. staging smaller than a block: flagged, no out-of-bounds write
    st = _status()
    buf = torch.full((n + 64,), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.decode(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"], out=buf[:n], max_block_elems=1000, status=st)
    torch.cuda.synchronize()
    assert st.item() & _lib.STATUS_TRUNCATED
    assert torch.all(buf[n:] == 7.0)
    # 3. output positions running backwards / past the end
    pos = g["output_positions"].copy()
    pos[1], pos[2] = pos[2], pos[1]
    pos[-1] = n + 100000
    st = _status()
    buf = torch.full((n + 64,), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.decode(d["luts"], d["enc"], d["sm"], torch.from_numpy(pos.view(np.uint8).copy()).to(DEV), d["gaps"],
               out=buf[:n], status=st)
    torch.cuda.synchronize()
    assert st.item() & _lib.STATUS_BAD_POSITIONS
    assert torch.all(buf[n:] == 7.0)
    # 4. random bytes as a stream: terminates, stays in bounds
    st = _status()
    noise = torch.randint(0, 256, (d["enc"].numel(),), dtype=torch.uint8, device=DEV)
    buf = torch.full((n + 64,), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.decode(d["luts"], noise, d["sm"], d["pos"], d["gaps"], out=buf[:n], status=st)
    torch.cuda.synchronize()
    assert torch.all(buf[n:] == 7.0)


def test_argument_errors_raise():
    from tests.conftest import load_golden
    d = _to_dev(load_golden("gauss_n3"))
    with pytest.raises(RuntimeError):
        ops.decode(d["luts"].cpu(), d["enc"], d["sm"], d["pos"], d["gaps"])
    with pytest.raises(_lib.DF11Error):
        ops.decode(d["luts"][:1], d["enc"], d["sm"], d["pos"], d["gaps"])       # n_luts = 1
    with pytest.raises(RuntimeError):
        ops.decode(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"],
                   out=torch.empty(1, dtype=torch.bfloat16, device=DEV))           # too small


@pytest.mark.parametrize("case", ["one_bit_codes", "eight_bit_codes", "deep_codes", "single_symbol"])
def test_synthetic_distributions(case):
    rng = np.random.default_rng(17)
    n = 700_000
    if case == "one_bit_codes":
        e = (rng.random(n) < 0.9).astype(np.uint16) * 3 + 100         # 90 % one symbol
    elif case == "eight_bit_codes":
        e = rng.integers(0, 240, size=n).astype(np.uint16)
    elif case == "deep_codes":
        p = 0.5 ** np.arange(1, 41)
        e = rng.choice(np.arange(60, 100), size=n, p=p / p.sum()).astype(np.uint16)
    else:
        e = np.full(n, 127, dtype=np.uint16)
    sm = rng.integers(0, 256, size=n).astype(np.uint16)
    w = (((sm & 0x80) << 8) | (e << 7) | (sm & 0x7F)).astype(np.uint16)
    weight = torch.from_numpy(w.view(np.int16)).view(torch.bfloat16)
    t, d, widest = _unit_from_weights([weight])
    st = _status()
    out = ops.decode(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"], max_block_elems=widest, status=st)
    aux = ops.prepare(d["luts"], d["enc"], d["pos"], d["gaps"], n, status=st)
    out2 = ops.decode_prepared(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"], aux, max_block_elems=widest,
                               status=st)
    torch.cuda.synchronize()
    assert st.item() == 0
    assert np.array_equal(_bits(out), w)
    assert np.array_equal(_bits(out2), w)


def test_row_wise_decode_matches_rows_of_the_full_decode(seek):
    g = torch.Generator().manual_seed(31)
    table = torch.randn(300, 1024, generator=g).to(torch.bfloat16)          # rows of two 512-element chunks
    t, d, widest = _unit_from_weights([table.flatten()])
    st = _status()
    aux = ops.prepare(d["luts"], d["enc"], d["pos"], d["gaps"], table.numel(), status=st)
    rows = torch.tensor([299, 0, 7, 7, 150, 298, 1], dtype=torch.int64, device=DEV)
    got = ops.decode_rows_prepared(d["luts"], d["enc"], d["sm"], aux, rows, 1024, status=st)
    torch.cuda.synchronize()
    assert st.item() == 0
    assert torch.equal(got.cpu().view(torch.int16), table[rows.cpu()].view(torch.int16))
    # an index outside the table is flagged and decodes row 0 instead of reading elsewhere
    bad = torch.tensor([5, 300, -1], dtype=torch.int64, device=DEV)
    got = ops.decode_rows_prepared(d["luts"], d["enc"], d["sm"], aux, bad, 1024, status=st)
    torch.cuda.synchronize()
    assert st.item() & _lib.STATUS_BAD_POSITIONS
    assert torch.equal(got[0].cpu().view(torch.int16), table[5].view(torch.int16))
    assert torch.equal(got[1].cpu().view(torch.int16), table[0].view(torch.int16))
    with pytest.raises(_lib.DF11Error):
        ops.decode_rows_prepared(d["luts"], d["enc"], d["sm"], aux, rows, 1000)      # not a multiple of 512


@pytest.mark.parametrize("n", [1025, 1536, 1537, 2048, 2049, 2560, 5000, 16 * 4096 + 3])
@pytest.mark.parametrize("case", ["one_bit_codes", "gaussian"])
def test_prepared_decode_around_the_last_chunks(n, case, seek):
    """Units of three and more 512-element chunks: all but the last two take the decoder's
    unchecked inner loop, the last two its general loop; both must give the oracle's bits."""
    rng = np.random.default_rng(n)
    if case == "one_bit_codes":
        e = (rng.random(n) < 0.97).astype(np.uint16) * 5 + 90
    else:
        e = np.clip(np.rint(rng.normal(120, 2.5, size=n)), 1, 239).astype(np.uint16)
    sm = rng.integers(0, 256, size=n).astype(np.uint16)
    w = (((sm & 0x80) << 8) | (e << 7) | (sm & 0x7F)).astype(np.uint16)
    t, d, widest = _unit_from_weights([torch.from_numpy(w.view(np.int16)).view(torch.bfloat16)])
    want = oracle.decode_c(t["luts"].numpy(), t["encoded_exponent"].numpy(), t["sign_mantissa"].numpy(),
                           t["output_positions"].numpy(), t["gaps"].numpy())
    st = _status()
    aux = ops.prepare(d["luts"], d["enc"], d["pos"], d["gaps"], n, status=st)
    buf = torch.full((n + 64,), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.decode_prepared(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"], aux, out=buf[:n], status=st)
    torch.cuda.synchronize()
    assert st.item() == 0
    assert np.array_equal(_bits(buf[:n]), want)
    assert np.array_equal(want, w)
    assert torch.all(buf[n:] == 7.0)


def test_prepared_decode_of_inconsistent_inputs_stays_in_bounds(seek):
    """A stream of random bytes, and seek points that belong to another stream: the output is
    meaningless, but every read and write stays inside the tensors and the launch returns."""
    rng = np.random.default_rng(5)
    n = 300_000
    e = np.clip(np.rint(rng.normal(120, 2.5, size=n)), 1, 239).astype(np.uint16)
    sm = rng.integers(0, 256, size=n).astype(np.uint16)
    w = (((sm & 0x80) << 8) | (e << 7) | (sm & 0x7F)).astype(np.uint16)
    t, d, widest = _unit_from_weights([torch.from_numpy(w.view(np.int16)).view(torch.bfloat16)])
    good_aux = ops.prepare(d["luts"], d["enc"], d["pos"], d["gaps"], n)
    noise = torch.randint(0, 256, (d["enc"].numel(),), dtype=torch.uint8, device=DEV)
    st = _status()
    for stream, aux in ((noise, good_aux),
                        (noise, ops.prepare(d["luts"], noise, d["pos"], d["gaps"], n, status=st)),
                        (d["enc"], torch.randint(0, 256, (good_aux.numel(),), dtype=torch.uint8, device=DEV))):
        aux = aux.clone()
        aux[:32768] = good_aux[:32768]                       # the decode table stays a valid one
        buf = torch.full((n + 64,), 7.0, dtype=torch.bfloat16, device=DEV)
        ops.decode_prepared(d["luts"], stream, d["sm"], d["pos"], d["gaps"], aux, out=buf[:n], status=st)
        torch.cuda.synchronize()
        assert torch.all(buf[n:] == 7.0)


@pytest.mark.parametrize("case", ["one_bit_codes", "gaussian", "deep_codes"])
def test_range_decode_gives_the_same_bits_as_the_whole_decode(case, seek):
    """df11_decode_range_prepared: any run of whole chunks (and a run that ends with the unit's
    ragged tail) equals the same elements of the whole-unit decode; nothing is written past it."""
    n = 700 * 1024 + 37
    rng = np.random.default_rng(len(case))
    if case == "one_bit_codes":
        e = (rng.random(n) < 0.97).astype(np.uint16) * 5 + 90
    elif case == "gaussian":
        e = np.clip(np.rint(rng.normal(120, 2.5, size=n)), 1, 239).astype(np.uint16)
    else:
        p = 0.5 ** np.arange(1, 41)
        e = rng.choice(np.arange(60, 100), size=n, p=p / p.sum()).astype(np.uint16)
    sm = rng.integers(0, 256, size=n).astype(np.uint16)
    w = (((sm & 0x80) << 8) | (e << 7) | (sm & 0x7F)).astype(np.uint16)
    t, d, widest = _unit_from_weights([torch.from_numpy(w.view(np.int16)).view(torch.bfloat16)])
    st = _status()
    aux = ops.prepare(d["luts"], d["enc"], d["pos"], d["gaps"], n, status=st)
    ce = ops.chunk_elements()
    assert ce == 32 * seek
    n_chunks = -(-n // ce)
    for first_chunk, chunks in ((0, 1), (0, n_chunks), (3, 200), (n_chunks - 3, 3), (n_chunks - 1, 1),
                                (n_chunks - 40, 38), (1, n_chunks - 3)):
        first = first_chunk * ce
        count = min(n, (first_chunk + chunks) * ce) - first
        buf = torch.full((count + 64,), 7.0, dtype=torch.bfloat16, device=DEV)
        got = ops.decode_range_prepared(d["luts"], d["enc"], d["sm"], aux, first, count, out=buf, status=st)
        torch.cuda.synchronize()
        assert st.item() == 0
        assert np.array_equal(_bits(got), w[first:first + count]), (first_chunk, chunks)
        assert torch.all(buf[count:] == 7.0)
    for first, count in ((5, ce), (0, ce + 1), (ce, n), (-ce, ce)):          # not on chunk boundaries / outside
        with pytest.raises(_lib.DF11Error):
            ops.decode_range_prepared(d["luts"], d["enc"], d["sm"], aux, first, count,
                                      out=torch.empty(n + ce, dtype=torch.bfloat16, device=DEV))


def test_a_wait_that_runs_out_sets_the_status_and_the_kernel_returns():
    """The bounded waits of the self-contained decoder: one format block's input copy is
    announced but never issued (nothing is in flight, nothing can fault), so the CTA that owns
    the block gives up after a few milliseconds, reports DF11_STATUS_TIMEOUT and returns.  The
    context stays usable: the same unit decodes bit-exactly right afterwards."""
    g = torch.Generator().manual_seed(77)
    w = (torch.randn(900_000, generator=g) * 0.02).to(torch.bfloat16)
    t, d, widest = _unit_from_weights([w])
    n_blocks = -(-d["enc"].numel() // 4096)
    assert n_blocks > 40
    st = _status()
    out = torch.zeros(w.numel(), dtype=torch.bfloat16, device=DEV)
    stream = torch.cuda.current_stream(torch.device(DEV)).cuda_stream
    rc = _lib.lib.df11_selftest_wait_timeout(
        d["luts"].data_ptr(), d["enc"].data_ptr(), d["sm"].data_ptr(), d["pos"].data_ptr(), d["gaps"].data_ptr(),
        out.data_ptr(), d["luts"].shape[0], d["enc"].numel(), w.numel(), widest, 17, st.data_ptr(), 0, stream)
    assert rc == _lib.DF11_OK
    torch.cuda.synchronize()
    assert st.item() & _lib.STATUS_TIMEOUT
    pos = t["output_positions"].numpy().view(np.uint32)
    # blocks of other CTAs are decoded as usual (one CTA per block at this size)
    assert torch.equal(out[:pos[17]].cpu().view(torch.int16), w[:pos[17]].view(torch.int16))
    assert torch.equal(out[pos[18]:].cpu().view(torch.int16), w[pos[18]:].view(torch.int16))
    st.zero_()
    again = ops.decode(d["luts"], d["enc"], d["sm"], d["pos"], d["gaps"], max_block_elems=widest, status=st)
    torch.cuda.synchronize()
    assert st.item() == 0 and torch.equal(again.cpu().view(torch.int16), w.view(torch.int16))
    assert _lib.lib.df11_selftest_wait_timeout(
        d["luts"].data_ptr(), d["enc"].data_ptr(), d["sm"].data_ptr(), d["pos"].data_ptr(), d["gaps"].data_ptr(),
        out.data_ptr(), d["luts"].shape[0], d["enc"].numel(), w.numel(), widest, n_blocks, st.data_ptr(), 0,
        stream) == _lib.DF11_ERR_BADARG


@pytest.mark.parametrize("m", [1, 2, 3, 4])
def test_fused_matrix_vector_product(m, seek):
    """df11_gemv_prepared against an fp32 product with the decoded weights: one BF16 rounding of
    the exact-product, fp32-accumulated sum (tolerance: one BF16 unit in the last place of the
    result plus fp32 accumulation noise), for two matrices inside one unit, with and without
    bias, including the unit's last chunks; reproducible bit for bit."""
    g = torch.Generator().manual_seed(40 + m)
    a = (torch.randn(1536, 2048, generator=g) * 0.02).to(torch.bfloat16)
    b = (torch.randn(520, 1024, generator=g) * 0.02).to(torch.bfloat16)          # ends the unit
    t, d, widest = _unit_from_weights([a.flatten(), b.flatten()])
    n = a.numel() + b.numel()
    st = _status()
    aux = ops.prepare(d["luts"], d["enc"], d["pos"], d["gaps"], n, status=st)
    for w, first, bias in ((a, 0, None), (b, a.numel(), (torch.randn(520, generator=g) * 0.1).to(torch.bfloat16))):
        x = torch.randn(m, w.shape[1], generator=g).to(torch.bfloat16).to(DEV)
        bias_d = bias.to(DEV) if bias is not None else None
        y = ops.gemv_prepared(d["luts"], d["enc"], d["sm"], aux, x, first, w.shape[0], w.shape[1], bias=bias_d, status=st)
        y2 = ops.gemv_prepared(d["luts"], d["enc"], d["sm"], aux, x, first, w.shape[0], w.shape[1], bias=bias_d, status=st)
        torch.cuda.synchronize()
        assert st.item() == 0
        want = x.double().cpu() @ w.double().T + (bias.double() if bias is not None else 0.0)
        err = (y.double().cpu() - want).abs()
        assert torch.all(err <= want.abs() * 2.0 ** -8 + 1e-5), float(err.max())
        assert torch.equal(y.view(torch.int16), y2.view(torch.int16))
        assert y.shape == (m, w.shape[0])
    with pytest.raises(_lib.DF11Error):
        ops.gemv_prepared(d["luts"], d["enc"], d["sm"], aux, x[:, :1000].contiguous(), 0, 16, 1000)   # not a multiple of 512


@pytest.mark.parametrize("rows,in_features", [(10656, 1024), (7104, 2048), (4096, 4096), (9472, 2048), (4736, 8192)])
def test_fused_product_with_longer_runs(rows, in_features, seek):
    """Shapes that make the fused kernel choose its different work splits (on a 148-SM part with
    32 resident warps per SM: single chunks; runs of 2 of a row's 4 chunks plus the adding-up
    kernel; one whole row per warp on a shrunk grid; whole rows in two full rounds; runs of 8 of
    a row's 16 chunks plus the adding-up kernel); same tolerance as above, two activation
    vectors, with bias."""
    g = torch.Generator().manual_seed(rows)
    w = (torch.randn(rows, in_features, generator=g) * 0.02).to(torch.bfloat16)
    pad = (torch.randn(3000, generator=g) * 0.02).to(torch.bfloat16)        # the matrix does not end the unit
    t, d, widest = _unit_from_weights([w.flatten(), pad])
    st = _status()
    aux = ops.prepare(d["luts"], d["enc"], d["pos"], d["gaps"], w.numel() + pad.numel(), status=st)
    x = torch.randn(2, in_features, generator=g).to(torch.bfloat16).to(DEV)
    bias = (torch.randn(rows, generator=g) * 0.1).to(torch.bfloat16)
    y = ops.gemv_prepared(d["luts"], d["enc"], d["sm"], aux, x, 0, rows, in_features, bias=bias.to(DEV), status=st)
    y2 = ops.gemv_prepared(d["luts"], d["enc"], d["sm"], aux, x, 0, rows, in_features, bias=bias.to(DEV), status=st)
    torch.cuda.synchronize()
    assert st.item() == 0
    want = x.double().cpu() @ w.double().T + bias.double()
    err = (y.double().cpu() - want).abs()
    assert torch.all(err <= want.abs() * 2.0 ** -8 + 1e-5), float(err.max())
    assert torch.equal(y.view(torch.int16), y2.view(torch.int16))


@pytest.mark.parametrize("n", [1, 15, 4095, 4096, 4097, 100_003, (1 << 20) + 5])
@pytest.mark.parametrize("case", ["gaussian", "one_bit_codes", "eight_bit_codes", "deep_codes"])
def test_gpu_bit_packer_is_byte_identical_to_the_host_packer(n, case):
    """df11_encode_device_* against df11_encode_host (itself pinned to the reference's `encode`
    by the CPU tests): stream, gaps and output positions, with and without a padding code."""
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
    if (hist > 0).sum() < 2:                                   # a one-symbol alphabet still needs a code
        hist[(int(e[0]) + 1) % 240] += 1
    lens = codec.code_lengths(hist)
    vals = codec.canonical_codes(lens)
    for pad in ((0, 0), (5, 0b10110), (2, 3), (32, 0xDEADBEEF)):
        enc_h, gaps_h, pos_h = codec.pack_exponents(e, lens, vals, n_threads=3, pad=pad)
        enc_d, gaps_d, pos_d = codec.pack_exponents_gpu(torch.from_numpy(e).to(DEV), lens, vals, pad=pad)
        assert np.array_equal(enc_d.cpu().numpy(), enc_h)
        assert np.array_equal(gaps_d.cpu().numpy(), gaps_h)
        assert np.array_equal(pos_d.cpu().numpy().view(np.uint32), pos_h)


def test_encode_weights_on_the_gpu_round_trips():
    g = torch.Generator().manual_seed(77)
    w = (torch.randn(700_001, generator=g) * 0.02).to(torch.bfloat16)
    on_host = codec.encode_weights([w])
    on_gpu = codec.encode_weights([w.to(DEV)])
    for k in on_host:
        assert torch.equal(on_host[k], on_gpu[k]), k
    d = {k: v.to(DEV) for k, v in on_gpu.items() if k != "split_positions"}
    out = ops.decode(d["luts"], d["encoded_exponent"], d["sign_mantissa"], d["output_positions"], d["gaps"])
    assert torch.equal(out.cpu().view(torch.int16), w.view(torch.int16))


def test_unit_of_more_than_2_to_the_31_elements():
    """An unsharded Llama-405B block has 3.19 G weights: element and byte offsets pass 2^31 (the
    reference kernel indexes with `int`, decode.cu:26-34).  Packed on the GPU, decoded by both
    kernels, compared with the original weights bit for bit.  Needs about 30 GB of device memory."""
    import bench
    if torch.cuda.get_device_properties(0).total_memory < 60e9:
        pytest.skip("needs a GPU with 60 GB")
    n = 2 * 16384 * 16384 + 2 * 1024 * 16384 + 3 * 16384 * 53248          # 3 187 671 040
    assert n > 2 ** 31
    u = bench.make_unit(n, 0.02, seed=405, device=torch.device(DEV), keep_weights=True)
    want = u.pop("weights").view(torch.int16)
    st = _status()
    out = torch.empty(n, dtype=torch.bfloat16, device=DEV)
    aux = ops.prepare(u["luts"], u["enc"], u["pos"], u["gaps"], n, status=st)
    ops.decode_prepared(u["luts"], u["enc"], u["sm"], u["pos"], u["gaps"], aux, out=out, status=st)
    torch.cuda.synchronize()
    assert st.item() == 0 and torch.equal(out.view(torch.int16), want)
    out.zero_()
    ops.decode(u["luts"], u["enc"], u["sm"], u["pos"], u["gaps"], out=out, max_block_elems=u["widest"], status=st)
    torch.cuda.synchronize()
    assert st.item() == 0 and torch.equal(out.view(torch.int16), want)
    del out, want, aux, u
    torch.cuda.empty_cache()


def test_empty_and_one_element_units():
    """Nothing to decode is not an error (no launch, output untouched); a unit of one element and
    one of 17 (a group and a bit) decode through every entry point."""
    from tests.conftest import load_golden
    d = _to_dev(load_golden("gauss_n3"))
    guard = torch.full((8,), 7.0, dtype=torch.bfloat16, device=DEV)
    empty_u8 = torch.empty(0, dtype=torch.uint8, device=DEV)
    for fn in (lambda: _lib.lib.df11_decode(d["luts"].data_ptr(), d["enc"].data_ptr(), d["sm"].data_ptr(),
                                            d["pos"].data_ptr(), d["gaps"].data_ptr(), guard.data_ptr(),
                                            d["luts"].shape[0], 0, 0, 0, None, 0, None),
               lambda: _lib.lib.df11_decode_prepared(d["luts"].data_ptr(), d["enc"].data_ptr(), d["sm"].data_ptr(),
                                                     d["pos"].data_ptr(), d["gaps"].data_ptr(), guard.data_ptr(),
                                                     guard.data_ptr(), d["luts"].shape[0], 0, 0, 0, None, 0, None)):
        assert fn() == 0
    torch.cuda.synchronize()
    assert torch.all(guard == 7.0) and empty_u8.numel() == 0
    with pytest.raises(ValueError):
        codec.encode_weights([torch.empty(0, dtype=torch.bfloat16)])
    for n in (1, 17):
        w = (torch.randn(n, generator=torch.Generator().manual_seed(n)) * 0.02).to(torch.bfloat16)
        for where in ("cpu", DEV):
            t, dd, widest = _unit_from_weights([w.to(where)])
            st = _status()
            out = ops.decode(dd["luts"], dd["enc"], dd["sm"], dd["pos"], dd["gaps"], max_block_elems=widest, status=st)
            aux = ops.prepare(dd["luts"], dd["enc"], dd["pos"], dd["gaps"], n, status=st)
            out2 = ops.decode_prepared(dd["luts"], dd["enc"], dd["sm"], dd["pos"], dd["gaps"], aux, status=st)
            torch.cuda.synchronize()
            assert st.item() == 0
            assert torch.equal(out.cpu().view(torch.int16), w.view(torch.int16))
            assert torch.equal(out2.cpu().view(torch.int16), w.view(torch.int16))
