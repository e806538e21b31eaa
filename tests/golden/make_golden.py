"""Generates tests/golden/*.npz by running the REFERENCE's own codec functions.

Run in the build container only (needs the read-only reference checkout):

    python tests/golden/make_golden.py [path of the reference checkout]

The reference's ``dfloat11/dfloat11_utils.py`` is imported unmodified, by file
path.  Its one missing dependency, the third-party ``dahuffman`` package
(pinned ==0.4.2 in the reference's setup.py:20, absent here), is satisfied by
the stand-in in ``oracle/standin/`` -- an independent Huffman builder that only
decides WHICH prefix code is used; everything recorded below (LUT rows, bit
stream, gaps, output positions, sign/mantissa split) is computed by reference
code from that code table.

Every fixture stores the original BF16 bit patterns (``w``), the six DF11
tensors as the reference produced them, and the code table in the reference's
dict iteration order (``table_syms/bits/vals`` + ``eof_bits/eof_val``).
"""
import contextlib
import importlib.util
import io
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REFERENCE = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(ROOT), "reference")   # beside the repository

sys.path.insert(0, os.path.join(ROOT, "oracle", "standin"))
spec = importlib.util.spec_from_file_location(
    "ref_dfloat11_utils", os.path.join(REFERENCE, "dfloat11", "dfloat11_utils.py"))
ref = importlib.util.module_from_spec(spec)
spec.loader.exec_module(ref)
ref.tqdm = lambda x, *a, **k: x          # silence progress bars only


def bf16_from_float(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16)


def bf16_from_parts(exponent: np.ndarray, rng: np.random.Generator) -> torch.Tensor:
    sm = rng.integers(0, 256, size=exponent.size, dtype=np.uint16)
    w = ((sm & 0x80) << 8) | (exponent.astype(np.uint16) << 7) | (sm & 0x7F)
    return torch.from_numpy(w.astype(np.uint16).view(np.int16)).view(torch.bfloat16)


def table_arrays(codec):
    syms, bits, vals = [], [], []
    eof = None
    for key, (b, v) in codec.get_code_table().items():
        if isinstance(key, int):
            syms.append(key), bits.append(b), vals.append(v)
        else:
            eof = (b, v)
    return (np.asarray(syms, np.int32), np.asarray(bits, np.int32),
            np.asarray(vals, np.uint64), eof)


def run_reference(weights, counter=None):
    """weights: list of 1-D bf16 tensors making up one compressed unit."""
    with contextlib.redirect_stdout(io.StringIO()):
        if counter is None:
            _, counter = ref.get_codec(torch.cat(weights))
        codec, _, table = ref.get_32bit_codec(counter)
        luts = ref.get_luts(table)
        encoded, sm, pos, gaps, split = ref.encode_weights(weights, codec, 8, 512)
    syms, bits, vals, eof = table_arrays(codec)
    return dict(
        w=torch.cat(weights).view(torch.int16).numpy().view(np.uint16),
        luts=luts.numpy(), encoded=encoded.numpy(), sign_mantissa=sm.numpy(),
        output_positions=pos.numpy().astype(np.uint32), gaps=gaps.numpy(),
        split_positions=split.numpy().astype(np.int64),
        table_syms=syms, table_bits=bits, table_vals=vals,
        eof_bits=np.int32(eof[0]), eof_val=np.uint64(eof[1]),
    )


def total_bits(exponents, counter):
    with contextlib.redirect_stdout(io.StringIO()):
        codec, _, _ = ref.get_32bit_codec(counter)
    t = codec.get_code_table()
    return sum(t[int(e)][0] for e in exponents), {k: v[0] for k, v in t.items() if isinstance(k, int)}


def exps_of(w):
    return ((w.view(torch.int16).numpy().view(np.uint16) >> 7) & 0xFF).astype(np.int64)


def counter_of(w):
    vals, cnt = np.unique(exps_of(w), return_counts=True)
    return {int(v): int(c) for v, c in zip(vals, cnt)}


def pad_to_bits(w, counter, target_multiple, rng):
    """Append elements (using only exponents already in `counter`) until the coded
    length is an exact multiple of `target_multiple` bits."""
    bits, lens = total_bits(exps_of(w), counter)
    by_len = {}
    for s, l in lens.items():
        by_len.setdefault(l, s)
    short = sorted(by_len)[:2]
    assert len(short) == 2 and np.gcd(short[0], short[1]) == 1, short
    a, b = short
    need = (-bits) % target_multiple
    while True:
        sol = [y for y in range(a) if need - b * y >= 0 and (need - b * y) % a == 0]
        if sol:
            break
        need += target_multiple
    y = sol[0]
    extra = np.asarray([by_len[b]] * y + [by_len[a]] * ((need - b * y) // a))
    if extra.size:
        w = torch.cat([w, bf16_from_parts(extra, rng)])
    bits2, _ = total_bits(exps_of(w), counter)
    assert bits2 % target_multiple == 0, (bits2, target_multiple)
    return w


def main():
    out = {}
    g = torch.Generator().manual_seed(0)

    # 1. Gaussian weights N(0, 0.02), three sub-weights in one unit, several format blocks
    parts = [bf16_from_float(torch.randn(n, generator=g) * 0.02) for n in (10000, 20000, 10000)]
    out["gauss_multi"] = run_reference(parts)

    # 2./3. tiny units
    out["gauss_n1"] = run_reference([bf16_from_float(torch.randn(1, generator=g) * 0.02)])
    out["gauss_n3"] = run_reference([bf16_from_float(torch.randn(3, generator=g) * 0.02)])

    # 4. N(0,1) "embedding-like" weights
    out["gauss_wide"] = run_reference([bf16_from_float(torch.randn(30000, generator=g))])

    rng = np.random.default_rng(0)

    # 5. two exponents 50/50: shortest code is 1 bit -> > 20000 elements per format block
    e = rng.integers(0, 2, size=50000) + 120
    out["two_exponents"] = run_reference([bf16_from_parts(e, rng)])

    # 6. 240 equiprobable exponents (values 0..239): 7/8-bit codes, root table full
    e = rng.integers(0, 240, size=30000)
    out["uniform_240"] = run_reference([bf16_from_parts(e, rng)])

    # 7. long codes: counts 2^i make the Huffman tree degenerate.  40 symbols push the
    #    unconstrained tree past 32 bits, so the reference's length limiter
    #    (dfloat11_utils.py:49-63) runs; 32 symbols give a 32-bit deepest code without
    #    it (four LUT levels).  Data is a small sample that contains every symbol (the
    #    code table need not match the data it encodes).
    for name, nsym in (("long_codes", 40), ("deep_codes", 32)):
        counter = {100 + i: 2 ** i for i in range(nsym)}
        probs = np.asarray([1.0 / (i + 1) for i in range(nsym)][::-1])
        e = np.concatenate([np.arange(100, 100 + nsym),
                            rng.choice(np.arange(100, 100 + nsym), size=6000, p=probs / probs.sum())])
        rng.shuffle(e)
        out[name] = run_reference([bf16_from_parts(e, rng)], counter=counter)

    # 8. stream ends exactly on a byte boundary (no end-of-stream padding byte)
    w = bf16_from_float(torch.randn(5000, generator=g) * 0.02)
    c = counter_of(w)
    out["byte_aligned_end"] = run_reference([pad_to_bits(w, c, 8, rng)], counter=c)

    # 9. stream ends exactly on a 4096-byte format-block boundary
    w = bf16_from_float(torch.randn(20000, generator=g) * 0.02)
    c = counter_of(w)
    out["block_aligned_end"] = run_reference([pad_to_bits(w, c, 4096 * 8, rng)], counter=c)

    # 10. stream ends exactly on an 8-byte window boundary plus one short tail window
    w = bf16_from_float(torch.randn(3000, generator=g) * 0.02)
    c = counter_of(w)
    w = pad_to_bits(w, c, 64, rng)
    w = torch.cat([w, bf16_from_float(torch.randn(2, generator=g) * 0.02).clamp(0.01, 0.03)])
    out["window_aligned_plus2"] = run_reference([w], counter=counter_of(w))

    # 11. single-exponent units (700 zeros; 700 copies of one exponent)
    out["all_zero"] = lambda: run_reference([torch.zeros(700, dtype=torch.bfloat16)])
    out["single_exponent"] = lambda: run_reference([bf16_from_parts(np.full(700, 121), rng)])

    # The reference LUT builder fails on some code tables (dfloat11_utils.py:103-106 reads
    # `curr_val` before assignment when index 0 of a row is unmapped); record what
    # happened instead of a fixture where it does.
    notes = []
    for name in list(out):
        if callable(out[name]):
            try:
                out[name] = out[name]()
            except Exception as exc:  # noqa: BLE001 - recording the reference's behaviour
                notes.append(f"{name}: reference raised {type(exc).__name__}: {exc}")
                del out[name]

    for name, d in out.items():
        assert d["encoded"].size > 0
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **d)
        print(f"{name:24s} n_elements={d['w'].size:7d} n_bytes={d['encoded'].size:7d} "
              f"n_luts={d['luts'].shape[0]} max_len={int(d['table_bits'].max())} "
              f"gaps={d['gaps'].size} pos={d['output_positions'].tolist()[:4]}...")
    with open(os.path.join(HERE, "NOTES.txt"), "w") as f:
        f.write("Cases for which the reference codec raised instead of producing tensors:\n")
        f.write("\n".join(notes) + ("\n" if notes else "(none)\n"))
    print("\n".join(notes))


if __name__ == "__main__":
    main()
