"""Stand-in for the third-party ``dahuffman`` package (pinned ``==0.4.2`` by the
reference's ``setup.py:20``), which is not installed here and cannot be fetched.

TEST INFRASTRUCTURE ONLY.  It exists so that the reference's *unmodified*
``dfloat11/dfloat11_utils.py`` can be imported (it does ``from dahuffman import
HuffmanCodec`` at ``dfloat11_utils.py:18``) by the fixture generator in
``tests/golden/make_golden.py``.  It is an independent heap-based Huffman
builder, not a reproduction of that library: only the members the reference
touches are provided:

* ``HuffmanCodec.from_frequencies(counter)``   (``dfloat11_utils.py:32,38,57``)
* ``codec.get_code_table()`` -> ``{symbol: (n_bits, value)}`` with one extra
  non-int end-of-stream key                       (``dfloat11_utils.py:39,58``)
* ``codec._table`` / ``codec._eof``              (``dfloat11_utils.py:135,153``)
* ``codec.print_code_table()``                   (``dfloat11.py:554``)

Which prefix code a Huffman builder assigns (tree shape under frequency ties) is
a free choice: the DF11 format is self-describing through its ``luts`` tensor, so
decode parity does not depend on reproducing the real library's tie-breaks.
Parity for *code assignment* is therefore unpinned; parity of everything
downstream of a given code table (LUT layout, bit packing, gaps, output
positions, decode) is pinned through the reference's own functions.
"""
import heapq
import itertools
import sys


class _EndOfStream:
    """Sentinel symbol appended to every alphabet with frequency 1."""

    def __repr__(self):
        return "_EOF"

    # sort after every integer symbol so tie-breaking is deterministic
    def __lt__(self, other):
        return False

    def __gt__(self, other):
        return True


_EOF = _EndOfStream()


class HuffmanCodec:
    def __init__(self, table, eof):
        self._table = table
        self._eof = eof

    @classmethod
    def from_frequencies(cls, frequencies, eof=_EOF):
        freqs = dict(frequencies)
        freqs[eof] = 1
        tick = itertools.count()
        # heap items: (weight, insertion order, tree); tree = symbol leaf or (left, right)
        # The end-of-stream leaf is inserted first, so among equal weights it is merged
        # first; the lighter subtree of every merge becomes the '1' branch, which keeps
        # the end-of-stream code at the all-ones end of the code space (the reference's
        # LUT builder needs index 0 of every row to belong to a real symbol,
        # dfloat11_utils.py:103-106).
        heap = [(freqs[eof], next(tick), ("leaf", eof))]
        for sym in sorted((s for s in freqs if s is not eof)):
            heap.append((freqs[sym], next(tick), ("leaf", sym)))
        heapq.heapify(heap)
        if len(heap) == 1:
            w, _, leaf = heap[0]
            return cls({leaf[1]: (1, 0)}, eof)
        while len(heap) > 1:
            wa, _, a = heapq.heappop(heap)
            wb, _, b = heapq.heappop(heap)
            heapq.heappush(heap, (wa + wb, next(tick), ("node", b, a)))
        table = {}
        stack = [(heap[0][2], 0, 0)]
        while stack:
            node, depth, value = stack.pop()
            if node[0] == "leaf":
                table[node[1]] = (depth, value)
            else:
                stack.append((node[1], depth + 1, (value << 1)))
                stack.append((node[2], depth + 1, (value << 1) | 1))
        return cls(table, eof)

    def get_code_table(self):
        return self._table

    def print_code_table(self, out=sys.stdout):
        for sym, (bits, val) in sorted(self._table.items(), key=lambda kv: (kv[1][0], kv[1][1])):
            out.write(f"{bits:4d} {bin(val)[2:].rjust(bits, '0'):>34s} {sym!r}\n")
