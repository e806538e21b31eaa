"""Reading DF11 safetensors files without intermediate copies.

The reference loads every file with ``safetensors.torch.load_file`` (a full copy of the file in
pageable host memory) and then, for ``cpu_offload``, copies the two large tensors of every unit
once more into pinned memory with ``Tensor.pin_memory()`` (dfloat11/dfloat11.py:215-219,256-263);
resident models are moved to the GPU afterwards by ``model.to(device)``, one synchronous
pageable copy per tensor.  Here a file is memory-mapped, and a large tensor goes from the page
cache straight to where it will live:

* ``cpu_offload``: one copy, page cache -> a pinned host tensor of its own;
* resident on a known CUDA device: page cache -> one of two pinned staging buffers ->
  ``cudaMemcpyAsync`` on a copy stream, so the host-side read of tensor i+1 overlaps the
  host->device copy of tensor i;
* anything else: one copy into an ordinary tensor.

The file format (8-byte little-endian header length, JSON header with ``dtype`` / ``shape`` /
``data_offsets`` per tensor, then the raw little-endian data) is the public safetensors layout.
"""
from __future__ import annotations

import json
import mmap
import struct
from typing import Tuple

import numpy as np
import torch

_DTYPES = {
    "U8": (np.uint8, torch.uint8), "I8": (np.int8, torch.int8), "BOOL": (np.bool_, torch.bool),
    "I16": (np.int16, torch.int16), "U16": (np.uint16, torch.uint16), "F16": (np.float16, torch.float16),
    "BF16": (np.uint16, torch.bfloat16),            # numpy has no bfloat16: read as 16-bit words, view in torch
    "I32": (np.int32, torch.int32), "U32": (np.uint32, torch.uint32), "F32": (np.float32, torch.float32),
    "I64": (np.int64, torch.int64), "U64": (np.uint64, torch.uint64), "F64": (np.float64, torch.float64),
}


class MappedFile:
    """A safetensors file mapped read-only; tensors are numpy views into the mapping until copied."""

    def __init__(self, path: str):
        self.path = path
        self._file = open(path, "rb")
        head = self._file.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: not a safetensors file (too short)")
        (n_header,) = struct.unpack("<Q", head)
        size = self._file.seek(0, 2)
        if n_header > size - 8:
            raise ValueError(f"{path}: header length {n_header} exceeds the file")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_COPY)   # private: never written, never copied
        self.header = json.loads(self._map[8:8 + n_header].decode("utf-8"))
        self.header.pop("__metadata__", None)
        self._base = 8 + n_header
        self._bytes = np.frombuffer(self._map, dtype=np.uint8)
        for name, meta in self.header.items():
            a, b = meta["data_offsets"]
            if meta["dtype"] not in _DTYPES or a > b or self._base + b > size:
                raise ValueError(f"{path}: bad entry for tensor '{name}'")

    def names(self):
        # in file order, which is the order the tensors were saved in
        return sorted(self.header, key=lambda n: self.header[n]["data_offsets"][0])

    def nbytes(self, name: str) -> int:
        a, b = self.header[name]["data_offsets"]
        return b - a

    def raw(self, name: str) -> np.ndarray:
        """The tensor's bytes as a uint8 view into the mapping (no copy)."""
        a, b = self.header[name]["data_offsets"]
        return self._bytes[self._base + a:self._base + b]

    def torch_dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.header[name]["dtype"]][1]

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.header[name]["shape"])

    def tensor(self, name: str, pin: bool = False) -> torch.Tensor:
        """A tensor that owns its memory: one copy out of the mapping, into pinned memory if asked."""
        raw = self.raw(name)
        out = torch.empty(raw.size, dtype=torch.uint8, pin_memory=pin and torch.cuda.is_available())
        if raw.size:
            out.copy_(torch.from_numpy(raw))              # torch's host copy runs on several threads
        return out.view(self.torch_dtype(name)).reshape(self.shape(name))

    def close(self) -> None:
        self._bytes = None
        try:
            self._map.close()
        except BufferError:          # a view is still alive somewhere; the mapping goes with it
            pass
        self._file.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class DeviceUploader:
    """Host -> device copies of large tensors through two pinned staging buffers and a copy
    stream: while ``cudaMemcpyAsync`` moves one tensor, the host already reads the next one out
    of the page cache into the other buffer."""

    def __init__(self, device: torch.device, staging_bytes: int = 64 << 20):
        self.device = torch.device(device)
        self.stream = torch.cuda.Stream(device=self.device)
        self._staging = [None, None]
        self._busy = [None, None]            # event recorded after the copy that reads a buffer
        self._min = staging_bytes
        self._turn = 0
        self.stats = dict(tensors=0, bytes=0)

    def upload(self, raw: np.ndarray, dtype: torch.dtype, shape) -> torch.Tensor:
        """Queues the copy of ``raw`` (a uint8 view into a mapping) and returns the device tensor;
        ``finish`` must be called before it is used on another stream."""
        n = int(raw.size)
        out = torch.empty(n, dtype=torch.uint8, device=self.device)
        self.stream.wait_stream(torch.cuda.current_stream(self.device))   # whatever used that memory before is over
        done = 0
        while done < n:
            k = self._turn
            self._turn ^= 1
            if self._staging[k] is None:
                self._staging[k] = torch.empty(self._min, dtype=torch.uint8, pin_memory=True)
            if self._busy[k] is not None:
                self._busy[k].synchronize()                   # the copy that last read this buffer is over
            piece = min(n - done, self._staging[k].numel())
            self._staging[k][:piece].copy_(torch.from_numpy(raw[done:done + piece]))
            with torch.cuda.stream(self.stream):
                out[done:done + piece].copy_(self._staging[k][:piece], non_blocking=True)
                self._busy[k] = torch.cuda.Event()
                self._busy[k].record(self.stream)
            done += piece
        self.stats["tensors"] += 1
        self.stats["bytes"] += n
        return out.view(dtype).reshape(shape)

    def finish(self) -> None:
        self.stream.synchronize()
        self._staging = [None, None]
        self._busy = [None, None]
