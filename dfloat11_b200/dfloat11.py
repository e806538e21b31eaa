"""Host side of the decompression path: scratch buffers, the forward pre-hook, the loader,
device placement and the public model API.

This module mirrors the reference's ``dfloat11/dfloat11.py`` name for name -- ``TensorManager``
(:52-100), ``get_hook`` / ``decode_hook`` (:103-176), ``load_and_replace_tensors`` (:179-308),
``get_no_split_classes`` (:311-333), ``DFloat11Model.from_pretrained`` / ``from_single_file``
(:336-493) and ``compress_model`` (:496-636) -- with the same arguments, module attributes and
on-disk layout, so that code written against the reference keeps working.  What differs:

* the kernel is launched through the C ABI of libdf11 on torch's current stream (the
  reference goes through cupy's stream, dfloat11.py:142-151);
* every unit gets, on first use on a device, the auxiliary buffer of the fast decoder
  (``module.df11_aux``; set ``DF11_PREPARED=0`` to decode with no extra memory instead);
* ``cpu_offload`` copies the next unit's compressed tensors host->device on a side stream,
  into one of two reusable staging slots, while the current unit is being decoded and used
  (the reference issues the copy on the compute stream inside the hook, dfloat11.py:123-128);
* the loader resolves tensor names through dictionaries built once (the reference rebuilds
  ``state_dict()`` per tensor, dfloat11.py:224-228) and validates every unit before it can
  be launched;
* device placement is done here (accelerate is not a dependency).
"""
from __future__ import annotations

import json
import logging
import os
import re
import sys
import weakref
from sys import stderr
from typing import Dict, List, Optional, Union

import numpy as np
import torch
import torch.nn as nn

from . import _lib, codec, ops

log = logging.getLogger("dfloat11")

# Format constants (dfloat11.py:44-49); baked into every DF11 file's gaps / output_positions.
version = "0.5.0"
bytes_per_thread = 8
threads_per_block = (512,)
offloaded_tensor_names = ("encoded_exponent", "sign_mantissa")
_unit_tensor_names = ("luts", "encoded_exponent", "sign_mantissa", "output_positions", "gaps", "split_positions")


class _Flags:
    """The environment switches of the hook.  Reading five variables costs more host time than
    launching a decode, so inside a forward pass of a model marked by ``_mark_root`` they are
    read once, when that pass starts; a unit called on its own reads them on every call."""

    in_forward = False
    prepared = True
    decode_ahead = False
    ahead_window = False
    sparse = True
    fused = False
    nvtx = False
    check_status = False
    slab_head = True
    side_on_host = True
    offload_prepared = False

    @classmethod
    def read(cls) -> None:
        env = os.environ.get
        cls.prepared = env("DF11_PREPARED", "1") != "0"
        cls.decode_ahead = env("DF11_DECODE_AHEAD", "0") in ("1", "2")
        cls.ahead_window = env("DF11_DECODE_AHEAD", "0") == "2"
        cls.sparse = env("DF11_SPARSE_EMBEDDING", "1") != "0"
        cls.fused = env("DF11_FUSED_GEMV", "0") == "1"
        cls.nvtx = env("DF11_NVTX", "0") == "1"
        cls.check_status = env("DF11_CHECK_STATUS", "0") == "1"
        cls.slab_head = env("DF11_SLAB_HEAD", "1") != "0"
        cls.side_on_host = env("DF11_SIDE_TENSORS_ON_HOST", "1") != "0"
        cls.offload_prepared = env("DF11_OFFLOAD_PREPARED", "0") == "1"

    @classmethod
    def current(cls):
        if not cls.in_forward:
            cls.read()
        return cls


def _use_prepared() -> bool:
    return _Flags.current().prepared


class TensorManager:
    """BF16 scratch tensors per device, shared by every compressed unit (dfloat11.py:52-100).

    The reference keeps one tensor per device, and a unit's decode overwrites what the previous
    unit left there; correctness rests on stream order alone.  Here a device has a few such
    tensors ("slots"): slot 0 is the reference's; decode-ahead alternates between slots 0 and 1
    so that the next unit can be decompressed while the current one still computes, and the
    rows of a sparsely decoded lookup table live in slot 2.
    """

    _tensors: Dict[tuple, torch.Tensor] = {}
    _users: Dict[tuple, "weakref.WeakSet"] = {}
    # Elements the scratch of slots 0 / 1 is given at least: the largest unit that is decoded as a
    # whole among the models loaded so far, so that the scratch is allocated once instead of
    # growing unit by unit (a grown-out-of tensor stays alive as long as a layer holds a view of it).
    min_elements = 0

    @staticmethod
    def allocate_bfloat16(device, n_elements: int, slot: int = 0) -> torch.Tensor:
        """A BF16 tensor of exactly ``n_elements`` on ``device``: a slice of the device's scratch,
        which is replaced by a larger one when it is too small."""
        device = torch.device(device)
        if device.type == "cuda" and device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        key = (device, slot)
        existing = TensorManager._tensors.get(key)
        if existing is not None:
            if existing.numel() >= n_elements:
                return existing[:n_elements]
            del TensorManager._tensors[key]
            del existing
            # the layers that still hold views of the old tensor let go of them (their hooks make new
            # ones before their next forward), or the old tensor would stay allocated beside the new
            for user in list(TensorManager._users.pop(key, ())):
                _drop_views(user)
            if device.type == "cuda":
                torch.cuda.empty_cache()
        size = max(n_elements, TensorManager.min_elements) if slot in (0, 1) else n_elements
        new_tensor = torch.empty(size, dtype=torch.bfloat16, device=device)
        log.info("Allocated %d bf16 on device %s (slot %d)", size, device, slot)
        TensorManager._tensors[key] = new_tensor
        return new_tensor[:n_elements]

    @staticmethod
    def note_user(module: nn.Module, tensor: torch.Tensor) -> None:
        """Remembers that ``module``'s layers hold views of the scratch ``tensor`` is a slice of."""
        for key, scratch in TensorManager._tensors.items():
            if scratch.data_ptr() == tensor.data_ptr():
                TensorManager._users.setdefault(key, weakref.WeakSet()).add(module)
                return

    @staticmethod
    def release(device=None) -> None:
        """Drop the scratch of one device (or of all)."""
        if device is None:
            TensorManager._tensors.clear()
            TensorManager._users.clear()
            TensorManager.min_elements = 0
        else:
            device = torch.device(device)
            for key in [k for k in TensorManager._tensors if k[0] == device]:
                del TensorManager._tensors[key]


_status_words: Dict[torch.device, torch.Tensor] = {}
_counters = dict(decodes=0, decoded_elements=0, prepares=0, sparse_lookups=0, fused_products=0, slab_products=0)


def _status_word(device: torch.device) -> torch.Tensor:
    """One int32 per device into which every decode launched by the hooks ORs its
    ``DF11_STATUS_*`` bits (the reference's kernel has no such channel: bad tensors make it
    read out of bounds or spin, decode.cu:116-118)."""
    word = _status_words.get(device)
    if word is None:
        word = _status_words[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return word


def check_status(reset: bool = True) -> None:
    """Raises ``DF11Error`` if a decode launched by the hooks since the last check met
    inconsistent tensors (bad table, bad positions, truncated block, timed-out copy) or an
    embedding index outside its table, or if a one-kernel all-reduce of the partitioned mode gave
    up waiting for a peer.  Synchronises with the devices, so it is not called per forward unless
    ``DF11_CHECK_STATUS=1`` is set."""
    names = {_lib.STATUS_BAD_TABLE: "bad table", _lib.STATUS_BAD_POSITIONS: "bad positions or index",
             _lib.STATUS_TRUNCATED: "truncated block", _lib.STATUS_TIMEOUT: "copy timed out"}
    for device, word in _status_words.items():
        bits = int(word.item())
        if bits:
            if reset:
                word.zero_()
            what = ", ".join(n for b, n in names.items() if bits & b) or "unknown"
            raise _lib.DF11Error(_lib.DF11_ERR_CORRUPT, f"decode on {device} reported status {bits} ({what})")
    comm = sys.modules.get(__package__ + ".comm")       # only if the partitioned mode set it up
    if comm is not None:
        for instance in comm.PeerAllReduce._instances.values():
            if instance is not None:
                instance.check()


def stats() -> dict:
    """Counters of the host side since import: decodes launched by the hooks, elements they
    produced, auxiliary buffers built, sparse embedding lookups, fused products, bytes copied
    host->device by ``cpu_offload`` and how often the next unit's copy was already under way,
    decode-ahead hits and misses, and the scratch held per device."""
    out = dict(_counters)
    out["offload"] = {str(d): dict(s.stats) for d, s in _OffloadStager._by_device.items()}
    out["decode_ahead"] = {str(d): dict(a.stats) for d, a in _DecodeAhead._by_device.items()}
    out["scratch_bytes"] = {f"{d}/slot{slot}": t.numel() * 2 for (d, slot), t in TensorManager._tensors.items()}
    return out


class _OffloadStager:
    """Per-device machinery of ``cpu_offload``: a copy stream and two staging slots.

    Units are visited in a fixed cyclic order (``module.df11_next_offloaded``).  While unit i is
    decoded, the pinned host tensors of unit i+1 are already on their way into the other slot
    (``cudaMemcpyAsync`` on the copy stream).  A slot is handed back to the copy stream by an
    event recorded on the compute stream after the decode that read it.
    """

    _by_device: Dict[torch.device, "_OffloadStager"] = {}

    def __init__(self, device: torch.device):
        self.device = device
        self.stream = torch.cuda.Stream(device=device)
        self.slots = [dict(buf={}, ready=None, free=None, owner=None) for _ in range(2)]
        self.stats = dict(h2d_bytes=0, copies=0, prefetch_hits=0)

    @classmethod
    def get(cls, device: torch.device) -> "_OffloadStager":
        if device not in cls._by_device:
            cls._by_device[device] = cls(device)
        return cls._by_device[device]

    def _issue(self, module: nn.Module, keep: Optional[nn.Module] = None) -> dict:
        # a free slot if there is one, otherwise the one that does not hold `keep`
        slot = next((s for s in self.slots if s["owner"] is None), None)
        if slot is None:
            slot = next(s for s in self.slots if s["owner"] is not keep)
        compute = torch.cuda.current_stream(self.device)
        nvtx = _Flags.current().nvtx
        if nvtx:
            torch.cuda.nvtx.range_push("df11.h2d")
        with torch.cuda.stream(self.stream):
            if slot["free"] is not None:
                self.stream.wait_event(slot["free"])
            for name, host in module.offloaded_tensors.items():
                buf = slot["buf"].get(name)
                if buf is None or buf.numel() < host.numel() or buf.numel() > host.numel() + host.numel() // 4:
                    # sized for the unit it holds: a slot that took a vocabulary-sized unit gives that
                    # memory back when a transformer block follows (units of one size reuse the buffer)
                    slot["buf"].pop(name, None)
                    buf = None
                    buf = torch.empty(host.numel(), dtype=torch.uint8, device=self.device)
                    buf.record_stream(compute)
                    slot["buf"][name] = buf
                buf[:host.numel()].copy_(host, non_blocking=True)
                self.stats["h2d_bytes"] += host.numel()
                self.stats["copies"] += 1
            slot["ready"] = torch.cuda.Event()
            slot["ready"].record(self.stream)
        if nvtx:
            torch.cuda.nvtx.range_pop()
        slot["owner"] = module
        return slot

    def fetch(self, module: nn.Module) -> Dict[str, torch.Tensor]:
        """Device views of the unit's offloaded tensors, valid for work queued on the current
        stream after this call; also starts the copy of the unit that follows."""
        slot = next((s for s in self.slots if s["owner"] is module and s["ready"] is not None), None)
        if slot is None:
            slot = self._issue(module)
        else:
            self.stats["prefetch_hits"] += 1
        torch.cuda.current_stream(self.device).wait_event(slot["ready"])
        views = {name: slot["buf"][name][:host.numel()] for name, host in module.offloaded_tensors.items()}
        # prefetch the unit that runs next (the loader links the offloaded units in forward order)
        nxt = getattr(module, "df11_next_offloaded", None)
        if nxt is not None and nxt is not module and nxt.luts.device == self.device and not any(s["owner"] is nxt and s["ready"] is not None for s in self.slots):
            self._issue(nxt, keep=module)
        return views

    def done(self, module: nn.Module) -> None:
        """Call after the decode of ``module`` has been queued: its slot may be overwritten
        once that decode has run."""
        for s in self.slots:
            if s["owner"] is module:
                s["free"] = torch.cuda.Event()
                s["free"].record(torch.cuda.current_stream(self.device))
                s["ready"] = None
                s["owner"] = None


def _use_decode_ahead() -> bool:
    return _Flags.current().decode_ahead


def _sparse_enabled() -> bool:
    return _Flags.current().sparse


class _DecodeAhead:
    """Per device: decompress the unit that is expected next on a second stream while the
    current unit computes (the reference decodes in the stream of the forward pass, so the
    GPU does nothing else meanwhile, dfloat11.py:119-151).

    The order of the units is learned from the hooks themselves: every hook notes which unit
    ran before it in the same forward.  After a unit's own decode is queued, the unit that
    followed it last time is decoded on the side stream into the other scratch slot, by a
    launch that leaves part of every SM to the kernels of the forward pass
    (``df11_decode_prepared_shared``).  Its hook then only waits for that decode.  A wrong guess
    costs the wasted decode and nothing else: the hook decodes in-stream as usual.
    Batch-1 generation spends most of its time in small latency-bound kernels; this is where
    the decode hides.
    """

    _by_device: Dict[torch.device, "_DecodeAhead"] = {}

    def __init__(self, device: torch.device):
        self.device = device
        self.stream = torch.cuda.Stream(device=device)
        self.prev: Optional[nn.Module] = None      # unit whose hook ran last in this forward
        self.pending = None                        # (module, slot, done event, tensor, elements decoded)
        self.armed = None                          # windowed mode: (current unit, its successor), not yet launched
        self.slot = 0                              # slot that holds the weights of `prev`
        self.stats = dict(hits=0, misses=0, wasted=0, launched=0)

    @classmethod
    def get(cls, device: torch.device) -> "_DecodeAhead":
        if device not in cls._by_device:
            cls._by_device[device] = cls(device)
        return cls._by_device[device]

    @classmethod
    def end_of_forward(cls) -> None:
        """Joins whatever is still in flight and forgets the last unit, so that "last unit of
        one forward -> first unit of the next" is never learned as an order."""
        for ahead in cls._by_device.values():
            if ahead.pending is not None:
                torch.cuda.current_stream(ahead.device).wait_event(ahead.pending[2])
                ahead.pending = None
                ahead.stats["wasted"] += 1
            ahead.prev = None
            ahead.armed = None

    @staticmethod
    def eligible(unit: nn.Module, device: torch.device) -> bool:
        """Resident on this device, auxiliary buffer already built, decoded as a whole."""
        if hasattr(unit, "offloaded_tensors"):
            return False
        aux = unit.__dict__.get("df11_aux")
        if aux is None or aux.device != device or unit.luts.device != device:
            return False
        return not (isinstance(unit, nn.Embedding) and _sparse_enabled())

    def claim(self, module: nn.Module, n_elements: int):
        """``(tensor, n)``: the scratch tensor of ``module`` whose first ``n`` elements were decoded
        ahead (valid for work queued on the current stream after this call), or ``(None, 0)``."""
        pending, self.pending = self.pending, None
        self.armed = None
        if pending is None:
            self.stats["misses"] += 1
            return None, 0
        unit, slot, done, tensor, upto = pending
        torch.cuda.current_stream(self.device).wait_event(done)    # nobody writes a slot after this
        if unit is module and tensor.numel() == n_elements:
            self.stats["hits"] += 1
            self.slot = slot
            return tensor, upto
        self.stats["wasted"] += 1
        self.stats["misses"] += 1
        return None, 0

    def fresh_slot(self) -> int:
        self.slot ^= 1
        return self.slot

    def after(self, module: nn.Module, light: bool = False) -> None:
        """Call when ``module``'s own decode has been queued: learn the order, start the next.
        ``light``: this unit's forward is too short to hide anything behind."""
        if self.pending is not None:                   # a guess nobody claimed: join it before going on
            torch.cuda.current_stream(self.device).wait_event(self.pending[2])
            self.pending = None
            self.stats["wasted"] += 1
        if self.prev is not None and self.prev is not module:
            self.prev.__dict__["df11_next_unit"] = module
        self.prev = module
        self.armed = None
        nxt = module.__dict__.get("df11_next_unit")
        if nxt is None or nxt is module or not self.eligible(nxt, self.device):
            return
        if _Flags.current().ahead_window and not light:
            # windowed: nothing yet; the first part of the next unit is decompressed when this
            # unit's trigger layer has run (see `window`), the rest by the next unit's own hook
            if self._window_hook(module):
                self.armed = (module, nxt)
            return
        self._launch(module, nxt, light, None)

    def _window_hook(self, unit: nn.Module) -> bool:
        """Registers, once per unit, a forward hook on the layer after which the unit's forward
        leaves most of the GPU idle for a while (``DF11_AHEAD_AFTER``, default ``v_proj``: rotary
        embedding, cache update and attention follow).  False if the unit has no such layer."""
        d = unit.__dict__
        if "df11_window_hook" not in d:
            name = os.environ.get("DF11_AHEAD_AFTER", "v_proj")
            layer = next((m for n, m in unit.named_modules() if n.split(".")[-1] == name), None)
            if layer is None:
                d["df11_window_hook"] = None
            else:
                ref = weakref.ref(unit)
                d["df11_window_hook"] = layer.register_forward_hook(
                    lambda _m, _i, _o: _DecodeAhead.window(ref()))
        return d["df11_window_hook"] is not None

    @classmethod
    def window(cls, unit: Optional[nn.Module]) -> None:
        """The trigger layer of ``unit`` has run: start on its successor now."""
        if unit is None or not _Flags.current().ahead_window:
            return
        for ahead in cls._by_device.values():
            if ahead.armed is not None and ahead.armed[0] is unit:
                (_, nxt), ahead.armed = ahead.armed, None
                n = nxt.sign_mantissa.numel()
                chunk = ops.chunk_elements()
                part = int(n * float(os.environ.get("DF11_AHEAD_FRACTION", "0.4"))) // chunk * chunk
                if part > 0:
                    ahead._launch(unit, nxt, False, part)

    def _launch(self, module: nn.Module, nxt: nn.Module, light: bool, part: Optional[int]) -> None:
        n_next = nxt.sign_mantissa.numel()
        n_this = module.sign_mantissa.numel() if not hasattr(module, "offloaded_tensors") else n_next
        ctas = int(os.environ.get("DF11_AHEAD_CTAS", "1"))
        if light or n_next > 2 * n_this:
            ctas = 0                                   # nothing to share the GPU with: full speed
        slot = self.slot ^ 1
        tensor = TensorManager.allocate_bfloat16(self.device, n_next, slot=slot)
        main = torch.cuda.current_stream(self.device)
        queued = torch.cuda.Event()
        queued.record(main)                            # the slot's previous reader has been queued before this
        self.stream.wait_event(queued)
        with torch.cuda.stream(self.stream):
            if part is None:
                pos, gaps = _side_tensors(nxt, self.device)
                ops.decode_prepared(nxt.luts, nxt.encoded_exponent, nxt.sign_mantissa, pos, gaps, nxt.df11_aux,
                                    out=tensor, ctas_per_sm=ctas, status=_status_word(self.device))
            else:
                ops.decode_range_prepared(nxt.luts, nxt.encoded_exponent, nxt.sign_mantissa, nxt.df11_aux, 0, part,
                                          out=tensor, ctas_per_sm=ctas, status=_status_word(self.device))
            done = torch.cuda.Event()
            done.record(self.stream)
        self.pending = (nxt, slot, done, tensor, n_next if part is None else part)
        self.stats["launched"] += 1


def _start_of_forward_hook(_module, _inputs):
    _Flags.read()
    _Flags.in_forward = True


def _end_of_forward_hook(_module, _inputs, _output):
    _Flags.in_forward = False
    if _DecodeAhead._by_device:
        _DecodeAhead.end_of_forward()
    if _Flags.check_status:
        check_status()


def _mark_root(model: nn.Module) -> None:
    """Called once all units of a model are armed.  Lets the hooks see where a forward pass of the
    whole model starts and ends (the environment switches are read once per pass; decode-ahead
    joins what is in flight), sizes the shared scratch for the largest unit that is decoded as a
    whole, gives large single-Linear units their slab-wise forward and links the offloaded units
    in forward order for the prefetcher."""
    units = [m for m in model.modules() if isinstance(getattr(m, "split_positions", None), list)
             and (hasattr(m, "luts") or hasattr(m, "offloaded_tensors"))]
    def elements(m):
        t = m.offloaded_tensors.get("sign_mantissa") if hasattr(m, "offloaded_tensors") else None
        return (t if t is not None else m.sign_mantissa).numel()
    whole = [elements(m) for m in units
             if not isinstance(m, (nn.Embedding, nn.Linear)) or elements(m) < SLAB_MIN_ELEMENTS]
    if whole:
        TensorManager.min_elements = max(TensorManager.min_elements, max(whole))
    for m in units:
        if _slab_rows(m):
            _install_slabbed(m)
    # offloaded units in definition (= forward) order; a lookup table that can be read row by row out
    # of pinned memory is never staged, so it is not part of the ring
    ring = [m for m in units if hasattr(m, "offloaded_tensors")
            and not (isinstance(m, nn.Embedding) and m.max_norm is None and m.embedding_dim % ops.chunk_elements() == 0)]
    for a, b in zip(ring, ring[1:] + ring[:1]):
        a.__dict__["df11_next_offloaded"] = b          # a plain reference, not a registered submodule
    if not model.__dict__.get("df11_root_hooked"):
        model.register_forward_pre_hook(_start_of_forward_hook)
        model.register_forward_hook(_end_of_forward_hook, always_call=True)
        model.__dict__["df11_root_hooked"] = True


def _drop_views(module: nn.Module) -> None:
    """Takes back the weight views handed to a unit's layers (the scratch they point into is
    going away); the unit's hook hands out new ones before its next forward."""
    d = module.__dict__
    d["df11_injected"] = None
    d["df11_fast"] = None
    layers = [module] if isinstance(module, (nn.Linear, nn.Embedding)) else getattr(module, "weight_injection_modules", [])
    for layer in layers:
        if "weight" not in layer._parameters:
            layer.__dict__.pop("weight", None)
            layer.weight = None


def _inject_weights(module: nn.Module, reconstructed: torch.Tensor) -> None:
    """Hand the decoded BF16 buffer to the layers as views (dfloat11.py:154-166).

    The scratch tensor lives at the same address from one forward to the next, so the views
    handed out last time are still the right ones: they are only made again when the buffer
    has moved (first use, growth, another slot or device).  The reference re-creates them on
    every forward, which costs more host time than launching the decode."""
    key = (reconstructed.data_ptr(), reconstructed.numel())
    if module.__dict__.get("df11_injected") == key:
        return
    if isinstance(module, nn.Linear):
        module.weight = reconstructed.view(module.out_features, module.in_features)
    elif isinstance(module, nn.Embedding):
        module.weight = reconstructed.view(module.num_embeddings, module.embedding_dim)
    else:
        weights = torch.tensor_split(reconstructed, module.split_positions)
        for sub_module, weight in zip(module.weight_injection_modules, weights):
            sub_module.weight = weight.view(sub_module.out_features, sub_module.in_features)
    module.__dict__["df11_injected"] = key
    TensorManager.note_user(module, reconstructed)


def _sparse_embedding(module: nn.Module, inputs, n_elements: int) -> bool:
    """Whether this forward of an ``nn.Embedding`` unit can decode just the looked-up rows."""
    if not isinstance(module, nn.Embedding) or not _sparse_enabled():
        return False
    if not inputs or not isinstance(inputs[0], torch.Tensor) or inputs[0].is_floating_point():
        return False
    if module.max_norm is not None or module.embedding_dim % ops.chunk_elements():
        return False
    return 0 < inputs[0].numel() * module.embedding_dim < n_elements      # else the whole table is cheaper


def _use_fused_gemv() -> bool:
    return _Flags.current().fused


FUSED_MAX_ROWS = 4          # activation vectors one fused product takes (df11_gemv_prepared)


def _fused_layers(module: nn.Module):
    """(layer, first element of its weight inside the unit) for every Linear of a unit, or None
    when the unit cannot take the fused product (a lookup table, rows that are not multiples
    of a chunk -- 512 or 1024 elements, tensors kept on the host)."""
    if hasattr(module, "offloaded_tensors") or isinstance(module, nn.Embedding):
        return None
    layers = [module] if isinstance(module, nn.Linear) else list(getattr(module, "weight_injection_modules", []))
    chunk = ops.chunk_elements()
    if not layers or not all(isinstance(l, nn.Linear) and l.in_features % chunk == 0 for l in layers):
        return None
    starts = [0] + list(module.split_positions)
    if len(starts) != len(layers):
        return None
    return list(zip(layers, starts))


# Layers that are fed the same activations and lie next to each other in a unit: one fused
# product over their stacked rows serves all of them (three launches become one).
FUSED_FAMILIES = (("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj"), ("to_q", "to_k", "to_v"))


def _fused_groups(module: nn.Module, layers):
    """Splits ``layers`` [(layer, first element)] into runs that one product can serve."""
    leaf = {id(m): name.rsplit(".", 1)[-1] for name, m in module.named_modules()}
    groups, i = [], 0
    while i < len(layers):
        first_layer = layers[i][0]
        family = next((f for f in FUSED_FAMILIES if leaf.get(id(first_layer)) in f), ())
        j = i + 1
        while (j < len(layers) and leaf.get(id(layers[j][0])) in family
               and layers[j][0].in_features == first_layer.in_features
               and (layers[j][0].bias is None) == (first_layer.bias is None)):
            j += 1
        groups.append(layers[i:j])
        i = j
    return groups


def _install_fused(module: nn.Module) -> bool:
    """Gives every Linear of the unit a forward that multiplies straight from the compressed
    weights when it is called with at most FUSED_MAX_ROWS activation vectors, and otherwise
    decompresses the unit (once per forward of the unit) and calls the ordinary product."""
    state = module.__dict__.get("df11_fused")
    if state is not None:
        return bool(state)
    layers = _fused_layers(module)
    module.__dict__["df11_fused"] = layers or []
    if not layers:
        return False
    import torch.nn.functional as F

    def fused_ok(x, layer):
        rows = x.numel() // layer.in_features
        return (module.__dict__.get("df11_undecoded") and 0 < rows <= FUSED_MAX_ROWS and x.is_cuda
                and x.dtype == torch.bfloat16 and _use_fused_gemv())

    def product(x, first, n_rows, in_features, bias):
        rows = x.numel() // in_features
        _counters["fused_products"] += 1
        return ops.gemv_prepared(module.luts, module.encoded_exponent, module.sign_mantissa, module.df11_aux,
                                 x.reshape(rows, in_features).contiguous(), first, n_rows, in_features, bias=bias,
                                 status=_status_word(module.luts.device))

    def ordinary(x, layer):
        if module.__dict__.get("df11_undecoded"):
            _decode_whole_unit(module, module.luts.device)
        return F.linear(x, layer.weight, getattr(layer, "bias", None))

    def make_forward(group, k):
        layer, first = group[k]
        lead_first = group[0][1]
        total_rows = sum(l.out_features for l, _ in group)
        offset = sum(l.out_features for l, _ in group[:k])
        shared = group_state[id(group[0][0])]

        def forward(x):
            if not fused_ok(x, layer):
                return ordinary(x, layer)
            if len(group) == 1:
                y = product(x, first, layer.out_features, layer.in_features, getattr(layer, "bias", None))
                return y.view(*x.shape[:-1], layer.out_features)
            cached = shared.get("result")
            if k > 0 and cached is not None and cached[0] is x and cached[1] == x._version:
                y = cached[2]                                   # the leader already multiplied for everybody
            elif k == 0:
                if "bias" not in shared:
                    biases = [l.bias for l, _ in group]
                    shared["bias"] = None if biases[0] is None else torch.cat([b.detach() for b in biases])
                y = product(x, lead_first, total_rows, layer.in_features, shared["bias"])
                shared["result"] = (x, x._version, y)
            else:                                               # other activations than the leader's: on its own
                y = product(x, first, layer.out_features, layer.in_features, getattr(layer, "bias", None))
                return y.view(*x.shape[:-1], layer.out_features)
            return y[:, offset:offset + layer.out_features].reshape(*x.shape[:-1], layer.out_features)
        return forward

    group_state = {}
    for group in _fused_groups(module, layers):
        group_state[id(group[0][0])] = {}
        for k in range(len(group)):
            group[k][0].forward = make_forward(group, k)
    return True


def _side_tensors(module: nn.Module, device: torch.device):
    """(output_positions, gaps) as the launches want them.  Only ``df11_prepare`` and the
    self-contained decoder read these two; once a unit's auxiliary buffer exists they are kept on
    the host (0.026 bytes per weight given back to the device) and the fast decoder's entry
    points, which never read them, get another device tensor of the unit in their place."""
    pos, gaps = module.output_positions, module.gaps
    if pos.device == device and gaps.device == device:
        return pos, gaps
    return module.luts, module.luts


def _side_tensors_on_device(module: nn.Module, device: torch.device):
    """The real ``output_positions`` / ``gaps`` on ``device`` (moved back if they were parked on the host)."""
    if module.output_positions.device != device:
        module.output_positions = module.output_positions.to(device)
    if module.gaps.device != device:
        module.gaps = module.gaps.to(device)
    return module.output_positions, module.gaps


def _park_side_tensors(module: nn.Module) -> None:
    if _Flags.current().side_on_host and module.gaps.is_cuda and not torch.cuda.is_current_stream_capturing():
        module.gaps = module.gaps.cpu()
        module.output_positions = module.output_positions.cpu()


# A unit that is one large Linear layer (an output head over a vocabulary of 100 000 and more) is
# multiplied slab by slab when it is called with a few activation vectors: a slab of its rows is
# decompressed into the scratch the transformer blocks use, multiplied, and overwritten by the
# next slab.  Each output row is the same dot product whether the library multiplies the whole
# matrix or a block of its rows (checked bit for bit on the GPU for these shapes by
# tests/test_model_api.py), and the scratch never has to hold the whole matrix: 0.4 GB instead of
# 1.24 GB for a Qwen3-8B head.
SLAB_MIN_ELEMENTS = 1 << 27
SLAB_MAX_ROWS_IN = 4            # activation vectors up to which the slab path is taken


def _slab_rows(module: nn.Module) -> int:
    """Rows per slab of a slab-capable unit, 0 if the unit is not one."""
    if not isinstance(module, nn.Linear) or module.in_features % 1024:
        return 0
    if module.out_features * module.in_features < SLAB_MIN_ELEMENTS:
        return 0
    budget = TensorManager.min_elements or (1 << 26)
    rows = min(module.out_features, max(8, budget // module.in_features // 8 * 8))
    n_slabs = -(-module.out_features // rows)
    return min(module.out_features, (-(-module.out_features // n_slabs) + 7) // 8 * 8)


def _install_slabbed(module: nn.Module) -> None:
    """Gives a slab-capable Linear unit a forward that multiplies slab by slab when the hook left
    the unit undecoded (``df11_pending``), and calls the ordinary product otherwise."""
    if module.__dict__.get("df11_slabbed") is not None:
        return
    module.__dict__["df11_slabbed"] = True
    import torch.nn.functional as F

    def forward(x):
        pending = module.__dict__.pop("df11_pending", None)
        if pending is None:
            return F.linear(x, module.weight, module.bias)
        encoded_exponent, sign_mantissa, aux, stager, device = pending
        n_in, n_out = module.in_features, module.out_features
        rows = _slab_rows(module) or n_out
        m = x.numel() // n_in
        x2 = x.reshape(m, n_in)
        y = torch.empty(m, n_out, dtype=x.dtype, device=x.device)
        scratch = TensorManager.allocate_bfloat16(device, min(rows, n_out) * n_in)
        status = _status_word(device)
        for r0 in range(0, n_out, rows):
            r1 = min(n_out, r0 + rows)
            ops.decode_range_prepared(module.luts, encoded_exponent, sign_mantissa, aux, r0 * n_in, (r1 - r0) * n_in,
                                      out=scratch, status=status)
            w = scratch[:(r1 - r0) * n_in].view(r1 - r0, n_in)
            if m == 1 and module.bias is None:
                torch.mm(x2, w.t(), out=y[:, r0:r1])
            else:
                y[:, r0:r1] = F.linear(x2, w, None if module.bias is None else module.bias[r0:r1])
        _counters["slab_products"] += 1
        if stager is not None:
            stager.done(module)
        return y.view(*x.shape[:-1], n_out)

    module.forward = forward


def _decode_whole_unit(module: nn.Module, device: torch.device) -> None:
    """Decompress a resident, prepared unit into the scratch tensor and hand out the views."""
    n_elements = module.sign_mantissa.numel()
    reconstructed = TensorManager.allocate_bfloat16(device, n_elements)
    pos, gaps = _side_tensors(module, device)
    ops.decode_prepared(module.luts, module.encoded_exponent, module.sign_mantissa, pos, gaps, module.df11_aux,
                        out=reconstructed, max_block_elems=getattr(module, "max_block_elems", 0),
                        status=_status_word(device))
    _counters["decodes"] += 1
    _counters["decoded_elements"] += n_elements
    _inject_weights(module, reconstructed)
    module.__dict__["df11_undecoded"] = False


def get_hook(threads_per_block, bytes_per_thread):
    """Forward pre-hook that decompresses a unit's weights right before its forward
    (dfloat11.py:103-176).  The two arguments are the format constants; only 512 / 8 exist."""
    threads_per_block = tuple(threads_per_block)
    if threads_per_block[0] != 512 or bytes_per_thread != 8:
        raise ValueError("DF11 files are laid out for 512 threads per block and 8 bytes per thread "
                         f"(got {threads_per_block[0]} / {bytes_per_thread})")

    raw_stream = torch._C._cuda_getCurrentRawStream
    decode_prepared_c = _lib.lib.df11_decode_prepared

    def decode_hook(module, inputs):
        # Steady state of a resident unit: same compressed tensors, same auxiliary buffer, same
        # scratch as last time -> one call through the C ABI with the pointers kept from then,
        # the weight views of last time still valid.  Anything else takes the full path below.
        d = module.__dict__
        fast = d.get("df11_fast")
        if fast is not None:
            flags = _Flags.current()
            if (flags.prepared and not flags.fused and not flags.decode_ahead and not flags.nvtx
                    and d["_buffers"].get("encoded_exponent") is fast[0] and d.get("df11_aux") is fast[1]
                    and TensorManager._tensors.get(fast[2]) is fast[3]):
                rc = decode_prepared_c(*fast[4], raw_stream(fast[5]))
                if rc:
                    _lib.check(rc)
                d["df11_undecoded"] = False
                _counters["decodes"] += 1
                _counters["decoded_elements"] += fast[4][9]
                return None
        if _Flags.current().nvtx:                  # DF11_NVTX=1: one range per unit in profiler timelines
            torch.cuda.nvtx.range_push(f"df11.decode {type(module).__name__}")
            try:
                return full_path(module, inputs)
            finally:
                torch.cuda.nvtx.range_pop()
        return full_path(module, inputs)

    def full_path(module, inputs):
        d = module.__dict__
        device = module.luts.device
        if device.type != "cuda":
            raise RuntimeError("DF11 weights can only be decompressed on a CUDA device; move the model to "
                               f"one (this unit's tables are on {device})")
        status = _status_word(device)
        flags = _Flags.current()
        offloaded = hasattr(module, "offloaded_tensors")
        d["df11_undecoded"] = False
        d.pop("df11_pending", None)
        d.pop("df11_fast", None)          # whatever this pass injects replaces what the short path relied on

        if flags.prepared and offloaded and _sparse_embedding(module, inputs, module.offloaded_tensors[
                "sign_mantissa"].numel()) and all(t.is_pinned() for t in module.offloaded_tensors.values()):
            # An offloaded lookup table: the kernel reads the few rows it needs straight out of the
            # pinned host tensors (page-locked memory is addressable from the device), instead of
            # staging the whole compressed table on the device first as dfloat11.py:122-128 does
            # (0.83 GB per forward for a 152 k-row table of 4096 columns).
            host = module.offloaded_tensors
            aux = d.get("df11_aux")
            if aux is None or aux.device != device:
                pos, gaps = _side_tensors_on_device(module, device)
                aux = ops.prepare(module.luts, host["encoded_exponent"], pos, gaps, host["sign_mantissa"].numel(),
                                  status=status)
                module.df11_aux = aux
                _counters["prepares"] += 1
                _park_side_tensors(module)
            return sparse_lookup(module, inputs, host["encoded_exponent"], host["sign_mantissa"], aux, device, status,
                                 None, None)

        # compressed tensors: resident buffers, or the staging slot of the offload pipeline
        stager = None
        if offloaded:
            stager = _OffloadStager.get(device)
            staged = stager.fetch(module)
            encoded_exponent, sign_mantissa = staged["encoded_exponent"], staged["sign_mantissa"]
        else:
            encoded_exponent, sign_mantissa = module.encoded_exponent, module.sign_mantissa

        n_elements = sign_mantissa.numel()
        widest = getattr(module, "max_block_elems", 0)

        # An offloaded unit is bound by its host -> device copy (some 55 GB/s against 2 000 for the
        # slowest decoder), so it takes the self-contained kernel and keeps no auxiliary buffer on
        # the device: that is what offloading is for.  Units whose partial decode needs seek points
        # (a slab-wise head, a lookup table) keep theirs; DF11_OFFLOAD_PREPARED=1 gives every unit one.
        prepared = flags.prepared and (stager is None or flags.offload_prepared or d.get("df11_slabbed")
                                       or isinstance(module, nn.Embedding) or d.get("df11_aux") is not None)
        if prepared:
            aux = d.get("df11_aux")
            if aux is None or aux.device != device:
                # once per unit and device: decode table + seek points (derived data, never saved)
                pos, gaps = _side_tensors_on_device(module, device)
                aux = ops.prepare(module.luts, encoded_exponent, pos, gaps, n_elements, status=status)
                module.df11_aux = aux
                _counters["prepares"] += 1
                _park_side_tensors(module)
            if flags.fused and stager is None:
                # decode lazily: the unit's Linear layers multiply straight from the compressed
                # weights while they are called with a few activation vectors (generation), and
                # decompress the whole unit the first time one of them is not (prefill).  A unit
                # that is itself the Linear runs its first such call the ordinary way: torch has
                # already picked that call's forward when this hook installs the new one.
                fresh = d.get("df11_fused") is None
                if _install_fused(module) and not (fresh and isinstance(module, nn.Linear)):
                    d["df11_undecoded"] = True
                    return None
            if (flags.slab_head and d.get("df11_slabbed") and not d.get("df11_fused") and inputs
                    and isinstance(inputs[0], torch.Tensor)
                    and 0 < inputs[0].numel() // module.in_features <= SLAB_MAX_ROWS_IN):
                # a large single Linear called with a few activation vectors: its forward (installed at
                # load time) decompresses and multiplies slab by slab
                d["df11_pending"] = (encoded_exponent, sign_mantissa, aux, stager, device)
                d["df11_undecoded"] = True
                return None
            ahead = _DecodeAhead.get(device) if flags.decode_ahead else None
            if _sparse_embedding(module, inputs, n_elements):
                return sparse_lookup(module, inputs, encoded_exponent, sign_mantissa, aux, device, status, stager, ahead)
            reconstructed, upto = ahead.claim(module, n_elements) if ahead is not None else (None, 0)
            pos, gaps = _side_tensors(module, device)
            if reconstructed is not None and upto < n_elements:
                # the first part was decompressed beside the previous unit's forward; the rest now
                ops.decode_range_prepared(module.luts, encoded_exponent, sign_mantissa, aux, upto, n_elements - upto,
                                          out=reconstructed[upto:], status=status)
                _counters["decodes"] += 1
                _counters["decoded_elements"] += n_elements - upto
            if reconstructed is None:
                slot = ahead.fresh_slot() if ahead is not None else 0
                reconstructed = TensorManager.allocate_bfloat16(device, n_elements, slot=slot)
                ops.decode_prepared(module.luts, encoded_exponent, sign_mantissa, pos, gaps, aux, out=reconstructed,
                                    max_block_elems=widest, status=status)
                _counters["decodes"] += 1
                _counters["decoded_elements"] += n_elements
            _inject_weights(module, reconstructed)
            if stager is not None:
                stager.done(module)
            if ahead is not None:
                ahead.after(module)
            elif stager is None and not isinstance(module, nn.Embedding) and not d.get("df11_slabbed"):
                # remember what the next call of this unit can reuse as it is
                key = (device, slot)
                d["df11_fast"] = (
                    encoded_exponent, aux, key, TensorManager._tensors.get(key),
                    (module.luts.data_ptr(), encoded_exponent.data_ptr(), sign_mantissa.data_ptr(),
                     pos.data_ptr(), gaps.data_ptr(), aux.data_ptr(),
                     reconstructed.data_ptr(), module.luts.shape[0], encoded_exponent.numel(), n_elements,
                     int(widest), status.data_ptr(), device.index),
                    device.index)
            return None

        pos, gaps = _side_tensors_on_device(module, device)
        reconstructed = TensorManager.allocate_bfloat16(device, n_elements)
        ops.decode(module.luts, encoded_exponent, sign_mantissa, pos, gaps,
                   out=reconstructed, max_block_elems=widest, status=status)
        _counters["decodes"] += 1
        _counters["decoded_elements"] += n_elements
        _inject_weights(module, reconstructed)
        if stager is not None:
            stager.done(module)

    def sparse_lookup(module, inputs, encoded_exponent, sign_mantissa, aux, device, status, stager, ahead):
        # A lookup table: decompress only the rows that are asked for (the reference decodes the
        # whole table on every forward, dfloat11.py:158-161) and look them up by their position in
        # that small result.  During this forward ``module.weight`` is that [number of ids,
        # embedding_dim] tensor, not the whole table; an id outside the table yields row 0 and sets
        # the status word (see check_status), where F.embedding would raise a device-side assert.
        ids = inputs[0]
        if ids.device != device:
            ids = ids.to(device)
        rows = ops.decode_rows_prepared(module.luts, encoded_exponent, sign_mantissa, aux,
                                        ids.reshape(-1).to(torch.int64), module.embedding_dim,
                                        out=TensorManager.allocate_bfloat16(
                                            device, ids.numel() * module.embedding_dim, slot=2),
                                        status=status)
        _counters["sparse_lookups"] += 1
        module.weight = rows
        module.__dict__["df11_injected"] = None        # the whole-table view is gone
        if stager is not None:
            stager.done(module)
        if ahead is not None:
            ahead.after(module, light=True)
        return (torch.arange(ids.numel(), device=device).view(ids.shape),) + tuple(inputs[1:])

    return decode_hook


def _positions_u32(tensor: torch.Tensor) -> np.ndarray:
    """``output_positions`` is stored as a byte view of uint32 values (dfloat11.py:596)."""
    arr = tensor.cpu().numpy()
    return arr.view(np.uint32) if arr.dtype == np.uint8 else arr.astype(np.uint32)


def _finish_unit(module: nn.Module, full_name: str) -> None:
    """Checks a freshly loaded unit and derives what the launches need from it."""
    have = {n: getattr(module, n, None) for n in ("luts", "output_positions", "gaps")}
    enc = getattr(module, "encoded_exponent", None)
    sm = getattr(module, "sign_mantissa", None)
    if hasattr(module, "offloaded_tensors"):
        enc = module.offloaded_tensors.get("encoded_exponent", enc)
        sm = module.offloaded_tensors.get("sign_mantissa", sm)
    missing = [n for n, t in dict(have, encoded_exponent=enc, sign_mantissa=sm).items() if t is None]
    if missing:
        raise ValueError(f"DF11 unit '{full_name}' is incomplete: missing {', '.join(missing)}")
    widest = codec.validate_unit(have["luts"], enc, sm, have["output_positions"], have["gaps"])
    module.max_block_elems = widest
    # kept for code that reads the reference's attribute (dfloat11.py:299-306)
    module.shared_mem_size = threads_per_block[0] * 4 + 4 + widest * 2
    if not hasattr(module, "split_positions"):
        module.split_positions = []


def load_and_replace_tensors(
    model,
    directory_path,
    dfloat11_config,
    cpu_offload=False,
    cpu_offload_blocks=None,
    pin_memory=True,
    from_single_file=False,
    device=None,
):
    """Loads DF11 safetensors into ``model`` and arms on-the-fly decompression (dfloat11.py:179-308).

    Ordinary tensors are copied into the matching parameters / buffers.  The six tensors of a
    compressed unit become buffers of the module named by their prefix (``split_positions``
    a Python list); with ``cpu_offload`` the two large ones stay in (pinned) host memory in
    ``module.offloaded_tensors``.  The module gets the decode hook and loses the ``weight``
    attributes the hook will supply.

    Files are memory-mapped and every tensor is copied once, to where it will live
    (``safetensors_io``): offloaded tensors into pinned memory of their own, and -- when
    ``device`` names the CUDA device the model is about to be moved to (not in the reference's
    signature) -- the large tensors of resident units straight to that device through pinned
    staging, the copy of one overlapping the host-side read of the next.
    """
    from .safetensors_io import DeviceUploader, MappedFile

    tpb = dfloat11_config["threads_per_block"]
    bpt = dfloat11_config["bytes_per_thread"]
    pattern_dict = dfloat11_config["pattern_dict"] or {}
    hook = get_hook(tpb, bpt)

    if from_single_file:
        files = [directory_path]
    else:
        files = sorted(os.path.join(directory_path, f) for f in os.listdir(directory_path)
                       if f.endswith(".safetensors"))
    params = dict(model.named_parameters())
    buffers = dict(model.named_buffers())
    modules = dict(model.named_modules())
    units: Dict[str, nn.Module] = {}
    uploader = None
    if device is not None and torch.device(device).type == "cuda" and torch.cuda.is_available():
        uploader = DeviceUploader(torch.device(device))

    for file_path in files:
        with MappedFile(file_path) as mapped:
            for tensor_name in mapped.names():
                target = params.get(tensor_name)
                if target is None:
                    target = buffers.get(tensor_name)
                if target is not None:
                    shape = mapped.shape(tensor_name)
                    if tuple(target.shape) != shape:
                        # the reference prints and goes on with the uninitialised tensor
                        # (dfloat11.py:230-232); a model that silently computes with garbage is worse
                        raise ValueError(f"Shape mismatch for {tensor_name}: model {tuple(target.shape)} vs loaded "
                                         f"{shape}")
                    with torch.no_grad():
                        target.copy_(torch.from_numpy(mapped.raw(tensor_name)).view(mapped.torch_dtype(tensor_name))
                                     .reshape(shape))
                    continue

                module_path, _, leaf = tensor_name.rpartition(".")
                module = modules.get(module_path)
                if module is None:
                    print(f"Cannot find module path for {tensor_name}", file=stderr)
                    continue
                if leaf not in _unit_tensor_names:
                    # an ordinary tensor the model has no place for (a bias of a layer that has none
                    # here): not part of a compressed unit, so nothing to arm
                    print(f"No parameter or buffer for {tensor_name}; skipped", file=stderr)
                    continue
                units[module_path] = module

                if leaf == "split_positions":
                    module.split_positions = mapped.tensor(tensor_name).tolist()
                elif (cpu_offload and (cpu_offload_blocks is None or cpu_offload_blocks > 0)
                      and leaf in offloaded_tensor_names):
                    if not hasattr(module, "offloaded_tensors"):
                        module.offloaded_tensors = {}
                    module.offloaded_tensors[leaf] = mapped.tensor(tensor_name, pin=pin_memory)
                    if (cpu_offload_blocks is not None and cpu_offload_blocks > 0
                            and len(module.offloaded_tensors) == len(offloaded_tensor_names)):
                        cpu_offload_blocks -= 1
                elif uploader is not None and leaf in offloaded_tensor_names:
                    module.register_buffer(leaf, uploader.upload(mapped.raw(tensor_name), mapped.torch_dtype(tensor_name),
                                                                 mapped.shape(tensor_name)))
                else:
                    module.register_buffer(leaf, mapped.tensor(tensor_name))

                if leaf == "encoded_exponent":
                    module.register_forward_pre_hook(hook)
                    _remove_weights(module, module_path, pattern_dict)
    if uploader is not None:
        uploader.finish()
        log.info("loader: %d large tensors, %.2f GB, host -> %s through pinned staging", uploader.stats["tensors"],
                 uploader.stats["bytes"] / 1e9, uploader.device)

    for name, module in units.items():
        _finish_unit(module, name)

    _mark_root(model)
    return model


def _remove_weights(module: nn.Module, module_path: str, pattern_dict) -> None:
    """Deletes the ``weight`` attributes that the hook supplies (dfloat11.py:273-298)."""
    def drop(target):
        if "weight" in target._parameters:
            del target._parameters["weight"]
        elif hasattr(target, "weight"):
            delattr(target, "weight")

    if isinstance(module, (nn.Linear, nn.Embedding)):
        drop(module)
        return
    for pattern, attr_names in pattern_dict.items():
        if re.fullmatch(pattern, module_path):
            module.weight_injection_modules = []
            for attr_path in attr_names:
                target = module
                for part in attr_path.split("."):
                    target = getattr(target, part)
                drop(target)
                module.weight_injection_modules.append(target)
            return
    raise ValueError(f"compressed unit '{module_path}' is neither a Linear / Embedding nor matched by "
                     "`pattern_dict`, so its weights cannot be injected")


def get_no_split_classes(model, pattern_dict):
    """Class names of the modules matched by ``pattern_dict``: a compressed unit must stay on one
    device together with its decompression buffer (dfloat11.py:311-333)."""
    no_split_classes = []
    for pattern in pattern_dict or {}:
        for full_name, sub_module in model.named_modules():
            if re.fullmatch(pattern, full_name):
                class_name = sub_module.__class__.__name__
                if class_name not in no_split_classes:
                    no_split_classes.append(class_name)
    return no_split_classes


class DFloat11Model:
    """Loads models whose weights are stored in the DF11 format (dfloat11.py:336-493)."""

    @classmethod
    def from_pretrained(
        cls,
        dfloat11_model_name_or_path: str,
        device: Optional[str] = None,
        device_map: str = "auto",
        max_memory: Optional[Dict[Union[int, str], Union[int, str]]] = None,
        bfloat16_model=None,
        cpu_offload: bool = False,
        cpu_offload_blocks: Optional[int] = None,
        pin_memory: bool = True,
        from_single_file: bool = False,
        pattern_dict: Optional[Dict[str, List[str]]] = None,
        *,
        tp_size: int = 1,
        tp_rank: int = 0,
        tp_group=None,
        **kwargs,
    ):
        """Same arguments and behaviour as the reference's ``from_pretrained`` (dfloat11.py:343-464):
        resolve the path, build the model skeleton (or take ``bfloat16_model``), read
        ``dfloat11_config``, load and arm the compressed units, place the model on ``device``
        or spread whole units over the visible GPUs.

        ``tp_size`` / ``tp_rank`` / ``tp_group`` (keyword-only, not in the reference) select the
        partitioned mode of ``dfloat11_b200.tp``: the directory must have been written by
        ``compress_model_tp`` with the same ``tp_size``; this rank loads ``rank{r}-of-{T}/``,
        its Linear layers take the shard shapes and row-parallel layers all-reduce over
        ``tp_group``."""
        path = _resolve_path(dfloat11_model_name_or_path, from_single_file)
        if tp_size > 1:
            from .tp import rank_directory
            if os.path.isdir(rank_directory(path, tp_size, tp_rank)):
                path = rank_directory(path, tp_size, tp_rank)

        if bfloat16_model is not None:
            if from_single_file:
                config = {"dfloat11_config": {"version": version, "threads_per_block": threads_per_block,
                                              "bytes_per_thread": bytes_per_thread, "pattern_dict": pattern_dict}}
            else:
                with open(os.path.join(path, "config.json"), "r", encoding="utf-8") as f:
                    config = json.load(f)
            model = bfloat16_model
        else:
            from transformers import AutoConfig, AutoModelForCausalLM, GenerationConfig
            try:
                from transformers.initialization import no_init_weights
            except ImportError:  # older transformers
                from transformers.modeling_utils import no_init_weights
            config = AutoConfig.from_pretrained(path)
            with no_init_weights():
                model = AutoModelForCausalLM.from_config(config, dtype=torch.bfloat16, **kwargs)
                model.tie_weights()
                model.eval()
            try:
                model.generation_config = GenerationConfig.from_pretrained(path)
            except Exception:  # noqa: BLE001 - optional file
                pass

        if isinstance(config, dict) and "dfloat11_config" in config:
            dfloat11_config = config["dfloat11_config"]
        elif hasattr(config, "dfloat11_config"):
            dfloat11_config = config.dfloat11_config
        else:
            raise AttributeError('"dfloat11_config" not found: it is expected to be found in the config file or '
                                 "passed as an argument.")

        if tp_size > 1:
            from .tp import apply_tensor_parallel
            apply_tensor_parallel(model, dfloat11_config["pattern_dict"], tp_size, tp_rank, group=tp_group)

        load_and_replace_tensors(model, path, dfloat11_config, cpu_offload=cpu_offload,
                                 cpu_offload_blocks=cpu_offload_blocks, pin_memory=pin_memory,
                                 from_single_file=from_single_file, device=device)

        if not cpu_offload:
            model_bytes = sum(t.numel() * t.element_size() for t in model.state_dict().values())
            print(f"Total model size: {model_bytes / 1e9:0.4f} GB", file=stderr)

        if device:
            model = model.to(device)
        else:
            assert device_map == "auto", "device_map should be 'auto' if no specific device is provided."
            from .placement import dispatch_model, infer_device_map
            no_split = get_no_split_classes(model, dfloat11_config["pattern_dict"])
            mapping = infer_device_map(model, no_split_module_classes=no_split, max_memory=max_memory)
            model = dispatch_model(model, mapping)
            if any(p.device.type == "cpu" for p in model.parameters()):
                print("Warning: Some model layers are on CPU. For inference, ensure the model is fully loaded "
                      "onto CUDA-compatible GPUs.", file=stderr)
        return model

    @classmethod
    def from_single_file(
        cls,
        dfloat11_model_path: str,
        pattern_dict: Dict[str, List[str]],
        bfloat16_model,
        device: Optional[str] = None,
        device_map: str = "auto",
        max_memory: Optional[Dict[Union[int, str], Union[int, str]]] = None,
        cpu_offload: bool = False,
        cpu_offload_blocks: Optional[int] = None,
        pin_memory: bool = True,
    ):
        return cls.from_pretrained(
            dfloat11_model_name_or_path=dfloat11_model_path, device=device, device_map=device_map,
            max_memory=max_memory, bfloat16_model=bfloat16_model, cpu_offload=cpu_offload,
            cpu_offload_blocks=cpu_offload_blocks, pin_memory=pin_memory, from_single_file=True,
            pattern_dict=pattern_dict)


def _resolve_path(name_or_path: str, from_single_file: bool) -> str:
    """dfloat11.py:377-390, with the hub download optional (it needs a network)."""
    if from_single_file:
        if os.path.isfile(name_or_path):
            return name_or_path
        if os.path.isdir(name_or_path):
            raise IsADirectoryError("Expected `dfloat11_model_name_or_path` to be the path to a safetensors file, "
                                    f'but found a directory: "{name_or_path}".')
        raise FileNotFoundError(f'The file "{name_or_path}" does not exist.')
    if os.path.exists(name_or_path):
        return name_or_path
    local = name_or_path.replace("/", "__")
    if not os.path.exists(local):
        try:
            from huggingface_hub import snapshot_download
        except ImportError as exc:
            raise FileNotFoundError(f'"{name_or_path}" is not a local path and huggingface_hub is not '
                                    "installed to download it") from exc
        snapshot_download(name_or_path, local_dir=local)
    return local


def _unit_weights(full_name: str, sub_module: nn.Module, attr_names) -> List[torch.Tensor]:
    """Flattened BF16 weights of one unit, in the order they are concatenated, removed from
    their modules (dfloat11.py:528-550)."""
    if isinstance(sub_module, (nn.Embedding, nn.Linear)):
        targets = [("", sub_module)]
    else:
        targets = []
        for attr_path in attr_names:
            target = sub_module
            for part in attr_path.split("."):
                target = getattr(target, part)
            targets.append((attr_path, target))
    weights = []
    for attr_path, target in targets:
        where = f"{full_name}.{attr_path}" if attr_path else full_name
        assert target.weight.data.dtype == torch.bfloat16, \
            f"Expected weights to be in bfloat16 format for compression, but '{where}' has dtype " \
            f"{target.weight.data.dtype}"
        weights.append(target.weight.data.detach().flatten())        # stays where it is: a GPU packs there
        delattr(target, "weight")
    return weights


def check_unit(tensors: Dict[str, torch.Tensor], weights: List[torch.Tensor], device="cuda:0") -> bool:
    """Decompresses freshly made DF11 tensors on the GPU and compares them with the original
    weights, bit for bit -- the reference's self-check (dfloat11.py:560-591)."""
    dev = torch.device(device)
    d = {k: tensors[k].to(dev) for k in ("luts", "encoded_exponent", "sign_mantissa", "output_positions", "gaps")}
    widest = codec.validate_unit(tensors["luts"], tensors["encoded_exponent"], tensors["sign_mantissa"],
                                 tensors["output_positions"], tensors["gaps"])
    out = ops.decode(d["luts"], d["encoded_exponent"], d["sign_mantissa"], d["output_positions"], d["gaps"],
                     max_block_elems=widest)
    want = torch.cat([w.reshape(-1) for w in weights]).view(torch.int16).to(out.device)
    return bool(torch.equal(out.view(torch.int16), want))


def compress_model(
    model,
    pattern_dict: Dict[str, List[str]],
    save_path: str,
    block_range: List[int] = [0, 10000],
    save_single_file: bool = True,
    check_correctness: bool = True,
):
    """Compresses the matched modules of a BF16 model into DF11 and saves it (dfloat11.py:496-636).

    Same arguments, same files: ``model.safetensors`` (or one file per unit plus the model's own
    ``save_pretrained``) and a ``config.json`` carrying ``dfloat11_config``.  ``check_correctness``
    decompresses every unit on ``cuda:0`` and compares it with the original weights.
    """
    from safetensors.torch import save_file

    os.makedirs(save_path, exist_ok=True)
    if check_correctness and not torch.cuda.is_available():
        raise RuntimeError("check_correctness decompresses on cuda:0; no CUDA device is available")

    block_index = 0
    save_model = True
    for pattern, attr_names in pattern_dict.items():
        for full_name, sub_module in list(model.named_modules()):
            if not re.fullmatch(pattern, full_name):
                continue
            if not save_single_file:
                if "." in full_name:
                    parent_name, child_name = full_name.rsplit(".", 1)
                    setattr(model.get_submodule(parent_name), child_name, None)
                else:
                    setattr(model, full_name, None)

            block_index += 1
            if block_index <= block_range[0]:
                continue
            elif block_index > block_range[1]:
                save_model = False
                break

            weights = _unit_weights(full_name, sub_module, attr_names)
            if torch.cuda.is_available() and os.environ.get("DF11_HOST_ENCODER", "0") != "1":
                weights = [w.to("cuda:0") for w in weights]      # packed there: same bytes, far less time
            tensors = codec.encode_weights(weights)
            n = tensors["sign_mantissa"].numel()
            stored = sum(tensors[k].numel() for k in ("encoded_exponent", "sign_mantissa", "output_positions", "gaps"))
            log.info("%s: %d elements, %.2f%% of BF16", full_name, n, stored * 100 / (2 * n))

            if check_correctness and not check_unit(tensors, weights):
                raise RuntimeError("Correctness check failed: the decompressed weights do not match the original "
                                   f'weights for module "{full_name}".')

            for key in ("luts", "encoded_exponent", "sign_mantissa", "output_positions", "gaps", "split_positions"):
                sub_module.register_buffer(key, tensors[key])

            if not save_single_file:
                state_dict = {f"{full_name}.{key}": value for key, value in sub_module.state_dict().items()}
                save_file(state_dict, os.path.join(save_path, full_name.replace(".", "_") + ".safetensors"))

    if save_model:
        dfloat11_config = {"version": version, "threads_per_block": threads_per_block,
                           "bytes_per_thread": bytes_per_thread, "pattern_dict": pattern_dict}
        if hasattr(model, "config"):
            try:
                model.config.dfloat11_config = dfloat11_config
            except Exception:  # noqa: BLE001
                pass

        if hasattr(model, "save_pretrained") and not save_single_file:
            model.save_pretrained(save_path)
        else:
            save_file({k: v.contiguous() for k, v in model.state_dict().items()},
                      os.path.join(save_path, "model.safetensors"))

        save_config = True
        config_path = os.path.join(save_path, "config.json")
        if os.path.exists(config_path):
            with open(config_path, "r", encoding="utf-8") as f:
                existing = json.load(f)
            if isinstance(existing.get("dfloat11_config"), dict):
                save_config = False
        if save_config:
            existing = {}
            if os.path.exists(config_path):
                with open(config_path, "r", encoding="utf-8") as f:
                    existing = json.load(f)
            existing["dfloat11_config"] = dfloat11_config
            with open(config_path, "w", encoding="utf-8") as f:
                json.dump(existing, f, indent=2)


def compress_in_place(model, pattern_dict: Dict[str, List[str]], cpu_offload: bool = False,
                      pin_memory: bool = True):
    """Turns the matched modules of a BF16 model into armed DF11 units without going through
    files: what ``compress_model`` followed by ``DFloat11Model.from_pretrained`` leaves behind,
    on the devices the modules are already on.  (No counterpart in the reference, which always
    saves and reloads; used by the benchmark and handy for experiments.)"""
    hook = get_hook(threads_per_block, bytes_per_thread)
    for pattern, attr_names in pattern_dict.items():
        for full_name, sub_module in list(model.named_modules()):
            if not re.fullmatch(pattern, full_name):
                continue
            device = next(sub_module.parameters()).device
            weights = _unit_weights(full_name, sub_module, attr_names)
            tensors = codec.encode_weights(weights)
            del weights
            sub_module.split_positions = tensors.pop("split_positions").tolist()
            for key, value in tensors.items():
                if cpu_offload and key in offloaded_tensor_names:
                    if not hasattr(sub_module, "offloaded_tensors"):
                        sub_module.offloaded_tensors = {}
                    sub_module.offloaded_tensors[key] = value.pin_memory() if pin_memory else value
                else:
                    sub_module.register_buffer(key, value.to(device), persistent=False)
            if not isinstance(sub_module, (nn.Linear, nn.Embedding)):
                sub_module.weight_injection_modules = []
                for attr_path in attr_names:
                    target = sub_module
                    for part in attr_path.split("."):
                        target = getattr(target, part)
                    sub_module.weight_injection_modules.append(target)
            _finish_unit(sub_module, full_name)
            sub_module.register_forward_pre_hook(hook)
    _mark_root(model)
    # A BF16 weight that is only kept alive by a reference cycle (module bookkeeping of the host
    # framework) would otherwise stay allocated until the collector happens to run: a vocabulary-sized
    # matrix, 1 GB and more, held beside the compressed model.
    import gc
    gc.collect()
    return model
