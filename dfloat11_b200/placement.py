"""Device placement for models with compressed units.

The reference hands placement to accelerate (``get_balanced_memory`` + ``infer_auto_device_map``
+ ``dispatch_model`` with ``no_split_module_classes``, dfloat11/dfloat11.py:455-460).  This is
the small part of that behaviour the decompression path needs, without the dependency:
whole blocks are assigned to GPUs in definition order under a balanced (or given) byte
budget, a block listed as "no split" is never divided, and every placed block moves its
inputs to its own device before running.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Union

import torch
import torch.nn as nn


def module_bytes(module: nn.Module) -> int:
    """Bytes of the parameters and buffers held by ``module`` (host-resident offloaded tensors
    do not count: they never live on the device all at once)."""
    seen, total = set(), 0
    for t in list(module.parameters()) + list(module.buffers()):
        if id(t) not in seen:
            seen.add(id(t))
            total += t.numel() * t.element_size()
    return total


def _placement_units(model: nn.Module, no_split: Iterable[str]) -> List[tuple]:
    """(name, module) pairs that are placed as a whole, in definition order."""
    no_split = set(no_split)
    out = []

    def walk(name, module):
        children = list(module.named_children())
        own = any(True for _ in module.parameters(recurse=False)) or any(True for _ in module.buffers(recurse=False))
        if not children or module.__class__.__name__ in no_split or own:
            out.append((name, module))
            return
        for child_name, child in children:
            walk(f"{name}.{child_name}" if name else child_name, child)

    walk("", model)
    return out


def infer_device_map(model: nn.Module, no_split_module_classes: Iterable[str] = (),
                     max_memory: Optional[Dict[Union[int, str], Union[int, str]]] = None,
                     devices: Optional[List[int]] = None) -> Dict[str, torch.device]:
    """Assigns every placement unit to a CUDA device, filling devices in order."""
    if devices is None:
        devices = list(range(torch.cuda.device_count()))
    if not devices:
        raise RuntimeError("no CUDA device to place the model on")
    units = _placement_units(model, no_split_module_classes)
    sizes = [module_bytes(m) for _, m in units]
    if max_memory:
        budgets = [_parse_bytes(max_memory.get(d, max_memory.get(str(d), 0))) for d in devices]
    else:
        even = sum(sizes) / len(devices)
        budgets = [even * 1.02 + max(sizes, default=0) * 0.5] * len(devices)   # balanced, with slack for one block
    mapping, d, used = {}, 0, 0
    for (name, _), size in zip(units, sizes):
        while d < len(devices) - 1 and used + size > budgets[d] and used > 0:
            d, used = d + 1, 0
        mapping[name] = torch.device("cuda", devices[d])
        used += size
    return mapping


def _parse_bytes(v) -> float:
    if isinstance(v, (int, float)):
        return float(v)
    s = str(v).strip().upper()
    for suffix, mult in (("GIB", 2 ** 30), ("MIB", 2 ** 20), ("GB", 1e9), ("MB", 1e6), ("KB", 1e3)):
        if s.endswith(suffix):
            return float(s[:-len(suffix)]) * mult
    return float(s)


def _move(obj, device):
    if isinstance(obj, torch.Tensor):
        return obj.to(device, non_blocking=True) if obj.device != device else obj
    if isinstance(obj, tuple) and hasattr(obj, "_fields"):          # a named tuple
        return type(obj)(*(_move(o, device) for o in obj))
    if isinstance(obj, (list, tuple)):
        return type(obj)(_move(o, device) for o in obj)
    if isinstance(obj, dict):
        moved = {k: _move(v, device) for k, v in obj.items()}
        if type(obj) is dict:
            return moved
        try:                                                        # transformers' ModelOutput and the like
            return type(obj)(**moved)
        except TypeError:
            return moved
    return obj


def _first_tensor_device(*objs):
    for obj in objs:
        if isinstance(obj, torch.Tensor):
            return obj.device
        if isinstance(obj, (list, tuple)):
            found = _first_tensor_device(*obj)
            if found is not None:
                return found
        if isinstance(obj, dict):
            found = _first_tensor_device(*obj.values())
            if found is not None:
                return found
    return None


def dispatch_model(model: nn.Module, device_map: Dict[str, torch.device]) -> nn.Module:
    """Moves every placement unit to its device and makes it pull its inputs there."""
    for name, device in device_map.items():
        module = model.get_submodule(name) if name else model
        module.to(device)

        def pre_hook(mod, args, kwargs, _device=device):
            return _move(args, _device), _move(kwargs, _device)

        module.register_forward_pre_hook(pre_hook, with_kwargs=True)

    if len(set(device_map.values())) > 1 and "" not in device_map:
        # what the whole model returns goes back to the device its inputs came from (accelerate's
        # io_same_device of the reference's dispatch_model, dfloat11.py:460), so that callers such
        # as `generate` can go on combining it with their own tensors
        def root_post_hook(mod, args, kwargs, output):
            device = _first_tensor_device(args, kwargs)
            return output if device is None else _move(output, device)

        model.register_forward_hook(root_post_hook, with_kwargs=True)
    model.df11_device_map = dict(device_map)
    return model
