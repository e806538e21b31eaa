"""Partitioned (tensor-parallel) mode: every GPU holds and decompresses only its own shards.

The reference has no such mode -- its only multi-GPU form places whole units on different
devices (dfloat11/dfloat11.py:455-460, see ``placement.py``).  Here the weights of a unit are
sharded BEFORE compression, because a Huffman stream cannot be re-cut without decoding it:

* column-parallel layers (q/k/v/gate/up: rows of the ``[out, in]`` weight) keep a contiguous
  block of output rows per rank;
* row-parallel layers (o/down: columns) keep a block of input columns per rank, and their
  partial outputs are summed over the ranks (``all_reduce``, NCCL over NVLink on GPUs);
* each rank's shards of a unit are concatenated in the usual order and compressed as one
  ordinary DF11 unit, saved under ``<save_path>/rank{r}-of-{T}/`` in the ordinary layout;
* embeddings and the output head stay whole on every rank (replicated).

Decompression itself never communicates: the only collective is the activation all-reduce
after each row-parallel layer (two per transformer block).
"""
from __future__ import annotations

import copy
import os
import re
from typing import Dict, List, Optional

import torch
import torch.nn as nn

COLUMN_PARALLEL = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj", "to_q", "to_k", "to_v")
ROW_PARALLEL = ("o_proj", "down_proj", "to_out.0")


def default_plan(attr_names) -> Dict[str, str]:
    """'column' / 'row' for every sub-layer of a unit, by the usual layer names."""
    plan = {}
    for attr in attr_names:
        if attr.endswith(COLUMN_PARALLEL):
            plan[attr] = "column"
        elif attr.endswith(ROW_PARALLEL):
            plan[attr] = "row"
        else:
            raise ValueError(f"no tensor-parallel rule for layer '{attr}'; pass an explicit plan")
    return plan


def shard_weight(weight: torch.Tensor, kind: str, tp_size: int, rank: int) -> torch.Tensor:
    """This rank's contiguous shard of an ``[out, in]`` weight."""
    dim = 0 if kind == "column" else 1
    if weight.shape[dim] % tp_size:
        raise ValueError(f"dimension {dim} of a {tuple(weight.shape)} weight does not divide by {tp_size}")
    return weight.chunk(tp_size, dim=dim)[rank].contiguous()


def unshard_weights(shards: List[torch.Tensor], kind: str) -> torch.Tensor:
    return torch.cat(shards, dim=0 if kind == "column" else 1)


def _resolve(module: nn.Module, attr_path: str) -> nn.Module:
    for part in attr_path.split("."):
        module = getattr(module, part)
    return module


def apply_tensor_parallel(model: nn.Module, pattern_dict: Dict[str, List[str]], tp_size: int, tp_rank: int,
                          group=None, plan: Optional[Dict[str, str]] = None) -> nn.Module:
    """Turns the Linear layers of every multi-layer unit matched by ``pattern_dict`` into this
    rank's shards (slicing a weight that is present, only fixing the shapes when it is not)
    and makes every row-parallel layer sum its output over ``group``."""
    if tp_size == 1:
        return model
    import torch.distributed as dist

    def all_reduce_output(_module, _inputs, output):
        dist.all_reduce(output, group=group)
        return output

    for pattern, attr_names in pattern_dict.items():
        if not attr_names:
            continue                                    # single Linear / Embedding units stay whole
        unit_plan = plan or default_plan(attr_names)
        for full_name, unit in model.named_modules():
            if not re.fullmatch(pattern, full_name):
                continue
            for attr in attr_names:
                layer = _resolve(unit, attr)
                kind = unit_plan[attr]
                if getattr(layer, "df11_tp", None):
                    continue
                if getattr(layer, "weight", None) is not None:
                    shard = shard_weight(layer.weight.data, kind, tp_size, tp_rank)
                    layer.weight = nn.Parameter(shard, requires_grad=False)
                if kind == "column":
                    layer.out_features //= tp_size
                    if layer.bias is not None:
                        layer.bias = nn.Parameter(layer.bias.data.chunk(tp_size)[tp_rank].contiguous(),
                                                  requires_grad=False)
                else:
                    layer.in_features //= tp_size
                    if layer.bias is not None and tp_rank != 0:
                        layer.bias = None               # the bias is added once, by rank 0
                    layer.register_forward_hook(all_reduce_output)
                layer.df11_tp = (kind, tp_size, tp_rank)
    model.df11_tp = (tp_size, tp_rank)
    return model


def rank_directory(save_path: str, tp_size: int, tp_rank: int) -> str:
    return os.path.join(save_path, f"rank{tp_rank}-of-{tp_size}")


def compress_model_tp(model: nn.Module, pattern_dict: Dict[str, List[str]], save_path: str, tp_size: int,
                      plan: Optional[Dict[str, str]] = None, check_correctness: bool = False,
                      ranks: Optional[List[int]] = None) -> List[str]:
    """Writes one ordinary DF11 model directory per rank, holding that rank's shards.

    ``ranks`` limits the work to some ranks (every rank of a job can write its own)."""
    from .dfloat11 import compress_model
    written = []
    for rank in (range(tp_size) if ranks is None else ranks):
        shard_model = copy.deepcopy(model)
        apply_shards_only(shard_model, pattern_dict, tp_size, rank, plan)
        path = rank_directory(save_path, tp_size, rank)
        compress_model(shard_model, pattern_dict, path, save_single_file=False,
                       check_correctness=check_correctness)
        written.append(path)
    return written


def apply_shards_only(model, pattern_dict, tp_size, tp_rank, plan=None):
    """``apply_tensor_parallel`` without the all-reduce hooks (for compression, where no process
    group exists)."""
    for pattern, attr_names in pattern_dict.items():
        if not attr_names:
            continue
        unit_plan = plan or default_plan(attr_names)
        for full_name, unit in model.named_modules():
            if not re.fullmatch(pattern, full_name):
                continue
            for attr in attr_names:
                layer = _resolve(unit, attr)
                kind = unit_plan[attr]
                layer.weight = nn.Parameter(shard_weight(layer.weight.data, kind, tp_size, tp_rank),
                                            requires_grad=False)
                if kind == "column":
                    layer.out_features //= tp_size
                else:
                    layer.in_features //= tp_size
    return model
