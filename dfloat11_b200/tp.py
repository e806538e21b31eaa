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
* the vocabulary is cut into one block of rows per rank: the token embedding (``nn.Embedding``
  unit) looks up the ids it holds and the ranks' results are summed (every other rank
  contributes zeros, so the sum is exact); the output head (a single ``nn.Linear`` unit) is
  column-parallel and the ranks' logit slices are gathered.  A vocabulary that does not divide
  by the number of ranks stays replicated.

Decompression itself never communicates: the collectives are the activation all-reduce after
each row-parallel layer (two per transformer block), the all-reduce of the embedding lookup and
the all-gather of the logits.  The two all-reduces are one kernel of this library over NVLink peer
memory (``comm.py``) wherever its buffers can be set up on every rank, and NCCL's otherwise or with
``DF11_PEER_ALLREDUCE=0``; the all-gather is NCCL's.
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


def _shard_layer(layer: nn.Linear, kind: str, tp_size: int, tp_rank: int) -> None:
    """Cuts a Linear layer down to this rank's shard: the weight when it is present (a skeleton
    whose weights the loader supplies has none), the shapes, and the bias -- a column-parallel
    bias is cut like the rows it belongs to, a row-parallel bias is added once, by rank 0."""
    if getattr(layer, "weight", None) is not None:
        layer.weight = nn.Parameter(shard_weight(layer.weight.data, kind, tp_size, tp_rank), requires_grad=False)
    if kind == "column":
        layer.out_features //= tp_size
        if layer.bias is not None:
            layer.bias = nn.Parameter(layer.bias.data.chunk(tp_size)[tp_rank].contiguous(), requires_grad=False)
    else:
        layer.in_features //= tp_size
        if layer.bias is not None and tp_rank != 0:
            layer.bias = None
    layer.df11_tp = (kind, tp_size, tp_rank)


def _shard_embedding(module: nn.Embedding, tp_size: int, tp_rank: int) -> None:
    rows = module.num_embeddings // tp_size
    if getattr(module, "weight", None) is not None:
        module.weight = nn.Parameter(module.weight.data[tp_rank * rows:(tp_rank + 1) * rows].contiguous(),
                                     requires_grad=False)
    module.num_embeddings = rows
    if module.padding_idx is not None:          # only affects gradients; the row itself is data
        module.padding_idx = None
    module.df11_tp = ("vocab", tp_size, tp_rank)


def _single_units(model: nn.Module, pattern_dict):
    """(name, module) of the units that are one Embedding or one Linear (empty attribute list)."""
    for pattern, attr_names in pattern_dict.items():
        if attr_names:
            continue
        for full_name, unit in model.named_modules():
            if re.fullmatch(pattern, full_name) and isinstance(unit, (nn.Embedding, nn.Linear)):
                yield full_name, unit


def _vocab_shardable(unit: nn.Module, tp_size: int) -> bool:
    rows = unit.num_embeddings if isinstance(unit, nn.Embedding) else unit.out_features
    return rows % tp_size == 0 and rows >= tp_size


def apply_shards_only(model, pattern_dict, tp_size, tp_rank, plan=None, vocab_parallel=True):
    """The sharding of ``apply_tensor_parallel`` without its communication hooks (for
    compression, where no process group exists): weights, shapes and biases become this rank's."""
    for pattern, attr_names in pattern_dict.items():
        if not attr_names:
            continue
        unit_plan = plan or default_plan(attr_names)
        for full_name, unit in model.named_modules():
            if not re.fullmatch(pattern, full_name):
                continue
            for attr in attr_names:
                layer = _resolve(unit, attr)
                if getattr(layer, "df11_tp", None):
                    continue
                _shard_layer(layer, unit_plan[attr], tp_size, tp_rank)
    if vocab_parallel:
        for _name, unit in _single_units(model, pattern_dict):
            if getattr(unit, "df11_tp", None) or not _vocab_shardable(unit, tp_size):
                continue
            if isinstance(unit, nn.Embedding):
                _shard_embedding(unit, tp_size, tp_rank)
            else:
                _shard_layer(unit, "column", tp_size, tp_rank)
    model.df11_tp = (tp_size, tp_rank)
    return model


def apply_tensor_parallel(model: nn.Module, pattern_dict: Dict[str, List[str]], tp_size: int, tp_rank: int,
                          group=None, plan: Optional[Dict[str, str]] = None, vocab_parallel: bool = True) -> nn.Module:
    """Turns the Linear layers of every multi-layer unit matched by ``pattern_dict`` into this
    rank's shards (slicing a weight that is present, only fixing the shapes when it is not),
    makes every row-parallel layer sum its output over ``group``, and -- ``vocab_parallel`` --
    cuts single-module units along the vocabulary: an ``nn.Embedding`` looks up the ids of its
    own block of rows and the ranks' results are summed; a single ``nn.Linear`` (the output
    head) becomes column-parallel and its output is gathered over ``group``."""
    if tp_size == 1:
        return model
    import torch.distributed as dist
    own_all_reduce = os.environ.get("DF11_PEER_ALLREDUCE", "1") != "0"

    peer = [None, False]          # the one-kernel all-reduce over NVLink peer memory, set up at its first use

    def sum_over_ranks(output):
        if own_all_reduce and output.is_cuda:
            if not peer[1]:
                from .comm import PeerAllReduce
                peer[0], peer[1] = PeerAllReduce.get(group, output.device), True
            if peer[0] is not None and peer[0].all_reduce_(output):
                return output
        dist.all_reduce(output, group=group)
        return output

    def all_reduce_output(_module, _inputs, output):
        return sum_over_ranks(output)

    def local_ids(module, args):
        # ids of other ranks' rows look up row 0 here and are zeroed afterwards
        ids = args[0]
        rows = module.num_embeddings
        local = ids - module.df11_tp[2] * rows
        mine = (local >= 0) & (local < rows)
        module.__dict__["df11_tp_mine"] = mine
        return (torch.where(mine, local, torch.zeros_like(local)),) + tuple(args[1:])

    def sum_lookups(module, _inputs, output):
        output = output * module.__dict__.pop("df11_tp_mine").unsqueeze(-1).to(output.dtype)
        return sum_over_ranks(output)

    def gather_output(_module, _inputs, output):
        parts = [torch.empty_like(output) for _ in range(tp_size)]
        dist.all_gather(parts, output.contiguous(), group=group)
        return torch.cat(parts, dim=-1)

    fresh = [m for m in model.modules() if isinstance(m, (nn.Linear, nn.Embedding)) and not getattr(m, "df11_tp", None)]
    apply_shards_only(model, pattern_dict, tp_size, tp_rank, plan, vocab_parallel)
    for module in fresh:
        kind = getattr(module, "df11_tp", (None,))[0]
        if kind == "row":
            module.register_forward_hook(all_reduce_output)
        elif kind == "vocab":
            module.register_forward_pre_hook(local_ids)
            module.register_forward_hook(sum_lookups)
        elif kind == "column" and any(module is u for _n, u in _single_units(model, pattern_dict)):
            module.register_forward_hook(gather_output)
    return model


def rank_directory(save_path: str, tp_size: int, tp_rank: int) -> str:
    return os.path.join(save_path, f"rank{tp_rank}-of-{tp_size}")


def compress_model_tp(model: nn.Module, pattern_dict: Dict[str, List[str]], save_path: str, tp_size: int,
                      plan: Optional[Dict[str, str]] = None, check_correctness: bool = False,
                      ranks: Optional[List[int]] = None, vocab_parallel: bool = True) -> List[str]:
    """Writes one ordinary DF11 model directory per rank, holding that rank's shards.

    ``ranks`` limits the work to some ranks (every rank of a job can write its own)."""
    from .dfloat11 import compress_model
    written = []
    for rank in (range(tp_size) if ranks is None else ranks):
        shard_model = copy.deepcopy(model)
        apply_shards_only(shard_model, pattern_dict, tp_size, rank, plan, vocab_parallel)
        path = rank_directory(save_path, tp_size, rank)
        compress_model(shard_model, pattern_dict, path, save_single_file=False,
                       check_correctness=check_correctness)
        written.append(path)
    return written
