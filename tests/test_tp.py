"""Partitioned (tensor-parallel) mode: sharding identities on one process, the all-reduce wiring
on two gloo ranks (CPU), and -- on a box with two GPUs -- DF11 shards against BF16 shards."""
import copy
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import dfloat11_b200 as df11
from dfloat11_b200 import codec, tp
from oracle import df11_oracle as oracle
from tests.test_model_api import LLAMA_PATTERNS, tiny_llama

BLOCK = LLAMA_PATTERNS[r"model\.layers\.\d+"]


def test_shard_compress_decode_reassemble_is_identity():
    model = tiny_llama()
    layer = model.model.layers[1]
    plan = tp.default_plan(BLOCK)
    assert plan["self_attn.q_proj"] == "column" and plan["mlp.down_proj"] == "row"
    T = 2
    decoded = []
    for rank in range(T):
        shards = [tp.shard_weight(layer.get_submodule(a).weight.data, plan[a], T, rank) for a in BLOCK]
        t = codec.encode_weights([s.flatten() for s in shards])
        out = oracle.decode_c(t["luts"].numpy(), t["encoded_exponent"].numpy(), t["sign_mantissa"].numpy(),
                              t["output_positions"].numpy(), t["gaps"].numpy())
        flat = torch.from_numpy(out.view(np.int16)).view(torch.bfloat16)
        parts = torch.tensor_split(flat, t["split_positions"].tolist())
        decoded.append([p.view(s.shape) for p, s in zip(parts, shards)])
    for i, a in enumerate(BLOCK):
        whole = tp.unshard_weights([decoded[r][i] for r in range(T)], plan[a])
        assert torch.equal(whole, layer.get_submodule(a).weight.data)


def test_compress_model_tp_writes_one_directory_per_rank(tmp_path):
    model = tiny_llama()
    paths = tp.compress_model_tp(model, LLAMA_PATTERNS, str(tmp_path), tp_size=2)
    assert [os.path.basename(p) for p in paths] == ["rank0-of-2", "rank1-of-2"]
    skeleton = tiny_llama(seed=9)
    loaded = df11.DFloat11Model.from_pretrained(str(tmp_path), device="cpu", bfloat16_model=skeleton,
                                                tp_size=2, tp_rank=1)
    q = loaded.model.layers[0].self_attn.q_proj
    o = loaded.model.layers[0].self_attn.o_proj
    assert (q.out_features, q.in_features) == (128, 256) and (o.out_features, o.in_features) == (256, 128)
    n = sum(m.out_features * m.in_features for m in loaded.model.layers[0].weight_injection_modules)
    assert loaded.model.layers[0].sign_mantissa.numel() == n
    assert loaded.lm_head.sign_mantissa.numel() == 1024 * 256           # replicated, not sharded


def _tp_worker(rank, world, port, use_cuda, path, ids, want, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world)
    try:
        if use_cuda:
            torch.cuda.set_device(rank)
            dev = f"cuda:{rank}"
            bf16 = tiny_llama().to(dev)
            tp.apply_tensor_parallel(bf16, LLAMA_PATTERNS, world, rank)
            df = df11.DFloat11Model.from_pretrained(path, device=dev, bfloat16_model=tiny_llama(seed=5),
                                                    tp_size=world, tp_rank=rank)
            with torch.no_grad():
                a = bf16(input_ids=ids.to(dev)).logits
                b = df(input_ids=ids.to(dev)).logits
            q.put((rank, bool(torch.equal(a, b)), float((a.float().cpu() - want).abs().max())))
        else:
            model = tiny_llama().float()
            tp.apply_tensor_parallel(model, LLAMA_PATTERNS, world, rank)
            with torch.no_grad():
                got = model(input_ids=ids).logits
            q.put((rank, True, float((got - want).abs().max())))
    finally:
        dist.destroy_process_group()


def _run_ranks(world, use_cuda, path=None):
    ids = torch.randint(0, 1024, (2, 17), generator=torch.Generator().manual_seed(4))
    ref = tiny_llama().float() if not use_cuda else tiny_llama()
    with torch.no_grad():
        want = ref(input_ids=ids).logits.float()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_tp_worker, args=(r, world, port, use_cuda, path, ids, want, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return sorted(results)


def test_all_reduce_wiring_on_two_gloo_ranks():
    results = _run_ranks(2, use_cuda=False)
    assert [r[0] for r in results] == [0, 1]
    for _, _, err in results:                       # fp32 on CPU: only the summation order differs
        assert err < 1e-3


@pytest.mark.gpu
def test_df11_shards_match_bf16_shards_on_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    tp.compress_model_tp(tiny_llama(), LLAMA_PATTERNS, str(tmp_path), tp_size=2)
    results = _run_ranks(2, use_cuda=True, path=str(tmp_path))
    for _, identical, err in results:
        assert identical                            # same TP degree: bit-identical logits
        assert err < 0.25                           # and close to the unsharded BF16 model
